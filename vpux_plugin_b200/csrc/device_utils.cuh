// Device-side element access and the exact arithmetic of the reference's scalar helpers.
// Every floating-point step that must match the host bit for bit uses a round-to-nearest intrinsic so that
// no fused multiply-add is formed (the library is also compiled with -fmad=false).
#pragma once
#include <utility>

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "../../include/vfold.h"

namespace vf {

// error flag slots written by kernels, read back by flags_check()
enum : int {
    VF_FLAG_CHECKED_CAST = 0,  // a checked_cast would have thrown
    VF_FLAG_QUANT_RANGE = 1,   // calcScaleAndZeroPoint failed for some unit
    VF_FLAG_OVERFLOW = 2,      // an output buffer was too small (Sparsify with supplied counts)
    VF_FLAG_TABLE_RANGE = 3,   // weights table: post-shift needed / bias outside int32
    VF_FLAG_TABLE_ALIGN = 4,   // weights table: pointer not 16-byte aligned
    VF_FLAG_NAN = 5,           // NaN met where the reference's behaviour is undefined
    VF_FLAG_NOT_NORMAL = 6     // ScalarMultInverse of zero, a subnormal, an infinity or NaN
};

__device__ __forceinline__ void set_flag(int* flags, int slot) {
    if (flags) atomicOr(&flags[slot], 1);
}

// ---- programmatic dependent launch ---------------------------------------------------------------------
// The short kernels of a batch call follow one another on a stream, each reading what the one before wrote. A
// kernel launched through launch_chained() (below) may be brought onto the SMs while the kernel before it is
// still draining: chain_enter() is the first statement of every thread of such a kernel. It lets the kernel after
// this one do the same, and then waits until the kernel before this one has completed and its writes are
// visible. Without a chained launch on either side both instructions do nothing.
__device__ __forceinline__ void chain_enter() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

#ifdef __CUDACC__
// Launches `kernel` so that it may overlap the tail of the kernel enqueued before it on `st`; the kernel's first
// statement must be chain_enter().
template <typename... KArgs, typename... Args>
inline cudaError_t launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}
#endif

// ---- fp16 / bf16 ------------------------------------------------------------------------------------
// float16::float16(float) (src/vpux_utils/src/core/type/float16.cpp:30-108). An exhaustive sweep of all 2^32
// inputs against the reference class shows:
//  - results that are normal fp16 numbers, zero or infinity equal IEEE round-to-nearest-even;
//  - NaNs keep the sign and the top ten payload bits, with bit 0 forced when those are all zero (:59-65);
//  - for |x| < 2^-14 (fp16-subnormal results) the routine first rounds the mantissa at normal precision and,
//    when that carries, enters the subnormal branch with the incremented exponent but the original mantissa
//    (:77-107). 90112 inputs therefore differ from IEEE (e.g. 0x347FF000 -> 0x0008, IEEE 0x0004). That range is
//    evaluated with the routine's own integer steps so the bits match the reference.
static __device__ __noinline__ uint16_t f32_to_f16_bits_tiny(uint32_t u) {
    const uint32_t sign = u & 0x80000000u;
    const uint32_t e32 = (u >> 23) & 0xFFu;
    if (e32 == 0) return uint16_t(sign >> 16);
    int be16 = int(e32) - 112;
    uint32_t frac = (u & 0x007FFFFFu) << 3;
    if ((frac & 0x0001FFFFu) == 0x00018000u || (frac & 0x00007FFFu) != 0) {
        frac += 0x00008000u;
        if (frac & 0x7C000000u) {
            frac &= 0x7C000000u;
            be16++;
        }
    }
    frac &= 0x03FF0000u;
    if (be16 > 0) return uint16_t((sign | (uint32_t(be16) << 26) | frac) >> 16);
    frac = 0x04000000u | ((u & 0x007FFFFFu) << 3);
    const uint32_t shift = be16 < -30 ? 0u : (1u << (1 - be16));
    const uint32_t sticky = (frac & (shift - 1u)) ? 1u : 0u;
    if (1 - be16 > 31) frac = 0;
    else frac >>= (1 - be16);
    frac |= sticky;
    if ((frac & 0x0001FFFFu) == 0x00018000u || (frac & 0x00007FFFu) != 0) frac += 0x00008000u;
    return uint16_t((sign | frac) >> 16);
}

__device__ __forceinline__ uint16_t f32_to_f16_bits(float f) {
    const uint32_t u = __float_as_uint(f);
    const uint32_t a = u & 0x7FFFFFFFu;
    if (a > 0x7F800000u) {
        uint32_t frac = (u >> 13) & 0x3FFu;
        if (frac == 0) frac = 1;
        return uint16_t(((u >> 16) & 0x8000u) | 0x7C00u | frac);
    }
    if (a < 0x38800000u) return f32_to_f16_bits_tiny(u);  // |x| < 2^-14
    return __half_as_ushort(__float2half_rn(f));
}
// CvtHelper<float16>::cvt (dialect/const/utils/content.hpp:41-55): infinities clamp to +-65504
__device__ __forceinline__ uint16_t f32_to_f16_clamped_bits(float f) {
    uint16_t h = f32_to_f16_bits(f);
    if ((h & 0x7FFFu) == 0x7C00u) h = uint16_t((h & 0x8000u) | 0x7BFFu);
    return h;
}
// float16::operator float (src/vpux_utils/src/core/type/float16.cpp:118-144) widens the bits, so a NaN keeps its
// sign and payload; the hardware conversion would return the canonical NaN.
__device__ __forceinline__ float f16_bits_to_f32(uint16_t h) {
    const float f = __half2float(__ushort_as_half(h));
    const bool nan = (h & 0x7C00u) == 0x7C00u && (h & 0x03FFu) != 0;
    return nan ? __uint_as_float((uint32_t(h & 0x8000u) << 16) | 0x7F800000u | (uint32_t(h & 0x03FFu) << 13)) : f;
}
// bfloat16::round_to_nearest_even (src/vpux_utils/include/vpux/utils/core/type/bfloat16.hpp:85-87):
// half an ulp is added only when the kept LSB is 1, then the low half is truncated.
__device__ __forceinline__ uint16_t f32_to_bf16_bits(float f) {
    const uint32_t u = __float_as_uint(f);
    return uint16_t((u + ((u & 0x00010000u) >> 1)) >> 16);
}
__device__ __forceinline__ float bf16_bits_to_f32(uint16_t b) {
    return __uint_as_float(uint32_t(b) << 16);
}

// float8_e4m3 (src/vpux_utils/src/core/type/float8_e4m3.cpp): no infinities, 0x7f / 0xff are NaN.
// Decoding (:125-129) is a table lookup in the reference; the table holds sign-less (exp, mantissa) values.
__host__ __device__ __forceinline__ uint32_t f8e4m3_bits_to_f32_bits(uint8_t b) {
    const uint32_t sign = uint32_t(b & 0x80u) << 24, mag = b & 0x7Fu;
    if (mag == 0x7Fu) return sign | 0x7FC00000u;
    const uint32_t e = mag >> 3, m = mag & 7u;
    if (e == 0) {  // subnormal: m * 2^-9, exact in f32
        if (m == 0) return sign;
        const int lead = m >= 4 ? 2 : (m >= 2 ? 1 : 0);  // position of the leading one
        return sign | (uint32_t(127 - 9 + lead) << 23) | ((m << (23 - lead)) & 0x007FFFFFu);
    }
    return sign | ((e + 120u) << 23) | (m << 20);
}
// f32_to_f8e4m3_bits (:52-113): round to nearest even on the 3 kept mantissa bits, overflow and NaN / Inf
// give NaN, f32 subnormals give a signed zero. Inputs below 2^-37 make the reference shift a 32-bit value by
// 32 or more (undefined); they give a signed zero here, the value every in-range shift produces.
__host__ __device__ __forceinline__ uint8_t f32_bits_to_f8e4m3_bits(uint32_t u) {
    uint8_t out = uint8_t((u & 0x80000000u) >> 24);
    const uint32_t e_field = u & 0x7F800000u;
    if (e_field == 0x7F800000u) return out | 0x7Fu;
    if (e_field == 0) return out;
    int32_t e8 = int32_t(e_field >> 23) - 120;
    uint32_t frac = (u & 0x007FFFFFu) << 4;  // f8 mantissa in bits 24..26, the rest below
    if ((frac & 0x01FFFFFFu) == 0x01800000u || (frac & 0x007FFFFFu) != 0) {
        frac += 0x00800000u;
        if (frac & 0x78000000u) {
            frac &= 0x78000000u;
            ++e8;
        }
    }
    frac &= 0x07000000u;
    if (e8 > 15) return out | 0x7Fu;
    if (e8 > 0) return out | uint8_t((uint32_t(e8) << 3) | (frac >> 24));
    frac = 0x08000000u | ((u & 0x007FFFFFu) << 4);  // hidden one restored
    const int rshift = 1 - e8;                        // >= 1
    if (rshift >= 32) return out;
    const uint32_t lost_mask = e8 < -15 ? 0xFFFFFFFFu : ((1u << rshift) - 1u);
    const uint32_t sticky = (frac & lost_mask) ? 1u : 0u;
    frac = (frac >> rshift) | sticky;
    if ((frac & 0x01FFFFFFu) == 0x01800000u || (frac & 0x007FFFFFu) != 0) frac += 0x00800000u;
    return out | uint8_t(frac >> 24);
}
// float8_e5m2 (src/vpux_utils/src/core/type/float8_e5m2.cpp:27-84): the value goes through float16, whose
// low byte is rounded to nearest even unless the result would leave the finite range, then truncated.
__host__ __device__ __forceinline__ uint8_t f16_bits_to_f8e5m2_bits(uint16_t h) {
    const bool can_round = (h & 0x7F00u) < 0x7B00u;
    const bool is_naninf = (h & 0x7C00u) == 0x7C00u;
    if (!is_naninf && can_round) {
        const uint16_t grs = h & 0x00FFu, tie = h & 0x0180u;
        h = uint16_t(h + ((grs > 0x0080u || tie == 0x0180u) ? 0x0100u : 0u));
    }
    return uint8_t(h >> 8);
}

// ---- getValues<float>() / getValues<intN>() element reads -------------------------------------------
// Content::getValues<T>() converts the storage element through checked_cast
// (src/vpux_utils/include/vpux/utils/core/checked_cast.hpp:43-141); a failing check sets VF_FLAG_CHECKED_CAST.
__device__ __forceinline__ float load_as_f32(const void* p, int dt, int64_t i, int* flags) {
    switch (dt) {
    case VF_DT_F32: return static_cast<const float*>(p)[i];
    case VF_DT_F16: return f16_bits_to_f32(static_cast<const uint16_t*>(p)[i]);
    case VF_DT_BF16: return bf16_bits_to_f32(static_cast<const uint16_t*>(p)[i]);
    case VF_DT_F8E4M3FN: return __uint_as_float(f8e4m3_bits_to_f32_bits(static_cast<const uint8_t*>(p)[i]));
    case VF_DT_F8E5M2: return f16_bits_to_f32(uint16_t(uint16_t(static_cast<const uint8_t*>(p)[i]) << 8));
    case VF_DT_F64: {
        const double d = static_cast<const double*>(p)[i];
        const float f = __double2float_rn(d);
        if (double(f) != d) set_flag(flags, VF_FLAG_CHECKED_CAST);
        return f;
    }
    case VF_DT_I8: return float(static_cast<const int8_t*>(p)[i]);
    case VF_DT_U8: return float(static_cast<const uint8_t*>(p)[i]);
    case VF_DT_I16: return float(static_cast<const int16_t*>(p)[i]);
    case VF_DT_U16: return float(static_cast<const uint16_t*>(p)[i]);
    case VF_DT_I32: {
        const int32_t v = static_cast<const int32_t*>(p)[i];
        const float f = __int2float_rn(v);
        if (int64_t(f) != int64_t(v)) set_flag(flags, VF_FLAG_CHECKED_CAST);
        return f;
    }
    case VF_DT_U32: {
        const uint32_t v = static_cast<const uint32_t*>(p)[i];
        const float f = __uint2float_rn(v);
        if (uint64_t(f) != uint64_t(v)) set_flag(flags, VF_FLAG_CHECKED_CAST);
        return f;
    }
    case VF_DT_I64: {
        const long long v = static_cast<const long long*>(p)[i];
        const float f = __ll2float_rn(v);
        if (f >= 9223372036854775808.0f || (long long)(f) != v) set_flag(flags, VF_FLAG_CHECKED_CAST);
        return f;
    }
    case VF_DT_U64: {
        const unsigned long long v = static_cast<const unsigned long long*>(p)[i];
        const float f = __ull2float_rn(v);
        if (f >= 18446744073709551616.0f || (unsigned long long)(f) != v) set_flag(flags, VF_FLAG_CHECKED_CAST);
        return f;
    }
    default: return 0.f;
    }
}

__device__ __forceinline__ void int_limits_dev(int dt, double& lo, double& hi) {
    switch (dt) {
    case VF_DT_I8: lo = -128.0; hi = 127.0; break;
    case VF_DT_U8: lo = 0.0; hi = 255.0; break;
    case VF_DT_I16: lo = -32768.0; hi = 32767.0; break;
    case VF_DT_U16: lo = 0.0; hi = 65535.0; break;
    case VF_DT_I32: lo = -2147483648.0; hi = 2147483647.0; break;
    case VF_DT_U32: lo = 0.0; hi = 4294967295.0; break;
    case VF_DT_I64: lo = -9223372036854775808.0; hi = 9223372036854775807.0; break;
    default: lo = 0.0; hi = 18446744073709551615.0; break;
    }
}

// getValues<Int>()[i] with Int described by `out` (an integer dtype of >= 8 bits)
__device__ __forceinline__ long long load_as_int(const void* p, int dt, int64_t i, int out, int* flags) {
    double lo, hi;
    int_limits_dev(out, lo, hi);
    switch (dt) {
    case VF_DT_F32:
    case VF_DT_F16:
    case VF_DT_BF16:
    case VF_DT_F8E4M3FN:
    case VF_DT_F8E5M2: {
        // checked_cast<Int>(float): compared in float against float(limit), then truncated (:106-117)
        const float f = load_as_f32(p, dt, i, nullptr);
        const float fhi = __double2float_rn(hi), flo = __double2float_rn(lo);
        bool ok = (f <= fhi) && (f >= flo);
        // float(limit) may round up to 2^31 / 2^32 / 2^63: the comparison passes in the reference and the
        // conversion is then undefined; report it
        if (ok && double(f) > hi) ok = false;
        if (!ok) {
            set_flag(flags, VF_FLAG_CHECKED_CAST);
            return 0;
        }
        return (long long)(f);
    }
    case VF_DT_F64: {
        const double d = static_cast<const double*>(p)[i];
        if (!(d <= hi) || !(d >= lo)) {
            set_flag(flags, VF_FLAG_CHECKED_CAST);
            return 0;
        }
        return (long long)(d);
    }
    case VF_DT_U64: {
        const unsigned long long v = static_cast<const unsigned long long*>(p)[i];
        if (double(v) > hi) set_flag(flags, VF_FLAG_CHECKED_CAST);
        return (long long)(v);
    }
    default: {
        long long v;
        switch (dt) {
        case VF_DT_I8: v = static_cast<const int8_t*>(p)[i]; break;
        case VF_DT_U8: v = static_cast<const uint8_t*>(p)[i]; break;
        case VF_DT_I16: v = static_cast<const int16_t*>(p)[i]; break;
        case VF_DT_U16: v = static_cast<const uint16_t*>(p)[i]; break;
        case VF_DT_I32: v = static_cast<const int32_t*>(p)[i]; break;
        case VF_DT_U32: v = static_cast<const uint32_t*>(p)[i]; break;
        default: v = static_cast<const long long*>(p)[i]; break;
        }
        if (double(v) < lo || double(v) > hi) set_flag(flags, VF_FLAG_CHECKED_CAST);
        return v;
    }
    }
}

__device__ __forceinline__ void store_int(void* p, int dt, int64_t i, long long v) {
    switch (dt) {
    case VF_DT_I8:
    case VF_DT_U8: static_cast<uint8_t*>(p)[i] = uint8_t(v); break;
    case VF_DT_I16:
    case VF_DT_U16: static_cast<uint16_t*>(p)[i] = uint16_t(v); break;
    case VF_DT_I32:
    case VF_DT_U32: static_cast<uint32_t*>(p)[i] = uint32_t(v); break;
    default: static_cast<long long*>(p)[i] = v; break;
    }
}

// ---- Quantize ---------------------------------------------------------------------------------------
// std::round for float: half away from zero, exact for |v| < 2^23
__device__ __forceinline__ float round_half_away(float v) {
    const float t = truncf(v);
    const float d = fabsf(__fsub_rn(v, t));  // exact
    return d >= 0.5f ? __fadd_rn(t, copysignf(1.0f, v)) : t;
}

struct QuantParams {  // createQuantizeFn (attributes/quantize.cpp:91-106), all fields fp32 as in the host lambda
    float in_low, in_high, q_low, q_high, levels_m1, range, q_range;
};

// fakeQuantize (src/vpux_compiler/src/utils/quantization.cpp:995-1003) followed by static_cast<int64_t>:
// seven individually rounded fp32 operations, then truncation toward zero.
__device__ __forceinline__ long long quantize_exact(float x, const QuantParams& q) {
    float r;
    if (x <= q.in_low) {
        r = q.q_low;
    } else if (x > q.in_high) {
        r = q.q_high;
    } else {
        float t = __fsub_rn(x, q.in_low);
        t = __fdiv_rn(t, q.range);
        t = __fmul_rn(t, q.levels_m1);
        t = round_half_away(t);
        t = __fdiv_rn(t, q.levels_m1);
        t = __fmul_rn(t, q.q_range);
        r = __fadd_rn(t, q.q_low);
    }
    return (long long)(r);
}

// dequantize (include/vpux/compiler/utils/quantization.hpp:208-210)
__device__ __forceinline__ float dequantize_exact(long long q, double scale, long long zp) {
    return __double2float_rn(__dmul_rn(double(q - zp), scale));
}

__device__ __forceinline__ QuantParams make_quant_params(double scale, long long zp, long long qmin, long long qmax) {
    QuantParams p;
    p.in_low = dequantize_exact(qmin, scale, zp);
    p.in_high = dequantize_exact(qmax, scale, zp);
    p.q_low = float(qmin);
    p.q_high = float(qmax);
    p.levels_m1 = __fsub_rn(float(qmax - qmin + 1), 1.0f);
    p.range = __fsub_rn(p.in_high, p.in_low);
    p.q_range = __fsub_rn(p.q_high, p.q_low);
    return p;
}

// calcScaleAndZeroPoint (src/vpux_compiler/src/utils/quantization.cpp:574-636), FP64. Returns false where the
// reference returns failure().
__device__ __forceinline__ bool calc_scale_zp(double qmin, double qmax, double rmin, double rmax, double& scale,
                                              long long& zp) {
    const double eps = 2.220446049250313e-16;
    if (fabs(rmax - rmin) < eps) {
        if (fabs(rmin) < eps) {
            scale = 1.0;
            zp = 0;
        } else if (rmin >= eps) {
            scale = rmin;
            zp = 0;
        } else {
            scale = -rmin;
            zp = 2;
        }
        return true;
    }
    const bool has_zero = (rmin <= 0 && rmax >= 0) || (rmin >= 0 && rmax <= 0);
    if (!has_zero) return false;
    scale = __ddiv_rn(__dsub_rn(rmax, rmin), __dsub_rn(qmax, qmin));
    if (fabs(scale) <= eps) return false;
    const double x = __dsub_rn(qmin, __ddiv_rn(rmin, scale));
    zp = (long long)(round(x));
    return true;
}

// ---- misc ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// ---- sparsity test ------------------------------------------------------------------------------------
// element != sparsify value, in the logical storage type (utils/sparsity.cpp:47-63,
// attributes/sparsify.cpp:143-152, attributes/get_sparsity_map.cpp:44-52). Floating types compare as
// float, so -0.0 counts as zero.
__device__ __forceinline__ bool is_dense(const void* p, int dt, int64_t i, long long iv, float fv) {
    switch (dt) {
    case VF_DT_I8: return static_cast<const int8_t*>(p)[i] != int8_t(iv);
    case VF_DT_U8: return static_cast<const uint8_t*>(p)[i] != uint8_t(iv);
    case VF_DT_F16: return f16_bits_to_f32(static_cast<const uint16_t*>(p)[i]) != fv;
    case VF_DT_BF16: return bf16_bits_to_f32(static_cast<const uint16_t*>(p)[i]) != fv;
    case VF_DT_F8E4M3FN:
    case VF_DT_F8E5M2: return (static_cast<const uint8_t*>(p)[i] & 0x7Fu) != 0;  // compared as float with 0: -0 is zero, NaN is not
    default: return static_cast<const float*>(p)[i] != fv;
    }
}

__device__ __forceinline__ float sparse_value_as_float(int dt, long long v) {
    float f = float(v);
    if (dt == VF_DT_F16) f = f16_bits_to_f32(f32_to_f16_bits(f));
    if (dt == VF_DT_BF16) f = bf16_bits_to_f32(f32_to_bf16_bits(f));
    return f;
}

}  // namespace vf
