// General-path kernels: one kernel per #const transformation, for every storage type the reference's
// Content::getValues<T>() accepts. These back vf_fold() for arbitrary transformation lists; the weight
// quantization hot path has its own fused kernels (kernels_rowquant.cu).
#include <cuda_fp8.h>

#include "device_utils.cuh"
#include "kernels.h"

namespace vf {

namespace {

constexpr int kBlock = 256;
// items per thread step of the elementwise kernels, their loads issued together (measured in the same call: eight is
// 2 % faster than four for the sub-byte unpack and Rescale, 20 % slower for PadWithZero, whose indices take registers)
constexpr int kInFlight = 4, kInFlightWide = 8;

inline int grid_for(int64_t n, int per_thread = 1) {
    const int64_t blocks = (n + int64_t(kBlock) * per_thread - 1) / (int64_t(kBlock) * per_thread);
    // grid-stride loops: cap at a few waves of the device's SMs
    const int64_t cap = int64_t(sm_count_hint()) * 16;
    return int(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

inline bool aligned16(const void* a, const void* b) {
    return ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b)) & 15u) == 0;
}

#define VF_BY_ELEM_SIZE(es, CALL)                                                   \
    switch (es) {                                                                   \
    case 1: { constexpr int ES = 1; CALL; break; }                                  \
    case 2: { constexpr int ES = 2; CALL; break; }                                  \
    case 4: { constexpr int ES = 4; CALL; break; }                                  \
    case 8: { constexpr int ES = 8; CALL; break; }                                  \
    case 16: { constexpr int ES = 16; CALL; break; }                                \
    default: raise(VF_ERR_UNSUPPORTED, "element size %d", es);                      \
    }
// I = uint32_t while every index of the launch stays below 2^31, int64_t otherwise
#define VF_BY_INDEX_WIDTH(n, CALL)                                                  \
    if ((n) < (int64_t(1) << 31)) { using I = uint32_t; CALL; } else { using I = int64_t; CALL; }

// ------------------------------------------------------------------------------------------------------
// Quantize — attributes/quantize.cpp:108-212
// ------------------------------------------------------------------------------------------------------
__global__ void k_quantize(const void* __restrict__ in, int in_dt, int in_splat, void* __restrict__ out, int out_dt,
                           int64_t n, const double* __restrict__ scales, const int64_t* __restrict__ zps,
                           int64_t axis_size, int64_t inner, long long qmin, long long qmax, int* flags) {
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    QuantParams qp = make_quant_params(scales[0], zps[0], qmin, qmax);
    int64_t cur = 0;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        if (axis_size > 1) {
            const int64_t a = (i / inner) % axis_size;
            if (a != cur) {
                cur = a;
                qp = make_quant_params(scales[a], zps[a], qmin, qmax);
            }
        }
        const float x = load_as_f32(in, in_dt, in_splat ? 0 : i, flags);
        if (x != x) set_flag(flags, VF_FLAG_NAN);
        store_int(out, out_dt, i, quantize_exact(x, qp));
    }
}

// Dequantize — attributes/dequantize.cpp:42-108
__global__ void k_dequantize(const void* __restrict__ in, int in_dt, int in_splat, float* __restrict__ out, int64_t n,
                             const double* __restrict__ scales, const int64_t* __restrict__ zps, int64_t axis_size,
                             int64_t inner, int* flags) {
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        const int64_t a = axis_size > 1 ? (i / inner) % axis_size : 0;
        const long long q = load_as_int(in, in_dt, in_splat ? 0 : i, VF_DT_I64, flags);
        out[i] = dequantize_exact(q, scales[a], zps[a]);
    }
}

// Rescale / Add — attributes/rescale.cpp:67-82, attributes/add.cpp:62-77
__global__ void k_rescale_add(const void* __restrict__ in, int in_dt, int in_splat, float* __restrict__ out,
                              int64_t n, float c, int is_add, int* flags) {
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float v = load_as_f32(in, in_dt, in_splat ? 0 : i, flags);
        out[i] = is_add ? __fadd_rn(v, c) : __fmul_rn(v, c);
    }
}

// ---- eight elements per thread step ---------------------------------------------------------------------
// The elementwise transformations on dense float / 8-bit buffers: one 16-byte load (two for f32) and one or two
// 16-byte stores per step, the per-axis parameters looked up once per step (the launchers take this path only
// when a step never straddles two channels: inner % 8 == 0).
template <int DT>
struct Bytes8 { static constexpr int value = (DT == VF_DT_F32 ? 4 : (DT == VF_DT_F16 || DT == VF_DT_BF16) ? 2 : 1) * 8; };

template <int DT>
__device__ __forceinline__ void load8(const void* __restrict__ in, int64_t g, uint8_t* buf) {
    if (Bytes8<DT>::value == 32) {
        reinterpret_cast<uint4*>(buf)[0] = __ldg(reinterpret_cast<const uint4*>(in) + 2 * g);
        reinterpret_cast<uint4*>(buf)[1] = __ldg(reinterpret_cast<const uint4*>(in) + 2 * g + 1);
    } else if (Bytes8<DT>::value == 16) {
        reinterpret_cast<uint4*>(buf)[0] = __ldg(reinterpret_cast<const uint4*>(in) + g);
    } else {
        reinterpret_cast<uint2*>(buf)[0] = __ldg(reinterpret_cast<const uint2*>(in) + g);
    }
}
template <int BYTES>
__device__ __forceinline__ void store8(void* __restrict__ out, int64_t g, const uint8_t* buf) {
    if (BYTES == 32) {
        reinterpret_cast<uint4*>(out)[2 * g] = reinterpret_cast<const uint4*>(buf)[0];
        reinterpret_cast<uint4*>(out)[2 * g + 1] = reinterpret_cast<const uint4*>(buf)[1];
    } else if (BYTES == 16) {
        reinterpret_cast<uint4*>(out)[g] = reinterpret_cast<const uint4*>(buf)[0];
    } else {
        reinterpret_cast<uint2*>(out)[g] = reinterpret_cast<const uint2*>(buf)[0];
    }
}

// Quantize of floating-point input to 8-bit storage with fakeQuantize as written (ranges whose tail is not the
// identity on the indices, and launches too large for the 32-bit unit count of k_quantize_rows): eight elements per
// thread step.
template <int IN, typename I>
__global__ void k_quantize8(const void* __restrict__ in, uint8_t* __restrict__ out, I n_groups, const double* __restrict__ scales,
                            const int64_t* __restrict__ zps, I axis_size, I inner8, long long qmin, long long qmax, int* flags) {
    const I stride = I(gridDim.x) * I(blockDim.x);
    for (I g = I(blockIdx.x) * I(blockDim.x) + I(threadIdx.x); g < n_groups; g += stride) {
        const I a = axis_size > 1 ? (g / inner8) % axis_size : I(0);
        const QuantParams qp = make_quant_params(scales[a], zps[a], qmin, qmax);
        __align__(16) uint8_t ib[Bytes8<IN>::value];
        __align__(8) uint8_t ob[8];
        load8<IN>(in, int64_t(g), ib);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const float x = load_as_f32(ib, IN, k, flags);
            if (x != x) set_flag(flags, VF_FLAG_NAN);
            ob[k] = uint8_t(quantize_exact(x, qp));
        }
        store8<8>(out, int64_t(g), ob);
    }
}

// The same by rows: a block iteration covers a chunk of kRowUnroll * blockDim groups of ONE row of the quantized
// axis, so the row's parameters (two FP64 products, a division) and the row index (two integer divisions) are
// computed once per chunk instead of once per group. Used when a row holds at least one chunk's worth of groups; a
// per-tensor type is one row.
constexpr int kRowUnroll = 4;
template <int IN, typename I>
__global__ void k_quantize8_rows(const void* __restrict__ in, uint8_t* __restrict__ out, I n_rows, I chunks_per_row,
                                 const double* __restrict__ scales, const int64_t* __restrict__ zps, I axis_size, I inner8,
                                 long long qmin, long long qmax, int* flags) {
    const I n_chunks = n_rows * chunks_per_row;
    for (I chunk = blockIdx.x; chunk < n_chunks; chunk += gridDim.x) {
        const I row = chunk / chunks_per_row, c_in_row = chunk - row * chunks_per_row;
        const I a = axis_size > 1 ? row % axis_size : I(0);
        const QuantParams qp = make_quant_params(scales[a], zps[a], qmin, qmax);
        const I g0 = c_in_row * I(kRowUnroll) * I(blockDim.x) + I(threadIdx.x);
#pragma unroll
        for (int u = 0; u < kRowUnroll; ++u) {
            const I gr = g0 + I(u) * I(blockDim.x);
            if (gr >= inner8) break;
            const int64_t g = int64_t(row) * int64_t(inner8) + int64_t(gr);
            __align__(16) uint8_t ib[Bytes8<IN>::value];
            __align__(8) uint8_t ob[8];
            load8<IN>(in, g, ib);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const float x = load_as_f32(ib, IN, k, flags);
                if (x != x) set_flag(flags, VF_FLAG_NAN);
                ob[k] = uint8_t(quantize_exact(x, qp));
            }
            store8<8>(out, g, ob);
        }
    }
}

template <int IN, typename I>
__global__ void k_dequantize8_rows(const void* __restrict__ in, float* __restrict__ out, I n_rows, I chunks_per_row,
                                   const double* __restrict__ scales, const int64_t* __restrict__ zps, I axis_size, I inner8) {
    const I n_chunks = n_rows * chunks_per_row;
    for (I chunk = blockIdx.x; chunk < n_chunks; chunk += gridDim.x) {
        const I row = chunk / chunks_per_row, c_in_row = chunk - row * chunks_per_row;
        const I a = axis_size > 1 ? row % axis_size : I(0);
        const double scale = scales[a];
        const long long zp = zps[a];
        // q - zp as a 32-bit integer turns into a double without the conversion unit: the integer, biased by 2^31,
        // is placed in the low word of 2^52 + 2^51 and the bias subtracted again (exact); zero points beyond 2^30
        // take the plain conversion
        const bool small_zp = zp > -(1ll << 30) && zp < (1ll << 30);
        const int zp32 = int(zp);
        const I g0 = c_in_row * I(kRowUnroll) * I(blockDim.x) + I(threadIdx.x);
        // all loads of the chunk are issued before the first value is needed
        __align__(8) uint8_t ibs[kRowUnroll][8];
        const int64_t row0 = int64_t(row) * int64_t(inner8);
#pragma unroll
        for (int u = 0; u < kRowUnroll; ++u) {
            const I gr = g0 + I(u) * I(blockDim.x);
            if (gr < inner8) load8<IN>(in, row0 + int64_t(gr), ibs[u]);
        }
#pragma unroll
        for (int u = 0; u < kRowUnroll; ++u) {
            const I gr = g0 + I(u) * I(blockDim.x);
            if (gr >= inner8) break;
            const int64_t g = row0 + int64_t(gr);
            const uint8_t* ib = ibs[u];
            __align__(16) float ob[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const int q32 = IN == VF_DT_I8 ? int(int8_t(ib[k])) : int(ib[k]);
                if (small_zp) {
                    const double d = __dsub_rn(__hiloint2double(0x43380000, (q32 - zp32) ^ int(0x80000000)), 6755401588539392.0);
                    ob[k] = __double2float_rn(__dmul_rn(d, scale));
                } else {
                    ob[k] = dequantize_exact((long long)(q32), scale, zp);
                }
            }
            store8<32>(out, g, reinterpret_cast<const uint8_t*>(ob));
        }
    }
}

template <int IN, typename I>
__global__ void k_dequantize8(const void* __restrict__ in, float* __restrict__ out, I n_groups, const double* __restrict__ scales,
                              const int64_t* __restrict__ zps, I axis_size, I inner8) {
    const I stride = I(gridDim.x) * I(blockDim.x);
    for (I g = I(blockIdx.x) * I(blockDim.x) + I(threadIdx.x); g < n_groups; g += stride) {
        const I a = axis_size > 1 ? (g / inner8) % axis_size : I(0);
        const double scale = scales[a];
        const long long zp = zps[a];
        __align__(8) uint8_t ib[8];
        __align__(16) float ob[8];
        load8<IN>(in, int64_t(g), ib);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const long long q = IN == VF_DT_I8 ? (long long)(int8_t(ib[k])) : (long long)(ib[k]);
            ob[k] = dequantize_exact(q, scale, zp);
        }
        store8<32>(out, int64_t(g), reinterpret_cast<const uint8_t*>(ob));
    }
}

// ---- Quantize / Dequantize by rows, on packed pairs ------------------------------------------------------------
// A warp takes a unit: kPairU 16-byte loads (Quantize) or kDequantU 4-byte loads (Dequantize) per lane of ONE row of the
// quantized axis, all issued before the first value is needed. The row's constants are computed once per unit and
// the arithmetic runs on packed two-wide fp32 instructions (each half is the same IEEE operation as the scalar one).
namespace pairs {

constexpr float kMagic = 12582912.0f;  // 1.5 * 2^23: the ulp is 1, the low mantissa bits hold an integer
constexpr int kPairU = 8;      // 16-byte loads per lane and unit (Quantize: 0.88 of the copy rate with four, 0.93 with eight)
constexpr int kDequantU = 16;  // 4-byte loads per lane and unit (Dequantize)
constexpr float kRangeLo = 7.8886091e-31f, kRangeHi = 1.2676506e30f;  // 2^-100, 2^100

__device__ __forceinline__ float2 dup(float v) {
    return make_float2(v, v);
}

// one 16-byte load of floating-point input as pairs
template <int IN>
struct Step;
template <>
struct Step<VF_DT_F32> {
    static constexpr int kElems = 4, kPairs = 2;
    static __device__ __forceinline__ float2 pair(const uint4& d, int i) {
        return i == 0 ? make_float2(__uint_as_float(d.x), __uint_as_float(d.y)) : make_float2(__uint_as_float(d.z), __uint_as_float(d.w));
    }
    static __device__ __forceinline__ bool has_nan(const uint4& d) {
        return (d.x & 0x7FFFFFFFu) > 0x7F800000u || (d.y & 0x7FFFFFFFu) > 0x7F800000u || (d.z & 0x7FFFFFFFu) > 0x7F800000u ||
               (d.w & 0x7FFFFFFFu) > 0x7F800000u;
    }
};
__device__ __forceinline__ uint32_t word_of(const uint4& d, int i) {
    return i == 0 ? d.x : i == 1 ? d.y : i == 2 ? d.z : d.w;
}
template <>
struct Step<VF_DT_F16> {
    static constexpr int kElems = 8, kPairs = 4;
    static __device__ __forceinline__ float2 pair(const uint4& d, int i) {
        uint32_t w = word_of(d, i);
        return __half22float2(*reinterpret_cast<__half2*>(&w));
    }
    static __device__ __forceinline__ bool has_nan(const uint4& d) {
        bool r = false;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t w = word_of(d, i);
            r |= (w & 0x7FFFu) > 0x7C00u || ((w >> 16) & 0x7FFFu) > 0x7C00u;
        }
        return r;
    }
};
template <>
struct Step<VF_DT_BF16> {
    static constexpr int kElems = 8, kPairs = 4;
    static __device__ __forceinline__ float2 pair(const uint4& d, int i) {
        const uint32_t w = word_of(d, i);
        return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xFFFF0000u));
    }
    static __device__ __forceinline__ bool has_nan(const uint4& d) {
        bool r = false;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t w = word_of(d, i);
            r |= (w & 0x7FFFu) > 0x7F80u || ((w >> 16) & 0x7FFFu) > 0x7F80u;
        }
        return r;
    }
};

// fakeQuantize's middle branch with its own operation sequence (utils/quantization.cpp:995-1003), branch-free:
//   a = fl(x - inLow); the division fl(a / range) as q0 = fl(a y), q = fma(fma(-q0, range, a), y, q0) with
//   y = RN(1 / range), which is the correctly rounded quotient for 2^-100 <= range <= 2^100; e = fl(q (L-1));
//   roundf(e) = floor(e + 1/2) as two additions rounded toward minus infinity, the second onto the integer grid
//   at 1.5 * 2^23 + qmin, so the low byte of the result is the code in two's complement.
// The outer branches (x <= inLow -> qmin, x > inHigh -> qmax) coincide with clamping x to [inLow, inHigh] first:
// x = inLow gives a = 0, x = inHigh gives a = range exactly, and every step is monotonic in x.
struct RowQ {
    float lo, hi;
    float2 nlow, y, nrange, lm1, cm;
};
__device__ __forceinline__ RowQ row_consts(const QuantParams& qp, long long qmin) {
    RowQ q;
    q.lo = qp.in_low;
    q.hi = qp.in_high;
    q.nlow = dup(-qp.in_low);
    q.y = dup(__frcp_rn(qp.range));
    q.nrange = dup(-qp.range);
    q.lm1 = dup(qp.levels_m1);
    q.cm = dup(__fadd_rn(kMagic, float(qmin)));
    return q;
}
__device__ __forceinline__ float2 quant_pair(float2 x, const RowQ& q, float2& nan_acc) {
    nan_acc = __ffma2_rn(x, dup(0.f), nan_acc);  // NaN once any element was NaN or infinite
    x.x = fminf(fmaxf(x.x, q.lo), q.hi);
    x.y = fminf(fmaxf(x.y, q.lo), q.hi);
    const float2 a = __fadd2_rn(x, q.nlow);
    const float2 q0 = __fmul2_rn(a, q.y);
    const float2 d = __ffma2_rn(__ffma2_rn(q0, q.nrange, a), q.y, q0);
    const float2 e = __fmul2_rn(d, q.lm1);
    return __fadd2_rd(__fadd2_rd(e, dup(0.5f)), q.cm);
}
// the codes of one load: four bytes (f32 input) or eight
template <int IN>
__device__ __forceinline__ uint2 quant_step(const uint4& d, const RowQ& q, float2& nan_acc) {
    uint32_t b[Step<IN>::kPairs];
#pragma unroll
    for (int i = 0; i < Step<IN>::kPairs; ++i) {
        const float2 m = quant_pair(Step<IN>::pair(d, i), q, nan_acc);
        b[i] = __byte_perm(__float_as_uint(m.x), __float_as_uint(m.y), 0x0040);
    }
    if (Step<IN>::kPairs == 2) return make_uint2(__byte_perm(b[0], b[1], 0x5410), 0u);
    return make_uint2(__byte_perm(b[0], b[1], 0x5410), __byte_perm(b[2], b[Step<IN>::kPairs - 1], 0x5410));
}
// rows whose range is outside the packed sequence's bounds: fakeQuantize as written, one element at a time
template <int IN>
__device__ __noinline__ uint2 quant_step_scalar(uint4 d, QuantParams qp, int* flags) {
    uint32_t r[2] = {0u, 0u};
#pragma unroll
    for (int k = 0; k < Step<IN>::kElems; ++k) {
        const float x = load_as_f32(&d, IN, k, flags);
        if (x != x) set_flag(flags, VF_FLAG_NAN);
        r[k >> 2] |= (uint32_t(quantize_exact(x, qp)) & 0xFFu) << (8 * (k & 3));
    }
    return make_uint2(r[0], r[1]);
}

}  // namespace pairs

// Quantize of floating-point input to 8-bit codes when the tail of fakeQuantize is the identity on the indices of
// the storage range (tail_is_identity): a row is everything inside the quantized axis (the whole tensor for a
// per-tensor type), row_steps its length in 16-byte loads.
template <int IN>
__global__ void __launch_bounds__(256) k_quantize_rows(const uint4* __restrict__ in, uint8_t* __restrict__ out, uint32_t n_units,
                                                       uint32_t chunks_per_row, uint32_t axis_size, int64_t row_steps,
                                                       const double* __restrict__ scales, const int64_t* __restrict__ zps,
                                                       long long qmin, long long qmax, int* flags) {
    using namespace pairs;
    using S = Step<IN>;
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t n_warps = (gridDim.x * blockDim.x) >> 5;
    for (uint32_t unit = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; unit < n_units; unit += n_warps) {
        const uint32_t row = unit / chunks_per_row, c = unit - row * chunks_per_row;
        const uint32_t a = axis_size > 1 ? row % axis_size : 0u;
        const int64_t s0 = int64_t(c) * (kPairU * 32) + lane;
        const int64_t base = int64_t(row) * row_steps;
        uint4 d[kPairU];
#pragma unroll
        for (int u = 0; u < kPairU; ++u) {
            const int64_t s = s0 + u * 32;
            d[u] = s < row_steps ? __ldg(in + base + s) : make_uint4(0u, 0u, 0u, 0u);
        }
        const QuantParams qp = make_quant_params(scales[a], zps[a], qmin, qmax);
        const bool packed = qp.range >= kRangeLo && qp.range <= kRangeHi;  // false for a NaN range as well
        const RowQ q = row_consts(qp, qmin);
        float2 nan_acc = dup(0.f);
#pragma unroll
        for (int u = 0; u < kPairU; ++u) {
            const int64_t s = s0 + u * 32;
            if (s >= row_steps) break;
            const uint2 codes = packed ? quant_step<IN>(d[u], q, nan_acc) : quant_step_scalar<IN>(d[u], qp, flags);
            if (S::kElems == 4) reinterpret_cast<uint32_t*>(out)[base + s] = codes.x;
            else reinterpret_cast<uint2*>(out)[base + s] = codes;
        }
        if (nan_acc.x != nan_acc.x || nan_acc.y != nan_acc.y) {  // rare: tell NaN from infinity
            bool any = false;
#pragma unroll
            for (int u = 0; u < kPairU; ++u) any |= S::has_nan(d[u]);
            if (any) set_flag(flags, VF_FLAG_NAN);
        }
    }
}

// Dequantize of 8-bit codes, fl32(double(q - zp) * scale) (include/vpux/compiler/utils/quantization.hpp:208-210), in
// fp32: with n = q - zp, s_hi = fl32(scale) and s_lo = fl32(scale - s_hi) the value fma(n, s_hi, fl(n s_lo)) differs
// from the FP64 product by about 2^-47 of it, so it rounds to the same float unless the product lies that close to
// a rounding boundary. There are only 256 codes: a preparation launch evaluates both for every code of every entry
// of the quantized axis and records whether they agree everywhere; entries where they do not, or whose zero point
// is beyond 2^20, keep the FP64 evaluation.
struct DequantRow {
    float s_hi, s_lo, ncz;  // ncz = -(magic + zero point [+ 128 for signed codes])
    uint32_t ok;
};
__global__ void k_dequant_rows_prepare(const double* __restrict__ scales, const int64_t* __restrict__ zps, uint32_t n_axis,
                                       int is_signed, DequantRow* __restrict__ rows) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t a = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (a >= n_axis) return;
    const double scale = scales[a];
    const long long zp = zps[a];
    bool ok = zp > -(1ll << 20) && zp < (1ll << 20);
    const float s_hi = __double2float_rn(scale);
    const float s_lo = __double2float_rn(__dsub_rn(scale, double(s_hi)));
    if (ok) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const int byte = int(lane) + 32 * k;
            const int code = is_signed ? int(int8_t(byte)) : byte;
            const float exact = dequantize_exact((long long)(code), scale, zp);
            const float nf = float(code - int(zp));
            const float fast = __fmaf_rn(nf, s_hi, __fmul_rn(nf, s_lo));
            ok &= __float_as_uint(exact) == __float_as_uint(fast);
        }
    }
    ok = __all_sync(0xFFFFFFFFu, ok);
    if (lane == 0) {
        DequantRow r;
        r.s_hi = s_hi;
        r.s_lo = s_lo;
        r.ncz = ok ? -(pairs::kMagic + float(int(zp) + (is_signed ? 128 : 0))) : 0.f;
        r.ok = ok ? 1u : 0u;
        rows[a] = r;
    }
}
template <int IN>
__device__ __noinline__ float4 dequant_word_f64(uint32_t w, double scale, long long zp) {
    float ob[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const uint32_t b = (w >> (8 * k)) & 0xFFu;
        ob[k] = dequantize_exact(IN == VF_DT_I8 ? (long long)(int8_t(b)) : (long long)(b), scale, zp);
    }
    return make_float4(ob[0], ob[1], ob[2], ob[3]);
}
// A lane takes one 32-bit word (four codes) per load and stores one 16-byte vector of four floats: every load and
// every store of a warp is one contiguous run (128 and 512 bytes). row_words is the row's length in words.
template <int IN>
__global__ void __launch_bounds__(256) k_dequantize_rows(const uint32_t* __restrict__ in, float4* __restrict__ out, uint32_t n_units,
                                                         uint32_t chunks_per_row, uint32_t axis_size, int64_t row_words,
                                                         const DequantRow* __restrict__ rows, const double* __restrict__ scales,
                                                         const int64_t* __restrict__ zps) {
    using namespace pairs;
    constexpr int kU = kDequantU;  // sixteen words in flight per lane (eight measured 0.85 of the copy rate, sixteen 0.89)
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t n_warps = (gridDim.x * blockDim.x) >> 5;
    for (uint32_t unit = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; unit < n_units; unit += n_warps) {
        const uint32_t row = unit / chunks_per_row, c = unit - row * chunks_per_row;
        const uint32_t a = axis_size > 1 ? row % axis_size : 0u;
        const int64_t w0 = int64_t(c) * (kU * 32) + lane;
        const int64_t base = int64_t(row) * row_words;
        uint32_t d[kU];
#pragma unroll
        for (int u = 0; u < kU; ++u) {
            const int64_t w = w0 + u * 32;
            d[u] = w < row_words ? __ldg(in + base + w) : 0u;
        }
        const uint4 rw = __ldg(reinterpret_cast<const uint4*>(rows) + a);
        const float2 s_hi = dup(__uint_as_float(rw.x)), s_lo = dup(__uint_as_float(rw.y)), ncz = dup(__uint_as_float(rw.z));
        if (rw.w) {
#pragma unroll
            for (int u = 0; u < kU; ++u) {
                const int64_t w = w0 + u * 32;
                if (w >= row_words) break;
                const uint32_t x = IN == VF_DT_I8 ? d[u] ^ 0x80808080u : d[u];  // code + 128 as an unsigned byte
                float2 r[2];
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    // the byte under the bit pattern of the magic constant: magic + byte as a float
                    const float2 m = make_float2(__uint_as_float(__byte_perm(x, 0x4B400000u, 0x7650 + 2 * j)),
                                                 __uint_as_float(__byte_perm(x, 0x4B400000u, 0x7651 + 2 * j)));
                    const float2 n = __fadd2_rn(m, ncz);  // exact
                    r[j] = __ffma2_rn(n, s_hi, __fmul2_rn(n, s_lo));
                }
                __stcs(out + base + w, make_float4(r[0].x, r[0].y, r[1].x, r[1].y));  // written once, not read again here
            }
        } else {
            const double scale = scales[a];
            const long long zp = zps[a];
#pragma unroll
            for (int u = 0; u < kU; ++u) {
                const int64_t w = w0 + u * 32;
                if (w >= row_words) break;
                out[base + w] = dequant_word_f64<IN>(d[u], scale, zp);
            }
        }
    }
}

// Rescale / Add with four elements per lane and item: one 16-byte (f32) or 8-byte (16-bit types) load and one 16-byte
// store, so every access of a warp is one contiguous run of whole sectors; eight items per thread step, their loads
// issued together.
template <int IN>
__global__ void k_rescale_add4(const void* __restrict__ in, float4* __restrict__ out, int64_t n_items, float c, int is_add, int* flags) {
    constexpr int kU = kInFlightWide;
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t t0 = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; t0 < n_items; t0 += kU * stride) {
        float4 v[kU];
#pragma unroll
        for (int u = 0; u < kU; ++u) {
            const int64_t t = t0 + u * stride;
            v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (t < n_items) {
                if (IN == VF_DT_F32) {
                    v[u] = __ldg(reinterpret_cast<const float4*>(in) + t);
                } else {
                    const uint2 w = __ldg(reinterpret_cast<const uint2*>(in) + t);
                    v[u] = make_float4(load_as_f32(&w, IN, 0, flags), load_as_f32(&w, IN, 1, flags), load_as_f32(&w, IN, 2, flags),
                                       load_as_f32(&w, IN, 3, flags));
                }
            }
        }
#pragma unroll
        for (int u = 0; u < kU; ++u) {
            const int64_t t = t0 + u * stride;
            if (t >= n_items) break;
            const float4 x = v[u];
            out[t] = is_add ? make_float4(__fadd_rn(x.x, c), __fadd_rn(x.y, c), __fadd_rn(x.z, c), __fadd_rn(x.w, c))
                            : make_float4(__fmul_rn(x.x, c), __fmul_rn(x.y, c), __fmul_rn(x.z, c), __fmul_rn(x.w, c));
        }
    }
}

// copyTo element conversion — utils/content.cpp:84-97,180-183 with CvtHelper (utils/content.hpp:33-87)
__global__ void k_convert(const void* __restrict__ in, int in_dt, int in_splat, void* __restrict__ out, int out_dt,
                          int64_t n, int* flags) {
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        const int64_t s = in_splat ? 0 : i;
        switch (out_dt) {
        case VF_DT_F32: static_cast<float*>(out)[i] = load_as_f32(in, in_dt, s, flags); break;
        case VF_DT_F16: static_cast<uint16_t*>(out)[i] = f32_to_f16_clamped_bits(load_as_f32(in, in_dt, s, flags)); break;
        case VF_DT_BF16: static_cast<uint16_t*>(out)[i] = f32_to_bf16_bits(load_as_f32(in, in_dt, s, flags)); break;
        case VF_DT_F8E4M3FN: static_cast<uint8_t*>(out)[i] = f32_bits_to_f8e4m3_bits(__float_as_uint(load_as_f32(in, in_dt, s, flags))); break;
        case VF_DT_F8E5M2: static_cast<uint8_t*>(out)[i] = f16_bits_to_f8e5m2_bits(f32_to_f16_bits(load_as_f32(in, in_dt, s, flags))); break;
        case VF_DT_F64: {
            double d;
            if (in_dt == VF_DT_F64) d = static_cast<const double*>(in)[s];
            else if (in_dt == VF_DT_F32 || in_dt == VF_DT_F16 || in_dt == VF_DT_BF16 || in_dt == VF_DT_F8E4M3FN || in_dt == VF_DT_F8E5M2)
                d = double(load_as_f32(in, in_dt, s, flags));
            else if (in_dt == VF_DT_U64) d = double(static_cast<const unsigned long long*>(in)[s]);
            else d = double(load_as_int(in, in_dt, s, VF_DT_I64, flags));
            static_cast<double*>(out)[i] = d;
            break;
        }
        default: store_int(out, out_dt, i, load_as_int(in, in_dt, s, out_dt, flags));
        }
    }
}

// copySubByteContent, packing branch — utils/content.cpp:131-152
__global__ void k_pack_subbyte(const void* __restrict__ in, int in_dt, uint8_t* __restrict__ out, int64_t n_out,
                               int per_byte, int* flags) {
    const int bits = 8 / per_byte;
    const unsigned mask = (1u << bits) - 1u;
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t o = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; o < n_out; o += stride) {
        unsigned byte = 0;
        for (int k = 0; k < per_byte; ++k) {
            const long long v = load_as_int(in, in_dt, o * per_byte + k, VF_DT_I8, flags);
            byte |= (unsigned(v) & mask) << (k * bits);
        }
        out[o] = uint8_t(byte);
    }
}

// subByteConversion — utils/convert_utils.cpp:17-75: 1-, 2- or 4-bit elements (low bits first) to one byte
// each. A thread expands 8 elements: it reads `BITS` input bytes as one word and writes 8 bytes. `sign` selects
// the sign-extending branch (:47-66), otherwise the masking branch (:28-46).
template <int BITS>
__device__ __forceinline__ uint2 expand8(uint32_t w, int sign) {  // eight elements of BITS bits -> eight bytes
    if (BITS == 4) {
        // even nibbles and odd nibbles as bytes, interleaved by two byte permutes; a set bit 3 times 0x1E is 0xF0, the
        // sign extension of a 4-bit value (no carry between bytes)
        uint32_t lo = w & 0x0F0F0F0Fu, hi = (w >> 4) & 0x0F0F0F0Fu;
        if (sign) {
            lo |= (lo & 0x08080808u) * 0x1Eu;
            hi |= (hi & 0x08080808u) * 0x1Eu;
        }
        return make_uint2(__byte_perm(lo, hi, 0x5140), __byte_perm(lo, hi, 0x7362));
    }
    constexpr unsigned kMask = (1u << BITS) - 1u;
    uint32_t r[2] = {0u, 0u};
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        uint32_t v = (w >> (k * BITS)) & kMask;
        if (sign) v = uint32_t(int32_t(v << (32 - BITS)) >> (32 - BITS)) & 0xFFu;
        r[k >> 2] |= v << (8 * (k & 3));
    }
    return make_uint2(r[0], r[1]);
}

// 16 elements per item: 2 * BITS input bytes in one load, one 16-byte store, so every load and every store of a warp
// is one contiguous run; eight items per thread step, their loads issued together (both buffers aligned)
template <int BITS>
__global__ void k_unpack_subbyte_x16(const uint8_t* __restrict__ in, uint4* __restrict__ out, int64_t n_items, int sign) {
    constexpr int kU = kInFlightWide;
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t t0 = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; t0 < n_items; t0 += kU * stride) {
        uint32_t w[kU][2];
#pragma unroll
        for (int u = 0; u < kU; ++u) {
            const int64_t t = t0 + u * stride;
            w[u][0] = w[u][1] = 0u;
            if (t < n_items) {
                if (BITS == 4) {
                    const uint2 x = __ldg(reinterpret_cast<const uint2*>(in) + t);
                    w[u][0] = x.x, w[u][1] = x.y;
                } else if (BITS == 2) {
                    const uint32_t x = __ldg(reinterpret_cast<const uint32_t*>(in) + t);
                    w[u][0] = x & 0xFFFFu, w[u][1] = x >> 16;
                } else {
                    const uint32_t x = __ldg(reinterpret_cast<const uint16_t*>(in) + t);
                    w[u][0] = x & 0xFFu, w[u][1] = x >> 8;
                }
            }
        }
#pragma unroll
        for (int u = 0; u < kU; ++u) {
            const int64_t t = t0 + u * stride;
            if (t >= n_items) break;
            const uint2 a = expand8<BITS>(w[u][0], sign), b = expand8<BITS>(w[u][1], sign);
            out[t] = make_uint4(a.x, a.y, b.x, b.y);
        }
    }
}

template <int BITS>
__global__ void k_unpack_subbyte(const uint8_t* __restrict__ in, uint8_t* __restrict__ out, int64_t n_out, int sign) {
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    const int64_t groups = (n_out + 7) / 8;
    const bool aligned = (reinterpret_cast<uintptr_t>(in) % BITS) == 0 && (reinterpret_cast<uintptr_t>(out) % 8) == 0;
    for (int64_t g = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; g < groups; g += stride) {
        const int64_t o0 = g * 8;
        const int left = int(n_out - o0 < 8 ? n_out - o0 : 8);
        uint32_t w = 0;
        if (aligned && left == 8) {
            if (BITS == 4) w = *reinterpret_cast<const uint32_t*>(in + g * 4);
            else if (BITS == 2) w = *reinterpret_cast<const uint16_t*>(in + g * 2);
            else w = in[g];
        } else {
            const int nbytes = (left * BITS + 7) / 8;
            for (int b = 0; b < nbytes; ++b) w |= uint32_t(in[g * BITS + b]) << (8 * b);
        }
        const uint2 r2 = expand8<BITS>(w, sign);
        if (aligned && left == 8) {
            *reinterpret_cast<uint2*>(out + o0) = r2;
        } else {
            const uint32_t r[2] = {r2.x, r2.y};
            for (int k = 0; k < left; ++k) out[o0 + k] = uint8_t(r[k >> 2] >> (8 * (k & 3)));
        }
    }
}

// SwizzleConstant — BufferSwizzleTransform::swizzle (utils/swizzle_transform.hpp:56-76) with
// AddressTransform::getPhysicalAddress (attributes/swizzle_transform.cpp:71-83): every chunk of the RAM-cut
// data width (16 bytes on NPU37XX, 32 on NPU40XX) moves to its staggered address inside its RAM-cut block.
// A pure permutation of 16-byte vectors: one vector per thread step, loads and stores both 16 bytes wide.
// The source holds `in_bytes` valid bytes; what lies behind them up to the swizzled size reads as `pad`.
__global__ void k_swizzle(const uint4* __restrict__ in, uint64_t in_bytes, uint32_t pad, uint4* __restrict__ out, int64_t n_vec,
                          uint32_t log2w, uint32_t stagger_mask, uint32_t shift, uint32_t cut_mask) {
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    const int64_t full = int64_t(in_bytes / 16);
    const uint32_t pad4 = pad * 0x01010101u;
    for (int64_t v = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; v < n_vec; v += stride) {
        uint4 x;
        if (v < full) {
            x = __ldg(in + v);
        } else {  // the vector that straddles the end of the data, and the padding behind it
            uint32_t w[4] = {pad4, pad4, pad4, pad4};
            const uint8_t* b = reinterpret_cast<const uint8_t*>(in);
            for (int k = 0; k < 16; ++k) {
                const uint64_t at = uint64_t(v) * 16 + k;
                if (at < in_bytes) w[k >> 2] = (w[k >> 2] & ~(0xFFu << (8 * (k & 3)))) | (uint32_t(b[at]) << (8 * (k & 3)));
            }
            x = make_uint4(w[0], w[1], w[2], w[3]);
        }
        const uint32_t addr = uint32_t(v) << 4;
        const uint32_t dpu = addr & ~((1u << log2w) - 1u);  // the chunk this vector belongs to
        uint32_t s = dpu >> log2w;
        s &= (1u << 11) - 1u;
        s >>= 5;
        s &= stagger_mask;
        s <<= shift;
        uint32_t phy = (dpu + s) & cut_mask;
        phy += dpu & ~cut_mask;
        out[(phy + (addr - dpu)) >> 4] = x;
    }
}

// BitPack<4> — attributes/bit_pack.cpp:146-151
__global__ void k_bitpack4(const void* __restrict__ in, int in_dt, uint8_t* __restrict__ out, int64_t n_out,
                           int* flags) {
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t o = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; o < n_out; o += stride) {
        const unsigned lo = unsigned(load_as_int(in, in_dt, 2 * o, VF_DT_U8, flags)) & 0xFu;
        const unsigned hi = unsigned(load_as_int(in, in_dt, 2 * o + 1, VF_DT_U8, flags)) & 0xFu;
        out[o] = uint8_t((hi << 4) + lo);
    }
}

// u8 fast path of BitPack: 16 codes in, 8 bytes out per thread step
__global__ void k_bitpack4_u8(const uint4* __restrict__ in, uint2* __restrict__ out, int64_t n_vec) {
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t v = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; v < n_vec; v += stride) {
        const uint4 x = in[v];
        auto pack = [](unsigned w) {  // 4 bytes -> 2 bytes (low nibble first)
            const unsigned a = w & 0x0F0F0F0Fu;
            const unsigned b = a | (a >> 4);  // byte0|byte1<<4 in bits 0..7, byte2|byte3<<4 in bits 16..23
            return (b & 0xFFu) | ((b >> 8) & 0xFF00u);
        };
        uint2 r;
        r.x = pack(x.x) | (pack(x.y) << 16);
        r.y = pack(x.z) | (pack(x.w) << 16);
        out[v] = r;
    }
}

__global__ void k_fill_bytes(uint8_t* out, uint8_t value, uint64_t bytes) {
    const uint64_t stride = uint64_t(gridDim.x) * blockDim.x;
    for (uint64_t i = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < bytes; i += stride) out[i] = value;
}

// ------------------------------------------------------------------------------------------------------
// layout
// ------------------------------------------------------------------------------------------------------
template <int ES>
struct ElemOf;
template <> struct ElemOf<1> { using T = uint8_t; };
template <> struct ElemOf<2> { using T = uint16_t; };
template <> struct ElemOf<4> { using T = uint32_t; };
template <> struct ElemOf<8> { using T = uint64_t; };
template <> struct ElemOf<16> { using T = uint4; };

// The layout kernels work on a geometry the launchers have simplified on the host: neighbouring dims that are
// contiguous on both sides are merged, a contiguous innermost dim is regrouped into elements of up to 16 bytes,
// and the index arithmetic runs in 32 bits (I = uint32_t) whenever all extents allow it.

// memPermuteTransformation — utils/transformations.cpp:889-939, gathered from the output side so that the
// stores are coalesced
template <int ES, typename I>
__global__ void k_permute(const void* __restrict__ in, void* __restrict__ out, Geom g, I n) {
    using T = typename ElemOf<ES>::T;
    const I stride = I(gridDim.x) * I(blockDim.x);
    for (I o = I(blockIdx.x) * I(blockDim.x) + I(threadIdx.x); o < n; o += stride) {
        I rem = o, src = 0;
#pragma unroll
        for (int d = VF_MAX_RANK - 1; d >= 0; --d) {
            if (d < g.rank) {
                const I os = I(g.out_shape[d]);
                const I q = rem / os;
                src += (rem - q * os) * I(g.src_stride[d]);
                rem = q;
            }
        }
        static_cast<T*>(out)[o] = static_cast<const T*>(in)[src];
    }
}

// The same permutation through a 64 x 64 shared-memory tile, for geometries whose innermost output dim is not
// the innermost input dim: dim `a` (innermost on the output side) and dim `b` (the one with source stride 1)
// span the tile, so that the loads run along b and the stores along a, both coalesced. One CTA of 32 x 8 threads
// per tile; blockIdx.x enumerates (other dims, tiles along a, tiles along b).
constexpr int kTile = 64;
template <int ES, typename I>
__global__ void __launch_bounds__(256) k_permute_tiled(const void* __restrict__ in, void* __restrict__ out, Geom g, int b, I tiles_a,
                                                       I tiles_b, I dst_stride_b) {
    using T = typename ElemOf<ES>::T;
    __shared__ T tile[kTile][kTile + 1];
    const int a = g.rank - 1;
    I rem = I(blockIdx.x);
    const I tb = rem % tiles_b;
    rem /= tiles_b;
    const I ta = rem % tiles_a;
    rem /= tiles_a;
    I src0 = 0, dst0 = 0, dst_mul = 1;  // base offsets from the coordinates of the other dims
#pragma unroll
    for (int d = VF_MAX_RANK - 1; d >= 0; --d) {
        if (d < g.rank) {
            const I os = I(g.out_shape[d]);
            if (d != a && d != b) {
                const I q = rem / os;
                const I c = rem - q * os;
                rem = q;
                src0 += c * I(g.src_stride[d]);
                dst0 += c * dst_mul;
            }
            dst_mul *= os;
        }
    }
    const I ea = I(g.out_shape[a]), eb = I(g.out_shape[b]);
    const I a0 = ta * kTile, b0 = tb * kTile;
    const I sa = I(g.src_stride[a]);
#pragma unroll
    for (int i = 0; i < kTile; i += 8) {  // rows of the tile run along a, columns along b (source stride 1)
        const I ia = a0 + threadIdx.y + i;
#pragma unroll
        for (int c = 0; c < kTile; c += 32) {
            const I ib = b0 + threadIdx.x + c;
            if (ia < ea && ib < eb) tile[threadIdx.y + i][threadIdx.x + c] = static_cast<const T*>(in)[src0 + ia * sa + ib];
        }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < kTile; i += 8) {  // stores: rows along b, columns along a (destination stride 1)
        const I ib = b0 + threadIdx.y + i;
#pragma unroll
        for (int c = 0; c < kTile; c += 32) {
            const I ia = a0 + threadIdx.x + c;
            if (ia < ea && ib < eb) static_cast<T*>(out)[dst0 + ib * dst_stride_b + ia] = tile[threadIdx.x + c][threadIdx.y + i];
        }
    }
}

// The transposition of the two innermost output dims when together they are ONE contiguous block of the source
// (OIYX -> OYXI: per output channel the IC x KY*KX slice becomes KY*KX x IC). A chunk is a contiguous piece of the
// source: several whole slices when they are small and follow each other in memory (a 64 x 3 x 3 f16 slice is
// 1152 bytes), one slice, or `rows` rows of a slice that does not fit. It is copied into shared memory with 16-byte
// asynchronous copies, starting at the 16-byte boundary at or below the chunk, and written out as 16-byte vectors
// of consecutive a: eight lanes (f16, ea = 64) cover one output row, a warp four rows, contiguous in memory. Each
// element costs one shared-memory read. The CTAs are persistent with a ring of three buffers: the copies of a
// CTA's next two chunks are in flight while it writes this one (it takes more than 100 KB in flight per SM to keep
// the memory busy).
__device__ __forceinline__ void cp_async16_part(void* smem_dst, const void* gsrc, int src_bytes) {
    const uint32_t sdst = uint32_t(__cvta_generic_to_shared(smem_dst));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(sdst), "l"(gsrc), "r"(src_bytes) : "memory");  // the rest is zero-filled
}
struct SliceGeom {
    uint32_t ea, eb;          // rows (source) / columns of a slice; the output slice is eb x ea
    uint32_t rows;            // rows per chunk (== ea unless the slice is cut)
    uint32_t chunks_a;        // chunks per slice
    uint32_t per_group;       // whole slices per chunk (1 when the slice is cut)
    uint32_t groups;          // chunks along the slice-index dim
    uint32_t n_slices;        // extent of the slice-index dim (the dim just outside the slice; 1 if there is none)
    int64_t slice_src;        // source stride of the slice-index dim (== ea * eb when per_group > 1)
    int n_outer;              // dims outside the slice-index dim
    int64_t outer_shape[VF_MAX_RANK], outer_src[VF_MAX_RANK], outer_dst[VF_MAX_RANK];
};
constexpr int kSliceStages = 3;  // chunks in flight per CTA: the one being written and the copies of the next two
template <int ES>
__global__ void __launch_bounds__(256) k_transpose_slices(const uint8_t* __restrict__ in, uint8_t* __restrict__ out, SliceGeom g,
                                                          int64_t n_chunks, uint32_t buf_vecs, int64_t total_bytes) {
    constexpr uint32_t VE = 16 / ES;  // elements per output vector
    extern __shared__ uint4 slice_smem[];
    using T = typename ElemOf<ES>::T;
    const uint32_t ea = g.ea, eb = g.eb;

    struct Chunk {
        int64_t dst0;    // element offset of the chunk's first slice in the output
        int64_t start;   // 16-byte aligned byte offset in the source at or below the chunk
        uint32_t a0, ta; // first row and rows (per slice) of the chunk
        uint32_t ns;     // slices in the chunk
        uint32_t lead;   // bytes in front of the chunk inside its first vector
    };
    auto locate = [&](int64_t idx) -> Chunk {
        Chunk c;
        int64_t rem = idx;
        const uint32_t ca = uint32_t(rem % g.chunks_a);
        rem /= g.chunks_a;
        const uint32_t grp = uint32_t(rem % g.groups);
        rem /= g.groups;
        const uint32_t s0 = grp * g.per_group;
        int64_t src0 = int64_t(s0) * g.slice_src, dst0 = int64_t(s0) * ea * eb;
        for (int k = 0; k < g.n_outer; ++k) {
            const int64_t q = rem / g.outer_shape[k];
            const int64_t cc = rem - q * g.outer_shape[k];
            rem = q;
            src0 += cc * g.outer_src[k];
            dst0 += cc * g.outer_dst[k];
        }
        c.dst0 = dst0;
        c.ns = min(g.per_group, g.n_slices - s0);
        c.a0 = ca * g.rows;
        c.ta = min(g.rows, ea - c.a0);
        const int64_t first = (src0 + int64_t(c.a0) * eb) * ES;  // byte offset of the chunk in the source
        c.start = first & ~int64_t(15);
        c.lead = uint32_t(first - c.start);
        return c;
    };
    // the copy of chunk `idx` into buffer `slot`, as one group of asynchronous copies (an empty group past the end)
    auto fetch = [&](int64_t idx, int slot) {
        if (idx < n_chunks) {
            const Chunk c = locate(idx);
            uint4* buf = slice_smem + slot * buf_vecs;
            const uint32_t n_vec = (c.lead + c.ns * c.ta * eb * ES + 15u) >> 4;
            for (uint32_t v = threadIdx.x; v < n_vec; v += blockDim.x) {
                const int64_t p = c.start + int64_t(v) * 16;
                const int64_t left = total_bytes - p;  // the last vector of the buffer may be cut short
                cp_async16_part(buf + v, in + p, left >= 16 ? 16 : int(left));
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    int64_t idx = blockIdx.x;
    if (idx >= n_chunks) return;
    const int64_t stride = gridDim.x;
#pragma unroll
    for (int s = 0; s < kSliceStages - 1; ++s) fetch(idx + s * stride, s);
    int cur = 0;
    for (; idx < n_chunks; idx += stride) {
        int ahead = cur + kSliceStages - 1;
        if (ahead >= kSliceStages) ahead -= kSliceStages;
        fetch(idx + (kSliceStages - 1) * stride, ahead);
        asm volatile("cp.async.wait_group %0;" ::"n"(kSliceStages - 1) : "memory");
        __syncthreads();  // every thread's copies of this chunk have landed
        const Chunk c = locate(idx);
        const T* sm = reinterpret_cast<const T*>(reinterpret_cast<const uint8_t*>(slice_smem + cur * buf_vecs) + c.lead);
        // output vectors of the chunk in output order: (slice, column ib, row block iab), iab fastest. With several
        // slices per chunk a slice is whole (ta == ea) and the chunk's output is one contiguous run.
        const uint32_t nab = c.ta / VE, per_slice = nab * eb, n_out = c.ns * per_slice;
        uint32_t sl = threadIdx.x / per_slice, rem = threadIdx.x - sl * per_slice;
        uint32_t ib = rem / nab, iab = rem - ib * nab;
        const uint32_t step_s = blockDim.x / per_slice, step_r = blockDim.x - step_s * per_slice;
        const uint32_t step_b = step_r / nab, step_a = step_r - step_b * nab;
        for (uint32_t v = threadIdx.x; v < n_out; v += blockDim.x) {
            __align__(16) T e[VE];
            const T* col = sm + sl * (c.ta * eb) + iab * VE * eb + ib;
#pragma unroll
            for (uint32_t k = 0; k < VE; ++k) e[k] = col[k * eb];
            *reinterpret_cast<uint4*>(out + (c.dst0 + int64_t(sl) * ea * eb + int64_t(ib) * ea + c.a0 + iab * VE) * ES) =
                    *reinterpret_cast<const uint4*>(e);
            iab += step_a;
            ib += step_b;
            sl += step_s;
            if (iab >= nab) {
                iab -= nab;
                ++ib;
            }
            if (ib >= eb) {
                ib -= eb;
                ++sl;
            }
        }
        __syncthreads();  // this buffer is the target of the copy issued in the next iteration
        if (++cur == kSliceStages) cur = 0;
    }
}

// SubView of 1- / 2- / 4-bit storage — subByteTransform, attributes/subview.cpp:20-160: elements are gathered bit
// field by bit field, low bits first. One thread per output byte (its 8 / BITS elements), so no two threads
// touch the same byte.
__global__ void k_subview_subbyte(const uint8_t* __restrict__ in, uint8_t* __restrict__ out, Geom g, int64_t n_elems, int bits) {
    const int per = 8 / bits;
    const unsigned mask = (1u << bits) - 1u;
    const int64_t n_bytes = (n_elems + per - 1) / per;
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t ob = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; ob < n_bytes; ob += stride) {
        unsigned byte = 0;
        for (int k = 0; k < per; ++k) {
            const int64_t o = ob * per + k;
            if (o >= n_elems) break;
            int64_t rem = o, src = 0;
#pragma unroll
            for (int d = VF_MAX_RANK - 1; d >= 0; --d) {
                if (d < g.rank) {
                    const int64_t c = rem % g.out_shape[d];
                    rem /= g.out_shape[d];
                    src += (c + g.offset[d]) * g.src_stride[d];
                }
            }
            const unsigned v = (unsigned(in[src / per]) >> (unsigned(src % per) * bits)) & mask;
            byte |= v << (k * bits);
        }
        out[ob] = uint8_t(byte);
    }
}

template <int ES>
__device__ __forceinline__ typename ElemOf<ES>::T wide_fill(const uint8_t* __restrict__ fill, int fill_es) {
    // the fill element (fill_es bytes) repeated over the ES bytes of a regrouped element
    __align__(16) uint8_t buf[ES];
#pragma unroll
    for (int k = 0; k < ES; ++k) buf[k] = fill[k % fill_es];
    return *reinterpret_cast<typename ElemOf<ES>::T*>(buf);
}

// PadWithZero — attributes/pad_with_zero.cpp:111-268 + Content::fillWithZero utils/content.cpp:190-237
// Division of a 32-bit index by an extent known at launch (Granlund-Montgomery): q = (t + ((n - t) >> 1)) >> (l - 1)
// with t = umulhi(m, n), l = ceil(log2 d), m = floor(2^32 (2^l - d) / d) + 1; d = 1 has l = 0 and is passed through.
struct FastDivs {
    uint32_t mul[VF_MAX_RANK];
    uint32_t sh[VF_MAX_RANK];  // l; 0: the divisor is 1
};
__device__ __forceinline__ uint32_t fast_div(uint32_t n, uint32_t mul, uint32_t l) {
    if (l == 0) return n;
    const uint32_t t = __umulhi(mul, n);
    return (t + ((n - t) >> 1)) >> (l - 1);
}
template <typename I>
__device__ __forceinline__ I div_extent(I n, I d, const FastDivs& f, int k) {
    return n / d;
}
template <>
__device__ __forceinline__ uint32_t div_extent<uint32_t>(uint32_t n, uint32_t d, const FastDivs& f, int k) {
    return fast_div(n, f.mul[k], f.sh[k]);
}

// Four output elements per thread step, their loads issued together (an SM needs on the order of 100 KB in flight
// to keep the memory busy: one 16-byte load per thread is a third of that).
template <int ES, typename I>
__global__ void k_pad(const void* __restrict__ in, int in_splat, void* __restrict__ out, Geom g, FastDivs fd, I n,
                      const uint8_t* __restrict__ fill, int fill_es, I n_fill, int fill_dim) {
    using T = typename ElemOf<ES>::T;
    constexpr int kU = kInFlight;
    const I stride = I(gridDim.x) * I(blockDim.x);
    for (I o0 = I(blockIdx.x) * I(blockDim.x) + I(threadIdx.x); o0 < n; o0 += I(kU) * stride) {
        T v[kU];
        I fcs[kU];
        bool ins[kU];
#pragma unroll
        for (int u = 0; u < kU; ++u) {
            const I o = o0 + I(u) * stride;
            I rem = o, src = 0, fc = 0;
            bool inside = o < n;
#pragma unroll
            for (int d = VF_MAX_RANK - 1; d >= 0; --d) {
                if (d < g.rank) {
                    const I os = I(g.out_shape[d]);
                    const I q = div_extent<I>(rem, os, fd, d);
                    const I c = rem - q * os;
                    rem = q;
                    if (d == fill_dim) fc = c;
                    const I ci = c - I(g.offset[d]);  // wraps below zero for I = uint32_t: caught by the range test
                    inside &= c >= I(g.offset[d]) && ci < I(g.in_shape[d]);
                    src += ci * I(g.src_stride[d]);
                }
            }
            ins[u] = inside;
            fcs[u] = fc;
            if (inside) v[u] = static_cast<const T*>(in)[in_splat ? I(0) : src];
        }
#pragma unroll
        for (int u = 0; u < kU; ++u) {
            const I o = o0 + I(u) * stride;
            if (o >= n) break;
            if (!ins[u]) v[u] = wide_fill<ES>(fill + (n_fill > 1 ? fcs[u] : I(0)) * I(fill_es), fill_es);
            static_cast<T*>(out)[o] = v[u];
        }
    }
}

// SubView — attributes/subview.cpp:390-432
template <int ES, typename I>
__global__ void k_subview(const void* __restrict__ in, void* __restrict__ out, Geom g, I n) {
    using T = typename ElemOf<ES>::T;
    const I stride = I(gridDim.x) * I(blockDim.x);
    for (I o = I(blockIdx.x) * I(blockDim.x) + I(threadIdx.x); o < n; o += stride) {
        I rem = o, src = 0;
#pragma unroll
        for (int d = VF_MAX_RANK - 1; d >= 0; --d) {
            if (d < g.rank) {
                const I os = I(g.out_shape[d]);
                const I q = rem / os;
                src += (rem - q * os + I(g.offset[d])) * I(g.src_stride[d]);
                rem = q;
            }
        }
        static_cast<T*>(out)[o] = static_cast<const T*>(in)[src];
    }
}

// ------------------------------------------------------------------------------------------------------
// sparsity
// ------------------------------------------------------------------------------------------------------
// sparsity of single tensors (is_dense / sparse_value_as_float: device_utils.cuh)
// One warp per output channel: ballot gives 32 bitmap bits at a time (LSB = lowest index, as
// get_sparsity_map.cpp:44-53 packs them) and popc gives the count.
__global__ void k_sparsity_scan(const void* __restrict__ in, int dt, int64_t oc, int64_t work, long long sv,
                                int64_t* __restrict__ counts, uint8_t* __restrict__ map, int64_t map_row_bytes) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = (int64_t(gridDim.x) * blockDim.x) >> 5;
    const float fv = sparse_value_as_float(dt, sv);
    for (int64_t c = warp; c < oc; c += nwarps) {
        const int64_t base = c * work;
        int64_t cnt = 0;
        for (int64_t i = 0; i < work; i += 32) {
            const bool d = (i + lane < work) && is_dense(in, dt, base + i + lane, sv, fv);
            const unsigned bits = __ballot_sync(0xffffffffu, d);
            cnt += __popc(bits);
            if (map && lane < 4) {
                const int64_t byte = (i >> 3) + lane;
                if (byte * 8 < work) map[c * map_row_bytes + byte] = uint8_t(bits >> (8 * lane));
            }
        }
        if (map) {  // zero the padding up to the 128-bit aligned row
            for (int64_t b = ((work + 7) >> 3) + lane; b < map_row_bytes; b += 32) map[c * map_row_bytes + b] = 0;
        }
        if (counts && lane == 0) counts[c] = cnt;
    }
}

// Single-block exclusive scan of align16(count*es): offsets[0..oc], total in offsets[oc].
__global__ void k_sparse_offsets(const int64_t* __restrict__ counts, int64_t oc, int es, int64_t* __restrict__ offsets) {
    __shared__ long long warp_sums[32];
    __shared__ long long carry_s;
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    if (tid == 0) carry_s = 0;
    __syncthreads();
    for (int64_t base = 0; base < oc; base += blockDim.x) {
        const int64_t i = base + tid;
        long long v = 0;
        if (i < oc) v = ((counts[i] * es + 15) / 16) * 16;
        long long incl = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const long long t = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += t;
        }
        if (lane == 31) warp_sums[wid] = incl;
        __syncthreads();
        if (wid == 0) {
            long long w = lane < (blockDim.x >> 5) ? warp_sums[lane] : 0;
            long long wi = w;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const long long t = __shfl_up_sync(0xffffffffu, wi, o);
                if (lane >= o) wi += t;
            }
            warp_sums[lane] = wi - w;  // exclusive
        }
        __syncthreads();
        const long long carry = carry_s;
        const long long excl = carry + warp_sums[wid] + incl - v;
        if (i < oc) offsets[i] = excl;
        __syncthreads();
        if (tid == blockDim.x - 1) carry_s = excl + v;
        __syncthreads();
    }
    if (tid == 0) offsets[oc] = carry_s;
}

// Sparsify — attributes/sparsify.cpp:120-161. One warp per output channel; within a 32-element step the
// destination of a kept element is the running count plus popc of the lower lanes' ballot bits.
template <int ES>
__global__ void k_sparse_compact(const void* __restrict__ in, int dt, int64_t oc, int64_t work, long long sv,
                                 const int64_t* __restrict__ offsets, uint8_t* __restrict__ out, uint64_t capacity,
                                 int* flags) {
    using T = typename ElemOf<ES>::T;
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = (int64_t(gridDim.x) * blockDim.x) >> 5;
    const float fv = sparse_value_as_float(dt, sv);
    for (int64_t c = warp; c < oc; c += nwarps) {
        const int64_t base = c * work;
        const uint64_t obyte = uint64_t(offsets[c]);
        int64_t run = 0;
        for (int64_t i = 0; i < work; i += 32) {
            const bool d = (i + lane < work) && is_dense(in, dt, base + i + lane, sv, fv);
            const unsigned bits = __ballot_sync(0xffffffffu, d);
            if (d) {
                const uint64_t pos = obyte + uint64_t(run + __popc(bits & ((1u << lane) - 1u))) * ES;
                if (pos + ES <= capacity) *reinterpret_cast<T*>(out + pos) = static_cast<const T*>(in)[base + i + lane];
                else set_flag(flags, VF_FLAG_OVERFLOW);
            }
            run += __popc(bits);
        }
        // zero the gap up to the next channel's 16-byte aligned start (the reference pre-zeroes the buffer)
        const uint64_t end = obyte + uint64_t(run) * ES;
        const uint64_t next = uint64_t(offsets[c + 1]);
        for (uint64_t b = end + lane; b < next && b < capacity; b += 32) out[b] = 0;
    }
}

// ------------------------------------------------------------------------------------------------------
// unit statistics → calcScaleAndZeroPoint
// ------------------------------------------------------------------------------------------------------
__global__ void k_unit_stats(const void* __restrict__ in, int in_dt, int64_t units, int64_t len, int range_mode,
                             long long qmin, long long qmax, double* __restrict__ scales, int64_t* __restrict__ zps,
                             float* __restrict__ rmin, float* __restrict__ rmax, int* flags) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = (int64_t(gridDim.x) * blockDim.x) >> 5;
    for (int64_t u = warp; u < units; u += nwarps) {
        float mn = 0.f, mx = 0.f;
        for (int64_t i = lane; i < len; i += 32) {
            const float v = load_as_f32(in, in_dt, u * len + i, flags);
            mn = v < mn ? v : mn;
            mx = v > mx ? v : mx;
        }
        mn = warp_min(mn);
        mx = warp_max(mx);
        if (range_mode == VF_RANGE_ABSMAX) {
            const float a = fmaxf(-mn, mx);
            mn = -a;
            mx = a;
        }
        if (lane == 0) {
            double sc = 0.0;
            long long zp = 0;
            if (!calc_scale_zp(double(qmin), double(qmax), double(mn), double(mx), sc, zp)) {
                set_flag(flags, VF_FLAG_QUANT_RANGE);
            }
            zp = zp < qmin ? qmin : (zp > qmax ? qmax : zp);
            if (scales) scales[u] = sc;
            if (zps) zps[u] = zp;
            if (rmin) rmin[u] = mn;
            if (rmax) rmax[u] = mx;
        }
    }
}

// ------------------------------------------------------------------------------------------------------
// weights table — dialect/VPU/utils/nce_sparsity.cpp:97-136,195-231,317-347 with the NPU37XX converters
// (NPU37XX/dialect/VPU/impl/nce_sparsity_converters.cpp:14-42)
// ------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void weights_table_row(const TableArgs& a, int64_t oc, int32_t* __restrict__ table, int* flags) {
    const double ws = a.weights_quantized ? a.d_wscale[a.n_wscale > 1 ? oc : 0] : 1.0;
    const double is = a.d_in_scale ? a.d_in_scale[oc] : a.in_scale;
    const double os = a.d_out_scale ? a.d_out_scale[oc] : a.out_scale;

    int32_t wp, sp;
    if (a.d_nnz_offsets) wp = int32_t(a.wbase + a.d_nnz_offsets[oc]);
    else if (a.d_wptrs) wp = a.d_wptrs[oc];
    else wp = int32_t(a.wbase + int64_t(a.wstep) * oc);
    if (a.d_sptrs) sp = a.d_sptrs[oc];
    else sp = int32_t(a.sbase + int64_t(a.sstep) * oc);
    if (wp % 16 != 0) set_flag(flags, VF_FLAG_TABLE_ALIGN);
    if (sp != VF_SPARSITY_PTR_WHEN_NO_SPARSITY && sp % 16 != 0) set_flag(flags, VF_FLAG_TABLE_ALIGN);

    // rescale and its 15-bit approximation: approximate<>() utils/quantization.hpp:65-77
    const double rescale = __dmul_rn(__ddiv_rn(__dmul_rn(ws, is), os), a.const_scale);
    int exponent = 0;
    const double mantissa = frexp(rescale, &exponent);
    const double m = floor(__dmul_rn(mantissa, 32768.0));
    if (exponent > 15) set_flag(flags, VF_FLAG_TABLE_RANGE);          // postShift != 0 — quantization.cpp:429-432
    const int shift = 15 - exponent;
    if (shift > 255) set_flag(flags, VF_FLAG_CHECKED_CAST);          // checked_cast<uint8_t>(bits - exponent)
    if (!(m >= -32768.0 && m <= 32767.0)) set_flag(flags, VF_FLAG_CHECKED_CAST);  // checked_cast<int16_t>(mult)
    int32_t ms;
    if (a.in_is_float) {
        ms = __float_as_int(__double2float_rn(rescale));
    } else {
        const int32_t mult = int32_t(m);
        ms = int32_t((uint32_t(shift) << 8) | (uint32_t(mult) << 16));
    }

    int32_t bias = 0;
    if (a.d_bias) {
        const float b = a.d_bias[a.bias_is_splat ? 0 : oc];
        if (a.in_quantized) {
            // getRescaledBias: bias / (weightsScale * inScale) in FP64, strict int32 range, then std::round
            const double rb = __ddiv_rn(double(b), __dmul_rn(ws, is));
            if (!(rb > -2147483648.0 && rb < 2147483647.0)) {
                set_flag(flags, VF_FLAG_TABLE_RANGE);
            } else {
                bias = int32_t(round(rb));
            }
        } else {
            float bv = b;
            if (a.weights_quantized) bv = __double2float_rn(__ddiv_rn(double(bv), ws));  // float /= double
            bias = __float_as_int(bv);
        }
    }
    table[oc * 4 + 0] = wp;
    table[oc * 4 + 1] = sp;
    table[oc * 4 + 2] = ms;
    table[oc * 4 + 3] = bias;
}

__global__ void k_weights_table(TableArgs a, int32_t* __restrict__ table, int* flags) {
    const int64_t oc = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (oc < a.oc) weights_table_row(a, oc, table, flags);
}

// Many tables per launch: thread u handles row u - unit_begin of the table whose range holds u.
__global__ void k_weights_table_batch(const TableArgs* __restrict__ tabs, int n, int64_t total, int* flags) {
    chain_enter();
    // the tables' first rows, copied into shared memory once per CTA: the search below is a chain of dependent
    // loads, each an L2 round trip when it runs on the table in device memory
    constexpr int kStaged = 512;
    __shared__ int64_t begins[kStaged];
    const bool staged = n <= kStaged;
    if (staged) {
        for (int i = threadIdx.x; i < n; i += blockDim.x) begins[i] = tabs[i].unit_begin;
        __syncthreads();
    }
    const int64_t u = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (u >= total) return;
    int lo = 0, hi = n - 1;
    while (lo < hi) {  // last table whose unit_begin <= u
        const int mid = (lo + hi + 1) >> 1;
        if ((staged ? begins[mid] : tabs[mid].unit_begin) <= u) lo = mid;
        else hi = mid - 1;
    }
    const TableArgs a = tabs[lo];
    weights_table_row(a, u - a.unit_begin, a.d_table, flags);
}

// ---- Reverse / Broadcast / ExpandDilated / ScalarMultInverse ------------------------------------------
template <int ES>
struct ElemBits;
template <>
struct ElemBits<1> { using type = uint8_t; };
template <>
struct ElemBits<2> { using type = uint16_t; };
template <>
struct ElemBits<4> { using type = uint32_t; };
template <>
struct ElemBits<8> { using type = uint64_t; };

template <>
struct ElemBits<16> { using type = uint4; };

// Index arithmetic runs in 32 bits whenever the buffer has fewer than 2^31 elements (64-bit divisions cost an
// order of magnitude more).
template <typename I>
__device__ __forceinline__ I first_index() {
    return I(blockIdx.x) * I(blockDim.x) + I(threadIdx.x);
}
template <typename I>
__device__ __forceinline__ I index_stride() {
    return I(gridDim.x) * I(blockDim.x);
}

// the elements of one 16-byte vector in reverse order
template <int ES>
__device__ __forceinline__ uint4 reverse_vec(uint4 v) {
    if (ES == 1) return make_uint4(__byte_perm(v.w, 0, 0x0123), __byte_perm(v.z, 0, 0x0123), __byte_perm(v.y, 0, 0x0123), __byte_perm(v.x, 0, 0x0123));
    if (ES == 2) return make_uint4(__byte_perm(v.w, 0, 0x1032), __byte_perm(v.z, 0, 0x1032), __byte_perm(v.y, 0, 0x1032), __byte_perm(v.x, 0, 0x1032));
    if (ES == 4) return make_uint4(v.w, v.z, v.y, v.x);
    return make_uint4(v.z, v.w, v.x, v.y);
}

// Reverse — attributes/reverse.cpp:46-80: every run of `run` consecutive elements of the buffer is reversed.
// Vector form (run a multiple of the 16 / ES elements of a vector, both buffers 16-byte aligned): output vector
// j of a run is input vector (last - j) with its elements reversed.
template <int ES, typename I>
__global__ void k_reverse_vec(const uint4* __restrict__ in, uint4* __restrict__ out, I n_vec, I run_vec) {
    const I stride = index_stride<I>();
    for (I v = first_index<I>(); v < n_vec; v += stride) {
        const I r = v % run_vec;
        out[v] = reverse_vec<ES>(__ldg(in + (v - r + (run_vec - 1 - r))));
    }
}
template <int ES, typename I>
__global__ void k_reverse(const void* __restrict__ in, void* __restrict__ out, I n, I run) {
    using T = typename ElemBits<ES>::type;
    const I stride = index_stride<I>();
    for (I i = first_index<I>(); i < n; i += stride) {
        const I r = i % run;
        static_cast<T*>(out)[i] = static_cast<const T*>(in)[i - r + (run - 1 - r)];
    }
}

// Broadcast — attributes/broadcast.cpp:85-124: each block of `after` elements is written `factor` times in a row.
// ES is the widest power of two (up to 16 bytes) that divides the block size and both addresses.
template <int ES, typename I>
__global__ void k_broadcast(const void* __restrict__ in, void* __restrict__ out, I n_out, I after, I factor) {
    using T = typename ElemBits<ES>::type;
    const I stride = index_stride<I>();
    const I group = after * factor;
    // one element per thread step: neighbouring threads read neighbouring source elements and a source block is
    // read `factor` times in a row, from the L1 (four strided elements per thread lose that: 0.89 -> 0.70)
    for (I o = first_index<I>(); o < n_out; o += stride) {
        const I pre = o / group;
        static_cast<T*>(out)[o] = static_cast<const T*>(in)[pre * after + (o - pre * group) % after];
    }
}

// ExpandDilated — attributes/expand_dilated.cpp:88-131: raw OIYX index arithmetic whatever the dims order;
// positions between the taps hold the fill value (zero, or the zero point of output channel `fill` index)
// One output row (dkx elements) per thread step: the divisions happen once per row, the taps of a row are
// consecutive input elements, and neighbouring threads write neighbouring rows.
template <int ES, typename I>
__global__ void k_expand_dilated(const void* __restrict__ in, int in_splat, void* __restrict__ out, I n_rows, I dky, I dkx, I ky,
                                 I kx, I dil_y, I dil_x, const void* __restrict__ fill, I n_fill, I fill_stride, I fill_extent) {
    using T = typename ElemBits<ES>::type;
    const I stride = index_stride<I>();
    for (I row = first_index<I>(); row < n_rows; row += stride) {
        const I plane = row / dky, y = row - plane * dky;
        const I ty = y / dil_y;
        const bool tap_row = ty * dil_y == y;
        const T* src = static_cast<const T*>(in) + (in_splat ? I(0) : (plane * ky + ty) * kx);
        T* dst = static_cast<T*>(out) + row * dkx;
        I next_tap = 0, tap = 0;  // x of the next tap and its index in the input row
        for (I x = 0; x < dkx; ++x) {
            T v;
            if (tap_row && x == next_tap) {
                v = src[in_splat ? I(0) : tap];
                ++tap;
                next_tap += dil_x;
            } else {
                const I o = row * dkx + x;
                v = static_cast<const T*>(fill)[n_fill > 1 ? (o / fill_stride) % fill_extent : I(0)];
            }
            dst[x] = v;
        }
    }
}

// The same transformation, output-centric: each thread step produces 16 bytes of consecutive output (full-width
// coalesced stores). A table in shared memory maps a position inside one dilated plane (dky * dkx elements) to
// the tap it copies, or to -1 for a gap, so a step costs one division (its plane) and per element one table
// read and one gathered load. Every input element is read exactly once. Needs a 16-byte aligned output,
// ES < 16 and a plane that fits the table.
template <int ES, typename I>
__global__ void k_expand_dilated_lut(const void* __restrict__ in, int in_splat, void* __restrict__ out, I n_out, I dky, I dkx,
                                     I ky, I kx, I dil_y, I dil_x, const void* __restrict__ fill, I n_fill, I fill_stride,
                                     I fill_extent) {
    using T = typename ElemBits<ES>::type;
    constexpr int VEC = 16 / ES;
    extern __shared__ int tap_of[];
    const I plane_out = dky * dkx, plane_in = ky * kx;
    for (I p = threadIdx.x; p < plane_out; p += blockDim.x) {
        const I y = p / dkx, x = p - y * dkx;
        const I ty = y / dil_y, tx = x / dil_x;
        tap_of[p] = (ty * dil_y == y && tx * dil_x == x) ? int(ty * kx + tx) : -1;
    }
    __syncthreads();
    const T* src = static_cast<const T*>(in);
    const T* fv = static_cast<const T*>(fill);
    const T fill0 = fv[0];
    const I n_steps = (n_out + I(VEC - 1)) / I(VEC);
    const I stride = index_stride<I>();
    for (I step = first_index<I>(); step < n_steps; step += stride) {
        const I o = step * I(VEC);
        I plane = o / plane_out;
        I p = o - plane * plane_out;
        I base = in_splat ? I(0) : plane * plane_in;
        union {
            T v[VEC];
            uint4 q;
        } pack;
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
            const int tap = tap_of[p];
            T v;
            if (tap >= 0) {
                v = src[in_splat ? I(0) : base + I(tap)];
            } else {
                v = n_fill > 1 ? fv[((o + I(k)) / fill_stride) % fill_extent] : fill0;
            }
            pack.v[k] = v;
            if (++p == plane_out) {
                p = 0;
                base += in_splat ? I(0) : plane_in;
            }
        }
        if (o + I(VEC) <= n_out) {
            static_cast<uint4*>(out)[step] = pack.q;
        } else {
            for (int k = 0; k < VEC && o + I(k) < n_out; ++k) static_cast<T*>(out)[o + I(k)] = pack.v[k];
        }
    }
}

// The same transformation a chunk of planes at a time, through shared memory, for a single fill value: the chunk's
// input planes (contiguous) arrive as 16-byte vectors, the output stage is filled with the fill value by 16-byte
// stores, every tap is moved to its place in its dilated plane (one 2-byte load and store per input element), and
// the stage leaves as 16-byte vectors. Per output element that is about one shared-memory access and no index
// arithmetic, against a table read, a gathered load and a division per vector in the kernel above. A chunk is a
// multiple of 16 planes, so chunks start on 16-byte boundaries on both sides.
template <int ES>
__global__ void __launch_bounds__(256) k_expand_dilated_planes(const uint8_t* __restrict__ in, uint8_t* __restrict__ out, int64_t n_planes,
                                                               uint32_t planes_per_chunk, uint32_t plane_in, uint32_t plane_out, uint32_t kx,
                                                               uint32_t dkx, uint32_t dil_y, uint32_t dil_x, const uint8_t* __restrict__ fill) {
    using T = typename ElemBits<ES>::type;
    extern __shared__ uint4 dil_smem[];
    const uint32_t in_vecs = (planes_per_chunk * plane_in * ES + 15u) / 16u;
    uint4* s_in = dil_smem;
    uint4* s_out = dil_smem + in_vecs;
    __align__(16) uint8_t fb[16];
#pragma unroll
    for (int k = 0; k < 16; ++k) fb[k] = fill[k % ES];
    const uint4 fill_vec = *reinterpret_cast<const uint4*>(fb);
    const int64_t n_chunks = (n_planes + planes_per_chunk - 1) / planes_per_chunk;
    for (int64_t chunk = blockIdx.x; chunk < n_chunks; chunk += gridDim.x) {
        const int64_t p0 = chunk * planes_per_chunk;
        const uint32_t np = uint32_t(min(int64_t(planes_per_chunk), n_planes - p0));
        const uint32_t in_bytes = np * plane_in * ES, out_bytes = np * plane_out * ES;
        const uint8_t* src = in + p0 * plane_in * ES;
        uint8_t* dst = out + p0 * plane_out * ES;
        for (uint32_t v = threadIdx.x; v * 16 < in_bytes; v += blockDim.x) {
            if (v * 16 + 16 <= in_bytes) {
                s_in[v] = __ldg(reinterpret_cast<const uint4*>(src) + v);
            } else {  // the last vector of the last chunk may be cut short
                uint8_t* sb = reinterpret_cast<uint8_t*>(s_in + v);
                for (uint32_t k = 0; v * 16 + k < in_bytes; ++k) sb[k] = src[v * 16 + k];
            }
        }
        for (uint32_t v = threadIdx.x; v * 16 < out_bytes; v += blockDim.x) s_out[v] = fill_vec;
        __syncthreads();
        const T* ti = reinterpret_cast<const T*>(s_in);
        T* to = reinterpret_cast<T*>(s_out);
        for (uint32_t p = threadIdx.x; p < np; p += blockDim.x) {
            const T* pi = ti + p * plane_in;
            T* po = to + p * plane_out;
            uint32_t ty = 0, tx = 0;
            for (uint32_t t = 0; t < plane_in; ++t) {
                po[ty * dil_y * dkx + tx * dil_x] = pi[t];
                if (++tx == kx) {
                    tx = 0;
                    ++ty;
                }
            }
        }
        __syncthreads();
        for (uint32_t v = threadIdx.x; v * 16 < out_bytes; v += blockDim.x) {
            if (v * 16 + 16 <= out_bytes) {
                reinterpret_cast<uint4*>(dst)[v] = s_out[v];
            } else {
                const uint8_t* sb = reinterpret_cast<const uint8_t*>(s_out + v);
                for (uint32_t k = 0; v * 16 + k < out_bytes; ++k) dst[v * 16 + k] = sb[k];
            }
        }
        __syncthreads();  // the stages are rewritten by the next chunk
    }
}

// ScalarMultInverse — attributes/inverse.cpp:52-66: 1.f / v in f32; zero, subnormal, infinite or NaN input throws
__device__ __forceinline__ float inverse_checked(float v, int* flags) {
    const uint32_t e = (__float_as_uint(v) >> 23) & 0xFFu;
    if (e == 0u || e == 0xFFu) set_flag(flags, VF_FLAG_NOT_NORMAL);
    return __fdiv_rn(1.0f, v);
}
__global__ void k_inverse(const void* __restrict__ in, int in_dt, float* __restrict__ out, int64_t n, int* flags) {
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
        out[i] = inverse_checked(load_as_f32(in, in_dt, i, flags), flags);
}
__global__ void k_inverse_f32x4(const float4* __restrict__ in, float4* __restrict__ out, int64_t n_vec, int* flags) {
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n_vec; i += stride) {
        const float4 v = __ldg(in + i);
        out[i] = make_float4(inverse_checked(v.x, flags), inverse_checked(v.y, flags), inverse_checked(v.z, flags), inverse_checked(v.w, flags));
    }
}

// copyTo between floating types, eight elements per thread step (16-byte accesses where the type allows):
// the same conversions as k_convert, chosen at compile time.
template <int DT>
struct FloatBytes { static constexpr int value = DT == VF_DT_F32 ? 4 : (DT == VF_DT_F16 || DT == VF_DT_BF16) ? 2 : 1; };
template <int IN, int OUT>
__global__ void k_convert_float8(const void* __restrict__ in, void* __restrict__ out, int64_t n_groups, int* flags) {
    constexpr int IB = FloatBytes<IN>::value * 8, OB = FloatBytes<OUT>::value * 8;  // bytes of eight elements
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t g = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; g < n_groups; g += stride) {
        __align__(16) uint8_t ib[IB];
        __align__(16) uint8_t ob[OB];
        if (IB == 32) {
            reinterpret_cast<uint4*>(ib)[0] = __ldg(reinterpret_cast<const uint4*>(in) + 2 * g);
            reinterpret_cast<uint4*>(ib)[1] = __ldg(reinterpret_cast<const uint4*>(in) + 2 * g + 1);
        } else if (IB == 16) {
            reinterpret_cast<uint4*>(ib)[0] = __ldg(reinterpret_cast<const uint4*>(in) + g);
        } else {
            reinterpret_cast<uint2*>(ib)[0] = __ldg(reinterpret_cast<const uint2*>(in) + g);
        }
        if (OUT == VF_DT_F8E4M3FN) {
            // The reference's sequence (src/vpux_utils/src/core/type/float8_e4m3.cpp:52-113) rounds to nearest even
            // onto 3 mantissa bits and turns everything that would round above 448 (|x| > 464, infinities, NaN)
            // into the NaN pattern. It rounds the mantissa BEFORE it looks at the exponent: below 2^-7 (subnormal
            // results) a mantissa of 1.1111... carries into the exponent first and the subnormal is then rounded
            // from twice the value. The conversion instruction rounds two elements at a time; it is given 2x for
            // those inputs, and pairs with an element beyond 464 (the instruction would saturate) take the
            // sequence as written.
#pragma unroll
            for (int k = 0; k < 8; k += 2) {
                float f0 = load_as_f32(ib, IN, k, flags), f1 = load_as_f32(ib, IN, k + 1, flags);
                uint32_t two;
                if (fabsf(f0) <= 464.f && fabsf(f1) <= 464.f) {  // false for NaN
                    const uint32_t u0 = __float_as_uint(f0), u1 = __float_as_uint(f1);
                    if ((u0 & 0x7FFFFFFFu) < 0x3C000000u && (u0 & 0x00780000u) == 0x00780000u) f0 = __fmul_rn(f0, 2.f);
                    if ((u1 & 0x7FFFFFFFu) < 0x3C000000u && (u1 & 0x00780000u) == 0x00780000u) f1 = __fmul_rn(f1, 2.f);
                    two = __nv_cvt_float2_to_fp8x2(make_float2(f0, f1), __NV_SATFINITE, __NV_E4M3);
                } else {
                    two = uint32_t(f32_bits_to_f8e4m3_bits(__float_as_uint(f0))) | (uint32_t(f32_bits_to_f8e4m3_bits(__float_as_uint(f1))) << 8);
                }
                reinterpret_cast<uint16_t*>(ob)[k >> 1] = uint16_t(two);
            }
        } else {
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const float f = load_as_f32(ib, IN, k, flags);
                if (OUT == VF_DT_F32) reinterpret_cast<float*>(ob)[k] = f;
                else if (OUT == VF_DT_F16) reinterpret_cast<uint16_t*>(ob)[k] = f32_to_f16_clamped_bits(f);
                else if (OUT == VF_DT_BF16) reinterpret_cast<uint16_t*>(ob)[k] = f32_to_bf16_bits(f);
                else ob[k] = f16_bits_to_f8e5m2_bits(f32_to_f16_bits(f));
            }
        }
        if (OB == 32) {
            reinterpret_cast<uint4*>(out)[2 * g] = reinterpret_cast<uint4*>(ob)[0];
            reinterpret_cast<uint4*>(out)[2 * g + 1] = reinterpret_cast<uint4*>(ob)[1];
        } else if (OB == 16) {
            reinterpret_cast<uint4*>(out)[g] = reinterpret_cast<uint4*>(ob)[0];
        } else {
            reinterpret_cast<uint2*>(out)[g] = reinterpret_cast<uint2*>(ob)[0];
        }
    }
}

// RelocateWeightsTable — attributes/relocate_weights_table.cpp:203-292. One thread per table row of four
// 32-bit entries: columns 0 and 1 are rewritten from the cluster's base pointers, columns 2 and 3 are copied.
// The steps between consecutive channels come from the first two rows of the INPUT table, so the pass writes a
// new buffer. Rows past `oc` (a table inside a larger fused constant) are copied unchanged by the caller.
__global__ void k_relocate(const int32_t* __restrict__ in, int32_t* __restrict__ out, RelocateArgs a, int* flags) {
    const int64_t oc = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (oc >= a.oc) return;
    int32_t row[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) row[c] = a.in_splat ? in[0] : in[oc * 4 + c];
    uint32_t wstep = 0, sstep = 0;  // int32 differences; they wrap like the two's-complement machine the reference runs on
    if (a.oc >= 2 && !a.in_splat) {
        wstep = uint32_t(in[4]) - uint32_t(in[0]);
        sstep = uint32_t(in[5]) - uint32_t(in[1]);
    }
    int cl = 0;  // cluster of this channel: boundaries the reference's sequential walk has crossed at oc
    for (int c = 1; c < a.n_clusters; ++c) cl += a.cross[c] <= oc ? 1 : 0;
    const int64_t rel = oc - a.offsets[cl];
    const int64_t step = a.d_steps ? a.d_steps[oc] : int64_t(int32_t(wstep)) * rel;
    const uint32_t woff = a.d_steps ? a.wptr_offset : uint32_t(a.channel_offset) * wstep;
    const int64_t w = int64_t(a.weights_ptr[cl]) + step;
    if (w < INT32_MIN || w > INT32_MAX) set_flag(flags, VF_FLAG_CHECKED_CAST);
    row[0] = int32_t(uint32_t(w) + woff);
    if (row[1] != 0xFFFFFF) {  // SPARSITY_PTR_WHEN_NO_SPARSITY stays
        const int64_t s = int64_t(a.sparsity_ptr) + rel * int64_t(int32_t(sstep));
        if (s < INT32_MIN || s > INT32_MAX) set_flag(flags, VF_FLAG_CHECKED_CAST);
        row[1] = int32_t(uint32_t(s) + uint32_t(a.channel_offset) * sstep);
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) out[oc * 4 + c] = row[c];
}

// ------------------------------------------------------------------------------------------------------
// synthetic weights
// ------------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint64_t mix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

__device__ __forceinline__ float synth_value(uint64_t key, uint64_t g, float c, float omult, uint64_t omask,
                                             int mask_zero, int dense_mod, int64_t row_len) {
    const uint64_t h = mix64(key + g);
    const int sum = int(h & 0xFFFF) + int((h >> 16) & 0xFFFF) + int((h >> 32) & 0xFFFF) + int((h >> 48) & 0xFFFF) - 131070;
    float v = __fmul_rn(float(sum), c);
    const uint64_t h2 = mix64(h);
    if (omult != 0.f && (h2 & omask) == 0) v = __fmul_rn(v, omult);
    if (mask_zero) {
        bool dense = false;
        if (dense_mod > 0 && row_len > 0) {
            const uint64_t row = g / uint64_t(row_len);
            dense = (mix64(key ^ (row * 0x9E3779B97F4A7C15ull + 0x632BE59BD9B4E019ull)) % uint64_t(dense_mod)) == 0;
        }
        if (!dense && ((h2 >> 40) & 1)) v = 0.f;
    }
    return v;
}

template <int DT>
__global__ void k_synth(void* __restrict__ dst, uint64_t count, uint64_t key, uint64_t first, float c, float omult,
                        uint64_t omask, int mask_zero, int dense_mod, int64_t row_len) {
    const uint64_t stride = uint64_t(gridDim.x) * blockDim.x;
    for (uint64_t i = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += stride) {
        const float v = synth_value(key, first + i, c, omult, omask, mask_zero, dense_mod, row_len);
        if (DT == VF_DT_F32) static_cast<float*>(dst)[i] = v;
        else if (DT == VF_DT_F16) static_cast<uint16_t*>(dst)[i] = __half_as_ushort(__float2half_rn(v));
        else static_cast<uint16_t*>(dst)[i] = __bfloat16_as_ushort(__float2bfloat16_rn(v));
    }
}

__global__ void k_pack_params(const double* __restrict__ scales, const int64_t* __restrict__ zps, int64_t units,
                              uint16_t* __restrict__ scales_f16, uint8_t* __restrict__ zps_u4) {
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t u = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; u < units; u += stride) {
        if (scales_f16) scales_f16[u] = f32_to_f16_bits(__double2float_rn(scales[u]));
        if (zps_u4 && (u & 1) == 0) {
            const unsigned lo = unsigned(zps[u]) & 0xFu;
            const unsigned hi = u + 1 < units ? (unsigned(zps[u + 1]) & 0xFu) : 0u;
            zps_u4[u >> 1] = uint8_t((hi << 4) | lo);
        }
    }
}

uint64_t mix64_host(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

void post_launch(vf_ctx* ctx, int n = 1) {
    VF_CUDA(cudaGetLastError());
    ctx->launches += uint64_t(n);
}

}  // namespace

// ======================================================================================================
// launch wrappers
// ======================================================================================================
void launch_quantize(vf_ctx* ctx, const void* in, int in_dt, bool in_splat, void* out, int out_dt, int64_t n,
                     const double* d_scales, const int64_t* d_zps, int64_t axis_size, int64_t inner, int64_t qmin,
                     int64_t qmax) {
    if (n <= 0) return;
    const bool f_in = in_dt == VF_DT_F32 || in_dt == VF_DT_F16 || in_dt == VF_DT_BF16;
    if (!in_splat && f_in && (out_dt == VF_DT_I8 || out_dt == VF_DT_U8) && n % 8 == 0 && (axis_size <= 1 || inner % 8 == 0) &&
        aligned16(in, out)) {
        const int64_t groups = n / 8, inner8 = axis_size > 1 ? inner / 8 : 1;
        const int grid = grid_for(groups);
        uint8_t* o = static_cast<uint8_t*>(out);
        const bool fast = qmax - qmin <= 255 && qmax > qmin && tail_is_identity(qmin, qmax);
        if (fast) {  // packed pairs, a warp per chunk of a row
            const int64_t eps = in_dt == VF_DT_F32 ? 4 : 8;
            const int64_t row_elems = axis_size > 1 ? inner : n, n_rows = n / row_elems, row_steps = row_elems / eps;
            const int64_t per_unit = int64_t(pairs::kPairU) * 32, chunks_per_row = (row_steps + per_unit - 1) / per_unit;
            if (chunks_per_row < (int64_t(1) << 31) && n_rows * chunks_per_row < (int64_t(1) << 31)) {
                const int64_t n_units = n_rows * chunks_per_row;
                const int rgrid = int(std::min<int64_t>((n_units + 7) / 8, int64_t(ctx->sm_count) * 16));
                const uint4* src = static_cast<const uint4*>(in);
#define VF_QR(IN)                                                                                                                 \
    k_quantize_rows<IN><<<rgrid, kBlock, 0, ctx->stream>>>(src, o, uint32_t(n_units), uint32_t(chunks_per_row), uint32_t(axis_size), \
                                                           row_steps, d_scales, d_zps, qmin, qmax, ctx->d_flags)
                if (in_dt == VF_DT_F32) VF_QR(VF_DT_F32);
                else if (in_dt == VF_DT_F16) VF_QR(VF_DT_F16);
                else VF_QR(VF_DT_BF16);
#undef VF_QR
                post_launch(ctx);
                return;
            }
        }
        // by rows: the quantized axis and everything outside it index the row, what is inside it is the row
        const int64_t row_len = axis_size > 1 ? inner8 : groups, n_rows = groups / row_len;
        const int64_t chunk = int64_t(kRowUnroll) * kBlock, chunks_per_row = (row_len + chunk - 1) / chunk;
        if (row_len >= chunk && row_len < (int64_t(1) << 31) && n_rows * chunks_per_row < (int64_t(1) << 31)) {
            const int64_t n_chunks = n_rows * chunks_per_row;
            const int rgrid = int(std::min<int64_t>(n_chunks, int64_t(ctx->sm_count) * 16));
            using I = uint32_t;
#define VF_Q8R(IN)                                                                                                                      \
    k_quantize8_rows<IN, I><<<rgrid, kBlock, 0, ctx->stream>>>(in, o, I(n_rows), I(chunks_per_row), d_scales, d_zps, I(axis_size),      \
                                                               I(row_len), qmin, qmax, ctx->d_flags);
            if (in_dt == VF_DT_F32) { VF_Q8R(VF_DT_F32) }
            else if (in_dt == VF_DT_F16) { VF_Q8R(VF_DT_F16) }
            else { VF_Q8R(VF_DT_BF16) }
#undef VF_Q8R
            post_launch(ctx);
            return;
        }
#define VF_Q8(IN)                                                                                                                       \
    VF_BY_INDEX_WIDTH(groups, (k_quantize8<IN, I><<<grid, kBlock, 0, ctx->stream>>>(in, o, I(groups), d_scales, d_zps, I(axis_size),    \
                                                                                    I(inner8), qmin, qmax, ctx->d_flags)));
        if (in_dt == VF_DT_F32) { VF_Q8(VF_DT_F32); }
        else if (in_dt == VF_DT_F16) { VF_Q8(VF_DT_F16); }
        else { VF_Q8(VF_DT_BF16); }
#undef VF_Q8
        post_launch(ctx);
        return;
    }
    k_quantize<<<grid_for(n), kBlock, 0, ctx->stream>>>(in, in_dt, in_splat, out, out_dt, n, d_scales, d_zps, axis_size,
                                                        inner, qmin, qmax, ctx->d_flags);
    post_launch(ctx);
}

void launch_dequantize(vf_ctx* ctx, const void* in, int in_dt, bool in_splat, float* out, int64_t n,
                       const double* d_scales, const int64_t* d_zps, int64_t axis_size, int64_t inner) {
    if (n <= 0) return;
    if (!in_splat && (in_dt == VF_DT_I8 || in_dt == VF_DT_U8) && n % 8 == 0 && (axis_size <= 1 || inner % 8 == 0) &&
        aligned16(in, out)) {
        const int64_t groups = n / 8, inner8 = axis_size > 1 ? inner / 8 : 1;
        const int grid = grid_for(groups);
        const int64_t row_len = axis_size > 1 ? inner8 : groups, n_rows = groups / row_len;
        {  // packed pairs, a warp per chunk of a row; the per-entry constants come from a preparation launch
            const int64_t row_words = row_len * 2;
            const int64_t per_unit = int64_t(pairs::kDequantU) * 32, cpr = (row_words + per_unit - 1) / per_unit;
            const int64_t n_axis = axis_size > 1 ? axis_size : 1;
            if (cpr < (int64_t(1) << 31) && n_rows * cpr < (int64_t(1) << 31) && n_axis < (int64_t(1) << 28)) {
                const int64_t n_units = n_rows * cpr;
                DBuf rows(ctx, size_t(n_axis) * sizeof(DequantRow));
                k_dequant_rows_prepare<<<unsigned((n_axis + 7) / 8), kBlock, 0, ctx->stream>>>(d_scales, d_zps, uint32_t(n_axis), in_dt == VF_DT_I8,
                                                                                              static_cast<DequantRow*>(rows.p));
                post_launch(ctx);
                const int rgrid = int(std::min<int64_t>((n_units + 7) / 8, int64_t(ctx->sm_count) * 16));
                if (in_dt == VF_DT_I8)
                    k_dequantize_rows<VF_DT_I8><<<rgrid, kBlock, 0, ctx->stream>>>(static_cast<const uint32_t*>(in), reinterpret_cast<float4*>(out),
                                                                                   uint32_t(n_units), uint32_t(cpr), uint32_t(axis_size), row_words,
                                                                                   static_cast<const DequantRow*>(rows.p), d_scales, d_zps);
                else
                    k_dequantize_rows<VF_DT_U8><<<rgrid, kBlock, 0, ctx->stream>>>(static_cast<const uint32_t*>(in), reinterpret_cast<float4*>(out),
                                                                                   uint32_t(n_units), uint32_t(cpr), uint32_t(axis_size), row_words,
                                                                                   static_cast<const DequantRow*>(rows.p), d_scales, d_zps);
                post_launch(ctx);
                return;
            }
        }
        const int64_t chunk = int64_t(kRowUnroll) * kBlock, chunks_per_row = (row_len + chunk - 1) / chunk;
        if (row_len >= chunk && row_len < (int64_t(1) << 31) && n_rows * chunks_per_row < (int64_t(1) << 31)) {
            const int64_t n_chunks = n_rows * chunks_per_row;
            const int rgrid = int(std::min<int64_t>(n_chunks, int64_t(ctx->sm_count) * 16));
            using I = uint32_t;
            if (in_dt == VF_DT_I8)
                k_dequantize8_rows<VF_DT_I8, I><<<rgrid, kBlock, 0, ctx->stream>>>(in, out, I(n_rows), I(chunks_per_row), d_scales, d_zps,
                                                                                   I(axis_size), I(row_len));
            else
                k_dequantize8_rows<VF_DT_U8, I><<<rgrid, kBlock, 0, ctx->stream>>>(in, out, I(n_rows), I(chunks_per_row), d_scales, d_zps,
                                                                                   I(axis_size), I(row_len));
            post_launch(ctx);
            return;
        }
        if (in_dt == VF_DT_I8) {
            VF_BY_INDEX_WIDTH(groups, (k_dequantize8<VF_DT_I8, I><<<grid, kBlock, 0, ctx->stream>>>(in, out, I(groups), d_scales, d_zps,
                                                                                                    I(axis_size), I(inner8))));
        } else {
            VF_BY_INDEX_WIDTH(groups, (k_dequantize8<VF_DT_U8, I><<<grid, kBlock, 0, ctx->stream>>>(in, out, I(groups), d_scales, d_zps,
                                                                                                    I(axis_size), I(inner8))));
        }
        post_launch(ctx);
        return;
    }
    k_dequantize<<<grid_for(n), kBlock, 0, ctx->stream>>>(in, in_dt, in_splat, out, n, d_scales, d_zps, axis_size, inner,
                                                          ctx->d_flags);
    post_launch(ctx);
}

void launch_rescale_add(vf_ctx* ctx, const void* in, int in_dt, bool in_splat, float* out, int64_t n, float c,
                        bool is_add) {
    if (n <= 0) return;
    int64_t done = 0;
    if (!in_splat && n >= 4 && aligned16(in, out) && (in_dt == VF_DT_F32 || in_dt == VF_DT_F16 || in_dt == VF_DT_BF16)) {
        const int64_t items = n / 4;
        const int grid = grid_for(items, kInFlightWide);
        float4* o4 = reinterpret_cast<float4*>(out);
        if (in_dt == VF_DT_F32) k_rescale_add4<VF_DT_F32><<<grid, kBlock, 0, ctx->stream>>>(in, o4, items, c, is_add, ctx->d_flags);
        else if (in_dt == VF_DT_F16) k_rescale_add4<VF_DT_F16><<<grid, kBlock, 0, ctx->stream>>>(in, o4, items, c, is_add, ctx->d_flags);
        else k_rescale_add4<VF_DT_BF16><<<grid, kBlock, 0, ctx->stream>>>(in, o4, items, c, is_add, ctx->d_flags);
        post_launch(ctx);
        done = items * 4;
    }
    if (done < n) {
        k_rescale_add<<<grid_for(n - done), kBlock, 0, ctx->stream>>>(static_cast<const char*>(in) + done * (dtype_bits(in_dt) / 8), in_dt,
                                                                      in_splat, out + done, n - done, c, is_add, ctx->d_flags);
        post_launch(ctx);
    }
}

template <int IN>
bool launch_convert_float8_out(vf_ctx* ctx, const void* in, void* out, int out_dt, int64_t groups) {
    const int grid = grid_for(groups);
    switch (out_dt) {
    case VF_DT_F32: k_convert_float8<IN, VF_DT_F32><<<grid, kBlock, 0, ctx->stream>>>(in, out, groups, ctx->d_flags); return true;
    case VF_DT_F16: k_convert_float8<IN, VF_DT_F16><<<grid, kBlock, 0, ctx->stream>>>(in, out, groups, ctx->d_flags); return true;
    case VF_DT_BF16: k_convert_float8<IN, VF_DT_BF16><<<grid, kBlock, 0, ctx->stream>>>(in, out, groups, ctx->d_flags); return true;
    case VF_DT_F8E4M3FN: k_convert_float8<IN, VF_DT_F8E4M3FN><<<grid, kBlock, 0, ctx->stream>>>(in, out, groups, ctx->d_flags); return true;
    case VF_DT_F8E5M2: k_convert_float8<IN, VF_DT_F8E5M2><<<grid, kBlock, 0, ctx->stream>>>(in, out, groups, ctx->d_flags); return true;
    default: return false;
    }
}

void launch_convert(vf_ctx* ctx, const void* in, int in_dt, bool in_splat, void* out, int out_dt, int64_t n) {
    if (n <= 0) return;
    int64_t done = 0;
    if (!in_splat && n >= 8 && in_dt != out_dt && aligned16(in, out)) {  // float -> float, eight elements per thread step
        const int64_t groups = n / 8;
        bool ok = false;
        switch (in_dt) {
        case VF_DT_F32: ok = launch_convert_float8_out<VF_DT_F32>(ctx, in, out, out_dt, groups); break;
        case VF_DT_F16: ok = launch_convert_float8_out<VF_DT_F16>(ctx, in, out, out_dt, groups); break;
        case VF_DT_BF16: ok = launch_convert_float8_out<VF_DT_BF16>(ctx, in, out, out_dt, groups); break;
        case VF_DT_F8E4M3FN: ok = launch_convert_float8_out<VF_DT_F8E4M3FN>(ctx, in, out, out_dt, groups); break;
        case VF_DT_F8E5M2: ok = launch_convert_float8_out<VF_DT_F8E5M2>(ctx, in, out, out_dt, groups); break;
        default: break;
        }
        if (ok) {
            post_launch(ctx);
            done = groups * 8;
        }
    }
    if (done < n) {
        const char* tin = static_cast<const char*>(in) + (in_splat ? 0 : done * (dtype_bits(in_dt) / 8));
        char* tout = static_cast<char*>(out) + done * (dtype_bits(out_dt) / 8);
        k_convert<<<grid_for(n - done), kBlock, 0, ctx->stream>>>(tin, in_dt, in_splat, tout, out_dt, n - done, ctx->d_flags);
        post_launch(ctx);
    }
}

void launch_pack_subbyte(vf_ctx* ctx, const void* in, int in_dt, uint8_t* out, int64_t n_in, int per_byte) {
    const int64_t n_out = n_in / per_byte;
    if (n_out <= 0) return;
    k_pack_subbyte<<<grid_for(n_out), kBlock, 0, ctx->stream>>>(in, in_dt, out, n_out, per_byte, ctx->d_flags);
    post_launch(ctx);
}

void launch_bitpack4(vf_ctx* ctx, const void* in, int in_dt, uint8_t* out, int64_t n_in) {
    const int64_t n_out = n_in / 2;
    if (n_out <= 0) return;
    const bool aligned = (reinterpret_cast<uintptr_t>(in) % 16 == 0) && (reinterpret_cast<uintptr_t>(out) % 8 == 0);
    if (in_dt == VF_DT_U8 && aligned && n_in % 16 == 0) {
        k_bitpack4_u8<<<grid_for(n_in / 16), kBlock, 0, ctx->stream>>>(static_cast<const uint4*>(in),
                                                                     reinterpret_cast<uint2*>(out), n_in / 16);
    } else {
        k_bitpack4<<<grid_for(n_out), kBlock, 0, ctx->stream>>>(in, in_dt, out, n_out, ctx->d_flags);
    }
    post_launch(ctx);
}

void launch_fill_bytes(vf_ctx* ctx, void* out, uint8_t value, uint64_t bytes) {
    if (!bytes) return;
    k_fill_bytes<<<grid_for(int64_t(bytes)), kBlock, 0, ctx->stream>>>(static_cast<uint8_t*>(out), value, bytes);
    post_launch(ctx);
}

static int64_t out_numel(const Geom& g) {
    int64_t n = 1;
    for (int i = 0; i < g.rank; ++i) n *= g.out_shape[i];
    return n;
}

// ---- host-side simplification of a layout geometry ---------------------------------------------------------
// kind: 0 permute (offset / in_shape unused), 1 subview (source coordinate = c + offset), 2 pad (c - offset,
// inside while below in_shape). `keep` is a dim that must stay as it is (the per-channel fill dim of a pad), or -1.
static void merge_dims(Geom& g, int kind, int& keep) {
    for (int d = g.rank - 2; d >= 0; --d) {
        const int e = d + 1;
        if (d == keep || e == keep) continue;
        bool ok;
        if (kind == 0) {
            ok = g.src_stride[d] == g.src_stride[e] * g.out_shape[e];
        } else {  // the inner dim is taken whole, and the outer one steps over exactly one inner extent
            ok = g.offset[e] == 0 && g.out_shape[e] == g.in_shape[e] && g.src_stride[d] == g.src_stride[e] * g.in_shape[e];
        }
        if (!ok) continue;
        g.offset[d] = g.offset[d] * g.out_shape[e];
        g.in_shape[d] = g.in_shape[d] * g.in_shape[e];
        g.out_shape[d] = g.out_shape[d] * g.out_shape[e];
        g.src_stride[d] = g.src_stride[e];
        for (int k = e; k + 1 < g.rank; ++k) {
            g.out_shape[k] = g.out_shape[k + 1];
            g.in_shape[k] = g.in_shape[k + 1];
            g.src_stride[k] = g.src_stride[k + 1];
            g.offset[k] = g.offset[k + 1];
        }
        --g.rank;
        if (keep > e) --keep;
    }
}

// Regroups a contiguous innermost dim into elements of up to 16 bytes; returns the new element size.
static int widen(Geom& g, int kind, int es, const void* in, const void* out, bool in_splat, int keep) {
    const int L = g.rank - 1;
    if (L < 0 || g.src_stride[L] != 1 || in_splat || L == keep) return es;
    int w = es;
    const uintptr_t addr = reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out);
    while (w < 16) {
        const int64_t k = 2 * w / es;  // elements per regrouped element if we double once more
        bool ok = g.out_shape[L] % k == 0 && (addr % uintptr_t(2 * w)) == 0;
        if (kind != 0) ok = ok && g.in_shape[L] % k == 0 && g.offset[L] % k == 0;
        for (int d = 0; d < L && ok; ++d) ok = g.src_stride[d] % k == 0;
        if (!ok) break;
        w *= 2;
    }
    const int64_t k = w / es;
    if (k > 1) {
        g.out_shape[L] /= k;
        g.in_shape[L] /= k;
        g.offset[L] /= k;
        for (int d = 0; d < L; ++d) g.src_stride[d] /= k;
    }
    return w;
}

static int64_t max_index(const Geom& g, int kind) {  // largest element index any side of the launch can reach
    int64_t src = 0;
    for (int d = 0; d < g.rank; ++d) {
        const int64_t ext = kind == 0 ? g.out_shape[d] : (kind == 1 ? g.out_shape[d] + g.offset[d] : std::max(g.in_shape[d], g.out_shape[d]));
        src += ext * g.src_stride[d];
    }
    return std::max(src, out_numel(g));
}

void launch_permute(vf_ctx* ctx, const void* in, void* out, const Geom& g0, int es0) {
    Geom g = g0;
    if (out_numel(g) <= 0) return;
    int keep = -1;
    merge_dims(g, 0, keep);
    const int es = widen(g, 0, es0, in, out, false, -1);
    const int64_t n = out_numel(g);
    const bool small = max_index(g, 0) < (int64_t(1) << 31);
    // a dim other than the innermost output dim is contiguous in the source: transpose through shared memory
    int b = -1;
    const int a = g.rank - 1;
    for (int d = 0; d < a; ++d)
        if (g.src_stride[d] == 1 && g.out_shape[d] >= 8) b = d;
    if (es <= 4 && a >= 1 && g.src_stride[a - 1] == 1 && g.src_stride[a] == g.out_shape[a - 1] && g.out_shape[a - 1] >= 2 &&
        (g.out_shape[a] * es) % 16 == 0 && aligned16(in, out)) {
        // the two innermost output dims are one contiguous block of the source: whole chunks through shared memory
        const int64_t ea = g.out_shape[a], eb = g.out_shape[a - 1], ve = 16 / es;
        const int64_t budget = 24 * 1024 - 32;  // per buffer, three buffers per CTA
        const int64_t slice_bytes = ea * eb * es;
        SliceGeom sg{};
        sg.ea = uint32_t(ea);
        sg.eb = uint32_t(eb);
        const int o = a - 2;  // the dim that enumerates the slices (none for a rank-2 geometry)
        sg.n_slices = o >= 0 ? uint32_t(g.out_shape[o]) : 1u;
        sg.slice_src = o >= 0 ? g.src_stride[o] : 0;
        int64_t rows = ea, per_group = 1;
        if (slice_bytes > budget) {  // cut the slice into chunks of (nearly) equal row counts
            const int64_t max_rows = budget / (eb * es) / ve * ve;
            const int64_t pieces = max_rows > 0 ? (ea + max_rows - 1) / max_rows : 0;
            rows = pieces > 0 ? ((ea + pieces - 1) / pieces + ve - 1) / ve * ve : 0;
        } else if (o >= 0 && g.src_stride[o] == ea * eb) {  // consecutive slices are contiguous: several per chunk
            per_group = std::min<int64_t>(budget / slice_bytes, sg.n_slices);
        }
        sg.rows = uint32_t(rows);
        sg.chunks_a = rows > 0 ? uint32_t((ea + rows - 1) / rows) : 0u;
        sg.per_group = uint32_t(per_group);
        sg.groups = uint32_t((sg.n_slices + per_group - 1) / per_group);
        int64_t n_chunks = int64_t(sg.chunks_a) * sg.groups, dst_stride = ea * eb * int64_t(sg.n_slices);
        for (int d = o - 1; d >= 0; --d) {  // innermost of the outer dims first: the chunk index is decomposed that way
            sg.outer_shape[sg.n_outer] = g.out_shape[d];
            sg.outer_src[sg.n_outer] = g.src_stride[d];
            sg.outer_dst[sg.n_outer] = dst_stride;
            ++sg.n_outer;
            dst_stride *= g.out_shape[d];
            n_chunks *= g.out_shape[d];
        }
        const bool bank_stride = (ve * eb * es) % 128 == 0;  // lanes of a store vector would meet in one bank
        const bool fits32 = ea < (int64_t(1) << 31) && eb < (int64_t(1) << 31) && ea * eb < (int64_t(1) << 31) && (o < 0 || g.out_shape[o] < (int64_t(1) << 31));
        if (rows * es >= 64 && !bank_stride && fits32 && n_chunks < (int64_t(1) << 40)) {
            int64_t src_elems = 1;
            for (int d = 0; d < g.rank; ++d) src_elems += (g.out_shape[d] - 1) * g.src_stride[d];
            const int64_t total_bytes = src_elems * es;  // the last byte the launch may read lies inside the source buffer
            const uint32_t buf_vecs = uint32_t((per_group * rows * eb * es + 15 + 15) / 16);
            const size_t smem = size_t(buf_vecs) * 16 * kSliceStages;
            const int64_t per_sm = std::max<int64_t>(1, std::min<int64_t>(8, (216 * 1024) / int64_t(smem + 1024)));
            const unsigned blocks = unsigned(std::min<int64_t>(n_chunks, int64_t(ctx->sm_count) * per_sm));
            const uint8_t* src = static_cast<const uint8_t*>(in);
            uint8_t* dst = static_cast<uint8_t*>(out);
#define VF_SLICES(ES_)                                                                                                           \
    {                                                                                                                            \
        if (smem > 48 * 1024) VF_CUDA(cudaFuncSetAttribute(k_transpose_slices<ES_>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem))); \
        k_transpose_slices<ES_><<<blocks, kBlock, smem, ctx->stream>>>(src, dst, sg, n_chunks, buf_vecs, total_bytes);          \
    }
            if (es == 1) VF_SLICES(1) else if (es == 2) VF_SLICES(2) else VF_SLICES(4)
#undef VF_SLICES
            post_launch(ctx);
            return;
        }
    }
    if (es <= 8 && b >= 0 && g.src_stride[a] != 1 && g.out_shape[a] >= 8) {
        const int64_t ta = (g.out_shape[a] + kTile - 1) / kTile, tb = (g.out_shape[b] + kTile - 1) / kTile;
        int64_t others = 1, dst_stride_b = 1;
        for (int d = 0; d < g.rank; ++d)
            if (d != a && d != b) others *= g.out_shape[d];
        for (int d = b + 1; d < g.rank; ++d) dst_stride_b *= g.out_shape[d];
        const int64_t blocks = others * ta * tb;
        if (blocks < (int64_t(1) << 31)) {
            const dim3 block(32, 8);
            if (small) {
                using I = uint32_t;
                VF_BY_ELEM_SIZE(es, (k_permute_tiled<(ES > 8 ? 8 : ES), I><<<unsigned(blocks), block, 0, ctx->stream>>>(in, out, g, b, I(ta), I(tb), I(dst_stride_b))));
            } else {
                using I = int64_t;
                VF_BY_ELEM_SIZE(es, (k_permute_tiled<(ES > 8 ? 8 : ES), I><<<unsigned(blocks), block, 0, ctx->stream>>>(in, out, g, b, I(ta), I(tb), I(dst_stride_b))));
            }
            post_launch(ctx);
            return;
        }
    }
    const int grid = grid_for(n);
    if (small) {
        using I = uint32_t;
        VF_BY_ELEM_SIZE(es, (k_permute<ES, I><<<grid, kBlock, 0, ctx->stream>>>(in, out, g, I(n))));
    } else {
        using I = int64_t;
        VF_BY_ELEM_SIZE(es, (k_permute<ES, I><<<grid, kBlock, 0, ctx->stream>>>(in, out, g, I(n))));
    }
    post_launch(ctx);
}

void launch_pad(vf_ctx* ctx, const void* in, bool in_splat, void* out, const Geom& g0, int es0, const void* d_fill,
                int64_t n_fill, int fill_dim) {
    Geom g = g0;
    if (out_numel(g) <= 0) return;
    int keep = n_fill > 1 ? fill_dim : -1;
    if (!in_splat) merge_dims(g, 2, keep);
    const int es = widen(g, 2, es0, in, out, in_splat, keep);
    const int64_t n = out_numel(g);
    const int grid = grid_for(n, kInFlight);
    const uint8_t* fill = static_cast<const uint8_t*>(d_fill);
    const int fd = n_fill > 1 ? keep : 0;
    FastDivs divs{};
    for (int d = 0; d < g.rank; ++d) {  // used by the 32-bit instantiation only (every extent is below 2^31 there)
        const uint64_t e = uint64_t(g.out_shape[d]);
        uint32_t l = 0;
        while ((uint64_t(1) << l) < e) ++l;
        divs.sh[d] = l;
        divs.mul[d] = e > 1 ? uint32_t(((uint64_t(1) << 32) * ((uint64_t(1) << l) - e)) / e + 1) : 0u;
    }
    if (max_index(g, 2) < (int64_t(1) << 31)) {
        using I = uint32_t;
        VF_BY_ELEM_SIZE(es, (k_pad<ES, I><<<grid, kBlock, 0, ctx->stream>>>(in, in_splat, out, g, divs, I(n), fill, es0, I(n_fill), fd)));
    } else {
        using I = int64_t;
        VF_BY_ELEM_SIZE(es, (k_pad<ES, I><<<grid, kBlock, 0, ctx->stream>>>(in, in_splat, out, g, divs, I(n), fill, es0, I(n_fill), fd)));
    }
    post_launch(ctx);
}

void launch_subview_subbyte(vf_ctx* ctx, const void* in, void* out, const Geom& g, int bits) {
    const int64_t n = out_numel(g);
    if (n <= 0) return;
    const int64_t n_bytes = (n * bits + 7) / 8;
    k_subview_subbyte<<<grid_for(n_bytes), kBlock, 0, ctx->stream>>>(static_cast<const uint8_t*>(in), static_cast<uint8_t*>(out), g, n, bits);
    post_launch(ctx);
}

void launch_subview(vf_ctx* ctx, const void* in, void* out, const Geom& g0, int es0) {
    Geom g = g0;
    if (out_numel(g) <= 0) return;
    int keep = -1;
    merge_dims(g, 1, keep);
    const int es = widen(g, 1, es0, in, out, false, -1);
    const int64_t n = out_numel(g);
    const int grid = grid_for(n);
    if (max_index(g, 1) < (int64_t(1) << 31)) {
        using I = uint32_t;
        VF_BY_ELEM_SIZE(es, (k_subview<ES, I><<<grid, kBlock, 0, ctx->stream>>>(in, out, g, I(n))));
    } else {
        using I = int64_t;
        VF_BY_ELEM_SIZE(es, (k_subview<ES, I><<<grid, kBlock, 0, ctx->stream>>>(in, out, g, I(n))));
    }
    post_launch(ctx);
}

void preload_sparsity_kernels() {
    cudaFuncAttributes a;
    VF_CUDA(cudaFuncGetAttributes(&a, k_sparsity_scan));
    VF_CUDA(cudaFuncGetAttributes(&a, k_sparse_offsets));
    VF_CUDA(cudaFuncGetAttributes(&a, k_sparse_compact<1>));
    VF_CUDA(cudaFuncGetAttributes(&a, k_sparse_compact<2>));
    VF_CUDA(cudaFuncGetAttributes(&a, k_sparse_compact<4>));
}

void launch_sparsity_scan(vf_ctx* ctx, const void* in, int dt, int64_t oc, int64_t work, int64_t sparse_value,
                          int64_t* d_counts, uint8_t* d_map, int64_t map_row_bytes) {
    if (oc <= 0) return;
    const int64_t blocks = (oc + 7) / 8;  // 8 warps per block, one channel per warp
    k_sparsity_scan<<<int(std::min<int64_t>(blocks, int64_t(ctx->sm_count) * 8)), 256, 0, ctx->stream>>>(in, dt, oc, work, sparse_value,
                                                                                      d_counts, d_map, map_row_bytes);
    post_launch(ctx);
}

void launch_sparse_offsets(vf_ctx* ctx, const int64_t* d_counts, int64_t oc, int es, int64_t* d_offsets) {
    k_sparse_offsets<<<1, 1024, 0, ctx->stream>>>(d_counts, oc, es, d_offsets);
    post_launch(ctx);
}

void launch_sparse_compact(vf_ctx* ctx, const void* in, int dt, int64_t oc, int64_t work, int64_t sparse_value,
                           const int64_t* d_offsets, uint8_t* out, uint64_t capacity) {
    if (oc <= 0) return;
    const int64_t blocks = (oc + 7) / 8;
    const int grid = int(std::min<int64_t>(blocks, int64_t(ctx->sm_count) * 8));
    const int es = dtype_bits(dt) / 8;
    switch (es) {
    case 1: k_sparse_compact<1><<<grid, 256, 0, ctx->stream>>>(in, dt, oc, work, sparse_value, d_offsets, out, capacity, ctx->d_flags); break;
    case 2: k_sparse_compact<2><<<grid, 256, 0, ctx->stream>>>(in, dt, oc, work, sparse_value, d_offsets, out, capacity, ctx->d_flags); break;
    default: k_sparse_compact<4><<<grid, 256, 0, ctx->stream>>>(in, dt, oc, work, sparse_value, d_offsets, out, capacity, ctx->d_flags); break;
    }
    post_launch(ctx);
}

void launch_unit_stats(vf_ctx* ctx, const void* in, int in_dt, int64_t units, int64_t unit_len, int range_mode,
                       int64_t qmin, int64_t qmax, double* d_scales, int64_t* d_zps, float* d_rmin, float* d_rmax) {
    if (units <= 0) return;
    const int64_t blocks = (units + 7) / 8;
    k_unit_stats<<<int(std::min<int64_t>(blocks, int64_t(ctx->sm_count) * 16)), 256, 0, ctx->stream>>>(
            in, in_dt, units, unit_len, range_mode, qmin, qmax, d_scales, d_zps, d_rmin, d_rmax, ctx->d_flags);
    post_launch(ctx);
}

void launch_pack_params(vf_ctx* ctx, const double* d_scales, const int64_t* d_zps, int64_t units,
                        uint16_t* scales_f16, uint8_t* zps_u4) {
    if (units <= 0 || (!scales_f16 && !zps_u4)) return;
    k_pack_params<<<grid_for(units), kBlock, 0, ctx->stream>>>(d_scales, d_zps, units, scales_f16, zps_u4);
    post_launch(ctx);
}

void launch_weights_table(vf_ctx* ctx, const TableArgs& a, int32_t* d_table) {
    if (a.oc <= 0) return;
    k_weights_table<<<int((a.oc + 127) / 128), 128, 0, ctx->stream>>>(a, d_table, ctx->d_flags);
    post_launch(ctx);
}

void launch_swizzle(vf_ctx* ctx, const void* in, uint64_t in_bytes, uint8_t pad, void* out, uint64_t bytes, int swizzle_key, int arch) {
    if (!bytes) return;
    if (bytes >= (1ull << 32)) raise(VF_ERR_UNSUPPORTED, "swizzled constants are addressed with 32 bits");
    // AddressTransform::setStaggerBits — attributes/swizzle_transform.cpp:37-56
    const uint32_t bits = uint32_t(swizzle_key) % 6u;
    uint32_t shift = 9u - bits, log2w = 4u, cut_mask = (1u << 9) - 1u;
    if (arch == VF_ARCH_NPU40XX) {
        shift += 1;
        log2w += 1;
        cut_mask = (1u << 10) - 1u;
    }
    const int64_t n_vec = int64_t(bytes / 16);
    k_swizzle<<<grid_for(n_vec), kBlock, 0, ctx->stream>>>(static_cast<const uint4*>(in), std::min<uint64_t>(in_bytes, bytes), pad,
                                                          static_cast<uint4*>(out), n_vec, log2w, (1u << bits) - 1u, shift, cut_mask);
    post_launch(ctx);
}

template <int BITS>
void launch_unpack_bits(vf_ctx* ctx, const uint8_t* in, uint8_t* out, int64_t n_out, int s) {
    int64_t done = 0;
    if (n_out >= 16 && (reinterpret_cast<uintptr_t>(in) % (2 * BITS)) == 0 && (reinterpret_cast<uintptr_t>(out) % 16) == 0) {
        const int64_t items = n_out / 16;
        k_unpack_subbyte_x16<BITS><<<grid_for(items, kInFlightWide), kBlock, 0, ctx->stream>>>(in, reinterpret_cast<uint4*>(out), items, s);
        post_launch(ctx);
        done = items * 16;
    }
    if (done < n_out) {
        k_unpack_subbyte<BITS><<<grid_for((n_out - done + 7) / 8), kBlock, 0, ctx->stream>>>(in + done * BITS / 8, out + done, n_out - done, s);
        post_launch(ctx);
    }
}

void launch_unpack_subbyte(vf_ctx* ctx, const uint8_t* in, uint8_t* out, int64_t n_out, int bits, bool sign_extend) {
    if (n_out <= 0) return;
    const int s = sign_extend ? 1 : 0;
    switch (bits) {
    case 1: launch_unpack_bits<1>(ctx, in, out, n_out, s); break;
    case 2: launch_unpack_bits<2>(ctx, in, out, n_out, s); break;
    case 4: launch_unpack_bits<4>(ctx, in, out, n_out, s); break;
    default: raise(VF_ERR_UNSUPPORTED, "Invalid number of elements per byte for %d-bit elements", bits);
    }
}

void launch_weights_table_batch(vf_ctx* ctx, std::vector<TableArgs>& tabs, const std::vector<OffsetsJob>* offsets_first) {
    if (tabs.empty()) {
        if (offsets_first) launch_offsets_batch(ctx, *offsets_first);
        return;
    }
    int64_t total = 0;
    for (auto& t : tabs) {
        t.unit_begin = total;
        total += t.oc;
    }
    // the two job lists travel as one upload, and nothing stands between the two kernels
    const size_t n_off = offsets_first ? offsets_first->size() : 0;
    const size_t off_bytes = (n_off * sizeof(OffsetsJob) + 15) & ~size_t(15), tab_bytes = tabs.size() * sizeof(TableArgs);
    std::vector<char> both(off_bytes + tab_bytes);
    if (n_off) std::memcpy(both.data(), offsets_first->data(), n_off * sizeof(OffsetsJob));
    std::memcpy(both.data() + off_bytes, tabs.data(), tab_bytes);
    DBuf d;
    const char* d_both = static_cast<const char*>(upload_table(ctx, both.data(), both.size(), d));
    launch_offsets_batch_at(ctx, reinterpret_cast<const OffsetsJob*>(d_both), int(n_off));
    const TableArgs* d_tabs = reinterpret_cast<const TableArgs*>(d_both + off_bytes);
    VF_CUDA(launch_chained(k_weights_table_batch, int((total + 127) / 128), 128, 0, ctx->stream, d_tabs, int(tabs.size()), total, ctx->d_flags));
    ctx->launches += 1;
}

void launch_relocate(vf_ctx* ctx, const int32_t* in, int32_t* out, const RelocateArgs& a) {
    if (a.oc <= 0) return;
    k_relocate<<<int((a.oc + 127) / 128), 128, 0, ctx->stream>>>(in, out, a, ctx->d_flags);
    post_launch(ctx);
}

void launch_reverse(vf_ctx* ctx, const void* in, void* out, int64_t n, int64_t run, int es) {
    if (n <= 0) return;
    const int epv = 16 / es;
    if (es <= 8 && run % epv == 0 && aligned16(in, out)) {
        const int64_t nv = n / epv, rv = run / epv;
        VF_BY_ELEM_SIZE(es, VF_BY_INDEX_WIDTH(nv, (k_reverse_vec<ES, I><<<grid_for(nv), kBlock, 0, ctx->stream>>>(
                                                          static_cast<const uint4*>(in), static_cast<uint4*>(out), I(nv), I(rv)))));
    } else {
        VF_BY_ELEM_SIZE(es, VF_BY_INDEX_WIDTH(n, (k_reverse<ES, I><<<grid_for(n), kBlock, 0, ctx->stream>>>(in, out, I(n), I(run)))));
    }
    post_launch(ctx);
}

void launch_broadcast(vf_ctx* ctx, const void* in, void* out, int64_t n_out, int64_t after, int64_t factor, int es) {
    if (n_out <= 0) return;
    // copy in the widest unit that divides the repeated block and both addresses
    int wide = es;
    const uintptr_t addr = reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out);
    while (wide < 16 && (after * es) % (wide * 2) == 0 && (addr % uintptr_t(wide * 2)) == 0) wide *= 2;
    const int64_t k = wide / es;
    const int64_t n = n_out / k, a = after / k;
    VF_BY_ELEM_SIZE(wide, VF_BY_INDEX_WIDTH(n, (k_broadcast<ES, I><<<grid_for(n), kBlock, 0, ctx->stream>>>(in, out, I(n), I(a), I(factor)))));
    post_launch(ctx);
}

void launch_expand_dilated(vf_ctx* ctx, const void* in, bool in_splat, void* out, int64_t n_out, int64_t dky, int64_t dkx,
                           int64_t ky, int64_t kx, int64_t dil_y, int64_t dil_x, const void* d_fill, int64_t n_fill,
                           int64_t fill_stride, int64_t fill_extent, int es) {
    if (n_out <= 0) return;
    const int64_t n_rows = n_out / dkx;
    {  // a single fill value, planes small enough for a chunk of at least 16 in shared memory: whole chunks staged
        const int64_t plane_in = ky * kx, plane_out = dky * dkx, n_planes = plane_out > 0 ? n_out / plane_out : 0;
        const int64_t per_plane = (plane_in + plane_out) * es;
        int64_t ppc = per_plane > 0 ? std::min<int64_t>(256, (40 * 1024) / per_plane) / 16 * 16 : 0;
        if (!in_splat && n_fill == 1 && es <= 8 && ppc >= 16 && n_planes >= 1 && n_planes * plane_out == n_out && plane_in >= 1 &&
            aligned16(in, out)) {
            const uint32_t in_vecs = uint32_t((ppc * plane_in * es + 15) / 16), out_vecs = uint32_t((ppc * plane_out * es + 15) / 16);
            const size_t smem = size_t(in_vecs + out_vecs) * 16;
            const int64_t n_chunks = (n_planes + ppc - 1) / ppc;
            const int64_t per_sm = std::max<int64_t>(1, std::min<int64_t>(8, (200 * 1024) / int64_t(smem + 1024)));
            const unsigned blocks = unsigned(std::min<int64_t>(n_chunks, int64_t(ctx->sm_count) * per_sm));
            const uint8_t* src = static_cast<const uint8_t*>(in);
            uint8_t* dst = static_cast<uint8_t*>(out);
            const uint8_t* fv = static_cast<const uint8_t*>(d_fill);
#define VF_DIL_PLANES(ES_)                                                                                                           \
    k_expand_dilated_planes<ES_><<<blocks, kBlock, smem, ctx->stream>>>(src, dst, n_planes, uint32_t(ppc), uint32_t(plane_in),          \
                                                                      uint32_t(plane_out), uint32_t(kx), uint32_t(dkx), uint32_t(dil_y), \
                                                                      uint32_t(dil_x), fv)
            switch (es) {
            case 1: VF_DIL_PLANES(1); break;
            case 2: VF_DIL_PLANES(2); break;
            case 4: VF_DIL_PLANES(4); break;
            default: VF_DIL_PLANES(8); break;
            }
#undef VF_DIL_PLANES
            post_launch(ctx);
            return;
        }
    }
    constexpr int64_t kMaxPlane = 8192;  // table entries (32 KiB of shared memory)
    if (es < 16 && reinterpret_cast<uintptr_t>(out) % 16 == 0 && dky * dkx <= kMaxPlane) {
        const int64_t n_steps = (n_out * es + 15) / 16;
        const size_t smem = size_t(dky * dkx) * sizeof(int);
        switch (es) {
#define VF_EXPAND_LUT(ES_)                                                                                                          \
    case ES_:                                                                                                                       \
        VF_BY_INDEX_WIDTH(n_out + 16, (k_expand_dilated_lut<ES_, I><<<grid_for(n_steps), kBlock, smem, ctx->stream>>>(              \
                                          in, in_splat ? 1 : 0, out, I(n_out), I(dky), I(dkx), I(ky), I(kx), I(dil_y), I(dil_x), d_fill, \
                                          I(n_fill), I(fill_stride), I(fill_extent))));                                            \
        break;
            VF_EXPAND_LUT(1)
            VF_EXPAND_LUT(2)
            VF_EXPAND_LUT(4)
            VF_EXPAND_LUT(8)
#undef VF_EXPAND_LUT
        default: raise(VF_ERR_UNSUPPORTED, "ExpandDilated: element size");
        }
        post_launch(ctx);
        return;
    }
    VF_BY_ELEM_SIZE(es, VF_BY_INDEX_WIDTH(n_out, (k_expand_dilated<ES, I><<<grid_for(n_rows), kBlock, 0, ctx->stream>>>(
                                                         in, in_splat ? 1 : 0, out, I(n_rows), I(dky), I(dkx), I(ky), I(kx), I(dil_y), I(dil_x),
                                                         d_fill, I(n_fill), I(fill_stride), I(fill_extent)))));
    post_launch(ctx);
}

void launch_inverse(vf_ctx* ctx, const void* in, int in_dt, float* out, int64_t n) {
    if (n <= 0) return;
    int64_t done = 0;
    if (in_dt == VF_DT_F32 && n >= 4 && aligned16(in, out)) {
        done = n / 4 * 4;
        k_inverse_f32x4<<<grid_for(done / 4), kBlock, 0, ctx->stream>>>(static_cast<const float4*>(in), reinterpret_cast<float4*>(out), done / 4, ctx->d_flags);
        post_launch(ctx);
    }
    if (done < n) {
        k_inverse<<<grid_for(n - done), kBlock, 0, ctx->stream>>>(static_cast<const char*>(in) + done * (dtype_bits(in_dt) / 8), in_dt, out + done,
                                                                 n - done, ctx->d_flags);
        post_launch(ctx);
    }
}

void launch_synth(vf_ctx* ctx, const vf_synth_spec& s, void* dst, uint64_t count) {
    if (!count) return;
    const uint64_t key = mix64_host(s.seed ^ mix64_host(s.tensor_id));
    // sum of four uniform 16-bit integers, centred: standard deviation sqrt((65536^2 - 1) / 3)
    const float c = float(double(s.sigma) / sqrt((65536.0 * 65536.0 - 1.0) / 3.0));
    const uint64_t omask = s.outlier_log2 > 0 ? ((1ull << s.outlier_log2) - 1) : 0;
    const int grid = grid_for(int64_t(count));
    switch (s.dtype) {
    case VF_DT_F32:
        k_synth<VF_DT_F32><<<grid, kBlock, 0, ctx->stream>>>(dst, count, key, s.first_elem, c, s.outlier_mult, omask, s.mask_zero, s.dense_row_mod, s.row_len);
        break;
    case VF_DT_F16:
        k_synth<VF_DT_F16><<<grid, kBlock, 0, ctx->stream>>>(dst, count, key, s.first_elem, c, s.outlier_mult, omask, s.mask_zero, s.dense_row_mod, s.row_len);
        break;
    case VF_DT_BF16:
        k_synth<VF_DT_BF16><<<grid, kBlock, 0, ctx->stream>>>(dst, count, key, s.first_elem, c, s.outlier_mult, omask, s.mask_zero, s.dense_row_mod, s.row_len);
        break;
    default: raise(VF_ERR_UNSUPPORTED, "synthetic weights are f32 / f16 / bf16");
    }
    post_launch(ctx);
}

}  // namespace vf
