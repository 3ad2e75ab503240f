// Fused weight-quantization kernels (the hot path): range statistics, calcScaleAndZeroPoint, Quantize and
// the store stage (BitPack / OIYX->OYXI reorder / zero padding / Dequantize copy) in ONE pass over the
// input. All of them are bandwidth-bound: the unit (group chunk or row) is staged in shared memory with
// 16-byte asynchronous copies (cp.async), statistics are reduced on packed 16-bit pairs with shuffles, the
// quantization sweep re-reads shared memory, stores are 4..16 bytes per lane and coalesced. One launch
// processes a whole table of tensors so that small tensors do not pay a launch and a tail each.
//
// Arithmetic contract: codes equal the reference's fakeQuantize chain bit for bit. The per-element fast path
// evaluates  t = fma(x, inv, c)  with inv = fl((L-1)/range), c = fl(-inLow*inv)  instead of the reference's
// fl(fl((x-inLow)/range) * (L-1)); both lie within 7.6e-5 of each other for 8-bit ranges, so whenever t is
// further than kGuard from a rounding boundary (x.5) both round to the same integer. Elements inside the guard
// band (about 0.04 %) are recomputed with the exact operation sequence.
#include <algorithm>
#include <vector>

#include "device_utils.cuh"
#include "kernels.h"

namespace vf {

namespace {

constexpr float kMagic = 12582912.0f;  // 1.5 * 2^23: adding it rounds to the nearest integer (ties to even)
constexpr int kMagicBits = 0x4B400000; // its bit pattern; the low byte is zero
constexpr float kGuard = 2.0e-4f;

struct UnitQ {  // per-unit constants
    float inv;     // fl((L-1) / range)
    float c;       // fl(-inLow * inv) (+ bias, see k_row)
    float in_low;  // exact path
    float range;   // fl(inHigh - inLow)
};

struct LaunchParams {  // uniform over all jobs of one launch
    int range_mode;
    int qmin, qmax, lm1;
    int dequant_dt;
    int njobs;
    int64_t total_units;  // chunks (k_group) or rows (k_row / k_conv) over all jobs
};

// Per-unit parameters from the unit's range; executed by one lane per unit.
__device__ __forceinline__ void derive_unit(float mn, float mx, const LaunchParams& p, double& scale, long long& zp,
                                            UnitQ& u, int* flags) {
    mn = fminf(mn, 0.f);  // the range always contains zero (calcScaleAndZeroPoint requires it)
    mx = fmaxf(mx, 0.f);
    if (p.range_mode == VF_RANGE_ABSMAX) {
        const float a = fmaxf(-mn, mx);
        mn = -a;
        mx = a;
    }
    if (!calc_scale_zp(double(p.qmin), double(p.qmax), double(mn), double(mx), scale, zp)) {
        set_flag(flags, VF_FLAG_QUANT_RANGE);
        scale = 1.0;
        zp = 0;
    }
    zp = zp < p.qmin ? p.qmin : (zp > p.qmax ? p.qmax : zp);
    u.in_low = dequantize_exact(p.qmin, scale, zp);
    const float in_high = dequantize_exact(p.qmax, scale, zp);
    u.range = __fsub_rn(in_high, u.in_low);
    u.inv = __fdiv_rn(float(p.lm1), u.range);
    u.c = __fmul_rn(-u.in_low, u.inv);
}

// The exact operation sequence of fakeQuantize's middle branch, as an index n in [0, L-1]. The first two
// branches (x <= inLow -> qLow, x > inHigh -> qHigh) coincide with the clamp: x <= inLow gives a <= 0,
// x > inHigh gives fl(x - inLow) >= range.
__device__ __noinline__ int quant_index_exact(float x, float in_low, float range, int lm1) {
    const float a = __fsub_rn(x, in_low);
    float e = __fdiv_rn(a, range);
    e = __fmul_rn(e, float(lm1));
    const int n = int(round_half_away(e));
    return min(max(n, 0), lm1);
}

// ---- 16-bit pair helpers ---------------------------------------------------------------------------------
template <typename InT>
struct P2;
template <>
struct P2<__half> {
    using T = __half2;
    static __device__ __forceinline__ float lo(uint32_t w) { return __half2float(__ushort_as_half(uint16_t(w))); }
    static __device__ __forceinline__ float hi(uint32_t w) { return __half2float(__ushort_as_half(uint16_t(w >> 16))); }
};
template <>
struct P2<__nv_bfloat16> {
    using T = __nv_bfloat162;
    static __device__ __forceinline__ float lo(uint32_t w) { return __uint_as_float(w << 16); }
    static __device__ __forceinline__ float hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }
};

template <typename InT>
__device__ __forceinline__ typename P2<InT>::T as_p2(uint32_t w) {
    return *reinterpret_cast<typename P2<InT>::T*>(&w);
}
template <typename T2>
__device__ __forceinline__ uint32_t as_u32(T2 v) {
    return *reinterpret_cast<uint32_t*>(&v);
}

// min and max of the eight 16-bit values of a 16-byte vector, as (min, -max) packed in one 32-bit pair so that
// a single packed-min reduces both.
template <typename InT>
__device__ __forceinline__ uint32_t minnegmax8(const uint4& d) {
    using T2 = typename P2<InT>::T;
    const T2 a = as_p2<InT>(d.x), b = as_p2<InT>(d.y), c = as_p2<InT>(d.z), e = as_p2<InT>(d.w);
    const T2 mn = __hmin2(__hmin2(a, b), __hmin2(c, e));
    const T2 mx = __hmax2(__hmax2(a, b), __hmax2(c, e));
    const T2 mn1 = __hmin2(mn, __lowhigh2highlow(mn));        // both halves: min
    const T2 ng1 = __hneg2(__hmax2(mx, __lowhigh2highlow(mx)));  // both halves: -max
    return __byte_perm(as_u32(mn1), as_u32(ng1), 0x5410);     // (lo = min, hi = -max)
}
template <typename InT>
__device__ __forceinline__ uint32_t pmin(uint32_t x, uint32_t y) {
    return as_u32(__hmin2(as_p2<InT>(x), as_p2<InT>(y)));
}

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc, bool valid) {
    const uint32_t s = uint32_t(__cvta_generic_to_shared(smem_dst));
    const int n = valid ? 16 : 0;  // src-size 0: the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gsrc), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
    asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
}

// Fast quantization of the eight elements of one vector: returns the eight rounded values as floats with the
// magic constant still added (bit pattern = kMagicBits + n) and whether any of them fell into the guard band.
template <typename InT>
__device__ __forceinline__ bool quant8(const uint4& d, float inv, float c, float* m) {
    const uint32_t w[4] = {d.x, d.y, d.z, d.w};
    bool bad = false;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float x0 = P2<InT>::lo(w[i]), x1 = P2<InT>::hi(w[i]);
        const float t0 = __fmaf_rn(x0, inv, c), t1 = __fmaf_rn(x1, inv, c);
        m[2 * i] = __fadd_rn(t0, kMagic);
        m[2 * i + 1] = __fadd_rn(t1, kMagic);
        const float r0 = __fsub_rn(t0, __fsub_rn(m[2 * i], kMagic));
        const float r1 = __fsub_rn(t1, __fsub_rn(m[2 * i + 1], kMagic));
        bad |= fabsf(r0) > 0.5f - kGuard;
        bad |= fabsf(r1) > 0.5f - kGuard;
    }
    return bad;
}

// Exact recomputation of the eight elements (rare). Everything travels by value so that the caller's
// registers never need an address: returns the eight indices n (0..255) as bytes.
template <typename InT>
__device__ __noinline__ uint2 quant8_exact_bytes(uint4 d, float in_low, float range, int lm1) {
    uint2 r;
    r.x = uint32_t(quant_index_exact(P2<InT>::lo(d.x), in_low, range, lm1)) |
          (uint32_t(quant_index_exact(P2<InT>::hi(d.x), in_low, range, lm1)) << 8) |
          (uint32_t(quant_index_exact(P2<InT>::lo(d.y), in_low, range, lm1)) << 16) |
          (uint32_t(quant_index_exact(P2<InT>::hi(d.y), in_low, range, lm1)) << 24);
    r.y = uint32_t(quant_index_exact(P2<InT>::lo(d.z), in_low, range, lm1)) |
          (uint32_t(quant_index_exact(P2<InT>::hi(d.z), in_low, range, lm1)) << 8) |
          (uint32_t(quant_index_exact(P2<InT>::lo(d.w), in_low, range, lm1)) << 16) |
          (uint32_t(quant_index_exact(P2<InT>::hi(d.w), in_low, range, lm1)) << 24);
    return r;
}

// Overwrites m[] with the patterns kMagicBits + n + bias of the exactly recomputed elements.
#define VF_QUANT8_EXACT(InT, d, in_low, range, lm1, bias, m)                                       \
    do {                                                                                           \
        const uint2 ex_ = quant8_exact_bytes<InT>(d, in_low, range, lm1);                          \
        _Pragma("unroll") for (int k_ = 0; k_ < 4; ++k_) {                                         \
            m[k_] = __int_as_float(kMagicBits + int((ex_.x >> (8 * k_)) & 0xFFu) + (bias));        \
            m[4 + k_] = __int_as_float(kMagicBits + int((ex_.y >> (8 * k_)) & 0xFFu) + (bias));    \
        }                                                                                          \
    } while (0)

// Dequantize + copyTo of one code into a 16-bit float type
__device__ __forceinline__ uint16_t dequant16(int code, long long zp, double scale, int dt) {
    const float f = dequantize_exact(code, scale, zp);
    return dt == VF_DT_F16 ? f32_to_f16_clamped_bits(f) : f32_to_bf16_bits(f);
}

__device__ __forceinline__ int find_job(const RowQuantArgs* __restrict__ jobs, int njobs, int64_t unit) {
    int lo = 0, hi = njobs - 1;
    while (lo < hi) {  // last job whose unit_begin <= unit
        const int mid = (lo + hi + 1) >> 1;
        if (jobs[mid].unit_begin <= unit) lo = mid;
        else hi = mid - 1;
    }
    return lo;
}

// ======================================================================================================
// K_group: units of G consecutive elements (per-group quantization), 2-byte input.
// A warp owns a chunk of 32 consecutive groups (32*G elements): each lane copies V = G/8 vectors into the
// warp's shared-memory stage; every group is reduced by the G/8 lanes that hold it; lane g then derives the
// parameters of group g (all 32 lanes busy in the FP64 section); parameters travel back by shuffle for the
// quantization sweep. Warps loop over the chunks of all jobs of the launch.
// ======================================================================================================
template <typename InT, int G, bool PACK4>
__global__ void __launch_bounds__(256, 3) k_group(const RowQuantArgs* __restrict__ jobs, LaunchParams p, int* flags) {
    constexpr int V = G / 8;       // vectors per lane per chunk
    constexpr int LPG = G / 8;     // lanes per group within one vector row
    constexpr int GPL = 32 / LPG;  // groups completed per vector row
    extern __shared__ uint4 smem_u4[];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    uint4* stage = smem_u4 + wid * (V * 32);
    const int64_t nwarps = int64_t(gridDim.x) * (blockDim.x >> 5);

    for (int64_t chunk = int64_t(blockIdx.x) * (blockDim.x >> 5) + wid; chunk < p.total_units; chunk += nwarps) {
        const int j = find_job(jobs, p.njobs, chunk);
        const RowQuantArgs& J = jobs[j];
        const int64_t total_groups = J.rows * (J.cols / G);
        const int64_t g0 = (chunk - J.unit_begin) * 32;
        const int64_t total_elems = total_groups * G;
        const int64_t e0 = g0 * G;
        const uint4* src = reinterpret_cast<const uint4*>(static_cast<const InT*>(J.in) + e0);

#pragma unroll
        for (int v = 0; v < V; ++v) {
            const int64_t e = e0 + int64_t(v) * 256 + lane * 8;
            cp_async16(stage + v * 32 + lane, src + v * 32 + lane, e < total_elems);
        }
        cp_async_wait_all();  // each lane reads back only what it copied itself: no warp barrier needed

        // ---- statistics: lane g ends up with (min, -max) of group g0+g ---------------------------------
        uint32_t mine = 0;
#pragma unroll 4
        for (int v = 0; v < V; ++v) {
            uint32_t r = minnegmax8<InT>(stage[v * 32 + lane]);
#pragma unroll
            for (int o = LPG / 2; o > 0; o >>= 1) r = pmin<InT>(r, __shfl_xor_sync(0xffffffffu, r, o));
            const uint32_t t = __shfl_sync(0xffffffffu, r, ((lane - v * GPL) & (GPL - 1)) * LPG);
            if (lane / GPL == v) mine = t;
        }

        // ---- parameters of group g0+lane ----------------------------------------------------------------
        double scale;
        long long zp;
        UnitQ u;
        derive_unit(P2<InT>::lo(mine), -P2<InT>::hi(mine), p, scale, zp, u, flags);
        const int64_t g = g0 + lane;
        const bool g_ok = g < total_groups;
        if (g_ok) {
            if (J.scales) J.scales[g] = scale;
            if (J.zps) J.zps[g] = zp;
            if (J.scales_f16) J.scales_f16[g] = f32_to_f16_bits(__double2float_rn(scale));
        }
        if (J.zps_u4) {
            const int hi = __shfl_down_sync(0xffffffffu, int(zp), 1);
            if ((lane & 1) == 0 && g_ok) {
                const int hv = (g + 1 < total_groups) ? (hi & 0xF) : 0;
                J.zps_u4[g >> 1] = uint8_t((hv << 4) | (int(zp) & 0xF));
            }
        }

        // ---- quantize + store ----------------------------------------------------------------------------
        const int add = p.qmin;  // code = n + qmin
#pragma unroll 2
        for (int v = 0; v < V; ++v) {
            const int owner = v * GPL + lane / LPG;
            const float inv = __shfl_sync(0xffffffffu, u.inv, owner);
            const float c = __shfl_sync(0xffffffffu, u.c, owner);
            const uint4 d = stage[v * 32 + lane];
            float m[8];
            const bool bad = quant8<InT>(d, inv, c, m);
            if (__any_sync(0xffffffffu, bad)) {
                const float in_low = __shfl_sync(0xffffffffu, u.in_low, owner);
                const float range = __shfl_sync(0xffffffffu, u.range, owner);
                if (bad) VF_QUANT8_EXACT(InT, d, in_low, range, p.lm1, 0, m);
            }
            const int64_t e = e0 + int64_t(v) * 256 + lane * 8;
            const bool ok = e < total_elems;
            int code[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) code[i] = __float_as_int(m[i]);  // kMagicBits + n
            if (PACK4) {
                // sum of (kMagicBits + n_i) << 4i; the constant part is removed once
                uint32_t w = uint32_t(code[0]);
#pragma unroll
                for (int i = 1; i < 8; ++i) w += uint32_t(code[i]) << (4 * i);
                constexpr uint32_t kC = uint32_t(kMagicBits) * 0x11111111u;
                w -= kC;
                if (add != 0) {  // signed 4-bit ranges: add qmin to every nibble, modulo 16
                    const uint32_t q = uint32_t(add) & 0xFu;
                    w = ((w & 0x0F0F0F0Fu) + q * 0x01010101u) & 0x0F0F0F0Fu | ((((w >> 4) & 0x0F0F0F0Fu) + q * 0x01010101u) & 0x0F0F0F0Fu) << 4;
                }
                if (ok) reinterpret_cast<uint32_t*>(J.codes)[e >> 3] = w;
            } else {
                uint2 w;
                w.x = uint32_t((code[0] + add) & 0xFF) | (uint32_t((code[1] + add) & 0xFF) << 8) |
                      (uint32_t((code[2] + add) & 0xFF) << 16) | (uint32_t((code[3] + add) & 0xFF) << 24);
                w.y = uint32_t((code[4] + add) & 0xFF) | (uint32_t((code[5] + add) & 0xFF) << 8) |
                      (uint32_t((code[6] + add) & 0xFF) << 16) | (uint32_t((code[7] + add) & 0xFF) << 24);
                if (ok) reinterpret_cast<uint2*>(J.codes)[e >> 3] = w;
            }
            if (J.dequant) {  // optional Dequantize copy (not on the benchmarked path): exact FP64 formula
                const double sc = __shfl_sync(0xffffffffu, scale, owner);
                const int z = __shfl_sync(0xffffffffu, int(zp), owner);
                for (int i = 0; i < 8; ++i) {
                    const int q = ((code[i] - kMagicBits) + add);
                    if (!ok) continue;
                    if (p.dequant_dt == VF_DT_F32) static_cast<float*>(J.dequant)[e + i] = dequantize_exact(q, sc, z);
                    else static_cast<uint16_t*>(J.dequant)[e + i] = dequant16(q, z, sc, p.dequant_dt);
                }
            }
        }
    }
}

// ======================================================================================================
// K_row: one unit per row, 16-byte aligned rows of a [rows, cols] matrix (per-output-channel quantization of
// linear weights), 2-byte input. One CTA per row, looping over the rows of all jobs; the row is staged in
// shared memory. The optional Dequantize copy uses a per-row table of the L possible outputs (each entry
// computed with the exact FP64 formula), so the sweep costs one shared-memory lookup per element.
// ======================================================================================================
template <typename InT>
__global__ void __launch_bounds__(256) k_row(const RowQuantArgs* __restrict__ jobs, LaunchParams p, int* flags) {
    extern __shared__ uint4 smem_u4[];
    __shared__ uint32_t s_red[8];
    __shared__ UnitQ s_u;
    __shared__ double s_scale;
    __shared__ long long s_zp;
    __shared__ uint32_t s_lut[256];  // dequantized value of code index n (16-bit types in the low half)
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int bias = p.qmin;  // code = n + qmin

    for (int64_t row = blockIdx.x; row < p.total_units; row += gridDim.x) {
        const int j = find_job(jobs, p.njobs, row);
        const RowQuantArgs& J = jobs[j];
        const int64_t r = row - J.unit_begin;
        const int64_t cols = J.cols;
        const int nvec = int(cols >> 3);
        const uint4* src = reinterpret_cast<const uint4*>(static_cast<const InT*>(J.in) + r * cols);
        for (int i = tid; i < nvec; i += 256) cp_async16(smem_u4 + i, src + i, true);
        cp_async_wait_all();

        uint32_t acc = 0;
        for (int i = tid; i < nvec; i += 256) acc = pmin<InT>(acc, minnegmax8<InT>(smem_u4[i]));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc = pmin<InT>(acc, __shfl_xor_sync(0xffffffffu, acc, o));
        if (lane == 0) s_red[wid] = acc;
        __syncthreads();
        if (wid == 0) {
            acc = lane < 8 ? s_red[lane] : 0u;
#pragma unroll
            for (int o = 4; o > 0; o >>= 1) acc = pmin<InT>(acc, __shfl_xor_sync(0xffffffffu, acc, o));
            if (lane == 0) {
                double scale;
                long long zp;
                UnitQ u;
                derive_unit(P2<InT>::lo(acc), -P2<InT>::hi(acc), p, scale, zp, u, flags);
                // shift the rounding target by qmin so that the low byte of (t + magic) is the signed code.
                // The shift is exact only for the constant, so it is applied to c before the fma; the guard
                // band covers the additional rounding error (|c + qmin| <= 255).
                u.c = __fadd_rn(u.c, float(bias));
                s_u = u;
                s_scale = scale;
                s_zp = zp;
                if (J.scales) J.scales[r] = scale;
                if (J.zps) J.zps[r] = zp;
                if (J.scales_f16) J.scales_f16[r] = f32_to_f16_bits(__double2float_rn(scale));
            }
        }
        __syncthreads();
        const UnitQ u = s_u;
        if (J.dequant) {
            if (tid <= p.lm1) {
                const float f = dequantize_exact(tid + bias, s_scale, s_zp);
                s_lut[tid] = p.dequant_dt == VF_DT_F32 ? __float_as_uint(f)
                             : (p.dequant_dt == VF_DT_F16 ? f32_to_f16_clamped_bits(f) : f32_to_bf16_bits(f));
            }
            __syncthreads();
        }
        uint2* codes = reinterpret_cast<uint2*>(static_cast<uint8_t*>(J.codes) + r * cols);
        for (int i = tid; i < nvec; i += 256) {
            const uint4 d = smem_u4[i];
            float m[8];
            const bool bad = quant8<InT>(d, u.inv, u.c, m);
            if (bad) VF_QUANT8_EXACT(InT, d, u.in_low, u.range, p.lm1, bias, m);
            uint32_t b[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) b[k] = __float_as_uint(m[k]);  // low byte = code (two's complement)
            uint2 w;
            w.x = __byte_perm(__byte_perm(b[0], b[1], 0x0040), __byte_perm(b[2], b[3], 0x0040), 0x5410);
            w.y = __byte_perm(__byte_perm(b[4], b[5], 0x0040), __byte_perm(b[6], b[7], 0x0040), 0x5410);
            codes[i] = w;
            if (J.dequant) {
                uint32_t q[8];
#pragma unroll
                for (int k = 0; k < 8; ++k) q[k] = s_lut[(b[k] - uint32_t(bias)) & 0xFFu];
                if (p.dequant_dt == VF_DT_F32) {
                    float4* dst = reinterpret_cast<float4*>(static_cast<float*>(J.dequant) + r * cols);
                    dst[2 * i] = make_float4(__uint_as_float(q[0]), __uint_as_float(q[1]), __uint_as_float(q[2]), __uint_as_float(q[3]));
                    dst[2 * i + 1] = make_float4(__uint_as_float(q[4]), __uint_as_float(q[5]), __uint_as_float(q[6]), __uint_as_float(q[7]));
                } else {
                    uint4 o;
                    o.x = __byte_perm(q[0], q[1], 0x5410);
                    o.y = __byte_perm(q[2], q[3], 0x5410);
                    o.z = __byte_perm(q[4], q[5], 0x5410);
                    o.w = __byte_perm(q[6], q[7], 0x5410);
                    reinterpret_cast<uint4*>(static_cast<uint16_t*>(J.dequant) + r * cols)[i] = o;
                }
            }
        }
        __syncthreads();  // stage, s_u and s_lut are rewritten by the next row
    }
}

// ======================================================================================================
// K_conv: one unit per output channel of a convolution weight, any row length / alignment, any of
// f32 / f16 / bf16. One warp per row, looping over the rows of all jobs. The quantized row is staged in
// shared memory at its OYXI position (ic padded to ic_pad) and written out with coalesced 32-bit stores; rows
// beyond `rows` (channel padding) are zero. Two sweeps over the row: the second one hits L1/L2.
// ======================================================================================================
__global__ void __launch_bounds__(256) k_conv(const RowQuantArgs* __restrict__ jobs, LaunchParams p, int in_dt,
                                              int stage_bytes, int* flags) {
    extern __shared__ uint4 smem_u4[];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    uint8_t* stage = reinterpret_cast<uint8_t*>(smem_u4) + size_t(wid) * size_t(stage_bytes);
    const int64_t nwarps = int64_t(gridDim.x) * (blockDim.x >> 5);

    for (int64_t row = int64_t(blockIdx.x) * (blockDim.x >> 5) + wid; row < p.total_units; row += nwarps) {
        const int j = find_job(jobs, p.njobs, row);
        const RowQuantArgs& J = jobs[j];
        const int64_t r = row - J.unit_begin;
        const int64_t khw = J.khw > 0 ? J.khw : 1;
        const int64_t ic = J.khw > 0 ? J.ic : J.cols;
        const int64_t ic_pad = J.khw > 0 ? J.ic_pad : J.cols;
        const int64_t out_row_bytes = khw * ic_pad;
        uint8_t* out = static_cast<uint8_t*>(J.codes) + r * out_row_bytes;
        if (r >= J.rows) {  // padded output channel: PadWithZero fills plain integer types with zero bytes
            for (int64_t b = lane; b < out_row_bytes; b += 32) out[b] = 0;
            continue;
        }
        const int64_t base = r * J.cols;
        float mn = 0.f, mx = 0.f;
        for (int64_t i = lane; i < J.cols; i += 32) {
            const float x = load_as_f32(J.in, in_dt, base + i, nullptr);
            mn = fminf(mn, x);
            mx = fmaxf(mx, x);
        }
        mn = warp_min(mn);
        mx = warp_max(mx);
        double scale = 0.0;
        long long zp = 0;
        UnitQ u;
        if (lane == 0) {
            derive_unit(mn, mx, p, scale, zp, u, flags);
            if (J.scales) J.scales[r] = scale;
            if (J.zps) J.zps[r] = zp;
            if (J.scales_f16) J.scales_f16[r] = f32_to_f16_bits(__double2float_rn(scale));
        }
        u.inv = __shfl_sync(0xffffffffu, u.inv, 0);
        u.c = __shfl_sync(0xffffffffu, u.c, 0);
        u.in_low = __shfl_sync(0xffffffffu, u.in_low, 0);
        u.range = __shfl_sync(0xffffffffu, u.range, 0);
        if (ic_pad != ic) {
            for (int64_t b = lane; b < out_row_bytes; b += 32) stage[b] = 0;
            __syncwarp();
        }
        for (int64_t i = lane; i < J.cols; i += 32) {
            const float x = load_as_f32(J.in, in_dt, base + i, nullptr);
            const float t = __fmaf_rn(x, u.inv, u.c);
            const float m = __fadd_rn(t, kMagic);
            int n = __float_as_int(m) - kMagicBits;
            const float resid = __fsub_rn(t, __fsub_rn(m, kMagic));
            if (fabsf(resid) > 0.5f - kGuard) n = quant_index_exact(x, u.in_low, u.range, p.lm1);
            n = min(max(n, 0), p.lm1);
            // input index i = icIdx * khw + s  ->  output index s * ic_pad + icIdx
            const int64_t ici = i / khw, s = i - ici * khw;
            stage[s * ic_pad + ici] = uint8_t(n + p.qmin);
        }
        __syncwarp();
        if (((reinterpret_cast<uintptr_t>(out) | uintptr_t(out_row_bytes)) & 3) == 0) {
            const uint32_t* s32 = reinterpret_cast<const uint32_t*>(stage);
            uint32_t* o32 = reinterpret_cast<uint32_t*>(out);
            for (int64_t w = lane; w < (out_row_bytes >> 2); w += 32) o32[w] = s32[w];
        } else {
            for (int64_t b = lane; b < out_row_bytes; b += 32) out[b] = stage[b];
        }
        __syncwarp();
    }
}

void post_launch(vf_ctx* ctx) {
    VF_CUDA(cudaGetLastError());
    ctx->launches += 1;
}

template <typename K>
void set_smem(K kernel, size_t bytes) {
    VF_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(bytes)));
}

template <typename InT, int G>
void launch_group_g(vf_ctx* ctx, const RowQuantArgs* d_jobs, const LaunchParams& p, bool pack4) {
    const size_t smem = size_t(8) * (G / 8) * 32 * 16;  // 8 warps x (G/8 * 32) vectors
    // persistent grid: three CTAs per SM (launch bounds), every warp strides over the chunk list
    const int64_t want = (p.total_units + 7) / 8;
    const int grid = int(std::min<int64_t>(want, 148 * 3));
    if (pack4) {
        set_smem(k_group<InT, G, true>, smem);
        k_group<InT, G, true><<<grid, 256, smem, ctx->stream>>>(d_jobs, p, ctx->d_flags);
    } else {
        set_smem(k_group<InT, G, false>, smem);
        k_group<InT, G, false><<<grid, 256, smem, ctx->stream>>>(d_jobs, p, ctx->d_flags);
    }
    post_launch(ctx);
}

template <typename InT>
void launch_group_t(vf_ctx* ctx, const RowQuantArgs* d_jobs, const LaunchParams& p, int64_t group, bool pack4) {
    switch (group) {
    case 32: launch_group_g<InT, 32>(ctx, d_jobs, p, pack4); break;
    case 64: launch_group_g<InT, 64>(ctx, d_jobs, p, pack4); break;
    case 128: launch_group_g<InT, 128>(ctx, d_jobs, p, pack4); break;
    default: raise(VF_ERR_UNSUPPORTED, "fused group kernel handles groups of 32, 64 or 128");
    }
}

}  // namespace

// Which fused kernel covers `a`? 0 = none, 1 = group, 2 = row, 3 = conv
int rowquant_kind(const RowQuantArgs& a) {
    const bool two_byte = a.in_dt == VF_DT_F16 || a.in_dt == VF_DT_BF16;
    const bool aligned16 = reinterpret_cast<uintptr_t>(a.in) % 16 == 0;
    if (a.group > 0) {
        if (two_byte && aligned16 && a.khw == 0 && a.rows_pad == a.rows && (a.group == 32 || a.group == 64 || a.group == 128) &&
            reinterpret_cast<uintptr_t>(a.codes) % 8 == 0 && (!a.dequant || reinterpret_cast<uintptr_t>(a.dequant) % 16 == 0))
            return 1;
        return 0;
    }
    if (two_byte && aligned16 && a.khw == 0 && a.rows_pad == a.rows && !a.pack4 && !a.zps_u4 && a.cols % 8 == 0 &&
        a.cols >= 1024 && a.cols <= 96 * 1024 && reinterpret_cast<uintptr_t>(a.codes) % 8 == 0 &&
        (!a.dequant || reinterpret_cast<uintptr_t>(a.dequant) % 16 == 0))
        return 2;
    if (!a.pack4 && !a.dequant && !a.zps_u4) {
        const int64_t out_row = a.khw > 0 ? a.khw * a.ic_pad : a.cols;
        if (out_row <= 24 * 1024) return 3;
    }
    return 0;
}

// Launches every job of `jobs` (all of kind `kind` and sharing the uniform parameters of jobs[0]) with one
// kernel. The job table is copied to device memory first.
void launch_rowquant_batch(vf_ctx* ctx, int kind, std::vector<RowQuantArgs>& jobs) {
    if (jobs.empty()) return;
    const RowQuantArgs& a0 = jobs[0];
    LaunchParams p{};
    p.range_mode = a0.range_mode;
    p.qmin = int(a0.qmin);
    p.qmax = int(a0.qmax);
    p.lm1 = int(a0.qmax - a0.qmin);
    p.dequant_dt = a0.dequant_dt;
    p.njobs = int(jobs.size());
    int64_t units = 0, max_cols = 0, max_out_row = 0;
    for (auto& a : jobs) {
        a.unit_begin = units;
        if (kind == 1) units += (a.rows * (a.cols / a.group) + 31) / 32;
        else if (kind == 2) units += a.rows;
        else units += a.rows_pad;
        max_cols = std::max(max_cols, a.cols);
        max_out_row = std::max(max_out_row, a.khw > 0 ? a.khw * a.ic_pad : a.cols);
    }
    p.total_units = units;
    DBuf table(ctx, jobs.size() * sizeof(RowQuantArgs));
    copy_in(ctx, table.p, jobs.data(), jobs.size() * sizeof(RowQuantArgs), VF_MEM_HOST);
    const RowQuantArgs* d_jobs = table.as<RowQuantArgs>();

    if (kind == 1) {
        if (a0.in_dt == VF_DT_F16) launch_group_t<__half>(ctx, d_jobs, p, a0.group, a0.pack4 != 0);
        else launch_group_t<__nv_bfloat16>(ctx, d_jobs, p, a0.group, a0.pack4 != 0);
    } else if (kind == 2) {
        const size_t smem = size_t(max_cols) * 2;
        const int per_sm = int(std::max<size_t>(1, std::min<size_t>(8, (200 * 1024) / (smem + 2048))));
        const int grid = int(std::min<int64_t>(units, int64_t(148) * per_sm));
        if (a0.in_dt == VF_DT_F16) {
            set_smem(k_row<__half>, smem);
            k_row<__half><<<grid, 256, smem, ctx->stream>>>(d_jobs, p, ctx->d_flags);
        } else {
            set_smem(k_row<__nv_bfloat16>, smem);
            k_row<__nv_bfloat16><<<grid, 256, smem, ctx->stream>>>(d_jobs, p, ctx->d_flags);
        }
        post_launch(ctx);
    } else if (kind == 3) {
        const int stage_bytes = int((max_out_row + 15) & ~int64_t(15));
        const size_t smem = size_t(stage_bytes) * 8;
        set_smem(k_conv, std::max<size_t>(smem, 16));
        const int64_t blocks = (units + 7) / 8;
        k_conv<<<int(std::min<int64_t>(blocks, 148 * 8)), 256, smem, ctx->stream>>>(d_jobs, p, a0.in_dt, stage_bytes, ctx->d_flags);
        post_launch(ctx);
    } else {
        raise(VF_ERR_UNSUPPORTED, "no fused kernel for this weight quantization pattern");
    }
}

// Jobs may share a launch when the launch-uniform parameters agree.
bool rowquant_compatible(const RowQuantArgs& a, const RowQuantArgs& b) {
    return a.in_dt == b.in_dt && a.group == b.group && a.range_mode == b.range_mode && a.qmin == b.qmin && a.qmax == b.qmax &&
           a.pack4 == b.pack4 && a.dequant_dt == b.dequant_dt && a.out_signed == b.out_signed;
}

}  // namespace vf
