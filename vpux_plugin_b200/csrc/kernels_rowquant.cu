// Fused weight-quantization kernels (the hot path): range statistics, calcScaleAndZeroPoint, Quantize and
// the store stage (BitPack / OIYX->OYXI reorder / zero padding / Dequantize copy) in ONE pass over the
// input. All of them are bandwidth-bound: 128-bit coalesced loads, the unit kept in registers between the
// statistics and the quantization sweep, shuffles for the reductions, no tensor cores.
//
// Arithmetic contract: codes equal the reference's fakeQuantize chain bit for bit. The per-element fast path
// evaluates  t = (x - inLow) * fl((L-1)/(inHigh-inLow))  (two roundings) instead of the reference's
// fl(fl((x-inLow)/(inHigh-inLow)) * (L-1)) (three roundings, one IEEE division); the two differ by at most
// (L-1)*2^-22 < 6.1e-5 for 8-bit ranges, so whenever t lies further than kGuard from a rounding boundary
// (x.5) both round to the same integer. Elements inside the guard band (about 0.04 %) are recomputed with
// the exact operation sequence.
#include <algorithm>

#include "device_utils.cuh"
#include "kernels.h"

namespace vf {

namespace {

constexpr float kMagic = 12582912.0f;  // 1.5 * 2^23: adding it rounds to the nearest integer
constexpr int kMagicBits = 0x4B400000;
constexpr float kGuard = 2.0e-4f;

struct UnitQ {  // per-unit constants of the fast path + what the exact path needs
    float in_low;
    float inv;    // fl((L-1) / range)
    float range;  // fl(inHigh - inLow)
};

// Per-unit parameters from the unit's range; executed by one lane per unit.
__device__ __forceinline__ void derive_unit(float mn, float mx, int range_mode, long long qmin, long long qmax,
                                            double& scale, long long& zp, UnitQ& u, int* flags) {
    if (range_mode == VF_RANGE_ABSMAX) {
        const float a = fmaxf(-mn, mx);
        mn = -a;
        mx = a;
    }
    if (!calc_scale_zp(double(qmin), double(qmax), double(mn), double(mx), scale, zp)) {
        set_flag(flags, VF_FLAG_QUANT_RANGE);
        scale = 1.0;
        zp = 0;
    }
    zp = zp < qmin ? qmin : (zp > qmax ? qmax : zp);
    u.in_low = dequantize_exact(qmin, scale, zp);
    const float in_high = dequantize_exact(qmax, scale, zp);
    u.range = __fsub_rn(in_high, u.in_low);
    u.inv = __fdiv_rn(float(qmax - qmin), u.range);
}

// Returns the code index n in [0, L-1] (code = n + qmin; the caller has verified on the host that the tail of
// fakeQuantize, trunc(fl(fl(n/(L-1))*(qHigh-qLow))+qLow), is the identity for this range).
__device__ __forceinline__ int quant_index(float x, const UnitQ& u, float lm1f, int lm1) {
    const float a = __fsub_rn(x, u.in_low);
    const float t = __fmul_rn(a, u.inv);
    const float m = __fadd_rn(t, kMagic);
    int n = __float_as_int(m) - kMagicBits;
    const float resid = __fsub_rn(t, __fsub_rn(m, kMagic));
    if (fabsf(resid) > 0.5f - kGuard) {
        // exact sequence: fl(fl(a / range) * (L-1)), rounded half away from zero
        float e = __fdiv_rn(a, u.range);
        e = __fmul_rn(e, lm1f);
        n = int(round_half_away(e));
    }
    return min(max(n, 0), lm1);
}

template <typename InT>
struct Vec8;  // eight 2-byte elements in one 16-byte load
template <>
struct Vec8<__half> {
    static __device__ __forceinline__ void unpack(const uint4& v, float* f) {
        const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 p = __half22float2(h[i]);
            f[2 * i] = p.x;
            f[2 * i + 1] = p.y;
        }
    }
};
template <>
struct Vec8<__nv_bfloat16> {
    static __device__ __forceinline__ void unpack(const uint4& v, float* f) {
        const uint32_t* w = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            f[2 * i] = __uint_as_float(w[i] << 16);
            f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
        }
    }
};

__device__ __forceinline__ void minmax8(const float* f, float& mn, float& mx) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        mn = fminf(mn, f[i]);
        mx = fmaxf(mx, f[i]);
    }
}

__device__ __forceinline__ uint4 ld_stream(const uint4* p) {  // read-once data: do not keep it in L1
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// Dequantize + copyTo for one code: float((q - zp) * scale) then the element conversion of `dt`
__device__ __forceinline__ uint16_t dequant16(int code, long long zp, double scale, int dt) {
    const float f = dequantize_exact(code, scale, zp);
    return dt == VF_DT_F16 ? f32_to_f16_clamped_bits(f) : f32_to_bf16_bits(f);
}

// ======================================================================================================
// K_group: units of G consecutive elements (per-group quantization), 2-byte input.
// A warp owns 32 consecutive groups: V = G/8 coalesced 16-byte loads per lane stay in registers; each group
// is reduced by the G/8 lanes that loaded it; lane g then derives the parameters of group g (all 32 lanes
// busy in the FP64 section); parameters travel back by shuffle for the quantization sweep.
// ======================================================================================================
template <typename InT, int G>
__global__ void __launch_bounds__(256) k_group(RowQuantArgs a, int64_t total_groups, int lm1, int* flags) {
    constexpr int V = G / 8;     // loads per lane
    constexpr int LPG = G / 8;   // lanes per group within one load
    constexpr int GPL = 32 / LPG;  // groups finished per load
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int64_t g0 = warp * 32;
    if (g0 >= total_groups) return;
    const int64_t total_elems = total_groups * G;
    const int64_t e0 = g0 * G;  // first element of this warp's chunk
    const uint4* src = reinterpret_cast<const uint4*>(static_cast<const InT*>(a.in) + e0);

    uint4 data[V];
#pragma unroll
    for (int v = 0; v < V; ++v) {
        const int64_t e = e0 + int64_t(v) * 256 + lane * 8;
        data[v] = e < total_elems ? ld_stream(src + v * 32 + lane) : make_uint4(0, 0, 0, 0);
    }

    // ---- statistics: lane g ends up with min/max of group g0+g ----------------------------------------
    float my_mn = 0.f, my_mx = 0.f;
#pragma unroll
    for (int v = 0; v < V; ++v) {
        float f[8];
        Vec8<InT>::unpack(data[v], f);
        float mn = 0.f, mx = 0.f;  // the range always contains zero
        minmax8(f, mn, mx);
#pragma unroll
        for (int o = LPG / 2; o > 0; o >>= 1) {
            mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        }
        const int srcl = ((lane - v * GPL) & (GPL - 1)) * LPG;
        const float tmn = __shfl_sync(0xffffffffu, mn, srcl);
        const float tmx = __shfl_sync(0xffffffffu, mx, srcl);
        if (lane / GPL == v) {
            my_mn = tmn;
            my_mx = tmx;
        }
    }

    // ---- parameters of group g0+lane -------------------------------------------------------------------
    double scale;
    long long zp;
    UnitQ u;
    derive_unit(my_mn, my_mx, a.range_mode, a.qmin, a.qmax, scale, zp, u, flags);
    const int64_t g = g0 + lane;
    const bool g_ok = g < total_groups;
    if (g_ok) {
        if (a.scales) a.scales[g] = scale;
        if (a.zps) a.zps[g] = zp;
        if (a.scales_f16) a.scales_f16[g] = f32_to_f16_bits(__double2float_rn(scale));
    }
    if (a.zps_u4) {
        const int hi = __shfl_down_sync(0xffffffffu, int(zp), 1);
        if ((lane & 1) == 0 && g_ok) {
            const int hv = (g + 1 < total_groups) ? (hi & 0xF) : 0;
            a.zps_u4[g >> 1] = uint8_t((hv << 4) | (int(zp) & 0xF));
        }
    }

    // ---- quantize + store ------------------------------------------------------------------------------
    const float lm1f = float(lm1);
    const int qmin = int(a.qmin);
    const int zpi = int(zp);
#pragma unroll
    for (int v = 0; v < V; ++v) {
        const int owner = v * GPL + lane / LPG;
        UnitQ q;
        q.in_low = __shfl_sync(0xffffffffu, u.in_low, owner);
        q.inv = __shfl_sync(0xffffffffu, u.inv, owner);
        q.range = __shfl_sync(0xffffffffu, u.range, owner);
        float f[8];
        Vec8<InT>::unpack(data[v], f);
        int c[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) c[i] = quant_index(f[i], q, lm1f, lm1) + qmin;
        const int64_t e = e0 + int64_t(v) * 256 + lane * 8;
        const bool ok = e < total_elems;
        if (a.pack4) {
            uint32_t w = 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) w |= uint32_t(c[i] & 0xF) << (4 * i);
            if (ok) reinterpret_cast<uint32_t*>(a.codes)[e >> 3] = w;
        } else {
            uint2 w;
            w.x = uint32_t(c[0] & 0xFF) | (uint32_t(c[1] & 0xFF) << 8) | (uint32_t(c[2] & 0xFF) << 16) | (uint32_t(c[3] & 0xFF) << 24);
            w.y = uint32_t(c[4] & 0xFF) | (uint32_t(c[5] & 0xFF) << 8) | (uint32_t(c[6] & 0xFF) << 16) | (uint32_t(c[7] & 0xFF) << 24);
            if (ok) reinterpret_cast<uint2*>(a.codes)[e >> 3] = w;
        }
        if (a.dequant) {
            const double sc = __shfl_sync(0xffffffffu, scale, owner);
            const int z = __shfl_sync(0xffffffffu, zpi, owner);
            if (a.dequant_dt == VF_DT_F32) {
                float4 o0, o1;
                o0.x = dequantize_exact(c[0], sc, z); o0.y = dequantize_exact(c[1], sc, z);
                o0.z = dequantize_exact(c[2], sc, z); o0.w = dequantize_exact(c[3], sc, z);
                o1.x = dequantize_exact(c[4], sc, z); o1.y = dequantize_exact(c[5], sc, z);
                o1.z = dequantize_exact(c[6], sc, z); o1.w = dequantize_exact(c[7], sc, z);
                if (ok) {
                    reinterpret_cast<float4*>(a.dequant)[(e >> 2)] = o0;
                    reinterpret_cast<float4*>(a.dequant)[(e >> 2) + 1] = o1;
                }
            } else {
                uint4 o;
                o.x = dequant16(c[0], z, sc, a.dequant_dt) | (uint32_t(dequant16(c[1], z, sc, a.dequant_dt)) << 16);
                o.y = dequant16(c[2], z, sc, a.dequant_dt) | (uint32_t(dequant16(c[3], z, sc, a.dequant_dt)) << 16);
                o.z = dequant16(c[4], z, sc, a.dequant_dt) | (uint32_t(dequant16(c[5], z, sc, a.dequant_dt)) << 16);
                o.w = dequant16(c[6], z, sc, a.dequant_dt) | (uint32_t(dequant16(c[7], z, sc, a.dequant_dt)) << 16);
                if (ok) reinterpret_cast<uint4*>(a.dequant)[e >> 3] = o;
            }
        }
    }
}

// ======================================================================================================
// K_row: one unit per row, long 16-byte aligned rows (per-output-channel quantization of linear weights),
// 2-byte input. One CTA per row; the row stays in registers (V 16-byte loads per thread).
// ======================================================================================================
template <typename InT, int V, int THREADS>
__global__ void __launch_bounds__(THREADS) k_row(RowQuantArgs a, int lm1, int* flags) {
    __shared__ float s_mn[32], s_mx[32];
    __shared__ double s_scale;
    __shared__ long long s_zp;
    __shared__ UnitQ s_u;
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int64_t nvec = a.cols >> 3;
    const float lm1f = float(lm1);
    const int qmin = int(a.qmin);

    for (int64_t row = blockIdx.x; row < a.rows; row += gridDim.x) {
        const uint4* src = reinterpret_cast<const uint4*>(static_cast<const InT*>(a.in) + row * a.cols);
        uint4 data[V];
#pragma unroll
        for (int v = 0; v < V; ++v) {
            const int64_t i = int64_t(v) * THREADS + tid;
            data[v] = i < nvec ? ld_stream(src + i) : make_uint4(0, 0, 0, 0);
        }
        float mn = 0.f, mx = 0.f;
#pragma unroll
        for (int v = 0; v < V; ++v) {
            float f[8];
            Vec8<InT>::unpack(data[v], f);
            minmax8(f, mn, mx);
        }
        mn = warp_min(mn);
        mx = warp_max(mx);
        if (lane == 0) {
            s_mn[wid] = mn;
            s_mx[wid] = mx;
        }
        __syncthreads();
        if (wid == 0) {
            mn = lane < THREADS / 32 ? s_mn[lane] : 0.f;
            mx = lane < THREADS / 32 ? s_mx[lane] : 0.f;
            mn = warp_min(mn);
            mx = warp_max(mx);
            if (lane == 0) {
                double scale;
                long long zp;
                UnitQ u;
                derive_unit(mn, mx, a.range_mode, a.qmin, a.qmax, scale, zp, u, flags);
                s_scale = scale;
                s_zp = zp;
                s_u = u;
                if (a.scales) a.scales[row] = scale;
                if (a.zps) a.zps[row] = zp;
                if (a.scales_f16) a.scales_f16[row] = f32_to_f16_bits(__double2float_rn(scale));
            }
        }
        __syncthreads();
        const UnitQ q = s_u;
        const double sc = s_scale;
        const int z = int(s_zp);
        uint2* codes = reinterpret_cast<uint2*>(static_cast<uint8_t*>(a.codes) + row * a.cols);
#pragma unroll
        for (int v = 0; v < V; ++v) {
            const int64_t i = int64_t(v) * THREADS + tid;
            if (i >= nvec) continue;
            float f[8];
            Vec8<InT>::unpack(data[v], f);
            int c[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) c[k] = quant_index(f[k], q, lm1f, lm1) + qmin;
            uint2 w;
            w.x = uint32_t(c[0] & 0xFF) | (uint32_t(c[1] & 0xFF) << 8) | (uint32_t(c[2] & 0xFF) << 16) | (uint32_t(c[3] & 0xFF) << 24);
            w.y = uint32_t(c[4] & 0xFF) | (uint32_t(c[5] & 0xFF) << 8) | (uint32_t(c[6] & 0xFF) << 16) | (uint32_t(c[7] & 0xFF) << 24);
            codes[i] = w;
            if (a.dequant) {
                if (a.dequant_dt == VF_DT_F32) {
                    float4 o0, o1;
                    o0.x = dequantize_exact(c[0], sc, z); o0.y = dequantize_exact(c[1], sc, z);
                    o0.z = dequantize_exact(c[2], sc, z); o0.w = dequantize_exact(c[3], sc, z);
                    o1.x = dequantize_exact(c[4], sc, z); o1.y = dequantize_exact(c[5], sc, z);
                    o1.z = dequantize_exact(c[6], sc, z); o1.w = dequantize_exact(c[7], sc, z);
                    float4* d = reinterpret_cast<float4*>(static_cast<float*>(a.dequant) + row * a.cols);
                    d[2 * i] = o0;
                    d[2 * i + 1] = o1;
                } else {
                    uint4 o;
                    o.x = dequant16(c[0], z, sc, a.dequant_dt) | (uint32_t(dequant16(c[1], z, sc, a.dequant_dt)) << 16);
                    o.y = dequant16(c[2], z, sc, a.dequant_dt) | (uint32_t(dequant16(c[3], z, sc, a.dequant_dt)) << 16);
                    o.z = dequant16(c[4], z, sc, a.dequant_dt) | (uint32_t(dequant16(c[5], z, sc, a.dequant_dt)) << 16);
                    o.w = dequant16(c[6], z, sc, a.dequant_dt) | (uint32_t(dequant16(c[7], z, sc, a.dequant_dt)) << 16);
                    reinterpret_cast<uint4*>(static_cast<uint16_t*>(a.dequant) + row * a.cols)[i] = o;
                }
            }
        }
        __syncthreads();  // s_* are rewritten by the next row
    }
}

// ======================================================================================================
// K_conv: one unit per output channel of a convolution weight, any row length / alignment, any of
// f32 / f16 / bf16. One warp per row. The quantized row is staged in shared memory at its OYXI position
// (ic padded to ic_pad) and written out with coalesced 32-bit stores; rows >= `rows` (channel padding)
// are zero. Two sweeps over the row: the second one hits L1/L2.
// ======================================================================================================
__global__ void __launch_bounds__(256) k_conv(RowQuantArgs a, int lm1, int64_t out_row_bytes, int* flags) {
    extern __shared__ uint8_t smem[];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    uint8_t* stage = smem + size_t(wid) * size_t((out_row_bytes + 15) & ~int64_t(15));
    const int64_t warp = int64_t(blockIdx.x) * (blockDim.x >> 5) + wid;
    const int64_t nwarps = int64_t(gridDim.x) * (blockDim.x >> 5);
    const float lm1f = float(lm1);
    const int qmin = int(a.qmin);
    const int64_t khw = a.khw > 0 ? a.khw : 1;
    const int64_t ic = a.khw > 0 ? a.ic : a.cols;
    const int64_t ic_pad = a.khw > 0 ? a.ic_pad : a.cols;

    for (int64_t row = warp; row < a.rows_pad; row += nwarps) {
        uint8_t* out = static_cast<uint8_t*>(a.codes) + row * out_row_bytes;
        if (row >= a.rows) {  // padded output channel: PadWithZero fills plain integer types with zero bytes
            for (int64_t b = lane; b < out_row_bytes; b += 32) out[b] = 0;
            continue;
        }
        const int64_t base = row * a.cols;
        float mn = 0.f, mx = 0.f;
        for (int64_t i = lane; i < a.cols; i += 32) {
            const float x = load_as_f32(a.in, a.in_dt, base + i, nullptr);
            mn = fminf(mn, x);
            mx = fmaxf(mx, x);
        }
        mn = warp_min(mn);
        mx = warp_max(mx);
        double scale;
        long long zp;
        UnitQ u;
        derive_unit(mn, mx, a.range_mode, a.qmin, a.qmax, scale, zp, u, flags);  // redundantly on every lane
        if (lane == 0) {
            if (a.scales) a.scales[row] = scale;
            if (a.zps) a.zps[row] = zp;
            if (a.scales_f16) a.scales_f16[row] = f32_to_f16_bits(__double2float_rn(scale));
        }
        if (ic_pad != ic) {
            for (int64_t b = lane; b < out_row_bytes; b += 32) stage[b] = 0;
            __syncwarp();
        }
        for (int64_t i = lane; i < a.cols; i += 32) {
            const float x = load_as_f32(a.in, a.in_dt, base + i, nullptr);
            const int c = quant_index(x, u, lm1f, lm1) + qmin;
            // input index i = icIdx * khw + s  ->  output index s * ic_pad + icIdx
            const int64_t ici = i / khw, s = i - ici * khw;
            stage[s * ic_pad + ici] = uint8_t(c);
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

template <typename InT>
void launch_group_t(vf_ctx* ctx, const RowQuantArgs& a, int64_t total_groups, int lm1) {
    const int64_t warps = (total_groups + 31) / 32;
    const int grid = int((warps + 7) / 8);
    switch (a.group) {
    case 32: k_group<InT, 32><<<grid, 256, 0, ctx->stream>>>(a, total_groups, lm1, ctx->d_flags); break;
    case 64: k_group<InT, 64><<<grid, 256, 0, ctx->stream>>>(a, total_groups, lm1, ctx->d_flags); break;
    case 128: k_group<InT, 128><<<grid, 256, 0, ctx->stream>>>(a, total_groups, lm1, ctx->d_flags); break;
    default: raise(VF_ERR_UNSUPPORTED, "fused group kernel handles groups of 32, 64 or 128");
    }
    post_launch(ctx);
}

template <typename InT>
void launch_row_t(vf_ctx* ctx, const RowQuantArgs& a, int lm1) {
    const int64_t nvec = a.cols / 8;
    const int grid = int(std::min<int64_t>(a.rows, 148 * 32));
    if (nvec <= 256) k_row<InT, 1, 256><<<grid, 256, 0, ctx->stream>>>(a, lm1, ctx->d_flags);
    else if (nvec <= 512) k_row<InT, 2, 256><<<grid, 256, 0, ctx->stream>>>(a, lm1, ctx->d_flags);
    else if (nvec <= 1024) k_row<InT, 4, 256><<<grid, 256, 0, ctx->stream>>>(a, lm1, ctx->d_flags);
    else if (nvec <= 2048) k_row<InT, 4, 512><<<grid, 512, 0, ctx->stream>>>(a, lm1, ctx->d_flags);
    else if (nvec <= 4096) k_row<InT, 8, 512><<<grid, 512, 0, ctx->stream>>>(a, lm1, ctx->d_flags);
    else k_row<InT, 8, 1024><<<grid, 1024, 0, ctx->stream>>>(a, lm1, ctx->d_flags);
    post_launch(ctx);
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
    if (two_byte && aligned16 && a.khw == 0 && a.rows_pad == a.rows && !a.pack4 && a.cols % 8 == 0 && a.cols >= 1024 &&
        a.cols <= 8 * 8192 && reinterpret_cast<uintptr_t>(a.codes) % 8 == 0 &&
        (!a.dequant || reinterpret_cast<uintptr_t>(a.dequant) % 16 == 0))
        return 2;
    if (!a.pack4 && !a.dequant && !a.zps_u4) {
        const int64_t out_row = a.khw > 0 ? a.khw * a.ic_pad : a.cols;
        if (out_row <= 24 * 1024) return 3;
    }
    return 0;
}

void launch_rowquant(vf_ctx* ctx, const RowQuantArgs& a) {
    const int lm1 = int(a.qmax - a.qmin);
    const int kind = rowquant_kind(a);
    if (kind == 1) {
        const int64_t total_groups = a.rows * a.cols / a.group;
        if (a.in_dt == VF_DT_F16) launch_group_t<__half>(ctx, a, total_groups, lm1);
        else launch_group_t<__nv_bfloat16>(ctx, a, total_groups, lm1);
    } else if (kind == 2) {
        if (a.in_dt == VF_DT_F16) launch_row_t<__half>(ctx, a, lm1);
        else launch_row_t<__nv_bfloat16>(ctx, a, lm1);
    } else if (kind == 3) {
        const int64_t out_row = a.khw > 0 ? a.khw * a.ic_pad : a.cols;
        const size_t per_warp = size_t((out_row + 15) & ~int64_t(15));
        const size_t smem = per_warp * 8;
        if (!ctx->conv_smem_set) {
            VF_CUDA(cudaFuncSetAttribute(k_conv, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
            ctx->conv_smem_set = true;
        }
        const int64_t blocks = (a.rows_pad + 7) / 8;
        k_conv<<<int(std::min<int64_t>(blocks, 148 * 8)), 256, smem, ctx->stream>>>(a, lm1, out_row, ctx->d_flags);
        post_launch(ctx);
    } else {
        raise(VF_ERR_UNSUPPORTED, "no fused kernel for this weight quantization pattern");
    }
}

}  // namespace vf
