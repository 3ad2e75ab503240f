// Fused weight-quantization kernels (the hot path): range statistics, calcScaleAndZeroPoint, Quantize and
// the store stage (BitPack / OIYX->OYXI reorder / zero padding / Dequantize copy) in ONE pass over the
// input. All of them are bandwidth-bound: the unit (group chunk or row) is staged in shared memory with
// 16-byte asynchronous copies (cp.async), statistics run on packed 16-bit pairs, the quantization sweep
// re-reads shared memory, stores are 16 bytes per lane. One launch processes a whole table of tensors so that
// small tensors do not pay a launch and a tail each.
//
// Arithmetic contract: codes equal the reference's fakeQuantize chain bit for bit. The per-element fast path
// evaluates  t = fma(x, inv, c)  with inv = fl((L-1)/range), c = fl(-inLow*inv)  instead of the reference's
// fl(fl((x-inLow)/range) * (L-1)). Six roundings separate the two (constant, reciprocal, fma; subtraction,
// division, multiplication), each at most 2^-24 * (L-1) in absolute terms, plus one more when qmin is folded
// into the constant: |t - reference| < 4.2e-7 * L. Whenever t is further than guard = 8e-7 * L from a rounding
// boundary (x.5) both round to the same integer; elements inside the guard band (2e-4 wide for 8-bit ranges,
// 1.3e-5 for 4-bit) are recomputed with the exact operation sequence.
#include <algorithm>
#include <vector>

#include "device_utils.cuh"
#include "kernels.h"

namespace vf {

namespace {

constexpr float kMagic = 12582912.0f;  // 1.5 * 2^23: adding it rounds to the nearest integer (ties to even)
constexpr int kMagicBits = 0x4B400000; // its bit pattern; the low byte is zero
constexpr float kGuardPerLevel = 8.0e-7f;

struct UnitQ {  // per-unit constants
    float inv;     // fl((L-1) / range)
    float c;       // fl(-inLow * inv) (+ qmin where noted)
    float in_low;  // exact path
    float range;   // fl(inHigh - inLow)
};

struct LaunchParams {  // uniform over all jobs of one launch
    int range_mode;
    int qmin, qmax, lm1;
    int dequant_dt;
    int njobs;
    float thr;            // 0.5 - guard: largest rounding residual the fast path accepts
    int64_t total_units;  // chunks (k_group) or rows (k_row / k_conv) over all jobs
};

// Per-unit parameters from the unit's range.
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
    static __device__ __forceinline__ float2 both(uint32_t w) { return __half22float2(*reinterpret_cast<__half2*>(&w)); }
};
template <>
struct P2<__nv_bfloat16> {
    using T = __nv_bfloat162;
    static __device__ __forceinline__ float lo(uint32_t w) { return __uint_as_float(w << 16); }
    static __device__ __forceinline__ float hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }
    static __device__ __forceinline__ float2 both(uint32_t w) { return make_float2(lo(w), hi(w)); }
};

template <typename InT>
__device__ __forceinline__ typename P2<InT>::T as_p2(uint32_t w) {
    return *reinterpret_cast<typename P2<InT>::T*>(&w);
}
template <typename T2>
__device__ __forceinline__ uint32_t as_u32(T2 v) {
    return *reinterpret_cast<uint32_t*>(&v);
}

// running element-wise min / max over 16-byte vectors (two 32-bit pair registers)
template <typename InT>
struct MinMax2 {
    using T2 = typename P2<InT>::T;
    T2 mn, mx;
    __device__ __forceinline__ MinMax2() {
        mn = as_p2<InT>(0u);
        mx = as_p2<InT>(0u);
    }
    __device__ __forceinline__ void add(const uint4& d) {
        const T2 a = as_p2<InT>(d.x), b = as_p2<InT>(d.y), c = as_p2<InT>(d.z), e = as_p2<InT>(d.w);
        mn = __hmin2(mn, __hmin2(__hmin2(a, b), __hmin2(c, e)));
        mx = __hmax2(mx, __hmax2(__hmax2(a, b), __hmax2(c, e)));
    }
    __device__ __forceinline__ float min_f() const {
        const uint32_t w = as_u32(mn);
        return fminf(P2<InT>::lo(w), P2<InT>::hi(w));
    }
    __device__ __forceinline__ float max_f() const {
        const uint32_t w = as_u32(mx);
        return fmaxf(P2<InT>::lo(w), P2<InT>::hi(w));
    }
};

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
// The largest rounding residual is tracked with max (no per-element branch); one comparison per vector.
// quant8_worst folds the vector's largest residual into `worst`, so a caller can test several vectors at once.
template <typename InT>
__device__ __forceinline__ void quant8_worst(const uint4& d, float inv, float c, float* m, float& worst) {
    // Packed two-wide fp32 instructions (sm_100): each is the same IEEE round-to-nearest operation on both
    // halves, so the results equal the scalar sequence bit for bit at half the issue slots. t - s is formed
    // as fma(s, -1, t): the product is exact, so it rounds once like the subtraction.
    const uint32_t w[4] = {d.x, d.y, d.z, d.w};
    const float2 inv2 = make_float2(inv, inv), c2 = make_float2(c, c);
    const float2 mg = make_float2(kMagic, kMagic), nmg = make_float2(-kMagic, -kMagic), neg1 = make_float2(-1.f, -1.f);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 x = P2<InT>::both(w[i]);
        const float2 t = __ffma2_rn(x, inv2, c2);
        const float2 mm = __fadd2_rn(t, mg);
        const float2 s = __fadd2_rn(mm, nmg);
        const float2 r = __ffma2_rn(s, neg1, t);
        m[2 * i] = mm.x;
        m[2 * i + 1] = mm.y;
        worst = fmaxf(worst, fmaxf(fabsf(r.x), fabsf(r.y)));
    }
}
template <typename InT>
__device__ __forceinline__ bool quant8(const uint4& d, float inv, float c, float thr, float* m) {
    float worst = 0.f;
    quant8_worst<InT>(d, inv, c, m, worst);
    return worst > thr;
}

// Repair of a vector that has an element in the guard band (rare): every element is re-evaluated, those inside
// the band with the exact sequence. Everything travels by value so that the caller's registers never need an
// address; returns the eight indices n (0..255) as bytes. `bias` is what the caller folded into c.
__device__ __forceinline__ uint32_t quant1_fix(float x, float inv, float c, float thr, float in_low, float range,
                                               int lm1, int bias) {
    const float t = __fmaf_rn(x, inv, c);
    const float m = __fadd_rn(t, kMagic);
    const float resid = __fsub_rn(t, __fsub_rn(m, kMagic));
    int n = (__float_as_int(m) - kMagicBits) - bias;
    if (fabsf(resid) > thr) n = quant_index_exact(x, in_low, range, lm1);
    return uint32_t(min(max(n, 0), lm1));
}
template <typename InT>
__device__ __noinline__ uint2 quant8_fix_bytes(uint4 d, float inv, float c, float thr, float in_low, float range,
                                               int lm1, int bias) {
    uint2 r;
    r.x = quant1_fix(P2<InT>::lo(d.x), inv, c, thr, in_low, range, lm1, bias) |
          (quant1_fix(P2<InT>::hi(d.x), inv, c, thr, in_low, range, lm1, bias) << 8) |
          (quant1_fix(P2<InT>::lo(d.y), inv, c, thr, in_low, range, lm1, bias) << 16) |
          (quant1_fix(P2<InT>::hi(d.y), inv, c, thr, in_low, range, lm1, bias) << 24);
    r.y = quant1_fix(P2<InT>::lo(d.z), inv, c, thr, in_low, range, lm1, bias) |
          (quant1_fix(P2<InT>::hi(d.z), inv, c, thr, in_low, range, lm1, bias) << 8) |
          (quant1_fix(P2<InT>::lo(d.w), inv, c, thr, in_low, range, lm1, bias) << 16) |
          (quant1_fix(P2<InT>::hi(d.w), inv, c, thr, in_low, range, lm1, bias) << 24);
    return r;
}

// Overwrites m[] with the patterns kMagicBits + n + bias of the repaired vector.
#define VF_QUANT8_FIX(InT, d, u, thr, lm1, bias, m)                                                        \
    do {                                                                                                   \
        const uint2 ex_ = quant8_fix_bytes<InT>(d, (u).inv, (u).c, thr, (u).in_low, (u).range, lm1, bias); \
        _Pragma("unroll") for (int k_ = 0; k_ < 4; ++k_) {                                                 \
            m[k_] = __int_as_float(kMagicBits + int((ex_.x >> (8 * k_)) & 0xFFu) + (bias));                \
            m[4 + k_] = __int_as_float(kMagicBits + int((ex_.y >> (8 * k_)) & 0xFFu) + (bias));            \
        }                                                                                                  \
    } while (0)

// eight patterns (kMagicBits + n) -> eight nibbles of n in one word, element 0 in the low nibble (BitPack<4>)
__device__ __forceinline__ uint32_t pack_nibbles(const float* m) {
    // summed as a tree (three dependent multiply-adds instead of seven)
    const uint32_t a = __float_as_uint(m[0]) + (__float_as_uint(m[1]) << 4);
    const uint32_t b = __float_as_uint(m[2]) + (__float_as_uint(m[3]) << 4);
    const uint32_t c = __float_as_uint(m[4]) + (__float_as_uint(m[5]) << 4);
    const uint32_t d = __float_as_uint(m[6]) + (__float_as_uint(m[7]) << 4);
    const uint32_t w = (a + (b << 8)) + ((c + (d << 8)) << 16);
    constexpr uint32_t kC = uint32_t(kMagicBits) * 0x11111111u;  // the magic part of the sum
    return w - kC;
}
// four patterns -> four low bytes
__device__ __forceinline__ uint32_t pack_bytes4(const float* m) {
    const uint32_t a = __byte_perm(__float_as_uint(m[0]), __float_as_uint(m[1]), 0x0040);
    const uint32_t b = __byte_perm(__float_as_uint(m[2]), __float_as_uint(m[3]), 0x0040);
    return __byte_perm(a, b, 0x5410);
}

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

__device__ __forceinline__ uint32_t lds_u16(uint32_t addr) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
// stores through the global window (no memory clobber: they never alias the shared-memory stage, so the
// compiler may move shared-memory loads across them; barriers still order them)
__device__ __forceinline__ void st_global_v2(void* p, uint32_t a, uint32_t b) {
    asm volatile("st.global.v2.u32 [%0], {%1, %2};" ::"l"(__cvta_generic_to_global(p)), "r"(a), "r"(b));
}
__device__ __forceinline__ void st_global_v4(void* p, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(__cvta_generic_to_global(p)), "r"(a), "r"(b), "r"(c), "r"(d));
}

// ======================================================================================================
// K_group: units of G consecutive elements (per-group quantization), 2-byte input.
// A warp owns a chunk of 32 consecutive groups (32*G elements, contiguous in memory). The chunk is copied
// into the warp's shared-memory stage with coalesced 16-byte cp.async (lane l copies vectors l, l+32, ...);
// afterwards LANE g OWNS GROUP g: it reads the group's V = G/8 vectors back (XOR-swizzled so that both access
// patterns are free of bank conflicts), reduces min/max on packed pairs, derives scale / zero point (all 32
// lanes busy in the FP64 section), quantizes and stores its own 16-byte pieces. No shuffles on the data path.
// Warps loop over the chunks of all jobs of the launch.
// ======================================================================================================
template <typename InT, int G, bool PACK4>
__global__ void __launch_bounds__(256, 3) k_group(const RowQuantArgs* __restrict__ jobs, LaunchParams p, int* flags) {
    constexpr int V = G / 8;  // vectors per group = vectors per lane per chunk
    extern __shared__ uint4 smem_u4[];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    uint4* stage = smem_u4 + wid * ((V + 1) * 32);
    const int64_t nwarps = int64_t(gridDim.x) * (blockDim.x >> 5);

    int j = 0;
    int64_t job_end = 0;  // first chunk of the next job
    // job fields, reloaded only when the warp moves to another job
    const InT* in = nullptr;
    uint8_t* codes = nullptr;
    double* o_scales = nullptr;
    int64_t* o_zps = nullptr;
    uint16_t* o_f16 = nullptr;
    uint8_t* o_u4 = nullptr;
    void* o_deq = nullptr;
    int64_t total_groups = 0, unit_begin = 0;

    for (int64_t chunk = int64_t(blockIdx.x) * (blockDim.x >> 5) + wid; chunk < p.total_units; chunk += nwarps) {
        if (chunk >= job_end) {
            j = find_job(jobs, p.njobs, chunk);
            const RowQuantArgs J = jobs[j];
            in = static_cast<const InT*>(J.in);
            codes = static_cast<uint8_t*>(J.codes);
            o_scales = J.scales;
            o_zps = J.zps;
            o_f16 = J.scales_f16;
            o_u4 = J.zps_u4;
            o_deq = J.dequant;
            total_groups = J.rows * (J.cols / G);
            unit_begin = J.unit_begin;
            job_end = j + 1 < p.njobs ? jobs[j + 1].unit_begin : p.total_units;
        }
        const int64_t g0 = (chunk - unit_begin) * 32;
        const int64_t total_elems = total_groups * G;
        const int64_t e0 = g0 * G;
        const uint4* src = reinterpret_cast<const uint4*>(in + e0);

        // vector i of the chunk is stored at i + i / V: every group's V vectors are followed by one vector of
        // padding, so the copy (lanes write consecutive vectors) and the sweeps (lane g reads group g, lane
        // stride V + 1 vectors) both spread over all banks
        const uint4* src_l = src + lane;
        uint4* dst_l = stage + lane + lane / V;
        if (e0 + int64_t(32) * G <= total_elems) {
#pragma unroll
            for (int v = 0; v < V; ++v) cp_async16(dst_l + v * 32 + (v * 32) / V, src_l + v * 32, true);
        } else {
#pragma unroll
            for (int v = 0; v < V; ++v)
                cp_async16(dst_l + v * 32 + (v * 32) / V, src_l + v * 32, e0 + int64_t(v * 32 + lane) * 8 < total_elems);
        }
        cp_async_wait_all();
        __syncwarp();  // lanes read vectors copied by other lanes

        // ---- statistics of group g0+lane ----------------------------------------------------------------
        const uint4* mine = stage + lane * (V + 1);
#define VF_MINE(k) mine[(k)]
        MinMax2<InT> mm;
#pragma unroll
        for (int k = 0; k < V; ++k) mm.add(VF_MINE(k));

        double scale;
        long long zp;
        UnitQ u;
        derive_unit(mm.min_f(), mm.max_f(), p, scale, zp, u, flags);
        const int64_t g = g0 + lane;
        const bool g_ok = g < total_groups;
        if (g_ok) {
            if (o_scales) o_scales[g] = scale;
            if (o_zps) o_zps[g] = zp;
            if (o_f16) o_f16[g] = f32_to_f16_bits(__double2float_rn(scale));
        }
        if (o_u4) {
            const int hi = __shfl_down_sync(0xffffffffu, int(zp), 1);
            if ((lane & 1) == 0 && g_ok) {
                const int hv = (g + 1 < total_groups) ? (hi & 0xF) : 0;
                o_u4[g >> 1] = uint8_t((hv << 4) | (int(zp) & 0xF));
            }
        }

        // ---- quantize + store: the lane's group is G consecutive codes ----------------------------------
        const int add = p.qmin;  // code = n + qmin
        if (PACK4) {
            uint4* dst = reinterpret_cast<uint4*>(codes + (e0 >> 1) + int64_t(lane) * (G / 2));
#pragma unroll 1
            for (int k4 = 0; k4 < V / 4; ++k4) {  // four vectors = 32 codes = 16 packed bytes
                // (one guard-band test per vector: testing the four vectors of a step together measured 9 % slower)
                uint32_t w[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const uint4 d = VF_MINE(k4 * 4 + q);
                    float m[8];
                    if (quant8<InT>(d, u.inv, u.c, p.thr, m)) VF_QUANT8_FIX(InT, d, u, p.thr, p.lm1, 0, m);
                    w[q] = pack_nibbles(m);
                    if (add != 0) {  // signed 4-bit ranges: add qmin to every nibble, modulo 16
                        const uint32_t qq = (uint32_t(add) & 0xFu) * 0x01010101u;
                        w[q] = (((w[q] & 0x0F0F0F0Fu) + qq) & 0x0F0F0F0Fu) | (((((w[q] >> 4) & 0x0F0F0F0Fu) + qq) & 0x0F0F0F0Fu) << 4);
                    }
                }
                if (g_ok) st_global_v4(dst + k4, w[0], w[1], w[2], w[3]);
            }
        } else {
            uint4* dst = reinterpret_cast<uint4*>(codes + e0 + int64_t(lane) * G);
#pragma unroll 1
            for (int k2 = 0; k2 < V / 2; ++k2) {  // two vectors = 16 codes = 16 bytes
                uint32_t w[4];
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                    const uint4 d = VF_MINE(k2 * 2 + q);
                    float m[8];
                    if (quant8<InT>(d, u.inv, u.c, p.thr, m)) VF_QUANT8_FIX(InT, d, u, p.thr, p.lm1, 0, m);
                    if (add != 0) {
#pragma unroll
                        for (int i = 0; i < 8; ++i) m[i] = __int_as_float(__float_as_int(m[i]) + add);
                    }
                    w[2 * q] = pack_bytes4(m);
                    w[2 * q + 1] = pack_bytes4(m + 4);
                }
                if (g_ok) st_global_v4(dst + k2, w[0], w[1], w[2], w[3]);
            }
        }
        if (o_deq && g_ok) {  // optional Dequantize copy (not on the benchmarked path): exact FP64 formula
            const int64_t eg = e0 + int64_t(lane) * G;
#pragma unroll 1
            for (int k = 0; k < V; ++k) {
                const uint4 d = VF_MINE(k);
                float m[8];
                if (quant8<InT>(d, u.inv, u.c, p.thr, m)) VF_QUANT8_FIX(InT, d, u, p.thr, p.lm1, 0, m);
#pragma unroll 1
                for (int i = 0; i < 8; ++i) {
                    const int q = (__float_as_int(m[i]) - kMagicBits) + add;
                    if (p.dequant_dt == VF_DT_F32) static_cast<float*>(o_deq)[eg + k * 8 + i] = dequantize_exact(q, scale, zp);
                    else static_cast<uint16_t*>(o_deq)[eg + k * 8 + i] = dequant16(q, zp, scale, p.dequant_dt);
                }
            }
        }
        __syncwarp();  // the stage is overwritten by the next chunk's copies
    }
}

// ======================================================================================================
// K_row: one unit per row, 16-byte aligned rows of a [rows, cols] matrix (per-output-channel quantization of
// linear weights), 2-byte input. A CTA of 256 threads is split into 256 / T independent row groups: the T
// threads of a group stage one row in shared memory and walk the rows of all jobs on their own, synchronising
// through the group's named barrier only. While one group sits in the scalar FP64 derivation of its row's
// scale, the other groups of the SM keep sweeping. The optional Dequantize copy uses a per-row table of the L
// possible outputs (each entry computed with the exact FP64 formula, indexed by the code byte), so the sweep
// costs one shared-memory lookup per element.
// ======================================================================================================
template <int T>
__device__ __forceinline__ void group_sync(int bar_id) {
    if (T == 256) __syncthreads();
    else asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "n"(T) : "memory");
}

template <typename InT, int T, int DQ>  // DQ: 0 = no dequantized copy, 1 = 16-bit float copy, 2 = f32 copy
__global__ void __launch_bounds__(256, 3) k_row(const RowQuantArgs* __restrict__ jobs, LaunchParams p, int stage_vecs,
                                             int* flags) {
    constexpr int THREADS = T;
    constexpr int kGroups = 256 / T;
    constexpr int kFixCap = 128;  // vectors noted for repair per row; beyond that the sweep repairs inline
    extern __shared__ uint4 smem_all[];
    struct GroupShared {
        float mn[T / 32], mx[T / 32];
        UnitQ u;
        double scale;
        long long zp;
        int fix[kFixCap];   // vectors with an element in the guard band
        int fix2[kFixCap];  // elements in the guard band
        int nfix, nfix2;
    };
    __shared__ GroupShared gs_all[kGroups];
    // dequantized value of code byte b: 16-bit entries (DQ == 1) or 32-bit entries; aligned to its size so that
    // an entry's address is the table's address OR the entry's offset
    __shared__ __align__(1024) uint32_t s_lut_all[kGroups][256];
    const int grp = threadIdx.x / T, tid = threadIdx.x % T, lane = tid & 31, wid = tid >> 5;
    GroupShared& gs = gs_all[grp];
    float* const s_mn = gs.mn;
    float* const s_mx = gs.mx;
    uint32_t* const s_lut = s_lut_all[grp];
    const uint32_t lut_sh = uint32_t(__cvta_generic_to_shared(s_lut));
    int* const s_fix = gs.fix;
    uint4* const smem_u4 = smem_all + size_t(grp) * size_t(stage_vecs);
    const int bar_id = 1 + grp;
    const int bias = p.qmin;  // code = n + qmin
    if (tid == 0) {  // made visible by the first barrier of the row loop
        gs.nfix = 0;
        gs.nfix2 = 0;
    }

    int j = 0;
    int64_t job_end = 0;
    const InT* in = nullptr;
    uint8_t* o_codes = nullptr;
    double* o_scales = nullptr;
    int64_t* o_zps = nullptr;
    uint16_t* o_f16 = nullptr;
    uint8_t* o_deq = nullptr;
    int64_t cols = 0, unit_begin = 0;

    const int64_t row_stride = int64_t(gridDim.x) * kGroups;
    for (int64_t row = int64_t(blockIdx.x) * kGroups + grp; row < p.total_units; row += row_stride) {
        if (row >= job_end) {
            j = find_job(jobs, p.njobs, row);
            const RowQuantArgs J = jobs[j];
            in = static_cast<const InT*>(J.in);
            o_codes = static_cast<uint8_t*>(J.codes);
            o_scales = J.scales;
            o_zps = J.zps;
            o_f16 = J.scales_f16;
            o_deq = static_cast<uint8_t*>(J.dequant);
            cols = J.cols;
            unit_begin = J.unit_begin;
            job_end = j + 1 < p.njobs ? jobs[j + 1].unit_begin : p.total_units;
        }
        const int64_t r = row - unit_begin;
        const int nvec = int(cols >> 3);
        const uint4* src = reinterpret_cast<const uint4*>(in + r * cols);
        for (int i = tid; i < nvec; i += THREADS) cp_async16(smem_u4 + i, src + i, true);
        cp_async_wait_all();  // every thread reads back only the vectors it copied itself

        MinMax2<InT> mm;
        for (int i = tid; i < nvec; i += THREADS) mm.add(smem_u4[i]);
        float mn = warp_min(mm.min_f()), mx = warp_max(mm.max_f());
        if (lane == 0) {
            s_mn[wid] = mn;
            s_mx[wid] = mx;
        }
        group_sync<T>(bar_id);
        if (wid == 0) {
            mn = lane < THREADS / 32 ? s_mn[lane] : 0.f;
            mx = lane < THREADS / 32 ? s_mx[lane] : 0.f;
            mn = warp_min(mn);
            mx = warp_max(mx);
            if (lane == 0) {
                double scale;
                long long zp;
                UnitQ u;
                derive_unit(mn, mx, p, scale, zp, u, flags);
                // shift the rounding target by qmin so that the low byte of (t + magic) is the code in two's
                // complement; the extra rounding of the constant stays inside the guard band (|c + qmin| <= 255)
                u.c = __fadd_rn(u.c, float(bias));
                gs.u = u;
                gs.scale = scale;
                gs.zp = zp;
                if (o_scales) o_scales[r] = scale;
                if (o_zps) o_zps[r] = zp;
                if (o_f16) o_f16[r] = f32_to_f16_bits(__double2float_rn(scale));
            }
        }
        group_sync<T>(bar_id);
        const UnitQ u = gs.u;
        if (DQ != 0) {
            const double scale = gs.scale;
            const long long zp = gs.zp;
            for (int n = tid; n <= p.lm1; n += THREADS) {
                const int code = n + bias;
                const float f = dequantize_exact(code, scale, zp);
                if (DQ == 2) s_lut[code & 0xFF] = __float_as_uint(f);
                else reinterpret_cast<uint16_t*>(s_lut)[code & 0xFF] = p.dequant_dt == VF_DT_F16 ? f32_to_f16_clamped_bits(f) : f32_to_bf16_bits(f);
            }
            group_sync<T>(bar_id);
        }
        uint8_t* const codes_row = o_codes + r * cols;
        uint8_t* const deq_row = DQ == 0 ? nullptr : o_deq + r * cols * (DQ == 1 ? 2 : 4);
        const float thr = p.thr;
        // The sweep handles kBatch vectors per step: all shared-memory loads of the step are issued first, then
        // the independent arithmetic chains and the stores.
        constexpr int kBatch = 4;
        for (int i0 = tid; i0 < nvec; i0 += kBatch * THREADS) {
            uint4 d[kBatch];
#pragma unroll
            for (int b = 0; b < kBatch; ++b) {
                const int i = i0 + b * THREADS;
                d[b] = i < nvec ? smem_u4[i] : make_uint4(0u, 0u, 0u, 0u);
            }
#pragma unroll
            for (int b = 0; b < kBatch; ++b) {
                const int i = i0 + b * THREADS;
                if (i >= nvec) break;
                float m[8];
                if (quant8<InT>(d[b], u.inv, u.c, thr, m)) {
                    // a vector with an element in the guard band is noted and repaired after the sweep, so the
                    // sweep itself never diverges into the exact sequence
                    const int slot = atomicAdd(&gs.nfix, 1);
                    if (slot < kFixCap) s_fix[slot] = i;
                    else VF_QUANT8_FIX(InT, d[b], u, thr, p.lm1, bias, m);
                }
                const uint32_t w0 = pack_bytes4(m), w1 = pack_bytes4(m + 4);
                st_global_v2(codes_row + size_t(i) * 8, w0, w1);
                if (DQ != 0) {
                    // table entry of byte k of w: shift the byte to the entry's offset, mask it and OR the table's
                    // (size-aligned) shared-memory address in, all in one logic instruction after the shift
                    constexpr int kSh = DQ == 1 ? 1 : 2;
                    constexpr uint32_t kMask = DQ == 1 ? 0x1FEu : 0x3FCu;
                    uint32_t q[8];
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const uint32_t o0 = ((k == 0 ? (w0 << kSh) : (w0 >> (8 * k - kSh))) & kMask) | lut_sh;
                        const uint32_t o1 = ((k == 0 ? (w1 << kSh) : (w1 >> (8 * k - kSh))) & kMask) | lut_sh;
                        q[k] = DQ == 1 ? lds_u16(o0) : lds_u32(o0);
                        q[4 + k] = DQ == 1 ? lds_u16(o1) : lds_u32(o1);
                    }
                    if (DQ == 2) {
                        st_global_v4(deq_row + size_t(i) * 32, q[0], q[1], q[2], q[3]);
                        st_global_v4(deq_row + size_t(i) * 32 + 16, q[4], q[5], q[6], q[7]);
                    } else {
                        st_global_v4(deq_row + size_t(i) * 16, __byte_perm(q[0], q[1], 0x5410), __byte_perm(q[2], q[3], 0x5410),
                                     __byte_perm(q[4], q[5], 0x5410), __byte_perm(q[6], q[7], 0x5410));
                    }
                }
            }
        }
        group_sync<T>(bar_id);
        // Repair in two steps so that the exact sequence runs on full warps: first one thread per element of
        // every noted vector lists the elements that really lie in the guard band, then the listed elements are
        // recomputed exactly and patched in place (the others keep what the sweep stored).
        const int nfix = min(gs.nfix, kFixCap);
        if (nfix > 0) {
            const uint16_t* row16 = reinterpret_cast<const uint16_t*>(smem_u4);
            auto patch = [&](int idx) {
                const float x = P2<InT>::lo(uint32_t(row16[idx]));
                const int code = quant_index_exact(x, u.in_low, u.range, p.lm1) + bias;
                codes_row[idx] = uint8_t(code);
                if (DQ == 1) reinterpret_cast<uint16_t*>(deq_row)[idx] = reinterpret_cast<const uint16_t*>(s_lut)[code & 0xFF];
                if (DQ == 2) reinterpret_cast<uint32_t*>(deq_row)[idx] = s_lut[code & 0xFF];
            };
            for (int e = tid; e < nfix * 8; e += THREADS) {
                const int idx = s_fix[e >> 3] * 8 + (e & 7);
                const float x = P2<InT>::lo(uint32_t(row16[idx]));
                const float t = __fmaf_rn(x, u.inv, u.c);
                const float mg = __fadd_rn(t, kMagic);
                if (fabsf(__fsub_rn(t, __fsub_rn(mg, kMagic))) > thr) {
                    const int slot = atomicAdd(&gs.nfix2, 1);
                    if (slot < kFixCap) gs.fix2[slot] = idx;
                    else patch(idx);
                }
            }
            group_sync<T>(bar_id);
            const int nfix2 = min(gs.nfix2, kFixCap);
            for (int e = tid; e < nfix2; e += THREADS) patch(gs.fix2[e]);
        }
        group_sync<T>(bar_id);  // u, the table and the repair list are rewritten by the next row
        if (tid == 0) {
            gs.nfix = 0;
            gs.nfix2 = 0;
        }
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
        const RowQuantArgs J = jobs[j];
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
        u.inv = u.c = u.in_low = u.range = 0.f;
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
            if (fabsf(resid) > p.thr) n = quant_index_exact(x, u.in_low, u.range, p.lm1);
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

// ======================================================================================================
// K_convv: the vectorised form of K_conv for 2-byte inputs whose rows are 16-byte multiples (every ResNet-style
// convolution with IC % 8 == 0). One warp per output channel: the row is copied into the warp's shared-memory
// stage with cp.async, min/max run on packed pairs, the codes are written back into the stage in input order
// (8 bytes per vector, over the vector they came from) and then copied out — straight for 1x1 kernels, transposed OIYX->OYXI otherwise
// (for every kernel tap s the lanes gather four codes of consecutive input channels and store one word).
// ======================================================================================================
template <typename InT>
__global__ void __launch_bounds__(256) k_convv(const RowQuantArgs* __restrict__ jobs, LaunchParams p, int in_vecs,
                                               int code_bytes, int* flags) {
    extern __shared__ uint4 smem_u4[];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    uint4* in_stage = smem_u4 + size_t(wid) * size_t(in_vecs);
    // the codes of vector v (8 bytes) overwrite the first half of the 16-byte slot the vector was read from
    const uint8_t* code_bytes_p = reinterpret_cast<const uint8_t*>(in_stage);
    (void)code_bytes;
    const int64_t nwarps = int64_t(gridDim.x) * (blockDim.x >> 5);
    const float thr = p.thr;
    int64_t job_end = 0;
    RowQuantArgs J;

    for (int64_t row = int64_t(blockIdx.x) * (blockDim.x >> 5) + wid; row < p.total_units; row += nwarps) {
        if (row >= job_end) {
            const int j = find_job(jobs, p.njobs, row);
            J = jobs[j];
            job_end = j + 1 < p.njobs ? jobs[j + 1].unit_begin : p.total_units;
        }
        const int64_t r = row - J.unit_begin;
        const int khw = J.khw > 0 ? int(J.khw) : 1;
        const int ic = J.khw > 0 ? int(J.ic) : int(J.cols);
        const int ic_pad = J.khw > 0 ? int(J.ic_pad) : int(J.cols);
        const int out_words = (khw * ic_pad) >> 2;
        uint32_t* out = reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(J.codes) + r * (int64_t(khw) * ic_pad));
        if (r >= J.rows) {  // padded output channel
            for (int w = lane; w < out_words; w += 32) out[w] = 0u;
            continue;
        }
        const int nvec = int(J.cols >> 3);
        const uint4* src = reinterpret_cast<const uint4*>(static_cast<const InT*>(J.in) + r * J.cols);
        for (int v = lane; v < nvec; v += 32) cp_async16(in_stage + v, src + v, true);
        cp_async_wait_all();  // each lane reads back only the vectors it copied itself

        MinMax2<InT> mm;
        for (int v = lane; v < nvec; v += 32) mm.add(in_stage[v]);
        const float mn = warp_min(mm.min_f()), mx = warp_max(mm.max_f());
        UnitQ u;
        u.inv = u.c = u.in_low = u.range = 0.f;
        if (lane == 0) {
            double scale;
            long long zp;
            derive_unit(mn, mx, p, scale, zp, u, flags);
            u.c = __fadd_rn(u.c, float(p.qmin));  // low byte of (t + magic) = code
            if (J.scales) J.scales[r] = scale;
            if (J.zps) J.zps[r] = zp;
            if (J.scales_f16) J.scales_f16[r] = f32_to_f16_bits(__double2float_rn(scale));
        }
        u.inv = __shfl_sync(0xffffffffu, u.inv, 0);
        u.c = __shfl_sync(0xffffffffu, u.c, 0);
        u.in_low = __shfl_sync(0xffffffffu, u.in_low, 0);
        u.range = __shfl_sync(0xffffffffu, u.range, 0);

        for (int v = lane; v < nvec; v += 32) {
            const uint4 d = in_stage[v];
            float m[8];
            if (quant8<InT>(d, u.inv, u.c, thr, m)) VF_QUANT8_FIX(InT, d, u, thr, p.lm1, p.qmin, m);
            *reinterpret_cast<uint2*>(in_stage + v) = make_uint2(pack_bytes4(m), pack_bytes4(m + 4));
        }
        __syncwarp();
        if (J.khw <= 0) {
            const uint32_t* c32 = reinterpret_cast<const uint32_t*>(in_stage);
            for (int w = lane; w < out_words; w += 32) out[w] = c32[(w >> 1) * 4 + (w & 1)];
        } else {
            const int icw = ic >> 2, padw = ic_pad >> 2;
            for (int s = 0; s < khw; ++s) {
                uint32_t* orow = out + s * padw;
                for (int w = lane; w < padw; w += 32) {
                    uint32_t word = 0;
                    if (w < icw) {
                        const int i0 = (w * 4) * khw + s;  // input index = channel * khw + tap
                        auto code_at = [&](int i) { return uint32_t(code_bytes_p[(i >> 3) * 16 + (i & 7)]); };
                        word = code_at(i0) | (code_at(i0 + khw) << 8) | (code_at(i0 + 2 * khw) << 16) | (code_at(i0 + 3 * khw) << 24);
                    }
                    orow[w] = word;
                }
            }
        }
        __syncwarp();  // both stages are rewritten by the next row
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
    const size_t smem = size_t(8) * (G / 8 + 1) * 32 * 16;  // 8 warps x 32 groups x (G/8 + 1 padding) vectors
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

template <typename InT, int T>
void launch_row_n(vf_ctx* ctx, const RowQuantArgs* d_jobs, const LaunchParams& p, int64_t max_cols, int dq) {
    constexpr int kGroups = 256 / T;
    const int stage_vecs = int((max_cols + 7) / 8);
    const size_t smem = size_t(kGroups) * size_t(stage_vecs) * 16;
    // persistent grid: as many CTAs as the runtime says fit an SM (shared memory and registers both count)
    auto ctas_per_sm = [&](auto kernel) {
        set_smem(kernel, smem);
        int n = 0;
        VF_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, 256, smem));
        return std::max(1, n);
    };
    const int per_sm = dq == 0 ? ctas_per_sm(k_row<InT, T, 0>) : dq == 1 ? ctas_per_sm(k_row<InT, T, 1>) : ctas_per_sm(k_row<InT, T, 2>);
    const int64_t ctas = (p.total_units + kGroups - 1) / kGroups;
    const int grid = int(std::min<int64_t>(ctas, int64_t(148) * int64_t(per_sm)));
    if (dq == 0) {
        k_row<InT, T, 0><<<grid, 256, smem, ctx->stream>>>(d_jobs, p, stage_vecs, ctx->d_flags);
    } else if (dq == 1) {
        k_row<InT, T, 1><<<grid, 256, smem, ctx->stream>>>(d_jobs, p, stage_vecs, ctx->d_flags);
    } else {
        k_row<InT, T, 2><<<grid, 256, smem, ctx->stream>>>(d_jobs, p, stage_vecs, ctx->d_flags);
    }
    post_launch(ctx);
}

template <typename InT>
void launch_row_t(vf_ctx* ctx, const RowQuantArgs* d_jobs, const LaunchParams& p, int64_t max_cols, int dq) {
    // threads per row: enough vectors per thread to amortise the per-row work, few enough that the rows in
    // flight on an SM (and with them the independent barriers) stay numerous
    if (max_cols <= 8192) launch_row_n<InT, 64>(ctx, d_jobs, p, max_cols, dq);
    else if (max_cols <= 16384) launch_row_n<InT, 128>(ctx, d_jobs, p, max_cols, dq);
    else launch_row_n<InT, 256>(ctx, d_jobs, p, max_cols, dq);
}

}  // namespace

// Which fused kernel covers `a`? 0 = none, 1 = group, 2 = row, 3 = conv (scalar), 4 = conv (vectorised)
int rowquant_kind(const RowQuantArgs& a) {
    const bool two_byte = a.in_dt == VF_DT_F16 || a.in_dt == VF_DT_BF16;
    const bool aligned16 = reinterpret_cast<uintptr_t>(a.in) % 16 == 0;
    if (a.group > 0) {
        if (two_byte && aligned16 && a.khw == 0 && a.rows_pad == a.rows && (a.group == 32 || a.group == 64 || a.group == 128) &&
            reinterpret_cast<uintptr_t>(a.codes) % 16 == 0)
            return 1;
        return 0;
    }
    if (two_byte && aligned16 && a.khw == 0 && a.rows_pad == a.rows && !a.pack4 && !a.zps_u4 && a.cols % 8 == 0 &&
        a.cols >= 1024 && a.cols <= 96 * 1024 && reinterpret_cast<uintptr_t>(a.codes) % 8 == 0 &&
        (!a.dequant || reinterpret_cast<uintptr_t>(a.dequant) % 16 == 0))
        return 2;
    if (!a.pack4 && !a.dequant && !a.zps_u4) {
        const int64_t out_row = a.khw > 0 ? a.khw * a.ic_pad : a.cols;
        const int64_t ic = a.khw > 0 ? a.ic : a.cols, ic_pad = a.khw > 0 ? a.ic_pad : a.cols;
        if (two_byte && aligned16 && a.cols % 8 == 0 && a.cols <= 4608 && out_row <= 4608 && ic % 4 == 0 && ic_pad % 4 == 0 &&
            reinterpret_cast<uintptr_t>(a.codes) % 4 == 0)
            return 4;
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
    p.thr = 0.5f - kGuardPerLevel * float(p.lm1 + 1);
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
    DBuf table;
    const RowQuantArgs* d_jobs =
            static_cast<const RowQuantArgs*>(upload_table(ctx, jobs.data(), jobs.size() * sizeof(RowQuantArgs), table));

    if (kind == 1) {
        if (a0.in_dt == VF_DT_F16) launch_group_t<__half>(ctx, d_jobs, p, a0.group, a0.pack4 != 0);
        else launch_group_t<__nv_bfloat16>(ctx, d_jobs, p, a0.group, a0.pack4 != 0);
    } else if (kind == 2) {
        const int dq = !a0.dequant ? 0 : (a0.dequant_dt == VF_DT_F32 ? 2 : 1);
        if (a0.in_dt == VF_DT_F16) launch_row_t<__half>(ctx, d_jobs, p, max_cols, dq);
        else launch_row_t<__nv_bfloat16>(ctx, d_jobs, p, max_cols, dq);
    } else if (kind == 4) {
        const int in_vecs = int((max_cols + 7) / 8);
        const int code_bytes = int((std::max(max_cols, max_out_row) + 15) & ~int64_t(15));
        const size_t smem = size_t(8) * size_t(in_vecs) * 16;
        const size_t per_sm = std::max<size_t>(1, std::min<size_t>(4, (220 * 1024) / (smem + 1024)));
        const int64_t blocks = (units + 7) / 8;
        const int grid = int(std::min<int64_t>(blocks, int64_t(148) * int64_t(per_sm)));
        if (a0.in_dt == VF_DT_F16) {
            set_smem(k_convv<__half>, smem);
            k_convv<__half><<<grid, 256, smem, ctx->stream>>>(d_jobs, p, in_vecs, code_bytes, ctx->d_flags);
        } else {
            set_smem(k_convv<__nv_bfloat16>, smem);
            k_convv<__nv_bfloat16><<<grid, 256, smem, ctx->stream>>>(d_jobs, p, in_vecs, code_bytes, ctx->d_flags);
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
    // long rows get their own launch: shared memory and block size are chosen per launch from the longest row
    const bool long_a = a.group == 0 && a.cols > 8192, long_b = b.group == 0 && b.cols > 8192;
    return a.in_dt == b.in_dt && a.group == b.group && a.range_mode == b.range_mode && a.qmin == b.qmin && a.qmax == b.qmax &&
           a.pack4 == b.pack4 && a.dequant_dt == b.dequant_dt && a.out_signed == b.out_signed &&
           (a.dequant != nullptr) == (b.dequant != nullptr) && long_a == long_b;
}

}  // namespace vf
