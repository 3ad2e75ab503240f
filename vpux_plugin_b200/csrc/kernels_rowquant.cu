// Fused weight-quantization kernels (the hot path): range statistics, calcScaleAndZeroPoint, Quantize and
// the store stage (BitPack / OIYX->OYXI reorder / zero padding / Dequantize copy) in ONE pass over the
// input. All of them are bandwidth-bound: the unit (group chunk or row) is staged in shared memory with
// 16-byte asynchronous copies (cp.async), statistics run on packed 16-bit pairs, the quantization sweep
// re-reads shared memory, stores are 16 bytes per lane. One launch processes a whole table of tensors so that
// small tensors do not pay a launch and a tail each. The per-unit parameters are either derived from the
// unit's own range or supplied by the caller (the Quantize attribute's scales and zero points).
//
// Arithmetic contract: codes equal the reference's fakeQuantize chain bit for bit. With the ideal index
//   T = x / scale + (zp - qmin)
// the reference evaluates e = fl(fl(fl(x - inLow) / range) * (L-1)) on the fp32 constants inLow = fl((qmin-zp)*scale),
// range = fl(inHigh - inLow) and rounds e half away from zero. The fast path evaluates ONE fused multiply-add
//   mm = fma(x, inv, magic + K),   inv = fl((L-1) / range),  magic = 1.5 * 2^23,  K an integer constant
// whose product is exact and whose sum is rounded once, to an integer (the ulp at magic is 1): the low bits of
// mm hold round(x * inv) + K. Against e the index x * inv + (zp - qmin) differs by at most 7 * 2^-24 * L
// (one rounding each in inv, inLow, the subtraction, the division and the multiplication, two in range),
// i.e. 4.2e-7 * L, so whenever x * inv is further than guard = 8e-7 * L from a rounding boundary (n + 0.5)
// both round to the same integer. The distance is the residual r = x * inv - round(x * inv), one more exact
// fused multiply-add; elements inside the guard band (2e-4 wide for 8-bit ranges, 1.3e-5 for 4-bit) are
// recomputed with the reference's own operation sequence.
//
// Where rounding boundaries are hit often (8-bit ranges, and bfloat16 data whose few mantissa bits put many
// elements exactly on a boundary) the kernels evaluate the reference's sequence itself, branch-free on packed
// pairs: a = fl(x - inLow); the division fl(a / range) as q0 = fl(a y), q = fma(fma(-q0, range, a), y, q0) with
// y = RN(1 / range), which is the correctly rounded quotient (Markstein's correction step with a correctly
// rounded reciprocal); e = fl(q (L-1)); and roundf(e) = floor(e + 1/2) as two additions rounded toward minus
// infinity, the second one onto the integer grid at 1.5 * 2^23. The clamps of fakeQuantize's outer branches are
// not evaluated per element: every step is monotonic in x, so a unit whose smallest and largest element stay
// inside [0, L-1] needs none, and a unit where they do not takes the scalar sequence.
#include <algorithm>
#include <type_traits>
#include <vector>

#include "device_utils.cuh"
#include "kernels.h"

namespace vf {

namespace {

constexpr float kMagic = 12582912.0f;  // 1.5 * 2^23: adding it rounds to the nearest integer (ties to even)
constexpr int kMagicBits = 0x4B400000; // its bit pattern; the low byte is zero
constexpr float kGuardPerLevel = 8.0e-7f;

struct UnitQ {  // per-unit constants
    float inv;     // (L-1) / range within a few ulps: the fast path only proposes, the guard band decides
    float zq;      // float(zp - qmin): index n = round(x * inv) + zq
    float in_low;  // exact path
    float range;   // fl(inHigh - inLow)
    float y;       // RN(1 / range): the exact path's division
};

struct LaunchParams {  // uniform over all jobs of one launch
    int range_mode;
    int qmin, qmax, lm1;
    int dequant_dt;
    int njobs;
    int given;            // parameters come from the jobs' given_scales / given_zps
    float thr;            // 0.5 - guard: largest rounding residual the fast path accepts
    double den, inv_den;  // qmax - qmin and RN(1 / (qmax - qmin))
    int64_t total_units;  // chunks (k_group) or rows (k_row / k_conv) over all jobs
    int64_t total_work;   // k_convv: sum of the units' costs
};

__device__ __forceinline__ void unit_consts(double scale, long long zp, const LaunchParams& p, UnitQ& u) {
    u.in_low = dequantize_exact(p.qmin, scale, zp);
    const float in_high = dequantize_exact(p.qmax, scale, zp);
    u.range = __fsub_rn(in_high, u.in_low);
    u.inv = __fdividef(float(p.lm1), u.range);
    u.y = __frcp_rn(u.range);
    u.zq = float(zp - p.qmin);
}

// Per-unit parameters from the unit's range: calcScaleAndZeroPoint (utils/quantization.cpp:574-636) with the two
// FP64 divisions made cheap. scale = (rMax - rMin) / (qMax - qMin) divides by a launch constant: one
// multiplication by the correctly rounded reciprocal and one correction step give the correctly rounded
// quotient. zp = round(qMin - rMin / scale) is an integer in the storage range: it is evaluated in fp32 first
// (error below 1e-4) and only a value within 1e-3 of a rounding boundary takes the FP64 division.
// the cases the cheap evaluation leaves out (kept out of line: two FP64 divisions and their temporaries): a zero
// point next to a rounding boundary (exact = true: scale is already final) and degenerate or extreme ranges
__device__ __noinline__ long long derive_unit_rare(float mn, float mx, int qmin, int qmax, bool exact, double& scale, int* flags) {
    long long zp;
    if (exact) return (long long)(round(__dsub_rn(double(qmin), __ddiv_rn(double(mn), scale))));
    if (!calc_scale_zp(double(qmin), double(qmax), double(mn), double(mx), scale, zp)) {
        set_flag(flags, VF_FLAG_QUANT_RANGE);
        scale = 1.0;
        zp = 0;
    }
    return zp;
}
__device__ __forceinline__ void derive_unit(float mn, float mx, const LaunchParams& p, double& scale, long long& zp,
                                            UnitQ& u, int* flags) {
    mn = fminf(mn, 0.f);  // the range always contains zero (calcScaleAndZeroPoint requires it)
    mx = fmaxf(mx, 0.f);
    if (p.range_mode == VF_RANGE_ABSMAX) {
        const float a = fmaxf(-mn, mx);
        mn = -a;
        mx = a;
    }
    const float df = __fsub_rn(mx, mn);
    if (df >= 7.8886091e-31f && df <= 1.2676506e30f) {  // 2^-100 .. 2^100: nothing under- or overflows below
        const double d = __dsub_rn(double(mx), double(mn));
        const double q0 = __dmul_rn(d, p.inv_den);
        scale = __fma_rn(__fma_rn(-q0, p.den, d), p.inv_den, q0);
        const float xf = __fmaf_rn(-mn, __fdividef(float(p.lm1), df), float(p.qmin));
        const float fl = floorf(xf);
        if (fabsf(__fsub_rn(__fsub_rn(xf, fl), 0.5f)) < 1.0e-3f) {
            zp = derive_unit_rare(mn, mx, p.qmin, p.qmax, true, scale, flags);
        } else {
            zp = (long long)(floorf(__fadd_rn(xf, 0.5f)));
        }
    } else {
        zp = derive_unit_rare(mn, mx, p.qmin, p.qmax, false, scale, flags);
    }
    zp = zp < p.qmin ? p.qmin : (zp > p.qmax ? p.qmax : zp);
    unit_consts(scale, zp, p, u);
}

// Supplied parameters need not cover the data. The fast path has no clamp, so it is used only when every
// element's index stays inside [-0.45, L-1 + 0.45] (anything closer to +-0.5 is in the guard band anyway) and
// the zero point lies in the storage range; other units take the exact sequence for every element.
__device__ __forceinline__ bool unit_fits(const UnitQ& u, float mn, float mx, long long zp, const LaunchParams& p) {
    const float lo = __fmaf_rn(mn, u.inv, u.zq), hi = __fmaf_rn(mx, u.inv, u.zq);
    return zp >= p.qmin && zp <= p.qmax && u.range >= 7.8886091e-31f && u.range <= 1.2676506e30f && lo >= -0.45f &&
           hi <= float(p.lm1) + 0.45f;
}

// The exact operation sequence of fakeQuantize's middle branch, as an index n in [0, L-1]. The first two
// branches (x <= inLow -> qLow, x > inHigh -> qHigh) coincide with the clamp for any x: x <= inLow gives
// fl(x - inLow) <= 0, x > inHigh gives fl(x - inLow) >= range (rounding is monotonic).
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
        mn = __hmin2_nan(mn, __hmin2_nan(__hmin2_nan(a, b), __hmin2_nan(c, e)));  // a NaN sticks to the running minimum
        mx = __hmax2(mx, __hmax2(__hmax2(a, b), __hmax2(c, e)));
    }
    // Quantize of a NaN is undefined in the reference (a NaN passes both comparisons of fakeQuantize and is cast
    // to an integer): the kernels report it
    __device__ __forceinline__ bool saw_nan() const {
        const uint32_t w = as_u32(mn);
        const float lo = P2<InT>::lo(w), hi = P2<InT>::hi(w);
        return lo != lo || hi != hi;
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
__device__ __forceinline__ void cp_async_commit() {
    asm volatile("cp.async.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void cp_async_wait() {  // at most N committed groups still in flight
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
    cp_async_commit();
    cp_async_wait<0>();
}

// ---- the fast quantizer on packed pairs --------------------------------------------------------------------
// Packed two-wide fp32 instructions (sm_100): each is the same IEEE round-to-nearest operation on both halves,
// so the results equal the scalar sequence bit for bit at half the issue slots.
struct PairQ {  // unit constants duplicated into both halves
    float2 inv;  // (L-1) / range
    float2 cm;   // magic + K
};
__device__ __forceinline__ float2 dup(float v) {
    return make_float2(v, v);
}
__device__ __forceinline__ PairQ pair_consts(float inv, float k) {
    PairQ q;
    q.inv = dup(inv);
    q.cm = dup(__fadd_rn(kMagic, k));  // exact: |k| is a small integer
    return q;
}
// One pair: mm = magic + K + round(x * inv) (as a float), sneg = -round(x * inv), and the largest |residual| so
// far. Only inv and cm are per-unit constants (few live registers: the sweep is unrolled over a whole group);
// negations go through multiplications by -1, which are exact.
__device__ __forceinline__ void quant2(const float2 x, const PairQ& q, float2& mm, float2& sneg, float& worst) {
    const float2 neg1 = dup(-1.f);
    mm = __ffma2_rn(x, q.inv, q.cm);
    sneg = __ffma2_rn(mm, neg1, q.cm);  // cm - mm, exact
    const float2 r = __ffma2_rn(x, q.inv, sneg);  // x * inv - round(x * inv): exact product, one rounding
    worst = fmaxf(worst, fmaxf(fabsf(r.x), fabsf(r.y)));
}

// ---- the exact sequence on packed pairs -------------------------------------------------------------------
struct ExactQ {
    float2 nlow, y, nrange, lm1, half;
    float2 cm;  // magic + K: the low bits of the result hold n + K
};
__device__ __forceinline__ ExactQ exact_consts(const UnitQ& u, int lm1, float k) {
    ExactQ q;
    q.nlow = dup(-u.in_low);
    q.y = dup(u.y);
    q.nrange = dup(-u.range);
    q.lm1 = dup(float(lm1));
    q.half = dup(0.5f);
    q.cm = dup(__fadd_rn(kMagic, k));
    return q;
}
// magic + K + roundf(fl(fl(fl(x - inLow) / range) * (L-1))) for both halves, unclamped
__device__ __forceinline__ float2 exact2(const float2 x, const ExactQ& q) {
    const float2 a = __fadd2_rn(x, q.nlow);
    const float2 q0 = __fmul2_rn(a, q.y);
    const float2 d = __ffma2_rn(__ffma2_rn(q0, q.nrange, a), q.y, q0);  // = fl(a / range)
    const float2 e = __fmul2_rn(d, q.lm1);
    return __fadd2_rd(__fadd2_rd(e, q.half), q.cm);  // floor(e + 1/2) on the integer grid
}
__device__ __forceinline__ float exact1_v(float x, const UnitQ& u, int lm1) {  // e + 1/2 rounded down, one element
    const float a = __fsub_rn(x, u.in_low);
    const float q0 = __fmul_rn(a, u.y);
    const float d = __fmaf_rn(__fmaf_rn(-q0, u.range, a), u.y, q0);
    return __fadd_rd(__fmul_rn(d, float(lm1)), 0.5f);
}
// The packed exact sequence has no clamp and divides through the reciprocal: it covers a unit whose range is
// far from the ends of the exponent range and whose smallest and largest element (every step is monotonic)
// give an index inside [0, L-1].
__device__ __forceinline__ bool unit_exact_ok(const UnitQ& u, float mn, float mx, const LaunchParams& p) {
    return u.range >= 7.8886091e-31f && u.range <= 1.2676506e30f && exact1_v(mn, u, p.lm1) >= 0.f &&
           exact1_v(mx, u, p.lm1) < float(p.lm1 + 1);
}
// Eight elements -> eight code bytes with the exact sequence (K = qmin: the low byte is the code). `s` (optional)
// receives code - zp of every element as floats; zpk = magic + zp.
template <typename InT, bool WANT_S>
__device__ __forceinline__ uint2 exact8_bytes(const uint4& d, const ExactQ& q, float2 nzpk, float2* s_out) {
    const uint32_t w[4] = {d.x, d.y, d.z, d.w};
    uint32_t b[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 m = exact2(P2<InT>::both(w[i]), q);
        b[i] = __byte_perm(__float_as_uint(m.x), __float_as_uint(m.y), 0x0040);
        if (WANT_S) s_out[i] = __fadd2_rn(m, nzpk);  // exact
    }
    return make_uint2(__byte_perm(b[0], b[1], 0x5410), __byte_perm(b[2], b[3], 0x5410));
}
// Eight elements -> eight nibbles with the exact sequence (K = 0: unsigned indices)
template <typename InT>
__device__ __forceinline__ uint32_t exact8_nibbles(const uint4& d, const ExactQ& q) {
    const float2 p16 = dup(16.f), nmg = dup(-kMagic);
    const float2 e01 = P2<InT>::both(d.x), e23 = P2<InT>::both(d.y), e45 = P2<InT>::both(d.z), e67 = P2<InT>::both(d.w);
    float2 ma = exact2(make_float2(e01.x, e23.x), q), mb = exact2(make_float2(e01.y, e23.y), q);
    const float2 c0 = __ffma2_rn(__fadd2_rn(mb, nmg), p16, ma);
    ma = exact2(make_float2(e45.x, e67.x), q);
    mb = exact2(make_float2(e45.y, e67.y), q);
    const float2 c1 = __ffma2_rn(__fadd2_rn(mb, nmg), p16, ma);
    const uint32_t lo = __byte_perm(__float_as_uint(c0.x), __float_as_uint(c0.y), 0x0040);
    const uint32_t hi = __byte_perm(__float_as_uint(c1.x), __float_as_uint(c1.y), 0x0040);
    return __byte_perm(lo, hi, 0x5410);
}

// Eight elements -> eight code bytes. K = zp, so the low byte of mm is the code in two's complement. `s` (optional)
// receives code - zp of every element as floats, in element order.
template <typename InT, bool WANT_S>
__device__ __forceinline__ uint2 quant8_bytes(const uint4& d, const PairQ& q, float& worst, float2* s_out) {
    const uint32_t w[4] = {d.x, d.y, d.z, d.w};
    uint32_t b[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 mm, sneg;
        quant2(P2<InT>::both(w[i]), q, mm, sneg, worst);
        b[i] = __byte_perm(__float_as_uint(mm.x), __float_as_uint(mm.y), 0x0040);
        if (WANT_S) s_out[i] = __ffma2_rn(sneg, dup(-1.f), dup(0.f));
    }
    return make_uint2(__byte_perm(b[0], b[1], 0x5410), __byte_perm(b[2], b[3], 0x5410));
}

// Eight elements -> one word of eight nibbles, element 0 in the low nibble (BitPack<4>). The unsigned index
// n = round(x * inv) + zq of an even element (K = 17 zq) and sixteen times the rounded product of its odd
// neighbour (K = zq) are added in floating point: the low byte of the sum is n_even + 16 n_odd.
template <typename InT>
__device__ __forceinline__ uint32_t quant8_nibbles(const uint4& d, const PairQ& qa, const PairQ& qb, float& worst) {
    const float2 n16 = dup(-16.f);
    const float2 e01 = P2<InT>::both(d.x), e23 = P2<InT>::both(d.y), e45 = P2<InT>::both(d.z), e67 = P2<InT>::both(d.w);
    float2 mma, sa, mmb, sb;
    quant2(make_float2(e01.x, e23.x), qa, mma, sa, worst);
    quant2(make_float2(e01.y, e23.y), qb, mmb, sb, worst);
    const float2 c0 = __ffma2_rn(sb, n16, mma);  // exact: small integers on top of magic
    quant2(make_float2(e45.x, e67.x), qa, mma, sa, worst);
    quant2(make_float2(e45.y, e67.y), qb, mmb, sb, worst);
    const float2 c1 = __ffma2_rn(sb, n16, mma);
    const uint32_t lo = __byte_perm(__float_as_uint(c0.x), __float_as_uint(c0.y), 0x0040);
    const uint32_t hi = __byte_perm(__float_as_uint(c1.x), __float_as_uint(c1.y), 0x0040);
    return __byte_perm(lo, hi, 0x5410);
}

// Repair of a vector that has an element in the guard band (rare), and the path of units the fast evaluation
// does not cover (`all`): every element is re-evaluated, those inside the band (or all) with the exact sequence.
// Everything travels by value so that the caller's registers never need an address; returns the eight indices
// n (0 .. L-1) as bytes.
__device__ __forceinline__ uint32_t quant1_fix(float x, const UnitQ u, float thr, int lm1, bool all) {
    const float cm = __fadd_rn(kMagic, u.zq);
    const float m = __fmaf_rn(x, u.inv, cm);
    const float s = __fsub_rn(m, cm);
    const float resid = __fmaf_rn(x, -u.inv, s);
    int n = __float_as_int(m) - kMagicBits;
    if (all || !(fabsf(resid) <= thr)) n = quant_index_exact(x, u.in_low, u.range, lm1);
    return uint32_t(min(max(n, 0), lm1));
}
template <typename InT>
__device__ __noinline__ uint2 quant8_fix_idx(uint4 d, UnitQ u, float thr, int lm1, bool all) {
    uint2 r;
    r.x = quant1_fix(P2<InT>::lo(d.x), u, thr, lm1, all) | (quant1_fix(P2<InT>::hi(d.x), u, thr, lm1, all) << 8) |
          (quant1_fix(P2<InT>::lo(d.y), u, thr, lm1, all) << 16) | (quant1_fix(P2<InT>::hi(d.y), u, thr, lm1, all) << 24);
    r.y = quant1_fix(P2<InT>::lo(d.z), u, thr, lm1, all) | (quant1_fix(P2<InT>::hi(d.z), u, thr, lm1, all) << 8) |
          (quant1_fix(P2<InT>::lo(d.w), u, thr, lm1, all) << 16) | (quant1_fix(P2<InT>::hi(d.w), u, thr, lm1, all) << 24);
    return r;
}
// index bytes -> code bytes (n + qmin in every byte, modulo 256)
__device__ __forceinline__ uint32_t idx_to_codes4(uint32_t idx, int qmin) {
    const uint32_t q = (uint32_t(qmin) & 0xFFu) * 0x01010101u;
    // byte-wise addition without carries between bytes
    return ((idx & 0x7F7F7F7Fu) + (q & 0x7F7F7F7Fu)) ^ ((idx ^ q) & 0x80808080u);
}
// four index bytes (each < 16) -> four nibbles in the low half word
__device__ __forceinline__ uint32_t idx_to_nibbles4(uint32_t idx) {
    return (idx & 0xFu) | ((idx >> 4) & 0xF0u) | ((idx >> 8) & 0xF00u) | ((idx >> 12) & 0xF000u);
}
// a word of unsigned 4-bit indices -> codes n + qmin, every nibble modulo 16
__device__ __forceinline__ uint32_t nibbles_add(uint32_t w, int qmin) {
    const uint32_t qq = (uint32_t(qmin) & 0xFu) * 0x01010101u;
    return (((w & 0x0F0F0F0Fu) + qq) & 0x0F0F0F0Fu) | (((((w >> 4) & 0x0F0F0F0Fu) + qq) & 0x0F0F0F0Fu) << 4);
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
// afterwards LANE g OWNS GROUP g: it reads the group's V = G/8 vectors back (one vector of padding per group
// keeps both access patterns free of bank conflicts), reduces min/max on packed pairs, derives scale / zero
// point (all 32 lanes busy in the FP64 section) and quantizes. The packed codes go back into the stage (over
// vectors the lane has already consumed) and leave as contiguous 16-byte stores of the whole warp. Warps loop
// over the chunks of all jobs of the launch.
// MODE: 0 = one code byte per element, 1 = BitPack<4> with qmin == 0, 2 = BitPack<4> with qmin != 0.
// ======================================================================================================
struct GroupJob {  // the job a warp is working on
    const void* in;
    uint8_t* codes;
    double* o_scales;
    int64_t* o_zps;
    uint16_t* o_f16;
    uint8_t* o_u4;
    void* o_deq;
    const double* g_scales;
    const int64_t* g_zps;
    int64_t total_groups, unit_begin, job_end;
};
template <typename InT, int G>
__device__ __forceinline__ void group_issue(uint4* stage, const GroupJob& S, int64_t chunk, int lane) {
    constexpr int V = G / 8;
    const int64_t e0 = (chunk - S.unit_begin) * 32 * G;
    const int64_t total_elems = S.total_groups * G;
    // vector i of the chunk is stored at i + i / V: every group's V vectors are followed by one vector of
    // padding, so the copy (lanes write consecutive vectors) and the sweeps (lane g reads group g, lane
    // stride V + 1 vectors) both spread over all banks
    const uint4* src_l = reinterpret_cast<const uint4*>(static_cast<const InT*>(S.in) + e0) + lane;
    uint4* dst_l = stage + lane + lane / V;
    if (e0 + int64_t(32) * G <= total_elems) {
#pragma unroll
        for (int v = 0; v < V; ++v) cp_async16(dst_l + v * 32 + (v * 32) / V, src_l + v * 32, true);
    } else {
#pragma unroll
        for (int v = 0; v < V; ++v)
            cp_async16(dst_l + v * 32 + (v * 32) / V, src_l + v * 32, e0 + int64_t(v * 32 + lane) * 8 < total_elems);
    }
}

// What the repair of a guard-band element needs beyond the fast path's constants: inLow, range and RN(1 / range).
struct UnitX {
    float in_low, range, y;
};
// The reference's sequence for one element with its clamp, division through the correctly rounded reciprocal
// (exact2, scalar): index n in [0, L-1].
__device__ __forceinline__ uint32_t exact1_index(float x, const UnitX& u, int lm1) {
    const float a = __fsub_rn(x, u.in_low);
    const float q0 = __fmul_rn(a, u.y);
    const float d = __fmaf_rn(__fmaf_rn(-q0, u.range, a), u.y, q0);
    const float v = __fadd_rd(__fmul_rn(d, float(lm1)), 0.5f);
    return uint32_t(min(max(int(floorf(v)), 0), lm1));
}

// Repair of a vector with an element in the guard band (about one vector in 500 of fp16 weights: mostly exact
// ties x * (L-1) / range = n + 1/2, which 16-bit data on a common grid produce), out of line so that the sweep
// stays small: every element is re-evaluated, those in the band (all of them in a unit the fast evaluation does
// not cover) with the exact sequence. A fast value can lie one outside [0, L-1] next to the ends of the range —
// always inside the band — which is why the word is rebuilt instead of patched. `have_x`: inLow / range / y are
// valid; otherwise they are derived here from the unit's range and zero point.
template <typename InT>
__device__ __noinline__ uint32_t repair8_nibbles(uint4 d, float inv, float zq, float thr, int lm1, bool fast, float in_low, float range,
                                                float y) {
    UnitX ux;
    ux.in_low = in_low;
    ux.range = range;
    ux.y = y;
    const uint32_t wd[4] = {d.x, d.y, d.z, d.w};
    uint32_t r = 0;
    const float cm = __fadd_rn(kMagic, zq);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float x = (i & 1) ? P2<InT>::hi(wd[i >> 1]) : P2<InT>::lo(wd[i >> 1]);
        const float m = __fmaf_rn(x, inv, cm);
        const float resid = __fmaf_rn(x, -inv, __fsub_rn(m, cm));
        int n = __float_as_int(m) - kMagicBits;
        if (!fast) n = quant_index_exact(x, ux.in_low, ux.range, lm1);
        else if (!(fabsf(resid) <= thr)) n = int(exact1_index(x, ux, lm1));
        r |= uint32_t(min(max(n, 0), lm1)) << (4 * i);
    }
    return r;
}

template <typename InT, int G, int MODE>
__device__ __forceinline__ void group_chunk(uint4* stage, const GroupJob& J, int64_t chunk, const LaunchParams& p, int lane,
                                            int* flags) {
    constexpr int V = G / 8;
    constexpr bool PACK4 = MODE != 0;
    // bfloat16 data sits on rounding boundaries too often for the guard-band scheme: exact sequence throughout
    constexpr bool EXACT = !std::is_same<InT, __half>::value;
    constexpr int VPS = PACK4 ? 4 : 2;  // input vectors per 16 bytes of codes
    constexpr int OV = V / VPS;         // 16-byte code vectors per group
    const int64_t g0 = (chunk - J.unit_begin) * 32;
    const int64_t e0 = g0 * G;
    uint4* mine = stage + lane * (V + 1);

    // ---- statistics of group g0 + lane --------------------------------------------------------------------
    MinMax2<InT> mm;
#pragma unroll
    for (int k = 0; k < V; ++k) mm.add(mine[k]);
    const float mn = mm.min_f(), mx = mm.max_f();
    if (mm.saw_nan()) set_flag(flags, VF_FLAG_NAN);

    const int64_t g = g0 + lane;
    const bool g_ok = g < J.total_groups;
    double scale = 1.0;
    long long zp = 0;
    UnitQ u;
    u.inv = u.zq = u.in_low = u.range = u.y = 0.f;
    bool fast = true;
    if (p.given) {
        scale = g_ok ? J.g_scales[g] : 1.0;
        zp = g_ok ? J.g_zps[g] : 0;
        unit_consts(scale, zp, p, u);
        fast = EXACT ? unit_exact_ok(u, mn, mx, p) : unit_fits(u, mn, mx, zp, p);
    } else {
        derive_unit(mn, mx, p, scale, zp, u, flags);
        fast = EXACT ? unit_exact_ok(u, mn, mx, p) : (u.range >= 7.8886091e-31f && u.range <= 1.2676506e30f);
        const int zpi = int(zp);
        const uint32_t s16 = f32_to_f16_bits(__double2float_rn(scale));
        if (g_ok) {
            if (J.o_scales) J.o_scales[g] = scale;
            if (J.o_zps) J.o_zps[g] = zp;
            if (J.o_f16) J.o_f16[g] = uint16_t(s16);
        }
        if (J.o_u4) {
            const int hi = __shfl_down_sync(0xffffffffu, zpi, 1);
            if ((lane & 1) == 0 && g_ok) {
                const int hv = (g + 1 < J.total_groups) ? (hi & 0xF) : 0;
                J.o_u4[g >> 1] = uint8_t((hv << 4) | (zpi & 0xF));
            }
        }
    }

    if (J.o_deq && g_ok) {  // optional Dequantize copy (not on the benchmarked path): exact FP64 formula
        const int64_t eg = e0 + int64_t(lane) * G;
#pragma unroll 1
        for (int k = 0; k < V; ++k) {
            const uint2 idx = quant8_fix_idx<InT>(mine[k], u, p.thr, p.lm1, !fast);
#pragma unroll 1
            for (int i = 0; i < 8; ++i) {
                const int q = int(((i < 4 ? idx.x : idx.y) >> (8 * (i & 3))) & 0xFFu) + p.qmin;
                if (p.dequant_dt == VF_DT_F32) static_cast<float*>(J.o_deq)[eg + k * 8 + i] = dequantize_exact(q, scale, zp);
                else static_cast<uint16_t*>(J.o_deq)[eg + k * 8 + i] = dequant16(q, zp, scale, p.dequant_dt);
            }
        }
    }

    // ---- quantize: the lane's group is G consecutive codes; code vector k replaces input vector k ----------
    if (PACK4 && !EXACT) {
        // guard-band path; a vector with an element in the band is rebuilt by repair8_nibbles
        const PairQ qa = pair_consts(u.inv, 17.f * u.zq), qb = pair_consts(u.inv, u.zq);
#pragma unroll
        for (int k4 = 0; k4 < OV; ++k4) {
            uint32_t w[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const uint4 d = mine[k4 * 4 + q];
                float worst = 0.f;
                w[q] = quant8_nibbles<InT>(d, qa, qb, worst);
                if (!fast || !(worst <= p.thr))  // (one test per vector: testing several together measured slower)
                    w[q] = repair8_nibbles<InT>(d, u.inv, u.zq, p.thr, p.lm1, fast, u.in_low, u.range, u.y);
                if (MODE == 2) w[q] = nibbles_add(w[q], p.qmin);
            }
            mine[k4] = make_uint4(w[0], w[1], w[2], w[3]);
        }
    } else if (PACK4) {
        const ExactQ eq = exact_consts(u, p.lm1, 0.f);
#pragma unroll
        for (int k4 = 0; k4 < OV; ++k4) {
            uint32_t w[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const uint4 d = mine[k4 * 4 + q];
                if (fast) {
                    w[q] = exact8_nibbles<InT>(d, eq);
                } else {
                    const uint2 idx = quant8_fix_idx<InT>(d, u, p.thr, p.lm1, true);
                    w[q] = idx_to_nibbles4(idx.x) | (idx_to_nibbles4(idx.y) << 16);
                }
                if (MODE == 2) w[q] = nibbles_add(w[q], p.qmin);
            }
            mine[k4] = make_uint4(w[0], w[1], w[2], w[3]);
        }
    } else {
        const float zpf = __fadd_rn(u.zq, float(p.qmin));  // K = zp: the low byte of mm is the code
        const PairQ qc = pair_consts(u.inv, zpf);
        const ExactQ eq = exact_consts(u, p.lm1, float(p.qmin));
#pragma unroll
        for (int k2 = 0; k2 < OV; ++k2) {
            uint2 c[2];
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                const uint4 d = mine[k2 * 2 + q];
                bool redo = !fast;
                if (EXACT) {
                    c[q] = exact8_bytes<InT, false>(d, eq, dup(0.f), nullptr);
                } else {
                    float worst = 0.f;
                    c[q] = quant8_bytes<InT, false>(d, qc, worst, nullptr);
                    redo |= !(worst <= p.thr);
                }
                if (redo) {
                    const uint2 idx = quant8_fix_idx<InT>(d, u, p.thr, p.lm1, !fast);
                    c[q] = make_uint2(idx_to_codes4(idx.x, p.qmin), idx_to_codes4(idx.y, p.qmin));
                }
            }
            mine[k2] = make_uint4(c[0].x, c[0].y, c[1].x, c[1].y);
        }
    }
    __syncwarp();
    // ---- copy-out: the chunk's codes are 32 * OV consecutive 16-byte vectors --------------------------------
    uint4* outv = reinterpret_cast<uint4*>(J.codes + (PACK4 ? (e0 >> 1) : e0));
#pragma unroll
    for (int it = 0; it < OV; ++it) {
        const int o = it * 32 + lane;
        const int gg = o / OV, k = o % OV;
        if (g0 + gg < J.total_groups) {
            const uint4 v = stage[gg * (V + 1) + k];
            st_global_v4(outv + o, v.x, v.y, v.z, v.w);
        }
    }
}

__device__ __forceinline__ void load_group_job(GroupJob& J, const RowQuantArgs* __restrict__ jobs, const LaunchParams& p, int64_t chunk,
                                               int G) {
    const int j = find_job(jobs, p.njobs, chunk);
    const RowQuantArgs& A = jobs[j];
    J.in = A.in;
    J.codes = static_cast<uint8_t*>(A.codes);
    J.o_scales = A.scales;
    J.o_zps = A.zps;
    J.o_f16 = A.scales_f16;
    J.o_u4 = A.zps_u4;
    J.o_deq = A.dequant;
    J.g_scales = A.given_scales;
    J.g_zps = A.given_zps;
    J.total_groups = A.rows * (A.cols / G);
    J.unit_begin = A.unit_begin;
    J.job_end = j + 1 < p.njobs ? jobs[j + 1].unit_begin : p.total_units;
}
template <typename InT, int G, int MODE>
__global__ void __launch_bounds__(256, 3) k_group(const RowQuantArgs* __restrict__ jobs, LaunchParams p, int* flags) {
    constexpr int V = G / 8;
    constexpr int kStageVecs = (V + 1) * 32;
    extern __shared__ uint4 smem_u4[];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int wpb = blockDim.x >> 5;
    uint4* stage = smem_u4 + wid * kStageVecs;
    const int64_t nwarps = int64_t(gridDim.x) * wpb;
    GroupJob J;
    J.job_end = 0;
    for (int64_t chunk = int64_t(blockIdx.x) * wpb + wid; chunk < p.total_units; chunk += nwarps) {
        if (chunk >= J.job_end) load_group_job(J, jobs, p, chunk, G);
        group_issue<InT, G>(stage, J, chunk, lane);
        cp_async_wait_all();
        __syncwarp();  // lanes read vectors copied by other lanes
        group_chunk<InT, G, MODE>(stage, J, chunk, p, lane, flags);
        __syncwarp();  // the stage is overwritten by the next chunk's copies
    }
}

// ======================================================================================================
// K_row: one unit per row, 16-byte aligned rows of a [rows, cols] matrix (per-output-channel quantization of
// linear weights), 2-byte input. A CTA of 256 threads is split into 256 / T independent row groups: the T
// threads of a group stage one row in shared memory and walk the rows of all jobs on their own, synchronising
// through the group's named barrier only. While one group sits in the scalar FP64 derivation of its row's
// scale, the other groups of the SM keep sweeping.
// The optional Dequantize copy in float16 is computed arithmetically: code - zp is already at hand as a float,
// one packed multiply by fl32(scale) and one packed conversion give two outputs. That product can differ from
// the reference's fl32(double(code - zp) * scale) by one ulp, which changes the float16 only next to a float16
// rounding boundary, in the subnormal range or at the overflow clamp: per row, every code whose product lies
// there is compared with the exact FP64 formula, and a row with a differing code falls back to a table of the L
// exact outputs indexed by the code byte (also used for float32 and bfloat16 copies).
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
    extern __shared__ uint4 smem_all[];
    struct GroupShared {
        float mn[T / 32], mx[T / 32];
        UnitQ u;
        double scale;
        long long zp;
        int fast;      // the packed exact sequence covers this row (unit_exact_ok)
        int need_lut;  // the arithmetic float16 copy is not exact for this row
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
    uint4* const smem_u4 = smem_all + size_t(grp) * size_t(stage_vecs);
    const int bar_id = 1 + grp;
    const int qmin = p.qmin;
    const bool arith_dt = DQ == 1 && p.dequant_dt == VF_DT_F16;
    if (tid == 0) gs.need_lut = 0;  // made visible by the first barrier of the row loop

    int j = 0;
    int64_t job_end = 0;
    const InT* in = nullptr;
    uint8_t* o_codes = nullptr;
    double* o_scales = nullptr;
    int64_t* o_zps = nullptr;
    uint16_t* o_f16 = nullptr;
    uint8_t* o_deq = nullptr;
    const double* g_scales = nullptr;
    const int64_t* g_zps = nullptr;
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
            g_scales = J.given_scales;
            g_zps = J.given_zps;
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
        if (mm.saw_nan()) set_flag(flags, VF_FLAG_NAN);
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
                if (p.given) {
                    scale = g_scales[r];
                    zp = g_zps[r];
                    unit_consts(scale, zp, p, u);
                } else {
                    derive_unit(mn, mx, p, scale, zp, u, flags);
                    if (o_scales) o_scales[r] = scale;
                    if (o_zps) o_zps[r] = zp;
                    if (o_f16) o_f16[r] = f32_to_f16_bits(__double2float_rn(scale));
                }
                gs.u = u;
                gs.scale = scale;
                gs.zp = zp;
                gs.fast = unit_exact_ok(u, mn, mx, p) ? 1 : 0;
            }
        }
        group_sync<T>(bar_id);
        const UnitQ u = gs.u;
        const bool fast = gs.fast != 0;
        const float sh = __double2float_rn(gs.scale);
        const int zpi = int(gs.zp);
        bool lut = DQ != 0 && !arith_dt;
        if (arith_dt) {
            // which codes could the arithmetic copy get wrong? (see the kernel's header)
            const double scale = gs.scale;
            const long long zp = gs.zp;
            for (int n = tid; n <= p.lm1; n += THREADS) {
                const int code = n + qmin;
                const float prod = __fmul_rn(float(code - zpi), sh);
                const uint32_t a = __float_as_uint(prod) & 0x7FFFFFFFu, m13 = a & 0x1FFFu;
                const bool safe = code == zpi || (a >= 0x38800000u && a < 0x477FE000u && (m13 < 0x0FFFu || m13 > 0x1001u));
                if (!safe) {
                    const uint16_t exact = f32_to_f16_clamped_bits(dequantize_exact(code, scale, zp));
                    if (exact != __half_as_ushort(__float2half_rn(prod))) atomicOr(&gs.need_lut, 1);
                }
            }
            group_sync<T>(bar_id);
            lut = gs.need_lut != 0;
        }
        if (lut) {
            const double scale = gs.scale;
            const long long zp = gs.zp;
            for (int n = tid; n <= p.lm1; n += THREADS) {
                const int code = n + qmin;
                const float f = dequantize_exact(code, scale, zp);
                if (DQ == 2) s_lut[code & 0xFF] = __float_as_uint(f);
                else reinterpret_cast<uint16_t*>(s_lut)[code & 0xFF] = p.dequant_dt == VF_DT_F16 ? f32_to_f16_clamped_bits(f) : f32_to_bf16_bits(f);
            }
            group_sync<T>(bar_id);
        }
        uint8_t* const codes_row = o_codes ? o_codes + r * cols : nullptr;
        uint8_t* const deq_row = DQ == 0 ? nullptr : o_deq + r * cols * (DQ == 1 ? 2 : 4);
        if (fast) {
            // K = qmin: the low byte of the result is the code in two's complement; minus (magic + zp): code - zp
            const ExactQ eq = exact_consts(u, p.lm1, float(qmin));
            const float2 nzpk = dup(-__fadd_rn(kMagic, float(zpi)));
            const float2 sh2 = dup(sh);
            constexpr int kDeqBytes = DQ == 2 ? 32 : 16;  // dequantized bytes per vector
            auto one = [&](const uint4& d, uint8_t* cdst, uint8_t* ddst) {
                float2 s[4];
                const uint2 c = exact8_bytes<InT, DQ == 1>(d, eq, nzpk, s);
                if (codes_row) st_global_v2(cdst, c.x, c.y);
                if (DQ == 1 && !lut) {
                    uint32_t h[4];
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const float2 v = __fmul2_rn(s[k], sh2);
                        h[k] = as_u32(__floats2half2_rn(v.x, v.y));
                    }
                    st_global_v4(ddst, h[0], h[1], h[2], h[3]);
                } else if (DQ != 0) {
                    // table entry of byte k of w: shift the byte to the entry's offset, mask it and OR the table's
                    // (size-aligned) shared-memory address in, all in one logic instruction after the shift
                    constexpr int kSh = DQ == 1 ? 1 : 2;
                    constexpr uint32_t kMask = DQ == 1 ? 0x1FEu : 0x3FCu;
                    const uint32_t w0 = c.x, w1 = c.y;
                    uint32_t q[8];
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const uint32_t o0 = ((k == 0 ? (w0 << kSh) : (w0 >> (8 * k - kSh))) & kMask) | lut_sh;
                        const uint32_t o1 = ((k == 0 ? (w1 << kSh) : (w1 >> (8 * k - kSh))) & kMask) | lut_sh;
                        q[k] = DQ == 1 ? lds_u16(o0) : lds_u32(o0);
                        q[4 + k] = DQ == 1 ? lds_u16(o1) : lds_u32(o1);
                    }
                    if (DQ == 2) {
                        st_global_v4(ddst, q[0], q[1], q[2], q[3]);
                        st_global_v4(ddst + 16, q[4], q[5], q[6], q[7]);
                    } else {
                        st_global_v4(ddst, __byte_perm(q[0], q[1], 0x5410), __byte_perm(q[2], q[3], 0x5410),
                                     __byte_perm(q[4], q[5], 0x5410), __byte_perm(q[6], q[7], 0x5410));
                    }
                }
            };
            // The sweep handles kBatch vectors per step: all shared-memory loads of the step are issued first, then
            // the independent arithmetic chains and the stores. Pointers advance by constants; the ragged end of the
            // row is a loop of its own.
            constexpr int kBatch = 4;
            const int full = nvec / (kBatch * THREADS);
            const uint4* sp = smem_u4 + tid;
            uint8_t* cp = codes_row + size_t(tid) * 8;
            uint8_t* dp = deq_row + size_t(tid) * kDeqBytes;
            for (int it = 0; it < full; ++it) {
                uint4 d[kBatch];
#pragma unroll
                for (int b = 0; b < kBatch; ++b) d[b] = sp[b * THREADS];
#pragma unroll
                for (int b = 0; b < kBatch; ++b) one(d[b], cp + b * THREADS * 8, dp + b * THREADS * kDeqBytes);
                sp += kBatch * THREADS;
                cp += kBatch * THREADS * 8;
                dp += kBatch * THREADS * kDeqBytes;
            }
            for (int i = full * kBatch * THREADS + tid; i < nvec; i += THREADS)
                one(smem_u4[i], codes_row + size_t(i) * 8, deq_row + size_t(i) * kDeqBytes);
        } else {
            // a row the packed sequence does not cover (parameters that do not contain the data, a range at the end
            // of the exponent range): the scalar sequence with its clamp for every element
            const uint16_t* row16 = reinterpret_cast<const uint16_t*>(smem_u4);
            const double scale = gs.scale;
            const long long zp = gs.zp;
            for (int idx = tid; idx < int(cols); idx += THREADS) {
                const float x = P2<InT>::lo(uint32_t(row16[idx]));
                const int code = quant_index_exact(x, u.in_low, u.range, p.lm1) + qmin;
                if (codes_row) codes_row[idx] = uint8_t(code);
                if (DQ == 1) reinterpret_cast<uint16_t*>(deq_row)[idx] = dequant16(code, zp, scale, p.dequant_dt);
                if (DQ == 2) reinterpret_cast<float*>(deq_row)[idx] = dequantize_exact(code, scale, zp);
            }
        }
        group_sync<T>(bar_id);  // the stage, u and the table are rewritten by the next row
        if (tid == 0) gs.need_lut = 0;
    }
}

// ======================================================================================================
// K_conv: one unit per output channel of a convolution weight, any row length / alignment, any of
// f32 / f16 / bf16. One warp per row, looping over the rows of all jobs. The quantized row is staged in
// shared memory at its OYXI position (ic padded to ic_pad) and written out with coalesced 32-bit stores; rows
// beyond `rows` (channel padding) are zero. Two sweeps over the row: the second one hits L1/L2.
// ======================================================================================================
template <int IN_DT>  // the input type as a constant (the element load then has no type switch), 0: `in_dt_arg`
__global__ void __launch_bounds__(256) k_conv(const RowQuantArgs* __restrict__ jobs, LaunchParams p, int in_dt_arg,
                                              int stage_bytes, int* flags) {
    const int in_dt = IN_DT ? IN_DT : in_dt_arg;
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
        const int cols = int(J.cols);  // (rows of this kernel are at most 8192 elements)
        float mn = 0.f, mx = 0.f;
        bool nan = false;
        for (int i0 = lane; i0 < cols; i0 += 128) {  // four loads on their way before the first is used
            float x[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) x[k] = i0 + 32 * k < cols ? load_as_f32(J.in, in_dt, base + i0 + 32 * k, nullptr) : 0.f;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                nan |= x[k] != x[k];
                mn = fminf(mn, x[k]);
                mx = fmaxf(mx, x[k]);
            }
        }
        if (nan) set_flag(flags, VF_FLAG_NAN);  // undefined in the reference: reported
        mn = warp_min(mn);
        mx = warp_max(mx);
        double scale = 0.0;
        long long zp = 0;
        UnitQ u;
        u.inv = u.zq = u.in_low = u.range = u.y = 0.f;
        int fast = 1;
        if (lane == 0) {
            if (p.given) {
                scale = J.given_scales[r];
                zp = J.given_zps[r];
                unit_consts(scale, zp, p, u);
                fast = unit_fits(u, mn, mx, zp, p) ? 1 : 0;
            } else {
                derive_unit(mn, mx, p, scale, zp, u, flags);
                fast = (u.range >= 7.8886091e-31f && u.range <= 1.2676506e30f) ? 1 : 0;
                if (J.scales) J.scales[r] = scale;
                if (J.zps) J.zps[r] = zp;
                if (J.scales_f16) J.scales_f16[r] = f32_to_f16_bits(__double2float_rn(scale));
            }
        }
        u.inv = __shfl_sync(0xffffffffu, u.inv, 0);
        u.zq = __shfl_sync(0xffffffffu, u.zq, 0);
        u.in_low = __shfl_sync(0xffffffffu, u.in_low, 0);
        u.range = __shfl_sync(0xffffffffu, u.range, 0);
        fast = __shfl_sync(0xffffffffu, fast, 0);
        if (ic_pad != ic) {
            for (int64_t b = lane; b < out_row_bytes; b += 32) stage[b] = 0;
            __syncwarp();
        }
        const float cm = __fadd_rn(kMagic, u.zq);
        // input index i = icIdx * khw + s  ->  output index s * ic_pad + icIdx; a lane's i advances by 32, so its
        // (icIdx, s) advance by (32 / khw, 32 % khw) with a carry instead of being divided out per element
        const int khw32 = int(khw), icp32 = int(ic_pad);
        const int dq = 32 / khw32, dr = 32 % khw32;
        int ici = lane / khw32, sp = lane % khw32;
        for (int i0 = lane; i0 < cols; i0 += 128) {
            float xs[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) xs[k] = i0 + 32 * k < cols ? load_as_f32(J.in, in_dt, base + i0 + 32 * k, nullptr) : 0.f;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                if (i0 + 32 * k >= cols) break;
                const float x = xs[k];
                const float m = __fmaf_rn(x, u.inv, cm);
                int n = __float_as_int(m) - kMagicBits;
                const float resid = __fmaf_rn(x, -u.inv, __fsub_rn(m, cm));
                if (!fast || !(fabsf(resid) <= p.thr)) n = quant_index_exact(x, u.in_low, u.range, p.lm1);
                n = min(max(n, 0), p.lm1);
                stage[sp * icp32 + ici] = uint8_t(n + p.qmin);
                ici += dq;
                sp += dr;
                if (sp >= khw32) {
                    sp -= khw32;
                    ++ici;
                }
            }
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
// convolution with IC % 8 == 0). One warp per output channel, and nothing of the input is staged: the lanes read
// the row with 16-byte loads into registers, min/max run on packed pairs, and the second pass quantizes the
// registers (rows longer than 1024 elements read all but their last 1024 again, from the caches). A 1x1 kernel's
// codes go straight to the output row; otherwise they are collected in the warp's shared-memory stage as a dense
// byte row in input order and copied out transposed OIYX->OYXI: the (tap, channel block) pairs of the output row
// are dealt out over the lanes, every lane gathers the codes of 16 (or 4) consecutive input channels of one tap
// and stores them as one vector. Without an input stage a CTA needs one byte of shared memory per element of its
// eight rows, so four CTAs fit an SM whatever the row length.
// ======================================================================================================
template <int W>  // bytes per lane and store: 16 or 4; `lanes` lanes (sub = 0 .. lanes - 1) share the row
__device__ __forceinline__ void convv_copy_out(const uint8_t* cb, uint8_t* out, int khw, int ic, int ic_pad, int sub, int lanes) {
    const int blocks = ic_pad / W;           // channel blocks per tap
    const int total = khw * blocks;          // stores of the row
    const int qs = lanes / blocks, rs = lanes % blocks;
    int s = sub / blocks, cblk = sub % blocks;
    for (int o = sub; o < total; o += lanes) {
        const int c0 = cblk * W;
        uint32_t w[W / 4];
#pragma unroll
        for (int k = 0; k < W / 4; ++k) {
            uint32_t word = 0;
            const int c = c0 + 4 * k;
            const uint8_t* src = cb + c * khw + s;  // input index = channel * khw + tap
            if (c + 3 < ic) {
                word = uint32_t(src[0]) | (uint32_t(src[khw]) << 8) | (uint32_t(src[2 * khw]) << 16) | (uint32_t(src[3 * khw]) << 24);
            } else if (c < ic) {  // the last channels of a count that is no multiple of 4; the rest is padding
                word = uint32_t(src[0]);
                if (c + 1 < ic) word |= uint32_t(src[khw]) << 8;
                if (c + 2 < ic) word |= uint32_t(src[2 * khw]) << 16;
            }
            w[k] = word;
        }
        uint8_t* dst = out + size_t(s) * ic_pad + c0;
        if (W == 16) st_global_v4(dst, w[0], w[1], w[2], w[3]);
        else *reinterpret_cast<uint32_t*>(dst) = w[0];
        s += qs;
        cblk += rs;
        if (cblk >= blocks) {
            cblk -= blocks;
            ++s;
        }
    }
}

// A row the packed sequence does not cover (its range or its extreme indices are out of bounds): every element
// with the scalar sequence, read again from global memory. Rare, and kept out of line.
// A row of 2-byte elements read as 16-byte vectors of eight; rows that are not whole aligned vectors (the stem of
// a network: 3 x 7 x 7 elements) are assembled from 2-byte loads, the missing elements of the last vector as zeros.
struct ConvRow {
    const uint16_t* p;
    int cols;
    bool vec_ok;
    __device__ __forceinline__ uint4 vec(int v) const {
        if (vec_ok) return __ldg(reinterpret_cast<const uint4*>(p) + v);
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int e = 8 * v + 2 * i;
            const uint32_t lo = e < cols ? uint32_t(__ldg(p + e)) : 0u, hi = e + 1 < cols ? uint32_t(__ldg(p + e + 1)) : 0u;
            w[i] = lo | (hi << 16);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
};
template <typename InT>
__device__ __noinline__ void convv_row_scalar(ConvRow src, int nvec, int sub, int lanes, UnitQ u, float thr, int lm1, int qmin, uint2* dst) {
    for (int v = sub; v < nvec; v += lanes) {
        const uint2 idx = quant8_fix_idx<InT>(src.vec(v), u, thr, lm1, true);
        dst[v] = make_uint2(idx_to_codes4(idx.x, qmin), idx_to_codes4(idx.y, qmin));
    }
}

__device__ __forceinline__ void prefetch_l2(const void* p) {
    asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}

// The fields of a job K_convv needs, read once per tensor a warp works on
struct ConvJob {
    const RowQuantArgs* args;      // the side outputs and supplied parameters are read where they are used
    const void* in;
    uint8_t* codes;
    int rows, rows_pad, cols, row_vecs;  // row_vecs: 16-byte vectors per input row, the last one possibly ragged
    int vec_ok;                    // rows are whole, 16-byte aligned vectors
    int khw, ic, ic_pad;           // khw == 0: the codes are the output row as they are
    int out_bytes;                 // bytes of an output row
    int lpr;
    int64_t unit_begin, unit_end, work_begin;
    int unit_cost;
};
__device__ __forceinline__ void load_conv_job(const RowQuantArgs* __restrict__ jobs, int j, const LaunchParams& p, ConvJob& J) {
    const RowQuantArgs& A = jobs[j];
    J.args = &A;
    J.in = A.in;
    J.codes = static_cast<uint8_t*>(A.codes);
    J.rows = int(A.rows);
    J.rows_pad = int(A.rows_pad);
    J.cols = int(A.cols);
    J.row_vecs = int((A.cols + 7) >> 3);
    J.vec_ok = (A.cols & 7) == 0 && (reinterpret_cast<uintptr_t>(A.in) & 15) == 0;
    J.khw = int(A.khw);
    J.ic = A.khw > 0 ? int(A.ic) : int(A.cols);
    J.ic_pad = A.khw > 0 ? int(A.ic_pad) : int(A.cols);
    J.out_bytes = (A.khw > 0 ? int(A.khw) : 1) * J.ic_pad;
    J.lpr = A.lanes_per_row;
    J.unit_begin = A.unit_begin;
    J.unit_end = j + 1 < p.njobs ? jobs[j + 1].unit_begin : p.total_units;
    J.work_begin = A.work_begin;
    J.unit_cost = A.unit_cost;
}

__device__ __forceinline__ void convv_prefetch_unit(const ConvJob& J, int64_t u, int lane) {
    const int rows_per_unit = 32 / J.lpr;
    const int64_t r0 = u * rows_per_unit;
    const int rows_there = min(rows_per_unit, J.rows - int(r0));
    if (rows_there <= 0) return;
    const char* base = static_cast<const char*>(J.in) + r0 * int64_t(J.cols) * 2;
    const int64_t bytes = int64_t(rows_there) * J.cols * 2;
    for (int64_t o = int64_t(lane) * 128; o < bytes; o += 32 * 128) prefetch_l2(base + o);
}

// One unit of K_convv: 32 / LPR consecutive output channels of one tensor, LPR lanes each. Every group runs the
// same instruction stream (same tensor, same row length); a group without a row (past the tensor's last channel)
// loads nothing and stores nothing but takes part in the shuffles.
template <typename InT>
__device__ __forceinline__ void convv_unit(const ConvJob& J, int64_t unit_in_job, const LaunchParams& p, uint4* stage, int stage_vecs,
                                           int lane, int* flags) {
    constexpr int kB = 4;             // vectors per lane and batch
    const int LPR = J.lpr;            // 8, 16 or 32 (one code path: the tensor's value is uniform over the warp)
    const int lpr_shift = LPR == 8 ? 3 : (LPR == 16 ? 4 : 5);
    const int RPW = 32 >> lpr_shift;  // rows per warp
    const int sub = lane & (LPR - 1), grp = lane >> lpr_shift;
    const int r = int(unit_in_job) * RPW + grp;
    const int out_bytes = J.out_bytes;
    uint8_t* out = J.codes + int64_t(r) * out_bytes;
    const bool live = r < J.rows;
    if (!live && r < J.rows_pad) {  // padded output channel
        uint32_t* o32 = reinterpret_cast<uint32_t*>(out);
        for (int w = sub; w < (out_bytes >> 2); w += LPR) o32[w] = 0u;
    }
    const int row_vecs = J.row_vecs;
    const int nvec = live ? row_vecs : 0;
    const int nb = (row_vecs + kB * LPR - 1) / (kB * LPR);
    const ConvRow src{static_cast<const uint16_t*>(J.in) + int64_t(live ? r : 0) * J.cols, J.cols, J.vec_ok != 0};
    // first pass: the range. The vectors of the last batch stay in registers for the second pass (rows of up to
    // 32 LPR elements are read once); earlier batches are read again, from the caches.
    uint4 d[kB];
    MinMax2<InT> mm;
    for (int b = 0; b < nb; ++b) {
#pragma unroll
        for (int k = 0; k < kB; ++k) {
            const int v = (b * kB + k) * LPR + sub;
            d[k] = make_uint4(0u, 0u, 0u, 0u);  // zeros do not move a range that contains zero
            if ((b * kB + k) * LPR < row_vecs && v < nvec) d[k] = src.vec(v);
        }
#pragma unroll
        for (int k = 0; k < kB; ++k) mm.add(d[k]);
    }
    if (mm.saw_nan()) set_flag(flags, VF_FLAG_NAN);
    float mn = mm.min_f(), mx = mm.max_f();
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        if (o < LPR) {
            mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        }
    }
    // every lane of the group evaluates the row's parameters (same inputs, same results): nothing to broadcast
    UnitQ u;
    {
        double scale;
        long long zp;
        if (p.given) {
            scale = live ? J.args->given_scales[r] : 1.0;
            zp = live ? J.args->given_zps[r] : 0;
            unit_consts(scale, zp, p, u);
        } else {
            derive_unit(mn, mx, p, scale, zp, u, flags);
            if (sub == 0 && live) {
                const RowQuantArgs& A = *J.args;
                if (A.scales) A.scales[r] = scale;
                if (A.zps) A.zps[r] = zp;
                if (A.scales_f16) A.scales_f16[r] = f32_to_f16_bits(__double2float_rn(scale));
            }
        }
    }
    const bool fast = unit_exact_ok(u, mn, mx, p);

    // second pass, last batch first. The codes of a 1x1 kernel are the output row as they are; otherwise they
    // are collected in the group's part of the stage for the transposed copy-out.
    const bool direct = J.khw <= 0 && J.vec_ok && (reinterpret_cast<uintptr_t>(J.codes) & 7) == 0;
    uint4* my_stage = stage + grp * (stage_vecs >> (5 - lpr_shift));
    uint2* dst2 = reinterpret_cast<uint2*>(direct ? static_cast<void*>(out) : static_cast<void*>(my_stage));
    const ExactQ eq = exact_consts(u, p.lm1, float(p.qmin));  // K = qmin: the low byte is the code
    for (int b = nb - 1; b >= 0; --b) {
        if (b != nb - 1) {
#pragma unroll
            for (int k = 0; k < kB; ++k) d[k] = src.vec((b * kB + k) * LPR + sub);  // every batch but the last is full
        }
#pragma unroll
        for (int k = 0; k < kB; ++k) {
            if ((b * kB + k) * LPR >= row_vecs) break;  // uniform over the warp
            const int v = (b * kB + k) * LPR + sub;
            if (v < nvec && fast) dst2[v] = exact8_bytes<InT, false>(d[k], eq, dup(0.f), nullptr);
        }
    }
    if (!fast) convv_row_scalar<InT>(src, nvec, sub, LPR, u, p.thr, p.lm1, p.qmin, dst2);
    if (direct) return;  // uniform over the warp: a property of the tensor
    __syncwarp();
    if (live) {
        const bool out16 = (reinterpret_cast<uintptr_t>(J.codes) & 15) == 0 && (out_bytes & 15) == 0;
        if (J.khw <= 0) {
            const uint32_t* c32 = reinterpret_cast<const uint32_t*>(my_stage);
            uint32_t* o32 = reinterpret_cast<uint32_t*>(out);
            for (int w = sub; w < (out_bytes >> 2); w += LPR) o32[w] = c32[w];
        } else if (out16 && (J.ic_pad & 15) == 0) {
            convv_copy_out<16>(reinterpret_cast<const uint8_t*>(my_stage), out, J.khw, J.ic, J.ic_pad, sub, LPR);
        } else {
            convv_copy_out<4>(reinterpret_cast<const uint8_t*>(my_stage), out, J.khw, J.ic, J.ic_pad, sub, LPR);
        }
    }
    __syncwarp();  // the stage is rewritten by the next unit
}

// lanes per row of K_convv: the fewest (8, 16 or 32) that hold the row in one batch of four vectors per lane
inline int convv_lanes_per_row(int64_t cols) {
    return cols <= 256 ? 8 : (cols <= 512 ? 16 : 32);
}
// Relative cost of one unit, in warp instructions / 8: what does not depend on the row length plus the batches
inline int convv_unit_cost(int64_t cols, int64_t khw, int lanes_per_row) {
    const int64_t steps = (cols / 8 + lanes_per_row - 1) / lanes_per_row;  // vectors per lane
    return int(30 + steps * (khw > 0 ? 12 : 8));
}

// The units of all tensors form one list, each with a cost, and the total is cut into kConvvChunksPerWarp equal
// chunks per warp; a chunk's units are those whose cumulative cost starts inside it. A warp starts with the chunk
// of its own number and then takes the next free one from a counter (a zeroed word behind the job table), so that
// the warps end together although the cost is only an estimate. A chunk's units are consecutive: the job is
// searched once per chunk, in a copy of the jobs' first costs in shared memory, and a tensor's fields are read
// once per tensor and chunk.
constexpr int kConvvChunksPerWarp = 2;  // (1: 54.4 us, 2: 51.7, 3: 52.4, 5: 55.5, 8: 61.2 for the 54 ResNet-50 tensors: a chunk costs its search)
constexpr int kConvvStagedJobs = 512;

template <typename InT>
__global__ void __launch_bounds__(256, 4) k_convv(const RowQuantArgs* __restrict__ jobs, LaunchParams p, int stage_vecs,
                                                  unsigned int* next_chunk, int* flags) {
    extern __shared__ uint4 smem_u4[];
    __shared__ int64_t s_work_begin[kConvvStagedJobs];
    const bool staged = p.njobs <= kConvvStagedJobs;
    if (staged) {
        for (int i = threadIdx.x; i < p.njobs; i += blockDim.x) s_work_begin[i] = jobs[i].work_begin;
        __syncthreads();
    }
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    uint4* stage = smem_u4 + size_t(wid) * size_t(stage_vecs);  // codes, one byte per element in input order
    const int64_t nwarps = int64_t(gridDim.x) * (blockDim.x >> 5);
    const int64_t nchunks = nwarps * kConvvChunksPerWarp;
    const int64_t cw = p.total_work / nchunks, cr = p.total_work % nchunks;
    // warps of one CTA start far apart (chunk = wid * gridDim + blockIdx): a CTA's rows differ in length
    int64_t chunk = int64_t(wid) * gridDim.x + blockIdx.x;
    int j = -1;
    ConvJob J;
    for (;;) {
        const int64_t W0 = cw * chunk + min(chunk, cr), W1 = cw * (chunk + 1) + min(chunk + 1, cr);
        if (W0 < W1) {
            int lo = 0, hi = p.njobs - 1;
            while (lo < hi) {  // last job whose work_begin <= W0
                const int mid = (lo + hi + 1) >> 1;
                if ((staged ? s_work_begin[mid] : jobs[mid].work_begin) <= W0) lo = mid;
                else hi = mid - 1;
            }
            if (lo != j) load_conv_job(jobs, j = lo, p, J);
            int64_t unit = J.unit_begin + (W0 - J.work_begin + J.unit_cost - 1) / J.unit_cost;
            bool first = true;
            for (;;) {
                while (unit >= J.unit_end && j + 1 < p.njobs) load_conv_job(jobs, ++j, p, J);
                if (unit >= J.unit_end) break;
                const int64_t u = unit - J.unit_begin;
                if (J.work_begin + u * J.unit_cost >= W1) break;
                // the rows of the chunk's next unit are on their way into the L2 while this one is worked on (the
                // first unit's own rows, past the first batch, as well)
                if (first) convv_prefetch_unit(J, u, lane);
                first = false;
                if (unit + 1 < J.unit_end) convv_prefetch_unit(J, u + 1, lane);
                convv_unit<InT>(J, u, p, stage, stage_vecs, lane, flags);
                ++unit;
            }
        }
        unsigned int got = 0;
        if (lane == 0) got = atomicAdd(next_chunk, 1u);
        chunk = nwarps + int64_t(__shfl_sync(0xffffffffu, got, 0));
        if (chunk >= nchunks) return;
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

template <typename InT, int G, int MODE>
void launch_group_s(vf_ctx* ctx, const RowQuantArgs* d_jobs, const LaunchParams& p) {
    const size_t smem = size_t(8) * (G / 8 + 1) * 32 * 16;  // 8 warps x 32 groups x (G/8 + 1 padding) vectors
    // persistent grid: three CTAs per SM (launch bounds), every warp strides over the chunk list
    const int64_t want = (p.total_units + 7) / 8;
    const int grid = int(std::min<int64_t>(want, int64_t(ctx->sm_count) * 3));
    set_smem(k_group<InT, G, MODE>, smem);
    k_group<InT, G, MODE><<<grid, 256, smem, ctx->stream>>>(d_jobs, p, ctx->d_flags);
    post_launch(ctx);
}

template <typename InT, int G>
void launch_group_g(vf_ctx* ctx, const RowQuantArgs* d_jobs, const LaunchParams& p, bool pack4) {
    if (!pack4) launch_group_s<InT, G, 0>(ctx, d_jobs, p);
    else if (p.qmin == 0) launch_group_s<InT, G, 1>(ctx, d_jobs, p);
    else launch_group_s<InT, G, 2>(ctx, d_jobs, p);
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
    const int grid = int(std::min<int64_t>(ctas, int64_t(ctx->sm_count) * int64_t(per_sm)));
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
    const bool row_ok = two_byte && aligned16 && a.khw == 0 && a.rows_pad == a.rows && !a.pack4 && !a.zps_u4 && a.cols % 8 == 0 &&
                        a.cols >= 1024 && a.cols <= 96 * 1024 && reinterpret_cast<uintptr_t>(a.codes) % 8 == 0 &&
                        (!a.dequant || reinterpret_cast<uintptr_t>(a.dequant) % 16 == 0);
    bool convv_ok = false, conv_ok = false;
    if (!a.pack4 && !a.dequant && !a.zps_u4 && a.codes) {
        const int64_t out_row = a.khw > 0 ? a.khw * a.ic_pad : a.cols;
        const int64_t ic_pad = a.khw > 0 ? a.ic_pad : a.cols;
        // rows that are not whole aligned vectors are taken when they are copied out transposed (the stem)
        const bool vec_rows = aligned16 && a.cols % 8 == 0;
        convv_ok = two_byte && (vec_rows || a.khw > 0) && a.cols <= 4608 && out_row <= 4608 && ic_pad % 4 == 0 &&
                   reinterpret_cast<uintptr_t>(a.codes) % 4 == 0 && reinterpret_cast<uintptr_t>(a.in) % 2 == 0;
        // the scalar kernel is for the short rows of convolutions (fp32 input, odd sizes): a warp walks a row element by
        // element, so long rows are left to the general kernels, which read them as vectors
        conv_ok = out_row <= 8192 && a.cols <= 8192;
    }
    // a convolution weight (it came with an OIYX -> OYXI reorder: ic is set) stays with the other convolutions of its
    // network in one launch, also where its 1x1 rows would suit the row kernel
    if (convv_ok && a.ic > 0) return 4;
    if (row_ok) return 2;
    if (convv_ok) return 4;
    if (conv_ok) return 3;
    return 0;
}

// Launches every job of `jobs` (all of kind `kind` and sharing the uniform parameters of jobs[0]) with one
// kernel. The job table is copied to device memory first.
void launch_rowquant_batch(vf_ctx* ctx, int kind, std::vector<RowQuantArgs>& jobs) {
    if (jobs.empty()) return;
    const RowQuantArgs a0 = jobs[0];
    LaunchParams p{};
    p.range_mode = a0.range_mode;
    p.qmin = int(a0.qmin);
    p.qmax = int(a0.qmax);
    p.lm1 = int(a0.qmax - a0.qmin);
    p.dequant_dt = a0.dequant_dt;
    p.njobs = int(jobs.size());
    p.given = a0.given_scales != nullptr;
    p.thr = 0.5f - kGuardPerLevel * float(p.lm1 + 1);
    p.den = double(p.lm1);
    p.inv_den = 1.0 / p.den;
    int64_t units = 0, max_cols = 0, max_out_row = 0;
    for (auto& a : jobs) {
        a.unit_begin = units;
        if (kind == 1) units += (a.rows * (a.cols / a.group) + 31) / 32;
        else if (kind == 2) units += a.rows;
        else if (kind == 4) {
            a.lanes_per_row = convv_lanes_per_row(a.cols);
            const int64_t rpw = 32 / a.lanes_per_row;
            const int64_t n_units = (a.rows_pad + rpw - 1) / rpw;
            a.unit_cost = convv_unit_cost(a.cols, a.khw, a.lanes_per_row);
            a.work_begin = p.total_work;
            p.total_work += n_units * a.unit_cost;
            units += n_units;
        } else units += a.rows_pad;
        max_cols = std::max(max_cols, a.cols);
        max_out_row = std::max(max_out_row, a.khw > 0 ? a.khw * a.ic_pad : a.cols);
    }
    p.total_units = units;
    if (kind == 4) jobs.push_back(RowQuantArgs{});  // a zeroed entry behind the table: K_convv's chunk counter
    DBuf table;
    const RowQuantArgs* d_jobs =
            static_cast<const RowQuantArgs*>(upload_table(ctx, jobs.data(), jobs.size() * sizeof(RowQuantArgs), table));
    if (kind == 4) jobs.pop_back();

    if (kind == 1) {
        if (a0.in_dt == VF_DT_F16) launch_group_t<__half>(ctx, d_jobs, p, a0.group, a0.pack4 != 0);
        else launch_group_t<__nv_bfloat16>(ctx, d_jobs, p, a0.group, a0.pack4 != 0);
    } else if (kind == 2) {
        const int dq = !a0.dequant ? 0 : (a0.dequant_dt == VF_DT_F32 ? 2 : 1);
        if (a0.in_dt == VF_DT_F16) launch_row_t<__half>(ctx, d_jobs, p, max_cols, dq);
        else launch_row_t<__nv_bfloat16>(ctx, d_jobs, p, max_cols, dq);
    } else if (kind == 4) {
        // the stage holds codes only, and only rows that are copied out transposed (or to a misaligned buffer) use it:
        // the rows of a warp side by side, each in a 16-byte multiple
        int64_t stage_vecs64 = 4;
        for (auto& a : jobs)
            if (a.khw > 0 || (reinterpret_cast<uintptr_t>(a.codes) & 7) != 0)
                stage_vecs64 = std::max(stage_vecs64, ((a.cols + 15) / 16) * (32 / a.lanes_per_row));
        const int stage_vecs = int(stage_vecs64);
        const size_t smem = size_t(8) * size_t(stage_vecs) * 16;
        const size_t per_sm = std::max<size_t>(1, std::min<size_t>(4, (220 * 1024) / (smem + 1024)));
        const int64_t blocks = (units + 7) / 8;
        const int grid = int(std::min<int64_t>(blocks, int64_t(ctx->sm_count) * int64_t(per_sm)));
        unsigned int* next_chunk = reinterpret_cast<unsigned int*>(const_cast<RowQuantArgs*>(d_jobs + p.njobs));
        if (a0.in_dt == VF_DT_F16) {
            set_smem(k_convv<__half>, smem);
            k_convv<__half><<<grid, 256, smem, ctx->stream>>>(d_jobs, p, stage_vecs, next_chunk, ctx->d_flags);
        } else {
            set_smem(k_convv<__nv_bfloat16>, smem);
            k_convv<__nv_bfloat16><<<grid, 256, smem, ctx->stream>>>(d_jobs, p, stage_vecs, next_chunk, ctx->d_flags);
        }
        post_launch(ctx);
    } else if (kind == 3) {
        const int stage_bytes = int((max_out_row + 15) & ~int64_t(15));
        const size_t smem = size_t(stage_bytes) * 8;
        const int64_t blocks = (units + 7) / 8;
        const int grid = int(std::min<int64_t>(blocks, int64_t(ctx->sm_count) * 8));
        auto go = [&](auto kernel) {
            set_smem(kernel, std::max<size_t>(smem, 16));
            kernel<<<grid, 256, smem, ctx->stream>>>(d_jobs, p, a0.in_dt, stage_bytes, ctx->d_flags);
        };
        if (a0.in_dt == VF_DT_F32) go(k_conv<VF_DT_F32>);
        else if (a0.in_dt == VF_DT_F16) go(k_conv<VF_DT_F16>);
        else if (a0.in_dt == VF_DT_BF16) go(k_conv<VF_DT_BF16>);
        else go(k_conv<0>);
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
           (a.dequant != nullptr) == (b.dequant != nullptr) && long_a == long_b &&
           (a.given_scales != nullptr) == (b.given_scales != nullptr);
}

}  // namespace vf
