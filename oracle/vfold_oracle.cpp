// CPU oracle for the constant-folding path — TEST INFRASTRUCTURE ONLY (see vfold_oracle.h).
//
// Every function restates one piece of the reference compiler and cites it. Paths are relative to the
// reference project root; CD = src/vpux_compiler/src/dialect/const, VC = src/vpux_compiler.
// Build: g++ -std=c++17 -O2 -ffp-contract=off -fno-fast-math (no -march): the reference is built with the
// compiler's default x86-64 flags, i.e. scalar SSE2 IEEE arithmetic without FMA contraction.

#include "vfold_oracle.h"

#include <algorithm>
#include <cfloat>
#include <climits>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <functional>
#include <limits>
#include <stdexcept>
#include <string>
#include <thread>
#include <vector>

namespace {

// ---------------------------------------------------------------------------------------------
// errors: the reference throws vpux::Exception (src/vpux_utils/include/vpux/utils/core/error.hpp:25-50);
// here an exception carries the status code and is converted at the C boundary.
// ---------------------------------------------------------------------------------------------
struct OrcError : std::runtime_error {
    int code;
    OrcError(int c, const std::string& m): std::runtime_error(m), code(c) {
    }
};

[[noreturn]] void fail(int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    throw OrcError(code, buf);
}

int guard(char* err, size_t errlen, const std::function<void()>& body) {
    try {
        body();
        if (err && errlen) err[0] = 0;
        return VF_OK;
    } catch (const OrcError& e) {
        if (err && errlen) snprintf(err, errlen, "%s", e.what());
        return e.code;
    } catch (const std::exception& e) {
        if (err && errlen) snprintf(err, errlen, "%s", e.what());
        return VF_ERR_INVALID_ARG;
    }
}

// ---------------------------------------------------------------------------------------------
// scalar types
// ---------------------------------------------------------------------------------------------
uint32_t f2u(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    return u;
}
float u2f(uint32_t u) {
    float f;
    memcpy(&f, &u, 4);
    return f;
}

// float16::float16(float) — src/vpux_utils/src/core/type/float16.cpp:30-108
uint16_t f32_to_f16(float value) {
    const uint32_t iv = f2u(value);
    const uint32_t smask = 0x80000000u, emask_32 = 0x7F800000u, fmask_32 = 0x007fffffu;
    const uint32_t emask_16 = 0x7c000000u, fmask_16 = 0x03ff0000u;
    const uint32_t rhalf_16 = 0x0001ffffu, rnorm_16 = 0x00007fffu, reven_16 = 0x00008000u, rodd_16 = 0x00018000u;

    const uint32_t biased_exp_field_32 = iv & emask_32;
    uint32_t frac = (iv & fmask_32) << 3;
    if (biased_exp_field_32 == emask_32) {  // Inf / NaN, :56-69
        if (frac != 0) {
            frac &= fmask_16;
            if (frac == 0) frac = 0x00010000u;
        }
        return uint16_t(((iv & smask) | emask_16 | frac) >> 16);
    }
    if (biased_exp_field_32 == 0) {  // fp32 zero / subnormal -> signed zero, :71-74
        return uint16_t((iv & smask) >> 16);
    }
    int16_t biased_exp_16 = int16_t(int32_t(biased_exp_field_32 >> 23) - 127 + 15);
    if ((frac & rhalf_16) == rodd_16 || (frac & rnorm_16) != 0) {  // :77-83
        frac += reven_16;
        if (0 != (frac & emask_16)) {
            frac &= emask_16;
            biased_exp_16++;
        }
    }
    frac &= fmask_16;
    if (biased_exp_16 > 30) {  // overflow -> Inf, :85-89
        return uint16_t(((iv & smask) | emask_16) >> 16);
    }
    if (biased_exp_16 > 0) {
        return uint16_t(((iv & smask) | (uint32_t(biased_exp_16) << 26) | frac) >> 16);
    }
    // fp16 subnormal result, :94-107
    frac = 0x04000000u | ((iv & fmask_32) << 3);
    const uint32_t shift = biased_exp_16 < -30 ? 0u : (1u << (1 - biased_exp_16));
    const uint32_t sticky = (frac & (shift - 1)) ? 1u : 0u;
    if (1 + (-biased_exp_16) > 31)
        frac = 0;
    else
        frac >>= 1 + (-biased_exp_16);
    frac |= sticky;
    if (((frac & rhalf_16) == rodd_16) || ((frac & rnorm_16) != 0)) {
        frac += reven_16;
    }
    return uint16_t(((iv & smask) | frac) >> 16);
}

// float16::operator float — float16.cpp:118-144
float f16_to_f32(uint16_t h) {
    uint32_t exp = 0x1F & (h >> 10);
    uint32_t fexp = exp + 127 - 15;
    uint32_t frac = h & 0x03FF;
    if (exp == 0) {
        if (frac == 0) {
            fexp = 0;
        } else {
            fexp++;
            while (0 == (frac & 0x0400)) {
                fexp--;
                frac <<= 1;
            }
            frac &= 0x03FF;
        }
    } else if (exp == 0x1F) {
        fexp = 0xFF;
    }
    frac <<= 13;
    return u2f((uint32_t(h & 0x8000) << 16) | (fexp << 23) | frac);
}

// bfloat16::round_to_nearest_even — src/vpux_utils/include/vpux/utils/core/type/bfloat16.hpp:85-87.
// Adds half an ulp only when the kept LSB is set; not IEEE round-to-nearest-even.
uint16_t f32_to_bf16(float value) {
    const uint32_t u = f2u(value);
    return uint16_t((u + ((u & 0x00010000u) >> 1)) >> 16);
}
// bfloat16::operator float — src/vpux_utils/src/core/type/bfloat16.cpp:61-67
float bf16_to_f32(uint16_t b) {
    return u2f(uint32_t(b) << 16);
}

// CvtHelper<float16>::cvt — VC/include/vpux/compiler/dialect/const/utils/content.hpp:41-55:
// an infinite fp16 result is clamped into [lowest, max] = +-65504 (float16.hpp:218-229). NaN passes.
uint16_t f32_to_f16_clamped(float v) {
    uint16_t h = f32_to_f16(v);
    if ((h & 0x7FFF) == 0x7C00) {
        h = uint16_t((h & 0x8000) | 0x7BFF);
    }
    return h;
}

// ---------------------------------------------------------------------------------------------
// 8-bit floats — src/vpux_utils/src/core/type/float8_e4m3.cpp, float8_e5m2.cpp
// ---------------------------------------------------------------------------------------------
// float8_e4m3::operator float (:125-129): the reference looks |bits| up in a table of the 128 magnitudes
// (subnormals m * 2^-9, normals (1 + m/8) * 2^(e-7), 0x7f = NaN) and ors the sign in.
float f8e4m3_to_f32(uint8_t b) {
    const uint32_t mag = b & 0x7Fu;
    float v;
    if (mag == 0x7Fu) v = std::numeric_limits<float>::quiet_NaN();
    else if ((mag >> 3) == 0) v = std::ldexp(float(mag & 7u), -9);
    else v = std::ldexp(1.0f + float(mag & 7u) / 8.0f, int(mag >> 3) - 7);
    uint32_t u;
    memcpy(&u, &v, 4);
    u |= uint32_t(b & 0x80u) << 24;
    memcpy(&v, &u, 4);
    return v;
}
// f32_to_f8e4m3_bits (:52-113). For |value| < 2^-37 the reference shifts a 32-bit word by 32 or more, which is
// undefined; every defined shift of that branch yields a signed zero and so does this restatement.
uint8_t f32_to_f8e4m3(float value) {
    const uint32_t f32_s_mask = 0x80000000u, f32_e_mask = 0x7F800000u, f32_m_mask = 0x007FFFFFu;
    const uint32_t f8_e_mask = 0x78u << 24, f8_m_mask = 0x07u << 24, f8_m_hidden_one_mask = 0x08000000u;
    const uint32_t round_half = 0x01FFFFFFu, round_norm = 0x007FFFFFu, round_even = 0x00800000u, round_odd = 0x01800000u;
    uint32_t bits;
    memcpy(&bits, &value, 4);
    uint8_t f8 = uint8_t((bits & f32_s_mask) >> 24);
    const uint32_t e_field = bits & f32_e_mask;
    if (e_field == f32_e_mask) return uint8_t(f8 | 0x7Fu);  // no infinity in this type: NaN
    if (e_field == 0) return f8;
    int32_t exp8 = int32_t(e_field >> 23) - (127 - 7);
    uint32_t fractional = (bits & f32_m_mask) << 4;
    if ((fractional & round_half) == round_odd || (fractional & round_norm) != 0) {
        fractional += round_even;
        if (fractional & f8_e_mask) {
            fractional &= f8_e_mask;
            ++exp8;
        }
    }
    fractional &= f8_m_mask;
    if (exp8 > 15) return uint8_t(f8 | 0x7Fu);
    if (exp8 > 0) return uint8_t(f8 | (exp8 << 3) | (fractional >> 24));
    fractional = f8_m_hidden_one_mask | ((bits & f32_m_mask) << 4);
    const int32_t by = 1 - exp8;
    if (by >= 32) return f8;
    const int32_t shift = exp8 < -15 ? 0 : int32_t(1u << by);
    const uint32_t sticky = (fractional & uint32_t(shift - 1)) ? 1u : 0u;
    fractional = (fractional >> by) | sticky;
    if ((fractional & round_half) == round_odd || (fractional & round_norm) != 0) fractional += round_even;
    return uint8_t(f8 | (fractional >> 24));
}
// f32_to_f8e5m2_bits (:76-80) over emulate_f8e5m2_on_fp16 (:27-74); float8_e5m2::operator float (:94-96)
uint8_t f32_to_f8e5m2(float value) {
    uint16_t h = f32_to_f16(value);
    const bool can_round = (h & 0x7F00) < 0x7B00;
    const bool is_naninf = (h & 0x7C00) == 0x7C00;
    const uint16_t rnmask = h & 0x00FF, rnmask_tie = h & 0x0180;
    if (!is_naninf && can_round) h = uint16_t(h + (((rnmask > 0x0080) || (rnmask_tie == 0x0180)) << 8));
    h &= 0xFF00;
    return uint8_t(h >> 8);
}
float f8e5m2_to_f32(uint8_t b) {
    return f16_to_f32(uint16_t(uint16_t(b) << 8));
}

// ---------------------------------------------------------------------------------------------
// dtype helpers
// ---------------------------------------------------------------------------------------------
int dtype_bits(int dt) {
    switch (dt) {
    case VF_DT_F32: return 32;
    case VF_DT_F16: return 16;
    case VF_DT_BF16: return 16;
    case VF_DT_F64: return 64;
    case VF_DT_I8: case VF_DT_U8: return 8;
    case VF_DT_F8E4M3FN: case VF_DT_F8E5M2: return 8;
    case VF_DT_I16: case VF_DT_U16: return 16;
    case VF_DT_I32: case VF_DT_U32: return 32;
    case VF_DT_I64: case VF_DT_U64: return 64;
    case VF_DT_I4: case VF_DT_U4: return 4;
    case VF_DT_I1: return 1;
    default: fail(VF_ERR_INVALID_ARG, "bad dtype %d", dt);
    }
}
bool dtype_is_float(int dt) {
    return dt == VF_DT_F32 || dt == VF_DT_F16 || dt == VF_DT_BF16 || dt == VF_DT_F64 || dt == VF_DT_F8E4M3FN || dt == VF_DT_F8E5M2;
}
bool dtype_is_signed_int(int dt) {
    return dt == VF_DT_I8 || dt == VF_DT_I16 || dt == VF_DT_I32 || dt == VF_DT_I64 || dt == VF_DT_I4;
}
bool dtype_is_int(int dt) {
    return !dtype_is_float(dt) && dt != VF_DT_INVALID;
}
void int_limits(int dt, double& lo, double& hi) {
    switch (dt) {
    case VF_DT_I8: lo = -128; hi = 127; break;
    case VF_DT_U8: lo = 0; hi = 255; break;
    case VF_DT_I16: lo = -32768; hi = 32767; break;
    case VF_DT_U16: lo = 0; hi = 65535; break;
    case VF_DT_I32: lo = -2147483648.0; hi = 2147483647.0; break;
    case VF_DT_U32: lo = 0; hi = 4294967295.0; break;
    case VF_DT_I64: lo = -9223372036854775808.0; hi = 9223372036854775807.0; break;
    case VF_DT_U64: lo = 0; hi = 18446744073709551615.0; break;
    default: fail(VF_ERR_UNSUPPORTED, "no integer limits for dtype %d", dt);
    }
}

// ---------------------------------------------------------------------------------------------
// types
// ---------------------------------------------------------------------------------------------
struct Elem {
    int kind = VF_ELEM_PLAIN;
    int dtype = VF_DT_INVALID;
    int expressed = VF_DT_INVALID;
    int axis = -1;
    int64_t qmin = 0, qmax = 0;
    std::vector<double> scales;
    std::vector<int64_t> zps;
    bool quantized() const {
        return kind != VF_ELEM_PLAIN;
    }
};

struct Type {
    Elem elem;
    int rank = 0;
    uint32_t order = 0;
    int64_t shape[VF_MAX_RANK] = {};
    int64_t numel() const {
        int64_t n = 1;
        for (int i = 0; i < rank; ++i) n *= shape[i];
        return n;
    }
};

Elem elem_from_pod(const vf_elem_type& e) {
    Elem r;
    r.kind = e.kind;
    r.dtype = e.dtype;
    r.expressed = e.expressed;
    r.axis = e.axis;
    r.qmin = e.qmin;
    r.qmax = e.qmax;
    if (r.kind != VF_ELEM_PLAIN) {
        if (e.nparams <= 0 || !e.scales || !e.zps) fail(VF_ERR_INVALID_ARG, "quantized type without parameters");
        r.scales.assign(e.scales, e.scales + e.nparams);
        r.zps.assign(e.zps, e.zps + e.nparams);
        if (r.kind == VF_ELEM_QUANT_UNIFORM && e.nparams != 1) fail(VF_ERR_SHAPE, "uniform type needs 1 param");
        // a quantized type cannot be built with such a scale: mlir::quant::UniformQuantized[PerAxis]Type::verify
        // rejects scale <= 0, infinities and NaN ("illegal scale")
        for (double sc : r.scales)
            if (!(sc > 0.0) || std::isinf(sc)) fail(VF_ERR_INVALID_ARG, "illegal scale");
    }
    return r;
}

uint32_t identity_order(int rank) {
    uint32_t c = 0;
    for (int i = 0; i < rank; ++i) c = (c << 4) | uint32_t(i + 1);
    return c;
}

// DimsOrder: perm[memDim] = logical dim (0-based) — VC/src/core/attributes/dims_order.cpp
void order_to_perm(uint32_t order, int rank, int* perm) {
    if (order == 0) order = identity_order(rank);
    bool seen[VF_MAX_RANK] = {false, false, false, false, false};
    for (int i = rank - 1; i >= 0; --i) {
        int d = int(order & 0xF) - 1;
        order >>= 4;
        if (d < 0 || d >= rank || seen[d]) fail(VF_ERR_INVALID_ARG, "bad dims order");
        seen[d] = true;
        perm[i] = d;
    }
    if (order != 0) fail(VF_ERR_INVALID_ARG, "dims order rank mismatch");
}

Type type_from_pod(const vf_tensor_type& t) {
    Type r;
    if (t.rank < 1 || t.rank > VF_MAX_RANK) fail(VF_ERR_INVALID_ARG, "bad rank %d", t.rank);
    r.elem = elem_from_pod(t.elem);
    r.rank = t.rank;
    r.order = t.order ? t.order : identity_order(t.rank);
    for (int i = 0; i < t.rank; ++i) r.shape[i] = t.shape[i];
    int perm[VF_MAX_RANK];
    order_to_perm(r.order, r.rank, perm);
    if (r.elem.kind == VF_ELEM_QUANT_PER_AXIS) {
        if (r.elem.axis < 0 || r.elem.axis >= r.rank) fail(VF_ERR_INVALID_ARG, "bad quantized axis");
    }
    return r;
}

void mem_shape(const Type& t, int64_t* ms) {
    int perm[VF_MAX_RANK];
    order_to_perm(t.order, t.rank, perm);
    for (int i = 0; i < t.rank; ++i) ms[i] = t.shape[perm[i]];
}

// getTotalAllocSize for a compact tensor: bits rounded up to bytes
uint64_t type_bytes(const Type& t) {
    const uint64_t bits = uint64_t(dtype_bits(t.elem.dtype)) * uint64_t(t.numel());
    return (bits + 7) / 8;
}

// ---------------------------------------------------------------------------------------------
// Content — CI/utils/content.hpp:166-352: logical type + storage element type + splat flag
// ---------------------------------------------------------------------------------------------
struct Content {
    Type type;
    int storage = VF_DT_INVALID;
    bool splat = false;
    std::vector<uint8_t> own;
    const uint8_t* ptr = nullptr;
    uint64_t nbytes = 0;
    const uint8_t* data() const {
        return ptr;
    }
    uint8_t* mdata() {
        return own.data();
    }
    // Content::allocTempBuffer — CD/utils/content.cpp:34-48
    static Content alloc(const Type& type, int storage, bool splat, int64_t raw_bytes = -1) {
        Content c;
        c.type = type;
        c.storage = storage;
        c.splat = splat;
        uint64_t n = raw_bytes >= 0 ? uint64_t(raw_bytes)
                                    : (uint64_t(dtype_bits(storage)) * uint64_t(splat ? 1 : type.numel()) + 7) / 8;
        c.own.assign(n, 0);
        c.ptr = c.own.data();
        c.nbytes = n;
        return c;
    }
};

// checked_cast — src/vpux_utils/include/vpux/utils/core/checked_cast.hpp:43-141
struct Val {  // one element read from storage, as the widest lossless carrier of its class
    bool is_float;
    double f;  // float-class value (f32/f16/bf16 widened exactly)
    float ff;  // the same value as the fp32 the reference passes by value (keeps signalling-NaN payloads)
    int64_t i;
    uint64_t u;
    bool is_unsigned;
};

Val load_val(const uint8_t* p, int dt, int64_t idx) {
    Val v{};
    switch (dt) {
    case VF_DT_F32: { float f; memcpy(&f, p + idx * 4, 4); v.is_float = true; v.f = f; v.ff = f; break; }
    case VF_DT_F16: { uint16_t h; memcpy(&h, p + idx * 2, 2); v.is_float = true; v.ff = f16_to_f32(h); v.f = v.ff; break; }
    case VF_DT_BF16: { uint16_t h; memcpy(&h, p + idx * 2, 2); v.is_float = true; v.ff = bf16_to_f32(h); v.f = v.ff; break; }
    case VF_DT_F64: { double d; memcpy(&d, p + idx * 8, 8); v.is_float = true; v.f = d; break; }
    case VF_DT_F8E4M3FN: v.is_float = true; v.ff = f8e4m3_to_f32(p[idx]); v.f = v.ff; break;
    case VF_DT_F8E5M2: v.is_float = true; v.ff = f8e5m2_to_f32(p[idx]); v.f = v.ff; break;
    case VF_DT_I8: v.i = int8_t(p[idx]); break;
    case VF_DT_U8: v.is_unsigned = true; v.u = p[idx]; v.i = p[idx]; break;
    case VF_DT_I16: { int16_t x; memcpy(&x, p + idx * 2, 2); v.i = x; break; }
    case VF_DT_U16: { uint16_t x; memcpy(&x, p + idx * 2, 2); v.is_unsigned = true; v.u = x; v.i = x; break; }
    case VF_DT_I32: { int32_t x; memcpy(&x, p + idx * 4, 4); v.i = x; break; }
    case VF_DT_U32: { uint32_t x; memcpy(&x, p + idx * 4, 4); v.is_unsigned = true; v.u = x; v.i = x; break; }
    case VF_DT_I64: { int64_t x; memcpy(&x, p + idx * 8, 8); v.i = x; break; }
    case VF_DT_U64: { uint64_t x; memcpy(&x, p + idx * 8, 8); v.is_unsigned = true; v.u = x; v.i = int64_t(x); break; }
    default: fail(VF_ERR_UNSUPPORTED, "getValues: unsupported storage dtype %d", dt);
    }
    return v;
}

// getValues<float>()[i]: CvtHelper<float>::cvt = checked_cast<float>(storage value) — content.hpp:33-39
float val_as_float(const Val& v, int storage) {
    if (v.is_float) {
        if (storage == VF_DT_F64) {  // checked_cast<float>(double): must round-trip, checked_cast.hpp:133-139
            float f = float(v.f);
            if (double(f) != v.f) fail(VF_ERR_CHECKED_CAST, "Can not safely cast %g from double to float", v.f);
            return f;
        }
        return v.ff;
    }
    if (v.is_unsigned) {  // checked_cast.hpp:125-131
        float f = float(v.u);
        if (uint64_t(f) != v.u) fail(VF_ERR_CHECKED_CAST, "Can not safely cast integer to float");
        return f;
    }
    float f = float(v.i);  // checked_cast.hpp:117-123
    if (int64_t(f) != v.i) fail(VF_ERR_CHECKED_CAST, "Can not safely cast integer to float");
    return f;
}

// getValues<IntT>()[i] for an integer OutT described by dtype `out`
int64_t val_as_int(const Val& v, int storage, int out) {
    double lo, hi;
    int_limits(out, lo, hi);
    if (v.is_float) {
        // checked_cast<Int>(float/double) — checked_cast.hpp:106-117; the comparison is done in the input
        // floating type against static_cast<InT>(limit).
        if (storage == VF_DT_F64) {
            if (!(v.f <= hi) || !(v.f >= lo)) fail(VF_ERR_CHECKED_CAST, "Can not safely cast %g to integer", v.f);
        } else {
            const float fv = float(v.f);
            if (!(fv <= float(hi)) || !(fv >= float(lo)))
                fail(VF_ERR_CHECKED_CAST, "Can not safely cast %g to integer", v.f);
            if (out == VF_DT_I64 && fv >= 9223372036854775808.0f)
                fail(VF_ERR_CHECKED_CAST, "float to int64 overflow");
            if (out == VF_DT_I32 && fv >= 2147483648.0f) fail(VF_ERR_CHECKED_CAST, "float to int32 overflow");
            if (out == VF_DT_U32 && fv >= 4294967296.0f) fail(VF_ERR_CHECKED_CAST, "float to uint32 overflow");
        }
        return int64_t(v.f);  // truncation toward zero
    }
    if (v.is_unsigned) {
        if (double(v.u) > hi) fail(VF_ERR_CHECKED_CAST, "Can not safely cast %llu", (unsigned long long)v.u);
        return int64_t(v.u);
    }
    if (double(v.i) < lo || double(v.i) > hi) fail(VF_ERR_CHECKED_CAST, "Can not safely cast %lld", (long long)v.i);
    return v.i;
}

struct Reader {  // ContentRange: splat reads element 0 for every index — content.hpp:113-122
    const Content& c;
    explicit Reader(const Content& cc): c(cc) {
    }
    Val at(int64_t i) const {
        return load_val(c.data(), c.storage, c.splat ? 0 : i);
    }
    float f(int64_t i) const {
        return val_as_float(at(i), c.storage);
    }
    int64_t i64(int64_t i, int out = VF_DT_I64) const {
        return val_as_int(at(i), c.storage, out);
    }
};

void store_int(uint8_t* p, int dt, int64_t idx, int64_t v) {
    switch (dt) {
    case VF_DT_I8: case VF_DT_U8: p[idx] = uint8_t(v); break;
    case VF_DT_I16: case VF_DT_U16: { uint16_t x = uint16_t(v); memcpy(p + idx * 2, &x, 2); break; }
    case VF_DT_I32: case VF_DT_U32: { uint32_t x = uint32_t(v); memcpy(p + idx * 4, &x, 4); break; }
    case VF_DT_I64: case VF_DT_U64: { memcpy(p + idx * 8, &v, 8); break; }
    default: fail(VF_ERR_UNSUPPORTED, "store_int: dtype %d", dt);
    }
}

// ---------------------------------------------------------------------------------------------
// loop_nd — VC/src/utils/loop.cpp:23-228: one dimension is split into contiguous chunks, the first one whose
// extent >= #threads, else the largest; every chunk runs on its own worker.
// ---------------------------------------------------------------------------------------------
void parallel_nd(int nthreads, const std::vector<int64_t>& dims,
                 const std::function<void(const int64_t* begin, const int64_t* end)>& body) {
    for (auto d : dims)
        if (d <= 0) return;
    const size_t nd = dims.size();
    std::vector<int64_t> b(nd, 0), e(dims);
    if (nthreads <= 1) {
        body(b.data(), e.data());
        return;
    }
    int part = -1;
    size_t maxi = 0;
    for (size_t i = 0; i < nd; ++i) {
        if (part < 0 && dims[i] >= nthreads) part = int(i);
        if (dims[i] > dims[maxi]) maxi = i;
    }
    int64_t use = nthreads;
    if (part < 0) {
        part = int(maxi);
        use = dims[maxi];
    }
    const int64_t per = (dims[part] + use - 1) / use;
    std::vector<std::thread> th;
    std::vector<std::string> errs(use);
    std::vector<int> codes(use, 0);
    for (int64_t t = 0; t < use; ++t) {
        const int64_t lo = per * t, hi = std::min(lo + per, dims[part]);
        if (lo >= hi) break;
        th.emplace_back([&, t, lo, hi] {
            std::vector<int64_t> bb(b), ee(e);
            bb[part] = lo;
            ee[part] = hi;
            try {
                body(bb.data(), ee.data());
            } catch (const OrcError& ex) {
                codes[t] = ex.code;
                errs[t] = ex.what();
            }
        });
    }
    for (auto& x : th) x.join();
    for (int64_t t = 0; t < use; ++t)
        if (codes[t]) throw OrcError(codes[t], errs[t]);
}

// ---------------------------------------------------------------------------------------------
// quantization arithmetic
// ---------------------------------------------------------------------------------------------
// dequantize() — VC/include/vpux/compiler/utils/quantization.hpp:208-210
float dequantize_value(int64_t q, double scale, int64_t zp) {
    return static_cast<float>((q - zp) * scale);
}

// fakeQuantize() — VC/src/utils/quantization.cpp:995-1003 (all operands float, one rounding per operation)
float fake_quantize(float inVal, float inLow, float inHigh, float qLow, float qHigh, float fLevels) {
    if (inVal <= inLow) {
        return qLow;
    } else if (inVal > inHigh) {
        return qHigh;
    } else {
        return std::round((inVal - inLow) / (inHigh - inLow) * (fLevels - 1)) / (fLevels - 1) * (qHigh - qLow) + qLow;
    }
}

// createQuantizeFn — CD/attributes/quantize.cpp:91-106
struct Quantizer {
    float inMin, inMax, qMin, qMax, levels;
    Quantizer(double scale, int64_t zp, int64_t qmin, int64_t qmax) {
        inMin = dequantize_value(qmin, scale, zp);
        inMax = dequantize_value(qmax, scale, zp);
        qMin = float(qmin);
        qMax = float(qmax);
        levels = float(qmax - qmin + 1);
    }
    int64_t operator()(float x) const {
        // the lambda takes a double, fakeQuantize takes float: float -> double -> float is exact
        const double xd = x;
        const float fq = fake_quantize(float(xd), inMin, inMax, qMin, qMax, levels);
        // a NaN passes both comparisons of fakeQuantize and reaches static_cast<int64_t>(NaN), which is undefined:
        // both sides of the parity tests refuse it
        if (std::isnan(fq)) fail(VF_ERR_NAN, "Quantize met a NaN: its conversion to an integer is undefined in the reference");
        return static_cast<int64_t>(fq);
    }
};

// calcScaleAndZeroPoint — VC/src/utils/quantization.cpp:574-636
bool calc_scale_zp(double qMinFP, double qMaxFP, double rMin, double rMax, double& scaleOut, int64_t& zpOut) {
    const double eps = std::numeric_limits<double>::epsilon();
    if (std::fabs(rMax - rMin) < eps) {
        const double scale = rMin;
        if (std::fabs(scale) < eps) {
            scaleOut = 1.0;
            zpOut = 0;
            return true;
        }
        if (scale >= eps) {
            scaleOut = scale;
            zpOut = 0;
            return true;
        }
        if (scale <= -eps) {
            scaleOut = scale * (-1);
            zpOut = 2;
            return true;
        }
        return false;
    }
    const bool containsZero = (rMin <= 0 && rMax >= 0) || (rMin >= 0 && rMax <= 0);
    if (!containsZero) return false;
    const double scale = (rMax - rMin) / (qMaxFP - qMinFP);
    if (std::fabs(scale) <= eps) return false;
    const double x = qMinFP - rMin / scale;
    scaleOut = scale;
    zpOut = static_cast<int64_t>(std::round(x));
    return true;
}

// approximate<int32_t>(15, target) + QuantizationApproximation ctor —
// VC/include/vpux/compiler/utils/quantization.hpp:65-77, VC/src/utils/quantization.cpp:426-433
void approximate15(double target, int32_t& mult, int32_t& shift) {
    const int bits = 15;
    int exponent = 0;
    const double mantissa = std::frexp(target, &exponent);
    const double m = std::floor(mantissa * std::pow(2, bits));
    if (!(m <= 2147483647.0) || !(m >= -2147483648.0)) fail(VF_ERR_CHECKED_CAST, "mult out of int32");
    mult = int32_t(m);
    if (exponent > bits) {
        fail(VF_ERR_RANGE, "approximate %g: postShift %d is not supported", target, bits - exponent);
    }
    const int s = bits - exponent;
    if (s < 0 || s > 255) fail(VF_ERR_CHECKED_CAST, "shift %d does not fit uint8", s);
    shift = s;
}

// ---------------------------------------------------------------------------------------------
// type inference per transformation (inferOutputType / inferOutputSplat)
// ---------------------------------------------------------------------------------------------
int normalized_storage(const Elem& e) {  // normalizeQuantStorageType — quantization.cpp:118-132
    return e.dtype;                      // vf_dtype already carries the signedness
}

bool all_equal(const std::vector<int64_t>& v) {
    return std::adjacent_find(v.begin(), v.end(), std::not_equal_to<>()) == v.end();
}

// expandScalesAndZP — VC/src/utils/quantization.cpp:168-224
Elem expand_scales_zp(const Elem& e, const int64_t* before, const int64_t* after) {
    const int64_t pb = before[e.axis], pa = after[e.axis];
    if (pb == 0 && pa == 0) return e;
    if (e.scales.empty() || e.zps.empty()) fail(VF_ERR_SHAPE, "Can't get value for expand scales");
    if (!all_equal(e.zps)) fail(VF_ERR_ZERO_POINTS, "All zero points should be equal");
    Elem r = e;
    r.scales.assign(size_t(pb), e.scales.front());
    r.scales.insert(r.scales.end(), e.scales.begin(), e.scales.end());
    r.scales.insert(r.scales.end(), size_t(pa), e.scales.back());
    r.zps.assign(size_t(pb), e.zps.front());
    r.zps.insert(r.zps.end(), e.zps.begin(), e.zps.end());
    r.zps.insert(r.zps.end(), size_t(pa), e.zps.back());
    return r;
}

void validate_per_axis(const Type& t) {  // validateQuantElemType — quantization.cpp:74-116
    if (t.elem.kind == VF_ELEM_QUANT_PER_AXIS) {
        if (t.elem.axis < 0 || t.elem.axis >= t.rank) fail(VF_ERR_SHAPE, "quantized axis outside rank");
        if (int64_t(t.elem.scales.size()) != t.shape[t.elem.axis])
            fail(VF_ERR_SHAPE, "Number of scales '%zu' in per-axis quantized type do not match the quantized dimension size '%lld'",
                 t.elem.scales.size(), (long long)t.shape[t.elem.axis]);
    }
}


int64_t align_up(int64_t v, int64_t a) {
    return (v + a - 1) / a * a;
}

// Sparsify compressType — CD/attributes/sparsify.cpp:93-101 (VPU_WEIGHT_SET_BYTE_ALIGNMENT = 16, nce_invariant.hpp:36)
Type compress_type(const Type& in, const std::vector<int64_t>& counts) {
    const int64_t eb = dtype_bits(in.elem.dtype) / 8;
    int64_t total = 0;
    for (auto n : counts) total += align_up(n * eb, 16);
    Type r;
    r.rank = 4;
    r.order = in.order;
    r.shape[0] = total;
    r.shape[1] = r.shape[2] = r.shape[3] = 1;
    r.elem.kind = VF_ELEM_PLAIN;
    r.elem.dtype = VF_DT_U8;
    return r;
}

Type infer_one(const Type& in, bool in_splat, const vf_transform& t, bool& out_splat) {
    Type out = in;
    out_splat = in_splat;
    switch (t.kind) {
    case VF_T_CAST_ELEM_TYPE:     // cast_elem_type.cpp:27-33
    case VF_T_CONVERT_ELEM_TYPE:  // convert_elem_type.cpp:40-46
        out.elem = elem_from_pod(t.elem);
        validate_per_axis(out);
        break;
    case VF_T_DEQUANTIZE: {  // dequantize.cpp:19-36
        if (!in.elem.quantized()) fail(VF_ERR_NOT_QUANTIZED, "Got non quantized type in 'DequantizeAttr'");
        Elem e;
        e.kind = VF_ELEM_PLAIN;
        e.dtype = in.elem.expressed;
        out.elem = e;
        if (in.elem.kind == VF_ELEM_QUANT_PER_AXIS) out_splat = false;
        break;
    }
    case VF_T_QUANTIZE: {  // quantize.cpp:22-27, 64-74
        Elem q = elem_from_pod(t.elem);
        if (!q.quantized()) fail(VF_ERR_INVALID_ARG, "Can't quantize to empty type");
        if (!dtype_is_int(q.dtype) || dtype_bits(q.dtype) < 8)
            fail(VF_ERR_UNSUPPORTED, "Const.Quantize supports only integer byte+ storage type");
        Elem e;
        e.kind = VF_ELEM_PLAIN;
        e.dtype = normalized_storage(q);
        out.elem = e;
        out_splat = false;
        break;
    }
    case VF_T_RESCALE:
    case VF_T_ADD:
        break;
    case VF_T_RESHAPE:                      // reshape.cpp:74-77 -> changeShape, VC/src/core/type_interfaces.cpp:208-231
    case VF_T_CHANGE_SHAPE_AND_ELEM_TYPE: {  // change_shape_and_elem_type.cpp:62-66 -> changeShapeElemType :253-269
        if (t.rank < 1 || t.rank > VF_MAX_RANK) fail(VF_ERR_INVALID_ARG, "bad reshape rank");
        int64_t n = 1;
        for (int i = 0; i < t.rank; ++i) n *= t.a[i];
        if (n != in.numel()) fail(VF_ERR_SHAPE, "Reshape changes the number of elements");
        out.rank = t.rank;
        for (int i = 0; i < VF_MAX_RANK; ++i) out.shape[i] = i < t.rank ? t.a[i] : 0;
        const bool origIsIdentity = in.order == identity_order(in.rank);
        if (origIsIdentity) out.order = identity_order(t.rank);
        else if (in.rank != t.rank) fail(VF_ERR_SHAPE, "Order is incompatible with the new shape");
        if (t.kind == VF_T_CHANGE_SHAPE_AND_ELEM_TYPE) {
            out.elem = elem_from_pod(t.elem);
        } else if (in.elem.kind == VF_ELEM_QUANT_PER_AXIS) {
            // getQuantizedAxis — VC/src/utils/types.cpp:140-162
            const int axis = in.elem.axis;
            if (axis >= 0 && axis < in.rank && in.shape[axis] != 1) {
                int64_t fullSizeIncludingAxis = 1;
                for (int i = 0; i <= axis; ++i) fullSizeIncludingAxis *= in.shape[i];
                int64_t accumSize = 1;
                for (int i = 0; i < t.rank; ++i) {
                    accumSize *= t.a[i];
                    if (accumSize == fullSizeIncludingAxis && t.a[i] == in.shape[axis]) {
                        out.elem.axis = i;
                        break;
                    }
                    if (accumSize > fullSizeIncludingAxis) break;
                }
            }
        }
        if (out.elem.kind == VF_ELEM_QUANT_PER_AXIS) {  // validateQuantElemType — VC/src/utils/quantization.cpp:86-116
            if (out.elem.axis < 0 || out.elem.axis >= out.rank) fail(VF_ERR_SHAPE, "Quantized axis is out of main type rank");
            if (int64_t(out.elem.scales.size()) != out.shape[out.elem.axis])
                fail(VF_ERR_SHAPE, "Number of scales in per-axis quantized type do not match the quantized dimension size");
        }
        break;
    }
    case VF_T_REORDER:      // reorder.cpp:60-77: changeDimsOrder
    case VF_T_LAYOUT_CAST:  // layout_cast.cpp:60-80
    {
        int perm[VF_MAX_RANK];
        order_to_perm(t.order, in.rank, perm);  // validates rank / permutation (reorder.cpp:19-30)
        out.order = t.order ? t.order : identity_order(in.rank);
        if (t.kind == VF_T_LAYOUT_CAST) break;
        break;
    }
    case VF_T_TRANSPOSE:      // transpose.cpp:60-94: logical dims permuted, layout kept identity-relative
    case VF_T_MEM_PERMUTE: {  // mem_permute.cpp:70-115
        // Both are expressed through inferOutputType helpers that depend on MLIR affine maps; the restatement
        // covers the form the folding pipeline uses: output logical shape = input shape permuted by `order`
        // for Transpose; for MemPermute the logical shape is recomputed from the permuted memory shape.
        int inPerm[VF_MAX_RANK], p[VF_MAX_RANK];
        order_to_perm(in.order, in.rank, inPerm);
        if (t.kind == VF_T_TRANSPOSE) {
            order_to_perm(t.order, in.rank, p);
            for (int i = 0; i < in.rank; ++i) out.shape[i] = in.shape[p[i]];
            if (in.elem.kind == VF_ELEM_QUANT_PER_AXIS) {
                for (int i = 0; i < in.rank; ++i)
                    if (p[i] == in.elem.axis) {
                        out.elem.axis = i;
                        break;
                    }
            }
            out.order = in.order;
        } else {
            int64_t ims[VF_MAX_RANK], oms[VF_MAX_RANK];
            mem_shape(in, ims);
            order_to_perm(t.mem_perm, in.rank, p);
            for (int i = 0; i < in.rank; ++i) oms[i] = ims[p[i]];
            int dstPerm[VF_MAX_RANK];
            order_to_perm(t.order, in.rank, dstPerm);
            for (int i = 0; i < in.rank; ++i) out.shape[dstPerm[i]] = oms[i];
            out.order = t.order ? t.order : identity_order(in.rank);
            if (in.elem.kind == VF_ELEM_QUANT_PER_AXIS) {
                int inMemAxis = -1;
                for (int i = 0; i < in.rank; ++i)
                    if (inPerm[i] == in.elem.axis) inMemAxis = i;
                for (int i = 0; i < in.rank; ++i)
                    if (p[i] == inMemAxis) out.elem.axis = dstPerm[i];
            }
        }
        break;
    }
    case VF_T_PAD_WITH_ZERO: {  // pad_with_zero.cpp:93-101 -> TensorNDTypeInterface::pad, type_interfaces.cpp:332-360
        if (t.rank != in.rank) fail(VF_ERR_SHAPE, "Paddings and input shape are not consistent");
        for (int i = 0; i < in.rank; ++i) out.shape[i] = in.shape[i] + t.a[i] + t.b[i];
        if (in.elem.kind == VF_ELEM_QUANT_PER_AXIS) out.elem = expand_scales_zp(in.elem, t.a, t.b);
        validate_per_axis(out);
        out_splat = false;
        break;
    }
    case VF_T_SUBVIEW: {  // subview.cpp:60-90: getTensorType(extractDenseTile); per-axis params are sliced
        if (t.rank != in.rank) fail(VF_ERR_SHAPE, "SubView rank mismatch");
        for (int i = 0; i < in.rank; ++i) {
            if (t.a[i] < 0 || t.b[i] <= 0 || t.a[i] + t.b[i] > in.shape[i]) fail(VF_ERR_SHAPE, "SubView out of bounds");
            out.shape[i] = t.b[i];
        }
        if (in.elem.kind == VF_ELEM_QUANT_PER_AXIS) {
            const int ax = in.elem.axis;
            out.elem.scales.assign(in.elem.scales.begin() + t.a[ax], in.elem.scales.begin() + t.a[ax] + t.b[ax]);
            out.elem.zps.assign(in.elem.zps.begin() + t.a[ax], in.elem.zps.begin() + t.a[ax] + t.b[ax]);
        }
        break;
    }
    case VF_T_BIT_PACK: {  // bit_pack.cpp:25-36, 73-126
        if (t.width != 4) fail(VF_ERR_UNSUPPORTED, "BitPackAttr does not support any bitwidth except for 4");
        if (!in.elem.quantized() && dtype_is_float(in.elem.dtype))
            fail(VF_ERR_UNSUPPORTED, "Bit pack does not support float inputs.");
        if (in_splat) fail(VF_ERR_SPLAT, "Bit pack does not support splat inputs.");
        out.elem.dtype = dtype_is_signed_int(in.elem.dtype) ? VF_DT_I4 : VF_DT_U4;
        out_splat = false;
        break;
    }
    case VF_T_GET_SPARSITY_MAP: {  // get_sparsity_map.cpp:68-80 + inferWeightsSparsityMapShape nce_sparsity.cpp:308-315
        if (in.rank != 4) fail(VF_ERR_SHAPE, "Expected data shape to be 4D");
        const int64_t work = in.shape[1] * in.shape[2] * in.shape[3];
        out.shape[0] = in.shape[0];
        out.shape[1] = out.shape[2] = 1;
        out.shape[3] = align_up(work, 128);
        out.order = identity_order(4);
        Elem e;
        e.kind = VF_ELEM_PLAIN;
        e.dtype = VF_DT_I1;
        out.elem = e;
        out_splat = false;
        break;
    }
    case VF_T_SPARSIFY: {  // sparsify.cpp:103-118
        if (t.compress_output) {
            if (!t.num_actual) fail(VF_ERR_INVALID_ARG, "Missing number of actual elements");
            std::vector<int64_t> counts(t.num_actual, t.num_actual + t.n_num_actual);
            Type ti = in;
            ti.elem.dtype = in.elem.dtype;
            out = compress_type(ti, counts);
        }
        out_splat = false;
        break;
    }
    case VF_T_SWIZZLE_CONSTANT: {  // swizzle_transform.cpp:127-156
        const int64_t arch = t.a[1];
        if (arch != VF_ARCH_NPU37XX && arch != VF_ARCH_NPU40XX)
            fail(VF_ERR_UNSUPPORTED, "Architecture %lld does not support swizzling", (long long)arch);
        if (t.a[0] < 0) fail(VF_ERR_INVALID_ARG, "negative swizzle key");
        const int64_t total = int64_t((uint64_t(in.numel()) * uint64_t(dtype_bits(in.elem.dtype)) + 7) / 8);
        const int64_t new_size = align_up(total, arch == VF_ARCH_NPU40XX ? 1024 : 512);  // swizzling_utils.hpp:26-27
        for (int i = 0; i < in.rank; ++i) out.shape[i] = 1;
        if (!in.elem.quantized() && dtype_bits(in.elem.dtype) == 1) {
            out.shape[0] = new_size * 8;
        } else if (!in.elem.quantized() && in.elem.dtype == VF_DT_F16) {
            out.shape[0] = new_size / 2;
        } else {
            out.shape[0] = new_size;
            Elem e;
            e.kind = VF_ELEM_PLAIN;
            e.dtype = VF_DT_U8;
            out.elem = e;
        }
        out_splat = false;
        break;
    }
    case VF_T_REVERSE: {  // reverse.cpp:35-44; the checks of transform() :46-105
        if (in.elem.kind == VF_ELEM_QUANT_PER_AXIS) fail(VF_ERR_UNSUPPORTED, "Unexpected data type");
        const int dt = in.elem.dtype;
        if (dt != VF_DT_I8 && dt != VF_DT_U8 && dt != VF_DT_F16 && dt != VF_DT_BF16 && dt != VF_DT_F32)
            fail(VF_ERR_UNSUPPORTED, "Unexpected data type: %d", dt);
        if (!in_splat && (t.a[0] < 0 || t.a[0] >= in.rank - 1))
            fail(VF_ERR_INVALID_ARG, "Const::Content::reverse: got unexpected content dimension %lld", (long long)t.a[0]);
        break;
    }
    case VF_T_BROADCAST: {  // broadcast.cpp:66-83
        const int64_t axis = t.a[0], value = t.a[1];
        if (axis < 0 || axis >= in.rank) fail(VF_ERR_INVALID_ARG, "Broadcast axis");
        if (value < in.shape[axis]) fail(VF_ERR_SHAPE, "Value cannot be broadcasted due to new value's size is less than old one");
        vf_transform pad{};
        pad.kind = VF_T_PAD_WITH_ZERO;
        pad.rank = in.rank;
        pad.b[axis] = value - in.shape[axis];
        bool ignored;
        out = infer_one(in, in_splat, pad, ignored);
        break;
    }
    case VF_T_EXPAND_DILATED: {  // expand_dilated.cpp:72-82 with getDilatedType, VC/src/utils/dilated_utils.cpp:11-34
        if (in.rank != 4) fail(VF_ERR_SHAPE, "Got invalid tensor rank");
        if (t.a[0] < 1 || t.a[1] < 1) fail(VF_ERR_INVALID_ARG, "dilations must be positive");
        out.shape[2] = in.shape[2] + (in.shape[2] - 1) * (t.a[0] - 1);
        out.shape[3] = in.shape[3] + (in.shape[3] - 1) * (t.a[1] - 1);
        if (out.elem.kind == VF_ELEM_QUANT_PER_AXIS && int64_t(out.elem.scales.size()) != out.shape[out.elem.axis])
            fail(VF_ERR_SHAPE, "Number of scales in per-axis quantized type do not match the quantized dimension size");
        out_splat = false;
        break;
    }
    case VF_T_SCALAR_MULT_INVERSE:  // inverse.cpp:40-50
        break;
    case VF_T_RELOCATE_WEIGHTS_TABLE: {  // relocate_weights_table.cpp:194-200
        const vf_relocate& r = t.relocate;
        if (r.n_clusters < 1 || r.n_clusters > VF_MAX_CLUSTERS) fail(VF_ERR_INVALID_ARG, "RelocateWeightsTable with %d clusters", r.n_clusters);
        if (in.elem.quantized() || dtype_bits(in.elem.dtype) != 32 || dtype_is_float(in.elem.dtype))
            fail(VF_ERR_UNSUPPORTED, "RelocateWeightsTable patches tables of 32-bit integers");
        if (r.weights_table_size < 0 || r.weights_table_size / 4 > in.numel())
            fail(VF_ERR_SHAPE, "weightsTableSize %lld exceeds the constant", (long long)r.weights_table_size);
        out_splat = in_splat;
        break;
    }
    default:
        fail(VF_ERR_INVALID_ARG, "unknown transformation kind %d", t.kind);
    }
    return out;
}

int position_requirement(int kind) {  // CI/attr_interfaces.hpp:24-28; bit_pack.cpp:160-162; sparsify.cpp:209-211
    switch (kind) {
    case VF_T_SWIZZLE_CONSTANT:    // swizzle_transform.cpp:221-223
    case VF_T_BIT_PACK: return 2;  // LAST
    case VF_T_SPARSIFY:
    case VF_T_GET_SPARSITY_MAP: return 1;  // PREFERRED_LAST
    default: return 0;
    }
}

void check_positions(const vf_transform* t, int n) {  // content.cpp:585-588
    if (n >= 2 && position_requirement(t[n - 2].kind) == 2)
        fail(VF_ERR_POSITION, "At most 1 attribute with LAST requirement allowed!");
}

// ---------------------------------------------------------------------------------------------
// transformations
// ---------------------------------------------------------------------------------------------
void axis_sizes(const Type& t, int logical_axis, int64_t& outer, int64_t& axisSize, int64_t& inner) {
    int perm[VF_MAX_RANK];
    int64_t ms[VF_MAX_RANK];
    order_to_perm(t.order, t.rank, perm);
    mem_shape(t, ms);
    int memAxis = -1;
    for (int i = 0; i < t.rank; ++i)
        if (perm[i] == logical_axis) memAxis = i;
    inner = 1;
    for (int i = memAxis + 1; i < t.rank; ++i) inner *= ms[i];
    axisSize = ms[memAxis];
    if (inner == 0) fail(VF_ERR_SHAPE, "Inner size is zero");
    if (axisSize == 0) fail(VF_ERR_SHAPE, "Quantized axis size is zero");
    outer = t.numel() / (axisSize * inner);
    if (outer == 0) fail(VF_ERR_SHAPE, "Outer size is zero");
}

// QuantizeAttr::transform — CD/attributes/quantize.cpp:108-212
Content tf_quantize(const Content& in, const vf_transform& t, int nthreads) {
    bool osplat;
    const Type outType = infer_one(in.type, in.splat, t, osplat);
    const Elem q = elem_from_pod(t.elem);
    const bool perAxis = q.kind == VF_ELEM_QUANT_PER_AXIS;
    Content out = Content::alloc(outType, q.dtype, perAxis ? false : in.splat);  // allocateTempBuffer :77-87
    Reader r(in);
    const int64_t nOut = out.splat ? 1 : outType.numel();
    if (!perAxis) {
        const Quantizer qz(q.scales[0], q.zps[0], q.qmin, q.qmax);
        for (int64_t i = 0; i < nOut; ++i) store_int(out.mdata(), q.dtype, i, qz(r.f(i)));
    } else {
        int64_t outer, axisSize, inner;
        axis_sizes(in.type, q.axis, outer, axisSize, inner);
        if (int64_t(q.scales.size()) != axisSize) fail(VF_ERR_SHAPE, "Wrong scales size");
        if (int64_t(q.zps.size()) != axisSize) fail(VF_ERR_SHAPE, "Wrong zeroPoints size");
        std::vector<Quantizer> qs;
        for (int64_t i = 0; i < axisSize; ++i) qs.emplace_back(q.scales[i], q.zps[i], q.qmin, q.qmax);
        const int64_t axisTotal = axisSize * inner;
        parallel_nd(nthreads, {outer, axisSize, inner}, [&](const int64_t* b, const int64_t* e) {
            for (int64_t o = b[0]; o < e[0]; ++o)
                for (int64_t a = b[1]; a < e[1]; ++a)
                    for (int64_t i = b[2]; i < e[2]; ++i) {
                        const int64_t idx = o * axisTotal + a * inner + i;
                        store_int(out.mdata(), q.dtype, idx, qs[a](r.f(idx)));
                    }
        });
    }
    return out;
}

// DequantizeAttr::transform — CD/attributes/dequantize.cpp:42-108
Content tf_dequantize(const Content& in, const vf_transform& t, int nthreads) {
    bool osplat;
    const Type outType = infer_one(in.type, in.splat, t, osplat);
    const Elem& q = in.type.elem;
    Content out = Content::alloc(outType, VF_DT_F32, osplat);
    Reader r(in);
    float* o = reinterpret_cast<float*>(out.mdata());
    const int64_t nOut = out.splat ? 1 : outType.numel();
    if (q.kind == VF_ELEM_QUANT_UNIFORM) {
        for (int64_t i = 0; i < nOut; ++i) o[i] = dequantize_value(r.i64(i), q.scales[0], q.zps[0]);
    } else {
        int64_t outer, axisSize, inner;
        axis_sizes(in.type, q.axis, outer, axisSize, inner);
        if (int64_t(q.scales.size()) != axisSize || int64_t(q.zps.size()) != axisSize)
            fail(VF_ERR_SHAPE, "Wrong scales size");
        const int64_t axisTotal = axisSize * inner;
        parallel_nd(nthreads, {outer, axisSize, inner}, [&](const int64_t* b, const int64_t* e) {
            for (int64_t oo = b[0]; oo < e[0]; ++oo)
                for (int64_t a = b[1]; a < e[1]; ++a)
                    for (int64_t i = b[2]; i < e[2]; ++i) {
                        const int64_t idx = oo * axisTotal + a * inner + i;
                        o[idx] = dequantize_value(r.i64(idx), q.scales[a], q.zps[a]);
                    }
        });
    }
    return out;
}

// RescaleAttr::transform / AddAttr::transform — rescale.cpp:67-82, add.cpp:62-77
Content tf_rescale_add(const Content& in, bool is_add, double value, const Type& outType) {
    Content out = Content::alloc(outType, VF_DT_F32, in.splat);
    Reader r(in);
    float* o = reinterpret_cast<float*>(out.mdata());
    const float c = static_cast<float>(value);
    const int64_t n = out.splat ? 1 : outType.numel();
    for (int64_t i = 0; i < n; ++i) o[i] = is_add ? r.f(i) + c : r.f(i) * c;
    return out;
}

// ConvertElemTypeAttr::transform (quant -> quant) — convert_elem_type.cpp:22-29,48-60;
// getValueRangeOffset — CD/utils/transformations.cpp:863-881; sub-byte unpacking convert_elem_type.cpp:62-79
// with subByteConversion, VC/src/utils/convert_utils.cpp:17-75.
Content sub_byte_conversion(const Content& in, const Type& outType, bool outSplat, int bits) {
    Content out = Content::alloc(outType, outType.elem.dtype, outSplat);
    const int per = 8 / bits;
    const uint8_t* src = in.ptr;
    const uint64_t nbytes = (uint64_t(bits) * uint64_t(in.splat ? 1 : in.type.numel()) + 7) / 8;
    const int64_t n = out.splat ? 1 : outType.numel();
    // the output type picks the branch; 1-bit values are always treated as unsigned (:27)
    if (outType.elem.dtype == VF_DT_U8 || bits == 1) {
        const unsigned mask = (1u << bits) - 1u;
        uint8_t* dst = out.mdata();
        if (in.splat) {
            const uint8_t first = uint8_t(src[0] & mask);  // :33-36
            for (int64_t i = 0; i < n; ++i) dst[i] = first;
        } else {
            for (uint64_t b = 0; b < nbytes; ++b)
                for (int k = 0; k < per; ++k) {
                    const int64_t o = int64_t(b) * per + k;
                    if (o < n) dst[o] = uint8_t((src[b] >> (k * bits)) & mask);
                }
        }
    } else {
        const int8_t* s8 = reinterpret_cast<const int8_t*>(src);
        int8_t* dst = reinterpret_cast<int8_t*>(out.mdata());
        const int rshift = 8 - bits;
        if (in.splat) {
            const int8_t second = int8_t(s8[0] >> rshift);  // the last element of the first byte (:53-56)
            for (int64_t i = 0; i < n; ++i) dst[i] = second;
        } else {
            for (uint64_t b = 0; b < nbytes; ++b)
                for (int k = 0; k < per; ++k) {
                    const int64_t o = int64_t(b) * per + k;
                    if (o >= n) continue;
                    const int lshift = rshift - k * bits;
                    int8_t v = int8_t(uint8_t(s8[b]) << lshift);
                    v = int8_t(v >> rshift);
                    dst[o] = v;
                }
        }
    }
    return out;
}

Content tf_convert(const Content& in, const vf_transform& t) {
    bool osplat;
    const Type outType = infer_one(in.type, in.splat, t, osplat);
    const Elem& qi = in.type.elem;
    const Elem& qo = outType.elem;
    if (!qi.quantized() && !qo.quantized()) {
        const int bits = dtype_bits(qi.dtype);
        const bool out_byte = qo.dtype == VF_DT_I8 || qo.dtype == VF_DT_U8;
        const bool same_sign = dtype_is_signed_int(qi.dtype) == dtype_is_signed_int(qo.dtype);
        if (dtype_is_int(qi.dtype) && bits < 8 && out_byte && (same_sign || bits == 1) && in.storage == qi.dtype)
            return sub_byte_conversion(in, outType, osplat, bits);
        fail(VF_ERR_UNSUPPORTED, "Unsupported conversion");
    }
    if (qi.quantized() && qo.quantized()) {
        if (!dtype_is_int(qi.dtype) || !dtype_is_int(qo.dtype) || dtype_bits(qi.dtype) != dtype_bits(qo.dtype))
            fail(VF_ERR_UNSUPPORTED, "Unsupported conversion");
        if (!all_equal(qi.zps) || !all_equal(qo.zps)) fail(VF_ERR_UNSUPPORTED, "Unsupported conversion");
        const int64_t offset = qo.zps[0] - qi.zps[0];
        return tf_rescale_add(in, true, double(offset), outType);
    }
    fail(VF_ERR_UNSUPPORTED, "Unsupported conversion");
}

void strides_of(const int64_t* shape, int rank, int64_t* st) {
    int64_t s = 1;
    for (int i = rank - 1; i >= 0; --i) {
        st[i] = s;
        s *= shape[i];
    }
}

// memPermuteTransformation — CD/utils/transformations.cpp:889-939 (generic per-element form; the optimised
// NCHW<->NHWC routine, mem_permute_optimized.cpp:58-101, produces the same bytes)
Content move_buffer(Content& in, const Type& type);

Content tf_permute(Content& in, const Type& outType, const int* memPerm, int nthreads) {
    bool identity = true;
    for (int i = 0; i < in.type.rank; ++i) identity &= memPerm[i] == i;
    if (in.splat || identity) {  // :898-899 moveBuffer
        return move_buffer(in, outType);
    }
    Content out = Content::alloc(outType, in.storage, false);
    if (out.nbytes != in.nbytes) fail(VF_ERR_SHAPE, "Storage buffer size mismatch in 'memPermuteTransformation'");
    const int es = dtype_bits(in.storage) / 8;
    if (es < 1) fail(VF_ERR_UNSUPPORTED, "sub-byte permute");
    const int rank = in.type.rank;
    int64_t ims[VF_MAX_RANK], oms[VF_MAX_RANK], ost[VF_MAX_RANK];
    mem_shape(in.type, ims);
    for (int i = 0; i < rank; ++i) oms[i] = ims[memPerm[i]];
    strides_of(oms, rank, ost);
    // out mem dim i takes in mem dim memPerm[i]  => in mem dim j contributes stride ost[inv[j]]
    int64_t contrib[VF_MAX_RANK];
    for (int i = 0; i < rank; ++i) contrib[memPerm[i]] = ost[i];
    const int64_t n = in.type.numel();
    parallel_nd(nthreads, {n}, [&](const int64_t* b, const int64_t* e) {
        for (int64_t lin = b[0]; lin < e[0]; ++lin) {
            int64_t rem = lin, o = 0;
            for (int d = rank - 1; d >= 0; --d) {
                const int64_t c = rem % ims[d];
                rem /= ims[d];
                o += c * contrib[d];
            }
            memcpy(out.mdata() + o * es, in.data() + lin * es, size_t(es));
        }
    });
    return out;
}

// ReorderAttr::transform — reorder.cpp:79-99: memPerm maps input memory dims onto the output order
Content tf_reorder(Content& in, const vf_transform& t, int nthreads) {
    bool osplat;
    const Type outType = infer_one(in.type, in.splat, t, osplat);
    int ip[VF_MAX_RANK], op[VF_MAX_RANK], mp[VF_MAX_RANK];
    order_to_perm(in.type.order, in.type.rank, ip);
    order_to_perm(outType.order, outType.rank, op);
    for (int i = 0; i < in.type.rank; ++i)
        for (int j = 0; j < in.type.rank; ++j)
            if (ip[j] == op[i]) mp[i] = j;
    return tf_permute(in, outType, mp, nthreads);
}

Content tf_mem_permute(Content& in, const vf_transform& t, int nthreads) {
    bool osplat;
    const Type outType = infer_one(in.type, in.splat, t, osplat);
    int mp[VF_MAX_RANK];
    if (t.kind == VF_T_TRANSPOSE) {
        // Transpose keeps the layout and permutes logical dims: memory dims move with them (transpose.cpp:96-104)
        int ip[VF_MAX_RANK], p[VF_MAX_RANK];
        order_to_perm(in.type.order, in.type.rank, ip);
        order_to_perm(t.order, in.type.rank, p);
        for (int i = 0; i < in.type.rank; ++i) {
            const int outLogical = ip[i];         // out mem dim i holds out logical dim ip[i]
            const int inLogical = p[outLogical];  // which is input logical dim p[.]
            for (int j = 0; j < in.type.rank; ++j)
                if (ip[j] == inLogical) mp[i] = j;
        }
    } else {
        order_to_perm(t.mem_perm, in.type.rank, mp);
    }
    return tf_permute(in, outType, mp, nthreads);
}

// Content::fillWithZero — CD/utils/content.cpp:190-237
void fill_with_zero(Content& c) {
    const Elem& e = c.type.elem;
    auto put = [&](int64_t idx, int64_t zp) {
        switch (c.storage) {
        case VF_DT_F32: {
            float f = float(zp);
            if (int64_t(f) != zp) fail(VF_ERR_CHECKED_CAST, "zero point not representable");
            memcpy(c.mdata() + idx * 4, &f, 4);
            break;
        }
        case VF_DT_F16: {
            uint16_t h = f32_to_f16(float(zp));
            memcpy(c.mdata() + idx * 2, &h, 2);
            break;
        }
        case VF_DT_BF16: {
            uint16_t h = f32_to_bf16(float(zp));
            memcpy(c.mdata() + idx * 2, &h, 2);
            break;
        }
        default: {
            double lo, hi;
            int_limits(c.storage, lo, hi);
            if (double(zp) < lo || double(zp) > hi) fail(VF_ERR_CHECKED_CAST, "zero point outside storage type");
            store_int(c.mdata(), c.storage, idx, zp);
        }
        }
    };
    if (e.kind == VF_ELEM_QUANT_PER_AXIS) {
        if (c.type.rank != 4) fail(VF_ERR_UNSUPPORTED, "Unsupported shape size %d", c.type.rank);
        if (e.axis != 0) fail(VF_ERR_UNSUPPORTED, "Only per-channel quantization is supported");
        int perm[VF_MAX_RANK];
        int64_t ms[VF_MAX_RANK], st[VF_MAX_RANK];
        order_to_perm(c.type.order, 4, perm);
        mem_shape(c.type, ms);
        strides_of(ms, 4, st);
        int64_t lst[4];  // stride of each logical dim
        for (int i = 0; i < 4; ++i) lst[perm[i]] = st[i];
        for (int64_t oc = 0; oc < c.type.shape[0]; ++oc)
            for (int64_t ic = 0; ic < c.type.shape[1]; ++ic)
                for (int64_t h = 0; h < c.type.shape[2]; ++h)
                    for (int64_t w = 0; w < c.type.shape[3]; ++w)
                        put(oc * lst[0] + ic * lst[1] + h * lst[2] + w * lst[3], e.zps[size_t(oc)]);
    } else if (e.kind == VF_ELEM_QUANT_UNIFORM) {
        const int64_t n = int64_t(c.nbytes) / (dtype_bits(c.storage) / 8);
        for (int64_t i = 0; i < n; ++i) put(i, e.zps[0]);
    } else {
        std::fill(c.own.begin(), c.own.end(), uint8_t(0));
    }
}

// PadWithZeroAttr::transform — pad_with_zero.cpp:111-268 (generic form :244-264; the 1..4-D fast paths
// compute the same indices)
Content tf_pad(const Content& in, const vf_transform& t, int nthreads) {
    bool osplat;
    const Type outType = infer_one(in.type, in.splat, t, osplat);
    Content out = Content::alloc(outType, in.storage, false);
    fill_with_zero(out);
    const int es = dtype_bits(in.storage) / 8;
    if (es < 1) fail(VF_ERR_UNSUPPORTED, "sub-byte pad");
    const int rank = in.type.rank;
    int perm[VF_MAX_RANK];
    int64_t ims[VF_MAX_RANK], oms[VF_MAX_RANK], ost[VF_MAX_RANK], mpad[VF_MAX_RANK];
    order_to_perm(in.type.order, rank, perm);
    mem_shape(in.type, ims);
    mem_shape(outType, oms);
    strides_of(oms, rank, ost);
    for (int i = 0; i < rank; ++i) mpad[i] = t.a[perm[i]];
    const int64_t n = in.type.numel();
    parallel_nd(nthreads, {n}, [&](const int64_t* b, const int64_t* e) {
        for (int64_t lin = b[0]; lin < e[0]; ++lin) {
            int64_t rem = lin, o = 0;
            for (int d = rank - 1; d >= 0; --d) {
                const int64_t c = rem % ims[d];
                rem /= ims[d];
                o += (c + mpad[d]) * ost[d];
            }
            const int64_t src = in.splat ? 0 : lin;
            memcpy(out.mdata() + o * es, in.data() + src * es, size_t(es));
        }
    });
    return out;
}

// SubViewAttr::transform — subview.cpp:390-432 (byte-sized storage only here)
Content tf_subview(Content& in, const vf_transform& t, int nthreads) {
    bool osplat;
    const Type outType = infer_one(in.type, in.splat, t, osplat);
    if (in.splat) {
        return move_buffer(in, outType);
    }
    Content out = Content::alloc(outType, in.storage, false);
    const int es = dtype_bits(in.storage) / 8;
    const int rank = in.type.rank;
    int perm[VF_MAX_RANK];
    int64_t ims[VF_MAX_RANK], oms[VF_MAX_RANK], ist[VF_MAX_RANK], moff[VF_MAX_RANK];
    order_to_perm(in.type.order, rank, perm);
    mem_shape(in.type, ims);
    mem_shape(outType, oms);
    strides_of(ims, rank, ist);
    for (int i = 0; i < rank; ++i) moff[i] = t.a[perm[i]];
    const int64_t n = outType.numel();
    if (es < 1) {  // subByteTransform — subview.cpp:20-160: bit fields, low bits first, into a zeroed buffer
        const int storageElemTypeSize = dtype_bits(in.storage);
        const int64_t elemPerByte = 8 / storageElemTypeSize;
        const unsigned mask = (1u << storageElemTypeSize) - 1u;
        std::memset(out.mdata(), 0, out.nbytes);
        for (int64_t outMemInd1D = 0; outMemInd1D < n; ++outMemInd1D) {
            int64_t rem = outMemInd1D, inMemInd1D = 0;
            for (int d = rank - 1; d >= 0; --d) {
                inMemInd1D += (rem % oms[d] + moff[d]) * ist[d];
                rem /= oms[d];
            }
            const unsigned subByteValue = (unsigned(in.data()[inMemInd1D / elemPerByte]) >> ((inMemInd1D % elemPerByte) * storageElemTypeSize)) & mask;
            out.mdata()[outMemInd1D / elemPerByte] |= uint8_t(subByteValue << ((outMemInd1D % elemPerByte) * storageElemTypeSize));
        }
        return out;
    }
    parallel_nd(nthreads, {n}, [&](const int64_t* b, const int64_t* e) {
        for (int64_t lin = b[0]; lin < e[0]; ++lin) {
            int64_t rem = lin, s = 0;
            for (int d = rank - 1; d >= 0; --d) {
                const int64_t c = rem % oms[d];
                rem /= oms[d];
                s += (c + moff[d]) * ist[d];
            }
            memcpy(out.mdata() + lin * es, in.data() + s * es, size_t(es));
        }
    });
    return out;
}

// BitPackAttr::transform — bit_pack.cpp:132-154; values are read through getValues<uint8_t>()
Content tf_bitpack(const Content& in, const vf_transform& t) {
    bool osplat;
    if (in.splat) fail(VF_ERR_SPLAT, "Bit pack does not support splat inputs.");
    const Type outType = infer_one(in.type, in.splat, t, osplat);
    const int64_t n = in.type.numel();
    if (n % 2 != 0) fail(VF_ERR_ODD_COUNT, "Storage buffer size is odd, which is unexpected for 4 bit packing.");
    Content out = Content::alloc(outType, VF_DT_U8, false, int64_t(type_bytes(outType)));
    Reader r(in);
    for (int64_t i = 0; i < n; i += 2) {
        const uint8_t lsn = uint8_t(r.i64(i, VF_DT_U8)) & 0x0f;
        const uint8_t msn = uint8_t(r.i64(i + 1, VF_DT_U8)) & 0x0f;
        out.mdata()[i / 2] = uint8_t((msn << 4) + lsn);
    }
    return out;
}

// getSparsifyValue — VC/src/utils/sparsity.cpp:12-26
int64_t sparsify_value(const Elem& e) {
    if (e.kind == VF_ELEM_QUANT_UNIFORM) return e.zps[0];
    if (e.kind == VF_ELEM_QUANT_PER_AXIS) {
        if (!all_equal(e.zps)) fail(VF_ERR_ZERO_POINTS, "Not all zero-points are equal");
        return e.zps[0];
    }
    return 0;
}

// Element of the logical storage type (i8/u8/f16/bf16/f32) read through getValues<StorageType>() and compared
// with checked_cast<StorageType>(sparsifyValue); floating types compare as float, so -0.0 equals 0.
struct SparseElem {
    bool is_zero;
    uint8_t bytes[4];
};

struct SparseReader {
    Reader r;
    int dt;
    int es;
    float fval;
    int64_t ival;
    SparseReader(const Content& c, int64_t value): r(c), dt(c.type.elem.dtype) {
        const bool f8 = dt == VF_DT_F8E4M3FN || dt == VF_DT_F8E5M2;  // sparsify.cpp:197-200, get_sparsity_map.cpp:111-116
        if (dt != VF_DT_I8 && dt != VF_DT_U8 && dt != VF_DT_F16 && dt != VF_DT_BF16 && dt != VF_DT_F32 && !f8)
            fail(VF_ERR_UNSUPPORTED, "Unexpected weights data type");
        if (f8 && value != 0) fail(VF_ERR_UNSUPPORTED, "8-bit float storage with a non-zero zero point");
        es = dtype_bits(dt) / 8;
        ival = value;
        if (dt == VF_DT_I8 && (value < -128 || value > 127)) fail(VF_ERR_CHECKED_CAST, "sparsify value outside i8");
        if (dt == VF_DT_U8 && (value < 0 || value > 255)) fail(VF_ERR_CHECKED_CAST, "sparsify value outside u8");
        fval = float(value);
        if (dt == VF_DT_F16) fval = f16_to_f32(f32_to_f16(fval));
        if (dt == VF_DT_BF16) fval = bf16_to_f32(f32_to_bf16(fval));
    }
    SparseElem at(int64_t i) const {
        SparseElem e{};
        switch (dt) {
        case VF_DT_I8:
        case VF_DT_U8: {
            const int64_t v = r.i64(i, dt);
            e.bytes[0] = uint8_t(v);
            e.is_zero = v == ival;
            break;
        }
        case VF_DT_F16: {
            const uint16_t h = f32_to_f16_clamped(r.f(i));
            memcpy(e.bytes, &h, 2);
            e.is_zero = f16_to_f32(h) == fval;
            break;
        }
        case VF_DT_BF16: {
            const uint16_t h = f32_to_bf16(r.f(i));
            memcpy(e.bytes, &h, 2);
            e.is_zero = bf16_to_f32(h) == fval;
            break;
        }
        case VF_DT_F8E4M3FN: {
            e.bytes[0] = f32_to_f8e4m3(r.f(i));
            e.is_zero = f8e4m3_to_f32(e.bytes[0]) == fval;
            break;
        }
        case VF_DT_F8E5M2: {
            e.bytes[0] = f32_to_f8e5m2(r.f(i));
            e.is_zero = f8e5m2_to_f32(e.bytes[0]) == fval;
            break;
        }
        default: {
            const float f = r.f(i);
            memcpy(e.bytes, &f, 4);
            e.is_zero = f == fval;
        }
        }
        return e;
    }
};

// countNonSparseElementsPerOC — VC/src/utils/sparsity.cpp:35-84
std::vector<int64_t> count_nnz(const Content& in, int nthreads) {
    if (in.type.rank != 4) fail(VF_ERR_SHAPE, "Const::Content::sparsify: got unxpected content shape %d", in.type.rank);
    const int64_t OC = in.type.shape[0], work = in.type.shape[1] * in.type.shape[2] * in.type.shape[3];
    SparseReader sr(in, sparsify_value(in.type.elem));
    std::vector<int64_t> counts(size_t(OC), 0);
    parallel_nd(nthreads, {OC}, [&](const int64_t* b, const int64_t* e) {
        for (int64_t oc = b[0]; oc < e[0]; ++oc) {
            int64_t c = 0;
            for (int64_t i = oc * work; i < (oc + 1) * work; ++i) c += sr.at(i).is_zero ? 0 : 1;
            counts[size_t(oc)] = c;
        }
    });
    return counts;
}

// SparsifyAttr::transform — CD/attributes/sparsify.cpp:120-203
Content tf_sparsify(const Content& in, const vf_transform& t, int nthreads) {
    if (in.type.rank != 4) fail(VF_ERR_SHAPE, "Expected 4D input shape");
    std::vector<int64_t> counts = t.num_actual ? std::vector<int64_t>(t.num_actual, t.num_actual + t.n_num_actual)
                                               : count_nnz(in, nthreads);
    for (auto c : counts)
        if (c < 0) fail(VF_ERR_INVALID_ARG, "Got negative elem number value in 'numActualElements'");
    const Type outType = compress_type(in.type, counts);
    Content out = Content::alloc(outType, VF_DT_U8, false);
    const int64_t OC = in.type.shape[0], work = in.type.shape[1] * in.type.shape[2] * in.type.shape[3];
    SparseReader sr(in, sparsify_value(in.type.elem));
    const int64_t es = sr.es;
    int64_t outIdx = 0;  // in elements
    for (int64_t oc = 0; oc < OC; ++oc) {
        for (int64_t i = oc * work; i < (oc + 1) * work; ++i) {
            const SparseElem e = sr.at(i);
            if (e.is_zero) continue;
            if (uint64_t((outIdx + 1) * es) > out.nbytes) fail(VF_ERR_SHAPE, "numActualElements too small");
            memcpy(out.mdata() + outIdx * es, e.bytes, size_t(es));
            ++outIdx;
        }
        const int64_t byteIdx = outIdx * es;
        if (byteIdx % 16 != 0) outIdx = align_up(byteIdx, 16) / es;
    }
    return out;
}

// GetSparsityMapAttr::transform — CD/attributes/get_sparsity_map.cpp:21-57,82-119
Content tf_sparsity_map(const Content& in, const vf_transform& t) {
    bool osplat;
    const Type outType = infer_one(in.type, in.splat, t, osplat);
    const int64_t OC = outType.shape[0];
    const int64_t inWork = in.type.shape[1] * in.type.shape[2] * in.type.shape[3];
    const int64_t outWork = outType.shape[3];
    Content out = Content::alloc(outType, VF_DT_I1, false);
    SparseReader sr(in, sparsify_value(in.type.elem));
    if (inWork % 8 != 0)  // the reference loop reads bits of the next channel in this case; rejected instead
        fail(VF_ERR_SHAPE, "GetSparsityMap needs IC*KY*KX to be a multiple of 8");
    for (int64_t oc = 0; oc < OC; ++oc) {
        int64_t outIdx = oc * outWork / 8;
        for (int64_t i = 0; i < inWork; i += 8) {
            uint8_t byte = 0;
            for (int b = 0; b < 8; ++b)
                if (!sr.at(oc * inWork + i + b).is_zero) byte |= uint8_t(1u << b);
            out.mdata()[outIdx++] = byte;
        }
    }
    return out;
}

Content move_buffer(Content& in, const Type& type) {  // Content::moveBuffer — CD/utils/content.cpp:54-58
    Content out = std::move(in);
    if (!out.own.empty()) out.ptr = out.own.data();
    out.type = type;
    return out;
}

uint64_t copy_to(const Content& c, uint8_t* dst, uint64_t dst_bytes);

// SwizzleConstantAttr::transform — CD/attributes/swizzle_transform.cpp:163-215 with
// BufferSwizzleTransform::swizzle (VC/include/vpux/compiler/utils/swizzle_transform.hpp:56-76) and
// AddressTransform (swizzle_transform.cpp:37-83)
Content tf_swizzle(const Content& in, const vf_transform& t) {
    bool osplat;
    const Type outType = infer_one(in.type, in.splat, t, osplat);
    const uint32_t key = uint32_t(t.a[0]);
    const bool npu40 = t.a[1] == VF_ARCH_NPU40XX;
    const uint64_t inTotal = type_bytes(in.type);
    const uint64_t newSize = uint64_t(align_up(int64_t(inTotal), npu40 ? 1024 : 512));
    std::vector<uint8_t> values(newSize, 0);
    copy_to(in, values.data(), inTotal);
    if (newSize > inTotal) {
        const uint8_t pad = in.splat ? values[0] : uint8_t(0);
        std::fill(values.begin() + long(inTotal), values.end(), pad);
    }
    Content out = Content::alloc(outType, outType.elem.dtype, false, int64_t(newSize));
    if (in.splat) {
        std::memcpy(out.mdata(), values.data(), newSize);
        return out;
    }
    // setStaggerBits
    const uint32_t staggerBits = key % 6u;
    const uint32_t staggerMask = (1u << staggerBits) - 1u;
    uint32_t shift = 9u - staggerBits, log2Width = 4u, ramCutMask = (1u << 9) - 1u;
    if (npu40) {
        ++shift;
        ++log2Width;
        ramCutMask = (1u << 10) - 1u;
    }
    const uint32_t width = 1u << log2Width;
    const uint64_t iterations = ((newSize + width - 1) >> log2Width);
    uint32_t dpuAddr = 0;
    for (uint64_t i = 0; i < iterations; ++i) {
        uint32_t stagger = dpuAddr >> log2Width;  // getPhysicalAddress
        stagger &= (1u << 11) - 1u;
        stagger >>= 5;
        stagger &= staggerMask;
        stagger <<= shift;
        uint32_t phy = dpuAddr + stagger;
        phy &= ramCutMask;
        phy += dpuAddr & ~ramCutMask;
        std::memcpy(out.mdata() + phy, values.data() + dpuAddr, width);
        dpuAddr += width;
    }
    return out;
}

// ReverseAttr::transform — CD/attributes/reverse.cpp:46-105
Content tf_reverse(Content& in, const vf_transform& t) {
    bool osplat;
    const Type outType = infer_one(in.type, in.splat, t, osplat);
    if (in.splat) return move_buffer(in, outType);
    int64_t spatialDims = 1;
    for (int i = in.type.rank - 1; i > t.a[0]; --i) spatialDims *= in.type.shape[i];
    Content out = Content::alloc(outType, outType.elem.dtype, false);
    const uint64_t es = uint64_t(dtype_bits(outType.elem.dtype) / 8);
    copy_to(in, out.mdata(), type_bytes(in.type));  // getValues<StorageType>() copied into the new buffer
    const int64_t n = outType.numel();
    uint8_t* p = out.mdata();
    std::vector<uint8_t> tmp(es);
    for (int64_t first = 0; first + spatialDims <= n; first += spatialDims)
        for (int64_t lo = first, hi = first + spatialDims - 1; lo < hi; ++lo, --hi) {
            std::memcpy(tmp.data(), p + uint64_t(lo) * es, es);
            std::memcpy(p + uint64_t(lo) * es, p + uint64_t(hi) * es, es);
            std::memcpy(p + uint64_t(hi) * es, tmp.data(), es);
        }
    return out;
}

// BroadcastAttr::transform — CD/attributes/broadcast.cpp:85-124
Content tf_broadcast(Content& in, const vf_transform& t) {
    bool osplat;
    const Type outType = infer_one(in.type, in.splat, t, osplat);
    if (in.splat) return move_buffer(in, outType);  // the single element is copied (:91-93)
    if (dtype_bits(in.storage) < 8) fail(VF_ERR_UNSUPPORTED, "Broadcast of sub-byte storage");
    Content out = Content::alloc(outType, in.storage, false);
    int perm[VF_MAX_RANK];
    int64_t ms[VF_MAX_RANK];
    order_to_perm(in.type.order ? in.type.order : identity_order(in.type.rank), in.type.rank, perm);
    for (int i = 0; i < in.type.rank; ++i) ms[i] = in.type.shape[perm[i]];
    int index = 0;
    for (int i = 0; i < in.type.rank; ++i)
        if (perm[i] == t.a[0]) index = i;
    int64_t preDims = 1, afterDims = 1;
    for (int i = 0; i < index; ++i) preDims *= ms[i];
    for (int i = index; i < in.type.rank; ++i) afterDims *= ms[i];
    const int64_t expandDim = ms[index], value = t.a[1];
    if (expandDim == 0 || value % expandDim) fail(VF_ERR_SHAPE, "Can't broadcast from %lld to %lld", (long long)expandDim, (long long)value);
    const int64_t factor = value / expandDim;
    const uint64_t singleCopySize = uint64_t(afterDims) * uint64_t(dtype_bits(in.storage) / 8);
    for (int64_t pre = 0; pre < preDims; ++pre)
        for (int64_t f = 0; f < factor; ++f)
            std::memcpy(out.mdata() + singleCopySize * uint64_t(pre * factor + f), in.ptr + singleCopySize * uint64_t(pre), singleCopySize);
    return out;
}

// ExpandDilatedAttr::transform — CD/attributes/expand_dilated.cpp:88-131
Content tf_expand_dilated(const Content& in, const vf_transform& t) {
    bool osplat;
    const Type outType = infer_one(in.type, in.splat, t, osplat);
    if (dtype_bits(in.storage) < 8) fail(VF_ERR_UNSUPPORTED, "ExpandDilated of sub-byte storage");
    Content out = Content::alloc(outType, in.storage, false);
    fill_with_zero(out);
    const uint64_t es = uint64_t(dtype_bits(in.storage) / 8);
    const int64_t OC = in.type.shape[0], IC = in.type.shape[1], KY = in.type.shape[2], KX = in.type.shape[3];
    const int64_t dKY = outType.shape[2], dKX = outType.shape[3];
    for (int64_t oc = 0; oc < OC; ++oc)
        for (int64_t ic = 0; ic < IC; ++ic)
            for (int64_t ky = 0; ky < KY; ++ky)
                for (int64_t kx = 0; kx < KX; ++kx) {
                    const int64_t dky = ky + (t.a[0] - 1) * ky, dkx = kx + (t.a[1] - 1) * kx;
                    const int64_t outRawInd = dkx + dky * dKX + ic * dKX * dKY + oc * dKX * dKY * IC;
                    const int64_t inRawInd = kx + ky * KX + ic * KX * KY + oc * KX * KY * IC;
                    std::memcpy(out.mdata() + uint64_t(outRawInd) * es, in.ptr + (in.splat ? 0 : uint64_t(inRawInd) * es), es);
                }
    return out;
}

// ScalarMultInverseAttr::transform — CD/attributes/inverse.cpp:52-66
Content tf_inverse(const Content& in, const vf_transform& t) {
    bool osplat;
    const Type outType = infer_one(in.type, in.splat, t, osplat);
    Content out = Content::alloc(outType, VF_DT_F32, in.splat);
    Reader r(in);
    float* o = reinterpret_cast<float*>(out.mdata());
    const int64_t n = out.splat ? 1 : outType.numel();
    for (int64_t i = 0; i < n; ++i) {
        const float v = r.f(i);
        if (!std::isnormal(v)) fail(VF_ERR_NOT_NORMAL, "Taking inverse of a non-normal (e.g. zero/nan/...) float");
        o[i] = 1.f / v;
    }
    return out;
}

// RelocateWeightsTableAttr::transform — CD/attributes/relocate_weights_table.cpp:203-292
Content tf_relocate(const Content& in, const vf_transform& t) {
    bool osplat;
    const Type outType = infer_one(in.type, in.splat, t, osplat);
    const vf_relocate& r = t.relocate;
    Content out = Content::alloc(outType, outType.elem.dtype, false);
    copy_to(in, out.mdata(), type_bytes(in.type));  // a splat is filled in (:211-213), anything else is copied
    int32_t* values = reinterpret_cast<int32_t*>(out.mdata());
    const int64_t entries = r.weights_table_size / 4;
    const int64_t perOC = 4;  // WEIGHT_TABLE_NUM_ELEMENTS_PER_OC
    uint32_t weightStep = 0, sparsityStep = 0;  // int32 in the reference; unsigned here so that overflow wraps
    if (entries >= 2 * perOC) {
        weightStep = uint32_t(values[perOC]) - uint32_t(values[0]);
        sparsityStep = uint32_t(values[perOC + 1]) - uint32_t(values[1]);
    }
    if (r.channel_offset < INT32_MIN || r.channel_offset > INT32_MAX) fail(VF_ERR_CHECKED_CAST, "channelOffset outside int32");
    const uint32_t chanOff = uint32_t(int32_t(r.channel_offset));
    uint32_t weightsPtrOffset = chanOff * weightStep;
    const uint32_t sparsityPtrOffset = chanOff * sparsityStep;
    const int64_t OC = entries / perOC;
    bool segmented = false;
    for (int c = 1; c < r.n_clusters; ++c) segmented = segmented || r.offsets[c] != r.offsets[c - 1];
    auto new_cluster = [&](int64_t oc, int cl) { return segmented && cl + 1 < r.n_clusters && oc >= r.offsets[cl + 1]; };
    std::vector<int64_t> ptrSteps(size_t(std::max<int64_t>(OC, 0)));
    if (r.num_elems) {
        if (r.channel_offset < 0 || r.n_num_elems < OC + r.channel_offset)
            fail(VF_ERR_SHAPE, "Invalid weights compression with %lld elements for %lld channels", (long long)r.n_num_elems, (long long)OC);
        if (r.weights_elem_bit_size <= 0) fail(VF_ERR_INVALID_ARG, "Missing weights element type attribute");
        const int64_t alignment = r.alignment ? r.alignment : 16;  // VPU_WEIGHT_SET_BYTE_ALIGNMENT
        if (alignment < 0) fail(VF_ERR_INVALID_ARG, "negative weightsCompression alignment");
        auto setBytes = [&](int64_t oc) { return align_up((r.num_elems[oc] * r.weights_elem_bit_size + 7) / 8, alignment); };
        int64_t sliced = 0;
        for (int64_t oc = 0; oc < r.channel_offset; ++oc) sliced += setBytes(oc);
        weightsPtrOffset = uint32_t(sliced);
        int64_t ptrOffset = 0;
        int cl = 0;
        for (int64_t oc = 0; oc < OC; ++oc) {
            if (new_cluster(oc, cl)) {
                ++cl;
                ptrOffset = 0;
            }
            ptrSteps[size_t(oc)] = ptrOffset;
            ptrOffset += setBytes(oc + r.channel_offset);
        }
    } else {
        int cl = 0;
        for (int64_t oc = 0; oc < OC; ++oc) {
            if (new_cluster(oc, cl)) ++cl;
            ptrSteps[size_t(oc)] = int64_t(int32_t(weightStep)) * (oc - r.offsets[cl]);
        }
    }
    int cl = 0;
    for (int64_t oc = 0; oc < OC; ++oc) {
        if (new_cluster(oc, cl)) ++cl;
        const int64_t w = int64_t(r.weights_ptr[cl]) + ptrSteps[size_t(oc)];
        if (w < INT32_MIN || w > INT32_MAX) fail(VF_ERR_CHECKED_CAST, "weights pointer %lld outside int32", (long long)w);
        values[oc * perOC] = int32_t(uint32_t(w) + weightsPtrOffset);
        if (values[oc * perOC + 1] != 0xFFFFFF) {  // SPARSITY_PTR_WHEN_NO_SPARSITY (nce_sparsity.hpp:34)
            const int64_t sp = int64_t(r.sparsity_ptr) + (oc - r.offsets[cl]) * int64_t(int32_t(sparsityStep));
            if (sp < INT32_MIN || sp > INT32_MAX) fail(VF_ERR_CHECKED_CAST, "sparsity pointer %lld outside int32", (long long)sp);
            values[oc * perOC + 1] = int32_t(uint32_t(sp) + sparsityPtrOffset);
        }
    }
    return out;
}

Content apply(Content& in, const vf_transform& t, int nthreads) {
    bool osplat;
    switch (t.kind) {
    case VF_T_CAST_ELEM_TYPE:
    case VF_T_RESHAPE:
    case VF_T_CHANGE_SHAPE_AND_ELEM_TYPE:  // change_shape_and_elem_type.cpp:77-79
    case VF_T_LAYOUT_CAST: {  // moveBuffer: cast_elem_type.cpp:35-37, reshape.cpp:87-89, layout_cast.cpp:82-84
        const Type ty = infer_one(in.type, in.splat, t, osplat);
        return move_buffer(in, ty);
    }
    case VF_T_CONVERT_ELEM_TYPE: return tf_convert(in, t);
    case VF_T_DEQUANTIZE: return tf_dequantize(in, t, nthreads);
    case VF_T_QUANTIZE: return tf_quantize(in, t, nthreads);
    case VF_T_RESCALE: return tf_rescale_add(in, false, t.value, in.type);
    case VF_T_ADD: return tf_rescale_add(in, true, t.value, in.type);
    case VF_T_REORDER: return tf_reorder(in, t, nthreads);
    case VF_T_MEM_PERMUTE:
    case VF_T_TRANSPOSE: return tf_mem_permute(in, t, nthreads);
    case VF_T_PAD_WITH_ZERO: return tf_pad(in, t, nthreads);
    case VF_T_SUBVIEW: return tf_subview(in, t, nthreads);
    case VF_T_BIT_PACK: return tf_bitpack(in, t);
    case VF_T_GET_SPARSITY_MAP: return tf_sparsity_map(in, t);
    case VF_T_SPARSIFY: return tf_sparsify(in, t, nthreads);
    case VF_T_SWIZZLE_CONSTANT: return tf_swizzle(in, t);
    case VF_T_RELOCATE_WEIGHTS_TABLE: return tf_relocate(in, t);
    case VF_T_REVERSE: return tf_reverse(in, t);
    case VF_T_BROADCAST: return tf_broadcast(in, t);
    case VF_T_EXPAND_DILATED: return tf_expand_dilated(in, t);
    case VF_T_SCALAR_MULT_INVERSE: return tf_inverse(in, t);
    default: fail(VF_ERR_INVALID_ARG, "unknown transformation kind %d", t.kind);
    }
}

Content wrap_base(const vf_content& b) {  // wrapBaseContent — content.cpp:310-318
    Content c;
    c.type = type_from_pod(b.type);
    c.storage = b.storage_dtype;
    c.splat = b.is_splat != 0;
    c.ptr = static_cast<const uint8_t*>(b.data);
    c.nbytes = b.nbytes;
    const uint64_t need = (uint64_t(dtype_bits(c.storage)) * uint64_t(c.splat ? 1 : c.type.numel()) + 7) / 8;
    if (!c.ptr || c.nbytes < need) fail(VF_ERR_SHAPE, "base buffer holds %llu bytes, %llu needed",
                                        (unsigned long long)c.nbytes, (unsigned long long)need);
    return c;
}

// Content::copyTo — CD/utils/content.cpp:161-184 (+ copySubByteContent :101-155, fillBuf :84-97)
uint64_t copy_to(const Content& c, uint8_t* dst, uint64_t dst_bytes) {
    const int edt = c.type.elem.dtype;
    const int bits = dtype_bits(edt);
    if (bits < 8) {
        if (c.splat) {
            const int shifts = 8 / bits;
            uint8_t sub = 0;
            if (c.storage == VF_DT_I1)
                sub = c.data()[0] & 1;
            else
                sub = uint8_t(int8_t(Reader(c).i64(0, VF_DT_I8)));
            uint8_t byte = 0;
            for (int s = 0; s < shifts; ++s) byte = uint8_t((byte << bits) + sub);
            std::fill(dst, dst + dst_bytes, byte);
            return dst_bytes;
        }
        if (dst_bytes < c.nbytes) {
            if (c.nbytes % dst_bytes != 0) fail(VF_ERR_BUFFER_TOO_SMALL, "Cannot pack sub-byte elements into buffer");
            Reader r(c);
            const uint64_t n = c.nbytes / uint64_t(dtype_bits(c.storage) / 8);
            const uint64_t perByte = n / dst_bytes;
            if (perByte > 8 || (perByte & (perByte - 1)) != 0) fail(VF_ERR_SHAPE, "Invalid number of elements per byte");
            const int b = int(8 / perByte);
            const uint8_t mask = uint8_t((1u << b) - 1);
            for (uint64_t idx = 0; idx < n; idx += perByte) {
                uint8_t byte = 0, shift = 0;
                for (uint64_t k = 0; k < perByte; ++k) {
                    byte |= uint8_t((uint8_t(int8_t(r.i64(int64_t(idx + k), VF_DT_I8))) & mask) << shift);
                    shift = uint8_t(shift + b);
                }
                dst[idx / perByte] = byte;
            }
            return dst_bytes;
        }
        memcpy(dst, c.data(), c.nbytes);
        return c.nbytes;
    }
    const bool trivial = edt == c.storage;
    if (!c.splat && trivial) {
        if (dst_bytes < c.nbytes)
            fail(VF_ERR_BUFFER_TOO_SMALL, "Byte sizes of the target buffer '%llu' is smaller then storage buffer '%llu'",
                 (unsigned long long)dst_bytes, (unsigned long long)c.nbytes);
        memcpy(dst, c.data(), c.nbytes);
        return c.nbytes;
    }
    const int64_t n = c.type.numel();
    const uint64_t need = uint64_t(n) * uint64_t(bits / 8);
    if (dst_bytes < need) fail(VF_ERR_BUFFER_TOO_SMALL, "Buffer is not enough to hold actual elements");
    Reader r(c);
    for (int64_t i = 0; i < n; ++i) {
        switch (edt) {
        case VF_DT_F32: {
            const float f = r.f(i);
            memcpy(dst + i * 4, &f, 4);
            break;
        }
        case VF_DT_F16: {
            const uint16_t h = f32_to_f16_clamped(r.f(i));
            memcpy(dst + i * 2, &h, 2);
            break;
        }
        case VF_DT_BF16: {
            const uint16_t h = f32_to_bf16(r.f(i));
            memcpy(dst + i * 2, &h, 2);
            break;
        }
        case VF_DT_F8E4M3FN: dst[i] = f32_to_f8e4m3(r.f(i)); break;  // CvtHelper<float8_e4m3>, content.hpp:66-71
        case VF_DT_F8E5M2: dst[i] = f32_to_f8e5m2(r.f(i)); break;    // CvtHelper<float8_e5m2>, content.hpp:74-79
        case VF_DT_F64: {
            const Val v = r.at(i);
            const double d = v.is_float ? v.f : (v.is_unsigned ? double(v.u) : double(v.i));
            memcpy(dst + i * 8, &d, 8);
            break;
        }
        default: store_int(dst, edt, i, r.i64(i, edt));
        }
    }
    return need;
}

void export_type(const Type& t, vf_tensor_type* out, double* sb, int64_t* zb, int64_t cap) {
    if (!out) return;
    memset(out, 0, sizeof(*out));
    out->rank = t.rank;
    out->order = t.order;
    for (int i = 0; i < t.rank; ++i) out->shape[i] = t.shape[i];
    out->elem.kind = t.elem.kind;
    out->elem.dtype = t.elem.dtype;
    out->elem.expressed = t.elem.expressed;
    out->elem.axis = t.elem.axis;
    out->elem.qmin = t.elem.qmin;
    out->elem.qmax = t.elem.qmax;
    out->elem.nparams = int64_t(t.elem.scales.size());
    if (t.elem.quantized()) {
        if (!sb || !zb || cap < int64_t(t.elem.scales.size()))
            fail(VF_ERR_BUFFER_TOO_SMALL, "parameter buffers too small for the result type");
        std::copy(t.elem.scales.begin(), t.elem.scales.end(), sb);
        std::copy(t.elem.zps.begin(), t.elem.zps.end(), zb);
        out->elem.scales = sb;
        out->elem.zps = zb;
    }
}

// ---------------------------------------------------------------------------------------------
// row statistics → parameters
// ---------------------------------------------------------------------------------------------
void unit_geometry(const Type& t, const vf_quant_spec& s, int64_t& units, int64_t& unit_len) {
    const int64_t n = t.numel();
    if (s.group_size > 0) {
        const int64_t cols = t.shape[t.rank - 1];
        if (t.order != identity_order(t.rank)) fail(VF_ERR_UNSUPPORTED, "group quantization needs a row-major tensor");
        if (cols % s.group_size != 0) fail(VF_ERR_SHAPE, "group size does not divide the row length");
        unit_len = s.group_size;
        units = n / unit_len;
    } else {
        if (t.order != identity_order(t.rank)) fail(VF_ERR_UNSUPPORTED, "per-channel statistics need dim 0 outermost");
        units = t.shape[0];
        unit_len = units ? n / units : 0;
    }
}

void derive_params(const Content& in, const vf_quant_spec& s, std::vector<double>& scales, std::vector<int64_t>& zps,
                   std::vector<float>& mins, std::vector<float>& maxs, int nthreads) {
    int64_t units, len;
    unit_geometry(in.type, s, units, len);
    scales.assign(size_t(units), 0.0);
    zps.assign(size_t(units), 0);
    mins.assign(size_t(units), 0.f);
    maxs.assign(size_t(units), 0.f);
    Reader r(in);
    std::vector<int> bad(size_t(units), 0);
    parallel_nd(nthreads, {units}, [&](const int64_t* b, const int64_t* e) {
        for (int64_t u = b[0]; u < e[0]; ++u) {
            float mn = 0.f, mx = 0.f;  // the range always contains zero (calcScaleAndZeroPoint requires it)
            for (int64_t i = 0; i < len; ++i) {
                const float v = r.f(u * len + i);
                mn = v < mn ? v : mn;
                mx = v > mx ? v : mx;
            }
            if (s.range_mode == VF_RANGE_ABSMAX) {
                const float a = std::max(-mn, mx);
                mn = -a;
                mx = a;
            }
            mins[size_t(u)] = mn;
            maxs[size_t(u)] = mx;
            double sc;
            int64_t zp;
            if (!calc_scale_zp(double(s.qmin), double(s.qmax), double(mn), double(mx), sc, zp)) {
                bad[size_t(u)] = 1;
                continue;
            }
            zp = std::min(std::max(zp, s.qmin), s.qmax);
            scales[size_t(u)] = sc;
            zps[size_t(u)] = zp;
        }
    });
    for (auto b : bad)
        if (b) fail(VF_ERR_QUANT_RANGE, "calcScaleAndZeroPoint failed for a unit");
}

// ---------------------------------------------------------------------------------------------
// synthetic weights
// ---------------------------------------------------------------------------------------------
uint64_t mix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
// IEEE 754 round-to-nearest-even binary32 -> binary16 (the generator's definition; NOT the reference's
// float16 class, which deviates from IEEE for some subnormal results). No NaN/Inf reaches this.
uint16_t rne_f16(float f) {
    const uint32_t u = f2u(f);
    const uint32_t sign = (u >> 16) & 0x8000u;
    const int32_t e = int32_t((u >> 23) & 0xFF) - 127 + 15;
    uint32_t m = u & 0x7FFFFFu;
    if (e >= 31) return uint16_t(sign | 0x7C00u);
    if (e <= 0) {
        if (e < -10) return uint16_t(sign);
        m |= 0x800000u;
        const int sh = 14 - e;
        uint32_t r = m >> sh;
        const uint32_t rem = m & ((1u << sh) - 1u), half = 1u << (sh - 1);
        if (rem > half || (rem == half && (r & 1u))) ++r;
        return uint16_t(sign | r);
    }
    uint32_t r = (uint32_t(e) << 10) | (m >> 13);
    const uint32_t rem = m & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (r & 1u))) ++r;
    return uint16_t(sign | r);
}
uint16_t rne_bf16(float f) {
    const uint32_t u = f2u(f);
    return uint16_t((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);
}

}  // namespace

// =================================================================================================
// C entry points
// =================================================================================================
extern "C" {

uint16_t orc_f32_to_f16(uint32_t b) {
    return f32_to_f16(u2f(b));
}
uint32_t orc_f16_to_f32(uint16_t h) {
    return f2u(f16_to_f32(h));
}
uint16_t orc_f32_to_bf16(uint32_t b) {
    return f32_to_bf16(u2f(b));
}
uint32_t orc_bf16_to_f32(uint16_t h) {
    return f2u(bf16_to_f32(h));
}
uint16_t orc_f32_to_f16_clamped(uint32_t b) {
    return f32_to_f16_clamped(u2f(b));
}

uint8_t orc_f32_to_f8e4m3(uint32_t b) {
    return f32_to_f8e4m3(u2f(b));
}
uint32_t orc_f8e4m3_to_f32(uint8_t v) {
    return f2u(f8e4m3_to_f32(v));
}
uint8_t orc_f32_to_f8e5m2(uint32_t b) {
    return f32_to_f8e5m2(u2f(b));
}
uint32_t orc_f8e5m2_to_f32(uint8_t v) {
    return f2u(f8e5m2_to_f32(v));
}

void orc_f32_to_f16_n(const uint32_t* in, uint16_t* out, uint64_t n) {
    for (uint64_t i = 0; i < n; ++i) out[i] = f32_to_f16(u2f(in[i]));
}
void orc_f32_to_bf16_n(const uint32_t* in, uint16_t* out, uint64_t n) {
    for (uint64_t i = 0; i < n; ++i) out[i] = f32_to_bf16(u2f(in[i]));
}

int orc_calc_scale_zp(double qmin, double qmax, double rmin, double rmax, double* scale, int64_t* zp) {
    return calc_scale_zp(qmin, qmax, rmin, rmax, *scale, *zp) ? VF_OK : VF_ERR_QUANT_RANGE;
}
float orc_fake_quantize(float v, float lo, float hi, float ql, float qh, float levels) {
    return fake_quantize(v, lo, hi, ql, qh, levels);
}
int64_t orc_quantize_value(float x, double scale, int64_t zp, int64_t qmin, int64_t qmax) {
    return Quantizer(scale, zp, qmin, qmax)(x);
}
float orc_dequantize_value(int64_t q, double scale, int64_t zp) {
    return dequantize_value(q, scale, zp);
}
int orc_mult_shift(double rescale, int32_t* word, int32_t* mult, int32_t* shift) {
    return guard(nullptr, 0, [&] {
        int32_t m, s;
        approximate15(rescale, m, s);
        if (m < -32768 || m > 32767) fail(VF_ERR_CHECKED_CAST, "mult does not fit int16");
        *mult = m;
        *shift = s;
        *word = (s << 8) | int32_t(uint32_t(m) << 16);
    });
}

int orc_infer_type(const vf_tensor_type* base, int base_is_splat, const vf_transform* t, int n, vf_tensor_type* out,
                   int* out_is_splat, double* sb, int64_t* zb, int64_t cap, uint64_t* out_bytes, char* err,
                   size_t errlen) {
    return guard(err, errlen, [&] {
        Type ty = type_from_pod(*base);
        bool splat = base_is_splat != 0;
        check_positions(t, n);
        for (int i = 0; i < n; ++i) {
            bool os;
            ty = infer_one(ty, splat, t[i], os);
            splat = os;
        }
        export_type(ty, out, sb, zb, cap);
        if (out_is_splat) *out_is_splat = splat;
        if (out_bytes) *out_bytes = type_bytes(ty);
    });
}

int orc_fold(const vf_content* base, const vf_transform* t, int n, void* dst, uint64_t dst_bytes,
             uint64_t* dst_written, vf_tensor_type* out_type, double* sb, int64_t* zb, int64_t cap, int nthreads,
             char* err, size_t errlen) {
    return guard(err, errlen, [&] {
        check_positions(t, n);
        Content c = wrap_base(*base);
        for (int i = 0; i < n; ++i) {  // ContentAttr::fold — content.cpp:392-394
            Content next = apply(c, t[i], nthreads);
            c = std::move(next);
            if (!c.own.empty()) c.ptr = c.own.data();
        }
        export_type(c.type, out_type, sb, zb, cap);
        const uint64_t w = copy_to(c, static_cast<uint8_t*>(dst), dst_bytes);
        if (dst_written) *dst_written = w;
    });
}

int orc_row_stats(const vf_content* base, const vf_quant_spec* spec, double* scales, int64_t* zps, float* rmin,
                  float* rmax, int64_t n_units, int nthreads, char* err, size_t errlen) {
    return guard(err, errlen, [&] {
        Content c = wrap_base(*base);
        std::vector<double> s;
        std::vector<int64_t> z;
        std::vector<float> mn, mx;
        derive_params(c, *spec, s, z, mn, mx, nthreads);
        if (int64_t(s.size()) != n_units) fail(VF_ERR_SHAPE, "n_units mismatch: %lld vs %zu", (long long)n_units, s.size());
        if (scales) std::copy(s.begin(), s.end(), scales);
        if (zps) std::copy(z.begin(), z.end(), zps);
        if (rmin) std::copy(mn.begin(), mn.end(), rmin);
        if (rmax) std::copy(mx.begin(), mx.end(), rmax);
    });
}

int orc_quantize_fold(const vf_content* base, const vf_quant_spec* spec, const vf_transform* t, int n, void* dst,
                      uint64_t dst_bytes, uint64_t* dst_written, const vf_quant_outputs* outs, int nthreads,
                      char* err, size_t errlen) {
    return guard(err, errlen, [&] {
        Content in = wrap_base(*base);
        std::vector<double> s;
        std::vector<int64_t> z;
        std::vector<float> mn, mx;
        derive_params(in, *spec, s, z, mn, mx, nthreads);
        int64_t units, len;
        unit_geometry(in.type, *spec, units, len);

        // Quantize: per-channel goes through the per-axis transformation itself; per-group is the reference's
        // unrolled form (one uniform Quantize per [row, group] slice, concatenated), computed slice by slice.
        Content codes;
        if (spec->group_size == 0) {
            vf_transform q{};
            q.kind = VF_T_QUANTIZE;
            q.elem.kind = VF_ELEM_QUANT_PER_AXIS;
            q.elem.dtype = spec->storage_dtype;
            q.elem.expressed = spec->expressed;
            q.elem.axis = 0;
            q.elem.qmin = spec->qmin;
            q.elem.qmax = spec->qmax;
            q.elem.nparams = units;
            q.elem.scales = s.data();
            q.elem.zps = z.data();
            codes = tf_quantize(in, q, nthreads);
        } else {
            Type ot = in.type;
            ot.elem = Elem();
            ot.elem.dtype = spec->storage_dtype;
            codes = Content::alloc(ot, spec->storage_dtype, false);
            Reader r(in);
            parallel_nd(nthreads, {units}, [&](const int64_t* b, const int64_t* e) {
                for (int64_t u = b[0]; u < e[0]; ++u) {
                    const Quantizer qz(s[size_t(u)], z[size_t(u)], spec->qmin, spec->qmax);
                    for (int64_t i = 0; i < len; ++i)
                        store_int(codes.mdata(), spec->storage_dtype, u * len + i, qz(r.f(u * len + i)));
                }
            });
        }
        if (!codes.own.empty()) codes.ptr = codes.own.data();

        if (outs) {
            if (outs->scales) std::copy(s.begin(), s.end(), outs->scales);
            if (outs->zps) std::copy(z.begin(), z.end(), outs->zps);
            if (outs->scales_f16)
                for (int64_t u = 0; u < units; ++u) outs->scales_f16[u] = f32_to_f16(float(s[size_t(u)]));
            if (outs->zps_u4_packed) {
                for (int64_t u = 0; u < units; u += 2) {
                    const uint8_t lo = uint8_t(z[size_t(u)]) & 0xF;
                    const uint8_t hi = (u + 1 < units) ? (uint8_t(z[size_t(u + 1)]) & 0xF) : 0;
                    outs->zps_u4_packed[u / 2] = uint8_t((hi << 4) + lo);
                }
            }
            if (outs->dequant) {
                // [CastElemType<q>, Dequantize] on the codes, then copyTo in the requested float type
                Content qc = codes;
                if (!qc.own.empty()) qc.ptr = qc.own.data();
                Content deq;
                if (spec->group_size == 0) {
                    qc.type.elem.kind = VF_ELEM_QUANT_PER_AXIS;
                    qc.type.elem.dtype = spec->storage_dtype;
                    qc.type.elem.expressed = outs->dequant_dtype;
                    qc.type.elem.axis = 0;
                    qc.type.elem.qmin = spec->qmin;
                    qc.type.elem.qmax = spec->qmax;
                    qc.type.elem.scales = s;
                    qc.type.elem.zps = z;
                    vf_transform d{};
                    d.kind = VF_T_DEQUANTIZE;
                    deq = tf_dequantize(qc, d, nthreads);
                } else {
                    Type dt = in.type;
                    dt.elem = Elem();
                    dt.elem.dtype = outs->dequant_dtype;
                    deq = Content::alloc(dt, VF_DT_F32, false);
                    Reader r(qc);
                    float* o = reinterpret_cast<float*>(deq.mdata());
                    for (int64_t u = 0; u < units; ++u)
                        for (int64_t i = 0; i < len; ++i)
                            o[u * len + i] = dequantize_value(r.i64(u * len + i), s[size_t(u)], z[size_t(u)]);
                }
                if (!deq.own.empty()) deq.ptr = deq.own.data();
                copy_to(deq, static_cast<uint8_t*>(outs->dequant), outs->dequant_bytes);
            }
        }

        check_positions(t, n);
        Content c = std::move(codes);
        if (!c.own.empty()) c.ptr = c.own.data();
        for (int i = 0; i < n; ++i) {
            Content next = apply(c, t[i], nthreads);
            c = std::move(next);
            if (!c.own.empty()) c.ptr = c.own.data();
        }
        const uint64_t w = copy_to(c, static_cast<uint8_t*>(dst), dst_bytes);
        if (dst_written) *dst_written = w;
    });
}

int orc_nnz_per_oc(const vf_content* content, int64_t* counts, int nthreads, char* err, size_t errlen) {
    return guard(err, errlen, [&] {
        Content c = wrap_base(*content);
        auto v = count_nnz(c, nthreads);
        std::copy(v.begin(), v.end(), counts);
    });
}

int orc_sparsify(const vf_content* content, void* data, uint64_t data_bytes, uint64_t* data_written, void* map,
                 uint64_t map_bytes, int64_t* counts, int nthreads, char* err, size_t errlen) {
    return guard(err, errlen, [&] {
        Content c = wrap_base(*content);
        if (counts) {
            auto v = count_nnz(c, nthreads);
            std::copy(v.begin(), v.end(), counts);
        }
        if (data) {
            vf_transform t{};
            t.kind = VF_T_SPARSIFY;
            Content o = tf_sparsify(c, t, nthreads);
            if (data_bytes < o.nbytes) fail(VF_ERR_BUFFER_TOO_SMALL, "sparse data buffer too small");
            memcpy(data, o.data(), o.nbytes);
            if (data_written) *data_written = o.nbytes;
        }
        if (map) {
            vf_transform t{};
            t.kind = VF_T_GET_SPARSITY_MAP;
            Content o = tf_sparsity_map(c, t);
            if (map_bytes < o.nbytes) fail(VF_ERR_BUFFER_TOO_SMALL, "sparsity map buffer too small");
            memcpy(map, o.data(), o.nbytes);
        }
    });
}

// NCESparsity::getWeightsTable — VC/src/dialect/VPU/utils/nce_sparsity.cpp:171-231 with getMultShiftFunc :97-136,
// getBiasFunc :36-95, getRescaledBias :317-347 and the NPU37XX converters
// (VC/src/NPU37XX/dialect/VPU/impl/nce_sparsity_converters.cpp:14-42).
int orc_weights_table(const vf_weights_table_desc* d, int32_t* table, int nthreads, char* err, size_t errlen) {
    return guard(err, errlen, [&] {
        const int64_t OC = d->oc;
        if (OC <= 0) fail(VF_ERR_SHAPE, "OC must be positive");
        if (d->in_elem.dtype == VF_DT_INVALID || d->out_elem.dtype == VF_DT_INVALID)
            fail(VF_ERR_INVALID_ARG, "Can't create weights table without operation input/output types");
        const bool hasW = d->weights_elem.dtype != VF_DT_INVALID;
        const Elem in = elem_from_pod(d->in_elem), out = elem_from_pod(d->out_elem);
        const Elem w = hasW ? elem_from_pod(d->weights_elem) : Elem();
        const bool inQ = in.quantized(), outQ = out.quantized(), wQ = hasW && w.quantized();
        if (hasW && inQ && !wQ) fail(VF_ERR_UNSUPPORTED, "Unsupported In/Wt mixed precision");

        auto bcast = [&](const std::vector<double>& v, const char* what) {  // broadcast(): size 1 or OC
            std::vector<double> r(size_t(OC), 1.0);
            if (v.size() == 1)
                std::fill(r.begin(), r.end(), v[0]);
            else if (int64_t(v.size()) == OC)
                r = v;
            else
                fail(VF_ERR_SHAPE, "%s scales: %zu values for %lld channels", what, v.size(), (long long)OC);
            return r;
        };
        const auto inS = bcast(inQ ? in.scales : std::vector<double>{1.0}, "input");
        const auto outS = bcast(outQ ? out.scales : std::vector<double>{1.0}, "output");
        const auto wS = bcast(wQ ? w.scales : std::vector<double>{1.0}, "weights");
        const double constMul = d->has_const_scale ? d->const_scale : 1.0;

        // pointer columns — :176-189; sparse layout per relocate_weights_table.cpp:261-270
        std::vector<int32_t> wp(static_cast<size_t>(OC), 0), sp(static_cast<size_t>(OC), 0);
        if (d->nnz_counts) {
            const int64_t eb = std::max<int64_t>(1, dtype_bits(hasW ? w.dtype : VF_DT_U8) / 8);
            int64_t off = d->weights_ptr_base;
            for (int64_t oc = 0; oc < OC; ++oc) {
                wp[size_t(oc)] = int32_t(off);
                off += align_up(d->nnz_counts[oc] * eb, 16);
            }
        } else if (d->weights_ptrs) {
            std::copy(d->weights_ptrs, d->weights_ptrs + OC, wp.begin());
        } else {
            int32_t off = d->weights_ptr_base;
            for (int64_t oc = 0; oc < OC; ++oc) {
                wp[size_t(oc)] = off;
                off += d->weights_ptr_step;
            }
        }
        if (d->sparsity_ptrs) {
            std::copy(d->sparsity_ptrs, d->sparsity_ptrs + OC, sp.begin());
        } else {
            int32_t off = d->sparsity_ptr_base;
            for (int64_t oc = 0; oc < OC; ++oc) {
                sp[size_t(oc)] = off;
                off += d->sparsity_ptr_step;
            }
        }

        const bool isQuant = inQ && outQ, isFloat = !inQ && !outQ, isMixed = !isQuant && !isFloat;
        const bool quantBias = isQuant || (inQ && isMixed);
        const bool inIsFloatForPPE = !inQ && dtype_is_float(in.dtype);

        std::vector<double> rescaledBias;
        if (d->has_bias && quantBias) {  // getRescaledBias :317-347
            rescaledBias.resize(size_t(OC));
            for (int64_t oc = 0; oc < OC; ++oc) {
                const double denom = wS[size_t(oc)] * inS[size_t(oc)];
                const double b = double(d->bias[d->bias_is_splat ? 0 : oc]);
                const double v = b / denom;
                if (v <= double(std::numeric_limits<int32_t>::min()) || v >= double(std::numeric_limits<int32_t>::max()))
                    fail(VF_ERR_RANGE, "Rescaled bias value is out of range");
                rescaledBias[size_t(oc)] = v;
            }
        }

        parallel_nd(nthreads, {OC}, [&](const int64_t* b, const int64_t* e) {
            for (int64_t oc = b[0]; oc < e[0]; ++oc) {
                if (wp[size_t(oc)] % 16 != 0) fail(VF_ERR_ALIGNMENT, "weightsPtrs[%lld] must be multiple of 16", (long long)oc);
                if (sp[size_t(oc)] != VF_SPARSITY_PTR_WHEN_NO_SPARSITY && sp[size_t(oc)] % 16 != 0)
                    fail(VF_ERR_ALIGNMENT, "sparsityPtrs[%lld] must be aligned to 16", (long long)oc);
                // mult/shift column — :110-135
                const double rescale = (wS[size_t(oc)] * inS[size_t(oc)]) / outS[size_t(oc)] * constMul;
                int32_t mult, shift;
                approximate15(rescale, mult, shift);
                if (mult < -32768 || mult > 32767) fail(VF_ERR_CHECKED_CAST, "mult does not fit int16");
                int32_t ms;
                if (inIsFloatForPPE) {
                    ms = int32_t(f2u(float(rescale)));  // toHex — :141-143
                } else {
                    ms = (shift << 8) | int32_t(uint32_t(int32_t(int16_t(mult))) << 16);  // converters.cpp:22-29
                }
                // bias column — :36-95
                int32_t bias = 0;
                if (d->has_bias) {
                    if (quantBias) {
                        const double rb = std::round(rescaledBias[size_t(oc)]);  // converters.cpp:37-39
                        if (inQ) {
                            if (!(rb <= 2147483647.0) || !(rb >= -2147483648.0)) fail(VF_ERR_CHECKED_CAST, "bias");
                            bias = int32_t(rb);
                        } else {
                            bias = int32_t(f2u(float(rescaledBias[size_t(oc)])));
                        }
                    } else {
                        float bv = d->bias[d->bias_is_splat ? 0 : oc];
                        if (wQ) bv /= wS[size_t(oc)];  // float /= double, :79-86
                        const double real = bv;
                        if (inQ) {
                            bias = int32_t(std::round(real));
                        } else {
                            bias = int32_t(f2u(float(real)));
                        }
                    }
                } else {
                    // `return 0.0f` converted to int32 — :40-44
                    bias = 0;
                }
                table[oc * 4 + 0] = wp[size_t(oc)];
                table[oc * 4 + 1] = sp[size_t(oc)];
                table[oc * 4 + 2] = ms;
                table[oc * 4 + 3] = bias;
            }
        });
    });
}

int orc_synth_fill(const vf_synth_spec* s, void* dst, uint64_t count, int nthreads) {
    const uint64_t key = mix64(s->seed ^ mix64(s->tensor_id));
    // sum of four uniform 16-bit integers, centred: standard deviation sqrt((65536^2 - 1) / 3)
    const float c = float(double(s->sigma) / std::sqrt((65536.0 * 65536.0 - 1.0) / 3.0));
    const uint64_t omask = s->outlier_log2 > 0 ? ((1ull << s->outlier_log2) - 1) : 0;
    auto body = [&](uint64_t lo, uint64_t hi) {
        for (uint64_t i = lo; i < hi; ++i) {
            const uint64_t g = s->first_elem + i;
            const uint64_t h = mix64(key + g);
            const int32_t sum = int32_t(h & 0xFFFF) + int32_t((h >> 16) & 0xFFFF) + int32_t((h >> 32) & 0xFFFF) +
                                int32_t((h >> 48) & 0xFFFF) - 131070;
            float v = float(sum) * c;
            const uint64_t h2 = mix64(h);
            if (s->outlier_mult != 0.f && (h2 & omask) == 0) v = v * s->outlier_mult;
            if (s->mask_zero) {
                bool dense = false;
                if (s->dense_row_mod > 0 && s->row_len > 0) {
                    const uint64_t row = g / uint64_t(s->row_len);
                    dense = (mix64(key ^ (row * 0x9E3779B97F4A7C15ull + 0x632BE59BD9B4E019ull)) %
                             uint64_t(s->dense_row_mod)) == 0;
                }
                if (!dense && ((h2 >> 40) & 1)) v = 0.f;
            }
            switch (s->dtype) {
            case VF_DT_F32: static_cast<float*>(dst)[i] = v; break;
            case VF_DT_F16: static_cast<uint16_t*>(dst)[i] = rne_f16(v); break;
            default: static_cast<uint16_t*>(dst)[i] = rne_bf16(v); break;
            }
        }
    };
    if (nthreads <= 1 || count < 65536) {
        body(0, count);
    } else {
        std::vector<std::thread> th;
        const uint64_t per = (count + nthreads - 1) / nthreads;
        for (int t = 0; t < nthreads; ++t) {
            const uint64_t lo = per * t, hi = std::min<uint64_t>(count, lo + per);
            if (lo >= hi) break;
            th.emplace_back(body, lo, hi);
        }
        for (auto& x : th) x.join();
    }
    return VF_OK;
}

}  // extern "C"
