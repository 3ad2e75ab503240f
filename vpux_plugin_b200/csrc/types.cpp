// Host type model and per-transformation type inference (inferOutputType / inferOutputSplat of the
// reference's #const.* attributes). Pure host code: no CUDA calls.
#include <algorithm>
#include <cmath>
#include <limits>
#include <unordered_map>

#include "common.h"

namespace vf {

void raise(int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    throw Error(code, buf);
}

int dtype_bits(int dt) {
    static const int bits[] = {0, 32, 16, 16, 64, 8, 8, 16, 16, 32, 32, 64, 64, 4, 4, 1, 8, 8};
    if (dt <= VF_DT_INVALID || dt > VF_DT_F8E5M2) raise(VF_ERR_INVALID_ARG, "invalid dtype %d", dt);
    return bits[dt];
}
bool dtype_is_float(int dt) {
    return dt == VF_DT_F32 || dt == VF_DT_F16 || dt == VF_DT_BF16 || dt == VF_DT_F64 || dt == VF_DT_F8E4M3FN || dt == VF_DT_F8E5M2;
}
bool dtype_is_int(int dt) {
    return dt >= VF_DT_I8 && dt <= VF_DT_I1;
}
bool dtype_is_signed(int dt) {
    return dt == VF_DT_I8 || dt == VF_DT_I16 || dt == VF_DT_I32 || dt == VF_DT_I64 || dt == VF_DT_I4;
}
void dtype_int_limits(int dt, double& lo, double& hi) {
    const int b = dtype_bits(dt);
    if (!dtype_is_int(dt) || b < 8) raise(VF_ERR_UNSUPPORTED, "dtype %d has no byte-sized integer range", dt);
    if (dtype_is_signed(dt)) {
        lo = -std::ldexp(1.0, b - 1);
        hi = std::ldexp(1.0, b - 1) - 1.0;
    } else {
        lo = 0.0;
        hi = std::ldexp(1.0, b) - 1.0;
    }
}

uint32_t identity_order(int rank) {
    uint32_t code = 0;
    for (int i = 1; i <= rank; ++i) code = (code << 4) | uint32_t(i);
    return code;
}

void order_to_perm(uint32_t order, int rank, int* perm) {
    if (rank < 1 || rank > VF_MAX_RANK) raise(VF_ERR_INVALID_ARG, "rank %d outside 1..%d", rank, VF_MAX_RANK);
    uint32_t code = order ? order : identity_order(rank);
    uint32_t used = 0;
    for (int m = rank - 1; m >= 0; --m, code >>= 4) {
        const int d = int(code & 0xFu) - 1;
        if (d < 0 || d >= rank || (used >> d & 1u)) raise(VF_ERR_INVALID_ARG, "order %#x is not a permutation of rank %d", order, rank);
        used |= 1u << d;
        perm[m] = d;
    }
    if (code) raise(VF_ERR_INVALID_ARG, "order %#x has more digits than rank %d", order, rank);
}

// ------------------------------------------------------------------------------------------------------
namespace {
thread_local std::unordered_map<const double*, int64_t> tl_checked;
thread_local int tl_check_depth = 0;
}  // namespace
ParamCheckScope::ParamCheckScope() {
    if (tl_check_depth++ == 0) tl_checked.clear();
}
ParamCheckScope::~ParamCheckScope() {
    if (--tl_check_depth == 0) tl_checked.clear();
}

Elem Elem::from(const vf_elem_type& e, bool check_scales) {
    Elem r;
    r.kind = e.kind;
    r.dtype = e.dtype;
    if (e.kind < VF_ELEM_PLAIN || e.kind > VF_ELEM_QUANT_PER_AXIS) raise(VF_ERR_INVALID_ARG, "bad element kind %d", e.kind);
    dtype_bits(e.dtype);
    if (e.kind == VF_ELEM_PLAIN) return r;
    r.expressed = e.expressed;
    r.axis = e.kind == VF_ELEM_QUANT_PER_AXIS ? e.axis : -1;
    r.qmin = e.qmin;
    r.qmax = e.qmax;
    if (!e.scales || !e.zps || e.nparams < 1) raise(VF_ERR_INVALID_ARG, "quantized element type without scales/zero points");
    if (e.kind == VF_ELEM_QUANT_UNIFORM && e.nparams != 1) raise(VF_ERR_SHAPE, "uniform quantized type takes exactly one scale");
    r.scales.borrow(e.scales, size_t(e.nparams));
    r.zps.borrow(e.zps, size_t(e.nparams));
    // a quantized type cannot be built with such a scale: mlir::quant::UniformQuantized[PerAxis]Type::verify
    // rejects scale <= 0, infinities and NaN ("illegal scale")
    if (!check_scales) return r;
    if (tl_check_depth > 0 && e.nparams > 64) {
        const auto it = tl_checked.find(e.scales);
        if (it != tl_checked.end() && it->second >= e.nparams) return r;
    }
    // (counted without a branch so that the loop runs on vector registers: a network's per-channel scales are
    // tens of thousands of values per batch call)
    size_t illegal = 0;
    for (const double sc : r.scales) illegal += size_t(!((sc > 0.0) & (sc < HUGE_VAL)));
    if (illegal)
        for (const double sc : r.scales)
            if (!(sc > 0.0) || std::isinf(sc)) raise(VF_ERR_INVALID_ARG, "illegal scale: %g", sc);
    if (tl_check_depth > 0 && e.nparams > 64) tl_checked[e.scales] = e.nparams;
    return r;
}

bool Elem::single_zp(int64_t& zp) const {
    if (!quantized() || zps.empty()) return false;
    for (size_t i = 1; i < zps.size(); ++i)
        if (zps[i] != zps[0]) return false;
    zp = zps[0];
    return true;
}

Type Type::from(const vf_tensor_type& t) {
    Type r;
    if (t.rank < 1 || t.rank > VF_MAX_RANK) raise(VF_ERR_INVALID_ARG, "rank %d outside 1..%d", t.rank, VF_MAX_RANK);
    r.rank = t.rank;
    r.order = t.order ? t.order : identity_order(t.rank);
    int p[VF_MAX_RANK];
    order_to_perm(r.order, r.rank, p);
    for (int i = 0; i < r.rank; ++i) {
        if (t.shape[i] < 0) raise(VF_ERR_SHAPE, "negative extent");
        r.shape[i] = t.shape[i];
    }
    r.elem = Elem::from(t.elem);
    if (r.elem.kind == VF_ELEM_QUANT_PER_AXIS) {
        if (r.elem.axis < 0 || r.elem.axis >= r.rank) raise(VF_ERR_INVALID_ARG, "quantized dimension %d outside rank %d", r.elem.axis, r.rank);
        if (int64_t(r.elem.scales.size()) != r.shape[r.elem.axis])
            raise(VF_ERR_SHAPE, "Number of scales '%zu' in per-axis quantized type do not match the quantized dimension size '%lld'",
                  r.elem.scales.size(), (long long)r.shape[r.elem.axis]);
    }
    return r;
}

int64_t Type::numel() const {
    int64_t n = 1;
    for (int i = 0; i < rank; ++i) n *= shape[i];
    return n;
}
uint64_t Type::alloc_bytes() const {
    return (uint64_t(numel()) * uint64_t(dtype_bits(elem.dtype)) + 7u) / 8u;
}
void Type::perm(int* p) const {
    order_to_perm(order, rank, p);
}
void Type::mem_shape(int64_t* ms) const {
    int p[VF_MAX_RANK];
    perm(p);
    for (int i = 0; i < rank; ++i) ms[i] = shape[p[i]];
}

void Type::export_to(vf_tensor_type* out, double* sb, int64_t* zb, int64_t cap) const {
    if (!out) return;
    std::memset(out, 0, sizeof(*out));
    out->rank = rank;
    out->order = order;
    for (int i = 0; i < rank; ++i) out->shape[i] = shape[i];
    out->elem.kind = elem.kind;
    out->elem.dtype = elem.dtype;
    out->elem.expressed = elem.expressed;
    out->elem.axis = elem.axis;
    out->elem.qmin = elem.qmin;
    out->elem.qmax = elem.qmax;
    if (elem.quantized()) {
        const int64_t n = int64_t(elem.scales.size());
        if (!sb || !zb || cap < n) raise(VF_ERR_BUFFER_TOO_SMALL, "result type has %lld quantization parameters; buffers hold %lld", (long long)n, (long long)cap);
        std::copy(elem.scales.begin(), elem.scales.end(), sb);
        std::copy(elem.zps.begin(), elem.zps.end(), zb);
        out->elem.nparams = n;
        out->elem.scales = sb;
        out->elem.zps = zb;
    }
}

// ------------------------------------------------------------------------------------------------------
// Sparsify: compressed type (attributes/sparsify.cpp:93-101), weight sets aligned to 16 bytes
// (dialect/VPU/utils/nce_invariant.hpp:36)
// ------------------------------------------------------------------------------------------------------
Type compress_type(const Type& in, const int64_t* counts, int64_t n) {
    const int64_t eb = dtype_bits(in.elem.dtype) / 8;
    int64_t total = 0;
    for (int64_t i = 0; i < n; ++i) {
        if (counts[i] < 0) raise(VF_ERR_INVALID_ARG, "Got negative elem number value '%lld' in 'numActualElements' for 'SparsifyAttr'", (long long)counts[i]);
        total += align_up(counts[i] * eb, 16);
    }
    Type r;
    r.rank = 4;
    r.order = in.order;
    r.shape[0] = total;
    r.shape[1] = r.shape[2] = r.shape[3] = 1;
    r.elem = Elem::plain(VF_DT_U8);
    return r;
}

static void check_per_axis(const Type& t) {
    if (t.elem.kind != VF_ELEM_QUANT_PER_AXIS) return;
    if (t.elem.axis < 0 || t.elem.axis >= t.rank) raise(VF_ERR_SHAPE, "quantized dimension outside rank");
    if (int64_t(t.elem.scales.size()) != t.shape[t.elem.axis])
        raise(VF_ERR_SHAPE, "Number of scales '%zu' in per-axis quantized type do not match the quantized dimension size '%lld'",
              t.elem.scales.size(), (long long)t.shape[t.elem.axis]);
}

// getQuantizedAxis (utils/types.cpp:140-162): where the quantized axis lands after a reshape, or -1
int quantized_axis(int axis, const int64_t* prev, int prev_rank, const int64_t* next, int next_rank) {
    if (axis < 0 || axis >= prev_rank || prev[axis] == 1) return -1;
    int64_t full = 1;
    for (int i = 0; i <= axis; ++i) full *= prev[i];
    int64_t acc = 1;
    for (int i = 0; i < next_rank; ++i) {
        acc *= next[i];
        if (acc == full && next[i] == prev[axis]) return i;
        if (acc > full) break;
    }
    return -1;
}

Type infer_one(const Type& in, bool in_splat, const vf_transform& t, bool& out_splat) {
    Type out = in;
    out_splat = in_splat;
    switch (t.kind) {
    case VF_T_CAST_ELEM_TYPE:
    case VF_T_CONVERT_ELEM_TYPE:
        out.elem = Elem::from(t.elem);
        check_per_axis(out);
        return out;

    case VF_T_DEQUANTIZE:
        if (!in.elem.quantized()) raise(VF_ERR_NOT_QUANTIZED, "Got non quantized type in 'DequantizeAttr'");
        out.elem = Elem::plain(in.elem.expressed);
        if (in.elem.kind == VF_ELEM_QUANT_PER_AXIS) out_splat = false;
        return out;

    case VF_T_QUANTIZE: {
        const Elem q = Elem::from(t.elem);
        if (!q.quantized()) raise(VF_ERR_INVALID_ARG, "Can't quantize to empty type");
        if (!dtype_is_int(q.dtype) || dtype_bits(q.dtype) < 8) raise(VF_ERR_UNSUPPORTED, "Const.Quantize supports only integer byte+ storage type");
        out.elem = Elem::plain(q.dtype);
        out_splat = false;
        return out;
    }

    case VF_T_RESCALE:
    case VF_T_ADD:
        return out;

    case VF_T_RESHAPE:
    case VF_T_CHANGE_SHAPE_AND_ELEM_TYPE: {
        // changeShape / changeShapeElemType of a ranked tensor (core/type_interfaces.cpp:208-231, 253-269): an
        // identity order follows the new rank, any other order must fit it; a per-axis type keeps its axis where
        // getQuantizedAxis finds it in the new shape
        if (t.rank < 1 || t.rank > VF_MAX_RANK) raise(VF_ERR_INVALID_ARG, "Reshape rank %d", t.rank);
        int64_t n = 1;
        for (int i = 0; i < t.rank; ++i) n *= t.a[i];
        if (n != in.numel()) raise(VF_ERR_SHAPE, "Reshape to %lld elements from %lld", (long long)n, (long long)in.numel());
        out.rank = t.rank;
        for (int i = 0; i < VF_MAX_RANK; ++i) out.shape[i] = i < t.rank ? t.a[i] : 0;
        if (in.order == identity_order(in.rank)) out.order = identity_order(t.rank);
        else if (t.rank != in.rank) raise(VF_ERR_SHAPE, "Order '%x' is incompatible with the new shape", in.order);
        if (t.kind == VF_T_CHANGE_SHAPE_AND_ELEM_TYPE) {
            out.elem = Elem::from(t.elem);
        } else if (in.elem.kind == VF_ELEM_QUANT_PER_AXIS) {
            const int axis = quantized_axis(in.elem.axis, in.shape, in.rank, t.a, t.rank);
            if (axis >= 0) out.elem.axis = axis;
        }
        if (out.elem.kind == VF_ELEM_QUANT_PER_AXIS && (out.elem.axis < 0 || out.elem.axis >= out.rank))
            raise(VF_ERR_SHAPE, "Quantized axis '%d' is out of main type rank '%d'", out.elem.axis, out.rank);
        check_per_axis(out);
        return out;
    }

    case VF_T_REORDER:
    case VF_T_LAYOUT_CAST: {
        int p[VF_MAX_RANK];
        order_to_perm(t.order, in.rank, p);
        out.order = t.order ? t.order : identity_order(in.rank);
        return out;
    }

    case VF_T_TRANSPOSE: {
        int p[VF_MAX_RANK];
        order_to_perm(t.order, in.rank, p);
        for (int i = 0; i < in.rank; ++i) out.shape[i] = in.shape[p[i]];
        if (in.elem.kind == VF_ELEM_QUANT_PER_AXIS)
            for (int i = 0; i < in.rank; ++i)
                if (p[i] == in.elem.axis) out.elem.axis = i;
        return out;
    }

    case VF_T_MEM_PERMUTE: {
        int mp[VF_MAX_RANK], dp[VF_MAX_RANK], ip[VF_MAX_RANK];
        int64_t ims[VF_MAX_RANK];
        order_to_perm(t.mem_perm, in.rank, mp);
        order_to_perm(t.order, in.rank, dp);
        in.perm(ip);
        in.mem_shape(ims);
        for (int i = 0; i < in.rank; ++i) out.shape[dp[i]] = ims[mp[i]];
        out.order = t.order ? t.order : identity_order(in.rank);
        if (in.elem.kind == VF_ELEM_QUANT_PER_AXIS) {
            int in_mem_axis = 0;
            for (int i = 0; i < in.rank; ++i)
                if (ip[i] == in.elem.axis) in_mem_axis = i;
            for (int i = 0; i < in.rank; ++i)
                if (mp[i] == in_mem_axis) out.elem.axis = dp[i];
        }
        return out;
    }

    case VF_T_PAD_WITH_ZERO: {
        if (t.rank != in.rank) raise(VF_ERR_SHAPE, "Paddings and input shape are not consistent");
        for (int i = 0; i < in.rank; ++i) {
            if (t.a[i] < 0 || t.b[i] < 0) raise(VF_ERR_INVALID_ARG, "negative padding");
            out.shape[i] = in.shape[i] + t.a[i] + t.b[i];
        }
        if (in.elem.kind == VF_ELEM_QUANT_PER_AXIS) {
            // expandScalesAndZP (utils/quantization.cpp:168-224): replicate the first / last channel's
            // parameters; every zero point must be the same when the quantized axis itself is padded
            const int64_t pb = t.a[in.elem.axis], pa = t.b[in.elem.axis];
            if (pb || pa) {
                int64_t zp;
                if (!in.elem.single_zp(zp)) raise(VF_ERR_ZERO_POINTS, "All zero points should be equal");
                out.elem.scales.assign(size_t(pb), in.elem.scales.front());
                out.elem.scales.append(in.elem.scales.begin(), in.elem.scales.end());
                out.elem.scales.append(size_t(pa), in.elem.scales.back());
                out.elem.zps.assign(out.elem.scales.size(), zp);
            }
        }
        check_per_axis(out);
        out_splat = false;
        return out;
    }

    case VF_T_SUBVIEW: {
        if (t.rank != in.rank) raise(VF_ERR_SHAPE, "SubView rank mismatch");
        for (int i = 0; i < in.rank; ++i) {
            if (t.a[i] < 0 || t.b[i] < 1 || t.a[i] + t.b[i] > in.shape[i]) raise(VF_ERR_SHAPE, "SubView [%lld, %lld) outside extent %lld", (long long)t.a[i], (long long)(t.a[i] + t.b[i]), (long long)in.shape[i]);
            out.shape[i] = t.b[i];
        }
        if (in.elem.kind == VF_ELEM_QUANT_PER_AXIS) {
            const int ax = in.elem.axis;
            out.elem.scales.assign(in.elem.scales.begin() + t.a[ax], in.elem.scales.begin() + t.a[ax] + t.b[ax]);
            out.elem.zps.assign(in.elem.zps.begin() + t.a[ax], in.elem.zps.begin() + t.a[ax] + t.b[ax]);
        }
        return out;
    }

    case VF_T_BIT_PACK:
        if (t.width != 4) raise(VF_ERR_UNSUPPORTED, "BitPackAttr does not support any bitwidth except for 4 at this point.");
        if (!in.elem.quantized() && dtype_is_float(in.elem.dtype)) raise(VF_ERR_UNSUPPORTED, "Bit pack does not support float inputs.");
        if (in_splat) raise(VF_ERR_SPLAT, "Bit pack does not support splat inputs.");
        out.elem.dtype = dtype_is_signed(in.elem.dtype) ? VF_DT_I4 : VF_DT_U4;
        out_splat = false;
        return out;

    case VF_T_GET_SPARSITY_MAP: {
        if (in.rank != 4) raise(VF_ERR_SHAPE, "Expected data shape to be 4D");
        out.shape[0] = in.shape[0];
        out.shape[1] = out.shape[2] = 1;
        out.shape[3] = align_up(in.shape[1] * in.shape[2] * in.shape[3], 128);  // inferWeightsSparsityMapShape
        out.order = identity_order(4);
        out.elem = Elem::plain(VF_DT_I1);
        out_splat = false;
        return out;
    }

    case VF_T_SPARSIFY:
        if (t.compress_output) {
            if (!t.num_actual) raise(VF_ERR_INVALID_ARG, "Missing number of actual elements");
            out = compress_type(in, t.num_actual, t.n_num_actual);
        }
        out_splat = false;
        return out;

    case VF_T_SWIZZLE_CONSTANT: {  // swizzle_transform.cpp:127-156: a flat buffer of the swizzling-aligned size
        const int64_t arch = t.a[1];
        if (arch != VF_ARCH_NPU37XX && arch != VF_ARCH_NPU40XX) raise(VF_ERR_UNSUPPORTED, "Architecture %lld does not support swizzling", (long long)arch);
        if (t.a[0] < 0) raise(VF_ERR_INVALID_ARG, "negative swizzle key");
        const int64_t new_size = align_up(int64_t(in.alloc_bytes()), swizzle_size_alignment(int(arch)));
        for (int i = 0; i < in.rank; ++i) out.shape[i] = 1;
        if (!in.elem.quantized() && dtype_bits(in.elem.dtype) == 1) {
            out.shape[0] = new_size * 8;  // 1-bit types keep their type
        } else if (!in.elem.quantized() && in.elem.dtype == VF_DT_F16) {
            out.shape[0] = new_size / 2;
        } else {
            out.shape[0] = new_size;
            out.elem = Elem::plain(VF_DT_U8);
        }
        out_splat = false;
        return out;
    }

    case VF_T_RELOCATE_WEIGHTS_TABLE: {  // relocate_weights_table.cpp:194-200: type and splatness pass through
        const vf_relocate& r = t.relocate;
        if (r.n_clusters < 1 || r.n_clusters > VF_MAX_CLUSTERS) raise(VF_ERR_INVALID_ARG, "RelocateWeightsTable with %d clusters (1..%d)", r.n_clusters, VF_MAX_CLUSTERS);
        if (in.elem.quantized() || dtype_bits(in.elem.dtype) != 32 || dtype_is_float(in.elem.dtype))
            raise(VF_ERR_UNSUPPORTED, "RelocateWeightsTable patches tables of 32-bit integers");
        if (r.weights_table_size < 0 || r.weights_table_size / 4 > in.numel())
            raise(VF_ERR_SHAPE, "weightsTableSize %lld exceeds the constant (%lld entries)", (long long)r.weights_table_size, (long long)in.numel());
        out_splat = in_splat;
        return out;
    }

    case VF_T_REVERSE: {  // reverse.cpp:35-44, 46-105
        Elem e = in.elem;
        if (e.kind == VF_ELEM_QUANT_PER_AXIS) raise(VF_ERR_UNSUPPORTED, "Unexpected data type: per-axis quantized");
        const int dt = e.dtype;
        if (dt != VF_DT_I8 && dt != VF_DT_U8 && dt != VF_DT_F16 && dt != VF_DT_BF16 && dt != VF_DT_F32)
            raise(VF_ERR_UNSUPPORTED, "Unexpected data type: %d", dt);
        if (!in_splat && (t.a[0] < 0 || t.a[0] >= in.rank - 1))
            raise(VF_ERR_INVALID_ARG, "Const::Content::reverse: got unexpected content dimension %lld", (long long)t.a[0]);
        return out;
    }

    case VF_T_BROADCAST: {  // broadcast.cpp:66-83: the type is padded behind `axis` up to `value`
        const int64_t axis = t.a[0], value = t.a[1];
        if (axis < 0 || axis >= in.rank) raise(VF_ERR_INVALID_ARG, "Broadcast axis %lld", (long long)axis);
        if (value < in.shape[axis])
            raise(VF_ERR_SHAPE, "Value cannot be broadcasted due to new value's size is less than old one: %lld < %lld", (long long)value, (long long)in.shape[axis]);
        vf_transform pad{};
        pad.kind = VF_T_PAD_WITH_ZERO;
        pad.rank = in.rank;
        pad.b[axis] = value - in.shape[axis];
        bool ignored;
        out = infer_one(in, in_splat, pad, ignored);
        return out;  // splatness passes through
    }

    case VF_T_EXPAND_DILATED: {  // getDilatedType, utils/dilated_utils.cpp:11-34
        if (in.rank != 4) raise(VF_ERR_SHAPE, "Got invalid tensor rank '4'");
        if (t.a[0] < 1 || t.a[1] < 1) raise(VF_ERR_INVALID_ARG, "dilations must be positive");
        out.shape[2] = in.shape[2] + (in.shape[2] - 1) * (t.a[0] - 1);
        out.shape[3] = in.shape[3] + (in.shape[3] - 1) * (t.a[1] - 1);
        check_per_axis(out);
        out_splat = false;
        return out;
    }

    case VF_T_SCALAR_MULT_INVERSE:  // inverse.cpp:40-50
        return out;

    default:
        raise(VF_ERR_INVALID_ARG, "unknown transformation kind %d", t.kind);
    }
}

int64_t swizzle_size_alignment(int arch) {  // utils/swizzling_utils.hpp:26-27
    return arch == VF_ARCH_NPU40XX ? 1024 : 512;
}

void check_positions(const vf_transform* t, int n) {
    // attributes/content.cpp:585-588 — a LAST transformation (BitPack, SwizzleConstant) may only be the final one
    if (n >= 2 && (t[n - 2].kind == VF_T_BIT_PACK || t[n - 2].kind == VF_T_SWIZZLE_CONSTANT))
        raise(VF_ERR_POSITION, "At most 1 attribute with LAST requirement allowed!");
}

bool calc_scale_zp_host(double qmin, double qmax, double rmin, double rmax, double& scale, int64_t& zp) {
    const double eps = std::numeric_limits<double>::epsilon();
    if (std::fabs(rmax - rmin) < eps) {
        if (std::fabs(rmin) < eps) {
            scale = 1.0;
            zp = 0;
        } else if (rmin > 0) {
            scale = rmin;
            zp = 0;
        } else {
            scale = -rmin;
            zp = 2;
        }
        return true;
    }
    if (!((rmin <= 0 && rmax >= 0) || (rmin >= 0 && rmax <= 0))) return false;
    scale = (rmax - rmin) / (qmax - qmin);
    if (std::fabs(scale) <= eps) return false;
    zp = int64_t(std::round(qmin - rmin / scale));
    return true;
}

// getMaxIntermediateSize — const/passes/constant_folding.cpp:20-31
uint64_t max_intermediate_size(Type ty, bool splat, const vf_transform* t, int n) {
    uint64_t most = ty.alloc_bytes();
    for (int i = 0; i < n; ++i) {
        bool s;
        ty = infer_one(ty, splat, t[i], s);
        splat = s;
        most = std::max<uint64_t>(most, ty.alloc_bytes());
    }
    return most;
}

}  // namespace vf

extern "C" {

int vf_abi_version(void) {
    return VF_ABI_VERSION;
}

const char* vf_status_string(int s) {
    switch (s) {
    case VF_OK: return "ok";
    case VF_ERR_INVALID_ARG: return "invalid argument";
    case VF_ERR_UNSUPPORTED: return "unsupported type or transformation";
    case VF_ERR_SHAPE: return "shape mismatch";
    case VF_ERR_NOT_QUANTIZED: return "element type is not quantized";
    case VF_ERR_ZERO_POINTS: return "zero points are not all equal";
    case VF_ERR_SPLAT: return "splat input not supported";
    case VF_ERR_ODD_COUNT: return "odd element count";
    case VF_ERR_POSITION: return "transformation position requirement violated";
    case VF_ERR_CHECKED_CAST: return "value does not fit the destination type";
    case VF_ERR_BUFFER_TOO_SMALL: return "destination buffer too small";
    case VF_ERR_ALIGNMENT: return "pointer not 16-byte aligned";
    case VF_ERR_RANGE: return "value outside representable range";
    case VF_ERR_QUANT_RANGE: return "cannot derive scale / zero point from range";
    case VF_ERR_NOT_NORMAL: return "inverse of a non-normal float";
    case VF_ERR_NAN: return "NaN met by Quantize";
    case VF_ERR_CUDA: return "CUDA error";
    case VF_ERR_NO_DEVICE: return "no CUDA device";
    case VF_ERR_OOM: return "out of memory";
    case VF_ERR_CAPACITY: return "request exceeds built-in capacity";
    case VF_ERR_NOT_RUN: return "job not run";
    default: return "unknown status";
    }
}

int vf_infer_type(const vf_tensor_type* base, int base_is_splat, const vf_transform* t, int n, vf_tensor_type* out,
                  int* out_is_splat, double* scales_buf, int64_t* zps_buf, int64_t params_cap, uint64_t* out_bytes,
                  char* err, size_t errlen) {
    return vf::guard(err, errlen, [&] {
        if (!base || (n > 0 && !t) || n < 0) vf::raise(VF_ERR_INVALID_ARG, "NULL argument");
        vf::Type ty = vf::Type::from(*base);
        bool splat = base_is_splat != 0;
        vf::check_positions(t, n);
        for (int i = 0; i < n; ++i) {
            bool s;
            ty = vf::infer_one(ty, splat, t[i], s);
            splat = s;
        }
        ty.export_to(out, scales_buf, zps_buf, params_cap);
        if (out_is_splat) *out_is_splat = splat ? 1 : 0;
        if (out_bytes) *out_bytes = ty.alloc_bytes();
    });
}

int vf_max_intermediate_size(const vf_tensor_type* base, int base_is_splat, const vf_transform* t, int n,
                             uint64_t* out_bytes, char* err, size_t errlen) {
    return vf::guard(err, errlen, [&] {
        if (!base || !out_bytes || (n > 0 && !t) || n < 0) vf::raise(VF_ERR_INVALID_ARG, "NULL argument");
        *out_bytes = vf::max_intermediate_size(vf::Type::from(*base), base_is_splat != 0, t, n);
    });
}

int vf_plan_shards(int mode, int world, int64_t ntensors, const uint64_t* bytes, const int64_t* rows,
                   int64_t row_align, int64_t* row_begin, int64_t* row_end, char* err, size_t errlen) {
    return vf::guard(err, errlen, [&] {
        if (world < 1 || ntensors < 0 || !rows || !row_begin || !row_end) vf::raise(VF_ERR_INVALID_ARG, "bad shard plan arguments");
        if (mode == 0) {
            // whole tensors, longest-processing-time-first: sort by size descending, give each to the
            // least-loaded rank (ties -> lowest rank) — deterministic on every rank
            if (!bytes) vf::raise(VF_ERR_INVALID_ARG, "mode 0 needs tensor sizes");
            std::vector<int64_t> idx(static_cast<size_t>(ntensors), 0);
            for (int64_t i = 0; i < ntensors; ++i) idx[size_t(i)] = i;
            std::stable_sort(idx.begin(), idx.end(), [&](int64_t a, int64_t b) { return bytes[a] > bytes[b]; });
            std::vector<uint64_t> load(size_t(world), 0);
            for (int64_t i = 0; i < ntensors * world; ++i) row_begin[i] = row_end[i] = 0;
            for (int64_t k : idx) {
                int best = 0;
                for (int r = 1; r < world; ++r)
                    if (load[size_t(r)] < load[size_t(best)]) best = r;
                load[size_t(best)] += bytes[k];
                row_begin[k * world + best] = 0;
                row_end[k * world + best] = rows[k];
            }
        } else if (mode == 1) {
            const int64_t al = row_align > 0 ? row_align : 1;
            for (int64_t k = 0; k < ntensors; ++k) {
                const int64_t blocks = (rows[k] + al - 1) / al;
                for (int r = 0; r < world; ++r) {
                    const int64_t b0 = blocks * r / world, b1 = blocks * (r + 1) / world;
                    row_begin[k * world + r] = std::min(rows[k], b0 * al);
                    row_end[k * world + r] = std::min(rows[k], b1 * al);
                }
            }
        } else {
            vf::raise(VF_ERR_INVALID_ARG, "unknown shard mode %d", mode);
        }
    });
}

}  // extern "C"
