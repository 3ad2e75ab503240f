// Transformation-list optimiser: what Const::ContentSetup::addTransformation does every time a transformation
// is appended (attributes/content.cpp:530-588) — insert by position requirement, then run the local rewrite
// rules until none applies:
//   fuseConsecutiveTransformations  utils/transformations.cpp:385-476
//   foldTransformation              utils/transformations.cpp:482-513
//   moveSubViewBefore               utils/transformations.cpp:519-651 (with the prepare*Swap helpers :77-322)
//   moveReshapeBefore               utils/transformations.cpp:657-712
// Pure host code. A shorter list means fewer passes over the data on the device, and a SubView moved to the
// front means only the needed slab is uploaded and folded.
// Not covered: Fuse as a list entry (moveTransformationIntoFuse); the library folds fused constants through
// vf_fuse, whose parts carry their own lists.
#include <algorithm>
#include <functional>

#include "common.h"

namespace vf {

namespace {

struct Item {
    vf_transform t{};
    Elem elem;                    // CastElemType / ConvertElemType / Quantize target
    std::vector<int64_t> counts;  // Sparsify numActualElements
};
using List = std::vector<Item>;

int position(int kind) {  // attr_interfaces.hpp:24-28
    if (kind == VF_T_BIT_PACK || kind == VF_T_SWIZZLE_CONSTANT) return 2;
    if (kind == VF_T_SPARSIFY || kind == VF_T_GET_SPARSITY_MAP) return 1;
    return 0;
}

vf_transform pod_of(const Item& it) {  // borrows the item's arrays
    vf_transform t = it.t;
    t.elem = vf_elem_type{};
    t.elem.kind = it.elem.kind;
    t.elem.dtype = it.elem.dtype;
    t.elem.expressed = it.elem.expressed;
    t.elem.axis = it.elem.axis;
    t.elem.qmin = it.elem.qmin;
    t.elem.qmax = it.elem.qmax;
    t.elem.nparams = int64_t(it.elem.scales.size());
    t.elem.scales = it.elem.scales.empty() ? nullptr : it.elem.scales.data();
    t.elem.zps = it.elem.zps.empty() ? nullptr : it.elem.zps.data();
    t.num_actual = it.counts.empty() ? nullptr : it.counts.data();
    t.n_num_actual = int64_t(it.counts.size());
    return t;
}

// type after the first `count` transformations (Const::inferFinalType)
Type infer_prefix(const Type& base, const List& l, size_t count) {
    Type cur = base;
    bool splat = false;
    for (size_t i = 0; i < count; ++i) {
        bool os;
        cur = infer_one(cur, splat, pod_of(l[i]), os);
        splat = os;
    }
    return cur;
}

bool same_type(const Type& a, const Type& b) {
    if (a.rank != b.rank || a.order != b.order) return false;
    for (int i = 0; i < a.rank; ++i)
        if (a.shape[i] != b.shape[i]) return false;
    const Elem &x = a.elem, &y = b.elem;
    return x.kind == y.kind && x.dtype == y.dtype && x.expressed == y.expressed && x.axis == y.axis && x.qmin == y.qmin &&
           x.qmax == y.qmax && x.scales == y.scales && x.zps == y.zps;
}

uint32_t perm_to_code(const int* perm, int rank) {
    uint32_t code = 0;
    for (int i = 0; i < rank; ++i) code = (code << 4) | uint32_t(perm[i] + 1);
    return code;
}

// getPermutationFromOrders: r[i] = memory dim of the input that holds what output memory dim i holds
void reorder_perm(uint32_t in_order, uint32_t out_order, int rank, int* r) {
    int ip[VF_MAX_RANK], op[VF_MAX_RANK];
    order_to_perm(in_order ? in_order : identity_order(rank), rank, ip);
    order_to_perm(out_order ? out_order : identity_order(rank), rank, op);
    for (int i = 0; i < rank; ++i)
        for (int j = 0; j < rank; ++j)
            if (ip[j] == op[i]) r[i] = j;
}

using Result = std::pair<size_t, bool>;  // (new current position, something changed)

// ---- fuseConsecutiveTransformations ---------------------------------------------------------------------
Result fuse_consecutive(List& l, size_t cur, const Type& base) {
    if (cur == 0 || cur >= l.size()) return {cur, false};
    Item& prev = l[cur - 1];
    Item& curr = l[cur];
    const int pk = prev.t.kind, ck = curr.t.kind;
    bool fused = false;
    Item merged = curr;
    if (pk == VF_T_SUBVIEW && ck == VF_T_SUBVIEW) {
        for (int i = 0; i < curr.t.rank; ++i) merged.t.a[i] = prev.t.a[i] + curr.t.a[i];
        fused = true;
    } else if (pk == VF_T_ADD && ck == VF_T_ADD) {
        merged.t.value = prev.t.value + curr.t.value;
        fused = true;
    } else if (pk == VF_T_RESCALE && ck == VF_T_RESCALE) {
        merged.t.value = prev.t.value * curr.t.value;
        fused = true;
    } else if ((pk == VF_T_RESHAPE && ck == VF_T_RESHAPE) || (pk == VF_T_REORDER && ck == VF_T_REORDER) ||
               (pk == VF_T_CAST_ELEM_TYPE && ck == VF_T_CAST_ELEM_TYPE)) {
        fused = true;  // the later one wins
    } else if ((pk == VF_T_REORDER && ck == VF_T_MEM_PERMUTE) || (pk == VF_T_MEM_PERMUTE && ck == VF_T_REORDER)) {
        const Type in_type = infer_prefix(base, l, cur - 1);
        const int rank = in_type.rank;
        int c[VF_MAX_RANK], m[VF_MAX_RANK], r[VF_MAX_RANK];
        uint32_t last_order;
        if (pk == VF_T_MEM_PERMUTE) {  // MemPermute then Reorder: c[i] = m[r[i]]
            bool os;
            const Type mid = infer_one(in_type, false, pod_of(prev), os);
            order_to_perm(prev.t.mem_perm ? prev.t.mem_perm : identity_order(rank), rank, m);
            reorder_perm(mid.order, curr.t.order, rank, r);
            for (int i = 0; i < rank; ++i) c[i] = m[r[i]];
            last_order = curr.t.order;
        } else {  // Reorder then MemPermute: c[i] = r[m[i]]
            order_to_perm(curr.t.mem_perm ? curr.t.mem_perm : identity_order(rank), rank, m);
            reorder_perm(in_type.order, prev.t.order, rank, r);
            for (int i = 0; i < rank; ++i) c[i] = r[m[i]];
            last_order = curr.t.order;
        }
        merged = Item{};
        merged.t.kind = VF_T_MEM_PERMUTE;
        merged.t.order = last_order;
        merged.t.mem_perm = perm_to_code(c, rank);
        fused = true;
    }
    if (!fused) return {cur, false};
    l[cur - 1] = merged;
    l.erase(l.begin() + long(cur));
    return {cur - 1, true};
}

// ---- foldTransformation ---------------------------------------------------------------------------------
Result fold_noop(List& l, size_t cur, const Type& base) {
    if (cur >= l.size()) return {cur, false};
    const int k = l[cur].t.kind;
    if (k != VF_T_REORDER && k != VF_T_MEM_PERMUTE) return {cur, false};
    const Type in_type = infer_prefix(base, l, cur);
    bool os;
    const Type out_type = infer_one(in_type, false, pod_of(l[cur]), os);
    if (!same_type(in_type, out_type)) return {cur, false};
    if (k == VF_T_MEM_PERMUTE) {
        int m[VF_MAX_RANK];
        order_to_perm(l[cur].t.mem_perm ? l[cur].t.mem_perm : identity_order(in_type.rank), in_type.rank, m);
        for (int i = 0; i < in_type.rank; ++i)
            if (m[i] != i) return {cur, false};
    }
    l.erase(l.begin() + long(cur));
    return {cur, true};
}

// ---- moveSubViewBefore ----------------------------------------------------------------------------------
// sliceInputShape (transformations.cpp:39-72): SubView parameters on the input of a Reshape
bool slice_input_shape(const int64_t* rin, int nin, const int64_t* rout, int nout, const int64_t* off, const int64_t* shp,
                       int64_t* new_off, int64_t* new_shp) {
    for (int i = 0; i < nin; ++i) {
        new_off[i] = 0;
        new_shp[i] = rin[i];
    }
    int64_t in_low = 1, out_low = 1;
    int id = nin - 1;
    for (int od = nout - 1; od >= 0; --od) {
        const bool sliced = off[od] > 0 || shp[od] < rout[od];
        if (!sliced) {
            out_low *= rout[od];
            continue;
        }
        for (; id >= 0; --id) {
            if (rin[id] == rout[od] && in_low == out_low) break;
            in_low *= rin[id];
        }
        if (id < 0 || rin[id] != rout[od] || in_low != out_low) return false;
        new_off[id] = off[od];
        new_shp[id] = shp[od];
        out_low *= rout[od];
    }
    return true;
}

Result move_subview_before(List& l, size_t cur, const Type& base) {
    if (cur == 0 || cur >= l.size()) return {cur, false};
    if (l[cur].t.kind != VF_T_SUBVIEW) return {cur, false};
    Item& prev = l[cur - 1];
    Item& sub = l[cur];
    const Type prev_in = infer_prefix(base, l, cur - 1);
    const int rank = sub.t.rank;
    switch (prev.t.kind) {
    case VF_T_ADD:
    case VF_T_RESCALE:
    case VF_T_DEQUANTIZE:
    case VF_T_REORDER: break;
    case VF_T_CAST_ELEM_TYPE:
    case VF_T_CONVERT_ELEM_TYPE:
        if (prev.elem.kind == VF_ELEM_QUANT_PER_AXIS) {  // tileScalesAndZP: the slice of the quantized axis
            const int ax = prev.elem.axis;
            if (ax < 0 || ax >= rank || sub.t.a[ax] + sub.t.b[ax] > int64_t(prev.elem.scales.size())) return {cur, false};
            prev.elem.scales.assign(prev.elem.scales.begin() + sub.t.a[ax], prev.elem.scales.begin() + sub.t.a[ax] + sub.t.b[ax]);
            prev.elem.zps.assign(prev.elem.zps.begin() + sub.t.a[ax], prev.elem.zps.begin() + sub.t.a[ax] + sub.t.b[ax]);
        }
        break;
    case VF_T_TRANSPOSE: {  // prepareTransposeSwap: offsets follow the permutation back to the input dims
        int p[VF_MAX_RANK];
        order_to_perm(prev.t.order ? prev.t.order : identity_order(rank), rank, p);
        int64_t no[VF_MAX_RANK], ns[VF_MAX_RANK];
        for (int i = 0; i < rank; ++i) {
            no[p[i]] = sub.t.a[i];
            ns[p[i]] = sub.t.b[i];
        }
        for (int i = 0; i < rank; ++i) {
            sub.t.a[i] = no[i];
            sub.t.b[i] = ns[i];
        }
        break;
    }
    case VF_T_RESHAPE: {  // prepareReshapeSwap
        int64_t no[VF_MAX_RANK], ns[VF_MAX_RANK];
        if (!slice_input_shape(prev_in.shape, prev_in.rank, prev.t.a, prev.t.rank, sub.t.a, sub.t.b, no, ns)) return {cur, false};
        prev.t.rank = sub.t.rank;  // Reshape to the SubView's shape ...
        for (int i = 0; i < sub.t.rank; ++i) prev.t.a[i] = sub.t.b[i];
        sub.t.rank = prev_in.rank;  // ... of a SubView taken on the Reshape's input
        for (int i = 0; i < prev_in.rank; ++i) {
            sub.t.a[i] = no[i];
            sub.t.b[i] = ns[i];
        }
        break;
    }
    case VF_T_CHANGE_SHAPE_AND_ELEM_TYPE: {  // prepareChangeShapeSwap (:125-155)
        int64_t no[VF_MAX_RANK], ns[VF_MAX_RANK];
        if (!slice_input_shape(prev_in.shape, prev_in.rank, prev.t.a, prev.t.rank, sub.t.a, sub.t.b, no, ns)) return {cur, false};
        if (prev.elem.kind == VF_ELEM_QUANT_PER_AXIS) {  // the type of the slice: parameters of the kept channels
            const int ax = prev.elem.axis;
            if (ax < 0 || ax >= rank || sub.t.a[ax] < 0 || sub.t.a[ax] + sub.t.b[ax] > int64_t(prev.elem.scales.size())) return {cur, false};
            prev.elem.scales.assign(prev.elem.scales.begin() + sub.t.a[ax], prev.elem.scales.begin() + sub.t.a[ax] + sub.t.b[ax]);
            prev.elem.zps.assign(prev.elem.zps.begin() + sub.t.a[ax], prev.elem.zps.begin() + sub.t.a[ax] + sub.t.b[ax]);
        }
        prev.t.rank = sub.t.rank;
        for (int i = 0; i < sub.t.rank; ++i) prev.t.a[i] = sub.t.b[i];
        sub.t.rank = prev_in.rank;
        for (int i = 0; i < prev_in.rank; ++i) {
            sub.t.a[i] = no[i];
            sub.t.b[i] = ns[i];
        }
        break;
    }
    case VF_T_PAD_WITH_ZERO: {  // preparePadWithZeroSwap
        int64_t no[VF_MAX_RANK], ns[VF_MAX_RANK], pb[VF_MAX_RANK], pa[VF_MAX_RANK];
        for (int i = 0; i < rank; ++i) {
            const int64_t lo = sub.t.a[i], hi = sub.t.a[i] + sub.t.b[i];
            const int64_t before = prev.t.a[i], after = prev.t.b[i], extent = prev_in.shape[i];
            const int64_t padded = before + extent + after;
            if (lo >= before + extent || hi <= before) return {cur, false};  // a view of padding only
            pa[i] = after;
            pb[i] = before;
            if (lo < before) {
                pb[i] -= lo;
                no[i] = 0;
            } else {
                no[i] = lo - before;
                pb[i] = 0;
            }
            if (hi > before + extent) pa[i] -= padded - hi;
            else pa[i] = 0;
            ns[i] = sub.t.b[i] - pb[i] - pa[i];
        }
        for (int i = 0; i < rank; ++i) {
            sub.t.a[i] = no[i];
            sub.t.b[i] = ns[i];
            prev.t.a[i] = pb[i];
            prev.t.b[i] = pa[i];
        }
        break;
    }
    case VF_T_RELOCATE_WEIGHTS_TABLE: {  // prepareRelocateWeightsTableSwap (:157-270)
        vf_relocate r = prev.t.relocate;
        const int64_t sub_size = sub.t.b[0], sub_off = sub.t.a[0];
        if (sub_size <= 1) return {cur, false};  // one channel cannot give the pointer steps
        for (int d = rank - 1; d >= 1; --d)      // only slices of the channel dim
            if (sub.t.a[d] > 0 || sub.t.b[d] < prev_in.shape[d]) return {cur, false};
        const uint64_t total_channels = uint64_t(prev_in.shape[0]);
        if (total_channels == 0) return {cur, false};
        const uint64_t entry = uint64_t(r.weights_table_size) / 4 / total_channels;
        bool different = false;
        for (int c = 1; c < r.n_clusters; ++c) different = different || r.offsets[c] != r.offsets[c - 1];
        if (different) {  // the slice must be exactly one cluster's channels
            int idx = -1;
            for (int c = 0; c < r.n_clusters && idx < 0; ++c)
                if (r.offsets[c] == sub_off) idx = c;
            if (idx < 0) return {cur, false};
            if (idx + 1 < r.n_clusters && r.offsets[idx + 1] - sub_off != sub_size) return {cur, false};
            if (r.num_elems) {  // the compression entries of the slice
                if (r.compression_axis != 0) return {cur, false};
                if (sub_off < 0 || sub_off + sub_size > r.n_num_elems) return {cur, false};
                r.num_elems += sub_off;
                r.n_num_elems = sub_size;
            }
            r.weights_ptr[0] = r.weights_ptr[idx];
            r.offsets[0] = 0;
            r.n_clusters = 1;
        } else {  // same cluster everywhere: the slice only shifts the first channel
            r.channel_offset += sub_off;
        }
        r.weights_table_size = int64_t(entry * uint64_t(sub_size) * 4);
        prev.t.relocate = r;
        break;
    }
    default: return {cur, false};
    }
    const bool was_pad = prev.t.kind == VF_T_PAD_WITH_ZERO;
    std::swap(l[cur - 1], l[cur]);
    if (!was_pad) return {cur - 1, true};
    // a SubView that covers its whole input and a PadWithZero that pads nothing are dropped (:614-648)
    size_t sub_pos = cur - 1, pad_pos = cur;
    Type in_type = prev_in;
    bool os, sub_folded = false;
    Type out = infer_one(in_type, false, pod_of(l[sub_pos]), os);
    if (same_type(out, in_type)) {
        l.erase(l.begin() + long(sub_pos));
        pad_pos = sub_pos;
        sub_folded = true;
    } else {
        in_type = out;
    }
    out = infer_one(in_type, false, pod_of(l[pad_pos]), os);
    if (same_type(out, in_type)) {
        l.erase(l.begin() + long(pad_pos));
    }
    if (sub_folded) return {l.size(), true};
    return {pad_pos - 1, true};
}

// ---- moveReshapeBefore ----------------------------------------------------------------------------------
Result move_reshape_before(List& l, size_t cur, const Type& base) {
    if (cur == 0 || cur >= l.size()) return {cur, false};
    if (l[cur].t.kind != VF_T_RESHAPE) return {cur, false};
    const Item& prev = l[cur - 1];
    const Type prev_in = infer_prefix(base, l, cur - 1);
    switch (prev.t.kind) {
    case VF_T_ADD:
    case VF_T_RESCALE: break;
    case VF_T_CAST_ELEM_TYPE:  // not for casts that behave like QuantCast (:326-336)
        if (prev_in.elem.quantized() || prev.elem.quantized()) return {cur, false};
        break;
    case VF_T_DEQUANTIZE:
        if (prev_in.elem.kind == VF_ELEM_QUANT_PER_AXIS) {  // prepareDequantizeSwap (:338-378)
            // the quantized axis must be found again in the new shape, counting from the innermost dim; the
            // Reshape then becomes a ChangeShapeAndElemType that carries the per-axis type with the new axis
            Item& reshape = l[cur];
            const int dim = prev_in.elem.axis;
            int64_t in_lower = 1;
            for (int i = dim; i < prev_in.rank; ++i) in_lower *= prev_in.shape[i];
            int64_t out_lower = 1;
            int new_dim = reshape.t.rank - 1;
            for (; new_dim >= 0; --new_dim) {
                out_lower *= reshape.t.a[new_dim];
                if (out_lower >= in_lower) break;
            }
            if (new_dim < 0 || out_lower != in_lower || reshape.t.a[new_dim] != prev_in.shape[dim]) return {cur, false};
            reshape.t.kind = VF_T_CHANGE_SHAPE_AND_ELEM_TYPE;
            reshape.elem = prev_in.elem;
            reshape.elem.axis = new_dim;
        }
        break;
    default: return {cur, false};
    }
    std::swap(l[cur - 1], l[cur]);
    return {cur - 1, true};
}

void add_transformation(List& l, Item item, const Type& base) {
    // upper bound on the position requirement keeps [NONE..., PREFERRED_LAST..., LAST...] stable
    size_t pos = l.size();
    for (size_t i = 0; i < l.size(); ++i) {
        if (position(l[i].t.kind) > position(item.t.kind)) {
            pos = i;
            break;
        }
    }
    l.insert(l.begin() + long(pos), std::move(item));
    using Rule = Result (*)(List&, size_t, const Type&);
    const Rule rules[] = {fuse_consecutive, fold_noop, move_subview_before, move_reshape_before};
    bool optimized = true;
    size_t cur = pos;
    int guard = 0;
    while (optimized) {
        optimized = false;
        for (Rule rule : rules) {
            const Result r = rule(l, cur, base);
            if (r.second) {
                cur = r.first;
                optimized = true;
                break;
            }
        }
        if (++guard > 10000) raise(VF_ERR_INVALID_ARG, "transformation list does not reach a fixed point");
    }
    const size_t n = l.size();
    if (n >= 2 && position(l[n - 2].t.kind) == 2) raise(VF_ERR_POSITION, "At most 1 attribute with LAST requirement allowed!");
}

}  // namespace

}  // namespace vf

extern "C" int vf_optimize_transforms(const vf_tensor_type* base, const vf_transform* t, int n, vf_transform* out, int out_cap,
                                      int* n_out, double* scales_buf, int64_t* zps_buf, int64_t params_cap, char* err,
                                      size_t errlen) {
    using namespace vf;
    return guard(err, errlen, [&] {
        if (!base || (n > 0 && !t) || n < 0 || !out || !n_out) raise(VF_ERR_INVALID_ARG, "NULL argument");
        const Type bt = Type::from(*base);
        List l;
        for (int i = 0; i < n; ++i) {
            Item it;
            it.t = t[i];
            const int k = t[i].kind;
            if (k == VF_T_CAST_ELEM_TYPE || k == VF_T_CONVERT_ELEM_TYPE || k == VF_T_QUANTIZE || k == VF_T_CHANGE_SHAPE_AND_ELEM_TYPE) it.elem = Elem::from(t[i].elem);
            if (k == VF_T_SPARSIFY && t[i].num_actual) it.counts.assign(t[i].num_actual, t[i].num_actual + t[i].n_num_actual);
            add_transformation(l, std::move(it), bt);
        }
        if (int(l.size()) > out_cap) raise(VF_ERR_BUFFER_TOO_SMALL, "optimised list has %zu entries, room for %d", l.size(), out_cap);
        int64_t used = 0;
        for (size_t i = 0; i < l.size(); ++i) {
            vf_transform o = pod_of(l[i]);
            const int64_t np = int64_t(l[i].elem.scales.size());
            if (np > 0) {  // quantization parameters move into the caller's buffers
                if (!scales_buf || !zps_buf || used + np > params_cap)
                    raise(VF_ERR_BUFFER_TOO_SMALL, "optimised list carries more than %lld quantization parameters", (long long)params_cap);
                std::copy(l[i].elem.scales.begin(), l[i].elem.scales.end(), scales_buf + used);
                std::copy(l[i].elem.zps.begin(), l[i].elem.zps.end(), zps_buf + used);
                o.elem.scales = scales_buf + used;
                o.elem.zps = zps_buf + used;
                used += np;
            }
            if (!l[i].counts.empty()) {  // numActualElements: the rules never rewrite them, point back at the input
                for (int j = 0; j < n; ++j)
                    if (t[j].kind == VF_T_SPARSIFY && t[j].num_actual) {
                        o.num_actual = t[j].num_actual;
                        o.n_num_actual = t[j].n_num_actual;
                    }
            }
            out[i] = o;
        }
        *n_out = int(l.size());
    });
}
