// Fold executor: Const::ContentAttr::fold() + Const::Content::copyTo() on the device
// (attributes/content.cpp:371-397, utils/content.cpp:161-184), plus the remaining C entry points.
#include <algorithm>
#include <cmath>

#include "fold_internal.h"
#include "fused.h"

namespace vf {

namespace {

void strides_of(const int64_t* shape, int rank, int64_t* st) {
    int64_t s = 1;
    for (int i = rank - 1; i >= 0; --i) {
        st[i] = s;
        s *= shape[i];
    }
}

template <class T>
DBuf upload_vec(vf_ctx* ctx, const std::vector<T>& v) {
    DBuf b(ctx, v.size() * sizeof(T));
    copy_in(ctx, b.p, v.data(), v.size() * sizeof(T), VF_MEM_HOST);
    return b;
}
template <class T>
DBuf upload_vec(vf_ctx* ctx, const Params<T>& v) {
    DBuf b(ctx, v.size() * sizeof(T));
    copy_in(ctx, b.p, v.data(), v.size() * sizeof(T), VF_MEM_HOST);
    return b;
}

// wrapBaseContent (attributes/content.cpp:310-318): device memory is borrowed, host memory is uploaded
DContent upload_base(vf_ctx* ctx, const vf_content& b, vf_stats* stats) {
    DContent c;
    c.type = Type::from(b.type);
    c.storage = b.storage_dtype;
    c.splat = b.is_splat != 0;
    const uint64_t need = (uint64_t(dtype_bits(c.storage)) * uint64_t(c.count()) + 7u) / 8u;
    if (!b.data || b.nbytes < need) raise(VF_ERR_SHAPE, "base buffer holds %llu bytes, %llu needed", (unsigned long long)b.nbytes, (unsigned long long)need);
    c.nbytes = need;
    if (b.mem_kind == VF_MEM_DEVICE) {
        c.d = b.data;
    } else {
        c.own = DBuf(ctx, need);
        copy_in(ctx, c.own.p, b.data, need, b.mem_kind);
        c.d = c.own.p;
        if (stats) stats->h2d_bytes += need;
    }
    if (stats) stats->bytes_in += need;
    return c;
}

DContent alloc_like(vf_ctx* ctx, const Type& type, int storage, bool splat, int64_t raw_bytes = -1) {
    DContent c;
    c.type = type;
    c.storage = storage;
    c.splat = splat;
    c.nbytes = raw_bytes >= 0 ? uint64_t(raw_bytes) : (uint64_t(dtype_bits(storage)) * uint64_t(c.count()) + 7u) / 8u;
    // A dense buffer whose storage is the logical element type is what copyTo would copy byte for byte: write it
    // where it has to end up. (If this turns out to be a scratch buffer of the transformation, the result is
    // copied over it afterwards, in stream order.)
    // (a sub-byte logical type is copied as stored whenever the destination holds all of it)
    const bool as_stored = (storage == type.elem.dtype && dtype_bits(storage) >= 8) || dtype_bits(type.elem.dtype) < 8;
    if (ctx->final_dst && !splat && as_stored && c.nbytes > 0 &&
        c.nbytes <= ctx->final_bytes && (reinterpret_cast<uintptr_t>(ctx->final_dst) & 15u) == 0) {
        c.own = DBuf::borrow(ctx->final_dst, c.nbytes);
        ctx->final_dst = nullptr;
    } else {
        c.own = DBuf(ctx, c.nbytes);
    }
    c.d = c.own.p;
    return c;
}

void axis_sizes(const Type& t, int axis, int64_t& outer, int64_t& axis_size, int64_t& inner) {
    int p[VF_MAX_RANK];
    int64_t ms[VF_MAX_RANK];
    t.perm(p);
    t.mem_shape(ms);
    int m = 0;
    for (int i = 0; i < t.rank; ++i)
        if (p[i] == axis) m = i;
    inner = 1;
    for (int i = m + 1; i < t.rank; ++i) inner *= ms[i];
    axis_size = ms[m];
    if (inner == 0) raise(VF_ERR_SHAPE, "Inner size is zero");
    if (axis_size == 0) raise(VF_ERR_SHAPE, "Quantized axis size is zero");
    outer = t.numel() / (axis_size * inner);
    if (outer == 0) raise(VF_ERR_SHAPE, "Outer size is zero");
}

// ---- host conversions of a zero point into a storage element (Content::fillWithZero) -----------------
uint16_t host_f32_to_f16(float f) {  // IEEE round-to-nearest-even; zero points are small integers
    uint32_t u;
    std::memcpy(&u, &f, 4);
    const uint32_t sign = (u >> 16) & 0x8000u;
    const int32_t e = int32_t((u >> 23) & 0xFF) - 127 + 15;
    uint32_t m = u & 0x7FFFFFu;
    if (((u >> 23) & 0xFF) == 0xFF) return uint16_t(sign | 0x7C00u | (m ? 0x200u : 0));
    if (e >= 31) return uint16_t(sign | 0x7C00u);
    if (e <= 0) {
        if (e < -10) return uint16_t(sign);
        m |= 0x800000u;
        const int sh = 14 - e;
        uint32_t r = m >> sh;
        const uint32_t rem = m & ((1u << sh) - 1), half = 1u << (sh - 1);
        if (rem > half || (rem == half && (r & 1))) ++r;
        return uint16_t(sign | r);
    }
    uint32_t r = (uint32_t(e) << 10) | (m >> 13);
    const uint32_t rem = m & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (r & 1))) ++r;
    return uint16_t(sign | r);
}

void zp_to_storage(int storage, int64_t zp, uint8_t* out) {
    switch (storage) {
    case VF_DT_F32: {
        const float f = float(zp);
        if (int64_t(f) != zp) raise(VF_ERR_CHECKED_CAST, "zero point %lld is not representable in f32", (long long)zp);
        std::memcpy(out, &f, 4);
        return;
    }
    case VF_DT_F16: {
        const uint16_t h = host_f32_to_f16(float(zp));
        std::memcpy(out, &h, 2);
        return;
    }
    case VF_DT_BF16: {
        const float f = float(zp);
        uint32_t u;
        std::memcpy(&u, &f, 4);
        const uint16_t h = uint16_t((u + ((u & 0x00010000u) >> 1)) >> 16);
        std::memcpy(out, &h, 2);
        return;
    }
    default: {
        double lo, hi;
        dtype_int_limits(storage, lo, hi);
        if (double(zp) < lo || double(zp) > hi) raise(VF_ERR_CHECKED_CAST, "zero point %lld outside the storage type", (long long)zp);
        std::memcpy(out, &zp, size_t(dtype_bits(storage) / 8));  // little endian
    }
    }
}

// getSparsifyValue — utils/sparsity.cpp:12-26
int64_t sparsify_value(const Elem& e) {
    if (!e.quantized()) return 0;
    int64_t zp;
    if (!e.single_zp(zp)) raise(VF_ERR_ZERO_POINTS, "Not all zero-points are equal");
    if (zp != 0 && (e.dtype == VF_DT_F8E4M3FN || e.dtype == VF_DT_F8E5M2))
        raise(VF_ERR_UNSUPPORTED, "8-bit float storage with a non-zero zero point");
    return zp;
}

void check_sparse_dtype(int dt) {
    if (dt != VF_DT_I8 && dt != VF_DT_U8 && dt != VF_DT_F16 && dt != VF_DT_BF16 && dt != VF_DT_F32 && dt != VF_DT_F8E4M3FN &&
        dt != VF_DT_F8E5M2)
        raise(VF_ERR_UNSUPPORTED, "Unexpected weights data type: %d", dt);
}

// the view getValues<LogicalT>() gives: a dense buffer in the logical element type
DContent materialise_logical(vf_ctx* ctx, DContent& in) {
    const int dt = in.type.elem.dtype;
    if (in.storage == dt && !in.splat) {
        DContent v;
        v.type = in.type;
        v.storage = dt;
        v.d = in.d;
        v.nbytes = in.nbytes;
        return v;
    }
    DContent v = alloc_like(ctx, in.type, dt, false);
    launch_convert(ctx, in.d, in.storage, in.splat, v.own.p, dt, in.type.numel());
    return v;
}

// ------------------------------------------------------------------------------------------------------
// one transformation
// ------------------------------------------------------------------------------------------------------
DContent move_buffer(DContent& in, const Type& t) {  // Content::moveBuffer
    DContent out = std::move(in);
    out.type = t;
    return out;
}

DContent do_quantize(vf_ctx* ctx, DContent& in, const vf_transform& t) {
    bool os;
    const Type ot = infer_one(in.type, in.splat, t, os);
    const Elem q = Elem::from(t.elem);
    const bool per_axis = q.kind == VF_ELEM_QUANT_PER_AXIS;
    DContent out = alloc_like(ctx, ot, q.dtype, per_axis ? false : in.splat);
    int64_t axis_size = 1, inner = 1, outer = 1;
    if (per_axis) {
        axis_sizes(in.type, q.axis, outer, axis_size, inner);
        if (int64_t(q.scales.size()) != axis_size) raise(VF_ERR_SHAPE, "Wrong scales size '%zu', expected '%lld'", q.scales.size(), (long long)axis_size);
        if (int64_t(q.zps.size()) != axis_size) raise(VF_ERR_SHAPE, "Wrong zeroPoints size '%zu', expected '%lld'", q.zps.size(), (long long)axis_size);
    }
    DBuf ds = upload_vec(ctx, q.scales), dz = upload_vec(ctx, q.zps);
    launch_quantize(ctx, in.d, in.storage, in.splat, out.own.p, q.dtype, out.count(), ds.as<double>(), dz.as<int64_t>(),
                    axis_size, inner, q.qmin, q.qmax);
    return out;
}

DContent do_dequantize(vf_ctx* ctx, DContent& in, const vf_transform& t) {
    bool os;
    const Type ot = infer_one(in.type, in.splat, t, os);
    const Elem& q = in.type.elem;
    DContent out = alloc_like(ctx, ot, VF_DT_F32, os);
    int64_t axis_size = 1, inner = 1, outer = 1;
    if (q.kind == VF_ELEM_QUANT_PER_AXIS) {
        axis_sizes(in.type, q.axis, outer, axis_size, inner);
        if (int64_t(q.scales.size()) != axis_size || int64_t(q.zps.size()) != axis_size) raise(VF_ERR_SHAPE, "Wrong scales size");
    }
    DBuf ds = upload_vec(ctx, q.scales), dz = upload_vec(ctx, q.zps);
    launch_dequantize(ctx, in.d, in.storage, in.splat, out.own.as<float>(), out.count(), ds.as<double>(),
                      dz.as<int64_t>(), axis_size, inner);
    return out;
}

DContent do_rescale_add(vf_ctx* ctx, DContent& in, const Type& ot, double value, bool is_add) {
    DContent out = alloc_like(ctx, ot, VF_DT_F32, in.splat);
    launch_rescale_add(ctx, in.d, in.storage, in.splat, out.own.as<float>(), out.count(), float(value), is_add);
    return out;
}

DContent do_convert(vf_ctx* ctx, DContent& in, const vf_transform& t) {
    bool os;
    const Type ot = infer_one(in.type, in.splat, t, os);
    const Elem &qi = in.type.elem, &qo = ot.elem;
    if (qi.quantized() && qo.quantized()) {
        // getValueRangeOffset — utils/transformations.cpp:863-881
        int64_t zi, zo;
        if (!dtype_is_int(qi.dtype) || !dtype_is_int(qo.dtype) || dtype_bits(qi.dtype) != dtype_bits(qo.dtype) ||
            !qi.single_zp(zi) || !qo.single_zp(zo))
            raise(VF_ERR_UNSUPPORTED, "Unsupported conversion between quantized types");
        return do_rescale_add(ctx, in, ot, double(zo - zi), true);
    }
    if (qi.quantized()) raise(VF_ERR_UNSUPPORTED, "Unsupported conversion from a quantized type to a plain one");
    // sub-byte unpacking — convert_elem_type.cpp:66-79, utils/convert_utils.cpp:17-75. Signless types travel as
    // the unsigned dtypes of this ABI, so "same signedness" is (i4 -> i8) or (u4 -> u8); 1-bit inputs go
    // anywhere and always take the masking branch.
    const int bits = dtype_bits(qi.dtype);
    const bool out_byte = qo.dtype == VF_DT_I8 || qo.dtype == VF_DT_U8;
    const bool same_sign = dtype_is_signed(qi.dtype) == dtype_is_signed(qo.dtype);
    if (!qo.quantized() && dtype_is_int(qi.dtype) && bits < 8 && out_byte && (same_sign || bits == 1) && in.storage == qi.dtype) {
        const bool sign = qo.dtype == VF_DT_I8 && bits != 1;
        DContent out = alloc_like(ctx, ot, qo.dtype, in.splat);
        if (in.splat) {
            // the masking branch unpacks the first element of the byte, the sign-extending branch the last one
            // (convert_utils.cpp:33-36, 53-56): one byte in, one element out
            uint8_t src = 0;
            VF_CUDA(cudaMemcpyAsync(&src, in.d, 1, cudaMemcpyDeviceToHost, ctx->stream));
            VF_CUDA(cudaStreamSynchronize(ctx->stream));
            const uint8_t v = sign ? uint8_t(int8_t(src) >> (8 - bits)) : uint8_t(src & ((1u << bits) - 1u));
            copy_in(ctx, out.own.p, &v, 1, VF_MEM_HOST);
            VF_CUDA(cudaStreamSynchronize(ctx->stream));  // `v` leaves scope
        } else {
            launch_unpack_subbyte(ctx, static_cast<const uint8_t*>(in.d), out.own.as<uint8_t>(), ot.numel(), bits, sign);
        }
        return out;
    }
    raise(VF_ERR_UNSUPPORTED, "Unsupported conversion: neither quantized -> quantized nor a sub-byte unpack");
}

DContent do_permute(vf_ctx* ctx, DContent& in, const Type& ot, const int* mp) {
    const int rank = in.type.rank;
    bool ident = true;
    for (int i = 0; i < rank; ++i) ident &= mp[i] == i;
    if (in.splat || ident) return move_buffer(in, ot);
    const int bits = dtype_bits(in.storage);
    if (bits < 8) raise(VF_ERR_UNSUPPORTED, "memory permutation of sub-byte storage");
    DContent out = alloc_like(ctx, ot, in.storage, false);
    if (out.nbytes != in.nbytes) raise(VF_ERR_SHAPE, "Storage buffer size mismatch in 'memPermuteTransformation'");
    Geom g{};
    g.rank = rank;
    int64_t ims[VF_MAX_RANK], ist[VF_MAX_RANK];
    in.type.mem_shape(ims);
    strides_of(ims, rank, ist);
    for (int i = 0; i < rank; ++i) {
        g.in_shape[i] = ims[i];
        g.out_shape[i] = ims[mp[i]];
        g.src_stride[i] = ist[mp[i]];
    }
    launch_permute(ctx, in.d, out.own.p, g, bits / 8);
    return out;
}

DContent do_reorder(vf_ctx* ctx, DContent& in, const vf_transform& t) {
    bool os;
    const Type ot = infer_one(in.type, in.splat, t, os);
    int ip[VF_MAX_RANK], op[VF_MAX_RANK], mp[VF_MAX_RANK];
    in.type.perm(ip);
    ot.perm(op);
    for (int i = 0; i < ot.rank; ++i)
        for (int j = 0; j < ot.rank; ++j)
            if (ip[j] == op[i]) mp[i] = j;
    return do_permute(ctx, in, ot, mp);
}

DContent do_transpose(vf_ctx* ctx, DContent& in, const vf_transform& t) {
    bool os;
    const Type ot = infer_one(in.type, in.splat, t, os);
    int mp[VF_MAX_RANK];
    if (t.kind == VF_T_MEM_PERMUTE) {
        order_to_perm(t.mem_perm, in.type.rank, mp);
    } else {
        int ip[VF_MAX_RANK], p[VF_MAX_RANK];
        in.type.perm(ip);
        order_to_perm(t.order, in.type.rank, p);
        for (int i = 0; i < in.type.rank; ++i) {
            const int in_logical = p[ip[i]];
            for (int j = 0; j < in.type.rank; ++j)
                if (ip[j] == in_logical) mp[i] = j;
        }
    }
    return do_permute(ctx, in, ot, mp);
}

// fill values of Content::fillWithZero (utils/content.cpp:190-237) for a buffer of type `ot` stored as `storage`:
// zero, the zero point, or one zero point per output channel (`fill_dim` = memory dim that holds dim 0)
void zero_fill_values(const Type& ot, int storage, std::vector<uint8_t>& fill, int64_t& n_fill, int& fill_dim) {
    const int es = dtype_bits(storage) / 8;
    int p[VF_MAX_RANK];
    ot.perm(p);
    n_fill = 1;
    fill_dim = 0;
    const Elem& e = ot.elem;
    if (e.kind == VF_ELEM_QUANT_PER_AXIS) {
        if (ot.rank != 4) raise(VF_ERR_UNSUPPORTED, "Unsupported shape size %d", ot.rank);
        if (e.axis != 0) raise(VF_ERR_UNSUPPORTED, "Only per-channel quantization is supported");
        n_fill = ot.shape[0];
        fill.assign(size_t(n_fill) * es, 0);
        for (int64_t i = 0; i < n_fill; ++i) zp_to_storage(storage, e.zps[size_t(i)], fill.data() + i * es);
        for (int i = 0; i < ot.rank; ++i)
            if (p[i] == 0) fill_dim = i;
    } else if (e.kind == VF_ELEM_QUANT_UNIFORM) {
        fill.assign(size_t(es), 0);
        zp_to_storage(storage, e.zps[0], fill.data());
    } else {
        fill.assign(size_t(es), 0);
    }
}

DContent do_pad(vf_ctx* ctx, DContent& in, const vf_transform& t) {
    bool os;
    const Type ot = infer_one(in.type, in.splat, t, os);
    const int bits = dtype_bits(in.storage);
    if (bits < 8) raise(VF_ERR_UNSUPPORTED, "PadWithZero of sub-byte storage");
    const int es = bits / 8;
    DContent out = alloc_like(ctx, ot, in.storage, false);
    const int rank = in.type.rank;
    int p[VF_MAX_RANK];
    int64_t ims[VF_MAX_RANK], oms[VF_MAX_RANK], ist[VF_MAX_RANK];
    in.type.perm(p);
    in.type.mem_shape(ims);
    ot.mem_shape(oms);
    strides_of(ims, rank, ist);
    Geom g{};
    g.rank = rank;
    for (int i = 0; i < rank; ++i) {
        g.in_shape[i] = ims[i];
        g.out_shape[i] = oms[i];
        g.src_stride[i] = ist[i];
        g.offset[i] = t.a[p[i]];
    }
    std::vector<uint8_t> fill;
    int64_t n_fill = 1;
    int fill_dim = 0;
    zero_fill_values(ot, in.storage, fill, n_fill, fill_dim);
    DBuf dfill = upload_vec(ctx, fill);
    launch_pad(ctx, in.d, in.splat, out.own.p, g, es, dfill.p, n_fill, fill_dim);
    return out;
}

DContent do_subview(vf_ctx* ctx, DContent& in, const vf_transform& t) {
    bool os;
    const Type ot = infer_one(in.type, in.splat, t, os);
    if (in.splat) return move_buffer(in, ot);
    const int bits = dtype_bits(in.storage);
    DContent out = alloc_like(ctx, ot, in.storage, false);
    const int rank = in.type.rank;
    int p[VF_MAX_RANK];
    int64_t ims[VF_MAX_RANK], oms[VF_MAX_RANK], ist[VF_MAX_RANK];
    in.type.perm(p);
    in.type.mem_shape(ims);
    ot.mem_shape(oms);
    strides_of(ims, rank, ist);
    Geom g{};
    g.rank = rank;
    for (int i = 0; i < rank; ++i) {
        g.in_shape[i] = ims[i];
        g.out_shape[i] = oms[i];
        g.src_stride[i] = ist[i];
        g.offset[i] = t.a[p[i]];
    }
    if (bits < 8) launch_subview_subbyte(ctx, in.d, out.own.p, g, bits);  // subByteTransform, subview.cpp:20-160
    else launch_subview(ctx, in.d, out.own.p, g, bits / 8);
    return out;
}

DContent do_bitpack(vf_ctx* ctx, DContent& in, const vf_transform& t) {
    if (in.splat) raise(VF_ERR_SPLAT, "Bit pack does not support splat inputs.");
    bool os;
    const Type ot = infer_one(in.type, in.splat, t, os);
    const int64_t n = in.type.numel();
    if (n % 2 != 0) raise(VF_ERR_ODD_COUNT, "Storage buffer size is odd, which is unexpected for 4 bit packing.");
    if (dtype_bits(in.storage) < 8) raise(VF_ERR_UNSUPPORTED, "BitPack of sub-byte storage");
    DContent out = alloc_like(ctx, ot, VF_DT_U8, false, int64_t(ot.alloc_bytes()));
    launch_bitpack4(ctx, in.d, in.storage, out.own.as<uint8_t>(), n);
    return out;
}

DContent do_sparsity_map(vf_ctx* ctx, DContent& in, const vf_transform& t) {
    bool os;
    const Type ot = infer_one(in.type, in.splat, t, os);
    check_sparse_dtype(in.type.elem.dtype);
    const int64_t sv = sparsify_value(in.type.elem);
    const int64_t work = in.type.shape[1] * in.type.shape[2] * in.type.shape[3];
    if (work % 8 != 0) raise(VF_ERR_SHAPE, "GetSparsityMap needs IC*KY*KX (%lld) to be a multiple of 8", (long long)work);
    DContent v = materialise_logical(ctx, in);
    DContent out = alloc_like(ctx, ot, VF_DT_I1, false);
    launch_sparsity_scan(ctx, v.d, v.storage, ot.shape[0], work, sv, nullptr, out.own.as<uint8_t>(), ot.shape[3] / 8);
    return out;
}

// Sparsify — attributes/sparsify.cpp:163-203. The folded content always carries the compressed type.
DContent do_sparsify(vf_ctx* ctx, DContent& in, const vf_transform& t, DBuf* keep_counts = nullptr) {
    if (in.type.rank != 4) raise(VF_ERR_SHAPE, "Expected 4D input shape");
    const int dt = in.type.elem.dtype;
    check_sparse_dtype(dt);
    const int es = dtype_bits(dt) / 8;
    const int64_t sv = sparsify_value(in.type.elem);
    if ((dt == VF_DT_I8 && (sv < -128 || sv > 127)) || (dt == VF_DT_U8 && (sv < 0 || sv > 255)))
        raise(VF_ERR_CHECKED_CAST, "sparsify value %lld outside the element type", (long long)sv);
    const int64_t oc = in.type.shape[0], work = in.type.shape[1] * in.type.shape[2] * in.type.shape[3];
    DContent v = materialise_logical(ctx, in);

    DBuf counts(ctx, size_t(oc) * 8), offsets(ctx, size_t(oc + 1) * 8);
    launch_sparsity_scan(ctx, v.d, dt, oc, work, sv, counts.as<int64_t>(), nullptr, 0);
    launch_sparse_offsets(ctx, counts.as<int64_t>(), oc, es, offsets.as<int64_t>());

    uint64_t capacity;
    Type ot;
    const bool supplied = t.num_actual != nullptr;
    if (supplied) {
        if (t.n_num_actual != oc) raise(VF_ERR_SHAPE, "numActualElements has %lld entries for %lld channels", (long long)t.n_num_actual, (long long)oc);
        ot = compress_type(in.type, t.num_actual, t.n_num_actual);
        capacity = uint64_t(ot.shape[0]);
    } else {
        capacity = uint64_t(oc) * uint64_t(align_up(work * es, 16));
    }
    DBuf data(ctx, capacity ? capacity : 1);
    if (supplied) VF_CUDA(cudaMemsetAsync(data.p, 0, capacity, ctx->stream));
    launch_sparse_compact(ctx, v.d, dt, oc, work, sv, offsets.as<int64_t>(), data.as<uint8_t>(), capacity);
    if (!supplied) {
        int64_t total = 0;
        VF_CUDA(cudaMemcpyAsync(&total, offsets.as<int64_t>() + oc, 8, cudaMemcpyDeviceToHost, ctx->stream));
        VF_CUDA(cudaStreamSynchronize(ctx->stream));
        ot = Type();
        ot.rank = 4;
        ot.order = in.type.order;
        ot.shape[0] = total;
        ot.shape[1] = ot.shape[2] = ot.shape[3] = 1;
        ot.elem = Elem::plain(VF_DT_U8);
    }
    DContent out;
    out.type = ot;
    out.storage = VF_DT_U8;
    out.splat = false;
    out.nbytes = uint64_t(ot.shape[0]);
    out.own = std::move(data);
    out.d = out.own.p;
    if (keep_counts) *keep_counts = std::move(counts);
    return out;
}

DContent do_swizzle(vf_ctx* ctx, DContent& in, const vf_transform& t);
DContent do_relocate(vf_ctx* ctx, DContent& in, const vf_transform& t);
DContent do_reverse(vf_ctx* ctx, DContent& in, const vf_transform& t);
DContent do_broadcast(vf_ctx* ctx, DContent& in, const vf_transform& t);
DContent do_expand_dilated(vf_ctx* ctx, DContent& in, const vf_transform& t);
DContent do_inverse(vf_ctx* ctx, DContent& in, const vf_transform& t);

DContent apply(vf_ctx* ctx, DContent& in, const vf_transform& t) {
    bool os;
    switch (t.kind) {
    case VF_T_CAST_ELEM_TYPE:
    case VF_T_RESHAPE:
    case VF_T_CHANGE_SHAPE_AND_ELEM_TYPE:
    case VF_T_LAYOUT_CAST: {
        const Type ot = infer_one(in.type, in.splat, t, os);
        return move_buffer(in, ot);
    }
    case VF_T_CONVERT_ELEM_TYPE: return do_convert(ctx, in, t);
    case VF_T_DEQUANTIZE: return do_dequantize(ctx, in, t);
    case VF_T_QUANTIZE: return do_quantize(ctx, in, t);
    case VF_T_RESCALE: return do_rescale_add(ctx, in, in.type, t.value, false);
    case VF_T_ADD: return do_rescale_add(ctx, in, in.type, t.value, true);
    case VF_T_REORDER: return do_reorder(ctx, in, t);
    case VF_T_MEM_PERMUTE:
    case VF_T_TRANSPOSE: return do_transpose(ctx, in, t);
    case VF_T_PAD_WITH_ZERO: return do_pad(ctx, in, t);
    case VF_T_SUBVIEW: return do_subview(ctx, in, t);
    case VF_T_BIT_PACK: return do_bitpack(ctx, in, t);
    case VF_T_GET_SPARSITY_MAP: return do_sparsity_map(ctx, in, t);
    case VF_T_SPARSIFY: return do_sparsify(ctx, in, t);
    case VF_T_SWIZZLE_CONSTANT: return do_swizzle(ctx, in, t);
    case VF_T_RELOCATE_WEIGHTS_TABLE: return do_relocate(ctx, in, t);
    case VF_T_REVERSE: return do_reverse(ctx, in, t);
    case VF_T_BROADCAST: return do_broadcast(ctx, in, t);
    case VF_T_EXPAND_DILATED: return do_expand_dilated(ctx, in, t);
    case VF_T_SCALAR_MULT_INVERSE: return do_inverse(ctx, in, t);
    default: raise(VF_ERR_INVALID_ARG, "unknown transformation kind %d", t.kind);
    }
}

// Content::copyTo — utils/content.cpp:161-184 (+ copySubByteContent :101-155)
uint64_t copy_to(vf_ctx* ctx, DContent& c, void* dst, uint64_t dst_bytes, int dst_kind, vf_stats* stats) {
    const int edt = c.type.elem.dtype;
    const int bits = dtype_bits(edt);
    const bool to_dev = dst_kind == VF_MEM_DEVICE;
    uint64_t written = 0;
    auto emit = [&](const void* dev_src, uint64_t n) {  // result already in a device buffer
        if (dev_src != dst) copy_out(ctx, dst, dst_kind, dev_src, n);
        if (!to_dev && stats) stats->d2h_bytes += n;
        written = n;
    };
    if (!dst && dst_bytes) raise(VF_ERR_INVALID_ARG, "dst is NULL");
    if (bits < 8) {
        if (c.splat) {
            // every byte repeats the sub-byte value; read it on the host (one element)
            uint8_t raw[8] = {0};
            VF_CUDA(cudaMemcpyAsync(raw, c.d, size_t(std::max(1, dtype_bits(c.storage) / 8)), cudaMemcpyDeviceToHost, ctx->stream));
            VF_CUDA(cudaStreamSynchronize(ctx->stream));
            uint8_t sub;
            if (c.storage == VF_DT_I1) {
                sub = raw[0] & 1;
            } else {
                DBuf one(ctx, 1);
                launch_convert(ctx, c.d, c.storage, true, one.p, VF_DT_I8, 1);
                VF_CUDA(cudaMemcpyAsync(&sub, one.p, 1, cudaMemcpyDeviceToHost, ctx->stream));
                VF_CUDA(cudaStreamSynchronize(ctx->stream));
            }
            uint8_t byte = 0;
            for (int s = 0; s < 8 / bits; ++s) byte = uint8_t((byte << bits) + sub);
            DBuf tmp;
            void* target = dst;
            if (!to_dev) {
                tmp = DBuf(ctx, dst_bytes);
                target = tmp.p;
            }
            launch_fill_bytes(ctx, target, byte, dst_bytes);
            if (!to_dev) emit(tmp.p, dst_bytes);
            written = dst_bytes;
            return written;
        }
        if (dst_bytes < c.nbytes) {
            if (dst_bytes == 0 || c.nbytes % dst_bytes != 0) raise(VF_ERR_BUFFER_TOO_SMALL, "Cannot pack sub-byte elements into buffer: source data size '%llu', target data size '%llu'", (unsigned long long)c.nbytes, (unsigned long long)dst_bytes);
            const uint64_t n = c.nbytes / uint64_t(dtype_bits(c.storage) / 8);
            const uint64_t per = n / dst_bytes;
            if (per > 8 || (per & (per - 1)) != 0) raise(VF_ERR_SHAPE, "Invalid number of elements per byte '%llu'", (unsigned long long)per);
            DBuf tmp;
            void* target = dst;
            if (!to_dev) {
                tmp = DBuf(ctx, dst_bytes);
                target = tmp.p;
            }
            launch_pack_subbyte(ctx, c.d, c.storage, static_cast<uint8_t*>(target), int64_t(n), int(per));
            if (!to_dev) emit(tmp.p, dst_bytes);
            written = dst_bytes;
            return written;
        }
        emit(c.d, c.nbytes);
        return written;
    }
    if (!c.splat && edt == c.storage) {
        if (dst_bytes < c.nbytes) raise(VF_ERR_BUFFER_TOO_SMALL, "Byte sizes of the target buffer '%llu' is smaller then storage buffer '%llu'", (unsigned long long)dst_bytes, (unsigned long long)c.nbytes);
        emit(c.d, c.nbytes);
        return written;
    }
    const int64_t n = c.type.numel();
    const uint64_t need = uint64_t(n) * uint64_t(bits / 8);
    if (dst_bytes < need) raise(VF_ERR_BUFFER_TOO_SMALL, "Buffer with byte size '%llu' is not enough to hold actual elements with '%llu' byte size", (unsigned long long)dst_bytes, (unsigned long long)need);
    if (to_dev) {
        launch_convert(ctx, c.d, c.storage, c.splat, dst, edt, n);
        written = need;
    } else {
        DBuf tmp(ctx, need);
        launch_convert(ctx, c.d, c.storage, c.splat, tmp.p, edt, n);
        emit(tmp.p, need);
    }
    return written;
}

// SwizzleConstant — attributes/swizzle_transform.cpp:163-215: materialise the content as copyTo would, pad it
// to the swizzling-aligned size (zeros, or the first byte of a splat) and permute its RAM-cut chunks.
DContent do_swizzle(vf_ctx* ctx, DContent& in, const vf_transform& t) {
    bool os;
    const Type ot = infer_one(in.type, in.splat, t, os);
    const uint64_t in_total = in.type.alloc_bytes();
    const uint64_t new_size = uint64_t(align_up(int64_t(in_total), swizzle_size_alignment(int(t.a[1]))));
    DContent out;
    const bool plain = !in.splat && in.storage == in.type.elem.dtype && dtype_bits(in.storage) >= 8 && in.nbytes == in_total &&
                       (reinterpret_cast<uintptr_t>(in.d) & 15u) == 0;
    if (plain) {  // the storage bytes are what copyTo would produce: permute them straight from where they are
        out = alloc_like(ctx, ot, ot.elem.dtype, false, int64_t(new_size));
        launch_swizzle(ctx, in.d, in_total, 0, out.own.p, new_size, int(t.a[0]), int(t.a[1]));
        return out;
    }
    DBuf lin(ctx, new_size);
    copy_to(ctx, in, lin.p, in_total, VF_MEM_DEVICE, nullptr);
    if (new_size > in_total) {
        uint8_t pad = 0;
        if (in.splat) {
            VF_CUDA(cudaMemcpyAsync(&pad, lin.p, 1, cudaMemcpyDeviceToHost, ctx->stream));
            VF_CUDA(cudaStreamSynchronize(ctx->stream));
        }
        launch_fill_bytes(ctx, lin.as<uint8_t>() + in_total, pad, new_size - in_total);
    }
    out = alloc_like(ctx, ot, ot.elem.dtype, false, int64_t(new_size));
    if (in.splat) {  // every chunk holds the same bytes: nothing to permute
        VF_CUDA(cudaMemcpyAsync(out.own.p, lin.p, new_size, cudaMemcpyDeviceToDevice, ctx->stream));
    } else {
        launch_swizzle(ctx, lin.p, new_size, 0, out.own.p, new_size, int(t.a[0]), int(t.a[1]));
    }
    return out;
}

// RelocateWeightsTable — attributes/relocate_weights_table.cpp:203-292. The host prepares what depends on the
// attribute alone (cluster boundaries, and with weightsCompression the byte offset of every channel's
// compressed weight set); the kernel reads the pointer steps from the table itself and patches the rows.
DContent do_relocate(vf_ctx* ctx, DContent& in, const vf_transform& t) {
    bool os;
    const Type ot = infer_one(in.type, in.splat, t, os);
    const vf_relocate& r = t.relocate;
    DContent lin = materialise_logical(ctx, in);  // a splat is filled in, like the reference's copyTo into a temp buffer
    DContent out = alloc_like(ctx, ot, ot.elem.dtype, false);
    RelocateArgs a{};
    a.oc = r.weights_table_size / 4 / 4;  // numWTEntries / WEIGHT_TABLE_NUM_ELEMENTS_PER_OC
    a.n_clusters = r.n_clusters;
    a.sparsity_ptr = r.sparsity_ptr;
    if (r.channel_offset < INT32_MIN || r.channel_offset > INT32_MAX) raise(VF_ERR_CHECKED_CAST, "channelOffset %lld outside int32", (long long)r.channel_offset);
    a.channel_offset = int32_t(r.channel_offset);
    bool segmented = false;
    for (int c = 0; c < r.n_clusters; ++c) {
        a.weights_ptr[c] = r.weights_ptr[c];
        a.offsets[c] = r.offsets[c];
        if (c && r.offsets[c] != r.offsets[c - 1]) segmented = true;
    }
    // the reference walks the channels in order and moves to cluster c + 1 at the first channel >= offsets[c + 1],
    // one cluster per channel at most: cluster c + 1 starts at cross[c + 1]
    a.cross[0] = -1;
    for (int c = 1; c < r.n_clusters; ++c) a.cross[c] = segmented ? std::max(r.offsets[c], a.cross[c - 1] + 1) : INT64_MAX;
    DBuf d_steps;
    if (r.num_elems) {
        if (r.channel_offset < 0 || r.n_num_elems < a.oc + r.channel_offset)
            raise(VF_ERR_SHAPE, "Invalid weights compression with %lld elements for %lld channels", (long long)r.n_num_elems, (long long)a.oc);
        if (r.weights_elem_bit_size <= 0) raise(VF_ERR_INVALID_ARG, "Missing weights element type attribute");
        const int64_t alignment = r.alignment ? r.alignment : 16;  // VPU_WEIGHT_SET_BYTE_ALIGNMENT
        if (alignment < 0) raise(VF_ERR_INVALID_ARG, "negative weightsCompression alignment");
        auto set_bytes = [&](int64_t oc) { return align_up((r.num_elems[oc] * r.weights_elem_bit_size + 7) / 8, alignment); };
        int64_t front = 0;
        for (int64_t oc = 0; oc < r.channel_offset; ++oc) front += set_bytes(oc);
        a.wptr_offset = uint32_t(front);
        std::vector<int64_t> steps(size_t(std::max<int64_t>(a.oc, 1)));
        int64_t ptr = 0;
        int cl = 0;
        for (int64_t oc = 0; oc < a.oc; ++oc) {
            if (cl + 1 < r.n_clusters && oc >= a.cross[cl + 1]) {
                ++cl;
                ptr = 0;
            }
            steps[size_t(oc)] = ptr;
            ptr += set_bytes(oc + r.channel_offset);
        }
        d_steps = upload_vec(ctx, steps);
        a.d_steps = d_steps.as<int64_t>();
    }
    const uint64_t patched = uint64_t(std::max<int64_t>(a.oc, 0)) * 16;  // the kernel writes these rows whole
    if (out.nbytes > patched)
        VF_CUDA(cudaMemcpyAsync(static_cast<char*>(out.own.p) + patched, static_cast<const char*>(lin.d) + patched, out.nbytes - patched,
                                cudaMemcpyDeviceToDevice, ctx->stream));
    launch_relocate(ctx, static_cast<const int32_t*>(lin.d), out.own.as<int32_t>(), a);
    return out;
}

// Reverse — attributes/reverse.cpp:46-105: the content in its logical element type, every run of the dims
// behind `axis` reversed in place (raw buffer order)
DContent do_reverse(vf_ctx* ctx, DContent& in, const vf_transform& t) {
    bool os;
    const Type ot = infer_one(in.type, in.splat, t, os);
    if (in.splat) return move_buffer(in, ot);
    int64_t run = 1;
    for (int i = in.type.rank - 1; i > t.a[0]; --i) run *= in.type.shape[i];
    DContent lin = materialise_logical(ctx, in);
    DContent out = alloc_like(ctx, ot, ot.elem.dtype, false);
    launch_reverse(ctx, lin.d, out.own.p, ot.numel(), std::max<int64_t>(run, 1), dtype_bits(ot.elem.dtype) / 8);
    return out;
}

// Broadcast — attributes/broadcast.cpp:85-124: storage bytes; the block from the broadcast memory dim inwards
// is repeated value / extent times
DContent do_broadcast(vf_ctx* ctx, DContent& in, const vf_transform& t) {
    bool os;
    const Type ot = infer_one(in.type, in.splat, t, os);
    if (in.splat) return move_buffer(in, ot);
    const int bits = dtype_bits(in.storage);
    if (bits < 8) raise(VF_ERR_UNSUPPORTED, "Broadcast of sub-byte storage");
    int p[VF_MAX_RANK];
    int64_t ims[VF_MAX_RANK];
    in.type.perm(p);
    in.type.mem_shape(ims);
    int index = 0;
    for (int i = 0; i < in.type.rank; ++i)
        if (p[i] == t.a[0]) index = i;
    int64_t after = 1;
    for (int i = index; i < in.type.rank; ++i) after *= ims[i];
    const int64_t extent = ims[index], value = t.a[1];
    if (extent == 0 || value % extent) raise(VF_ERR_SHAPE, "Can't broadcast from %lld to %lld", (long long)extent, (long long)value);
    DContent out = alloc_like(ctx, ot, in.storage, false);
    launch_broadcast(ctx, in.d, out.own.p, ot.numel(), after, value / extent, bits / 8);
    return out;
}

// ExpandDilated — attributes/expand_dilated.cpp:88-131
DContent do_expand_dilated(vf_ctx* ctx, DContent& in, const vf_transform& t) {
    bool os;
    const Type ot = infer_one(in.type, in.splat, t, os);
    const int bits = dtype_bits(in.storage);
    if (bits < 8) raise(VF_ERR_UNSUPPORTED, "ExpandDilated of sub-byte storage");
    DContent out = alloc_like(ctx, ot, in.storage, false);
    std::vector<uint8_t> fill;
    int64_t n_fill = 1;
    int fill_dim = 0;
    zero_fill_values(ot, in.storage, fill, n_fill, fill_dim);
    int64_t oms[VF_MAX_RANK];
    ot.mem_shape(oms);
    int64_t fill_stride = 1;
    for (int i = fill_dim + 1; i < ot.rank; ++i) fill_stride *= oms[i];
    DBuf dfill = upload_vec(ctx, fill);
    launch_expand_dilated(ctx, in.d, in.splat, out.own.p, ot.numel(), ot.shape[2], ot.shape[3], in.type.shape[2], in.type.shape[3],
                          t.a[0], t.a[1], dfill.p, n_fill, fill_stride, oms[fill_dim], bits / 8);
    return out;
}

// ScalarMultInverse — attributes/inverse.cpp:52-66
DContent do_inverse(vf_ctx* ctx, DContent& in, const vf_transform& t) {
    bool os;
    const Type ot = infer_one(in.type, in.splat, t, os);
    DContent out = alloc_like(ctx, ot, VF_DT_F32, in.splat);
    launch_inverse(ctx, in.d, in.storage, out.own.as<float>(), out.count());
    return out;
}

struct CallScope {  // per-call bookkeeping: context lock, device, error flags, launch statistics
    vf_ctx* ctx;
    std::unique_lock<std::mutex> lock;
    DeviceGuard dev;
    uint64_t launches0;
    vf_stats* stats;
    CallScope(vf_ctx* c, vf_stats* s): ctx(check(c)), lock(c->mu), dev(c->device), launches0(c->launches), stats(s) {
        if (stats) std::memset(stats, 0, sizeof(*stats));
        flags_clear(ctx);
        if (stats && ctx->time_ev[0]) cudaEventRecord(ctx->time_ev[0], ctx->stream);
    }
    static vf_ctx* check(vf_ctx* c) {
        if (!c) raise(VF_ERR_INVALID_ARG, "ctx is NULL");
        return c;
    }
    bool finished = false;
    bool may_defer = false;  // set by calls that touched device memory only
    void finish() {
        if (may_defer && (ctx->opt_flags & VF_OPT_ASYNC)) {
            VF_CUDA(cudaGetLastError());
            ctx->deferred = true;  // the next synchronising call reports what these kernels found
        } else {
            const bool timed = stats && ctx->time_ev[0] && ctx->stream == ctx->main_stream;
            if (timed) cudaEventRecord(ctx->time_ev[1], ctx->stream);
            flags_check(ctx);
            if (timed) cudaEventElapsedTime(&stats->device_ms, ctx->time_ev[0], ctx->time_ev[1]);
        }
        finished = true;
        if (stats) stats->kernels_launched = int32_t(ctx->launches - launches0);
    }
    // A call that ends early (an exception on its way to the caller) still waits for what it enqueued: the
    // caller's buffers and the context's job-table area must not be in use once the call has returned.
    ~CallScope() {
        if (finished) return;
        cudaStreamSynchronize(ctx->main_stream);
        if (ctx->lane_stream) cudaStreamSynchronize(ctx->lane_stream);
        cudaGetLastError();
    }
};

void* out_ptr(vf_ctx* ctx, void* user, int kind, size_t bytes, DBuf& tmp) {
    if (!user) return nullptr;
    if (kind == VF_MEM_DEVICE) return user;
    tmp = DBuf(ctx, bytes);
    return tmp.p;
}
void out_flush(vf_ctx* ctx, void* user, int kind, size_t bytes, DBuf& tmp) {
    if (user && kind != VF_MEM_DEVICE) copy_out(ctx, user, kind, tmp.p, bytes);
}

int64_t unit_count(const Type& t, const vf_quant_spec& s, int64_t& unit_len) {
    if (t.order != identity_order(t.rank)) raise(VF_ERR_UNSUPPORTED, "weight quantization needs dim 0 outermost (row-major) input");
    if (s.group_size > 0) {
        const int64_t cols = t.shape[t.rank - 1];
        if (cols % s.group_size != 0) raise(VF_ERR_SHAPE, "group size %lld does not divide the row length %lld", (long long)s.group_size, (long long)cols);
        unit_len = s.group_size;
        return t.numel() / unit_len;
    }
    const int64_t units = t.shape[0];
    unit_len = units ? t.numel() / units : 0;
    return units;
}

void check_spec(const vf_quant_spec& s) {
    if (s.storage_dtype != VF_DT_I8 && s.storage_dtype != VF_DT_U8) raise(VF_ERR_UNSUPPORTED, "weight quantization stores i8 or u8 codes");
    double lo, hi;
    dtype_int_limits(s.storage_dtype, lo, hi);
    if (s.qmin >= s.qmax || double(s.qmin) < lo || double(s.qmax) > hi) raise(VF_ERR_INVALID_ARG, "storage range [%lld, %lld] does not fit the storage type", (long long)s.qmin, (long long)s.qmax);
    if (s.range_mode != VF_RANGE_MINMAX && s.range_mode != VF_RANGE_ABSMAX) raise(VF_ERR_INVALID_ARG, "unknown range mode");
    if (s.group_size < 0) raise(VF_ERR_INVALID_ARG, "negative group size");
}

}  // namespace

// Unfused composition with the general kernels: unit statistics, Quantize with the derived parameters, the
// remaining transformations, copyTo. Also the reference implementation the fused kernels are tested against.
static void quantize_fold_general(vf_ctx* ctx, DContent& base, const vf_quant_spec& spec, const vf_transform* t, int n,
                                  void* dst, uint64_t dst_bytes, int dst_kind, uint64_t* dst_written,
                                  const vf_quant_outputs* outs, vf_stats* stats) {
    int64_t unit_len = 0;
    const int64_t units = unit_count(base.type, spec, unit_len);
    if (base.splat) raise(VF_ERR_SPLAT, "weight quantization of a splat constant is not supported");
    if (base.storage != VF_DT_F32 && base.storage != VF_DT_F16 && base.storage != VF_DT_BF16)
        raise(VF_ERR_UNSUPPORTED, "weight quantization takes f32 / f16 / bf16 input");
    DBuf ds(ctx, size_t(units) * 8), dz(ctx, size_t(units) * 8);
    launch_unit_stats(ctx, base.d, base.storage, units, unit_len, spec.range_mode, spec.qmin, spec.qmax, ds.as<double>(),
                      dz.as<int64_t>(), nullptr, nullptr);
    Type ct = base.type;
    ct.elem = Elem::plain(spec.storage_dtype);
    DContent codes = alloc_like(ctx, ct, spec.storage_dtype, false);
    launch_quantize(ctx, base.d, base.storage, false, codes.own.p, spec.storage_dtype, ct.numel(), ds.as<double>(),
                    dz.as<int64_t>(), units, unit_len, spec.qmin, spec.qmax);
    if (outs) {
        const int k = outs->mem_kind;
        if (outs->scales) copy_out(ctx, outs->scales, k, ds.p, size_t(units) * 8);
        if (outs->zps) copy_out(ctx, outs->zps, k, dz.p, size_t(units) * 8);
        if (outs->scales_f16 || outs->zps_u4_packed) {
            DBuf t0, t1;
            const size_t zb = size_t((units + 1) / 2);
            uint16_t* d16 = static_cast<uint16_t*>(out_ptr(ctx, outs->scales_f16, k, size_t(units) * 2, t0));
            uint8_t* d4 = static_cast<uint8_t*>(out_ptr(ctx, outs->zps_u4_packed, k, zb, t1));
            launch_pack_params(ctx, ds.as<double>(), dz.as<int64_t>(), units, d16, d4);
            out_flush(ctx, outs->scales_f16, k, size_t(units) * 2, t0);
            out_flush(ctx, outs->zps_u4_packed, k, zb, t1);
        }
        if (outs->dequant) {
            // [CastElemType<q>, Dequantize] on the codes, then copyTo in the requested float type
            const int ddt = outs->dequant_dtype;
            if (ddt != VF_DT_F16 && ddt != VF_DT_F32 && ddt != VF_DT_BF16) raise(VF_ERR_UNSUPPORTED, "dequantized copy is f16 / bf16 / f32");
            const uint64_t need = uint64_t(ct.numel()) * uint64_t(dtype_bits(ddt) / 8);
            if (outs->dequant_bytes < need) raise(VF_ERR_BUFFER_TOO_SMALL, "dequantized copy needs %llu bytes", (unsigned long long)need);
            DBuf f32(ctx, size_t(ct.numel()) * 4), t2;
            launch_dequantize(ctx, codes.d, spec.storage_dtype, false, f32.as<float>(), ct.numel(), ds.as<double>(),
                              dz.as<int64_t>(), units, unit_len);
            void* dd = out_ptr(ctx, outs->dequant, k, need, t2);
            launch_convert(ctx, f32.p, VF_DT_F32, false, dd, ddt, ct.numel());
            out_flush(ctx, outs->dequant, k, need, t2);
            if (stats) stats->bytes_out += need;
        }
    }
    check_positions(t, n);
    DContent cur = std::move(codes);
    for (int i = 0; i < n; ++i) {
        DContent next = apply(ctx, cur, t[i]);
        cur = std::move(next);
    }
    const uint64_t w = copy_to(ctx, cur, dst, dst_bytes, dst_kind, stats);
    if (dst_written) *dst_written = w;
    if (stats) stats->bytes_out += w;
}

// ---- folding without copyTo (the background folder's cache keeps Const::Content objects) -----------------
static DContent borrow(const Folded& f) {  // a cached content as the executor's working type (nothing owned)
    DContent c;
    c.type = f.type;
    c.storage = f.storage;
    c.splat = f.splat;
    c.d = f.data;
    c.nbytes = f.nbytes;
    return c;
}

Folded fold_keep(vf_ctx* ctx, const vf_content* base, const Folded* resume, const vf_transform* t, int n) {
    if ((n > 0 && !t) || n < 0 || (!base && !resume)) raise(VF_ERR_INVALID_ARG, "NULL argument");
    check_positions(t, n);
    CallScope scope(ctx, nullptr);
    DContent cur = resume ? borrow(*resume) : upload_base(ctx, *base, nullptr);
    for (int i = 0; i < n; ++i) {
        DContent next = apply(ctx, cur, t[i]);
        cur = std::move(next);
    }
    Folded f;
    f.type = cur.type;
    f.type.elem.scales.own();  // the cache entry outlives the request whose arrays the type may borrow
    f.type.elem.zps.own();
    f.storage = cur.storage;
    f.splat = cur.splat;
    f.nbytes = cur.nbytes;
    // Content::copyUnownedBuffer: the cache owns its bytes, whatever the folded content borrowed
    VF_CUDA(cudaMallocAsync(&f.data, size_t(std::max<uint64_t>(f.nbytes, 1)), ctx->stream));
    cudaError_t e = f.nbytes ? cudaMemcpyAsync(f.data, cur.d, size_t(f.nbytes), cudaMemcpyDeviceToDevice, ctx->stream) : cudaSuccess;
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) {
        cudaFreeAsync(f.data, ctx->stream);
        raise(VF_ERR_CUDA, "copy of the folded content failed: %s", cudaGetErrorString(e));
    }
    try {
        scope.finish();
    } catch (...) {
        cudaFreeAsync(f.data, ctx->stream);
        throw;
    }
    return f;
}

void* upload_keep(vf_ctx* ctx, const vf_content& base, uint64_t* nbytes) {
    CallScope scope(ctx, nullptr);
    const uint64_t count = base.is_splat ? 1 : uint64_t(Type::from(base.type).numel());
    const uint64_t need = (uint64_t(dtype_bits(base.storage_dtype)) * count + 7u) / 8u;
    if (!base.data || base.nbytes < need) raise(VF_ERR_SHAPE, "base buffer holds %llu bytes, %llu needed", (unsigned long long)base.nbytes, (unsigned long long)need);
    void* d = nullptr;
    VF_CUDA(cudaMallocAsync(&d, size_t(std::max<uint64_t>(need, 1)), ctx->stream));
    try {
        copy_in(ctx, d, base.data, size_t(need), base.mem_kind);
        VF_CUDA(cudaStreamSynchronize(ctx->stream));
        scope.finish();
    } catch (...) {
        cudaFreeAsync(d, ctx->stream);
        throw;
    }
    if (nbytes) *nbytes = need;
    return d;
}

uint64_t copy_folded(vf_ctx* ctx, const Folded& f, void* dst, uint64_t dst_bytes, int dst_mem_kind, vf_tensor_type* out_type,
                     double* scales_buf, int64_t* zps_buf, int64_t params_cap) {
    CallScope scope(ctx, nullptr);
    DContent cur = borrow(f);
    cur.type.export_to(out_type, scales_buf, zps_buf, params_cap);
    const uint64_t w = copy_to(ctx, cur, dst, dst_bytes, dst_mem_kind, nullptr);
    scope.finish();
    return w;
}

// Fused jobs of a batch that wait for their shared launch (vf_fold_batch): the uploaded bases stay alive until then.
struct FusedBatch {
    std::vector<FusedJob> jobs;
    std::vector<DContent> bases;
    std::vector<int> owner;
};
constexpr uint64_t kFoldDeferred = ~uint64_t(0);

// ContentAttr::fold() + Content::copyTo() of one constant, enqueued on the context's stream (the caller owns the
// call scope and decides when the host waits). Returns the bytes written. A list that starts with a parameterised
// Quantize and that a single-pass kernel covers (fused_prepare_given) runs as ONE launch instead of one launch and
// one intermediate buffer per transformation; with `batch` such a job is only collected (kFoldDeferred is
// returned) so that the jobs of a group share their launches.
uint64_t fold_one(vf_ctx* ctx, const vf_content& base, const vf_transform* t, int n, void* dst, uint64_t dst_bytes, int dst_mem_kind,
                  vf_tensor_type* out_type, double* scales_buf, int64_t* zps_buf, int64_t params_cap, vf_stats* stats,
                  FusedBatch* batch = nullptr, int owner = 0) {
    DContent cur = upload_base(ctx, base, stats);
    // the destination doubles as the last transformation's output buffer when it is device memory that does
    // not overlap the base content
    const char* b0 = static_cast<const char*>(base.data);
    const char* d0 = static_cast<const char*>(dst);
    const bool disjoint = base.mem_kind != VF_MEM_DEVICE || dst_mem_kind != VF_MEM_DEVICE || d0 + dst_bytes <= b0 || b0 + base.nbytes <= d0;
    if (!(ctx->opt_flags & VF_OPT_DISABLE_FUSION) && n > 0 && disjoint) {
        FusedJob fj;
        Type ot;
        if (fused_prepare_given(ctx, cur, t, n, dst, dst_bytes, dst_mem_kind, fj, &ot)) {
            fj.h_base = base.data;
            ot.export_to(out_type, scales_buf, zps_buf, params_cap);
            if (stats) stats->fused = 1;
            if (batch) {
                batch->jobs.push_back(std::move(fj));
                batch->bases.push_back(std::move(cur));
                batch->owner.push_back(owner);
                return kFoldDeferred;
            }
            std::vector<FusedJob> one;
            one.push_back(std::move(fj));
            DBuf params;
            fused_upload_params(ctx, one, params);
            fused_launch(ctx, one, 0, 1);
            fused_params_enqueued(ctx);
            uint64_t w = 0;
            fused_finish(ctx, one[0], &w, stats);
            return w;
        }
    }
    const bool direct = dst && dst_mem_kind == VF_MEM_DEVICE && disjoint;
    struct Hint {
        vf_ctx* c;
        ~Hint() { c->final_dst = nullptr; }
    } hint{ctx};
    for (int i = 0; i < n; ++i) {  // ContentAttr::fold — attributes/content.cpp:392-394
        if (direct && i == n - 1) {
            ctx->final_dst = dst;
            ctx->final_bytes = dst_bytes;
        }
        DContent next = apply(ctx, cur, t[i]);
        cur = std::move(next);
    }
    ctx->final_dst = nullptr;
    cur.type.export_to(out_type, scales_buf, zps_buf, params_cap);
    const uint64_t w = copy_to(ctx, cur, dst, dst_bytes, dst_mem_kind, stats);
    if (stats) stats->bytes_out += w;
    return w;
}

}  // namespace vf

using namespace vf;

extern "C" {

int vf_fold(vf_ctx* ctx, const vf_content* base, const vf_transform* t, int n, void* dst, uint64_t dst_bytes,
            int dst_mem_kind, uint64_t* dst_written, vf_tensor_type* out_type, double* scales_buf, int64_t* zps_buf,
            int64_t params_cap, vf_stats* stats, char* err, size_t errlen) {
    return guard(err, errlen, [&] {
        if (!base || (n > 0 && !t) || n < 0) raise(VF_ERR_INVALID_ARG, "NULL argument");
        ParamCheckScope checked;
        check_positions(t, n);
        CallScope scope(ctx, stats);
        const uint64_t w = fold_one(ctx, *base, t, n, dst, dst_bytes, dst_mem_kind, out_type, scales_buf, zps_buf, params_cap, stats);
        if (dst_written) *dst_written = w;
        scope.may_defer = base->mem_kind == VF_MEM_DEVICE && (!dst || dst_mem_kind == VF_MEM_DEVICE);
        scope.finish();
    });
}

int vf_fold_batch(vf_ctx* ctx, vf_fold_job* jobs, int njobs, const vf_fold_batch_options* opts,
                  vf_fold_batch_stats* batch_stats, vf_stats* stats, char* err, size_t errlen) {
    return guard(err, errlen, [&] {
        if (njobs < 0 || (njobs > 0 && !jobs)) raise(VF_ERR_INVALID_ARG, "NULL argument");
        ParamCheckScope checked;
        const uint64_t threshold = opts && opts->threshold_bytes ? opts->threshold_bytes : 300ull * 1024 * 1024;
        const uint64_t tiny = opts && opts->tiny_threshold_bytes ? opts->tiny_threshold_bytes : 1024;
        vf_fold_batch_stats bs{};
        for (int j = 0; j < njobs; ++j) {
            vf_fold_job& jb = jobs[j];
            jb.status = VF_ERR_NOT_RUN;
            jb.dst_written = 0;
            if ((jb.n > 0 && !jb.t) || jb.n < 0) raise(VF_ERR_INVALID_ARG, "job %d: NULL transformation list", j);
        }
        for (int j = 0; j < njobs; ++j) {  // the sizes of all constants come first, as in the pass (:100-104)
            vf_fold_job& jb = jobs[j];
            try {
                check_positions(jb.t, jb.n);
                jb.max_intermediate = max_intermediate_size(Type::from(jb.base.type), jb.base.is_splat != 0, jb.t, jb.n);
            } catch (const Error& e) {
                jb.status = e.code;
                raise(e.code, "job %d: %s", j, e.what());
            }
        }
        CallScope scope(ctx, stats);
        // Jobs a single-pass kernel covers are collected while their group is walked and launched together when
        // the group closes: compatible jobs share one launch, and two lists over the same constant (codes and
        // dequantized copy) one pass.
        FusedBatch fused;
        bool all_device = true;
        for (int j = 0; j < njobs; ++j) all_device &= jobs[j].base.mem_kind == VF_MEM_DEVICE && jobs[j].dst_mem_kind == VF_MEM_DEVICE;
        auto launch_fused = [&]() {
            if (fused.jobs.empty()) return;
            fused_merge_pairs(fused.jobs);
            DBuf params;
            fused_upload_params(ctx, fused.jobs, params);
            fused_launch(ctx, fused.jobs, 0, fused.jobs.size());
            fused_params_enqueued(ctx);
            for (size_t k = 0; k < fused.jobs.size(); ++k) {
                uint64_t w = 0;
                fused_finish(ctx, fused.jobs[k], &w, stats);
                jobs[fused.owner[k]].dst_written = w;
                jobs[fused.owner[k]].status = VF_OK;
            }
            fused.jobs.clear();
            fused.bases.clear();
            fused.owner.clear();
        };
        auto run = [&](int j, int group) {
            vf_fold_job& jb = jobs[j];
            jb.group = group;
            try {
                const uint64_t w = fold_one(ctx, jb.base, jb.t, jb.n, jb.dst, jb.dst_bytes, jb.dst_mem_kind, nullptr, nullptr, nullptr, 0,
                                            stats, &fused, j);
                if (w == kFoldDeferred) return;
                jb.dst_written = w;
                jb.status = VF_OK;
            } catch (const Error& e) {
                jb.status = e.code;
                try {  // the jobs collected before this one still run, as they would have in list order
                    launch_fused();
                } catch (const Error&) {
                }
                raise(e.code, "job %d: %s", j, e.what());
            }
        };
        // What the kernels of the jobs enqueued so far have found is read here, once per group: the host waits
        // for the stream, so everything those jobs allocated is free again before the next group starts.
        bool last_wait = false;
        auto wait = [&](const char* what, int index) {
            launch_fused();
            ++bs.synchronisations;
            if (last_wait && all_device && (ctx->opt_flags & VF_OPT_ASYNC)) {
                // pipelined batches over device memory: what the last group's kernels report is returned by the
                // context's next synchronising call
                VF_CUDA(cudaGetLastError());
                ctx->deferred = true;
                return;
            }
            try {
                flags_check(ctx);
                ctx->table_used = 0;  // nothing is in flight: the job-table area starts over
            } catch (const Error& e) {
                if (index < 0) raise(e.code, "%s: %s", what, e.what());
                raise(e.code, "%s %d: %s", what, index, e.what());
            }
        };
        // the first sweep: constants within the tiny threshold (constant_folding.cpp:100-109)
        std::vector<int> big;
        for (int j = 0; j < njobs; ++j) {
            if (jobs[j].max_intermediate > tiny) {
                big.push_back(j);
                continue;
            }
            run(j, VF_GROUP_TINY);
            ++bs.tiny;
        }
        if (bs.tiny) {
            last_wait = big.empty();
            wait("the constants within the tiny threshold", -1);
        }
        // the others in order (constant_folding.cpp:113-158)
        size_t at = 0;
        while (at < big.size()) {
            const int j = big[at];
            if (jobs[j].max_intermediate > threshold) {
                run(j, VF_GROUP_ALONE);
                last_wait = at + 1 == big.size();
                wait("job", j);
                ++bs.alone;
                ++at;
                continue;
            }
            uint64_t in_flight = 0;
            const int group = bs.groups++;
            while (in_flight <= threshold && at < big.size()) {
                in_flight += jobs[big[at]].max_intermediate;
                run(big[at], group);
                ++at;
            }
            bs.max_group_bytes = std::max(bs.max_group_bytes, in_flight);
            last_wait = at == big.size();
            wait("group", group);
        }
        if (batch_stats) *batch_stats = bs;
        scope.finished = true;
        if (stats) stats->kernels_launched = int32_t(ctx->launches - scope.launches0);
    });
}

int vf_fuse(vf_ctx* ctx, vf_fuse_part* parts, int nparts, void* dst, uint64_t dst_bytes, int dst_mem_kind,
            uint64_t* dst_written, vf_stats* stats, char* err, size_t errlen) {
    return guard(err, errlen, [&] {
        if (nparts < 0 || (nparts > 0 && !parts) || (!dst && dst_bytes)) raise(VF_ERR_INVALID_ARG, "NULL argument");
        for (int p = 0; p < nparts; ++p) {
            if (!parts[p].base) continue;
            if ((parts[p].n > 0 && !parts[p].t) || parts[p].n < 0) raise(VF_ERR_INVALID_ARG, "part %d: NULL transformation list", p);
            check_positions(parts[p].t, parts[p].n);
        }
        CallScope scope(ctx, stats);
        uint64_t at = 0;  // FuseAttr::transform — attributes/fuse_transform.cpp:31-63
        for (int p = 0; p < nparts; ++p) {
            vf_fuse_part& part = parts[p];
            part.offset = at;
            part.bytes = 0;
            if (!part.base) continue;  // an absent constant (no sparsity map, no activations ...)
            DContent cur = upload_base(ctx, *part.base, stats);
            for (int i = 0; i < part.n; ++i) {
                DContent next = apply(ctx, cur, part.t[i]);
                cur = std::move(next);
            }
            // appendContentToVector (:20-29): the part's total allocation size, checked against what is left
            const uint64_t need = cur.type.alloc_bytes();
            if (at + need > dst_bytes)
                raise(VF_ERR_BUFFER_TOO_SMALL, "Overflow during fusing buffer size %llu, size after copying %llu", (unsigned long long)dst_bytes,
                      (unsigned long long)(at + need));
            const uint64_t w = copy_to(ctx, cur, static_cast<char*>(dst) + at, need, dst_mem_kind, stats);
            part.bytes = w;
            at += w;
        }
        if (dst_written) *dst_written = at;
        if (stats) stats->bytes_out += at;
        scope.finish();
    });
}

int vf_row_stats(vf_ctx* ctx, const vf_content* base, const vf_quant_spec* spec, double* scales, int64_t* zps,
                 float* rmin, float* rmax, int64_t n_units, int out_mem_kind, char* err, size_t errlen) {
    return guard(err, errlen, [&] {
        if (!base || !spec) raise(VF_ERR_INVALID_ARG, "NULL argument");
        check_spec(*spec);
        CallScope scope(ctx, nullptr);
        DContent in = upload_base(ctx, *base, nullptr);
        if (in.splat) raise(VF_ERR_SPLAT, "statistics of a splat constant are not supported");
        int64_t len = 0;
        const int64_t units = unit_count(in.type, *spec, len);
        if (units != n_units) raise(VF_ERR_SHAPE, "n_units is %lld, the tensor has %lld units", (long long)n_units, (long long)units);
        DBuf t0, t1, t2, t3;
        double* ds = static_cast<double*>(out_ptr(ctx, scales, out_mem_kind, size_t(units) * 8, t0));
        int64_t* dz = static_cast<int64_t*>(out_ptr(ctx, zps, out_mem_kind, size_t(units) * 8, t1));
        float* dmin = static_cast<float*>(out_ptr(ctx, rmin, out_mem_kind, size_t(units) * 4, t2));
        float* dmax = static_cast<float*>(out_ptr(ctx, rmax, out_mem_kind, size_t(units) * 4, t3));
        launch_unit_stats(ctx, in.d, in.storage, units, len, spec->range_mode, spec->qmin, spec->qmax, ds, dz, dmin, dmax);
        out_flush(ctx, scales, out_mem_kind, size_t(units) * 8, t0);
        out_flush(ctx, zps, out_mem_kind, size_t(units) * 8, t1);
        out_flush(ctx, rmin, out_mem_kind, size_t(units) * 4, t2);
        out_flush(ctx, rmax, out_mem_kind, size_t(units) * 4, t3);
        scope.finish();
    });
}

int vf_quantize_fold(vf_ctx* ctx, const vf_content* base, const vf_quant_spec* spec, const vf_transform* t, int n,
                     void* dst, uint64_t dst_bytes, int dst_mem_kind, uint64_t* dst_written,
                     const vf_quant_outputs* outs, vf_stats* stats, char* err, size_t errlen) {
    return guard(err, errlen, [&] {
        if (!base || !spec || (n > 0 && !t) || n < 0) raise(VF_ERR_INVALID_ARG, "NULL argument");
        check_spec(*spec);
        CallScope scope(ctx, stats);
        DContent in = upload_base(ctx, *base, stats);
        const bool allow_fused = !(ctx->opt_flags & VF_OPT_DISABLE_FUSION);
        std::vector<FusedJob> fj(1);
        if (allow_fused && fused_prepare(ctx, in, *spec, t, n, dst, dst_bytes, dst_mem_kind, outs, fj[0])) {
            fused_launch(ctx, fj, 0, 1);
            fused_finish(ctx, fj[0], dst_written, stats);
            if (stats) stats->fused = 1;
        } else {
            fj.clear();
            quantize_fold_general(ctx, in, *spec, t, n, dst, dst_bytes, dst_mem_kind, dst_written, outs, stats);
        }
        scope.finish();
    });
}

int vf_quantize_fold_batch(vf_ctx* ctx, vf_quant_job* jobs, int njobs, vf_stats* stats, char* err, size_t errlen) {
    return guard(err, errlen, [&] {
        if (njobs < 0 || (njobs > 0 && !jobs)) raise(VF_ERR_INVALID_ARG, "NULL argument");
        CallScope scope(ctx, stats);
        // Jobs that map onto a fused kernel are collected into job tables: consecutive compatible jobs run as
        // ONE launch. Device-resident jobs therefore cost one launch per pattern for the whole batch. Jobs with
        // host memory are flushed every kFlushBytes of device staging so that uploads, kernels and downloads
        // of successive sub-batches follow each other on the stream with bounded staging memory. One
        // synchronisation at the end.
        // Sub-batches alternate between two stream lanes, so the downloads of one sub-batch overlap the uploads
        // of the next (PCIe is full duplex); everything a sub-batch allocates is freed on its own lane.
        constexpr uint64_t kFlushBytes = 512ull << 20;
        const bool allow_fused = !(ctx->opt_flags & VF_OPT_DISABLE_FUSION);
        bool any_host = false;
        for (int j = 0; j < njobs; ++j) {
            const vf_quant_job& jb = jobs[j];
            any_host |= jb.base.mem_kind != VF_MEM_DEVICE || jb.dst_mem_kind != VF_MEM_DEVICE || jb.outs.mem_kind != VF_MEM_DEVICE;
        }
        struct LaneGuard {  // whatever happens, the context ends up on its main stream
            vf_ctx* c;
            ~LaneGuard() {
                c->stream = c->main_stream;
            }
        } lane_guard{ctx};
        int lane = 0;
        if (any_host) {
            VF_CUDA(cudaEventRecord(ctx->lane_ev[0], ctx->main_stream));
            VF_CUDA(cudaStreamWaitEvent(ctx->lane_stream, ctx->lane_ev[0], 0));
        }
        std::vector<DContent> bases;
        std::vector<FusedJob> fj;
        std::vector<int> owner;
        uint64_t staged = 0;
        auto flush = [&](bool switch_lane) {
            if (fj.empty()) return;
            fused_launch(ctx, fj, 0, fj.size());
            for (size_t k = 0; k < fj.size(); ++k) {
                uint64_t w = 0;
                fused_finish(ctx, fj[k], &w, stats);
                jobs[owner[k]].dst_written = w;
            }
            if (stats) stats->fused = 1;
            fj.clear();
            bases.clear();
            owner.clear();
            staged = 0;
            if (any_host && switch_lane) {
                lane ^= 1;
                ctx->stream = lane ? ctx->lane_stream : ctx->main_stream;
            }
        };
        for (int j = 0; j < njobs; ++j) {
            vf_quant_job& jb = jobs[j];
            jb.status = VF_OK;
            check_spec(jb.spec);
            DContent in = upload_base(ctx, jb.base, stats);
            FusedJob cand;
            if (allow_fused && fused_prepare(ctx, in, jb.spec, jb.t, jb.n, jb.dst, jb.dst_bytes, jb.dst_mem_kind, &jb.outs, cand)) {
                staged += in.own.bytes + cand.tc.buf.bytes + cand.td.buf.bytes;
                bases.push_back(std::move(in));
                fj.push_back(std::move(cand));
                owner.push_back(j);
                if (staged >= kFlushBytes) flush(true);
            } else {
                flush(false);  // stay on this lane: `in` was uploaded on it
                uint64_t w = 0;
                quantize_fold_general(ctx, in, jb.spec, jb.t, jb.n, jb.dst, jb.dst_bytes, jb.dst_mem_kind, &w, &jb.outs, stats);
                jb.dst_written = w;
            }
        }
        flush(false);
        ctx->stream = ctx->main_stream;
        if (any_host) {  // join the second lane before the final synchronisation
            VF_CUDA(cudaEventRecord(ctx->lane_ev[1], ctx->lane_stream));
            VF_CUDA(cudaStreamWaitEvent(ctx->main_stream, ctx->lane_ev[1], 0));
        }
        scope.may_defer = !any_host;
        scope.finish();
    });
}

int vf_nnz_per_oc(vf_ctx* ctx, const vf_content* content, int64_t* counts, int out_mem_kind, char* err,
                  size_t errlen) {
    return guard(err, errlen, [&] {
        if (!content || !counts) raise(VF_ERR_INVALID_ARG, "NULL argument");
        CallScope scope(ctx, nullptr);
        DContent in = upload_base(ctx, *content, nullptr);
        if (in.type.rank != 4) raise(VF_ERR_SHAPE, "Const::Content::sparsify: got unxpected content shape %d", in.type.rank);
        check_sparse_dtype(in.type.elem.dtype);
        const int64_t sv = sparsify_value(in.type.elem);
        const int64_t oc = in.type.shape[0], work = in.type.shape[1] * in.type.shape[2] * in.type.shape[3];
        DContent v = materialise_logical(ctx, in);
        DBuf tmp;
        int64_t* dc = static_cast<int64_t*>(out_ptr(ctx, counts, out_mem_kind, size_t(oc) * 8, tmp));
        launch_sparsity_scan(ctx, v.d, v.storage, oc, work, sv, dc, nullptr, 0);
        out_flush(ctx, counts, out_mem_kind, size_t(oc) * 8, tmp);
        scope.finish();
    });
}

// Sparsify + GetSparsityMap + counts of `n` tensors: all tensors share three launches (counts and bitmaps,
// offsets, compaction; the compaction's second read of the weights is served from L2 for anything smaller
// than the cache) and ONE read-back of the compressed sizes.
// Returns true when the call was deferred (VF_OPT_ASYNC, everything in device memory): the sizes are still on
// their way and the next synchronising call completes the jobs.
static bool sparsify_many(vf_ctx* ctx, vf_sparsify_job* jobs, int n, int out_mem_kind, vf_stats* stats, bool may_defer = false) {
    struct PerJob {
        DContent in, v;
        DBuf tcounts, tmap, tdata, counts_dev, offsets;
        int64_t oc = 0, row_bytes = 0;
    };
    std::vector<PerJob> pj(static_cast<size_t>(n));
    std::vector<SparseJob> sj(static_cast<size_t>(n));
    for (int j = 0; j < n; ++j) {
        vf_sparsify_job& jb = jobs[j];
        PerJob& p = pj[j];
        jb.status = VF_OK;
        jb.data_written = 0;
        p.in = upload_base(ctx, jb.content, stats);
        if (p.in.type.rank != 4) raise(VF_ERR_SHAPE, "Expected 4D input shape");
        const int dt = p.in.type.elem.dtype;
        check_sparse_dtype(dt);
        const int64_t oc = p.in.type.shape[0], work = p.in.type.shape[1] * p.in.type.shape[2] * p.in.type.shape[3];
        p.oc = oc;
        p.row_bytes = align_up(work, 128) / 8;
        if (jb.map) {
            if (work % 8 != 0) raise(VF_ERR_SHAPE, "GetSparsityMap needs IC*KY*KX (%lld) to be a multiple of 8", (long long)work);
            if (jb.map_bytes < uint64_t(oc * p.row_bytes)) raise(VF_ERR_BUFFER_TOO_SMALL, "sparsity map needs %lld bytes", (long long)(oc * p.row_bytes));
        }
        p.v = materialise_logical(ctx, p.in);
        SparseJob& s = sj[j];
        s.in = p.v.d;
        s.dt = dt;
        s.es = dtype_bits(dt) / 8;
        s.oc = oc;
        s.work = work;
        s.sv = sparsify_value(p.in.type.elem);
        s.counts = static_cast<int64_t*>(out_ptr(ctx, jb.counts, out_mem_kind, size_t(oc) * 8, p.tcounts));
        if (!s.counts) {
            p.counts_dev = DBuf(ctx, size_t(oc) * 8);
            s.counts = p.counts_dev.as<int64_t>();
        }
        s.map = static_cast<uint8_t*>(out_ptr(ctx, jb.map, out_mem_kind, size_t(oc * p.row_bytes), p.tmap));
        s.map_row_bytes = p.row_bytes;
        s.data = static_cast<uint8_t*>(out_ptr(ctx, jb.data, out_mem_kind, jb.data_bytes, p.tdata));
        s.capacity = jb.data_bytes;
        s.offsets = nullptr;
    }
    // one scratch allocation for the offsets of all tensors and the per-tensor totals
    size_t off_elems = 0;
    for (int j = 0; j < n; ++j)
        if (sj[j].data) off_elems += size_t(sj[j].oc + 1);
    DBuf own_scratch;
    int64_t* scratch = static_cast<int64_t*>(call_scratch(ctx, vf_ctx::kScratchSparsify, (off_elems + size_t(n)) * 8));
    if (!scratch) {
        own_scratch = DBuf(ctx, (off_elems + size_t(n)) * 8);
        scratch = own_scratch.as<int64_t>();
    }
    int64_t* const d_totals = scratch;  // [n], then the offsets
    off_elems = size_t(n);
    for (int j = 0; j < n; ++j) {
        if (!sj[j].data) continue;
        sj[j].offsets = scratch + off_elems;
        off_elems += size_t(sj[j].oc + 1);
    }
    launch_sparsify_batch(ctx, sj, d_totals);
    bool all_device = out_mem_kind == VF_MEM_DEVICE;
    for (int j = 0; j < n; ++j) all_device &= jobs[j].content.mem_kind == VF_MEM_DEVICE;
    if (may_defer && all_device && (ctx->opt_flags & VF_OPT_ASYNC) && ctx->sizes_host && ctx->sizes_used + size_t(n) <= vf_ctx::kSizesCap) {
        VF_CUDA(cudaMemcpyAsync(ctx->sizes_host + ctx->sizes_used, d_totals, size_t(n) * 8, cudaMemcpyDeviceToHost, ctx->stream));
        ctx->pending_sizes.push_back(vf_ctx::PendingSizes{jobs, n, ctx->sizes_used});
        ctx->sizes_used += size_t(n);
        if (stats)
            for (int j = 0; j < n; ++j) stats->bytes_out += jobs[j].map ? uint64_t(pj[j].oc * pj[j].row_bytes) : 0;
        return true;
    }
    std::vector<int64_t> total_host(static_cast<size_t>(n), 0);
    VF_CUDA(cudaMemcpyAsync(total_host.data(), d_totals, size_t(n) * 8, cudaMemcpyDeviceToHost, ctx->stream));
    VF_CUDA(cudaStreamSynchronize(ctx->stream));
    for (int j = 0; j < n; ++j) {
        vf_sparsify_job& jb = jobs[j];
        PerJob& p = pj[j];
        const uint64_t total = uint64_t(total_host[j]);
        if (jb.data && total > jb.data_bytes) {
            jb.status = VF_ERR_BUFFER_TOO_SMALL;
            raise(VF_ERR_BUFFER_TOO_SMALL, "compressed weights need %llu bytes, buffer holds %llu", (unsigned long long)total, (unsigned long long)jb.data_bytes);
        }
        if (jb.data) {
            out_flush(ctx, jb.data, out_mem_kind, total, p.tdata);
            if (out_mem_kind != VF_MEM_DEVICE && stats) stats->d2h_bytes += total;
        }
        out_flush(ctx, jb.counts, out_mem_kind, size_t(p.oc) * 8, p.tcounts);
        out_flush(ctx, jb.map, out_mem_kind, size_t(p.oc * p.row_bytes), p.tmap);
        jb.data_written = total;
        if (stats) stats->bytes_out += total + (jb.map ? uint64_t(p.oc * p.row_bytes) : 0);
    }
    return false;
}

int vf_sparsify(vf_ctx* ctx, const vf_content* content, void* data, uint64_t data_bytes, uint64_t* data_written,
                void* map, uint64_t map_bytes, int64_t* counts, int out_mem_kind, vf_stats* stats, char* err,
                size_t errlen) {
    return guard(err, errlen, [&] {
        if (!content) raise(VF_ERR_INVALID_ARG, "NULL argument");
        CallScope scope(ctx, stats);
        vf_sparsify_job jb{};
        jb.content = *content;
        jb.data = data;
        jb.data_bytes = data_bytes;
        jb.map = map;
        jb.map_bytes = map_bytes;
        jb.counts = counts;
        sparsify_many(ctx, &jb, 1, out_mem_kind, stats);
        if (data_written) *data_written = jb.data_written;
        scope.finish();
    });
}

int vf_sparsify_batch(vf_ctx* ctx, vf_sparsify_job* jobs, int njobs, int out_mem_kind, vf_stats* stats, char* err,
                      size_t errlen) {
    return guard(err, errlen, [&] {
        if (njobs < 0 || (njobs > 0 && !jobs)) raise(VF_ERR_INVALID_ARG, "NULL argument");
        CallScope scope(ctx, stats);
        if (njobs > 0) scope.may_defer = sparsify_many(ctx, jobs, njobs, out_mem_kind, stats, true);
        scope.finish();
    });
}

}  // extern "C"

// Translates one weights-table descriptor into kernel arguments. Host arrays are uploaded into buffers kept in
// `keep`; a count array queues an entry in `offs` (the prefix sums are launched by the caller, for all tables at
// once). `w_scales` / `w_kind`: optional replacement of the weight scales by an array of `oc` values that may
// already live in device memory (the scales a quantization job of the same tensor derived).
// `arena`: device memory for the prefix sums of all tables of the call ((oc + 1) * 8 bytes each), carved in order
static TableArgs table_prepare(vf_ctx* ctx, const vf_weights_table_desc* d, const double* w_scales, int w_kind, int32_t* d_table,
                               std::vector<DBuf>& keep, std::vector<OffsetsJob>& offs, int64_t*& arena) {
    {
        if (!d) raise(VF_ERR_INVALID_ARG, "NULL argument");
        if (d->oc <= 0) raise(VF_ERR_SHAPE, "OC must be positive");
        if (d->in_elem.dtype == VF_DT_INVALID || d->out_elem.dtype == VF_DT_INVALID)
            raise(VF_ERR_INVALID_ARG, "Can't create weights table without operation input/output types");
        const int64_t oc = d->oc;
        const Elem in = Elem::from(d->in_elem), out = Elem::from(d->out_elem);
        const bool has_w = d->weights_elem.dtype != VF_DT_INVALID;
        const Elem w = has_w ? Elem::from(d->weights_elem, w_scales == nullptr) : Elem();
        if (has_w && in.quantized() && !w.quantized()) raise(VF_ERR_UNSUPPORTED, "Unsupported In/Wt mixed precision");
        auto check_n = [&](const Elem& e, const char* what) {
            if (e.quantized() && e.scales.size() != 1 && int64_t(e.scales.size()) != oc)
                raise(VF_ERR_SHAPE, "%s scales: %zu values for %lld channels", what, e.scales.size(), (long long)oc);
        };
        check_n(in, "input");
        check_n(out, "output");
        if (!w_scales) check_n(w, "weights");

        auto upload = [&](const void* src, size_t bytes, int kind) {  // -> device pointer, buffer kept alive
            keep.emplace_back(ctx, bytes);
            copy_in(ctx, keep.back().p, src, bytes, kind);
            return keep.back().p;
        };
        TableArgs a{};
        a.oc = oc;
        a.d_table = d_table;
        a.in_quantized = in.quantized();
        a.out_quantized = out.quantized();
        a.weights_quantized = has_w && w.quantized();
        a.in_is_float = !in.quantized() && dtype_is_float(in.dtype);
        a.const_scale = d->has_const_scale ? d->const_scale : 1.0;
        if (a.weights_quantized && w_scales) {
            a.d_wscale = w_kind == VF_MEM_DEVICE ? w_scales : static_cast<const double*>(upload(w_scales, size_t(oc) * 8, w_kind));
            a.n_wscale = oc;
        } else {
            const std::vector<double> ws = a.weights_quantized ? w.scales.vec() : std::vector<double>{1.0};
            a.d_wscale = static_cast<const double*>(upload(ws.data(), ws.size() * 8, VF_MEM_HOST));
            a.n_wscale = int64_t(ws.size());
        }
        a.in_scale = in.quantized() ? in.scales[0] : 1.0;
        a.out_scale = out.quantized() ? out.scales[0] : 1.0;
        if (in.quantized() && in.scales.size() > 1) a.d_in_scale = static_cast<const double*>(upload(in.scales.data(), in.scales.size() * 8, VF_MEM_HOST));
        if (out.quantized() && out.scales.size() > 1) a.d_out_scale = static_cast<const double*>(upload(out.scales.data(), out.scales.size() * 8, VF_MEM_HOST));
        a.wbase = d->weights_ptr_base;
        a.wstep = d->weights_ptr_step;
        a.sbase = d->sparsity_ptr_base;
        a.sstep = d->sparsity_ptr_step;
        if (d->weights_ptrs) a.d_wptrs = static_cast<const int32_t*>(upload(d->weights_ptrs, size_t(oc) * 4, VF_MEM_HOST));
        if (d->sparsity_ptrs) a.d_sptrs = static_cast<const int32_t*>(upload(d->sparsity_ptrs, size_t(oc) * 4, VF_MEM_HOST));
        if (d->nnz_counts) {
            const int64_t* dc = d->nnz_counts;
            if (d->nnz_mem_kind != VF_MEM_DEVICE) dc = static_cast<const int64_t*>(upload(d->nnz_counts, size_t(oc) * 8, d->nnz_mem_kind));
            int64_t* doff = arena;
            arena += oc + 1;
            const int eb = std::max(1, dtype_bits(has_w ? w.dtype : VF_DT_U8) / 8);
            offs.push_back(OffsetsJob{dc, oc, eb, doff});
            a.d_nnz_offsets = doff;
        }
        if (d->has_bias) {
            if (!d->bias) raise(VF_ERR_INVALID_ARG, "has_bias without a bias pointer");
            const size_t nb = size_t(d->bias_is_splat ? 1 : oc) * 4;
            a.d_bias = d->bias_mem_kind == VF_MEM_DEVICE ? d->bias : static_cast<const float*>(upload(d->bias, nb, d->bias_mem_kind));
            a.bias_is_splat = d->bias_is_splat;
        }
        return a;
    }
}

extern "C" {

int vf_weights_table(vf_ctx* ctx, const vf_weights_table_desc* d, int32_t* table, int out_mem_kind, char* err,
                     size_t errlen) {
    return guard(err, errlen, [&] {
        if (!d || !table) raise(VF_ERR_INVALID_ARG, "NULL argument");
        CallScope scope(ctx, nullptr);
        std::vector<DBuf> keep;
        std::vector<OffsetsJob> offs;
        keep.reserve(16);
        DBuf tmp;
        int32_t* dt = static_cast<int32_t*>(out_ptr(ctx, table, out_mem_kind, size_t(d->oc > 0 ? d->oc : 0) * 16, tmp));
        DBuf sums(ctx, d->nnz_counts && d->oc > 0 ? size_t(d->oc + 1) * 8 : 0);
        int64_t* arena = sums.as<int64_t>();
        const TableArgs a = table_prepare(ctx, d, nullptr, VF_MEM_HOST, dt, keep, offs, arena);
        launch_offsets_batch(ctx, offs);
        launch_weights_table(ctx, a, dt);
        out_flush(ctx, table, out_mem_kind, size_t(d->oc) * 16, tmp);
        scope.finish();
    });
}

int vf_weights_table_batch(vf_ctx* ctx, vf_weights_table_job* jobs, int njobs, int out_mem_kind, char* err, size_t errlen) {
    return guard(err, errlen, [&] {
        if (njobs < 0 || (njobs > 0 && !jobs)) raise(VF_ERR_INVALID_ARG, "NULL argument");
        CallScope scope(ctx, nullptr);
        std::vector<DBuf> keep;
        std::vector<OffsetsJob> offs;
        std::vector<TableArgs> tabs;
        std::vector<DBuf> stage(static_cast<size_t>(njobs));
        keep.reserve(size_t(njobs) * 8 + 8);  // pointers into `keep` entries stay valid: no reallocation below
        tabs.reserve(size_t(njobs));
        size_t sum_entries = 0;  // one allocation for the prefix sums of all sparse tables
        for (int j = 0; j < njobs; ++j)
            if (jobs[j].desc.nnz_counts && jobs[j].desc.oc > 0) sum_entries += size_t(jobs[j].desc.oc) + 1;
        DBuf own_sums;
        int64_t* arena = sum_entries ? static_cast<int64_t*>(call_scratch(ctx, vf_ctx::kScratchTables, sum_entries * 8)) : nullptr;
        if (sum_entries && !arena) {
            own_sums = DBuf(ctx, sum_entries * 8);
            arena = own_sums.as<int64_t>();
        }
        for (int j = 0; j < njobs; ++j) {
            vf_weights_table_job& jb = jobs[j];
            jb.status = VF_OK;
            if (!jb.table) raise(VF_ERR_INVALID_ARG, "job %d: table is NULL", j);
            int32_t* dt = static_cast<int32_t*>(out_ptr(ctx, jb.table, out_mem_kind, size_t(jb.desc.oc > 0 ? jb.desc.oc : 0) * 16, stage[j]));
            try {
                tabs.push_back(table_prepare(ctx, &jb.desc, jb.weights_scales, jb.scales_mem_kind, dt, keep, offs, arena));
            } catch (const Error& e) {
                jb.status = e.code;
                throw;
            }
        }
        launch_weights_table_batch(ctx, tabs, &offs);
        for (int j = 0; j < njobs; ++j) out_flush(ctx, jobs[j].table, out_mem_kind, size_t(jobs[j].desc.oc) * 16, stage[j]);
        scope.may_defer = out_mem_kind == VF_MEM_DEVICE;
        scope.finish();
    });
}

int vf_synth_fill(vf_ctx* ctx, const vf_synth_spec* spec, void* dst, uint64_t count, char* err, size_t errlen) {
    return guard(err, errlen, [&] {
        if (!spec || !dst) raise(VF_ERR_INVALID_ARG, "NULL argument");
        CallScope scope(ctx, nullptr);
        launch_synth(ctx, *spec, dst, count);
        scope.finish();
    });
}

}  // extern "C"
