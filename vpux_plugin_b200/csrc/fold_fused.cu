// Pattern matcher in front of the fused weight-quantization kernels: recognises the transformation lists
// that upstream passes build for weights (Quantize [+ Reorder<NHWC>] [+ PadWithZero] | [+ BitPack]) and maps
// them onto the job tables of kernels_rowquant.cu. Anything else is declined and takes the general path.
#include <algorithm>
#include <cstring>
#include <unordered_map>

#include "fused.h"

namespace vf {

namespace {

// The fast quantizer returns n = round((x - inLow) / range * (L-1)) and emits code n + qmin. That equals the
// reference only if the tail of fakeQuantize is the identity on integers:
//   trunc(fl(fl(fl(n / (L-1)) * (qHigh - qLow)) + qLow)) == n + qmin   for all n in [0, L-1]
// (utils/quantization.cpp:1001). True for the usual ranges (0..255, -128..127, -127..127, 0..15, -8..7) but not
// for every range (e.g. -120..120), so it is evaluated here with the same fp32 operations.
bool tail_is_identity_uncached(int64_t qmin, int64_t qmax);

}  // namespace

bool tail_is_identity(int64_t qmin, int64_t qmax) {  // a batch asks the same question for every job
    static thread_local int64_t last_min = 1, last_max = 0;
    static thread_local bool last = false;
    if (qmin != last_min || qmax != last_max) {
        last = tail_is_identity_uncached(qmin, qmax);
        last_min = qmin;
        last_max = qmax;
    }
    return last;
}

namespace {

bool tail_is_identity_uncached(int64_t qmin, int64_t qmax) {
    const volatile float lm1 = float(qmax - qmin + 1) - 1.0f;
    const volatile float qlow = float(qmin), qhigh = float(qmax);
    const volatile float qrange = qhigh - qlow;
    for (int64_t n = 0; n <= qmax - qmin; ++n) {
        volatile float t = float(n);
        t = t / lm1;
        t = t * qrange;
        t = t + qlow;
        if (int64_t(t) != n + qmin) return false;
    }
    return true;
}

}  // namespace

void* OutStage::bind(vf_ctx* ctx, void* u, int k, size_t n) {
    user = u;
    kind = k;
    bytes = n;
    if (!u) return nullptr;
    if (k == VF_MEM_DEVICE) return u;
    buf = DBuf(ctx, n);
    return buf.p;
}

void OutStage::flush(vf_ctx* ctx, vf_stats* stats) {
    if (user && kind != VF_MEM_DEVICE) {
        copy_out(ctx, user, kind, buf.p, bytes);
        if (stats) stats->d2h_bytes += bytes;
    }
}

bool fused_prepare(vf_ctx* ctx, const DContent& base, const vf_quant_spec& spec, const vf_transform* t, int n,
                   void* dst, uint64_t dst_bytes, int dst_kind, const vf_quant_outputs* outs, FusedJob& job) {
    const Type& bt = base.type;
    if (base.splat || bt.elem.quantized()) return false;
    if (base.storage != VF_DT_F32 && base.storage != VF_DT_F16 && base.storage != VF_DT_BF16) return false;
    if (bt.order != identity_order(bt.rank)) return false;
    if (spec.qmax - spec.qmin > 255 || !tail_is_identity(spec.qmin, spec.qmax)) return false;
    if (bt.numel() == 0) return false;

    RowQuantArgs& a = job.a;
    a = RowQuantArgs{};
    a.in = base.d;
    a.in_dt = base.storage;
    a.range_mode = spec.range_mode;
    a.qmin = spec.qmin;
    a.qmax = spec.qmax;
    a.out_signed = spec.storage_dtype == VF_DT_I8;
    a.group = spec.group_size;

    int64_t units;
    uint64_t out_bytes;
    int i = 0;
    if (spec.group_size > 0) {
        a.cols = bt.shape[bt.rank - 1];
        a.rows = bt.numel() / a.cols;
        a.rows_pad = a.rows;
        if (a.cols % spec.group_size != 0) return false;
        units = bt.numel() / spec.group_size;
        if (i < n && t[i].kind == VF_T_BIT_PACK) {
            if (t[i].width != 4 || bt.numel() % 2 != 0) return false;
            a.pack4 = 1;
            ++i;
        }
        out_bytes = a.pack4 ? uint64_t(bt.numel() / 2) : uint64_t(bt.numel());
    } else {
        a.rows = bt.shape[0];
        a.cols = bt.numel() / a.rows;
        a.rows_pad = a.rows;
        units = a.rows;
        int64_t row_out = a.cols;
        if (i < n && t[i].kind == VF_T_REORDER) {
            if (bt.rank != 4 || t[i].order != VF_ORDER_NHWC) return false;
            a.ic = bt.shape[1];
            a.khw = bt.shape[2] * bt.shape[3];
            a.ic_pad = a.ic;
            ++i;
            if (i < n && t[i].kind == VF_T_PAD_WITH_ZERO) {
                // only trailing padding of the channel dims; the codes are a plain integer type here, so the
                // fill value is zero (Content::fillWithZero, utils/content.cpp:233-236)
                const vf_transform& p = t[i];
                if (p.rank != 4 || p.a[0] || p.a[1] || p.a[2] || p.a[3] || p.b[2] || p.b[3] || p.b[0] < 0 || p.b[1] < 0) return false;
                a.rows_pad = a.rows + p.b[0];
                a.ic_pad = a.ic + p.b[1];
                ++i;
            }
            if (a.khw == 1 && a.ic_pad == a.ic) a.khw = 0;  // 1x1 kernels: the reorder moves nothing
            row_out = a.khw > 0 ? a.khw * a.ic_pad : a.cols;
        }
        out_bytes = uint64_t(a.rows_pad) * uint64_t(row_out);
    }
    if (i != n) return false;  // something the store stage does not cover

    if (outs && outs->dequant) {
        const int ddt = outs->dequant_dtype;
        if (ddt != VF_DT_F16 && ddt != VF_DT_F32 && ddt != VF_DT_BF16) return false;
        if (a.khw > 0 || a.rows_pad != a.rows || a.pack4) return false;
        a.dequant_dt = ddt;
    }
    if (outs && outs->zps_u4_packed && a.group == 0) return false;  // packed zero points: per-group kernel only

    if (!dst) raise(VF_ERR_INVALID_ARG, "dst is NULL");
    if (dst_bytes < out_bytes) raise(VF_ERR_BUFFER_TOO_SMALL, "Byte sizes of the target buffer '%llu' is smaller then storage buffer '%llu'", (unsigned long long)dst_bytes, (unsigned long long)out_bytes);
    a.codes = job.tc.bind(ctx, dst, dst_kind, out_bytes);
    job.out_bytes = out_bytes;
    job.dq_bytes = 0;
    if (outs) {
        const int k = outs->mem_kind;
        a.scales = static_cast<double*>(job.ts.bind(ctx, outs->scales, k, size_t(units) * 8));
        a.zps = static_cast<int64_t*>(job.tz.bind(ctx, outs->zps, k, size_t(units) * 8));
        a.scales_f16 = static_cast<uint16_t*>(job.t16.bind(ctx, outs->scales_f16, k, size_t(units) * 2));
        a.zps_u4 = static_cast<uint8_t*>(job.t4.bind(ctx, outs->zps_u4_packed, k, size_t((units + 1) / 2)));
        if (outs->dequant) {
            job.dq_bytes = uint64_t(bt.numel()) * uint64_t(dtype_bits(outs->dequant_dtype) / 8);
            if (outs->dequant_bytes < job.dq_bytes) raise(VF_ERR_BUFFER_TOO_SMALL, "dequantized copy needs %llu bytes", (unsigned long long)job.dq_bytes);
            a.dequant = job.td.bind(ctx, outs->dequant, k, job.dq_bytes);
        }
    }
    job.kind = rowquant_kind(a);
    return job.kind != 0;
}

namespace {

bool same_params(const vf_elem_type& a, const vf_elem_type& b) {
    if (a.kind != b.kind || a.dtype != b.dtype || a.axis != b.axis || a.qmin != b.qmin || a.qmax != b.qmax || a.nparams != b.nparams ||
        a.expressed != b.expressed)
        return false;
    if (a.scales != b.scales && std::memcmp(a.scales, b.scales, size_t(a.nparams) * sizeof(double)) != 0) return false;
    if (a.zps != b.zps && std::memcmp(a.zps, b.zps, size_t(a.nparams) * sizeof(int64_t)) != 0) return false;
    return true;
}

}  // namespace

bool fused_prepare_given(vf_ctx* ctx, const DContent& base, const vf_transform* t, int n, void* dst, uint64_t dst_bytes,
                         int dst_kind, FusedJob& job, Type* out_type) {
    if (n < 1 || base.splat || base.type.elem.quantized()) return false;
    if (base.storage != VF_DT_F32 && base.storage != VF_DT_F16 && base.storage != VF_DT_BF16) return false;
    if (base.storage != base.type.elem.dtype) return false;
    if (base.type.order != identity_order(base.type.rank) || base.type.numel() == 0) return false;
    int i = 0;
    Type ty = base.type;
    bool splat = false;
    if (t[i].kind == VF_T_RESHAPE && n >= 2) {  // a leading Reshape only renames the units
        if (t[i].rank != 2) return false;
        ty = infer_one(ty, splat, t[i], splat);
        ++i;
    }
    if (t[i].kind != VF_T_QUANTIZE) return false;
    const vf_elem_type& q = t[i].elem;
    if (q.kind != VF_ELEM_QUANT_PER_AXIS || q.axis != 0 || (q.dtype != VF_DT_I8 && q.dtype != VF_DT_U8)) return false;
    if (!q.scales || !q.zps || q.nparams != ty.shape[0] || q.qmax <= q.qmin || q.qmax - q.qmin > 255) return false;
    double lo, hi;
    dtype_int_limits(q.dtype, lo, hi);
    if (double(q.qmin) < lo || double(q.qmax) > hi || !tail_is_identity(q.qmin, q.qmax)) return false;
    const int qi = i;
    ty = infer_one(ty, splat, t[i], splat);
    ++i;

    RowQuantArgs& a = job.a;
    a = RowQuantArgs{};
    a.in = base.d;
    a.in_dt = base.storage;
    a.range_mode = VF_RANGE_MINMAX;
    a.qmin = q.qmin;
    a.qmax = q.qmax;
    a.out_signed = q.dtype == VF_DT_I8;
    a.rows = ty.shape[0];
    a.cols = ty.numel() / a.rows;
    a.rows_pad = a.rows;
    uint64_t out_bytes = uint64_t(ty.numel());
    bool to_dequant = false;
    if (i < n && t[i].kind == VF_T_BIT_PACK) {
        // (BitPack reads its input through getValues<uint8_t>(): negative codes fail the checked cast, bit_pack.cpp:146-151)
        if (t[i].width != 4 || q.qmin < 0 || ty.rank != 2 || (a.cols != 32 && a.cols != 64 && a.cols != 128) || ty.numel() % 2 != 0) return false;
        a.group = a.cols;  // every row is one group: the per-group kernel with one group per unit
        a.pack4 = 1;
        out_bytes = uint64_t(ty.numel() / 2);
        ty = infer_one(ty, splat, t[i], splat);
        ++i;
    } else if (i + 1 < n && t[i].kind == VF_T_CAST_ELEM_TYPE && t[i + 1].kind == VF_T_DEQUANTIZE) {
        if (!same_params(q, t[i].elem)) return false;
        const int ddt = q.expressed;
        if (ddt != VF_DT_F16 && ddt != VF_DT_F32 && ddt != VF_DT_BF16) return false;
        ty = infer_one(ty, splat, t[i], splat);
        ty = infer_one(ty, splat, t[i + 1], splat);
        a.dequant_dt = ddt;
        to_dequant = true;
        i += 2;
    } else if (i < n && t[i].kind == VF_T_REORDER) {
        if (ty.rank != 4 || t[i].order != VF_ORDER_NHWC) return false;
        a.ic = ty.shape[1];
        a.khw = ty.shape[2] * ty.shape[3];
        a.ic_pad = a.ic;
        ty = infer_one(ty, splat, t[i], splat);
        ++i;
        if (i < n && t[i].kind == VF_T_PAD_WITH_ZERO) {
            const vf_transform& p = t[i];
            if (p.rank != 4 || p.a[0] || p.a[1] || p.a[2] || p.a[3] || p.b[2] || p.b[3] || p.b[0] < 0 || p.b[1] < 0) return false;
            a.rows_pad = a.rows + p.b[0];
            a.ic_pad = a.ic + p.b[1];
            ty = infer_one(ty, splat, t[i], splat);
            ++i;
        }
        if (a.khw == 1 && a.ic_pad == a.ic) a.khw = 0;
        out_bytes = uint64_t(a.rows_pad) * uint64_t(a.khw > 0 ? a.khw * a.ic_pad : a.cols);
    }
    if (i != n) return false;
    (void)qi;

    if (!dst) raise(VF_ERR_INVALID_ARG, "dst is NULL");
    job.dst_is_dequant = to_dequant;
    job.out_bytes = to_dequant ? 0 : out_bytes;
    job.dq_bytes = to_dequant ? uint64_t(ty.numel()) * uint64_t(dtype_bits(a.dequant_dt) / 8) : 0;
    const uint64_t need = to_dequant ? job.dq_bytes : out_bytes;
    // probe which kernel would take the job before anything is allocated (pointers only matter for alignment)
    a.codes = to_dequant ? nullptr : (dst_kind == VF_MEM_DEVICE ? dst : reinterpret_cast<void*>(uintptr_t(256)));
    a.dequant = to_dequant ? (dst_kind == VF_MEM_DEVICE ? dst : reinterpret_cast<void*>(uintptr_t(256))) : nullptr;
    a.given_scales = reinterpret_cast<const double*>(uintptr_t(256));
    if (rowquant_kind(a) == 0) return false;
    if (dst_bytes < need) raise(VF_ERR_BUFFER_TOO_SMALL, "Byte sizes of the target buffer '%llu' is smaller then storage buffer '%llu'", (unsigned long long)dst_bytes, (unsigned long long)need);
    if (to_dequant) a.dequant = job.td.bind(ctx, dst, dst_kind, need);
    else a.codes = job.tc.bind(ctx, dst, dst_kind, need);
    // (a.given_scales keeps its non-NULL placeholder until fused_upload_params has made the device copies)
    job.h_scales = q.scales;
    job.h_zps = q.zps;
    job.n_params = q.nparams;
    job.kind = rowquant_kind(a);
    if (out_type) *out_type = ty;
    return job.kind != 0;
}

void fused_merge_pairs(std::vector<FusedJob>& jobs) {
    // candidates that write the dequantized copy only, by the base content they read
    std::unordered_multimap<const void*, size_t> by_base;
    for (size_t k = 0; k < jobs.size(); ++k) {
        const FusedJob& d = jobs[k];
        if (!d.merged && d.kind == 2 && d.dst_is_dequant && !d.a.codes) by_base.emplace(d.h_base, k);
    }
    if (by_base.empty()) return;
    for (size_t i = 0; i < jobs.size(); ++i) {
        FusedJob& c = jobs[i];  // candidate that writes codes only
        if (c.merged || c.kind != 2 || !c.a.given_scales || c.dst_is_dequant || c.a.dequant) continue;
        const auto range = by_base.equal_range(c.h_base);
        for (auto it = range.first; it != range.second; ++it) {
            FusedJob& d = jobs[it->second];
            if (it->second == i || d.merged) continue;
            if (d.a.rows != c.a.rows || d.a.cols != c.a.cols || d.a.qmin != c.a.qmin || d.a.qmax != c.a.qmax || d.a.in_dt != c.a.in_dt ||
                d.n_params != c.n_params)
                continue;
            if (d.h_scales != c.h_scales && std::memcmp(d.h_scales, c.h_scales, size_t(c.n_params) * 8) != 0) continue;
            if (d.h_zps != c.h_zps && std::memcmp(d.h_zps, c.h_zps, size_t(c.n_params) * 8) != 0) continue;
            c.a.dequant = d.a.dequant;
            c.a.dequant_dt = d.a.dequant_dt;
            d.merged = true;
            break;
        }
    }
}

void fused_upload_params(vf_ctx* ctx, std::vector<FusedJob>& jobs, DBuf& holder) {
    size_t total = 0;
    for (const FusedJob& j : jobs)
        if (!j.merged && j.h_scales) total += size_t(j.n_params) * 16;
    if (!total) return;
    const bool staged = total <= ctx->staging_bytes;
    char* dev = nullptr;
    char* host = nullptr;
    int turn = 0;
    if (staged) {
        turn = ctx->param_turn ^= 1;
        if (ctx->param_cap[turn] < total) {  // grow (rare): nothing may still read the old buffer
            VF_CUDA(cudaStreamSynchronize(ctx->stream));
            VF_CUDA(cudaStreamSynchronize(ctx->lane_stream));
            if (ctx->param_dev[turn]) VF_CUDA(cudaFree(ctx->param_dev[turn]));
            ctx->param_dev[turn] = nullptr;
            ctx->param_cap[turn] = 0;
            const size_t cap = std::max<size_t>(total + total / 4, size_t(1) << 20);
            VF_CUDA(cudaMalloc(&ctx->param_dev[turn], cap));
            ctx->param_cap[turn] = cap;
            ctx->param_used[turn] = false;
        }
        dev = static_cast<char*>(ctx->param_dev[turn]);
        VF_CUDA(cudaEventSynchronize(ctx->staging_ev[0]));  // the staging buffer's previous transfer is done
        host = static_cast<char*>(ctx->staging[0]);
    } else {
        holder = DBuf(ctx, total);
        dev = holder.as<char>();
    }
    size_t at = 0;
    for (FusedJob& j : jobs) {
        if (j.merged || !j.h_scales) continue;
        const size_t nb = size_t(j.n_params) * 8;
        if (staged) {
            std::memcpy(host + at, j.h_scales, nb);
            std::memcpy(host + at + nb, j.h_zps, nb);
        } else {
            copy_in(ctx, dev + at, j.h_scales, nb, VF_MEM_HOST);
            copy_in(ctx, dev + at + nb, j.h_zps, nb, VF_MEM_HOST);
        }
        j.a.given_scales = reinterpret_cast<const double*>(dev + at);
        j.a.given_zps = reinterpret_cast<const int64_t*>(dev + at + nb);
        at += 2 * nb;
    }
    if (staged) {
        cudaStream_t up = ctx->lane_stream;
        // the kernels that read this buffer two uploads ago must be done before it is overwritten
        if (ctx->param_used[turn]) VF_CUDA(cudaStreamWaitEvent(up, ctx->param_used_ev[turn], 0));
        VF_CUDA(cudaMemcpyAsync(dev, host, total, cudaMemcpyHostToDevice, up));
        VF_CUDA(cudaEventRecord(ctx->staging_ev[0], up));
        VF_CUDA(cudaEventRecord(ctx->param_ready_ev, up));
        VF_CUDA(cudaStreamWaitEvent(ctx->stream, ctx->param_ready_ev, 0));
        ctx->param_used[turn] = true;  // fused_params_enqueued records the event
    }
}

void fused_params_enqueued(vf_ctx* ctx) {
    const int turn = ctx->param_turn;
    if (ctx->param_used[turn]) VF_CUDA(cudaEventRecord(ctx->param_used_ev[turn], ctx->stream));
}

void fused_launch(vf_ctx* ctx, std::vector<FusedJob>& jobs, size_t begin, size_t end) {
    // jobs are independent, so they are regrouped: all jobs with the same kernel and launch-uniform parameters
    // share one launch, wherever they sit in the batch
    std::vector<char> done(end - begin, 0);
    for (size_t i = begin; i < end; ++i) done[i - begin] = jobs[i].merged ? 1 : 0;
    std::vector<RowQuantArgs> table;
    for (size_t i = begin; i < end; ++i) {
        if (done[i - begin]) continue;
        table.clear();
        for (size_t k = i; k < end; ++k) {
            if (!done[k - begin] && jobs[k].kind == jobs[i].kind && rowquant_compatible(jobs[i].a, jobs[k].a)) {
                table.push_back(jobs[k].a);
                done[k - begin] = 1;
            }
        }
        launch_rowquant_batch(ctx, jobs[i].kind, table);
    }
}

void fused_finish(vf_ctx* ctx, FusedJob& job, uint64_t* dst_written, vf_stats* stats) {
    job.tc.flush(ctx, stats);
    job.ts.flush(ctx, stats);
    job.tz.flush(ctx, stats);
    job.t16.flush(ctx, stats);
    job.t4.flush(ctx, stats);
    job.td.flush(ctx, stats);
    if (dst_written) *dst_written = job.dst_is_dequant ? job.dq_bytes : job.out_bytes;
    if (stats) stats->bytes_out += job.out_bytes + job.dq_bytes;
}

}  // namespace vf
