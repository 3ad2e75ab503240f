// Pattern matcher in front of the fused weight-quantization kernels: recognises the transformation lists
// that upstream passes build for weights (Quantize [+ Reorder<NHWC>] [+ PadWithZero] | [+ BitPack]) and maps
// them onto the job tables of kernels_rowquant.cu. Anything else is declined and takes the general path.
#include <algorithm>

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

void fused_launch(vf_ctx* ctx, std::vector<FusedJob>& jobs, size_t begin, size_t end) {
    // jobs are independent, so they are regrouped: all jobs with the same kernel and launch-uniform parameters
    // share one launch, wherever they sit in the batch
    std::vector<char> done(end - begin, 0);
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
    if (dst_written) *dst_written = job.out_bytes;
    if (stats) stats->bytes_out += job.out_bytes + job.dq_bytes;
}

}  // namespace vf
