// Host-side interface between the fold entry points and the fused weight-quantization kernels.
#pragma once

#include <vector>

#include "kernels.h"

namespace vf {

// Device staging for an output that the caller wants in host memory: the kernel writes `buf`, flush() copies
// it out. For device-memory outputs the kernel writes the caller's buffer directly.
struct OutStage {
    DBuf buf;
    void* user = nullptr;
    int kind = VF_MEM_DEVICE;
    size_t bytes = 0;
    void* bind(vf_ctx* ctx, void* u, int k, size_t n);
    void flush(vf_ctx* ctx, vf_stats* stats);
};

struct FusedJob {
    RowQuantArgs a{};
    int kind = 0;  // rowquant_kind
    OutStage tc, ts, tz, t16, t4, td;
    uint64_t out_bytes = 0, dq_bytes = 0;
    // parameterised Quantize (fused_prepare_given): where the attribute's scales / zero points are on the host (also
    // to recognise two lists over the same constant), and which output the destination is. Their device copies
    // are made for all jobs of a launch at once (fused_upload_params).
    const double* h_scales = nullptr;
    const int64_t* h_zps = nullptr;
    int64_t n_params = 0;
    const void* h_base = nullptr;  // where the caller's base content lives (host or device)
    bool dst_is_dequant = false;  // the list ends in Dequantize: the destination receives the dequantized copy
    bool merged = false;          // this job's output is written by another job's launch entry (fused_merge_pairs)
};

// Fills `job` when (spec, t[0..n)) is a pattern the fused kernels cover; false otherwise (nothing launched).
bool fused_prepare(vf_ctx* ctx, const DContent& base, const vf_quant_spec& spec, const vf_transform* t, int n,
                   void* dst, uint64_t dst_bytes, int dst_kind, const vf_quant_outputs* outs, FusedJob& job);
// The same for the list shapes a compiler pass builds, where the Quantize attribute carries its parameters
// (attributes/quantize.cpp:108-212):
//   [Quantize<per-axis(0)>]                                         -> codes
//   [Quantize<per-axis(0)>, Reorder<NHWC> [, PadWithZero]]          -> codes in OYXI order, channels padded
//   [[Reshape<[units, G]>,] Quantize<per-axis(0)>, BitPack<4>]      -> packed codes (G = 32 / 64 / 128)
//   [Quantize<per-axis(0)>, CastElemType<the same type>, Dequantize]-> the dequantized copy in the expressed type
// `out_type` receives the type of the folded content. False: not covered, nothing was launched or allocated.
bool fused_prepare_given(vf_ctx* ctx, const DContent& base, const vf_transform* t, int n, void* dst, uint64_t dst_bytes,
                         int dst_kind, FusedJob& job, Type* out_type);
// Two jobs of a batch that quantize the same constant with the same parameters, one for the codes and one for
// the dequantized copy, become one entry of the launch: the input is read once for both outputs.
void fused_merge_pairs(std::vector<FusedJob>& jobs);
// Copies the supplied scales / zero points of all (unmerged) jobs to the device in ONE transfer and points the jobs
// at their slices. The transfer goes through the context's pinned staging buffer into one of two persistent
// device buffers on the context's second stream, so in pipelined use it overlaps the previous call's kernels; the
// launching stream waits for it. Call fused_params_enqueued once the launches that read the parameters are enqueued.
// (`holder` owns the memory of the rare transfer that does not fit the staging buffer.)
void fused_upload_params(vf_ctx* ctx, std::vector<FusedJob>& jobs, DBuf& holder);
void fused_params_enqueued(vf_ctx* ctx);
// Launches jobs[begin, end): consecutive compatible jobs share one kernel launch.
void fused_launch(vf_ctx* ctx, std::vector<FusedJob>& jobs, size_t begin, size_t end);
// Copies host-bound outputs out (asynchronously on the context's stream) and reports sizes.
void fused_finish(vf_ctx* ctx, FusedJob& job, uint64_t* dst_written, vf_stats* stats);

}  // namespace vf
