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
};

// Fills `job` when (spec, t[0..n)) is a pattern the fused kernels cover; false otherwise (nothing launched).
bool fused_prepare(vf_ctx* ctx, const DContent& base, const vf_quant_spec& spec, const vf_transform* t, int n,
                   void* dst, uint64_t dst_bytes, int dst_kind, const vf_quant_outputs* outs, FusedJob& job);
// Launches jobs[begin, end): consecutive compatible jobs share one kernel launch.
void fused_launch(vf_ctx* ctx, std::vector<FusedJob>& jobs, size_t begin, size_t end);
// Copies host-bound outputs out (asynchronously on the context's stream) and reports sizes.
void fused_finish(vf_ctx* ctx, FusedJob& job, uint64_t* dst_written, vf_stats* stats);

}  // namespace vf
