// vf_sparsify_noalloc: weight sparsification for callers that are not allowed to allocate device memory.
//
// Who needs this: the compiler can be embedded in a long-running service (an inference server that compiles
// models on demand) whose own allocator has claimed the device's memory up front and hands the fold a fixed
// arena for inputs and outputs. In such a process a cudaMalloc from a library either fails (nothing is left
// outside the arena) or, worse, succeeds by synchronising the whole device and stalling the server's streams.
// The regular vf_sparsify draws its per-call scratch (per-channel counts and output offsets) from the CUDA
// memory pool; this variant keeps that scratch in a fixed array that is part of the loaded module instead.
//
// Cost and limits: every GPU that loads the library holds the array (1 MiB + 256 B) until the process exits.
// At most VF_NOALLOC_MAX_OC output channels per call. All calls on a device share the one array: it still
// holds the previous call's counts and offsets when the next call starts (both are fully rewritten before they
// are read, nothing relies on zeros), and two calls that overlap on the GPU — different contexts or streams on
// the same device — would overwrite each other's offsets. Callers must serialise their calls per device.
//
// Set-up happens in vf_ctx_create, not in the entry point: with the context's device current it looks up the
// array's device address (cudaGetSymbolAddress; in host code the array's name is only a handle for the runtime, not
// an address a kernel could use) and makes the runtime load the three kernels the entry point launches. Loading a
// module lets the driver allocate device memory for its code and for this array, which is exactly what must not
// happen later inside the embedder's allocation-free phase — so create the context before the embedder's allocator
// claims the GPU, and before any stream capture. The address is kept in the context: a context created after a
// cudaDeviceReset looks it up again.
#include "kernels.h"

namespace {

constexpr int64_t kMaxOC = VF_NOALLOC_MAX_OC;

// counts[kMaxOC] followed by offsets[kMaxOC + 1], both int64
static __device__ __align__(256) unsigned char g_noalloc_scratch[(2 * kMaxOC + 1) * 8 + 248];

}  // namespace

namespace vf {

void noalloc_prepare(vf_ctx* ctx) {  // the context's device is current
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || !p) raise(VF_ERR_CUDA, "cudaGetSymbolAddress(scratch) failed: %s", cudaGetErrorString(e));
    ctx->noalloc_scratch = p;
    preload_sparsity_kernels();
}

}  // namespace vf

extern "C" int vf_sparsify_noalloc(vf_ctx* ctx, const void* weights, int32_t dtype, int64_t oc, int64_t work,
                                   int64_t sparse_value, void* data, uint64_t data_bytes, uint64_t* data_written,
                                   void* map, uint64_t map_bytes, int64_t* counts, char* err, size_t errlen) {
    using namespace vf;
    return guard(err, errlen, [&] {
        if (!ctx || !weights) raise(VF_ERR_INVALID_ARG, "NULL argument");
        if (dtype != VF_DT_I8 && dtype != VF_DT_U8 && dtype != VF_DT_F16 && dtype != VF_DT_BF16 && dtype != VF_DT_F32)
            raise(VF_ERR_UNSUPPORTED, "Unexpected weights data type: %d", dtype);
        if (oc < 1 || work < 1) raise(VF_ERR_SHAPE, "oc and work must be positive");
        if (oc > kMaxOC)
            raise(VF_ERR_CAPACITY, "%lld output channels exceed the built-in scratch of vf_sparsify_noalloc (%lld); use vf_sparsify",
                  (long long)oc, (long long)kMaxOC);
        const int es = dtype_bits(dtype) / 8;
        const int64_t row_bytes = align_up(work, 128) / 8;
        if (map) {
            if (work % 8 != 0) raise(VF_ERR_SHAPE, "GetSparsityMap needs IC*KY*KX (%lld) to be a multiple of 8", (long long)work);
            if (map_bytes < uint64_t(oc * row_bytes)) raise(VF_ERR_BUFFER_TOO_SMALL, "sparsity map needs %lld bytes", (long long)(oc * row_bytes));
        }
        if ((dtype == VF_DT_I8 && (sparse_value < -128 || sparse_value > 127)) || (dtype == VF_DT_U8 && (sparse_value < 0 || sparse_value > 255)))
            raise(VF_ERR_CHECKED_CAST, "sparsify value %lld outside the element type", (long long)sparse_value);

        std::unique_lock<std::mutex> lock(ctx->mu);
        DeviceGuard dev(ctx->device);
        unsigned char* scratch = static_cast<unsigned char*>(ctx->noalloc_scratch);
        if (!scratch) raise(VF_ERR_INVALID_ARG, "context without the built-in scratch");
        int64_t* d_counts = counts ? counts : reinterpret_cast<int64_t*>(scratch);
        int64_t* d_offsets = reinterpret_cast<int64_t*>(scratch + size_t(kMaxOC) * 8);

        flags_clear(ctx);
        launch_sparsity_scan(ctx, weights, dtype, oc, work, sparse_value, d_counts, static_cast<uint8_t*>(map), row_bytes);
        uint64_t total_host = 0;
        if (data) {
            launch_sparse_offsets(ctx, d_counts, oc, es, d_offsets);
            launch_sparse_compact(ctx, weights, dtype, oc, work, sparse_value, d_offsets, static_cast<uint8_t*>(data), data_bytes);
            int64_t total = 0;
            VF_CUDA(cudaMemcpyAsync(&total, d_offsets + oc, 8, cudaMemcpyDeviceToHost, ctx->stream));
            VF_CUDA(cudaStreamSynchronize(ctx->stream));
            total_host = uint64_t(total);
        }
        if (data_written) *data_written = total_host;  // also when the buffer is too small: the size that is needed
        if (data && total_host > data_bytes) {
            raise(VF_ERR_BUFFER_TOO_SMALL, "compressed weights need %llu bytes, buffer holds %llu", (unsigned long long)total_host, (unsigned long long)data_bytes);
        }
        flags_check(ctx);  // synchronises
    });
}
