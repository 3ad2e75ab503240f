// Context: one device, one stream, stream-ordered scratch from the device memory pool, pinned bounce
// buffers for pageable host memory, and the device-side error flags.
#include <algorithm>

#include "kernels.h"

namespace vf {

int sm_count_hint() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

void* dalloc(vf_ctx* ctx, size_t bytes) {
    void* p = nullptr;
    VF_CUDA(cudaMallocFromPoolAsync(&p, bytes ? bytes : 1, ctx->pool, ctx->stream));
    return p;
}

void dfree(vf_ctx* ctx, void* p) {
    if (p) cudaFreeAsync(p, ctx->stream);
}

// Pageable host memory goes through two pinned bounce buffers so the copy engine and the host memcpy
// overlap; pinned and device memory are handed to the copy engine directly.
void copy_in(vf_ctx* ctx, void* dst_dev, const void* src, size_t bytes, int src_kind) {
    if (!bytes) return;
    if (src_kind == VF_MEM_DEVICE) {
        VF_CUDA(cudaMemcpyAsync(dst_dev, src, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
        return;
    }
    if (src_kind == VF_MEM_HOST_PINNED) {
        VF_CUDA(cudaMemcpyAsync(dst_dev, src, bytes, cudaMemcpyHostToDevice, ctx->stream));
        return;
    }
    size_t off = 0;
    int k = 0;
    while (off < bytes) {
        const size_t n = std::min<size_t>(ctx->staging_bytes, bytes - off);
        VF_CUDA(cudaEventSynchronize(ctx->staging_ev[k]));  // previous use of this bounce buffer is done
        std::memcpy(ctx->staging[k], static_cast<const char*>(src) + off, n);
        VF_CUDA(cudaMemcpyAsync(static_cast<char*>(dst_dev) + off, ctx->staging[k], n, cudaMemcpyHostToDevice, ctx->stream));
        VF_CUDA(cudaEventRecord(ctx->staging_ev[k], ctx->stream));
        off += n;
        k ^= 1;
    }
}

void copy_out(vf_ctx* ctx, void* dst, int dst_kind, const void* src_dev, size_t bytes) {
    if (!bytes) return;
    if (dst_kind == VF_MEM_DEVICE) {
        VF_CUDA(cudaMemcpyAsync(dst, src_dev, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
        return;
    }
    if (dst_kind == VF_MEM_HOST_PINNED) {
        VF_CUDA(cudaMemcpyAsync(dst, src_dev, bytes, cudaMemcpyDeviceToHost, ctx->stream));
        return;
    }
    size_t off = 0;
    int k = 0;
    size_t pending_off[2] = {0, 0}, pending_n[2] = {0, 0};
    while (off < bytes || pending_n[0] || pending_n[1]) {
        if (pending_n[k]) {  // drain the older transfer of this bounce buffer
            VF_CUDA(cudaEventSynchronize(ctx->staging_ev[k]));
            std::memcpy(static_cast<char*>(dst) + pending_off[k], ctx->staging[k], pending_n[k]);
            pending_n[k] = 0;
        }
        if (off < bytes) {
            const size_t n = std::min<size_t>(ctx->staging_bytes, bytes - off);
            VF_CUDA(cudaMemcpyAsync(ctx->staging[k], static_cast<const char*>(src_dev) + off, n, cudaMemcpyDeviceToHost, ctx->stream));
            VF_CUDA(cudaEventRecord(ctx->staging_ev[k], ctx->stream));
            pending_off[k] = off;
            pending_n[k] = n;
            off += n;
        }
        k ^= 1;
    }
}

const void* upload_table(vf_ctx* ctx, const void* src, size_t bytes, DBuf& fallback) {
    const size_t need = (bytes + 255) & ~size_t(255);
    if (ctx->deferred && ctx->table_host && need <= vf_ctx::kTableBytes && ctx->table_used + need > vf_ctx::kTableBytes) {
        // deferred calls still read their tables: wait for them before the area is reused from the start
        VF_CUDA(cudaStreamSynchronize(ctx->stream));
        ctx->table_used = 0;
    }
    if (ctx->table_host && ctx->table_used + need <= vf_ctx::kTableBytes) {
        if (ctx->table_used == 0 && ctx->table_unchecked) {
            // the area starts over although nobody waited for the kernels that read it (a call that ended in an
            // error): they have to finish before their tables are overwritten
            VF_CUDA(cudaStreamSynchronize(ctx->main_stream));
            VF_CUDA(cudaStreamSynchronize(ctx->lane_stream));
            ctx->table_unchecked = false;
        }
        char* h = ctx->table_host + ctx->table_used;
        char* d = ctx->table_dev + ctx->table_used;
        ctx->table_used += need;
        std::memcpy(h, src, bytes);
        VF_CUDA(cudaMemcpyAsync(d, h, bytes, cudaMemcpyHostToDevice, ctx->table_stream));
        VF_CUDA(cudaEventRecord(ctx->table_ev, ctx->table_stream));
        VF_CUDA(cudaStreamWaitEvent(ctx->stream, ctx->table_ev, 0));
        ctx->table_unchecked = true;
        return d;
    }
    fallback = DBuf(ctx, bytes);
    copy_in(ctx, fallback.p, src, bytes, VF_MEM_HOST);
    return fallback.p;
}

void* call_scratch(vf_ctx* ctx, int slot, size_t bytes) {
    if (bytes <= ctx->call_scratch_cap[slot] && ctx->call_scratch[slot]) return ctx->call_scratch[slot];
    if (ctx->stream != ctx->main_stream) return nullptr;  // (a lane of a batch: the caller takes a buffer of its own)
    if (ctx->call_scratch[slot]) cudaFreeAsync(ctx->call_scratch[slot], ctx->main_stream);  // after the kernels that read it
    ctx->call_scratch[slot] = nullptr;
    ctx->call_scratch_cap[slot] = 0;
    const size_t cap = std::max<size_t>(bytes + bytes / 2, size_t(64) << 10);
    VF_CUDA(cudaMallocFromPoolAsync(&ctx->call_scratch[slot], cap, ctx->pool, ctx->main_stream));
    ctx->call_scratch_cap[slot] = cap;
    return ctx->call_scratch[slot];
}

// The flags are zero unless a call found something or ended early: only then is the next call's clearing real.
void flags_clear(vf_ctx* ctx) {
    if (ctx->deferred) return;  // unchecked work is in flight: its flags and job tables stay as they are
    ctx->table_used = 0;  // a new call: the previous call's job tables are no longer in use
    if (ctx->flags_dirty) VF_CUDA(cudaMemsetAsync(ctx->d_flags, 0, sizeof(int) * kNumFlags, ctx->stream));
    ctx->flags_dirty = true;  // until flags_check has seen them all zero
}

void flags_check(vf_ctx* ctx) {
    VF_CUDA(cudaMemcpyAsync(ctx->h_flags, ctx->d_flags, sizeof(int) * kNumFlags, cudaMemcpyDeviceToHost, ctx->stream));
    VF_CUDA(cudaStreamSynchronize(ctx->stream));
    VF_CUDA(cudaGetLastError());
    ctx->deferred = false;  // everything enqueued so far has finished and is being checked now
    ctx->table_unchecked = false;
    // deferred vf_sparsify_batch calls: their sizes have arrived
    const vf_sparsify_job* too_small = nullptr;
    for (const vf_ctx::PendingSizes& ps : ctx->pending_sizes) {
        for (int j = 0; j < ps.n; ++j) {
            vf_sparsify_job& jb = ps.jobs[j];
            jb.data_written = uint64_t(ctx->sizes_host[ps.first + size_t(j)]);
            if (jb.data && jb.data_written > jb.data_bytes) {
                jb.status = VF_ERR_BUFFER_TOO_SMALL;
                if (!too_small) too_small = &jb;
            }
        }
    }
    ctx->pending_sizes.clear();
    ctx->sizes_used = 0;
    const int* f = ctx->h_flags;
    bool any = false;
    for (int i = 0; i < kNumFlags; ++i) any |= f[i] != 0;
    ctx->flags_dirty = any;
    if (too_small)  // (the compaction kernel's overflow flag is the same finding)
        raise(VF_ERR_BUFFER_TOO_SMALL, "compressed weights need %llu bytes, buffer holds %llu", (unsigned long long)too_small->data_written,
              (unsigned long long)too_small->data_bytes);
    if (f[0]) raise(VF_ERR_CHECKED_CAST, "Can not safely cast a value to the destination element type");
    if (f[1]) raise(VF_ERR_QUANT_RANGE, "calcScaleAndZeroPoint failed: range without zero or scale too small");
    if (f[2]) raise(VF_ERR_SHAPE, "numActualElements smaller than the number of non-sparse elements");
    if (f[3]) raise(VF_ERR_RANGE, "weights table: scale needs a post-shift or rescaled bias is out of range");
    if (f[4]) raise(VF_ERR_ALIGNMENT, "weights table: pointer must be a multiple of 16");
    if (f[5]) raise(VF_ERR_NAN, "Quantize met a NaN: its conversion to an integer is undefined in the reference");
    if (f[6]) raise(VF_ERR_NOT_NORMAL, "Taking inverse of a non-normal (e.g. zero/nan/...) float");
}

}  // namespace vf

extern "C" {

int vf_ctx_create(int device, const vf_options* opts, void* external_stream, vf_ctx** out, char* err, size_t errlen) {
    return vf::guard(err, errlen, [&] {
        if (!out) vf::raise(VF_ERR_INVALID_ARG, "out is NULL");
        *out = nullptr;
        int ndev = 0;
        if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) {
            cudaGetLastError();
            vf::raise(VF_ERR_NO_DEVICE, "no CUDA device available: this library has no CPU path");
        }
        if (device < 0 || device >= ndev) vf::raise(VF_ERR_NO_DEVICE, "device %d outside 0..%d", device, ndev - 1);
        vf::DeviceGuard g(device);
        vf_ctx* c = new vf_ctx();
        try {
            c->device = device;
            VF_CUDA(cudaDeviceGetAttribute(&c->sm_count, cudaDevAttrMultiProcessorCount, device));
            if (external_stream) {
                c->stream = static_cast<cudaStream_t>(external_stream);
            } else {
                VF_CUDA(cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking));
                c->own_stream = true;
            }
            c->main_stream = c->stream;
            VF_CUDA(cudaStreamCreateWithFlags(&c->lane_stream, cudaStreamNonBlocking));
            for (int k = 0; k < 2; ++k) VF_CUDA(cudaEventCreateWithFlags(&c->lane_ev[k], cudaEventDisableTiming));
            c->opt_flags = opts ? opts->flags : 0;
            c->staging_bytes = (opts && opts->staging_bytes) ? opts->staging_bytes : (64ull << 20);
            for (int k = 0; k < 2; ++k) {
                VF_CUDA(cudaMallocHost(&c->staging[k], c->staging_bytes));
                VF_CUDA(cudaEventCreateWithFlags(&c->staging_ev[k], cudaEventDisableTiming));
            }
            VF_CUDA(cudaMalloc(&c->d_flags, sizeof(int) * vf::kNumFlags));
            VF_CUDA(cudaMallocHost(&c->h_flags, sizeof(int) * vf::kNumFlags));
            VF_CUDA(cudaMemset(c->d_flags, 0, sizeof(int) * vf::kNumFlags));
            VF_CUDA(cudaMallocHost(reinterpret_cast<void**>(&c->table_host), vf_ctx::kTableBytes));
            VF_CUDA(cudaMallocHost(reinterpret_cast<void**>(&c->sizes_host), vf_ctx::kSizesCap * sizeof(int64_t)));
            VF_CUDA(cudaMalloc(reinterpret_cast<void**>(&c->table_dev), vf_ctx::kTableBytes));
            VF_CUDA(cudaStreamCreateWithFlags(&c->table_stream, cudaStreamNonBlocking));
            VF_CUDA(cudaEventCreateWithFlags(&c->table_ev, cudaEventDisableTiming));
            // scratch pool of this context: freed scratch stays cached in it instead of going back to the driver on
            // every synchronisation; the device's default pool (and whoever else uses it) is left as it is
            cudaMemPoolProps props{};
            props.allocType = cudaMemAllocationTypePinned;
            props.handleTypes = cudaMemHandleTypeNone;
            props.location.type = cudaMemLocationTypeDevice;
            props.location.id = device;
            VF_CUDA(cudaMemPoolCreate(&c->pool, &props));
            uint64_t thr = UINT64_MAX;
            VF_CUDA(cudaMemPoolSetAttribute(c->pool, cudaMemPoolAttrReleaseThreshold, &thr));
            VF_CUDA(cudaEventCreateWithFlags(&c->param_ready_ev, cudaEventDisableTiming));
            for (int k = 0; k < 2; ++k) VF_CUDA(cudaEventCreateWithFlags(&c->param_used_ev[k], cudaEventDisableTiming));
            if (c->opt_flags & VF_OPT_TIMING)
                for (int k = 0; k < 2; ++k) VF_CUDA(cudaEventCreate(&c->time_ev[k]));
            vf::noalloc_prepare(c);
        } catch (...) {
            vf_ctx_destroy(c);
            throw;
        }
        *out = c;
    });
}

void vf_ctx_destroy(vf_ctx* c) {
    if (!c) return;
    vf::DeviceGuard g(c->device);
    if (c->stream) cudaStreamSynchronize(c->stream);
    for (int k = 0; k < 2; ++k) {
        if (c->staging[k]) cudaFreeHost(c->staging[k]);
        if (c->staging_ev[k]) cudaEventDestroy(c->staging_ev[k]);
    }
    for (void* sp : c->call_scratch)
        if (sp) cudaFreeAsync(sp, c->main_stream);
    if (c->main_stream) cudaStreamSynchronize(c->main_stream);
    if (c->table_stream) {
        cudaStreamSynchronize(c->table_stream);
        cudaStreamDestroy(c->table_stream);
    }
    if (c->table_ev) cudaEventDestroy(c->table_ev);
    if (c->table_host) cudaFreeHost(c->table_host);
    if (c->sizes_host) cudaFreeHost(c->sizes_host);
    if (c->table_dev) cudaFree(c->table_dev);
    if (c->d_flags) cudaFree(c->d_flags);
    if (c->h_flags) cudaFreeHost(c->h_flags);
    if (c->lane_stream) cudaStreamSynchronize(c->lane_stream);
    for (int k = 0; k < 2; ++k)
        if (c->lane_ev[k]) cudaEventDestroy(c->lane_ev[k]);
    if (c->lane_stream) cudaStreamDestroy(c->lane_stream);
    for (int k = 0; k < 2; ++k) {
        if (c->time_ev[k]) cudaEventDestroy(c->time_ev[k]);
        if (c->param_used_ev[k]) cudaEventDestroy(c->param_used_ev[k]);
        if (c->param_dev[k]) cudaFree(c->param_dev[k]);
    }
    if (c->param_ready_ev) cudaEventDestroy(c->param_ready_ev);
    if (c->pool) cudaMemPoolDestroy(c->pool);
    if (c->own_stream && c->main_stream) cudaStreamDestroy(c->main_stream);
    delete c;
}

int vf_ctx_synchronize(vf_ctx* c, char* err, size_t errlen) {
    return vf::guard(err, errlen, [&] {
        if (!c) vf::raise(VF_ERR_INVALID_ARG, "ctx is NULL");
        std::lock_guard<std::mutex> lock(c->mu);
        vf::DeviceGuard g(c->device);
        if (c->deferred) vf::flags_check(c);  // reports what the deferred calls' kernels found
        else VF_CUDA(cudaStreamSynchronize(c->stream));
    });
}

void* vf_ctx_stream(vf_ctx* c) {
    return c ? c->stream : nullptr;
}
int vf_ctx_device(vf_ctx* c) {
    return c ? c->device : -1;
}
uint64_t vf_ctx_launch_count(vf_ctx* c) {
    return c ? c->launches : 0;
}

}  // extern "C"
