// Shared host-side declarations of libvfold: status/exception plumbing, the host type model that mirrors
// vpux::NDTypeInterface for the Const path, and the context.
#pragma once

#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <algorithm>
#include <cstring>
#include <mutex>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/vfold.h"

namespace vf {

// ------------------------------------------------------------------------------------------------------
// errors — reference VPUX_THROW sites become vf::Error(status, message); converted at the C boundary
// ------------------------------------------------------------------------------------------------------
struct Error : std::runtime_error {
    int code;
    Error(int c, const std::string& m): std::runtime_error(m), code(c) {
    }
};

[[noreturn]] void raise(int code, const char* fmt, ...);

#define VF_CUDA(expr)                                                                                      \
    do {                                                                                                   \
        cudaError_t e_ = (expr);                                                                           \
        if (e_ != cudaSuccess) {                                                                           \
            ::vf::raise(e_ == cudaErrorMemoryAllocation ? VF_ERR_OOM : VF_ERR_CUDA, "%s failed: %s", #expr, \
                        cudaGetErrorString(e_));                                                           \
        }                                                                                                  \
    } while (0)

template <class F>
int guard(char* err, size_t errlen, F&& body) {
    try {
        body();
        if (err && errlen) err[0] = 0;
        return VF_OK;
    } catch (const Error& e) {
        if (err && errlen) snprintf(err, errlen, "%s", e.what());
        return e.code;
    } catch (const std::exception& e) {
        if (err && errlen) snprintf(err, errlen, "%s", e.what());
        return VF_ERR_INVALID_ARG;
    }
}

// ------------------------------------------------------------------------------------------------------
// dtypes
// ------------------------------------------------------------------------------------------------------
int dtype_bits(int dt);
bool dtype_is_float(int dt);
bool dtype_is_int(int dt);
bool dtype_is_signed(int dt);
void dtype_int_limits(int dt, double& lo, double& hi);

inline int64_t align_up(int64_t v, int64_t a) {
    return (v + a - 1) / a * a;
}

// ------------------------------------------------------------------------------------------------------
// host type model
// ------------------------------------------------------------------------------------------------------
// Scales / zero points of a quantized element type. A type read from the caller's descriptor borrows the caller's
// arrays (they stay valid for the duration of the call) instead of copying them: per-channel types of large
// weight tensors carry hundreds of thousands of entries and a fold looks at its types many times. The first
// modification (padding or slicing the quantized axis) makes a private copy.
template <class T>
class Params {
    const T* p_ = nullptr;
    size_t n_ = 0;
    std::vector<T> own_;
    void sync() {
        p_ = own_.data();
        n_ = own_.size();
    }
    void materialise() {
        if (own_.empty() && n_) {
            std::vector<T> tmp(p_, p_ + n_);
            own_.swap(tmp);
            sync();
        }
    }

public:
    Params() = default;
    Params(const Params& o) {
        *this = o;
    }
    Params& operator=(const Params& o) {
        if (this == &o) return *this;
        own_ = o.own_;
        n_ = o.n_;
        p_ = o.own_.empty() ? o.p_ : own_.data();
        return *this;
    }
    Params& operator=(const std::vector<T>& v) {
        own_ = v;
        sync();
        return *this;
    }
    void borrow(const T* p, size_t n) {
        own_.clear();
        p_ = p;
        n_ = n;
    }
    size_t size() const { return n_; }
    bool empty() const { return n_ == 0; }
    const T* data() const { return p_; }
    const T& operator[](size_t i) const { return p_[i]; }
    const T& front() const { return p_[0]; }
    const T& back() const { return p_[n_ - 1]; }
    const T* begin() const { return p_; }
    const T* end() const { return p_ + n_; }
    void assign(size_t n, const T& v) {
        std::vector<T> tmp(n, v);
        own_.swap(tmp);
        sync();
    }
    template <class It>
    void assign(It a, It b) {
        std::vector<T> tmp(a, b);  // the range may lie inside this object
        own_.swap(tmp);
        sync();
    }
    template <class It>
    void append(It a, It b) {
        std::vector<T> tmp(a, b);
        materialise();
        own_.insert(own_.end(), tmp.begin(), tmp.end());
        sync();
    }
    void append(size_t n, const T& v) {
        materialise();
        own_.insert(own_.end(), n, v);
        sync();
    }
    void own() { materialise(); }  // for a type that outlives the call it was read in
    std::vector<T> vec() const { return std::vector<T>(begin(), end()); }
    bool operator==(const Params& o) const { return n_ == o.n_ && std::equal(begin(), end(), o.begin()); }
    bool operator!=(const Params& o) const { return !(*this == o); }
};

struct Elem {
    int kind = VF_ELEM_PLAIN;
    int dtype = VF_DT_INVALID;
    int expressed = VF_DT_INVALID;
    int axis = -1;
    int64_t qmin = 0, qmax = 0;
    Params<double> scales;
    Params<int64_t> zps;
    bool quantized() const {
        return kind != VF_ELEM_PLAIN;
    }
    static Elem plain(int dt) {
        Elem e;
        e.dtype = dt;
        return e;
    }
    // check_scales = false: the caller does not use the type's scales (they are supplied elsewhere)
    static Elem from(const vf_elem_type& e, bool check_scales = true);
    bool single_zp(int64_t& zp) const;  // extractSingleZeroPoint
};

struct Type {
    Elem elem;
    int rank = 0;
    uint32_t order = 0;
    int64_t shape[VF_MAX_RANK] = {};

    static Type from(const vf_tensor_type& t);
    int64_t numel() const;
    uint64_t alloc_bytes() const;            // getTotalAllocSize of the compact tensor
    void perm(int* p) const;                 // p[memDim] = logical dim
    void mem_shape(int64_t* ms) const;       // shape in memory order
    void export_to(vf_tensor_type* out, double* sb, int64_t* zb, int64_t cap) const;
};

// While one of these is alive on a thread, Elem::from checks an array of scales only the first time it meets it:
// a fold parses the same attribute several times (sizes, types, the fold itself), and the arrays of per-channel
// types are long. Entry points create one for the duration of the call, in which the arrays cannot change.
struct ParamCheckScope {
    ParamCheckScope();
    ~ParamCheckScope();
    ParamCheckScope(const ParamCheckScope&) = delete;
    ParamCheckScope& operator=(const ParamCheckScope&) = delete;
};

uint32_t identity_order(int rank);
void order_to_perm(uint32_t order, int rank, int* perm);

// inferOutputType / inferOutputSplat of one transformation (pure host)
Type infer_one(const Type& in, bool in_splat, const vf_transform& t, bool& out_splat);
uint64_t max_intermediate_size(Type ty, bool splat, const vf_transform* t, int n);
void check_positions(const vf_transform* t, int n);
int64_t swizzle_size_alignment(int arch);  // bytes a swizzled buffer's size is aligned to
Type compress_type(const Type& in, const int64_t* counts, int64_t n);

// Whether the tail of fakeQuantize (/(L-1) * (qHigh-qLow) + qLow, truncate) maps every index n to n + qmin for
// this storage range, evaluated with the reference's fp32 operations (fold_fused.cu).
bool tail_is_identity(int64_t qmin, int64_t qmax);

// calcScaleAndZeroPoint on the host (used for validation of tiny inputs and by tests of the planner)
bool calc_scale_zp_host(double qmin, double qmax, double rmin, double rmax, double& scale, int64_t& zp);

}  // namespace vf

// ------------------------------------------------------------------------------------------------------
// context
// ------------------------------------------------------------------------------------------------------
struct vf_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;  // the stream all helpers enqueue on (swapped between lanes inside a batch)
    bool own_stream = false;
    cudaStream_t main_stream = nullptr;  // the context's own / the caller's stream
    cudaStream_t lane_stream = nullptr;  // second lane for batches with host memory: its transfers overlap lane 0's
    cudaEvent_t lane_ev[2] = {nullptr, nullptr};
    uint64_t staging_bytes = 0;
    void* staging[2] = {nullptr, nullptr};  // pinned bounce buffers for pageable host memory
    cudaEvent_t staging_ev[2] = {nullptr, nullptr};
    // job tables of the batched launches: a pinned staging area and its device twin, filled front to back within
    // one call (calls are synchronous, so the area is free again when the next call starts)
    static constexpr size_t kTableBytes = 1u << 20;
    char* table_host = nullptr;
    char* table_dev = nullptr;
    size_t table_used = 0;
    // The tables travel on a stream of their own, so that an upload does not queue behind the kernels already on
    // `stream`; the kernel that reads a table waits for `table_ev`. `table_unchecked`: uploads have been issued
    // since flags_check last waited for the stream (an area restarted in that state is fenced first).
    cudaStream_t table_stream = nullptr;
    cudaEvent_t table_ev = nullptr;
    bool table_unchecked = false;
    // Scratch that the batched sparsify and weights-table calls need on every call (offsets and totals; prefix
    // sums): kept between calls and grown when a call needs more, instead of two pool requests and two releases per
    // call. Every user is enqueued on the context's main stream, so a call's kernels have finished with a slot
    // before the next call's kernels write it.
    enum { kScratchSparsify = 0, kScratchTables = 1, kScratchSlots = 2 };
    void* call_scratch[kScratchSlots] = {nullptr, nullptr};
    size_t call_scratch_cap[kScratchSlots] = {0, 0};
    int* d_flags = nullptr;  // device error flags (see VF_FLAG_* in device_utils.cuh)
    int* h_flags = nullptr;  // pinned mirror
    bool flags_dirty = false;  // the device flags may be non-zero (a call found something or ended early)
    bool deferred = false;     // VF_OPT_ASYNC: calls have returned whose kernels are still unchecked
    // VF_OPT_ASYNC, vf_sparsify_batch over device memory: the compressed sizes travel to this pinned area behind the
    // kernels; the next synchronising call writes them into the callers' jobs and checks the capacities
    struct PendingSizes {
        vf_sparsify_job* jobs;
        int n;
        size_t first;  // index of the batch's first entry in sizes_host
    };
    static constexpr size_t kSizesCap = 8192;
    int64_t* sizes_host = nullptr;
    size_t sizes_used = 0;
    std::vector<PendingSizes> pending_sizes;
    uint64_t launches = 0;
    int32_t opt_flags = 0;
    int sm_count = 1;            // multiprocessors of the device: persistent grids are sized in multiples of it
    cudaMemPool_t pool = nullptr;  // scratch comes from a pool the context owns (the device's default pool stays untouched)
    void* noalloc_scratch = nullptr;  // device address of vf_sparsify_noalloc's built-in array on this device
    cudaEvent_t time_ev[2] = {nullptr, nullptr};  // VF_OPT_TIMING
    // device copies of supplied quantization parameters: two persistent buffers used in turn, filled on the second
    // stream so that the upload for one call overlaps the kernels of the call before it
    void* param_dev[2] = {nullptr, nullptr};
    size_t param_cap[2] = {0, 0};
    cudaEvent_t param_ready_ev = nullptr;             // the upload has landed
    cudaEvent_t param_used_ev[2] = {nullptr, nullptr};  // the kernels that read buffer k have been enqueued before this
    bool param_used[2] = {false, false};
    int param_turn = 0;
    bool conv_smem_set = false;  // dynamic shared memory limit of the conv kernel raised on this device
    // vf_fold, last transformation, device destination: the output buffer may be the destination itself, which
    // saves the final copy (see alloc_like)
    void* final_dst = nullptr;
    uint64_t final_bytes = 0;
    std::mutex mu;  // serialises calls on this context
};

namespace vf {

constexpr int kNumFlags = 8;

// Multiprocessors of the current device (queried once per device): grid-stride launches are capped at a few
// waves of it.
int sm_count_hint();

struct DeviceGuard {
    int prev = -1;
    explicit DeviceGuard(int dev) {
        cudaGetDevice(&prev);
        if (prev != dev) cudaSetDevice(dev);
        else prev = -1;
    }
    ~DeviceGuard() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

// Stream-ordered scratch allocation from the device's memory pool.
void* dalloc(vf_ctx* ctx, size_t bytes);
void dfree(vf_ctx* ctx, void* p);

struct DBuf {  // RAII scratch buffer
    vf_ctx* ctx = nullptr;
    void* p = nullptr;
    size_t bytes = 0;
    DBuf() = default;
    DBuf(vf_ctx* c, size_t n): ctx(c), p(n ? dalloc(c, n) : nullptr), bytes(n) {
    }
    DBuf(const DBuf&) = delete;
    DBuf& operator=(const DBuf&) = delete;
    DBuf(DBuf&& o) noexcept: ctx(o.ctx), p(o.p), bytes(o.bytes) {
        o.p = nullptr;
    }
    DBuf& operator=(DBuf&& o) noexcept {
        if (this != &o) {
            reset();
            ctx = o.ctx;
            p = o.p;
            bytes = o.bytes;
            o.p = nullptr;
        }
        return *this;
    }
    ~DBuf() {
        reset();
    }
    void reset() {
        if (p && ctx) dfree(ctx, p);
        p = nullptr;
    }
    static DBuf borrow(void* ptr, size_t n) {  // caller-owned memory: never freed (ctx stays NULL)
        DBuf b;
        b.p = ptr;
        b.bytes = n;
        return b;
    }
    template <class T>
    T* as() const {
        return static_cast<T*>(p);
    }
};

// host <-> device transfers that honour the memory kind of the host side
void copy_in(vf_ctx* ctx, void* dst_dev, const void* src, size_t bytes, int src_kind);
void copy_out(vf_ctx* ctx, void* dst, int dst_kind, const void* src_dev, size_t bytes);
// Copies a job table to the device and returns where it is. Small tables go through the context's table area
// (one asynchronous copy, nothing allocated); `fallback` owns the memory of a table that does not fit.
const void* upload_table(vf_ctx* ctx, const void* src, size_t bytes, DBuf& fallback);
// At least `bytes` of device scratch from slot `slot` of the context (see vf_ctx::call_scratch); NULL when the
// context is not on its main stream (the caller then takes a buffer of its own).
void* call_scratch(vf_ctx* ctx, int slot, size_t bytes);
void flags_clear(vf_ctx* ctx);
// synchronises the stream and raises if a kernel recorded an error
void flags_check(vf_ctx* ctx);

// Device-resident Const::Content
struct DContent {
    Type type;
    int storage = VF_DT_INVALID;
    bool splat = false;
    const void* d = nullptr;  // device pointer (borrowed or owned by `own`)
    uint64_t nbytes = 0;
    DBuf own;
    int64_t count() const {
        return splat ? 1 : type.numel();
    }
};

}  // namespace vf
