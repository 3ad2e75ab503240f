// Folding in the background with a cache of folded contents — the GPU counterpart of
// Const::BackgroundConstantFolding (const/utils/constant_folding_in_background.cpp:17-241) and
// Const::ConstantFoldingCache (const/utils/constant_folding_cache.cpp:15-245).
//
// The compiler thread enqueues requests; worker threads, each with its own context (one stream each, so their
// kernels overlap on the device), fold them and keep the folded Const::Content in device memory. The cache is
// keyed by a canonical serialisation of (base content identity, transformation list). The identity of a base
// is either the caller's id or a 128-bit hash of its bytes computed by a kernel at memory speed, which is what
// lets equal constants in different buffers share one entry.
#include <algorithm>
#include <atomic>
#include <condition_variable>
#include <deque>
#include <memory>
#include <string>
#include <thread>
#include <unordered_map>

#include "fold_internal.h"

namespace vf {

namespace {

// ---- content hash ---------------------------------------------------------------------------------------
__host__ __device__ inline uint64_t mix64(uint64_t z) {
    z ^= z >> 33;
    z *= 0xFF51AFD7ED558CCDull;
    z ^= z >> 33;
    z *= 0xC4CEB9FE1A85EC53ull;
    z ^= z >> 33;
    return z;
}

// The buffer is read as 16-byte vectors (a, b) of two 8-byte words, missing bytes as zero. Vector i has the key
// k = (i + 1) * K; two 64 x 64 -> 128 bit products of differently keyed copies of (a, b) are folded (low ^ high
// half) and summed into the two halves of the hash. Addition commutes, so the result does not depend on how the
// vectors are spread over threads; the keys make it depend on where a vector stands. A 16-byte aligned buffer is
// read one vector per load; any other buffer, and the last partial vector, are assembled from 8-byte or single-byte
// loads.
__device__ __forceinline__ uint64_t word_from_bytes(const uint8_t* __restrict__ p, uint64_t nbytes, uint64_t w) {
    uint64_t v = 0;
    for (int b = 0; b < 8; ++b)
        if (w * 8 + b < nbytes) v |= uint64_t(p[w * 8 + b]) << (8 * b);
    return v;
}
__host__ __device__ inline uint64_t swap_halves(uint64_t v) {
    return (v << 32) | (v >> 32);
}

constexpr int kHashLoads = 8;
__global__ void __launch_bounds__(256, 4) k_hash128(const uint8_t* __restrict__ p, uint64_t nbytes, unsigned long long* __restrict__ acc) {
    const uint64_t words = (nbytes + 7) / 8, vecs = (words + 1) / 2;
    const uint64_t tid = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    const uint64_t stride = uint64_t(gridDim.x) * blockDim.x;
    uint64_t h1 = 0, h2 = 0;
    constexpr uint64_t K = 0x9E3779B97F4A7C15ull, K2 = 0xD6E8FEB86659FD93ull, K3 = 0xA0761D6478BD642Full;
    auto add = [&](uint64_t k, uint64_t a, uint64_t b) {
        const uint64_t ks = swap_halves(k);
        const uint64_t x = a ^ k, y = b ^ ks ^ K2;
        h1 += (x * y) ^ __umul64hi(x, y);
        const uint64_t x2 = (a ^ K3) + ks, y2 = (b ^ K2) + k;
        h2 += (x2 * y2) ^ __umul64hi(x2, y2);
    };
    const unsigned mis = unsigned(reinterpret_cast<uintptr_t>(p) & 15u);
    const uint64_t whole = mis == 0 ? nbytes / 16 : 0;  // vectors read with one 16-byte load
    {
        const uint4* __restrict__ q = reinterpret_cast<const uint4*>(p);
        uint64_t k = (tid + 1) * K;  // advanced by additions
        const uint64_t kstep = stride * K;
        uint64_t v = tid;
        for (; v + (kHashLoads - 1) * stride < whole; v += kHashLoads * stride) {  // eight loads in flight per thread
            uint4 x[kHashLoads];
#pragma unroll
            for (int u = 0; u < kHashLoads; ++u) x[u] = __ldg(q + v + u * stride);
#pragma unroll
            for (int u = 0; u < kHashLoads; ++u, k += kstep)
                add(k, uint64_t(x[u].x) | (uint64_t(x[u].y) << 32), uint64_t(x[u].z) | (uint64_t(x[u].w) << 32));
        }
        for (; v < whole; v += stride, k += kstep) {
            const uint4 x = __ldg(q + v);
            add(k, uint64_t(x.x) | (uint64_t(x.y) << 32), uint64_t(x.z) | (uint64_t(x.w) << 32));
        }
    }
    const bool aligned8 = (mis & 7u) == 0;
    auto word = [&](uint64_t w) -> uint64_t {
        if (w >= words) return 0;
        return aligned8 && (w + 1) * 8 <= nbytes ? reinterpret_cast<const uint64_t*>(p)[w] : word_from_bytes(p, nbytes, w);
    };
    for (uint64_t v = whole + tid; v < vecs; v += stride) add((v + 1) * K, word(2 * v), word(2 * v + 1));  // ragged end, or all of a misaligned buffer
    for (int o = 16; o > 0; o >>= 1) {
        h1 += __shfl_down_sync(0xFFFFFFFFu, h1, o);
        h2 += __shfl_down_sync(0xFFFFFFFFu, h2, o);
    }
    if ((threadIdx.x & 31) == 0) {
        atomicAdd(&acc[0], static_cast<unsigned long long>(h1));
        atomicAdd(&acc[1], static_cast<unsigned long long>(h2));
    }
}

uint64_t storage_bytes(const vf_content& c) {
    const uint64_t count = c.is_splat ? 1 : uint64_t(Type::from(c.type).numel());
    return (uint64_t(dtype_bits(c.storage_dtype)) * count + 7u) / 8u;
}

void hash_device(vf_ctx* ctx, const void* d, uint64_t nbytes, uint64_t out[2]) {
    std::unique_lock<std::mutex> lock(ctx->mu);
    DeviceGuard dev(ctx->device);
    DBuf acc(ctx, 16);
    VF_CUDA(cudaMemsetAsync(acc.p, 0, 16, ctx->stream));
    const uint64_t words = (nbytes + 7) / 8;
    if (words) {
        const uint64_t blocks = std::min<uint64_t>((words / 2 + 255) / 256 + 1, uint64_t(ctx->sm_count) * 4);  // four resident CTAs per SM
        k_hash128<<<int(blocks), 256, 0, ctx->stream>>>(static_cast<const uint8_t*>(d), nbytes, acc.as<unsigned long long>());
        VF_CUDA(cudaGetLastError());
        ++ctx->launches;
    }
    uint64_t h[2];
    VF_CUDA(cudaMemcpyAsync(h, acc.p, 16, cudaMemcpyDeviceToHost, ctx->stream));
    VF_CUDA(cudaStreamSynchronize(ctx->stream));
    out[0] = mix64(h[0] ^ nbytes);
    out[1] = mix64(h[1] + nbytes);
}

// ---- canonical serialisation (the cache key) ------------------------------------------------------------
template <class T>
void put(std::string& s, const T& v) {
    s.append(reinterpret_cast<const char*>(&v), sizeof(T));
}
template <class T>
void put_array(std::string& s, const T* p, int64_t n) {
    put(s, n);
    if (p && n > 0) s.append(reinterpret_cast<const char*>(p), size_t(n) * sizeof(T));
}

void put_elem(std::string& s, const vf_elem_type& e) {
    put(s, e.kind);
    put(s, e.dtype);
    if (e.kind == VF_ELEM_PLAIN) return;
    put(s, e.expressed);
    put(s, e.axis);
    put(s, e.qmin);
    put(s, e.qmax);
    put_array(s, e.scales, e.nparams);
    put_array(s, e.zps, e.nparams);
}

void put_transform(std::string& s, const vf_transform& t) {
    put(s, t.kind);
    switch (t.kind) {
    case VF_T_CAST_ELEM_TYPE:
    case VF_T_CONVERT_ELEM_TYPE:
    case VF_T_QUANTIZE: put_elem(s, t.elem); break;
    case VF_T_RESCALE:
    case VF_T_ADD: put(s, t.value); break;
    case VF_T_RESHAPE: put_array(s, t.a, t.rank); break;
    case VF_T_CHANGE_SHAPE_AND_ELEM_TYPE:
        put_array(s, t.a, t.rank);
        put_elem(s, t.elem);
        break;
    case VF_T_REVERSE: put(s, t.a[0]); break;
    case VF_T_BROADCAST:
    case VF_T_EXPAND_DILATED:
        put(s, t.a[0]);
        put(s, t.a[1]);
        break;
    case VF_T_REORDER:
    case VF_T_TRANSPOSE:
    case VF_T_LAYOUT_CAST: put(s, t.order); break;
    case VF_T_MEM_PERMUTE:
        put(s, t.order);
        put(s, t.mem_perm);
        break;
    case VF_T_PAD_WITH_ZERO:
    case VF_T_SUBVIEW:
    case VF_T_SWIZZLE_CONSTANT:
        put_array(s, t.a, t.rank);
        put_array(s, t.b, t.kind == VF_T_SWIZZLE_CONSTANT ? 0 : t.rank);
        break;
    case VF_T_BIT_PACK: put(s, t.width); break;
    case VF_T_SPARSIFY:
        put(s, t.compress_output);
        put_array(s, t.num_actual, t.num_actual ? t.n_num_actual : 0);
        break;
    case VF_T_RELOCATE_WEIGHTS_TABLE: {
        const vf_relocate& r = t.relocate;
        put(s, r.sparsity_ptr);
        put_array(s, r.weights_ptr, r.n_clusters);
        put_array(s, r.offsets, r.n_clusters);
        put(s, r.weights_table_size);
        put(s, r.weights_elem_bit_size);
        put(s, r.channel_offset);
        const int32_t compressed = r.num_elems ? 1 : 0;
        put(s, compressed);
        if (compressed) {
            put_array(s, r.num_elems, r.n_num_elems);
            put(s, r.compression_axis);
            put(s, r.alignment);
        }
        break;
    }
    default: break;  // Dequantize, GetSparsityMap, ScalarMultInverse: no parameters
    }
}

std::string list_key(const vf_transform* t, int n) {
    std::string s;
    for (int i = 0; i < n; ++i) put_transform(s, t[i]);
    return s;
}

// ---- owned copies of what a request refers to -------------------------------------------------------------
void check_transform(const vf_transform& t) {
    if (t.rank < 0 || t.rank > VF_MAX_RANK) raise(VF_ERR_INVALID_ARG, "transformation with rank %d", t.rank);
    if (t.kind == VF_T_RELOCATE_WEIGHTS_TABLE && (t.relocate.n_clusters < 1 || t.relocate.n_clusters > VF_MAX_CLUSTERS))
        raise(VF_ERR_INVALID_ARG, "RelocateWeightsTable with %d clusters", t.relocate.n_clusters);
    if (t.elem.kind != VF_ELEM_PLAIN && t.elem.nparams < 0) raise(VF_ERR_INVALID_ARG, "negative parameter count");
}

struct OwnedList {
    std::vector<vf_transform> t;
    std::deque<std::vector<double>> f64;   // a deque never moves its elements: the pointers below stay valid
    std::deque<std::vector<int64_t>> i64;
    OwnedList() = default;
    OwnedList(const OwnedList&) = delete;
    OwnedList& operator=(const OwnedList&) = delete;
    const int64_t* keep(const int64_t* p, int64_t n) {
        if (!p || n <= 0) return nullptr;
        i64.emplace_back(p, p + n);
        return i64.back().data();
    }
    void assign(const vf_transform* src, int n) {
        if (n < 0 || (n > 0 && !src)) raise(VF_ERR_INVALID_ARG, "NULL transformation list");
        t.assign(src, src + n);
        for (vf_transform& x : t) {
            check_transform(x);
            if (x.elem.kind != VF_ELEM_PLAIN && x.elem.nparams > 0) {
                if (!x.elem.scales || !x.elem.zps) raise(VF_ERR_INVALID_ARG, "quantized type without parameters");
                f64.emplace_back(x.elem.scales, x.elem.scales + x.elem.nparams);
                x.elem.scales = f64.back().data();
                x.elem.zps = keep(x.elem.zps, x.elem.nparams);
            }
            x.num_actual = keep(x.num_actual, x.n_num_actual);
            if (x.kind == VF_T_RELOCATE_WEIGHTS_TABLE && x.relocate.num_elems) {
                static const int64_t kNone = 0;
                const int64_t* p = keep(x.relocate.num_elems, x.relocate.n_num_elems);
                x.relocate.num_elems = p ? p : &kNone;
            }
        }
    }
};

struct OwnedBase {
    vf_content c{};
    uint64_t id = 0;
    std::vector<double> scales;
    std::vector<int64_t> zps;
    OwnedBase() = default;
    OwnedBase(const OwnedBase&) = delete;
    OwnedBase& operator=(const OwnedBase&) = delete;
    void assign(const vf_content* b, uint64_t base_id) {
        if (!b) raise(VF_ERR_INVALID_ARG, "base is NULL");
        c = *b;
        id = base_id;
        if (c.type.elem.kind != VF_ELEM_PLAIN && c.type.elem.nparams > 0) {
            if (!c.type.elem.scales || !c.type.elem.zps) raise(VF_ERR_INVALID_ARG, "quantized type without parameters");
            scales.assign(c.type.elem.scales, c.type.elem.scales + c.type.elem.nparams);
            zps.assign(c.type.elem.zps, c.type.elem.zps + c.type.elem.nparams);
            c.type.elem.scales = scales.data();
            c.type.elem.zps = zps.data();
        }
        (void)Type::from(c.type);  // validates rank and order
        const uint64_t need = storage_bytes(c);
        if (!c.data || c.nbytes < need) raise(VF_ERR_SHAPE, "base buffer holds %llu bytes, %llu needed", (unsigned long long)c.nbytes, (unsigned long long)need);
    }
};

struct Request {
    enum Kind { FOLD, EQUIVALENCE, TERMINATE } kind = FOLD;
    OwnedBase base;
    OwnedList list;      // the attribute to fold (for EQUIVALENCE: the new attribute)
    OwnedList original;  // EQUIVALENCE: the attribute whose cached result may be re-keyed
    int new_index = -1;
};

struct DevCopy {  // a device copy of a host base, released on the context's stream
    vf_ctx* ctx = nullptr;
    void* p = nullptr;
    DevCopy() = default;
    DevCopy(const DevCopy&) = delete;
    DevCopy& operator=(const DevCopy&) = delete;
    ~DevCopy() {
        if (!p) return;
        DeviceGuard dev(ctx->device);
        cudaFreeAsync(p, ctx->main_stream);
    }
};

struct Resolved {  // a base as the workers use it: readable by the device, with the key prefix that names it
    vf_content c{};
    std::string key;
    DevCopy copy;
};

void resolve(vf_ctx* ctx, const OwnedBase& b, Resolved& r) {
    r.c = b.c;
    std::string& s = r.key;
    put(s, b.c.type.rank);
    put(s, b.c.type.order);
    put_array(s, b.c.type.shape, b.c.type.rank);
    put_elem(s, b.c.type.elem);
    put(s, b.c.storage_dtype);
    put(s, b.c.is_splat);
    const uint64_t need = storage_bytes(b.c);
    put(s, need);
    if (b.id) {
        s.push_back('I');
        put(s, b.id);
        return;
    }
    if (b.c.mem_kind != VF_MEM_DEVICE) {  // hashed where it will be folded: one upload serves both
        r.copy.ctx = ctx;
        r.copy.p = upload_keep(ctx, b.c, nullptr);
        r.c.data = r.copy.p;
        r.c.mem_kind = VF_MEM_DEVICE;
    }
    uint64_t h[2];
    hash_device(ctx, r.c.data, need, h);
    s.push_back('H');
    put(s, h[0]);
    put(s, h[1]);
}

struct Entry {  // details::CachedContent
    Folded f;
    std::atomic<int> ref_count{1};
    int device = 0;
    cudaStream_t free_stream = nullptr;
    ~Entry() {
        if (!f.data) return;
        DeviceGuard dev(device);
        cudaFreeAsync(f.data, free_stream);
    }
};

}  // namespace

}  // namespace vf

using namespace vf;

struct vf_folder {
    int device = 0;
    uint64_t limit = 0;
    double threshold = 0.8;
    bool collect = false;
    cudaStream_t free_stream = nullptr;
    vf_ctx* front = nullptr;  // foreground calls (has_content / fold) run here
    std::vector<vf_ctx*> worker_ctx;
    std::vector<std::thread> workers;

    std::mutex qmu;  // request queue
    std::condition_variable qcv, idle_cv;
    std::deque<std::shared_ptr<Request>> queue;
    int active = 0;

    std::mutex cmu;  // cache map
    std::unordered_map<std::string, std::shared_ptr<Entry>> cache;
    uint64_t used = 0;

    std::mutex smu;  // statistics maxima and the last error
    vf_folder_stats st{};
    std::string last_error;

    void note_max(uint64_t vf_folder_stats::*field, uint64_t v) {
        std::lock_guard<std::mutex> lock(smu);
        if (st.*field < v) st.*field = v;
    }
    void count(uint64_t vf_folder_stats::*field) {
        if (!collect) return;
        std::lock_guard<std::mutex> lock(smu);
        ++(st.*field);
    }

    // ---- ConstantFoldingCache ------------------------------------------------------------------------
    bool has_content(const std::string& key) {  // :30-37
        std::lock_guard<std::mutex> lock(cmu);
        auto it = cache.find(key);
        if (it == cache.end()) return false;
        ++it->second->ref_count;
        return true;
    }
    std::shared_ptr<Entry> get_content(const std::string& key) {  // :120-135
        std::shared_ptr<Entry> e;
        {
            std::lock_guard<std::mutex> lock(cmu);
            auto it = cache.find(key);
            if (it != cache.end()) {
                e = it->second;
                --e->ref_count;
            }
        }
        count(e ? &vf_folder_stats::hits : &vf_folder_stats::misses);
        return e;
    }
    bool remove_locked(const std::string& key) {
        auto it = cache.find(key);
        if (it == cache.end()) return false;
        used -= it->second->f.nbytes;
        cache.erase(it);
        return true;
    }
    bool remove_content(const std::string& key) {  // :96-108
        bool removed;
        {
            std::lock_guard<std::mutex> lock(cmu);
            removed = remove_locked(key);
        }
        if (removed) count(&vf_folder_stats::erased);
        return removed;
    }
    void clean_up_locked(uint64_t& erased) {  // :51-70: lowest refCount first, down to limit * threshold
        std::vector<std::pair<int, const std::string*>> order;
        order.reserve(cache.size());
        for (const auto& kv : cache) order.emplace_back(kv.second->ref_count.load(), &kv.first);
        std::stable_sort(order.begin(), order.end(), [](const auto& a, const auto& b) { return a.first < b.first; });
        std::vector<std::string> victims;
        uint64_t left = used;
        for (const auto& o : order) {
            victims.push_back(*o.second);
            left -= cache[*o.second]->f.nbytes;
            if (double(left) <= double(limit) * threshold) break;
        }
        for (const std::string& k : victims) erased += remove_locked(k) ? 1 : 0;
    }
    void add_content(const std::string& key, Folded&& f) {  // :72-94
        auto e = std::make_shared<Entry>();
        e->f = std::move(f);
        e->device = device;
        e->free_stream = free_stream;
        uint64_t erased = 0, now_used, now_size;
        {
            std::lock_guard<std::mutex> lock(cmu);
            remove_locked(key);  // a second result for the same key replaces the first
            used += e->f.nbytes;
            cache.emplace(key, std::move(e));
            now_used = used;
            now_size = cache.size();
            if (used >= limit) clean_up_locked(erased);
        }
        if (!collect) return;
        std::lock_guard<std::mutex> lock(smu);
        ++st.added;
        st.erased += erased;
        st.max_memory_used = std::max<uint64_t>(st.max_memory_used, now_used);
        st.max_cache_size = std::max<uint64_t>(st.max_cache_size, now_size);
    }
    bool replace_key(const std::string& from, const std::string& to) {  // replaceContentAttr :137-148
        std::lock_guard<std::mutex> lock(cmu);
        auto it = cache.find(from);
        if (it == cache.end()) return false;
        std::shared_ptr<Entry> e = it->second;
        cache.erase(it);
        auto old = cache.find(to);
        if (old != cache.end()) {
            used -= old->second->f.nbytes;
            cache.erase(old);
        }
        cache.emplace(to, std::move(e));
        return true;
    }

    // ---- BackgroundConstantFolding -------------------------------------------------------------------
    void enqueue(std::shared_ptr<Request> r) {
        size_t depth;
        {
            std::lock_guard<std::mutex> lock(qmu);
            queue.push_back(std::move(r));
            depth = queue.size();
        }
        qcv.notify_one();
        if (collect) note_max(&vf_folder_stats::max_queue, depth);
    }

    bool try_partial(vf_ctx* ctx, const Request& req, const Resolved& base, const std::string& key) {  // :65-100
        const int n = int(req.list.t.size());
        const int idx = req.new_index;
        if (idx < 0 || idx >= n) return false;  // no new transformation, or nothing would be left to apply
        const std::string partial_key = base.key + list_key(req.list.t.data(), idx);
        std::shared_ptr<Entry> partial = get_content(partial_key);
        if (!partial) return false;
        Folded f = fold_keep(ctx, nullptr, &partial->f, req.list.t.data() + idx, n - idx);
        add_content(key, std::move(f));
        remove_content(partial_key);
        count(&vf_folder_stats::partial);
        return true;
    }

    void process(vf_ctx* ctx, const Request& req) {  // processFoldingRequest :118-162
        Resolved base;
        resolve(ctx, req.base, base);
        const std::string key = base.key + list_key(req.list.t.data(), int(req.list.t.size()));
        if (req.kind == Request::EQUIVALENCE) {
            const std::string orig = base.key + list_key(req.original.t.data(), int(req.original.t.size()));
            if (replace_key(orig, key)) return;
        }
        if (has_content(key)) {
            count(&vf_folder_stats::duplicated);
            return;
        }
        if (try_partial(ctx, req, base, key)) return;
        Folded f = fold_keep(ctx, &base.c, nullptr, req.list.t.data(), int(req.list.t.size()));
        add_content(key, std::move(f));
    }

    void work(vf_ctx* ctx) {
        for (;;) {
            std::shared_ptr<Request> r;
            {
                std::unique_lock<std::mutex> lock(qmu);
                qcv.wait(lock, [&] { return !queue.empty(); });
                r = std::move(queue.front());
                queue.pop_front();
                if (r->kind == Request::TERMINATE) return;
                ++active;
            }
            try {
                process(ctx, *r);
            } catch (const std::exception& e) {  // the request is dropped; a foreground fold reports the error itself
                std::lock_guard<std::mutex> lock(smu);
                ++st.failed;
                last_error = e.what();
            }
            {
                std::lock_guard<std::mutex> lock(qmu);
                --active;
            }
            idle_cv.notify_all();
        }
    }
};

extern "C" {

int vf_content_hash(vf_ctx* ctx, const vf_content* content, uint64_t out[2], char* err, size_t errlen) {
    return guard(err, errlen, [&] {
        if (!ctx || !content || !out) raise(VF_ERR_INVALID_ARG, "NULL argument");
        OwnedBase b;
        b.assign(content, 0);
        const uint64_t need = storage_bytes(b.c);
        DevCopy copy;
        const void* d = b.c.data;
        if (b.c.mem_kind != VF_MEM_DEVICE) {
            copy.ctx = ctx;
            copy.p = upload_keep(ctx, b.c, nullptr);
            d = copy.p;
        }
        hash_device(ctx, d, need, out);
    });
}

int vf_folder_create(int device, const vf_folder_options* opts, vf_folder** out, char* err, size_t errlen) {
    return guard(err, errlen, [&] {
        if (!out) raise(VF_ERR_INVALID_ARG, "out is NULL");
        *out = nullptr;
        std::unique_ptr<vf_folder> f(new vf_folder);
        f->device = device;
        f->limit = opts && opts->memory_limit_bytes ? opts->memory_limit_bytes : (4ull << 30);
        f->threshold = opts && opts->clean_threshold > 0 ? opts->clean_threshold : 0.8;
        f->collect = opts && opts->collect_statistics;
        const int n = opts && opts->max_concurrent_tasks > 0 ? opts->max_concurrent_tasks : 2;
        if (n > 64) raise(VF_ERR_INVALID_ARG, "at most 64 folding threads");
        char e[256];
        auto make_ctx = [&] {
            vf_ctx* c = nullptr;
            vf_options o{};
            o.staging_bytes = 16u << 20;  // per bounce buffer; a folder holds one context per worker plus one
            const int st = vf_ctx_create(device, &o, nullptr, &c, e, sizeof(e));
            if (st != VF_OK) raise(st, "%s", e);
            return c;
        };
        try {
            f->front = make_ctx();
            for (int i = 0; i < n; ++i) f->worker_ctx.push_back(make_ctx());
            DeviceGuard dev(device);
            VF_CUDA(cudaStreamCreateWithFlags(&f->free_stream, cudaStreamNonBlocking));
        } catch (...) {
            if (f->front) vf_ctx_destroy(f->front);
            for (vf_ctx* c : f->worker_ctx) vf_ctx_destroy(c);
            throw;
        }
        vf_folder* raw = f.release();
        for (int i = 0; i < n; ++i) raw->workers.emplace_back([raw, i] { raw->work(raw->worker_ctx[size_t(i)]); });
        *out = raw;
    });
}

void vf_folder_destroy(vf_folder* f) {
    if (!f) return;
    for (size_t i = 0; i < f->workers.size(); ++i) {  // one termination token per worker, behind what is queued
        auto r = std::make_shared<Request>();
        r->kind = Request::TERMINATE;
        f->enqueue(std::move(r));
    }
    for (std::thread& t : f->workers) t.join();
    f->cache.clear();
    {
        DeviceGuard dev(f->device);
        cudaStreamSynchronize(f->free_stream);
        cudaStreamDestroy(f->free_stream);
    }
    for (vf_ctx* c : f->worker_ctx) vf_ctx_destroy(c);
    vf_ctx_destroy(f->front);
    delete f;
}

int vf_folder_enqueue(vf_folder* f, const vf_content* base, uint64_t base_id, const vf_transform* t, int n, int new_index,
                      char* err, size_t errlen) {
    return guard(err, errlen, [&] {
        if (!f) raise(VF_ERR_INVALID_ARG, "folder is NULL");
        auto r = std::make_shared<Request>();
        r->base.assign(base, base_id);
        r->list.assign(t, n);
        r->new_index = new_index;
        f->enqueue(std::move(r));
    });
}

int vf_folder_enqueue_equivalence(vf_folder* f, const vf_content* base, uint64_t base_id, const vf_transform* t_orig, int n_orig,
                                  const vf_transform* t_new, int n_new, char* err, size_t errlen) {
    return guard(err, errlen, [&] {
        if (!f) raise(VF_ERR_INVALID_ARG, "folder is NULL");
        auto r = std::make_shared<Request>();
        r->kind = Request::EQUIVALENCE;
        r->base.assign(base, base_id);
        r->original.assign(t_orig, n_orig);
        r->list.assign(t_new, n_new);
        f->enqueue(std::move(r));
    });
}

int vf_folder_wait_idle(vf_folder* f, char* err, size_t errlen) {
    return guard(err, errlen, [&] {
        if (!f) raise(VF_ERR_INVALID_ARG, "folder is NULL");
        std::unique_lock<std::mutex> lock(f->qmu);
        f->idle_cv.wait(lock, [&] { return f->queue.empty() && f->active == 0; });
    });
}

int vf_folder_has_content(vf_folder* f, const vf_content* base, uint64_t base_id, const vf_transform* t, int n, int* found,
                          char* err, size_t errlen) {
    return guard(err, errlen, [&] {
        if (!f || !found) raise(VF_ERR_INVALID_ARG, "NULL argument");
        OwnedBase b;
        b.assign(base, base_id);
        if (n < 0 || (n > 0 && !t)) raise(VF_ERR_INVALID_ARG, "NULL transformation list");
        for (int i = 0; i < n; ++i) check_transform(t[i]);
        Resolved r;
        resolve(f->front, b, r);
        *found = f->has_content(r.key + list_key(t, n)) ? 1 : 0;
    });
}

int vf_folder_remove(vf_folder* f, const vf_content* base, uint64_t base_id, const vf_transform* t, int n, char* err,
                     size_t errlen) {
    return guard(err, errlen, [&] {
        if (!f) raise(VF_ERR_INVALID_ARG, "folder is NULL");
        OwnedBase b;
        b.assign(base, base_id);
        if (n < 0 || (n > 0 && !t)) raise(VF_ERR_INVALID_ARG, "NULL transformation list");
        for (int i = 0; i < n; ++i) check_transform(t[i]);
        Resolved r;
        resolve(f->front, b, r);
        f->remove_content(r.key + list_key(t, n));
    });
}

int vf_folder_fold(vf_folder* f, const vf_content* base, uint64_t base_id, const vf_transform* t, int n, void* dst,
                   uint64_t dst_bytes, int dst_mem_kind, uint64_t* dst_written, vf_tensor_type* out_type, double* scales_buf,
                   int64_t* zps_buf, int64_t params_cap, int* from_cache, char* err, size_t errlen) {
    return guard(err, errlen, [&] {
        if (!f) raise(VF_ERR_INVALID_ARG, "folder is NULL");
        OwnedBase b;
        b.assign(base, base_id);
        if (n < 0 || (n > 0 && !t)) raise(VF_ERR_INVALID_ARG, "NULL transformation list");
        for (int i = 0; i < n; ++i) check_transform(t[i]);
        Resolved r;
        resolve(f->front, b, r);
        std::shared_ptr<Entry> hit = f->get_content(r.key + list_key(t, n));
        if (from_cache) *from_cache = hit ? 1 : 0;
        if (hit) {  // Content::copyTo of the cached content
            const uint64_t w = copy_folded(f->front, hit->f, dst, dst_bytes, dst_mem_kind, out_type, scales_buf, zps_buf, params_cap);
            if (dst_written) *dst_written = w;
            return;
        }
        // fold(bypassCache): not added to the cache, as in the reference
        char e[512] = {0};
        const int st = vf_fold(f->front, &r.c, t, n, dst, dst_bytes, dst_mem_kind, dst_written, out_type, scales_buf, zps_buf,
                               params_cap, nullptr, e, sizeof(e));
        if (st != VF_OK) raise(st, "%s", e);
    });
}

int vf_folder_last_error(vf_folder* f, char* buf, size_t buflen) {
    if (!f || !buf || !buflen) return VF_ERR_INVALID_ARG;
    std::lock_guard<std::mutex> lock(f->smu);
    snprintf(buf, buflen, "%s", f->last_error.c_str());
    return VF_OK;
}

int vf_folder_statistics(vf_folder* f, vf_folder_stats* out) {
    if (!f || !out) return VF_ERR_INVALID_ARG;
    uint64_t used, size;
    {
        std::lock_guard<std::mutex> lock(f->cmu);
        used = f->used;
        size = f->cache.size();
    }
    std::lock_guard<std::mutex> lock(f->smu);
    *out = f->st;
    out->memory_used = used;
    out->cache_size = size;
    return VF_OK;
}

}  // extern "C"
