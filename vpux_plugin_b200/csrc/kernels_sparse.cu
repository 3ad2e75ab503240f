// Sparsify + GetSparsityMap for a whole list of weight tensors in three launches
// (attributes/sparsify.cpp:120-161, attributes/get_sparsity_map.cpp:30-66, utils/sparsity.cpp:35-84).
//
// A warp owns one output channel (one row of `work` elements). Rows that allow it are read with 16-byte
// loads: the non-sparse test runs on a whole vector and yields a bit mask, the bitmap is written from the
// masks directly, and the compaction packs the kept elements in a per-warp shared-memory stage that is
// written out in aligned 16-byte vectors. Every compacted row starts on a 16-byte boundary and is padded
// with zeros up to the next one, so whole-vector stores never touch a neighbouring row.
#include <algorithm>

#include "device_utils.cuh"
#include "kernels.h"

namespace vf {

namespace {

constexpr unsigned kFull = 0xffffffffu;
constexpr int kWarps = 8;  // warps per CTA

template <int ES>
struct ElemT;
template <> struct ElemT<1> { using T = uint8_t; };
template <> struct ElemT<2> { using T = uint16_t; };
template <> struct ElemT<4> { using T = uint32_t; };

// The search for a unit's job is a chain of dependent loads: on the job table in device memory each step costs an
// L2 round trip, which for rows of a few hundred bytes is as long as reading the row. A CTA therefore copies the
// jobs' first units into shared memory once (tables of up to kStagedJobs entries) and searches there.
constexpr int kStagedJobs = 512;

__device__ __forceinline__ void stage_unit_begins(const SparseJob* __restrict__ jobs, int njobs, int64_t* begins) {
    if (njobs <= kStagedJobs) {
        for (int i = threadIdx.x; i < njobs; i += blockDim.x) begins[i] = jobs[i].unit_begin;
        __syncthreads();
    }
}

__device__ __forceinline__ int find_sparse_job(const SparseJob* __restrict__ jobs, const int64_t* begins, int njobs, int64_t unit) {
    int lo = 0, hi = njobs - 1;
    if (njobs <= kStagedJobs) {
        while (lo < hi) {  // last job whose unit_begin <= unit
            const int mid = (lo + hi + 1) >> 1;
            if (begins[mid] <= unit) lo = mid;
            else hi = mid - 1;
        }
        return lo;
    }
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (jobs[mid].unit_begin <= unit) lo = mid;
        else hi = mid - 1;
    }
    return lo;
}

// Bit k of the result is set when element k of the 16-byte vector differs from the sparsify value.
template <int ES>
__device__ __forceinline__ uint32_t dense_mask(const uint4& v, int dt, uint32_t iv_rep, float fv) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t m = 0;
    if (ES == 1) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            // 8-bit floats compare as float with zero: the sign bit does not count
            const uint32_t x = (dt == VF_DT_F8E4M3FN || dt == VF_DT_F8E5M2) ? (w[k] & 0x7F7F7F7Fu) : w[k];
            const uint32_t ne = __vcmpne4(x, iv_rep);  // 0xff in every byte that differs
            m |= (((ne & 0x08040201u) * 0x01010101u) >> 24) << (4 * k);
        }
    } else if (ES == 2) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const uint16_t h = uint16_t(w[k >> 1] >> (16 * (k & 1)));
            const float f = dt == VF_DT_F16 ? f16_bits_to_f32(h) : bf16_bits_to_f32(h);
            m |= uint32_t(f != fv) << k;
        }
    } else {
#pragma unroll
        for (int k = 0; k < 4; ++k) m |= uint32_t(__uint_as_float(w[k]) != fv) << k;
    }
    return m;
}

__device__ __forceinline__ int warp_sum(int v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(kFull, v, o);
    return v;
}

// ------------------------------------------------------------------------------------------------------
// pass 1: per-channel counts and bitmap rows
// ------------------------------------------------------------------------------------------------------
template <int ES>
__device__ __forceinline__ int scan_row_vec(const SparseJob& J, int64_t c, int lane, uint32_t iv_rep, float fv) {
    constexpr int EPV = 16 / ES;
    const uint4* row = reinterpret_cast<const uint4*>(static_cast<const char*>(J.in) + c * J.work * ES);
    const int64_t nvec = J.work / EPV;
    uint8_t* mrow = J.map ? J.map + c * J.map_row_bytes : nullptr;
    int cnt = 0;
    for (int64_t v0 = 0; v0 < nvec; v0 += 32) {
        const int64_t v = v0 + lane;
        uint32_t m = 0;
        if (v < nvec) m = dense_mask<ES>(__ldg(row + v), J.dt, iv_rep, fv);
        cnt += __popc(m);
        if (mrow) {  // LSB = lowest index (get_sparsity_map.cpp:44-53)
            if (ES == 1) {
                if (v < nvec) *reinterpret_cast<uint16_t*>(mrow + v * 2) = uint16_t(m);
            } else if (ES == 2) {
                if (v < nvec) mrow[v] = uint8_t(m);
            } else {
                const uint32_t hi = __shfl_down_sync(kFull, m, 1);
                if (!(lane & 1) && v < nvec) mrow[v >> 1] = uint8_t(m | (hi << 4));
            }
        }
    }
    return cnt;
}

__device__ __forceinline__ int scan_row_scalar(const SparseJob& J, int64_t c, int lane, float fv) {
    const int64_t base = c * J.work;
    uint8_t* mrow = J.map ? J.map + c * J.map_row_bytes : nullptr;
    int cnt = 0;
    for (int64_t i = 0; i < J.work; i += 32) {
        const bool d = (i + lane < J.work) && is_dense(J.in, J.dt, base + i + lane, J.sv, fv);
        const unsigned bits = __ballot_sync(kFull, d);
        cnt += d ? 1 : 0;
        if (mrow && lane < 4) {
            const int64_t byte = (i >> 3) + lane;
            if (byte * 8 < J.work) mrow[byte] = uint8_t(bits >> (8 * lane));
        }
    }
    return cnt;
}

__global__ void __launch_bounds__(kWarps * 32) k_sparse_scan_batch(const SparseJob* __restrict__ jobs, int njobs,
                                                                   int64_t total_units) {
    chain_enter();
    __shared__ int64_t begins[kStagedJobs];
    stage_unit_begins(jobs, njobs, begins);
    const int lane = threadIdx.x & 31;
    const int64_t warp = int64_t(blockIdx.x) * kWarps + (threadIdx.x >> 5);
    const int64_t nwarps = int64_t(gridDim.x) * kWarps;
    for (int64_t u = warp; u < total_units; u += nwarps) {
        const SparseJob J = jobs[find_sparse_job(jobs, begins, njobs, u)];
        const int64_t c = u - J.unit_begin;
        const float fv = sparse_value_as_float(J.dt, J.sv);
        const uint32_t iv_rep = uint32_t(uint8_t(J.sv)) * 0x01010101u;
        int cnt;
        if (!J.vec) cnt = scan_row_scalar(J, c, lane, fv);
        else if (J.es == 1) cnt = scan_row_vec<1>(J, c, lane, iv_rep, fv);
        else if (J.es == 2) cnt = scan_row_vec<2>(J, c, lane, iv_rep, fv);
        else cnt = scan_row_vec<4>(J, c, lane, iv_rep, fv);
        cnt = warp_sum(cnt);
        if (J.map) {  // zero the padding up to the 128-bit aligned row
            uint8_t* mrow = J.map + c * J.map_row_bytes;
            for (int64_t b = ((J.work + 7) >> 3) + lane; b < J.map_row_bytes; b += 32) mrow[b] = 0;
        }
        if (lane == 0) J.counts[c] = cnt;
    }
}

// ------------------------------------------------------------------------------------------------------
// pass 2: one CTA per tensor, exclusive scan of align16(count * es) -> offsets[0..oc], total -> totals[j]
// ------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void block_offsets(const int64_t* __restrict__ counts, int64_t oc, int es, int64_t* __restrict__ offsets,
                                              int64_t* total_out) {
    __shared__ long long warp_sums[32];
    __shared__ long long carry_s;
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    if (tid == 0) carry_s = 0;
    __syncthreads();
    for (int64_t base = 0; base < oc; base += blockDim.x) {
        const int64_t i = base + tid;
        long long v = 0;
        if (i < oc) v = ((counts[i] * es + 15) / 16) * 16;
        long long incl = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const long long t = __shfl_up_sync(kFull, incl, o);
            if (lane >= o) incl += t;
        }
        if (lane == 31) warp_sums[wid] = incl;
        __syncthreads();
        if (wid == 0) {
            const long long w = warp_sums[lane];
            long long wi = w;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const long long t = __shfl_up_sync(kFull, wi, o);
                if (lane >= o) wi += t;
            }
            warp_sums[lane] = wi - w;  // exclusive
        }
        __syncthreads();
        const long long excl = carry_s + warp_sums[wid] + incl - v;
        if (i < oc) offsets[i] = excl;
        __syncthreads();
        if (tid == blockDim.x - 1) carry_s = excl + v;
        __syncthreads();
    }
    if (tid == 0) {
        offsets[oc] = carry_s;
        if (total_out) *total_out = carry_s;
    }
}

__global__ void __launch_bounds__(1024) k_sparse_offsets_batch(const SparseJob* __restrict__ jobs,
                                                               int64_t* __restrict__ totals) {
    chain_enter();
    const SparseJob J = jobs[blockIdx.x];
    if (!J.offsets) {
        if (threadIdx.x == 0) totals[blockIdx.x] = 0;
        return;
    }
    block_offsets(J.counts, J.oc, J.es, J.offsets, totals + blockIdx.x);
}

__global__ void __launch_bounds__(1024) k_offsets_batch(const OffsetsJob* __restrict__ jobs) {
    chain_enter();
    const OffsetsJob J = jobs[blockIdx.x];
    block_offsets(J.counts, J.oc, J.es, J.offsets, nullptr);
}

// ------------------------------------------------------------------------------------------------------
// pass 3: compaction
// ------------------------------------------------------------------------------------------------------
// `stage` is this warp's shared-memory buffer of 33 vectors: up to 15 bytes carried over from the previous
// step plus the kept elements of 32 vectors.
template <int ES>
__device__ __forceinline__ void compact_row_vec(const SparseJob& J, int64_t c, int lane, uint4* stage, uint32_t iv_rep,
                                                float fv, int* flags) {
    using T = typename ElemT<ES>::T;
    constexpr int EPV = 16 / ES;
    T* sbuf = reinterpret_cast<T*>(stage);
    const uint4* row = reinterpret_cast<const uint4*>(static_cast<const char*>(J.in) + c * J.work * ES);
    const int64_t nvec = J.work / EPV;
    const uint64_t obyte = uint64_t(J.offsets[c]);
    const uint64_t room = obyte < J.capacity ? J.capacity - obyte : 0;
    uint4* out = reinterpret_cast<uint4*>(J.data + obyte);
    int fill = 0;           // elements carried in the stage (< EPV)
    uint64_t flushed = 0;   // vectors already written
    for (int64_t v0 = 0; v0 < nvec; v0 += 32) {
        const int64_t v = v0 + lane;
        uint4 x = make_uint4(0, 0, 0, 0);
        uint32_t m = 0;
        if (v < nvec) {
            x = __ldg(row + v);
            m = dense_mask<ES>(x, J.dt, iv_rep, fv);
        }
        const int n = __popc(m);
        int incl = n;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(kFull, incl, o);
            if (lane >= o) incl += t;
        }
        const int total = __shfl_sync(kFull, incl, 31);
        int pos = fill + incl - n;
        const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
        for (int k = 0; k < EPV; ++k) {
            if ((m >> k) & 1u) {
                const uint32_t word = w[(k * ES) >> 2];
                sbuf[pos++] = T(word >> (8 * ((k * ES) & 3)));
            }
        }
        __syncwarp();
        const int have = fill + total;
        const int nv = have / EPV;  // <= 32
        if (lane < nv) {
            if ((flushed + uint64_t(lane) + 1) * 16 <= room) out[flushed + lane] = stage[lane];
            else set_flag(flags, VF_FLAG_OVERFLOW);
        }
        const int rem = have - nv * EPV;
        T carry = 0;
        if (lane < rem) carry = sbuf[nv * EPV + lane];
        __syncwarp();
        if (lane < rem) sbuf[lane] = carry;
        __syncwarp();
        flushed += uint64_t(nv);
        fill = rem;
    }
    if (fill > 0) {  // last, partly filled vector: the gap up to the next channel's start is zero
        if (lane >= fill && lane < EPV) sbuf[lane] = 0;
        __syncwarp();
        if (lane == 0) {
            if ((flushed + 1) * 16 <= room) out[flushed] = stage[0];
            else set_flag(flags, VF_FLAG_OVERFLOW);
        }
        __syncwarp();
    }
}

template <int ES>
__device__ __forceinline__ void compact_row_scalar(const SparseJob& J, int64_t c, int lane, float fv, int* flags) {
    using T = typename ElemT<ES>::T;
    const int64_t base = c * J.work;
    const uint64_t obyte = uint64_t(J.offsets[c]);
    int64_t run = 0;
    for (int64_t i = 0; i < J.work; i += 32) {
        const bool d = (i + lane < J.work) && is_dense(J.in, J.dt, base + i + lane, J.sv, fv);
        const unsigned bits = __ballot_sync(kFull, d);
        if (d) {
            const uint64_t pos = obyte + uint64_t(run + __popc(bits & ((1u << lane) - 1u))) * ES;
            if (pos + ES <= J.capacity) *reinterpret_cast<T*>(J.data + pos) = static_cast<const T*>(J.in)[base + i + lane];
            else set_flag(flags, VF_FLAG_OVERFLOW);
        }
        run += __popc(bits);
    }
    const uint64_t end = obyte + uint64_t(run) * ES;
    const uint64_t next = uint64_t(J.offsets[c + 1]);
    for (uint64_t b = end + lane; b < next && b < J.capacity; b += 32) J.data[b] = 0;
}

__global__ void __launch_bounds__(kWarps * 32) k_sparse_compact_batch(const SparseJob* __restrict__ jobs, int njobs,
                                                                      int64_t total_units, int* flags) {
    chain_enter();
    __shared__ uint4 stage_all[kWarps][34];
    __shared__ int64_t begins[kStagedJobs];
    stage_unit_begins(jobs, njobs, begins);
    const int lane = threadIdx.x & 31;
    uint4* stage = stage_all[threadIdx.x >> 5];
    const int64_t warp = int64_t(blockIdx.x) * kWarps + (threadIdx.x >> 5);
    const int64_t nwarps = int64_t(gridDim.x) * kWarps;
    for (int64_t u = warp; u < total_units; u += nwarps) {
        const SparseJob J = jobs[find_sparse_job(jobs, begins, njobs, u)];
        if (!J.data) continue;
        const int64_t c = u - J.unit_begin;
        const float fv = sparse_value_as_float(J.dt, J.sv);
        const uint32_t iv_rep = uint32_t(uint8_t(J.sv)) * 0x01010101u;
        if (J.vec) {
            if (J.es == 1) compact_row_vec<1>(J, c, lane, stage, iv_rep, fv, flags);
            else if (J.es == 2) compact_row_vec<2>(J, c, lane, stage, iv_rep, fv, flags);
            else compact_row_vec<4>(J, c, lane, stage, iv_rep, fv, flags);
        } else {
            if (J.es == 1) compact_row_scalar<1>(J, c, lane, fv, flags);
            else if (J.es == 2) compact_row_scalar<2>(J, c, lane, fv, flags);
            else compact_row_scalar<4>(J, c, lane, fv, flags);
        }
    }
}

}  // namespace

void launch_sparsify_batch(vf_ctx* ctx, std::vector<SparseJob>& jobs, int64_t* d_totals) {
    if (jobs.empty()) return;
    int64_t units = 0;
    bool any_data = false;
    for (auto& j : jobs) {
        j.unit_begin = units;
        units += j.oc;
        const auto a16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
        j.vec = a16(j.in) && (j.work * j.es) % 16 == 0 && (!j.map || (a16(j.map) && j.map_row_bytes % 16 == 0)) &&
                (!j.data || a16(j.data));
        any_data |= j.data != nullptr;
    }
    DBuf table;
    const SparseJob* d_jobs = static_cast<const SparseJob*>(upload_table(ctx, jobs.data(), jobs.size() * sizeof(SparseJob), table));
    const int grid = int(std::min<int64_t>((units + kWarps - 1) / kWarps, int64_t(ctx->sm_count) * 8));
    const int njobs = int(jobs.size());
    VF_CUDA(launch_chained(k_sparse_scan_batch, grid, kWarps * 32, 0, ctx->stream, d_jobs, njobs, units));
    VF_CUDA(launch_chained(k_sparse_offsets_batch, njobs, 1024, 0, ctx->stream, d_jobs, d_totals));
    ctx->launches += 2;
    if (any_data) {
        VF_CUDA(launch_chained(k_sparse_compact_batch, grid, kWarps * 32, 0, ctx->stream, d_jobs, njobs, units, ctx->d_flags));
        ctx->launches += 1;
    }
}

void launch_offsets_batch(vf_ctx* ctx, const std::vector<OffsetsJob>& jobs) {
    if (jobs.empty()) return;
    DBuf d;
    const OffsetsJob* d_jobs = static_cast<const OffsetsJob*>(upload_table(ctx, jobs.data(), jobs.size() * sizeof(OffsetsJob), d));
    launch_offsets_batch_at(ctx, d_jobs, int(jobs.size()));
}

void launch_offsets_batch_at(vf_ctx* ctx, const OffsetsJob* d_jobs, int njobs) {
    if (njobs <= 0) return;
    VF_CUDA(launch_chained(k_offsets_batch, njobs, 1024, 0, ctx->stream, d_jobs));
    ctx->launches += 1;
}

}  // namespace vf
