// Host-callable launch wrappers of the CUDA kernels. Every wrapper enqueues on ctx->stream and bumps
// ctx->launches by the number of kernels it launched.
#pragma once

#include "common.h"

namespace vf {

struct Geom {  // index geometry shared by the layout kernels (rank <= VF_MAX_RANK, memory order)
    int rank;
    int64_t in_shape[VF_MAX_RANK];   // input memory shape
    int64_t out_shape[VF_MAX_RANK];  // output memory shape
    int64_t src_stride[VF_MAX_RANK]; // for each OUTPUT memory dim: stride (elements) into the input buffer
    int64_t offset[VF_MAX_RANK];     // per output memory dim: pad-before (pad) or subview offset
};

// ---- elementwise (general path) ----------------------------------------------------------------------
// Quantize with supplied parameters. per-tensor: n_params == 1. per-axis: params indexed by
// (idx / inner) % axis_size. `d_scales`/`d_zps` are device arrays.
void launch_quantize(vf_ctx* ctx, const void* in, int in_dt, bool in_splat, void* out, int out_dt, int64_t n,
                     const double* d_scales, const int64_t* d_zps, int64_t axis_size, int64_t inner, int64_t qmin,
                     int64_t qmax);
void launch_dequantize(vf_ctx* ctx, const void* in, int in_dt, bool in_splat, float* out, int64_t n,
                       const double* d_scales, const int64_t* d_zps, int64_t axis_size, int64_t inner);
void launch_rescale_add(vf_ctx* ctx, const void* in, int in_dt, bool in_splat, float* out, int64_t n, float c,
                        bool is_add);
// copyTo element conversion: storage dtype -> logical dtype (byte-sized), splat-aware
void launch_convert(vf_ctx* ctx, const void* in, int in_dt, bool in_splat, void* out, int out_dt, int64_t n);
// copyTo sub-byte packing: `per_byte` elements of `in` (read as int8) into each output byte, low bits first
void launch_pack_subbyte(vf_ctx* ctx, const void* in, int in_dt, uint8_t* out, int64_t n_in, int per_byte);
// subByteConversion: `n_out` elements of `bits` (1 / 2 / 4) bits each, low bits first, to one byte each
void launch_unpack_subbyte(vf_ctx* ctx, const uint8_t* in, uint8_t* out, int64_t n_out, int bits, bool sign_extend);
// SwizzleConstant: permutes the 16- / 32-byte chunks of a buffer whose size is a multiple of 512 / 1024 bytes
// `in` holds in_bytes valid bytes (16-byte aligned start); the rest of the `bytes` of the swizzled buffer reads as `pad`
void launch_swizzle(vf_ctx* ctx, const void* in, uint64_t in_bytes, uint8_t pad, void* out, uint64_t bytes, int swizzle_key, int arch);
// BitPack<4>: reads pairs through getValues<uint8_t>()
void launch_bitpack4(vf_ctx* ctx, const void* in, int in_dt, uint8_t* out, int64_t n_in);
void launch_fill_bytes(vf_ctx* ctx, void* out, uint8_t value, uint64_t bytes);

// ---- layout ----------------------------------------------------------------------------------------
// out[o] = in[sum_d coord_d(o) * src_stride[d]]   (arbitrary memory permutation, element size es bytes)
void launch_permute(vf_ctx* ctx, const void* in, void* out, const Geom& g, int es);
// PadWithZero: windows the input into the output; outside the window writes fill[dim0 index] or fill[0].
// `d_fill` is a device array of `n_fill` elements of size es (already converted to the storage type);
// n_fill == 1: uniform fill; otherwise indexed by the coordinate along output memory dim `fill_dim`.
void launch_pad(vf_ctx* ctx, const void* in, bool in_splat, void* out, const Geom& g, int es, const void* d_fill,
                int64_t n_fill, int fill_dim);
void launch_subview(vf_ctx* ctx, const void* in, void* out, const Geom& g, int es);
// the same on 1- / 2- / 4-bit storage (bit fields, low bits first)
void launch_subview_subbyte(vf_ctx* ctx, const void* in, void* out, const Geom& g, int bits);

// ---- sparsity --------------------------------------------------------------------------------------
// Per output channel: non-sparse count and (optionally) the sparsity bitmap row.
// `in` holds OC rows of `work` elements of logical dtype `dt` (i8/u8/f16/bf16/f32).
void launch_sparsity_scan(vf_ctx* ctx, const void* in, int dt, int64_t oc, int64_t work, int64_t sparse_value,
                          int64_t* d_counts, uint8_t* d_map, int64_t map_row_bytes);
// Exclusive prefix sum of align16(count*es) -> d_offsets[oc+1] (bytes); total at d_offsets[oc]
void launch_sparse_offsets(vf_ctx* ctx, const int64_t* d_counts, int64_t oc, int es, int64_t* d_offsets);
// Per-OC stream compaction into `out` at d_offsets; zero-fills each channel's alignment gap. `capacity`
// is the byte size of `out`; an overflow sets VF_FLAG_OVERFLOW and drops the excess.
void launch_sparse_compact(vf_ctx* ctx, const void* in, int dt, int64_t oc, int64_t work, int64_t sparse_value,
                           const int64_t* d_offsets, uint8_t* out, uint64_t capacity);

// Many tensors per launch. One entry per tensor; all pointers are device pointers.
struct SparseJob {
    const void* in;         // [oc][work] elements of logical dtype `dt`
    int dt, es;             // element type and its size in bytes
    int64_t oc, work;
    long long sv;           // sparsify value
    int64_t* counts;        // [oc], always written
    uint8_t* map;           // optional bitmap, rows of map_row_bytes
    int64_t map_row_bytes;
    int64_t* offsets;       // [oc + 1] byte offsets of the compacted rows (scratch); NULL when `data` is NULL
    uint8_t* data;          // optional compacted output
    uint64_t capacity;      // bytes behind `data`
    int vec;                // rows, map and data allow 16-byte accesses (set by launch_sparsify_batch)
    int64_t unit_begin;     // index of this tensor's first output channel in the launch (set by the launcher)
};
// Three launches for the whole list: counts + bitmaps, per-tensor offsets (total bytes of tensor j into
// d_totals[j]; 0 for tensors without `data`), compaction. An overflow of `capacity` sets VF_FLAG_OVERFLOW.
void launch_sparsify_batch(vf_ctx* ctx, std::vector<SparseJob>& jobs, int64_t* d_totals);
// Exclusive prefix sums of align16(count * es) for many count arrays in one launch (one CTA per entry).
struct OffsetsJob {
    const int64_t* counts;  // [oc]
    int64_t oc;
    int es;
    int64_t* offsets;       // [oc + 1]
};
void launch_offsets_batch(vf_ctx* ctx, const std::vector<OffsetsJob>& jobs);
// The same for a job list that is in device memory already.
void launch_offsets_batch_at(vf_ctx* ctx, const OffsetsJob* d_jobs, int njobs);

// Makes the runtime load the kernels of the three launchers above (cudaFuncGetAttributes, nothing is launched):
// module loading may allocate device memory, which vf_sparsify_noalloc must not do once the embedder owns the GPU.
void preload_sparsity_kernels();
// Set-up of vf_sparsify_noalloc for a new context (noalloc.cu); the context's device is current.
void noalloc_prepare(vf_ctx* ctx);

// ---- statistics --------------------------------------------------------------------------------------
// min/max (over values and 0) or absmax per unit of `unit_len` consecutive elements, then
// calcScaleAndZeroPoint. Any output may be NULL.
void launch_unit_stats(vf_ctx* ctx, const void* in, int in_dt, int64_t units, int64_t unit_len, int range_mode,
                       int64_t qmin, int64_t qmax, double* d_scales, int64_t* d_zps, float* d_rmin, float* d_rmax);

// ---- weights table -----------------------------------------------------------------------------------
struct TableArgs {
    int64_t oc;
    const double* d_wscale;  // [oc] or [1]
    int64_t n_wscale;
    double in_scale, out_scale;  // broadcast per-tensor activation scales (per-channel ones go via arrays)
    const double* d_in_scale;    // optional [oc]
    const double* d_out_scale;   // optional [oc]
    double const_scale;
    int in_quantized, out_quantized, weights_quantized, in_is_float;
    const int32_t* d_wptrs;  // optional explicit
    const int32_t* d_sptrs;
    int32_t wbase, wstep, sbase, sstep;
    const int64_t* d_nnz_offsets;  // optional: column 0 = wbase + offsets[oc] (exclusive prefix sums, bytes)
    const float* d_bias;           // optional
    int bias_is_splat;
    int32_t* d_table;              // batch launches: where this table goes
    int64_t unit_begin;            // batch launches: index of this table's first row (set by the launcher)
};
void launch_weights_table(vf_ctx* ctx, const TableArgs& a, int32_t* d_table);
// All tables of `tabs` (each with its d_table) in one launch over a device copy of the list.
// `offsets_first`: prefix-sum jobs whose results the tables read; their kernel is launched right before the tables'.
void launch_weights_table_batch(vf_ctx* ctx, std::vector<TableArgs>& tabs, const std::vector<OffsetsJob>* offsets_first = nullptr);

// Reverse: every run of `run` consecutive elements reversed; Broadcast: every block of `after` elements written
// `factor` times; ExpandDilated: OIYX taps spread by the dilations, the gaps filled from `d_fill` (n_fill == 1:
// one value, else indexed by (o / fill_stride) % fill_extent); ScalarMultInverse: 1.f / v as f32
void launch_reverse(vf_ctx* ctx, const void* in, void* out, int64_t n, int64_t run, int es);
void launch_broadcast(vf_ctx* ctx, const void* in, void* out, int64_t n_out, int64_t after, int64_t factor, int es);
void launch_expand_dilated(vf_ctx* ctx, const void* in, bool in_splat, void* out, int64_t n_out, int64_t dky, int64_t dkx,
                           int64_t ky, int64_t kx, int64_t dil_y, int64_t dil_x, const void* d_fill, int64_t n_fill,
                           int64_t fill_stride, int64_t fill_extent, int es);
void launch_inverse(vf_ctx* ctx, const void* in, int in_dt, float* out, int64_t n);

// RelocateWeightsTable: rows [0, oc) of a weights table `in` -> `out` with columns 0 / 1 rebased
struct RelocateArgs {
    int64_t oc;                            // rows to patch
    int in_splat;                          // `in` holds one element
    int n_clusters;
    int32_t weights_ptr[VF_MAX_CLUSTERS];
    int64_t offsets[VF_MAX_CLUSTERS];      // first channel of each cluster
    int64_t cross[VF_MAX_CLUSTERS];        // first row that belongs to cluster c (cross[0] unused)
    int32_t sparsity_ptr;
    int32_t channel_offset;
    const int64_t* d_steps;                // optional [oc]: byte offset of each channel's compressed weight set
    uint32_t wptr_offset;                  // with d_steps: bytes of the channel_offset sets sliced away in front
};
void launch_relocate(vf_ctx* ctx, const int32_t* in, int32_t* out, const RelocateArgs& a);

// ---- synthetic weights -------------------------------------------------------------------------------
void launch_synth(vf_ctx* ctx, const vf_synth_spec& s, void* dst, uint64_t count);

// ---- fused weight quantization (hot path) ------------------------------------------------------------
struct RowQuantArgs {
    const void* in;
    int in_dt;               // F32 / F16 / BF16
    int64_t rows, cols;      // tensor viewed as [rows, cols] row-major
    int64_t group;           // 0: one unit per row, else units of `group` elements along cols
    int range_mode;
    int64_t qmin, qmax;
    int out_signed;          // codes stored as i8 (1) or u8 (0)
    // store stage
    int pack4;               // BitPack<4> of the codes
    // OIYX -> OYXI permutation inside a row: cols = ic * khw; output row = khw * ic_pad (pad lanes = 0);
    // khw == 0 disables the permutation
    int64_t ic, khw, ic_pad;
    int64_t rows_pad;        // output rows (>= rows); extra rows are zero
    void* codes;
    // side outputs (device pointers, may be NULL)
    double* scales;
    int64_t* zps;
    uint16_t* scales_f16;
    uint8_t* zps_u4;
    void* dequant;
    int dequant_dt;
    // parameters supplied by the caller (the Quantize attribute's scales / zero points, device arrays with one
    // entry per unit) instead of derived from the data; NULL: derive them. `codes` may then be NULL when only
    // the dequantized copy is wanted (row kernel).
    const double* given_scales;
    const int64_t* given_zps;
    int64_t unit_begin;      // filled by launch_rowquant_batch: index of this job's first chunk / row in the launch
    int lanes_per_row;       // filled by launch_rowquant_batch (k_convv): 8, 16 or 32 lanes share an output channel
    int unit_cost;           // (k_convv) relative cost of one of this job's units
    int64_t work_begin;      // (k_convv) sum of the costs of all units in front of this job
};
// Launches all `jobs` (same kind, pairwise rowquant_compatible) with ONE kernel over a device job table.
void launch_rowquant_batch(vf_ctx* ctx, int kind, std::vector<RowQuantArgs>& jobs);
bool rowquant_compatible(const RowQuantArgs& a, const RowQuantArgs& b);
// 0: no fused kernel covers `a`; 1: per-group kernel (k_group); 2: row kernel (k_row); 3: scalar convolution-row
// kernel (k_conv); 4: vectorised convolution-row kernel (k_convv)
int rowquant_kind(const RowQuantArgs& a);
// derived parameters -> float16 scales and 4-bit packed zero points (either output may be NULL)
void launch_pack_params(vf_ctx* ctx, const double* d_scales, const int64_t* d_zps, int64_t units,
                        uint16_t* scales_f16, uint8_t* zps_u4);

}  // namespace vf
