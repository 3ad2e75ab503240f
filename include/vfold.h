/*
 * vfold.h — C ABI of the B200 constant-folding library (libvfold.so).
 *
 * The library is a drop-in for the data path behind the NPU compiler's
 *   Const::ContentAttr::fold()  +  Const::Content::copyTo()
 * (src/vpux_compiler/src/dialect/const/attributes/content.cpp:371-397,
 *  src/vpux_compiler/src/dialect/const/utils/content.cpp:161-184)
 * and for VPU::NCESparsity::getWeightsTable()
 * (src/vpux_compiler/src/dialect/VPU/utils/nce_sparsity.cpp:171-231).
 *
 * Conventions
 *  - Plain C: POD structs, raw pointers and sizes. No exceptions cross the ABI.
 *  - Every function returns VF_OK (0) or a negative vf_status and, when `err`
 *    is non-NULL, writes a NUL-terminated message into (err, errlen).
 *    Each reference VPUX_THROW on this path maps to one status code; the
 *    predicate is checked on the host before anything is launched.
 *  - Input buffers are borrowed for the duration of the call; outputs are
 *    written into caller-owned memory (host, pinned host, or device memory
 *    of the context's device). The library owns only its streams and its
 *    scratch pool.
 *  - All entry points are thread-safe and re-entrant per context; calls on
 *    one context are serialised on that context's stream.
 *  - There is no CPU fallback: without a CUDA device vf_ctx_create fails.
 */
#ifndef VFOLD_H_
#define VFOLD_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define VF_MAX_RANK 6
#define VF_ABI_VERSION 1

/* ------------------------------------------------------------------ */
/* status codes                                                        */
/* ------------------------------------------------------------------ */
typedef enum vf_status {
    VF_OK = 0,
    VF_ERR_INVALID_ARG = -1,      /* NULL pointer, bad rank, bad enum value                            */
    VF_ERR_UNSUPPORTED = -2,      /* reference throws "Unsupported ..." for this type/shape            */
    VF_ERR_SHAPE = -3,            /* shape / size / params-count mismatch                              */
    VF_ERR_NOT_QUANTIZED = -4,    /* Dequantize on a non-quantized type (dequantize.cpp:43-44)         */
    VF_ERR_ZERO_POINTS = -5,      /* "Not all zero-points are equal" (sparsity.cpp:19-23,
                                     quantization.cpp:197-198)                                         */
    VF_ERR_SPLAT = -6,            /* BitPack on splat input (bit_pack.cpp:133)                         */
    VF_ERR_ODD_COUNT = -7,        /* BitPack on odd element count (bit_pack.cpp:137)                   */
    VF_ERR_POSITION = -8,         /* more than one LAST transformation (content.cpp:585-588)           */
    VF_ERR_CHECKED_CAST = -9,     /* checked_cast range failure during element conversion
                                     (checked_cast.hpp:106-117); reported after the kernels ran        */
    VF_ERR_BUFFER_TOO_SMALL = -10,/* copyTo destination smaller than required (content.cpp:172-174)    */
    VF_ERR_ALIGNMENT = -11,       /* weights-table pointer not 16-aligned (nce_sparsity.cpp:216-222)   */
    VF_ERR_RANGE = -12,           /* post-shift needed / rescaled bias outside int32
                                     (quantization.cpp:429-432, nce_sparsity.cpp:340-345)              */
    VF_ERR_QUANT_RANGE = -13,     /* calcScaleAndZeroPoint failure (quantization.cpp:612-625)          */
    VF_ERR_NOT_NORMAL = -14,      /* ScalarMultInverse of a non-normal float (inverse.cpp:58-59)       */
    VF_ERR_NAN = -15,             /* Quantize met a NaN: the reference converts it to an integer, which
                                     is undefined (quantize.cpp:91-106); reported after the kernels ran   */
    VF_ERR_CUDA = -20,            /* a CUDA runtime call failed; message carries cudaGetErrorString    */
    VF_ERR_NO_DEVICE = -21,       /* no usable CUDA device                                             */
    VF_ERR_OOM = -22,             /* device or pinned allocation failed                                */
    VF_ERR_CAPACITY = -23,        /* fixed-capacity entry point: request exceeds the built-in maximum  */
    VF_ERR_NOT_RUN = -24          /* a job of a batch that an earlier job's failure kept from running  */
} vf_status;

/* ------------------------------------------------------------------ */
/* element types                                                       */
/* ------------------------------------------------------------------ */
typedef enum vf_dtype {
    VF_DT_INVALID = 0,
    VF_DT_F32 = 1,
    VF_DT_F16 = 2,
    VF_DT_BF16 = 3,
    VF_DT_F64 = 4,
    VF_DT_I8 = 5,
    VF_DT_U8 = 6,
    VF_DT_I16 = 7,
    VF_DT_U16 = 8,
    VF_DT_I32 = 9,
    VF_DT_U32 = 10,
    VF_DT_I64 = 11,
    VF_DT_U64 = 12,
    VF_DT_I4 = 13,
    VF_DT_U4 = 14,
    VF_DT_I1 = 15, /* 1-bit, signless; sparsity maps */
    VF_DT_F8E4M3FN = 16, /* vpux::type::float8_e4m3 (no infinities) */
    VF_DT_F8E5M2 = 17    /* vpux::type::float8_e5m2 */
} vf_dtype;

typedef enum vf_elem_kind {
    VF_ELEM_PLAIN = 0,         /* builtin integer / float type                                   */
    VF_ELEM_QUANT_UNIFORM = 1, /* !quant.uniform<storage:expressed, scale:zp>                    */
    VF_ELEM_QUANT_PER_AXIS = 2 /* !quant.uniform<storage:expressed:axis, {s0:z0, s1:z1, ...}>    */
} vf_elem_kind;

/* Mirror of an MLIR element type as the Const dialect sees it. For quantized
 * kinds `dtype` is the (sign-normalised) storage type, `qmin/qmax` are
 * storageTypeMin/Max, and scales/zps point at `nparams` host values that the
 * caller keeps alive for the call. */
typedef struct vf_elem_type {
    int32_t kind;      /* vf_elem_kind */
    int32_t dtype;     /* vf_dtype: plain type, or quantized storage type */
    int32_t expressed; /* vf_dtype of the expressed float type (quantized kinds) */
    int32_t axis;      /* quantized (logical) dimension for PER_AXIS, else -1 */
    int64_t qmin;
    int64_t qmax;
    int64_t nparams; /* 1 for UNIFORM, size of the quantized dimension for PER_AXIS */
    const double* scales;
    const int64_t* zps;
} vf_elem_type;

/* DimsOrder code as in the reference (core/attributes/dims_order.cpp:38-59):
 * hex digits list the logical dims from the outermost to the innermost memory
 * dim, 1-based. NCHW/OIYX = 0x1234, NHWC/OYXI = 0x1342. 0 means "identity". */
typedef uint32_t vf_dims_order;
#define VF_ORDER_NCHW 0x1234u
#define VF_ORDER_NHWC 0x1342u
#define VF_ORDER_OIYX 0x1234u
#define VF_ORDER_OYXI 0x1342u

typedef struct vf_tensor_type {
    vf_elem_type elem;
    int32_t rank;
    vf_dims_order order;
    int64_t shape[VF_MAX_RANK]; /* logical shape */
} vf_tensor_type;

typedef enum vf_mem_kind {
    VF_MEM_HOST = 0,        /* pageable host memory */
    VF_MEM_HOST_PINNED = 1, /* page-locked host memory */
    VF_MEM_DEVICE = 2       /* device memory of the context's device */
} vf_mem_kind;

/* Const::Content as a POD: a typed view over a byte buffer. The logical type
 * (`type`) and the storage element type may differ — CastElemType changes only
 * the former (utils/content.hpp:166-171,348-351). A splat stores one element. */
typedef struct vf_content {
    vf_tensor_type type;
    int32_t storage_dtype; /* vf_dtype of the bytes in `data` */
    int32_t is_splat;
    int32_t mem_kind; /* vf_mem_kind of `data` */
    int32_t reserved;
    const void* data;
    uint64_t nbytes;
} vf_content;

/* ------------------------------------------------------------------ */
/* transformations (#const.* attributes)                               */
/* ------------------------------------------------------------------ */
typedef enum vf_transform_kind {
    VF_T_CAST_ELEM_TYPE = 1,    /* #const.CastElemType     cast_elem_type.cpp:35-37   (elem)        */
    VF_T_CONVERT_ELEM_TYPE = 2, /* #const.ConvertElemType  convert_elem_type.cpp:48-82 (elem)       */
    VF_T_DEQUANTIZE = 3,        /* #const.Dequantize       dequantize.cpp:42-108                    */
    VF_T_QUANTIZE = 4,          /* #const.Quantize         quantize.cpp:108-212        (elem)       */
    VF_T_RESCALE = 5,           /* #const.Rescale          rescale.cpp:67-82           (value)      */
    VF_T_ADD = 6,               /* #const.Add              add.cpp:62-77               (value)      */
    VF_T_RESHAPE = 7,           /* #const.Reshape          reshape.cpp:87-89           (a = shape)  */
    VF_T_REORDER = 8,           /* #const.Reorder          reorder.cpp:79-99           (order)      */
    VF_T_MEM_PERMUTE = 9,       /* #const.MemPermute       mem_permute.cpp:117-122 (order, mem_perm)*/
    VF_T_TRANSPOSE = 10,        /* #const.Transpose        transpose.cpp:96-104        (order)      */
    VF_T_LAYOUT_CAST = 11,      /* #const.LayoutCast       layout_cast.cpp:82-84       (order)      */
    VF_T_PAD_WITH_ZERO = 12,    /* #const.PadWithZero      pad_with_zero.cpp:111-268   (a, b)       */
    VF_T_BIT_PACK = 13,         /* #const.BitPack          bit_pack.cpp:132-154        (width)      */
    VF_T_GET_SPARSITY_MAP = 14, /* #const.GetSparsityMap   get_sparsity_map.cpp:82-119              */
    VF_T_SPARSIFY = 15,         /* #const.Sparsify         sparsify.cpp:163-203 (compress, counts)  */
    VF_T_SUBVIEW = 16,          /* #const.SubView          subview.cpp:390-432 (a = offset, b = shape) */
    VF_T_SWIZZLE_CONSTANT = 17, /* #const.SwizzleConstant  swizzle_transform.cpp:163-215
                                   (a[0] = swizzle key 0..5, a[1] = arch: VF_ARCH_NPU37XX / VF_ARCH_NPU40XX) */
    VF_T_RELOCATE_WEIGHTS_TABLE = 18, /* #const.RelocateWeightsTable relocate_weights_table.cpp:203-292 (relocate) */
    VF_T_REVERSE = 19,            /* #const.Reverse           reverse.cpp:46-105          (a[0] = axis)              */
    VF_T_BROADCAST = 20,          /* #const.Broadcast         broadcast.cpp:66-124        (a[0] = axis, a[1] = value) */
    VF_T_EXPAND_DILATED = 21,     /* #const.ExpandDilated     expand_dilated.cpp:72-131   (a[0], a[1] = dilations Y, X) */
    VF_T_SCALAR_MULT_INVERSE = 22,/* #const.ScalarMultInverse inverse.cpp:40-66                                      */
    VF_T_CHANGE_SHAPE_AND_ELEM_TYPE = 23 /* #const.ChangeShapeAndElemType change_shape_and_elem_type.cpp:62-79
                                            (a = shape, elem) */
} vf_transform_kind;

/* VPU::ArchKind values SwizzleConstant carries (VPU/attributes.td:47-50) */
#define VF_ARCH_NPU37XX 3
#define VF_ARCH_NPU40XX 4

/* Parameters of #const.RelocateWeightsTable (const/attributes.td:697-748). Entry c of `weights_ptr` and of
 * `offsets` describes cluster c: the base address of its weights and the first channel it owns. */
#define VF_MAX_CLUSTERS 8
typedef struct vf_relocate {
    int32_t n_clusters;                   /* 1 .. VF_MAX_CLUSTERS */
    int32_t sparsity_ptr;                 /* sparsityPtr */
    int32_t weights_ptr[VF_MAX_CLUSTERS]; /* weightsPtr */
    int64_t offsets[VF_MAX_CLUSTERS];     /* offsets (channels) */
    int64_t weights_table_size;           /* weightsTableSize, bytes: the first size / 16 rows are patched */
    int64_t weights_elem_bit_size;        /* weightsElemBitSize; 0 = absent */
    const int64_t* num_elems;             /* weightsCompression numElems per channel (host), NULL = no compression */
    int64_t n_num_elems;
    int64_t compression_axis;             /* weightsCompression axis (only the optimiser reads it) */
    int64_t alignment;                    /* weightsCompression alignment; 0 = VPU_WEIGHT_SET_BYTE_ALIGNMENT (16) */
    int64_t channel_offset;               /* channelOffset; 0 = absent */
} vf_relocate;

typedef struct vf_transform {
    int32_t kind;              /* vf_transform_kind */
    int32_t rank;              /* number of valid entries in a[] / b[] */
    vf_elem_type elem;         /* CastElemType / ConvertElemType / Quantize target element type */
    vf_dims_order order;       /* Reorder / Transpose / LayoutCast / MemPermute destination order */
    vf_dims_order mem_perm;    /* MemPermute: permutation of the memory dims */
    int64_t a[VF_MAX_RANK];    /* padBefore | new shape | subview offset */
    int64_t b[VF_MAX_RANK];    /* padAfter  | subview shape */
    double value;              /* Rescale scale | Add bias */
    int32_t width;             /* BitPack width (only 4 is accepted, bit_pack.cpp:25-36) */
    int32_t compress_output;   /* Sparsify<compressOutputType> */
    const int64_t* num_actual; /* Sparsify: optional numActualElements (host), else NULL */
    int64_t n_num_actual;
    vf_relocate relocate;      /* RelocateWeightsTable */
} vf_transform;

/* ------------------------------------------------------------------ */
/* context                                                             */
/* ------------------------------------------------------------------ */
typedef struct vf_ctx vf_ctx;

#define VF_OPT_DISABLE_FUSION 1 /* run vf_quantize_fold through the unfused general kernels (for cross-checks) */
/* Pipelined calls: vf_fold, vf_fold_batch, vf_quantize_fold_batch, vf_weights_table_batch and vf_sparsify_batch
 * calls whose tensors ALL live in device memory return as soon as their work is enqueued on the context's stream,
 * so the host prepares the next batch while the GPU runs this one (what the background folder does with its
 * thread pool, const/utils/constant_folding_in_background.cpp:154-194). Host-side checks (shapes, types, sizes)
 * still fail the call itself; what a kernel reports (a checked_cast, a range without zero, a table range) is
 * returned by the next synchronising call of the context — any call that touches host memory, vf_sparsify,
 * vf_sparsify_noalloc or vf_ctx_synchronize — and the buffers of a deferred call must stay alive until then. A
 * deferred vf_sparsify_batch leaves `data_written` of its jobs at 0; the synchronising call fills them in (the job
 * array must stay alive, too) and reports a compressed set that did not fit its buffer (VF_ERR_BUFFER_TOO_SMALL;
 * nothing is written past a buffer's end). */
#define VF_OPT_ASYNC 2
/* Synchronous calls that take a vf_stats also measure the device time between their first and their last
 * enqueued operation (a pair of CUDA events on the context's stream) into vf_stats.device_ms. */
#define VF_OPT_TIMING 4

typedef struct vf_options {
    uint64_t staging_bytes; /* size of each pinned staging buffer for pageable host I/O (0 = 64 MiB) */
    int32_t flags;          /* bitwise OR of VF_OPT_* */
    int32_t reserved;
} vf_options;

/* Per-call statistics (the reference only logs; this is the hook for metrics). */
typedef struct vf_stats {
    uint64_t bytes_in;        /* bytes of the base content consumed */
    uint64_t bytes_out;       /* bytes written to the destination */
    uint64_t h2d_bytes;
    uint64_t d2h_bytes;
    int32_t kernels_launched; /* library kernels launched by the call */
    int32_t fused;            /* 1 when the call ran on a fused single-pass kernel */
    float device_ms;          /* device time of the call's work on the stream (0 unless the context was created
                                 with VF_OPT_TIMING and the call synchronised) */
    int32_t reserved;
} vf_stats;

int vf_abi_version(void);
const char* vf_status_string(int status);

/* One context = one device + one stream + one scratch pool of its own (the device's default memory pool is
 * not touched). `external_stream` (a cudaStream_t, may be NULL) makes the context enqueue on the caller's
 * stream instead of creating its own. Creation is also where everything vf_sparsify_noalloc needs is set up
 * (see there): create contexts before an embedding process hands the GPU's memory to its own allocator. */
int vf_ctx_create(int device, const vf_options* opts, void* external_stream, vf_ctx** out, char* err, size_t errlen);
void vf_ctx_destroy(vf_ctx* ctx);
int vf_ctx_synchronize(vf_ctx* ctx, char* err, size_t errlen);
void* vf_ctx_stream(vf_ctx* ctx); /* the cudaStream_t the context launches on */
int vf_ctx_device(vf_ctx* ctx);
/* Total kernels launched by this context since creation (monotonic). */
uint64_t vf_ctx_launch_count(vf_ctx* ctx);

/* ------------------------------------------------------------------ */
/* fold                                                                */
/* ------------------------------------------------------------------ */

/* = ContentAttr::inferFinalTypeAndSplat (content.cpp:519-528): runs
 * inferOutputType / inferOutputSplat of every transformation over `base`.
 * `out->elem.scales/zps` are redirected into (scales_buf, zps_buf), which must
 * hold `params_cap` entries each (may be NULL when no per-axis type results).
 * `out_bytes` receives the byte size copyTo() needs (getTotalAllocSize; for
 * Sparsify<false> this is the size of the *uncompressed* type, as in the
 * reference). Pure host function — needs no context. */
int vf_infer_type(const vf_tensor_type* base, int base_is_splat, const vf_transform* t, int n, vf_tensor_type* out,
                  int* out_is_splat, double* scales_buf, int64_t* zps_buf, int64_t params_cap, uint64_t* out_bytes,
                  char* err, size_t errlen);

/* = the rewriting ContentSetup::addTransformation performs whenever a transformation is appended
 * (content.cpp:530-588): t[0..n) are added one at a time — inserted by position requirement, then
 * fuseConsecutiveTransformations, foldTransformation, moveSubViewBefore and moveReshapeBefore
 * (utils/transformations.cpp:385-712) run until none applies. The resulting list folds to the same bytes with
 * fewer passes, and a SubView that reaches the front lets the caller upload only the slab it selects.
 * `out` receives at most `out_cap` entries (n is always enough), `*n_out` their number. Quantization
 * parameters of the resulting entries are stored in (scales_buf, zps_buf), `params_cap` entries each;
 * numActualElements arrays keep pointing at the caller's. Pure host function. The rules that move a
 * transformation into a Fuse work on the parts of a fused constant and live in the host mirrors. */
int vf_optimize_transforms(const vf_tensor_type* base, const vf_transform* t, int n, vf_transform* out, int out_cap,
                           int* n_out, double* scales_buf, int64_t* zps_buf, int64_t params_cap, char* err,
                           size_t errlen);

/* = ContentAttr::fold() followed by Content::copyTo(dst): applies the
 * transformation list to `base` on the GPU and materialises the result in
 * the final *logical* element type into `dst` (mem kind `dst_mem_kind`).
 * `out_type` (optional) receives the folded type, with scales/zps redirected
 * into the optional buffers as in vf_infer_type. `dst_written` (optional)
 * receives the bytes actually produced — for Sparsify this is the compressed
 * size (sparsify.cpp:176-182), which differs from the inferred type's size.
 * Synchronous: returns after `dst` is complete. */
int vf_fold(vf_ctx* ctx, const vf_content* base, const vf_transform* t, int n, void* dst, uint64_t dst_bytes,
            int dst_mem_kind, uint64_t* dst_written, vf_tensor_type* out_type, double* scales_buf, int64_t* zps_buf,
            int64_t params_cap, vf_stats* stats, char* err, size_t errlen);

/* = FuseAttr::transform (attributes/fuse_transform.cpp:31-63): the constants of one NCE operation — weights
 * table, weights, sparsity map, activations, in that order — are folded one after the other and laid end to
 * end in `dst` exactly as copyTo() materialises each (1-bit maps arrive packed eight per byte). A part whose
 * `base` is NULL is absent. `offset` / `bytes` receive where each part landed. */
typedef struct vf_fuse_part {
    const vf_content* base;
    const vf_transform* t;
    int32_t n;
    int32_t reserved;
    uint64_t offset; /* out */
    uint64_t bytes;  /* out */
} vf_fuse_part;
int vf_fuse(vf_ctx* ctx, vf_fuse_part* parts, int nparts, void* dst, uint64_t dst_bytes, int dst_mem_kind,
            uint64_t* dst_written, vf_stats* stats, char* err, size_t errlen);

/* ------------------------------------------------------------------ */
/* range statistics → scale / zero-point                               */
/* ------------------------------------------------------------------ */
typedef enum vf_range_mode {
    VF_RANGE_MINMAX = 0, /* rMin = min(row, 0), rMax = max(row, 0)            (asymmetric)  */
    VF_RANGE_ABSMAX = 1  /* rMin = -absmax(row), rMax = +absmax(row)          (symmetric)   */
} vf_range_mode;

/* How a weight tensor is cut into quantization units:
 *   group_size == 0 : one unit per index of logical dim 0 (per-output-channel);
 *   group_size  > 0 : the tensor is viewed as [rows, cols] row-major and every
 *                     run of `group_size` consecutive elements of a row is a unit
 *                     (the reference expresses this by unrolling the group axis,
 *                     IE/transforms/passes/unroll_group_quantize.cpp). */
typedef struct vf_quant_spec {
    int32_t storage_dtype; /* VF_DT_I8 or VF_DT_U8 (Quantize cannot target sub-byte storage, quantize.cpp:22-27) */
    int32_t range_mode;    /* vf_range_mode */
    int64_t qmin, qmax;    /* storageTypeMin/Max, e.g. -127..127, 0..255, 0..15 */
    int64_t group_size;    /* 0 = per output channel */
    int32_t expressed;     /* vf_dtype of the expressed type recorded in the result type */
    int32_t reserved;
} vf_quant_spec;

/* Per-unit ranges reduced on the GPU, then calcScaleAndZeroPoint
 * (utils/quantization.cpp:574-636) per unit in FP64. Outputs (any may be NULL)
 * are arrays of `n_units` in host or device memory (`out_mem_kind`). */
int vf_row_stats(vf_ctx* ctx, const vf_content* base, const vf_quant_spec* spec, double* scales, int64_t* zps,
                 float* rmin, float* rmax, int64_t n_units, int out_mem_kind, char* err, size_t errlen);

/* Optional side outputs of vf_quantize_fold. Every pointer may be NULL. */
typedef struct vf_quant_outputs {
    int32_t mem_kind;       /* vf_mem_kind of all pointers below */
    int32_t reserved;
    double* scales;         /* [n_units] FP64 scales (what the #const.Quantize type would carry) */
    int64_t* zps;           /* [n_units] zero points */
    uint16_t* scales_f16;   /* [n_units] float16((float)scale) bit patterns */
    uint8_t* zps_u4_packed; /* [ceil(n_units/2)] zero points as 4-bit, low nibble first (BitPack layout) */
    void* dequant;          /* same shape/order as the quantized result: Dequantize + copyTo in `dequant_dtype` */
    int32_t dequant_dtype;  /* VF_DT_F16 / VF_DT_F32 / VF_DT_BF16 */
    int32_t reserved2;
    uint64_t dequant_bytes;
} vf_quant_outputs;

/* Fused weight-quantization fold. Semantically identical to
 *     (scales, zps) = vf_row_stats(base, spec)
 *     vf_fold(base, [Quantize<spec, scales, zps>, t[0], ..., t[n-1]])
 * with t[] drawn from {Reorder, PadWithZero, BitPack}, but reads `base`
 * from HBM exactly once. When `outs->dequant` is set it additionally writes
 *     vf_fold(codes, [CastElemType<q>, Dequantize]) materialised as outs->dequant_dtype. */
int vf_quantize_fold(vf_ctx* ctx, const vf_content* base, const vf_quant_spec* spec, const vf_transform* t, int n,
                     void* dst, uint64_t dst_bytes, int dst_mem_kind, uint64_t* dst_written,
                     const vf_quant_outputs* outs, vf_stats* stats, char* err, size_t errlen);

/* ------------------------------------------------------------------ */
/* sparsity                                                            */
/* ------------------------------------------------------------------ */

/* = countNonSparseElementsPerOC (utils/sparsity.cpp:35-84). `counts` holds
 * shape[0] entries in host or device memory. */
int vf_nnz_per_oc(vf_ctx* ctx, const vf_content* content, int64_t* counts, int out_mem_kind, char* err,
                  size_t errlen);

/* One pass over a folded weight tensor producing what SparsifyWeightsPass
 * (VPU/transforms/passes/sparsify_weights.cpp:143-229) materialises as two
 * constants — [CastElemType<q>, Sparsify<false>] and [CastElemType<q>,
 * GetSparsityMap] — plus the per-OC counts. `data_written` receives the
 * compressed byte size. Any of data/map/counts may be NULL. */
int vf_sparsify(vf_ctx* ctx, const vf_content* content, void* data, uint64_t data_bytes, uint64_t* data_written,
                void* map, uint64_t map_bytes, int64_t* counts, int out_mem_kind, vf_stats* stats, char* err,
                size_t errlen);

/* vf_sparsify over many weight tensors per call: what SparsifyWeightsPass does for every NCE operation of a
 * network (sparsify_weights.cpp:143-229). All tensors share three kernel launches and one read-back of the
 * compressed sizes, so a set of small convolution weights costs microseconds instead of one synchronous
 * round trip per tensor. Per job: any of data/map/counts may be NULL; `data_written` receives the compressed
 * byte size. All outputs of the call live in memory of kind `out_mem_kind`. The first failing job ends the
 * call; its `status` holds the code that is also returned. */
typedef struct vf_sparsify_job {
    vf_content content;
    void* data;
    uint64_t data_bytes;
    void* map;
    uint64_t map_bytes;
    int64_t* counts;
    uint64_t data_written; /* out */
    int32_t status;        /* out */
    int32_t reserved;
} vf_sparsify_job;
int vf_sparsify_batch(vf_ctx* ctx, vf_sparsify_job* jobs, int njobs, int out_mem_kind, vf_stats* stats, char* err,
                      size_t errlen);

/* Allocation-free variant of vf_sparsify. It has no counterpart in the reference: it exists for embedders
 * that forbid device allocations while the compiler runs (for example a serving process whose allocator owns
 * all device memory and hands the fold a fixed arena — a cudaMalloc there fails or stalls every stream).
 * The per-call scratch (per-channel counts and output offsets) lives in a fixed array inside the library
 * image, 1 MiB per GPU that loads the library, so at most VF_NOALLOC_MAX_OC output channels per call;
 * larger requests return VF_ERR_CAPACITY. The call makes no cudaMalloc / cudaFree / memory-pool request.
 *   weights      : [oc][work] elements of `dtype` (i8 / u8 / f16 / bf16 / f32) in DEVICE memory
 *   sparse_value : element value treated as zero (the zero point; 0 for plain types)
 *   data, map, counts : DEVICE memory, laid out exactly as vf_sparsify writes them; each may be NULL
 *   data_written : the compressed size; when the call fails with VF_ERR_BUFFER_TOO_SMALL, the size `data` needs
 * All calls on one GPU share the scratch array and it keeps the previous call's contents (everything read is
 * rewritten first); calls that overlap in time on the same GPU race on it — serialise them.
 * What has to happen once per device happens in vf_ctx_create, not here: the array's device address is looked
 * up and the kernels this call launches are loaded. Loading them lets the CUDA driver allocate device memory
 * (code, and the array itself), so create the context before the embedder's allocator claims the GPU and before
 * any stream capture; after that no call of this function allocates. */
#define VF_NOALLOC_MAX_OC 65536
int vf_sparsify_noalloc(vf_ctx* ctx, const void* weights, int32_t dtype, int64_t oc, int64_t work,
                        int64_t sparse_value, void* data, uint64_t data_bytes, uint64_t* data_written, void* map,
                        uint64_t map_bytes, int64_t* counts, char* err, size_t errlen);

/* ------------------------------------------------------------------ */
/* weights table                                                       */
/* ------------------------------------------------------------------ */
#define VF_SPARSITY_PTR_WHEN_NO_SPARSITY 0xFFFFFF /* nce_sparsity.hpp:33 */

typedef struct vf_weights_table_desc {
    vf_elem_type in_elem;      /* activation input element type  */
    vf_elem_type out_elem;     /* activation output element type */
    vf_elem_type weights_elem; /* kind/dtype == 0/0 (VF_DT_INVALID) means "no weights type" */
    int64_t oc;
    /* pointer columns: either explicit arrays (host, [oc]) or base + step */
    const int32_t* weights_ptrs;
    const int32_t* sparsity_ptrs;
    int32_t weights_ptr_base, weights_ptr_step;
    int32_t sparsity_ptr_base, sparsity_ptr_step; /* base VF_SPARSITY_PTR_WHEN_NO_SPARSITY + step 0 = dense */
    /* sparse layout: when nnz_counts != NULL (mem kind nnz_mem_kind), column 0 is the exclusive prefix sum of
     * align16(nnz * weights element bytes) starting at weights_ptr_base, as RelocateWeightsTable lays compressed
     * weight sets out (relocate_weights_table.cpp:261-270) */
    const int64_t* nnz_counts;
    int32_t nnz_mem_kind;
    int32_t has_bias;
    const float* bias; /* [oc] fp32 (host or device per bias_mem_kind) */
    int32_t bias_mem_kind;
    int32_t bias_is_splat;
    int32_t has_const_scale;
    int32_t reserved;
    double const_scale;
} vf_weights_table_desc;

/* = NCESparsity::getWeightsTable with the NPU37XX converters
 * (NPU37XX/dialect/VPU/impl/nce_sparsity_converters.cpp:14-42).
 * `table` receives oc*4 int32 (host or device). */
int vf_weights_table(vf_ctx* ctx, const vf_weights_table_desc* desc, int32_t* table, int out_mem_kind, char* err,
                     size_t errlen);

/* The weights tables of many NCE operations in one call (one kernel launch for all rows of all tables, one
 * more for all sparse-pointer prefix sums): what createWeightsTableTensor does per operation
 * (VPU/utils/const_utils.cpp:24-41), batched like the constants themselves. `weights_scales` (optional) holds
 * desc.oc FP64 weight scales in memory of kind `scales_mem_kind` and replaces the scale values of
 * desc.weights_elem, which then only describes the type: pass the `scales` output of the tensor's
 * vf_quantize_fold job (device memory) and the table is built without a round trip through the host. */
typedef struct vf_weights_table_job {
    vf_weights_table_desc desc;
    const double* weights_scales;
    int32_t scales_mem_kind; /* vf_mem_kind of weights_scales */
    int32_t status;          /* out */
    int32_t* table;          /* [desc.oc * 4], memory kind = the call's out_mem_kind */
} vf_weights_table_job;
int vf_weights_table_batch(vf_ctx* ctx, vf_weights_table_job* jobs, int njobs, int out_mem_kind, char* err,
                           size_t errlen);

/* ------------------------------------------------------------------ */
/* batches and sharding                                                */
/* ------------------------------------------------------------------ */
typedef struct vf_quant_job {
    vf_content base;
    vf_quant_spec spec;
    const vf_transform* t;
    int32_t n;
    int32_t dst_mem_kind;
    void* dst;
    uint64_t dst_bytes;
    vf_quant_outputs outs;   /* outs.scales in device memory feeds vf_weights_table_batch directly */
    uint64_t dst_written;    /* out */
    int32_t status;          /* out: per-job status */
    int32_t reserved;
} vf_quant_job;

/* Many constants per call: jobs are enqueued back to back on the context's
 * stream (small convolution weights share launches through a row table) and
 * the call synchronises once at the end. Mirrors ConstantFoldingPass folding a
 * batch of constants concurrently (const/passes/constant_folding.cpp:85-159). */
int vf_quantize_fold_batch(vf_ctx* ctx, vf_quant_job* jobs, int njobs, vf_stats* stats, char* err, size_t errlen);

/* = getMaxIntermediateSize (const/passes/constant_folding.cpp:20-31): the largest total allocation size among
 * the base type and the type after each transformation. Pure host function. */
int vf_max_intermediate_size(const vf_tensor_type* base, int base_is_splat, const vf_transform* t, int n,
                             uint64_t* out_bytes, char* err, size_t errlen);

/* One constant of a ConstantFoldingPass run. */
typedef struct vf_fold_job {
    vf_content base;
    const vf_transform* t;
    int32_t n;
    int32_t dst_mem_kind;
    void* dst;
    uint64_t dst_bytes;
    uint64_t dst_written;      /* out: as vf_fold */
    uint64_t max_intermediate; /* out: vf_max_intermediate_size of the job */
    int32_t group;             /* out: VF_GROUP_TINY, VF_GROUP_ALONE, or the index (0, 1, ...) of the group it ran in */
    int32_t status;            /* out: VF_OK once the job has been folded */
} vf_fold_job;
#define VF_GROUP_TINY (-1)
#define VF_GROUP_ALONE (-2)

typedef struct vf_fold_batch_options {
    uint64_t threshold_bytes;      /* the pass's size threshold (0 = 300 MiB, constant_folding.cpp:74) */
    uint64_t tiny_threshold_bytes; /* constants up to this size are folded first (0 = 1024, :83) */
} vf_fold_batch_options;

typedef struct vf_fold_batch_stats {
    int32_t tiny;             /* jobs folded in the first sweep */
    int32_t alone;            /* jobs above the threshold, folded one at a time */
    int32_t groups;           /* groups of jobs folded concurrently */
    int32_t synchronisations; /* host waits of the whole call */
    uint64_t max_group_bytes; /* largest sum of max_intermediate over a group */
} vf_fold_batch_stats;

/* = ConstantFoldingPass::safeRunOnFunc (const/passes/constant_folding.cpp:85-159) over `jobs` in place of the
 * function's const.Declare ops, each folded as foldSingleConstant does (fold + copyTo into the job's
 * destination, :33-43). The schedule is the pass's: constants whose largest intermediate is at most
 * `tiny_threshold_bytes` are folded first; the others are walked in order — one above `threshold_bytes` is
 * folded on its own, the rest are collected into groups while the running sum of their sizes has not passed the
 * threshold (so a group may end one job above it, as in the pass). Where the pass hands a group to its thread
 * pool, the jobs of a group are enqueued back to back on the context's stream here and the host waits once per
 * group: the threshold bounds the device memory in flight exactly as it bounds the pass's host memory.
 * The first failing job ends the call with its status (its index is in `err`); jobs folded before it keep
 * VF_OK, the others VF_ERR_NOT_RUN. A transformation list whose types do not infer fails before any job runs,
 * since the sizes of all constants are computed first. What a kernel reports for a group (a checked_cast ...) is returned when
 * the group is waited for and names the group. */
int vf_fold_batch(vf_ctx* ctx, vf_fold_job* jobs, int njobs, const vf_fold_batch_options* opts,
                  vf_fold_batch_stats* batch_stats, vf_stats* stats, char* err, size_t errlen);

/* Shard planner for multi-GPU runs (pure host). Units are independent, so
 * there is no collective: `mode` 0 assigns whole tensors to ranks by
 * longest-processing-time-first on `bytes[i]`; `mode` 1 cuts every tensor
 * into `world` contiguous output-channel slabs of rows[i] (slab boundaries
 * rounded to `row_align` rows). Output: for tensor i, ranks own rows
 * [row_begin[i*world + r], row_end[i*world + r]). */
int vf_plan_shards(int mode, int world, int64_t ntensors, const uint64_t* bytes, const int64_t* rows,
                   int64_t row_align, int64_t* row_begin, int64_t* row_end, char* err, size_t errlen);

/* ------------------------------------------------------------------ */
/* folding in the background with a cache of folded contents           */
/* ------------------------------------------------------------------ */
/* Replaces Const::BackgroundConstantFolding + Const::ConstantFoldingCache
 * (const/utils/constant_folding_in_background.cpp:17-241, constant_folding_cache.cpp:15-245): requests are
 * queued by the compiler thread, folded by worker threads (each with its own context and stream on the
 * device), and the folded Const::Content objects stay in device memory, keyed by (base content,
 * transformation list). A later fold of the same attribute is a device-to-destination copy.
 *
 * Identity of a base content: `base_id` != 0 is the caller's identity of the bytes (the reference's uniqued
 * attribute pointer); `base_id` == 0 makes the library hash the bytes on the GPU (vf_content_hash), so equal
 * bytes in different buffers share one cache entry. `base->data` is borrowed: it must stay valid until the
 * request has been processed (vf_folder_wait_idle) — the reference's ContentAttr keeps its base alive as well.
 * Transformation lists are copied at the call. */
typedef struct vf_folder vf_folder;

typedef struct vf_folder_options {
    uint64_t memory_limit_bytes; /* memoryUsageLimit: bytes of folded contents the cache may hold (0 = 4 GiB) */
    double clean_threshold;      /* cacheCleanThreshold: a clean-up shrinks the cache to this share of the limit (0 = 0.8) */
    int32_t max_concurrent_tasks;/* worker threads = streams folding at the same time (0 = 2) */
    int32_t collect_statistics;
} vf_folder_options;

/* details::CacheStatistics (constant_folding_cache.hpp:102-124) plus what the log line adds */
typedef struct vf_folder_stats {
    uint64_t added;             /* numElementsAddedToCache */
    uint64_t erased;            /* numElementsErasedFromCache */
    uint64_t hits;              /* numCacheHits */
    uint64_t misses;            /* numCacheMisses */
    uint64_t duplicated;        /* numDuplicatedRequests */
    uint64_t max_queue;         /* maximum number of requests in queue */
    uint64_t max_cache_size;    /* maximum number of elements in cache */
    uint64_t max_memory_used;   /* maximum memory used by cache */
    uint64_t memory_used;       /* current memory used by cache */
    uint64_t cache_size;        /* current number of elements */
    uint64_t failed;            /* requests whose fold raised an error (nothing is cached for them) */
    uint64_t partial;           /* requests folded from a cached prefix (tryFoldingPartially) */
} vf_folder_stats;

int vf_folder_create(int device, const vf_folder_options* opts, vf_folder** out, char* err, size_t errlen);
/* Sends the termination token, waits for the workers (stopFoldingListener) and frees the cache. */
void vf_folder_destroy(vf_folder* folder);

/* FoldingRequest{attr, newTransformation}: `new_index` is the position of the transformation that was just
 * appended to `t` (the request is then tried from the cached content of t[0 .. new_index)), or -1. */
int vf_folder_enqueue(vf_folder* folder, const vf_content* base, uint64_t base_id, const vf_transform* t, int n,
                      int new_index, char* err, size_t errlen);
/* EquivalenceRequest{originalAttr, newAttr}: both lists fold to the same content; a cached result of the
 * original is re-keyed to the new list, otherwise the new list is folded. */
int vf_folder_enqueue_equivalence(vf_folder* folder, const vf_content* base, uint64_t base_id, const vf_transform* t_orig,
                                  int n_orig, const vf_transform* t_new, int n_new, char* err, size_t errlen);
/* Blocks until the queue is empty and no worker is folding (tests use it where the reference's sleep). */
int vf_folder_wait_idle(vf_folder* folder, char* err, size_t errlen);
/* ConstantFoldingCache::hasContent: `*found`; a hit raises the entry's priority (refCount + 1). */
int vf_folder_has_content(vf_folder* folder, const vf_content* base, uint64_t base_id, const vf_transform* t, int n,
                          int* found, char* err, size_t errlen);
/* ContentAttr::fold() + copyTo() through the cache (attributes/content.cpp:371-397): a cached content is
 * copied out (`*from_cache` = 1, its refCount drops by one), anything else is folded now and not cached.
 * Arguments as vf_fold. */
int vf_folder_fold(vf_folder* folder, const vf_content* base, uint64_t base_id, const vf_transform* t, int n, void* dst,
                   uint64_t dst_bytes, int dst_mem_kind, uint64_t* dst_written, vf_tensor_type* out_type,
                   double* scales_buf, int64_t* zps_buf, int64_t params_cap, int* from_cache, char* err, size_t errlen);
/* ConstantFoldingCache::removeContent */
int vf_folder_remove(vf_folder* folder, const vf_content* base, uint64_t base_id, const vf_transform* t, int n,
                     char* err, size_t errlen);
int vf_folder_statistics(vf_folder* folder, vf_folder_stats* out);
/* Message of the last request that failed in a worker (empty if none). */
int vf_folder_last_error(vf_folder* folder, char* buf, size_t buflen);
/* 128-bit hash of a content's storage bytes, computed on the GPU (host memory is uploaded first). The same
 * bytes give the same hash wherever they live and however the buffer is aligned. */
int vf_content_hash(vf_ctx* ctx, const vf_content* content, uint64_t out[2], char* err, size_t errlen);

/* ------------------------------------------------------------------ */
/* synthetic weights (measurement support)                             */
/* ------------------------------------------------------------------ */
typedef struct vf_synth_spec {
    uint64_t seed;
    uint64_t tensor_id;
    int32_t dtype;          /* VF_DT_F32 / VF_DT_F16 / VF_DT_BF16 */
    int32_t reserved;
    float sigma;            /* standard deviation of the bell-shaped base distribution */
    float outlier_mult;     /* elements selected with probability 2^-outlier_log2 are multiplied by this (0 = off) */
    int32_t outlier_log2;
    int32_t mask_zero;      /* 1: zero each element with probability 1/2 ...                          */
    int32_t dense_row_mod;  /* ... except rows whose hash % dense_row_mod == 0 (0 = no dense rows)     */
    int32_t reserved2;
    int64_t row_len;        /* elements per row (for the row hash) */
    uint64_t first_elem;    /* global index of element 0 of this buffer (so slabs re-derive identically) */
} vf_synth_spec;

/* Fills `dst` (device memory) with `count` deterministic pseudo-random
 * weights. The sequence is defined by integer hashing plus one IEEE multiply
 * and one round-to-nearest-even conversion, so a host restatement produces the
 * same bits. */
int vf_synth_fill(vf_ctx* ctx, const vf_synth_spec* spec, void* dst, uint64_t count, char* err, size_t errlen);

#ifdef __cplusplus
}
#endif
#endif /* VFOLD_H_ */
