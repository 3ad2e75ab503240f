"""ctypes mirror of include/vfold.h.

Only POD layouts, enum values and small helpers that build descriptors live
here; the same structures are accepted by libvfold.so (the product) and by the
CPU oracle used in tests, so a test can hand identical inputs to both.
"""
import ctypes as C

import numpy as np

VF_MAX_RANK = 6

# vf_status
VF_OK = 0
VF_ERR_INVALID_ARG = -1
VF_ERR_UNSUPPORTED = -2
VF_ERR_SHAPE = -3
VF_ERR_NOT_QUANTIZED = -4
VF_ERR_ZERO_POINTS = -5
VF_ERR_SPLAT = -6
VF_ERR_ODD_COUNT = -7
VF_ERR_POSITION = -8
VF_ERR_CHECKED_CAST = -9
VF_ERR_BUFFER_TOO_SMALL = -10
VF_ERR_ALIGNMENT = -11
VF_ERR_RANGE = -12
VF_ERR_QUANT_RANGE = -13
VF_ERR_NOT_NORMAL = -14
VF_ERR_NAN = -15
VF_ERR_CUDA = -20
VF_ERR_NO_DEVICE = -21
VF_ERR_OOM = -22
VF_ERR_CAPACITY = -23
VF_ERR_NOT_RUN = -24
VF_GROUP_TINY, VF_GROUP_ALONE = -1, -2

# vf_dtype
(VF_DT_INVALID, VF_DT_F32, VF_DT_F16, VF_DT_BF16, VF_DT_F64, VF_DT_I8, VF_DT_U8, VF_DT_I16, VF_DT_U16, VF_DT_I32,
 VF_DT_U32, VF_DT_I64, VF_DT_U64, VF_DT_I4, VF_DT_U4, VF_DT_I1, VF_DT_F8E4M3FN, VF_DT_F8E5M2) = range(18)

DTYPE_BITS = {
    VF_DT_F32: 32, VF_DT_F16: 16, VF_DT_BF16: 16, VF_DT_F64: 64, VF_DT_I8: 8, VF_DT_U8: 8, VF_DT_I16: 16,
    VF_DT_U16: 16, VF_DT_I32: 32, VF_DT_U32: 32, VF_DT_I64: 64, VF_DT_U64: 64, VF_DT_I4: 4, VF_DT_U4: 4, VF_DT_I1: 1,
    VF_DT_F8E4M3FN: 8, VF_DT_F8E5M2: 8,
}
# numpy carrier for the raw bytes of each dtype (bf16 travels as uint16 bit patterns)
DTYPE_NUMPY = {
    VF_DT_F32: np.float32, VF_DT_F16: np.float16, VF_DT_BF16: np.uint16, VF_DT_F64: np.float64, VF_DT_I8: np.int8,
    VF_DT_U8: np.uint8, VF_DT_I16: np.int16, VF_DT_U16: np.uint16, VF_DT_I32: np.int32, VF_DT_U32: np.uint32,
    VF_DT_I64: np.int64, VF_DT_U64: np.uint64, VF_DT_F8E4M3FN: np.uint8, VF_DT_F8E5M2: np.uint8,
}

VF_ELEM_PLAIN, VF_ELEM_QUANT_UNIFORM, VF_ELEM_QUANT_PER_AXIS = 0, 1, 2
VF_MEM_HOST, VF_MEM_HOST_PINNED, VF_MEM_DEVICE = 0, 1, 2

(VF_T_CAST_ELEM_TYPE, VF_T_CONVERT_ELEM_TYPE, VF_T_DEQUANTIZE, VF_T_QUANTIZE, VF_T_RESCALE, VF_T_ADD, VF_T_RESHAPE,
 VF_T_REORDER, VF_T_MEM_PERMUTE, VF_T_TRANSPOSE, VF_T_LAYOUT_CAST, VF_T_PAD_WITH_ZERO, VF_T_BIT_PACK,
 VF_T_GET_SPARSITY_MAP, VF_T_SPARSIFY, VF_T_SUBVIEW, VF_T_SWIZZLE_CONSTANT, VF_T_RELOCATE_WEIGHTS_TABLE, VF_T_REVERSE,
 VF_T_BROADCAST, VF_T_EXPAND_DILATED, VF_T_SCALAR_MULT_INVERSE, VF_T_CHANGE_SHAPE_AND_ELEM_TYPE) = range(1, 24)
VF_ARCH_NPU37XX, VF_ARCH_NPU40XX = 3, 4

VF_RANGE_MINMAX, VF_RANGE_ABSMAX = 0, 1
VF_SPARSITY_PTR_WHEN_NO_SPARSITY = 0xFFFFFF

ORDER_NCHW = 0x1234
ORDER_NHWC = 0x1342


class ElemType(C.Structure):
    _fields_ = [("kind", C.c_int32), ("dtype", C.c_int32), ("expressed", C.c_int32), ("axis", C.c_int32),
                ("qmin", C.c_int64), ("qmax", C.c_int64), ("nparams", C.c_int64),
                ("scales", C.POINTER(C.c_double)), ("zps", C.POINTER(C.c_int64))]


class TensorType(C.Structure):
    _fields_ = [("elem", ElemType), ("rank", C.c_int32), ("order", C.c_uint32), ("shape", C.c_int64 * VF_MAX_RANK)]


class Content(C.Structure):
    _fields_ = [("type", TensorType), ("storage_dtype", C.c_int32), ("is_splat", C.c_int32), ("mem_kind", C.c_int32),
                ("reserved", C.c_int32), ("data", C.c_void_p), ("nbytes", C.c_uint64)]


VF_MAX_CLUSTERS = 8


class Relocate(C.Structure):
    _fields_ = [("n_clusters", C.c_int32), ("sparsity_ptr", C.c_int32), ("weights_ptr", C.c_int32 * VF_MAX_CLUSTERS),
                ("offsets", C.c_int64 * VF_MAX_CLUSTERS), ("weights_table_size", C.c_int64),
                ("weights_elem_bit_size", C.c_int64), ("num_elems", C.POINTER(C.c_int64)), ("n_num_elems", C.c_int64),
                ("compression_axis", C.c_int64), ("alignment", C.c_int64), ("channel_offset", C.c_int64)]


class Transform(C.Structure):
    _fields_ = [("kind", C.c_int32), ("rank", C.c_int32), ("elem", ElemType), ("order", C.c_uint32),
                ("mem_perm", C.c_uint32), ("a", C.c_int64 * VF_MAX_RANK), ("b", C.c_int64 * VF_MAX_RANK),
                ("value", C.c_double), ("width", C.c_int32), ("compress_output", C.c_int32),
                ("num_actual", C.POINTER(C.c_int64)), ("n_num_actual", C.c_int64), ("relocate", Relocate)]


class Options(C.Structure):
    _fields_ = [("staging_bytes", C.c_uint64), ("flags", C.c_int32), ("reserved", C.c_int32)]


class Stats(C.Structure):
    _fields_ = [("bytes_in", C.c_uint64), ("bytes_out", C.c_uint64), ("h2d_bytes", C.c_uint64),
                ("d2h_bytes", C.c_uint64), ("kernels_launched", C.c_int32), ("fused", C.c_int32),
                ("device_ms", C.c_float), ("reserved", C.c_int32)]


class QuantSpec(C.Structure):
    _fields_ = [("storage_dtype", C.c_int32), ("range_mode", C.c_int32), ("qmin", C.c_int64), ("qmax", C.c_int64),
                ("group_size", C.c_int64), ("expressed", C.c_int32), ("reserved", C.c_int32)]


class QuantOutputs(C.Structure):
    _fields_ = [("mem_kind", C.c_int32), ("reserved", C.c_int32), ("scales", C.c_void_p), ("zps", C.c_void_p),
                ("scales_f16", C.c_void_p), ("zps_u4_packed", C.c_void_p), ("dequant", C.c_void_p),
                ("dequant_dtype", C.c_int32), ("reserved2", C.c_int32), ("dequant_bytes", C.c_uint64)]


class WeightsTableDesc(C.Structure):
    _fields_ = [("in_elem", ElemType), ("out_elem", ElemType), ("weights_elem", ElemType), ("oc", C.c_int64),
                ("weights_ptrs", C.POINTER(C.c_int32)), ("sparsity_ptrs", C.POINTER(C.c_int32)),
                ("weights_ptr_base", C.c_int32), ("weights_ptr_step", C.c_int32),
                ("sparsity_ptr_base", C.c_int32), ("sparsity_ptr_step", C.c_int32),
                ("nnz_counts", C.c_void_p), ("nnz_mem_kind", C.c_int32), ("has_bias", C.c_int32),
                ("bias", C.c_void_p), ("bias_mem_kind", C.c_int32), ("bias_is_splat", C.c_int32),
                ("has_const_scale", C.c_int32), ("reserved", C.c_int32), ("const_scale", C.c_double)]


class QuantJob(C.Structure):
    _fields_ = [("base", Content), ("spec", QuantSpec), ("t", C.POINTER(Transform)), ("n", C.c_int32),
                ("dst_mem_kind", C.c_int32), ("dst", C.c_void_p), ("dst_bytes", C.c_uint64), ("outs", QuantOutputs),
                ("dst_written", C.c_uint64), ("status", C.c_int32), ("reserved", C.c_int32)]


class FoldJob(C.Structure):
    _fields_ = [("base", Content), ("t", C.POINTER(Transform)), ("n", C.c_int32), ("dst_mem_kind", C.c_int32),
                ("dst", C.c_void_p), ("dst_bytes", C.c_uint64), ("dst_written", C.c_uint64),
                ("max_intermediate", C.c_uint64), ("group", C.c_int32), ("status", C.c_int32)]


class FoldBatchOptions(C.Structure):
    _fields_ = [("threshold_bytes", C.c_uint64), ("tiny_threshold_bytes", C.c_uint64)]


class FoldBatchStats(C.Structure):
    _fields_ = [("tiny", C.c_int32), ("alone", C.c_int32), ("groups", C.c_int32), ("synchronisations", C.c_int32),
                ("max_group_bytes", C.c_uint64)]


class WeightsTableJob(C.Structure):
    _fields_ = [("desc", WeightsTableDesc), ("weights_scales", C.c_void_p), ("scales_mem_kind", C.c_int32),
                ("status", C.c_int32), ("table", C.c_void_p)]


class SparsifyJob(C.Structure):
    _fields_ = [("content", Content), ("data", C.c_void_p), ("data_bytes", C.c_uint64), ("map", C.c_void_p),
                ("map_bytes", C.c_uint64), ("counts", C.c_void_p), ("data_written", C.c_uint64),
                ("status", C.c_int32), ("reserved", C.c_int32)]


class FusePart(C.Structure):
    _fields_ = [("base", C.POINTER(Content)), ("t", C.POINTER(Transform)), ("n", C.c_int32), ("reserved", C.c_int32),
                ("offset", C.c_uint64), ("bytes", C.c_uint64)]


class SynthSpec(C.Structure):
    _fields_ = [("seed", C.c_uint64), ("tensor_id", C.c_uint64), ("dtype", C.c_int32), ("reserved", C.c_int32),
                ("sigma", C.c_float), ("outlier_mult", C.c_float), ("outlier_log2", C.c_int32),
                ("mask_zero", C.c_int32), ("dense_row_mod", C.c_int32), ("reserved2", C.c_int32),
                ("row_len", C.c_int64), ("first_elem", C.c_uint64)]


# ----------------------------------------------------------------------------------------------------
# Python-side type objects. They own the numpy arrays the POD structs point into.
# ----------------------------------------------------------------------------------------------------
class Elem:
    """Element type: plain dtype, !quant.uniform, or per-axis !quant.uniform."""

    def __init__(self, dtype, kind=VF_ELEM_PLAIN, expressed=VF_DT_INVALID, axis=-1, qmin=0, qmax=0, scales=None,
                 zps=None):
        self.kind, self.dtype, self.expressed, self.axis = int(kind), int(dtype), int(expressed), int(axis)
        self.qmin, self.qmax = int(qmin), int(qmax)
        self.scales = None if scales is None else np.ascontiguousarray(scales, dtype=np.float64).reshape(-1)
        self.zps = None if zps is None else np.ascontiguousarray(zps, dtype=np.int64).reshape(-1)

    @staticmethod
    def plain(dtype):
        return Elem(dtype)

    @staticmethod
    def uniform(storage, expressed, scale, zp, qmin, qmax):
        return Elem(storage, VF_ELEM_QUANT_UNIFORM, expressed, -1, qmin, qmax, [scale], [zp])

    @staticmethod
    def per_axis(storage, expressed, scales, zps, axis, qmin, qmax):
        return Elem(storage, VF_ELEM_QUANT_PER_AXIS, expressed, axis, qmin, qmax, scales, zps)

    @property
    def quantized(self):
        return self.kind != VF_ELEM_PLAIN

    def pod(self):
        e = ElemType()
        e.kind, e.dtype, e.expressed, e.axis = self.kind, self.dtype, self.expressed, self.axis
        e.qmin, e.qmax = self.qmin, self.qmax
        if self.scales is not None:
            e.nparams = len(self.scales)
            e.scales = self.scales.ctypes.data_as(C.POINTER(C.c_double))
            e.zps = self.zps.ctypes.data_as(C.POINTER(C.c_int64))
        return e

    @staticmethod
    def from_pod(e):
        if e.kind == VF_ELEM_PLAIN:
            return Elem(e.dtype)
        n = int(e.nparams)
        return Elem(e.dtype, e.kind, e.expressed, e.axis, e.qmin, e.qmax, np.ctypeslib.as_array(e.scales, (n,)).copy(),
                    np.ctypeslib.as_array(e.zps, (n,)).copy())

    def __eq__(self, o):
        if not isinstance(o, Elem):
            return NotImplemented
        same = (self.kind, self.dtype, self.qmin, self.qmax) == (o.kind, o.dtype, o.qmin, o.qmax)
        if not same:
            return False
        if self.kind == VF_ELEM_PLAIN:
            return True
        return (self.expressed == o.expressed and self.axis == o.axis and np.array_equal(self.scales, o.scales)
                and np.array_equal(self.zps, o.zps))

    def __repr__(self):
        if self.kind == VF_ELEM_PLAIN:
            return f"Elem(dt={self.dtype})"
        return (f"Elem(q{self.kind} dt={self.dtype}:{self.expressed} axis={self.axis} [{self.qmin},{self.qmax}] "
                f"scales={self.scales} zps={self.zps})")


def identity_order(rank):
    code = 0
    for i in range(rank):
        code = (code << 4) | (i + 1)
    return code


class TType:
    """Tensor type: logical shape + element type + DimsOrder code."""

    def __init__(self, shape, elem, order=0):
        self.shape = [int(s) for s in shape]
        self.elem = elem if isinstance(elem, Elem) else Elem(elem)
        self.order = int(order) if order else identity_order(len(self.shape))

    def pod(self):
        t = TensorType()
        t.elem = self.elem.pod()
        t.rank = len(self.shape)
        t.order = self.order
        for i, s in enumerate(self.shape):
            t.shape[i] = s
        return t

    @staticmethod
    def from_pod(t):
        return TType([t.shape[i] for i in range(t.rank)], Elem.from_pod(t.elem), t.order)

    @property
    def numel(self):
        return int(np.prod(self.shape, dtype=np.int64))

    def nbytes(self):
        return (self.numel * DTYPE_BITS[self.elem.dtype] + 7) // 8

    def __eq__(self, o):
        return isinstance(o, TType) and self.shape == o.shape and self.elem == o.elem and self.order == o.order

    def __repr__(self):
        return f"TType({self.shape}, {self.elem}, order={self.order:#x})"


def make_content(ttype, array, storage_dtype=None, is_splat=False, mem_kind=VF_MEM_HOST, ptr=None, nbytes=None):
    """Build a vf_content over a numpy array (host) or a raw pointer (device). Returns (pod, keepalive)."""
    c = Content()
    pod_t = ttype.pod()
    c.type = pod_t
    c.storage_dtype = int(storage_dtype if storage_dtype is not None else ttype.elem.dtype)
    c.is_splat = 1 if is_splat else 0
    c.mem_kind = mem_kind
    keep = [ttype, pod_t]
    if ptr is not None:
        c.data = ptr
        c.nbytes = int(nbytes)
    else:
        arr = np.ascontiguousarray(array)
        keep.append(arr)
        c.data = arr.ctypes.data
        c.nbytes = arr.nbytes
    return c, keep


def make_transforms(items):
    """items: list of Transform → contiguous ctypes array."""
    arr = (Transform * max(1, len(items)))()
    for i, t in enumerate(items):
        arr[i] = t
    return arr


class FolderOptions(C.Structure):
    _fields_ = [("memory_limit_bytes", C.c_uint64), ("clean_threshold", C.c_double), ("max_concurrent_tasks", C.c_int32),
                ("collect_statistics", C.c_int32)]


class FolderStats(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("added", "erased", "hits", "misses", "duplicated", "max_queue", "max_cache_size",
                                          "max_memory_used", "memory_used", "cache_size", "failed", "partial")]
