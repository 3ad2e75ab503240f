"""Host-side mirror of the reference's Const dialect builder API.

`ContentSetup` collects a transformation list with the same method names and
ordering rules as the reference's `Const::ContentSetup`
(src/vpux_compiler/include/vpux/compiler/dialect/const/attributes/content.hpp:103-134,
insertion rules src/vpux_compiler/src/dialect/const/attributes/content.cpp:530-588);
`ContentAttr.fold()` hands base + list to a backend (`vpux_plugin_b200.lib.Library`
for the GPU product) and returns the materialised bytes, i.e. fold() + copyTo().
"""
import ctypes as C

import numpy as np

from . import abi
from .abi import Elem, TType, Transform

_NONE, _PREFERRED_LAST, _LAST = 0, 1, 2


def _position(kind):
    # attr_interfaces.hpp:24-28; BitPack is LAST (bit_pack.cpp:160-162), Sparsify / GetSparsityMap are
    # PREFERRED_LAST (sparsify.cpp:209-211, get_sparsity_map.cpp:125-127)
    if kind in (abi.VF_T_BIT_PACK, abi.VF_T_SWIZZLE_CONSTANT):  # swizzle_transform.cpp:221-223
        return _LAST
    if kind in (abi.VF_T_SPARSIFY, abi.VF_T_GET_SPARSITY_MAP):
        return _PREFERRED_LAST
    return _NONE


class ContentSetup:
    def __init__(self, base_type, _items=None):
        self.base_type = base_type
        self._items = list(_items or [])  # (Transform, keepalive)

    def clone(self):
        return ContentSetup(self.base_type, self._items)

    # -- insertion ---------------------------------------------------------------------------------
    def _add(self, t, keep=None):
        new = self.clone()
        pos = len(new._items)
        p = _position(t.kind)
        # upper_bound on the position requirement keeps [NONE..., PREFERRED_LAST..., LAST...] stable
        for i, (u, _) in enumerate(new._items):
            if _position(u.kind) > p:
                pos = i
                break
        new._items.insert(pos, (t, keep))
        if len(new._items) >= 2 and _position(new._items[-2][0].kind) == _LAST:
            raise ValueError("At most 1 attribute with LAST requirement allowed!")
        return new

    @staticmethod
    def _t(kind):
        t = Transform()
        t.kind = kind
        return t

    def _with_elem(self, kind, elem):
        elem = elem if isinstance(elem, Elem) else Elem(elem)
        t = self._t(kind)
        t.elem = elem.pod()
        return self._add(t, elem)

    # -- the reference's builder methods ----------------------------------------------------------
    def castElemType(self, elem):
        return self._with_elem(abi.VF_T_CAST_ELEM_TYPE, elem)

    def convertElemType(self, elem):
        return self._with_elem(abi.VF_T_CONVERT_ELEM_TYPE, elem)

    def quantize(self, elem):
        return self._with_elem(abi.VF_T_QUANTIZE, elem)

    def dequantize(self):
        return self._add(self._t(abi.VF_T_DEQUANTIZE))

    def rescale(self, scale):
        t = self._t(abi.VF_T_RESCALE)
        t.value = float(scale)
        return self._add(t)

    def add(self, bias):
        t = self._t(abi.VF_T_ADD)
        t.value = float(bias)
        return self._add(t)

    def reshape(self, shape):
        t = self._t(abi.VF_T_RESHAPE)
        t.rank = len(shape)
        for i, s in enumerate(shape):
            t.a[i] = int(s)
        return self._add(t)

    def reorder(self, order):
        t = self._t(abi.VF_T_REORDER)
        t.order = int(order)
        return self._add(t)

    def transpose(self, order):
        t = self._t(abi.VF_T_TRANSPOSE)
        t.order = int(order)
        return self._add(t)

    def memPermute(self, dst_order, mem_perm):
        t = self._t(abi.VF_T_MEM_PERMUTE)
        t.order = int(dst_order)
        t.mem_perm = int(mem_perm)
        return self._add(t)

    def layoutCast(self, order):
        t = self._t(abi.VF_T_LAYOUT_CAST)
        t.order = int(order)
        return self._add(t)

    def padWithZero(self, pad_before, pad_after):
        if len(pad_before) != len(pad_after):
            raise ValueError("Got non consistent 'padBefore' and 'padAfter' values in 'PadWithZeroAttr'")
        t = self._t(abi.VF_T_PAD_WITH_ZERO)
        t.rank = len(pad_before)
        for i, (b, a) in enumerate(zip(pad_before, pad_after)):
            t.a[i], t.b[i] = int(b), int(a)
        return self._add(t)

    def subview(self, offset, shape):
        t = self._t(abi.VF_T_SUBVIEW)
        t.rank = len(offset)
        for i, (o, s) in enumerate(zip(offset, shape)):
            t.a[i], t.b[i] = int(o), int(s)
        return self._add(t)

    def bitPack(self, width):
        t = self._t(abi.VF_T_BIT_PACK)
        t.width = int(width)
        return self._add(t)

    def swizzleConstant(self, swizzle_key, arch):
        t = self._t(abi.VF_T_SWIZZLE_CONSTANT)
        t.rank = 2
        t.a[0], t.a[1] = int(swizzle_key), int(arch)
        return self._add(t)

    def relocateWeightsTablePointers(self, weights_ptr, sparsity_ptr, offsets, weights_table_size,
                                     weights_elem_bit_size=0, weights_compression=None, channel_offset=0):
        """content_setup.cpp:82-92. `weights_compression` is None or a dict {"axis", "numElems", "alignment"}
        (VPUIP::SparsityCompressionAttr; alignment 0 / missing = the 16-byte default)."""
        if len(weights_ptr) != len(offsets) or not 1 <= len(offsets) <= abi.VF_MAX_CLUSTERS:
            raise ValueError("weightsPtr and offsets need one entry per cluster (1..%d)" % abi.VF_MAX_CLUSTERS)
        t = self._t(abi.VF_T_RELOCATE_WEIGHTS_TABLE)
        r = t.relocate
        r.n_clusters = len(offsets)
        r.sparsity_ptr = int(sparsity_ptr)
        for i, (w, o) in enumerate(zip(weights_ptr, offsets)):
            r.weights_ptr[i], r.offsets[i] = int(w), int(o)
        r.weights_table_size = int(weights_table_size)
        r.weights_elem_bit_size = int(weights_elem_bit_size or 0)
        r.channel_offset = int(channel_offset or 0)
        keep = None
        if weights_compression is not None:
            keep = np.ascontiguousarray(weights_compression["numElems"], dtype=np.int64)
            r.num_elems = keep.ctypes.data_as(C.POINTER(C.c_int64))
            r.n_num_elems = len(keep)
            r.compression_axis = int(weights_compression.get("axis", 0))
            r.alignment = int(weights_compression.get("alignment", 0) or 0)
        return self._add(t, keep)

    def reverse(self, axis):
        t = self._t(abi.VF_T_REVERSE)
        t.rank = 1
        t.a[0] = int(axis)
        return self._add(t)

    def broadcast(self, axis, value):
        t = self._t(abi.VF_T_BROADCAST)
        t.rank = 2
        t.a[0], t.a[1] = int(axis), int(value)
        return self._add(t)

    def expandDilated(self, dilations):
        t = self._t(abi.VF_T_EXPAND_DILATED)
        t.rank = 2
        t.a[0], t.a[1] = int(dilations[0]), int(dilations[1])
        return self._add(t)

    def scalarMultInverse(self):
        return self._add(self._t(abi.VF_T_SCALAR_MULT_INVERSE))

    def changeShapeAndElemType(self, shape, elem):
        elem = elem if isinstance(elem, Elem) else Elem(elem)
        t = self._t(abi.VF_T_CHANGE_SHAPE_AND_ELEM_TYPE)
        t.rank = len(shape)
        for i, s in enumerate(shape):
            t.a[i] = int(s)
        t.elem = elem.pod()
        return self._add(t, elem)

    def getSparsityMap(self):
        return self._add(self._t(abi.VF_T_GET_SPARSITY_MAP))

    def sparsify(self, compress_output_type, num_actual_elements=None):
        t = self._t(abi.VF_T_SPARSIFY)
        t.compress_output = 1 if compress_output_type else 0
        keep = None
        if num_actual_elements is not None:
            keep = np.ascontiguousarray(num_actual_elements, dtype=np.int64)
            if (keep < 0).any():
                raise ValueError("Got negative elem number value in 'numActualElements' for 'SparsifyAttr'")
            t.num_actual = keep.ctypes.data_as(C.POINTER(C.c_int64))
            t.n_num_actual = len(keep)
        return self._add(t, keep)

    def optimized(self):
        """The list after the rewriting the reference applies on every insertion (content.cpp:530-588: fuse
        consecutive transformations, drop no-op reorders, move SubView / Reshape towards the front). The builder
        methods above keep the list exactly as given so that tests control it; call this to get the list the
        reference's ContentSetup would hold."""
        from . import lib
        tr, n = self.transforms()
        out, n_out, keep = lib.optimize_transforms(self.base_type, tr, n)
        items = []
        for i in range(n_out):
            t = Transform()
            C.memmove(C.byref(t), C.byref(out[i]), C.sizeof(Transform))
            items.append((t, keep if i == 0 else None))
        res = ContentSetup(self.base_type, items)
        res._keep_src = [k for _, k in self._items]  # numActualElements arrays are shared with this setup
        return res

    # -- access ------------------------------------------------------------------------------------
    def transforms(self):
        return abi.make_transforms([t for t, _ in self._items]), len(self._items)

    def names(self):
        return [t.kind for t, _ in self._items]


class Folded:
    """Result of fold() + copyTo(): the folded type and the materialised bytes."""

    def __init__(self, ttype, is_splat, raw, written):
        self.type, self.is_splat, self.raw, self.written = ttype, is_splat, raw, written

    def bytes(self):
        return self.raw[:self.written]

    def values(self, np_dtype=None):
        dt = np_dtype or abi.DTYPE_NUMPY[self.type.elem.dtype]
        return self.bytes().view(dt)


class ContentAttr:
    """base content + transformation list, as Const::ContentAttr (attributes/content.hpp)."""

    def __init__(self, base, base_type, setup=None, is_splat=False, storage_dtype=None):
        self.base = np.ascontiguousarray(base)
        self.base_type = base_type
        self.setup = setup if setup is not None else ContentSetup(base_type)
        self.is_splat = bool(is_splat)
        self.storage_dtype = storage_dtype if storage_dtype is not None else base_type.elem.dtype

    def infer(self, backend):
        tr, n = self.setup.transforms()
        return backend.infer_type(self.base_type, self.is_splat, tr, n)

    def fold(self, backend, dst_bytes=None):
        tr, n = self.setup.transforms()
        content, keep = abi.make_content(self.base_type, self.base, self.storage_dtype, self.is_splat)
        out_type, out_splat, need = backend.infer_type(self.base_type, self.is_splat, tr, n)
        cap = int(dst_bytes if dst_bytes is not None else need)
        dst = np.zeros(max(cap, 1), dtype=np.uint8)
        written, ftype = backend.fold(content, tr, n, dst, cap)
        del keep
        return Folded(ftype, out_splat, dst, written)


def foldConstants(library, attrs, threshold_bytes=0, tiny_threshold_bytes=0):
    """ConstantFoldingPass over a list of ContentAttr (const/passes/constant_folding.cpp:85-159): every constant
    is folded into a host buffer of its own with the pass's schedule (the small ones first, the large ones in
    groups under the size threshold). Returns ([Folded], abi.FoldBatchStats, [group of each constant])."""
    jobs = (abi.FoldJob * len(attrs))()
    keep, outs, types = [], [], []
    for j, a in enumerate(attrs):
        tr, n = a.setup.transforms()
        content, k = abi.make_content(a.base_type, a.base, a.storage_dtype, a.is_splat)
        out_type, out_splat, need = library.infer_type(a.base_type, a.is_splat, tr, n)
        dst = np.zeros(max(int(need), 1), dtype=np.uint8)
        jobs[j].base, jobs[j].t, jobs[j].n = content, tr, n
        jobs[j].dst_mem_kind, jobs[j].dst, jobs[j].dst_bytes = abi.VF_MEM_HOST, dst.ctypes.data, int(need)
        keep.append((tr, k, content))
        outs.append(dst)
        types.append((out_type, out_splat))
    stats = library.fold_batch(jobs, threshold_bytes, tiny_threshold_bytes)
    folded = [Folded(t, s, d, int(jobs[j].dst_written)) for j, ((t, s), d) in enumerate(zip(types, outs))]
    del keep
    return folded, stats, [int(jobs[j].group) for j in range(len(attrs))]


class FusedConstant:
    """Const::FuseAttr (attributes/fuse_transform.cpp:31-63) with the list that follows it: the constants of one
    NCE operation — weights table, weights, sparsity map, activations — folded one after the other into one flat
    buffer of `fused_type`. `subview` and `relocateWeightsTablePointers` apply the rules that move a following
    transformation into the Fuse (moveTransformationIntoFuse, utils/transformations.cpp:831-862); what cannot
    be moved stays behind the Fuse and is applied to the fused bytes."""

    def __init__(self, fused_type, weightsTable=None, weights=None, sparsity=None, activations=None, trailing=None):
        self.fused_type = fused_type
        self.weightsTable, self.weights, self.sparsity, self.activations = weightsTable, weights, sparsity, activations
        self.trailing = trailing if trailing is not None else ContentSetup(fused_type)

    def parts(self):
        return [self.weightsTable, self.weights, self.sparsity, self.activations]

    @staticmethod
    def _type_of(attr):
        from . import lib
        tr, n = attr.setup.transforms()
        t, _, nbytes = lib.infer_type(attr.base_type, attr.is_splat, tr, n)
        return t, int(nbytes)

    @staticmethod
    def _with(attr, setup):
        return ContentAttr(attr.base, attr.base_type, setup.optimized(), attr.is_splat, attr.storage_dtype)

    # -- moveTransformationIntoFuse: RelocateWeightsTable joins the weights table's own list (:842-846) ----------
    def relocateWeightsTablePointers(self, *args, **kwargs):
        if self.trailing.names() or self.weightsTable is None:
            return self._behind(self.trailing.relocateWeightsTablePointers(*args, **kwargs))
        wt = self._with(self.weightsTable, self.weightsTable.setup.relocateWeightsTablePointers(*args, **kwargs))
        return FusedConstant(self.fused_type, wt, self.weights, self.sparsity, self.activations)

    def _behind(self, trailing):
        return FusedConstant(self.fused_type, self.weightsTable, self.weights, self.sparsity, self.activations, trailing)

    # -- moveSubViewIntoFuse (:687-826) ----------------------------------------------------------------------
    def subview(self, offset, shape):
        offset, shape = [int(v) for v in offset], [int(v) for v in shape]
        fs = list(self.fused_type.shape)
        movable = (not self.trailing.names() and self.sparsity is None and len(fs) == 4 and len(offset) == 4 and
                   len(shape) == 4 and all(fs[d] == 1 and offset[d] == 0 and shape[d] == 1 for d in range(3)))
        if not movable:
            return self._behind(self.trailing.subview(offset, shape))
        elem_bytes = abi.DTYPE_BITS[self.fused_type.elem.dtype] // 8
        sub_start = offset[3] * elem_bytes
        sub_end = sub_start + shape[3] * elem_bytes
        at = 0
        new = []
        for attr in (self.weightsTable, self.weights, self.activations):
            if attr is None:
                new.append(None)
                continue
            moved, at = self._slice_part(attr, at, sub_start, sub_end)
            new.append(moved)
        ft = TType([1, 1, 1, shape[3]], self.fused_type.elem, self.fused_type.order)
        return FusedConstant(ft, new[0], new[1], None, new[2])

    @classmethod
    def _slice_part(cls, attr, c_start, sub_start, sub_end):
        """getNewConstant (:757-805): the part of `attr` inside [sub_start, sub_end) of the fused buffer, as a
        SubView on its own shape plus, where that cannot express it, a flat Reshape + SubView."""
        ctype, cbytes = cls._type_of(attr)
        c_end = c_start + cbytes
        if ctype.elem.quantized:  # sliced quantized axes would no longer match their parameters: storage type
            attr = cls._with(attr, attr.setup.castElemType(ctype.elem.dtype))
            ctype, cbytes = cls._type_of(attr)
        bits = abi.DTYPE_BITS[ctype.elem.dtype]
        # getOverlapRegionBounds (:716-727), kept as written: a view that starts before the constant and ends
        # at or behind its end does not count as overlapping
        lo = hi = 0
        if c_end > c_start and sub_end > sub_start and ((c_start <= sub_start < c_end) or (c_start < sub_end < c_end)):
            lo = max(sub_start, c_start)
            hi = min(sub_end, c_end)
        if lo == 0 and hi == 0:
            return None, c_end
        flat_off = (lo - c_start) * 8 // bits
        flat_n = (hi - lo) * 8 // bits
        # getNonFlatSubViewOffsetAndShape (:729-755): slice the outermost dim that covers the range
        dims = list(ctype.shape)
        off = [0] * len(dims)
        shp = list(dims)
        prev_stride, num, d = 1, 1, len(dims) - 1
        while d >= 0:
            num *= dims[d]
            if num >= flat_n + flat_off:
                break
            prev_stride = num
            d -= 1
        off[d] = flat_off // prev_stride
        covered = off[d] * prev_stride
        shp[d] = -(-(flat_n + flat_off) // prev_stride) - off[d]
        for k in range(d):
            shp[k] = 1
        if shp != dims:
            attr = cls._with(attr, attr.setup.subview(off, shp))
        _, nbytes = cls._type_of(attr)
        flat_total = nbytes * 8 // bits
        if not (flat_total == flat_n and flat_off - covered == 0):
            attr = cls._with(attr, attr.setup.reshape([1, 1, 1, flat_total])
                             .subview([0, 0, 0, flat_off - covered], [1, 1, 1, flat_n]))
        return attr, c_end

    # -- folding ----------------------------------------------------------------------------------------------
    def fold(self, library):
        """vf_fuse over the parts, then whatever stayed behind the Fuse through vf_fold on the fused bytes."""
        need = int(np.prod(self.fused_type.shape)) * abi.DTYPE_BITS[self.fused_type.elem.dtype] // 8
        raw, _ = library.fuse(self.parts(), need)
        if not self.trailing.names():
            return Folded(self.fused_type, False, np.ascontiguousarray(raw), len(raw))
        base = np.zeros(need, np.uint8)
        base[:len(raw)] = raw
        return ContentAttr(base.view(abi.DTYPE_NUMPY[self.fused_type.elem.dtype]), self.fused_type, self.trailing).fold(library)
