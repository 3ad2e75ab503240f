"""ctypes binding of libvfold.so — the GPU product behind the reference-shaped host API.

`Library` exposes the same method surface as the CPU oracle used in tests
(infer_type / fold / row_stats / quantize_fold / nnz_per_oc / sparsify /
weights_table / synth_fill), but every computation runs in CUDA kernels on the
context's device. There is no CPU fallback: a missing library or device raises.
"""
import ctypes as C
import os

import numpy as np

from . import abi

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libvfold.so")


class VfoldError(RuntimeError):
    def __init__(self, status, msg):
        super().__init__(f"[{status}] {msg}")
        self.status = status


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(f"{LIB_PATH} is missing: build it with `python -m vpux_plugin_b200.build` "
                          "(the package has no CPU fallback)")
    lib = C.CDLL(LIB_PATH)
    for name in ("vf_infer_type", "vf_optimize_transforms", "vf_fold", "vf_fuse", "vf_row_stats", "vf_quantize_fold", "vf_quantize_fold_batch",
                 "vf_nnz_per_oc", "vf_sparsify", "vf_sparsify_batch", "vf_weights_table", "vf_weights_table_batch", "vf_synth_fill", "vf_plan_shards",
                 "vf_ctx_create", "vf_ctx_synchronize", "vf_abi_version", "vf_ctx_device", "vf_fold_batch", "vf_max_intermediate_size"):
        getattr(lib, name).restype = C.c_int
    lib.vf_ctx_destroy.restype = None
    lib.vf_ctx_destroy.argtypes = [C.c_void_p]
    lib.vf_ctx_stream.restype = C.c_void_p
    lib.vf_ctx_stream.argtypes = [C.c_void_p]
    lib.vf_ctx_device.argtypes = [C.c_void_p]
    lib.vf_ctx_launch_count.restype = C.c_uint64
    lib.vf_ctx_launch_count.argtypes = [C.c_void_p]
    lib.vf_status_string.restype = C.c_char_p
    lib.vf_status_string.argtypes = [C.c_int]
    return lib


_lib = None


def raw():
    global _lib
    if _lib is None:
        _lib = _load()
    return _lib


def _ptr(x):
    """numpy array -> host pointer; int -> raw (device) pointer; None -> NULL."""
    if x is None:
        return None
    if isinstance(x, np.ndarray):
        return C.c_void_p(x.ctypes.data)
    return C.c_void_p(int(x))


def plan_shards(mode, world, nbytes, rows, row_align=1):
    """vf_plan_shards: returns (row_begin, row_end) arrays of shape [ntensors, world]."""
    n = len(rows)
    b = np.ascontiguousarray(nbytes, np.uint64)
    r = np.ascontiguousarray(rows, np.int64)
    rb = np.zeros((n, world), np.int64)
    re = np.zeros((n, world), np.int64)
    err = C.create_string_buffer(512)
    st = raw().vf_plan_shards(int(mode), int(world), C.c_int64(n), _ptr(b), _ptr(r), C.c_int64(row_align), _ptr(rb),
                              _ptr(re), err, C.c_size_t(512))
    if st != 0:
        raise VfoldError(st, err.value.decode(errors="replace"))
    return rb, re


def infer_type(base_type, is_splat, transforms, n, params_cap=1 << 16):
    """vf_infer_type (pure host; needs no device)."""
    out = abi.TensorType()
    osplat = C.c_int(0)
    sb = np.empty(params_cap, np.float64)  # the library writes what the result type uses
    zb = np.empty(params_cap, np.int64)
    nbytes = C.c_uint64(0)
    err = C.create_string_buffer(512)
    bt = base_type.pod()
    st = raw().vf_infer_type(C.byref(bt), int(is_splat), transforms, n, C.byref(out), C.byref(osplat), _ptr(sb),
                             _ptr(zb), C.c_int64(params_cap), C.byref(nbytes), err, C.c_size_t(512))
    if st != 0:
        raise VfoldError(st, err.value.decode(errors="replace"))
    return abi.TType.from_pod(out), bool(osplat.value), nbytes.value


def max_intermediate_size(base_type, is_splat, transforms, n):
    """vf_max_intermediate_size (pure host) = getMaxIntermediateSize, const/passes/constant_folding.cpp:20-31."""
    out = C.c_uint64(0)
    err = C.create_string_buffer(512)
    bt = base_type.pod()
    st = raw().vf_max_intermediate_size(C.byref(bt), int(is_splat), transforms, n, C.byref(out), err, C.c_size_t(512))
    if st != 0:
        raise VfoldError(st, err.value.decode(errors="replace"))
    return out.value


def optimize_transforms(base_type, transforms, n, params_cap=1 << 16):
    """vf_optimize_transforms (pure host): returns (ctypes array of abi.Transform, count, keepalive)."""
    out = (abi.Transform * max(n, 1))()
    n_out = C.c_int(0)
    sb = np.empty(params_cap, np.float64)  # the library writes what the result type uses
    zb = np.empty(params_cap, np.int64)
    err = C.create_string_buffer(512)
    bt = base_type.pod()
    st = raw().vf_optimize_transforms(C.byref(bt), transforms, n, out, max(n, 1), C.byref(n_out), _ptr(sb), _ptr(zb),
                                      C.c_int64(params_cap), err, C.c_size_t(512))
    if st != 0:
        raise VfoldError(st, err.value.decode(errors="replace"))
    return out, n_out.value, (sb, zb, transforms)


class Library:
    """One vf_ctx (device + stream + scratch pool)."""

    def __init__(self, device=0, stream=None, disable_fusion=False, staging_bytes=0, pipelined=False, timing=False):
        """pipelined=True sets VF_OPT_ASYNC: batch calls over device memory return once enqueued; call
        synchronize() to wait and to learn what their kernels reported. timing=True sets VF_OPT_TIMING:
        synchronous calls report their device time in last_stats.device_ms."""
        self.lib = raw()
        self.ctx = C.c_void_p()
        opts = abi.Options()
        opts.staging_bytes = staging_bytes
        opts.flags = (1 if disable_fusion else 0) | (2 if pipelined else 0) | (4 if timing else 0)
        err = C.create_string_buffer(512)
        st = self.lib.vf_ctx_create(int(device), C.byref(opts), C.c_void_p(stream) if stream else None,
                                    C.byref(self.ctx), err, C.c_size_t(512))
        if st != 0:
            raise VfoldError(st, err.value.decode(errors="replace"))
        self.device = device
        self.last_stats = abi.Stats()

    def close(self):
        if self.ctx:
            self.lib.vf_ctx_destroy(self.ctx)
            self.ctx = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- plumbing -------------------------------------------------------------------------------------
    @staticmethod
    def _err():
        return C.create_string_buffer(512)

    @staticmethod
    def _check(st, err):
        if st != 0:
            raise VfoldError(st, err.value.decode(errors="replace"))

    @property
    def stream(self):
        return self.lib.vf_ctx_stream(self.ctx)

    @property
    def launch_count(self):
        return int(self.lib.vf_ctx_launch_count(self.ctx))

    def synchronize(self):
        err = self._err()
        self._check(self.lib.vf_ctx_synchronize(self.ctx, err, C.c_size_t(512)), err)

    # -- fold ---------------------------------------------------------------------------------------------
    def infer_type(self, base_type, is_splat, transforms, n, params_cap=1 << 16):
        return infer_type(base_type, is_splat, transforms, n, params_cap)

    def fold(self, content, transforms, n, dst, dst_bytes, params_cap=1 << 16, dst_mem_kind=abi.VF_MEM_HOST):
        out = abi.TensorType()
        sb = np.empty(params_cap, np.float64)  # the library writes what the result type uses
        zb = np.empty(params_cap, np.int64)
        written = C.c_uint64(0)
        err = self._err()
        st = self.lib.vf_fold(self.ctx, C.byref(content), transforms, n, _ptr(dst), C.c_uint64(dst_bytes),
                              int(dst_mem_kind), C.byref(written), C.byref(out), _ptr(sb), _ptr(zb),
                              C.c_int64(params_cap), C.byref(self.last_stats), err, C.c_size_t(512))
        self._check(st, err)
        return written.value, abi.TType.from_pod(out)

    def fuse(self, attrs, dst_bytes):
        """vf_fuse over a list of const.ContentAttr (None = absent part): returns (bytes, [(offset, size), ...])."""
        parts = (abi.FusePart * len(attrs))()
        keep = []
        for p, a in zip(parts, attrs):
            if a is None:
                continue
            c, k = abi.make_content(a.base_type, a.base, a.storage_dtype, a.is_splat)
            tr, n = a.setup.transforms()
            p.base, p.t, p.n = C.pointer(c), tr, n
            keep += [c, k, tr]
        dst = np.zeros(max(int(dst_bytes), 1), np.uint8)
        written = C.c_uint64(0)
        err = self._err()
        st = self.lib.vf_fuse(self.ctx, parts, len(attrs), _ptr(dst), C.c_uint64(dst_bytes), abi.VF_MEM_HOST,
                              C.byref(written), C.byref(self.last_stats), err, C.c_size_t(512))
        self._check(st, err)
        return dst[:written.value], [(int(p.offset), int(p.bytes)) for p in parts]

    def row_stats(self, content, spec, n_units):
        scales = np.zeros(n_units, np.float64)
        zps = np.zeros(n_units, np.int64)
        rmin = np.zeros(n_units, np.float32)
        rmax = np.zeros(n_units, np.float32)
        err = self._err()
        st = self.lib.vf_row_stats(self.ctx, C.byref(content), C.byref(spec), _ptr(scales), _ptr(zps), _ptr(rmin),
                                   _ptr(rmax), C.c_int64(n_units), abi.VF_MEM_HOST, err, C.c_size_t(512))
        self._check(st, err)
        return scales, zps, rmin, rmax

    def quantize_fold(self, content, spec, transforms, n, dst, dst_bytes, outs=None, dst_mem_kind=abi.VF_MEM_HOST):
        written = C.c_uint64(0)
        err = self._err()
        st = self.lib.vf_quantize_fold(self.ctx, C.byref(content), C.byref(spec), transforms, n, _ptr(dst),
                                       C.c_uint64(dst_bytes), int(dst_mem_kind), C.byref(written),
                                       C.byref(outs) if outs is not None else None, C.byref(self.last_stats), err,
                                       C.c_size_t(512))
        self._check(st, err)
        return written.value

    def quantize_fold_batch(self, jobs):
        """jobs: ctypes array of abi.QuantJob."""
        err = self._err()
        st = self.lib.vf_quantize_fold_batch(self.ctx, jobs, len(jobs), C.byref(self.last_stats), err, C.c_size_t(512))
        self._check(st, err)

    def fold_batch(self, jobs, threshold_bytes=0, tiny_threshold_bytes=0):
        """jobs: ctypes array of abi.FoldJob, folded with ConstantFoldingPass's schedule
        (const/passes/constant_folding.cpp:85-159). Returns abi.FoldBatchStats; every job's `dst_written`,
        `max_intermediate`, `group` and `status` are filled in, also when the call raises."""
        opts = abi.FoldBatchOptions(int(threshold_bytes), int(tiny_threshold_bytes))
        bs = abi.FoldBatchStats()
        err = self._err()
        st = self.lib.vf_fold_batch(self.ctx, jobs, len(jobs), C.byref(opts), C.byref(bs), C.byref(self.last_stats), err,
                                    C.c_size_t(512))
        self._check(st, err)
        return bs

    def nnz_per_oc(self, content, oc):
        counts = np.zeros(oc, np.int64)
        err = self._err()
        st = self.lib.vf_nnz_per_oc(self.ctx, C.byref(content), _ptr(counts), abi.VF_MEM_HOST, err, C.c_size_t(512))
        self._check(st, err)
        return counts

    def sparsify(self, content, data, mapbuf, counts, out_mem_kind=abi.VF_MEM_HOST, data_bytes=None, map_bytes=None):
        written = C.c_uint64(0)
        err = self._err()
        db = data_bytes if data_bytes is not None else (data.nbytes if data is not None else 0)
        mb = map_bytes if map_bytes is not None else (mapbuf.nbytes if mapbuf is not None else 0)
        st = self.lib.vf_sparsify(self.ctx, C.byref(content), _ptr(data), C.c_uint64(db), C.byref(written),
                                  _ptr(mapbuf), C.c_uint64(mb), _ptr(counts), int(out_mem_kind),
                                  C.byref(self.last_stats), err, C.c_size_t(512))
        self._check(st, err)
        return written.value

    def sparsify_batch(self, jobs, out_mem_kind=abi.VF_MEM_HOST):
        """jobs: ctypes array of abi.SparsifyJob; `data_written` of every job is filled in."""
        err = self._err()
        st = self.lib.vf_sparsify_batch(self.ctx, jobs, len(jobs), int(out_mem_kind), C.byref(self.last_stats), err,
                                        C.c_size_t(512))
        self._check(st, err)

    def weights_table(self, desc, oc, table=None, out_mem_kind=abi.VF_MEM_HOST):
        if table is None:
            table = np.zeros(oc * 4, np.int32)
        err = self._err()
        st = self.lib.vf_weights_table(self.ctx, C.byref(desc), _ptr(table), int(out_mem_kind), err, C.c_size_t(512))
        self._check(st, err)
        return table

    def weights_table_batch(self, jobs, out_mem_kind=abi.VF_MEM_HOST):
        """jobs: ctypes array of abi.WeightsTableJob (tables in memory of kind `out_mem_kind`)."""
        err = self._err()
        st = self.lib.vf_weights_table_batch(self.ctx, jobs, len(jobs), int(out_mem_kind), err, C.c_size_t(512))
        self._check(st, err)

    def synth_fill_device(self, spec, dst_ptr, count):
        err = self._err()
        st = self.lib.vf_synth_fill(self.ctx, C.byref(spec), C.c_void_p(int(dst_ptr)), C.c_uint64(count), err,
                                    C.c_size_t(512))
        self._check(st, err)


class Folder:
    """vf_folder: folding in the background with a cache of folded contents, the counterpart of
    Const::BackgroundConstantFolding + Const::ConstantFoldingCache
    (const/utils/constant_folding_in_background.cpp, constant_folding_cache.cpp).

    Takes const.ContentAttr objects. Also a fold backend: `attr.fold(folder)` is ContentAttr::fold() through the
    cache. `base_id` = 0 lets the library hash the base bytes on the GPU; the base arrays of queued attributes
    are kept alive here until wait_idle() / close()."""

    def __init__(self, device=0, memory_limit_bytes=0, clean_threshold=0.0, max_concurrent_tasks=0, collect_statistics=True):
        self.lib = raw()
        for name in ("vf_folder_create", "vf_folder_enqueue", "vf_folder_enqueue_equivalence", "vf_folder_wait_idle",
                     "vf_folder_has_content", "vf_folder_fold", "vf_folder_remove", "vf_folder_statistics", "vf_content_hash"):
            getattr(self.lib, name).restype = C.c_int
        self.lib.vf_folder_destroy.restype = None
        self.lib.vf_folder_destroy.argtypes = [C.c_void_p]
        opts = abi.FolderOptions(int(memory_limit_bytes), float(clean_threshold), int(max_concurrent_tasks),
                                 1 if collect_statistics else 0)
        self.h = C.c_void_p()
        err = C.create_string_buffer(512)
        st = self.lib.vf_folder_create(int(device), C.byref(opts), C.byref(self.h), err, C.c_size_t(512))
        if st != 0:
            raise VfoldError(st, err.value.decode(errors="replace"))
        self._keep = []
        self.from_cache = None  # whether the last fold() was served from the cache

    def close(self):
        if self.h:
            self.lib.vf_folder_destroy(self.h)
            self.h = C.c_void_p()
            self._keep = []

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @staticmethod
    def _check(st, err):
        if st != 0:
            raise VfoldError(st, err.value.decode(errors="replace"))

    @staticmethod
    def _parts(attr):
        content, keep = abi.make_content(attr.base_type, attr.base, attr.storage_dtype, attr.is_splat)
        tr, n = attr.setup.transforms()
        return content, tr, n, (keep, attr)

    def enqueue(self, attr, new_index=-1, base_id=0):
        content, tr, n, keep = self._parts(attr)
        self._keep.append(keep)
        err = C.create_string_buffer(512)
        self._check(self.lib.vf_folder_enqueue(self.h, C.byref(content), C.c_uint64(base_id), tr, n, int(new_index), err,
                                               C.c_size_t(512)), err)

    def enqueue_equivalence(self, original, new, base_id=0):
        content, tr0, n0, keep0 = self._parts(original)
        _, tr1, n1, keep1 = self._parts(new)
        self._keep += [keep0, keep1]
        err = C.create_string_buffer(512)
        self._check(self.lib.vf_folder_enqueue_equivalence(self.h, C.byref(content), C.c_uint64(base_id), tr0, n0, tr1, n1,
                                                           err, C.c_size_t(512)), err)

    def wait_idle(self):
        err = C.create_string_buffer(512)
        self._check(self.lib.vf_folder_wait_idle(self.h, err, C.c_size_t(512)), err)
        self._keep = []

    def has_content(self, attr, base_id=0):
        content, tr, n, keep = self._parts(attr)
        found = C.c_int(0)
        err = C.create_string_buffer(512)
        self._check(self.lib.vf_folder_has_content(self.h, C.byref(content), C.c_uint64(base_id), tr, n, C.byref(found),
                                                   err, C.c_size_t(512)), err)
        return bool(found.value)

    def remove(self, attr, base_id=0):
        content, tr, n, keep = self._parts(attr)
        err = C.create_string_buffer(512)
        self._check(self.lib.vf_folder_remove(self.h, C.byref(content), C.c_uint64(base_id), tr, n, err, C.c_size_t(512)), err)

    def last_error(self):
        buf = C.create_string_buffer(512)
        self.lib.vf_folder_last_error.restype = C.c_int
        self.lib.vf_folder_last_error(self.h, buf, C.c_size_t(512))
        return buf.value.decode(errors="replace")

    def statistics(self):
        s = abi.FolderStats()
        self.lib.vf_folder_statistics(self.h, C.byref(s))
        return {n: int(getattr(s, n)) for n, _ in abi.FolderStats._fields_}

    # -- fold backend (what const.ContentAttr.fold calls) ---------------------------------------------
    def infer_type(self, base_type, is_splat, transforms, n):
        return infer_type(base_type, is_splat, transforms, n)

    def fold(self, content, transforms, n, dst, dst_bytes, params_cap=1 << 16, dst_mem_kind=abi.VF_MEM_HOST, base_id=0):
        out = abi.TensorType()
        sb = np.empty(params_cap, np.float64)  # the library writes what the result type uses
        zb = np.empty(params_cap, np.int64)
        written = C.c_uint64(0)
        hit = C.c_int(0)
        err = C.create_string_buffer(512)
        st = self.lib.vf_folder_fold(self.h, C.byref(content), C.c_uint64(base_id), transforms, n, _ptr(dst),
                                     C.c_uint64(dst_bytes), int(dst_mem_kind), C.byref(written), C.byref(out), _ptr(sb),
                                     _ptr(zb), C.c_int64(params_cap), C.byref(hit), err, C.c_size_t(512))
        self._check(st, err)
        self.from_cache = bool(hit.value)
        return written.value, abi.TType.from_pod(out)


def content_hash(library, content):
    """vf_content_hash on a Library's context: (h0, h1)."""
    out = (C.c_uint64 * 2)()
    err = C.create_string_buffer(512)
    library.lib.vf_content_hash.restype = C.c_int
    st = library.lib.vf_content_hash(library.ctx, C.byref(content), out, err, C.c_size_t(512))
    if st != 0:
        raise VfoldError(st, err.value.decode(errors="replace"))
    return int(out[0]), int(out[1])
