"""vf_sparsify_noalloc against vf_sparsify, through the C ABI, on two consecutive calls.

The allocation-free entry point serves embedders that must not allocate device memory while the compiler
runs (a serving process whose allocator owns the whole GPU): its scratch is a fixed array inside the library.
Because that array is shared by every call and keeps the previous call's contents, the second call here uses
a different shape and sparsity pattern than the first: stale counts or offsets would show up as a mismatch.
Collected last (file name) so that a failure here cannot hide any other test under `pytest -x`.
"""
import ctypes as C

import numpy as np
import pytest

from vpux_plugin_b200 import abi
from vpux_plugin_b200.abi import TType

pytestmark = pytest.mark.gpu


def _run_pair(gpu, torch, rng, oc, work, dtype, np_dtype, density):
    n = oc * work
    keep = rng.random(n) < density
    if dtype in (abi.VF_DT_I8, abi.VF_DT_U8):
        x = (rng.integers(1, 100, n) * keep).astype(np_dtype)
    else:
        x = (rng.standard_normal(n) * keep).astype(np_dtype)
    es = x.itemsize
    row = (work + 127) // 128 * 16
    cap = oc * ((work * es + 15) // 16 * 16)
    dev = torch.device("cuda", 0)
    xd = torch.from_numpy(x.view(np.uint8).copy()).to(dev)

    def bufs():
        return (torch.full((cap,), 0xAB, dtype=torch.uint8, device=dev), torch.full((oc * row,), 0xCD, dtype=torch.uint8, device=dev),
                torch.full((oc,), -7, dtype=torch.int64, device=dev))

    # existing entry point, device outputs
    d0, m0, c0 = bufs()
    content, keepalive = abi.make_content(TType([oc, work, 1, 1], dtype), None, ptr=xd.data_ptr(), nbytes=n * es,
                                          mem_kind=abi.VF_MEM_DEVICE)
    w0 = gpu.sparsify(content, d0.data_ptr(), m0.data_ptr(), c0.data_ptr(), out_mem_kind=abi.VF_MEM_DEVICE,
                      data_bytes=cap, map_bytes=oc * row)
    # allocation-free entry point
    d1, m1, c1 = bufs()
    written = C.c_uint64(0)
    err = C.create_string_buffer(512)
    st = gpu.lib.vf_sparsify_noalloc(gpu.ctx, C.c_void_p(xd.data_ptr()), C.c_int32(dtype), C.c_int64(oc), C.c_int64(work),
                                     C.c_int64(0), C.c_void_p(d1.data_ptr()), C.c_uint64(cap), C.byref(written),
                                     C.c_void_p(m1.data_ptr()), C.c_uint64(oc * row), C.c_void_p(c1.data_ptr()), err,
                                     C.c_size_t(512))
    assert st == 0, err.value
    assert written.value == w0
    assert torch.equal(d0[:w0], d1[:w0])
    assert torch.equal(m0, m1)
    assert torch.equal(c0, c1)
    # counts kept in the built-in scratch instead of a caller buffer
    d2, m2, _ = bufs()
    st = gpu.lib.vf_sparsify_noalloc(gpu.ctx, C.c_void_p(xd.data_ptr()), C.c_int32(dtype), C.c_int64(oc), C.c_int64(work),
                                     C.c_int64(0), C.c_void_p(d2.data_ptr()), C.c_uint64(cap), C.byref(written),
                                     C.c_void_p(m2.data_ptr()), C.c_uint64(oc * row), None, err, C.c_size_t(512))
    assert st == 0, err.value
    assert written.value == w0 and torch.equal(d0[:w0], d2[:w0]) and torch.equal(m0, m2)


def test_noalloc_sparsify_matches_regular_entry_point_twice(gpu):
    import torch
    gpu.lib.vf_sparsify_noalloc.restype = C.c_int
    rng = np.random.default_rng(2024)
    # two calls in a row on the shared scratch: large and sparse first, then small and dense
    _run_pair(gpu, torch, rng, oc=2048, work=4608, dtype=abi.VF_DT_I8, np_dtype=np.int8, density=0.3)
    _run_pair(gpu, torch, rng, oc=37, work=72, dtype=abi.VF_DT_F16, np_dtype=np.float16, density=0.9)


def test_noalloc_rejects_more_channels_than_the_scratch_holds(gpu):
    import torch
    gpu.lib.vf_sparsify_noalloc.restype = C.c_int
    x = torch.zeros(16, dtype=torch.uint8, device="cuda")
    err = C.create_string_buffer(512)
    st = gpu.lib.vf_sparsify_noalloc(gpu.ctx, C.c_void_p(x.data_ptr()), C.c_int32(abi.VF_DT_U8), C.c_int64(65537),
                                     C.c_int64(8), C.c_int64(0), None, C.c_uint64(0), None, None, C.c_uint64(0), None,
                                     err, C.c_size_t(512))
    assert st == abi.VF_ERR_CAPACITY
    assert b"exceed" in err.value
