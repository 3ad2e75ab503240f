"""vf_sparsify_noalloc against vf_sparsify and the CPU oracle, through the C ABI, on two consecutive calls.

The allocation-free entry point serves embedders that must not allocate device memory while the compiler
runs (a serving process whose allocator owns the whole GPU): its scratch is a fixed array inside the library.
Because that array is shared by every call and keeps the previous call's contents, the second call here uses
a different shape and sparsity pattern than the first: stale counts or offsets would show up as a mismatch.
Collected last (file name) so that a failure here cannot hide any other test under `pytest -x`.
"""
import ctypes as C
import os

import numpy as np
import pytest

from vpux_plugin_b200 import abi
from vpux_plugin_b200.abi import TType

pytestmark = pytest.mark.gpu


def _noalloc(gpu, x_ptr, dtype, oc, work, data, cap, mp, map_bytes, counts):
    written = C.c_uint64(0)
    err = C.create_string_buffer(512)
    st = gpu.lib.vf_sparsify_noalloc(gpu.ctx, C.c_void_p(x_ptr), C.c_int32(dtype), C.c_int64(oc), C.c_int64(work), C.c_int64(0),
                                     C.c_void_p(data) if data else None, C.c_uint64(cap), C.byref(written),
                                     C.c_void_p(mp) if mp else None, C.c_uint64(map_bytes), C.c_void_p(counts) if counts else None,
                                     err, C.c_size_t(512))
    return st, written.value, err.value


def _run_pair(gpu, oracle, torch, rng, oc, work, dtype, np_dtype, density):
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
        b = (torch.full((cap,), 0xAB, dtype=torch.uint8, device=dev), torch.full((oc * row,), 0xCD, dtype=torch.uint8, device=dev),
             torch.full((oc,), -7, dtype=torch.int64, device=dev))
        torch.cuda.synchronize()  # the fills run on torch's stream, the library on its own: finish them first
        return b

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
    # third column: the CPU oracle's Sparsify / GetSparsityMap / counts of the same tensor
    hc, hk = abi.make_content(TType([oc, work, 1, 1], dtype), x)
    hd, hm, hcnt = np.zeros(cap, np.uint8), np.zeros(oc * row, np.uint8), np.zeros(oc, np.int64)
    hw = oracle.sparsify(hc, hd, hm, hcnt)
    assert hw == written.value
    assert np.array_equal(d1[:hw].cpu().numpy(), hd[:hw]) and np.array_equal(m1.cpu().numpy(), hm) and np.array_equal(c1.cpu().numpy(), hcnt)
    # counts kept in the built-in scratch instead of a caller buffer
    d2, m2, _ = bufs()
    st = gpu.lib.vf_sparsify_noalloc(gpu.ctx, C.c_void_p(xd.data_ptr()), C.c_int32(dtype), C.c_int64(oc), C.c_int64(work),
                                     C.c_int64(0), C.c_void_p(d2.data_ptr()), C.c_uint64(cap), C.byref(written),
                                     C.c_void_p(m2.data_ptr()), C.c_uint64(oc * row), None, err, C.c_size_t(512))
    assert st == 0, err.value
    assert written.value == w0 and torch.equal(d0[:w0], d2[:w0]) and torch.equal(m0, m2)


def test_noalloc_sparsify_matches_regular_entry_point_twice(gpu, oracle):
    import torch
    gpu.lib.vf_sparsify_noalloc.restype = C.c_int
    rng = np.random.default_rng(2024)
    # two calls in a row on the shared scratch: large and sparse first, then small and dense
    _run_pair(gpu, oracle, torch, rng, oc=2048, work=4608, dtype=abi.VF_DT_I8, np_dtype=np.int8, density=0.3)
    _run_pair(gpu, oracle, torch, rng, oc=37, work=72, dtype=abi.VF_DT_F16, np_dtype=np.float16, density=0.9)


def test_noalloc_requests_no_device_memory_and_handles_the_limit(gpu):
    """What the entry point exists for: once the context is there, a call changes neither the free device memory
    nor what the context's pool holds. Run on the largest channel count the built-in array takes (the offsets of the
    last channel sit in its last slot), with the compacted data only, with the bitmap only, and with a buffer that
    is too small (the needed size comes back)."""
    import torch
    gpu.lib.vf_sparsify_noalloc.restype = C.c_int
    dev = torch.device("cuda", 0)
    oc, work = 65536, 8
    rng = np.random.default_rng(7)
    x = (rng.integers(1, 100, oc * work) * (rng.random(oc * work) < 0.5)).astype(np.uint8)
    xd = torch.from_numpy(x).to(dev)
    cap, row = oc * 16, 16
    d0 = torch.zeros(cap, dtype=torch.uint8, device=dev)
    m0 = torch.zeros(oc * row, dtype=torch.uint8, device=dev)
    c0 = torch.zeros(oc, dtype=torch.int64, device=dev)
    torch.cuda.synchronize()  # the fills run on torch's stream, the library on its own
    content, keep = abi.make_content(TType([oc, work, 1, 1], abi.VF_DT_U8), None, ptr=xd.data_ptr(), nbytes=oc * work, mem_kind=abi.VF_MEM_DEVICE)
    w0 = gpu.sparsify(content, d0.data_ptr(), m0.data_ptr(), c0.data_ptr(), out_mem_kind=abi.VF_MEM_DEVICE, data_bytes=cap, map_bytes=oc * row)
    d1, m1 = torch.zeros_like(d0), torch.zeros_like(m0)
    torch.cuda.synchronize()
    st, w, msg = _noalloc(gpu, xd.data_ptr(), abi.VF_DT_U8, oc, work, d1.data_ptr(), cap, m1.data_ptr(), oc * row, None)  # warm-up
    assert st == 0, msg
    d1.zero_()
    m1.zero_()
    torch.cuda.synchronize()

    # the device-wide figure only means something while no other process works on the GPU (test workers in parallel do)
    alone = "PYTEST_XDIST_WORKER" not in os.environ

    def call(*a):  # free device memory right before and right after the call (no torch work in between)
        free0 = torch.cuda.mem_get_info(0)[0]
        r = _noalloc(gpu, *a)
        torch.cuda.synchronize()
        assert not alone or torch.cuda.mem_get_info(0)[0] == free0, "a call of vf_sparsify_noalloc changed the free device memory"
        return r

    st, w, msg = call(xd.data_ptr(), abi.VF_DT_U8, oc, work, d1.data_ptr(), cap, None, 0, None)  # data only
    assert st == 0 and w == w0, msg
    st, w, msg = call(xd.data_ptr(), abi.VF_DT_U8, oc, work, None, 0, m1.data_ptr(), oc * row, None)  # bitmap only
    assert st == 0 and w == 0, msg
    assert torch.equal(d1[:w0], d0[:w0]) and torch.equal(m1, m0)
    st, w, msg = call(xd.data_ptr(), abi.VF_DT_U8, oc, work, d1.data_ptr(), 1024, None, 0, None)  # too small
    assert st == abi.VF_ERR_BUFFER_TOO_SMALL and w == w0, (st, w, msg)


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
