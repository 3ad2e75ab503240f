"""GPU parity: every entry point of libvfold.so against the CPU oracle on the same seeded inputs.

Integer / byte outputs must be bit-exact. Floating outputs (dequantize, rescale) are compared bit for bit
as well — the stated tolerance for them is 1 fp16 ULP, and the kernels use the reference's exact
operation order, so any difference is reported.
"""
import ctypes as C

import numpy as np
import pytest

import reference_cases as rc
from vpux_plugin_b200 import abi, workloads as wl
from vpux_plugin_b200.abi import Elem, TType
from vpux_plugin_b200.const import ContentAttr, ContentSetup

pytestmark = pytest.mark.gpu

F32, F16, BF16, I8, U8, I32 = abi.VF_DT_F32, abi.VF_DT_F16, abi.VF_DT_BF16, abi.VF_DT_I8, abi.VF_DT_U8, abi.VF_DT_I32


def bf16_bits(x):
    import torch
    return torch.from_numpy(np.ascontiguousarray(x, np.float32)).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)


def both(attr, gpu, oracle, dst_bytes=None):
    a = attr.fold(gpu, dst_bytes)
    b = attr.fold(oracle, dst_bytes)
    assert a.type == b.type, (a.type, b.type)
    assert a.written == b.written
    assert np.array_equal(a.bytes(), b.bytes()), f"{int((a.bytes() != b.bytes()).sum())} differing bytes"
    return a


# ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("case", rc.FOLD_CASES + rc.TABLE_CASES, ids=lambda c: c.__name__)
def test_reference_vectors_on_gpu(case, gpu):
    case(gpu)


# ---------------------------------------------------------------------------------------------------------
# randomized differential tests, one transformation (or short chain) at a time
# ---------------------------------------------------------------------------------------------------------
def _rand(rng, shape, dt):
    x = rng.standard_normal(shape).astype(np.float32)
    if dt == F32:
        return x
    if dt == F16:
        return x.astype(np.float16)
    return bf16_bits(x)


@pytest.mark.parametrize("dt", [F32, F16, BF16])
@pytest.mark.parametrize("storage,qmin,qmax", [(I8, -128, 127), (I8, -127, 127), (U8, 0, 255), (U8, 0, 15),
                                               (I8, -120, 120), (abi.VF_DT_I16, -32768, 32767), (I32, -1000, 1000)])
def test_quantize_per_tensor(gpu, oracle, dt, storage, qmin, qmax):
    rng = np.random.default_rng(1)
    t = TType([3, 5, 7], dt)
    x = _rand(rng, t.shape, dt)
    q = Elem.uniform(storage, F32, 0.013, (qmin + qmax) // 2 + 3, qmin, qmax)
    both(ContentAttr(x, t, ContentSetup(t).quantize(q)), gpu, oracle)


@pytest.mark.parametrize("axis", [0, 1, 3])
@pytest.mark.parametrize("order", [abi.ORDER_NCHW, abi.ORDER_NHWC])
def test_quantize_dequantize_per_axis(gpu, oracle, axis, order):
    rng = np.random.default_rng(2)
    shape = [6, 5, 3, 4]
    t = TType(shape, F16, order)
    x = _rand(rng, shape, F16)
    n = shape[axis]
    scales = rng.uniform(0.001, 0.05, n)
    zps = rng.integers(-20, 20, n)
    q = Elem.per_axis(I8, F16, scales, zps, axis, -127, 127)
    both(ContentAttr(x, t, ContentSetup(t).quantize(q)), gpu, oracle)
    codes = rng.integers(-127, 128, shape).astype(np.int8)
    tq = TType(shape, I8, order)
    for expressed in (F16, F32, BF16):
        qe = Elem.per_axis(I8, expressed, scales, zps, axis, -127, 127)
        both(ContentAttr(codes, tq, ContentSetup(tq).castElemType(qe).dequantize()), gpu, oracle)


def test_dequantize_fp16_overflow_clamps(gpu, oracle):
    """copyTo of an fp32 value beyond the fp16 range clamps to +-65504 (utils/content.hpp:41-55)."""
    t = TType([1, 8], I8)
    codes = np.array([-128, -100, -1, 0, 1, 50, 100, 127], np.int8)
    q = Elem.uniform(I8, F16, 1000.0, 0, -128, 127)
    out = both(ContentAttr(codes, t, ContentSetup(t).castElemType(q).dequantize()), gpu, oracle)
    v = out.values(np.float16).astype(np.float32)
    assert v[0] == -65504.0 and v[-1] == 65504.0 and v[3] == 0.0


def test_f32_to_f16_matches_reference_including_subnormal_quirk(gpu, oracle):
    """CastElemType<f16> on f32 storage converts at copyTo through float16(float) (float16.cpp:30-108)."""
    rng = np.random.default_rng(3)
    special = np.array([0x347FF000, 0x32FFF000, 0x33000000, 0x33000001, 0x387FFFFF, 0x38800000, 0x477FEFFF,
                        0x477FF000, 0x7F800000, 0xFF800000, 0x7FC00000, 0x7F800001, 0xFFC12345, 0x00000001,
                        0x80000000, 0x38000000, 0x37FFFFFF], np.uint32)
    # every mantissa with eleven leading ones across the subnormal-result exponents (the carry cases)
    exps = np.arange(100, 114, dtype=np.uint32)
    carry = ((exps[:, None] << 23) | (0x7FF000 + np.arange(0, 0x1000, 7, dtype=np.uint32))[None, :]).reshape(-1)
    rnd = rng.integers(0, 1 << 32, 1 << 20, dtype=np.uint64).astype(np.uint32)
    tiny = (rng.integers(0, 1 << 23, 1 << 20, dtype=np.uint64).astype(np.uint32)
            | (rng.integers(90, 114, 1 << 20, dtype=np.uint64).astype(np.uint32) << 23))
    bits = np.concatenate([special, carry, carry | 0x80000000, rnd, tiny])
    t = TType([bits.size], F32)
    out = both(ContentAttr(bits.view(np.float32), t, ContentSetup(t).castElemType(F16)), gpu, oracle)
    from oracle import ReferenceTypes
    if ReferenceTypes.available():  # the reference's own class, compiled unmodified
        ref = ReferenceTypes().f32_to_f16(bits)
        got = out.values(np.uint16)
        inf = (ref & 0x7FFF) == 0x7C00  # copyTo clamps infinities
        assert np.array_equal(got[~inf], ref[~inf])
        assert ((got[inf] & 0x7FFF) == 0x7BFF).all()


@pytest.mark.parametrize("dt", [F32, F16, BF16, I8, U8, I32])
def test_rescale_add(gpu, oracle, dt):
    rng = np.random.default_rng(4)
    t = TType([4, 33], dt)
    x = _rand(rng, t.shape, dt) if dt in (F32, F16, BF16) else rng.integers(0, 100, t.shape).astype(abi.DTYPE_NUMPY[dt])
    both(ContentAttr(x, t, ContentSetup(t).rescale(0.37).add(1.25)), gpu, oracle)
    if dt in (F32, F16, BF16):  # several vector steps per thread and a tail of three elements
        t2 = TType([5, 4099], dt)
        x2 = _rand(rng, t2.shape, dt)
        both(ContentAttr(x2, t2, ContentSetup(t2).rescale(-1.5)), gpu, oracle)
        both(ContentAttr(x2, t2, ContentSetup(t2).add(0.001)), gpu, oracle)


@pytest.mark.parametrize("dt,es", [(U8, 1), (F16, 2), (F32, 4)])
@pytest.mark.parametrize("shape,order_in,order_out", [
    ([2, 3, 4, 5], abi.ORDER_NCHW, abi.ORDER_NHWC), ([2, 3, 4, 5], abi.ORDER_NHWC, abi.ORDER_NCHW),
    ([7, 16, 3, 3], abi.ORDER_NCHW, 0x3412), ([5, 1, 1, 9], abi.ORDER_NCHW, abi.ORDER_NHWC),
    ([2, 3, 4, 5, 6], 0x12345, 0x13452), ([3, 4], 0x12, 0x21), ([4, 5, 6], 0x123, 0x312)])
def test_reorder(gpu, oracle, dt, es, shape, order_in, order_out):
    rng = np.random.default_rng(5)
    t = TType(shape, dt, order_in)
    x = rng.integers(0, 255, int(np.prod(shape)) * es).astype(np.uint8).view(abi.DTYPE_NUMPY[dt])
    both(ContentAttr(x, t, ContentSetup(t).reorder(order_out)), gpu, oracle)


@pytest.mark.parametrize("dt,es", [(U8, 1), (F16, 2), (F32, 4)])
@pytest.mark.parametrize("shape", [
    [5, 64, 3, 3], [3, 32, 5, 5], [2, 200, 7, 7], [2, 2048, 3, 3], [3, 16, 1, 2],      # whole slices through shared memory
    [50, 64, 3, 3], [131, 128, 1, 3],                                                  # several slices per chunk, a ragged last chunk
    [3, 64, 3, 171], [2, 80, 1, 1000], [2, 24, 3, 200], [1, 16, 37, 19], [2, 208, 9, 33],  # slices too large for it: 64 x 64 tiles
    [4, 48, 4, 4], [2, 16, 8, 16]])                                                      # row strides that are multiples of 128 bytes
def test_reorder_oiyx_to_oyxi_transposes(gpu, oracle, dt, es, shape):
    """OIYX -> OYXI through both transposes (slices staged whole in shared memory, and tiles): channel counts of one
    and several chunks with ragged ends, kernel sizes whose rows start at every alignment, slices of a few hundred
    bytes up to more than the shared memory holds, and the same shapes with two leading dims."""
    rng = np.random.default_rng(shape[1] + shape[3])
    t = TType(shape, dt)
    x = rng.integers(0, 255, int(np.prod(shape)) * es).astype(np.uint8).view(abi.DTYPE_NUMPY[dt])
    both(ContentAttr(x, t, ContentSetup(t).reorder(abi.ORDER_NHWC)), gpu, oracle)
    t5 = TType([2] + shape, dt)
    x5 = np.concatenate([x, x[::-1]])
    both(ContentAttr(x5, t5, ContentSetup(t5).reorder(0x12453)), gpu, oracle)


def test_transpose_and_mem_permute(gpu, oracle):
    rng = np.random.default_rng(6)
    t = TType([2, 3, 4, 5], F16, abi.ORDER_NHWC)
    x = _rand(rng, t.shape, F16)
    both(ContentAttr(x, t, ContentSetup(t).transpose(0x2143)), gpu, oracle)
    both(ContentAttr(x, t, ContentSetup(t).memPermute(abi.ORDER_NCHW, 0x4213)), gpu, oracle)


@pytest.mark.parametrize("order", [abi.ORDER_NCHW, abi.ORDER_NHWC])
def test_pad_variants(gpu, oracle, order):
    rng = np.random.default_rng(7)
    shape = [3, 5, 2, 4]
    t = TType(shape, F16, order)
    x = _rand(rng, shape, F16)
    both(ContentAttr(x, t, ContentSetup(t).padWithZero([1, 0, 2, 0], [0, 3, 0, 1])), gpu, oracle)
    codes = rng.integers(0, 255, shape).astype(np.uint8)
    tq = TType(shape, U8, order)
    qu = Elem.uniform(U8, F16, 0.1, 77, 0, 255)
    both(ContentAttr(codes, tq, ContentSetup(tq).castElemType(qu).padWithZero([0, 1, 1, 1], [2, 0, 0, 3])), gpu, oracle)
    qa = Elem.per_axis(U8, F16, [0.1, 0.2, 0.3], [9, 9, 9], 0, 0, 255)
    both(ContentAttr(codes, tq, ContentSetup(tq).castElemType(qa).padWithZero([1, 1, 0, 0], [2, 0, 1, 0])), gpu, oracle)
    # unequal zero points: padding inside a channel takes that channel's zero point
    qb = Elem.per_axis(U8, F16, [0.1, 0.2, 0.3], [3, 60, 200], 0, 0, 255)
    both(ContentAttr(codes, tq, ContentSetup(tq).castElemType(qb).padWithZero([0, 2, 0, 1], [0, 1, 1, 0])), gpu, oracle)


def test_subview(gpu, oracle):
    rng = np.random.default_rng(8)
    t = TType([6, 8, 3, 3], I8, abi.ORDER_NHWC)
    x = rng.integers(-128, 127, t.shape).astype(np.int8)
    q = Elem.per_axis(I8, F16, np.linspace(0.1, 0.6, 6), np.zeros(6), 0, -127, 127)
    out = both(ContentAttr(x, t, ContentSetup(t).castElemType(q).subview([2, 0, 0, 0], [3, 8, 3, 3])), gpu, oracle)
    assert out.type.elem.scales.tolist() == np.linspace(0.1, 0.6, 6)[2:5].tolist()


@pytest.mark.parametrize("dt", [I8, U8, F16, BF16, F32])
@pytest.mark.parametrize("shape", [[5, 8, 1, 1], [3, 4, 3, 2], [17, 16, 3, 3], [2, 40, 1, 1]])
def test_sparsify_and_map(gpu, oracle, dt, shape):
    rng = np.random.default_rng(9)
    n = int(np.prod(shape))
    keep = rng.random(n) < 0.45
    keep[:shape[1] * shape[2] * shape[3]] = True  # first channel dense
    if dt in (I8, U8):
        x = (rng.integers(1, 100, n) * keep).astype(abi.DTYPE_NUMPY[dt])
    elif dt == BF16:
        x = bf16_bits(rng.standard_normal(n) * keep)
    else:
        x = (rng.standard_normal(n) * keep).astype(abi.DTYPE_NUMPY[dt])
        x[3] = -0.0  # negative zero counts as zero
    t = TType(shape, dt)
    both(ContentAttr(x, t, ContentSetup(t).sparsify(False)), gpu, oracle, dst_bytes=n * 4 + 16 * shape[0])
    both(ContentAttr(x, t, ContentSetup(t).getSparsityMap()), gpu, oracle)
    c, keepalive = abi.make_content(t, x)
    assert np.array_equal(gpu.nnz_per_oc(c, shape[0]), oracle.nnz_per_oc(c, shape[0]))
    # combined entry point
    cap = n * 4 + 16 * shape[0]
    row = (shape[1] * shape[2] * shape[3] + 127) // 128 * 16
    outs = []
    for be in (gpu, oracle):
        data, mp, cnt = np.zeros(cap, np.uint8), np.zeros(shape[0] * row, np.uint8), np.zeros(shape[0], np.int64)
        w = be.sparsify(c, data, mp, cnt)
        outs.append((w, data[:w].copy(), mp, cnt))
    assert outs[0][0] == outs[1][0]
    for a, b in zip(outs[0][1:], outs[1][1:]):
        assert np.array_equal(a, b)


@pytest.mark.parametrize("density", [0.0, 0.07, 0.5, 0.93, 1.0])
def test_sparsify_batch(gpu, oracle, density):
    """Many tensors per call: long rows (several 32-vector steps with a carried remainder), rows that do not
    allow 16-byte accesses, every element type, a quantized type with a non-zero zero point, jobs without
    data / map / counts."""
    rng = np.random.default_rng(int(density * 100) + 3)
    specs = [([64, 128, 3, 3], I8, None), ([7, 512, 3, 3], U8, 3), ([5, 8, 1, 1], I8, None), ([33, 64, 1, 1], U8, 200),
             ([9, 72, 2, 2], F16, None), ([3, 4, 3, 2], F16, None), ([4, 136, 1, 1], BF16, None),
             ([6, 100, 1, 2], F32, None), ([2, 16, 7, 7], I8, None), ([130, 16, 1, 1], I8, None)]
    jobs = (abi.SparsifyJob * len(specs))()
    keep, expect, bufs = [], [], []
    for j, (shape, dt, zp) in enumerate(specs):
        n = int(np.prod(shape))
        work = n // shape[0]
        m = rng.random(n) < density
        if dt in (I8, U8):
            fill = 0 if zp is None else zp
            vals = rng.integers(1, 100, n)
            vals[vals == fill] += 1
            x = np.where(m, vals, fill).astype(abi.DTYPE_NUMPY[dt])
        elif dt == BF16:
            x = bf16_bits((rng.standard_normal(n) + 3.0) * m)
        else:
            x = ((rng.standard_normal(n) + 3.0) * m).astype(abi.DTYPE_NUMPY[dt])
            if n > 5 and not m[5]:
                x[5] = -0.0
        elem = dt if zp is None else Elem.uniform(dt, F16, 0.25, zp, 0, 255)
        c, k = abi.make_content(TType(shape, elem), x, storage_dtype=dt)
        row = (work + 127) // 128 * 16
        cap = n * x.itemsize + 16 * shape[0]
        want_data, want_map, want_cnt = j != 2, (work % 8 == 0) and j != 3, j != 4
        od, om, oc_ = np.zeros(cap, np.uint8), np.zeros(shape[0] * row, np.uint8), np.zeros(shape[0], np.int64)
        w = oracle.sparsify(c, od if want_data else None, om if want_map else None, oc_ if want_cnt else None)
        gd, gm, gc = np.full(cap, 0xAB, np.uint8), np.full(shape[0] * row, 0xAB, np.uint8), np.full(shape[0], -1, np.int64)
        jb = jobs[j]
        jb.content = c
        if want_data:
            jb.data, jb.data_bytes = gd.ctypes.data, cap
        if want_map:
            jb.map, jb.map_bytes = gm.ctypes.data, gm.nbytes
        if want_cnt:
            jb.counts = gc.ctypes.data
        keep += [c, k, x]
        expect.append((w, od, om, oc_, want_data, want_map, want_cnt))
        bufs.append((gd, gm, gc))
    gpu.sparsify_batch(jobs)
    assert gpu.last_stats.kernels_launched <= 4
    for j, ((w, od, om, oc_, want_data, want_map, want_cnt), (gd, gm, gc)) in enumerate(zip(expect, bufs)):
        if want_data:
            assert jobs[j].data_written == w, j
            assert np.array_equal(gd[:w], od[:w]), j
        if want_map:
            assert np.array_equal(gm, om), j
        if want_cnt:
            assert np.array_equal(gc, oc_), j


@pytest.mark.parametrize("fill", [0, 1, 0x7F, 0x80, 0xC8, 0xFF])
def test_sparsify_batch_every_byte_value(gpu, oracle, fill):
    """8-bit rows that hold every byte value next to the sparsify value `fill`, in runs of every length from 0 to
    40 kept and dropped elements: the mask arithmetic on whole words and the word-wise compaction see every
    combination of kept bytes inside a word and every alignment of the compacted run."""
    rng = np.random.default_rng(fill + 11)
    oc, work = 24, 4608
    x = np.empty((oc, work), np.uint8)
    for r in range(oc):
        row, at = [], 0
        while at < work:
            keep_n, drop_n = int(rng.integers(0, 41)), int(rng.integers(0, 41))
            vals = rng.integers(0, 256, keep_n)
            vals[vals == fill] = (fill + 1 + r) % 256 if (fill + 1 + r) % 256 != fill else (fill + 2) % 256
            row += [vals, np.full(drop_n, fill)]
            at += keep_n + drop_n
        x[r] = np.concatenate(row)[:work]
    x[0, :256] = np.arange(256)  # every value once, `fill` among them
    shape = [oc, work // 9, 3, 3]
    elem = U8 if fill == 0 else Elem.uniform(U8, F16, 0.25, fill, 0, 255)
    c, k = abi.make_content(TType(shape, elem), x.reshape(-1), storage_dtype=U8)
    row_bytes = (work + 127) // 128 * 16
    cap = oc * work + 16 * oc
    od, om, ocnt = np.zeros(cap, np.uint8), np.zeros(oc * row_bytes, np.uint8), np.zeros(oc, np.int64)
    w = oracle.sparsify(c, od, om, ocnt)
    gd, gm, gc = np.full(cap, 0xAB, np.uint8), np.full(oc * row_bytes, 0xAB, np.uint8), np.full(oc, -1, np.int64)
    jobs = (abi.SparsifyJob * 1)()
    jobs[0].content, jobs[0].data, jobs[0].data_bytes = c, gd.ctypes.data, cap
    jobs[0].map, jobs[0].map_bytes, jobs[0].counts = gm.ctypes.data, gm.nbytes, gc.ctypes.data
    gpu.sparsify_batch(jobs)
    assert jobs[0].data_written == w
    assert np.array_equal(gc, ocnt)
    assert np.array_equal(gm, om)
    assert np.array_equal(gd[:w], od[:w])


def test_sparsify_batch_buffer_too_small(gpu):
    x = np.ones([4, 16, 1, 1], np.int8)
    c, _k = abi.make_content(TType([4, 16, 1, 1], I8), x)
    jobs = (abi.SparsifyJob * 1)()
    out = np.zeros(32, np.uint8)
    jobs[0].content, jobs[0].data, jobs[0].data_bytes = c, out.ctypes.data, 32
    from vpux_plugin_b200.lib import VfoldError
    with pytest.raises(VfoldError) as e:
        gpu.sparsify_batch(jobs)
    assert e.value.status == abi.VF_ERR_BUFFER_TOO_SMALL
    assert jobs[0].status == abi.VF_ERR_BUFFER_TOO_SMALL


def test_sparsify_batch_pipelined_sizes_arrive_with_the_next_synchronisation(oracle):
    """VF_OPT_ASYNC, everything in device memory: vf_sparsify_batch returns once enqueued with data_written still 0;
    vf_ctx_synchronize fills the sizes in, and reports a compressed set that did not fit (nothing written past
    the end of its buffer)."""
    import torch
    from vpux_plugin_b200.lib import Library, VfoldError
    lib = Library(device=0, pipelined=True)
    dev = torch.device("cuda", 0)
    rng = np.random.default_rng(5)
    shapes = [[64, 128, 3, 3], [33, 64, 1, 1], [130, 16, 1, 1]]
    jobs = (abi.SparsifyJob * len(shapes))()
    keep, expect = [], []
    for j, shape in enumerate(shapes):
        n = int(np.prod(shape))
        work = n // shape[0]
        x = np.where(rng.random(n) < 0.4, rng.integers(1, 100, n), 0).astype(np.int8)
        hc, hk = abi.make_content(TType(shape, I8), x)
        row = (work + 127) // 128 * 16
        cap = n + 16 * shape[0]
        od, om, oc_ = np.zeros(cap, np.uint8), np.zeros(shape[0] * row, np.uint8), np.zeros(shape[0], np.int64)
        w = oracle.sparsify(hc, od, om, oc_)
        src = torch.from_numpy(x.view(np.uint8)).to(dev)
        data = torch.full((cap + 64,), 0xAB, dtype=torch.uint8, device=dev)
        mp = torch.zeros(shape[0] * row, dtype=torch.uint8, device=dev)
        cnt = torch.zeros(shape[0], dtype=torch.int64, device=dev)
        c, k = abi.make_content(TType(shape, I8), None, ptr=src.data_ptr(), nbytes=n, mem_kind=abi.VF_MEM_DEVICE)
        jobs[j].content, jobs[j].data, jobs[j].data_bytes = c, data.data_ptr(), cap
        jobs[j].map, jobs[j].map_bytes, jobs[j].counts = mp.data_ptr(), mp.numel(), cnt.data_ptr()
        keep += [src, k, hk]
        expect.append((w, od, om, oc_, data, mp, cnt, cap))
    torch.cuda.synchronize()
    for _ in range(3):  # several calls in flight
        lib.sparsify_batch(jobs, out_mem_kind=abi.VF_MEM_DEVICE)
    lib.synchronize()
    for j, (w, od, om, oc_, data, mp, cnt, cap) in enumerate(expect):
        assert jobs[j].data_written == w, j
        got = data.cpu().numpy()
        assert np.array_equal(got[:w], od[:w]) and (got[cap:] == 0xAB).all(), j
        assert np.array_equal(mp.cpu().numpy(), om) and np.array_equal(cnt.cpu().numpy(), oc_), j
    # a buffer that is too small: the call returns, the synchronisation reports it, the bytes behind the buffer stay
    small = expect[0][0] - 48
    jobs[0].data_bytes = small
    expect[0][4][small:] = 0xCD
    torch.cuda.synchronize()
    lib.sparsify_batch(jobs, out_mem_kind=abi.VF_MEM_DEVICE)
    with pytest.raises(VfoldError) as e:
        lib.synchronize()
    assert e.value.status == abi.VF_ERR_BUFFER_TOO_SMALL and jobs[0].status == abi.VF_ERR_BUFFER_TOO_SMALL
    assert jobs[0].data_written == expect[0][0]  # the size that is needed
    assert (expect[0][4].cpu().numpy()[small:] == 0xCD).all()
    jobs[0].data_bytes = expect[0][7]
    lib.sparsify_batch(jobs, out_mem_kind=abi.VF_MEM_DEVICE)  # the context stays usable
    lib.synchronize()
    assert jobs[0].data_written == expect[0][0]
    lib.close()


@pytest.mark.parametrize("src,dst", [(abi.VF_DT_U4, U8), (abi.VF_DT_I4, I8), (abi.VF_DT_I1, I8), (abi.VF_DT_I1, U8)])
@pytest.mark.parametrize("n", [1, 7, 8, 9, 63, 4096, 100003])
def test_convert_elem_type_unpacks_sub_byte(gpu, oracle, src, dst, n):
    """ConvertElemType on 1- and 4-bit storage (convert_utils.cpp:17-75): element counts that are not multiples
    of eight exercise the tail, the large one the vector path; splats take their own branch."""
    rng = np.random.default_rng(n)
    bits = 1 if src == abi.VF_DT_I1 else 4
    raw = rng.integers(0, 256, (n * bits + 7) // 8).astype(np.uint8)
    t = TType([n], src)
    both(ContentAttr(raw, t, ContentSetup(t).convertElemType(dst), storage_dtype=src), gpu, oracle)
    both(ContentAttr(raw[:1], t, ContentSetup(t).convertElemType(dst), is_splat=True, storage_dtype=src), gpu, oracle)


def _physical(addr, key, arch):
    """AddressTransform::getPhysicalAddress (swizzle_transform.cpp:71-83) on whole-chunk addresses."""
    log2w, cut = (5, (1 << 10) - 1) if arch == abi.VF_ARCH_NPU40XX else (4, (1 << 9) - 1)
    bits = key % 6
    shift = 9 - bits + (1 if arch == abi.VF_ARCH_NPU40XX else 0)
    s = (((addr >> log2w) & 0x7FF) >> 5) & ((1 << bits) - 1)
    return (((addr + (s << shift)) & cut) + (addr & ~cut)), 1 << log2w


@pytest.mark.parametrize("arch", [abi.VF_ARCH_NPU37XX, abi.VF_ARCH_NPU40XX])
@pytest.mark.parametrize("key", [0, 1, 3, 5])
@pytest.mark.parametrize("dt,n", [(U8, 100000), (F16, 33333), (F32, 5000), (I8, 512)])
def test_swizzle_constant(gpu, oracle, arch, key, dt, n):
    """GPU == oracle, and the result is the chunk permutation the address transform defines (checked here
    independently of both), padded with zeros to the swizzling-aligned size."""
    rng = np.random.default_rng(key * 10 + n)
    x = rng.integers(0, 256, n * abi.DTYPE_NUMPY[dt]().itemsize).astype(np.uint8).view(abi.DTYPE_NUMPY[dt])
    t = TType([n], dt)
    out = both(ContentAttr(x, t, ContentSetup(t).swizzleConstant(key, arch)), gpu, oracle).bytes()
    align = 1024 if arch == abi.VF_ARCH_NPU40XX else 512
    raw = x.view(np.uint8)
    assert out.size == (raw.size + align - 1) // align * align
    padded = np.zeros(out.size, np.uint8)
    padded[:raw.size] = raw
    expect = np.zeros_like(padded)
    w = _physical(0, key, arch)[1]
    for a in range(0, out.size, w):
        p = _physical(a, key, arch)[0]
        expect[p:p + w] = padded[a:a + w]
    assert np.array_equal(out, expect)
    assert np.array_equal(np.sort(out), np.sort(padded))  # a permutation of the padded bytes


def test_fuse_lays_the_folded_constants_end_to_end(gpu, oracle):
    """vf_fuse = FuseAttr::transform (fuse_transform.cpp:31-63): weights table, weights, sparsity map, activations,
    each folded and materialised like copyTo(); the map is 1-bit data packed eight per byte; absent parts skip."""
    rng = np.random.default_rng(41)
    oc, ic = 16, 32
    tt = TType([oc, 1, 1, 4], I32)
    table = rng.integers(0, 1 << 20, oc * 4).astype(np.int32)
    wt = TType([oc, ic, 1, 1], I8)
    w = (rng.integers(-100, 100, oc * ic) * (rng.random(oc * ic) < 0.5)).astype(np.int8)
    q = Elem.per_axis(I8, F16, rng.uniform(0.01, 0.1, oc), np.zeros(oc, np.int64), 0, -127, 127)
    parts = [ContentAttr(table, tt, ContentSetup(tt)),
             ContentAttr(w, wt, ContentSetup(wt).castElemType(q).reorder(abi.ORDER_NHWC).sparsify(False)),
             ContentAttr(w, wt, ContentSetup(wt).castElemType(q).reorder(abi.ORDER_NHWC).getSparsityMap()),
             None]
    cap = 1 << 16
    fused, where = gpu.fuse(parts, cap)
    expect, at = [], 0
    for p, (off, size) in zip(parts, where):
        assert off == at
        if p is None:
            assert size == 0
            continue
        b = p.fold(oracle, cap).bytes()
        assert size == b.size
        expect.append(b)
        at += size
    assert np.array_equal(fused, np.concatenate(expect))
    assert where[2][1] == oc * 16  # 32 one-bit values per channel in rows of 128 bits
    assert _status(lambda: gpu.fuse(parts, 100)) == abi.VF_ERR_BUFFER_TOO_SMALL


def test_convert_elem_type_rejects_sign_changes(gpu, oracle):
    t = TType([8], abi.VF_DT_U4)
    raw = np.zeros(4, np.uint8)
    for be in (gpu, oracle):
        assert _status(lambda: ContentAttr(raw, t, ContentSetup(t).convertElemType(I8), storage_dtype=abi.VF_DT_U4).fold(be)) \
            == abi.VF_ERR_UNSUPPORTED


def test_sparsify_quantized_with_supplied_counts(gpu, oracle):
    rng = np.random.default_rng(10)
    shape = [4, 8, 2, 2]
    x = rng.integers(0, 4, shape).astype(np.uint8)
    t = TType(shape, U8)
    q = Elem.uniform(U8, F16, 0.5, 2, 0, 255)
    c, _k = abi.make_content(TType(shape, q), x, storage_dtype=U8)
    counts = oracle.nnz_per_oc(c, 4)
    both(ContentAttr(x, t, ContentSetup(t).castElemType(q).sparsify(True, counts)), gpu, oracle)
    both(ContentAttr(x, t, ContentSetup(t).castElemType(q).sparsify(True, counts + 5)), gpu, oracle)


def test_bitpack_paths(gpu, oracle):
    rng = np.random.default_rng(11)
    for n in (6, 32, 4096 + 16, 1000):
        x = rng.integers(0, 16, n).astype(np.uint8)
        t = TType([1, n], U8)
        both(ContentAttr(x, t, ContentSetup(t).bitPack(4)), gpu, oracle)
    xi = rng.integers(0, 8, 64).astype(np.int8)
    t = TType([64], I8)
    both(ContentAttr(xi, t, ContentSetup(t).bitPack(4)), gpu, oracle)


# ---------------------------------------------------------------------------------------------------------
# error behaviour: same status code from both sides
# ---------------------------------------------------------------------------------------------------------
def _status(fn):
    try:
        fn()
    except Exception as e:  # VfoldError / OracleError both carry .status
        return e.status
    return 0


@pytest.mark.parametrize("build,status", [
    (lambda: ContentAttr(np.array([-1, 2], np.int8), TType([2], I8), ContentSetup(TType([2], I8)).bitPack(4)),
     abi.VF_ERR_CHECKED_CAST),  # getValues<uint8_t>() of a negative value
    (lambda: ContentAttr(np.arange(3, dtype=np.uint8), TType([3], U8), ContentSetup(TType([3], U8)).bitPack(4)),
     abi.VF_ERR_ODD_COUNT),
    (lambda: ContentAttr(np.zeros(4, np.float32), TType([4], F32), ContentSetup(TType([4], F32)).dequantize()),
     abi.VF_ERR_NOT_QUANTIZED),
    (lambda: ContentAttr(np.zeros(16, np.uint8), TType([2, 2, 2, 2], U8), ContentSetup(TType([2, 2, 2, 2], U8))
                         .castElemType(Elem.per_axis(U8, F16, [1, 1], [3, 4], 0, 0, 255)).sparsify(False)),
     abi.VF_ERR_ZERO_POINTS),
    (lambda: ContentAttr(np.zeros(16, np.uint8), TType([2, 2, 2, 2], U8), ContentSetup(TType([2, 2, 2, 2], U8))
                         .castElemType(Elem.per_axis(U8, F16, [1, 1], [3, 4], 0, 0, 255))
                         .padWithZero([1, 0, 0, 0], [0, 0, 0, 0])), abi.VF_ERR_ZERO_POINTS),
    (lambda: ContentAttr(np.full(4, 300.0, np.float32), TType([4], F32), ContentSetup(TType([4], F32)).castElemType(U8)),
     abi.VF_ERR_CHECKED_CAST),  # copyTo float -> u8 out of range throws instead of saturating
    (lambda: ContentAttr(np.zeros(4, np.float16), TType([4], F16), ContentSetup(TType([4], F16))
                         .quantize(Elem.uniform(abi.VF_DT_U4, F16, 1.0, 0, 0, 15))), abi.VF_ERR_UNSUPPORTED),
])
def test_error_codes_match(gpu, oracle, build, status):
    attr = build()
    assert _status(lambda: attr.fold(gpu, 64)) == status
    assert _status(lambda: attr.fold(oracle, 64)) == status


def test_copy_to_buffer_too_small(gpu, oracle):
    t = TType([16], F32)
    attr = ContentAttr(np.zeros(16, np.float32), t, ContentSetup(t))
    assert _status(lambda: attr.fold(gpu, 8)) == abi.VF_ERR_BUFFER_TOO_SMALL
    assert _status(lambda: attr.fold(oracle, 8)) == abi.VF_ERR_BUFFER_TOO_SMALL


# ---------------------------------------------------------------------------------------------------------
# statistics, fused weight quantization, synthetic generator
# ---------------------------------------------------------------------------------------------------------
def test_synth_generator_bits(gpu, oracle):
    import torch
    for spec in (wl.c1_tensors()[0], wl.resnet50_tensors(sparse=True)[5], wl.llama2_7b_tensors()[0],
                 wl.llama3_70b_tensors()[1]):
        n = min(spec.numel, 1 << 20)
        first = 12345 * 8
        s = spec.synth_spec(0xABCDEF, first)
        ref = oracle.synth_fill(s, n)
        buf = torch.empty(n * abi.DTYPE_BITS[spec.dtype] // 8, dtype=torch.uint8, device="cuda")
        gpu.synth_fill_device(s, buf.data_ptr(), n)
        got = buf.cpu().numpy().view(ref.dtype)
        assert np.array_equal(got.view(np.uint8), ref.view(np.uint8)), spec.name


def _quant_fold(be, spec_t, x, qspec, transforms, out_bytes, units, want=("scales", "zps"), dequant_dt=None):
    t = TType(list(spec_t), abi.VF_DT_F16 if x.dtype == np.float16 else (F32 if x.dtype == np.float32 else BF16))
    c, keep = abi.make_content(t, x)
    tr = abi.make_transforms(transforms)
    dst = np.zeros(out_bytes, np.uint8)
    outs = abi.QuantOutputs()
    outs.mem_kind = abi.VF_MEM_HOST
    res = {}
    if "scales" in want:
        res["scales"] = np.zeros(units, np.float64)
        outs.scales = res["scales"].ctypes.data
    if "zps" in want:
        res["zps"] = np.zeros(units, np.int64)
        outs.zps = res["zps"].ctypes.data
    if "f16" in want:
        res["f16"] = np.zeros(units, np.uint16)
        outs.scales_f16 = res["f16"].ctypes.data
    if "u4" in want:
        res["u4"] = np.zeros((units + 1) // 2, np.uint8)
        outs.zps_u4_packed = res["u4"].ctypes.data
    if dequant_dt is not None:
        n = int(np.prod(spec_t))
        res["dequant"] = np.zeros(n * abi.DTYPE_BITS[dequant_dt] // 8, np.uint8)
        outs.dequant = res["dequant"].ctypes.data
        outs.dequant_dtype = dequant_dt
        outs.dequant_bytes = res["dequant"].nbytes
    w = be.quantize_fold(c, qspec, tr, len(transforms), dst, out_bytes, outs)
    res["codes"] = dst[:w].copy()
    return res


def _same(a, b):
    assert a.keys() == b.keys()
    for k in a:
        assert np.array_equal(a[k], b[k]), f"{k}: {int((a[k] != b[k]).sum())} of {a[k].size} differ"


@pytest.mark.parametrize("group", [32, 64, 128])
@pytest.mark.parametrize("dt", [F16, BF16])
@pytest.mark.parametrize("rows,cols", [(4, 4096), (3, 1408), (33, 128), (1, 256)])
def test_group_u4_fused_matches_oracle_and_general(gpu, oracle, group, dt, rows, cols):
    from vpux_plugin_b200.lib import Library
    rng = np.random.default_rng(12)
    x = rng.standard_normal((rows, cols)).astype(np.float32) * 0.02
    x[rng.random((rows, cols)) < 0.001] *= 20
    x[0, :group] = 0  # an all-zero group
    x[-1, -group:] = np.abs(x[-1, -group:])  # an all-positive group
    x = x.astype(np.float16) if dt == F16 else bf16_bits(x)
    units = rows * cols // group
    args = ((rows, cols), x, wl.spec_u4_group(group), [wl.t_bitpack()], rows * cols // 2, units)
    ref = _quant_fold(oracle, *args, want=("scales", "zps", "f16", "u4"))
    got = _quant_fold(gpu, *args, want=("scales", "zps", "f16", "u4"))
    assert gpu.last_stats.fused == 1 and gpu.last_stats.kernels_launched == 1
    _same(got, ref)
    general = Library(device=0, disable_fusion=True)
    gen = _quant_fold(general, *args, want=("scales", "zps", "f16", "u4"))
    assert general.last_stats.fused == 0
    _same(gen, ref)
    # unpacked u8 codes and a dequantized fp16 copy
    args2 = ((rows, cols), x, wl.spec_u4_group(group), [], rows * cols, units)
    _same(_quant_fold(gpu, *args2, dequant_dt=F16), _quant_fold(oracle, *args2, dequant_dt=F16))


@pytest.mark.parametrize("dt", [F16, BF16])
@pytest.mark.parametrize("rows,cols", [(5, 8192), (3, 28672), (7, 4096), (2, 1024), (9, 11008), (2, 40000)])
@pytest.mark.parametrize("ddt", [F16, F32])
def test_row_i8_with_dequant_fused(gpu, oracle, dt, rows, cols, ddt):
    rng = np.random.default_rng(13)
    x = rng.standard_normal((rows, cols)).astype(np.float32) * 0.02
    x[1] = 0  # all-zero row: scale 1.0, zero point 0
    x[0] *= 1e-3  # tiny scale: dequantized values reach the fp16 subnormal range
    x = x.astype(np.float16) if dt == F16 else bf16_bits(x)
    args = ((rows, cols), x, wl.spec_i8_sym(ddt), [], rows * cols, rows)
    ref = _quant_fold(oracle, *args, want=("scales", "zps", "f16"), dequant_dt=ddt)
    got = _quant_fold(gpu, *args, want=("scales", "zps", "f16"), dequant_dt=ddt)
    assert gpu.last_stats.fused == 1
    _same(got, ref)
    # asymmetric u8 through the same kernel
    args = ((rows, cols), x, wl.spec_u8_asym(), [], rows * cols, rows)
    _same(_quant_fold(gpu, *args), _quant_fold(oracle, *args))


@pytest.mark.parametrize("dt", [F16, BF16])
def test_rows_and_groups_made_of_exact_ties(gpu, oracle, dt):
    """Every element sits exactly on a rounding boundary (x * (L-1) / range = integer + 1/2 in exact
    arithmetic), so every vector enters the guard band: the repair lists overflow, the inline repair runs, and
    half-away rounding must agree with the reference for each element. Rows: absmax 127 * 2^-7, values
    (2m+1) * 2^-8. Groups of 128 (u4): min 0, max 15 * 2^-4, values (2m+1) * 2^-5."""
    rng = np.random.default_rng(31)
    to = (lambda a: a.astype(np.float16)) if dt == F16 else bf16_bits
    for rows, cols in ((6, 8192), (2, 28672), (3, 2048)):
        m = rng.integers(-60, 60, (rows, cols))
        x = ((2 * m + 1) * 2.0 ** -8).astype(np.float32)
        x[:, 0] = 127 * 2.0 ** -7
        x[0, 1] = -127 * 2.0 ** -7
        args = ((rows, cols), to(x), wl.spec_i8_sym(F16), [], rows * cols, rows)
        _same(_quant_fold(gpu, *args, want=("scales", "zps"), dequant_dt=F16),
              _quant_fold(oracle, *args, want=("scales", "zps"), dequant_dt=F16))
        assert gpu.last_stats.fused == 1
        args = ((rows, cols), to(x), wl.spec_u8_asym(), [], rows * cols, rows)
        _same(_quant_fold(gpu, *args), _quant_fold(oracle, *args))
    rows, cols = 8, 4096
    m = rng.integers(0, 15, (rows, cols))
    x = ((2 * m + 1) * 2.0 ** -5).astype(np.float32)
    x[:, ::128] = 0.0
    x[:, 1::128] = 15 * 2.0 ** -4
    args = ((rows, cols), to(x), wl.spec_u4_group(128), [wl.t_bitpack()], rows * cols // 2, rows * cols // 128)
    _same(_quant_fold(gpu, *args, want=("scales", "zps", "f16", "u4")), _quant_fold(oracle, *args, want=("scales", "zps", "f16", "u4")))
    assert gpu.last_stats.fused == 1
    # convolution rows through the per-channel kernels
    shape = (16, 64, 3, 3)
    m = rng.integers(-60, 60, shape)
    xc = ((2 * m + 1) * 2.0 ** -8).astype(np.float32)
    xc[:, 0, 0, 0] = 127 * 2.0 ** -7
    ts, oshape = wl.conv_pipeline(shape)
    args = (shape, to(xc), wl.spec_i8_sym(), ts, int(np.prod(oshape)), shape[0])
    _same(_quant_fold(gpu, *args), _quant_fold(oracle, *args))


@pytest.mark.parametrize("dt", [F32, F16, BF16])
@pytest.mark.parametrize("shape,pad_oc,pad_ic", [((60, 64, 3, 3), 64, None), ((64, 3, 7, 7), None, 16),
                                                 ((16, 8, 1, 1), None, None), ((5, 3, 3, 3), 8, 4),
                                                 ((12, 512, 3, 3), None, None), ((1000, 2048, 1, 1), None, None)])
@pytest.mark.parametrize("sym", [True, False])
def test_conv_quantize_reorder_pad_fused(gpu, oracle, dt, shape, pad_oc, pad_ic, sym):
    rng = np.random.default_rng(14)
    x = rng.standard_normal(shape).astype(np.float32) * 0.05
    x = x if dt == F32 else (x.astype(np.float16) if dt == F16 else bf16_bits(x))
    ts, oshape = wl.conv_pipeline(shape, pad_oc, pad_ic)
    spec = wl.spec_i8_sym() if sym else wl.spec_u8_asym()
    args = (shape, x, spec, ts, int(np.prod(oshape)), shape[0])
    ref = _quant_fold(oracle, *args)
    got = _quant_fold(gpu, *args)
    assert gpu.last_stats.fused == 1
    _same(got, ref)
    # the same pipeline through vf_row_stats + vf_fold (Quantize with explicit parameters, unfused)
    t = TType(list(shape), dt)
    c, keep = abi.make_content(t, x)
    s, z, mn, mx = gpu.row_stats(c, spec, shape[0])
    so, zo, mno, mxo = oracle.row_stats(c, spec, shape[0])
    assert np.array_equal(s, so) and np.array_equal(z, zo) and np.array_equal(mn, mno) and np.array_equal(mx, mxo)
    q = Elem.per_axis(spec.storage_dtype, F16, s, z, 0, spec.qmin, spec.qmax)
    setup = ContentSetup(t).quantize(q).reorder(abi.ORDER_NHWC)
    if len(ts) > 1:
        setup = setup.padWithZero([0, 0, 0, 0], [oshape[0] - shape[0], oshape[1] - shape[1], 0, 0])
    out = ContentAttr(x, t, setup).fold(gpu)
    assert np.array_equal(out.bytes(), ref["codes"])


def test_quantize_refuses_nan(gpu, oracle):
    """fakeQuantize lets a NaN through both comparisons and the result is cast to int64: undefined in the reference,
    refused on both sides here (VF_ERR_NAN)."""
    x = np.linspace(-1, 1, 4096).astype(np.float32)
    x[1234] = np.nan
    t = TType([4096], F32)
    for q in (Elem.uniform(I8, F32, 0.01, 0, -127, 127),):
        for be in (gpu, oracle):
            with pytest.raises(Exception) as e:
                ContentAttr(x, t, ContentSetup(t).quantize(q)).fold(be)
            assert e.value.status == abi.VF_ERR_NAN
    # the context stays usable
    x[1234] = 0.0
    both(ContentAttr(x, t, ContentSetup(t).quantize(q)), gpu, oracle)


@pytest.mark.parametrize("dt", [F32, F16, BF16])
def test_fused_kernels_refuse_nan(gpu, oracle, dt):
    """The single-pass kernels (groups, long rows, convolution rows with and without a transposed copy-out; ranges
    derived from the data or supplied) report a NaN like the general path, and the context stays usable."""
    rng = np.random.default_rng(77)

    def nan_at(x, i):
        bad = x.copy()
        if dt == BF16:
            bad.reshape(-1)[i] = 0x7FC0
        else:
            bad.reshape(-1)[i] = np.nan
        return bad

    def conv(x):
        return x if dt == F32 else (x.astype(np.float16) if dt == F16 else bf16_bits(x))

    cases = []
    for shape in ((12, 64, 3, 3), (40, 256, 1, 1), (9, 3, 7, 7)):  # transposed rows, straight rows, the scalar kernel
        x = conv(rng.standard_normal(shape).astype(np.float32) * 0.05)
        ts, oshape = wl.conv_pipeline(shape, None, None)
        cases.append((shape, x, wl.spec_i8_sym(), ts, int(np.prod(oshape)), shape[0]))
    if dt != F32:
        x = conv(rng.standard_normal((3, 8192)).astype(np.float32) * 0.02)
        cases.append(((3, 8192), x, wl.spec_i8_sym(), [], 3 * 8192, 3))
        cases.append(((3, 8192), x, wl.spec_u4_group(128), [wl.t_bitpack()], 3 * 8192 // 2, 3 * 64))
    for shape, x, spec, ts, nbytes, units in cases:
        bad = nan_at(x, x.size * 2 // 3 + 5)
        for be in (gpu, oracle):
            assert _status(lambda: _quant_fold(be, shape, bad, spec, ts, nbytes, units)) == abi.VF_ERR_NAN, (shape, be)
        _same(_quant_fold(gpu, shape, x, spec, ts, nbytes, units), _quant_fold(oracle, shape, x, spec, ts, nbytes, units))
        if len(shape) == 4:  # the same through vf_fold with supplied parameters
            t = TType(list(shape), dt)
            q = Elem.per_axis(I8, F16, rng.uniform(1e-3, 1e-2, shape[0]).tolist(), [0] * shape[0], 0, -127, 127)
            for be in (gpu, oracle):
                assert _status(lambda: ContentAttr(bad, t, ContentSetup(t).quantize(q).reorder(abi.ORDER_NHWC)).fold(be)) == abi.VF_ERR_NAN
            both(ContentAttr(x, t, ContentSetup(t).quantize(q).reorder(abi.ORDER_NHWC)), gpu, oracle)


def test_device_time_of_a_call_is_reported_on_request(oracle):
    from vpux_plugin_b200.lib import Library
    lib = Library(device=0, timing=True)
    x = np.random.default_rng(3).standard_normal((64, 8192)).astype(np.float16)
    t = TType([64, 8192], F16)
    ContentAttr(x, t, ContentSetup(t).castElemType(F32).rescale(0.5)).fold(lib)
    assert 0.0 < lib.last_stats.device_ms < 1000.0
    plain = Library(device=0)
    ContentAttr(x, t, ContentSetup(t).castElemType(F32).rescale(0.5)).fold(plain)
    assert plain.last_stats.device_ms == 0.0


def test_quantize_fold_unusual_range_takes_general_path(gpu, oracle):
    """[-120, 120] is a range where fakeQuantize's tail is not the identity; the fused kernels decline it."""
    rng = np.random.default_rng(15)
    x = (rng.standard_normal((4, 2048)) * 0.02).astype(np.float16)
    spec = wl.spec_i8_sym()
    spec.qmin, spec.qmax = -120, 120
    args = ((4, 2048), x, spec, [], 4 * 2048, 4)
    got = _quant_fold(gpu, *args)
    assert gpu.last_stats.fused == 0
    _same(got, _quant_fold(oracle, *args))


def test_weights_table_random(gpu, oracle):
    rng = np.random.default_rng(16)
    oc = 300
    ws = rng.uniform(1e-4, 5e-2, oc)
    bias = (rng.standard_normal(oc) * 0.01).astype(np.float32)
    d, keep = wl.weights_table_desc(oc, ws, 576, bias)
    assert np.array_equal(gpu.weights_table(d, oc), oracle.weights_table(d, oc))
    counts = rng.integers(0, 577, oc).astype(np.int64)
    d, keep = wl.weights_table_desc(oc, ws, 576, bias, sparse_counts=counts, sparsity_step=80)
    tg, to = gpu.weights_table(d, oc), oracle.weights_table(d, oc)
    assert np.array_equal(tg, to)
    assert tg.reshape(oc, 4)[1, 0] == (counts[0] + 15) // 16 * 16
    # float activations: column 2 is the fp32 bit pattern, bias divided by the weight scale in fp32
    d = abi.WeightsTableDesc()
    fe = Elem(F16)
    we = Elem.per_axis(I8, F16, ws, np.zeros(oc), 0, -127, 127)
    d.in_elem, d.out_elem, d.weights_elem, d.oc = fe.pod(), fe.pod(), we.pod(), oc
    d.weights_ptr_step, d.sparsity_ptr_base = 64, abi.VF_SPARSITY_PTR_WHEN_NO_SPARSITY
    d.has_bias, d.bias, d.bias_mem_kind = 1, bias.ctypes.data, abi.VF_MEM_HOST
    assert np.array_equal(gpu.weights_table(d, oc), oracle.weights_table(d, oc))
    # a scale above 2^15 needs a post-shift: rejected
    d2, keep2 = wl.weights_table_desc(2, np.array([1e9, 1.0]), 16)
    assert _status(lambda: gpu.weights_table(d2, 2)) == abi.VF_ERR_RANGE
    assert _status(lambda: oracle.weights_table(d2, 2)) == abi.VF_ERR_RANGE
    d3, keep3 = wl.weights_table_desc(2, np.array([1.0, 1.0]), 24)
    assert _status(lambda: gpu.weights_table(d3, 2)) == abi.VF_ERR_ALIGNMENT
    assert _status(lambda: oracle.weights_table(d3, 2)) == abi.VF_ERR_ALIGNMENT


def test_pipelined_batches_defer_kernel_errors_to_the_next_synchronisation(oracle):
    """VF_OPT_ASYNC: device-resident batch calls return once enqueued; results equal the synchronous ones, a
    kernel-side failure is reported by synchronize() and does not stick to later calls."""
    import torch
    from vpux_plugin_b200.lib import Library
    lib = Library(device=0, pipelined=True)
    dev = torch.device("cuda", 0)
    oc = 300
    rng = np.random.default_rng(23)
    ws = rng.uniform(1e-4, 5e-2, oc)

    def job(scales):
        d, keep = wl.weights_table_desc(oc, scales, 576)
        tab = torch.full((oc * 4,), -1, dtype=torch.int32, device=dev)
        torch.cuda.synchronize()  # the fill runs on torch's stream, the library on its own
        jobs = (abi.WeightsTableJob * 1)()
        jobs[0].desc, jobs[0].table = d, tab.data_ptr()
        return jobs, tab, d, keep

    good = [job(ws) for _ in range(40)]  # many calls in flight before the first synchronisation
    for jobs, _, _, _ in good:
        lib.weights_table_batch(jobs, out_mem_kind=abi.VF_MEM_DEVICE)
    lib.synchronize()
    exp = oracle.weights_table(good[0][2], oc)
    for _, tab, _, _ in good:
        assert np.array_equal(tab.cpu().numpy(), exp)
    bad_scales = ws.copy()
    bad_scales[7] = 1e9  # needs a post-shift: the kernel flags it
    bad = job(bad_scales)
    lib.weights_table_batch(bad[0], out_mem_kind=abi.VF_MEM_DEVICE)  # returns: nothing has been checked yet
    assert _status(lib.synchronize) == abi.VF_ERR_RANGE
    again = job(ws)
    lib.weights_table_batch(again[0], out_mem_kind=abi.VF_MEM_DEVICE)
    lib.synchronize()
    assert np.array_equal(again[1].cpu().numpy(), exp)
    # a call that touches host memory synchronises by itself
    host_tab = lib.weights_table(good[0][2], oc)
    assert np.array_equal(host_tab, exp)
    lib.close()


def test_pipelined_fold_calls_defer_and_report_at_synchronisation(oracle):
    """VF_OPT_ASYNC: vf_fold over device memory returns once enqueued; results equal the oracle's after
    vf_ctx_synchronize, and what a kernel finds (a NaN in Quantize) is reported there, not by the call."""
    import torch
    from vpux_plugin_b200.lib import Library
    lib = Library(device=0, pipelined=True)
    dev = torch.device("cuda", 0)
    rng = np.random.default_rng(41)
    shape = [24, 64, 3, 3]
    t = TType(shape, F16)
    x = (rng.standard_normal(shape) * 0.05).astype(np.float16)
    n = x.size
    q = Elem.per_axis(I8, F16, rng.uniform(1e-3, 1e-2, shape[0]).tolist(), [0] * shape[0], 0, -127, 127)
    setups = [ContentSetup(t).quantize(q).reorder(abi.ORDER_NHWC), ContentSetup(t).reorder(abi.ORDER_NHWC),
              ContentSetup(t).castElemType(F32).rescale(0.5), ContentSetup(t).padWithZero([0, 0, 0, 0], [8, 0, 0, 0])]
    src = torch.from_numpy(x.view(np.uint8).reshape(-1)).to(dev)
    c, keep = abi.make_content(t, None, F16, False, abi.VF_MEM_DEVICE, ptr=src.data_ptr(), nbytes=n * 2)
    outs = []
    for s in setups:
        tr, k = s.transforms()
        _, _, nbytes = lib.infer_type(t, False, tr, k)
        dst = torch.full((nbytes,), 0xEE, dtype=torch.uint8, device=dev)
        outs.append((s, tr, k, dst, nbytes))
    torch.cuda.synchronize()
    for _ in range(2):
        for s, tr, k, dst, nbytes in outs:
            lib.fold(c, tr, k, dst.data_ptr(), nbytes, dst_mem_kind=abi.VF_MEM_DEVICE)
    lib.synchronize()
    for s, tr, k, dst, nbytes in outs:
        ref = ContentAttr(x, t, s).fold(oracle)
        assert np.array_equal(dst.cpu().numpy(), ref.bytes())
    bad = x.copy()
    bad.reshape(-1)[77] = np.nan
    src.copy_(torch.from_numpy(bad.view(np.uint8).reshape(-1)))
    torch.cuda.synchronize()
    s, tr, k, dst, nbytes = outs[0]
    lib.fold(c, tr, k, dst.data_ptr(), nbytes, dst_mem_kind=abi.VF_MEM_DEVICE)  # returns: nothing has been checked yet
    assert _status(lib.synchronize) == abi.VF_ERR_NAN
    src.copy_(torch.from_numpy(x.view(np.uint8).reshape(-1)))
    torch.cuda.synchronize()
    lib.fold(c, tr, k, dst.data_ptr(), nbytes, dst_mem_kind=abi.VF_MEM_DEVICE)
    lib.synchronize()
    assert np.array_equal(dst.cpu().numpy(), ContentAttr(x, t, s).fold(oracle).bytes())
    lib.close()


def test_pipelined_steps_run_through_the_job_table_area_many_times(gpu, oracle):
    """VF_OPT_ASYNC, 700 steps of quantize-fold + Sparsify/GetSparsityMap + weights tables of twelve convolution
    weights without a synchronisation in between: the job tables of the batched launches go through the context's
    1 MiB area about five times (it starts over only after the calls that still read it have finished), and the
    queue of deferred compressed sizes fills up once. The outputs of the last step equal those of a single step,
    which are checked against the oracle."""
    import torch
    from vpux_plugin_b200.lib import Library
    lib = Library(device=0, pipelined=True)
    dev = torch.device("cuda", 0)
    rng = np.random.default_rng(77)
    shapes = [[32, 16, 3, 3], [64, 64, 1, 1], [16, 3, 7, 7], [48, 32, 3, 3], [128, 256, 1, 1], [8, 16, 1, 1],
              [24, 64, 3, 3], [256, 128, 1, 1], [40, 16, 3, 3], [64, 512, 1, 1], [16, 32, 1, 1], [96, 48, 3, 3]]
    n_t = len(shapes)
    qjobs, sjobs, tjobs = (abi.QuantJob * n_t)(), (abi.SparsifyJob * n_t)(), (abi.WeightsTableJob * n_t)()
    spec = wl.spec_i8_sym()
    keep, outs, xs = [], [], []
    for j, shape in enumerate(shapes):
        x = (rng.standard_normal(shape) * 0.05 * (rng.random(shape) < 0.5)).astype(np.float16)
        x[0] = np.abs(x[0]) + 0.01  # one dense channel
        xs.append(x)
        ts, oshape = wl.conv_pipeline(shape, pad_ic_to=16 if shape[1] == 3 else None)
        tr = abi.make_transforms(ts)
        oc, work = oshape[0], oshape[1] * oshape[2] * oshape[3]
        src = torch.from_numpy(x.view(np.uint8).reshape(-1)).to(dev)
        codes = torch.empty(oc * work, dtype=torch.uint8, device=dev)
        sc = torch.empty(oc, dtype=torch.float64, device=dev)
        o = abi.QuantOutputs()
        o.mem_kind, o.scales = abi.VF_MEM_DEVICE, sc.data_ptr()
        c, k = abi.make_content(TType(shape, F16), None, ptr=src.data_ptr(), nbytes=x.nbytes, mem_kind=abi.VF_MEM_DEVICE)
        qj = qjobs[j]
        qj.base, qj.spec, qj.t, qj.n = c, spec, tr, len(ts)
        qj.dst, qj.dst_bytes, qj.dst_mem_kind, qj.outs = codes.data_ptr(), codes.numel(), abi.VF_MEM_DEVICE, o
        row = (work + 127) // 128 * 16
        cap = oc * ((work + 15) // 16 * 16)
        cc, kc = abi.make_content(TType(list(oshape), I8, abi.ORDER_NHWC), None, ptr=codes.data_ptr(), nbytes=codes.numel(), mem_kind=abi.VF_MEM_DEVICE)
        data = torch.zeros(cap, dtype=torch.uint8, device=dev)
        mp = torch.empty(oc * row, dtype=torch.uint8, device=dev)
        cnt = torch.empty(oc, dtype=torch.int64, device=dev)
        sj = sjobs[j]
        sj.content, sj.data, sj.data_bytes = cc, data.data_ptr(), cap
        sj.map, sj.map_bytes, sj.counts = mp.data_ptr(), oc * row, cnt.data_ptr()
        bias = torch.from_numpy((rng.standard_normal(oc) * 0.01).astype(np.float32)).to(dev)
        d, kd = wl.weights_table_desc(oc, np.ones(oc), 0)
        d.has_bias, d.bias, d.bias_mem_kind = 1, bias.data_ptr(), abi.VF_MEM_DEVICE
        d.nnz_counts, d.nnz_mem_kind = cnt.data_ptr(), abi.VF_MEM_DEVICE
        d.sparsity_ptr_base, d.sparsity_ptr_step = 0, row
        tab = torch.empty(oc * 4, dtype=torch.int32, device=dev)
        tj = tjobs[j]
        tj.desc, tj.table = d, tab.data_ptr()
        tj.weights_scales, tj.scales_mem_kind = sc.data_ptr(), abi.VF_MEM_DEVICE
        keep += [tr, src, k, ts, kc, kd, bias]
        outs.append({"codes": codes, "scales": sc, "data": data, "map": mp, "counts": cnt, "table": tab, "oshape": oshape})

    def step():
        lib.quantize_fold_batch(qjobs)
        lib.sparsify_batch(sjobs, out_mem_kind=abi.VF_MEM_DEVICE)
        lib.weights_table_batch(tjobs, out_mem_kind=abi.VF_MEM_DEVICE)

    def snapshot():
        return [{k: v.cpu().numpy().copy() for k, v in o.items() if k != "oshape"} for o in outs]

    step()
    lib.synchronize()
    first = snapshot()
    sizes = [int(sjobs[j].data_written) for j in range(n_t)]
    for j, (x, o, f) in enumerate(zip(xs, outs, first)):  # the single step against the oracle
        oshape = o["oshape"]
        oc, work = oshape[0], oshape[1] * oshape[2] * oshape[3]
        ts, _ = wl.conv_pipeline(shapes[j], pad_ic_to=16 if shapes[j][1] == 3 else None)
        cx, kx = abi.make_content(TType(shapes[j], F16), x)
        ref_codes, ref_scales = np.zeros(oc * work, np.uint8), np.zeros(oc, np.float64)
        ro = abi.QuantOutputs()
        ro.mem_kind, ro.scales = abi.VF_MEM_HOST, ref_scales.ctypes.data
        assert oracle.quantize_fold(cx, spec, abi.make_transforms(ts), len(ts), ref_codes, oc * work, ro) == oc * work
        assert np.array_equal(f["codes"], ref_codes), j
        assert np.array_equal(f["scales"], ref_scales), j
        q = Elem.per_axis(I8, F16, ref_scales, np.zeros(oc, np.int64), 0, -127, 127)
        c, k = abi.make_content(TType(list(oshape), q, abi.ORDER_NHWC), f["codes"].view(np.int8), storage_dtype=I8)
        od, om, ocnt = np.zeros(f["data"].size, np.uint8), np.zeros(f["map"].size, np.uint8), np.zeros(oc, np.int64)
        w = oracle.sparsify(c, od, om, ocnt)
        assert w == sizes[j] and np.array_equal(f["data"][:w], od[:w]) and np.array_equal(f["map"], om) and np.array_equal(f["counts"], ocnt), j
    for o in outs:
        for k, v in o.items():
            if k != "oshape":
                v.fill_(0 if k == "data" else 0x5A if v.dtype == torch.uint8 else 0)
    torch.cuda.synchronize()
    for _ in range(700):
        step()
    lib.synchronize()
    for j, (a, b) in enumerate(zip(snapshot(), first)):
        for k in a:
            assert np.array_equal(a[k], b[k]), (j, k)
        assert int(sjobs[j].data_written) == sizes[j]
    lib.close()


def test_batches_of_seventy_small_tensors(gpu, oracle):
    """Seventy tensors of 1-39 channels per call: Sparsify + GetSparsityMap + counts, then weights tables with sparse
    pointers from those counts (more jobs than any network-shaped case of this suite, most of them a few rows)."""
    rng = np.random.default_rng(70)
    n_t = 70
    sjobs, tjobs = (abi.SparsifyJob * n_t)(), (abi.WeightsTableJob * n_t)()
    keep, expect, bufs, tabs, texp = [], [], [], [], []
    for j in range(n_t):
        oc, ic, k = int(rng.integers(1, 40)), 16 * int(rng.integers(1, 5)), int(rng.choice([1, 3]))
        shape = [oc, ic, k, k]
        n, work = int(np.prod(shape)), ic * k * k
        x = (rng.integers(1, 100, n) * (rng.random(n) < 0.5)).astype(np.int8)
        c, kc = abi.make_content(TType(shape, I8), x)
        row, cap = (work + 127) // 128 * 16, n + 16 * oc
        od, om, ocnt = np.zeros(cap, np.uint8), np.zeros(oc * row, np.uint8), np.zeros(oc, np.int64)
        w = oracle.sparsify(c, od, om, ocnt)
        gd, gm, gc = np.full(cap, 0xAB, np.uint8), np.full(oc * row, 0xAB, np.uint8), np.full(oc, -1, np.int64)
        sjobs[j].content, sjobs[j].data, sjobs[j].data_bytes = c, gd.ctypes.data, cap
        sjobs[j].map, sjobs[j].map_bytes, sjobs[j].counts = gm.ctypes.data, gm.nbytes, gc.ctypes.data
        expect.append((w, od, om, ocnt))
        bufs.append((gd, gm, gc))
        d, kd = wl.weights_table_desc(oc, rng.uniform(1e-4, 5e-2, oc), 0, None, sparse_counts=ocnt, sparsity_step=row)
        texp.append(oracle.weights_table(d, oc))
        tab = np.full(oc * 4, -1, np.int32)
        tjobs[j].desc, tjobs[j].table = d, tab.ctypes.data
        tabs.append(tab)
        keep += [c, kc, x, kd]
    gpu.sparsify_batch(sjobs)
    for j, ((w, od, om, ocnt), (gd, gm, gc)) in enumerate(zip(expect, bufs)):
        assert sjobs[j].data_written == w and np.array_equal(gd[:w], od[:w]) and np.array_equal(gm, om) and np.array_equal(gc, ocnt), j
    gpu.weights_table_batch(tjobs)
    for j, (tab, ref) in enumerate(zip(tabs, texp)):
        assert np.array_equal(tab, ref), j


def test_weights_table_batch(gpu, oracle):
    """Many tables per call (dense and sparse pointers, with and without bias, 1..2500 channels); weight scales
    either inside the descriptor or as a separate FP64 array; one launch for all rows."""
    rng = np.random.default_rng(17)
    ocs = [1, 16, 64, 300, 1000, 2500, 33]
    jobs = (abi.WeightsTableJob * len(ocs))()
    tables, expect, keep = [], [], []
    for j, oc in enumerate(ocs):
        ws = rng.uniform(1e-4, 5e-2, oc)
        bias = (rng.standard_normal(oc) * 0.01).astype(np.float32) if j % 2 == 0 else None
        counts = rng.integers(0, 577, oc).astype(np.int64) if j % 3 == 1 else None
        d, k = wl.weights_table_desc(oc, ws, 576, bias, sparse_counts=counts, sparsity_step=80 if counts is not None else 0)
        expect.append(oracle.weights_table(d, oc))
        tab = np.full(oc * 4, -1, np.int32)
        jobs[j].desc, jobs[j].table = d, tab.ctypes.data
        if j >= 4:  # scales passed beside the descriptor; the descriptor's own values must then be ignored
            wrong = abi.Elem.per_axis(I8, F16, np.full(oc, 123.0), np.zeros(oc, np.int64), 0, -127, 127)
            jobs[j].desc.weights_elem = wrong.pod()
            sc = np.ascontiguousarray(ws, np.float64)
            jobs[j].weights_scales, jobs[j].scales_mem_kind = sc.ctypes.data, abi.VF_MEM_HOST
            keep += [wrong, sc]
        tables.append(tab)
        keep += [d, k]
    l0 = gpu.launch_count
    gpu.weights_table_batch(jobs)
    assert gpu.launch_count - l0 == 2  # all prefix sums + all rows
    for j, (tab, exp) in enumerate(zip(tables, expect)):
        assert np.array_equal(tab, exp), j
    # an invalid job ends the call and is marked
    jobs[2].desc.weights_ptr_step = 24
    assert _status(lambda: gpu.weights_table_batch(jobs)) == abi.VF_ERR_ALIGNMENT


# ---------------------------------------------------------------------------------------------------------
# RelocateWeightsTable (relocate_weights_table.cpp:203-292)
def _relocate_case(rng, oc, n_cl, compressed, chan, tail=0):
    tab = np.zeros((oc + tail, 4), np.int32)
    tab[:oc, 0] = np.arange(oc) * (int(rng.integers(1, 512)) * 16)
    no_sparsity = (rng.integers(0, 8, oc) == 0) & (np.arange(oc) >= 2)  # rows 0 and 1 give the pointer steps
    tab[:oc, 1] = np.where(no_sparsity, 0xFFFFFF, np.arange(oc) * int(rng.integers(0, 64)))
    tab[:, 2:] = rng.integers(-(1 << 31), 1 << 31, (oc + tail, 2), dtype=np.int64).astype(np.int32)
    bounds = sorted(int(v) for v in rng.choice(np.arange(1, oc), n_cl - 1, replace=False)) if n_cl > 1 else []
    offs = [0] + bounds
    comp = None
    if compressed:
        comp = {"axis": 0, "numElems": rng.integers(0, 5000, oc + chan), "alignment": int(rng.choice([0, 16, 32]))}
    t = TType([oc + tail, 1, 1, 4], abi.VF_DT_I32)
    s = ContentSetup(t).relocateWeightsTablePointers([int(v) for v in rng.integers(0, 1 << 22, n_cl)],
                                                     int(rng.integers(0, 1 << 22)), offs, oc * 16,
                                                     int(rng.choice([4, 8, 16])), comp, chan)
    return ContentAttr(tab, t, s)


@pytest.mark.gpu
@pytest.mark.parametrize("oc,n_cl,compressed,chan,tail", [
    (1, 1, False, 0, 0), (2, 1, False, 3, 0), (64, 2, False, 0, 0), (64, 4, True, 0, 0), (1000, 8, True, 0, 3),
    (4096, 6, False, 0, 0), (4096, 1, True, 17, 0), (8192, 8, True, 0, 1)])
def test_relocate_weights_table(gpu, oracle, oc, n_cl, compressed, chan, tail):
    rng = np.random.default_rng(oc * 31 + n_cl)
    both(_relocate_case(rng, oc, n_cl, compressed, chan, tail), gpu, oracle)


@pytest.mark.gpu
def test_relocate_weights_table_cluster_walk(gpu, oracle):
    """Cluster offsets that repeat or go backwards: the reference moves on by one cluster per channel at most."""
    rng = np.random.default_rng(5)
    tab = np.zeros((12, 4), np.int32)
    tab[:, 0] = np.arange(12) * 32
    tab[:, 1] = np.arange(12) * 4
    t = TType([12, 1, 1, 4], abi.VF_DT_I32)
    for offs in ([0, 0, 5], [0, 3, 3, 3], [0, 7, 2], [4, 0, 6], [0, 20], [0, 1, 2, 3, 4, 5, 6, 7]):
        ptrs = [int(v) for v in rng.integers(0, 1 << 20, len(offs))]
        both(ContentAttr(tab, t, ContentSetup(t).relocateWeightsTablePointers(ptrs, 9, offs, 12 * 16, 16)), gpu, oracle)


@pytest.mark.gpu
def test_relocate_weights_table_errors(gpu, oracle):
    from vpux_plugin_b200.lib import VfoldError
    t = TType([4, 1, 1, 4], abi.VF_DT_I32)
    tab = np.zeros((4, 4), np.int32)
    tab[:, 0] = np.arange(4) * (1 << 29)  # weightsPtr + 3 steps leaves int32: checked_cast throws
    s = ContentSetup(t).relocateWeightsTablePointers([1 << 30], 0, [0], 64, 16)
    for be in (gpu, oracle):
        with pytest.raises(Exception) as e:
            ContentAttr(tab, t, s).fold(be)
        assert e.value.status == abi.VF_ERR_CHECKED_CAST
    with pytest.raises(VfoldError) as e:  # too few numElems for the channels
        ContentAttr(tab, t, ContentSetup(t).relocateWeightsTablePointers(
            [0], 0, [0], 64, 16, {"numElems": [1, 2, 3]})).fold(gpu)
    assert e.value.status == abi.VF_ERR_SHAPE
    with pytest.raises(VfoldError) as e:  # a table larger than the constant
        ContentAttr(tab, t, ContentSetup(t).relocateWeightsTablePointers([0], 0, [0], 80, 16)).fold(gpu)
    assert e.value.status == abi.VF_ERR_SHAPE
    f = TType([4, 1, 1, 4], F32)
    with pytest.raises(VfoldError) as e:  # not a table of 32-bit integers
        ContentAttr(tab.astype(np.float32), f, ContentSetup(f).relocateWeightsTablePointers([0], 0, [0], 64, 16)).fold(gpu)
    assert e.value.status == abi.VF_ERR_UNSUPPORTED


# ---------------------------------------------------------------------------------------------------------
# Reverse / Broadcast / ExpandDilated / ScalarMultInverse / ChangeShapeAndElemType and Reshape's type rules
@pytest.mark.gpu
@pytest.mark.parametrize("dt", [F32, F16, abi.VF_DT_BF16, I8, U8])
@pytest.mark.parametrize("axis", [0, 1, 2])
def test_reverse(gpu, oracle, dt, axis):
    rng = np.random.default_rng(axis * 7 + dt)
    shape = [3, 5, 4, 7]
    t = TType(shape, dt)
    x = rng.integers(0, 200, shape).astype(abi.DTYPE_NUMPY.get(dt, np.uint16))
    both(ContentAttr(x, t, ContentSetup(t).reverse(axis)), gpu, oracle)
    if dt == F32:  # storage f32 under an f16 type: the values are converted on the way
        both(ContentAttr(x * 0.37, t, ContentSetup(t).castElemType(F16).reverse(axis)), gpu, oracle)
    if dt == U8:
        q = Elem.uniform(U8, F32, 0.1, 3, 0, 255)
        both(ContentAttr(x, t, ContentSetup(t).castElemType(q).reorder(abi.ORDER_NHWC).reverse(axis)), gpu, oracle)


@pytest.mark.gpu
def test_reverse_errors(gpu):
    from vpux_plugin_b200.lib import VfoldError
    t = TType([2, 3, 4], abi.VF_DT_I32)
    with pytest.raises(VfoldError) as e:
        ContentAttr(np.zeros(24, np.int32), t, ContentSetup(t).reverse(0)).fold(gpu)
    assert e.value.status == abi.VF_ERR_UNSUPPORTED
    t = TType([2, 3, 4], F32)
    with pytest.raises(VfoldError) as e:
        ContentAttr(np.zeros(24, np.float32), t, ContentSetup(t).reverse(2)).fold(gpu)
    assert e.value.status == abi.VF_ERR_INVALID_ARG


@pytest.mark.gpu
@pytest.mark.parametrize("order", [0x1234, abi.ORDER_NHWC, 0x4321])
@pytest.mark.parametrize("axis,value", [(0, 6), (1, 9), (2, 4), (3, 10)])
def test_broadcast(gpu, oracle, order, axis, value):
    rng = np.random.default_rng(axis + order)
    shape = [2, 3, 4, 5]
    t = TType(shape, F16)
    x = rng.standard_normal(shape).astype(np.float16)
    s = ContentSetup(t).reorder(order).broadcast(axis, value)
    if value % shape[axis]:
        from vpux_plugin_b200.lib import VfoldError
        with pytest.raises(VfoldError) as e:
            ContentAttr(x, t, s).fold(gpu)
        assert e.value.status == abi.VF_ERR_SHAPE
        with pytest.raises(Exception):
            ContentAttr(x, t, s).fold(oracle)
    else:
        both(ContentAttr(x, t, s), gpu, oracle)
    one = TType([1, 1, 1, 1], F32)
    both(ContentAttr(np.array([2.5], np.float32), one, ContentSetup(one).broadcast(axis, value), is_splat=True), gpu, oracle)


@pytest.mark.gpu
@pytest.mark.parametrize("dil", [(1, 1), (2, 3), (3, 1)])
def test_expand_dilated(gpu, oracle, dil):
    rng = np.random.default_rng(dil[0] * 5 + dil[1])
    shape = [4, 6, 3, 5]
    t = TType(shape, U8)
    x = rng.integers(0, 256, shape).astype(np.uint8)
    both(ContentAttr(x, t, ContentSetup(t).expandDilated(dil)), gpu, oracle)
    q = Elem.uniform(U8, F32, 0.05, 131, 0, 255)  # the gaps hold the zero point
    both(ContentAttr(x, t, ContentSetup(t).castElemType(q).expandDilated(dil)), gpu, oracle)
    qa = Elem.per_axis(U8, F32, [0.1, 0.2, 0.3, 0.4], [1, 20, 3, 40], 0, 0, 255)  # ... of their output channel
    both(ContentAttr(x, t, ContentSetup(t).castElemType(qa).expandDilated(dil)), gpu, oracle)
    both(ContentAttr(x, t, ContentSetup(t).castElemType(qa).reorder(abi.ORDER_NHWC).expandDilated(dil)), gpu, oracle)
    tf = TType(shape, F16)
    both(ContentAttr(np.array([1.5], np.float16), tf, ContentSetup(tf).expandDilated(dil), is_splat=True), gpu, oracle)


@pytest.mark.gpu
@pytest.mark.parametrize("dt,np_dt", [(U8, np.uint8), (F16, np.float16), (F32, np.float32)])
@pytest.mark.parametrize("shape,dil", [([5, 7, 3, 3], (2, 2)), ([33, 17, 5, 1], (4, 2)), ([3, 3, 1, 7], (1, 5)), ([16, 31, 3, 3], (6, 6)),
                                       ([61, 37, 3, 3], (2, 2)), ([64, 40, 2, 2], (3, 2)), ([7, 9, 9, 9], (8, 8))])
def test_expand_dilated_vector_steps(gpu, oracle, dt, np_dt, shape, dil):
    """Output sizes that are not multiples of the 16-byte store unit, rows shorter and longer than one unit, plane
    counts of one partial chunk, several chunks with a ragged last one, and planes too large to be staged."""
    rng = np.random.default_rng(sum(shape) + dil[0])
    x = rng.integers(1, 120, shape).astype(np_dt)
    t = TType(shape, dt)
    out = both(ContentAttr(x, t, ContentSetup(t).expandDilated(dil)), gpu, oracle)
    dky, dkx = (shape[2] - 1) * dil[0] + 1, (shape[3] - 1) * dil[1] + 1
    want = np.zeros(shape[:2] + [dky, dkx], np_dt)
    want[:, :, ::dil[0], ::dil[1]] = x
    assert np.array_equal(out.values(np_dt).reshape(want.shape), want)


@pytest.mark.gpu
def test_scalar_mult_inverse(gpu, oracle):
    from vpux_plugin_b200.lib import VfoldError
    rng = np.random.default_rng(12)
    t = TType([64, 129], F32)
    x = (rng.standard_normal((64, 129)) * 100).astype(np.float32)
    x[x == 0] = 1.0
    both(ContentAttr(x, t, ContentSetup(t).scalarMultInverse()), gpu, oracle)
    h = TType([64, 129], F16)
    both(ContentAttr(x.astype(np.float16), h, ContentSetup(h).scalarMultInverse()), gpu, oracle)
    for bad in (0.0, np.inf, np.nan, 1e-40):
        y = x.copy()
        y[17, 5] = bad
        for be in (gpu, oracle):
            with pytest.raises(Exception) as e:
                ContentAttr(y, t, ContentSetup(t).scalarMultInverse()).fold(be)
            assert e.value.status == abi.VF_ERR_NOT_NORMAL
    # the context is usable afterwards
    both(ContentAttr(x, t, ContentSetup(t).scalarMultInverse()), gpu, oracle)


@pytest.mark.gpu
def test_reshape_type_rules(gpu, oracle):
    """changeShape (core/type_interfaces.cpp:208-231): a non-identity order survives a reshape of the same rank
    and rejects another rank; a per-axis type follows its axis into the new shape."""
    rng = np.random.default_rng(13)
    t = TType([2, 3, 4, 5], F16)
    x = rng.standard_normal([2, 3, 4, 5]).astype(np.float16)
    a = both(ContentAttr(x, t, ContentSetup(t).reorder(abi.ORDER_NHWC).reshape([6, 1, 4, 5]).reorder(0x1234)), gpu, oracle)
    assert a.type.order in (0, 0x1234)
    mid = ContentAttr(x, t, ContentSetup(t).reorder(abi.ORDER_NHWC).reshape([6, 1, 4, 5])).infer(gpu)[0]
    assert mid.order == abi.ORDER_NHWC
    for be in (gpu, oracle):
        with pytest.raises(Exception) as e:
            ContentAttr(x, t, ContentSetup(t).reorder(abi.ORDER_NHWC).reshape([6, 20])).fold(be)
        assert e.value.status == abi.VF_ERR_SHAPE
    q = Elem.per_axis(U8, F32, [0.5, 0.25, 0.125], [1, 2, 3], 1, 0, 255)
    tu = TType([2, 3, 4, 5], U8)
    u = rng.integers(0, 256, [2, 3, 4, 5]).astype(np.uint8)
    s = ContentSetup(tu).castElemType(q)
    out = both(ContentAttr(u, tu, s.reshape([2, 3, 20]).dequantize()), gpu, oracle)
    assert out.type.shape[:3] == [2, 3, 20]
    moved = ContentAttr(u, tu, s.reshape([1, 2, 3, 20])).infer(gpu)[0]
    assert moved.elem.axis == 2
    for be in (gpu, oracle):  # the axis cannot be found in the new shape and no longer fits it
        with pytest.raises(Exception) as e:
            ContentAttr(u, tu, s.reshape([6, 4, 5])).fold(be)
        assert e.value.status == abi.VF_ERR_SHAPE


@pytest.mark.gpu
def test_fold_into_device_memory_matches_fold_into_host_memory(gpu):
    """With a device destination the last transformation writes its output there directly; the bytes are the
    ones a host destination receives, also when the destination is the base buffer itself (in place)."""
    import torch
    rng = np.random.default_rng(77)
    t = TType([6, 8, 3, 5], F32)
    x = rng.standard_normal(t.shape).astype(np.float32)
    q = Elem.uniform(I8, F32, 0.05, 0, -127, 127)
    setups = [ContentSetup(t).quantize(q), ContentSetup(t).reorder(abi.ORDER_NHWC), ContentSetup(t).padWithZero([0, 0, 1, 1], [2, 0, 0, 1]),
              ContentSetup(t).subview([1, 2, 0, 1], [3, 4, 3, 2]), ContentSetup(t).castElemType(F16).reverse(1),
              ContentSetup(t).rescale(0.5).add(1.0), ContentSetup(t).castElemType(F16), ContentSetup(t).swizzleConstant(3, abi.VF_ARCH_NPU40XX),
              ContentSetup(t).transpose(0x2143), ContentSetup(t).broadcast(0, 12), ContentSetup(t).scalarMultInverse()]
    xd = torch.from_numpy(x).cuda()
    for s in setups:
        attr = ContentAttr(x, t, s)
        ref = attr.fold(gpu)
        tr, n = s.transforms()
        for in_place in (False, True):
            src = xd.clone()
            c, keep = abi.make_content(t, None, F32, False, abi.VF_MEM_DEVICE, ptr=src.data_ptr(), nbytes=x.nbytes)
            cap = max(ref.written, 1)
            if in_place:
                if cap > x.nbytes:
                    continue
                dst = src.view(torch.uint8).reshape(-1)
            else:
                dst = torch.full((cap + 64,), 0xAB, dtype=torch.uint8, device="cuda")
                torch.cuda.synchronize()  # the fill runs on torch's stream, the library on its own
            written, ftype = gpu.fold(c, tr, n, dst.data_ptr(), cap, dst_mem_kind=abi.VF_MEM_DEVICE)
            torch.cuda.synchronize()
            out = dst.cpu().numpy().reshape(-1)
            assert written == ref.written and ftype == ref.type
            assert np.array_equal(out[:written], ref.bytes()), (s.names(), in_place)
            if not in_place:
                assert (out[cap:] == 0xAB).all()


@pytest.mark.gpu
@pytest.mark.parametrize("dt", [abi.VF_DT_I1, abi.VF_DT_U4, abi.VF_DT_I4])
@pytest.mark.parametrize("shape,off,sub", [
    ([1001], [37], [555]),
    ([7, 13, 5, 3], [1, 2, 0, 1], [5, 9, 5, 2]),
    ([3, 64, 9, 32], [1, 16, 2, 8], [2, 32, 5, 16]),
    ([2, 3, 4, 5, 6], [0, 1, 1, 2, 3], [2, 2, 2, 3, 3]),
    ([64, 4096], [3, 1024], [40, 2047]),
])
def test_subview_of_sub_byte_storage(gpu, oracle, dt, shape, off, sub):
    """subview.cpp:20-160 (subByteTransform): bit fields gathered into a freshly packed buffer; the oracle walks
    element by element, the kernel packs one output byte per thread."""
    bits = 1 if dt == abi.VF_DT_I1 else 4
    n = int(np.prod(shape))
    rng = np.random.default_rng(n + bits)
    raw = rng.integers(0, 256, (n * bits + 7) // 8, dtype=np.uint8)
    t = TType(shape, dt)
    attr = ContentAttr(raw, t, ContentSetup(t).subview(off, sub), storage_dtype=dt)
    out = both(attr, gpu, oracle)
    assert out.type.shape == sub and out.written == (int(np.prod(sub)) * bits + 7) // 8
    # independent check against numpy on the unpacked values
    per = 8 // bits
    vals = ((raw[:, None] >> (np.arange(per) * bits)) & ((1 << bits) - 1)).reshape(-1)[:n].reshape(shape)
    want = vals[tuple(slice(o, o + s) for o, s in zip(off, sub))].reshape(-1)
    got = ((out.bytes()[:, None] >> (np.arange(per) * bits)) & ((1 << bits) - 1)).reshape(-1)[:want.size]
    assert np.array_equal(got, want)
    # followed by a conversion to bytes (the shape the reference's lit cases have)
    conv = ContentAttr(raw, t, ContentSetup(t).subview(off, sub).convertElemType(U8 if dt == abi.VF_DT_U4 else I8),
                       storage_dtype=dt)
    both(conv, gpu, oracle)


@pytest.mark.gpu
def test_rank_six_layout_transformations(gpu, oracle):
    rng = np.random.default_rng(66)
    shape = [2, 3, 2, 4, 3, 5]
    t = TType(shape, F16)
    x = rng.standard_normal(shape).astype(np.float16)
    for s in (ContentSetup(t).reorder(0x132546), ContentSetup(t).transpose(0x654321),
              ContentSetup(t).padWithZero([0, 1, 0, 0, 2, 0], [1, 0, 0, 3, 0, 1]),
              ContentSetup(t).subview([1, 0, 1, 2, 0, 1], [1, 3, 1, 2, 3, 3]),
              ContentSetup(t).reorder(0x213465).subview([0, 1, 0, 0, 1, 2], [2, 2, 2, 4, 2, 3]).reorder(0x123456).reshape([2, 2, 8, 6]),
              ContentSetup(t).reverse(2), ContentSetup(t).broadcast(2, 6).reorder(0x654321)):
        both(ContentAttr(x, t, s), gpu, oracle)


@pytest.mark.gpu
@pytest.mark.parametrize("dt", [F32, F16])
@pytest.mark.parametrize("qmin,qmax,storage", [(0, 255, U8), (-128, 127, I8), (-127, 127, I8), (0, 15, U8), (-120, 120, I8)])
@pytest.mark.parametrize("inner", [512, 3000])  # 3000: rows long enough for the by-rows kernel, with a ragged last chunk
def test_general_quantize_on_rounding_boundaries(gpu, oracle, dt, qmin, qmax, storage, inner):
    """Quantize with given parameters (quantize.cpp:108-212): values on and next to the .5 boundaries of every
    level, where the fast evaluation must hand over to the exact sequence; [-120, 120] is a range whose
    fakeQuantize tail is not the identity (all elements take the exact sequence)."""
    rng = np.random.default_rng(qmax * 3 + dt)
    oc = 24
    scales = rng.uniform(0.003, 0.9, oc)
    zps = rng.integers(qmin, qmax + 1, oc) if qmin == 0 else np.zeros(oc, np.int64)
    levels = qmax - qmin
    x = np.empty((oc, inner), np.float64)
    for c in range(oc):
        lo = (qmin - zps[c]) * scales[c]
        step = (qmax - qmin) * scales[c] / levels
        k = rng.integers(-2, levels + 2, inner)
        x[c] = lo + (k + 0.5) * step
    x32 = x.astype(np.float32)
    near = np.stack([np.nextafter(x32, np.float32(np.inf)), x32, np.nextafter(x32, np.float32(-np.inf))], 0)
    data = np.concatenate([near[i] for i in range(3)], axis=1)  # [oc, 3 * inner]
    np_dt = np.float32 if dt == F32 else np.float16
    data = data.astype(np_dt)
    t = TType([oc, 3 * inner], dt)
    q = Elem.per_axis(storage, F32, scales.tolist(), [int(z) for z in zps], 0, qmin, qmax)
    both(ContentAttr(data, t, ContentSetup(t).quantize(q)), gpu, oracle)
    qt = Elem.uniform(storage, F32, float(scales[0]), int(zps[0]), qmin, qmax)
    both(ContentAttr(data, t, ContentSetup(t).quantize(qt)), gpu, oracle)
    special = data.copy()
    special[0, :8] = [np.inf, -np.inf, 1e30 if dt == F32 else 6e4, -1e30 if dt == F32 else -6e4, 0.0, -0.0, 1e-30 if dt == F32 else 6e-8, 3.0]
    both(ContentAttr(special, t, ContentSetup(t).quantize(q)), gpu, oracle)


@pytest.mark.gpu
@pytest.mark.parametrize("storage,np_dt,qmin,qmax", [(I8, np.int8, -128, 127), (U8, np.uint8, 0, 255)])
@pytest.mark.parametrize("shape,axis", [([6, 9000], 0), ([3, 5, 8200], 1), ([4, 16, 8], 0), ([2, 70000], 1)])
def test_general_dequantize_by_rows(gpu, oracle, storage, np_dt, qmin, qmax, shape, axis):
    """Dequantize (dequantize.cpp:42-108) of every code, with rows inside the quantized axis long and short, whole
    and ragged against the kernel's chunk size; per-axis and per-tensor."""
    rng = np.random.default_rng(shape[-1] + axis)
    n = shape[axis]
    x = rng.integers(qmin, qmax + 1, shape).astype(np_dt)
    x.reshape(-1)[:qmax - qmin + 1] = np.arange(qmin, qmax + 1).astype(np_dt)
    t = TType(shape, storage)
    if n <= 64:
        qa = Elem.per_axis(storage, F32, rng.uniform(1e-3, 2.0, n).tolist(), [int(z) for z in rng.integers(qmin, qmax + 1, n)], axis, qmin, qmax)
        both(ContentAttr(x, t, ContentSetup(t).castElemType(qa).dequantize()), gpu, oracle)
    qt = Elem.uniform(storage, F16, 0.0123456789, int(rng.integers(qmin, qmax + 1)), qmin, qmax)
    both(ContentAttr(x, t, ContentSetup(t).castElemType(qt).dequantize()), gpu, oracle)
    for zp in ((1 << 30) - 1, 1 << 30, -(1 << 30), (1 << 33) + 5, -(1 << 40)):  # around and beyond the 32-bit difference
        qz = Elem.uniform(storage, F32, 0.37, zp, qmin, qmax)
        both(ContentAttr(x, t, ContentSetup(t).castElemType(qz).dequantize()), gpu, oracle)


@pytest.mark.gpu
@pytest.mark.parametrize("dt", [F32, F16, BF16])
@pytest.mark.parametrize("storage,qmin,qmax", [(I8, -128, 127), (U8, 0, 255), (U8, 0, 15)])
def test_general_quantize_by_rows_ranges_and_special_values(gpu, oracle, dt, storage, qmin, qmax):
    """Quantize with given parameters over rows of several lengths (shorter than, equal to and ragged against a warp's
    unit), scales from far below to far above the bounds of the packed sequence (those rows take fakeQuantize as
    written), data well outside the quantized range, infinities, zeros and denormals; NaN is refused."""
    rng = np.random.default_rng(qmax + dt)
    for inner, oc in ((8, 40), (512, 12), (1032, 7), (4096 + 24, 3)):
        mags = np.array([1e-36, 1e-33, 3e-31, 1e-20, 1e-3, 0.05, 7.0, 1e20, 1e28, 4e29, 1e33])
        if dt == F16:
            mags = np.array([1e-36, 1e-9, 1e-5, 1e-3, 0.05, 7.0, 200.0, 1e20])
        scales = rng.choice(mags, oc) * rng.uniform(0.5, 2.0, oc)
        zps = rng.integers(qmin, qmax + 1, oc)
        x = rng.standard_normal((oc, inner)) * (scales * (qmax - qmin) * 0.7)[:, None] + ((((qmin + qmax) / 2) - zps) * scales)[:, None]
        x = np.clip(x, -3e38, 3e38)
        x[0, :8] = [np.inf, -np.inf, 3e38, -3e38, 0.0, -0.0, 1e-45, -1e-40]
        t = TType([oc, inner], dt)
        if dt == F32:
            data = x.astype(np.float32)
        elif dt == F16:
            data = np.clip(x, -65504, 65504).astype(np.float16)
            data[0, :2] = [np.inf, -np.inf]
        else:
            data = bf16_bits(x.astype(np.float32))
        q = Elem.per_axis(storage, F32, scales.tolist(), [int(z) for z in zps], 0, qmin, qmax)
        both(ContentAttr(data, t, ContentSetup(t).quantize(q)), gpu, oracle)
        qt = Elem.uniform(storage, F32, float(scales[-1]), int(zps[-1]), qmin, qmax)
        both(ContentAttr(data, t, ContentSetup(t).quantize(qt)), gpu, oracle)
    bad = data.copy()
    bad.reshape(-1)[5000 % bad.size] = np.float32(np.nan) if dt != BF16 else 0x7FC1
    for be in (gpu, oracle):
        assert _status(lambda: ContentAttr(bad, t, ContentSetup(t).quantize(q)).fold(be)) == abi.VF_ERR_NAN
    both(ContentAttr(data, t, ContentSetup(t).quantize(q)), gpu, oracle)  # the context stays usable


@pytest.mark.gpu
@pytest.mark.parametrize("storage,np_dt,qmin,qmax", [(I8, np.int8, -128, 127), (U8, np.uint8, 0, 255)])
def test_general_dequantize_scales_next_to_rounding_boundaries(gpu, oracle, storage, np_dt, qmin, qmax):
    """Dequantize is the FP64 product rounded to fp32. Scales built so that (code - zp) * scale lies within an FP64
    rounding error of the midpoint of two floats for one code per row, scales whose products are denormal or
    overflow, and zero points around 2^20, where the fp32 evaluation has to hand over to the FP64 one."""
    rng = np.random.default_rng(7 + qmax)
    rows = 96
    scales = np.empty(rows, np.float64)
    zps = rng.integers(qmin, qmax + 1, rows)
    for r in range(rows):
        n = 2 * (r % 60) + 3  # an odd multiplier: n * scale sits on the midpoint, up to the rounding of the scale
        s_hi = np.float64(np.float32(rng.uniform(1e-3, 2.0)))
        p = n * s_hi
        ulp = 2.0 ** (np.floor(np.log2(p)) - 23)
        tie = (np.floor(p / ulp) + 0.5) * ulp
        scales[r] = s_hi - (p - tie) / n
        code = int(zps[r]) + n
        if code > qmax:
            zps[r] = qmax - n if qmax - n >= qmin else qmin
    scales[-6:] = [1e-42, 3e-39, 2.9e36, 1e38, 1.0000000001, 0.1]
    zps[-3:] = [(1 << 20) - 1, 1 << 20, -(1 << 20) - 7]
    shape = [rows, 1544]
    x = rng.integers(qmin, qmax + 1, shape).astype(np_dt)
    x[:, :qmax - qmin + 1] = np.arange(qmin, qmax + 1).astype(np_dt)[None, :]
    t = TType(shape, storage)
    qa = Elem.per_axis(storage, F32, scales.tolist(), [int(z) for z in zps], 0, qmin, qmax)
    both(ContentAttr(x, t, ContentSetup(t).castElemType(qa).dequantize()), gpu, oracle)
    t2 = TType([2, rows, 264], storage)
    qa2 = Elem.per_axis(storage, F32, scales.tolist(), [int(z) for z in zps], 1, qmin, qmax)
    both(ContentAttr(np.ascontiguousarray(x[:, :528].reshape(rows, 2, 264).transpose(1, 0, 2)), t2,
                     ContentSetup(t2).castElemType(qa2).dequantize()), gpu, oracle)


@pytest.mark.gpu
def test_layout_kernels_beyond_two_to_the_31_elements(gpu):
    """More than 2^31 elements switch the layout kernels to 64-bit index arithmetic: a transpose applied twice and a
    pad followed by the view of the original region both give the input back (checked on the device)."""
    import torch
    rows, cols = 65544, 32768  # 2.15e9 u8 elements
    x = torch.randint(0, 256, (rows, cols), dtype=torch.uint8, device="cuda")
    n = rows * cols
    t = TType([rows, cols], U8)

    def run(ttype, src, setup, out_elems):
        c, keep = abi.make_content(ttype, None, U8, False, abi.VF_MEM_DEVICE, ptr=src.data_ptr(), nbytes=src.numel())
        dst = torch.empty(out_elems, dtype=torch.uint8, device="cuda")
        tr, k = setup.transforms()
        written, ftype = gpu.fold(c, tr, k, dst.data_ptr(), out_elems, dst_mem_kind=abi.VF_MEM_DEVICE)
        assert written == out_elems
        return dst, ftype

    y, ty = run(t, x, ContentSetup(t).transpose(0x21), n)
    assert ty.shape == [cols, rows]
    assert torch.equal(y.view(cols, rows)[:7, :9], x[:9, :7].t())
    z, tz = run(ty, y, ContentSetup(ty).transpose(0x21), n)
    assert torch.equal(z.view(rows, cols), x)
    del y, z
    p, tp = run(t, x, ContentSetup(t).padWithZero([3, 0], [0, 5]), (rows + 3) * (cols + 5))
    assert tp.shape == [rows + 3, cols + 5]
    pv = p.view(rows + 3, cols + 5)
    assert int(pv[:3].max()) == 0 and int(pv[:, cols:].max()) == 0
    v, tv = run(tp, p, ContentSetup(tp).subview([3, 0], [rows, cols]), n)
    assert torch.equal(v.view(rows, cols), x)
