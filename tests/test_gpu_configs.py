"""The five benchmark workloads end to end on the GPU against the CPU oracle.

C1–C3 are compared in full. C4 and C5 run at their full sizes on the device (device-resident synthetic
weights); since the oracle cannot fold 13–140 GB in test time, randomly chosen rows are regenerated on the host
from (seed, tensor, offset), folded by the oracle and compared with the corresponding slice of the GPU output,
next to size-independent properties (code ranges, scale/zero-point consistency).
"""
import ctypes as C

import numpy as np
import pytest

from vpux_plugin_b200 import abi, workloads as wl
from vpux_plugin_b200.abi import Elem, TType

pytestmark = pytest.mark.gpu


def _outs(units, mem_kind=abi.VF_MEM_HOST, f16=False, u4=False):
    o = abi.QuantOutputs()
    o.mem_kind = mem_kind
    res = {"scales": np.zeros(units, np.float64), "zps": np.zeros(units, np.int64)}
    o.scales, o.zps = res["scales"].ctypes.data, res["zps"].ctypes.data
    if f16:
        res["f16"] = np.zeros(units, np.uint16)
        o.scales_f16 = res["f16"].ctypes.data
    if u4:
        res["u4"] = np.zeros((units + 1) // 2, np.uint8)
        o.zps_u4_packed = res["u4"].ctypes.data
    return o, res


def _fold_conv(be, spec, x, qspec, ts, oshape):
    t = TType(list(spec.shape), spec.dtype)
    c, keep = abi.make_content(t, x)
    out_bytes = int(np.prod(oshape))
    dst = np.zeros(out_bytes, np.uint8)
    o, res = _outs(spec.shape[0])
    w = be.quantize_fold(c, qspec, abi.make_transforms(ts), len(ts), dst, out_bytes, o)
    res["codes"] = dst[:w]
    return res


def test_c1_single_conv(gpu, oracle):
    spec = wl.c1_tensors()[0]
    x = oracle.synth_fill(spec.synth_spec(wl.SEEDS["c1"]), spec.numel)
    ts, oshape = wl.conv_pipeline(spec.shape, pad_oc_to=64)
    a = _fold_conv(gpu, spec, x, wl.spec_u8_asym(), ts, oshape)
    b = _fold_conv(oracle, spec, x, wl.spec_u8_asym(), ts, oshape)
    assert gpu.last_stats.fused == 1
    for k in b:
        assert np.array_equal(a[k], b[k]), k
    assert a["codes"].size == 64 * 3 * 3 * 64
    assert (a["codes"].reshape(64, -1)[60:] == 0).all()  # padded channels are zero: the codes are plain u8


def _resnet_inputs(oracle, sparse):
    specs = wl.resnet50_tensors(sparse=sparse)
    seed = wl.SEEDS["c3" if sparse else "c2"]
    return specs, seed, [oracle.synth_fill(s.synth_spec(seed), s.numel) for s in specs]


def _resnet_batch(gpu, specs, xs):
    """All 54 tensors through ONE vf_quantize_fold_batch call (host buffers)."""
    jobs = (abi.QuantJob * len(specs))()
    keep, res = [], []
    qspec = wl.spec_i8_sym()
    for j, (s, x) in enumerate(zip(specs, xs)):
        ts, oshape = wl.conv_pipeline(s.shape, pad_ic_to=16 if s.name == "stem" else None)
        tr = abi.make_transforms(ts)
        c, k = abi.make_content(TType(list(s.shape), s.dtype), x)
        dst = np.zeros(int(np.prod(oshape)), np.uint8)
        o, r = _outs(s.shape[0])
        jb = jobs[j]
        jb.base, jb.spec, jb.t, jb.n = c, qspec, tr, len(ts)
        jb.dst, jb.dst_bytes, jb.dst_mem_kind, jb.outs = dst.ctypes.data, dst.size, abi.VF_MEM_HOST, o
        r["codes"] = dst
        r["oshape"] = oshape
        keep += [tr, k, ts]
        res.append(r)
    gpu.quantize_fold_batch(jobs)
    for j in range(len(specs)):
        assert jobs[j].status == 0 and jobs[j].dst_written == res[j]["codes"].size
    return res


def test_c2_resnet50_quantize_reorder_pad_and_weights_tables(gpu, oracle_mt):
    specs, seed, xs = _resnet_inputs(oracle_mt, sparse=False)
    got = _resnet_batch(gpu, specs, xs)
    assert gpu.last_stats.fused == 1
    assert gpu.last_stats.kernels_launched <= 4  # conv-row kernel + long-row kernel(s), not one per tensor
    total_oc = 0
    for s, x, g in zip(specs, xs, got):
        ts, oshape = wl.conv_pipeline(s.shape, pad_ic_to=16 if s.name == "stem" else None)
        ref = _fold_conv(oracle_mt, s, x, wl.spec_i8_sym(), ts, oshape)
        for k in ref:
            assert np.array_equal(g[k], ref[k]), (s.name, k)
        oc = s.shape[0]
        total_oc += oc
        bias = oracle_mt.synth_fill(wl.bias_for(seed, s.tensor_id, oc), oc)
        step = oshape[1] * oshape[2] * oshape[3]
        d, keep = wl.weights_table_desc(oc, g["scales"], step, bias)
        assert np.array_equal(gpu.weights_table(d, oc), oracle_mt.weights_table(d, oc)), s.name
    assert total_oc == 27_560


def test_c3_resnet50_sparse_weights(gpu, oracle_mt):
    specs, seed, xs = _resnet_inputs(oracle_mt, sparse=True)
    got = _resnet_batch(gpu, specs, xs)
    dense_channels = 0
    for s, x, g in zip(specs, xs, got):
        oshape = g["oshape"]
        oc, work = oshape[0], oshape[1] * oshape[2] * oshape[3]
        q = Elem.per_axis(abi.VF_DT_I8, abi.VF_DT_F16, g["scales"], g["zps"], 0, -127, 127)
        t = TType(list(oshape), q, abi.ORDER_NHWC)
        c, keep = abi.make_content(t, g["codes"].view(np.int8), storage_dtype=abi.VF_DT_I8)
        cap = oc * ((work + 15) // 16 * 16)
        row = (work + 127) // 128 * 16
        out = []
        for be in (gpu, oracle_mt):
            data, mp, cnt = np.zeros(cap, np.uint8), np.zeros(oc * row, np.uint8), np.zeros(oc, np.int64)
            w = be.sparsify(c, data, mp, cnt)
            out.append((w, data[:w].copy(), mp, cnt))
        assert out[0][0] == out[1][0], s.name
        for a, b in zip(out[0][1:], out[1][1:]):
            assert np.array_equal(a, b), s.name
        cnt = out[0][3]
        dense_channels += int((cnt > 0.9 * work).sum())
        # compaction keeps memory order: expanding with the bitmap restores the codes
        codes = g["codes"].view(np.int8).reshape(oc, work)
        bits = np.unpackbits(out[0][2].reshape(oc, row), axis=1, bitorder="little")[:, :work].astype(bool)
        assert np.array_equal(bits, codes != 0)
        # weights table with sparse pointers: column 0 = running sum of 16-byte aligned set sizes
        bias = oracle_mt.synth_fill(wl.bias_for(seed, s.tensor_id, oc), oc)
        d, keep2 = wl.weights_table_desc(oc, g["scales"], 0, bias, sparse_counts=cnt, sparsity_step=row)
        tab = gpu.weights_table(d, oc)
        assert np.array_equal(tab, oracle_mt.weights_table(d, oc)), s.name
        offs = np.concatenate([[0], np.cumsum((cnt + 15) // 16 * 16)[:-1]])
        assert np.array_equal(tab.reshape(oc, 4)[:, 0], offs)
    assert 0.05 * 27_560 < dense_channels < 0.16 * 27_560  # about one channel in ten is left dense


# ---------------------------------------------------------------------------------------------------------
# C4 / C5 at full size, device resident
# ---------------------------------------------------------------------------------------------------------
def _device_batch(gpu, torch, tensors, seed, qspec, transforms, is_group, row_ranges=None):
    dev = torch.device("cuda", 0)
    jobs = (abi.QuantJob * len(tensors))()
    tr = abi.make_transforms(transforms)
    keep, outs = [tr], []
    for j, t in enumerate(tensors):
        r0, r1 = (0, t.rows) if row_ranges is None else row_ranges[j]
        rows, cols = r1 - r0, t.row_len
        n, es = rows * cols, abi.DTYPE_BITS[t.dtype] // 8
        src = torch.empty(n * es, dtype=torch.uint8, device=dev)
        gpu.synth_fill_device(t.synth_spec(seed, r0 * cols), src.data_ptr(), n)
        o = abi.QuantOutputs()
        o.mem_kind = abi.VF_MEM_DEVICE
        if is_group:
            units = n // 128
            dst = torch.empty(n // 2, dtype=torch.uint8, device=dev)
            s16 = torch.empty(units, dtype=torch.int16, device=dev)
            z4 = torch.empty((units + 1) // 2, dtype=torch.uint8, device=dev)
            o.scales_f16, o.zps_u4_packed = s16.data_ptr(), z4.data_ptr()
            side = {"f16": s16, "u4": z4}
        else:
            dst = torch.empty(n, dtype=torch.uint8, device=dev)
            dq = torch.empty(n, dtype=torch.int16, device=dev)
            sc = torch.empty(rows, dtype=torch.float64, device=dev)
            o.dequant, o.dequant_dtype, o.dequant_bytes, o.scales = dq.data_ptr(), abi.VF_DT_F16, n * 2, sc.data_ptr()
            side = {"dequant": dq, "scales": sc}
        c, k = abi.make_content(TType([rows, cols], t.dtype), None, ptr=src.data_ptr(), nbytes=n * es, mem_kind=abi.VF_MEM_DEVICE)
        jb = jobs[j]
        jb.base, jb.spec, jb.t, jb.n = c, qspec, tr, len(transforms)
        jb.dst, jb.dst_bytes, jb.dst_mem_kind, jb.outs = dst.data_ptr(), dst.numel(), abi.VF_MEM_DEVICE, o
        keep += [src, k]
        outs.append((dst, side, r0, rows, cols))
    gpu.quantize_fold_batch(jobs)
    return outs, keep


def test_c4_llama2_7b_full_size_spot_checked(gpu, oracle):
    import torch
    tensors = wl.llama2_7b_tensors()
    seed = wl.SEEDS["c4"]
    outs, keep = _device_batch(gpu, torch, tensors, seed, wl.spec_u4_group(128), [wl.t_bitpack()], True)
    assert gpu.last_stats.fused == 1 and gpu.last_stats.kernels_launched == 1  # 225 tensors, one launch
    rng = np.random.default_rng(44)
    for _ in range(160):
        j = int(rng.integers(0, len(tensors)))
        t = tensors[j]
        dst, side, r0, rows, cols = outs[j]
        r = int(rng.integers(0, rows))
        x = oracle.synth_fill(t.synth_spec(seed, r * cols), cols)
        c, k = abi.make_content(TType([1, cols], t.dtype), x)
        ref = np.zeros(cols // 2, np.uint8)
        o, res = _outs(cols // 128, f16=True, u4=(cols // 128) % 2 == 0)
        oracle.quantize_fold(c, wl.spec_u4_group(128), abi.make_transforms([wl.t_bitpack()]), 1, ref, ref.size, o)
        g0 = r * cols // 128
        assert np.array_equal(dst[r * cols // 2:(r + 1) * cols // 2].cpu().numpy(), ref), (t.name, r)
        assert np.array_equal(side["f16"][g0:g0 + cols // 128].cpu().numpy().view(np.uint16), res["f16"]), (t.name, r)
        if "u4" in res:
            assert np.array_equal(side["u4"][g0 // 2:(g0 + cols // 128) // 2].cpu().numpy(), res["u4"]), (t.name, r)
    # size-independent property over a whole tensor: the extremes of every group land on the ends of the code
    # range. (When -min/scale is an exact x.5 tie — e.g. max == -min on the fp16 grid — the zero point rounds
    # away and the minimum itself sits on a tie that rounds to code 1, so the low end is 0 or 1.)
    dst, side, _, rows, cols = outs[0]
    nib = dst[: 4096 * 64]
    lo, hi = (nib & 0xF).view(-1, 64), (nib >> 4).view(-1, 64)
    gmin = torch.minimum(lo.min(dim=1).values, hi.min(dim=1).values)
    gmax = torch.maximum(lo.max(dim=1).values, hi.max(dim=1).values)
    assert int(gmin.max()) <= 1 and int(gmax.min()) >= 14
    assert float((gmin == 0).float().mean()) > 0.99 and float((gmax == 15).float().mean()) > 0.99
    del outs, keep
    torch.cuda.empty_cache()


def test_c5_llama3_70b_slab_full_size_spot_checked(gpu, oracle):
    import torch
    from vpux_plugin_b200.lib import plan_shards
    tensors = wl.llama3_70b_tensors()
    seed = wl.SEEDS["c5"]
    rb, re_ = plan_shards(1, 8, [t.nbytes for t in tensors], [t.rows for t in tensors], 1)
    slab = 5  # the slab of rank 5 of an 8-GPU job
    ranges = [(int(rb[i, slab]), int(re_[i, slab])) for i in range(len(tensors))]
    outs, keep = _device_batch(gpu, torch, tensors, seed, wl.spec_i8_sym(abi.VF_DT_F16), [], False, ranges)
    assert gpu.last_stats.fused == 1 and gpu.last_stats.kernels_launched == 2  # short-row and long-row launch
    rng = np.random.default_rng(55)
    for _ in range(120):
        j = int(rng.integers(0, len(tensors)))
        t = tensors[j]
        dst, side, r0, rows, cols = outs[j]
        r = int(rng.integers(0, rows))
        x = oracle.synth_fill(t.synth_spec(seed, (r0 + r) * cols), cols)
        c, k = abi.make_content(TType([1, cols], t.dtype), x)
        ref = np.zeros(cols, np.uint8)
        o, res = _outs(1)
        dq = np.zeros(cols, np.uint16)
        o.dequant, o.dequant_dtype, o.dequant_bytes = dq.ctypes.data, abi.VF_DT_F16, dq.nbytes
        oracle.quantize_fold(c, wl.spec_i8_sym(abi.VF_DT_F16), abi.make_transforms([]), 0, ref, ref.size, o)
        assert np.array_equal(dst[r * cols:(r + 1) * cols].cpu().numpy(), ref), (t.name, r)
        assert np.array_equal(side["dequant"][r * cols:(r + 1) * cols].cpu().numpy().view(np.uint16), dq), (t.name, r)
        assert side["scales"][r].item() == res["scales"][0]
    # round-trip property on a whole tensor: dequantized value == code * fp16-rounded scale step, |code| <= 127,
    # and every row reaches |code| == 127
    dst, side, _, rows, cols = outs[0]
    codes = dst.view(torch.int8).view(rows, cols)
    assert int(codes.abs().max(dim=1).values.min()) == 127 and int(codes.min()) >= -127
    deq = side["dequant"].view(torch.float16).view(rows, cols).double()
    assert torch.allclose(deq, codes.double() * side["scales"].view(-1, 1), rtol=2 ** -10, atol=1e-7)
    del outs, keep
    torch.cuda.empty_cache()


# ---------------------------------------------------------------------------------------------------------
# whole-output digests: every byte of a full-size output is compared, through the 128-bit content hash
# ---------------------------------------------------------------------------------------------------------
def _mix64(z):
    z = z ^ (z >> np.uint64(33))
    z = z * np.uint64(0xFF51AFD7ED558CCD)
    z = z ^ (z >> np.uint64(33))
    z = z * np.uint64(0xC4CEB9FE1A85EC53)
    return z ^ (z >> np.uint64(33))


def _mulhi64(x, y):
    """High half of the 128-bit product of two uint64 arrays."""
    m = np.uint64(0xFFFFFFFF)
    s32 = np.uint64(32)
    xl, xh, yl, yh = x & m, x >> s32, y & m, y >> s32
    ll, lh, hl, hh = xl * yl, xl * yh, xh * yl, xh * yh
    mid = (ll >> s32) + (lh & m) + (hl & m)
    return hh + (lh >> s32) + (hl >> s32) + (mid >> s32)


def hash128_host(buf):
    """vf_content_hash restated with numpy: the buffer as 16-byte vectors (a, b) of two 8-byte words (missing bytes
    zero), vector i keyed with (i + 1) * K; two differently keyed 64 x 64 -> 128 bit products per vector, each folded
    (low ^ high) and summed; the length mixed in last. For hashing the oracle's outputs."""
    b = np.ascontiguousarray(buf).view(np.uint8).reshape(-1)
    n = b.size
    if n % 16:
        b = np.concatenate([b, np.zeros(16 - n % 16, np.uint8)])
    v = b.view(np.uint64).reshape(-1, 2)
    a_, b_ = v[:, 0], v[:, 1]
    K, K2, K3 = np.uint64(0x9E3779B97F4A7C15), np.uint64(0xD6E8FEB86659FD93), np.uint64(0xA0761D6478BD642F)
    s32 = np.uint64(32)
    with np.errstate(over="ignore"):
        k = np.arange(1, a_.size + 1, dtype=np.uint64) * K
        ks = (k << s32) | (k >> s32)
        x, y = a_ ^ k, b_ ^ ks ^ K2
        h1 = ((x * y) ^ _mulhi64(x, y)).sum(dtype=np.uint64)
        x2, y2 = (a_ ^ K3) + ks, (b_ ^ K2) + k
        h2 = ((x2 * y2) ^ _mulhi64(x2, y2)).sum(dtype=np.uint64)
        return int(_mix64(h1 ^ np.uint64(n))), int(_mix64(h2 + np.uint64(n)))


def _device_hash(gpu, t):
    from vpux_plugin_b200.lib import content_hash
    n = int(t.numel() * t.element_size())
    c, k = abi.make_content(TType([n], abi.VF_DT_U8), None, abi.VF_DT_U8, False, abi.VF_MEM_DEVICE, ptr=t.data_ptr(), nbytes=n)
    return content_hash(gpu, c)


def test_hash_restatement_matches_the_device_hash(gpu):
    import torch
    rng = np.random.default_rng(5)
    for n in (1, 7, 8, 4096, 100003):
        x = rng.integers(0, 256, n).astype(np.uint8)
        t = torch.from_numpy(x).cuda()
        assert _device_hash(gpu, t) == hash128_host(x), n


def test_c4_whole_tensor_digest(gpu, oracle_mt):
    """Every byte of the folded lm_head (32000 x 4096 fp16 -> 65.5 MB of packed codes, 1 M scales and zero points):
    the device hash of the GPU's outputs against the same hash of the oracle's."""
    import torch
    t = wl.llama2_7b_tensors()[-1]
    assert t.name == "lm_head"
    seed = wl.SEEDS["c4"]
    outs, keep = _device_batch(gpu, torch, [t], seed, wl.spec_u4_group(128), [wl.t_bitpack()], True)
    dst, side, _, rows, cols = outs[0]
    n = rows * cols
    x = oracle_mt.synth_fill(t.synth_spec(seed, 0), n)
    c, k = abi.make_content(TType([rows, cols], t.dtype), x)
    ref = np.zeros(n // 2, np.uint8)
    o, res = _outs(n // 128, f16=True, u4=True)
    oracle_mt.quantize_fold(c, wl.spec_u4_group(128), abi.make_transforms([wl.t_bitpack()]), 1, ref, ref.size, o)
    assert _device_hash(gpu, dst) == hash128_host(ref)
    assert _device_hash(gpu, side["f16"]) == hash128_host(res["f16"])
    assert _device_hash(gpu, side["u4"]) == hash128_host(res["u4"])


@pytest.mark.parametrize("name,slab", [("l0.k", 0), ("l0.q", 3), ("l0.down", 7)])
def test_c5_whole_slab_digest(gpu, oracle_mt, name, slab):
    """One whole output-channel slab per row width of the per-channel kernel (8192 columns on 64 and 128 threads'
    rows, 28672 columns on 256): codes, dequantized fp16 copy and scales, every byte through the digest."""
    import torch
    from vpux_plugin_b200.lib import plan_shards
    tensors = wl.llama3_70b_tensors(layers=1)
    t = [x for x in tensors if x.name == name][0]
    rb, re_ = plan_shards(1, 8, [t.nbytes], [t.rows], 1)
    r0, r1 = int(rb[0, slab]), int(re_[0, slab])
    seed = wl.SEEDS["c5"]
    outs, keep = _device_batch(gpu, torch, [t], seed, wl.spec_i8_sym(abi.VF_DT_F16), [], False, [(r0, r1)])
    dst, side, _, rows, cols = outs[0]
    n = rows * cols
    x = oracle_mt.synth_fill(t.synth_spec(seed, r0 * cols), n)
    c, k = abi.make_content(TType([rows, cols], t.dtype), x)
    ref = np.zeros(n, np.uint8)
    o, res = _outs(rows)
    dq = np.zeros(n, np.uint16)
    o.dequant, o.dequant_dtype, o.dequant_bytes = dq.ctypes.data, abi.VF_DT_F16, dq.nbytes
    oracle_mt.quantize_fold(c, wl.spec_i8_sym(abi.VF_DT_F16), abi.make_transforms([]), 0, ref, ref.size, o)
    assert _device_hash(gpu, dst) == hash128_host(ref)
    assert _device_hash(gpu, side["dequant"]) == hash128_host(dq)
    assert _device_hash(gpu, side["scales"]) == hash128_host(res["scales"])


def test_c5_first_and_last_rows_of_every_slab(gpu, oracle):
    """The rows at both ends of all eight output-channel slabs of one tensor of each shape."""
    import torch
    from vpux_plugin_b200.lib import plan_shards
    tensors = wl.llama3_70b_tensors(layers=1)
    seed = wl.SEEDS["c5"]
    for t in [x for x in tensors if x.name in ("l0.q", "l0.k", "l0.gate", "l0.down", "lm_head")]:
        rb, re_ = plan_shards(1, 8, [t.nbytes], [t.rows], 1)
        cols = t.row_len
        for slab in range(8):
            r0, r1 = int(rb[0, slab]), int(re_[0, slab])
            for a, b in ((r0, r0 + 2), (r1 - 2, r1)):
                outs, keep = _device_batch(gpu, torch, [t], seed, wl.spec_i8_sym(abi.VF_DT_F16), [], False, [(a, b)])
                dst, side, _, rows, _ = outs[0]
                x = oracle.synth_fill(t.synth_spec(seed, a * cols), rows * cols)
                c, k = abi.make_content(TType([rows, cols], t.dtype), x)
                ref = np.zeros(rows * cols, np.uint8)
                o, res = _outs(rows)
                dq = np.zeros(rows * cols, np.uint16)
                o.dequant, o.dequant_dtype, o.dequant_bytes = dq.ctypes.data, abi.VF_DT_F16, dq.nbytes
                oracle.quantize_fold(c, wl.spec_i8_sym(abi.VF_DT_F16), abi.make_transforms([]), 0, ref, ref.size, o)
                assert np.array_equal(dst.cpu().numpy(), ref), (t.name, slab, a)
                assert np.array_equal(side["dequant"].cpu().numpy().view(np.uint16), dq), (t.name, slab, a)
                assert np.array_equal(side["scales"].cpu().numpy(), res["scales"]), (t.name, slab, a)
