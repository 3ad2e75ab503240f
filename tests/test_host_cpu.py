"""Host-side tests that need no GPU: the C ABI library loads and exports what include/vfold.h declares, the
pure-host entry points (type inference, shard planning, status strings) work, the oracle reproduces its
committed golden digests, and the multi-rank sharding logic assembles bit-identical results (gloo, 2 ranks)."""
import ctypes as C
import hashlib
import json
import os
import re
import sys

import numpy as np
import pytest

import reference_cases as rc
from vpux_plugin_b200 import abi, workloads as wl
from vpux_plugin_b200.abi import Elem, TType
from vpux_plugin_b200.const import ContentAttr, ContentSetup

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    from vpux_plugin_b200 import lib
    header = open(os.path.join(ROOT, "include", "vfold.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    names = sorted(set(re.findall(r"\b(vf_[a-z0-9_]+)\s*\(", header)))
    assert "vf_fold" in names and "vf_weights_table" in names and len(names) >= 18
    L = lib.raw()
    for n in names:
        assert hasattr(L, n), f"{n} declared in vfold.h but not exported by libvfold.so"
    assert L.vf_abi_version() == 1
    assert L.vf_status_string(abi.VF_ERR_ZERO_POINTS) == b"zero points are not all equal"


def test_context_creation_fails_loudly_without_a_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    from vpux_plugin_b200.lib import Library, VfoldError
    with pytest.raises(VfoldError) as e:
        Library(device=0)
    assert e.value.status == abi.VF_ERR_NO_DEVICE
    assert "no CPU path" in str(e.value)


class _HostOnly:
    """infer_type from libvfold.so (pure host) behind the backend interface of the reference cases."""

    def infer_type(self, *a, **k):
        from vpux_plugin_b200 import lib
        return lib.infer_type(*a, **k)


def _random_setups(rng):
    F32, F16, I8, U8 = abi.VF_DT_F32, abi.VF_DT_F16, abi.VF_DT_I8, abi.VF_DT_U8
    shape = [int(rng.integers(1, 6)) for _ in range(4)]
    shape[1] *= 8
    t = TType(shape, F16)
    q_ax = Elem.per_axis(I8, F16, rng.uniform(0.01, 0.1, shape[0]), np.full(shape[0], 3), 0, -127, 127)
    q_un = Elem.uniform(U8, F16, 0.02, 128, 0, 255)
    s = ContentSetup(t)
    yield t, s.quantize(q_ax).reorder(abi.ORDER_NHWC).padWithZero([0, 0, 0, 0], [2, 3, 0, 0])
    yield t, s.castElemType(q_ax).padWithZero([1, 0, 0, 0], [0, 0, 1, 0]).reorder(abi.ORDER_NHWC)
    yield t, s.castElemType(q_un).dequantize().rescale(2.0).add(1.0)
    yield t, s.quantize(q_un).getSparsityMap()
    yield t, s.quantize(q_un).bitPack(4)
    yield t, s.castElemType(q_ax).subview([0, 0, 0, 0], [1, shape[1], shape[2], shape[3]]).dequantize()
    yield t, s.transpose(0x2143).reshape([int(np.prod(shape))])
    yield t, s.quantize(q_un).sparsify(True, rng.integers(0, 5, shape[0]))
    yield t, s.memPermute(abi.ORDER_NHWC, 0x1342)


def test_infer_type_matches_oracle(oracle):
    rng = np.random.default_rng(0)
    host = _HostOnly()
    for _ in range(20):
        for t, setup in _random_setups(rng):
            tr, n = setup.transforms()
            a = host.infer_type(t, False, tr, n)
            b = oracle.infer_type(t, False, tr, n)
            assert a[0] == b[0] and a[1] == b[1] and a[2] == b[2], (setup.names(), a, b)


@pytest.mark.parametrize("bad,status", [
    (lambda t: ContentSetup(t).dequantize(), abi.VF_ERR_NOT_QUANTIZED),
    (lambda t: ContentSetup(t).bitPack(8), abi.VF_ERR_UNSUPPORTED),
    (lambda t: ContentSetup(t).padWithZero([0, 0], [0, 0]), abi.VF_ERR_SHAPE),
    (lambda t: ContentSetup(t).reorder(0x1224), abi.VF_ERR_INVALID_ARG),
    (lambda t: ContentSetup(t).quantize(Elem.uniform(abi.VF_DT_I4, abi.VF_DT_F16, 1.0, 0, -8, 7)), abi.VF_ERR_UNSUPPORTED),
])
def test_infer_type_errors_match_oracle(oracle, bad, status):
    t = TType([2, 8, 1, 1], abi.VF_DT_F16)
    tr, n = bad(t).transforms()
    for be in (_HostOnly(), oracle):
        with pytest.raises(Exception) as e:
            be.infer_type(t, False, tr, n)
        assert e.value.status == status


def test_plan_shards_properties():
    from vpux_plugin_b200.lib import plan_shards
    ts = wl.llama2_7b_tensors()
    nbytes = [t.nbytes for t in ts]
    rows = [t.rows for t in ts]
    for world in (1, 2, 4, 8):
        rb, re_ = plan_shards(0, world, nbytes, rows)
        owned = (re_ > rb).sum(axis=1)
        assert (owned == 1).all()  # every tensor on exactly one rank, whole
        load = np.array([sum(nbytes[i] for i in range(len(ts)) if re_[i, r] > rb[i, r]) for r in range(world)])
        assert load.sum() == sum(nbytes)
        assert load.max() - load.min() <= max(nbytes)  # LPT bound
    ts = wl.llama3_70b_tensors(layers=2)
    rows = [t.rows for t in ts]
    rb, re_ = plan_shards(1, 8, [t.nbytes for t in ts], rows, row_align=16)
    for i, r in enumerate(rows):
        assert rb[i, 0] == 0 and re_[i, 7] == r
        assert (rb[i, 1:] == re_[i, :-1]).all()  # contiguous, disjoint, complete
        assert (rb[i] % 16 == 0).all()


def test_oracle_matches_committed_golden_digests():
    sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
    import make_golden
    want = json.load(open(os.path.join(ROOT, "tests", "golden", "oracle_golden.json")))
    assert make_golden.build() == want


def test_resnet50_shape_set_matches_the_workload_definition():
    shapes = wl.resnet50_shapes()
    assert len(shapes) == 54
    conv = sum(int(np.prod(s)) for _, s in shapes[:-1])
    assert conv == 23_454_912 and conv + 2_048_000 == 25_502_912
    assert sum(s[0] for _, s in shapes) == 27_560
    assert sum(t.numel for t in wl.llama2_7b_tensors()) == 6_607_077_376
    assert sum(t.numel for t in wl.llama3_70b_tensors()) == 70_552_387_584


# ---------------------------------------------------------------------------------------------------------
# two ranks over gloo: each rank folds its shard (with the CPU oracle standing in for the device), rank 0
# assembles and compares with the unsharded result
# ---------------------------------------------------------------------------------------------------------
def _rank_main(rank, world, port, q):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import torch
    from oracle import Oracle
    from vpux_plugin_b200.lib import plan_shards
    cpu = Oracle()
    ts = [wl.TensorSpec(f"t{i}", (64 + 32 * i, 512), abi.VF_DT_F16, 0.02, i, outlier_mult=20.0, outlier_log2=10) for i in range(5)]
    seed = wl.SEEDS["c4"]
    digests = []
    for mode in (0, 1):
        rb, re_ = plan_shards(mode, world, [t.nbytes for t in ts], [t.rows for t in ts], 8)
        pieces = []
        for i, t in enumerate(ts):
            r0, r1 = int(rb[i, rank]), int(re_[i, rank])
            if r1 <= r0:
                continue
            rows, cols = r1 - r0, t.row_len
            x = cpu.synth_fill(t.synth_spec(seed, r0 * cols), rows * cols)  # slab regenerated from its offset
            tt = abi.TType([rows, cols], t.dtype)
            c, keep = abi.make_content(tt, x)
            dst = np.zeros(rows * cols // 2, np.uint8)
            cpu.quantize_fold(c, wl.spec_u4_group(128), abi.make_transforms([wl.t_bitpack()]), 1, dst, dst.size)
            pieces.append((i, r0, dst))
        gathered = [None] * world
        dist.all_gather_object(gathered, pieces)
        if rank == 0:
            h = hashlib.sha256()
            for i, r0, dst in sorted((p for g in gathered for p in g), key=lambda p: (p[0], p[1])):
                h.update(dst.tobytes())
            digests.append(h.hexdigest())
    if rank == 0:
        h = hashlib.sha256()
        for t in ts:
            x = cpu.synth_fill(t.synth_spec(seed), t.numel)
            c, keep = abi.make_content(abi.TType(list(t.shape), t.dtype), x)
            dst = np.zeros(t.numel // 2, np.uint8)
            cpu.quantize_fold(c, wl.spec_u4_group(128), abi.make_transforms([wl.t_bitpack()]), 1, dst, dst.size)
            h.update(dst.tobytes())
        q.put((digests, h.hexdigest()))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_sharding_reassembles_bit_identically():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 1000
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    digests, whole = q.get(timeout=240)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert digests[0] == whole  # whole tensors per rank
    assert digests[1] == whole  # output-channel slabs per rank


def test_reference_case_list_is_complete():
    assert len(rc.FOLD_CASES) == 37 and len(rc.TABLE_CASES) == 3


def test_max_intermediate_size_follows_the_pass():
    """getMaxIntermediateSize (const/passes/constant_folding.cpp:20-31): the largest allocation among the base type
    and the type after each transformation."""
    from vpux_plugin_b200 import lib
    from vpux_plugin_b200.abi import TType
    from vpux_plugin_b200.const import ContentSetup
    t = TType([16, 3, 3, 3], abi.VF_DT_F32)                                   # 1728 bytes
    tr, n = ContentSetup(t).transforms()
    assert lib.max_intermediate_size(t, False, tr, n) == 1728
    tr, n = ContentSetup(t).castElemType(abi.VF_DT_F16).transforms()           # shrinks: the base stays the largest
    assert lib.max_intermediate_size(t, False, tr, n) == 1728
    s = ContentSetup(t).padWithZero([0, 0, 0, 0], [0, 13, 0, 0]).castElemType(abi.VF_DT_F16)
    tr, n = s.transforms()                                                     # 16x16x3x3 f32 in the middle
    assert lib.max_intermediate_size(t, False, tr, n) == 16 * 16 * 9 * 4
    s = ContentSetup(t).castElemType(abi.VF_DT_F16).subview([0, 0, 0, 0], [4, 3, 3, 3]).broadcast(0, 64)
    tr, n = s.transforms()
    assert lib.max_intermediate_size(t, False, tr, n) == 64 * 27 * 2
    assert lib.raw().vf_status_string(abi.VF_ERR_NOT_RUN) == b"job not run"


@pytest.mark.parametrize("bad", [0.0, -0.0, -1e-3, float("inf"), float("-inf"), float("nan")])
@pytest.mark.parametrize("where", [0, 1, 2047, 4095, 4096, 4999])
def test_a_quantized_type_with_an_illegal_scale_is_refused_wherever_it_sits(bad, where):
    """mlir::quant::UniformQuantizedPerAxisType::verify rejects scale <= 0, infinities and NaN ("illegal scale");
    the library's check runs over the whole array at once, so the position must not matter. Subnormal and
    very large finite scales are legal."""
    from vpux_plugin_b200 import lib
    n = 5000
    scales = np.linspace(1e-3, 2e-3, n)
    scales[7], scales[8] = 5e-324, 1.7e308  # legal extremes
    t = TType([n, 8], abi.VF_DT_F32)
    q = Elem.per_axis(abi.VF_DT_I8, abi.VF_DT_F16, scales, np.zeros(n, np.int64), 0, -127, 127)
    tr, k = ContentSetup(t).quantize(q).transforms()
    out, _, nbytes = lib.infer_type(t, False, tr, k)
    assert nbytes == n * 8
    scales[where] = bad
    q = Elem.per_axis(abi.VF_DT_I8, abi.VF_DT_F16, scales, np.zeros(n, np.int64), 0, -127, 127)
    tr, k = ContentSetup(t).quantize(q).transforms()
    with pytest.raises(lib.VfoldError) as e:
        lib.infer_type(t, False, tr, k)
    assert e.value.status == abi.VF_ERR_INVALID_ARG and "illegal scale" in str(e.value)
