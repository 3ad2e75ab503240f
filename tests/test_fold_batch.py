"""vf_fold_batch — ConstantFoldingPass::safeRunOnFunc (const/passes/constant_folding.cpp:85-159) over a list of
constants: the schedule (tiny constants first, large ones alone, the rest in groups under the size threshold) is
checked against a restatement of the pass's loop, every folded result against a single vf_fold and the CPU oracle."""
import numpy as np
import pytest

from vpux_plugin_b200 import abi
from vpux_plugin_b200.abi import Elem, TType
from vpux_plugin_b200.const import ContentAttr, ContentSetup, foldConstants
from vpux_plugin_b200.lib import VfoldError, max_intermediate_size

pytestmark = pytest.mark.gpu

F32, F16, I8, U8 = abi.VF_DT_F32, abi.VF_DT_F16, abi.VF_DT_I8, abi.VF_DT_U8


def pass_schedule(sizes, threshold, tiny):
    """constant_folding.cpp:100-158 on the list of getMaxIntermediateSize values: the group of every constant."""
    group = [None] * len(sizes)
    big = []
    for i, s in enumerate(sizes):
        if s > tiny:
            big.append(i)
        else:
            group[i] = abi.VF_GROUP_TINY
    at, g = 0, 0
    while at < len(big):
        if sizes[big[at]] > threshold:
            group[big[at]] = abi.VF_GROUP_ALONE
            at += 1
            continue
        total = 0
        while total <= threshold and at < len(big):
            total += sizes[big[at]]
            group[big[at]] = g
            at += 1
        g += 1
    return group, g


def weights(rng, shape, dt=np.float32):
    return (rng.standard_normal(shape) * 0.1).astype(dt)


def model_constants(rng):
    """A small network's worth of constants: biases and scales (tiny), convolution weights of several sizes with
    the lists the compiler attaches to them, one large fully-connected matrix."""
    attrs = []
    q = Elem.uniform(U8, F32, 0.01, 128, 0, 255)
    for oc, ic, k in [(16, 3, 3), (32, 16, 3), (64, 32, 1), (8, 8, 1), (128, 64, 3), (64, 64, 3), (256, 128, 1), (24, 24, 5)]:
        t = TType([oc, ic, k, k], F32)
        attrs.append(ContentAttr(weights(rng, t.shape), t, ContentSetup(t).castElemType(F16).reorder(abi.ORDER_NHWC)))
        tb = TType([1, oc, 1, 1], F32)
        attrs.append(ContentAttr(weights(rng, tb.shape), tb, ContentSetup(tb).castElemType(F16)))
        tq = TType([oc, ic, k, k], U8)
        attrs.append(ContentAttr(rng.integers(0, 256, tq.shape).astype(np.uint8), tq,
                                 ContentSetup(tq).castElemType(q).dequantize().padWithZero([0, 0, 0, 0], [0, (-ic) % 16, 0, 0])))
    t = TType([512, 1024], F32)
    attrs.append(ContentAttr(weights(rng, t.shape), t, ContentSetup(t).castElemType(F16).reshape([512, 1024, 1, 1])))
    t = TType([1, 1, 1, 1], F32)
    attrs.append(ContentAttr(np.array([2.5], np.float32), t, ContentSetup(t).broadcast(1, 64).castElemType(F16), is_splat=True))
    return attrs


@pytest.mark.parametrize("threshold", [0, 64 * 1024, 512 * 1024, 1 << 40])
def test_schedule_and_results(gpu, oracle, threshold):
    rng = np.random.default_rng(7)
    attrs = model_constants(rng)
    sizes = []
    for a in attrs:
        tr, n = a.setup.transforms()
        sizes.append(max_intermediate_size(a.base_type, a.is_splat, tr, n))
    folded, stats, groups = foldConstants(gpu, attrs, threshold_bytes=threshold)
    eff = threshold if threshold else 300 * 1024 * 1024
    want_groups, n_groups = pass_schedule(sizes, eff, 1024)
    assert groups == want_groups
    assert stats.tiny == want_groups.count(abi.VF_GROUP_TINY) and stats.tiny >= 8
    assert stats.alone == want_groups.count(abi.VF_GROUP_ALONE)
    assert stats.groups == n_groups
    assert stats.synchronisations == (1 if stats.tiny else 0) + stats.alone + stats.groups
    if n_groups:
        assert stats.max_group_bytes == max(sum(s for s, g in zip(sizes, want_groups) if g == k) for k in range(n_groups))
    for a, f in zip(attrs, folded):
        single = a.fold(gpu)
        ref = a.fold(oracle)
        assert f.type == single.type == ref.type and f.written == single.written == ref.written
        assert np.array_equal(f.bytes(), single.bytes()) and np.array_equal(f.bytes(), ref.bytes())


def test_thresholds_of_the_pass_by_default(gpu):
    """300 MB and 1 KB (constant_folding.cpp:74, 83): a 1024-byte constant is tiny, one of 1028 bytes is not."""
    a = TType([256], F32)
    b = TType([257], F32)
    attrs = [ContentAttr(np.ones(256, np.float32), a, ContentSetup(a).castElemType(F16)),
             ContentAttr(np.ones(257, np.float32), b, ContentSetup(b).castElemType(F16))]
    _, stats, groups = foldConstants(gpu, attrs)
    assert groups == [abi.VF_GROUP_TINY, 0] and stats.tiny == 1 and stats.groups == 1 and stats.alone == 0


def test_empty_batch(gpu):
    folded, stats, groups = foldConstants(gpu, [])
    assert folded == [] and groups == [] and stats.synchronisations == 0


def _jobs(attrs, dst_bytes):
    jobs = (abi.FoldJob * len(attrs))()
    keep = []
    for j, a in enumerate(attrs):
        tr, n = a.setup.transforms()
        c, k = abi.make_content(a.base_type, a.base, a.storage_dtype, a.is_splat)
        dst = np.zeros(max(dst_bytes[j], 1), np.uint8)
        jobs[j].base, jobs[j].t, jobs[j].n = c, tr, n
        jobs[j].dst_mem_kind, jobs[j].dst, jobs[j].dst_bytes = abi.VF_MEM_HOST, dst.ctypes.data, dst_bytes[j]
        keep.append((tr, k, dst))
    return jobs, keep


def test_failing_job_ends_the_batch(gpu):
    """A constant the reference throws on stops the pass; the jobs behind it are reported as not run."""
    rng = np.random.default_rng(3)
    t = TType([64, 64, 3, 3], F32)
    ok = ContentAttr(weights(rng, t.shape), t, ContentSetup(t).castElemType(F16))
    full = 64 * 64 * 9 * 2
    jobs, keep = _jobs([ok, ok, ok], [full, full - 2, full])                              # content.cpp:172-174
    with pytest.raises(VfoldError) as e:
        gpu.fold_batch(jobs)
    assert e.value.status == abi.VF_ERR_BUFFER_TOO_SMALL and "job 1" in str(e.value)
    assert [jobs[j].status for j in range(3)] == [abi.VF_OK, abi.VF_ERR_BUFFER_TOO_SMALL, abi.VF_ERR_NOT_RUN]
    assert np.array_equal(keep[0][2].view(np.float16), ok.base.astype(np.float16).reshape(-1))
    # a list whose types do not infer fails while the sizes are computed, before anything runs
    bad = ContentAttr(weights(rng, t.shape), t, ContentSetup(t).dequantize())           # dequantize.cpp:43-44
    jobs, keep = _jobs([ok, bad, ok], [full, full * 2, full])
    with pytest.raises(VfoldError) as e:
        gpu.fold_batch(jobs)
    assert e.value.status == abi.VF_ERR_NOT_QUANTIZED and "job 1" in str(e.value)
    assert [jobs[j].status for j in range(3)] == [abi.VF_ERR_NOT_RUN, abi.VF_ERR_NOT_QUANTIZED, abi.VF_ERR_NOT_RUN]
    # the context stays usable
    out = ok.fold(gpu)
    assert np.array_equal(out.values(np.float16), ok.base.astype(np.float16).reshape(-1))


def test_kernel_reported_failure_names_the_group(gpu):
    """A checked_cast that fails on the device is found when the group is waited for."""
    t = TType([4096], F32)
    fine = ContentAttr(np.full(4096, 3.0, np.float32), t, ContentSetup(t).castElemType(U8))
    over = ContentAttr(np.full(4096, 300.0, np.float32), t, ContentSetup(t).castElemType(U8))  # 300 does not fit u8
    with pytest.raises(VfoldError) as e:
        foldConstants(gpu, [fine, over, fine])
    assert e.value.status == abi.VF_ERR_CHECKED_CAST and "group 0" in str(e.value)
    assert fine.fold(gpu).bytes().tolist() == [3] * 4096
