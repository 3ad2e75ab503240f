"""vf_folder — folding in the background with a cache of folded contents — after the reference's own tests of
Const::BackgroundConstantFolding (tests/unit/vpux_compiler/dialect/const/constant_folding_in_background_tests.cpp,
cited as BG:lines) plus what the cache promises in constant_folding_cache.hpp: duplicates are folded once,
a request continues from a cached prefix, an equivalence request re-keys a result, the memory limit evicts the
entries with the lowest reference count first. Every folded result is compared with the CPU oracle."""
import numpy as np
import pytest

from vpux_plugin_b200 import abi
from vpux_plugin_b200.abi import Elem, TType
from vpux_plugin_b200.const import ContentAttr, ContentSetup

pytestmark = pytest.mark.gpu

F32, F16, I8, U8 = abi.VF_DT_F32, abi.VF_DT_F16, abi.VF_DT_I8, abi.VF_DT_U8


@pytest.fixture()
def folder():
    from vpux_plugin_b200.lib import Folder
    f = Folder(device=0, max_concurrent_tasks=1)
    yield f
    f.close()


def _same(folder, oracle, attr, expect_cached):
    a = attr.fold(folder)
    assert folder.from_cache == expect_cached
    b = attr.fold(oracle)
    assert a.type == b.type and a.written == b.written
    assert np.array_equal(a.bytes(), b.bytes())
    return a


@pytest.mark.parametrize("threads", [1, 2, 3, 4, 5])
def test_compilation_flow(threads, oracle):
    """BG:36-52, 88-106: a splat of 1.0 with five Add(1.0); the request is queued when the attribute is built and
    the later fold() finds 6.0 in the cache."""
    from vpux_plugin_b200.lib import Folder
    folder = Folder(device=0, max_concurrent_tasks=threads, memory_limit_bytes=3 * 1024 * 1024, clean_threshold=0.8)
    try:
        t = TType([100], F32)
        s = ContentSetup(t)
        for _ in range(5):
            s = s.add(1.0)
        attr = ContentAttr(np.array([1.0], np.float32), t, s, is_splat=True)
        folder.enqueue(attr)
        folder.wait_idle()
        out = _same(folder, oracle, attr, True)
        assert out.values(np.float32).tolist() == [6.0] * 100
        st = folder.statistics()
        assert st["added"] == 1 and st["hits"] == 1 and st["failed"] == 0
    finally:
        folder.close()


def test_multiple_compilations(oracle):
    """BG:108-150: two folders (one per compilation) at the same time, the second with mixed transformations."""
    import threading
    from vpux_plugin_b200.lib import Folder
    t = TType([100], F32)
    same = ContentSetup(t)
    for _ in range(5):
        same = same.add(1.0)
    attrs = [ContentAttr(np.array([1.0], np.float32), t, same, is_splat=True),
             ContentAttr(np.array([0.0], np.float32), t,
                         ContentSetup(t).padWithZero([10], [10]).add(1.0).rescale(3.0).subview([0], [100]), is_splat=True)]
    expected = [6.0, 3.0]
    results = [None, None]

    def compile_one(i):
        folder = Folder(device=0, max_concurrent_tasks=2)
        try:
            folder.enqueue(attrs[i])
            folder.wait_idle()
            results[i] = (attrs[i].fold(folder).values(np.float32).tolist(), folder.from_cache)
        finally:
            folder.close()

    threads = [threading.Thread(target=compile_one, args=(i,)) for i in range(2)]
    for th in threads:
        th.start()
    for th in threads:
        th.join()
    for i in range(2):
        vals, cached = results[i]
        assert cached and vals == [expected[i]] * 100
        assert np.array_equal(np.array(vals, np.float32), attrs[i].fold(oracle).values(np.float32))


def test_equivalence_request(folder, oracle):
    """BG:156-196: two SubViews folded in the background, then an equivalence request to the fused SubView: the
    cached result is found under the new attribute."""
    t = TType([100], F32)
    base = np.array([1.0], np.float32)
    attr1 = ContentAttr(base, t, ContentSetup(t).subview([0], [50]).subview([10], [30]), is_splat=True)
    attr2 = ContentAttr(base, t, ContentSetup(t).subview([0], [30]), is_splat=True)
    folder.enqueue(attr1)
    folder.enqueue_equivalence(attr1, attr2)
    folder.wait_idle()
    assert folder.has_content(attr2)
    assert not folder.has_content(attr1)
    st = folder.statistics()
    assert st["added"] == 1  # re-keyed, not folded again
    _same(folder, oracle, attr2, True)
    # without a cached original the new attribute is folded
    attr3 = ContentAttr(base, t, ContentSetup(t).add(2.0).add(3.0), is_splat=True)
    attr4 = ContentAttr(base, t, ContentSetup(t).add(5.0), is_splat=True)
    folder.enqueue_equivalence(attr3, attr4)
    folder.wait_idle()
    assert folder.has_content(attr4) and folder.statistics()["added"] == 2


def test_duplicates_and_content_hash(folder, oracle):
    """The same attribute queued twice is folded once, and so are equal bytes in two different buffers (the
    base is named by the hash of its bytes); different bytes get their own entry."""
    rng = np.random.default_rng(3)
    t = TType([64, 33], F16)
    x = rng.standard_normal((64, 33)).astype(np.float16)
    s = ContentSetup(t).rescale(0.5)
    a1 = ContentAttr(x, t, s)
    a2 = ContentAttr(x.copy(), t, s)
    y = x.copy()
    y[63, 32] = np.float16(7.0)
    a3 = ContentAttr(y, t, s)
    for a in (a1, a1, a2, a3):
        folder.enqueue(a)
    folder.wait_idle()
    st = folder.statistics()
    assert st["added"] == 2 and st["duplicated"] == 2 and st["cache_size"] == 2
    _same(folder, oracle, a2, True)
    _same(folder, oracle, a3, True)
    # the caller's own identity of a base (the reference's uniqued attribute) is a different name
    folder.enqueue(a1, base_id=77)
    folder.wait_idle()
    assert folder.statistics()["added"] == 3
    assert folder.has_content(a1, base_id=77) and not folder.has_content(a1, base_id=78)


def test_partial_folding(folder, oracle):
    """tryFoldingPartially (constant_folding_in_background.cpp:65-100): a request whose new transformation was
    appended continues from the cached result of the shorter list, which is then dropped. The cached content
    keeps its storage type: CastElemType leaves f32 storage behind, and Add must read that, not f16."""
    rng = np.random.default_rng(4)
    t = TType([8, 40], F32)
    x = (rng.standard_normal((8, 40)) * 3).astype(np.float32)
    s1 = ContentSetup(t).castElemType(F16)
    s2 = s1.add(0.3337)
    s3 = s2.reorder(0x21)
    a1, a2, a3 = (ContentAttr(x, t, s) for s in (s1, s2, s3))
    folder.enqueue(a1)
    folder.enqueue(a2, new_index=1)
    folder.enqueue(a3, new_index=2)
    folder.wait_idle()
    st = folder.statistics()
    assert st["partial"] == 2 and st["added"] == 3 and st["cache_size"] == 1 and st["failed"] == 0
    assert not folder.has_content(a1) and not folder.has_content(a2)
    _same(folder, oracle, a3, True)
    _same(folder, oracle, a2, False)  # no longer cached: folded directly


def test_memory_limit_evicts_lowest_ref_count_first(oracle):
    """cleanUpCache (constant_folding_cache.cpp:51-70): when the limit is reached entries go in order of their
    reference count until the cache is down to limit * threshold."""
    from vpux_plugin_b200.lib import Folder
    folder = Folder(device=0, max_concurrent_tasks=1, memory_limit_bytes=4000, clean_threshold=0.5)
    try:
        t = TType([100], F32)  # 400 bytes each
        attrs = [ContentAttr(np.full(100, float(i), np.float32), t, ContentSetup(t).add(1.0)) for i in range(10)]
        for a in attrs[:9]:
            folder.enqueue(a)
        folder.wait_idle()
        assert folder.statistics()["memory_used"] == 3600 and folder.statistics()["erased"] == 0
        for a in attrs[5:9]:  # asked for again: more likely to be needed
            assert folder.has_content(a)
        folder.enqueue(attrs[9])  # reaches 4000 bytes: clean down to 2000
        folder.wait_idle()
        st = folder.statistics()
        assert st["memory_used"] == 2000 and st["erased"] == 5 and st["max_memory_used"] == 4000
        assert st["cache_size"] == 5 and st["max_cache_size"] == 10
        kept = [folder.has_content(a) for a in attrs]
        assert kept[5:9] == [True] * 4 and sum(kept) == 5
        for a, k in zip(attrs, kept):
            _same(folder, oracle, a, k)
    finally:
        folder.close()


def test_failed_request_is_dropped(folder, oracle):
    t = TType([4, 4], F32)
    x = np.arange(16, dtype=np.float32)
    bad = ContentAttr(x, t, ContentSetup(t).dequantize())  # not a quantized type
    good = ContentAttr(x, t, ContentSetup(t).add(1.0))
    folder.enqueue(bad)
    folder.enqueue(good)
    folder.wait_idle()
    st = folder.statistics()
    assert st["failed"] == 1 and st["added"] == 1
    _same(folder, oracle, good, True)
    from vpux_plugin_b200.lib import VfoldError
    with pytest.raises(VfoldError) as e:
        bad.fold(folder)
    assert e.value.status == abi.VF_ERR_NOT_QUANTIZED


def test_remove(folder):
    t = TType([16], F32)
    a = ContentAttr(np.arange(16, dtype=np.float32), t, ContentSetup(t).add(1.0))
    folder.enqueue(a)
    folder.wait_idle()
    assert folder.has_content(a)
    folder.remove(a)
    assert not folder.has_content(a) and folder.statistics()["memory_used"] == 0


def test_many_requests_from_many_workers(oracle):
    """Weight-shaped requests with repeats over four workers: every result matches the oracle."""
    from vpux_plugin_b200.lib import Folder
    rng = np.random.default_rng(9)
    folder = Folder(device=0, max_concurrent_tasks=4)
    try:
        q = Elem.uniform(I8, F32, 0.02, 0, -127, 127)
        attrs = []
        for i in range(24):
            oc, ic = int(rng.integers(8, 40)), int(rng.integers(4, 20)) * 8
            t = TType([oc, ic, 1, 1], F32)
            x = rng.standard_normal((oc, ic, 1, 1)).astype(np.float32)
            x[rng.random(x.shape) < 0.5] = 0.0  # sparse enough for the compacted data to fit the dense size
            s = ContentSetup(t).quantize(q).castElemType(q).reorder(abi.ORDER_NHWC)
            if i % 3 == 0:
                s = s.getSparsityMap()
            elif i % 3 == 1:
                s = s.sparsify(False)
            attrs.append(ContentAttr(x, t, s))
        order = [int(v) for v in rng.integers(0, len(attrs), 96)] + list(range(len(attrs)))
        for i in order:
            folder.enqueue(attrs[i])
        folder.wait_idle()
        st = folder.statistics()
        assert st["failed"] == 0, folder.last_error()
        assert st["cache_size"] == len(attrs) and st["added"] + st["duplicated"] == len(order)
        for a in attrs:
            _same(folder, oracle, a, True)
    finally:
        folder.close()


def test_reference_vectors_through_the_folder(folder):
    """The fold goldens with the folder as the backend (cache misses: folded directly)."""
    import reference_cases as rc
    for case in (rc.quantize, rc.dequantize, rc.reorder, rc.pad, rc.bit_pack, rc.get_sparsity_map, rc.sparsify,
                 rc.relocate_weights_table):
        case(folder)


def test_content_hash(gpu):
    """Equal bytes hash equally wherever they live and however they are aligned; any changed byte, or a
    different length, changes the hash."""
    import torch
    from vpux_plugin_b200.lib import content_hash
    rng = np.random.default_rng(11)
    raw = rng.integers(0, 256, 100_003 + 16, dtype=np.uint8)
    dev = torch.from_numpy(raw).cuda()

    def h(arr_or_ptr, n, device=False):
        t = TType([n], U8)
        if device:
            c, keep = abi.make_content(t, None, U8, False, abi.VF_MEM_DEVICE, ptr=int(arr_or_ptr), nbytes=n)
        else:
            c, keep = abi.make_content(t, arr_or_ptr, U8, False)
        return content_hash(gpu, c)

    for n in (0, 1, 7, 8, 9, 4096, 100_003):
        ref = h(raw[:n].copy(), n)
        for off in (1, 3, 8):
            shifted = raw.copy()
            shifted[off:off + n] = raw[:n]
            d = torch.from_numpy(shifted).cuda()
            assert h(d.data_ptr() + off, n, device=True) == ref, (n, off)
        assert h(dev.data_ptr(), n, device=True) == ref
        if n:
            changed = raw[:n].copy()
            changed[n - 1] ^= 1
            assert h(changed, n) != ref
            assert h(raw[:n + 1].copy(), n + 1) != ref
    # a splat hashes its single element
    t = TType([1000], F32)
    c, keep = abi.make_content(t, np.array([2.5], np.float32), F32, True)
    c2, keep2 = abi.make_content(TType([1], F32), np.array([2.5], np.float32), F32, False)
    assert content_hash(gpu, c) == content_hash(gpu, c2)
