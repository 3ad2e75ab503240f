"""The rules that move a transformation into a Fuse (moveTransformationIntoFuse / moveSubViewIntoFuse,
utils/transformations.cpp:687-862) on const.FusedConstant: the rewritten part lists are the expectations of the
reference's content_setup.cpp (cited as CS:lines); on the GPU the rewritten Fuse folds to the same bytes as the
plain Fuse followed by the transformation."""
import numpy as np
import pytest

from vpux_plugin_b200 import abi
from vpux_plugin_b200.abi import TType
from vpux_plugin_b200.const import ContentAttr, ContentSetup, FusedConstant

I8, I4, I32, U8 = abi.VF_DT_I8, abi.VF_DT_I4, abi.VF_DT_I32, abi.VF_DT_U8
SUBVIEW, RESHAPE, CAST, RELOCATE = abi.VF_T_SUBVIEW, abi.VF_T_RESHAPE, abi.VF_T_CAST_ELEM_TYPE, abi.VF_T_RELOCATE_WEIGHTS_TABLE


def const(shape, values, dt=I8):
    t = TType(shape, dt)
    return ContentAttr(np.asarray(values, abi.DTYPE_NUMPY[dt]).reshape(shape), t, ContentSetup(t))


def listed(attr):
    """[(kind, a, b)] of a part's transformations."""
    tr, n = attr.setup.transforms()
    return [(tr[i].kind, [tr[i].a[k] for k in range(tr[i].rank)], [tr[i].b[k] for k in range(tr[i].rank)]) for i in range(n)]


def fused12(weights_shape):
    wt = const([4, 1, 1, 1], [1, 1, 1, 1])
    w = const(weights_shape, [1] * 8)
    return FusedConstant(TType([1, 1, 1, 12], I8), wt, w)


def test_subview_splits_the_fused_constant_in_half():
    """CS:1767-1793"""
    lower = fused12([4, 2, 1, 1]).subview([0, 0, 0, 0], [1, 1, 1, 6])
    assert lower.trailing.names() == [] and lower.fused_type.shape == [1, 1, 1, 6]
    assert listed(lower.weightsTable) == []
    assert listed(lower.weights) == [(SUBVIEW, [0, 0, 0, 0], [1, 2, 1, 1])]
    upper = fused12([4, 2, 1, 1]).subview([0, 0, 0, 6], [1, 1, 1, 6])
    assert upper.weightsTable is None
    assert listed(upper.weights) == [(SUBVIEW, [1, 0, 0, 0], [3, 2, 1, 1])]


def test_subview_unaligned_view_into_weights():
    """CS:1795-1815: the view is not a whole number of rows — a row SubView, then a flat Reshape + SubView"""
    f = fused12([4, 1, 1, 2]).subview([0, 0, 0, 7], [1, 1, 1, 3])
    assert f.weightsTable is None
    assert listed(f.weights) == [(SUBVIEW, [1, 0, 0, 0], [2, 1, 1, 2]), (RESHAPE, [1, 1, 1, 4], [0, 0, 0, 0]),
                                 (SUBVIEW, [0, 0, 0, 1], [1, 1, 1, 3])]


def test_subview_unaligned_view_into_unslicable_weights():
    """CS:1817-1835"""
    f = fused12([2, 1, 2, 2]).subview([0, 0, 0, 7], [1, 1, 1, 3])
    assert f.weightsTable is None
    assert listed(f.weights) == [(RESHAPE, [1, 1, 1, 8], [0, 0, 0, 0]), (SUBVIEW, [0, 0, 0, 3], [1, 1, 1, 3])]


def test_subview_into_sub_byte_weights():
    """CS:1837-1870: offsets are counted in 4-bit elements; the SubView moves in front of the cast"""
    wt = const([4, 1, 1, 1], [1, 1, 1, 1])
    t = TType([4, 1, 1, 4], I8)
    w = ContentAttr(np.array([10], np.int8), t, ContentSetup(t).castElemType(I4), is_splat=True)
    f = FusedConstant(TType([1, 1, 1, 12], I8), wt, w).subview([0, 0, 0, 8], [1, 1, 1, 4])
    got = listed(f.weights)
    assert len(got) == 2 and got[0] == (SUBVIEW, [2, 0, 0, 0], [2, 1, 1, 4]) and got[1][0] == CAST


def test_subview_stays_behind_a_sparse_or_non_flat_fuse():
    """CS:1872-1909"""
    wt = const([4, 1, 1, 1], [1, 1, 1, 1])
    w = const([4, 2, 1, 1], [1] * 8)
    sp = const([1, 1, 1, 1], [1])
    f = FusedConstant(TType([1, 1, 1, 13], I8), wt, w, sp).subview([0, 0, 0, 0], [1, 1, 1, 7])
    assert listed(f.weights) == [] and f.sparsity is sp and f.fused_type.shape == [1, 1, 1, 13]
    tr, n = f.trailing.transforms()
    assert n == 1 and tr[0].kind == SUBVIEW and [tr[0].b[k] for k in range(4)] == [1, 1, 1, 7]
    g = FusedConstant(TType([6, 1, 1, 2], I8), wt, w).subview([0, 0, 0, 0], [3, 1, 1, 2])
    assert listed(g.weights) == [] and g.trailing.names() == [SUBVIEW]


def test_relocate_joins_the_weights_table():
    """CS:1721-1763: Fuse + RelocateWeightsTable becomes one Fuse whose weights table carries the relocation"""
    wt = const([4, 1, 1, 4], np.arange(16), I32)
    w = const([4, 4, 1, 1], np.arange(16))
    f = FusedConstant(TType([1, 1, 1, 80], U8), wt, w).relocateWeightsTablePointers([100], 200, [0], 64)
    assert f.trailing.names() == []
    got = listed(f.weightsTable)
    assert len(got) == 1 and got[0][0] == RELOCATE and listed(f.weights) == []


@pytest.mark.gpu
@pytest.mark.parametrize("wshape", [[16, 8, 1, 1], [16, 2, 2, 2], [8, 4, 2, 2]])
def test_moved_subview_folds_to_the_same_bytes(gpu, wshape):
    rng = np.random.default_rng(sum(wshape))
    oc = wshape[0]
    wt = const([oc, 1, 1, 4], rng.integers(0, 1 << 20, oc * 4), I32)
    w = const(wshape, rng.integers(-128, 128, int(np.prod(wshape))))
    total = oc * 16 + int(np.prod(wshape))
    plain = FusedConstant(TType([1, 1, 1, total], U8), wt, w)
    whole = plain.fold(gpu).bytes()
    assert len(whole) == total
    cases = [(0, total // 2), (total // 2, total - total // 2 - 1), (oc * 16, total - oc * 16), (oc * 16 + 3, 29),
             (oc * 16 - 8, 8), (8, 12), (oc * 16 - 4, 37), (4, total - 5)]  # whole elements of each constant, as the rule assumes
    for off, n in cases:
        moved = plain.subview([0, 0, 0, off], [1, 1, 1, n])
        assert moved.trailing.names() == []
        assert np.array_equal(moved.fold(gpu).bytes(), whole[off:off + n]), (off, n)
    # a view that starts before the last constant and covers it to its end drops that constant, exactly as
    # getOverlapRegionBounds is written (transformations.cpp:716-727): pinned as the reference behaves
    quirk = plain.subview([0, 0, 0, 0], [1, 1, 1, total])
    assert quirk.weights is None and quirk.weightsTable is not None
    # what cannot move stays behind the Fuse and is applied to the fused bytes
    behind = FusedConstant(TType([1, 1, 1, total], U8), wt, w, trailing=ContentSetup(TType([1, 1, 1, total], U8)).add(0.0))
    assert np.array_equal(behind.subview([0, 0, 0, 5], [1, 1, 1, 50]).fold(gpu).bytes(), whole[5:55])


@pytest.mark.gpu
def test_moved_relocation_folds_like_the_relocated_table(gpu, oracle):
    oc = 16
    table = np.zeros((oc, 1, 1, 4), np.int32)
    table[:, 0, 0, 0] = np.arange(oc) * 64
    table[:, 0, 0, 1] = np.arange(oc) * 16
    table[:, 0, 0, 2:] = 7
    wt = const([oc, 1, 1, 4], table, I32)
    w = const([oc, 16, 1, 1], np.arange(oc * 16) % 100)
    f = FusedConstant(TType([1, 1, 1, oc * 32], U8), wt, w).relocateWeightsTablePointers([4096], 8192, [0], oc * 16)
    got = f.fold(gpu).bytes()
    t = TType([oc, 1, 1, 4], I32)
    want = ContentAttr(table, t, ContentSetup(t).relocateWeightsTablePointers([4096], 8192, [0], oc * 16)).fold(oracle)
    assert np.array_equal(got[:oc * 16], want.bytes()) and np.array_equal(got[oc * 16:].view(np.int8), w.base.reshape(-1))
