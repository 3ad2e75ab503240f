"""vf_optimize_transforms (pure host) against the reference's own expectations for ContentSetup's rewriting
(tests/unit/vpux_compiler/dialect/const/content_setup.cpp, cited as CS:lines), and the property that the
rewritten list folds to the same bytes as the original one (oracle on CPU, library on the GPU)."""
import numpy as np
import pytest

from vpux_plugin_b200 import abi
from vpux_plugin_b200.abi import Elem, TType
from vpux_plugin_b200.const import ContentAttr, ContentSetup

F32, F16, I8, U8 = abi.VF_DT_F32, abi.VF_DT_F16, abi.VF_DT_I8, abi.VF_DT_U8
CHW, HWC, WHC, HCW = 0x123, 0x231, 0x321, 0x213
HCNW, NHWC = 0x3214, 0x1342
K = abi


def _items(setup):
    out = []
    for t, _ in setup._items:
        k, r = t.kind, t.rank
        if k == K.VF_T_SUBVIEW:
            out.append(("subview", list(t.a[:r]), list(t.b[:r])))
        elif k == K.VF_T_PAD_WITH_ZERO:
            out.append(("pad", list(t.a[:r]), list(t.b[:r])))
        elif k == K.VF_T_RESHAPE:
            out.append(("reshape", list(t.a[:r])))
        elif k == K.VF_T_ADD:
            out.append(("add", t.value))
        elif k == K.VF_T_RESCALE:
            out.append(("rescale", t.value))
        elif k == K.VF_T_REORDER:
            out.append(("reorder", t.order))
        elif k == K.VF_T_TRANSPOSE:
            out.append(("transpose", t.order))
        elif k == K.VF_T_MEM_PERMUTE:
            out.append(("mempermute", t.order, t.mem_perm))
        elif k in (K.VF_T_CAST_ELEM_TYPE, K.VF_T_CONVERT_ELEM_TYPE):
            e = t.elem
            n = e.nparams if e.kind != K.VF_ELEM_PLAIN else 0
            out.append(("cast" if k == K.VF_T_CAST_ELEM_TYPE else "convert", e.kind, e.dtype,
                        [e.scales[i] for i in range(n)], [e.zps[i] for i in range(n)]))
        elif k == K.VF_T_CHANGE_SHAPE_AND_ELEM_TYPE:
            e = t.elem
            n = e.nparams if e.kind != K.VF_ELEM_PLAIN else 0
            out.append(("changeshape", list(t.a[:r]), e.axis, [e.scales[i] for i in range(n)]))
        elif k == K.VF_T_DEQUANTIZE:
            out.append(("dequantize",))
        elif k == K.VF_T_RELOCATE_WEIGHTS_TABLE:
            r = t.relocate
            out.append(("relocate", list(r.weights_ptr[:r.n_clusters]), r.sparsity_ptr, list(r.offsets[:r.n_clusters]),
                        r.weights_table_size, r.channel_offset,
                        [r.num_elems[i] for i in range(r.n_num_elems)] if r.num_elems else None))
        else:
            out.append((k,))
    return out


def S(shape, dt=I8):
    return ContentSetup(TType(list(shape), dt))


def test_fuse_rules():
    # CS:720-747 FuseSubView
    assert _items(S([1, 7, 5]).subview([0, 1, 2], [1, 6, 3]).subview([0, 1, 1], [1, 2, 1]).optimized()) == [
        ("subview", [0, 2, 3], [1, 2, 1])]
    # CS:749-767 FuseAdd, CS:769-787 FuseRescale
    assert _items(S([1, 7, 5]).add(1).add(2).optimized()) == [("add", 3.0)]
    assert _items(S([1, 7, 5]).rescale(2).rescale(5).optimized()) == [("rescale", 10.0)]
    # CS:789-808 FuseReshape, CS:810-828 FuseReorder, CS:830-853 FuseCastElemType: the later one wins
    assert _items(S([1, 7, 5]).reshape([7, 5]).reshape([5, 7]).optimized()) == [("reshape", [5, 7])]
    assert _items(S([4, 8, 3]).reorder(HWC).reorder(WHC).optimized()) == [("reorder", WHC)]
    assert _items(S([4, 8, 3], F32).castElemType(F16).castElemType(abi.VF_DT_BF16).optimized()) == [
        ("cast", K.VF_ELEM_PLAIN, abi.VF_DT_BF16, [], [])]
    # CS:1911-1943 Reorder and MemPermute fuse into one MemPermute, both ways
    assert _items(S([4, 6, 8]).reorder(HWC).memPermute(WHC, HCW).optimized()) == [("mempermute", WHC, WHC)]
    assert _items(S([4, 6, 8]).memPermute(WHC, WHC).reorder(HWC).optimized()) == [("mempermute", HWC, HWC)]


def test_fold_rules():
    # CS:1945-1999: a Reorder / MemPermute that changes nothing is dropped, one that changes the type is kept
    assert _items(S([4, 6, 8]).reorder(CHW).optimized()) == []
    assert _items(S([2, 1, 1]).reorder(HWC).optimized()) == [("reorder", HWC)]
    assert _items(S([4, 6, 8]).memPermute(CHW, CHW).optimized()) == []
    assert _items(S([2, 1, 1]).memPermute(HWC, HWC).optimized()) == [("mempermute", HWC, HWC)]


def test_move_subview_before():
    off, shp = [0, 1, 1], [1, 2, 1]
    # CS:855-877 Add, CS:932-954 Rescale, CS:879-901 Reorder: plain swaps
    assert _items(S([4, 8, 3]).add(1).subview(off, shp).optimized()) == [("subview", off, shp), ("add", 1.0)]
    assert _items(S([4, 8, 3]).rescale(2).subview(off, shp).optimized()) == [("subview", off, shp), ("rescale", 2.0)]
    assert _items(S([4, 8, 3]).reorder(WHC).subview(off, shp).optimized()) == [("subview", off, shp), ("reorder", WHC)]
    # CS:903-930 Transpose: offsets and extents are permuted back
    assert _items(S([4, 8, 3]).transpose(WHC).subview([0, 1, 2], [3, 2, 1]).optimized()) == [
        ("subview", [2, 1, 0], [1, 2, 3]), ("transpose", WHC)]
    # CS:1132-1155 CastElemType, CS:1257-1294 quantized: a per-axis type is sliced with the view
    assert _items(S([4, 8, 3], F32).castElemType(F16).subview(off, shp).optimized()) == [
        ("subview", off, shp), ("cast", K.VF_ELEM_PLAIN, F16, [], [])]
    per_tensor = Elem.uniform(U8, F32, 0.078, 128, 0, 255)
    per_axis = Elem.per_axis(U8, F32, [2, 0.5], [127, 127], 0, 0, 255)
    assert _items(S([2, 8, 3], U8).castElemType(per_tensor).subview(off, shp).optimized()) == [
        ("subview", off, shp), ("cast", K.VF_ELEM_QUANT_UNIFORM, U8, [0.078], [128])]
    assert _items(S([2, 8, 3], U8).castElemType(per_axis).subview(off, shp).optimized()) == [
        ("subview", off, shp), ("cast", K.VF_ELEM_QUANT_PER_AXIS, U8, [2.0], [127])]
    # CS:1447-1474: the view travels past a long run of Add / Rescale pairs
    s = S([4, 8, 3], F32)
    for i in range(10):
        s = s.add(1 + i).rescale(2 + i)
    got = _items(s.subview([0, 1, 1], [1, 4, 2]).optimized())
    assert got[0] == ("subview", [0, 1, 1], [1, 4, 2]) and len(got) == 21
    assert got[1::2] == [("add", float(1 + i)) for i in range(10)]
    assert got[2::2] == [("rescale", float(2 + i)) for i in range(10)]


def test_move_subview_before_pad():
    # CS:956-1008: a view of padding only stays behind the PadWithZero
    for pb, pa, off, shp in (([0, 0, 0], [0, 0, 256], [0, 0, 256], [1, 1, 128]),
                             ([0, 0, 256], [0, 0, 0], [0, 0, 0], [1, 1, 256])):
        assert _items(S([1, 1, 256]).padWithZero(pb, pa).subview(off, shp).optimized()) == [
            ("pad", pb, pa), ("subview", off, shp)]
    # CS:1010-1040: view over data and padding -> smaller view, smaller padding
    assert _items(S([1, 8, 256]).padWithZero([0, 0, 128], [0, 0, 128]).subview([0, 2, 64], [1, 4, 384]).optimized()) == [
        ("subview", [0, 2, 0], [1, 4, 256]), ("pad", [0, 0, 64], [0, 0, 64])]
    # CS:1042-1068: view inside the data -> the padding disappears
    assert _items(S([1, 8, 256]).padWithZero([0, 0, 128], [0, 0, 128]).subview([0, 2, 192], [1, 4, 64]).optimized()) == [
        ("subview", [0, 2, 64], [1, 4, 64])]
    # CS:1070-1092: the view undoes the padding -> nothing is left
    assert _items(S([1, 8, 256]).padWithZero([0, 0, 0], [0, 8, 0]).subview([0, 0, 0], [1, 8, 256]).optimized()) == []


@pytest.mark.parametrize("base,reshape,off,shp,exp_reshape,exp_off,exp_shp", [
    # CS:1311-1325 swapReshapeAndSubViewParams (the 6-D case exceeds this library's rank limit)
    ([1, 16, 1, 8], [16, 8, 1, 1], [0, 0, 0, 0], [8, 8, 1, 1], [8, 8, 1, 1], [0, 0, 0, 0], [1, 8, 1, 8]),
    ([1, 16, 1, 8], [16, 8, 1, 1], [8, 0, 0, 0], [8, 8, 1, 1], [8, 8, 1, 1], [0, 8, 0, 0], [1, 8, 1, 8]),
    ([1, 16, 8, 8], [1, 16, 64], [0, 0, 0], [1, 8, 64], [1, 8, 64], [0, 0, 0, 0], [1, 8, 8, 8]),
    ([1, 16, 8], [1, 16, 2, 4], [0, 0, 0, 0], [1, 8, 2, 4], [1, 8, 2, 4], [0, 0, 0], [1, 8, 8])])
def test_swap_reshape_and_subview(base, reshape, off, shp, exp_reshape, exp_off, exp_shp):
    assert _items(S(base).reshape(reshape).subview(off, shp).optimized()) == [
        ("subview", exp_off, exp_shp), ("reshape", exp_reshape)]


@pytest.mark.parametrize("base,reshape,off,shp", [
    # CS:1346-1349 doNotswapReshapeAndSubViewParams
    ([1, 16, 1, 8], [128, 1], [0, 0], [64, 1]), ([1, 16, 48, 1], [1, 16, 12, 4], [0, 0, 9, 0], [1, 16, 3, 4])])
def test_do_not_swap_reshape_and_subview(base, reshape, off, shp):
    assert _items(S(base).reshape(reshape).subview(off, shp).optimized()) == [("reshape", reshape), ("subview", off, shp)]


def _comp(num_elems):
    return None if num_elems is None else {"axis": 0, "numElems": num_elems, "alignment": 16}


# CS:1621-1648 swapRelocateWeightsTableAndSubView: (base shape, SubView, Relocate in, Relocate expected), a Relocate
# given as (weightsPtr, sparsityPtr, offsets, weightsTableSize, channelOffset, numElems)
RELOCATE_SWAPS = [
    ([4, 1, 1, 4], ([0, 0, 0, 0], [2, 1, 1, 4]), ([100], 16777215, [0], 64, 0, None), ([100], 16777215, [0], 32, 0, None)),
    ([4, 1, 1, 4], ([1, 0, 0, 0], [2, 1, 1, 4]), ([100], 16777215, [0], 64, 0, None), ([100], 16777215, [0], 32, 1, None)),
    ([4, 1, 1, 4], ([2, 0, 0, 0], [2, 1, 1, 4]), ([100], 200, [0], 64, 0, [1, 2, 3, 4]), ([100], 200, [0], 32, 2, [1, 2, 3, 4])),
    ([4, 1, 1, 4], ([2, 0, 0, 0], [2, 1, 1, 4]), ([100], 200, [0], 64, 2, [1, 2, 3, 4]), ([100], 200, [0], 32, 4, [1, 2, 3, 4])),
    ([8, 1, 1, 4], ([4, 0, 0, 0], [2, 1, 1, 4]), ([100, 200, 300, 400], 16777215, [0, 2, 4, 6], 128, 0, None),
     ([300], 16777215, [0], 32, 0, None)),
    ([8, 1, 1, 4], ([4, 0, 0, 0], [2, 1, 1, 4]), ([100, 200, 300, 400], 200, [0, 2, 4, 6], 128, 0, [1, 2, 3, 4, 5, 6, 7, 8]),
     ([300], 200, [0], 32, 0, [5, 6])),
]


def _relocate(s, p):
    wp, sp, offs, size, chan, ne = p
    return s.relocateWeightsTablePointers(wp, sp, offs, size, 16, _comp(ne), chan)


@pytest.mark.parametrize("base,sub,rin,rexp", RELOCATE_SWAPS)
def test_swap_relocate_weights_table_and_subview(base, sub, rin, rexp):
    got = _items(_relocate(S(base, abi.VF_DT_I32), rin).subview(*sub).optimized())
    assert got == [("subview", sub[0], sub[1]), ("relocate",) + tuple(rexp)]


def test_do_not_swap_relocate_weights_table_and_subview():
    # CS:1655-1685: a slice that starts inside a cluster stays behind the Relocate
    rin = ([100, 200, 300, 400], 16777215, [0, 2, 4, 6], 128, 0, None)
    got = _items(_relocate(S([8, 1, 1, 4], abi.VF_DT_I32), rin).subview([3, 0, 0, 0], [2, 1, 1, 4]).optimized())
    assert got == [("relocate",) + tuple(rin), ("subview", [3, 0, 0, 0], [2, 1, 1, 4])]
    # transformations.cpp:166-170, 175-188: one channel, or a slice of another dim, is not swapped either
    rin = ([100], 7, [0], 64, 0, None)
    for sub in (([1, 0, 0, 0], [1, 1, 1, 4]), ([0, 0, 0, 1], [2, 1, 1, 2])):
        got = _items(_relocate(S([4, 1, 1, 4], abi.VF_DT_I32), rin).subview(*sub).optimized())
        assert got == [("relocate",) + tuple(rin), ("subview", sub[0], sub[1])]


def _relocate_fold_pair(be, seed, n=60):
    """Relocate then SubView folds to the same table as the rewritten SubView then Relocate."""
    rng = np.random.default_rng(seed)
    swapped = 0
    for _ in range(n):
        n_cl = int(rng.integers(1, 4))
        per = int(rng.integers(2, 5))
        oc = n_cl * per
        wstep, sstep = int(rng.integers(1, 64)) * 16, int(rng.integers(0, 9))
        tab = np.zeros((oc, 4), np.int32)
        tab[:, 0] = np.arange(oc) * wstep
        tab[:, 1] = np.arange(oc) * sstep if sstep else 0xFFFFFF
        tab[:, 2:] = rng.integers(-1000, 1000, (oc, 2))
        segmented = n_cl > 1 and rng.integers(0, 2) == 1
        offs = [c * per for c in range(n_cl)] if segmented else [0] * n_cl
        ne = [int(v) for v in rng.integers(1, 200, oc)] if rng.integers(0, 2) else None
        rin = ([int(v) for v in rng.integers(0, 1 << 20, n_cl)], int(rng.integers(0, 1 << 20)), offs, oc * 16, 0, ne)
        if segmented and rng.integers(0, 4):
            c = int(rng.integers(0, n_cl))
            sub = ([c * per, 0, 0, 0], [per, 1, 1, 4])
        else:
            lo = int(rng.integers(0, oc - 1))
            sub = ([lo, 0, 0, 0], [int(rng.integers(1, oc - lo + 1)), 1, 1, 4])
        t = TType([oc, 1, 1, 4], abi.VF_DT_I32)
        s = _relocate(ContentSetup(t), rin).subview(*sub)
        so = s.optimized()
        a = ContentAttr(tab, t, s).fold(be)
        b = ContentAttr(tab, t, so).fold(be)
        assert a.type == b.type and np.array_equal(a.bytes(), b.bytes()), (rin, sub)
        swapped += so.names()[0] == K.VF_T_SUBVIEW
    assert swapped > n // 4


def test_relocate_swap_folds_to_the_same_table_on_the_oracle(oracle):
    _relocate_fold_pair(oracle, 31)


@pytest.mark.gpu
def test_relocate_swap_folds_to_the_same_table_on_the_gpu(gpu):
    _relocate_fold_pair(gpu, 32)


def _per_axis(axis, n):
    # the reference's test types: u8 storage, f16 expressed, scales 1..n, zero points 0 (CS:478-496)
    return Elem.per_axis(U8, F16, [float(i + 1) for i in range(n)], [0] * n, axis, 0, 255)


# CS:1377-1403 swapChangeShapeAndElemTypeAndSubViewParams: base shape, (cast axis, n), (changeShape shape, axis, n),
# SubView -> expected cast scales, changeShape (shape, axis, scales), SubView.
CHANGE_SHAPE_SWAPS = [
    ([1, 4, 1, 2], (1, 4), ([4, 2, 1, 1], 0, 4), ([0, 0, 0, 0], [3, 2, 1, 1]),
     [1.0, 2.0, 3.0], ([3, 2, 1, 1], 0, [1.0, 2.0, 3.0]), ([0, 0, 0, 0], [1, 3, 1, 2])),
    ([1, 4, 1, 2], (1, 4), ([4, 2, 1, 1], 0, 4), ([1, 0, 0, 0], [2, 2, 1, 1]),
     [2.0, 3.0], ([2, 2, 1, 1], 0, [2.0, 3.0]), ([0, 1, 0, 0], [1, 2, 1, 2])),
    ([1, 4, 2, 2], (1, 4), ([1, 4, 4], 1, 4), ([0, 0, 0], [1, 2, 4]),
     [1.0, 2.0], ([1, 2, 4], 1, [1.0, 2.0]), ([0, 0, 0, 0], [1, 2, 2, 2])),
    ([1, 8, 4], (1, 8), ([1, 8, 2, 2], 1, 8), ([0, 1, 0, 0], [1, 4, 2, 2]),
     [2.0, 3.0, 4.0, 5.0], ([1, 4, 2, 2], 1, [2.0, 3.0, 4.0, 5.0]), ([0, 1, 0], [1, 4, 4])),
    ([1, 8, 6, 4, 3, 3], (1, 8), ([8, 6, 4, 9], 0, 8), ([2, 1, 0, 0], [4, 3, 4, 9]),
     [3.0, 4.0, 5.0, 6.0], ([4, 3, 4, 9], 0, [3.0, 4.0, 5.0, 6.0]), ([0, 2, 1, 0, 0, 0], [1, 4, 3, 4, 3, 3])),
]


@pytest.mark.parametrize("base,cast,change,sub,exp_cast,exp_change,exp_sub", CHANGE_SHAPE_SWAPS)
def test_swap_change_shape_and_elem_type_and_subview(base, cast, change, sub, exp_cast, exp_change, exp_sub):
    s = S(base, U8).castElemType(_per_axis(*cast)).changeShapeAndElemType(change[0], _per_axis(change[1], change[2]))
    got = _items(s.subview(*sub).optimized())
    assert got[0] == ("subview", exp_sub[0], exp_sub[1])
    assert got[1][0] == "cast" and got[1][3] == exp_cast
    assert got[2] == ("changeshape", exp_change[0], exp_change[1], exp_change[2])
    assert len(got) == 3


@pytest.mark.parametrize("base,cast,change,sub", [
    ([1, 4, 1, 2], (1, 4), ([8, 1], 0, 8), ([0, 0], [4, 1])),
    ([1, 8, 8, 2], (1, 8), ([1, 8, 4, 4], 1, 8), ([0, 0, 3, 0], [1, 8, 1, 4]))])
def test_do_not_swap_change_shape_and_elem_type_and_subview(base, cast, change, sub):
    # CS:1433-1440
    s = S(base, U8).castElemType(_per_axis(*cast)).changeShapeAndElemType(change[0], _per_axis(change[1], change[2]))
    got = _items(s.subview(*sub).optimized())
    assert [g[0] for g in got] == ["cast", "changeshape", "subview"]
    assert got[1] == ("changeshape", change[0], change[1], [float(i + 1) for i in range(change[2])])
    assert got[2] == ("subview", sub[0], sub[1])


@pytest.mark.parametrize("base,reshape,cast_axis,new_axis", [
    ([2, 3, 1, 1], [1, 2, 3, 1], 1, 2), ([1, 2, 3, 1], [2, 1, 3, 1], 2, 2), ([1, 3, 1, 2], [3, 2, 1, 1], 1, 0)])
def test_swap_quantize_transformations_and_reshape(base, reshape, cast_axis, new_axis):
    # CS:1547-1576: a Reshape behind the Dequantize of a per-axis type moves in front of it as a
    # ChangeShapeAndElemType with the axis found in the new shape
    got = _items(S(base, U8).castElemType(_per_axis(cast_axis, 3)).dequantize().reshape(reshape).optimized())
    assert got[0][0] == "cast" and got[0][3] == [1.0, 2.0, 3.0]
    assert got[1] == ("changeshape", reshape, new_axis, [1.0, 2.0, 3.0])
    assert got[2] == ("dequantize",) and len(got) == 3


def test_swap_per_tensor_quantize_transformations_and_reshape():
    # CS:1578-1602: per-tensor types need no ChangeShapeAndElemType
    q = Elem.uniform(U8, F32, 0.078, 128, 0, 255)
    got = _items(S([16, 32, 1, 1], U8).castElemType(q).dequantize().reshape([16, 8, 2, 2]).optimized())
    assert [g[0] for g in got] == ["cast", "reshape", "dequantize"] and got[1] == ("reshape", [16, 8, 2, 2])


def test_per_axis_reshape_rewrites_fold_to_the_same_bytes(oracle):
    rng = np.random.default_rng(41)
    for base, reshape, axis in (([2, 3, 1, 1], [1, 2, 3, 1], 1), ([1, 2, 3, 1], [2, 1, 3, 1], 2), ([4, 6, 2, 2], [4, 6, 4], 1)):
        t = TType(base, U8)
        x = rng.integers(0, 256, base).astype(np.uint8)
        n = base[axis]
        q = Elem.per_axis(U8, F32, [0.5 * (i + 1) for i in range(n)], [int(v) for v in rng.integers(0, 9, n)], axis, 0, 255)
        s = ContentSetup(t).castElemType(q).dequantize().reshape(reshape)
        so = s.optimized()
        assert K.VF_T_CHANGE_SHAPE_AND_ELEM_TYPE in so.names()
        a, b = ContentAttr(x, t, s).fold(oracle), ContentAttr(x, t, so).fold(oracle)
        assert a.type == b.type and np.array_equal(a.bytes(), b.bytes())


def test_move_reshape_before_and_chains():
    # CS:1480-1545: Reshape moves before Add / Rescale / a plain CastElemType
    assert _items(S([4, 8, 3]).add(1).reshape([1, 2, 1]).optimized())[0][0] == "reshape"
    assert _items(S([4, 8, 3]).rescale(2).reshape([8, 12]).optimized()) == [("reshape", [8, 12]), ("rescale", 2.0)]
    assert _items(S([4, 8, 3], F32).castElemType(F16).reshape([8, 12]).optimized()) == [
        ("reshape", [8, 12]), ("cast", K.VF_ELEM_PLAIN, F16, [], [])]
    # ... but not before a cast to a quantized type (it behaves like QuantCast)
    q = Elem.uniform(U8, F32, 0.1, 0, 0, 255)
    assert _items(S([4, 8, 3], U8).castElemType(q).reshape([8, 12]).optimized())[0][0] == "cast"
    # CS:1692-1719 MoveSubViewReshapeBeforeAdd
    assert _items(S([4, 8, 3]).add(1).subview([0, 1, 1], [1, 4, 2]).reshape([1, 2, 4]).optimized()) == [
        ("subview", [0, 1, 1], [1, 4, 2]), ("reshape", [1, 2, 4]), ("add", 1.0)]
    # CS:1094-1130 SwapMemPermAndSubViewMultipleInstances
    s = S([4096, 11008, 1, 1]).transpose(HCNW).subview([0, 8192, 0, 0], [1, 2816, 4096, 1])
    s = s.subview([0, 0, 0, 0], [1, 2816, 320, 1]).reorder(NHWC).subview([0, 1000, 0, 0], [1, 1816, 320, 1])
    s = s.subview([0, 0, 0, 0], [1, 1000, 320, 1]).reshape([10, 100, 32, 10])
    assert _items(s.optimized()) == [("subview", [0, 9192, 0, 0], [320, 1000, 1, 1]), ("transpose", HCNW),
                                     ("reorder", NHWC), ("reshape", [10, 100, 32, 10])]


def test_position_requirements_survive():
    s = S([1, 1, 3, 3], F32).rescale(10.0).bitPack(4).sparsify(False).castElemType(F16)
    assert s.optimized().names() == [K.VF_T_RESCALE, K.VF_T_CAST_ELEM_TYPE, K.VF_T_SPARSIFY, K.VF_T_BIT_PACK]


def _random_chain(rng):
    """A chain over an fp16 [N, C, H, W] tensor mixing the rewritable transformations."""
    shape = [int(rng.integers(2, 5)), int(rng.integers(2, 5)) * 2, int(rng.integers(1, 4)), int(rng.integers(2, 5))]
    t = TType(shape, F16)
    s = ContentSetup(t)
    cur = list(shape)
    for _ in range(int(rng.integers(2, 7))):
        op = int(rng.integers(0, 8))
        if op == 0:
            s = s.add(float(rng.integers(-3, 4)))
        elif op == 1:
            s = s.rescale(float(rng.choice([0.5, 2.0, 0.25])))
        elif op == 2:
            off = [int(rng.integers(0, max(1, d // 2))) for d in cur]
            shp = [int(rng.integers(1, d - o + 1)) for d, o in zip(cur, off)]
            s = s.subview(off, shp)
            cur = shp
        elif op == 3:
            pb = [int(rng.integers(0, 2)) for _ in cur]
            pa = [int(rng.integers(0, 3)) for _ in cur]
            s = s.padWithZero(pb, pa)
            cur = [d + b + a for d, b, a in zip(cur, pb, pa)]
        elif op == 4:
            s = s.reorder(int(rng.choice([0x1234, 0x1342, 0x1243, 0x2134])))
        elif op == 5:
            order = int(rng.choice([0x1243, 0x2134, 0x4321, 0x1342]))
            s = s.transpose(order)
            p = [int(ch) - 1 for ch in f"{order:x}"]
            cur = [cur[p[i]] for i in range(4)]
        elif op == 6:
            s = s.castElemType(F32 if rng.integers(0, 2) else F16)
        else:
            s = s.memPermute(int(rng.choice([0x1234, 0x1342])), int(rng.choice([0x1234, 0x2143, 0x4321])))
            return t, s  # shape bookkeeping ends here
    return t, s


def _fold_pair(be, seed, n=120):
    rng = np.random.default_rng(seed)
    shorter = 0
    for _ in range(n):
        t, s = _random_chain(rng)
        x = rng.standard_normal(t.shape).astype(np.float16)
        try:
            a = ContentAttr(x, t, s).fold(be)
        except Exception:
            continue  # the random chain itself is invalid (e.g. a view outside the tensor after a transpose)
        so = s.optimized()
        b = ContentAttr(x, t, so).fold(be)
        assert a.type == b.type, (s.names(), so.names())
        assert np.array_equal(a.bytes(), b.bytes()), (s.names(), so.names())
        shorter += len(so.names()) < len(s.names())
    assert shorter > n // 10


def test_optimised_list_folds_to_the_same_bytes_on_the_oracle(oracle):
    _fold_pair(oracle, 21)


@pytest.mark.gpu
def test_optimised_list_folds_to_the_same_bytes_on_the_gpu(gpu):
    _fold_pair(gpu, 22)
