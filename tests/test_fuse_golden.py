"""#const.Fuse against the folded constants of the reference's own lit test
(tests/lit/NPU/dialect/const/passes/constant_folding.mlir:627-676, extracted into tests/golden/fuse_golden.json by
tests/golden/make_fuse_golden.py): weights table and weights, each folded and materialised like copyTo(), laid
end to end (fuse_transform.cpp:31-63). The oracle folds the parts one by one; the GPU goes through vf_fuse."""
import json
import os

import numpy as np
import pytest

from vpux_plugin_b200 import abi
from vpux_plugin_b200.abi import Elem, TType
from vpux_plugin_b200.const import ContentAttr, ContentSetup

F16, I32, I8, I4 = abi.VF_DT_F16, abi.VF_DT_I32, abi.VF_DT_I8, abi.VF_DT_I4
GOLD = json.load(open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "fuse_golden.json")))


def _parts(name):
    g = GOLD[name]
    tt = TType([16, 1, 1, 4], I32)
    tv = np.asarray(g["weights_table"]["values"], np.int32)
    table = ContentAttr(tv, tt, ContentSetup(tt), is_splat=tv.size == 1)
    wv = np.asarray(g["weights"]["values"], np.float16)
    if name == "FoldSplatFusedConstant":  # :632-636 [CastElemType<si4>, CastElemType<!quant.uniform<i4:f16, 1.15...>>, Reorder<NHWC>]
        wt = TType([16, 1, 1, 4], F16)
        q = Elem.uniform(I4, F16, 1.1534313725490195, 0, -8, 7)
        s = ContentSetup(wt).castElemType(I4).castElemType(q).reorder(abi.ORDER_NHWC)
    elif name == "FoldFusedSignedQuantizedWeightsMixedPrecision":  # :648-652 si8, !quant.uniform<i8<-127:127>:f16, 0.0078...>
        wt = TType([16, 16, 1, 1], F16)
        q = Elem.uniform(I8, F16, 0.0078740157480314959, 0, -127, 127)
        s = ContentSetup(wt).castElemType(I8).castElemType(q).reorder(abi.ORDER_NHWC)
    else:  # :663-667 [Reorder<NHWC>] into a fused constant of f16
        wt = TType([16, 16, 1, 1], F16)
        s = ContentSetup(wt).reorder(abi.ORDER_NHWC)
    weights = ContentAttr(wv, wt, s, is_splat=wv.size == 1)
    if g["result"]["type"].endswith("xf16"):
        expected = np.asarray(g["result"]["values"], np.float16).view(np.uint8)
    else:
        expected = np.asarray(g["result"]["values"], np.uint8)
    return [table, weights, None, None], expected


@pytest.mark.parametrize("name", sorted(GOLD))
def test_oracle_folds_the_fused_parts_like_the_reference(name, oracle):
    parts, expected = _parts(name)
    got = np.concatenate([p.fold(oracle).bytes() for p in parts if p is not None])
    assert got.size == expected.size and np.array_equal(got, expected)


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(GOLD))
def test_vf_fuse_matches_the_reference(name, gpu):
    parts, expected = _parts(name)
    fused, where = gpu.fuse(parts, expected.size)
    assert fused.size == expected.size and np.array_equal(fused, expected)
    assert where[0] == (0, 256) and where[1][0] == 256 and where[2][1] == 0 and where[3][1] == 0
