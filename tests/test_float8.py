"""8-bit floats: the oracle against the reference's own unit vectors
(tests/unit/vpux_utils/core/float8_e4m3_tests.cpp cited as E4:lines, float8_e5m2_tests.cpp as E5:lines), then the
GPU against the oracle on every code and on a dense sample of floats, through the fold path (CastElemType +
copyTo is CvtHelper<float8>::cvt, content.hpp:66-79), and Sparsify / GetSparsityMap on 8-bit float weights
(sparsify.cpp:197-200, get_sparsity_map.cpp:111-116)."""
import math

import numpy as np
import pytest

from vpux_plugin_b200 import abi
from vpux_plugin_b200.abi import TType
from vpux_plugin_b200.const import ContentAttr, ContentSetup

F32, E4, E5 = abi.VF_DT_F32, abi.VF_DT_F8E4M3FN, abi.VF_DT_F8E5M2


def test_e4m3_reference_vectors(oracle):
    inf = float("inf")
    assert oracle.f32_to_f8(inf) == 0x7F and oracle.f32_to_f8(-inf) == 0xFF          # E4:24-34: no infinity, NaN
    assert oracle.f32_to_f8(float("nan")) == 0x7F                                      # E4:98-104
    assert oracle.f32_to_f8(0.0009765625) == 0x00                                      # E4:156-160 half the lowest subnormal
    assert oracle.f32_to_f8(0.00097656273283064365387) == 0x01                         # E4:162-166 just above it
    assert oracle.f32_to_f8(0.129) == 0x20 and oracle.f32_to_f8(-0.281) == 0xA9        # E4:168-180
    assert oracle.f32_to_f8(460.0) == 0x7E and oracle.f32_to_f8(560.0) == 0x7F         # E4:182-194
    assert oracle.f32_to_f8(-460.0) == 0xFE and oracle.f32_to_f8(-760.0) == 0xFF       # E4:196-208
    assert oracle.f8_to_f32(0b00001000) == 2.0 ** -6 and oracle.f8_to_f32(0b01111110) == 448.0  # E4:116-128 min / max
    assert oracle.f8_to_f32(0b00000001) == 2.0 ** -9                                   # E4:137-142 denorm_min
    # E4:224-283: the table of all 256 codes — subnormals m * 2^-9, normals (1 + m/8) * 2^(e-7), 0x7f / 0xff NaN —
    # decodes to those values and each value encodes back to its code
    for code in range(256):
        e, m, neg = (code >> 3) & 15, code & 7, code >> 7
        v = oracle.f8_to_f32(code)
        if code & 0x7F == 0x7F:
            assert math.isnan(v)
            continue
        exp = m * 2.0 ** -9 if e == 0 else (1 + m / 8) * 2.0 ** (e - 7)
        assert v == (-exp if neg else exp) and math.copysign(1, v) == (-1 if neg else 1)
        assert oracle.f32_to_f8(v) == code


def test_e5m2_reference_vectors(oracle):
    inf = float("inf")
    f = lambda v: oracle.f32_to_f8(v, e5m2=True)
    assert f(inf) == 0b01111100 and f(-inf) == 0b11111100                              # E5:27-38
    assert f(float("nan")) == 0b01111110                                               # E5:133-139
    assert f(0.00006103515625) == 0b00000100 and f(57344.0) == 0b01111011              # E5:152-164 min / max
    assert f(-57344.0) == 0b11111011 and f(0.0000152587890625) == 0b00000001           # E5:166-178
    assert f(65520.0) == 0b01111100 and f(65519.9) == 0b01111011                       # E5:192-202
    assert f(-65520.0) == 0b11111100 and f(-65519.9) == 0b11111011                     # E5:204-214
    assert oracle.f8_to_f32(0b00111010, e5m2=True) == 0.75                             # E5:21-25
    for code in range(256):  # E5:300-325: a code is the high byte of the float16 with the same value
        v = oracle.f8_to_f32(code, e5m2=True)
        h = float(np.uint16(code << 8).view(np.float16))
        assert (math.isnan(v) and math.isnan(h)) or v == h
        if not math.isnan(v):
            assert f(v) == code


def _sample():
    rng = np.random.default_rng(8)
    codes = np.arange(256, dtype=np.uint8)
    vals = [rng.standard_normal(20000).astype(np.float32) * s for s in (1e-3, 0.05, 1.0, 30.0, 500.0, 7e4)]
    # ties and neighbours of every representable magnitude, and the edge values
    edges = np.array([0.0, -0.0, np.inf, -np.inf, np.nan, 1e-30, -1e-30, 2.0 ** -10, 2.0 ** -17, 448.0, 464.0, 465.0, 57344.0,
                      61440.0, 65504.0, 65520.0, 1e38], np.float32)
    grid = np.concatenate([np.float32(2.0) ** np.arange(-20, 18, dtype=np.float32) * np.float32(1 + k / 32) for k in range(32)])
    near = np.concatenate([np.nextafter(grid, np.float32(np.inf)), np.nextafter(grid, np.float32(-np.inf))])
    return codes, np.concatenate(vals + [edges, grid, near, -grid, -near]).astype(np.float32)


@pytest.mark.gpu
@pytest.mark.parametrize("dt", [E4, E5])
def test_float8_conversions_match_the_oracle(gpu, oracle, dt):
    codes, vals = _sample()
    t = TType([len(vals)], F32)
    a = ContentAttr(vals, t, ContentSetup(t).castElemType(dt)).fold(gpu).bytes()
    b = ContentAttr(vals, t, ContentSetup(t).castElemType(dt)).fold(oracle).bytes()
    assert np.array_equal(a, b), vals[np.nonzero(a != b)[0][:8]]
    tc = TType([256], dt)
    a = ContentAttr(codes, tc, ContentSetup(tc).castElemType(F32)).fold(gpu).bytes()
    b = ContentAttr(codes, tc, ContentSetup(tc).castElemType(F32)).fold(oracle).bytes()
    assert np.array_equal(a, b)
    # 8-bit float storage read as integers and as f16 (checked_cast through float)
    small = codes[(codes & 0x7F) < 0x50]
    ts = TType([len(small)], dt)
    for to in (abi.VF_DT_I32, abi.VF_DT_F16):
        a = ContentAttr(small, ts, ContentSetup(ts).castElemType(to)).fold(gpu).bytes()
        b = ContentAttr(small, ts, ContentSetup(ts).castElemType(to)).fold(oracle).bytes()
        assert np.array_equal(a, b)


@pytest.mark.gpu
@pytest.mark.parametrize("dt", [E4, E5])
def test_float8_rounding_of_every_exponent_and_boundary(gpu, oracle, dt):
    """Every sign, exponent and leading seven mantissa bits of a float (all rounding boundaries of a 2- or 3-bit
    mantissa lie there, subnormal results included) with the bits below them all clear, lowest set, just below,
    on and just above the half, and all set; from f32, and the f16 / bf16 values among them from their own type."""
    hi = np.arange(65536, dtype=np.uint32) << 16
    lows = np.array([0x0000, 0x0001, 0x7FFF, 0x8000, 0x8001, 0xFFFF], np.uint32)
    vals = (hi[:, None] | lows[None, :]).reshape(-1).view(np.float32)
    t = TType([len(vals)], F32)
    a = ContentAttr(vals, t, ContentSetup(t).castElemType(dt)).fold(gpu).bytes()
    b = ContentAttr(vals, t, ContentSetup(t).castElemType(dt)).fold(oracle).bytes()
    assert np.array_equal(a, b), vals[np.nonzero(a != b)[0][:8]]
    halves = np.arange(65536, dtype=np.uint16)
    for src in (abi.VF_DT_F16, abi.VF_DT_BF16):
        th = TType([65536], src)
        a = ContentAttr(halves, th, ContentSetup(th).castElemType(dt)).fold(gpu).bytes()
        b = ContentAttr(halves, th, ContentSetup(th).castElemType(dt)).fold(oracle).bytes()
        assert np.array_equal(a, b), halves[np.nonzero(a != b)[0][:8]]


@pytest.mark.gpu
@pytest.mark.parametrize("dt", [E4, E5])
def test_float8_sparsity(gpu, oracle, dt):
    rng = np.random.default_rng(dt)
    shape = [24, 16, 3, 3]
    x = rng.integers(0, 256, shape).astype(np.uint8)
    x[rng.random(shape) < 0.5] = 0
    x[rng.random(shape) < 0.1] = 0x80  # -0.0 counts as zero
    t = TType(shape, dt)
    for s in (ContentSetup(t).getSparsityMap(), ContentSetup(t).sparsify(False), ContentSetup(t).reorder(abi.ORDER_NHWC).sparsify(False)):
        a, b = ContentAttr(x, t, s).fold(gpu), ContentAttr(x, t, s).fold(oracle)
        assert a.type == b.type and a.written == b.written and np.array_equal(a.bytes(), b.bytes())
    c, keep = abi.make_content(t, x, dt, False)
    counts = oracle.nnz_per_oc(c, shape[0])
    assert np.array_equal(gpu.nnz_per_oc(c, shape[0]), counts)
    assert np.array_equal(counts, ((x.reshape(shape[0], -1) & 0x7F) != 0).sum(axis=1))


@pytest.mark.gpu
def test_float16_decodes_every_code_like_the_oracle(gpu, oracle):
    """float16::operator float widens the bits: NaNs keep sign and payload (float16.cpp:118-144)."""
    codes = np.arange(65536, dtype=np.uint16).view(np.float16)
    t = TType([65536], abi.VF_DT_F16)
    a = ContentAttr(codes, t, ContentSetup(t).castElemType(F32)).fold(gpu).bytes()
    b = ContentAttr(codes, t, ContentSetup(t).castElemType(F32)).fold(oracle).bytes()
    assert np.array_equal(a, b)
