"""Known-answer cases transcribed from the reference's own tests.

Each function takes a backend (the CPU oracle or the GPU library — both expose
infer_type / fold / weights_table) and asserts the expected bytes. `UT` is
tests/unit/vpux_compiler/dialect/const/content_tests.cpp of the reference; lit
files are under tests/lit/NPU.
"""
import numpy as np

from vpux_plugin_b200 import abi
from vpux_plugin_b200.abi import Elem, TType
from vpux_plugin_b200.const import ContentAttr, ContentSetup

F32, F16, I8, U8, I32 = abi.VF_DT_F32, abi.VF_DT_F16, abi.VF_DT_I8, abi.VF_DT_U8, abi.VF_DT_I32


def _gen(n, dt):
    return np.arange(n).astype(dt)  # generateValues<T>, UT:43-51


def quantize(be):
    """UT:2440-2469 Quantize"""
    t = TType([1, 16], F32)
    vals = np.array([-2.0 + 0.25 * i for i in range(16)], np.float32)
    q = Elem.uniform(I8, F32, 1.0 / 127.0, 56, -127, 127)
    out = ContentAttr(vals, t, ContentSetup(t).quantize(q)).fold(be)
    assert out.type == TType([1, 16], I8)
    exp = [-127, -127, -127, -103, -71, -39, -7, 24, 56, 88, 120, 127, 127, 127, 127, 127]
    assert out.values(np.int8).tolist() == exp


def per_axis_quantize(be):
    """UT:2471-2510 PerAxisQuantize"""
    t = TType([2, 16], F32)
    vals = np.array([[-2.0 + 0.25 * j for j in range(16)]] * 2, np.float32)
    q = Elem.per_axis(I8, F32, [1.0 / 127.0, 0.003], [56, -21], 0, -127, 127)
    out = ContentAttr(vals, t, ContentSetup(t).quantize(q)).fold(be)
    a0 = [-127, -127, -127, -103, -71, -39, -7, 24, 56, 88, 120, 127, 127, 127, 127, 127]
    a1 = [-127, -127, -127, -127, -127, -127, -127, -104, -21, 62, 127, 127, 127, 127, 127, 127]
    assert out.values(np.int8).tolist() == a0 + a1


def dequantize_quantize(be):
    """UT:2512-2540 DequantizeQuantize: castElemType(q).dequantize().quantize(q) is the identity"""
    t = TType([1, 16], I8)
    vals = np.array([-120 + 15 * i for i in range(16)], np.int8)
    q = Elem.uniform(I8, F16, 0.003, 56, -120, 120)
    out = ContentAttr(vals, t, ContentSetup(t).castElemType(q).dequantize().quantize(q)).fold(be)
    assert out.values(np.int8).tolist() == vals.tolist()


def quant_cast(be):
    """UT:726-752 QuantCast (CastElemType to a quantized type moves the buffer)"""
    t = TType([1, 16], U8)
    vals = _gen(16, np.uint8)
    q = Elem.uniform(U8, F32, 0.078431372549019607, 128, 0, 255)
    out = ContentAttr(vals, t, ContentSetup(t).castElemType(q)).fold(be)
    assert out.type == TType([1, 16], q)
    assert out.values(np.uint8).tolist() == list(range(16))


def dequantize(be):
    """UT:754-788 Dequantize"""
    t = TType([1, 16], I8)
    vals = np.array([((i % 3) - 1) * 127 for i in range(16)], np.int8)
    q = Elem.uniform(I8, F32, 2.0 / 254.0, 0, -127, 127)
    out = ContentAttr(vals, t, ContentSetup(t).castElemType(q).dequantize()).fold(be)
    assert out.type == TType([1, 16], F32)
    exp = np.array([float((i % 3) - 1) for i in range(16)], np.float32)
    np.testing.assert_allclose(out.values(np.float32), exp, rtol=4 * np.finfo(np.float32).eps)  # EXPECT_FLOAT_EQ


def reorder(be):
    """UT:906-939 Reorder NCHW -> NHWC"""
    N, Cc, H, W = 1, 2, 2, 2
    t = TType([N, Cc, H, W], F32)
    vals = _gen(8, np.float32)
    out = ContentAttr(vals, t, ContentSetup(t).reorder(abi.ORDER_NHWC)).fold(be)
    assert out.type == TType([N, Cc, H, W], F32, abi.ORDER_NHWC)
    got = out.values(np.float32)
    for c in range(Cc):
        for h in range(H):
            for w in range(W):
                assert got[c + w * Cc + h * Cc * W] == vals[w + h * W + c * W * H]


def _check_padded(act, exp, buf, pad, zp, act_off=0, org_off=0):  # checkPaddedBuffer, UT:63-89
    IC, IH, IW = buf
    PC, PH, PW = pad
    for c in range(IC + 2 * PC):
        for h in range(IH + 2 * PH):
            for w in range(IW + 2 * PW):
                ni = w + h * (IW + 2 * PW) + c * (IW + 2 * PW) * (IH + 2 * PH) + act_off
                if c < PC or c >= IC + PC or h < PH or h >= IH + PH or w < PW or w >= IW + PW:
                    assert act[ni] == zp, (c, h, w)
                else:
                    oi = (w - PW) + (h - PH) * IW + (c - PC) * IW * IH + org_off
                    assert act[ni] == exp[oi], (c, h, w)


def pad(be):
    """UT:976-1002 Pad"""
    t = TType([1, 2, 3], I32)
    vals = _gen(6, np.int32)
    out = ContentAttr(vals, t, ContentSetup(t).padWithZero([1, 1, 1], [1, 1, 1])).fold(be)
    assert out.type == TType([3, 4, 5], I32)
    _check_padded(out.values(np.int32), vals, (1, 2, 3), (1, 1, 1), 0)


def pad_splat(be):
    """UT:1004-1030 PadSplat"""
    t = TType([1, 2, 3], I32)
    out = ContentAttr(np.array([42], np.int32), t, ContentSetup(t).padWithZero([1, 1, 1], [1, 1, 1]),
                      is_splat=True).fold(be)
    assert not out.is_splat
    _check_padded(out.values(np.int32), np.full(6, 42, np.int32), (1, 2, 3), (1, 1, 1), 0)


def pad_uniform_quant(be):
    """UT:1032-1070 PadUniformQuant: f32 storage, padding holds the zero point"""
    OC, IC, IH, IW = 2, 1, 2, 3
    t = TType([OC, IC, IH, IW], F32)
    vals = _gen(12, np.float32)
    zp = 128
    q = Elem.uniform(U8, F32, 0.078431372549019607, zp, 0, 255)
    P = 2
    attr = ContentAttr(vals, t, ContentSetup(t).castElemType(q).padWithZero([0, P, P, P], [0, P, P, P]))
    out = attr.fold(be)
    # the bytes come back through copyTo in the logical u8 type; the storage was f32 (values 0..11 and 128.0)
    got = out.values(np.uint8).astype(np.float32)
    for oc in range(OC):
        _check_padded(got, vals, (IC, IH, IW), (P, P, P), zp, oc * (IC + 2 * P) * (IW + 2 * P) * (IH + 2 * P),
                      oc * IC * IW * IH)


def pad_per_axis_quant(be):
    """UT:1072-1123 PadPerAxisQuant: scales/zps replicated onto the padded channels"""
    OC, IC, IH, IW = 2, 1, 2, 3
    t = TType([OC, IC, IH, IW], F32)
    vals = _gen(12, np.float32)
    zp = 127
    q = Elem.per_axis(U8, F32, [0.5, 0.5], [zp, zp], 0, 0, 255)
    POC = PIC = PH = PW = 2
    attr = ContentAttr(vals, t, ContentSetup(t).castElemType(q).padWithZero([POC, PIC, PH, PW], [POC, PIC, PH, PW]))
    out = attr.fold(be)
    assert out.type.elem.zps.tolist() == [zp] * (OC + 2 * POC)
    assert out.type.elem.scales.tolist() == [0.5] * (OC + 2 * POC)
    got = out.values(np.uint8).astype(np.float32)
    ch = IC * IW * IH
    exp = np.concatenate([np.full(ch * POC, zp, np.float32), vals, np.full(ch * POC, zp, np.float32)])
    for oc in range(OC + 2 * POC):
        _check_padded(got, exp, (IC, IH, IW), (PIC, PH, PW), zp, oc * (IC + 2 * PIC) * (IW + 2 * PW) * (IH + 2 * PH),
                      oc * ch)


def bit_pack(be):
    """UT:1246-1274 BitPack"""
    t = TType([1, 2, 3], I8)
    vals = np.array([1, 2, 3, 4, 5, 6], np.int8)
    out = ContentAttr(vals, t, ContentSetup(t).bitPack(4)).fold(be)
    assert out.type == TType([1, 2, 3], abi.VF_DT_I4)
    assert out.bytes().tolist() == [0x21, 0x43, 0x65]


def bit_pack_quant(be):
    """UT:1276-1315 BitPackQuant"""
    t = TType([1, 2, 3], I8)
    vals = np.array([1, 2, 3, 1, 2, 3], np.int8)
    q = Elem.uniform(I8, F32, 1.0, 0, -4, 3)
    out = ContentAttr(vals, t, ContentSetup(t).castElemType(q).bitPack(4)).fold(be)
    assert out.type == TType([1, 2, 3], Elem.uniform(abi.VF_DT_I4, F32, 1.0, 0, -4, 3))
    assert out.bytes().tolist() == [0x21, 0x13, 0x32]


def get_sparsity_map(be):
    """UT:1536-1569 GetSparsityMap"""
    t = TType([1, 1, 2, 8], U8)
    vals = np.array([0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 0, 11, 0, 13, 14, 15], np.uint8)
    out = ContentAttr(vals, t, ContentSetup(t).getSparsityMap()).fold(be)
    assert out.type == TType([1, 1, 1, 128], abi.VF_DT_I1)
    assert out.bytes().tolist() == [0xFE, 0xEB] + [0] * 14


def get_sparsity_map_quantized(be):
    """UT:1571-1618 GetSparsityMapQuantized (zero point 7 marks the sparse value)"""
    t = TType([1, 1, 2, 8], U8)
    vals = np.array([7, 0, 1, 2, 3, 4, 5, 6, 7, 8, 7, 10, 7, 12, 13, 14], np.uint8)
    q = Elem.uniform(U8, F32, 1.0, 7, 0, 14)
    out = ContentAttr(vals, t, ContentSetup(t).castElemType(q).getSparsityMap()).fold(be)
    assert out.bytes().tolist() == [0xFE, 0xEA] + [0] * 14


_SP_VALS = np.array([0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 0, 11, 0, 13, 14, 15,
                     16, 0, 18, 19, 20, 0, 22, 23, 24, 25, 26, 0, 0, 29, 30, 31], np.uint8)
_SP_EXP = [1, 2, 3, 4, 5, 6, 7, 8, 9, 11, 13, 14, 15, 0, 0, 0,
           16, 18, 19, 20, 22, 23, 24, 25, 26, 29, 30, 31, 0, 0, 0, 0]


def sparsify(be):
    """UT:1620-1646 Sparsify<false>: folded bytes are compressed, the attribute type is not"""
    t = TType([2, 1, 2, 8], U8)
    attr = ContentAttr(_SP_VALS, t, ContentSetup(t).sparsify(False))
    out = attr.fold(be)
    assert attr.infer(be)[0] == t  # inferred (attribute) type stays uncompressed
    assert out.type == TType([32, 1, 1, 1], U8)  # folded content type is the compressed one
    assert out.bytes().tolist() == _SP_EXP


def sparsify_true(be):
    """UT:1648-1679 Sparsify<true, numActualElements>"""
    t = TType([2, 1, 2, 8], U8)
    attr = ContentAttr(_SP_VALS, t, ContentSetup(t).sparsify(True, [13, 12]))
    out = attr.fold(be)
    assert attr.infer(be)[0] == TType([32, 1, 1, 1], U8)
    assert out.type == TType([32, 1, 1, 1], U8)
    assert out.bytes().tolist() == _SP_EXP


def sparsify_quantized(be):
    """UT:1681-1722 SparsifyQuantized (zero point 16)"""
    t = TType([2, 1, 2, 8], U8)
    vals = np.array([16, 1, 2, 3, 4, 5, 6, 7, 8, 9, 16, 11, 16, 13, 14, 15,
                     16, 16, 18, 19, 20, 16, 22, 23, 24, 25, 26, 16, 16, 29, 30, 31], np.uint8)
    exp = [1, 2, 3, 4, 5, 6, 7, 8, 9, 11, 13, 14, 15, 0, 0, 0,
           18, 19, 20, 22, 23, 24, 25, 26, 29, 30, 31, 0, 0, 0, 0, 0]
    q = Elem.uniform(U8, F32, 1.0, 16, 0, 31)
    out = ContentAttr(vals, t, ContentSetup(t).castElemType(q).sparsify(False)).fold(be)
    assert out.bytes().tolist() == exp


def position_requirement(be):
    """UT:1724-1749 PositionRequirement: SwizzleConstant is LAST, Sparsify PREFERRED_LAST; the same with BitPack"""
    t = TType([1, 1, 3, 3], F32)
    s = ContentSetup(t).rescale(10.0).swizzleConstant(5, abi.VF_ARCH_NPU37XX).sparsify(False).castElemType(F16)
    assert s.names() == [abi.VF_T_RESCALE, abi.VF_T_CAST_ELEM_TYPE, abi.VF_T_SPARSIFY, abi.VF_T_SWIZZLE_CONSTANT]
    s = ContentSetup(t).rescale(10.0).bitPack(4).sparsify(False).castElemType(F16)
    assert s.names() == [abi.VF_T_RESCALE, abi.VF_T_CAST_ELEM_TYPE, abi.VF_T_SPARSIFY, abi.VF_T_BIT_PACK]


def convert_elem_type_i8_u8(be):
    """UT:2276-2330 ConvertElemType Roundtrip, I8_to_U8: values shift by zpOut - zpIn = 128 and back"""
    t = TType([1, 2, 3, 4], F16)
    i8 = Elem.uniform(I8, F32, 0.5, 0, -128, 127)
    u8 = Elem.uniform(U8, F32, 0.5, 128, 0, 255)
    vals = np.array([(-128 + i) if i % 2 == 0 else (127 - i) for i in range(24)], np.float16)
    s = ContentSetup(t).castElemType(i8).convertElemType(u8)
    out = ContentAttr(vals, t, s).fold(be)
    assert out.values(np.uint8).astype(np.float32).tolist() == (vals.astype(np.float32) + 128).tolist()
    back = ContentAttr(vals, t, s.convertElemType(i8)).fold(be)
    assert back.values(np.int8).astype(np.float32).tolist() == vals.astype(np.float32).tolist()


def convert_elem_type_u4_i4(be):
    """UT:2332-2353 U4_to_I4: offset -8; copyTo packs two 4-bit values per byte (content.cpp:131-152)"""
    t = TType([1, 2, 3, 4], F16)
    u4 = Elem.uniform(abi.VF_DT_U4, F32, 1.0, 8, 0, 15)
    i4 = Elem.uniform(abi.VF_DT_I4, F32, 1.0, 0, -8, 7)
    vals = np.array([i % 15 for i in range(24)], np.float16)
    out = ContentAttr(vals, t, ContentSetup(t).castElemType(u4).convertElemType(i4)).fold(be)
    packed = out.bytes()
    assert len(packed) == 12
    nib = np.stack([packed & 0xF, packed >> 4], axis=1).reshape(-1).astype(np.int64)
    exp = (vals.astype(np.int64) - 8) & 0xF
    assert nib.tolist() == exp.tolist()


def quantize_splat(be):
    """lit dialect/const/passes/constant_folding.mlir:695-709 QuantizeSplat: 5.0 / 0.5 -> 10"""
    t = TType([1, 16, 3, 3], F16)
    q = Elem.uniform(U8, F16, 0.5, 0, 0, 255)
    out = ContentAttr(np.array([5.0], np.float16), t, ContentSetup(t).quantize(q), is_splat=True).fold(be)
    assert out.values(np.uint8).tolist() == [10] * 144


def const_fold_chain(be):
    """lit dialect/const/passes/constant_folding.mlir:9-30 ConstFold: cast chain + Dequantize + Reorder<YXOI>"""
    t = TType([16, 3, 1, 1], F32)
    q = Elem.uniform(U8, F16, 0.0039215686274509803, 0, 0, 255)
    s = ContentSetup(t).castElemType(F16).castElemType(U8).castElemType(q).dequantize().reorder(0x3412)
    attr = ContentAttr(np.array([1.0], np.float32), t, s, is_splat=True)
    out = attr.fold(be)
    assert out.type == TType([16, 3, 1, 1], F16, 0x3412)
    v = out.values(np.float16)
    assert v.shape == (48,) and (v == np.float16(np.float32(0.0039215686274509803))).all()


def _wt_desc(in_elem, out_elem, w_elem, oc, wbase, wstep, sbase, sstep):
    d = abi.WeightsTableDesc()
    d.in_elem, d.out_elem, d.weights_elem = in_elem.pod(), out_elem.pod(), w_elem.pod()
    d.oc = oc
    d.weights_ptr_base, d.weights_ptr_step = wbase, wstep
    d.sparsity_ptr_base, d.sparsity_ptr_step = sbase, sstep
    return d, (in_elem, out_elem, w_elem)


def weights_table_fixed_point(be):
    """lit dialect/VPU/passes/lower_ops_to_se_nce_37XX_40XX.mlir:9-11,58-61: u8 in/out, u8 weights 0.25"""
    d, keep = _wt_desc(Elem.uniform(U8, F16, 0.0151786074918859, 128, 0, 255),
                       Elem.uniform(U8, F16, 0.0257227579752604, 128, 0, 255),
                       Elem.uniform(U8, F16, 0.25, 0, 0, 255), 16, 0, 64, 0, 0)
    tab = be.weights_table(d, 16).reshape(16, 4)
    assert tab[:, 0].tolist() == [64 * i for i in range(16)]
    assert tab[:, 1].tolist() == [0] * 16
    assert tab[:, 2].tolist() == [1267142912] * 16
    assert tab[:, 3].tolist() == [0] * 16


def weights_table_float_scale(be):
    """lit conversion/passes/IE2VPU/convert_IE_to_VPU_NCE_37XX_40XX.mlir:1026-1050: f16 activations, i4
    weights of scale 1.3385416666666667 -> column 2 holds the fp32 bit pattern of the scale"""
    d, keep = _wt_desc(Elem(F16), Elem(F16), Elem.uniform(abi.VF_DT_I4, F16, 1.3385416666666667, 0, -8, 7), 16, 0,
                       16, 0, 0)
    tab = be.weights_table(d, 16).reshape(16, 4)
    assert tab[:, 0].tolist() == [16 * i for i in range(16)]
    assert tab[:, 2].tolist() == [1068193109] * 16
    assert tab[:, 3].tolist() == [0] * 16


def copy_to_i4(be):
    """UT:440-466 CopyTo_I4: CastElemType to a 4-bit integer packs two values per byte at copyTo, low nibble first"""
    t = TType([4], U8)
    out = ContentAttr(np.array([1, 7, 10, 15], np.uint8), t, ContentSetup(t).castElemType(abi.VF_DT_U4)).fold(be)
    assert not out.is_splat
    assert out.bytes().tolist() == [0x71, 0xFA]


def copy_to_i1(be):
    """UT:468-496 CopyTo_I1: eight 1-bit values per byte, element 0 in bit 0"""
    t = TType([16], U8)
    vals = np.array([0, 0, 0, 1, 0, 0, 1, 1, 1, 1, 1, 1, 1, 1, 1, 0], np.uint8)
    out = ContentAttr(vals, t, ContentSetup(t).castElemType(abi.VF_DT_I1)).fold(be)
    assert out.bytes().tolist() == [0xC8, 0x7F]


def convert_elem_type_sub_byte(be):
    """tests/unit/vpux_compiler/dialect/const/attributes/convert_elem_type.cpp:41-308 and lit
    dialect/const/passes/constant_folding.mlir:713-830: ConvertElemType unpacks 1- and 4-bit constants to bytes.
    Signless and unsigned 4-bit types take the masking branch (U4 here), signed ones are sign-extended (I4);
    a splat yields the first element of its byte when masking and the last one when sign-extending."""
    U4, I4, I1 = abi.VF_DT_U4, abi.VF_DT_I4, abi.VF_DT_I1
    packed = np.array([0x66, 0x85, 0x2F, 0xDE], np.uint8)

    def run(vals, shape, src, dst, splat=False):
        t = TType(shape, src)
        out = ContentAttr(np.asarray(vals, np.uint8), t, ContentSetup(t).convertElemType(dst), is_splat=splat,
                          storage_dtype=src).fold(be)
        assert out.type == TType(shape, dst) and out.is_splat == splat
        return out.bytes().tolist()

    assert run(packed, [1, 1, 2, 4], U4, U8) == [0x06, 0x06, 0x05, 0x08, 0x0F, 0x02, 0x0E, 0x0D]  # UT:74-106, 141-173
    assert run([0xDD], [1, 1, 2, 4], U4, U8, splat=True) == [0x0D] * 8                              # UT:41-72, 108-139
    assert run(packed, [1, 1, 2, 4], I4, I8) == [0x06, 0x06, 0x05, 0xF8, 0xFF, 0x02, 0xFE, 0xFD]  # UT:208-240
    assert run([0xDD], [1, 1, 2, 4], I4, I8, splat=True) == [0xFD] * 8                              # UT:175-206
    assert run([0x0D, 0x82], [1, 1, 2, 8], I1, I8) == [1, 0, 1, 1, 0, 0, 0, 0, 0, 1, 0, 0, 0, 0, 0, 1]  # UT:275-308
    assert run([0xFF], [1, 1, 2, 8], I1, I8, splat=True) == [1] * 16                                 # UT:242-273
    assert run([0x10, 0x32, 0x54, 0x76], [2, 4], U4, U8) == list(range(8))                         # lit :757-775
    assert run([0x22], [2, 4], U4, U8, splat=True) == [2] * 8                                       # lit :739-755
    assert run([0xEE], [2, 4], I4, I8, splat=True) == [0xFE] * 8                                    # lit :777-793 (-2)


def swizzle_constant(be):
    """UT:1872-2180 SwizzleConstant_*: the result is a flat buffer of the swizzling-aligned size (512 bytes on
    NPU37XX) whose first chunk stays in place; 1-bit and fp16 constants keep their element type, the rest
    become u8; a splat pads with its own bytes and is no longer a splat."""
    arch = abi.VF_ARCH_NPU37XX

    def run(vals, shape, dt, cast=None, splat=False):
        t = TType(shape, dt)
        s = ContentSetup(t)
        if cast is not None:
            s = s.castElemType(cast)
        out = ContentAttr(np.asarray(vals), t, s.swizzleConstant(5, arch), is_splat=splat).fold(be)
        assert not out.is_splat and out.written == 512
        return out

    bits = [0, 0, 0, 1, 0, 0, 1, 1, 1, 1, 1, 1, 1, 1, 1, 0]
    o = run(np.array(bits, np.uint8), [1, 1, 4, 4], U8, cast=abi.VF_DT_I1)          # UT:1872-1909
    assert o.type == TType([4096, 1, 1, 1], abi.VF_DT_I1) and o.bytes()[:2].tolist() == [0xC8, 0x7F]
    o = run(np.array([1, 7, 10, 15], np.uint8), [1, 1, 2, 2], U8, cast=abi.VF_DT_U4)  # UT:1911-1950
    assert o.type == TType([512, 1, 1, 1], U8) and o.bytes()[:2].tolist() == [0x71, 0xFA]
    o = run(np.array([255, 100, 0, 1], np.uint8), [1, 1, 2, 2], U8)                  # UT:1952-1984
    assert o.type == TType([512, 1, 1, 1], U8) and o.bytes()[:4].tolist() == [255, 100, 0, 1]
    o = run(np.array([700, 800, 900, 900], np.float32), [1, 1, 2, 2], F32)           # UT:1986-2018
    assert o.bytes()[:16].view(np.float32).tolist() == [700, 800, 900, 900]
    o = run(np.array([1], np.uint8), [1, 1, 4, 4], U8, cast=abi.VF_DT_I1, splat=True)  # UT:2020-2060
    assert o.bytes().tolist() == [0xFF] * 512
    o = run(np.array([7], np.uint8), [1, 1, 2, 2], U8, splat=True)                   # after UT:2104-2140
    assert o.bytes().tolist() == [7] * 512


def relocate_weights_table(be):
    """lit dialect/const/passes/constant_folding.mlir:566-625 (Relocate*): columns 0 / 1 of each table row are
    rebased on the cluster's weights pointer and the sparsity pointer; the steps between channels come from
    the first two rows; a table inside a larger fused constant is patched over weightsTableSize bytes only;
    with weightsCompression the weights pointers follow the aligned compressed set sizes."""
    I32 = abi.VF_DT_I32

    def run(vals, shape, setup_fn, splat=False):
        t = TType(shape, I32)
        out = ContentAttr(np.asarray(vals, np.int32), t, setup_fn(ContentSetup(t)), is_splat=splat).fold(be)
        return out.values(np.int32).tolist()

    five = [1, 2, 3, 3, 2, 4, 4, 4, 3, 6, 5, 5, 4, 8, 6, 6, 5, 10, 7, 7]
    # :566-581 single cluster, and the same table sliced first (channelOffset = 2)
    assert run(five, [5, 1, 1, 4], lambda s: s.relocateWeightsTablePointers([10], 15, [0], 80, 16)) == \
        [10, 15, 3, 3, 11, 17, 4, 4, 12, 19, 5, 5, 13, 21, 6, 6, 14, 23, 7, 7]
    assert run(five, [5, 1, 1, 4], lambda s: s.subview([2, 0, 0, 0], [2, 1, 1, 4]).relocateWeightsTablePointers(
        [10], 15, [0], 32, 16, channel_offset=2)) == [12, 19, 5, 5, 13, 21, 6, 6]
    # :585-593 a table of 3 rows at the front of a fused constant
    fused = [1, 2, 1, 2, 2, 4, 2, 3, 3, 6, 4, 5, 0, 0, 0, 0]
    assert run(fused, [1, 1, 1, 16], lambda s: s.relocateWeightsTablePointers([10], 15, [0], 48, 16)) == \
        [10, 15, 1, 2, 11, 17, 2, 3, 12, 19, 4, 5, 0, 0, 0, 0]
    # :597-611 two clusters of two channels
    four = five[:16]
    assert run(four, [4, 1, 1, 4], lambda s: s.relocateWeightsTablePointers([10, 20], 5, [0, 2], 64, 16)) == \
        [10, 5, 3, 3, 11, 7, 4, 4, 20, 5, 5, 5, 21, 7, 6, 6]
    assert run(four, [4, 1, 1, 4], lambda s: s.subview([2, 0, 0, 0], [2, 1, 1, 4]).relocateWeightsTablePointers(
        [20], 5, [0], 32, 16, channel_offset=0)) == [20, 5, 5, 5, 21, 7, 6, 6]
    # :615-624 compressed weights: 24 fp16 elements per channel = 48 bytes, five channels sliced away in front
    sparse = [1, 2, 3, 3, 21, 4, 4, 4, 41, 6, 5, 5, 61, 8, 6, 6, 81, 10, 7, 7]
    comp = {"axis": 0, "numElems": [24] * 10, "alignment": 16}
    assert run(sparse, [5, 1, 1, 4], lambda s: s.relocateWeightsTablePointers(
        [10], 15, [0], 80, 16, weights_compression=comp, channel_offset=5)) == \
        [250, 25, 3, 3, 298, 27, 4, 4, 346, 29, 5, 5, 394, 31, 6, 6, 442, 33, 7, 7]
    # a row whose sparsity pointer says "no sparsity" keeps it (relocate_weights_table.cpp:286-289)
    nosp = [0, 0xFFFFFF, 9, 9, 16, 0xFFFFFF, 9, 9]
    assert run(nosp, [2, 1, 1, 4], lambda s: s.relocateWeightsTablePointers([100], 7, [0], 32, 16)) == \
        [100, 0xFFFFFF, 9, 9, 116, 0xFFFFFF, 9, 9]
    # a splat table is filled in first (:207-214): equal rows, so both steps are zero
    assert run([3], [2, 1, 1, 4], lambda s: s.relocateWeightsTablePointers([100], 7, [0], 32, 16), splat=True) == \
        [100, 7, 3, 3, 100, 7, 3, 3]


def reverse(be):
    """UT:813-846 ReverseCWise, UT:848-881 ReverseNWise, UT:883-906 Reverse_Splat: the dims behind the axis are
    reversed as one run."""
    N, C, H, W = 2, 3, 4, 5
    t = TType([N, C, H, W], F32)
    vals = np.arange(N * C * H * W, dtype=np.float32)
    x = vals.reshape(N, C, H, W)
    out = ContentAttr(vals, t, ContentSetup(t).reverse(1)).fold(be)
    assert out.type == t and not out.is_splat
    assert np.array_equal(out.values(np.float32).reshape(N, C, H, W), x[:, :, ::-1, ::-1])
    out = ContentAttr(vals, t, ContentSetup(t).reverse(0)).fold(be)
    assert np.array_equal(out.values(np.float32).reshape(N, C, H, W), x[:, ::-1, ::-1, ::-1])
    out = ContentAttr(np.array([42.0], np.float32), t, ContentSetup(t).reverse(0), is_splat=True).fold(be)
    assert out.is_splat and out.values(np.float32).tolist() == [42.0] * (N * C * H * W)


def expand_dilated(be):
    """UT:1435-1482 ExpandDilated, UT:1484-1533 ExpandDilated_Splat: a 5x5 kernel with dilations 3x3 becomes
    13x13 with zeros between the taps; the result is never a splat."""
    OC, IC, KY, KX, dil = 2, 2, 5, 5, 3
    I32 = abi.VF_DT_I32
    t = TType([OC, IC, KY, KX], I32)
    dK = KY + (KY - 1) * (dil - 1)
    for vals in (np.arange(OC * IC * KY * KX, dtype=np.int32), np.full(OC * IC * KY * KX, 42, np.int32)):
        out = ContentAttr(vals, t, ContentSetup(t).expandDilated([dil, dil])).fold(be)
        assert out.type == TType([OC, IC, dK, dK], I32) and not out.is_splat
        exp = np.zeros((OC, IC, dK, dK), np.int32)
        exp[:, :, ::dil, ::dil] = vals.reshape(OC, IC, KY, KX)
        assert np.array_equal(out.values(np.int32).reshape(OC, IC, dK, dK), exp)


def scalar_mult_inverse(be):
    """UT:2181-2211 ScalarMultInverse, UT:2213-2238 ScalarMultInverse_Splat: 1.f / v in f32."""
    t = TType([1, 2, 3, 4], F32)
    vals = np.arange(24, dtype=np.float32)
    vals[0] = 42.0
    out = ContentAttr(vals, t, ContentSetup(t).scalarMultInverse()).fold(be)
    assert out.type == t and not out.is_splat
    assert np.array_equal(out.values(np.float32), np.float32(1.0) / vals)
    out = ContentAttr(np.array([42.0], np.float32), t, ContentSetup(t).scalarMultInverse(), is_splat=True).fold(be)
    assert out.is_splat and np.array_equal(out.values(np.float32), np.full(24, np.float32(1.0) / np.float32(42.0)))


def change_shape_and_elem_type(be):
    """UT:1752-1776, UT:1778-1820 (per-axis types whose axis moves with the shape), UT:1822-1843 (float storage
    read as si32): only the type changes, the bytes stay."""
    t = TType([2, 1, 1, 8], U8)
    vals = np.arange(16, dtype=np.uint8)
    q = Elem.uniform(U8, F32, 0.078431372549019607, 128, 0, 255)
    out = ContentAttr(vals, t, ContentSetup(t).changeShapeAndElemType([1, 2, 1, 8], q)).fold(be)
    assert out.type == TType([1, 2, 1, 8], q) and not out.is_splat and out.bytes().tolist() == vals.tolist()
    q1 = Elem.per_axis(U8, F16, [0.5, 0.5], [127, 127], 0, 0, 255)
    q2 = Elem.per_axis(U8, F16, [0.5, 0.5], [127, 127], 1, 0, 255)
    s1 = ContentSetup(t).castElemType(q1)
    o1 = ContentAttr(vals, t, s1).fold(be)
    o2 = ContentAttr(vals, t, s1.changeShapeAndElemType([1, 2, 1, 8], q2)).fold(be)
    assert o1.type == TType([2, 1, 1, 8], q1) and o2.type == TType([1, 2, 1, 8], q2) and o1.type != o2.type
    assert o1.bytes().tolist() == vals.tolist() and o2.bytes().tolist() == vals.tolist()
    tf = TType([2, 1, 1, 8], F32)
    fv = np.arange(16, dtype=np.float32)
    out = ContentAttr(fv, tf, ContentSetup(tf).changeShapeAndElemType([1, 2, 1, 8], abi.VF_DT_I32)).fold(be)
    assert out.type == TType([1, 2, 1, 8], abi.VF_DT_I32) and out.values(np.int32).tolist() == list(range(16))


def broadcast(be):
    """lit dialect/VPU/passes/multi_cluster_for_concat_37XX.mlir:234 and add_explicit_padding_before_nce_permute.mlir:265
    (the lists only; no folded values are checked there): a 1x1x1x1 constant broadcast over dim 0, two broadcasts in a
    row, and a non-splat block repeated along a middle dim (broadcast.cpp:94-121)."""
    t = TType([1, 1, 1, 1], F32)
    s = ContentSetup(t).broadcast(0, 16).reshape([16, 1, 1, 1]).castElemType(F16)
    out = ContentAttr(np.array([0.015625], np.float32), t, s).fold(be)
    assert out.type == TType([16, 1, 1, 1], F16) and out.values(np.float16).tolist() == [0.015625] * 16
    t2 = TType([1, 1], F16)
    out = ContentAttr(np.array([3.0], np.float16), t2, ContentSetup(t2).broadcast(1, 77).broadcast(0, 77)).fold(be)
    assert out.type == TType([77, 77], F16) and out.values(np.float16).tolist() == [3.0] * (77 * 77)
    t3 = TType([2, 3, 2], U8)
    x = np.arange(12, dtype=np.uint8).reshape(2, 3, 2)
    out = ContentAttr(x, t3, ContentSetup(t3).broadcast(1, 6)).fold(be)
    assert out.type == TType([2, 6, 2], U8)
    assert np.array_equal(out.values(np.uint8).reshape(2, 6, 2), np.concatenate([x, x], axis=1))


def subview_sub_byte(be):
    """lit dialect/const/passes/constant_folding.mlir:56-314 (I1Subview*, I4Subview*): SubView on 1- and 4-bit
    storage gathers bit fields, low bits first (subview.cpp:20-160)."""
    I1, I4 = abi.VF_DT_I1, abi.VF_DT_I4

    def bits(vals):  # 1-bit values -> packed bytes, element 0 in bit 0
        return np.packbits(np.asarray(vals, np.uint8), bitorder="little")

    def run(raw, shape, dt, off, shp, convert=None, splat=False):
        t = TType(shape, dt)
        s = ContentSetup(t).subview(off, shp)
        if convert is not None:
            s = s.convertElemType(convert)
        out = ContentAttr(np.asarray(raw, np.uint8), t, s, is_splat=splat, storage_dtype=dt).fold(be)
        return out

    def unbits(out, n):
        return np.unpackbits(out.bytes(), bitorder="little")[:n].tolist()

    o = run([0xFF], [1, 32, 3, 3], I1, [0, 16, 0, 0], [1, 16, 3, 3], splat=True)               # :56-67 splat stays true
    assert o.is_splat and set(unbits(o, 144)) == {1}
    assert unbits(run(bits([1, 0, 0, 1, 1, 1, 0, 1, 1, 0]), [10], I1, [3], [4]), 4) == [1, 1, 1, 0]   # :72-85
    assert unbits(run(bits([1, 0, 1, 0]), [1, 4], I1, [0, 2], [1, 2]), 2) == [1, 0]                     # :90-102
    d3 = [0, 0, 1, 1, 0, 1, 1, 1, 1, 0, 0, 1, 1, 1, 0, 1, 0, 0, 0, 1, 0, 1, 1, 1, 0, 1, 0, 1, 1, 0, 1, 0]
    assert unbits(run(bits(d3), [1, 4, 8], I1, [0, 2, 4], [1, 2, 4]), 8) == [0, 1, 1, 1, 1, 0, 1, 0]  # :107-122
    d4 = [0] * 8 + [1] * 8 + [0, 1] * 4 + [1, 0] * 4
    assert unbits(run(bits(d4), [1, 32, 1, 1], I1, [0, 16, 0, 0], [1, 16, 1, 1]), 16) == [0, 1] * 4 + [1, 0] * 4  # :127-145
    d5 = [0, 1, 1, 0, 1, 1, 0, 0, 1, 0, 1, 0, 1, 1, 1, 0, 0, 0, 1, 1, 0, 1, 0, 1]
    assert unbits(run(bits(d5), [1, 2, 3, 4, 1], I1, [0, 1, 1, 1, 0], [1, 1, 2, 3, 1]), 6) == [0, 1, 1, 1, 0, 1]  # :150-163
    I8 = abi.VF_DT_I8
    assert run([0x22, 0x22], [4], I4, [2], [2], I8).values(np.int8).tolist() == [2, 2]                 # :168-188 blob 2222
    assert run([0x21, 0x43], [4], I4, [2], [2], I8).values(np.int8).tolist() == [3, 4]                 # :192-212
    b8 = [0x10, 0x32, 0x54, 0x76]
    assert run(b8, [2, 4], I4, [1, 2], [1, 2], I8).values(np.int8).tolist() == [6, 7]                  # :216-237
    assert run(b8, [2, 4, 1], I4, [1, 2, 0], [1, 2, 1], I8).values(np.int8).tolist() == [6, 7]         # :241-262
    b16 = b8 + [0x67, 0x45, 0x23, 0x01]
    assert run(b16, [2, 4, 2, 1], I4, [1, 2, 1, 0], [1, 2, 1, 1], I8).values(np.int8).tolist() == [2, 0]        # :266-287
    assert run(b16, [2, 4, 2, 1, 1], I4, [1, 2, 1, 0, 0], [1, 2, 1, 1, 1], I8).values(np.int8).tolist() == [2, 0]  # :291-312


def broadcast_non_splat(be):
    """lit dialect/const/passes/constant_folding.mlir:316-417 (broadcastNonSplat*): the block from the broadcast
    dim inwards is repeated."""
    def run(vals, dt, setup_fn):
        vals = np.asarray(vals)
        t = TType(list(vals.shape), dt)
        return ContentAttr(vals, t, setup_fn(ContentSetup(t))).fold(be)

    i8 = lambda v: np.asarray(v, np.int8)
    o = run(i8([1, 2, 3]), I8, lambda s: s.reshape([1, 3, 1, 1]).broadcast(0, 3).reshape([1, 9, 1, 1]))          # :316-326
    assert o.values(np.int8).tolist() == [1, 2, 3] * 3
    o = run(i8([1, 2, 3]), I8, lambda s: s.reshape([1, 3, 1, 1]).broadcast(2, 3).reshape([1, 9, 1, 1]))          # :330-340
    assert o.values(np.int8).tolist() == [1, 1, 1, 2, 2, 2, 3, 3, 3]
    o = run(i8([1, 2, 3, 4, 5, 6]), I8, lambda s: s.reshape([1, 3, 1, 2]).broadcast(2, 2))                       # :344-356
    assert o.type.shape == [1, 3, 2, 2] and o.values(np.int8).tolist() == [1, 2, 1, 2, 3, 4, 3, 4, 5, 6, 5, 6]
    o = run(i8(range(1, 13)), I8, lambda s: s.reshape([1, 3, 2, 2]).broadcast(2, 4))                             # :360-371
    assert o.values(np.int8).tolist() == [1, 2, 3, 4, 1, 2, 3, 4, 5, 6, 7, 8, 5, 6, 7, 8, 9, 10, 11, 12, 9, 10, 11, 12]
    h = np.asarray([[[[1, 2, 3, 4]]]], np.float16)
    o = run(h, F16, lambda s: s.castElemType(F16).reshape([1, 1, 1, 4]).broadcast(1, 4).broadcast(2, 4))         # :375-392
    assert o.type.shape == [1, 4, 4, 4] and o.values(np.float16).tolist() == [1.0, 2.0, 3.0, 4.0] * 16
    h = np.asarray([[[[1], [2], [3], [4]]]], np.float16)
    o = run(h, F16, lambda s: s.castElemType(F16).reshape([1, 1, 4, 1]).broadcast(1, 4).broadcast(3, 4))         # :396-413
    assert o.values(np.float16).tolist() == [v for _ in range(4) for v in (1.0, 2.0, 3.0, 4.0) for _ in range(4)]


def const_fold_i4(be):
    """lit dialect/const/passes/constant_folding.mlir:416-428 ConstFoldI4: f16 [1,0,1,2] cast to a quantized si4 type and
    reordered folds to the packed bytes [1, 33] (element 0 in the low nibble)."""
    t = TType([1, 4, 1, 1], F16)
    q = Elem.uniform(abi.VF_DT_I4, F16, 0.0039215686274509803, 0, -8, 7)
    s = ContentSetup(t).castElemType(abi.VF_DT_I4).castElemType(q).reorder(0x3412)
    out = ContentAttr(np.array([1, 0, 1, 2], np.float16).reshape(1, 4, 1, 1), t, s).fold(be)
    assert out.type.shape == [1, 4, 1, 1] and out.type.order == 0x3412
    assert out.bytes().tolist() == [1, 33]


def dequantize_per_axis_splat(be):
    """lit dialect/const/passes/constant_folding.mlir:466-563 ConstFoldDequantizeAxis0..4: a splat 1.0 cast to a per-axis
    u8 type dequantizes to (1 - zp[c]) * scale[c] along the quantized axis."""
    sc = [1.0, 0.5, 0.25, 0.125, 0.1, 0.2, 0.4, 0.8]
    zp = [128, 64, 32, 16, 128, 128, 128, 128]
    want = [-127.0, -31.5, -7.75, -1.875, -12.7031, -25.4063, -50.8125, -101.625]   # as printed at :539
    for shape, axis in (([1, 2, 4, 8], 0), ([1, 2, 4, 8], 1), ([1, 2, 4, 8], 2), ([1, 2, 4, 8], 3), ([2, 2, 2, 2, 2], 4)):
        n = shape[axis]
        t = TType(shape, F16)
        q = Elem.per_axis(U8, F16, sc[:n], zp[:n], axis, 0, 255)
        s = ContentSetup(t).castElemType(U8).castElemType(q).dequantize()
        out = ContentAttr(np.array([1.0], np.float16), t, s, is_splat=True).fold(be)
        assert out.type == TType(shape, F16)
        got = out.values(np.float16).reshape(shape).astype(np.float64)
        idx = np.arange(n).reshape([n if d == axis else 1 for d in range(len(shape))])
        exp = np.broadcast_to(np.asarray(want[:n])[idx], shape)
        assert np.abs(got - exp).max() <= 1e-4 * 128, (axis, got.ravel()[:8])           # 6 printed digits
        exact = np.asarray([np.float16(np.float32((1 - z) * s_)) for s_, z in zip(sc[:n], zp[:n])], np.float64)
        assert (got == np.broadcast_to(exact[idx], shape)).all()


def fold_with_swizzling(be):
    """lit dialect/const/passes/constant_folding.mlir:849-910 ConstFoldWithSwizzling*: SwizzleConstant works on the
    content its predecessors produced (not the raw storage), 1-bit constants keep their type, and the result has
    the aligned size whatever the shape before it."""
    arch = abi.VF_ARCH_NPU37XX
    t = TType([100, 1, 1, 384], abi.VF_DT_I1)                                           # :849-851
    out = ContentAttr(np.array([0xFF], np.uint8), t, ContentSetup(t).swizzleConstant(5, arch), is_splat=True,
                      storage_dtype=abi.VF_DT_I1).fold(be)
    assert out.type == TType([40960, 1, 1, 1], abi.VF_DT_I1) and out.written == 5120
    assert (out.bytes()[:4800] == 0xFF).all()                                           # dense<true> of the check line
    t = TType([32, 1, 1, 1], F16)                                                       # :881-897
    q = Elem.uniform(U8, F16, 1.0, 0, 0, 254)
    s = (ContentSetup(t).castElemType(U8).castElemType(q).reorder(0x1342).reorder(0x1234).reshape([32, 1, 1, 1])
         .padWithZero([0, 0, 0, 0], [0, 15, 0, 0]).reorder(0x1342).subview([0, 0, 0, 0], [16, 16, 1, 1])
         .swizzleConstant(5, arch))
    out = ContentAttr(np.array([1.0], np.float16), t, s, is_splat=True).fold(be)
    assert out.type.shape == [512, 1, 1, 1] and out.written == 512
    assert out.bytes()[:16].tolist() == [1] + [0] * 15                                  # prefix of the check line
    b = out.bytes()
    assert int(b.sum()) == 16 and sorted(set(np.flatnonzero(b) % 16)) == [0]
    t = TType([1, 1, 3, 1], U8)                                                         # :902-908
    s = ContentSetup(t).reshape([3, 1, 1, 1]).broadcast(0, 768).swizzleConstant(5, arch)
    out = ContentAttr(np.array([1, 2, 3], np.uint8).reshape(1, 1, 3, 1), t, s).fold(be)
    assert out.type == TType([1024, 1, 1, 1], U8) and out.written == 1024      # content shape != the op's 768
    b = out.bytes()
    assert b[:16].tolist() == ([1, 2, 3] * 6)[:16] and np.bincount(b, minlength=4).tolist() == [256, 256, 256, 256]


def sparsity_ptr_stepping(be):
    """lit dialect/VPU/passes/recompute_sparsity_ptrs.mlir:12-31: a 16x16x4x4 filter has sparsity-map rows of
    align(256, 128) / 8 = 32 bytes (map type 16x1x1x256xi1), so the sparsity pointers step by 32"""
    t = TType([16, 16, 4, 4], F16)
    attr = ContentAttr(np.zeros(16 * 16 * 16, np.float16), t, ContentSetup(t).reorder(abi.ORDER_NHWC).getSparsityMap())
    mt = attr.infer(be)[0]
    assert mt == TType([16, 1, 1, 256], abi.VF_DT_I1)
    row_bytes = mt.shape[3] // 8
    d, keep = _wt_desc(Elem(F16), Elem(F16), Elem(F16), 16, 0, 16, 0, row_bytes)
    tab = be.weights_table(d, 16).reshape(16, 4)
    assert tab[:, 1].tolist() == [32 * i for i in range(16)]


FOLD_CASES = [quantize, per_axis_quantize, dequantize_quantize, quant_cast, dequantize, reorder, pad, pad_splat,
              pad_uniform_quant, pad_per_axis_quant, bit_pack, bit_pack_quant, get_sparsity_map,
              get_sparsity_map_quantized, sparsify, sparsify_true, sparsify_quantized, position_requirement,
              convert_elem_type_i8_u8, convert_elem_type_u4_i4, quantize_splat, const_fold_chain, copy_to_i4,
              copy_to_i1, convert_elem_type_sub_byte, swizzle_constant, relocate_weights_table, reverse, expand_dilated,
              scalar_mult_inverse, change_shape_and_elem_type, broadcast, subview_sub_byte, broadcast_non_splat,
              const_fold_i4, dequantize_per_axis_splat, fold_with_swizzling]
TABLE_CASES = [weights_table_fixed_point, weights_table_float_scale, sparsity_ptr_stepping]
