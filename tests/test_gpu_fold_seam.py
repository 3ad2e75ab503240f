"""The reference's own call shape on the single-pass kernels: Const::ContentAttr::fold() receives a list whose
Quantize attribute CARRIES its scales and zero points (attributes/quantize.cpp:108-212, built by
IE/transforms/passes/split_fake_quant.cpp). vf_fold / vf_fold_batch recognise the lists upstream passes attach to
weights and run them as one launch; every result is compared with the CPU oracle's fold of the same list and with
the library's own one-kernel-per-transformation path (VF_OPT_DISABLE_FUSION)."""
import numpy as np
import pytest

from vpux_plugin_b200 import abi, workloads as wl
from vpux_plugin_b200.abi import Elem, TType
from vpux_plugin_b200.const import ContentAttr, ContentSetup, foldConstants

pytestmark = pytest.mark.gpu

F32, F16, BF16, I8, U8 = abi.VF_DT_F32, abi.VF_DT_F16, abi.VF_DT_BF16, abi.VF_DT_I8, abi.VF_DT_U8


def bf16_bits(x):
    import torch
    return torch.from_numpy(np.ascontiguousarray(x, np.float32)).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)


def cast(x, dt):
    return x.astype(np.float32) if dt == F32 else (x.astype(np.float16) if dt == F16 else bf16_bits(x))


@pytest.fixture(scope="module")
def unfused():
    from vpux_plugin_b200.lib import Library
    return Library(device=0, disable_fusion=True)


def derived(oracle, t, x, spec):
    c, keep = abi.make_content(t, x)
    s, z, _, _ = oracle.row_stats(c, spec, t.shape[0])
    return s, z


def three_way(attr, gpu, unfused, oracle, launches=1):
    ref = attr.fold(oracle)
    got = attr.fold(gpu)
    assert gpu.last_stats.fused == 1 and gpu.last_stats.kernels_launched == launches, (gpu.last_stats.fused, gpu.last_stats.kernels_launched)
    gen = attr.fold(unfused)
    assert unfused.last_stats.fused == 0
    assert got.type == ref.type == gen.type and got.written == ref.written == gen.written
    assert np.array_equal(got.bytes(), ref.bytes()), f"{int((got.bytes() != ref.bytes()).sum())} bytes differ from the oracle"
    assert np.array_equal(gen.bytes(), ref.bytes())
    return got


@pytest.mark.parametrize("dt", [F32, F16, BF16])
@pytest.mark.parametrize("shape,pad_oc,pad_ic", [((60, 64, 3, 3), 64, None), ((64, 3, 7, 7), None, 16), ((16, 8, 1, 1), None, None),
                                                 ((12, 512, 3, 3), None, None), ((24, 256, 1, 1), None, None), ((7, 32, 3, 3), 8, 48)])
@pytest.mark.parametrize("how", ["derived", "tight", "random"])
def test_conv_lists(gpu, unfused, oracle, dt, shape, pad_oc, pad_ic, how):
    """[Quantize<per-axis(0)>, Reorder<NHWC>, PadWithZero]: parameters as the data's own ranges give them,
    parameters whose range covers a third of the data (most elements clamp), and arbitrary ones."""
    rng = np.random.default_rng(21)
    x = cast(rng.standard_normal(shape) * 0.05, dt)
    t = TType(list(shape), dt)
    oc = shape[0]
    for spec in (wl.spec_i8_sym(), wl.spec_u8_asym()):
        s, z = derived(oracle, t, x, spec)
        if how == "tight":
            s = s / 3.0
        elif how == "random":
            s = rng.uniform(1e-4, 1e-2, oc)
            z = rng.integers(spec.qmin, spec.qmax + 1, oc)
        q = Elem.per_axis(spec.storage_dtype, F16, s, z, 0, spec.qmin, spec.qmax)
        setup = ContentSetup(t).quantize(q).reorder(abi.ORDER_NHWC)
        if pad_oc or pad_ic:
            setup = setup.padWithZero([0, 0, 0, 0], [(pad_oc or oc) - oc, (pad_ic or shape[1]) - shape[1], 0, 0])
        three_way(ContentAttr(x, t, setup), gpu, unfused, oracle)
        three_way(ContentAttr(x, t, ContentSetup(t).quantize(q)), gpu, unfused, oracle)


@pytest.mark.parametrize("dt", [F16, BF16])
@pytest.mark.parametrize("rows,cols", [(5, 8192), (3, 28672), (2, 1024), (9, 11008)])
@pytest.mark.parametrize("expressed", [F16, F32, BF16])
def test_row_lists_codes_and_dequantized_copy(gpu, unfused, oracle, dt, rows, cols, expressed):
    """[Quantize<per-axis(0)>] and [Quantize, CastElemType<q>, Dequantize] (config 5's two lists)."""
    rng = np.random.default_rng(22)
    x = rng.standard_normal((rows, cols)) * 0.02
    x[1] = 0
    x[0] *= 1e-3  # tiny scale: the dequantized values reach the fp16 subnormal range
    if rows > 4:
        x[4] *= 2.0e5  # fp16 overflow: the copy clamps to +-65504
    x = cast(x, dt)
    t = TType([rows, cols], dt)
    spec = wl.spec_i8_sym(expressed)
    s, z = derived(oracle, t, x, spec)
    for k, (scales, zps) in enumerate([(s, z), (s / 2.5, z + 3), (rng.uniform(1e-4, 1e-2, rows), rng.integers(-100, 100, rows))]):
        q = Elem.per_axis(I8, expressed, scales, zps, 0, -127, 127)
        three_way(ContentAttr(x, t, ContentSetup(t).quantize(q)), gpu, unfused, oracle)
        three_way(ContentAttr(x, t, ContentSetup(t).quantize(q).castElemType(q).dequantize()), gpu, unfused, oracle)
    # a CastElemType to a DIFFERENT quantized type is not the pattern: general path, same answer
    q = Elem.per_axis(I8, expressed, s, z, 0, -127, 127)
    q2 = Elem.per_axis(I8, expressed, s * 2, z, 0, -127, 127)
    attr = ContentAttr(x, t, ContentSetup(t).quantize(q).castElemType(q2).dequantize())
    got, ref = attr.fold(gpu), attr.fold(oracle)
    assert gpu.last_stats.fused == 0 and np.array_equal(got.bytes(), ref.bytes())


@pytest.mark.parametrize("dt", [F16, BF16])
def test_lists_on_exact_ties(gpu, unfused, oracle, dt):
    """Every element on a rounding boundary of the supplied parameters (scale 2^-7, values (2m+1) 2^-8)."""
    rng = np.random.default_rng(23)
    for rows, cols in ((4, 8192), (2, 28672), (3, 2048)):
        m = rng.integers(-60, 60, (rows, cols))
        x = cast((2 * m + 1) * 2.0 ** -8, dt)
        t = TType([rows, cols], dt)
        q = Elem.per_axis(I8, F16, np.full(rows, 2.0 ** -7), rng.integers(-5, 6, rows), 0, -127, 127)
        three_way(ContentAttr(x, t, ContentSetup(t).quantize(q)), gpu, unfused, oracle)
        three_way(ContentAttr(x, t, ContentSetup(t).quantize(q).castElemType(q).dequantize()), gpu, unfused, oracle)
    shape = (16, 64, 3, 3)
    m = rng.integers(-60, 60, shape)
    x = cast((2 * m + 1) * 2.0 ** -8, dt)
    t = TType(list(shape), dt)
    q = Elem.per_axis(I8, F16, np.full(16, 2.0 ** -7), np.zeros(16, np.int64), 0, -127, 127)
    three_way(ContentAttr(x, t, ContentSetup(t).quantize(q).reorder(abi.ORDER_NHWC)), gpu, unfused, oracle)


@pytest.mark.parametrize("group", [32, 64, 128])
@pytest.mark.parametrize("dt", [F16, BF16])
def test_group_list_with_bitpack(gpu, unfused, oracle, group, dt):
    """Config 4 as a list: the tensor reshaped to [units, group], Quantize<u8 0:15> per unit, BitPack<4>."""
    rng = np.random.default_rng(24)
    rows, cols = 6, 1024
    x = rng.standard_normal((rows, cols)) * 0.02
    x[rng.random((rows, cols)) < 0.002] *= 20
    x = cast(x, dt)
    t = TType([rows, cols], dt)
    units = rows * cols // group
    tu = TType([units, group], dt)
    for how in ("derived", "random"):
        if how == "derived":
            s, z = derived(oracle, tu, x, wl.spec_u4_group(0))
        else:
            s, z = rng.uniform(1e-3, 1e-2, units), rng.integers(0, 16, units)
        q = Elem.per_axis(U8, F16, s, z, 0, 0, 15)
        three_way(ContentAttr(x, t, ContentSetup(t).reshape([units, group]).quantize(q).bitPack(4)), gpu, unfused, oracle)
    # signed codes: BitPack reads getValues<uint8_t>(), so a negative code fails the checked cast (bit_pack.cpp:146-151)
    qs = Elem.per_axis(I8, F16, rng.uniform(1e-3, 1e-2, units), rng.integers(-8, 8, units), 0, -8, 7)
    attr = ContentAttr(x, t, ContentSetup(t).reshape([units, group]).quantize(qs).bitPack(4))
    for be in (gpu, oracle):
        with pytest.raises(Exception) as e:
            attr.fold(be)
        assert e.value.status == abi.VF_ERR_CHECKED_CAST


def test_lists_the_kernels_do_not_cover_take_the_general_path(gpu, oracle):
    rng = np.random.default_rng(25)
    x = (rng.standard_normal((4, 2048)) * 0.02).astype(np.float16)
    t = TType([4, 2048], F16)
    cases = [
        Elem.per_axis(I8, F16, np.full(4, 0.001), np.zeros(4, np.int64), 0, -120, 120),   # fakeQuantize's tail is not the identity
        Elem.per_axis(I8, F16, np.full(2048, 0.001), np.zeros(2048, np.int64), 1, -127, 127),  # another axis
        Elem.uniform(I8, F16, 0.001, 0, -127, 127),                                      # per tensor
    ]
    for q in cases:
        attr = ContentAttr(x, t, ContentSetup(t).quantize(q))
        got, ref = attr.fold(gpu), attr.fold(oracle)
        assert gpu.last_stats.fused == 0
        assert np.array_equal(got.bytes(), ref.bytes())


def test_a_scale_no_quantized_type_can_carry_is_refused(gpu, oracle):
    """mlir::quant::UniformQuantizedPerAxisType::verify refuses scale <= 0: such an attribute cannot exist."""
    x = np.zeros((4, 2048), np.float16)
    t = TType([4, 2048], F16)
    q = Elem.per_axis(I8, F16, np.array([0.001, -0.001, 0.001, 0.001]), np.zeros(4, np.int64), 0, -127, 127)
    for be in (gpu, oracle):
        with pytest.raises(Exception) as e:
            ContentAttr(x, t, ContentSetup(t).quantize(q)).fold(be)
        assert e.value.status == abi.VF_ERR_INVALID_ARG


def test_fold_batch_shares_launches_and_reads_a_constant_once(gpu, oracle):
    """ConstantFoldingPass over config-5-like constants: the codes and the dequantized copy of every tensor are two
    const.Declare ops over the same base; the batch runs each tensor as one entry of one launch."""
    rng = np.random.default_rng(26)
    attrs = []
    for rows, cols in ((6, 8192), (4, 8192), (3, 4096)):
        x = bf16_bits(rng.standard_normal((rows, cols)) * 0.02)
        t = TType([rows, cols], BF16)
        s, z = derived(oracle, t, x, wl.spec_i8_sym(F16))
        q = Elem.per_axis(I8, F16, s, z, 0, -127, 127)
        attrs.append(ContentAttr(x, t, ContentSetup(t).quantize(q)))
        attrs.append(ContentAttr(x, t, ContentSetup(t).quantize(q).castElemType(q).dequantize()))
    # conv weights with their lists and an unrelated constant on the general path
    for shape in ((32, 64, 3, 3), (64, 32, 1, 1)):
        x = (rng.standard_normal(shape) * 0.05).astype(np.float16)
        t = TType(list(shape), F16)
        s, z = derived(oracle, t, x, wl.spec_i8_sym())
        q = Elem.per_axis(I8, F16, s, z, 0, -127, 127)
        attrs.append(ContentAttr(x, t, ContentSetup(t).quantize(q).reorder(abi.ORDER_NHWC)))
    tb = TType([1, 64, 1, 1], F32)
    attrs.append(ContentAttr(rng.standard_normal(tb.shape).astype(np.float32), tb, ContentSetup(tb).castElemType(F16)))
    before = gpu.launch_count
    folded, stats, groups = foldConstants(gpu, attrs)
    launched = gpu.launch_count - before
    # one row launch for the three merged tensors, one convolution launch, one conversion of the bias
    assert launched == 3, launched
    for a, f in zip(attrs, folded):
        ref = a.fold(oracle)
        assert f.type == ref.type and f.written == ref.written
        assert np.array_equal(f.bytes(), ref.bytes())


def test_device_resident_fold_of_a_list(gpu, oracle):
    """Base and destination in device memory: the kernel writes the destination directly."""
    import torch
    rng = np.random.default_rng(27)
    rows, cols = 12, 8192
    x = bf16_bits(rng.standard_normal((rows, cols)) * 0.02)
    t = TType([rows, cols], BF16)
    s, z = derived(oracle, t, x, wl.spec_i8_sym(F16))
    q = Elem.per_axis(I8, F16, s, z, 0, -127, 127)
    src = torch.from_numpy(x.view(np.int16)).cuda()
    c, keep = abi.make_content(t, None, ptr=src.data_ptr(), nbytes=x.nbytes, mem_kind=abi.VF_MEM_DEVICE)
    for setup, nbytes in ((ContentSetup(t).quantize(q), rows * cols), (ContentSetup(t).quantize(q).castElemType(q).dequantize(), rows * cols * 2)):
        tr, n = setup.transforms()
        dst = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
        torch.cuda.synchronize()  # the fill runs on torch's stream, the library on its own
        w, _ = gpu.fold(c, tr, n, dst.data_ptr(), nbytes, dst_mem_kind=abi.VF_MEM_DEVICE)
        assert gpu.last_stats.fused == 1 and gpu.last_stats.kernels_launched == 1
        ref = ContentAttr(x, t, setup).fold(oracle)
        assert w == ref.written and np.array_equal(dst.cpu().numpy(), ref.bytes())
