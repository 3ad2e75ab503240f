"""The five weight-fold workloads as shape lists plus their transformation pipelines.

Only weight *shapes* of the named public architectures are used; values are synthetic
(`vf_synth_fill`: integer-hash bell curve, one IEEE multiply, round-to-nearest-even). Every tensor
is identified by (seed, tensor_id), so any slab can be regenerated on the host for checking.
"""
import math
from dataclasses import dataclass, field

import numpy as np

from . import abi

SEEDS = {"c1": 0xC0FFEE01, "c2": 0xC0FFEE02, "c3": 0xC0FFEE03, "c4": 0xC0FFEE04, "c5": 0xC0FFEE05}

# activation types used for the weights tables of the convolution workloads (the workload definition leaves
# them open): u8 input of scale 2^-6 and u8 output of scale 2^-4, zero point 128
ACT_IN = dict(scale=2.0 ** -6, zp=128)
ACT_OUT = dict(scale=2.0 ** -4, zp=128)


@dataclass
class TensorSpec:
    name: str
    shape: tuple
    dtype: int
    sigma: float
    tensor_id: int
    outlier_mult: float = 0.0
    outlier_log2: int = 0
    mask_zero: int = 0
    dense_row_mod: int = 0
    extra: dict = field(default_factory=dict)

    @property
    def numel(self):
        return int(np.prod(self.shape, dtype=np.int64))

    @property
    def nbytes(self):
        return self.numel * abi.DTYPE_BITS[self.dtype] // 8

    @property
    def rows(self):
        return int(self.shape[0])

    @property
    def row_len(self):
        return self.numel // self.rows

    def synth_spec(self, seed, first_elem=0):
        s = abi.SynthSpec()
        s.seed, s.tensor_id, s.dtype = seed, self.tensor_id, self.dtype
        s.sigma = self.sigma
        s.outlier_mult, s.outlier_log2 = self.outlier_mult, self.outlier_log2
        s.mask_zero, s.dense_row_mod = self.mask_zero, self.dense_row_mod
        s.row_len = self.row_len
        s.first_elem = first_elem
        return s


def c1_tensors():
    """One 3x3 convolution weight, O=60 I=64, fp32, ~N(0, 0.05)."""
    return [TensorSpec("conv", (60, 64, 3, 3), abi.VF_DT_F32, 0.05, 0)]


def resnet50_shapes():
    """ResNet-50 v1.5 convolution weights (OIYX) followed by the FC weight as [1000, 2048, 1, 1]."""
    shapes = [("stem", (64, 3, 7, 7))]
    in_ch = 64
    for si, (blocks, width) in enumerate(zip((3, 4, 6, 3), (64, 128, 256, 512))):
        for b in range(blocks):
            p = f"layer{si + 1}.{b}"
            shapes.append((p + ".conv1", (width, in_ch, 1, 1)))
            shapes.append((p + ".conv2", (width, width, 3, 3)))
            shapes.append((p + ".conv3", (width * 4, width, 1, 1)))
            if b == 0:
                shapes.append((p + ".downsample", (width * 4, in_ch, 1, 1)))
            in_ch = width * 4
    shapes.append(("fc", (1000, 2048, 1, 1)))
    return shapes


def resnet50_tensors(sparse=False):
    """fp16 Kaiming-normal weights (sigma = sqrt(2 / fan_in)); `sparse` applies the Bernoulli(1/2) zero mask
    with one output channel in ten left dense."""
    out = []
    for i, (name, shp) in enumerate(resnet50_shapes()):
        fan_in = shp[1] * shp[2] * shp[3]
        out.append(TensorSpec(name, shp, abi.VF_DT_F16, math.sqrt(2.0 / fan_in), i, mask_zero=1 if sparse else 0,
                              dense_row_mod=10 if sparse else 0))
    return out


def llama2_7b_tensors(layers=32, hidden=4096, ffn=11008, vocab=32000):
    """fp16 ~N(0, 0.02) with one element in 1024 multiplied by 20."""
    out = []
    tid = 0

    def add(name, shape):
        nonlocal tid
        out.append(TensorSpec(name, shape, abi.VF_DT_F16, 0.02, tid, outlier_mult=20.0, outlier_log2=10))
        tid += 1

    for l in range(layers):
        for n in ("q", "k", "v", "o"):
            add(f"l{l}.{n}", (hidden, hidden))
        add(f"l{l}.gate", (ffn, hidden))
        add(f"l{l}.up", (ffn, hidden))
        add(f"l{l}.down", (hidden, ffn))
    add("lm_head", (vocab, hidden))
    return out


def llama3_70b_tensors(layers=80, hidden=8192, kv=1024, ffn=28672, vocab=128256):
    """bf16 ~N(0, 0.02)."""
    out = []
    tid = 0

    def add(name, shape):
        nonlocal tid
        out.append(TensorSpec(name, shape, abi.VF_DT_BF16, 0.02, tid))
        tid += 1

    for l in range(layers):
        add(f"l{l}.q", (hidden, hidden))
        add(f"l{l}.k", (kv, hidden))
        add(f"l{l}.v", (kv, hidden))
        add(f"l{l}.o", (hidden, hidden))
        add(f"l{l}.gate", (ffn, hidden))
        add(f"l{l}.up", (ffn, hidden))
        add(f"l{l}.down", (hidden, ffn))
    add("embed", (vocab, hidden))
    add("lm_head", (vocab, hidden))
    return out


# ---- quantization specs --------------------------------------------------------------------------------
def spec_u8_asym():
    s = abi.QuantSpec()
    s.storage_dtype, s.range_mode, s.qmin, s.qmax, s.group_size = abi.VF_DT_U8, abi.VF_RANGE_MINMAX, 0, 255, 0
    s.expressed = abi.VF_DT_F32
    return s


def spec_i8_sym(expressed=abi.VF_DT_F16):
    s = abi.QuantSpec()
    s.storage_dtype, s.range_mode, s.qmin, s.qmax, s.group_size = abi.VF_DT_I8, abi.VF_RANGE_ABSMAX, -127, 127, 0
    s.expressed = expressed
    return s


def spec_u4_group(group=128):
    s = abi.QuantSpec()
    s.storage_dtype, s.range_mode, s.qmin, s.qmax, s.group_size = abi.VF_DT_U8, abi.VF_RANGE_MINMAX, 0, 15, group
    s.expressed = abi.VF_DT_F16
    return s


def t_reorder(order=abi.ORDER_NHWC):
    t = abi.Transform()
    t.kind, t.order = abi.VF_T_REORDER, order
    return t


def t_pad(before, after):
    t = abi.Transform()
    t.kind, t.rank = abi.VF_T_PAD_WITH_ZERO, len(before)
    for i, (b, a) in enumerate(zip(before, after)):
        t.a[i], t.b[i] = b, a
    return t


def t_bitpack(width=4):
    t = abi.Transform()
    t.kind, t.width = abi.VF_T_BIT_PACK, width
    return t


def conv_pipeline(shape, pad_oc_to=None, pad_ic_to=None):
    """[Reorder<NHWC>, PadWithZero] for an OIYX convolution weight; returns (transform list, output shape)."""
    o, i, kh, kw = shape
    ts = [t_reorder()]
    po = (pad_oc_to - o) if pad_oc_to else 0
    pi = (pad_ic_to - i) if pad_ic_to else 0
    if po or pi:
        ts.append(t_pad([0, 0, 0, 0], [po, pi, 0, 0]))
    return ts, (o + po, i + pi, kh, kw)


def weights_table_desc(oc, w_scales, ptr_step, bias=None, sparse_counts=None, sparsity_step=0):
    """Descriptor for a convolution with ACT_IN / ACT_OUT activations and per-channel i8 weights."""
    in_e = abi.Elem.uniform(abi.VF_DT_U8, abi.VF_DT_F16, ACT_IN["scale"], ACT_IN["zp"], 0, 255)
    out_e = abi.Elem.uniform(abi.VF_DT_U8, abi.VF_DT_F16, ACT_OUT["scale"], ACT_OUT["zp"], 0, 255)
    w_e = abi.Elem.per_axis(abi.VF_DT_I8, abi.VF_DT_F16, w_scales, np.zeros(oc, np.int64), 0, -127, 127)
    d = abi.WeightsTableDesc()
    d.in_elem, d.out_elem, d.weights_elem = in_e.pod(), out_e.pod(), w_e.pod()
    d.oc = oc
    d.weights_ptr_base, d.weights_ptr_step = 0, ptr_step
    if sparse_counts is not None:
        d.nnz_counts = sparse_counts.ctypes.data
        d.nnz_mem_kind = abi.VF_MEM_HOST
        d.sparsity_ptr_base, d.sparsity_ptr_step = 0, sparsity_step
    else:
        d.sparsity_ptr_base, d.sparsity_ptr_step = abi.VF_SPARSITY_PTR_WHEN_NO_SPARSITY, 0
    keep = [in_e, out_e, w_e, sparse_counts]
    if bias is not None:
        b = np.ascontiguousarray(bias, np.float32)
        d.has_bias, d.bias, d.bias_mem_kind = 1, b.ctypes.data, abi.VF_MEM_HOST
        keep.append(b)
    return d, keep


def bias_for(seed, tensor_id, oc):
    """fp32 bias ~N(0, 0.01) for the weights tables, from the same generator (tensor ids offset by 1000)."""
    s = abi.SynthSpec()
    s.seed, s.tensor_id, s.dtype, s.sigma, s.row_len = seed, 1000 + tensor_id, abi.VF_DT_F32, 0.01, oc
    return s
