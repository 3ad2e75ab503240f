"""Regenerates tests/golden/oracle_golden.json from the CPU oracle.

The fixture freezes (a) the first values of the synthetic weight generator for every workload's first tensor
and (b) SHA-256 digests of the oracle's folded outputs for workload C1 and a small slice of C4 / C5, so that an
accidental change of the generator or of the oracle arithmetic is caught without a GPU.
Run from the repository root:  python tests/golden/make_golden.py
"""
import hashlib
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import Oracle  # noqa: E402
from vpux_plugin_b200 import abi, workloads as wl  # noqa: E402


def fold(cpu, spec, x, qspec, transforms, out_bytes, units, dequant_dt=None):
    t = abi.TType(list(spec.shape), spec.dtype)
    c, keep = abi.make_content(t, x)
    dst = np.zeros(out_bytes, np.uint8)
    scales, zps = np.zeros(units, np.float64), np.zeros(units, np.int64)
    outs = abi.QuantOutputs()
    outs.mem_kind, outs.scales, outs.zps = abi.VF_MEM_HOST, scales.ctypes.data, zps.ctypes.data
    dq = None
    if dequant_dt is not None:
        dq = np.zeros(spec.numel * abi.DTYPE_BITS[dequant_dt] // 8, np.uint8)
        outs.dequant, outs.dequant_dtype, outs.dequant_bytes = dq.ctypes.data, dequant_dt, dq.nbytes
    w = cpu.quantize_fold(c, qspec, abi.make_transforms(transforms), len(transforms), dst, out_bytes, outs)
    h = hashlib.sha256()
    h.update(dst[:w].tobytes())
    h.update(scales.tobytes())
    h.update(zps.tobytes())
    if dq is not None:
        h.update(dq.tobytes())
    return h.hexdigest()


def build():
    cpu = Oracle(nthreads=4)
    out = {"synth": {}, "folds": {}}
    firsts = {"c1": wl.c1_tensors()[0], "c2": wl.resnet50_tensors()[0], "c3": wl.resnet50_tensors(sparse=True)[1],
              "c4": wl.llama2_7b_tensors(layers=1)[0], "c5": wl.llama3_70b_tensors(layers=1)[0]}
    for key, spec in firsts.items():
        v = cpu.synth_fill(spec.synth_spec(wl.SEEDS[key]), 16)
        out["synth"][key] = [int(b) for b in v.view(np.uint8)]
    spec = wl.c1_tensors()[0]
    x = cpu.synth_fill(spec.synth_spec(wl.SEEDS["c1"]), spec.numel)
    ts, oshape = wl.conv_pipeline(spec.shape, pad_oc_to=64)
    out["folds"]["c1"] = fold(cpu, spec, x, wl.spec_u8_asym(), ts, int(np.prod(oshape)), 60)
    spec = wl.TensorSpec("l0.q[:64]", (64, 4096), abi.VF_DT_F16, 0.02, 0, outlier_mult=20.0, outlier_log2=10)
    x = cpu.synth_fill(spec.synth_spec(wl.SEEDS["c4"]), spec.numel)
    out["folds"]["c4_slice"] = fold(cpu, spec, x, wl.spec_u4_group(128), [wl.t_bitpack()], spec.numel // 2, spec.numel // 128)
    spec = wl.TensorSpec("l0.q[:16]", (16, 8192), abi.VF_DT_BF16, 0.02, 0)
    x = cpu.synth_fill(spec.synth_spec(wl.SEEDS["c5"]), spec.numel)
    out["folds"]["c5_slice"] = fold(cpu, spec, x, wl.spec_i8_sym(), [], spec.numel, 16, dequant_dt=abi.VF_DT_F16)
    return out


if __name__ == "__main__":
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "oracle_golden.json")
    with open(path, "w") as f:
        json.dump(build(), f, indent=1)
    print("wrote", path)
