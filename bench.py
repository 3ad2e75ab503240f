#!/usr/bin/env python
"""Weight-fold benchmark: input GB/s of the Const fold hot path on B200.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c4|c5slab|c2|c3|c1|next] [--impl reference]

One step = one pass of the fold over the whole workload (every tensor of this rank's shard). The default
workload is the Llama-2-7B-shaped set (fp16 -> per-group-128 asymmetric u4, bit-packed, fp16 scales and packed
u4 zero points; 13.2 GB of input), the largest configuration that fits one GPU; with N > 1 the tensors are
sharded across ranks (longest-processing-time-first, no collective). Prints ONE JSON line on rank 0.

`value`  : device-resident throughput (inputs already in HBM), CUDA events on the launching stream,
           max over ranks.
`e2e`    : same metric through the C ABI with pinned HOST buffers; H2D and D2H inside the timed region; with the
           rate plain copies of the same buffers reach (`copy_ceiling`).
`roofline`: algorithmic bytes of the launches in the timed region / their device time, against the measured
           HBM copy peak.
`cpu_baseline`: the CPU oracle (a port of the reference's fold code) on a bounded sample (>= 1 GB), host threads.
`configs`: the other configurations, one block each (not the headline): c1, c2, c3 (whole step and the sparsify
           stage) on rank 0, and the Llama-3-70B-shaped set by output-channel slabs on every rank — the whole set
           at 4 and 8 GPUs (two slabs / one slab per GPU), one slab per GPU at 1 and 2 GPUs. Each with its
           roofline fraction and a 128-bit digest of its outputs (k_hash128).
`fold_seam`: the reference's own call shape — vf_fold_batch over lists whose Quantize attribute carries the
           parameters — for the 70B slab and the ResNet-50 set.
`--impl reference`: times the CPU port alone, on all host threads, each step the same bounded sample.
`--workload next`: not a headline line — the kernels of the rows around the hot path (SwizzleConstant, sub-byte
           unpack, Reverse, Broadcast, ExpandDilated, ScalarMultInverse, 8-bit float conversion, RelocateWeightsTable,
           the content hash), one at a time, each with its own GB/s, share of the HBM peak and CPU-oracle figure.
"""
import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from vpux_plugin_b200 import abi, workloads as wl  # noqa: E402

FALLBACK_HBM_GBS = 6650.0  # HBM copy rate used only when no measured-peaks file accompanies the benchmark


_RESULT_FD = None


def claim_stdout():
    """Keeps the process's stdout for the one JSON line: file descriptor 1 is pointed at stderr for everything
    else (NCCL prints its version banner on stdout whatever NCCL_DEBUG_FILE says)."""
    global _RESULT_FD
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)


def emit(line):
    data = (json.dumps(line) + "\n").encode()
    sys.stdout.flush()
    if _RESULT_FD is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_RESULT_FD, data)


def parse():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=10)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--workload", default="c4")
    p.add_argument("--impl", default="b200")
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--sync-calls", action="store_true",
                   help="device-resident arm: every library call synchronises (default: pipelined calls, VF_OPT_ASYNC)")
    p.add_argument("--no-cpu", action="store_true")
    p.add_argument("--no-configs", action="store_true", help="default workload only: leave out the blocks of the other configurations")
    p.add_argument("--scale", type=float, default=1.0, help="fraction of the layer count (for profiling captures)")
    p.add_argument("--profile", action="store_true",
                   help="profiling capture mode: no end-to-end / CPU legs, warm-up count taken as given")
    return p.parse_args()


# ---------------------------------------------------------------------------------------------------------
# workload definitions
# ---------------------------------------------------------------------------------------------------------
class Workload:
    def __init__(self, key, scale):
        self.key = key
        if key == "c4":
            layers = max(1, int(round(32 * scale)))
            self.tensors = wl.llama2_7b_tensors(layers=layers)
            self.spec = wl.spec_u4_group(128)
            self.desc = ("c4: Llama-2-7B-shaped linear weights (%d layers + lm_head), fp16 N(0,0.02) with 1/1024 "
                         "outliers x20 -> per-group(128) asymmetric u4, bit-packed, fp16 scales + packed u4 zero "
                         "points" % layers)
            self.alg_bytes_per_elem = 2.0 + 0.5 + (2.0 + 0.5) / 128.0
            self.kernel = "k_group<half,128>"
            self.shard_mode = 0
        elif key == "c5slab":
            # one eighth (by output-channel slabs) of the Llama-3-70B-shaped set: what each GPU of an 8-GPU job holds
            layers = max(1, int(round(80 * scale)))
            self.tensors = wl.llama3_70b_tensors(layers=layers)
            self.spec = wl.spec_i8_sym(abi.VF_DT_F16)
            self.desc = ("c5slab: 1/8 output-channel slab of Llama-3-70B-shaped weights (%d layers + embed + lm_head), "
                         "bf16 N(0,0.02) -> per-channel symmetric i8 + dequantized fp16 copy" % layers)
            self.alg_bytes_per_elem = 2.0 + 1.0 + 2.0
            self.kernel = "k_row<bf16>"
            self.shard_mode = 1
        elif key in ("c1", "c2", "c3"):
            # convolution weights: small (<= 51 MB), so the L2 is flushed between timed steps
            self.tensors = wl.c1_tensors() if key == "c1" else wl.resnet50_tensors(sparse=key == "c3")
            self.spec = wl.spec_u8_asym() if key == "c1" else wl.spec_i8_sym()
            self.desc = {"c1": "c1: conv 60x64x3x3 fp32 -> per-channel asymmetric u8, OIYX->OYXI, O padded to 64",
                         "c2": "c2: ResNet-50 v1.5 weight set (53 convs + FC) fp16 -> per-channel symmetric i8, OIYX->OYXI, "
                               "stem IC 3->16",
                         "c3": "c3: ResNet-50 v1.5 weight set, Bernoulli(1/2) masked with 1 channel in 10 dense: c2 fold, then "
                               "Sparsify + GetSparsityMap + per-channel counts on the folded i8 codes"}[key]
            self.alg_bytes_per_elem = {"c1": 4.0 + 64.0 / 60.0, "c2": 3.0, "c3": 2.0 + 1.0 + 1.0 + 0.55 + 0.125}[key]
            self.kernel = {"c1": "k_conv (fp32 input)", "c2": "k_convv<half> + k_weights_table_batch",
                           "c3": "k_convv<half> + k_sparse_scan_batch + k_sparse_offsets_batch + k_sparse_compact_batch + table kernels"}[key]
            self.shard_mode = 0
            self.seed = wl.SEEDS[key]
            return
        else:
            raise SystemExit(f"unknown workload {key}")
        self.seed = wl.SEEDS["c4" if key == "c4" else "c5"]


def shard(workload, world, rank, slab_world=None):
    """[(TensorSpec, row_begin, row_end)] owned by `rank`."""
    from vpux_plugin_b200.lib import plan_shards
    ts = workload.tensors
    if workload.key == "c5slab":
        # fixed 8-way slabbing defines the per-GPU unit of work; rank r of an N-GPU job takes slab r
        rb, re = plan_shards(1, 8, [t.nbytes for t in ts], [t.rows for t in ts], 1)
        return [(t, int(rb[i, rank % 8]), int(re[i, rank % 8])) for i, t in enumerate(ts)]
    rb, re = plan_shards(0, world, [t.nbytes for t in ts], [t.rows for t in ts], 1)
    return [(t, int(rb[i, rank]), int(re[i, rank])) for i, t in enumerate(ts) if re[i, rank] > rb[i, rank]]


# ---------------------------------------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------------------------------------
class ClockSampler:
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    # NVML event-reason bits (nvml.h): sw_power_cap, hw_slowdown, sw_thermal_slowdown, hw_thermal_slowdown
    BITS = ((0x4, "sw_power_cap"), (0x8, "hw_slowdown"), (0x20, "sw_thermal_slowdown"), (0x40, "hw_thermal_slowdown"))

    def __init__(self, uuid):
        """Samples SM clock and throttle reasons of the GPU while the timed region runs: through NVML from a
        thread every 2 ms (read-only queries), else through an `nvidia-smi -lms` child."""
        self.thread = None
        try:
            import threading

            import pynvml
            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode() if hasattr(uuid, "encode") else uuid)
            self.samples, self.mask, self.stop_flag = [], 0, False
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))

            def poll():
                while not self.stop_flag:
                    try:
                        self.samples.append(float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)))
                        self.mask |= int(pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(h))
                    except pynvml.NVMLError:
                        pass
                    time.sleep(0.002)

            self.thread = threading.Thread(target=poll, daemon=True)
            self.thread.start()
            self.p = None
            return
        except Exception:  # no NVML binding or no such device: fall back to nvidia-smi
            self.thread = None
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        try:
            self.p = subprocess.Popen(["nvidia-smi", "-i", uuid, f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                       "-lms", "100"], stdout=self.f, stderr=subprocess.DEVNULL)
        except OSError:
            self.p = None

    def stop(self):
        if self.thread is not None:
            self.stop_flag = True
            self.thread.join(timeout=2)
            sm = self.samples
            return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": self.max_mhz, "samples": len(sm),
                    "reasons": sorted(name for bit, name in self.BITS if self.mask & bit), "source": "nvml"}
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.p.kill()
        self.f.flush()
        self.f.seek(0)
        sm, mx, reasons = [], [], set()
        for line in self.f:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.f.name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ---------------------------------------------------------------------------------------------------------
# the CPU arm (oracle port of the reference's fold code)
# ---------------------------------------------------------------------------------------------------------
CPU_THREADS_MODEL = ("port of the reference's fold code; every transformation is split over all host threads the way "
                     "loop_nd splits its first dimension, including the per-group Quantize and BitPack that the reference "
                     "runs on one thread (quantize.cpp:123-125, bit_pack.cpp:146-151): the figure favours the CPU")


def cpu_sample(workload, min_bytes=1 << 30):
    """The first tensors of the workload (this rank-0 shard order) up to `min_bytes` of input: for the Llama-2 shaped
    set three whole layers (1.2 GB), for the 70B slab five layers' slabs."""
    from vpux_plugin_b200.lib import plan_shards
    ts = workload.tensors
    if workload.key == "c5slab":
        rb, re = plan_shards(1, 8, [t.nbytes for t in ts], [t.rows for t in ts], 1)
        parts = [(t, int(rb[i, 0]), int(re[i, 0])) for i, t in enumerate(ts)]
    else:
        parts = [(t, 0, t.rows) for t in ts]
    out, total = [], 0
    for t, r0, r1 in parts:
        out.append((t, r0, r1))
        total += (r1 - r0) * t.row_len * abi.DTYPE_BITS[t.dtype] // 8
        if total >= min_bytes:
            break
    return out, total


def cpu_arm(workload, steps=1, warmup=0, min_bytes=1 << 30):
    """Times the oracle on a bounded sample of `workload`; returns (GB/s, cores, sample description, ms/step)."""
    from oracle import Oracle
    cores = os.cpu_count() or 1
    cpu = Oracle(nthreads=cores)
    parts, total = cpu_sample(workload, min_bytes)
    work = []
    for t, r0, r1 in parts:
        rows, cols = r1 - r0, t.row_len
        n = rows * cols
        spec = wl.TensorSpec(t.name, (rows, cols), t.dtype, t.sigma, t.tensor_id, t.outlier_mult, t.outlier_log2)
        x = cpu.synth_fill(spec.synth_spec(workload.seed, r0 * cols), n)
        c, keep = abi.make_content(abi.TType([rows, cols], t.dtype), x)
        outs = abi.QuantOutputs()
        outs.mem_kind = abi.VF_MEM_HOST
        if workload.key == "c4":
            units = n // 128
            side = [np.zeros(units, np.uint16), np.zeros((units + 1) // 2, np.uint8)]
            outs.scales_f16, outs.zps_u4_packed = side[0].ctypes.data, side[1].ctypes.data
            tr, ntr, ob = abi.make_transforms([wl.t_bitpack()]), 1, n // 2
        else:
            side = [np.zeros(n, np.uint16)]
            outs.dequant, outs.dequant_dtype, outs.dequant_bytes = side[0].ctypes.data, abi.VF_DT_F16, side[0].nbytes
            tr, ntr, ob = abi.make_transforms([]), 0, n
        work.append((c, keep, tr, ntr, np.zeros(ob, np.uint8), ob, outs, side))

    def run():
        t0 = time.perf_counter()
        for c, keep, tr, ntr, dst, ob, outs, side in work:
            cpu.quantize_fold(c, workload.spec, tr, ntr, dst, ob, outs)
        return time.perf_counter() - t0

    for _ in range(warmup):
        run()
    tot = sum(run() for _ in range(steps))
    names = f"{parts[0][0].name} .. {parts[-1][0].name}"
    sample = (f"{len(parts)} tensors ({names}; {total / 1e9:.2f} GB of "
              f"{'fp16' if parts[0][0].dtype == abi.VF_DT_F16 else 'bf16'} input) per step")
    return total * steps / tot / 1e9, cores, sample, tot / steps * 1e3


def reference_arm(args, workload):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    v, cores, sample, ms = cpu_arm(workload, steps=args.steps, warmup=args.warmup)
    line = {
        "impl": "reference", "metric": "weight_fold_input_throughput", "value": v, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload.desc},
        "cpu_baseline": {"value": v, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample,
                         "threads_model": CPU_THREADS_MODEL},
        "e2e": {"value": v, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "CPU port of the reference's fold code (the reference itself needs MLIR/OpenVINO and cannot be built here)",
    }
    emit(line)


# ---------------------------------------------------------------------------------------------------------
# helpers of the GPU arms
# ---------------------------------------------------------------------------------------------------------
def hbm_peak():
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        return float(json.load(open(peaks_path))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return FALLBACK_HBM_GBS, "fallback"


def profiled_traffic(name):
    """DRAM bytes per element of the dominant kernel from the committed ncu summary of a smaller case of the same
    kernel (dram__bytes_read.sum + dram__bytes_write.sum over the elements of the captured launch; traffic grows in
    proportion to the elements). The summary records which kernel source it was taken from: a summary older than
    the source gives no figure."""
    import hashlib
    import re
    path = os.path.join(ROOT, "profiles", name)
    src = os.path.join(ROOT, "vpux_plugin_b200", "csrc", "kernels_rowquant.cu")
    if not os.path.exists(path) or not os.path.exists(src):
        return None, "no summary"
    text = open(path).read()
    m = re.search(r"traffic_bytes_per_elem:\s*([0-9.]+)", text)
    h = re.search(r"kernel_source_sha16:\s*([0-9a-f]{16})", text)
    if not m or not h:
        return None, "summary without a traffic line"
    if hashlib.sha256(open(src, "rb").read()).hexdigest()[:16] != h.group(1):
        return None, "summary predates the kernel source"
    return float(m.group(1)), "profiles/" + name


def mix_digest(parts):
    """One 128-bit value for a list of per-buffer hashes (order matters)."""
    h0, h1 = 0x9E3779B97F4A7C15, 0xD6E8FEB86659FD93
    for i, (a, b) in enumerate(parts):
        h0 = ((h0 ^ a) * 0x100000001B3 + i) & 0xFFFFFFFFFFFFFFFF
        h1 = ((h1 + b) * 0xA0761D6478BD642F + i) & 0xFFFFFFFFFFFFFFFF
    return f"{h0:016x}{h1:016x}"


def device_digest(lib, buffers):
    """vf_content_hash (k_hash128) of every output buffer: drift of any output byte shows in the record."""
    from vpux_plugin_b200.lib import content_hash
    parts = []
    for t in buffers:
        n = int(t.numel() * t.element_size())
        c, k = abi.make_content(abi.TType([n], abi.VF_DT_U8), None, abi.VF_DT_U8, False, abi.VF_MEM_DEVICE, ptr=t.data_ptr(), nbytes=n)
        parts.append(content_hash(lib, c))
    return mix_digest(parts)


class QuantCase:
    """Device-resident quantize-fold of a list of (TensorSpec, row_begin, row_end): inputs generated on the device,
    outputs preallocated, one vf_quantize_fold_batch per step."""

    def __init__(self, lib, torch, dev, workload, mine):
        self.lib, self.torch, self.workload, self.mine = lib, torch, workload, mine
        self.is_c4 = workload.key == "c4"
        self.jobs = (abi.QuantJob * len(mine))()
        self.keep, self.srcs, self.outs, self.scales = [], [], [], []
        self.in_bytes = self.elems = 0
        self.tr = abi.make_transforms([wl.t_bitpack()] if self.is_c4 else [])
        self.ntr = 1 if self.is_c4 else 0
        for j, (t, r0, r1) in enumerate(mine):
            rows, cols = r1 - r0, t.row_len
            n = rows * cols
            es = abi.DTYPE_BITS[t.dtype] // 8
            src = torch.empty(n * es, dtype=torch.uint8, device=dev)
            lib.synth_fill_device(t.synth_spec(workload.seed, r0 * cols), src.data_ptr(), n)
            outs = abi.QuantOutputs()
            outs.mem_kind = abi.VF_MEM_DEVICE
            if self.is_c4:
                units = n // 128
                dst = torch.empty(n // 2, dtype=torch.uint8, device=dev)
                s16 = torch.empty(units, dtype=torch.int16, device=dev)
                z4 = torch.empty((units + 1) // 2, dtype=torch.uint8, device=dev)
                outs.scales_f16, outs.zps_u4_packed = s16.data_ptr(), z4.data_ptr()
                side = [s16, z4]
            else:
                dst = torch.empty(n, dtype=torch.uint8, device=dev)
                dq = torch.empty(n, dtype=torch.int16, device=dev)
                sc = torch.empty(rows, dtype=torch.float64, device=dev)
                outs.dequant, outs.dequant_dtype, outs.dequant_bytes = dq.data_ptr(), abi.VF_DT_F16, n * 2
                outs.scales = sc.data_ptr()
                side = [dq, sc]
                self.scales.append(sc)
            c, k = abi.make_content(abi.TType([rows, cols], t.dtype), None, ptr=src.data_ptr(), nbytes=n * es, mem_kind=abi.VF_MEM_DEVICE)
            jb = self.jobs[j]
            jb.base, jb.spec, jb.t, jb.n = c, workload.spec, self.tr, self.ntr
            jb.dst, jb.dst_bytes, jb.dst_mem_kind, jb.outs = dst.data_ptr(), dst.numel(), abi.VF_MEM_DEVICE, outs
            self.keep.append(k)
            self.srcs.append(src)
            self.outs.append([dst] + side)
            self.in_bytes += n * es
            self.elems += n

    def step(self):
        self.lib.quantize_fold_batch(self.jobs)

    def digest(self):
        return device_digest(self.lib, [b for o in self.outs for b in o])


def timed_steps(torch, dist, world, dev, stream, lib, fn, steps, warmup):
    """`steps` calls of fn between CUDA events on the library's stream, barrier and synchronisation on both sides,
    maximum over the ranks; milliseconds for all the steps."""
    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(warmup):
        fn()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        fn()
    e1.record(stream)
    torch.cuda.synchronize()
    lib.synchronize()  # raises if a kernel of the pipelined calls reported an error
    ms = e0.elapsed_time(e1)
    barrier()
    if world > 1:
        tms = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
        ms = float(tms.item())
    return ms


def copy_ceiling(torch, stream_pairs, host_in, dev_in, dev_out, host_out, steps):
    """The same pinned host buffers moved with plain cudaMemcpyAsync, uploads on one stream and downloads on another,
    no kernels: what the end-to-end figure could reach at most on this box. Returns seconds per step."""
    s_up, s_dn = stream_pairs

    def once():
        with torch.cuda.stream(s_up):
            for h, d in zip(host_in, dev_in):
                d.copy_(h, non_blocking=True)
        with torch.cuda.stream(s_dn):
            for d, h in zip(dev_out, host_out):
                h.copy_(d, non_blocking=True)

    once()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        once()
    torch.cuda.synchronize()
    return (time.perf_counter() - t0) / steps


def e2e_case(torch, dist, world, dev, lib, case, steps):
    """The case through vf_quantize_fold_batch with pinned host input and output buffers; returns the e2e dict."""
    mine, workload = case.mine, case.workload
    host_jobs = (abi.QuantJob * len(mine))()
    hk, h_in, h_out, d_out = [], [], [], []
    h2d = d2h = 0
    for j, (t, r0, r1) in enumerate(mine):
        rows, cols = r1 - r0, t.row_len
        n = rows * cols
        es = abi.DTYPE_BITS[t.dtype] // 8
        hin = torch.empty(n * es, dtype=torch.uint8, pin_memory=True)
        hin.copy_(case.srcs[j])
        outs = abi.QuantOutputs()
        outs.mem_kind = abi.VF_MEM_HOST_PINNED
        if case.is_c4:
            units = n // 128
            hdst = torch.empty(n // 2, dtype=torch.uint8, pin_memory=True)
            h16 = torch.empty(units, dtype=torch.int16, pin_memory=True)
            h4 = torch.empty((units + 1) // 2, dtype=torch.uint8, pin_memory=True)
            outs.scales_f16, outs.zps_u4_packed = h16.data_ptr(), h4.data_ptr()
            side = [h16, h4]
        else:
            hdst = torch.empty(n, dtype=torch.uint8, pin_memory=True)
            hdq = torch.empty(n, dtype=torch.int16, pin_memory=True)
            hsc = torch.empty(rows, dtype=torch.float64, pin_memory=True)
            outs.dequant, outs.dequant_dtype, outs.dequant_bytes = hdq.data_ptr(), abi.VF_DT_F16, n * 2
            outs.scales = hsc.data_ptr()
            side = [hdq, hsc]
        c, k = abi.make_content(abi.TType([rows, cols], t.dtype), None, ptr=hin.data_ptr(), nbytes=n * es, mem_kind=abi.VF_MEM_HOST_PINNED)
        jb = host_jobs[j]
        jb.base, jb.spec, jb.t, jb.n = c, workload.spec, case.tr, case.ntr
        jb.dst, jb.dst_bytes, jb.dst_mem_kind, jb.outs = hdst.data_ptr(), hdst.numel(), abi.VF_MEM_HOST_PINNED, outs
        hk += [k]
        h_in.append(hin)
        h_out += [hdst] + side
        d_out += case.outs[j]
        h2d += n * es
        d2h += sum(int(x.numel() * x.element_size()) for x in [hdst] + side)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    lib.quantize_fold_batch(host_jobs)  # warm-up
    barrier()
    t0 = time.perf_counter()  # host wall clock brackets fully synchronous calls (each returns after its last D2H)
    for _ in range(steps):
        lib.quantize_fold_batch(host_jobs)
    torch.cuda.synchronize()
    dt = (time.perf_counter() - t0) / steps
    barrier()
    ceil = copy_ceiling(torch, (torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)), h_in, case.srcs, d_out, h_out, max(1, min(steps, 3)))
    barrier()
    in_bytes = float(case.in_bytes)
    if world > 1:
        tt = torch.tensor([dt, ceil], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        dt, ceil = float(tt[0].item()), float(tt[1].item())
        tb = torch.tensor([float(h2d), float(d2h), in_bytes], device=dev, dtype=torch.float64)
        dist.all_reduce(tb)
        h2d, d2h, in_bytes = int(tb[0].item()), int(tb[1].item()), float(tb[2].item())
    return {"value": in_bytes / dt / 1e9, "unit": "GB/s", "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
            "steps": steps, "path": "vf_quantize_fold_batch with pinned host input and output buffers",
            "copy_ceiling": {"value": in_bytes / ceil / 1e9, "unit": "GB/s",
                             "what": "the same pinned buffers moved by plain cudaMemcpyAsync, uploads and downloads on two streams, no kernels"},
            "fraction_of_copy_ceiling": ceil / dt}


def seam_c5(torch, lib, case, steps, warmup, stream, peak):
    """The reference's own call shape for the per-channel workload: vf_fold_batch over two lists per tensor,
    [Quantize<per-axis(0), the attribute's scales>] and [Quantize, CastElemType<q>, Dequantize], the parameters being
    the ones the data-derived run produced. Same device buffers as the case."""
    from vpux_plugin_b200.const import ContentSetup
    from vpux_plugin_b200.abi import Elem, TType
    n_t = len(case.mine)
    jobs = (abi.FoldJob * (2 * n_t))()
    keep = []
    for j, (t, r0, r1) in enumerate(case.mine):
        rows, cols = r1 - r0, t.row_len
        tt = TType([rows, cols], t.dtype)
        scales = case.scales[j].cpu().numpy()
        q = Elem.per_axis(abi.VF_DT_I8, abi.VF_DT_F16, scales, np.zeros(rows, np.int64), 0, -127, 127)
        s0 = ContentSetup(tt).quantize(q)
        s1 = ContentSetup(tt).quantize(q).castElemType(q).dequantize()
        for k, (setup, out) in enumerate(((s0, case.outs[j][0]), (s1, case.outs[j][1]))):
            tr, n = setup.transforms()
            jb = jobs[2 * j + k]
            jb.base, jb.t, jb.n = case.jobs[j].base, tr, n
            jb.dst, jb.dst_bytes, jb.dst_mem_kind = out.data_ptr(), int(out.numel() * out.element_size()), abi.VF_MEM_DEVICE
            keep += [setup, tr]
    before = case.digest()
    l0 = lib.launch_count
    # the pass's size threshold bounds memory in flight; device-resident constants allocate nothing, so one group
    fn = lambda: lib.fold_batch(jobs, threshold_bytes=1 << 60)
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    launches = lib.launch_count - l0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    # steady state of a pipelined pass: the timed region starts when an untimed call's kernels end, so the host-side
    # preparation of every timed call (milliseconds for 1124 jobs) overlaps the kernels of the call before it
    fn()
    e0.record(stream)
    t0 = time.perf_counter()
    for _ in range(steps):
        fn()
    host_us = (time.perf_counter() - t0) / steps * 1e6
    e1.record(stream)
    torch.cuda.synchronize()
    lib.synchronize()
    ms = e0.elapsed_time(e1) / steps
    achieved = case.elems * 5.0 / (ms * 1e-3) / 1e9
    return {"workload": "c5slab through vf_fold_batch: per tensor [Quantize<per-axis, given scales>] and [Quantize, CastElemType<q>, Dequantize]",
            "jobs": 2 * n_t, "launches_per_call": launches // max(1, warmup), "fused": int(lib.last_stats.fused),
            "ms_per_step": ms, "host_us_per_step": host_us, "value": case.in_bytes / (ms * 1e-3) / 1e9, "unit": "GB/s",
            "roofline": {"bound": "hbm", "kernel": "k_row<bf16> (supplied parameters)", "achieved": achieved, "peak": peak, "frac": achieved / peak},
            "same_bytes_as_data_derived_run": case.digest() == before}
class ConvCase:
    """Workloads c1-c3 (convolution weight sets, 0.14-51 MB), device resident: quantize-fold of every tensor in one
    batch call, (c3) Sparsify + GetSparsityMap + counts of the folded codes in a second one, (c2, c3) the weights
    tables in a third. The set fits the L2, so every step is timed on its own with 256 MiB written in between."""

    def __init__(self, lib, torch, dev, key):
        self.lib, self.torch, self.key = lib, torch, key
        self.workload = workload = Workload(key, 1.0)
        specs = workload.tensors
        self.jobs = (abi.QuantJob * len(specs))()
        self.keep, self.folded, self.outputs = [], [], []
        self.in_bytes = self.elems = 0
        for j, s in enumerate(specs):
            if key == "c1":
                ts, oshape = wl.conv_pipeline(s.shape, pad_oc_to=64)
            else:
                ts, oshape = wl.conv_pipeline(s.shape, pad_ic_to=16 if s.name == "stem" else None)
            tr = abi.make_transforms(ts)
            src = torch.empty(s.nbytes, dtype=torch.uint8, device=dev)
            lib.synth_fill_device(s.synth_spec(workload.seed), src.data_ptr(), s.numel)
            dst = torch.empty(int(np.prod(oshape)), dtype=torch.uint8, device=dev)
            sc = torch.empty(s.shape[0], dtype=torch.float64, device=dev)
            o = abi.QuantOutputs()
            o.mem_kind, o.scales = abi.VF_MEM_DEVICE, sc.data_ptr()
            c, k = abi.make_content(abi.TType(list(s.shape), s.dtype), None, ptr=src.data_ptr(), nbytes=s.nbytes, mem_kind=abi.VF_MEM_DEVICE)
            jb = self.jobs[j]
            jb.base, jb.spec, jb.t, jb.n = c, workload.spec, tr, len(ts)
            jb.dst, jb.dst_bytes, jb.dst_mem_kind, jb.outs = dst.data_ptr(), dst.numel(), abi.VF_MEM_DEVICE, o
            self.keep += [tr, src, k, ts]
            self.folded.append((dst, oshape, sc))
            self.outputs += [dst, sc]
            self.in_bytes += s.nbytes
            self.elems += s.numel
        self.sjobs = None
        self.sparse = []
        if key == "c3":  # sparsify stage on the folded codes (zero point 0: plain i8 view)
            self.sjobs = (abi.SparsifyJob * len(self.folded))()
            for j, (dst, oshape, sc) in enumerate(self.folded):
                oc, work = oshape[0], oshape[1] * oshape[2] * oshape[3]
                row = (work + 127) // 128 * 16
                cap = oc * ((work + 15) // 16 * 16)
                c, k = abi.make_content(abi.TType(list(oshape), abi.VF_DT_I8, abi.ORDER_NHWC), None, ptr=dst.data_ptr(), nbytes=dst.numel(), mem_kind=abi.VF_MEM_DEVICE)
                data = torch.zeros(cap, dtype=torch.uint8, device=dev)
                mp = torch.empty(oc * row, dtype=torch.uint8, device=dev)
                cnt = torch.empty(oc, dtype=torch.int64, device=dev)
                self.sparse.append((c, k, data, mp, cnt, cap, oc * row))
                sj = self.sjobs[j]
                sj.content, sj.data, sj.data_bytes = c, data.data_ptr(), cap
                sj.map, sj.map_bytes, sj.counts = mp.data_ptr(), oc * row, cnt.data_ptr()
                self.outputs += [mp, cnt]
        self.tjobs = None
        if key in ("c2", "c3"):  # one weights table per tensor: scales from the fold's device output, fp32 bias
            self.tjobs = (abi.WeightsTableJob * len(specs))()
            for j, s in enumerate(specs):
                oc = s.shape[0]
                oshape = self.folded[j][1]
                bias = torch.empty(oc, dtype=torch.float32, device=dev)
                lib.synth_fill_device(wl.bias_for(workload.seed, s.tensor_id, oc), bias.data_ptr(), oc)
                d, k = wl.weights_table_desc(oc, np.ones(oc), oshape[1] * oshape[2] * oshape[3])
                d.has_bias, d.bias, d.bias_mem_kind = 1, bias.data_ptr(), abi.VF_MEM_DEVICE
                if key == "c3":  # sparse pointers: prefix sums of the aligned set sizes, bitmap rows
                    d.weights_ptr_step = 0
                    d.nnz_counts, d.nnz_mem_kind = self.sparse[j][4].data_ptr(), abi.VF_MEM_DEVICE
                    d.sparsity_ptr_base, d.sparsity_ptr_step = 0, self.sparse[j][6] // oc
                tab = torch.empty(oc * 4, dtype=torch.int32, device=dev)
                tj = self.tjobs[j]
                tj.desc, tj.table = d, tab.data_ptr()
                tj.weights_scales, tj.scales_mem_kind = self.jobs[j].outs.scales, abi.VF_MEM_DEVICE
                self.keep += [bias, k]
                self.outputs.append(tab)

    def step(self):
        self.lib.quantize_fold_batch(self.jobs)
        if self.sjobs is not None:
            self.lib.sparsify_batch(self.sjobs, out_mem_kind=abi.VF_MEM_DEVICE)
        if self.tjobs is not None:
            self.lib.weights_table_batch(self.tjobs, out_mem_kind=abi.VF_MEM_DEVICE)

    def timed(self, stream, flush, steps, warmup, fn=None):
        """(device ms per step, host microseconds per step the calls themselves took)"""
        torch, lib = self.torch, self.lib
        fn = fn or self.step
        for _ in range(warmup):
            fn()
        lib.synchronize()
        torch.cuda.synchronize()
        ms = host = 0.0
        for _ in range(steps):
            flush.fill_(1)  # evicts the previous step's inputs and outputs from the 126 MB L2
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            t0 = time.perf_counter()
            fn()
            host += time.perf_counter() - t0
            e1.record(stream)
            lib.synchronize()  # reports what the step's kernels flagged
            torch.cuda.synchronize()
            ms += e0.elapsed_time(e1)
        return ms / steps, host / steps * 1e6

    def digest(self):
        bufs = list(self.outputs)
        for c, k, data, mp, cnt, cap, mb in self.sparse:  # the compacted data up to its written size
            bufs.append(data)
        return device_digest(self.lib, bufs)

    def report(self, stream, flush, steps, warmup, peak):
        ms, host_us = self.timed(stream, flush, steps, warmup)
        w = self.workload
        achieved = self.elems * w.alg_bytes_per_elem / (ms * 1e-3) / 1e9
        out = {"workload": w.desc, "input_bytes": self.in_bytes, "ms_per_step": ms, "value": self.in_bytes / (ms * 1e-3) / 1e9, "unit": "GB/s",
               "host_us_per_step": host_us, "launches_per_step": None,
               "roofline": {"bound": "hbm", "kernel": w.kernel, "achieved": achieved, "peak": peak, "frac": achieved / peak,
                            "note": "whole step: every launch of the step and the gaps between them; L2 flushed before every step"}}
        l0 = self.lib.launch_count
        self.step()
        self.lib.synchronize()
        out["launches_per_step"] = int(self.lib.launch_count - l0)
        if self.sjobs is not None:  # the sparsify stage alone, on the folded i8 codes
            sms, _ = self.timed(stream, flush, steps, 1, fn=lambda: self.lib.sparsify_batch(self.sjobs, out_mem_kind=abi.VF_MEM_DEVICE))
            code_bytes = sum(int(d.numel()) for d, _, _ in self.folded)
            out["stage"] = {"name": "Sparsify + GetSparsityMap + counts on the folded i8 codes", "input_bytes": code_bytes, "ms_per_step": sms,
                            "value": code_bytes / (sms * 1e-3) / 1e9, "unit": "GB/s", "roofline_frac": code_bytes * 1.7 / (sms * 1e-3) / 1e9 / peak}
        out["digest"] = self.digest()
        return out


def seam_c2(torch, lib, case, stream, flush, steps, warmup, peak):
    """Config 2 through vf_fold_batch: per tensor the list [Quantize<per-axis(0), given>, Reorder<NHWC>(, PadWithZero)]."""
    from vpux_plugin_b200.const import ContentSetup
    from vpux_plugin_b200.abi import Elem, TType
    specs = case.workload.tensors
    jobs = (abi.FoldJob * len(specs))()
    keep = []
    before = device_digest(lib, [d for d, _, _ in case.folded])
    for j, s in enumerate(specs):
        dst, oshape, sc = case.folded[j]
        tt = TType(list(s.shape), s.dtype)
        q = Elem.per_axis(abi.VF_DT_I8, abi.VF_DT_F16, sc.cpu().numpy(), np.zeros(s.shape[0], np.int64), 0, -127, 127)
        setup = ContentSetup(tt).quantize(q).reorder(abi.ORDER_NHWC)
        if tuple(oshape) != (s.shape[0], s.shape[1], s.shape[2], s.shape[3]):
            setup = setup.padWithZero([0, 0, 0, 0], [oshape[0] - s.shape[0], oshape[1] - s.shape[1], 0, 0])
        tr, n = setup.transforms()
        jb = jobs[j]
        jb.base, jb.t, jb.n = case.jobs[j].base, tr, n
        jb.dst, jb.dst_bytes, jb.dst_mem_kind = dst.data_ptr(), dst.numel(), abi.VF_MEM_DEVICE
        keep += [setup, tr]
    ms, host_us = case.timed(stream, flush, steps, warmup, fn=lambda: lib.fold_batch(jobs, threshold_bytes=1 << 60))
    l0 = lib.launch_count
    lib.fold_batch(jobs, threshold_bytes=1 << 60)
    lib.synchronize()
    achieved = case.elems * 3.0 / (ms * 1e-3) / 1e9
    return {"workload": "c2 through vf_fold_batch: per tensor [Quantize<per-axis, given scales>, Reorder<NHWC>(, PadWithZero)]",
            "jobs": len(specs), "launches_per_call": int(lib.launch_count - l0), "fused": int(lib.last_stats.fused), "ms_per_step": ms,
            "host_us_per_step": host_us, "value": case.in_bytes / (ms * 1e-3) / 1e9, "unit": "GB/s",
            "roofline": {"bound": "hbm", "kernel": "k_convv / k_conv / k_row (supplied parameters)", "achieved": achieved, "peak": peak, "frac": achieved / peak},
            "same_bytes_as_data_derived_run": device_digest(lib, [d for d, _, _ in case.folded]) == before}


# ---------------------------------------------------------------------------------------------------------
# the GPU arm
# ---------------------------------------------------------------------------------------------------------
def c5_slabs_of(world, rank):
    """Output-channel slabs (of the fixed 8-way cut of every tensor) a rank folds: N = 8 and N = 4 cover the whole
    70B-shaped set (one and two slabs per GPU: 35 GB in + 53 GB out fit), N = 1 and 2 fold one slab per GPU."""
    if world >= 8:
        return [rank % 8], "strong"
    if world == 4:
        return [2 * rank, 2 * rank + 1], "strong"
    return [rank], "weak"


def gpu_arm(args, workload):
    import torch
    import torch.distributed as dist

    from vpux_plugin_b200.lib import Library, plan_shards

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    stream = torch.cuda.Stream(device=dev)  # the library launches on this stream; the timing events are recorded on it
    torch.cuda.set_stream(stream)
    # device-resident arm: the K steps are K batch calls enqueued back to back (VF_OPT_ASYNC), one
    # synchronisation at the end; the end-to-end arm below moves host memory and synchronises in every call
    lib = Library(device=local, stream=stream.cuda_stream, pipelined=not args.sync_calls)
    peak, peak_src = hbm_peak()
    warmup = args.warmup if args.profile else max(3, args.warmup)

    mine = shard(workload, world, rank)
    case = QuantCase(lib, torch, dev, workload, mine)
    uuid = "GPU-" + str(torch.cuda.get_device_properties(local).uuid).replace("GPU-", "")
    total_in = torch.tensor([float(case.in_bytes), float(case.elems)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(total_in)
    total_in_bytes, total_elems = float(total_in[0].item()), float(total_in[1].item())

    sampler = ClockSampler(uuid) if rank == 0 else None
    l0 = lib.launch_count
    ms = timed_steps(torch, dist, world, dev, stream, lib, case.step, args.steps, warmup)
    launches = (lib.launch_count - l0) // (args.steps + warmup)  # library kernels launched per step
    clocks = sampler.stop() if sampler else None
    value = total_in_bytes * args.steps / (ms * 1e-3) / 1e9
    digest = None if args.profile else case.digest()

    # ---- the reference's own call shape on the same buffers (per-channel workload) -------------------------
    seam = {}
    if workload.key == "c5slab" and world == 1 and not args.profile:
        seam["c5slab"] = seam_c5(torch, lib, case, min(args.steps, 5), 2, stream, peak)

    # ---- end to end: pinned host buffers in and out, copies inside the timed region ----------------------
    e2e = None
    if not args.no_e2e and not args.profile:
        e2e = e2e_case(torch, dist, world, dev, lib, case, min(args.steps, 5))

    # roofline of the dominant kernel: every launch in the timed region is that kernel; per-GPU figure
    alg_bytes = total_elems / world * workload.alg_bytes_per_elem * args.steps
    achieved = alg_bytes / (ms * 1e-3) / 1e9
    tpe, tsrc = profiled_traffic({"c4": "k_group_c4.md", "c5slab": "k_row_c5slab.md"}[workload.key])
    n_launch = max(1, launches)
    roofline = {"bound": "hbm", "kernel": workload.kernel, "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak, "peak_source": peak_src,
                "algorithmic_bytes_per_launch": total_elems / world * workload.alg_bytes_per_elem / n_launch,
                "avg_launch_us": ms * 1e3 / args.steps / n_launch,
                "traffic": (tpe * total_elems / world / n_launch) if tpe else None, "traffic_source": tsrc}
    input_desc = {"input_bytes": int(total_in_bytes), "tensors_rank0": len(mine)}
    del case
    torch.cuda.empty_cache()

    # ---- the other configurations (not the headline: one block each) ---------------------------------------
    configs = {}
    if workload.key == "c4" and not args.profile and not args.no_configs:
        steps_c = min(args.steps, 10)
        if rank == 0:
            flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
            for key in ("c1", "c2", "c3"):
                cc = ConvCase(lib, torch, dev, key)
                configs[key] = cc.report(stream, flush, steps_c, 3, peak)
                if key == "c2":
                    seam["c2"] = seam_c2(torch, lib, cc, stream, flush, steps_c, 3, peak)
                del cc
            del flush
            torch.cuda.empty_cache()
        if world > 1:
            # the other ranks sleep on the rendezvous store meanwhile: their preparation of the next block (host
            # work for 1124 jobs each) would share the host's cores with the calls timed above
            store = dist.distributed_c10d._get_default_store()
            if rank == 0:
                store.set("small_configs_done", "1")
            else:
                store.wait(["small_configs_done"])
        # the 70B-shaped set by output-channel slabs: every rank folds its slab(s)
        w5 = Workload("c5slab", args.scale)
        slabs, scaling = c5_slabs_of(world, rank)
        rb, re = plan_shards(1, 8, [t.nbytes for t in w5.tensors], [t.rows for t in w5.tensors], 1)
        mine5 = [(t, int(rb[i, sl]), int(re[i, sl])) for sl in slabs for i, t in enumerate(w5.tensors)]
        c5 = QuantCase(lib, torch, dev, w5, mine5)
        tot5 = torch.tensor([float(c5.in_bytes), float(c5.elems)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(tot5)
        ms5 = timed_steps(torch, dist, world, dev, stream, lib, c5.step, steps_c, 3) / steps_c
        per_gpu_elems = float(tot5[1].item()) / world
        ach5 = per_gpu_elems * 5.0 / (ms5 * 1e-3) / 1e9
        tpe5, tsrc5 = profiled_traffic("k_row_c5slab.md")
        blk = {"workload": w5.desc + (" — %d slab(s) per GPU, %d GPU(s)" % (len(slabs), world)), "scaling": scaling,
               "input_bytes": int(tot5[0].item()), "ms_per_step": ms5, "value": float(tot5[0].item()) / (ms5 * 1e-3) / 1e9, "unit": "GB/s",
               "roofline": {"bound": "hbm", "kernel": w5.kernel, "achieved": ach5, "peak": peak, "frac": ach5 / peak,
                            "traffic": tpe5 * per_gpu_elems / 2 if tpe5 else None, "traffic_source": tsrc5,
                            "note": "two launches per step (rows up to 8192 elements, longer rows)"},
               "digest_rank0": c5.digest()}
        if world == 1:
            seam["c5slab"] = seam_c5(torch, lib, c5, min(steps_c, 5), 2, stream, peak)
            configs["c5slab"] = blk
        else:
            configs["c5"] = blk
        del c5
        torch.cuda.empty_cache()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    cpu = None
    if not args.no_cpu and not args.profile and world == 1:
        v, cores, sample, _ = cpu_arm(workload)
        cpu = {"value": v, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample, "threads_model": CPU_THREADS_MODEL}

    line = {
        "metric": "weight_fold_input_throughput", "value": value, "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
        "scaling": "weak" if workload.key == "c5slab" else "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": workload.desc, **input_desc,
                   "sharding": "whole tensors, longest-processing-time-first" if workload.shard_mode == 0 else
                   "output-channel slabs", "l2": "inputs (GBs) far larger than the 126 MB L2; no flush needed",
                   "calls": "synchronous" if args.sync_calls else "pipelined (VF_OPT_ASYNC): K batch calls enqueued back to back, "
                   "one synchronisation after the last"},
        "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "clocks": clocks, "gpu_launches": int(launches * args.steps),
        "digest": digest,
    }
    if configs:
        line["configs"] = configs
    if seam:
        line["fold_seam"] = seam
    emit(line)
    if world > 1:
        dist.destroy_process_group()


def conv_arm(args, workload):
    """--workload c1 | c2 | c3 as a line of its own (single GPU)."""
    import torch

    from vpux_plugin_b200.lib import Library

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    stream = torch.cuda.Stream(device=dev)
    torch.cuda.set_stream(stream)
    # the calls of a step are enqueued without a synchronisation in between (VF_OPT_ASYNC); every step ends with one
    lib = Library(device=0, stream=stream.cuda_stream, pipelined=not args.sync_calls)
    peak, peak_src = hbm_peak()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    warmup = args.warmup if args.profile else max(3, args.warmup)
    uuid = "GPU-" + str(torch.cuda.get_device_properties(0).uuid).replace("GPU-", "")
    case = ConvCase(lib, torch, dev, workload.key)
    sampler = ClockSampler(uuid)
    l0 = lib.launch_count
    rep = case.report(stream, flush, args.steps, warmup, peak)
    clocks = sampler.stop()
    line = {
        "metric": "weight_fold_input_throughput", "value": rep["value"], "unit": "GB/s",
        "n_gpus": 1, "steps": args.steps, "warmup": warmup, "ms_per_step": rep["ms_per_step"], "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload.desc, "input_bytes": case.in_bytes, "tensors_rank0": len(workload.tensors),
                   "l2": "256 MiB written between timed steps (inputs fit the 126 MB L2)",
                   "calls": "synchronous" if args.sync_calls else "pipelined (VF_OPT_ASYNC) within a step, one synchronisation per step"},
        "roofline": dict(rep["roofline"], unit="GB/s", peak_source=peak_src, traffic=None),
        "cpu_baseline": None, "e2e": None, "clocks": clocks, "gpu_launches": int(lib.launch_count - l0),
        "host_us_per_step": rep["host_us_per_step"], "digest": rep["digest"],
    }
    if "stage" in rep:
        line["stage"] = rep["stage"]
    if workload.key == "c2" and not args.profile:
        line["fold_seam"] = {"c2": seam_c2(torch, lib, case, stream, flush, args.steps, 3, peak)}
    emit(line)


def next_arm(args):
    """--workload next: the kernels behind the callers and data formats either side of the hot path (blob assembly,
    import-side unpacking, the remaining transformations, the content hash of the folding cache), one at a time on
    inputs larger than L2, each through vf_fold with device buffers. Per kernel: algorithmic bytes (input + output)
    over the CUDA-event time of the call, against the measured HBM copy peak, and the CPU oracle on a bounded
    sample of the same input beside it."""
    import torch

    from oracle import Oracle
    from vpux_plugin_b200.const import ContentSetup
    from vpux_plugin_b200.lib import Library, content_hash

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    stream = torch.cuda.Stream(device=dev)
    torch.cuda.set_stream(stream)
    lib = Library(device=0, stream=stream.cuda_stream, pipelined=True)
    orc = Oracle(nthreads=1)
    F32, F16, U8, I8, I32 = abi.VF_DT_F32, abi.VF_DT_F16, abi.VF_DT_U8, abi.VF_DT_I8, abi.VF_DT_I32
    TT = abi.TType
    mib = max(16, int(2048 * args.scale))
    n8 = mib << 20  # bytes of the 8-bit inputs
    oc = 4096
    ops = [  # name, reference site, base type, storage dtype, list builder
        ("SwizzleConstant", "swizzle_transform.cpp:163-215", TT([n8], U8), U8, lambda s: s.swizzleConstant(5, abi.VF_ARCH_NPU40XX)),
        ("subByteConversion u4->u8", "convert_utils.cpp:17-75", TT([oc, n8 // oc], abi.VF_DT_U4), abi.VF_DT_U4, lambda s: s.convertElemType(U8)),
        ("Reverse f16", "reverse.cpp:46-105", TT([oc, 4, n8 // oc // 8], F16), F16, lambda s: s.reverse(0)),
        ("Broadcast x4 u8", "broadcast.cpp:85-124", TT([oc, 1, n8 // oc // 4], U8), U8, lambda s: s.broadcast(1, 4)),
        ("ExpandDilated 3x3 d2 f16", "expand_dilated.cpp:88-131", TT([n8 // 2 // 25 // 64, 64, 3, 3], F16), F16, lambda s: s.expandDilated([2, 2])),
        ("ScalarMultInverse f32", "inverse.cpp:52-66", TT([n8 // 4], F32), F32, lambda s: s.scalarMultInverse()),
        ("CastElemType f32->f8e4m3 + copyTo", "content.hpp:66-71", TT([n8 // 4], F32), F32, lambda s: s.castElemType(abi.VF_DT_F8E4M3FN)),
        ("RelocateWeightsTable 1M rows", "relocate_weights_table.cpp:203-292", TT([1 << 20, 1, 1, 4], I32), I32,
         lambda s: s.relocateWeightsTablePointers([1 << 10, 1 << 20], 64, [0, 1 << 19], 16 << 20, 16)),
        # the general (unfused) kernels of the path itself, one transformation per call
        ("Quantize per-axis f32->i8", "quantize.cpp:108-212", TT([oc, n8 // oc // 4], F32), F32,
         lambda s: s.quantize(abi.Elem.per_axis(I8, F32, [0.01 + 1e-5 * i for i in range(oc)], [0] * oc, 0, -127, 127))),
        ("Dequantize per-axis i8->f32", "dequantize.cpp:42-108", TT([oc, n8 // oc // 4], I8), I8,
         lambda s: s.castElemType(abi.Elem.per_axis(I8, F32, [0.01 + 1e-5 * i for i in range(oc)], [0] * oc, 0, -127, 127)).dequantize()),
        ("Rescale f32", "rescale.cpp:67-82", TT([n8 // 4], F32), F32, lambda s: s.rescale(0.5)),
        ("Reorder OIYX->OYXI f16, 64 x 3 x 3 kernels", "reorder.cpp:79-99", TT([n8 // 2 // 64 // 9, 64, 3, 3], F16), F16, lambda s: s.reorder(abi.ORDER_NHWC)),
        ("Reorder OIYX->OYXI f16, rows of 4095", "reorder.cpp:79-99", TT([oc, 64, 3, n8 // 2 // oc // 64 // 3], F16), F16, lambda s: s.reorder(abi.ORDER_NHWC)),
        ("PadWithZero IC 48->64 f16", "pad_with_zero.cpp:111-268", TT([oc, 48, 3, n8 // 2 // oc // 48 // 3], F16), F16,
         lambda s: s.padWithZero([0, 0, 0, 0], [0, 16, 0, 0])),
        ("SubView half the channels f16", "subview.cpp:390-432", TT([oc, n8 // 2 // oc], F16), F16,
         lambda s: s.subview([s.base_type.shape[0] // 4, 0], [s.base_type.shape[0] // 2, s.base_type.shape[1]])),
        ("BitPack<4> u8", "bit_pack.cpp:132-154", TT([n8], U8), U8, lambda s: s.bitPack(4)),
    ]
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peak, peak_src = float(json.load(open(peaks_path))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    else:
        peak, peak_src = FALLBACK_HBM_GBS, "fallback"
    sampler = ClockSampler("GPU-" + str(torch.cuda.get_device_properties(0).uuid).replace("GPU-", ""))
    rows, samples = [], []
    total_bytes = total_ms = 0.0
    launches0 = lib.launch_count
    for name, site, t, storage, build in ops:
        setup = build(ContentSetup(t))
        tr, n = setup.transforms()
        numel = int(np.prod(t.shape))
        in_bytes = numel * abi.DTYPE_BITS[storage] // 8
        src = torch.empty(in_bytes, dtype=torch.uint8, device=dev)
        if storage == I32:  # a table whose pointer columns step by 16
            src.view(torch.int32).copy_(torch.arange(in_bytes // 4, device=dev, dtype=torch.int32) // 4 * 16 % (1 << 20))
        elif name.startswith("BitPack"):
            src.random_(0, 16)
        else:
            src.random_(1, 120)
        if storage == F32:  # finite, normal floats
            src.view(torch.float32).copy_(torch.rand(in_bytes // 4, device=dev) + 0.5)
        if storage == F16:
            src.view(torch.float16).copy_((torch.rand(in_bytes // 2, device=dev) - 0.5).half())
        c, keep = abi.make_content(t, None, storage, False, abi.VF_MEM_DEVICE, ptr=src.data_ptr(), nbytes=in_bytes)
        _, _, out_bytes = lib.infer_type(t, False, tr, n)
        dst = torch.empty(out_bytes, dtype=torch.uint8, device=dev)
        for _ in range(max(3, args.warmup)):
            lib.fold(c, tr, n, dst.data_ptr(), out_bytes, dst_mem_kind=abi.VF_MEM_DEVICE)
        lib.synchronize()
        torch.cuda.synchronize()
        # the calls are pipelined (VF_OPT_ASYNC): each returns once its work is enqueued, so the stream runs the
        # kernels of consecutive calls back to back and the per-call figure is device time, not launch latency
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.steps):
            lib.fold(c, tr, n, dst.data_ptr(), out_bytes, dst_mem_kind=abi.VF_MEM_DEVICE)
        e1.record(stream)
        lib.synchronize()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / args.steps
        # the CPU oracle runs on a bounded sample of the same input AFTER all GPU timings (an idle GPU between two
        # kernels would drop its clocks): keep the sample's type and bytes
        sample = None
        if not args.no_cpu:
            rows_all = t.shape[0]
            take = max(1, min(rows_all, int(rows_all * (8 << 20) / max(in_bytes, 1))))
            if name.startswith("Relocate"):
                take = rows_all  # the table is its own sample (the transformation's size is in its parameters)
            if "per-axis" in name:  # the parameters are per row: keep the rows, shorten them
                last = max(8, t.shape[-1] * take // rows_all // 8 * 8)
                ts = TT(list(t.shape[:-1]) + [last], t.elem.dtype, t.order)
                sb = in_bytes // t.shape[-1] * last
            else:
                ts = TT([take] + list(t.shape[1:]), t.elem.dtype, t.order) if take != rows_all else t
                sb = in_bytes * take // rows_all
            sample = (ts, src[:sb].cpu().numpy(), sb)
        alg = in_bytes + out_bytes
        if name.startswith("SubView"):
            alg = 2 * out_bytes  # only the viewed part of the input has to be read
        rows.append({"kernel": name, "reference": site, "input_bytes": in_bytes, "output_bytes": out_bytes, "ms": ms,
                     "achieved_gbs": alg / (ms * 1e-3) / 1e9, "frac": alg / (ms * 1e-3) / 1e9 / peak, "cpu_oracle_gbs": None})
        samples.append((build, storage, sample))
        total_bytes += alg
        total_ms += ms
        del src, dst
    # the content hash of the folding cache (vf_content_hash): one read of the buffer
    hb = n8
    src = torch.empty(hb, dtype=torch.uint8, device=dev).random_(0, 255)
    c, keep = abi.make_content(TT([hb], U8), None, U8, False, abi.VF_MEM_DEVICE, ptr=src.data_ptr(), nbytes=hb)
    for _ in range(3):
        content_hash(lib, c)
    ms = 0.0
    for _ in range(args.steps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        content_hash(lib, c)
        e1.record(stream)
        torch.cuda.synchronize()
        ms += e0.elapsed_time(e1)
    ms /= args.steps
    rows.append({"kernel": "content hash (k_hash128)", "reference": "constant_folding_cache.hpp:62-79 (hash of the attribute)",
                 "input_bytes": hb, "output_bytes": 16, "ms": ms, "achieved_gbs": hb / (ms * 1e-3) / 1e9,
                 "frac": hb / (ms * 1e-3) / 1e9 / peak, "cpu_oracle_gbs": None})
    total_bytes += hb
    total_ms += ms
    clocks = sampler.stop()
    for row, (build, storage, sample) in zip(rows, samples):
        if sample is None:
            continue
        ts, host, sb = sample
        hsetup = build(ContentSetup(ts))  # keeps the attribute's parameter arrays alive
        htr, hn = hsetup.transforms()
        hc, hkeep = abi.make_content(ts, host, storage, False)
        _, _, hob = orc.infer_type(ts, False, htr, hn)
        hdst = np.zeros(max(hob, 1), np.uint8)
        t0 = time.perf_counter()
        orc.fold(hc, htr, hn, hdst, hob)
        row["cpu_oracle_gbs"] = (sb + hob) / (time.perf_counter() - t0) / 1e9
    emit({"metric": "next_rows_throughput", "value": total_bytes / (total_ms * 1e-3) / 1e9, "unit": "GB/s", "n_gpus": 1,
          "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": total_ms, "higher_is_better": True,
          "scaling": "strong", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
          "config": {"workload": "next: one kernel at a time, %d MiB of 8-bit input each (larger than the 126 MB L2)" % mib},
          "roofline": {"bound": "hbm", "peak": peak, "peak_source": peak_src, "unit": "GB/s",
                       "achieved": total_bytes / (total_ms * 1e-3) / 1e9, "frac": total_bytes / (total_ms * 1e-3) / 1e9 / peak,
                       "traffic": None, "note": "input + output bytes of every call over its CUDA-event time; per kernel in `kernels`"},
          "kernels": rows, "cpu_baseline": None, "e2e": None, "clocks": clocks,
          "gpu_launches": int(lib.launch_count - launches0)})


def main():
    args = parse()
    claim_stdout()
    if args.workload == "next":
        next_arm(args)
        return
    workload = Workload(args.workload, args.scale)
    if args.impl == "reference":
        reference_arm(args, workload)
    elif args.workload in ("c1", "c2", "c3"):
        conv_arm(args, workload)
    else:
        gpu_arm(args, workload)


if __name__ == "__main__":
    main()
