#!/usr/bin/env python
"""Benchmark of the int8 convolution path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference] [--no-graph]

Default workload: the ShuffleNetV2-1.0x int8 backbone on 256 images of 3x320x320 per GPU (metric
shufflenetv2_int8_images_per_s); `--workload nanodet_plus_320` is the detector (2048 images per step, sharded over the GPUs);
the other names are single layers (metric int8_conv_tops). A step is one pass of the path (quantize -> int8 convolution ->
fused requantize/dequantize, layer after layer for the graphs) over seeded synthetic activations that are already resident
in HBM. The batch is larger than the 126 MB L2, so every step streams from HBM (no flush needed). Times are CUDA events
recorded on the stream the kernels are launched on; with several GPUs (one process per GPU, torchrun) each rank runs its
own shard on its own GPU (no collective on the data path) and the step time is the maximum over ranks.

Rank 0 prints one JSON line. value: whole-job throughput, device-resident (graph workloads replay a captured CUDA graph of
the forward); e2e: the same through the public call with pinned host buffers, copies included; roofline: the dominant
kernel (or layer kind) against the measured HBM / int8 tensor peak; cpu_baseline: the reference's CPU path on this box's
host cores; clocks: SM clock and throttle reasons sampled during the timed region; gpu_launches: kernels in the timed region.
`--impl reference` times the reference's own CPU implementation (oracle/_ref, or the C restatement
when the compiled reference is absent) on the host cores, on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
sys.path.insert(1, str(ROOT / "tests"))  # graph_walk (activation-scale calibration, output self-check) and the checker bindings

ACT_NONE, ACT_RELU, ACT_LRELU, ACT_RELU6 = 0, 1, 2, 3

# name -> geometry. Batch sizes and shapes are the ones the benchmark configurations name.
WORKLOADS = {
    # pointwise sweep (config 3): N=128, fp32 NCHW in, ReLU6, int8 out
    "pw_512_1024_hw56": dict(cin=512, cout=1024, k=1, stride=1, pad=0, groups=1, n=128, h=56, w=56, term=101, act=ACT_RELU6, in_f32=True),
    "pw_256_512_hw56": dict(cin=256, cout=512, k=1, stride=1, pad=0, groups=1, n=128, h=56, w=56, term=101, act=ACT_RELU6, in_f32=True),
    "pw_64_256_hw56": dict(cin=64, cout=256, k=1, stride=1, pad=0, groups=1, n=128, h=56, w=56, term=101, act=ACT_RELU6, in_f32=True),
    "pw_512_1024_hw28": dict(cin=512, cout=1024, k=1, stride=1, pad=0, groups=1, n=128, h=28, w=28, term=101, act=ACT_RELU6, in_f32=True),
    "pw_256_512_hw28": dict(cin=256, cout=512, k=1, stride=1, pad=0, groups=1, n=128, h=28, w=28, term=101, act=ACT_RELU6, in_f32=True),
    "pw_64_256_hw28": dict(cin=64, cout=256, k=1, stride=1, pad=0, groups=1, n=128, h=28, w=28, term=101, act=ACT_RELU6, in_f32=True),
    "pw_512_1024_hw14": dict(cin=512, cout=1024, k=1, stride=1, pad=0, groups=1, n=128, h=14, w=14, term=101, act=ACT_RELU6, in_f32=True),
    "pw_256_512_hw14": dict(cin=256, cout=512, k=1, stride=1, pad=0, groups=1, n=128, h=14, w=14, term=101, act=ACT_RELU6, in_f32=True),
    "pw_64_256_hw14": dict(cin=64, cout=256, k=1, stride=1, pad=0, groups=1, n=128, h=14, w=14, term=101, act=ACT_RELU6, in_f32=True),
    # the same layers fed by a requantizing producer (int8 NHWC in): the tensor-bound form
    "pw_512_1024_hw56_s8": dict(cin=512, cout=1024, k=1, stride=1, pad=0, groups=1, n=128, h=56, w=56, term=101, act=ACT_RELU6, in_f32=False),
    "pw_256_512_hw56_s8": dict(cin=256, cout=512, k=1, stride=1, pad=0, groups=1, n=128, h=56, w=56, term=101, act=ACT_RELU6, in_f32=False),
    "pw_64_256_hw56_s8": dict(cin=64, cout=256, k=1, stride=1, pad=0, groups=1, n=128, h=56, w=56, term=101, act=ACT_RELU6, in_f32=False),
    # ShuffleNetV2-1.0x stage-3 unit shapes at batch 256 (116 channels, 20x20): the layers the graph workload is made of
    "sn_pw1_116_hw20": dict(cin=116, cout=116, k=1, stride=1, pad=0, groups=1, n=256, h=20, w=20, term=102, act=ACT_RELU, in_f32=True),
    "sn_pw2_116_hw20": dict(cin=116, cout=116, k=1, stride=1, pad=0, groups=1, n=256, h=20, w=20, term=2, act=ACT_RELU, in_f32=False),
    "sn_dw_116_hw20": dict(cin=116, cout=116, k=3, stride=1, pad=1, groups=116, n=256, h=20, w=20, term=101, act=ACT_NONE, in_f32=False, w_std=0.1),
    "sn_pw1_58_hw40": dict(cin=58, cout=58, k=1, stride=1, pad=0, groups=1, n=256, h=40, w=40, term=102, act=ACT_RELU, in_f32=True),
    "sn_pw2_58_hw40": dict(cin=58, cout=58, k=1, stride=1, pad=0, groups=1, n=256, h=40, w=40, term=2, act=ACT_RELU, in_f32=False),
    "sn_dw_58_hw40": dict(cin=58, cout=58, k=3, stride=1, pad=1, groups=58, n=256, h=40, w=40, term=101, act=ACT_NONE, in_f32=False, w_std=0.1),
    # depthwise (config 2): N=64, C=256, 56x56, ReLU, int8 out
    "dw3x3s1_c256": dict(cin=256, cout=256, k=3, stride=1, pad=1, groups=256, n=64, h=56, w=56, term=101, act=ACT_RELU, in_f32=True, w_std=0.1),
    "dw3x3s2_c256": dict(cin=256, cout=256, k=3, stride=2, pad=1, groups=256, n=64, h=56, w=56, term=101, act=ACT_RELU, in_f32=True, w_std=0.1),
    "dw3x3s1_c256_s8": dict(cin=256, cout=256, k=3, stride=1, pad=1, groups=256, n=64, h=56, w=56, term=101, act=ACT_RELU, in_f32=False, w_std=0.1),
    "dw3x3s2_c256_s8": dict(cin=256, cout=256, k=3, stride=2, pad=1, groups=256, n=64, h=56, w=56, term=101, act=ACT_RELU, in_f32=False, w_std=0.1),
    # dense 3x3 (config 1 batched): fp32 in, fp32 out
    "dense3x3_64_hw56_n256": dict(cin=64, cout=64, k=3, stride=1, pad=1, groups=1, n=256, h=56, w=56, term=2, act=ACT_NONE, in_f32=True),
    "dense3x3_64_hw56_n256_s8": dict(cin=64, cout=64, k=3, stride=1, pad=1, groups=1, n=256, h=56, w=56, term=102, act=ACT_RELU, in_f32=False),
    # wider 3x3 layers (not in the benchmark configurations): where the tensor cores, not the per-tile overheads, set the pace
    "dense3x3_128_hw56_n128_s8": dict(cin=128, cout=128, k=3, stride=1, pad=1, groups=1, n=128, h=56, w=56, term=102, act=ACT_RELU, in_f32=False),
    "dense3x3_64_256_hw56_n128_s8": dict(cin=64, cout=256, k=3, stride=1, pad=1, groups=1, n=128, h=56, w=56, term=102, act=ACT_RELU, in_f32=False),
    "dense3x3_256_hw28_n128_s8": dict(cin=256, cout=256, k=3, stride=1, pad=1, groups=1, n=128, h=28, w=28, term=102, act=ACT_RELU, in_f32=False),
}
DEFAULT_WORKLOAD = "shufflenetv2_320"


def nhwc_channels(c):
    return (c + 15) & ~15


def make_layer_arrays(wl, seed=0x0771E5):
    """Seeded weights/scales with the distributions the configurations name (host numpy)."""
    rng = np.random.default_rng(seed)
    cin_g = wl["cin"] // wl["groups"]
    wf = rng.normal(0.0, wl.get("w_std", 0.05), size=(wl["cout"], cin_g, wl["k"], wl["k"])).astype(np.float32)
    amax = np.abs(wf).reshape(wl["cout"], -1).max(axis=1)
    w_scales = (np.float32(127.0) / amax).astype(np.float32)
    weight = np.clip(np.rint(wf * w_scales[:, None, None, None]), -127, 127).astype(np.int8)
    bias = rng.normal(0.0, 0.01, size=(wl["cout"],)).astype(np.float32)
    depthwise = wl["groups"] > 1
    in_scales = np.full((wl["groups"] if depthwise else 1,), 127.0, np.float32)  # activations are uniform[-1,1]
    # output scale: |y| rarely exceeds 4 sigma of the pre-activation
    sigma = wl.get("w_std", 0.05) * np.sqrt(cin_g * wl["k"] * wl["k"] / 3.0)
    top = min(4.0 * sigma, 6.0) if wl["act"] == ACT_RELU6 else 4.0 * sigma
    out_scales = np.full((wl["groups"] if depthwise else 1,), 127.0 / max(top, 1e-3), np.float32)
    return weight, bias, w_scales, in_scales, out_scales


def out_hw(wl):
    oh = (wl["h"] + 2 * wl["pad"] - (wl["k"] - 1) - 1) // wl["stride"] + 1
    ow = (wl["w"] + 2 * wl["pad"] - (wl["k"] - 1) - 1) // wl["stride"] + 1
    return oh, ow


def algorithmic_work(wl, n):
    """ops = 2*N*Cout*(Cin/groups)*k*k*OH*OW; bytes = input + weights + output at their boundary dtypes."""
    oh, ow = out_hw(wl)
    ops = 2.0 * n * wl["cout"] * (wl["cin"] // wl["groups"]) * wl["k"] * wl["k"] * oh * ow
    in_b = n * wl["cin"] * wl["h"] * wl["w"] * (4 if wl["in_f32"] else 1)
    out_b = n * wl["cout"] * oh * ow * (1 if wl["term"] > 100 else 4)
    w_b = wl["cout"] * (wl["cin"] // wl["groups"]) * wl["k"] * wl["k"]
    return ops, in_b + out_b + w_b


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured (MEASURED_PEAKS.json)"
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


def max_over_ranks(values, dist, device=None):
    """Element-wise maximum of a list of per-rank numbers over all ranks (the slowest rank sets the step time)."""
    if dist is None:
        return [float(v) for v in values]
    import torch
    if device is None:  # this rank's own GPU, whatever device the library made current last
        device = f"cuda:{os.environ.get('LOCAL_RANK', '0')}"
    t = torch.tensor([float(v) for v in values], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(v) for v in t.tolist()]


def whole_job_rate(units_per_rank, world, step_ms):
    """Weak scaling: every rank processes units_per_rank units per step; the job's rate uses the slowest rank's time."""
    return units_per_rank * world / (step_ms * 1e-3)


class ClockSampler:
    """nvidia-smi clock/throttle samples during the timed region."""

    Q = "index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, device):
        self.device, self.proc, self.lines = device, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(self.device)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.t.join(timeout=2)
        sm, mx, reasons = [], None, set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx = float(f[2])
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(sm)}


def int8_tensor_peak_tops():
    """Dense int8 tensor throughput of this GPU, measured live with the library GEMM (cuBLASLt through
    torch._int_mm, 8192^3, best of 10): the denominator for tensor-bound int8 kernels."""
    import torch
    n = 8192
    a = torch.randint(-127, 127, (n, n), dtype=torch.int8, device="cuda")
    b = torch.randint(-127, 127, (n, n), dtype=torch.int8, device="cuda").t().contiguous().t()
    for _ in range(3):
        torch._int_mm(a, b)
    torch.cuda.synchronize()
    best = 1e9
    for _ in range(10):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        torch._int_mm(a, b)
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1))
    del a, b
    torch.cuda.empty_cache()
    return 2.0 * n ** 3 / best / 1e9


# ----------------------------------------------------------------------------------------------------
# reference arm / CPU baseline


class _Desc(C.Structure):
    _fields_ = [(k, C.c_int) for k in ("cin", "cout", "kh", "kw", "sh", "sw", "ph", "pw", "dh", "dw", "groups", "bias_term",
                                       "int8_scale_term", "act_type")] + [("act_param0", C.c_float)]


def cpu_threads():
    """Host threads the CPU arm runs on: every core this process may use, whatever OMP_NUM_THREADS the launcher exported
    (torchrun sets it to 1 for its workers)."""
    return max(1, len(os.sched_getaffinity(0)))


def cpu_reference_time(wl, images, warmup=1, iters=None, packed=1, force_port=False):
    """Time the reference's CPU int8 ConvolutionLayer on `images` single-image forwards (its int8 path is
    batch-1), on cpu_threads() OpenMP threads (set explicitly). Returns (seconds per image, kind, cores)."""
    ref_so = ROOT / "oracle" / "_ref" / "libotter_ref.so"
    port_so = ROOT / "oracle" / "_build" / "libotter_oracle.so"
    weight, bias, w_scales, in_scales, out_scales = make_layer_arrays(wl)
    d = _Desc(wl["cin"], wl["cout"], wl["k"], wl["k"], wl["stride"], wl["stride"], wl["pad"], wl["pad"], 1, 1, wl["groups"], 1, wl["term"],
              wl["act"], 0.0)
    rng = np.random.default_rng(1)
    fp = lambda a, t: a.ctypes.data_as(C.POINTER(t))  # noqa: E731
    if wl["in_f32"]:
        x = rng.uniform(-1, 1, size=(1, wl["cin"], wl["h"], wl["w"])).astype(np.float32)
        xf, xs = fp(x, C.c_float), None
    else:
        x = rng.integers(-127, 128, size=(1, wl["cin"], wl["h"], wl["w"]), dtype=np.int8)
        xf, xs = None, fp(x, C.c_int8)
    if ref_so.exists() and not force_port:
        lib = C.CDLL(str(ref_so))
        lib.ref_conv_int8_time_ms.restype = C.c_double
        lib.ref_max_threads.restype = C.c_int
        lib.ref_set_threads.argtypes = [C.c_int]
        lib.ref_set_threads.restype = None
        lib.ref_set_threads(cpu_threads())
        cores = lib.ref_max_threads()
        mean = C.c_double()
        best = lib.ref_conv_int8_time_ms(C.byref(d), fp(weight, C.c_int8), fp(bias, C.c_float), fp(w_scales, C.c_float), fp(in_scales, C.c_float),
                                         in_scales.size, fp(out_scales, C.c_float), out_scales.size, xf, xs, wl["h"], wl["w"], packed, warmup, images,
                                         C.byref(mean))
        if best < 0:
            raise RuntimeError("reference forward failed")
        return mean.value / 1e3, "reference", cores
    if not port_so.exists():
        subprocess.run(["make", "-s", "-C", str(ROOT / "oracle"), "port"], check=True)
    lib = C.CDLL(str(port_so))
    lib.orc_max_threads.restype = C.c_int
    lib.orc_set_threads.argtypes = [C.c_int]
    lib.orc_set_threads.restype = None
    lib.orc_set_threads(cpu_threads())
    cores = lib.orc_max_threads()
    oh, ow = out_hw(wl)
    y8 = np.empty((1, wl["cout"], oh, ow), np.int8)
    yf = np.empty((1, wl["cout"], oh, ow), np.float32)
    t = []
    for i in range(warmup + images):
        t0 = time.perf_counter()
        lib.orc_conv_int8_forward(C.byref(d), fp(weight, C.c_int8), fp(bias, C.c_float), fp(w_scales, C.c_float), fp(in_scales, C.c_float),
                                  in_scales.size, fp(out_scales, C.c_float), out_scales.size, xf, xs, 1, wl["h"], wl["w"], 0, None, None,
                                  fp(yf, C.c_float) if wl["term"] < 100 else None, fp(y8, C.c_int8) if wl["term"] > 100 else None)
        if i >= warmup:
            t.append(time.perf_counter() - t0)
    return float(np.mean(t)), "port", cores


def cpu_sample_images(wl, budget_s=12.0):
    """How many single-image forwards fit a ~10-30 s CPU budget (estimated from one timed image)."""
    per_img, kind, cores = cpu_reference_time(wl, images=1, warmup=1)
    return max(2, min(256, int(budget_s / max(per_img, 1e-4)))), per_img


def run_reference_arm(args, wl):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    ops_img, _ = algorithmic_work(wl, 1)
    images, _ = cpu_sample_images(wl, budget_s=2.5)  # per step; K steps stay within a few minutes
    secs = []
    kind, cores = None, None
    for i in range(args.warmup + args.steps):
        per_img, kind, cores = cpu_reference_time(wl, images=images, warmup=0)
        if i >= args.warmup:
            secs.append(per_img * images)
    step_s = float(np.mean(secs))
    value = ops_img * images / step_s / 1e12
    sample = f"{images} single-image forwards per step of the layer (the reference int8 path is batch-1), OpenMP {cores} threads"
    print(json.dumps({
        "impl": "reference", "metric": "int8_conv_tops", "value": value, "unit": "TOP/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": step_s * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "s8xs8->s32", "data": "synthetic", "config": {"workload": args.workload, **{k: wl[k] for k in ("cin", "cout", "k", "stride", "groups", "h", "w")},
                                                              "images_per_step": images},
        "cpu_baseline": {"value": value, "unit": "TOP/s", "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "TOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ----------------------------------------------------------------------------------------------------
# GPU arm


def run_gpu_arm(args, wl):
    from tensor_b200 import F32_NCHW, S8_NHWC, ConvInt8, Context, library
    library()  # fails loudly when the CUDA library has not been built
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        if os.environ.get("NCCL_DEBUG", "").upper() in ("", "VERSION"):
            os.environ["NCCL_DEBUG"] = "WARN"  # NCCL's version banner goes to stdout and would precede the JSON line
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    n = wl["n"]  # per-GPU batch (weak scaling)
    oh, ow = out_hw(wl)
    weight, bias, w_scales, in_scales, out_scales = make_layer_arrays(wl)
    ctx = Context(local_rank)
    layer = ConvInt8(ctx, cin=wl["cin"], cout=wl["cout"], kh=wl["k"], kw=wl["k"], sh=wl["stride"], sw=wl["stride"], ph=wl["pad"], pw=wl["pad"],
                     groups=wl["groups"], bias_term=1, int8_scale_term=wl["term"], act_type=wl["act"], weight=weight, bias=bias,
                     w_scales=w_scales, in_scales=in_scales, out_scales=out_scales)
    in_dtype = F32_NCHW if wl["in_f32"] else S8_NHWC
    out_dtype = S8_NHWC if wl["term"] > 100 else F32_NCHW
    rng = np.random.default_rng(1234 + rank)
    lib = ctx.lib
    # synthetic activations, generated once into pinned host memory (the e2e leg copies from there)
    if wl["in_f32"]:
        in_shape, in_np = (n, wl["cin"], wl["h"], wl["w"]), np.float32
    else:
        in_shape, in_np = (n, wl["h"], wl["w"], nhwc_channels(wl["cin"])), np.int8
    in_bytes = int(np.prod(in_shape)) * np.dtype(in_np).itemsize
    out_shape = (n, oh, ow, nhwc_channels(wl["cout"])) if out_dtype == S8_NHWC else (n, wl["cout"], oh, ow)
    out_bytes = int(np.prod(out_shape)) * (1 if out_dtype == S8_NHWC else 4)
    hin, hout = C.c_void_p(), C.c_void_p()
    assert lib.ott_host_alloc(in_bytes, C.byref(hin)) == 0 and lib.ott_host_alloc(out_bytes, C.byref(hout)) == 0
    host_in = np.ctypeslib.as_array(C.cast(hin, C.POINTER(C.c_uint8)), shape=(in_bytes,)).view(in_np).reshape(in_shape)
    chunk = max(1, n // 16)
    for i in range(0, n, chunk):
        m = min(chunk, n - i)
        if wl["in_f32"]:
            host_in[i:i + m] = rng.random(size=(m,) + in_shape[1:], dtype=np.float32) * 2.0 - 1.0
        else:
            host_in[i:i + m] = rng.integers(-127, 128, size=(m,) + in_shape[1:], dtype=np.int8)
            host_in[i:i + m, ..., wl["cin"]:] = 0
    din, dout = ctx.malloc(in_bytes), ctx.malloc(out_bytes)
    ctx.check(lib.ott_memcpy_h2d(ctx.h, C.c_void_p(din), hin, in_bytes))
    ctx.sync()

    def step():
        layer.forward(din, in_dtype, n, wl["h"], wl["w"], dout, out_dtype)

    def barrier():
        ctx.sync()
        if dist is not None:
            dist.barrier()

    int8_peak = None
    if rank == 0 and not args.no_peak:
        try:
            int8_peak = int8_tensor_peak_tops()
        except Exception as e:  # the measurement is informative, never required
            print(f"int8 peak measurement skipped: {e}", file=sys.stderr)

    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    e0, e1 = ctx.event(), ctx.event()
    l0 = ctx.launch_count()
    barrier()
    # per-kernel timing of the dominant kernel: events around each step's launches would serialise the
    # stream; the step itself is at most two kernels, so the whole timed region is timed once and the
    # dominant kernel's share is measured separately below.
    ctx.record(e0)
    for _ in range(args.steps):
        step()
    ctx.record(e1)
    barrier()
    ms_total = ctx.elapsed_ms(e0, e1)
    launches = ctx.launch_count() - l0
    # dominant-kernel duration: the convolution kernel alone on int8 activations that an untimed
    # quantize pass left in HBM (same shapes, same launch configuration)
    conv_ms = None
    fused_prologue = layer.kernel_kind == 1  # the tiled depthwise kernel quantizes fp32 input itself: one kernel per step
    if wl["in_f32"] and not fused_prologue:
        cpad = nhwc_channels(wl["cin"])
        dq = ctx.malloc(n * wl["h"] * wl["w"] * cpad)
        ctx.quantize(din, n, wl["cin"], wl["h"], wl["w"], in_scales, 0, dq)
        for _ in range(2):
            layer.forward(dq, S8_NHWC, n, wl["h"], wl["w"], dout, out_dtype)
        ctx.sync()
        k0, k1 = ctx.event(), ctx.event()
        ctx.record(k0)
        for _ in range(args.steps):
            layer.forward(dq, S8_NHWC, n, wl["h"], wl["w"], dout, out_dtype)
        ctx.record(k1)
        ctx.sync()
        conv_ms = ctx.elapsed_ms(k0, k1) / args.steps
        ctx.free(dq)
    else:
        conv_ms = ms_total / args.steps
    clocks = sampler.stop() if rank == 0 else None

    # end-to-end leg: the host-buffer entry point (H2D of the inputs, kernels, D2H of the outputs) per step
    e2e_steps = max(1, min(args.steps, args.e2e_steps))
    for _ in range(1):
        ctx.check(lib.ott_conv_int8_forward_host(ctx.h, layer.h, hin, in_dtype, n, wl["h"], wl["w"], hout, out_dtype))
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        ctx.check(lib.ott_conv_int8_forward_host(ctx.h, layer.h, hin, in_dtype, n, wl["h"], wl["w"], hout, out_dtype))
    barrier()
    e2e_s = (time.perf_counter() - t0) / e2e_steps

    step_ms = ms_total / args.steps
    step_ms, e2e_s, conv_ms = max_over_ranks([step_ms, e2e_s, conv_ms], dist)
    ops, alg_bytes = algorithmic_work(wl, n)
    value = ops * world / (step_ms * 1e-3) / 1e12
    e2e_value = ops * world / e2e_s / 1e12

    if rank == 0:
        hbm_peak, hbm_src = measured_peaks()
        # the dense convolution kernels read int8 (a separate quantize kernel ran before them); the depthwise
        # kernel reads the fp32 input itself
        _, conv_bytes = algorithmic_work(wl if fused_prologue else {**wl, "in_f32": False}, n)
        ai = ops / conv_bytes
        tensor_peak = int8_peak if int8_peak else 3000.0
        tensor_src = "measured live: torch._int_mm 8192^3 int8 (cuBLASLt), best of 10" if int8_peak else "3000 TOP/s, earlier torch._int_mm measurement on this pool"
        if ai * hbm_peak / 1e3 < tensor_peak:  # HBM-bound kernel
            achieved = conv_bytes / (conv_ms * 1e-3) / 1e9
            roof = {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                    "traffic": None, "peak_source": hbm_src}
        else:
            achieved = ops / (conv_ms * 1e-3) / 1e12
            roof = {"bound": "tensor", "achieved": achieved, "peak": tensor_peak, "unit": "TOP/s", "frac": achieved / tensor_peak,
                    "traffic": None, "peak_source": tensor_src}
        roof["kernel"] = lib.ott_conv_int8_kernel_name(ctx.h, layer.h, in_dtype if fused_prologue else S8_NHWC, out_dtype, wl["h"], wl["w"]).decode()
        roof["kernel_ms"] = conv_ms
        roof["algorithmic_bytes_per_launch"] = conv_bytes
        roof["ops_per_launch"] = ops
        traffic_file = ROOT / "profiles" / "traffic.json"
        if traffic_file.exists():
            roof["traffic"] = json.loads(traffic_file.read_text()).get(args.workload)
        cpu = None
        if not args.no_cpu:
            images, _ = cpu_sample_images(wl)
            per_img, kind, cores = cpu_reference_time(wl, images=images, warmup=1)
            ops_img, _ = algorithmic_work(wl, 1)
            cpu = {"value": ops_img / per_img / 1e12, "unit": "TOP/s", "cores": cores, "kind": kind,
                   "sample": f"{images} single-image forwards of the same layer ({per_img * 1e3:.2f} ms each; the reference int8 path is batch-1)"}
        print(json.dumps({
            "metric": "int8_conv_tops", "value": value, "unit": "TOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": step_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "s8xs8->s32",
            "data": "synthetic",
            "config": {"workload": args.workload, **{k: wl[k] for k in ("cin", "cout", "k", "stride", "groups", "h", "w")},
                       "batch_per_gpu": n, "input": "fp32 NCHW" if wl["in_f32"] else "int8 NHWC",
                       "output": "int8 NHWC" if wl["term"] > 100 else "fp32 NCHW",
                       "l2": f"inputs {in_bytes / 1e6:.0f} MB + outputs {out_bytes / 1e6:.0f} MB per step exceed the 126 MB L2; no flush"},
            "clocks": clocks, "gpu_launches": int(launches),
            "e2e": {"value": e2e_value, "unit": "TOP/s", "h2d_bytes_per_step": in_bytes, "d2h_bytes_per_step": out_bytes,
                    "ms_per_step": e2e_s * 1e3, "steps": e2e_steps},
            "roofline": roof, "cpu_baseline": cpu,
        }))
    layer.close()
    ctx.free(din)
    ctx.free(dout)
    lib.ott_host_free(hin)
    lib.ott_host_free(hout)
    ctx.close()
    if dist is not None:
        dist.destroy_process_group()


# ----------------------------------------------------------------------------------------------------
# whole-graph workload: ShuffleNetV2-1.0x int8 backbone (configuration 4), images/s

# Graph workloads. `batch` = images per GPU and step (weak scaling); `total` = images per step over all GPUs (strong scaling, the
# batch is sharded); `chunk` = images per Net forward inside a step.
NET_WORKLOADS = {
    "shufflenetv2_320": dict(height=320, width=320, batch=256, chunk=256, graph="shufflenetv2", outputs=("conv5",),
                             metric="shufflenetv2_int8_images_per_s", title="ShuffleNetV2-1.0x backbone, int8 convolutions, fp32 glue"),
    "nanodet_plus_320": dict(height=320, width=320, total=2048, chunk=256, graph="nanodet_plus", outputs=("head8", "head16", "head32", "head64"),
                             metric="nanodet_plus_int8_images_per_s",
                             title="NanoDet-Plus-style detector: ShuffleNetV2-1.0x backbone + 96-channel Ghost-PAN neck + 4 heads (80 classes, "
                                   "reg_max 7), int8 convolutions, fp32 glue"),
}


def graph_layers(cfg, batch=1):
    from tensor_b200 import graphs
    build = {"shufflenetv2": graphs.shufflenetv2_layers, "nanodet_plus": graphs.nanodet_plus_layers}[cfg["graph"]]
    return build(cfg["height"], cfg["width"], batch=batch)


def _layer_wl(g, hw, in_f32):
    """A graph convolution as a WORKLOADS-style dictionary (for the CPU reference timing)."""
    return dict(cin=g["cin"], cout=g["cout"], k=g["k"], stride=g["stride"], pad=g["pad"], groups=g["groups"], n=1, h=hw[0], w=hw[1],
                term=g["term"], act=g["act"], in_f32=in_f32, w_std=0.1 if g["groups"] > 1 else 0.05)


def net_cpu_reference_time(layers, height, width, reps=2):
    """Seconds per image of the reference's CPU int8 path, summed over the graph's convolution layers, each timed alone
    on one image (a whole-Net run of this graph is impossible in the reference: its packed path corrupts memory on the
    58/116-channel depthwise layers and miscomputes the 58/116-wide pointwise ones). Per layer the path that is valid
    for its widths is used: packed when Cin%8==0 and Cout%4==0 (and the stem), unpacked for other dense layers, the C
    restatement for depthwise layers whose channel count is not a multiple of 8. Glue layers are not timed."""
    from tensor_b200 import graphs
    geo = graphs.conv_geometry(layers)
    hws, _ = graphs.conv_input_hw(layers, height, width)
    int8_blobs = {n for n, g in geo.items() if g["term"] > 100}
    total, how, cores, kind = 0.0, {"packed": 0, "unpacked": 0, "port": 0}, 1, "reference"
    for name, g in geo.items():
        wl = _layer_wl(g, hws[name], in_f32=g["input"] not in int8_blobs)
        dw = g["groups"] > 1
        if dw and g["cin"] % 8 != 0:
            t, k, cores_l = cpu_reference_time(wl, images=reps, warmup=1, force_port=True)
            how["port"] += 1
        elif dw or (g["cin"] % 8 == 0 and g["cout"] % 4 == 0) or g["cin"] == 3:
            t, k, cores_l = cpu_reference_time(wl, images=reps, warmup=1, packed=1)
            how["packed"] += 1
        else:
            t, k, cores_l = cpu_reference_time(wl, images=reps, warmup=1, packed=0)
            how["unpacked"] += 1
        if k == "port" and not (dw and g["cin"] % 8 != 0):
            kind = "port"
        cores = max(cores, cores_l)
        total += t
    return total, how, cores, kind


def run_net_reference_arm(args, cfg):
    if int(os.environ.get("RANK", "0")) != 0:
        return
    layers = graph_layers(cfg)
    secs = []
    for i in range(args.warmup + args.steps):
        t, how, cores, kind = net_cpu_reference_time(layers, cfg["height"], cfg["width"], reps=1)
        if i >= args.warmup:
            secs.append(t)
    per_img = float(np.mean(secs))
    sample = (f"one image per step: sum of the {sum(how.values())} convolution layers timed one by one on the reference's CPU int8 path "
              f"({how['packed']} packed, {how['unpacked']} unpacked, {how['port']} depthwise layers with C%8!=0 on the C restatement because the "
              f"reference cannot run them); glue layers not included; OpenMP {cores} threads")
    value = 1.0 / per_img
    print(json.dumps({
        "impl": "reference", "metric": cfg["metric"], "value": value, "unit": "images/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_img * 1e3, "higher_is_better": True,
        "scaling": "strong" if "total" in cfg else "weak",
        "vs_baseline": None, "dtype": "s8xs8->s32", "data": "synthetic",
        "config": {"workload": args.workload, "input": f"3x{cfg['height']}x{cfg['width']} fp32", "images_per_step": 1},
        "cpu_baseline": {"value": value, "unit": "images/s", "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def build_calibrated_net(cfg, batch, device, seed=0x0771E5):
    """The workload's Net on `device` with seeded weights and activation scales calibrated on one synthetic image, the
    convolutions of the calibration walk running through the GPU library's own layer objects."""
    from graph_walk import calibrate
    from tensor_b200 import F32_NCHW, S8_NHWC, ConvInt8, Context, Net, graphs, nhwc_channels as nc
    layers = graph_layers(cfg, batch)
    params = graphs.make_params(layers, seed)
    x1 = np.random.default_rng(seed).random(size=(1, 3, cfg["height"], cfg["width"]), dtype=np.float32)
    with Context(device) as ctx:
        def conv(name, g, p, a, as_float):
            term = g["term"] - 100 if (as_float and g["term"] > 100) else g["term"]
            layer = ConvInt8(ctx, cin=g["cin"], cout=g["cout"], kh=g["k"], kw=g["k"], sh=g["stride"], sw=g["stride"], ph=g["pad"], pw=g["pad"],
                             groups=g["groups"], bias_term=1, int8_scale_term=term, act_type=g["act"], act_param0=g["act_param0"],
                             weight=p["weight"], bias=p["bias"], w_scales=p["w_scales"], in_scales=p["in_scales"],
                             out_scales=p["out_scales"] if term > 100 else None)
            if a.dtype == np.int8:
                xin = np.zeros((a.shape[0], a.shape[2], a.shape[3], nc(a.shape[1])), np.int8)
                xin[..., :a.shape[1]] = a.transpose(0, 2, 3, 1)
                in_dtype = S8_NHWC
            else:
                xin, in_dtype = a, F32_NCHW
            y = layer.forward_host(xin, in_dtype, S8_NHWC if term > 100 else F32_NCHW)
            layer.close()
            if term > 100:
                y = np.ascontiguousarray(y[..., :g["cout"]].transpose(0, 3, 1, 2))
            return y
        calibrate(layers, params, x1, conv)
    net = Net(device)
    for l in layers:
        net.add_layer(**l)
    net.compile()
    for name, p in params.items():
        net.set_conv_params(name, p["weight"], p["bias"], p["w_scales"], p["in_scales"], p["out_scales"])
    return net, layers, params


def checker_outputs(layers, params, x, outputs):
    """The graph on host images x through the layer-by-layer CPU checker (C restatement of the reference's int8 layer,
    numpy glue layers): what every output blob must equal bit for bit. Used outside the timed regions only."""
    from graph_support import oracle_conv, oracle_upsample
    from graph_walk import walk
    return walk(layers, np.ascontiguousarray(x), oracle_conv(params), want=list(outputs), upsample_fn=oracle_upsample)


def e2e_record(n, world, proc_s, copy_s, group_s, group_parity, in_bytes, out_bytes, steps):
    """The end-to-end entry of the line. One GPU: ott_net_forward on pinned host buffers. Several GPUs: the headline is
    ott_net_group_forward driven by one process (when it ran), and the one-process-per-GPU figure stands beside it."""
    rec = {"unit": "images/s", "steps": steps, "h2d_bytes_per_step": in_bytes * (world if group_s else 1), "d2h_bytes_per_step": out_bytes * (world if group_s else 1),
           "copy_only_ms": copy_s * 1e3,
           "copy_only": "the step's host->device and device->host copies alone, same chunks and streams, no kernels (per GPU, slowest rank)"}
    if group_s:
        rec.update({"value": n * world / group_s, "ms_per_step": group_s * 1e3,
                    "call": f"ott_net_group_forward: one process, one Net replica and host thread per GPU, {n * world} images per call",
                    "parity_checked": group_parity,
                    "one_process_per_gpu": {"value": n * world / proc_s, "ms_per_step": proc_s * 1e3, "call": "ott_net_forward in every rank, slowest rank"}})
    else:
        rec.update({"value": n * world / proc_s, "ms_per_step": proc_s * 1e3, "call": "ott_net_forward"})
    return rec


def kernel_records(device, names, int8_peak, hbm_peak, steps=10, warmup=3):
    """The single-layer configurations as one record each: the layer's convolution kernel timed alone with CUDA events
    on the context's stream (input resident in HBM and larger than L2 together with the output), against the roof that
    bounds it: the measured int8 GEMM peak when 2*ops/bytes * HBM peak exceeds it, else the measured HBM peak."""
    from tensor_b200 import F32_NCHW, S8_NHWC, ConvInt8, Context
    out = {}
    with Context(device) as ctx:
        lib = ctx.lib
        for name in names:
            wl = WORKLOADS[name]
            n = wl["n"]
            oh, ow = out_hw(wl)
            weight, bias, w_scales, in_scales, out_scales = make_layer_arrays(wl)
            layer = ConvInt8(ctx, cin=wl["cin"], cout=wl["cout"], kh=wl["k"], kw=wl["k"], sh=wl["stride"], sw=wl["stride"], ph=wl["pad"],
                             pw=wl["pad"], groups=wl["groups"], bias_term=1, int8_scale_term=wl["term"], act_type=wl["act"], weight=weight,
                             bias=bias, w_scales=w_scales, in_scales=in_scales, out_scales=out_scales)
            in_dtype = F32_NCHW if wl["in_f32"] else S8_NHWC
            out_dtype = S8_NHWC if wl["term"] > 100 else F32_NCHW
            if wl["in_f32"]:
                img_shape, in_np = (wl["cin"], wl["h"], wl["w"]), np.float32
            else:
                img_shape, in_np = (wl["h"], wl["w"], nhwc_channels(wl["cin"])), np.int8
            img_bytes = int(np.prod(img_shape)) * np.dtype(in_np).itemsize
            out_bytes = n * oh * ow * (nhwc_channels(wl["cout"]) if out_dtype == S8_NHWC else wl["cout"] * 4)
            din, dout = ctx.malloc(n * img_bytes), ctx.malloc(out_bytes)
            rng = np.random.default_rng(99)
            # eight distinct random images, repeated over the batch (the kernels' time does not depend on the values)
            for i in range(min(n, 8)):
                if wl["in_f32"]:
                    a = rng.random(size=img_shape, dtype=np.float32) * 2.0 - 1.0
                else:
                    a = rng.integers(-127, 128, size=img_shape, dtype=np.int8)
                    a[..., wl["cin"]:] = 0
                for j in range(i, n, 8):
                    ctx.check(lib.ott_memcpy_h2d(ctx.h, C.c_void_p(din + j * img_bytes), a.ctypes.data_as(C.c_void_p), img_bytes))
                ctx.sync()
            fused = layer.kernel_kind == 1  # the tiled depthwise kernel quantizes fp32 input itself
            src, src_dtype, dq = din, in_dtype, None
            if wl["in_f32"] and not fused:
                dq = ctx.malloc(n * wl["h"] * wl["w"] * nhwc_channels(wl["cin"]))
                ctx.quantize(din, n, wl["cin"], wl["h"], wl["w"], in_scales, 0, dq)
                src, src_dtype = dq, S8_NHWC
            for _ in range(warmup):
                layer.forward(src, src_dtype, n, wl["h"], wl["w"], dout, out_dtype)
            ctx.sync()
            e0, e1 = ctx.event(), ctx.event()
            ctx.record(e0)
            for _ in range(steps):
                layer.forward(src, src_dtype, n, wl["h"], wl["w"], dout, out_dtype)
            ctx.record(e1)
            ctx.sync()
            ms = ctx.elapsed_ms(e0, e1) / steps
            ops, byts = algorithmic_work(wl if fused else {**wl, "in_f32": False}, n)
            tops, gbs = ops / (ms * 1e-3) / 1e12, byts / (ms * 1e-3) / 1e9
            tensor_bound = int8_peak is not None and (ops / byts) * hbm_peak / 1e3 >= int8_peak
            rec = {"kernel": lib.ott_conv_int8_kernel_name(ctx.h, layer.h, src_dtype, out_dtype, wl["h"], wl["w"]).decode(),
                   "ms": ms, "tops": tops, "gbs": gbs, "ops": ops, "algorithmic_bytes": byts, "launches_timed": steps,
                   "input": "fp32 NCHW" if (wl["in_f32"] and fused) else "int8 NHWC", "output": "int8 NHWC" if wl["term"] > 100 else "fp32 NCHW",
                   "bound": "tensor" if tensor_bound else "hbm",
                   "frac": tops / int8_peak if tensor_bound else gbs / hbm_peak}
            if int8_peak:
                rec["frac_of_int8_peak"] = tops / int8_peak
            rec["frac_of_hbm_peak"] = gbs / hbm_peak
            out[name] = rec
            layer.close()
            for p_ in (din, dout, dq):
                if p_:
                    ctx.free(p_)
            lib.ott_alloc_release_cached(ctx.h)
    return out


KERNEL_RECORD_WORKLOADS = ("pw_512_1024_hw56_s8", "pw_256_512_hw56_s8", "pw_64_256_hw56_s8", "dense3x3_64_hw56_n256_s8", "dw3x3s1_c256",
                           "dw3x3s2_c256", "dw3x3s1_c256_s8", "dw3x3s2_c256_s8")


def detect_record(ctx, graph, outputs, images, height, reps=3):
    """The detector's decode step (NanodetPlusDetectionOutput: proposals, sort, NMS; ott_nanodet_detect) on the head blobs one
    replayed chunk left on the device, timed by itself with the host clock (the call ends with the rows on the host). It is
    not part of the timed step: the reference's layer decodes one image, and the benchmark's outputs are the heads."""
    strides = [8, 16, 32, 64][:len(outputs)]
    ptrs, grids = [], []
    for i in range(len(outputs)):
        dptr, shp = graph.output(i)
        ptrs.append(dptr)
        grids.append(int(shp[2]))
        num_class = int(shp[1]) - 32
    arr = (C.c_void_p * len(ptrs))(*ptrs)
    gh = np.array(grids, np.int32)
    st = np.array(strides, np.int32)
    cells = int((gh.astype(np.int64) ** 2).sum())
    rows = np.zeros((images, cells, 6), np.float32)
    counts = np.zeros(images, np.int32)

    def run():
        ctx.check(ctx.lib.ott_nanodet_detect(ctx.h, arr, gh.ctypes.data, gh.ctypes.data, st.ctypes.data, len(ptrs), images, num_class, 8,
                                             C.c_float(0.4), C.c_float(0.5), rows.ctypes.data, counts.ctypes.data, cells))
    run()
    ctx.sync()
    t0 = time.perf_counter()
    for _ in range(reps):
        run()
    dt = (time.perf_counter() - t0) / reps
    return {"ms_per_chunk": dt * 1e3, "images": images, "images_per_s": images / dt, "detections": int(counts.sum()),
            "what": "ott_nanodet_detect on the heads of one chunk: proposals, per-image sort and NMS on the GPU, one copy of the rows to the host; "
                    "host clock; not included in the timed step"}


def run_net_gpu_arm(args, cfg):
    from tensor_b200 import graphs, library
    library()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        if os.environ.get("NCCL_DEBUG", "").upper() in ("", "VERSION"):
            os.environ["NCCL_DEBUG"] = "WARN"  # NCCL's version banner goes to stdout and would precede the JSON line
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    H, W = cfg["height"], cfg["width"]
    strong = "total" in cfg and not args.batch
    n = args.batch or (cfg["total"] // world if strong else cfg["batch"])  # images per GPU and step
    chunk = min(args.chunk or cfg["chunk"], n)
    outputs = list(cfg["outputs"])
    net, layers, params = build_calibrated_net(cfg, chunk, local_rank)
    ctx = net.context()
    lib = ctx.lib
    _, macs = graphs.conv_input_hw(layers, H, W)
    out_elems = [int(np.prod(net.blob_shape(o)[1:])) for o in outputs]  # per image
    in_bytes, out_bytes = n * 3 * H * W * 4, n * sum(out_elems) * 4
    hin = C.c_void_p()
    assert lib.ott_host_alloc(in_bytes, C.byref(hin)) == 0
    houts = []
    for e in out_elems:
        hp = C.c_void_p()
        assert lib.ott_host_alloc(n * e * 4, C.byref(hp)) == 0
        houts.append(hp)
    host_in = np.ctypeslib.as_array(C.cast(hin, C.POINTER(C.c_float)), shape=(n, 3, H, W))
    rng = np.random.default_rng(4321 + rank)
    for i in range(0, n, 16):
        host_in[i:i + 16] = rng.random(size=host_in[i:i + 16].shape, dtype=np.float32)
    din = ctx.malloc(in_bytes)
    ctx.check(lib.ott_memcpy_h2d(ctx.h, C.c_void_p(din), hin, in_bytes))
    ctx.sync()
    img_bytes = 3 * H * W * 4
    chunks = [(b0, min(chunk, n - b0)) for b0 in range(0, n, chunk)]

    # one CUDA graph per chunk: the ~56 (ShuffleNetV2) or ~125 (detector) kernels of a forward replay as one launch
    chunk_graphs = [net.capture("data", C.c_void_p(din + b0 * img_bytes), (nb, 3, H, W), outputs) for b0, nb in chunks] if args.graph else None

    def step():  # one pass over this GPU's n images, `chunk` images per Net forward, everything resident on the device
        if chunk_graphs:
            for g in chunk_graphs:
                g.launch()
            return
        for b0, nb in chunks:
            net.forward_raw("data", C.c_void_p(din + b0 * img_bytes), True, (nb, 3, H, W), outputs, None)

    def barrier():
        ctx.sync()
        if dist is not None:
            dist.barrier()

    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    # The K-step region is timed `repeats` times back to back (events on the Net's stream, a barrier around each); the
    # reported step time is the median repeat, so that a change of a per cent or two shows above the run-to-run noise.
    repeat_ms, launches = [], 0
    for _ in range(max(1, args.repeats)):
        e0, e1 = ctx.event(), ctx.event()
        l0 = ctx.launch_count()
        barrier()
        ctx.record(e0)
        for _ in range(args.steps):
            step()
        ctx.record(e1)
        barrier()
        repeat_ms.append(ctx.elapsed_ms(e0, e1) / args.steps)
        launches = ctx.launch_count() - l0
    repeat_ms = max_over_ranks(repeat_ms, dist)  # per repeat, the slowest rank
    step_ms = float(np.median(repeat_ms))
    clocks = sampler.stop() if rank == 0 else None

    # Output self-check, outside every timed region: the first and the last image of this rank's batch, as the replayed
    # graphs left them on the device, against the layer-by-layer CPU checker, bit for bit.
    parity = None
    if chunk_graphs and not args.no_check:
        check_imgs = sorted({0, n - 1})
        want = [checker_outputs(layers, params, host_in[i:i + 1], outputs) for i in check_imgs]
        parity = True
        for ci, i in enumerate(check_imgs):
            gi, off = i // chunk, i % chunk
            for oi, o in enumerate(outputs):
                dptr, shp = chunk_graphs[gi].output(oi)
                per = int(np.prod(shp[1:]))
                got = ctx.to_host(dptr + off * per * 4, (1,) + tuple(shp[1:]), np.float32)
                parity = parity and bool(np.array_equal(got.view(np.int32), want[ci][o].view(np.int32)))
    # per-layer device times of one chunk (events around every layer; serialised) -> the dominant layer kind and its share.
    # One profiling pass per output blob; a layer that several outputs need is counted once (its longest time).
    cshape = (chunks[0][1], 3, H, W)
    prof = None
    for o in outputs:
        net.profile("data", C.c_void_p(din), True, cshape, o)
        p_o = net.profile("data", C.c_void_p(din), True, cshape, o)
        prof = p_o if prof is None else [(t_, nm, max(a, b)) for (t_, nm, a), (_, _, b) in zip(prof, p_o)]

    # end to end: host fp32 images in (pinned), host fp32 outputs out, every step
    e2e_steps = max(1, min(args.steps, args.e2e_steps))
    shape = (n, 3, H, W)
    out_ptrs = [h.value for h in houts]
    net.forward_raw("data", hin, False, shape, outputs, out_ptrs)
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        net.forward_raw("data", hin, False, shape, outputs, out_ptrs)
    barrier()
    e2e_s = (time.perf_counter() - t0) / e2e_steps

    # the same step with the kernels left out: this rank's input batch up, its outputs down, through the two copy streams the
    # host-buffer forward uses, in the same chunks. What remains of e2e above this is pipeline fill/drain and launch cost.
    dout = ctx.malloc(out_bytes)
    host_chunk = 64

    def copy_only():
        for b0 in range(0, n, host_chunk):
            nb = min(host_chunk, n - b0)
            ctx.check(lib.ott_memcpy_overlapped(ctx.h, 0, C.c_void_p(din + b0 * img_bytes), C.c_void_p(hin.value + b0 * img_bytes), nb * img_bytes))
            off = 0
            for hp, e in zip(houts, out_elems):
                ctx.check(lib.ott_memcpy_overlapped(ctx.h, 1, C.c_void_p(hp.value + b0 * e * 4), C.c_void_p(dout + off + b0 * e * 4), nb * e * 4))
                off += n * e * 4
        ctx.sync()

    saved_out = [np.ctypeslib.as_array(C.cast(hp, C.POINTER(C.c_float)), shape=(n * e,)).copy() for hp, e in zip(houts, out_elems)] if parity is not None else None
    copy_only()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        copy_only()
    barrier()
    copy_s = (time.perf_counter() - t0) / e2e_steps
    ctx.free(dout)
    if saved_out is not None:  # the copy-only leg overwrote the host outputs the self-check below reads
        for hp, e, sv in zip(houts, out_elems, saved_out):
            np.ctypeslib.as_array(C.cast(hp, C.POINTER(C.c_float)), shape=(n * e,))[:] = sv

    # Several GPUs: the product's own multi-GPU call. Rank 0 alone builds one Net replica per GPU (ott_net_group_*) and pushes
    # the whole job's batch, world * n images in one pinned buffer, through ott_net_group_forward: one process, one host thread
    # per GPU. The other ranks wait on the host (a gloo barrier), their GPUs idle.
    group_e2e_s, group_parity = None, None
    if world > 1:
        import torch.distributed as tdist
        side = tdist.new_group(backend="gloo")
        tdist.barrier(group=side)
        if rank == 0:
            from tensor_b200 import NetGroup
            group = NetGroup(list(range(world)))
            for m in group.members:
                for l in layers:
                    m.add_layer(**l)
                m.compile()
                for name, p in params.items():
                    m.set_conv_params(name, p["weight"], p["bias"], p["w_scales"], p["in_scales"], p["out_scales"])
            gn = n * world
            ghin = C.c_void_p()
            assert lib.ott_host_alloc(gn * img_bytes, C.byref(ghin)) == 0
            gin = np.ctypeslib.as_array(C.cast(ghin, C.POINTER(C.c_float)), shape=(gn, 3, H, W))
            for r in range(world):
                gin[r * n:(r + 1) * n] = host_in  # the same images on every GPU: the check below knows their outputs
            ghouts = []
            for e in out_elems:
                hp = C.c_void_p()
                assert lib.ott_host_alloc(gn * e * 4, C.byref(hp)) == 0
                ghouts.append(hp)
            gptrs = [h.value for h in ghouts]
            group.forward_raw("data", ghin, (gn, 3, H, W), outputs, gptrs)
            t0 = time.perf_counter()
            for _ in range(e2e_steps):
                group.forward_raw("data", ghin, (gn, 3, H, W), outputs, gptrs)
            group_e2e_s = (time.perf_counter() - t0) / e2e_steps
            if parity is not None:
                group_parity = True
                for ci, i in enumerate(check_imgs):
                    for r in (0, world - 1):
                        for oi, (o, e) in enumerate(zip(outputs, out_elems)):
                            got = np.ctypeslib.as_array(C.cast(ghouts[oi], C.POINTER(C.c_float)), shape=(gn, e))[r * n + i]
                            group_parity = group_parity and bool(np.array_equal(got.view(np.int32), want[ci][o].reshape(-1).view(np.int32)))
            group.close()
            lib.ott_host_free(ghin)
            for hp in ghouts:
                lib.ott_host_free(hp)
            torch.cuda.set_device(local_rank)  # the replicas made other devices current on this thread
        tdist.barrier(group=side)

    parity_e2e = None
    if parity is not None:
        parity_e2e = True
        for ci, i in enumerate(check_imgs):
            for oi, (o, e) in enumerate(zip(outputs, out_elems)):
                got = np.ctypeslib.as_array(C.cast(houts[oi], C.POINTER(C.c_float)), shape=(n, e))[i]
                parity_e2e = parity_e2e and bool(np.array_equal(got.view(np.int32), want[ci][o].reshape(-1).view(np.int32)))
    if dist is not None and parity is not None:  # every rank checks its own shard; the line carries the conjunction
        import torch
        flags = torch.tensor([int(parity), int(parity_e2e)], device=f"cuda:{local_rank}")
        dist.all_reduce(flags, op=dist.ReduceOp.MIN)
        parity, parity_e2e = bool(flags[0].item()), bool(flags[1].item())
    e2e_s, copy_s = max_over_ranks([e2e_s, copy_s], dist)
    value = whole_job_rate(n, world, step_ms)
    int8_peak, kernels = None, None
    if rank == 0 and world == 1 and not args.no_peak:
        try:
            int8_peak = int8_tensor_peak_tops()
        except Exception as e:  # informative, never required
            print(f"int8 peak measurement skipped: {e}", file=sys.stderr)
    if rank == 0:
        hbm_peak, hbm_src = measured_peaks()
        if world == 1 and not args.no_kernels:
            # the other half of the metric: the single-layer configurations' kernels against their roofs, same process, after
            # the graph steps (the Net's buffers are released first)
            lib.ott_alloc_release_cached(ctx.h)
            kernels = kernel_records(local_rank, KERNEL_RECORD_WORKLOADS, int8_peak, hbm_peak)
        geo = graphs.conv_geometry(layers)
        hws, _ = graphs.conv_input_hw(layers, H, W)
        by_type = {}
        for t_, nm, ms in prof:
            key = t_ if t_ != "Convolution" else ("Convolution/depthwise" if geo[nm]["groups"] > 1 else
                                                  ("Convolution/1x1" if geo[nm]["k"] == 1 else "Convolution/stem3x3"))
            by_type[key] = by_type.get(key, 0.0) + ms
        total_prof = sum(by_type.values())
        # dominant layer kind: its layers' algorithmic bytes (boundary dtypes) over their measured device time
        int8_blobs = {k for k, g in geo.items() if g["term"] > 100}
        routing = {li["name"]: li for li in net.layer_infos()}  # which layers hand over / take over int8 through the glue layers
        kind_of = lambda g: "Convolution/depthwise" if g["groups"] > 1 else ("Convolution/1x1" if g["k"] == 1 else "Convolution/stem3x3")  # noqa: E731
        dom = max((k for k in by_type if k.startswith("Convolution")), key=lambda k: by_type[k])
        dom_bytes = dom_ops = dom_ms = 0.0
        dom_layers = 0
        for t_, nm, ms in prof:
            if t_ != "Convolution" or kind_of(geo[nm]) != dom:
                continue
            g = geo[nm]
            r = routing.get(nm, {})
            wl = _layer_wl(g, hws[nm], in_f32=g["input"] not in int8_blobs and not r.get("gathered_sources"))
            ops, byts = algorithmic_work(wl, cshape[0])
            if r.get("out_int8_channels") or r.get("out_f32_channels"):
                # a layer that stores its channels quantized for their readers, and only the others in fp32
                oh_, ow_ = out_hw(wl)
                byts -= cshape[0] * wl["cout"] * oh_ * ow_ * (1 if wl["term"] > 100 else 4)
                byts += cshape[0] * oh_ * ow_ * (r["out_int8_channels"] + 4 * r["out_f32_channels"])
            dom_bytes += byts
            dom_ops += ops
            dom_ms += ms
            dom_layers += 1
        ach = dom_bytes / (dom_ms * 1e-3) / 1e9
        dom_kernel = {"Convolution/1x1": "dense_umma_kernel (+ quantize_nchw_to_nhwc_kernel where the input is fp32)", "Convolution/depthwise": "depthwise_tiled_kernel",
                      "Convolution/stem3x3": "dense_stem_pool_kernel"}[dom]
        roof = {"bound": "hbm", "achieved": ach, "peak": hbm_peak, "unit": "GB/s", "frac": ach / hbm_peak, "traffic": None,
                "peak_source": hbm_src, "kernel": f"{dom_kernel}: the {dom_layers} {dom} layers of the graph",
                "kernel_ms": dom_ms / dom_layers, "algorithmic_bytes_per_launch": dom_bytes / dom_layers, "ops_per_launch": dom_ops / dom_layers,
                "launches_per_step": dom_layers,
                "timed": "serialised per-layer pass (CUDA events around every layer of one forward, kernels launched one by one: no graph "
                         "replay, no overlap between consecutive kernels); the headline step is the replayed graph",
                "frac_scaled_to_timed_step": (dom_bytes / (by_type[dom] / total_prof * step_ms * 1e-3) / 1e9) / hbm_peak,
                "time_share_by_layer_kind": {k: round(v / total_prof, 4) for k, v in sorted(by_type.items(), key=lambda kv: -kv[1])},
                "profiled_ms_per_step": total_prof,
                "top_layers_ms": [[nm_, round(ms_, 4)] for _, nm_, ms_ in sorted(prof, key=lambda p: -p[2])[:12]]}
        traffic_file = ROOT / "profiles" / "traffic.json"
        if traffic_file.exists():
            roof["traffic"] = json.loads(traffic_file.read_text()).get(args.workload)
        decode = None
        if cfg["graph"] == "nanodet_plus" and chunk_graphs:
            decode = detect_record(ctx, chunk_graphs[0], outputs, chunks[0][1], H)
        cpu = None
        if not args.no_cpu:
            per_img, how, cores, kind = net_cpu_reference_time(graph_layers(cfg), H, W, reps=3)
            cpu = {"value": 1.0 / per_img, "unit": "images/s", "cores": cores, "kind": kind,
                   "sample": f"3 images: sum of the convolution layers timed one by one, N=1 ({how['packed']} packed, {how['unpacked']} unpacked reference "
                             f"layers, {how['port']} depthwise layers with C%8!=0 on the C restatement); glue layers not included"}
        print(json.dumps({
            "metric": cfg["metric"], "value": value, "unit": "images/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": step_ms, "repeats": len(repeat_ms), "repeat_ms_per_step": [round(v, 5) for v in repeat_ms],
            "parity_checked": parity, "parity_checked_e2e": parity_e2e,
            "parity_check": None if parity is None else f"images {check_imgs} of rank 0's batch (every rank checks its own), outputs {outputs}, bit for bit against the layer-by-layer CPU checker",
            "higher_is_better": True, "scaling": "strong" if strong else "weak",
            "vs_baseline": None, "dtype": "s8xs8->s32", "data": "synthetic",
            "config": {"workload": args.workload, "graph": cfg["title"], "batch_per_gpu": n, "images_per_forward": chunk,
                       "input": f"3x{H}x{W} fp32 NCHW",
                       "output": ", ".join("%s %dx%dx%d fp32" % ((o,) + tuple(net.blob_shape(o)[1:])) for o in outputs),
                       "conv_gop_per_image": 2 * macs / 1e9, "cuda_graph": bool(chunk_graphs),
                       "l2": f"input batch {in_bytes / 1e6:.0f} MB and every stage's activations exceed the 126 MB L2; no flush"},
            "conv_tops": 2.0 * macs * n * world / (step_ms * 1e-3) / 1e12,
            "clocks": clocks, "gpu_launches": int(launches),
            "e2e": e2e_record(n, world, e2e_s, copy_s, group_e2e_s, group_parity, in_bytes, out_bytes, e2e_steps),
            "roofline": roof, "cpu_baseline": cpu,
            "int8_peak": None if int8_peak is None else {"tops": int8_peak, "how": "torch._int_mm 8192^3 int8 (cuBLASLt), best of 10, CUDA events, same process"},
            "kernels": kernels,
            **({"decode": decode} if decode else {}),
        }))
    for g in chunk_graphs or []:
        g.close()
    net.close()
    if dist is not None:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS) + sorted(NET_WORKLOADS))
    ap.add_argument("--batch", type=int, default=0, help="per-GPU batch of a graph workload (default: the configuration's)")
    ap.add_argument("--chunk", type=int, default=0, help="graph workloads: images per Net forward inside a step (default: the configuration's)")
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-graph", dest="graph", action="store_false", help="graph workloads: launch every kernel of a forward separately "
                    "instead of replaying the captured CUDA graph")
    ap.add_argument("--no-peak", action="store_true", help="skip the live int8 GEMM peak measurement")
    ap.add_argument("--repeats", type=int, default=5, help="graph workloads: how many times the K-step region is timed (the median is reported)")
    ap.add_argument("--no-check", action="store_true", help="graph workloads: skip the bit-for-bit output self-check against the CPU checker")
    ap.add_argument("--no-kernels", action="store_true", help="graph workloads: skip the single-layer kernel records")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.workload in NET_WORKLOADS:
        cfg = NET_WORKLOADS[args.workload]
        if args.impl == "reference":
            run_net_reference_arm(args, cfg)
        else:
            run_net_gpu_arm(args, cfg)
        return
    wl = WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference_arm(args, wl)
    else:
        run_gpu_arm(args, wl)


if __name__ == "__main__":
    main()
