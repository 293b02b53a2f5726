#!/usr/bin/env python
"""Benchmark of the fused-op hot path (softmax / RMSNorm / LayerNorm) on B200.

Workload: the fused-op micro-bench configuration -- (a) fp32 softmax over the
last axis of logits[32,16,1024,1024] ~ N(0,4) under a causal -inf mask, (b) bf16
RMSNorm and LayerNorm over x[16384,4096] ~ N(0,1), gamma ~ N(1,0.02), beta = 0,
eps = 1e-6.  One "step" is one pass of all three kernels over that batch.

Bytes.  GB/s figures count the bytes a pass MUST move: every output byte written once and every input byte that can
influence an output read once.  Under the causal mask the inputs right of the diagonal influence nothing (their
outputs are exactly 0), so the softmax counts 2^31 output bytes + the lower triangle of the logits at the 16-byte
granularity the kernel loads at (1,077,936,128 B) = 3,225,419,776 B; each norm counts 2*2^26*2 = 268,435,456 B.
A step is 3,762,290,688 B.  The dense count the configuration table quotes (read everything once + write once =
4,294,967,296 B for the softmax, 4,831,838,208 B per step) is reported beside it under keys named "dense".

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

One process per GPU (torchrun sets RANK / LOCAL_RANK / WORLD_SIZE); every rank
runs the full batch on its own data (weak scaling, no collective on the data
path); rank 0 prints ONE JSON line.  `value` is device-resident throughput;
`e2e` is the same metric through the reference-facing host-pointer call from
pinned host memory, every byte copied in and out inside the timed region:
b200_execute_host_sliced walks the batch in 16 slices so uploads, kernels and
downloads overlap (the unsliced b200_execute_host time is reported beside it).
`--impl reference` times the CPU restatement of the same ops on the host cores.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

SM_SHAPE = (32, 16, 1024, 1024)
NORM_SHAPE = (16384, 4096)
EPS = 1e-6
E2E_SLICES = int(os.environ.get("B200MLX_E2E_SLICES", "16"))  # leading-axis slices of the end-to-end leg (must divide 32 softmax batches and 16384 norm rows)


def causal_softmax_bytes(shape, elt=4, vec_bytes=16):
    """Bytes a causal softmax over the last axis must move: the whole output, plus for row q of each [Sq, Sk] plane
    the first q+1 inputs rounded up to whole 16-byte vectors (what lies right of the diagonal cannot change any output)."""
    sq, sk = shape[-2], shape[-1]
    planes = int(np.prod(shape[:-2]))
    per_vec = vec_bytes // elt
    q = np.arange(sq, dtype=np.int64)
    read = int((np.minimum(-(-(q + 1) // per_vec) * per_vec, sk) * elt).sum()) * planes
    return read + int(np.prod(shape)) * elt


SM_DENSE_BYTES = 2 * int(np.prod(SM_SHAPE)) * 4          # read everything once + write once
SM_BYTES = causal_softmax_bytes(SM_SHAPE)                  # what the causal pass must move
NORM_BYTES = 2 * int(np.prod(NORM_SHAPE)) * 2
STEP_BYTES = SM_BYTES + 2 * NORM_BYTES
STEP_DENSE_BYTES = SM_DENSE_BYTES + 2 * NORM_BYTES
# DRAM traffic of one causal softmax launch at the configuration's size, from an ncu capture of exactly that launch
# (dram__bytes_read.sum, dram__bytes_write.sum; the capture and its command are in
# profiles/softmax_causal_f32_rows524288x1024.md).  bench.py checks it against SM_BYTES and says so in the line.
SM_NCU_DRAM_READ, SM_NCU_DRAM_WRITE = 1_107_461_888, 2_092_402_176   # 55 MB of the 2^31 output bytes were still dirty in L2 when the kernel ended
METRIC = "GB/s (softmax/norm)"
def config_dict():
    """The workload description both arms print (identical, so the two lines are comparable key by key)."""
    return {"workload": WORKLOAD, "l2": "inputs larger than L2: every step streams 3.8 GB through a 126 MB L2",
            "per_gpu_batch": "full (weak scaling, no data-path collective)", "bytes_per_step": STEP_BYTES,
            "dense_bytes_per_step": STEP_DENSE_BYTES, "bytes": BYTES_NOTE}


BYTES_NOTE = ("bytes that must move: all outputs + the inputs that can influence them (causal softmax: lower triangle at 16-byte "
              "granularity); the dense read-all + write-all count is reported under 'dense' keys")
WORKLOAD = ("fused-op micro-bench: fp32 causal softmax logits[32,16,1024,1024] + bf16 RMSNorm + bf16 LayerNorm x[16384,4096], "
            "eps 1e-6")


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            return json.load(fh), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


# ----------------------------------------------------------------------------- inputs ---
def make_inputs(seed: int, sm_shape=SM_SHAPE, norm_shape=NORM_SHAPE, logits_out=None):
    """Seeded synthetic inputs (PCG64): logits ~ N(0, 4) fp32, x ~ N(0,1) bf16, gamma ~ N(1, 0.02) bf16, beta = 0."""
    import ml_dtypes
    rng = np.random.default_rng(seed)
    n = int(np.prod(sm_shape))
    logits = logits_out if logits_out is not None else np.empty(n, dtype=np.float32)
    chunk = 1 << 24
    for lo in range(0, n, chunk):
        hi = min(n, lo + chunk)
        rng.standard_normal(hi - lo, dtype=np.float32, out=logits[lo:hi])
        logits[lo:hi] *= 2.0
    x = rng.standard_normal(int(np.prod(norm_shape)), dtype=np.float32).astype(ml_dtypes.bfloat16).reshape(norm_shape)
    gamma = (1.0 + 0.02 * rng.standard_normal(norm_shape[1], dtype=np.float32)).astype(ml_dtypes.bfloat16)
    beta = np.zeros(norm_shape[1], dtype=ml_dtypes.bfloat16)
    return logits.reshape(sm_shape), x, gamma, beta


# ------------------------------------------------------------------------ clock sampler ---
class ClockSampler:
    """Samples SM clock, power and clock-event reasons of one GPU through NVML while a region runs (read-only)."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap",
               0x80: "hw_power_brake_slowdown", 0x2: "applications_clocks_setting", 0x100: "display_clock_setting", 0x10: "sync_boost"}

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz, self.power = [], set(), None, []
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = index
            if visible:
                ids = [v for v in visible.split(",") if v.strip()]
                if index < len(ids) and ids[index].strip().isdigit():
                    phys = int(ids[index])
            self._h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _run(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                self.power.append(nv.nvmlDeviceGetPowerUsage(self._h) / 1000.0)
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.002)

    def __enter__(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        return {"sm_mhz": float(np.median(self.samples)), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples), "power_w_max": max(self.power) if self.power else None}


# --------------------------------------------------------------------------- CPU legs ---
def cpu_pass(cport, logits, x, gamma, beta, out_sm, out_n):
    cport.softmax_f32(logits, 1.0, True, logits.shape[-2], out=out_sm)
    cport.norm(x, gamma, None, EPS, True, out=out_n)
    cport.norm(x, gamma, beta, EPS, False, out=out_n)


def verify_against_oracle(cport, logits, x, gamma, beta, out_sm, out_rms, out_ln, samples=64, seed=7):
    """Compares sampled rows of the three outputs with the CPU restatement (oracle/oracle_c.c, itself pinned to the
    float64 oracle by the tests).  Softmax rows are taken as whole [Sq, Sk] planes' rows: a row's mask depends on its
    position inside its plane.  Returns (ok, worst violation of |got-want| <= rtol*|want| + atol)."""
    rng = np.random.default_rng(seed)
    worst = -np.inf
    planes = logits.reshape(-1, logits.shape[-2], logits.shape[-1])
    got_planes = out_sm.reshape(planes.shape)
    for pi in rng.choice(planes.shape[0], size=4, replace=False):   # 4 planes x 16 rows
        want = cport.softmax_f32(planes[pi], 1.0, True, planes.shape[1])
        rows = rng.choice(planes.shape[1], size=samples // 4, replace=False)
        g, w = got_planes[pi][rows].astype(np.float64), want[rows].astype(np.float64)
        worst = max(worst, float((np.abs(g - w) - (1e-5 * np.abs(w) + 1e-7)).max()))
    rows = np.sort(rng.choice(x.shape[0], size=samples, replace=False))
    xs = np.ascontiguousarray(x[rows])
    for got, want in ((out_rms[rows], cport.norm(xs, gamma, None, EPS, True)), (out_ln[rows], cport.norm(xs, gamma, beta, EPS, False))):
        g, w = got.astype(np.float64), want.astype(np.float64)
        worst = max(worst, float((np.abs(g - w) - (8e-3 * np.abs(w) + 4e-4)).max()))   # bf16: one ulp is 2^-8 relative
    return bool(worst <= 0), worst


def run_cpu_baseline(logits, x, gamma, beta, passes=3):
    """The CPU restatement on the whole configuration (the same batch the GPU arm runs), best of `passes`."""
    from oracle import cport
    cport.use_all_cores()   # torchrun exports OMP_NUM_THREADS=1
    out_sm, out_n = np.empty_like(logits), np.empty_like(x)
    cpu_pass(cport, logits, x, gamma, beta, out_sm, out_n)  # warm-up (page faults, thread pool)
    best = float("inf")
    for _ in range(passes):
        t0 = time.perf_counter()
        cpu_pass(cport, logits, x, gamma, beta, out_sm, out_n)
        best = min(best, time.perf_counter() - t0)
    return {"value": STEP_BYTES / best / 1e9, "unit": "GB/s", "cores": cport.num_threads(), "kind": "port", "ms_per_step": best * 1e3,
            "sample": f"the whole configuration: softmax on logits{list(logits.shape)} + RMSNorm + LayerNorm on x{list(x.shape)}, "
                      f"best of {passes} passes after one warm-up; bytes counted as in the GPU arm ({STEP_BYTES} per step)"}


def run_reference_arm(args, rank, world):
    """The CPU implementation of the path on the host cores.  The reference's own implementation is Apple-only
    (MPSGraph), and GoMLX's pure-Go CPU backend needs a Go toolchain that is absent, so this times the C
    restatement (oracle/oracle_c.c) with every host thread OpenMP gives it, on the whole configuration."""
    if rank != 0:
        return
    from oracle import cport
    cport.use_all_cores()   # torchrun exports OMP_NUM_THREADS=1
    logits, x, gamma, beta = make_inputs(0)
    out_sm, out_n = np.empty_like(logits), np.empty_like(x)
    for _ in range(max(1, min(args.warmup, 3))):
        cpu_pass(cport, logits, x, gamma, beta, out_sm, out_n)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_pass(cport, logits, x, gamma, beta, out_sm, out_n)
    dt = time.perf_counter() - t0
    value = STEP_BYTES * args.steps / dt / 1e9
    sample = f"each step = the whole configuration: softmax on logits{list(SM_SHAPE)} + RMSNorm + LayerNorm on x{list(NORM_SHAPE)}"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": config_dict(),
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cport.num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "reference's own MPSGraph path and GoMLX's Go CPU backend are unavailable on this box; C restatement timed instead",
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------- GPU arm ---
def time_bare_copies(torch, device, uploads, downloads, barrier, reps=3):
    """ms per repetition of cudaMemcpyAsync over the given pinned (pointer, nbytes) lists, H2D and D2H concurrently."""
    rt = ctypes.CDLL("libcudart.so.12")
    rt.cudaMemcpyAsync.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_void_p]
    rt.cudaMemcpyAsync.restype = ctypes.c_int
    H2D, D2H = 1, 2
    dev = f"cuda:{device}"
    d_up = [torch.empty(n, dtype=torch.uint8, device=dev) for _, n in uploads]
    d_down = [torch.empty(n, dtype=torch.uint8, device=dev) for _, n in downloads]
    s_up, s_down = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)

    def once():
        for (hp, n), d in zip(uploads, d_up):
            if rt.cudaMemcpyAsync(d.data_ptr(), hp, n, H2D, s_up.cuda_stream) != 0:
                raise RuntimeError("cudaMemcpyAsync H2D failed")
        for (hp, n), d in zip(downloads, d_down):
            if rt.cudaMemcpyAsync(hp, d.data_ptr(), n, D2H, s_down.cuda_stream) != 0:
                raise RuntimeError("cudaMemcpyAsync D2H failed")
    once()
    torch.cuda.synchronize()
    barrier()
    e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
    e0.record(s_up)
    s_down.wait_event(e0)
    for _ in range(reps):
        once()
    e1.record(s_up)
    e2.record(s_down)
    torch.cuda.synchronize()
    return max(e0.elapsed_time(e1), e0.elapsed_time(e2)) / reps


def compile_graph(b200, backend, name, shapes_in, build):
    builder = backend.Builder(name)
    f = builder.Main()
    params = [f.Parameter(f"p{i}", s) for i, s in enumerate(shapes_in)]
    outs = build(f, *params)
    f.Return(list(outs) if isinstance(outs, (list, tuple)) else [outs], None)
    return builder, builder.Compile()


def run_b200_arm(args, rank, local_rank, world):
    import torch
    import torch.distributed as dist

    import go_darwinml_b200 as b200

    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    backend = b200.New(f"device={local_rank}")
    L = b200.lib()
    from go_darwinml_b200 import _lib as libmod

    def host_alloc(nbytes, dtype, shape):
        err = libmod.B200Error()
        p = L.b200_host_alloc(nbytes, ctypes.byref(err))
        if err.code:
            raise RuntimeError(L.take_string(err.message))
        buf = (ctypes.c_char * nbytes).from_address(p)
        return p, np.frombuffer(buf, dtype=dtype).reshape(shape)

    # pinned host copies of the inputs and of the outputs (e2e leg)
    import ml_dtypes
    bf16 = np.dtype(ml_dtypes.bfloat16)
    n_sm, n_norm = int(np.prod(SM_SHAPE)), int(np.prod(NORM_SHAPE))
    p_logits, h_logits = host_alloc(n_sm * 4, np.float32, (n_sm,))
    logits, x, gamma, beta = make_inputs(rank, logits_out=h_logits)
    p_x, h_x = host_alloc(n_norm * 2, bf16, NORM_SHAPE)
    h_x[...] = x
    p_g, h_g = host_alloc(NORM_SHAPE[1] * 2, bf16, (NORM_SHAPE[1],))
    h_g[...] = gamma
    p_b, h_b = host_alloc(NORM_SHAPE[1] * 2, bf16, (NORM_SHAPE[1],))
    h_b[...] = beta
    p_osm, h_osm = host_alloc(n_sm * 4, np.float32, SM_SHAPE)
    p_orms, h_orms = host_alloc(n_norm * 2, bf16, NORM_SHAPE)
    p_oln, h_oln = host_alloc(n_norm * 2, bf16, NORM_SHAPE)

    D = b200.dtypes
    s_logits, s_x, s_g = b200.Shape(D.Float32, SM_SHAPE), b200.Shape(D.BFloat16, NORM_SHAPE), b200.Shape(D.BFloat16, (NORM_SHAPE[1],))
    _, exe_sm = compile_graph(b200, backend, "softmax", [s_logits], lambda f, a: f.FusedSoftmaxMasked(a, 1.0, True, None))
    _, exe_sm_plain = compile_graph(b200, backend, "softmax_plain", [s_logits], lambda f, a: f.FusedSoftmaxMasked(a, 1.0, False, None))
    _, exe_rms = compile_graph(b200, backend, "rms", [s_x, s_g], lambda f, a, g: f.FusedRMSNorm(a, [-1], EPS, g))
    _, exe_ln = compile_graph(b200, backend, "ln", [s_x, s_g, s_g], lambda f, a, g, b: f.FusedLayerNorm(a, [-1], EPS, g, b))
    _, exe_all = compile_graph(b200, backend, "all", [s_logits, s_x, s_g, s_g],
                               lambda f, a, xx, g, b: (f.FusedSoftmaxMasked(a, 1.0, True, None), f.FusedRMSNorm(xx, [-1], EPS, g),
                                                      f.FusedLayerNorm(xx, [-1], EPS, g, b)))
    d_logits = backend.BufferFromFlatData(local_rank, h_logits, s_logits)
    d_x = backend.BufferFromFlatData(local_rank, h_x.reshape(-1), s_x)
    d_g = backend.BufferFromFlatData(local_rank, h_g, s_g)
    d_b = backend.BufferFromFlatData(local_rank, h_b, s_g)
    backend.Synchronize(local_rank)

    err = libmod.B200Error()
    stream = torch.cuda.ExternalStream(L.b200_device_stream(local_rank, ctypes.byref(err)), device=local_rank)

    def step(ev=None):
        """One pass of the hot path on device-resident inputs; optionally brackets the softmax launch with events."""
        if ev:
            ev[0].record(stream)
        o1 = exe_sm.Execute([d_logits], None, local_rank)
        if ev:
            ev[1].record(stream)
        o2 = exe_rms.Execute([d_x, d_g], None, local_rank)
        if ev:
            ev[2].record(stream)
        o3 = exe_ln.Execute([d_x, d_g, d_b], None, local_rank)
        if ev:
            ev[3].record(stream)
        for o in o1 + o2 + o3:
            backend.BufferFinalize(o)

    def barrier():
        backend.Synchronize(local_rank)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(args.steps)]
    t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(local_rank)
    with sampler:
        t_start.record(stream)
        for i in range(args.steps):
            step(evs[i])
        t_end.record(stream)
        backend.Synchronize(local_rank)
        torch.cuda.synchronize()
    barrier()
    elapsed_ms = t_start.elapsed_time(t_end)
    sm_ms = float(np.mean([e[0].elapsed_time(e[1]) for e in evs]))
    rms_ms = float(np.mean([e[1].elapsed_time(e[2]) for e in evs]))
    ln_ms = float(np.mean([e[2].elapsed_time(e[3]) for e in evs]))

    # the unmasked softmax on the same logits: every byte is read and written, so its GB/s is a plain bandwidth figure
    def plain_step():
        for o in exe_sm_plain.Execute([d_logits], None, local_rank):
            backend.BufferFinalize(o)
    for _ in range(3):
        plain_step()
    backend.Synchronize(local_rank)
    p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    p0.record(stream)
    for _ in range(10):
        plain_step()
    p1.record(stream)
    backend.Synchronize(local_rank)
    plain_ms = p0.elapsed_time(p1) / 10

    # ---- e2e: host pointers in, host pointers out, through b200_execute_host ----
    in_ptrs = (ctypes.c_void_p * 4)(p_logits, p_x, p_g, p_b)
    in_sizes = (ctypes.c_int64 * 4)(n_sm * 4, n_norm * 2, NORM_SHAPE[1] * 2, NORM_SHAPE[1] * 2)
    in_dtypes = (ctypes.c_int * 4)(int(D.Float32), int(D.BFloat16), int(D.BFloat16), int(D.BFloat16))
    shp = [(ctypes.c_int64 * 4)(*SM_SHAPE), (ctypes.c_int64 * 2)(*NORM_SHAPE), (ctypes.c_int64 * 1)(NORM_SHAPE[1]), (ctypes.c_int64 * 1)(NORM_SHAPE[1])]
    in_shapes = (ctypes.POINTER(ctypes.c_int64) * 4)(*[ctypes.cast(s, ctypes.POINTER(ctypes.c_int64)) for s in shp])
    in_ranks = (ctypes.c_int * 4)(4, 2, 1, 1)
    out_ptrs = (ctypes.c_void_p * 3)(p_osm, p_orms, p_oln)
    out_sizes = (ctypes.c_int64 * 3)(n_sm * 4, n_norm * 2, n_norm * 2)
    out_dtypes = (ctypes.c_int * 3)(int(D.Float32), int(D.BFloat16), int(D.BFloat16))
    oshp = [(ctypes.c_int64 * 4)(*SM_SHAPE), (ctypes.c_int64 * 2)(*NORM_SHAPE), (ctypes.c_int64 * 2)(*NORM_SHAPE)]
    out_shapes = (ctypes.POINTER(ctypes.c_int64) * 3)(*[ctypes.cast(s, ctypes.POINTER(ctypes.c_int64)) for s in oshp])
    out_ranks = (ctypes.c_int * 3)(4, 2, 2)

    def e2e_step():
        e = libmod.B200Error()
        ok = L.b200_execute_host(exe_all.handle, in_ptrs, in_sizes, in_dtypes, in_shapes, in_ranks, 4, out_ptrs, out_sizes, out_dtypes,
                                 out_shapes, out_ranks, 3, ctypes.byref(e))
        if not ok:
            raise RuntimeError(L.take_string(e.message))

    # The same call over E2E_SLICES leading-axis slices (b200_execute_host_sliced): the executable is compiled for one
    # slice, and the upload of slice s+1, the kernels of slice s and the download of slice s-1 overlap.
    sl_sm, sl_norm = (SM_SHAPE[0] // E2E_SLICES,) + tuple(SM_SHAPE[1:]), (NORM_SHAPE[0] // E2E_SLICES, NORM_SHAPE[1])
    _, exe_slice = compile_graph(b200, backend, "all_slice", [b200.Shape(D.Float32, sl_sm), b200.Shape(D.BFloat16, sl_norm), s_g, s_g],
                                 lambda f, a, xx, g, b: (f.FusedSoftmaxMasked(a, 1.0, True, None), f.FusedRMSNorm(xx, [-1], EPS, g),
                                                        f.FusedLayerNorm(xx, [-1], EPS, g, b)))
    sliced_flags = (ctypes.c_int * 4)(1, 1, 0, 0)

    def e2e_sliced_step():
        e = libmod.B200Error()
        ok = L.b200_execute_host_sliced(exe_slice.handle, in_ptrs, sliced_flags, 4, out_ptrs, 3, E2E_SLICES, ctypes.byref(e))
        if not ok:
            raise RuntimeError(L.take_string(e.message))

    def time_host_calls(fn, n):
        fn()
        barrier()
        e_start, e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e_start.record(stream)
        for _ in range(n):
            fn()
        e_end.record(stream)
        backend.Synchronize(local_rank)
        torch.cuda.synchronize()
        return e_start.elapsed_time(e_end)

    e2e_steps = max(3, min(args.steps, 10))
    e2e_whole_ms = time_host_calls(e2e_step, 3) / 3
    e2e_sampler = ClockSampler(local_rank)
    with e2e_sampler:
        e2e_ms = time_host_calls(e2e_sliced_step, e2e_steps)
    h2d = n_sm * 4 + n_norm * 2 + 2 * NORM_SHAPE[1] * 2
    d2h = n_sm * 4 + 2 * n_norm * 2

    # The outputs of the last end-to-end step are in host memory: check sampled rows against the CPU restatement
    # (outside every timed region).
    from oracle import cport
    cport.use_all_cores()
    verified, verify_worst = verify_against_oracle(cport, h_logits.reshape(SM_SHAPE), h_x, h_g, h_b, h_osm, h_orms, h_oln)

    # Yardstick for the end-to-end figure: the same pinned buffers moved by bare cudaMemcpyAsync calls, uploads on one
    # stream and downloads on another at the same time, no kernels.  It shows what the box's host<->device path
    # gives this process, i.e. how much of the end-to-end time is the copies themselves.
    copy_floor_ms = None
    try:
        copy_floor_ms = time_bare_copies(torch, local_rank, [(p_logits, n_sm * 4), (p_x, n_norm * 2)],
                                         [(p_osm, n_sm * 4), (p_orms, n_norm * 2), (p_oln, n_norm * 2)], barrier)
    except Exception as ex:  # noqa: BLE001  (a yardstick must never sink the line)
        copy_floor_ms = f"unavailable: {type(ex).__name__}: {ex}"

    # the other configurations (DotGeneral sweep, transformer forwards); never allowed to sink the headline line
    extras, extras_error = None, None
    if not args.no_extras:
        for o in (d_logits, d_x, d_g, d_b):
            backend.BufferFinalize(o)
        L.b200_device_trim(local_rank)
        try:
            extras = run_extras(b200, backend, L, libmod, torch, stream, local_rank, world, measured_peaks()[0])
        except Exception as ex:  # noqa: BLE001
            extras_error = f"{type(ex).__name__}: {ex}"
    gpt_ms = extras["gpt2_small_fwd_bf16"]["ms_per_forward"] if extras else 0.0
    llama_ms = extras["llama_1b_fwd_bf16"]["ms_per_forward"] if extras else 0.0

    # max over ranks, on device-measured times
    from go_darwinml_b200.sharding import max_over_ranks
    own = {"rank": rank, "ms_per_step": elapsed_ms / args.steps, "e2e_ms_per_step": e2e_ms / e2e_steps, "gpt2_ms_per_forward": gpt_ms,
           "llama_ms_per_forward": llama_ms, "verified": verified}
    per_rank = [own]
    if world > 1:
        per_rank = [None] * world
        dist.all_gather_object(per_rank, own)
    elapsed_ms, e2e_ms, gpt_ms, llama_ms = max_over_ranks([elapsed_ms, e2e_ms, gpt_ms, llama_ms], device=f"cuda:{local_rank}")

    if rank == 0:
        peaks, peak_src = measured_peaks()
        hbm = peaks["hbm_gbs"]
        ms_per_step = elapsed_ms / args.steps
        value = world * STEP_BYTES / (ms_per_step * 1e-3) / 1e9
        e2e_value = world * STEP_BYTES / (e2e_ms / e2e_steps * 1e-3) / 1e9
        achieved = SM_BYTES / (sm_ms * 1e-3) / 1e9
        traffic = SM_NCU_DRAM_READ + SM_NCU_DRAM_WRITE

        def kern(ms, nbytes, **more):
            d = {"ms": ms, "GB/s": nbytes / ms / 1e6, "frac_of_peak": nbytes / ms / 1e6 / hbm, "bytes": nbytes}
            d.update(more)
            return d
        line = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": config_dict(),
            "dense": {"value": world * STEP_DENSE_BYTES / (ms_per_step * 1e-3) / 1e9, "unit": "GB/s",
                      "note": "the same time over the read-all + write-all byte count; under the causal mask the kernel never loads what "
                              "lies right of the diagonal, so this is an effective rate, not a bandwidth"},
            "verified": bool(all(r["verified"] for r in per_rank)),
            "verified_how": "64 sampled rows of each of the three outputs of the last end-to-end step on every rank against the CPU restatement "
                            f"(fp32 rel 1e-5, bf16 rel 8e-3); worst violation on rank 0 {verify_worst:.2e} (<= 0 passes)",
            "clocks": sampler.summary(),
            "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps,
                    "ms_per_step": e2e_ms / e2e_steps,
                    "call": f"b200_execute_host_sliced, {E2E_SLICES} batch slices, pinned host buffers, copies overlapped with kernels",
                    "unsliced_ms_per_step": e2e_whole_ms, "unsliced_call": "b200_execute_host", "clocks": e2e_sampler.summary(),
                    "bare_copy_ms_per_step_rank0": copy_floor_ms,
                    "bare_copy_note": "the same pinned buffers through plain cudaMemcpyAsync, uploads and downloads on two streams at once, "
                                      "no kernels: the floor the host<->device path of this box sets for one step"},
            "gpu_launches": args.steps * (exe_sm.NumLaunches() + exe_rms.NumLaunches() + exe_ln.NumLaunches()),
            "roofline": {"bound": "hbm", "kernel": "softmax_rows_kernel<float,8,32> (causal)", "achieved": achieved,
                         "peak": hbm, "unit": "GB/s", "frac": achieved / hbm, "peak_source": peak_src,
                         "traffic": traffic, "bytes_per_launch": SM_BYTES, "dense_bytes_per_launch": SM_DENSE_BYTES,
                         "dense_GB/s": SM_DENSE_BYTES / sm_ms / 1e6, "ms_per_launch": sm_ms,
                         "traffic_vs_bytes": traffic / SM_BYTES,
                         "note": "achieved = bytes the causal pass must move (all outputs + lower-triangle inputs in 16-byte vectors) / launch "
                                 "time; traffic = ncu dram read + write of this very launch size"},
            "kernels": {"softmax_causal_f32": kern(sm_ms, SM_BYTES, dense_GBps=SM_DENSE_BYTES / sm_ms / 1e6),
                        "softmax_plain_f32": kern(plain_ms, SM_DENSE_BYTES, note="same logits, no mask: read all + write all; timed apart from the step"),
                        "rms_norm_bf16": kern(rms_ms, NORM_BYTES), "layer_norm_bf16": kern(ln_ms, NORM_BYTES)},
        }
        if world > 1:
            line["per_rank"] = per_rank
        if extras:
            extras["gpt2_small_fwd_bf16"]["tokens_per_s_all_gpus"] = world * 16 * 1024 / (gpt_ms * 1e-3)   # batch 16 per GPU (weak)
            extras["llama_1b_fwd_bf16"]["tokens_per_s_all_gpus"] = 64 // world * world * 2048 / (llama_ms * 1e-3)  # batch 64 in total (strong)
            line["extras"] = extras
        if extras_error:
            line["extras_error"] = extras_error
        if world == 1:
            line["cpu_baseline"] = run_cpu_baseline(h_logits.reshape(SM_SHAPE), h_x, h_g, h_b)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


# ----------------------------------------------------------- other configurations (extras) ---
def run_extras(b200, backend, L, libmod, torch, stream, local_rank, world, peaks):
    """DotGeneral sweep (TFLOP/s) and the two transformer forwards (tokens/s).  Reported next to the headline
    metric; inputs and weights are seeded random tensors created on the device and wrapped as buffers."""
    import go_darwinml_b200.workloads as W
    dev = f"cuda:{local_rank}"
    gen = torch.Generator(device=dev).manual_seed(1234 + local_rank)
    out = {}

    def timed(fn, iters, warmup=2):
        for _ in range(warmup):
            fn()
        backend.Synchronize(local_rank)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(iters):
            fn()
        e1.record(stream)
        backend.Synchronize(local_rank)
        return e0.elapsed_time(e1) / iters

    # --- DotGeneral sweep: [8,M,K]x[8,K,N] and [8,K,M]x[8,K,N], M=N=K in {1024,4096,8192}, bf16 and fp32 ---
    sweep = {}
    for dt_name, tdt, code in (("bf16", torch.bfloat16, 6), ("f32", torch.float32, 7)):
        for n in (1024, 4096, 8192):
            a = torch.randn(8, n, n, generator=gen, device=dev, dtype=torch.float32).to(tdt)
            b = torch.randn(8, n, n, generator=gen, device=dev, dtype=torch.float32).to(tdt)
            c = torch.empty(8, n, n, device=dev, dtype=tdt)
            for form, a_kmajor in (("BMK_BKN", 1), ("BKM_BKN", 0)):
                def launch():
                    e = libmod.B200Error()
                    if not L.b200_k_gemm(local_rank, a.data_ptr(), b.data_ptr(), c.data_ptr(), 8, n, n, n, a_kmajor, 0, code, None, 0,
                                         ctypes.byref(e)):
                        raise RuntimeError(L.take_string(e.message))
                ms = timed(launch, 5 if n == 8192 else 10)
                tf = 2 * 8 * n ** 3 / (ms * 1e-3) / 1e12
                sweep[f"{dt_name}_{form}_{n}"] = {"ms": ms, "TFLOP/s": tf, "frac_of_bf16_peak": tf / peaks["bf16_tflops"]}
            del a, b, c
    out["dot_general_sweep"] = sweep

    def model_tokens_per_s(name, cfg, shapes, forward, flops_per_token, iters):
        bufs, dts, keep = W.make_device_params(b200, torch, shapes, cfg, local_rank)
        builder, exe = W.build_executable(b200, backend, name, [(s, d) for (_, s), d in zip(shapes, dts)], forward)

        def run():
            for o in exe.Execute(bufs, None, local_rank):
                backend.BufferFinalize(o)
        ms = timed(run, iters, warmup=3)   # the second run with the same buffers records the CUDA graph: keep that out of the timing
        tokens = cfg.batch * cfg.seq
        res = {"ms_per_forward": ms, "tokens_per_s_this_gpu": tokens / (ms * 1e-3), "batch_this_gpu": cfg.batch,
               "launches_per_forward": exe.NumLaunches(), "TFLOP/s": tokens * flops_per_token / (ms * 1e-3) / 1e12,
               "arena_GiB": L.b200_exec_arena_bytes(exe.handle) / 2 ** 30}
        exe.Finalize()
        builder.Finalize()
        L.b200_device_trim(local_rank)
        return res

    g = W.GPT2Config()
    out["gpt2_small_fwd_bf16"] = model_tokens_per_s("gpt2", g, W.gpt2_param_shapes(g),
                                                   lambda f, *p: W.gpt2_forward(f, g, int(b200.dtypes.BFloat16), *p),
                                                   W.gpt2_flops_per_token(g), 20)
    # Incremental decoding of the same model: 64 greedy steps from one start token per sequence inside ONE executable (a
    # While loop that runs on the device once the plan is replayed; KV caches of 1024 positions extended in place).
    n_new = 64
    dshapes = W.gpt2_decode_param_shapes(g)
    dec = model_tokens_per_s("gpt2-decode", g, dshapes, lambda f, *p: W.gpt2_greedy_decode(f, g, int(b200.dtypes.BFloat16), n_new, *p), 0.0, 5)
    out["gpt2_small_greedy_decode_bf16"] = {
        "ms_per_call": dec["ms_per_forward"], "new_tokens_per_sequence": n_new, "batch_this_gpu": g.batch, "cache_positions": g.seq,
        "ms_per_step": dec["ms_per_forward"] / n_new, "tokens_per_s_this_gpu": g.batch * n_new / (dec["ms_per_forward"] * 1e-3),
        "launches_outside_the_loop": dec["launches_per_forward"], "arena_GiB": dec["arena_GiB"],
        "note": "every step attends over the whole 1024-position cache under a position mask; weights (0.25 GB) are re-read from HBM each step"}
    lc = W.LlamaConfig(batch=64 // world)  # batch 64 sharded by batch across the GPUs
    out["llama_1b_fwd_bf16"] = model_tokens_per_s("llama", lc, W.llama_param_shapes(lc),
                                                 lambda f, *p: W.llama_forward(f, lc, int(b200.dtypes.BFloat16), *p),
                                                 W.llama_flops_per_token(lc), 20)
    # Incremental decoding of the Llama-shaped model: batch 16 per GPU, 32 greedy steps in one executable, grouped-query
    # attention (32 heads on 8 KV heads) over 2048-position caches, rotary embedding at the loop-carried position.
    ld = W.LlamaConfig(batch=16)
    n_new_l = 32
    ldec = model_tokens_per_s("llama-decode", ld, W.llama_decode_param_shapes(ld),
                              lambda f, *p: W.llama_greedy_decode(f, ld, int(b200.dtypes.BFloat16), n_new_l, *p), 0.0, 5)
    weight_bytes = 2 * (sum(int(np.prod(sh)) for nm, sh in W.llama_param_shapes(ld) if nm not in ("ids", "embed", "rope_cos", "rope_sin")))
    out["llama_1b_greedy_decode_bf16"] = {
        "ms_per_call": ldec["ms_per_forward"], "new_tokens_per_sequence": n_new_l, "batch_this_gpu": ld.batch, "cache_positions": ld.seq,
        "ms_per_step": ldec["ms_per_forward"] / n_new_l, "tokens_per_s_this_gpu": ld.batch * n_new_l / (ldec["ms_per_forward"] * 1e-3),
        "launches_outside_the_loop": ldec["launches_per_forward"], "arena_GiB": ldec["arena_GiB"],
        "weight_GB_read_per_step": weight_bytes / 1e9,
        "weights_GB/s": weight_bytes / 1e9 / (ldec["ms_per_forward"] / n_new_l * 1e-3),
        "note": "every step reads all the weights once (the step's floor at the copy rate) and attends over the whole cache under a position mask"}
    if world > 1:
        # The one optional exchange of the path: a weight split by columns over the ranks, the all-gather of the result
        # fused into the GEMM epilogue (peer stores over NVLink), checked bit for bit against the single-GPU GEMM and
        # timed beside GEMM + NCCL all-gather.  Every rank takes part; rank 0 reports.
        from go_darwinml_b200.sharding import column_sharded_matmul_check
        out["column_sharded_matmul"] = column_sharded_matmul_check(backend, local_rank, int(os.environ.get("RANK", "0")), world,
                                                                   8192, 16384, 4096, iters=10, warmup=3)
    return out


def ml_dtypes_bf16():
    import ml_dtypes
    return ml_dtypes.bfloat16


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-extras", action="store_true", help="skip the DotGeneral sweep and the transformer forwards")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference_arm(args, rank, world)
    else:
        run_b200_arm(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
