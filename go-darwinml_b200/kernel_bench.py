"""Times ONE kernel of libb200mlx.so through its direct C-ABI entry point.

  python go-darwinml_b200/kernel_bench.py softmax  --rows 65536 --cols 1024 --dtype f32 [--causal] [--iters 20]
  python go-darwinml_b200/kernel_bench.py rmsnorm  --rows 16384 --cols 4096 --dtype bf16
  python go-darwinml_b200/kernel_bench.py layernorm --rows 16384 --cols 4096 --dtype bf16
  python go-darwinml_b200/kernel_bench.py gemm --batch 8 --m 4096 --n 4096 --k 4096 --dtype bf16 [--a-km] [--b-nk] [--act gelu]
  python go-darwinml_b200/kernel_bench.py ewise --expr chain4 --rows 65536 --cols 2048 --dtype bf16   # 4 leaves, 6 ops: the run-time compiled path
  python go-darwinml_b200/kernel_bench.py reduce --expr sumsq --rows 16384 --cols 4096 --dtype bf16   # ReduceSum(x * x) over rows, one fused launch
  python go-darwinml_b200/kernel_bench.py decode-attention --batch 64 --heads 12 --kv-heads 12 --seq 1024 --bhsd --dtype bf16   # one query over a KV cache
  python go-darwinml_b200/kernel_bench.py few-rows --m 16 --n 3072 --k 768 --dtype bf16 --act gelu   # a decoding step's projection
  python go-darwinml_b200/kernel_bench.py copy --rows 16384 --cols 4096 --dtype bf16    # yardstick, not a kernel of this library
  python go-darwinml_b200/kernel_bench.py fill --rows 524288 --cols 1024 --dtype f32    # yardstick: write-only stream

Inputs are seeded random tensors resident in HBM; timing is CUDA events on the
library's stream after warm-up; between timed launches a buffer twice the size
of L2 is READ unless the operands exceed L2 anyway (a flush that writes would
leave L2 full of dirty lines, whose write-back the timed kernel then pays for).  Prints one JSON line with the
mean launch time, the achieved GB/s (algorithmic bytes) or TFLOP/s, and the
fraction of the measured peak when MEASURED_PEAKS.json is present.  Small shapes
of this tool are what the ncu captures under profiles/ were taken on.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

DT = {"f32": (7, 4), "bf16": (6, 2), "f16": (5, 2)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["softmax", "rmsnorm", "layernorm", "gemm", "attention", "decode-attention", "few-rows", "ewise", "reduce", "copy", "fill"])
    ap.add_argument("--rows", type=int, default=65536)
    ap.add_argument("--cols", type=int, default=1024)
    ap.add_argument("--seq-q", type=int, default=0)
    ap.add_argument("--causal", action="store_true")
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--a-km", action="store_true", help="A stored [batch, K, M]")
    ap.add_argument("--b-nk", action="store_true", help="B stored [batch, N, K]")
    ap.add_argument("--act", default="none", choices=["none", "gelu", "relu", "silu", "tanh"],
                    help="gemm: add a bias [N] and this activation in the epilogue (a dense layer)")
    ap.add_argument("--expr", default="add", choices=["add", "bias", "rope", "chain", "chain4", "sumsq", "sum", "colsum"],
                    help="ewise / reduce: which fused chain to time")
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--bhsd", action="store_true")
    ap.add_argument("--dtype", default="f32", choices=list(DT))
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--device", type=int, default=0)
    ap.add_argument("--no-flush", action="store_true")
    args = ap.parse_args()

    import torch

    import go_darwinml_b200 as b200
    from go_darwinml_b200 import _lib as libmod

    backend = b200.New(f"device={args.device}")
    L = b200.lib()
    code, es = DT[args.dtype]
    torch.cuda.set_device(args.device)
    err = libmod.B200Error()
    stream = torch.cuda.ExternalStream(L.b200_device_stream(args.device, ctypes.byref(err)), device=args.device)
    tdt = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}[args.dtype]
    gen = torch.Generator(device=f"cuda:{args.device}").manual_seed(0)

    def rand(*shape, scale=1.0):
        return (torch.randn(*shape, generator=gen, device=f"cuda:{args.device}", dtype=torch.float32) * scale).to(tdt)

    def check(ok, e):
        if not ok:
            raise RuntimeError(L.take_string(e.message))

    if args.kernel == "softmax":
        x, y = rand(args.rows, args.cols, scale=2.0), torch.empty(args.rows, args.cols, device=f"cuda:{args.device}", dtype=tdt)
        seq_q = args.seq_q or min(args.rows, args.cols)
        work, unit, kind = 2 * args.rows * args.cols * es, "GB/s", "hbm"
        operand_bytes = work

        def launch():
            e = libmod.B200Error()
            check(L.b200_k_softmax(args.device, x.data_ptr(), y.data_ptr(), args.rows, args.cols, code, 1.0, int(args.causal), seq_q,
                                   ctypes.byref(e)), e)
    elif args.kernel in ("rmsnorm", "layernorm"):
        x, y = rand(args.rows, args.cols), torch.empty(args.rows, args.cols, device=f"cuda:{args.device}", dtype=tdt)
        g, b = (1 + 0.02 * rand(args.cols).float()).to(tdt), torch.zeros(args.cols, device=f"cuda:{args.device}", dtype=tdt)
        work, unit, kind = 2 * args.rows * args.cols * es, "GB/s", "hbm"
        operand_bytes = work

        def launch():
            e = libmod.B200Error()
            if args.kernel == "rmsnorm":
                check(L.b200_k_rms_norm(args.device, x.data_ptr(), g.data_ptr(), y.data_ptr(), args.rows, args.cols, code, 1e-6, ctypes.byref(e)), e)
            else:
                check(L.b200_k_layer_norm(args.device, x.data_ptr(), g.data_ptr(), b.data_ptr(), y.data_ptr(), args.rows, args.cols, code, 1e-6,
                                          ctypes.byref(e)), e)
    elif args.kernel == "copy":
        # Yardstick only: the CUDA runtime's device-to-device copy of a [rows, cols] tensor, timed like the kernels above.
        # It shows what fraction of the measured peak (taken on a far larger copy) a plain copy of THIS size reaches.
        x, y = rand(args.rows, args.cols), torch.empty(args.rows, args.cols, device=f"cuda:{args.device}", dtype=tdt)
        work, unit, kind = 2 * args.rows * args.cols * es, "GB/s", "hbm"
        operand_bytes = work

        def launch():
            with torch.cuda.stream(stream):
                y.copy_(x, non_blocking=True)
    elif args.kernel == "fill":
        # Yardstick only: the CUDA runtime's memset of a [rows, cols] tensor -- what a write-only stream of this size reaches.
        y = torch.empty(args.rows, args.cols, device=f"cuda:{args.device}", dtype=tdt)
        work, unit, kind = args.rows * args.cols * es, "GB/s", "hbm"
        operand_bytes = 2 * work

        def launch():
            with torch.cuda.stream(stream):
                y.zero_()
    elif args.kernel == "ewise":
        # a fused elementwise chain compiled through the graph layer (one launch); bytes = distinct inputs + output
        npdt = {"f32": np.float32, "bf16": __import__("ml_dtypes").bfloat16, "f16": np.float16}[args.dtype]
        S = lambda *d: b200.Shape(b200.dtypes.from_numpy(np.dtype(npdt)), d)
        R, C = args.rows, args.cols
        builder = backend.Builder("ewise")
        f = builder.Main()
        if args.expr == "add":
            shapes = [(R, C), (R, C)]
            ps = [f.Parameter(f"p{i}", S(*sh)) for i, sh in enumerate(shapes)]
            y = f.Add(ps[0], ps[1])
        elif args.expr == "bias":
            shapes = [(R, C), (C,)]
            ps = [f.Parameter(f"p{i}", S(*sh)) for i, sh in enumerate(shapes)]
            y = f.Add(ps[0], f.BroadcastInDim(ps[1], S(R, C), [1]))
        elif args.expr == "rope":
            H, Dh = C // 64, 64
            shapes = [(R, H, Dh), (R, H, Dh), (R, Dh), (R, Dh)]
            ps = [f.Parameter(f"p{i}", S(*sh)) for i, sh in enumerate(shapes)]
            cb = f.BroadcastInDim(ps[2], S(R, H, Dh), [0, 2])
            sb = f.BroadcastInDim(ps[3], S(R, H, Dh), [0, 2])
            y = f.Add(f.Mul(ps[0], cb), f.Mul(ps[1], sb))
        elif args.expr == "chain4":
            # 4 leaves, 6 ops, outside the two templated shapes: tanh((x * w + b) * y) - max(x, y)
            shapes = [(R, C), (C,), (R,), (R, C)]
            ps = [f.Parameter(f"p{i}", S(*sh)) for i, sh in enumerate(shapes)]
            t = f.Add(f.Mul(ps[0], f.BroadcastInDim(ps[1], S(R, C), [1])), f.BroadcastInDim(ps[2], S(R, C), [0]))
            y = f.Sub(f.Tanh(f.Mul(t, ps[3])), f.Max(ps[0], ps[3]))
        else:
            shapes = [(R, C), (C,), (C,)]
            ps = [f.Parameter(f"p{i}", S(*sh)) for i, sh in enumerate(shapes)]
            y = f.Tanh(f.Add(f.Mul(ps[0], f.BroadcastInDim(ps[1], S(R, C), [1])), f.BroadcastInDim(ps[2], S(R, C), [1])))
        f.Return([y], None)
        exe = builder.Compile()
        tens = [rand(*sh) for sh in shapes]
        bufs = []
        for t, sh in zip(tens, shapes):
            e = libmod.B200Error()
            bufs.append(b200.Buffer(L.b200_buffer_wrap(args.device, t.data_ptr(), code, (ctypes.c_int64 * len(sh))(*sh), len(sh), ctypes.byref(e))))
        work = (sum(t.numel() for t in tens) + R * C) * es
        unit, kind = "GB/s", "hbm"
        operand_bytes = work
        print(exe.Describe().strip(), file=sys.stderr)

        def launch():
            for o in exe.Execute(bufs, None, args.device):
                backend.BufferFinalize(o)
    elif args.kernel == "reduce":
        # a Reduce whose operand is an elementwise chain, compiled through the graph layer; bytes = input + output
        npdt = {"f32": np.float32, "bf16": __import__("ml_dtypes").bfloat16, "f16": np.float16}[args.dtype]
        S = lambda *d: b200.Shape(b200.dtypes.from_numpy(np.dtype(npdt)), d)
        R, C = args.rows, args.cols
        builder = backend.Builder("reduce")
        f = builder.Main()
        x = f.Parameter("x", S(R, C))
        if args.expr == "sumsq":
            y, out_elems = f.ReduceSum(f.Mul(x, x), 1), R
        elif args.expr == "colsum":
            y, out_elems = f.ReduceSum(x, 0), C
        else:
            y, out_elems = f.ReduceSum(x, 1), R
        f.Return([y], None)
        exe = builder.Compile()
        t = rand(R, C)
        e = libmod.B200Error()
        bufs = [b200.Buffer(L.b200_buffer_wrap(args.device, t.data_ptr(), code, (ctypes.c_int64 * 2)(R, C), 2, ctypes.byref(e)))]
        work = (R * C + out_elems) * es
        unit, kind = "GB/s", "hbm"
        operand_bytes = work
        print(exe.Describe().strip(), file=sys.stderr)

        def launch():
            for o in exe.Execute(bufs, None, args.device):
                backend.BufferFinalize(o)
    elif args.kernel in ("decode-attention", "few-rows"):
        # the decoding step's two kernels, through the graph layer (one launch each)
        npdt = {"bf16": __import__("ml_dtypes").bfloat16, "f16": np.float16}[args.dtype]
        S = lambda *d: b200.Shape(b200.dtypes.from_numpy(np.dtype(npdt)), d)
        builder = backend.Builder(args.kernel)
        f = builder.Main()
        if args.kernel == "decode-attention":
            # one query position per (batch, head) over a cache of --seq keys under a position mask; bytes = K and V
            B, H, Hkv, Sk = args.batch, args.heads, args.kv_heads, args.seq
            shp = (lambda h, s: (B, h, s, 64)) if args.bhsd else (lambda h, s: (B, s, h, 64))
            shapes = [shp(H, 1), shp(Hkv, Sk), shp(Hkv, Sk)]
            ps = [f.Parameter(f"p{i}", S(*sh)) for i, sh in enumerate(shapes)]
            mask = f.Parameter("mask", b200.Shape(b200.dtypes.Bool, (1, 1, 1, Sk)))
            mask_t = (torch.arange(Sk, device=f"cuda:{args.device}") <= Sk - 2).reshape(1, 1, 1, Sk).contiguous()
            y = f.FusedScaledDotProductAttention(ps[0], ps[1], ps[2], mask, H, Hkv, 0 if args.bhsd else 1, 0.125, False)
            work = 2 * B * Hkv * Sk * 64 * es
        else:
            # X[m <= 16, k] W[k, n] (+ bias and --act): bytes = W
            M, N, K = args.m, args.n, args.k
            act = ["none", "gelu", "relu", "silu", "tanh"].index(args.act)
            shapes = [(M, K), (K, N)] + ([(N,)] if act else [])
            ps = [f.Parameter(f"p{i}", S(*sh)) for i, sh in enumerate(shapes)]
            y = f.FusedDense(ps[0], ps[1], ps[2] if act else None, act)
            work = K * N * es
        f.Return([y], None)
        exe = builder.Compile()
        tens = [rand(*sh, scale=0.05 if args.kernel == "few-rows" else 1.0) for sh in shapes]
        bufs = []
        for t, sh in zip(tens, shapes):
            e = libmod.B200Error()
            bufs.append(b200.Buffer(L.b200_buffer_wrap(args.device, t.data_ptr(), code, (ctypes.c_int64 * len(sh))(*sh), len(sh), ctypes.byref(e))))
        if args.kernel == "decode-attention":
            e = libmod.B200Error()
            bufs.append(b200.Buffer(L.b200_buffer_wrap(args.device, mask_t.data_ptr(), int(b200.dtypes.Bool), (ctypes.c_int64 * 4)(1, 1, 1, Sk), 4,
                                                       ctypes.byref(e))))
        unit, kind = "GB/s", "hbm"
        operand_bytes = work
        print(exe.Describe().strip(), file=sys.stderr)

        def launch():
            for o in exe.Execute(bufs, None, args.device):
                backend.BufferFinalize(o)
    elif args.kernel == "attention":
        B, H, Hkv, S = args.batch, args.heads, args.kv_heads, args.seq
        shp = (lambda h: (B, h, S, 64)) if args.bhsd else (lambda h: (B, S, h, 64))
        q, kk, v = rand(*shp(H)), rand(*shp(Hkv)), rand(*shp(Hkv))
        o = torch.empty_like(q)
        work = 4 * B * H * S * S * 64 * (0.5 if args.causal else 1.0)
        unit, kind = "TFLOP/s", "tensor"
        operand_bytes = (q.numel() * 2 + kk.numel() * 2) * es

        def launch():
            e = libmod.B200Error()
            check(L.b200_k_attention(args.device, q.data_ptr(), kk.data_ptr(), v.data_ptr(), o.data_ptr(), B, H, Hkv, S, S, 64,
                                     int(not args.bhsd), int(args.causal), 0.125, code, ctypes.byref(e)), e)
    else:
        B, M, N, K = args.batch, args.m, args.n, args.k
        a = rand(B, K, M) if args.a_km else rand(B, M, K)
        bb = rand(B, N, K) if args.b_nk else rand(B, K, N)
        c = torch.empty(B, M, N, device=f"cuda:{args.device}", dtype=tdt)
        work, unit, kind = 2 * B * M * N * K, "TFLOP/s", "tensor"
        operand_bytes = (a.numel() + bb.numel() + c.numel()) * es

        act = ["none", "gelu", "relu", "silu", "tanh"].index(args.act)
        bias = rand(N) if act else None

        def launch():
            e = libmod.B200Error()
            check(L.b200_k_gemm(args.device, a.data_ptr(), bb.data_ptr(), c.data_ptr(), B, M, N, K, int(not args.a_km), int(args.b_nk), code,
                                bias.data_ptr() if act else None, act, ctypes.byref(e)), e)

    torch.cuda.synchronize()
    flush = None
    if not args.no_flush and operand_bytes < 512 << 20:
        flush = torch.zeros(256 << 20, dtype=torch.uint8, device=f"cuda:{args.device}")
        flush_sink = torch.zeros((), dtype=torch.int64, device=f"cuda:{args.device}")
    for _ in range(args.warmup):
        launch()
    backend.Synchronize(args.device)
    times = []
    for _ in range(args.iters):
        if flush is not None:
            with torch.cuda.stream(stream):
                flush_sink.copy_(flush.view(torch.int64).sum(), non_blocking=True)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        launch()
        e1.record(stream)
        backend.Synchronize(args.device)
        times.append(e0.elapsed_time(e1))
    ms = float(np.mean(times))
    best = float(np.min(times))
    achieved = work / (ms * 1e-3) / (1e9 if kind == "hbm" else 1e12)
    out = {"kernel": args.kernel, "args": {k: v for k, v in vars(args).items() if k != "kernel"}, "ms_mean": ms, "ms_best": best,
           "achieved": achieved, "unit": unit, "l2": "flushed between launches" if flush is not None else "operands exceed L2"}
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        with open(peaks_path) as fh:
            peaks = json.load(fh)
        peak = peaks["hbm_gbs"] if kind == "hbm" else peaks["bf16_tflops"]
        out["peak"], out["frac_of_measured"] = peak, achieved / peak
    print(json.dumps(out))


if __name__ == "__main__":
    main()
