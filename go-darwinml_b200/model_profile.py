"""Per-step timing of one forward pass of a benchmark model, through b200_execute_profiled.

  python go-darwinml_b200/model_profile.py llama --batch 8
  python go-darwinml_b200/model_profile.py gpt2 --batch 16

Prints the launch plan with CUDA-event times per step, then the same times grouped by step kind.
"""
from __future__ import annotations

import argparse
import collections
import os
import re
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("model", choices=["gpt2", "llama"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--device", type=int, default=0)
    ap.add_argument("--full", action="store_true", help="print every step, not only the per-kind table")
    args = ap.parse_args()
    import torch

    import go_darwinml_b200 as b200
    import go_darwinml_b200.workloads as W

    backend = b200.New(f"device={args.device}")
    code = int(b200.dtypes.BFloat16)
    if args.model == "gpt2":
        cfg = W.GPT2Config(batch=args.batch)
        shapes, fwd, fpt = W.gpt2_param_shapes(cfg), (lambda f, *p: W.gpt2_forward(f, cfg, code, *p)), W.gpt2_flops_per_token(cfg)
    else:
        cfg = W.LlamaConfig(batch=args.batch)
        shapes, fwd, fpt = W.llama_param_shapes(cfg), (lambda f, *p: W.llama_forward(f, cfg, code, *p)), W.llama_flops_per_token(cfg)
    bufs, dts, keep = W.make_device_params(b200, torch, shapes, cfg, args.device)
    builder, exe = W.build_executable(b200, backend, args.model, [(s, d) for (_, s), d in zip(shapes, dts)], fwd)
    for _ in range(2):
        for o in exe.Execute(bufs, None, args.device):
            backend.BufferFinalize(o)
    backend.Synchronize(args.device)
    outs, report = exe.ExecuteProfiled(bufs)
    for o in outs:
        backend.BufferFinalize(o)
    if args.full:
        print(report)
    kinds = collections.OrderedDict()
    total = 0.0
    for line in report.splitlines():
        m = re.match(r"\s*([0-9.]+) ms\s+[0-9.]+%\s+(\w+(?:\[[A-Za-z ]+)?)", line)
        if not m or "total of" in line:
            continue
        ms, kind = float(m.group(1)), m.group(2).split("[")[0] if not m.group(2).startswith(("ewise", "move")) else m.group(2)
        kinds.setdefault(kind, [0, 0.0])
        kinds[kind][0] += 1
        kinds[kind][1] += ms
        total += ms
    print(f"{args.model} batch {cfg.batch} seq {cfg.seq}: {total:.3f} ms per forward, {cfg.batch * cfg.seq / total * 1e3:,.0f} tokens/s, "
          f"{cfg.batch * cfg.seq * fpt / total / 1e9:.1f} TFLOP/s, {exe.NumLaunches()} launches")
    for kind, (n, ms) in sorted(kinds.items(), key=lambda kv: -kv[1][1]):
        print(f"  {ms:10.3f} ms  {100 * ms / total:5.1f}%  x{n:<4d} {kind}")


if __name__ == "__main__":
    main()
