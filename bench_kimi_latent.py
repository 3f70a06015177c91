"""Latency of the Kimi-K3 latent MoE block on one GPU.

    python bench_kimi_latent.py --tokens 8 --steps 10 --warmup 3

Geometry: the reference's ``kimi-k3-*-layer-ep8`` cases (megabench/cases.py:315-334: 896 experts, top-16,
hidden 7168, latent 3584, intermediate 3072, two shared experts, 8 sequences per rank), every expert
on this GPU (the reference's ``serial`` form). Inputs are seeded random tensors in the right formats,
made on the device (``synthetic.kimi_latent_inputs``). Timing: CUDA events on the current stream for
every call, the L2 flushed before each step; prints one JSON line with the median latency, the bytes
a call has to read (dense bf16 matrices, the router, the MXFP4 matrices of the experts that were hit)
and the fraction of the measured copy bandwidth that they stand for.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

from bench_ep import L2_FLUSH_BYTES, flush_l2  # noqa: E402
from bench_megamoe import measured_hbm_peak  # noqa: E402
from vibe_megakernel_b200 import synthetic  # noqa: E402
from vibe_megakernel_b200.kimi_latent import LatentMoe, LatentMoeConfig  # noqa: E402


def measure(tokens: int, experts: int = 896, topk: int = 16, hidden: int = 7168, latent: int = 3584, inter: int = 3072,
            shared: int = 2, steps: int = 10, warmup: int = 3, seed: int = 0, device=None, flush: torch.Tensor | None = None) -> dict:
    device = torch.device(device if device is not None else "cuda:0")
    values, normalized = synthetic.kimi_latent_inputs(tokens, experts, topk, hidden, latent, inter, shared, seed, device)
    layer = LatentMoe(LatentMoeConfig(hidden, latent, inter, experts, topk, shared), max_tokens=tokens, device=device)
    if flush is None:
        flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=device)
    out = None
    for _ in range(warmup):
        flush_l2(flush)
        out = layer.forward(values, normalized, check_status=True)
    torch.cuda.synchronize(device)
    times = []
    for _ in range(steps):
        flush_l2(flush)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        layer.forward(values, normalized)
        b.record()
        torch.cuda.synchronize(device)
        times.append(a.elapsed_time(b) * 1e3)
    times.sort()
    median = times[len(times) // 2]
    hit = int(torch.unique(out["expert_ids"]).numel())
    dense = 2 * (2 * latent * hidden + 3 * shared * inter * hidden) + 4 * experts * hidden
    per_expert = 3 * latent * inter // 2 + 3 * latent * inter // 32
    algorithmic = dense + hit * per_expert + 4 * tokens * hidden
    peak, kind = measured_hbm_peak()
    gbs = algorithmic / median / 1e3
    return {"metric": "Kimi-K3 latent MoE block latency", "value": round(median, 2), "unit": "us", "min_us": round(times[0], 2),
            "steps": steps, "warmup": warmup,
            "config": {"workload": f"kimi-k3 layer MoE block, all experts on one GPU: T={tokens} E={experts} top{topk} H={hidden} "
                                   f"L={latent} I={inter} shared={shared}", "l2": "flushed before every step", "data": "synthetic"},
            "experts_hit": hit, "algorithmic_bytes": algorithmic, "launches": layer.launches(),
            "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": peak, "unit": "GB/s", "frac": round(gbs / peak, 4),
                         "peak_kind": kind},
            "dtype": "mxfp4 x bf16 (as two e4m3 pieces) -> f32; dense bf16 -> f32"}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--seed", type=int, default=0)
    args = ap.parse_args()
    torch.cuda.set_device(0)
    print(json.dumps(measure(args.tokens, steps=args.steps, warmup=args.warmup, seed=args.seed)))


if __name__ == "__main__":
    main()
