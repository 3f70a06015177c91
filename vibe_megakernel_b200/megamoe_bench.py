"""Latency of the routed experts in the MegaMoE-native formats on one GPU.

    python -m vibe_megakernel_b200.megamoe_bench --tokens 512 --steps 10 --warmup 3

Geometry: the reference's ``megamoe-layer-deepseek-v4-pro`` cases (megabench/cases.py:380-388: 384
experts, top-6, hidden 7168, intermediate 3072), every expert on this GPU (its ``serial`` form).
Inputs are seeded random codes in the right formats, made on the device: packed E2M1 weight bytes with
E8M0 scales near 2^-7, E4M3 rows with scales near 2^-7, routing drawn like the reference's ``route``
(log-normal expert popularity, Gumbel top-k, weights that sum to 2.5; megabench/tasks/megamoe.py:65-80).
Timing: CUDA events on the current stream for every call, the L2 flushed before each step; prints
one JSON line with the median latency, the bytes of the experts that were hit, and the fraction of the
measured copy bandwidth that they stand for.
"""

from __future__ import annotations

import argparse
import json
from pathlib import Path

import torch

from .ep_bench import L2_FLUSH_BYTES, flush_l2
from .megamoe import MegaMoe, MegaMoeConfig


def make_inputs(tokens: int, experts: int, topk: int, hidden: int, inter: int, seed: int, device) -> dict:
    gen = torch.Generator(device=device).manual_seed(seed)
    u8 = torch.uint8

    def codes(*shape):
        return torch.randint(0, 256, shape, dtype=u8, device=device, generator=gen)

    def scales(center, *shape):
        return torch.randint(center - 2, center + 3, shape, dtype=u8, device=device, generator=gen)

    values = {}
    x = (torch.randn((tokens, hidden), device=device, generator=gen) * 50.0).clamp(-448.0, 448.0)
    values["x"] = x.to(torch.float8_e4m3fn)
    values["x_scales"] = scales(120, tokens, hidden // 32)
    popularity = 0.4 * torch.randn((experts,), device=device, generator=gen)
    uniform = torch.rand((tokens, experts), device=device, generator=gen).clamp(1e-12, 1 - 1e-7)
    values["topk_idx"] = (popularity - torch.log(-torch.log(uniform))).topk(topk, -1).indices
    score = torch.nn.functional.softplus(torch.randn((tokens, topk), device=device, generator=gen)).sqrt()
    values["topk_weights"] = score / score.sum(-1, keepdim=True) * 2.5
    values["l1_blocks"] = codes(experts, 2 * inter, hidden // 32, 16)
    values["l1_scales"] = scales(120, experts, 2 * inter, hidden // 32)
    values["l2_blocks"] = codes(experts, hidden, inter // 32, 16)
    values["l2_scales"] = scales(121, experts, hidden, inter // 32)
    return values


def measured_hbm_peak() -> tuple[float, str]:
    path = Path(__file__).resolve().parent.parent / "MEASURED_PEAKS.json"
    if path.exists():
        return float(json.loads(path.read_text())["hbm_gbs"]), "of measured"
    return 6650.0, "of fallback"


def measure(tokens: int, experts: int = 384, topk: int = 6, hidden: int = 7168, inter: int = 3072, steps: int = 10,
            warmup: int = 3, seed: int = 0, device=None, flush: torch.Tensor | None = None) -> dict:
    """One measurement as a dict (the JSON line of ``main``)."""
    device = torch.device(device if device is not None else "cuda:0")
    values = make_inputs(tokens, experts, topk, hidden, inter, seed, device)
    layer = MegaMoe(MegaMoeConfig(hidden, inter, experts, topk, 10.0), max_tokens=tokens, device=device)
    if flush is None:
        flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=device)
    for _ in range(warmup):
        flush_l2(flush)
        layer.run(values, check_status=True)
    torch.cuda.synchronize(device)
    times = []
    for _ in range(steps):
        flush_l2(flush)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        layer.run(values)
        b.record()
        torch.cuda.synchronize(device)
        times.append(a.elapsed_time(b) * 1e3)
    layer.run(values, check_status=True)
    times.sort()
    median = times[len(times) // 2]
    hit = int(torch.unique(values["topk_idx"]).numel())
    rows = tokens * topk
    per_expert = 3 * hidden * inter // 2 + 3 * hidden * inter // 32       # codes + scales
    algorithmic = hit * per_expert + rows * (hidden + hidden // 32) * 2 + rows * (inter + inter // 32) * 2
    flops = 2.0 * rows * 3 * hidden * inter
    peak, kind = measured_hbm_peak()
    gbs = algorithmic / median / 1e3
    return {
        "metric": "MXFP4 MegaMoE routed experts latency", "value": round(median, 2), "unit": "us",
        "min_us": round(times[0], 2), "steps": steps, "warmup": warmup,
        "config": {"workload": f"megamoe-layer-deepseek-v4-pro shape, all experts on one GPU: T={tokens} "
                               f"E={experts} top{topk} H={hidden} I={inter}",
                   "l2": "flushed before every step", "data": "synthetic"},
        "experts_hit": hit, "routed_rows": rows, "algorithmic_bytes": algorithmic,
        "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": peak, "unit": "GB/s", "frac": round(gbs / peak, 4),
                     "peak_kind": kind},
        "tflops": round(flops / median / 1e6, 1), "dtype": "mxfp4 x e4m3 -> f32",
    }


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=512)
    ap.add_argument("--experts", type=int, default=384)
    ap.add_argument("--topk", type=int, default=6)
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--inter", type=int, default=3072)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--seed", type=int, default=0)
    args = ap.parse_args()
    torch.cuda.set_device(0)
    print(json.dumps(measure(args.tokens, args.experts, args.topk, args.hidden, args.inter, args.steps, args.warmup,
                             args.seed)))


if __name__ == "__main__":
    main()
