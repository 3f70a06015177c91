"""Latency of the routed experts in the MegaMoE-native formats on one GPU.

    python bench_megamoe.py --tokens 512 --steps 10 --warmup 3

Geometry: the reference's ``megamoe-layer-deepseek-v4-pro`` cases (megabench/cases.py:380-388: 384
experts, top-6, hidden 7168, intermediate 3072), every expert on this GPU (its ``serial`` form).
Inputs are seeded random codes in the right formats, made on the device (``synthetic.megamoe_inputs``).
Timing: CUDA events on the current stream for every call, the L2 flushed before each step; prints
one JSON line with the median latency, the bytes of the experts that were hit, and the fraction of the
measured copy bandwidth that they stand for.
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
from vibe_megakernel_b200.megamoe import MegaMoe, MegaMoeConfig  # noqa: E402
from vibe_megakernel_b200.synthetic import megamoe_inputs as make_inputs  # noqa: E402


def measured_hbm_peak() -> tuple[float, str]:
    path = ROOT / "MEASURED_PEAKS.json"
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
