"""Latency of the routed experts in the MegaMoE-native formats on one GPU.

    python bench_megamoe.py --tokens 512 --steps 10 --warmup 3
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 bench_megamoe.py --tokens 512   # expert parallel

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


def rank_inputs(tokens: int, experts: int, topk: int, hidden: int, inter: int, seed: int, rank: int, world: int, device) -> dict:
    """Inputs of one rank of an expert-parallel run: its own token rows with global routing, and the
    matrices of its experts [rank*E/world, (rank+1)*E/world). Deterministic per (seed, rank), so that
    another rank can rebuild them."""
    local = experts // world
    mine = make_inputs(tokens, experts, topk, hidden, inter, seed * 1000 + rank, device)
    own = make_inputs(1, local, min(topk, local), hidden, inter, seed * 1000 + 500 + rank, device)
    for key in ("l1_blocks", "l1_scales", "l2_blocks", "l2_scales"):
        mine[key] = own[key]
    return mine


def measure_ep(tokens: int, experts: int = 384, topk: int = 6, hidden: int = 7168, inter: int = 3072, steps: int = 10,
               warmup: int = 3, seed: int = 0) -> dict | None:
    """The expert-parallel form on all ranks of the job (one process per GPU, launched by
    torch.distributed.run): ``tokens`` rows per rank, experts split contiguously, rows exchanged as peer
    stores by the kernels. The reference's cases: megabench/cases.py:380-388 (8 ranks, 512 and 4096 tokens
    per rank). Latency = median over steps of the slowest rank."""
    import os
    import torch.distributed as dist
    from vibe_megakernel_b200.megamoe import MegaMoeEp
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local_rank = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist.init_process_group("cpu:gloo,cuda:nccl", device_id=device)
    values = rank_inputs(tokens, experts, topk, hidden, inter, seed, rank, world, device)
    config = MegaMoeConfig(hidden, inter, experts, topk, 10.0)
    layer = MegaMoeEp(config, max_tokens=tokens, device=device)
    flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=device)
    out = None
    for _ in range(warmup):
        flush_l2(flush)
        out = layer.run(values, check_status=True)
    torch.cuda.synchronize(device)
    dist.barrier()
    pairs = []
    for _ in range(steps):
        flush_l2(flush)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        layer.run(values)
        b.record()
        pairs.append((a, b))
    torch.cuda.synchronize(device)
    dist.barrier()
    mine = torch.tensor([a.elapsed_time(b) * 1e3 for a, b in pairs], dtype=torch.float64)
    dist.all_reduce(mine, op=dist.ReduceOp.MAX)          # per step, the slowest rank
    median = float(mine.sort().values[steps // 2])
    launches = layer.launches()
    # expert parallel == serial at this size: rank 0 rebuilds the whole problem and runs it on one GPU
    ys, idx = [None] * world, [None] * world
    dist.all_gather_object(ys, out["y"].cpu())
    dist.all_gather_object(idx, values["topk_idx"].cpu())
    hit_local = torch.unique(torch.cat(idx))
    busiest = max(int(((hit_local >= r * (experts // world)) & (hit_local < (r + 1) * (experts // world))).sum()) for r in range(world))
    equal = None
    if rank == 0 and tokens * world * topk <= 32768:
        parts = [rank_inputs(tokens, experts, topk, hidden, inter, seed, r, world, device) for r in range(world)]
        full = {k: torch.cat([p[k] for p in parts]) for k in parts[0]}
        del parts
        serial = MegaMoe(config, max_tokens=tokens * world, device=device).run(full, check_status=True)["y"].cpu()
        equal = bool(torch.equal(torch.cat(ys), serial))
    dist.barrier()
    layer.close()
    line = None
    if rank == 0:
        per_expert = 3 * hidden * inter // 2 + 3 * hidden * inter // 32
        peak, kind = measured_hbm_peak()
        rows = tokens * world * topk
        line = {"metric": "MXFP4 MegaMoE routed experts latency (expert parallel)", "value": round(median, 2), "unit": "us",
                "n_gpus": world, "steps": steps, "warmup": warmup,
                "config": {"workload": f"megamoe-layer-deepseek-v4-pro-ep{world}-t{tokens}: T={tokens} per rank, E={experts} top{topk} "
                                       f"H={hidden} I={inter}", "l2": "flushed before every step", "data": "synthetic",
                           "exchange": "in-kernel peer stores over NVLink, no NCCL call per layer"},
                "ep_equals_serial": equal, "launches_per_step_per_gpu": launches,
                "busiest_rank_experts_hit": busiest,
                "roofline": {"bound": "hbm", "achieved": round(busiest * per_expert / median / 1e3, 1), "peak": peak, "unit": "GB/s",
                             "frac": round(busiest * per_expert / median / 1e3 / peak, 4), "peak_kind": kind,
                             "what": "MXFP4 bytes of the experts hit on the busiest rank / latency"},
                "tflops": round(2.0 * rows * 3 * hidden * inter / median / 1e6, 1),
                "reference_floor_ms": {512: 0.212, 4096: 0.722}.get(tokens),       # megabench/sol.py:160-188
                "dtype": "mxfp4 x e4m3 -> f32"}
    dist.destroy_process_group()
    return line


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
    import os
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:       # launched by torch.distributed.run: the expert-parallel form
        line = measure_ep(args.tokens, args.experts, args.topk, args.hidden, args.inter, args.steps, args.warmup, args.seed)
        if line is not None:
            print(json.dumps(line), flush=True)
        return
    torch.cuda.set_device(0)
    print(json.dumps(measure(args.tokens, args.experts, args.topk, args.hidden, args.inter, args.steps, args.warmup,
                             args.seed)))


if __name__ == "__main__":
    main()
