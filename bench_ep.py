"""Benchmark arm for N > 1 GPUs: the same layer, experts sharded over the ranks, the batch split evenly.

Launched by ``python -m torch.distributed.run --nproc-per-node N bench.py --gpus N ...``: one process
per GPU. Total work is fixed as N grows (strong scaling): every rank holds E/N experts and batch/N
tokens. Timing: barrier + synchronize, K steps each bracketed by CUDA events on the rank's stream with
an L2 flush before it, synchronize + barrier; a rank's time is the mean of its step times and the
reported latency is the maximum over ranks.

Two exchanges are timed on the same inputs: the product path (rows stored into the owner's memory by
the dispatching kernel, bounded flag waits, no collective call) and the reference's host-driven
NCCL all-to-all around the same kernels (``ep_collective``), at the headline batch and over the
configuration's batch sweep.
"""

from __future__ import annotations

import os
import time

import torch
import torch.distributed as dist

from vibe_megakernel_b200 import synthetic
from vibe_megakernel_b200.ep import EpMoeLayer
from vibe_megakernel_b200.ep_collective import EpCollectiveLayer
from vibe_megakernel_b200.layer import LayerConfig

L2_FLUSH_BYTES = 512 << 20


def _reduce(value: float, op) -> float:
    t = torch.tensor([value], dtype=torch.float64)
    dist.all_reduce(t, op=op)       # CPU tensor: carried by Gloo
    return float(t[0])


def flush_l2(buf: torch.Tensor) -> None:
    """Evict the L2: write a buffer four times its size, then read it back, so that the cache is
    left holding clean lines (after the write alone the timed region would also pay for writing
    126 MB of dirty lines back to HBM, which is 5 % of a small layer call and none of its work)."""
    buf.zero_()
    buf.view(torch.int64).sum()


def _timed(fn, steps: int, warmup: int, flush: torch.Tensor, median: bool = False) -> float:
    """Mean (or median) step time in ms, maximum over ranks."""
    for _ in range(warmup):
        flush_l2(flush)
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    pairs = []
    for _ in range(steps):
        flush_l2(flush)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        pairs.append((a, b))
    torch.cuda.synchronize()
    dist.barrier()
    times = sorted(a.elapsed_time(b) for a, b in pairs)
    mine = times[len(times) // 2] if median else sum(times) / steps
    return _reduce(mine, dist.ReduceOp.MAX)


def one_gpu_result(geo, config, args, batch: int, dev) -> torch.Tensor:
    """The whole batch through the one-GPU layer on this GPU (every expert generated here)."""
    from vibe_megakernel_b200.layer import MoeLayer
    full = synthetic.make_inputs(geo, batch, args.seed, dev)
    out = MoeLayer(config, max_tokens=batch, device=dev).forward(full, check_status=True)
    y = out["y"].cpu()
    del full, out
    torch.cuda.empty_cache()
    return y


def run(args, geo, metric: str, peak: float, peak_kind: str, clock_sampler, config_line: dict) -> dict | None:
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", str(args.gpus)))
    local_rank = int(os.environ.get("LOCAL_RANK", str(rank)))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} needs {args.gpus} ranks (torch.distributed.run), got WORLD_SIZE={world}")
    if args.batch % world or geo.experts % world:
        raise SystemExit("batch and experts must divide the number of GPUs")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    # Gloo carries set-up objects and the max-over-ranks; NCCL is only used by the comparison arm.
    dist.init_process_group("cpu:gloo,cuda:nccl", device_id=dev)
    config = LayerConfig.from_geometry(geo)
    batches = [args.batch] if args.no_sweep else sorted(
        {b for b in synthetic.BATCHES[args.config] if b % world == 0 and b >= world} | {args.batch})
    t0 = time.time()
    values = synthetic.make_inputs(geo, max(batches) // world, args.seed, dev, rank=rank, world=world)
    torch.cuda.synchronize()
    gen_s = time.time() - t0
    flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=dev)
    local = geo.experts // world

    def measure(batch: int, steps: int, warmup: int, full: bool):
        tokens = batch // world
        inputs = dict(values)
        # this rank's rows of THIS batch (global rows rank*tokens..): what the one-GPU run of the same batch sees
        inputs["x"] = synthetic.normal_rows(args.seed, "x", batch, geo.hidden, 1.0, dev,
                                            row_range=(rank * tokens, (rank + 1) * tokens)).to(torch.bfloat16)
        layer = EpMoeLayer(config, max_tokens=tokens, device=dev)
        out = layer.forward(inputs, check_status=True)
        ids_all = [None] * world
        dist.all_gather_object(ids_all, out["expert_ids"].cpu())
        ids_all = torch.cat(ids_all)
        mine_hit = int(torch.unique(ids_all[(ids_all >= rank * local) & (ids_all < (rank + 1) * local)]).numel())
        rank_bytes = (mine_hit + geo.shared) * geo.expert_bytes() + 4 * geo.experts * geo.hidden + 4 * tokens * geo.hidden
        busiest = _reduce(float(rank_bytes), dist.ReduceOp.MAX)
        ms = _timed(lambda: layer.forward(inputs), steps, warmup, flush)
        layer.check_device_status()
        res = {"batch": batch, "tokens_per_gpu": tokens, "peer_store_us": round(ms * 1e3, 2),
               "distinct_experts": int(torch.unique(ids_all).numel()), "busiest_rank_bytes": int(busiest),
               "busiest_rank_gbs": round(busiest / (ms * 1e-3) / 1e9, 1)}
        extra = None
        launches = layer.launches()
        if full:
            # end to end through the plugin file, as the reference's harness would drive it: build(case)
            # with the execution context of this rank, x from pinned host memory, y back to it
            from vibe_megakernel_b200 import submission
            case = {"id": f"fp8-moe-layer-{geo.name}-ep{world}-b{batch}", "family": "fp8_moe_layer", "model": geo.name,
                    "phase": "moe_layer", "gpus": world, "tp": 1, "ep": world,
                    "params": {"tokens": tokens, "hidden": geo.hidden, "intermediate": geo.inter, "experts": geo.experts,
                               "topk": geo.topk, "shared_experts": geo.shared, "router_groups": geo.n_group,
                               "router_top_groups": geo.topk_group},
                    "moe": {"scoring": geo.scoring, "scaling": geo.scaling},
                    "execution": {"rank": rank, "world_size": world, "tp_rank": 0, "ep_rank": rank, "backend": dist.get_backend(),
                                  "device": str(dev), "tp_group": None, "ep_group": None}}
            plugin = submission.build(case)
            x_host = inputs["x"].cpu().pin_memory()
            y_host = torch.empty_like(x_host).pin_memory()
            x_dev = torch.empty_like(inputs["x"])
            e2e_inputs = dict(inputs)
            e2e_inputs["x"] = x_dev

            def e2e_step():
                x_dev.copy_(x_host, non_blocking=True)
                y_host.copy_(plugin(e2e_inputs)["y"], non_blocking=True)

            e2e_ms = _timed(e2e_step, steps, warmup, flush)
            same = bool(torch.equal(y_host, out["y"].cpu()))
            plugin.layer.close()
            # correctness across GPUs at full geometry: rank 0 runs the whole batch on one GPU
            ys = [None] * world
            dist.all_gather_object(ys, out["y"].cpu())
            equal_one_gpu, differing = None, None
            if rank == 0:
                alone = one_gpu_result(geo, config, args, batch, dev)
                together = torch.cat(ys)
                equal_one_gpu = bool(torch.equal(together, alone))
                gap = (together.float() - alone.float()).abs()
                differing = {"elements": int((gap > 0).sum()), "rows": int((gap > 0).any(1).sum()), "max_abs": float(gap.max())}
            extra = {"e2e_us": e2e_ms * 1e3, "io_bytes": _reduce(float(x_host.numel() * 2), dist.ReduceOp.SUM),
                     "agree": _reduce(1.0 if same else 0.0, dist.ReduceOp.SUM) == world, "busiest": busiest, "ms": ms,
                     "equal_one_gpu": equal_one_gpu, "differing": differing, "launches": launches}
            dist.barrier()
        layer.close()
        collective = EpCollectiveLayer(config, max_tokens=tokens, device=dev)
        alt = collective.forward(inputs)
        res["collective_equals_peer_store"] = _reduce(1.0 if torch.equal(alt["y"], out["y"]) else 0.0,
                                                      dist.ReduceOp.SUM) == world
        res["nccl_all_to_all_us"] = round(_timed(lambda: collective.forward(inputs), max(steps, 20), warmup, flush,
                                                 median=True) * 1e3, 2)       # median of >= 20: the host-driven arm is noisy
        return res, extra

    sweep = []
    with clock_sampler(local_rank) as clocks:
        head, extra = measure(args.batch, args.steps, args.warmup, True)
        for b in batches:
            sweep.append(head if b == args.batch else measure(b, max(5, args.steps // 2), 3, False)[0])
    line = None
    if rank == 0:
        latency_us = extra["ms"] * 1e3
        achieved = extra["busiest"] / (latency_us * 1e-6) / 1e9
        line = {
            "metric": metric, "value": round(latency_us, 2), "unit": "us", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(extra["ms"], 5), "higher_is_better": False, "scaling": "strong",
            "vs_baseline": None, "dtype": "fp8_e4m3 (fp32 accumulate)", "data": "synthetic",
            "config": config_line,
            "protocol": {"parallelism": f"expert parallel over {world} GPUs: {args.batch // world} tokens and {local} experts per GPU",
                         "exchange": "in-kernel peer stores over NVLink, bounded flag waits, no NCCL call per layer",
                         "l2": "flushed between steps (512 MiB write, then read back: no dirty lines left)",
                         "e2e_io": "x bf16 host->device and y bf16 device->host per step on every rank, through the plugin "
                                   "file's build(case with execution) -> run(inputs); weights resident in HBM",
                         "input_generation_s": round(gen_s, 1)},
            "e2e": {"value": round(extra["e2e_us"], 2), "unit": "us", "h2d_bytes_per_step": int(extra["io_bytes"]),
                    "d2h_bytes_per_step": int(extra["io_bytes"]), "plugin_path_equals_direct_path": extra["agree"]},
            "ep_equals_one_gpu": extra["equal_one_gpu"], "ep_vs_one_gpu_differing": extra["differing"],
            "gpu_launches": extra["launches"] * args.steps * world, "launches_per_step_per_gpu": extra["launches"],
            "clocks": clocks.summary(),
            "roofline": {"bound": "hbm", "kernel": "whole layer on the busiest rank (weights of the experts it is hit on)",
                         "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s", "frac": round(achieved / peak, 4),
                         "peak_kind": f"of {peak_kind}", "traffic": None,
                         "algorithmic_bytes_per_launch": int(extra["busiest"])},
            "exchange_comparison": sweep,
        }
    dist.barrier()
    dist.destroy_process_group()
    return line
