"""Benchmark of the FP8 MoE decode layer.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--config deepseek_v3] [--batch 64] [--no-sweep]

A step is one layer call over one batch of seeded synthetic tokens (weights and activations
follow the benchmark's distributions; there is no dataset). One JSON line is printed by rank 0.

  value        layer latency in microseconds, inputs resident in HBM, CUDA events per step,
               L2 flushed between steps (max over ranks when N > 1)
  e2e          the same call through the plugin API with x in pinned host memory: host->device
               copy of x, layer, device->host copy of y, all inside the timed region
  roofline     the gate/up grouped GEMM kernel: algorithmic bytes / its event-timed duration
  cpu_baseline the CPU oracle (a port of the reference's Python) on the host cores, bounded sample
  sweep        latency / achieved GB/s for the other batch sizes of the configuration

`--impl reference` times the CPU oracle alone (the reference has no implementation of this path
other than its PyTorch code, which the oracle restates) with all host threads.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

from vibe_megakernel_b200 import synthetic  # noqa: E402

METRIC = "fp8_moe_decode_layer_latency_us"
L2_FLUSH_BYTES = 512 << 20


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--config", default="deepseek_v3", choices=sorted(synthetic.GEOMETRIES))
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--no-sweep", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--experts", type=int, default=0, help="shrink the routed expert count (profiling captures only)")
    ap.add_argument("--expert-load", action="store_true",
                    help="print the per-expert load of --config at --batch under the GPU router, and exit")
    return ap.parse_args()


def geometry_of(args):
    geo = synthetic.GEOMETRIES[args.config]
    if args.experts:
        import dataclasses
        geo = dataclasses.replace(geo, name=f"{geo.name}-e{args.experts}", experts=args.experts)
    return geo


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        d = json.loads(path.read_text())
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.file = None

    def __enter__(self):
        try:
            self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self) -> dict:
        if self.proc is None or self.file is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.file.flush()
        rows = [r.split(",") for r in Path(self.file.name).read_text().splitlines() if r.count(",") >= 6]
        os.unlink(self.file.name)
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm = sorted(float(r[0]) for r in rows)
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = [n for i, n in enumerate(names) if any(r[3 + i].strip() == "Active" for r in rows)]
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": float(rows[0][1]), "samples": len(rows),
                "power_w_max": max(float(r[2]) for r in rows), "reasons": reasons}


def layer_case(geo, tokens: int) -> dict:
    """The case dict the plugin's build() takes (layout of the reference's Case.to_dict())."""
    return {"id": f"fp8-moe-layer-{geo.name}-b{tokens}", "family": "fp8_moe_layer", "model": geo.name,
            "phase": "moe_layer", "gpus": 1, "tp": 1, "ep": 1,
            "params": {"tokens": tokens, "hidden": geo.hidden, "intermediate": geo.inter, "experts": geo.experts,
                       "topk": geo.topk, "shared_experts": geo.shared, "router_groups": geo.n_group,
                       "router_top_groups": geo.topk_group},
            "moe": {"scoring": geo.scoring, "scaling": geo.scaling}}


def timed_steps(fn, steps: int, warmup: int, flush: torch.Tensor, barrier=None) -> list[float]:
    """Per-step device times in ms: L2 is flushed (a 512 MiB write, then read back) before every step,
    outside its events."""
    from bench_ep import flush_l2
    for _ in range(warmup):
        flush_l2(flush)
        fn()
    torch.cuda.synchronize()
    if barrier:
        barrier()
    pairs = []
    for _ in range(steps):
        flush_l2(flush)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        pairs.append((a, b))
    torch.cuda.synchronize()
    if barrier:
        barrier()
    return [a.elapsed_time(b) for a, b in pairs]


def gate_up_bytes(geo, distinct: int) -> int:
    """Algorithmic bytes of one gate/up GEMM launch: payload and block scales of gate and up of every
    expert that is hit (and of the shared expert)."""
    per_expert = 2 * geo.inter * geo.hidden + 8 * (geo.inter // 128) * (geo.hidden // 128)
    return (distinct + geo.shared) * per_expert


# DRAM traffic of one gate/up GEMM launch per unit (one expert hit by the batch), from an ncu capture
# (--set full) of this kernel on a small case of the DeepSeek-V3 geometry (64 routed experts, batch 8):
# dram__bytes_read.sum + dram__bytes_write.sum = 1,322,132,000 + 3,483,392 B for 45 units. Traffic
# grows in proportion to the experts hit, every weight byte being read once.
NCU_GATE_UP_TRAFFIC_PER_UNIT = {(7168, 2048): (1_322_132_000 + 3_483_392) / 45}


def gate_up_traffic(geo, distinct: int):
    per_unit = NCU_GATE_UP_TRAFFIC_PER_UNIT.get((geo.hidden, geo.inter))
    return None if per_unit is None else int(round((distinct + geo.shared) * per_unit))


def workload_config(geo, args) -> dict:
    """The `config` of a bench line: the same dict for the GPU arm and the CPU reference arm."""
    return {"workload": f"{geo.name} FP8 MoE decode layer, batch {args.batch}: H={geo.hidden} I={geo.inter} "
                        f"E={geo.experts}+{geo.shared} top{geo.topk} {geo.scoring}",
            "batch": args.batch, "seed": args.seed}


def oracle_spec(geo):
    from oracle import moe_oracle as O
    return O.LayerSpec(geo.hidden, geo.inter, geo.experts, geo.topk, geo.shared, geo.scoring, geo.n_group,
                       geo.topk_group, geo.scaling)


def host_problem(geo, values: dict, tokens: int):
    """The first ``tokens`` rows of the batch as a CPU problem for the oracle: only the experts those
    tokens hit are copied to the host. Returns (host tensors, expert id -> index map, experts hit)."""
    from oracle import moe_oracle as O
    x = values["x"][:tokens].cpu()
    router = values["router"].cpu()
    bias = values["router_bias"].cpu() if "router_bias" in values else None
    ids, _ = O.route_tokens(oracle_spec(geo), x, router, bias)
    hit = sorted(set(ids.flatten().tolist()))
    slot = {e: k for k, e in enumerate(hit)}
    index = torch.tensor(hit, device=values["gate"].device)
    host = {"x": x, "router": router}
    if bias is not None:
        host["router_bias"] = bias
    for name in ("gate", "up", "down"):
        host[name] = values[name][index].cpu()
        host[name + "_scale"] = values[name + "_scale"][index].cpu()
    for name in values:
        if name.startswith("shared_"):
            host[name] = values[name].cpu()
    return host, slot, len(hit)


def cpu_oracle_passes(geo, values: dict, tokens: int, threads: int, warmup: int, steps: int, budget_s: float):
    """Times whole oracle passes over the first ``tokens`` rows on ``threads`` host threads (the
    reference's arithmetic: whole-matrix dequantisation per expert that is hit, bf16 GEMMs). Stops
    early when ``budget_s`` is spent. Returns (seconds of every timed pass, warm-up passes run, experts hit)."""
    from oracle import moe_oracle as O
    torch.set_num_threads(threads)
    spec = oracle_spec(geo)
    host, slot, hit = host_problem(geo, values, tokens)
    end = time.time() + budget_s
    warm = 0
    for _ in range(warmup):
        O.moe_layer(spec, host, expert_slot=slot)
        warm += 1
        if time.time() > end:
            break
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        O.moe_layer(spec, host, expert_slot=slot)
        times.append(time.perf_counter() - t0)
        if time.time() > end:
            break
    return times, warm, hit


def measure_batch(geo, values: dict, tokens: int, steps: int, warmup: int, flush, peak: float, *, full: bool):
    """Latency, stage times and roofline figures of one batch size on this GPU."""
    from vibe_megakernel_b200 import submission
    from vibe_megakernel_b200.layer import LayerConfig, MoeLayer
    inputs = dict(values)
    inputs["x"] = values["x"][:tokens].contiguous()
    layer = MoeLayer(LayerConfig.from_geometry(geo), max_tokens=tokens)
    out = layer.forward(inputs, check_status=True)
    distinct = int(torch.unique(out["expert_ids"]).numel())
    launches = layer.launches()
    ms = timed_steps(lambda: layer.forward(inputs), steps, warmup, flush)
    layer.check_device_status(tokens)
    latency_us = 1e3 * sum(ms) / len(ms)
    # the same call replayed from a CUDA graph (what a decode loop would do): no launch cost on the host
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        layer.forward(inputs)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        graph_out = layer.forward(inputs)
    graph_ms = timed_steps(graph.replay, max(3, steps // 2), 3, flush)
    assert torch.equal(graph_out["y"], out["y"]), "graph replay and direct call disagree"
    # stage times: separate profiled passes, same inputs and flush protocol
    layer.profile(True)
    stages = {k: 0.0 for k in MoeLayer.STAGES}
    reps = max(3, min(steps, 10))
    from bench_ep import flush_l2
    for _ in range(reps):
        flush_l2(flush)
        layer.forward(inputs)
        for k, v in layer.stage_ms().items():
            stages[k] += v / reps
    layer.profile(False)
    total_bytes = synthetic.algorithmic_bytes(geo, tokens, distinct)
    g_bytes = gate_up_bytes(geo, distinct)
    g_gbs = g_bytes / (stages["gate_up_gemm"] * 1e-3) / 1e9
    res = {"batch": tokens, "latency_us": round(latency_us, 2), "min_us": round(1e3 * min(ms), 2),
           "p50_us": round(1e3 * sorted(ms)[len(ms) // 2], 2),
           "graph_replay_us": round(1e3 * sum(graph_ms) / len(graph_ms), 2),
           "distinct_experts": distinct, "algorithmic_bytes": total_bytes,
           "layer_gbs": round(total_bytes / (latency_us * 1e-6) / 1e9, 1),
           "layer_frac_of_measured_peak": round(total_bytes / (latency_us * 1e-6) / 1e9 / peak, 4),
           "layer_frac_of_8tbs": round(total_bytes / (latency_us * 1e-6) / 1e9 / 8000.0, 4),
           "stage_us": {k: round(v * 1e3, 2) for k, v in stages.items()},
           "gate_up_gbs": round(g_gbs, 1), "launches": launches}
    if not full:
        return res, None
    # end to end through the plugin API: x starts in pinned host memory, y ends there
    run = submission.build(layer_case(geo, tokens))
    x_host = inputs["x"].cpu().pin_memory()
    y_host = torch.empty_like(x_host).pin_memory()
    x_dev = torch.empty_like(inputs["x"])
    e2e_inputs = dict(inputs)
    e2e_inputs["x"] = x_dev

    def e2e_step():
        x_dev.copy_(x_host, non_blocking=True)
        y_host.copy_(run(e2e_inputs)["y"], non_blocking=True)

    e2e_ms = timed_steps(e2e_step, steps, warmup, flush)
    assert torch.equal(y_host, out["y"].cpu()), "plugin path and direct path disagree"
    # the layer with the step either side of it (RMSNorm in front, residual add behind): one more launch
    gamma = torch.ones(geo.hidden, dtype=torch.bfloat16, device=inputs["x"].device)
    block_ms = timed_steps(lambda: layer.block_forward(inputs, gamma, 1e-6, weight_in_fp32=True),
                           max(3, steps // 2), 3, flush)
    layer.check_device_status(tokens)
    extra = {"ms": ms, "e2e_us": 1e3 * sum(e2e_ms) / len(e2e_ms), "io_bytes": x_host.numel() * 2,
             "gate_up_ms": stages["gate_up_gemm"], "gate_up_bytes": g_bytes, "distinct": distinct,
             "launches": launches, "block_us": 1e3 * sum(block_ms) / len(block_ms)}
    return res, extra


def main_single(args) -> dict:
    geo = geometry_of(args)
    peak, peak_kind = measured_peaks()
    torch.cuda.set_device(0)
    dev = torch.device("cuda:0")
    batches = sorted(set(synthetic.BATCHES[args.config]) | {args.batch})
    t0 = time.time()
    values = synthetic.make_inputs(geo, max(batches), args.seed, dev)
    torch.cuda.synchronize()
    gen_s = time.time() - t0
    flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=dev)
    sweep = []
    with ClockSampler(0) as clocks:      # covers the headline batch and the sweep
        head, extra = measure_batch(geo, values, args.batch, args.steps, args.warmup, flush, peak, full=True)
        if not args.no_sweep:
            for b in batches:
                if b == args.batch:
                    sweep.append(head)
                else:
                    sweep.append(measure_batch(geo, values, b, max(5, args.steps // 2), 3, flush, peak, full=False)[0])
    clock_summary = clocks.summary()
    line = {
        "metric": METRIC, "value": head["latency_us"], "unit": "us", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(head["latency_us"] / 1e3, 5), "higher_is_better": False,
        "scaling": "strong", "vs_baseline": None, "dtype": "fp8_e4m3 (fp32 accumulate)", "data": "synthetic",
        "config": workload_config(geo, args),
        "protocol": {"l2": "flushed between steps (512 MiB write, then read back: no dirty lines left)",
                     "e2e_io": "x bf16 host->device and y bf16 device->host per step; weights resident in HBM",
                     "input_generation_s": round(gen_s, 1)},
        "e2e": {"value": round(extra["e2e_us"], 2), "unit": "us", "h2d_bytes_per_step": extra["io_bytes"],
                "d2h_bytes_per_step": extra["io_bytes"]},
        "gpu_launches": extra["launches"] * args.steps,
        "launches_per_step": extra["launches"],
        "clocks": clock_summary,
        "roofline": {"bound": "hbm", "kernel": "grouped_gemm_kernel<dual> (gate/up GEMM + SwiGLU + requantisation)",
                     "achieved": round(extra["gate_up_bytes"] / (extra["gate_up_ms"] * 1e-3) / 1e9, 1), "peak": peak,
                     "unit": "GB/s", "frac": round(extra["gate_up_bytes"] / (extra["gate_up_ms"] * 1e-3) / 1e9 / peak, 4),
                     "peak_kind": f"of {peak_kind}", "traffic": gate_up_traffic(geo, extra["distinct"]),
                     "traffic_source": "ncu dram bytes of a smaller case of the same kernel, scaled by experts hit",
                     "algorithmic_bytes_per_launch": extra["gate_up_bytes"],
                     "kernel_us": round(extra["gate_up_ms"] * 1e3, 2)},
        "layer": {k: head[k] for k in ("distinct_experts", "algorithmic_bytes", "layer_gbs",
                                       "layer_frac_of_measured_peak", "layer_frac_of_8tbs", "stage_us")},
        "block_with_norm_and_residual_us": round(extra["block_us"], 2),
        "sweep": sweep,
    }
    if not args.no_sweep:
        # The routed experts in the MegaMoE-native formats (MXFP4 weights, E4M3 rows with E8M0 scales;
        # megabench/cases.py:380-388, all 384 experts on this GPU) at decode batch sizes, as extra lines
        # beside the headline: they do not enter `value`.
        import bench_megamoe as megamoe_bench
        line["megamoe_native"] = []
        for tokens in (1, 64):
            m = megamoe_bench.measure(tokens, steps=max(5, args.steps // 2), warmup=3, seed=args.seed, device=dev, flush=flush)
            line["megamoe_native"].append({"tokens": tokens, "latency_us": m["value"], "experts_hit": m["experts_hit"],
                                           "algorithmic_bytes": m["algorithmic_bytes"],
                                           "frac_of_measured_peak": m["roofline"]["frac"], "workload": m["config"]["workload"]})
    if not args.no_cpu_baseline:
        # one whole pass of the CPU oracle over the full batch on all host threads (measured, not
        # scaled), and a one-thread point on the first two tokens scaled by the experts they hit
        threads = os.cpu_count() or 1
        times, _, hit = cpu_oracle_passes(geo, values, args.batch, threads, 0, 1, 120.0)
        line["cpu_baseline"] = {"value": round(times[0] * 1e6, 1), "unit": "us", "cores": threads, "kind": "port",
                                "sample": f"one whole oracle layer pass over the batch of {args.batch} tokens ({hit} routed "
                                          f"experts + {geo.shared} shared, whole-matrix dequantisation per expert as the "
                                          f"reference does), {times[0]:.2f} s, no warm-up pass, not scaled"}
        few = min(2, args.batch)
        one, _, hit_few = cpu_oracle_passes(geo, values, few, 1, 0, 1, 60.0)
        scale = (hit + geo.shared) / (hit_few + geo.shared)
        line["cpu_baseline"]["one_thread"] = {
            "value": round(one[0] * scale * 1e6, 1), "unit": "us", "cores": 1,
            "sample": f"oracle pass over the first {few} token(s) ({hit_few} routed experts + {geo.shared} shared) on one "
                      f"thread, {one[0]:.2f} s, scaled x{scale:.2f} by experts hit to the full batch"}
    return line


def main_reference(args) -> dict | None:
    """The reference's CPU implementation of the path: the oracle port on all host threads, rank 0 only.
    A step is one whole oracle pass over the full batch of the GPU arm's configuration (same inputs:
    they are generated on the GPU when there is one, which takes seconds instead of minutes, and
    copied to the host). Runs --warmup passes and --steps timed passes unless the time budget
    (about four minutes) ends first; the line says how many ran."""
    if int(os.environ.get("RANK", "0")) != 0:
        return None
    geo = geometry_of(args)
    threads = os.cpu_count() or 1
    dev = "cuda:0" if torch.cuda.is_available() else "cpu"
    t0 = time.time()
    x = synthetic.normal_rows(args.seed, "x", args.batch, geo.hidden, 1.0, dev).to(torch.bfloat16)
    router = synthetic.normal_rows(args.seed, "router", geo.experts, geo.hidden, geo.router_std, dev)
    bias = synthetic.router_bias(geo, args.seed, dev)
    from oracle import moe_oracle as O
    ids, _ = O.route_tokens(oracle_spec(geo), x.cpu(), router.cpu(), None if bias is None else bias.cpu())
    hit_ids = sorted(set(ids.flatten().tolist()))
    values = synthetic.make_inputs(geo, args.batch, args.seed, dev, experts=hit_ids)
    # make_inputs holds the hit experts in list order: present them to host_problem as a whole layer
    full = dict(values)
    gen_s = time.time() - t0
    spec = oracle_spec(geo)
    host = {k: v.cpu() for k, v in full.items()}
    slot = {e: k for k, e in enumerate(hit_ids)}
    torch.set_num_threads(threads)
    end = time.time() + 235.0
    warm = 0
    for _ in range(args.warmup):
        O.moe_layer(spec, host, expert_slot=slot)
        warm += 1
        if time.time() > end - 60:
            break
    times = []
    for _ in range(args.steps):
        t1 = time.perf_counter()
        O.moe_layer(spec, host, expert_slot=slot)
        times.append(time.perf_counter() - t1)
        if time.time() > end:
            break
    value = sum(times) / len(times) * 1e6
    what = (f"each step = one whole oracle layer pass over the batch of {args.batch} tokens ({len(hit_ids)} routed experts + "
            f"{geo.shared} shared, whole-matrix dequantisation per expert as the reference does), mean {value / 1e6:.2f} s, "
            f"not scaled; {warm} of {args.warmup} warm-up and {len(times)} of {args.steps} timed passes ran inside the time "
            f"budget; inputs generated on {dev} in {gen_s:.0f} s")
    return {"impl": "reference", "metric": METRIC, "value": round(value, 1), "unit": "us", "n_gpus": args.gpus,
            "steps": len(times), "warmup": warm, "ms_per_step": round(value / 1e3, 3),
            "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "bf16 (fp32 accumulate), CPU",
            "data": "synthetic", "config": workload_config(geo, args),
            "cpu_baseline": {"value": round(value, 1), "unit": "us", "cores": threads, "kind": "port", "sample": what},
            "e2e": {"value": round(value, 1), "unit": "us", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}


def expert_load(args) -> None:
    """How many routed rows each expert receives at --batch (the library's router on cuda:0, whose ids
    are those of the CPU oracle), and the rows each rank owns with the experts split over 2, 4 and 8."""
    from vibe_megakernel_b200.layer import LayerConfig, MoeLayer
    geo = geometry_of(args)
    tokens, seed = args.batch, args.seed
    x = synthetic.normal_rows(seed, "x", tokens, geo.hidden, 1.0, "cuda").to(torch.bfloat16)
    router = synthetic.normal_rows(seed, "router", geo.experts, geo.hidden, geo.router_std, "cuda")
    ids, _ = MoeLayer(LayerConfig.from_geometry(geo), max_tokens=tokens).route(x, router, synthetic.router_bias(geo, seed, "cuda"))
    load = torch.bincount(ids.flatten().cpu(), minlength=geo.experts)
    rows = tokens * geo.topk
    mean = rows / geo.experts
    print(f"{geo.name}, {tokens} tokens, seed {seed}: {rows} routed rows over {geo.experts} experts (mean {mean:.1f})")
    print(f"  experts hit {int((load > 0).sum())}, hottest {int(load.max())} rows ({load.max() / mean:.1f}x mean), "
          f"median {int(load.median())}, coldest {int(load.min())}")
    top = torch.sort(load, descending=True).values
    for share in (1, 5, 10, 25, 50):
        k = max(1, geo.experts * share // 100)
        print(f"  hottest {share:2d} % of the experts ({k:3d}) take {100 * int(top[:k].sum()) / rows:5.1f} % of the rows")
    edges = [0, 1, 2, 4, 8, 16, 32, 64, 128, 256, 1 << 30]
    for lo, hi in zip(edges[:-1], edges[1:]):
        n = int(((load >= lo) & (load < hi)).sum())
        if n:
            print(f"  {lo:4d} <= rows < {hi if hi < (1 << 30) else 'inf':>4}: {n:3d} experts")
    for world in (2, 4, 8):
        if geo.experts % world == 0:
            per = load.reshape(world, -1).sum(1).tolist()
            hit = (load.reshape(world, -1) > 0).sum(1).tolist()
            print(f"  {world} ranks: rows per rank {per}, experts hit per rank {hit}")


def main():
    args = parse_args()
    if args.expert_load:
        expert_load(args)
        return
    if args.impl == "reference":
        line = main_reference(args)
    elif args.gpus == 1:
        line = main_single(args)
    else:
        import bench_ep as ep_bench
        peak, peak_kind = measured_peaks()
        line = ep_bench.run(args, geometry_of(args), METRIC, peak, peak_kind, ClockSampler,
                            workload_config(geometry_of(args), args))
    if line is not None:
        print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
