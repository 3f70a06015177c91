"""Layer geometries and seeded synthetic inputs for the FP8 MoE decode layer.

The five geometries are the ones the benchmark is quoted on. Inputs follow the
reference's convention of naming every tensor and deriving an independent
generator seed from (seed, tensor name, row block), so that a rank's shard is a
slice of the single-rank problem (megabench/tasks/distributed.py:25-47,
megabench/tests/test_megamoe.py:150-158). Tensor names and layouts are the
MoE-block names of megabench/tasks/frontier.py:157-176 without the layer prefix.

Weights are quantised here, at generation time, to e4m3 with one fp32 scale per
128x128 block (scale = max(amax, 1e-4) / 448), which is how a checkpoint would
store them; this is input preparation, not part of the timed layer.
"""

from __future__ import annotations

import hashlib
from dataclasses import dataclass, asdict

import torch

ROW_BLOCK = 128
FP8_MAX = 448.0


@dataclass(frozen=True)
class MoeGeometry:
    name: str
    hidden: int
    inter: int
    experts: int
    topk: int
    shared: int            # shared experts (0 or 1)
    scoring: str           # "sigmoid" | "softmax" | "sqrt_softplus" | "softmax_biased"
    n_group: int
    topk_group: int
    scaling: float
    weight_std: float = 0.02
    router_std: float = 0.01
    bias_kind: str = "none"   # "none" | "normal" | "zipf"
    bias_std: float = 0.01
    zipf_c: float = 0.5
    zipf_s: float = 1.1

    def to_dict(self) -> dict:
        return asdict(self)

    def expert_bytes(self) -> int:
        """Bytes of one expert's payload and block scales (what a layer call must stream)."""
        h, i = self.hidden, self.inter
        cb = lambda v: -(-v // 128)
        return 3 * i * h + 4 * (cb(2 * i) * cb(h) + cb(h) * cb(i))


GEOMETRIES = {
    "tiny": MoeGeometry("tiny", 1024, 512, 16, 4, 1, "softmax", 1, 1, 1.0),
    "deepseek_v3": MoeGeometry("deepseek_v3", 7168, 2048, 256, 8, 1, "sigmoid", 8, 4, 2.5,
                               bias_kind="normal"),
    "kimi_k2": MoeGeometry("kimi_k2", 7168, 2048, 384, 8, 1, "sigmoid", 1, 1, 2.827,
                           router_std=7168 ** -0.5, bias_kind="zipf"),
    "qwen3_30b_a3b": MoeGeometry("qwen3_30b_a3b", 2048, 768, 128, 8, 0, "softmax", 1, 1, 1.0),
    "mixtral_8x7b": MoeGeometry("mixtral_8x7b", 4096, 14336, 8, 2, 0, "softmax", 1, 1, 1.0),
}

BATCHES = {
    "tiny": (4,),
    "deepseek_v3": (1, 8, 32, 64, 128),
    "kimi_k2": (64, 256, 1024),
    "qwen3_30b_a3b": (1, 2, 4, 8, 16, 32, 64, 128, 256, 512),
    "mixtral_8x7b": (1, 16, 128, 2048),
}


def seed_of(seed: int, name: str) -> int:
    digest = hashlib.blake2b(f"moe-b200/{seed}/{name}".encode(), digest_size=8).digest()
    return int.from_bytes(digest, "little") & ((1 << 63) - 1)


def _normal(seed: int, name: str, shape, std: float, device) -> torch.Tensor:
    gen = torch.Generator(device=device).manual_seed(seed_of(seed, name))
    return torch.randn(shape, generator=gen, device=device, dtype=torch.float32) * std


def normal_rows(seed: int, name: str, rows: int, cols: int, std: float, device,
                row_range: tuple[int, int] | None = None) -> torch.Tensor:
    """fp32 rows [r0, r1) of a canonical [rows, cols] matrix sampled in 128-row blocks."""
    r0, r1 = row_range or (0, rows)
    out = torch.empty((r1 - r0, cols), device=device, dtype=torch.float32)
    for start in range(r0 // ROW_BLOCK * ROW_BLOCK, r1, ROW_BLOCK):
        end = min(start + ROW_BLOCK, rows)
        block = _normal(seed, f"{name}:{start}", (end - start, cols), std, device)
        lo, hi = max(start, r0), min(end, r1)
        out[lo - r0:hi - r0] = block[lo - start:hi - start]
    return out


def block_quantize_weight(w: torch.Tensor):
    """e4m3 payload + fp32 scale per 128x128 block of a [R, C] fp32 matrix (R, C multiples of 128)."""
    r, c = w.shape
    if r % 128 or c % 128:
        raise ValueError("weight dimensions must be multiples of 128")
    blocks = w.reshape(r // 128, 128, c // 128, 128)
    amax = blocks.abs().amax(dim=(1, 3))
    scale = torch.clamp(amax, min=1e-4) / FP8_MAX
    q = torch.clamp(blocks / scale[:, None, :, None], -FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q.reshape(r, c), scale


def fp8_matrix(seed: int, name: str, rows: int, cols: int, std: float, device):
    return block_quantize_weight(_normal(seed, name, (rows, cols), std, device))


def router_bias(geo: MoeGeometry, seed: int, device) -> torch.Tensor | None:
    if geo.bias_kind == "none":
        return torch.zeros(geo.experts, device=device, dtype=torch.float32) if geo.scoring != "softmax" else None
    if geo.bias_kind == "normal":
        return _normal(seed, "router_bias", (geo.experts,), geo.bias_std, device)
    if geo.bias_kind == "zipf":
        gen = torch.Generator(device="cpu").manual_seed(seed_of(seed, "zipf_rank"))
        rank = torch.randperm(geo.experts, generator=gen).to(torch.float32) + 1.0
        return (geo.zipf_c * rank ** (-geo.zipf_s)).to(device)
    raise ValueError(geo.bias_kind)


def make_inputs(geo: MoeGeometry, tokens: int, seed: int, device, *, rank: int = 0, world: int = 1,
                experts: range | None = None) -> dict[str, torch.Tensor]:
    """Inputs of one rank: its ``tokens`` rows of x (global rows rank*tokens...), the replicated
    router / bias / shared expert, and its contiguous slice of routed experts.

    ``experts`` overrides which routed experts are materialised (used by tests that only need
    the experts a routing actually hits); tensors then hold those experts in the given order.
    """
    if geo.experts % world:
        raise ValueError("experts must divide the number of ranks")
    h, i = geo.hidden, geo.inter
    total = tokens * world
    local = geo.experts // world
    mine = experts if experts is not None else range(rank * local, (rank + 1) * local)
    out: dict[str, torch.Tensor] = {}
    out["x"] = normal_rows(seed, "x", total, h, 1.0, device,
                           row_range=(rank * tokens, (rank + 1) * tokens)).to(torch.bfloat16)
    out["router"] = normal_rows(seed, "router", geo.experts, h, geo.router_std, device)
    bias = router_bias(geo, seed, device)
    if bias is not None:
        out["router_bias"] = bias
    n = len(mine)
    for name, r, c in (("gate", i, h), ("up", i, h), ("down", h, i)):
        payload = torch.empty((n, r, c), device=device, dtype=torch.float8_e4m3fn)
        scales = torch.empty((n, r // 128, c // 128), device=device, dtype=torch.float32)
        for k, e in enumerate(mine):
            payload[k], scales[k] = fp8_matrix(seed, f"{name}:{e}", r, c, geo.weight_std, device)
        out[name], out[name + "_scale"] = payload, scales
    if geo.shared:
        for name, r, c in (("shared_gate", i, h), ("shared_up", i, h), ("shared_down", h, i)):
            out[name], out[name + "_scale"] = fp8_matrix(seed, name, r, c, geo.weight_std, device)
    return out


def algorithmic_bytes(geo: MoeGeometry, tokens: int, distinct_experts: int) -> int:
    """Bytes a layer call has to move: payload and scales of every expert that is hit (plus the
    shared expert), the fp32 router, x in and y out. Scratch and requantised intermediates are
    not counted (megabench/sol.py:160-188 counts weights the same way)."""
    return ((distinct_experts + geo.shared) * geo.expert_bytes()
            + 4 * geo.experts * geo.hidden + 4 * tokens * geo.hidden)


def megamoe_inputs(tokens: int, experts: int, topk: int, hidden: int, inter: int, seed: int, device) -> dict:
    """Seeded random inputs of the routed experts in the MegaMoE-native formats, made on ``device``
    (tensor names and layouts of megabench/tasks/megamoe.py:86-113): packed E2M1 weight bytes with E8M0
    scales near 2^-7, E4M3 rows with scales near 2^-7, routing drawn like the reference's ``route``
    (log-normal expert popularity, Gumbel top-k, weights that sum to 2.5; megabench/tasks/megamoe.py:65-80)."""
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


def kimi_latent_inputs(tokens: int, experts: int, topk: int, hidden: int, latent: int, inter: int, shared: int, seed: int,
                       device) -> tuple[dict, torch.Tensor]:
    """Seeded random inputs of the Kimi-K3 latent MoE block made on ``device``: (values, normalized).
    Tensor names, layouts and scales follow megabench/tasks/kimi_layer.py:107-125 (dense matrices bf16
    ~N(0, 1/fan_in), router logits of unit variance, a small selection bias); the MXFP4 expert matrices
    are random codes with E8M0 scales around the value that gives them the same spread."""
    import math
    gen = torch.Generator(device=device).manual_seed(seed)
    bf = torch.bfloat16

    def dense(rows, cols, fan_in):
        return (torch.randn((rows, cols), device=device, generator=gen) * fan_in ** -0.5).to(bf)

    def mx(rows, cols):
        center = 127 + round(math.log2(cols ** -0.5 / 2.9))       # E2M1 codes have an rms of about 2.9
        blocks = torch.randint(0, 256, (experts, rows, cols // 32, 16), dtype=torch.uint8, device=device, generator=gen)
        scales = torch.randint(center - 1, center + 2, (experts, rows, cols // 32), dtype=torch.uint8, device=device, generator=gen)
        return blocks, scales

    values = {"router": dense(experts, hidden, hidden),
              "router_bias": torch.randn((experts,), device=device, generator=gen) * 0.1,
              "latent_down": dense(latent, hidden, hidden), "latent_up": dense(hidden, latent, latent),
              "latent_norm": (torch.randn((latent,), device=device, generator=gen) / 10 + 1).to(bf),
              "shared_gate": dense(shared * inter, hidden, hidden), "shared_up": dense(shared * inter, hidden, hidden),
              "shared_down": dense(hidden, shared * inter, shared * inter)}
    for name, rows, cols in (("gate", inter, latent), ("up", inter, latent), ("down", latent, inter)):
        values[name + "_blocks"], values[name + "_scales"] = mx(rows, cols)
    normalized = torch.randn((tokens, hidden), device=device, generator=gen).to(bf)
    return values, normalized
