"""Plugin file for the reference harness: ``build(case) -> run(inputs) -> outputs``.

Protocol: megabench/README.md:83-104 and megabench/harness/runner.py:69-87. ``case`` is the
harness' case dict; the layer geometry is read from ``case["params"]`` (integers, as the
reference's Case admits) with the non-integer knobs in ``case["moe"]``:

    params: hidden, intermediate, experts, topk, shared_experts, router_groups, router_top_groups,
            swiglu_limit (the clamp of megabench/tasks/megamoe.py:43-44,116-122; absent or 0 = none)
    moe:    {"scoring": "sigmoid"|"softmax"|"sqrt_softplus"|"softmax_biased", "scaling": float,
             "weight_before_requant": bool (routing weight inside SwiGLU, megamoe.py:122,176-182)}

``run`` takes the tensors named in megabench/tasks/frontier.py:157-176 (without the layer prefix)
and returns ``y`` (bf16 [T, H]), ``expert_ids`` (int64 [T, topk], choice order) and ``order``
(int64 [T*topk], the stable expert grouping of the flattened ids). Inputs are not modified; all
work is enqueued on the current torch stream.
"""

from __future__ import annotations

import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

from vibe_megakernel_b200.layer import LayerConfig, MoeLayer  # noqa: E402


def build(case: dict):
    p = case["params"]
    extra = case.get("moe", {})
    config = LayerConfig(hidden=p["hidden"], inter=p["intermediate"], experts=p["experts"], topk=p["topk"],
                         shared=p.get("shared_experts", 0), scoring=extra.get("scoring", "sigmoid"),
                         n_group=p.get("router_groups", 1), topk_group=p.get("router_top_groups", 1),
                         scaling=float(extra.get("scaling", 1.0)), swiglu_limit=float(p.get("swiglu_limit", 0.0)),
                         weight_before_requant=bool(extra.get("weight_before_requant", False)))
    if case.get("gpus", 1) != 1:
        raise NotImplementedError("expert-parallel execution is built through vibe_megakernel_b200.ep")
    layer = MoeLayer(config, max_tokens=p.get("tokens", p.get("batch", 1)))

    def run(inputs: dict):
        out = layer.forward(inputs)
        return {"y": out["y"], "expert_ids": out["expert_ids"], "order": out["order"]}

    return run
