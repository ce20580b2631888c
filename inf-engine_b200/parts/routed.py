"""A mixture of gated feed-forward experts, chosen and run on the device: a sigmoid router with groups, or (``score``
"softmax_top") the largest logits plus a bias, weighted by the softmax over the chosen logits alone.

Per token, with x the part's input (``RoutedExpertsSpec`` states the rule in full):

    s = sigmoid(router x)                      float32 products and sums
    choice = s + correction                    for the choice only; groups of experts, the best groups kept
    chosen = the ``top`` largest choice scores among the kept groups
    weight = s[chosen] / (sum of them + eps) * route_scale
    out = sum weight_e * down_e(silu(gate_e x) * up_e x)  +  sigmoid(shared_gate x) * shared(x)

The router's product also carries the shared expert's gate (one more row).  Nothing waits for the device: the
(token, choice) pairs are sorted by expert in one small kernel, and two grouped products walk the sorted pairs in
tiles that never span two experts (``csrc/routed.cu``), so the part may sit inside a captured decode step.  A
pair's result does not depend on where it lands in the sorted order, nor on what else the step holds.
"""

from __future__ import annotations

import torch

from .. import kernels
from ..weights.loader import ExpectedTensor
from .feedforward import GatedMLP
from .linear import Linear
from .registry import register_feedforward


@register_feedforward("routed_experts")
class RoutedExperts:
    graph_safe = True

    @staticmethod
    def expected_tensors(spec):
        out = {}
        for e in range(spec.n_experts):
            p = f"{spec.expert_prefix}{e}."
            out[p + "gate"] = ExpectedTensor((spec.intermediate, spec.hidden))
            out[p + "up"] = ExpectedTensor((spec.intermediate, spec.hidden))
            out[p + "down"] = ExpectedTensor((spec.hidden, spec.intermediate))
        out[spec.router] = ExpectedTensor((spec.n_experts, spec.hidden))
        if spec.correction is not None:
            out[spec.correction] = ExpectedTensor((spec.n_experts,))
        if spec.router_bias is not None:
            out[spec.router_bias] = ExpectedTensor((spec.n_experts,))
        if spec.shared is not None:
            out.update(GatedMLP.expected_tensors(spec.shared))
            out[spec.shared_gate] = ExpectedTensor((1, spec.hidden))
        return out

    def __init__(self, spec, tensors, rt):
        E = spec.n_experts
        if E % spec.n_groups or not 0 < spec.keep_groups <= spec.n_groups:
            raise ValueError(f"{E} experts in {spec.n_groups} groups of which {spec.keep_groups} are kept: not possible")
        if not 0 < spec.top <= spec.keep_groups * (E // spec.n_groups):
            raise ValueError(f"{spec.top} experts cannot be chosen from {spec.keep_groups} groups of {E // spec.n_groups}")
        if spec.score not in kernels.ROUTE_SCORES:
            raise ValueError(f"router score {spec.score!r} is not built (known: {', '.join(kernels.ROUTE_SCORES)})")
        if spec.score == "softmax_top" and (spec.n_groups != 1 or spec.correction is not None):
            raise ValueError("a router whose weights are the softmax over the chosen logits has no groups and no correction")
        if spec.score != "softmax_top" and spec.router_bias is not None:
            raise ValueError("a bias of the router's logits belongs to the softmax over the chosen logits")
        self.spec = spec
        self.rt = rt
        names = [f"{spec.expert_prefix}{e}." for e in range(E)]
        every = [tensors[p + k] for p in names for k in ("gate", "up", "down")]
        dtype = torch.float32 if any(t.dtype is torch.float32 for t in every) else every[0].dtype
        # [experts, 2 * intermediate, hidden] with rows alternating gate_j, up_j: a thread of the product's epilogue
        # then holds both halves of a pair; [experts, hidden, intermediate] for the way back
        self.gate_up = torch.stack([torch.stack([tensors[p + "gate"].to(dtype), tensors[p + "up"].to(dtype)], dim=1)
                                    .reshape(2 * spec.intermediate, spec.hidden) for p in names]).contiguous()
        self.down = torch.stack([tensors[p + "down"].to(dtype) for p in names]).contiguous()
        rows = [tensors[spec.router]] + ([tensors[spec.shared_gate].reshape(1, spec.hidden)] if spec.shared is not None else [])
        rdtype = torch.float32 if any(t.dtype is torch.float32 for t in rows) else rows[0].dtype
        self.router = torch.cat([t.to(rdtype) for t in rows], dim=0).contiguous()
        self.correction = tensors[spec.correction].contiguous() if spec.correction is not None else None
        if spec.router_bias is not None:
            self.correction = tensors[spec.router_bias].contiguous()      # the route kernel adds it to the logits
        self.shared = GatedMLP(spec.shared, tensors, rt) if spec.shared is not None else None

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        s, rt, ws = self.spec, self.rt, self.rt.ws
        n, E, top = x.shape[0], s.n_experts, s.top
        n_pairs = n * top
        logits = ws.take("moe_logits", (n, self.router.shape[0]), torch.float32)
        # float32 products and sums whatever the activation type; few outputs: a warp per (token, expert)
        (kernels.gemm_rowdot if self.router.shape[0] <= 128 else kernels.gemm_simt)(x, self.router, logits)
        ids = ws.take("moe_ids", (n, top), torch.int32)
        weights = ws.take("moe_weights", (n, top), torch.float32)
        gate = ws.take("moe_gate", (n,), torch.float32) if self.shared is not None else None
        kernels.moe_route(logits, self.correction, ids, weights, gate, E, top, s.n_groups, s.keep_groups, s.route_scale,
                          s.weight_eps, gate_col=E if self.shared is not None else -1, score=s.score)
        sorted_pairs = ws.take("moe_sorted", (n_pairs,), torch.int32)
        tiles = ws.take("moe_tiles", (kernels.moe_max_tiles(n_pairs, E), 4), torch.int32)
        kernels.moe_sort(ids, E, sorted_pairs, tiles)
        hidden = ws.take("moe_hidden", (n_pairs, s.intermediate), rt.act_dtype)       # in sorted order
        kernels.moe_gemm(x, self.gate_up, hidden, sorted_pairs, tiles, top, gather=True, scatter=False, epi="silu_mul")
        y = ws.take("moe_pairs_out", (n_pairs, s.hidden), torch.float32)               # in the pairs' own order
        kernels.moe_gemm(hidden, self.down, y, sorted_pairs, tiles, top, gather=False, scatter=True)
        shared = self.shared.forward(x, ctx) if self.shared is not None else None
        out = ws.take("moe_out", (n, s.hidden), torch.float32)
        kernels.moe_combine(y, weights, gate, shared, out)
        return out
