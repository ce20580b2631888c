"""Dense gated feed-forward: ``down(silu(gate(x)) * up(x))`` (engine/llama_mlp.py:30-33); other activations of the
gate, clamps of both branches and an offset of the up branch are options of the spec (``kernels.glu_act``).

Gate and up are one matrix product over the row-concatenated weights
[2*intermediate, hidden]; the activation and the product by ``up`` are one
kernel in float32 arithmetic.

``PolyNormMLP``: ``down(act(up(x) + b_up)) + b_down`` with the PolyNorm activation,
a polynomial of the normalised first three powers of each token's hidden vector
(its bias add, sums and norms are one float32 kernel).
"""

from __future__ import annotations

import torch

from .. import kernels
from ..weights.loader import ExpectedTensor
from .linear import Linear, stream_into_residual, stream_normed
from .registry import register_feedforward


@register_feedforward("gated_mlp")
class GatedMLP:
    graph_safe = True

    @staticmethod
    def expected_tensors(spec):
        return {
            spec.gate_proj: ExpectedTensor((spec.intermediate, spec.hidden)),
            spec.up_proj: ExpectedTensor((spec.intermediate, spec.hidden)),
            spec.down_proj: ExpectedTensor((spec.hidden, spec.intermediate)),
        }

    def __init__(self, spec, tensors, rt):
        if spec.activation not in kernels.GLU_KINDS:
            raise ValueError(f"activation {spec.activation!r} is not built (known: {sorted(kernels.GLU_KINDS)})")
        # the products' fused epilogues know silu(gate) * up only; any other activation is a kernel of its own
        self.plain_silu = spec.activation == "silu" and spec.up_offset == 0.0
        self.spec = spec
        self.rt = rt
        gate, up = tensors[spec.gate_proj], tensors[spec.up_proj]
        dtype = torch.float32 if torch.float32 in (gate.dtype, up.dtype) else gate.dtype
        # rows alternate gate_j, up_j: one thread of a product's epilogue then holds both halves of a pair
        both = torch.stack([gate.to(dtype), up.to(dtype)], dim=1).reshape(2 * spec.intermediate, spec.hidden)
        self.gate_up = Linear(both.contiguous(), rt, "gate_up")
        self.down = Linear(tensors[spec.down_proj], rt, "down")

    def can_fuse(self, n_tokens: int, norm) -> bool:
        return (self.plain_silu and hasattr(norm, "fusable_rms") and self.gate_up.streams(n_tokens, normed=True)
                and self.down.streams(n_tokens))

    def forward_fused(self, residual: torch.Tensor, norm, ctx) -> None:
        """residual += down(silu(gate(n)) * up(n)) with n = norm(residual), in two launches: the norm rides in
        the first product's prologue, the activation in its epilogue, the sum in the second's epilogue."""
        n = residual.shape[0]
        s, ws = self.spec, self.rt.ws
        h = ws.take("ff_hidden", (n, s.intermediate), torch.bfloat16)
        stream_normed(self.gate_up, residual, h, n, "silu_mul", norm, ctx)
        stream_into_residual(self.down, h, residual, n, ctx, self.rt)

    TCGEN05_MIN_ROWS = 128     # below one tile of rows the library product is the better choice

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        n = x.shape[0]
        s, ws, dt = self.spec, self.rt.ws, self.rt.act_dtype
        h = ws.take("ff_hidden", (n, s.intermediate), dt)
        w = self.gate_up.weight
        if (dt is torch.bfloat16 and w.dtype is torch.bfloat16 and n >= self.TCGEN05_MIN_ROWS
                and kernels.gemm_tcgen05_supports(n, 2 * s.intermediate, s.hidden, x.stride(0), w.stride(0))):
            # gate/up on the tcgen05 tensor cores with the gated activation in the epilogue: the [n, 2*intermediate]
            # matrix never goes to memory
            act = None if self.plain_silu else \
                ((s.act_alpha, s.act_limit, s.up_offset) if s.activation == "clamped_swish" else (1.0, float("inf"), s.up_offset))
            kernels.gemm_tcgen05(x, w, h, "silu_mul", act=act)
        else:
            gu = self.gate_up(x, ws.take("ff_gate_up", (n, 2 * s.intermediate), dt))
            if self.plain_silu:
                kernels.silu_mul(gu, h, interleaved=True)
            else:
                kernels.glu_act(gu, h, s.activation, interleaved=True, alpha=s.act_alpha, limit=s.act_limit,
                                up_offset=s.up_offset)
        return self.down(h, ws.take("ff_out", (n, s.hidden), dt))


@register_feedforward("polynorm_mlp")
class PolyNormMLP:
    graph_safe = True

    @staticmethod
    def expected_tensors(spec):
        out = {spec.up_proj: ExpectedTensor((spec.intermediate, spec.hidden))}
        if spec.up_bias is not None:
            out[spec.up_bias] = ExpectedTensor((spec.intermediate,))
        out[spec.down_proj] = ExpectedTensor((spec.hidden, spec.intermediate))
        if spec.down_bias is not None:
            out[spec.down_bias] = ExpectedTensor((spec.hidden,))
        out[spec.coef] = ExpectedTensor((4,), init="gain")
        return out

    def __init__(self, spec, tensors, rt):
        self.spec = spec
        self.rt = rt
        self.up = Linear(tensors[spec.up_proj], rt, "up")            # its bias rides in the activation kernel
        self.coef = tensors[spec.coef]
        self.up_bias = tensors[spec.up_bias].to(self.coef.dtype) if spec.up_bias is not None else None
        self.down = Linear(tensors[spec.down_proj], rt, "down",
                           bias=tensors[spec.down_bias] if spec.down_bias is not None else None)
        self.eps = float(spec.eps)

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        n = x.shape[0]
        s, ws, dt = self.spec, self.rt.ws, self.rt.act_dtype
        z = self.up(x, ws.take("ff_up", (n, s.intermediate), dt))
        h = ws.take("ff_hidden", (n, s.intermediate), dt)
        kernels.polynorm(z, self.up_bias, self.coef, h, self.eps)
        return self.down(h, ws.take("ff_out", (n, s.hidden), dt))
