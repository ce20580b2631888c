"""A recurrent block around a real-gated linear recurrent unit, and mixers that run side by side.

``GatedLinearRecurrence`` (``width`` channels), with x the mixer's input:

    y = gelu_tanh(y_proj x + y_bias)                          one product for both branches, biases added to it
    u = conv(x_proj x + x_bias)                               a short causal convolution per channel, with a bias
    r = sigmoid(A_b u_b + a_b),  i = sigmoid(I_b u_b + i_b)   per block b of n_blocks equal parts (float32 products)
    a = exp(-decay_scale * r * softplus(lam))
    S <- a S + sqrt(1 - a^2) (i * u);   out = o_proj (S * y)  S: float32, one vector a request, zero at the start

The gates, the decay, the state and the product with y are float32 (``csrc/sequence.cu``); the step's tokens of
every request run in order from the state that the step before left.

``ParallelMixer`` runs several mixers on the same input and adds what they return; each branch carries its weight
in the sum as its own ``out_scale``.  When every branch ends in an output projection (``forward_core`` returns what
goes into it) the branches' results are laid side by side and ONE product over the column-concatenated output
weights gives the sum.
"""

from __future__ import annotations

import torch

from .. import kernels
from ..cache.manager import CacheRequirement
from ..weights.loader import ExpectedTensor
from .gated_delta import conv_state_requirement, same_dtype
from .linear import Linear
from .registry import build_mixer, mixer_class, register_mixer


@register_mixer("gated_linear_recurrence")
class GatedLinearRecurrence:
    graph_safe = True

    @staticmethod
    def expected_tensors(spec):
        w, bs = spec.width, spec.width // max(spec.n_blocks, 1)
        out = {
            spec.y_proj: ExpectedTensor((w, spec.hidden)), spec.y_bias: ExpectedTensor((w,)),
            spec.x_proj: ExpectedTensor((w, spec.hidden)), spec.x_bias: ExpectedTensor((w,)),
            spec.conv.weight: ExpectedTensor((w, spec.conv.taps)),
        }
        if spec.conv.bias is not None:
            out[spec.conv.bias] = ExpectedTensor((w,))
        out[spec.a_gate] = ExpectedTensor((spec.n_blocks, bs, bs))
        out[spec.a_gate_bias] = ExpectedTensor((spec.n_blocks, bs))
        out[spec.i_gate] = ExpectedTensor((spec.n_blocks, bs, bs))
        out[spec.i_gate_bias] = ExpectedTensor((spec.n_blocks, bs))
        out[spec.lam] = ExpectedTensor((w,))
        out[spec.o_proj] = ExpectedTensor((spec.hidden, w))
        return out

    def __init__(self, spec, tensors, rt):
        if spec.n_blocks <= 0 or spec.width % spec.n_blocks:
            raise ValueError(f"a width of {spec.width} does not split into {spec.n_blocks} equal blocks")
        if not 1 <= spec.conv.taps <= kernels.CONV_MAX_TAPS:
            raise ValueError(f"a short convolution has 1 to {kernels.CONV_MAX_TAPS} taps, not {spec.conv.taps}")
        self.spec = spec
        self.rt = rt
        ws = [tensors[spec.y_proj], tensors[spec.x_proj]]
        dtype = torch.float32 if any(w.dtype is torch.float32 for w in ws) else ws[0].dtype
        bias = torch.cat([tensors[spec.y_bias].float(), tensors[spec.x_bias].float()]).to(dtype)
        self.proj = Linear(torch.cat([w.to(dtype) for w in ws], dim=0).contiguous(), rt, "recurrence_proj", bias=bias)
        conv = [tensors[spec.conv.weight]] + ([tensors[spec.conv.bias]] if spec.conv.bias is not None else [])
        conv = same_dtype(conv)
        self.conv_weight, self.conv_bias = conv[0], (conv[1] if len(conv) > 1 else None)
        self.a_gate, self.i_gate = tensors[spec.a_gate].contiguous(), tensors[spec.i_gate].contiguous()
        self.a_bias, self.i_bias, self.lam = same_dtype([tensors[spec.a_gate_bias].reshape(-1),
                                                         tensors[spec.i_gate_bias].reshape(-1), tensors[spec.lam]])
        self.o_weight = tensors[spec.o_proj]
        self.o = Linear(self.o_weight, rt, "o")
        self.core_width = spec.width

    def cache_requirement(self) -> CacheRequirement:
        s = self.spec
        return CacheRequirement(kind="several", parts=(
            CacheRequirement(kind="state", state_shape=(s.width,), state_dtype=torch.float32),
            conv_state_requirement(s.conv.taps, s.width, self.rt.act_dtype)))

    def forward_core(self, x: torch.Tensor, ctx, cache, out: torch.Tensor) -> None:
        """``out`` ([n, width], may be a column slice) = out_scale * S * y: what goes into the output projection."""
        s, rt = self.spec, self.rt
        n, w = x.shape[0], s.width
        state, conv_state = cache.parts
        proj = self.proj(x, rt.ws.take("recurrence_proj", (n, 2 * w), rt.act_dtype))
        u = rt.ws.take("recurrence_u", (n, w), rt.act_dtype)
        kernels.causal_conv(proj[:, w:], self.conv_weight, self.conv_bias, conv_state.state, u, ctx.q_start, ctx.slots,
                            ctx.n_requests, activation=None, write_state=cache.write, max_q_len=ctx.max_q_len)
        gates = rt.ws.take("recurrence_gates", (n, 2 * w), torch.float32)
        kernels.gemm_simt_batched(u, self.a_gate, gates[:, :w])
        kernels.gemm_simt_batched(u, self.i_gate, gates[:, w:])
        kernels.linear_recurrence(u, proj[:, :w], gates[:, :w], gates[:, w:], self.a_bias, self.i_bias, self.lam,
                                  state.state, out, ctx.q_start, ctx.slots, ctx.n_requests, s.decay_scale, s.out_scale,
                                  write_state=cache.write)

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        rt = self.rt
        n = x.shape[0]
        mixed = rt.ws.take("recurrence_mixed", (n, self.spec.width), rt.act_dtype)
        self.forward_core(x, ctx, cache, mixed)
        return self.o(mixed, rt.ws.take("mixer_out", (n, self.spec.hidden), rt.act_dtype))


@register_mixer("mingru")
class MinGRU:
    """A gated recurrence whose gates read the current token only (``MinGRUSpec``): one product for z, u and the
    output gate, one scan kernel from there to ``S * silu(gate)`` in float32 (``csrc/gating.cu``), the output product.
    The state is one float32 vector a request; the step's tokens of every request run in order from the state the step
    before left."""

    graph_safe = True

    @staticmethod
    def expected_tensors(spec):
        w = spec.width
        return {
            spec.z_proj: ExpectedTensor((w, spec.hidden)), spec.z_bias: ExpectedTensor((w,)),
            spec.x_proj: ExpectedTensor((w, spec.hidden)), spec.x_bias: ExpectedTensor((w,)),
            spec.gate_proj: ExpectedTensor((w, spec.hidden)),
            spec.o_proj: ExpectedTensor((spec.hidden, w)),
        }

    def __init__(self, spec, tensors, rt):
        self.spec = spec
        self.rt = rt
        ws = [tensors[spec.z_proj], tensors[spec.x_proj], tensors[spec.gate_proj]]
        dtype = torch.float32 if any(w.dtype is torch.float32 for w in ws) else ws[0].dtype
        self.proj = Linear(torch.cat([w.to(dtype) for w in ws], dim=0).contiguous(), rt, "mingru_proj")
        self.z_bias, self.x_bias = same_dtype([tensors[spec.z_bias], tensors[spec.x_bias]])     # added in float32 by the scan
        self.o = Linear(tensors[spec.o_proj], rt, "o")

    def cache_requirement(self) -> CacheRequirement:
        return CacheRequirement(kind="state", state_shape=(self.spec.width,), state_dtype=torch.float32)

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        s, rt = self.spec, self.rt
        n, w = x.shape[0], s.width
        proj = self.proj(x, rt.ws.take("mingru_proj", (n, 3 * w), rt.act_dtype))
        mixed = rt.ws.take("mingru_mixed", (n, w), rt.act_dtype)
        kernels.mingru_scan(proj[:, :w], proj[:, w:2 * w], proj[:, 2 * w:], self.z_bias, self.x_bias, cache.state, mixed,
                            ctx.q_start, ctx.slots, ctx.n_requests, write_state=cache.write, max_q_len=ctx.max_q_len)
        return self.o(mixed, rt.ws.take("mixer_out", (n, s.hidden), rt.act_dtype))


@register_mixer("parallel")
class ParallelMixer:
    @staticmethod
    def expected_tensors(spec):
        out = {}
        for b in spec.branches:
            out.update(mixer_class(b).expected_tensors(b))
        return out

    def __init__(self, spec, tensors, rt):
        if not spec.branches:
            raise ValueError("a parallel mixer needs at least one branch")
        self.spec = spec
        self.rt = rt
        self.branches = [build_mixer(b, tensors, rt) for b in spec.branches]
        self.graph_safe = all(getattr(b, "graph_safe", False) for b in self.branches)
        # one output product for all branches when each can say what goes into its own
        self.joint = all(hasattr(b, "forward_core") and hasattr(b, "o_weight") for b in self.branches)
        if self.joint:
            ws = [b.o_weight for b in self.branches]
            dtype = torch.float32 if any(w.dtype is torch.float32 for w in ws) else ws[0].dtype
            self.o = Linear(torch.cat([w.to(dtype) for w in ws], dim=1).contiguous(), rt, "o")
            self.widths = [b.core_width for b in self.branches]
            for b in self.branches:          # the branches' own output weights are not used again
                b.o_weight = None
                b.o = None

    def cache_requirement(self) -> CacheRequirement:
        return CacheRequirement(kind="several", parts=tuple(b.cache_requirement() for b in self.branches))

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        rt = self.rt
        n = x.shape[0]
        if self.joint:
            cores = rt.ws.take("parallel_cores", (n, sum(self.widths)), rt.act_dtype)
            at = 0
            for b, view, w in zip(self.branches, cache.parts, self.widths):
                b.forward_core(x, ctx, view, cores[:, at:at + w])
                at += w
            return self.o(cores, rt.ws.take("mixer_out", (n, self.spec.hidden), rt.act_dtype))
        total = None
        for b, view in zip(self.branches, cache.parts):
            y = b.forward(x, ctx, view)
            if total is None:
                total = rt.ws.take("parallel_sum", tuple(y.shape), torch.float32)
                total.zero_()
            kernels.residual_add(total, y)
        return total
