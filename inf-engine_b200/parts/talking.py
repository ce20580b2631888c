"""Attention whose softmax weights are mixed across heads after the softmax ("talking heads"), under a sliding window.

Per token, with x the mixer's input (``TalkingAttentionSpec`` states the rule in full):

    q, k, v = one product over the row-concatenated weights (the output gate's rows ride in it too); biases added
    every query head, key head and value head divided by its root mean square (no gain); k and v cached so
    w_g(i, j) = softmax_j(q_g(i) . k_c(g)(j) * scale) over the keys the window lets i see
    w'_h(i, j) = sum_g talk[h, g] w_g(i, j);  o_h(i) = sum_j w'_h(i, j) v_c(h)(j)
    out = o_proj (o * sigmoid(gate x))

Mixing the weights and then applying them to a head's own values is the same sum as applying every UNMIXED head's
weights to that head's values and mixing the results: o_h = sum_g talk[h, g] A[g, c(h)], A[g, c] = sum_j w_g(i, j)
v_c(j).  So the attention kernels of the package run as they are, each query head over ALL value heads at once: the
value heads of a token lie side by side in one cached row (one value head of kv_heads x v_head_dim numbers, in slices
of at most 256 where that is wider), and one kernel then forms the sum over g, times the output gate.  Scores, maxima,
weights and sums are float32 whatever the storage type (``latent.attend_float32``), the mix is float32.
"""

from __future__ import annotations

import torch

from .. import kernels
from ..cache.manager import CacheRequirement
from ..weights.loader import ExpectedTensor
from .latent import attend_float32
from .linear import Linear, stack_rows
from .registry import register_mixer

MAX_VALUE_ROW = 256           # the attention kernels take value rows up to this many numbers


@register_mixer("talking_attention")
class TalkingAttention:
    graph_safe = True

    @staticmethod
    def expected_tensors(spec):
        H, G, d, dv = spec.n_heads, spec.n_kv_heads, spec.head_dim, spec.v_head_dim
        out = {}
        for name, bias, width in ((spec.q_proj, spec.q_bias, H * d), (spec.k_proj, spec.k_bias, G * d),
                                  (spec.v_proj, spec.v_bias, G * dv)):
            out[name] = ExpectedTensor((width, spec.hidden))
            if bias is not None:
                out[bias] = ExpectedTensor((width,))
        if spec.talk is not None:
            out[spec.talk] = ExpectedTensor((H, H))
        if spec.gate_proj is not None:
            out[spec.gate_proj] = ExpectedTensor((H * dv, spec.hidden))
        out[spec.o_proj] = ExpectedTensor((spec.hidden, H * dv))
        return out

    def __init__(self, spec, tensors, rt):
        H, G, d, dv = spec.n_heads, spec.n_kv_heads, spec.head_dim, spec.v_head_dim
        if G <= 0 or H % G:
            raise ValueError(f"{H} query heads are not a multiple of {G} kv heads")
        if not (0 < d <= 256 and 0 < dv <= MAX_VALUE_ROW):
            raise ValueError(f"attention kernels take head sizes up to 256, not {d} and {dv}")
        if spec.window is not None and spec.window <= 0:
            raise ValueError("an attention window must be positive")
        self.spec = spec
        self.rt = rt
        ws = [tensors[spec.q_proj], tensors[spec.k_proj], tensors[spec.v_proj]]
        if spec.gate_proj is not None:
            ws.append(tensors[spec.gate_proj])
        dtype = torch.float32 if any(w.dtype is torch.float32 for w in ws) else ws[0].dtype
        stacked, self.cols = stack_rows(ws, dtype)
        self.proj = Linear(stacked, rt, "talking_proj")
        self.q_width, self.k_width, self.v_width, self.out_width = H * d, G * d, G * dv, H * dv
        biases = [tensors[n] for n in (spec.q_bias, spec.k_bias, spec.v_bias) if n is not None]
        bdtype = torch.float32 if any(b.dtype is torch.float32 for b in biases) else (biases[0].dtype if biases else None)
        pick = lambda n: tensors[n].to(bdtype).contiguous() if n is not None else None
        self.q_bias, self.k_bias, self.v_bias = pick(spec.q_bias), pick(spec.k_bias), pick(spec.v_bias)
        # without a mixing matrix every head keeps its own weights: the identity
        self.talk = (tensors[spec.talk].float() if spec.talk is not None
                     else torch.eye(H, dtype=torch.float32, device=ws[0].device)).contiguous()
        self.o = Linear(tensors[spec.o_proj], rt, "o")
        # value heads a launch of the attention takes at once: whole heads, rows of at most MAX_VALUE_ROW numbers
        self.slice_heads = max(1, min(G, MAX_VALUE_ROW // dv))

    def cache_requirement(self) -> CacheRequirement:
        s = self.spec
        # the value heads of a token side by side in one row: every query head reads all of them
        return CacheRequirement(kind="kv", n_kv_heads=s.n_kv_heads, head_dim=s.head_dim, window=s.window,
                                dtype=self.rt.act_dtype, v_head_dim=s.n_kv_heads * s.v_head_dim, n_v_heads=1)

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        s, rt = self.spec, self.rt
        n = x.shape[0]
        H, G, d, dv = s.n_heads, s.n_kv_heads, s.head_dim, s.v_head_dim
        cols = self.cols
        proj = self.proj(x, rt.ws.take("talking_proj", (n, cols[-1]), rt.act_dtype))
        q, k, v = (proj[:, cols[0]:cols[0] + self.q_width], proj[:, cols[1]:cols[1] + self.k_width],
                   proj[:, cols[2]:cols[2] + self.v_width])
        gate = proj[:, cols[3]:cols[3] + self.out_width] if s.gate_proj is not None else None
        kvctx = ctx.kv[cache.group]
        kpool, vpool = (cache.k, cache.v) if cache.write else (None, None)
        kernels.qkv_prepare(q, H, k, G, d, v, G, dv, kvctx.slot_mapping, kpool, vpool, ctx.page_size, s.norm_eps,
                            q_bias=self.q_bias, k_bias=self.k_bias, v_bias=self.v_bias, q_norm=s.qk_norm,
                            k_norm=s.qk_norm, v_norm=s.v_norm, pool_v_heads=1)
        out = rt.ws.take("talking_out", (n, self.out_width), rt.act_dtype)
        row = G * dv
        values = cache.v.view(cache.v.shape[0], -1, row)            # [pages, page_size, all value heads of a token]
        for c0 in range(0, G, self.slice_heads):
            nc = min(self.slice_heads, G - c0)
            unmixed = rt.ws.take("talking_unmixed", (n, H * nc * dv), rt.act_dtype)
            # the slice's value heads are the first nc * dv numbers of rows that start c0 * dv into the cached row
            attend_float32(q, unmixed, cache.k, values[:, :, c0 * dv:], ctx, kvctx, H, G, d, nc * dv, float(s.scale),
                           None, n_v_heads=1, v_row=row, window=s.window)
            kernels.talk_combine(unmixed, self.talk, gate, out, H, G, dv, first_v_head=c0, slice_v_heads=nc)
        return self.o(out, rt.ws.take("mixer_out", (n, s.hidden), rt.act_dtype))
