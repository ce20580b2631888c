"""The matrix memory of xLSTM (mLSTM) as a mixer: a recurrent layer whose cache is, per head and request, a
``head_dim x v_head_dim`` float32 matrix, a normaliser vector and a running maximum of the log gates.

With x the mixer's input, per token (``MatrixMemorySpec`` states the rule in full):

    q, k (heads x head_dim), v, gate (heads x v_head_dim) = one product of x in the activation type
    zi, zf (heads)                                        = one product of x with float32 sums and results
    i = cap tanh((zi + b_i) / cap),  f = logsigmoid(cap tanh((zf + b_f) / cap))
    m' = max(f + m, i);  S <- exp(f + m - m') S + exp(i - m') k v^T;  n likewise with k;  m <- m'
    o = S^T (q / sqrt(head_dim)) / (max(|n . q / sqrt(head_dim)|, exp(-m)) + 1e-6)
    out = o_proj (o / rms(o per head) * out_gain * sigmoid(gate))

Everything from the gates' pre-activations to the gated output is float32 inside two kernels
(``csrc/matrix_memory.cu``); the step's tokens of every request run in order from the state the step before left (all
zeros for a new request, the maximum too), so a whole prompt, a portion and a single decoded token take the same path.
"""

from __future__ import annotations

import torch

from .. import kernels
from ..cache.manager import CacheRequirement
from ..weights.loader import ExpectedTensor
from .gated_delta import same_dtype
from .linear import Linear, stack_rows
from .registry import register_mixer


@register_mixer("matrix_memory")
class MatrixMemory:
    graph_safe = True          # request bounds and state slots are read on the device

    @staticmethod
    def expected_tensors(spec):
        H, d, dv = spec.n_heads, spec.head_dim, spec.v_head_dim
        return {
            spec.q_proj: ExpectedTensor((H * d, spec.hidden)),
            spec.k_proj: ExpectedTensor((H * d, spec.hidden)),
            spec.v_proj: ExpectedTensor((H * dv, spec.hidden)),
            spec.gate_proj: ExpectedTensor((H * dv, spec.hidden)),
            spec.o_proj: ExpectedTensor((spec.hidden, H * dv)),
            spec.out_gain: ExpectedTensor((H * dv,), init="gain"),
            spec.i_proj: ExpectedTensor((H, spec.hidden)),
            spec.i_bias: ExpectedTensor((H,)),
            spec.f_proj: ExpectedTensor((H, spec.hidden)),
            spec.f_bias: ExpectedTensor((H,)),
        }

    def __init__(self, spec, tensors, rt):
        if not spec.gate_cap > 0:
            raise ValueError("the cap of the gates' pre-activations must be positive")
        self.spec = spec
        self.rt = rt
        H, d, dv = spec.n_heads, spec.head_dim, spec.v_head_dim
        self.qk, self.vw = H * d, H * dv
        # columns of the one projection: q | k | v | gate
        ws = [tensors[n] for n in (spec.q_proj, spec.k_proj, spec.v_proj, spec.gate_proj)]
        dtype = torch.float32 if any(w.dtype is torch.float32 for w in ws) else ws[0].dtype
        stacked, self.cols = stack_rows(ws, dtype)
        self.proj = Linear(stacked, rt, "matrix_memory_proj")
        gs = [tensors[spec.i_proj], tensors[spec.f_proj]]
        gdtype = torch.float32 if any(g.dtype is torch.float32 for g in gs) else gs[0].dtype
        self.gate_rows = torch.cat([g.to(gdtype) for g in gs], dim=0).contiguous()      # [2 heads, hidden]: i, then f
        self.i_bias, self.f_bias = same_dtype([tensors[spec.i_bias], tensors[spec.f_bias]])
        self.out_gain = tensors[spec.out_gain].contiguous()
        self.o = Linear(tensors[spec.o_proj], rt, "o")
        self.state_floats = kernels.mlstm_state_floats(d, dv)

    def cache_requirement(self) -> CacheRequirement:
        return CacheRequirement(kind="state", state_shape=(self.spec.n_heads, self.state_floats), state_dtype=torch.float32)

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        s, rt = self.spec, self.rt
        n = x.shape[0]
        H, d, dv = s.n_heads, s.head_dim, s.v_head_dim
        c = self.cols
        proj = self.proj(x, rt.ws.take("matrix_memory_proj", (n, c[-1]), rt.act_dtype))
        q, k = proj[:, c[0]:c[0] + self.qk], proj[:, c[1]:c[1] + self.qk]
        v, gate = proj[:, c[2]:c[2] + self.vw], proj[:, c[3]:c[3] + self.vw]
        # the gates' pre-activations: float32 products, sums and results whatever the activation type
        z = rt.ws.take("matrix_memory_gates", (n, 2 * H), torch.float32)
        (kernels.gemm_rowdot if 2 * H <= 128 else kernels.gemm_simt)(x, self.gate_rows, z)
        o = rt.ws.take("matrix_memory_o", (n, self.vw), torch.float32)
        kernels.mlstm_scan(q, k, v, z, self.i_bias, self.f_bias, s.gate_cap, cache.state, o, ctx.q_start, ctx.slots,
                           ctx.n_requests, H, d, dv, write_state=cache.write)
        mixed = rt.ws.take("matrix_memory_mixed", (n, self.vw), rt.act_dtype)
        kernels.mlstm_finish(o, self.out_gain, gate, mixed, H, dv, s.norm_eps)
        return self.o(mixed, rt.ws.take("mixer_out", (n, s.hidden), rt.act_dtype))
