"""Attention over a compressed key/value vector, attention with two score maps a head, and what they share.

``LatentAttention``: per token the cache holds one row ``[c, k_rot]``: the compressed vector c (``kv_rank`` numbers,
RMS-normed) and a rotated key part that all heads share.  A head's unrotated key is ``k_up_h c`` and its value
``v_up_h c``, so its score is ``q_un . (k_up_h c) + q_rot . k_rot = (k_up_h^T q_un) . c + q_rot . k_rot``: the query is
carried over to the compressed space once (a product per head, ``heads_product``), every head then reads the SAME
cached rows (attention with one key head whose values are the first ``kv_rank`` dimensions of its keys), and the
head's output ``v_up_h (sum_j w_j c_j)`` is one more product per head.  Nothing per head is ever stored per token.

``DifferentialAttention``: the two maps of a head are attention heads of their own that share a value head: 2 x heads
query heads over 2 x kv_heads key heads and kv_heads value heads.  The query rows are reordered once at load
(``[kv head, map, head in group]``) so that the query heads of one key head lie side by side, as the attention
kernels expect; a kernel then forms ``a1 - lambda a2``, norms it, and applies the output gate.

Both keep scores, maxima, weights and sums in float32 whatever the storage type: a block per (token, head) whose
warps split the keys for requests that bring a few tokens; for prompt portions the tensor-core kernel with float32
scores (``kernels.attention_wide``: bfloat16 storage, head sizes that are multiples of 16) or else the float32 tile
kernel on CUDA cores.
"""

from __future__ import annotations

import torch

from .. import kernels
from ..cache.manager import CacheRequirement
from ..weights.loader import ExpectedTensor
from .linear import Linear, stack_rows
from .registry import build_position, position_class, register_mixer

SMALL_REQUEST_TOKENS = 4      # requests that bring at most this many tokens get the split-key rows kernel


WIDE_SMALL_MIN_GROUP = 4      # query heads a key head from which decode tokens take the tensor-core kernel too


def attend_float32(q, out, kpool, vpool, ctx, kvctx, n_heads: int, n_kv_heads: int, head_dim: int, v_head_dim: int,
                   scale: float, chunk: int | None, n_v_heads: int | None = None, v_row: int | None = None,
                   window: int | None = None, sink: torch.Tensor | None = None) -> None:
    """Causal attention of the step's queries over the paged keys with float32 scores, maxima, weights and sums.
    Requests of at most ``SMALL_REQUEST_TOKENS`` tokens (decode tokens): a block per (token, head) whose warps split the
    keys, or, in bfloat16 storage with head sizes that are multiples of 16 and several query heads a key head, the
    tensor-core kernel with the keys split over blocks (every key row is then loaded once for all those heads).  The
    others (prompt portions), through a work list: the tensor-core kernel under the same conditions, else the float32
    tile kernel.  ``window``: a query sees itself and the window - 1 keys before it.  ``sink`` (float32 [n_heads]): a
    term exp(sink_h) without key or value in the denominator of head h."""
    group = n_heads // n_kv_heads
    max_rows = SMALL_REQUEST_TOKENS * group
    if ctx.max_q_len <= SMALL_REQUEST_TOKENS:
        n_small = ctx.n_requests
    else:
        n_small = sum(1 for n in ctx.host["q_lens"] if n <= SMALL_REQUEST_TOKENS)
    extra = dict(v_head_dim=v_head_dim, chunk=chunk or 0, n_v_heads=n_v_heads, v_row=v_row, sink=sink)
    wide = (kpool.dtype is torch.bfloat16 and kernels.attention_wide_supports(q, out, head_dim, v_head_dim, v_row)
            and kpool.data_ptr() % 16 == 0 and vpool.data_ptr() % 16 == 0)
    if n_small:
        if wide and group >= WIDE_SMALL_MIN_GROUP:
            rows = kernels.ATTENTION_WIDE_ROWS
            # the longest run of keys a small request may see, from the tile boundary below its first key
            keys = min(ctx.keys_cap, chunk + SMALL_REQUEST_TOKENS) if chunk else ctx.keys_cap
            if window:
                keys = min(keys, window + SMALL_REQUEST_TOKENS)
            n_splits, split_keys = kernels.attention_wide_splits(head_dim, v_head_dim, keys + 64,
                                                                  ctx.n_requests * -(-max_rows // rows) * n_kv_heads)
            words = kernels.attention_wide_small_scratch(head_dim, v_head_dim, ctx.n_requests, max_rows, n_kv_heads, n_splits)
            scratch = ctx.rt.ws.take("attn_wide_scratch", (words,), torch.float32) if words else None
            kernels.attention_wide_small(q, out, kpool, vpool, kvctx.block_table, ctx.q_start, ctx.ctx_before, ctx.n_requests,
                                         max_rows, n_heads, n_kv_heads, head_dim, ctx.page_size, window, scale, n_splits,
                                         split_keys, scratch, **extra)
        else:
            kernels.attention_rows(q, out, kpool, vpool, kvctx.block_table, ctx.q_start, ctx.ctx_before, ctx.n_requests,
                                   max_rows, n_heads, n_kv_heads, head_dim, ctx.page_size, window, scale, **extra)
        if n_small == ctx.n_requests:
            return
    if wide:
        # prompt portions in bfloat16 storage: tensor cores, with float32 scores and the weights in two bfloat16 terms
        work_req, work_pair0, n_work = ctx.attention_work(group, kernels.ATTENTION_WIDE_ROWS, max_rows if n_small else 0)
        kernels.attention_wide(q, out, kpool, vpool, kvctx.block_table, ctx.q_start, ctx.ctx_before, work_req, work_pair0,
                               n_work, n_heads, n_kv_heads, head_dim, ctx.page_size, window, scale, **extra)
        return
    work_req, work_pair0, n_work = ctx.attention_work(group, 32, max_rows if n_small else 0)
    kernels.attention_general(q, out, kpool, vpool, kvctx.block_table, ctx.q_start, ctx.ctx_before, work_req, work_pair0,
                              n_work, n_heads, n_kv_heads, head_dim, ctx.page_size, window, scale, **extra)


LIBRARY_HEADS_MIN_ROWS = 64   # rows from which a per-head product in bfloat16 goes to the library's batched product


def heads_product(x: torch.Tensor, x_head: int, w: torch.Tensor, out: torch.Tensor, o_head: int) -> None:
    """A product per head, ``out[m, h * o_head + j] = sum_k x[m, h * x_head + k] * w[h, k, j]`` with float32 sums, as
    ``Linear`` chooses for a projection: float32 operands and few rows (decode tokens, inside captured steps) take this
    package's kernel, whose sums do not depend on the batch; prompt portions in bfloat16 take the library's batched
    product on tensor cores, with the heads as the batch (the rows of ``x`` and ``out`` are read and written in place
    through their strides)."""
    H, K, N = w.shape
    m = x.shape[0]
    if (m >= LIBRARY_HEADS_MIN_ROWS and x.dtype is torch.bfloat16 and w.dtype is torch.bfloat16
            and out.dtype is torch.bfloat16 and x.stride(1) == 1 and out.stride(1) == 1):
        torch.bmm(x.as_strided((H, m, K), (x_head, x.stride(0), 1)), w,
                  out=out.as_strided((H, m, N), (o_head, out.stride(0), 1)))
        return
    kernels.heads_gemm(x, x_head, w, out, o_head)


def _rotation(position):
    """(inv_freq, rot_dims, neighbours, mult) of a position part that turns dimensions, or nothing to turn."""
    if getattr(position, "inv_freq", None) is None:
        return None, 0, False, 1.0
    return position.inv_freq, position.rot_dims, position.neighbours, position.mult


def _common_dtype(ws):
    return torch.float32 if any(w.dtype is torch.float32 for w in ws) else ws[0].dtype


@register_mixer("latent_attention")
class LatentAttention:
    graph_safe = True

    @staticmethod
    def expected_tensors(spec):
        qd = spec.head_dim + spec.rot_dim
        out = {}
        if spec.q_rank:
            out[spec.q_down] = ExpectedTensor((spec.q_rank, spec.hidden))
            out[spec.q_norm] = ExpectedTensor((spec.q_rank,), init="gain")
        out.update({
            spec.q_proj: ExpectedTensor((spec.n_heads * qd, spec.q_rank or spec.hidden)),
            spec.down_proj: ExpectedTensor((spec.kv_rank + spec.rot_dim, spec.hidden)),
            spec.latent_norm: ExpectedTensor((spec.kv_rank,), init="gain"),
            spec.k_up: ExpectedTensor((spec.n_heads * spec.head_dim, spec.kv_rank)),
            spec.v_up: ExpectedTensor((spec.n_heads * spec.v_head_dim, spec.kv_rank)),
        })
        out.update(position_class(spec.position).expected_tensors(spec.position))
        if spec.sink is not None:
            out[spec.sink] = ExpectedTensor((spec.n_heads,))
        if spec.head_gate is not None:
            out[spec.head_gate] = ExpectedTensor((spec.n_heads, spec.hidden))
        out[spec.o_proj] = ExpectedTensor((spec.hidden, spec.n_heads * spec.v_head_dim))
        return out

    def __init__(self, spec, tensors, rt):
        self.spec = spec
        self.rt = rt
        H, d, r, kr, dv = spec.n_heads, spec.head_dim, spec.rot_dim, spec.kv_rank, spec.v_head_dim
        self.q_dim, self.row_dim = d + r, kr + r
        if self.row_dim > 256 or kr > 256:
            raise ValueError(f"the attention kernels take rows up to 256, not a compressed row of {self.row_dim}")
        self.position = build_position(spec.position, tensors, rt)
        inv_freq, rot_dims, _, _ = _rotation(self.position)
        if inv_freq is not None and rot_dims != r:
            raise ValueError(f"the rotation turns {rot_dims} dimensions, the rotated part has {r}")
        if spec.window is not None and (spec.window <= 0 or spec.chunk):
            raise ValueError("a window must be positive, and a layer has a window or chunks, not both")
        # one product of the mixer's input: the queries (or, with queries through a compressed vector of their own, that
        # vector before its norm), the key/value row, and the heads' output gates
        self.q_rank = int(spec.q_rank or 0)
        if self.q_rank and r:
            raise NotImplementedError("queries through a compressed vector together with a rotated part are not built")
        ws = [tensors[spec.q_down] if self.q_rank else tensors[spec.q_proj], tensors[spec.down_proj]]
        if spec.head_gate is not None:
            ws.append(tensors[spec.head_gate])
        stacked, self.cols = stack_rows(ws, _common_dtype(ws))
        self.proj = Linear(stacked, rt, "latent_proj")
        self.q_width = H * self.q_dim
        self.first_width = self.q_rank or self.q_width
        self.gate_width = H if spec.head_gate is not None else 0
        self.latent_gain = tensors[spec.latent_norm].contiguous()
        if self.q_rank:
            self.q_up = Linear(tensors[spec.q_proj], rt, "latent_q_up")
            self.q_gain = tensors[spec.q_norm].contiguous()
            if self.q_gain.dtype != self.latent_gain.dtype:
                self.q_gain, self.latent_gain = self.q_gain.float(), self.latent_gain.float()
        self.sink = tensors[spec.sink].float().contiguous() if spec.sink is not None else None
        # the query's way into the compressed space, a matrix per head: [[k_up_h, 0], [0, 1]] maps [q_un, q_rot] to
        # [k_up_h^T q_un, q_rot] (the rotated part passes through exactly)
        uk = tensors[spec.k_up]
        absorb = torch.zeros((H, self.q_dim, self.row_dim), dtype=uk.dtype, device=uk.device)
        absorb[:, :d, :kr] = uk.view(H, d, kr)
        if r:
            absorb[:, d:, kr:] = torch.eye(r, dtype=uk.dtype, device=uk.device)
        self.absorb = absorb.contiguous()
        self.expand = tensors[spec.v_up].view(H, dv, kr).transpose(1, 2).contiguous()      # [H, kv_rank, v_head_dim]
        self.o = Linear(tensors[spec.o_proj], rt, "o")

    def cache_requirement(self) -> CacheRequirement:
        s = self.spec
        return CacheRequirement(kind="kv", n_kv_heads=1, head_dim=self.row_dim, v_head_dim=s.kv_rank, dtype=self.rt.act_dtype,
                                values_in_keys=True, chunk=s.chunk, window=s.window)

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        s, rt = self.spec, self.rt
        n = x.shape[0]
        H, kr = s.n_heads, s.kv_rank
        cols = self.cols
        proj = self.proj(x, rt.ws.take("latent_proj", (n, cols[-1]), rt.act_dtype))
        q, row = proj[:, :self.first_width], proj[:, cols[1]:cols[1] + self.row_dim]
        kvctx = ctx.kv[cache.group]
        inv_freq, rot_dims, neighbours, mult = _rotation(self.position)
        kpool = cache.k if cache.write else None
        if self.q_rank:
            # the norms of both compressed vectors and the cache write (the queries' vector is one "head" of q_rank
            # numbers here), then the queries' expansion
            kernels.head_prepare(q, 1, self.q_rank, row, 1, self.row_dim, ctx.positions, kvctx.slot_mapping, kpool,
                                 ctx.page_size, q_gain=self.q_gain, q_norm_dims=self.q_rank, k_gain=self.latent_gain,
                                 k_norm_dims=kr, eps=s.norm_eps)
            q = self.q_up(q, rt.ws.take("latent_q", (n, self.q_width), rt.act_dtype))
        else:
            # norm of the compressed part, rotation of the shared key part and of every head's rotated part, cache write
            kernels.head_prepare(q, H, self.q_dim, row, 1, self.row_dim, ctx.positions, kvctx.slot_mapping, kpool,
                                 ctx.page_size, k_gain=self.latent_gain, k_norm_dims=kr, eps=s.norm_eps,
                                 inv_freq=inv_freq, rot_dims=rot_dims, q_rot_off=s.head_dim, k_rot_off=kr,
                                 neighbours=neighbours, mult=mult)
        qc = rt.ws.take("latent_qc", (n, H * self.row_dim), rt.act_dtype)
        heads_product(q, self.q_dim, self.absorb, qc, self.row_dim)
        mixed = rt.ws.take("latent_mixed", (n, H * kr), rt.act_dtype)
        attend_float32(qc, mixed, cache.k, cache.k, ctx, kvctx, H, 1, self.row_dim, kr, float(s.scale), s.chunk,
                       n_v_heads=1, v_row=self.row_dim, window=s.window, sink=self.sink)
        heads = rt.ws.take("latent_heads", (n, H * s.v_head_dim), rt.act_dtype)
        heads_product(mixed, kr, self.expand, heads, s.v_head_dim)
        if self.gate_width:
            # a head's output times sigmoid of its gate
            kernels.gate_mul(heads, proj[:, cols[2]:cols[2] + H], group=s.v_head_dim)
        return self.o(heads, rt.ws.take("mixer_out", (n, s.hidden), rt.act_dtype))



@register_mixer("differential_attention")
class DifferentialAttention:
    graph_safe = True

    @staticmethod
    def expected_tensors(spec):
        H, G, d, dv = spec.n_heads, spec.n_kv_heads, spec.head_dim, spec.v_head_dim
        out = {
            spec.q_proj: ExpectedTensor((H * 2 * d, spec.hidden)),
            spec.k_proj: ExpectedTensor((G * 2 * d, spec.hidden)),
            spec.v_proj: ExpectedTensor((G * dv, spec.hidden)),
        }
        for name in (spec.q_norm, spec.k_norm):
            if name is not None:
                out[name] = ExpectedTensor((d,), init="gain")
        for name in (spec.lambda_q1, spec.lambda_k1, spec.lambda_q2, spec.lambda_k2):
            out[name] = ExpectedTensor((d,))
        out.update(position_class(spec.position).expected_tensors(spec.position))
        if spec.gate_proj is not None:
            out[spec.gate_proj] = ExpectedTensor((H * dv, spec.hidden))
        out[spec.o_proj] = ExpectedTensor((spec.hidden, H * dv))
        return out

    def __init__(self, spec, tensors, rt):
        H, G, d, dv = spec.n_heads, spec.n_kv_heads, spec.head_dim, spec.v_head_dim
        if H % G:
            raise ValueError(f"{H} query heads are not a multiple of {G} kv heads")
        if d > 256 or dv > 256:
            raise ValueError(f"attention kernels take head sizes up to 256, not {d} and {dv}")
        self.spec = spec
        self.rt = rt
        rep = H // G
        self.position = build_position(spec.position, tensors, rt)
        _, rot_dims, _, _ = _rotation(self.position)
        if rot_dims > d:
            raise ValueError(f"the rotation turns {rot_dims} dimensions, a map has {d}")
        wq = tensors[spec.q_proj]
        # query rows from [head, map] to [kv head, map, head in group]: the heads that read one key head side by side
        wq = wq.view(G, rep, 2, d, spec.hidden).permute(0, 2, 1, 3, 4).reshape(H * 2 * d, spec.hidden)
        ws = [wq, tensors[spec.k_proj], tensors[spec.v_proj]] + ([tensors[spec.gate_proj]] if spec.gate_proj is not None else [])
        dtype = _common_dtype(ws)
        self.proj = Linear(torch.cat([w.to(dtype) for w in ws], dim=0).contiguous(), rt, "diff_proj")
        self.q_width, self.k_width, self.v_width, self.out_width = 2 * H * d, 2 * G * d, G * dv, H * dv
        self.proj_width = self.q_width + self.k_width + self.v_width + (self.out_width if spec.gate_proj is not None else 0)
        gains = [tensors[n] for n in (spec.q_norm, spec.k_norm) if n is not None]
        gdtype = _common_dtype(gains) if gains else None
        self.q_gain = tensors[spec.q_norm].to(gdtype).contiguous() if spec.q_norm is not None else None
        self.k_gain = tensors[spec.k_norm].to(gdtype).contiguous() if spec.k_norm is not None else None
        f = lambda name: tensors[name].double()
        self.lam = float(torch.exp((f(spec.lambda_q1) * f(spec.lambda_k1)).sum())
                         - torch.exp((f(spec.lambda_q2) * f(spec.lambda_k2)).sum()) + spec.lambda_init)
        self.o = Linear(tensors[spec.o_proj], rt, "o")

    def cache_requirement(self) -> CacheRequirement:
        s = self.spec
        return CacheRequirement(kind="kv", n_kv_heads=2 * s.n_kv_heads, head_dim=s.head_dim, v_head_dim=s.v_head_dim,
                                dtype=self.rt.act_dtype, n_v_heads=s.n_kv_heads, chunk=s.chunk)

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        s, rt = self.spec, self.rt
        n = x.shape[0]
        H, G, d, dv = s.n_heads, s.n_kv_heads, s.head_dim, s.v_head_dim
        proj = self.proj(x, rt.ws.take("diff_proj", (n, self.proj_width), rt.act_dtype))
        a, b, c = self.q_width, self.q_width + self.k_width, self.q_width + self.k_width + self.v_width
        q, k, v = proj[:, :a], proj[:, a:b], proj[:, b:c]
        gate = proj[:, c:] if s.gate_proj is not None else None
        kvctx = ctx.kv[cache.group]
        inv_freq, rot_dims, neighbours, mult = _rotation(self.position)
        kpool, vpool = (cache.k, cache.v) if cache.write else (None, None)
        kernels.head_prepare(q, 2 * H, d, k, 2 * G, d, ctx.positions, kvctx.slot_mapping, kpool, ctx.page_size,
                             q_gain=self.q_gain, q_norm_dims=d, k_gain=self.k_gain, k_norm_dims=d, eps=s.norm_eps,
                             inv_freq=inv_freq, rot_dims=rot_dims, neighbours=neighbours, mult=mult, v=v, vpool=vpool,
                             n_v_heads=G, v_head_dim=dv)
        maps = rt.ws.take("diff_maps", (n, 2 * H * dv), rt.act_dtype)
        attend_float32(q, maps, cache.k, cache.v, ctx, kvctx, 2 * H, 2 * G, d, dv, float(s.scale), s.chunk, n_v_heads=G)
        out = rt.ws.take("diff_out", (n, self.out_width), rt.act_dtype)
        kernels.diff_combine(maps, gate, out, H, G, dv, self.lam, s.norm_eps, 1.0 - s.lambda_init)
        return self.o(out, rt.ws.take("mixer_out", (n, s.hidden), rt.act_dtype))
