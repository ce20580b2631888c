"""A decoder put together from parts: token table, blocks run in the order of
the schedule, final norm on the rows whose logits are wanted, head
(engine/llama_model.py:128-149).  The reference computes logits for every
position (:148); here the head runs on the gathered rows only and its result
is float32."""

from __future__ import annotations

import torch

from .. import kernels
from ..cache.manager import CacheManager, CacheRequirement
from .attention import CacheView
from .linear import Linear, stream_normed
from ..weights.loader import ExpectedTensor
from .registry import block_class, build_block, build_norm, norm_class, register_model


@register_model("decoder")
class DecoderModel:
    @staticmethod
    def expected_tensors(spec) -> dict:
        """The token table, the layers in order, the final norm, the head."""
        out = {spec.embedding: ExpectedTensor((spec.vocab_size, spec.hidden))}
        for blk in spec.layers:
            out.update(block_class(blk).expected_tensors(blk))
        out.update(norm_class(spec.final_norm).expected_tensors(spec.final_norm))
        if spec.head is not None:
            out[spec.head] = ExpectedTensor((spec.vocab_size, spec.hidden))
        return out

    def __init__(self, spec, tensors: dict, rt):
        self.spec = spec
        self.rt = rt
        self.embedding = tensors[spec.embedding]
        self.layers = [build_block(b, tensors, rt) for b in spec.layers]
        self.final_norm = build_norm(spec.final_norm, tensors, rt)
        head = tensors[spec.head] if spec.head is not None else self.embedding   # tied: one buffer
        self.head = Linear(head, rt, "head")
        for i, e in enumerate(spec.schedule):
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"schedule entry {i} names layer {e.layer}, the model has {len(self.layers)}")
            if e.cache_from is not None and not (0 <= e.cache_from < i and spec.schedule[e.cache_from].cache_from is None):
                raise ValueError(f"schedule entry {i} must read the cache of an earlier entry that owns one")
        # a decode step is captured as a graph only if every block that runs says it may be
        self.graph_safe = all(getattr(self.layers[e.layer], "graph_safe", False) for e in spec.schedule)
        self._views: list[CacheView] | None = None

    # ------------------------------------------------------------------ cache
    def cache_requirements(self) -> list[CacheRequirement]:
        """One requirement per schedule entry; a run that reads another run's cache needs none."""
        reqs = []
        for e in self.spec.schedule:
            if e.cache_from is not None:
                reqs.append(CacheRequirement(kind="none"))
            else:
                # a block that keeps something of its own beside its mixer's cache says so itself
                blk = self.layers[e.layer]
                reqs.append(blk.cache_requirement() if hasattr(blk, "cache_requirement") else blk.mixer.cache_requirement())
        return reqs

    def bind_cache(self, manager: CacheManager) -> None:
        def view(b, write: bool) -> CacheView:
            if b.kind == "kv":
                g = manager.kv_groups[b.group]
                return CacheView("kv", b.group, g.k[b.row], g.v[b.row], None, write=write)
            if b.kind == "state":
                g = manager.state_groups[b.group]
                return CacheView("state", b.group, None, None, g.data[b.row], write=write)
            if b.kind == "several":
                return CacheView("several", write=write, parts=[view(part, write) for part in b.parts])
            return CacheView("none")

        views = []
        for i, e in enumerate(self.spec.schedule):
            src = i if e.cache_from is None else e.cache_from
            views.append(view(manager.bindings[src], e.cache_from is None))
        self._views = views

    # ---------------------------------------------------------------- forward
    def embed(self, ctx) -> torch.Tensor:
        """The float32 residual stream [n_tokens, hidden] that the first block meets."""
        residual = self.rt.ws.take("residual", (ctx.n_tokens, self.spec.hidden), torch.float32)
        kernels.embed_gather(ctx.token_ids, self.embedding, residual)
        return residual

    def before_entry(self, i: int, residual, pending, ctx):
        """What a derived top level does to the stream right before schedule entry ``i`` runs; nothing here."""
        return residual, pending

    def finish_logits(self, logits: torch.Tensor, ctx) -> torch.Tensor:
        """What a derived top level does to the head's float32 logits (in place) before they leave; nothing here."""
        return logits

    def forward(self, ctx) -> torch.Tensor | None:
        """Run the step's tokens through every scheduled layer; float32 logits
        [n_wanted, vocab] at ``ctx.logit_rows`` (None when nothing is wanted)."""
        assert self._views is not None, "bind_cache() first"
        rt, spec = self.rt, self.spec
        n = ctx.n_tokens
        residual = self.embed(ctx)
        pending = None
        ctx.handover = None
        ctx.residual_cast = None
        last = len(spec.schedule) - 1
        for i, e in enumerate(spec.schedule):
            # the norm that the residual meets after this block: the next block's first, or the final one
            nxt = self.layers[spec.schedule[i + 1].layer] if i < last else None
            ctx.norm_after_block = getattr(nxt, "mixer_norm", None) if nxt is not None else self.final_norm
            ctx.last_block = i == last
            residual, pending = self.before_entry(i, residual, pending, ctx)
            residual, pending = self.layers[e.layer].forward(residual, pending, ctx, self._views[i])
        ctx.norm_after_block = None
        m = ctx.n_logits
        if m == 0:
            return None
        return self.finish_logits(self._head_logits(residual, pending, ctx, n, m), ctx)

    def _head_logits(self, residual, pending, ctx, n: int, m: int) -> torch.Tensor:
        rt, spec = self.rt, self.spec
        logits = rt.ws.take("logits", (m, spec.vocab_size), torch.float32)
        if self.head.streams(m, normed=True) and hasattr(self.final_norm, "fusable_rms"):
            # final norm on the gathered rows inside the head product
            if pending is not None:
                kernels.residual_add(residual, pending)
                ctx.handover = None
            if m == n and getattr(ctx, "handover", None) is not None:
                # every row is wanted (a decode step): the last block may have prepared the final norm's input
                return stream_normed(self.head, residual, logits, m, "f32", self.final_norm, ctx)
            gain, eps = self.final_norm.fusable_rms()
            return self.head.stream(residual, logits, m, "f32", gain, eps, row_index=ctx.logit_rows)
        h = self.final_norm.gather_norm(residual, pending, ctx.logit_rows, m)
        return self.head(h, logits)


@register_model("bigram_decoder")
class BigramDecoderModel(DecoderModel):
    """``DecoderModel`` whose first residual is the token embedding plus a hashed bigram embedding
    (``BigramDecoderSpec``).  The previous token of a sequence is part of its state: one int32 word in a state slot
    of the cache manager beside the layers' caches, read and updated on the device by the embedding kernel, so a
    portion of a prompt, a decoded token and a token whose id is still on the device take the same path."""

    @staticmethod
    def expected_tensors(spec) -> dict:
        out = DecoderModel.expected_tensors(spec)
        first = {spec.embedding: out.pop(spec.embedding), spec.bigram: ExpectedTensor((spec.bigram_buckets + 1, spec.hidden))}
        first.update(out)
        return first

    def __init__(self, spec, tensors: dict, rt):
        super().__init__(spec, tensors, rt)
        if spec.bigram_buckets <= 0:
            raise ValueError("a hashed bigram embedding needs a positive number of buckets")
        self.bigram = tensors[spec.bigram].to(self.embedding.dtype)
        self._prev_token: torch.Tensor | None = None

    def cache_requirements(self) -> list[CacheRequirement]:
        """The layers' requirements and, after them, the model's own: the last token of every request."""
        return super().cache_requirements() + [CacheRequirement(kind="state", state_shape=(1,), state_dtype=torch.int32)]

    def bind_cache(self, manager: CacheManager) -> None:
        super().bind_cache(manager)
        b = manager.bindings[len(self.spec.schedule)]
        self._prev_token = manager.state_groups[b.group].data[b.row].view(-1)     # [max_requests]

    def embed(self, ctx) -> torch.Tensor:
        s = self.spec
        residual = self.rt.ws.take("residual", (ctx.n_tokens, s.hidden), torch.float32)
        kernels.embed_bigram(ctx.token_ids, ctx.positions, ctx.q_start, ctx.slots, ctx.n_requests, self.embedding,
                             self.bigram, self._prev_token, residual, s.bigram_buckets, s.bigram_mul_prev,
                             s.bigram_mul_cur)
        return residual


@register_model("reinject_decoder")
class ReinjectDecoderModel(DecoderModel):
    """``DecoderModel`` whose token embedding is multiplied by a constant and added to the residual stream again right
    before the schedule entries that the spec names (``ReinjectDecoderSpec``): the scaled embedding of the step's
    tokens is kept in a buffer of its own beside the stream."""

    def __init__(self, spec, tensors: dict, rt):
        super().__init__(spec, tensors, rt)
        self.reinject = frozenset(int(i) for i in spec.reinject_before)
        for i in self.reinject:
            if not 0 < i < len(spec.schedule):
                raise ValueError(f"the embedding cannot be added again before schedule entry {i}")
        self._embedded = None

    def embed(self, ctx) -> torch.Tensor:
        residual = super().embed(ctx)
        self._embedded = self.rt.ws.take("embedded", tuple(residual.shape), torch.float32) if self.reinject else None
        if self.spec.embedding_scale != 1.0 or self._embedded is not None:
            kernels.scale_rows(residual, self.spec.embedding_scale, self._embedded)
        return residual

    def before_entry(self, i: int, residual, pending, ctx):
        if i not in self.reinject:
            return residual, pending
        if pending is not None:
            kernels.residual_add(residual, pending)
        kernels.residual_add(residual, self._embedded)
        ctx.handover = None
        ctx.residual_cast = None
        return residual, None


@register_model("pass_offset_decoder")
class PassOffsetDecoderModel(DecoderModel):
    """``DecoderModel`` whose first residual is the token embedding times a constant plus a sinusoidal position vector,
    and which adds a learned vector to the stream right before the schedule entries that the spec names
    (``PassOffsetDecoderSpec``): the vector of a pass before the first layer of every pass of a repeated group."""

    @staticmethod
    def expected_tensors(spec) -> dict:
        out = DecoderModel.expected_tensors(spec)
        if spec.pass_offsets is None:
            return out
        rows = 1 + max((r for _, r in spec.offset_before), default=0)
        first = {spec.embedding: out.pop(spec.embedding), spec.pass_offsets: ExpectedTensor((rows, spec.hidden))}
        first.update(out)
        return first

    def __init__(self, spec, tensors: dict, rt):
        super().__init__(spec, tensors, rt)
        self.offsets = {}
        for entry, row in spec.offset_before:
            if not 0 <= entry < len(spec.schedule) or spec.pass_offsets is None:
                raise ValueError(f"no vector can be added before schedule entry {entry}")
            self.offsets[int(entry)] = tensors[spec.pass_offsets][int(row)].contiguous()

    def embed(self, ctx) -> torch.Tensor:
        residual = super().embed(ctx)
        s = self.spec
        if s.sinusoid_base > 0:
            kernels.scale_add_sinusoid(residual, ctx.positions, s.embedding_scale, s.sinusoid_base)
        elif s.embedding_scale != 1.0:
            kernels.scale_rows(residual, s.embedding_scale)
        return residual

    def before_entry(self, i: int, residual, pending, ctx):
        row = self.offsets.get(i)
        if row is None:
            return residual, pending
        if pending is not None:
            kernels.residual_add(residual, pending)
        kernels.add_row(residual, row)
        ctx.handover = None
        ctx.residual_cast = None
        return residual, None
