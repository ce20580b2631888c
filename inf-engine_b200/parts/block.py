"""Residual blocks.  The pre-norm block: ``x += mixer(norm(x)); x += ff(norm(x))``
(engine/llama_block.py:50-62); beside it a block that norms its sublayers' outputs, a pre-norm block with gates per
coordinate, and a block with a norm before and after each sublayer whose mixer may read shifted inputs.  The sums are folded into the norm that follows
them: a block hands on the residual and a delta that is not added yet.  A block
whose spec has no feed-forward is the first half alone."""

from __future__ import annotations

from .. import kernels
from ..weights.loader import ExpectedTensor
from .linear import Linear
from .registry import (
    build_feedforward,
    build_mixer,
    build_norm,
    feedforward_class,
    mixer_class,
    norm_class,
    register_block,
)


@register_block("prenorm")
class PreNormBlock:
    @staticmethod
    def expected_tensors(spec):
        out = {}
        out.update(norm_class(spec.mixer_norm).expected_tensors(spec.mixer_norm))
        out.update(mixer_class(spec.mixer).expected_tensors(spec.mixer))
        if spec.feedforward is not None:
            out.update(norm_class(spec.ff_norm).expected_tensors(spec.ff_norm))
            out.update(feedforward_class(spec.feedforward).expected_tensors(spec.feedforward))
        return out

    def __init__(self, spec, tensors, rt):
        self.spec = spec
        self.mixer_norm = build_norm(spec.mixer_norm, tensors, rt)
        self.mixer = build_mixer(spec.mixer, tensors, rt)
        self.ff_norm = build_norm(spec.ff_norm, tensors, rt) if spec.feedforward is not None else None
        self.feedforward = build_feedforward(spec.feedforward, tensors, rt) if spec.feedforward is not None else None

    @property
    def graph_safe(self) -> bool:
        """Whether a step through this block may be captured as a CUDA graph: every part says that it reads the
        batch's numbers on the device only and never waits for the device (a part that says nothing does not)."""
        return all(getattr(p, "graph_safe", False) for p in (self.mixer, self.feedforward) if p is not None)

    def forward(self, residual, pending, ctx, cache):
        n = ctx.n_tokens
        ctx.residual_cast = None      # this block changes the residual without keeping a cast copy of it
        # a part may offer forward_fused(residual, norm, ...): it applies the norm and adds its own
        # result into the residual inside its kernels (worth it for the few rows of a decode step)
        # ctx.upcoming_norm tells a fused part which norm follows its product into the residual (it may prepare
        # that norm's input); ctx.handover is what the part before prepared, void as soon as the residual changes
        after_block = getattr(ctx, "norm_after_block", None)
        ff_fuses = self.feedforward is not None and _fuses(self.feedforward, n, self.ff_norm)
        if _fuses(self.mixer, n, self.mixer_norm):
            if pending is not None:
                kernels.residual_add(residual, pending)
                ctx.handover = None
            ctx.upcoming_norm = self.ff_norm if ff_fuses else None
            self.mixer.forward_fused(residual, self.mixer_norm, ctx, cache)
            a = None
        else:
            ctx.handover = None
            h = self.mixer_norm.add_norm(residual, pending)
            a = self.mixer.forward(h, ctx, cache)
        if self.feedforward is None:
            ctx.handover = None
            ctx.upcoming_norm = None
            return residual, a
        if ff_fuses:
            if a is not None:
                kernels.residual_add(residual, a)
                ctx.handover = None
            ctx.upcoming_norm = after_block
            self.feedforward.forward_fused(residual, self.ff_norm, ctx)
            ctx.upcoming_norm = None
            return residual, None
        ctx.handover = None
        ctx.upcoming_norm = None
        h = self.ff_norm.add_norm(residual, a)
        m = self.feedforward.forward(h, ctx)
        return residual, m


@register_block("outnorm")
class OutputNormBlock:
    """``x += norm1(mixer(x)); x += norm2(ff(x))``: the sublayers read the residual stream itself and the norm sits
    on what they return.  The residual is float32; a sublayer's input is its rows in the activation type (the
    residual itself on the 32-bit path), which the norm kernel of the sublayer before leaves behind as it adds."""

    @staticmethod
    def expected_tensors(spec):
        return PreNormBlock.expected_tensors(spec)

    def __init__(self, spec, tensors, rt):
        self.spec = spec
        self.rt = rt
        self.mixer_norm = build_norm(spec.mixer_norm, tensors, rt)
        self.mixer = build_mixer(spec.mixer, tensors, rt)
        self.ff_norm = build_norm(spec.ff_norm, tensors, rt) if spec.feedforward is not None else None
        self.feedforward = build_feedforward(spec.feedforward, tensors, rt) if spec.feedforward is not None else None
        for norm in (self.mixer_norm, self.ff_norm):
            if norm is not None and not hasattr(norm, "accumulate"):
                raise ValueError(f"a block that norms its sublayers' outputs needs a norm with accumulate(); "
                                 f"{type(norm).__name__} has none")

    @property
    def graph_safe(self) -> bool:
        return all(getattr(p, "graph_safe", False) for p in (self.mixer, self.feedforward) if p is not None)

    def _input(self, residual, ctx):
        """The residual rows as a sublayer reads them."""
        if self.rt.exact:
            return residual
        if ctx.residual_cast is None:
            ctx.residual_cast = self.rt.ws.take("block_in", tuple(residual.shape), self.rt.act_dtype)
            kernels.cast_rows(residual, ctx.residual_cast)
        return ctx.residual_cast

    def _next_input(self, residual, wanted: bool):
        if self.rt.exact or not wanted:
            return None
        return self.rt.ws.take("block_in", tuple(residual.shape), self.rt.act_dtype)

    def forward(self, residual, pending, ctx, cache):
        ctx.handover = None
        ctx.upcoming_norm = None
        if pending is not None:
            kernels.residual_add(residual, pending)
            ctx.residual_cast = None
        a = self.mixer.forward(self._input(residual, ctx), ctx, cache)
        last = getattr(ctx, "last_block", False)
        nxt = self._next_input(residual, self.feedforward is not None or not last)
        self.mixer_norm.accumulate(residual, a, nxt)
        ctx.residual_cast = nxt
        if self.feedforward is not None:
            m = self.feedforward.forward(self._input(residual, ctx), ctx)
            nxt = self._next_input(residual, not last)
            self.ff_norm.accumulate(residual, m, nxt)
            ctx.residual_cast = nxt
        return residual, None


@register_block("gated_prenorm")
class GatedPreNormBlock:
    """``x += sigmoid(W1 h + b1) * mixer(h)`` with h = norm1(x), then ``x += sigmoid(W2 h + b2) * ff(h)`` with h =
    norm2(x): a pre-norm block whose sublayers' results pass a gate per coordinate that reads what the sublayer reads.
    The gate's product is in the activation type; the sigmoid, the product with the sublayer's result and the sum
    into the residual are one float32 kernel.  A sublayer without a gate tensor is added as it is."""

    @staticmethod
    def expected_tensors(spec):
        d = spec.mixer_norm.size
        out = {}
        out.update(norm_class(spec.mixer_norm).expected_tensors(spec.mixer_norm))
        out.update(mixer_class(spec.mixer).expected_tensors(spec.mixer))
        if spec.feedforward is not None:
            out.update(norm_class(spec.ff_norm).expected_tensors(spec.ff_norm))
            out.update(feedforward_class(spec.feedforward).expected_tensors(spec.feedforward))
        for w, b, there in ((spec.mixer_gate, spec.mixer_gate_bias, True),
                            (spec.ff_gate, spec.ff_gate_bias, spec.feedforward is not None)):
            if there and w is not None:
                out[w] = ExpectedTensor((d, d))
                if b is not None:
                    out[b] = ExpectedTensor((d,))
        return out

    def __init__(self, spec, tensors, rt):
        self.spec = spec
        self.rt = rt
        self.mixer_norm = build_norm(spec.mixer_norm, tensors, rt)
        self.mixer = build_mixer(spec.mixer, tensors, rt)
        self.ff_norm = build_norm(spec.ff_norm, tensors, rt) if spec.feedforward is not None else None
        self.feedforward = build_feedforward(spec.feedforward, tensors, rt) if spec.feedforward is not None else None

        def gate(w, b, name):
            if w is None:
                return None, None
            return Linear(tensors[w], rt, name), (tensors[b].contiguous() if b is not None else None)

        self.mixer_gate, self.mixer_gate_bias = gate(spec.mixer_gate, spec.mixer_gate_bias, "mixer_gate")
        self.ff_gate, self.ff_gate_bias = gate(spec.ff_gate, spec.ff_gate_bias, "ff_gate") \
            if spec.feedforward is not None else (None, None)

    @property
    def graph_safe(self) -> bool:
        return all(getattr(p, "graph_safe", False) for p in (self.mixer, self.feedforward) if p is not None)

    def _add(self, residual, y, h, gate, bias):
        if gate is None:
            kernels.residual_add(residual, y)
            return
        g = gate(h, self.rt.ws.take("sublayer_gate", tuple(y.shape), self.rt.act_dtype))
        kernels.gated_residual_add(residual, y, g, bias)

    def forward(self, residual, pending, ctx, cache):
        ctx.handover = None
        ctx.upcoming_norm = None
        ctx.residual_cast = None
        h = self.mixer_norm.add_norm(residual, pending)
        self._add(residual, self.mixer.forward(h, ctx, cache), h, self.mixer_gate, self.mixer_gate_bias)
        if self.feedforward is not None:
            h = self.ff_norm.add_norm(residual, None)
            self._add(residual, self.feedforward.forward(h, ctx), h, self.ff_gate, self.ff_gate_bias)
        return residual, None


@register_block("sandwich")
class SandwichBlock:
    """``x += out_norm1(mixer(shift(norm1(x))))``, then ``x += out_norm2(ff(norm2(x)))``: a norm before and a norm after
    each sublayer.  ``shift`` (optional) replaces the mixer's input h by ``h + (h' - h) * mu`` with h' the h of the
    token before and mu a learned vector; the last h of every request is state of the run, kept beside the mixer's own
    cache (the run's requirement is then the pair, the mixer's first).  The residual is float32; the norm after a
    sublayer and the sum into the residual are one kernel, which after the mixer also forms the feed-forward's normed
    input."""

    @staticmethod
    def expected_tensors(spec):
        out = {}
        out.update(norm_class(spec.mixer_norm).expected_tensors(spec.mixer_norm))
        if spec.feedforward is not None:
            out.update(norm_class(spec.ff_norm).expected_tensors(spec.ff_norm))
        out.update(norm_class(spec.mixer_out_norm).expected_tensors(spec.mixer_out_norm))
        if spec.feedforward is not None:
            out.update(norm_class(spec.ff_out_norm).expected_tensors(spec.ff_out_norm))
        out.update(mixer_class(spec.mixer).expected_tensors(spec.mixer))
        if spec.feedforward is not None:
            out.update(feedforward_class(spec.feedforward).expected_tensors(spec.feedforward))
        if spec.token_shift is not None:
            out[spec.token_shift] = ExpectedTensor((spec.mixer_norm.size,))
        return out

    def __init__(self, spec, tensors, rt):
        self.spec = spec
        self.rt = rt
        self.mixer_norm = build_norm(spec.mixer_norm, tensors, rt)
        self.mixer_out_norm = build_norm(spec.mixer_out_norm, tensors, rt)
        self.mixer = build_mixer(spec.mixer, tensors, rt)
        has_ff = spec.feedforward is not None
        self.ff_norm = build_norm(spec.ff_norm, tensors, rt) if has_ff else None
        self.ff_out_norm = build_norm(spec.ff_out_norm, tensors, rt) if has_ff else None
        self.feedforward = build_feedforward(spec.feedforward, tensors, rt) if has_ff else None
        for norm in (self.mixer_out_norm, self.ff_out_norm):
            if norm is not None and not hasattr(norm, "accumulate"):
                raise ValueError(f"the norm after a sublayer needs accumulate(); {type(norm).__name__} has none")
        self.shift = tensors[spec.token_shift].contiguous() if spec.token_shift is not None else None

    @property
    def graph_safe(self) -> bool:
        return all(getattr(p, "graph_safe", False) for p in (self.mixer, self.feedforward) if p is not None)

    def cache_requirement(self):
        """The mixer's requirement, and beside it the last input row of every request when inputs are shifted."""
        from ..cache.manager import CacheRequirement
        own = self.mixer.cache_requirement()
        if self.shift is None:
            return own
        last = CacheRequirement(kind="state", state_shape=(self.spec.mixer_norm.size,), state_dtype=self.rt.act_dtype)
        return CacheRequirement(kind="several", parts=(own, last))

    def forward(self, residual, pending, ctx, cache):
        ctx.handover = None
        ctx.upcoming_norm = None
        ctx.residual_cast = None
        h = self.mixer_norm.add_norm(residual, pending)
        mixer_cache = cache
        if self.shift is not None:
            mixer_cache, last = cache.parts
            shifted = self.rt.ws.take("shifted", tuple(h.shape), self.rt.act_dtype)
            kernels.token_shift(h, shifted, self.shift, last.state, ctx.q_start, ctx.ctx_before, ctx.slots,
                                ctx.n_requests, write_state=cache.write)
            h = shifted
        y = self.mixer.forward(h, ctx, mixer_cache)
        if self.feedforward is None:
            self.mixer_out_norm.accumulate(residual, y)
            return residual, None
        # the norm after the mixer, the sum into the residual and the norm before the feed-forward: one kernel
        fused = getattr(self.mixer_out_norm, "accumulate_then_norm", None)
        h = fused(residual, y, self.ff_norm) if fused is not None else None
        if h is None:
            self.mixer_out_norm.accumulate(residual, y)
            h = self.ff_norm.add_norm(residual, None)
        self.ff_out_norm.accumulate(residual, self.feedforward.forward(h, ctx))
        return residual, None


def _fuses(part, n_tokens: int, norm) -> bool:
    can = getattr(part, "can_fuse", None)
    return bool(can and can(n_tokens, norm))
