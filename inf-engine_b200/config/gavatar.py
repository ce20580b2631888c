"""Typed configuration of the Gavatar decoder, read from ``config.json``.

A Gavatar model multiplies its token embedding by a constant and adds a sinusoidal position vector, runs layers with a
norm before AND after each sublayer (``x += norm_b(part(norm_a(x)))``, every norm an RMS norm whose stored weight lies
around zero), may run a group of neighbouring layers several times in a row with the same weights (a cache or state per
pass; a learned vector of the pass is added to the stream before each pass, the first too), and ends in the same kind
of norm and an untied head.  What a layer's mixer reads is first blended with the previous token's input (token shift,
a learned weight per coordinate).  Three kinds of mixer, in whatever order the file lists the layers:

* ``attention``: grouped-query attention without positions under a sliding window; biases on q, k and v; every query,
  key and value head divided by its root mean square; the softmax weights mixed across heads by a learned matrix; an
  output gate per coordinate.
* ``latent_attention``: queries, keys and values expanded from compressed, normed vectors (only the key/value vector is
  cached); a sliding window; a learned sink in the softmax's denominator; an output gate per head.
* ``mlstm``: the matrix memory of xLSTM with capped, stabilised exponential gates.

The feed-forward is a mixture of gated experts: the experts with the largest router logits, weighted by the softmax
over the chosen logits alone.

    {"architecture": "Gavatar", "vocab": V, "width": d, "norm": {"eps": e}, "embedding": {"scale": s},
     "loop": {"start": a, "stop": b, "times": n},
     "layers": [{"type": "attention", "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "mask": {"size"}}, "mlp": M | null},
                {"type": "latent_attention", "mixer": {"heads", "dim", "vdim", "q_rank", "kv_rank", "scale", "mask": {"size"}}, "mlp": M | null},
                {"type": "mlstm", "mixer": {"heads", "dim", "vdim", "gate_cap"}, "mlp": M | null}]}
    M = {"kind": "moe", "expert": {"ff": f}, "router": {"experts": E, "top": k}}

Tensor names: ``embed``, ``loop.step``, ``l<i>.norm1``, ``l<i>.norm1b``, ``l<i>.norm2``, ``l<i>.norm2b``, ``l<i>.shift``,
``l<i>.mix.*``, ``l<i>.mlp.router`` (+ ``.b``), ``l<i>.mlp.e<j>.gate|up|down``, ``final.norm``, ``head``.
"""

from __future__ import annotations

from dataclasses import dataclass, field

from .fovunex import NO_POSITION_LIMIT, _need, _nonneg_int, _pos_int
from .llama import ConfigError
from .spec import (
    BlockSpec,
    LatentAttentionSpec,
    MatrixMemorySpec,
    NormSpec,
    PassOffsetDecoderSpec,
    RoutedExpertsSpec,
    ScheduleEntry,
    TalkingAttentionSpec,
)

# The design fixes these.
SINUSOID_BASE = 10000.0         # the position vector's angles are p * 10000^(-2i / width)
PASS_OFFSETS = "loop.step"      # tensor [times, width]: row t is added to the stream before pass t


@dataclass(frozen=True)
class GavatarMoE:
    experts: int
    top: int
    ff: int


@dataclass(frozen=True)
class GavatarAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int | None = None


@dataclass(frozen=True)
class GavatarLatent:
    heads: int
    dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    window: int | None = None


@dataclass(frozen=True)
class GavatarMLSTM:
    heads: int
    dim: int
    vdim: int
    gate_cap: float


@dataclass(frozen=True)
class GavatarLayer:
    type: str                                   # "attention" | "latent_attention" | "mlstm"
    mixer: object = None
    mlp: GavatarMoE | None = None
    shift: bool = True                          # whether the layer has a token-shift weight


def _parse_window(mask, where: str) -> int | None:
    if not mask:
        return None
    return _pos_int(_need(mask, "size", where), where + ".size")


def _parse_mlp(mlp, where: str) -> GavatarMoE | None:
    if mlp is None:
        return None
    kind = _need(mlp, "kind", where)
    if kind != "moe":
        raise ConfigError(f"config.json: {where}.kind {kind!r} is not built (known: moe)")
    router = _need(mlp, "router", where)
    experts = _pos_int(_need(router, "experts", where + ".router"), where + ".router.experts")
    top = _pos_int(_need(router, "top", where + ".router"), where + ".router.top")
    if top > experts:
        raise ConfigError(f"config.json: {where}.router: {top} of {experts} experts cannot be chosen")
    ff = _pos_int(_need(_need(mlp, "expert", where), "ff", where + ".expert"), where + ".expert.ff")
    return GavatarMoE(experts, top, ff)


@dataclass(frozen=True)
class GavatarConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float = 1.0
    layers: tuple[GavatarLayer, ...] = field(default_factory=tuple)
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1
    eos_token_id: int | None = None

    # names other parts of the package ask a configuration for
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    @property
    def max_position_embeddings(self) -> int:
        return NO_POSITION_LIMIT

    # ---- reading and writing config.json
    @classmethod
    def from_dict(cls, d: dict, tensor_shapes: dict | None = None) -> "GavatarConfig":
        """``tensor_shapes`` (name -> shape of the checkpoint beside the file, optional) settles what the file leaves to
        the tensors: the queries' compressed size when ``q_rank`` is absent, and whether a layer shifts its inputs."""
        shapes = tensor_shapes or {}
        vocab = _pos_int(_need(d, "vocab", "the top level"), "vocab")
        width = _pos_int(_need(d, "width", "the top level"), "width")
        eps = float(_need(_need(d, "norm", "the top level"), "eps", "'norm'"))
        if not eps > 0:
            raise ConfigError("config.json: norm.eps must be positive")
        emb = d.get("embedding") or {}
        raw = _need(d, "layers", "the top level")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, e in enumerate(raw):
            where = f"layers[{i}]"
            kind = _need(e, "type", where)
            m = _need(e, "mixer", where)
            mw = where + ".mixer"
            mlp = _parse_mlp(e.get("mlp"), where + ".mlp")
            if kind in ("attention", "latent_attention", "mlstm"):
                heads = _pos_int(_need(m, "heads", mw), mw + ".heads")
                dim = _pos_int(_need(m, "dim", mw), mw + ".dim")
                vdim = _pos_int(m.get("vdim", dim), mw + ".vdim")
            if kind == "attention":
                kv = _pos_int(m.get("kv_heads", heads), mw + ".kv_heads")
                if heads % kv:
                    raise ConfigError(f"config.json: {mw}: {heads} heads are not a multiple of {kv} kv_heads")
                mixer = GavatarAttention(heads, kv, dim, vdim, float(m.get("scale", dim ** -0.5)),
                                         _parse_window(m.get("mask"), mw + ".mask"))
            elif kind == "latent_attention":
                q_rank = m.get("q_rank")
                if q_rank is None and f"l{i}.mix.dq" in shapes:
                    q_rank = shapes[f"l{i}.mix.dq"][0]
                if q_rank is None:
                    raise ConfigError(f"config.json: {mw} lacks 'q_rank'")
                mixer = GavatarLatent(heads, dim, vdim, _pos_int(q_rank, mw + ".q_rank"),
                                      _pos_int(_need(m, "kv_rank", mw), mw + ".kv_rank"),
                                      float(m.get("scale", dim ** -0.5)), _parse_window(m.get("mask"), mw + ".mask"))
            elif kind == "mlstm":
                cap = float(_need(m, "gate_cap", mw))
                if not cap > 0:
                    raise ConfigError(f"config.json: {mw}.gate_cap must be positive")
                mixer = GavatarMLSTM(heads, dim, vdim, cap)
            else:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not built (known: attention, latent_attention, mlstm)")
            shift = bool(e.get("shift", True)) and (not shapes or f"l{i}.shift" in shapes)
            layers.append(GavatarLayer(kind, mixer, mlp, shift))
        loop = d.get("loop")
        start, stop, times = 0, 0, 1
        if loop:
            start = _nonneg_int(_need(loop, "start", "'loop'"), "loop.start")
            stop = _nonneg_int(_need(loop, "stop", "'loop'"), "loop.stop")
            times = _pos_int(_need(loop, "times", "'loop'"), "loop.times")
            if not start <= stop <= len(layers):
                raise ConfigError(f"config.json: loop {start}..{stop} does not lie within the {len(layers)} layers")
            if start == stop:
                start, stop, times = 0, 0, 1
        return cls(architecture=str(d.get("architecture") or (d.get("architectures") or ["Gavatar"])[0]), vocab=vocab,
                   width=width, norm_eps=eps, embedding_scale=float(emb.get("scale", 1.0)), layers=tuple(layers),
                   loop_start=start, loop_stop=stop, loop_times=times, eos_token_id=d.get("eos_token_id"))

    def to_hf_dict(self) -> dict:
        layers = []
        for L in self.layers:
            x = L.mixer
            if L.type == "attention":
                mixer = {"heads": x.heads, "kv_heads": x.kv_heads, "dim": x.dim, "vdim": x.vdim, "scale": x.scale}
            elif L.type == "latent_attention":
                mixer = {"heads": x.heads, "dim": x.dim, "vdim": x.vdim, "q_rank": x.q_rank, "kv_rank": x.kv_rank,
                         "scale": x.scale}
            else:
                mixer = {"heads": x.heads, "dim": x.dim, "vdim": x.vdim, "gate_cap": x.gate_cap}
            if L.type != "mlstm" and x.window is not None:
                mixer["mask"] = {"size": x.window}
            mlp = None if L.mlp is None else {"kind": "moe", "expert": {"ff": L.mlp.ff},
                                              "router": {"experts": L.mlp.experts, "top": L.mlp.top}}
            entry = {"type": L.type, "mixer": mixer, "mlp": mlp}
            if not L.shift:
                entry["shift"] = False
            layers.append(entry)
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "norm": {"eps": self.norm_eps}, "embedding": {"scale": self.embedding_scale}, "layers": layers}
        if self.loop_stop > self.loop_start:
            out["loop"] = {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}
        if self.eos_token_id is not None:
            out["eos_token_id"] = self.eos_token_id
        return out

    to_dict = to_hf_dict

    # ---- the model as data
    def _norm(self, name: str) -> NormSpec:
        return NormSpec("rmsnorm", self.width, self.norm_eps, name, unit_offset=True)

    def _mixer_spec(self, L: GavatarLayer, m: str):
        x = L.mixer
        if L.type == "attention":
            return TalkingAttentionSpec(
                kind="talking_attention", hidden=self.width, n_heads=x.heads, n_kv_heads=x.kv_heads, head_dim=x.dim,
                v_head_dim=x.vdim, scale=x.scale, norm_eps=self.norm_eps, qk_norm=True, v_norm=True, window=x.window,
                q_proj=m + "q", k_proj=m + "k", v_proj=m + "v", q_bias=m + "q.b", k_bias=m + "k.b", v_bias=m + "v.b",
                talk=m + "talk", gate_proj=m + "g", o_proj=m + "o")
        if L.type == "latent_attention":
            return LatentAttentionSpec(
                kind="latent_attention", hidden=self.width, n_heads=x.heads, head_dim=x.dim, rot_dim=0,
                v_head_dim=x.vdim, kv_rank=x.kv_rank, scale=x.scale, norm_eps=self.norm_eps, q_proj=m + "uq",
                down_proj=m + "dkv", latent_norm=m + "dkv.norm", k_up=m + "uk", v_up=m + "uv", o_proj=m + "o",
                q_rank=x.q_rank, q_down=m + "dq", q_norm=m + "dq.norm", window=x.window, sink=m + "sink",
                head_gate=m + "g")
        return MatrixMemorySpec(
            kind="matrix_memory", hidden=self.width, n_heads=x.heads, head_dim=x.dim, v_head_dim=x.vdim,
            gate_cap=x.gate_cap, norm_eps=self.norm_eps, q_proj=m + "q", k_proj=m + "k", v_proj=m + "v",
            i_proj=m + "i", i_bias=m + "i.b", f_proj=m + "f", f_bias=m + "f.b", gate_proj=m + "g",
            out_gain=m + "norm", o_proj=m + "o")

    def run_order(self) -> list[tuple[int, int | None]]:
        """(layer, number of the pass that begins with this run or None) for every run of a layer, in order."""
        n = len(self.layers)
        if self.loop_stop <= self.loop_start:
            return [(i, None) for i in range(n)]
        order = [(i, None) for i in range(self.loop_start)]
        for t in range(self.loop_times):
            order += [(i, t if i == self.loop_start else None) for i in range(self.loop_start, self.loop_stop)]
        return order + [(i, None) for i in range(self.loop_stop, n)]

    def model_spec(self) -> PassOffsetDecoderSpec:
        layers = []
        for i, L in enumerate(self.layers):
            p = f"l{i}."
            if L.mlp is None:
                ff_norm, ff_out_norm, ff = None, None, None
            else:
                f = p + "mlp."
                ff_norm, ff_out_norm = self._norm(p + "norm2"), self._norm(p + "norm2b")
                ff = RoutedExpertsSpec(kind="routed_experts", hidden=self.width, intermediate=L.mlp.ff,
                                       n_experts=L.mlp.experts, top=L.mlp.top, router=f + "router", expert_prefix=f + "e",
                                       score="softmax_top", router_bias=f + "router.b")
            layers.append(BlockSpec(kind="sandwich", mixer_norm=self._norm(p + "norm1"),
                                    mixer=self._mixer_spec(L, p + "mix."), ff_norm=ff_norm, feedforward=ff,
                                    mixer_out_norm=self._norm(p + "norm1b"), ff_out_norm=ff_out_norm,
                                    token_shift=p + "shift" if L.shift else None))
        order = self.run_order()
        looped = self.loop_stop > self.loop_start
        return PassOffsetDecoderSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden=self.width, max_positions=NO_POSITION_LIMIT,
            embedding="embed", layers=tuple(layers), schedule=tuple(ScheduleEntry(layer=i) for i, _ in order),
            final_norm=self._norm("final.norm"), head="head", embedding_scale=self.embedding_scale,
            sinusoid_base=SINUSOID_BASE, pass_offsets=PASS_OFFSETS if looped else None,
            offset_before=tuple((k, t) for k, (_, t) in enumerate(order) if t is not None),
            optional_tensors=() if looped else (PASS_OFFSETS,))
