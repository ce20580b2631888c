"""Typed configuration of the Fovunex decoder, read from ``config.json``.

A Fovunex model multiplies its token embedding by a constant, runs pre-norm layers whose norm has ONE learned number
as its gain and whose sublayers are gated coordinate by coordinate (``x += sigmoid(W h + b) * part(h)``, h = norm(x)),
may run a group of neighbouring layers several times in a row with the same weights (a cache or state per pass; the
embedding is added to the stream again before every pass but the first), and ends in the same norm and an untied head.
Three kinds of layer, in whatever order the file lists them:

* ``latent_attention``: causal softmax attention whose keys and values are expanded from one compressed vector a token;
  part of every query head and one shared key part are rotated in neighbouring pairs, optionally with frequencies
  blended for a longer context (YaRN).
* ``attention``: grouped-query attention with two score maps a head (differential attention), a norm of every query and
  key map, a rotation in halves of the first dimensions, an optional mask that keeps a query inside its chunk of
  positions, a norm of each head's output and an output gate.
* ``mingru``: a gated recurrence whose gates read the current token only.

The feed-forward is dense with clamped gate and up branches and the activation ``g sigmoid(1.702 g) (u + 1)``.

    {"architecture": "Fovunex", "vocab": V, "width": d, "norm": {"eps": e}, "embedding": {"scale": s},
     "loop": {"start": a, "stop": b, "times": n},
     "layers": [{"type": "latent_attention", "mixer": {"heads", "dim", "rot_dim", "vdim", "kv_rank", "scale",
                                                       "rot": {"base", "dims", "scaling": {"factor", "original", "fast", "slow"}}},
                 "mlp": M | null},
                {"type": "attention", "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "diff",
                                                "rot": {"base", "dims"}, "mask": {"size"}}, "mlp": M | null},
                {"type": "mingru", "mixer": {"width"}, "mlp": M | null}]}
    M = {"kind": "dense", "ff": f, "limit": c}

Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.rg1`` (+ ``.b``), ``l<i>.rg2`` (+ ``.b``), ``l<i>.mix.*``,
``l<i>.mlp.*``, ``final.norm``, ``head``.
"""

from __future__ import annotations

from dataclasses import dataclass, field

from .llama import ConfigError
from .spec import (
    BlockSpec,
    DifferentialAttentionSpec,
    GatedMLPSpec,
    LatentAttentionSpec,
    MinGRUSpec,
    NormSpec,
    PositionSpec,
    ReinjectDecoderSpec,
    ScheduleEntry,
    YarnScaling,
)

# The design fixes these.
SWISH_ALPHA = 1.702             # the feed-forward's activation is g sigmoid(1.702 g)
UP_OFFSET = 1.0                 # ... times (u + 1)
YARN_MULT_SLOPE = 0.1           # cosine and sine of a blended rotation take 0.1 ln(factor) + 1
NO_POSITION_LIMIT = 1 << 30


def _need(d, key: str, where: str):
    if not isinstance(d, dict) or key not in d:
        raise ConfigError(f"config.json: {where} lacks '{key}'")
    return d[key]


def _pos_int(v, what: str) -> int:
    if isinstance(v, float) and v.is_integer():
        v = int(v)
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config.json: {what} must be a positive integer, got {v!r}")
    return v


def _nonneg_int(v, what: str) -> int:
    if isinstance(v, float) and v.is_integer():
        v = int(v)
    if isinstance(v, bool) or not isinstance(v, int) or v < 0:
        raise ConfigError(f"config.json: {what} must be an integer of zero or more, got {v!r}")
    return v


@dataclass(frozen=True)
class FovunexRotation:
    base: float
    dims: int
    scaling: YarnScaling | None = None


@dataclass(frozen=True)
class FovunexMLP:
    ff: int
    limit: float


@dataclass(frozen=True)
class FovunexLatent:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot: FovunexRotation | None = None
    chunk: int | None = None


@dataclass(frozen=True)
class FovunexAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    diff: float
    rot: FovunexRotation | None = None
    chunk: int | None = None


@dataclass(frozen=True)
class FovunexMinGRU:
    width: int


@dataclass(frozen=True)
class FovunexLayer:
    type: str                                   # "latent_attention" | "attention" | "mingru"
    mixer: object = None
    mlp: FovunexMLP | None = None


def _parse_rot(rot, where: str, limit: int) -> FovunexRotation | None:
    if not rot:
        return None
    dims = _nonneg_int(_need(rot, "dims", where), where + ".dims")
    if dims == 0:
        return None
    if dims % 2 or dims > limit:
        raise ConfigError(f"config.json: {where}.dims must be even and at most {limit}, got {dims}")
    base = float(_need(rot, "base", where))
    if not base > 0:
        raise ConfigError(f"config.json: {where}.base must be positive")
    sc = rot.get("scaling")
    scaling = None
    if sc:
        w = where + ".scaling"
        scaling = YarnScaling(factor=float(_need(sc, "factor", w)), original=float(_need(sc, "original", w)),
                              fast=float(_need(sc, "fast", w)), slow=float(_need(sc, "slow", w)),
                              mult_slope=YARN_MULT_SLOPE)
        if not (scaling.factor > 0 and scaling.original > 0 and scaling.fast > 0 and scaling.slow > 0):
            raise ConfigError(f"config.json: {w}: factor, original, fast and slow must be positive")
    return FovunexRotation(base, dims, scaling)


def _parse_chunk(mask, where: str) -> int | None:
    if not mask:
        return None
    return _pos_int(_need(mask, "size", where), where + ".size")


def _parse_mlp(mlp, where: str) -> FovunexMLP | None:
    if mlp is None:
        return None
    kind = _need(mlp, "kind", where)
    if kind != "dense":
        raise ConfigError(f"config.json: {where}.kind {kind!r} is not built (known: dense)")
    limit = float(_need(mlp, "limit", where))
    if not limit > 0:
        raise ConfigError(f"config.json: {where}.limit must be positive")
    return FovunexMLP(_pos_int(_need(mlp, "ff", where), where + ".ff"), limit)


@dataclass(frozen=True)
class FovunexConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float = 1.0
    layers: tuple[FovunexLayer, ...] = field(default_factory=tuple)
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
    def from_dict(cls, d: dict) -> "FovunexConfig":
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
            if kind == "latent_attention":
                heads = _pos_int(_need(m, "heads", mw), mw + ".heads")
                dim = _pos_int(_need(m, "dim", mw), mw + ".dim")
                rot_dim = _nonneg_int(m.get("rot_dim", 0), mw + ".rot_dim")
                rot = m.get("rot")
                if rot and rot_dim:
                    rot = _parse_rot(dict(rot, dims=rot.get("dims", rot_dim)), mw + ".rot", rot_dim)
                    if rot is not None and rot.dims != rot_dim:
                        raise ConfigError(f"config.json: {mw}.rot.dims must equal rot_dim={rot_dim}, got {rot.dims}")
                else:
                    rot = None
                mixer = FovunexLatent(heads, dim, rot_dim, _pos_int(m.get("vdim", dim), mw + ".vdim"),
                                      _pos_int(_need(m, "kv_rank", mw), mw + ".kv_rank"),
                                      float(m.get("scale", (dim + rot_dim) ** -0.5)), rot,
                                      _parse_chunk(m.get("mask"), mw + ".mask"))
            elif kind == "attention":
                heads = _pos_int(_need(m, "heads", mw), mw + ".heads")
                kv = _pos_int(m.get("kv_heads", heads), mw + ".kv_heads")
                if heads % kv:
                    raise ConfigError(f"config.json: {mw}: {heads} heads are not a multiple of {kv} kv_heads")
                dim = _pos_int(_need(m, "dim", mw), mw + ".dim")
                diff = float(_need(m, "diff", mw))
                mixer = FovunexAttention(heads, kv, dim, _pos_int(m.get("vdim", dim), mw + ".vdim"),
                                         float(m.get("scale", dim ** -0.5)), diff, _parse_rot(m.get("rot"), mw + ".rot", dim),
                                         _parse_chunk(m.get("mask"), mw + ".mask"))
            elif kind == "mingru":
                mixer = FovunexMinGRU(_pos_int(_need(m, "width", mw), mw + ".width"))
            else:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not built (known: latent_attention, attention, mingru)")
            layers.append(FovunexLayer(kind, mixer, mlp))
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
        return cls(architecture=str(d.get("architecture") or (d.get("architectures") or ["Fovunex"])[0]), vocab=vocab,
                   width=width, norm_eps=eps, embedding_scale=float(emb.get("scale", 1.0)), layers=tuple(layers),
                   loop_start=start, loop_stop=stop, loop_times=times, eos_token_id=d.get("eos_token_id"))

    def to_hf_dict(self) -> dict:
        def rot_dict(r: FovunexRotation | None):
            if r is None:
                return None
            out = {"base": r.base, "dims": r.dims}
            if r.scaling is not None:
                s = r.scaling
                out["scaling"] = {"factor": s.factor, "original": s.original, "fast": s.fast, "slow": s.slow}
            return out

        layers = []
        for L in self.layers:
            x = L.mixer
            if L.type == "latent_attention":
                mixer = {"heads": x.heads, "dim": x.dim, "rot_dim": x.rot_dim, "vdim": x.vdim, "kv_rank": x.kv_rank,
                         "scale": x.scale}
            elif L.type == "attention":
                mixer = {"heads": x.heads, "kv_heads": x.kv_heads, "dim": x.dim, "vdim": x.vdim, "scale": x.scale,
                         "diff": x.diff}
            else:
                mixer = {"width": x.width}
            if L.type != "mingru":
                if x.rot is not None:
                    mixer["rot"] = rot_dict(x.rot)
                if x.chunk is not None:
                    mixer["mask"] = {"size": x.chunk}
            mlp = None if L.mlp is None else {"kind": "dense", "ff": L.mlp.ff, "limit": L.mlp.limit}
            layers.append({"type": L.type, "mixer": mixer, "mlp": mlp})
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
        return NormSpec("rmsnorm", self.width, self.norm_eps, name, scalar=True)

    @staticmethod
    def _position(r: FovunexRotation | None, layout: str, head_dim: int) -> PositionSpec:
        if r is None:
            return PositionSpec(kind="none")
        return PositionSpec(kind="rotary_partial", head_dim=head_dim, theta=r.base, rot_dims=r.dims, layout=layout,
                            yarn=r.scaling)

    def _mixer_spec(self, L: FovunexLayer, m: str):
        x = L.mixer
        if L.type == "latent_attention":
            return LatentAttentionSpec(
                kind="latent_attention", hidden=self.width, n_heads=x.heads, head_dim=x.dim, rot_dim=x.rot_dim,
                v_head_dim=x.vdim, kv_rank=x.kv_rank, scale=x.scale, norm_eps=self.norm_eps,
                position=self._position(x.rot, "neighbours", x.rot_dim), chunk=x.chunk, q_proj=m + "q",
                down_proj=m + "dkv", latent_norm=m + "dkv.norm", k_up=m + "uk", v_up=m + "uv", o_proj=m + "o")
        if L.type == "attention":
            return DifferentialAttentionSpec(
                kind="differential_attention", hidden=self.width, n_heads=x.heads, n_kv_heads=x.kv_heads,
                head_dim=x.dim, v_head_dim=x.vdim, scale=x.scale, norm_eps=self.norm_eps, lambda_init=x.diff,
                position=self._position(x.rot, "halves", x.dim), chunk=x.chunk, q_proj=m + "q", k_proj=m + "k",
                v_proj=m + "v", q_norm=m + "q.norm", k_norm=m + "k.norm", lambda_q1=m + "lq1", lambda_k1=m + "lk1",
                lambda_q2=m + "lq2", lambda_k2=m + "lk2", gate_proj=m + "g", o_proj=m + "o")
        return MinGRUSpec(kind="mingru", hidden=self.width, width=x.width, z_proj=m + "z", z_bias=m + "z.b",
                          x_proj=m + "x", x_bias=m + "x.b", gate_proj=m + "g", o_proj=m + "o")

    def run_order(self) -> list[tuple[int, bool]]:
        """(layer, whether the embedding is added again before it) for every run of a layer, in order."""
        n = len(self.layers)
        if self.loop_stop <= self.loop_start:
            return [(i, False) for i in range(n)]
        order = [(i, False) for i in range(self.loop_start)]
        for t in range(self.loop_times):
            order += [(i, t > 0 and i == self.loop_start) for i in range(self.loop_start, self.loop_stop)]
        return order + [(i, False) for i in range(self.loop_stop, n)]

    def model_spec(self) -> ReinjectDecoderSpec:
        layers = []
        for i, L in enumerate(self.layers):
            p = f"l{i}."
            if L.mlp is None:
                ff_norm, ff, ff_gate = None, None, None
            else:
                f = p + "mlp."
                ff_norm, ff_gate = self._norm(p + "norm2"), p + "rg2"
                ff = GatedMLPSpec(kind="gated_mlp", hidden=self.width, intermediate=L.mlp.ff, activation="clamped_swish",
                                  act_alpha=SWISH_ALPHA, act_limit=L.mlp.limit, up_offset=UP_OFFSET, gate_proj=f + "gate",
                                  up_proj=f + "up", down_proj=f + "down")
            layers.append(BlockSpec(kind="gated_prenorm", mixer_norm=self._norm(p + "norm1"),
                                    mixer=self._mixer_spec(L, p + "mix."), ff_norm=ff_norm, feedforward=ff,
                                    mixer_gate=p + "rg1", mixer_gate_bias=p + "rg1.b", ff_gate=ff_gate,
                                    ff_gate_bias=ff_gate + ".b" if ff_gate else None))
        order = self.run_order()
        return ReinjectDecoderSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden=self.width, max_positions=NO_POSITION_LIMIT,
            embedding="embed", layers=tuple(layers), schedule=tuple(ScheduleEntry(layer=i) for i, _ in order),
            final_norm=self._norm("final.norm"), head="head", embedding_scale=self.embedding_scale,
            reinject_before=tuple(k for k, (_, add) in enumerate(order) if add))
