"""Small Fovunex configurations for the tests, and model folders made from them.

They differ from one another in every size and constant: width, vocabulary, embedding scale (one of them 1), order and
number of layers, which layers run several times (a middle group three times, the whole model twice, none), head counts
and groups, key and value head sizes (equal and unequal, none a power of two), the rotated share (a part, the whole
head, none), rotations with and without blended frequencies on either kind of attention, chunks (shorter than a page,
a multiple of the page, none; on the latent attention as well), compressed sizes, recurrence widths, feed-forward
sizes and limits, layers without a feed-forward.
"""

from __future__ import annotations

import json
from pathlib import Path

import torch


def _mlp(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def _rot(base, dims, scaling=None):
    out = {"base": base, "dims": dims}
    if scaling is not None:
        out["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return out


def _latent(heads, dim, rot_dim, vdim, kv_rank, scale, rot, chunk, mlp):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale}
    if rot is not None:
        m["rot"] = rot
    if chunk is not None:
        m["mask"] = {"size": chunk}
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def _diff(heads, kv, dim, vdim, scale, diff, rot, chunk, mlp):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff}
    if rot is not None:
        m["rot"] = rot
    if chunk is not None:
        m["mask"] = {"size": chunk}
    return {"type": "attention", "mixer": m, "mlp": mlp}


def _gru(width, mlp):
    return {"type": "mingru", "mixer": {"width": width}, "mlp": mlp}


def _model(vocab, width, eps, scale, layers, loop=None):
    d = {"architecture": "Fovunex", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": scale},
         "layers": layers}
    if loop is not None:
        d["loop"] = dict(zip(("start", "stop", "times"), loop))
    return d


# differential attention first with half of each map rotated and a chunk shorter than two pages of 8; a recurrence in
# the middle; a latent attention with blended frequencies and no feed-forward; the last two layers run three times
FVX_A = _model(211, 64, 1e-5, 3.0, [
    _diff(4, 2, 16, 24, 0.3, 0.2, _rot(1000.0, 8), 21, _mlp(40, 1.0)),
    _gru(48, _mlp(56, 2.5)),
    _latent(3, 8, 4, 12, 20, 0.33, _rot(300.0, 4, (2.0, 16, 4.0, 1.0)), None, None),
], loop=(1, 3, 3))
# no loop, an embedding scale of one; one latent head with values as large as the compressed vector and a chunk of 9
# on the latent attention; as many kv heads as heads with the whole map rotated by blended frequencies and no chunk
FVX_B = _model(157, 96, 1e-6, 1.0, [
    _latent(1, 24, 8, 24, 24, 0.2, _rot(50.0, 8), 9, _mlp(72, 0.7)),
    _diff(3, 3, 12, 12, 0.25, 0.5, _rot(500.0, 12, (3.0, 24, 6.0, 0.5)), None, _mlp(24, 1.5)),
])
# sizes that are multiples of nothing much: width 100, heads of 10 and 6, a recurrence of 35 channels; one kv head
# under five heads without any rotation, a chunk of two pages; the whole model runs twice
FVX_C = _model(131, 100, 1e-5, 0.5, [
    _latent(5, 10, 6, 6, 14, 0.4, _rot(100.0, 6), None, _mlp(20, 1.2)),
    _diff(5, 1, 10, 6, 0.35, 0.1, None, 16, None),
    _gru(35, _mlp(12, 3.0)),
], loop=(0, 3, 2))
# head sizes that are multiples of 16, which the tensor-core attention of prompt portions takes: two maps of 16 over
# values of 32 in chunks of 40, a compressed row of 32 + 16; the attention layers run twice
FVX_W = _model(300, 128, 1e-5, 4.0, [
    _diff(4, 2, 16, 32, 0.25, 0.3, _rot(1000.0, 8), 40, _mlp(96, 1.5)),
    _latent(3, 16, 16, 16, 32, 0.2, _rot(400.0, 16, (2.0, 32, 8.0, 1.0)), None, _mlp(64, 2.0)),
    _gru(80, None),
], loop=(0, 2, 2))
# one mechanism each
FVX_LAT = _model(120, 48, 1e-5, 2.0, [_latent(4, 12, 4, 8, 16, 0.3, _rot(200.0, 4, (4.0, 32, 8.0, 1.0)), None, None)])
FVX_DIFF = _model(120, 48, 1e-5, 2.0, [_diff(6, 3, 12, 8, 0.3, 0.4, _rot(1000.0, 6), 19, None)])
FVX_GRU = _model(120, 48, 1e-5, 2.0, [_gru(56, None)])
FVX_FF = _model(120, 48, 1e-6, 2.0, [_gru(16, _mlp(28, 0.8))])

MODELS = {"fvx_a": FVX_A, "fvx_b": FVX_B, "fvx_c": FVX_C, "fvx_w": FVX_W, "fvx_lat": FVX_LAT, "fvx_diff": FVX_DIFF, "fvx_gru": FVX_GRU,
          "fvx_ff": FVX_FF}
SEEDS = {"fvx_w": 48, "fvx_a": 41, "fvx_b": 42, "fvx_c": 43, "fvx_lat": 44, "fvx_diff": 45, "fvx_gru": 46, "fvx_ff": 47}


def lively(tensors: dict) -> None:
    """Random tensors drawn N(0, std) leave some mechanisms almost idle; give them values that matter: norm gains away
    from one, gate biases of order one, head norms that make the attention sharp, lambda vectors that make the two
    maps' weights differ, recurrence gates from almost shut to almost open, candidates on both sides of zero, and
    feed-forward branches that reach their limits."""
    g = torch.Generator().manual_seed(78)
    for name, t in tensors.items():
        f = t.float()
        if name.endswith((".norm1", ".norm2")) or name == "final.norm":
            f = 0.6 + 0.9 * torch.rand(f.shape, generator=g)
        elif name.endswith((".rg1.b", ".rg2.b")):
            f = torch.randn(f.shape, generator=g)
        elif name.endswith((".q.norm", ".k.norm")):
            f = 1.5 + torch.rand(f.shape, generator=g)
        elif name.endswith(".dkv.norm"):
            f = 0.5 + torch.rand(f.shape, generator=g)
        elif name.endswith((".lq1", ".lk1", ".lq2", ".lk2")):
            f = torch.randn(f.shape, generator=g) * 0.25
        elif name.endswith(".z.b"):
            f = torch.linspace(-5.0, 5.0, f.numel()).reshape(f.shape)
        elif name.endswith(".x.b"):
            f = torch.randn(f.shape, generator=g)
        elif name.endswith((".mlp.gate", ".mlp.up", ".uk", ".uv", ".mix.z", ".mix.x")):
            f = f * 3
        else:
            continue
        tensors[name] = f.to(t.dtype)


def make_fovunex_dir(tmp, name: str, store_dtype: str = "bfloat16", std: float = 0.08, fix=None, config: dict | None = None,
                     seed: int | None = None) -> Path:
    """A model folder with random weights for ``MODELS[name]`` (or ``config``); ``fix(tensors)`` may change them."""
    from inf_engine_b200.config import parse_config_dict
    from inf_engine_b200.parts import expected_tensors
    from inf_engine_b200.weights import random_tensors, write_safetensors

    d = config if config is not None else MODELS[name]
    out = Path(tmp) / f"{name}_{store_dtype}"
    out.mkdir(parents=True, exist_ok=True)
    cfg = parse_config_dict(d)
    tensors = random_tensors(expected_tensors(cfg.model_spec()), SEEDS.get(name, 7) if seed is None else seed, std=std,
                             store_dtype=store_dtype)
    lively(tensors)
    if fix is not None:
        fix(tensors)
    (out / "config.json").write_text(json.dumps(d, indent=1))
    write_safetensors(out / "model.safetensors", tensors, metadata={"format": "pt"})
    return out
