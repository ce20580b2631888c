"""Small Gavatar configurations for the tests, and model folders made from them.

They differ from one another in every size and constant: width, vocabulary, embedding scale (one of them 1), order and
number of layers, which layers run several times (a middle group three times, the whole model twice, none), head
counts and groups (kv heads equal to the heads, one kv head, a group in between), key and value head sizes (equal and
unequal, most no power of two), windows (shorter than a page, across several pages, none), compressed sizes, gate
caps, experts and how many a token runs (one, some, all of them), layers without a feed-forward, and one attention
layer whose value heads, side by side, are wider than one launch of the attention kernels takes.
"""

from __future__ import annotations

import json
from pathlib import Path

import torch


def _moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def _att(heads, kv, dim, vdim, scale, window, mlp):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    return {"type": "attention", "mixer": m, "mlp": mlp}


def _lat(heads, dim, vdim, q_rank, kv_rank, scale, window, mlp):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def _mem(heads, dim, vdim, cap, mlp):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}, "mlp": mlp}


def _model(vocab, width, eps, scale, layers, loop=None):
    d = {"architecture": "Gavatar", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": scale},
         "layers": layers}
    if loop is not None:
        d["loop"] = dict(zip(("start", "stop", "times"), loop))
    return d


# talking attention first with a window shorter than three pages of 8; a matrix memory in the middle; a latent
# attention without a feed-forward; the last two layers run three times
GAV_A = _model(211, 64, 1e-5, 3.0, [
    _att(4, 2, 16, 24, 0.3, 21, _moe(6, 2, 40)),
    _mem(2, 12, 20, 8.0, _moe(5, 1, 24)),
    _lat(3, 8, 12, 20, 24, 0.33, 13, None),
], loop=(1, 3, 3))
# no loop, an embedding scale of one; one latent head that sees every key; as many kv heads as heads under a window of
# nine; a token runs all three experts
GAV_B = _model(157, 96, 1e-6, 1.0, [
    _lat(1, 24, 24, 16, 24, 0.2, None, _moe(4, 3, 72)),
    _att(3, 3, 12, 12, 0.25, 9, _moe(3, 3, 24)),
])
# sizes that are multiples of nothing much: width 100, heads of 10, 6 and 14; one kv head under five heads; the whole
# model runs twice; a window of exactly two pages
GAV_C = _model(131, 100, 1e-5, 0.5, [
    _lat(5, 10, 6, 7, 14, 0.4, 40, _moe(7, 2, 20)),
    _att(5, 1, 10, 6, 0.35, 16, None),
    _mem(5, 10, 14, 15.0, _moe(2, 1, 12)),
], loop=(0, 3, 2))
# head sizes that are multiples of 16, which the tensor-core attention of prompt portions takes, and four latent heads
# over one cached row, which send decode tokens there too; the attention layers run twice
GAV_W = _model(300, 128, 1e-5, 4.0, [
    _att(4, 2, 16, 32, 0.25, 40, _moe(8, 2, 96)),
    _lat(4, 16, 16, 24, 32, 0.2, 56, _moe(4, 1, 64)),
    _mem(2, 32, 32, 10.0, None),
], loop=(0, 2, 2))
# three value heads of 96 side by side are wider than a launch of the attention kernels takes: two launches
GAV_S = _model(180, 80, 1e-5, 2.0, [_att(6, 3, 16, 96, 0.3, 33, None)])
# one mechanism each
GAV_ATT = _model(120, 48, 1e-5, 2.0, [_att(6, 3, 12, 8, 0.3, 19, None)])
GAV_LAT = _model(120, 48, 1e-5, 2.0, [_lat(4, 12, 8, 10, 16, 0.3, None, None)])
GAV_MEM = _model(120, 48, 1e-5, 2.0, [_mem(3, 8, 24, 6.0, None)])
GAV_MOE = _model(120, 48, 1e-6, 2.0, [_mem(1, 16, 16, 15.0, _moe(9, 4, 28))])

MODELS = {"gav_a": GAV_A, "gav_b": GAV_B, "gav_c": GAV_C, "gav_w": GAV_W, "gav_s": GAV_S, "gav_att": GAV_ATT,
          "gav_lat": GAV_LAT, "gav_mem": GAV_MEM, "gav_moe": GAV_MOE}
SEEDS = {"gav_a": 51, "gav_b": 52, "gav_c": 53, "gav_w": 54, "gav_s": 55, "gav_att": 56, "gav_lat": 57, "gav_mem": 58,
         "gav_moe": 59}


def lively(tensors: dict) -> None:
    """Random tensors drawn N(0, std) leave some mechanisms almost idle; give them values that matter: norm weights
    away from zero, shift weights across [0, 1], biases of order one, a mixing matrix of the heads that is far from the
    identity, sinks that take a real share of the denominator, input and forget gates from almost shut to wide open,
    router biases that move the choice."""
    g = torch.Generator().manual_seed(79)
    for name, t in tensors.items():
        f = t.float()
        if name.endswith((".norm1", ".norm2", ".norm1b", ".norm2b")) or name == "final.norm":
            f = 0.8 * torch.rand(f.shape, generator=g) - 0.4
        elif name.endswith(".shift"):
            f = torch.rand(f.shape, generator=g)
        elif name.endswith((".q.b", ".k.b", ".v.b")):
            f = 0.5 * torch.randn(f.shape, generator=g)
        elif name.endswith(".talk"):
            f = torch.eye(f.shape[0]) * 0.7 + 0.4 * torch.randn(f.shape, generator=g)
        elif name.endswith(".sink"):
            f = torch.randn(f.shape, generator=g)
        elif name.endswith((".dq.norm", ".dkv.norm", ".mix.norm")):
            f = 0.6 + 0.9 * torch.rand(f.shape, generator=g)
        elif name.endswith(".i.b"):
            f = torch.linspace(-2.0, 3.0, f.numel()).reshape(f.shape)
        elif name.endswith(".f.b"):
            f = torch.linspace(0.5, 5.0, f.numel()).reshape(f.shape)
        elif name.endswith(".router.b"):
            f = 0.3 * torch.randn(f.shape, generator=g)
        elif name.endswith((".mix.i", ".mix.f", ".uq", ".uk", ".uv", ".router")) or ".mlp.e" in name:
            f = f * 3
        elif name == "loop.step":
            f = torch.randn(f.shape, generator=g)
        else:
            continue
        tensors[name] = f.to(t.dtype)


def make_gavatar_dir(tmp, name: str, store_dtype: str = "bfloat16", std: float = 0.08, fix=None, config: dict | None = None,
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
