"""The Fovunex family without a GPU: configuration and its errors, the tensor table, the order of layer runs, the
cache groups its mixers ask for (keys that hold their values, fewer value heads than key heads, pages given back
behind a chunk), the blended rotation frequencies against the plain rule, and the plain implementation's own
consistency (a recurrence carried over a cut, masks, rotations)."""

import copy
import math

import pytest
import torch

import plain_fovunex as plain
from fovunex_models import MODELS, make_fovunex_dir
from helpers import plain_inputs, random_tokens

from inf_engine_b200.cache.manager import CacheManager, CacheRequirement
from inf_engine_b200.config import ConfigError, FovunexConfig, PositionSpec, YarnScaling, parse_config_dict
from inf_engine_b200.parts import expected_tensors
from inf_engine_b200.parts.positions import partial_rotation_frequencies


def test_config_round_trip_and_specs():
    for name, d in MODELS.items():
        cfg = parse_config_dict(d)
        assert isinstance(cfg, FovunexConfig)
        assert cfg.to_hf_dict() == d, name
        spec = cfg.model_spec()
        assert spec.kind == "reinject_decoder" and spec.head == "head" and spec.embedding_scale == d["embedding"]["scale"]
        assert [e.layer for e in spec.schedule] == [i for i, _ in plain.layer_order(d)]
        assert list(spec.reinject_before) == [k for k, (_, add) in enumerate(plain.layer_order(d)) if add]
        for blk, L in zip(spec.layers, d["layers"]):
            assert blk.kind == "gated_prenorm" and blk.mixer_norm.scalar
            assert (blk.feedforward is None) == (L["mlp"] is None)


def test_order_of_runs():
    cfg = parse_config_dict(MODELS["fvx_a"])
    assert cfg.run_order() == [(0, False), (1, False), (2, False), (1, True), (2, False), (1, True), (2, False)]
    cfg = parse_config_dict(MODELS["fvx_c"])
    assert cfg.run_order() == [(0, False), (1, False), (2, False), (0, True), (1, False), (2, False)]
    d = copy.deepcopy(MODELS["fvx_c"])
    d["loop"] = {"start": 1, "stop": 2, "times": 1}
    assert parse_config_dict(d).model_spec().reinject_before == ()


def test_tensor_table():
    t = expected_tensors(parse_config_dict(MODELS["fvx_a"]).model_spec())
    assert t["embed"].shape == (211, 64) and t["head"].shape == (211, 64)
    assert t["l0.norm1"].shape == () and t["final.norm"].shape == ()
    assert t["l0.mix.q"].shape == (4 * 2 * 16, 64) and t["l0.mix.k"].shape == (2 * 2 * 16, 64)
    assert t["l0.mix.v"].shape == (2 * 24, 64) and t["l0.mix.g"].shape == (4 * 24, 64) and t["l0.mix.o"].shape == (64, 96)
    assert t["l0.mix.q.norm"].shape == (16,) and t["l0.mix.lk2"].shape == (16,)
    assert t["l0.rg1"].shape == (64, 64) and t["l0.rg2.b"].shape == (64,)
    assert t["l1.mix.z"].shape == (48, 64) and t["l1.mix.x.b"].shape == (48,) and t["l1.mix.o"].shape == (64, 48)
    assert t["l2.mix.q"].shape == (3 * 12, 64) and t["l2.mix.dkv"].shape == (24, 64) and t["l2.mix.dkv.norm"].shape == (20,)
    assert t["l2.mix.uk"].shape == (3 * 8, 20) and t["l2.mix.uv"].shape == (3 * 12, 20) and t["l2.mix.o"].shape == (64, 36)
    assert "l2.norm2" not in t and "l2.rg2" not in t and "l2.mlp.gate" not in t
    assert t["l0.mlp.gate"].shape == (40, 64) and t["l0.mlp.down"].shape == (64, 40)


@pytest.mark.parametrize("change, text", [
    (lambda d: d["layers"][0].update(type="conv"), "not built"),
    (lambda d: d["layers"][0]["mlp"].update(kind="moe"), "not built"),
    (lambda d: d["layers"][0]["mixer"].update(kv_heads=3), "multiple"),
    (lambda d: d["layers"][0]["mixer"]["rot"].update(dims=7), "even"),
    (lambda d: d["layers"][2]["mixer"]["rot"].update(dims=2), "rot_dim"),
    (lambda d: d.update(loop={"start": 2, "stop": 5, "times": 2}), "loop"),
    (lambda d: d["layers"][0]["mixer"].pop("diff"), "diff"),
    (lambda d: d.pop("width"), "width"),
])
def test_config_errors(change, text):
    d = copy.deepcopy(MODELS["fvx_a"])
    change(d)
    with pytest.raises(ConfigError, match=text):
        parse_config_dict(d)


def test_blended_frequencies_follow_the_plain_rule():
    for dims, base, sc in ((4, 300.0, (2.0, 16, 4.0, 1.0)), (12, 500.0, (3.0, 24, 6.0, 0.5)), (64, 10000.0, (8.0, 4096, 32.0, 1.0)),
                           (6, 100.0, None)):
        yarn = YarnScaling(*[float(x) for x in sc]) if sc else None
        f, mult = partial_rotation_frequencies(PositionSpec(kind="rotary_partial", theta=base, rot_dims=dims, yarn=yarn))
        rot = {"base": base, "dims": dims}
        if sc:
            rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), sc))
        pos = torch.tensor([0, 1, 7, 1000])
        cos, sin = plain.rotation_angles(rot, pos)
        a = pos.double()[:, None] * f[None, :]
        assert torch.allclose(cos, torch.cos(a) * mult, atol=1e-12) and torch.allclose(sin, torch.sin(a) * mult, atol=1e-12)
    # worked by hand: dims 4, base 300, original 16, fast 4, slow 1: dim(t) = 4 ln(16 / (2 pi t)) / (2 ln 300)
    lo = max(math.floor(4 * math.log(16 / (2 * math.pi * 4)) / (2 * math.log(300))), 0)
    hi = min(math.ceil(4 * math.log(16 / (2 * math.pi * 1)) / (2 * math.log(300))), 3)
    assert (lo, hi) == (0, 1)
    f, mult = partial_rotation_frequencies(PositionSpec(kind="rotary_partial", theta=300.0, rot_dims=4,
                                                        yarn=YarnScaling(2.0, 16.0, 4.0, 1.0)))
    assert torch.allclose(f, torch.tensor([1.0, 300.0 ** -0.5 / 2.0], dtype=torch.float64))
    assert mult == pytest.approx(0.1 * math.log(2.0) + 1.0)


def test_cache_groups_of_the_mixers():
    latent = CacheRequirement(kind="kv", n_kv_heads=1, head_dim=24, v_head_dim=20, dtype=torch.float32, values_in_keys=True)
    diff = CacheRequirement(kind="kv", n_kv_heads=4, head_dim=16, v_head_dim=24, dtype=torch.float32, n_v_heads=2, chunk=21)
    state = CacheRequirement(kind="state", state_shape=(48,), state_dtype=torch.float32)
    m = CacheManager([diff, state, latent, state, latent], page_size=8, n_pages=12, max_requests=2)
    assert len(m.kv_groups) == 2 and len(m.state_groups) == 1
    m.allocate_storage("cpu")
    g_diff, g_lat = m.kv_groups
    assert g_diff.k.shape == (1, 12, 4, 8, 16) and g_diff.v.shape == (1, 12, 2, 8, 24)
    assert g_lat.v is g_lat.k and g_lat.k.shape == (2, 12, 1, 8, 24)
    assert m.storage_bytes() == 4 * (12 * 8 * (4 * 16 + 2 * 24) + 2 * 12 * 8 * 24 + 2 * 2 * 48)
    # pages wholly before the chunk of the next token go back to the pool; the other group keeps everything
    m.open("a")
    assert m.reserve("a", 50)
    m.advance("a", 50)                      # next token 50 lies in the chunk that starts at 42: pages 0..4 are free
    assert g_diff.tables["a"][:5] == [-1] * 5 and all(p >= 0 for p in g_diff.tables["a"][5:])
    assert all(p >= 0 for p in g_lat.tables["a"])
    assert g_diff.pool.n_free == 12 - 2 and g_lat.pool.n_free == 12 - 7
    m.check()
    m.advance("a", 41)
    m.close("a")
    m.check()
    assert g_diff.pool.n_free == 12 and g_lat.pool.n_free == 12


def test_plain_recurrence_carries_over_a_cut_and_masks_cut_where_they_should(tmp_path):
    cfg, w = plain_inputs(make_fovunex_dir(tmp_path, "fvx_gru"))
    h = torch.randn(30, 48, dtype=torch.float64)
    whole, s_end = plain.mingru(h, cfg["layers"][0]["mixer"], w, "l0.mix.")
    a, s_mid = plain.mingru(h[:11], cfg["layers"][0]["mixer"], w, "l0.mix.")
    b, s_b = plain.mingru(h[11:], cfg["layers"][0]["mixer"], w, "l0.mix.", state=s_mid)
    assert torch.allclose(torch.cat([a, b]), whole, atol=1e-12) and torch.allclose(s_b, s_end, atol=1e-12)
    m = plain.causal_mask(10, 4)
    assert m[5].tolist() == [False] * 4 + [True, True] + [False] * 4 and m[8].tolist() == [False] * 8 + [True, False]
    assert plain.causal_mask(3).tolist() == [[True, False, False], [True, True, False], [True, True, True]]
    # a chunked model's logits after a chunk's start do not depend on what came before it
    cfg, w = plain_inputs(make_fovunex_dir(tmp_path, "fvx_diff"))
    toks = random_tokens(cfg["vocab"], 45, 3)
    other = random_tokens(cfg["vocab"], 19, 4) + toks[19:]
    x, y = plain.forward(cfg, w, toks), plain.forward(cfg, w, other)
    assert torch.allclose(x[19:], y[19:], atol=1e-9) and not torch.allclose(x[:19], y[:19], atol=1e-3)


def test_plain_rotations_keep_lengths_and_depend_on_distance_only():
    rot = {"base": 100.0, "dims": 6}
    x = torch.randn(1, 1, 6, dtype=torch.float64)
    y = torch.randn(1, 1, 6, dtype=torch.float64)
    for fn in (plain.rotate_halves, plain.rotate_interleaved):
        dots = []
        for p in (0, 5, 40):
            cq, sq = plain.rotation_angles(rot, torch.tensor([p + 3]))
            ck, sk = plain.rotation_angles(rot, torch.tensor([p]))
            q, k = fn(x, cq, sq), fn(y, ck, sk)
            assert torch.allclose(q.norm(), x.norm())
            dots.append(float((q * k).sum()))
        assert dots[0] == pytest.approx(dots[1], abs=1e-12) and dots[0] == pytest.approx(dots[2], abs=1e-12)
    assert not torch.allclose(plain.rotate_halves(x, cq, sq), plain.rotate_interleaved(x, cq, sq))


def test_every_mechanism_matters_in_the_test_models(tmp_path):
    """Leaving a mechanism out of the plain model moves its logits: a test model in which it did not would not test it."""
    folder = make_fovunex_dir(tmp_path, "fvx_a")
    cfg, w = plain_inputs(folder)
    toks = random_tokens(cfg["vocab"], 60, 9)
    base = plain.forward(cfg, w, toks)

    def moved(cfg2=None, w2=None):
        other = plain.forward(cfg2 or cfg, w2 or w, toks)
        return float(((other - base).norm(dim=-1) / base.norm(dim=-1)).max())

    c = copy.deepcopy(cfg); c["loop"]["times"] = 2
    assert moved(c) > 0.05
    c = copy.deepcopy(cfg); c["embedding"]["scale"] = 1.0
    assert moved(c) > 0.05
    c = copy.deepcopy(cfg); c["layers"][0]["mixer"]["mask"]["size"] = 22
    assert moved(c) > 0.01
    c = copy.deepcopy(cfg); c["layers"][0]["mixer"]["diff"] = 0.25
    assert moved(c) > 0.01
    c = copy.deepcopy(cfg); c["layers"][2]["mixer"]["rot"].pop("scaling")
    assert moved(c) > 0.01
    c = copy.deepcopy(cfg); c["layers"][0]["mlp"]["limit"] = 0.5
    assert moved(c) > 0.01
    for name in ("l0.rg1.b", "l1.mix.z.b", "l1.mix.x.b", "l0.mix.lq1", "l2.mix.dkv.norm", "l0.mix.k.norm", "l1.norm2"):
        w2 = dict(w); w2[name] = torch.zeros_like(w[name]) if name.endswith(".b") or ".lq" in name else torch.ones_like(w[name])
        assert moved(w2=w2) > 0.005, name
