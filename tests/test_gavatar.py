"""The Gavatar family without a GPU: configuration and its errors, the tensor table, the order of layer runs and where
the passes' vectors are added, the cache groups its layers ask for (a token's value heads in one row, a compressed row
under a window, the shifted input's last row beside the mixer's own cache), and the plain implementation's own
consistency (windows, the sink, mixed heads, the matrix memory carried over any prefix, the router)."""

import copy

import pytest
import torch

import plain_gavatar as plain
from gavatar_models import MODELS, make_gavatar_dir
from helpers import plain_inputs, random_tokens

from inf_engine_b200.cache.manager import CacheManager, CacheRequirement
from inf_engine_b200.config import ConfigError, GavatarConfig, parse_config_dict
from inf_engine_b200.parts import expected_tensors


def test_config_round_trip_and_specs():
    for name, d in MODELS.items():
        cfg = parse_config_dict(d)
        assert isinstance(cfg, GavatarConfig)
        assert cfg.to_hf_dict() == d, name
        spec = cfg.model_spec()
        assert spec.kind == "pass_offset_decoder" and spec.head == "head" and spec.sinusoid_base == 10000.0
        assert spec.embedding_scale == d["embedding"]["scale"]
        order = plain.run_order(d)
        assert [e.layer for e in spec.schedule] == [i for i, _ in order]
        assert list(spec.offset_before) == [(k, t) for k, (_, t) in enumerate(order) if t is not None]
        assert (spec.pass_offsets is None) == ("loop" not in d)
        for blk, L in zip(spec.layers, d["layers"]):
            assert blk.kind == "sandwich" and blk.mixer_norm.unit_offset and blk.mixer_out_norm.unit_offset
            assert blk.token_shift is not None
            assert (blk.feedforward is None) == (L["mlp"] is None) == (blk.ff_out_norm is None)
            if L["mlp"] is not None:
                assert blk.feedforward.score == "softmax_top" and blk.feedforward.top == L["mlp"]["router"]["top"]


def test_order_of_runs():
    cfg = parse_config_dict(MODELS["gav_a"])
    assert cfg.run_order() == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (1, 2), (2, None)]
    cfg = parse_config_dict(MODELS["gav_c"])
    assert cfg.run_order() == [(0, 0), (1, None), (2, None), (0, 1), (1, None), (2, None)]
    d = copy.deepcopy(MODELS["gav_c"])
    d["loop"] = {"start": 1, "stop": 2, "times": 1}
    assert parse_config_dict(d).model_spec().offset_before == ((1, 0),)          # one pass still takes its vector
    d["loop"] = {"start": 2, "stop": 2, "times": 4}
    assert parse_config_dict(d).model_spec().pass_offsets is None


def test_tensor_table():
    t = expected_tensors(parse_config_dict(MODELS["gav_a"]).model_spec())
    assert t["embed"].shape == (211, 64) and t["head"].shape == (211, 64) and t["loop.step"].shape == (3, 64)
    for n in ("l0.norm1", "l0.norm1b", "l0.norm2", "l0.norm2b", "l0.shift", "final.norm"):
        assert t[n].shape == (64,), n
    assert t["l0.mix.q"].shape == (4 * 16, 64) and t["l0.mix.q.b"].shape == (64,)
    assert t["l0.mix.k"].shape == (2 * 16, 64) and t["l0.mix.v"].shape == (2 * 24, 64) and t["l0.mix.v.b"].shape == (48,)
    assert t["l0.mix.talk"].shape == (4, 4) and t["l0.mix.g"].shape == (96, 64) and t["l0.mix.o"].shape == (64, 96)
    assert t["l0.mlp.router"].shape == (6, 64) and t["l0.mlp.router.b"].shape == (6,)
    assert t["l0.mlp.e5.gate"].shape == (40, 64) and t["l0.mlp.e0.down"].shape == (64, 40) and "l0.mlp.e6.up" not in t
    assert t["l1.mix.q"].shape == (24, 64) and t["l1.mix.v"].shape == (40, 64) and t["l1.mix.norm"].shape == (40,)
    assert t["l1.mix.i"].shape == (2, 64) and t["l1.mix.f.b"].shape == (2,)
    assert t["l2.mix.dq"].shape == (20, 64) and t["l2.mix.dq.norm"].shape == (20,) and t["l2.mix.uq"].shape == (24, 20)
    assert t["l2.mix.dkv"].shape == (24, 64) and t["l2.mix.uk"].shape == (24, 24) and t["l2.mix.uv"].shape == (36, 24)
    assert t["l2.mix.sink"].shape == (3,) and t["l2.mix.g"].shape == (3, 64) and t["l2.mix.o"].shape == (64, 36)
    assert "l2.norm2" not in t and "l2.norm2b" not in t and "l2.mlp.router" not in t
    assert "loop.step" not in expected_tensors(parse_config_dict(MODELS["gav_b"]).model_spec())


def test_sizes_that_the_tensors_settle():
    d = copy.deepcopy(MODELS["gav_lat"])
    d["layers"][0]["mixer"].pop("q_rank")
    with pytest.raises(ConfigError, match="q_rank"):
        parse_config_dict(d)
    shapes = {"l0.mix.dq": (10, 48)}
    cfg = parse_config_dict(d, shapes)
    assert cfg.layers[0].mixer.q_rank == 10 and not cfg.layers[0].shift          # no shift tensor in the file
    assert cfg.model_spec().layers[0].token_shift is None


@pytest.mark.parametrize("change, text", [
    (lambda d: d["layers"][0].update(type="conv"), "not built"),
    (lambda d: d["layers"][0]["mlp"].update(kind="dense"), "not built"),
    (lambda d: d["layers"][0]["mixer"].update(kv_heads=3), "multiple"),
    (lambda d: d["layers"][0]["mlp"]["router"].update(top=7), "cannot be chosen"),
    (lambda d: d["layers"][1]["mixer"].update(gate_cap=0.0), "gate_cap"),
    (lambda d: d["layers"][2]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda d: d.update(loop={"start": 2, "stop": 5, "times": 2}), "loop"),
    (lambda d: d["layers"][0]["mixer"]["mask"].update(size=0), "positive"),
    (lambda d: d.pop("width"), "width"),
])
def test_config_errors(change, text):
    d = copy.deepcopy(MODELS["gav_a"])
    change(d)
    with pytest.raises(ConfigError, match=text):
        parse_config_dict(d)


def test_cache_groups_of_the_layers():
    talking = CacheRequirement(kind="kv", n_kv_heads=2, head_dim=16, window=21, dtype=torch.float32, v_head_dim=48, n_v_heads=1)
    latent = CacheRequirement(kind="kv", n_kv_heads=1, head_dim=24, v_head_dim=24, dtype=torch.float32, values_in_keys=True,
                              window=13)
    last = CacheRequirement(kind="state", state_shape=(64,), state_dtype=torch.float32)
    memory = CacheRequirement(kind="state", state_shape=(2, 12 * 20 + 13), state_dtype=torch.float32)
    runs = [CacheRequirement(kind="several", parts=(x, last)) for x in (talking, memory, latent, memory, latent)]
    m = CacheManager(runs, page_size=8, n_pages=12, max_requests=2)
    assert len(m.kv_groups) == 2 and len(m.state_groups) == 2
    assert [b.kind for b in m.bindings] == ["several"] * 5 and [p.kind for p in m.bindings[1].parts] == ["state", "state"]
    m.allocate_storage("cpu")
    g_talk, g_lat = m.kv_groups
    assert g_talk.k.shape == (1, 12, 2, 8, 16) and g_talk.v.shape == (1, 12, 1, 8, 48)
    assert g_lat.v is g_lat.k and g_lat.k.shape == (2, 12, 1, 8, 24)
    shift_rows = [g for g in m.state_groups if g.shape == (64,)][0]
    assert shift_rows.data.shape == (5, 2, 64)                                    # a row per run and request
    # pages behind each window go back to its own pool
    m.open("a")
    assert m.reserve("a", 50)
    m.advance("a", 50)                      # the next token, 50, sees keys from 30 (window 21) and from 38 (window 13)
    assert g_talk.tables["a"][:3] == [-1] * 3 and g_talk.tables["a"][3] >= 0
    assert g_lat.tables["a"][:4] == [-1] * 4 and g_lat.tables["a"][4] >= 0
    m.check()
    m.close("a")
    assert g_talk.pool.n_free == 12 and g_lat.pool.n_free == 12


def test_plain_windows_sink_and_mixed_heads():
    m = plain.window_mask(6, 3)
    assert m[4].tolist() == [False, False, True, True, True, False] and m[1].tolist() == [True, True] + [False] * 4
    assert plain.window_mask(3, None).tolist() == [[True, False, False], [True, True, False], [True, True, True]]
    g = torch.Generator().manual_seed(0)
    q, k = torch.randn(5, 2, 4, generator=g, dtype=torch.float64), torch.randn(5, 2, 4, generator=g, dtype=torch.float64)
    vis = plain.window_mask(5, 3)
    p = plain.attention_weights(q, k, 0.5, vis)
    assert torch.allclose(p.sum(-1), torch.ones(2, 5, dtype=torch.float64)) and float(p[:, 4, :2].abs().max()) == 0.0
    sink = torch.tensor([0.3, -50.0], dtype=torch.float64)
    ps = plain.attention_weights(q, k, 0.5, vis, sink)
    s0 = (q[3, 0] * k[1:4, 0]).sum(-1) * 0.5            # by hand: head 0, query 3 sees keys 1..3 and the sink
    want = torch.exp(s0) / (torch.exp(s0).sum() + torch.exp(sink[0]))
    assert torch.allclose(ps[0, 3, 1:4], want) and float(ps[0, 3].sum()) < 1.0
    assert torch.allclose(ps[1], p[1], atol=1e-12)       # a sink far below every score takes nothing


def test_plain_matrix_memory_does_not_look_ahead_and_starts_from_zero(tmp_path):
    cfg, w = plain_inputs(make_gavatar_dir(tmp_path, "gav_mem"))
    mix = cfg["layers"][0]["mixer"]
    h = torch.randn(30, 48, dtype=torch.float64)
    whole = plain.mlstm(h, mix, w, "l0.mix.", 1e-5)
    assert torch.allclose(plain.mlstm(h[:11], mix, w, "l0.mix.", 1e-5), whole[:11], atol=1e-12)
    # by hand, the first token of one head: m = max(f + 0, i), S = exp(i - m) k v^T, n = exp(i - m) k
    H, d, dv, cap = mix["heads"], mix["dim"], mix["vdim"], mix["gate_cap"]
    x = h[:1]
    q = (x @ w["l0.mix.q"].double().t()).reshape(H, d)[0] * d ** -0.5
    k = (x @ w["l0.mix.k"].double().t()).reshape(H, d)[0]
    v = (x @ w["l0.mix.v"].double().t()).reshape(H, dv)[0]
    i = cap * torch.tanh(((x @ w["l0.mix.i"].double().t())[0, 0] + w["l0.mix.i.b"].double()[0]) / cap)
    f = torch.nn.functional.logsigmoid(cap * torch.tanh(((x @ w["l0.mix.f"].double().t())[0, 0] + w["l0.mix.f.b"].double()[0]) / cap))
    m = torch.maximum(f, i)
    o = torch.exp(i - m) * (k @ q) * v / (torch.maximum((torch.exp(i - m) * (k @ q)).abs(), torch.exp(-m)) + 1e-6)
    o = o / torch.sqrt((o * o).mean() + 1e-5) * w["l0.mix.norm"].double()[:dv] * torch.sigmoid(x @ w["l0.mix.g"].double().t())[0, :dv]
    got = plain.mlstm(x, mix, {**w, "l0.mix.o": torch.eye(H * dv)}, "l0.mix.", 1e-5)
    assert torch.allclose(got[0, :dv], o, atol=1e-10)


def test_plain_router_takes_the_largest_logits_and_weighs_them_alone(tmp_path):
    cfg, w = plain_inputs(make_gavatar_dir(tmp_path, "gav_moe"))
    h = torch.randn(7, 48, dtype=torch.float64)
    ids, wts = plain.route(h, cfg["layers"][0]["mlp"]["router"], w, "l0.mlp.")
    z = h @ w["l0.mlp.router"].double().t() + w["l0.mlp.router.b"].double()
    for t in range(7):
        order = sorted(range(9), key=lambda e: -float(z[t, e]))[:4]
        assert ids[t].tolist() == order
        e = torch.exp(z[t, order] - z[t, order[0]])
        assert torch.allclose(wts[t], e / e.sum()) and float(wts[t].sum()) == pytest.approx(1.0)


def test_every_mechanism_matters_in_the_test_models(tmp_path):
    """Leaving a mechanism out of the plain model moves its logits: a test model in which it did not would not test it."""
    folder = make_gavatar_dir(tmp_path, "gav_a")
    cfg, w = plain_inputs(folder)
    toks = random_tokens(cfg["vocab"], 60, 9)
    base = plain.forward(cfg, w, toks)

    def moved(cfg2=None, w2=None, tokens=None):
        other = plain.forward(cfg2 or cfg, w2 or w, tokens or toks)
        return float(((other - base).norm(dim=-1) / base.norm(dim=-1)).max())

    c = copy.deepcopy(cfg); c["loop"]["times"] = 2
    assert moved(c) > 0.05
    c = copy.deepcopy(cfg); c["embedding"]["scale"] = 1.0
    assert moved(c) > 0.05
    c = copy.deepcopy(cfg); c["layers"][0]["mixer"]["mask"]["size"] = 22
    assert moved(c) > 0.003
    c = copy.deepcopy(cfg); c["layers"][2]["mixer"]["mask"]["size"] = 12
    assert moved(c) > 0.003
    c = copy.deepcopy(cfg); c["layers"][1]["mixer"]["gate_cap"] = 2.0
    assert moved(c) > 0.01
    c = copy.deepcopy(cfg); c["layers"][0]["mlp"]["router"]["top"] = 3
    assert moved(c) > 0.01
    zero = (".b", ".shift", ".sink", "loop.step")
    for name in ("l0.mix.q.b", "l0.mix.v.b", "l0.shift", "l1.shift", "l2.mix.sink", "loop.step", "l1.mix.i.b", "l1.mix.f.b",
                 "l0.mlp.router.b", "l0.mix.talk", "l2.mix.dq.norm", "l2.mix.dkv.norm", "l1.mix.norm", "l0.norm1b", "l0.norm2b"):
        w2 = dict(w)
        if name.endswith(".talk"):
            w2[name] = torch.eye(w[name].shape[0])
        elif name.endswith(zero) or name.endswith(("norm1b", "norm2b")):
            w2[name] = torch.zeros_like(w[name])
        else:
            w2[name] = torch.ones_like(w[name])
        assert moved(w2=w2) > 0.003, name
    # the position vector: the same tokens one place later give other logits even where no layer could tell
    cfg1, w1 = plain_inputs(make_gavatar_dir(tmp_path, "gav_moe"))
    t1 = random_tokens(cfg1["vocab"], 6, 2)
    a, b = plain.forward(cfg1, w1, t1[:1]), plain.forward(cfg1, w1, [t1[3], t1[0]])
    assert float((a[0] - b[1]).abs().max()) > 1e-3
