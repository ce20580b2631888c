"""The Gavatar family on the GPU against the plain implementation: each new kernel alone, each mechanism alone in a
one-layer model, whole prompts against token-by-token decoding and portions down to two tokens, batches of unequal
requests with pages and state slots used again, the first tokens of a sequence, keys just inside and just outside a
window in prompts and in decoding (in every attention kernel, with a sink), a far key that must stand out, long
decoding, greedy generation through the engine and its scheduler, the command line and the trace replay.  Every test
runs in 32-bit and in bfloat16."""

import copy
import math
import os
import subprocess
import sys

import pytest
import torch

import plain_gavatar as plain
from gavatar_models import MODELS, make_gavatar_dir
import helpers
from helpers import BF16_NEAR_TIE, plain_inputs, random_tokens, run_trace
from test_gpu_fovunex import NEAR_TIE_NOISE, Ref, close, dev_i32, k, load, stepped
from test_gpu_fovunex import assert_close as assert_rows_close

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = ["float32", "bfloat16"]
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


# A router picks the experts with the largest logits: where the last one chosen lies barely above the best one left
# out, rounding decides which of two experts a token runs, and the row (and, through the shifted input, the next one)
# says nothing about the engine.  Such rows are left out of the comparison: a gap below this share of the logits'
# spread.  What is left must still be a good part of every sequence.
CLOSE_CALL = {"float32": 2e-4, "bfloat16": 0.04}


class GavRef(Ref):
    def __init__(self, logits, noise=None, keep=None):
        super().__init__(logits, noise)
        self.keep = keep if keep is not None else torch.ones(logits.shape[0], dtype=torch.bool)

    def __getitem__(self, idx):
        return GavRef(self.logits[idx], None if self.noise is None else self.noise[idx], self.keep[idx])


def reference(w, cfg, toks, dtype):
    """The plain model's logits, for bfloat16 how far rounding alone moves each row (the plain model with bfloat16
    rounding where the engine rounds, against itself without: a row's bound is made of that), and which rows rest on
    no close call of a router."""
    gaps = []
    logits = plain.forward(cfg, w, toks, gaps=gaps)
    keep = torch.ones(len(toks), dtype=torch.bool)
    if gaps:
        keep = torch.stack(gaps).min(dim=0).values >= CLOSE_CALL[dtype]
        keep[1:] &= keep[:-1].clone()
    if dtype == "float32":
        return GavRef(logits, None, keep)
    rounded = plain.forward(cfg, w, toks, round_to=torch.bfloat16)
    return GavRef(logits, (rounded - logits).norm(dim=-1) / logits.norm(dim=-1).clamp_min(1e-6), keep)


def assert_close(got, ref, dtype, what="", noise=1.0):
    got = got.double().cpu()
    assert got.shape == ref.logits.shape and torch.isfinite(got).all(), what
    keep = ref.keep
    assert int(keep.sum()) >= max(1, keep.numel() // 4), f"{what}: only {int(keep.sum())} of {keep.numel()} rows rest on no close call"
    assert_rows_close(got[keep], Ref(ref.logits[keep], None if ref.noise is None else ref.noise[keep]), dtype, what, noise)


def routers_for(dtype):
    """In bfloat16 the input of a router carries the rounding of everything before it, and with random routers every
    sequence of some length has a close call whose other outcome reaches all later rows through the states.  The
    bfloat16 runs of the whole models therefore use routers that decide by a wide margin (biases a unit apart over a
    small token-dependent part; the weights of the chosen experts still follow the token); the 32-bit runs keep the
    random routers, whose choices change from token to token, and the route kernel is tested alone."""
    if dtype != "bfloat16":
        return None

    def fix(t):
        g = torch.Generator().manual_seed(17)
        for name in list(t):
            if name.endswith(".router"):
                t[name] = (t[name].float() * 0.03).to(t[name].dtype)
            elif name.endswith(".router.b"):
                n = t[name].numel()
                t[name] = (torch.arange(n, dtype=torch.float32)[torch.randperm(n, generator=g)] - n / 2).to(t[name].dtype)
    return fix


def steady_tokens(cfg, w, n: int, seed: int) -> list[int]:
    """``n`` random tokens on which the model is well conditioned: the plain model in 32-bit agrees with itself in
    64-bit well within the bound that any implementation gets (a router's close call between two experts, or a gate at
    the edge of its cap, would otherwise decide a test)."""
    for s in range(seed, seed + 50):
        toks = random_tokens(cfg["vocab"], n, s)
        a, b = plain.forward(cfg, w, toks), plain.forward_float32(cfg, w, toks)
        if float((a - b).abs().max()) <= 0.25 * helpers.tolerance("float32", a):
            return toks
    raise AssertionError("no well-conditioned sequence in 50 seeds")


# =============================================================== kernels alone
@pytest.mark.parametrize("dtype", DTYPES)
def test_stream_kernels(dtype):
    """The scaled embedding plus the position vector at positions near and far, a row added to every token, and gates per
    coordinate and per head on rows with a stride."""
    dt = TORCH[dtype]
    g = torch.Generator().manual_seed(3)
    for n, d in ((7, 37), (5, 64)):
        x = torch.randn(n, d, generator=g)
        pos = torch.tensor([0, 1, 2, 77, 1000, 4097, 100000][:n], dtype=torch.int32)
        xd = x.to(DEV)
        k().scale_add_sinusoid(xd, pos.to(DEV), 3.5, 10000.0)
        want = x.double() * 3.5 + plain.sinusoid(pos, d)
        assert torch.allclose(xd.double().cpu(), want, atol=3e-6)
        row = torch.randn(d, generator=g).to(dt)
        k().add_row(xd, row.to(DEV))
        assert torch.allclose(xd.double().cpu(), want + row.double(), atol=3e-6)
    for group, d, pad, gpad in ((1, 30, 5, 3), (6, 30, 5, 3), (10, 40, 5, 3), (1, 64, 8, 8), (16, 64, 8, 3)):   # the last two: 16-byte forms
        buf = torch.randn(9, d + pad, generator=g).to(dt)
        gate = torch.randn(9, d // group + gpad, generator=g).to(dt)
        bd = buf.to(DEV)
        k().gate_mul(bd[:, :d], gate.to(DEV)[:, :d // group], group=group)
        want = buf.double()[:, :d] * torch.sigmoid(gate.double()[:, :d // group]).repeat_interleave(group, dim=1)
        assert close(bd[:, :d], want, dtype, rel=1e-2) and torch.equal(bd[:, d:].cpu(), buf[:, d:])


@pytest.mark.parametrize("dtype", DTYPES)
def test_norm_into_the_residual_with_the_norm_that_follows(dtype):
    """residual += norm(y) * gain and, in the same kernel, the next norm of the new residual."""
    dt = TORCH[dtype]
    g = torch.Generator().manual_seed(9)
    for n, d in ((5, 37), (9, 192), (3, 2048)):
        res, y = torch.randn(n, d, generator=g), (torch.randn(n, d + 3, generator=g) * 2).to(dt)
        g1, g2 = 1 + 0.3 * torch.randn(d, generator=g), 1 + 0.3 * torch.randn(d, generator=g)
        rd, out = res.to(DEV), torch.empty(n, d, dtype=dt, device=DEV)
        k().outnorm_accumulate_norm(rd, y.to(DEV)[:, :d], g1.to(DEV), 1e-5, g2.to(DEV), 1e-6, out)
        want_res = res.double() + plain.rms(y.double()[:, :d], 1e-5) * g1.double()
        assert torch.allclose(rd.double().cpu(), want_res, atol=2e-5, rtol=2e-5)
        assert close(out, plain.rms(want_res, 1e-6) * g2.double(), dtype, rel=1e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d", [45, 64])                   # rows that take the 16-byte form in bfloat16, and rows that do not
def test_token_shift_carries_the_last_row_over_any_cut(dtype, d):
    """Three requests of unequal length in slots out of order; whole, cut into portions (down to one token) and with a
    request left out of a step, the shifted rows are the same; a new request in a used slot starts from zeros when the
    slot was cleared."""
    dt = TORCH[dtype]
    g = torch.Generator().manual_seed(5)
    lens, slots = [13, 1, 6], [2, 0, 3]
    mu = torch.rand(d, generator=g).to(dt)
    hs = [torch.randn(L, d, generator=g).to(dt) for L in lens]
    wants = [plain.token_shift(h.double(), mu.double()) for h in hs]

    def run(plan):
        state = torch.zeros(4, d, dtype=dt, device=DEV)
        done = [0] * 3
        got = [[] for _ in lens]
        for step in plan:                       # step: {request: tokens}
            reqs = [r for r in range(3) if step.get(r)]
            rows = torch.cat([hs[r][done[r]:done[r] + step[r]] for r in reqs]).to(DEV)
            starts = [0]
            for r in reqs:
                starts.append(starts[-1] + step[r])
            out = torch.empty_like(rows)
            k().token_shift(rows, out, mu.to(DEV), state, dev_i32(starts), dev_i32([done[r] for r in reqs]),
                            dev_i32([slots[r] for r in reqs]), len(reqs))
            for i, r in enumerate(reqs):
                got[r].append(out[starts[i]:starts[i + 1]].cpu())
                done[r] += step[r]
        return [torch.cat(x) for x in got], state

    whole, state = run([{0: 13, 1: 1, 2: 6}])
    cut, state2 = run([{0: 5, 2: 1}, {0: 1, 1: 1}, {0: 2, 2: 3}, {2: 2, 0: 5}])
    for r in range(3):
        assert close(whole[r], wants[r], dtype, rel=1e-2), r
        assert torch.equal(whole[r], cut[r]), r
        assert torch.equal(state[slots[r]].cpu(), hs[r][-1]) and torch.equal(state2[slots[r]].cpu(), hs[r][-1])
    assert float(state[1].abs().max()) == 0.0                     # a slot nobody held


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, kv, hd, hdv, wide_row", [(4, 2, 16, 24, True), (3, 3, 12, 12, False), (5, 1, 10, 6, True)])
def test_qkv_prepare_kernel(dtype, heads, kv, hd, hdv, wide_row):
    dt = TORCH[dtype]
    g = torch.Generator().manual_seed(heads)
    n, ps, eps = 11, 4, 1e-5
    width = heads * hd + kv * hd + kv * hdv
    buf = torch.randn(n, width + 3, generator=g).to(dt)
    qb, kb, vb = (torch.randn(w_, generator=g).to(dt) for w_ in (heads * hd, kv * hd, kv * hdv))
    slots = torch.randperm(6 * ps, generator=g)[:n].to(torch.int32)
    slots[4] = -1                                                  # padding: nothing is stored
    pool_v = 1 if wide_row else kv
    kpool = torch.zeros(6, kv, ps, hd, dtype=dt, device=DEV)
    vpool = torch.zeros(6, pool_v, ps, kv * hdv // pool_v, dtype=dt, device=DEV)
    bd = buf.to(DEV)
    a, b = heads * hd, heads * hd + kv * hd
    k().qkv_prepare(bd[:, :a], heads, bd[:, a:b], kv, hd, bd[:, b:width], kv, hdv, slots.to(DEV), kpool, vpool, ps, eps,
                    q_bias=qb.to(DEV), k_bias=kb.to(DEV), v_bias=vb.to(DEV), q_norm=True, k_norm=True, v_norm=True,
                    pool_v_heads=pool_v)
    x = buf.double()
    q = plain.rms((x[:, :a] + qb.double()).reshape(n, heads, hd), eps)
    kk = plain.rms((x[:, a:b] + kb.double()).reshape(n, kv, hd), eps)
    v = plain.rms((x[:, b:width] + vb.double()).reshape(n, kv, hdv), eps)
    assert close(bd[:, :a], q.reshape(n, -1), dtype, rel=1e-2) and torch.equal(bd[:, width:].cpu(), buf[:, width:])
    for t in range(n):
        s = int(slots[t])
        if s < 0:
            continue
        assert close(kpool[s // ps, :, s % ps], kk[t], dtype, rel=1e-2)
        assert close(vpool[s // ps, :, s % ps].reshape(kv, hdv), v[t], dtype, rel=1e-2)
    assert int((kpool != 0).any(dim=-1).sum()) == (n - 1) * kv


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, kv, hdv, slice_heads, gated, pad", [(4, 2, 24, 2, True, 8), (6, 3, 8, 2, True, 2), (5, 1, 6, 1, False, 2),
                                                                    (3, 3, 10, 1, True, 2), (8, 2, 16, 1, False, 8)])
def test_talk_combine_kernel(dtype, heads, kv, hdv, slice_heads, gated, pad):
    """Every query head's weights applied to every value head, mixed into the heads' outputs, in slices of value heads."""
    dt = TORCH[dtype]
    g = torch.Generator().manual_seed(heads * 10 + kv)
    n, rep = 9, heads // kv
    a = torch.randn(n, heads, kv, hdv, generator=g).to(dt)
    talk = torch.randn(heads, heads, generator=g)
    gate = torch.randn(n, heads * hdv, generator=g).to(dt)
    out = torch.zeros(n, heads * hdv + pad, dtype=dt, device=DEV)      # a pad of 8 keeps rows on 16 bytes (the vector form)
    for c0 in range(0, kv, slice_heads):
        nc = min(slice_heads, kv - c0)
        part = a[:, :, c0:c0 + nc].reshape(n, heads * nc * hdv).to(DEV)
        k().talk_combine(part, talk.to(DEV), gate.to(DEV) if gated else None, out[:, :heads * hdv], heads, kv, hdv,
                         first_v_head=c0, slice_v_heads=nc)
    own = torch.stack([a.double()[:, :, h // rep] for h in range(heads)], dim=1)            # [n, h, g, hdv]
    want = torch.einsum("hg,nhgd->nhd", talk.double(), own).reshape(n, -1)
    if gated:
        want = want * torch.sigmoid(gate.double())
    assert close(out[:, :heads * hdv], want, dtype, rel=1e-2) and float(out[:, heads * hdv:].abs().max()) == 0.0


def plain_memory(q, kk, v, zi, zf, cap):
    """S^T q over its denominator for one head from zero state; q is already scaled.  Returns rows and (S, n, m)."""
    T, d = q.shape
    S, nn, m = torch.zeros(d, v.shape[1], dtype=torch.float64), torch.zeros(d, dtype=torch.float64), torch.zeros((), dtype=torch.float64)
    out = []
    for t in range(T):
        i = cap * torch.tanh(zi[t] / cap)
        f = plain.logsigmoid(cap * torch.tanh(zf[t] / cap))
        m2 = torch.maximum(f + m, i)
        a, b = torch.exp(f + m - m2), torch.exp(i - m2)
        S = a * S + b * kk[t][:, None] * v[t][None, :]
        nn = a * nn + b * kk[t]
        m = m2
        out.append(S.t() @ q[t] / (torch.maximum((nn @ q[t]).abs(), torch.exp(-m)) + 1e-6))
    return torch.stack(out), (S, nn, m)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, dk, dv", [(3, 8, 24), (2, 12, 20), (2, 32, 32), (1, 64, 128), (2, 40, 300), (1, 130, 16)])
def test_matrix_memory_kernel_carries_its_state_over_any_cut(dtype, heads, dk, dv):
    """Requests of unequal length in slots out of order, whole and in portions down to one token: the same rows to the
    last bit (the scan is sequential), and the plain recurrence's to rounding; head sizes that take one, several and
    many threads a column and one or several column chunks; gates from shut to wide open, capped."""
    dt = TORCH[dtype]
    g = torch.Generator().manual_seed(dk + dv)
    lens, slots, cap = [37, 1, 19], [3, 0, 1], 6.0
    words = k().mlstm_state_floats(dk, dv)
    data = []
    for L in lens:
        q = torch.randn(L, heads * dk, generator=g).to(dt)
        kk = (torch.randn(L, heads * dk, generator=g) * 0.7).to(dt)
        v = torch.randn(L, heads * dv, generator=g).to(dt)
        z = torch.randn(L, 2 * heads, generator=g) * 4.0
        data.append((q, kk, v, z))
    ib = torch.linspace(-1.0, 2.0, heads).to(dt)
    fb = torch.linspace(0.5, 4.0, heads).to(dt)

    def run(plan):
        state = torch.zeros(4, heads, words, dtype=torch.float32, device=DEV)
        done = [0] * 3
        got = [[] for _ in lens]
        for step in plan:
            reqs = [r for r in range(3) if step.get(r)]
            cat = lambda j: torch.cat([data[r][j][done[r]:done[r] + step[r]] for r in reqs]).to(DEV)
            starts = [0]
            for r in reqs:
                starts.append(starts[-1] + step[r])
            out = torch.empty(starts[-1], heads * dv, dtype=torch.float32, device=DEV)
            k().mlstm_scan(cat(0), cat(1), cat(2), cat(3), ib.to(DEV), fb.to(DEV), cap, state, out, dev_i32(starts),
                           dev_i32([slots[r] for r in reqs]), len(reqs), heads, dk, dv)
            for i, r in enumerate(reqs):
                got[r].append(out[starts[i]:starts[i + 1]].cpu())
                done[r] += step[r]
        return [torch.cat(x) for x in got], state.cpu()

    whole, state = run([{0: 37, 1: 1, 2: 19}])
    cut, state2 = run([{0: 5, 2: 1}, {0: 1, 1: 1}, {0: 17, 2: 16}, {2: 2, 0: 14}])
    assert torch.equal(state, state2)
    for r, L in enumerate(lens):
        assert torch.equal(whole[r], cut[r]), r
        q, kk, v, z = (x.double() for x in data[r])
        for h in range(heads):
            want, (S, nn, m) = plain_memory(q[:, h * dk:(h + 1) * dk] * dk ** -0.5, kk[:, h * dk:(h + 1) * dk],
                                            v[:, h * dv:(h + 1) * dv], z[:, h] + ib.double()[h], z[:, heads + h] + fb.double()[h], cap)
            got = whole[r][:, h * dv:(h + 1) * dv].double()
            assert torch.allclose(got, want, rtol=2e-4, atol=2e-4 * float(want.abs().max())), (r, h, float((got - want).abs().max()))
            st = state[slots[r], h].double()
            assert torch.allclose(st[:dk * dv].reshape(dk, dv), S, rtol=1e-4, atol=1e-4 * float(S.abs().max()) + 1e-7)
            chunks = (words - dk * dv) // (dk + 1)
            for c in range(chunks):                              # every chunk's copy of the normaliser and the maximum
                tail = st[dk * dv + c * (dk + 1):dk * dv + (c + 1) * (dk + 1)]
                assert torch.allclose(tail[:dk], nn, rtol=1e-4, atol=1e-6) and float(tail[dk]) == pytest.approx(float(m), abs=1e-5)
    # the finish: head norm, gain, sigmoid gate
    o = torch.randn(6, heads * dv, generator=g)
    gain, gate = torch.rand(heads * dv, generator=g).to(dt) + 0.5, torch.randn(6, heads * dv, generator=g).to(dt)
    out = torch.empty(6, heads * dv, dtype=dt, device=DEV)
    k().mlstm_finish(o.to(DEV), gain.to(DEV), gate.to(DEV), out, heads, dv, 1e-5)
    want = plain.rms(o.double().reshape(6, heads, dv), 1e-5).reshape(6, -1) * gain.double() * torch.sigmoid(gate.double())
    assert close(out, want, dtype, rel=1e-2)


def test_router_of_the_largest_logits():
    """The largest logits (bias added), ties to the lower index, weights the softmax over the chosen alone; one, some
    and all of the experts."""
    g = torch.Generator().manual_seed(2)
    for n_experts, top in ((16, 4), (5, 1), (3, 3), (70, 6)):
        z = torch.randn(33, n_experts + 2, generator=g) * 2
        z[5, 1] = z[5, 0]                                         # a tie
        bias = torch.randn(n_experts, generator=g)
        ids = torch.empty(33, top, dtype=torch.int32, device=DEV)
        wts = torch.empty(33, top, dtype=torch.float32, device=DEV)
        k().moe_route(z.to(DEV)[:, :n_experts], bias.to(DEV), ids, wts, None, n_experts, top, 1, 1, 1.0, 0.0, score="softmax_top")
        zz = z[:, :n_experts].double() + bias.double()
        for t in range(33):
            order = sorted(range(n_experts), key=lambda e: (-float(zz[t, e]), e))[:top]
            assert ids[t].tolist() == order, t
            e = torch.exp(zz[t, order] - zz[t, order[0]])
            assert torch.allclose(wts[t].double().cpu(), e / e.sum(), atol=1e-6)


@pytest.mark.parametrize("kernel", ["rows", "general", "wide", "wide_small"])
@pytest.mark.parametrize("layout", ["row_slice", "values_in_keys"])
def test_a_key_stands_out_only_inside_the_window_and_the_sink_takes_its_share(kernel, layout):
    """One key among hundreds dominates every score; a query sees it while it lies inside the window and not one
    position later, at edges that are no page or tile borders, with released pages poisoned; the sink's term joins the
    denominator once.  ``row_slice``: the values are a slice of a wider cached row that holds all value heads of a
    token; ``values_in_keys``: the first dimensions of the key row.  Every attention kernel, float32 kernels in both
    storage types."""
    for dt in ([torch.bfloat16] if kernel.startswith("wide") else [torch.float32, torch.bfloat16]):
        g = torch.Generator().manual_seed(13)
        ps, window, T, scale = 8, 43, 170, 0.5
        if layout == "row_slice":
            n_heads, n_k, hd, hdv, row, off = 8, 2, 16, 32, 96, 32           # value columns 32..63 of a row of 96
        else:
            n_heads, n_k, hd, hdv, row, off = 4, 1, 48, 32, 48, 0
        group = n_heads // n_k
        hot = 61
        kk = torch.randn(T, n_k, hd, generator=g) * 0.3
        q = torch.randn(T, n_heads, hd, generator=g) * 0.3
        direction = torch.randn(hd, generator=g)
        if layout == "values_in_keys":
            direction[:hdv] = 0
        direction /= direction.norm()
        kk[hot] += 30 * direction
        q += 2 * direction
        sink = torch.tensor([0.0, 3.0, -2.0, 1.0, 65.0, 0.5, -30.0, 2.0][:n_heads])
        kk, q = kk.to(dt), q.to(dt)
        vrow = kk[:, 0, :].clone() if layout == "values_in_keys" else torch.randn(T, row, generator=g).to(dt)
        n_pages = -(-T // ps)
        perm = torch.randperm(n_pages + 3, generator=g)[:n_pages]
        kpool = torch.full((n_pages + 3, n_k, ps, hd), float("nan"), dtype=dt)
        vpool = torch.full((n_pages + 3, 1, ps, row), float("nan"), dtype=dt)
        for t in range(T):
            kpool[perm[t // ps], :, t % ps] = kk[t]
            vpool[perm[t // ps], 0, t % ps] = vrow[t]
        qd, kd, vd = q.double(), kk.double(), vrow.double()[:, off:off + hdv]
        want = torch.zeros(T, n_heads, hdv, dtype=torch.float64)
        for t in range(T):
            lo = max(0, t - window + 1)
            for h in range(n_heads):
                s = (kd[lo:t + 1, h // group] @ qd[t, h]) * scale
                e = torch.exp(s - s.max())
                want[t, h] = (e / (e.sum() + torch.exp(sink[h].double() - s.max()))) @ vd[lo:t + 1]
        kp = kpool.to(DEV)
        vp = kp if layout == "values_in_keys" else vpool.to(DEV).view(n_pages + 3, ps, row)[:, :, off:]
        small = kernel in ("rows", "wide_small")
        qpos = [hot, hot + 1, hot + window - 2, hot + window - 1, hot + window, hot + window + 1, 150, 169, 7, 0] if small \
            else list(range(30, T))
        out = torch.empty(len(qpos), n_heads * hdv, dtype=dt, device=DEV)
        qrows = q[qpos].reshape(len(qpos), -1).to(DEV)
        extra = dict(v_head_dim=hdv, n_v_heads=1, v_row=row, sink=sink.to(DEV))
        table = perm.to(torch.int32)
        if small:
            R = len(qpos)
            tables = []
            for p in qpos:                       # pages wholly before the query's window are released
                t_ = table.clone()
                t_[:max(0, p - window + 1) // ps] = -1
                tables.append(t_)
            args = (qrows, out, kp, vp, torch.stack(tables).to(DEV), dev_i32(range(R + 1)), dev_i32(qpos), R, group,
                    n_heads, n_k, hd, ps, window, scale)
            if kernel == "rows":
                k().attention_rows(*args, **extra)
            else:
                n_splits, split_keys = k().attention_wide_splits(hd, hdv, window + 64, R * n_k)
                words = k().attention_wide_small_scratch(hd, hdv, R, group, n_k, n_splits)
                scratch = torch.empty(max(words, 1), dtype=torch.float32, device=DEV)
                k().attention_wide_small(*args, n_splits, split_keys, scratch, **extra)
        else:
            t_ = table.clone()
            t_[:max(0, 30 - window + 1) // ps] = -1
            rows = k().ATTENTION_WIDE_ROWS if kernel == "wide" else 32
            work = [(0, p0) for p0 in range(0, len(qpos) * group, rows)]
            fn = k().attention_wide if kernel == "wide" else k().attention_general
            fn(qrows, out, kp, vp, t_[None].to(DEV), dev_i32([0, len(qpos)]), dev_i32([30]), dev_i32([w_[0] for w_ in work]),
               dev_i32([w_[1] for w_ in work]), len(work), n_heads, n_k, hd, ps, window, scale, **extra)
        got = out.double().cpu().reshape(len(qpos), n_heads, hdv)
        assert torch.isfinite(got).all()
        name = "float32" if dt is torch.float32 else "bfloat16"
        for i, p in enumerate(qpos):
            assert close(got[i], want[p], name, rel=3e-2), (kernel, p, float((got[i] - want[p]).abs().max()))
            sees = hot <= p < hot + window
            near_hot = float((got[i, 0] - vd[hot]).abs().max()) < 0.05 * float(vd[hot].abs().max())
            assert near_hot == sees, (kernel, p, sees)
        # the sinks did something: head 4's (far above its scores elsewhere) leaves almost nothing where the key is not seen
        if n_heads > 4:
            i = qpos.index(150)
            assert float(got[i, 4].abs().max()) < 1e-3 and float(got[i, 6].abs().max()) > 1e-2


# =============================================================== whole models
LENGTH = {"gav_a": 97, "gav_b": 70, "gav_c": 131, "gav_w": 150, "gav_s": 80, "gav_att": 75, "gav_lat": 60, "gav_mem": 50,
          "gav_moe": 41}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(MODELS))
def test_whole_prompt_decoding_and_portions_agree_with_the_plain_model(tmp_path, name, dtype):
    folder = make_gavatar_dir(tmp_path, name, fix=routers_for(dtype))
    cfg, w = plain_inputs(folder)
    toks = steady_tokens(cfg, w, LENGTH[name], 21)
    ref = reference(w, cfg, toks, dtype)
    r = load(folder, dtype, page_size=8)
    T = len(toks)
    assert_close(stepped(r, "whole", toks, [T]), ref, dtype, f"{name}: whole")
    assert_close(stepped(r, "decode", toks, [T - 40] + [1] * 40), ref, dtype, f"{name}: decoded one by one")
    assert_close(stepped(r, "one", toks[:30], [1]), ref[:30], dtype, f"{name}: token by token from the start")
    assert_close(stepped(r, "cut", toks, [7, 2, 16, 3, 2, 17, 2, 31, 1, 5]), ref, dtype, f"{name}: portions")
    assert_close(stepped(r, "pairs", toks[:40], [2]), ref[:40], dtype, f"{name}: portions of two")
    r.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["gav_a", "gav_b", "gav_c", "gav_w"])
def test_unequal_requests_in_one_batch_with_pages_and_slots_used_again(tmp_path, name, dtype):
    """Seven requests, at most three live, portions of some beside decoded tokens of others, some left out of a step;
    the pool holds exactly what the fullest moment needs and free pages are filled with NaN."""
    import random
    from inf_engine_b200 import StepEntry

    folder = make_gavatar_dir(tmp_path, name, fix=routers_for(dtype))
    cfg, w = plain_inputs(folder)
    lengths = [45, 17, 80, 3, 33, 64, 1]
    reqs = {f"q{i}": steady_tokens(cfg, w, n, 40 + 100 * i) for i, n in enumerate(lengths)}
    refs = {rid: reference(w, cfg, t, dtype) for rid, t in reqs.items()}
    rng = random.Random(7)
    plan, waiting, live = [], list(reqs), {}
    while waiting or live:
        while waiting and len(live) < 3:
            rid = waiting.pop(0)
            live[rid] = [0, max(1, len(reqs[rid]) - rng.choice([2, 6, 12]))]
        step, ended = [], []
        for rid, st in list(live.items()):
            if rng.random() < 0.25 and len(live) > 1:
                continue
            n = 1 if st[0] >= st[1] else min(rng.choice([2, 3, 5, 11, 24]), st[1] - st[0])
            step.append((rid, st[0], n))
            st[0] += n
            if st[0] == len(reqs[rid]):
                ended.append(rid)
                del live[rid]
        if step:
            plan.append((step, ended))
    ps = 8
    held, most = {}, 0
    for step, ended in plan:
        for rid, p, n in step:
            held[rid] = -(-(p + n) // ps)
        most = max(most, sum(held.values()))
        for rid in ended:
            held.pop(rid)
    r = load(folder, dtype, page_size=ps, n_pages=max(most, 1), max_requests=3, poison_free_pages=True)
    got = {rid: [] for rid in reqs}
    slots_seen = {}
    for step, ended in plan:
        for rid, p, n in step:
            if not r.is_open(rid):
                assert r.open(rid)
                slots_seen[rid] = r.cache.slots[rid]
        lg = r.step([StepEntry(rid, reqs[rid][p:p + n], list(range(n))) for rid, p, n in step]).cpu()
        at = 0
        for rid, p, n in step:
            got[rid].append(lg[at:at + n].clone())
            at += n
        for rid in ended:
            r.close(rid)
        r.cache.check()
    assert len(set(slots_seen.values())) <= 3 < len(slots_seen)              # slots were used again
    for rid in reqs:
        assert_close(torch.cat(got[rid]), refs[rid], dtype, f"{name}: {rid} in mixed batches")


@pytest.mark.parametrize("dtype", DTYPES)
def test_first_tokens_of_a_sequence_and_a_slot_that_another_request_held(tmp_path, dtype):
    """Sequences of one, two and three tokens in one batch; then new requests in the slots they held: what the old
    requests left there (matrix memories with their maxima, last input rows, of every pass) must not reach the new ones."""
    from inf_engine_b200 import StepEntry

    folder = make_gavatar_dir(tmp_path, "gav_a", fix=routers_for(dtype))
    cfg, w = plain_inputs(folder)
    r = load(folder, dtype, max_requests=3)
    first = {"a": random_tokens(211, 1, 1), "b": random_tokens(211, 2, 100), "c": random_tokens(211, 3, 200)}
    for rid in first:
        r.open(rid)
    lg = r.step([StepEntry(rid, t, list(range(len(t)))) for rid, t in first.items()]).cpu()
    at = 0
    for rid, t in first.items():
        assert_close(lg[at:at + len(t)], reference(w, cfg, t, dtype), dtype, f"first tokens of {rid}")
        at += len(t)
    more = [9, 9, 120]
    for i, tok in enumerate(more):
        lg = r.step([StepEntry("b", [tok], [0])]).cpu()
        assert_close(lg, reference(w, cfg, first["b"] + more[:i + 1], dtype)[-1:], dtype, "second and later tokens")
    for rid in first:
        r.close(rid)
    second = {"d": random_tokens(211, 9, 300), "e": random_tokens(211, 1, 400), "f": random_tokens(211, 2, 500)}
    for rid in second:
        r.open(rid)
    lg = r.step([StepEntry(rid, t, list(range(len(t)))) for rid, t in second.items()]).cpu()
    at = 0
    for rid, t in second.items():
        assert_close(lg[at:at + len(t)], reference(w, cfg, t, dtype), dtype, f"{rid} in a slot used before")
        at += len(t)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["gav_att", "gav_b", "gav_c", "gav_w"])
def test_edges_of_the_windows_in_prompts_and_in_decoding(tmp_path, name, dtype):
    """The attention is made sharp (a larger score scale) so that one key more or less changes the logits far beyond
    rounding; the sequence runs over several windows, in pages of 8, so that pages behind a window are given back."""
    config = copy.deepcopy(MODELS[name])
    for L in config["layers"]:
        if "mask" in L["mixer"]:
            L["mixer"]["scale"] *= 6.0 if L["type"] == "attention" else 2.5
    folder = make_gavatar_dir(tmp_path, name, config=config, fix=routers_for(dtype))
    cfg, w = plain_inputs(folder)
    sizes = [L["mixer"]["mask"]["size"] for L in cfg["layers"] if "mask" in L["mixer"]]
    size = max(sizes)
    toks = steady_tokens(cfg, w, 3 * size + 5, 8)
    ref = reference(w, cfg, toks, dtype)
    # the faults this must catch: a window one position longer or shorter
    for delta in (1, -1):
        other = copy.deepcopy(cfg)
        for L in other["layers"]:
            if "mask" in L["mixer"]:
                L["mixer"]["mask"]["size"] += delta
        wrong = plain.forward(other, w, toks)
        moved = (wrong - ref.logits).norm(dim=-1).div(ref.logits.norm(dim=-1))[min(sizes) - 1:]
        assert float(moved.max()) > 0.02, (delta, float(moved.max()))
    r = load(folder, dtype, page_size=8)
    noise = 1.5
    assert_close(stepped(r, "whole", toks, [len(toks)]), ref, dtype, f"{name}: window edges in a prompt", noise=noise)
    assert_close(stepped(r, "decode", toks, [3] + [1] * (len(toks) - 3)), ref, dtype, f"{name}: window edges in decoding", noise=noise)
    assert_close(stepped(r, "cut", toks, [size - 1, 2, 1, 1, 5, 11]), ref, dtype, f"{name}: portions around a window's length", noise=noise)
    assert_close(stepped(r, "cut2", toks, [size, size + 1, 2]), ref, dtype, f"{name}: portions as long as a window", noise=noise)
    r.cache.check()
    for g in r.cache.kv_groups:
        assert g.pool.n_free == g.pool.n_pages


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("windows", [(1, 2), (2, 1), (500, 8)])
def test_the_shortest_windows_and_one_longer_than_the_sequence(tmp_path, dtype, windows):
    """A window of one key (a token sees itself alone), of two, and one that no sequence of the test fills, on either
    kind of attention, in a prompt, decoded and in portions of two."""
    from gavatar_models import _att, _lat, _model, _moe
    config = _model(90, 48, 1e-5, 1.5, [_att(4, 2, 12, 8, 0.5, windows[0], None), _lat(2, 12, 8, 10, 16, 0.5, windows[1], _moe(3, 1, 20))])
    folder = make_gavatar_dir(tmp_path, "windows", config=config, fix=routers_for(dtype))
    cfg, w = plain_inputs(folder)
    toks = steady_tokens(cfg, w, 45, 5)
    ref = reference(w, cfg, toks, dtype)
    r = load(folder, dtype, page_size=8)
    assert_close(stepped(r, "whole", toks, [45]), ref, dtype, f"windows {windows}: whole")
    assert_close(stepped(r, "decode", toks, [5] + [1] * 40), ref, dtype, f"windows {windows}: decoded")
    assert_close(stepped(r, "pairs", toks, [2]), ref, dtype, f"windows {windows}: portions of two")
    r.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_far_key_is_found_by_the_latent_attention(tmp_path, dtype):
    """A latent attention without a window, made sharp; the test first shows that swapping one token 250 and more
    positions back moves the last positions' plain logits, then the engine must agree with the plain model there, in a
    prompt and decoded (the kernels alone are tested with a key that dominates)."""
    config = copy.deepcopy(MODELS["gav_lat"])
    config["layers"][0]["mixer"]["scale"] *= 3.0
    folder = make_gavatar_dir(tmp_path, "gav_lat", config=config)
    cfg, w = plain_inputs(folder)
    toks = steady_tokens(cfg, w, 300, 12)
    ref = reference(w, cfg, toks, dtype)
    swapped = list(toks)
    swapped[5] = (toks[5] + 17) % cfg["vocab"]
    moved = (plain.forward(cfg, w, swapped)[250:] - ref.logits[250:]).norm(dim=-1) / ref.logits[250:].norm(dim=-1)
    assert float(moved.max()) > 1e-3
    r = load(folder, dtype, page_size=8, n_pages=80)
    assert_close(stepped(r, "whole", toks, [300]), ref, dtype, "far key in a prompt", noise=1.5)
    assert_close(stepped(r, "decode", toks, [250] + [1] * 50), ref, dtype, "far key in decoding", noise=1.5)


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(tmp_path, dtype):
    """Four tokens of prompt and 200 decoded one by one through the decode graphs: the matrix memories of every pass,
    the last input rows and both caches are carried over 200 steps, past every window."""
    folder = make_gavatar_dir(tmp_path, "gav_a", fix=routers_for(dtype))
    cfg, w = plain_inputs(folder)
    toks = steady_tokens(cfg, w, 204, 77)
    ref = reference(w, cfg, toks, dtype)
    r = load(folder, dtype, page_size=8)
    got = stepped(r, "long", toks, [4] + [1] * 200)
    assert r.graphs.replays >= 150
    assert_close(got, ref, dtype, "long decoding")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["gav_a", "gav_c"])
def test_greedy_generation_through_the_entry_point(tmp_path, name, dtype):
    """``Engine.run_offline``: scheduler, portions of prompts under a token budget, decode graphs, device sampling.
    Every generated token must be the plain model's choice (or tie with it within bfloat16's noise)."""
    from inf_engine_b200 import Engine, Request

    folder = make_gavatar_dir(tmp_path, name, fix=routers_for(dtype))
    cfg, w = plain_inputs(folder)
    prompts = [random_tokens(cfg["vocab"], n, 60 + 100 * n) for n in (3, 41, 18, 1, 70)]
    outs = []
    for pipeline in (True, False):
        engine = Engine.from_dir(folder, dtype=dtype, n_total_blocks=24, block_size=8, max_requests=3,
                                 max_tokens_per_step=32, chunk=13, pipeline=pipeline)
        out = engine.run_offline([Request(i, p, max_new_tokens=10) for i, p in enumerate(prompts)])
        engine.runner.cache.check()
        assert engine.runner.cache.n_open == 0 and engine.runner.graphs.replays > 0
        outs.append(out)
        for i, p in enumerate(prompts):
            assert len(out[i]) == 10
            logits = plain.forward(cfg, w, p + out[i])
            for j, tok in enumerate(out[i]):
                row = logits[len(p) + j - 1]
                slack = 0.0 if dtype == "float32" else BF16_NEAR_TIE * NEAR_TIE_NOISE * max(1.0, float(row.abs().max()))
                assert float(row.max() - row[tok]) <= slack, f"{name} {dtype}: request {i}, token {j}"
    if dtype == "float32":
        assert outs[0] == outs[1]


def test_command_line_and_trace_replay(tmp_path):
    folder = make_gavatar_dir(tmp_path, "gav_b")
    cfg, w = plain_inputs(folder)
    prompt = random_tokens(cfg["vocab"], 12, 5)
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "generate_llama"), "--model-dir", str(folder),
                           "--prompt-ids", ",".join(map(str, prompt)), "--n", "6", "--dtype", "float32"],
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    ids = [int(t) for t in proc.stdout.strip().splitlines()[-1].split(": ")[1].split(",")]
    logits = plain.forward(cfg, w, prompt + ids)
    assert ids == [int(logits[len(prompt) + j - 1].argmax()) for j in range(6)]
    from test_gpu_replay import schedules
    for dtype in DTYPES:
        (tmp_path / dtype).mkdir()
        folder = make_gavatar_dir(tmp_path / dtype, "gav_b", fix=routers_for(dtype))
        cfg, w = plain_inputs(folder)
        requests = {str(i): steady_tokens(cfg, w, n, 300 + 50 * i) for i, n in enumerate([70, 45, 130, 20, 97, 33])}
        trace = schedules("gav", requests, seed=3)
        got = run_trace(folder, dtype, trace, tmp_path / f"out_{dtype}", cfg["vocab"], page_size=8)
        refs = {rid: reference(w, cfg, t, dtype) for rid, t in requests.items()}
        for prefix in "wdpm":
            for rid, t in requests.items():
                rows = [got.get((prefix + rid, p)) for p in range(len(t))]
                if rows[0] is None:
                    continue
                assert_close(torch.stack(rows), refs[rid], dtype, f"replay {prefix}{rid}")
