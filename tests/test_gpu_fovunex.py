"""The Fovunex family on the GPU against the plain implementation: each new kernel alone, each mechanism alone in a
one-layer model, whole prompts against token-by-token decoding and portions down to two tokens, batches of unequal
requests with pages and state slots used again, the first tokens of a sequence, keys just inside and just outside a
chunk in prompts and in decoding, a far key that must stand out, long decoding, greedy generation through the engine
and its scheduler, the command line and the trace replay.  Every test runs in 32-bit and in bfloat16."""

import copy
import math
import os
import subprocess
import sys

import pytest
import torch

import plain_fovunex as plain
from fovunex_models import MODELS, make_fovunex_dir
import helpers
from helpers import BF16_NEAR_TIE, plain_inputs, random_tokens, run_trace

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = ["float32", "bfloat16"]
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# bfloat16: a differential head's output a1 - lambda a2 is divided by its own root mean square; where the two maps
# nearly agree (the first tokens of a sequence or of a chunk, above all) the rounding of its inputs enters at full
# size, and no fixed bound tells that from a fault.  So a row's bound is three times the error that rounding alone
# causes there (the plain model with bfloat16 rounding where the engine rounds, against itself without) plus a floor.
# That error is one draw of a heavy-tailed quantity on such rows (measured on a B200: over a request the engine's mean
# error equals the mean of rounding alone, 0.037 against 0.031, 0.013 against 0.012, 0.012 against 0.013, while single
# rows right after a sharp differential layer reach 1.3 times their bound), so one row in fifty (one at least) may
# exceed its bound, none by more than a factor of 2.5, and the mean over a request's rows is bounded as well.
F32_NOISE = 2.0
BF16_FLOOR = 0.03
NEAR_TIE_NOISE = 4.0


class Ref:
    def __init__(self, logits, noise=None):
        self.logits, self.noise = logits, noise

    def __getitem__(self, idx):
        return Ref(self.logits[idx], None if self.noise is None else self.noise[idx])


def reference(w, cfg, toks, dtype):
    logits = plain.forward(cfg, w, toks)
    if dtype == "float32":
        return Ref(logits)
    rounded = plain.forward(cfg, w, toks, round_to=torch.bfloat16)
    return Ref(logits, (rounded - logits).norm(dim=-1) / logits.norm(dim=-1).clamp_min(1e-6))


def assert_close(got, ref, dtype, what="", noise=1.0):
    got, want = got.double().cpu(), ref.logits.double().cpu()
    assert got.shape == want.shape and torch.isfinite(got).all(), what
    if dtype == "float32":
        tol = F32_NOISE * helpers.tolerance(dtype, want)
        worst = float((got - want).abs().max())
        helpers.STATS.append({"what": what, "dtype": dtype, "max_abs": worst, "tol": tol})
        assert worst <= tol, f"{what}: max |diff| {worst:.3e} > {tol:.3e}; worst row {int((got - want).abs().max(dim=-1).values.argmax())}"
        return
    rel = (got - want).norm(dim=-1) / want.norm(dim=-1).clamp_min(1e-6)
    bound = noise * (3.0 * ref.noise + BF16_FLOOR)
    helpers.STATS.append({"what": what, "dtype": dtype, "rows": int(rel.numel()), "row_max": float(rel.max()),
                          "row_mean": float(rel.mean()), "worst_of_bound": float((rel / bound).max())})
    bad = (rel > bound).nonzero().flatten().tolist()
    far = (rel > 2.5 * bound).nonzero().flatten().tolist()
    assert len(bad) <= max(1, rel.numel() // 50) and not far, (
        f"{what}: relative error of row {bad[0]} is {float(rel[bad[0]]):.3e} > {float(bound[bad[0]]):.3e} "
        f"(rounding alone: {float(ref.noise[bad[0]]):.3e}; rows over their bound: {bad[:20]}; far over: {far[:20]})")
    if rel.numel() >= 8:
        assert float(rel.mean()) <= noise * (2.0 * float(ref.noise.mean()) + BF16_FLOOR / 2), \
            f"{what}: mean relative row error {float(rel.mean()):.3e}, rounding alone {float(ref.noise.mean()):.3e}"


def k():
    from inf_engine_b200 import kernels
    return kernels


def dev_i32(x):
    return torch.as_tensor(x, dtype=torch.int32).to(DEV)


def close(got, want, dtype, rel=2e-2, atol=2e-5):
    """float32: element by element against the float64 oracle; bfloat16: against the largest value of the tensor."""
    got, want = got.double().cpu(), want.double().cpu()
    if dtype == "float32":
        return torch.allclose(got, want, atol=atol, rtol=2e-5)
    return float((got - want).abs().max()) <= rel * max(1.0, float(want.abs().max()))


# =============================================================== kernels alone
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("neighbours, q_hd, q_off, k_hd, k_off, k_norm, rot, yarn", [
    (True, 12, 8, 24, 20, 20, 4, (2.0, 16, 4.0, 1.0)),       # the latent layout: a part of every head, one wide key row
    (False, 16, 0, 16, 0, 16, 8, None),                       # halves of the first dimensions of whole-normed heads
    (False, 10, 0, 10, 0, 10, 0, None),                       # no rotation at all
    (True, 6, 0, 6, 0, 0, 6, (3.0, 24, 6.0, 0.5)),            # the whole head in neighbouring pairs, no norm
])
def test_head_prepare_kernel(dtype, neighbours, q_hd, q_off, k_hd, k_off, k_norm, rot, yarn):
    """Norm of the first dimensions, rotation at an offset in either layout at positions up to a million, cache write
    into scattered slots; a padding token (slot -1) writes nothing."""
    dt = TORCH[dtype]
    g = torch.Generator().manual_seed(3)
    n, qh, kh, vh, hdv, ps, pages = 7, 5, (1 if q_off else 2), 1, 6, 4, 6
    q = torch.randn(n, qh * q_hd + 3, generator=g).to(dt)
    kk = torch.randn(n, kh * k_hd + 5, generator=g).to(dt)
    v = torch.randn(n, vh * hdv, generator=g).to(dt)
    q_gain = (1 + torch.rand(q_hd, generator=g)).to(dt) if not q_off and k_norm else None
    k_gain = (1 + torch.rand(max(k_norm, 1), generator=g)).to(dt) if k_norm else None
    positions = [0, 1, 2, 77, 1000003, 5, 9]
    slots = [5, 0, 23, 9, 14, -1, 3]
    rd = {"base": 300.0, "dims": rot}
    if yarn:
        rd["scaling"] = dict(zip(("factor", "original", "fast", "slow"), yarn))
    eps = 1e-5

    def prep(x, heads, hd, off, gain, norm_dims):
        x = x.double()[:, :heads * hd].reshape(n, heads, hd).clone()
        if gain is not None:
            x[..., :norm_dims] = plain.rms(x[..., :norm_dims], eps) * gain.double()
        if rot:
            cos, sin = plain.rotation_angles(rd, torch.tensor(positions))
            fn = plain.rotate_interleaved if neighbours else plain.rotate_halves
            x[..., off:off + rot] = fn(x[..., off:off + rot], cos, sin)
        return x

    want_q = prep(q, qh, q_hd, q_off, q_gain, q_hd)
    want_k = prep(kk, kh, k_hd, k_off, k_gain, k_norm)
    kpool = torch.full((pages, kh, ps, k_hd), 7.0, dtype=dt, device=DEV)
    vpool = torch.full((pages, vh, ps, hdv), 7.0, dtype=dt, device=DEV)
    inv_freq = mult = None
    if rot:
        from inf_engine_b200.config import PositionSpec, YarnScaling
        from inf_engine_b200.parts.positions import partial_rotation_frequencies
        f, mult = partial_rotation_frequencies(PositionSpec(kind="rotary_partial", theta=300.0, rot_dims=rot,
                                                            yarn=YarnScaling(*map(float, yarn)) if yarn else None))
        inv_freq = f.to(DEV)
    qd, kd = q.to(DEV), kk.to(DEV)
    k().head_prepare(qd[:, :qh * q_hd], qh, q_hd, kd[:, :kh * k_hd], kh, k_hd, dev_i32(positions), dev_i32(slots), kpool, ps,
                     q_gain=q_gain.to(DEV) if q_gain is not None else None, q_norm_dims=q_hd,
                     k_gain=k_gain.to(DEV) if k_gain is not None else None, k_norm_dims=k_norm, eps=eps,
                     inv_freq=inv_freq, rot_dims=rot, q_rot_off=q_off, k_rot_off=k_off, neighbours=neighbours,
                     mult=mult or 1.0, v=v.to(DEV), vpool=vpool, n_v_heads=vh, v_head_dim=hdv)
    torch.cuda.synchronize()
    assert close(qd[:, :qh * q_hd].reshape(n, qh, q_hd), want_q, dtype)
    assert torch.equal(qd[:, qh * q_hd:].cpu(), q[:, qh * q_hd:])                       # columns beside the heads stay
    written = torch.zeros(pages * ps, dtype=torch.bool)
    for i, s in enumerate(slots):
        if s < 0:
            continue
        written[s] = True
        assert close(kpool[s // ps, :, s % ps], want_k[i], dtype), i
        assert torch.equal(vpool[s // ps, :, s % ps].cpu().reshape(-1), v[i])
    untouched = kpool.permute(0, 2, 1, 3).reshape(pages * ps, -1)[~written]
    assert bool((untouched == 7.0).all())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m, heads, kd, nd", [(1, 3, 12, 24), (19, 5, 14, 6), (70, 2, 40, 100)])
def test_heads_gemm_kernel(dtype, m, heads, kd, nd):
    dt = TORCH[dtype]
    g = torch.Generator().manual_seed(5)
    x = torch.randn(m, heads * (kd + 3) + 2, generator=g).to(dt)
    w = torch.randn(heads, kd, nd, generator=g).to(dt)
    out = torch.full((m, heads * (nd + 1) + 4), 9.0, dtype=dt, device=DEV)
    k().heads_gemm(x.to(DEV), kd + 3, w.to(DEV), out, nd + 1)
    for h in range(heads):
        want = x.double()[:, h * (kd + 3):h * (kd + 3) + kd] @ w[h].double()
        assert close(out[:, h * (nd + 1):h * (nd + 1) + nd], want, dtype)
        assert bool((out[:, h * (nd + 1) + nd] == 9.0).all())


@pytest.mark.parametrize("m, heads, kd, nd", [(64, 3, 12, 24), (150, 5, 14, 6), (300, 2, 48, 80), (5, 2, 16, 16)])
def test_per_head_product_of_prompt_portions_in_bfloat16(m, heads, kd, nd):
    """From 64 rows on the bfloat16 product goes to the library's batched product, read and written in place through
    strided rows (heads that are not packed, columns that must stay untouched); below that the kernel runs."""
    from inf_engine_b200.parts.latent import heads_product
    g = torch.Generator().manual_seed(6)
    x = torch.randn(m, heads * (kd + 3) + 2, generator=g).bfloat16()
    w = torch.randn(heads, kd, nd, generator=g).bfloat16()
    out = torch.full((m, heads * (nd + 1) + 4), 9.0, dtype=torch.bfloat16, device=DEV)
    out2 = out.clone()
    heads_product(x.to(DEV), kd + 3, w.to(DEV), out, nd + 1)
    k().heads_gemm(x.to(DEV), kd + 3, w.to(DEV), out2, nd + 1)
    for h in range(heads):
        want = x.double()[:, h * (kd + 3):h * (kd + 3) + kd] @ w[h].double()
        assert close(out[:, h * (nd + 1):h * (nd + 1) + nd], want, "bfloat16")
        assert bool((out[:, h * (nd + 1) + nd] == 9.0).all())
        # the two ways differ by the order of a float32 sum only: at most one bfloat16 step of the result
        d = (out[:, h * (nd + 1):h * (nd + 1) + nd].double() - out2[:, h * (nd + 1):h * (nd + 1) + nd].double()).abs().cpu()
        assert bool((d <= 2.0 ** -7 * want.abs().clamp(min=0.25)).all())
    assert bool((out[:, heads * (nd + 1):] == 9.0).all())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, kv, dv, gated", [(4, 2, 24, True), (3, 3, 12, False), (5, 1, 6, True), (2, 1, 80, True),
                                                  (6, 2, 32, True), (5, 5, 64, True), (3, 1, 128, False), (2, 2, 256, True)])
def test_diff_combine_kernel(dtype, heads, kv, dv, gated):
    dt = TORCH[dtype]
    g = torch.Generator().manual_seed(6)
    n, rep, lam, eps, mult = 9, heads // kv, 0.37, 1e-5, 0.8
    maps = torch.randn(n, kv, 2, rep, dv, generator=g).to(dt)
    gate = torch.randn(n, heads * dv, generator=g).to(dt) if gated else None
    a1 = maps[:, :, 0].double().reshape(n, heads, dv)
    a2 = maps[:, :, 1].double().reshape(n, heads, dv)
    want = (plain.rms(a1 - lam * a2, eps) * mult).reshape(n, heads * dv)
    if gated:
        want = want * torch.sigmoid(gate.double())
    out = torch.empty(n, heads * dv, dtype=dt, device=DEV)
    k().diff_combine(maps.reshape(n, -1).to(DEV), gate.to(DEV) if gated else None, out, heads, kv, dv, lam, eps, mult)
    assert close(out, want, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n, d, pad", [(11, 37, 3), (70, 64, 8)])       # odd sizes; rows that take the 16-byte forms
def test_gates_scale_and_activation_kernels(dtype, n, d, pad):
    dt = TORCH[dtype]
    g = torch.Generator().manual_seed(7)
    res = torch.randn(n, d, generator=g)
    y, gp = torch.randn(n, d + pad, generator=g).to(dt), (3 * torch.randn(n, d, generator=g)).to(dt)
    b = torch.randn(d, generator=g).to(dt)
    r = res.to(DEV)
    k().gated_residual_add(r, y.to(DEV)[:, :d], gp.to(DEV), b.to(DEV))
    want = res.double() + torch.sigmoid(gp.double() + b.double()) * y.double()[:, :d]
    assert torch.allclose(r.double().cpu(), want, atol=1e-5)
    r2 = res.to(DEV)
    k().gated_residual_add(r2, y.to(DEV)[:, :d], gp.to(DEV), None)
    assert torch.allclose(r2.double().cpu(), res.double() + torch.sigmoid(gp.double()) * y.double()[:, :d], atol=1e-5)
    x, keep = res.to(DEV), torch.zeros(n, d, device=DEV)
    k().scale_rows(x, 12.5, keep)
    assert torch.equal(x.cpu(), res * 12.5) and torch.equal(keep, x)
    gu = (2.5 * torch.randn(n, 2 * d, generator=g)).to(dt)
    for inter in (False, True):
        gg = gu.double()[:, 0::2] if inter else gu.double()[:, :d]
        uu = gu.double()[:, 1::2] if inter else gu.double()[:, d:]
        out = torch.empty(n, d, dtype=dt, device=DEV)
        k().glu_act(gu.to(DEV), out, "clamped_swish", interleaved=inter, alpha=1.702, limit=1.3, up_offset=1.0)
        gc = gg.clamp(max=1.3)
        assert close(out, gc * torch.sigmoid(1.702 * gc) * (uu.clamp(-1.3, 1.3) + 1.0), dtype)
        assert float((gg > 1.3).float().mean()) > 0.1 and float((uu < -1.3).float().mean()) > 0.1
        k().glu_act(gu.to(DEV), out, "silu", interleaved=inter)
        assert close(out, gg * torch.sigmoid(gg) * uu, dtype)


@pytest.mark.parametrize("M, N, K, bn", [(200, 320, 128, 128), (384, 1024, 256, 256), (129, 96, 64, 256)])
def test_clamped_activation_in_the_epilogue_of_the_tensor_core_product(M, N, K, bn):
    """Gate and up as alternating weight rows; both branches reach their limits; full tiles and edge tiles."""
    g = torch.Generator().manual_seed(M + N)
    bf = torch.bfloat16
    a = torch.randn(M, K, generator=g).to(bf)
    w = (torch.randn(N, K, generator=g) * 0.25).to(bf)
    ref = a.double() @ w.double().T
    gg, uu = ref[:, 0::2], ref[:, 1::2]
    limit, alpha, off = 1.7, 1.702, 1.0
    assert float((gg > limit).float().mean()) > 0.1 and float((uu < -limit).float().mean()) > 0.1
    gc = gg.clamp(max=limit)
    want = gc * torch.sigmoid(alpha * gc) * (uu.clamp(-limit, limit) + off)
    h = torch.full((M, N // 2), float("nan"), device=DEV, dtype=bf)
    k().gemm_tcgen05(a.to(DEV), w.to(DEV), h, "silu_mul", bn, act=(alpha, limit, off))
    assert float((h.double().cpu() - want).abs().max()) <= 1e-2 * max(1.0, float(want.abs().max()))
    # no clamp at all: a limit of infinity, the plain activation with an offset
    want = gg * torch.sigmoid(gg) * (uu + 0.5)
    k().gemm_tcgen05(a.to(DEV), w.to(DEV), h, "silu_mul", bn, act=(1.0, float("inf"), 0.5))
    assert float((h.double().cpu() - want).abs().max()) <= 1e-2 * max(1.0, float(want.abs().max()))
    torch.cuda.synchronize()
    assert k().gemm_tcgen05_error() == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("lens, in_runs", [([13, 1, 6], False), ([13, 1, 6], True), ([213, 1, 40], True)])
def test_mingru_scan_kernel_carries_its_state_over_any_cut(dtype, lens, in_runs):
    """Three requests of unequal length in slots out of order, a padding row, gates from almost shut to almost open,
    a state that is not zero at the start, a run that may not write; token by token, and with every request's tokens
    cut into runs that are scanned side by side (more runs than tokens, and runs of unequal length)."""
    dt = TORCH[dtype]
    g = torch.Generator().manual_seed(8)
    width = 70
    hint = 1000 if in_runs else 0
    slots = [2, -1, 0, 3]
    zb, ub = torch.linspace(-6, 6, width).to(dt), torch.randn(width, generator=g).to(dt)
    state0 = torch.randn(5, width, generator=g)
    seqs = [(2 * torch.randn(L, 3 * width, generator=g)).to(dt) for L in lens]

    def plain_scan(x, s):
        z = torch.sigmoid(x[:, :width].double() + zb.double())
        u = x[:, width:2 * width].double() + ub.double()
        c = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
        gt = x[:, 2 * width:].double()
        out = []
        s = s.double().clone()
        for t in range(x.shape[0]):
            s = (1 - z[t]) * s + z[t] * c[t]
            out.append(s * gt[t] * torch.sigmoid(gt[t]))
        return torch.stack(out), s

    for cuts in ([100], [1], [2, 5, 1, 3]):
        state = state0.to(DEV)
        done = [0, 0, 0]
        got = [[], [], []]
        i = 0
        while any(d < L for d, L in zip(done, lens)):
            take = [min(cuts[i % len(cuts)], L - d) for d, L in zip(done, lens)]
            i += 1
            rows, q_start, sl = [], [0], []
            order = [0, None, 1, 2]             # the padding row sits second
            for r in order:
                if r is None:
                    rows.append(torch.zeros(1, 3 * width, dtype=dt)); q_start.append(q_start[-1] + 1); sl.append(-1)
                elif take[r]:
                    rows.append(seqs[r][done[r]:done[r] + take[r]]); q_start.append(q_start[-1] + take[r]); sl.append([2, 0, 3][r])
            x = torch.cat(rows).to(DEV)
            out = torch.empty(x.shape[0], width, dtype=dt, device=DEV)
            before = state.clone()
            k().mingru_scan(x[:, :width], x[:, width:2 * width], x[:, 2 * width:], zb.to(DEV), ub.to(DEV), state, out,
                            dev_i32(q_start), dev_i32(sl), len(sl), write_state=False, max_q_len=hint)
            assert torch.equal(state, before)
            k().mingru_scan(x[:, :width], x[:, width:2 * width], x[:, 2 * width:], zb.to(DEV), ub.to(DEV), state, out,
                            dev_i32(q_start), dev_i32(sl), len(sl), max_q_len=hint)
            at = 0
            for j, s_ in enumerate(sl):
                nrow = q_start[j + 1] - q_start[j]
                if s_ >= 0:
                    r = {2: 0, 0: 1, 3: 2}[s_]
                    got[r].append(out[at:at + nrow].cpu())
                    done[r] += nrow
                at += nrow
        for r, slot in enumerate([2, 0, 3]):
            want, s_end = plain_scan(seqs[r], state0[slot])
            assert close(torch.cat(got[r]), want, dtype), (cuts, r)
            assert torch.allclose(state[slot].double().cpu(), s_end, atol=2e-5 if dtype == "float32" else 3e-2)
        assert torch.equal(state[1].cpu(), state0[1]) and torch.equal(state[4].cpu(), state0[4])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows_kernel", [False, True])
@pytest.mark.parametrize("shape", ["shared_values", "values_in_keys"])
def test_a_key_stands_out_only_inside_the_chunk(dtype, rows_kernel, shape):
    """One key among hundreds is made to dominate (its dot product with every query is large); the output must be that
    key's value for queries of its chunk after it and must not see it from the next chunk on, at chunk edges that are
    no page or tile borders, with released pages poisoned; with two key heads a value head, and with values that are
    the first dimensions of the key rows."""
    dt = TORCH[dtype]
    g = torch.Generator().manual_seed(11)
    ps, chunk, T = 8, 37, 150
    if shape == "shared_values":
        n_heads, n_k, n_v, hd, hdv, v_row = 4, 2, 1, 12, 20, None
    else:
        n_heads, n_k, n_v, hd, hdv, v_row = 3, 1, 1, 24, 18, 24
    hot = 40                                     # in the chunk 37..73
    kk = torch.randn(T, n_k, hd, generator=g) * 0.3
    v = torch.randn(T, n_v, hdv, generator=g)
    q = torch.randn(T, n_heads, hd, generator=g) * 0.3
    direction = torch.randn(hd, generator=g)
    direction /= direction.norm()
    if shape == "values_in_keys":
        direction[:hdv] = 0                      # the values are the keys' first dimensions: mark the key in the others
        direction /= direction.norm()
    kk[hot] += 30 * direction
    q += 2 * direction
    kk, v, q = kk.to(dt), v.to(dt), q.to(dt)
    if shape == "values_in_keys":
        v = kk[:, :, :hdv].clone()
    n_pages = -(-T // ps)
    perm = torch.randperm(n_pages + 3, generator=g)[:n_pages]
    kpool = torch.full((n_pages + 3, n_k, ps, hd), float("nan"), dtype=dt)
    vpool = torch.full((n_pages + 3, n_v, ps, hdv), float("nan"), dtype=dt)
    for t in range(T):
        kpool[perm[t // ps], :, t % ps] = kk[t]
        vpool[perm[t // ps], :, t % ps] = v[t]
    table = perm.to(torch.int32).clone()
    group = n_heads // n_k
    qd, kd, vd = q.double(), kk.double(), v.double()
    want = torch.zeros(T, n_heads, hdv, dtype=torch.float64)
    for t in range(T):
        lo = (t // chunk) * chunk
        for h in range(n_heads):
            c = h // group
            s = (kd[lo:t + 1, c] @ qd[t, h]) * 0.5
            want[t, h] = torch.softmax(s, 0) @ vd[lo:t + 1, c // (n_k // n_v)]
    # queries as a prompt portion (tile kernel) or as decode tokens of requests at different lengths (rows kernel)
    kp = kpool.to(DEV)
    vp = kp if shape == "values_in_keys" else vpool.to(DEV)
    if rows_kernel:
        qpos = [hot, hot + 1, 73, 74, 75, 110, 111, 149, 36, 37]
    else:
        qpos = list(range(30, T))
    out = torch.empty(len(qpos), n_heads * hdv, dtype=dt, device=DEV)
    qrows = q[qpos].reshape(len(qpos), -1).to(DEV)
    extra = dict(v_head_dim=hdv, chunk=chunk, n_v_heads=n_v, v_row=v_row)
    if rows_kernel:
        R = len(qpos)
        tables = []
        for p in qpos:                           # pages wholly before the query's chunk are released
            t_ = table.clone()
            t_[:((p // chunk) * chunk) // ps] = -1
            tables.append(t_)
        k().attention_rows(qrows, out, kp, vp, torch.stack(tables).to(DEV), dev_i32(range(R + 1)), dev_i32(qpos), R, group * 4,
                           n_heads, n_k, hd, ps, None, 0.5, **extra)
    else:
        t_ = table.clone()
        t_[:((30 // chunk) * chunk) // ps] = -1
        work = [(0, p0) for p0 in range(0, len(qpos) * group, 32)]
        k().attention_general(qrows, out, kp, vp, t_[None].to(DEV), dev_i32([0, len(qpos)]), dev_i32([30]),
                              dev_i32([w_[0] for w_ in work]), dev_i32([w_[1] for w_ in work]), len(work), n_heads, n_k, hd,
                              ps, None, 0.5, **extra)
    got = out.double().cpu().reshape(len(qpos), n_heads, hdv)
    assert torch.isfinite(got).all()
    for i, p in enumerate(qpos):
        assert close(got[i], want[p], dtype, rel=3e-2), p
        sees = hot <= p < 74
        near_hot = float((got[i, 0] - vd[hot, 0]).abs().max()) < 0.05 * float(vd[hot, 0].abs().max())
        assert near_hot == sees, (p, sees)


@pytest.mark.parametrize("dk, dv, n_heads, n_k, n_v, in_keys, chunk, window, ps", [
    (64, 128, 8, 4, 2, False, 37, None, 16),      # two key heads a value head, values twice the keys
    (16, 16, 3, 1, 1, False, None, None, 8),      # the smallest sizes, three heads over one
    (48, 80, 6, 2, 1, False, 50, None, 16),
    (256, 192, 5, 1, 1, True, None, None, 16),    # values inside the key rows; the short key tile
    (80, 48, 7, 1, 1, True, 21, None, 8),
    (32, 16, 4, 4, 4, False, None, 29, 8),        # a window
    (144, 112, 2, 2, 2, False, 64, None, 32),
    (256, 256, 2, 1, 1, False, None, None, 16),
])
def test_tensor_core_attention_with_float32_scores(dk, dv, n_heads, n_k, n_v, in_keys, chunk, window, ps):
    """The tensor-core kernel for prompt portions against attention written out in float64: two requests of unequal
    length in one step (one continues after 45 cached tokens, a count that is no multiple of a page or a tile), pages
    in random order, unwritten slots poisoned, pages before the visible keys released, a key that dominates every
    score of its request so that a mask that is one key off shows, rows of q and out with columns beside the heads."""
    dt = torch.bfloat16
    g = torch.Generator().manual_seed(dk * 7 + dv)
    lens, before = [131, 70], [45, 0]
    group = n_heads // n_k
    scale = 0.4 / math.sqrt(dk)
    qs, outs, tables, wants = [], [], [], []
    n_pages_each = [-(-(b + L) // ps) for L, b in zip(lens, before)]
    total_pages = sum(n_pages_each) + 3
    perm = torch.randperm(total_pages, generator=g)
    kpool = torch.full((total_pages, n_k, ps, dk), float("nan"), dtype=dt)
    vpool = kpool if in_keys else torch.full((total_pages, n_v, ps, dv), float("nan"), dtype=dt)
    at = 0
    for r, (L, b) in enumerate(zip(lens, before)):
        T = b + L
        kk = torch.randn(T, n_k, dk, generator=g)
        hot = b + 9
        direction = torch.randn(dk, generator=g)
        if in_keys:
            direction[:dv] = 0
        direction /= direction.norm()
        kk[hot] += 12 * math.sqrt(dk) * direction
        q = torch.randn(L, n_heads, dk, generator=g) + 2 * direction
        kk, q = kk.to(dt), q.to(dt)
        v = kk[:, :, :dv].clone() if in_keys else torch.randn(T, n_v, dv, generator=g).to(dt)
        pages = perm[at:at + n_pages_each[r]]
        at += n_pages_each[r]
        for t in range(T):
            kpool[pages[t // ps], :, t % ps] = kk[t]
            if not in_keys:
                vpool[pages[t // ps], :, t % ps] = v[t]
        table = torch.full((max(n_pages_each),), -1, dtype=torch.int32)
        table[:len(pages)] = pages.to(torch.int32)
        first_seen = 0
        if chunk:
            first_seen = (b // chunk) * chunk
        if window:
            first_seen = max(first_seen, b - window + 1)
        table[:first_seen // ps] = -1              # nothing before the first query's first visible key is held
        tables.append(table)
        want = torch.zeros(L, n_heads, dv, dtype=torch.float64)
        for t in range(L):
            p_ = b + t
            lo = max((p_ // chunk) * chunk if chunk else 0, p_ - window + 1 if window else 0)
            for h in range(n_heads):
                c = h // group
                sc = (kk.double()[lo:p_ + 1, c] @ q.double()[t, h]) * scale
                want[t, h] = torch.softmax(sc, 0) @ v.double()[lo:p_ + 1, c // (n_k // n_v)]
        wants.append(want)
        qs.append(q.reshape(L, n_heads * dk))
    n = sum(lens)
    qrows = torch.zeros(n, n_heads * dk + 8, dtype=dt)
    qrows[:, :n_heads * dk] = torch.cat(qs)
    out = torch.full((n, n_heads * dv + 2), 5.0, dtype=dt, device=DEV)
    rows = k().ATTENTION_WIDE_ROWS
    work = [(r, p0) for r, L in enumerate(lens) for p0 in range(0, L * group, rows)]
    kp = kpool.to(DEV)
    vp = kp if in_keys else vpool.to(DEV)
    qd = qrows.to(DEV)
    assert k().attention_wide_supports(qd[:, :n_heads * dk], out[:, :n_heads * dv], dk, dv, dk if in_keys else None)
    k().attention_wide(qd[:, :n_heads * dk], out[:, :n_heads * dv], kp, vp, torch.stack(tables).to(DEV), dev_i32([0, lens[0], n]),
                       dev_i32(before), dev_i32([w_[0] for w_ in work]), dev_i32([w_[1] for w_ in work]), len(work), n_heads, n_k,
                       dk, ps, window, scale, v_head_dim=dv, chunk=chunk or 0, n_v_heads=n_v, v_row=dk if in_keys else None)
    got = out[:, :n_heads * dv].double().cpu().reshape(n, n_heads, dv)
    assert torch.isfinite(got).all() and bool((out[:, n_heads * dv:] == 5.0).all())
    want = torch.cat(wants)
    err = (got - want).abs().amax(dim=(1, 2))
    bound = 1.2e-2 * want.abs().amax(dim=(1, 2)).clamp(min=0.05)        # the output's own bfloat16 rounding and a little
    bad = torch.nonzero(err > bound).flatten().tolist()
    assert not bad, (bad[:8], float(err.max()))
    # and the general kernel agrees to the output's rounding
    out2 = torch.empty(n, n_heads * dv, dtype=dt, device=DEV)
    work32 = [(r, p0) for r, L in enumerate(lens) for p0 in range(0, L * group, 32)]
    k().attention_general(qd[:, :n_heads * dk], out2, kp, vp, torch.stack(tables).to(DEV), dev_i32([0, lens[0], n]), dev_i32(before),
                          dev_i32([w_[0] for w_ in work32]), dev_i32([w_[1] for w_ in work32]), len(work32), n_heads, n_k, dk, ps,
                          window, scale, v_head_dim=dv, chunk=chunk or 0, n_v_heads=n_v, v_row=dk if in_keys else None)
    diff = (out2.double().cpu().reshape(n, n_heads, dv) - got).abs().amax(dim=(1, 2))
    assert bool((diff <= bound).all()), float(diff.max())


@pytest.mark.parametrize("dk, dv, n_heads, n_k, n_v, in_keys, chunk, ps", [
    (48, 32, 6, 1, 1, True, None, 8),            # six heads over one compressed row
    (64, 128, 16, 4, 2, False, 37, 16),          # two maps a head over shared values, chunks
    (256, 192, 40, 1, 1, True, None, 16),        # more rows than one tile holds: two tiles a request
    (16, 16, 4, 4, 4, False, 50, 8),             # one head a key head
])
@pytest.mark.parametrize("n_splits", [1, 3, 0])
def test_tensor_core_attention_of_decode_tokens_with_split_keys(dk, dv, n_heads, n_k, n_v, in_keys, chunk, ps, n_splits):
    """Requests that bring one to three tokens at unequal lengths (one at the very start of its sequence, one right
    after a chunk's edge), a request that brings too many rows and must be left alone, and a padding request without
    tokens; one run of keys, three, or as many as the host would choose; against float64 and against the rows kernel."""
    dt = torch.bfloat16
    g = torch.Generator().manual_seed(dk + dv + n_heads)
    group = n_heads // n_k
    scale = 0.5 / math.sqrt(dk)
    lens, before = [1, 3, 2, 1, 9, 0, 1], [0, 200, 73, 74, 30, 0, 333]
    max_rows = 4 * group
    per = [-(-(b + L) // ps) for L, b in zip(lens, before)]
    total_pages = sum(per) + 2
    perm = torch.randperm(total_pages, generator=g)
    kpool = torch.full((total_pages, n_k, ps, dk), float("nan"), dtype=dt)
    vpool = kpool if in_keys else torch.full((total_pages, n_v, ps, dv), float("nan"), dtype=dt)
    tables, qs, wants, at = [], [], [], 0
    for L, b, npg in zip(lens, before, per):
        T = b + L
        kk = torch.randn(T, n_k, dk, generator=g).to(dt)
        v = kk[:, :, :dv].clone() if in_keys else torch.randn(T, n_v, dv, generator=g).to(dt)
        q = torch.randn(L, n_heads, dk, generator=g).to(dt)
        pages = perm[at:at + npg]
        at += npg
        for t in range(T):
            kpool[pages[t // ps], :, t % ps] = kk[t]
            if not in_keys:
                vpool[pages[t // ps], :, t % ps] = v[t]
        table = torch.full((max(per),), -1, dtype=torch.int32)
        table[:npg] = pages.to(torch.int32)
        if chunk:
            table[:((b // chunk) * chunk) // ps] = -1
        tables.append(table)
        want = torch.zeros(L, n_heads, dv, dtype=torch.float64)
        for t in range(L):
            p_ = b + t
            lo = (p_ // chunk) * chunk if chunk else 0
            for h in range(n_heads):
                c = h // group
                sc = (kk.double()[lo:p_ + 1, c] @ q.double()[t, h]) * scale
                want[t, h] = torch.softmax(sc, 0) @ v.double()[lo:p_ + 1, c // (n_k // n_v)]
        wants.append(want)
        qs.append(q.reshape(L, n_heads * dk))
    n = sum(lens)
    starts = [0]
    for L in lens:
        starts.append(starts[-1] + L)
    qd = torch.cat(qs).to(DEV)
    kp = kpool.to(DEV)
    vp = kp if in_keys else vpool.to(DEV)
    extra = dict(v_head_dim=dv, chunk=chunk or 0, n_v_heads=n_v, v_row=dk if in_keys else None)
    R = len(lens)
    if n_splits == 0:
        keys = min(max(b + L for L, b in zip(lens, before)), chunk + 4 if chunk else 1 << 30) + 64
        n_splits, split_keys = k().attention_wide_splits(dk, dv, keys, R * -(-max_rows // 64) * n_k)
        assert n_splits * split_keys >= keys
    else:
        tile = 64 if dk + dv <= 256 else 32
        split_keys = -(-(max(b + L for L, b in zip(lens, before)) + 64) // (n_splits * tile)) * tile
    words = k().attention_wide_small_scratch(dk, dv, R, max_rows, n_k, n_splits)
    scratch = torch.full((max(words, 1),), float("nan"), device=DEV)
    out = torch.full((n, n_heads * dv), 5.0, dtype=dt, device=DEV)
    k().attention_wide_small(qd, out, kp, vp, torch.stack(tables).to(DEV), dev_i32(starts), dev_i32(before), R, max_rows, n_heads, n_k,
                             dk, ps, None, scale, n_splits, split_keys, scratch if words else None, **extra)
    out2 = torch.full((n, n_heads * dv), 5.0, dtype=dt, device=DEV)
    k().attention_rows(qd, out2, kp, vp, torch.stack(tables).to(DEV), dev_i32(starts), dev_i32(before), R, max_rows, n_heads, n_k, dk,
                       ps, None, scale, **extra)
    got, got2 = out.double().cpu().reshape(n, n_heads, dv), out2.double().cpu().reshape(n, n_heads, dv)
    big = slice(starts[4], starts[5])                        # nine tokens: more rows than max_rows, left alone by both
    assert bool((got[big] == 5.0).all()) and bool((got2[big] == 5.0).all())
    want = torch.cat(wants)
    keep = torch.ones(n, dtype=torch.bool)
    keep[big] = False
    assert torch.isfinite(got[keep]).all()
    bound = 1.2e-2 * want.abs().amax(dim=(1, 2)).clamp(min=0.05)
    assert bool(((got - want).abs().amax(dim=(1, 2)) <= bound)[keep].all())
    assert bool(((got - got2).abs().amax(dim=(1, 2)) <= bound)[keep].all())


# =============================================================== whole models
def load(folder, dtype, page_size=16, n_pages=64, max_requests=4, **kw):
    from inf_engine_b200 import ModelRunner
    return ModelRunner.from_dir(folder, dtype=dtype, page_size=page_size, n_pages=n_pages, max_requests=max_requests, **kw)


def stepped(r, rid, tokens, sizes, end=True):
    """Logits of every position of ``tokens``, fed in portions of ``sizes`` (repeated as needed)."""
    from inf_engine_b200 import StepEntry
    r.open(rid)
    out, p, i = [], 0, 0
    while p < len(tokens):
        n = min(sizes[i % len(sizes)], len(tokens) - p)
        out.append(r.step([StepEntry(rid, tokens[p:p + n], list(range(n)))]).cpu().clone())
        p += n
        i += 1
    if end:
        r.close(rid)
    return torch.cat(out)


def steady_tokens(cfg, w, n: int, seed: int) -> list[int]:
    """``n`` random tokens on which the model is well conditioned.  A differential head divides a1 - lambda a2 by its
    root mean square, and sharpened attention turns the last bits of a score into a share of a weight: on some rows of
    some sequences the plain model in 32-bit disagrees with itself in 64-bit by as much as the bound allows any
    implementation.  Such a sequence says nothing about the product, so the next seed is taken."""
    for s in range(seed, seed + 50):
        toks = random_tokens(cfg["vocab"], n, s)
        a, b = plain.forward(cfg, w, toks), plain.forward_float32(cfg, w, toks)
        if float((a - b).abs().max()) <= 0.25 * helpers.tolerance("float32", a):
            return toks
    raise AssertionError("no well-conditioned sequence in 50 seeds")


LENGTH = {"fvx_a": 97, "fvx_b": 70, "fvx_c": 131, "fvx_w": 150, "fvx_lat": 60, "fvx_diff": 75, "fvx_gru": 50, "fvx_ff": 41}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(MODELS))
def test_whole_prompt_decoding_and_portions_agree_with_the_plain_model(tmp_path, name, dtype):
    folder = make_fovunex_dir(tmp_path, name)
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
@pytest.mark.parametrize("name", ["fvx_a", "fvx_b", "fvx_c", "fvx_w"])
def test_unequal_requests_in_one_batch_with_pages_and_slots_used_again(tmp_path, name, dtype):
    """Seven requests, at most three live, portions of some beside decoded tokens of others, some left out of a step;
    the pool holds exactly what the fullest moment needs and free pages are filled with NaN."""
    import random
    from inf_engine_b200 import StepEntry

    folder = make_fovunex_dir(tmp_path, name)
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
    requests left there (their recurrent states, of every pass) must not reach the new ones."""
    from inf_engine_b200 import StepEntry

    folder = make_fovunex_dir(tmp_path, "fvx_a")
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
@pytest.mark.parametrize("name", ["fvx_diff", "fvx_b", "fvx_c"])
def test_edges_of_the_chunks_in_prompts_and_in_decoding(tmp_path, name, dtype):
    """The attention is made sharp (head-norm gains and the compressed vector's gain times 2.5) so that one key more
    or less changes the logits far beyond rounding; the sequence runs over several chunks, in pages of 8, so that
    pages behind a chunk are given back."""
    def fix(t):
        for n in list(t):
            if n.endswith((".q.norm", ".k.norm", ".dkv.norm")):
                t[n] = (t[n].float() * 2.5).to(t[n].dtype)
    folder = make_fovunex_dir(tmp_path, name, fix=fix)
    cfg, w = plain_inputs(folder)
    size = [L["mixer"]["mask"]["size"] for L in cfg["layers"] if "mask" in L["mixer"]][0]
    toks = steady_tokens(cfg, w, 4 * size + 5, 8)
    ref = reference(w, cfg, toks, dtype)
    # the faults this must catch: a chunk one position longer or shorter
    for delta in (1, -1):
        other = copy.deepcopy(cfg)
        for L in other["layers"]:
            if "mask" in L["mixer"]:
                L["mixer"]["mask"]["size"] += delta
        wrong = plain.forward(other, w, toks)
        moved = (wrong - ref.logits).norm(dim=-1).div(ref.logits.norm(dim=-1))[size - 1:]
        assert float(moved.max()) > 0.02, (delta, float(moved.max()))
    r = load(folder, dtype, page_size=8)
    noise = 1.5
    assert_close(stepped(r, "whole", toks, [len(toks)]), ref, dtype, f"{name}: chunk edges in a prompt", noise=noise)
    assert_close(stepped(r, "decode", toks, [3] + [1] * (len(toks) - 3)), ref, dtype, f"{name}: chunk edges in decoding", noise=noise)
    assert_close(stepped(r, "cut", toks, [size - 1, 2, 1, 1, 5, 11]), ref, dtype, f"{name}: portions around a chunk's edge", noise=noise)
    assert_close(stepped(r, "cut2", toks, [size, size + 1, 2]), ref, dtype, f"{name}: portions that end on an edge", noise=noise)
    r.cache.check()
    g = [g_ for g_ in r.cache.kv_groups if g_.chunk][0]
    assert g.pool.n_free == g.pool.n_pages


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_far_key_is_found_by_the_latent_attention(tmp_path, dtype):
    """The compressed vector's gain is tripled, which makes the latent attention sharp; the test first shows that
    swapping one token 250 and more positions back moves the last positions' plain logits, then the engine must agree
    with the plain model there, in a prompt and decoded (the kernels alone are tested with a key that dominates)."""
    folder = make_fovunex_dir(tmp_path, "fvx_lat", fix=lambda t: t.__setitem__("l0.mix.dkv.norm", (t["l0.mix.dkv.norm"].float() * 3).to(t["l0.mix.dkv.norm"].dtype)))
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
    """Four tokens of prompt and 200 decoded one by one through the decode graphs: the recurrent states of every pass
    and both caches are carried over 200 steps."""
    folder = make_fovunex_dir(tmp_path, "fvx_a")
    cfg, w = plain_inputs(folder)
    toks = steady_tokens(cfg, w, 204, 77)
    ref = reference(w, cfg, toks, dtype)
    r = load(folder, dtype, page_size=8)
    got = stepped(r, "long", toks, [4] + [1] * 200)
    assert r.graphs.replays >= 150
    assert_close(got, ref, dtype, "long decoding")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["fvx_a", "fvx_c"])
def test_greedy_generation_through_the_entry_point(tmp_path, name, dtype):
    """``Engine.run_offline``: scheduler, portions of prompts under a token budget, decode graphs, device sampling.
    Every generated token must be the plain model's choice (or tie with it within bfloat16's noise)."""
    from inf_engine_b200 import Engine, Request

    folder = make_fovunex_dir(tmp_path, name)
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
    folder = make_fovunex_dir(tmp_path, "fvx_b")
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
        requests = {str(i): steady_tokens(cfg, w, n, 300 + 50 * i) for i, n in enumerate([70, 45, 130, 20, 97, 33])}
        trace = schedules("fvx", requests, seed=3)
        got = run_trace(folder, dtype, trace, tmp_path / f"out_{dtype}", cfg["vocab"], page_size=8)
        refs = {rid: reference(w, cfg, t, dtype) for rid, t in requests.items()}
        for prefix in "wdpm":
            for rid, t in requests.items():
                rows = [got.get((prefix + rid, p)) for p in range(len(t))]
                if rows[0] is None:
                    continue
                assert_close(torch.stack(rows), refs[rid], dtype, f"replay {prefix}{rid}")
