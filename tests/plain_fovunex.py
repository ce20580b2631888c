"""A plain, slow Fovunex decoder in float64 on the CPU: whole sequences, no cache, one function per mechanism.

It shares no code with the package and is the oracle of the tests.  ``cfg`` is the ``config.json`` dictionary and
``w`` maps tensor names to torch tensors.  ``round_to`` (a torch dtype or None) rounds where an engine that keeps its
activations in that type rounds: the results of matrix products and what is kept in the cache; norms, scores, softmax
weights, the recurrence and the residual stream stay float64 whatever it is.
"""

from __future__ import annotations

import math

import torch

F = torch.float64


def rnd(x: torch.Tensor, round_to) -> torch.Tensor:
    return x if round_to is None else x.to(round_to).to(F)


def lin(w: torch.Tensor, x: torch.Tensor, round_to=None) -> torch.Tensor:
    """W x for every row of x; W is stored [out, in]."""
    return rnd(x @ w.to(F).t(), round_to)


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def scalar_norm(x, g, eps, round_to=None):
    return rnd(rms(x, eps) * g.to(F).reshape(()), round_to)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotation_angles(rot: dict, positions: torch.Tensor):
    """cos and sin [T, dims / 2] of position * frequency, with the YaRN blend of frequencies and the common
    multiplier of both when ``rot`` carries a ``scaling`` entry."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=F)
    f = base ** (-2.0 * i / dims)
    mult = 1.0
    sc = rot.get("scaling")
    if sc:
        factor, orig = float(sc["factor"]), float(sc["original"])

        def dim_of(t):
            return dims * math.log(orig / (2.0 * math.pi * t)) / (2.0 * math.log(base))

        lo = max(math.floor(dim_of(float(sc["fast"]))), 0)
        hi = min(math.ceil(dim_of(float(sc["slow"]))), dims - 1)
        ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
        f = f / factor * ramp + f * (1.0 - ramp)
        mult = 0.1 * math.log(factor) + 1.0
    a = positions.to(F)[:, None] * f[None, :]
    return torch.cos(a) * mult, torch.sin(a) * mult


def rotate_interleaved(x, cos, sin):
    """x [T, heads, dims]: dimension 2i is paired with 2i + 1."""
    u, v = x[..., 0::2], x[..., 1::2]
    c, s = cos[:, None, :], sin[:, None, :]
    out = torch.empty_like(x)
    out[..., 0::2] = u * c - v * s
    out[..., 1::2] = v * c + u * s
    return out


def rotate_halves(x, cos, sin):
    """x [T, heads, dims]: dimension i is paired with i + dims / 2."""
    h = x.shape[-1] // 2
    u, v = x[..., :h], x[..., h:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([u * c - v * s, v * c + u * s], dim=-1)


def softmax_attention(q, k, v, scale: float, visible: torch.Tensor):
    """q [T, H, d], k [T, H, d], v [T, H, dv], visible [T, T] bool (row: query, column: key)."""
    s = torch.einsum("ihd,jhd->hij", q, k) * scale
    s = s.masked_fill(~visible[None], float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("hij,jhd->ihd", p, v)


def causal_mask(T: int, chunk: int | None = None) -> torch.Tensor:
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    m = j <= i
    if chunk:
        m = m & (i // chunk == j // chunk)
    return m


def latent_attention(h, m: dict, w: dict, p: str, eps: float, round_to=None):
    T = h.shape[0]
    H, d, r, dv, kr = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    q = lin(w[p + "q"], h, round_to).reshape(T, H, d + r)
    dkv = lin(w[p + "dkv"], h, round_to)
    c = rnd(rms(dkv[:, :kr], eps) * w[p + "dkv.norm"].to(F), round_to)
    k_rot = dkv[:, kr:].reshape(T, 1, r)
    q_un, q_rot = q[..., :d], q[..., d:]
    rot = m.get("rot")
    if rot:
        cos, sin = rotation_angles(dict(rot, dims=r), torch.arange(T))
        q_rot = rnd(rotate_interleaved(q_rot, cos, sin), round_to)
        k_rot = rnd(rotate_interleaved(k_rot, cos, sin), round_to)
    k_un = lin(w[p + "uk"], c, round_to).reshape(T, H, d)
    v = lin(w[p + "uv"], c, round_to).reshape(T, H, dv)
    qq = torch.cat([q_un, q_rot], dim=-1)
    kk = torch.cat([k_un, k_rot.expand(T, H, r)], dim=-1)
    mask = m.get("mask")
    o = softmax_attention(qq, kk, v, float(m["scale"]), causal_mask(T, int(mask["size"]) if mask else None))
    return lin(w[p + "o"], rnd(o.reshape(T, H * dv), round_to), round_to)


def differential_attention(h, m: dict, w: dict, p: str, eps: float, round_to=None):
    T = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m.get("kv_heads", m["heads"])), int(m["dim"]), int(m.get("vdim", m["dim"]))
    diff = float(m["diff"])
    q = lin(w[p + "q"], h, round_to).reshape(T, H * 2, d)
    k = lin(w[p + "k"], h, round_to).reshape(T, G * 2, d)
    v = lin(w[p + "v"], h, round_to).reshape(T, G, dv)
    q = rms(q, eps) * w[p + "q.norm"].to(F)
    k = rms(k, eps) * w[p + "k.norm"].to(F)
    rot = m.get("rot")
    if rot:
        n = int(rot["dims"])
        cos, sin = rotation_angles(rot, torch.arange(T))
        q = torch.cat([rotate_halves(q[..., :n], cos, sin), q[..., n:]], dim=-1)
        k = torch.cat([rotate_halves(k[..., :n], cos, sin), k[..., n:]], dim=-1)
    q, k = rnd(q, round_to), rnd(k, round_to)
    q = q.reshape(T, H, 2, d)
    k = k.reshape(T, G, 2, d)
    rep = H // G
    mask = m.get("mask")
    visible = causal_mask(T, int(mask["size"]) if mask else None)
    ke = k.repeat_interleave(rep, dim=1)          # [T, H, 2, d]: query head h reads key/value head h // rep
    ve = v.repeat_interleave(rep, dim=1)
    a1 = softmax_attention(q[:, :, 0], ke[:, :, 0], ve, float(m["scale"]), visible)
    a2 = softmax_attention(q[:, :, 1], ke[:, :, 1], ve, float(m["scale"]), visible)
    lam = (torch.exp((w[p + "lq1"].to(F) * w[p + "lk1"].to(F)).sum())
           - torch.exp((w[p + "lq2"].to(F) * w[p + "lk2"].to(F)).sum()) + diff)
    o = rms(a1 - lam * a2, eps) * (1.0 - diff)
    o = o.reshape(T, H * dv) * torch.sigmoid(lin(w[p + "g"], h, round_to))
    return lin(w[p + "o"], rnd(o, round_to), round_to)


def mingru(h, m: dict, w: dict, p: str, round_to=None, state=None):
    """Returns (output, final state); ``state`` [width] is where the sequence starts (zeros when None)."""
    T = h.shape[0]
    z = torch.sigmoid(lin(w[p + "z"], h, round_to) + w[p + "z.b"].to(F))      # the bias joins in full precision
    u = lin(w[p + "x"], h, round_to) + w[p + "x.b"].to(F)
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    s = torch.zeros(z.shape[1], dtype=F) if state is None else state.to(F).clone()
    out = torch.empty_like(z)
    for t in range(T):
        s = (1.0 - z[t]) * s + z[t] * cand[t]
        out[t] = s
    g = lin(w[p + "g"], h, round_to)
    y = out * (g * torch.sigmoid(g))
    return lin(w[p + "o"], rnd(y, round_to), round_to), s


def dense_ff(h, f: dict, w: dict, p: str, round_to=None):
    limit = float(f["limit"])
    g = lin(w[p + "gate"], h, round_to).clamp(max=limit)
    u = lin(w[p + "up"], h, round_to).clamp(-limit, limit)
    y = g * torch.sigmoid(1.702 * g) * (u + 1.0)
    return lin(w[p + "down"], rnd(y, round_to), round_to)


def layer_order(cfg: dict) -> list[tuple[int, bool]]:
    """(layer, add the embedding output before it) for every run of a layer."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    order = [(i, False) for i in range(start)]
    for t in range(times):
        for i in range(start, stop):
            order.append((i, t > 0 and i == start))
    order += [(i, False) for i in range(stop, n)]
    return order


def gate_of(w, name, h, round_to=None):
    return torch.sigmoid(lin(w[name], h, round_to) + w[name + ".b"].to(F))


def forward(cfg: dict, w: dict, tokens, round_to=None, return_layers: bool = False):
    """Logits [T, vocab] of one whole sequence (and the residual stream after every layer run)."""
    eps = float(cfg["norm"]["eps"])
    ids = torch.as_tensor(tokens, dtype=torch.long)
    x0 = w["embed"].to(F)[ids] * float(cfg["embedding"]["scale"])
    x = x0.clone()
    seen = []
    for i, add in layer_order(cfg):
        L = cfg["layers"][i]
        p = f"l{i}."
        if add:
            x = x + x0
        h = scalar_norm(x, w[p + "norm1"], eps, round_to)
        kind = L["type"]
        if kind == "latent_attention":
            y = latent_attention(h, L["mixer"], w, p + "mix.", eps, round_to)
        elif kind == "attention":
            y = differential_attention(h, L["mixer"], w, p + "mix.", eps, round_to)
        elif kind == "mingru":
            y, _ = mingru(h, L["mixer"], w, p + "mix.", round_to)
        else:
            raise ValueError(kind)
        x = x + gate_of(w, p + "rg1", h, round_to) * y
        if L.get("mlp") is not None:
            h = scalar_norm(x, w[p + "norm2"], eps, round_to)
            x = x + gate_of(w, p + "rg2", h, round_to) * dense_ff(h, L["mlp"], w, p + "mlp.", round_to)
        seen.append(x.clone())
    h = scalar_norm(x, w["final.norm"], eps, round_to)
    logits = lin(w["head"], h)
    return (logits, torch.stack(seen)) if return_layers else logits


def forward_float32(cfg: dict, w: dict, tokens):
    """The same model with every operation in float32: how far it lies from the float64 result says how well
    conditioned a sequence is (a row on which the two disagree says little about any implementation)."""
    global F
    F = torch.float32
    try:
        return forward(cfg, w, tokens).double()
    finally:
        F = torch.float64
