"""A plain, slow Gavatar decoder in float64 on the CPU: whole sequences, no cache, one function per mechanism.

It shares no code with the package and is the oracle of the tests.  ``cfg`` is the ``config.json`` dictionary and
``w`` maps tensor names to torch tensors.  ``round_to`` (a torch dtype or None) rounds where an engine that keeps its
activations in that type rounds: the results of matrix products and what is kept in the cache; norms, scores, softmax
weights, the recurrence, the router and the residual stream stay float64 whatever it is.
"""

from __future__ import annotations

import math

import torch

F = torch.float64


def rnd(x: torch.Tensor, round_to) -> torch.Tensor:
    return x if round_to is None else x.to(round_to).to(F)


def lin(w: torch.Tensor, x: torch.Tensor, round_to=None, bias: torch.Tensor | None = None) -> torch.Tensor:
    """W x (+ b) for every row of x; W is stored [out, in]."""
    y = x @ w.to(F).t()
    if bias is not None:
        y = y + bias.to(F)
    return rnd(y, round_to)


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def offset_norm(x, g, eps):
    """RMS norm whose stored weight lies around zero."""
    return rms(x, eps) * (1.0 + g.to(F))


def sinusoid(positions: torch.Tensor, width: int, base: float = 10000.0) -> torch.Tensor:
    """[T, width]: entry 2i is sin(p base^(-2i / width)), entry 2i + 1 the cosine of the same angle."""
    i = torch.arange((width + 1) // 2, dtype=F)
    a = positions.to(F)[:, None] * base ** (-2.0 * i / width)[None, :]
    out = torch.zeros(positions.shape[0], 2 * i.shape[0], dtype=F)
    out[:, 0::2] = torch.sin(a)
    out[:, 1::2] = torch.cos(a)
    return out[:, :width]


def token_shift(h: torch.Tensor, mu: torch.Tensor) -> torch.Tensor:
    """h_t + (h_(t-1) - h_t) * mu, with zeros before the first token."""
    prev = torch.cat([torch.zeros_like(h[:1]), h[:-1]], dim=0)
    return h + (prev - h) * mu.to(F)


def window_mask(T: int, window: int | None) -> torch.Tensor:
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    m = j <= i
    if window:
        m = m & (i - j < window)
    return m


def attention_weights(q, k, scale: float, visible: torch.Tensor, sink: torch.Tensor | None = None):
    """Softmax weights [H, T, T] of q [T, H, d] over k [T, H, d]; with ``sink`` [H] the denominator also holds
    exp(sink), which has no key."""
    s = torch.einsum("ihd,jhd->hij", q, k) * scale
    s = s.masked_fill(~visible[None], float("-inf"))
    if sink is None:
        return torch.softmax(s, dim=-1)
    T = s.shape[-1]
    s = torch.cat([s, sink.to(F)[:, None, None].expand(-1, T, 1)], dim=-1)
    return torch.softmax(s, dim=-1)[..., :T]


def talking_attention(h, m: dict, w: dict, p: str, eps: float, round_to=None):
    """Grouped-query attention under a sliding window whose softmax weights are mixed across heads."""
    T = h.shape[0]
    H, d, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    G = int(m.get("kv_heads", H))
    rep = H // G
    q = lin(w[p + "q"], h, round_to, w[p + "q.b"]).reshape(T, H, d)
    k = lin(w[p + "k"], h, round_to, w[p + "k.b"]).reshape(T, G, d)
    v = lin(w[p + "v"], h, round_to, w[p + "v.b"]).reshape(T, G, dv)
    q, k, v = rnd(rms(q, eps), round_to), rnd(rms(k, eps), round_to), rnd(rms(v, eps), round_to)
    mask = m.get("mask")
    kk = k.repeat_interleave(rep, dim=1)
    vv = v.repeat_interleave(rep, dim=1)
    p_ = attention_weights(q, kk, float(m["scale"]), window_mask(T, int(mask["size"]) if mask else None))
    p_ = torch.einsum("hg,gij->hij", w[p + "talk"].to(F), p_)
    o = torch.einsum("hij,jhd->ihd", p_, vv).reshape(T, H * dv)
    o = o * torch.sigmoid(lin(w[p + "g"], h, round_to))
    return lin(w[p + "o"], rnd(o, round_to), round_to)


def latent_attention(h, m: dict, w: dict, p: str, eps: float, round_to=None):
    """Attention whose queries, keys and values are expanded from compressed vectors; a sink in the softmax."""
    T = h.shape[0]
    H, d, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    cq = rnd(rms(lin(w[p + "dq"], h, round_to), eps) * w[p + "dq.norm"].to(F), round_to)
    q = lin(w[p + "uq"], cq, round_to).reshape(T, H, d)
    c = rnd(rms(lin(w[p + "dkv"], h, round_to), eps) * w[p + "dkv.norm"].to(F), round_to)
    k = lin(w[p + "uk"], c, round_to).reshape(T, H, d)
    v = lin(w[p + "uv"], c, round_to).reshape(T, H, dv)
    mask = m.get("mask")
    p_ = attention_weights(q, k, float(m["scale"]), window_mask(T, int(mask["size"]) if mask else None), w[p + "sink"])
    o = torch.einsum("hij,jhd->ihd", p_, v)
    o = o * torch.sigmoid(lin(w[p + "g"], h, round_to))[:, :, None]
    return lin(w[p + "o"], rnd(o.reshape(T, H * dv), round_to), round_to)


def logsigmoid(x):
    return torch.minimum(x, torch.zeros_like(x)) - torch.log1p(torch.exp(-x.abs()))


def mlstm(h, m: dict, w: dict, p: str, eps: float, round_to=None, gates_round_to=None):
    """The matrix memory of xLSTM with a running maximum that starts at zero."""
    T = h.shape[0]
    H, d, dv, cap = int(m["heads"]), int(m["dim"]), int(m["vdim"]), float(m["gate_cap"])
    q = lin(w[p + "q"], h, round_to).reshape(T, H, d) * d ** -0.5
    k = lin(w[p + "k"], h, round_to).reshape(T, H, d)
    v = lin(w[p + "v"], h, round_to).reshape(T, H, dv)
    ig = cap * torch.tanh(lin(w[p + "i"], h, gates_round_to, w[p + "i.b"]) / cap)
    fg = logsigmoid(cap * torch.tanh(lin(w[p + "f"], h, gates_round_to, w[p + "f.b"]) / cap))
    S = torch.zeros(H, d, dv, dtype=F)
    n = torch.zeros(H, d, dtype=F)
    mx = torch.zeros(H, dtype=F)
    out = torch.zeros(T, H, dv, dtype=F)
    for t in range(T):
        m_new = torch.maximum(fg[t] + mx, ig[t])
        a = torch.exp(fg[t] + mx - m_new)
        b = torch.exp(ig[t] - m_new)
        S = a[:, None, None] * S + b[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = a[:, None] * n + b[:, None] * k[t]
        mx = m_new
        num = torch.einsum("hdv,hd->hv", S, q[t])
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-mx)) + 1e-6
        out[t] = num / den[:, None]
    o = rms(out, eps).reshape(T, H * dv) * w[p + "norm"].to(F) * torch.sigmoid(lin(w[p + "g"], h, round_to))
    return lin(w[p + "o"], rnd(o, round_to), round_to)


def route(h, r: dict, w: dict, p: str, gaps: list | None = None):
    """(chosen experts [T, top], their weights [T, top]): the largest logits, softmax over those alone.  ``gaps`` takes,
    per token, how far the last chosen logit lies above the best one left out, in units of the logits' spread (a small
    gap is a close call that rounding may decide either way)."""
    z = lin(w[p + "router"], h, None, w[p + "router.b"])
    k = int(r["top"])
    top = torch.topk(z, k, dim=-1)
    if gaps is not None and k < z.shape[-1]:
        both = torch.topk(z, k + 1, dim=-1).values
        gaps.append((both[:, k - 1] - both[:, k]) / z.std().clamp_min(1e-12))
    return top.indices, torch.softmax(top.values, dim=-1)


def expert(x, w: dict, p: str, round_to=None):
    g = lin(w[p + "gate"], x, None)
    u = lin(w[p + "up"], x, None)
    return lin(w[p + "down"], rnd(g * torch.sigmoid(g) * u, round_to), None)


def mixture(h, mlp: dict, w: dict, p: str, round_to=None, gaps: list | None = None):
    ids, wts = route(h, mlp["router"], w, p, gaps)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(ids[t].tolist(), wts[t]):
            out[t] += a * expert(h[t:t + 1], w, f"{p}e{e}.", round_to)[0]
    return out


MIXERS = {"attention": talking_attention, "latent_attention": latent_attention, "mlstm": mlstm}


def run_order(cfg: dict) -> list[tuple[int, int | None]]:
    """(layer, number of the pass that begins with this run or None) for every run of a layer."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop or int(loop["stop"]) <= int(loop["start"]):
        return [(i, None) for i in range(n)]
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    order = [(i, None) for i in range(a)]
    for t in range(times):
        order += [(i, t if i == a else None) for i in range(a, b)]
    return order + [(i, None) for i in range(b, n)]


def forward(cfg: dict, w: dict, tokens: list[int], round_to=None, collect: list | None = None,
            gaps: list | None = None) -> torch.Tensor:
    """Logits [T, vocab] of a whole sequence; ``collect`` takes the residual stream after every run of a layer, ``gaps``
    the routers' margins of every run of a mixture (see ``route``)."""
    eps = float(cfg["norm"]["eps"])
    width = int(cfg["width"])
    T = len(tokens)
    x = w["embed"].to(F)[torch.tensor(tokens)] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    x = x + sinusoid(torch.arange(T), width)
    for i, step in run_order(cfg):
        L = cfg["layers"][i]
        p = f"l{i}."
        if step is not None:
            x = x + w["loop.step"].to(F)[step]
        h = rnd(offset_norm(x, w[p + "norm1"], eps), round_to)
        if p + "shift" in w:
            h = rnd(token_shift(h, w[p + "shift"]), round_to)
        x = x + offset_norm(MIXERS[L["type"]](h, L["mixer"], w, p + "mix.", eps, round_to), w[p + "norm1b"], eps)
        if L.get("mlp") is not None:
            h = rnd(offset_norm(x, w[p + "norm2"], eps), round_to)
            x = x + offset_norm(mixture(h, L["mlp"], w, p + "mlp.", round_to, gaps), w[p + "norm2b"], eps)
        if collect is not None:
            collect.append(x.clone())
    return lin(w["head"], rnd(offset_norm(x, w["final.norm"], eps), round_to), None)


def forward_float32(cfg: dict, w: dict, tokens: list[int]) -> torch.Tensor:
    """The same model with every number a 32-bit float (how far 32-bit arithmetic alone moves the logits)."""
    global F
    F = torch.float32
    try:
        return forward(cfg, w, tokens).double()
    finally:
        F = torch.float64
