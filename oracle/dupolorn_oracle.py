"""Float64 restatement of the Dupolorn design, one function per mechanism.  Slow and plain on purpose: the tests hold the
CUDA path against it, and it shares no code with the package.

Notation: W is the model width, t a time index inside one sequence, h the input of a sublayer.

  embedding        x_t = E[id_t] * s  +  B[(id_{t-1} * a + id_t * b) mod n]      (t = 0: row n of B)
  layer i          u  = avg_i                                   (avg_0 = x, see depth average)
                   h1 = u / rms(u) * g1 ;  h2 = u / rms(u) * g2                  (g1, g2 scalars)
                   hc = h1 + conv(h1),  conv(h1)_t = sum_j c[:, j] * h1_{t - taps + 1 + j}   (zeros before the sequence)
                   X_{i+1} = u + mixer(hc) + ff(h2)
  depth average    avg_{i+1} = sum_{j <= i+1} d_i[j] * X_j ,  X_0 = x
  output           softcap * tanh(head(avg_L / rms(avg_L) * g) / softcap)

Mixers: latent attention (keys and values expanded from one cached latent vector per token plus one rotated key part shared
by all heads; optionally a per-head sink in the softmax denominator and a sigmoid output gate) and the matrix-memory
recurrence of mLSTM in its stabilised form.  Feed-forwards: dense gated GELU, or routed experts with sigmoid scores whose
weight scales the expert's input, plus one shared expert.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def embed_tokens(ids: List[int], embed: torch.Tensor, scale: float, bigram: Optional[torch.Tensor], buckets: int, mul_prev: int,
                 mul_cur: int) -> torch.Tensor:
    rows = []
    for t, tok in enumerate(ids):
        x = embed[tok].to(F64) * scale
        if bigram is not None:
            r = buckets if t == 0 else (ids[t - 1] * mul_prev + tok * mul_cur) % buckets
            x = x + bigram[r].to(F64)
        rows.append(x)
    return torch.stack(rows)


def causal_conv(h: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """h [T, W], w [W, taps]: out_t = sum_j w[:, j] * h_{t - taps + 1 + j}."""
    T, taps = h.shape[0], w.shape[1]
    out = torch.zeros_like(h)
    for j in range(taps):
        back = taps - 1 - j                 # tap j reads the input `back` steps earlier
        if back < T:
            out[back:] += w[:, j].to(F64) * h[:T - back]
    return out


def rotate_pairs(v: torch.Tensor, pos, base: float, dims: int) -> torch.Tensor:
    """The leading `dims` entries of the last axis, pair (2i, 2i+1) turned by pos * base^(-2i/dims).  pos: a number, or a
    tensor that broadcasts against v without its last axis."""
    out = v.clone()
    pos = torch.as_tensor(pos, dtype=F64)
    for i in range(dims // 2):
        a = pos * base ** (-2.0 * i / dims)
        c, s = torch.cos(a), torch.sin(a)
        u, w = v[..., 2 * i].clone(), v[..., 2 * i + 1].clone()
        out[..., 2 * i] = u * c - w * s
        out[..., 2 * i + 1] = w * c + u * s
    return out


def latent_attention(h: torch.Tensor, m: dict, w: Dict[str, torch.Tensor], p: str, eps: float, sink: bool, gate: bool) -> torch.Tensor:
    """h [T, W] -> [T, W].  Keys and values are expanded from the latent for every token (no absorption): the plainest form."""
    T = h.shape[0]
    H, dim, rd, vd, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    base, rdims = float(m["rot"]["base"]), int(m["rot"]["dims"])
    f = lambda n: w[p + n].to(F64)
    q = (h @ f("q").T).reshape(T, H, dim + rd)
    dkv = h @ f("dkv").T
    c = rms_unit(dkv[:, :rank], eps) * f("dkv.norm")
    ku = (c @ f("uk").T).reshape(T, H, dim)
    v = (c @ f("uv").T).reshape(T, H, vd)
    t = torch.arange(T, dtype=F64)
    qr = rotate_pairs(q[:, :, dim:], t[:, None], base, rdims)
    kr = rotate_pairs(dkv[:, rank:], t, base, rdims)
    visible = torch.tril(torch.ones(T, T, dtype=torch.bool))
    out = torch.zeros(T, H, vd, dtype=F64)
    for hh in range(H):
        s = (q[:, hh, :dim] @ ku[:, hh].T + qr[:, hh] @ kr.T) * m["scale"]          # [query, key]
        s = s.masked_fill(~visible, -math.inf)
        mx = s.max(-1, keepdim=True).values
        if sink:
            mx = torch.maximum(mx, f("sink")[hh])
        e = torch.exp(s - mx)
        den = e.sum(-1, keepdim=True) + (torch.exp(f("sink")[hh] - mx) if sink else 0.0)
        out[:, hh] = (e / den) @ v[:, hh]
    a = out.reshape(T, H * vd)
    if gate:
        a = a * torch.sigmoid(h @ f("g").T)
    return a @ f("o").T


def mlstm(h: torch.Tensor, m: dict, w: Dict[str, torch.Tensor], p: str, eps: float, state: Optional[dict] = None) -> torch.Tensor:
    """Token-by-token recurrence.  state (optional, updated in place): S [H, dim, vdim], n [H, dim], m [H]."""
    T = h.shape[0]
    H, dim, vd, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    f = lambda n: w[p + n].to(F64)
    q = (h @ f("q").T).reshape(T, H, dim) * dim ** -0.5
    k = (h @ f("k").T).reshape(T, H, dim)
    v = (h @ f("v").T).reshape(T, H, vd)
    ig = cap * torch.tanh((h @ f("i").T + f("i.b")) / cap)
    fg = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ f("f").T + f("f.b")) / cap))
    if state is None:
        state = {}
    S = state.setdefault("S", torch.zeros(H, dim, vd, dtype=F64))
    n = state.setdefault("n", torch.zeros(H, dim, dtype=F64))
    mm = state.setdefault("m", torch.zeros(H, dtype=F64))
    out = torch.zeros(T, H, vd, dtype=F64)
    for t in range(T):                       # all heads at once
        m_new = torch.maximum(fg[t] + mm, ig[t])
        a, b = torch.exp(fg[t] + mm - m_new), torch.exp(ig[t] - m_new)
        S.mul_(a[:, None, None]).add_(b[:, None, None] * k[t][:, :, None] * v[t][:, None, :])
        n.mul_(a[:, None]).add_(b[:, None] * k[t])
        mm.copy_(m_new)
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-m_new)) + 1e-6
        out[t] = torch.einsum("hdv,hd->hv", S, q[t]) / den[:, None]
    o = rms_unit(out, eps).reshape(T, H * vd) * f("norm") * torch.sigmoid(h @ f("g").T)
    return o @ f("o").T


def dense_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    f = lambda n: w[p + n].to(F64)
    return (gelu_tanh(h @ f("gate").T) * (h @ f("up").T)) @ f("down").T


def relu2_expert(h: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    return torch.relu(h @ up.to(F64).T) ** 2 @ down.to(F64).T


def route_sigmoid(h: torch.Tensor, router: torch.Tensor, top: int):
    """(ids [T, top], weights [T, top]): the `top` largest sigmoid scores, ties to the lowest index, weights = the scores."""
    s = torch.sigmoid(h @ router.to(F64).T)
    ids, wts = [], []
    for t in range(h.shape[0]):
        order = sorted(range(s.shape[1]), key=lambda e: (-float(s[t, e]), e))[:top]
        ids.append(order)
        wts.append([float(s[t, e]) for e in order])
    return ids, wts


def moe_ff(h: torch.Tensor, f: dict, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    ids, wts = route_sigmoid(h, w[p + "router"], int(f["router"]["top"]))
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, wt in zip(ids[t], wts[t]):
            out[t] += relu2_expert(wt * h[t], w[f"{p}e{e}.up"], w[f"{p}e{e}.down"])
    if f.get("shared"):
        out = out + relu2_expert(h, w[p + "shared.up"], w[p + "shared.down"])
    return out


def forward(cfg: dict, w: Dict[str, torch.Tensor], ids: List[int], streams: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence; `streams` (optional list) receives avg_{i+1}, what layer i hands on."""
    eps = float(cfg["norm"]["eps"])
    bg = (cfg.get("embedding") or {}).get("bigram")
    x = embed_tokens(ids, w["embed"], float((cfg.get("embedding") or {}).get("scale", 1.0)), w.get("bigram") if bg else None,
                     int(bg["buckets"]) if bg else 0, int(bg["mul_prev"]) if bg else 0, int(bg["mul_cur"]) if bg else 0)
    X = [x]
    u = x
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        unit = rms_unit(u, eps)
        h1, h2 = unit * w[p + "norm1"].to(F64), unit * w[p + "norm2"].to(F64)
        hc = h1 + causal_conv(h1, w[p + "canon1"]) if p + "canon1" in w else h1
        kind = L["type"]
        if kind == "mlstm":
            y = mlstm(hc, L["mixer"], w, p + "mix.", eps)
        elif kind in ("latent_attention", "latent_attention_2"):
            second = kind == "latent_attention_2"
            y = latent_attention(hc, L["mixer"], w, p + "mix.", eps, sink=second, gate=second)
        else:
            raise ValueError(kind)
        f = L.get("mlp")
        if f:
            y = y + (dense_ff(h2, w, p + "mlp.") if f["kind"] == "dense" else moe_ff(h2, f, w, p + "mlp."))
        X.append(u + y)
        d = w[p + "dwa"].to(F64) if p + "dwa" in w else None
        u = sum(d[j] * X[j] for j in range(len(X))) if d is not None else X[-1]
        if streams is not None:
            streams.append(u)
    z = (rms_unit(u, eps) * w["final.norm"].to(F64)) @ w["head"].to(F64).T
    cap = cfg.get("logit_softcap")
    return cap * torch.tanh(z / cap) if cap else z


def greedy(cfg: dict, w: Dict[str, torch.Tensor], prompt: List[int], n: int) -> List[int]:
    ids, out = list(prompt), []
    for _ in range(n):
        tok = int(forward(cfg, w, ids)[-1].argmax())
        out.append(tok)
        ids.append(tok)
    return out
