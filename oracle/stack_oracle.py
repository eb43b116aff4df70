"""Plain, slow restatement of the Bopilorn design in torch float64 on the CPU: one function per mechanism, written from
the equations below and sharing no code with the product path.  Used by tests only.

Notation: x residual stream [T, W]; p positions [T]; H query heads, G key/value heads, d query/key head size, e value head size.

  LN(v; w)          = (v - mean v) / sqrt(mean (v - mean v)^2 + eps) * w
  unit(v)           = v / sqrt(mean v^2 + eps)
  R(v, a)           = rotation of the pairs (v[2i], v[2i+1]) by the angles a[i]:  (u cos a - w sin a, w cos a + u sin a)
  f_i(base, n)      = base^(-2i/n), i < n/2
  YaRN              : c(t) = n ln(original / (2 pi t)) / (2 ln base); lo = max(floor c(fast), 0); hi = min(ceil c(slow), n-1);
                      r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1); f'_i = f_i / factor * r_i + f_i (1 - r_i);
                      cos and sin are multiplied by 0.1 ln(factor) + 1
  attention         : q = unit(W_q h) * w_qn, k = unit(W_k h) * w_kn  (unit over the WHOLE projection, all heads at once)
                      q_h, k_g: first `dims` entries of each head rotated by p f'; v_g = R(unit(W_v h per head), p f(base, e))
                      a_i = softmax_j<=i(q_i . k_j * scale); o_i = R(sum_j a_ij v_j, -p_i f(base, e)); y = W_o concat_h o
  experts           : s = softmax(W_r h); c = s + bias; groups of neighbours, group score = max c in the group, experts outside
                      the `keep` best groups get c = -inf; chosen = `top` largest c; y = sum_chosen s_e * down_e(silu(gate_e h) * up_e h)
  layer             : x += LN(attention(LN(x; n1)); n1b);  x += LN(experts(LN(x; n2)); n2b)
  model             : x = embed[token] * scale; layers; logits = head LN(x; final)
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch

F = torch.float64


def layer_norm(v: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    mu = v.mean(-1, keepdim=True)
    dev = v - mu
    return dev / torch.sqrt((dev * dev).mean(-1, keepdim=True) + eps) * w


def unit_rms(v: torch.Tensor, eps: float) -> torch.Tensor:
    return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps)


def rotary_frequencies(base: float, n: int, scaling: Optional[dict] = None) -> Tuple[torch.Tensor, float]:
    i = torch.arange(n // 2, dtype=F)
    f = torch.exp(-2.0 * i / n * math.log(base))
    if not scaling:
        return f, 1.0
    ln_b = math.log(base)
    c = lambda t: n * math.log(scaling["original"] / (2.0 * math.pi * t)) / (2.0 * ln_b)
    lo = max(math.floor(c(scaling["fast"])), 0)
    hi = min(math.ceil(c(scaling["slow"])), n - 1)
    r = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / scaling["factor"] * r + f * (1.0 - r), 0.1 * math.log(scaling["factor"]) + 1.0


def rotate_pairs(v: torch.Tensor, angles: torch.Tensor, mag: float = 1.0) -> torch.Tensor:
    """v [..., n'] with n' >= 2 * angles.shape[-1]; the leading pairs rotate, the rest passes.  angles broadcast to v[..., :n/2]."""
    n = 2 * angles.shape[-1]
    out = v.clone()
    u, w = v[..., 0:n:2], v[..., 1:n:2]
    c, s = torch.cos(angles) * mag, torch.sin(angles) * mag
    out[..., 0:n:2] = u * c - w * s
    out[..., 1:n:2] = w * c + u * s
    return out


def attention(h: torch.Tensor, p: torch.Tensor, wq, wk, wv, wo, wqn, wkn, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (unit_rms(h @ wq.T, eps) * wqn).view(T, H, d)
    k = (unit_rms(h @ wk.T, eps) * wkn).view(T, G, d)
    v = unit_rms((h @ wv.T).view(T, G, e), eps)
    rot = m.get("rot")
    pf = p.to(F)
    if rot:
        if rot["dims"] > 0:
            f, mag = rotary_frequencies(rot["base"], rot["dims"], rot.get("scaling"))
            ang = pf[:, None, None] * f[None, None, :]
            q, k = rotate_pairs(q, ang, mag), rotate_pairs(k, ang, mag)
        fv, _ = rotary_frequencies(rot["base"], e)
        vang = pf[:, None, None] * fv[None, None, :]
        v = rotate_pairs(v, vang)
    out = torch.zeros(T, H, e, dtype=F)
    for hh in range(H):
        g = hh // (H // G)
        s = (q[:, hh] @ k[:, g].T) * m["scale"]
        s = s.masked_fill(p[None, :] > p[:, None], float("-inf"))
        out[:, hh] = torch.softmax(s, -1) @ v[:, g]
    if rot:
        out = rotate_pairs(out, -vang)
    return out.reshape(T, H * e) @ wo.T


def route(h: torch.Tensor, wr: torch.Tensor, bias: Optional[torch.Tensor], r: dict) -> Tuple[torch.Tensor, torch.Tensor]:
    """(chosen expert ids [T, top], their weights [T, top])."""
    E, top = r["experts"], r["top"]
    s = torch.softmax(h @ wr.T, -1)
    c = s + bias if bias is not None else s.clone()
    g = r.get("groups")
    if g and g["count"] > 1:
        n, keep = g["count"], g["keep"]
        score = c.view(-1, n, E // n).max(-1).values
        kept = torch.zeros_like(score, dtype=torch.bool)
        kept.scatter_(1, score.topk(keep, -1).indices, True)
        c = c.masked_fill(~kept.repeat_interleave(E // n, dim=1), float("-inf"))
    idx = c.topk(top, -1).indices
    return idx, s.gather(1, idx)


def experts(h: torch.Tensor, idx: torch.Tensor, wts: torch.Tensor, gate: List[torch.Tensor], up: List[torch.Tensor],
            down: List[torch.Tensor]) -> torch.Tensor:
    y = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(idx.shape[1]):
            n = int(idx[t, j])
            a = gate[n] @ h[t]
            y[t] += wts[t, j] * (down[n] @ (a * torch.sigmoid(a) * (up[n] @ h[t])))
    return y


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens, positions=None, streams: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence given whole; `streams` (a list) receives the residual stream after every layer."""
    w = {k: v.to(F) for k, v in w.items()}
    eps = cfg["norm"]["eps"]
    tok = torch.as_tensor(tokens, dtype=torch.long)
    p = torch.arange(len(tok)) if positions is None else torch.as_tensor(positions)
    x = w["embed"][tok] * cfg["embedding"]["scale"]
    for i, L in enumerate(cfg["layers"]):
        n = f"l{i}."
        y = attention(layer_norm(x, w[n + "norm1"], eps), p, w[n + "mix.q"], w[n + "mix.k"], w[n + "mix.v"], w[n + "mix.o"],
                      w[n + "mix.q.norm"], w[n + "mix.k.norm"], L["mixer"], eps)
        x = x + layer_norm(y, w[n + "norm1b"], eps)
        if L.get("mlp"):
            h = layer_norm(x, w[n + "norm2"], eps)
            r = L["mlp"]["router"]
            idx, wts = route(h, w[n + "mlp.router"], w.get(n + "mlp.correction"), r)
            E = r["experts"]
            y = experts(h, idx, wts, [w[f"{n}mlp.e{j}.gate"] for j in range(E)], [w[f"{n}mlp.e{j}.up"] for j in range(E)],
                        [w[f"{n}mlp.e{j}.down"] for j in range(E)])
            x = x + layer_norm(y, w[n + "norm2b"], eps)
        if streams is not None:
            streams.append(x.clone())
    return layer_norm(x, w["final.norm"], eps) @ w["head"].T


def greedy(cfg: dict, w: Dict[str, torch.Tensor], prompt: List[int], n: int) -> Tuple[List[int], List[float]]:
    """n greedy tokens after `prompt` (whole-sequence recomputation each time) and the top-1/top-2 margin of each choice."""
    ids, margins = list(prompt), []
    for _ in range(n):
        l = forward(cfg, w, ids)[-1]
        top = l.topk(2).values
        margins.append(float(top[0] - top[1]))
        ids.append(int(l.argmax()))
    return ids[len(prompt):], margins
