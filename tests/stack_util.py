"""Small Bopilorn configurations with random weights for the tests: a config.json-shaped dict, bf16-exact weights under the
checkpoint's tensor names, and helpers that drive a StackRunner through the engine."""
import json
import os

import numpy as np
import torch

from conftest import pkg


def make_cfg(width=96, vocab=200, layers=None, eps=1e-5, scale=2.0):
    """layers: list of dicts(heads, kv_heads, dim, vdim, rot_dims, base, scaling, att_scale, moe) -- see layer()."""
    return {"architecture": "Bopilorn", "embedding": {"scale": scale}, "norm": {"eps": eps}, "vocab": vocab, "width": width,
            "layers": layers or [layer(), layer(kv_heads=2, dim=32, vdim=48, rot_dims=16, scaling=None,
                                               moe=dict(experts=6, top=2, groups=3, keep=2, ff=40))]}


def layer(heads=4, kv_heads=1, dim=48, vdim=32, rot_dims=None, base=10000.0, att_scale=0.25,
          scaling=dict(factor=4.0, original=64, fast=16.0, slow=2.0), moe=dict(experts=8, top=3, groups=4, keep=2, ff=24)):
    rot = {"base": base, "dims": dim if rot_dims is None else rot_dims}
    if scaling:
        rot["scaling"] = dict(scaling)
    mlp = None
    if moe:
        mlp = {"kind": "moe", "expert": {"ff": moe["ff"]},
               "router": {"experts": moe["experts"], "top": moe["top"], "groups": {"count": moe["groups"], "keep": moe["keep"]}}}
    return {"type": "attention", "mixer": {"dim": dim, "vdim": vdim, "heads": heads, "kv_heads": kv_heads, "rot": rot,
                                           "scale": att_scale}, "mlp": mlp}


def bf16_exact(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.bfloat16).to(torch.float32)


def make_weights(cfg, seed=0, std=None):
    g = torch.Generator().manual_seed(seed)
    W, V = cfg["width"], cfg["vocab"]

    def mat(o, i, s=None):
        return bf16_exact(torch.randn(o, i, generator=g) * (s if s is not None else (std or i ** -0.5)))

    def vec(n, jitter=0.1):
        return bf16_exact(1.0 + jitter * torch.randn(n, generator=g))

    w = {"embed": mat(V, W, 1.0), "head": mat(V, W), "final.norm": vec(W)}
    for i, L in enumerate(cfg["layers"]):
        m, p = L["mixer"], f"l{i}."
        for n in ("norm1", "norm1b", "norm2", "norm2b"):
            w[p + n] = vec(W)
        w[p + "mix.q"] = mat(m["heads"] * m["dim"], W)
        w[p + "mix.k"] = mat(m["kv_heads"] * m["dim"], W)
        w[p + "mix.v"] = mat(m["kv_heads"] * m["vdim"], W)
        w[p + "mix.q.norm"] = vec(m["heads"] * m["dim"])
        w[p + "mix.k.norm"] = vec(m["kv_heads"] * m["dim"])
        w[p + "mix.o"] = mat(W, m["heads"] * m["vdim"])
        if L["mlp"]:
            r, ff = L["mlp"]["router"], L["mlp"]["expert"]["ff"]
            w[p + "mlp.router"] = mat(r["experts"], W, 3.0 * W ** -0.5)   # spread-out scores: few near-ties
            w[p + "mlp.correction"] = bf16_exact(0.1 * torch.randn(r["experts"], generator=g))
            for e in range(r["experts"]):
                w[f"{p}mlp.e{e}.gate"] = mat(ff, W)
                w[f"{p}mlp.e{e}.up"] = mat(ff, W)
                w[f"{p}mlp.e{e}.down"] = mat(W, ff)
    return w


def product_config(cfg):
    return pkg("config").BopilornConfig.from_dict(cfg, name="test")


def make_runner(cfg, w, dtype="float32", **kw):
    kw.setdefault("max_tokens", 512)
    kw.setdefault("max_model_len", 1024)
    kw.setdefault("block_size", 16)
    kw.setdefault("n_blocks", 80)
    kw.setdefault("max_logit_rows", 512)
    r = pkg("runner").make_runner(product_config(cfg), dtype=dtype, **kw)
    r.load_weights({k: v.clone() for k, v in w.items()})
    return r


def make_engine(r, max_seqs=4):
    return pkg("engine").LLMEngine(r, max_num_batched_tokens=r.max_tokens, max_num_seqs=max_seqs, max_model_len=r.max_model_len)


def replay(eng, schedule, prompts):
    """schedule: list of steps, each a list of (name, n_new) in batch order; every row's logits are kept.
    Returns {name: [T, vocab] fp32} in position order; requests are released when their prompt ends."""
    E = pkg("engine")
    live, at, out = {}, {}, {n: [] for n in prompts}
    for step in schedule:
        items = []
        for name, n in step:
            lo = at.get(name, 0)
            toks = prompts[name][lo:lo + n]
            if name not in live:
                live[name] = E.Request(name, list(toks), max_tokens=0)
                eng.add_request(live[name])
            else:
                live[name].prompt_ids.extend(toks)
            items.append((live[name], n, list(range(n))))
            at[name] = lo + n
        rows = eng.step_given(items)
        logits = eng.runner.logits_last(rows)
        k = 0
        for name, n in step:
            out[name].append(logits[k:k + n])
            k += n
            if at[name] == len(prompts[name]):
                eng.abort_request(name)
                del live[name]
    return {n: np.concatenate(v) for n, v in out.items() if v}


def rel_rms(got, want):
    """Per row: rms over the vocabulary of the centred difference, over the rms of the centred reference logits."""
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    ref = want - want.mean(-1, keepdims=True)
    return np.sqrt((d ** 2).mean(-1)) / np.sqrt((ref ** 2).mean(-1)).mean()


def write_checkpoint(path, cfg, w):
    from safetensors.torch import save_file
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in w.items()}, os.path.join(path, "model.safetensors"))
