"""Small Dupolorn configurations with random weights for the tests: a config.json-shaped dict and bf16-exact weights under the
checkpoint's tensor names.  The engine helpers (replay, rel_rms, write_checkpoint, make_engine) are those of stack_util."""
import torch

from conftest import pkg
from stack_util import bf16_exact


def latent(second=False, heads=3, dim=24, rot_dim=16, vdim=20, kv_rank=40, base=5000.0, rot_dims=None, scale=0.2, mlp=None):
    return {"type": "latent_attention_2" if second else "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale,
                      "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims}}, "mlp": mlp}


def mlstm(heads=2, dim=40, vdim=24, cap=12.0, mlp=None):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}, "mlp": mlp}


def dense(ff=72):
    return {"kind": "dense", "ff": ff}


def moe(experts=6, top=2, ff=40, shared=56):
    d = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        d["shared"] = {"ff": shared}
    return d


def make_cfg(width=96, vocab=150, layers=None, taps=4, buckets=97, mul_prev=31, mul_cur=5, softcap=20.0, eps=1e-5, scale=3.0):
    if layers is None:
        layers = [mlstm(mlp=moe()), latent(mlp=dense()), latent(second=True, heads=2, dim=16, rot_dim=24, rot_dims=16, vdim=36, kv_rank=28,
                                                                 mlp=moe(experts=5, top=1, ff=24, shared=0)), mlstm(heads=3, dim=24, vdim=40)]
    return {"architecture": "Dupolorn", "canon": {"taps": taps},
            "embedding": {"scale": scale, "bigram": {"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur}},
            "norm": {"eps": eps}, "logit_softcap": softcap, "vocab": vocab, "width": width, "layers": layers}


def make_weights(cfg, seed=0):
    g = torch.Generator().manual_seed(seed)
    W, V = cfg["width"], cfg["vocab"]

    def mat(o, i, s=None):
        return bf16_exact(torch.randn(o, i, generator=g) * (s if s is not None else i ** -0.5))

    def vec(n, mean=1.0, jitter=0.1):
        return bf16_exact(mean + jitter * torch.randn(n, generator=g))

    w = {"embed": mat(V, W, 1.0), "bigram": mat(cfg["embedding"]["bigram"]["buckets"] + 1, W, 0.7), "head": mat(V, W, 3.0 * W ** -0.5),
         "final.norm": vec(1)[0]}
    for i, L in enumerate(cfg["layers"]):
        m, p = L["mixer"], f"l{i}."
        w[p + "norm1"], w[p + "norm2"] = vec(1, 1.2)[0], vec(1, 0.8)[0]
        w[p + "canon1"] = mat(W, cfg["canon"]["taps"], 0.3)
        d = torch.rand(i + 2, generator=g) * 0.3
        d[-1] += 0.6
        w[p + "dwa"] = bf16_exact(d)
        H = m["heads"]
        if L["type"] == "mlstm":
            w[p + "mix.q"], w[p + "mix.k"] = mat(H * m["dim"], W), mat(H * m["dim"], W)
            w[p + "mix.v"], w[p + "mix.g"] = mat(H * m["vdim"], W), mat(H * m["vdim"], W)
            w[p + "mix.i"], w[p + "mix.f"] = mat(H, W, 2.0 * W ** -0.5), mat(H, W, 2.0 * W ** -0.5)
            w[p + "mix.i.b"], w[p + "mix.f.b"] = vec(H, 0.0, 0.5), vec(H, 2.0, 1.0)
            w[p + "mix.norm"] = vec(H * m["vdim"])
        else:
            w[p + "mix.q"] = mat(H * (m["dim"] + m["rot_dim"]), W)
            w[p + "mix.dkv"] = mat(m["kv_rank"] + m["rot_dim"], W)
            w[p + "mix.dkv.norm"] = vec(m["kv_rank"])
            w[p + "mix.uk"] = mat(H * m["dim"], m["kv_rank"], 2.0 * m["kv_rank"] ** -0.5)
            w[p + "mix.uv"] = mat(H * m["vdim"], m["kv_rank"])
            if L["type"] == "latent_attention_2":
                w[p + "mix.sink"] = vec(H, 0.5, 1.5)
                w[p + "mix.g"] = mat(H * m["vdim"], W)
        w[p + "mix.o"] = mat(W, H * m["vdim"])
        f = L["mlp"]
        if f and f["kind"] == "dense":
            w[p + "mlp.gate"], w[p + "mlp.up"], w[p + "mlp.down"] = mat(f["ff"], W), mat(f["ff"], W), mat(W, f["ff"])
        elif f:
            w[p + "mlp.router"] = mat(f["router"]["experts"], W, 3.0 * W ** -0.5)   # spread-out scores: few near-ties
            for e in range(f["router"]["experts"]):
                w[f"{p}mlp.e{e}.up"], w[f"{p}mlp.e{e}.down"] = mat(f["expert"]["ff"], W), mat(W, f["expert"]["ff"])
            if f.get("shared"):
                w[p + "mlp.shared.up"], w[p + "mlp.shared.down"] = mat(f["shared"]["ff"], W), mat(W, f["shared"]["ff"])
    return w


def product_config(cfg):
    return pkg("config").DupolornConfig.from_dict(cfg, name="test")


def make_runner(cfg, w, dtype="float32", **kw):
    kw.setdefault("max_tokens", 512)
    kw.setdefault("max_model_len", 1024)
    kw.setdefault("block_size", 16)
    kw.setdefault("n_blocks", 80)
    kw.setdefault("max_logit_rows", 512)
    kw.setdefault("n_state_slots", 5)
    r = pkg("runner").make_runner(product_config(cfg), dtype=dtype, **kw)
    r.load_weights({k: v.clone() for k, v in w.items()})
    return r
