"""GPU parity of layer-list models (the Bopilorn design) against oracle/stack_oracle.py: every mechanism alone through its
per-kernel entry point, then whole models through the runner, the engine's externally scheduled steps and its own scheduler.

The 32-bit serving mode is held to the float64 oracle tightly (it shares every rounding point with nothing); the bf16 mode
is held to it within bf16 noise, and to itself across schedules."""
import ctypes as C

import numpy as np
import pytest
import torch

import stack_util as U
from conftest import pkg
from oracle import stack_oracle as SO

pytestmark = pytest.mark.gpu
F32_TOL = 2e-5      # relative rms of a logit row, 32-bit mode against the float64 oracle
DEV = "cuda"


def lib():
    return pkg("_abi").lib()


def check(rc):
    pkg("_abi").check(rc)


_KEEP = []     # device copies stay referenced while kernels that got only their addresses may still run


def dev(t, dtype=None):
    d = t.to(device=DEV, dtype=dtype or t.dtype).contiguous()
    _KEEP.append(d)
    del _KEEP[:-64]
    return d


def sync():
    torch.cuda.synchronize()


# ---- mechanisms alone ------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("f32", [1, 0])
@pytest.mark.parametrize("width", [96, 200, 1030])
def test_layer_norm_sandwich(f32, width):
    g = torch.Generator().manual_seed(width)
    T, parts = 7, 3
    adt = torch.float32 if f32 else torch.bfloat16
    x = torch.randn(T, width, generator=g) * 3 + 0.5
    y = (torch.randn(T, width, generator=g) * 2 - 1).to(adt)
    yp = torch.randn(T, parts, width, generator=g)
    wa, wb = 1 + 0.2 * torch.randn(width, generator=g), 1 + 0.2 * torch.randn(width, generator=g)
    eps = 1e-3
    for use_parts in (False, True):
        xd, out = dev(x.clone()), torch.zeros(T, width, dtype=adt, device=DEV)
        check(lib().b200_layernorm_stream(f32, xd.data_ptr(), None if use_parts else dev(y).data_ptr(),
                                          dev(yp).data_ptr() if use_parts else None, parts, dev(wa).data_ptr(), dev(wb).data_ptr(),
                                          out.data_ptr(), None, T, width, eps, None))
        sync()
        yy = yp.double().sum(1) if use_parts else y.double()
        want_x = x.double() + SO.layer_norm(yy, wa.double(), eps)
        want_h = SO.layer_norm(want_x, wb.double(), eps)
        assert torch.allclose(xd.cpu().double(), want_x, atol=2e-5, rtol=1e-5)
        assert torch.allclose(out.cpu().double(), want_h, atol=2e-5 if f32 else 3e-2, rtol=1e-5 if f32 else 1e-2)
    # pre-norm only, through a row gather (the logit rows)
    rows = torch.tensor([5, 0, 5], dtype=torch.int32)
    xd, out = dev(x.clone()), torch.zeros(3, width, dtype=adt, device=DEV)
    check(lib().b200_layernorm_stream(f32, xd.data_ptr(), None, None, 0, None, dev(wb).data_ptr(), out.data_ptr(), dev(rows).data_ptr(),
                                      3, width, eps, None))
    sync()
    assert torch.equal(xd.cpu(), x)
    assert torch.allclose(out.cpu().double(), SO.layer_norm(x[rows.long()].double(), wb.double(), eps), atol=2e-5 if f32 else 3e-2,
                          rtol=1e-5 if f32 else 1e-2)


def _tables(base, dims, scaling, vdim, n_pos):
    Cf = pkg("config")
    rot = Cf.RotarySpec(base=base, dims=dims, **(dict(scaled=True, **scaling) if scaling else {})).table(n_pos) if dims else None
    return rot, Cf.RotarySpec(base=base, dims=vdim).table(n_pos)


@pytest.mark.parametrize("heads,kv,dim,vdim,rot_dims,scaling", [
    (4, 2, 32, 48, 16, None), (3, 1, 24, 8, 24, dict(factor=4.0, original=64, fast=16.0, slow=2.0)), (2, 2, 16, 16, 0, None)])
def test_qk_norm_rotation_and_cache_write(heads, kv, dim, vdim, rot_dims, scaling):
    g = torch.Generator().manual_seed(heads * 100 + dim)
    T, bs, nb, eps, base = 9, 8, 12, 1e-5, 1000.0
    pos = torch.tensor([0, 1, 2, 7, 8, 9, 300, 301, 511], dtype=torch.int32)
    slots = torch.tensor([5 * bs + 0, 5 * bs + 1, 5 * bs + 2, 5 * bs + 7, 2 * bs + 0, 2 * bs + 1, 11 * bs + 4, 11 * bs + 5, 7],
                         dtype=torch.int32)
    qn, kn, vn = heads * dim, kv * dim, kv * vdim
    qkv = torch.randn(T, qn + kn + vn, generator=g) * 2
    qw, kw = 1 + 0.3 * torch.randn(qn, generator=g), 1 + 0.3 * torch.randn(kn, generator=g)
    rot, vrot = _tables(base, rot_dims, scaling, vdim, 512)
    kc, vc = torch.zeros(nb, kv, bs, dim, device=DEV), torch.zeros(nb, kv, bs, vdim, device=DEV)
    qo = torch.zeros(T, qn, device=DEV)
    check(lib().b200_qk_norm_rotate_cache(1, dev(qkv).data_ptr(), dev(qw).data_ptr(), dev(kw).data_ptr(), dev(pos).data_ptr(),
                                          dev(slots).data_ptr(), dev(rot).data_ptr() if rot is not None else None, rot_dims,
                                          dev(vrot).data_ptr(), qo.data_ptr(), kc.data_ptr(), vc.data_ptr(), T, heads, kv, dim, vdim,
                                          bs, eps, 512, None))
    sync()
    x = qkv.double()
    q = (SO.unit_rms(x[:, :qn], eps) * qw.double()).view(T, heads, dim)
    k = (SO.unit_rms(x[:, qn:qn + kn], eps) * kw.double()).view(T, kv, dim)
    v = SO.unit_rms(x[:, qn + kn:].view(T, kv, vdim), eps)
    p = pos.double()
    if rot_dims:
        f, mag = SO.rotary_frequencies(base, rot_dims, scaling)
        q, k = SO.rotate_pairs(q, p[:, None, None] * f, mag), SO.rotate_pairs(k, p[:, None, None] * f, mag)
    v = SO.rotate_pairs(v, p[:, None, None] * SO.rotary_frequencies(base, vdim)[0])
    assert torch.allclose(qo.cpu().double().view(T, heads, dim), q, atol=3e-5)
    kcc, vcc = kc.cpu().double(), vc.cpu().double()
    for t in range(T):
        b, o = int(slots[t]) // bs, int(slots[t]) % bs
        assert torch.allclose(kcc[b, :, o], k[t], atol=3e-5), t
        assert torch.allclose(vcc[b, :, o], v[t], atol=3e-5), t
    assert int((kcc.abs().sum(-1) > 0).sum()) == T * kv      # nothing else was written


@pytest.mark.parametrize("heads,kv,dim,vdim,rot_dims", [(4, 2, 64, 96, 32), (2, 1, 128, 128, 128), (3, 3, 80, 64, 0)])
def test_wide_cache_rows_keep_a_zero_tail(heads, kv, dim, vdim, rot_dims):
    """bf16 rows into 128-wide query and cache rows: the head's dimensions match the oracle, the tail is written as zero (the
    caches start as NaN), other slots stay untouched."""
    g = torch.Generator().manual_seed(heads + dim)
    T, bs, nb, eps, base, R = 5, 4, 6, 1e-5, 1000.0, 128
    pos = torch.tensor([0, 1, 9, 300, 511], dtype=torch.int32)
    slots = torch.tensor([0, 1, 2 * bs + 3, 5 * bs, 4 * bs + 1], dtype=torch.int32)
    qn, kn, vn = heads * dim, kv * dim, kv * vdim
    qkv = U.bf16_exact(torch.randn(T, qn + kn + vn, generator=g) * 2)
    qw, kw = 1 + 0.3 * torch.randn(qn, generator=g), 1 + 0.3 * torch.randn(kn, generator=g)
    rot, vrot = _tables(base, rot_dims, None, vdim, 512)
    kc = torch.full((nb, kv, bs, R), float("nan"), dtype=torch.bfloat16, device=DEV)
    vc = torch.full((nb, kv, bs, R), float("nan"), dtype=torch.bfloat16, device=DEV)
    qo = torch.full((T, heads, R), float("nan"), dtype=torch.bfloat16, device=DEV)
    check(lib().b200_qk_norm_rotate_cache_wide(dev(qkv, torch.bfloat16).data_ptr(), dev(qw).data_ptr(), dev(kw).data_ptr(),
                                               dev(pos).data_ptr(), dev(slots).data_ptr(), dev(rot).data_ptr() if rot is not None else None,
                                               rot_dims, dev(vrot).data_ptr(), qo.data_ptr(), kc.data_ptr(), vc.data_ptr(), T, heads, kv,
                                               dim, vdim, bs, eps, 512, R, R, None))
    sync()
    x = qkv.double()
    q = (SO.unit_rms(x[:, :qn], eps) * qw.double()).view(T, heads, dim)
    k = (SO.unit_rms(x[:, qn:qn + kn], eps) * kw.double()).view(T, kv, dim)
    v = SO.unit_rms(x[:, qn + kn:].view(T, kv, vdim), eps)
    p = pos.double()
    if rot_dims:
        f, mag = SO.rotary_frequencies(base, rot_dims, None)
        q, k = SO.rotate_pairs(q, p[:, None, None] * f, mag), SO.rotate_pairs(k, p[:, None, None] * f, mag)
    v = SO.rotate_pairs(v, p[:, None, None] * SO.rotary_frequencies(base, vdim)[0])
    qc, kcc, vcc = qo.cpu().double(), kc.cpu().double(), vc.cpu().double()
    assert torch.allclose(qc[..., :dim], q, atol=3e-2, rtol=1e-2) and (qc[..., dim:] == 0).all()
    written = set()
    for t in range(T):
        b, o = int(slots[t]) // bs, int(slots[t]) % bs
        written.add((b, o))
        assert torch.allclose(kcc[b, :, o, :dim], k[t], atol=3e-2, rtol=1e-2) and (kcc[b, :, o, dim:] == 0).all(), t
        assert torch.allclose(vcc[b, :, o, :vdim], v[t], atol=3e-2, rtol=1e-2) and (vcc[b, :, o, vdim:] == 0).all(), t
    for b in range(nb):
        for o in range(bs):
            if (b, o) not in written:
                assert torch.isnan(kcc[b, :, o]).all() and torch.isnan(vcc[b, :, o]).all()


@pytest.mark.parametrize("heads,vdim,row,rotated", [(3, 96, 128, True), (2, 128, 128, True), (4, 64, 128, False), (1, 2, 2, True)])
def test_output_rows_turn_back_and_pack(heads, vdim, row, rotated):
    g = torch.Generator().manual_seed(vdim)
    T, base = 6, 1000.0
    pos = torch.tensor([0, 1, 5, 130, 400, 511], dtype=torch.int32)
    a = U.bf16_exact(torch.randn(T, heads, row, generator=g))
    vrot = pkg("config").RotarySpec(base=base, dims=vdim).table(512)
    src = dev(a, torch.bfloat16)
    out = src if row == vdim else torch.full((T, heads, vdim), float("nan"), dtype=torch.bfloat16, device=DEV)
    check(lib().b200_rotate_back_rows(src.data_ptr(), row, out.data_ptr(), dev(pos).data_ptr(), dev(vrot).data_ptr() if rotated else None,
                                      T, heads, vdim, 512, None))
    sync()
    want = a[..., :vdim].double()
    if rotated:
        want = SO.rotate_pairs(want, -pos.double()[:, None, None] * SO.rotary_frequencies(base, vdim)[0])
    assert torch.allclose(out.cpu().double(), want, atol=2e-2, rtol=1e-2)


def _attn_oracle(q, k, v, ctx, scale, fv, qpos):
    """q [H, d], k [n, G, d], v [n, G, e] of one sequence; the row sees the first ctx keys."""
    H, G = q.shape[0], k.shape[1]
    out = torch.zeros(H, v.shape[-1], dtype=torch.float64)
    for h in range(H):
        g = h // (H // G)
        a = torch.softmax((k[:ctx, g] @ q[h]) * scale, 0)
        out[h] = a @ v[:ctx, g]
    return SO.rotate_pairs(out, -(qpos * fv)[None, :]) if fv is not None else out


@pytest.mark.parametrize("shared", [0, 1])
@pytest.mark.parametrize("f32", [1, 0])
@pytest.mark.parametrize("heads,kv,dim,vdim", [(4, 2, 32, 48), (6, 1, 24, 8), (2, 2, 16, 160)])
def test_paged_attention_edges_far_keys_and_both_kernels(f32, heads, kv, dim, vdim, shared):
    g = torch.Generator().manual_seed(dim * 7 + vdim)
    bs, n_seq_tokens, base, scale = 16, 700, 10000.0, 0.3
    nb = (n_seq_tokens + bs - 1) // bs
    cdt = torch.float32 if f32 else torch.bfloat16
    k = torch.randn(n_seq_tokens, kv, dim, generator=g)
    v = torch.randn(n_seq_tokens, kv, vdim, generator=g)
    far = 3                                     # a key far back, three tokens into the first block
    k, v = k.to(cdt).float(), v.to(cdt).float()
    perm = torch.randperm(nb + 5, generator=g)[:nb]
    kc, vc = torch.zeros(nb + 5, kv, bs, dim, dtype=cdt), torch.zeros(nb + 5, kv, bs, vdim, dtype=cdt)
    for j in range(n_seq_tokens):
        kc[perm[j // bs], :, j % bs], vc[perm[j // bs], :, j % bs] = k[j].to(cdt), v[j].to(cdt)
    # rows: the first tokens, both sides of block borders, and long contexts; the last rows form one run of consecutive tokens
    ctxs = [1, 2, 3, 15, 16, 17, 31, 32, 33, 127, 128, 129, 700, 640] + list(range(660, 700))
    T = len(ctxs)
    q = torch.randn(T, heads, dim, generator=g)
    # rows 12 and 13 look straight at the far key: its score stands out by ~40, so a lost or misplaced key 3 changes everything
    for r in (12, 13):
        q[r] = k[far, [h // (heads // kv) for h in range(heads)]] * (40.0 / scale / dim)
    pos = torch.tensor([c - 1 for c in ctxs], dtype=torch.int32)
    _, vrot = _tables(base, 0, None, vdim, 1024)
    fv = SO.rotary_frequencies(base, vdim)[0]
    bt = perm.to(torch.int32)[None, :].contiguous()
    want = torch.stack([_attn_oracle(q[t].double(), k.double(), v.double(), ctxs[t], scale, fv, float(pos[t])) for t in range(T)])
    assert want[12].abs().max() > 0 and torch.allclose(SO.rotate_pairs(want[12], (float(pos[12]) * fv)[None]),
                                                       v[far, [h // (heads // kv) for h in range(heads)]].double(), atol=5e-2)
    ws = torch.zeros(int(lib().b200_paged_attn_anydim_workspace_bytes(T)), dtype=torch.uint8, device=DEV)
    seq = torch.zeros(T, dtype=torch.int32)
    if True:
        out = torch.zeros(T, heads, vdim, dtype=cdt, device=DEV)
        check(lib().b200_paged_attn_anydim(f32, dev(q).data_ptr(), dev(kc).data_ptr(), dev(vc).data_ptr(), dev(bt).data_ptr(), bt.shape[1],
                                           dev(seq).data_ptr(), dev(torch.tensor(ctxs, dtype=torch.int32)).data_ptr(),
                                           dev(pos).data_ptr(), dev(vrot).data_ptr(), 1024, out.data_ptr(), T, heads, kv, dim, vdim, bs,
                                           scale, shared, ws.data_ptr(), None))
        sync()
        assert torch.allclose(out.cpu().double(), want, atol=2e-5 if f32 else 2e-2, rtol=0 if f32 else 2e-2), shared


@pytest.mark.parametrize("experts,top,groups,keep", [(8, 3, 4, 2), (6, 1, 1, 1), (12, 4, 3, 3), (64, 6, 8, 3), (5, 5, 1, 1)])
def test_router_against_the_oracle(experts, top, groups, keep):
    g = torch.Generator().manual_seed(experts)
    T, W = 40, 72
    x = torch.randn(T, W, generator=g)
    wr = U.bf16_exact(torch.randn(experts, W, generator=g) * 0.5)
    bias = torch.randn(experts, generator=g) * 0.3 - 0.5        # negative choice scores happen
    ids = torch.zeros(T, top, dtype=torch.int32, device=DEV)
    wts = torch.zeros(T, top, device=DEV)
    check(lib().b200_moe_route(1, dev(x).data_ptr(), dev(wr, torch.bfloat16).data_ptr(), dev(bias).data_ptr(), T, W, experts, top, groups,
                               keep, ids.data_ptr(), wts.data_ptr(), None))
    sync()
    r = dict(experts=experts, top=top, groups=dict(count=groups, keep=keep))
    wi, ww = SO.route(x.double(), wr.double(), bias.double(), r)
    assert torch.equal(ids.cpu().long().sort(-1).values, wi.sort(-1).values)
    got = torch.zeros(T, experts, dtype=torch.float64).scatter_(1, ids.cpu().long(), wts.cpu().double())
    assert torch.allclose(got, torch.zeros(T, experts, dtype=torch.float64).scatter_(1, wi, ww), atol=1e-6)


@pytest.mark.parametrize("T,W,experts,top,groups,keep", [(1, 72, 8, 3, 4, 2), (40, 136, 12, 4, 3, 3), (300, 64, 64, 6, 8, 3), (17, 520, 132, 5, 1, 1),
                                                         (33, 80, 6, 2, 3, 2), (5, 64, 5, 5, 1, 1)])
def test_router_with_tensor_core_logits(T, W, experts, top, groups, keep):
    """bf16 rows: logits from the tcgen05 linear with fp32 output (one and several token tiles, more experts than a slab),
    then the per-token selection.  The logits against float64, the choice against the oracle."""
    g = torch.Generator().manual_seed(T)
    x = U.bf16_exact(torch.randn(T, W, generator=g))
    wr = U.bf16_exact(torch.randn(experts, W, generator=g) * 0.5)
    bias = torch.randn(experts, generator=g) * 0.3 - 0.5
    ids = torch.zeros(T, top, dtype=torch.int32, device=DEV)
    wts = torch.zeros(T, top, device=DEV)
    logits = torch.full((T, experts), float("nan"), device=DEV)
    check(lib().b200_moe_route_linear(dev(x, torch.bfloat16).data_ptr(), dev(wr, torch.bfloat16).data_ptr(), dev(bias).data_ptr(), T, W,
                                      experts, top, groups, keep, ids.data_ptr(), wts.data_ptr(), logits.data_ptr(), None))
    sync()
    assert torch.allclose(logits.cpu().double(), x.double() @ wr.double().T, atol=1e-4, rtol=1e-5)
    r = dict(experts=experts, top=top, groups=dict(count=groups, keep=keep))
    wi, ww = SO.route(x.double(), wr.double(), bias.double(), r)
    assert torch.equal(ids.cpu().long().sort(-1).values, wi.sort(-1).values)
    got = torch.zeros(T, experts, dtype=torch.float64).scatter_(1, ids.cpu().long(), wts.cpu().double())
    assert torch.allclose(got, torch.zeros(T, experts, dtype=torch.float64).scatter_(1, wi, ww), atol=1e-6)


@pytest.mark.parametrize("f32", [1, 0])
@pytest.mark.parametrize("T,W,ff,experts,top", [(5, 72, 40, 6, 2), (150, 96, 24, 4, 3), (70, 64, 130, 3, 1)])
def test_experts_token_and_grouped_forms(f32, T, W, ff, experts, top):
    g = torch.Generator().manual_seed(T)
    adt = torch.float32 if f32 else torch.bfloat16
    x = torch.randn(T, W, generator=g).to(adt)
    gate = [U.bf16_exact(torch.randn(ff, W, generator=g) * W ** -0.5) for _ in range(experts)]
    up = [U.bf16_exact(torch.randn(ff, W, generator=g) * W ** -0.5) for _ in range(experts)]
    down = [U.bf16_exact(torch.randn(W, ff, generator=g) * ff ** -0.5) for _ in range(experts)]
    ids = torch.stack([torch.randperm(experts, generator=g)[:top] for _ in range(T)]).to(torch.int32)
    wts = torch.rand(T, top, generator=g)
    gu = torch.cat([torch.cat([gate[e], up[e]], 0) for e in range(experts)], 0)
    dn = torch.cat(down, 0)
    parts = torch.zeros(T, top, W, device=DEV)
    ws = torch.zeros(int(lib().b200_moe_workspace_bytes(T, top, experts, W, ff)), dtype=torch.uint8, device=DEV)
    check(lib().b200_moe_experts(f32, dev(x).data_ptr(), dev(gu, torch.bfloat16).data_ptr(), dev(dn, torch.bfloat16).data_ptr(),
                                 dev(ids).data_ptr(), dev(wts).data_ptr(), T, W, ff, experts, top, parts.data_ptr(), ws.data_ptr(), None))
    sync()
    want = SO.experts(x.double(), ids.long(), wts.double(), [t.double() for t in gate], [t.double() for t in up], [t.double() for t in down])
    # bf16 activations with width and ff multiples of 8 take the tensor-core form, which rounds gate|up and the activated
    # rows to bf16 between its two products
    tc = not f32 and W % 8 == 0 and ff % 8 == 0
    assert torch.allclose(parts.cpu().double().sum(1), want, atol=3e-2 if tc else 3e-5)


def _experts_rounded(x, ids, wts, gate, up, down):
    """The tensor-core form's roundings: bf16 gate and up rows, bf16 silu, bf16 product, fp32 down rows times the weight."""
    rb = lambda t: t.to(torch.bfloat16).double()
    T, top = ids.shape
    out = torch.zeros(T, top, down[0].shape[0], dtype=torch.float64)
    for t in range(T):
        for j in range(top):
            e = int(ids[t, j])
            gt, ut = rb(gate[e].double() @ x[t].double()), rb(up[e].double() @ x[t].double())
            a = rb(rb(gt * torch.sigmoid(gt)) * ut)
            out[t, j] = (down[e].double() @ a) * wts[t, j].double()
    return out


@pytest.mark.parametrize("T,W,ff,experts,top", [(1, 64, 64, 8, 2), (3, 136, 72, 5, 5), (40, 64, 200, 4, 2), (300, 256, 136, 6, 3),
                                                (700, 128, 64, 3, 1), (3000, 64, 64, 4, 3), (100, 64, 128, 4, 1), (200, 72, 64, 4, 1)])
def test_experts_tensor_core_form(T, W, ff, experts, top):
    """Every token-tile size, runs that end inside a tile, experts nobody chose, slab rows past an expert's last row, ff
    that is and is not a multiple of 64 (activation in the epilogue or as a step of its own), more pairs than the grouping
    kernel holds in shared memory at a time."""
    g = torch.Generator().manual_seed(T + W)
    x = torch.randn(T, W, generator=g).to(torch.bfloat16)
    gate = [U.bf16_exact(torch.randn(ff, W, generator=g) * W ** -0.5) for _ in range(experts)]
    up = [U.bf16_exact(torch.randn(ff, W, generator=g) * W ** -0.5) for _ in range(experts)]
    down = [U.bf16_exact(torch.randn(W, ff, generator=g) * ff ** -0.5) for _ in range(experts)]
    ids = torch.stack([torch.randperm(experts, generator=g)[:top] for _ in range(T)]).to(torch.int32)
    if top == 1:
        ids[ids == experts - 1] = 0   # the last expert gets no token
    wts = torch.rand(T, top, generator=g)
    gu = torch.cat([torch.cat([gate[e], up[e]], 0) for e in range(experts)], 0)
    dn = torch.cat(down, 0)
    parts = torch.full((T, top, W), float("nan"), device=DEV)
    ws = torch.zeros(int(lib().b200_moe_workspace_bytes(T, top, experts, W, ff)), dtype=torch.uint8, device=DEV)
    for _ in range(2):   # the second call finds the first one's tables in the workspace
        check(lib().b200_moe_experts(0, dev(x).data_ptr(), dev(gu, torch.bfloat16).data_ptr(), dev(dn, torch.bfloat16).data_ptr(),
                                     dev(ids).data_ptr(), dev(wts).data_ptr(), T, W, ff, experts, top, parts.data_ptr(), ws.data_ptr(), None))
    sync()
    want = _experts_rounded(x, ids, wts, gate, up, down)
    got = parts.cpu().double()
    assert torch.isfinite(got).all()
    assert torch.allclose(got, want, atol=4e-3, rtol=4e-3)


@pytest.mark.parametrize("T,n,k", [(1, 5, 7), (70, 130, 33), (64, 64, 16)])
def test_fp32_linear(T, n, k):
    g = torch.Generator().manual_seed(n)
    x, w = torch.randn(T, k, generator=g), U.bf16_exact(torch.randn(n, k, generator=g))
    y = torch.zeros(T, n, device=DEV)
    check(lib().b200_linear_simt(1, 1, dev(x).data_ptr(), k, dev(w, torch.bfloat16).data_ptr(), y.data_ptr(), n, T, n, k, None))
    sync()
    assert torch.allclose(y.cpu().double(), x.double() @ w.double().T, atol=1e-4)


# ---- whole models ------------------------------------------------------------------------------------------------------------
ODD = dict(width=72, vocab=97, scale=0.5, eps=1e-6, layers=[
    U.layer(heads=2, kv_heads=2, dim=16, vdim=16, rot_dims=16, scaling=None, base=500.0, att_scale=0.5, moe=None),
    U.layer(heads=6, kv_heads=3, dim=8, vdim=24, rot_dims=4, att_scale=1.0, moe=dict(experts=5, top=1, groups=1, keep=1, ff=16)),
    U.layer(heads=3, kv_heads=1, dim=40, vdim=8, rot_dims=40, scaling=dict(factor=16.0, original=32, fast=8.0, slow=1.0),
            moe=dict(experts=9, top=4, groups=3, keep=3, ff=50))])


def _prompt(cfg, n, seed):
    return torch.randint(0, cfg["vocab"], (n,), generator=torch.Generator().manual_seed(seed)).tolist()


@pytest.fixture(scope="module")
def model_a():
    cfg = U.make_cfg()
    return cfg, U.make_weights(cfg, seed=11)


@pytest.fixture(scope="module")
def model_odd():
    cfg = U.make_cfg(**ODD)
    return cfg, U.make_weights(cfg, seed=12)


ODD2 = dict(width=54, vocab=61, scale=1.0, eps=1e-5, layers=[
    U.layer(heads=3, kv_heads=1, dim=6, vdim=10, rot_dims=2, base=77.0, att_scale=0.4, moe=dict(experts=3, top=2, groups=1, keep=1, ff=7)),
    U.layer(heads=1, kv_heads=1, dim=2, vdim=2, rot_dims=2, scaling=None, att_scale=1.0, moe=dict(experts=2, top=1, groups=2, keep=1, ff=1))])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sizes_no_vector_access_fits(dtype):
    """Width, ff and head sizes that are multiples of neither 8 nor 4 (the scalar forms of every kernel), one head, one
    key/value pair per head, one expert per group, in both serving modes."""
    cfg = U.make_cfg(**ODD2)
    w = U.make_weights(cfg, seed=14)
    ids = _prompt(cfg, 45, 9)
    want = SO.forward(cfg, w, ids).numpy()
    r = U.make_runner(cfg, w, dtype)
    eng = U.make_engine(r)
    got = U.replay(eng, [[("p", 20)], [("p", 2)]] + [[("p", 1)]] * 23, {"p": ids})["p"]
    r.close()
    e = U.rel_rms(got, want)
    if dtype == "float32":
        assert e.max() < F32_TOL
    else:
        assert np.median(e) < 0.03 and (e < 0.15).mean() > 0.9, (float(np.median(e)), float(e.max()))


@pytest.mark.parametrize("which", ["a", "odd"])
def test_whole_prompt_and_stream_against_the_oracle_fp32(which, model_a, model_odd):
    cfg, w = model_a if which == "a" else model_odd
    ids = _prompt(cfg, 75, 1)
    r = U.make_runner(cfg, w, "float32")
    tap = r.set_stream_tap(True)
    eng = U.make_engine(r)
    got = U.replay(eng, [[("p", 75)]], {"p": ids})["p"]
    streams = []
    want = SO.forward(cfg, w, ids, streams=streams).numpy()
    assert U.rel_rms(got, want).max() < F32_TOL
    t = tap[:len(streams) * 75 * cfg["width"]].view(len(streams), 75, cfg["width"]).cpu().double()
    for l, s in enumerate(streams):
        assert torch.allclose(t[l], s, atol=1e-4, rtol=1e-5), l
    r.close()


def test_every_schedule_gives_the_oracles_logits_fp32(model_a):
    """Prefill against token-by-token decoding, portions down to two tokens, unequal requests batched, a long decode tail,
    and blocks that are freed and taken again (the pool holds 12 blocks of 16; the four requests need 22)."""
    cfg, w = model_a
    prompts = {"a": _prompt(cfg, 70, 2), "b": _prompt(cfg, 37, 3), "c": _prompt(cfg, 3, 4), "d": _prompt(cfg, 90, 5)}
    want = {n: SO.forward(cfg, w, p).numpy() for n, p in prompts.items()}
    r = U.make_runner(cfg, w, "float32", n_blocks=12, max_tokens=128)
    eng = U.make_engine(r)
    schedules = {
        "token by token": [[("c", 1)]] * 3 + [[("b", 1)]] * 37,
        "portions": [[("a", n)] for n in (2, 14, 1, 16, 17, 2, 2, 3, 13)],
        "prefill then a long decode": [[("d", 30)]] + [[("d", 1)]] * 60,
        "mixed": ([[("a", 33), ("c", 1)], [("c", 1), ("b", 2), ("a", 2)], [("b", 30), ("a", 1), ("c", 1)]] +
                  [[("a", 1), ("b", 1)]] * 5 + [[("a", 29)]] + [[("d", 64)], [("d", 2)], [("d", 24)]]),
    }
    for name, sched in schedules.items():
        got = U.replay(eng, sched, prompts)
        assert len(eng.blocks.free) == 12, name
        for n, l in got.items():
            assert l.shape[0] == len(prompts[n]), (name, n)
            assert U.rel_rms(l, want[n]).max() < F32_TOL, (name, n)
    r.close()


def test_bf16_mode_within_bf16_noise_and_equal_across_schedules(model_a):
    cfg, w = model_a
    prompts = {"a": _prompt(cfg, 70, 2), "b": _prompt(cfg, 37, 3)}
    want = {n: SO.forward(cfg, w, p).numpy() for n, p in prompts.items()}
    r = U.make_runner(cfg, w, "bfloat16", n_blocks=12, max_tokens=128)
    eng = U.make_engine(r)
    whole = U.replay(eng, [[("a", 70)], [("b", 37)]], prompts)
    mixed = U.replay(eng, [[("a", 40), ("b", 2)], [("b", 20), ("a", 1)]] + [[("a", 1), ("b", 1)]] * 15 + [[("a", 14)]], prompts)
    for n in prompts:
        e = U.rel_rms(whole[n], want[n])
        assert np.median(e) < 0.03 and (e < 0.1).mean() > 0.9, (n, float(np.median(e)), float(e.max()))
        d = U.rel_rms(mixed[n], whole[n])      # the same arithmetic up to summation order (and a rare router near-tie)
        assert np.median(d) < 0.02 and (d < 0.1).mean() > 0.9, (n, float(np.median(d)), float(d.max()))
    r.close()


WIDE = dict(width=128, vocab=160, scale=1.5, eps=1e-5, layers=[
    U.layer(heads=4, kv_heads=1, dim=128, vdim=128, rot_dims=64, att_scale=0.09, moe=dict(experts=8, top=2, groups=2, keep=1, ff=64)),
    U.layer(heads=2, kv_heads=2, dim=128, vdim=128, rot_dims=128, scaling=None, att_scale=0.12, moe=None),
    U.layer(heads=4, kv_heads=2, dim=64, vdim=96, rot_dims=32, att_scale=0.12, moe=dict(experts=4, top=2, groups=1, keep=1, ff=72)),
    U.layer(heads=2, kv_heads=1, dim=80, vdim=128, rot_dims=80, att_scale=0.11, moe=None),
    U.layer(heads=2, kv_heads=1, dim=128, vdim=32, rot_dims=8, att_scale=0.09, moe=None)])


def test_128_wide_heads_take_the_tensor_core_attention_and_agree_with_the_generic_kernels():
    """bf16 mode with blocks of 128 tokens: layers with keys and values of 64 to 128 dimensions run the tcgen05 attention
    kernels (several group sizes in one model, so the row plan is rebuilt between layers; narrower heads sit in 128-wide
    cache rows with a zero tail), the last layer (32-wide values) keeps the generic kernels.  Against the
    oracle within bf16 noise, against the same model in blocks of 16 (generic kernels everywhere), and across schedules:
    keys beyond one and two blocks, portions that end at and next to a block border, decoding over a border."""
    cfg = U.make_cfg(**WIDE)
    w = U.make_weights(cfg, seed=13)
    prompts = {"a": _prompt(cfg, 300, 6), "b": _prompt(cfg, 131, 7), "c": _prompt(cfg, 40, 8)}
    want = {n: SO.forward(cfg, w, p).numpy() for n, p in prompts.items()}
    r = U.make_runner(cfg, w, "bfloat16", block_size=128, n_blocks=6, max_tokens=512, max_model_len=512)
    eng = U.make_engine(r)
    whole = U.replay(eng, [[("a", 300)], [("b", 131)], [("c", 40)]], prompts)
    mixed = U.replay(eng, [[("a", 127), ("b", 2)], [("a", 1), ("b", 126), ("c", 38)], [("a", 130), ("b", 1), ("c", 1)]] +
                     [[("a", 1), ("b", 1), ("c", 1)]] + [[("a", 1), ("b", 1)]] + [[("a", 1)]] * 20 + [[("a", 20)]], prompts)
    assert len(eng.blocks.free) == 6
    r.close()
    r16 = U.make_runner(cfg, w, "bfloat16", block_size=16, n_blocks=40, max_tokens=512, max_model_len=512)
    small = U.replay(U.make_engine(r16), [[("a", 300)], [("b", 131)], [("c", 40)]], prompts)
    r16.close()
    for n in prompts:
        e = U.rel_rms(whole[n], want[n])      # five layers of bf16 rounding; a wrong key, row or rotation gives errors near 1
        assert np.median(e) < 0.05 and (e < 0.15).mean() > 0.9, (n, float(np.median(e)), float(e.max()))
        for other in (mixed, small):
            d = U.rel_rms(other[n], whole[n])
            assert np.median(d) < 0.05 and (d < 0.15).mean() > 0.9, (n, float(np.median(d)), float(d.max()))


def test_greedy_generation_through_the_engines_own_scheduler(model_odd, tmp_path):
    """Checkpoint directory -> registry -> runner -> LLMEngine.generate (continuous batching, chunked prefill with a token
    budget of 16) against the oracle's greedy tokens.  The samplers read the logits in bf16 in both serving modes, so a mismatch
    is allowed only where the oracle's top-1/top-2 margin is below bf16 resolution at logit magnitude ~4."""
    cfg, w = model_odd
    C, R, E, Wt = pkg("config"), pkg("runner"), pkg("engine"), pkg("weights")
    U.write_checkpoint(str(tmp_path / "m"), cfg, w)
    pc = C.load_model_config(str(tmp_path / "m"))
    r = R.make_runner(pc, dtype="float32", max_tokens=16, max_model_len=256, block_size=16, n_blocks=24)
    r.load_weights(Wt.load_safetensors_dir(str(tmp_path / "m")))
    eng = E.LLMEngine(r, max_num_batched_tokens=16, max_num_seqs=3, max_model_len=256)
    prompts = [_prompt(cfg, n, 20 + n) for n in (5, 41, 18, 2)]
    outs = eng.generate(prompts, max_tokens=24)
    for p, o in zip(prompts, outs):
        ref, margins = SO.greedy(cfg, w, p, 24)
        for i, (a, b) in enumerate(zip(o, ref)):
            if a != b:
                assert margins[i] < 0.05, (i, margins[i])
                break
    assert len(eng.blocks.free) == 24
    r.close()
