"""GPU parity of the Dupolorn design against oracle/dupolorn_oracle.py: every mechanism alone through its per-kernel entry point
(with inputs built so that a lost key, a dropped sink, a stale state or a wrong tail shows), then whole models through the
runner, externally scheduled steps of the engine, and its own scheduler.  32-bit mode is held to the float64 oracle tightly;
bf16 mode within bf16 noise, and to itself across schedules."""
import math

import numpy as np
import pytest
import torch

import dupolorn_util as D
import stack_util as U
from conftest import pkg
from oracle import dupolorn_oracle as O

pytestmark = pytest.mark.gpu
F32_TOL = 2e-5
DEV = "cuda"
_KEEP = []


def lib():
    return pkg("_abi").lib()


def check(rc):
    pkg("_abi").check(rc)


def dev(t, dtype=None):
    d = t.to(device=DEV, dtype=dtype or t.dtype).contiguous()
    _KEEP.append(d)
    del _KEEP[:-64]
    return d


def i32(x):
    return dev(torch.tensor(x, dtype=torch.int32))


def sync():
    torch.cuda.synchronize()


def _prompt(cfg, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()


def _portions(total, sizes):
    """Cut `total` rows into portions cycling through `sizes`."""
    out, at, i = [], 0, 0
    while at < total:
        n = min(sizes[i % len(sizes)], total - at)
        out.append((at, n))
        at += n
        i += 1
    return out


# ---- mechanisms alone ------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("f32", [1, 0])
@pytest.mark.parametrize("taps,width", [(1, 40), (2, 96), (3, 100), (5, 264), (8, 72)])
def test_input_convolution_in_portions_with_tails_in_slots(f32, taps, width):
    """Two sequences advance side by side in portions of 1, 2, 3 and more rows (shorter and longer than the tail); the
    second one starts later in a slot the first left dirty."""
    g = torch.Generator().manual_seed(taps * 11 + width)
    n = {"a": 41, "b": 23}
    h = {k: torch.randn(v, width, generator=g) for k, v in n.items()}
    w = U.bf16_exact(torch.randn(width, taps, generator=g) * 0.4)
    want = {k: (h[k].double() + O.causal_conv(h[k].double(), w)) for k in n}
    hist = max(taps - 1, 1)
    tails = dev(torch.full((3, hist * width + 5), 7.5))         # dirty slots; stride not a multiple of the width
    got = {k: torch.zeros(v, width) for k, v in n.items()}
    sched = {"a": _portions(41, [1, 2, 1, 3, 9, 1, 1, 2, 12]), "b": _portions(23, [2, 1, 1, 7, 1, 3])}
    slot = {"a": 2, "b": 0}
    adt = torch.float32 if f32 else torch.bfloat16
    for step in range(max(len(v) for v in sched.values())):
        names = [k for k in ("a", "b") if step < len(sched[k])]
        rows = torch.cat([h[k][sched[k][step][0]:sched[k][step][0] + sched[k][step][1]] for k in names])
        pos, rts, start = [], [], [0]
        for si, k in enumerate(names):
            lo, cnt = sched[k][step]
            pos += list(range(lo, lo + cnt))
            rts += [si] * cnt
            start.append(start[-1] + cnt)
        T = rows.shape[0]
        out = torch.zeros(T, width, dtype=adt, device=DEV)
        check(lib().b200_canon_conv(f32, dev(rows).data_ptr(), dev(w).data_ptr(), out.data_ptr(), T, width, taps, i32(pos).data_ptr(),
                                    i32(rts).data_ptr(), i32(start).data_ptr(), i32([slot[k] for k in names]).data_ptr(),
                                    tails.data_ptr(), tails.shape[1], None))
        sync()
        for si, k in enumerate(names):
            lo, cnt = sched[k][step]
            got[k][lo:lo + cnt] = out[start[si]:start[si + 1]].float().cpu()
    for k in n:
        assert torch.allclose(got[k].double(), want[k], atol=1e-5 if f32 else 3e-2, rtol=0 if f32 else 2e-2), k


def test_bigram_rows_first_token_and_previous_token_across_steps():
    g = torch.Generator().manual_seed(5)
    V, W, buckets, mp, mc, scale = 90, 72, 37, 1009, 13, 2.5
    E, B = U.bf16_exact(torch.randn(V, W, generator=g)), U.bf16_exact(torch.randn(buckets + 1, W, generator=g))
    ids = torch.randint(0, V, (30,), generator=g).tolist()
    want = O.embed_tokens(ids, E, scale, B, buckets, mp, mc)
    state = dev(torch.full((4, 6), 77, dtype=torch.int32))      # slot stride 6 ints; a dirty previous token
    got = []
    for lo, n in _portions(30, [1, 1, 4, 2, 9]):
        out = torch.zeros(n, W, device=DEV)
        check(lib().b200_embed_bigram(i32(ids[lo:lo + n]).data_ptr(), dev(E, torch.bfloat16).data_ptr(), dev(B, torch.bfloat16).data_ptr(),
                                      out.data_ptr(), n, W, V, scale, i32(list(range(lo, lo + n))).data_ptr(), i32([0] * n).data_ptr(),
                                      i32([0, n]).data_ptr(), i32([3]).data_ptr(), 1, state.data_ptr(), 6, buckets, mp, mc, None))
        sync()
        got.append(out.cpu())
    assert torch.allclose(torch.cat(got).double(), want, atol=1e-6)
    assert int(state[3, 0]) == ids[-1] and int(state[2, 0]) == 77


@pytest.mark.parametrize("f32", [1, 0])
def test_closing_sum_depth_average_and_the_two_norms(f32):
    g = torch.Generator().manual_seed(9)
    T, W, n_res, top, eps = 7, 100, 4, 3, 1e-5
    adt = torch.float32 if f32 else torch.bfloat16
    u = torch.randn(T, W, generator=g)
    ym, yf, ys = (torch.randn(T, W, generator=g).to(adt).float() for _ in range(3))
    parts = torch.randn(T, top, W, generator=g)
    res = torch.randn(n_res, T, W, generator=g)
    dwa, g1, g2 = torch.rand(n_res, generator=g), torch.tensor([1.3]), torch.tensor([0.6])
    x_new = u.double() + (ym.double() + yf.double() + parts.double().sum(1) + ys.double())
    avg = sum(dwa[j].double() * res[j].double() for j in range(n_res - 1)) + dwa[-1].double() * x_new
    unit = O.rms_unit(avg, eps)
    d_u, d_res = dev(u.clone()), dev(res.clone())
    h1f = torch.zeros(T, W, device=DEV)
    h1a, h2 = torch.zeros(T, W, dtype=adt, device=DEV), torch.zeros(T, W, dtype=adt, device=DEV)
    check(lib().b200_parallel_close(f32, d_u.data_ptr(), dev(ym, adt).data_ptr(), dev(yf, adt).data_ptr(), dev(parts).data_ptr(), top,
                                    dev(ys, adt).data_ptr(), d_res.data_ptr(), T * W, n_res, dev(dwa).data_ptr(), dev(g1).data_ptr(),
                                    dev(g2).data_ptr(), h1f.data_ptr(), h1a.data_ptr(), h2.data_ptr(), T, W, eps, None))
    sync()
    assert torch.allclose(d_res[-1].cpu().double(), x_new, atol=1e-5)
    assert torch.allclose(d_u.cpu().double(), avg, atol=1e-5)
    assert torch.allclose(h1f.cpu().double(), unit * 1.3, atol=1e-5)
    tol = dict(atol=1e-5) if f32 else dict(atol=2e-2, rtol=1e-2)
    assert torch.allclose(h1a.float().cpu().double(), unit * float(g1), **tol) and torch.allclose(h2.float().cpu().double(), unit * float(g2), **tol)


def _latent_scores_oracle(q, rows, ctx, rank, scale, sink):
    """q [heads, rank + rd] float64 against cache rows [n, rank + rd]; the values are the rows' leading `rank` entries."""
    s = (rows[:ctx] @ q.T).T * scale                      # [heads, ctx]
    mx = s.max(-1, keepdim=True).values
    if sink is not None:
        mx = torch.maximum(mx, sink[:, None])
    e = torch.exp(s - mx)
    den = e.sum(-1, keepdim=True) + (torch.exp(sink[:, None] - mx) if sink is not None else 0.0)
    return (e / den) @ rows[:ctx, :rank]


@pytest.mark.parametrize("shared", [0, 1])
@pytest.mark.parametrize("f32", [1, 0])
@pytest.mark.parametrize("heads,rank,rd,with_sink", [(3, 40, 16, True), (6, 24, 8, False), (2, 136, 32, True)])
def test_attention_over_latent_rows_sink_far_keys_and_block_borders(f32, heads, rank, rd, with_sink, shared):
    """One kv head whose values are the leading entries of its key rows (the value cache IS the key cache), a per-head sink,
    contexts on both sides of block borders, and two rows that look straight at a key far back."""
    g = torch.Generator().manual_seed(rank * 3 + rd)
    bs, n_tok, scale, krow = 16, 600, 0.25, rank + rd
    nb = (n_tok + bs - 1) // bs
    cdt = torch.float32 if f32 else torch.bfloat16
    rows = torch.randn(n_tok, krow, generator=g).to(cdt).float()
    perm = torch.randperm(nb + 4, generator=g)[:nb]
    kc = torch.zeros(nb + 4, 1, bs, krow, dtype=cdt)
    for j in range(n_tok):
        kc[perm[j // bs], 0, j % bs] = rows[j].to(cdt)
    ctxs = [1, 2, 3, 15, 16, 17, 31, 32, 33, 127, 128, 129, 600, 560] + list(range(565, 600))
    T, far = len(ctxs), 5
    q = torch.randn(T, heads, krow, generator=g)
    for r in (12, 13):
        q[r] = rows[far][None, :] * (40.0 / scale / krow)
    sink = (torch.randn(heads, generator=g) * 2.0 + 1.0) if with_sink else None
    want = torch.stack([_latent_scores_oracle(q[t].double(), rows.double(), ctxs[t], rank, scale, sink.double() if with_sink else None)
                        for t in range(T)])
    assert torch.allclose(want[12], rows[far, :rank].double().expand(heads, rank), atol=5e-2)      # the far key decides row 12
    if with_sink:      # a sink that is left out shows: the first row's single weight is well below one
        assert (want[0].abs().sum(-1) < 0.9 * rows[0, :rank].abs().sum()).any()
    ws = torch.zeros(int(lib().b200_paged_attn_anydim_workspace_bytes(T)), dtype=torch.uint8, device=DEV)
    d_kc = dev(kc)
    out = torch.zeros(T, heads, rank, dtype=cdt, device=DEV)
    check(lib().b200_paged_attn_anydim_ex(f32, dev(q).data_ptr(), d_kc.data_ptr(), d_kc.data_ptr(), dev(perm.to(torch.int32)[None, :]).data_ptr(),
                                          nb, i32([0] * T).data_ptr(), i32(ctxs).data_ptr(), i32([c - 1 for c in ctxs]).data_ptr(),
                                          out.data_ptr(), T, heads, 1, krow, rank, bs, scale, shared, ws.data_ptr(), krow, krow,
                                          dev(sink).data_ptr() if with_sink else None, None))
    sync()
    assert torch.allclose(out.float().cpu().double(), want, atol=2e-5 if f32 else 2e-2, rtol=0 if f32 else 2e-2)


@pytest.mark.parametrize("splits", [1, 3, 16])
@pytest.mark.parametrize("heads,rank,rd,with_sink", [(3, 32, 16, True), (6, 128, 32, False), (16, 512, 64, True), (20, 64, 0, True), (1, 16, 16, False)])
def test_latent_attention_on_the_tensor_cores(heads, rank, rd, with_sink, splits):
    """Decode rows and runs of consecutive rows (pairs of one CTA with different context lengths; more heads than a CTA holds
    pairs), contexts around tile (64) and block borders, a key far back that decides two rows, the sink; the context walked by
    one CTA or split over several (more splits than short contexts have tiles: empty shares) and merged."""
    g = torch.Generator().manual_seed(rank + heads)
    bs, n_tok, scale, krow = 16, 600, 0.25, rank + rd
    assert lib().b200_latent_attn_supported(heads, krow, rank) == 1 and lib().b200_latent_attn_supported(heads, krow + 8, rank) == 0
    nb = (n_tok + bs - 1) // bs
    rows = torch.randn(n_tok, krow, generator=g).to(torch.bfloat16).float()
    perm = torch.randperm(nb + 4, generator=g)[:nb]
    kc = torch.zeros(nb + 4, 1, bs, krow, dtype=torch.bfloat16)
    for j in range(n_tok):
        kc[perm[j // bs], 0, j % bs] = rows[j].to(torch.bfloat16)
    ctxs = [1, 2, 3, 15, 16, 17, 63, 64, 65, 127, 128, 129, 600, 560] + list(range(1, 40)) + list(range(565, 600))
    seq = [i for i in range(14)] + [14] * 39 + [15] * 35        # 14 decode rows of their own, then two runs (the table is shared)
    T, far = len(ctxs), 5
    q = torch.randn(T, heads, krow, generator=g).to(torch.bfloat16).float()
    for r in (12, 13):
        q[r] = (rows[far][None, :] * (40.0 / scale / krow)).to(torch.bfloat16).float()
    sink = (torch.randn(heads, generator=g) * 2.0 + 1.0) if with_sink else None
    want = torch.stack([_latent_scores_oracle(q[t].double(), rows.double(), ctxs[t], rank, scale, sink.double() if with_sink else None)
                        for t in range(T)])
    assert torch.allclose(want[12], rows[far, :rank].double().expand(heads, rank), atol=5e-2)
    ws = torch.zeros(int(lib().b200_paged_attn_anydim_workspace_bytes(T)), dtype=torch.uint8, device=DEV)
    bt = perm.to(torch.int32)[None, :].repeat(16, 1).contiguous()
    out = torch.full((T, heads, rank), float("nan"), dtype=torch.bfloat16, device=DEV)
    part = torch.full((T * heads * splits * (rank + 2),), float("nan"), device=DEV)
    check(lib().b200_latent_attn(dev(q).data_ptr(), dev(kc).data_ptr(), dev(bt).data_ptr(), nb, i32(seq).data_ptr(), i32(ctxs).data_ptr(),
                                 out.data_ptr(), T, heads, krow, rank, bs, scale, dev(sink).data_ptr() if with_sink else None, ws.data_ptr(),
                                 splits, part.data_ptr() if splits > 1 else None, None))
    sync()
    assert torch.isfinite(out.float()).all()
    assert torch.allclose(out.float().cpu().double(), want, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("f32", [1, 0])
@pytest.mark.parametrize("heads,dim,rd,rot_dims,rank,vdim,gate", [(3, 24, 16, 16, 40, 20, True), (2, 16, 24, 8, 28, 36, False), (5, 70, 2, 2, 9, 3, True),
                                                                  (4, 32, 16, 16, 48, 40, True), (2, 144, 64, 64, 256, 72, False)])
def test_latent_rows_rotation_and_the_per_head_expansions(f32, heads, dim, rd, rot_dims, rank, vdim, gate):
    g = torch.Generator().manual_seed(dim + rank)
    T, bs, eps, base = 11, 8, 1e-5, 3000.0
    adt = torch.float32 if f32 else torch.bfloat16
    qh, krow = dim + rd, rank + rd
    # inner sizes that are multiples of 16 take the tensor-core form in bf16 mode (rows that allow 16-byte copies and rows that
    # do not), everything else and the 32-bit mode the CUDA-core form
    ld = heads * qh + krow + (heads * vdim if gate else 0) + (3 if dim != 32 else 0)
    qkv = torch.randn(T, ld, generator=g).to(adt).float()
    nw = U.bf16_exact(1 + 0.2 * torch.randn(rank, generator=g))
    pos = [0, 1, 2, 7, 8, 9, 63, 64, 100, 511, 300]
    slots = torch.randperm(5 * bs, generator=g)[:T].tolist()
    table = pkg("config").RotarySpec(base=base, dims=rot_dims).table(512)
    cache = torch.zeros(5 * bs, krow, dtype=adt, device=DEV)
    qfull = torch.zeros(T, heads, krow, device=DEV)
    check(lib().b200_latent_prep(f32, dev(qkv, adt).data_ptr(), ld, dev(nw).data_ptr(), i32(pos).data_ptr(), i32(slots).data_ptr(),
                                 dev(table).data_ptr(), rot_dims, 512, qfull.data_ptr(), cache.data_ptr(), T, heads, dim, rd, rank, eps, None))
    uk = U.bf16_exact(torch.randn(heads, dim, rank, generator=g) * 0.3)      # [h][dim][rank]: the plain key of head h is uk[h] c
    uk_t = uk.transpose(1, 2).contiguous()
    check(lib().b200_head_linear(f32, 1, dev(qkv, adt).data_ptr(), ld, qh, dev(uk_t, torch.bfloat16).data_ptr(), qfull.data_ptr(),
                                 heads * krow, krow, None, 0, 0, T, heads, rank, dim, None))
    sync()
    dq = qkv.double()
    for t in range(T):
        dkv = dq[t, heads * qh:heads * qh + krow]
        c = O.rms_unit(dkv[:rank], eps) * nw.double()
        kr = O.rotate_pairs(dkv[rank:], pos[t], base, rot_dims)
        tol = dict(atol=1e-5) if f32 else dict(atol=3e-2, rtol=1e-2)
        assert torch.allclose(cache[slots[t]].float().cpu().double(), torch.cat([c, kr]), **tol), t
        for h in range(heads):
            qrow = dq[t, h * qh:(h + 1) * qh]
            assert torch.allclose(qfull[t, h, rank:].cpu().double(), O.rotate_pairs(qrow[dim:], pos[t], base, rot_dims), atol=1e-5), (t, h)
            assert torch.allclose(qfull[t, h, :rank].cpu().double(), uk[h].double().T @ qrow[:dim], atol=1e-4), (t, h)
    # the value expansion with its output gate
    lat = torch.randn(T, heads, rank, generator=g).to(adt).float()
    uv = U.bf16_exact(torch.randn(heads, vdim, rank, generator=g) * 0.3)
    out = torch.zeros(T, heads, vdim, dtype=adt, device=DEV)
    d_qkv = dev(qkv, adt)
    goff = heads * qh + krow
    check(lib().b200_head_linear(f32, 0, dev(lat, adt).data_ptr(), heads * rank, rank, dev(uv, torch.bfloat16).data_ptr(), out.data_ptr(),
                                 heads * vdim, vdim, d_qkv.data_ptr() + goff * d_qkv.element_size() if gate else None, ld, vdim, T, heads,
                                 vdim, rank, None))
    sync()
    want = torch.einsum("hvr,thr->thv", uv.double(), lat.double())
    if gate:
        want = want * torch.sigmoid(dq[:, goff:goff + heads * vdim].reshape(T, heads, vdim))
    assert torch.allclose(out.float().cpu().double(), want, atol=1e-5 if f32 else 3e-2, rtol=0 if f32 else 2e-2)


@pytest.mark.parametrize("f32", [1, 0])
@pytest.mark.parametrize("heads,dim,vdim", [(2, 40, 24), (1, 96, 70), (3, 16, 33), (2, 200, 8)])
def test_recurrence_in_portions_with_state_in_slots(f32, heads, dim, vdim):
    """Two sequences in portions of changing size next to each other, one in a slot that an earlier sequence left full; 300
    tokens of the longer one show that the running maximum keeps the state in range."""
    g = torch.Generator().manual_seed(dim + vdim)
    W, cap, eps = 64, 9.0, 1e-5
    m = {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}
    hd, hv = heads * dim, heads * vdim
    w = {"q": U.bf16_exact(torch.randn(hd, W, generator=g) * W ** -0.5), "k": U.bf16_exact(torch.randn(hd, W, generator=g) * W ** -0.5),
         "v": U.bf16_exact(torch.randn(hv, W, generator=g) * W ** -0.5), "g": U.bf16_exact(torch.randn(hv, W, generator=g) * W ** -0.5),
         "i": U.bf16_exact(torch.randn(heads, W, generator=g) * 0.4), "f": U.bf16_exact(torch.randn(heads, W, generator=g) * 0.4),
         "i.b": torch.randn(heads, generator=g), "f.b": 2.0 + torch.randn(heads, generator=g), "norm": 1 + 0.2 * torch.randn(hv, generator=g),
         "o": torch.eye(hv)}
    n = {"a": 300, "b": 45}
    adt = torch.float32 if f32 else torch.bfloat16
    x = {k: torch.randn(v, W, generator=g).to(adt).float() for k, v in n.items()}
    want = {k: O.mlstm(x[k].double(), m, w, "", eps) for k in n}       # o = identity: the gated, normed heads themselves
    fused_w = torch.cat([w["q"], w["k"], w["v"], w["g"]]).double()
    gates_w, gates_b = torch.cat([w["i"], w["f"]]), torch.cat([w["i.b"], w["f.b"]])
    sf = int(lib().b200_mlstm_state_floats(heads, dim, vdim))
    state = dev(torch.full((3, sf + 4), 3.25))
    sched = {"a": _portions(300, [1, 2, 64, 1, 1, 33, 3, 100]), "b": _portions(45, [2, 1, 1, 1, 17, 1, 5])}
    slot = {"a": 1, "b": 2}
    got = {k: torch.zeros(v, hv) for k, v in n.items()}
    ld = 2 * hd + 2 * hv
    for step in range(max(len(v) for v in sched.values())):
        names = [k for k in ("a", "b") if step < len(sched[k])]
        rows = torch.cat([x[k][sched[k][step][0]:sched[k][step][0] + sched[k][step][1]] for k in names])
        pos, start = [], [0]
        for k in names:
            lo, cnt = sched[k][step]
            pos += list(range(lo, lo + cnt))
            start.append(start[-1] + cnt)
        T = rows.shape[0]
        qkv = dev((rows.double() @ fused_w.T).float(), adt)       # the projections are not under test here
        gates = torch.zeros(T, 2 * heads, device=DEV)
        check(lib().b200_mlstm_gates(f32, dev(rows, adt).data_ptr(), dev(gates_w, torch.bfloat16).data_ptr(), dev(gates_b).data_ptr(),
                                     gates.data_ptr(), T, W, heads, cap, None))
        oraw = torch.zeros(T, hv, device=DEV)
        check(lib().b200_mlstm_scan(f32, qkv.data_ptr(), ld, 0, hd, 2 * hd, gates.data_ptr(), i32(pos).data_ptr(), i32(start).data_ptr(),
                                    i32([slot[k] for k in names]).data_ptr(), state.data_ptr(), state.shape[1], oraw.data_ptr(), len(names),
                                    heads, dim, vdim, None))
        out = torch.zeros(T, hv, dtype=adt, device=DEV)
        check(lib().b200_head_norm_gate(f32, oraw.data_ptr(), dev(w["norm"]).data_ptr(), qkv.data_ptr() + (2 * hd + hv) * qkv.element_size(),
                                        ld, out.data_ptr(), T, heads, vdim, eps, None))
        sync()
        for si, k in enumerate(names):
            lo, cnt = sched[k][step]
            got[k][lo:lo + cnt] = out[start[si]:start[si + 1]].float().cpu()
    for k in n:
        if f32:
            assert torch.allclose(got[k].double(), want[k], atol=2e-4, rtol=1e-4), k
        else:      # bf16 projections feed a long recurrence: most entries close, none wild
            d = (got[k].double() - want[k]).abs()
            assert d.median() < 0.03 and (d < 0.25).float().mean() > 0.98, (k, float(d.median()), float(d.max()))


@pytest.mark.parametrize("f32", [1, 0])
@pytest.mark.parametrize("T,W,experts,top", [(1, 72, 8, 3), (40, 136, 5, 1), (150, 64, 12, 4), (9, 100, 4, 4)])
def test_sigmoid_router_against_the_oracle(f32, T, W, experts, top):
    g = torch.Generator().manual_seed(T + experts)
    adt = torch.float32 if f32 else torch.bfloat16
    x = torch.randn(T, W, generator=g).to(adt).float()
    wr = U.bf16_exact(torch.randn(experts, W, generator=g) * 3.0 * W ** -0.5)
    ids, wts = torch.zeros(T, top, dtype=torch.int32, device=DEV), torch.zeros(T, top, device=DEV)
    check(lib().b200_moe_route_scores(f32, dev(x, adt).data_ptr(), dev(wr, torch.bfloat16).data_ptr(), T, W, experts, top, 1, ids.data_ptr(),
                                      wts.data_ptr(), None))
    sync()
    want_ids, want_w = O.route_sigmoid(x.double(), wr, top)
    assert ids.cpu().tolist() == want_ids
    assert torch.allclose(wts.cpu().double(), torch.tensor(want_w, dtype=torch.float64), atol=1e-6)
    assert (wts.sum(-1) > 1.0).any() or top == 1        # the weights are the scores themselves, not shares of one


@pytest.mark.parametrize("f32", [1, 0])
@pytest.mark.parametrize("T,W,ff,experts,top", [(5, 72, 40, 6, 2), (150, 96, 24, 4, 3), (70, 64, 130, 3, 1), (260, 100, 36, 5, 2),
                                                (1, 64, 64, 8, 2), (700, 128, 72, 3, 1), (3000, 64, 64, 4, 3)])
def test_ungated_experts_with_the_weight_on_their_input(f32, T, W, ff, experts, top):
    """The CUDA-core token and grouped forms (32-bit mode; sizes no vector access fits) and the grouped tensor-core form (bf16
    with width and ff multiples of 8: every token-tile size, experts nobody chose)."""
    g = torch.Generator().manual_seed(T + ff)
    adt = torch.float32 if f32 else torch.bfloat16
    x = torch.randn(T, W, generator=g).to(adt).float()
    up = U.bf16_exact(torch.randn(experts, ff, W, generator=g) * W ** -0.5)
    down = U.bf16_exact(torch.randn(experts, W, ff, generator=g) * ff ** -0.5)
    ids = torch.stack([torch.randperm(experts, generator=g)[:top] for _ in range(T)]).to(torch.int32)
    wts = torch.rand(T, top, generator=g) * 0.9 + 0.05      # NOT a factor of the output: relu(w z)^2 = w^2 relu(z)^2
    if top == 1:
        ids[ids == experts - 1] = 0        # the last expert gets no token
    want = torch.stack([torch.stack([O.relu2_expert(wts[t, k].double() * x[t].double(), up[ids[t, k]], down[ids[t, k]]) for k in range(top)])
                        for t in range(T)])
    ws = torch.zeros(int(lib().b200_moe_workspace_bytes(T, top, experts, W, ff)), dtype=torch.uint8, device=DEV)
    parts = torch.full((T, top, W), float("nan"), device=DEV)
    check(lib().b200_moe_experts_form(f32, dev(x, adt).data_ptr(), dev(up, torch.bfloat16).data_ptr(), dev(down, torch.bfloat16).data_ptr(),
                                      dev(ids).data_ptr(), dev(wts).data_ptr(), T, W, ff, experts, top, parts.data_ptr(), ws.data_ptr(), 0, 2, 1,
                                      None))
    sync()
    assert torch.isfinite(parts).all()
    assert torch.allclose(parts.cpu().double(), want, atol=2e-5 if f32 else 3e-2, rtol=1e-5 if f32 else 3e-2)


@pytest.mark.parametrize("f32", [1, 0])
def test_feed_forward_activations(f32):
    g = torch.Generator().manual_seed(3)
    adt = torch.float32 if f32 else torch.bfloat16
    T, ff = 9, 50
    gu = (torch.randn(T, 2 * ff, generator=g) * 2).to(adt).float()
    out = torch.zeros(T, ff, dtype=adt, device=DEV)
    check(lib().b200_ff_act(f32, dev(gu, adt).data_ptr(), out.data_ptr(), T, ff, 1, 1, None))
    sync()
    tol = dict(atol=1e-5) if f32 else dict(atol=2e-2, rtol=1e-2)
    assert torch.allclose(out.float().cpu().double(), O.gelu_tanh(gu[:, :ff].double()) * gu[:, ff:].double(), **tol)
    d = dev(gu[:, :ff].contiguous(), adt)
    check(lib().b200_ff_act(f32, d.data_ptr(), d.data_ptr(), T, ff, 0, 2, None))
    sync()
    assert torch.allclose(d.float().cpu().double(), torch.relu(gu[:, :ff].double()) ** 2, **tol)


# ---- whole models ----------------------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def model_a():
    cfg = D.make_cfg()
    return cfg, D.make_weights(cfg, 1)


ALONE = {
    "recurrence alone": [D.mlstm()],
    "latent attention alone": [D.latent()],
    "latent attention with sink and gate, part of the rotated dimensions turning": [D.latent(second=True, rot_dim=24, rot_dims=8)],
    "dense feed-forward": [D.latent(heads=1, dim=8, rot_dim=4, vdim=8, kv_rank=12, mlp=D.dense(ff=50))],
    "experts, two per token, no shared one": [D.mlstm(heads=1, dim=8, vdim=8, mlp=D.moe(experts=7, top=2, ff=20, shared=0))],
}


@pytest.mark.parametrize("which", list(ALONE))
def test_one_layer_models_and_their_streams_fp32(which):
    cfg = D.make_cfg(width=72, layers=ALONE[which], taps=2, buckets=11)
    w = D.make_weights(cfg, 4)
    ids = _prompt(cfg, 50, 1)
    r = D.make_runner(cfg, w, "float32")
    tap = r.set_stream_tap(True)
    got = U.replay(U.make_engine(r), [[("p", 50)]], {"p": ids})["p"]
    streams = []
    want = O.forward(cfg, w, ids, streams=streams).numpy()
    assert U.rel_rms(got, want).max() < F32_TOL
    t = tap[:50 * cfg["width"]].view(50, cfg["width"]).cpu().double()
    assert torch.allclose(t, streams[0], atol=1e-4, rtol=1e-5)
    r.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("variant", ["odd sizes", "one tap, no shared expert, uncapped", "no rotated part, every expert chosen"])
def test_other_sizes_and_constants(dtype, variant):
    """Widths and head sizes no vector access or TMA box fits, a convolution of one tap, logits without a cap, a first layer
    that is a recurrence and a last one without a feed-forward."""
    if variant == "odd sizes":
        cfg = D.make_cfg(width=100, vocab=131, taps=3, buckets=50, mul_prev=7, mul_cur=3, layers=[
            D.mlstm(heads=1, dim=34, vdim=50, mlp=D.dense(ff=44)), D.latent(heads=5, dim=10, rot_dim=6, rot_dims=2, vdim=14, kv_rank=18, mlp=D.moe(experts=3, top=3, ff=20, shared=12)),
            D.latent(second=True, heads=1, dim=130, rot_dim=2, vdim=6, kv_rank=22)])
    elif variant.startswith("one tap"):
        cfg = D.make_cfg(width=64, taps=1, softcap=0.0, layers=[D.latent(second=True, mlp=D.moe(experts=4, top=2, ff=32, shared=0)), D.mlstm(mlp=D.dense(ff=64))])
    else:      # keys without a rotated part (tensor-core shapes: rows of 32 and 48), eight taps, a router that keeps all experts
        cfg = D.make_cfg(width=128, taps=8, buckets=1, layers=[
            D.latent(heads=4, dim=16, rot_dim=0, rot_dims=0, vdim=8, kv_rank=32, mlp=D.moe(experts=3, top=3, ff=16, shared=8)),
            D.latent(second=True, heads=17, dim=8, rot_dim=16, rot_dims=16, vdim=8, kv_rank=32)])
    w = D.make_weights(cfg, 6)
    ids = _prompt(cfg, 45, 2)
    want = O.forward(cfg, w, ids).numpy()
    r = D.make_runner(cfg, w, dtype)
    eng = U.make_engine(r)
    whole = U.replay(eng, [[("p", 45)]], {"p": ids})["p"]
    cut = U.replay(eng, [[("p", n)] for n in (2, 7, 1, 1, 16, 2, 16)], {"p": ids})["p"]
    if dtype == "float32":
        assert U.rel_rms(whole, want).max() < F32_TOL and U.rel_rms(cut, want).max() < F32_TOL
    else:
        e = U.rel_rms(whole, want)
        assert np.median(e) < 0.03 and (e < 0.15).mean() > 0.9, (float(np.median(e)), float(e.max()))
        d = U.rel_rms(cut, whole)
        assert np.median(d) < 0.02 and (d < 0.15).mean() > 0.9, (float(np.median(d)), float(d.max()))
    r.close()


def test_every_schedule_gives_the_oracles_logits_fp32(model_a):
    """Prefill against token-by-token decoding, portions down to two tokens, unequal requests batched, a long decode tail,
    blocks and state slots that are freed and taken again (12 blocks of 16 where the four requests need 22; four slots for
    the requests of all schedules)."""
    cfg, w = model_a
    prompts = {"a": _prompt(cfg, 70, 2), "b": _prompt(cfg, 37, 3), "c": _prompt(cfg, 3, 4), "d": _prompt(cfg, 90, 5)}
    want = {n: O.forward(cfg, w, p).numpy() for n, p in prompts.items()}
    r = D.make_runner(cfg, w, "float32", n_blocks=12, max_tokens=128)
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


def test_graph_replay_gives_the_same_logits_as_eager_steps(model_a):
    """Steps of equal shape replay one captured graph: sequence bounds, slots and positions must come from the step's device
    metadata, not from what was captured."""
    cfg, w = model_a
    prompts = {"a": _prompt(cfg, 40, 7), "b": _prompt(cfg, 40, 8)}
    sched = [[("a", 8), ("b", 8)]] * 3 + [[("a", 1), ("b", 1)]] * 16
    out = []
    for graphs in (False, True):
        r = D.make_runner(cfg, w, "float32", graphs=graphs)
        out.append(U.replay(U.make_engine(r), sched, prompts))
        r.close()
    for n in prompts:
        assert np.array_equal(out[0][n], out[1][n]), n


def test_bf16_mode_within_bf16_noise_and_equal_across_schedules(model_a):
    cfg, w = model_a
    prompts = {"a": _prompt(cfg, 70, 2), "b": _prompt(cfg, 37, 3)}
    want = {n: O.forward(cfg, w, p).numpy() for n, p in prompts.items()}
    r = D.make_runner(cfg, w, "bfloat16", n_blocks=12, max_tokens=128)
    eng = U.make_engine(r)
    whole = U.replay(eng, [[("a", 70)], [("b", 37)]], prompts)
    mixed = U.replay(eng, [[("a", 40), ("b", 2)], [("b", 20), ("a", 1)]] + [[("a", 1), ("b", 1)]] * 15 + [[("a", 14)]], prompts)
    for n in prompts:
        e = U.rel_rms(whole[n], want[n])
        assert np.median(e) < 0.03 and (e < 0.1).mean() > 0.9, (n, float(np.median(e)), float(e.max()))
        d = U.rel_rms(mixed[n], whole[n])
        assert np.median(d) < 0.02 and (d < 0.1).mean() > 0.9, (n, float(np.median(d)), float(d.max()))
    r.close()


def test_greedy_generation_through_the_engines_own_scheduler(model_a, tmp_path):
    """A checkpoint directory goes through the registry, the weight loader, LLMEngine.generate and the scheduler (which hands
    out blocks and state slots and overlaps steps); three prompts of unequal length decode side by side."""
    cfg, w = model_a
    path = str(tmp_path / "ckpt")
    U.write_checkpoint(path, cfg, w)
    pc = pkg("config").load_model_config(path)
    assert type(pc).__name__ == "DupolornConfig"
    r = pkg("runner").make_runner(pc, dtype="float32", max_tokens=64, max_model_len=256, block_size=16, n_blocks=40, n_state_slots=4)
    r.load_weights(pkg("weights").load_safetensors_dir(path))
    eng = pkg("engine").LLMEngine(r, max_num_batched_tokens=64, max_num_seqs=8, max_model_len=256)
    assert eng.scheduler.max_seqs == 3          # bounded by the state slots
    prompts = [_prompt(cfg, 21, 11), _prompt(cfg, 5, 12), _prompt(cfg, 70, 13), _prompt(cfg, 9, 14)]
    got = eng.generate(prompts, max_tokens=12)
    for p, out in zip(prompts, got):
        ids = list(p)
        for tok in out:      # every emitted token is the oracle's arg-max, or within fp32 noise of it
            z = O.forward(cfg, w, ids)[-1]
            assert tok == int(z.argmax()) or float(z.max() - z[tok]) < 1e-3 * float(z.abs().max())
            ids.append(tok)
    r.close()
