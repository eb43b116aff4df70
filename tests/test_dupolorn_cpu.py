"""Host side of the Dupolorn design: registry and configuration reader, weight mapping, the scheduler's state slots, and the
float64 oracle's own invariants (what the GPU tests then hold the kernels to)."""
import json

import numpy as np
import pytest
import torch

import dupolorn_util as D
import stack_util as U
from conftest import pkg
from oracle import dupolorn_oracle as O


def _ids(cfg, n, seed):
    return torch.randint(0, cfg["vocab"], (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def test_registry_reads_every_part_of_the_configuration(tmp_path):
    cfg = D.make_cfg()
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    c = pkg("config").load_model_config(str(tmp_path))
    C = pkg("config")
    assert isinstance(c, C.DupolornConfig) and C.is_stack_config(c)
    assert (c.width, c.vocab, c.canon_taps, c.bigram_buckets, c.bigram_mul_prev, c.bigram_mul_cur) == (96, 150, 4, 97, 31, 5)
    assert c.logit_softcap == 20.0 and c.embed_scale == 3.0 and c.norm_eps == 1e-5 and c.needs_state
    kinds = [type(L.mixer).__name__ for L in c.layers]
    assert kinds == ["MLSTMSpec", "LatentAttentionSpec", "LatentAttentionSpec", "MLSTMSpec"]
    a, b = c.layers[1].mixer, c.layers[2].mixer
    assert (a.sink, a.gate, b.sink, b.gate) == (False, False, True, True)
    assert b.rot.dims == 16 and b.rot_dim == 24                 # fewer dimensions turn than the rotated part has
    assert c.layers[0].mlp.kind == "moe" and c.layers[0].mlp.shared_ff == 56 and c.layers[2].mlp.shared_ff == 0
    assert c.layers[1].mlp.kind == "dense" and c.layers[3].mlp is None
    assert c.kv_bytes_per_token() == 2 * ((40 + 16) + (28 + 24))
    with pytest.raises(ValueError):
        C.DupolornConfig.from_dict(dict(cfg, layers=[{"type": "window_attention", "mixer": {}}]))
    with pytest.raises(ValueError):
        bad = dict(cfg, architecture="Nopelorn")
        (tmp_path / "config.json").write_text(json.dumps(bad))
        C.load_model_config(str(tmp_path))


def test_weight_mapping_fuses_projections_and_transposes_the_key_expansion():
    cfg = D.make_cfg()
    w = D.make_weights(cfg, 2)
    pc = D.product_config(cfg)
    A = pkg("_abi")
    out = {}
    for layer, kind, t in pkg("weights").dupolorn_weights(w, pc):
        out[(layer, kind)] = t
    assert out[(0, A.SW_FINAL_NORM)].shape == (1,) and out[(0, A.SW_BIGRAM)].shape == (98, 96)
    m = cfg["layers"][0]["mixer"]
    assert out[(0, A.SW_QKV)].shape == (2 * m["heads"] * m["dim"] + 2 * m["heads"] * m["vdim"], 96)
    assert out[(0, A.SW_GATES)].shape == (2 * m["heads"], 96) and out[(0, A.SW_GATES_BIAS)].shape == (2 * m["heads"],)
    assert torch.equal(out[(0, A.SW_GATES)][m["heads"]:], w["l0.mix.f"])
    m1 = cfg["layers"][1]["mixer"]
    assert out[(1, A.SW_QKV)].shape == (m1["heads"] * (m1["dim"] + m1["rot_dim"]) + m1["kv_rank"] + m1["rot_dim"], 96)
    ukt = out[(1, A.SW_UK_T)].reshape(m1["heads"], m1["kv_rank"], m1["dim"])
    uk = w["l1.mix.uk"].reshape(m1["heads"], m1["dim"], m1["kv_rank"])
    assert torch.equal(ukt[2], uk[2].T)
    m2 = cfg["layers"][2]["mixer"]
    assert out[(2, A.SW_QKV)].shape[0] == m2["heads"] * (m2["dim"] + m2["rot_dim"]) + m2["kv_rank"] + m2["rot_dim"] + m2["heads"] * m2["vdim"]
    assert (2, A.SW_SINK) in out and (1, A.SW_SINK) not in out
    assert out[(0, A.SW_EXPERT_GATE_UP)].shape == (6 * 40, 96) and out[(0, A.SW_EXPERT_DOWN)].shape == (6 * 96, 40)
    assert (0, A.SW_SHARED_UP) in out and (2, A.SW_SHARED_UP) not in out and (3, A.SW_NORM_MLP_PRE) not in out
    assert out[(3, A.SW_DEPTH_AVG)].shape == (5,) and out[(1, A.SW_CANON)].shape == (96, 4)


class _FakeRunner:
    """What the engine needs of a runner: sizes, and a step that records the batch."""
    def __init__(self, slots):
        self.n_blocks, self.block_size, self.max_tokens, self.max_model_len, self.n_state_slots = 16, 16, 64, 256, slots
        self.batches = []

    def step(self, b):
        self.batches.append(b)
        return np.zeros(len(b.logit_rows), dtype=np.int32)


def test_scheduler_hands_state_slots_out_and_takes_them_back():
    E = pkg("engine")
    r = _FakeRunner(slots=4)
    eng = E.LLMEngine(r, max_num_batched_tokens=64, max_num_seqs=16, max_model_len=256)
    assert eng.scheduler.max_seqs == 3                              # one slot per scheduler row
    reqs = {n: E.Request(n, [1, 2, 3, 4, 5], max_tokens=0) for n in "abcd"}
    for n in "abc":
        eng.add_request(reqs[n])
    eng.step_given([(reqs["a"], 2, [1]), (reqs["b"], 5, []), (reqs["c"], 1, [0])])
    b = r.batches[-1]
    assert len(b.seq_slots) == 3 and len(set(b.seq_slots)) == 3 and all(0 <= s < 4 for s in b.seq_slots)
    assert list(b.seq_slots) == [reqs[n].row for n in "abc"]
    slot_b = reqs["b"].row
    eng.add_request(reqs["d"])
    with pytest.raises(ValueError):                                 # a fourth live sequence has no slot
        eng.step_given([(reqs["d"], 1, [0])])
    eng.abort_request("b")
    eng.step_given([(reqs["a"], 3, [2]), (reqs["d"], 2, [])])
    b = r.batches[-1]
    assert list(b.seq_slots) == [reqs["a"].row, reqs["d"].row] and reqs["d"].row == slot_b       # the freed slot is used again
    assert list(b.positions) == [2, 3, 4, 0, 1]
    # the decode fast path names the slots too
    for n in "ad":
        reqs[n].max_tokens = 4
    reqs["d"].n_computed = 5
    eng.scheduler.running = [reqs["a"], reqs["d"]]
    reqs["a"].output_ids.append(7), reqs["d"].output_ids.append(8)
    sched = [E.Scheduled(reqs["a"], 1, True), E.Scheduled(reqs["d"], 1, True)]
    fb = eng.scheduler.build_batch(sched)
    assert list(fb.seq_slots) == [reqs["a"].row, reqs["d"].row]


def test_packed_step_buffer_carries_the_slots_behind_the_block_tables():
    R = pkg("runner")
    fake = R.StackRunner.__new__(R.StackRunner)
    fake.n_state_slots = 3
    buf = np.zeros(64, dtype=np.int32)
    b = R.StepBatch(ids=[5, 6, 7], positions=[0, 1, 9], slots=[16, 17, 41], ctx_lens=[1, 2, 10], row_to_seq=[0, 0, 1], logit_rows=[1, 2],
                    block_tables=[[1], [2, 4]], seq_slots=[2, 0])
    T, Rr, S, stride, n = fake.pack(b, buf)
    assert (T, Rr, S, stride) == (3, 2, 2, 2) and n == 5 * 3 + 2 + 2 * 2 + 2
    assert list(buf[17:21]) == [1, 0, 2, 4] and list(buf[21:23]) == [2, 0]
    b.seq_slots = [2]
    with pytest.raises(ValueError):
        fake.pack(b, buf)


# ---- the oracle's own invariants ----------------------------------------------------------------------------------------------
def test_oracle_is_causal_and_its_first_token_uses_the_spare_bigram_row():
    cfg = D.make_cfg()
    w = D.make_weights(cfg, 3)
    ids = _ids(cfg, 30, 1)
    full = O.forward(cfg, w, ids)
    assert torch.allclose(O.forward(cfg, w, ids[:17]), full[:17], atol=1e-9)
    w2 = dict(w)
    w2["bigram"] = w["bigram"].clone()
    w2["bigram"][-1] += 1.0
    moved = O.forward(cfg, w2, ids)
    assert not torch.allclose(moved[0], full[0], atol=1e-3)        # position 0 reads the last row ...
    x0 = O.embed_tokens(ids, w["embed"], 3.0, w["bigram"], 97, 31, 5)
    x1 = O.embed_tokens(ids, w2["embed"], 3.0, w2["bigram"], 97, 31, 5)
    assert torch.equal(x0[1:], x1[1:])                             # ... and no other position does
    assert full.abs().max() <= 20.0                                # the cap


def test_oracle_recurrence_carries_its_state_and_convolution_its_tail():
    g = torch.Generator().manual_seed(0)
    m = {"heads": 2, "dim": 12, "vdim": 10, "gate_cap": 8.0}
    W = 24
    w = {k: torch.randn(n, W, generator=g) * 0.3 for k, n in (("q", 24), ("k", 24), ("v", 20), ("g", 20), ("i", 2), ("f", 2))}
    w.update({"i.b": torch.zeros(2), "f.b": torch.ones(2), "norm": torch.ones(20), "o": torch.eye(20)})
    x = torch.randn(40, W, generator=g, dtype=torch.float64)
    whole = O.mlstm(x, m, w, "", 1e-6)
    st = {}
    parts = torch.cat([O.mlstm(x[a:b], m, w, "", 1e-6, st) for a, b in ((0, 1), (1, 3), (3, 24), (24, 40))])
    assert torch.allclose(parts, whole, atol=1e-10)
    assert float(st["m"].min()) > -8.0 - 1e-9                      # the running maximum never falls below -cap
    cw = torch.randn(W, 3, generator=g)
    y = O.causal_conv(x, cw)
    assert torch.allclose(y[0], cw[:, 2].double() * x[0]) and torch.allclose(y[5], cw[:, 0].double() * x[3] + cw[:, 1].double() * x[4] + cw[:, 2].double() * x[5])


def test_oracle_attention_sink_takes_weight_and_rotation_depends_on_distance_only():
    cfg = D.make_cfg(layers=[D.latent(second=True)])
    w = D.make_weights(cfg, 5)
    m = cfg["layers"][0]["mixer"]
    g = torch.Generator().manual_seed(1)
    h = torch.randn(12, 96, generator=g, dtype=torch.float64)
    a = O.latent_attention(h, m, w, "l0.mix.", 1e-5, sink=True, gate=False)
    w2 = dict(w)
    w2["l0.mix.sink"] = w["l0.mix.sink"] + 30.0                    # a huge sink swallows the whole softmax
    b = O.latent_attention(h, m, w2, "l0.mix.", 1e-5, sink=True, gate=False)
    assert b.abs().max() < 1e-6 * a.abs().max()
    q = torch.randn(16, generator=g, dtype=torch.float64)
    k = torch.randn(16, generator=g, dtype=torch.float64)
    d1 = O.rotate_pairs(q, 9, 5000.0, 16) @ O.rotate_pairs(k, 4, 5000.0, 16)
    d2 = O.rotate_pairs(q, 105, 5000.0, 16) @ O.rotate_pairs(k, 100, 5000.0, 16)
    assert abs(float(d1 - d2)) < 1e-9
    part = O.rotate_pairs(q, 9, 5000.0, 8)
    assert torch.equal(part[8:], q[8:]) and not torch.allclose(part[:8], q[:8])


def test_oracle_experts_weight_scales_the_input():
    g = torch.Generator().manual_seed(2)
    h = torch.randn(4, 10, generator=g, dtype=torch.float64)
    up, down = torch.randn(6, 10, generator=g), torch.randn(10, 6, generator=g)
    assert torch.allclose(O.relu2_expert(0.5 * h, up, down), 0.25 * O.relu2_expert(h, up, down))
    ids, wts = O.route_sigmoid(h, torch.randn(5, 10, generator=g), 2)
    assert all(len(set(r)) == 2 for r in ids) and all(0 < x < 1 for r in wts for x in r) and all(r[0] >= r[1] for r in wts)
