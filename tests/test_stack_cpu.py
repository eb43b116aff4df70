"""Host-side pieces of layer-list models: config.json reading and the model registry, rotation tables against the oracle's
frequencies, checkpoint-name mapping, the externally scheduled engine step, and the oracle's own consistency."""
import numpy as np
import pytest
import torch

import stack_util as U
from conftest import pkg
from oracle import stack_oracle as SO


def test_registry_picks_the_class_by_config_json(tmp_path):
    C = pkg("config")
    cfg = U.make_cfg()
    U.write_checkpoint(str(tmp_path / "m"), cfg, U.make_weights(cfg))
    pc = C.load_model_config(str(tmp_path / "m"))
    assert isinstance(pc, C.BopilornConfig) and C.is_stack_config(pc)
    assert pc.n_layers == 2 and pc.width == 96 and pc.vocab == 200 and pc.embed_scale == 2.0
    a0, a1 = pc.layers[0].mixer, pc.layers[1].mixer
    assert (a0.heads, a0.kv_heads, a0.dim, a0.vdim, a0.rot.dims, a0.rot.scaled) == (4, 1, 48, 32, 48, True)
    assert (a1.kv_heads, a1.rot.dims, a1.rot.scaled, a1.value_rot.dims) == (2, 16, False, 48)
    assert (pc.layers[1].mlp.experts, pc.layers[1].mlp.top, pc.layers[1].mlp.groups, pc.layers[1].mlp.keep) == (6, 2, 3, 2)
    (tmp_path / "bad").mkdir()
    (tmp_path / "bad" / "config.json").write_text('{"architecture": "Nonesuch"}')
    with pytest.raises(ValueError):
        C.load_model_config(str(tmp_path / "bad"))


def test_optional_parts_of_the_config():
    C = pkg("config")
    cfg = U.make_cfg(layers=[U.layer(moe=None), U.layer(scaling=None, moe=dict(experts=4, top=1, groups=1, keep=1, ff=8))])
    del cfg["layers"][1]["mlp"]["router"]["groups"]
    pc = C.BopilornConfig.from_dict(cfg)
    assert pc.layers[0].mlp is None
    assert (pc.layers[1].mlp.groups, pc.layers[1].mlp.keep) == (1, 1)
    assert not pc.layers[1].mixer.rot.scaled


@pytest.mark.parametrize("scaling", [None, dict(factor=8.0, original=128, fast=32.0, slow=1.0), dict(factor=2.0, original=4096, fast=4.0, slow=2.0)])
@pytest.mark.parametrize("dims,base", [(64, 50000.0), (16, 100.0), (2, 10000.0)])
def test_rotation_table_matches_the_oracle(scaling, dims, base):
    C = pkg("config")
    spec = C.RotarySpec(base=base, dims=dims, **(dict(scaled=True, **scaling) if scaling else {}))
    f, mag = SO.rotary_frequencies(base, dims, scaling)
    t = spec.table(300)
    assert t.shape == (300, 2, dims // 2) and t.dtype == torch.float32
    ang = torch.arange(300, dtype=torch.float64)[:, None] * f[None]
    assert torch.allclose(t[:, 0].double(), ang.cos() * mag, atol=1e-6)
    assert torch.allclose(t[:, 1].double(), ang.sin() * mag, atol=1e-6)


def test_weight_mapping_shapes_and_order():
    A, Wt = pkg("_abi"), pkg("weights")
    cfg = U.make_cfg()
    w = U.make_weights(cfg)
    items = list(Wt.bopilorn_weights(w, U.product_config(cfg)))
    kinds = {(l, k): t for l, k, t in items}
    m = cfg["layers"][1]["mixer"]
    assert kinds[(1, A.SW_QKV)].shape == (m["heads"] * m["dim"] + m["kv_heads"] * (m["dim"] + m["vdim"]), 96)
    assert torch.equal(kinds[(1, A.SW_QKV)][m["heads"] * m["dim"]:][:m["kv_heads"] * m["dim"]], w["l1.mix.k"])
    gu = kinds[(1, A.SW_EXPERT_GATE_UP)].view(6, 2, 40, 96)
    assert torch.equal(gu[3, 0], w["l1.mlp.e3.gate"]) and torch.equal(gu[3, 1], w["l1.mlp.e3.up"])
    assert torch.equal(kinds[(1, A.SW_EXPERT_DOWN)].view(6, 96, 40)[5], w["l1.mlp.e5.down"])
    assert torch.equal(kinds[(0, A.SW_ROUTER_BIAS)], w["l0.mlp.correction"])


class FakeRunner:
    """Records the batches the engine builds."""
    block_size, n_blocks, max_tokens, max_model_len = 4, 6, 64, 24

    def __init__(self):
        self.batches = []

    def step(self, b):
        self.batches.append(b)
        return np.zeros(len(b.logit_rows), dtype=np.int32)


def test_given_steps_build_the_batch_and_reuse_blocks():
    E = pkg("engine")
    r = FakeRunner()
    eng = E.LLMEngine(r, max_num_batched_tokens=64, max_num_seqs=4, max_model_len=24)
    a = E.Request("a", list(range(10, 17)), max_tokens=0)
    b = E.Request("b", [1, 2], max_tokens=0)
    eng.add_request(a)
    eng.add_request(b)
    assert eng.step_given([(a, 7, [0, 6]), (b, 2, [])]) == 2
    bt = r.batches[-1]
    assert list(bt.ids) == list(range(10, 17)) + [1, 2]
    assert list(bt.positions) == [0, 1, 2, 3, 4, 5, 6, 0, 1] and list(bt.ctx_lens) == [1, 2, 3, 4, 5, 6, 7, 1, 2]
    assert list(bt.logit_rows) == [0, 6] and list(bt.row_to_seq) == [0] * 7 + [1] * 2
    assert len(a.block_table) == 2 and len(b.block_table) == 1 and a.n_computed == 7
    slots_a = [a.block_table[p // 4] * 4 + p % 4 for p in range(7)]
    assert list(bt.slots[:7]) == slots_a
    # a single token of `a` beside a portion of a new request; b is left out of the step
    a.prompt_ids.append(99)
    c = E.Request("c", [5, 6, 7, 8, 9], max_tokens=0)
    eng.add_request(c)
    assert eng.step_given([(c, 5, [4]), (a, 1, [0])]) == 2
    bt = r.batches[-1]
    assert list(bt.positions) == [0, 1, 2, 3, 4, 7] and list(bt.logit_rows) == [4, 5]
    # the pool is 6 blocks: a(2) + b(1) + c(2) leaves one; a step that needs two is refused before taking any
    d = E.Request("d", list(range(8)), max_tokens=0)
    eng.add_request(d)
    free = len(eng.blocks.free)
    with pytest.raises(E.OutOfBlocks):
        eng.step_given([(d, 8, [])])
    assert len(eng.blocks.free) == free
    used = set(a.block_table)
    eng.abort_request("a")
    assert eng.step_given([(d, 8, [7])]) == 1
    assert set(d.block_table) & used          # freed blocks are taken again
    with pytest.raises(ValueError):
        eng.step_given([(d, 1, [])])          # no token left to run


def test_oracle_rows_do_not_depend_on_what_follows():
    cfg = U.make_cfg()
    w = U.make_weights(cfg, seed=3)
    ids = torch.randint(0, cfg["vocab"], (12,), generator=torch.Generator().manual_seed(1)).tolist()
    full = SO.forward(cfg, w, ids)
    part = SO.forward(cfg, w, ids[:7])
    assert torch.allclose(full[:7], part, atol=1e-9)


def test_oracle_router_groups_and_weights():
    h = torch.eye(4, dtype=torch.float64)[:1]
    wr = torch.tensor([[4.0, 0, 0, 0], [3.0, 0, 0, 0], [3.5, 0, 0, 0], [1.0, 0, 0, 0]], dtype=torch.float64)
    s = torch.softmax(wr[:, 0], 0)
    # the bias lifts expert 3 into the choice, yet its weight stays the plain score
    idx, wt = SO.route(h, wr, torch.tensor([0, 0, 0, 10.0], dtype=torch.float64), dict(experts=4, top=2))
    assert idx[0].tolist() == [3, 0] and torch.allclose(wt[0], s[[3, 0]])
    # two groups of two, keep one: group {0, 1} wins on its best member, expert 2 (second best overall) is out
    idx, _ = SO.route(h, wr, None, dict(experts=4, top=2, groups=dict(count=2, keep=1)))
    assert sorted(idx[0].tolist()) == [0, 1]
    # negative choice scores still beat a dropped group
    idx, _ = SO.route(h, wr, torch.tensor([-5.0, -5.0, 0, 0], dtype=torch.float64), dict(experts=4, top=2, groups=dict(count=2, keep=1)))
    assert sorted(idx[0].tolist()) == [2, 3]
