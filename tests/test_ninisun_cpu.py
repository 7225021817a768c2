"""Host-side parts of the Ninisun path that need no GPU: config parsing, the rotary frequency table, the per-step run /
segment lists, the recurrent state slots, and the oracle's own consistency."""
import math

import numpy as np
import pytest
import torch

import ninisun_oracle as O
from pg_b200 import registry, scheduler
from pg_b200.ninisun import NinisunConfig, RotaryCfg
from pg_b200.pool import PagePool
from pg_b200.ragged_engine import RaggedEngine


def test_config_reads_every_size_and_constant():
    cfg = O.make_config(width=40, vocab=77, eps=3e-4, layers=[
        O.layer(O.attn(heads=6, kv_heads=3, dim=10, vdim=4, scale=0.7, rot_dims=6, base=123.0, window=11, keep_first=5), 24),
        O.layer(O.parallel(heads=2, kv_heads=1, dim=8, vdim=12, scale=0.2, rot_dims=4, base=9.0, scaling=(3.0, 50, 7.0, 0.5),
                           r_heads=5, r_dim=6, left_scale=0.25, right_scale=1.5), 0),
        O.layer(O.attn(window=0, rot_dims=0, v_mix=False), 8)])
    c = NinisunConfig.from_dict(cfg)
    assert (c.vocab, c.width, c.eps) == (77, 40, 3e-4)
    a = c.layers[0].attn
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.scale, a.window, a.keep_first, a.v_mix) == (6, 3, 10, 4, 0.7, 11, 5, True)
    assert (a.rot.dims, a.rot.base, a.rot.scaling, a.sigmoid, a.biased) == (6, 123.0, None, False, False)
    p = c.layers[1]
    assert (p.kind, p.delta.heads, p.delta.dim, p.left_scale, p.right_scale, p.ff) == ("parallel", 5, 6, 0.25, 1.5, 0)
    assert p.attn.sigmoid and p.attn.biased and p.attn.rot.scaling["factor"] == 3.0 and p.attn.window == 0
    assert c.layers[2].attn.rot is None and c.layers[2].attn.window == 0 and not c.layers[2].attn.v_mix
    assert registry.resolve(cfg).__name__ == "NinisunEngine"


def test_config_rejects_what_the_design_does_not_have():
    bad = O.make_config(layers=[O.layer(O.attn(heads=5, kv_heads=2))])
    with pytest.raises(ValueError):
        NinisunConfig.from_dict(bad)
    bad = O.make_config(layers=[{"type": "convolution", "mixer": O.attn(), "mlp": None}])
    with pytest.raises(ValueError):
        NinisunConfig.from_dict(bad)
    bad = O.make_config(layers=[O.layer(O.attn(vdim=16)), O.layer(O.attn(vdim=8))])     # mixed values of two widths
    with pytest.raises(ValueError):
        NinisunConfig.from_dict(bad)
    bad = O.make_config(layers=[O.layer(O.attn(dim=8, rot_dims=10))])
    with pytest.raises(ValueError):
        NinisunConfig.from_dict(bad)


@pytest.mark.parametrize("dims,base,scaling", [(8, 10000.0, None), (16, 300000.0, (3.0, 2048, 24.0, 2.0)),
                                               (6, 77.0, (2.5, 100, 8.0, 0.5)), (32, 1e6, (8.0, 4096, 1.0, 1.0))])
def test_rotary_table_matches_the_oracle(dims, base, scaling):
    f, mag = RotaryCfg(dims, base, dict(zip(("factor", "original", "fast", "slow"), scaling)) if scaling else None).table()
    pos = [0, 1, 17, 1000]
    cos, sin = O.rotary_table(O.rot(dims, base, scaling), pos)
    ang = torch.tensor(pos, dtype=torch.float64)[:, None] * f[None, :]
    assert torch.allclose(torch.cos(ang) * mag, cos, atol=1e-12) and torch.allclose(torch.sin(ang) * mag, sin, atol=1e-12)
    if scaling is None:
        assert mag == 1.0 and torch.allclose(f, base ** (-2.0 * torch.arange(dims // 2, dtype=torch.float64) / dims))
    else:
        assert mag == pytest.approx(0.1 * math.log(scaling[0]) + 1.0)
        plain = base ** (-2.0 * torch.arange(dims // 2, dtype=torch.float64) / dims)
        assert bool(((f <= plain + 1e-15) & (f >= plain / scaling[0] - 1e-15)).all())


def test_runs_and_segments_of_a_step():
    slots = np.array([2, 2, 2, 0, 3, 3], dtype=np.int64)
    pos = np.array([5, 6, 7, 0, 9, 10], dtype=np.int64)
    bounds = RaggedEngine._runs(slots, pos)
    assert bounds.tolist() == [0, 3, 4, 6]
    assert RaggedEngine._segments(slots, bounds) == [2, 0, 3, 0, 3, 1, 3, 4, 2]
    with pytest.raises(ValueError):                      # a gap inside one sequence's tokens
        RaggedEngine._segments(np.array([1, 1, 1]), RaggedEngine._runs(np.array([1, 1, 1]), np.array([0, 1, 3])))
    with pytest.raises(ValueError):                      # a sequence whose tokens are not one block of rows
        s2, p2 = np.array([1, 4, 1]), np.array([0, 0, 1])
        RaggedEngine._segments(s2, RaggedEngine._runs(s2, p2))


class _Engine(PagePool):
    """Stand-in with a recurrent state: the "model" adds the fed token ids into its slot's state."""
    max_positions = None

    class cfg:
        vocab = 4

    def __init__(self, pages, page_size=4):
        self.page_size, self.device = page_size, torch.device("cpu")
        self._init_pool(pages)

    def new_slot_state(self, slots):
        return scheduler.SlotState(slots, {1: (2, 3)}, self.device)

    def forward_tokens(self, kv, ids, slots, positions, rows, layer_sink=None):
        for t, s in zip(ids, slots):
            kv.state.layers[1][s] += float(t)
        return torch.zeros(len(rows), self.cfg.vocab)

    def check_errors(self, sync=False):
        pass


def test_state_slots_are_zeroed_for_a_new_sequence_and_kept_between_steps():
    eng = _Engine(pages=9)
    b = scheduler.RaggedBatcher(eng, slots=2)
    st = b.kv.state.layers[1]
    assert st.shape == (2, 2, 3) and b.kv.state.bytes() == 2 * 6 * 4
    b.admit("a"), b.admit("b")
    b.run_entries([("a", [1, 2], []), ("b", [10], [])])
    b.run_entries([("a", [3], [])])                       # a skipped step for b leaves its state alone
    assert float(st[b.slot_of["a"]][0, 0]) == 6.0 and float(st[b.slot_of["b"]][0, 0]) == 10.0
    slot_a = b.slot_of["a"]
    b.finish("a")
    b.admit("c")                                          # takes a's slot: its state starts from zero
    assert b.slot_of["c"] == slot_a and float(st[slot_a].abs().max()) == 0.0 and float(st[b.slot_of["b"]][0, 0]) == 10.0
    b.close()


def test_oracle_recurrence_carries_its_state_and_masks_as_stated():
    g = torch.Generator().manual_seed(4)
    T, N, d = 9, 2, 5
    r, k, v = (torch.randn(T, N, d, generator=g, dtype=torch.float64) for _ in range(3))
    w, a = torch.rand(T, N, d, generator=g, dtype=torch.float64), torch.rand(T, N, d, generator=g, dtype=torch.float64)
    whole, S = O.delta_rule(r, k, v, w, a)
    first, S1 = O.delta_rule(r[:4], k[:4], v[:4], w[:4], a[:4])
    rest, S2 = O.delta_rule(r[4:], k[4:], v[4:], w[4:], a[4:], S1)
    assert torch.allclose(torch.cat([first, rest]), whole) and torch.allclose(S2, S)
    u0 = k[0, 0] / torch.sqrt((k[0, 0] ** 2).sum() + 1e-6)              # first step from the zero state: S = k v^T
    assert torch.allclose(whole[0, 0], v[0, 0] * (k[0, 0] * r[0, 0]).sum()) and u0.norm() < 1.0
    vis = O.visible(12, 4, 2)
    assert vis[11].tolist() == [True, True] + [False] * 6 + [True] * 4 and not bool(torch.triu(vis, 1).any())
    assert O.visible(5, 0, 0).tolist() == torch.tril(torch.ones(5, 5)).bool().tolist()
