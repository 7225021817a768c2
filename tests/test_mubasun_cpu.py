"""Host-side pieces of the Mubasun path that need no GPU: configuration reader, model registry, safetensors
reader / writer, the ragged scheduler's bookkeeping over the slot cache (with a stand-in engine), and the oracle's
own consistency (a prompt run whole equals the same prompt run in portions or token by token)."""
import json

import pytest
import torch

import mubasun_oracle as O
from pg_b200.checkpoint import read_safetensors, write_safetensors
from pg_b200.mubasun import MubasunConfig, distance_slopes
from pg_b200.pool import PagePool
from pg_b200 import registry, scheduler


def test_config_reader_takes_every_size_from_the_dictionary():
    cfg = O.make_config(width=40, groups=5, vocab=77, max_positions=99, eps=3e-4, layers=[
        O.layer(O.attn(heads=6, kv_heads=3, dim=8, vdim=24, window=17, scale=0.5), O.moe(experts=3, identity=2, top=3, ff=16, shared=8)),
        O.layer(O.attn(heads=6, kv_heads=3, dim=8, vdim=24, window=0, kv_from=0), O.dense(12)),
        O.layer(O.attn(heads=2, kv_heads=2, dim=4, vdim=4), None)])
    c = MubasunConfig.from_dict(cfg)
    assert (c.vocab, c.width, c.max_positions, c.eps, c.groups) == (77, 40, 99, 3e-4, 5)
    m0, m1 = c.layers[0].mixer, c.layers[1].mixer
    assert (m0.heads, m0.kv_heads, m0.dim, m0.vdim, m0.window, m0.scale, m0.kv_from) == (6, 3, 8, 24, 17, 0.5, None)
    assert m1.kv_from == 0 and m1.window == 0
    f0 = c.layers[0].mlp
    assert (f0.kind, f0.experts, f0.identity, f0.top, f0.ff, f0.shared_ff, f0.router_scale) == ("moe", 3, 2, 3, 16, 8, 1.5)
    assert c.layers[1].mlp.kind == "dense" and c.layers[1].mlp.ff == 12 and c.layers[2].mlp is None


@pytest.mark.parametrize("bad", ["forward_ref", "chained_ref", "shape", "heads", "kind"])
def test_config_reader_rejects_what_the_design_does_not_have(bad):
    layers = [O.layer(O.attn(), O.dense()), O.layer(O.attn(kv_from=0), None), O.layer(O.attn(), None)]
    if bad == "forward_ref":
        layers[0]["mixer"]["kv_from"] = 2
    elif bad == "chained_ref":
        layers[2]["mixer"]["kv_from"] = 1
    elif bad == "shape":
        layers[1]["mixer"]["vdim"] = 8
    elif bad == "heads":
        layers[2]["mixer"]["kv_heads"] = 3
    else:
        layers[0]["mlp"] = {"kind": "conv"}
    with pytest.raises((ValueError, KeyError)):
        MubasunConfig.from_dict(O.make_config(layers=layers))


def test_slopes():
    assert distance_slopes(8).tolist() == pytest.approx([2.0 ** (-(h + 1)) for h in range(8)])
    assert distance_slopes(3).tolist() == pytest.approx([2.0 ** (-8 * (h + 1) / 3) for h in range(3)])


def test_registry_picks_the_engine_by_config():
    from pg_b200.engine import PaliGemmaEngine
    from pg_b200.mubasun import MubasunEngine
    assert registry.resolve({"architecture": "Mubasun"}) is MubasunEngine
    assert registry.resolve({"vision_config": {}, "text_config": {}}) is PaliGemmaEngine
    assert "Mubasun" in registry.architectures()
    with pytest.raises(ValueError):
        registry.resolve({"architecture": "nothing of the kind"})


def test_safetensors_round_trip(tmp_path):
    t = {"a.b": torch.randn(3, 5).to(torch.bfloat16), "n": torch.arange(7, dtype=torch.int32), "f": torch.randn(2, 2, 2),
         "empty": torch.zeros(0, 4)}
    path = str(tmp_path / "m.safetensors")
    write_safetensors(path, t)
    back = read_safetensors(path)
    assert set(back) == set(t)
    for k in t:
        assert back[k].dtype == t[k].dtype and back[k].shape == t[k].shape and torch.equal(back[k], t[k])
    with open(path, "rb") as f:                      # the layout itself: length, JSON, data
        n = int.from_bytes(f.read(8), "little")
        hdr = json.loads(f.read(n))
    assert hdr["n"] == {"dtype": "I32", "shape": [7], "data_offsets": hdr["n"]["data_offsets"]}


class _Engine(PagePool):
    """Stand-in with the engine's interface: logits row = (slot's sequence length so far, position, token)."""

    class cfg:
        max_positions = 1000
        vocab = 8

    def __init__(self, pages, page_size=4):
        self.page_size, self.device = page_size, torch.device("cpu")
        self._init_pool(pages)
        self.calls = []

    def forward_tokens(self, kv, ids, slots, positions, rows, layer_sink=None):
        table = kv.page_table
        for s, p in zip(slots, positions):                      # every position has a page of its own sequence
            assert int(table[s, p // self.page_size]) in kv.pages[s]
        self.calls.append((list(ids), list(slots), list(positions), list(rows)))
        out = torch.zeros(len(rows), self.cfg.vocab)
        for i, r in enumerate(rows):
            out[i, (ids[r] + 1) % self.cfg.vocab] = 1.0         # "next token" = id + 1
        return out

    def check_errors(self, sync=False):
        pass


def test_ragged_batcher_positions_slots_and_page_reuse():
    eng = _Engine(pages=7)                                       # 6 usable pages of 4 tokens + the parking page
    b = scheduler.RaggedBatcher(eng, slots=2)
    assert len(eng._free) == 6
    b.admit("a"), b.admit("b")
    with pytest.raises(RuntimeError):
        b.admit("c")
    b.run_entries([("a", [1, 2, 3, 4, 5], [4]), ("b", [6], [0])])
    ids, slots, pos, rows = eng.calls[-1]
    assert (slots, pos, rows) == ([0] * 5 + [1], [0, 1, 2, 3, 4, 0], [4, 5])
    b.run_entries([("b", [7, 7], []), ("a", [1], [0])])
    assert eng.calls[-1][1:] == ([1, 1, 0], [1, 2, 5], [2])
    assert len(eng._free) == 6 - 2 - 1
    pages_a = list(b.kv.pages[0])
    b.finish("a")
    assert len(eng._free) == 5 and "a" not in b.slot_of
    b.admit("c")                                                  # takes a's slot and, first of all, a's pages
    b.run_entries([("c", list(range(8)), [7])])
    assert b.slot_of["c"] == 0 and set(b.kv.pages[0]) == set(pages_a)
    assert eng.calls[-1][2] == list(range(8))
    b.finish("b"), b.finish("c")
    assert sorted(eng._free) == [p for p in range(7) if p != b.kv.parking]
    b.close()
    assert sorted(eng._free) == list(range(7))


def test_ragged_batcher_generation_chunks_prompts_and_mixes_decode(monkeypatch):
    from pg_b200 import generate
    monkeypatch.setattr(generate, "_pick", lambda eng, logits, sample, step: logits.argmax(-1))
    eng = _Engine(pages=40)
    b = scheduler.RaggedBatcher(eng, slots=2, token_budget=4)
    r0 = b.submit([1, 2, 3, 4, 5, 6], 3)                        # read in portions of <= 4 tokens
    r1 = b.submit([5], 2)
    r2 = b.submit([2, 2], 2, eos_token_id=3)                     # waits for a slot; stops at its first token
    done = b.run()
    assert done[r0].tokens == [7, 0, 1] and done[r1].tokens == [6, 7] and done[r2].tokens == [3]
    first = eng.calls[0]
    assert first[0] == [1, 2, 3, 4] and first[3] == []          # budget: only a portion of the first prompt
    mixed = [c for c in eng.calls if len(set(c[1])) == 2]
    assert mixed and any(len(c[0]) > 2 for c in mixed)           # a prompt portion beside a decode token
    assert sorted(eng._free) == [p for p in range(40) if p != b.kv.parking]
    with pytest.raises(ValueError):
        b.submit([1] * 2000, 5)
    b.close()


def test_oracle_portions_equal_the_whole_prompt():
    cfg = O.make_config(layers=[O.layer(O.attn(window=6), O.moe()), O.layer(O.attn(window=6, kv_from=0), O.dense())])
    orc = O.Oracle(cfg, O.make_checkpoint(cfg, 3))
    toks = torch.randint(0, cfg["vocab"], (20,), generator=torch.Generator().manual_seed(0)).tolist()
    whole = orc.logits(toks)
    cache, parts, at = orc.new_cache(), [], 0
    for n in (1, 2, 5, 1, 11):
        parts.append(orc.run(toks[at:at + n], cache, at))
        at += n
    assert torch.allclose(torch.cat(parts), whole, atol=1e-10)
    # a key just outside the window has no influence at all, one just inside has
    other = list(toks)
    other[10] = (other[10] + 1) % cfg["vocab"]
    lg = orc.logits(other)
    assert torch.equal(lg[:10], whole[:10]) and not torch.allclose(lg[15], whole[15], atol=1e-9)
