"""Host-side pieces of the layer-by-layer family that need no GPU: the configuration reader and registry, the state
slot allocator, the paged cache with per-layer shapes, and the ragged scheduler's planning against a fake engine."""
import pytest
import torch

from dli_b200 import models, sokevik
from dli_b200.batching import RaggedBatcher
from dli_b200.engine import PagedKVCache
from dli_b200.state_cache import StateSlots


def small_config():
    return {"architecture": "Sokevik", "vocab": 31, "width": 24, "norm": {"eps": 1e-5}, "canon": {"taps": 3}, "layers": [
        {"type": "attention", "mlp": {"kind": "dense", "ff": 40},
         "mixer": {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 10, "scale": 0.25, "mask": {"size": 7},
                   "rot": {"base": 77.0, "dims": 4, "scaling": {"factor": 2.0, "low": 1.0, "high": 2.0, "original": 16}}}},
        {"type": "mlstm", "mlp": None, "mixer": {"heads": 2, "dim": 5, "vdim": 12, "gate_cap": 3.0}},
        {"type": "attention", "mlp": {"kind": "dense", "ff": 40}, "weights_of": 0,
         "mixer": {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 10, "scale": 0.25, "mask": {"size": 7},
                   "rot": {"base": 77.0, "dims": 4, "scaling": {"factor": 2.0, "low": 1.0, "high": 2.0, "original": 16}}}}]}


def test_registry_and_config_reader():
    cfg = small_config()
    assert models.family(cfg) == "sokevik"
    assert models.family({"model_type": "llama"}) == "uniform"
    with pytest.raises(ValueError):
        models.family({"model_type": "bert"})
    spec = models.spec_from_config(cfg)
    assert (spec.vocab, spec.width, spec.taps, spec.n_layers) == (31, 24, 3, 3)
    a, r = spec.layers[0].mixer, spec.layers[1].mixer
    assert (a.kind, a.heads, a.kv_heads, a.dim, a.vdim, a.chunk, a.rot_dims, a.scale) == ("attention", 4, 2, 6, 10, 7, 4, 0.25)
    assert a.rot_scaling == {"factor": 2.0, "low": 1.0, "high": 2.0, "original": 16} and a.sink and a.head_gate
    assert (r.kind, r.heads, r.dim, r.vdim, r.gate_cap) == ("mlstm", 2, 5, 12, 3.0)
    assert spec.layers[1].ff == 0 and spec.layers[0].ff == 40
    assert spec.source(2) == 0 and spec.source(1) == 1
    bad = small_config()
    bad["layers"][1]["type"] = "conv"
    with pytest.raises(ValueError):
        models.spec_from_config(bad)


def test_random_state_dict_has_the_checkpoint_names_and_shapes():
    spec = models.spec_from_config(small_config())
    sd = sokevik.random_state_dict(spec, seed=3)
    assert "l2.mix.q" not in sd and "l2.norm1" not in sd            # layer 2 borrows layer 0's tensors
    assert sd["l0.mix.q"].shape == (24, 24) and sd["l0.mix.k"].shape == (12, 24) and sd["l0.mix.v"].shape == (20, 24)
    assert sd["l0.mix.g"].shape == (4, 24) and sd["l0.mix.sink"].shape == (4,) and sd["l0.mix.q.norm"].shape == (6,)
    assert sd["l1.mix.i"].shape == (2, 24) and sd["l1.mix.f.b"].shape == (2,) and sd["l1.mix.norm"].shape == (24,)
    assert sd["l0.canon2"].shape == (24, 3) and "l1.canon2" not in sd and sd["l0.norm2b"].shape == ()
    t = sokevik.model_tensors(spec, sd)
    assert sorted(t["layers"]) == [0, 1] and t["layers"][1]["out_norm"] is sd["l1.mix.norm"]


def test_state_slots_and_paged_cache_shapes():
    s = StateSlots(3, "cpu")
    t = s.add(("S", 0), 2, 4, 5)
    assert t.shape == (3, 2, 4, 5) and t.dtype == torch.float32 and s[("S", 0)] is t
    a, b, c = s.alloc(), s.alloc(), s.alloc()
    assert sorted((a, b, c)) == [0, 1, 2]
    with pytest.raises(RuntimeError):
        s.alloc()
    s.release(b)
    s.release(b)                     # twice is harmless
    assert s.alloc() == b
    kv = PagedKVCache(2, 0, 0, 4, 3, 32, "cpu", pool_tokens=40, layer_shapes=[(2, 6, 10), (1, 8, 8)], dtype=torch.float32)
    assert kv.k[0].shape == (10, 2, 4, 6) and kv.v[0].shape == (10, 2, 4, 10) and kv.v[1].shape == (10, 1, 4, 8)
    assert kv.reserve(1, 9) and kv.capacity(1) == 12 and not kv.reserve(1, 12)
    kv.reserve(0, 28)
    with pytest.raises(RuntimeError):
        kv.reserve(2, 5)
    kv.release(1)
    assert kv.reserve(2, 5)
    legacy = PagedKVCache(2, 2, 8, 4, 1, 16, "cpu")
    assert legacy.k[1].shape == (4, 2, 4, 8) and legacy.k[1].dtype == torch.bfloat16


class FakeEngine:
    """Answers every wanted row with logits whose argmax is (sum of the sequence's tokens so far) % vocab."""
    max_batch, max_seq_len, eos_token_ids, vocab = 2, 64, (), 11

    def __init__(self):
        self.device = torch.device("cpu")
        self.seqs, self.free, self.calls = {}, [1, 0], []

    def open_sequence(self):
        s = self.free.pop()
        self.seqs[s] = []
        return s

    def close_sequence(self, s):
        del self.seqs[s]
        self.free.append(s)

    def step(self, batch, want):
        self.calls.append([(s, len(t)) for s, t in batch])
        rows = []
        for (s, toks), w in zip(batch, want):
            for j, t in enumerate(toks):
                self.seqs[s].append(int(t))
                if j in w:
                    rows.append(sum(self.seqs[s]) % self.vocab)
        return torch.nn.functional.one_hot(torch.tensor(rows, dtype=torch.long), self.vocab).to(torch.bfloat16) * 5


def test_ragged_scheduler_plans_portions_beside_decoding(monkeypatch):
    from dli_b200 import ops
    monkeypatch.setattr(ops, "argmax", lambda logits: logits.float().argmax(-1).to(torch.int32))
    eng = FakeEngine()
    sched = RaggedBatcher(eng, chunk=4)
    prompts = [[1, 2, 3, 4, 5, 6, 7, 8, 9], [3, 3], [5]]
    futs = [sched.submit(p, max_length=len(p) + 3) for p in prompts]
    n = 0
    while not all(f.done() for f in futs):
        sched.step()
        n += 1
        assert n < 50

    def expect(p):
        seq = list(p)
        for _ in range(3):
            seq.append(sum(seq) % eng.vocab)
        return seq

    for f, p in zip(futs, prompts):
        assert f.result().tolist() == expect(p)
    # first step: 4 tokens of the long prompt (the budget), nothing of the second; then the second prompt enters and
    # later decodes beside the long prompt's portions; the third request waits for a slot
    assert eng.calls[0] == [(0, 4)] and eng.calls[1] == [(0, 4)]
    assert any(len(c) == 2 and {n for _, n in c} == {1} for c in eng.calls)         # two requests decoding together
    assert any(len(c) == 2 and sorted(n for _, n in c) != [1, 1] for c in eng.calls)  # a portion beside a single token
    assert max(len(c) for c in eng.calls) <= 2 and sorted(eng.free) == [0, 1]
    # rejected at the door
    assert isinstance(sched.submit([], 5).exception(), ValueError)
    assert isinstance(sched.submit([1, 2, 3], 3).exception(), ValueError)
    assert isinstance(sched.submit([1], 100).exception(), ValueError)
