"""The layer-by-layer decoder family on the ragged engine against the plain float64 oracle (oracle/hybrid_ref.py).

Small made-up configurations with random weights.  The float32 engine must agree with the oracle to ~1e-4 of the
logits' spread at EVERY position — a mask that is one token off, a lost state, a forgotten sink or a stale slot
changes logits by orders of magnitude more — whatever the schedule: whole prompts, token-by-token decoding, portions
down to two tokens, mixed batches, small page pools and reused slots.  The bfloat16 engine is held to a bf16-sized
bound and to agreement between schedules.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import hybrid_ref as R  # noqa: E402


def attn(heads=4, kv=2, dim=16, vdim=24, chunk=8, rot_dims=8, scale=0.3, scaling=True):
    rot = {"base": 1000.0, "dims": rot_dims}
    if scaling:
        rot["scaling"] = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale,
                                           "mask": {"size": chunk}, "rot": rot}}


def mlstm(heads=3, dim=10, vdim=40, cap=9.0):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}}


def config(layers, width=64, vocab=97, taps=3, eps=1e-5):
    out = []
    for L, ff in layers:
        L = dict(L)
        L["mlp"] = {"kind": "dense", "ff": ff} if ff else None
        out.append(L)
    return {"architecture": "Sokevik", "vocab": vocab, "width": width, "norm": {"eps": eps}, "canon": {"taps": taps},
            "layers": out}


def cfg_a():
    """attention + mlp, an mlstm without mlp, a layer sharing layer 0's weights, an mlstm WITH mlp."""
    a = attn()
    shared = dict(a, weights_of=0)
    return config([(a, 128), (mlstm(), 0), (shared, 128), (mlstm(heads=1, dim=8, vdim=32), 96)])


def cfg_b():
    """other sizes: taps 2, no frequency scaling, full rotation, one kv head per head, odd vocabulary, an attention layer
    without feed-forward, an mlstm first, width that is not a multiple of 64."""
    return config([(mlstm(heads=2, dim=12, vdim=16, cap=5.0), 72), (attn(heads=2, kv=2, dim=12, vdim=8, chunk=5,
                   rot_dims=12, scale=0.5, scaling=False), 0), (attn(heads=3, kv=1, dim=8, vdim=16, chunk=16, rot_dims=4), 64)],
                  width=48, vocab=53, taps=2)


def cfg_c():
    """one tap (the convolution sees the current input only), one head everywhere, chunk of one position, no scaling."""
    return config([(attn(heads=1, kv=1, dim=8, vdim=8, chunk=1, rot_dims=2, scale=1.0, scaling=False), 32),
                   (mlstm(heads=1, dim=4, vdim=4, cap=2.0), 0)], width=16, vocab=19, taps=1)


def build(cfg, dtype, seed=0, max_batch=4, max_seq_len=256, pool=None, page_size=4):
    from dli_b200 import sokevik
    from dli_b200.ragged_engine import RaggedEngine

    spec = sokevik.spec_from_config(cfg)
    sd = sokevik.random_state_dict(spec, seed=seed, std=0.15)
    eng = RaggedEngine(spec, max_batch=max_batch, max_seq_len=max_seq_len, page_size=page_size, kv_pool_tokens=pool,
                       dtype=dtype)
    eng.load_tensors(sokevik.model_tensors(spec, sd))
    return eng, sd


def prompt(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def rel_err(got, ref):
    """Per position: RMS of the logit difference (mean removed) over the RMS spread of the reference logits."""
    d = got.double().cpu() - ref
    d = d - d.mean(-1, keepdim=True)
    spread = (ref - ref.mean(-1, keepdim=True)).pow(2).mean().sqrt()
    return d.pow(2).mean(-1).sqrt() / spread


def run_schedule(eng, toks, cuts):
    """One sequence alone, cut into portions of the given sizes (the rest token by token); logits at every position."""
    slot = eng.open_sequence()
    out, at = [], 0
    sizes = list(cuts)
    while at < len(toks):
        n = sizes.pop(0) if sizes else 1
        n = min(n, len(toks) - at)
        out.append(eng.step([(slot, toks[at:at + n])], [list(range(n))]).float().cpu())
        at += n
    eng.close_sequence(slot)
    return torch.cat(out)


TOL32, TOL16 = 2e-4, 0.08


@pytest.mark.parametrize("make", [cfg_a, cfg_b, cfg_c])
def test_whole_prompt_float32_matches_oracle_at_every_position(make):
    cfg = make()
    eng, sd = build(cfg, torch.float32)
    toks = prompt(45, cfg["vocab"], 1)
    ref = R.forward(cfg, sd, toks)
    assert rel_err(run_schedule(eng, toks, [45]), ref).max() < TOL32


def test_residual_stream_after_every_layer():
    cfg = cfg_a()
    eng, sd = build(cfg, torch.float32)
    toks = prompt(19, cfg["vocab"], 2)
    layers = []
    R.forward(cfg, sd, toks, layers)
    eng.layer_trace = []
    run_schedule(eng, toks, [19])
    assert len(eng.layer_trace) == len(layers)
    for got, ref in zip(eng.layer_trace, layers):
        assert (got.double().cpu() - ref).abs().max() < 1e-4 * ref.abs().max()


@pytest.mark.parametrize("make", [cfg_a, cfg_b, cfg_c])
@pytest.mark.parametrize("cuts", [[], [1, 1, 2], [2, 2, 3, 5, 7, 11], [17, 2, 16, 3], [30]])
def test_portions_and_decoding_float32(make, cuts):
    """Token by token from the first token; portions of 2..; a prompt then decoding across several chunk edges."""
    cfg = make()
    eng, sd = build(cfg, torch.float32)
    toks = prompt(52, cfg["vocab"], 3)
    ref = R.forward(cfg, sd, toks)
    assert rel_err(run_schedule(eng, toks, cuts), ref).max() < TOL32


@pytest.mark.parametrize("make", [cfg_a, cfg_b])
def test_bfloat16_engine_is_close_and_schedules_agree(make):
    cfg = make()
    eng, sd = build(cfg, torch.bfloat16)
    toks = prompt(40, cfg["vocab"], 4)
    ref = R.forward(cfg, sd, toks)
    whole = run_schedule(eng, toks, [40])
    parts = run_schedule(eng, toks, [7, 2, 9, 3])
    assert rel_err(whole, ref).max() < TOL16
    assert rel_err(parts, ref).max() < TOL16
    assert rel_err(parts, whole.double()).max() < TOL16


def test_mixed_batches_of_unequal_requests_match_each_alone():
    """Four requests of different lengths move through shared steps in portions of different sizes, some decoding
    while others are in their prompt, some skipping steps; each position equals the oracle's for that request alone."""
    cfg = cfg_a()
    eng, sd = build(cfg, torch.float32, pool=160, max_seq_len=160)
    lens = [37, 9, 58, 1]
    reqs = [prompt(n, cfg["vocab"], 10 + i) for i, n in enumerate(lens)]
    refs = [R.forward(cfg, sd, t) for t in reqs]
    slots = [eng.open_sequence() for _ in reqs]
    at = [0] * len(reqs)
    got = [[] for _ in reqs]
    pattern = [[5, 2, 9, 1], [1, 0, 16, 0], [3, 1, 1, 0], [0, 3, 2, 0], [8, 1, 7, 0], [1, 1, 1, 0], [19, 1, 22, 0]]
    k = 0
    while any(a < n for a, n in zip(at, lens)):
        sizes = pattern[k % len(pattern)]
        k += 1
        batch, want, who = [], [], []
        for i, n in enumerate(sizes):
            n = min(n, lens[i] - at[i])
            if n > 0:
                batch.append((slots[i], reqs[i][at[i]:at[i] + n]))
                want.append(list(range(n)))
                who.append((i, n))
        if not batch:
            continue
        lg = eng.step(batch, want).float().cpu()
        o = 0
        for i, n in who:
            got[i].append(lg[o:o + n])
            o += n
            at[i] += n
    for i in range(len(reqs)):
        assert rel_err(torch.cat(got[i]), refs[i]).max() < TOL32, f"request {i}"


def test_pages_and_slots_are_used_again():
    """A pool that holds two sequences at most and two slots: six sequences pass through in turn, each against the
    oracle; a slot's previous state (recurrent memory, convolution tails, pages) must not leak into the next one."""
    cfg = cfg_a()
    eng, sd = build(cfg, torch.float32, max_batch=2, pool=64, max_seq_len=64, page_size=4)
    for r in range(3):
        ta, tb = prompt(29 + r, cfg["vocab"], 20 + r), prompt(11 + 2 * r, cfg["vocab"], 30 + r)
        ra, rb = R.forward(cfg, sd, ta), R.forward(cfg, sd, tb)
        sa, sb = eng.open_sequence(), eng.open_sequence()
        la = [eng.step([(sa, ta[:13])], [list(range(13))])]
        both = eng.step([(sa, ta[13:]), (sb, tb)], [list(range(len(ta) - 13)), list(range(len(tb)))])
        la.append(both[:len(ta) - 13])
        assert rel_err(torch.cat(la), ra).max() < TOL32
        assert rel_err(both[len(ta) - 13:], rb).max() < TOL32
        eng.close_sequence(sb if r % 2 else sa)   # give the slots back in changing order
        eng.close_sequence(sa if r % 2 else sb)
    assert len(eng.kv.free) == eng.kv.num_pages and len(eng.slots.free) == 2
    with pytest.raises(RuntimeError):
        s = [eng.open_sequence(), eng.open_sequence()]
        try:
            eng.step([(s[0], prompt(40, cfg["vocab"], 1)), (s[1], prompt(40, cfg["vocab"], 2))])
        finally:
            for x in s:
                eng.close_sequence(x)


def test_long_decoding_float32():
    """150 tokens one by one: every chunk edge of both attention layers is crossed many times, pages fill and follow."""
    cfg = cfg_b()
    eng, sd = build(cfg, torch.float32)
    toks = prompt(150, cfg["vocab"], 5)
    ref = R.forward(cfg, sd, toks)
    assert rel_err(run_schedule(eng, toks, [3]), ref).max() < TOL32


def test_greedy_generation_through_the_scheduler():
    """generate() -> RaggedBatcher -> step(): three prompts of one length share steps; tokens equal the oracle's greedy
    continuation (float32 engine: no near-ties at these sizes)."""
    cfg = cfg_a()
    eng, sd = build(cfg, torch.float32, max_batch=3)
    eng.prefill_chunk = 8   # prompts go in portions of at most 8 tokens per step, shared between the requests
    ids = torch.tensor([prompt(13, cfg["vocab"], 40 + i) for i in range(3)])
    out = eng.generate(ids, max_length=13 + 6)
    for b in range(3):
        assert out[b].tolist() == R.greedy(cfg, sd, ids[b].tolist(), 6)
    assert len(eng.slots.free) == 3 and len(eng.kv.free) == eng.kv.num_pages


def test_scheduler_requests_of_unequal_length_and_sampling_is_keyed_by_position():
    from dli_b200.batching import RaggedBatcher

    cfg = cfg_b()
    eng, sd = build(cfg, torch.float32, max_batch=2)   # float32: the same bits whatever shares the step
    pa, pb, pc = prompt(21, cfg["vocab"], 50), prompt(5, cfg["vocab"], 51), prompt(9, cfg["vocab"], 52)

    def run(prompts, chunk):
        sched = RaggedBatcher(eng, chunk=chunk)
        futs = [sched.submit(p, max_length=len(p) + 5, do_sample=True, seed=7 + i) for i, p in enumerate(prompts)]
        while not all(f.done() for f in futs):
            sched.step()
        return [f.result().tolist() for f in futs]

    together = run([pa, pb, pc], chunk=6)      # three requests on two slots: the third waits for a slot
    alone = [run([p], chunk=64)[0] for p in (pa, pb, pc)]
    # seeds follow the submission order in run(); alone[i] used seed 7, so compare the first request only for tokens
    assert together[0] == alone[0]
    assert [len(t) for t in together] == [26, 10, 14]


def test_bfloat16_portions_on_the_tensor_core_attention():
    """Head sizes that have a tensor-core tile: portions of 16 rows and more take that kernel, shorter steps the
    row-wise one; both against the oracle and against each other."""
    cfg = config([(attn(heads=4, kv=2, dim=64, vdim=64, chunk=50, rot_dims=32, scale=0.125), 128), (mlstm(), 0),
                  (attn(heads=2, kv=1, dim=64, vdim=128, chunk=33, rot_dims=64, scale=0.125), 0)], width=128)
    eng, sd = build(cfg, torch.bfloat16, max_seq_len=256, page_size=16)
    toks = prompt(170, cfg["vocab"], 6)
    ref = R.forward(cfg, sd, toks)
    whole = run_schedule(eng, toks, [170])
    parts = run_schedule(eng, toks, [70, 3, 64, 20])
    eng.tc_min_rows = 10 ** 9
    rowwise = run_schedule(eng, toks, [170])
    for got in (whole, parts, rowwise):
        assert rel_err(got, ref).max() < TOL16
    assert rel_err(whole, rowwise.double()).max() < TOL16 / 2


def test_decode_steps_replayed_as_a_graph_equal_eager_steps():
    """Steps of single tokens are captured once per batch size and replayed; the logits equal the eager launches' bit
    for bit, also when the batch size changes back and forth and a sequence leaves in between."""
    cfg = cfg_a()
    outs = []
    for graph in (True, False):
        eng, sd = build(cfg, torch.float32, max_batch=3)
        eng.use_cuda_graph = graph
        seqs = [prompt(n, cfg["vocab"], 60 + i) for i, n in enumerate((30, 30, 30))]
        slots = [eng.open_sequence() for _ in seqs]
        got = [eng.step([(slots[i], seqs[i][:9]) for i in range(3)])]
        for t in range(9, 20):
            got.append(eng.step([(slots[i], [seqs[i][t]]) for i in range(3)]))
        eng.close_sequence(slots[1])
        for t in range(20, 30):
            got.append(eng.step([(slots[i], [seqs[i][t]]) for i in (0, 2)]))
            if t % 3 == 0:
                got.append(eng.step([(slots[0], [5])]))
                seqs[0].insert(t + 1, 5)
                seqs[0].pop()
        outs.append(torch.cat([g.float().cpu() for g in got]))
        if graph:
            assert any(isinstance(v, tuple) for v in eng._graphs.values())
    assert torch.equal(outs[0], outs[1])
