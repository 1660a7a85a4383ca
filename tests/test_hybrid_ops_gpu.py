"""Each mechanism of the ragged fp32-residual path alone, kernel against the oracle's function for it
(oracle/hybrid_ref.py), on inputs made so that a fault shows: one score that stands out for a key far back, at a
page border, just inside and just outside a chunk or window; a sink that dominates; slots holding garbage."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import hybrid_ref as R  # noqa: E402

DEV = "cuda:0"


def meta(entries):
    """entries: [(slot, n, start)] -> (row_ent, ent) int32 on the device."""
    row_ent, ent, r = [], [], 0
    for i, (slot, n, start) in enumerate(entries):
        ent += [slot, r, n, start]
        row_ent += [i] * n
        r += n
    return (torch.tensor(row_ent, dtype=torch.int32, device=DEV), torch.tensor(ent, dtype=torch.int32, device=DEV))


def test_scalar_norms_and_residual_add():
    from dli_b200 import ops

    torch.manual_seed(0)
    x = torch.randn(5, 72, device=DEV) * 3
    y = torch.randn(5, 72, device=DEV)
    hn = torch.empty_like(x)
    ops.scalar_rmsnorm(x, 1.7, 1e-5, hn)
    assert torch.allclose(hn.double().cpu(), R.rms_unit(x.double().cpu(), 1e-5) * 1.7, atol=1e-5)
    for ydt in (torch.float32, torch.bfloat16):
        x2, yy = x.clone(), y.to(ydt)
        ops.postnorm_add_norm(yy, x2, 0.6, 1e-5, hn, 1.3)
        want_x = x.double().cpu() + R.rms_unit(yy.double().cpu(), 1e-5) * 0.6
        assert torch.allclose(x2.double().cpu(), want_x, atol=1e-5)
        assert torch.allclose(hn.double().cpu(), R.rms_unit(want_x, 1e-5) * 1.3, atol=1e-5)


@pytest.mark.parametrize("taps", [2, 4, 7])
def test_causal_conv_portions_tails_and_slot_reuse(taps):
    """Three sequences in slots holding garbage; portions of 1, 2 and more rows, shorter and longer than the taps."""
    from dli_b200 import ops

    torch.manual_seed(taps)
    d, lens, slots = 40, [23, 9, 14], [2, 0, 3]
    w = torch.randn(d, taps, device=DEV)
    hs = [torch.randn(n, d, device=DEV) for n in lens]
    want = [h.double().cpu() + R.causal_conv(h.double().cpu(), w.double().cpu()) for h in hs]
    tail = torch.full((4, taps - 1, d), 1e6, device=DEV)
    at = [0, 0, 0]
    got = [[], [], []]
    sizes = [[1, 2, 1], [2, 1, 5], [1, 1, 1], [9, 2, 3], [3, 3, 4], [7, 0, 0]]
    for step in sizes:
        ents, parts = [], []
        for i, n in enumerate(step):
            n = min(n, lens[i] - at[i])
            if n:
                ents.append((slots[i], n, at[i]))
                parts.append((i, n))
        h = torch.cat([hs[i][at[i]:at[i] + n] for i, n in parts])
        row_ent, ent = meta(ents)
        out = torch.empty_like(h)
        ops.causal_conv_ragged(h, tail, w, row_ent, ent, out)
        o = 0
        for i, n in parts:
            got[i].append(out[o:o + n])
            o += n
            at[i] += n
    for i in range(3):
        assert at[i] == lens[i]
        assert torch.allclose(torch.cat(got[i]).double().cpu(), want[i], atol=1e-4)


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(1, 40, 24), (70, 130, 100), (3, 64, 256)])
def test_linear_any(dt, shape):
    from dli_b200 import ops

    M, N, K = shape
    torch.manual_seed(1)
    x, w = torch.randn(M, K, device=DEV).to(dt), torch.randn(N, K, device=DEV).to(dt)
    out = torch.empty(M, N, dtype=dt, device=DEV)
    ops.linear_any(x, w, out)
    ref = x.double() @ w.double().T
    tol = 1e-4 if dt == torch.float32 else 0.02 * ref.abs().max().item()
    assert (out.double() - ref).abs().max() < tol


def attn_oracle(q, k, v, g, m, sink, qn, kn, eps):
    """Through the oracle's mixer with identity projections: h = [q | k | v | g] columns."""
    T = q.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    h = torch.cat((q, k, v, g), dim=1).double()
    n = h.shape[1]
    eye = torch.eye(n, dtype=torch.float64)
    P = {"q": eye[:H * D], "k": eye[H * D:H * D + G * D], "v": eye[H * D + G * D:H * D + G * D + G * V],
         "g": eye[H * D + G * D + G * V:], "o": torch.eye(H * V, dtype=torch.float64), "q.norm": qn.double(),
         "k.norm": kn.double(), "sink": sink.double()}
    return R.attention_mixer(h, P, "", m, eps)


def run_attn(q, k, v, g, m, sink, qn, kn, eps, cuts, page_size, dt=torch.float32, window=0, tc=False):
    """The kernels on one sequence cut into portions `cuts`, pages handed out in a scrambled order."""
    from dli_b200 import ops
    from dli_b200.ragged_engine import rot_frequencies

    T = q.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rot = m["rot"]
    proj = torch.cat((q, k, v, g), dim=1).to(dt).to(DEV).contiguous()
    n_pages = (T + page_size - 1) // page_size
    perm = torch.randperm(n_pages + 3, generator=torch.Generator().manual_seed(3))[:n_pages].to(torch.int32)
    pt = torch.zeros(2, n_pages, dtype=torch.int32)
    pt[1] = perm
    pt = pt.to(DEV)
    kc = torch.full((n_pages + 3, G, page_size, D), 7.0, dtype=dt, device=DEV)
    vc = torch.full((n_pages + 3, G, page_size, V), -5.0, dtype=dt, device=DEV)
    pos = torch.arange(T, dtype=torch.float64)[:, None]
    aq = pos * rot_frequencies(rot["base"], rot["dims"], rot.get("scaling"))[None]
    av = pos * rot_frequencies(rot["base"], V, None)[None]
    cq, sq, cv, sv = (t.float().to(DEV).contiguous() for t in (aq.cos(), aq.sin(), av.cos(), av.sin()))
    out = torch.empty(T, H * V, dtype=dt, device=DEV)
    at = 0
    for n in cuts:
        n = min(n, T - at)
        if n <= 0:
            break
        row_ent, ent = meta([(1, n, at)])
        qbuf = torch.empty(n, H * D, dtype=torch.float32, device=DEV)
        pr = proj[at:at + n].contiguous()
        ops.attn_prep_append(pr, qbuf, kc, vc, row_ent, ent, pt, H, G, D, V, rot["dims"], 0, H * D, H * D + G * D,
                             qn.float().to(DEV), kn.float().to(DEV), eps, cq, sq, cv, sv)
        o = torch.empty(n, H * V, dtype=dt, device=DEV)
        if tc:
            tiles = torch.tensor([[0, q0] for q0 in range(0, n, 64)], dtype=torch.int32, device=DEV)
            ops.attn_ragged_tc(qbuf, kc, vc, pr, o, ent, tiles, pt, H, G, D, V, m["scale"], chunk=m["mask"]["size"],
                               window=window, sink=sink.float().to(DEV), g_off=H * D + G * D + G * V, cos_v=cv, sin_v=sv)
        else:
            ops.attn_ragged(qbuf, kc, vc, pr, o, row_ent, ent, pt, H, G, D, V, m["scale"], chunk=m["mask"]["size"],
                            window=window, sink=sink.float().to(DEV), g_off=H * D + G * D + G * V, cos_v=cv, sin_v=sv)
        out[at:at + n] = o
        at += n
    assert at == T
    return out


@pytest.mark.parametrize("cuts", [[200], [1] * 200, [37, 2, 2, 50, 1, 1, 1, 3, 64, 64], [150] + [1] * 50])
def test_attention_random_inputs_all_options(cuts):
    torch.manual_seed(2)
    m = {"heads": 6, "kv_heads": 2, "dim": 12, "vdim": 20, "scale": 0.4, "mask": {"size": 48},
         "rot": {"base": 300.0, "dims": 8, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 32}}}
    T = 140
    q, k = torch.randn(T, 6 * 12), torch.randn(T, 2 * 12)
    v, g = torch.randn(T, 2 * 20), torch.randn(T, 6)
    sink, qn, kn = torch.randn(6), torch.rand(12) + 0.5, torch.rand(12) + 0.5
    ref = attn_oracle(q, k, v, g, m, sink, qn, kn, 1e-5)
    got = run_attn(q, k, v, g, m, sink, qn, kn, 1e-5, cuts, page_size=8)
    assert (got.double().cpu() - ref).abs().max() < 2e-4


@pytest.mark.parametrize("cuts", [[300], [130, 2] + [1] * 170])
@pytest.mark.parametrize("target", ["first_in_chunk", "last_of_previous_chunk", "page_border", "far_in_chunk"])
def test_attention_one_key_stands_out(cuts, target):
    """The query at position i has a large score with ONE key j (and small ones elsewhere): inside the chunk the
    output is v_j turned by j - i ... by the oracle; just outside it, v_j must not appear at all."""
    torch.manual_seed(4)
    chunk, page = 128, 16
    # one rotated pair (dims 0, 1); the direction that carries the signal (3) is outside it.  The head norm (unit
    # weights) brings every q and k to unit RMS: the marked pair scores 8 * scale, every other key exactly 0.
    m = {"heads": 2, "kv_heads": 1, "dim": 8, "vdim": 8, "scale": 4.0, "mask": {"size": chunk},
         "rot": {"base": 50.0, "dims": 2}}
    T = 260
    i = 250                                    # chunk of i: positions 128..255
    j = {"first_in_chunk": 128, "last_of_previous_chunk": 127, "page_border": 143, "far_in_chunk": 129}[target]
    q, k = torch.randn(T, 16), torch.randn(T, 8)
    v, g = torch.randn(T, 8), torch.zeros(T, 2)
    k[:, 3] = 0
    q[i, :8] = 0
    q[i, 3] = 1.0                              # head 0 of position i asks for direction 3 ...
    k[j] = 0
    k[j, 3] = 1.0                              # ... which only key j has
    sink, ones = torch.tensor([-30.0, -30.0]), torch.ones(8)
    ref = attn_oracle(q, k, v, g, m, sink, ones, ones, 1e-6)
    got = run_attn(q, k, v, g, m, sink, ones, ones, 1e-6, cuts, page_size=page)
    assert (got.double().cpu() - ref).abs().max() < 2e-4
    # and the reference itself shows the case: with the key visible, head 0's weight sits on it
    inside = j >= 128
    av = torch.arange(T, dtype=torch.float64)[:, None] * R.frequencies(50.0, 8)[None]
    vj_at_i = R.turn_pairs(R.turn_pairs(v[j].double(), av[j]), -av[i]) * 0.5   # gate sigmoid(0)
    close = (ref[i, :8] - vj_at_i).abs().max() < 1e-3
    assert bool(close) == inside


@pytest.mark.parametrize("dims", [(64, 64), (128, 128), (64, 128), (128, 256)])
@pytest.mark.parametrize("cuts", [[230], [100, 3, 64, 63], [17, 1, 130, 2, 80]])
def test_attention_tensor_core_tiles_against_oracle(dims, cuts):
    """The tensor-core kernel on portions that start anywhere (also single rows beside them): chunk edges that are no
    multiple of the tile, pages smaller than the tile, grouped heads, sink, gate, value rotation; bf16 operands."""
    D, V = dims
    torch.manual_seed(7)
    m = {"heads": 4, "kv_heads": 2, "dim": D, "vdim": V, "scale": D ** -0.5, "mask": {"size": 75},
         "rot": {"base": 1000.0, "dims": D // 2, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}}}
    T = 230
    bf = lambda t: t.to(torch.bfloat16).float()  # noqa: E731  (inputs that bf16 holds exactly)
    q, k = bf(torch.randn(T, 4 * D)), bf(torch.randn(T, 2 * D))
    v, g = bf(torch.randn(T, 2 * V)), bf(torch.randn(T, 4))
    sink, qn, kn = torch.randn(4), torch.rand(D) + 0.5, torch.rand(D) + 0.5
    ref = attn_oracle(q, k, v, g, m, sink, qn, kn, 1e-5)
    got = run_attn(q, k, v, g, m, sink, qn, kn, 1e-5, cuts, page_size=16, dt=torch.bfloat16, tc=True)
    plain = run_attn(q, k, v, g, m, sink, qn, kn, 1e-5, cuts, page_size=16, dt=torch.bfloat16, tc=False)
    assert (got.double().cpu() - ref).abs().max() < 0.03
    assert (plain.double().cpu() - ref).abs().max() < 0.03
    assert (got.double().cpu() - ref).pow(2).mean().sqrt() < 0.004


@pytest.mark.parametrize("j", [149, 150, 212])
def test_attention_tensor_core_one_key_stands_out(j):
    """Query 220 (chunk 150..224) against ONE matching key: the last position of the previous chunk (never seen), the
    first of its own, and one in the middle; bf16 rounding cannot hide a weight of one."""
    torch.manual_seed(8)
    D = V = 64
    m = {"heads": 2, "kv_heads": 1, "dim": D, "vdim": V, "scale": 4.0, "mask": {"size": 75}, "rot": {"base": 50.0, "dims": 2}}
    T, i = 230, 220
    q, k = torch.randn(T, 2 * D), torch.randn(T, D)
    v, g = torch.randn(T, V).to(torch.bfloat16).float(), torch.zeros(T, 2)
    k[:, 3] = 0
    q[i, :D] = 0
    q[i, 3] = 1.0
    k[j] = 0
    k[j, 3] = 1.0
    sink, ones = torch.tensor([-30.0, -30.0]), torch.ones(D)
    ref = attn_oracle(q, k, v, g, m, sink, ones, ones, 1e-6)
    got = run_attn(q, k, v, g, m, sink, ones, ones, 1e-6, [130, 100], page_size=16, dt=torch.bfloat16, tc=True)
    assert (got.double().cpu()[i] - ref[i]).abs().max() < 0.02
    av = torch.arange(T, dtype=torch.float64)[:, None] * R.frequencies(50.0, V)[None]
    vj_at_i = R.turn_pairs(R.turn_pairs(v[j].double(), av[j]), -av[i]) * 0.5
    assert bool((got.double().cpu()[i, :V] - vj_at_i).abs().max() < 0.02) == (j >= 150)


def test_attention_sink_takes_weight_and_window_option():
    torch.manual_seed(5)
    m = {"heads": 2, "kv_heads": 2, "dim": 8, "vdim": 8, "scale": 0.5, "mask": {"size": 0},
         "rot": {"base": 100.0, "dims": 4}}
    T = 40
    q, k, v, g = torch.randn(T, 16), torch.randn(T, 16), torch.randn(T, 16), torch.randn(T, 2)
    ones = torch.ones(8)
    big = torch.tensor([25.0, -25.0])           # head 0: the sink swallows the softmax; head 1: it is negligible
    ref = attn_oracle(q, k, v, g, m, big, ones, ones, 1e-6)
    got = run_attn(q, k, v, g, m, big, ones, ones, 1e-6, [11, 1, 1, 27], page_size=4)
    assert (got.double().cpu() - ref).abs().max() < 2e-4
    assert ref[:, :8].abs().max() < 1e-6 and ref[:, 8:].abs().max() > 1e-2
    # sliding window (an option of the kernel other designs use): against a direct computation
    from dli_b200 import ops  # noqa: F401
    w = 6
    got_w = run_attn(q, k, v, g, m, big, ones, ones, 1e-6, [40], page_size=4, window=w)
    got_full = run_attn(q, k, v, g, m, big, ones, ones, 1e-6, [40], page_size=4)
    assert torch.allclose(got_w[:w], got_full[:w], atol=1e-6) and not torch.allclose(got_w[w + 3:], got_full[w + 3:], atol=1e-3)


def mlstm_oracle(q, k, v, g, ig, fg, m, ib, fb, nw, eps):
    H, D, V = m["heads"], m["dim"], m["vdim"]
    h = torch.cat((q, k, v, g, ig, fg), dim=1).double()
    eye = torch.eye(h.shape[1], dtype=torch.float64)
    o = [0, H * D, 2 * H * D, 2 * H * D + H * V, 2 * H * D + 2 * H * V, 2 * H * D + 2 * H * V + H, 2 * H * D + 2 * H * V + 2 * H]
    P = {n: eye[o[i]:o[i + 1]] for i, n in enumerate("qkvgif")}
    P.update({"i.b": ib.double(), "f.b": fb.double(), "norm": nw.double(), "o": torch.eye(H * V, dtype=torch.float64)})
    return R.mlstm_mixer(h, P, "", m, eps)


@pytest.mark.parametrize("dims", [(2, 56, 96), (3, 10, 40), (1, 130, 33)])
@pytest.mark.parametrize("cuts", [[90], [1] * 90, [2, 2, 31, 1, 1, 40, 13], [70, 20], [300]])
@pytest.mark.parametrize("blocked", [False, True, "parallel"])
def test_mlstm_portions_and_dirty_slots(dims, cuts, blocked):
    """Token by token (blocked=False), 64 positions at a time in order (True) and with the blocks of a portion in
    parallel ("parallel"): portions longer and shorter than a block, a block that ends inside a portion, against the
    oracle's loop."""
    from dli_b200 import ops

    H, D, V = dims
    torch.manual_seed(6)
    m = {"heads": H, "dim": D, "vdim": V, "gate_cap": 6.0}
    T = 90 if cuts != [300] else 300
    q, k, v, g = torch.randn(T, H * D), torch.randn(T, H * D), torch.randn(T, H * V), torch.randn(T, H * V)
    ig, fg = 4 * torch.randn(T, H), 4 * torch.randn(T, H) + 2   # beyond the cap on both sides
    ib, fb, nw = torch.randn(H), torch.randn(H), torch.rand(H * V) + 0.5
    ref = mlstm_oracle(q, k, v, g, ig, fg, m, ib, fb, nw, 1e-5)
    proj = torch.cat((q, k, v, g, ig, fg), dim=1).to(DEV).contiguous()
    S = torch.full((3, H, D, V), 9e3, device=DEV)   # slots hold garbage: position 0 starts from zero regardless
    n = torch.full((3, H, D), -4e3, device=DEV)
    mm = torch.full((3, H), 55.0, device=DEV)
    out = torch.empty(T, H * V, device=DEV)
    at = 0
    for c in cuts:
        c = min(c, T - at)
        if c <= 0:
            break
        _, ent = meta([(2, c, at)])
        pr = proj[at:at + c].contiguous()
        o = torch.empty(c, H * V, device=DEV)
        offs = (0, H * D, 2 * H * D, 2 * H * D + 2 * H * V, 2 * H * D + 2 * H * V + H, 2 * H * D + H * V)
        if blocked == "parallel":
            tiles = torch.tensor([[0, q0] for q0 in range(0, c, 64)], dtype=torch.int32, device=DEV)
            scr = torch.full((ops.mlstm_parallel_scratch_floats(tiles.shape[0], H, D, V),), float("nan"), device=DEV)
            ops.mlstm_ragged_parallel(pr, torch.empty(c * H * V, device=DEV), o, ent, tiles, scr, H, D, V, *offs,
                                      ib.to(DEV), fb.to(DEV), 6.0, nw.to(DEV), 1e-5, S, n, mm)
        else:
            ops.mlstm_ragged(pr, torch.empty(c * H * V, device=DEV), o, ent, H, D, V, *offs, ib.to(DEV), fb.to(DEV),
                             6.0, nw.to(DEV), 1e-5, S, n, mm, blocked=blocked)
        out[at:at + c] = o
        at += c
    assert at == T
    assert (out.double().cpu() - ref).abs().max() < 3e-4 * max(1.0, ref.abs().max().item())


def test_rot_frequencies_match_the_oracle():
    from dli_b200.ragged_engine import rot_frequencies

    sc = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 256}
    for dims in (8, 64):
        for s in (None, sc):
            assert torch.allclose(rot_frequencies(10000.0, dims, s), R.frequencies(10000.0, dims, s), rtol=1e-12)
    f = R.frequencies(10000.0, 64, sc)
    plain = R.frequencies(10000.0, 64)
    ratio = (plain / f)
    assert ratio.min() == 1.0 and abs(ratio.max().item() - 8.0) < 1e-9 and ((ratio > 1.001) & (ratio < 7.999)).any()
