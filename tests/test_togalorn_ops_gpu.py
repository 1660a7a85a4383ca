"""Each mechanism of the Togalorn design alone, kernels against the oracle's function for it (oracle/togalorn_ref.py),
on inputs made so that a fault shows: a softmax so sharp that every query picks ONE key somewhere among hundreds, over
page borders; a state-space layer that forgets slowly, so that a lost state shows at the end; slots holding garbage; a
router whose choice differs from its weights because of the correction."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import togalorn_ref as R  # noqa: E402
from test_togalorn_engine_gpu import config, latent, mamba, moe  # noqa: E402

DEV = "cuda:0"


def one_layer_engine(layer, mlp=None, width=32, page_size=4, max_seq_len=512, seed=0, std=0.3, groups=2):
    from dli_b200 import togalorn
    from dli_b200.ragged_engine import RaggedEngine

    cfg = config([(layer, mlp)], width=width, groups=groups)
    spec = togalorn.spec_from_config(cfg)
    sd = togalorn.random_state_dict(spec, seed=seed, std=std)
    eng = RaggedEngine(spec, max_batch=4, max_seq_len=max_seq_len, page_size=page_size, dtype=torch.float32)
    eng.load_tensors(togalorn.model_tensors(spec, sd))
    return eng, cfg, sd


def step_views(eng, entries):
    """entries [(slot, n, start)] -> the device views a step hands to the mixers (tokens unused here)."""
    row_ent, ent, r = [], [], 0
    for i, (slot, n, start) in enumerate(entries):
        ent += [slot, r, n, start]
        row_ent += [i] * n
        r += n
    z = torch.zeros(1, dtype=torch.int32, device=DEV)
    return (z, torch.tensor(row_ent, dtype=torch.int32, device=DEV), torch.tensor(ent, dtype=torch.int32, device=DEV), z, z), r


def tiles_of(entries):
    """(entry, first row of every 64-row block within the entry), as a step builds them."""
    t = [[i, q0] for i, (_, n, _) in enumerate(entries) for q0 in range(0, n, 64)]
    return torch.tensor(t, dtype=torch.int32, device=DEV)


def run_mixer(eng, kind, u, cuts, slot_order=(2,)):
    """u [T, n_proj]: the mixer's input projection (made on the host), fed through the engine's mixer kernels in
    portions of the given sizes (then token by token) -> the mixer's output before its out-projection [T, H*V]."""
    m, P = eng.spec.layers[0].mixer, eng.layers[0]
    T = u.shape[0]
    for _ in range(slot_order[0]):   # take a slot that is not the first one
        eng.open_sequence()
    slot = eng.open_sequence()
    n_proj = P["w_proj"].shape[0]
    outs, at, sizes = [], 0, list(cuts)
    while at < T:
        n = min(sizes.pop(0) if sizes else 1, T - at)
        eng._workspace(n)
        if eng.attn_layers:
            eng.kv.reserve(slot, at + n)
            eng.kv.commit()
        views, rows = step_views(eng, [(slot, n, at)])
        views = views[:4] + (tiles_of([(slot, n, at)]),)
        proj = torch.zeros(n, n_proj, device=DEV)
        proj[:, :u.shape[1]] = u[at:at + n].float().to(DEV)
        mix = torch.empty(n, m.heads * m.vdim, device=DEV)
        if kind == "latent_attention":
            eng._latent_attention(0, m, P, proj, mix, n, views)
        else:
            eng._mamba2(0, m, P, proj, mix, n, views, long_step=n >= 16)   # portions: block-wise, in parallel from 65 rows
        outs.append(mix.double().cpu())
        at += n
    return torch.cat(outs)


@pytest.mark.parametrize("groups", [1, 3, 8])
def test_grouped_rms_norm(groups):
    from dli_b200 import ops

    torch.manual_seed(groups)
    x = torch.randn(7, 48, device=DEV) * torch.linspace(0.1, 30, 48, device=DEV)  # groups of very different size
    w = torch.randn(48, device=DEV)
    hn, he = torch.empty_like(x), torch.empty(7, 48, dtype=torch.bfloat16, device=DEV)
    ops.group_rmsnorm(x, w, groups, 1e-5, hn=hn, he=he)
    want = R.grouped_rms_norm(x.double().cpu(), w.double().cpu(), groups, 1e-5)
    assert torch.allclose(hn.double().cpu(), want, atol=1e-5, rtol=1e-5)
    assert torch.allclose(he.double().cpu(), want, atol=2e-2, rtol=1e-2)
    if groups > 1:
        assert not torch.allclose(want, R.grouped_rms_norm(x.double().cpu(), w.double().cpu(), 1, 1e-5), atol=1e-2)


def test_side_by_side_residual_add_and_loop_entry_rows():
    from dli_b200 import ops

    torch.manual_seed(0)
    x, h = torch.randn(5, 24, device=DEV), torch.randn(5, 24, device=DEV)
    y1, y2, a = torch.randn(5, 24, device=DEV), torch.randn(5, 24, device=DEV), torch.rand(5, device=DEV)
    want = x + y1 + y2 + a[:, None] * h
    got = ops.residual_add2(x.clone(), y1, y2, a, h)
    assert torch.allclose(got, want, atol=1e-6)
    assert torch.allclose(ops.residual_add2(x.clone(), y1), x + y1, atol=1e-6)
    cat = torch.empty(5, 48, device=DEV)
    ops.concat_cast(x, h, cat)
    assert torch.equal(cat, torch.cat((x, h), 1))
    out = torch.empty_like(x)
    ops.rows_bias_f32(y1, a.repeat(5)[:24].contiguous(), out)
    assert torch.allclose(out, y1 + a.repeat(5)[:24], atol=1e-6)


@pytest.mark.parametrize("cuts", [[300], [3, 2, 61, 100], [250]])
def test_latent_attention_sharp_scores_over_hundreds_of_keys(cuts):
    """scale 6: nearly every query gives most of its weight to one key, wherever among the <= 300 earlier positions it
    lies (pages of 4 positions); one position off, a wrong page or a missing rotation picks another key."""
    L = latent(heads=2, dim=6, rot_dim=8, vdim=10, kv_rank=16, q_rank=12, scale=6.0, base=50.0)
    eng, cfg, sd = one_layer_engine(L)
    m = cfg["layers"][0]["mixer"]
    P = R.sub(sd, "l0.mix.")
    torch.manual_seed(1)
    T = 300
    h = torch.randn(T, 32, dtype=torch.float64)
    u = torch.cat((h @ P["dq"].T, h @ P["dkv"].T, h @ P["g"].T), 1)
    want = R.latent_attention(h, P, m, 1e-5)
    got = run_mixer(eng, "latent_attention", u, cuts) @ P["o"].T
    assert (got - want).abs().max() < 1e-4 * want.abs().max()
    # the test is sharp: without the rotated part the result differs grossly
    m2 = dict(m, rot=dict(m["rot"], base=1e9))
    assert (R.latent_attention(h, P, m2, 1e-5) - want).abs().max() > 0.05 * want.abs().max()


@pytest.mark.parametrize("cuts", [[120], [1, 2, 3, 50], [64, 2], [5, 115]])
def test_state_space_mixer_with_slow_forgetting(cuts):
    """A_log very negative: the state forgets over hundreds of tokens, so the last outputs carry the first inputs; the
    slot holds garbage before (state and convolution history)."""
    L = mamba(heads=3, vdim=8, state=20, groups=1, norm_groups=2, conv=4)
    eng, cfg, sd = one_layer_engine(L)
    sd["l0.mix.A_log"] = torch.full((3,), -5.0).to(torch.bfloat16)
    sd["l0.mix.dt_bias"] = torch.tensor([-1.0, 0.0, 2.0]).to(torch.bfloat16)
    from dli_b200 import togalorn
    eng.load_tensors(togalorn.model_tensors(eng.spec, sd))
    for t in eng.slots.tensors.values():
        t.fill_(1e4)
    m = cfg["layers"][0]["mixer"]
    P = R.sub(sd, "l0.mix.")
    torch.manual_seed(2)
    T = 120
    h = torch.randn(T, 32, dtype=torch.float64)
    u = h @ P["in"].T
    want = R.mamba2(h, P, m, 1e-5)
    got = run_mixer(eng, "mamba2", u, cuts) @ P["o"].T
    assert (got - want).abs().max() < 1e-4 * want.abs().max()
    # sharp: dropping the first 20 inputs changes the last output
    h2 = h.clone()
    h2[:20] = 0
    assert (R.mamba2(h2, P, m, 1e-5)[-1] - want[-1]).abs().max() > 1e-3 * want.abs().max()


@pytest.mark.parametrize("experts,identity,top,shared", [(4, 2, 2, (16, 0.8)), (3, 0, 1, None), (2, 3, 4, (8, 2.0)), (5, 1, 6, None)])
def test_mixture_of_experts(experts, identity, top, shared):
    """Router (softmax over all outputs, choice by score + correction, weights from the scores alone), clamped gated
    experts, pass-through experts and the shared expert against the oracle; the correction is large enough to change
    the choice."""
    from dli_b200 import ops

    mlp = moe(experts=experts, identity=identity, top=top, ff=24, limit=0.7, shared=shared)
    eng, cfg, sd = one_layer_engine(mamba(), mlp)
    n_out = experts + identity
    sd["l0.mlp.correction"] = (torch.arange(n_out) % 3 * 0.3).to(torch.bfloat16)
    from dli_b200 import togalorn
    eng.load_tensors(togalorn.model_tensors(eng.spec, sd))
    P, Pr = eng.layers[0], R.sub(sd, "l0.mlp.")
    torch.manual_seed(3)
    rows, W = 37, 32
    h = torch.randn(rows, W, device=DEV)
    wts, idw = torch.empty(rows, experts, device=DEV), torch.empty(rows, device=DEV)
    si, sw = torch.empty(rows, top, dtype=torch.int32, device=DEV), torch.empty(rows, top, device=DEV)
    ops.moe_route(h, P["w_router"], P["corr"], wts, idw, si, sw, experts, top)
    s = torch.softmax(h.double().cpu() @ Pr["router"].T, -1)
    choice = torch.topk(s + Pr["correction"], top).indices
    assert torch.equal(si.cpu().sort(-1).values.long(), choice.sort(-1).values)
    if top < n_out:  # the correction changes the choice
        assert not torch.equal(choice.sort(-1).values, torch.topk(s, top).indices.sort(-1).values)
    gu = torch.empty(rows, P["w_gu"].shape[0], device=DEV)
    ops.linear_any(h, P["w_gu"], gu)
    e = eng.spec.layers[0].moe
    act = torch.empty(rows, e.total_ff, device=DEV)
    ops.moe_act(gu, wts, act, e.experts, e.ff, e.limit, e.shared_ff, e.shared_limit, e.alpha)
    y = torch.empty(rows, W, device=DEV)
    ops.linear_any(act, P["w_down"], y)
    got = y.double().cpu() + idw.double().cpu()[:, None] * h.double().cpu()
    want = R.moe(h.double().cpu(), Pr, mlp)
    assert (got - want).abs().max() < 1e-4 * want.abs().max()


@pytest.mark.parametrize("experts,identity,top,shared", [(4, 2, 2, (16, 0.8)), (3, 0, 1, None), (2, 3, 4, (8, 2.0))])
def test_chosen_experts_only_path_of_decode_rows(experts, identity, top, shared):
    """bfloat16 decode rows read only the chosen experts' weights: same result as the path over all experts (both round
    the projections' outputs to bfloat16) and as the oracle."""
    from dli_b200 import ops, togalorn
    from dli_b200.ragged_engine import RaggedEngine

    mlp = moe(experts=experts, identity=identity, top=top, ff=24, limit=0.7, shared=shared)
    cfg = config([(mamba(), mlp)], width=32, groups=2)
    spec = togalorn.spec_from_config(cfg)
    sd = togalorn.random_state_dict(spec, seed=5, std=0.3)
    eng = RaggedEngine(spec, max_batch=4, max_seq_len=64, page_size=4, dtype=torch.bfloat16)
    eng.load_tensors(togalorn.model_tensors(spec, sd))
    P, Pr, e = eng.layers[0], R.sub(sd, "l0.mlp."), spec.layers[0].moe
    assert ops.moe_sel_supported(32, e.ff, e.shared_ff, e.top)
    torch.manual_seed(4)
    rows = 5
    h = torch.randn(rows, 32, device=DEV)
    he = h.to(torch.bfloat16)
    wts, idw = torch.empty(rows, experts, device=DEV), torch.empty(rows, device=DEV)
    si, sw = torch.empty(rows, top, dtype=torch.int32, device=DEV), torch.empty(rows, top, device=DEV)
    ops.moe_route(h, P["w_router"], P["corr"], wts, idw, si, sw, experts, top)
    act_sel = torch.empty(rows, top * e.ff + e.shared_ff, dtype=torch.bfloat16, device=DEV)
    y = torch.empty(rows, 32, dtype=torch.bfloat16, device=DEV)
    ops.moe_sel(he, P["w_gu"], P["w_down"], si, sw, act_sel, y, e.experts, e.top, e.ff, e.limit, e.shared_ff, e.shared_limit)
    gu = torch.empty(rows, P["w_gu"].shape[0], dtype=torch.bfloat16, device=DEV)
    ops.linear_any(he, P["w_gu"], gu)
    act = torch.empty(rows, e.total_ff, dtype=torch.bfloat16, device=DEV)
    ops.moe_act(gu, wts, act, e.experts, e.ff, e.limit, e.shared_ff, e.shared_limit, e.alpha)
    y_all = torch.empty(rows, 32, dtype=torch.bfloat16, device=DEV)
    ops.linear_any(act, P["w_down"], y_all)
    scale = y_all.float().abs().max()
    assert (y.float() - y_all.float()).abs().max() <= 0.02 * scale
    got = y.double().cpu() + idw.double().cpu()[:, None] * he.double().cpu()
    want = R.moe(he.double().cpu(), Pr, mlp)
    assert (got - want).abs().max() < 0.03 * want.abs().max()
