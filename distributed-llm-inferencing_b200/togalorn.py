"""The Togalorn design: a decoder whose layers are listed in config.json, each a latent-attention mixer or a
state-space (Mamba-2) mixer that reads the layer's one grouped RMS norm through a short causal convolution, with a
mixture-of-experts feed-forward reading the same norm beside it (x += mixer + feed-forward).  A range of layers may
run several times in a row with the same weights; every pass has caches and states of its own and starts from a
projection of [x | embedding output] plus a per-pass vector.  This module is the model definition only — the
configuration reader, the checkpoint's tensor names and synthetic weights; the step function, caches and kernels
are ragged_engine.RaggedEngine's.

config.json keys read here: architecture, vocab, width, embedding.scale, norm {eps, groups}, canon.taps,
loop {start, stop, times}, layers[] with type, mlp (null or {kind: moe, expert {ff, limit}, router {experts,
identity, top}, shared {ff, limit}}) and mixer: latent_attention {heads, dim, rot_dim, vdim, kv_rank, q_rank, scale,
rot {base, dims}}, mamba2 {heads, vdim, state, groups, norm_groups, conv}.
Tensor names: embed, head, final.norm, loop.in [width, 2 width], loop.step [times, width], l<i>.norm1 [width],
l<i>.canon1 [width, taps]; latent attention l<i>.mix.{dq, dq.norm, uq, dkv, dkv.norm, uk, uv, g, o}; mamba2
l<i>.mix.{in, conv, conv.b, dt_bias, A_log, D, norm, o}; l<i>.mlp.{router, correction, e<k>.{gate,up,down},
shared.{gate,up,down}}.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from .ragged_engine import HybridSpec, LayerSpec, MixerSpec, MoESpec

ARCHITECTURE = "Togalorn"
EXPERT_ALPHA = 1.702  # g * sigmoid(alpha * g) in the experts


def _mixer(i: int, L: dict) -> MixerSpec:
    m = L["mixer"]
    if L["type"] == "latent_attention":
        rot = m.get("rot") or {}
        rd = int(m.get("rot_dim", 0))
        if rd and int(rot.get("dims", rd)) != rd:
            raise ValueError(f"layer {i}: rot.dims {rot.get('dims')} differs from rot_dim {rd}")
        return MixerSpec(kind="latent_attention", heads=int(m["heads"]), kv_heads=1, dim=int(m["dim"]), vdim=int(m["vdim"]),
                         scale=float(m["scale"]), rot_dims=rd, rot_base=float(rot.get("base", 10000.0)),
                         kv_rank=int(m["kv_rank"]), q_rank=int(m["q_rank"]), out_gate=True)
    if L["type"] == "mamba2":
        return MixerSpec(kind="mamba2", heads=int(m["heads"]), kv_heads=int(m["heads"]), dim=0, vdim=int(m["vdim"]),
                         state=int(m["state"]), groups=int(m.get("groups", 1)), norm_groups=int(m.get("norm_groups", 1)),
                         conv_taps=int(m["conv"]))
    raise ValueError(f"layer {i}: unknown mixer type {L['type']!r}")


def _moe(i: int, mlp) -> MoESpec:
    if mlp is None:
        return None
    if mlp.get("kind") != "moe":
        raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
    r, sh = mlp["router"], mlp.get("shared")
    return MoESpec(experts=int(r["experts"]), identity=int(r.get("identity", 0)), top=int(r["top"]),
                   ff=int(mlp["expert"]["ff"]), limit=float(mlp["expert"]["limit"]),
                   shared_ff=int(sh["ff"]) if sh else 0, shared_limit=float(sh["limit"]) if sh else 0.0, alpha=EXPERT_ALPHA)


def spec_from_config(cfg: dict) -> HybridSpec:
    """The layer RUNS in order: a looped range appears once per pass, later passes naming the first pass's run as the
    owner of their weights (`weights_of`) and `ckpt` the checkpoint's layer; `reenter` marks the first run of a pass."""
    if cfg.get("architecture") != ARCHITECTURE:
        raise ValueError(f"not a {ARCHITECTURE} config")
    n = len(cfg["layers"])
    lp = cfg.get("loop")
    a, b, times = (int(lp["start"]), int(lp["stop"]), int(lp["times"])) if lp else (0, 0, 0)
    if lp and not (0 <= a < b <= n and times >= 1):
        raise ValueError(f"loop {lp} does not fit {n} layers")
    order = [(i, None) for i in range(a)]
    for t in range(times):
        order += [(i, t) for i in range(a, b)]
    order += [(i, None) for i in range(b, n)]
    first_run: Dict[int, int] = {}
    layers: List[LayerSpec] = []
    for run, (i, t) in enumerate(order):
        L = cfg["layers"][i]
        layers.append(LayerSpec(mixer=_mixer(i, L), moe=_moe(i, L.get("mlp")), parallel=True, ckpt=i,
                                weights_of=first_run.get(i), reenter=t if (t is not None and i == a) else None))
        first_run.setdefault(i, run)
    return HybridSpec(arch="togalorn", vocab=int(cfg["vocab"]), width=int(cfg["width"]), eps=float(cfg["norm"]["eps"]),
                      taps=int(cfg["canon"]["taps"]), layers=layers, embed_scale=float(cfg["embedding"]["scale"]),
                      norm_groups=int(cfg["norm"]["groups"]), loop_passes=times)


def layer_tensors(spec: HybridSpec, sd: Dict[str, torch.Tensor], run: int) -> dict:
    """The checkpoint's tensors of layer run `run` under the names the engine uses."""
    L = spec.layers[run]
    p = f"l{L.ckpt}."
    out = {"norm1": sd[p + "norm1"], "canon1": sd[p + "canon1"], "o": sd[p + "mix.o"]}
    if L.mixer.kind == "latent_attention":
        for k in ("dq", "uq", "dkv", "uk", "uv", "g"):
            out[k] = sd[p + "mix." + k]
        out.update(dq_norm=sd[p + "mix.dq.norm"], dkv_norm=sd[p + "mix.dkv.norm"])
    else:
        out.update({"in": sd[p + "mix.in"], "conv": sd[p + "mix.conv"], "conv_b": sd[p + "mix.conv.b"],
                    "dt_bias": sd[p + "mix.dt_bias"], "A_log": sd[p + "mix.A_log"], "D": sd[p + "mix.D"],
                    "out_norm": sd[p + "mix.norm"]})
    if L.moe is not None:
        q = p + "mlp."
        out.update(router=sd[q + "router"], correction=sd[q + "correction"],
                   experts=[(sd[f"{q}e{k}.gate"], sd[f"{q}e{k}.up"], sd[f"{q}e{k}.down"]) for k in range(L.moe.experts)],
                   shared=(sd[q + "shared.gate"], sd[q + "shared.up"], sd[q + "shared.down"]) if L.moe.shared_ff else None)
    return out


def model_tensors(spec: HybridSpec, sd: Dict[str, torch.Tensor]) -> dict:
    out = {"embed": sd["embed"], "head": sd["head"], "final_norm": sd["final.norm"],
           "layers": {i: layer_tensors(spec, sd, i) for i, L in enumerate(spec.layers) if L.weights_of is None}}
    if spec.loop_passes:
        out.update(loop_in=sd["loop.in"], loop_step=sd["loop.step"])
    return out


def random_state_dict(spec: HybridSpec, seed: int = 0, std: float = 0.05, device="cpu") -> Dict[str, torch.Tensor]:
    """Synthetic weights under the checkpoint's names (benchmarks and tests; there are no checkpoints offline)."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    W = spec.width

    def n(*shape, s=std, mean=0.0):
        return (mean + s * torch.randn(tuple(shape), generator=g)).to(torch.bfloat16).to(device)

    sd = {"embed": n(spec.vocab, W, s=1.0 / max(spec.embed_scale, 1e-6)), "head": n(spec.vocab, W),
          "final.norm": n(W, mean=1.0, s=0.1)}
    if spec.loop_passes:
        sd["loop.in"] = torch.cat((n(W, W, s=0.7 / W ** 0.5) + torch.eye(W).to(torch.bfloat16).to(device) * 0.5,
                                   n(W, W, s=0.7 / W ** 0.5)), dim=1).contiguous()
        sd["loop.step"] = n(spec.loop_passes, W, s=0.1)
    for L in spec.layers:
        if L.weights_of is not None:
            continue
        m, p = L.mixer, f"l{L.ckpt}."
        sd[p + "norm1"] = n(W, mean=1.0, s=0.1)
        sd[p + "canon1"] = n(W, spec.taps, s=0.2)
        if m.kind == "latent_attention":
            H, D, R, V, K, Q = m.heads, m.dim, m.rot_dims, m.vdim, m.kv_rank, m.q_rank
            sd[p + "mix.dq"], sd[p + "mix.dq.norm"] = n(Q, W), n(Q, mean=1.0, s=0.1)
            sd[p + "mix.uq"] = n(H * (D + R), Q, s=1.0 / Q ** 0.5)
            sd[p + "mix.dkv"], sd[p + "mix.dkv.norm"] = n(K + R, W), n(K, mean=1.0, s=0.1)
            sd[p + "mix.uk"], sd[p + "mix.uv"] = n(H * D, K, s=1.0 / K ** 0.5), n(H * V, K, s=1.0 / K ** 0.5)
            sd[p + "mix.g"], sd[p + "mix.o"] = n(H * V, W), n(W, H * V)
        else:
            inner, gn = m.heads * m.vdim, m.groups * m.state
            sd[p + "mix.in"] = n(2 * inner + 2 * gn + m.heads, W)
            sd[p + "mix.conv"], sd[p + "mix.conv.b"] = n(inner + 2 * gn, m.conv_taps, s=0.3), n(inner + 2 * gn, s=0.1)
            sd[p + "mix.dt_bias"], sd[p + "mix.A_log"] = n(m.heads, mean=-1.0, s=1.0), n(m.heads, mean=0.0, s=0.7)
            sd[p + "mix.D"], sd[p + "mix.norm"] = n(m.heads, mean=1.0, s=0.3), n(inner, mean=1.0, s=0.1)
            sd[p + "mix.o"] = n(W, inner)
        if L.moe is not None:
            e, q = L.moe, p + "mlp."
            sd[q + "router"], sd[q + "correction"] = n(e.experts + e.identity, W, s=0.5), n(e.experts + e.identity, s=0.05)
            for k in range(e.experts):
                sd[f"{q}e{k}.gate"], sd[f"{q}e{k}.up"], sd[f"{q}e{k}.down"] = n(e.ff, W), n(e.ff, W), n(W, e.ff)
            if e.shared_ff:
                sd[q + "shared.gate"], sd[q + "shared.up"] = n(e.shared_ff, W), n(e.shared_ff, W)
                sd[q + "shared.down"] = n(W, e.shared_ff)
    return sd
