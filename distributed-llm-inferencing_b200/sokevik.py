"""The Sokevik design: a decoder whose layers are listed one by one in config.json, each an attention mixer or a
matrix-memory recurrent mixer (mLSTM), optionally followed by a gated feed-forward, some layers sharing another
layer's weights.  This module is the model definition only — the configuration reader, the checkpoint's tensor
names and synthetic weights; the step function, caches and kernels are ragged_engine.RaggedEngine's.

config.json keys read here: architecture, vocab, width, norm.eps, canon.taps, layers[] with type, weights_of,
mlp (null or {kind: dense, ff}) and mixer: attention {heads, kv_heads, dim, vdim, scale, mask.size,
rot {base, dims, scaling {factor, low, high, original}}}, mlstm {heads, dim, vdim, gate_cap}.
Tensor names: embed, head, final.norm, l<i>.norm1 / norm1b / norm2 / norm2b (one number each), l<i>.canon1 /
canon2 [width, taps], l<i>.mix.{q,k,v,g,o}, attention: .q.norm, .k.norm, .sink; mlstm: .norm, .i, .i.b, .f, .f.b;
l<i>.mlp.{gate,up,down}.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from .ragged_engine import HybridSpec, LayerSpec, MixerSpec

ARCHITECTURE = "Sokevik"


def spec_from_config(cfg: dict) -> HybridSpec:
    if cfg.get("architecture") != ARCHITECTURE:
        raise ValueError(f"not a {ARCHITECTURE} config")
    layers: List[LayerSpec] = []
    for i, L in enumerate(cfg["layers"]):
        m = L["mixer"]
        if L["type"] == "attention":
            rot = m.get("rot") or {}
            mask = m.get("mask") or {}
            mx = MixerSpec(kind="attention", heads=int(m["heads"]), kv_heads=int(m.get("kv_heads", m["heads"])),
                           dim=int(m["dim"]), vdim=int(m["vdim"]), scale=float(m["scale"]),
                           rot_dims=int(rot.get("dims", 0)), rot_base=float(rot.get("base", 10000.0)),
                           rot_scaling=dict(rot["scaling"]) if rot.get("scaling") else None,
                           chunk=int(mask.get("size", 0)), qk_norm=True, rotate_values=bool(rot), sink=True,
                           head_gate=True)
        elif L["type"] == "mlstm":
            mx = MixerSpec(kind="mlstm", heads=int(m["heads"]), kv_heads=int(m["heads"]), dim=int(m["dim"]),
                           vdim=int(m["vdim"]), gate_cap=float(m["gate_cap"]))
        else:
            raise ValueError(f"layer {i}: unknown mixer type {L['type']!r}")
        mlp = L.get("mlp")
        if mlp is not None and mlp.get("kind", "dense") != "dense":
            raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
        layers.append(LayerSpec(mixer=mx, ff=int(mlp["ff"]) if mlp else 0, weights_of=L.get("weights_of")))
    return HybridSpec(arch="sokevik", vocab=int(cfg["vocab"]), width=int(cfg["width"]), eps=float(cfg["norm"]["eps"]),
                      taps=int(cfg["canon"]["taps"]), layers=layers)


def layer_tensors(spec: HybridSpec, sd: Dict[str, torch.Tensor], i: int) -> dict:
    """The checkpoint's tensors of layer i under the names the engine uses."""
    L = spec.layers[i]
    p = f"l{i}."
    out = {"norm1": sd[p + "norm1"], "norm1b": sd[p + "norm1b"], "canon1": sd[p + "canon1"]}
    for n in "qkvgo":
        out[n] = sd[p + "mix." + n]
    if L.mixer.kind == "attention":
        out.update(q_norm=sd[p + "mix.q.norm"], k_norm=sd[p + "mix.k.norm"], sink=sd[p + "mix.sink"])
    else:
        out.update(out_norm=sd[p + "mix.norm"], i=sd[p + "mix.i"], i_b=sd[p + "mix.i.b"], f=sd[p + "mix.f"],
                   f_b=sd[p + "mix.f.b"])
    if L.ff:
        out.update(norm2=sd[p + "norm2"], norm2b=sd[p + "norm2b"], canon2=sd[p + "canon2"], gate=sd[p + "mlp.gate"],
                   up=sd[p + "mlp.up"], down=sd[p + "mlp.down"])
    return out


def model_tensors(spec: HybridSpec, sd: Dict[str, torch.Tensor]) -> dict:
    return {"embed": sd["embed"], "head": sd["head"], "final_norm": sd["final.norm"],
            "layers": {i: layer_tensors(spec, sd, i) for i, L in enumerate(spec.layers) if L.weights_of is None}}


def random_state_dict(spec: HybridSpec, seed: int = 0, std: float = 0.05, device="cpu") -> Dict[str, torch.Tensor]:
    """Synthetic weights under the checkpoint's names (benchmarks and tests; there are no checkpoints offline)."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    W = spec.width

    def n(*shape, s=std, mean=0.0):
        return (mean + s * torch.randn(tuple(shape), generator=g)).to(torch.bfloat16).to(device)

    sd = {"embed": n(spec.vocab, W, s=1.0), "head": n(spec.vocab, W), "final.norm": n(mean=1.0, s=0.1)}
    for i, L in enumerate(spec.layers):
        if L.weights_of is not None:
            continue
        m, p = L.mixer, f"l{i}."
        sd[p + "norm1"], sd[p + "norm1b"] = n(mean=1.0, s=0.1), n(mean=1.0, s=0.1)
        sd[p + "canon1"] = n(W, spec.taps, s=0.2)
        if m.kind == "attention":
            sd[p + "mix.q"], sd[p + "mix.k"] = n(m.heads * m.dim, W), n(m.kv_heads * m.dim, W)
            sd[p + "mix.v"], sd[p + "mix.g"] = n(m.kv_heads * m.vdim, W), n(m.heads, W)
            sd[p + "mix.q.norm"], sd[p + "mix.k.norm"] = n(m.dim, mean=1.0, s=0.2), n(m.dim, mean=1.0, s=0.2)
            sd[p + "mix.sink"] = n(m.heads, s=1.0)
        else:
            sd[p + "mix.q"], sd[p + "mix.k"] = n(m.heads * m.dim, W), n(m.heads * m.dim, W)
            sd[p + "mix.v"], sd[p + "mix.g"] = n(m.heads * m.vdim, W), n(m.heads * m.vdim, W)
            sd[p + "mix.norm"] = n(m.heads * m.vdim, mean=1.0, s=0.2)
            sd[p + "mix.i"], sd[p + "mix.f"] = n(m.heads, W), n(m.heads, W)
            sd[p + "mix.i.b"], sd[p + "mix.f.b"] = n(m.heads, s=1.0), n(m.heads, mean=2.0, s=1.0)
        sd[p + "mix.o"] = n(W, m.heads * m.vdim)
        if L.ff:
            sd[p + "norm2"], sd[p + "norm2b"] = n(mean=1.0, s=0.1), n(mean=1.0, s=0.1)
            sd[p + "canon2"] = n(W, spec.taps, s=0.2)
            sd[p + "mlp.gate"], sd[p + "mlp.up"], sd[p + "mlp.down"] = n(L.ff, W), n(L.ff, W), n(W, L.ff)
    return sd
