"""Plain restatement of the Togalorn design in float64: whole sequences, Python loops, one function per mechanism.

It is the oracle of the tests and imports nothing of the product.  A model is (cfg, sd): the dictionary of
config.json and the tensors under the checkpoint's names.  Notation: T tokens, W width, lists of positions are
0-based per sequence.
"""
from __future__ import annotations

import math
from typing import Dict, List, Tuple

import torch

F64 = torch.float64


def grouped_rms_norm(x: torch.Tensor, w: torch.Tensor, groups: int, eps: float) -> torch.Tensor:
    """x [..., n] cut into `groups` consecutive parts, each divided by sqrt(mean(part^2) + eps); then times w."""
    shp = x.shape
    p = x.reshape(*shp[:-1], groups, shp[-1] // groups)
    p = p / torch.sqrt((p * p).mean(-1, keepdim=True) + eps)
    return p.reshape(shp) * w


def causal_conv(h: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """h [T, C], w [C, taps]: out_t = sum_j w[:, j] * h_(t - taps + 1 + j), zero before the start."""
    T, taps = h.shape[0], w.shape[1]
    out = torch.zeros_like(h)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += w[:, j] * h[s]
    return out


def rotate_pairs(v: torch.Tensor, pos: int, base: float, dims: int) -> torch.Tensor:
    """The first `dims` entries of v as pairs (2i, 2i+1), each turned by pos * base^(-2i/dims)."""
    out = v.clone()
    for i in range(dims // 2):
        a = pos * base ** (-2.0 * i / dims)
        u, w = v[2 * i], v[2 * i + 1]
        out[2 * i] = u * math.cos(a) - w * math.sin(a)
        out[2 * i + 1] = w * math.cos(a) + u * math.sin(a)
    return out


def softplus(x):
    return torch.where(x > 30, x, torch.log1p(torch.exp(torch.clamp(x, max=30))))


def silu(x):
    return x * torch.sigmoid(x)


def latent_attention(h: torch.Tensor, P: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    """h [T, W] -> [T, W].  P: dq, dq.norm, uq, dkv, dkv.norm, uk, uv, g, o."""
    T = h.shape[0]
    H, D, R, V, K = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    base, rdims = float(m["rot"]["base"]), int(m["rot"]["dims"])
    cq = grouped_rms_norm(h @ P["dq"].T, P["dq.norm"], 1, eps)
    q = (cq @ P["uq"].T).reshape(T, H, D + R)
    kv = h @ P["dkv"].T
    c = grouped_rms_norm(kv[:, :K], P["dkv.norm"], 1, eps)
    kr = torch.stack([rotate_pairs(kv[t, K:], t, base, rdims) for t in range(T)])
    kn = (c @ P["uk"].T).reshape(T, H, D)
    v = (c @ P["uv"].T).reshape(T, H, V)
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for t in range(T):
        for hh in range(H):
            qr = rotate_pairs(q[t, hh, D:], t, base, rdims)
            s = (kn[:t + 1, hh] @ q[t, hh, :D] + kr[:t + 1] @ qr) * m["scale"]
            p = torch.softmax(s, 0)
            out[t, hh] = p @ v[:t + 1, hh]
    gate = torch.sigmoid(h @ P["g"].T)
    return (out.reshape(T, H * V) * gate) @ P["o"].T


def mamba2(h: torch.Tensor, P: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    """h [T, W] -> [T, W].  P: in, conv, conv.b, dt_bias, A_log, D, norm, o."""
    T = h.shape[0]
    H, V, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * V
    u = h @ P["in"].T
    z, xbc, dt = u[:, :inner], u[:, inner:2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, P["conv"]) + P["conv.b"])
    x = xbc[:, :inner].reshape(T, H, V)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + P["dt_bias"])
    y = torch.zeros(T, H, V, dtype=h.dtype)
    for hh in range(H):
        g = hh // (H // G)
        S = torch.zeros(N, V, dtype=h.dtype)
        for t in range(T):
            S = torch.exp(-torch.exp(P["A_log"][hh]) * dt[t, hh]) * S + dt[t, hh] * torch.outer(B[t, g], x[t, hh])
            y[t, hh] = S.T @ C[t, g] + P["D"][hh] * x[t, hh]
    y = y.reshape(T, inner) * silu(z)
    return grouped_rms_norm(y, P["norm"], m["norm_groups"], eps) @ P["o"].T


def expert(h: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor, limit: float) -> torch.Tensor:
    g = torch.clamp(h @ gate.T, max=limit)
    u = torch.clamp(h @ up.T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def moe(h: torch.Tensor, P: Dict[str, torch.Tensor], mlp: dict) -> torch.Tensor:
    """h [T, W] -> [T, W].  P: router, correction, e<k>.gate/up/down, shared.gate/up/down."""
    r = mlp["router"]
    E, I, top = int(r["experts"]), int(r.get("identity", 0)), int(r["top"])
    s = torch.softmax(h @ P["router"].T, -1)
    choice = s + P["correction"]
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        idx = torch.topk(choice[t], top).indices.tolist()
        wsum = sum(s[t, k] for k in idx) + 1e-20
        for k in idx:
            if k >= E:
                assert k < E + I
                y = h[t]
            else:
                y = expert(h[t:t + 1], P[f"e{k}.gate"], P[f"e{k}.up"], P[f"e{k}.down"], float(mlp["expert"]["limit"]))[0]
            out[t] += s[t, k] / wsum * y
    if mlp.get("shared"):
        out = out + expert(h, P["shared.gate"], P["shared.up"], P["shared.down"], float(mlp["shared"]["limit"]))
    return out


def sub(sd: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v.to(F64) for k, v in sd.items() if k.startswith(prefix)}


def layer_runs(cfg: dict) -> List[Tuple[int, int]]:
    """(layer, pass) for every layer run in order; pass = -1 outside the loop, else the number of the pass."""
    n = len(cfg["layers"])
    lp = cfg.get("loop")
    if not lp:
        return [(i, -1) for i in range(n)]
    a, b, times = int(lp["start"]), int(lp["stop"]), int(lp["times"])
    runs = [(i, -1) for i in range(a)]
    for t in range(times):
        runs += [(i, t) for i in range(a, b)]
    return runs + [(i, -1) for i in range(b, n)]


def forward(cfg: dict, sd: Dict[str, torch.Tensor], tokens: List[int]):
    """-> logits [T, vocab], the residual stream after every layer run [runs, T, W]."""
    eps, groups = float(cfg["norm"]["eps"]), int(cfg["norm"]["groups"])
    x0 = sd["embed"].to(F64)[torch.tensor(tokens)] * float(cfg["embedding"]["scale"])
    x = x0.clone()
    trace = []
    lp = cfg.get("loop")
    for li, t in layer_runs(cfg):
        L = cfg["layers"][li]
        if t >= 0 and li == int(lp["start"]):
            x = torch.cat((x, x0), -1) @ sd["loop.in"].to(F64).T + sd["loop.step"].to(F64)[t]
        p = f"l{li}."
        h = grouped_rms_norm(x, sd[p + "norm1"].to(F64), groups, eps)
        hm = h + causal_conv(h, sd[p + "canon1"].to(F64))
        if L["type"] == "latent_attention":
            y = latent_attention(hm, sub(sd, p + "mix."), L["mixer"], eps)
        elif L["type"] == "mamba2":
            y = mamba2(hm, sub(sd, p + "mix."), L["mixer"], eps)
        else:
            raise ValueError(L["type"])
        if L.get("mlp"):
            y = y + moe(h, sub(sd, p + "mlp."), L["mlp"])
        x = x + y
        trace.append(x.clone())
    hf = grouped_rms_norm(x, sd["final.norm"].to(F64), groups, eps)
    return hf @ sd["head"].to(F64).T, torch.stack(trace)


def greedy(cfg: dict, sd: Dict[str, torch.Tensor], prompt: List[int], n_new: int) -> List[int]:
    """The prompt followed by n_new tokens, each the argmax of the logits at the last position."""
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(forward(cfg, sd, toks)[0][-1].argmax()))
    return toks
