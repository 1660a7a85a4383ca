"""Plain, slow float64 reference of the layer-by-layer decoder family (Sokevik), one function per mechanism.

Whole sequences only, no cache, no batching, no kernels: every function takes the full [T, ...] input of ONE
sequence and loops where a loop is the clearest form.  The GPU tests compare the engine — whatever way it cuts a
sequence into steps, batches, pages and slots — with these.  Nothing here is imported by the product.

Notation: x residual stream [T, W]; h the input of a sublayer; P a dict of float64 tensors under the checkpoint's
names; cfg the config.json dict.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last dim."""
    return x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)


def causal_conv(h, w):
    """y[t, c] = sum_j w[c, j] * h[t - (taps - 1) + j, c], rows before the start are zero."""
    T, W = h.shape
    taps = w.shape[1]
    y = torch.zeros_like(h)
    for t in range(T):
        for j in range(taps):
            src = t - (taps - 1) + j
            if src >= 0:
                y[t] += w[:, j] * h[src]
    return y


def frequencies(base, dims, scaling=None):
    out = []
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if scaling:
            wavelength = 2.0 * math.pi / f
            short, long_ = scaling["original"] / scaling["high"], scaling["original"] / scaling["low"]
            if wavelength > long_:
                f = f / scaling["factor"]
            elif wavelength >= short:
                s = (scaling["original"] / wavelength - scaling["low"]) / (scaling["high"] - scaling["low"])
                f = (1.0 - s) * f / scaling["factor"] + s * f
        out.append(f)
    return torch.tensor(out, dtype=F64)


def turn_pairs(x, angle):
    """Rotate the pairs (x[..., 2i], x[..., 2i+1]) by angle[..., i]."""
    y = x.clone()
    a, b = x[..., 0::2], x[..., 1::2]
    y[..., 0::2] = a * torch.cos(angle) - b * torch.sin(angle)
    y[..., 1::2] = b * torch.cos(angle) + a * torch.sin(angle)
    return y


def visible(i, j, chunk=0, window=0):
    if j > i:
        return False
    if chunk and i // chunk != j // chunk:
        return False
    if window and j <= i - window:
        return False
    return True


def attention_mixer(h, P, pre, m, eps):
    T = h.shape[0]
    H, G, D, V = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m["vdim"]
    q = (h @ P[pre + "q"].T).reshape(T, H, D)
    k = (h @ P[pre + "k"].T).reshape(T, G, D)
    v = (h @ P[pre + "v"].T).reshape(T, G, V)
    q = rms_unit(q, eps) * P[pre + "q.norm"]
    k = rms_unit(k, eps) * P[pre + "k.norm"]
    rot = m.get("rot")
    pos = torch.arange(T, dtype=F64)
    if rot:
        rd = rot["dims"]
        ang = pos[:, None, None] * frequencies(rot["base"], rd, rot.get("scaling"))[None, None, :]
        q = torch.cat((turn_pairs(q[..., :rd], ang), q[..., rd:]), dim=-1)
        k = torch.cat((turn_pairs(k[..., :rd], ang), k[..., rd:]), dim=-1)
        ang_v = pos[:, None, None] * frequencies(rot["base"], V)[None, None, :]
        v = turn_pairs(v, ang_v)
    chunk = (m.get("mask") or {}).get("size", 0)
    out = torch.zeros(T, H, V, dtype=F64)
    for hh in range(H):
        g = hh // (H // G)
        sink = P[pre + "sink"][hh]
        for i in range(T):
            js = [j for j in range(i + 1) if visible(i, j, chunk)]
            s = torch.stack([(q[i, hh] * k[j, g]).sum() * m["scale"] for j in js])
            top = torch.maximum(s.max(), sink)
            w = torch.exp(s - top)
            den = w.sum() + torch.exp(sink - top)
            out[i, hh] = (w[:, None] * v[js, g]).sum(dim=0) / den
    if rot:
        out = turn_pairs(out, -ang_v)
    gate = torch.sigmoid(h @ P[pre + "g"].T)
    out = out * gate[:, :, None]
    return out.reshape(T, H * V) @ P[pre + "o"].T


def soft_cap(x, cap):
    return cap * torch.tanh(x / cap)


def mlstm_mixer(h, P, pre, m, eps):
    T = h.shape[0]
    H, D, V, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = (h @ P[pre + "q"].T).reshape(T, H, D) / math.sqrt(D)
    k = (h @ P[pre + "k"].T).reshape(T, H, D)
    v = (h @ P[pre + "v"].T).reshape(T, H, V)
    log_i = soft_cap(h @ P[pre + "i"].T + P[pre + "i.b"], cap)
    log_f = torch.nn.functional.logsigmoid(soft_cap(h @ P[pre + "f"].T + P[pre + "f.b"], cap))
    out = torch.zeros(T, H, V, dtype=F64)
    for hh in range(H):
        S = torch.zeros(D, V, dtype=F64)
        n = torch.zeros(D, dtype=F64)
        m_run = torch.tensor(0.0, dtype=F64)
        for t in range(T):
            m_new = torch.maximum(log_f[t, hh] + m_run, log_i[t, hh])
            keep, take = torch.exp(log_f[t, hh] + m_run - m_new), torch.exp(log_i[t, hh] - m_new)
            S = keep * S + take * torch.outer(k[t, hh], v[t, hh])
            n = keep * n + take * k[t, hh]
            m_run = m_new
            den = torch.maximum((n * q[t, hh]).sum().abs(), torch.exp(-m_run)) + 1e-6
            out[t, hh] = (S.T @ q[t, hh]) / den
    out = rms_unit(out, eps).reshape(T, H * V) * P[pre + "norm"]
    out = out * torch.sigmoid(h @ P[pre + "g"].T)
    return out @ P[pre + "o"].T


def feed_forward(h, P, pre):
    a = h @ P[pre + "gate"].T
    return (a * torch.sigmoid(a) * (h @ P[pre + "up"].T)) @ P[pre + "down"].T


def forward(cfg, P, tokens, layers_out=None):
    """tokens: list of ints of ONE sequence -> float64 logits [T, vocab]."""
    eps = cfg["norm"]["eps"]
    P = {k: v.to(F64) for k, v in P.items()}
    x = P["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    for i, L in enumerate(cfg["layers"]):
        p = "l%d." % L.get("weights_of", i)
        h = rms_unit(x, eps) * P[p + "norm1"]
        h = h + causal_conv(h, P[p + "canon1"])
        mixer = attention_mixer if L["type"] == "attention" else mlstm_mixer
        x = x + rms_unit(mixer(h, P, p + "mix.", L["mixer"], eps), eps) * P[p + "norm1b"]
        if L.get("mlp"):
            h = rms_unit(x, eps) * P[p + "norm2"]
            h = h + causal_conv(h, P[p + "canon2"])
            x = x + rms_unit(feed_forward(h, P, p + "mlp."), eps) * P[p + "norm2b"]
        if layers_out is not None:
            layers_out.append(x.clone())
    return (rms_unit(x, eps) * P["final.norm"]) @ P["head"].T


def greedy(cfg, P, prompt, n_new):
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(forward(cfg, P, toks)[-1].argmax()))
    return toks
