"""RaggedEngine — a decoder whose layers are of different kinds, run on RAGGED steps.

ShardEngine (engine.py) serves uniform Llama / GPT-2 stacks on rectangular batches with a bf16 residual stream.
This engine serves stacks described layer by layer (HybridSpec): every layer has a token mixer — softmax attention
with its options, or a matrix-memory recurrent cell — and optionally a gated feed-forward; every sublayer is wrapped
in a pre-norm and a post-norm with one weight each and reads its input through a short causal convolution; layers
may share another layer's weights while keeping a cache / state of their own.  The residual stream, norms, rotation
angles, scores, softmax weights, convolution and recurrent state are fp32; projections run in the element type of the
engine (bf16 on the tcgen05 / GEMV kernels of ops.linear, or float32 on the CUDA-core GEMM).

One call of step() takes the NEXT TOKENS of any number of live sequences — a portion of a prompt of any length
beside single decoded tokens — as one batch: projections and feed-forwards run over all rows at once, attention
reads and extends the paged key/value cache (engine.PagedKVCache), recurrent layers and the input convolutions
read and advance the sequence's state slot (state_cache.StateSlots).  The result at a position does not depend
on how the sequence was cut into steps, on the other rows, or on the pages and slot it got, beyond rounding.
batching.RaggedBatcher schedules requests onto step(); generate() is that scheduler behind ShardEngine's signature.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from . import ops
from .engine import PagedKVCache
from .state_cache import StateSlots

BF = torch.bfloat16


@dataclass
class MixerSpec:
    kind: str                      # "attention" or "mlstm"
    heads: int
    kv_heads: int
    dim: int                       # query / key size per head
    vdim: int                      # value size per head
    # attention
    scale: float = 1.0
    rot_dims: int = 0              # leading dims of q / k that are rotated (interleaved pairs); 0 = none
    rot_base: float = 10000.0
    rot_scaling: Optional[dict] = None   # {factor, low, high, original}: wavelength-dependent frequency scaling
    chunk: int = 0                 # > 0: a position sees only its own block of `chunk` positions
    window: int = 0                # > 0: a position sees the last `window` positions
    qk_norm: bool = False
    rotate_values: bool = False    # values rotated by their position, outputs turned back by theirs
    sink: bool = False             # one extra softmax term per head without key or value
    head_gate: bool = False        # sigmoid gate per head on the output
    # mlstm
    gate_cap: float = 0.0


@dataclass
class LayerSpec:
    mixer: MixerSpec
    ff: int = 0                    # feed-forward size, 0 = no feed-forward sublayer
    weights_of: Optional[int] = None


@dataclass
class HybridSpec:
    arch: str
    vocab: int
    width: int
    eps: float
    taps: int                      # taps of the input convolutions (1: the current input only, no state)
    layers: List[LayerSpec] = field(default_factory=list)

    @property
    def n_layers(self) -> int:
        return len(self.layers)

    def source(self, i: int) -> int:
        j = self.layers[i].weights_of
        return i if j is None else j


def rot_frequencies(base: float, dims: int, scaling: Optional[dict]) -> torch.Tensor:
    """float64 [dims/2]: f_i = base^(-2i/dims), then the wavelength-dependent scaling of long-context Llama
    checkpoints: wavelengths below original/high keep f, above original/low use f/factor, between them a linear
    blend in original/wavelength."""
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float64)
    if not scaling:
        return f
    fac, lo, hi, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
    out = []
    for fi in f.tolist():
        wl = 2.0 * math.pi / fi
        if wl < orig / hi:
            out.append(fi)
        elif wl > orig / lo:
            out.append(fi / fac)
        else:
            s = (orig / wl - lo) / (hi - lo)
            out.append((1.0 - s) * fi / fac + s * fi)
    return torch.tensor(out, dtype=torch.float64)


def _ceil(a: int, b: int) -> int:
    return (a + b - 1) // b * b


class RaggedEngine:
    def __init__(self, spec: HybridSpec, device: str = "cuda:0", max_batch: int = 4, max_seq_len: int = 2048,
                 page_size: int = 16, kv_pool_tokens: Optional[int] = None, dtype=BF):
        if not torch.cuda.is_available():
            raise RuntimeError("RaggedEngine needs a CUDA device: this package has no CPU path")
        if dtype not in (BF, torch.float32):
            raise ValueError("dtype: torch.bfloat16 or torch.float32")
        self.spec, self.dtype = spec, dtype
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        self.max_batch, self.max_seq_len = int(max_batch), int(max_seq_len)
        self.is_first = self.is_last = self.has_head = True
        self.attn_layers = [i for i, L in enumerate(spec.layers) if L.mixer.kind == "attention"]
        shapes = [(spec.layers[i].mixer.kv_heads, spec.layers[i].mixer.dim, spec.layers[i].mixer.vdim)
                  for i in self.attn_layers]
        self.kv = PagedKVCache(len(shapes), 0, 0, page_size, self.max_batch, self.max_seq_len, self.device,
                               pool_tokens=kv_pool_tokens, layer_shapes=shapes, dtype=dtype)
        self.kv_index = {li: n for n, li in enumerate(self.attn_layers)}
        self.slots = StateSlots(self.max_batch, self.device)
        for i, L in enumerate(spec.layers):
            if spec.taps > 1:
                self.slots.add(("tail1", i), spec.taps - 1, spec.width)
                if L.ff:
                    self.slots.add(("tail2", i), spec.taps - 1, spec.width)
            if L.mixer.kind == "mlstm":
                m = L.mixer
                self.slots.add(("S", i), m.heads, m.dim, m.vdim)
                self.slots.add(("n", i), m.heads, m.dim)
                self.slots.add(("m", i), m.heads)
        self.lengths: Dict[int, int] = {}          # slot -> tokens the sequence holds
        self.w: Dict[str, object] = {}
        self.layers: Dict[int, dict] = {}
        self._tables: Dict[tuple, Tuple[torch.Tensor, torch.Tensor]] = {}
        self._ws_rows = 0
        self._meta_cap = 0
        self._graphs: Dict[tuple, object] = {}
        self.use_cuda_graph = os.environ.get("DLI_RAGGED_GRAPH", "1") == "1"
        self.eos_token_ids: tuple = ()
        self.pad_token_id: Optional[int] = None
        self.prefill_chunk: Optional[int] = None   # tokens of a prompt per step (None: the scheduler's default)
        self.tc_min_rows = int(os.environ.get("DLI_RAGGED_TC_MIN_ROWS", "16"))  # portions from this size: tensor-core attention
        self.mlstm_parallel_max_floats = 1 << 28   # scratch bound (1 GiB) of the block-parallel mLSTM; beyond it: blocks in order
        self.layer_trace: Optional[list] = None    # set to [] to collect the residual stream after every layer
        ops.set_pdl(os.environ.get("DLI_PDL", "1") == "1")

    # ------------------------------------------------------------------ weights
    def _table(self, base: float, dims: int, scaling: Optional[dict]):
        """fp32 cos / sin [max_seq_len, dims/2] of position * frequency, angles taken in float64 on the host."""
        key = (base, dims, tuple(sorted(scaling.items())) if scaling else None)
        if key not in self._tables:
            f = rot_frequencies(base, dims, scaling)
            ang = torch.arange(self.max_seq_len, dtype=torch.float64)[:, None] * f[None, :]
            self._tables[key] = (ang.cos().float().contiguous().to(self.device),
                                 ang.sin().float().contiguous().to(self.device))
        return self._tables[key]

    def load_tensors(self, t: dict) -> None:
        """t: {"embed", "head", "final_norm", "layers": {i: {...}}} with the layer tensors named as in
        sokevik.layer_tensors (any dtype / device); linear weights [out, in]."""
        dev, E = self.device, self.dtype
        s = self.spec

        def mat(*ws, pad_rows=True):
            """Rows of several [out, in] matrices stacked (padded to a multiple of 16 rows with zeros)."""
            w = torch.cat([x.reshape(-1, x.shape[-1]) for x in ws], dim=0).to(E)
            pad = _ceil(w.shape[0], 16) - w.shape[0] if pad_rows else 0
            if pad:
                w = torch.cat((w, torch.zeros(pad, w.shape[1], dtype=E)), dim=0)
            return w.contiguous().to(dev)

        def vec(x):
            return x.to(torch.float32).reshape(-1).contiguous().to(dev)

        self.w = {"embed": t["embed"].to(E).contiguous().to(dev), "head": mat(t["head"]),
                  "final_norm": float(t["final_norm"])}
        self.layers = {}
        for i, src in t["layers"].items():
            L, m = s.layers[i], s.layers[i].mixer
            d = {"norm1": float(src["norm1"]), "norm1b": float(src["norm1b"])}
            d["canon1"] = src["canon1"].to(torch.float32).contiguous().to(dev)
            qn, kn, vn = m.heads * m.dim, m.kv_heads * m.dim, m.kv_heads * m.vdim
            if m.kind == "attention":
                d["w_proj"] = mat(src["q"], src["k"], src["v"], src["g"]) if m.head_gate else mat(src["q"], src["k"], src["v"])
                d["off"] = {"q": 0, "k": qn, "v": qn + kn, "g": qn + kn + vn if m.head_gate else -1}
                d["q_norm"] = vec(src["q_norm"]) if m.qk_norm else None
                d["k_norm"] = vec(src["k_norm"]) if m.qk_norm else None
                d["sink"] = vec(src["sink"]) if m.sink else None
            else:
                gn = m.heads * m.vdim
                d["w_proj"] = mat(src["q"], src["k"], src["v"], src["g"], src["i"], src["f"])
                d["off"] = {"q": 0, "k": qn, "v": 2 * qn, "g": 2 * qn + gn, "i": 2 * qn + 2 * gn,
                            "f": 2 * qn + 2 * gn + m.heads}
                d["i_b"], d["f_b"], d["out_norm"] = vec(src["i_b"]), vec(src["f_b"]), vec(src["out_norm"])
            d["wo"] = mat(src["o"], pad_rows=False)
            if L.ff:
                d["norm2"], d["norm2b"] = float(src["norm2"]), float(src["norm2b"])
                d["canon2"] = src["canon2"].to(torch.float32).contiguous().to(dev)
                # the tensor-core path interleaves gate and up rows so that silu(gate) * up is the GEMM's epilogue
                d["packed"] = E == BF and L.ff % 128 == 0 and s.width % 8 == 0
                if d["packed"]:
                    d["w_gu"] = ops.pack_gate_up(src["gate"].to(BF), src["up"].to(BF)).to(dev)
                else:
                    d["w_gu"] = torch.cat((src["gate"], src["up"]), dim=0).to(E).contiguous().to(dev)
                d["w_down"] = mat(src["down"], pad_rows=False)
            self.layers[i] = d

    def weight_bytes(self) -> int:
        total = self.w["embed"].numel() * self.w["embed"].element_size() + self.w["head"].numel() * self.w["head"].element_size()
        for d in self.layers.values():
            total += sum(v.numel() * v.element_size() for v in d.values() if isinstance(v, torch.Tensor))
        return total

    def unload(self) -> None:
        self._graphs.clear()
        self._sk = None
        self.w.clear()
        self.layers.clear()
        self.kv.release_all()
        self.kv.k.clear()
        self.kv.v.clear()
        self.slots.tensors.clear()
        self._ws_rows = 0
        torch.cuda.empty_cache()

    # ------------------------------------------------------------------ sequences
    def open_sequence(self) -> int:
        """Admit a sequence: a state slot, which is also its row of the page table.  Pages come with the tokens."""
        slot = self.slots.alloc()
        self.lengths[slot] = 0
        return slot

    def close_sequence(self, slot: int) -> None:
        """Give back the sequence's pages and slot."""
        self.kv.release(slot)
        self.slots.release(slot)
        self.lengths.pop(slot, None)

    # ------------------------------------------------------------------ workspace
    def _workspace(self, rows: int) -> None:
        if rows <= self._ws_rows:
            return
        s, dev, E = self.spec, self.device, self.dtype
        rows = _ceil(rows, 64)
        mx = [L.mixer for L in s.layers]
        n_proj = max(d["w_proj"].shape[0] for d in self.layers.values())
        n_mix = max(m.heads * m.vdim for m in mx)
        n_q = max([m.heads * m.dim for m in mx if m.kind == "attention"] or [1])
        ff = max([L.ff for L in s.layers] or [0])
        f32 = torch.float32
        self._x = torch.empty(rows, s.width, dtype=f32, device=dev)
        self._hn = torch.empty(rows, s.width, dtype=f32, device=dev)
        self._hc = torch.empty(rows, s.width, dtype=E, device=dev)
        self._proj = torch.empty(rows * n_proj, dtype=E, device=dev)
        self._qbuf = torch.empty(rows * n_q, dtype=f32, device=dev)
        self._mix = torch.empty(rows * n_mix, dtype=E, device=dev)
        self._oscr = torch.empty(rows * n_mix, dtype=f32, device=dev)
        self._y = torch.empty(rows, s.width, dtype=E, device=dev)
        self._act = torch.empty(rows * max(ff, 1), dtype=E, device=dev)
        self._gu = torch.empty(rows * max(2 * ff, 1), dtype=E, device=dev)
        self._hw = torch.empty(max(self.max_batch, 8), s.width, dtype=E, device=dev)
        self._ws_rows = rows
        self._graphs.clear()  # captured graphs hold the old workspace pointers

    def _lin(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """out = x @ w.T: the framework's bf16 projection (tcgen05 GEMM / weight-streaming GEMV) where its alignment
        rules hold, else the CUDA-core GEMM (float32 engines, odd shapes)."""
        if self.dtype == BF and x.shape[1] % 8 == 0 and w.shape[0] % 8 == 0:
            if 2 < x.shape[0] <= 128 and x.shape[1] % 64 == 0 and w.shape[0] % 16 == 0:
                # few rows (batched decode, short portions): the split-K weight stream on every SM, as the uniform
                # stacks' batched decode does
                return ops.linear_splitk(x, w, self._splitk(), out=out)
            return ops.linear(x, w, out=out)
        return ops.linear_any(x, w, out)

    def _splitk(self) -> torch.Tensor:
        """Zero-filled scratch of the split-K projections (self-resetting; calls are ordered on one stream)."""
        if getattr(self, "_sk", None) is None:
            n_max = max([self.w["head"].shape[0]] + [max(d["w_proj"].shape[0], d["w_gu"].shape[0] if "w_gu" in d else 0,
                                                         self.spec.width) for d in self.layers.values()])
            self._sk = torch.zeros(ops.gemm_splitk_scratch_bytes(128, n_max), dtype=torch.uint8, device=self.device)
        return self._sk

    # ------------------------------------------------------------------ one step
    def step(self, batch: Sequence[Tuple[int, Sequence[int]]], want: Optional[Sequence[Sequence[int]]] = None):
        """batch: [(slot, next tokens)] — every live sequence at most once; want[i]: indices into entry i's tokens
        whose logits are asked for (default: the last one of each entry).  Runs the tokens on top of what earlier
        steps left in the caches and slots and returns the logits [sum(len(want[i])), vocab] (engine dtype, device),
        rows in the order of the entries and of want."""
        s, dev, E = self.spec, self.device, self.dtype
        if want is None:
            want = [[len(t) - 1] for _, t in batch]
        rows = sum(len(t) for _, t in batch)
        if rows == 0:
            return torch.empty(0, s.vocab, dtype=E, device=dev)
        n_ent = len(batch)
        tokens: List[int] = []
        row_ent: List[int] = []
        ent: List[int] = []
        want_rows: List[int] = []
        grew = False
        seen = set()
        for i, (slot, toks) in enumerate(batch):
            if slot not in self.lengths or slot in seen or len(toks) == 0:
                raise ValueError(f"step: slot {slot} is not live, appears twice or brings no tokens")
            seen.add(slot)
            start = self.lengths[slot]
            if start + len(toks) > self.max_seq_len:
                raise ValueError(f"sequence of {start + len(toks)} tokens exceeds max_seq_len {self.max_seq_len}")
            if self.attn_layers:
                grew |= self.kv.reserve(slot, start + len(toks))
            ent += [slot, len(tokens), len(toks), start]
            want_rows += [len(tokens) + int(j) for j in want[i]]
            row_ent += [i] * len(toks)
            tokens += [int(t) for t in toks]
        if grew:
            self.kv.commit()
        # steps that hold a portion of a prompt run attention in 64-row query tiles on the tensor cores
        tiles: List[int] = []
        if any(len(t) >= self.tc_min_rows for _, t in batch):
            for i, (_, toks) in enumerate(batch):
                for q0 in range(0, len(toks), 64):
                    tiles += [i, q0]
        # one host -> device copy of the step's description: tokens | row_ent | ent | want_rows | tiles (16-byte aligned parts)
        r4, e4, w4 = _ceil(rows, 4), 4 * n_ent, _ceil(max(len(want_rows), 1), 4)
        total = 2 * r4 + e4 + w4 + len(tiles)
        if total > self._meta_cap:
            self._meta_cap = _ceil(total, 1024)
            # a ring of pinned staging buffers: the host may run ahead of the device by several steps, and a buffer
            # is written again only after the copy that read it has finished
            self._meta_ring = [(torch.zeros(self._meta_cap, dtype=torch.int32).pin_memory(), torch.cuda.Event())
                               for _ in range(4)]
            self._meta_turn = 0
            self._meta_dev = torch.zeros(self._meta_cap, dtype=torch.int32, device=dev)
            self._graphs.clear()  # captured graphs hold the old buffer's addresses
        self._meta_turn = (self._meta_turn + 1) % len(self._meta_ring)
        mh, copied = self._meta_ring[self._meta_turn]
        copied.synchronize()
        mh[:rows] = torch.tensor(tokens, dtype=torch.int32)
        mh[r4:r4 + rows] = torch.tensor(row_ent, dtype=torch.int32)
        mh[2 * r4:2 * r4 + e4] = torch.tensor(ent, dtype=torch.int32)
        if want_rows:
            mh[2 * r4 + e4:2 * r4 + e4 + len(want_rows)] = torch.tensor(want_rows, dtype=torch.int32)
        if tiles:
            mh[2 * r4 + e4 + w4:total] = torch.tensor(tiles, dtype=torch.int32)
        md = self._meta_dev
        md[:total].copy_(mh[:total], non_blocking=True)
        copied.record()
        d_tok, d_rent, d_ent = md[:rows], md[r4:r4 + rows], md[2 * r4:2 * r4 + e4]
        d_want = md[2 * r4 + e4:2 * r4 + e4 + len(want_rows)]
        d_tiles = md[2 * r4 + e4 + w4:total]

        self._workspace(rows)
        long_step = any(len(t) >= self.tc_min_rows for _, t in batch)  # a portion of a prompt is in the step
        nw = len(want_rows)
        views = (d_tok, d_rent, d_ent, d_want, d_tiles)
        # a step of single tokens (decode) has the same launches every time: the device buffers of its description sit
        # at fixed addresses per batch size, so it is captured once as a CUDA graph and replayed
        if self.use_cuda_graph and rows == n_ent and self.layer_trace is None:
            logits = self._graphed_forward(rows, n_ent, nw, views)
        else:
            logits = self._forward(rows, n_ent, nw, views, long_step, bool(tiles), None)
        for slot, toks in batch:
            self.lengths[slot] += len(toks)
        if logits is None:
            return torch.empty(0, s.vocab, dtype=E, device=dev)
        return logits[:, :s.vocab]

    def _graphed_forward(self, rows, n_ent, nw, views):
        key = (rows, nw)
        hit = self._graphs.get(key)
        if hit is None:
            # first use: run it (this also sets every kernel's attributes); the capture happens at the second use,
            # because a capture does not execute and the step must advance the caches exactly once
            self._graphs[key] = "warm"
            return self._forward(rows, n_ent, nw, views, False, False, None)
        if hit == "warm":
            out = torch.empty(max(nw, 1), self.w["head"].shape[0], dtype=self.dtype, device=self.device)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            n0 = ops.launch_count
            with torch.cuda.graph(g, capture_error_mode="thread_local"):
                self._forward(rows, n_ent, nw, views, False, False, out)
            self._graphs[key] = hit = (g, out, ops.launch_count - n0)
        g, out, launches = hit
        g.replay()
        ops.launch_count += launches
        return out[:nw].clone() if nw else None

    def _forward(self, rows, n_ent, nw, views, long_step, use_tiles, logits_out):
        """Every kernel of one step, in order; logits_out: where the logits go (a buffer of fixed address under capture)."""
        s, dev, E = self.spec, self.device, self.dtype
        d_tok, d_rent, d_ent, d_want, d_tiles = views
        tiles = use_tiles
        W = s.width
        x, hn, hc = self._x[:rows], self._hn[:rows], self._hc[:rows]
        y = self._y[:rows]
        single = rows == n_ent and s.taps > 1 and self.layer_trace is None  # decode rows: norm + convolution fused

        def enter_sublayer(y_prev, g_post, g_next, tail, taps_w):
            """Close the previous sublayer (x += postnorm(y_prev)) and open the next one: hc = its normed and convolved
            input.  One kernel for decode rows, norm kernel + convolution (+ tail shift) otherwise."""
            if single:
                ops.postnorm_add_norm_conv_single(y_prev, x, tail, taps_w, d_ent, hc, g_post, g_next, s.eps)
                return
            if y_prev is None:
                ops.scalar_rmsnorm(x, g_next, s.eps, hn)
            else:
                ops.postnorm_add_norm(y_prev, x, g_post, s.eps, hn, g_next)
            ops.causal_conv_ragged(hn, tail, taps_w, d_rent, d_ent, hc)  # one tap: no tail, h * (1 + w)

        ops.embedding_f32(d_tok, self.w["embed"], x)
        pt = self.kv.page_table
        y_prev, g_prev = None, 1.0
        for li, L in enumerate(s.layers):
            P, m = self.layers[s.source(li)], L.mixer
            enter_sublayer(y_prev, g_prev, P["norm1"], self.slots.tensors.get(("tail1", li)), P.get("canon1"))
            n_proj = P["w_proj"].shape[0]
            proj = self._proj[:rows * n_proj].view(rows, n_proj)
            self._lin(hc, P["w_proj"], proj)
            n_mix = m.heads * m.vdim
            mix = self._mix[:rows * n_mix].view(rows, n_mix)
            off = P["off"]
            if m.kind == "attention":
                kc, vc = self.kv.k[self.kv_index[li]], self.kv.v[self.kv_index[li]]
                cq, sq = self._table(m.rot_base, m.rot_dims, m.rot_scaling) if m.rot_dims else (None, None)
                cv, sv = self._table(m.rot_base, m.vdim, None) if m.rotate_values else (None, None)
                qbuf = self._qbuf[:rows * m.heads * m.dim].view(rows, m.heads * m.dim)
                ops.attn_prep_append(proj, qbuf, kc, vc, d_rent, d_ent, pt, m.heads, m.kv_heads, m.dim, m.vdim,
                                     m.rot_dims, off["q"], off["k"], off["v"], P["q_norm"], P["k_norm"], s.eps,
                                     cq, sq, cv, sv)
                if tiles and m.scale > 0 and ops.attn_ragged_tc_supported(m.dim, m.vdim, E):
                    ops.attn_ragged_tc(qbuf, kc, vc, proj, mix, d_ent, d_tiles, pt, m.heads, m.kv_heads, m.dim, m.vdim,
                                       m.scale, chunk=m.chunk, window=m.window, sink=P["sink"], g_off=off["g"],
                                       cos_v=cv, sin_v=sv)
                else:
                    ops.attn_ragged(qbuf, kc, vc, proj, mix, d_rent, d_ent, pt, m.heads, m.kv_heads, m.dim, m.vdim,
                                    m.scale, chunk=m.chunk, window=m.window, sink=P["sink"], g_off=off["g"], cos_v=cv,
                                    sin_v=sv)
            else:
                oscr = self._oscr[:rows * n_mix]
                n_tiles = d_tiles.numel() // 2
                need = ops.mlstm_parallel_scratch_floats(n_tiles, m.heads, m.dim, m.vdim) if tiles and n_tiles > n_ent else 0
                if need and need <= self.mlstm_parallel_max_floats and m.dim <= 224:
                    # some entry spans several 64-position blocks: all blocks in parallel
                    if getattr(self, "_mlstm_scr", None) is None or self._mlstm_scr.numel() < need:
                        self._mlstm_scr = torch.empty(need, dtype=torch.float32, device=dev)
                    ops.mlstm_ragged_parallel(proj, oscr, mix, d_ent, d_tiles, self._mlstm_scr, m.heads, m.dim, m.vdim,
                                              off["q"], off["k"], off["v"], off["i"], off["f"], off["g"], P["i_b"],
                                              P["f_b"], m.gate_cap, P["out_norm"], s.eps, self.slots[("S", li)],
                                              self.slots[("n", li)], self.slots[("m", li)])
                else:
                    ops.mlstm_ragged(proj, oscr, mix, d_ent, m.heads, m.dim, m.vdim, off["q"], off["k"], off["v"], off["i"],
                                     off["f"], off["g"], P["i_b"], P["f_b"], m.gate_cap, P["out_norm"], s.eps,
                                     self.slots[("S", li)], self.slots[("n", li)], self.slots[("m", li)], blocked=long_step)
            self._lin(mix, P["wo"], y)
            g_post = P["norm1b"]
            if L.ff:
                enter_sublayer(y, g_post, P["norm2"], self.slots.tensors.get(("tail2", li)), P.get("canon2"))
                act = self._act[:rows * L.ff].view(rows, L.ff)
                if P["packed"] and 2 < rows <= 128 and W % 64 == 0:
                    ops.linear_splitk_gated_silu(hc, P["w_gu"], self._splitk(), out=act)
                elif P["packed"]:
                    ops.linear_gated_silu(hc, P["w_gu"], out=act)
                else:
                    gu = self._gu[:rows * 2 * L.ff].view(rows, 2 * L.ff)
                    self._lin(hc, P["w_gu"], gu)
                    ops.silu_mul(gu, act)
                self._lin(act, P["w_down"], y)
                g_post = P["norm2b"]
            y_prev, g_prev = y, g_post
            if self.layer_trace is not None:
                # the residual stream after the layer (debugging): close the sublayer now and open the next without it
                ops.postnorm_add_norm(y, x, g_post, s.eps)
                self.layer_trace.append(x.clone())
                y_prev = None
        if y_prev is None:
            ops.scalar_rmsnorm(x, self.w["final_norm"], s.eps, hn)
        else:
            ops.postnorm_add_norm(y_prev, x, g_prev, s.eps, hn, self.w["final_norm"])
        if nw == 0:
            return None
        hw = self._hw[:nw] if nw <= self._hw.shape[0] else torch.empty(nw, W, dtype=E, device=dev)
        ops.gather_cast(hn, d_want, hw)
        vp = self.w["head"].shape[0]
        logits = logits_out[:nw] if logits_out is not None else torch.empty(nw, vp, dtype=E, device=dev)
        self._lin(hw, self.w["head"], logits)
        return logits

    # ------------------------------------------------------------------ public API
    @torch.no_grad()
    def generate(self, input_ids: torch.Tensor, max_length: int, do_sample: bool = False, temperature: float = 0.8,
                 top_k: int = 50, top_p: float = 0.95, seed: int = 0, deadline: Optional[float] = None,
                 on_tokens=None, **_):
        """ShardEngine.generate's signature and behaviour (int [B, T] prompts -> int64 [B, <= max_length] on the host, greedy or
        the sampling call), run by the ragged scheduler: prompts go in portions beside the decoding rows."""
        import time as _time

        from .batching import RaggedBatcher
        from .engine import apply_eos, check_max_length

        B, T = input_ids.shape
        check_max_length(T, max_length)
        sched = RaggedBatcher(self, chunk=self.prefill_chunk or 512, temperature=temperature, top_k=top_k, top_p=top_p)
        futs = [sched.submit(input_ids[b], max_length=max_length, do_sample=do_sample, seed=seed + b,
                             timeout=None if deadline is None else max(0.0, deadline - _time.time()))
                for b in range(B)]
        n = 0
        while not all(f.done() for f in futs):
            sched.step()
            n += 1
            if on_tokens is not None and (n & 7) == 0 and B == 1:
                on_tokens(torch.cat((input_ids[0].cpu().long(), torch.tensor(futs[0].request.out, dtype=torch.int64)))[None])
        outs = [f.result() for f in futs]
        width = max(len(o) for o in outs)
        pad = self.pad_token_id if self.pad_token_id is not None else (self.eos_token_ids[0] if self.eos_token_ids else 0)
        out = torch.full((B, width), int(pad), dtype=torch.int64)
        for b, o in enumerate(outs):
            out[b, :len(o)] = o
        new = apply_eos(out[:, T:], tuple(self.eos_token_ids), self.pad_token_id)
        return torch.cat((input_ids.cpu().long(), new), dim=1)
