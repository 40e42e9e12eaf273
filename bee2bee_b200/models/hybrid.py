"""A piece of a *hybrid* decoder on one B200: every layer names its own token mixer.

Family ``kepovik``: gated sigmoid attention over the paged KV cache or a generalized delta-rule recurrence with a
per-sequence fp32 state, joined by several residual streams (hyper-connections), behind a token + hashed token-pair
embedding; sublayers run one after the other.

Family ``repudra``: parallel blocks -- one norm (a single gain) feeds the mixer AND the feed-forward (xIELU), their
outputs join ONE fp32 residual through layer-scale vectors.  Mixers: causal softmax attention (norm over the whole q / k
projection, rotary positions on part of each head with YaRN frequencies, per-head value norm, key width != value width)
beside an mLSTM matrix memory, their width-normed outputs averaged; diag-gated linear attention; a delta rule with a
decay per key channel behind short convolutions.  Each mixer kind is a method here and a kernel family in
``csrc/seqmix.cu`` with its constants as arguments, so other layer mixes can be described by a config alone.

Family ``lonulix``: post-norm layers -- ``x <- groupnorm(alpha x + gate * sublayer(x))``, the sublayers read the residual
itself and their results pass a sigmoid gate computed from it.  Mixers: latent attention (keys and values are
up-projections of ONE cached latent per token plus a rotary key slice common to all heads; served in the absorbed form, so
the paged cache holds ``[rotated part | latent]`` rows only) and HGRN2 (keyless linear attention: a forget gate with a learned lower
bound, and its complement as the write strength).  Feed-forward: gated silu, or routed gelu experts (softmax router, selection-only correction,
group-limited top-k, identity experts).

Family ``fisopel``: parallel blocks with a norm each for the mixer and the feed-forward (``x <- x + mixer(norm1 x) +
ff(norm2 x)``), a range of layers that runs several times with the same weights (a cache per pass; the residual entering a
pass is ``W_in [x ; embedding output]``), logits from the embedding table.  Mixers: softmax attention with a per-head q / k
norm, capped scores, a window that keeps the first keys in sight and a sink in the denominator; gated latent attention (keys
absorbed into the queries, values up-projected per head behind the attention, rotary part in the half-split pairing with
YaRN frequencies).  Feed-forward: gated silu experts chosen by their router logits beside a shared expert.

Same interface as ``native.NativePiece`` (the runner drives both through ``forward(BatchMeta)``): a flat batch of spans
(prompt portions of any length beside single decoded tokens), physical KV slots and block tables from the page allocator,
logits for the rows named by ``last_idx``.  What is new here and lives next to the shared machinery:

* ``state`` / ``prev_tok``: one recurrent state per delta-rule layer and the last token, indexed by the *batch slot*
  of the sequence (``BatchMeta.seq_slot``); a span that starts at position 0 starts from a zero state, so a slot that is
  used again needs no clearing.
* ``streams``: the residual is ``[tokens, streams, width]`` in fp32; ``ops.hc_step`` applies the stream mixing of the
  sublayer that just ran and produces the normed input of the next one in a single pass (``ops.ls_join`` for the
  one-stream parallel blocks: layer scale, optional width norm of the joining outputs, next norm).
* per-slot state of the recurrent mixers: ``state`` [slots, heads, dk, dv], the mLSTM normaliser and running maximum,
  the last ``taps - 1`` inputs of the short convolutions -- all fp32, all indexed by batch slot like ``prev_tok``.
* precision: streams, norms, scores, decays and the state are fp32 in every mode; ``dtype`` only selects what feeds the
  matrix products and what the KV cache holds (bf16 on the tcgen05 GEMM, or float32 through cuBLAS for bit-faithful runs).

Launches per layer (kepovik): attention 5 (+3 with a feed-forward), delta rule 7.  The reference has no counterpart
(it delegates every architecture to ``transformers``, /root/reference/bee2bee/hf.py:23-44).
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Dict, Iterable, Optional

import torch
import torch.nn.functional as F

from .. import ops
from .config import LayerSpec, ModelConfig
from .weights import Tensors


@dataclass
class _Mix:
    """one token mixer of a parallel-block layer: where its projections sit in the layer's fused GEMM output, its own
    matrices and small fp32 parameters, and what it contributes to the residual join"""
    spec: LayerSpec
    key: str = ""                       # name of its caches / states
    idx: int = 0                        # position among the mixers of its layer (scratch buffers are per position)
    off: Dict[str, int] = field(default_factory=dict)       # column of each projection in the fused output
    w_o: torch.Tensor = None
    w2: Optional[torch.Tensor] = None   # second level of the low-rank gate projections
    rank: int = 0
    f: Dict[str, torch.Tensor] = field(default_factory=dict)
    join_w: Optional[torch.Tensor] = None    # coordinate-wise weight of its output in the residual join
    join_norm: bool = False                  # its output is divided by its root mean square over the width first
    amp: float = 1.0                         # rotary amplitude
    w_uv: Optional[torch.Tensor] = None      # latent attention with an output gate: [heads, vdim, kv_rank] value up-projections


@dataclass
class _Layer:
    spec: LayerSpec
    w_cat: torch.Tensor = None          # attention: [q | k | v | gate]; delta rule: [r | k | v | gate | a | w1]
    w_o: torch.Tensor = None
    w2: Optional[torch.Tensor] = None   # delta rule: decay low-rank up-projection
    rank: int = 0
    f: Dict[str, torch.Tensor] = field(default_factory=dict)     # small fp32 parameters
    w_up: Optional[torch.Tensor] = None
    w_down: Optional[torch.Tensor] = None
    w_glu: Optional[torch.Tensor] = None   # post-norm dense feed-forward, bf16: [gate | up] interleaved for the gated GEMM epilogue
    ff_off: Dict[str, int] = field(default_factory=dict)    # routed experts: columns of router / gate block / up block
    mix: tuple = ()                     # parallel blocks: the mixers that read the layer's input side by side
    act_params: tuple = (0.0, 0.0)      # xIELU: softplus(p), 1/2 + softplus(q)


# projections of each mixer kind that read the layer input, in the order they are stacked into the fused GEMM
_PROJ = {"softmax_attention": ("q", "k", "v"), "mlstm": ("q", "k", "v", "g", "i", "f"),
         "gla": ("q", "k", "v", "g", "a1"), "channel_delta": ("q", "k", "v", "b", "a1", "g1")}


class HybridPiece:
    def __init__(self, cfg: ModelConfig, layers: Iterable[int], first: bool, last: bool, tensors: Tensors,
                 device: torch.device, max_tokens: int, max_seqs: int, num_pages: int, quant: str = "bf16",
                 units: Optional[tuple] = None, dtype: torch.dtype = torch.bfloat16, state_slots: int = 0,
                 max_out_rows: int = 0):
        assert cfg.hybrid, "HybridPiece serves configs with per-layer mixer specs"
        if not (first and last):
            raise ValueError(f"{cfg.name}: recurrent state and residual streams are not handed between GPUs yet; "
                             "hybrid models run as a single piece")
        if quant != "bf16":
            raise ValueError(f"{cfg.name}: quantised weights are not implemented for hybrid models")
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("dtype must be bfloat16 or float32")
        self.cfg, self.layers, self.first, self.last = cfg, list(layers), first, last
        self.device = dev = torch.device(device)
        self.dtype = dtype
        self.max_tokens, self.max_seqs, self.num_pages = max_tokens, max_seqs, num_pages
        self.state_slots = max(1, state_slots or max_seqs)
        self.max_out_rows = max(max_out_rows, max_seqs)
        self.head_mode, self.tail_mode = 0, 2
        self.fp8 = self.mx = self.mx_fuse = self.mx_hand = False
        self.max_splits = 1
        self.ns = max(1, cfg.streams)
        W = cfg.hidden_size
        self.Wp = ops.pad_to(W, 64)
        f32 = torch.float32

        def mat(*names, k_mult=64):          # row-concatenated, padded to the GEMM tile, in the operand dtype
            w = torch.cat([tensors[n].to(device=dev, dtype=f32) for n in names], 0)
            return ops.pad_weight(w, 128, k_mult).to(dtype).contiguous()

        def vec(name):
            return tensors[name].to(device=dev, dtype=f32).contiguous()

        self.parallel_blocks = cfg.block_layout == "parallel"
        self.post_norm = cfg.block_layout == "post_norm"
        # parallel blocks: the feed-forward reads the same input as the mixers, so its two GEMMs run on a second stream
        # beside the recurrences (which are sequential in the tokens and leave most SMs idle), and the second of two
        # mixers side by side on a third; B2B_HYBRID_OVERLAP=0: one stream
        self.overlap_ff = (self.parallel_blocks and dtype == torch.bfloat16
                           and os.environ.get("B2B_HYBRID_OVERLAP", "1") == "1")
        self._side = torch.cuda.Stream(device=dev) if self.overlap_ff else None
        self._side2 = torch.cuda.Stream(device=dev) if self.overlap_ff else None     # second mixer of a parallel pair
        self.caps_logits = self.parallel_blocks and cfg.final_softcap > 0     # the piece applies the logit soft cap itself
        self.L: Dict[int, _Layer] = {}
        for l in self.layers:
            sp, p = cfg.layer_specs[l], f"l{l}."
            L = _Layer(spec=sp)
            if self.parallel_blocks:
                self.L[l] = self._build_parallel_block(L, l, tensors, mat, vec)
                continue
            if self.post_norm:
                self.L[l] = self._build_post_norm_layer(L, l, tensors, mat, vec)
                continue
            if sp.mixer == "attention":
                L.w_cat = mat(p + "mix.q", p + "mix.k", p + "mix.v", p + "mix.g")
                for n in ("q.norm", "k.norm", "pb"):
                    L.f[n] = vec(p + "mix." + n)
            else:
                L.rank = tensors[p + "mix.w1"].shape[0]
                L.w_cat = mat(p + "mix.r", p + "mix.k", p + "mix.v", p + "mix.g", p + "mix.a", p + "mix.w1")
                L.w2 = mat(p + "mix.w2")
                for n in ("w0", "a.b", "norm"):
                    L.f[n] = vec(p + "mix." + n)
            L.w_o = mat(p + "mix.o")
            L.f["norm1"] = vec(p + "norm1")
            if sp.ff:
                L.w_up, L.w_down = mat(p + "mlp.up"), mat(p + "mlp.down", k_mult=128)   # K of down = padded rows of up
                L.f["norm2"] = vec(p + "norm2")
            if cfg.streams:
                for q in ("hc1", "hc2") if sp.ff else ("hc1",):
                    for n in ("in", "out", "mix"):
                        L.f[f"{q}.{n}"] = vec(f"{p}{q}.{n}")
            self.L[l] = L
        self.embed = tensors["embed"].to(device=dev, dtype=dtype).contiguous()
        self.pair = tensors["bigram"].to(device=dev, dtype=dtype).contiguous() if cfg.pair_buckets else None
        self.final_norm = vec("final.norm").reshape(-1)
        self.w_head = mat("embed" if cfg.tie_embeddings else "head")
        self.w_loop = mat("loop.in") if cfg.loop_in else None       # [x ; embedding output] -> the residual entering a pass
        self.runs = [r for r in cfg.layer_runs() if r[0] in self.L]  # (layer, pass, first of a pass) in execution order
        self._pass = 0
        self.vocab_pad = self.w_head.shape[0]

        # ---- per-sequence state (indexed by batch slot) and the paged KV cache of the attention layers
        self.prev_tok = torch.zeros(self.state_slots, device=dev, dtype=torch.int32)
        self.state: Dict[int, torch.Tensor] = {}
        self.k_cache: Dict[object, torch.Tensor] = {}
        self.v_cache: Dict[object, torch.Tensor] = {}
        self.nstate: Dict[str, torch.Tensor] = {}      # mLSTM normaliser [slots, heads, dk] and running maximum [slots, heads]
        self.mstate: Dict[str, torch.Tensor] = {}
        self.conv_tail: Dict[str, torch.Tensor] = {}   # short convolutions: the last taps - 1 inputs [slots, taps - 1, channels]
        for l in self.layers:
            sp = cfg.layer_specs[l]
            if self.parallel_blocks or self.post_norm:
                for self._pass in sorted({p for ll, p, _ in self.runs if ll == l}):     # a cache / state per pass of a looped layer
                    for mx in self.L[l].mix:
                        self._alloc_mixer_state(mx, num_pages)
                self._pass = 0
                continue
            if sp.mixer == "attention":
                self.k_cache[l] = torch.zeros((num_pages, ops.PAGE, sp.kv_heads, sp.dim), device=dev, dtype=dtype)
                self.v_cache[l] = torch.zeros((num_pages, ops.PAGE, sp.kv_heads, sp.vdim), device=dev, dtype=dtype)
            else:
                self.state[l] = torch.zeros((self.state_slots, sp.heads, sp.dim, sp.dim), device=dev, dtype=f32)
        # ---- activations (every buffer is keyed by its logical width so zero padding is never dirtied)
        self.streams = torch.zeros((max_tokens, self.ns, W), device=dev, dtype=f32)
        self._bufs: Dict[tuple, torch.Tensor] = {}
        self.h = self._buf("h", dtype, self.Wp)
        self.h2 = self._buf("h2", dtype, self.Wp) if cfg.ff_norm else None
        self.last_x = torch.zeros((self.max_out_rows, self.Wp), device=dev, dtype=dtype)
        self.logits = torch.zeros((self.max_out_rows, self.vocab_pad), device=dev, dtype=f32)
        self._ones = torch.ones(self.ns, device=dev, dtype=f32)
        self.debug_layers: Optional[list] = None     # tests: set to [] to collect the stream sum after every layer

    # ------------------------------------------------------------------ helpers
    def _buf(self, tag: str, dtype: torch.dtype, width: int) -> torch.Tensor:
        key = (tag, dtype, width)
        b = self._bufs.get(key)
        if b is None:
            b = self._bufs[key] = torch.zeros((self.max_tokens, width), device=self.device, dtype=dtype)
        return b

    def _key(self, mx: _Mix) -> str:
        """name of the cache / state of mixer ``mx`` in the current pass of the loop (pass 0: the mixer's own key)"""
        return mx.key if self._pass == 0 else f"{mx.key}@{self._pass}"

    def _matrices(self):
        if self.w_loop is not None:
            yield self.w_loop
        for L in self.L.values():
            for t in (L.w_cat, L.w_o, L.w2, L.w_up, L.w_down, L.w_glu):
                if t is not None:
                    yield t
            for mx in L.mix:
                for t in (mx.w_o, mx.w2, mx.w_uv):
                    if t is not None:
                        yield t

    def weight_bytes(self) -> int:
        n = sum(t.numel() * t.element_size() for t in self._matrices())
        n += self.w_head.numel() * self.w_head.element_size() + self.embed.numel() * self.embed.element_size()
        return n + (self.pair.numel() * self.pair.element_size() if self.pair is not None else 0)

    def streamed_weight_bytes(self) -> int:
        """bytes a decode step streams: every matrix except the embedding tables (one row per sequence is gathered)"""
        n = sum(t.numel() * t.element_size() for t in self._matrices())
        return n + self.w_head.numel() * self.w_head.element_size()

    def state_bytes_per_seq(self) -> int:
        return sum(s[0].numel() * 4 for d in (self.state, self.nstate, self.mstate, self.conv_tail) for s in d.values())

    def n_launches(self) -> int:
        if self.post_norm:
            n = 3                                        # embedding, its operand copy, final norm (head GEMM: the runner)
            for L in self.L.values():
                n += 3 + (5 if L.spec.mixer == "latent_attention" else 3)      # fused projection, output projection, join
                if L.spec.ff:
                    n += 4 + (1 if L.spec.ff_kind == "moe" else 0)
            return n
        if self.parallel_blocks:
            per = {"softmax_attention": 3, "mlstm": 4, "gla": 5, "channel_delta": 7, "latent_attention": 5}
            n = 2 + (1 if self.caps_logits else 0)       # embedding, final join + norm (+ soft cap; head GEMM: the runner)
            n += 1 if self.w_loop is not None else 0     # copy of the embedding output
            for l, _, first in self.runs:
                L = self.L[l]
                n += 2 + sum(per[mx.spec.mixer] for mx in L.mix)                             # join + fused projection
                n += (4 if L.spec.ff_kind == "moe" else 2) if L.spec.ff else 0
                n += 2 if (first and self.w_loop is not None) else 0
            return n
        n = 3          # embedding, final stream sum + norm, previous-token commit (+ the head GEMM counted by the runner)
        for L in self.L.values():
            n += (5 if L.spec.mixer == "attention" else 7) + (3 if L.spec.ff else 0)
        return n

    # ------------------------------------------------------------------ forward
    def forward(self, m, x_in=None, hand=None, out_x=None, h_in=None) -> torch.Tensor:
        """Runs all layers for the spans described by ``m`` (``native.BatchMeta`` with ``seq_slot``); returns fp32
        logits ``[m.n_out or m.n_seqs, vocab_pad]`` for the token rows ``m.last_idx`` (decode: one row per sequence)."""
        c = self.cfg
        T, S, mq = m.n_tokens, m.n_seqs, m.max_q
        eps, mult = c.norm_eps, c.residual_mult
        st = self.streams[:T]
        seq_slot = m.seq_slot
        assert seq_slot is not None, "hybrid models need BatchMeta.seq_slot (state slot of every sequence)"
        if self.parallel_blocks:
            return self._forward_parallel_blocks(m)
        if self.post_norm:
            return self._forward_post_norm(m)
        ops.hyb_embed(m.ids, m.positions, m.q_start, m.q_len, seq_slot, self.prev_tok, self.embed, self.pair,
                      c.pair_buckets, c.pair_mul_prev, c.pair_mul_cur, st, S, mq)
        h = self.h[:T]
        pend = None                      # (y, mix, out) of the sublayer whose output has not joined the streams yet

        def pre(pend, L, q):
            kw = {}
            if pend is not None:
                kw = dict(y=pend[0], mix=pend[1], outw=pend[2], mult=mult)
            ops.hc_step(st, m.q_start, m.q_len, S, mq, inw=L.f.get(f"hc{q}.in"), gamma=L.f[f"norm{q}"], eps=eps, h=h, **kw)

        for l in self.layers:
            L = self.L[l]
            pre(pend, L, 1)
            y = self._attention(l, L, h, m) if L.spec.mixer == "attention" else self._delta(l, L, h, m)
            pend = (y, L.f.get("hc1.mix"), L.f.get("hc1.out"))
            if L.spec.ff:
                pre(pend, L, 2)
                hid = self._buf("ff", self.dtype, L.w_up.shape[0])[:T]
                ops.linear(L.w_up, h, hid, act=ops.ACT_RELU_SQ)
                y = ops.linear(L.w_down, hid, self._buf("y", torch.float32, L.w_down.shape[0])[:T])
                pend = (y, L.f.get("hc2.mix"), L.f.get("hc2.out"))
            if self.debug_layers is not None:
                self.debug_layers.append(self._debug_sum(st, pend, T))
        # output rows only: last sublayer joins the streams, streams are summed, model norm
        R = m.n_out or S
        if m.last_idx is not None:
            rows = m.last_idx
        else:
            rows = m.q_start           # decode: one token per sequence, row = q_start
        xl = self.last_x[:R]
        kw = dict(y=pend[0], mix=pend[1], outw=pend[2], mult=mult) if pend is not None else {}
        ops.hc_step(st, m.q_start, m.q_len, S, mq, inw=self._ones, gamma=self.final_norm, eps=eps, h=xl, rows=rows,
                    n_rows=R, **kw)
        ops.hyb_commit_prev(m.ids, m.q_start, m.q_len, seq_slot, self.prev_tok, S)
        return ops.linear(self.w_head, xl, self.logits[:R])

    # ================================================================== parallel blocks (one residual, layer scale)
    def _build_parallel_block(self, L: _Layer, l: int, tensors: Tensors, mat, vec) -> _Layer:
        """Layer ``l`` of a parallel-block model: the input projections of all its mixers are stacked into ONE matrix
        (one GEMM per layer for q / k / v / gates / low-rank gate inputs); every mixer remembers its columns."""
        sp, p, dev = L.spec, f"l{l}.", self.device
        W = self.cfg.hidden_size
        L.f["norm1"] = vec(p + "norm1").reshape(-1)
        ls1 = vec(p + "ls1") if self.cfg.layer_scale else torch.ones(W, device=dev)
        col, mixes = 0, []
        blocks = []                       # row blocks of the fused projection, in float64
        for j, leaf in enumerate(sp.leaves):
            q = p + "mix." + (("left.", "right.")[j] if sp.mixer == "parallel" else "")
            mx = _Mix(spec=leaf, key=f"{l}.{j}", idx=j)
            if leaf.mixer == "latent_attention":
                for n, w in self._latent_rows(mx, q, tensors):
                    mx.off[n] = col
                    col += w.shape[0]
                    blocks.append(w)
            else:
                for n in _PROJ[leaf.mixer]:
                    mx.off[n] = col
                    col += tensors[q + n].shape[0]
                    blocks.append(tensors[q + n].to(device=dev, dtype=torch.float64))
            mx.w_o = mat(q + "o")
            if leaf.mixer == "latent_attention":
                pass
            elif leaf.mixer == "softmax_attention":
                mx.f["q.norm"], mx.f["k.norm"] = vec(q + "q.norm"), vec(q + "k.norm")
                if leaf.sink:
                    mx.f["sink"] = vec(q + "sink")
                rot = leaf.rot
                freq = rot.frequencies() if rot is not None and rot.dims > 0 else [0.0]
                mx.f["freq"] = torch.tensor(freq, dtype=torch.float64).to(device=dev, dtype=torch.float32)
                mx.amp = rot.amplitude if rot is not None else 1.0
            elif leaf.mixer == "mlstm":
                for n in ("i.b", "f.b", "norm"):
                    mx.f[n] = vec(q + n)
            elif leaf.mixer == "gla":
                mx.rank = tensors[q + "a1"].shape[0]
                mx.w2 = mat(q + "a2")
                mx.f["zbias"], mx.f["norm"] = vec(q + "a2.b"), vec(q + "norm")
            else:                                   # channel_delta: [a2 0; 0 g2] applied to the stacked [a1 | g1] outputs
                a2, g2 = tensors[q + "a2"].to(device=dev, dtype=torch.float32), tensors[q + "g2"].to(device=dev, dtype=torch.float32)
                mx.rank = a2.shape[1] + g2.shape[1]
                w2 = torch.zeros((a2.shape[0] + g2.shape[0], mx.rank), device=dev)
                w2[:a2.shape[0], :a2.shape[1]] = a2
                w2[a2.shape[0]:, a2.shape[1]:] = g2
                mx.w2 = ops.pad_weight(w2, 128, 64).to(self.dtype).contiguous()
                mx.f["conv"] = torch.cat([vec(q + n + ".conv") for n in ("q", "k", "v")], 0).contiguous()
                mx.f["zbias"], mx.f["A_log"], mx.f["norm"] = vec(q + "dt_bias"), vec(q + "A_log"), vec(q + "norm")
            if sp.mixer == "parallel":              # mean of the width-normed outputs: fold 1/n, the norm weight, layer scale
                mx.join_w = (vec(q + "out") * ls1 / len(sp.leaves)).contiguous()
                mx.join_norm = True
            else:
                mx.join_w = ls1 if self.cfg.layer_scale else None
            mixes.append(mx)
        L.mix = tuple(mixes)
        L.w_cat = ops.pad_weight(torch.cat(blocks, 0).to(torch.float32), 128, 64).to(self.dtype).contiguous()
        if sp.ff:
            if self.cfg.ff_norm:
                L.f["norm2"] = vec(p + "norm2")
            L.f["ls2"] = vec(p + "ls2") if self.cfg.layer_scale else None
            if sp.ff_kind == "moe":
                self._build_routed_ff(L, p, tensors)
                return L
            L.w_up, L.w_down = mat(p + "mlp.up"), mat(p + "mlp.down", k_mult=128)
            a = vec(p + "mlp.act")
            L.act_params = (float(F.softplus(a[0])), float(0.5 + F.softplus(a[1])))
            if L.f["ls2"] is None:
                L.f["ls2"] = torch.ones(W, device=dev)
        return L

    def _latent_rows(self, mx: _Mix, q: str, tensors: Tensors):
        """Row blocks (name, float64 matrix) that gated latent attention adds to the fused projection of its layer, and the
        mixer's own tensors.  Served with the keys absorbed: ``q_h . (U_k,h c) = (U_k,h^T q_h) . c``, so per head the query
        rows become ``[rotated part | U_k,h^T W_q,h]`` (``rot_dim + kv_rank`` channels) and attention runs over the cached
        rows ``[rotated key part | latent]``.  The values cannot be folded into the output projection (the output gate
        multiplies the concatenated heads in between): the per-head up-projections stay a tensor of their own.  Rotary
        pairs stored half-split (channel i with i + dims/2) are interleaved here, on the query rows and on the key rows
        alike, so that the kernels turn adjacent channels; the dot products do not notice."""
        sp, dev, f64 = mx.spec, self.device, torch.float64
        H, D, R, V, C = sp.heads, sp.dim, sp.rot_dim, sp.vdim, sp.kv_rank
        W = self.cfg.hidden_size
        wq = tensors[q + "q"].to(device=dev, dtype=f64).view(H, D + R, W)
        dkv = tensors[q + "dkv"].to(device=dev, dtype=f64)
        uk = tensors[q + "uk"].to(device=dev, dtype=f64).view(H, D, C)
        rd = sp.rot.dims if sp.rot is not None else 0
        perm = torch.arange(R, device=dev)
        if rd and sp.rot.half:
            perm[:rd] = torch.arange(rd, device=dev).view(2, rd // 2).t().reshape(-1)       # new 2i <- i, new 2i+1 <- i + rd/2
        qa = torch.cat([wq[:, D:][:, perm], torch.einsum("hdc,hdw->hcw", uk, wq[:, :D])], 1)     # [H, R + C, W]
        kv = torch.cat([dkv[:C], dkv[C:][perm]], 0)
        mx.f["dkv.norm"] = tensors[q + "dkv.norm"].to(device=dev, dtype=torch.float32).contiguous()
        mx.f["freq"], mx.f["freq_lo"] = ops.split_frequencies(sp.rot.frequencies() if rd else [0.0], dev)
        mx.amp = sp.rot.amplitude if rd else 1.0
        mx.w_uv = tensors[q + "uv"].to(device=dev, dtype=torch.float32).view(H, V, C).to(self.dtype).contiguous()
        rows = [("qa", qa.reshape(H * (R + C), W)), ("dkv", kv)]
        if sp.out_gate:
            rows.append(("g", tensors[q + "g"].to(device=dev, dtype=f64)))
        return rows

    def _build_routed_ff(self, L: _Layer, p: str, tensors: Tensors) -> None:
        """Gated experts chosen by their router logits, beside a shared expert: ONE up matrix ``[router | gate rows of
        the shared expert and of every expert | their up rows]`` and ONE down matrix with the down-projections side by
        side, so a token's weighted expert sum is a column scaling between two GEMMs (no sorting, no host)."""
        sp, dev, f64 = L.spec, self.device, torch.float64
        W = self.cfg.hidden_size
        names = (["shared"] if sp.shared_ff else []) + [f"e{e}" for e in range(sp.experts)]

        def t64(n):
            return tensors[n].to(device=dev, dtype=f64)

        router = t64(p + "mlp.router")
        pad = router.new_zeros(((-router.shape[0]) % 4, W))          # the blocks behind it start at multiples of four
        gates = torch.cat([t64(f"{p}mlp.{n}.gate") for n in names], 0)
        ups = torch.cat([t64(f"{p}mlp.{n}.up") for n in names], 0)
        n_r, n_h = router.shape[0] + pad.shape[0], gates.shape[0]
        L.ff_off = {"router": 0, "gate": n_r, "up": n_r + n_h, "hidden": n_h}
        L.w_up = ops.pad_weight(torch.cat([router, pad, gates, ups], 0).to(torch.float32), 128, 64).to(self.dtype).contiguous()
        down = torch.cat([t64(f"{p}mlp.{n}.down") for n in names], 1)
        L.w_down = ops.pad_weight(down.to(torch.float32), 128, 64).to(self.dtype).contiguous()

    def _alloc_mixer_state(self, mx: _Mix, num_pages: int) -> None:
        sp, dev, f32 = mx.spec, self.device, torch.float32
        key = self._key(mx)
        if sp.mixer == "latent_attention":      # one row per token: [rotated key part | latent]; the values are its latent slice
            self.k_cache[key] = torch.zeros((num_pages, ops.PAGE, 1, sp.rot_dim + sp.kv_rank), device=dev, dtype=self.dtype)
            self.v_cache[key] = self.k_cache[key][..., sp.rot_dim:]
            return
        if sp.mixer == "softmax_attention":
            self.k_cache[key] = torch.zeros((num_pages, ops.PAGE, sp.kv_heads, sp.dim), device=dev, dtype=self.dtype)
            self.v_cache[key] = torch.zeros((num_pages, ops.PAGE, sp.kv_heads, sp.vdim), device=dev, dtype=self.dtype)
            return
        self.state[key] = torch.zeros((self.state_slots, sp.heads, sp.dim, sp.vdim), device=dev, dtype=f32)
        if sp.mixer == "mlstm":
            self.nstate[key] = torch.zeros((self.state_slots, sp.heads, sp.dim), device=dev, dtype=f32)
            self.mstate[key] = torch.zeros((self.state_slots, sp.heads), device=dev, dtype=f32)
        elif sp.mixer == "channel_delta":
            ch, taps = mx.f["conv"].shape                 # the taps are the tensor's, whatever the config says
            self.conv_tail[key] = torch.zeros((self.state_slots, max(1, taps - 1), ch), device=dev, dtype=f32)

    def _forward_parallel_blocks(self, m) -> torch.Tensor:
        """x = scale * embed;  per layer: h = norm(x), x += sum of the layer-scaled mixer / feed-forward outputs (all
        read the same h);  logits = cap(head(norm(x))).  The join of layer l and the norm of layer l + 1 are one kernel."""
        c = self.cfg
        T, S, mq = m.n_tokens, m.n_seqs, m.max_q
        eps, W = c.norm_eps, c.hidden_size
        x = self.streams[:T].view(T, W)
        ops.hyb_embed(m.ids, m.positions, m.q_start, m.q_len, m.seq_slot, self.prev_tok, self.embed, None, 0, 0, 0,
                      self.streams[:T], S, mq, scale=c.embed_scale)
        h = self.h[:T]
        pend: list = []
        hcat = None
        if self.w_loop is not None:                  # operand of the loop's input matrix: [residual | embedding output]
            hcat = self._buf("loop", self.dtype, self.w_loop.shape[1])[:T]
            ops.act_cols(x, 0, hcat[:, W:], W, ops.COLS_COPY, T)
        for l, self._pass, enters in self.runs:
            L = self.L[l]
            replace = False
            if enters and hcat is not None:
                # the outputs of the layer before join the residual, which becomes the left half of the operand; the
                # product REPLACES the residual (joined by the norm kernel below)
                ops.ls_join(x, m.q_start, m.q_len, S, mq, terms=pend, h=hcat[:, :W])
                pend = [(ops.linear(self.w_loop, hcat, self._buf("yin", torch.float32, self.w_loop.shape[0])[:T]), None, False)]
                replace = True
            two = self.cfg.ff_norm and L.spec.ff > 0
            hf = self.h2[:T] if two else h           # what the feed-forward reads
            ops.ls_join(x, m.q_start, m.q_len, S, mq, terms=pend, gamma=L.f["norm1"], eps=eps, h=h, replace=replace,
                        gamma2=L.f["norm2"] if two else None, h2=hf if two else None)
            proj = ops.linear(L.w_cat, h, self._buf("proj", torch.float32, L.w_cat.shape[0])[:T])
            pend = []
            joins = []
            main = torch.cuda.current_stream()
            if self.overlap_ff and (L.spec.ff or len(L.mix) > 1):      # fork: h and the fused projection are queued
                fork = torch.cuda.Event()
                fork.record(main)

            def beside(stream, fn):
                """fn on ``stream`` behind the fork; the main stream joins before the next residual update"""
                with torch.cuda.stream(stream):
                    stream.wait_event(fork)
                    out = fn()
                    done = torch.cuda.Event()
                    done.record(stream)
                joins.append(done)
                return out

            yff = None
            if L.spec.ff and self.overlap_ff:
                yff = beside(self._side, lambda: self._ff(L, hf, T))
            for j, mx in enumerate(L.mix):
                run = getattr(self, "_mix_" + mx.spec.mixer)
                ybuf = self._buf(f"y{j}", torch.float32, mx.w_o.shape[0])[:T]
                if j > 0 and self.overlap_ff:
                    y = beside(self._side2, lambda: run(mx, proj, m, ybuf))
                else:
                    y = run(mx, proj, m, ybuf)
                pend.append((y, mx.join_w, mx.join_norm))
            if L.spec.ff:
                pend.append((yff if yff is not None else self._ff(L, hf, T), L.f["ls2"], False))
            for done in joins:
                main.wait_event(done)
            if self.debug_layers is not None:
                self.debug_layers.append(self._debug_join(x, pend, T))
        self._pass = 0
        R = m.n_out or S
        rows = m.last_idx if m.last_idx is not None else m.q_start
        xl = self.last_x[:R]
        ops.ls_join(x, m.q_start, m.q_len, S, mq, terms=pend, gamma=self.final_norm, eps=eps, h=xl, rows=rows, n_rows=R)
        logits = ops.linear(self.w_head, xl, self.logits[:R])
        if self.caps_logits:
            ops.act_cols(logits, 0, logits, logits.shape[1], ops.COLS_SOFTCAP, R, p0=c.final_softcap)
        return logits

    # ================================================================== post-norm layers (the norm follows the residual addition)
    def _build_post_norm_layer(self, L: _Layer, l: int, tensors: Tensors, mat, vec) -> _Layer:
        """Layer ``l`` of a post-norm model.  No norm sits in front of a sublayer (its input is the residual), so the residual gate of a sublayer
        is stacked under its input projections: ONE matrix per sublayer.  Latent attention is served in the absorbed form:
        per head the key up-projection is folded into the query up-projection (``q_h . (U_k c) = (U_k^T q_h) . c``) and
        the value up-projection into the output projection, so attention runs over the cached rows directly."""
        sp, p, dev = L.spec, f"l{l}.", self.device
        q = p + "mix."
        f64 = torch.float64

        def t64(n):
            return tensors[n].to(device=dev, dtype=f64)

        def stack(ws):
            return ops.pad_weight(torch.cat(ws, 0).to(torch.float32), 128, 64).to(self.dtype).contiguous()

        mx = _Mix(spec=sp, key=f"{l}.0", idx=0)
        W = self.cfg.hidden_size
        if sp.mixer == "latent_attention":
            H, D, R, V, C, Q = sp.heads, sp.dim, sp.rot_dim, sp.vdim, sp.kv_rank, sp.q_rank
            rows = [t64(q + "dq"), t64(q + "dkv")]
            mx.off.update({"dq": 0, "dkv": Q})
            uq, uk = t64(q + "uq").view(H, D + R, Q), t64(q + "uk").view(H, D, C)
            uv, wo = t64(q + "uv").view(H, V, C), t64(q + "o").view(W, H, V)
            qa = torch.cat([uq[:, D:], torch.einsum("hdc,hdq->hcq", uk, uq[:, :D])], 1)          # [H, R + C, Q]
            mx.w2 = stack([qa.reshape(H * (R + C), Q)])
            mx.w_o = stack([torch.einsum("whv,hvc->whc", wo, uv).reshape(W, H * C)])
            mx.rank = Q
            mx.f["dq.norm"], mx.f["dkv.norm"] = vec(q + "dq.norm"), vec(q + "dkv.norm")
            freq = sp.rot.frequencies() if sp.rot is not None and sp.rot.dims > 0 else [0.0]
            mx.f["freq"], mx.f["freq_lo"] = ops.split_frequencies(freq, dev)
        elif sp.mixer == "hgrn2":
            kd = sp.heads * sp.dim
            rows = [t64(q + "q"), t64(q + "f"), t64(q + "v")]
            mx.off.update({"q": 0, "f": kd, "v": 2 * kd})
            mx.w_o = mat(q + "o")
            for n in ("f.b", "lower", "norm"):
                mx.f[n] = vec(q + n)
        else:
            raise ValueError(f"{self.cfg.name}: layer {l} has mixer {sp.mixer!r}, which post-norm layers do not have")
        mx.off["rg"] = sum(r.shape[0] for r in rows)
        L.w_cat = stack(rows + [t64(p + "rg1")])
        L.f["rg1.b"], L.f["norm1"] = vec(p + "rg1.b"), vec(p + "norm1")
        L.mix = (mx,)
        if sp.ff:
            L.f["rg2.b"], L.f["norm2"] = vec(p + "rg2.b"), vec(p + "norm2")
            if sp.ff_kind == "moe":         # [router | residual gate | up-projections of all experts]; down-projections side by side
                ups = [t64(f"{p}mlp.e{e}.up") for e in range(sp.experts)]
                router = t64(p + "mlp.router")
                pad = router.new_zeros(((-router.shape[0]) % 4, W))      # the blocks behind it start at multiples of four
                L.w_up = stack([router, pad, t64(p + "rg2")] + ups)
                L.w_down = stack([torch.cat([t64(f"{p}mlp.e{e}.down") for e in range(sp.experts)], 1)])
                L.f["correction"] = vec(p + "mlp.correction")
            elif self.dtype == torch.bfloat16 and sp.ff % 64 == 0 and os.environ.get("B2B_POSTNORM_GLU", "0") == "1":
                # optional: the gated-silu epilogue of the tcgen05 GEMM writes the bf16 hidden rows itself (each 128-row tile
                # holds 64 gate and 64 up rows); the residual gate then needs a GEMM of its own with fp32 output.  Measured
                # on B200: prefill + 0.5 %, decode steps 2-4 % slower at widths 1024 / 2048 (two more GEMM launches per step
                # against two small elementwise launches less), so the stacked GEMM below is the default
                gu = ops.glu_interleave_rows(t64(p + "mlp.gate").float(), t64(p + "mlp.up").float())
                L.w_glu = ops.pad_weight(gu, 128, 64).to(self.dtype).contiguous()
                L.w_up = stack([t64(p + "rg2")])
                L.w_down = mat(p + "mlp.down")
            else:                           # [gate | up | residual gate], activation by a kernel of its own
                L.w_up = stack([t64(p + "mlp.gate"), t64(p + "mlp.up"), t64(p + "rg2")])
                L.w_down = mat(p + "mlp.down")
        return L

    def _forward_post_norm(self, m) -> torch.Tensor:
        """x = scale * embed;  per sublayer: x <- groupnorm(alpha x + sigmoid(R x + b) * sublayer(x)) * w;  logits =
        head(groupnorm(x) * w).  The residual lives in fp32; ``h`` is its copy in the operand type of the matrix products."""
        c = self.cfg
        T, S, mq = m.n_tokens, m.n_seqs, m.max_q
        W, f32 = c.hidden_size, torch.float32
        norm = dict(alpha=c.skip_scale, groups=c.norm_groups, eps=c.norm_eps)
        x = self.streams[:T].view(T, W)
        ops.hyb_embed(m.ids, m.positions, m.q_start, m.q_len, m.seq_slot, self.prev_tok, self.embed, None, 0, 0, 0,
                      self.streams[:T], S, mq, scale=c.embed_scale)
        h = self.h[:T]
        ops.act_cols(x, 0, h, W, ops.COLS_COPY, T)
        for l in self.layers:
            L = self.L[l]
            mx = L.mix[0]
            proj = ops.linear(L.w_cat, h, self._buf("proj", f32, L.w_cat.shape[0])[:T])
            y = getattr(self, "_mix_" + mx.spec.mixer)(mx, proj, m, self._buf("y0", f32, mx.w_o.shape[0])[:T])
            gate = dict(gate=proj, off_g=mx.off["rg"], gbias=L.f["rg1.b"]) if c.gated_residual else {}
            ops.post_norm_join(x, w=L.f["norm1"], h=h, y=y, **gate, **norm)
            if L.spec.ff:
                sp = L.spec
                p2 = ops.linear(L.w_up, h, self._buf("proj2", f32, L.w_up.shape[0])[:T])
                hid = self._buf("ff", self.dtype, L.w_down.shape[1])[:T]
                idw = None
                if sp.ff_kind == "moe":
                    n_out = ops.pad_to(sp.experts + sp.identity, 4)      # router rows (zero-padded), then gate, then experts
                    wt = self._buf("route", f32, max(1, sp.experts))[:T]
                    idw = self._buf("keep", f32, 1)[:T]
                    ops.moe_route(p2, 0, L.f["correction"], sp.experts, sp.route_groups, sp.route_keep, sp.top,
                                  sp.route_scale, wt, idw, T)
                    ops.gated_cols(p2, n_out + W, 0, hid, sp.experts * sp.expert_ff, ops.GATE_GELU, T, wt=wt, per=sp.expert_ff)
                    off_g = n_out
                    if not sp.identity:
                        idw = None
                elif L.w_glu is not None:
                    ops.gemm(L.w_glu, h, out=hid, epi=ops.EPI_GLU, act_gelu=ops.ACT_SILU)
                    off_g = 0
                else:
                    ops.gated_cols(p2, 0, sp.ff, hid, sp.ff, ops.GATE_SILU, T)
                    off_g = 2 * sp.ff
                y = ops.linear(L.w_down, hid, self._buf("yff", f32, L.w_down.shape[0])[:T])
                gate = dict(gate=p2, off_g=off_g, gbias=L.f["rg2.b"]) if c.gated_residual else {}
                ops.post_norm_join(x, w=L.f["norm2"], h=h, y=y, idw=idw, **gate, **norm)
            if self.debug_layers is not None:
                self.debug_layers.append(x[:T].clone())
        R = m.n_out or S
        rows = m.last_idx if m.last_idx is not None else m.q_start
        xl = self.last_x[:R]
        ops.post_norm_join(x, w=self.final_norm, h=xl, rows=rows, n_rows=R, alpha=1.0, groups=c.norm_groups, eps=c.norm_eps)
        return ops.linear(self.w_head, xl, self.logits[:R])

    def _mix_latent_attention(self, mx: _Mix, proj: torch.Tensor, m, y: torch.Tensor) -> torch.Tensor:
        sp, T = mx.spec, m.n_tokens
        H, R, C, Q, V = sp.heads, sp.rot_dim, sp.kv_rank, sp.q_rank, sp.vdim
        kc, vc = self.k_cache[self._key(mx)], self.v_cache[self._key(mx)]
        rdims = sp.rot.dims if sp.rot is not None else 0
        if Q > 0:                       # queries from a normed latent: a second GEMM gives the absorbed query rows
            cq = self._buf(f"cq{Q}", self.dtype, mx.w2.shape[1])[:T]
            ops.latent_prep(proj, mx.off["dq"], Q, mx.off["dkv"], C, R, mx.f["dq.norm"], mx.f["dkv.norm"], mx.f["freq"],
                            rdims, m.positions, m.slots, cq, kc, self.cfg.norm_eps, T, amp=mx.amp, freq_lo=mx.f["freq_lo"])
            qa, off_q = ops.linear(mx.w2, cq, self._buf("qa", torch.float32, mx.w2.shape[0])[:T]), 0
        else:                           # queries straight from the layer input: their absorbed rows are in the fused projection
            ops.latent_prep(proj, 0, 0, mx.off["dkv"], C, R, mx.f["dkv.norm"], mx.f["dkv.norm"], mx.f["freq"], rdims,
                            m.positions, m.slots, self.h[:T], kc, self.cfg.norm_eps, T, amp=mx.amp, freq_lo=mx.f["freq_lo"])
            qa, off_q = proj, mx.off["qa"]
        q = self._buf(f"q{mx.idx}", torch.float32, H * (R + C))[:T]
        ops.rot_heads(qa, off_q, q, H, R + C, mx.f["freq"], rdims, m.positions, T, slots=m.slots, amp=mx.amp,
                      freq_lo=mx.f["freq_lo"])
        ao = self._buf(f"mix{mx.idx}.{H * C}", self.dtype, ops.pad_to(H * C, 64))[:T]
        ops.softmax_attention(q, kc, vc, ao, m.block_table, m.q_start, m.q_len, m.kv_len, m.n_seqs, m.max_q, H, 1, R + C, C,
                              sp.window, sp.scale)
        if mx.w_uv is not None:         # values per head behind the attention, times the output gate of the concatenated heads
            go = self._buf(f"gate{mx.idx}.{H * V}", self.dtype, mx.w_o.shape[1])[:T]
            ops.head_up_gate(ao, mx.w_uv, go, T, H, V, C, gate=proj if sp.out_gate else None,
                             off_g=mx.off["g"] if sp.out_gate else 0)
            ao = go
        return ops.linear(mx.w_o, ao, y)

    def _mix_hgrn2(self, mx: _Mix, proj: torch.Tensor, m, y: torch.Tensor) -> torch.Tensor:
        sp, T = mx.spec, m.n_tokens
        H, dk, dv = sp.heads, sp.dim, sp.vdim
        o = self._buf("o0", torch.float32, H * dv)[:T]
        ops.lin_scan(ops.SCAN_HGRN2, proj, mx.off["q"], mx.off["q"], proj, mx.off["v"], self.state[self._key(mx)], o, m.q_start,
                     m.q_len, m.kv_len, m.seq_slot, m.n_seqs, m.max_q, H, H, dk, dv, z=proj, off_z=mx.off["f"],
                     zbias=mx.f["f.b"], hparam=mx.f["lower"])
        do = self._buf(f"mix0.{H * dv}", self.dtype, mx.w_o.shape[1])[:T]
        ops.scan_post(o, o, 0, mx.f["norm"], ops.POST_NONE, None, do, T, H, dv, self.cfg.norm_eps)
        return ops.linear(mx.w_o, do, y)

    def _ff(self, L: _Layer, h: torch.Tensor, T: int) -> torch.Tensor:
        """down(xIELU(up(h))): the activation is the epilogue of the up-projection; routed experts: see ``_ff_routed``"""
        if L.spec.ff_kind == "moe":
            return self._ff_routed(L, h, T)
        hid = self._buf("ff", self.dtype, L.w_up.shape[0])[:T]
        ops.linear(L.w_up, h, hid, act=ops.ACT_XIELU, act_params=L.act_params)
        return ops.linear(L.w_down, hid, self._buf("yff", torch.float32, L.w_down.shape[0])[:T])

    def _ff_routed(self, L: _Layer, h: torch.Tensor, T: int) -> torch.Tensor:
        """shared expert + the ``top`` experts with the largest router logits, weighted by the softmax over those logits:
        one GEMM (router logits, all gate rows, all up rows), the router, ``silu(gate) * up * weight`` per hidden column,
        one GEMM over the down-projections side by side"""
        sp, o, f32 = L.spec, L.ff_off, torch.float32
        p2 = ops.linear(L.w_up, h, self._buf("proj2", f32, L.w_up.shape[0])[:T])
        wt = self._buf("route", f32, max(1, sp.experts))[:T]
        idw = self._buf("keep", f32, 1)[:T]
        ops.moe_route(p2, o["router"], None, sp.experts, 1, 1, sp.top, 1.0, wt, idw, T)
        hid = self._buf("ff", self.dtype, L.w_down.shape[1])[:T]
        ops.gated_cols(p2, o["gate"], o["up"], hid, o["hidden"], ops.GATE_SILU, T, wt=wt, per=sp.expert_ff, both=True,
                       lead=sp.shared_ff)
        return ops.linear(L.w_down, hid, self._buf("yff", f32, L.w_down.shape[0])[:T])

    def _debug_join(self, x: torch.Tensor, terms, T: int) -> torch.Tensor:
        """the residual after the pending outputs have joined it (plain torch, tests only)"""
        W, eps = self.cfg.hidden_size, self.cfg.norm_eps
        v = x[:T].clone()
        for y, w, normed in terms:
            y = y[:T, :W]
            if normed:
                y = y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps)
            v += y * w if w is not None else y
        return v

    def _mix_softmax_attention(self, mx: _Mix, proj: torch.Tensor, m, y: torch.Tensor) -> torch.Tensor:
        sp, T = mx.spec, m.n_tokens
        H, G, D, V = sp.heads, sp.kv_heads, sp.dim, sp.vdim
        kc, vc = self.k_cache[self._key(mx)], self.v_cache[self._key(mx)]
        q = self._buf(f"q{mx.idx}", torch.float32, H * D)[:T]
        if sp.qk_norm == "head":        # a norm per head (one weight vector for all heads), no rotation, values as they are
            assert sp.rot is None and not sp.v_norm and mx.off["k"] == mx.off["q"] + H * D and mx.off["v"] == mx.off["k"] + G * D
            ops.attn_prep(proj[:, mx.off["q"]:], mx.f["q.norm"], mx.f["k.norm"], m.slots, q, kc, vc, T, H, G, D, V,
                          self.cfg.norm_eps)
        else:
            ops.rot_attn_prep(proj, mx.off["q"], mx.off["k"], mx.off["v"], mx.f["q.norm"], mx.f["k.norm"], mx.f["freq"],
                              sp.rot.dims if sp.rot is not None else 0, mx.amp, m.positions, m.slots, q, kc, vc, T, H, G, D,
                              V, self.cfg.norm_eps)
        ao = self._buf(f"mix{mx.idx}.{H * V}", self.dtype, mx.w_o.shape[1])[:T]
        ops.softmax_attention(q, kc, vc, ao, m.block_table, m.q_start, m.q_len, m.kv_len, m.n_seqs, m.max_q, H, G, D, V,
                              sp.window, sp.scale, softcap=sp.softcap, keep_first=sp.keep_first, sink=mx.f.get("sink"))
        return ops.linear(mx.w_o, ao, y)

    def _scan_out(self, mx: _Mix, o, gate, off_g, act, aux, m, y) -> torch.Tensor:
        sp, T = mx.spec, m.n_tokens
        do = self._buf(f"mix{mx.idx}.{sp.heads * sp.vdim}", self.dtype, mx.w_o.shape[1])[:T]
        ops.scan_post(o, gate, off_g, mx.f["norm"], act, aux, do, T, sp.heads, sp.vdim, self.cfg.norm_eps)
        return ops.linear(mx.w_o, do, y)

    def _mix_mlstm(self, mx: _Mix, proj: torch.Tensor, m, y: torch.Tensor) -> torch.Tensor:
        sp, T = mx.spec, m.n_tokens
        H, dk, dv = sp.heads, sp.dim, sp.vdim
        qs = dk ** -0.5
        aux = self._buf(f"aux{mx.idx}", torch.float32, 4 * H)[:T]
        ops.mlstm_gates(proj, mx.off["q"], mx.off["k"], mx.off["i"], mx.off["f"], mx.f["i.b"], mx.f["f.b"], sp.gate_cap, qs,
                        self.nstate[self._key(mx)], self.mstate[self._key(mx)], aux, m.q_start, m.q_len, m.kv_len, m.seq_slot, m.n_seqs,
                        H, dk)
        o = self._buf(f"o{mx.idx}", torch.float32, H * dv)[:T]
        ops.lin_scan(ops.SCAN_MLSTM, proj, mx.off["q"], mx.off["k"], proj, mx.off["v"], self.state[self._key(mx)], o, m.q_start,
                     m.q_len, m.kv_len, m.seq_slot, m.n_seqs, m.max_q, H, H, dk, dv, aux=aux, qscale=qs)
        return self._scan_out(mx, o, proj, mx.off["g"], 0, aux, m, y)

    def _low_rank(self, mx: _Mix, proj: torch.Tensor, off: int, T: int) -> torch.Tensor:
        """second level of the low-rank gate projections: columns off .. off + rank of the fused output -> operand -> GEMM"""
        lr = self._buf(f"lr{mx.idx}.{mx.rank}", self.dtype, mx.w2.shape[1])[:T]
        ops.act_cols(proj, off, lr, mx.rank, ops.COLS_COPY, T)
        return ops.linear(mx.w2, lr, self._buf(f"lora{mx.idx}", torch.float32, mx.w2.shape[0])[:T])

    def _mix_gla(self, mx: _Mix, proj: torch.Tensor, m, y: torch.Tensor) -> torch.Tensor:
        sp, T = mx.spec, m.n_tokens
        H, dk, dv = sp.heads, sp.dim, sp.vdim
        z = self._low_rank(mx, proj, mx.off["a1"], T)
        o = self._buf(f"o{mx.idx}", torch.float32, H * dv)[:T]
        ops.lin_scan(ops.SCAN_GLA, proj, mx.off["q"], mx.off["k"], proj, mx.off["v"], self.state[self._key(mx)], o, m.q_start,
                     m.q_len, m.kv_len, m.seq_slot, m.n_seqs, m.max_q, H, H, dk, dv, z=z, zbias=mx.f["zbias"],
                     qscale=dk ** -0.5, inv_tau=1.0 / sp.tau)
        return self._scan_out(mx, o, proj, mx.off["g"], 1, None, m, y)

    def _mix_channel_delta(self, mx: _Mix, proj: torch.Tensor, m, y: torch.Tensor) -> torch.Tensor:
        sp, T = mx.spec, m.n_tokens
        H, G, dk, dv = sp.heads, sp.kv_heads, sp.dim, sp.vdim
        cw = mx.f["conv"]
        conv = self._buf(f"conv{mx.idx}", torch.float32, cw.shape[0])[:T]
        ops.short_conv(proj, mx.off["q"], cw, self.conv_tail[self._key(mx)], conv, m.q_start, m.q_len, m.kv_len, m.seq_slot,
                       m.n_seqs, m.max_q)
        z = self._low_rank(mx, proj, mx.off["a1"], T)           # [decay steps (H * dk) | output gate (H * dv)]
        o = self._buf(f"o{mx.idx}", torch.float32, H * dv)[:T]
        ops.lin_scan(ops.SCAN_DELTA, conv, 0, G * dk, conv, 2 * G * dk, self.state[self._key(mx)], o, m.q_start, m.q_len,
                     m.kv_len, m.seq_slot, m.n_seqs, m.max_q, H, G, dk, dv, z=z, zbias=mx.f["zbias"], hparam=mx.f["A_log"],
                     beta=proj, off_b=mx.off["b"], qscale=dk ** -0.5)
        return self._scan_out(mx, o, z, H * dk, 0, None, m, y)

    def _debug_sum(self, st: torch.Tensor, pend, T: int) -> torch.Tensor:
        """sum of the streams after the pending sublayer output has joined them (plain torch, tests only)"""
        W, mult = self.cfg.hidden_size, self.cfg.residual_mult
        y, mix, outw = pend
        mix = mix if mix is not None else torch.ones((1, 1), device=st.device)
        outw = outw if outw is not None else torch.ones(1, device=st.device)
        new = torch.einsum("kj,tkw->tjw", mix, st) + mult * outw[None, :, None] * y[:T, None, :W]
        return new.sum(1).clone()

    def _attention(self, l: int, L: _Layer, h: torch.Tensor, m) -> torch.Tensor:
        sp, c = L.spec, self.cfg
        T = m.n_tokens
        H, G, D, V = sp.heads, sp.kv_heads, sp.dim, sp.vdim
        proj = ops.linear(L.w_cat, h, self._buf("proj", torch.float32, L.w_cat.shape[0])[:T])
        q = self._buf("q", torch.float32, H * D)[:T]
        ops.attn_prep(proj, L.f["q.norm"], L.f["k.norm"], m.slots, q, self.k_cache[l], self.v_cache[l], T, H, G, D, V,
                      c.norm_eps)
        ao = self._buf(f"mix{H * V}", self.dtype, L.w_o.shape[1])[:T]
        ops.sig_attention(q, self.k_cache[l], self.v_cache[l], proj, H * D + G * D + G * V, L.f["pb"], ao, m.block_table,
                          m.q_start, m.q_len, m.kv_len, m.n_seqs, m.max_q, H, G, D, V, sp.chunk, sp.scale)
        return ops.linear(L.w_o, ao, self._buf("y", torch.float32, L.w_o.shape[0])[:T])

    def _delta(self, l: int, L: _Layer, h: torch.Tensor, m) -> torch.Tensor:
        sp, c = L.spec, self.cfg
        T = m.n_tokens
        H, D = sp.heads, sp.dim
        d = H * D
        proj = ops.linear(L.w_cat, h, self._buf("proj", torch.float32, L.w_cat.shape[0])[:T])
        th = self._buf(f"lr{L.rank}", self.dtype, L.w2.shape[1])[:T]
        ops.act_cols(proj, 5 * d, th, L.rank, 1, T)                      # tanh of the low-rank decay projection
        lora = ops.linear(L.w2, th, self._buf("lora", torch.float32, L.w2.shape[0])[:T])
        o = self._buf("o", torch.float32, d)[:T]
        ops.delta_scan(proj, 0, d, 2 * d, 4 * d, lora, L.f["w0"], L.f["a.b"], self.state[l], o, m.q_start, m.q_len,
                       m.kv_len, m.seq_slot, m.n_seqs, m.max_q, H, D, D)
        do = self._buf(f"mix{d}", self.dtype, L.w_o.shape[1])[:T]
        ops.delta_post(o, proj, 3 * d, L.f["norm"], do, T, H, D, c.norm_eps)
        return ops.linear(L.w_o, do, self._buf("y", torch.float32, L.w_o.shape[0])[:T])
