"""Model architecture descriptions for the decoder families the mesh serves.

The reference ships no model configs (it defers to ``transformers``,
/root/reference/bee2bee/hf.py:23-32); these presets are the public architectures named in
BASELINE.json (distilgpt2, Llama-3-8B, Zephyr-7B-beta = Mistral-7B, gemma-2-2b) plus tiny
variants of each family for tests.  A config can also be read from a Hugging Face
``config.json`` (``ModelConfig.from_hf_dict``) so ``serve-hf --model <local dir>`` works.
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import asdict, dataclass, field
from typing import Dict, List, Optional, Tuple


@dataclass
class RotarySpec:
    """Rotary positions on the first ``dims`` channels of every head, channel 2i paired with 2i+1 (``half``: channel i
    paired with i + dims/2), frequency of pair i ``base ** (-2i / dims)``.  ``factor`` > 0: YaRN -- pairs that turn fewer than ``slow`` times within ``original``
    positions are slowed by ``factor``, pairs that turn more than ``fast`` times keep their frequency, a linear ramp in
    between; cos and sin are multiplied by ``0.1 ln(factor) + 1``."""
    dims: int = 0
    base: float = 10000.0
    factor: float = 0.0
    original: int = 0
    fast: float = 32.0
    slow: float = 1.0
    half: bool = False

    def frequencies(self) -> List[float]:
        """angle per position of every rotated pair (float64 arithmetic; the kernels round them to fp32)"""
        n = self.dims // 2
        f = [self.base ** (-2.0 * i / self.dims) for i in range(n)]
        if self.factor > 0:
            def turn_dim(turns: float) -> float:
                return self.dims * math.log(self.original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.base))
            lo = max(math.floor(turn_dim(self.fast)), 0)
            hi = min(math.ceil(turn_dim(self.slow)), self.dims - 1)
            for i in range(n):
                ramp = min(1.0, max(0.0, (i - lo) / max(hi - lo, 0.001)))
                f[i] = f[i] / self.factor * ramp + f[i] * (1.0 - ramp)
        return f

    @property
    def amplitude(self) -> float:
        return 0.1 * math.log(self.factor) + 1.0 if self.factor > 0 else 1.0


@dataclass
class LayerSpec:
    """One layer of a heterogeneous (hybrid) decoder: which token mixer it has and whether it has a feed-forward.

    ``mixer`` = "attention": gated sigmoid attention (no softmax, linear distance bias, keys limited to the query's
    block of ``chunk`` positions; 0 = all earlier keys) over ``kv_heads`` shared key/value heads.
    ``mixer`` = "general_delta": generalized delta-rule recurrence with a [dim, dim] fp32 state per head.
    ``mixer`` = "softmax_attention": causal softmax attention over the paged cache (``window`` > 0: only the last
    ``window`` keys), RMS norm over the whole q / k projection, optional rotary positions (``rot``), per-head value norm.
    ``mixer`` = "mlstm": matrix memory with exponential input gate, running maximum and normaliser (``gate_cap``).
    ``mixer`` = "gla": linear attention with a decay per key channel, ``sigmoid(z) ** (1 / tau)``, z low-rank.
    ``mixer`` = "channel_delta": delta rule with a decay per key channel, short convolutions (``conv`` taps) on q/k/v.
    ``mixer`` = "parallel": the mixers in ``sub`` read the same input; their width-normed outputs are averaged.
    ``mixer`` = "latent_attention": softmax attention whose keys and values are up-projections of one cached latent of
    ``kv_rank`` channels per token plus ``rot_dim`` rotated key channels shared by all heads; queries are produced from a
    latent of ``q_rank`` channels and carry ``dim`` plain + ``rot_dim`` rotated channels per head; ``window`` as above.
    ``mixer`` = "hgrn2": linear attention without keys: the write strength of a channel is the complement of its forget
    gate (which is bounded below by a learned vector), ``S <- diag(f) S + (1 - f) v^T``, read with ``silu`` queries.
    ``ff_kind`` = "moe": ``experts`` small feed-forwards (``expert_ff`` wide, no gate) of which a token uses ``top``,
    chosen by a softmax router; consecutive experts are bundled into ``route_groups`` equal groups and only the
    ``route_keep`` best-scoring groups may supply experts; the last
    ``identity`` outputs of the router bypass the experts (they hand the input through); weights are renormalised and multiplied by ``route_scale``.
    ``route_kind`` = "logit_topk": the ``top`` largest router logits are chosen and weighted by the softmax over the chosen
    logits alone; ``expert_gated``: an expert is ``down(silu(gate h) * up h)``; ``shared_ff`` > 0: one more expert of that
    width runs for every token with weight 1.
    Softmax attention options: ``qk_norm`` "whole" (RMS norm over the whole q / k projection) or "head" (per head, one
    weight vector shared by the heads); ``v_norm`` (values normed per head); ``softcap`` > 0 (``score <- cap tanh(score /
    cap)``); ``keep_first`` (with ``window``: the first keys stay visible); ``sink`` (a learned score per head joins the
    softmax denominator).  Latent attention: ``q_rank`` 0 = queries come straight from the layer input; ``out_gate``: the
    concatenated heads are multiplied by ``sigmoid(W_g h)`` in front of the output projection."""
    mixer: str = "attention"
    heads: int = 1
    kv_heads: int = 1
    dim: int = 64                    # query / key channels per head
    vdim: int = 64                   # value channels per head
    chunk: int = 0
    scale: float = 1.0               # score multiplier
    ff: int = 0                      # feed-forward width, 0 = the layer has no feed-forward sublayer
    ff_kind: str = "dense"
    window: int = 0                  # softmax attention: keys visible to a query, 0 = all earlier ones
    rot: Optional[RotarySpec] = None
    gate_cap: float = 0.0            # mlstm: soft cap of the gate pre-activations
    tau: float = 1.0                 # gla: decay temperature
    conv: int = 0                    # channel_delta: taps of the short convolution
    rank: int = 0                    # width of the low-rank gate projections (random init only; checkpoints: tensor shape)
    sub: Tuple["LayerSpec", ...] = ()
    q_rank: int = 0                  # latent attention: width of the query latent
    kv_rank: int = 0                 # latent attention: width of the cached key/value latent
    rot_dim: int = 0                 # latent attention: rotated channels per query head = width of the shared rotated key
    experts: int = 0                 # moe: real experts
    top: int = 0                     # moe: experts (identity ones included) a token uses
    expert_ff: int = 0               # moe: hidden width of one expert
    route_groups: int = 1
    route_keep: int = 1
    identity: int = 0                # moe: router outputs that pass the feed-forward input through unchanged
    route_scale: float = 1.0
    route_kind: str = "softmax_corrected"
    expert_gated: bool = False
    shared_ff: int = 0
    qk_norm: str = "whole"
    v_norm: bool = True
    softcap: float = 0.0
    keep_first: int = 0
    sink: bool = False
    out_gate: bool = False

    @property
    def leaves(self) -> Tuple["LayerSpec", ...]:
        return self.sub if self.mixer == "parallel" else (self,)


@dataclass
class ModelConfig:
    name: str = "tiny-llama"
    family: str = "llama"            # gpt2 | llama | mistral | gemma2 | kepovik | repudra | lonulix | fisopel
    vocab_size: int = 512
    hidden_size: int = 256
    n_layers: int = 2
    n_heads: int = 2
    n_kv_heads: int = 1
    head_dim: int = 128
    ffn_size: int = 512
    max_position: int = 8192
    norm: str = "rms"                # rms | ln
    norm_eps: float = 1e-5
    act: str = "silu"                # silu | gelu_tanh
    glu: bool = True
    rope_theta: float = 10000.0      # <= 0: learned absolute positions (GPT-2)
    tie_embeddings: bool = False
    bias: bool = False               # GPT-2 style biases on every linear
    sliding_window: int = 0          # 0 = full attention
    window_pattern: str = "all"      # all | alternate (Gemma-2: even layers are local)
    attn_softcap: float = 0.0
    final_softcap: float = 0.0
    query_scale: float = 0.0         # 0 -> 1/sqrt(head_dim); Gemma-2: query_pre_attn_scalar ** -0.5
    post_norms: bool = False         # Gemma-2 post-attention / post-FFN norms
    gemma_norm: bool = False         # RMSNorm weight stored as (w - 1)
    embed_scale: float = 1.0         # Gemma: sqrt(hidden)
    eos_token_id: int = -1
    bos_token_id: int = -1
    # ---- hybrid graphs (family "kepovik"): per-layer mixers, several residual streams, hashed token-pair embedding
    layer_specs: Tuple[LayerSpec, ...] = ()
    streams: int = 0                 # residual streams mixed by hyper-connections; 0 = one plain residual
    residual_mult: float = 1.0       # every sublayer output is scaled by this before it joins the residual
    pair_buckets: int = 0            # rows of the hashed (previous token, token) table, 0 = none (+1 row for "no previous")
    pair_mul_prev: int = 0
    pair_mul_cur: int = 0
    block_layout: str = "sequential"  # sequential: norm -> mixer -> join, norm -> ff -> join; parallel: one norm feeds both;
    #                                   post_norm: x <- norm(skip_scale * x + sublayer(x)), no norm in front of a sublayer
    norm_groups: int = 1             # post_norm: the RMS norm is taken over this many consecutive parts of the width
    skip_scale: float = 1.0          # post_norm: the residual is multiplied by this before the sublayer result is added
    gated_residual: bool = False     # post_norm: sublayer results are multiplied by sigmoid(W x + b) before the sum
    scalar_norm: bool = False        # block / model norms have ONE gain (a single number) instead of one per coordinate
    layer_scale: bool = False        # sublayer outputs are multiplied coordinate-wise by learned vectors before the join
    ff_norm: bool = False            # parallel blocks: the feed-forward reads a norm of its own (norm2) of the same residual
    # layers loop_start .. loop_stop-1 run loop_times times in a row with the same weights (a cache per pass); with loop_in, the
    # residual entering each pass is replaced by W_in [x ; embedding output]
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1
    loop_in: bool = False

    # ------------------------------------------------------------------ derived
    @property
    def hybrid(self) -> bool:
        return bool(self.layer_specs)

    @property
    def recurrent(self) -> bool:
        """True when some layer keeps per-sequence state besides the paged KV cache (no prefix sharing, no piece split)."""
        return any(leaf.mixer not in ("attention", "softmax_attention", "latent_attention")
                   for sp in self.layer_specs for leaf in sp.leaves) \
            or self.pair_buckets > 0

    def layer_runs(self) -> List[Tuple[int, int, bool]]:
        """(layer, pass, first layer of a pass of the loop) in execution order"""
        n = self.n_layers
        if self.loop_stop <= self.loop_start:
            return [(l, 0, False) for l in range(n)]
        runs = [(l, 0, False) for l in range(self.loop_start)]
        for p in range(max(1, self.loop_times)):
            runs += [(l, p, l == self.loop_start) for l in range(self.loop_start, self.loop_stop)]
        return runs + [(l, 0, False) for l in range(self.loop_stop, n)]

    @property
    def q_dim(self) -> int:
        return self.n_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.n_kv_heads * self.head_dim

    @property
    def softmax_scale(self) -> float:
        return self.query_scale if self.query_scale > 0 else 1.0 / math.sqrt(self.head_dim)

    def layer_window(self, layer: int) -> int:
        if self.sliding_window <= 0:
            return 0
        if self.window_pattern == "alternate":
            return self.sliding_window if layer % 2 == 0 else 0
        return self.sliding_window

    def param_count(self) -> int:
        if self.hybrid:
            from .weights import hybrid_tensor_specs
            n = 0
            for _, shape, _ in hybrid_tensor_specs(self, range(self.n_layers), True, True):
                k = 1
                for v in shape:
                    k *= v
                n += k
            return n
        h, f = self.hidden_size, self.ffn_size
        per = h * (self.q_dim + 2 * self.kv_dim) + self.q_dim * h + (3 if self.glu else 2) * h * f
        emb = self.vocab_size * h * (1 if self.tie_embeddings else 2)
        return self.n_layers * per + emb

    def to_dict(self) -> Dict:
        return asdict(self)

    # --------------------------------------------------------------- HF interop
    @staticmethod
    def from_kepovik_dict(d: Dict, name: str = "") -> "ModelConfig":
        """``config.json`` of a Kepovik checkpoint: ``layers`` lists {type, mixer sizes, mlp | null} per layer."""
        specs = []
        for lay in d["layers"]:
            m, mlp = lay.get("mixer") or {}, lay.get("mlp")
            kind = lay["type"]
            if kind not in ("attention", "general_delta"):
                raise ValueError(f"{name or 'kepovik'}: unknown layer type {kind!r}")
            if mlp and mlp.get("kind", "dense") != "dense":
                raise ValueError(f"{name or 'kepovik'}: feed-forward kind {mlp.get('kind')!r} is not implemented")
            heads, dim = int(m["heads"]), int(m["dim"])
            specs.append(LayerSpec(mixer=kind, heads=heads, kv_heads=int(m.get("kv_heads", heads)), dim=dim,
                                   vdim=int(m.get("vdim", dim)), chunk=int((m.get("mask") or {}).get("size", 0)),
                                   scale=float(m.get("scale", 1.0)), ff=int(mlp["ff"]) if mlp else 0))
        pair = (d.get("embedding") or {}).get("bigram") or {}
        width = int(d["width"])
        att = [sp for sp in specs if sp.mixer == "attention"] or specs
        return ModelConfig(
            name=name or "kepovik", family="kepovik", vocab_size=int(d["vocab"]), hidden_size=width, n_layers=len(specs),
            n_heads=max(sp.heads for sp in att), n_kv_heads=max(sp.kv_heads for sp in att),
            head_dim=max(sp.dim for sp in att), ffn_size=max([sp.ff for sp in specs] + [0]), max_position=1 << 30,
            norm="rms", norm_eps=float((d.get("norm") or {}).get("eps", 1e-6)), act="relu_sq", glu=False, rope_theta=0.0,
            gemma_norm=True, layer_specs=tuple(specs), streams=int(d.get("streams", 0)),
            residual_mult=float(d.get("residual_mult", 1.0)), pair_buckets=int(pair.get("buckets", 0)),
            pair_mul_prev=int(pair.get("mul_prev", 0)), pair_mul_cur=int(pair.get("mul_cur", 0)))

    def to_kepovik_dict(self) -> Dict:
        layers = []
        for sp in self.layer_specs:
            if sp.mixer == "attention":
                m = {"dim": sp.dim, "heads": sp.heads, "kv_heads": sp.kv_heads, "scale": sp.scale, "vdim": sp.vdim}
                if sp.chunk:
                    m["mask"] = {"size": sp.chunk}
            else:
                m = {"dim": sp.dim, "heads": sp.heads}
            layers.append({"type": sp.mixer, "mixer": m, "mlp": {"ff": sp.ff, "kind": sp.ff_kind} if sp.ff else None})
        d = {"architecture": "Kepovik", "layers": layers, "norm": {"eps": self.norm_eps},
             "residual_mult": self.residual_mult, "vocab": self.vocab_size, "width": self.hidden_size}
        if self.streams:
            d["streams"] = self.streams
        if self.pair_buckets:
            d["embedding"] = {"bigram": {"buckets": self.pair_buckets, "mul_prev": self.pair_mul_prev,
                                         "mul_cur": self.pair_mul_cur}}
        return d

    @staticmethod
    def from_repudra_dict(d: Dict, name: str = "") -> "ModelConfig":
        """``config.json`` of a Repudra checkpoint: ``layers`` lists {type, mixer sizes, mlp | null} per layer; types
        ``parallel`` (softmax attention beside an mLSTM matrix memory), ``gla``, ``channel_delta``."""
        who = name or "repudra"

        def leaf(kind: str, m: Dict) -> LayerSpec:
            heads, dim = int(m["heads"]), int(m["dim"])
            rot = None
            if m.get("rot"):
                r = m["rot"]
                sc = r.get("scaling") or {}
                rot = RotarySpec(dims=int(r["dims"]), base=float(r["base"]), factor=float(sc.get("factor", 0.0)),
                                 original=int(sc.get("original", 0)), fast=float(sc.get("fast", 32.0)),
                                 slow=float(sc.get("slow", 1.0)))
                if rot.dims % 2 or rot.dims > dim:
                    raise ValueError(f"{who}: rotary dims {rot.dims} do not fit a head of {dim} channels")
            return LayerSpec(mixer=kind, heads=heads, kv_heads=int(m.get("kv_heads", heads)), dim=dim,
                             vdim=int(m.get("vdim", dim)), scale=float(m.get("scale", dim ** -0.5)),
                             window=int(m.get("window", 0) or 0), rot=rot, gate_cap=float(m.get("gate_cap", 0.0)),
                             tau=float(m.get("tau", 1.0)), conv=int(m.get("conv", 0)), rank=int(m.get("rank", 0)))

        specs = []
        for lay in d["layers"]:
            m, mlp, kind = lay.get("mixer") or {}, lay.get("mlp"), lay["type"]
            if mlp and mlp.get("kind", "dense") != "dense":
                raise ValueError(f"{who}: feed-forward kind {mlp.get('kind')!r} is not implemented")
            ff = int(mlp["ff"]) if mlp else 0
            if kind == "parallel":
                left, right = leaf("softmax_attention", m["left"]), leaf("mlstm", m["right"])
                sp = LayerSpec(mixer="parallel", heads=left.heads, kv_heads=left.kv_heads, dim=left.dim, vdim=left.vdim,
                               scale=left.scale, sub=(left, right))
            elif kind in ("gla", "channel_delta"):
                sp = leaf(kind, m)
            else:
                raise ValueError(f"{who}: unknown layer type {kind!r}")
            sp.ff = ff
            for lf in sp.leaves:
                if lf.heads % lf.kv_heads:
                    raise ValueError(f"{who}: {lf.heads} heads cannot share {lf.kv_heads} key heads")
            specs.append(sp)
        width = int(d["width"])
        att = [lf for sp in specs for lf in sp.leaves if lf.mixer == "softmax_attention"] or specs
        return ModelConfig(
            name=name or "repudra", family="repudra", vocab_size=int(d["vocab"]), hidden_size=width, n_layers=len(specs),
            n_heads=max(sp.heads for sp in att), n_kv_heads=max(sp.kv_heads for sp in att),
            head_dim=max(sp.dim for sp in att), ffn_size=max([sp.ff for sp in specs] + [0]), max_position=1 << 30,
            norm="rms", norm_eps=float((d.get("norm") or {}).get("eps", 1e-6)), act="xielu", glu=False, rope_theta=0.0,
            embed_scale=float((d.get("embedding") or {}).get("scale", 1.0)),
            final_softcap=float(d.get("logit_softcap") or 0.0), layer_specs=tuple(specs), streams=0,
            block_layout="parallel", scalar_norm=True, layer_scale=True)

    def to_repudra_dict(self) -> Dict:
        def leaf(sp: LayerSpec) -> Dict:
            if sp.mixer == "softmax_attention":
                m = {"dim": sp.dim, "heads": sp.heads, "kv_heads": sp.kv_heads, "scale": sp.scale, "vdim": sp.vdim}
                if sp.window:
                    m["window"] = sp.window
                if sp.rot:
                    m["rot"] = {"base": sp.rot.base, "dims": sp.rot.dims}
                    if sp.rot.factor > 0:
                        m["rot"]["scaling"] = {"factor": sp.rot.factor, "fast": sp.rot.fast,
                                               "original": sp.rot.original, "slow": sp.rot.slow}
                return m
            m = {"dim": sp.dim, "heads": sp.heads, "vdim": sp.vdim}
            if sp.mixer == "mlstm":
                m["gate_cap"] = sp.gate_cap
            elif sp.mixer == "gla":
                m["tau"] = sp.tau
            else:
                m.update({"conv": sp.conv, "kv_heads": sp.kv_heads})
            if sp.rank:
                m["rank"] = sp.rank
            return m

        layers = []
        for sp in self.layer_specs:
            mixer = {"left": leaf(sp.sub[0]), "right": leaf(sp.sub[1])} if sp.mixer == "parallel" else leaf(sp)
            layers.append({"type": sp.mixer, "mixer": mixer, "mlp": {"ff": sp.ff, "kind": sp.ff_kind} if sp.ff else None})
        return {"architecture": "Repudra", "embedding": {"scale": self.embed_scale}, "layers": layers,
                "logit_softcap": self.final_softcap, "norm": {"eps": self.norm_eps}, "vocab": self.vocab_size,
                "width": self.hidden_size}

    @staticmethod
    def from_lonulix_dict(d: Dict, name: str = "") -> "ModelConfig":
        """``config.json`` of a Lonulix checkpoint: ``layers`` lists {type, mixer sizes, mlp | null} per layer; types
        ``latent_attention`` and ``hgrn2``; ``mlp.kind`` ``dense`` (gated, silu) or ``moe`` (routed gelu experts)."""
        who = name or "lonulix"
        specs = []
        for lay in d["layers"]:
            m, mlp, kind = lay.get("mixer") or {}, lay.get("mlp"), lay["type"]
            heads, dim = int(m["heads"]), int(m["dim"])
            vdim = int(m.get("vdim", dim))
            if kind == "latent_attention":
                rot_dim = int(m.get("rot_dim", 0))
                r = m.get("rot") or {}
                rot = RotarySpec(dims=int(r.get("dims", rot_dim)), base=float(r.get("base", 10000.0))) if rot_dim else None
                if rot is not None and (rot.dims % 2 or rot.dims > rot_dim):
                    raise ValueError(f"{who}: rotary dims {rot.dims} do not fit {rot_dim} rotated channels")
                sp = LayerSpec(mixer=kind, heads=heads, kv_heads=1, dim=dim, vdim=vdim,
                               scale=float(m.get("scale", (dim + rot_dim) ** -0.5)),
                               window=int((m.get("mask") or {}).get("size", 0) or 0), rot=rot,
                               q_rank=int(m["q_rank"]), kv_rank=int(m["kv_rank"]), rot_dim=rot_dim)
            elif kind == "hgrn2":
                sp = LayerSpec(mixer=kind, heads=heads, kv_heads=heads, dim=dim, vdim=vdim)
            else:
                raise ValueError(f"{who}: unknown layer type {kind!r}")
            if mlp:
                fk = mlp.get("kind", "dense")
                if fk == "dense":
                    sp.ff = int(mlp["ff"])
                elif fk == "moe":
                    r, g = mlp["router"], (mlp["router"].get("groups") or {})
                    sp.ff_kind, sp.expert_ff = "moe", int(mlp["expert"]["ff"])
                    sp.experts, sp.top, sp.identity = int(r["experts"]), int(r["top"]), int(r.get("identity", 0))
                    sp.route_groups, sp.route_keep = int(g.get("count", 1)), int(g.get("keep", g.get("count", 1)))
                    sp.route_scale = float(r.get("scale", 1.0))
                    sp.ff = sp.experts * sp.expert_ff
                    if (sp.experts + sp.identity) % sp.route_groups:
                        raise ValueError(f"{who}: {sp.experts + sp.identity} router outputs do not form {sp.route_groups} equal groups")
                else:
                    raise ValueError(f"{who}: feed-forward kind {fk!r} is not implemented")
            specs.append(sp)
        width = int(d["width"])
        norm = d.get("norm") or {}
        if width % int(norm.get("groups", 1)):
            raise ValueError(f"{who}: width {width} does not split into {norm.get('groups')} norm groups")
        att = [sp for sp in specs if sp.mixer == "latent_attention"] or specs
        return ModelConfig(
            name=name or "lonulix", family="lonulix", vocab_size=int(d["vocab"]), hidden_size=width, n_layers=len(specs),
            n_heads=max(sp.heads for sp in att), n_kv_heads=1, head_dim=max(sp.dim + sp.rot_dim for sp in att),
            ffn_size=max([sp.ff for sp in specs] + [0]), max_position=1 << 30, norm="rms",
            norm_eps=float(norm.get("eps", 1e-6)), act="silu", glu=True, rope_theta=0.0,
            embed_scale=float((d.get("embedding") or {}).get("scale", 1.0)), layer_specs=tuple(specs), streams=0,
            block_layout="post_norm", norm_groups=int(norm.get("groups", 1)),
            skip_scale=float(d.get("postln_alpha", 1.0)), gated_residual=True)

    def to_lonulix_dict(self) -> Dict:
        layers = []
        for sp in self.layer_specs:
            if sp.mixer == "latent_attention":
                m = {"dim": sp.dim, "heads": sp.heads, "kv_rank": sp.kv_rank, "q_rank": sp.q_rank, "rot_dim": sp.rot_dim,
                     "scale": sp.scale, "vdim": sp.vdim}
                if sp.rot is not None:
                    m["rot"] = {"base": sp.rot.base, "dims": sp.rot.dims}
                if sp.window:
                    m["mask"] = {"size": sp.window}
            else:
                m = {"dim": sp.dim, "heads": sp.heads, "vdim": sp.vdim}
            if not sp.ff:
                mlp = None
            elif sp.ff_kind == "moe":
                mlp = {"expert": {"ff": sp.expert_ff}, "kind": "moe",
                       "router": {"experts": sp.experts, "groups": {"count": sp.route_groups, "keep": sp.route_keep},
                                  "identity": sp.identity, "scale": sp.route_scale, "top": sp.top}}
            else:
                mlp = {"ff": sp.ff, "kind": "dense"}
            layers.append({"type": sp.mixer, "mixer": m, "mlp": mlp})
        return {"architecture": "Lonulix", "embedding": {"scale": self.embed_scale}, "layers": layers,
                "norm": {"eps": self.norm_eps, "groups": self.norm_groups}, "postln_alpha": self.skip_scale,
                "vocab": self.vocab_size, "width": self.hidden_size}

    @staticmethod
    def from_fisopel_dict(d: Dict, name: str = "") -> "ModelConfig":
        """``config.json`` of a Fisopel checkpoint: ``layers`` lists {type, mixer sizes, mlp | null}; types ``attention``
        (grouped heads, per-head q / k norm, capped scores, window with kept first keys, sink) and ``latent_attention``
        (gated); ``mlp.kind`` ``moe`` (gated silu experts beside a shared one); ``loop`` repeats a range of layers."""
        who = name or "fisopel"
        specs = []
        for lay in d["layers"]:
            m, mlp, kind = lay.get("mixer") or {}, lay.get("mlp"), lay["type"]
            heads, dim = int(m["heads"]), int(m["dim"])
            vdim = int(m.get("vdim", dim))
            if kind == "attention":
                mask = m.get("mask") or {}
                sp = LayerSpec(mixer="softmax_attention", heads=heads, kv_heads=int(m.get("kv_heads", heads)), dim=dim,
                               vdim=vdim, scale=float(m.get("scale", dim ** -0.5)), window=int(mask.get("size", 0) or 0),
                               keep_first=int(mask.get("keep_first", 0) or 0), softcap=float(m.get("softcap", 0.0) or 0.0),
                               qk_norm="head", v_norm=False, sink=True)
                if sp.heads % sp.kv_heads:
                    raise ValueError(f"{who}: {sp.heads} heads cannot share {sp.kv_heads} key heads")
            elif kind == "latent_attention":
                rot_dim = int(m.get("rot_dim", 0))
                r = m.get("rot") or {}
                sc = r.get("scaling") or {}
                rot = RotarySpec(dims=int(r.get("dims", rot_dim)), base=float(r.get("base", 10000.0)),
                                 factor=float(sc.get("factor", 0.0)), original=int(sc.get("original", 0)),
                                 fast=float(sc.get("fast", 32.0)), slow=float(sc.get("slow", 1.0)), half=True) if rot_dim else None
                if rot is not None and (rot.dims % 2 or rot.dims > rot_dim):
                    raise ValueError(f"{who}: rotary dims {rot.dims} do not fit {rot_dim} rotated channels")
                sp = LayerSpec(mixer=kind, heads=heads, kv_heads=1, dim=dim, vdim=vdim,
                               scale=float(m.get("scale", (dim + rot_dim) ** -0.5)), rot=rot, q_rank=0,
                               kv_rank=int(m["kv_rank"]), rot_dim=rot_dim, out_gate=True)
            else:
                raise ValueError(f"{who}: unknown layer type {kind!r}")
            if mlp:
                if mlp.get("kind", "moe") != "moe":
                    raise ValueError(f"{who}: feed-forward kind {mlp.get('kind')!r} is not implemented")
                r = mlp["router"]
                sp.ff_kind, sp.expert_ff, sp.experts, sp.top = "moe", int(mlp["expert"]["ff"]), int(r["experts"]), int(r["top"])
                sp.route_kind, sp.expert_gated = "logit_topk", True
                sp.shared_ff = int((mlp.get("shared") or {}).get("ff", 0))
                sp.ff = sp.experts * sp.expert_ff + sp.shared_ff
                if not 0 < sp.top <= sp.experts:
                    raise ValueError(f"{who}: {sp.top} of {sp.experts} experts cannot be chosen")
            specs.append(sp)
        width, n = int(d["width"]), len(specs)
        loop = d.get("loop") or {}
        start, stop = int(loop.get("start", 0)), int(loop.get("stop", 0))
        if loop and not (0 <= start < stop <= n and int(loop.get("times", 1)) >= 1):
            raise ValueError(f"{who}: loop {loop!r} does not fit {n} layers")
        att = [sp for sp in specs if sp.mixer == "softmax_attention"] or specs
        return ModelConfig(
            name=name or "fisopel", family="fisopel", vocab_size=int(d["vocab"]), hidden_size=width, n_layers=n,
            n_heads=max(sp.heads for sp in att), n_kv_heads=max(sp.kv_heads for sp in att),
            head_dim=max(sp.dim for sp in att), ffn_size=max([sp.ff for sp in specs] + [0]), max_position=1 << 30,
            norm="rms", norm_eps=float((d.get("norm") or {}).get("eps", 1e-6)), act="silu", glu=True, rope_theta=0.0,
            tie_embeddings=True, embed_scale=float((d.get("embedding") or {}).get("scale", 1.0)),
            layer_specs=tuple(specs), streams=0, block_layout="parallel", ff_norm=True, loop_start=start if loop else 0,
            loop_stop=stop if loop else 0, loop_times=int(loop.get("times", 1)), loop_in=bool(loop))

    def to_fisopel_dict(self) -> Dict:
        layers = []
        for sp in self.layer_specs:
            if sp.mixer == "softmax_attention":
                m = {"dim": sp.dim, "heads": sp.heads, "kv_heads": sp.kv_heads, "scale": sp.scale, "softcap": sp.softcap,
                     "vdim": sp.vdim}
                if sp.window:
                    m["mask"] = {"keep_first": sp.keep_first, "size": sp.window}
            else:
                m = {"dim": sp.dim, "heads": sp.heads, "kv_rank": sp.kv_rank, "rot_dim": sp.rot_dim, "scale": sp.scale,
                     "vdim": sp.vdim}
                if sp.rot is not None:
                    m["rot"] = {"base": sp.rot.base, "dims": sp.rot.dims}
                    if sp.rot.factor > 0:
                        m["rot"]["scaling"] = {"factor": sp.rot.factor, "fast": sp.rot.fast,
                                               "original": sp.rot.original, "slow": sp.rot.slow}
            mlp = None
            if sp.ff:
                mlp = {"expert": {"ff": sp.expert_ff}, "kind": "moe", "router": {"experts": sp.experts, "top": sp.top}}
                if sp.shared_ff:
                    mlp["shared"] = {"ff": sp.shared_ff}
            layers.append({"type": "attention" if sp.mixer == "softmax_attention" else sp.mixer, "mixer": m, "mlp": mlp})
        d = {"architecture": "Fisopel", "embedding": {"scale": self.embed_scale}, "layers": layers,
             "norm": {"eps": self.norm_eps}, "vocab": self.vocab_size, "width": self.hidden_size}
        if self.loop_in:
            d["loop"] = {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}
        return d

    @staticmethod
    def from_hf_dict(d: Dict, name: str = "") -> "ModelConfig":
        if str(d.get("architecture", "")).lower() == "fisopel":
            return ModelConfig.from_fisopel_dict(d, name)
        if str(d.get("architecture", "")).lower() == "lonulix":
            return ModelConfig.from_lonulix_dict(d, name)
        if str(d.get("architecture", "")).lower() == "kepovik":
            return ModelConfig.from_kepovik_dict(d, name)
        if str(d.get("architecture", "")).lower() == "repudra":
            return ModelConfig.from_repudra_dict(d, name)
        mt = d.get("model_type", "llama")
        if mt == "gpt2":
            h = d.get("n_embd", 768)
            nh = d.get("n_head", 12)
            return ModelConfig(
                name=name or "gpt2", family="gpt2", vocab_size=d.get("vocab_size", 50257), hidden_size=h,
                n_layers=d.get("n_layer", 12), n_heads=nh, n_kv_heads=nh, head_dim=h // nh,
                ffn_size=d.get("n_inner") or 4 * h, max_position=d.get("n_positions", 1024), norm="ln",
                norm_eps=d.get("layer_norm_epsilon", 1e-5), act="gelu_tanh", glu=False, rope_theta=0.0,
                tie_embeddings=True, bias=True, eos_token_id=d.get("eos_token_id", 50256),
                bos_token_id=d.get("bos_token_id", 50256))
        # checkpoints the loader would map wrongly are rejected instead of loading "successfully" 
        if d.get("attention_bias") or d.get("mlp_bias"):
            raise ValueError(f"{name or mt}: attention_bias / mlp_bias checkpoints (Qwen-style) are not supported: "
                             "the weight map carries no bias tensors for this family")
        rs = d.get("rope_scaling")
        if rs and (rs.get("rope_type") or rs.get("type") or "default") not in ("default",):
            raise ValueError(f"{name or mt}: rope_scaling {rs!r} is not implemented (plain RoPE only)")
        h = d["hidden_size"]
        nh = d["num_attention_heads"]
        hd = d.get("head_dim") or h // nh
        common = dict(
            name=name or mt, vocab_size=d["vocab_size"], hidden_size=h, n_layers=d["num_hidden_layers"], n_heads=nh,
            n_kv_heads=d.get("num_key_value_heads", nh), head_dim=hd, ffn_size=d["intermediate_size"],
            max_position=d.get("max_position_embeddings", 8192), norm="rms", norm_eps=d.get("rms_norm_eps", 1e-5),
            rope_theta=float(d.get("rope_theta", 10000.0)), tie_embeddings=bool(d.get("tie_word_embeddings", False)),
            eos_token_id=_first_int(d.get("eos_token_id", -1)), bos_token_id=_first_int(d.get("bos_token_id", -1)))
        if mt == "gemma2":
            return ModelConfig(
                family="gemma2", act="gelu_tanh", glu=True, sliding_window=d.get("sliding_window", 4096),
                window_pattern="alternate", attn_softcap=float(d.get("attn_logit_softcapping") or 0.0),
                final_softcap=float(d.get("final_logit_softcapping") or 0.0),
                query_scale=float(d.get("query_pre_attn_scalar", hd)) ** -0.5, post_norms=True, gemma_norm=True,
                embed_scale=math.sqrt(h), **{**common, "tie_embeddings": True})
        if mt == "mistral":
            return ModelConfig(family="mistral", act="silu", glu=True, sliding_window=d.get("sliding_window") or 0,
                               **common)
        return ModelConfig(family="llama", act="silu", glu=True, **common)

    def to_hf_dict(self) -> Dict:
        """A ``config.json`` that ``transformers`` accepts for this architecture (Kepovik: its own format)."""
        if self.family == "kepovik":
            return self.to_kepovik_dict()
        if self.family == "repudra":
            return self.to_repudra_dict()
        if self.family == "lonulix":
            return self.to_lonulix_dict()
        if self.family == "fisopel":
            return self.to_fisopel_dict()
        if self.family == "gpt2":
            return {"model_type": "gpt2", "architectures": ["GPT2LMHeadModel"], "vocab_size": self.vocab_size,
                    "n_embd": self.hidden_size, "n_layer": self.n_layers, "n_head": self.n_heads,
                    "n_positions": self.max_position, "n_ctx": self.max_position, "n_inner": self.ffn_size,
                    "activation_function": "gelu_new", "layer_norm_epsilon": self.norm_eps,
                    "bos_token_id": self.bos_token_id, "eos_token_id": self.eos_token_id,
                    "resid_pdrop": 0.0, "embd_pdrop": 0.0, "attn_pdrop": 0.0}
        base = {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
                "num_hidden_layers": self.n_layers, "num_attention_heads": self.n_heads,
                "num_key_value_heads": self.n_kv_heads, "head_dim": self.head_dim,
                "intermediate_size": self.ffn_size, "max_position_embeddings": self.max_position,
                "rms_norm_eps": self.norm_eps, "rope_theta": self.rope_theta,
                "tie_word_embeddings": self.tie_embeddings, "bos_token_id": self.bos_token_id,
                "eos_token_id": self.eos_token_id, "attention_bias": False, "mlp_bias": False,
                "attention_dropout": 0.0}
        if self.family == "gemma2":
            base.update({"model_type": "gemma2", "architectures": ["Gemma2ForCausalLM"],
                         "hidden_activation": "gelu_pytorch_tanh", "sliding_window": self.sliding_window,
                         "attn_logit_softcapping": self.attn_softcap or None,
                         "final_logit_softcapping": self.final_softcap or None,
                         "query_pre_attn_scalar": round(self.softmax_scale ** -2)})
        elif self.family == "mistral":
            base.update({"model_type": "mistral", "architectures": ["MistralForCausalLM"], "hidden_act": "silu",
                         "sliding_window": self.sliding_window or None})
        else:
            base.update({"model_type": "llama", "architectures": ["LlamaForCausalLM"], "hidden_act": "silu"})
        return base


def _first_int(v) -> int:
    if isinstance(v, (list, tuple)):
        return int(v[0]) if v else -1
    return -1 if v is None else int(v)


def _gpt2(name, layers, hidden, heads):
    return ModelConfig(name=name, family="gpt2", vocab_size=50257, hidden_size=hidden, n_layers=layers, n_heads=heads,
                       n_kv_heads=heads, head_dim=hidden // heads, ffn_size=4 * hidden, max_position=1024, norm="ln",
                       norm_eps=1e-5, act="gelu_tanh", glu=False, rope_theta=0.0, tie_embeddings=True, bias=True,
                       eos_token_id=50256, bos_token_id=50256)


PRESETS: Dict[str, ModelConfig] = {
    "distilgpt2": _gpt2("distilgpt2", 6, 768, 12),
    "gpt2": _gpt2("gpt2", 12, 768, 12),
    "llama-3-8b": ModelConfig(name="llama-3-8b", family="llama", vocab_size=128256, hidden_size=4096, n_layers=32,
                              n_heads=32, n_kv_heads=8, head_dim=128, ffn_size=14336, max_position=8192,
                              norm_eps=1e-5, rope_theta=500000.0, eos_token_id=128001, bos_token_id=128000),
    "zephyr-7b-beta": ModelConfig(name="zephyr-7b-beta", family="mistral", vocab_size=32000, hidden_size=4096,
                                  n_layers=32, n_heads=32, n_kv_heads=8, head_dim=128, ffn_size=14336,
                                  max_position=32768, norm_eps=1e-5, rope_theta=10000.0, sliding_window=4096,
                                  eos_token_id=2, bos_token_id=1),
    "gemma-2-2b": ModelConfig(name="gemma-2-2b", family="gemma2", vocab_size=256000, hidden_size=2304, n_layers=26,
                              n_heads=8, n_kv_heads=4, head_dim=256, ffn_size=9216, max_position=8192,
                              norm_eps=1e-6, act="gelu_tanh", rope_theta=10000.0, tie_embeddings=True,
                              sliding_window=4096, window_pattern="alternate", attn_softcap=50.0, final_softcap=30.0,
                              query_scale=256 ** -0.5, post_norms=True, gemma_norm=True,
                              embed_scale=math.sqrt(2304), eos_token_id=1, bos_token_id=2),
    # tiny variants (tests / smoke): same code paths, kernel-friendly shapes
    "tiny-llama": ModelConfig(name="tiny-llama", family="llama", vocab_size=512, hidden_size=256, n_layers=4,
                              n_heads=4, n_kv_heads=2, head_dim=128, ffn_size=512, rope_theta=500000.0,
                              eos_token_id=1, bos_token_id=0),
    "tiny-mistral": ModelConfig(name="tiny-mistral", family="mistral", vocab_size=512, hidden_size=256, n_layers=4,
                                n_heads=4, n_kv_heads=2, head_dim=128, ffn_size=512, sliding_window=96,
                                eos_token_id=1, bos_token_id=0),
    "tiny-gemma2": ModelConfig(name="tiny-gemma2", family="gemma2", vocab_size=512, hidden_size=256, n_layers=4,
                               n_heads=2, n_kv_heads=1, head_dim=256, ffn_size=512, norm_eps=1e-6, act="gelu_tanh",
                               tie_embeddings=True, sliding_window=96, window_pattern="alternate", attn_softcap=50.0,
                               final_softcap=30.0, query_scale=256 ** -0.5, post_norms=True, gemma_norm=True,
                               embed_scale=16.0, eos_token_id=1, bos_token_id=0),
    "tiny-gpt2": _gpt2("tiny-gpt2", 4, 128, 2),
    # Llama-3-8B layer shapes (hidden 4096, GQA 32:8, FFN 14336), 8 layers, small vocabulary: multi-GPU correctness
    # tests at the real GEMM / handoff tile shapes without 16 GB of weights
    "mini-llama-4096": ModelConfig(name="mini-llama-4096", family="llama", vocab_size=32000, hidden_size=4096,
                                   n_layers=8, n_heads=32, n_kv_heads=8, head_dim=128, ffn_size=14336,
                                   rope_theta=500000.0, eos_token_id=1, bos_token_id=0),
}
def _kepovik(name, width, vocab, layers, streams=2, mult=0.5, buckets=251):
    specs = []
    for kind, heads, kv, dim, vdim, chunk, ff in layers:
        specs.append(LayerSpec(mixer=kind, heads=heads, kv_heads=kv, dim=dim, vdim=vdim, chunk=chunk,
                               scale=dim ** -0.5, ff=ff))
    att = [sp for sp in specs if sp.mixer == "attention"] or specs
    return ModelConfig(name=name, family="kepovik", vocab_size=vocab, hidden_size=width, n_layers=len(specs),
                       n_heads=max(sp.heads for sp in att), n_kv_heads=max(sp.kv_heads for sp in att),
                       head_dim=max(sp.dim for sp in att), ffn_size=max(sp.ff for sp in specs), max_position=1 << 30,
                       norm="rms", norm_eps=1e-6, act="relu_sq", glu=False, rope_theta=0.0, gemma_norm=True,
                       layer_specs=tuple(specs), streams=streams, residual_mult=mult, pair_buckets=buckets,
                       pair_mul_prev=13, pair_mul_cur=5, eos_token_id=-1, bos_token_id=-1)


# hybrid test preset: two attention layers (grouped KV heads, 96-position blocks) around two delta-rule layers
PRESETS["tiny-kepovik"] = _kepovik("tiny-kepovik", 128, 512, [
    ("attention", 4, 2, 32, 64, 96, 256), ("general_delta", 2, 2, 32, 32, 0, 0),
    ("general_delta", 2, 2, 32, 32, 0, 256), ("attention", 4, 2, 32, 64, 96, 0)])


def _repudra(name, width, vocab, layers, softcap=20.0):
    """layers: ("parallel", (H, G, D, V, rot dims), (H, D, V), ff) | ("gla", H, D, V, ff) | ("channel_delta", H, G, D, V, ff)"""
    specs = []
    for lay in layers:
        if lay[0] == "parallel":
            (h, g, d, v, rd), (rh, rdim, rv), ff = lay[1], lay[2], lay[3]
            rot = RotarySpec(dims=rd, base=100000.0, factor=4.0, original=1024) if rd else None
            left = LayerSpec(mixer="softmax_attention", heads=h, kv_heads=g, dim=d, vdim=v, scale=d ** -0.5, rot=rot)
            right = LayerSpec(mixer="mlstm", heads=rh, kv_heads=rh, dim=rdim, vdim=rv, gate_cap=12.0)
            specs.append(LayerSpec(mixer="parallel", heads=h, kv_heads=g, dim=d, vdim=v, scale=left.scale, ff=ff,
                                   sub=(left, right)))
        elif lay[0] == "gla":
            _, h, d, v, ff = lay
            specs.append(LayerSpec(mixer="gla", heads=h, kv_heads=h, dim=d, vdim=v, tau=8.0, ff=ff))
        else:
            _, h, g, d, v, ff = lay
            specs.append(LayerSpec(mixer="channel_delta", heads=h, kv_heads=g, dim=d, vdim=v, conv=4, ff=ff))
    att = [lf for sp in specs for lf in sp.leaves if lf.mixer == "softmax_attention"] or specs
    return ModelConfig(name=name, family="repudra", vocab_size=vocab, hidden_size=width, n_layers=len(specs),
                       n_heads=max(sp.heads for sp in att), n_kv_heads=max(sp.kv_heads for sp in att),
                       head_dim=max(sp.dim for sp in att), ffn_size=max(sp.ff for sp in specs), max_position=1 << 30,
                       norm="rms", norm_eps=1e-5, act="xielu", glu=False, rope_theta=0.0, embed_scale=width ** 0.5,
                       final_softcap=softcap, layer_specs=tuple(specs), block_layout="parallel", scalar_norm=True,
                       layer_scale=True, eos_token_id=-1, bos_token_id=-1)


# parallel-block hybrid test preset: attention + matrix memory, diag-gated linear attention, channel-decay delta rule
PRESETS["tiny-repudra"] = _repudra("tiny-repudra", 128, 512, [
    ("parallel", (4, 2, 32, 48, 16), (2, 32, 32), 256), ("gla", 2, 32, 64, 256), ("channel_delta", 4, 2, 32, 32, 0),
    ("parallel", (4, 2, 32, 48, 16), (2, 32, 32), 0)])


def _lonulix(name, width, vocab, layers, groups=2, alpha=2.0, embed_scale=2.0):
    """layers: ("latent_attention", H, dim, rot_dim, vdim, q_rank, kv_rank, window, mlp) | ("hgrn2", H, dim, vdim, mlp);
    mlp: 0 (none) | ff (dense) | (experts, expert_ff, top, groups, keep, identity, scale)"""
    specs = []
    for lay in layers:
        if lay[0] == "latent_attention":
            _, h, d, r, v, qr, kr, win, mlp = lay
            sp = LayerSpec(mixer="latent_attention", heads=h, kv_heads=1, dim=d, vdim=v, scale=(d + r) ** -0.5, window=win,
                           rot=RotarySpec(dims=r, base=10000.0) if r else None, q_rank=qr, kv_rank=kr, rot_dim=r)
        else:
            _, h, d, v, mlp = lay
            sp = LayerSpec(mixer="hgrn2", heads=h, kv_heads=h, dim=d, vdim=v)
        if isinstance(mlp, tuple):
            e, eff, top, gc, gk, ident, sc = mlp
            sp.ff_kind, sp.experts, sp.expert_ff, sp.top, sp.route_groups, sp.route_keep = "moe", e, eff, top, gc, gk
            sp.identity, sp.route_scale, sp.ff = ident, sc, e * eff
        else:
            sp.ff = int(mlp)
        specs.append(sp)
    att = [sp for sp in specs if sp.mixer == "latent_attention"] or specs
    return ModelConfig(name=name, family="lonulix", vocab_size=vocab, hidden_size=width, n_layers=len(specs),
                       n_heads=max(sp.heads for sp in att), n_kv_heads=1, head_dim=max(sp.dim + sp.rot_dim for sp in att),
                       ffn_size=max(sp.ff for sp in specs), max_position=1 << 30, norm="rms", norm_eps=1e-5, act="silu",
                       glu=True, rope_theta=0.0, embed_scale=embed_scale, layer_specs=tuple(specs),
                       block_layout="post_norm", norm_groups=groups, skip_scale=alpha, gated_residual=True,
                       eos_token_id=-1, bos_token_id=-1)


# post-norm hybrid test preset: latent attention (window 48) with routed experts, HGRN2 with a dense gated feed-forward,
# HGRN2 without a feed-forward, latent attention over all earlier keys with a dense feed-forward
PRESETS["tiny-lonulix"] = _lonulix("tiny-lonulix", 128, 512, [
    ("latent_attention", 4, 16, 8, 24, 48, 40, 48, (6, 64, 2, 4, 2, 2, 1.5)), ("hgrn2", 2, 32, 48, 192),
    ("hgrn2", 4, 16, 16, 0), ("latent_attention", 2, 32, 16, 32, 64, 32, 0, 256)])


def _fisopel(name, width, vocab, layers, loop=None, embed_scale=2.0):
    """layers: ("attention", H, G, dim, vdim, window, keep_first, softcap, mlp) | ("latent_attention", H, dim, rot_dim, vdim,
    kv_rank, yarn factor, mlp); mlp: 0 (none) | (experts, expert_ff, top, shared_ff); loop: (start, stop, times)"""
    specs = []
    for lay in layers:
        if lay[0] == "attention":
            _, h, g, d, v, win, keep, cap, mlp = lay
            sp = LayerSpec(mixer="softmax_attention", heads=h, kv_heads=g, dim=d, vdim=v, scale=d ** -0.5, window=win,
                           keep_first=keep, softcap=cap, qk_norm="head", v_norm=False, sink=True)
        else:
            _, h, d, r, v, kr, fac, mlp = lay
            rot = RotarySpec(dims=r, base=10000.0, factor=fac, original=64 if fac > 0 else 0, half=True) if r else None
            sp = LayerSpec(mixer="latent_attention", heads=h, kv_heads=1, dim=d, vdim=v, scale=(d + r) ** -0.5, rot=rot,
                           q_rank=0, kv_rank=kr, rot_dim=r, out_gate=True)
        if mlp:
            e, eff, top, sh = mlp
            sp.ff_kind, sp.experts, sp.expert_ff, sp.top, sp.shared_ff = "moe", e, eff, top, sh
            sp.route_kind, sp.expert_gated, sp.ff = "logit_topk", True, e * eff + sh
        specs.append(sp)
    att = [sp for sp in specs if sp.mixer == "softmax_attention"] or specs
    lp = loop or (0, 0, 1)
    return ModelConfig(name=name, family="fisopel", vocab_size=vocab, hidden_size=width, n_layers=len(specs),
                       n_heads=max(sp.heads for sp in att), n_kv_heads=max(sp.kv_heads for sp in att),
                       head_dim=max(sp.dim for sp in att), ffn_size=max(sp.ff for sp in specs), max_position=1 << 30,
                       norm="rms", norm_eps=1e-5, act="silu", glu=True, rope_theta=0.0, tie_embeddings=True,
                       embed_scale=embed_scale, layer_specs=tuple(specs), block_layout="parallel", ff_norm=True,
                       loop_start=lp[0], loop_stop=lp[1], loop_times=lp[2], loop_in=loop is not None,
                       eos_token_id=-1, bos_token_id=-1)


# looped parallel-block test preset: windowed attention with kept first keys and a sink + routed experts, gated latent
# attention (YaRN rotary part) + routed experts, both run twice; then latent attention without a feed-forward
PRESETS["tiny-fisopel"] = _fisopel("tiny-fisopel", 128, 512, [
    ("attention", 4, 2, 32, 16, 40, 6, 30.0, (6, 32, 2, 48)), ("latent_attention", 3, 16, 16, 24, 48, 4.0, (5, 32, 3, 0)),
    ("latent_attention", 2, 32, 8, 32, 40, 0.0, 0)], loop=(0, 2, 2))
PRESETS["tiny-gpt2"].vocab_size = 384
PRESETS["tiny-gpt2"].eos_token_id = 1
PRESETS["tiny-gpt2"].bos_token_id = 0

ALIASES = {
    "meta-llama/meta-llama-3-8b": "llama-3-8b", "meta-llama/llama-3-8b": "llama-3-8b", "llama3": "llama-3-8b",
    "llama-3-8b-instruct": "llama-3-8b", "huggingfaceh4/zephyr-7b-beta": "zephyr-7b-beta",
    "zephyr": "zephyr-7b-beta", "mistral-7b": "zephyr-7b-beta", "google/gemma-2-2b": "gemma-2-2b",
    "gemma2:2b": "gemma-2-2b", "gemma2": "gemma-2-2b", "distilbert/distilgpt2": "distilgpt2",
    "openai-community/gpt2": "gpt2",
}


def resolve_config(model: str) -> ModelConfig:
    """Preset name, alias, or a local directory containing ``config.json``."""
    if os.path.isdir(model) and os.path.exists(os.path.join(model, "config.json")):
        with open(os.path.join(model, "config.json")) as f:
            return ModelConfig.from_hf_dict(json.load(f), name=os.path.basename(os.path.normpath(model)))
    key = model.lower()
    key = ALIASES.get(key, key)
    if key in PRESETS:
        return PRESETS[key]
    tail = key.split("/")[-1]
    tail = ALIASES.get(tail, tail)
    if tail in PRESETS:
        return PRESETS[tail]
    raise KeyError(f"unknown model '{model}' (presets: {sorted(PRESETS)})")


def split_layers(n_layers: int, pieces: int) -> List[range]:
    """Contiguous layer ranges, earlier pieces take the remainder (26 over 4 -> 7/7/6/6)."""
    pieces = max(1, min(pieces, n_layers))
    base, rem = divmod(n_layers, pieces)
    out, start = [], 0
    for i in range(pieces):
        n = base + (1 if i < rem else 0)
        out.append(range(start, start + n))
        start += n
    return out


def balanced_split(cfg: "ModelConfig", pieces: int) -> List[range]:
    """Contiguous layer ranges that minimise the heaviest piece when the last piece also streams the
    lm_head (Llama-3-8B: the 1.05 GB head weighs 2.4 decoder layers) -- the wavefront runs at the pace
    of its slowest stage.  Falls back to ``split_layers`` when the head is negligible."""
    pieces = max(1, min(pieces, cfg.n_layers))
    h, f = cfg.hidden_size, cfg.ffn_size
    layer = h * (cfg.q_dim + 2 * cfg.kv_dim) + cfg.q_dim * h + (3 if cfg.glu else 2) * h * f
    head = cfg.vocab_size * h
    if pieces == 1 or head < 0.5 * layer:
        return split_layers(cfg.n_layers, pieces)
    best, best_cost = None, None
    for last_n in range(1, cfg.n_layers - pieces + 2):
        rest = split_layers(cfg.n_layers - last_n, pieces - 1)
        cost = max(max(len(r) for r in rest) * layer, last_n * layer + head)
        if best_cost is None or cost <= best_cost:     # ties -> the more even split (larger last piece)
            best, best_cost = rest + [range(cfg.n_layers - last_n, cfg.n_layers)], cost
    return best


def supports_half_layer_pieces(cfg: "ModelConfig") -> bool:
    """A piece boundary may fall between the attention and the MLP block of a layer when both boundary GEMMs
    are the fused kinds the handoff needs: O-proj with residual epilogue (tail) and gate/up with the RMSNorm
    folded in (head) -- the Llama / Mistral graphs."""
    return cfg.norm == "rms" and not cfg.post_norms and cfg.glu and not cfg.bias


UNITS_PER_LAYER = 3       # attention block (QKV GEMM, attention, O-proj) | gate/up GEMM | down GEMM


def piece_units(cfg: "ModelConfig", pieces: int, bounds: Optional[List[int]] = None) -> List[tuple]:
    """Piece boundaries in THIRD-OF-A-LAYER units: unit 3l is the attention block of layer l (QKV GEMM, attention,
    O-proj), 3l+1 its gate/up GEMM, 3l+2 its down GEMM -- any GEMM can be the fused tail GEMM of a piece and any GEMM
    its head.  Returns ``pieces`` contiguous ``(u0, u1)`` ranges that minimise the heaviest stage of the wavefront under
    a bytes-plus-launch-latency cost model (a decode step is weight-bandwidth bound with a few us of fixed cost per
    kernel); the last piece also carries the lm_head and the sampler.  Llama-3-8B over 8 GPUs: whole layers give
    5/4/4/4/4/4/4/3 (+head) = 0.81 of the ideal stage time, half layers (round 1) 0.92, thirds 0.97.  ``bounds``
    overrides the search (tests).  Graphs without the fused RMSNorm / GLU epilogues are cut at whole layers."""
    UPL = UNITS_PER_LAYER
    U = UPL * cfg.n_layers
    if cfg.hybrid:
        return [(0, U)]          # recurrent state and residual streams are not handed between GPUs: one piece
    if bounds is not None:
        assert bounds[0] == 0 and bounds[-1] == U and all(a < b for a, b in zip(bounds, bounds[1:])), bounds
        return list(zip(bounds[:-1], bounds[1:]))
    pieces = max(1, min(pieces, cfg.n_layers))
    if pieces == 1 or not supports_half_layer_pieces(cfg):
        return [(UPL * r.start, UPL * r.stop) for r in balanced_split(cfg, pieces)]
    # stage time model fitted to the measured decode step (profiles/decode_layer_breakdown.md, B200, 32 sequences):
    # weight bytes at the measured 6.4 TB/s plus a fixed cost per kernel; the last piece adds the lm_head GEMM and the
    # sampler.  Llama-3-8B: attention block 34.1 us (measured 34.7), gate/up 40.7 (39.4), down 25.3 (24.9), head 201 (211).
    h, f = cfg.hidden_size, cfg.ffn_size
    us_per_elem = 2.0 / 6.4e6                            # bf16 element -> microseconds of HBM streaming
    launch = 7.0
    attn = (h * (cfg.q_dim + 2 * cfg.kv_dim) + cfg.q_dim * h) * us_per_elem + 3 * launch
    gu = 2 * h * f * us_per_elem + 4.0
    down = h * f * us_per_elem + launch
    head = cfg.vocab_size * h * us_per_elem + launch + 30.0
    cost = [(attn, gu, down)[u % UPL] for u in range(U)]
    pre = [0.0]
    for c in cost:
        pre.append(pre[-1] + c)
    INF = float("inf")
    # best[k][u]: minimal max-stage cost of covering units [0, u) with k pieces
    best = [[INF] * (U + 1) for _ in range(pieces + 1)]
    arg = [[0] * (U + 1) for _ in range(pieces + 1)]
    best[0][0] = 0.0
    for k in range(1, pieces + 1):
        for u in range(k, U + 1):
            for v in range(k - 1, u - 1):          # every piece spans >= 2 units (no lone GEMM)
                if best[k - 1][v] == INF:
                    continue
                stage = pre[u] - pre[v] + (head if (k == pieces and u == U) else 0.0)
                c = max(best[k - 1][v], stage)
                if c < best[k][u]:
                    best[k][u], arg[k][u] = c, v
    out, u = [], U
    for k in range(pieces, 0, -1):
        v = arg[k][u]
        out.append((v, u))
        u = v
    return out[::-1]


def unit_layers(units: tuple) -> range:
    """layers touched by a ``(u0, u1)`` unit range"""
    return range(units[0] // UNITS_PER_LAYER, (units[1] - 1) // UNITS_PER_LAYER + 1)
