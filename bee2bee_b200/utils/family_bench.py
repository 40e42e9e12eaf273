"""Side-by-side throughput of two model families at equal size (``bench.py --families``): the hybrid Kepovik graph
next to the closest uniform decoder (Llama), or (``--family repudra``) the parallel-block Repudra graph next to the
closest hybrid (Kepovik), or (``--family lonulix``) the post-norm Lonulix graph next to Repudra (the other family whose
attention and recurrences run on the kernels of ``csrc/seqmix.cu``), or (``--family fisopel``) the looped Fisopel graph next
to Lonulix (the other family with latent attention and routed experts); random weights, layer shapes of real models.

Per width it reports (1) prefill and decode tokens/s through the same ``GpuRunner`` calls that serving uses (chunked
graph prefill, CUDA-graph decode steps), timed with CUDA events, and (2) a per-kernel breakdown of one eager prefill
chunk and one eager decode step: device time per entry point, algorithmic FLOPs and bytes, and the fraction of the
measured roofline (max of FLOPs / measured bf16 GEMM peak and bytes / measured copy bandwidth) -- L2 is flushed before
every timed kernel, so the fractions are cold-cache figures that compare the two families, not absolute bests.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List

import torch

from ..models.config import LayerSpec, ModelConfig, RotarySpec

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def kepovik_sized(width: int, vocab: int = 32000, chunk: int = 256, streams: int = 4) -> ModelConfig:
    """six layers: attention+ff, delta, attention+ff, delta+ff, attention, delta; 128-wide heads"""
    H = width // 128
    a = LayerSpec(mixer="attention", heads=H, kv_heads=max(1, H // 4), dim=128, vdim=128, chunk=chunk, scale=128 ** -0.5,
                  ff=4 * width)
    d = LayerSpec(mixer="general_delta", heads=H, kv_heads=H, dim=128, vdim=128)
    a0 = LayerSpec(mixer="attention", heads=H, kv_heads=max(1, H // 4), dim=128, vdim=128, chunk=chunk, scale=128 ** -0.5)
    dff = LayerSpec(mixer="general_delta", heads=H, kv_heads=H, dim=128, vdim=128, ff=4 * width)
    specs = (a, d, a, dff, a0, d)
    return ModelConfig(name=f"mini-kepovik-{width}", family="kepovik", vocab_size=vocab, hidden_size=width,
                       n_layers=len(specs), n_heads=H, n_kv_heads=max(1, H // 4), head_dim=128, ffn_size=4 * width,
                       max_position=1 << 30, norm="rms", norm_eps=1e-6, act="relu_sq", glu=False, rope_theta=0.0,
                       gemma_norm=True, layer_specs=specs, streams=streams, residual_mult=0.5, pair_buckets=65521,
                       pair_mul_prev=13, pair_mul_cur=5)


def repudra_sized(width: int, vocab: int = 32000) -> ModelConfig:
    """six parallel-block layers with 128-wide heads: attention (GQA 4:1, rotary on half of each head, YaRN) beside an
    mLSTM + ff, GLA + ff, channel-decay delta rule + ff, then the same three mixers without feed-forward; the layer matrices
    hold 52.1 - 52.8 width^2 parameters, ``kepovik_sized(width)`` 52.5 - 52.7 width^2"""
    H = width // 128
    rot = RotarySpec(dims=64, base=500000.0, factor=4.0, original=8192)

    def par(ff):
        left = LayerSpec(mixer="softmax_attention", heads=H, kv_heads=max(1, H // 4), dim=128, vdim=128, scale=128 ** -0.5,
                         rot=rot)
        right = LayerSpec(mixer="mlstm", heads=max(1, H // 2), kv_heads=max(1, H // 2), dim=128, vdim=128, gate_cap=12.0)
        return LayerSpec(mixer="parallel", heads=H, kv_heads=left.kv_heads, dim=128, vdim=128, scale=left.scale, ff=ff,
                         sub=(left, right))

    def gla(ff):
        return LayerSpec(mixer="gla", heads=H, kv_heads=H, dim=128, vdim=128, tau=8.0, rank=64, ff=ff)

    def cd(ff):
        return LayerSpec(mixer="channel_delta", heads=H, kv_heads=H, dim=128, vdim=128, conv=4, rank=64, ff=ff)

    specs = (par(4 * width), gla(4 * width), cd(4 * width), par(0), gla(0), cd(0))
    return ModelConfig(name=f"mini-repudra-{width}", family="repudra", vocab_size=vocab, hidden_size=width,
                       n_layers=len(specs), n_heads=H, n_kv_heads=max(1, H // 4), head_dim=128, ffn_size=4 * width,
                       max_position=1 << 30, norm="rms", norm_eps=1e-5, act="xielu", glu=False, rope_theta=0.0,
                       embed_scale=width ** 0.5, final_softcap=30.0, layer_specs=specs, block_layout="parallel",
                       scalar_norm=True, layer_scale=True)


def lonulix_sized(width: int, vocab: int = 32000) -> ModelConfig:
    """six post-norm layers: HGRN2 (128-wide heads) + gated feed-forward, latent attention (window 1024) + routed experts,
    HGRN2 + gated feed-forward, latent attention over all keys + routed experts, HGRN2, latent attention (window 1024).
    Latent attention: width / 128 heads of 64 plain + 32 rotated query/key channels and 128 value channels over a cached
    latent of 96 channels (cache row: 128 channels per token for all heads together), query latent width / 2.  Experts:
    8 of width / 2 hidden channels in 2 groups (1 kept) beside 2 identity experts, 2 per token.  The layer matrices hold
    about 52 width^2 parameters, as ``repudra_sized(width)`` and ``kepovik_sized(width)`` do."""
    H = width // 128
    ff = max(128, (3 * width // 2) // 128 * 128)

    def latt(window):
        return LayerSpec(mixer="latent_attention", heads=H, kv_heads=1, dim=64, vdim=128, scale=96 ** -0.5, window=window,
                         rot=RotarySpec(dims=32, base=10000.0), q_rank=width // 2, kv_rank=96, rot_dim=32)

    def hgrn():
        return LayerSpec(mixer="hgrn2", heads=H, kv_heads=H, dim=128, vdim=128)

    def dense(sp):
        sp.ff = ff
        return sp

    def routed(sp):
        sp.ff_kind, sp.experts, sp.expert_ff, sp.top, sp.identity = "moe", 8, width // 2, 2, 2
        sp.route_groups, sp.route_keep, sp.route_scale, sp.ff = 2, 1, 2.0, 8 * (width // 2)
        return sp

    specs = (dense(hgrn()), routed(latt(1024)), dense(hgrn()), routed(latt(0)), hgrn(), latt(1024))
    return ModelConfig(name=f"mini-lonulix-{width}", family="lonulix", vocab_size=vocab, hidden_size=width,
                       n_layers=len(specs), n_heads=H, n_kv_heads=1, head_dim=128, ffn_size=max(sp.ff for sp in specs),
                       max_position=1 << 30, norm="rms", norm_eps=1e-6, act="silu", glu=True, rope_theta=0.0,
                       embed_scale=2.0, layer_specs=specs, block_layout="post_norm", norm_groups=4, skip_scale=2.0,
                       gated_residual=True)


def fisopel_sized(width: int, vocab: int = 32000) -> ModelConfig:
    """four parallel-block layers, the middle two run twice (six layer runs, as many as the six-layer models above):
    attention (width / 128 heads of 128 channels, grouped 4:1, per-head q / k norm, scores capped at 30, window 1024 with 64
    kept first keys, sink), gated latent attention (width / 128 heads of 64 plain + 32 rotated query/key channels and 128
    value channels over a cached latent of 96 channels, YaRN x 4), attention, latent attention; every layer has 8 gated
    experts of 3 width / 8 hidden channels (2 per token) beside a shared one of the same size.  The layer matrices hold
    about 53 width^2 parameters, as ``lonulix_sized(width)`` does."""
    H = width // 128
    eff = max(128, (3 * width // 8) // 128 * 128)

    def routed(sp):
        sp.ff_kind, sp.experts, sp.expert_ff, sp.top, sp.shared_ff = "moe", 8, eff, 2, eff
        sp.route_kind, sp.expert_gated, sp.ff = "logit_topk", True, 9 * eff
        return sp

    def att():
        return routed(LayerSpec(mixer="softmax_attention", heads=H, kv_heads=max(1, H // 4), dim=128, vdim=128,
                                scale=128 ** -0.5, window=1024, keep_first=64, softcap=30.0, qk_norm="head", v_norm=False,
                                sink=True))

    def latt():
        rot = RotarySpec(dims=32, base=10000.0, factor=4.0, original=2048, half=True)
        return routed(LayerSpec(mixer="latent_attention", heads=H, kv_heads=1, dim=64, vdim=128, scale=96 ** -0.5, rot=rot,
                                q_rank=0, kv_rank=96, rot_dim=32, out_gate=True))

    specs = (att(), latt(), att(), latt())
    return ModelConfig(name=f"mini-fisopel-{width}", family="fisopel", vocab_size=vocab, hidden_size=width,
                       n_layers=len(specs), n_heads=H, n_kv_heads=max(1, H // 4), head_dim=128,
                       ffn_size=max(sp.ff for sp in specs), max_position=1 << 30, norm="rms", norm_eps=1e-5, act="silu",
                       glu=True, rope_theta=0.0, tie_embeddings=True, embed_scale=2.0, layer_specs=specs,
                       block_layout="parallel", ff_norm=True, loop_start=1, loop_stop=3, loop_times=2, loop_in=True)


def llama_sized(width: int, layer_params: int, n_layers: int = 4, vocab: int = 32000) -> ModelConfig:
    """Llama layers (GQA 4:1, SwiGLU) whose matrices hold about ``layer_params`` parameters in ``n_layers`` layers"""
    H = width // 128
    kv = max(1, H // 4)
    attn = width * (H + 2 * kv) * 128 + H * 128 * width
    ffn = max(128, int(round((layer_params / n_layers - attn) / (3 * width) / 128)) * 128)
    return ModelConfig(name=f"mini-llama-{width}", family="llama", vocab_size=vocab, hidden_size=width,
                       n_layers=n_layers, n_heads=H, n_kv_heads=kv, head_dim=128, ffn_size=ffn, rope_theta=500000.0,
                       eos_token_id=1, bos_token_id=0)


def layer_params(cfg: ModelConfig) -> int:
    if not cfg.hybrid:
        h, f = cfg.hidden_size, cfg.ffn_size
        return cfg.n_layers * (h * (cfg.q_dim + 2 * cfg.kv_dim) + cfg.q_dim * h + 3 * h * f)
    if cfg.family != "kepovik":          # every matrix of the layers (embedding and head excluded)
        from ..models.weights import hybrid_tensor_specs
        return sum(shape[0] * shape[1] for name, shape, kind in hybrid_tensor_specs(cfg, range(cfg.n_layers), False, False)
                   if kind == "w" and len(shape) == 2)
    W, n = cfg.hidden_size, 0
    for sp in cfg.layer_specs:
        if sp.mixer == "attention":
            n += W * (sp.heads * sp.dim + sp.kv_heads * (sp.dim + sp.vdim) + sp.heads * sp.vdim) + sp.heads * sp.vdim * W
        else:
            n += 6 * W * sp.heads * sp.dim + 2 * max(8, sp.dim // 4) * W
        n += 2 * W * sp.ff
    return n


# ------------------------------------------------------------------------------------------------ kernel timing
class KernelTimer:
    """Wraps the kernel entry points of the extension: every call is bracketed by CUDA events after an L2 flush."""

    def __init__(self, device, hint: Dict):
        from .. import ops

        self.C = ops.native()
        self.names = [n for n in ops._KERNEL_ENTRY_POINTS if hasattr(self.C, n)]
        self.saved = {n: getattr(self.C, n) for n in self.names}
        self.rows: List[dict] = []
        self.hint = hint
        self.flush = torch.empty(192 << 20, dtype=torch.uint8, device=device)

    def __enter__(self):
        for n in self.names:
            setattr(self.C, n, self._wrap(n, self.saved[n]))
        return self

    def __exit__(self, *exc):
        for n in self.names:
            setattr(self.C, n, self.saved[n])

    def _wrap(self, name, fn):
        def call(*a, **kw):
            self.flush.fill_(1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record(torch.cuda.current_stream())
            r = fn(*a, **kw)
            e1.record(torch.cuda.current_stream())
            torch.cuda.synchronize()
            flops, nbytes, tc = cost(name, a, self.hint)
            self.rows.append({"kernel": name, "ms": e0.elapsed_time(e1), "flops": flops, "bytes": nbytes, "tensor_core": tc})
            return r
        return call


def _nb(t) -> int:
    return t.numel() * t.element_size()


def cost(name: str, a, hint: Dict):
    """(algorithmic FLOPs, bytes, runs on tensor cores) of one kernel call; ``hint``: tokens T, sequences S, span q,
    context ctx (keys before the span), and for attention the visible keys per query."""
    T, S, q, ctx = hint["T"], hint["S"], hint["q"], hint["ctx"]
    if name == "gemm":
        w, x = a[0], a[1]
        n, k = w.shape
        out_b = 4 if a[14] else 2
        return 2.0 * x.shape[0] * n * k, _nb(w) + _nb(x) + x.shape[0] * n * out_b + (x.shape[0] * n * 2 if a[7] else 0), True
    if name == "attention":
        n_q, n_kv, hd = a[10], a[11], a[12]
        keys = S * (q * ctx + q * (q + 1) / 2)                       # causal
        kv_bytes = S * (ctx + q) * n_kv * hd * 2 * 2
        return 4.0 * n_q * hd * keys, kv_bytes + 2 * T * n_q * hd * 2, True
    if name == "sig_attention":
        H, G, D, V, chunk = a[13], a[14], a[15], a[16], a[17]
        if chunk:
            per_q = [((ctx + i) % chunk) + 1 for i in range(q)]
        else:
            per_q = [ctx + i + 1 for i in range(q)]
        keys = S * float(sum(per_q))
        elt = a[1].element_size()
        kv_bytes = S * min(ctx + q, (max(per_q) + q)) * G * (D + V) * elt
        return 2.0 * H * (D + V) * keys, kv_bytes + T * H * D * 4 + 2 * T * H * V * 4, False
    if name == "delta_scan":
        H, dk, dv = a[16], a[17], a[18]
        return 9.0 * T * H * dk * dv, 2 * S * H * dk * dv * 4 + T * H * (4 * dk + 2 * dv) * 4, False
    if name == "hc_step":
        st = a[0]
        ns, W = st.shape[1], st.shape[2]
        rows = a[4] if a[3] is not None else T
        rw = (2 if (a[7] is not None and a[3] is None) else 1) * rows * ns * W * 4
        return 0.0, rw + (rows * W * 4 if a[7] is not None else 0) + (rows * W * 2 if a[14] is not None else 0), False
    if name == "hyb_embed":
        st = a[12]
        return 0.0, T * st.shape[1] * st.shape[2] * 4 + 2 * T * st.shape[2] * 2, False
    if name == "attn_prep":
        H, G, D, V = a[8], a[9], a[10], a[11]
        return 0.0, T * ((H + G) * D + G * V) * 4 + T * H * D * 4 + T * G * (D + V) * 2, False
    if name == "delta_post":
        H, dv = a[6], a[7]
        return 0.0, T * H * dv * (4 + 4 + 2), False
    if name == "act_cols":
        return 0.0, T * a[3] * 6, False
    if name == "ls_join":
        W = a[0].shape[-1]
        rows = a[4] if a[3] is not None else T
        n_terms = sum(1 for i in (7, 10, 13) if a[i] is not None)
        return 0.0, rows * W * 4 * ((1 if a[3] is not None else 2) + n_terms) + (rows * W * a[19].element_size()
                                                                                   if a[19] is not None else 0), False
    if name == "rot_attn_prep":
        H, G, D, V = a[15], a[16], a[17], a[18]
        return 0.0, T * ((H + G) * D + G * V) * 4 + T * H * D * 4 + T * G * (D + V) * a[12].element_size(), False
    if name == "softmax_attention":
        H, G, D, V = a[10], a[11], a[12], a[13]
        keys = S * (q * ctx + q * (q + 1) / 2)                       # causal
        kv_bytes = S * (ctx + q) * G * (D + V) * a[1].element_size()
        return 2.0 * H * (D + V) * keys, kv_bytes + T * H * D * 4 + T * H * V * a[3].element_size(), q >= 16
    if name == "short_conv":
        return 0.0, 2 * T * a[2].shape[0] * 4, False
    if name == "mlstm_gates":
        H, dk = a[17], a[18]
        return 4.0 * T * H * dk, T * H * (2 * dk + 6) * 4 + 2 * S * H * dk * 4, False
    if name == "lin_scan":
        H, dk, dv = a[23], a[25], a[26]
        return (8.0 if a[0] == 1 else 6.0) * T * H * dk * dv, 2 * S * H * dk * dv * 4 + T * H * (3 * dk + 2 * dv) * 4, False
    if name == "scan_post":
        H, dv = a[8], a[9]
        return 0.0, T * H * dv * (4 + 4 + 2), False
    if name == "post_norm_join":
        W = a[0].shape[-1]
        rows = a[2]
        gathered = a[1] is not None
        terms = (1 if a[3] is not None else 0) + (1 if a[4] is not None else 0)
        return 0.0, rows * W * 4 * ((1 if gathered else 2) + terms) + rows * W * a[12].element_size(), False
    if name == "latent_prep":
        return 0.0, T * (a[2] + a[4] + a[5]) * 4 + T * a[2] * a[12].element_size() + T * (a[4] + a[5]) * a[13].element_size(), False
    if name == "rot_heads":
        return 0.0, 2 * T * a[3] * a[4] * 4, False
    if name == "moe_route":
        return 0.0, T * (a[3] + a[4] + 1) * 4, False
    if name == "gated_cols":
        n = a[6]
        return 0.0, T * n * ((4 if (a[3] is not None and not a[9]) else 8) + a[5].element_size()), False
    if name == "head_up_gate":
        Tn, H, V, C = a[5], a[6], a[7], a[8]
        elt = a[0].element_size()
        return 2.0 * Tn * H * V * C, Tn * H * C * elt + H * V * C * elt + Tn * H * V * ((4 if a[2] is not None else 0) + elt), False
    if name in ("rmsnorm", "layernorm", "add"):
        return 0.0, 3 * _nb(a[0]), False
    if name == "embed":
        return 0.0, 2 * _nb(a[4]), False
    if name == "sample":
        return 0.0, _nb(a[0]), False
    return 0.0, 0, False


def summarize(rows: List[dict], peaks: Dict) -> List[dict]:
    bw = (peaks.get("hbm_gbs") or 6650.0) * 1e9
    fl = (peaks.get("bf16_tflops") or 1590.0) * 1e12
    agg: Dict[str, dict] = {}
    for r in rows:
        g = agg.setdefault(r["kernel"], {"kernel": r["kernel"], "calls": 0, "ms": 0.0, "flops": 0.0, "bytes": 0.0})
        g["calls"] += 1
        g["ms"] += r["ms"]
        g["flops"] += r["flops"]
        g["bytes"] += r["bytes"]
    out = []
    for g in agg.values():
        floor_ms = max(g["flops"] / fl, g["bytes"] / bw) * 1e3
        g["roofline_ms"] = floor_ms
        g["bound"] = "compute" if g["flops"] / fl > g["bytes"] / bw else "memory"
        g["frac_of_measured_roofline"] = floor_ms / g["ms"] if g["ms"] > 0 else None
        g["tflops"] = g["flops"] / g["ms"] / 1e9 if g["ms"] > 0 else 0.0
        g["gbps"] = g["bytes"] / g["ms"] / 1e6 if g["ms"] > 0 else 0.0
        out.append(g)
    return sorted(out, key=lambda g: -g["ms"])


# ------------------------------------------------------------------------------------------------------ driver
def bench_family(cfg: ModelConfig, device, prompt_len: int, batch: int, steps: int, warmup: int, ctx: int, peaks: Dict) -> dict:
    from ..engine.runner import GpuRunner, SeqInit

    torch.cuda.set_device(device)
    n_pf = 4
    max_seq = ((max(prompt_len, ctx) + steps + warmup + 80) // 64 + 1) * 64
    ppseq = max_seq // 64
    res = {"model": cfg.name, "family": cfg.family, "layer_params": layer_params(cfg)}
    gen = torch.Generator().manual_seed(1)

    def prompt(n):
        return torch.randint(2, cfg.vocab_size, (n,), generator=gen).tolist()

    def seqs(n, length, first_slot=0):
        return [SeqInit(slot=first_slot + i, prompt=prompt(length),
                        pages=list(range(1 + (first_slot + i) * ppseq, 1 + (first_slot + i + 1) * ppseq)),
                        temperature=0.0, top_p=1.0, repetition_penalty=1.0, seed=i) for i in range(n)]

    flush = torch.empty(192 << 20, dtype=torch.uint8, device=device)
    for mode in ("graphs", "eager"):
        r = GpuRunner(cfg, "", 0, 1, device, max_batch=batch, groups=1, max_seq_len=max_seq,
                      max_prefill_tokens=min(2048, prompt_len), num_pages=1 + batch * ppseq, use_graphs=mode == "graphs")
        if mode == "graphs":
            # ---- prefill: n_pf prompts of prompt_len tokens, chunked by the runner
            pf = seqs(n_pf, prompt_len)
            times = []
            for it in range(warmup + 3):
                flush.fill_(1)
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(r.stream)
                r.prefill(pf)
                e1.record(r.stream)
                r.sync()
                torch.cuda.synchronize()
                if it >= warmup:
                    times.append(e0.elapsed_time(e1))
                r.release([s.slot for s in pf])
            ms = sorted(times)[len(times) // 2]
            res["prefill"] = {"tokens": n_pf * prompt_len, "ms": ms, "tokens_per_s": n_pf * prompt_len / ms * 1e3,
                              "timing": "CUDA events, median of 3 after warm-up, L2 flushed between runs"}
            # ---- decode: `batch` sequences with `ctx` tokens of context, graph replays
            r.prefill(seqs(batch, ctx))
            r.decode(warmup)
            r.sync()
            flush.fill_(1)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(r.stream)
            r.decode(steps)
            e1.record(r.stream)
            r.sync()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            res["decode"] = {"batch": batch, "context": ctx, "steps": steps, "ms_per_step": ms / steps,
                             "tokens_per_s": batch * steps / ms * 1e3, "launches_per_step": r.launches_per_decode_step(),
                             "streamed_weight_bytes": r.piece.streamed_weight_bytes(),
                             "hbm_frac_of_measured": (r.piece.streamed_weight_bytes() / (ms / steps / 1e3) / 1e9 /
                                                      peaks["hbm_gbs"]) if peaks.get("hbm_gbs") else None}
        else:
            # ---- per-kernel: one eager prefill chunk of one prompt, one eager decode step
            one = seqs(1, min(2048, prompt_len))
            r.prefill(one)                                   # warm (descriptor caches, buffers)
            r.sync()
            r.release([0])
            hint = {"T": len(one[0].prompt), "S": 1, "q": len(one[0].prompt), "ctx": 0}
            with KernelTimer(device, hint) as kt:
                with torch.cuda.stream(r.stream):
                    r.prefill(one)
                r.sync()
            res["prefill_kernels"] = summarize(kt.rows, peaks)
            r.release([0])
            r.prefill(seqs(batch, ctx))
            r.decode(2)
            r.sync()
            hint = {"T": batch, "S": batch, "q": 1, "ctx": ctx + 3}
            with KernelTimer(device, hint) as kt:
                with torch.cuda.stream(r.stream):
                    r._decode_group(0)
                r.sync()
            res["decode_kernels"] = summarize(kt.rows, peaks)
        r.close()
        del r
        torch.cuda.empty_cache()
    return res


def run(widths, prompt_len=2048, batch=32, steps=32, warmup=3, ctx=512, device="cuda:0", family="kepovik") -> List[dict]:
    peaks = {}
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            peaks = json.load(f)
    except Exception:
        pass
    out = []
    for w in widths:
        kep = kepovik_sized(w)
        if family == "fisopel":
            pair = (fisopel_sized(w), lonulix_sized(w))
        elif family == "lonulix":
            pair = (lonulix_sized(w), repudra_sized(w))
        else:
            pair = (repudra_sized(w), kep) if family == "repudra" else (kep, llama_sized(w, layer_params(kep)))
        for cfg in pair:
            out.append(bench_family(cfg, torch.device(device), prompt_len, batch, steps, warmup, ctx, peaks))
    return out
