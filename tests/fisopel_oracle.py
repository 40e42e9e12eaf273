"""Plain float64 restatement of the Fisopel design, one function per mechanism; shares no code with the served model.

Notation: ``P`` maps tensor names to float64 tensors, ``cfg`` is the checkpoint's ``config.json`` as a dict, token rows are
the leading dimension.  A layer is ``x <- x + mixer(n1(x)) + ff(n2(x))`` with two RMS norms of the same ``x``; layers
``loop.start .. loop.stop - 1`` run ``loop.times`` times, and the residual entering every pass is ``W_in [x ; e]`` with ``e``
the scaled embedding.  Logits are ``E n(x)`` with the embedding table ``E`` itself.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch

F64 = torch.float64


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


# ------------------------------------------------------------------------------------------------ rotary positions
def rotary_table(rot: Dict) -> Tuple[torch.Tensor, float]:
    """(angle per position of every pair, amplitude).  With ``scaling``: pairs whose wavelength exceeds ``original / slow``
    are slowed by ``factor``, those below ``original / fast`` are kept, linear blend between (on the pair index)."""
    n, base = rot["dims"], rot["base"]
    w = torch.tensor([base ** (-2.0 * i / n) for i in range(n // 2)], dtype=F64)
    sc = rot.get("scaling")
    if not sc:
        return w, 1.0

    def index_of(turns: float) -> float:
        return n * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo, hi = max(math.floor(index_of(sc["fast"])), 0), min(math.ceil(index_of(sc["slow"])), n - 1)
    ramp = ((torch.arange(n // 2, dtype=F64) - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return w / sc["factor"] * ramp + w * (1.0 - ramp), 0.1 * math.log(sc["factor"]) + 1.0


def rotate_split_halves(x: torch.Tensor, pos: torch.Tensor, rot: Optional[Dict]) -> torch.Tensor:
    """x [T, ..., d]: channel i < dims/2 is paired with channel i + dims/2; channels from ``dims`` on pass unchanged"""
    if not rot or not rot.get("dims"):
        return x
    n = rot["dims"]
    w, amp = rotary_table(rot)
    ang = pos.to(F64)[:, None] * w[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [n // 2]
    c, s = (torch.cos(ang) * amp).view(shape), (torch.sin(ang) * amp).view(shape)
    a, b = x[..., :n // 2], x[..., n // 2:n]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., n:]], -1)


# ------------------------------------------------------------------------------------------------ masks and softmax
def visible(T: int, window: int, keep_first: int) -> torch.Tensor:
    """[query, key] booleans: causal; with a window only the last ``window`` keys and the first ``keep_first`` ones"""
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    ok = j <= i
    if window > 0:
        ok = ok & ((i - j < window) | (j < keep_first))
    return ok


def softmax_with_sink(scores: torch.Tensor, ok: torch.Tensor, sink: Optional[torch.Tensor]) -> torch.Tensor:
    """rows of weights over the visible keys; ``sink`` (a number) adds exp(sink) to the denominator and nothing else"""
    s = scores.masked_fill(~ok, -float("inf"))
    top = s.max(-1, keepdim=True).values
    if sink is not None:
        top = torch.maximum(top, sink.reshape(1, 1))
    e = torch.exp(s - top)
    den = e.sum(-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(sink - top)
    return e / den


# ------------------------------------------------------------------------------------------------ mixers
def grouped_attention(h: torch.Tensor, P: Dict, p: str, m: Dict, eps: float) -> torch.Tensor:
    """grouped key/value heads, RMS norm per head on q and k (one weight vector each), no positions in the scores, capped
    scores, window with kept first keys, a sink per head"""
    T = h.shape[0]
    H, G, D, V = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m.get("vdim", m["dim"])
    q = rms((h @ P[p + "q"].T).view(T, H, D), eps) * P[p + "q.norm"]
    k = rms((h @ P[p + "k"].T).view(T, G, D), eps) * P[p + "k.norm"]
    v = (h @ P[p + "v"].T).view(T, G, V)
    mask = m.get("mask") or {}
    ok = visible(T, int(mask.get("size", 0) or 0), int(mask.get("keep_first", 0) or 0))
    cap = float(m.get("softcap", 0.0) or 0.0)
    out = []
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * m["scale"]
        if cap > 0:
            s = cap * torch.tanh(s / cap)
        out.append(softmax_with_sink(s, ok, P[p + "sink"][hd]) @ v[:, g])
    return torch.cat(out, -1) @ P[p + "o"].T


def latent_attention(h: torch.Tensor, P: Dict, p: str, m: Dict, eps: float) -> torch.Tensor:
    """keys and values are per-head up-projections of one normed latent per token; every head's key also carries one
    rotated part common to all heads; queries are [plain | rotated] per head; the concatenated heads pass a sigmoid gate"""
    T = h.shape[0]
    H, D, R, V, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    q = (h @ P[p + "q"].T).view(T, H, D + R)
    down = h @ P[p + "dkv"].T
    c = rms(down[:, :C], eps) * P[p + "dkv.norm"]
    k_rot = rotate_split_halves(down[:, C:], pos, m.get("rot"))                 # [T, R], one for all heads
    q_rot = rotate_split_halves(q[..., D:], pos, m.get("rot"))
    k = (c @ P[p + "uk"].T).view(T, H, D)
    v = (c @ P[p + "uv"].T).view(T, H, V)
    ok = visible(T, 0, 0)
    out = []
    for hd in range(H):
        s = (q[:, hd, :D] @ k[:, hd].T + q_rot[:, hd] @ k_rot.T) * m["scale"]
        out.append(softmax_with_sink(s, ok, None) @ v[:, hd])
    return (torch.cat(out, -1) * torch.sigmoid(h @ P[p + "g"].T)) @ P[p + "o"].T


# ------------------------------------------------------------------------------------------------ feed-forward
def gated_expert(h: torch.Tensor, P: Dict, p: str) -> torch.Tensor:
    return (silu(h @ P[p + "gate"].T) * (h @ P[p + "up"].T)) @ P[p + "down"].T


def route(z: torch.Tensor, top: int) -> Tuple[List[List[int]], List[List[float]]]:
    """per token: the ``top`` largest logits (lowest index among equals), weighted by the softmax over those alone"""
    idx, wts = [], []
    for row in z.tolist():
        order = sorted(range(len(row)), key=lambda j: (-row[j], j))[:top]
        big = max(row[j] for j in order)
        e = [math.exp(row[j] - big) for j in order]
        idx.append(order)
        wts.append([v / sum(e) for v in e])
    return idx, wts


def routed_ff(h: torch.Tensor, P: Dict, p: str, mlp: Dict) -> torch.Tensor:
    idx, wts = route(h @ P[p + "router"].T, mlp["router"]["top"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j, w in zip(idx[t], wts[t]):
            out[t] += w * gated_expert(h[t:t + 1], P, f"{p}e{j}.")[0]
    if mlp.get("shared"):
        out = out + gated_expert(h, P, p + "shared.")
    return out


# ------------------------------------------------------------------------------------------------ the model
def layer_order(cfg: Dict) -> List[Tuple[int, bool]]:
    """(layer, a pass of the loop begins here) in the order the layers run"""
    n, lp = len(cfg["layers"]), cfg.get("loop")
    if not lp:
        return [(i, False) for i in range(n)]
    a, b = lp["start"], lp["stop"]
    inside = [(i, i == a) for i in range(a, b)]
    return [(i, False) for i in range(a)] + inside * lp["times"] + [(i, False) for i in range(b, n)]


def forward(cfg: Dict, P: Dict, tokens: List[int]):
    """-> (logits [T, vocab], residual after every layer run)"""
    P = {k: v.to(F64) for k, v in P.items()}
    eps = cfg["norm"]["eps"]
    e = P["embed"][torch.tensor(tokens)] * (cfg.get("embedding") or {}).get("scale", 1.0)
    x, trail = e, []
    for i, begins in layer_order(cfg):
        lay, p = cfg["layers"][i], f"l{i}."
        if begins:
            x = torch.cat([x, e], -1) @ P["loop.in"].T
        h = rms(x, eps) * P[p + "norm1"]
        mix = grouped_attention if lay["type"] == "attention" else latent_attention
        y = mix(h, P, p + "mix.", lay["mixer"], eps)
        if lay.get("mlp"):
            y = y + routed_ff(rms(x, eps) * P[p + "norm2"], P, p + "mlp.", lay["mlp"])
        x = x + y
        trail.append(x)
    return (rms(x, eps) * P["final.norm"]) @ P["embed"].T, trail
