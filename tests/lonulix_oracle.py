"""Plain float64 restatement of the Lonulix design, one function per mechanism, token by token where the design is a
recurrence.  It reads the checkpoint's own ``config.json`` dictionary and tensor names and shares no code with the served
model (``bee2bee_b200/models/hybrid.py`` and the kernels under ``csrc/``); slow on purpose.

Notation: ``x`` [T, W] is one sequence, ``P`` maps tensor names to float64 tensors, ``m`` is a layer's ``mixer``
dictionary.  Linear weights are [out, in].
"""
from __future__ import annotations

import math
from typing import Dict, List, Tuple

import torch

F64 = torch.float64


def rms(v: torch.Tensor, eps: float) -> torch.Tensor:
    return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps)


def group_norm(x: torch.Tensor, w: torch.Tensor, groups: int, eps: float) -> torch.Tensor:
    """RMS norm taken separately over ``groups`` consecutive equal slices of the width, then the weight"""
    T, W = x.shape
    return (rms(x.reshape(T, groups, W // groups), eps).reshape(T, W)) * w


def rotate_pairs(v: torch.Tensor, pos: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """v [T, ..., D]: channels (2i, 2i+1) for 2i < dims turn by pos * base^(-2i/dims); the rest pass"""
    out = v.clone()
    shape = [v.shape[0]] + [1] * (v.dim() - 2)
    for i in range(dims // 2):
        a = pos.to(F64) * (base ** (-2.0 * i / dims))
        c, s = torch.cos(a).reshape(shape), torch.sin(a).reshape(shape)
        u, w = v[..., 2 * i], v[..., 2 * i + 1]
        out[..., 2 * i] = u * c - w * s
        out[..., 2 * i + 1] = w * c + u * s
    return out


def latent_attention(h: torch.Tensor, P: Dict[str, torch.Tensor], p: str, m: Dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, D, R, V, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    rot = m.get("rot") or {"dims": 0, "base": 10000.0}
    window = int((m.get("mask") or {}).get("size", 0))
    pos = torch.arange(T)
    cq = rms(h @ P[p + "dq"].T, eps) * P[p + "dq.norm"]
    q = (cq @ P[p + "uq"].T).reshape(T, H, D + R)
    q_n, q_r = q[..., :D], rotate_pairs(q[..., D:], pos, rot["dims"], rot["base"])
    dkv = h @ P[p + "dkv"].T
    c = rms(dkv[:, :C], eps) * P[p + "dkv.norm"]
    k_r = rotate_pairs(dkv[:, C:], pos, rot["dims"], rot["base"])          # one rotated key part for all heads
    k_n = (c @ P[p + "uk"].T).reshape(T, H, D)
    v = (c @ P[p + "uv"].T).reshape(T, H, V)
    out = torch.zeros(T, H, V, dtype=F64)
    for i in range(T):
        lo = max(0, i - window + 1) if window > 0 else 0
        for hd in range(H):
            s = (k_n[lo:i + 1, hd] @ q_n[i, hd] + k_r[lo:i + 1] @ q_r[i, hd]) * m["scale"]
            out[i, hd] = torch.softmax(s, 0) @ v[lo:i + 1, hd]
    return out.reshape(T, H * V) @ P[p + "o"].T


def hgrn2(h: torch.Tensor, P: Dict[str, torch.Tensor], p: str, m: Dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = torch.nn.functional.silu(h @ P[p + "q"].T).reshape(T, H, D)
    v = (h @ P[p + "v"].T).reshape(T, H, V)
    low = P[p + "lower"]
    f = (low + (1.0 - low) * torch.sigmoid(h @ P[p + "f"].T + P[p + "f.b"])).reshape(T, H, D)
    S = torch.zeros(H, D, V, dtype=F64)
    o = torch.zeros(T, H, V, dtype=F64)
    for t in range(T):
        S = f[t][:, :, None] * S + (1.0 - f[t])[:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = rms(o, eps) * P[p + "norm"]
    return o.reshape(T, H * V) @ P[p + "o"].T


def dense_ff(h: torch.Tensor, P: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return (torch.nn.functional.silu(h @ P[p + "gate"].T) * (h @ P[p + "up"].T)) @ P[p + "down"].T


def route(h: torch.Tensor, P: Dict[str, torch.Tensor], p: str, r: Dict) -> Tuple[List[List[int]], List[List[float]]]:
    """per token: the chosen expert indices (identity experts count from r['experts'] on) and their weights"""
    E = r["experts"] + int(r.get("identity", 0))
    g = r.get("groups") or {"count": 1, "keep": 1}
    s = torch.softmax(h @ P[p + "router"].T, -1)
    choice = s + P[p + "correction"]
    per = E // g["count"]
    idx, wts = [], []
    for t in range(h.shape[0]):
        gs = [max(float(choice[t, j]) for j in range(k * per, (k + 1) * per)) for k in range(g["count"])]
        kept = sorted(range(g["count"]), key=lambda k: -gs[k])[:g["keep"]]
        cand = [j for j in range(E) if j // per in kept]
        cand.sort(key=lambda j: -float(choice[t, j]))
        ch = cand[:r["top"]]
        tot = sum(float(s[t, j]) for j in ch) + 1e-20
        idx.append(ch)
        wts.append([float(s[t, j]) / tot * r["scale"] for j in ch])
    return idx, wts


def moe_ff(h: torch.Tensor, P: Dict[str, torch.Tensor], p: str, mlp: Dict) -> torch.Tensor:
    r = mlp["router"]
    idx, wts = route(h, P, p, r)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j, w in zip(idx[t], wts[t]):
            if j >= r["experts"]:
                out[t] += w * h[t]
            else:
                z = P[f"{p}e{j}.up"] @ h[t]
                a = 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))
                out[t] += w * (P[f"{p}e{j}.down"] @ a)
    return out


def forward(cfg: Dict, P: Dict[str, torch.Tensor], tokens: List[int]):
    """-> (logits [T, vocab], residual after every layer [L, T, W])"""
    P = {k: v.to(F64) for k, v in P.items()}
    eps, groups = cfg["norm"]["eps"], int(cfg["norm"].get("groups", 1))
    alpha = float(cfg.get("postln_alpha", 1.0))
    x = P["embed"][torch.tensor(tokens)] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    after = []
    for l, lay in enumerate(cfg["layers"]):
        p = f"l{l}."
        mix = {"latent_attention": latent_attention, "hgrn2": hgrn2}[lay["type"]]
        y = mix(x, P, p + "mix.", lay["mixer"], eps) * torch.sigmoid(x @ P[p + "rg1"].T + P[p + "rg1.b"])
        x = group_norm(alpha * x + y, P[p + "norm1"], groups, eps)
        mlp = lay.get("mlp")
        if mlp:
            y = dense_ff(x, P, p + "mlp.") if mlp["kind"] == "dense" else moe_ff(x, P, p + "mlp.", mlp)
            y = y * torch.sigmoid(x @ P[p + "rg2"].T + P[p + "rg2.b"])
            x = group_norm(alpha * x + y, P[p + "norm2"], groups, eps)
        after.append(x.clone())
    logits = group_norm(x, P["final.norm"], groups, eps) @ P["head"].T
    return logits, torch.stack(after)
