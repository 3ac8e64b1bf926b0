"""Plain, slow restatement of the Gigezen design in float64 torch on the CPU: one function per mechanism.

It reads the configuration as the ``config.json`` dictionary and the weights as a ``name -> tensor`` dictionary, and
shares no code with the framework's execution path.  Sequences are always recomputed from their first token, so the
oracle has no cache whose faults it could share with the product.

Notation: x residual stream [T, W]; h normed input of a layer; p positions; c latent [T, R]; kr rotated shared key
part [T, rot]; per head: qn / qr unrotated / rotated query parts.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F = torch.float64


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def zero_centred_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """Gains stored around zero."""
    return unit_rms(x, eps) * (1.0 + w)


def rotate_half(x: torch.Tensor, p: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [T, ..., n >= dims]: the first ``dims`` entries are rotated in pairs (i, i + dims/2), the rest pass."""
    out = x.clone()
    half = dims // 2
    for t in range(x.shape[0]):
        for i in range(half):
            ang = float(p[t]) * base ** (-2.0 * i / dims)
            cs, sn = math.cos(ang), math.sin(ang)
            u, v = x[t, ..., i], x[t, ..., i + half]
            out[t, ..., i] = u * cs - v * sn
            out[t, ..., i + half] = v * cs + u * sn
    return out


def latent_rows(h: torch.Tensor, w_dkv: torch.Tensor, gain: torch.Tensor, p: torch.Tensor, m: dict, eps: float):
    """What a cache-owning layer stores per token: (c [T, R], kr [T, rot])."""
    R = m["kv_rank"]
    d = h @ w_dkv.T
    c = unit_rms(d[:, :R], eps) * gain
    kr = rotate_half(d[:, R:], p, m["rot"]["dims"], m["rot"]["base"])
    return c, kr


def window_visible(i: int, j: int, size: int) -> bool:
    return 0 <= i - j < size


def latent_attention(h: torch.Tensor, p: torch.Tensor, c: torch.Tensor, kr: torch.Tensor, w: Dict[str, torch.Tensor],
                     m: dict) -> torch.Tensor:
    """h [T, W] -> mixer output [T, W]; keys / values are expanded per head from the latent rows of the same T
    positions (explicit form: k = W_uk c, v = W_uv c)."""
    T = h.shape[0]
    H, dim, rot, vd = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    q = (h @ w["q"].T).view(T, H, dim + rot)
    qn, qr = q[..., :dim], rotate_half(q[..., dim:], p, m["rot"]["dims"], m["rot"]["base"])
    k = (c @ w["uk"].T).view(T, H, dim)
    v = (c @ w["uv"].T).view(T, H, vd)
    heads = torch.zeros(T, H, vd, dtype=F)
    for hd in range(H):
        for i in range(T):
            js = [j for j in range(T) if window_visible(int(p[i]), int(p[j]), m["mask"]["size"])]
            s = torch.stack([(qn[i, hd] @ k[j, hd] + qr[i, hd] @ kr[j]) * m["scale"] for j in js])
            a = torch.softmax(s, 0)
            heads[i, hd] = sum(a[n] * v[j, hd] for n, j in enumerate(js))
    return heads.reshape(T, H * vd) @ w["o"].T


def clamped_gated_unit(h: torch.Tensor, w: Dict[str, torch.Tensor], limit: float) -> torch.Tensor:
    g = torch.clamp(h @ w["gate"].T, max=limit)
    u = torch.clamp(h @ w["up"].T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w["down"].T


def route(h: torch.Tensor, w_router: torch.Tensor, r: dict):
    """-> (chosen expert ids [T, top] (descending score), their scores [T, top], all scores [T, E])."""
    E, top = r["experts"], r["top"]
    G, keep = r.get("groups", {}).get("count", 1), r.get("groups", {}).get("keep", 1)
    s = torch.softmax(h @ w_router.T, -1)
    ids, wts = [], []
    for t in range(s.shape[0]):
        per = E // G
        gscore = [max(float(s[t, g * per + e]) for e in range(per)) for g in range(G)]
        kept = sorted(range(G), key=lambda g: (-gscore[g], g))[:keep]
        allowed = [e for e in range(E) if e // per in kept]
        best = sorted(allowed, key=lambda e: (-float(s[t, e]), e))[:top]
        ids.append(best)
        wts.append([float(s[t, e]) for e in best])
    return torch.tensor(ids), torch.tensor(wts, dtype=F), s


def expert(h: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    a = h @ gate.T
    return ((a * torch.sigmoid(a)) * (h @ up.T)) @ down.T


def mixture(h: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str, ml: dict) -> torch.Tensor:
    ids, wts, _ = route(h, w[prefix + "router"], ml["router"])
    out = torch.zeros(h.shape[0], w[prefix + "e0.down"].shape[0], dtype=F)
    for t in range(h.shape[0]):
        for k, e in enumerate(ids[t].tolist()):
            q = f"{prefix}e{e}."
            out[t] += wts[t, k] * expert(h[t:t + 1], w[q + "gate"], w[q + "up"], w[q + "down"])[0]
    return out


def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens: List[int], layers_out: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence from its first token."""
    w = {k: v.to(F) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    T = len(tokens)
    p = torch.arange(T)
    x = w["embed"][torch.tensor(tokens)]
    rows = {}
    for i, L in enumerate(cfg["layers"]):
        pre, m = f"l{i}.", L["mixer"]
        h = zero_centred_norm(x, w[pre + "norm1"], eps)
        if m.get("kv_from") is None:
            rows[i] = latent_rows(h, w[pre + "mix.dkv"], w[pre + "mix.dkv.norm"], p, m, eps)
        c, kr = rows[i if m.get("kv_from") is None else m["kv_from"]]
        mix = latent_attention(h, p, c, kr, {k: w[pre + "mix." + k] for k in ("q", "uk", "uv", "o")}, m)
        ml = L.get("mlp")
        if ml is None:
            ff = 0.0
        elif ml["kind"] == "dense":
            ff = clamped_gated_unit(h, {k: w[pre + "mlp." + k] for k in ("gate", "up", "down")}, ml["limit"])
        else:
            ff = mixture(h, w, pre + "mlp.", ml)
        x = x + (mix + ff)
        if layers_out is not None:
            layers_out.append(x.clone())
    return zero_centred_norm(x, w["final.norm"], eps) @ w["head"].T


def greedy(cfg: dict, weights: Dict[str, torch.Tensor], prompt: List[int], n_new: int) -> List[int]:
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(forward(cfg, weights, toks)[-1].argmax()))
    return toks[len(prompt):]
