"""A plain, slow restatement of the Seledra design in float64: one function per mechanism, working on whole sequences
with explicit loops, from the ``config.json`` dictionary and a ``name -> tensor`` dictionary.  Shares no code with the
product path (no cache, no state object: decoding is checked against the full-sequence pass)."""
import math

import torch

F = torch.float64


def rms_normalise(x, eps):
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def soft_plus(x):
    return torch.where(x > 30, x, torch.log1p(torch.exp(torch.clamp(x, max=30))))


def swish(x):
    return x / (1 + torch.exp(-x))


def sink_softmax(scores, sink=1.0):
    """Rows of scores (masked entries = -inf) -> weights exp(s) / (sink + sum exp(s))."""
    top = torch.clamp(scores.max(-1, keepdim=True).values, min=0.0)
    e = torch.exp(scores - top)
    return e / (sink * torch.exp(-top) + e.sum(-1, keepdim=True))


def attention_mixer(spec, w, pre, h, eps, shared):
    """h [T, W] -> [T, W].  ``shared`` carries the first value-mixing layer's values from layer to layer."""
    H, G, dk, dv = spec["heads"], spec["kv_heads"], spec["dim"], spec["vdim"]
    T = h.shape[0]
    q = h @ w[pre + "q"].T + w[pre + "q.b"]
    k = h @ w[pre + "k"].T + w[pre + "k.b"]
    v = h @ w[pre + "v"].T + w[pre + "v.b"]
    q = rms_normalise(q, eps) * w[pre + "q.norm"]           # over all heads at once
    k = rms_normalise(k, eps) * w[pre + "k.norm"]
    v = rms_normalise(v.reshape(T, G, dv), eps)             # per head, no gain
    if spec.get("v_mix"):
        if "values" not in shared:
            shared["values"] = v
        else:
            lam = w[pre + "vmix"]
            v = (1 - lam) * v + lam * shared["values"]
    q, k = q.reshape(T, H, dk), k.reshape(T, G, dk)
    gate = torch.sigmoid(h @ w[pre + "g"].T)                # [T, H]
    out = torch.zeros(T, H, dv, dtype=F)
    for head in range(H):
        g = head // (H // G)
        for i in range(T):
            s = (k[: i + 1, g] @ q[i, head]) * spec["scale"] * w[pre + "temp"][head]
            p = sink_softmax(s[None, :])[0]
            out[i, head] = (p[:, None] * v[: i + 1, g]).sum(0) * gate[i, head]
    return out.reshape(T, H * dv) @ w[pre + "o"].T


def causal_conv(x, taps_w):
    """x [T, C], taps_w [C, taps] (last column = current token) -> silu of the causal convolution."""
    T, taps = x.shape[0], taps_w.shape[1]
    y = torch.zeros_like(x)
    for i in range(T):
        for b in range(taps):
            if i - b >= 0:
                y[i] += taps_w[:, taps - 1 - b] * x[i - b]
    return swish(y)


def delta_mixer(spec, w, pre, h, eps, unit_eps=1e-6):
    H, G, dk, dv = spec["heads"], spec["kv_heads"], spec["dim"], spec["vdim"]
    T = h.shape[0]
    q = causal_conv(h @ w[pre + "q"].T, w[pre + "q.conv"]).reshape(T, G, dk)
    k = causal_conv(h @ w[pre + "k"].T, w[pre + "k.conv"]).reshape(T, G, dk)
    v = causal_conv(h @ w[pre + "v"].T, w[pre + "v.conv"]).reshape(T, H, dv)
    q = q / torch.sqrt(q.pow(2).sum(-1, keepdim=True) + unit_eps) / math.sqrt(dk)
    k = k / torch.sqrt(k.pow(2).sum(-1, keepdim=True) + unit_eps)
    beta = torch.sigmoid(h @ w[pre + "b"].T)
    decay = torch.exp(-torch.exp(w[pre + "A_log"]) * soft_plus(h @ w[pre + "a"].T + w[pre + "dt_bias"]))
    read = torch.zeros(T, H, dv, dtype=F)
    for head in range(H):
        g = head // (H // G)
        S = torch.zeros(dk, dv, dtype=F)
        for i in range(T):
            S = decay[i, head] * S
            u = beta[i, head] * (v[i, head] - S.T @ k[i, g])
            S = S + k[i, g][:, None] * u[None, :]
            read[i, head] = S.T @ q[i, g]
    read = rms_normalise(read, eps) * w[pre + "norm"] * swish(h @ w[pre + "g"].T).reshape(T, H, dv)
    return read.reshape(T, H * dv) @ w[pre + "o"].T


def xielu(z, params):
    a_pos, a_neg = soft_plus(params[0]), 0.5 + soft_plus(params[1])
    neg = torch.clamp(z, max=0.0)
    return torch.where(z > 0, a_pos * z * z + 0.5 * z, a_neg * (torch.expm1(neg) - neg) + 0.5 * z)


def feed_forward(w, pre, h):
    return xielu(h @ w[pre + "up"].T, w[pre + "act"]) @ w[pre + "down"].T


def forward(cfg, weights, tokens, layers_out=None):
    """Logits [T, vocab] (float64) of a whole sequence; ``layers_out`` collects the stream after every layer."""
    w = {k: v.to(F) for k, v in weights.items()}
    eps, m = cfg["norm"]["eps"], cfg.get("residual_mult", 1.0)
    T = len(tokens)
    x = w["embed"][torch.tensor(tokens)] + w["pos"][:T]
    shared = {}
    for i, L in enumerate(cfg["layers"]):
        pre = f"l{i}."
        h = rms_normalise(x, eps) * w[pre + "norm1"]
        if L["type"] == "attention":
            x = x + m * attention_mixer(L["mixer"], w, pre + "mix.", h, eps, shared)
        elif L["type"] == "delta":
            x = x + m * delta_mixer(L["mixer"], w, pre + "mix.", h, eps)
        else:
            raise ValueError(L["type"])
        if L.get("mlp") is not None:
            x = x + m * feed_forward(w, pre + "mlp.", rms_normalise(x, eps) * w[pre + "norm2"])
        if layers_out is not None:
            layers_out.append(x.clone())
    return (rms_normalise(x, eps) * w["final.norm"]) @ w["head"].T


def greedy(cfg, weights, prompt, n):
    toks = list(prompt)
    out = []
    for _ in range(n):
        nxt = int(forward(cfg, weights, toks)[-1].argmax())
        out.append(nxt)
        toks.append(nxt)
    return out
