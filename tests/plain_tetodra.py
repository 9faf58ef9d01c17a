"""Tetodra, plainly: whole sequences, no cache, no batching, float64 unless told otherwise; one
function per mechanism.  It shares no code with the engine and is what the engine is compared with.

``weights`` maps tensor names to torch tensors (any float type), ``cfg`` is the dictionary of
config.json.  Notation: T tokens, D the model width, rows are tokens.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def layer_norm(x, w, eps):
    """Mean taken off, divided by the root of the mean squared deviation, times a gain; no bias."""
    d = x - x.mean(-1, keepdim=True)
    return d / torch.sqrt((d * d).mean(-1, keepdim=True) + eps) * w


def silu(z):
    return z * torch.sigmoid(z)


def log_sigmoid(z):
    return -torch.nn.functional.softplus(-z)


def causal_conv(x: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """x [T, C], taps [C, K]; y[t, c] = sum_j taps[c, K-1-j] x[t-j, c], zeros before the start."""
    T, C = x.shape
    K = taps.shape[1]
    y = torch.zeros_like(x)
    for j in range(K):
        if j < T:
            y[j:] += x[:T - j] * taps[:, K - 1 - j]
    return y


# ---------------------------------------------------------------- attention
def distance_bucket(n: int, rows: int, far: float) -> int:
    """Row of a table of ``rows`` learned biases for a key ``n`` tokens back: one row per distance in the
    first half, then rows that widen geometrically until ``far``, beyond which the last row serves."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def rotate_half(x: torch.Tensor, positions: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """x [T, heads, d]: elements i and i + dims/2 of the first ``dims`` turn by position * base^(-2i/dims)."""
    half = dims // 2
    freq = base ** (-2.0 * torch.arange(half, dtype=x.dtype) / dims)
    ang = positions.to(x.dtype).view(-1, 1, 1) * freq
    c, s = torch.cos(ang), torch.sin(ang)
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], dim=-1)


def softmax_attention(q, k, v, scale: float, bias: Optional[torch.Tensor] = None,
                      sink: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q [T, H, dk], k [T, G, dk], v [T, G, dv]; causal; ``bias`` [H, T, T] is added to the scaled score;
    ``sink`` [H]: exp(sink) joins the denominator and nothing else."""
    T, H, _ = q.shape
    G = k.shape[1]
    rep = H // G
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    mask = torch.tril(torch.ones(T, T, dtype=torch.bool))
    for h in range(H):
        s = (q[:, h] @ k[:, h // rep].T) * scale
        if bias is not None:
            s = s + bias[h]
        s = s.masked_fill(~mask, float("-inf"))
        top = s.max(-1, keepdim=True).values
        if sink is not None:
            top = torch.maximum(top, sink[h].expand_as(top))
        e = torch.exp(s - top)
        den = e.sum(-1, keepdim=True)
        if sink is not None:
            den = den + torch.exp(sink[h] - top)
        out[:, h] = (e / den) @ v[:, h // rep]
    return out


def attention_keys_as_values(h, w, p, m, eps):
    """Queries and keys normed per head with a gain, values are the keys as projected; a temperature on the
    queries that grows with the position; a learned bias by bucketed distance; a learned sink."""
    H, G, dk = m["heads"], m["kv_heads"], m["dim"]
    T = h.shape[0]
    q = (h @ w[p + "q"].T).view(T, H, dk)
    k = (h @ w[p + "k"].T).view(T, G, dk)
    v = k
    q = rms_unit(q, eps) * w[p + "q.norm"]
    k = rms_unit(k, eps) * w[p + "k.norm"]
    pos = torch.arange(T)
    temp = 1.0 + m["q_temp"]["coef"] * torch.log(torch.floor((pos + 1).to(h.dtype) / m["q_temp"]["every"]) + 1.0)
    q = q * temp.view(T, 1, 1)
    rel = w[p + "rel"]
    rows = rel.shape[0]
    idx = torch.tensor([[distance_bucket(i - j, rows, m["bias_max"]) if j <= i else 0 for j in range(T)]
                        for i in range(T)])
    bias = rel[idx].permute(2, 0, 1)                     # [H, T, T]
    o = softmax_attention(q, k, v, m["scale"], bias=bias, sink=w[p + "sink"])
    return o.reshape(T, -1) @ w[p + "o"].T


def attention_rotary(h, w, p, m):
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    pos = torch.arange(T)
    q = rotate_half((h @ w[p + "q"].T).view(T, H, dk), pos, m["rot"]["base"], m["rot"]["dims"])
    k = rotate_half((h @ w[p + "k"].T).view(T, G, dk), pos, m["rot"]["base"], m["rot"]["dims"])
    v = (h @ w[p + "v"].T).view(T, G, dv)
    return softmax_attention(q, k, v, m["scale"]).reshape(T, -1) @ w[p + "o"].T


# ---------------------------------------------------------------- recurrences
def matrix_memory(h, w, p, m, eps, trace: Optional[dict] = None):
    """A matrix S and a vector n per head, written with exp(input gate) and kept with exp(forget gate), both
    held under a running maximum of their logarithms that starts at zero."""
    H, dk, dv, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    T = h.shape[0]
    q = (h @ w[p + "q"].T).view(T, H, dk) * dk ** -0.5
    k = (h @ w[p + "k"].T).view(T, H, dk)
    v = (h @ w[p + "v"].T).view(T, H, dv)
    gi = cap * torch.tanh((h @ w[p + "i"].T + w[p + "i.b"]) / cap)                      # [T, H], logarithms
    gf = log_sigmoid(cap * torch.tanh((h @ w[p + "f"].T + w[p + "f.b"]) / cap))
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for hd in range(H):
        S = torch.zeros(dk, dv, dtype=h.dtype)
        n = torch.zeros(dk, dtype=h.dtype)
        top = torch.zeros((), dtype=h.dtype)
        for t in range(T):
            new_top = torch.maximum(gf[t, hd] + top, gi[t, hd])
            keep, write = torch.exp(gf[t, hd] + top - new_top), torch.exp(gi[t, hd] - new_top)
            S = keep * S + write * torch.outer(k[t, hd], v[t, hd])
            n = keep * n + write * k[t, hd]
            top = new_top
            out[t, hd] = S.T @ q[t, hd] / (torch.maximum((n @ q[t, hd]).abs(), torch.exp(-top)) + 1e-6)
        if trace is not None:
            trace.setdefault("state", []).append((S, n, top))
    out = rms_unit(out, eps).reshape(T, H * dv) * w[p + "norm"] * torch.sigmoid(h @ w[p + "g"].T)
    return out @ w[p + "o"].T


def gated_linear_attention(h, w, p, m, eps, trace: Optional[dict] = None):
    """S <- diag(alpha) S + k v^T with a decay per key channel, alpha = sigmoid(z)^(1/tau)."""
    H, dk, dv, tau = m["heads"], m["dim"], m["vdim"], m["tau"]
    T = h.shape[0]
    q = (h @ w[p + "q"].T).view(T, H, dk) * dk ** -0.5
    k = (h @ w[p + "k"].T).view(T, H, dk)
    v = (h @ w[p + "v"].T).view(T, H, dv)
    z = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "a2.b"]
    alpha = torch.exp(log_sigmoid(z) / tau).view(T, H, dk)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for hd in range(H):
        S = torch.zeros(dk, dv, dtype=h.dtype)
        for t in range(T):
            S = alpha[t, hd].unsqueeze(1) * S + torch.outer(k[t, hd], v[t, hd])
            out[t, hd] = S.T @ q[t, hd]
        if trace is not None:
            trace.setdefault("state", []).append(S)
    out = (rms_unit(out, eps) * w[p + "norm"]).reshape(T, H * dv) * silu(h @ w[p + "g"].T)
    return out @ w[p + "o"].T


def gated_delta(h, w, p, m, eps, trace: Optional[dict] = None):
    """Delta rule with one decay per head; short convolutions and SiLU on q, k, v; unit q and k."""
    heads, kv_heads, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = silu(causal_conv(h @ w[p + "q"].T, w[p + "q.conv"])).view(T, kv_heads, dk)
    k = silu(causal_conv(h @ w[p + "k"].T, w[p + "k.conv"])).view(T, kv_heads, dk)
    v = silu(causal_conv(h @ w[p + "v"].T, w[p + "v.conv"])).view(T, heads, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[p + "b"].T)
    decay = torch.exp(-torch.exp(w[p + "A_log"]) * torch.nn.functional.softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))
    rep = heads // kv_heads
    out = torch.zeros(T, heads, dv, dtype=h.dtype)
    for hd in range(heads):
        S = torch.zeros(dk, dv, dtype=h.dtype)
        for t in range(T):
            kt, qt = k[t, hd // rep], q[t, hd // rep]
            S = decay[t, hd] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ kt)
            S = S + torch.outer(kt, u)
            out[t, hd] = S.T @ qt
        if trace is not None:
            trace.setdefault("state", []).append(S)
    out = (rms_unit(out, eps) * w[p + "norm"]).reshape(T, heads * dv) * silu(h @ w[p + "g"].T)
    return out @ w[p + "o"].T


# ---------------------------------------------------------------- layers and the model
def gated_ff(h, w, p):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def mixer(h, w, p, layer, eps):
    m, kind = layer["mixer"], layer["type"]
    if kind == "delta":
        return gated_delta(h, w, p, m, eps)
    if kind == "parallel":
        left = attention_keys_as_values(h, w, p + "left.", m["left"], eps)
        right = matrix_memory(h, w, p + "right.", m["right"], eps)
    elif kind == "parallel_2":
        left = attention_rotary(h, w, p + "left.", m["left"])
        right = gated_linear_attention(h, w, p + "right.", m["right"], eps)
    else:
        raise ValueError(kind)
    return m["left_scale"] * left + m["right_scale"] * right


def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64,
            layers_out: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence from its start."""
    w = {k: v.to(dtype) for k, v in weights.items() if v.is_floating_point()}
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens)] * cfg["embedding"]["scale"]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = layer_norm(x, w[p + "norm1"], eps)
        delta = mixer(h, w, p + "mix.", layer, eps) * w[p + "ls1"]
        if layer.get("mlp") is not None:
            delta = delta + gated_ff(h, w, p + "mlp.") * w[p + "ls2"]
        x = x + cfg["residual_mult"] * delta
        if layers_out is not None:
            layers_out.append(x)
    return layer_norm(x, w["final.norm"], eps) @ w["embed"].T
