"""Pevolorn, plainly: whole sequences, no cache, no batching, float64 unless told otherwise; one
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


def silu(z):
    return z * torch.sigmoid(z)


def relu_squared(z):
    return torch.clamp(z, min=0.0) ** 2


def causal_conv(x: torch.Tensor, taps: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [T, C], taps [C, K]; y[t, c] = bias[c] + sum_j taps[c, K-1-j] x[t-j, c], zeros before the start."""
    T, C = x.shape
    K = taps.shape[1]
    y = torch.zeros_like(x)
    for j in range(K):
        if j < T:
            y[j:] += x[:T - j] * taps[:, K - 1 - j]
    return y if bias is None else y + bias


def rotate_half(x: torch.Tensor, positions: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """x [T, heads, d]: elements i and i + dims/2 of the first ``dims`` turn by position * base^(-2i/dims)."""
    half = dims // 2
    freq = base ** (-2.0 * torch.arange(half, dtype=x.dtype) / dims)
    ang = positions.to(x.dtype).view(-1, 1, 1) * freq
    c, s = torch.cos(ang), torch.sin(ang)
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], dim=-1)


def causal_softmax_attention(q, k, v, scale: float, softcap: Optional[float] = None) -> torch.Tensor:
    """q [T, H, dk], k [T, G, dk], v [T, G, dv]; query head h reads key/value head h // (H / G); the scaled
    score goes through cap tanh(s / cap) if there is a cap; position i sees j <= i."""
    T, H, _ = q.shape
    rep = H // k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    mask = torch.tril(torch.ones(T, T, dtype=torch.bool))
    for h in range(H):
        s = (q[:, h] @ k[:, h // rep].T) * scale
        if softcap:
            s = softcap * torch.tanh(s / softcap)
        s = s.masked_fill(~mask, float("-inf"))
        out[:, h] = torch.softmax(s, dim=-1) @ v[:, h // rep]
    return out


# ---------------------------------------------------------------- mixers
def latent_keys(x: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float):
    """(latent c [T, kv_rank], rotated shared key part [T, rot_dim]) of the layer that owns W_dkv."""
    T = x.shape[0]
    rank, rot = m["kv_rank"], m["rot_dim"]
    dkv = x @ w[p + "dkv"].T
    c = rms_unit(dkv[:, :rank], eps) * w[p + "dkv.norm"]
    pos = torch.arange(T)
    kr = rotate_half(dkv[:, rank:].view(T, 1, rot), pos, m["rot"]["base"], m["rot"]["dims"]).view(T, rot)
    return c, kr


def latent_attention(x: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float, latents) -> torch.Tensor:
    """``latents`` = (c, rotated key part) of this layer or of the layer it borrows them from."""
    T = x.shape[0]
    H, dn, dr, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    c, kr = latents
    q = (x @ w[p + "q"].T).view(T, H, dn + dr)
    pos = torch.arange(T)
    q = torch.cat([q[..., :dn], rotate_half(q[..., dn:], pos, m["rot"]["base"], m["rot"]["dims"])], dim=-1)
    k_plain = (c @ w[p + "uk"].T).view(T, H, dn)
    k = torch.cat([k_plain, kr.view(T, 1, dr).expand(T, H, dr)], dim=-1)
    v = (c @ w[p + "uv"].T).view(T, H, dv)
    o = causal_softmax_attention(q, k, v, m["scale"])
    o = o * torch.sigmoid(x @ w[p + "g"].T).view(T, H, 1)
    return o.reshape(T, H * dv) @ w[p + "o"].T


def gated_softcap_attention(x: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    """Grouped-query attention with biases on its projections, a rotation of part of each head, unit queries
    and keys (after the rotation), a capped score and one sigmoid gate per head."""
    T = x.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (x @ w[p + "q"].T + w[p + "q.b"]).view(T, H, dk)
    k = (x @ w[p + "k"].T + w[p + "k.b"]).view(T, G, dk)
    v = (x @ w[p + "v"].T + w[p + "v.b"]).view(T, G, dv)
    pos = torch.arange(T)
    q = rms_unit(rotate_half(q, pos, m["rot"]["base"], m["rot"]["dims"]), eps)
    k = rms_unit(rotate_half(k, pos, m["rot"]["base"], m["rot"]["dims"]), eps)
    o = causal_softmax_attention(q, k, v, m["scale"], m.get("softcap"))
    o = o * torch.sigmoid(x @ w[p + "g"].T).view(T, H, 1)
    return o.reshape(T, H * dv) @ w[p + "o"].T + w[p + "o.b"]


def state_space(x: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    """A selective state space with one decay per head: per head S [N, P] <- exp(-exp(A_log) dt) S + dt B u^T,
    y = S^T C + D u; y silu(z), then an RMS norm in ``norm_groups`` parts, a weight, the output product."""
    T = x.shape[0]
    H, P, N, G, taps = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
    inner = H * P
    proj = x @ w[p + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    assert dt.shape[1] == H and w[p + "conv"].shape[1] == taps
    xbc = silu(causal_conv(xbc, w[p + "conv"], w[p + "conv.b"]))
    u = xbc[:, :inner].view(T, H, P)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = torch.nn.functional.softplus(dt + w[p + "dt_bias"])
    rate = torch.exp(w[p + "A_log"])
    y = torch.zeros(T, H, P, dtype=x.dtype)
    per = H // G
    for h in range(H):
        S = torch.zeros(N, P, dtype=x.dtype)
        g = h // per
        for t in range(T):
            S = torch.exp(-rate[h] * dt[t, h]) * S + dt[t, h] * torch.outer(B[t, g], u[t, h])
            y[t, h] = S.T @ C[t, g] + w[p + "D"][h] * u[t, h]
    y = y.reshape(T, inner) * silu(z)
    parts = m["norm_groups"]
    y = rms_unit(y.view(T, parts, inner // parts), eps).reshape(T, inner) * w[p + "norm"]
    return y @ w[p + "o"].T


# ---------------------------------------------------------------- feed-forward
def route(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, r: dict):
    """(chosen [T, top] indices among experts + identity, their weights [T, top])."""
    s = torch.softmax(h @ w[p + "router"].T, dim=-1)
    choice = s + w[p + "correction"]
    total = s.shape[1]
    count, keep = r["groups"]["count"], r["groups"]["keep"]
    size = total // count
    best = choice.view(-1, count, size).max(-1).values
    kept = torch.topk(best, keep, dim=-1).indices
    allowed = torch.zeros(h.shape[0], count, dtype=torch.bool)
    allowed.scatter_(1, kept, True)
    masked = choice.masked_fill(~allowed.repeat_interleave(size, dim=1), float("-inf"))
    chosen = torch.topk(masked, r["top"], dim=-1).indices
    return chosen, torch.gather(s, 1, chosen)


def router_margin(h, w, p, r) -> torch.Tensor:
    """Per token the smallest gap between a choice the router makes and the best one it does not (group choice
    and expert choice alike), relative to the two scores that meet there: rounding moves a score in proportion
    to itself (the correction is a constant), so a gap that is small beside its scores may fall either way."""
    s = torch.softmax(h @ w[p + "router"].T, dim=-1)
    choice = s + w[p + "correction"]
    count, keep, top = r["groups"]["count"], r["groups"]["keep"], r["top"]
    T, total = s.shape
    size = total // count
    gap = torch.full((T,), math.inf, dtype=h.dtype)
    best, arg = choice.view(T, count, size).max(-1)
    s_best = torch.gather(s.view(T, count, size), 2, arg.unsqueeze(-1)).squeeze(-1)
    order = torch.argsort(best, dim=-1, descending=True)
    if keep < count:
        a, b = order[:, keep - 1:keep], order[:, keep:keep + 1]
        gap = ((best.gather(1, a) - best.gather(1, b)) / (s_best.gather(1, a) + s_best.gather(1, b))).squeeze(1)
    allowed = torch.zeros(T, count, dtype=torch.bool)
    allowed.scatter_(1, order[:, :keep], True)
    masked = choice.masked_fill(~allowed.repeat_interleave(size, dim=1), float("-inf"))
    order = torch.argsort(masked, dim=-1, descending=True)
    if top < keep * size:
        a, b = order[:, top - 1:top], order[:, top:top + 1]
        rel = ((masked.gather(1, a) - masked.gather(1, b)) / (s.gather(1, a) + s.gather(1, b))).squeeze(1)
        gap = torch.minimum(gap, rel)
    return gap


def expert(h, up, down):
    return relu_squared(h @ up.T) @ down.T


def mixture(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, mlp: dict, gaps_out: Optional[list] = None) -> torch.Tensor:
    r = mlp["router"]
    if gaps_out is not None:
        gaps_out.append(router_margin(h, w, p, r))
    real = r["experts"]
    chosen, weights = route(h, w, p, r)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, s in zip(chosen[t].tolist(), weights[t]):
            if e >= real:
                out[t] += s * h[t]
            else:
                out[t] += s * expert(h[t], w[f"{p}e{e}.up"], w[f"{p}e{e}.down"])
    if mlp.get("shared"):
        out = out + expert(h, w[p + "shared.up"], w[p + "shared.down"])
    return out


# ---------------------------------------------------------------- the model
def offset_norm(x, w, eps):
    return rms_unit(x, eps) * (1.0 + w)


def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64,
            layers_out: Optional[list] = None, gaps_out: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence.  ``layers_out`` receives the stream after every layer,
    ``gaps_out`` every router's margin per token (``router_margin``)."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps, alpha = cfg["norm"]["eps"], cfg["postln_alpha"]
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)]
    latents = {}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        if layer["type"] == "latent_attention":
            src = m.get("kv_from")
            if src is None:
                latents[i] = latent_keys(x, w, p + "mix.", m, eps)
                src = i
            a = latent_attention(x, w, p + "mix.", m, eps, latents[src])
        elif layer["type"] == "parallel":
            a = m["left_scale"] * gated_softcap_attention(x, w, p + "mix.left.", m["left"], eps) \
                + m["right_scale"] * state_space(x, w, p + "mix.right.", m["right"], eps)
        else:
            raise ValueError(layer["type"])
        x = offset_norm(alpha * x + a, w[p + "norm1"], eps)
        if layer.get("mlp") is not None:
            x = offset_norm(alpha * x + mixture(x, w, p + "mlp.", layer["mlp"], gaps_out), w[p + "norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    x = offset_norm(x, w["final.norm"], eps)
    return x @ w["embed"].T


def decisive_tokens(cfg, w, tokens, seed, threshold=0.12, tries=1000):
    """``tokens`` with some of them drawn again until no router of the model meets a near-tie anywhere in the
    sequence (every margin above ``threshold``).  In 16-bit arithmetic a near-tie falls either way, and the row
    then differs by a whole expert; a comparison of logits wants prompts on which the design's answer does not
    hang on the last bit.  Tokens before the first near-tie stay as they are (the model is causal), so the search
    moves from left to right."""
    g = torch.Generator().manual_seed(seed)
    tokens = list(tokens)
    for _ in range(tries):
        gaps = []
        forward(cfg, w, tokens, gaps_out=gaps)
        if not gaps:
            return tokens
        close = (torch.stack(gaps).min(0).values < threshold).nonzero().flatten()
        if close.numel() == 0:
            return tokens
        tokens[int(close[0])] = int(torch.randint(0, cfg["vocab"], (1,), generator=g))
    raise RuntimeError("no sequence without near-ties found")
