"""Attention whose keys and values come from one small vector per token.

For the row's input x (H heads; per head ``plain_dim`` unrotated and ``rot_dim`` rotated query/key
elements, values of ``value_dim``; latents of ``q_rank`` and ``kv_rank``):

  c_q       = rmsnorm(x Wdq^T) (plain gain);  q = c_q Wuq^T, per head [plain | rotated]
  c, k_r    = x Wdkv^T split after kv_rank elements: c = rmsnorm(first part) (plain gain), k_r is rotated and
              shared by all heads
  per head  k = [Wuk_h c | k_r], v = Wuv_h c;  score = (q . k) * scale
  rotation  neighbours (2i, 2i + 1) of the first ``rot_dims`` elements of the rotated part:
            (u, v) -> (u cos a - v sin a, v cos a + u sin a), a = position * f_i, f_i = base^(-2i / rot_dims);
            with ``scaling`` (factor, original, fast, slow) the slow frequencies are divided by factor along
            a ramp, and cos and sin are multiplied by 0.1 ln(factor) + 1 (``rotation_frequencies``)
  visible   keys j <= i, and i - j < ``window`` if there is one
  softmax   with ``sink`` the denominator also holds exp(z_h), a learned number per head without key or value
  out       = (concatenated heads * sigmoid(x Wg^T)) Wo^T if ``output_gate``; with ``gate_per_head`` Wg has one row
            per head and a head is multiplied by one number

Options: ``q_rank=0`` projects the queries directly, q = x Wq^T (tensor ``q_name``), with no latent and no norm
on their side.  ``rotation='half'`` pairs element i with i + rot_dims / 2 instead of its neighbour.
``borrows_cache``: the layer has no Wdkv; it reads the cache of another layer (the run order names which), whose
latents and rotated key parts it uses with its own Wuk and Wuv, and writes nothing.

Only [c | k_r] is cached (one plane of one head per token).  The per-head matrices are applied on the
query's side: q_h . (Wuk_h c) = (Wuk_h^T q_h) . c, and sum_j p_j (Wuv_h c_j) = Wuv_h (sum_j p_j c_j), so the
attention kernels see multi-query attention with keys [c | k_r] and values c (``values_in_keys``), and two
batched products of the library stand before and behind them.
"""
from __future__ import annotations

import math
from typing import Dict, Optional, Sequence, Tuple

import torch

from .. import ops
from .registry import register
from .spec import CacheSpec, ParamSpec, StateSpec


def rotation_frequencies(dims: int, base: float, scaling: Optional[dict] = None) -> Tuple[torch.Tensor, float]:
    """(float32 frequencies of the dims / 2 pairs, factor on cos and sin).  ``scaling`` holds ``factor``,
    ``original``, ``fast`` and ``slow``: with dim(t) = dims ln(original / (2 pi t)) / (2 ln base),
    lo = max(floor(dim(fast)), 0), hi = min(ceil(dim(slow)), dims - 1) and ramp_i = clamp((i - lo) /
    max(hi - lo, 0.001), 0, 1), the frequency is f_i / factor * ramp_i + f_i (1 - ramp_i).  Computed in float64."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = float(base) ** (-2.0 * i / dims)
    if not scaling:
        return f.to(torch.float32), 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def dim_of(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(float(base)))

    lo = max(math.floor(dim_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(dim_of(float(scaling["slow"]))), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return (f / factor * ramp + f * (1.0 - ramp)).to(torch.float32), 0.1 * math.log(factor) + 1.0


@register("mixer", "latent_attention")
class LatentAttention:
    graph_safe = True
    NAMES = ("dq", "dq.norm", "uq", "dkv", "dkv.norm", "uk", "uv", "sink", "g", "o")

    def __init__(self, hidden_size: int, heads: int, plain_dim: int, rot_dim: int, value_dim: int, q_rank: int,
                 kv_rank: int, scale: float, norm_eps: float, rot_base: float, dtype: torch.dtype, device,
                 rot_dims: Optional[int] = None, scaling: Optional[dict] = None, window: Optional[int] = None,
                 sink: bool = False, output_gate: bool = False, names: Sequence[str] = NAMES,
                 q_name: str = "q", rotation: str = "neighbours", gate_per_head: bool = False,
                 borrows_cache: bool = False):
        rot_dims = rot_dim if rot_dims is None else rot_dims
        if rotation not in ("neighbours", "half"):
            raise ValueError(f"rotation {rotation!r} is neither 'neighbours' nor 'half'")
        if gate_per_head and not output_gate:
            raise ValueError("a gate per head is an output gate: give output_gate=True")
        self.q_name, self.half_pairs, self.gate_per_head = q_name, rotation == "half", bool(gate_per_head)
        self.borrows_cache = bool(borrows_cache)
        if rot_dims % 2 or not 0 <= rot_dims <= rot_dim:
            raise ValueError(f"rot_dims {rot_dims} must be even and at most rot_dim {rot_dim}")
        if window is not None and window <= 0:
            raise ValueError(f"window must be positive (or None), got {window}")
        self.hidden, self.heads, self.dn, self.dr, self.dv = hidden_size, heads, plain_dim, rot_dim, value_dim
        self.q_rank, self.rank, self.scale, self.norm_eps = q_rank, kv_rank, float(scale), float(norm_eps)
        self.rot_dims, self.window, self.sink, self.output_gate = rot_dims, window, bool(sink), bool(output_gate)
        self.dtype, self.device, self.names = dtype, device, tuple(names)
        freq, self.mag = rotation_frequencies(rot_dims, rot_base, scaling) if rot_dims else (torch.zeros(1), 1.0)
        self.freq = freq.to(device)

    # ---- weights
    @classmethod
    def param_specs(cls, hidden_size, heads, plain_dim, rot_dim, value_dim, q_rank, kv_rank, sink=False,
                    output_gate=False, names=NAMES, q_name="q", gate_per_head=False, borrows_cache=False,
                    **_) -> Dict[str, ParamSpec]:
        dq, dq_norm, uq, dkv, dkv_norm, uk, uv, sink_name, g, o = names
        specs = {
            uk: ParamSpec((heads * plain_dim, kv_rank)), uv: ParamSpec((heads * value_dim, kv_rank)),
            o: ParamSpec((hidden_size, heads * value_dim)),
        }
        if q_rank:
            specs.update({dq: ParamSpec((q_rank, hidden_size)), dq_norm: ParamSpec((q_rank,), "norm"),
                          uq: ParamSpec((heads * (plain_dim + rot_dim), q_rank))})
        else:
            specs[q_name] = ParamSpec((heads * (plain_dim + rot_dim), hidden_size))
        if not borrows_cache:
            specs.update({dkv: ParamSpec((kv_rank + rot_dim, hidden_size)), dkv_norm: ParamSpec((kv_rank,), "norm")})
        if sink:
            specs[sink_name] = ParamSpec((heads,), "unit")
        if output_gate:
            specs[g] = ParamSpec((heads if gate_per_head else heads * value_dim, hidden_size))
        return specs

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        dq, dq_norm, uq, dkv, dkv_norm, uk, uv, sink_name, g, o = self.names
        # one product for [query latent or queries | key/value latent and shared key part | gate]; with direct
        # queries every piece starts on a multiple of eight rows, so that the views of its result stay on 16-byte
        # boundaries
        self.q_cols = self.q_rank if self.q_rank else self.heads * (self.dn + self.dr)
        parts, at, self.col = [], 0, {}
        for key, w in (("q", t[dq] if self.q_rank else t[self.q_name]),
                       ("c", None if self.borrows_cache else t[dkv]), ("g", t[g] if self.output_gate else None)):
            if w is None:
                continue
            self.col[key] = at
            rows = w.shape[0]
            parts.append(w)
            pad = 0 if self.q_rank else -rows % 8        # (a query latent and c stay neighbours: one kernel norms both)
            if pad:
                parts.append(torch.zeros((pad, self.hidden), dtype=w.dtype, device=w.device))
            at += rows + pad
        self.w_in = torch.cat(parts, dim=0).contiguous()
        self.q_gain = t[dq_norm].to(torch.float32).contiguous() if self.q_rank else None
        self.c_gain = None if self.borrows_cache else t[dkv_norm].to(torch.float32).contiguous()
        self.w_uq = t[uq].contiguous() if self.q_rank else None
        self.w_uk = t[uk].view(self.heads, self.dn, self.rank).contiguous()                       # q_h -> Wuk_h^T q_h
        self.w_uv_t = t[uv].view(self.heads, self.dv, self.rank).transpose(1, 2).contiguous()     # latent mix -> value
        self.sink_logits = t[sink_name].to(torch.float32).contiguous() if self.sink else None
        self.w_o = t[o].contiguous()

    # ---- what the cache manager has to provide
    def cache_spec(self) -> Optional[CacheSpec]:
        return CacheSpec(((1, self.rank + self.dr),), self.window)

    def state_spec(self) -> Optional[StateSpec]:
        return None

    def workspace_floats(self, tokens: int) -> int:
        per_head = self.dn + self.dr + 2 * (self.rank + self.dr) + self.rank + 2 * self.dv
        return tokens * (self.q_rank + self.rank + self.dr + self.heads * per_head)

    # ---- one step
    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        tokens, H = x.shape[0], self.heads
        (plane,) = cache.planes
        proj = ops.linear(x, self.w_in, out_dtype=self.dtype)
        if self.borrows_cache and cache.writes:
            raise ValueError("a layer that borrows another's latents must not write the cache (writes_cache=False)")
        if self.q_rank:                  # [query latent | c | shared key part] lie side by side: one kernel norms both
            cq = ops.latent_norm_store(proj, self.q_rank, self.rank, self.dr, self.rot_dims, self.q_gain, self.c_gain,
                                       self.norm_eps, self.freq, self.mag, ctx.positions, ctx.token_slot,
                                       cache.block_table, plane, cache.page_size, store=cache.writes,
                                       half_pairs=self.half_pairs)
            q = ops.linear(cq, self.w_uq, out_dtype=self.dtype)
        else:
            if not self.borrows_cache:
                ops.latent_norm_store(proj[:, self.col["c"]:], 0, self.rank, self.dr, self.rot_dims, None, self.c_gain,
                                      self.norm_eps, self.freq, self.mag, ctx.positions, ctx.token_slot,
                                      cache.block_table, plane, cache.page_size, store=cache.writes,
                                      half_pairs=self.half_pairs)
            q = proj[:, :self.q_cols]
        q_plain = q.view(tokens, H, self.dn + self.dr)[:, :, :self.dn].transpose(0, 1)             # [H, T, dn]
        lat = torch.bmm(q_plain, self.w_uk)                                                        # [H, T, rank]
        q_full = ops.latent_query(q, lat, H, self.dn, self.dr, self.rot_dims, self.rank, self.freq, self.mag,
                                  ctx.positions, ctx.token_slot, half_pairs=self.half_pairs)
        mix = torch.empty((tokens, H * self.rank), dtype=self.dtype, device=x.device)
        ops.attention_biased(q_full, plane, plane, ctx.positions, ctx.token_slot, cache.block_table, cache.page_size,
                             H, 1, self.rank + self.dr, self.rank, self.scale, mix, window=self.window or 0,
                             sink=self.sink, sink_logits=self.sink_logits, ctx=ctx, values_in_keys=True)
        o = torch.bmm(mix.view(tokens, H, self.rank).transpose(0, 1), self.w_uv_t)                 # [H, T, dv]
        gate = None
        if self.output_gate:
            at = self.col["g"]
            gate = proj[:, at:at + (H if self.gate_per_head else H * self.dv)]
        out = ops.heads_gate(o, gate, ctx.token_slot, per_head=self.gate_per_head)
        return ops.linear(out, self.w_o, out_dtype=self.dtype)
