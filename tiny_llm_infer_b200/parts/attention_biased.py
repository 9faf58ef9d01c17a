"""Grouped-query attention whose queries, keys and score are changed between the projections and the
softmax, with an output gate.  Every step is a parameter, so other designs can pick their own mix:

  q, k        per head divided by their root mean square over the head (``unit_norm_eps``; None: not), then,
              with ``qk_gains``, multiplied by a learned gain of the head's width (tensors ``<q>.norm``, ``<k>.norm``,
              shared by the heads); ``position`` (a part of the position registry that the norm kernel can apply
              itself, such as ``rotary_half`` over part of the head): q and k turned by their positions
  values      projected by Wv, or, ``values_are_keys``, the keys as projected, before their norm (no Wv)
  temperature ``q_temperature`` (coef, every): the query at position p times 1 + coef ln(floor((p + 1) / every) + 1)
  score       s = (q . k) * scale;  ``softcap`` c: s <- c tanh(s / c);  ``bias_slopes`` m_h: s <- s - m_h (i - j)
              (``slope_exponent`` e instead of explicit slopes: m_h = 2^(-e (h + 1) / heads));
              ``distance_bias`` (rows B, far D): s <- s + rel[bucket(i - j), h] with a learned table ``rel`` [B, heads]
              whose first B/2 rows serve one distance each and whose other rows widen geometrically up to D:
              bucket(n) = n for n < B/2, else min(B - 1, B/2 + floor(ln(n / (B/2)) / ln(D / (B/2)) (B - B/2)))
  visible     j <= i, within the query's own chunk of ``chunk`` positions counted from 0 (None: no
              chunks), and within ``window`` keys back (None: no window)
  softmax     ``sink``: one is added to the denominator (a key of score 0 that carries no value); with
              ``learned_sink`` exp(z_h) instead, z_h a learned number per head (tensor ``sink``)
  gate        ``output_gate``: the concatenated heads are multiplied by sigmoid(Wg x), x the mixer's input; with
              ``gate_per_head`` Wg has one row per head and a head is multiplied by one number
  biases      ``biases``: q, k, v and the output product have biases (tensors ``<name>`` + ``bias_suffix``), added in
              float32 where the norm kernel reads the projections; the output's is added by the product, or, with
              ``defer_output_bias``, left as ``deferred_bias`` for the block's sum kernel to add

Keys have width ``key_dim`` and values ``value_dim``; they are two planes of the paged cache.  With a
chunk or a window the cache keeps only the keys a later query can still see (a chunk never reaches
further back than a window of the same size).  The projections q | k | v | gate are one product with
the row-wise concatenation of their weights; the norm of q and k and the write of k and v are one
kernel; the gate is applied where the attention kernel writes its result.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .. import ops
from .registry import lookup, register
from .spec import CacheSpec, ParamSpec, PartSpec, StateSpec


def slopes_from_exponent(heads: int, exponent: float):
    return [2.0 ** (-exponent * (h + 1) / heads) for h in range(heads)]


def distance_buckets(rows: int, far: float) -> List[int]:
    """Row of a table of ``rows`` biases for every distance 0 .. ceil(far): one row per distance below rows / 2,
    then rows that widen geometrically until ``far``; every distance beyond the list has the row of its last
    entry (the table's last row, which distances reach at ``far`` at the latest)."""
    half = rows // 2
    if half < 1 or not far > half:
        raise ValueError(f"a distance table of {rows} rows reaching to {far} has no geometric part")
    out = []
    for n in range(int(math.ceil(far)) + 1):
        if n < half:
            out.append(n)
        else:
            out.append(min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half)))))
    return out


@register("mixer", "biased_attention")
class BiasedAttention:
    graph_safe = True
    NAMES = ("q", "k", "v", "o", "g")

    def __init__(self, hidden_size: int, q_heads: int, kv_heads: int, key_dim: int, value_dim: int,
                 scale: float, dtype: torch.dtype, device, unit_norm_eps: Optional[float] = None,
                 softcap: Optional[float] = None, slope_exponent: Optional[float] = None,
                 bias_slopes: Optional[Sequence[float]] = None, chunk: Optional[int] = None,
                 window: Optional[int] = None, sink: bool = False, output_gate: bool = False,
                 names: Sequence[str] = NAMES, qk_gains: bool = False, gain_suffix: str = ".norm",
                 position: Optional[PartSpec] = None, values_are_keys: bool = False,
                 q_temperature: Optional[Tuple[float, int]] = None,
                 distance_bias: Optional[Tuple[int, float]] = None, bias_name: str = "rel",
                 learned_sink: bool = False, sink_name: str = "sink", gate_per_head: bool = False,
                 biases: bool = False, bias_suffix: str = ".b", defer_output_bias: bool = False):
        if q_heads % kv_heads:
            raise ValueError(f"{q_heads} query heads cannot share {kv_heads} key/value heads")
        if unit_norm_eps is not None and not unit_norm_eps > 0.0:
            raise ValueError(f"unit_norm_eps must be positive (or None for no head norm), got {unit_norm_eps}")
        for what, v in (("chunk", chunk), ("window", window)):
            if v is not None and v <= 0:
                raise ValueError(f"{what} must be positive (or None), got {v}")
        if softcap is not None and not softcap > 0.0:
            raise ValueError(f"softcap must be positive (or None), got {softcap}")
        self.hidden, self.q_heads, self.kv_heads = hidden_size, q_heads, kv_heads
        self.dk, self.dv = key_dim, value_dim
        self.scale, self.softcap = float(scale), softcap
        self.unit_norm_eps, self.chunk, self.window = unit_norm_eps, chunk, window
        self.sink, self.output_gate = bool(sink), bool(output_gate)
        self.dtype, self.device, self.names = dtype, device, tuple(names)
        if bias_slopes is None and slope_exponent is not None:
            bias_slopes = slopes_from_exponent(q_heads, slope_exponent)
        self.slopes = None
        if bias_slopes is not None:
            if len(bias_slopes) != q_heads:
                raise ValueError(f"{len(bias_slopes)} slopes for {q_heads} heads")
            self.slopes = torch.tensor(list(bias_slopes), dtype=torch.float64).to(torch.float32).to(device)
        self.qk_gains, self.gain_suffix = bool(qk_gains), gain_suffix
        if self.qk_gains and unit_norm_eps is None:
            raise ValueError("gains on queries and keys come with their norm: give unit_norm_eps")
        self.values_are_keys = bool(values_are_keys)
        if self.values_are_keys and key_dim != value_dim:
            raise ValueError(f"keys of width {key_dim} cannot be values of width {value_dim}")
        self.q_temperature = None
        if q_temperature is not None:
            coef, every = q_temperature
            if int(every) <= 0:
                raise ValueError(f"the query temperature counts positions in runs of {every}")
            self.q_temperature = (float(coef), int(every))
        self.distance_bias, self.bias_name = None, bias_name
        if distance_bias is not None:
            rows, far = distance_bias
            self.distance_bias = (int(rows), float(far))
            self._buckets = distance_buckets(int(rows), float(far))
        self.learned_sink, self.sink_name = bool(learned_sink), sink_name
        if self.learned_sink and not self.sink:
            raise ValueError("a learned sink is a sink: give sink=True")
        self.inv_freq, self.rot_dims = None, 0
        if position is not None:
            part = lookup("position", position.kind)(dtype=dtype, device=device, **position.params)
            if not hasattr(part, "fused_rotary"):
                raise ValueError(f"position encoding {position.kind!r} cannot be applied by the norm kernel")
            self.inv_freq, self.rot_dims = part.fused_rotary()
            if self.rot_dims > key_dim:
                raise ValueError(f"a rotation of {self.rot_dims} elements in heads of {key_dim}")
        self.gate_per_head, self.biases, self.bias_suffix = bool(gate_per_head), bool(biases), bias_suffix
        self.defer_output_bias = bool(defer_output_bias) and self.biases
        if self.gate_per_head and not self.output_gate:
            raise ValueError("a gate per head is an output gate: give output_gate=True")
        self.in_bias = self.out_bias = self.deferred_bias = None
        self.q_gain = self.k_gain = self.bias_table = self.sink_logits = None
        self.w_in = self.w_o = None

    # ---- weights
    @classmethod
    def param_specs(cls, hidden_size, q_heads, kv_heads, key_dim, value_dim, output_gate=False,
                    names=NAMES, qk_gains=False, gain_suffix=".norm", values_are_keys=False, distance_bias=None,
                    bias_name="rel", learned_sink=False, sink_name="sink", gate_per_head=False, biases=False,
                    bias_suffix=".b", **_) -> Dict[str, ParamSpec]:
        q, k, v, o, g = names
        specs = {
            q: ParamSpec((q_heads * key_dim, hidden_size)),
            k: ParamSpec((kv_heads * key_dim, hidden_size)),
            o: ParamSpec((hidden_size, q_heads * value_dim)),
        }
        if not values_are_keys:
            specs[v] = ParamSpec((kv_heads * value_dim, hidden_size))
        if output_gate:
            specs[g] = ParamSpec((q_heads if gate_per_head else q_heads * value_dim, hidden_size))
        if biases:
            for name in (q, k, o) + (() if values_are_keys else (v,)):
                specs[name + bias_suffix] = ParamSpec((specs[name].shape[0],), "unit")
        if qk_gains:
            specs[q + gain_suffix] = ParamSpec((key_dim,), "norm")
            specs[k + gain_suffix] = ParamSpec((key_dim,), "norm")
        if distance_bias is not None:
            specs[bias_name] = ParamSpec((int(distance_bias[0]), q_heads), "unit")
        if learned_sink:
            specs[sink_name] = ParamSpec((q_heads,), "unit")
        return specs

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        q, k, v, o, g = self.names
        parts = [t[q], t[k]] + ([] if self.values_are_keys else [t[v]]) + ([t[g]] if self.output_gate else [])
        common = torch.float32 if any(p.dtype == torch.float32 for p in parts) else parts[0].dtype
        if sum(p.shape[0] for p in parts) % 8:            # rows of the fused product stay whole 16-byte pieces
            parts.append(torch.zeros((-sum(p.shape[0] for p in parts) % 8, self.hidden), dtype=common, device=parts[0].device))
        self.w_in = torch.cat([p.to(common) for p in parts], dim=0).contiguous()
        self.w_o = t[o].contiguous()
        if self.biases:
            names = [q, k] + ([] if self.values_are_keys else [v])
            self.in_bias = torch.cat([t[n + self.bias_suffix].to(torch.float32) for n in names]).contiguous()
            if self.defer_output_bias:
                self.deferred_bias = t[o + self.bias_suffix].to(torch.float32).contiguous()
            else:
                self.out_bias = t[o + self.bias_suffix].contiguous()
        if self.qk_gains:
            self.q_gain = t[q + self.gain_suffix].to(self.dtype).contiguous()
            self.k_gain = t[k + self.gain_suffix].to(self.dtype).contiguous()
        if self.distance_bias is not None:
            # the learned rows spread out by distance once, [heads, distances]: the kernels look a distance up
            # directly and use the last entry for everything beyond
            rel = t[self.bias_name].to(torch.float32)
            index = torch.tensor(self._buckets, dtype=torch.long, device=rel.device)
            self.bias_table = rel[index].t().contiguous()
        if self.learned_sink:
            self.sink_logits = t[self.sink_name].to(torch.float32).contiguous()

    # ---- what the cache manager has to provide
    def reach(self) -> Optional[int]:
        """Keys back from a query (itself included) that the mask can let through, None for all."""
        limits = [v for v in (self.chunk, self.window) if v is not None]
        return min(limits) if limits else None

    def cache_spec(self) -> Optional[CacheSpec]:
        return CacheSpec(((self.kv_heads, self.dk), (self.kv_heads, self.dv)), self.reach())

    def state_spec(self) -> Optional[StateSpec]:
        return None

    def workspace_floats(self, tokens: int) -> int:
        width_in = (self.q_heads + self.kv_heads) * self.dk + (self.kv_heads + 2 * self.q_heads) * self.dv
        return tokens * (width_in + self.q_heads * self.dk)

    # ---- one step
    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        tokens = x.shape[0]
        proj = ops.linear(x, self.w_in, out_dtype=self.dtype)
        q = torch.empty((tokens, self.q_heads * self.dk), dtype=self.dtype, device=x.device)
        k_plane, v_plane = cache.planes
        ops.qkv_unit_store(proj, q, ctx.positions, ctx.token_slot, cache.block_table, k_plane, v_plane,
                           cache.page_size, self.q_heads, self.kv_heads, self.dk, self.dv,
                           self.unit_norm_eps, q_gain=self.q_gain, k_gain=self.k_gain, store=cache.writes,
                           inv_freq=self.inv_freq, rot_dims=self.rot_dims, q_temperature=self.q_temperature,
                           values_are_keys=self.values_are_keys, bias=self.in_bias)
        gate = None
        if self.output_gate:
            at = (self.q_heads + self.kv_heads) * self.dk + (0 if self.values_are_keys else self.kv_heads * self.dv)
            gate = proj[:, at:at + (self.q_heads if self.gate_per_head else self.q_heads * self.dv)]
        out = torch.empty((tokens, self.q_heads * self.dv), dtype=self.dtype, device=x.device)
        ops.attention_biased(q, k_plane, v_plane, ctx.positions, ctx.token_slot, cache.block_table,
                             cache.page_size, self.q_heads, self.kv_heads, self.dk, self.dv, self.scale, out,
                             softcap=self.softcap or 0.0, chunk=self.chunk or 0, window=self.window or 0,
                             sink=self.sink, slopes=self.slopes, gate=gate, ctx=ctx, sink_logits=self.sink_logits,
                             distance_bias=self.bias_table, gate_per_head=self.gate_per_head)
        return ops.linear(out, self.w_o, out_dtype=self.dtype, bias=self.out_bias)
