"""The delta rule with a decay per head and key channel: a mixer whose memory is a matrix S [dk, dv] per
(request, head) instead of a cache that grows with the sequence.

For the row's input x (T rows, H heads, KH heads of queries and keys, G = H / KH value heads per key head):

  q, k, v   = x Wq^T, x Wk^T, x Wv^T, each through a causal convolution over time per channel (``conv_taps``
              taps, the last one the current token's, zeros before the sequence) and SiLU
  q, k      per head divided by sqrt(sum of squares + ``unit_eps``); q also times dk^(-1/2)
  beta      = sigmoid(x Wb^T), one per head
  g         = exp(-exp(A_log_h) softplus((x Wa1^T) Wa2^T + dt_bias)), one per head and key channel
  per head  S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q      (in this order)
  out       = (o / rms(o) * w_norm * sigmoid((x Wg1^T) Wg2^T)) Wo^T, the rms over dv with ``norm_eps``

Everything from the convolution's output on is float32; S and the convolution's last taps - 1 inputs are the
request's state (``StateSpec``), which the cache manager zeroes at admission and which the kernels update in
place, so a prompt may come in portions of any size and a decoded token is a portion of one.

Two things can be chosen otherwise.  ``decay_per_head``: one decay per head, g = exp(-exp(A_log_h) softplus(x Wa^T +
dt_bias)) with Wa [heads, hidden] and no low rank (the kernels spread it over the head's key channels).
``full_gate``: the gate's logits are x Wg^T with Wg [heads * dv, hidden], part of the fused input product, and
``gate_act`` says what is made of them (``sigmoid`` or ``silu``).

Products: one for q | k | v | beta, one for the two low ranks (a1 | g1), one for both second halves (a
block-diagonal weight, float32 result), one for the output; three kernels in between (``ops.delta_rule``).
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence

import torch

from .. import ops
from .registry import register
from .spec import CacheSpec, ParamSpec, StateSpec

SCAN_MAX_ROWS = 16      # rows of a column of S that one thread of the scan kernel keeps (csrc/delta_rule.cu)


def scan_lanes(key_dim: int) -> int:
    """Lanes that share a column of S in the scan kernel; the state's layout follows from it."""
    r = 4
    while r < 32 and -(-key_dim // r) > SCAN_MAX_ROWS:
        r *= 2
    return r


def state_floats(heads: int, kv_heads: int, key_dim: int, value_dim: int, taps: int) -> int:
    r = scan_lanes(key_dim)
    per = -(-key_dim // r)
    return heads * per * r * value_dim + (taps - 1) * (2 * kv_heads * key_dim + heads * value_dim)


@register("mixer", "channel_delta")
class ChannelDeltaRule:
    graph_safe = True
    NAMES = ("q", "k", "v", "b", "A_log", "norm", "a1", "a2", "dt_bias", "g1", "g2", "o")

    def __init__(self, hidden_size: int, heads: int, kv_heads: int, key_dim: int, value_dim: int, conv_taps: int,
                 decay_rank: int, gate_rank: int, norm_eps: float, dtype: torch.dtype, device,
                 unit_eps: float = 1e-6, conv_suffix: str = ".conv", names: Sequence[str] = NAMES,
                 decay_per_head: bool = False, full_gate: bool = False, gate_act: str = "sigmoid"):
        if heads % kv_heads:
            raise ValueError(f"{heads} heads cannot share {kv_heads} heads of queries and keys")
        if -(-key_dim // scan_lanes(key_dim)) > SCAN_MAX_ROWS:
            raise ValueError(f"keys of width {key_dim} are wider than the scan kernel takes ({32 * SCAN_MAX_ROWS})")
        if conv_taps < 1:
            raise ValueError("the convolution needs at least one tap")
        self.hidden, self.heads, self.kv_heads, self.dk, self.dv = hidden_size, heads, kv_heads, key_dim, value_dim
        self.taps, self.decay_rank, self.gate_rank = conv_taps, decay_rank, gate_rank
        self.norm_eps, self.unit_eps = float(norm_eps), float(unit_eps)
        self.dtype, self.device, self.conv_suffix, self.names = dtype, device, conv_suffix, tuple(names)
        self.channels = 2 * kv_heads * key_dim + heads * value_dim
        self.decay_per_head, self.full_gate, self.gate_act = bool(decay_per_head), bool(full_gate), gate_act
        if gate_act not in ops.GATE_ACTS:
            raise ValueError(f"gate activation {gate_act!r}; known: {sorted(ops.GATE_ACTS)}")
        self._checked = False

    # ---- weights
    @classmethod
    def param_specs(cls, hidden_size, heads, kv_heads, key_dim, value_dim, conv_taps, decay_rank, gate_rank,
                    conv_suffix: str = ".conv", names=NAMES, decay_per_head: bool = False, full_gate: bool = False,
                    **_) -> Dict[str, ParamSpec]:
        """``names``: q, k, v, b, A_log, norm, a1, a2, dt_bias, g1, g2, o.  With ``decay_per_head`` a1 names the
        one decay projection and a2 is not read; with ``full_gate`` g1 names the one gate projection and g2 is
        not read."""
        q, k, v, b, a_log, norm, a1, a2, dt_bias, g1, g2, o = names
        qk, vd = kv_heads * key_dim, heads * value_dim
        specs = {
            q: ParamSpec((qk, hidden_size)), q + conv_suffix: ParamSpec((qk, conv_taps), "unit"),
            k: ParamSpec((qk, hidden_size)), k + conv_suffix: ParamSpec((qk, conv_taps), "unit"),
            v: ParamSpec((vd, hidden_size)), v + conv_suffix: ParamSpec((vd, conv_taps), "unit"),
            b: ParamSpec((heads, hidden_size)), a_log: ParamSpec((heads,), "unit"), norm: ParamSpec((value_dim,), "norm"),
            o: ParamSpec((hidden_size, vd)),
        }
        if decay_per_head:
            specs.update({a1: ParamSpec((heads, hidden_size)), dt_bias: ParamSpec((heads,), "unit")})
        else:
            specs.update({a1: ParamSpec((decay_rank, hidden_size)), a2: ParamSpec((heads * key_dim, decay_rank)),
                          dt_bias: ParamSpec((heads * key_dim,), "unit")})
        if full_gate:
            specs[g1] = ParamSpec((vd, hidden_size))
        else:
            specs.update({g1: ParamSpec((gate_rank, hidden_size)), g2: ParamSpec((vd, gate_rank))})
        return specs

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        q, k, v, b, a_log, norm, a1, a2, dt_bias, g1, g2, o = self.names
        cs = self.conv_suffix
        # fused input product: q | k | v | (the full gate) | beta, its rows padded so that the result's rows lie on
        # 16-byte steps
        first = [t[q], t[k], t[v]] + ([t[g1]] if self.full_gate else []) + [t[b]]
        rows = sum(p.shape[0] for p in first)
        self.gate_col = self.channels if self.full_gate else None
        self.beta_col = self.channels + (self.heads * self.dv if self.full_gate else 0)
        pad = torch.zeros((-rows % 8, self.hidden), dtype=t[q].dtype, device=t[q].device)
        self.w_in = torch.cat(first + [pad], dim=0).contiguous()
        self.conv_w = torch.cat([t[q + cs], t[k + cs], t[v + cs]], dim=0).to(self.w_in.dtype).contiguous()
        self.conv_t = self.conv_w.t().contiguous()                                            # [taps, channels]
        # what is left of the decay and the gate: nothing, one plain product, or the two low ranks and their
        # block-diagonal second halves
        low = ([] if self.decay_per_head else [t[a1]]) + ([] if self.full_gate else [t[g1]])
        self.w_low = torch.cat(low, dim=0).contiguous() if low else None
        self.w_decay = t[a1].contiguous() if self.decay_per_head else None
        ra = 0 if self.decay_per_head else self.decay_rank
        rg = 0 if self.full_gate else self.gate_rank
        self.second_split = 0 if self.decay_per_head else self.heads * self.dk
        if low:
            rows2 = self.second_split + (0 if self.full_gate else self.heads * self.dv)
            second = torch.zeros((rows2, ra + rg), dtype=t[a1].dtype, device=t[a1].device)
            if not self.decay_per_head:
                second[:self.second_split, :ra] = t[a2]
            if not self.full_gate:
                second[self.second_split:, ra:] = t[g2]
            self.w_second = second.contiguous()
        self.dt_bias = t[dt_bias].to(torch.float32).contiguous()
        self.rate = torch.exp(t[a_log].to(torch.float32)).contiguous()
        self.out_weight = t[norm].to(torch.float32).contiguous()
        self.w_o = t[o].contiguous()

    # ---- what the cache manager has to provide
    def cache_spec(self) -> Optional[CacheSpec]:
        return None

    def state_spec(self) -> Optional[StateSpec]:
        return StateSpec((state_floats(self.heads, self.kv_heads, self.dk, self.dv, self.taps),), "float32")

    def workspace_floats(self, tokens: int) -> int:
        return tokens * (2 * self.channels + 3 * self.heads * (self.dk + self.dv))

    # ---- one step
    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        if not self._checked:
            want = ops.delta_rule_state_floats(self.heads, self.kv_heads, self.dk, self.dv, self.taps)
            if want != cache.state.shape[1]:
                raise ValueError(f"the scan kernel wants a state of {want} floats, the slots have {cache.state.shape[1]}")
            self._checked = True
        proj = ops.linear(x, self.w_in, out_dtype=self.dtype)
        second = None
        if self.w_low is not None:
            low = ops.linear(x, self.w_low, out_dtype=self.dtype)
            second = ops.linear(low, self.w_second, out_dtype=torch.float32)
        split = self.second_split
        a = ops.linear(x, self.w_decay, out_dtype=torch.float32) if self.decay_per_head else second[:, :split]
        gate = proj[:, self.gate_col:self.gate_col + self.heads * self.dv] if self.full_gate else second[:, split:]
        out = ops.delta_rule(proj, self.conv_w, self.taps, a, self.dt_bias, self.rate, gate,
                             self.out_weight, self.norm_eps, ctx.token_slot, ctx.seg_info, cache.state, self.heads,
                             self.kv_heads, self.dk, self.dv, self.dk ** -0.5, self.unit_eps, self.dtype, conv_t=self.conv_t,
                             decay_per_head=self.decay_per_head, beta_col=self.beta_col, gate_act=self.gate_act)
        return ops.linear(out, self.w_o, out_dtype=self.dtype)
