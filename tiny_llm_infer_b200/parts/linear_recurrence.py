"""Mixers whose memory is a matrix S [dk, dv] per (request, head) that every token decays and writes to without
the delta rule's correction: S <- decay S + k (w v)^T, o = S^T q.  They share the scan kernel of the delta rule
(``ops.linear_recurrence``); the state is float32, zeroed at admission and carried from step to step, so a prompt
may come in portions of any size.  For the row's input x, with q = x Wq^T times dk^(-1/2), k = x Wk^T (heads x dk)
and v = x Wv^T (heads x dv):

``gated_linear``   a decay per key channel, alpha = sigmoid(z)^(1/tau) with z = (x Wa1^T) Wa2^T + bias (a low rank),
                   w = 1.  The read-out is divided by its root mean square per head (``norm_eps``), times a weight of
                   dv numbers shared by the heads, times SiLU(x Wg^T).

``matrix_memory``  two scalar gates per head that come as logarithms, each logit capped as cap tanh(. / cap):
                   i = capped(x Wi^T + bi), f = logsigmoid(capped(x Wf^T + bf)).  A running maximum m (it starts at
                   zero) keeps the exponentials in range: m' = max(f + m, i), decay = exp(f + m - m'), w = exp(i -
                   m').  A vector n <- decay n + w k is kept beside S, and o = S^T q / (max(|n . q|, exp(-m')) +
                   ``floor_eps``).  The read-out is divided by its root mean square per head, times a weight of
                   heads x dv numbers, times sigmoid(x Wg^T).

Both end with the output product Wo.  Products: one for q | k | v | gate; one for the gates' logits (float32
result; ``gated_linear``: the low rank first); the output.
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence

import torch

from .. import ops
from .delta_rule import SCAN_MAX_ROWS, scan_lanes
from .registry import register
from .spec import CacheSpec, ParamSpec, StateSpec


class _LinearRecurrence:
    graph_safe = True
    KIND = ""

    def _init_common(self, hidden_size, heads, key_dim, value_dim, norm_eps, dtype, device):
        if -(-key_dim // scan_lanes(key_dim)) > SCAN_MAX_ROWS:
            raise ValueError(f"keys of width {key_dim} are wider than the scan kernel takes ({32 * SCAN_MAX_ROWS})")
        self.hidden, self.heads, self.dk, self.dv = hidden_size, heads, key_dim, value_dim
        self.norm_eps, self.dtype, self.device = float(norm_eps), dtype, device
        self._checked = False

    def _pad_rows(self, parts):
        rows = sum(p.shape[0] for p in parts)
        pad = torch.zeros((-rows % 8, self.hidden), dtype=parts[0].dtype, device=parts[0].device)
        return torch.cat(list(parts) + [pad], dim=0).contiguous()

    def cache_spec(self) -> Optional[CacheSpec]:
        return None

    def state_spec(self) -> Optional[StateSpec]:
        per = -(-self.dk // scan_lanes(self.dk)) * scan_lanes(self.dk)
        cols = self.dv + 1 if self.KIND == "log_gates" else self.dv
        return StateSpec((self.heads * per * cols + (self.heads * cols if self.KIND == "log_gates" else 0),), "float32")

    def workspace_floats(self, tokens: int) -> int:
        return tokens * self.heads * (4 * self.dk + 5 * self.dv + 8)

    def _check_state(self, cache) -> None:
        if not self._checked:
            want = ops.linear_recurrence_state_floats(self.KIND, self.heads, self.dk, self.dv)
            if want != cache.state.shape[1]:
                raise ValueError(f"the scan kernel wants a state of {want} floats, the slots have {cache.state.shape[1]}")
            self._checked = True


@register("mixer", "gated_linear")
class GatedLinearAttention(_LinearRecurrence):
    KIND = "channel_decay"
    NAMES = ("q", "k", "v", "g", "o", "norm", "a1", "a2")

    def __init__(self, hidden_size: int, heads: int, key_dim: int, value_dim: int, decay_rank: int, tau: float,
                 norm_eps: float, dtype: torch.dtype, device, gate_act: str = "silu", bias_suffix: str = ".b",
                 names: Sequence[str] = NAMES):
        self._init_common(hidden_size, heads, key_dim, value_dim, norm_eps, dtype, device)
        if not tau > 0.0:
            raise ValueError(f"tau must be positive, got {tau}")
        self.decay_rank, self.tau, self.gate_act = int(decay_rank), float(tau), gate_act
        self.bias_suffix, self.names = bias_suffix, tuple(names)

    @classmethod
    def param_specs(cls, hidden_size, heads, key_dim, value_dim, decay_rank, bias_suffix: str = ".b", names=NAMES,
                    **_) -> Dict[str, ParamSpec]:
        q, k, v, g, o, norm, a1, a2 = names
        qk, vd = heads * key_dim, heads * value_dim
        return {q: ParamSpec((qk, hidden_size)), k: ParamSpec((qk, hidden_size)), v: ParamSpec((vd, hidden_size)),
                g: ParamSpec((vd, hidden_size)), o: ParamSpec((hidden_size, vd)), norm: ParamSpec((value_dim,), "norm"),
                a1: ParamSpec((decay_rank, hidden_size)), a2: ParamSpec((qk, decay_rank)),
                a2 + bias_suffix: ParamSpec((qk,), "unit")}

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        q, k, v, g, o, norm, a1, a2 = self.names
        self.w_in = self._pad_rows([t[q], t[k], t[v], t[g]])
        self.w_a1, self.w_a2 = t[a1].contiguous(), t[a2].contiguous()
        self.z_bias = t[a2 + self.bias_suffix].to(torch.float32).contiguous()
        self.out_weight = t[norm].to(torch.float32).contiguous()
        self.w_o = t[o].contiguous()

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        self._check_state(cache)
        proj = ops.linear(x, self.w_in, out_dtype=self.dtype)
        z = ops.linear(ops.linear(x, self.w_a1, out_dtype=self.dtype), self.w_a2, out_dtype=torch.float32)
        at = self.heads * (2 * self.dk + self.dv)
        out = ops.linear_recurrence(proj, self.KIND, z, self.z_bias, 1.0 / self.tau, proj[:, at:at + self.heads * self.dv],
                                    self.gate_act, self.out_weight, False, self.norm_eps, ctx.token_slot, ctx.seg_info,
                                    cache.state, self.heads, self.dk, self.dv, self.dk ** -0.5, self.dtype)
        return ops.linear(out, self.w_o, out_dtype=self.dtype)


@register("mixer", "matrix_memory")
class MatrixMemory(_LinearRecurrence):
    KIND = "log_gates"
    NAMES = ("q", "k", "v", "g", "o", "norm", "i", "f")

    def __init__(self, hidden_size: int, heads: int, key_dim: int, value_dim: int, gate_cap: float, norm_eps: float,
                 dtype: torch.dtype, device, floor_eps: float = 1e-6, gate_act: str = "sigmoid",
                 bias_suffix: str = ".b", names: Sequence[str] = NAMES):
        self._init_common(hidden_size, heads, key_dim, value_dim, norm_eps, dtype, device)
        if not gate_cap > 0.0:
            raise ValueError(f"the gates' cap must be positive, got {gate_cap}")
        self.gate_cap, self.floor_eps, self.gate_act = float(gate_cap), float(floor_eps), gate_act
        self.bias_suffix, self.names = bias_suffix, tuple(names)

    @classmethod
    def param_specs(cls, hidden_size, heads, key_dim, value_dim, bias_suffix: str = ".b", names=NAMES,
                    **_) -> Dict[str, ParamSpec]:
        q, k, v, g, o, norm, i, f = names
        qk, vd = heads * key_dim, heads * value_dim
        return {q: ParamSpec((qk, hidden_size)), k: ParamSpec((qk, hidden_size)), v: ParamSpec((vd, hidden_size)),
                g: ParamSpec((vd, hidden_size)), o: ParamSpec((hidden_size, vd)), norm: ParamSpec((vd,), "norm"),
                i: ParamSpec((heads, hidden_size)), i + bias_suffix: ParamSpec((heads,), "unit"),
                f: ParamSpec((heads, hidden_size)), f + bias_suffix: ParamSpec((heads,), "unit")}

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        q, k, v, g, o, norm, i, f = self.names
        self.w_in = self._pad_rows([t[q], t[k], t[v], t[g]])
        self.w_gates = torch.cat([t[i], t[f]], dim=0).contiguous()
        self.z_bias = torch.cat([t[i + self.bias_suffix], t[f + self.bias_suffix]]).to(torch.float32).contiguous()
        self.out_weight = t[norm].to(torch.float32).contiguous()
        self.w_o = t[o].contiguous()

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        self._check_state(cache)
        proj = ops.linear(x, self.w_in, out_dtype=self.dtype)
        z = ops.linear(x, self.w_gates, out_dtype=torch.float32)
        at = self.heads * (2 * self.dk + self.dv)
        out = ops.linear_recurrence(proj, self.KIND, z, self.z_bias, self.gate_cap, proj[:, at:at + self.heads * self.dv],
                                    self.gate_act, self.out_weight, True, self.norm_eps, ctx.token_slot, ctx.seg_info,
                                    cache.state, self.heads, self.dk, self.dv, self.dk ** -0.5, self.dtype,
                                    floor_eps=self.floor_eps)
        return ops.linear(out, self.w_o, out_dtype=self.dtype)
