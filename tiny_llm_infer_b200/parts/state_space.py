"""A selective state space with one decay per head (the form whose recurrence is also a masked attention), as a
mixer.  For the row's input x, with H heads of width P (``head_dim``), a state of N rows (``state``) and G
``groups`` (head h uses group h // (H / G)):

  W_in x = [z: H P | u: H P | B: G N | C: G N | dt: H]
  u, B, C  pass a causal convolution per channel (``conv_taps`` taps with a bias, zeros before the start) and SiLU
  dt       = softplus(dt + dt_bias), no clamp
  per head S <- exp(-exp(A_log_h) dt) S + dt B u^T  (S is N x P, starts at zero);  y = S^T C + D_h u
  out      = W_o (rmsnorm_parts(y silu(z)) * weight): the gate comes before the norm, which divides each of
             ``norm_groups`` equal parts of the row by its own root mean square

The state (S of every head in the scan kernel's layout, then the convolution's last taps - 1 inputs) is float32,
zeroed at admission and carried from step to step, so a prompt may come in portions of any size.  The recurrence
runs on the scan kernel of the delta rule in its form with one decay per head for all rows of S and no correction
(keys B, queries C, values dt u); everything behind the projection is float32.  Tensors: ``in``, ``conv``,
``conv.b``, ``dt_bias``, ``A_log``, ``D``, ``norm``, ``o`` (``names``).
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence

import torch

from .. import ops
from .delta_rule import SCAN_MAX_ROWS, scan_lanes
from .registry import register
from .spec import CacheSpec, ParamSpec, StateSpec


@register("mixer", "state_space")
class StateSpace:
    graph_safe = True
    NAMES = ("in", "conv", "conv.b", "dt_bias", "A_log", "D", "norm", "o")

    def __init__(self, hidden_size: int, heads: int, head_dim: int, state: int, groups: int, conv_taps: int,
                 norm_groups: int, norm_eps: float, dtype: torch.dtype, device, names: Sequence[str] = NAMES):
        if heads % groups:
            raise ValueError(f"{heads} heads cannot share {groups} groups")
        if (heads * head_dim) % norm_groups:
            raise ValueError(f"a row of {heads * head_dim} cannot be normed in {norm_groups} equal parts")
        if conv_taps < 1:
            raise ValueError(f"a convolution of {conv_taps} taps")
        if -(-state // scan_lanes(state)) > SCAN_MAX_ROWS:
            raise ValueError(f"a state of {state} rows is wider than the scan kernel takes ({32 * SCAN_MAX_ROWS})")
        self.hidden, self.heads, self.p, self.n, self.groups = hidden_size, heads, head_dim, state, groups
        self.taps, self.norm_groups, self.norm_eps = conv_taps, norm_groups, float(norm_eps)
        self.dtype, self.device, self.names = dtype, device, tuple(names)
        self.inner = heads * head_dim
        self.channels = self.inner + 2 * groups * state
        self._checked = False

    @classmethod
    def param_specs(cls, hidden_size, heads, head_dim, state, groups, conv_taps, names=NAMES, **_) -> Dict[str, ParamSpec]:
        w_in, conv, conv_b, dt_bias, a_log, d, norm, o = names
        inner = heads * head_dim
        channels = inner + 2 * groups * state
        return {w_in: ParamSpec((inner + channels + heads, hidden_size)),
                conv: ParamSpec((channels, conv_taps), "unit"), conv_b: ParamSpec((channels,), "unit"),
                dt_bias: ParamSpec((heads,), "unit"), a_log: ParamSpec((heads,), "unit"), d: ParamSpec((heads,), "unit"),
                norm: ParamSpec((inner,), "norm"), o: ParamSpec((hidden_size, inner))}

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        w_in, conv, conv_b, dt_bias, a_log, d, norm, o = self.names
        w = t[w_in]
        pad = torch.zeros((-w.shape[0] % 8, self.hidden), dtype=w.dtype, device=w.device)
        self.w_in = torch.cat([w, pad], dim=0).contiguous()
        self.conv_w = t[conv].to(self.dtype).contiguous()
        self.conv_t = self.conv_w.t().contiguous()                  # [taps, channels]: eight channels per access
        self.conv_b = t[conv_b].to(torch.float32).contiguous()
        self.dt_bias = t[dt_bias].to(torch.float32).contiguous()
        self.rate = torch.exp(t[a_log].to(torch.float32)).contiguous()       # the decay is exp(-rate dt)
        self.skip = t[d].to(torch.float32).contiguous()
        self.out_weight = t[norm].to(torch.float32).contiguous()
        self.w_o = t[o].contiguous()

    def cache_spec(self) -> Optional[CacheSpec]:
        return None

    def state_spec(self) -> Optional[StateSpec]:
        lanes = scan_lanes(self.n)
        per = -(-self.n // lanes) * lanes
        return StateSpec((self.heads * per * self.p + (self.taps - 1) * self.channels,), "float32")

    def workspace_floats(self, tokens: int) -> int:
        return tokens * (2 * self.inner + self.channels + 2 * self.heads + 3 * self.inner + 2 * self.groups * self.n)

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        if not self._checked:
            want = ops.state_space_state_floats(self.heads, self.groups, self.n, self.p, self.taps)
            if want != cache.state.shape[1]:
                raise ValueError(f"the scan kernel wants a state of {want} floats, the slots have {cache.state.shape[1]}")
            self._checked = True
        proj = ops.linear(x, self.w_in, out_dtype=self.dtype)
        y = ops.state_space(proj, self.conv_w, self.conv_b, self.taps, self.dt_bias, self.rate, self.skip,
                            self.out_weight, self.norm_eps, self.norm_groups, ctx.token_slot, ctx.seg_info,
                            cache.state, self.heads, self.groups, self.n, self.p, self.dtype, conv_t=self.conv_t)
        return ops.linear(y, self.w_o, out_dtype=self.dtype)
