"""Mixture of experts as a feed-forward part: a router chooses ``top`` of ``experts`` small gated
feed-forward units per token, an optional shared unit runs for every token, and the results are summed.

  z = Wr x in float32; score s = sigmoid(z) (``router_scores='sigmoid'``) or the softmax of the chosen
  experts' logits (``'softmax'``); the experts with the largest z are chosen, lowest index on ties
  expert e: Wd_e (act(Wg_e u) * (Wu_e u)); with ``weight_on='input'`` u = s_e x and the outputs are
  summed as they are, with ``'output'`` u = x and the outputs are weighted by s_e
  out = sum over the chosen experts + shared(x)

Options that other routers use, each a parameter:

  ``gated=False``        an expert is Wd_e act(Wu_e u), two matrices (``names`` = up, down) and any elementwise activation
  ``router_scores='softmax_all'``  s = softmax(z) over all experts, the weights are the chosen experts' s as they are
  ``correction``         a learned vector added to the scores for the choice only (tensor ``correction_name``)
  ``groups=(count, keep)``  experts form ``count`` equal groups of neighbours; only experts of the ``keep`` groups whose
                         best member's choice score is largest can be chosen
  ``identity``           the router's last ``identity`` outputs are experts without matrices whose output is their
                         input; they count as experts for the scores, the groups and the choice

The step's rows are sorted by expert on the device (``ops.MoePlan``); the experts' gate|up product
gathers its rows from the tokens and applies the activation in its epilogue, the down product leaves
rows that one kernel sums per token, in float32, with the shared unit's output.  Steps with many rows run
both products on the grouped tcgen05 kernel (row tiles of 128 per expert), steps with few on mma.sync
tiles of 64 rows that read the chosen experts' weights once.  Nothing is read by the host,
so steps with this part are captured as CUDA graphs like the others.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import ops
from .registry import lookup, register
from .spec import ParamSpec, PartSpec


@register("feed_forward", "moe")
class MixtureOfExperts:
    graph_safe = True

    def __init__(self, hidden_size: int, experts: int, top: int, expert_size: int, dtype: torch.dtype, device,
                 activation: str = "silu", router_scores: str = "sigmoid", weight_on: str = "input",
                 shared: Optional[PartSpec] = None, router_name: str = "router", expert_prefix: str = "e",
                 names=("gate", "up", "down"), gated: bool = True, correction: bool = False,
                 correction_name: str = "correction", groups=None, identity: int = 0):
        if not 0 < top <= experts + identity:
            raise ValueError(f"top {top} of {experts} experts")
        if router_scores not in ("sigmoid", "softmax", "softmax_all") or weight_on not in ("input", "output"):
            raise ValueError(f"router_scores {router_scores!r} / weight_on {weight_on!r}")
        known = ops.ACTIVATIONS if gated else ops.ELEMENTWISE_ACTIVATIONS
        if activation not in known:
            raise ValueError(f"activation {activation!r} is not one of {sorted(known)}")
        self.gated, self.correction, self.correction_name = bool(gated), bool(correction), correction_name
        self.identity = int(identity)
        self.groups = (1, 1) if groups is None else (int(groups[0]), int(groups[1]))
        count, keep = self.groups
        total = experts + self.identity
        if self.identity < 0 or count <= 0 or total % count or not 0 < keep <= count or keep * (total // count) < top:
            raise ValueError(f"{count} groups (keep {keep}) over {experts} + {self.identity} experts, top {top}")
        # the kernel that scores all experts serves every router that needs more than the largest logits
        self.full_router = router_scores == "softmax_all" or self.correction or count > 1 or self.identity > 0
        if self.full_router and router_scores == "softmax":
            raise ValueError("a softmax over the chosen experts has no correction, groups or identity experts")
        if self.identity and weight_on == "input":
            raise ValueError("identity experts weigh their output")
        if len(names) != (3 if gated else 2):
            raise ValueError(f"{'gated' if gated else 'plain'} experts have {3 if gated else 2} matrices, got names {names}")
        self.w_correction = None
        self.hidden, self.experts, self.top, self.inter = hidden_size, experts, top, expert_size
        self.dtype, self.device, self.activation = dtype, device, activation
        self.router_scores, self.weight_on = router_scores, weight_on
        self.router_name, self.expert_prefix, self.names = router_name, expert_prefix, tuple(names)
        self.shared_spec = shared
        self.shared = None
        if shared is not None:
            self.shared = lookup("feed_forward", shared.kind)(dtype=dtype, device=device, **shared.params)
        self.w_router = self.w_gate_up = self.w_down = None

    @classmethod
    def param_specs(cls, hidden_size, experts, top, expert_size, shared: Optional[PartSpec] = None,
                    router_name: str = "router", expert_prefix: str = "e", names=("gate", "up", "down"),
                    gated: bool = True, correction: bool = False, correction_name: str = "correction", identity: int = 0,
                    **_) -> Dict[str, ParamSpec]:
        specs = {router_name: ParamSpec((experts + identity, hidden_size))}
        if correction:
            specs[correction_name] = ParamSpec((experts + identity,), "small")
        for e in range(experts):
            p = f"{expert_prefix}{e}."
            for name in names[:-1]:
                specs[p + name] = ParamSpec((expert_size, hidden_size))
            specs[p + names[-1]] = ParamSpec((hidden_size, expert_size))
        if shared is not None:
            for k, v in lookup("feed_forward", shared.kind).param_specs(**shared.params).items():
                specs[shared.prefix + k] = v
        return specs

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        self.w_router = t[self.router_name].contiguous()
        if self.correction:
            self.w_correction = t[self.correction_name].to(torch.float32).contiguous()
        if self.shared is not None:
            n = len(self.shared_spec.prefix)
            self.shared.load({k[n:]: v for k, v in t.items() if k.startswith(self.shared_spec.prefix)})
        down = self.names[-1]
        self.w_down = torch.stack([t[f"{self.expert_prefix}{e}.{down}"] for e in range(self.experts)]).contiguous()
        if not self.gated:
            self.interleaved = False
            self.w_up = torch.stack([t[f"{self.expert_prefix}{e}.{self.names[0]}"] for e in range(self.experts)]).contiguous()
            return
        gate, up, down = self.names
        # gate and up of an expert as one matrix, their rows interleaved by eight where the width allows
        # (the layout whose products apply the activation in their epilogue), else stacked
        self.interleaved = self.inter % 8 == 0
        stacks = []
        for e in range(self.experts):
            p = f"{self.expert_prefix}{e}."
            if self.interleaved:
                stacks.append(ops.interleave_gate_up(t[p + gate], t[p + up]))
            else:
                stacks.append(torch.cat([t[p + gate], t[p + up]], dim=0))
        self.w_gate_up = torch.stack(stacks).contiguous()                       # [E, 2 I, H]

    def workspace_floats(self, tokens: int) -> int:
        own = tokens * self.top * (self.inter + self.hidden) + tokens * self.experts
        shared = int(self.shared.workspace_floats(tokens)) if hasattr(self.shared, "workspace_floats") else 0
        return own + shared

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        z = ops.linear(x, self.w_router, out_dtype=torch.float32)
        if self.full_router:
            ids, weights = ops.moe_route_grouped(z, self.top, "sigmoid" if self.router_scores == "sigmoid" else "softmax",
                                                 self.w_correction, *self.groups)
        else:
            ids, weights = ops.moe_route(z, self.top, softmax_weights=self.router_scores == "softmax")
        rows = ids.numel()
        w_first = self.w_gate_up if self.gated else self.w_up
        tensor_cores = (self.interleaved or not self.gated) and x.dtype == w_first.dtype \
            and ops.moe_tcgen05_pays(rows, self.experts, self.inter, self.hidden, x.dtype)
        plan = ops.MoePlan(ids, self.experts + self.identity, ops.MOE_TCGEN05_TILE if tensor_cores else None,
                           real=self.experts)
        on_input = self.weight_on == "input"
        act = ops.moe_grouped(x, w_first, plan, self.top, gated=self.gated, gather=True,
                              weights=weights if on_input else None, act=self.activation,
                              interleaved=self.interleaved, unary=not self.gated)
        y = ops.moe_grouped(act, self.w_down, plan, self.top, gated=False, gather=False)
        shared = self.shared.forward(x, ctx) if self.shared is not None else None
        return ops.moe_combine(y, plan, self.top, shared, self.dtype, weights=None if on_input else weights,
                               identity_input=x if self.identity else None)
