"""RMSNorm, fused with the residual sum that precedes it.

x = gain * v / sqrt(mean(v^2) + eps) with eps inside the root and the gain multiplying
directly, no "1 + gain" (reference: kernels/src/rmsnorm_kernel_cuda.cu:17-38).  The
reference adds the residual in a separate half-precision kernel
(model/src/qwen3_paged_batch.cpp:273-279); here the sum is float32 and happens in the
same pass that computes the norm.

``offset``: the checkpoint stores the gain minus this number (a weight "around zero" has offset 1); the
sum gain = offset + stored weight is made once at load, in float32, and kept in float32.  ``float32_gain``
keeps a plain gain in float32 too (a model whose other norms do, so that one kernel sees one gain type).

A block that norms a sub-layer's output before the residual sum hands that output on as a
``NormedDelta`` (``wrap``): the norm that follows takes it as its ``delta`` and does the output's norm,
the sum and its own norm in one kernel, h += g_post * d / sqrt(mean(d^2) + eps_post) in float32.

A block that norms after the sum (``of_sum``) makes the norm's result the stream itself:
h <- gain * v / sqrt(mean(v^2) + eps) with v = alpha h + sum_i c_i d_i (+ a bias), in one kernel that also leaves
the new stream in the storage type for the next sub-layer; between such blocks the stream travels as a
``StreamCopy`` (nothing is left to add).
"""
from __future__ import annotations

from dataclasses import dataclass

from typing import Dict, List, Optional

import torch

from .. import ops
from .registry import register
from .spec import ParamSpec


@dataclass
class NormedDelta:
    """A sub-layer's output that is to be normed (gain, eps) before it is added to the stream."""
    delta: torch.Tensor
    gain: torch.Tensor
    eps: float


@dataclass
class StreamCopy:
    """The stream as it stands, in the storage type: what a block that norms after its sums hands on in place of
    an output still to be added."""
    x: torch.Tensor


@register("norm", "rmsnorm")
class RMSNorm:
    def __init__(self, width: int, eps: float, dtype: torch.dtype, device, name: str = "weight",
                 offset: float = 0.0, float32_gain: bool = False):
        self.width, self.eps, self.dtype, self.device = int(width), float(eps), dtype, device
        self.name, self.offset, self.float32_gain = name, float(offset), bool(float32_gain)
        self.gain: Optional[torch.Tensor] = None

    @classmethod
    def param_specs(cls, width: int, eps: float, name: str = "weight", offset: float = 0.0,
                    float32_gain: bool = False) -> Dict[str, ParamSpec]:
        """``name``: what the gain is called behind the part's prefix in the checkpoint."""
        return {name: ParamSpec((int(width),), "norm_zero" if offset else "norm")}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        gain = tensors[self.name]
        if self.offset or self.float32_gain:
            gain = gain.to(torch.float32) + self.offset
        self.gain = gain.contiguous()

    def wrap(self, delta: torch.Tensor) -> NormedDelta:
        """``delta`` with this norm still to be applied to it, by the norm that adds it to the stream."""
        return NormedDelta(delta, self.gain, self.eps)

    def of_sum(self, h: torch.Tensor, alpha: float, deltas, coefs, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        """h <- norm(alpha h + sum_i coefs[i] deltas[i] (+ bias)), written back as the stream; returns it in the
        storage type.  The gain must be float32 (``offset`` or ``float32_gain``)."""
        out = torch.empty((h.shape[0], self.width), dtype=self.dtype, device=h.device)
        return ops.sum_rmsnorm(h, list(deltas), list(coefs), alpha, self.gain, self.eps, out, bias=bias)

    def forward(self, h: torch.Tensor, delta, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        n = h.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.width), dtype=self.dtype, device=h.device)
        if isinstance(delta, StreamCopy):
            delta = None
        if isinstance(delta, NormedDelta):
            post = delta.gain if delta.gain.dtype == self.gain.dtype else delta.gain.to(self.gain.dtype)
            return ops.add_rmsnorm(h, delta.delta, self.gain, self.eps, out, rows, post_gain=post, post_eps=delta.eps)
        return ops.add_rmsnorm(h, delta, self.gain, self.eps, out, rows)


@dataclass
class ScaledDeltas:
    """Outputs of sub-layers that all read one norm's output, each still to be multiplied column by column by a
    float32 vector of its own (layer scale, mixing weight and residual multiplier folded into one) and added to
    the stream, by the norm that follows."""
    deltas: List[torch.Tensor]
    scales: List[torch.Tensor]


@register("norm", "layernorm")
class LayerNorm:
    """x = gain * (v - mean(v)) / sqrt(mean((v - mean(v))^2) + eps), no bias, fused with the residual sum that
    precedes it: ``delta`` is None, one output in the storage type (added as it is), or ``ScaledDeltas``.  The
    sum, the mean and the variance are float32."""

    def __init__(self, width: int, eps: float, dtype: torch.dtype, device, name: str = "weight"):
        self.width, self.eps, self.dtype, self.device, self.name = int(width), float(eps), dtype, device, name
        self.gain: Optional[torch.Tensor] = None
        self._ones: Optional[torch.Tensor] = None

    @classmethod
    def param_specs(cls, width: int, eps: float, name: str = "weight") -> Dict[str, ParamSpec]:
        return {name: ParamSpec((int(width),), "norm")}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.gain = tensors[self.name].contiguous()

    def forward(self, h: torch.Tensor, delta, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        n = h.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.width), dtype=self.dtype, device=h.device)
        if delta is None or isinstance(delta, StreamCopy):
            deltas, scales = [], []
        elif isinstance(delta, ScaledDeltas):
            deltas, scales = delta.deltas, delta.scales
        else:
            if self._ones is None:
                self._ones = torch.ones(self.width, dtype=torch.float32, device=h.device)
            deltas, scales = [delta], [self._ones]
        return ops.scaled_add_layernorm(h, deltas, scales, self.gain, self.eps, out, rows)


@register("norm", "column_scale")
class ColumnScale:
    """A learned vector that a sub-layer's output is multiplied by, column by column, before the residual sum
    (a layer scale).  It has no ``forward``: the block folds it, with its other constants, into the vector that
    the next norm's kernel applies (``ScaledDeltas``)."""

    def __init__(self, width: int, dtype: torch.dtype, device, name: str = "weight"):
        self.width, self.dtype, self.device, self.name = int(width), dtype, device, name
        self.scale: Optional[torch.Tensor] = None

    @classmethod
    def param_specs(cls, width: int, name: str = "weight") -> Dict[str, ParamSpec]:
        return {name: ParamSpec((int(width),), "norm")}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.scale = tensors[self.name].to(torch.float32).contiguous()
