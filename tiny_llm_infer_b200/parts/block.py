"""Arrangements of parts in a layer.

``prenorm``: h += pending; a = mixer(norm1(h)); h += a; m = ffn(norm2(h)); pending = m.
This is the reference's decoder layer (model/src/qwen3_paged_batch.cpp:146-301) with the
two residual sums moved into the norm that follows them; the sum left over after the
last layer is taken by the model's final norm.

``sandwich``: a norm before and after each sub-layer, h += norm1b(mixer(norm1(h))), then
h += norm2b(ffn(norm2(h))).  The output norms are not run on their own: the sub-layer's output goes
on as a ``NormedDelta`` and the next norm kernel (this layer's norm2, the next layer's norm1, or
the model's last norm) norms it, adds it and norms the sum.  ``sandwich_mixer`` is the same layer
without a feed-forward.

``stream_*``: the sub-layers read the residual stream itself, and only their outputs are normed:
h += norm1(mixer(h)), then h += norm2(ffn(h)), then h += norm3(side(h)), where the feed-forward and the
side input (a feed-forward that also looks at the step's tokens) are each there or not: ``stream_mixer``,
``stream_mixer_ffn``, ``stream_mixer_side``, ``stream_mixer_ffn_side``.  Every sum is one kernel that norms the
output, adds it in float32 and hands the stream on in the storage type; the last output goes on as a
``NormedDelta`` like the sandwich's.

``parallel_*``: one norm, and every sub-layer reads its output: with x = norm1(h),
h += m * (ls1 * sum_i c_i mixer_i(x) + ls2 * ffn(x)), where ls1 and ls2 are learned vectors (``column_scale``
parts), the c_i weigh the mixers and m is the residual multiplier.  One mixer (``parallel_mixer``,
``parallel_mixer_ffn``) or two side by side (``parallel_pair``, ``parallel_pair_ffn``, roles ``left`` and
``right``, each with a cache of its own).  The outputs go on as ``ScaledDeltas``: the norm kernel that follows
multiplies, adds in float32 and norms in one pass.

``postnorm_*``: the norm comes after the sum and its result is the stream: h <- norm1(alpha h + sum_i c_i mixer_i(h)),
then, where the layer has a feed-forward, h <- norm2(alpha h + ffn(h)); the sub-layers read the stream itself.  One
mixer (``postnorm_mixer``, ``postnorm_mixer_ffn``) or two side by side with weights c_i (``postnorm_pair``,
``postnorm_pair_ffn``, roles ``left`` and ``right``).  Every sum with its norm is one kernel (``RMSNorm.of_sum``),
which also leaves the stream in the storage type; it travels from block to block as a ``StreamCopy``.  A mixer
that says ``deferred_bias`` (a bias of its output product that it has not added) gets it added in that kernel.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import ops
from .norm import NormedDelta, ScaledDeltas, StreamCopy
from .registry import register


class Block:
    """Base of the arrangements.  A block class declares ``roles``: the names of the parts it
    arranges and, for each, the registry it is chosen from (``norm``, ``mixer``,
    ``feed_forward``); any number of each.  The model builds the parts a layer's description
    gives for these names and hands them over; they become attributes under their role names.
    ``forward(h, pending, ctx, cache)``: ``cache`` is the ``LayerCacheView`` of the block's mixer,
    or, for a block with several mixers, the list of their views in the order of ``roles``."""
    roles: Dict[str, str] = {}

    def __init__(self, parts: Dict[str, object]):
        self.parts = {role: parts[role] for role in self.roles}
        for role, part in self.parts.items():
            setattr(self, role, part)

    def mixers(self) -> List[object]:
        """The block's mixers in the order of ``roles`` (the cache manager and the run order give
        each a cache of its own)."""
        return [self.parts[role] for role, category in self.roles.items() if category == "mixer"]


@register("block", "prenorm")
class PreNormBlock(Block):
    roles = {"norm1": "norm", "mixer": "mixer", "norm2": "norm", "ffn": "feed_forward"}

    def forward(self, h: torch.Tensor, pending: Optional[torch.Tensor], ctx, cache) -> torch.Tensor:
        x = self.norm1.forward(h, pending)
        a = self.mixer.forward(x, ctx, cache)
        x = self.norm2.forward(h, a)
        return self.ffn.forward(x, ctx)


@register("block", "sandwich")
class SandwichBlock(Block):
    roles = {"norm1": "norm", "mixer": "mixer", "norm1b": "norm",
             "norm2": "norm", "ffn": "feed_forward", "norm2b": "norm"}

    def forward(self, h: torch.Tensor, pending, ctx, cache):
        x = self.norm1.forward(h, pending)
        a = self.mixer.forward(x, ctx, cache)
        x = self.norm2.forward(h, self.norm1b.wrap(a))
        return self.norm2b.wrap(self.ffn.forward(x, ctx))


@register("block", "sandwich_mixer")
class SandwichMixerBlock(Block):
    roles = {"norm1": "norm", "mixer": "mixer", "norm1b": "norm"}

    def forward(self, h: torch.Tensor, pending, ctx, cache):
        x = self.norm1.forward(h, pending)
        return self.norm1b.wrap(self.mixer.forward(x, ctx, cache))


def _stream(h: torch.Tensor, pending, dtype: torch.dtype) -> torch.Tensor:
    """h += pending (normed first if it is a ``NormedDelta``); the stream in the storage type."""
    if isinstance(pending, StreamCopy):
        return pending.x
    out = torch.empty(h.shape, dtype=dtype, device=h.device)
    if isinstance(pending, NormedDelta):
        return ops.stream_add(h, pending.delta, out, post_gain=pending.gain, post_eps=pending.eps)
    return ops.stream_add(h, pending, out)


def _stream_block(name: str, with_ffn: bool, with_side: bool) -> type:
    roles = {"mixer": "mixer", "norm1": "norm"}
    if with_ffn:
        roles.update({"ffn": "feed_forward", "norm2": "norm"})
    if with_side:
        roles.update({"side": "feed_forward", "norm3": "norm"})

    class StreamBlock(Block):
        def forward(self, h: torch.Tensor, pending, ctx, cache):
            dtype = self.norm1.dtype
            pending = self.norm1.wrap(self.mixer.forward(_stream(h, pending, dtype), ctx, cache))
            if with_ffn:
                pending = self.norm2.wrap(self.ffn.forward(_stream(h, pending, dtype), ctx))
            if with_side:
                pending = self.norm3.wrap(self.side.forward(_stream(h, pending, dtype), ctx))
            return pending

    StreamBlock.roles = roles
    StreamBlock.__name__ = StreamBlock.__qualname__ = "".join(w.title() for w in name.split("_")) + "Block"
    return register("block", name)(StreamBlock)


for _ffn in (False, True):
    for _side in (False, True):
        _stream_block("stream_mixer" + ("_ffn" if _ffn else "") + ("_side" if _side else ""), _ffn, _side)


def _parallel_block(name: str, mixer_roles, with_ffn: bool) -> type:
    roles = {"norm1": "norm"}
    roles.update({role: "mixer" for role in mixer_roles})
    roles["ls1"] = "norm"
    if with_ffn:
        roles.update({"ffn": "feed_forward", "ls2": "norm"})

    class ParallelBlock(Block):
        def __init__(self, parts: Dict[str, object], residual_mult: float = 1.0, mixer_weights=None):
            super().__init__(parts)
            self.residual_mult = float(residual_mult)
            self.mixer_weights = [1.0] * len(mixer_roles) if mixer_weights is None else [float(w) for w in mixer_weights]
            if len(self.mixer_weights) != len(mixer_roles):
                raise ValueError(f"{len(self.mixer_weights)} weights for {len(mixer_roles)} mixers")
            self._scales: Optional[List[torch.Tensor]] = None

        def scales(self) -> List[torch.Tensor]:
            """Per output the float32 vector it is multiplied by before the sum (made once, after the load)."""
            if self._scales is None:
                out = [self.ls1.scale * (self.residual_mult * w) for w in self.mixer_weights]
                if with_ffn:
                    out.append(self.ls2.scale * self.residual_mult)
                self._scales = [v.contiguous() for v in out]
            return self._scales

        def forward(self, h: torch.Tensor, pending, ctx, cache):
            x = self.norm1.forward(h, pending)
            views = cache if isinstance(cache, (list, tuple)) else [cache]
            deltas = [mixer.forward(x, ctx, view) for mixer, view in zip(self.mixers(), views)]
            if with_ffn:
                deltas.append(self.ffn.forward(x, ctx))
            return ScaledDeltas(deltas, self.scales())

    ParallelBlock.roles = roles
    ParallelBlock.__name__ = ParallelBlock.__qualname__ = "".join(w.title() for w in name.split("_")) + "Block"
    return register("block", name)(ParallelBlock)


for _roles, _name in ((("mixer",), "parallel_mixer"), (("left", "right"), "parallel_pair")):
    for _ffn in (False, True):
        _parallel_block(_name + ("_ffn" if _ffn else ""), _roles, _ffn)


def _postnorm_block(name: str, mixer_roles, with_ffn: bool) -> type:
    roles = {role: "mixer" for role in mixer_roles}
    roles["norm1"] = "norm"
    if with_ffn:
        roles.update({"ffn": "feed_forward", "norm2": "norm"})

    class PostNormBlock(Block):
        def __init__(self, parts: Dict[str, object], alpha: float = 1.0, mixer_weights=None):
            super().__init__(parts)
            self.alpha = float(alpha)
            self.mixer_weights = [1.0] * len(mixer_roles) if mixer_weights is None else [float(w) for w in mixer_weights]
            if len(self.mixer_weights) != len(mixer_roles):
                raise ValueError(f"{len(self.mixer_weights)} weights for {len(mixer_roles)} mixers")
            self._bias: Optional[torch.Tensor] = None
            self._bias_made = False

        def mixer_bias(self) -> Optional[torch.Tensor]:
            """The weighted sum of the biases that the mixers left to the norm's kernel (made once, after the load)."""
            if not self._bias_made:
                for mixer, w in zip(self.mixers(), self.mixer_weights):
                    b = getattr(mixer, "deferred_bias", None)
                    if b is not None:
                        self._bias = b.to(torch.float32) * w if self._bias is None else self._bias + b.to(torch.float32) * w
                if self._bias is not None:
                    self._bias = self._bias.contiguous()
                self._bias_made = True
            return self._bias

        def forward(self, h: torch.Tensor, pending, ctx, cache):
            if isinstance(pending, StreamCopy):
                x = pending.x
            else:                                   # the first block of a model, or one behind a block of another kind
                x = _stream(h, pending, self.norm1.dtype)
            views = cache if isinstance(cache, (list, tuple)) else [cache]
            deltas = [mixer.forward(x, ctx, view) for mixer, view in zip(self.mixers(), views)]
            x = self.norm1.of_sum(h, self.alpha, deltas, self.mixer_weights, bias=self.mixer_bias())
            if with_ffn:
                x = self.norm2.of_sum(h, self.alpha, [self.ffn.forward(x, ctx)], [1.0])
            return StreamCopy(x)

    PostNormBlock.roles = roles
    PostNormBlock.__name__ = PostNormBlock.__qualname__ = "".join(w.title() for w in name.split("_")) + "Block"
    return register("block", name)(PostNormBlock)


for _roles, _name in ((("mixer",), "postnorm_mixer"), (("left", "right"), "postnorm_pair")):
    for _ffn in (False, True):
        _postnorm_block(_name + ("_ffn" if _ffn else ""), _roles, _ffn)
