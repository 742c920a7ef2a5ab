"""Arrangements of a mixer, a feed-forward and their norms.

``prenorm`` is the reference's block (``model/block.py:119-146``):
``h = x + Mixer(Norm_a(x)); out = h + FeedForward(Norm_b(h))``.  The residual
stream ``x`` is float32 and updated in place; each addition is done by the norm
that follows it, so a block hands its last sub-layer output on without adding it.
"""

from __future__ import annotations

import torch

from .base import Block, LayerCache, PartSpec, Runtime, TensorSpec
from .registry import FEED_FORWARDS, MIXERS, NORMS, register_block


@register_block("prenorm")
class PreNormBlock(Block):
    def __init__(self, mixer: PartSpec, mixer_norm: PartSpec, feed_forward: PartSpec,
                 feed_forward_norm: PartSpec):
        self.mixer_norm = NORMS.build(mixer_norm)
        self.mixer = MIXERS.build(mixer)
        self.feed_forward_norm = NORMS.build(feed_forward_norm)
        self.feed_forward = FEED_FORWARDS.build(feed_forward)

    def _children(self):
        return (("mixer_norm", self.mixer_norm), ("mixer", self.mixer),
                ("feed_forward_norm", self.feed_forward_norm), ("feed_forward", self.feed_forward))

    def tensors(self) -> dict[str, TensorSpec]:
        out: dict[str, TensorSpec] = {}
        for prefix, part in self._children():
            for name, spec in part.tensors().items():
                out[f"{prefix}.{name}"] = spec
        return out

    def bind(self, tensors: dict[str, torch.Tensor], rt: Runtime) -> None:
        super().bind(tensors, rt)
        for prefix, part in self._children():
            own = {k[len(prefix) + 1:]: v for k, v in tensors.items() if k.startswith(prefix + ".")}
            part.bind(own, rt)

    def first_norm(self):
        return self.mixer_norm

    def forward(self, residual, delta, ctx, cache: LayerCache | None):
        # ctx.partial_sums_ok tells a sub-layer whether the norm that will add its output takes
        # partial sums: for the mixer that is this block's second norm, for the feed-forward
        # whatever follows the block (the model said so in ctx.next_takes_partial_sums)
        after_block = getattr(ctx, "next_takes_partial_sums", False)
        h = self.mixer_norm.add_forward(residual, delta, ctx)
        ctx.partial_sums_ok = self.feed_forward_norm.takes_partial_sums
        mixed = self.mixer.forward(h, ctx, cache)
        h = self.feed_forward_norm.add_forward(residual, mixed, ctx)
        ctx.partial_sums_ok = after_block
        out = self.feed_forward.forward(h, ctx)
        ctx.partial_sums_ok = False
        return out


@register_block("postnorm")
class PostNormBlock(Block):
    """Norm after the sum: ``x <- N1(alpha x + Mixer(x))`` and, where the block has a
    feed-forward, ``x <- N2(alpha x + FeedForward(x))``.  The sub-layers read the stream itself.

    The stream stays float32; each update is one kernel that also leaves the new rows rounded
    to the activation dtype, which is what the next sub-layer's products read.  The block
    hands nothing on to be added (it returns None) and notes in ``ctx.stream_rounded`` where
    the rounded rows are, so that a post-norm block that follows need not round them again.
    ``mixer_norm`` and ``feed_forward_norm`` must be norms with ``weight`` and ``eps``
    (RMS norms); ``feed_forward`` may be None.
    """

    def __init__(self, mixer: PartSpec, mixer_norm: PartSpec, feed_forward: PartSpec | None = None,
                 feed_forward_norm: PartSpec | None = None, alpha: float = 1.0):
        if (feed_forward is None) != (feed_forward_norm is None):
            raise ValueError("a feed-forward and its norm come together")
        self.alpha = float(alpha)
        self.mixer = MIXERS.build(mixer)
        self.mixer_norm = NORMS.build(mixer_norm)
        self.feed_forward = FEED_FORWARDS.build(feed_forward) if feed_forward is not None else None
        self.feed_forward_norm = NORMS.build(feed_forward_norm) if feed_forward_norm is not None else None

    def _children(self):
        out = [("mixer_norm", self.mixer_norm), ("mixer", self.mixer)]
        if self.feed_forward is not None:
            out += [("feed_forward_norm", self.feed_forward_norm), ("feed_forward", self.feed_forward)]
        return out

    def tensors(self) -> dict[str, TensorSpec]:
        out: dict[str, TensorSpec] = {}
        for prefix, part in self._children():
            for name, spec in part.tensors().items():
                out[f"{prefix}.{name}"] = spec
        return out

    def bind(self, tensors: dict[str, torch.Tensor], rt: Runtime) -> None:
        super().bind(tensors, rt)
        for prefix, part in self._children():
            own = {k[len(prefix) + 1:]: v for k, v in tensors.items() if k.startswith(prefix + ".")}
            part.bind(own, rt)

    def first_norm(self):
        return None   # what the block before hands over is added as it is

    def forward(self, residual, delta, ctx, cache: LayerCache | None):
        from .. import ops
        n, width = residual.shape
        if isinstance(delta, ops.PartialSums):
            delta = delta.tensor()
        noted = getattr(ctx, "stream_rounded", None)
        if delta is None and noted is not None and noted[0] is residual:
            x = noted[1]
        else:
            x = ctx.ws.get("postnorm.stream", (n, width), self.rt.dtype)
            ops.residual_cast(residual, x, delta)
        # both of this block's sums are formed by a kernel that takes partial sums
        ctx.partial_sums_ok = True
        mixed = self.mixer.forward(x, ctx, cache)
        x = ctx.ws.get("postnorm.stream", (n, width), self.rt.dtype)
        ops.scaled_add_rmsnorm(residual, self.mixer_norm.weight, self.alpha, self.mixer_norm.eps,
                               x, mixed)
        if self.feed_forward is not None:
            out = self.feed_forward.forward(x, ctx)
            ops.scaled_add_rmsnorm(residual, self.feed_forward_norm.weight, self.alpha,
                                   self.feed_forward_norm.eps, x, out)
        ctx.partial_sums_ok = False
        ctx.stream_rounded = (residual, x)
        return None
