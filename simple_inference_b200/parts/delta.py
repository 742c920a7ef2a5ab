"""Generalised delta rule: a mixer with a matrix state per head.

Per token and head (key channel c, value channel d, both of ``head_dim``):

    decay_c = exp(-exp(-1/2) * sigmoid(w0 + W2 tanh(W1 x))_c)      per-channel forgetting
    rate_c  = sigmoid(Wa x + ba)_c                                 per-channel removal rate
    u       = k / sqrt(sum_c k_c^2 + 1e-6)                         the unit key
    S      <- diag(decay) S - (rate * u)(u^T S) + k v^T            both terms read the old S
    o       = S^T r

then each head's ``o`` is divided by its root mean square, the heads together are scaled by a
gain, gated by ``sigmoid(Wg x)`` and projected by ``Wo``.  The state starts at zero, is
float32, and lives in the request's state slot from step to step; the scan runs in token
order, so a request's outputs do not depend on how its tokens were cut into steps.

The six projections of x are one matrix product ``[r | k | v | g | a | low]``; everything
after it is float32 (``csrc/delta_rule.cu``).  The constants ``exp(-1/2)`` and ``1e-6`` are
fixed by the rule; sizes (heads, head size, inner width of the decay projection) and the
norm's epsilon are parameters.
"""

from __future__ import annotations

import torch

from .. import ops
from .base import LayerCache, Mixer, Runtime, StateSpec, TensorSpec
from .registry import register_mixer


@register_mixer("general_delta")
class GeneralDelta(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, decay_rank: int,
                 norm_eps: float = 1e-6):
        if head_dim > 256:
            raise ValueError(f"head_dim {head_dim}: the recurrence kernel keeps up to 256 key "
                             f"channels of a state column in registers")
        self.hidden_size = int(hidden_size)
        self.num_heads = int(num_heads)
        self.head_dim = int(head_dim)
        self.rank = int(decay_rank)
        self.eps = float(norm_eps)
        self.width = self.num_heads * self.head_dim

    def tensors(self) -> dict[str, TensorSpec]:
        w, h = self.width, self.hidden_size
        out = {name: TensorSpec((w, h)) for name in ("r", "k", "v", "g", "a")}
        out["w1"] = TensorSpec((self.rank, h))
        out["w2"] = TensorSpec((w, self.rank))
        out["w0"] = TensorSpec((w,), kind="vector", init="zeros")
        out["a_bias"] = TensorSpec((w,), kind="vector", init="zeros")
        out["norm"] = TensorSpec((w,), kind="vector", init="gain")
        out["o"] = TensorSpec((h, w))
        return out

    def cache_spec(self) -> StateSpec:
        return StateSpec((self.num_heads, self.head_dim, self.head_dim), "float32")

    def bind(self, tensors: dict[str, torch.Tensor], rt: Runtime) -> None:
        super().bind(tensors, rt)
        self.w_proj = torch.cat([tensors[n] for n in ("r", "k", "v", "g", "a", "w1")],
                                dim=0).contiguous()
        self.w2t = tensors["w2"].t().contiguous()   # [rank, width]: channels side by side
        self.w0 = tensors["w0"].float().contiguous()
        self.a_bias = tensors["a_bias"].float().contiguous()
        self.gain = tensors["norm"].contiguous()
        self.w_o = tensors["o"]

    def forward(self, x: torch.Tensor, ctx, cache: LayerCache) -> torch.Tensor:
        n = x.shape[0]
        proj = ctx.ws.get("delta.proj", (n, 5 * self.width + self.rank), x.dtype)
        ops.linear(x, self.w_proj, proj)
        prep = ctx.ws.get("delta.prep", (n, 6 * self.width), torch.float32)
        ops.delta_prepare(proj, self.w2t, self.w0, self.a_bias, prep, self.num_heads, self.head_dim,
                          self.rank)
        o = ctx.ws.get("delta.o", (n, self.width), torch.float32)
        ops.delta_recurrence(prep, ctx.cu_q, ctx.seq_slots, cache.state, o, ctx.n_seqs,
                             self.num_heads, self.head_dim)
        mixed = ctx.ws.get("delta.mixed", (n, self.width), x.dtype)
        ops.delta_output(o, proj, self.gain, mixed, self.num_heads, self.head_dim, self.eps)
        return ops.linear_for_residual(mixed, self.w_o, ctx.ws, "delta.out",
                                       getattr(ctx, "partial_sums_ok", False))
