"""Grouped-query attention over a sliding window, with pooled blocks before the window.

A query at position i sees the tokens j with ``0 <= i - j < window`` and, for every block of
``pool`` positions that lies wholly before the window (``b*pool + pool - 1 <= i - window``),
one key and one value: the means of the block's keys and values as the cache holds them.
Tokens that left the window while their block is not yet complete-and-passed are not seen.
Tokens and blocks share one softmax of ``scale * q.k``.

Other constants of the kind, all parameters: keys and values of different head sizes
(``key_dim``, ``value_dim``); an RMS norm with a gain over the WHOLE query projection and
over the whole key projection (all heads at once) before rotation; rotary positions on the
first ``rotary.dims`` dimensions of each query and key head (halves layout, optional YaRN
scaling, ``parts/rope.py``); optionally rotated values: the value of position j is turned
by j over all of ``value_dim`` with the plain frequencies of the same base, cached so, and a
head's output at position i is turned back by -i.  Without ``window`` every earlier token is
seen and nothing is pooled.

Memory (``cache_spec``): a composite of two paged planes caches.  The *token cache* has a
row per token and a window of ``max(window, pool)`` tokens (a block's row is made when its
last token arrives, from the rows of its tokens), so its pages return to the pool as the
window passes them.  The *block cache* has a row per ``pool`` tokens and keeps them all.
"""

from __future__ import annotations

import torch

from .. import ops
from .base import (CompositeSpec, KeyValuePlanesSpec, LayerCache, Mixer, Runtime, TensorSpec)
from .registry import register_mixer
from .rope import yarn_frequencies

BLOCK_ROWS_PER_PAGE = 16   # pooled blocks on one page of the block cache


@register_mixer("pooled_window_attention")
class PooledWindowAttention(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, key_dim: int,
                 value_dim: int, scale: float, window: int | None = None, pool: int | None = None,
                 rotary: dict | None = None, rotate_values: bool = False,
                 qk_norm_eps: float = 1e-6):
        if num_heads % num_kv_heads != 0:
            raise ValueError(f"{num_heads} query heads do not divide into {num_kv_heads} groups")
        if pool and not window:
            raise ValueError("pooled blocks need a window to lie before")
        if rotate_values and (rotary is None or value_dim % 2 != 0):
            raise ValueError("rotated values need a rotary base and an even value size")
        if value_dim > 256:
            raise ValueError(f"value_dim {value_dim}: the attention kernel takes up to 256")
        self.hidden_size = int(hidden_size)
        self.num_heads = int(num_heads)
        self.num_kv_heads = int(num_kv_heads)
        self.key_dim = int(key_dim)
        self.value_dim = int(value_dim)
        self.scale = float(scale)
        self.window = int(window) if window else None
        self.pool = int(pool) if pool else None
        self.rotary = dict(rotary) if rotary else None
        self.rotate_values = bool(rotate_values)
        self.eps = float(qk_norm_eps)
        self.rot_dims = int(self.rotary["dims"]) if self.rotary else 0
        if self.rot_dims > self.key_dim or self.rot_dims % 2 != 0:
            raise ValueError(f"rotary dims {self.rot_dims} must be even and at most {self.key_dim}")
        self.q_width = self.num_heads * self.key_dim
        self.k_width = self.num_kv_heads * self.key_dim
        self.v_width = self.num_kv_heads * self.value_dim
        self.out_width = self.num_heads * self.value_dim

    def tensors(self) -> dict[str, TensorSpec]:
        return {
            "wq": TensorSpec((self.q_width, self.hidden_size)),
            "wk": TensorSpec((self.k_width, self.hidden_size)),
            "wv": TensorSpec((self.v_width, self.hidden_size)),
            "wo": TensorSpec((self.hidden_size, self.out_width)),
            "q_norm": TensorSpec((self.q_width,), kind="vector", init="gain"),
            "k_norm": TensorSpec((self.k_width,), kind="vector", init="gain"),
        }

    def cache_spec(self):
        keep = None if self.window is None else max(self.window, self.pool or 0)
        tokens = KeyValuePlanesSpec(self.num_kv_heads, self.key_dim, self.value_dim, window=keep)
        if self.pool is None:
            return tokens
        blocks = KeyValuePlanesSpec(self.num_kv_heads, self.key_dim, self.value_dim, window=None,
                                    page_size=self.pool * BLOCK_ROWS_PER_PAGE,
                                    tokens_per_row=self.pool)
        return CompositeSpec((tokens, blocks))

    def bind(self, tensors: dict[str, torch.Tensor], rt: Runtime) -> None:
        super().bind(tensors, rt)
        self.w_qkv = torch.cat([tensors["wq"], tensors["wk"], tensors["wv"]], dim=0).contiguous()
        self.w_o = tensors["wo"]
        self.q_gain = tensors["q_norm"].contiguous()
        self.k_gain = tensors["k_norm"].contiguous()
        self.freq_qk, self.amplitude, self.freq_v = None, 1.0, None
        if self.rotary:
            f, self.amplitude = yarn_frequencies(self.rot_dims, self.rotary["base"],
                                                 self.rotary.get("scaling"))
            self.freq_qk = f.to(rt.device)
            if self.rotate_values:
                self.freq_v = yarn_frequencies(self.value_dim, self.rotary["base"], None)[0].to(rt.device)

    def forward(self, x: torch.Tensor, ctx, cache: LayerCache) -> torch.Tensor:
        n = x.shape[0]
        tok, blk = (cache.members if cache.members is not None else (cache, None))
        qkv = ctx.ws.get("wpattn.qkv", (n, self.q_width + self.k_width + self.v_width), x.dtype)
        ops.linear(x, self.w_qkv, qkv)
        tok_rows = tok.spec.rows(tok.page_size)
        ops.window_pool_prepare(qkv, ctx.positions, self.q_gain, self.k_gain, self.freq_qk,
                                self.amplitude, self.rot_dims, self.freq_v, ctx.kv_slots[tok.group],
                                tok.pool, self.num_heads, self.num_kv_heads, self.key_dim,
                                self.value_dim, tok_rows, self.eps, cache.writes)
        tok_table = ctx.block_tables[tok.group]
        blk_rows, blk_table, blk_pool = 0, None, None
        if blk is not None:
            blk_rows, blk_table, blk_pool = blk.spec.rows(blk.page_size), ctx.block_tables[blk.group], blk.pool
            if cache.writes:
                ops.window_pool_summarise(ctx.positions, ctx.tok_seq, tok.pool, tok_table, tok_rows,
                                          blk_pool, blk_table, blk_rows, n, self.num_kv_heads,
                                          self.key_dim, self.value_dim, self.pool)
        mixed = ctx.ws.get("wpattn.mixed", (n, self.out_width), x.dtype)
        splits, scratch = 1, None
        if x.dtype == torch.bfloat16:   # a decode step has too few tiles for the GPU: share their keys out
            splits = ops.window_pool_key_splits(n, ctx.n_seqs, self.num_kv_heads, self.window, self.pool,
                                                ctx.max_kv_len)
            if splits > 1:
                most = ops.window_pool_scratch_rows(ops.WINDOW_POOL_SPLIT_MAX_TOKENS,
                                                    ops.WINDOW_POOL_SPLIT_MAX_TOKENS, self.num_kv_heads,
                                                    ops.WINDOW_POOL_MAX_SPLITS)
                scratch = ctx.ws.get("wpattn.parts", (most, self.value_dim + 2), torch.float32,
                                     row_cap=most)
        ops.window_pool_attention(qkv, ctx.positions, ctx.tok_seq, tok.pool, tok_table, tok_rows,
                                  blk_pool, blk_table, blk_rows, mixed, self.num_heads,
                                  self.num_kv_heads, self.key_dim, self.value_dim, self.scale,
                                  self.window, self.pool, self.freq_v, ctx.cu_q, ctx.n_seqs, splits,
                                  scratch)
        return ops.linear_for_residual(mixed, self.w_o, ctx.ws, "wpattn.proj",
                                       getattr(ctx, "partial_sums_ok", False))
