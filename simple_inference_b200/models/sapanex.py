"""``Sapanex``: a decoder whose layers are listed one by one in config.json.

Each layer is a post-norm block, ``x <- N1(alpha x + Mix(x))`` and then, where the layer has a
feed-forward, ``x <- N2(alpha x + FF(x))``; the mixer is either grouped-query attention over a
sliding window with pooled blocks before it (``pooled_window_attention``) or a generalised
delta rule with a matrix state per head (``general_delta``); the feed-forward is a squared-ReLU
pair of matrices.  The embedding is scaled, the output head is the embedding table itself.

This module only translates a ``SapanexConfig`` into a ``ModelPlan`` and names the
checkpoint's tensors (``l<i>.mix.*``, ``l<i>.mlp.*``, ``l<i>.norm1/2``, ``embed``,
``final.norm``).
"""

from __future__ import annotations

from ..config.registry import register_architecture
from ..config.sapanex_config import (AttentionMixerConfig, DeltaMixerConfig, SapanexConfig,
                                     SapanexLayer)
from ..parts.base import PartSpec
from .plan import LayerPlan, ModelPlan


def _attention(cfg: SapanexConfig, m: AttentionMixerConfig, p: str) -> tuple[PartSpec, dict]:
    rot = None
    if m.rot is not None:
        rot = {"dims": m.rot.dims, "base": m.rot.base,
               "scaling": m.rot.scaling.to_dict() if m.rot.scaling else None}
    spec = PartSpec("pooled_window_attention", {
        "hidden_size": cfg.width, "num_heads": m.heads, "num_kv_heads": m.kv_heads,
        "key_dim": m.dim, "value_dim": m.vdim, "scale": m.scale, "window": m.window,
        "pool": m.pool, "rotary": rot, "rotate_values": rot is not None,
        "qk_norm_eps": cfg.eps})
    names = {"wq": f"{p}.mix.q", "wk": f"{p}.mix.k", "wv": f"{p}.mix.v", "wo": f"{p}.mix.o",
             "q_norm": f"{p}.mix.q.norm", "k_norm": f"{p}.mix.k.norm"}
    return spec, names


def _delta(cfg: SapanexConfig, m: DeltaMixerConfig, p: str, low_rank: int) -> tuple[PartSpec, dict]:
    spec = PartSpec("general_delta", {"hidden_size": cfg.width, "num_heads": m.heads,
                                      "head_dim": m.dim, "decay_rank": low_rank,
                                      "norm_eps": cfg.eps})
    names = {k: f"{p}.mix.{k}" for k in ("r", "k", "v", "g", "a", "w1", "w2", "w0", "norm", "o")}
    names["a_bias"] = f"{p}.mix.a.b"
    return spec, names


def sapanex_layer_plan(cfg: SapanexConfig, index: int, layer: SapanexLayer,
                       decay_rank: int | None = None) -> LayerPlan:
    p = f"l{index}"
    if isinstance(layer.mixer, AttentionMixerConfig):
        mixer, names = _attention(cfg, layer.mixer, p)
    else:
        # the width of the decay's inner projection is given by the tensor's shape alone
        mixer, names = _delta(cfg, layer.mixer, p, decay_rank or layer.mixer.decay_rank
                              or default_decay_rank(cfg.width))
    names = {f"mixer.{k}": v for k, v in names.items()}
    norm = PartSpec("rmsnorm", {"hidden_size": cfg.width, "eps": cfg.eps})
    ffn = None
    names["mixer_norm.weight"] = f"{p}.norm1"
    if layer.mlp is not None:
        ffn = PartSpec("relu2", {"hidden_size": cfg.width, "intermediate_size": layer.mlp.ff})
        names["feed_forward.w_up"] = f"{p}.mlp.up"
        names["feed_forward.w_down"] = f"{p}.mlp.down"
        names["feed_forward_norm.weight"] = f"{p}.norm2"
    block = PartSpec("postnorm", {"mixer": mixer, "mixer_norm": norm, "feed_forward": ffn,
                                  "feed_forward_norm": norm if ffn is not None else None,
                                  "alpha": cfg.postln_alpha})
    return LayerPlan(block, names)


def default_decay_rank(width: int) -> int:
    """Inner width of the decay's two-matrix projection when no checkpoint says otherwise
    (random-weights mode): a sixteenth of the model's width, at least 8."""
    return max(8, width // 16)


def sapanex_plan(cfg: SapanexConfig, tensor_shapes: dict[str, tuple[int, ...]] | None = None) -> ModelPlan:
    """``tensor_shapes``: shapes found in a checkpoint; sizes that config.json leaves to the
    tensors (the decay projection's inner width) are read from there."""
    layers = []
    for i, layer in enumerate(cfg.layers):
        rank = None
        if tensor_shapes and f"l{i}.mix.w1" in tensor_shapes:
            rank = int(tensor_shapes[f"l{i}.mix.w1"][0])
        layers.append(sapanex_layer_plan(cfg, i, layer, rank))
    return ModelPlan(
        hidden_size=cfg.width,
        vocab_size=cfg.vocab,
        layers=layers,
        run_order=ModelPlan.sequential(len(layers)),
        final_norm=PartSpec("rmsnorm", {"hidden_size": cfg.width, "eps": cfg.eps}),
        tie_embeddings=True,
        embedding_names={"weight": "embed"},
        final_norm_names={"weight": "final.norm"},
        head_names={},
        max_positions=cfg.max_position_embeddings,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width,
                                               "scale": cfg.embedding_scale}),
    )


register_architecture("Sapanex", SapanexConfig, sapanex_plan, reads_shapes=True)
