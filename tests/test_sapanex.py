"""Sapanex on the CPU: configuration, plan and tensor names, rotation frequencies, the cache
manager's composite entries, and the plain implementation's own consistency."""

from __future__ import annotations

import copy
import json
import math

import pytest
import torch

from simple_inference_b200.cache.manager import CacheManager
from simple_inference_b200.config import ConfigError, SapanexConfig, architecture_of, read_config
from simple_inference_b200.models.plan import DecoderModel
from simple_inference_b200.parts.base import CompositeSpec, KeyValuePlanesSpec, StateSpec
from simple_inference_b200.parts.rope import yarn_frequencies
from simple_inference_b200.weights import write_random_model
from simple_inference_b200.weights.loader import tensor_shapes
from tests import plain_sapanex as plain
from tests.sapanex_util import (CONFIG_X, CONFIG_Y, YARN, attention_layer, config, delta_layer,
                                make_weights, tokens, write_model)


def test_config_is_read_by_its_architecture_name_and_round_trips():
    arch = architecture_of(CONFIG_Y)
    assert arch.name == "Sapanex" and arch.config_class is SapanexConfig
    cfg = SapanexConfig.from_dict(CONFIG_Y)
    assert cfg.vocab_size == 131 and cfg.hidden_size == 88 and cfg.eps == 3e-6
    assert cfg.embedding_scale == 1.0 and cfg.postln_alpha == 1.0
    a = cfg.layers[2].mixer
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.window, a.pool) == (3, 1, 40, 56, 30, 1)
    assert a.rot.dims == 4 and a.rot.base == 77777.0 and a.rot.scaling.factor == 1.5
    assert cfg.layers[1].mixer.rot.scaling is None and cfg.layers[1].mlp is None
    assert cfg.layers[3].mlp.ff == 72 and cfg.layers[3].mixer.decay_rank == 3
    again = SapanexConfig.from_dict(json.loads(json.dumps(cfg.to_dict())))
    assert again.to_dict() == cfg.to_dict()


@pytest.mark.parametrize("breaker,word", [
    (lambda c: c.pop("postln_alpha"), "postln_alpha"),
    (lambda c: c["layers"][0].update(type="convolution"), "convolution"),
    (lambda c: c["layers"][1]["mixer"].pop("vdim"), "vdim"),
    (lambda c: c["layers"][1]["mixer"].update(heads=5, kv_heads=2), "divide"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "even"),
    (lambda c: c["layers"][2]["mlp"].update(kind="routed"), "dense"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c.update(layers=[]), "no layers"),
])
def test_config_errors_name_what_is_wrong(breaker, word):
    cfg = copy.deepcopy(CONFIG_Y)
    breaker(cfg)
    with pytest.raises(ConfigError, match=word):
        SapanexConfig.from_dict(cfg)


def test_plan_names_every_tensor_and_reads_the_decay_width_from_the_checkpoint(tmp_path):
    cfg = copy.deepcopy(CONFIG_X)
    w = make_weights(cfg, 1)
    # a checkpoint's config.json does not say how wide the decay's inner projection is
    for name in ("l1.mix.w1", "l2.mix.w1"):
        w[name] = torch.zeros(3, cfg["width"])
    for name in ("l1.mix.w2", "l2.mix.w2"):
        w[name] = torch.zeros(w[name].shape[0], 3)
    folder = write_model(tmp_path, cfg, w)
    arch, typed = read_config(folder)
    assert arch.reads_shapes
    model = DecoderModel(arch.plan_for(typed, tensor_shapes(folder)))
    specs = model.tensor_specs()
    assert set(specs) == set(w)
    for name, spec in specs.items():
        assert tuple(spec.shape) == tuple(w[name].shape), name
    assert specs["l1.mix.w0"].kind == "vector" and specs["l0.mix.q.norm"].kind == "vector"
    assert "l1.norm2" not in specs and "l2.norm2" in specs and "l3.mlp.up" not in specs
    # two attention layers of equal sizes share their page groups; every delta layer has a state
    kinds = [type(s).__name__ for s in model.cache_specs()]
    assert kinds == ["CompositeSpec", "StateSpec", "StateSpec", "CompositeSpec"]
    assert model.cache_specs()[0] == model.cache_specs()[3]


def test_random_weights_mode_writes_a_sapanex_folder(tmp_path):
    folder = write_random_model(tmp_path, CONFIG_Y, seed=3)
    shapes = tensor_shapes(folder)
    assert shapes["l0.mix.w1"] == (5, 88) and shapes["l3.mix.w2"] == (40, 3)
    assert shapes["l2.mix.o"] == (88, 3 * 56) and shapes["l1.mix.k.norm"] == (6 * 24,)
    arch, typed = read_config(folder)
    assert typed.to_dict() == SapanexConfig.from_dict(CONFIG_Y).to_dict()


@pytest.mark.parametrize("dims,base,scaling", [
    (8, 10000.0, None), (8, 10000.0, YARN), (24, 500.0, {"factor": 1.5, "original": 20, "fast": 3.0, "slow": 0.5}),
    (2, 77777.0, {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}),
    (64, 1e6, {"factor": 1.0, "original": 8, "fast": 2.0, "slow": 1.0}),
])
def test_rotation_frequencies(dims, base, scaling):
    got, amp = yarn_frequencies(dims, base, scaling)
    want, want_amp = plain.rotary_frequencies(dims, base, scaling)
    assert got.dtype == torch.float32 and got.shape == (dims // 2,)
    assert torch.allclose(got.double(), want, rtol=1e-7, atol=0)
    assert amp == pytest.approx(want_amp)
    if scaling is None:
        assert amp == 1.0 and got[0] == 1.0
    else:
        plain_f, _ = plain.rotary_frequencies(dims, base, None)
        assert (want <= plain_f + 1e-15).all() and (want >= plain_f / scaling["factor"] - 1e-15).all()


def test_which_tokens_and_blocks_a_position_sees():
    assert plain.visible_tokens(3, 5) == [0, 1, 2, 3]
    assert plain.visible_tokens(9, 5) == [5, 6, 7, 8, 9]
    # block b of 4 positions is seen once its last position is at most i - 5
    assert plain.visible_blocks(7, 5, 4) == []
    assert plain.visible_blocks(8, 5, 4) == [0]          # 3 <= 8 - 5
    assert plain.visible_blocks(11, 5, 4) == [0]         # 7 > 11 - 5: positions 4..6 are seen by no one
    assert plain.visible_blocks(12, 5, 4) == [0, 1]
    assert plain.visible_blocks(12, 5, 1) == list(range(8))


def test_plain_delta_rule_carries_its_state():
    cfg = config([delta_layer(dim=8, heads=2)], width=16, vocab=11)
    w = {k: v.double() for k, v in make_weights(cfg, 2).items()}
    h = torch.randn(9, 16, dtype=torch.float64, generator=torch.Generator().manual_seed(0))
    m = cfg["layers"][0]["mixer"]
    whole, last = plain.general_delta_mixer(h, w, "l0.mix.", m, 1e-5)
    first, s = plain.general_delta_mixer(h[:4], w, "l0.mix.", m, 1e-5)
    rest, s2 = plain.general_delta_mixer(h[4:], w, "l0.mix.", m, 1e-5, state=s)
    assert torch.allclose(torch.cat([first, rest]), whole, atol=1e-12)
    assert torch.allclose(s2, last, atol=1e-12)
    # one step by hand: S1 = k v^T, o = S1^T r
    r, k, v = (h[:1] @ w["l0.mix." + n].T for n in "rkv")
    s1 = torch.einsum("hc,hd->hcd", k.view(2, 8), v.view(2, 8))
    _, got = plain.general_delta_mixer(h[:1], w, "l0.mix.", m, 1e-5)
    assert torch.allclose(got, s1, atol=1e-12)


def _manager(specs, **kw):
    args = dict(page_size=4, num_pages=lambda ps: 12, max_requests=2, max_step_tokens=8,
                dtype=torch.float32, device="cpu")
    args.update(kw)
    return CacheManager(specs, **args)


def test_cache_manager_composite_entries_windows_and_reuse():
    tok = KeyValuePlanesSpec(2, 6, 10, window=5)
    blk = KeyValuePlanesSpec(2, 6, 10, window=None, page_size=12, tokens_per_row=3)
    state = StateSpec((2, 4, 4))
    cm = _manager([CompositeSpec((tok, blk)), state, CompositeSpec((tok, blk)), None])
    assert len(cm.groups) == 2 and cm.groups[0].page_size == 4 and cm.groups[1].page_size == 12
    assert cm.groups[0].pool.shape == (2, 13, 2 * 4 * 16) and cm.groups[1].pool.shape == (2, 13, 2 * 4 * 16)
    views = cm.layer_caches()
    assert views[3] is None and views[1].state.shape == (3, 2, 4, 4)
    t0, b0 = views[0].members
    assert t0.group == 0 and b0.group == 1 and t0.page_size == 4 and b0.page_size == 12
    assert views[2].members[0].pool.data_ptr() != t0.pool.data_ptr()
    assert views[0].with_writes(False).members[1].writes is False

    cm.admit("a", 8)
    views[1].state[cm.slot("a")] += 1.0
    for _ in range(5):
        cm.reserve_to("a", cm.length("a") + 8)
        cm.extend("a", 8)
    # 40 tokens: the token cache keeps the pages of the last 5 + 8 tokens, the block cache all four
    table = cm.block_table("a", 0)
    assert all(p < 0 for p in table[:7]) and all(p >= 0 for p in table[7:]) and len(table) == 10
    assert all(p >= 0 for p in cm.block_table("a", 1)) and len(cm.block_table("a", 1)) == 4
    # min-heap allocator: the pages given back by the window were handed out again to "a" itself
    assert len({p for p in table if p >= 0}) == 3 and max(table) < 6   # ten logical pages so far
    cm.release("a")
    cm.admit("b", 8)
    assert cm.slot("b") == 0 and float(views[1].state[0].abs().sum()) == 0.0   # slot used again, zeroed
    cm.extend("b", 8)
    assert cm.block_table("b", 0) == [0, 1] and cm.block_table("b", 1) == [0]
    for g in cm.groups:
        g.allocator.check()


def test_attention_cache_keeps_a_block_whole_when_blocks_are_longer_than_the_window():
    from simple_inference_b200.parts.pooled_attention import PooledWindowAttention
    mixer = PooledWindowAttention(32, 2, 1, 8, 8, 0.3, window=5, pool=9,
                                  rotary={"dims": 4, "base": 100.0, "scaling": None}, rotate_values=True)
    tok, blk = mixer.cache_spec().members
    assert tok.window == 9 and tok.tokens_per_row == 1
    assert blk.window is None and blk.tokens_per_row == 9 and blk.page_size % 9 == 0
    plain_window = PooledWindowAttention(32, 2, 1, 8, 8, 0.3, window=None, pool=None)
    assert isinstance(plain_window.cache_spec(), KeyValuePlanesSpec) and plain_window.cache_spec().window is None
    with pytest.raises(ValueError):
        PooledWindowAttention(32, 2, 1, 8, 8, 0.3, window=None, pool=4)
