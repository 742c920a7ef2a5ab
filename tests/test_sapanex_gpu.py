"""The Sapanex design in the framework against the plain implementation (tests/plain_sapanex.py).

Every test builds a small model of its own, writes it as a checkpoint, loads it the way
generation does and drives the framework's step function, cache manager and kernels; the
expected logits come from the plain whole-sequence implementation in float64.
"""

from __future__ import annotations

import pytest
import torch

from tests import plain_sapanex as plain
from tests.sapanex_util import (CONFIG_X, CONFIG_Y, YARN, Driver, attention_layer, config,
                                delta_layer, make_weights, relative_error, tokens, write_model)

pytestmark = pytest.mark.gpu

FP32_TOL = 2e-5     # measured: below 3e-6
BF16_TOL = 6e-2     # measured: up to 2.5e-2 on these sharpened models
TOL = {"float32": FP32_TOL, "bfloat16": BF16_TOL}


def oracle(cfg, weights, toks, layers_out=None):
    return plain.forward(cfg, weights, toks, layers_out=layers_out).float()


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, cfg, seed in (("X", CONFIG_X, 5), ("Y", CONFIG_Y, 6)):
        w = make_weights(cfg, seed)
        out[name] = (cfg, w, write_model(tmp_path_factory.mktemp("sapanex_" + name), cfg, w))
    return out


# ------------------------------------------------------------ each mechanism alone

@pytest.mark.parametrize("kind", ["attention", "attention_ff", "delta", "delta_ff"])
def test_one_layer_of_each_kind_in_float32(tmp_path, kind):
    layer = {"attention": attention_layer(scaling=YARN), "attention_ff": attention_layer(ff=72),
             "delta": delta_layer(), "delta_ff": delta_layer(ff=40, rank=4)}[kind]
    cfg = config([layer], width=48, vocab=61, alpha=1.5)
    w = make_weights(cfg, 21)
    folder = write_model(tmp_path, cfg, w)
    toks = tokens(70, cfg["vocab"], 3)
    got = Driver(folder, "float32").run_cut("a", toks, [len(toks)])
    assert relative_error(got, oracle(cfg, w, toks)) < FP32_TOL


def test_residual_stream_after_every_layer(models):
    """The stream after each layer, read off the framework's own buffers between the blocks."""
    cfg, w, folder = models["X"]
    toks = tokens(50, cfg["vocab"], 9)
    want = []
    oracle(cfg, w, toks, layers_out=want)
    d = Driver(folder, "float32")
    seen = []
    for block in d.model.blocks:
        inner = block.forward

        def spy(residual, delta, ctx, cache, _inner=inner):
            out = _inner(residual, delta, ctx, cache)
            assert out is None   # a post-norm block hands nothing on to be added
            seen.append(residual.clone().cpu())
            return out
        block.forward = spy
    d.run_cut("a", toks, [len(toks)])
    assert len(seen) == len(want)
    for i, (a, b) in enumerate(zip(seen, want)):
        assert relative_error(a, b.float()) < FP32_TOL, f"layer {i}"


def test_row_kernels_of_the_post_norm_block():
    from simple_inference_b200 import ops
    g = torch.Generator().manual_seed(0)
    n, width, alpha, eps = 7, 100, 2.5, 1e-4
    x = torch.randn(n, width, generator=g)
    gain = 1 + 0.3 * torch.randn(width, generator=g)
    d = torch.randn(n, width, generator=g).to(torch.bfloat16)

    def expect(x, delta):
        y = alpha * x.double() + delta.double()
        return (y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps) * gain.double()).float()

    res = x.cuda().clone()
    out = torch.empty(n, width, dtype=torch.bfloat16, device="cuda")
    ops.scaled_add_rmsnorm(res, gain.cuda().to(torch.bfloat16), alpha, eps, out, d.cuda())
    y = alpha * x.double() + d.double()
    want_b = (y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps)
              * gain.to(torch.bfloat16).double()).float()
    assert torch.allclose(res.cpu(), want_b, atol=2e-6, rtol=2e-6)
    assert torch.equal(out, res.to(torch.bfloat16))
    # float32, the addend as slices of a product cut along k
    parts = torch.randn(3, n, width, generator=g)
    res = x.cuda().clone()
    out32 = torch.empty(n, width, device="cuda")
    ops.scaled_add_rmsnorm(res, gain.cuda(), alpha, eps, out32,
                           ops.PartialSums(parts.cuda().contiguous(), torch.float32))
    assert torch.allclose(res.cpu(), expect(x, parts.sum(0)), atol=3e-6, rtol=3e-6)
    assert torch.equal(res, out32)
    # without an addend, and without a rounded copy
    res = x.cuda().clone()
    ops.scaled_add_rmsnorm(res, gain.cuda(), alpha, eps, None, None)
    assert torch.allclose(res.cpu(), expect(x, torch.zeros_like(x)), atol=3e-6, rtol=3e-6)
    # squared rectifier, rounding of the stream, scaled embedding
    h = torch.randn(5, 33, generator=g).cuda()
    assert torch.allclose(ops.relu2(h, torch.empty_like(h)), torch.relu(h) ** 2)
    res = x.cuda().clone()
    rounded = ops.residual_cast(res, torch.empty(n, width, dtype=torch.bfloat16, device="cuda"), d.cuda())
    assert torch.allclose(res.cpu(), x + d.float()) and torch.equal(rounded, res.to(torch.bfloat16))
    table = torch.randn(11, 20, generator=g).to(torch.bfloat16).cuda()
    ids = torch.tensor([3, 0, 10], dtype=torch.int32, device="cuda")
    emb = ops.embed_gather(table, ids, torch.empty(3, 20, device="cuda"), 12.5)
    assert torch.equal(emb, table[ids.long()].float() * 12.5)


# ------------------------------------------------- whole prompts, decoding, portions

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["X", "Y"])
def test_whole_prompt(models, name, dtype):
    cfg, w, folder = models[name]
    toks = tokens(150, cfg["vocab"], 17)
    got = Driver(folder, dtype).run_cut("a", toks, [len(toks)])
    assert relative_error(got, oracle(cfg, w, toks)) < TOL[dtype]


@pytest.mark.parametrize("dtype,graphs", [("float32", False), ("bfloat16", False), ("bfloat16", True)])
@pytest.mark.parametrize("name", ["X", "Y"])
def test_token_by_token_equals_the_whole_prompt(models, name, dtype, graphs):
    """Long decoding: every token alone through the cache and the state, from the first one;
    the windows pass over decoded tokens and pooled blocks are made from decoded tokens."""
    cfg, w, folder = models[name]
    toks = tokens(120, cfg["vocab"], 23)
    got = Driver(folder, dtype, graphs=graphs).run_cut("a", toks, [1])
    assert relative_error(got, oracle(cfg, w, toks)) < TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cuts", [[2], [3], [5, 2, 11, 1, 1, 7], [16], [17], [64, 1]])
def test_portions_of_several_sizes(models, dtype, cuts):
    cfg, w, folder = models["X"]
    toks = tokens(131, cfg["vocab"], 29)
    got = Driver(folder, dtype).run_cut("a", toks, cuts)
    assert relative_error(got, oracle(cfg, w, toks)) < TOL[dtype]


def test_float32_does_not_depend_on_the_cut(models):
    cfg, w, folder = models["Y"]
    toks = tokens(90, cfg["vocab"], 31)
    d = Driver(folder, "float32")
    whole = d.run_cut("a", toks, [len(toks)])
    for cuts in ([1], [2], [7, 3], [64, 1], [70, 20]):   # below and above the row counts where kernels change
        assert relative_error(d.run_cut("a", toks, cuts), whole) < 1e-7   # measured 0.0: the same sums in the same order


# --------------------------------------------------------------- batches and reuse

@pytest.mark.parametrize("dtype,graphs", [("float32", False), ("bfloat16", True)])
def test_unequal_requests_together_equal_each_alone(models, dtype, graphs):
    cfg, w, folder = models["X"]
    vocab = cfg["vocab"]
    reqs = {"a": tokens(75, vocab, 1), "b": tokens(33, vocab, 2), "c": tokens(1, vocab, 3),
            "d": tokens(58, vocab, 4)}
    want = {r: oracle(cfg, w, t) for r, t in reqs.items()}
    d = Driver(folder, dtype, graphs=graphs)
    got = {r: [] for r in reqs}
    done = {r: 0 for r in reqs}
    # portions of some beside single tokens of others; "c" joins late, "b" pauses for two steps
    plan = [{"a": 20, "b": 5}, {"a": 1, "b": 9, "d": 2}, {"a": 1, "d": 30}, {"a": 1, "c": 1, "d": 1},
            {"a": 17, "b": 1, "d": 1}, {"a": 1, "b": 1, "d": 1}]
    step = 0
    while any(done[r] < len(reqs[r]) for r in reqs):
        sizes = plan[step] if step < len(plan) else {r: 1 for r in reqs}
        entries = [(r, reqs[r][done[r]:done[r] + n]) for r, n in sizes.items()
                   if done[r] < len(reqs[r])]
        entries = [(r, t) for r, t in entries if t]
        for (r, t), rows in zip(entries, d.step(entries)):
            got[r].append(rows)
            done[r] += len(t)
        step += 1
    for r in reqs:
        assert relative_error(torch.cat(got[r]), want[r]) < TOL[dtype], r


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_pages_and_slots_that_are_used_again(models, dtype):
    """A pool of a few pages and two slots: requests come and go, every page and slot serves
    several of them, and each request's logits are those it has alone in a fresh cache."""
    cfg, w, folder = models["X"]
    vocab = cfg["vocab"]
    d = Driver(folder, dtype, pool_tokens=128, page_size=8, slots=2, max_step_tokens=64)
    seen_pages, seen_slots = {}, {}
    for k in range(6):
        a, b = tokens(40 + 3 * k, vocab, 50 + k), tokens(17 + k, vocab, 70 + k)
        got_a = [d.step([("a", a[:25])])[0]]
        rows = d.step([("a", a[25:26]), ("b", b[:10])])
        got_a.append(rows[0]); got_b = [rows[1]]
        for g in range(len(d.cache.groups)):
            for r in ("a", "b"):
                for page in d.cache.block_table(r, g):
                    if page >= 0:
                        seen_pages.setdefault((g, page), set()).add((k, r))
        for r in ("a", "b"):
            seen_slots.setdefault(d.cache.slot(r), set()).add((k, r))
        rows = d.step([("a", a[26:]), ("b", b[10:])], end=("b",))
        got_a.append(rows[0]); got_b.append(rows[1])
        d.cache.release("a")
        assert relative_error(torch.cat(got_a), oracle(cfg, w, a)) < TOL[dtype]
        assert relative_error(torch.cat(got_b), oracle(cfg, w, b)) < TOL[dtype]
        for grp in d.cache.groups:
            grp.allocator.check()
    assert max(len(v) for v in seen_pages.values()) >= 4
    assert all(len(v) >= 3 for v in seen_slots.values()) and len(seen_slots) == 2


# ------------------------------------------- the tensor-core attention kernel by itself

def _paged_case(G, kd, vd, W, P, seqs, seed, rows=16, blk_rows=4):
    """Random queries and caches for sequences given as (context length, tokens in the step).
    Pages are handed out in random order; table entries before what a step may read point at
    a page of huge values, so that a read outside the window shows."""
    g = torch.Generator().manual_seed(seed)
    n_pages = sum((c + rows - 1) // rows for c, _ in seqs) + 1
    n_bpages = sum((c // P + blk_rows - 1) // blk_rows + 1 for c, _ in seqs) + 1
    tok_pool = torch.randn(n_pages, G * rows * (kd + vd), generator=g)
    blk_pool = torch.randn(n_bpages, G * blk_rows * (kd + vd), generator=g)
    tok_pool[0] = 3e4; blk_pool[0] = 3e4                    # the poisoned pages
    free = (torch.randperm(n_pages - 1, generator=g) + 1).tolist()
    bfree = (torch.randperm(n_bpages - 1, generator=g) + 1).tolist()
    max_pages = max((c + rows - 1) // rows for c, _ in seqs)
    max_bpages = max((c // P + blk_rows - 1) // blk_rows + 1 for c, _ in seqs)
    tok_table = torch.zeros(len(seqs), max_pages, dtype=torch.int32)
    blk_table = torch.zeros(len(seqs), max_bpages, dtype=torch.int32)
    positions, tok_seq, cu_q = [], [], [0]
    for s, (ctx, nq) in enumerate(seqs):
        first = max(0, ctx - nq - W + 1)                    # first token any query of the step sees
        for lp in range(first // rows, (ctx + rows - 1) // rows):
            tok_table[s, lp] = free.pop()
        n_blocks = max(0, (ctx - 1 - W + 1)) // P           # blocks the last query sees
        for lp in range((n_blocks + blk_rows - 1) // blk_rows):
            blk_table[s, lp] = bfree.pop()
        positions += list(range(ctx - nq, ctx))
        tok_seq += [s] * nq
        cu_q.append(cu_q[-1] + nq)
    return dict(tok_pool=tok_pool, blk_pool=blk_pool, tok_table=tok_table, blk_table=blk_table,
                positions=torch.tensor(positions, dtype=torch.int32),
                tok_seq=torch.tensor(tok_seq, dtype=torch.int32),
                cu_q=torch.tensor(cu_q, dtype=torch.int32), rows=rows, blk_rows=blk_rows)


@pytest.mark.parametrize("H,G,kd,vd,W,P", [(8, 2, 64, 80, 40, 8), (3, 1, 128, 128, 24, 5),
                                             (10, 2, 16, 32, 7, 16), (4, 4, 32, 16, 100, 3),
                                             (20, 1, 32, 32, 50, 4), (6, 3, 48, 96, 2000, 64)])
def test_tensor_core_attention_equals_the_generic_kernel(H, G, kd, vd, W, P):
    """Portions of prompts (from position 0, in mid-sequence, over page borders), single decoded
    tokens and a first token in one batch; bfloat16 caches; the generic kernel, which the other
    tests hold against the plain implementation, is the yardstick."""
    from simple_inference_b200 import ops
    seqs = [(300, 37), (1, 1), (150, 1), (64, 64), (500, 16), (W + P, 1), (W + P - 1, 1), (33, 17)]
    case = _paged_case(G, kd, vd, W, P, seqs, seed=kd + W)
    n = int(case["cu_q"][-1])
    g = torch.Generator().manual_seed(1)
    q = (torch.randn(n, H * kd + 24, generator=g) * 1.5).to(torch.bfloat16).cuda()
    freq_v = (10000.0 ** (-torch.arange(vd // 2, dtype=torch.float64) * 2 / vd)).float().cuda()
    dev = {k: (v.to(torch.bfloat16).cuda() if v.dtype == torch.float32 else v.cuda())
           for k, v in case.items() if isinstance(v, torch.Tensor)}
    outs = []
    for cu_q, splits in ((None, 1), (dev["cu_q"], 1), (dev["cu_q"], 3), (dev["cu_q"], 8)):
        out = torch.zeros(n, H * vd, dtype=torch.bfloat16, device="cuda")
        scratch = None
        if splits > 1:   # tiles of few rows shared out among blocks, joined by a second kernel
            scratch = torch.full((ops.window_pool_scratch_rows(n, len(seqs), G, splits), vd + 2),
                                 float("nan"), device="cuda")
        ops.window_pool_attention(q, dev["positions"], dev["tok_seq"], dev["tok_pool"], dev["tok_table"],
                                  case["rows"], dev["blk_pool"], dev["blk_table"], case["blk_rows"], out,
                                  H, G, kd, vd, 0.6 / kd ** 0.5 * 4, W, P, freq_v, cu_q, len(seqs),
                                  splits, scratch)
        outs.append(out.float().cpu())
    generic = outs[0]
    assert generic.abs().max() < 100   # nobody read a poisoned page
    for fast in outs[1:]:
        assert torch.isfinite(fast).all()
        assert (fast - generic).abs().max() < 0.04 * generic.abs().max()
        assert relative_error(fast, generic) < 0.03


@pytest.mark.parametrize("rows", [1, 9, 16, 40, 130, 300])
def test_squared_relu_as_the_epilogue_of_the_product(rows):
    from simple_inference_b200 import ops
    g = torch.Generator().manual_seed(rows)
    x = torch.randn(rows, 192, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(328, 192, generator=g) * 0.1).to(torch.bfloat16).cuda()
    out = ops.linear_relu2(x, w, torch.empty(rows, 328, dtype=torch.bfloat16, device="cuda"))
    ops.check_status(x.device)
    want = torch.relu(x.float() @ w.float().T) ** 2
    assert (out.float() - want).abs().max() <= 0.01 * want.abs().max() + 1e-3
    x32, w32 = x.float(), w.float()
    out32 = ops.linear_relu2(x32, w32, torch.empty(rows, 328, device="cuda"))
    assert torch.allclose(out32, want, rtol=1e-5, atol=1e-5)
