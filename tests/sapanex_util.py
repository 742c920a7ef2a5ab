"""Helpers of the Sapanex tests: small configurations, weights made for the tests, and a
driver that runs schedules of steps through the framework's step function.

The weights are not the random-weights mode's: matrices have unit-variance outputs so that
activations are of order one, queries and keys are sharpened through the configuration's
``scale``, and the delta rule's decay bias can be pushed towards "keep everything", so that a
key or a token far back, or one position beyond a window's edge, moves the logits by much
more than rounding does.
"""

from __future__ import annotations

import copy
import json
from pathlib import Path

import torch
from safetensors.torch import save_file


def attention_layer(dim=16, heads=4, kv_heads=2, vdim=24, window=12, pool=4, rot_dims=8,
                    base=10000.0, scaling=None, scale=None, ff=None):
    mixer = {"dim": dim, "heads": heads, "kv_heads": kv_heads, "vdim": vdim,
             "mask": {"size": window, "pool": pool} if window else None,
             "rot": {"base": base, "dims": rot_dims, "scaling": scaling},
             "scale": scale if scale is not None else 3.0 / dim ** 0.5}
    return {"type": "attention", "mixer": mixer,
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def delta_layer(dim=16, heads=3, ff=None, rank=None):
    mixer = {"dim": dim, "heads": heads}
    if rank:
        mixer["decay_rank"] = rank
    return {"type": "general_delta", "mixer": mixer,
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def config(layers, width=64, vocab=97, alpha=2.0, eps=1e-5, embed_scale=4.0):
    return {"architecture": "Sapanex", "embedding": {"scale": embed_scale},
            "layers": copy.deepcopy(layers), "norm": {"eps": eps}, "postln_alpha": alpha,
            "vocab": vocab, "width": width}


YARN = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}

# Two configurations that differ in every size, constant and in the order of their layers.
CONFIG_X = config([
    attention_layer(dim=16, heads=4, kv_heads=2, vdim=24, window=12, pool=4, rot_dims=8,
                    scaling=YARN, ff=96),
    delta_layer(dim=16, heads=3),
    delta_layer(dim=16, heads=3, ff=80),
    attention_layer(dim=16, heads=4, kv_heads=2, vdim=24, window=12, pool=4, rot_dims=8,
                    scaling=YARN),
], width=64, vocab=97, alpha=2.0, eps=1e-5, embed_scale=4.0)

CONFIG_Y = config([
    delta_layer(dim=24, heads=2, rank=5),
    attention_layer(dim=24, heads=6, kv_heads=6, vdim=24, window=9, pool=7, rot_dims=24,
                    base=500.0, scaling=None, scale=0.7, ff=None),
    attention_layer(dim=40, heads=3, kv_heads=1, vdim=56, window=30, pool=1, rot_dims=4,
                    base=77777.0, scaling={"factor": 1.5, "original": 20, "fast": 3.0, "slow": 0.5},
                    ff=50),
    delta_layer(dim=40, heads=1, ff=72, rank=3),
], width=88, vocab=131, alpha=1.0, eps=3e-6, embed_scale=1.0)


def decay_rank_of(cfg: dict, index: int) -> int:
    mixer = cfg["layers"][index]["mixer"]
    return int(mixer.get("decay_rank") or max(8, cfg["width"] // 16))


def make_weights(cfg: dict, seed: int, long_memory: bool = False) -> dict[str, torch.Tensor]:
    """Tensors by checkpoint name, float32 values that bfloat16 holds exactly."""
    g = torch.Generator().manual_seed(seed)

    def matrix(rows, cols, gain=1.0):
        return torch.randn(rows, cols, generator=g) * (gain / cols ** 0.5)

    def gains(n):
        return 1.0 + 0.2 * torch.randn(n, generator=g)

    width = cfg["width"]
    w = {"embed": torch.randn(cfg["vocab"], width, generator=g) * 0.5, "final.norm": gains(width)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        w[p + "norm1"] = gains(width)
        if layer["type"] == "attention":
            H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            w[p + "mix.q"], w[p + "mix.k"] = matrix(H * D, width), matrix(G * D, width)
            w[p + "mix.v"], w[p + "mix.o"] = matrix(G * V, width), matrix(width, H * V)
            w[p + "mix.q.norm"], w[p + "mix.k.norm"] = gains(H * D), gains(G * D)
        else:
            hd, rank = m["heads"] * m["dim"], decay_rank_of(cfg, i)
            for name in ("r", "k", "v", "g", "a"):
                w[p + "mix." + name] = matrix(hd, width)
            w[p + "mix.w1"], w[p + "mix.w2"] = matrix(rank, width), matrix(hd, rank, 2.0)
            # strongly negative biases make the decay close to one and the removal rate close
            # to nought: the state then remembers tokens from hundreds of steps back
            w[p + "mix.w0"] = torch.randn(hd, generator=g) + (-7.0 if long_memory else 0.0)
            w[p + "mix.a.b"] = torch.randn(hd, generator=g) * 0.5 + (-6.0 if long_memory else 0.0)
            w[p + "mix.norm"] = gains(hd)
            w[p + "mix.o"] = matrix(width, hd)
        if layer.get("mlp"):
            ff = layer["mlp"]["ff"]
            w[p + "norm2"] = gains(width)
            w[p + "mlp.up"], w[p + "mlp.down"] = matrix(ff, width), matrix(width, ff)
    return {k: v.to(torch.bfloat16).to(torch.float32).contiguous() for k, v in w.items()}


def write_model(folder, cfg: dict, weights: dict[str, torch.Tensor]) -> Path:
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    save_file({k: v.to(torch.bfloat16) for k, v in weights.items()}, str(folder / "model.safetensors"))
    (folder / "config.json").write_text(json.dumps(cfg, indent=1))
    return folder


def tokens(n: int, vocab: int, seed: int) -> list[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def relative_error(got: torch.Tensor, want: torch.Tensor) -> float:
    """Largest row-wise ``rms(got - want) / rms(want)``."""
    got, want = got.double(), want.double()
    num = (got - want).pow(2).mean(-1).sqrt()
    den = want.pow(2).mean(-1).sqrt().clamp_min(1e-12)
    return float((num / den).max())


def fraction_over(got: torch.Tensor, want: torch.Tensor, tol: float) -> float:
    """Share of the rows whose ``rms(got - want) / rms(want)`` exceeds ``tol``."""
    got, want = got.double(), want.double()
    err = (got - want).pow(2).mean(-1).sqrt() / want.pow(2).mean(-1).sqrt().clamp_min(1e-12)
    return float((err > tol).double().mean())


class Driver:
    """A model loaded as generation loads it, a cache manager and the step function."""

    def __init__(self, folder, dtype: str, pool_tokens: int = 2048, page_size: int = 16,
                 slots: int = 4, max_step_tokens: int = 1024, graphs: bool = False):
        from simple_inference_b200.cache.manager import CacheManager
        from simple_inference_b200.engine.runner import ModelRunner
        from simple_inference_b200.models.load import load_model
        self.cfg, self.model = load_model(folder, dtype, "cuda")
        rt = self.model.rt
        self.cache = CacheManager(self.model.cache_specs(), page_size,
                                  lambda ps: (pool_tokens + ps - 1) // ps + slots, slots,
                                  max_step_tokens, dtype=rt.dtype, device=rt.device)
        self.runner = ModelRunner(self.model, self.cache, rt, max_step_tokens, slots, pool_tokens,
                                  cuda_graphs=graphs, max_logit_rows=max_step_tokens)

    def step(self, entries, end=()) -> list[torch.Tensor]:
        """``entries``: (request, tokens) pairs; logits of every token, per entry."""
        from simple_inference_b200 import ops
        from simple_inference_b200.engine.batch import StepEntry
        batch = []
        for rid, toks in entries:
            if not self.cache.is_admitted(rid):
                self.cache.admit(rid, len(toks))
            else:
                self.cache.reserve_to(rid, self.cache.length(rid) + len(toks))
            batch.append(StepEntry(rid, list(toks), list(range(len(toks)))))
        logits = self.runner.step(batch).float().cpu()
        ops.check_status(self.model.rt.device)
        out, r = [], 0
        for _, toks in entries:
            out.append(logits[r:r + len(toks)].clone())
            r += len(toks)
        for rid in end:
            self.cache.release(rid)
        return out

    def run_cut(self, rid, toks, cuts) -> torch.Tensor:
        """One request alone, in portions of the sizes ``cuts`` (the last size repeats)."""
        rows, i, k = [], 0, 0
        while i < len(toks):
            n = min(cuts[min(k, len(cuts) - 1)], len(toks) - i)
            rows.append(self.step([(rid, toks[i:i + n])])[0])
            i, k = i + n, k + 1
        self.cache.release(rid)
        return torch.cat(rows)
