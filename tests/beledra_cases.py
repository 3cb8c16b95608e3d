"""Small Beledra configurations, weights that make faults show, and the two ways to run a request:
through the engine's step function (any cut into steps) and through the plain implementation."""
from __future__ import annotations

import copy
import math

import numpy as np
import torch

import plain_beledra as plain


def attention_layer(heads=4, kv_heads=2, dim=16, vdim=24, window=21, bias_max=40, bias_rows=12, ff=48, scale=None):
    return {"type": "attention",
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": window},
                      "scale": dim ** -0.5 if scale is None else scale, "bias_max": bias_max, "bias_rows": bias_rows},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def diff_layer(heads=2, kv_heads=1, dim=16, vdim=40, window=19, diff=0.3, rot_dims=8, base=500.0, scaling=True,
               kv_from=None, ff=48, scale=None):
    rot = None
    if rot_dims:
        rot = {"dims": rot_dims, "base": base}
        if scaling:
            rot["scaling"] = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": window},
             "scale": dim ** -0.5 if scale is None else scale, "diff": diff}
    if rot:
        mixer["rot"] = rot
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "attention_2", "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def mlstm_layer(heads=2, dim=8, vdim=24, gate_cap=10.0, ff=None):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": gate_cap},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def config(layers, vocab=96, width=32, eps=1e-5):
    return {"architecture": "Beledra", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "layers": copy.deepcopy(layers)}


# every mixer, a layer without feed-forward, a reader of another layer's keys with a WIDER window than the
# owner's, windows that are no multiples of pages or tiles
MIXED = config([attention_layer(), diff_layer(window=19), mlstm_layer(), diff_layer(window=27, kv_from=1),
                attention_layer(heads=2, kv_heads=2, dim=8, vdim=8, window=33, bias_rows=6, bias_max=17)])


def draw_weights(cfg: dict, seed: int = 0, dtype=torch.bfloat16) -> dict:
    """name -> tensor (as stored: ``dtype``) from the framework's seeded generator, with the small tensors
    redrawn so that each mechanism carries weight: a bias table of spread 2, map weights that move lambda
    off its offset, gate biases that keep a long memory, norm weights off 1."""
    from snowllm_b200.loader import build_model
    from snowllm_b200.weights import random_tensors
    model = build_model(cfg, "float32")
    tensors = random_tensors(model, seed, torch.float32, fan_in_scaled=True, norm_jitter=0.2)
    gen = torch.Generator().manual_seed(seed + 1)
    for name, t in tensors.items():
        leaf = name.split(".mix.")[-1]
        if leaf == "rel":
            tensors[name] = torch.randn(t.shape, generator=gen) * 2.0
        elif leaf in ("lq1", "lk1", "lq2", "lk2"):
            tensors[name] = torch.randn(t.shape, generator=gen) * 0.3
        elif leaf == "i.b":
            tensors[name] = torch.randn(t.shape, generator=gen)
        elif leaf == "f.b":
            tensors[name] = 3.0 + torch.randn(t.shape, generator=gen)
        elif leaf in ("i", "f"):
            tensors[name] = t * 2.0
    return {k: v.to(dtype) for k, v in tensors.items()}


def write_folder(path, cfg: dict, tensors: dict):
    from snowllm_b200.loader import build_model
    from snowllm_b200.weights import write_model_folder
    return write_model_folder(path, build_model(cfg, "float32").config.to_json_dict(), tensors)


def plain_logits(cfg, tensors, tokens, layers_out=None, rounded=False):
    return plain.forward({"config": cfg, "tensors": tensors}, list(tokens), torch.float64, layers_out, rounded)


def tokens_for(cfg, n: int, seed: int = 0) -> list:
    g = torch.Generator().manual_seed(1000 + seed)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()


def run_cuts(replay, name: str, tokens, cuts, want_all=True, end=True):
    """Feed ``tokens`` of request ``name`` in steps of the sizes ``cuts``; logits of every position [T, V]."""
    out, at = [], 0
    for n in cuts:
        part = tokens[at:at + n]
        last = at + n >= len(tokens)
        got = replay.step([{"id": name, "tokens": part, "want": list(range(len(part)))}],
                          [name] if last and end else [])
        out.append(got.double())
        at += n
    assert at == len(tokens)
    return torch.cat(out, 0)


def cuts_of(total: int, sizes) -> list:
    """``sizes`` repeated until ``total`` tokens are used up (the last cut shortened)."""
    out, at, i = [], 0, 0
    while at < total:
        n = min(sizes[i % len(sizes)], total - at)
        out.append(n)
        at += n
        i += 1
    return out


def relative_error(got, want) -> float:
    """Root mean square of the difference over the root mean square of ``want``, rows' means taken off."""
    d = got.double() - want.double()
    d = d - d.mean(-1, keepdim=True)
    w = want.double() - want.double().mean(-1, keepdim=True)
    return float(torch.sqrt((d * d).mean()) / torch.sqrt((w * w).mean()))


def worst_row_error(got, want) -> float:
    d = got.double() - want.double()
    d = d - d.mean(-1, keepdim=True)
    w = want.double() - want.double().mean(-1, keepdim=True)
    scale = float(torch.sqrt((w * w).mean()))
    return float(torch.sqrt((d * d).mean(-1)).max()) / scale
