"""Small Zafopel configurations, weights that make faults show, and helpers to run a request through the
engine's step function (any cut into steps) and through the plain implementation."""
from __future__ import annotations

import copy

import torch

import plain_zafopel as plain
from beledra_cases import cuts_of, relative_error, run_cuts, tokens_for, worst_row_error  # noqa: F401


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def moe(ff=24, experts=5, top=2):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def window_layer(heads=3, dim=24, rot_dim=8, vdim=20, kv_rank=40, window=21, base=300.0, rot_dims=None, scale=None,
                 kv_from=None, mlp="moe"):
    """latent_attention: direct queries, a sliding window."""
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
             "scale": (dim + rot_dim) ** -0.5 if scale is None else scale,
             "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims}}
    if window is not None:
        mixer["mask"] = {"size": window}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": mixer, "mlp": moe() if mlp == "moe" else mlp}


def sink_layer(heads=2, dim=16, rot_dim=16, vdim=24, kv_rank=48, q_rank=28, base=5000.0, rot_dims=None, scale=None,
               mlp="dense"):
    """latent_attention_2: queries through a latent, causal, a sink per head."""
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
             "scale": (dim + rot_dim) ** -0.5 if scale is None else scale,
             "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims}}
    return {"type": "latent_attention_2", "mixer": mixer, "mlp": dense() if mlp == "dense" else mlp}


def config(layers, vocab=96, width=32, eps=1e-5):
    return {"architecture": "Zafopel", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "layers": copy.deepcopy(layers)}


# both mixers, both feed-forwards and a layer without one, a reader of another layer's rows with a WIDER
# window than the owner's, windows that are no multiples of pages or tiles, one and several picks
MIXED = config([sink_layer(),
                window_layer(window=19),
                sink_layer(heads=5, dim=8, rot_dim=4, vdim=8, kv_rank=24, q_rank=12, mlp=moe(16, 3, 1)),
                window_layer(window=27, kv_from=1, mlp=None),
                window_layer(heads=2, dim=8, rot_dim=12, vdim=16, kv_rank=36, window=33, rot_dims=8, mlp=dense(56))])


def draw_weights(cfg: dict, seed: int = 0, dtype=torch.bfloat16) -> dict:
    """name -> tensor (as stored: ``dtype``) from the framework's seeded generator, with the small tensors
    redrawn so that each mechanism carries weight: sinks of spread 2, norm slopes and offsets off 1 and 0,
    routers whose scores are spread out."""
    from snowllm_b200.loader import build_model
    from snowllm_b200.weights import random_tensors
    model = build_model(cfg, "float32")
    tensors = random_tensors(model, seed, torch.float32, fan_in_scaled=True, norm_jitter=0.2)
    gen = torch.Generator().manual_seed(seed + 1)
    for name, t in tensors.items():
        if name.endswith(".sink"):
            tensors[name] = torch.randn(t.shape, generator=gen) * 2.0
        elif name.endswith(".alpha"):
            tensors[name] = 0.6 + 0.8 * torch.rand(t.shape, generator=gen)
        elif name.endswith("norm1.b") or name == "final.norm.b":
            tensors[name] = torch.randn(t.shape, generator=gen) * 0.2
        elif name.endswith(".router"):
            tensors[name] = t * 4.0
    return {k: v.to(dtype) for k, v in tensors.items()}


def write_folder(path, cfg: dict, tensors: dict):
    from snowllm_b200.loader import build_model
    from snowllm_b200.weights import write_model_folder
    return write_model_folder(path, build_model(cfg, "float32").config.to_json_dict(), tensors)


def plain_logits(cfg, tensors, tokens, layers_out=None, rounded=False, **kw):
    return plain.forward({"config": cfg, "tensors": tensors}, list(tokens), torch.float64, layers_out, rounded, **kw)
