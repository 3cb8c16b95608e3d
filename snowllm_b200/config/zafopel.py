"""Typed configuration of the Zafopel design, read from its config.json.

    {"architecture": "Zafopel", "vocab": V, "width": W, "norm": {"eps": e},
     "layers": [{"type": T, "mixer": {...}, "mlp": {...} | null}, ...]}

``type`` names the layer's mixer; ``mixer`` holds that mixer's sizes and constants:

* ``latent_attention``:   heads, dim, rot_dim, vdim, kv_rank, scale, rot {dims, base}, mask.size (the
                          window; without it the layer sees every earlier key), kv_from (optional: the
                          layer whose cached latent rows it reads; it then has no latent projection)
* ``latent_attention_2``: heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, rot {dims, base}; causal, with
                          a sink per head

``mlp``: ``{"kind": "dense", "ff": F}``, ``{"kind": "moe", "expert": {"ff": F}, "router": {"experts": E,
"top": k}}`` or null.  Every size and constant comes from the file; what is missing or unusable is
reported in one ConfigError that lists every key."""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any

from ..errors import ConfigError
from .beledra import _is_int, _Reader

ARCHITECTURE = "Zafopel"
LAYER_TYPES = ("latent_attention", "latent_attention_2")
MLP_KINDS = ("dense", "moe")


@dataclass(frozen=True)
class ZafopelLayer:
    type: str
    mixer: dict          # heads, dim, rot_dim, vdim, kv_rank, q_rank | None, scale, rot, window | None, kv_from | None
    mlp: dict | None     # {"kind": "dense", "ff"} | {"kind": "moe", "ff", "experts", "top"}


@dataclass(frozen=True)
class ZafopelConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    layers: tuple

    def to_json_dict(self) -> dict[str, Any]:
        """config.json content that reads back to this configuration."""
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.norm_eps},
                "layers": [{"type": l.type, "mixer": _mixer_json(l), "mlp": _mlp_json(l.mlp)} for l in self.layers]}


def _mixer_json(layer: ZafopelLayer) -> dict:
    m = copy.deepcopy(layer.mixer)
    window = m.pop("window", None)
    if window is not None:
        m["mask"] = {"size": window}
    for key in ("kv_from", "q_rank"):
        if m.get(key) is None:
            m.pop(key, None)
    return m


def _mlp_json(mlp):
    if mlp is None:
        return None
    if mlp["kind"] == "dense":
        return {"kind": "dense", "ff": mlp["ff"]}
    return {"kind": "moe", "expert": {"ff": mlp["ff"]}, "router": {"experts": mlp["experts"], "top": mlp["top"]}}


def _read_mixer(r: _Reader, kind: str, m: dict, w: str, i: int) -> dict:
    out = dict(heads=r.positive_int(m, "heads", w), dim=r.positive_int(m, "dim", w),
               rot_dim=r.positive_int(m, "rot_dim", w), vdim=r.positive_int(m, "vdim", w),
               kv_rank=r.positive_int(m, "kv_rank", w), scale=r.positive(m, "scale", w),
               q_rank=None, window=None, kv_from=None)
    rot = m.get("rot")
    rw = w + "rot."
    out["rot"] = dict(dims=r.positive_int(rot, "dims", rw), base=r.positive(rot, "base", rw))
    dims = out["rot"]["dims"]
    if dims and (dims % 2 or (out["rot_dim"] and dims > out["rot_dim"])):
        r.bad.append(f"{rw}dims={dims} (want an even number, at most rot_dim={out['rot_dim']})")
    if kind == "latent_attention_2":
        out["q_rank"] = r.positive_int(m, "q_rank", w)
    else:
        mask = m.get("mask")
        if mask is not None:
            out["window"] = r.positive_int(mask, "size", w + "mask.") or None
        src = m.get("kv_from")
        if src is not None and (not _is_int(src) or not 0 <= src < i):
            r.bad.append(f"{w}kv_from={src!r} (want an earlier layer)")
            src = None
        out["kv_from"] = src
    return out


def _read_mlp(r: _Reader, mlp, where: str):
    if mlp is None:
        return None
    kind = mlp.get("kind") if isinstance(mlp, dict) else None
    if kind not in MLP_KINDS:
        r.bad.append(f"{where}mlp.kind={kind!r} (want one of {MLP_KINDS})")
        return None
    if kind == "dense":
        return dict(kind="dense", ff=r.positive_int(mlp, "ff", where + "mlp."))
    out = dict(kind="moe", ff=r.positive_int(mlp.get("expert"), "ff", where + "mlp.expert."),
               experts=r.positive_int(mlp.get("router"), "experts", where + "mlp.router."),
               top=r.positive_int(mlp.get("router"), "top", where + "mlp.router."))
    if out["experts"] and out["top"] > out["experts"]:
        r.bad.append(f"{where}mlp.router.top={out['top']} exceeds experts={out['experts']}")
    return out


def read_zafopel_config(cfg: dict) -> ZafopelConfig:
    r = _Reader()
    vocab, width = r.positive_int(cfg, "vocab", ""), r.positive_int(cfg, "width", "")
    eps = r.positive(cfg.get("norm"), "eps", "norm.")
    raw_layers = cfg.get("layers")
    layers = []
    if not isinstance(raw_layers, list) or not raw_layers:
        r.missing.append("layers")
        raw_layers = []
    for i, layer in enumerate(raw_layers):
        where = f"layers[{i}]."
        kind = layer.get("type") if isinstance(layer, dict) else None
        if kind not in LAYER_TYPES:
            r.bad.append(f"{where}type={kind!r} (want one of {LAYER_TYPES})")
            layers.append(None)
            continue
        m = layer.get("mixer")
        if not isinstance(m, dict):
            r.missing.append(where + "mixer")
            layers.append(None)
            continue
        layers.append(ZafopelLayer(kind, _read_mixer(r, kind, m, where + "mixer.", i),
                                   _read_mlp(r, layer.get("mlp"), where)))
    # a layer that reads another's latent rows: the source projects its own, with the same row and rotation
    for i, layer in enumerate(layers):
        src = layer.mixer.get("kv_from") if layer is not None else None
        if src is None:
            continue
        other = layers[src]
        where = f"layers[{i}].mixer.kv_from={src}"
        if other is None or other.mixer.get("kv_from") is not None:
            r.bad.append(f"{where} (the source must be a layer with a latent projection of its own)")
        elif any(other.mixer[k] != layer.mixer[k] for k in ("kv_rank", "rot_dim", "rot")):
            r.bad.append(f"{where} (kv_rank, rot_dim and rotation must equal the source's)")
    if r.missing or r.bad:
        parts = []
        if r.missing:
            parts.append("missing keys: " + ", ".join(r.missing))
        if r.bad:
            parts.append("unusable values: " + "; ".join(r.bad))
        raise ConfigError(f"unsupported {ARCHITECTURE} configuration: " + " | ".join(parts))
    return ZafopelConfig(ARCHITECTURE, vocab, width, eps, tuple(layers))
