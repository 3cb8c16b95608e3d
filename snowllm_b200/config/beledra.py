"""Typed configuration of the Beledra design, read from its config.json.

    {"architecture": "Beledra", "vocab": V, "width": W, "norm": {"eps": e},
     "layers": [{"type": T, "mixer": {...}, "mlp": {"kind": "dense", "ff": F} | null}, ...]}

``type`` names the layer's mixer; ``mixer`` holds that mixer's sizes and constants:

* ``attention``:   heads, kv_heads, dim, vdim, scale, mask.size, bias_max (distance at which the bias
                   table's buckets reach their last row; the table's rows are the tensor's; ``bias_rows``
                   is an optional key for weights that are drawn, not read)
* ``attention_2``: heads, kv_heads, dim, vdim, scale, mask.size, diff, rot {dims, base, scaling {factor,
                   original, fast, slow}}, kv_from (optional: the layer whose keys and values it reads)
* ``mlstm``:       heads, dim, vdim, gate_cap

Every size and constant comes from the file (or, for the bias table's rows, from the tensor's shape);
what is missing or unusable is reported in one ConfigError that lists every key."""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any

from ..errors import ConfigError

ARCHITECTURE = "Beledra"
LAYER_TYPES = ("attention", "attention_2", "mlstm")
MLP_KINDS = ("dense",)


@dataclass(frozen=True)
class BeledraLayer:
    type: str
    mixer: dict
    mlp: dict | None


@dataclass(frozen=True)
class BeledraConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    layers: tuple

    def to_json_dict(self) -> dict[str, Any]:
        """config.json content that reads back to this configuration."""
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.norm_eps},
                "layers": [{"type": l.type, "mixer": _mixer_json(l), "mlp": copy.deepcopy(l.mlp)}
                           for l in self.layers]}


def _mixer_json(layer: BeledraLayer) -> dict:
    """The mixer's keys as config.json spells them (the typed form keeps ``window`` for mask.size)."""
    m = copy.deepcopy(layer.mixer)
    if layer.type == "mlstm":
        return m
    window = m.pop("window", None)
    if window is not None:
        m["mask"] = {"size": window}
    for key in ("kv_from", "rot", "bias_rows"):
        if key in m and m[key] is None:
            del m[key]
    if m.get("rot") is not None and m["rot"].get("scaling") is None:
        del m["rot"]["scaling"]
    return m


def _is_int(v) -> bool:
    return isinstance(v, int) and not isinstance(v, bool)


def _is_num(v) -> bool:
    return isinstance(v, (int, float)) and not isinstance(v, bool)


class _Reader:
    def __init__(self):
        self.missing: list[str] = []
        self.bad: list[str] = []

    def positive_int(self, d, key, where):
        v = d.get(key) if isinstance(d, dict) else None
        if v is None:
            self.missing.append(where + key)
            return 0
        if not _is_int(v) or v <= 0:
            self.bad.append(f"{where}{key}={v!r} (want a positive integer)")
            return 0
        return v

    def positive(self, d, key, where):
        v = d.get(key) if isinstance(d, dict) else None
        if v is None:
            self.missing.append(where + key)
            return 0.0
        if not _is_num(v) or not v > 0:
            self.bad.append(f"{where}{key}={v!r} (want a positive number)")
            return 0.0
        return float(v)

    def number(self, d, key, where):
        v = d.get(key) if isinstance(d, dict) else None
        if v is None:
            self.missing.append(where + key)
            return 0.0
        if not _is_num(v):
            self.bad.append(f"{where}{key}={v!r} (want a number)")
            return 0.0
        return float(v)


def _read_window(r: _Reader, m: dict, where: str):
    mask = m.get("mask")
    if mask is None:
        return None
    return r.positive_int(mask, "size", where + "mask.") or None


def _read_attention_common(r: _Reader, m: dict, where: str) -> dict:
    out = dict(heads=r.positive_int(m, "heads", where), kv_heads=r.positive_int(m, "kv_heads", where),
               dim=r.positive_int(m, "dim", where), vdim=r.positive_int(m, "vdim", where),
               scale=r.positive(m, "scale", where), window=_read_window(r, m, where))
    if out["heads"] and out["kv_heads"] and out["heads"] % out["kv_heads"]:
        r.bad.append(f"{where}heads={out['heads']} is no multiple of kv_heads={out['kv_heads']}")
    return out


def _read_rot(r: _Reader, m: dict, where: str, dim: int):
    rot = m.get("rot")
    if rot is None:
        return None
    w = where + "rot."
    out = dict(dims=r.positive_int(rot, "dims", w), base=r.positive(rot, "base", w), scaling=None)
    if out["dims"] and (out["dims"] % 2 or (dim and out["dims"] > dim)):
        r.bad.append(f"{w}dims={out['dims']} (want an even number, at most dim={dim})")
    if out["base"] == 1.0:
        r.bad.append(f"{w}base=1 (the frequencies need a base other than 1)")
    sc = rot.get("scaling")
    if sc is not None:
        ws = w + "scaling."
        out["scaling"] = dict(factor=r.positive(sc, "factor", ws), original=r.positive(sc, "original", ws),
                              fast=r.positive(sc, "fast", ws), slow=r.positive(sc, "slow", ws))
    return out


def read_beledra_config(cfg: dict) -> BeledraConfig:
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
            continue
        m = layer.get("mixer")
        if not isinstance(m, dict):
            r.missing.append(where + "mixer")
            continue
        w = where + "mixer."
        if kind == "attention":
            mixer = _read_attention_common(r, m, w)
            mixer["bias_max"] = r.positive(m, "bias_max", w)
            # optional: the bias table's rows, for weights that are drawn rather than read (a checkpoint's
            # table says it by its shape)
            mixer["bias_rows"] = r.positive_int(m, "bias_rows", w) if m.get("bias_rows") is not None else None
        elif kind == "attention_2":
            mixer = _read_attention_common(r, m, w)
            mixer["diff"] = r.number(m, "diff", w)
            mixer["rot"] = _read_rot(r, m, w, mixer["dim"])
            src = m.get("kv_from")
            if src is not None and (not _is_int(src) or not 0 <= src < i):
                r.bad.append(f"{w}kv_from={src!r} (want an earlier layer)")
                src = None
            mixer["kv_from"] = src
        else:
            mixer = dict(heads=r.positive_int(m, "heads", w), dim=r.positive_int(m, "dim", w),
                         vdim=r.positive_int(m, "vdim", w), gate_cap=r.positive(m, "gate_cap", w))
        mlp = layer.get("mlp")
        if mlp is not None:
            if not isinstance(mlp, dict) or mlp.get("kind") not in MLP_KINDS:
                r.bad.append(f"{where}mlp.kind={mlp.get('kind') if isinstance(mlp, dict) else mlp!r} "
                             f"(want one of {MLP_KINDS})")
                mlp = None
            else:
                mlp = dict(kind=mlp["kind"], ff=r.positive_int(mlp, "ff", where + "mlp."))
        layers.append(BeledraLayer(kind, mixer, mlp))
    # a layer that reads another's keys and values: the source has projections of its own and the same shape
    for i, layer in enumerate(layers):
        src = layer.mixer.get("kv_from") if layer.type == "attention_2" else None
        if src is None or src >= len(layers):
            continue
        other = layers[src]
        where = f"layers[{i}].mixer.kv_from={src}"
        if other.type != "attention_2" or other.mixer.get("kv_from") is not None:
            r.bad.append(f"{where} (the source must be an attention_2 layer with keys and values of its own)")
        elif any(other.mixer[k] != layer.mixer[k] for k in ("heads", "kv_heads", "dim", "vdim", "rot")):
            r.bad.append(f"{where} (head counts, sizes and rotation must equal the source's)")
    if r.missing or r.bad:
        parts = []
        if r.missing:
            parts.append("missing keys: " + ", ".join(r.missing))
        if r.bad:
            parts.append("unusable values: " + "; ".join(r.bad))
        raise ConfigError(f"unsupported {ARCHITECTURE} configuration: " + " | ".join(parts))
    return BeledraConfig(ARCHITECTURE, vocab, width, eps, tuple(layers))
