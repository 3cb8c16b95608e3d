"""Beledra as data: configuration -> ModelSpec.

A stack of layers whose norms sit on the sublayers' outputs (block ``output_norm``), each with one of
three mixers (``bias_attention``, ``diff_attention``, ``mlstm``) and a gated feed-forward with relu (or
none).  Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.<what>``,
``l<i>.mlp.{gate,up,down}``, ``final.norm``, ``head``.  A diff_attention layer with ``kv_from`` reads the
cache of the layer it names (run entry ``cache_of``), which then keeps the widest window among itself
and its readers.  This file only names parts and passes them their constants."""
from __future__ import annotations

from ..config.beledra import ARCHITECTURE, BeledraConfig, read_beledra_config
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunEntry

FF_ACTIVATION = "relu"


def _kept_windows(c: BeledraConfig) -> dict:
    """{layer that owns a cache -> positions its cache keeps}: its own window, or the widest among the
    layers that read its keys and values (None: every position)."""
    kept = {}
    for i, layer in enumerate(c.layers):
        if layer.type == "mlstm":
            continue
        owner = layer.mixer.get("kv_from")
        owner = i if owner is None else owner
        w = layer.mixer["window"]
        if owner not in kept:
            kept[owner] = w
        elif kept[owner] is not None:
            kept[owner] = None if w is None else max(kept[owner], w)
    return kept


def beledra_model_spec(c: BeledraConfig) -> ModelSpec:
    W, eps = c.width, c.norm_eps
    kept = _kept_windows(c)
    layers, run = [], []
    for i, layer in enumerate(c.layers):
        p, m = f"l{i}.mix.", layer.mixer
        cache_of = None
        if layer.type == "mlstm":
            mixer = PartSpec("mlstm",
                             dict(hidden_size=W, num_heads=m["heads"], head_dim=m["dim"], v_head_dim=m["vdim"],
                                  gate_cap=m["gate_cap"], head_norm_eps=eps),
                             dict(q_proj=p + "q", k_proj=p + "k", v_proj=p + "v", gate_proj=p + "g",
                                  out_proj=p + "o", norm=p + "norm", i_proj=p + "i", i_bias=p + "i.b",
                                  f_proj=p + "f", f_bias=p + "f.b"))
        else:
            cache_of = m.get("kv_from")
            owner = i if cache_of is None else cache_of
            common = dict(hidden_size=W, num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"],
                          v_head_dim=m["vdim"], scale=m["scale"], qk_norm_eps=eps, window=m["window"],
                          cache_window=kept[owner], reads_cache=cache_of is not None)
            names = dict(q_proj=p + "q", k_proj=p + "k", v_proj=p + "v", out_proj=p + "o",
                         q_norm=p + "q.norm", k_norm=p + "k.norm")
            if layer.type == "attention":
                mixer = PartSpec("bias_attention",
                                 dict(common, bias_far=m["bias_max"], bias_rows=m.get("bias_rows")),
                                 dict(names, rel=p + "rel"))
            else:
                rot = m.get("rot")
                position = {"kind": "none"}
                if rot is not None:
                    sc = rot.get("scaling") or {}
                    position = dict(kind="yarn", head_dim=m["dim"], theta=rot["base"], rot_dim=rot["dims"],
                                    factor=sc.get("factor", 1.0), original=sc.get("original"),
                                    fast=sc.get("fast", 32.0), slow=sc.get("slow", 1.0))
                mixer = PartSpec("diff_attention",
                                 dict(common, offset=m["diff"], head_norm_eps=eps, position=position),
                                 dict(names, gate_proj=p + "g", lq1=p + "lq1", lk1=p + "lk1", lq2=p + "lq2",
                                      lk2=p + "lk2"))
        norm = lambda name: PartSpec("rmsnorm", dict(size=W, eps=eps), dict(weight=name))
        ffn = ffn_norm = None
        if layer.mlp is not None:
            f = f"l{i}.mlp."
            ffn = PartSpec("gated", dict(hidden_size=W, intermediate_size=layer.mlp["ff"], activation=FF_ACTIVATION),
                           dict(gate=f + "gate", up=f + "up", down=f + "down"))
            ffn_norm = norm(f"l{i}.norm2")
        layers.append(LayerSpec("output_norm", mixer, ffn, norm(f"l{i}.norm1"), ffn_norm))
        run.append(RunEntry(i, cache_of))
    embedding = PartSpec("embedding", dict(vocab_size=c.vocab, hidden_size=W), dict(weight="embed"))
    head = PartSpec("linear_head", dict(vocab_size=c.vocab, hidden_size=W, tied=False), dict(weight="head"))
    return ModelSpec(architecture=c.architecture, vocab_size=c.vocab, hidden_size=W, embedding=embedding,
                     layers=layers, run=run, final_norm=norm("final.norm"), head=head)


register_architecture(ARCHITECTURE, read_beledra_config, beledra_model_spec)
