"""Zafopel as data: configuration -> ModelSpec.

A stack of parallel layers (block ``parallel``: one Dynamic Tanh norm, mixer and feed-forward both read its
output, x += mixer(h) + ff(h)).  The mixers are latent attention in two forms (``latent_attention``: direct
queries, a sliding window, optionally on another layer's cached rows; ``latent_attention_2``: queries
through a normalised latent, causal, a sink per head); the feed-forward is an ungated product pair with the
square of relu (``mlp``), sigmoid-routed experts whose weight multiplies their input (``sigmoid_moe`` with
``scale_input``), or none.  Tensor names: ``embed``, ``l<i>.norm1{,.b,.alpha}``, ``l<i>.mix.<what>``,
``l<i>.mlp.{up,down}`` or ``l<i>.mlp.{router, e<j>.{gate,up,down}}``, ``final.norm{,.b,.alpha}``, ``head``.
This file only names parts and passes them their constants."""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.zafopel import ARCHITECTURE, ZafopelConfig, read_zafopel_config
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunEntry

DENSE_ACTIVATION = "relu2"       # the dense feed-forward's activation: the square of relu


def _kept_windows(c: ZafopelConfig) -> dict:
    """{layer that owns a cache -> positions its cache keeps}: its own window, or the widest among the
    layers that read its rows (None: every position)."""
    kept = {}
    for i, layer in enumerate(c.layers):
        owner = layer.mixer["kv_from"]
        owner = i if owner is None else owner
        w = layer.mixer["window"]
        if owner not in kept:
            kept[owner] = w
        elif kept[owner] is not None:
            kept[owner] = None if w is None else max(kept[owner], w)
    return kept


def zafopel_model_spec(c: ZafopelConfig) -> ModelSpec:
    W, eps = c.width, c.norm_eps
    kept = _kept_windows(c)

    def norm(name):
        return PartSpec("dyt", dict(size=W), dict(weight=name, bias=name + ".b", alpha=name + ".alpha"))
    layers, run = [], []
    for i, layer in enumerate(c.layers):
        p, m = f"l{i}.mix.", layer.mixer
        cache_of = m["kv_from"]
        owner = i if cache_of is None else cache_of
        second = layer.type == "latent_attention_2"
        mixer = PartSpec(
            "latent_attention",
            dict(hidden_size=W, num_heads=m["heads"], head_dim=m["dim"], rot_dim=m["rot_dim"], v_head_dim=m["vdim"],
                 kv_rank=m["kv_rank"], q_rank=m["q_rank"], scale=m["scale"], norm_eps=eps,
                 position=dict(kind="rope_pairs", head_dim=m["rot_dim"], theta=m["rot"]["base"],
                               rot_dim=m["rot"]["dims"]),
                 window=m["window"], cache_window=kept[owner], sink=second, reads_cache=cache_of is not None),
            dict(q=p + "q", dq=p + "dq", dq_norm=p + "dq.norm", uq=p + "uq", dkv=p + "dkv",
                 dkv_norm=p + "dkv.norm", uk=p + "uk", uv=p + "uv", o=p + "o", sink=p + "sink"))
        ffn = None
        if layer.mlp is not None:
            f = f"l{i}.mlp."
            if layer.mlp["kind"] == "dense":
                ffn = PartSpec("mlp", dict(hidden_size=W, intermediate_size=layer.mlp["ff"],
                                           activation=DENSE_ACTIVATION), dict(up=f + "up", down=f + "down"))
            else:
                ffn = PartSpec("sigmoid_moe",
                               dict(hidden_size=W, intermediate_size=layer.mlp["ff"],
                                    num_experts=layer.mlp["experts"], top_k=layer.mlp["top"], norm_topk_prob=False,
                                    use_expert_bias=False, routed_scaling_factor=1.0, scale_input=True),
                               dict(router=f + "router", experts=f + "e", expert_gate="gate", expert_up="up",
                                    expert_down="down", fused_gate_up=f + "gate_up", fused_down=f + "down_all"))
        layers.append(LayerSpec("parallel", mixer, ffn, norm(f"l{i}.norm1"), None))
        run.append(RunEntry(i, cache_of))
    embedding = PartSpec("embedding", dict(vocab_size=c.vocab, hidden_size=W), dict(weight="embed"))
    head = PartSpec("linear_head", dict(vocab_size=c.vocab, hidden_size=W, tied=False), dict(weight="head"))
    return ModelSpec(architecture=c.architecture, vocab_size=c.vocab, hidden_size=W, embedding=embedding,
                     layers=layers, run=run, final_norm=norm("final.norm"), head=head)


register_architecture(ARCHITECTURE, read_zafopel_config, zafopel_model_spec)
