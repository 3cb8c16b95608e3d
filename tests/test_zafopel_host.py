"""Zafopel on the host: configuration, model spec, declared tensors, the rotary table, the cache book-keeping
of its window groups, and the plain implementation's own properties.  No GPU."""
from __future__ import annotations

import copy
import json
import math

import pytest
import torch

import plain_zafopel as plain
import zafopel_cases as cases
from snowllm_b200.cache import CacheManager
from snowllm_b200.config.registry import architectures, read_config_json
from snowllm_b200.config.zafopel import read_zafopel_config
from snowllm_b200.errors import ConfigError, WeightError
from snowllm_b200.loader import build_model
from snowllm_b200.parts.position import PairedRotaryPosition
from snowllm_b200.parts.spec import PagedKVSpec
from snowllm_b200.weights.loader import load_tensors


def test_architecture_is_registered_and_read_by_its_single_name(tmp_path):
    assert "Zafopel" in architectures()
    (tmp_path / "config.json").write_text(json.dumps(cases.MIXED))
    arch, cfg, _ = read_config_json(tmp_path)
    assert arch.name == "Zafopel" and cfg.width == cases.MIXED["width"] and len(cfg.layers) == 5
    assert read_zafopel_config(cfg.to_json_dict()) == cfg           # the written form reads back
    assert cfg.layers[1].mlp == {"kind": "moe", "ff": 24, "experts": 5, "top": 2} and cfg.layers[3].mlp is None


def test_every_problem_of_a_configuration_is_listed_at_once():
    bad = copy.deepcopy(cases.MIXED)
    del bad["width"]
    bad["layers"][0]["mixer"].pop("q_rank")
    bad["layers"][1]["mixer"]["rot"]["dims"] = 7
    bad["layers"][2]["mlp"]["router"]["top"] = 9                    # more picks than experts
    bad["layers"][3]["mixer"]["kv_from"] = 3                        # not an earlier layer
    bad["layers"][4]["mlp"]["kind"] = "gated"
    with pytest.raises(ConfigError) as e:
        read_zafopel_config(bad)
    text = str(e.value)
    for piece in ("width", "q_rank", "rot.dims=7", "top=9", "kv_from=3", "'gated'"):
        assert piece in text, (piece, text)


def test_reader_of_rows_must_match_its_source():
    bad = copy.deepcopy(cases.MIXED)
    bad["layers"][3]["mixer"]["kv_rank"] = 48
    with pytest.raises(ConfigError, match="must equal the source"):
        read_zafopel_config(bad)
    bad = copy.deepcopy(cases.MIXED)
    bad["layers"][4]["mixer"]["kv_from"] = 3                        # layer 3 reads layer 1 itself
    with pytest.raises(ConfigError, match="latent projection of its own"):
        read_zafopel_config(bad)


def test_model_spec_shares_the_cache_and_keeps_the_widest_window():
    model = build_model(cases.MIXED, "float32")
    assert [e.cache_of for e in model.spec.run] == [None, None, None, 1, None]
    assert all(layer.block == "parallel" and layer.ffn_norm is None for layer in model.spec.layers)
    specs = model.cache_specs()
    assert set(specs) == {0, 1, 2, 4}
    # one row of kv_rank + rot_dim per position for all heads, keys only; layer 1 sees 19 positions, its
    # reader 27: the cache keeps 27, each layer masks its own; causal layers keep everything
    assert specs[1] == PagedKVSpec(1, 40 + 8, 27, 0)
    assert specs[1].pool_shapes(5, 16) == ((5, 1, 16, 48),)
    assert specs[0] == PagedKVSpec(1, 48 + 16, None, 0) and specs[4] == PagedKVSpec(1, 36 + 12, 33, 0)
    mixers = [b.mixer for b in model.blocks]
    assert mixers[1].window == 19 and mixers[3].window == 27 and mixers[0].window is None
    assert [m.sink_on for m in mixers] == [True, False, True, False, False]
    assert [m.q_rank for m in mixers] == [28, None, 12, None, None]
    assert mixers[3].reads_cache and not mixers[1].reads_cache
    assert model.blocks[3].ffn is None and model.blocks[0].ffn.activation == "relu2"
    moe = model.blocks[1].ffn
    assert moe.scale_input and not moe.norm_topk_prob and moe.top_k == 2 and moe.num_experts == 5
    assert mixers[4].position.rot_dim == 8 and mixers[4].rot_dim == 12          # part of the rotated slice turns


def test_declared_tensors_and_their_names():
    model = build_model(cases.MIXED, "float32")
    names = {s.name: s for _, s in model.declare(lambda n: False)}
    assert names["l0.mix.dq"].shape == (28, 32) and names["l0.mix.uq"].shape == (2 * 32, 28)
    assert names["l0.mix.dq.norm"].shape == (28,) and names["l0.mix.sink"].shape == (2,)
    assert names["l1.mix.q"].shape == (3 * 32, 32) and names["l1.mix.dkv"].shape == (48, 32)
    assert names["l1.mix.uk"].shape == (3 * 24, 40) and names["l1.mix.uv"].shape == (3 * 20, 40)
    assert "l1.mix.sink" not in names and "l1.mix.dq" not in names
    assert "l3.mix.dkv" not in names and "l3.mix.dkv.norm" not in names and "l3.mix.q" in names
    assert names["l0.norm1.alpha"].shape == () and names["final.norm.b"].shape == (32,)
    assert not any(n.startswith("l3.mlp") for n in names) and "l0.norm2" not in names
    assert {"l1.mlp.router", "l1.mlp.e4.gate", "l1.mlp.e0.down", "l4.mlp.up", "l4.mlp.down"} <= set(names)
    assert "l1.mlp.e5.gate" not in names and names["l2.mlp.e2.up"].shape == (16, 32)


def test_missing_and_unexpected_tensors_are_listed():
    tensors = cases.draw_weights(cases.MIXED, dtype=torch.float32)
    del tensors["l2.mix.sink"]
    tensors["l3.mix.dkv"] = torch.zeros(48, 32)
    with pytest.raises(WeightError) as e:
        load_tensors(build_model(cases.MIXED, "float32"), tensors, "cpu")
    assert "l2.mix.sink" in str(e.value) and "l3.mix.dkv" in str(e.value)


@pytest.mark.parametrize("base,dims", [(300.0, 8), (5000.0, 16), (500000.0, 6), (2.0, 2)])
def test_paired_rotary_table_follows_the_formula(base, dims):
    got, n = PairedRotaryPosition(head_dim=dims + 4, theta=base, rot_dim=dims).rotary("cpu")
    assert n == dims and got.dtype == torch.float32 and got[0] == 1.0
    want = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float64)
    assert torch.allclose(got.double(), want, rtol=6e-8, atol=0)


def test_rotation_of_pairs_keeps_lengths_and_depends_on_distance_only():
    g = torch.Generator().manual_seed(1)
    q, k = torch.randn(1, 10, generator=g).double(), torch.randn(1, 10, generator=g).double()
    def at(x, p):
        return plain.rotate_pairs(x, torch.tensor([p]), 300.0, 6)
    assert torch.allclose(at(q, 7)[:, :6].norm(), q[:, :6].norm())
    assert torch.equal(at(q, 7)[:, 6:], q[:, 6:])                               # the rest passes unchanged
    a = (at(q, 40) * at(k, 33)).sum()
    b = (at(q, 107) * at(k, 100)).sum()
    assert float((a - b).abs()) < 1e-12
    # element 0 turns with element 1: a vector along 0 moves into 1 by sin
    e0 = torch.zeros(1, 6).double()
    e0[0, 0] = 1
    assert torch.allclose(at(e0, 1)[0, :2], torch.tensor([math.cos(1.0), math.sin(1.0)], dtype=torch.float64))


def test_window_groups_give_pages_back_and_take_them_again():
    model = build_model(cases.MIXED, "float32")
    cache = CacheManager(model.cache_specs(), 8, 12, 2, torch.float32, device=None)
    assert set(cache.groups) == {("paged", None), ("paged", 27), ("paged", 33)}
    a = cache.admit()
    assert cache.ensure(a, 50)
    cache.commit(a, 50)
    for (_, w), table in a.tables.items():
        first = 0 if w is None else (50 - w + 1) // 8
        assert all(p < 0 for p in table[:first]) and all(p >= 0 for p in table[first:7]), (w, table)
    b = cache.admit()
    assert cache.ensure(b, 40)
    cache.commit(b, 40)
    assert cache.admit() is None                                   # two slots
    assert not cache.ensure(b, 60)                                 # the group that keeps everything is full
    cache.free(a)
    c = cache.admit()
    assert c is not None and c.slot == a.slot                      # the slot is used again
    assert cache.ensure(c, 30)
    cache.free(b)
    cache.free(c)
    assert all(p.held() == 0 for p in cache.groups.values())


def test_plain_implementation_is_causal_respects_the_window_and_counts_the_sink_once():
    cfg = cases.config([cases.window_layer(window=9, mlp=cases.dense(16)), cases.window_layer(window=7, mlp=None)])
    tensors = {k: v.double() for k, v in cases.draw_weights(cfg, dtype=torch.float32).items()}
    toks = cases.tokens_for(cfg, 40)
    base = cases.plain_logits(cfg, tensors, toks)
    other = list(toks)
    other[39 - 15] = (other[39 - 15] + 1) % cfg["vocab"]            # one step beyond both windows chained
    assert torch.equal(cases.plain_logits(cfg, tensors, other)[-1], base[-1])
    other = list(toks)
    other[39 - 14] = (other[39 - 14] + 1) % cfg["vocab"]            # the farthest token that can matter
    assert not torch.equal(cases.plain_logits(cfg, tensors, other)[-1], base[-1])
    assert torch.equal(cases.plain_logits(cfg, tensors, toks[:25]), base[:25])  # causal
    # the sink: with one visible key of score s the weight is e^s / (e^s + e^sink)
    p = plain.softmax_rows(torch.tensor([[0.7, 5.0]], dtype=torch.float64), torch.tensor([[True, False]]),
                           torch.tensor(-0.2, dtype=torch.float64))
    assert float(p[0, 0]) == pytest.approx(math.exp(0.7) / (math.exp(0.7) + math.exp(-0.2)), rel=1e-12)
    assert float(p[0, 1]) == 0.0


def test_routed_experts_scale_their_input_not_their_output():
    g = torch.Generator().manual_seed(2)
    h = torch.randn(3, 8, generator=g).double()
    experts = [tuple(torch.randn(s, generator=g).double() for s in ((6, 8), (6, 8), (8, 6))) for _ in range(3)]
    ids, w = torch.tensor([[0, 2], [1, 0], [2, 1]]), torch.tensor([[0.9, 0.3], [0.5, 0.5], [0.2, 0.8]]).double()
    got = plain.routed_ff(h, (ids, w), experts)
    gate, up, down = experts[2]
    x = h[0] * 0.3
    second = (torch.nn.functional.silu(gate @ x) * (up @ x)) @ down.T
    gate, up, down = experts[0]
    x = h[0] * 0.9
    first = (torch.nn.functional.silu(gate @ x) * (up @ x)) @ down.T
    assert torch.allclose(got[0], first + second, atol=1e-12)
    # a gated expert is not linear in its input: the weight on the output gives something else
    x = h[0]
    unscaled = (torch.nn.functional.silu(gate @ x) * (up @ x)) @ down.T
    assert not torch.allclose(first, 0.9 * unscaled, atol=1e-6)
    ids2, w2 = plain.router_picks(h, torch.randn(4, 8, generator=g).double(), 2)
    assert ids2.shape == (3, 2) and bool((w2 > 0).all()) and bool((w2 < 1).all()) and bool((w2[:, 0] >= w2[:, 1]).all())


def test_command_line_writes_a_model_folder_that_the_loader_accepts(tmp_path):
    from snowllm_b200 import cli
    from snowllm_b200.weights.loader import check_against
    from snowllm_b200.weights.safetensors_io import Checkpoint
    src = tmp_path / "config.json"
    src.write_text(json.dumps(cases.MIXED))
    out = tmp_path / "model"
    assert cli.main(["random-weights", str(src), str(out), "--seed", "3"]) == 0
    arch, cfg, _ = read_config_json(out)
    assert arch.name == "Zafopel" and cfg == read_zafopel_config(cases.MIXED)
    model = build_model(out, "bfloat16")
    ck = Checkpoint(out)
    try:
        check_against([s for _, s in model.declare(ck.has)], ck.names(), ck.meta)
        assert tuple(ck.meta("l0.norm1.alpha")[1]) == () and tuple(ck.meta("l2.mix.sink")[1]) == (5,)
    finally:
        ck.close()


def test_bench_design_option_builds_both_models_at_equal_size():
    import bench
    name, ours_of, (other, theirs_of), _ = bench.DESIGNS["zafopel"]
    assert name == "Zafopel" and other == "lfm2_moe"
    for width, layers, ff in bench.DESIGN_SIZES.values():
        ours = build_model(ours_of(width, layers, ff), "bfloat16")
        theirs = build_model(theirs_of(width, layers, ff), "bfloat16")
        assert len(ours.run) == len(theirs.run) == layers
        assert ours.spec.hidden_size == theirs.spec.hidden_size == width
        mixers = [b.mixer for b in ours.blocks]
        assert {m.sink_on for m in mixers} == {True, False} and any(m.window for m in mixers)
        assert all(m.num_heads == theirs.blocks[0].mixer.num_heads for m in mixers)
        kinds = [type(b.ffn).__name__ for b in ours.blocks]
        assert kinds[0] == "MLP" and set(kinds[1:]) == {"SigmoidMoE"}
        routed, theirs_routed = ours.blocks[1].ffn, theirs.blocks[1].ffn
        assert (routed.num_experts, routed.top_k, routed.intermediate_size) == \
               (theirs_routed.num_experts, theirs_routed.top_k, theirs_routed.intermediate_size)
        if layers > 5:
            assert any(e.cache_of is not None for e in ours.run)
