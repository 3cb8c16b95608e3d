"""Beledra on the host: configuration, model spec, declared tensors, the tables worked out at load time,
and the cache book-keeping of its window groups.  No GPU."""
from __future__ import annotations

import copy
import json
import math

import pytest
import torch

import beledra_cases as cases
import plain_beledra as plain
from snowllm_b200.cache import CacheManager
from snowllm_b200.config.beledra import read_beledra_config
from snowllm_b200.config.registry import architectures, read_config_json
from snowllm_b200.errors import ConfigError, WeightError
from snowllm_b200.loader import build_model
from snowllm_b200.parts.attention_maps import DistanceBuckets
from snowllm_b200.parts.position import YarnRotaryPosition
from snowllm_b200.parts.spec import PagedKVSpec, SlotStateSpec
from snowllm_b200.weights.loader import load_tensors


def test_architecture_is_registered_and_read_by_its_single_name(tmp_path):
    assert "Beledra" in architectures()
    (tmp_path / "config.json").write_text(json.dumps(cases.MIXED))
    arch, cfg, _ = read_config_json(tmp_path)
    assert arch.name == "Beledra" and cfg.width == cases.MIXED["width"] and len(cfg.layers) == 5
    assert read_beledra_config(cfg.to_json_dict()) == cfg           # the written form reads back


def test_every_problem_of_a_configuration_is_listed_at_once():
    bad = copy.deepcopy(cases.MIXED)
    del bad["vocab"]
    bad["layers"][0]["mixer"]["heads"] = 3                          # no multiple of kv_heads
    bad["layers"][1]["mixer"]["rot"]["dims"] = 7
    bad["layers"][2]["mixer"].pop("gate_cap")
    bad["layers"][3]["mixer"]["kv_from"] = 2                        # an mlstm layer has no keys
    with pytest.raises(ConfigError) as e:
        read_beledra_config(bad)
    text = str(e.value)
    for piece in ("vocab", "heads=3", "rot.dims=7", "gate_cap", "kv_from=2"):
        assert piece in text, (piece, text)


def test_reader_of_keys_must_match_its_source():
    bad = copy.deepcopy(cases.MIXED)
    bad["layers"][3]["mixer"]["vdim"] = 48
    with pytest.raises(ConfigError, match="must equal the source"):
        read_beledra_config(bad)


def test_model_spec_shares_the_cache_and_keeps_the_widest_window():
    model = build_model(cases.MIXED, "float32")
    run = model.spec.run
    assert [e.cache_of for e in run] == [None, None, None, 1, None]
    specs = model.cache_specs()
    assert set(specs) == {0, 1, 2, 4}
    # layer 1 sees 19 positions, its reader 27: the cache keeps 27, each layer masks its own
    assert specs[1] == PagedKVSpec(1, 2 * 16, 27, 40, separate=True)
    assert model.blocks[1].mixer.window == 19 and model.blocks[3].mixer.window == 27
    assert specs[0] == PagedKVSpec(2, 16, 21, 24, separate=True)
    assert isinstance(specs[2], SlotStateSpec) and specs[2].shapes == ((2, 8, 24), (2, 8), (2,))
    assert specs[2].dtypes == ("f32", "f32", "f32")
    # keys and values of equal width still get pools of their own
    assert len(specs[4].pool_shapes(3, 16)) == 2 and not specs[4].fused
    assert model.blocks[2].ffn is None and model.blocks[0].ffn.activation == "relu"


def test_declared_tensors_and_their_names():
    model = build_model(cases.MIXED, "float32")
    names = {s.name: s for _, s in model.declare(lambda n: False)}
    assert names["l0.mix.rel"].shape == (12, 4)
    assert names["l1.mix.k"].shape == (1 * 2 * 16, 32) and names["l1.mix.q"].shape == (2 * 2 * 16, 32)
    assert "l3.mix.k" not in names and "l3.mix.v" not in names and "l3.mix.k.norm" not in names
    assert {"l3.mix.q", "l3.mix.q.norm", "l3.mix.g", "l3.mix.o", "l3.mix.lq1", "l3.mix.lk2"} <= set(names)
    assert names["l2.mix.i.b"].shape == (2,) and "l2.norm2" not in names and "l2.mlp.gate" not in names
    assert {"embed", "head", "final.norm", "l4.norm2", "l4.mlp.down"} <= set(names)


def test_bias_table_rows_come_from_the_checkpoint():
    cfg = copy.deepcopy(cases.MIXED)
    for layer in cfg["layers"]:
        layer["mixer"].pop("bias_rows", None)
    tensors = cases.draw_weights(cases.MIXED, dtype=torch.float32)        # tables of 12 and 6 rows
    model = build_model(cfg, "float32")
    load_tensors(model, tensors, "cpu")
    assert model.blocks[0].mixer.buckets.rows == 12 and model.blocks[4].mixer.buckets.rows == 6
    assert model.blocks[0].mixer.bias.shape == (4, 21)                    # [heads, window]
    del tensors["l3.mix.lq1"]
    tensors["l3.mix.k"] = torch.zeros(32, 32)
    with pytest.raises(WeightError) as e:
        load_tensors(build_model(cfg, "float32"), tensors, "cpu")
    assert "l3.mix.lq1" in str(e.value) and "l3.mix.k" in str(e.value)


@pytest.mark.parametrize("rows,far", [(12, 40), (24, 200), (6, 17), (8, 64), (16, 128), (2, 5), (9, 30.5)])
def test_distance_buckets_follow_the_formula(rows, far):
    b = DistanceBuckets(rows, far)
    for n in range(0, 400):
        assert b.bucket(n) == plain.distance_bucket(n, rows, far) or _exact_step(n, rows, far), (n, rows, far)
    sat = b.saturation()
    assert b.bucket(sat) == rows - 1 and (sat == rows // 2 or b.bucket(sat - 1) < rows - 1)
    assert all(b.bucket(n) == rows - 1 for n in range(sat, sat + 50))
    assert b.table(5) == [b.bucket(n) for n in range(5)]


def _exact_step(n, rows, far) -> bool:
    """Distances at which the formula's step is a whole number in exact arithmetic (floating point may land
    on either side): the product's table takes the upper bucket there."""
    half = rows // 2
    if n < half:
        return False
    step = math.log(n / half) / math.log(far / half) * (rows - half)
    return abs(step - round(step)) < 1e-9


def test_an_exact_step_takes_the_upper_bucket():
    b = DistanceBuckets(8, 64)                # half 4, ratio 16, 4 steps: distance 8 is step 1 exactly
    assert [b.bucket(n) for n in (7, 8, 15, 16, 31, 32, 63, 64, 1000)] == [4, 5, 5, 6, 6, 7, 7, 7, 7]


@pytest.mark.parametrize("rot", [
    {"dims": 8, "base": 500.0, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}},
    {"dims": 20, "base": 50000.0, "scaling": {"factor": 3.0, "original": 4096, "fast": 16.0, "slow": 2.0}},
    {"dims": 16, "base": 10000.0, "scaling": {"factor": 8.0, "original": 512, "fast": 4.0, "slow": 0.5}},
    {"dims": 6, "base": 100.0},
])
def test_yarn_table_follows_the_formula(rot):
    sc = rot.get("scaling") or {}
    pos = YarnRotaryPosition(head_dim=32, theta=rot["base"], rot_dim=rot["dims"], factor=sc.get("factor", 1.0),
                             original=sc.get("original"), fast=sc.get("fast", 32.0), slow=sc.get("slow", 1.0))
    want, magnitude = plain.yarn_frequencies(rot)
    got, dims = pos.rotary("cpu")
    assert dims == rot["dims"] and got.dtype == torch.float32
    assert torch.allclose(got.double(), torch.tensor(want, dtype=torch.float64), rtol=1e-7, atol=0)
    assert pos.magnitude == pytest.approx(magnitude, rel=1e-12)
    if sc:
        assert got[0] == pytest.approx(1.0)                       # the fastest pair keeps its frequency
        assert got[-1] < want[-1] * 1.0001


def test_window_groups_give_pages_back_and_take_them_again():
    model = build_model(cases.MIXED, "float32")
    cache = CacheManager(model.cache_specs(), 8, 12, 2, torch.float32, device=None)
    assert set(cache.groups) == {("paged", 21), ("paged", 27), ("paged", 33)}
    a = cache.admit()
    assert cache.ensure(a, 50)
    cache.commit(a, 50)
    # positions a query at 50 can still reach: from 50 - W + 1 on
    for (_, w), table in a.tables.items():
        first = (50 - w + 1) // 8
        assert all(p < 0 for p in table[:first]) and all(p >= 0 for p in table[first:7]), (w, table)
    held = {k: p.held() for k, p in cache.groups.items()}
    b = cache.admit()
    assert cache.ensure(b, 40)
    cache.commit(b, 40)
    assert cache.admit() is None                                   # two slots
    cache.free(a)
    assert {k: p.held() for k, p in cache.groups.items()} != held
    c = cache.admit()
    assert c is not None and c.slot == a.slot                      # the slot is used again
    assert cache.ensure(c, 30)
    cache.free(b)
    cache.free(c)
    assert all(p.held() == 0 for p in cache.groups.values())


def test_plain_implementation_is_causal_and_respects_each_window():
    """The oracle itself: a token beyond every window and the memory's reach cannot matter to attention-only
    models; the last token's logits do change when a token just inside the widest window changes."""
    cfg = cases.config([cases.attention_layer(window=9, ff=16), cases.diff_layer(window=7, ff=None)])
    tensors = {k: v.double() for k, v in cases.draw_weights(cfg, dtype=torch.float32).items()}
    toks = cases.tokens_for(cfg, 40)
    base = cases.plain_logits(cfg, tensors, toks)
    other = list(toks)
    other[39 - (9 - 1) - (7 - 1) - 1] = (other[39 - 15] + 1) % cfg["vocab"]     # one step beyond both windows chained
    assert torch.equal(cases.plain_logits(cfg, tensors, other)[-1], base[-1])
    other = list(toks)
    other[39 - (9 - 1) - (7 - 1)] = (other[39 - 14] + 1) % cfg["vocab"]         # the farthest token that can matter
    assert not torch.equal(cases.plain_logits(cfg, tensors, other)[-1], base[-1])
    assert torch.equal(cases.plain_logits(cfg, tensors, toks[:25]), base[:25])  # causal


def test_bench_design_option_builds_both_models_at_equal_size():
    import bench
    for width, layers, ff in bench.DESIGN_SIZES.values():
        ours = build_model(bench._beledra(width, layers, ff), "bfloat16")
        theirs = build_model(bench._lfm2_like(width, layers, ff), "bfloat16")
        assert len(ours.run) == len(theirs.run) == layers
        assert ours.spec.hidden_size == theirs.spec.hidden_size == width
        kinds = [type(b.mixer).__name__ for b in ours.blocks]
        assert {"BiasAttention", "DiffAttention", "MLstm"} == set(kinds)
        assert any(e.cache_of is not None for e in ours.run)


def test_command_line_writes_a_model_folder_that_the_loader_accepts(tmp_path):
    """``random-weights`` through the command line's own entry point, then the folder against the model's
    declarations (names, shapes, the bias table's rows from the optional key)."""
    from snowllm_b200 import cli
    from snowllm_b200.weights.loader import check_against
    from snowllm_b200.weights.safetensors_io import Checkpoint
    src = tmp_path / "config.json"
    src.write_text(json.dumps(cases.MIXED))
    out = tmp_path / "model"
    assert cli.main(["random-weights", str(src), str(out), "--seed", "3"]) == 0
    arch, cfg, _ = read_config_json(out)
    assert arch.name == "Beledra" and cfg == read_beledra_config(cases.MIXED)
    model = build_model(out, "bfloat16")
    ck = Checkpoint(out)
    try:
        check_against([s for _, s in model.declare(ck.has)], ck.names(), ck.meta)
        assert tuple(ck.meta("l0.mix.rel")[1]) == (12, 4) and tuple(ck.meta("l2.mix.i.b")[1]) == (2,)
    finally:
        ck.close()
