"""Beledra on the GPU against the plain implementation (tests/plain_beledra.py): every mixer alone, the
kernels on inputs that make a wrong key or a lost state show, and one model with every mechanism fed
whole, token by token, in portions and in mixed batches over pools that are used again."""
from __future__ import annotations

import math

import pytest
import torch

import beledra_cases as cases
import plain_beledra as plain

pytestmark = pytest.mark.gpu

F32_TOL = 5e-5          # float32 engine against the float64 plain implementation (rounding of five layers)
BF16_TOL = 0.06         # bfloat16 engine against the plain implementation on the same (rounded) weights


def load(cfg, tensors, dtype):
    from snowllm_b200.loader import build_model
    from snowllm_b200.weights.loader import load_tensors
    model = build_model(cfg, dtype)
    load_tensors(model, tensors, "cuda")
    return model


def replay(model, max_tokens=512, requests=4, page_size=16):
    from snowllm_b200.engine.replay import Replay
    return Replay(model, None, max_tokens, requests, page_size=page_size)


def reference(cfg, tensors, tokens, layers_out=None, rounded=False):
    return cases.plain_logits(cfg, {k: v.double() for k, v in tensors.items()}, tokens, layers_out, rounded)


def tolerance(dtype):
    return F32_TOL if dtype == "float32" else BF16_TOL


# --- each mechanism alone -------------------------------------------------------------------------

ALONE = {
    "bias_attention": [cases.attention_layer()],
    "bias_attention_no_ff_one_kv_head": [cases.attention_layer(heads=3, kv_heads=1, dim=8, vdim=16, window=5,
                                                               bias_rows=4, bias_max=9, ff=None)],
    "bias_attention_unaligned_rows": [cases.attention_layer(heads=2, kv_heads=2, dim=12, vdim=20, window=40)],
    "bias_attention_three_heads_per_kv_head": [cases.attention_layer(heads=6, kv_heads=2, dim=16, vdim=8, window=23)],
    "diff_attention": [cases.diff_layer()],
    "diff_attention_three_heads_one_kv_head": [cases.diff_layer(heads=3, kv_heads=1, dim=32, vdim=16, rot_dims=12,
                                                                window=45)],
    "diff_attention_plain_rotation_over_the_whole_head": [cases.diff_layer(rot_dims=16, scaling=False, dim=16, vdim=32,
                                                                           heads=4, kv_heads=2, diff=0.7)],
    "diff_attention_no_rotation": [cases.diff_layer(rot_dims=0, window=64, dim=8, vdim=16)],
    "diff_attention_reader": [cases.diff_layer(window=11), cases.diff_layer(window=30, kv_from=0, ff=None)],
    "mlstm": [cases.mlstm_layer()],
    "mlstm_wide": [cases.mlstm_layer(heads=1, dim=72, vdim=300, gate_cap=4.0, ff=32)],
    "mlstm_odd": [cases.mlstm_layer(heads=3, dim=6, vdim=10, gate_cap=25.0)],
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(ALONE))
def test_each_mixer_alone(name, dtype):
    cfg = cases.config(ALONE[name])
    tensors = cases.draw_weights(cfg, seed=len(name))
    tokens = cases.tokens_for(cfg, 70)
    want_layers = []
    want = reference(cfg, tensors, tokens, want_layers)
    model = load(cfg, tensors, dtype)
    rp = replay(model)
    rp.runner.taps = []
    got = cases.run_cuts(rp, "a", tokens, [len(tokens)])
    layers = [t for n, t in rp.runner.taps if n == "layer_out"]
    assert len(layers) == len(want_layers)
    for x, w in zip(layers, want_layers):
        assert cases.relative_error(x.cpu(), w) < tolerance(dtype)
    assert cases.worst_row_error(got, want) < tolerance(dtype) * 2
    # token by token through the cache and the state gives the same
    rp.runner.taps = None
    again = cases.run_cuts(rp, "b", tokens, [1] * len(tokens))
    assert cases.worst_row_error(again, want) < tolerance(dtype) * 2


# --- the attention kernel on keys that stand out ---------------------------------------------------

def plain_attention(q, k, v, scale, window, bias=None):
    """q [T, H, dk], k [T, dk], v [T, dv] of one kv head, all float64: out [T, H, dv]."""
    T = q.shape[0]
    out = torch.zeros(T, q.shape[1], v.shape[1], dtype=torch.float64)
    for i in range(T):
        lo = max(0, i - window + 1)
        for h in range(q.shape[1]):
            s = (k[lo:i + 1] @ q[i, h]) * scale
            if bias is not None:
                s = s + torch.stack([bias[h, min(i - j, bias.shape[1] - 1)] for j in range(lo, i + 1)])
            out[i, h] = torch.softmax(s, 0) @ v[lo:i + 1]
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tiled", [False, True])
def test_attention_kernel_sees_exactly_its_window(dtype, tiled):
    """One key per row is made to stand out: placed on the window's last position inside it owns the
    output, one position further it must not be seen at all.  Pages in a scrambled order."""
    from snowllm_b200.ops import kernels
    g = torch.Generator().manual_seed(5)
    T, H, dk, dv, P, window = 150, 4, 16, 24, 16, 37
    q = torch.randn(T, H, dk, generator=g).to(dtype)
    k = (torch.randn(T, dk, generator=g) * 0.1).to(dtype)
    v = torch.randn(T, dv, generator=g).to(dtype)
    inside, outside = 120, 131
    k[inside - (window - 1)] = (q[inside, 1].float() * 6).to(dtype)        # the farthest key row 120 sees
    k[outside - window] = (q[outside, 2].float() * 6).to(dtype)            # one beyond row 121's window
    bias = (torch.randn(H, 20, generator=g) * 1.5).float()
    pages = -(-T // P)
    order = torch.randperm(pages + 3, generator=g)[:pages].int()
    kpool = torch.zeros(pages + 3, 1, P, dk, dtype=dtype, device="cuda")
    vpool = torch.zeros(pages + 3, 1, P, dv, dtype=dtype, device="cuda")
    for t in range(T):
        kpool[order[t // P], 0, t % P] = k[t]
        vpool[order[t // P], 0, t % P] = v[t]
    positions = torch.arange(T, dtype=torch.int32, device="cuda")
    row_seg = torch.zeros(T, dtype=torch.int32, device="cuda")
    table = order.view(1, -1).cuda().contiguous()
    tiles, tile_rows = None, 1
    if tiled:
        tile_rows = kernels.split_attention_tile_rows(H, 1, 1, dk, dv, dtype, False)
        starts = list(range(0, T, tile_rows))
        tiles = torch.tensor([[s, min(tile_rows, T - s)] for s in starts], dtype=torch.int32, device="cuda")
    got = kernels.split_attention(q.cuda(), kpool, vpool, table, P, positions, row_seg, 0.25, window=window,
                                  bias=bias.cuda(), tiles=tiles, tile_rows=tile_rows, out_dtype=torch.float32)
    want = plain_attention(q.double(), k.double(), v.double(), 0.25, window, bias.double())
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert float((got.cpu().double() - want).abs().max()) < tol
    assert float((want[inside, 1] - v[inside - (window - 1)].double()).abs().max()) < 0.05     # the key owns the row
    assert float((got[inside, 1].cpu().double() - v[inside - (window - 1)].double()).abs().max()) < 0.05
    assert float((got[outside, 2].cpu().double() - v[outside - window].double()).abs().max()) > 0.3


def test_attention_kernel_two_maps_share_values_and_keep_rows_apart():
    from snowllm_b200.ops import kernels
    g = torch.Generator().manual_seed(6)
    T, H, G, dk, dv, P, window = 45, 2, 2, 8, 40, 8, 13
    q = torch.randn(T, H * 2, dk, generator=g)
    k = torch.randn(T, G, 2, dk, generator=g)
    v = torch.randn(T, G, dv, generator=g)
    kpool = torch.zeros(6, G, P, 2 * dk, device="cuda")
    vpool = torch.zeros(6, G, P, dv, device="cuda")
    for t in range(T):
        kpool[t // P, :, t % P] = k[t].reshape(G, 2 * dk)
        vpool[t // P, :, t % P] = v[t]
    positions = torch.arange(T, dtype=torch.int32, device="cuda")
    table = torch.arange(6, dtype=torch.int32, device="cuda").view(1, -1)
    got = kernels.split_attention(q.cuda(), kpool, vpool, table, P, positions, torch.zeros_like(positions), 0.5,
                                  maps=2, window=window)
    for h in range(H):
        for which in range(2):
            want = plain_attention(q[:, 2 * h + which:2 * h + which + 1].double(), k[:, h, which].double(),
                                   v[:, h].double(), 0.5, window)
            assert float((got[:, 2 * h + which].cpu().double() - want[:, 0]).abs().max()) < 1e-5


# --- the elementwise kernels ----------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_add_gated_act_and_head_norm_gate(dtype):
    from snowllm_b200.ops import kernels
    g = torch.Generator().manual_seed(7)
    M, H = 9, 100
    residual, y = torch.randn(M, H, generator=g), torch.randn(M, H, generator=g) * 3
    gamma = (1 + 0.3 * torch.randn(H, generator=g)).to(dtype)
    res = residual.clone().cuda()
    x = kernels.norm_add(res, y.cuda(), gamma.cuda(), 1e-3, dtype)
    want = residual.double() + plain.rms_norm(y.double(), gamma.double(), 1e-3)
    assert float((res.cpu().double() - want).abs().max()) < 1e-5
    assert float((x.cpu().double() - want).abs().max()) < (1e-5 if dtype == torch.float32 else 0.04)
    tol = 1e-5 if dtype == torch.float32 else 0.03
    gu = torch.randn(M, 2 * 24, generator=g).to(dtype)
    for act in ("relu", "gelu_tanh", "silu"):
        got = kernels.gated_act(gu.cuda(), act)
        want = plain.ACTIVATIONS[act](gu[:, :24].double()) * gu[:, 24:].double()
        assert float((got.cpu().double() - want).abs().max()) < tol, act
    heads, dv = 3, 20
    a = torch.randn(M, heads, 2, dv, generator=g)
    gate = torch.randn(M, 7 + heads * dv, generator=g).to(dtype)
    w = torch.randn(heads * dv, generator=g).to(dtype)
    got = kernels.head_norm_gate(a.cuda(), heads, dv, 1e-2, dtype, second=dv, lam=0.8, weight=w.cuda(),
                                 gate=gate.cuda(), gate_col=7, mult=0.6)
    o = plain.rms_normalise(a[:, :, 0].double() - 0.8 * a[:, :, 1].double(), 1e-2) * 0.6
    want = o.reshape(M, -1) * w.double() * torch.sigmoid(gate[:, 7:].double())
    assert float((got.cpu().double() - want).abs().max()) < tol


# --- one model with everything: cuts, batches, reuse ------------------------------------------------

@pytest.fixture(scope="module")
def mixed():
    tensors = cases.draw_weights(cases.MIXED, seed=3)
    prompts = {n: cases.tokens_for(cases.MIXED, t, seed=i) for i, (n, t) in
               enumerate((("a", 97), ("b", 41), ("c", 70), ("d", 3)))}
    want = {n: reference(cases.MIXED, tensors, p) for n, p in prompts.items()}
    # what rounding alone costs on this model: the plain implementation's rounding variant against itself
    noise = max(cases.worst_row_error(reference(cases.MIXED, tensors, p, rounded=True), want[n])
                for n, p in prompts.items())
    BOUND["bfloat16"] = 3 * noise
    return tensors, prompts, want


BOUND = {"float32": 2 * F32_TOL}       # bfloat16: three times the measured rounding noise, set by the fixture


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_of_every_size_agree_with_the_whole_prompt(mixed, dtype):
    tensors, prompts, want = mixed
    rp = replay(load(cases.MIXED, tensors, dtype), max_tokens=128, requests=2)
    toks = prompts["a"]
    whole = cases.run_cuts(rp, "whole", toks, [len(toks)])
    assert cases.worst_row_error(whole, want["a"]) < BOUND[dtype]
    same = 1e-5 if dtype == "float32" else BOUND[dtype]
    for sizes in ([2], [3, 16, 1, 29, 2], [16], [17, 1, 1, 1], [64, 2, 2], [1]):
        got = cases.run_cuts(rp, "cut", toks, cases.cuts_of(len(toks), sizes))
        assert cases.worst_row_error(got, whole) < same, sizes
        assert cases.worst_row_error(got, want["a"]) < BOUND[dtype], sizes
    assert all(p.held() == 0 for p in rp.cache.groups.values()) and rp.cache.slots.free_count == 2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_requests_in_one_batch_over_a_small_pool(mixed, dtype):
    """Portions of some requests beside single tokens of others; three slots and just enough pages, so that
    slots and pages are freed and used again; every request's logits equal those of its run alone."""
    tensors, prompts, want = mixed
    rp = replay(load(cases.MIXED, tensors, dtype), max_tokens=256, requests=3)
    plan = {"a": cases.cuts_of(97, [30, 1, 1, 2, 40, 1]), "b": cases.cuts_of(41, [1, 5, 1, 1, 20]),
            "c": cases.cuts_of(70, [2, 2, 1, 64, 1]), "d": [1, 2]}
    order = [("a", "b", "d"), ("a", "b", "c")]          # d ends early, c takes its slot and pages
    got = {n: [] for n in prompts}
    at = {n: 0 for n in prompts}
    turn = {n: 0 for n in prompts}
    live = list(order[0])
    waiting = ["c"]
    steps = 0
    while live:
        entries, ends = [], []
        for n in list(live):
            if steps % 3 == 2 and n == "b" and turn[n] < len(plan[n]) - 1 and len(live) > 1:
                continue                                 # a request may sit out a step
            size = plan[n][turn[n]]
            entries.append({"id": n, "tokens": prompts[n][at[n]:at[n] + size], "want": list(range(size))})
            at[n] += size
            turn[n] += 1
            if turn[n] == len(plan[n]):
                ends.append(n)
        logits = rp.step(entries, ends)
        row = 0
        for e in entries:
            got[e["id"]].append(logits[row:row + len(e["tokens"])].double())
            row += len(e["tokens"])
        for n in ends:
            live.remove(n)
            if waiting:
                live.append(waiting.pop(0))
        steps += 1
    for n in prompts:
        assert at[n] == len(prompts[n])
        assert cases.worst_row_error(torch.cat(got[n], 0), want[n]) < BOUND[dtype], n
    assert all(p.held() == 0 for p in rp.cache.groups.values()) and rp.cache.slots.free_count == 3


def test_long_decoding_past_every_window_and_page(mixed):
    tensors, _, _ = mixed
    toks = cases.tokens_for(cases.MIXED, 260, seed=9)
    want = reference(cases.MIXED, tensors, toks)
    rp = replay(load(cases.MIXED, tensors, "float32"), max_tokens=320, requests=1, page_size=8)
    got = cases.run_cuts(rp, "long", toks, [20] + [1] * 240)
    assert cases.worst_row_error(got, want) < F32_TOL * 4        # 260 tokens through the memory layer
    # the window groups hold only what their windows still reach
    assert all(p.held() == 0 for p in rp.cache.groups.values())


def test_a_token_just_outside_every_reach_does_not_matter(mixed):
    """Attention layers only (a memory layer reaches back without end): the last token's logits keep their
    bits when the token one step beyond the chained windows changes, and move as the plain implementation
    says when the last token inside changes; in a prompt's portion and decoded alone."""
    cfg = cases.config([cases.attention_layer(window=9, ff=16), cases.diff_layer(window=7, ff=None)])
    tensors = cases.draw_weights(cfg, seed=11)
    toks = cases.tokens_for(cfg, 48)
    reach = (9 - 1) + (7 - 1)
    rp = replay(load(cfg, tensors, "float32"), max_tokens=64, requests=1, page_size=8)
    for cuts in ([48], [40] + [1] * 8):
        base = cases.run_cuts(rp, "x", toks, cuts)[-1]
        beyond = list(toks)
        beyond[47 - reach - 1] = (toks[47 - reach - 1] + 1) % cfg["vocab"]
        assert torch.equal(cases.run_cuts(rp, "x", beyond, cuts)[-1], base)
        inside = list(toks)
        inside[47 - reach] = (toks[47 - reach] + 1) % cfg["vocab"]
        moved = cases.run_cuts(rp, "x", inside, cuts)[-1]
        want = reference(cfg, tensors, inside)[-1] - reference(cfg, tensors, toks)[-1]
        assert float(want.abs().max()) > 1e-4
        assert float(((moved - base) - want).abs().max()) < 2e-5


# --- through the loader, the scheduler and the sampler ----------------------------------------------

@pytest.mark.parametrize("dtype,eager", [("float32", False), ("float32", True), ("bfloat16", False)])
def test_greedy_generation_through_the_engine(tmp_path, mixed, dtype, eager):
    import snowllm_b200
    from snowllm_b200.engine import Engine, SamplingParams
    tensors, prompts, _ = mixed
    cases.write_folder(tmp_path, cases.MIXED, tensors)
    model = snowllm_b200.load(tmp_path, dtype, "cuda")
    engine = Engine(model, max_num_seqs=2, max_model_len=256, prefill_chunk=24, page_size=16, enforce_eager=eager)
    asked = [prompts["b"], prompts["d"], prompts["c"][:30]]
    outs = engine.generate(asked, SamplingParams(temperature=0, max_new_tokens=40))
    slack = 1e-4 if dtype == "float32" else 0.15
    for p, o in zip(asked, outs):
        assert len(o) == 40
        logits = reference(cases.MIXED, tensors, p + o)
        for i, tok in enumerate(o):
            row = logits[len(p) - 1 + i]
            assert float(row.max() - row[tok]) <= slack, (dtype, i, tok, int(row.argmax()))
    if not eager:
        assert engine.runner.graph_replays > 0


@pytest.mark.parametrize("rows", [5, 100, 4200])
@pytest.mark.parametrize("act", ["relu", "gelu_tanh", "silu"])
def test_products_apply_the_gate_at_their_store(rows, act):
    """The few-rows product, the tcgen05 product and the product on pairs of SMs, each with every activation,
    against the plain gate on float64 products of the same bfloat16 operands."""
    from snowllm_b200.ops import interleave_gate_up, linear_glu
    g = torch.Generator().manual_seed(rows)
    K, inter = 64, 48
    x = torch.randn(rows, K, generator=g).to(torch.bfloat16)
    gate = (torch.randn(inter, K, generator=g) * 0.3).to(torch.bfloat16)
    up = (torch.randn(inter, K, generator=g) * 0.3).to(torch.bfloat16)
    got = linear_glu(x.cuda(), interleave_gate_up(gate, up).cuda(), True, act)
    want = plain.ACTIVATIONS[act](x.double() @ gate.double().T) * (x.double() @ up.double().T)
    assert got.shape == (rows, inter)
    assert bool(((got.cpu().double() - want).abs() <= 0.008 * want.abs() + 1e-3).all())     # one bfloat16 rounding
    assert cases.relative_error(got.cpu(), want) < 0.003


def test_command_line_generates_with_the_design(tmp_path, mixed, capsys):
    import json

    from snowllm_b200 import cli
    tensors, prompts, _ = mixed
    cases.write_folder(tmp_path, cases.MIXED, tensors)
    prompt = prompts["b"][:20]
    rc = cli.main([str(tmp_path), "--prompt-ids", ",".join(map(str, prompt)), "--default-max-tokens", "12",
                   "--dtype", "float32", "--max-model-len", "256", "--kv-block-size", "16", "--max-num-seqs", "2"])
    assert rc == 0
    line = json.loads(capsys.readouterr().out.strip().splitlines()[0])
    assert line["prompt_tokens"] == 20 and len(line["tokens"]) == 12 and line["finish_reason"] == "length"
    logits = reference(cases.MIXED, tensors, prompt + line["tokens"])
    for i, tok in enumerate(line["tokens"]):
        row = logits[len(prompt) - 1 + i]
        assert float(row.max() - row[tok]) <= 1e-4
