"""Zafopel on the GPU against the plain implementation (tests/plain_zafopel.py): every mechanism alone, the
attention kernel on inputs that make a wrong key, a window one token off or a lost sink show, and one model
with everything fed whole, token by token, in portions and in mixed batches over pools that are used again."""
from __future__ import annotations

import math

import pytest
import torch

import plain_zafopel as plain
import zafopel_cases as cases

pytestmark = pytest.mark.gpu

F32_TOL = 5e-5          # float32 engine against the float64 plain implementation
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


def reference(cfg, tensors, tokens, layers_out=None, rounded=False, **kw):
    return cases.plain_logits(cfg, {k: v.double() for k, v in tensors.items()}, tokens, layers_out, rounded, **kw)


def engine_picks(rp):
    """{layer -> the experts the engine picked, [T, k]} from the taps of a run (in run order)."""
    ids = [t for n, t in rp.runner.taps if n == "moe_route"]
    return ids


def tolerance(dtype):
    return F32_TOL if dtype == "float32" else BF16_TOL


# --- each mechanism alone -------------------------------------------------------------------------

ALONE = {
    "window_moe": [cases.window_layer()],
    "window_one_head_one_pick_no_rotation_rest": [cases.window_layer(heads=1, dim=8, rot_dim=2, vdim=8, kv_rank=16,
                                                                     window=5, mlp=cases.moe(8, 2, 1))],
    "window_unaligned_rows": [cases.window_layer(heads=2, dim=12, rot_dim=6, vdim=10, kv_rank=20, window=40,
                                                 mlp=cases.dense(20))],
    "window_many_heads": [cases.window_layer(heads=20, dim=8, rot_dim=8, vdim=4, kv_rank=24, window=23, mlp=None)],
    "window_part_of_the_slice_turns": [cases.window_layer(rot_dim=12, rot_dims=4, kv_rank=36, window=64)],
    "causal_without_a_mask": [cases.window_layer(window=None, mlp=cases.dense(24))],
    "sink_dense": [cases.sink_layer()],
    "sink_wide_latent": [cases.sink_layer(heads=3, dim=32, rot_dim=8, vdim=16, kv_rank=160, q_rank=20,
                                          mlp=cases.moe(16, 4, 4))],
    "sink_odd": [cases.sink_layer(heads=7, dim=4, rot_dim=2, vdim=6, kv_rank=10, q_rank=6, mlp=None)],
    "reader": [cases.window_layer(window=11), cases.window_layer(window=30, kv_from=0, mlp=None)],
    "reader_sees_every_key": [cases.window_layer(window=9, mlp=None), cases.window_layer(window=None, kv_from=0)],
    # sizes that are multiples of nothing: the products leave the tensor cores, the gate its fused store
    "odd_sizes": [cases.sink_layer(heads=3, dim=12, rot_dim=6, vdim=10, kv_rank=20, q_rank=10, mlp=cases.moe(20, 3, 2)),
                  cases.window_layer(heads=5, dim=6, rot_dim=2, vdim=14, kv_rank=22, window=7, mlp=cases.moe(12, 7, 3)),
                  cases.window_layer(heads=5, dim=10, rot_dim=2, vdim=6, kv_rank=22, window=150, kv_from=1,
                                     mlp=cases.dense(30)),
                  cases.sink_layer(heads=33, dim=8, rot_dim=16, vdim=8, kv_rank=32, q_rank=40, mlp=cases.moe(8, 2, 2))],
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(ALONE))
def test_each_mechanism_alone(name, dtype):
    cfg = cases.config(ALONE[name], **({"width": 36, "vocab": 50} if name == "odd_sizes" else {}))
    tensors = cases.draw_weights(cfg, seed=len(name))
    tokens = cases.tokens_for(cfg, 70)
    model = load(cfg, tensors, dtype)
    rp = replay(model)
    rp.runner.taps = []
    got = cases.run_cuts(rp, "a", tokens, [len(tokens)])
    # the plain experts are put on the engine's picks: a near tie may fall either way, the rest must agree
    routed = [i for i, l in enumerate(cfg["layers"]) if l["mlp"] and l["mlp"]["kind"] == "moe"]
    force = dict(zip(routed, [t.cpu() for t in engine_picks(rp)]))
    want_layers, picks = [], []
    want = reference(cfg, tensors, tokens, want_layers, force_picks=force)
    reference(cfg, tensors, tokens, picks_out=picks)
    for (i, ids, _), mine in zip(picks, [force[i] for i in routed]):
        differ = (ids.sort(-1).values != mine.long().sort(-1).values).any(-1).float().mean()
        assert float(differ) <= (0.0 if dtype == "float32" else 0.1), (i, float(differ))
    layers = [t for n, t in rp.runner.taps if n == "layer_out"]
    assert len(layers) == len(want_layers)
    for x, w in zip(layers, want_layers):
        assert cases.relative_error(x.cpu(), w) < tolerance(dtype)
    assert cases.worst_row_error(got, want) < tolerance(dtype) * 2
    # token by token through the cache gives the same
    rp.runner.taps = None
    again = cases.run_cuts(rp, "b", tokens, [1] * len(tokens))
    assert cases.worst_row_error(again, want) < tolerance(dtype) * 2


# --- the attention kernel on keys that stand out ---------------------------------------------------

def plain_shared_row_attention(q, rows, r, scale, window, sink=None):
    """q [T, H, r + rd], rows [T, r + rd] (one row for all heads, its first r elements the value), float64:
    out [T, H, r]."""
    T, H = q.shape[:2]
    out = torch.zeros(T, H, r, dtype=torch.float64)
    for i in range(T):
        lo = 0 if window is None else max(0, i - window + 1)
        for h in range(H):
            s = (rows[lo:i + 1] @ q[i, h]) * scale
            m = s.max() if sink is None else torch.maximum(s.max(), sink[h])
            e = torch.exp(s - m)
            z = e.sum() + (0 if sink is None else torch.exp(sink[h] - m))
            out[i, h] = (e / z) @ rows[lo:i + 1, :r]
    return out


def paged(rows, P, dtype, gen, spare=3):
    """The rows in pages of P in a scrambled order: (pool [pages, 1, P, width], block table [1, pages])."""
    T, width = rows.shape
    pages = -(-T // P)
    order = torch.randperm(pages + spare, generator=gen)[:pages].int()
    pool = torch.zeros(pages + spare, 1, P, width, dtype=dtype, device="cuda")
    for t in range(T):
        pool[order[t // P], 0, t % P] = rows[t].to(dtype)
    return pool, order.view(1, -1).cuda().contiguous()


def run_kernel(q, pool, table, P, r, scale, window, sink, mode, chunk=64):
    """mode: 'rows' every row alone, 'tiles' rows of the request side by side, 'chunks' rows alone with their
    keys cut into chunks and merged."""
    from snowllm_b200.ops import kernels
    T, H = q.shape[:2]
    q_abs = q[:, :, :r].transpose(0, 1).contiguous().cuda()
    q_rot = q[:, :, r:].contiguous().cuda()
    positions = torch.arange(T, dtype=torch.int32, device="cuda")
    kw = dict(window=window, sink=None if sink is None else sink.float().cuda())
    if mode == "tiles":
        n = kernels.latent_attention_tile_rows(H, r, q.shape[2] - r, q.dtype)
        tiles = torch.tensor([[s, min(n, T - s)] for s in range(0, T, n)], dtype=torch.int32, device="cuda")
        kw.update(tiles=tiles, tile_rows=n)
    if mode == "chunks":
        # the most chunks any row spans
        kw.update(num_chunks=min((window - 1) // chunk + 2, (T - 1) // chunk + 1) if window else (T - 1) // chunk + 1,
                  chunk=chunk)
    return kernels.latent_attention(q_abs, q_rot, pool, table, P, positions, torch.zeros_like(positions), scale, **kw)


# row sizes (r, rd): the second of each pair is one the tensor-core kernel takes in bfloat16
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("mode", ["rows", "tiles", "chunks"])
@pytest.mark.parametrize("r,rd", [(24, 8), (32, 16)])
def test_attention_kernel_sees_exactly_its_window(dtype, mode, r, rd):
    """One key per row is made to stand out: on the window's last position inside it owns the output, one
    position further it must not be seen at all.  Pages in a scrambled order; the window is no multiple of
    the key tile, the page or the chunk."""
    g = torch.Generator().manual_seed(5)
    T, H, P, window = 150, 4, 16, 37
    q = torch.randn(T, H, r + rd, generator=g).to(dtype)
    rows = (torch.randn(T, r + rd, generator=g) * 0.1).to(dtype)
    rows[:, :r] = torch.randn(T, r, generator=g).to(dtype) * 0.1 + torch.arange(T)[:, None] * 0.01
    inside, outside = 120, 131
    rows[inside - (window - 1), r:] = (q[inside, 1, r:].float() * 20).to(dtype)    # the farthest key row 120 sees
    rows[outside - window, r:] = (q[outside, 2, r:].float() * 20).to(dtype)        # one beyond row 131's window
    pool, table = paged(rows, P, dtype, g)
    got = run_kernel(q, pool, table, P, r, 0.25, window, None, mode).float().cpu().double()
    want = plain_shared_row_attention(q.double(), rows.double(), r, 0.25, window)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert float((got - want).abs().max()) < tol
    own = rows[inside - (window - 1), :r].double()
    assert float((want[inside, 1] - own).abs().max()) < 0.02            # the key owns the row
    assert float((got[inside, 1] - own).abs().max()) < 0.03
    assert float((got[outside, 2] - rows[outside - window, :r].double()).abs().max()) > 0.05


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("mode", ["rows", "tiles", "chunks"])
@pytest.mark.parametrize("r,rd", [(40, 4), (48, 16)])
def test_attention_kernel_finds_a_far_key_and_counts_the_sink_once(dtype, mode, r, rd):
    """Causal rows over 300 keys in pages of 8.  Head 0 of the last row looks for the key at position 3 among
    hundreds; head 1's sink is so large that its output all but vanishes; head 2's so small that it does
    nothing; head 3 sits between (its share of the denominator is checked by the numbers)."""
    g = torch.Generator().manual_seed(8)
    T, H, P = 300, 4, 8
    q = torch.randn(T, H, r + rd, generator=g).to(dtype)
    rows = (torch.randn(T, r + rd, generator=g) * 0.2).to(dtype)
    looks = q[T - 1, 0, r:].float()
    rows[3, r:] = (looks * (100 / float(looks @ looks))).to(dtype)         # a score of 30 after the scale
    rows[3, :r] = 1.5
    sink = torch.tensor([-30.0, 200.0, -200.0, 0.5])
    pool, table = paged(rows, P, dtype, g)
    got = run_kernel(q, pool, table, P, r, 0.3, None, sink, mode).float().cpu().double()
    want = plain_shared_row_attention(q.double(), rows.double(), r, 0.3, None, sink.double())
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert float((got - want).abs().max()) < tol
    assert float((got[T - 1, 0] - 1.5).abs().max()) < 0.05              # the far key owns the row
    assert float(got[:, 1].abs().max()) < 1e-6                          # the sink took everything
    free = plain_shared_row_attention(q.double(), rows.double(), r, 0.3, None)
    assert float((got[:, 2] - free[:, 2]).abs().max()) < tol            # a sink far below does nothing
    assert float((want[:, 3] - free[:, 3]).abs().max()) > 0.01          # one in between takes its share
    # the first token of a sequence: one key, weight e^s / (e^s + e^sink)
    s = float((rows[0].double() @ q[0, 3].double()) * 0.3)
    share = math.exp(s) / (math.exp(s) + math.exp(0.5))
    assert float((got[0, 3] - share * rows[0, :r].double()).abs().max()) < tol


@pytest.mark.parametrize("mode", ["rows", "tiles", "chunks"])
@pytest.mark.parametrize("H,r,rd,window,sinks", [(16, 512, 64, None, True), (40, 64, 32, 150, False),
                                                 (6, 256, 16, 70, True), (3, 96, 48, None, False)])
def test_attention_kernel_on_the_tensor_cores_at_other_sizes(mode, H, r, rd, window, sinks):
    """bfloat16 rows of the widths and head counts a large model has (one, two and four tiles of 16 units, several
    groups of heads, values that do not fill a warp's columns), against the plain attention on the same rounded
    inputs."""
    g = torch.Generator().manual_seed(H)
    T, P = 210, 16
    q = (torch.randn(T, H, r + rd, generator=g) * 0.5).to(torch.bfloat16)
    rows = (torch.randn(T, r + rd, generator=g) * 0.3).to(torch.bfloat16)
    sink = torch.randn(H, generator=g) * 2 if sinks else None
    pool, table = paged(rows, P, torch.bfloat16, g)
    scale = (r + rd) ** -0.5 * 2
    got = run_kernel(q, pool, table, P, r, scale, window, sink, mode).float().cpu().double()
    want = plain_shared_row_attention(q.double(), rows.double(), r, scale, window, None if sink is None else sink.double())
    assert float((got - want).abs().max()) < 6e-3                       # one rounding of outputs below 1


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_prepare_normalises_rotates_and_writes_the_row(dtype):
    from snowllm_b200.ops import kernels
    from snowllm_b200.parts.position import PairedRotaryPosition
    g = torch.Generator().manual_seed(9)
    M, H, dim, rd, r, P, rot = 13, 3, 10, 6, 20, 4, 4
    q = torch.randn(M, 5 + H * (dim + rd), generator=g).to(dtype)
    kv = torch.randn(M, 7 + r + rd, generator=g).to(dtype)
    gamma = (1 + 0.3 * torch.randn(r, generator=g)).to(dtype)
    positions = torch.tensor([40, 41, 42, 0, 1, 2, 3, 4, 5, 6, 7, 8, 1000], dtype=torch.int32)
    row_seg = torch.tensor([0] * 3 + [1] * 9 + [2], dtype=torch.int32)
    table = torch.full((3, 251), 0, dtype=torch.int32)
    table[0, 10], table[1, 0], table[1, 1], table[1, 2], table[2, 250] = 5, 2, 7, 1, 3
    pool = torch.zeros(8, 1, P, r + rd, dtype=dtype, device="cuda")
    inv_freq, _ = PairedRotaryPosition(head_dim=rd, theta=50.0, rot_dim=rot).rotary("cuda")
    q_unrot, q_rot = kernels.latent_prepare(q.cuda(), 5, kv.cuda(), 7, gamma.cuda(), 1e-3, inv_freq, rot,
                                            positions.cuda(), row_seg.cuda(), table.cuda(), P, pool, H, dim, rd, r)
    tol = 1e-5 if dtype == torch.float32 else 0.03
    heads = q[:, 5:].double().view(M, H, dim + rd)
    assert torch.equal(q_unrot.cpu(), heads[..., :dim].transpose(0, 1).to(dtype))
    want_rot = plain.rotate_pairs(heads[..., dim:], positions, 50.0, rot)
    assert float((q_rot.cpu().double() - want_rot).abs().max()) < tol
    c = plain.rms_norm(kv[:, 7:7 + r].double(), gamma.double(), 1e-3)
    k_rot = plain.rotate_pairs(kv[:, 7 + r:].double(), positions, 50.0, rot)
    for m in range(M):
        pos = int(positions[m])
        row = pool[int(table[int(row_seg[m]), pos // P]), 0, pos % P].cpu().double()
        assert float((row[:r] - c[m]).abs().max()) < tol and float((row[r:] - k_rot[m]).abs().max()) < tol
    assert int((pool.float().abs().sum(-1) > 0).sum()) == M                     # nothing else was written


# --- the elementwise kernels ----------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_dynamic_tanh_sums_activation_rms_and_scaled_rows(dtype):
    from snowllm_b200.ops import kernels
    g = torch.Generator().manual_seed(7)
    M, H, k = 9, 100, 2
    residual, a, b = (torch.randn(M, H, generator=g) for _ in range(3))
    w, bias = (1 + 0.3 * torch.randn(H, generator=g)).to(dtype), (0.2 * torch.randn(H, generator=g)).to(dtype)
    alpha = torch.tensor(0.7).to(dtype)
    tol = 1e-5 if dtype == torch.float32 else 0.02
    # the two sublayers' outputs as tensors
    res = residual.clone().cuda()
    x = kernels.add_dyt(res, kernels.DeltaSum(a.cuda(), b.cuda()), w.cuda(), bias.cuda(), alpha.cuda(), dtype)
    total = residual.double() + (a.double() + b.double())
    assert float((res.cpu().double() - total).abs().max()) < 1e-6
    want = plain.dynamic_tanh(total, w.double(), bias.double(), alpha.double())
    assert float((x.cpu().double() - want).abs().max()) < tol
    # the second one still in pieces (routed experts' outputs), and only some rows
    y = torch.randn(M * k, H, generator=g)
    pair_pos = torch.randperm(M * k, generator=g).int()
    pw = torch.rand(M, k, generator=g)
    pieces = kernels.ExpertSum(y.cuda(), pair_pos.cuda(), pw.cuda())
    summed = (pw.double()[:, :, None] * y.double()[pair_pos.long()].view(M, k, H)).sum(1)
    rows = torch.tensor([8, 0, 3], dtype=torch.int32)
    res = residual.clone().cuda()
    x = kernels.add_dyt(res, kernels.DeltaSum(a.cuda(), pieces), w.cuda(), bias.cuda(), alpha.cuda(), dtype,
                        rows=rows.cuda())
    assert torch.equal(res.cpu(), residual)                                     # with rows the stream stays
    want = plain.dynamic_tanh(residual.double() + (a.double() + summed), w.double(), bias.double(), alpha.double())
    assert float((x.cpu().double() - want[rows.long()]).abs().max()) < tol
    res = residual.clone().cuda()
    kernels.add_dyt(res, pieces, w.cuda(), bias.cuda(), alpha.cuda(), dtype)
    assert float((res.cpu().double() - (residual.double() + summed)).abs().max()) < 1e-6
    x = kernels.add_dyt(res, None, w.cuda(), bias.cuda(), alpha.cuda(), dtype)      # nothing to add
    assert float((x.cpu().double() - plain.dynamic_tanh(res.cpu().double(), w.double(), bias.double(),
                                                         alpha.double())).abs().max()) < tol
    # activations, the square of relu among them
    z = (torch.randn(M, 37, generator=g) * 2).to(dtype)
    for act in ("relu2", "relu", "gelu_tanh", "silu"):
        got = kernels.act_rows(z.cuda(), act)
        assert float((got.cpu().double() - plain.ACTIVATIONS[act](z.double())).abs().max()) < 3 * tol, act
    # RMS norm of a slice of columns
    gamma = (1 + 0.3 * torch.randn(21, generator=g)).to(dtype)
    got = kernels.rms_cols(z.cuda(), 5, 21, gamma.cuda(), 1e-2)
    assert float((got.cpu().double() - plain.rms_norm(z[:, 5:26].double(), gamma.double(), 1e-2)).abs().max()) < tol
    # rows times their pick's weight, in expert order
    xs, ones = kernels.moe_scaled_rows(z.cuda(), pair_pos.cuda(), pw.cuda(), k)
    want = z.double()[pair_pos.long() // k] * pw.double().view(-1)[pair_pos.long()][:, None]
    assert float((xs.cpu().double() - want).abs().max()) < tol and bool((ones == 1).all())


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
    got = {n: [] for n in prompts}
    at = {n: 0 for n in prompts}
    turn = {n: 0 for n in prompts}
    live, waiting, steps = ["a", "b", "d"], ["c"], 0         # d ends early, c takes its slot and pages
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


def test_long_decoding_past_every_window_page_and_chunk(mixed):
    tensors, _, _ = mixed
    toks = cases.tokens_for(cases.MIXED, 560, seed=9)
    want = reference(cases.MIXED, tensors, toks)
    rp = replay(load(cases.MIXED, tensors, "float32"), max_tokens=576, requests=1, page_size=8)
    got = cases.run_cuts(rp, "long", toks, [20] + [1] * 540)      # decoded rows cross two chunks of 256 keys
    assert cases.worst_row_error(got, want) < F32_TOL * 2
    assert all(p.held() == 0 for p in rp.cache.groups.values())


def test_a_token_just_outside_every_reach_does_not_matter():
    """Window layers only: the last token's logits keep their bits when the token one step beyond the chained
    windows changes, and move as the plain implementation says when the last token inside changes; in a
    prompt's portion and decoded alone."""
    cfg = cases.config([cases.window_layer(window=9, mlp=cases.dense(16)),
                        cases.window_layer(heads=2, window=7, mlp=None)])
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
