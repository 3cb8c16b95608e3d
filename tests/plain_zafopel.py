"""A plain, slow implementation of the Zafopel design on the CPU: one function per mechanism, written from
the design's equations, whole sequences at a time, no cache.  It shares nothing with the engine: keys and
values are formed for every head from the latent (the engine never forms them), the softmax is a plain one
over an explicit mask, the experts are looped over.

Notation: x is a sequence's residual stream [T, width]; h = norm(x) the input of both sublayers; W x means
``x @ W.T`` for a weight stored [out, in].  Everything runs in ``dtype`` (float64 by default).

A model is a dict: ``config`` (the parsed config.json) and ``tensors`` (name -> tensor)."""
from __future__ import annotations

import math

import torch

# Where the 16-bit path stores a value (the norm's output, a projection's output, the cached row, what
# enters the output product), the rounding variant rounds it to bfloat16 and goes on in ``dtype``: how far
# that moves the logits is the measure of what rounding alone may cost.
ROUND = {"on": False}


def stored(x):
    return x.to(torch.bfloat16).to(x.dtype) if ROUND["on"] else x


def dynamic_tanh(x, w, b, alpha):
    """tanh(alpha x) w + b: a norm without statistics."""
    return torch.tanh(alpha * x) * w + b


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))


def relu2(z):
    return torch.relu(z) ** 2


ACTIVATIONS = {"relu": torch.relu, "gelu_tanh": gelu_tanh, "silu": torch.nn.functional.silu, "relu2": relu2}


def rotate_pairs(x, positions, base: float, dims: int):
    """x [T, ..., d]: elements (2i, 2i+1), i < dims/2, of the last axis turn by positions * base^(-2i/dims);
    the rest passes."""
    out = x.clone()
    shape = [x.shape[0]] + [1] * (x.dim() - 2)
    for i in range(dims // 2):
        a = positions.to(x.dtype) * base ** (-2.0 * i / dims)
        c, s = torch.cos(a).view(shape), torch.sin(a).view(shape)
        u, v = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = u * c - v * s
        out[..., 2 * i + 1] = v * c + u * s
    return out


def visible(T: int, window):
    """[T, T] bool: i sees j when 0 <= i - j (< window)."""
    d = torch.arange(T)[:, None] - torch.arange(T)[None, :]
    return (d >= 0) if window is None else (d >= 0) & (d < window)


def softmax_rows(s, mask, sink=None):
    """Softmax over the visible keys of each row of s [T, T]; ``sink``: one more term exp(sink) in the
    denominator that has no key."""
    s = s.masked_fill(~mask, -math.inf)
    m = s.max(-1, keepdim=True).values
    if sink is not None:
        m = torch.maximum(m, sink.expand_as(m))
    e = torch.exp(s - m)
    z = e.sum(-1, keepdim=True)
    if sink is not None:
        z = z + torch.exp(sink - m)
    return e / z


def latent_rows(h, w_dkv, w_norm, r: int, eps: float, base: float, dims: int):
    """What a layer caches per position: (latent c [T, r], rotated key part [T, rd])."""
    d = stored(h @ w_dkv.T)
    positions = torch.arange(h.shape[0])
    return stored(rms_norm(d[:, :r], w_norm, eps)), stored(rotate_pairs(d[:, r:], positions, base, dims))


def latent_attention(q, c, k_rot, w_uk, w_uv, w_o, heads, dim, rd, vdim, scale, window, sink, base, dims):
    """q [T, heads * (dim + rd)] laid out head by head as [dim unrotated, rd rotated]."""
    T = q.shape[0]
    q = q.view(T, heads, dim + rd)
    q_rot = rotate_pairs(q[..., dim:], torch.arange(T), base, dims)
    keys = (c @ w_uk.T).view(T, heads, dim)
    values = (c @ w_uv.T).view(T, heads, vdim)
    mask = visible(T, window)
    out = []
    for hd in range(heads):
        s = (q[:, hd, :dim] @ keys[:, hd].T + q_rot[:, hd] @ k_rot.T) * scale
        p = softmax_rows(s, mask, None if sink is None else sink[hd])
        out.append(p @ values[:, hd])
    return stored(torch.cat(out, -1)) @ w_o.T


def dense_ff(h, up, down, act="relu2"):
    return stored(ACTIVATIONS[act](stored(h @ up.T))) @ down.T


def router_picks(h, w_router, top: int):
    """(experts [T, top], their scores): the largest sigmoids of W_router h, not renormalised."""
    scores = torch.sigmoid(h @ w_router.T)
    w, ids = scores.topk(top, -1)
    return ids, w


def routed_ff(h, picks, experts):
    """sum over a token's picks of expert(w h): the weight multiplies the expert's INPUT.
    ``experts``: list of (gate, up, down)."""
    ids, w = picks
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(ids.shape[1]):
            gate, up, down = experts[int(ids[t, j])]
            x = stored(h[t] * w[t, j])
            out[t] += stored(torch.nn.functional.silu(stored(gate @ x)) * stored(up @ x)) @ down.T
    return out


def forward(model, tokens, dtype=torch.float64, layers_out=None, rounded=False, picks_out=None, force_picks=None):
    """Logits [T, vocab] of one sequence.  ``layers_out``: a list that gets the stream after every layer.
    ``picks_out`` gets each routed layer's (ids, weights); ``force_picks`` {layer -> ids} replaces a router's
    choice (the weights stay the router's scores of those experts)."""
    cfg = model["config"]
    W = {k: v.to(dtype) for k, v in model["tensors"].items()}
    eps = cfg["norm"]["eps"]
    ROUND["on"] = rounded
    try:
        x = W["embed"][torch.as_tensor(tokens)]
        cached = {}
        for i, layer in enumerate(cfg["layers"]):
            p, m = f"l{i}.", layer["mixer"]
            h = stored(dynamic_tanh(x, W[p + "norm1"], W[p + "norm1.b"], W[p + "norm1.alpha"]))
            r, base, dims = m["kv_rank"], m["rot"]["base"], m["rot"]["dims"]
            if layer["type"] == "latent_attention_2":
                cq = stored(rms_norm(stored(h @ W[p + "mix.dq"].T), W[p + "mix.dq.norm"], eps))
                q, window, sink = stored(cq @ W[p + "mix.uq"].T), None, W[p + "mix.sink"]
            else:
                q, sink = stored(h @ W[p + "mix.q"].T), None
                window = m["mask"]["size"] if m.get("mask") else None
            if m.get("kv_from") is not None:
                c, k_rot = cached[m["kv_from"]]
            else:
                c, k_rot = cached[i] = latent_rows(h, W[p + "mix.dkv"], W[p + "mix.dkv.norm"], r, eps, base, dims)
            y = latent_attention(q, c, k_rot, W[p + "mix.uk"], W[p + "mix.uv"], W[p + "mix.o"], m["heads"], m["dim"],
                                 m["rot_dim"], m["vdim"], m["scale"], window, sink, base, dims)
            mlp = layer["mlp"]
            if mlp is not None and mlp["kind"] == "dense":
                y = y + dense_ff(h, W[p + "mlp.up"], W[p + "mlp.down"])
            elif mlp is not None:
                ids, w = router_picks(h, W[p + "mlp.router"], mlp["router"]["top"])
                if force_picks is not None and i in force_picks:
                    ids = force_picks[i].long()
                    w = torch.sigmoid(h @ W[p + "mlp.router"].T).gather(1, ids)
                if picks_out is not None:
                    picks_out.append((i, ids, w))
                experts = [(W[f"{p}mlp.e{e}.gate"], W[f"{p}mlp.e{e}.up"], W[f"{p}mlp.e{e}.down"])
                           for e in range(mlp["router"]["experts"])]
                y = y + routed_ff(h, (ids, w), experts)
            x = x + y
            if layers_out is not None:
                layers_out.append(x.clone())
        h = stored(dynamic_tanh(x, W["final.norm"], W["final.norm.b"], W["final.norm.alpha"]))
        return h @ W["head"].T
    finally:
        ROUND["on"] = False
