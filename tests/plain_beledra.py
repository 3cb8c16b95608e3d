"""A plain, slow implementation of the Beledra design on the CPU: one function per mechanism, written
from the design's equations, whole sequences at a time, no cache.  It shares nothing with the engine.

Notation: x is a sequence's residual stream [T, width]; h the input of a sublayer; W x means
``x @ W.T`` for a weight stored [out, in].  Everything runs in ``dtype`` (float64 by default, so that
the engine's 32-bit results are compared with something sharper than themselves).

A model is a dict: ``config`` (the parsed config.json) and ``tensors`` (name -> tensor)."""
from __future__ import annotations

import math

import torch


# Where the 16-bit path stores a value (a sublayer's input, a projection's output, what enters the output
# product), the rounding variant of this implementation rounds it to bfloat16 and goes on in ``dtype``: how
# far that moves the logits is the measure of what rounding alone may cost.
ROUND = {"on": False}


def stored(x):
    return x.to(torch.bfloat16).to(x.dtype) if ROUND["on"] else x


def rms_normalise(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, w, eps):
    return rms_normalise(x, eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))


ACTIVATIONS = {"relu": torch.relu, "gelu_tanh": gelu_tanh, "silu": torch.nn.functional.silu}


def gated_ff(h, gate, up, down, act="relu"):
    h = stored(h)
    return stored(ACTIVATIONS[act](stored(h @ gate.T)) * stored(h @ up.T)) @ down.T


# --- distance bias --------------------------------------------------------------------------------

def distance_bucket(n: int, rows: int, far: float) -> int:
    """Row of the bias table for a key ``n`` positions back: one row per distance up to rows/2, then
    logarithmic steps that reach the last row at distance ``far``."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def window_mask(T: int, size):
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    d = i - j
    ok = d >= 0
    if size is not None:
        ok &= d < size
    return ok, d


def biased_attention(h, t, p, m, eps):
    """Windowed grouped-query attention with per-head norm of q and k and a learned bias per distance
    bucket and head.  ``t``: the layer's mixer tensors by short name; ``m``: the mixer's config."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    h = stored(h)
    q = stored(h @ t["q"].T).view(T, H, dk)
    k = stored(h @ t["k"].T).view(T, G, dk)
    v = stored(h @ t["v"].T).view(T, G, dv)
    q = stored(rms_norm(q, t["q.norm"], eps))
    k = stored(rms_norm(k, t["k.norm"], eps))
    ok, d = window_mask(T, (m.get("mask") or {}).get("size"))
    rel = t["rel"]
    rows = rel.shape[0]
    bucket = torch.tensor([[distance_bucket(int(n), rows, m["bias_max"]) if n >= 0 else 0 for n in row]
                           for row in d.tolist()])
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * m["scale"] + rel[bucket, head]
        s = s.masked_fill(~ok, -math.inf)
        out[:, head] = torch.softmax(s, -1) @ v[:, g]
    return stored(out.reshape(T, H * dv)) @ t["o"].T


# --- rotary positions with YaRN -------------------------------------------------------------------

def yarn_frequencies(rot):
    dims, base = rot["dims"], rot["base"]
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    scaling = rot.get("scaling")
    if not scaling:
        return f, 1.0
    factor, original = scaling["factor"], scaling["original"]

    def place(turns):
        return dims * math.log(original / (2 * math.pi * turns)) / (2 * math.log(base))
    lo = max(math.floor(place(scaling["fast"])), 0)
    hi = min(math.ceil(place(scaling["slow"])), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate(x, positions, rot):
    """x [T, heads, dim]: the first rot.dims elements of each head turn, element i with i + dims/2."""
    if not rot:
        return x
    dims = rot["dims"]
    f, magnitude = yarn_frequencies(rot)
    a = positions.to(x.dtype)[:, None] * torch.tensor(f, dtype=x.dtype)[None, :]        # [T, dims/2]
    c, s = (torch.cos(a) * magnitude)[:, None, :], (torch.sin(a) * magnitude)[:, None, :]
    u, w = x[..., :dims // 2], x[..., dims // 2:dims]
    return torch.cat((u * c - w * s, w * c + u * s, x[..., dims:]), -1)


# --- differential attention -----------------------------------------------------------------------

def differential_keys_values(h, t, m, eps, positions):
    T = h.shape[0]
    G, dk, dv = m["kv_heads"], m["dim"], m["vdim"]
    h = stored(h)
    k = stored(h @ t["k"].T).view(T, G * 2, dk)
    k = stored(rotate(rms_norm(k, t["k.norm"], eps), positions, m.get("rot")))
    return k.view(T, G, 2, dk), stored(h @ t["v"].T).view(T, G, dv)


def differential_attention(h, t, m, eps, kv):
    """Two softmax maps per head over the same values, the second taken off the first with the
    layer's weight; ``kv``: (keys [T, G, 2, dk] after norm and rotation, values [T, G, dv])."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    positions = torch.arange(T)
    h = stored(h)
    q = stored(h @ t["q"].T).view(T, H * 2, dk)
    q = stored(rotate(rms_norm(q, t["q.norm"], eps), positions, m.get("rot"))).view(T, H, 2, dk)
    k, v = kv
    ok, _ = window_mask(T, (m.get("mask") or {}).get("size"))
    lam = torch.exp((t["lq1"] * t["lk1"]).sum()) - torch.exp((t["lq2"] * t["lk2"]).sum()) + m["diff"]
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for head in range(H):
        g = head // (H // G)
        maps = []
        for which in range(2):
            s = (q[:, head, which] @ k[:, g, which].T) * m["scale"]
            s = s.masked_fill(~ok, -math.inf)
            maps.append(torch.softmax(s, -1) @ v[:, g])
        o = maps[0] - lam * maps[1]
        out[:, head] = rms_normalise(o, eps) * (1 - m["diff"])
    out = out.reshape(T, H * dv) * torch.sigmoid(stored(h @ t["g"].T))
    return stored(out) @ t["o"].T


# --- matrix memory (mLSTM) ------------------------------------------------------------------------

def mlstm(h, t, m, eps):
    """Token by token: a matrix S [dk, dv] and a vector n [dk] per head with exponential gates, kept
    in range by a running maximum that starts at 0."""
    T = h.shape[0]
    H, dk, dv, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    h = stored(h)
    q = (h @ t["q"].T).view(T, H, dk) * dk ** -0.5
    k = (h @ t["k"].T).view(T, H, dk)
    v = (h @ t["v"].T).view(T, H, dv)
    gi = cap * torch.tanh((h @ t["i"].T + t["i.b"]) / cap)                          # [T, H]
    gf = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ t["f"].T + t["f.b"]) / cap))
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for head in range(H):
        S = torch.zeros(dk, dv, dtype=h.dtype)
        n = torch.zeros(dk, dtype=h.dtype)
        mx = torch.zeros((), dtype=h.dtype)
        for step in range(T):
            new = torch.maximum(gf[step, head] + mx, gi[step, head])
            keep, take = torch.exp(gf[step, head] + mx - new), torch.exp(gi[step, head] - new)
            S = keep * S + take * torch.outer(k[step, head], v[step, head])
            n = keep * n + take * k[step, head]
            mx = new
            below = torch.maximum((n * q[step, head]).sum().abs(), torch.exp(-mx)) + 1e-6
            out[step, head] = (S.T @ q[step, head]) / below
    out = rms_normalise(out, eps).reshape(T, H * dv) * t["norm"] * torch.sigmoid(h @ t["g"].T)
    return stored(out) @ t["o"].T


# --- the model --------------------------------------------------------------------------------------

def mixer_tensors(tensors, layer: int, dtype):
    p = f"l{layer}.mix."
    return {k[len(p):]: v.to(dtype) for k, v in tensors.items() if k.startswith(p)}


def forward(model, tokens, dtype=torch.float64, layers_out=None, rounded=False):
    """Logits [T, vocab] of one whole sequence; ``layers_out`` (a list) receives the residual stream
    after every layer.  ``rounded``: the rounding variant (see ``stored``)."""
    ROUND["on"] = bool(rounded)
    try:
        return _forward(model, tokens, dtype, layers_out)
    finally:
        ROUND["on"] = False


def _forward(model, tokens, dtype, layers_out):
    cfg, ts = model["config"], model["tensors"]
    eps = cfg["norm"]["eps"]
    T = len(tokens)
    positions = torch.arange(T)
    x = ts["embed"].to(dtype)[torch.tensor(tokens)]
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        m, t = layer["mixer"], mixer_tensors(ts, i, dtype)
        if layer["type"] == "attention":
            y = biased_attention(x, t, None, m, eps)
        elif layer["type"] == "attention_2":
            src = m.get("kv_from")
            if src is None:
                kept[i] = differential_keys_values(x, t, m, eps, positions)
            y = differential_attention(x, t, m, eps, kept[i if src is None else src])
        elif layer["type"] == "mlstm":
            y = mlstm(x, t, m, eps)
        else:
            raise ValueError(layer["type"])
        x = x + rms_norm(y, ts[f"l{i}.norm1"].to(dtype), eps)
        if layer.get("mlp") is not None:
            f = f"l{i}.mlp."
            y = gated_ff(x, ts[f + "gate"].to(dtype), ts[f + "up"].to(dtype), ts[f + "down"].to(dtype))
            x = x + rms_norm(y, ts[f"l{i}.norm2"].to(dtype), eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    x = stored(rms_norm(x, ts["final.norm"].to(dtype), eps))
    return x @ ts["head"].to(dtype).T
