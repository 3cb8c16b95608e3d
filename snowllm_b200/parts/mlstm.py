"""Matrix-memory mixer (the mLSTM of xLSTM) with a state of fixed size per request (csrc/mlstm.cu).

One fused product gives q, k ([heads, head_dim]), v ([heads, v_head_dim]), the output gate's
pre-activation and the two gates' pre-activations per head, in float.  The recurrence runs token by
token per (request, head) on a float state (matrix S [head_dim, v_head_dim], vector n [head_dim] and a
running maximum m per head, all zero for a fresh request) that lives in the request's state slot:

    i = cap * tanh((W_i x + b_i) / cap);  f = logsigmoid(cap * tanh((W_f x + b_f) / cap))
    m' = max(f + m, i);  S' = exp(f + m - m') S + exp(i - m') k v^T;  n' = exp(f + m - m') n + exp(i - m') k
    o = S'^T q / (max(|n' . q|, exp(-m')) + 1e-6)   with q scaled by head_dim^(-1/2)

Each head's o is divided by its root mean square, the heads are weighted (``norm`` over heads *
v_head_dim), gated by sigmoid(W_g x) and projected out.  Gates, state, norms: float in every dtype."""
from __future__ import annotations

import torch

from ..errors import ConfigError
from ..ops import kernels, linear
from .attention_maps import pad_rows
from .base import Part
from .registry import register_mixer
from .spec import INIT_BIAS, INIT_ONES, KEEP_F32, KEEP_SMALL, SlotStateSpec, TensorSpec


class MLstm(Part):
    libraries = ("gemm", "gemm_skinny", "gemm_tc", "gemm_tc2", "mlstm", "sublayer")

    def __init__(self, dtype, names, *, hidden_size: int, num_heads: int, head_dim: int, v_head_dim: int,
                 gate_cap: float, head_norm_eps: float):
        super().__init__(dtype, names)
        if head_dim > 128 or v_head_dim > 1024:
            raise ConfigError(f"mlstm heads of {head_dim} x {v_head_dim}: the kernel keeps up to 128 x 1024")
        if not gate_cap > 0:
            raise ConfigError(f"gate_cap={gate_cap} must be positive")
        self.hidden_size, self.num_heads, self.head_dim, self.v_head_dim = hidden_size, num_heads, head_dim, v_head_dim
        self.gate_cap, self.head_norm_eps = float(gate_cap), float(head_norm_eps)
        self.w_in = self.wo = self.norm = self.bias_i = self.bias_f = None

    def cache_spec(self):
        H, dk, dv = self.num_heads, self.head_dim, self.v_head_dim
        return SlotStateSpec(((H, dk, dv), (H, dk), (H,)), ("f32", "f32", "f32"))

    def _columns(self):
        H, dk, dv = self.num_heads, self.head_dim, self.v_head_dim
        q = 0
        k = q + H * dk
        v = k + H * dk
        g = v + H * dv
        i = g + H * dv
        f = i + H
        return q, k, v, g, i, f

    def declare(self, has):
        W, H, dk, dv, n = self.hidden_size, self.num_heads, self.head_dim, self.v_head_dim, self.names
        return [TensorSpec("q_proj", n["q_proj"], (H * dk, W)), TensorSpec("k_proj", n["k_proj"], (H * dk, W)),
                TensorSpec("v_proj", n["v_proj"], (H * dv, W)), TensorSpec("gate_proj", n["gate_proj"], (H * dv, W)),
                TensorSpec("out_proj", n["out_proj"], (W, H * dv)),
                TensorSpec("norm", n["norm"], (H * dv,), INIT_ONES, KEEP_SMALL),
                TensorSpec("i_proj", n["i_proj"], (H, W)), TensorSpec("i_bias", n["i_bias"], (H,), INIT_BIAS, KEEP_F32),
                TensorSpec("f_proj", n["f_proj"], (H, W)), TensorSpec("f_bias", n["f_bias"], (H,), INIT_BIAS, KEEP_F32)]

    def bind(self, tensors):
        rows = [tensors[k] for k in ("q_proj", "k_proj", "v_proj", "gate_proj", "i_proj", "f_proj")]
        self.w_in = pad_rows(torch.cat(rows, 0), 16)
        self.wo, self.norm = tensors["out_proj"], tensors["norm"]
        self.bias_i, self.bias_f = tensors["i_bias"], tensors["f_bias"]

    def forward(self, ctx, x, cache, owns_cache=True):
        H, dk, dv = self.num_heads, self.head_dim, self.v_head_dim
        proj = linear(x, self.w_in, out_dtype=torch.float32)
        q, k, v, g, i, f = self._columns()
        s_mat, s_vec, s_max = cache.tensors
        raw = kernels.mlstm(proj, q, k, v, i, f, self.bias_i, self.bias_f, self.gate_cap, ctx.cu_seqlens,
                            ctx.seg_start, ctx.seg_slot, s_mat, s_vec, s_max, H, dk, dv)
        ctx.tap("mlstm_raw", raw)
        heads = kernels.head_norm_gate(raw, H, dv, self.head_norm_eps, self.dtype, weight=self.norm, gate=proj,
                                       gate_col=g)
        return linear(heads, self.wo, out_dtype=torch.float32)


register_mixer("mlstm", MLstm)
