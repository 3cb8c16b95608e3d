"""Latent attention (csrc/attention_latent.cu): keys and values of all heads come from one low-rank latent
per position, and only that latent and one rotated key part shared by all heads are cached.

    c      = rmsnorm(W_dkv x)[:r]            the latent, r = kv_rank
    k_rot  = rotate(W_dkv x)[r:r + rd]       one rotated key part for all heads, rd = rot_dim
    head h:  key = [W_uk_h c, k_rot], value = W_uv_h c, query = [q_unrot_h (dim), rotate(q_rot_h) (rd)]
    score  = (q_unrot_h . W_uk_h c + q_rot_h . k_rot) * scale

The up-projections are never applied to the cache.  The query takes W_uk in (q_abs_h = W_uk_h^T q_unrot_h, a
grouped product over the heads), the attention kernel works on the cached row alone (its first r elements
are also the value), and W_uv is applied to each head's weighted sum of latents (a second grouped product)
before the output product.  Prompts, portions and decoded rows all take this one path, so what a position
computes does not depend on how its sequence was cut.

Options, each a constructor parameter: ``q_rank`` (the query goes through a normalised latent of its own:
q = W_uq rmsnorm(W_dq x)), ``window`` (the last ``window`` keys; None: causal), ``sink`` (a learned number per
head whose exponential joins the softmax's denominator), ``reads_cache`` (no W_dkv: the layer attends over
the rows another layer cached).  ``cache_window`` is how many positions the owner of the cache keeps (None:
all of them; by default the layer's own window)."""
from __future__ import annotations

import torch

from ..errors import ConfigError, KernelError
from ..ops import grouped_linear, kernels, linear
from . import attention_plan as plan
from .attention_maps import attention_tiles, pad_rows
from .base import Part
from .registry import lookup, register_mixer
from .spec import INIT_ONES, KEEP_F32, KEEP_SMALL, PagedKVSpec, TensorSpec


class LatentAttention(Part):
    libraries = ("gemm", "gemm_skinny", "gemm_tc", "gemm_tc2", "attention_latent", "attention", "sublayer")

    def __init__(self, dtype, names, *, hidden_size: int, num_heads: int, head_dim: int, rot_dim: int,
                 v_head_dim: int, kv_rank: int, scale: float, norm_eps: float, position: dict,
                 q_rank: int | None = None, window: int | None = None, cache_window="own",
                 sink: bool = False, reads_cache: bool = False):
        super().__init__(dtype, names)
        if kv_rank > 512:
            raise ConfigError(f"kv_rank={kv_rank}: the latent attention kernel takes up to 512")
        self.hidden_size, self.num_heads, self.head_dim, self.rot_dim = hidden_size, num_heads, head_dim, rot_dim
        self.v_head_dim, self.kv_rank, self.q_rank = v_head_dim, kv_rank, q_rank
        self.scale, self.norm_eps, self.window, self.sink_on = float(scale), float(norm_eps), window, bool(sink)
        self.reads_cache = reads_cache
        # how many positions the cache keeps: "own" this layer's window; None every position (a reader of
        # these rows may see further than the layer that writes them)
        self.cache_window = window if cache_window == "own" else cache_window
        if window is None and self.cache_window is not None:
            raise ConfigError("a layer that sees every key cannot live on a cache that keeps a window")
        if window is not None and self.cache_window is not None and self.cache_window < window:
            raise ConfigError(f"cache_window={cache_window} is shorter than the layer's window {window}")
        pos = dict(position or {"kind": "none"})
        self.position = lookup("position", pos.pop("kind"))(**pos)
        if pos and getattr(self.position, "layout", None) != "pairs":
            raise ConfigError("latent attention rotates pairs (2i, 2i+1): its position encoding must be of that layout")
        self.w_in = self.w_uq = self.w_ukT = self.w_uv = self.wo = None
        self.q_norm = self.c_norm = self.sink = None
        self._offsets: dict = {}

    # -- sizes ----------------------------------------------------------------------------------
    @property
    def q_width(self) -> int:
        return self.num_heads * (self.head_dim + self.rot_dim)

    @property
    def row_width(self) -> int:
        return self.kv_rank + self.rot_dim

    def _columns(self):
        """(query part, latent part) column offsets of the first projection."""
        first = self.q_rank if self.q_rank else self.q_width
        return 0, first

    def cache_spec(self):
        # one row per position for all heads, keys only: its first kv_rank elements are the value as well
        return PagedKVSpec(1, self.row_width, self.cache_window, v_head_dim=0)

    def declare(self, has):
        W, H, n, r = self.hidden_size, self.num_heads, self.names, self.kv_rank
        if self.q_rank:
            specs = [TensorSpec("dq", n["dq"], (self.q_rank, W)),
                     TensorSpec("dq_norm", n["dq_norm"], (self.q_rank,), INIT_ONES, KEEP_SMALL),
                     TensorSpec("uq", n["uq"], (self.q_width, self.q_rank))]
        else:
            specs = [TensorSpec("q", n["q"], (self.q_width, W))]
        if not self.reads_cache:
            specs += [TensorSpec("dkv", n["dkv"], (self.row_width, W)),
                      TensorSpec("dkv_norm", n["dkv_norm"], (r,), INIT_ONES, KEEP_SMALL)]
        specs += [TensorSpec("uk", n["uk"], (H * self.head_dim, r)),
                  TensorSpec("uv", n["uv"], (H * self.v_head_dim, r)),
                  TensorSpec("o", n["o"], (W, H * self.v_head_dim))]
        if self.sink_on:
            specs.append(TensorSpec("sink", n["sink"], (H,), keep=KEEP_F32))
        return specs

    def bind(self, tensors):
        H, r = self.num_heads, self.kv_rank
        first = [tensors["dq"] if self.q_rank else tensors["q"]]
        if not self.reads_cache:
            first.append(tensors["dkv"])
        self.w_in = pad_rows(torch.cat(first, 0), 16)
        self.w_uq = tensors.get("uq")
        self.q_norm, self.c_norm = tensors.get("dq_norm"), tensors.get("dkv_norm")
        # per head: W_uk_h^T as the [out = r, in = dim] matrix of a grouped product, W_uv_h as [vdim, r]
        self.w_ukT = tensors["uk"].view(H, self.head_dim, r).transpose(1, 2).contiguous()
        self.w_uv = tensors["uv"].view(H, self.v_head_dim, r).contiguous()
        self.wo = tensors["o"]
        self.sink = tensors.get("sink")

    def _per_head(self, M: int, device):
        """(offsets [H + 1] of H groups of M rows; the rows m * H + h in head-major order), made once per M."""
        got = self._offsets.get(M)
        if got is None or got[0].device != device:
            H = self.num_heads
            offsets = (torch.arange(H + 1, dtype=torch.int64) * M).to(torch.int32)
            rows = (torch.arange(M, dtype=torch.int64)[None, :] * H + torch.arange(H, dtype=torch.int64)[:, None])
            if len(self._offsets) > 64:
                self._offsets.clear()
            got = self._offsets[M] = (offsets.to(device), rows.reshape(-1).to(torch.int32).to(device))
        return got

    # -- the step -------------------------------------------------------------------------------
    def forward(self, ctx, x, cache, owns_cache=True):
        if owns_cache == self.reads_cache:
            raise KernelError("a layer without a latent projection must read another layer's cache, "
                              "and one with it must own its cache")
        H, M, r, rd = self.num_heads, ctx.M, self.kv_rank, self.rot_dim
        proj = linear(x, self.w_in)
        q_col, kv_col = self._columns()
        if self.q_rank:
            q = linear(kernels.rms_cols(proj, q_col, self.q_rank, self.q_norm, self.norm_eps), self.w_uq)
            q_off = 0
        else:
            q, q_off = proj, q_col
        inv_freq, rot = self.position.rotary(x.device)
        q_unrot, q_rot = kernels.latent_prepare(q, q_off, proj, kv_col, self.c_norm, self.norm_eps, inv_freq, rot,
                                                ctx.positions, ctx.row_seg, cache.block_table, cache.page_size,
                                                cache.pool, H, self.head_dim, rd, r, write_kv=owns_cache)
        offsets, head_major = self._per_head(M, x.device)
        # the query takes W_uk in: one product per head over that head's M rows
        q_abs = grouped_linear(q_unrot.view(H * M, self.head_dim), self.w_ukT, offsets, H * M, M).view(H, M, r)
        ctx.tap("attention_q", (q_abs, q_rot))
        decode_only = max(ctx.host_seg_len) <= 1
        tile_rows = 1 if decode_only else kernels.latent_attention_tile_rows(H, r, rd, self.dtype)
        num_chunks, scratch, chunk = 1, None, kernels.LATENT_ATTENTION_CHUNK
        if decode_only:
            # rows of decoded tokens: their keys in chunks, one block each, merged in chunk order
            num_chunks = plan.chunks(ctx, self.window, None, chunk)
            if self.window:                # a captured step plans for its longest sequence; a window spans fewer
                num_chunks = min(num_chunks, (self.window - 1) // chunk + 2)
            if num_chunks > 1:
                scratch = ctx.scratch(kernels.attention_scratch_bytes(M, H, r, num_chunks))
        o_lat = kernels.latent_attention(q_abs, q_rot, cache.pool, cache.block_table, cache.page_size, ctx.positions,
                                         ctx.row_seg, self.scale, window=self.window, sink=self.sink,
                                         tiles=attention_tiles(ctx, tile_rows), tile_rows=tile_rows,
                                         num_chunks=num_chunks, scratch=scratch, chunk=chunk)
        ctx.tap("attention_o", o_lat)
        # W_uv on each head's weighted sum of latents, then the heads side by side for the output product
        v = grouped_linear(o_lat.view(M * H, r), self.w_uv, offsets, H * M, M, a_rows=head_major)
        heads = kernels.heads_to_rows(v.view(H, M, self.v_head_dim))
        ctx.tap("attention_heads", heads)
        return linear(heads, self.wo, out_dtype=torch.float32)


register_mixer("latent_attention", LatentAttention)
