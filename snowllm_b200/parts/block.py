"""How a layer's parts sit around the residual stream.

``prenorm`` (snowllm/models/lfm2/layers.py:91-104): x += mixer(norm(x)); x += ffn(norm(x)).
The float residual sum is fused into the norm that follows it, so a block takes the delta that the
previous block left and returns its own last delta; the model adds the final one.

``output_norm``: x += norm(mixer(x)); x += norm(ffn(x)).  The sums are made at once (nothing is left for
the next block), and the block hands on the stream's copy in the compute dtype.

``parallel``: h = norm(x); x += mixer(h) + ffn(h).  One norm, both sublayers read its output; the sum of
their outputs is left to the norm that follows (``kernels.DeltaSum``)."""
from __future__ import annotations

from ..ops import kernels
from ..trace import span
from .registry import register_block


class PreNormBlock:
    def __init__(self, mixer, ffn, mixer_norm, ffn_norm):
        self.mixer, self.ffn, self.mixer_norm, self.ffn_norm = mixer, ffn, mixer_norm, ffn_norm
        self._names = tuple(f"{what}:{type(part).__name__}" for what, part in
                            (("norm", mixer_norm), ("mixer", mixer), ("norm", ffn_norm), ("ffn", ffn)))

    def parts(self):
        return tuple(p for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn) if p is not None)

    def forward(self, ctx, residual, delta, cache, owns_cache=True):
        with span(self._names[0]):
            x = self.mixer_norm.forward(ctx, residual, delta)
        ctx.tap("mixer_in", x)
        with span(self._names[1]):
            delta = self.mixer.forward(ctx, x, cache, owns_cache)
        ctx.tap("mixer_out", delta)
        if self.ffn is None:
            return delta
        fused = getattr(self.ffn, "forward_from_residual", None)
        if fused is not None:          # a feed-forward that can take the norm before it into its first kernel
            with span(self._names[3]):
                out = fused(ctx, residual, delta, self.ffn_norm)
            if out is not None:
                ctx.tap("ffn_out", out)
                return out
        with span(self._names[2]):
            x = self.ffn_norm.forward(ctx, residual, delta)
        ctx.tap("ffn_in", x)
        with span(self._names[3]):
            delta = self.ffn.forward(ctx, x)
        ctx.tap("ffn_out", delta)
        return delta


class OutputNormBlock:
    """x += norm(mixer(x)); x += norm(ffn(x)): each norm sits on its sublayer's OUTPUT, and the sublayers
    read the residual stream itself.  The stream is float; its copy in the compute dtype, which the next
    sublayer reads, comes out of the kernel that adds the normalised output (``norm.add_normed``) and is
    handed from block to block through the step's memo.  A layer may have the mixer's sublayer alone."""

    def __init__(self, mixer, ffn, mixer_norm, ffn_norm):
        self.mixer, self.ffn, self.mixer_norm, self.ffn_norm = mixer, ffn, mixer_norm, ffn_norm
        self._names = tuple(f"{what}:{type(part).__name__}" for what, part in
                            (("mixer", mixer), ("norm", mixer_norm), ("ffn", ffn), ("norm", ffn_norm)))

    def parts(self):
        return tuple(p for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn) if p is not None)

    def forward(self, ctx, residual, delta, cache, owns_cache=True):
        if delta is not None:                      # a block of another arrangement left its sum to us
            kernels.residual_add(residual, delta.dense() if hasattr(delta, "dense") else delta)
        key = ("stream_copy", id(residual))
        x = ctx.memo.get(key)
        if x is None or delta is not None:
            x = residual if ctx.dtype == residual.dtype else kernels.cast_rows(residual, ctx.dtype)
        ctx.tap("mixer_in", x)
        with span(self._names[0]):
            y = self.mixer.forward(ctx, x, cache, owns_cache)
        ctx.tap("mixer_out", y)
        with span(self._names[1]):
            x = self.mixer_norm.add_normed(ctx, residual, y)
        if self.ffn is not None:
            ctx.tap("ffn_in", x)
            with span(self._names[2]):
                y = self.ffn.forward(ctx, x)
            y = y.dense() if hasattr(y, "dense") else y
            ctx.tap("ffn_out", y)
            with span(self._names[3]):
                x = self.ffn_norm.add_normed(ctx, residual, y)
        ctx.memo[key] = x
        if ctx.taps is not None:
            ctx.tap("layer_out", residual.clone())
        return None


class ParallelBlock:
    """h = norm(x); x += mixer(h) + ffn(h): the layer has ONE norm and both sublayers read its output.  The
    block leaves the two outputs as a ``kernels.DeltaSum``: the next norm forms a + b, adds it into the float
    residual and normalises in one kernel.  A layer may have the mixer alone."""
    single_norm = True         # the model builds it without a second norm

    def __init__(self, mixer, ffn, mixer_norm, ffn_norm=None):
        if ffn_norm is not None:
            raise ValueError("a parallel layer has one norm")
        self.mixer, self.ffn, self.mixer_norm, self.ffn_norm = mixer, ffn, mixer_norm, None
        self._names = tuple(f"{what}:{type(part).__name__}" for what, part in
                            (("norm", mixer_norm), ("mixer", mixer), ("ffn", ffn)))

    def parts(self):
        return tuple(p for p in (self.mixer_norm, self.mixer, self.ffn) if p is not None)

    def forward(self, ctx, residual, delta, cache, owns_cache=True):
        with span(self._names[0]):
            x = self.mixer_norm.forward(ctx, residual, delta)
        ctx.tap("mixer_in", x)
        with span(self._names[1]):
            out = self.mixer.forward(ctx, x, cache, owns_cache)
        ctx.tap("mixer_out", out)
        if self.ffn is not None:
            ctx.tap("ffn_in", x)
            with span(self._names[2]):
                f = self.ffn.forward(ctx, x)
            ctx.tap("ffn_out", f)
            out = kernels.DeltaSum(out, f)
        if ctx.taps is not None:
            ctx.tap("layer_out", residual + (out.dense() if hasattr(out, "dense") else out))
        return out


register_block("prenorm", PreNormBlock)
register_block("parallel", ParallelBlock)
register_block("output_norm", OutputNormBlock)
