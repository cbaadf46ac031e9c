"""Arrangements of a mixer, a feed-forward and their norms into a layer.

Pre-norm decoder block of the reference (``ginfer/core/layer/transformer/encoder.cc:33-39``):
``x = norm1(h)``, ``a = mixer(x)``, ``r = h + a``, ``y = norm2(r)``, ``m = ffn(y)``,
``h' = r + m``.  The last addition is left to whoever consumes the block's output (the next
block's first norm or the final norm), which fuses it with its normalisation.
"""
from __future__ import annotations

import os

import torch

from .base import Block, Summed, make_part, register_block

# Steps of at most this many tokens (bfloat16) fold the additions and normalisations into the
# neighbouring products: the product before a norm leaves the sum, its product with the norm's
# weight and partial sums of squares, the product behind it divides by the rms, and a layer of a
# decode step is 5 kernels (q/k/v, attention, output, gate/up, down) instead of 7.  Off (0) by
# default: on a B200 at the 1.5B shape, batch 8, the step takes 1.245 ms with it against 1.213 ms
# without.  The kernels of a step overlap (each starts, and loads its weights, while the one
# before still runs): the two norm kernels cost 3.1 us each, but they are also 6 us in which the
# products behind them fetch weights, and the epilogues that replace them lengthen the products
# (+0.9 us the output product, +2.4 us q/k/v) on the path every token waits for.
FOLD_MAX_TOKENS = int(os.environ.get("GINFER_B200_FOLD_MAX_TOKENS", "0"))


class PreNormBlock(Block):
    def __init__(self, layer_spec):
        self.spec = layer_spec
        self.mixer_norm = make_part("norm", layer_spec.mixer_norm)
        self.mixer = make_part("mixer", layer_spec.mixer)
        self.feed_forward_norm = make_part("norm", layer_spec.feed_forward_norm)
        self.feed_forward = make_part("feed_forward", layer_spec.feed_forward)

    def parts(self):
        return (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward)

    def tensor_specs(self):
        out = []
        for p in self.parts():
            out.extend(p.tensor_specs())
        return out

    takes_next_norm = True

    def first_norm(self):
        return self.mixer_norm

    def load(self, tensors, dtype, device):
        for p in self.parts():
            p.load(tensors, dtype, device)

    def forward(self, x, delta, ctx, cache, then=None):
        """``x`` is a tensor (with ``delta`` still to be added) or a :class:`Summed` state.  For
        short bf16 steps the additions and normalisations are folded into the neighbouring
        products where the parts can do that: the mixer's and the feed-forward's last product
        add the residual, leave the statistics of the sum and its product with the next norm's
        weight (``Summed``), and their first product divides by the rms (``LazyNorm``).
        ``then``: the norm that consumes this block's output."""
        fold = ctx.dtype == torch.bfloat16 and ctx.num_tokens <= FOLD_MAX_TOKENS
        # the state before the mixer, and its normalisation
        n = None
        if isinstance(x, Summed):
            h = x.tensor
            if fold and self.mixer.takes_lazy_norm:
                n = self.mixer_norm.lazy(x, ctx.dtype)
            if n is None:
                _, n = self.mixer_norm.forward(h, None, out_dtype=ctx.dtype)
        else:
            h, n = self.mixer_norm.forward(x, delta)            # h = x + delta
        if fold and self.mixer.adds_residual:
            a = self.mixer.forward(n, ctx, cache, then=self.feed_forward_norm,
                                   residual=h if h.dtype == torch.float32 else h.float())
        else:
            a = self.mixer.forward(n, ctx, cache)
        # the state before the feed-forward, and its normalisation
        n2 = None
        if isinstance(a, Summed):
            r = a.tensor
            if fold and self.feed_forward.takes_lazy_norm:
                n2 = self.feed_forward_norm.lazy(a, ctx.dtype)
            if n2 is None:
                _, n2 = self.feed_forward_norm.forward(r, None, out_dtype=ctx.dtype)
        else:
            r, n2 = self.feed_forward_norm.forward(h, a)        # r = h + a
        if fold and then is not None and self.feed_forward.adds_residual \
                and r.dtype == torch.float32:
            m = self.feed_forward.forward(n2, ctx, residual=r, then=then)
        else:
            m = self.feed_forward.forward(n2, ctx)
        if isinstance(m, Summed):
            return m, None
        return r, m                                             # meaning r + m


register_block("prenorm", PreNormBlock)


class OutputNormBlock(Block):
    """Norms on the sublayers' outputs: ``x <- x + norm1(mixer(x))``, then
    ``x <- x + norm2(ff(x))``; the sublayers read the stream itself.  The stream ``x`` is fp32;
    the kernel that adds a normed output to it also writes the sum rounded to the activation
    dtype, which is what the next sublayer's products read (it travels to the next block in
    ``ctx.extras["act_copy"]``; a block that does not find its own ``x`` there rounds it anew).
    A layer without a feed-forward is the first line alone."""

    def __init__(self, layer_spec):
        self.spec = layer_spec
        self.mixer = make_part("mixer", layer_spec.mixer)
        self.mixer_norm = make_part("norm", layer_spec.mixer_norm)
        self.feed_forward = self.feed_forward_norm = None
        if layer_spec.feed_forward is not None:
            self.feed_forward = make_part("feed_forward", layer_spec.feed_forward)
            self.feed_forward_norm = make_part("norm", layer_spec.feed_forward_norm)

    def parts(self):
        return tuple(p for p in (self.mixer_norm, self.mixer, self.feed_forward_norm,
                                 self.feed_forward) if p is not None)

    def tensor_specs(self):
        out = []
        for p in self.parts():
            out.extend(p.tensor_specs())
        return out

    def load(self, tensors, dtype, device):
        for p in self.parts():
            p.load(tensors, dtype, device)

    def forward(self, x, delta, ctx, cache):
        if delta is not None:
            x = x.float() + delta.float()
        elif x.dtype != torch.float32:
            x = x.float()
        kept = ctx.extras.get("act_copy")
        h = kept[1] if kept is not None and kept[0] is x else x.to(ctx.dtype)
        a = self.mixer.forward(h, ctx, cache)
        x, h = self.mixer_norm.add_output(x, a, ctx.dtype)
        if self.feed_forward is not None:
            m = self.feed_forward.forward(h, ctx)
            x, h = self.feed_forward_norm.add_output(x, m, ctx.dtype)
        ctx.extras["act_copy"] = (x, h)
        return x, None


register_block("outnorm", OutputNormBlock)


class ScaledPreNormBlock(Block):
    """Pre-norm sublayers on a 32-bit stream whose outputs are scaled before they are added:
    ``x <- x + mult * s1 * mixer(norm1(x))``, ``x <- x + mult * s2 * ff(norm2(x))`` with
    per-channel scales ``s1``, ``s2`` (tensors of the layer; a name of ``None`` means no scale),
    then, if the layer has one, a stream input (``after``, family ``stream_input``).  A layer
    without a feed-forward is the first line alone.

    Each addition is one kernel that also writes what the next step reads: the norm of the new
    stream for the sublayer behind it (also the first norm of the NEXT run, ``then``, which
    travels there in ``ctx.extras["prenormed"]``), or its rounding to the activation dtype for a
    stream input that multiplies it by a matrix."""

    takes_next_norm = True

    def __init__(self, layer_spec, residual_mult: float = 1.0, mixer_scale: str | None = None,
                 feed_forward_scale: str | None = None, after=None):
        self.spec = layer_spec
        self.mult = float(residual_mult)
        self.mixer_norm = make_part("norm", layer_spec.mixer_norm)
        self.mixer = make_part("mixer", layer_spec.mixer)
        self.feed_forward = self.feed_forward_norm = None
        if layer_spec.feed_forward is not None:
            self.feed_forward_norm = make_part("norm", layer_spec.feed_forward_norm)
            self.feed_forward = make_part("feed_forward", layer_spec.feed_forward)
        self.after = make_part("stream_input", after) if after is not None else None
        self.scale_names = (mixer_scale, feed_forward_scale if self.feed_forward else None)
        self.scales = [None, None]
        self.size = None

    def parts(self):
        return tuple(p for p in (self.mixer_norm, self.mixer, self.feed_forward_norm,
                                 self.feed_forward, self.after) if p is not None)

    def tensor_specs(self):
        from .base import TensorSpec
        out = []
        for p in self.parts():
            out.extend(p.tensor_specs())
        width = next(s.shape[0] for s in self.mixer_norm.tensor_specs())
        out += [TensorSpec(n, (width,), "f32") for n in self.scale_names if n]
        return out

    def first_norm(self):
        return self.mixer_norm

    def load(self, tensors, dtype, device):
        for p in self.parts():
            p.load(tensors, dtype, device)
        self.scales = [tensors[n].float().contiguous() if n else None for n in self.scale_names]

    def _add(self, x, y, scale, ctx, then, want_act=False):
        """``x + mult * scale * y`` -> ``(x', x' in the activation dtype or None, then(x'))``."""
        from ..ops import prenorm
        from .base import PairSum
        kw = {}
        if isinstance(y, PairSum):                   # the kernel adds a token's pairs up itself
            kw["pairs"] = (y.pos_of_pair, y.weights, y.top)
            y = y.rows
        fused = then.fused() if then is not None else None
        if then is not None and fused is None:       # a norm the kernel cannot apply: on its own
            x, act, _ = prenorm.stream_update(x, ctx.dtype, y=y, scale=scale, mult=self.mult,
                                              want_act=want_act, **kw)
            return x, act, then.forward(x, None, want_sum=False, out_dtype=ctx.dtype)[1]
        if fused is not None:
            kw.update(norm=fused[0], norm_weight=fused[1], norm_bias=fused[2], norm_eps=fused[3])
        return prenorm.stream_update(x, ctx.dtype, y=y, scale=scale, mult=self.mult,
                                     want_act=want_act, **kw)

    def forward(self, x, delta, ctx, cache, then=None):
        if delta is not None:
            x = x.float() + delta.float()
        elif x.dtype != torch.float32:
            x = x.float()
        kept = ctx.extras.pop("prenormed", None)
        if kept is not None and kept[0] is x and kept[1] is self.mixer_norm:
            n = kept[2]
        else:
            n = self.mixer_norm.forward(x, None, want_sum=False, out_dtype=ctx.dtype)[1]
        a = self.mixer.forward(n, ctx, cache)
        act_for_after = self.after is not None and self.after.wants_act
        n_next = None
        if self.feed_forward is not None:
            x, _, n2 = self._add(x, a, self.scales[0], ctx, self.feed_forward_norm)
            if self.feed_forward.can_defer_sum:
                f = self.feed_forward.forward(n2, ctx, defer_sum=True)
            else:
                f = self.feed_forward.forward(n2, ctx)
            x, act, n_next = self._add(x, f, self.scales[1], ctx,
                                       then if self.after is None else None, act_for_after)
        else:
            x, act, n_next = self._add(x, a, self.scales[0], ctx,
                                       then if self.after is None else None, act_for_after)
        if self.after is not None:
            x, n_next = self.after.forward(x, act, ctx, self.mult, then)
        if n_next is not None:
            ctx.extras["prenormed"] = (x, then, n_next)
        return x, None


register_block("scaled_prenorm", ScaledPreNormBlock)


class PostNormBlock(Block):
    """Norms behind the sums: ``x <- norm1(alpha * x + mixer(x))``, then
    ``x <- norm2(alpha * x + ff(x))``; the sublayers read the stream itself, and the normed sum IS
    the stream.  ``x`` is fp32; the kernel that forms a normed sum also writes it rounded to the
    activation dtype, which is what the next sublayer's products read (it travels to the next block
    in ``ctx.extras["act_copy"]``, as with :class:`OutputNormBlock`).  A routed feed-forward may
    hand over its pairs' rows (:class:`PairSum`) and the same kernel adds them up.  A layer
    without a feed-forward is the first line alone."""

    def __init__(self, layer_spec, alpha: float = 1.0):
        self.spec = layer_spec
        self.alpha = float(alpha)
        self.mixer = make_part("mixer", layer_spec.mixer)
        self.mixer_norm = make_part("norm", layer_spec.mixer_norm)
        self.feed_forward = self.feed_forward_norm = None
        if layer_spec.feed_forward is not None:
            self.feed_forward = make_part("feed_forward", layer_spec.feed_forward)
            self.feed_forward_norm = make_part("norm", layer_spec.feed_forward_norm)

    def parts(self):
        return tuple(p for p in (self.mixer_norm, self.mixer, self.feed_forward_norm,
                                 self.feed_forward) if p is not None)

    def tensor_specs(self):
        out = []
        for p in self.parts():
            out.extend(p.tensor_specs())
        return out

    def load(self, tensors, dtype, device):
        for p in self.parts():
            p.load(tensors, dtype, device)

    def forward(self, x, delta, ctx, cache):
        from .base import PairSum
        if delta is not None:
            x = x.float() + delta.float()
        elif x.dtype != torch.float32:
            x = x.float()
        kept = ctx.extras.get("act_copy")
        h = kept[1] if kept is not None and kept[0] is x else x.to(ctx.dtype)
        a = self.mixer.forward(h, ctx, cache)
        x, h = self.mixer_norm.post(x, a, self.alpha, ctx.dtype)
        if self.feed_forward is not None:
            if self.feed_forward.can_defer_sum:
                m = self.feed_forward.forward(h, ctx, defer_sum=True)
            else:
                m = self.feed_forward.forward(h, ctx)
            if isinstance(m, PairSum):
                x, h = self.feed_forward_norm.post(x, m.rows, self.alpha, ctx.dtype,
                                                   pairs=(m.pos_of_pair, m.weights, m.top))
            else:
                x, h = self.feed_forward_norm.post(x, m, self.alpha, ctx.dtype)
        ctx.extras["act_copy"] = (x, h)
        return x, None


register_block("postnorm", PostNormBlock)


class SandwichBlock(Block):
    """Norms before AND behind every sublayer on a 32-bit stream: ``x <- x + norm1b(mixer(norm1(
    x)))``, then ``x <- x + norm2b(ff(norm2(x)))``; a layer without a feed-forward is the first line
    alone.  ``mixer_out_norm`` / ``feed_forward_out_norm`` are the norms behind the sublayers (the
    layer's ``mixer_norm`` / ``feed_forward_norm`` the ones in front).

    ``depth_states = n`` > 0: the layer ends with an average over the model's depth.  Its result
    is kept as state ``n - 1`` of the step's history (``ctx.extras["depth_history"]``, made by the
    embedding, whose output is state 0) and what goes on to the next layer is ``sum_j w[j] *
    state_j`` over ``j < n`` with the layer's tensor ``depth_name`` (``n`` weights, 32-bit).

    Every sublayer ends in ONE kernel: output norm, addition, (average,) and the norm in front of
    the next sublayer, also the first norm of the NEXT run (``then``), which travels there in
    ``ctx.extras["prenormed"]``."""

    takes_next_norm = True

    def __init__(self, layer_spec, mixer_out_norm, feed_forward_out_norm=None,
                 depth_states: int = 0, depth_name: str = "dwa"):
        self.spec = layer_spec
        self.mixer_norm = make_part("norm", layer_spec.mixer_norm)
        self.mixer = make_part("mixer", layer_spec.mixer)
        self.mixer_out_norm = make_part("norm", mixer_out_norm)
        self.feed_forward = self.feed_forward_norm = self.feed_forward_out_norm = None
        if layer_spec.feed_forward is not None:
            self.feed_forward_norm = make_part("norm", layer_spec.feed_forward_norm)
            self.feed_forward = make_part("feed_forward", layer_spec.feed_forward)
            self.feed_forward_out_norm = make_part("norm", feed_forward_out_norm)
        for n in (self.mixer_norm, self.mixer_out_norm, self.feed_forward_norm,
                  self.feed_forward_out_norm):
            if n is not None and not hasattr(n, "weight32"):
                raise ValueError("the norms of this block are RMS norms (kind 'rmsnorm')")
        self.depth_states, self.depth_name = int(depth_states), depth_name
        if self.depth_states == 1 or self.depth_states < 0:
            raise ValueError("an average over the depth takes at least two states")
        self.depth_w = None

    def parts(self):
        return tuple(p for p in (self.mixer_norm, self.mixer, self.mixer_out_norm,
                                 self.feed_forward_norm, self.feed_forward,
                                 self.feed_forward_out_norm) if p is not None)

    def tensor_specs(self):
        from .base import TensorSpec
        out = []
        for p in self.parts():
            out.extend(p.tensor_specs())
        if self.depth_states:
            out.append(TensorSpec(self.depth_name, (self.depth_states,), "f32"))
        return out

    def first_norm(self):
        return self.mixer_norm

    def load(self, tensors, dtype, device):
        for p in self.parts():
            p.load(tensors, dtype, device)
        if self.depth_states:
            self.depth_w = tensors[self.depth_name].float().contiguous()

    def _end(self, x, y, out_norm, ctx, nxt, average=False, y_bias=None):
        """One sublayer's end -> ``(stream, norm of the stream for ``nxt`` or None)``.  ``y_bias``:
        a bias the sublayer left for this kernel to add to its output."""
        from ..ops import depth
        kw = {"y_bias": y_bias} if y_bias is not None else {}
        if average and self.depth_states:
            hist = ctx.extras.get("depth_history")
            if hist is None or hist.shape[0] < self.depth_states:
                raise RuntimeError("this layer averages over the depth, but the step has no "
                                   "history of that many states (the embedding makes it)")
            kw.update(history=hist, mix_weights=self.depth_w, n_before=self.depth_states - 1)
        fused = nxt is not None and hasattr(nxt, "weight32") and not nxt.weight_offset
        if fused:
            kw.update(next_weight=nxt.weight32(), next_eps=nxt.eps)
        x, n = depth.sandwich_update(x, y, out_norm.weight32(), out_norm.eps, ctx.dtype, **kw)
        if nxt is not None and not fused:
            n = nxt.forward(x, None, want_sum=False, out_dtype=ctx.dtype)[1]
        return x, n

    def forward(self, x, delta, ctx, cache, then=None):
        if delta is not None:
            x = x.float() + delta.float()
        elif x.dtype != torch.float32:
            x = x.float()
        kept = ctx.extras.pop("prenormed", None)
        if kept is not None and kept[0] is x and kept[1] is self.mixer_norm:
            n = kept[2]
        else:
            n = self.mixer_norm.forward(x, None, want_sum=False, out_dtype=ctx.dtype)[1]
        a = self.mixer.forward(n, ctx, cache)
        if self.feed_forward is not None:
            x, n2 = self._end(x, a, self.mixer_out_norm, ctx, self.feed_forward_norm)
            if getattr(self.feed_forward, "can_defer_bias", False):
                f, fb = self.feed_forward.forward(n2, ctx, defer_bias=True)
            else:
                f, fb = self.feed_forward.forward(n2, ctx), None
            x, n_next = self._end(x, f, self.feed_forward_out_norm, ctx, then, average=True,
                                  y_bias=fb)
        else:
            x, n_next = self._end(x, a, self.mixer_out_norm, ctx, then, average=True)
        if n_next is not None:
            ctx.extras["prenormed"] = (x, then, n_next)
        return x, None


register_block("sandwich", SandwichBlock)
