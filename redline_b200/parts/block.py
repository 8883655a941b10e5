"""Pre-norm residual block: h += mixer(norm(h)); h += ffn(norm(h)), the residual
stream h in float32 (reference: src/cuda/model/llama.cpp:116-139).  A layer without a
feed-forward stops after the first half.  Beside it the arrangements that norm a
sublayer's output: on both sides ("sandwich") or on the output only ("outnorm")."""

from __future__ import annotations

import torch

from .base import Block, op_mark, register


@register("block", "prenorm")
class PreNormBlock(Block):
    def first_norm(self):
        return self.mixer_norm

    @staticmethod
    def _fused(ctx, hand, norm, next_norm, call):
        """Runs a part's fused form with the hand-over fields of the context set for it; returns
        (taken, what the part left for ``next_norm``)."""
        ctx.hand_in = hand if (hand is not None and hand.norm is norm) else None
        ctx.next_norm, ctx.hand_out = next_norm, None
        try:
            taken = call()
            left = ctx.hand_out if taken else None
        finally:
            ctx.hand_in = ctx.hand_out = ctx.next_norm = None
        return taken, (left if (left is not None and left.norm is next_norm) else None)

    def forward(self, residual, pending, ctx, cache, state):
        rt = self.rt
        T = ctx.T
        x = None
        hand, ctx.block_hand = ctx.block_hand, None       # from the block before, for this block's first norm
        # small batches: the mixer and the feed-forward may fuse the norm into their first
        # kernel and the residual add into their last (nothing is then left pending)
        taken = False
        if pending is None:
            taken, hand = self._fused(ctx, hand, self.mixer_norm,
                                      self.ffn_norm if self.ffn is not None else ctx.block_next_norm,
                                      lambda: self.mixer.forward_into(residual, self.mixer_norm, ctx, cache, state))
        if taken:
            a = None
        else:
            hand = None
            x = rt.workspace.get("block.normed", (rt.max_tokens, residual.shape[1]), rt.dtype)[:T]
            self.mixer_norm.add_norm(residual, pending, x, rows=T)
            op_mark(ctx, "add+rmsnorm", nbytes=self._norm_bytes(residual, pending, x))
            a = self.mixer.forward(x, ctx, cache, state)
        if self.ffn is None:               # a layer with a mixer only: its output is what is left to add
            ctx.block_hand = hand if a is None else None
            return a
        if a is None:
            taken, hand = self._fused(ctx, hand, self.ffn_norm, ctx.block_next_norm,
                                      lambda: self.ffn.forward_into(residual, self.ffn_norm, ctx))
            if taken:
                ctx.block_hand = hand
                return None
        if x is None:
            x = rt.workspace.get("block.normed", (rt.max_tokens, residual.shape[1]), rt.dtype)[:T]
        self.ffn_norm.add_norm(residual, a, x, rows=T)
        op_mark(ctx, "add+rmsnorm", nbytes=self._norm_bytes(residual, a, x))
        return self.ffn.forward(x, ctx)

    @staticmethod
    def _norm_bytes(residual, delta, out) -> float:
        """The stream read (and written back when something is added), the addend read, the normed rows written."""
        n = residual.numel() * residual.element_size() * (2 if delta is not None else 1)
        n += out.numel() * out.element_size()
        if delta is not None:
            n += delta.numel() * delta.element_size()
        return float(n)


@register("block", "sandwich")
class SandwichBlock(Block):
    """h += norm_1b(mixer(norm_1(h))); h += norm_2b(ffn(norm_2(h))): every sublayer's input AND output is
    normed.  ``mixer_post_norm`` / ``ffn_post_norm`` are set by the model builder from the layer's spec.
    The add of a sublayer's normed output and the input norm of the sublayer after it are one kernel
    (``add_post_norm``), also across blocks: the block's last kernel norms the stream for the first norm of
    the block after it (``ctx.block_next_norm``) and leaves the result in ``ctx.block_normed``, which that
    block takes instead of running its first norm.  The block leaves nothing pending."""

    mixer_post_norm = None
    ffn_post_norm = None

    def parts(self):
        return super().parts() + [p for p in (self.mixer_post_norm, self.ffn_post_norm) if p is not None]

    def first_norm(self):
        return self.mixer_norm

    def forward(self, residual, pending, ctx, cache, state):
        rt = self.rt
        T = ctx.T
        ctx.block_hand = None
        ready, ctx.block_normed = ctx.block_normed, None
        x = rt.workspace.get("block.normed", (rt.max_tokens, residual.shape[1]), rt.dtype)[:T]
        if not (pending is None and ready is not None and ready[0] is self.mixer_norm):
            self.mixer_norm.add_norm(residual, pending, x, rows=T)
            op_mark(ctx, "add+norm", nbytes=PreNormBlock._norm_bytes(residual, pending, x))
        a = self.mixer.forward(x, ctx, cache, state)
        if self.ffn is None:
            self._last(self.mixer_post_norm, residual, a, x, ctx)
            return None
        if not self.mixer_post_norm.add_post_norm(residual, a, self.ffn_norm, x, rows=T):
            self.ffn_norm.add_norm(residual, None, x, rows=T)
        op_mark(ctx, "post_norm+add+norm", nbytes=PreNormBlock._norm_bytes(residual, a, x))
        f = self.ffn.forward(x, ctx)
        self._last(self.ffn_post_norm, residual, f, x, ctx)
        return None

    def _last(self, post_norm, residual, delta, x, ctx) -> None:
        """The block's last kernel: the normed add, and with it the first norm of the block after this one
        when that norm can share the kernel (x, this block's input buffer, is free by now)."""
        nxt = ctx.block_next_norm
        if nxt is not None and post_norm.add_post_norm(residual, delta, nxt, x, rows=ctx.T):
            ctx.block_normed = (nxt, x)
            op_mark(ctx, "post_norm+add+norm", nbytes=PreNormBlock._norm_bytes(residual, delta, x))
            return
        if nxt is None:
            post_norm.add_post_norm(residual, delta, None, None, rows=ctx.T)
        op_mark(ctx, "post_norm+add", nbytes=PreNormBlock._norm_bytes(residual, delta, x))


@register("block", "outnorm")
class OutNormBlock(Block):
    """h += norm_1(mixer(h)); h += norm_2(ffn(h)): the sublayers read the stream itself and only what they
    put out is normed.  ``mixer_post_norm`` / ``ffn_post_norm`` are set by the model builder from the
    layer's spec; ``mixer_norm`` and ``ffn_norm`` are None.  In a 16-bit engine the sublayers' products take
    the stream rounded to the activation type; the kernel that adds a sublayer's normed output also writes
    that rounded copy for the sublayer after it, across blocks too (``ctx.block_normed``), so every sublayer
    costs one row-wise kernel.  A float32 engine hands the sublayers the stream as it is.  The block leaves
    nothing pending."""

    reads_stream = True
    mixer_post_norm = None
    ffn_post_norm = None
    AS_IS = "the stream as it is"          # marks ctx.block_normed: the buffer holds the stream, not a norm of it

    def parts(self):
        return super().parts() + [p for p in (self.mixer_post_norm, self.ffn_post_norm) if p is not None]

    def forward(self, residual, pending, ctx, cache, state):
        rt = self.rt
        T = ctx.T
        ctx.block_hand = None
        ready, ctx.block_normed = ctx.block_normed, None
        copy = rt.dtype != torch.float32
        x = rt.workspace.get("block.normed", (rt.max_tokens, residual.shape[1]), rt.dtype)[:T] if copy else residual
        if pending is not None or (copy and not (ready is not None and ready[0] is self.AS_IS)):
            from ..ops import kernels
            kernels.sandwich_norm(residual, pending, None, None, x if copy else None, 0.0, kernels.NORM_RMS, rows=T)
            op_mark(ctx, "stream_copy", nbytes=PreNormBlock._norm_bytes(residual, pending, x))
        a = self.mixer.forward(x, ctx, cache, state)
        last = self.ffn is None
        nxt = copy and (not last or isinstance(ctx.block_next, OutNormBlock))
        self.mixer_post_norm.add_post_cast(residual, a, x if nxt else None, rows=T)
        op_mark(ctx, "post_norm+add", nbytes=PreNormBlock._norm_bytes(residual, a, x))
        if not last:
            f = self.ffn.forward(x, ctx)
            nxt = copy and isinstance(ctx.block_next, OutNormBlock)
            self.ffn_post_norm.add_post_cast(residual, f, x if nxt else None, rows=T)
            op_mark(ctx, "post_norm+add", nbytes=PreNormBlock._norm_bytes(residual, f, x))
        if nxt:
            ctx.block_normed = (self.AS_IS, x)
        return None
