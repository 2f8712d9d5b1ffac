"""Arrangements of a layer's parts."""

from __future__ import annotations

from .base import Block, register_block


class PreNormBlock(Block):
    """x += mixer(norm1(x)); x += ffn(norm2(x))  (``models/gpt2.py:435-438``).
    The residual stream x is float32; the sums are made in the mixer's and the
    feed-forward's last epilogue."""

    KIND = "pre_norm"
    PARTS = ("norm1", "mixer", "norm2", "ffn")

    def forward(self, x, ctx, caches):
        x = self.mixer.forward(self.norm1.forward(x, ctx), x, ctx, caches.get("mixer"))
        return self.ffn.forward(self.norm2.forward(x, ctx), x, ctx)

    def lower(self, builder, x, caches):
        h = self.norm1.lower(builder, x)
        x = self.mixer.lower(builder, h, x, caches.get("mixer"))
        builder.release(h)
        h = self.norm2.lower(builder, x)
        x = self.ffn.lower(builder, h, x)
        builder.release(h)
        return x


class SandwichBlock(Block):
    """Norm before and after each sublayer, a short convolution over time in front of each:
    x += norm1b(mixer(conv1(norm1(x)))); x += norm2b(ffn(conv2(norm2(x)))).  The closing norms carry
    the residual multiplier and add to the stream themselves (``RMSNorm.add_normed``); the norm
    in front and the convolution are one kernel (``TimeConv.forward``)."""

    KIND = "sandwich"
    PARTS = ("norm1", "conv1", "mixer", "norm1b", "norm2", "conv2", "ffn", "norm2b")

    def forward(self, x, ctx, caches):
        h = self.conv1.forward(x, self.norm1, ctx, caches["conv1"])
        x = self.norm1b.add_normed(x, self.mixer.forward(h, None, ctx, caches.get("mixer")))
        if "ffn" in self.parts:
            h = self.conv2.forward(x, self.norm2, ctx, caches["conv2"])
            x = self.norm2b.add_normed(x, self.ffn.forward(h, None, ctx))
        return x


class SandwichMixerBlock(SandwichBlock):
    """The same without a feed-forward."""

    KIND = "sandwich_mixer_only"
    PARTS = ("norm1", "conv1", "mixer", "norm1b")


register_block(PreNormBlock.KIND, PreNormBlock)
register_block(SandwichBlock.KIND, SandwichBlock)
register_block(SandwichMixerBlock.KIND, SandwichMixerBlock)


class PostNormBlock(Block):
    """The sublayers read the residual stream itself and only their outputs are normed:
    x += norm1(mixer(shift(x))); x += norm2(ffn(x)).  ``shift`` blends every channel of the
    mixer's input with the previous token's (``TokenShift``); it also brings the stream into the
    compute dtype, which a plain conversion does for the feed-forward.  The closing norms carry
    the residual multiplier and add to the stream themselves (``RMSNorm.add_normed``)."""

    KIND = "post_norm"
    PARTS = ("shift", "mixer", "norm1", "ffn", "norm2")

    def forward(self, x, ctx, caches):
        h = self.shift.forward(x, ctx, caches["shift"])
        x = self.norm1.add_normed(x, self.mixer.forward(h, None, ctx, caches.get("mixer")))
        if "ffn" in self.parts:
            x = self.norm2.add_normed(x, self.ffn.forward(self.shift.convert(x), None, ctx))
        return x


class PostNormMixerBlock(PostNormBlock):
    """The same without a feed-forward."""

    KIND = "post_norm_mixer_only"
    PARTS = ("shift", "mixer", "norm1")


register_block(PostNormBlock.KIND, PostNormBlock)
register_block(PostNormMixerBlock.KIND, PostNormMixerBlock)


class DoubleNormBlock(Block):
    """Norm before and after each sublayer, nothing else between:
    x += norm1b(mixer(norm1(x))); x += norm2b(ffn(norm2(x))).  The closing norms add to the stream
    themselves (``RMSNorm.add_normed``); the mixer's closing norm and the feed-forward's opening norm are
    one kernel (``RMSNorm.add_normed_then``)."""

    KIND = "double_norm"
    PARTS = ("norm1", "mixer", "norm1b", "norm2", "ffn", "norm2b")

    def forward(self, x, ctx, caches):
        y = self.mixer.forward(self.norm1.forward(x, ctx), None, ctx, caches.get("mixer"))
        if "ffn" not in self.parts:
            return self.norm1b.add_normed(x, y)
        h = self.norm1b.add_normed_then(x, y, self.norm2)
        return self.norm2b.add_normed(x, self.ffn.forward(h, None, ctx))


class DoubleNormMixerBlock(DoubleNormBlock):
    """The same without a feed-forward."""

    KIND = "double_norm_mixer_only"
    PARTS = ("norm1", "mixer", "norm1b")


register_block(DoubleNormBlock.KIND, DoubleNormBlock)
register_block(DoubleNormMixerBlock.KIND, DoubleNormMixerBlock)
