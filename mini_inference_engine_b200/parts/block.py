"""The arrangement of parts in a layer.  ``prenorm_residual`` is Llama's: the mixer and the
feed-forward each read a normed copy of the residual stream and add their output to it.  The sum
is fused into the *next* norm, so a block takes the pending ``delta`` and returns the next one
(inference_engine/model.py:169-184: the MLP output and the residual go into the next layer's fused
add+norm, after the last layer into the final norm)."""
from __future__ import annotations

from dataclasses import dataclass

from ..weights.loader import TensorSpec
from .base import Part, ResidualSink, StreamValue, register_part


def _sink_for(producer, consumer, norm, res, num_tokens):
    """The offer to ``producer`` (None if it would not take one): it may add to the stream itself when
    the part behind ``norm`` can take that norm as a factor on its first product."""
    if not getattr(producer, "takes_sink", False) or consumer is None or norm is None:
        return None
    ok = getattr(consumer, "defers_norm", None)
    return ResidualSink(res, norm) if ok is not None and ok(num_tokens) else None


class Block(Part):
    """An arrangement of parts.  ``roles`` names the parts it is made of and the category each is
    built from (role -> "mixer" | "feed_forward" | "norm" | ...); the model builds them from the
    layer's description and passes them to the constructor by role name.  A block has one cache: what
    ``cache_need()`` says (by default its ``mixer``'s need, nothing for a block without one)."""
    roles: dict = {}

    def __init__(self, **parts):
        for role, part in parts.items():
            setattr(self, role, part)
        self._roles = tuple(parts)

    def parts(self) -> list:
        return [getattr(self, r) for r in self._roles]

    def cache_need(self):
        mixer = getattr(self, "mixer", None)
        return mixer.cache_need() if mixer is not None else None

    def forward(self, delta, res, ctx, cache):
        raise NotImplementedError


class PreNormResidual(Block):
    roles = {"mixer": "mixer", "feed_forward": "feed_forward", "mixer_norm": "norm", "feed_forward_norm": "norm"}

    def forward(self, delta, res, ctx, cache, next_block=None):
        """``next_block``: the block that runs after this one, if it reads the stream through a norm
        and a mixer as this one does (then the feed-forward may prepare that norm's output)."""
        n = res.shape[0]
        x = self.mixer_norm(delta, res)
        sink = _sink_for(self.mixer, self.feed_forward, self.feed_forward_norm, res, n)
        a = self.mixer.forward(x, ctx, cache, sink) if sink is not None else self.mixer.forward(x, ctx, cache)
        x = self.feed_forward_norm(a, res)
        sink = _sink_for(self.feed_forward, getattr(next_block, "mixer", None), getattr(next_block, "mixer_norm", None), res, n)
        return self.feed_forward.forward(x, ctx, sink) if sink is not None else self.feed_forward.forward(x, ctx)


register_part("block", "prenorm_residual", PreNormResidual)


class Branches:
    """What a mixer may return instead of one tensor: several outputs that the block's norm adds together, each
    optionally RMS-normed over its row with ``inner_weights[k]`` first, the sum multiplied by ``coef``."""

    def __init__(self, deltas, inner_weights=(), coef: float = 1.0):
        self.deltas, self.inner_weights, self.coef = tuple(deltas), tuple(inner_weights), coef


class PostNormResidual(Block):
    """Norm after the sum: x <- mixer_norm(alpha x + mixer(x)), then x <- feed_forward_norm(alpha x + ff(x)); both
    sublayers read the stream itself.  The sum and the norm are one kernel (the norm's ``apply``), which also leaves
    the stream in the activation type for the next reader.  ``feed_forward`` may be absent (``has_feed_forward``
    False): the layer is then its mixer half only."""
    roles = {"mixer": "mixer", "feed_forward": "feed_forward", "mixer_norm": "norm", "feed_forward_norm": "norm"}

    def __init__(self, alpha: float = 1.0, **parts):
        super().__init__(**parts)
        self.alpha = float(alpha)

    def _summed(self, norm, res, y):
        if isinstance(y, Branches):
            return norm.apply(res, y.deltas, y.inner_weights, alpha=self.alpha, coef=y.coef)
        return norm.apply(res, (y,), alpha=self.alpha)

    def forward(self, delta, res, ctx, cache):
        if isinstance(delta, StreamValue):
            x = delta.x
        else:
            if delta is not None:
                raise ValueError("a post-norm block cannot take a pending sum from the block before it")
            x = res if self.mixer.rt.dtype == res.dtype else res.to(self.mixer.rt.dtype)
        x = self._summed(self.mixer_norm, res, self.mixer.forward(x, ctx, cache))
        if getattr(self, "feed_forward", None) is not None:
            x = self._summed(self.feed_forward_norm, res, self.feed_forward.forward(x, ctx))
        return StreamValue(x)


class PostNormMixerOnly(PostNormResidual):
    """The same without a feed-forward half."""
    roles = {"mixer": "mixer", "mixer_norm": "norm"}


register_part("block", "postnorm_residual", PostNormResidual)
register_part("block", "postnorm_mixer_only", PostNormMixerOnly)


class HyperConnection(Part):
    """How one sublayer is wired to a stream kept in ``streams`` copies x_1 .. x_S: it reads u = sum_s in[s] x_s and,
    with y its output, writes x_t <- sum_s mix[s, t] x_s + out[t] y into all copies at once (mix is indexed
    [from, to]).  The coefficients are tensors of the checkpoint: 'in' [S], 'out' [S], 'mix' [S, S]."""

    def __init__(self, streams: int):
        self.streams = streams

    def tensor_specs(self):
        S = self.streams
        return {"in": TensorSpec((S,), f"normal:{1.0 / S}:0.2"), "out": TensorSpec((S,), "normal:1:0.2"),
                "mix": TensorSpec((S, S), f"normal:{1.0 / S}:0.3")}

    def bind(self, tensors, rt):
        self.rt = rt
        small = lambda n: tensors[n].float().reshape(-1).to(rt.device).contiguous()      # read as float32 by the kernel
        self.in_coef, self.out_coef, self.mix = small("in"), small("out"), small("mix")


register_part("connection", "hyper", HyperConnection)


@dataclass
class PendingUpdate:
    """What a block over a stream in several copies leaves for the next reader of the stream: the output ``y`` of its
    last sublayer and the ``connection`` that says how it goes into the copies.  The next norm's kernel applies it."""
    y: object
    connection: object


class HyperConnected(Block):
    """A pre-norm layer over a stream kept in several copies: each sublayer reads a mixture of the copies through its
    norm and writes into all of them (``HyperConnection``).  The write of one sublayer and the read and norm of the
    next are one kernel (the norm's ``read``), so a block takes the pending update of the block before and returns
    its own; the norm in front of the output head applies the last one."""
    roles = {"mixer": "mixer", "feed_forward": "feed_forward", "mixer_norm": "norm", "feed_forward_norm": "norm",
             "mixer_connection": "connection", "feed_forward_connection": "connection"}

    def forward(self, delta, res, ctx, cache):
        if delta is not None and not isinstance(delta, PendingUpdate):
            raise ValueError("a block over several copies of the stream takes a pending update or nothing")
        x = self.mixer_norm.read(res, delta, self.mixer_connection)
        pending = PendingUpdate(self.mixer.forward(x, ctx, cache), self.mixer_connection)
        if getattr(self, "feed_forward", None) is None:
            return pending
        x = self.feed_forward_norm.read(res, pending, self.feed_forward_connection)
        return PendingUpdate(self.feed_forward.forward(x, ctx), self.feed_forward_connection)


class HyperConnectedMixerOnly(HyperConnected):
    """The same without a feed-forward half."""
    roles = {"mixer": "mixer", "mixer_norm": "norm", "mixer_connection": "connection"}


register_part("block", "hyper_connected", HyperConnected)
register_part("block", "hyper_connected_mixer_only", HyperConnectedMixerOnly)
