"""The arrangement of parts in a layer.  ``prenorm_residual`` is Llama's: the mixer and the
feed-forward each read a normed copy of the residual stream and add their output to it.  The sum
is fused into the *next* norm, so a block takes the pending ``delta`` and returns the next one
(inference_engine/model.py:169-184: the MLP output and the residual go into the next layer's fused
add+norm, after the last layer into the final norm)."""
from __future__ import annotations

from dataclasses import dataclass

from ..weights.loader import TensorSpec
from ..kernels import ops
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
    """``feed_forward`` (with its norm) may be absent: the layer is then its mixer half, and the mixer's output is what
    the next reader of the stream adds."""
    roles = {"mixer": "mixer", "feed_forward": "feed_forward", "mixer_norm": "norm", "feed_forward_norm": "norm"}
    optional_roles = ("feed_forward", "feed_forward_norm")

    def forward(self, delta, res, ctx, cache, next_block=None):
        """``next_block``: the block that runs after this one, if it reads the stream through a norm
        and a mixer as this one does (then the feed-forward may prepare that norm's output)."""
        n = res.shape[0]
        x = self.mixer_norm(delta, res)
        ff = getattr(self, "feed_forward", None)
        sink = _sink_for(self.mixer, ff, getattr(self, "feed_forward_norm", None), res, n)
        a = self.mixer.forward(x, ctx, cache, sink) if sink is not None else self.mixer.forward(x, ctx, cache)
        if ff is None:
            return a
        x = self.feed_forward_norm(a, res)
        sink = _sink_for(self.feed_forward, getattr(next_block, "mixer", None), getattr(next_block, "mixer_norm", None), res, n)
        return self.feed_forward.forward(x, ctx, sink) if sink is not None else self.feed_forward.forward(x, ctx)


register_part("block", "prenorm_residual", PreNormResidual)


class Branches:
    """What a mixer may return instead of one tensor: several outputs that the block's norm adds together, each
    optionally RMS-normed over its row with ``inner_weights[k]`` first, the sum multiplied by ``coef``."""

    def __init__(self, deltas, inner_weights=(), coef: float = 1.0, scaled=None, coefs=None):
        self.deltas, self.inner_weights, self.coef = tuple(deltas), tuple(inner_weights), coef
        self.coefs = tuple(coefs) if coefs is not None else None      # a coefficient per output instead of one for the sum
        self.scaled = scaled            # (h [T, W], w float32 [T]): one more output, w[t] * h[t] (norms that add by ``add_to``)


class StreamMix(Part):
    """The stream mixed with the embedding's output e (which the embedding kept, ``ctx.extras["embedding_output"]``) and
    shifted: x <- W [x; e] + b with W = 'in' [width, 2 width] (x's columns first) and b = row ``index`` of 'step' [rows,
    width].  Models that run a stretch of layers several times put one in front of every pass, all sharing the two
    tensors.  What the block before left to be added is added first, inside the kernel that joins the two streams for
    the product; the product leaves float32 and becomes the stream."""

    def __init__(self, hidden_size: int, rows: int, index: int):
        if not 0 <= index < rows:
            raise ValueError(f"shift {index} of {rows}")
        self.hidden_size, self.rows, self.index = hidden_size, rows, index

    def tensor_specs(self):
        h = self.hidden_size
        return {"in": TensorSpec((h, 2 * h), "fan_in"), "step": TensorSpec((self.rows, h), "normal:0:0.1")}

    def bind(self, tensors, rt):
        self.rt = rt
        self.w_in = rt.place(tensors["in"])
        self.shift = tensors["step"][self.index].float().to(rt.device).contiguous()

    def kernel_sources(self):
        return {"layer_norm"} | self.rt.product_sources(self.w_in)

    def apply(self, delta, res, ctx):
        from .norm import addends_of
        e = ctx.extras.get("embedding_output")
        if e is None:
            raise ValueError("mixing the stream with the embedding's output needs an embedding that keeps it (keep_output)")
        deltas, coefs = addends_of(delta)
        joined = self.rt.empty(res.shape[0], 2 * self.hidden_size)
        ops.stream_join(res, e, joined, deltas=deltas, coefs=coefs)
        res.copy_(self.rt.linear(joined, self.w_in, self.shift, out_dtype=res.dtype))


register_part("connection", "stream_mix", StreamMix)


class StreamMixStep(Block):
    """Not a layer but a step between layers: its one part rewrites the stream (``StreamMix``); nothing is left pending."""
    roles = {"mix": "connection"}

    def forward(self, delta, res, ctx, cache):
        self.mix.apply(delta, res, ctx)
        return None


register_part("block", "stream_mix_step", StreamMixStep)


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


class LayerScale(Part):
    """One learned factor per channel on a sublayer's output; the tensor is ``name`` [size]."""

    def __init__(self, size: int, name: str = "scale"):
        self.size, self.name = size, name

    def tensor_specs(self):
        return {self.name: TensorSpec((self.size,), "normal:0.5:0.2")}

    def bind(self, tensors, rt):
        self.rt = rt
        self.vec = tensors[self.name].float().to(rt.device).contiguous()


class DepthAverage(Part):
    """What a layer hands on is a weighted average over depth: with X_0 the embedding and X_j the result of layer j - 1, the
    stream after layer ``index`` becomes sum over j <= index + 1 of w[j] X_j.  The weights are the tensor ``name`` [index + 2]."""

    def __init__(self, index: int, name: str = "weights"):
        self.index, self.name = int(index), name

    def tensor_specs(self):
        n = self.index + 2
        return {self.name: TensorSpec((n,), f"normal:{1.0 / n}:0.1")}

    def bind(self, tensors, rt):
        self.rt = rt
        self.coef = tensors[self.name].float().to(rt.device).contiguous()


register_part("connection", "layer_scale", LayerScale)
register_part("connection", "depth_average", DepthAverage)


class OutputNormResidual(Block):
    """A layer whose norms sit on the sublayers' OUTPUTS: x <- x + scale_1 * norm_1(mixer(x)), then x <- x + scale_2 *
    norm_2(ff(x)); both sublayers read the stream itself.  Optional parts: per-channel scales on the normed outputs
    (``mixer_scale``, ``feed_forward_scale``), a feed-forward, an input taken from the token (``token_input``; its result is
    RMS-normed with ``token_input_norm`` and added), and a weighted average over the results of all layers so far
    (``depth``).  The sum, the norm and the copy of the stream for the next reader are one kernel per sublayer; the last of
    them also stores the layer's result and takes the average.  Takes and returns a ``LayeredStream``."""
    roles = {"mixer": "mixer", "feed_forward": "feed_forward", "mixer_norm": "norm", "feed_forward_norm": "norm",
             "mixer_scale": "connection", "feed_forward_scale": "connection", "token_input": "token_input",
             "token_input_norm": "norm", "depth": "connection"}
    optional_roles = ("feed_forward", "feed_forward_norm", "mixer_scale", "feed_forward_scale", "token_input", "token_input_norm", "depth")

    def __init__(self, **parts):
        super().__init__(**parts)
        for a, b in (("feed_forward", "feed_forward_norm"), ("token_input", "token_input_norm")):
            if (a in parts) != (b in parts):
                raise ValueError(f"a layer with a {a} needs a {b}, and the other way round")

    def kernel_sources(self):
        return {"stream_update"}

    def forward(self, delta, res, ctx, cache):
        from .embedding import LayeredStream
        if not isinstance(delta, LayeredStream):
            raise ValueError("a layer that norms its sublayers' outputs takes the stream from an embedding that hands on a LayeredStream")
        s = delta
        rt = self.mixer.rt
        vec = lambda role: getattr(self, role).vec if hasattr(self, role) else None
        fresh = (lambda: rt.empty(*res.shape)) if rt.dtype != res.dtype else (lambda: None)
        x = fresh()
        self.mixer_norm.add_to(res, self.mixer.forward(s.x, ctx, cache), vec=vec("mixer_scale"), act=x)
        x = res if x is None else x
        if hasattr(self, "feed_forward"):
            nxt = fresh()
            self.feed_forward_norm.add_to(res, self.feed_forward.forward(x, ctx), vec=vec("feed_forward_scale"), act=nxt)
            x = res if nxt is None else nxt
        y = norm = None
        if hasattr(self, "token_input"):
            y, norm = self.token_input.forward(x, s), self.token_input_norm
        depth = getattr(self, "depth", None)
        if y is not None or depth is not None:
            if depth is not None and (s.history is None or depth.index + 1 >= s.history.shape[0]):
                raise ValueError(f"the average over depth after layer {depth.index} needs a history of {depth.index + 2} entries")
            nxt = fresh()
            if norm is not None and getattr(self, "_input_vec", None) is None:
                self._input_vec = norm.weight.float().contiguous()        # the kernel reads float32
            ops.normed_add(res, (y,), vec=self._input_vec if norm is not None else None, eps=norm.eps if norm is not None else 0.0, act=nxt,
                           history=s.history if depth is not None else None, slot=depth.index + 1 if depth is not None else 0,
                           coef=depth.coef if depth is not None else None)
            x = res if nxt is None else nxt
        return LayeredStream(x, s.tokens, s.token_table, s.history)


register_part("block", "output_norm_residual", OutputNormResidual)
