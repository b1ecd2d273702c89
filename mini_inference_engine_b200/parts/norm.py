"""RMSNorm fused with the residual sum: ``res += delta; x = res * rsqrt(mean(res^2) + eps) * w``
(inference_engine/kernels/rmsnorm.py:13-32,56-65, where the residual stays in the model dtype;
here the residual stream is float32 in both modes)."""
from __future__ import annotations

from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import Part, StreamUpdated, StreamValue, register_part
from .embedding import LayeredStream


class RMSNorm(Part):
    def __init__(self, size: int, eps: float):
        self.size = size
        self.eps = eps

    def tensor_specs(self):
        return {"weight": TensorSpec((self.size,), init="ones")}

    def bind(self, tensors, rt):
        self.rt = rt
        self.weight = rt.place(tensors["weight"])

    def kernel_sources(self):
        return {"norm"}

    def deferred_args(self):
        """Weight and eps, for a product that folds this norm into its neighbours' epilogues."""
        return self.weight, self.eps

    def __call__(self, delta, res, rows=None):
        if isinstance(delta, StreamValue):               # the block before left the stream complete
            delta = None
        if isinstance(delta, StreamUpdated):             # the part before added its output to the stream itself
            if delta.norm is self and delta.deferred is not None and rows is None:
                return delta.deferred                    # and left this norm's output, short of a factor, for the next product
            delta = None
        n_out = rows.numel() if rows is not None else res.shape[0]
        out = self.rt.empty(n_out, self.size)
        return ops.add_rmsnorm(delta, res, self.weight, self.eps, out, rows)


register_part("norm", "rmsnorm", RMSNorm)


def addends_of(delta):
    """(tensors, coefficients) of what a sublayer left to be added to the stream: nothing, one output, or several
    outputs with a coefficient each (``Branches`` without inner norms)."""
    from .block import Branches
    if delta is None or isinstance(delta, (StreamValue, StreamUpdated)):
        return (), ()
    if isinstance(delta, Branches):
        if delta.inner_weights or delta.scaled is not None:
            raise ValueError("this norm adds plain outputs with coefficients; the branches came with norms of their own")
        return delta.deltas, delta.coefs if delta.coefs is not None else (delta.coef,) * len(delta.deltas)
    return (delta,), (1.0,)


class LayerNorm(Part):
    """Layer norm with a weight and no bias, fused with the sum in front of it: ``res += sum_k c_k delta_k``, then
    x = (res - mean) / sqrt(var + eps) * w with the variance as the mean of the squared deviations.  The addends are the
    output of the sublayer before (float32) or the several outputs of mixers side by side with their coefficients.
    ``center`` False leaves the mean out (an RMS norm over the same sums)."""

    def __init__(self, size: int, eps: float, center: bool = True):
        self.size, self.eps, self.center = size, eps, bool(center)

    def tensor_specs(self):
        return {"weight": TensorSpec((self.size,), "normal:1:0.1")}

    def bind(self, tensors, rt):
        self.rt = rt
        self.weight = tensors["weight"].float().to(rt.device).contiguous()      # read as float32 by the kernel

    def kernel_sources(self):
        return {"layer_norm"}

    def __call__(self, delta, res, rows=None):
        deltas, coefs = addends_of(delta)
        n_out = rows.numel() if rows is not None else res.shape[0]
        out = self.rt.empty(n_out, self.size)
        return ops.add_layernorm(res, self.weight, self.eps, out, deltas=deltas, coefs=coefs, rows=rows, center=self.center)


register_part("norm", "layernorm", LayerNorm)


class GroupRMSNorm(Part):
    """RMS norm with statistics per group: a row is cut into ``groups`` equal consecutive parts, each divided by
    sqrt(mean(part^2) + eps), and the whole multiplied by the weight.  It norms the stream itself (post-norm
    models): ``apply`` replaces the stream by norm(alpha * stream + coef * sum of branches), where a branch may first
    be RMS-normed over its whole row with a weight of its own (``inner_weights``), and returns the new stream in the
    activation type.  Called like the other norms (``norm(delta, res, rows)``) it adds nothing and norms a copy: the
    norm in front of the output head."""

    def __init__(self, size: int, eps: float, groups: int = 1):
        if groups < 1 or size % groups:
            raise ValueError(f"{groups} groups do not divide a width of {size}")
        self.size, self.eps, self.groups = size, eps, groups

    def tensor_specs(self):
        return {"weight": TensorSpec((self.size,), init="ones")}

    def bind(self, tensors, rt):
        self.rt = rt
        self.weight = tensors["weight"].float().to(rt.device).contiguous()      # read as float32 by the kernel (16-byte loads)

    def kernel_sources(self):
        return {"norm_group"}

    def apply(self, res, deltas=(), inner_weights=(), alpha: float = 1.0, coef: float = 1.0):
        """res <- norm(alpha * res + coef * sum(branches)) in place; returns it in the activation type (``res`` itself
        where that is float32)."""
        import torch
        out = None if self.rt.dtype == torch.float32 else self.rt.empty(res.shape[0], self.size)
        ops.stream_norm(res, self.weight, self.groups, self.eps, out, alpha=alpha, deltas=deltas,
                        inner_weights=inner_weights, coef=coef)
        return res if out is None else out

    def __call__(self, delta, res, rows=None):
        if isinstance(delta, (StreamValue, StreamUpdated)):
            delta = None
        if delta is not None:
            raise ValueError("a group norm of the stream takes its branches through apply()")
        if rows is None:
            return self.apply(res)
        out = self.rt.empty(rows.numel(), self.size)
        return ops.stream_norm(res, self.weight, self.groups, self.eps, out, rows=rows)


register_part("norm", "group_rmsnorm", GroupRMSNorm)


class DynamicTanh(Part):
    """Dynamic Tanh in the place of a norm: tanh(alpha x) * weight + bias per entry, with a learned scalar alpha -- no
    statistics of the row.  ``streams`` > 1: the stream is kept in that many copies side by side ([tokens, streams *
    size]); a reader takes one mixture of them and a writer updates all of them (``parts.block.HyperConnection``), and
    both happen in this norm's kernel, one pass over the stream: ``read`` applies the pending update of the sublayer
    before (in place), mixes the copies for the reader and squashes.  Called like the other norms
    (``norm(delta, res, rows)``) it reads the sum of the copies -- the norm in front of the output head; with one copy
    and a plain tensor as ``delta`` that is the usual fused ``res += delta; x = norm(res)``."""

    def __init__(self, size: int, streams: int = 1):
        if streams < 1 or streams > 8:
            raise ValueError(f"{streams} copies of the stream: the kernel takes 1 to 8")
        self.size, self.streams = size, streams

    def tensor_specs(self):
        return {"weight": TensorSpec((self.size,), "normal:1:0.1"), "b": TensorSpec((self.size,), "normal:0:0.1"),
                "alpha": TensorSpec((), "uniform:0.3:1")}

    def bind(self, tensors, rt):
        self.rt = rt
        small = lambda n: tensors[n].float().reshape(-1).to(rt.device).contiguous()      # read as float32 by the kernel
        self.weight, self.bias, self.alpha = small("weight"), small("b"), small("alpha")

    def kernel_sources(self):
        return {"hyper_norm"}

    def read(self, res, pending=None, reader=None, rows=None):
        """``pending``: a ``PendingUpdate`` (the output of the sublayer before and its connection) or None; ``reader``:
        the connection of the sublayer that reads (None: the plain sum of the copies)."""
        n_out = rows.numel() if rows is not None else res.shape[0]
        out = self.rt.empty(n_out, self.size)
        y = conn = None
        if pending is not None:
            y, conn = pending.y, pending.connection
        return ops.hyper_norm(res, self.streams, out, weight=self.weight, bias=self.bias, alpha=self.alpha, y=y,
                              mix=conn.mix if conn is not None else None, out_coef=conn.out_coef if conn is not None else None,
                              in_coef=reader.in_coef if reader is not None else None, rows=rows)

    def __call__(self, delta, res, rows=None):
        from .block import PendingUpdate
        if isinstance(delta, (StreamValue, StreamUpdated)):
            delta = None
        if delta is not None and not isinstance(delta, PendingUpdate):
            if self.streams != 1:
                raise ValueError("a stream kept in several copies takes its updates through a connection")
            delta = PendingUpdate(delta, None)
        return self.read(res, delta, None, rows)


register_part("norm", "dynamic_tanh", DynamicTanh)


class ScalarRMSNorm(Part):
    """RMS norm whose weight is ONE number for all channels: x / sqrt(mean(x^2) + eps) * g.  Called like the other norms
    (``norm(delta, res, rows)``) it norms the stream; ``add_to`` norms a sublayer's output and adds it to the stream (layers
    whose norm sits on the output only)."""

    def __init__(self, size: int, eps: float):
        self.size, self.eps = size, eps

    def tensor_specs(self):
        return {"weight": TensorSpec((), "normal:1:0.1")}

    def bind(self, tensors, rt):
        self.rt = rt
        self.gain = tensors["weight"].float().reshape(1).to(rt.device).contiguous()
        self.weight = self.gain.expand(self.size).contiguous()         # as a vector, for the kernel that norms the stream

    def kernel_sources(self):
        return {"norm", "stream_update"}

    def add_to(self, res, y, *, vec=None, act=None):
        """res += norm(y) * vec; ``y`` a tensor or ``Branches`` (its tensors, and one scaled by a number per row, are summed)."""
        from .block import Branches
        if isinstance(y, Branches):
            return ops.normed_add(res, y.deltas, scaled=y.scaled, gain=self.gain, vec=vec, eps=self.eps, act=act)
        return ops.normed_add(res, (y,), gain=self.gain, vec=vec, eps=self.eps, act=act)

    def __call__(self, delta, res, rows=None):
        if isinstance(delta, (StreamValue, StreamUpdated, LayeredStream)):
            delta = None
        n_out = rows.numel() if rows is not None else res.shape[0]
        out = self.rt.empty(n_out, self.size)
        return ops.add_rmsnorm(delta, res, self.weight, self.eps, out, rows)


register_part("norm", "scalar_rmsnorm", ScalarRMSNorm)
