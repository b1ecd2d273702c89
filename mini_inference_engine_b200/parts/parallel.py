"""Several mixers side by side on the same input: the result is the mean of their outputs, each first RMS-normed
over the model width with a weight of its own.  The norms and the mean are not computed here: the mixer returns
its branches (``Branches``) and the block's norm kernel takes them in, so the branch norms, the mean, the residual
sum and the block's own norm are one launch.  What the branches need of the past is declared as a tuple; each
branch gets its own ``LayerCache``."""
from __future__ import annotations

import os

import torch

from ..weights.loader import TensorSpec
from .base import Mixer, build_part, register_part
from .block import Branches

SIDE_BY_SIDE_STREAMS = os.environ.get("MIE_B200_BRANCH_STREAMS", "1") != "0"
_side_streams: dict = {}


def _side_stream(device):
    key = str(device)
    if key not in _side_streams:
        _side_streams[key] = torch.cuda.Stream(device=device)
    return _side_streams[key]


class ParallelMixers(Mixer):
    def __init__(self, hidden_size: int, branches: dict, scales=None):
        """``branches``: {name: PartSpec of a mixer}; a branch's tensors are '<name>.<its own>', its out-norm weight
        '<name>.out'."""
        if not 1 <= len(branches) <= 2:
            raise ValueError("the norm kernel adds one or two branches")
        # ``scales`` (one number per branch): the result is the weighted sum of the branches' outputs as they are -- no
        # out-norms, no '<name>.out' tensors, no mean
        if scales is not None and len(scales) != len(branches):
            raise ValueError("one scale per branch")
        self.scales = tuple(float(s) for s in scales) if scales is not None else None
        self.hidden_size = hidden_size
        self.names = list(branches)
        self.branches = [build_part("mixer", branches[n]) for n in self.names]

    def tensor_specs(self):
        specs = {}
        for name, b in zip(self.names, self.branches):
            specs.update({f"{name}.{k}": v for k, v in b.tensor_specs().items()})
            if self.scales is None:
                specs[f"{name}.out"] = TensorSpec((self.hidden_size,), "normal:1:0.1")
        return specs

    def bind(self, tensors, rt):
        self.rt = rt
        self.out_weights = []
        for name, b in zip(self.names, self.branches):
            b.bind({k: tensors[f"{name}.{k}"] for k in b.tensor_specs()}, rt)
            if self.scales is None:
                self.out_weights.append(tensors[f"{name}.out"].float().to(rt.device).contiguous())   # float32 for the norm kernel

    def cache_need(self):
        return tuple(b.cache_need() for b in self.branches)

    def kernel_sources(self):
        names = set()
        for b in self.branches:
            names |= b.kernel_sources()
        return names

    def forward(self, x, ctx, cache):
        if (len(self.branches) == 2 and SIDE_BY_SIDE_STREAMS and x.is_cuda
                and type(self.branches[0]) is not type(self.branches[1])):      # two of a kind would share their kernels' scratch
            # The branches depend on nothing of one another: the second runs on a stream of its own between a fork and a
            # join (events; inside a captured step they become two arms of the graph).  A decode step is a chain of
            # short kernels, and two chains of five side by side take the time of one.  Every tensor either branch
            # makes is used by the main stream only after the join, and the side stream starts only after the fork,
            # so the allocator's per-stream reuse stays ordered.
            main, side = torch.cuda.current_stream(), _side_stream(x.device)
            fork, join = torch.cuda.Event(), torch.cuda.Event()
            fork.record(main)
            side.wait_event(fork)
            with torch.cuda.stream(side):
                second = self.branches[1].forward(x, ctx, cache.parts[1])
                join.record(side)
            first = self.branches[0].forward(x, ctx, cache.parts[0])
            main.wait_event(join)
            outs = [first, second]
        else:
            outs = [b.forward(x, ctx, c) for b, c in zip(self.branches, cache.parts)]
        if self.scales is not None:
            return Branches(outs, coefs=self.scales)
        return Branches(outs, self.out_weights, coef=1.0 / len(outs))


register_part("mixer", "parallel", ParallelMixers)
