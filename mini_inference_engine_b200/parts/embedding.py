"""Token embedding (opens the float32 residual stream) and the output head
(inference_engine/model.py:96,113,168,185).  A tied head multiplies by the embedding table."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import Part, register_part


class Embedding(Part):
    def __init__(self, vocab_size: int, hidden_size: int, keep_output: bool = False):
        """``keep_output``: a copy of what the embedding leaves stays in ``ctx.extras["embedding_output"]`` for parts that
        read it again later in the step (float32, as the stream)."""
        self.vocab_size = vocab_size
        self.hidden_size = hidden_size
        self.keep_output = bool(keep_output)

    def tensor_specs(self):
        return {"weight": TensorSpec((self.vocab_size, self.hidden_size))}

    def bind(self, tensors, rt):
        self.rt = rt
        self.weight = rt.place(tensors["weight"])

    def kernel_sources(self):
        return {"embedding"}

    def forward(self, ctx):
        res = self.rt.empty(ctx.num_tokens, self.hidden_size, dtype=torch.float32)
        ops.embedding(self.weight, ctx.token_ids, res, ctx.token_feedback)
        if self.keep_output:
            ctx.extras["embedding_output"] = res.clone()
        return res


class LinearHead(Part):
    """logits = x W^T in float32; ``tied`` takes W from the embedding (same tensor name).  ``softcap`` c > 0: the logits
    become c tanh(logits / c)."""

    def __init__(self, vocab_size: int, hidden_size: int, tied: bool = False, softcap: float = 0.0):
        self.vocab_size = vocab_size
        self.hidden_size = hidden_size
        self.tied = tied
        self.softcap = float(softcap or 0.0)

    def tensor_specs(self):
        return {"weight": TensorSpec((self.vocab_size, self.hidden_size))}

    def bind(self, tensors, rt, shared=None):
        self.rt = rt
        self.weight = shared if shared is not None else rt.place(tensors["weight"])

    def kernel_sources(self):
        return self.rt.product_sources(self.weight) | ({"layer_norm"} if self.softcap > 0 else set())

    def forward(self, x):
        logits = self.rt.linear(x, self.weight, None, out_dtype=torch.float32)
        return ops.tanh_cap(logits, self.softcap) if self.softcap > 0 else logits


register_part("embedding", "embedding", Embedding)
register_part("head", "linear_head", LinearHead)


class NormedEmbedding(Embedding):
    """A token embedding followed by a norm of the stream (``norm``: the PartSpec of a norm with an ``apply``; its
    tensors are 'norm.<its own>').  Hands on the stream and its value in the activation type."""

    def __init__(self, vocab_size: int, hidden_size: int, norm):
        super().__init__(vocab_size, hidden_size)
        from .base import build_part
        self.norm = build_part("norm", norm)

    def tensor_specs(self):
        specs = {"weight": TensorSpec((self.vocab_size, self.hidden_size), "normal:0:1")}
        specs.update({"norm." + k: v for k, v in self.norm.tensor_specs().items()})
        return specs

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.norm.bind({k: tensors["norm." + k] for k in self.norm.tensor_specs()}, rt)

    def kernel_sources(self):
        return {"embedding"} | self.norm.kernel_sources()

    def forward(self, ctx):
        from .base import StreamValue
        res = super().forward(ctx)
        return res, StreamValue(self.norm.apply(res))


register_part("embedding", "normed_embedding", NormedEmbedding)


class ScaledEmbedding(Embedding):
    """A token embedding times a constant (multiplied in float32), opening a stream kept in ``copies`` copies side by
    side: [tokens, copies * hidden]."""

    def __init__(self, vocab_size: int, hidden_size: int, scale: float = 1.0, copies: int = 1):
        super().__init__(vocab_size, hidden_size)
        self.scale, self.copies = float(scale), int(copies)

    def tensor_specs(self):
        return {"weight": TensorSpec((self.vocab_size, self.hidden_size), "fan_in")}

    def forward(self, ctx):
        res = self.rt.empty(ctx.num_tokens, self.copies * self.hidden_size, dtype=torch.float32)
        return ops.embedding(self.weight, ctx.token_ids, res, ctx.token_feedback, scale=self.scale, copies=self.copies)


register_part("embedding", "scaled_embedding", ScaledEmbedding)


class LayeredStream:
    """What an embedding hands on beside the stream when later parts need more than the stream itself: ``x``, the stream
    in the activation type for its next reader (the stream itself in the 32-bit mode); ``tokens``, the step's token ids
    with fed-back tokens resolved (int32 [T]); ``token_table``, a table with one row per vocabulary entry from which layers
    take per-token inputs (or None); ``history``, float32 [entries, T, W], the results of the layers so far (entry 0: the
    embedding) for layers that read a weighted average over depth (or None).  A norm given one treats it as "nothing to add"."""

    def __init__(self, x, tokens, token_table=None, history=None):
        self.x, self.tokens, self.token_table, self.history = x, tokens, token_table, history


class PairEmbedding(Embedding):
    """A token embedding times a constant plus a row of a second table chosen by a hash of the token and the token before it:
    row (previous * mul_prev + token * mul_cur) mod buckets of 'pair' [buckets + 1, hidden], and row ``buckets`` for a
    sequence's first token (``buckets`` 0: no second table).  The token before a step's first token is kept per request
    in a state slot (one int32).  Optionally owns a per-token table 'side' [vocab, side_width] for the layers, and opens a
    history of ``history`` entries of the stream; hands on a ``LayeredStream``."""

    def __init__(self, vocab_size: int, hidden_size: int, scale: float = 1.0, buckets: int = 0, mul_prev: int = 0, mul_cur: int = 0,
                 side_width: int = 0, history: int = 0):
        super().__init__(vocab_size, hidden_size)
        if buckets < 0 or mul_prev < 0 or mul_cur < 0 or side_width < 0 or history < 0:
            raise ValueError("buckets, multipliers, side width and history must not be negative")
        self.scale, self.buckets, self.mul_prev, self.mul_cur = float(scale), int(buckets), int(mul_prev), int(mul_cur)
        self.side_width, self.history = int(side_width), int(history)

    def tensor_specs(self):
        specs = {"weight": TensorSpec((self.vocab_size, self.hidden_size), "fan_in")}
        if self.buckets:
            specs["pair"] = TensorSpec((self.buckets + 1, self.hidden_size), "normal:0:0.5")
        if self.side_width:
            specs["side"] = TensorSpec((self.vocab_size, self.side_width), "normal:0:1")
        return specs

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.pair = rt.place(tensors["pair"]) if self.buckets else None
        self.side = rt.place(tensors["side"]) if self.side_width else None
        if self.pair is not None and self.pair.dtype != self.weight.dtype:
            self.pair, self.weight = self.pair.float(), self.weight.float()

    def cache_need(self):
        from .base import StateNeed
        return StateNeed((1,), torch.int32)

    def forward(self, ctx, cache):
        T, W = ctx.num_tokens, self.hidden_size
        res = self.rt.empty(T, W, dtype=torch.float32)
        history = self.rt.empty(self.history, T, W, dtype=torch.float32) if self.history else None
        act = self.rt.empty(T, W) if self.rt.dtype == torch.bfloat16 else None
        tokens = torch.empty(T, dtype=torch.int32, device=res.device)
        ops.pair_embedding(self.weight, self.pair, ctx, cache.state, res, scale=self.scale, buckets=self.buckets, mul_prev=self.mul_prev,
                           mul_cur=self.mul_cur, first=history[0] if history is not None else None, act=act, resolved=tokens)
        return res, LayeredStream(act if act is not None else res, tokens, self.side, history)


register_part("embedding", "pair_embedding", PairEmbedding)


class TokenGatedInput(Part):
    """An input a layer takes from the token itself: with e the columns [index * dim, (index + 1) * dim) of the token's row
    of the embedding's per-token table, y = W_proj (gelu_tanh(W_gate x) * e).  Tensors 'gate' [dim, hidden], 'proj' [hidden, dim].
    The block norms y and adds it to the stream."""

    def __init__(self, hidden_size: int, dim: int, index: int):
        self.hidden_size, self.dim, self.index = hidden_size, int(dim), int(index)

    def tensor_specs(self):
        return {"gate": TensorSpec((self.dim, self.hidden_size), "fan_in"), "proj": TensorSpec((self.hidden_size, self.dim), "fan_in")}

    def bind(self, tensors, rt):
        self.rt = rt
        self.w_gate, self.w_proj = rt.place(tensors["gate"]), rt.place(tensors["proj"])

    def kernel_sources(self):
        return {"activation"} | self.rt.product_sources(self.w_gate, self.w_proj)

    def forward(self, x, stream):
        table = stream.token_table
        if table is None or (self.index + 1) * self.dim > table.shape[1]:
            raise ValueError(f"layer input {self.index} needs columns up to {(self.index + 1) * self.dim} of a per-token table")
        g = self.rt.linear(x, self.w_gate)
        if table.dtype != g.dtype:
            raise ValueError("the per-token table must be stored in the activation type")
        gated = ops.gelu_gate_rows(g, table, stream.tokens, self.index * self.dim, torch.empty_like(g))
        return self.rt.linear(gated, self.w_proj, None, out_dtype=torch.float32)


register_part("token_input", "gated_table", TokenGatedInput)
