"""SwiGLU feed-forward: down(silu(gate(x)) * up(x)).  gate and up are fused into one matrix
(inference_engine/model.py:109,180-181 concatenates them on the output dimension).  In bfloat16 the
fused matrix interleaves them instead -- row 2i = gate_i, row 2i+1 = up_i -- so that the tensor-core
product can apply SwiGLU in its epilogue while both values of a pair sit side by side."""
from __future__ import annotations

import math

import torch

from ..kernels import linear as linear_kernels
from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import FeedForward, register_part


class SwiGLU(FeedForward):
    def __init__(self, hidden_size: int, intermediate_size: int):
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size

    def tensor_specs(self):
        h, i = self.hidden_size, self.intermediate_size
        return {"gate_proj.weight": TensorSpec((i, h)), "up_proj.weight": TensorSpec((i, h)),
                "down_proj.weight": TensorSpec((h, i))}

    def bind(self, tensors, rt):
        self.rt = rt
        g, u = tensors["gate_proj.weight"], tensors["up_proj.weight"]
        if g.dtype != u.dtype:
            g, u = g.float(), u.float()
        self.interleaved = rt.dtype == torch.bfloat16 and g.dtype != torch.float32
        if self.interleaved:
            self.w_gate_up = rt.place(torch.stack((g, u), 1).reshape(2 * self.intermediate_size, self.hidden_size))
        else:
            self.w_gate_up = rt.place(torch.cat([g, u], 0))
        self.w_down = rt.place(tensors["down_proj.weight"])

    takes_sink = True

    def kernel_sources(self):
        return {"activation"} | self.rt.product_sources(self.w_gate_up, self.w_down)

    def defers_norm(self, num_tokens: int) -> bool:
        return self.rt.defers_norm(num_tokens, self.w_gate_up)

    def forward(self, x, ctx, sink=None):
        if self.interleaved:
            act = linear_kernels.linear_swiglu(x, self.w_gate_up, self.rt.dtype)
        else:
            gu = self.rt.linear(x, self.w_gate_up)
            act = self.rt.empty(x.shape[0], self.intermediate_size)
            ops.swiglu(gu, act)
        if sink is not None:
            done = self.rt.linear_into_stream(act, self.w_down, None, sink)
            if done is not None:
                return done
        return self.rt.linear(act, self.w_down)


register_part("feed_forward", "swiglu", SwiGLU)


class ClampedGLU(FeedForward):
    """A gated feed-forward with clamps: g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit),
    output W_down (g sigmoid(slope g) (u + shift)).  gate and up are one product; in bfloat16 the tensor-core
    products apply the gate to their float32 sums in the epilogue (rows interleaved, as for SwiGLU), elsewhere one
    kernel does in float32; the last product leaves float32 for the stream's sum."""

    def __init__(self, hidden_size: int, intermediate_size: int, limit: float, slope: float = 1.702, shift: float = 1.0):
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.limit, self.slope, self.shift = float(limit), float(slope), float(shift)

    def tensor_specs(self):
        h, i = self.hidden_size, self.intermediate_size
        return {"gate": TensorSpec((i, h), "fan_in"), "up": TensorSpec((i, h), "fan_in"), "down": TensorSpec((h, i), "fan_in")}

    def bind(self, tensors, rt):
        self.rt = rt
        g, u = tensors["gate"], tensors["up"]
        if g.dtype != u.dtype:
            g, u = g.float(), u.float()
        # in bfloat16 the rows alternate gate_i, up_i, as for SwiGLU: the tensor-core products then apply the gate in
        # their epilogue (the same epilogue with this part's constants)
        self.interleaved = rt.dtype == torch.bfloat16 and g.dtype != torch.float32
        if self.interleaved:
            self.w_gate_up = rt.place(torch.stack((g, u), 1).reshape(2 * self.intermediate_size, self.hidden_size))
        else:
            self.w_gate_up = rt.place(torch.cat([g, u], 0))
        self.w_down = rt.place(tensors["down"])

    def kernel_sources(self):
        return {"activation"} | self.rt.product_sources(self.w_gate_up, self.w_down)

    def forward(self, x, ctx):
        if self.interleaved:
            act = linear_kernels.linear_swiglu(x, self.w_gate_up, self.rt.dtype, glu=(self.limit, self.slope, self.shift))
        else:
            gu = self.rt.linear(x, self.w_gate_up)
            act = self.rt.empty(x.shape[0], self.intermediate_size)
            ops.glu_clamped(gu, act, self.limit, self.slope, self.shift)
        return self.rt.linear(act, self.w_down, None, out_dtype=torch.float32)


register_part("feed_forward", "clamped_glu", ClampedGLU)


class ActivatedMLP(FeedForward):
    """A feed-forward without a gate: W_down act(W_up h).  ``activation`` "xielu": two learned numbers p, q in the tensor
    'act' [2]; for z > 0, softplus(p) z^2 + z / 2; for z <= 0, (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2.  The last
    product leaves float32 for the stream's sum."""

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "xielu"):
        if activation != "xielu":
            raise ValueError(f"activation {activation!r}; this feed-forward has xielu")
        self.hidden_size, self.intermediate_size, self.activation = hidden_size, intermediate_size, activation

    def tensor_specs(self):
        h, i = self.hidden_size, self.intermediate_size
        return {"up": TensorSpec((i, h), "fan_in"), "down": TensorSpec((h, i), "fan_in"), "act": TensorSpec((2,), "normal:0:0.5")}

    def bind(self, tensors, rt):
        self.rt = rt
        self.w_up, self.w_down = rt.place(tensors["up"]), rt.place(tensors["down"])
        p, q = tensors["act"].double().tolist()              # constants of the model: their softplus once, in 64-bit
        softplus = lambda z: max(z, 0.0) + math.log1p(math.exp(-abs(z)))
        self.ap, self.an = softplus(p), 0.5 + softplus(q)

    def kernel_sources(self):
        return {"activation"} | self.rt.product_sources(self.w_up, self.w_down)

    def forward(self, x, ctx):
        act = linear_kernels.linear_xielu(x, self.w_up, self.ap, self.an, self.rt.dtype)      # the activation in the product's epilogue
        return self.rt.linear(act, self.w_down, None, out_dtype=torch.float32)


register_part("feed_forward", "activated_mlp", ActivatedMLP)


GROUPED_MIN_TOKENS = 32      # = kernels.linear.AUTO_MAX_TOKENS: above it the plain products are the library's too


class RoutedExperts(FeedForward):
    """A mixture of ``num_experts`` small feed-forward layers 'e<i>.up' [ff, hidden], 'e<i>.down' [hidden, ff] without
    biases, expert(h) = down act(up h).  Router logits 'router' [experts, hidden] are computed in float32; each token
    uses the ``top`` experts with the largest logits, weighted by the softmax over those logits only.

    All experts' up matrices are stacked into one and their down matrices laid side by side.  Many tokens (prompt
    portions, large batches): with the activations of the experts a token did not choose set to zero and those it chose
    multiplied by their weight, the layer is ONE wide feed-forward -- two products of the framework on the tensor cores
    and one kernel between them.  A handful of tokens (no more (token, expert) pairs than experts): every pair streams
    its own expert's rows and no others, so a decoding step reads only the experts that were chosen.  Many tokens in
    bfloat16 where a token uses at most half of the experts: the pairs are sorted by expert and both products run expert
    by expert over those rows (the library's grouped product), so no expert computes for a token that did not choose it."""

    def __init__(self, hidden_size: int, num_experts: int, top: int, expert_size: int, activation: str = "relu2", gated: bool = False,
                 score: str = "top_softmax", correction: bool = False, groups: int = 1, keep: int = 1, identity: int = 0, shared=None,
                 limit: float = 0.0):
        """``gated``: an expert is down(act(gate h) * (up h)) with a third matrix 'e<i>.gate'.  ``score`` "softmax": scores are
        the softmax over all router outputs, weights the chosen scores as they are; ``correction``: a tensor 'correction'
        [outputs] added to the scores for the choice only; ``groups`` / ``keep``: the outputs form that many equal groups of
        neighbours and only those of the ``keep`` groups with the largest choice score can be chosen.  ``identity``: that many
        router outputs behind the experts' stand for "the input itself" (no matrices).  ``shared``: the PartSpec of a
        feed-forward that every token goes through ('shared.*'), added to the sum.  With identity experts or a shared one
        ``forward`` returns the outputs as ``Branches`` for the block's norm to sum."""
        # ``score`` "sigmoid": the ``top`` largest logits are chosen and each weight is the sigmoid of its own logit, not
        # renormalized.  ``activation`` "clamped_in" (gated experts): the expert runs on the token scaled by its weight, which then does not touch its
        # output, and the hidden value is g sigmoid(1.702 g) (u + 1) with g = min(gate, limit), u = clamp(up, -limit, limit).
        outputs = num_experts + identity
        self.limit = float(limit or 0.0)
        if activation == "clamped_in" and not gated:
            raise ValueError("the clamped activation belongs to gated experts")
        if not 1 <= top <= outputs or num_experts < 1 or identity < 0:
            raise ValueError(f"top {top} of {num_experts} experts and {identity} identity experts")
        if activation not in ops.EXPERT_ACTIVATIONS:
            raise ValueError(f"activation {activation!r}; one of {', '.join(ops.EXPERT_ACTIVATIONS)}")
        if groups > 1 and (score != "softmax" or outputs % groups or not 1 <= keep <= groups or groups > 64 or top > keep * (outputs // groups)):
            raise ValueError(f"{groups} groups (keep {keep}) over {outputs} router outputs with top {top}: groups must divide the outputs, "
                             "hold at least top outputs between the kept ones, and belong to the softmax score")
        if score not in ("top_softmax", "softmax", "sigmoid"):
            raise ValueError(f"router score {score!r}; one of top_softmax, softmax, sigmoid")
        if (correction or identity) and score != "softmax":
            raise ValueError("a correction and identity experts belong to the softmax score")
        self.hidden_size, self.num_experts, self.top, self.expert_size, self.activation = hidden_size, num_experts, top, expert_size, activation
        self.gated, self.score, self.correction, self.groups, self.keep, self.identity = bool(gated), score, bool(correction), int(groups), int(keep), int(identity)
        self.outputs = outputs
        from .base import build_part
        self.shared = build_part("feed_forward", shared) if shared is not None else None

    def tensor_specs(self):
        h, F = self.hidden_size, self.expert_size
        specs = {"router": TensorSpec((self.outputs, h), "fan_in")}
        if self.correction:
            specs["correction"] = TensorSpec((self.outputs,), "normal:0:0.05")
        for e in range(self.num_experts):
            if self.gated:
                specs[f"e{e}.gate"] = TensorSpec((F, h), "fan_in")
            specs[f"e{e}.up"] = TensorSpec((F, h), "fan_in")
            specs[f"e{e}.down"] = TensorSpec((h, F), "fan_in")
        if self.shared is not None:
            specs.update({"shared." + k: v for k, v in self.shared.tensor_specs().items()})
        return specs

    def bind(self, tensors, rt):
        self.rt = rt
        ups = [tensors[f"e{e}.up"] for e in range(self.num_experts)]
        if self.gated:                                               # per expert its gate rows, then its up rows
            gates = [tensors[f"e{e}.gate"] for e in range(self.num_experts)]
            if len({t.dtype for t in ups + gates}) > 1:
                ups, gates = [t.float() for t in ups], [t.float() for t in gates]
            ups = [torch.cat([g, u], 0) for g, u in zip(gates, ups)]
        downs = [tensors[f"e{e}.down"] for e in range(self.num_experts)]
        if len({t.dtype for t in ups + downs}) > 1:
            ups, downs = [t.float() for t in ups], [t.float() for t in downs]
        self.w_up = rt.place(torch.cat(ups, 0))                      # [E * F, hidden] ([E * 2F, hidden] gated)
        self.w_down = rt.place(torch.cat(downs, 1))                  # [hidden, E * F]
        self.w_router = tensors["router"].float().to(rt.device).contiguous()      # float32: the router's product runs on CUDA cores in 32-bit
        self.rule = None
        if self.score != "top_softmax" or self.identity:
            self.rule = ops.RouteRule(self.score, tensors["correction"].float().to(rt.device).contiguous() if self.correction else None,
                                      self.groups, self.keep, self.num_experts if self.identity else None)
        if self.shared is not None:
            self.shared.bind({k: tensors["shared." + k] for k in self.shared.tensor_specs()}, rt)
        E, F, h = self.num_experts, self.expert_size, self.hidden_size
        self.grouped = (rt.dtype == torch.bfloat16 and self.w_up.dtype == torch.bfloat16 and 2 * self.top <= E and h % 8 == 0 and F % 8 == 0
                        and 2 * self.top <= self.outputs and hasattr(torch, "_grouped_mm") and rt.device.type == "cuda")
        if self.grouped:       # views of the stacked matrices, one [K, N] operand per expert; nothing is copied
            self.b_up = self.w_up.view(E, (2 if self.gated else 1) * F, h).transpose(1, 2)
            self.b_down = torch.as_strided(self.w_down, (E, F, h), (F, 1, E * F))

    def kernel_sources(self):
        shared = self.shared.kernel_sources() if self.shared is not None else set()
        return {"moe", "gemm_simt"} | self.rt.product_sources(self.w_up, self.w_down) | shared      # (gemm_simt: the router of a very wide model)

    def forward(self, x, ctx):
        """The chosen experts and the shared expert depend on nothing of one another.  For a handful of tokens both are short
        chains of kernels at a launch's latency each (router and the two pair kernels here, two or three launches there), so
        the shared expert runs on a stream of its own between a fork and a join (events; two arms of the graph inside a
        captured step) and the two chains take the time of one.  Only beside the pair kernels, which use no products of the
        runtime: the shared expert's products then have the runtime's kernels to themselves.  Every tensor either arm makes
        is used by the main stream only after the join, and the side stream starts only after the fork, so the allocator's
        per-stream reuse stays ordered."""
        from . import parallel
        shared = join = None
        one_kernel_router = x.is_contiguous() and (self.hidden_size + self.outputs) * 4 <= 200 * 1024
        if self.shared is not None and parallel.SIDE_BY_SIDE_STREAMS and x.is_cuda and one_kernel_router and self._pairs_serve(x):
            main, side = torch.cuda.current_stream(), parallel._side_stream(x.device)
            fork, join = torch.cuda.Event(), torch.cuda.Event()
            fork.record(main)
            side.wait_event(fork)
            with torch.cuda.stream(side):
                shared = self.shared.forward(x, ctx)
                join.record(side)
        if one_kernel_router:
            routed = ops.moe_router(x, self.w_router, self.top, rule=self.rule)          # logits, choice and weights in one kernel
        else:
            routed = ops.moe_route(self.rt.linear(x, self.w_router, None, out_dtype=torch.float32), self.top, self.rule)
        out = self._experts(x, routed[0], routed[1])
        if self.shared is None and len(routed) == 2:
            return out
        if join is not None:
            torch.cuda.current_stream().wait_event(join)
        elif self.shared is not None:
            shared = self.shared.forward(x, ctx)
        from .block import Branches
        return Branches([out] + ([shared] if shared is not None else []), scaled=(x, routed[2]) if len(routed) == 3 else None)

    def _pairs_serve(self, x) -> bool:
        return (x.shape[0] * self.top <= self.num_experts and x.is_contiguous()
                and (x.dtype == self.w_up.dtype or self.w_up.dtype == torch.float32)
                and ops.moe_pairs_fit(self.hidden_size, self.expert_size, self.top))

    def _experts(self, x, ids, wts):
        T = x.shape[0]
        if self._pairs_serve(x):
            out = torch.empty(T, self.hidden_size, dtype=torch.float32, device=x.device)
            return ops.moe_pairs(x, self.w_up, self.w_down, ids, wts, out, self.num_experts, self.activation, self.gated, self.limit)
        # up to the token count that the framework's own streaming product serves, the wide form reads every expert once at
        # that kernel's rate, which the grouped product does not reach on so few rows
        if self.grouped and x.dtype == torch.bfloat16 and x.is_contiguous() and T > GROUPED_MIN_TOKENS:
            ends, place, row_weight = ops.moe_sort(ids, wts, self.outputs)      # identity experts sort behind the last expert's rows
            ends = ends[:self.num_experts]
            rows = ops.moe_gather(x, place, self.top)
            up = ops.grouped_linear(rows, self.b_up, ends)
            hid = (ops.moe_glu(up, 1, self.activation, row_weight=row_weight, limit=self.limit) if self.gated
                   else ops.moe_act_rows(up, row_weight, self.activation))
            down = ops.grouped_linear(hid, self.b_down, ends)
            return ops.moe_combine(down, place, self.top, torch.empty(T, self.hidden_size, dtype=torch.float32, device=x.device),
                                   ids if self.identity else None, self.num_experts)
        up = self.rt.linear(x, self.w_up)
        if self.gated:
            act = ops.moe_glu(up, self.num_experts, self.activation, ids=ids, wts=wts, limit=self.limit)
        else:
            act = ops.moe_dense_act(up, ids, wts, torch.empty_like(up), self.num_experts, self.activation)
        return self.rt.linear(act, self.w_down, None, out_dtype=torch.float32)


register_part("feed_forward", "routed_experts", RoutedExperts)
