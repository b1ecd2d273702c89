"""Retention: linear attention with a fixed decay per head, no softmax and no denominator, as a recurrence over
a float32 state per request and head,

    S_t = decay_h S_{t-1} + k_t v_t^T,   o_t = S_t^T q_t,

with q and k rotated by position (k scaled by dim^-1/2 afterwards).  Each head's o is divided by its root mean
square, the heads are multiplied by silu(W_g h) and projected by W_o.  The four projections of the input are one
product; the rotation is one kernel, the recurrence with the state's update runs in chunks side by side, the
heads' norm and gate are another kernel.  The state
(``StateNeed``) lives in the cache manager's state slots, so prompt portions and decoded tokens continue it alike."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import Mixer, StateNeed, register_part
from .rope import rotary_frequencies


class Retention(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, dim: int, vdim: int, decay, rot_dims: int, rot_base: float,
                 eps: float, rot_scaling: dict | None = None):
        if len(decay) != num_heads:
            raise ValueError(f"{len(decay)} decays for {num_heads} heads")
        if rot_dims % 2 or rot_dims > dim:
            raise ValueError(f"rot_dims {rot_dims} must be even and at most dim {dim}")
        self.hidden_size, self.num_heads, self.dim, self.vdim = hidden_size, num_heads, dim, vdim
        self.decay = [float(d) for d in decay]
        self.rot_dims, self.rot_base, self.rot_scaling, self.eps = rot_dims, rot_base, rot_scaling, eps

    def tensor_specs(self):
        H, D, Dv, h = self.num_heads, self.dim, self.vdim, self.hidden_size
        return {"q": TensorSpec((H * D, h), "fan_in"), "k": TensorSpec((H * D, h), "fan_in"), "v": TensorSpec((H * Dv, h), "fan_in"),
                "g": TensorSpec((H * Dv, h), "fan_in"), "o": TensorSpec((h, H * Dv), "fan_in")}

    def bind(self, tensors, rt):
        self.rt = rt
        parts = [tensors[n] for n in "qkvg"]
        if len({p.dtype for p in parts}) > 1:
            parts = [p.float() for p in parts]
        self.w_qkvg = rt.place(torch.cat(parts, 0))
        self.w_o = rt.place(tensors["o"])
        self.decay_t = torch.tensor(self.decay, dtype=torch.float32, device=rt.device)
        self.freq = rotary_frequencies(self.rot_dims, self.rot_base, self.rot_scaling).to(rt.device)

    def cache_need(self):
        return StateNeed((self.num_heads, self.vdim, self.dim), torch.float32)

    def kernel_sources(self):
        return {"retention"} | self.rt.product_sources(self.w_qkvg, self.w_o)

    def forward(self, x, ctx, cache):
        H, D, Dv = self.num_heads, self.dim, self.vdim
        qkvg = self.rt.linear(x, self.w_qkvg)
        o = self.rt.empty(ctx.num_tokens, H * Dv, dtype=torch.float32)
        ops.retention_scan(qkvg, ctx.positions, ctx.row_q_start, ctx.row_q_len, ctx.state_slots, self.decay_t, self.freq,
                           cache.state, o, num_heads=H, dim=D, vdim=Dv, rot=self.rot_dims, k_scale=D ** -0.5,
                           max_q_len=ctx.max_q_len)
        gated = self.rt.empty(ctx.num_tokens, H * Dv)
        ops.head_rms_gate(o, qkvg[:, 2 * H * D + H * Dv:], gated, H, Dv, self.eps)
        return self.rt.linear(gated, self.w_o, None, out_dtype=torch.float32)


register_part("mixer", "retention", Retention)


class LightningAttention(Mixer):
    """Linear attention over activated projections: q = silu(W_q h), k = silu(W_k h), v = silu(W_v h), per head
    S_t = decay_h S_{t-1} + k_t v_t^T and o_t = S_t^T q_t with no rotation and no other scale.  All heads' outputs together are
    RMS-normed with the weight 'norm' [heads x vdim], multiplied by sigmoid(W_g h) and projected by W_o.  The four
    projections are one product; the activations ride in the recurrence's kernels (the same chunked scan as retention's),
    the norm and the gate are one more.  The float32 state per request and head lives in the state slots."""

    def __init__(self, hidden_size: int, num_heads: int, dim: int, vdim: int, decay, eps: float):
        if len(decay) != num_heads:
            raise ValueError(f"{len(decay)} decays for {num_heads} heads")
        self.hidden_size, self.num_heads, self.dim, self.vdim, self.eps = hidden_size, num_heads, dim, vdim, eps
        self.decay = [float(d) for d in decay]

    def tensor_specs(self):
        H, D, Dv, h = self.num_heads, self.dim, self.vdim, self.hidden_size
        return {"q": TensorSpec((H * D, h), "fan_in"), "k": TensorSpec((H * D, h), "fan_in"), "v": TensorSpec((H * Dv, h), "fan_in"),
                "g": TensorSpec((H * Dv, h), "fan_in"), "o": TensorSpec((h, H * Dv), "fan_in"), "norm": TensorSpec((H * Dv,), "normal:1:0.1")}

    def bind(self, tensors, rt):
        from .attention import _padded_rows
        self.rt = rt
        w, _ = _padded_rows([tensors[n] for n in "qkvg"])
        self.w_qkvg = rt.place(w)
        self.w_o = rt.place(tensors["o"])
        self.norm = tensors["norm"].float().to(rt.device).contiguous()
        self.decay_t = torch.tensor(self.decay, dtype=torch.float32, device=rt.device)

    def cache_need(self):
        return StateNeed((self.num_heads, self.vdim, self.dim), torch.float32)

    def kernel_sources(self):
        return {"retention"} | self.rt.product_sources(self.w_qkvg, self.w_o)

    def forward(self, x, ctx, cache):
        H, D, Dv = self.num_heads, self.dim, self.vdim
        qkvg = self.rt.linear(x, self.w_qkvg)
        o = self.rt.empty(ctx.num_tokens, H * Dv, dtype=torch.float32)
        ops.decay_scan(qkvg, ctx.positions, ctx.row_q_start, ctx.row_q_len, ctx.state_slots, cache.state, o, num_heads=H, dim=D,
                       vdim=Dv, max_q_len=ctx.max_q_len, decay=self.decay_t, act=True)
        gated = self.rt.empty(ctx.num_tokens, H * Dv)
        at = 2 * H * D + H * Dv
        ops.group_norm_gate(o, qkvg[:, at:at + H * Dv], gated, groups=1, size=H * Dv, eps=self.eps, weight=self.norm)
        return self.rt.linear(gated, self.w_o, None, out_dtype=torch.float32)


register_part("mixer", "lightning_attention", LightningAttention)
