"""A matrix memory with exponential gates (the mLSTM cell of xLSTM): linear attention whose decay and write strength are
computed per token and head, kept finite by a running maximum m of the log gates,

    i_t = cap tanh((W_i h + b_i) / cap)         f_t = logsigmoid(cap tanh((W_f h + b_f) / cap))         m_t = max(f_t + m_{t-1}, i_t)
    S_t = exp(f_t + m_{t-1} - m_t) S_{t-1} + exp(i_t - m_t) k_t v_t^T        n_t likewise with k_t alone
    o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)                    q = W_q h dim^-1/2, k = W_k h, v = W_v h

with S, n and m all zero for a fresh request (so the running maximum is never below the sum of the forget gates so far).  Each head's o is divided by its root mean
square; the heads together are multiplied by the weight 'norm' and by sigmoid(W_g h) and projected by W_o.

q|k|v|g are one product; the two gate rows per head are a second one that leaves float32.  The gates' chain runs token by
token per (request, head) in a scalar kernel; the state's recurrence is the framework's chunked scan with a decay and a key
factor per token, and n rides in it as one more value column fed with ones; the division, the head norm, the weight and the
gate are one kernel.  Two states (a tuple of needs): [heads, vdim + 1, dim] (column vdim is n) and m [heads], float32."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorSpec
from .attention import _padded_rows
from .base import Mixer, StateNeed, register_part


class MatrixMemory(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, dim: int, vdim: int, eps: float, gate_cap: float = 0.0):
        self.hidden_size, self.num_heads, self.dim, self.vdim, self.eps, self.gate_cap = hidden_size, num_heads, dim, vdim, eps, float(gate_cap or 0.0)

    def tensor_specs(self):
        H, D, Dv, h = self.num_heads, self.dim, self.vdim, self.hidden_size
        return {"q": TensorSpec((H * D, h), "fan_in"), "k": TensorSpec((H * D, h), "fan_in"), "v": TensorSpec((H * Dv, h), "fan_in"),
                "g": TensorSpec((H * Dv, h), "fan_in"), "o": TensorSpec((h, H * Dv), "fan_in"), "norm": TensorSpec((H * Dv,), "normal:1:0.1"),
                "i": TensorSpec((H, h), "fan_in"), "i.b": TensorSpec((H,), "normal:0:1"),
                "f": TensorSpec((H, h), "fan_in"), "f.b": TensorSpec((H,), "normal:3:1")}

    def bind(self, tensors, rt):
        self.rt = rt
        w, _ = _padded_rows([tensors[n] for n in "qkvg"])
        self.w_in = rt.place(w)
        gates, self.gate_rows = _padded_rows([tensors["i"], tensors["f"]])
        self.w_gates = rt.place(gates)
        self.w_o = rt.place(tensors["o"])
        small = lambda n: tensors[n].float().to(rt.device).contiguous()          # read as float32 by the kernels
        self.norm, self.b_i, self.b_f = small("norm"), small("i.b"), small("f.b")

    def cache_need(self):
        return (StateNeed((self.num_heads, self.vdim + 1, self.dim), torch.float32), StateNeed((self.num_heads,), torch.float32))

    def kernel_sources(self):
        return {"retention"} | self.rt.product_sources(self.w_in, self.w_gates, self.w_o)

    def forward(self, x, ctx, cache):
        H, D, Dv, T = self.num_heads, self.dim, self.vdim, ctx.num_tokens
        state, m_state = cache.parts[0].state, cache.parts[1].state
        proj = self.rt.linear(x, self.w_in)
        z = self.rt.linear(x, self.w_gates, None, out_dtype=torch.float32)
        if z.shape[1] != 2 * H:
            z = z[:, :2 * H].contiguous()
        keep, write, m = ops.gate_scan(z, self.b_i, self.b_f, self.gate_cap, ctx.row_q_start, ctx.row_q_len, ctx.state_slots, m_state, H)
        o = self.rt.empty(T, H * (Dv + 1), dtype=torch.float32)
        ops.decay_scan(proj, ctx.positions, ctx.row_q_start, ctx.row_q_len, ctx.state_slots, state, o, num_heads=H, dim=D, vdim=Dv,
                       max_q_len=ctx.max_q_len, tok_decay=keep, k_tok=write, ones=True, q_scale=D ** -0.5)
        gated = self.rt.empty(T, H * Dv)
        at = 2 * H * D + H * Dv
        ops.group_norm_gate(o, proj[:, at:at + H * Dv], gated, groups=H, size=Dv, eps=self.eps, weight=self.norm, m=m)
        return self.rt.linear(gated, self.w_o, None, out_dtype=torch.float32)


register_part("mixer", "matrix_memory", MatrixMemory)
