"""Grouped-query attention over the paged cache (the mixer of Llama).

Projections q, k, v are fused into one matrix by concatenation on the output dimension, as the
reference does (inference_engine/model.py:103-107); q and k are rotated by the position part, k and
v are written to the layer's pages, and every new token attends causally to its request's
positions through the block table -- prompt portions and single decoded tokens in one kernel
(the reference has three paths: inference_engine/model.py:128-159).  ``window`` (None for Llama)
limits a query at position p to keys in (p - window, p].
"""
from __future__ import annotations

import math

import torch

from ..kernels import attention as attn_kernels
from ..weights.loader import TensorSpec
from .base import KVNeed, Mixer, build_part, register_part


class Attention(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, position,
                 bias: bool = False, window: int | None = None, scale: float | None = None):
        if num_heads % num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if head_dim % 16 or not 16 <= head_dim <= 256:
            raise ValueError(f"head_dim {head_dim}: the attention kernels take multiples of 16 from 16 to 256")
        self.hidden_size = hidden_size
        self.num_heads = num_heads
        self.num_kv_heads = num_kv_heads
        self.head_dim = head_dim
        self.bias = bias
        self.window = window
        self.scale = scale if scale is not None else 1.0 / math.sqrt(head_dim)   # inference_engine/model.py:91
        self.position = build_part("position", position)

    def tensor_specs(self):
        H, Hkv, D, h = self.num_heads, self.num_kv_heads, self.head_dim, self.hidden_size
        specs = {"q_proj.weight": TensorSpec((H * D, h)), "k_proj.weight": TensorSpec((Hkv * D, h)),
                 "v_proj.weight": TensorSpec((Hkv * D, h)), "o_proj.weight": TensorSpec((h, H * D))}
        if self.bias:
            specs.update({"q_proj.bias": TensorSpec((H * D,), "zeros"), "k_proj.bias": TensorSpec((Hkv * D,), "zeros"),
                          "v_proj.bias": TensorSpec((Hkv * D,), "zeros")})
        specs.update(self.position.tensor_specs())       # a position encoding with tensors of its own
        return specs

    def bind(self, tensors, rt):
        self.rt = rt
        parts = [tensors[n + "_proj.weight"] for n in "qkv"]
        if len({p.dtype for p in parts}) > 1:          # mixed storage: widen to the widest
            parts = [p.float() for p in parts]
        self.w_qkv = rt.place(torch.cat(parts, 0))
        self.b_qkv = None
        if self.bias:
            self.b_qkv = rt.place(torch.cat([tensors[n + "_proj.bias"].float() for n in "qkv"], 0).to(
                torch.float32 if rt.dtype == torch.float32 else torch.bfloat16))
        self.w_o = rt.place(tensors["o_proj.weight"])
        self.position.bind({n: tensors[n] for n in self.position.tensor_specs()}, rt)

    def cache_need(self):
        return KVNeed(self.num_kv_heads, self.head_dim, self.window)

    takes_sink = True

    def kernel_sources(self):
        import torch as _torch
        names = self.rt.product_sources(self.w_qkv, self.w_o) | self.position.kernel_sources()
        if self.rt.dtype == _torch.float32 or self.head_dim > 128:
            names.add("attention_simt")
        if self.rt.dtype != _torch.float32 and self.head_dim <= 128:
            names |= {"attention_decode", "attention_prefill_tc" if self.head_dim in (64, 128) else "attention_prefill"}
        return names

    def defers_norm(self, num_tokens: int) -> bool:
        return self.rt.defers_norm(num_tokens, self.w_qkv)

    def forward(self, x, ctx, cache, sink=None):
        H, Hkv, D = self.num_heads, self.num_kv_heads, self.head_dim
        out = self.rt.empty(ctx.num_tokens, H * D)
        if getattr(self.position, "rotates_in_attention", None) and self.position.rotates_in_attention(x, self.w_qkv, ctx, cache):
            qkv = self.rt.linear(x, self.w_qkv, self.b_qkv)
            attn_kernels.attention(qkv, ctx, cache, out, H, Hkv, D, self.scale, self.window, rope=self.position.tables())
        else:
            qkv = self.position.project_rotate_and_store(x, self.w_qkv, self.b_qkv, ctx, cache, H, Hkv)
            attn_kernels.attention(qkv, ctx, cache, out, H, Hkv, D, self.scale, self.window)
        if sink is not None:
            done = self.rt.linear_into_stream(out, self.w_o, None, sink)
            if done is not None:
                return done
        return self.rt.linear(out, self.w_o)


class GatedAttention(Mixer):
    """Grouped-query softmax attention with the extras of some newer designs, each a parameter:

    * key/query size ``dim`` and value size ``vdim`` may differ (pages are as wide as the wider, tails zero);
    * ``qk_norm``: q and k are RMS-normed over their whole projection (all heads at once) with weights 'q.norm', 'k.norm';
    * rotation over the first ``rot_dims`` dims with frequencies that may be rescaled by wavelength (``rot_scaling``);
    * ``head_temp``: the score of head h is multiplied by 'temp'[h] (folded into the query);
    * ``chunk``: a query sees keys of its own block of that many positions only; ``window``: a sliding window;
    * ``gate``: the concatenated heads are multiplied by sigmoid(W_g h) before the output projection;
    * ``bias``: q, k and v have biases 'q.b', 'k.b', 'v.b', added in the projection;
    * ``qk_norm`` "head": the RMS norm is per head, with ``dim`` weights ('q.norm', 'k.norm') shared by all heads;
    * ``rot_pairing`` "interleaved": the rotation pairs entry 2i with 2i + 1 (default: i with i + rot_dims / 2);
    * ``q_temp`` (coef, every): the query at position p is multiplied by 1 + coef ln(floor((p + 1) / every) + 1);
    * ``softcap`` c: score <- c tanh(score / c) after the scale;
    * ``rel_bias`` (rows, far): a learned bias 'rel' [rows, heads] by distance n = p - j is added to the (scaled, capped) score:
      row n for n < rows / 2, else min(rows - 1, rows/2 + floor(ln(n / (rows/2)) / ln(far / (rows/2)) (rows - rows/2)));
      ``rows`` None: the table's rows come from the checkpoint's tensor (a random model gets 32);
    * ``sink``: a learned number per head ('sink') whose exponential is one more term of the softmax's denominator (nothing is scored for it, nothing read).

    q, k, v and the gate are one product; norm, rotation, temperature and the cache write one kernel; attention
    itself is the framework's paged kernels (decode and portions); the gate one more."""

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, dim: int, vdim: int, scale: float,
                 rot_dims: int, rot_base: float, eps: float, rot_scaling: dict | None = None, qk_norm: bool = True,
                 head_temp: bool = True, gate: bool = True, chunk: int | None = None, window: int | None = None,
                 bias: bool = False, rot_pairing: str = "half", q_temp=None, softcap: float = 0.0, rel_bias=None,
                 sink: bool = False):
        if rot_pairing not in ("half", "interleaved"):
            raise ValueError(f"rot_pairing {rot_pairing!r}; half or interleaved")
        if qk_norm not in (True, False, "head", "projection"):
            raise ValueError(f"qk_norm {qk_norm!r}; False, True / 'projection' or 'head'")
        if rel_bias is not None and rel_bias[0] is not None and (int(rel_bias[0]) < 2 or float(rel_bias[1]) <= int(rel_bias[0]) // 2):
            raise ValueError(f"rel_bias {rel_bias!r}: two rows or more, and a far distance beyond half of them")
        self.bias, self.rot_pairing, self.softcap, self.sink = bool(bias), rot_pairing, float(softcap or 0.0), bool(sink)
        self.q_temp = (float(q_temp[0]), int(q_temp[1])) if q_temp else None
        self.rel_bias = (int(rel_bias[0]) if rel_bias[0] is not None else None, float(rel_bias[1])) if rel_bias else None
        if num_heads % num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if rot_dims % 2 or rot_dims > dim:
            raise ValueError(f"rot_dims {rot_dims} must be even and at most dim {dim}")
        self.hidden_size, self.num_heads, self.num_kv_heads, self.dim, self.vdim = hidden_size, num_heads, num_kv_heads, dim, vdim
        self.padded = -(-max(dim, vdim) // 16) * 16          # the attention kernels take head sizes in steps of 16
        if self.padded > 256:
            raise ValueError(f"heads of {max(dim, vdim)}: the attention kernels take up to 256")
        self.scale, self.eps = float(scale), eps
        self.rot_dims, self.rot_base, self.rot_scaling = rot_dims, rot_base, rot_scaling
        self.qk_norm, self.head_temp, self.gate, self.chunk, self.window = qk_norm, head_temp, gate, chunk, window
        self.need = KVNeed(num_kv_heads, self.padded, window, chunk)

    def tensor_specs(self):
        H, G, D, Dv, h = self.num_heads, self.num_kv_heads, self.dim, self.vdim, self.hidden_size
        specs = {"q": TensorSpec((H * D, h), "fan_in"), "k": TensorSpec((G * D, h), "fan_in"), "v": TensorSpec((G * Dv, h), "fan_in"),
                 "o": TensorSpec((h, H * Dv), "fan_in")}
        if self.gate:
            specs["g"] = TensorSpec((H * Dv, h), "fan_in")
        if self.qk_norm == "head":
            specs.update({"q.norm": TensorSpec((D,), "normal:1:0.1"), "k.norm": TensorSpec((D,), "normal:1:0.1")})
        elif self.qk_norm:
            specs.update({"q.norm": TensorSpec((H * D,), "normal:1:0.1"), "k.norm": TensorSpec((G * D,), "normal:1:0.1")})
        if self.head_temp:
            specs["temp"] = TensorSpec((H,), "uniform:0.5:2")
        if self.bias:
            specs.update({"q.b": TensorSpec((H * D,), "normal:0:0.1"), "k.b": TensorSpec((G * D,), "normal:0:0.1"),
                          "v.b": TensorSpec((G * Dv,), "normal:0:0.1")})
        if self.rel_bias:
            specs["rel"] = TensorSpec((self.rel_bias[0] or -1, H), "normal:0:1", (self.rel_bias[0] or 32, H))
        if self.sink:
            specs["sink"] = TensorSpec((H,), "normal:0:1")
        return specs

    def bind(self, tensors, rt):
        from .rope import rotary_frequencies
        self.rt = rt
        parts = [tensors[n] for n in ("q", "k", "v") + (("g",) if self.gate else ())]
        if len({p.dtype for p in parts}) > 1:
            parts = [p.float() for p in parts]
        self.w_in = rt.place(torch.cat(parts, 0))
        self.w_o = rt.place(tensors["o"])
        small = lambda n: tensors[n].float().to(rt.device).contiguous()        # read as float32 by the kernel
        self.q_norm = small("q.norm") if self.qk_norm else None
        self.k_norm = small("k.norm") if self.qk_norm else None
        self.temp = small("temp") if self.head_temp else None
        self.freq = rotary_frequencies(self.rot_dims, self.rot_base, self.rot_scaling).to(rt.device)
        self.b_in = None
        if self.bias:
            b = torch.cat([tensors[n].float() for n in ("q.b", "k.b", "v.b")])
            b = torch.cat([b, torch.zeros(self.w_in.shape[0] - b.numel())])          # the gate's rows have none
            self.b_in = rt.place(b.to(torch.float32 if rt.dtype == torch.float32 else torch.bfloat16))
        dist = None
        if self.rel_bias:
            # the bias by distance as a table over distances 0 .. far: the bucket of every distance is worked out here, once,
            # in 64-bit; from ``far`` on the bucket no longer changes (the last row)
            import math
            rows, far = tensors["rel"].shape[0], self.rel_bias[1]
            half = rows // 2
            if rows < 2 or far <= half:
                raise ValueError(f"a bias table of {rows} rows with a far distance of {far}")
            bucket = lambda n: n if n < half else min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))
            idx = torch.tensor([bucket(n) for n in range(int(math.ceil(far)) + 1)], dtype=torch.long)
            dist = tensors["rel"].float()[idx].t().to(rt.device).contiguous()         # [H, far + 1]: a head's biases side by side
        from ..kernels import ops
        self.mods = None
        if self.softcap > 0 or self.sink or dist is not None:
            self.mods = ops.ScoreMods(self.softcap, small("sink") if self.sink else None, dist)

    def cache_need(self):
        return self.need

    def kernel_sources(self):
        names = self.rt.product_sources(self.w_in, self.w_o) | {"qk_norm_rope", "activation"}
        if self.rt.dtype == torch.float32 or self.padded > 128:
            names.add("attention_simt")
        else:
            names |= {"attention_decode", "attention_prefill_tc" if self.padded in (64, 128) else "attention_prefill"}
        return names

    def forward(self, x, ctx, cache):
        from ..kernels import ops
        H, G, D, Dv, DP = self.num_heads, self.num_kv_heads, self.dim, self.vdim, self.padded
        T = ctx.num_tokens
        proj = self.rt.linear(x, self.w_in, self.b_in)
        q = self.rt.empty(T, H, DP)
        ops.qk_norm_rope(proj, ctx.positions, ctx.slots[cache.group], self.freq, q, cache.k, cache.v, num_heads=H,
                         num_kv_heads=G, dim=D, vdim=Dv, rot=self.rot_dims, page_size=cache.page_size, eps=self.eps,
                         q_weight=self.q_norm, k_weight=self.k_norm, temp=self.temp, write_cache=cache.writes,
                         head_norm=self.qk_norm == "head", interleaved=self.rot_pairing == "interleaved", pos_temp=self.q_temp)
        heads = self.rt.empty(T, H, DP)
        attn_kernels.attention(q, ctx, cache, heads, H, G, DP, self.scale, self.need.mask(), q_stride=H * DP, mods=self.mods)
        if self.gate or DP != Dv:
            gated = self.rt.empty(T, H * Dv)
            if self.gate:
                ops.sigmoid_gate(heads, proj[:, (H + G) * D + G * Dv:], gated, H, Dv)
            else:
                gated.view(T, H, Dv).copy_(heads[:, :, :Dv])
        else:
            gated = heads.view(T, H * Dv)
        return self.rt.linear(gated, self.w_o, None, out_dtype=torch.float32)


def _padded_rows(parts, multiple: int = 8):
    """The matrices of ``parts`` stacked on the output dimension, with zero rows added up to a multiple of ``multiple``
    (the tensor-core products and 16-byte row accesses want that); returns (matrix, rows before the padding)."""
    if len({p.dtype for p in parts}) > 1:
        parts = [p.float() for p in parts]
    w = torch.cat(parts, 0)
    n = w.shape[0]
    if n % multiple:
        w = torch.cat([w, torch.zeros(multiple - n % multiple, w.shape[1], dtype=w.dtype)], 0)
    return w, n


def _attention_sources(rt, padded: int) -> set:
    if rt.dtype == torch.float32 or padded > 128:
        return {"attention_simt"}
    return {"attention_decode", "attention_prefill_tc" if padded in (64, 128) else "attention_prefill"}


class DifferentialAttention(Mixer):
    """Differential attention: every head has TWO softmax maps (queries and keys twice as wide, laid out head by head
    as [map 1 | map 2]) over the same values; the head's output is a1 - lambda a2, RMS-normed over its ``vdim`` values (no
    weight) and scaled by 1 - ``diff``, with lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff one number for the layer.
    Optionally (``gate``) each head is multiplied by sigmoid of one logit per head, 'g' [H, hidden].  No rotation.

    ``shares_kv``: the layer has no key/value projections; it attends over the cache of another layer (the run order
    names it) with its own queries.

    The two maps are run as 2H query heads over 2G key/value heads by the framework's paged attention kernels: the
    rows of 'q' are reordered at load time to [group, map, head in group], so that the kernels' rule "query head / (H / G)"
    finds key head 2g + m, and the rows of 'v' are doubled (each map reads its own copy of the values).  Pages are as wide
    as the wider of ``dim`` and ``vdim`` (tails zero).  The kernels leave the maps in float32 (also in bfloat16 mode: where
    lambda is near 1 the subtraction cancels, and maps rounded to bfloat16 would show); the subtraction, the norm and the
    gate are one kernel."""

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, dim: int, vdim: int, scale: float, diff: float,
                 eps: float, gate: bool = True, shares_kv: bool = False, window: int | None = None):
        if num_heads % num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        self.hidden_size, self.num_heads, self.num_kv_heads, self.dim, self.vdim = hidden_size, num_heads, num_kv_heads, dim, vdim
        self.padded = -(-max(dim, vdim) // 16) * 16
        if self.padded > 256:
            raise ValueError(f"heads of {max(dim, vdim)}: the attention kernels take up to 256")
        self.scale, self.diff, self.eps, self.gate, self.shares_kv, self.window = float(scale), float(diff), eps, gate, shares_kv, window
        self.need = KVNeed(2 * num_kv_heads, self.padded, window)

    def tensor_specs(self):
        H, G, D, Dv, h = self.num_heads, self.num_kv_heads, self.dim, self.vdim, self.hidden_size
        specs = {"q": TensorSpec((H * 2 * D, h), "fan_in"), "o": TensorSpec((h, H * Dv), "fan_in")}
        if not self.shares_kv:
            specs.update({"k": TensorSpec((G * 2 * D, h), "fan_in"), "v": TensorSpec((G * Dv, h), "fan_in")})
        specs.update({n: TensorSpec((D,), "normal:0:0.1") for n in ("lq1", "lk1", "lq2", "lk2")})
        if self.gate:
            specs["g"] = TensorSpec((H, h), "fan_in")
        return specs

    def bind(self, tensors, rt):
        import math
        self.rt = rt
        H, G, D, Dv, h = self.num_heads, self.num_kv_heads, self.dim, self.vdim, self.hidden_size
        r = H // G
        # query rows [g, i, m, D] -> [g, m, i, D]
        q = tensors["q"].reshape(G, r, 2, D, h).permute(0, 2, 1, 3, 4).reshape(H * 2 * D, h)
        parts = [q]
        if not self.shares_kv:
            v = tensors["v"].reshape(G, 1, Dv, h).expand(G, 2, Dv, h).reshape(2 * G * Dv, h)
            parts += [tensors["k"], v]
        if self.gate:
            parts.append(tensors["g"])
        w, self.rows_used = _padded_rows(parts)
        self.w_in = rt.place(w)
        self.w_o = rt.place(tensors["o"])
        f = lambda n: tensors[n].float()
        self.lam = float(math.exp(float((f("lq1") * f("lk1")).sum())) - math.exp(float((f("lq2") * f("lk2")).sum())) + self.diff)
        self.no_freq = torch.zeros(0, dtype=torch.float32, device=rt.device)

    def cache_need(self):
        return self.need

    def kernel_sources(self):
        return self.rt.product_sources(self.w_in, self.w_o) | {"qk_norm_rope", "diff_attention"} | _attention_sources(self.rt, self.padded)

    def forward(self, x, ctx, cache):
        from ..kernels import ops
        H, G, D, Dv, DP = self.num_heads, self.num_kv_heads, self.dim, self.vdim, self.padded
        T = ctx.num_tokens
        proj = self.rt.linear(x, self.w_in)
        q = self.rt.empty(T, 2 * H, DP)
        writes = cache.writes and not self.shares_kv
        # (without keys and values of its own the kernel reads the queries only)
        ops.qk_norm_rope(proj, ctx.positions, ctx.slots[cache.group], self.no_freq, q, cache.k, cache.v, num_heads=2 * H,
                         num_kv_heads=2 * G, dim=D, vdim=Dv, rot=0, page_size=cache.page_size, write_cache=writes)
        maps = self.rt.empty(T, 2 * H, DP, dtype=torch.float32)       # float32 also in bfloat16 mode: the maps are subtracted
        attn_kernels.attention(q, ctx, cache, maps, 2 * H, 2 * G, DP, self.scale, self.need.mask(), q_stride=2 * H * DP)
        gate_at = 2 * H * D + (0 if self.shares_kv else 2 * G * (D + Dv))
        out = self.rt.empty(T, H * Dv)
        ops.diff_combine(maps, proj[:, gate_at:gate_at + H] if self.gate else None, out, num_heads=H, group=H // G, vdim=Dv,
                         lam=self.lam, eps=self.eps, out_scale=1.0 - self.diff)
        return self.rt.linear(out, self.w_o, None, out_dtype=torch.float32)


class LatentAttention(Mixer):
    """Attention whose queries and keys/values go through low-rank latents.  c_q = RMSnorm(W_dq h) and q = W_uq c_q, per
    head [``dim`` plain | ``rot_dim`` rotated]; W_dkv h gives the latent c (RMS-normed, ``kv_rank`` entries) and one rotated
    key part of ``rot_dim`` entries that all heads share; per head the plain key is W_uk c and the value W_uv c.  Rotation
    pairs entry 2i with 2i + 1 over the first ``rot_dims`` entries of the rotated part.  Causal softmax attention, an
    output gate sigmoid(W_g h) on the concatenated heads, then W_o.

    The down-projections and the gate are one product; both RMS norms and the rotation of the shared key part one
    kernel; the up-projections of keys and values one product; queries and keys are put together per head (and keys
    and values written to the pages) by one more kernel, after which the framework's paged attention kernels run with as
    many key/value heads as query heads."""

    def __init__(self, hidden_size: int, num_heads: int, dim: int, rot_dim: int, vdim: int, q_rank: int, kv_rank: int,
                 scale: float, rot_dims: int, rot_base: float, eps: float, gate: bool = True, window: int | None = None):
        if rot_dims % 2 or rot_dims > rot_dim:
            raise ValueError(f"rot_dims {rot_dims} must be even and at most rot_dim {rot_dim}")
        self.hidden_size, self.num_heads, self.dim, self.rot_dim, self.vdim = hidden_size, num_heads, dim, rot_dim, vdim
        self.q_rank, self.kv_rank, self.scale, self.eps, self.gate, self.window = q_rank, kv_rank, float(scale), eps, gate, window
        self.rot_dims, self.rot_base = rot_dims, rot_base
        self.padded = -(-max(dim + rot_dim, vdim) // 16) * 16
        if self.padded > 256:
            raise ValueError(f"heads of {max(dim + rot_dim, vdim)}: the attention kernels take up to 256")
        self.need = KVNeed(num_heads, self.padded, window)

    def tensor_specs(self):
        H, D, R, Dv, h = self.num_heads, self.dim, self.rot_dim, self.vdim, self.hidden_size
        specs = {"dq": TensorSpec((self.q_rank, h), "fan_in"), "dq.norm": TensorSpec((self.q_rank,), "normal:1:0.1"),
                 "uq": TensorSpec((H * (D + R), self.q_rank), "fan_in"), "dkv": TensorSpec((self.kv_rank + R, h), "fan_in"),
                 "dkv.norm": TensorSpec((self.kv_rank,), "normal:1:0.1"), "uk": TensorSpec((H * D, self.kv_rank), "fan_in"),
                 "uv": TensorSpec((H * Dv, self.kv_rank), "fan_in"), "o": TensorSpec((h, H * Dv), "fan_in")}
        if self.gate:
            specs["g"] = TensorSpec((H * Dv, h), "fan_in")
        return specs

    def bind(self, tensors, rt):
        from .rope import rotary_frequencies
        self.rt = rt
        w, _ = _padded_rows([tensors["dq"], tensors["dkv"]] + ([tensors["g"]] if self.gate else []))
        self.w_down = rt.place(w)
        self.w_uq = rt.place(tensors["uq"])
        uk, uv = tensors["uk"], tensors["uv"]
        if uk.dtype != uv.dtype:
            uk, uv = uk.float(), uv.float()
        self.w_ukv = rt.place(torch.cat([uk, uv], 0))
        self.w_o = rt.place(tensors["o"])
        small = lambda n: tensors[n].float().to(rt.device).contiguous()
        self.q_norm, self.c_norm = small("dq.norm"), small("dkv.norm")
        self.freq = rotary_frequencies(self.rot_dims, self.rot_base).to(rt.device)

    def cache_need(self):
        return self.need

    def kernel_sources(self):
        return (self.rt.product_sources(self.w_down, self.w_uq, self.w_ukv, self.w_o) | {"latent_kv", "activation"}
                | _attention_sources(self.rt, self.padded))

    def forward(self, x, ctx, cache):
        from ..kernels import ops
        H, D, R, Dv, DP = self.num_heads, self.dim, self.rot_dim, self.vdim, self.padded
        T = ctx.num_tokens
        down = self.rt.linear(x, self.w_down)
        cq, c = self.rt.empty(T, self.q_rank), self.rt.empty(T, self.kv_rank)
        kr = self.rt.empty(T, R, dtype=torch.float32)
        ops.latent_norm_rope(down, ctx.positions, self.freq, self.q_norm, self.c_norm, self.eps, cq, c, kr, q_rank=self.q_rank,
                             kv_rank=self.kv_rank, rot_dim=R, rot=self.rot_dims)
        qu = self.rt.linear(cq, self.w_uq)
        kvu = self.rt.linear(c, self.w_ukv)
        q = self.rt.empty(T, H, DP)
        ops.latent_assemble(qu, kvu, kr, ctx.positions, ctx.slots[cache.group], self.freq, q, cache.k, cache.v, num_heads=H, dim=D,
                            rot_dim=R, vdim=Dv, rot=self.rot_dims, page_size=cache.page_size, write_cache=cache.writes)
        heads = self.rt.empty(T, H, DP)
        attn_kernels.attention(q, ctx, cache, heads, H, H, DP, self.scale, self.need.mask(), q_stride=H * DP)
        if self.gate or DP != Dv:
            gated = self.rt.empty(T, H * Dv)
            if self.gate:
                at = self.q_rank + self.kv_rank + R
                ops.sigmoid_gate(heads, down[:, at:at + H * Dv], gated, H, Dv)
            else:
                gated.view(T, H, Dv).copy_(heads[:, :, :Dv])
        else:
            gated = heads.view(T, H * Dv)
        return self.rt.linear(gated, self.w_o, None, out_dtype=torch.float32)


register_part("mixer", "attention", Attention)
register_part("mixer", "gated_attention", GatedAttention)
register_part("mixer", "differential_attention", DifferentialAttention)
register_part("mixer", "latent_attention", LatentAttention)
