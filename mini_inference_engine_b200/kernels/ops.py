"""Python faces of the CUDA kernels: each function checks shapes and types, then calls the
``extern "C"`` launcher of its library on torch's current stream.  Tensors are passed as raw
device pointers; nothing here computes on the host or through a library kernel, and there is no
other path: a tensor that is not on a CUDA device is refused.
"""
from __future__ import annotations

import ctypes
import math

import torch

from . import build
from .device import num_sms

F32, BF16 = 0, 1
_TAGS = {torch.float32: F32, torch.bfloat16: BF16}

_CUDA_ERRORS = {-1: "a size or option the kernel does not take", -2: "beyond the kernel's stated maximum"}


class KernelError(RuntimeError):
    pass


def tag(t: torch.Tensor) -> int:
    try:
        return _TAGS[t.dtype]
    except KeyError:
        raise KernelError(f"unsupported element type {t.dtype}; kernels take float32 and bfloat16") from None


def _ptr(t):
    if t is None:
        return ctypes.c_void_p(0)
    if not t.is_cuda:
        raise KernelError("kernels of this package run on CUDA tensors only; got a tensor on " + str(t.device))
    return ctypes.c_void_p(t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


before_launch: list = []     # callables run before any launch of this package (a pending chain of products goes first)


def _stream():
    """The current CUDA stream's handle.  Asked on every launch (a graph capture switches streams)."""
    for hook in before_launch:
        hook()
    return raw_stream()


def raw_stream():
    if _raw_stream is not None:                      # the direct query; a tenth of the cost of the Stream object
        return ctypes.c_void_p(_raw_stream(torch.cuda.current_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


launches = 0        # kernels of this package launched so far (captured launches count once, at capture)


def _check(code: int, what: str) -> None:
    global launches
    if code == 0:
        launches += 1
        return
    if code < 0:
        raise KernelError(f"{what}: refused, {_CUDA_ERRORS.get(code, code)}")
    raise KernelError(f"{what}: CUDA error {code} at launch")


# --------------------------------------------------------------------------- range report
# Four int32 in pinned host memory that the kernels write directly (code, kernel, index, value): see
# csrc/range_check.cuh.  Every library that checks ranges is told the address when it is loaded.
_RANGE_CODES = {1: "token id outside the vocabulary (or the fed-back tokens)", 2: "position outside the position table "
                "(or more positions than the block table covers)", 3: "cache slot outside the cache",
                4: "block-table entry outside the page pool", 5: "row index outside the batch"}
_RANGE_KERNELS = {1: "embedding", 2: "rope_cache", 3: "norm", 4: "attention_simt", 5: "attention_decode",
                  6: "attention_prefill", 7: "attention_prefill_tc", 8: "gemm_tcgen05 (q|k|v with rotation)",
                  9: "norm_group", 10: "qk_norm_rope", 11: "hyper_norm", 12: "latent_kv"}
_range_report: torch.Tensor | None = None
_range_told: set = set()


def range_report() -> torch.Tensor:
    global _range_report
    if _range_report is None:
        with torch.inference_mode(False):        # made inside a step, it would refuse to be cleared outside one
            _range_report = torch.zeros(4, dtype=torch.int32, pin_memory=True)
    return _range_report


def load(name: str):
    """The library of ``csrc/<name>.cu``, told where the range report lives if it checks ranges."""
    lib = build.load(name)
    if name not in _range_told:
        _range_told.add(name)
        if hasattr(lib, "mie_set_range_report"):
            lib.mie_set_range_report(ctypes.c_void_p(range_report().data_ptr()))
    return lib


def check_range_errors() -> None:
    """Raises if a kernel met an integer out of range since the last call (after a synchronise): the
    kernel skipped that access, so the step's result is not valid."""
    if _range_report is None:
        return
    code, kernel, index, value = _range_report.tolist()
    if code:
        _range_report.numpy()[:] = 0
        raise KernelError(f"{_RANGE_KERNELS.get(kernel, kernel)}: {_RANGE_CODES.get(code, code)}: "
                          f"value {value} at index {index}; the access was skipped and the step's output is not valid")


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


def _i32(t, name):
    _need(t.dtype == torch.int32 and t.is_contiguous(), f"{name} must be a contiguous int32 tensor")


# --------------------------------------------------------------------------- embedding

def embedding(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, feedback: torch.Tensor | None = None,
              scale: float = 1.0, copies: int = 1) -> torch.Tensor:
    """out[t] = table[ids[t]] * scale as float32 (the residual stream), written ``copies`` times side by side.  An id
    -(k+1) is replaced on the device by ``feedback[k]`` (a token the previous step sampled and the host has not read yet)."""
    if feedback is not None:
        _i32(feedback, "feedback")
    _i32(ids, "ids")
    V, h = table.shape
    _need(out.dtype == torch.float32 and out.shape == (ids.numel(), copies * h) and out.is_contiguous(),
          "embedding output must be contiguous float32 [tokens, copies * hidden]")
    _need(table.is_contiguous(), "embedding table must be contiguous")
    lib = load("embedding")
    _check(lib.mie_embedding(_ptr(table), tag(table), _ptr(ids), _ptr(feedback), _ptr(out), ids.numel(), h, V,
                             feedback.numel() if feedback is not None else 0, ctypes.c_float(scale), int(copies), _stream()),
           "embedding")
    return out


def pair_embedding(table: torch.Tensor, pair_table, ctx, last_token: torch.Tensor, out: torch.Tensor, *, scale: float, buckets: int = 0,
                   mul_prev: int = 0, mul_cur: int = 0, first=None, act=None, resolved=None) -> torch.Tensor:
    """out[t] = table[id] * scale + pair_table[(prev * mul_prev + id * mul_cur) mod buckets] (row ``buckets`` at a sequence's first
    token; no second table: the first term alone), float32.  The token in front of a batch row's first token is the
    sequence's ``last_token`` state (int32 [slots + 1, 1], indexed by ``ctx.state_slots``), which is left holding the row's
    last token.  ``first`` (float32) and ``act`` (bfloat16) receive copies of ``out``; ``resolved`` (int32 [T]) the token
    ids with fed-back tokens replaced."""
    V, h = table.shape
    T = ctx.num_tokens
    fb = ctx.token_feedback
    _need(table.is_contiguous() and out.dtype == torch.float32 and out.is_contiguous() and out.shape == (T, h), "out must be float32 [T, hidden]")
    if pair_table is not None:
        _need(pair_table.is_contiguous() and pair_table.shape == (buckets + 1, h) and pair_table.dtype == table.dtype,
              "the pair table must be [buckets + 1, hidden] in the embedding's type")
    _need(last_token.dtype == torch.int32 and last_token.is_contiguous(), "the last-token state must be contiguous int32")
    for t, name in ((first, "first"), (act, "act")):
        if t is not None:
            _need(t.is_contiguous() and t.numel() == T * h and t.dtype == (torch.float32 if name == "first" else torch.bfloat16),
                  f"{name} must be contiguous [T, hidden]")
    if resolved is not None:
        _i32(resolved, "resolved")
    if fb is not None:
        _i32(fb, "feedback")
    lib = load("embedding")
    _check(lib.mie_pair_embedding(_ptr(table), _ptr(pair_table), tag(table), _ptr(ctx.token_ids), _ptr(fb), _ptr(ctx.positions),
                                  _ptr(ctx.token_row), _ptr(ctx.row_q_start), _ptr(ctx.row_q_len), _ptr(ctx.state_slots),
                                  _ptr(last_token), _ptr(out), _ptr(first), _ptr(act), _ptr(resolved), T, h, V,
                                  fb.numel() if fb is not None else 0, ctypes.c_float(scale), int(buckets), ctypes.c_longlong(mul_prev),
                                  ctypes.c_longlong(mul_cur), ctx.num_rows, last_token.shape[0], _stream()), "pair_embedding")
    return out


def normed_add(res: torch.Tensor, addends=(), *, scaled=None, gain=None, vec=None, eps: float = 0.0, act=None, history=None,
               slot: int = 0, coef=None) -> torch.Tensor:
    """res += y / sqrt(mean(y^2) + eps) * gain * vec with y the sum of ``addends`` (up to three [T, W] tensors) and of
    ``scaled`` = (h [T, W], row_scale float32 [T]) as row_scale[t] * h[t]; ``gain`` one float32 on the device, ``vec`` float32
    [W], both optional.  With ``history`` (float32 [slots, T, W]) the new stream is stored as entry ``slot`` and ``res``
    becomes sum over j <= slot of coef[j] * history[j].  ``act`` (bfloat16 [T, W]) receives the rounded result.  Without
    addends nothing is added."""
    T, W = res.shape
    _need(res.dtype == torch.float32 and res.is_contiguous(), "the stream must be contiguous float32")
    addends = [a for a in addends if a is not None]
    _need(len(addends) <= 3, "at most three addends")
    for a in addends + ([scaled[0]] if scaled is not None else []):
        _need(a.is_contiguous() and a.shape == (T, W), "an addend must be contiguous [T, W]")
    if scaled is not None:
        _f32(scaled[1], "row scale", T)
    if gain is not None:
        _f32(gain, "gain", 1)
    if vec is not None:
        _f32(vec, "scale vector", W)
    if act is not None:
        _need(act.dtype == torch.bfloat16 and act.is_contiguous() and act.shape == (T, W), "act must be bfloat16 [T, W]")
    if history is not None:
        _need(history.dtype == torch.float32 and history.is_contiguous() and history.shape[1:] == (T, W) and 0 <= slot < history.shape[0],
              "history must be float32 [slots, T, W]")
        _f32(coef, "depth coefficients", slot + 1)
    pa = [(_ptr(a), tag(a)) for a in addends] + [(ctypes.c_void_p(0), 0)] * (3 - len(addends))
    lib = load("stream_update")
    _check(lib.mie_normed_add(_ptr(res), pa[0][0], pa[0][1], pa[1][0], pa[1][1], pa[2][0], pa[2][1], len(addends),
                              _ptr(scaled[0]) if scaled is not None else ctypes.c_void_p(0), tag(scaled[0]) if scaled is not None else 0,
                              _ptr(scaled[1]) if scaled is not None else ctypes.c_void_p(0), _ptr(gain), _ptr(vec), ctypes.c_float(eps),
                              _ptr(act), _ptr(history), ctypes.c_longlong(T * W), int(slot), _ptr(coef), T, W, _stream()), "normed_add")
    return res


def xielu(x: torch.Tensor, out: torch.Tensor, ap: float, an: float) -> torch.Tensor:
    """out = ap x^2 + x / 2 where x > 0, an (exp(x) - 1 - x) + x / 2 elsewhere."""
    _need(x.is_contiguous() and out.is_contiguous() and out.shape == x.shape and out.dtype == x.dtype, "xielu: contiguous tensors of one shape and type")
    _check(load("activation").mie_xielu(_ptr(x), _ptr(out), tag(x), ctypes.c_longlong(x.numel()), ctypes.c_float(ap), ctypes.c_float(an),
                                        _stream()), "xielu")
    return out


def gelu_gate_rows(g: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, first: int, out: torch.Tensor) -> torch.Tensor:
    """out[t, d] = gelu_tanh(g[t, d]) * table[ids[t], first + d]."""
    T, n = g.shape
    _need(g.is_contiguous() and out.is_contiguous() and out.shape == g.shape and out.dtype == g.dtype == table.dtype and table.is_contiguous(),
          "gate rows: contiguous tensors of one type")
    _i32(ids, "ids")
    _check(load("activation").mie_gelu_gate_rows(_ptr(g), _ptr(table), _ptr(ids), _ptr(out), tag(g), T, n, table.shape[1], int(first),
                                                 table.shape[0], _stream()), "gelu_gate_rows")
    return out


# --------------------------------------------------------------------------- norm

def add_rmsnorm(delta, res: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
                rows: torch.Tensor | None = None) -> torch.Tensor:
    """res += delta (in place, float32); out = rmsnorm(res) * weight.  With ``rows`` the inputs are
    gathered (output row b from input row rows[b]) and ``res`` is not written."""
    n = res.shape[-1]
    _need(res.dtype == torch.float32 and res.is_contiguous(), "the residual stream must be contiguous float32")
    _need(out.is_contiguous() and out.shape[-1] == n, "norm output must be contiguous [rows, n]")
    _need(weight.numel() == n and weight.is_contiguous(), f"norm weight must have {n} entries")
    if delta is not None:
        _need(delta.dtype == out.dtype and delta.shape == res.shape and delta.is_contiguous(),
              "delta must match the residual's shape and the output's type")
    num_rows = out.shape[0]
    if rows is not None:
        _i32(rows, "rows")
        _need(rows.numel() == num_rows, "one gathered row per output row")
    else:
        _need(res.shape[0] == num_rows, "output rows must match residual rows")
    lib = load("norm")
    _check(lib.mie_add_rmsnorm(_ptr(delta), _ptr(res), _ptr(weight), tag(weight), _ptr(out), tag(out),
                               _ptr(rows), num_rows, n, ctypes.c_float(eps), res.shape[0], _stream()), "add_rmsnorm")
    return out


# --------------------------------------------------------------------------- rope + cache write

def _delta_args(deltas, coefs, shape):
    """Up to two addends with their coefficients as kernel arguments (pointer, tag, coefficient each)."""
    _need(len(deltas) <= 2 and len(coefs) == len(deltas), "one or two addends, a coefficient each")
    out = []
    for d, c in zip(deltas, coefs):
        _need(d.is_contiguous() and tuple(d.shape) == tuple(shape) and d.dtype in (torch.float32, torch.bfloat16), "an addend must be contiguous, of the stream's shape, float32 or bfloat16")
        out += [_ptr(d), tag(d), ctypes.c_float(float(c))]
    for _ in range(2 - len(deltas)):
        out += [None, 0, ctypes.c_float(0.0)]
    return out


def add_layernorm(res: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor, *, deltas=(), coefs=(), rows=None, center: bool = True,
                  res_coef: float = 1.0) -> torch.Tensor:
    """res <- res_coef res + sum_k coefs[k] deltas[k] (in place; up to two addends, float32 or bfloat16), then
    out = (res - mean) / sqrt(var + eps) * weight per row (``center`` False: the mean is taken as 0, an RMS norm).  With ``rows``
    output row b comes from row rows[b] and the stream is left as it is."""
    T, n = res.shape
    _need(res.dtype == torch.float32 and res.is_contiguous(), "the stream must be contiguous float32")
    _need(weight.dtype == torch.float32 and weight.is_contiguous() and weight.numel() == n, "float32 norm weight [n]")
    n_out = T
    if rows is not None:
        _i32(rows, "rows")
        n_out = rows.numel()
    _need(out.is_contiguous() and tuple(out.shape) == (n_out, n), "norm output shape")
    _check(load("layer_norm").mie_add_layernorm(_ptr(res), ctypes.c_float(res_coef), *_delta_args(deltas, coefs, res.shape), _ptr(weight), _ptr(out),
                                                tag(out), _ptr(rows), n_out, n, ctypes.c_float(eps), int(center), T, _stream()), "add_layernorm")
    return out


def stream_join(res: torch.Tensor, extra: torch.Tensor, out: torch.Tensor, *, deltas=(), coefs=(), res_coef: float = 1.0) -> torch.Tensor:
    """out[t] = [res_coef res[t] + sum_k coefs[k] deltas[k][t] | extra[t]] in out's type (the stream is not written)."""
    T, n = res.shape
    _need(res.dtype == torch.float32 and res.is_contiguous() and extra.dtype == torch.float32 and extra.is_contiguous() and extra.shape == res.shape,
          "the stream and the second stream must be contiguous float32 of one shape")
    _need(out.is_contiguous() and tuple(out.shape) == (T, 2 * n), "joined rows are [T, 2 n]")
    _check(load("layer_norm").mie_stream_join(_ptr(res), ctypes.c_float(res_coef), *_delta_args(deltas, coefs, res.shape), _ptr(extra), _ptr(out),
                                              tag(out), T, n, _stream()), "stream_join")
    return out


def tanh_cap(x: torch.Tensor, cap: float) -> torch.Tensor:
    """x <- cap tanh(x / cap) in place (float32)."""
    _need(x.dtype == torch.float32 and x.is_contiguous(), "tanh_cap works on contiguous float32")
    _check(load("layer_norm").mie_tanh_cap(_ptr(x), ctypes.c_longlong(x.numel()), ctypes.c_float(cap), _stream()), "tanh_cap")
    return x


def rope_tables(inv_freq: torch.Tensor, max_pos: int):
    """cos, sin [max_pos, rotary_dim/2] float32 of p * inv_freq[j]."""
    _need(inv_freq.dtype == torch.float32 and inv_freq.is_contiguous(), "inv_freq must be float32")
    half = inv_freq.numel()
    cos = torch.empty(max_pos, half, dtype=torch.float32, device=inv_freq.device)
    sin = torch.empty_like(cos)
    lib = build.load("rope_cache")
    _check(lib.mie_rope_table(_ptr(inv_freq), _ptr(cos), _ptr(sin), max_pos, half, _stream()), "rope_table")
    return cos, sin


def rope_cache_write(qkv: torch.Tensor, positions, slots, cos, sin, k_cache, v_cache, num_heads: int,
                     num_kv_heads: int, head_dim: int, rotary_dim: int, page_size: int,
                     write_cache: bool = True) -> None:
    """Rotates q in place inside ``qkv`` [T, (H + 2 H_kv) D] and writes rotated k and v into their
    cache slots (pages laid out [page, kv_head, slot, D])."""
    T = qkv.shape[0]
    _need(qkv.is_contiguous() and qkv.shape[1] == (num_heads + 2 * num_kv_heads) * head_dim,
          "qkv must be contiguous [tokens, (H + 2 H_kv) * D]")
    _i32(positions, "positions")
    _i32(slots, "slots")
    _need(k_cache.dtype == qkv.dtype and v_cache.dtype == qkv.dtype, "cache type must match qkv")
    _need(cos.shape[1] * 2 == rotary_dim, "rotation table does not match rotary_dim")
    lib = load("rope_cache")
    _check(lib.mie_rope_cache_write(_ptr(qkv), tag(qkv), _ptr(positions), _ptr(slots), _ptr(cos), _ptr(sin),
                                    _ptr(k_cache), _ptr(v_cache), T, num_heads, num_kv_heads, head_dim,
                                    rotary_dim, page_size, cos.shape[0], int(write_cache),
                                    ctypes.c_longlong(k_cache.shape[0]), _stream()),
           "rope_cache_write")


# --------------------------------------------------------------------------- attention

class ScoreMods:
    """What an attention kernel does to a score between the scaled product and the softmax.  ``softcap`` c > 0: s <- c tanh(s / c).
    ``dist_bias`` float32 [heads, L]: the query at position p adds entry min(p - j, L - 1) of its head's row to the score of key j
    (after the cap).
    ``sink`` float32 [heads]: exp(sink[head]) is one more term of the softmax's denominator: a key that nothing scores and that carries no value."""

    def __init__(self, softcap: float = 0.0, sink=None, dist_bias=None):
        self.softcap, self.sink, self.dist_bias = float(softcap or 0.0), sink, dist_bias

    def args(self, num_heads: int):
        if self.sink is not None:
            _need(self.sink.dtype == torch.float32 and self.sink.is_contiguous() and self.sink.numel() == num_heads, "one float32 sink per head")
        if self.dist_bias is not None:
            _need(self.dist_bias.dtype == torch.float32 and self.dist_bias.is_contiguous() and self.dist_bias.dim() == 2
                  and self.dist_bias.shape[0] == num_heads and self.dist_bias.shape[1] >= 1, "distance bias must be float32 [heads, L]")
        return (ctypes.c_float(self.softcap), _ptr(self.sink), _ptr(self.dist_bias),
                int(self.dist_bias.shape[1]) if self.dist_bias is not None else 0)


_NO_MODS = ScoreMods()


def paged_attention(q: torch.Tensor, q_stride: int, k_cache, v_cache, block_tables, row_q_start, row_q_len,
                    row_ctx_len, num_tokens: int, out: torch.Tensor, num_heads: int, num_kv_heads: int,
                    head_dim: int, page_size: int, scale: float, window: int | None = None,
                    min_q_len: int = 1, mods: ScoreMods | None = None) -> torch.Tensor:
    """Causal attention of every new token over its request's pages (CUDA-core kernel, float32 or
    bfloat16).  ``q`` holds [H, D] at the start of each token row of ``q_stride`` elements.  Rows
    with fewer than ``min_q_len`` new tokens are left alone."""
    _need(head_dim % 16 == 0 and 16 <= head_dim <= 256,
          f"head_dim {head_dim}: this kernel takes multiples of 16 from 16 to 256")
    _need(num_heads % num_kv_heads == 0, "query heads must be a multiple of kv heads")
    for t, n in ((block_tables, "block_tables"), (row_q_start, "row_q_start"), (row_q_len, "row_q_len"),
                 (row_ctx_len, "row_ctx_len")):
        _i32(t, n)
    _need(q.dtype == k_cache.dtype == v_cache.dtype and out.dtype in (q.dtype, torch.float32),
          "q and caches must share a type; out has it too, or is float32")
    _need(out.is_contiguous(), "attention output must be contiguous")
    rows = row_q_len.numel()
    lib = load("attention_simt")
    _check(lib.mie_paged_attention(_ptr(q), ctypes.c_int64(q_stride), _ptr(k_cache), _ptr(v_cache),
                                   _ptr(block_tables), block_tables.shape[1], _ptr(row_q_start), _ptr(row_q_len),
                                   _ptr(row_ctx_len), rows, num_tokens, _ptr(out), tag(q), num_heads,
                                   num_kv_heads, head_dim, page_size, ctypes.c_float(scale),
                                   int(window or 0), int(min_q_len), ctypes.c_longlong(k_cache.shape[0]),
                                   int(out.dtype == torch.float32 and q.dtype != torch.float32), *(mods or _NO_MODS).args(num_heads),
                                   _stream()),
           "paged_attention")
    return out


def prefill_attention(q: torch.Tensor, q_stride: int, k_cache, v_cache, block_tables, row_q_start, row_q_len,
                      row_ctx_len, num_tokens: int, out: torch.Tensor, num_heads: int, num_kv_heads: int,
                      head_dim: int, page_size: int, scale: float, window: int | None = None,
                      min_q_len: int = 2, work=None, mods: ScoreMods | None = None) -> torch.Tensor:
    """Causal attention of prompt portions over their request's pages (bfloat16, tensor cores).
    Rows with fewer than ``min_q_len`` new tokens are left alone.  ``work`` = (rows, tokens): how many rows have
    ``min_q_len`` tokens or more and their tokens in sum, where the caller knows -- the launch then has blocks for the
    tiles those rows can have, not for every row of the step."""
    _need(q.dtype == torch.bfloat16 == k_cache.dtype == v_cache.dtype and out.dtype in (torch.bfloat16, torch.float32),
          "prefill attention is bfloat16 (its output bfloat16 or float32)")
    _need(head_dim % 16 == 0 and 16 <= head_dim <= 128,
          f"head_dim {head_dim}: the prefill kernel takes multiples of 16 from 16 to 128")
    _need(num_heads % num_kv_heads == 0, "query heads must be a multiple of kv heads")
    for t, n in ((block_tables, "block_tables"), (row_q_start, "row_q_start"), (row_q_len, "row_q_len"),
                 (row_ctx_len, "row_ctx_len")):
        _i32(t, n)
    _need(out.is_contiguous(), "attention output must be contiguous")
    lib = load("attention_prefill")
    _check(lib.mie_prefill_attention(_ptr(q), ctypes.c_int64(q_stride), _ptr(k_cache), _ptr(v_cache),
                                     _ptr(block_tables), block_tables.shape[1], _ptr(row_q_start), _ptr(row_q_len),
                                     _ptr(row_ctx_len), row_q_len.numel(), num_tokens, _ptr(out), num_heads,
                                     num_kv_heads, head_dim, page_size, ctypes.c_float(scale), int(window or 0),
                                     int(min_q_len), ctypes.c_longlong(k_cache.shape[0]), *_work_args(work),
                                     int(out.dtype == torch.float32), *(mods or _NO_MODS).args(num_heads), _stream()),
           "prefill_attention")
    return out


def prefill_attention_tc(q: torch.Tensor, q_stride: int, k_cache, v_cache, block_tables, row_q_start, row_q_len,
                         row_ctx_len, num_tokens: int, out: torch.Tensor, num_heads: int, num_kv_heads: int,
                         head_dim: int, page_size: int, scale: float, window: int | None = None,
                         min_q_len: int = 2, work=None, mods: ScoreMods | None = None) -> torch.Tensor:
    """Causal attention of prompt portions on tcgen05 (S and O in tensor memory, operands by TMA);
    head_dim 64 or 128.  ``work``: as for ``prefill_attention``."""
    _need(q.dtype == torch.bfloat16 == k_cache.dtype == v_cache.dtype and out.dtype in (torch.bfloat16, torch.float32),
          "prefill attention is bfloat16 (its output bfloat16 or float32)")
    _need(head_dim in (64, 128), f"head_dim {head_dim}: the tcgen05 prefill kernel takes 64 and 128")
    _need(q_stride % 8 == 0 and page_size >= 8, "the tcgen05 prefill kernel needs q rows and pages of whole 16-byte pieces")
    _need(num_heads % num_kv_heads == 0, "query heads must be a multiple of kv heads")
    for t, n in ((block_tables, "block_tables"), (row_q_start, "row_q_start"), (row_q_len, "row_q_len"),
                 (row_ctx_len, "row_ctx_len")):
        _i32(t, n)
    _need(out.is_contiguous() and k_cache.is_contiguous() and v_cache.is_contiguous(), "contiguous caches and output")
    lib = load("attention_prefill_tc")
    _check(lib.mie_prefill_attention_tc(_ptr(q), ctypes.c_int64(q_stride), _ptr(k_cache), _ptr(v_cache),
                                        ctypes.c_int64(k_cache.shape[0]), _ptr(block_tables), block_tables.shape[1],
                                        _ptr(row_q_start), _ptr(row_q_len), _ptr(row_ctx_len), row_q_len.numel(),
                                        num_tokens, _ptr(out), num_heads, num_kv_heads, head_dim, page_size,
                                        ctypes.c_float(scale), int(window or 0), int(min_q_len), *_work_args(work),
                                        int(out.dtype == torch.float32), *(mods or _NO_MODS).args(num_heads), _stream()),
           "prefill_attention_tc")
    return out


def _work_args(work):
    rows, tokens = work if work is not None else (0, 0)
    return int(rows), int(tokens)


def set_prefill_pairs(mode: int = -1) -> None:
    """Which tcgen05 prefill kernel serves head_dim 64: -1 chooses by the size of the launch (the default), 0 always
    one query tile a block, 1 always two query tiles side by side (csrc/attention_prefill_tc.cu)."""
    load("attention_prefill_tc").mie_prefill_attention_tc_pairs(int(mode))


def check_tc_errors() -> None:
    """Raises if a block of a tensor-core kernel gave up a bounded wait (call after a synchronise)."""
    for name, fn in (("attention_prefill_tc", "mie_prefill_attention_tc"), ("attention_decode", "mie_decode_attention")):
        lib = build._libs.get(name)
        if lib is not None and getattr(lib, fn + "_error")():
            getattr(lib, fn + "_clear_error")()
            raise KernelError(f"a block of {name} gave up waiting on a barrier; its output is not valid")


_workspaces: dict = {}
_outgrown: list = []          # scratch tensors that a larger one replaced; see _workspace


def _workspace(device, name: str, numel: int, dtype) -> torch.Tensor:
    """A persistent, zero-initialised scratch tensor per (device, name), grown on demand.  Kernels
    that use it leave it as they need to find it, so it is cleared only when it is (re)made.  A captured
    graph keeps the ADDRESS of the tensor it was captured with, so a tensor that has been outgrown is kept
    alive, never handed back to the allocator: graphs captured with it go on using it (each scratch tensor
    is self-contained, and the launches of one stream use them one after the other).  Sizes at least
    double, which bounds what is kept."""
    key = (str(device), name)
    t = _workspaces.get(key)
    if t is None or t.numel() < numel:
        if t is not None:
            _outgrown.append(t)
            numel = max(numel, 2 * t.numel())
        t = torch.zeros(max(numel, 1024), dtype=dtype, device=device)
        _workspaces[key] = t
    return t


def decode_splits(rows: int, kv_units: int, max_ctx: int, head_dim: int = 64) -> int:
    """How many parts to cut the context into (a cluster of 2, 4 or 8 blocks; the reference keeps 256 keys a
    part, inference_engine/kernels/decode_attention.py:117-125).

    Heads of up to 64: as many parts as still leave every block a place beside the others -- four blocks on an SM
    with page copies by TMA and two stages (``decode_uses_tma``, ``decode_stages``) -- and two 64-key tiles a part.
    Measured on B200 (32 q / 4 kv heads of 64, device time in a graph, context bound 960; the plan before ->
    this one): 512 keys, 20 / 32 rows 7.1 -> 6.4 / 8.2 -> 7.0 us (4 parts), 40 / 64 / 72 rows 10.5 -> 8.7 / 11.6 -> 9.2 /
    12.0 -> 9.4 us (2 parts), 80 / 96 rows 20.4 -> 11.3 / 20.6 -> 11.6 us (whole, by TMA, four stages); 960 keys, 16
    rows 8.4 -> 7.3 us (8 parts), 24 rows 11.8 -> 9.0, 64 rows 19.7 -> 14.2, 96 rows 36.4 -> 19.6 us.  One block
    more than the places (592) and the launch takes half as long again: 72 rows in two parts 9.4 us, 80 rows 16.3.
    Wider heads (two blocks on an SM): parts while the batch alone leaves SMs idle."""
    blocks = max(1, rows * kv_units)
    splits = 1
    if head_dim <= 64:
        most = -(-(-(-max(1, max_ctx) // 64)) // 2)            # two tiles a part at least
        while splits < 8 and blocks * splits * 2 <= decode_blocks_per_sm(head_dim) * num_sms() and splits * 2 <= most:
            splits *= 2
        return splits
    while splits < 8 and blocks * splits * 2 <= 2 * num_sms() and splits * 64 < max_ctx:
        splits *= 2
    return splits


LONG_PART_TILES = 8          # a part of a long context is at least this many 64-key tiles (512 keys)


def decode_blocks_per_sm(head_dim: int) -> int:
    """Blocks of the decode kernel that share an SM with page copies by TMA and three stages: a stage is 16 KB of
    keys and values per 64 columns of the head, beside 6 KB of static shared memory."""
    return 4 if head_dim <= 64 else 2


def decode_plan(rows: int, kv_units: int, max_ctx: int, tma_ok: bool, head_dim: int = 64) -> tuple[int, str, int]:
    """(splits, merge, min_part_tiles) for a decode launch whose contexts reach up to ``max_ctx``.

    Short contexts and few rows: the cluster merge of ``decode_splits`` (one launch, no global round trip).
    Long contexts (two parts of LONG_PART_TILES tiles or more) with 64 or more (row, kv head) units: a block
    walks its keys at about 16 ns a key whatever else runs (three or four 16 KB tiles in flight), so the
    bytes per second follow the number of blocks that run beside one another -- four per SM (two with heads
    of 128) with page copies by TMA, three stages and no receive slots of a cluster.  The context is then cut into as many
    parts as fill those places, merged through scratch memory, and a row shorter than the launch was laid
    out for is cut into fewer parts by the kernel (``min_part_tiles``).  Measured on B200, 32 q / 4 kv
    heads of 64, device time in a graph, cluster plan -> this plan: 64 rows x 8,192 keys 149 -> 90 us
    (5.96 TB/s), 32 x 8,192 72 -> 48 us, 16 x 8,192 38 -> 31 us, 64 x 2,048 36.8 -> 31.0 us, 32 x 2,048
    20.5 -> 17.8 us; 8 rows stay with the cluster of 8 (20.9 us at 8,192 keys against 24.2 us).  With 8 kv
    heads of 128 (32 rows x 2,048 keys) the whole context per block is the fastest plan (46.3 us; two parts
    62.7 us): 256 blocks already fill the two places an SM has."""
    units = max(1, rows * kv_units)
    clustered = decode_splits(rows, kv_units, max_ctx, head_dim)
    tiles = -(-max(1, max_ctx) // 64)
    if tma_ok and units >= 64 and tiles >= 2 * LONG_PART_TILES:
        parts = min(decode_blocks_per_sm(head_dim) * num_sms() // units, tiles // LONG_PART_TILES, 8 if head_dim <= 64 else 16)
        # Only where scratch allows MORE parts than a cluster (which takes 2, 4 or 8): with as many parts the cluster
        # is the faster merge (heads of 64, page copies by TMA, two stages; rows x keys, scratch -> cluster:
        # 64 x 2,048 31.5 -> 25.6 us, 64 x 3,400 45.5 -> 39.6, 32 x 2,048 18.2 -> 14.6, 16 x 2,048 17.6 -> 10.0 us);
        # three parts through scratch against two of a cluster win from about 3,400 keys on (48 x 7,000: 63.9
        # against 71.9 us; 48 x 2,048: 27.0 against 24.0 us)
        if parts >= 2 and parts > clustered:
            return parts, "scratch", LONG_PART_TILES
    return clustered, "cluster", 0


def decode_stages(blocks: int, max_ctx: int, splits: int, tma: bool = False, head_dim: int = 64, clustered: bool = True) -> int:
    """Tiles of 64 keys in flight per block.  Shared memory that attention does not take stays free
    for the prologue of the kernel after it (the output projection fills its ring with weights while
    attention still runs): measured on B200 in the whole decode step at batch 8, 512 keys, three
    stages 1.069 ms, four 1.087 ms, two 1.135 ms (two stages are slower by themselves).  Parts of
    more than four tiles want the deepest ring (batch 64, 512 keys: 12.7 us with four stages, 15.5 us
    with three; 2048 keys: 40 us with four, 60 us with two); more blocks than fit beside one another
    at four stages want two, which puts twice as many on an SM (batch 256, 512 keys: 34 us against
    46 us).  Heads of 128 with TMA copies: three stages (two blocks on an SM) up to six blocks per SM in the
    launch, two stages (three on an SM) beyond (32 kv heads of 128, 512 keys: 64 rows 87.9 against 98.0 us, 32 rows
    51.4 against 53.9 us; 8 kv heads, 64 rows 32.3 against 27.7 us)."""
    tiles = -(-(-(-max(1, max_ctx) // splits)) // 64)
    if head_dim > 64 and tma:
        return 2 if blocks > 6 * num_sms() else 3
    if tma and splits > 1 and clustered:
        return 2                          # the parts of a cluster by TMA: four blocks on an SM (see decode_splits)
    if tma and blocks <= 3 * num_sms():
        return 4                          # whole contexts by TMA, up to three blocks an SM (80 rows x 512 keys: 11.3 us; 128 rows want three stages: 13.0 against 21.0 us)
    if blocks > 3 * num_sms():
        return 3 if tma else 2            # TMA tiles are unpadded: three stages still put four blocks on an SM (256 x 512: 29.2 us, two stages 30.7)
    return 3 if tiles <= 4 else 4


def decode_uses_tma(blocks: int, head_dim: int = 64) -> bool:
    """Whether the decode kernel fetches keys and values a page per TMA copy instead of 16 bytes per
    cp.async.  Measured on B200 (32 q / 4 kv heads of 64): it pays where there are more blocks than
    fit beside one another at three or four padded stages of 16-byte copies, from two blocks per SM on (128 requests
    x 512 keys: 14.9 us against 20.6 us; 256 x 512: 29.2 against 34.4 us; 80 x 512, whole contexts: 11.3 against
    20.4 us; 16 x 960 in 8 parts: 7.3 against 12.0 us) and costs a little where each block walks a long part alone (64 x 2048: 42.9 against
    40.0 us; 8 x 512: 7.5 against 7.1 us) -- the copies were never the bound there, the softmax
    bookkeeping per 16 keys is.  Cache slots beyond a request's context are copied along with their
    page and must hold finite values (the cache storage starts as zeros).  Heads of 128: always -- a stage of
    cp.async copies is 34 KB there and the 16-byte copies are four times as many (8 rows x 512 keys, 8 kv heads:
    7.3 against 14.2 us; 1,024 keys 9.8 against 20.4 us; 32 kv heads, 1 row x 512 keys: 6.2 against 14.4 us)."""
    return head_dim > 64 or blocks > 2 * num_sms()


def decode_attention(q: torch.Tensor, q_stride: int, k_cache, v_cache, block_tables, row_q_start, row_q_len,
                     row_ctx_len, out: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int,
                     page_size: int, scale: float, window: int | None = None, max_ctx: int = 0,
                     splits: int | None = None, merge: str | None = None, stages: int | None = None,
                     tma: bool | None = None, min_part_tiles: int = 0, rope=None, mods: ScoreMods | None = None) -> torch.Tensor:
    """Attention of rows with exactly one new token (bfloat16, tensor cores, context split across
    blocks and merged in the same launch).  Rows with more new tokens are skipped.  ``merge`` =
    "cluster": 1, 2, 4 or 8 splits merged through distributed shared memory; "scratch": any number of
    splits merged through scratch memory in global memory, a row cut into at most (its tiles /
    ``min_part_tiles``) of them.  With neither ``splits`` nor ``merge`` given, ``decode_plan`` chooses.

    ``rope`` = (cos, sin), float32 [positions, head_dim / 2]: ``q`` holds the UNROTATED q|k|v activation of
    every row (keys ``num_heads`` heads in, values behind them), and the kernel rotates q and the new key by the
    row's position (context length - 1, the whole head as rotary width), uses them, and writes the new key and
    value into the cache -- the separate rotate-and-store launch is not needed then."""
    _need(q.dtype == torch.bfloat16 == k_cache.dtype == v_cache.dtype and out.dtype in (torch.bfloat16, torch.float32),
          "decode attention is bfloat16 (its output bfloat16 or float32)")
    _need(head_dim % 16 == 0 and 16 <= head_dim <= 128,
          f"head_dim {head_dim}: the decode kernel takes multiples of 16 from 16 to 128")
    _need(num_heads % num_kv_heads == 0, "query heads must be a multiple of kv heads")
    for t, n in ((block_tables, "block_tables"), (row_q_start, "row_q_start"), (row_q_len, "row_q_len"),
                 (row_ctx_len, "row_ctx_len")):
        _i32(t, n)
    rows = row_q_len.numel()
    cos = sin = None
    if rope is not None:
        cos, sin = rope
        _need(head_dim % 32 == 0, f"head_dim {head_dim}: rotation inside the decode kernel takes multiples of 32")
        _need(cos.dtype == torch.float32 == sin.dtype and cos.is_contiguous() and sin.is_contiguous()
              and cos.shape == sin.shape and cos.dim() == 2 and cos.shape[1] == head_dim // 2,
              "rope tables must be contiguous float32 [positions, head_dim / 2]")
        _need(q_stride >= (num_heads + 2 * num_kv_heads) * head_dim and q_stride % 8 == 0,
              "rotation inside the decode kernel reads q|k|v rows (16-byte aligned)")
    chunks = -(-(num_heads // num_kv_heads) // 16)
    tma_ok = head_dim in (64, 128) and page_size >= 8
    if splits is None and merge is None:
        splits, merge, min_part_tiles = decode_plan(rows, num_kv_heads * chunks, max_ctx or 1, tma_ok and tma is not False,
                                                    head_dim)
        if merge == "scratch" and tma is None:
            tma = True
    elif splits is None:
        splits = decode_splits(rows, num_kv_heads * chunks, max_ctx or 1, head_dim)
    merge = merge or "cluster"
    if tma is None:
        tma = decode_uses_tma(rows * num_kv_heads * chunks * splits, head_dim)
    tma = bool(tma) and tma_ok
    if stages is None:
        stages = decode_stages(rows * num_kv_heads * chunks * splits, max_ctx or 4096, splits, tma, head_dim,
                               clustered=merge == "cluster" and splits in (1, 2, 4, 8))
    part_o = part_lse = counters = None
    if merge == "cluster" and splits not in (1, 2, 4, 8):
        merge = "scratch"
    if splits > 1 and merge == "scratch":
        part_o = _workspace(q.device, "decode_part_o", rows * num_heads * splits * head_dim, torch.float32)
        part_lse = _workspace(q.device, "decode_part_lse", rows * num_heads * splits, torch.float32)
        counters = _workspace(q.device, "decode_counters", rows * num_kv_heads * chunks, torch.int32)
    lib = load("attention_decode")
    _check(lib.mie_decode_attention(_ptr(q), ctypes.c_int64(q_stride), _ptr(k_cache), _ptr(v_cache),
                                    _ptr(block_tables), block_tables.shape[1], _ptr(row_q_start), _ptr(row_q_len),
                                    _ptr(row_ctx_len), rows, _ptr(out), num_heads, num_kv_heads, head_dim,
                                    page_size, ctypes.c_float(scale), int(window or 0), int(splits),
                                    _ptr(part_o), _ptr(part_lse), _ptr(counters), int(stages or 0),
                                    ctypes.c_int64(k_cache.shape[0] if tma else 0), ctypes.c_int64(k_cache.shape[0]),
                                    int(min_part_tiles if merge == "scratch" else 0),
                                    _ptr(cos), _ptr(sin), int(cos.shape[0]) if cos is not None else 0,
                                    int(out.dtype == torch.float32), *(mods or _NO_MODS).args(num_heads), _stream()),
           "decode_attention")
    return out


# --------------------------------------------------------------------------- activation

def swiglu(gate_up: torch.Tensor, out: torch.Tensor, interleaved: bool = False) -> torch.Tensor:
    """out = silu(gate_up[:, :I]) * gate_up[:, I:]; with ``interleaved`` gate and up alternate:
    out[:, i] = silu(gate_up[:, 2i]) * gate_up[:, 2i + 1]."""
    T, two_i = gate_up.shape
    _need(two_i % 2 == 0 and out.shape == (T, two_i // 2) and out.dtype == gate_up.dtype
          and out.is_contiguous() and gate_up.is_contiguous(), "swiglu shapes/types do not match")
    lib = build.load("activation")
    _check(lib.mie_swiglu(_ptr(gate_up), _ptr(out), tag(out), T, two_i // 2, int(interleaved), _stream()), "swiglu")
    return out


# --------------------------------------------------------------------------- matrix product (CUDA cores)

def gemm_simt(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: torch.Tensor | None = None):
    """out[M, N] = x[M, K] @ w[N, K]^T (+ bias), float32 accumulation on CUDA cores."""
    M, K = x.shape
    N = w.shape[0]
    _need(w.shape[1] == K and out.shape == (M, N), f"gemm shapes: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    _need(x.is_contiguous() and w.is_contiguous() and out.is_contiguous(), "gemm operands must be contiguous")
    lib = build.load("gemm_simt")
    _check(lib.mie_gemm_simt(_ptr(x), tag(x), _ptr(w), tag(w), _ptr(bias), tag(bias) if bias is not None else 0,
                             _ptr(out), tag(out), M, N, K, _stream()),
           f"gemm_simt ({x.dtype}, {w.dtype} -> {out.dtype})")
    return out


# --------------------------------------------------------------------------- sampling

def sample(logits: torch.Tensor, temperature, request, position, seed: int, out: torch.Tensor,
           host_out: torch.Tensor | None = None, host_turn: torch.Tensor | None = None):
    """Token ids [rows] from float32 logits [rows, vocab]; per-row temperature (0 = greedy), request
    id (int64) and output position (int32) key the noise.  ``host_out``: a pinned host tensor
    [turns, n >= rows] int32 that also receives the tokens, in row ``host_turn[0]`` (a device int32
    tensor; row 0 without it), written by the kernel itself (pinned memory is addressable from the
    device), so that no copy has to follow."""
    rows, vocab = logits.shape
    _need(logits.dtype == torch.float32 and logits.is_contiguous(), "logits must be contiguous float32")
    _need(temperature.dtype == torch.float32 and request.dtype == torch.int64 and position.dtype == torch.int32
          and out.dtype == torch.int32, "sampling argument types")
    host_ptr, stride = ctypes.c_void_p(0), 0
    if host_out is not None:
        _need(host_out.dtype == torch.int32 and host_out.dim() == 2 and host_out.is_pinned() and host_out.is_contiguous()
              and host_out.shape[1] >= rows, "host_out must be a pinned int32 tensor [turns, n >= rows]")
        if host_turn is not None:
            _need(host_turn.is_cuda and host_turn.dtype == torch.int32 and host_turn.numel() >= 1, "host_turn must be a device int32 tensor")
        host_ptr, stride = ctypes.c_void_p(host_out.data_ptr()), host_out.shape[1]
    lib = build.load("sampling")
    _check(lib.mie_sample(_ptr(logits), _ptr(temperature), _ptr(request), _ptr(position),
                          ctypes.c_uint64(seed & ((1 << 64) - 1)), _ptr(out), rows, vocab, host_ptr,
                          _ptr(host_turn) if host_out is not None else ctypes.c_void_p(0), stride, _stream()), "sample")
    return out


# --------------------------------------------------------------------------- post-norm stream, grouped statistics

def _tagged(t):
    return (_ptr(t), tag(t)) if t is not None else (ctypes.c_void_p(0), 0)


def stream_norm(res: torch.Tensor, weight: torch.Tensor, groups: int, eps: float, out: torch.Tensor | None = None, *,
                alpha: float = 1.0, deltas=(), inner_weights=(), coef: float = 1.0, rows: torch.Tensor | None = None):
    """res <- gnorm(alpha * res + coef * sum_k b_k) * weight in place (float32), where b_k is ``deltas[k]`` or, with
    ``inner_weights[k]``, that delta RMS-normed over its whole row and multiplied by the weight; gnorm divides each
    of ``groups`` equal consecutive parts of a row by its own root mean square.  ``out`` (optional) receives the
    result in its own type.  With ``rows`` output row b comes from stream row rows[b] and ``res`` is not written."""
    n = res.shape[-1]
    _need(res.dtype == torch.float32 and res.is_contiguous(), "the residual stream must be contiguous float32")
    _need(weight.numel() == n and weight.is_contiguous(), f"norm weight must have {n} entries")
    _need(groups >= 1 and n % groups == 0, f"{groups} groups do not divide a row of {n}")
    _need(len(deltas) <= 2, "at most two branches are added")
    deltas = list(deltas) + [None] * (2 - len(deltas))
    inner = list(inner_weights) + [None] * (2 - len(inner_weights))
    d_tags = {tag(d) for d in deltas if d is not None}
    i_tags = {tag(w) for w in inner if w is not None}
    _need(len(d_tags) <= 1 and len(i_tags) <= 1, "branches (and their weights) must share a type")
    for d in deltas:
        if d is not None:
            _need(d.shape == res.shape and d.is_contiguous(), "a branch must match the stream's shape")
    for w in inner:
        if w is not None:
            _need(w.numel() == n and w.is_contiguous(), f"a branch's norm weight must have {n} entries")
    num_rows = res.shape[0]
    if rows is not None:
        _i32(rows, "rows")
        num_rows = rows.numel()
        _need(out is not None, "gathered rows need an output")
    if out is not None:
        _need(out.is_contiguous() and out.shape == (num_rows, n), "norm output must be contiguous [rows, n]")
    lib = load("norm_group")
    _check(lib.mie_stream_norm(_ptr(res), ctypes.c_float(alpha), _ptr(deltas[0]), _ptr(inner[0]), _ptr(deltas[1]), _ptr(inner[1]),
                               d_tags.pop() if d_tags else 0, i_tags.pop() if i_tags else 0, ctypes.c_float(coef),
                               _ptr(weight), tag(weight), int(groups), ctypes.c_float(eps), _ptr(out),
                               tag(out) if out is not None else 0, _ptr(rows), num_rows, n, res.shape[0], _stream()),
           "stream_norm")
    return out


# --------------------------------------------------------------------------- q/k norm, rotation, padded cache write

def qk_norm_rope(qkv: torch.Tensor, positions, slots, freq: torch.Tensor, q_out: torch.Tensor, k_cache, v_cache, *,
                 num_heads: int, num_kv_heads: int, dim: int, vdim: int, rot: int, page_size: int, eps: float = 0.0,
                 q_weight=None, k_weight=None, temp=None, q_scale: float = 1.0, k_scale: float = 1.0,
                 write_cache: bool = True, head_norm: bool = False, interleaved: bool = False, pos_temp=None) -> torch.Tensor:
    """From the fused projection rows [q: H x dim | k: G x dim | v: G x vdim | ...]: q and k optionally RMS-normed over
    their whole projection (``head_norm``: per head, with ``dim`` weights shared by the heads), rotated by position x ``freq``
    over their first ``rot`` dims (pairs (i, i + rot/2), or (2i, 2i + 1) with ``interleaved``), q scaled per head and, with
    ``pos_temp`` = (coef, every), by 1 + coef ln(floor((position + 1) / every) + 1); q written to ``q_out`` [T, H, DP] and k, v
    to their cache slots (pages [page, G, page_size, DP], tails zero)."""
    T = qkv.shape[0]
    DP = q_out.shape[-1]
    _need(qkv.dim() == 2 and qkv.stride(1) == 1
          and qkv.shape[1] >= (num_heads * dim + (num_kv_heads * (dim + vdim) if write_cache else 0)),
          "qkv rows must hold q, k and v (q alone when the cache is not written)")
    _need(q_out.is_contiguous() and q_out.shape == (T, num_heads, DP) and q_out.dtype == qkv.dtype, "q_out must be [T, H, DP]")
    _need(k_cache.dtype == qkv.dtype == v_cache.dtype and k_cache.shape[-1] == DP and k_cache.is_contiguous(), "cache type and width")
    _need(freq.dtype == torch.float32 and freq.numel() * 2 == rot and freq.is_contiguous(), "one float32 frequency per rotated pair")
    _i32(positions, "positions")
    _i32(slots, "slots")
    ws = [w for w in (q_weight, k_weight, temp) if w is not None]
    _need(len({w.dtype for w in ws}) <= 1 and all(w.is_contiguous() for w in ws), "norm weights and temperatures must share a type")
    if q_weight is not None:
        _need(q_weight.numel() == (dim if head_norm else num_heads * dim), "q norm weight size")
    if k_weight is not None:
        _need(k_weight.numel() == (dim if head_norm else num_kv_heads * dim), "k norm weight size")
    coef, every = (float(pos_temp[0]), int(pos_temp[1])) if pos_temp else (0.0, 0)
    if temp is not None:
        _need(temp.numel() == num_heads, "one temperature per head")
    lib = load("qk_norm_rope")
    _check(lib.mie_qk_norm_rope(_ptr(qkv), tag(qkv), ctypes.c_longlong(qkv.stride(0)), _ptr(positions), _ptr(slots), _ptr(freq),
                                _ptr(q_weight), _ptr(k_weight), _ptr(temp), tag(ws[0]) if ws else 0, ctypes.c_float(eps),
                                ctypes.c_float(q_scale), ctypes.c_float(k_scale), _ptr(q_out), _ptr(k_cache), _ptr(v_cache), T,
                                num_heads, num_kv_heads, dim, vdim, DP, rot, page_size, ctypes.c_longlong(k_cache.shape[0]),
                                int(write_cache), int(head_norm), int(interleaved), ctypes.c_float(coef), every, _stream()), "qk_norm_rope")
    return q_out


# --------------------------------------------------------------------------- retention

def retention_scan(qkv: torch.Tensor, positions, row_q_start, row_q_len, state_slots, decay, freq, state, out, *,
                   num_heads: int, dim: int, vdim: int, rot: int, k_scale: float, max_q_len: int) -> torch.Tensor:
    """S <- decay_h S + k v^T, o = S^T q for every new token of every row, from and to ``state`` [slots, H, vdim, dim]
    float32; q and k are rotated (angle = position x ``freq``) and k scaled first.  ``qkv`` rows hold
    [q: H x dim | k: H x dim | v: H x vdim | ...]; ``out`` [T, H * vdim] float32.  Rows longer than a chunk are cut
    into chunks that run side by side (``max_q_len``: the longest row the launch may meet)."""
    T = qkv.shape[0]
    _need(qkv.dim() == 2 and qkv.stride(1) == 1 and qkv.shape[1] >= num_heads * (2 * dim + vdim), "qkv rows must hold q, k and v")
    _need(state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (num_heads, vdim, dim),
          "state must be float32 [slots, H, vdim, dim]")
    _need(out.dtype == torch.float32 and out.is_contiguous() and out.shape == (T, num_heads * vdim), "out must be float32 [T, H * vdim]")
    _need(decay.dtype == torch.float32 and decay.numel() == num_heads, "one float32 decay per head")
    _need(freq.dtype == torch.float32 and freq.numel() * 2 == rot, "one float32 frequency per rotated pair")
    for t, n in ((positions, "positions"), (row_q_start, "row_q_start"), (row_q_len, "row_q_len"), (state_slots, "state_slots")):
        _i32(t, n)
    _need(positions.numel() == T, "one position per token")
    lib = load("retention")
    chunk = lib.mie_retention_chunk_tokens()
    chunks = 2 * (T // chunk) if max_q_len > chunk else 0
    scratch = _workspace(qkv.device, "retention_chunks", chunks * num_heads * vdim * dim, torch.float32) if chunks else None
    qr = torch.empty(2, T, num_heads * dim, dtype=torch.float32, device=qkv.device)
    _check(lib.mie_retention_scan(_ptr(qkv), tag(qkv), ctypes.c_longlong(qkv.stride(0)), _ptr(positions), _ptr(row_q_start),
                                  _ptr(row_q_len), _ptr(state_slots), _ptr(decay), _ptr(freq), ctypes.c_float(k_scale),
                                  _ptr(state), _ptr(qr[0]), _ptr(qr[1]), _ptr(scratch), ctypes.c_longlong(chunks), _ptr(out), T,
                                  row_q_len.numel(), int(max_q_len), num_heads, dim, vdim, rot, _stream()), "retention_scan")
    return out


def decay_scan(rows_in: torch.Tensor, positions, row_q_start, row_q_len, state_slots, state, out, *, num_heads: int, dim: int, vdim: int,
               max_q_len: int, decay=None, tok_decay=None, k_tok=None, act: bool = False, ones: bool = False, q_scale: float = 1.0,
               k_scale: float = 1.0, freq=None, rot: int = 0) -> torch.Tensor:
    """The general form of ``retention_scan``: S <- a S + k v^T, o = S^T q per head with a = ``decay`` [H] or, per token,
    ``tok_decay`` [T, H]; ``k_tok`` [T, H] is one more factor on a token's key; ``act``: q, k and v pass silu (no rotation
    then); ``ones``: the state and the output have a column more per head, fed with ones instead of a value (the decayed sum
    of the keys).  ``rows_in`` rows hold [q: H x dim | k: H x dim | v: H x vdim | ...]; state [slots, H, vdim + ones, dim] and
    out [T, H * (vdim + ones)] float32."""
    T = rows_in.shape[0]
    dv = vdim + int(ones)
    _need(rows_in.dim() == 2 and rows_in.stride(1) == 1 and rows_in.shape[1] >= num_heads * (2 * dim + vdim), "rows must hold q, k and v")
    _need(state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (num_heads, dv, dim),
          "state must be float32 [slots, H, vdim (+ 1), dim]")
    _need(out.dtype == torch.float32 and out.is_contiguous() and out.shape == (T, num_heads * dv), "out must be float32 [T, H * (vdim (+ 1))]")
    _need((decay is None) != (tok_decay is None), "a decay per head or per token and head, not both")
    if decay is not None:
        _need(decay.dtype == torch.float32 and decay.numel() == num_heads, "one float32 decay per head")
    for t_, n in ((tok_decay, "tok_decay"), (k_tok, "k_tok")):
        if t_ is not None:
            _need(t_.dtype == torch.float32 and t_.is_contiguous() and t_.shape == (T, num_heads), f"{n} must be float32 [T, H]")
    if freq is None:
        freq = torch.empty(0, dtype=torch.float32, device=rows_in.device)
    _need(freq.dtype == torch.float32 and freq.numel() * 2 == rot and not (act and rot), "one float32 frequency per rotated pair; no rotation of activated q, k")
    for t_, n in ((positions, "positions"), (row_q_start, "row_q_start"), (row_q_len, "row_q_len"), (state_slots, "state_slots")):
        _i32(t_, n)
    _need(positions.numel() == T, "one position per token")
    lib = load("retention")
    chunk = lib.mie_retention_chunk_tokens()
    chunks = 2 * (T // chunk) if max_q_len > chunk else 0
    scratch = _workspace(rows_in.device, "retention_chunks", chunks * num_heads * dv * dim, torch.float32) if chunks else None
    cdec = _workspace(rows_in.device, "retention_chunk_decay", (chunks + 1) * num_heads, torch.float32) if chunks and tok_decay is not None else None
    qr = torch.empty(2, T, num_heads * dim, dtype=torch.float32, device=rows_in.device)
    _check(lib.mie_decay_scan(_ptr(rows_in), tag(rows_in), ctypes.c_longlong(rows_in.stride(0)), _ptr(positions), _ptr(row_q_start),
                              _ptr(row_q_len), _ptr(state_slots), _ptr(decay), _ptr(freq), ctypes.c_float(q_scale), ctypes.c_float(k_scale),
                              _ptr(tok_decay), _ptr(k_tok), int(act), int(ones), _ptr(state), _ptr(qr[0]), _ptr(qr[1]), _ptr(scratch),
                              ctypes.c_longlong(chunks), _ptr(cdec), _ptr(out), T, row_q_len.numel(), int(max_q_len), num_heads, dim,
                              vdim, rot, _stream()), "decay_scan")
    return out


def gate_scan(z: torch.Tensor, bias_i, bias_f, cap: float, row_q_start, row_q_len, state_slots, m_state: torch.Tensor, num_heads: int):
    """Exponential gates with a running maximum, token by token per row and head: from z [T, 2H] float32 = [input | forget]
    pre-activations, i = cap tanh((zi + bias_i) / cap), f = logsigmoid(cap tanh((zf + bias_f) / cap)) (``cap`` 0: no cap),
    m_t = max(f + m_{t-1}, i), keep = exp(f + m_{t-1} - m_t), write = exp(i - m_t).  ``m_state`` [slots, H] float32 carries m.
    Returns (keep, write, m), float32 [T, H] each."""
    T = z.shape[0]
    _need(z.dtype == torch.float32 and z.is_contiguous() and z.shape == (T, 2 * num_heads), "gate pre-activations must be float32 [T, 2H]")
    _need(m_state.dtype == torch.float32 and m_state.is_contiguous() and tuple(m_state.shape[1:]) == (num_heads,), "m state must be float32 [slots, H]")
    for b in (bias_i, bias_f):
        if b is not None:
            _need(b.dtype == torch.float32 and b.is_contiguous() and b.numel() == num_heads, "one float32 gate bias per head")
    for t_, n in ((row_q_start, "row_q_start"), (row_q_len, "row_q_len"), (state_slots, "state_slots")):
        _i32(t_, n)
    keep, write, m = (torch.empty(T, num_heads, dtype=torch.float32, device=z.device) for _ in range(3))
    _check(load("retention").mie_gate_scan(_ptr(z), _ptr(bias_i), _ptr(bias_f), ctypes.c_float(cap), _ptr(row_q_start), _ptr(row_q_len),
                                           _ptr(state_slots), _ptr(m_state), _ptr(keep), _ptr(write), _ptr(m), row_q_len.numel(),
                                           num_heads, _stream()), "gate_scan")
    return keep, write, m


def group_norm_gate(o: torch.Tensor, gate, out: torch.Tensor, *, groups: int, size: int, eps: float, weight=None, silu: bool = False,
                    m=None) -> torch.Tensor:
    """o float32 [T, groups * stride] (stride = size, or size + 1 with ``m``): each group of ``size`` entries is divided by
    its root mean square, multiplied by ``weight`` (float32; indexed by the entry's place in the row modulo its length: size
    entries shared by the groups, or groups * size) and by sigmoid (``silu``: silu) of ``gate`` [T, groups * size] (a column
    slice of a wider tensor will do).  With ``m`` [T, groups]: the entry behind a group's outputs is a normalizer n and the
    group is first divided by max(|n|, exp(-m)) + 1e-6.  groups = 1 norms the whole row."""
    T = o.shape[0]
    stride = size + (1 if m is not None else 0)
    _need(o.dtype == torch.float32 and o.is_contiguous() and o.shape == (T, groups * stride), "o must be float32 [T, groups * (size (+ 1))]")
    _need(out.is_contiguous() and out.shape == (T, groups * size), "out must be contiguous [T, groups * size]")
    if gate is not None:
        _need(gate.stride(1) == 1 and gate.shape == out.shape and gate.dtype == out.dtype, "gate must match the output's shape and type")
    if weight is not None:
        _need(weight.dtype == torch.float32 and weight.is_contiguous() and weight.numel() in (size, groups * size), "float32 weight of size or groups * size entries")
    if m is not None:
        _need(m.dtype == torch.float32 and m.is_contiguous() and m.shape == (T, groups), "m must be float32 [T, groups]")
    _check(load("retention").mie_group_norm_gate(_ptr(o), stride, _ptr(m), _ptr(weight), weight.numel() if weight is not None else 0, _ptr(gate),
                                                 tag(out), ctypes.c_longlong(gate.stride(0) if gate is not None else 0), _ptr(out), T, groups,
                                                 size, ctypes.c_float(eps), int(m is not None), int(silu), _stream()), "group_norm_gate")
    return out


def head_rms_gate(o: torch.Tensor, gate: torch.Tensor, out: torch.Tensor, num_heads: int, vdim: int, eps: float) -> torch.Tensor:
    """out[t, h] = o[t, h] / rms(o[t, h]) * silu(gate[t, h]) per head of ``vdim`` entries; ``gate`` may be a column
    slice of a wider tensor."""
    T = o.shape[0]
    _need(o.dtype == torch.float32 and o.is_contiguous() and o.shape == (T, num_heads * vdim), "o must be float32 [T, H * vdim]")
    _need(gate.stride(1) == 1 and gate.shape == o.shape and gate.dtype == out.dtype, "gate must match o's shape and the output's type")
    _need(out.is_contiguous() and out.shape == o.shape, "out must be contiguous [T, H * vdim]")
    lib = load("retention")
    _check(lib.mie_head_rms_gate(_ptr(o), _ptr(gate), tag(gate), ctypes.c_longlong(gate.stride(0)), _ptr(out), T, num_heads, vdim,
                                 ctypes.c_float(eps), _stream()), "head_rms_gate")
    return out


# --------------------------------------------------------------------------- gated linear recurrence

def causal_conv(x: torch.Tensor, ctx_token_row, row_q_start, state_slots, taps, bias, state, u) -> torch.Tensor:
    """u[t] = bias + sum_j taps[:, j] x[t - (K-1) + j] per channel; inputs older than a row's portion come from rows
    1.. of ``state`` [slots, K, C] float32.  ``x`` may be a column slice; taps and bias float32; ``u`` float32 [T, C]."""
    T, C = x.shape
    K = taps.shape[1]
    _need(x.stride(1) == 1 and taps.shape == (C, K) and taps.is_contiguous() and taps.dtype == torch.float32, "conv taps must be float32 [channels, taps]")
    _need(bias is None or (bias.dtype == torch.float32 and bias.numel() == C), "conv bias must be float32, one per channel")
    _need(state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (K, C), "state must be float32 [slots, K, C]")
    _need(u.dtype == torch.float32 and u.is_contiguous() and u.shape == (T, C), "u must be float32 [T, C]")
    for t, n in ((ctx_token_row, "token_row"), (row_q_start, "row_q_start"), (state_slots, "state_slots")):
        _i32(t, n)
    lib = load("linear_recurrence")
    _check(lib.mie_causal_conv(_ptr(x), tag(x), ctypes.c_longlong(x.stride(0)), _ptr(ctx_token_row), _ptr(row_q_start),
                               _ptr(state_slots), _ptr(taps), _ptr(bias), _ptr(state), _ptr(u), T, C, K, _stream()),
           "causal_conv")
    return u


def recurrence_gates(u, w_a, b_a, w_i, b_i, lam, c_exp: float, a_out, b_out) -> None:
    """Block-diagonal gates and the recurrence's coefficients: a = exp(-c_exp * sigmoid(Wa u + ba) * softplus(lam)),
    b = sqrt(1 - a^2) * sigmoid(Wi u + bi) * u, all float32 (weights too)."""
    T, C = u.shape
    B, bw = w_a.shape[0], w_a.shape[1]
    _need(w_a.shape == (B, bw, bw) == w_i.shape and B * bw == C, "gate matrices must be [blocks, C / blocks, C / blocks]")
    ws = (w_a, b_a, w_i, b_i, lam)
    _need(all(w.dtype == torch.float32 and w.is_contiguous() for w in ws), "gate weights must be contiguous float32")
    _need(b_a.numel() == C == b_i.numel() == lam.numel(), "gate biases and lam have one entry per channel")
    for t in (u, a_out, b_out):
        _need(t.dtype == torch.float32 and t.is_contiguous() and t.shape == (T, C), "u, a and b must be float32 [T, C]")
    lib = load("linear_recurrence")
    _check(lib.mie_recurrence_gates(_ptr(u), _ptr(w_a), _ptr(b_a), _ptr(w_i), _ptr(b_i), _ptr(lam), ctypes.c_float(c_exp),
                                    _ptr(a_out), _ptr(b_out), T, C, B, _stream()), "recurrence_gates")


def recurrence_scan(a, b, y, x, row_q_start, row_q_len, state_slots, state, out, segments: int = 1) -> torch.Tensor:
    """s <- a s + b along every row's tokens from ``state`` [slots, K, C] (row 0), out = s * gelu_tanh(y); the last K-1
    inputs ``x`` of the convolution are moved into rows 1.. of the state.  ``x`` and ``y`` may be column slices."""
    T, C = a.shape
    K = state.shape[1]
    _need(x.stride(1) == 1 and y.stride(1) == 1 and x.shape == (T, C) == y.shape and x.dtype == y.dtype == out.dtype, "x, y must be [T, C]")
    _need(out.is_contiguous() and out.shape == (T, C), "out must be contiguous [T, C]")
    for t, n in ((row_q_start, "row_q_start"), (row_q_len, "row_q_len"), (state_slots, "state_slots")):
        _i32(t, n)
    lib = load("linear_recurrence")
    _check(lib.mie_recurrence_scan(_ptr(a), _ptr(b), _ptr(y), tag(y), ctypes.c_longlong(y.stride(0)), _ptr(x),
                                   ctypes.c_longlong(x.stride(0)), _ptr(row_q_start), _ptr(row_q_len), _ptr(state_slots),
                                   _ptr(state), _ptr(out), row_q_len.numel(), C, K, int(segments), _stream()), "recurrence_scan")
    return out


# --------------------------------------------------------------------------- gated activations

def glu_clamped(gate_up: torch.Tensor, out: torch.Tensor, limit: float, slope: float, shift: float,
                interleaved: bool = False) -> torch.Tensor:
    """out = g * sigmoid(slope * g) * (u + shift) with g = min(gate, limit), u = clamp(up, -limit, limit) from the
    fused projection [gate | up] (with ``interleaved``: columns gate_0, up_0, gate_1, ...); ``limit`` <= 0 leaves both
    unclamped."""
    T, two_i = gate_up.shape
    _need(two_i % 2 == 0 and out.shape == (T, two_i // 2) and out.dtype == gate_up.dtype
          and out.is_contiguous() and gate_up.is_contiguous(), "glu shapes/types do not match")
    lib = build.load("activation")
    _check(lib.mie_glu_clamped(_ptr(gate_up), _ptr(out), tag(out), T, two_i // 2, ctypes.c_float(limit), ctypes.c_float(slope),
                               ctypes.c_float(shift), int(interleaved), _stream()), "glu_clamped")
    return out


def sigmoid_gate(attn: torch.Tensor, gate: torch.Tensor, out: torch.Tensor, num_heads: int, vdim: int) -> torch.Tensor:
    """out[t, h * vdim + c] = attn[t, h, c] * sigmoid(gate[t, h * vdim + c]); ``attn`` [T, H, DP >= vdim], ``gate`` may be a
    column slice of a wider tensor."""
    T, DP = attn.shape[0], attn.shape[-1]
    _need(attn.is_contiguous() and attn.shape == (T, num_heads, DP) and DP >= vdim, "attn must be [T, H, DP]")
    _need(gate.stride(1) == 1 and gate.shape == (T, num_heads * vdim) and gate.dtype == attn.dtype == out.dtype, "gate must be [T, H * vdim]")
    _need(out.is_contiguous() and out.shape == (T, num_heads * vdim), "out must be contiguous [T, H * vdim]")
    lib = build.load("activation")
    _check(lib.mie_sigmoid_gate(_ptr(attn), _ptr(gate), ctypes.c_longlong(gate.stride(0)), _ptr(out), tag(out), T, num_heads, vdim, DP,
                                _stream()), "sigmoid_gate")
    return out


def default_scale(head_dim: int) -> float:
    return 1.0 / math.sqrt(head_dim)


# --------------------------------------------------------------------------- hyper-connections, Dynamic Tanh

def _f32(t, name, numel=None):
    _need(t.dtype == torch.float32 and t.is_contiguous() and (numel is None or t.numel() == numel),
          f"{name} must be contiguous float32" + (f" with {numel} entries" if numel is not None else ""))


def hyper_norm(res: torch.Tensor, streams: int, out: torch.Tensor, *, weight=None, bias=None, alpha=None, y=None, mix=None,
               out_coef=None, in_coef=None, rows: torch.Tensor | None = None) -> torch.Tensor:
    """One pass over a stream kept in ``streams`` copies, ``res`` [T, streams * W] float32: with a pending sublayer output
    ``y`` [T, W], x'_r = sum_s mix[s, r] x_s + out_coef[r] y (in place, unless ``rows``); then u = sum_r in_coef[r] x'_r and
    out = tanh(alpha u) weight + bias (u itself without a weight).  A missing mix / out_coef / in_coef is the identity /
    ones / ones.  With ``rows`` output row b comes from stream row rows[b] and ``res`` is not written."""
    T = res.shape[0]
    S = int(streams)
    _need(res.dim() == 2 and res.shape[1] % S == 0, "the streams must be [tokens, streams * width]")
    W = res.shape[1] // S
    _f32(res, "the streams")
    for t, name, n in ((weight, "norm weight", W), (bias, "norm bias", W), (alpha, "alpha", 1), (mix, "mix", S * S),
                       (out_coef, "out coefficients", S), (in_coef, "in coefficients", S)):
        if t is not None:
            _f32(t, name, n)
    _need((weight is None) == (bias is None), "Dynamic Tanh takes a weight and a bias")
    if y is not None:
        _need(y.shape == (T, W) and y.is_contiguous(), "a pending output must be contiguous [tokens, width]")
    num_out = T
    if rows is not None:
        _i32(rows, "rows")
        num_out = rows.numel()
    _need(out.is_contiguous() and out.shape == (num_out, W), "norm output must be contiguous [rows, width]")
    lib = load("hyper_norm")
    _check(lib.mie_hyper_norm(_ptr(res), _ptr(y), tag(y) if y is not None else 0, _ptr(mix), _ptr(out_coef), _ptr(in_coef),
                              _ptr(alpha), _ptr(weight), _ptr(bias), _ptr(out), tag(out), _ptr(rows), num_out, W, S, T,
                              0 if weight is not None else 1, _stream()), "hyper_norm")
    return out


# --------------------------------------------------------------------------- latent attention

def latent_norm_rope(down: torch.Tensor, positions, freq, q_weight, c_weight, eps: float, cq, c, kr, *, q_rank: int, kv_rank: int,
                     rot_dim: int, rot: int) -> None:
    """From rows [dq: q_rank | dkv: kv_rank + rot_dim | ...] of the down-projection: cq = rms(dq) q_weight, c =
    rms(dkv[:kv_rank]) c_weight (activation type), kr = dkv[kv_rank:] rotated by position x ``freq`` over its first ``rot``
    entries, entry 2i with 2i + 1 (float32)."""
    T = down.shape[0]
    _need(down.dim() == 2 and down.stride(1) == 1 and down.shape[1] >= q_rank + kv_rank + rot_dim, "down-projection rows too short")
    _f32(q_weight, "query latent norm weight", q_rank)
    _f32(c_weight, "key/value latent norm weight", kv_rank)
    _f32(freq, "frequencies", rot // 2)
    _i32(positions, "positions")
    _need(cq.shape == (T, q_rank) and c.shape == (T, kv_rank) and cq.dtype == c.dtype == down.dtype and cq.is_contiguous()
          and c.is_contiguous(), "latents must be contiguous [T, rank] in the activation type")
    _need(kr.shape == (T, rot_dim) and kr.dtype == torch.float32 and kr.is_contiguous(), "the shared key part must be float32 [T, rot_dim]")
    lib = load("latent_kv")
    _check(lib.mie_latent_norm_rope(_ptr(down), tag(down), ctypes.c_longlong(down.stride(0)), _ptr(positions), _ptr(freq),
                                    _ptr(q_weight), _ptr(c_weight), ctypes.c_float(eps), _ptr(cq), _ptr(c), _ptr(kr), T, q_rank,
                                    kv_rank, rot_dim, rot, _stream()), "latent_norm_rope")


def latent_assemble(qu: torch.Tensor, kvu: torch.Tensor, kr: torch.Tensor, positions, slots, freq, q_out, k_cache, v_cache, *,
                    num_heads: int, dim: int, rot_dim: int, vdim: int, rot: int, page_size: int, write_cache: bool = True) -> None:
    """q_out[t, h] = [qu[t, h, :dim] | rotate(qu[t, h, dim:]) | 0]; cache k[h] = [kvu.k[h] | kr | 0], v[h] = [kvu.v[h] | 0]
    with kvu rows [k: H x dim | v: H x vdim]; heads padded to the pages' width."""
    T, H, DP = qu.shape[0], num_heads, q_out.shape[-1]
    _need(qu.is_contiguous() and qu.shape == (T, H * (dim + rot_dim)), "qu must be contiguous [T, H * (dim + rot_dim)]")
    _need(kvu.is_contiguous() and kvu.shape == (T, H * (dim + vdim)) and kvu.dtype == qu.dtype, "kvu must be contiguous [T, H * (dim + vdim)]")
    _need(kr.shape == (T, rot_dim) and kr.dtype == torch.float32 and kr.is_contiguous(), "the shared key part must be float32 [T, rot_dim]")
    _need(q_out.is_contiguous() and q_out.shape == (T, H, DP) and q_out.dtype == qu.dtype, "q_out must be [T, H, DP]")
    _need(k_cache.dtype == qu.dtype == v_cache.dtype and k_cache.shape[-1] == DP and k_cache.shape[1] == H and k_cache.is_contiguous(),
          "cache type, heads and width")
    _f32(freq, "frequencies", rot // 2)
    _i32(positions, "positions")
    _i32(slots, "slots")
    lib = load("latent_kv")
    _check(lib.mie_latent_assemble(_ptr(qu), _ptr(kvu), tag(qu), _ptr(kr), _ptr(positions), _ptr(slots), _ptr(freq), _ptr(q_out),
                                   _ptr(k_cache), _ptr(v_cache), T, H, dim, rot_dim, vdim, DP, rot, page_size,
                                   ctypes.c_longlong(k_cache.shape[0]), int(write_cache), _stream()), "latent_assemble")


# --------------------------------------------------------------------------- differential attention

def diff_combine(maps: torch.Tensor, gate, out: torch.Tensor, *, num_heads: int, group: int, vdim: int, lam: float, eps: float,
                 out_scale: float) -> torch.Tensor:
    """out[t, h] = rmsnorm(a1 - lam a2) out_scale sigmoid(gate[t, h]) with a1, a2 heads (2g) group + i and (2g + 1) group + i of
    ``maps`` [T, 2H, DP] for h = g group + i; ``gate`` [T, H] may be a column slice (None: no gate)."""
    T, DP = maps.shape[0], maps.shape[-1]
    _need(maps.is_contiguous() and maps.shape == (T, 2 * num_heads, DP) and DP >= vdim, "maps must be [T, 2H, DP]")
    _need(out.is_contiguous() and out.shape == (T, num_heads * vdim) and maps.dtype in (out.dtype, torch.float32),
          "out must be contiguous [T, H * vdim]; maps in its type or float32")
    if gate is not None:
        _need(gate.stride(1) == 1 and gate.shape == (T, num_heads) and gate.dtype == out.dtype, "gate must be [T, H]")
    lib = load("diff_attention")
    _check(lib.mie_diff_combine(_ptr(maps), tag(maps), _ptr(gate), ctypes.c_longlong(gate.stride(0) if gate is not None else 0), _ptr(out),
                                tag(out), T, num_heads, group, vdim, DP, ctypes.c_float(lam), ctypes.c_float(eps),
                                ctypes.c_float(out_scale), _stream()), "diff_combine")
    return out


# --------------------------------------------------------------------------- gated delta rule

def delta_prepare(proj: torch.Tensor, low: torch.Tensor, taps, conv_state, token_row, row_q_start, state_slots, a_log, dt_bias,
                  qn, kn, vn, beta, decay, kq, *, num_heads: int, num_kv_heads: int, dim: int, vdim: int, unit_eps: float) -> None:
    """From rows [q: G x dim | k: G x dim | v: H x vdim | beta logits: H | ...] of the input projection and float32 rows
    [a: H x dim | ...] of the low-rank one: convolution over time + silu of q, k, v (float32 taps [channels, K], older inputs
    from ``conv_state`` [slots, K - 1, channels]), q and k unit vectors per head (q times dim^-1/2), beta = sigmoid,
    decay = exp(-exp(a_log[h]) softplus(a + dt_bias)), kq = k . q per key head.  All outputs float32."""
    T = proj.shape[0]
    H, G, D, Dv = num_heads, num_kv_heads, dim, vdim
    C = 2 * G * D + H * Dv
    K = taps.shape[1]
    _need(proj.dim() == 2 and proj.stride(1) == 1 and proj.shape[1] >= C + H, "projection rows must hold q, k, v and beta")
    _need(low.dtype == torch.float32 and low.stride(1) == 1 and low.shape[0] == T and low.shape[1] >= H * D, "low-rank rows must be float32")
    _f32(taps, "taps", C * K)
    _need(conv_state.dtype == torch.float32 and conv_state.is_contiguous() and tuple(conv_state.shape[1:]) == (max(K - 1, 0), C),
          "convolution state must be float32 [slots, K - 1, channels]")
    _f32(a_log, "A_log", H)
    _f32(dt_bias, "dt_bias", H * D)
    for t, n in ((qn, G * D), (kn, G * D), (vn, H * Dv), (beta, H), (decay, H * D), (kq, G)):
        _need(t.dtype == torch.float32 and t.is_contiguous() and t.shape == (T, n), "outputs must be float32 [T, n]")
    for t, n in ((token_row, "token_row"), (row_q_start, "row_q_start"), (state_slots, "state_slots")):
        _i32(t, n)
    lib = load("delta_rule")
    _check(lib.mie_delta_prepare(_ptr(proj), tag(proj), ctypes.c_longlong(proj.stride(0)), _ptr(low), ctypes.c_longlong(low.stride(0)),
                                 _ptr(taps), _ptr(conv_state), _ptr(token_row), _ptr(row_q_start), _ptr(state_slots), _ptr(a_log),
                                 _ptr(dt_bias), _ptr(qn), _ptr(kn), _ptr(vn), _ptr(beta), _ptr(decay), _ptr(kq), T, H, G, D, Dv, K,
                                 ctypes.c_float(D ** -0.5), ctypes.c_float(unit_eps), _stream()), "delta_prepare")


def conv_state_update(x: torch.Tensor, row_q_start, row_q_len, state_slots, conv_state) -> None:
    """The last K - 1 inputs ``x`` [T, >= channels] of every row's portion move into its slot of ``conv_state``
    [slots, K - 1, channels] (older rows of the state shift where the portion is shorter)."""
    Km1, C = conv_state.shape[1], conv_state.shape[2]
    _need(x.dim() == 2 and x.stride(1) == 1 and x.shape[1] >= C, "inputs must hold the channels")
    _need(conv_state.dtype == torch.float32 and conv_state.is_contiguous(), "convolution state must be contiguous float32")
    for t, n in ((row_q_start, "row_q_start"), (row_q_len, "row_q_len"), (state_slots, "state_slots")):
        _i32(t, n)
    lib = load("delta_rule")
    _check(lib.mie_conv_state_update(_ptr(x), tag(x), ctypes.c_longlong(x.stride(0)), _ptr(row_q_start), _ptr(row_q_len),
                                     _ptr(state_slots), _ptr(conv_state), row_q_len.numel(), C, Km1 + 1, _stream()), "conv_state_update")


def delta_scan(qn, kn, vn, beta, decay, kq, row_q_start, row_q_len, state_slots, state, out, *, num_heads: int, num_kv_heads: int,
               dim: int, vdim: int) -> torch.Tensor:
    """S <- decay S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q for every new token of every row, from and to
    ``state`` [slots, H, vdim, dim] float32.  ``out`` [T, H * vdim] float32."""
    T = qn.shape[0]
    H, G, D, Dv = num_heads, num_kv_heads, dim, vdim
    _need(state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (H, Dv, D), "state must be float32 [slots, H, vdim, dim]")
    for t, n in ((qn, G * D), (kn, G * D), (vn, H * Dv), (beta, H), (decay, H * D), (kq, G), (out, H * Dv)):
        _need(t.dtype == torch.float32 and t.is_contiguous() and t.shape == (T, n), "operands must be float32 [T, n]")
    for t, n in ((row_q_start, "row_q_start"), (row_q_len, "row_q_len"), (state_slots, "state_slots")):
        _i32(t, n)
    lib = load("delta_rule")
    _check(lib.mie_delta_scan(_ptr(qn), _ptr(kn), _ptr(vn), _ptr(beta), _ptr(decay), _ptr(kq), _ptr(row_q_start), _ptr(row_q_len),
                              _ptr(state_slots), _ptr(state), _ptr(out), row_q_len.numel(), H, G, D, Dv, _stream()), "delta_scan")
    return out


def head_norm_gate(o: torch.Tensor, gate, weight, out: torch.Tensor, num_heads: int, vdim: int, eps: float) -> torch.Tensor:
    """out[t, h] = o[t, h] / rms(o[t, h]) * weight * sigmoid(gate[t, h]) per head of ``vdim`` entries; ``gate`` float32
    [T, H * vdim], may be a column slice; ``weight`` float32 [vdim]; either may be None."""
    T = o.shape[0]
    _need(o.dtype == torch.float32 and o.is_contiguous() and o.shape == (T, num_heads * vdim), "o must be float32 [T, H * vdim]")
    if gate is not None:
        _need(gate.dtype == torch.float32 and gate.stride(1) == 1 and gate.shape == o.shape, "gate must be float32 [T, H * vdim]")
    if weight is not None:
        _f32(weight, "head norm weight", vdim)
    _need(out.is_contiguous() and out.shape == o.shape, "out must be contiguous [T, H * vdim]")
    lib = load("delta_rule")
    _check(lib.mie_head_norm_gate(_ptr(o), _ptr(gate), ctypes.c_longlong(gate.stride(0) if gate is not None else 0), _ptr(weight),
                                  _ptr(out), tag(out), T, num_heads, vdim, ctypes.c_float(eps), _stream()), "head_norm_gate")
    return out


# --------------------------------------------------------------------------- routed experts

# "clamped_in" (gated experts only): the expert runs on the token scaled by its weight; with g = min(w gate, limit), u = clamp(w up,
# -limit, limit) the hidden value is g sigmoid(1.702 g) (u + 1), and nothing multiplies the output
EXPERT_ACTIVATIONS = {"relu2": 0, "silu": 1, "gelu_tanh": 2, "clamped_in": 3}


class RouteRule:
    """How a router turns its outputs into a choice.  ``score`` "top_softmax": the ``top`` largest logits, weights = softmax
    over those.  ``score`` "softmax": scores = softmax over all outputs; the choice is by score + ``correction`` (float32
    [outputs], optional), limited to the ``keep`` best of ``groups`` equal groups of neighbouring outputs (a group's value is
    its largest choice score); weights = the chosen scores, not renormalized.  Outputs from ``real`` on (None: there are
    none) are identity experts; the sum of their chosen weights is returned per token."""

    def __init__(self, score: str = "top_softmax", correction=None, groups: int = 1, keep: int = 1, real: int | None = None):
        _need(score in ("top_softmax", "softmax", "sigmoid"), f"router score {score!r}; one of top_softmax, softmax, sigmoid")
        if correction is not None:
            _f32(correction, "router correction")
        # "sigmoid": the ``top`` largest logits, each chosen output's weight the sigmoid of its own logit (not renormalized)
        self.mode = {"top_softmax": 0, "softmax": 1, "sigmoid": 2}[score]
        self.correction, self.groups, self.keep, self.real = correction, int(groups), int(keep), real

    def args(self, outputs: int, tokens: int, device):
        """(ctypes arguments behind ``top``, the per-token rest weights or None)."""
        _need(self.correction is None or self.correction.numel() == outputs, "one correction per router output")
        real = outputs if self.real is None else int(self.real)
        rest = torch.empty(tokens, dtype=torch.float32, device=device) if real < outputs else None
        return (self.mode, _ptr(self.correction), self.groups, self.keep, real, _ptr(rest)), rest


_PLAIN_RULE = RouteRule()


def moe_route(logits: torch.Tensor, top: int, rule: RouteRule | None = None):
    """The choice of each row of float32 ``logits`` [T, outputs] under ``rule`` (default: the ``top`` largest, ties: lower index
    first, softmax over them): (ids int32 [T, top], weights float32 [T, top]), and with a rule that has identity experts a
    third value, float32 [T]: the sum of their weights."""
    T, E = logits.shape
    _f32(logits, "router logits")
    ids = torch.empty(T, top, dtype=torch.int32, device=logits.device)
    wts = torch.empty(T, top, dtype=torch.float32, device=logits.device)
    extra, rest = (rule or _PLAIN_RULE).args(E, T, logits.device)
    lib = load("moe")
    _check(lib.mie_moe_route(_ptr(logits), _ptr(ids), _ptr(wts), T, E, int(top), *extra, _stream()), "moe_route")
    return (ids, wts) if rule is None or rest is None else (ids, wts, rest)


def moe_router(x: torch.Tensor, w_router: torch.Tensor, top: int, logits: torch.Tensor | None = None, rule: RouteRule | None = None):
    """Router logits z = x w_router^T in float32 (``w_router`` float32 [E, h]; ``x`` widened) and the choice of ``moe_route`` in
    one kernel: (ids int32 [T, top], weights float32 [T, top]) (and the identity experts' weights, as ``moe_route``);
    ``logits`` float32 [T, E], if given, receives z."""
    T, h = x.shape
    E = w_router.shape[0]
    _need(x.is_contiguous() and w_router.dtype == torch.float32 and w_router.is_contiguous() and w_router.shape == (E, h),
          "router: contiguous x [T, h] and float32 weights [E, h]")
    if logits is not None:
        _need(logits.dtype == torch.float32 and logits.is_contiguous() and logits.shape == (T, E), "logits must be float32 [T, E]")
    ids = torch.empty(T, top, dtype=torch.int32, device=x.device)
    wts = torch.empty(T, top, dtype=torch.float32, device=x.device)
    extra, rest = (rule or _PLAIN_RULE).args(E, T, x.device)
    _check(load("moe").mie_moe_router(_ptr(x), tag(x), _ptr(w_router), _ptr(ids), _ptr(wts), _ptr(logits), T, h, E, int(top), *extra,
                                      _stream()), "moe_router")
    return (ids, wts) if rule is None or rest is None else (ids, wts, rest)


def moe_dense_act(up: torch.Tensor, ids, wts, act: torch.Tensor, num_experts: int, activation: str) -> torch.Tensor:
    """act[t, e, :] = weight(t, e) f(up[t, e, :]) for the experts token t chose, 0 for the others (``up`` [T, E * F])."""
    T = up.shape[0]
    _need(up.is_contiguous() and act.is_contiguous() and act.shape == up.shape and act.dtype == up.dtype and up.shape[1] % num_experts == 0,
          "up and act must be contiguous [T, E * F]")
    lib = load("moe")
    _check(lib.mie_moe_dense_act(_ptr(up), _ptr(ids), _ptr(wts), _ptr(act), tag(up), T, num_experts, up.shape[1] // num_experts,
                                 ids.shape[1], EXPERT_ACTIVATIONS[activation], _stream()), "moe_dense_act")
    return act


def moe_pairs_fit(hidden: int, expert_size: int, top: int) -> bool:
    """Whether ``moe_pairs`` takes these sizes (rows of whole 16-byte pieces; a token's hidden rows in shared memory)."""
    return bool(load("moe").mie_moe_pairs_fit(int(hidden), int(expert_size), int(top)))


def moe_pairs(x: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor, ids, wts, out: torch.Tensor, num_experts: int,
              activation: str, gated: bool = False, limit: float = 0.0) -> torch.Tensor:
    """The routed experts for a handful of tokens: every (token, chosen expert) pair reads its expert's rows of the
    stacked matrices ``w_up`` [E * F, h] and ``w_down`` [h, E * F] and nothing else.  out [T, h] float32 = sum over the
    token's pairs of weight * W_down[e] f(W_up[e] x).  ``gated``: ``w_up`` is [E * 2F, h], per expert F gate rows then F up rows,
    and the hidden row is f(gate x) * (up x).  A pair whose id is ``num_experts`` or more (an identity expert) adds nothing."""
    T, h = x.shape
    top = ids.shape[1]
    EF = w_down.shape[1]
    F = EF // num_experts
    _need(x.is_contiguous() and w_up.is_contiguous() and w_down.is_contiguous() and w_up.shape == ((2 if gated else 1) * EF, h)
          and w_down.shape == (h, EF) and w_up.dtype == w_down.dtype and F * num_experts == EF,
          "stacked expert matrices must be contiguous [E * F, h] ([E * 2F, h] gated) and [h, E * F]")
    _need(out.dtype == torch.float32 and out.is_contiguous() and out.shape == (T, h), "out must be float32 [T, h]")
    _need(ids.dtype == torch.int32 and ids.is_contiguous() and wts.dtype == torch.float32 and wts.is_contiguous() and wts.shape == ids.shape,
          "ids int32 and weights float32 [T, top]")
    hid = torch.empty(T * top, F, dtype=x.dtype, device=x.device)
    lib = load("moe")
    _check(lib.mie_moe_pairs(_ptr(x), tag(x), _ptr(w_up), _ptr(w_down), tag(w_up), _ptr(ids), _ptr(wts), _ptr(hid), _ptr(out), T, h,
                             int(num_experts), F, top, EXPERT_ACTIVATIONS[activation], int(gated), ctypes.c_float(limit), _stream()), "moe_pairs")
    return out


def moe_sort(ids: torch.Tensor, wts: torch.Tensor, num_experts: int):
    """Places for the (token, expert) pairs of ``ids`` [T, top] among rows sorted by expert: (ends int32 [E], one past each
    expert's last row; place int32 [T * top], the row of every pair; row_weight float32 [T * top], the pairs' weights by row)."""
    pairs = ids.numel()
    _need(ids.dtype == torch.int32 and ids.is_contiguous() and wts.dtype == torch.float32 and wts.is_contiguous() and wts.shape == ids.shape,
          "ids int32 and weights float32 [T, top]")
    ends = torch.empty(num_experts, dtype=torch.int32, device=ids.device)
    place = torch.empty(pairs, dtype=torch.int32, device=ids.device)
    row_weight = torch.empty(pairs, dtype=torch.float32, device=ids.device)
    _check(load("moe").mie_moe_sort(_ptr(ids), _ptr(wts), _ptr(ends), _ptr(place), _ptr(row_weight), pairs, int(num_experts), _stream()),
           "moe_sort")
    return ends, place, row_weight


def moe_gather(x: torch.Tensor, place: torch.Tensor, top: int) -> torch.Tensor:
    """rows[place[p]] = x[p // top]: the tokens' inputs where their pairs' rows are."""
    T, h = x.shape
    _need(x.is_contiguous() and place.numel() == T * top, "x must be contiguous [T, h] with top places a token")
    rows = torch.empty(T * top, h, dtype=x.dtype, device=x.device)
    _check(load("moe").mie_moe_gather(_ptr(x), _ptr(place), _ptr(rows), tag(x), T * top, h, int(top), _stream()), "moe_gather")
    return rows


def moe_act_rows(up: torch.Tensor, row_weight: torch.Tensor, activation: str) -> torch.Tensor:
    """up[r] <- row_weight[r] f(up[r]) in place."""
    _need(up.is_contiguous() and row_weight.numel() == up.shape[0] and row_weight.dtype == torch.float32, "one float32 weight a row")
    _check(load("moe").mie_moe_act_rows(_ptr(up), _ptr(row_weight), tag(up), up.shape[0], up.shape[1], EXPERT_ACTIVATIONS[activation],
                                        _stream()), "moe_act_rows")
    return up


def moe_combine(rows: torch.Tensor, place: torch.Tensor, top: int, out: torch.Tensor, ids=None, real: int = 0) -> torch.Tensor:
    """out[t] = sum over k of rows[place[t * top + k]], float32; with ``ids`` [T, top], only the pairs whose id is below ``real``."""
    T, h = out.shape
    _need(rows.is_contiguous() and rows.shape == (T * top, h) and out.dtype == torch.float32 and out.is_contiguous(), "rows [T * top, h], out float32 [T, h]")
    _check(load("moe").mie_moe_combine(_ptr(rows), _ptr(place), _ptr(out), tag(rows), T, h, int(top), _ptr(ids), int(real), _stream()),
           "moe_combine")
    return out


def moe_glu(gu: torch.Tensor, num_experts: int, activation: str, *, ids=None, wts=None, row_weight=None, limit: float = 0.0) -> torch.Tensor:
    """The activation of gated experts.  With ``ids``/``wts`` [T, top] and ``gu`` [T, E * 2F] (per expert F gate then F up
    entries): act [T, E * F] = weight f(gate) up for the experts a token chose, 0 for the others.  With ``row_weight`` [R] and
    ``gu`` [R, 2F]: hid [R, F] = row_weight f(gate) up, row by row."""
    R = gu.shape[0]
    per_row = row_weight is not None
    E = 1 if per_row else int(num_experts)
    _need(gu.is_contiguous() and gu.shape[1] % (2 * E) == 0, "gate|up rows must be contiguous [rows, E * 2F]")
    F = gu.shape[1] // (2 * E)
    w = row_weight if per_row else wts
    _need(w.dtype == torch.float32 and w.is_contiguous() and (w.numel() == R if per_row else (ids is not None and w.shape == ids.shape and ids.shape[0] == R)),
          "float32 weights: one a row, or [T, top] beside int32 ids")
    act = torch.empty(R, E * F, dtype=gu.dtype, device=gu.device)
    _check(load("moe").mie_moe_glu(_ptr(gu), _ptr(ids), _ptr(w), _ptr(act), tag(gu), R, E, F, 0 if per_row else ids.shape[1],
                                   EXPERT_ACTIVATIONS[activation], int(per_row), ctypes.c_float(limit), _stream()), "moe_glu")
    return act


def grouped_linear(rows: torch.Tensor, b: torch.Tensor, ends: torch.Tensor) -> torch.Tensor:
    """The product of row ranges with a matrix each: rows [R, K] bfloat16 sorted by group, b [groups, K, N] (any strides
    with one unit stride per matrix), ends int32 [groups] one past each group's last row -> [R, N] bfloat16.  The library's
    grouped product (float32 accumulation), as the plain products of prompt-sized steps are the library's."""
    _need(rows.is_cuda and rows.dtype == torch.bfloat16 == b.dtype and rows.is_contiguous() and ends.dtype == torch.int32,
          "grouped product: bfloat16 rows and matrices on the device, int32 ends")
    return torch._grouped_mm(rows, b, offs=ends)          # (not counted in ``launches``: that counts this package's own kernels)
