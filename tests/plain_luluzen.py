"""Plain, slow Luluzen: the oracle that the tests of this design compare with.

Whole sequences, no cache, no batching, on the CPU, one function per mechanism, written from the design's
equations and sharing no code with the package.  ``cfg`` is the parsed config.json, ``W`` a
``{tensor name: tensor}`` dict in the precision to compute in (float32 or float64).

The design in this file's notation (t: token index = position, x_t: residual stream):

  embedding          x_t = E[token_t]; e = x as the embedding leaves it
  order of layers    layers lo .. hi-1 run ``times`` times with the same weights; in front of every pass p,
                     x <- W_in [x; e] + step[p]; the other layers run once, in their place
  layer              x <- x + mixer(ln(x; w1));  x <- x + ff(ln(x; w2));  ln(v; w) = (v - mean) / sqrt(var + eps) w
  lightning          q, k, v = silu of their projections; per head S_t = d_h S_{t-1} + k_t v_t^T, o_t = S_t^T q_t;
                     all heads' o together / rms, times w, times sigmoid(Wg h), then Wo
  biased attention   q, k, v with biases; q, k RMS-normed per head with one weight for all heads; q_t times
                     1 + c ln(floor((t + 1) / n) + 1); score = q.k scale + rel[bucket(t - j), head]; causal softmax
  delta rule         q, k, v through a short causal convolution and silu; q, k unit vectors (q / sqrt(dim));
                     S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q; o / rms per head, w, sigmoid gate
  windowed attention q, k RMS-normed over the whole projection; pairs (2i, 2i + 1) of a head's first n dims turn by
                     t base^(-2i/n); score = c tanh(q.k scale / c); keys j in (t - w, t]; the softmax's denominator
                     also has exp(sink_head); heads times sigmoid(Wg h); then Wo
  matrix memory      log gates i, f capped by tanh; m_t = max(f + m_{t-1}, i); S_t = e^(f + m_{t-1} - m_t) S + e^(i - m_t) k v^T,
                     n_t likewise with k; o = S^T q / (max(|n.q|, e^-m) + 1e-6); per-head rms, w, sigmoid gate, Wo
  feed-forward       dense: Wd (gelu_tanh(Wg h) (Wu h));  experts: scores sigmoid(router h), the ``top`` largest,
                     sum over those of expert(s h), expert(z) = Wd (g sigmoid(1.702 g) (u + 1)), g = min(Wg z, L),
                     u = clip(Wu z, -L, L)
  head               logits = c tanh(E ln(x; w_final) / c)
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def rms_scale(v: torch.Tensor, eps: float) -> torch.Tensor:
    return v / torch.sqrt(v.pow(2).mean(-1, keepdim=True) + eps)


def layer_norm(v: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    mu = v.mean(-1, keepdim=True)
    var = (v - mu).pow(2).mean(-1, keepdim=True)
    return (v - mu) / torch.sqrt(var + eps) * w


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


# --------------------------------------------------------------------------- feed-forward

def dense_ff(h, W, p):
    return (gelu_tanh(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def expert(z, W, p, limit):
    g = torch.clamp(z @ W[p + "gate"].T, max=limit)
    u = torch.clamp(z @ W[p + "up"].T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ W[p + "down"].T


def router_choice(h, W, p, top):
    """(chosen experts [T, top], their scores) -- scores are sigmoids of the logits, taken as they are."""
    s = torch.sigmoid(h @ W[p + "router"].T)
    val, idx = torch.topk(s, top, dim=-1)
    return idx, val


MARGINS = None      # a list, while a caller wants them: per call of a router, per token the gap between the last chosen score and the next


def routed_ff(h, W, p, mlp):
    idx, val = router_choice(h, W, p, int(mlp["router"]["top"]))
    if MARGINS is not None and int(mlp["router"]["top"]) < int(mlp["router"]["experts"]):
        s = torch.sigmoid(h @ W[p + "router"].T).sort(-1, descending=True).values
        k = int(mlp["router"]["top"])
        MARGINS.append(s[:, k - 1] - s[:, k])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, s in zip(idx[t].tolist(), val[t]):
            out[t] += expert(s * h[t], W, f"{p}e{e}.", float(mlp["expert"]["limit"]))
    return out


def feed_forward(h, W, p, mlp):
    return dense_ff(h, W, p) if mlp["kind"] == "dense" else routed_ff(h, W, p, mlp)


# --------------------------------------------------------------------------- lightning

def decayed_outer_scan(q, k, v, decay):
    """q, k [T, H, D], v [T, H, Dv], decay [H]: S_t = decay S_{t-1} + k_t v_t^T, o_t = S_t^T q_t -> [T, H, Dv]."""
    T, H, D = q.shape
    S = torch.zeros(H, D, v.shape[-1], dtype=q.dtype)
    out = []
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out.append(torch.einsum("hdv,hd->hv", S, q[t]))
    return torch.stack(out)


def lightning(h, W, p, m, eps):
    T, H, D, Dv = h.shape[0], int(m["heads"]), int(m["dim"]), int(m["vdim"])
    q = F.silu(h @ W[p + "q"].T).reshape(T, H, D)
    k = F.silu(h @ W[p + "k"].T).reshape(T, H, D)
    v = F.silu(h @ W[p + "v"].T).reshape(T, H, Dv)
    o = decayed_outer_scan(q, k, v, torch.tensor(m["decay"], dtype=h.dtype)).reshape(T, H * Dv)
    o = rms_scale(o, eps) * W[p + "norm"] * torch.sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


# --------------------------------------------------------------------------- softmax attention, both kinds

def distance_bucket(n: int, rows: int, far: float) -> int:
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def softmax_attention(q, k, v, scale, *, window=None, softcap=None, sink=None, bias=None):
    """q [T, H, D], k [T, G, D], v [T, G, Dv]; ``bias`` [T, T, H] added to the scaled scores (row i, key j);
    ``sink`` [H] one more term exp(sink) in the denominator.  Returns [T, H, Dv]."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * scale
        if softcap is not None:
            s = softcap * torch.tanh(s / softcap)
        if bias is not None:
            s = s + bias[:, :, hd]
        i = torch.arange(T)[:, None]
        j = torch.arange(T)[None, :]
        seen = j <= i
        if window is not None:
            seen = seen & (i - j < window)
        s = s.masked_fill(~seen, float("-inf"))
        top = s.max(-1, keepdim=True).values
        if sink is not None:
            top = torch.maximum(top, sink[hd].reshape(1, 1).to(s.dtype))
        e = torch.exp(s - top)
        den = e.sum(-1, keepdim=True)
        if sink is not None:
            den = den + torch.exp(sink[hd].to(s.dtype) - top)
        out[:, hd] = (e / den) @ v[:, g]
    return out


def biased_attention(h, W, p, m, eps):
    T, H, G, D, Dv = h.shape[0], int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = (h @ W[p + "q"].T + W[p + "q.b"]).reshape(T, H, D)
    k = (h @ W[p + "k"].T + W[p + "k.b"]).reshape(T, G, D)
    v = (h @ W[p + "v"].T + W[p + "v.b"]).reshape(T, G, Dv)
    q = rms_scale(q, eps) * W[p + "q.norm"]
    k = rms_scale(k, eps) * W[p + "k.norm"]
    if m.get("q_temp"):
        pos = torch.arange(T)
        temp = 1.0 + float(m["q_temp"]["coef"]) * torch.log(torch.floor((pos + 1) / int(m["q_temp"]["every"])).to(h.dtype) + 1.0)
        q = q * temp[:, None, None]
    rel = W[p + "rel"]
    rows = rel.shape[0]
    bias = torch.zeros(T, T, H, dtype=h.dtype)
    for i in range(T):
        for j in range(i + 1):
            bias[i, j] = rel[distance_bucket(i - j, rows, float(m["bias_max"]))]
    o = softmax_attention(q, k, v, float(m["scale"]), bias=bias)
    return o.reshape(T, H * Dv) @ W[p + "o"].T


def turn_pairs(x, rot):
    """x [T, heads, dim]: entries 2i and 2i + 1 of a head's first ``dims`` entries turn by t base^(-2i/dims)."""
    n = int(rot["dims"])
    if n == 0:
        return x
    T = x.shape[0]
    f = torch.tensor([float(rot["base"]) ** (-2.0 * i / n) for i in range(n // 2)], dtype=torch.float64)
    ang = (torch.arange(T, dtype=torch.float64)[:, None] * f[None, :]).to(x.dtype)
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., 0:n:2], x[..., 1:n:2]
    out = x.clone()
    out[..., 0:n:2] = a * c - b * s
    out[..., 1:n:2] = b * c + a * s
    return out


def windowed_attention(h, W, p, m, eps):
    T, H, G, D, Dv = h.shape[0], int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = rms_scale(h @ W[p + "q"].T, eps) * W[p + "q.norm"]
    k = rms_scale(h @ W[p + "k"].T, eps) * W[p + "k.norm"]
    v = (h @ W[p + "v"].T).reshape(T, G, Dv)
    q, k = q.reshape(T, H, D), k.reshape(T, G, D)
    if m.get("rot"):
        q, k = turn_pairs(q, m["rot"]), turn_pairs(k, m["rot"])
    o = softmax_attention(q, k, v, float(m["scale"]), window=int(m["mask"]["size"]) if m.get("mask") else None,
                          softcap=float(m["softcap"]) if m.get("softcap") else None, sink=W.get(p + "sink"))
    o = o.reshape(T, H * Dv) * torch.sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


# --------------------------------------------------------------------------- gated delta rule

def short_conv(x, taps):
    """x [T, C], taps [C, K] (last column the current token's): y_t = sum_j taps[:, j] x_{t - (K-1) + j}, zeros before 0."""
    T, K = x.shape[0], taps.shape[1]
    padded = torch.cat([torch.zeros(K - 1, x.shape[1], dtype=x.dtype), x], 0)
    return sum(padded[j:j + T] * taps[:, j] for j in range(K))


def gated_delta(h, W, p, m, eps):
    T, H, G, D, Dv = h.shape[0], int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = F.silu(short_conv(h @ W[p + "q"].T, W[p + "q.conv"])).reshape(T, G, D)
    k = F.silu(short_conv(h @ W[p + "k"].T, W[p + "k.conv"])).reshape(T, G, D)
    v = F.silu(short_conv(h @ W[p + "v"].T, W[p + "v.conv"])).reshape(T, H, Dv)
    q = q / torch.sqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ W[p + "b"].T)                                               # [T, H]
    a = (h @ W[p + "a1"].T) @ W[p + "a2"].T + W[p + "dt_bias"]
    g = torch.exp(-torch.exp(W[p + "A_log"])[None, :, None] * F.softplus(a).reshape(T, H, D))      # [T, H, D]
    S = torch.zeros(H, D, Dv, dtype=h.dtype)
    out = []
    for t in range(T):
        for hd in range(H):
            kv = hd // (H // G)
            S[hd] = g[t, hd][:, None] * S[hd]
            u = beta[t, hd] * (v[t, hd] - S[hd].T @ k[t, kv])
            S[hd] = S[hd] + k[t, kv][:, None] * u[None, :]
        out.append(torch.stack([S[hd].T @ q[t, hd // (H // G)] for hd in range(H)]))
    o = torch.stack(out)                                                                  # [T, H, Dv]
    gate = torch.sigmoid((h @ W[p + "g1"].T) @ W[p + "g2"].T).reshape(T, H, Dv)
    o = rms_scale(o, eps) * W[p + "norm"] * gate
    return o.reshape(T, H * Dv) @ W[p + "o"].T


# --------------------------------------------------------------------------- matrix memory

def matrix_memory(h, W, p, m, eps):
    T, H, D, Dv, cap = h.shape[0], int(m["heads"]), int(m["dim"]), int(m["vdim"]), float(m["gate_cap"])
    q = (h @ W[p + "q"].T).reshape(T, H, D) * D ** -0.5
    k = (h @ W[p + "k"].T).reshape(T, H, D)
    v = (h @ W[p + "v"].T).reshape(T, H, Dv)
    gi = cap * torch.tanh((h @ W[p + "i"].T + W[p + "i.b"]) / cap)                       # [T, H]
    gf = F.logsigmoid(cap * torch.tanh((h @ W[p + "f"].T + W[p + "f.b"]) / cap))
    S = torch.zeros(H, D, Dv, dtype=h.dtype)
    n = torch.zeros(H, D, dtype=h.dtype)
    mx = torch.zeros(H, dtype=h.dtype)
    out = []
    for t in range(T):
        new = torch.maximum(gf[t] + mx, gi[t])
        keep, write = torch.exp(gf[t] + mx - new), torch.exp(gi[t] - new)
        S = keep[:, None, None] * S + write[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = keep[:, None] * n + write[:, None] * k[t]
        mx = new
        num = torch.einsum("hdv,hd->hv", S, q[t])
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-mx)) + 1e-6
        out.append(num / den[:, None])
    o = rms_scale(torch.stack(out), eps).reshape(T, H * Dv)
    o = o * W[p + "norm"] * torch.sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


# --------------------------------------------------------------------------- layers and the model

def mixer(h, W, p, layer, eps):
    kind, m = layer["type"], layer["mixer"]
    if kind == "lightning":
        return lightning(h, W, p, m, eps)
    if kind == "parallel":
        return (float(m["left_scale"]) * biased_attention(h, W, p + "left.", m["left"], eps)
                + float(m["right_scale"]) * gated_delta(h, W, p + "right.", m["right"], eps))
    if kind == "parallel_2":
        return (float(m["left_scale"]) * windowed_attention(h, W, p + "left.", m["left"], eps)
                + float(m["right_scale"]) * matrix_memory(h, W, p + "right.", m["right"], eps))
    raise ValueError(kind)


def layer_forward(x, W, i, layer, eps):
    p = f"l{i}."
    x = x + mixer(layer_norm(x, W[p + "norm1"], eps), W, p + "mix.", layer, eps)
    if layer.get("mlp") is not None:
        x = x + feed_forward(layer_norm(x, W[p + "norm2"], eps), W, p + "mlp.", layer["mlp"])
    return x


def run_order(cfg):
    """[(layer index, pass number or None)]: the pass number stands in front of a pass's first layer."""
    n, loop = len(cfg["layers"]), cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    lo, hi, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    order = [(i, None) for i in range(lo)]
    for t in range(times):
        order += [(i, t if i == lo else None) for i in range(lo, hi)]
    return order + [(i, None) for i in range(hi, n)]


def choice_margins(cfg, W, tokens):
    """Per token, the smallest gap over all its routers between the last chosen expert's score and the best one left out
    (infinity where no router chooses): how close the token came to another choice of experts."""
    global MARGINS
    MARGINS = []
    try:
        forward(cfg, W, tokens)
        out = torch.full((len(tokens),), float("inf"))
        for m in MARGINS:
            out = torch.minimum(out, m.float())
        return out
    finally:
        MARGINS = None


def forward(cfg, W, tokens, trace=None):
    """Logits [T, vocab] of a whole sequence; ``trace`` (a list) receives the stream after every layer run."""
    eps = float(cfg["norm"]["eps"])
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    e = x
    for i, t in run_order(cfg):
        if t is not None:
            x = torch.cat([x, e], -1) @ W["loop.in"].T + W["loop.step"][t]
        x = layer_forward(x, W, i, cfg["layers"][i], eps)
        if trace is not None:
            trace.append(x.clone())
    z = layer_norm(x, W["final.norm"], eps) @ W["embed"].T
    cap = cfg.get("logit_softcap")
    return float(cap) * torch.tanh(z / float(cap)) if cap else z
