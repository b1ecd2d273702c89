"""A plain, slow implementation of the Serotar design in float32 on the CPU: one function per mechanism, whole
sequences at once, no cache.  It shares no code with the package; tests compare the package with it.

Notation: T tokens, W model width, H heads, D key size, Dv value size, C latent size, E routed experts, I identity
experts.  Weights are given as a dict of float32 tensors by their checkpoint names; linear weights are [out, in]."""
from __future__ import annotations

import math

import torch


def lin(x, w):
    return x @ w.t()


def rms(x, eps):
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))


def softplus(z):
    return torch.nn.functional.softplus(z.double()).float()


def sub(p, prefix):
    """The tensors under ``prefix``, with the prefix taken off."""
    return {k[len(prefix):]: v for k, v in p.items() if k.startswith(prefix)}


# --------------------------------------------------------------------------- embedding

def bigram_rows(tokens, buckets, mul_prev, mul_cur):
    """Row of the pair table for every token: a hash of (previous, current); the first token takes the last row."""
    rows = [buckets]
    for a, b in zip(tokens[:-1], tokens[1:]):
        rows.append((a * mul_prev + b * mul_cur) % buckets)
    return torch.tensor(rows, dtype=torch.long)


def embedding(tokens, p, cfg):
    e = cfg["embedding"]
    x = p["embed"][torch.tensor(tokens)] * e["scale"]
    b = e.get("bigram")
    if b:
        x = x + p["bigram"][bigram_rows(tokens, b["buckets"], b["mul_prev"], b["mul_cur"])]
    return x


# --------------------------------------------------------------------------- mixer

def latent_attention(h, p, m, eps):
    """Causal softmax attention whose queries and keys/values come from low-rank latents; no positions."""
    T = h.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    cq = rms(lin(h, p["dq"]), eps) * p["dq.norm"]
    q = lin(cq, p["uq"]).view(T, H, D)
    c = rms(lin(h, p["dkv"]), eps) * p["dkv.norm"]
    k = lin(c, p["uk"]).view(T, H, D)
    v = lin(c, p["uv"]).view(T, H, Dv)
    s = torch.einsum("thd,uhd->htu", q, k) * m["scale"]
    mask = torch.ones(T, T, dtype=torch.bool).tril()
    w = torch.softmax(s.masked_fill(~mask, float("-inf")), -1)
    o = torch.einsum("htu,uhe->the", w, v).reshape(T, H * Dv)
    return lin(o, p["o"])


# --------------------------------------------------------------------------- feed-forward

def xielu(z, act):
    """Two learned numbers: a quadratic arm for z > 0 and an exponential arm for z <= 0, both with slope 1/2 at 0."""
    ap = softplus(act[0])
    an = 0.5 + softplus(act[1])
    return torch.where(z > 0, ap * z * z + 0.5 * z, an * (torch.expm1(torch.clamp(z, max=0.0)) - z) + 0.5 * z)


def dense_ff(h, p):
    return lin(xielu(lin(h, p["up"]), p["act"]), p["down"])


def gated_expert(h, p):
    g = lin(h, p["gate"])
    return lin(g * torch.sigmoid(g) * lin(h, p["up"]), p["down"])


def route(h, p, r):
    """For every token the chosen router outputs and their weights: softmax over all outputs, a correction added for
    the choice only, choice limited to the best groups, weights not renormalized.  Returns (ids [T, top], w [T, top])."""
    n = r["experts"] + r.get("identity", 0)
    s = torch.softmax(lin(h, p["router"]), -1)
    choice = s + p["correction"] if "correction" in p else s.clone()
    groups = r.get("groups")
    if groups:
        per = n // groups["count"]
        best = choice.view(-1, groups["count"], per).max(-1).values
        keep = best.topk(groups["keep"], -1).indices
        allowed = torch.zeros_like(best, dtype=torch.bool).scatter_(1, keep, True).repeat_interleave(per, 1)
        choice = choice.masked_fill(~allowed, float("-inf"))
    ids = choice.topk(r["top"], -1).indices
    return ids, s.gather(1, ids)


def moe_ff(h, p, mlp):
    r = mlp["router"]
    E = r["experts"]
    ids, w = route(h, p, r)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(ids[t].tolist(), w[t]):
            y = gated_expert(h[t:t + 1], sub(p, f"e{e}."))[0] if e < E else h[t]        # the last outputs are identity experts
            out[t] += a * y
    if mlp.get("shared"):
        out = out + gated_expert(h, sub(p, "shared."))
    return out


def feed_forward(h, p, mlp):
    return dense_ff(h, p) if mlp["kind"] == "dense" else moe_ff(h, p, mlp)


# --------------------------------------------------------------------------- a layer, the model

def scalar_norm(y, g, eps):
    return rms(y, eps) * g


def token_side(x, tokens, p, i, dim, side_table, eps):
    """A per-layer input that depends on the token alone, gated by the stream and RMS-normed before it is added."""
    e = side_table[torch.tensor(tokens)][:, i * dim:(i + 1) * dim]
    y = lin(gelu_tanh(lin(x, p["gate"])) * e, p["proj"])
    return rms(y, eps) * p["norm"]


def layer(x, tokens, p, i, cfg, side_table):
    L = cfg["layers"][i]
    eps = cfg["norm"]["eps"]
    x = x + scalar_norm(latent_attention(x, sub(p, "mix."), L["mixer"], eps), p["norm1"], eps) * p["ls1"]
    if L.get("mlp"):
        x = x + scalar_norm(feed_forward(x, sub(p, "mlp."), L["mlp"]), p["norm2"], eps) * p["ls2"]
    if cfg.get("token_side"):
        x = x + token_side(x, tokens, sub(p, "side."), i, cfg["token_side"]["dim"], side_table, eps)
    return x


def forward(tokens, p, cfg, trace=None):
    """Logits [T, vocab] of one whole sequence.  ``trace``: a list that receives the stream after every layer."""
    eps = cfg["norm"]["eps"]
    x = embedding(tokens, p, cfg)
    outs = [x]
    for i in range(len(cfg["layers"])):
        lp = sub(p, f"l{i}.")
        outs.append(layer(x, tokens, lp, i, cfg, p.get("side.embed")))
        x = sum(lp["dwa"][j] * outs[j] for j in range(i + 2)) if "dwa" in lp else outs[-1]
        if trace is not None:
            trace.append(x)
    return lin(scalar_norm(x, p["final.norm"], eps), p["head"])
