"""The mechanisms of the Serotar design one by one, built through the part registry with sizes of their own, against the
plain functions of ``plain_serotar``: the pair embedding with its last-token state, the update of the stream by normed
sublayer outputs with the average over depth, xIELU, the per-layer token input, the router's rule (scores over all outputs,
correction, groups, identity experts), gated experts in all three forms, and latent attention without positions.  Where
random weights would hide a lost key or a lost state, weights and inputs are made so that it shows."""
import math

import pytest
import torch

import plain_serotar as ps
import test_getizen_parts_gpu as harness
import helpers

pytestmark = pytest.mark.gpu
DEV = "cuda"
DTYPES = [torch.float32, torch.bfloat16]
rt_for, build, bind_random, Harness, run_in_portions, inputs = (harness.rt_for, harness.build, harness.bind_random, harness.Harness,
                                                                harness.run_in_portions, harness.inputs)


def close(got, want, dtype, what="", bf16=4e-2):
    if dtype == torch.bfloat16:
        got, want = got.float().cpu(), want.float().cpu()
        assert got.shape == want.shape and torch.isfinite(got).all(), what
        scale = max(want.abs().max().item(), 1e-6)
        err = (got - want).abs().max().item()
        assert err <= bf16 * scale, f"{what}: max abs error {err:.3e} > {bf16} x {scale:.3e}"
        return err / scale
    return helpers.close(got, want, dtype, what)


def weights_of(W):
    return {k[2:]: v for k, v in W.items()}


# ----------------------------------------------------------------------------------------------- embedding

class EmbeddingHarness:
    """Runs an embedding with per-request state over requests step by step: its own state slots and batch builder."""

    def __init__(self, emb, rt, slots):
        from mini_inference_engine_b200.cache.manager import CacheManager
        from mini_inference_engine_b200.cache.storage import CacheLayout, CacheStorage
        from mini_inference_engine_b200.engine.batch import BatchBuilder
        layout = CacheLayout.from_needs({"embedding": emb.cache_need()})
        self.emb = emb
        self.manager = CacheManager(layout.groups, 64, 16, slots)
        self.storage = CacheStorage(layout, 64, 16, slots, rt.dtype, DEV)
        self.cache = self.storage.layer_cache("embedding")
        self.builder = BatchBuilder(len(layout.groups), 16, DEV)

    def step(self, entries, feedback=None):
        """entries: [(request cache, token ids)] -> (stream rows per entry, the LayeredStream)."""
        from mini_inference_engine_b200.engine.batch import BatchRow
        rows = []
        for rc, toks in entries:
            assert self.manager.take_state_slot(rc) and self.manager.reserve(rc, len(toks))
            if rc.num_computed == 0:
                self.storage.clear_state_slot(rc.state_slot)
            rows.append(BatchRow(list(toks), rc.num_computed, rc.table_arrays(), rc.state_slot, []))
        ctx = self.builder.build(rows)
        ctx.token_feedback = feedback
        res, stream = self.emb.forward(ctx, self.cache)
        out, at = [], 0
        for rc, toks in entries:
            self.manager.advance(rc, len(toks))
            out.append(res[at:at + len(toks)].cpu())
            at += len(toks)
        return out, stream, res


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("buckets,mul_prev,mul_cur,width", [(97, 31, 7, 48), (1, 3, 2, 50), (1000003, 99991, 65537, 64)])
def test_pair_embedding_keeps_the_token_before_a_step(dt, buckets, mul_prev, mul_cur, width):
    from mini_inference_engine_b200.cache.manager import RequestCache
    rt = rt_for(dt)
    vocab = 120
    many = min(buckets, 4000)                 # (a table of a million rows would only slow the test: the hash is checked below)
    emb = build("embedding", "pair_embedding", vocab_size=vocab, hidden_size=width, scale=6.0, buckets=many, mul_prev=mul_prev,
                mul_cur=mul_cur, side_width=10, history=3)
    W = weights_of(bind_random(emb, rt, 21))
    cfg = dict(embedding=dict(scale=6.0, bigram=dict(buckets=many, mul_prev=mul_prev, mul_cur=mul_cur)))
    P = {"embed": W["weight"], "bigram": W["pair"]}
    g = torch.Generator().manual_seed(5)
    seqs = [torch.randint(0, vocab, (n,), generator=g).tolist() for n in (37, 1, 20, 9)]
    h = EmbeddingHarness(emb, rt, slots=2)
    # one request in portions down to one token; the state carries the token before each portion
    rc, at, got = RequestCache(), 0, []
    for n in (1, 1, 2, 16, 1, 3, 13):
        out, stream, res = h.step([(rc, seqs[0][at:at + n])])
        got.append(out[0])
        at += n
        assert stream.tokens.cpu().tolist() == seqs[0][at - n:at] and torch.equal(stream.history[0], res)
        if dt == torch.bfloat16:
            assert torch.equal(stream.x, res.to(torch.bfloat16))
    close(torch.cat(got), ps.embedding(seqs[0], P, cfg), torch.float32, "portions of one request")
    h.manager.free(rc)
    # two slots for three more requests: a slot that another request left holds that request's last token, and the first
    # token of the next one must not read it; two requests in one batch, cut at different places
    a, b = RequestCache(), RequestCache()
    o1, _, _ = h.step([(a, seqs[2][:7]), (b, seqs[1])])
    h.manager.free(b)
    c = RequestCache()
    o2, _, _ = h.step([(c, seqs[3][:1]), (a, seqs[2][7:8])])
    o3, _, _ = h.step([(a, seqs[2][8:]), (c, seqs[3][1:])])
    close(torch.cat([o1[0], o2[1], o3[0]]), ps.embedding(seqs[2], P, cfg), torch.float32, "a request beside others")
    close(o1[1], ps.embedding(seqs[1], P, cfg), torch.float32, "a request of one token")
    close(torch.cat([o2[0], o3[1]]), ps.embedding(seqs[3], P, cfg), torch.float32, "a request in a slot used before")
    # a token that the step before sampled on the device (id -(k+1) = entry k of the fed-back tokens), as the one before too
    fb = torch.tensor([seqs[0][5], seqs[0][6]], dtype=torch.int32, device=DEV)
    d = RequestCache()
    h.manager.free(a), h.manager.free(c)
    o4, _, _ = h.step([(d, seqs[0][:5])])
    o5, _, _ = h.step([(d, [-1])], feedback=fb)
    o6, s6, _ = h.step([(d, [-2, seqs[0][7]])], feedback=fb)
    close(torch.cat([o4[0], o5[0], o6[0]]), ps.embedding(seqs[0][:8], P, cfg), torch.float32, "fed-back tokens")
    assert s6.tokens.cpu().tolist() == seqs[0][6:8]


def test_pair_hash_of_large_multipliers():
    """The hash is taken in 64-bit: multipliers and token ids whose product passes 2^31."""
    rt = rt_for(torch.float32)
    vocab, buckets, mp, mc = 70000, 2039, 2000003, 1999993
    emb = build("embedding", "pair_embedding", vocab_size=vocab, hidden_size=8, scale=1.0, buckets=buckets, mul_prev=mp, mul_cur=mc)
    W = weights_of(bind_random(emb, rt, 22))
    from mini_inference_engine_b200.cache.manager import RequestCache
    toks = [69999, 69998, 12345, 69997, 3]
    out, _, _ = EmbeddingHarness(emb, rt, 1).step([(RequestCache(), toks)])
    rows = ps.bigram_rows(toks, buckets, mp, mc)
    assert rows.tolist()[1] == (69999 * mp + 69998 * mc) % buckets
    close(out[0], W["weight"][torch.tensor(toks)] + W["pair"][rows], torch.float32)


# ----------------------------------------------------------------------------------------------- the stream's update

@pytest.mark.parametrize("width", [48, 50, 2048])
def test_normed_outputs_are_added_and_layers_averaged_over_depth(width):
    from mini_inference_engine_b200.kernels import ops
    g = torch.Generator().manual_seed(7)
    T, eps = 11, 1e-5
    res = torch.randn(T, width, generator=g)
    a, b, c = (torch.randn(T, width, generator=g) for _ in range(3))
    h = torch.randn(T, width, generator=g).to(torch.bfloat16)
    w = torch.rand(T, generator=g)
    gain, vec = torch.tensor([1.3]), torch.randn(width, generator=g)
    dev = lambda t: t.to(DEV).contiguous()
    # three outputs of two types and one scaled by a number per row, a gain and a vector
    y = a + b.to(torch.bfloat16).float() + c + w[:, None] * h.float()
    want = res + ps.rms(y, eps) * gain * vec
    r, act = dev(res.clone()), torch.empty(T, width, dtype=torch.bfloat16, device=DEV)
    ops.normed_add(r, (dev(a), dev(b.to(torch.bfloat16)), dev(c)), scaled=(dev(h), dev(w)), gain=dev(gain), vec=dev(vec), eps=eps, act=act)
    close(r, want, torch.float32, "sum, norm, scale")
    assert torch.equal(act, r.to(torch.bfloat16))
    # one output, no gain, no vector
    r = dev(res.clone())
    ops.normed_add(r, (dev(a),), eps=eps)
    close(r, res + ps.rms(a, eps), torch.float32, "plain")
    # a history of four results: the new one is stored, the stream becomes the weighted sum
    hist = torch.randn(5, T, width, generator=g)
    coef = torch.tensor([0.4, -0.2, 0.3, 0.9])
    r, hd = dev(res.clone()), dev(hist.clone())
    ops.normed_add(r, (dev(a),), vec=dev(vec), eps=eps, history=hd, slot=3, coef=dev(coef), act=act)
    new = res + ps.rms(a, eps) * vec
    close(hd[3], new, torch.float32, "the stored result")
    assert torch.equal(hd[:3].cpu(), hist[:3]) and torch.equal(hd[4].cpu(), hist[4])
    close(r, coef[0] * hist[0] + coef[1] * hist[1] + coef[2] * hist[2] + coef[3] * new, torch.float32, "the average over depth")
    assert torch.equal(act, r.to(torch.bfloat16))
    # the average alone (a layer without anything to add behind its sublayers), first slot
    r, hd = dev(res.clone()), dev(hist.clone())
    ops.normed_add(r, (), history=hd, slot=1, coef=dev(coef[:2].clone()))
    close(hd[1], res, torch.float32)
    close(r, coef[0] * hist[0] + coef[1] * res, torch.float32, "average without an addend")


@pytest.mark.parametrize("dt", DTYPES)
def test_scalar_norm_in_front_of_the_head(dt):
    rt = rt_for(dt)
    norm = build("norm", "scalar_rmsnorm", size=50, eps=1e-5)
    W = weights_of(bind_random(norm, rt, 23))
    x = inputs(9, 50, 3, torch.float32)
    rows = torch.tensor([8, 0, 3], dtype=torch.int32, device=DEV)
    close(norm(None, x.to(DEV), rows=rows), ps.scalar_norm(x, W["weight"], 1e-5)[rows.cpu().long()], dt)


# ----------------------------------------------------------------------------------------------- feed-forward parts

@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("p,q", [(0.0, 0.0), (1.5, -2.0), (-3.0, 2.5)])
def test_dense_feed_forward_with_xielu(dt, p, q):
    from mini_inference_engine_b200.kernels import ops
    rt = rt_for(dt)
    z = torch.cat([torch.linspace(-30, 30, 241), torch.tensor([0.0, -1e-4, 1e-4])]).to(dt)
    act = torch.tensor([p, q])
    ap, an = math.log1p(math.exp(p)), 0.5 + math.log1p(math.exp(q))
    got = ops.xielu(z.to(DEV), torch.empty_like(z, device=DEV), ap, an)
    close(got, ps.xielu(z.float(), act), dt, "the activation alone", bf16=1e-2)
    for hid, ff in ((40, 72), (50, 30)):
        part = build("feed_forward", "activated_mlp", hidden_size=hid, intermediate_size=ff)
        W = weights_of(bind_random(part, rt, 24, {"act": act}))
        for T in (1, 40):
            x = inputs(T, hid, 50 + T, dt)
            got = part.forward(x.to(dt).to(DEV), None)
            assert got.dtype == torch.float32
            close(got, ps.dense_ff(x, W), dt, f"{T} tokens")


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("hid,dim,index", [(48, 8, 2), (50, 3, 0), (64, 24, 1)])
def test_token_input_gated_by_the_stream(dt, hid, dim, index):
    from mini_inference_engine_b200.parts.embedding import LayeredStream
    rt = rt_for(dt)
    part = build("token_input", "gated_table", hidden_size=hid, dim=dim, index=index)
    W = weights_of(bind_random(part, rt, 25))
    g = torch.Generator().manual_seed(3)
    vocab, T = 30, 21
    table = torch.randn(vocab, 3 * dim, generator=g).to(torch.bfloat16).float()
    tokens = torch.randint(0, vocab, (T,), generator=g)
    x = inputs(T, hid, 9, dt)
    want = ps.lin(ps.gelu_tanh(ps.lin(x, W["gate"])) * table[tokens][:, index * dim:(index + 1) * dim], W["proj"])
    stream = LayeredStream(None, tokens.int().to(DEV), table.to(dt).to(DEV))
    got = part.forward(x.to(dt).to(DEV), stream)
    assert got.dtype == torch.float32
    close(got, want, dt)


def test_xielu_in_the_epilogue_of_the_prompt_sized_product():
    """From 128 tokens on the up product of a bfloat16 model runs on pairs of SMs and applies the activation to its float32
    sums; the plain implementation applies it to the unrounded product too."""
    from mini_inference_engine_b200.kernels import linear as lk
    g = torch.Generator().manual_seed(11)
    ran = 0
    for T, hid, ff, p, q in ((2048, 128, 1792, 0.4, -0.6), (3000, 64, 3072, -1.0, 1.5), (4100, 72, 4600 // 8 * 8, 0.0, 0.0)):
        x = (torch.randn(T, hid, generator=g)).bfloat16()
        w = (torch.randn(ff, hid, generator=g) * hid ** -0.5 * 3).bfloat16()
        ap, an = math.log1p(math.exp(p)), 0.5 + math.log1p(math.exp(q))
        if not lk.takes_pair(T, w.to(DEV)):          # sizes that fill too few of this device's pairs of SMs
            continue
        ran += 1
        got = lk.linear_xielu(x.to(DEV), w.to(DEV), ap, an, torch.bfloat16)
        want = ps.xielu(x.float() @ w.float().t(), torch.tensor([p, q]))
        close(got, want, torch.bfloat16, f"{T} tokens", bf16=1e-2)
        # and the product followed by the activation kernel, which small steps use, agrees up to the rounding between them
        up = lk.linear(x[:8].to(DEV), w.to(DEV), None, torch.bfloat16)
        from mini_inference_engine_b200.kernels import ops
        close(ops.xielu(up, torch.empty_like(up), ap, an), want[:8], torch.bfloat16, "8 tokens", bf16=2e-2)
    if not ran:
        pytest.skip("the paired product takes none of these sizes on this device")


# ----------------------------------------------------------------------------------------------- router and experts

@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("width,outputs", [(1024, 5), (1000, 20), (2050, 3), (4096, 8), (512, 40), (333, 2)])
def test_router_logits_of_wide_inputs_do_not_depend_on_the_batch(dt, width, outputs):
    """Wide inputs with few outputs: a row's dot product is cut into column segments (16-byte and scalar paths); a token's
    logits are the same numbers whatever else is in the batch."""
    from mini_inference_engine_b200.kernels import ops
    g = torch.Generator().manual_seed(width + outputs)
    x = torch.randn(700, width, generator=g).to(dt)
    wr = torch.randn(outputs, width, generator=g) * width ** -0.5
    top = min(2, outputs)
    whole = torch.empty(700, outputs, device=DEV)
    ids, wts = ops.moe_router(x.to(DEV), wr.to(DEV), top, whole)
    want = x.double() @ wr.double().t()
    assert torch.allclose(whole.cpu().double(), want, atol=2e-5, rtol=1e-5)
    order = want.topk(top, -1).indices
    sure = (want.topk(top + 1, -1).values.diff(dim=-1).abs().min(-1).values > 1e-4) if outputs > top else torch.ones(700, dtype=torch.bool)
    assert torch.equal(ids.cpu().long()[sure], order[sure])
    for rows in ([0], [5, 6, 7], list(range(100, 109)), list(range(400, 700))):
        part = torch.empty(len(rows), outputs, device=DEV)
        ops.moe_router(x[rows].contiguous().to(DEV), wr.to(DEV), top, part)
        assert torch.equal(part, whole[rows]), f"rows {rows[:3]}.. of width {width}"


def test_expert_rows_are_summed_per_token_in_order():
    from mini_inference_engine_b200.kernels import ops
    g = torch.Generator().manual_seed(3)
    for T, top, h, real in ((37, 3, 64, 5), (300, 4, 1024, 6), (9, 2, 50, 4)):
        ids = torch.stack([torch.randperm(8, generator=g)[:top] for _ in range(T)]).int()
        place = torch.randperm(T * top, generator=g).int()
        for dt in DTYPES:
            rows = torch.randn(T * top, h, generator=g).to(dt)
            want = torch.zeros(T, h)
            for k in range(top):
                want += rows.float()[place.view(T, top)[:, k].long()] * (ids[:, k:k + 1] < real)
            got = ops.moe_combine(rows.to(DEV), place.to(DEV), top, torch.empty(T, h, device=DEV), ids.to(DEV), real)
            assert torch.allclose(got.cpu(), want, atol=1e-5), (T, top, h, dt)


def test_router_scores_all_outputs_and_chooses_within_the_best_groups():
    from mini_inference_engine_b200.kernels import ops
    g = torch.Generator().manual_seed(4)
    for outputs, top, groups, keep, real in ((6, 2, 3, 2, 5), (24, 6, 8, 3, 16), (10, 3, 2, 1, 8), (7, 2, 7, 4, 5), (12, 4, 1, 1, 12),
                                            (64, 8, 64, 9, 40), (6, 3, 2, 1, 3)):
        z = torch.randn(50, outputs, generator=g) * 2
        # corrections far below zero: every choice score is negative, so a group that is left out must count as minus
        # infinity -- counted as 0 it would win
        for corr in (torch.randn(outputs, generator=g) * 0.1, torch.randn(outputs, generator=g) * 0.1 - 2.0):
            r = dict(experts=real, identity=outputs - real, top=top)
            if groups > 1:
                r["groups"] = dict(count=groups, keep=keep)
            eye = torch.eye(outputs)                 # the plain router computes logits from an input: the input is the logits
            ids_w, w_w = ps.route(z, dict(router=eye, correction=corr), r)
            rule = ops.RouteRule("softmax", corr.to(DEV), groups, keep, real)
            out = ops.moe_route(z.to(DEV), top, rule)
            assert sorted(out[0].cpu().tolist()[7]) == sorted(ids_w.tolist()[7])
            assert torch.equal(out[0].cpu().long().sort(-1).values, ids_w.sort(-1).values), (outputs, groups, keep)
            order = out[0].cpu().long()
            assert torch.allclose(out[1].cpu(), torch.softmax(z, -1).gather(1, order), atol=1e-6)
            if real < outputs:
                rest = (out[1].cpu() * (order >= real)).sum(-1)
                assert torch.allclose(out[2].cpu(), rest, atol=1e-6)
            else:
                assert len(out) == 2
            # the same with the logits computed in the kernel
            for dt in DTYPES:
                x = torch.randn(50, 40, generator=g).to(dt)
                wr = torch.randn(outputs, 40, generator=g)
                logits = torch.empty(50, outputs, device=DEV)
                got = ops.moe_router(x.to(DEV), wr.to(DEV), top, logits, rule)
                ref = ops.moe_route(logits, top, rule)
                assert torch.allclose(logits.cpu(), x.float() @ wr.t(), atol=1e-4, rtol=1e-5)
                assert torch.equal(got[0], ref[0]) and torch.allclose(got[1], ref[1], atol=1e-6)
                if real < outputs:
                    assert torch.allclose(got[2], ref[2], atol=1e-6)


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("experts,top,ff,identity,groups,shared", [
    (6, 2, 24, 2, (2, 1), 16), (5, 1, 16, 0, None, None), (3, 3, 16, 3, (2, 1), 8), (1, 1, 8, 0, None, 24), (16, 4, 32, 8, (8, 3), 40),
    (40, 2, 16, 0, (5, 2), None), (5, 2, 10, 1, (3, 2), 6)])
def test_gated_experts_with_identity_and_shared_experts(dt, experts, top, ff, identity, groups, shared):
    """1 to 200 tokens: pairs that stream their own expert's rows, all experts as one wide feed-forward, and rows sorted by
    expert for the grouped product.  Router logits are well apart, so no choice is a close call."""
    from mini_inference_engine_b200.config import PartSpec
    from mini_inference_engine_b200.parts import Branches
    rt = rt_for(dt)
    hid = 40
    outputs = experts + identity
    count, keep = groups or (1, 1)
    sh = None if shared is None else PartSpec("clamped_glu", dict(hidden_size=hid, intermediate_size=shared, limit=0.0, slope=1.0, shift=0.0))
    part = build("feed_forward", "routed_experts", hidden_size=hid, num_experts=experts, top=top, expert_size=ff, activation="silu", gated=True,
                 score="softmax", correction=True, groups=count, keep=keep, identity=identity, shared=sh)
    g = torch.Generator().manual_seed(8)
    W = weights_of(bind_random(part, rt, 26, {"router": torch.randn(outputs, hid, generator=g), "correction": torch.randn(outputs, generator=g) * 0.3}))
    mlp = dict(kind="moe", router=dict(experts=experts, top=top, identity=identity), shared=None if shared is None else dict(ff=shared))
    if groups:
        mlp["router"]["groups"] = dict(count=count, keep=keep)
    for T in (1, 2, 3, 9, 50, 200):
        x = inputs(T, hid, 40 + T, dt)
        want = ps.moe_ff(x, W, mlp)
        out = part.forward(x.to(dt).to(DEV), None)
        if isinstance(out, Branches):
            got = sum(d.float() for d in out.deltas)
            if out.scaled is not None:
                got = got + out.scaled[1][:, None] * out.scaled[0].float()
        else:
            assert not identity and shared is None
            got = out
        close(got, want, dt, f"{T} tokens")


# ----------------------------------------------------------------------------------------------- latent attention without positions

def latent_params(**kw):
    p = dict(hidden_size=40, num_heads=3, dim=16, rot_dim=0, vdim=32, q_rank=24, kv_rank=40, scale=0.25, rot_dims=0, rot_base=1.0,
             eps=1e-5, gate=False)
    p.update(kw)
    return p


def plain_latent(params, W, x):
    m = dict(heads=params["num_heads"], dim=params["dim"], vdim=params["vdim"], scale=params["scale"])
    return ps.latent_attention(x, W, m, params["eps"])


LATENT_CASES = [latent_params(), latent_params(num_heads=1, dim=64, vdim=64, q_rank=8, kv_rank=16),       # one head of 64, ranks below the head
                latent_params(num_heads=2, dim=128, vdim=64, scale=0.09), latent_params(num_heads=5, dim=10, vdim=20, q_rank=7, kv_rank=9),
                latent_params(num_heads=2, dim=24, vdim=160)]


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("params", LATENT_CASES)
def test_latent_attention_whole_in_portions_and_in_batches(dt, params):
    rt = rt_for(dt)
    mixer = build("mixer", "latent_attention", **params)
    assert set(mixer.tensor_specs()) == {"dq", "dq.norm", "uq", "dkv", "dkv.norm", "uk", "uv", "o"}
    W = weights_of(bind_random(mixer, rt, 27))
    h = Harness(mixer, rt, pages=24, slots=3)
    hid = params["hidden_size"]
    x = inputs(75, hid, 1, dt)
    want = plain_latent(params, W, x)
    close(run_in_portions(h, x, [75]), want, dt, "whole")
    close(run_in_portions(h, x, [33, 1, 1, 14, 2, 17, 1, 1, 1, 1, 1, 1, 1]), want, dt, "portions and single tokens")
    xs = [inputs(n, hid, 20 + i, dt) for i, n in enumerate((40, 9, 61))]
    wants = [plain_latent(params, W, xi) for xi in xs]
    rcs = [h.new() for _ in xs]
    cuts = [(17, 23), (8, 1), (60, 1)]
    first = h.step([(rc, xi[:a]) for rc, xi, (a, _) in zip(rcs, xs, cuts)])
    second = h.step([(rc, xi[a:]) for rc, xi, (a, _) in zip(rcs, xs, cuts)])
    for i, (f, s) in enumerate(zip(first, second)):
        close(torch.cat([f, s], 0), wants[i], dt, f"request {i} of a batch")
    for rc in rcs:
        h.free(rc)
    h.manager.check()


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("far", [0, 15, 16, 31, 32, 250, 296])
def test_a_key_far_back_that_stands_out(dt, far):
    """Keys are made by the queries' matrices (equal ranks, equal norm weights) from the input shifted by one channel, so a
    key whose input is the query's input shifted back scores |q|^2, far above all others, while its value is unlike the
    queries' own: one key among 300 decides the last outputs, wherever it lies -- the first token, either side of a page
    border, hundreds of tokens back, just before the queries.  Lost in a portion or by a decoding step, the output is
    another altogether."""
    rt = rt_for(dt)
    params = latent_params(num_heads=2, dim=32, vdim=48, q_rank=24, kv_rank=24, scale=1.0)
    mixer = build("mixer", "latent_attention", **params)
    from mini_inference_engine_b200.weights.random_init import random_tensor
    specs = mixer.tensor_specs()
    same = {"dkv": torch.roll(random_tensor(28, "dq", specs["dq"], torch.bfloat16).float(), 1, dims=1), "uk": random_tensor(28, "uq", specs["uq"], torch.bfloat16).float(),
            "dkv.norm": random_tensor(28, "dq.norm", specs["dq.norm"], torch.bfloat16).float()}
    W = weights_of(bind_random(mixer, rt, 28, same))
    hid, T = params["hidden_size"], 300
    x = inputs(T, hid, 2, dt)
    g = torch.Generator().manual_seed(9)
    mark = torch.randn(hid, generator=g).to(dt).float()
    small = x[far].clone()
    x[far] = torch.roll(mark, 1)              # W_dkv x[far] = W_dq mark
    x[T - 3:] = mark + 0.05 * torch.randn(3, hid, generator=g).to(dt).float()
    without = x.clone()
    without[far] = small
    want, lost = plain_latent(params, W, x), plain_latent(params, W, without)
    assert (want[-3:] - lost[-3:]).abs().max() > 0.05 * want[-3:].abs().max(), "the planted key must matter"
    h = Harness(mixer, rt, pages=24, slots=1)
    close(run_in_portions(h, x, [T]), want, dt, "whole")
    close(run_in_portions(h, x, [T - 5, 2, 1, 1, 1]), want, dt, "the last queries decoded alone")
    close(run_in_portions(h, x, [7, 9, 1, 15, 2, 200, 61, 3, 2]), want, dt, "portions cut inside pages")


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("gated", [True, False])
def test_pair_kernels_give_a_token_the_same_sums_in_a_small_and_in_a_large_batch(dt, gated):
    """The experts' kernels for single (token, expert) pairs come in two forms, chosen by the size of the batch: one row a warp
    and four column steps at a time, or four rows a warp.  Both against the plain sum, and a token's result must be the same
    number for number whichever form its batch got: a row's sum runs over its columns in one order."""
    from mini_inference_engine_b200.kernels import ops
    g = torch.Generator().manual_seed(11)
    h, F, E, top, identity = 512, 136, 12, 4, 3
    wu = (torch.randn(E * (2 if gated else 1) * F, h, generator=g) * h ** -0.5).to(dt)
    wd = (torch.randn(h, E * F, generator=g) * F ** -0.5).to(dt)
    x = torch.randn(48, h, generator=g).to(dt)
    ids = torch.stack([torch.randperm(E + identity, generator=g)[:top] for _ in range(48)]).to(torch.int32)
    wts = torch.rand(48, top, generator=g) + 0.1
    want = torch.zeros(48, h, dtype=torch.float64)
    for t in range(48):
        for e, w in zip(ids[t].tolist(), wts[t].tolist()):
            if e >= E:
                continue                                   # an identity expert: the pair kernels add nothing for it
            if gated:
                gate = wu[e * 2 * F:e * 2 * F + F].double() @ x[t].double()
                up = wu[e * 2 * F + F:(e + 1) * 2 * F].double() @ x[t].double()
                hid = w * torch.nn.functional.silu(gate) * up
            else:
                hid = w * torch.nn.functional.silu(wu[e * F:(e + 1) * F].double() @ x[t].double())
            if dt == torch.bfloat16:
                hid = hid.to(dt).double()                  # the hidden row is stored in the activation type
            want[t] += wd[:, e * F:(e + 1) * F].double() @ hid
    outs = {}
    for T in (1, 2, 5, 48):                                # 48 tokens of 512: four rows a warp; the others: one row
        out = torch.empty(T, h, dtype=torch.float32, device=DEV)
        ops.moe_pairs(x[:T].contiguous().to(DEV), wu.to(DEV), wd.to(DEV), ids[:T].contiguous().to(DEV), wts[:T].contiguous().to(DEV), out, E,
                      "silu", gated=gated)
        outs[T] = out.cpu()
        tol = 2e-2 if dt == torch.bfloat16 else 1e-4
        assert (outs[T].double() - want[:T]).abs().max().item() <= tol * want.abs().max().item(), (T, dt, gated)
    for T in (1, 2, 5):
        assert torch.equal(outs[T], outs[48][:T]), f"a token's sums differ between a batch of {T} and a batch of 48"
