"""The mechanisms of the Luluzen design one by one, built through the part registry with sizes of their own, against the
plain functions of ``plain_luluzen``: the layer norm with its sums, the step that mixes the stream with the embedding's
output, the gelu-gated feed-forward, the experts weighted on their input, lightning attention, the matrix memory, softmax
attention with a bias by distance and a temperature by position, windowed attention with a cap and a sink, and mixers side
by side.  Mixers run a sequence whole, in portions down to one token, and several requests in one batch, from state slots
and pages that other requests used before."""
import pytest
import torch

import plain_luluzen as pz
from helpers import close
from test_getizen_parts_gpu import DEV, DTYPES, Harness, bind_random, build, inputs, rt_for, run_in_portions

pytestmark = pytest.mark.gpu


# ----------------------------------------------------------------------------------------------- norm, stream mix, head

@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("n", [48, 50, 1024])
def test_layer_norm_with_the_sums_in_front_of_it(dt, n):
    from mini_inference_engine_b200.parts import Branches
    rt = rt_for(dt)
    T, eps = 7, 3e-4
    norm = build("norm", "layernorm", size=n, eps=eps)
    W = bind_random(norm, rt, 3, {"weight": torch.randn(n)})
    res = torch.randn(T, n) + 5.0                      # a mean far from zero: the variance is that of the deviations
    d0, d1 = torch.randn(T, n) * 3, torch.randn(T, n) * 0.2
    r = res.clone().to(DEV)
    out = norm(Branches((d0.to(DEV), d1.to(DEV)), coefs=(1.25, -0.5)), r)
    want = res + 1.25 * d0 - 0.5 * d1
    close(r, want, torch.float32, "stream after the sum")
    close(out, pz.layer_norm(want, W["p.weight"], eps), dt, "two addends with coefficients")
    r = res.clone().to(DEV)
    close(norm(d0.to(DEV), r), pz.layer_norm(res + d0, W["p.weight"], eps), dt, "one addend")
    close(norm(d1.to(torch.bfloat16).to(DEV), res.clone().to(DEV)), pz.layer_norm(res + d1.to(torch.bfloat16).float(), W["p.weight"], eps), dt,
          "a bfloat16 addend")
    # rows gathered in front of the head: the pending sum is taken in, the stream is not written
    r = res.clone().to(DEV)
    rows = torch.tensor([5, 0, 5], dtype=torch.int32, device=DEV)
    close(norm(d0.to(DEV), r, rows), pz.layer_norm(res + d0, W["p.weight"], eps)[[5, 0, 5]], dt, "gathered rows")
    assert torch.equal(r.cpu(), res)
    # without the mean it is an RMS norm
    rms = build("norm", "layernorm", size=n, eps=eps, center=False)
    bind_random(rms, rt, 3, {"weight": W["p.weight"]})
    close(rms(None, res.clone().to(DEV)), pz.rms_scale(res, eps) * W["p.weight"], dt, "no centring")


@pytest.mark.parametrize("dt", DTYPES)
def test_stream_mixed_with_the_embedding_output(dt):
    from types import SimpleNamespace
    from mini_inference_engine_b200.parts import Branches
    rt = rt_for(dt)
    n, T = 40, 9
    mix = build("connection", "stream_mix", hidden_size=n, rows=3, index=2)
    W = bind_random(mix, rt, 4)
    res, e, d = torch.randn(T, n), inputs(T, n, 1, torch.bfloat16), torch.randn(T, n)
    ctx = SimpleNamespace(extras={"embedding_output": e.to(DEV)})
    r = res.clone().to(DEV)
    mix.apply(Branches((d.to(DEV),), coefs=(0.5,)), r, ctx)
    x = (res + 0.5 * d).to(dt).float()
    close(r, torch.cat([x, e], -1) @ W["p.in"].T + W["p.step"][2], dt, "mixed stream")
    with pytest.raises(ValueError):
        mix.apply(None, r, SimpleNamespace(extras={}))


def test_head_with_a_soft_cap():
    rt = rt_for(torch.float32)
    head = build("head", "linear_head", vocab_size=70, hidden_size=24, softcap=4.0)
    W = bind_random(head, rt, 5, {"weight": torch.randn(70, 24)})
    x = torch.randn(5, 24)
    z = x @ W["p.weight"].T
    assert (z.abs() > 4).any()
    close(head.forward(x.to(DEV)), 4.0 * torch.tanh(z / 4.0), torch.float32, "capped logits")


# ----------------------------------------------------------------------------------------------- feed-forward

@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("T", [1, 9, 200])
def test_gelu_gated_feed_forward(dt, T):
    from mini_inference_engine_b200.config.luluzen_config import GELU_CUBIC, GELU_SLOPE
    rt = rt_for(dt)
    ff = build("feed_forward", "clamped_glu", hidden_size=64, intermediate_size=144, limit=-GELU_CUBIC, slope=GELU_SLOPE, shift=0.0)
    W = bind_random(ff, rt, 6)
    x = inputs(T, 64, 1, dt) * 2
    close(ff.forward(x.to(dt).to(DEV), None), pz.dense_ff(x, W, "p."), dt, "gelu-gated feed-forward")


EXPERTS = [dict(num_experts=8, top=1, expert_size=24), dict(num_experts=5, top=5, expert_size=16), dict(num_experts=1, top=1, expert_size=40),
           dict(num_experts=17, top=3, expert_size=8)]


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("params", EXPERTS)
def test_experts_weighted_on_their_input(dt, params):
    """Every form of the experts (a pair a block for a handful of tokens, all experts as one wide layer, rows sorted by
    expert) against the plain sum; the clamp must bite, so that a weight on the output instead of the input would show."""
    rt = rt_for(dt)
    hidden, limit = 48, 0.6
    ff = build("feed_forward", "routed_experts", hidden_size=hidden, activation="clamped_in", gated=True, score="sigmoid", limit=limit, **params)
    W = bind_random(ff, rt, 7)
    mlp = dict(router=dict(experts=params["num_experts"], top=params["top"]), expert=dict(ff=params["expert_size"], limit=limit))
    for T in (1, 2, 7, 40, 200):
        x = inputs(T, hidden, 20 + T, dt) * 2
        want = pz.routed_ff(x, W, "p.", mlp)
        if T == 200:
            idx, val = pz.router_choice(x, W, "p.", params["top"])
            assert any((((x[t] * val[t, 0]) @ W[f"p.e{int(idx[t, 0])}.gate"].T) > limit).any() for t in range(T)), "the clamp must bite"
        got = ff.forward(x.to(dt).to(DEV), None).float().cpu()
        if dt == torch.bfloat16:               # a router whose scores nearly tie may choose otherwise on rounded inputs: such tokens are left out
            s = torch.sigmoid(x @ W["p.router"].T).sort(-1, descending=True).values
            k = params["top"]
            sure = torch.ones(T, dtype=torch.bool) if k == params["num_experts"] else (s[:, k - 1] - s[:, k]) > 0.02
            got, want = got[sure], want[sure]
        close(got, want, dt, f"{T} tokens")


# ----------------------------------------------------------------------------------------------- lightning attention

LIGHTNING = [dict(num_heads=3, dim=16, vdim=32, decay=(0.5, 0.9, 0.999)), dict(num_heads=1, dim=48, vdim=16, decay=(0.97,)),
             dict(num_heads=2, dim=80, vdim=40, decay=(1.0, 0.75)), dict(num_heads=1, dim=64, vdim=136, decay=(0.9,))]


def lightning_cfg(p):
    return dict(heads=p["num_heads"], dim=p["dim"], vdim=p["vdim"], decay=list(p["decay"]))


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("params", LIGHTNING)
def test_lightning_whole_in_portions_and_token_by_token(dt, params):
    rt = rt_for(dt)
    hidden, T = 24, 150                      # portions longer than a chunk of the recurrence's kernel run as several side by side
    mixer = build("mixer", "lightning_attention", hidden_size=hidden, eps=1e-5, **params)
    W = bind_random(mixer, rt, 8)
    x = inputs(T, hidden, 2, dt)
    want = pz.lightning(x, W, "p.", lightning_cfg(params), 1e-5)
    h = Harness(mixer, rt)
    close(run_in_portions(h, x, [T]), want, dt, "whole")
    close(run_in_portions(h, x, [9, 2, 70, 1, 1, 64, 2, 1]), want, dt, "portions")         # the slot was used before
    close(run_in_portions(h, x, [129, 21]), want, dt, "a portion of two chunks and one token")
    close(run_in_portions(h, x, [1] * T), want, dt, "token by token")


@pytest.mark.parametrize("dt", DTYPES)
def test_lightning_batch_of_unequal_requests_and_a_far_token(dt):
    rt = rt_for(dt)
    hidden = 32
    params = dict(num_heads=2, dim=32, vdim=32, decay=(0.999, 0.9995))
    mixer = build("mixer", "lightning_attention", hidden_size=hidden, eps=1e-5, **params)
    W = bind_random(mixer, rt, 9)
    m = lightning_cfg(params)
    xs = [inputs(n, hidden, 10 + i, dt) for i, n in enumerate((300, 7, 64))]
    xs[0][3] *= 8.0                                   # one early token that the state must still hold 296 tokens on
    wants = [pz.lightning(x, W, "p.", m, 1e-5) for x in xs]
    quiet = xs[0].clone()
    quiet[3] /= 8.0
    assert (pz.lightning(quiet, W, "p.", m, 1e-5)[-1] - wants[0][-1]).abs().max() > 0.05 * wants[0][-1].abs().max()
    h = Harness(mixer, rt, pages=32, slots=3)
    rcs = [h.new() for _ in xs]
    a = h.step([(rcs[0], xs[0][:250]), (rcs[1], xs[1][:6]), (rcs[2], xs[2][:63])])
    b = h.step([(rcs[1], xs[1][6:]), (rcs[0], xs[0][250:]), (rcs[2], xs[2][63:])])
    close(torch.cat([a[0], b[1]]), wants[0], dt, "long request")
    close(torch.cat([a[1], b[0]]), wants[1], dt, "short request")
    close(torch.cat([a[2], b[2]]), wants[2], dt, "third request")


# ----------------------------------------------------------------------------------------------- matrix memory

MEMORIES = [dict(num_heads=3, dim=16, vdim=32, gate_cap=15.0), dict(num_heads=1, dim=48, vdim=16, gate_cap=2.0),
            dict(num_heads=2, dim=128, vdim=128, gate_cap=0.0), dict(num_heads=5, dim=24, vdim=63, gate_cap=8.0)]


def close_memory(got, want, dt, what):
    """float32: entry by entry.  bfloat16: the read-out divides by |n . q|, a sum that may cancel to a small fraction of its
    terms, so q and k rounded to bfloat16 move single entries by several per cent where it does; the rows must agree in the
    root mean square, and no entry may be far off."""
    if dt == torch.float32:
        return close(got, want, dt, what)
    got, want = got.float().cpu(), want.float().cpu()
    assert torch.isfinite(got).all(), f"{what}: non-finite values"
    err = (got - want).pow(2).mean().sqrt() / want.pow(2).mean().sqrt()
    assert err <= 6e-2, f"{what}: relative root-mean-square error {err:.3e}"
    assert (got - want).abs().max() <= 0.25 * want.abs().max(), f"{what}: an entry is far off"


def memory_cfg(p):
    return dict(heads=p["num_heads"], dim=p["dim"], vdim=p["vdim"], gate_cap=p["gate_cap"] or 1e9)


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("params", MEMORIES)
def test_matrix_memory_whole_in_portions_and_token_by_token(dt, params):
    rt = rt_for(dt)
    hidden, T = 24, 150
    mixer = build("mixer", "matrix_memory", hidden_size=hidden, eps=1e-5, **params)
    # gates of both signs and sizes: the running maximum rises with large input gates and falls with the forget gates
    H = params["num_heads"]
    g = torch.Generator().manual_seed(1)
    W = bind_random(mixer, rt, 10, {"i": torch.randn(H, hidden, generator=g) * 1.5, "f": torch.randn(H, hidden, generator=g),
                                    "f.b": torch.randn(H, generator=g) + 1.0})
    x = inputs(T, hidden, 3, dt)
    want = pz.matrix_memory(x, W, "p.", memory_cfg(params), 1e-5)
    h = Harness(mixer, rt)
    close_memory(run_in_portions(h, x, [T]), want, dt, "whole")
    close_memory(run_in_portions(h, x, [9, 2, 70, 1, 1, 64, 2, 1]), want, dt, "portions")
    close_memory(run_in_portions(h, x, [129, 21]), want, dt, "a portion of two chunks and one token")
    close_memory(run_in_portions(h, x, [1] * T), want, dt, "token by token")


@pytest.mark.parametrize("dt", DTYPES)
def test_matrix_memory_first_tokens_batches_and_a_far_token(dt):
    """Forget gates close to 1 keep an early token for hundreds of tokens; the first tokens of a sequence run on the
    running maximum's start value (0: the normalizer's floor exp(-m) is 1 there)."""
    rt = rt_for(dt)
    hidden = 32
    params = dict(num_heads=2, dim=32, vdim=32, gate_cap=15.0)
    mixer = build("mixer", "matrix_memory", hidden_size=hidden, eps=1e-5, **params)
    g = torch.Generator().manual_seed(1)        # (a draw for which the early token's input gate opens)
    W = bind_random(mixer, rt, 11, {"f": torch.randn(2, hidden, generator=g) * 0.1, "f.b": torch.full((2,), 7.0),
                                    "i": torch.randn(2, hidden, generator=g) * 0.3, "i.b": torch.full((2,), -2.0)})
    m = memory_cfg(params)
    xs = [inputs(n, hidden, 30 + i, dt) for i, n in enumerate((300, 7, 64))]
    xs[0][3] *= 8.0
    wants = [pz.matrix_memory(x, W, "p.", m, 1e-5) for x in xs]
    quiet = xs[0].clone()
    quiet[3] /= 8.0
    assert (pz.matrix_memory(quiet, W, "p.", m, 1e-5)[-1] - wants[0][-1]).abs().max() > 0.05 * wants[0][-1].abs().max()
    h = Harness(mixer, rt, pages=32, slots=3)
    rcs = [h.new() for _ in xs]
    a = h.step([(rcs[0], xs[0][:250]), (rcs[1], xs[1][:6]), (rcs[2], xs[2][:63])])
    b = h.step([(rcs[1], xs[1][6:]), (rcs[0], xs[0][250:]), (rcs[2], xs[2][63:])])
    close_memory(torch.cat([a[0], b[1]]), wants[0], dt, "long request")
    close_memory(torch.cat([a[1], b[0]]), wants[1], dt, "short request")
    close_memory(torch.cat([a[2], b[2]]), wants[2], dt, "third request")


# ----------------------------------------------------------------------------------------------- softmax attention

BIASED = [dict(num_heads=4, num_kv_heads=2, dim=32, vdim=32, scale=0.2, q_temp=(0.5, 7), rel_bias=(8, 20.0)),
          dict(num_heads=3, num_kv_heads=3, dim=16, vdim=48, scale=0.3, q_temp=None, rel_bias=(32, 64.0)),        # a bucket border that is a whole number
          dict(num_heads=6, num_kv_heads=1, dim=64, vdim=32, scale=0.11, q_temp=(2.0, 1), rel_bias=(6, 90.5)),
          dict(num_heads=2, num_kv_heads=1, dim=128, vdim=128, scale=0.09, q_temp=(0.3, 40), rel_bias=(16, 33.0))]


def biased_part(hidden, p):
    return build("mixer", "gated_attention", hidden_size=hidden, eps=1e-5, rot_dims=0, rot_base=1.0, qk_norm="head", gate=False, bias=True,
                 head_temp=False, **p)


def biased_cfg(p):
    c = dict(heads=p["num_heads"], kv_heads=p["num_kv_heads"], dim=p["dim"], vdim=p["vdim"], scale=p["scale"], bias_max=p["rel_bias"][1])
    if p["q_temp"]:
        c["q_temp"] = dict(coef=p["q_temp"][0], every=p["q_temp"][1])
    return c


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("params", BIASED)
def test_biased_attention_whole_in_portions_and_token_by_token(dt, params):
    rt = rt_for(dt)
    hidden, T = 40, 100
    mixer = biased_part(hidden, params)
    W = bind_random(mixer, rt, 12)
    x = inputs(T, hidden, 3, dt)
    want = pz.biased_attention(x, W, "p.", biased_cfg(params), 1e-5)
    h = Harness(mixer, rt, pages=10)
    close(run_in_portions(h, x, [T]), want, dt, "whole")
    close(run_in_portions(h, x, [23, 2, 30, 1, 1, 20, 2, 21]), want, dt, "portions")        # pages were used before
    close(run_in_portions(h, x, [1] * T), want, dt, "token by token")
    assert h.manager.num_free(0) == 9


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("decode", [False, True])
def test_the_bias_alone_picks_the_keys_of_one_bucket(dt, decode):
    """Queries and keys are zero, so the scores are the bias; one row of the table towers above the others, and the output
    is the mean of the values whose distance falls into that row's bucket: a border that is one position off shows."""
    rt = rt_for(dt)
    hidden, p = 24, dict(num_heads=2, num_kv_heads=2, dim=16, vdim=16, scale=1.0, q_temp=(0.5, 16), rel_bias=(8, 40.0))
    zero = {n: torch.zeros(32, hidden) for n in ("q", "k")}
    zero.update({"q.b": torch.zeros(32), "k.b": torch.zeros(32)})
    T = 140
    x = inputs(T, hidden, 4, dt)
    for row in (0, 3, 4, 5, 6, 7):
        rel = torch.zeros(8, 2)
        rel[row] = 40.0
        mixer = biased_part(hidden, p)
        W = bind_random(mixer, rt, 13, dict(zero, rel=rel))
        want = pz.biased_attention(x, W, "p.", biased_cfg(p), 1e-5)
        h = Harness(mixer, rt, pages=16)
        got = run_in_portions(h, x, [100] + [1] * 40 if decode else [3, 97, 40])
        close(got, want, dt, f"bias row {row}")


WINDOWED = [dict(num_heads=4, num_kv_heads=2, dim=32, vdim=32, scale=0.2, rot_dims=8, rot_base=50.0, window=24, softcap=2.0),
            dict(num_heads=3, num_kv_heads=3, dim=16, vdim=48, scale=0.3, rot_dims=16, rot_base=1e4, window=16, softcap=0.0),
            dict(num_heads=6, num_kv_heads=1, dim=64, vdim=32, scale=0.5, rot_dims=0, rot_base=1e6, window=None, softcap=1.0),
            dict(num_heads=2, num_kv_heads=1, dim=128, vdim=96, scale=0.09, rot_dims=64, rot_base=1e3, window=1, softcap=30.0)]


def windowed_part(hidden, p, **more):
    return build("mixer", "gated_attention", hidden_size=hidden, eps=1e-5, rot_pairing="interleaved", qk_norm="projection", gate=True,
                 head_temp=False, sink=True, **dict(p, **more))


def windowed_cfg(p):
    c = dict(heads=p["num_heads"], kv_heads=p["num_kv_heads"], dim=p["dim"], vdim=p["vdim"], scale=p["scale"],
             rot=dict(base=p["rot_base"], dims=p["rot_dims"]))
    if p["window"]:
        c["mask"] = dict(size=p["window"])
    if p["softcap"]:
        c["softcap"] = p["softcap"]
    return c


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("params", WINDOWED)
def test_windowed_attention_whole_in_portions_and_token_by_token(dt, params):
    rt = rt_for(dt)
    hidden, T = 40, 100
    mixer = windowed_part(hidden, params)
    W = bind_random(mixer, rt, 14, {"sink": torch.tensor([1.0, -0.5, 3.0, 0.0, 2.0, -4.0][:params["num_heads"]])})
    x = inputs(T, hidden, 5, dt)
    cfg = windowed_cfg(params)
    want = pz.windowed_attention(x, W, "p.", cfg, 1e-5)
    no_sink = {k: v for k, v in W.items() if k != "p.sink"}
    assert (pz.windowed_attention(x, no_sink, "p.", cfg, 1e-5) - want).abs().max() > 0.05 * want.abs().max(), "the sink must matter"
    h = Harness(mixer, rt, pages=10)
    close(run_in_portions(h, x, [T]), want, dt, "whole")
    close(run_in_portions(h, x, [23, 2, 30, 1, 1, 20, 2, 21]), want, dt, "portions")
    close(run_in_portions(h, x, [1] * T), want, dt, "token by token")


STANDOUT = dict(num_heads=2, num_kv_heads=2, dim=16, vdim=16, scale=1.5, rot_dims=0, rot_base=1e4, window=24, softcap=40.0)
STANDOUT_PAIRS = ((70, 47), (70, 46), (71, 48), (95, 72), (95, 71), (23, 0), (24, 0), (24, 1), (200, 177), (200, 176), (200, 3), (40, 39))


def standout_case(hidden, query, planted, dt):
    """Inputs and weights for which the key at ``planted`` scores far above all others for the query at ``query``: W_k = -W_q
    and the planted input is minus the query's, so its key equals the query (the query's own key is its opposite), while its
    value is minus the query's own."""
    wq = torch.randn(32, hidden, generator=torch.Generator().manual_seed(1)) * hidden ** -0.5
    x = inputs(query + 1, hidden, 100 + query, dt)
    x[planted] = -x[query]
    return x, {"q": wq, "k": -wq, "q.norm": torch.ones(32), "k.norm": torch.ones(32), "sink": torch.zeros(2)}


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("decode", [False, True])
def test_a_key_that_stands_out_just_inside_and_just_outside_the_window(dt, decode):
    rt = rt_for(dt)
    mixer = windowed_part(32, STANDOUT)
    W = bind_random(mixer, rt, 15, standout_case(32, 1, 0, dt)[1])
    cfg = windowed_cfg(STANDOUT)
    for query, planted in STANDOUT_PAIRS:
        x, _ = standout_case(32, query, planted, dt)
        want = pz.windowed_attention(x, W, "p.", cfg, 1e-5)
        moved = x.clone()
        moved[planted] = inputs(1, 32, 999, dt)[0]
        seen = bool((want[query] - pz.windowed_attention(moved, W, "p.", cfg, 1e-5)[query]).abs().max() > 0.2 * want[query].abs().max())
        assert seen == (query - planted < 24), "the plain implementation disagrees with the window's rule"
        h = Harness(mixer, rt, pages=16)
        got = run_in_portions(h, x, [query, 1] if decode else ([5, query - 4] if query > 5 else [query + 1]))
        close(got[query], want[query], dt, f"query {query}, planted key {planted}")


# ----------------------------------------------------------------------------------------------- side by side

@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("kind", ["parallel", "parallel_2"])
def test_mixers_side_by_side_with_their_scales_under_the_layer_norm(dt, kind):
    from mini_inference_engine_b200.config import PartSpec
    rt = rt_for(dt)
    hidden, T, eps = 32, 90, 1e-5
    if kind == "parallel":
        left = dict(BIASED[0])
        right = dict(num_heads=4, num_kv_heads=2, dim=16, vdim=24, taps=3)
        branches = {"left": PartSpec("gated_attention", dict(hidden_size=hidden, eps=eps, rot_dims=0, rot_base=1.0, qk_norm="head", gate=False,
                                                             bias=True, head_temp=False, **left)),
                    "right": PartSpec("channel_delta", dict(hidden_size=hidden, eps=eps, **right))}
        m = dict(left=biased_cfg(left), right=dict(heads=4, kv_heads=2, dim=16, vdim=24, conv=3), left_scale=0.7, right_scale=-1.3)
    else:
        left = dict(WINDOWED[0])
        right = dict(num_heads=2, dim=16, vdim=40, gate_cap=6.0)
        branches = {"left": PartSpec("gated_attention", dict(hidden_size=hidden, eps=eps, rot_pairing="interleaved", qk_norm="projection",
                                                             gate=True, head_temp=False, sink=True, **left)),
                    "right": PartSpec("matrix_memory", dict(hidden_size=hidden, eps=eps, **right))}
        m = dict(left=windowed_cfg(left), right=memory_cfg(right), left_scale=0.7, right_scale=-1.3)
    mixer = build("mixer", "parallel", hidden_size=hidden, branches=branches, scales=(0.7, -1.3))
    W = bind_random(mixer, rt, 16)
    norm = build("norm", "layernorm", size=hidden, eps=eps)
    Wn = bind_random(norm, rt, 17, {"weight": torch.randn(hidden)})
    x = inputs(T, hidden, 6, dt)
    res0 = torch.randn(T, hidden)
    layer = dict(type=kind, mixer=m)
    mixed = pz.mixer(x, W, "p.", layer, eps)
    h = Harness(mixer, rt)
    from mini_inference_engine_b200.parts import Branches
    for portions in ([T], [7, 1, 70, 2, 10]):
        branches_out = run_in_portions(h, x, portions)                   # [T, 2, hidden]
        res = res0.clone().to(DEV)
        out = norm(Branches(tuple(branches_out[:, i].contiguous().to(DEV) for i in range(2)), coefs=mixer.scales), res)
        cmp = close_memory if kind == "parallel_2" else close
        cmp(res, res0 + mixed, dt, f"stream, portions {portions}")
        cmp(out, pz.layer_norm(res0 + mixed, Wn["p.weight"], eps), dt, f"normed, portions {portions}")
