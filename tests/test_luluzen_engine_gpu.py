"""Whole Luluzen models against the plain implementation (``plain_luluzen``): small configurations made here, with random
weights from the package's random-weights mode, run through the model runner (the step function, cache manager and kernels
of generation) whole, with the last tokens one by one, in portions down to two tokens, and as mixed batches with so few
pages and state slots that they are used again; then through ``bin/trace_run`` and through the engine's own entry point with
its scheduler."""
import json
import os
import random

import numpy as np
import pytest
import torch

import plain_luluzen as pz
from conftest import plain_weights
from replay_driver import Replay
from test_getizen_engine_gpu import run_schedule

pytestmark = pytest.mark.gpu
DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
# relative error of a row of logits (root mean square of the difference over that of the row).  float32: the order of sums.
# bfloat16: activations are rounded between kernels; the plain implementation rounds nothing.
TOL = {"float32": 3e-4, "bfloat16": 0.08}


def lightning(heads, dim, vdim, decay):
    return dict(type="lightning", mixer=dict(heads=heads, dim=dim, vdim=vdim, decay=decay))


def parallel(left, right, ls, rs):
    return dict(type="parallel", mixer=dict(left=left, right=right, left_scale=ls, right_scale=rs))


def parallel_2(left, right, ls, rs):
    return dict(type="parallel_2", mixer=dict(left=left, right=right, left_scale=ls, right_scale=rs))


def biased(heads, kv_heads, dim, vdim, far, temp=None):
    d = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=dim ** -0.5, bias_max=far)
    if temp:
        d["q_temp"] = dict(coef=temp[0], every=temp[1])
    return d


def windowed(heads, kv_heads, dim, vdim, window, rot, softcap=None):
    d = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=1.7 * dim ** -0.5)
    if window:
        d["mask"] = dict(size=window)
    if rot:
        d["rot"] = dict(base=rot[0], dims=rot[1])
    if softcap:
        d["softcap"] = softcap
    return d


def delta(heads, kv_heads, dim, vdim, conv):
    return dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=conv)


def memory(heads, dim, vdim, cap):
    return dict(heads=heads, dim=dim, vdim=vdim, gate_cap=cap)


def dense(ff):
    return dict(kind="dense", ff=ff)


def moe(experts, top, ff, limit):
    return dict(kind="moe", router=dict(experts=experts, top=top), expert=dict(ff=ff, limit=limit))


def with_mlp(layer, mlp):
    return dict(layer, mlp=mlp)


CONFIGS = {
    # the repeated stretch lies in the middle (layers 1 and 2, twice); two experts a token; a window that is no multiple of a
    # page; a layer without a feed-forward; three query heads a key head; key and value sizes differ everywhere
    "z_a": dict(architecture="Luluzen", vocab=150, width=48, norm=dict(eps=1e-5), logit_softcap=9.0, loop=dict(start=1, stop=3, times=2), layers=[
        with_mlp(lightning(2, 32, 16, [0.9, 0.995]), dense(64)),
        with_mlp(parallel(biased(6, 2, 16, 32, 20.0, (0.5, 9)), delta(4, 2, 16, 24, 3), 0.7, 1.3), moe(5, 2, 24, 1.0)),
        with_mlp(parallel_2(windowed(2, 2, 32, 16, 24, (30.0, 8), 5.0), memory(3, 16, 40, 4.0), 1.2, 0.5), None),
        with_mlp(lightning(3, 16, 48, [0.999, 0.5, 1.0]), moe(4, 1, 16, 0.5))]),
    # no repeated stretch, no cap on the logits; heads of 64 (in bfloat16 the tensor-core kernels); a window of exactly a page; no
    # temperature; a convolution of one tap; every expert for every token; one head
    "z_b": dict(architecture="Luluzen", vocab=97, width=64, norm=dict(eps=1e-6), layers=[
        with_mlp(parallel_2(windowed(1, 1, 64, 64, 16, (500.0, 64)), memory(1, 64, 64, 15.0), 1.0, 1.0), moe(3, 3, 32, 2.0)),
        with_mlp(parallel(biased(4, 1, 64, 48, 40.0), delta(2, 2, 32, 32, 1), 0.6, 1.1), dense(96)),
        with_mlp(lightning(1, 64, 64, [0.98]), dense(96))]),
    # the whole model repeated three times; heads of 128 (in bfloat16: page copies by TMA in decoding); a matrix memory with two
    # value columns a thread; no rotation, no window, no cap on the scores
    "z_c": dict(architecture="Luluzen", vocab=211, width=80, norm=dict(eps=1e-5), logit_softcap=30.0, loop=dict(start=0, stop=2, times=3), layers=[
        with_mlp(parallel_2(windowed(2, 1, 128, 128, None, None), memory(2, 128, 128, 50.0), 0.8, 0.9), moe(8, 1, 24, 2.0)),
        with_mlp(parallel(biased(2, 1, 128, 96, 100.0, (0.25, 32)), delta(3, 1, 24, 40, 4), 1.0, 0.5), None)]),
}
LENGTHS = {"z_a": [5, 77, 130, 2, 49, 24, 25], "z_b": [1, 70, 33, 129, 16, 17, 64], "z_c": [3, 100, 47, 150, 48, 49, 9]}
BIAS_ROWS = {"z_a": 8, "z_b": 32, "z_c": 6}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    from safetensors.torch import load_file, save_file
    from mini_inference_engine_b200.config import load_config
    from mini_inference_engine_b200.weights import write_model_folder
    out = {}
    for i, (name, c) in enumerate(CONFIGS.items()):
        d = str(tmp_path_factory.mktemp(name))
        write_model_folder(d, load_config(json.loads(json.dumps(c))), seed=60 + i)
        with open(os.path.join(d, "config.json")) as f:
            assert json.load(f) == json.loads(json.dumps(c)), "the configuration must survive writing and reading"
        # the rows of a bias table are in no key of the configuration: the model reads them from the tensor
        path = os.path.join(d, "model.safetensors")
        tensors = load_file(path)
        for k in [k for k in tensors if k.endswith(".rel")]:
            g = torch.Generator().manual_seed(7)
            tensors[k] = torch.randn(BIAS_ROWS[name], tensors[k].shape[1], generator=g).to(tensors[k].dtype)
        save_file(tensors, path)
        out[name] = d
    return out


def requests_for(name, seed=0):
    rng = random.Random(seed)
    return {f"r{i}": [rng.randrange(CONFIGS[name]["vocab"]) for _ in range(n)] for i, n in enumerate(LENGTHS[name])}


_plain: dict = {}


def plain_logits(name, folder, tokens):
    key = (name, tuple(tokens))
    if key not in _plain:
        _plain[key] = pz.forward(CONFIGS[name], plain_weights(folder), tokens)
    return _plain[key]


_models: dict = {}


def model_for(name, folder, dtype_name):
    from mini_inference_engine_b200.models import load_model
    key = (name, dtype_name)
    if key not in _models:
        _models[key] = load_model(folder, DTYPES[dtype_name], "cuda:0")[1]
    return _models[key]


def runner_for(name, folder, dtype_name, max_tokens, slots):
    from mini_inference_engine_b200.engine.runner import ModelRunner
    return ModelRunner(model_for(name, folder, dtype_name), -(-max_tokens // 16) + 1, 16, slots)


_margins: dict = {}


def plain_margins(name, folder, tokens):
    key = (name, tuple(tokens))
    if key not in _margins:
        _margins[key] = pz.choice_margins(CONFIGS[name], plain_weights(folder), tokens).numpy()
    return _margins[key]


def check(name, folder, dtype_name, got, reqs):
    """got[id][position] = logits row; every position of every request must be there and, in float32, close to the plain row.
    In bfloat16 two things move single rows of models this small far: a router whose best scores lie close together chooses
    another expert than the unrounded plain implementation (positions where the plain choice hung on a score gap under 0.05
    are not compared), and the first positions of a sequence, where the matrix memory's read-out is small beside the norm's
    eps and a per cent of difference in the input comes out eightfold in the plain implementation too; rows that follow
    such a token read its keys, values and states.  (In float32 the same holds for a gap under 1e-4: a request is compared up to
    its first such position.)  So in bfloat16 the typical row must be close (the median error under
    half the bound) and at most three rows in ten may be beyond the bound."""
    bad, errs = [], []
    for rid, toks in reqs.items():
        assert sorted(got[rid]) == list(range(len(toks))), f"{rid}: positions missing"
        want = plain_logits(name, folder, toks).numpy()
        margins = plain_margins(name, folder, toks)
        sure = margins >= 0.05
        if dtype_name == "float32":            # a choice that hangs on a gap of the size of float32's rounding may fall the other way, and
            sure = np.ones(len(toks), dtype=bool)      # the tokens behind read that token's keys, values and states: compared up to it
            close_calls = np.nonzero(margins < 1e-4)[0]
            if close_calls.size:
                sure[close_calls[0]:] = False
        for p in range(len(toks)):
            d = got[rid][p] - want[p]
            assert np.isfinite(d).all(), f"{name} {dtype_name} {rid}: position {p} is not finite"
            if not sure[p]:
                continue
            err = np.sqrt((d ** 2).mean()) / np.sqrt((want[p] ** 2).mean())
            errs.append(err)
            if err > TOL[dtype_name]:
                bad.append((rid, len(toks), p, p % 16, float(err)))
    allowed = 0 if dtype_name == "float32" else int(0.3 * len(errs))
    assert len(bad) <= allowed, (f"{name} {dtype_name}: {len(bad)} of {len(errs)} positions differ; first (request, length, position, page "
                                 f"offset, relative error): {bad[:6]}")
    assert np.median(errs) <= TOL[dtype_name] / 2, f"{name} {dtype_name}: median relative error {np.median(errs):.3e}"


CASES = [(n, d) for n in CONFIGS for d in DTYPES]


@pytest.mark.parametrize("name,dtype_name", CASES)
def test_whole_then_token_by_token_then_portions(name, dtype_name, folders):
    reqs = requests_for(name)
    runner = runner_for(name, folders[name], dtype_name, 192, 2)
    whole = [[(rid, len(t))] for rid, t in reqs.items()]
    check(name, folders[name], dtype_name, run_schedule(runner, reqs, whole), reqs)
    # most of a request in one step, its last tokens (up to 40: past the edges of every window) one by one
    decode = []
    for rid, t in reqs.items():
        tail = min(40, len(t) - 1)
        decode += ([[(rid, len(t) - tail)]] if len(t) > tail else []) + [[(rid, 1)]] * tail
    check(name, folders[name], dtype_name, run_schedule(runner, reqs, decode), reqs)
    rng = random.Random(1)
    portions = []
    for rid, t in reqs.items():
        left = len(t)
        while left:
            n = min(left, rng.choice([2, 2, 3, 5, 15, 16, 17, 31, 40, 1]))
            portions.append([(rid, n)])
            left -= n
    check(name, folders[name], dtype_name, run_schedule(runner, reqs, portions), reqs)


@pytest.mark.parametrize("name,dtype_name", CASES)
def test_mixed_batches_with_pages_and_slots_used_again(name, dtype_name, folders):
    """Up to three live requests: portions of some beside single tokens of others; the pool holds 208 positions and
    three state slots for seven requests, so both are used again, by requests of other lengths."""
    reqs = requests_for(name, seed=2)
    rng = random.Random(3)
    waiting, live, left, schedule = list(reqs), [], {r: len(t) for r, t in reqs.items()}, []
    held = lambda: sum(-(-(len(reqs[r]) - left[r]) // 16) * 16 for r in live)
    while waiting or live:
        while waiting and len(live) < 3 and held() + -(-len(reqs[waiting[0]]) // 16) * 16 + 16 * len(live) <= 208 - 16 * 3:
            live.append(waiting.pop(0))
        step = []
        for r in list(live):
            if rng.random() < 0.2 and len(live) > 1 and step:
                continue                                   # left out of this step, goes on later
            n = min(left[r], rng.choice([1, 1, 2, 7, 16, 33]))
            step.append((r, n))
            left[r] -= n
            if left[r] == 0:
                live.remove(r)
        schedule.append(step)
    assert any(len(s) == 3 for s in schedule) and any(len({n for _, n in s}) > 1 for s in schedule)
    runner = runner_for(name, folders[name], dtype_name, 416, 3)
    check(name, folders[name], dtype_name, run_schedule(runner, reqs, schedule), reqs)


@pytest.mark.parametrize("dtype_name", list(DTYPES))
def test_long_decoding_far_beyond_every_window_and_page(dtype_name, folders):
    name = "z_a"
    rng = random.Random(4)
    reqs = {"long": [rng.randrange(150) for _ in range(330)]}
    runner = runner_for(name, folders[name], dtype_name, 336, 1)
    check(name, folders[name], dtype_name, run_schedule(runner, reqs, [[("long", 3)]] + [[("long", 1)]] * 327), reqs)


@pytest.mark.parametrize("dtype_name", list(DTYPES))
def test_trace_replay_program(dtype_name, folders, tmp_path):
    name = "z_b"
    reqs = requests_for(name, seed=5)
    got = {}
    with Replay(folders[name], dtype_name, tmp_path / "out", max_tokens=448, vocab=CONFIGS[name]["vocab"]) as rp:
        ids = list(reqs)
        for a, b in zip(ids[0::2], ids[1::2] + [None]):
            ta, tb = reqs[a], reqs[b] if b else []
            ca = max(1, len(ta) // 2)
            first = [(a, ta[:ca], list(range(ca)))] + ([(b, tb, list(range(len(tb))))] if b else [])
            for (rid, toks, want), rows in zip(first, np.split(rp.step(first, end=[b] if b else []), [ca])):
                got.setdefault(rid, {}).update({p: rows[p] for p in want})
            if len(ta) > ca:
                rows = rp.step([(a, ta[ca:], list(range(len(ta) - ca)))], end=[a])
                got[a].update({ca + p: rows[p] for p in range(len(ta) - ca)})
    check(name, folders[name], dtype_name, got, reqs)


def plain_greedy(name, folder, prompt, n):
    ids = list(prompt)
    for _ in range(n):
        ids.append(int(plain_logits(name, folder, ids)[-1].argmax()))
    return ids[len(prompt):]


@pytest.mark.parametrize("name", list(CONFIGS))
def test_greedy_generation_through_the_engine(name, folders):
    """The engine's own entry point and scheduler, four ways: default (captured decode graphs), a token budget of 16
    (prompts go in portions beside decoding requests), no graphs, and a pool so small that requests are pushed out
    and recomputed (their state slots are cleared and used again).  float32: the plain implementation's tokens."""
    from mini_inference_engine_b200 import EngineConfig, LLMEngine, SamplingParams
    rng = random.Random(6)
    vocab = CONFIGS[name]["vocab"]
    prompts = [[rng.randrange(vocab) for _ in range(n)] for n in (5, 37, 20, 66, 2)]
    crowded = [[rng.randrange(vocab) for _ in range(n)] for n in (30, 29, 31, 5)]      # three of them outgrow seven pages together
    for overrides in (dict(), dict(max_num_batched_tokens=16), dict(use_cuda_graphs=False),
                      dict(num_blocks=8, max_num_seqs=3, max_num_batched_tokens=48)):
        ps = crowded if "num_blocks" in overrides else prompts
        want = [plain_greedy(name, folders[name], p, 12) for p in ps]
        eng = LLMEngine(folders[name], EngineConfig(max_model_len=128, **overrides), dtype=torch.float32, load_tokenizer=False,
                        verbose=False)
        outs = eng.generate(ps, SamplingParams(max_tokens=12, ignore_eos=True))
        assert [o.output_ids for o in outs] == want, f"{name} with {overrides}"
        if "num_blocks" in overrides:
            assert eng.scheduler.num_preemptions > 0
        eng.cache.check()


def test_greedy_generation_in_bfloat16_follows_the_plain_scores(folders):
    from mini_inference_engine_b200 import EngineConfig, LLMEngine, SamplingParams
    name = "z_b"
    rng = random.Random(7)
    prompts = [[rng.randrange(CONFIGS[name]["vocab"]) for _ in range(n)] for n in (9, 40)]
    eng = LLMEngine(folders[name], EngineConfig(max_model_len=128), dtype=torch.bfloat16, load_tokenizer=False, verbose=False)
    outs = eng.generate(prompts, SamplingParams(max_tokens=10, ignore_eos=True))
    for p, o in zip(prompts, outs):
        ids = list(p)
        for n, tok in enumerate(o.output_ids):
            row = plain_logits(name, folders[name], ids)[-1]
            assert row[tok] >= row.max() - 4 * TOL["bfloat16"] * row.pow(2).mean().sqrt(), f"output {n}: token {tok} is far from the plain top"
            ids.append(tok)


def test_command_line_generates_with_a_luluzen_folder(folders, capsys):
    from mini_inference_engine_b200.__main__ import main
    main(["generate", "--model", folders["z_a"], "--dtype", "float32", "--prompt-ids", "5,6,7", "--max-tokens", "4", "--ignore-eos",
          "--overrides", '{"num_blocks": 64, "max_model_len": 128}'])
    lines = [json.loads(l) for l in capsys.readouterr().out.splitlines() if l.startswith("{")]
    assert lines[0]["output_ids"] == plain_greedy("z_a", folders["z_a"], [5, 6, 7], 4)
