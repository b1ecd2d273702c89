"""What of the Luluzen design runs without a GPU: reading and writing its config.json, the model's description as data
(tensor names, the run order of a repeated stretch with a cache per run, the needs of mixers side by side), refusals, the
bias table's buckets, and the plain implementation on a model from the random-weights mode."""
import json
import math
import os

import pytest
import torch

import plain_luluzen as pz

CFG = dict(architecture="Luluzen", vocab=90, width=24, norm=dict(eps=1e-5), logit_softcap=12.0, loop=dict(start=1, stop=3, times=2), layers=[
    dict(type="lightning", mlp=dict(kind="dense", ff=40), mixer=dict(heads=2, dim=16, vdim=8, decay=[0.9, 0.99])),
    dict(type="parallel", mlp=dict(kind="moe", router=dict(experts=3, top=2), expert=dict(ff=16, limit=1.5)), mixer=dict(
        left_scale=0.5, right_scale=2.0,
        left=dict(heads=4, kv_heads=2, dim=8, vdim=16, scale=0.3, bias_max=30, q_temp=dict(coef=0.25, every=4)),
        right=dict(heads=4, kv_heads=2, dim=8, vdim=12, conv=3))),
    dict(type="parallel_2", mlp=None, mixer=dict(
        left_scale=1.5, right_scale=0.25,
        left=dict(heads=2, kv_heads=1, dim=16, vdim=8, scale=0.2, softcap=10.0, mask=dict(size=20), rot=dict(base=100.0, dims=4)),
        right=dict(heads=3, dim=8, vdim=16, gate_cap=5.0))),
    dict(type="lightning", mlp=dict(kind="moe", router=dict(experts=2, top=1), expert=dict(ff=8, limit=1.0)),
         mixer=dict(heads=1, dim=8, vdim=8, decay=[0.5])),
])


def test_config_round_trip_and_tensor_names(tmp_path):
    from mini_inference_engine_b200.config import load_config
    from mini_inference_engine_b200.models import expected_tensors
    from mini_inference_engine_b200.weights import write_model_folder
    cfg = load_config(json.loads(json.dumps(CFG)))
    assert type(cfg).__name__ == "LuluzenConfig" and cfg.to_dict() == json.loads(json.dumps(CFG))
    spec = cfg.model_spec()
    names = {spec.aliases.get(n, n): tuple(t.shape) for n, t in expected_tensors(spec).items()}
    assert names["embed"] == (90, 24) and names["final.norm"] == (24,) and names["loop.in"] == (24, 48) and names["loop.step"] == (2, 24)
    assert names["l0.mix.q"] == (32, 24) and names["l0.mix.v"] == (16, 24) and names["l0.mix.norm"] == (16,) and names["l0.mlp.gate"] == (40, 24)
    assert names["l1.mix.left.q"] == (32, 24) and names["l1.mix.left.q.b"] == (32,) and names["l1.mix.left.k.norm"] == (8,)
    assert names["l1.mix.left.v"] == (32, 24) and names["l1.mix.left.rel"] == (-1, 4) and names["l1.mix.left.o"] == (24, 64)
    assert names["l1.mix.right.q.conv"] == (16, 3) and names["l1.mix.right.v"] == (48, 24) and names["l1.mix.right.norm"] == (12,)
    assert names["l1.mix.right.a2"][0] == 32 and names["l1.mix.right.g2"][0] == 48 and names["l1.mix.right.dt_bias"] == (32,)
    assert names["l1.mlp.router"] == (3, 24) and names["l1.mlp.e2.gate"] == (16, 24) and names["l1.mlp.e0.down"] == (24, 16)
    assert names["l2.mix.left.q.norm"] == (32,) and names["l2.mix.left.k.norm"] == (16,) and names["l2.mix.left.sink"] == (2,)
    assert names["l2.mix.left.g"] == (16, 24) and names["l2.mix.right.i"] == (3, 24) and names["l2.mix.right.f.b"] == (3,)
    assert names["l2.mix.right.norm"] == (48,) and names["l2.mix.right.o"] == (24, 48)
    assert "l2.norm2" not in names and not any(n.startswith("l2.mlp") for n in names)      # a layer without a feed-forward
    assert not any(".out" in n or ".temp" in n for n in names)
    # the random-weights mode writes the checkpoint's own names, and the plain implementation runs on them
    folder = write_model_folder(str(tmp_path / "m"), cfg, seed=1)
    from safetensors.torch import load_file
    W = load_file(os.path.join(folder, "model.safetensors"))
    assert set(W) == set(names)
    trace = []
    logits = pz.forward(CFG, {k: v.float() for k, v in W.items()}, [3, 1, 4, 1, 5, 9, 2, 6], trace)
    assert logits.shape == (8, 90) and torch.isfinite(logits).all() and logits.abs().max() <= 12.0 and len(trace) == 6


def test_run_order_gives_every_pass_its_own_cache():
    from mini_inference_engine_b200.config import load_config
    from mini_inference_engine_b200.models import DecoderModel
    from mini_inference_engine_b200.parts import KVNeed, Runtime, StateNeed
    from mini_inference_engine_b200.weights.random_init import random_state
    from mini_inference_engine_b200.models import expected_tensors
    cfg = load_config(json.loads(json.dumps(CFG)))
    assert cfg.run_plan() == pz.run_order(CFG) == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (3, None)]
    spec = cfg.model_spec()
    kinds = [spec.layers[e.layer].block for e in spec.run_order]
    assert kinds == ["prenorm_residual", "stream_mix_step", "prenorm_residual", "prenorm_residual", "stream_mix_step", "prenorm_residual",
                     "prenorm_residual", "prenorm_residual"]
    layer_runs = [e for e in spec.run_order if spec.layers[e.layer].block == "prenorm_residual"]
    assert [e.layer for e in layer_runs] == [0, 1, 2, 1, 2, 3] and len({e.cache for e in layer_runs}) == 6
    mixes = [spec.layers[e.layer].parts["mix"].params["index"] for e in spec.run_order if spec.layers[e.layer].block == "stream_mix_step"]
    assert mixes == [0, 1]
    state = {spec.aliases.get(n, n): t for n, t in random_state(expected_tensors(spec), 3).items()}
    model = DecoderModel(spec, state, Runtime("cpu", torch.float32))
    lay = model.cache_layout
    assert [(g.window, g.chunk) for g in lay.groups] == [(None, None), (20, None)]
    kv = sorted((k, n.num_kv_heads, n.head_dim, n.window) for k, (g, n) in lay.kv.items())
    assert kv == [((1, 0), 2, 16, None), ((2, 0), 1, 16, 20), ((3, 0), 2, 16, None), ((4, 0), 1, 16, 20)]
    shapes = {k: tuple(n.shape) for k, n in lay.state.items()}
    assert shapes[0] == (2, 8, 16) and shapes[5] == (1, 8, 8)
    assert shapes[((1, 1), 0)] == (4, 12, 8) and shapes[((1, 1), 1)] == (2, 16 + 16 + 48) and shapes[((3, 1), 0)] == (4, 12, 8)
    assert shapes[((2, 1), 0)] == (3, 17, 8) and shapes[((2, 1), 1)] == (3,) and shapes[((4, 1), 1)] == (3,)
    # without a repeated stretch nothing is mixed and nothing kept
    plain = json.loads(json.dumps(CFG))
    del plain["loop"]
    spec = load_config(plain).model_spec()
    assert [e.layer for e in spec.run_order] == [0, 1, 2, 3] and spec.embedding.params["keep_output"] is False
    assert "loop.in" not in expected_tensors(spec)


@pytest.mark.parametrize("edit,word", [
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c["layers"][0].update(type="conv"), "conv"),
    (lambda c: c["layers"][0]["mixer"].update(decay=[0.9]), "decays"),
    (lambda c: c["layers"][0]["mlp"].update(kind="routed"), "routed"),
    (lambda c: c["layers"][1]["mixer"]["left"].pop("bias_max"), "bias_max"),
    (lambda c: c["layers"][1]["mixer"].pop("left_scale"), "left_scale"),
    (lambda c: c["layers"][2]["mixer"]["right"].pop("dim"), "dim"),
    (lambda c: c["layers"][1]["mlp"]["expert"].pop("limit"), "limit"),
    (lambda c: c["loop"].update(stop=5), "loop"),
    (lambda c: c["loop"].update(times=0), "loop"),
])
def test_configurations_that_are_refused(edit, word):
    from mini_inference_engine_b200.config import ConfigError, load_config
    c = json.loads(json.dumps(CFG))
    edit(c)
    with pytest.raises(ConfigError, match=word):
        load_config(c)


def test_bias_table_by_distance_follows_the_bucket_rule():
    """The attention part turns the table by bucket into a table by distance once, when it is bound."""
    from mini_inference_engine_b200.config import PartSpec
    from mini_inference_engine_b200.parts import Runtime, build_part
    for rows, far in ((8, 20.0), (32, 64.0), (6, 90.5), (16, 9.0)):
        part = build_part("mixer", PartSpec("gated_attention", dict(hidden_size=8, num_heads=2, num_kv_heads=1, dim=4, vdim=4, scale=1.0,
                                                                     rot_dims=0, rot_base=1.0, eps=1e-5, qk_norm=False, head_temp=False,
                                                                     gate=False, rel_bias=(None, far))))
        assert part.tensor_specs()["rel"].shape == (-1, 2)
        tensors = {n: torch.zeros(s.shape if -1 not in s.shape else (rows, 2)) for n, s in part.tensor_specs().items()}
        tensors["rel"] = torch.arange(rows, dtype=torch.float32)[:, None].expand(rows, 2).contiguous()
        part.bind(tensors, Runtime("cpu", torch.float32))
        table = part.mods.dist_bias
        assert table.shape == (2, math.ceil(far) + 1)
        for n in range(table.shape[1] + 5):
            assert table[1, min(n, table.shape[1] - 1)] == pz.distance_bucket(n, rows, far), (rows, far, n)


def test_preset_and_the_benchmark_pair_of_equal_size():
    """The shipped tiny preset reads back, and bench.py's --design option builds a Luluzen and a Llama configuration of the
    same width, heads and number of layer runs, the feed-forward matrices a token goes through as large as Llama's three."""
    import importlib.util

    from mini_inference_engine_b200.config import load_preset, preset_names
    assert "tiny-luluzen" in preset_names()
    cfg = load_preset("tiny-luluzen")
    assert type(cfg).__name__ == "LuluzenConfig" and cfg.loop is not None
    assert {l["type"] for l in cfg.layers} == {"lightning", "parallel", "parallel_2"}
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("bench_for_test", os.path.join(root, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    for size in bench.DESIGN_SIZES.values():
        z, l = bench.luluzen_configs(size)
        assert z.width == l.hidden_size == size["width"] and len(z.run_plan()) == l.num_hidden_layers == size["layers"]
        assert {x["type"] for x in z.layers} == {"lightning", "parallel", "parallel_2"}
        mlp = z.layers[1]["mlp"]
        used = mlp["router"]["top"] * mlp["expert"]["ff"] * 3
        assert abs(used - 3 * l.intermediate_size) <= 0.05 * 3 * l.intermediate_size
        left = z.layers[1]["mixer"]["left"]
        assert left["heads"] == l.num_attention_heads and left["dim"] == l.head_dim
