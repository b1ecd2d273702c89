"""The Serotar configuration on the CPU: what config.json turns into (parts, tensor names, caches and the embedding's own
state), optional keys that may be absent, configurations that are refused, the preset and the benchmark's pair."""
import copy
import json

import pytest
import torch

from mini_inference_engine_b200.config import ConfigError, load_config
from mini_inference_engine_b200.models import expected_tensors


def latent(heads, dim, vdim, q_rank, kv_rank, scale):
    return dict(heads=heads, dim=dim, vdim=vdim, q_rank=q_rank, kv_rank=kv_rank, scale=scale)


BASE = dict(architecture="Serotar", vocab=90, width=40, embedding=dict(scale=4.0, bigram=dict(buckets=61, mul_prev=11, mul_cur=3)),
            norm=dict(eps=1e-5), token_side=dict(dim=6), layers=[
    dict(type="latent_attention", mixer=latent(2, 8, 16, 12, 10, 0.3),
         mlp=dict(kind="moe", expert=dict(ff=12), router=dict(experts=4, top=2, identity=2, groups=dict(count=3, keep=2)), shared=dict(ff=20))),
    dict(type="latent_attention", mixer=latent(4, 16, 8, 10, 12, 0.25), mlp=None),
    dict(type="latent_attention", mixer=latent(1, 24, 24, 6, 6, 0.2), mlp=dict(kind="dense", ff=56))])


def names_of(spec):
    return {spec.aliases.get(n, n): tuple(t.shape) for n, t in expected_tensors(spec).items()}


def test_description_as_data():
    cfg = load_config(copy.deepcopy(BASE))
    assert cfg.to_dict() == BASE
    spec = cfg.model_spec()
    assert [l.block for l in spec.layers] == ["output_norm_residual"] * 3
    assert [l.parts["mixer"].kind for l in spec.layers] == ["latent_attention"] * 3
    assert [l.parts["feed_forward"].kind if "feed_forward" in l.parts else None for l in spec.layers] == ["routed_experts", None, "activated_mlp"]
    assert [(e.layer, e.cache, e.writes_cache) for e in spec.run_order] == [(0, 0, True), (1, 1, True), (2, 2, True)]
    e = spec.embedding.params
    assert (e["scale"], e["buckets"], e["mul_prev"], e["mul_cur"], e["side_width"], e["history"]) == (4.0, 61, 11, 3, 18, 4)
    m = spec.layers[0].parts["mixer"].params
    assert m["rot_dim"] == 0 and m["gate"] is False and m["scale"] == 0.3 and m["eps"] == 1e-5
    r = spec.layers[0].parts["feed_forward"].params
    assert (r["num_experts"], r["top"], r["identity"], r["groups"], r["keep"], r["gated"], r["score"], r["correction"]) == (4, 2, 2, 3, 2, True, "softmax", True)
    names = names_of(spec)
    assert names["embed"] == (90, 40) and names["bigram"] == (62, 40) and names["side.embed"] == (90, 18) and names["head"] == (90, 40)
    assert names["final.norm"] == () and names["l0.norm1"] == () and names["l0.norm2"] == () and "l1.norm2" not in names and "l1.ls2" not in names
    assert names["l0.ls1"] == (40,) and names["l2.ls2"] == (40,)
    assert [names[f"l{i}.dwa"] for i in range(3)] == [(2,), (3,), (4,)]
    assert names["l1.side.gate"] == (6, 40) and names["l1.side.proj"] == (40, 6) and names["l1.side.norm"] == (40,)
    assert names["l0.mix.dq"] == (12, 40) and names["l0.mix.dq.norm"] == (12,) and names["l0.mix.uq"] == (2 * 8, 12)
    assert names["l0.mix.dkv"] == (10, 40) and names["l0.mix.dkv.norm"] == (10,) and names["l0.mix.uk"] == (16, 10) and names["l0.mix.uv"] == (32, 10)
    assert names["l0.mix.o"] == (40, 32) and names["l1.mix.o"] == (40, 32) and "l0.mix.g" not in names
    assert names["l0.mlp.router"] == (6, 40) and names["l0.mlp.correction"] == (6,) and "l0.mlp.e4.up" not in names
    assert names["l0.mlp.e3.gate"] == (12, 40) and names["l0.mlp.e3.up"] == (12, 40) and names["l0.mlp.e3.down"] == (40, 12)
    assert names["l0.mlp.shared.gate"] == (20, 40) and names["l0.mlp.shared.down"] == (40, 20)
    assert names["l2.mlp.up"] == (56, 40) and names["l2.mlp.down"] == (40, 56) and names["l2.mlp.act"] == (2,)


def test_cache_needs_of_the_mixers_and_of_the_embedding():
    from mini_inference_engine_b200.parts import KVNeed, StateNeed, build_part
    spec = load_config(copy.deepcopy(BASE)).model_spec()
    needs = [build_part("mixer", l.parts["mixer"]).cache_need() for l in spec.layers]
    assert needs == [KVNeed(2, 16), KVNeed(4, 16), KVNeed(1, 32)]        # pages as wide as the wider of key and value, in steps of 16
    assert build_part("embedding", spec.embedding).cache_need() == StateNeed((1,), torch.int32)      # the token before a step


def test_optional_keys_may_be_absent(tmp_path):
    c = copy.deepcopy(BASE)
    c.pop("token_side")
    c["embedding"].pop("bigram")
    r = c["layers"][0]["mlp"]
    r.pop("shared")
    r["router"].pop("groups")
    r["router"].pop("identity")
    cfg = load_config(copy.deepcopy(c))
    assert cfg.to_dict() == c
    spec = cfg.model_spec()
    names = names_of(spec)
    assert "bigram" not in names and "side.embed" not in names and "l0.side.gate" not in names
    assert names["l0.mlp.router"] == (4, 40) and "l0.mlp.shared.up" not in names
    from mini_inference_engine_b200.weights import write_model_folder
    from mini_inference_engine_b200.weights.safetensors_io import read_file
    d = write_model_folder(str(tmp_path / "m"), cfg, seed=1)
    t = read_file(d + "/model.safetensors")
    assert t["l0.norm1"].shape == () and t["l2.dwa"].shape == (4,) and json.load(open(d + "/config.json")) == c


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][0].update(type="retention"), "not a mixer"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][1]["mixer"].update(heads=0), "positive"),
    (lambda c: c["layers"][2]["mlp"].update(kind="glu"), "not a feed-forward"),
    (lambda c: c["layers"][2]["mlp"].pop("ff"), "ff"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=7), "top"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "groups"),                # two kept groups hold four outputs
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=4), "groups"),    # six outputs in four groups
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(keep=4), "groups"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].pop("keep"), "keep"),
    (lambda c: c["layers"][0]["mlp"].pop("expert"), "expert"),
    (lambda c: c["embedding"]["bigram"].pop("mul_cur"), "mul_cur"),
    (lambda c: c["embedding"]["bigram"].update(buckets=0), "buckets"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c.update(layers=[]), "layers"),
])
def test_refused_configurations(change, word):
    c = copy.deepcopy(BASE)
    change(c)
    with pytest.raises(ConfigError, match=word):
        load_config(c)


def test_preset_and_the_benchmark_pair_of_equal_size():
    """The shipped tiny preset reads back, and bench.py's --design option builds a Serotar and a Llama configuration of the
    same width, heads and number of layers, the feed-forward matrices a token goes through as large as Llama's three."""
    import importlib.util
    import os

    from mini_inference_engine_b200.config import load_preset, preset_names
    assert "tiny-serotar" in preset_names()
    cfg = load_preset("tiny-serotar")
    assert [None if l["mlp"] is None else l["mlp"]["kind"] for l in cfg.layers] == ["dense", "moe", None, "moe"] and cfg.side_dim == 8
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("bench_for_test", os.path.join(root, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    for size in bench.DESIGN_SIZES.values():
        s, l = bench.serotar_configs(size)
        assert s.width == l.hidden_size == size["width"] and len(s.layers) == l.num_hidden_layers == size["layers"]
        assert [x["mlp"]["kind"] for x in s.layers] == ["dense"] + ["moe"] * (size["layers"] - 1)
        assert s.layers[0]["mlp"]["ff"] == l.intermediate_size
        mlp = s.layers[1]["mlp"]
        assert mlp["router"]["top"] * mlp["expert"]["ff"] + mlp["shared"]["ff"] == l.intermediate_size
        assert s.layers[0]["mixer"]["heads"] == l.num_attention_heads and s.layers[0]["mixer"]["dim"] == l.head_dim
        s.model_spec()
