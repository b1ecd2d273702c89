"""Randomly drawn Luluzen configurations -- width, layer order, the repeated stretch, head counts and groupings, key and value
sizes, windows, rotated dimensions, caps, bias tables, taps, experts and top, layers without a feed-forward -- each with random
weights, run through the model runner whole and in portions beside single tokens, against the plain implementation."""
import json
import os
import random

import pytest
import torch

import test_luluzen_engine_gpu as eng

pytestmark = pytest.mark.gpu


def draw(seed: int) -> dict:
    rng = random.Random(seed)
    width = rng.choice([32, 40, 64, 72, 96, 128])
    layers = []
    for i in range(rng.randint(2, 5)):
        kind = rng.choice(["lightning", "parallel", "parallel_2"])
        if kind == "lightning":
            heads = rng.choice([1, 2, 3, 4])
            m = dict(heads=heads, dim=rng.choice([8, 16, 32, 48, 64, 128]), vdim=rng.choice([8, 16, 24, 32, 64, 80]),
                     decay=[rng.choice([1.0, 0.999, 0.97, 0.9, 0.6, 0.3]) for _ in range(heads)])
        else:
            kv = rng.choice([1, 2, 3])
            dim = rng.choice([16, 32, 48, 64, 96, 128])
            left = dict(heads=kv * rng.choice([1, 2, 4]), kv_heads=kv, dim=dim, vdim=rng.choice([16, 32, 40, 64, 80, 96, 128]),
                        scale=round(rng.uniform(0.7, 2.0) * dim ** -0.5, 5))
            if kind == "parallel":
                left["bias_max"] = rng.choice([20, 33, 64, 120, 500])
                if rng.random() < 0.7:
                    left["q_temp"] = dict(coef=round(rng.uniform(0.05, 1.0), 3), every=rng.choice([1, 5, 16, 64, 128]))
                rkv = rng.choice([1, 2, 3])
                right = dict(heads=rkv * rng.choice([1, 2]), kv_heads=rkv, dim=rng.choice([8, 16, 32, 64, 96]), vdim=rng.choice([8, 16, 32, 48]),
                             conv=rng.randint(1, 5))
            else:
                if rng.random() < 0.8:
                    left["mask"] = dict(size=rng.choice([1, 7, 16, 24, 33, 64, 96]))
                if rng.random() < 0.8:
                    left["rot"] = dict(base=rng.choice([100.0, 1e4, 2.5e5]), dims=rng.choice([d for d in (2, 8, 16, 24, 32, 64, 128) if d <= dim]))
                if rng.random() < 0.7:
                    left["softcap"] = rng.choice([2.0, 10.0, 20.0, 50.0])
                right = dict(heads=rng.choice([1, 2, 3, 4]), dim=rng.choice([8, 16, 32, 48, 64, 128]), vdim=rng.choice([8, 16, 32, 64, 72, 128]),
                             gate_cap=rng.choice([2.0, 8.0, 15.0, 30.0]))
            m = dict(left=left, right=right, left_scale=round(rng.uniform(0.3, 1.5), 2), right_scale=round(rng.uniform(0.3, 1.5), 2))
        mlp = None
        if rng.random() > 0.15:
            if rng.random() < 0.35:
                mlp = dict(kind="dense", ff=rng.choice([24, 40, 64, 100, 160]))
            else:
                experts = rng.randint(1, 12)
                mlp = dict(kind="moe", expert=dict(ff=rng.choice([8, 12, 16, 24, 40]), limit=rng.choice([0.5, 1.0, 2.0, 7.0])),
                           router=dict(experts=experts, top=rng.randint(1, min(experts, 4))))
        layers.append(dict(type=kind, mixer=m, mlp=mlp))
    cfg = dict(architecture="Luluzen", vocab=rng.randint(50, 300), width=width, norm=dict(eps=rng.choice([1e-6, 1e-5])), layers=layers)
    if rng.random() < 0.75:
        lo = rng.randrange(len(layers))
        cfg["loop"] = dict(start=lo, stop=rng.randint(lo + 1, len(layers)), times=rng.randint(1, 3))
    if rng.random() < 0.7:
        cfg["logit_softcap"] = rng.choice([5.0, 15.0, 30.0])
    return cfg


@pytest.mark.parametrize("seed,dtype_name", [(s, "float32") for s in range(14)] + [(s, "bfloat16") for s in (2, 5, 9, 12)])
def test_a_drawn_configuration_whole_and_in_portions(seed, dtype_name, tmp_path):
    from safetensors.torch import load_file, save_file
    from mini_inference_engine_b200.config import load_config
    from mini_inference_engine_b200.weights import write_model_folder
    cfg = draw(seed)
    name = f"draw{seed}"
    eng.CONFIGS[name] = cfg
    try:
        folder = write_model_folder(str(tmp_path / name), load_config(json.loads(json.dumps(cfg))), seed=300 + seed)
        rng = random.Random(2000 + seed)
        path = os.path.join(folder, "model.safetensors")
        tensors = load_file(path)
        for k in [k for k in tensors if k.endswith(".rel")]:           # bias tables of other sizes than the random-weights mode's
            g = torch.Generator().manual_seed(seed)
            tensors[k] = torch.randn(rng.choice([4, 8, 16, 32, 38]), tensors[k].shape[1], generator=g).to(tensors[k].dtype)
        save_file(tensors, path)
        reqs = {f"r{i}": [rng.randrange(cfg["vocab"]) for _ in range(n)] for i, n in enumerate((rng.randint(1, 140), rng.randint(17, 90), 33))}
        runner = eng.runner_for(name, folder, dtype_name, 320, 3)
        eng.check(name, folder, dtype_name, eng.run_schedule(runner, reqs, [[(rid, len(t))] for rid, t in reqs.items()]), reqs)
        # all three at once: a portion of each, then single tokens of one beside portions of the others, on reused pages and slots
        left, schedule = {r: len(t) for r, t in reqs.items()}, []
        while any(left.values()):
            step = []
            for r in reqs:
                if left[r]:
                    n = min(left[r], rng.choice([1, 1, 2, 9, 16, 31]))
                    step.append((r, n))
                    left[r] -= n
            schedule.append(step)
        eng.check(name, folder, dtype_name, eng.run_schedule(runner, reqs, schedule), reqs)
    finally:
        eng.CONFIGS.pop(name, None)
        eng._models.pop((name, dtype_name), None)
        for k in [k for k in eng._plain if k[0] == name]:
            eng._plain.pop(k)
        for k in [k for k in eng._margins if k[0] == name]:
            eng._margins.pop(k)
