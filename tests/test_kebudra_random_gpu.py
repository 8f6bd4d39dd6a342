"""Randomly drawn Kebudra configurations -- copies of the stream, layer order, head counts and groupings, key, value, latent
and expert sizes, taps, experts and top, layers that borrow keys and values, layers without a feed-forward -- each with
random weights, run through the model runner whole and in portions beside single tokens, against the plain implementation."""
import json
import random

import numpy as np
import pytest
import torch

import test_kebudra_engine_gpu as eng

pytestmark = pytest.mark.gpu


def draw(seed: int) -> dict:
    rng = random.Random(seed)
    width = rng.choice([32, 40, 64, 72, 96, 100])
    layers, own_kv = [], []
    for i in range(rng.randint(2, 5)):
        kind = rng.choice(["attention", "latent_attention", "channel_delta"])
        if kind == "attention":
            if own_kv and rng.random() < 0.45:
                src = rng.choice(own_kv)
                m = dict(layers[src]["mixer"], diff=round(rng.uniform(0.05, 0.8), 3), kv_from=src)
            else:
                kv = rng.choice([1, 2, 3])
                dim = rng.choice([8, 16, 24, 32, 48, 64])
                m = dict(heads=kv * rng.choice([1, 2, 3]), kv_heads=kv, dim=dim, vdim=rng.choice([8, 16, 32, 40, 64, 96]),
                         scale=dim ** -0.5, diff=round(rng.uniform(0.05, 0.8), 3))
                own_kv.append(i)
        elif kind == "latent_attention":
            dim, rot = rng.choice([8, 16, 32, 64]), rng.choice([4, 8, 16, 32])
            m = dict(heads=rng.choice([1, 2, 3, 5]), dim=dim, rot_dim=rot, vdim=rng.choice([8, 16, 24, 64]), q_rank=rng.randint(6, 48),
                     kv_rank=rng.randint(6, 64), scale=(dim + rot) ** -0.5, rot=dict(base=rng.choice([100.0, 1e4, 2.5e5]), dims=rot))
        else:
            kv = rng.choice([1, 2, 3])
            m = dict(heads=kv * rng.choice([1, 2]), kv_heads=kv, dim=rng.choice([8, 16, 32, 64, 96]), vdim=rng.choice([8, 16, 32, 48]),
                     conv=rng.randint(1, 5), decay_rank=rng.randint(2, 12), gate_rank=rng.randint(2, 12))
        mlp = None
        if rng.random() > 0.15:
            experts = rng.randint(1, 12)
            mlp = dict(kind="moe", expert=dict(ff=rng.choice([8, 12, 16, 24, 40])), router=dict(experts=experts, top=rng.randint(1, min(experts, 4))))
        layers.append(dict(type=kind, mixer=m, mlp=mlp))
    return dict(architecture="Kebudra", vocab=rng.randint(50, 300), width=width, streams=rng.choice([1, 2, 3, 4]),
                embedding=dict(scale=round(width ** 0.5, 4)), norm=dict(eps=rng.choice([1e-6, 1e-5])), layers=layers)


@pytest.mark.parametrize("seed,dtype_name", [(s, "float32") for s in range(12)] + [(s, "bfloat16") for s in (3, 7, 11)])
def test_a_drawn_configuration_whole_and_in_portions(seed, dtype_name, tmp_path):
    from mini_inference_engine_b200.config import load_config
    from mini_inference_engine_b200.weights import write_model_folder
    cfg = draw(seed)
    name = f"draw{seed}"
    eng.CONFIGS[name] = cfg
    try:
        folder = write_model_folder(str(tmp_path / name), load_config(json.loads(json.dumps(cfg))), seed=200 + seed)
        rng = random.Random(1000 + seed)
        reqs = {f"r{i}": [rng.randrange(cfg["vocab"]) for _ in range(n)] for i, n in enumerate((rng.randint(1, 120), rng.randint(17, 90), 33))}
        runner = eng.runner_for(name, folder, dtype_name, 320, 3)
        eng.check(name, folder, dtype_name, eng.run_schedule(runner, reqs, [[(rid, len(t))] for rid, t in reqs.items()]), reqs)
        # all three at once: a portion of each, then single tokens of one beside portions of the others, on reused pages and slots
        left, at, schedule = {r: len(t) for r, t in reqs.items()}, 0, []
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
