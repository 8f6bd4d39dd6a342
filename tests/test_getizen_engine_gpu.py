"""Whole Getizen models against the plain implementation (``plain_getizen``): small configurations made here, with
random weights from the package's random-weights mode, run through the model runner (the step function, cache
manager and kernels of generation) whole, with the last tokens one by one, in portions down to two tokens, and as
mixed batches with so few pages and state slots that they are used again; then through ``bin/trace_run`` and through
the engine's own entry point with its scheduler."""
import json
import os
import random

import numpy as np
import pytest
import torch

import plain_getizen as pg
from conftest import plain_weights
from replay_driver import Replay

pytestmark = pytest.mark.gpu
DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
# relative error of a row of logits (root mean square of the difference over that of the row).  float32: the order of
# sums.  bfloat16: activations are rounded between kernels and the post-norm layers pass the differences on at full
# size; the plain implementation rounds nothing.
TOL = {"float32": 3e-4, "bfloat16": 0.12}


def retention(heads, dim, vdim, decay, dims, base=1e4):
    return dict(type="retention", mixer=dict(heads=heads, dim=dim, vdim=vdim, decay=decay, rot=dict(base=base, dims=dims)))


def parallel(heads, kv_heads, dim, vdim, chunk, dims, width, blocks, conv, scaling=None, base=1e4):
    rot = dict(base=base, dims=dims)
    if scaling:
        rot["scaling"] = scaling
    return dict(type="parallel", mixer=dict(
        left=dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=dim ** -0.5, mask=dict(size=chunk), rot=rot),
        right=dict(width=width, blocks=blocks, conv=conv)))


def with_mlp(layer, ff, limit):
    return dict(layer, mlp=None if ff is None else dict(kind="dense", ff=ff, limit=limit))


CONFIGS = {
    # starts with a parallel layer; key and value sizes differ everywhere; a block of positions that is no multiple of a
    # page; three norm groups; one layer without a feed-forward; three query heads a key head
    "g_a": dict(architecture="Getizen", vocab=150, width=48, postln_alpha=1.5, norm=dict(eps=1e-5, groups=3), layers=[
        with_mlp(parallel(6, 2, 16, 32, 24, 8, 40, 5, 3, scaling=dict(factor=4.0, low=1.0, high=8.0, original=32), base=30.0), 64, 1.0),
        with_mlp(retention(2, 32, 16, [0.9, 0.995], 16), None, 0),
        with_mlp(parallel(2, 2, 32, 16, 40, 32, 64, 1, 2), 80, 0.5),
        with_mlp(retention(3, 16, 48, [0.999, 0.5, 1.0], 0), 56, 3.0)]),
    # one norm group, alpha 1, one head, heads of 64 (the tensor-core kernel for portions in bfloat16), a convolution of
    # one tap next to one of six
    "g_b": dict(architecture="Getizen", vocab=97, width=64, postln_alpha=1.0, norm=dict(eps=1e-6, groups=1), layers=[
        with_mlp(retention(1, 64, 64, [0.98], 64, base=500.0), 96, 2.0),
        with_mlp(parallel(1, 1, 64, 64, 64, 64, 64, 4, 1), 96, 2.0),
        with_mlp(parallel(4, 1, 64, 48, 16, 32, 32, 2, 6), None, 0)]),
    # heads of 128 (in bfloat16: page copies by TMA in decoding, the tcgen05 kernel for portions), retention with eight
    # threads a value column, a recurrence wider than the model, five norm groups
    "g_c": dict(architecture="Getizen", vocab=211, width=80, postln_alpha=2.0, norm=dict(eps=1e-5, groups=5), layers=[
        with_mlp(retention(2, 128, 64, [0.97, 0.999], 64), 48, 4.0),
        with_mlp(parallel(2, 1, 128, 128, 48, 128, 96, 3, 4, scaling=dict(factor=2.0, low=1.0, high=2.0, original=64), base=1e3), 112, 1.0)]),
}
LENGTHS = {"g_a": [5, 77, 130, 2, 49, 24, 25], "g_b": [1, 70, 33, 129, 16, 17, 64], "g_c": [3, 100, 47, 150, 48, 49, 9]}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    from mini_inference_engine_b200.config import load_config
    from mini_inference_engine_b200.weights import write_model_folder
    out = {}
    for i, (name, c) in enumerate(CONFIGS.items()):
        d = str(tmp_path_factory.mktemp(name))
        write_model_folder(d, load_config(json.loads(json.dumps(c))), seed=40 + i)
        with open(os.path.join(d, "config.json")) as f:
            assert json.load(f) == json.loads(json.dumps(c)), "the configuration must survive writing and reading"
        out[name] = d
    return out


def requests_for(name, seed=0):
    rng = random.Random(seed)
    return {f"r{i}": [rng.randrange(CONFIGS[name]["vocab"]) for _ in range(n)] for i, n in enumerate(LENGTHS[name])}


_plain: dict = {}


def plain_logits(name, folder, tokens):
    key = (name, tuple(tokens))
    if key not in _plain:
        _plain[key] = pg.forward(CONFIGS[name], plain_weights(folder), tokens)
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


def check(name, folder, dtype_name, got, reqs):
    """got[id][position] = logits row; every position of every request must be there and close to the plain row."""
    for rid, toks in reqs.items():
        assert sorted(got[rid]) == list(range(len(toks))), f"{rid}: positions missing"
        want = plain_logits(name, folder, toks).numpy()
        for p in range(len(toks)):
            d = got[rid][p] - want[p]
            assert np.isfinite(d).all(), f"{name} {dtype_name} {rid}: position {p} is not finite"
            err = np.sqrt((d ** 2).mean()) / np.sqrt((want[p] ** 2).mean())
            assert err <= TOL[dtype_name], (f"{name} {dtype_name} request {rid} (length {len(toks)}): first wrong position {p} "
                                            f"(page offset {p % 16}), relative error {err:.3e}")


def run_schedule(runner, reqs, schedule):
    """schedule: steps of [(request id, number of tokens)]; all logits are asked for; a request is freed when it ends."""
    from mini_inference_engine_b200.cache.manager import RequestCache
    from mini_inference_engine_b200.kernels import ops
    live, at, got = {}, {}, {}
    for step in schedule:
        entries = []
        for rid, n in step:
            rc = live.setdefault(rid, RequestCache())
            lo = at.get(rid, 0)
            entries.append((rc, reqs[rid][lo:lo + n], list(range(n))))
        logits = runner.run(entries).cpu().numpy()
        ops.check_range_errors()
        i = 0
        for rid, n in step:
            lo = at.get(rid, 0)
            for j in range(n):
                got.setdefault(rid, {})[lo + j] = logits[i]
                i += 1
            at[rid] = lo + n
            if at[rid] == len(reqs[rid]):
                runner.cache.free(live.pop(rid))
    runner.cache.check()
    return got


CASES = [(n, d) for n in CONFIGS for d in DTYPES]


@pytest.mark.parametrize("name,dtype_name", CASES)
def test_whole_then_token_by_token_then_portions(name, dtype_name, folders):
    reqs = requests_for(name)
    runner = runner_for(name, folders[name], dtype_name, 192, 2)
    whole = [[(rid, len(t))] for rid, t in reqs.items()]
    check(name, folders[name], dtype_name, run_schedule(runner, reqs, whole), reqs)
    # most of a request in one step, its last tokens (up to 40: past the edges of every block of positions) one by one
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
def test_long_decoding_far_beyond_every_block_and_page(dtype_name, folders):
    name = "g_a"
    rng = random.Random(4)
    reqs = {"long": [rng.randrange(150) for _ in range(330)]}
    runner = runner_for(name, folders[name], dtype_name, 336, 1)
    check(name, folders[name], dtype_name, run_schedule(runner, reqs, [[("long", 3)]] + [[("long", 1)]] * 327), reqs)


@pytest.mark.parametrize("dtype_name", list(DTYPES))
def test_trace_replay_program(dtype_name, folders, tmp_path):
    name = "g_b"
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
    name = "g_b"
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


def test_command_line_generates_with_a_getizen_folder(folders, capsys):
    from mini_inference_engine_b200.__main__ import main
    main(["generate", "--model", folders["g_a"], "--dtype", "float32", "--prompt-ids", "5,6,7", "--max-tokens", "4", "--ignore-eos",
          "--overrides", '{"num_blocks": 64, "max_model_len": 128}'])
    lines = [json.loads(l) for l in capsys.readouterr().out.splitlines() if l.startswith("{")]
    assert lines[0]["output_ids"] == plain_greedy("g_a", folders["g_a"], [5, 6, 7], 4)
