"""What of the Getizen design runs without a GPU: reading and writing its config.json, the model's description as
data and its tensor names, refusals, the frequencies' rescaling, the cache manager's handling of a block of
positions, and the needs of a mixer made of two."""
import json
import os

import pytest
import torch

import plain_getizen as pg

CFG = dict(architecture="Getizen", vocab=90, width=24, postln_alpha=1.25, norm=dict(eps=1e-5, groups=3), layers=[
    dict(type="parallel", mlp=dict(kind="dense", ff=40, limit=1.5), mixer=dict(
        left=dict(heads=4, kv_heads=2, dim=8, vdim=16, scale=0.3, mask=dict(size=20),
                  rot=dict(base=100.0, dims=4, scaling=dict(factor=2.0, low=1.0, high=4.0, original=16))),
        right=dict(width=32, blocks=4, conv=3))),
    dict(type="retention", mlp=None, mixer=dict(heads=2, dim=16, vdim=8, decay=[0.9, 0.99], rot=dict(base=50.0, dims=16))),
])


def test_config_round_trip_and_tensor_names(tmp_path):
    from mini_inference_engine_b200.config import load_config
    from mini_inference_engine_b200.models import expected_tensors
    from mini_inference_engine_b200.weights import write_model_folder
    cfg = load_config(json.loads(json.dumps(CFG)))
    assert type(cfg).__name__ == "GetizenConfig" and cfg.to_dict() == json.loads(json.dumps(CFG))
    spec = cfg.model_spec()
    names = {spec.aliases.get(n, n): tuple(t.shape) for n, t in expected_tensors(spec).items()}
    assert names["embed"] == (90, 24) and names["embed.norm"] == (24,) and names["final.norm"] == (24,)
    assert names["l0.mix.left.q"] == (32, 24) and names["l0.mix.left.k"] == (16, 24) and names["l0.mix.left.v"] == (32, 24)
    assert names["l0.mix.left.g"] == (64, 24) and names["l0.mix.left.o"] == (24, 64) and names["l0.mix.left.temp"] == (4,)
    assert names["l0.mix.left.q.norm"] == (32,) and names["l0.mix.left.k.norm"] == (16,)
    assert names["l0.mix.right.ra"] == (4, 8, 8) and names["l0.mix.right.conv"] == (32, 3) and names["l0.mix.right.lam"] == (32,)
    assert names["l0.mix.left.out"] == (24,) and names["l0.mix.right.out"] == (24,)
    assert names["l0.mlp.gate"] == (40, 24) and names["l0.norm2"] == (24,)
    assert names["l1.mix.q"] == (32, 24) and names["l1.mix.v"] == (16, 24) and names["l1.mix.o"] == (24, 16)
    assert "l1.norm2" not in names and not any(n.startswith("l1.mlp") for n in names)      # a layer without a feed-forward
    # the random-weights mode writes the checkpoint's own names, and the plain implementation runs on them
    folder = write_model_folder(str(tmp_path / "m"), cfg, seed=1)
    from safetensors.torch import load_file
    W = load_file(os.path.join(folder, "model.safetensors"))
    assert set(W) == set(names)
    logits = pg.forward(CFG, {k: v.float() for k, v in W.items()}, [3, 1, 4, 1, 5, 9, 2, 6])
    assert logits.shape == (8, 90) and torch.isfinite(logits).all()


@pytest.mark.parametrize("edit,word", [
    (lambda c: c.pop("postln_alpha"), "postln_alpha"),
    (lambda c: c["layers"][0].update(type="conv"), "conv"),
    (lambda c: c["layers"][1]["mixer"].update(decay=[0.9]), "decays"),
    (lambda c: c["layers"][0]["mlp"].update(kind="routed"), "routed"),
    (lambda c: c["norm"].update(groups=5), "groups"),
    (lambda c: c["layers"][0]["mixer"]["right"].pop("blocks"), "blocks"),
])
def test_configurations_that_are_refused(edit, word):
    from mini_inference_engine_b200.config import ConfigError, load_config
    c = json.loads(json.dumps(CFG))
    edit(c)
    with pytest.raises(ConfigError, match=word):
        load_config(c)


def test_frequencies():
    from mini_inference_engine_b200.parts.rope import rotary_frequencies
    for rot in (dict(base=1e4, dims=64), dict(base=30.0, dims=16, scaling=dict(factor=4.0, low=1.0, high=8.0, original=32)),
                dict(base=5e5, dims=128, scaling=dict(factor=8.0, low=1.0, high=4.0, original=8192))):
        assert torch.allclose(rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling")), pg.frequencies(rot), rtol=1e-6, atol=0)


def test_pages_behind_the_newest_block_of_positions_go_back():
    from mini_inference_engine_b200.cache.manager import RELEASED, CacheManager, GroupSpec, RequestCache
    m = CacheManager([GroupSpec("chunk40", None, 40)], 12, 16, 2)
    rc = RequestCache()
    assert m.reserve(rc, 39)
    assert m.advance(rc, 39) == [[]]                      # the next query (39) still reads from position 0
    first_two = rc.tables[0][:2]
    assert m.reserve(rc, 1) and m.advance(rc, 1) == [first_two]
    # position 40 opens a new block: pages 0 and 1 (positions 0 - 31) hold nothing it reads, page 2 (32 - 47) does
    assert rc.tables[0][:2] == [RELEASED, RELEASED] and rc.tables[0][2] != RELEASED
    assert m.reserve(rc, 50)                              # a portion that crosses the next edge (80) keeps what its first query reads
    held = list(rc.tables[0])
    m.advance(rc, 50)                                     # 90 computed: the next query reads from 80 = page 5
    assert rc.tables[0][:5] == [RELEASED] * 5 and rc.tables[0][5] == held[5]
    m.free(rc)
    m.check()
    assert m.num_free(0) == 11


def test_needs_of_a_mixer_made_of_two():
    from mini_inference_engine_b200.cache.storage import CacheLayout
    from mini_inference_engine_b200.parts import KVNeed, StateNeed
    lay = CacheLayout.from_needs({0: StateNeed((2, 8, 16)), 1: (KVNeed(2, 16, None, 20), StateNeed((3, 32))),
                                  2: (KVNeed(2, 16, None, 20), StateNeed((3, 32))), 3: KVNeed(1, 32, 8, None)})
    assert [(g.window, g.chunk) for g in lay.groups] == [(None, 20), (8, None)]
    assert lay.composite == {1: 2, 2: 2} and lay.kv[(1, 0)][0] == 0 and lay.kv[3][0] == 1
    assert set(lay.state) == {0, (1, 1), (2, 1)}
    assert KVNeed(2, 16, None, 20).mask() == -20 and KVNeed(2, 16, 8).mask() == 8 and KVNeed(2, 16).mask() == 0


def test_preset_and_the_benchmark_pair_of_equal_size():
    """The shipped tiny preset reads back, and bench.py's --design option builds a Getizen and a Llama configuration of
    the same width, feed-forward, heads and number of layers."""
    import importlib.util

    from mini_inference_engine_b200.config import load_preset, preset_names
    assert "tiny-getizen" in preset_names()
    cfg = load_preset("tiny-getizen")
    assert [l["type"] for l in cfg.layers] == ["parallel", "retention", "parallel"] and cfg.norm_groups == 3
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("bench_for_test", os.path.join(root, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    for size in bench.DESIGN_SIZES.values():
        g, l = bench.design_configs(size)
        assert g.width == l.hidden_size == size["width"] and len(g.layers) == l.num_hidden_layers == size["layers"]
        par = next(x for x in g.layers if x["type"] == "parallel")
        assert par["mlp"]["ff"] == l.intermediate_size and par["mixer"]["left"]["heads"] == l.num_attention_heads
        assert par["mixer"]["left"]["kv_heads"] == l.num_key_value_heads and par["mixer"]["left"]["dim"] == l.head_dim
