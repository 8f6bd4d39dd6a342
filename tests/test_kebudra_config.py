"""The Kebudra configuration on the CPU: what config.json turns into (parts, tensor names, run order, caches), sizes
that come from the checkpoint's tensors, and configurations that are refused."""
import copy
import json

import pytest
import torch

from mini_inference_engine_b200.config import ConfigError, load_config
from mini_inference_engine_b200.models import expected_tensors

BASE = dict(architecture="Kebudra", vocab=90, width=32, streams=2, embedding=dict(scale=4.0), norm=dict(eps=1e-5), layers=[
    dict(type="attention", mixer=dict(heads=4, kv_heads=2, dim=8, vdim=16, scale=0.3, diff=0.25),
         mlp=dict(kind="moe", expert=dict(ff=12), router=dict(experts=3, top=2))),
    dict(type="channel_delta", mixer=dict(heads=2, kv_heads=1, dim=8, vdim=8, conv=3), mlp=None),
    dict(type="latent_attention", mixer=dict(heads=2, dim=8, rot_dim=4, vdim=8, q_rank=6, kv_rank=10, scale=0.2, rot=dict(base=100.0, dims=4)),
         mlp=dict(kind="moe", expert=dict(ff=8), router=dict(experts=2, top=1))),
    dict(type="attention", mixer=dict(heads=4, kv_heads=2, dim=8, vdim=16, scale=0.3, diff=0.1, kv_from=0), mlp=None)])


def test_description_as_data():
    cfg = load_config(copy.deepcopy(BASE))
    assert cfg.to_dict() == BASE
    spec = cfg.model_spec()
    assert [l.block for l in spec.layers] == ["hyper_connected", "hyper_connected_mixer_only", "hyper_connected", "hyper_connected_mixer_only"]
    assert [l.mixer.kind for l in spec.layers] == ["differential_attention", "channel_delta", "latent_attention", "differential_attention"]
    assert spec.embedding.params["copies"] == 2 and spec.embedding.params["scale"] == 4.0
    # the last layer reads the first layer's keys and values and writes none
    assert [(e.layer, e.cache, e.writes_cache) for e in spec.run_order] == [(0, 0, True), (1, 1, True), (2, 2, True), (3, 0, False)]
    names = {spec.aliases.get(n, n): tuple(t.shape) for n, t in expected_tensors(spec).items()}
    assert names["embed"] == (90, 32) and names["head"] == (90, 32) and names["final.norm.alpha"] == ()
    assert names["l0.hc1.mix"] == (2, 2) and names["l0.hc2.in"] == (2,) and "l1.hc2.in" not in names and "l1.norm2" not in names
    assert names["l0.mix.q"] == (4 * 2 * 8, 32) and names["l0.mix.k"] == (2 * 2 * 8, 32) and names["l0.mix.v"] == (2 * 16, 32)
    assert names["l0.mix.g"] == (4, 32) and names["l0.mix.lq1"] == (8,)
    assert "l3.mix.k" not in names and "l3.mix.v" not in names and names["l3.mix.q"] == (64, 32)
    assert names["l2.mix.dkv"] == (14, 32) and names["l2.mix.uq"] == (2 * 12, 6) and names["l2.mix.dkv.norm"] == (10,)
    assert names["l1.mix.q.conv"] == (8, 3) and names["l1.mix.v"] == (16, 32) and names["l1.mix.dt_bias"] == (16,)
    assert names["l1.mix.a1"] == (-1, 32) and names["l1.mix.a2"] == (16, -1)          # the ranks come from the checkpoint
    assert names["l0.mlp.router"] == (3, 32) and names["l0.mlp.e2.up"] == (12, 32) and names["l2.mlp.e1.down"] == (32, 8)


def test_cache_needs_follow_the_mixers():
    from mini_inference_engine_b200.parts import KVNeed, StateNeed, build_part
    spec = load_config(copy.deepcopy(BASE)).model_spec()
    needs = [build_part("mixer", l.mixer).cache_need() for l in spec.layers]
    assert needs[0] == KVNeed(4, 16) == needs[3]                   # two maps: twice the key heads; pages as wide as the wider of key and value
    assert needs[2] == KVNeed(2, 16)                               # 8 plain + 4 rotated, rounded up to the kernels' step
    assert needs[1] == (StateNeed((2, 8, 8), torch.float32), StateNeed((2, 8 + 8 + 16), torch.float32))


def test_ranks_come_from_the_tensors(tmp_path):
    """A low-rank pair whose rank config.json does not give: any rank in the file is taken, a pair that does not fit is not."""
    from mini_inference_engine_b200.weights.loader import TensorSpec, WeightError, check_and_bind
    spec = {"a1": TensorSpec((-1, 32), "fan_in", (8, 32)), "a2": TensorSpec((16, -1), "fan_in", (16, 8))}
    ok = check_and_bind({"a1": torch.zeros(5, 32), "a2": torch.zeros(16, 5)}, spec)
    assert ok["a1"].shape == (5, 32)
    with pytest.raises(WeightError):
        check_and_bind({"a1": torch.zeros(5, 31), "a2": torch.zeros(16, 5)}, spec)
    from mini_inference_engine_b200.weights import write_model_folder
    from mini_inference_engine_b200.weights.safetensors_io import read_file
    d = write_model_folder(str(tmp_path / "m"), load_config(copy.deepcopy(BASE)), seed=1)
    t = read_file(d + "/model.safetensors")
    assert t["l1.mix.a1"].shape[0] == t["l1.mix.a2"].shape[1] >= 1 and t["l1.norm1.alpha"].shape == ()
    assert json.load(open(d + "/config.json")) == BASE


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][0].update(type="retention"), "not a mixer"),
    (lambda c: c["layers"][0]["mixer"].pop("diff"), "diff"),
    (lambda c: c["layers"][2]["mixer"]["rot"].pop("base"), "base"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=1), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=3), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].update(vdim=8), "differs"),
    (lambda c: c["layers"][1]["mixer"].update(kv_from=0), "only an attention layer"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "not a feed-forward"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=4), "top"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "do not divide"),
    (lambda c: c.update(streams=9), "streams"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_refused_configurations(change, word):
    c = copy.deepcopy(BASE)
    change(c)
    with pytest.raises(ConfigError, match=word):
        load_config(c)


def test_preset_and_the_benchmark_pair_of_equal_size():
    """The shipped tiny preset reads back, and bench.py's --design option builds a Kebudra and a Llama configuration of the
    same width, heads and number of layers, the feed-forward matrices a token goes through as large as Llama's three."""
    import importlib.util
    import os

    from mini_inference_engine_b200.config import load_preset, preset_names
    assert "tiny-kebudra" in preset_names()
    cfg = load_preset("tiny-kebudra")
    assert [l["type"] for l in cfg.layers] == ["latent_attention", "channel_delta", "attention", "attention"] and cfg.streams == 2
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("bench_for_test", os.path.join(root, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    for size in bench.DESIGN_SIZES.values():
        k, l = bench.kebudra_configs(size)
        assert k.width == l.hidden_size == size["width"] and len(k.layers) == l.num_hidden_layers == size["layers"]
        assert {x["type"] for x in k.layers} == {"latent_attention", "channel_delta", "attention"}
        mlp = k.layers[0]["mlp"]
        used = mlp["router"]["top"] * mlp["expert"]["ff"] * 2
        assert abs(used - 3 * l.intermediate_size) <= 0.05 * 3 * l.intermediate_size
        lat = next(x for x in k.layers if x["type"] == "latent_attention")["mixer"]
        assert lat["heads"] == l.num_attention_heads and lat["dim"] + lat["rot_dim"] == l.head_dim
