"""Kebudra: a pre-norm decoder over a residual stream kept in several copies (hyper-connections), squashed by Dynamic
Tanh instead of normed, whose layers are listed one by one in config.json: differential attention (optionally over
another layer's keys and values), latent attention or a gated delta rule with per-channel decay as the mixer, and a
routed mixture of experts as the feed-forward.

config.json: ``architecture`` "Kebudra", ``vocab``, ``width``, ``streams``, ``embedding`` {scale}, ``norm`` {eps} and
``layers``, a list of {type, mixer, mlp}:

* type "attention": mixer {heads, kv_heads, dim, vdim, scale, diff, kv_from (optional: the layer whose keys and values
  this one reads)} -- parts.attention.DifferentialAttention;
* type "latent_attention": mixer {heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, rot {base, dims}} --
  parts.attention.LatentAttention;
* type "channel_delta": mixer {heads, kv_heads, dim, vdim, conv} -- parts.delta.ChannelDelta;
* mlp {kind "moe", expert {ff}, router {experts, top}} -- parts.feedforward.RoutedExperts -- or null.

Tensors: 'embed', 'head', 'final.norm' (+ '.b', '.alpha'), and per layer i 'l<i>.norm1', 'l<i>.norm2' (+ '.b', '.alpha'),
'l<i>.hc1.{in,out,mix}', 'l<i>.hc2.{in,out,mix}', 'l<i>.mix.*', 'l<i>.mlp.*'.  This class is the only place that knows these
names; everything else works from the ``ModelSpec`` it returns."""
from __future__ import annotations

import copy
from dataclasses import dataclass

from .model_config import ConfigError, LayerSpec, ModelSpec, PartSpec, RunEntry

MAX_POSITION = 1 << 20       # the design has no position limit (angles come from the position itself); the engine wants a bound

_MIXER_KEYS = {
    "attention": ("heads", "kv_heads", "dim", "vdim", "scale", "diff"),
    "latent_attention": ("heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank", "scale", "rot"),
    "channel_delta": ("heads", "kv_heads", "dim", "vdim", "conv"),
}


def _need(d: dict, keys, where: str):
    missing = [k for k in keys if k not in d]
    if missing:
        raise ConfigError(f"config.json: {where} lacks key(s): {', '.join(missing)}")


@dataclass(frozen=True)
class KebudraConfig:
    vocab: int
    width: int
    streams: int
    embedding_scale: float
    norm_eps: float
    layers: tuple            # the config's own dicts, checked
    architecture: str = "Kebudra"

    @classmethod
    def from_dict(cls, c: dict) -> "KebudraConfig":
        _need(c, ("vocab", "width", "norm", "layers"), "the model")
        _need(c["norm"], ("eps",), "norm")
        if not isinstance(c["layers"], list) or not c["layers"]:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, layer in enumerate(c["layers"]):
            where = f"layers[{i}]"
            _need(layer, ("type", "mixer"), where)
            kind, m = layer["type"], layer["mixer"]
            if kind not in _MIXER_KEYS:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not a mixer of this design ({', '.join(_MIXER_KEYS)})")
            _need(m, _MIXER_KEYS[kind], where + ".mixer")
            if kind == "latent_attention":
                _need(m["rot"], ("base", "dims"), where + ".mixer.rot")
            if kind != "latent_attention" and int(m["heads"]) % int(m["kv_heads"]):
                raise ConfigError(f"config.json: {where}.mixer: {m['kv_heads']} key heads do not divide {m['heads']} heads")
            src = m.get("kv_from")
            if src is not None:
                if kind != "attention":
                    raise ConfigError(f"config.json: {where}.mixer.kv_from: only an attention layer reads another layer's keys and values")
                if not (isinstance(src, int) and 0 <= src < i and c["layers"][src]["type"] == "attention"
                        and c["layers"][src]["mixer"].get("kv_from") is None):
                    raise ConfigError(f"config.json: {where}.mixer.kv_from must name an earlier attention layer with keys and values of its own")
                other = c["layers"][src]["mixer"]
                if any(int(other[k]) != int(m[k]) for k in ("kv_heads", "dim", "vdim")):
                    raise ConfigError(f"config.json: {where}.mixer reads layer {src}'s keys and values but differs from it in kv_heads, dim or vdim")
            mlp = layer.get("mlp")
            if mlp is not None:
                _need(mlp, ("kind", "expert", "router"), where + ".mlp")
                if mlp["kind"] != "moe":
                    raise ConfigError(f"config.json: {where}.mlp.kind {mlp['kind']!r} is not a feed-forward of this design (moe)")
                _need(mlp["expert"], ("ff",), where + ".mlp.expert")
                _need(mlp["router"], ("experts", "top"), where + ".mlp.router")
                if not 1 <= int(mlp["router"]["top"]) <= int(mlp["router"]["experts"]):
                    raise ConfigError(f"config.json: {where}.mlp.router: top must be between 1 and the number of experts")
            layers.append(copy.deepcopy(layer))
        cfg = cls(vocab=int(c["vocab"]), width=int(c["width"]), streams=int(c.get("streams", 1)),
                  embedding_scale=float((c.get("embedding") or {}).get("scale", 1.0)), norm_eps=float(c["norm"]["eps"]),
                  layers=tuple(layers), architecture=str(c.get("architecture", "Kebudra")))
        if cfg.vocab <= 0 or cfg.width <= 0 or not 1 <= cfg.streams <= 8:
            raise ConfigError("config.json: vocab and width must be positive and streams between 1 and 8")
        return cfg

    def to_dict(self) -> dict:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "streams": self.streams,
                "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
                "layers": copy.deepcopy(list(self.layers))}

    # ------------------------------------------------------------------ description as data
    def _norm(self, prefix: str) -> PartSpec:
        return PartSpec("dynamic_tanh", dict(size=self.width, streams=self.streams), prefix)

    def _mixer(self, layer: dict, prefix: str) -> PartSpec:
        m, kind = layer["mixer"], layer["type"]
        if kind == "attention":
            return PartSpec("differential_attention", dict(
                hidden_size=self.width, num_heads=int(m["heads"]), num_kv_heads=int(m["kv_heads"]), dim=int(m["dim"]),
                vdim=int(m["vdim"]), scale=float(m["scale"]), diff=float(m["diff"]), eps=self.norm_eps,
                shares_kv=m.get("kv_from") is not None), prefix)
        if kind == "latent_attention":
            return PartSpec("latent_attention", dict(
                hidden_size=self.width, num_heads=int(m["heads"]), dim=int(m["dim"]), rot_dim=int(m["rot_dim"]), vdim=int(m["vdim"]),
                q_rank=int(m["q_rank"]), kv_rank=int(m["kv_rank"]), scale=float(m["scale"]), rot_dims=int(m["rot"]["dims"]),
                rot_base=float(m["rot"]["base"]), eps=self.norm_eps), prefix)
        return PartSpec("channel_delta", dict(
            hidden_size=self.width, num_heads=int(m["heads"]), num_kv_heads=int(m["kv_heads"]), dim=int(m["dim"]), vdim=int(m["vdim"]),
            taps=int(m["conv"]), eps=self.norm_eps, decay_rank=m.get("decay_rank"), gate_rank=m.get("gate_rank")), prefix)

    def model_spec(self) -> ModelSpec:
        layers, run_order = [], []
        aliases = {"embed.weight": "embed", "head.weight": "head", "final.norm.weight": "final.norm"}
        connection = lambda prefix: PartSpec("hyper", dict(streams=self.streams), prefix)
        for i, layer in enumerate(self.layers):
            p = f"l{i}."
            parts = dict(mixer=self._mixer(layer, p + "mix."), mixer_norm=self._norm(p + "norm1."),
                         mixer_connection=connection(p + "hc1."))
            aliases[p + "norm1.weight"] = p + "norm1"
            mlp = layer.get("mlp")
            if mlp is not None:
                parts["feed_forward"] = PartSpec("routed_experts", dict(
                    hidden_size=self.width, num_experts=int(mlp["router"]["experts"]), top=int(mlp["router"]["top"]),
                    expert_size=int(mlp["expert"]["ff"])), p + "mlp.")
                parts["feed_forward_norm"] = self._norm(p + "norm2.")
                parts["feed_forward_connection"] = connection(p + "hc2.")
                aliases[p + "norm2.weight"] = p + "norm2"
            layers.append(LayerSpec("hyper_connected" if mlp is not None else "hyper_connected_mixer_only", parts))
            src = layer["mixer"].get("kv_from")
            run_order.append(RunEntry(i, i) if src is None else RunEntry(i, int(src), writes_cache=False))
        return ModelSpec(
            vocab_size=self.vocab, hidden_size=self.width,
            embedding=PartSpec("scaled_embedding", dict(vocab_size=self.vocab, hidden_size=self.width, scale=self.embedding_scale,
                                                        copies=self.streams), "embed."),
            layers=tuple(layers), run_order=tuple(run_order), final_norm=self._norm("final.norm."),
            head=PartSpec("linear_head", dict(vocab_size=self.vocab, hidden_size=self.width), "head."),
            max_position=MAX_POSITION, eos_token_id=-1, aliases=aliases)
