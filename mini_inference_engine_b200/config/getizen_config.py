"""Getizen: a decoder whose layers are listed one by one in config.json, each with a mixer of its own kind and
sizes, normed after every sum (post-norm) with RMS statistics per group.

config.json: ``architecture`` "Getizen", ``vocab``, ``width``, ``postln_alpha``, ``norm`` {eps, groups} and ``layers``,
a list of {type, mixer, mlp}:

* type "retention": mixer {heads, dim, vdim, decay [one per head], rot {base, dims}} -- parts.retention.Retention;
* type "parallel": mixer {left {heads, kv_heads, dim, vdim, scale, mask {size}, rot {base, dims, scaling {factor, low,
  high, original}}}, right {width, blocks, conv}} -- gated chunked attention beside a gated linear recurrence
  (parts.attention.GatedAttention, parts.recurrent.GatedLinearRecurrence, joined by parts.parallel.ParallelMixers);
* mlp {kind "dense", ff, limit} -- parts.feedforward.ClampedGLU -- or null for a layer without a feed-forward.

Tensors: 'embed', 'embed.norm', 'final.norm', and per layer i 'l<i>.norm1', 'l<i>.norm2', 'l<i>.mix.*', 'l<i>.mlp.*'.
The output head is the embedding table.  This class is the only place that knows these names; everything else
works from the ``ModelSpec`` it returns."""
from __future__ import annotations

import copy
from dataclasses import dataclass

from .model_config import ConfigError, LayerSpec, ModelSpec, PartSpec, RunEntry

MAX_POSITION = 1 << 20       # the design has no position limit (angles come from the position itself); the engine wants a bound


def _need(d: dict, keys, where: str):
    missing = [k for k in keys if k not in d]
    if missing:
        raise ConfigError(f"config.json: {where} lacks key(s): {', '.join(missing)}")


@dataclass(frozen=True)
class GetizenConfig:
    vocab: int
    width: int
    postln_alpha: float
    norm_eps: float
    norm_groups: int
    layers: tuple            # the config's own dicts, checked
    architecture: str = "Getizen"

    @classmethod
    def from_dict(cls, c: dict) -> "GetizenConfig":
        _need(c, ("vocab", "width", "postln_alpha", "norm", "layers"), "the model")
        _need(c["norm"], ("eps", "groups"), "norm")
        if not isinstance(c["layers"], list) or not c["layers"]:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, layer in enumerate(c["layers"]):
            where = f"layers[{i}]"
            _need(layer, ("type", "mixer"), where)
            m = layer["mixer"]
            if layer["type"] == "retention":
                _need(m, ("heads", "dim", "vdim", "decay", "rot"), where + ".mixer")
                _need(m["rot"], ("base", "dims"), where + ".mixer.rot")
                if len(m["decay"]) != m["heads"]:
                    raise ConfigError(f"config.json: {where}.mixer has {len(m['decay'])} decays for {m['heads']} heads")
            elif layer["type"] == "parallel":
                _need(m, ("left", "right"), where + ".mixer")
                _need(m["left"], ("heads", "kv_heads", "dim", "vdim", "scale", "rot"), where + ".mixer.left")
                _need(m["left"]["rot"], ("base", "dims"), where + ".mixer.left.rot")
                _need(m["right"], ("width", "blocks", "conv"), where + ".mixer.right")
                if m["left"].get("mask") is not None:
                    _need(m["left"]["mask"], ("size",), where + ".mixer.left.mask")
            else:
                raise ConfigError(f"config.json: {where}.type {layer['type']!r} is not a mixer of this design (retention, parallel)")
            mlp = layer.get("mlp")
            if mlp is not None:
                _need(mlp, ("kind", "ff", "limit"), where + ".mlp")
                if mlp["kind"] != "dense":
                    raise ConfigError(f"config.json: {where}.mlp.kind {mlp['kind']!r} is not a feed-forward of this design (dense)")
            layers.append(copy.deepcopy(layer))
        cfg = cls(vocab=int(c["vocab"]), width=int(c["width"]), postln_alpha=float(c["postln_alpha"]),
                  norm_eps=float(c["norm"]["eps"]), norm_groups=int(c["norm"]["groups"]), layers=tuple(layers),
                  architecture=str(c.get("architecture", "Getizen")))
        if cfg.vocab <= 0 or cfg.width <= 0 or cfg.norm_groups <= 0 or cfg.width % cfg.norm_groups:
            raise ConfigError("config.json: vocab, width and norm.groups must be positive, and the groups must divide the width")
        return cfg

    def to_dict(self) -> dict:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "postln_alpha": self.postln_alpha,
                "norm": {"eps": self.norm_eps, "groups": self.norm_groups}, "layers": copy.deepcopy(list(self.layers))}

    # ------------------------------------------------------------------ description as data
    def _norm(self, prefix: str) -> PartSpec:
        return PartSpec("group_rmsnorm", dict(size=self.width, eps=self.norm_eps, groups=self.norm_groups), prefix)

    def _mixer(self, layer: dict, prefix: str) -> PartSpec:
        m = layer["mixer"]
        if layer["type"] == "retention":
            return PartSpec("retention", dict(hidden_size=self.width, num_heads=int(m["heads"]), dim=int(m["dim"]),
                                              vdim=int(m["vdim"]), decay=tuple(float(d) for d in m["decay"]),
                                              rot_dims=int(m["rot"]["dims"]), rot_base=float(m["rot"]["base"]),
                                              rot_scaling=m["rot"].get("scaling"), eps=self.norm_eps), prefix)
        left, right = m["left"], m["right"]
        mask = left.get("mask")
        attention = PartSpec("gated_attention", dict(
            hidden_size=self.width, num_heads=int(left["heads"]), num_kv_heads=int(left["kv_heads"]), dim=int(left["dim"]),
            vdim=int(left["vdim"]), scale=float(left["scale"]), rot_dims=int(left["rot"]["dims"]),
            rot_base=float(left["rot"]["base"]), rot_scaling=left["rot"].get("scaling"), eps=self.norm_eps,
            chunk=int(mask["size"]) if mask else None))
        recurrence = PartSpec("gated_linear_recurrence", dict(hidden_size=self.width, width=int(right["width"]),
                                                              blocks=int(right["blocks"]), taps=int(right["conv"])))
        return PartSpec("parallel", dict(hidden_size=self.width, branches={"left": attention, "right": recurrence}), prefix)

    def model_spec(self) -> ModelSpec:
        layers, aliases = [], {"embed.weight": "embed", "embed.norm.weight": "embed.norm", "final.norm.weight": "final.norm"}
        for i, layer in enumerate(self.layers):
            p = f"l{i}."
            parts = dict(mixer=self._mixer(layer, p + "mix."), mixer_norm=self._norm(p + "norm1."))
            aliases[p + "norm1.weight"] = p + "norm1"
            mlp = layer.get("mlp")
            if mlp is not None:
                parts["feed_forward"] = PartSpec("clamped_glu", dict(hidden_size=self.width, intermediate_size=int(mlp["ff"]),
                                                                     limit=float(mlp["limit"])), p + "mlp.")
                parts["feed_forward_norm"] = self._norm(p + "norm2.")
                aliases[p + "norm2.weight"] = p + "norm2"
            layers.append(LayerSpec("postnorm_residual" if mlp is not None else "postnorm_mixer_only", parts,
                                    dict(alpha=self.postln_alpha)))
        return ModelSpec(
            vocab_size=self.vocab, hidden_size=self.width,
            embedding=PartSpec("normed_embedding", dict(vocab_size=self.vocab, hidden_size=self.width,
                                                        norm=self._norm("")), "embed."),
            layers=tuple(layers), run_order=tuple(RunEntry(i, i) for i in range(len(layers))),
            final_norm=self._norm("final.norm."),
            head=PartSpec("linear_head", dict(vocab_size=self.vocab, hidden_size=self.width, tied=True), "embed."),
            max_position=MAX_POSITION, eos_token_id=-1, aliases=aliases)
