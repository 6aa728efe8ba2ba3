"""Typed configuration of the Rarutar decoder, read from its config.json.

config.json: ``architecture`` ("Rarutar"), ``vocab``, ``width``, ``norm.eps``, ``embedding.scale`` and ``layers``, a list
whose entries give ``type``, the sizes of that mixer (``mixer``) and the feed-forward (``mlp``, or null for none):

* ``attention``: softmax attention with grouped key/value heads whose values are the keys as projected: ``heads``,
  ``kv_heads``, ``dim``, ``scale``, ``mask.size`` (a query sees the positions of its own chunk of that many, counted from
  position 0), ``rot`` = {``base``, ``dims``[, ``scaling``]}; queries and keys are divided by their root mean square after
  the rotation, every head has a sink in its softmax and a sigmoid gate on its output;
* ``mamba2``: a selective state space: ``heads``, ``vdim``, ``state``, ``groups``, ``conv`` (taps), ``norm_groups``;
* ``parallel``: ``left`` (softmax attention over a sliding window of ``mask.size`` positions with values of their own,
  ``vdim``, and a gate per head; ``rot.scaling`` = {``factor``, ``original``, ``fast``, ``slow``} stretches the slow
  frequencies) beside ``right`` (gated linear attention: ``heads``, ``dim``, ``vdim``, ``tau``), summed with ``left_scale``
  and ``right_scale``.

``mlp``: {``kind``: "dense", ``ff``, ``limit``}.  Every size and constant comes from the file (the inner size of the linear
attention's decay comes from its tensors; ``right.rank`` names it for the random-weights mode); only ``max_positions`` (the
rotary tables' length) has a default.

The model: token embedding times ``embedding.scale``; per layer x += mixer(norm1(x)), x += mlp(norm2(x)) with layer norms
that have a weight and a bias; a final norm and a head that is the embedding table.  Tensor names: ``embed``,
``l<i>.norm1|norm2`` (+ ``.b``), ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm`` (+ ``.b``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, replace
from typing import Any, Mapping

from .specs import ConfigError, LayerCall, LayerSpec, ModelSpec, PartSpec

DEFAULT_MAX_POSITIONS = 65536
MIXER_TYPES = ("attention", "mamba2", "parallel")
GLU_ALPHA = 1.702              # the feed-forward's activation g * sigmoid(1.702 g): fixed by the design


def _is_int(value) -> bool:
    return isinstance(value, int) and not isinstance(value, bool)


def _number(value) -> bool:
    return isinstance(value, (int, float)) and not isinstance(value, bool) and math.isfinite(value)


def _positive_int(raw: Mapping, key: str, where: str) -> int:
    value = raw.get(key)
    if not _is_int(value) or value <= 0:
        raise ConfigError(f"Invalid Rarutar config: {where}.{key} must be a positive integer.")
    return value


def _positive(raw: Mapping, key: str, where: str) -> float:
    value = raw.get(key)
    if not _number(value) or value <= 0:
        raise ConfigError(f"Invalid Rarutar config: {where}.{key} must be a positive number.")
    return float(value)


def _parse_rot(m: Mapping, dim: int, where: str) -> dict:
    rot = m.get("rot")
    if not isinstance(rot, Mapping):
        raise ConfigError(f"Invalid Rarutar config: {where}.rot is missing.")
    dims = rot.get("dims")
    if not _is_int(dims) or dims < 0 or dims % 2 or dims > dim:
        raise ConfigError(f"Invalid Rarutar config: {where}.rot.dims must be even and at most dim.")
    base = _positive(rot, "base", where + ".rot")
    if base <= 1:
        raise ConfigError(f"Invalid Rarutar config: {where}.rot.base must be above 1.")
    out = {"base": base, "dims": dims}
    scaling = rot.get("scaling")
    if scaling is not None:
        if not isinstance(scaling, Mapping):
            raise ConfigError(f"Invalid Rarutar config: {where}.rot.scaling must be an object.")
        out["scaling"] = {key: _positive(scaling, key, where + ".rot.scaling") for key in ("factor", "original", "fast", "slow")}
    return out


def _parse_softmax(m: Mapping, where: str, own_values: bool) -> dict:
    out = {"heads": _positive_int(m, "heads", where), "kv_heads": _positive_int(m, "kv_heads", where),
           "dim": _positive_int(m, "dim", where)}
    if out["heads"] % out["kv_heads"]:
        raise ConfigError(f"Invalid Rarutar config: {where}.heads must be a multiple of kv_heads.")
    out["vdim"] = _positive_int(m, "vdim", where) if own_values or "vdim" in m else out["dim"]
    if not own_values and out["vdim"] != out["dim"]:
        raise ConfigError(f"Invalid Rarutar config: {where}.vdim must equal dim: the values are the keys.")
    out["scale"] = _positive(m, "scale", where)
    if not isinstance(m.get("mask"), Mapping):
        raise ConfigError(f"Invalid Rarutar config: {where}.mask is missing.")
    out["mask"] = {"size": _positive_int(m["mask"], "size", where + ".mask")}
    out["rot"] = _parse_rot(m, out["dim"], where)
    return out


def _parse_mixer(index: int, kind: str, m: Mapping) -> dict:
    where = f"layers[{index}].mixer"
    if kind == "attention":
        return _parse_softmax(m, where, own_values=False)
    if kind == "mamba2":
        out = {key: _positive_int(m, key, where) for key in ("heads", "vdim", "state", "groups", "conv", "norm_groups")}
        if out["heads"] % out["groups"]:
            raise ConfigError(f"Invalid Rarutar config: {where}.heads must be a multiple of groups.")
        if (out["heads"] * out["vdim"]) % out["norm_groups"]:
            raise ConfigError(f"Invalid Rarutar config: {where}.norm_groups must divide heads * vdim.")
        if out["conv"] < 2:
            raise ConfigError(f"Invalid Rarutar config: {where}.conv must be at least 2 taps.")
        return out
    left, right = m.get("left"), m.get("right")
    if not isinstance(left, Mapping) or not isinstance(right, Mapping):
        raise ConfigError(f"Invalid Rarutar config: {where} needs left and right.")
    parsed_right = {"heads": _positive_int(right, "heads", where + ".right"), "dim": _positive_int(right, "dim", where + ".right"),
                    "vdim": _positive_int(right, "vdim", where + ".right"), "tau": _positive(right, "tau", where + ".right")}
    if right.get("rank") is not None:
        parsed_right["rank"] = _positive_int(right, "rank", where + ".right")
    out = {"left": _parse_softmax(left, where + ".left", own_values=True), "right": parsed_right}
    for key in ("left_scale", "right_scale"):
        if not _number(m.get(key)):
            raise ConfigError(f"Invalid Rarutar config: {where}.{key} must be a number.")
        out[key] = float(m[key])
    return out


def _parse_mlp(index: int, mlp) -> dict | None:
    where = f"layers[{index}].mlp"
    if mlp is None:
        return None
    if not isinstance(mlp, Mapping) or mlp.get("kind") != "dense":
        raise ConfigError(f"Invalid Rarutar config: {where} must be null or of kind 'dense'.")
    return {"kind": "dense", "ff": _positive_int(mlp, "ff", where), "limit": _positive(mlp, "limit", where)}


@dataclass(frozen=True)
class RarutarLayer:
    type: str
    mixer: dict
    mlp: dict | None

    def to_dict(self) -> dict:
        return {"type": self.type, "mixer": self.mixer, "mlp": self.mlp}


@dataclass(frozen=True)
class RarutarConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    layers: tuple
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_ids: tuple = ()

    architecture = "Rarutar"

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "RarutarConfig":
        if not isinstance(raw, Mapping) or raw.get("architecture") != cls.architecture:
            raise ConfigError("Invalid Rarutar config.")
        vocab, width = _positive_int(raw, "vocab", "config"), _positive_int(raw, "width", "config")
        if not isinstance(raw.get("norm"), Mapping):
            raise ConfigError("Invalid Rarutar config: norm is missing.")
        eps = _positive(raw["norm"], "eps", "config.norm")
        if not isinstance(raw.get("embedding"), Mapping) or not _number(raw["embedding"].get("scale")):
            raise ConfigError("Invalid Rarutar config: embedding.scale must be a number.")
        if not isinstance(raw.get("layers"), list) or not raw["layers"]:
            raise ConfigError("Invalid Rarutar config: layers must be a non-empty list.")
        layers = []
        for index, layer in enumerate(raw["layers"]):
            if not isinstance(layer, Mapping) or layer.get("type") not in MIXER_TYPES or not isinstance(layer.get("mixer"), Mapping):
                raise ConfigError(f"Invalid Rarutar config: layers[{index}] needs a type of {', '.join(MIXER_TYPES)} and a mixer.")
            layers.append(RarutarLayer(layer["type"], _parse_mixer(index, layer["type"], layer["mixer"]),
                                       _parse_mlp(index, layer.get("mlp"))))
        max_positions = raw.get("max_positions", DEFAULT_MAX_POSITIONS)
        if not _is_int(max_positions) or max_positions <= 0:
            raise ConfigError("Invalid Rarutar config: max_positions must be a positive integer.")
        eos_ids = ()
        if raw.get("eos_token_id") is not None:
            from .qwen2 import parse_eos_ids
            eos_ids = parse_eos_ids(raw["eos_token_id"], vocab)
        return cls(vocab=vocab, width=width, norm_eps=eps, embedding_scale=float(raw["embedding"]["scale"]), layers=tuple(layers),
                   max_positions=max_positions, eos_token_ids=eos_ids)

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
               "embedding": {"scale": self.embedding_scale}, "layers": [layer.to_dict() for layer in self.layers]}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            out["max_positions"] = self.max_positions
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out

    def with_eos(self, eos_token_id) -> "RarutarConfig":
        from .qwen2 import parse_eos_ids
        return replace(self, eos_token_ids=parse_eos_ids(eos_token_id, self.vocab))

    # ------------------------------------------------------------------ parts
    def _position(self, rot: dict) -> PartSpec:
        if not rot["dims"]:
            return PartSpec("none", {})
        return PartSpec("rope_yarn", {"dims": rot["dims"], "theta": rot["base"], "max_positions": self.max_positions,
                                      "scaling": rot.get("scaling")})

    def _softmax_spec(self, m: dict, stem: str, chunked: bool) -> PartSpec:
        """One softmax map per head; ``chunked``: the mixer whose values are its keys, with sinks and unit-norm vectors."""
        names = {key: stem + key for key in ("q", "k", "v", "o", "g", "sink")}
        return PartSpec("multimap_attention", {
            "hidden_size": self.width, "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"], "value_dim": m["vdim"],
            "scale": m["scale"], "position": self._position(m["rot"]), "maps": 1, "names": names,
            "mask": ("chunk" if chunked else "window", m["mask"]["size"]), "gate": True, "sink": chunked,
            "unit_norm_eps": self.norm_eps if chunked else 0.0, "value_from_key": chunked})

    def _mixer_spec(self, layer: RarutarLayer) -> PartSpec:
        m = layer.mixer
        if layer.type == "attention":
            return self._softmax_spec(m, "mix.", chunked=True)
        if layer.type == "mamba2":
            return PartSpec("selective_state_space", {
                "hidden_size": self.width, "heads": m["heads"], "value_dim": m["vdim"], "state": m["state"], "groups": m["groups"],
                "taps": m["conv"], "norm_groups": m["norm_groups"], "eps": self.norm_eps,
                "names": {"in": "mix.in", "conv": "mix.conv", "conv_bias": "mix.conv.b", "dt_bias": "mix.dt_bias",
                          "a_log": "mix.A_log", "skip": "mix.D", "norm": "mix.norm", "o": "mix.o"}})
        right = m["right"]
        linear = PartSpec("gated_linear_attention", {
            "hidden_size": self.width, "heads": right["heads"], "dim": right["dim"], "value_dim": right["vdim"], "tau": right["tau"],
            "eps": self.norm_eps, "decay_rank": right.get("rank")})
        return PartSpec("parallel_mixers", {"mixers": (self._softmax_spec(m["left"], "", chunked=False), linear),
                                            "scales": (m["left_scale"], m["right_scale"]), "names": ("mix.left.", "mix.right.")})

    def _mlp_spec(self, mlp: dict | None) -> PartSpec:
        if mlp is None:
            return PartSpec("none", {})
        return PartSpec("clamped_glu_mlp", {"hidden_size": self.width, "intermediate_size": mlp["ff"], "limit": mlp["limit"],
                                            "alpha": GLU_ALPHA, "names": {"gate": "mlp.gate", "up": "mlp.up", "down": "mlp.down"}})

    def model_spec(self) -> ModelSpec:
        norm = {"size": self.width, "eps": self.norm_eps, "suffix": "", "bias_suffix": ".b"}
        layers, order = [], []
        for index, layer in enumerate(self.layers):
            names = ("norm1",) + (("norm2",) if layer.mlp is not None else ())
            norms = tuple(PartSpec("layernorm", {**norm, "name": name}) for name in names)
            layers.append(LayerSpec("pre_norm", f"l{index}.", self._mixer_spec(layer), self._mlp_spec(layer.mlp), norms))
            # every layer call names a cache slot; a mixer that keeps nothing per token gets a slot without buffers
            order.append(LayerCall(layer=index, cache=index, writes_cache=True))
        return ModelSpec(
            architecture=self.architecture, hidden_size=self.width, vocab_size=self.vocab, max_positions=self.max_positions,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "hidden_size": self.width, "name": "embed", "suffix": "",
                                                   "scale": self.embedding_scale}),
            layers=tuple(layers), order=tuple(order),
            final_norm=PartSpec("layernorm", {**norm, "name": "final.norm"}),
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": self.width, "tied_to": "embed", "suffix": "",
                                      "any_inner_size": True}),
            eos_token_ids=self.eos_token_ids)
