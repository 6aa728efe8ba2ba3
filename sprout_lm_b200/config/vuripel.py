"""Typed configuration of the Vuripel decoder, read from its config.json.

config.json: ``architecture`` ("Vuripel"), ``vocab``, ``width``, ``norm.eps``, optionally ``token_side`` = {``dim``} (a
per-layer token input), optionally ``loop`` = {``start``, ``stop``, ``times``} (layers start .. stop - 1 run ``times`` times
in a row with the same weights), and ``layers``, a list whose entries give ``type``, the sizes of that mixer (``mixer``) and
the feed-forward (``mlp``, or null for none):

* ``mlstm``: a matrix memory with exponential gates: ``heads``, ``dim``, ``vdim``, ``gate_cap``;
* ``attention``: softmax attention without positions over grouped key/value heads: ``heads``, ``kv_heads``, ``dim``, ``vdim``,
  ``scale``, ``softcap``; biases on the projections, a sink per head in the softmax and a sigmoid gate per head;
* ``attention_2``: the same sizes; queries and keys are RMS-normed with a weight before a rotation of the first ``rot.dims``
  elements (``rot.base``), the scores are capped, and a query sees the last ``mask.size`` positions and the first
  ``mask.keep_first`` of the sequence.

``mlp``: {``kind``: "dense", ``ff``}: a gated feed-forward with the tanh form of gelu; or {``kind``: "moe", ``expert``:
{``ff``}, ``router``: {``experts``, ``top``, ``groups``: {``count``, ``keep``}}, ``shared``: {``ff``}}: routed experts
without gates (exact gelu), chosen among the best groups' experts by their softmax scores, which are the weights, and a
shared expert weighed by a sigmoid gate per token.  Every size and constant comes from the file; only ``max_positions`` (the
rotary tables' length) has a default.

The model: token embedding; per layer h = norm1(x), x += mixer(h) + mlp(h), then the per-layer token input; the looped span
restarts from the embedding's output plus a learned vector per pass; a final RMS norm and a head.  Tensor names: ``embed``,
``loop.step``, ``side.embed``, ``l<i>.norm1``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``l<i>.side.*``, ``final.norm``, ``head``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, replace
from typing import Any, Mapping

from .specs import ConfigError, LayerCall, LayerSpec, ModelSpec, PartSpec

DEFAULT_MAX_POSITIONS = 65536
MIXER_TYPES = ("mlstm", "attention", "attention_2")


def _is_int(value) -> bool:
    return isinstance(value, int) and not isinstance(value, bool)


def _number(value) -> bool:
    return isinstance(value, (int, float)) and not isinstance(value, bool) and math.isfinite(value)


def _positive_int(raw: Mapping, key: str, where: str) -> int:
    value = raw.get(key)
    if not _is_int(value) or value <= 0:
        raise ConfigError(f"Invalid Vuripel config: {where}.{key} must be a positive integer.")
    return value


def _positive(raw: Mapping, key: str, where: str) -> float:
    value = raw.get(key)
    if not _number(value) or value <= 0:
        raise ConfigError(f"Invalid Vuripel config: {where}.{key} must be a positive number.")
    return float(value)


def _optional_positive(raw: Mapping, key: str, where: str):
    if raw.get(key) is None:
        return None
    return _positive(raw, key, where)


def _parse_mixer(index: int, kind: str, m: Mapping) -> dict:
    where = f"layers[{index}].mixer"
    out = {"heads": _positive_int(m, "heads", where), "dim": _positive_int(m, "dim", where), "vdim": _positive_int(m, "vdim", where)}
    if kind == "mlstm":
        cap = _optional_positive(m, "gate_cap", where)
        if cap is not None:
            out["gate_cap"] = cap
        return out
    out["kv_heads"] = _positive_int(m, "kv_heads", where)
    if out["heads"] % out["kv_heads"]:
        raise ConfigError(f"Invalid Vuripel config: {where}.heads must be a multiple of kv_heads.")
    out["scale"] = _positive(m, "scale", where)
    cap = _optional_positive(m, "softcap", where)
    if cap is not None:
        out["softcap"] = cap
    if kind == "attention":
        return out
    rot = m.get("rot")
    if rot is not None:
        if not isinstance(rot, Mapping):
            raise ConfigError(f"Invalid Vuripel config: {where}.rot must be an object.")
        dims = rot.get("dims")
        if not _is_int(dims) or dims < 0 or dims % 2 or dims > out["dim"]:
            raise ConfigError(f"Invalid Vuripel config: {where}.rot.dims must be even and at most dim.")
        base = _positive(rot, "base", where + ".rot")
        if base <= 1:
            raise ConfigError(f"Invalid Vuripel config: {where}.rot.base must be above 1.")
        out["rot"] = {"base": base, "dims": dims}
    mask = m.get("mask")
    if mask is not None:
        if not isinstance(mask, Mapping):
            raise ConfigError(f"Invalid Vuripel config: {where}.mask must be an object.")
        keep = mask.get("keep_first", 0)
        if not _is_int(keep) or keep < 0:
            raise ConfigError(f"Invalid Vuripel config: {where}.mask.keep_first must be a non-negative integer.")
        out["mask"] = {"size": _positive_int(mask, "size", where + ".mask"), "keep_first": keep}
    return out


def _parse_mlp(index: int, mlp) -> dict | None:
    where = f"layers[{index}].mlp"
    if mlp is None:
        return None
    if not isinstance(mlp, Mapping) or mlp.get("kind") not in ("dense", "moe"):
        raise ConfigError(f"Invalid Vuripel config: {where} must be null or of kind 'dense' or 'moe'.")
    if mlp["kind"] == "dense":
        return {"kind": "dense", "ff": _positive_int(mlp, "ff", where)}
    expert, router = mlp.get("expert"), mlp.get("router")
    if not isinstance(expert, Mapping) or not isinstance(router, Mapping):
        raise ConfigError(f"Invalid Vuripel config: {where} needs expert and router.")
    out = {"kind": "moe", "expert": {"ff": _positive_int(expert, "ff", where + ".expert")},
           "router": {"experts": _positive_int(router, "experts", where + ".router"), "top": _positive_int(router, "top", where + ".router")}}
    experts, top = out["router"]["experts"], out["router"]["top"]
    groups = router.get("groups")
    count, keep = 1, 1
    if groups is not None:
        if not isinstance(groups, Mapping):
            raise ConfigError(f"Invalid Vuripel config: {where}.router.groups must be an object.")
        count, keep = _positive_int(groups, "count", where + ".router.groups"), _positive_int(groups, "keep", where + ".router.groups")
        out["router"]["groups"] = {"count": count, "keep": keep}
    if experts % count or keep > count or top > keep * (experts // count):
        raise ConfigError(f"Invalid Vuripel config: {where}.router: the groups must be equal, keep at most count, and the kept "
                          f"groups must hold at least top experts.")
    shared = mlp.get("shared")
    if shared is not None:
        if not isinstance(shared, Mapping):
            raise ConfigError(f"Invalid Vuripel config: {where}.shared must be an object.")
        out["shared"] = {"ff": _positive_int(shared, "ff", where + ".shared")}
    return out


@dataclass(frozen=True)
class VuripelLayer:
    type: str
    mixer: dict
    mlp: dict | None

    def to_dict(self) -> dict:
        return {"type": self.type, "mixer": self.mixer, "mlp": self.mlp}


@dataclass(frozen=True)
class VuripelConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: tuple
    side_dim: int | None = None
    loop: tuple | None = None                  # (start, stop, times)
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_ids: tuple = ()

    architecture = "Vuripel"

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "VuripelConfig":
        if not isinstance(raw, Mapping) or raw.get("architecture") != cls.architecture:
            raise ConfigError("Invalid Vuripel config.")
        vocab, width = _positive_int(raw, "vocab", "config"), _positive_int(raw, "width", "config")
        if not isinstance(raw.get("norm"), Mapping):
            raise ConfigError("Invalid Vuripel config: norm is missing.")
        eps = _positive(raw["norm"], "eps", "config.norm")
        if not isinstance(raw.get("layers"), list) or not raw["layers"]:
            raise ConfigError("Invalid Vuripel config: layers must be a non-empty list.")
        layers = []
        for index, layer in enumerate(raw["layers"]):
            if not isinstance(layer, Mapping) or layer.get("type") not in MIXER_TYPES or not isinstance(layer.get("mixer"), Mapping):
                raise ConfigError(f"Invalid Vuripel config: layers[{index}] needs a type of {', '.join(MIXER_TYPES)} and a mixer.")
            layers.append(VuripelLayer(layer["type"], _parse_mixer(index, layer["type"], layer["mixer"]),
                                       _parse_mlp(index, layer.get("mlp"))))
        side_dim = None
        if raw.get("token_side") is not None:
            if not isinstance(raw["token_side"], Mapping):
                raise ConfigError("Invalid Vuripel config: token_side must be an object.")
            side_dim = _positive_int(raw["token_side"], "dim", "config.token_side")
        loop = None
        if raw.get("loop") is not None:
            spec = raw["loop"]
            if not isinstance(spec, Mapping):
                raise ConfigError("Invalid Vuripel config: loop must be an object.")
            start, stop, times = spec.get("start"), spec.get("stop"), spec.get("times")
            if not _is_int(start) or not _is_int(stop) or not _is_int(times) or not 0 <= start < stop <= len(layers) or times < 1:
                raise ConfigError("Invalid Vuripel config: loop needs 0 <= start < stop <= layers and times >= 1.")
            loop = (start, stop, times)
        max_positions = raw.get("max_positions", DEFAULT_MAX_POSITIONS)
        if not _is_int(max_positions) or max_positions <= 0:
            raise ConfigError("Invalid Vuripel config: max_positions must be a positive integer.")
        eos_ids = ()
        if raw.get("eos_token_id") is not None:
            from .qwen2 import parse_eos_ids
            eos_ids = parse_eos_ids(raw["eos_token_id"], vocab)
        return cls(vocab=vocab, width=width, norm_eps=eps, layers=tuple(layers), side_dim=side_dim, loop=loop,
                   max_positions=max_positions, eos_token_ids=eos_ids)

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
               "layers": [layer.to_dict() for layer in self.layers]}
        if self.side_dim is not None:
            out["token_side"] = {"dim": self.side_dim}
        if self.loop is not None:
            out["loop"] = dict(zip(("start", "stop", "times"), self.loop))
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            out["max_positions"] = self.max_positions
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out

    def with_eos(self, eos_token_id) -> "VuripelConfig":
        from .qwen2 import parse_eos_ids
        return replace(self, eos_token_ids=parse_eos_ids(eos_token_id, self.vocab))

    # ------------------------------------------------------------------ parts
    def _mixer_spec(self, layer: VuripelLayer) -> PartSpec:
        m = layer.mixer
        if layer.type == "mlstm":
            return PartSpec("exp_gated_matrix_memory", {
                "hidden_size": self.width, "heads": m["heads"], "dim": m["dim"], "value_dim": m["vdim"], "eps": self.norm_eps,
                "gate_cap": m.get("gate_cap"),
                "names": {key: "mix." + key for key in ("q", "k", "v", "g", "o", "norm", "i", "f")} | {"i_bias": "mix.i.b", "f_bias": "mix.f.b"}})
        plain = layer.type == "attention"
        rot, mask = m.get("rot"), m.get("mask")
        position = PartSpec("none", {})
        if not plain and rot and rot["dims"]:
            position = PartSpec("rope_yarn", {"dims": rot["dims"], "theta": rot["base"], "max_positions": self.max_positions, "scaling": None})
        names = {key: "mix." + key for key in ("q", "k", "v", "o", "g", "sink")} | {"q_norm": "mix.q.norm", "k_norm": "mix.k.norm"}
        return PartSpec("multimap_attention", {
            "hidden_size": self.width, "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"], "value_dim": m["vdim"],
            "scale": m["scale"], "position": position, "maps": 1, "names": names, "softcap": m.get("softcap") or 0.0, "bias": True,
            "sink": plain, "gate": plain, "qk_norm_eps": 0.0 if plain else self.norm_eps,
            "mask": None if plain or not mask else ("window", mask["size"], mask["keep_first"])})

    def _mlp_spec(self, mlp: dict | None) -> PartSpec:
        if mlp is None:
            return PartSpec("none", {})
        if mlp["kind"] == "dense":
            return PartSpec("gated_mlp", {"hidden_size": self.width, "intermediate_size": mlp["ff"], "activation": "gelu_tanh",
                                          "names": {"gate": "mlp.gate", "up": "mlp.up", "down": "mlp.down"}})
        router, shared = mlp["router"], mlp.get("shared")
        groups = router.get("groups")
        return PartSpec("routed_experts", {
            "hidden_size": self.width, "experts": router["experts"], "identity": 0, "top": router["top"], "scale": 1.0,
            "expert_ff": mlp["expert"]["ff"], "expert_kind": "plain", "correction": False, "renormalize": False,
            "groups": (groups["count"], groups["keep"]) if groups else None,
            "shared_ff": shared["ff"] if shared else None, "shared_gate": bool(shared),
            "names": {"router": "mlp.router", "expert": "mlp.e{}.", "shared": "mlp.shared.", "shared_gate": "mlp.shared.sg"}})

    def run_order(self) -> tuple[tuple, tuple]:
        """(layer calls, the index in them of every pass's first call): a looped layer is called once per pass, each call
        with a cache slot and a state entry of its own."""
        n = len(self.layers)
        if self.loop is None:
            return tuple(LayerCall(layer=i, cache=i) for i in range(n)), ()
        start, stop, times = self.loop
        calls, starts = [LayerCall(layer=i, cache=i) for i in range(start)], []
        for t in range(times):
            starts.append(len(calls))
            for i in range(start, stop):
                slot = i if t == 0 else n + (t - 1) * (stop - start) + (i - start)
                calls.append(LayerCall(layer=i, cache=slot, state=slot))
        calls += [LayerCall(layer=i, cache=i) for i in range(stop, n)]
        return tuple(calls), tuple(starts)

    def model_spec(self) -> ModelSpec:
        norm = {"size": self.width, "eps": self.norm_eps, "suffix": ""}
        layers = []
        for index, layer in enumerate(self.layers):
            options = {}
            if self.side_dim is not None:
                options["side"] = PartSpec("gated_token_row", {
                    "hidden_size": self.width, "vocab_size": self.vocab, "dim": self.side_dim, "first": index * self.side_dim,
                    "columns": len(self.layers) * self.side_dim, "eps": self.norm_eps, "table": "side.embed",
                    "declares_table": index == 0})
            layers.append(LayerSpec("parallel_residual", f"l{index}.", self._mixer_spec(layer), self._mlp_spec(layer.mlp),
                                    (PartSpec("rmsnorm", {**norm, "name": "norm1"}),), options))
        order, starts = self.run_order()
        stream = PartSpec("loop_restart", {"hidden_size": self.width, "starts": starts, "name": "loop.step"}) if starts else None
        return ModelSpec(
            architecture=self.architecture, hidden_size=self.width, vocab_size=self.vocab, max_positions=self.max_positions,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "hidden_size": self.width, "name": "embed", "suffix": ""}),
            layers=tuple(layers), order=order, stream=stream,
            final_norm=PartSpec("rmsnorm", {**norm, "name": "final.norm"}),
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": self.width, "name": "head", "suffix": "",
                                      "any_inner_size": True}),
            eos_token_ids=self.eos_token_ids)
