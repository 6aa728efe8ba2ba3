"""Tiny Vuripel configurations and model folders for the tests.

The configurations differ in every size and constant and avoid choices that would hide a mix-up: key and value sizes of a
head differ, one attention has as many key/value heads as heads and one a single one, the rotated width is the whole vector,
a part of it, or nothing, windows are smaller than a page, larger than one, and no multiple of one, the kept first positions
are none, fewer than a page and more than a page, caps and scales differ per layer, a matrix memory has one head and no cap
on its gates, routers have one group, several groups of which some are kept, one expert per token and several, with and
without a shared expert, a layer has no feed-forward, the loop covers the first layers, inner layers or nothing and runs two
or three times, and one model has no per-layer token input.
"""
from __future__ import annotations

from pathlib import Path

import numpy as np
import torch

import plain_vuripel as plain


def mlstm(heads, dim, vdim, cap=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim}
    if cap is not None:
        m["gate_cap"] = cap
    return "mlstm", m


def attention(heads, kv_heads, dim, vdim, scale, softcap=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if softcap is not None:
        m["softcap"] = softcap
    return "attention", m


def attention_2(heads, kv_heads, dim, vdim, scale, softcap=None, mask=None, rot=None):
    m = attention(heads, kv_heads, dim, vdim, scale, softcap)[1]
    if mask is not None:
        m["mask"] = {"size": mask[0], "keep_first": mask[1]}
    if rot is not None:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
    return "attention_2", m


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, groups=None, shared=None):
    router = {"experts": experts, "top": top}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    out = {"kind": "moe", "expert": {"ff": ff}, "router": router}
    if shared is not None:
        out["shared"] = {"ff": shared}
    return out


def layer(mixer, mlp):
    return {"type": mixer[0], "mixer": mixer[1], "mlp": mlp}


# sizes that are no multiples of 8; inner layers run three times
A = {"architecture": "Vuripel", "vocab": 203, "width": 40, "norm": {"eps": 1e-5}, "token_side": {"dim": 6},
     "loop": {"start": 1, "stop": 3, "times": 3},
     "layers": [
         layer(attention_2(3, 3, 8, 12, 0.4, 2.0, (5, 2), (100.0, 4)), dense(56)),
         layer(mlstm(3, 12, 7, 3.0), moe(6, 2, 20, (3, 1), 12)),
         layer(attention(4, 2, 12, 6, 0.9, 1.2), None),
         layer(mlstm(1, 20, 20), dense(27)),
     ]}
# no loop, no token input; a router without groups that takes one expert
B = {"architecture": "Vuripel", "vocab": 190, "width": 64, "norm": {"eps": 1e-6},
     "layers": [
         layer(attention(2, 1, 16, 16, 0.5), moe(4, 1, 24)),
         layer(attention_2(4, 1, 16, 24, 0.25, 30.0, (33, 0), (3000.0, 16)), dense(48)),
         layer(mlstm(2, 16, 32, 10.0), moe(8, 3, 16, (4, 2), 40)),
         layer(attention_2(2, 2, 12, 20, 0.3, 15.0), None),
         layer(attention_2(6, 2, 8, 8, 0.6, None, (9, 11), (20.0, 2)), dense(40)),
     ]}
# sizes that the tensor-core kernels of the bfloat16 path are built for; the first two layers run twice
C = {"architecture": "Vuripel", "vocab": 277, "width": 128, "norm": {"eps": 1e-5}, "token_side": {"dim": 16},
     "loop": {"start": 0, "stop": 2, "times": 2},
     "layers": [
         layer(mlstm(2, 64, 64, 12.0), dense(160)),
         layer(attention_2(4, 2, 32, 64, 0.18, 20.0, (70, 3), (50000.0, 32)), moe(8, 2, 32, (4, 2), 64)),
         layer(attention(8, 2, 64, 128, 0.1, 25.0), dense(96)),
         layer(attention_2(4, 1, 64, 64, 0.11, 40.0, (100, 17), (20000.0, 48)), moe(4, 2, 40)),
     ]}
CONFIGS = {"A": (A, 3, 16), "B": (B, 4, 8), "C": (C, 5, 16)}            # name -> (config.json, seed, page size)
MIXER_SCALE = {"A": 6.0, "B": 3.0, "C": 1.5}


def make_model_dir(base, name: str) -> Path:
    """A folder written by the package's random-weights mode, then made harder: the mixers' matrices are scaled up so that
    they are a large share of the stream (a wrong key or a lost state must move the logits), the forget gates' biases are
    spread from fast to very slow (a state that is lost early shows hundreds of tokens later), the sinks are of the scores'
    size, the biases, the passes' vectors and the token rows are not small, and the routers' scores are well apart."""
    from sprout_lm_b200.config import parse_config
    from sprout_lm_b200.weights import write_random_model, write_safetensors
    from sprout_lm_b200.weights.safetensors_io import SafetensorsFile
    raw, seed, _ = CONFIGS[name]
    directory = write_random_model(Path(base) / f"vuripel_{name}", parse_config(raw), seed=seed)
    rng = np.random.default_rng(seed)
    tensors = {}
    handle = SafetensorsFile(directory / "model.safetensors")
    try:
        for key in handle.names():
            value = handle.tensor(key).float()
            n = value.numel()
            if key.endswith(".f.b"):
                value = torch.from_numpy(rng.permutation(np.linspace(0.5, 6.0, n)).astype(np.float32))
            elif key.endswith(".i.b"):
                value = torch.from_numpy(rng.uniform(-2.0, 1.0, n).astype(np.float32))
            elif key.endswith((".q.norm", ".k.norm")):
                value = torch.from_numpy(rng.uniform(0.3, 2.0, n).astype(np.float32))
            elif key.endswith(".sink"):
                value = torch.from_numpy(rng.uniform(-1.0, 2.0, n).astype(np.float32))
            elif key.endswith(".b") and value.dim() == 1:
                value = torch.from_numpy(rng.normal(0.0, 0.5, n).astype(np.float32))
            elif key == "loop.step":
                value = value * 25.0
            elif key == "side.embed":
                value = value * 40.0
            elif key.endswith((".mix.i", ".mix.f")):
                value = value * 30.0
            elif key.endswith((".router", ".shared.sg")):
                value = value * 25.0
            elif ".mix." in key and value.dim() == 2:
                value = value * MIXER_SCALE[name] * (4.0 if key.endswith(".g") else 1.0)
            elif (".mlp." in key or ".side." in key) and value.dim() == 2:
                value = value * (12.0 if ".mlp.e" in key else 8.0 if ".shared." in key else 3.0)
            elif key == "embed":
                value = value * 40.0
            elif key == "head":
                value = value * 8.0
            tensors[key] = value.to(torch.bfloat16)
    finally:
        handle.close()
    write_safetensors(directory / "model.safetensors", tensors, metadata={"format": "pt"})
    return directory


_models: dict = {}
_logits: dict = {}


def plain_model(directory):
    """(config.json as a dict, name -> float64 array)."""
    key = str(directory)
    if key not in _models:
        _models[key] = plain.read_model_folder(str(directory))
    return _models[key]


def plain_logits(directory, tokens) -> np.ndarray:
    key = (str(directory), tuple(tokens))
    if key not in _logits:
        _logits[key] = plain.forward(*plain_model(directory), list(tokens))
    return _logits[key]


def rounding_moves(directory, tokens) -> np.ndarray:
    """Per position, how far the plain implementation's logits move (``relative``) when its matrix products read and
    write bfloat16: what rounding alone does at that place of that model."""
    key = (str(directory), tuple(tokens), "rounded")
    if key not in _logits:
        want = plain_logits(directory, tokens)
        with plain.rounding(plain.to_bfloat16):
            moved = plain.forward(*plain_model(directory), list(tokens))
        _logits[key] = np.array([relative(a, b) for a, b in zip(moved, want)])
    return _logits[key]


def plain_greedy(directory, prompt, new_tokens: int) -> list:
    history, out = list(prompt), []
    for _ in range(new_tokens):
        row = plain.forward(*plain_model(directory), history)[-1]
        out.append(int(np.argmax(row)))
        history.append(out[-1])
    return out


def relative(got, want) -> float:
    """Root mean square of got - want over the vocabulary, divided by that of want about its mean."""
    spread = float(np.sqrt(np.mean((want - want.mean()) ** 2)))
    return float(np.sqrt(np.mean((np.asarray(got, dtype=np.float64) - want) ** 2))) / max(spread, 1e-6)


def compare(directory, requests: dict, got: dict, tol: float, label: str, page: int, rounded: bool = False):
    """Every place that came back against the plain implementation, by the root mean square of the difference over the
    vocabulary divided by the logits' own spread there (``relative``); a failure names the first wrong token and what is
    special about its place.  ``rounded`` (16-bit runs): a place's bar is ``tol`` or, where the model is touchy, three times
    what rounding the plain implementation's matrix products does there; and three places in a hundred may be over it (a
    router's nearly tied choice may fall either way in 16 bits; the 32-bit run of the same plan has no such allowance)."""
    assert got, "no logits came back"
    worst, first, over, places = 0.0, None, 0, 0
    for rid, tokens in requests.items():
        want = plain_logits(directory, tokens)
        bars = np.maximum(tol, 3.0 * rounding_moves(directory, tokens)) if rounded else np.full(len(tokens), tol)
        for pos in range(len(tokens)):
            if (rid, pos) not in got:
                continue
            err = relative(got[(rid, pos)], want[pos])
            places += 1
            if not np.isfinite(err) or err > bars[pos]:
                over += 1
                if first is None:
                    first = (f"{label}: request {rid} position {pos} of {len(tokens)} (position % {page} = {pos % page}) "
                             f"differs by {err:.3e} > {bars[pos]:.3e}")
            worst = max(worst, err) if np.isfinite(err) else float("inf")
    if over > (max(2, 3 * places // 100) if rounded else 0) or not np.isfinite(worst):
        raise AssertionError(f"{first}; {over} of {places} places are over the bar")
    return worst
