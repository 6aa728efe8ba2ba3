"""Tiny Rarutar configurations and model folders for the tests.

The configurations differ in every size and constant and avoid choices that would hide a mix-up: key and value sizes of
a head differ where the design lets them, one attention has as many key/value heads as heads and one a single one, the
rotated width is the whole vector in one mixer and a part of it in another, one rotation stretches its slow frequencies
and one does not, windows and chunks are smaller than a page, equal to one, and no multiple of one, a state space has
one group, as many groups as heads, and other numbers of norm parts than of groups, convolutions of 2, 3 and 4 taps, a
linear attention with one head, a layer without a feed-forward, and each model starts with another mixer.
"""
from __future__ import annotations

from pathlib import Path

import numpy as np
import torch

import plain_rarutar as plain


def rot(base, dims, scaling=None):
    out = {"base": base, "dims": dims}
    if scaling is not None:
        out["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return out


def softmax(heads, kv_heads, dim, vdim, scale, size, rotation):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": size}, "rot": rotation}


def attention(heads, kv_heads, dim, scale, chunk, rotation):
    return "attention", softmax(heads, kv_heads, dim, dim, scale, chunk, rotation)


def mamba2(heads, vdim, state, groups, conv, norm_groups):
    return "mamba2", {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}


def parallel(left, right, left_scale, right_scale):
    heads, dim, vdim, tau, rank = right
    return "parallel", {"left": left, "right": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "rank": rank},
                        "left_scale": left_scale, "right_scale": right_scale}


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def layer(mixer, mlp):
    return {"type": mixer[0], "mixer": mixer[1], "mlp": mlp}


A = {"architecture": "Rarutar", "vocab": 211, "width": 40, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.7},
     "layers": [
         layer(parallel(softmax(3, 3, 8, 12, 0.4, 5, rot(100.0, 4, (4.0, 16, 4.0, 1.0))), (1, 12, 8, 4.0, 5), 1.3, 0.4), dense(56, 0.8)),
         layer(mamba2(3, 8, 5, 1, 2, 3), None),
         layer(attention(4, 2, 12, 0.9, 7, rot(50.0, 12)), dense(24, 2.5)),
         layer(mamba2(4, 6, 16, 4, 4, 1), dense(32, 1.0)),
     ]}
B = {"architecture": "Rarutar", "vocab": 190, "width": 64, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
     "layers": [
         layer(attention(2, 2, 16, 0.5, 16, rot(10000.0, 8)), dense(48, 1.5)),
         layer(parallel(softmax(4, 1, 16, 16, 0.25, 33, rot(3000.0, 16)), (3, 8, 16, 1.0, 3), 0.5, 1.5), None),
         layer(attention(3, 1, 8, 1.2, 3, rot(20.0, 2, (2.0, 8, 2.0, 0.5))), dense(40, 3.0)),
         layer(parallel(softmax(2, 2, 12, 20, 0.3, 2, rot(700.0, 6, (16.0, 32, 8.0, 2.0))), (2, 20, 12, 9.0, 7), -0.7, 1.0), dense(72, 0.6)),
         layer(mamba2(2, 24, 12, 2, 3, 4), dense(16, 1.2)),
     ]}
# sizes that the tensor-core kernels of the bfloat16 path are built for
C = {"architecture": "Rarutar", "vocab": 277, "width": 128, "norm": {"eps": 1e-5}, "embedding": {"scale": 0.8},
     "layers": [
         layer(mamba2(4, 32, 64, 2, 4, 4), dense(160, 2.0)),
         layer(attention(4, 1, 64, 0.2, 100, rot(50000.0, 32)), dense(96, 1.0)),
         layer(parallel(softmax(4, 2, 32, 64, 0.3, 70, rot(8000.0, 32, (8.0, 64, 16.0, 1.0))), (2, 64, 32, 8.0, 8), 0.8, 1.1), dense(128, 1.5)),
         layer(attention(2, 2, 32, 0.3, 24, rot(500.0, 16)), None),
     ]}
CONFIGS = {"A": (A, 3, 16), "B": (B, 4, 8), "C": (C, 5, 16)}            # name -> (config.json, seed, page size)
MIXER_SCALE = {"A": 4.0, "B": 3.0, "C": 1.5}


def make_model_dir(base, name: str) -> Path:
    """A folder written by the package's random-weights mode, then made harder: the mixers' matrices are scaled up so
    that they are a large share of the stream (a wrong key or a lost state must move the logits), the decays' biases and
    rates are spread from fast to very slow (a state that is lost early shows hundreds of tokens later), the sinks are of
    the scores' size, the convolutions' and norms' biases are not small."""
    from sprout_lm_b200.config import parse_config
    from sprout_lm_b200.weights import write_random_model, write_safetensors
    from sprout_lm_b200.weights.safetensors_io import SafetensorsFile
    raw, seed, _ = CONFIGS[name]
    directory = write_random_model(Path(base) / f"rarutar_{name}", parse_config(raw), seed=seed)
    rng = np.random.default_rng(seed)
    tensors = {}
    handle = SafetensorsFile(directory / "model.safetensors")
    try:
        for key in handle.names():
            value = handle.tensor(key).float()
            n = value.numel()
            if key.endswith(".a2.b"):
                value = torch.from_numpy(rng.permutation(np.linspace(-1.0, 6.0, n)).astype(np.float32))
            elif key.endswith(".A_log"):
                value = torch.from_numpy(rng.permutation(np.linspace(-4.0, 0.5, n)).astype(np.float32))
            elif key.endswith(".dt_bias"):
                value = torch.from_numpy(rng.uniform(-2.0, 1.0, n).astype(np.float32))
            elif key.endswith(".D"):
                value = torch.from_numpy(rng.uniform(0.3, 1.5, n).astype(np.float32))
            elif key.endswith(".sink"):
                value = torch.from_numpy(rng.uniform(-1.0, 2.0, n).astype(np.float32))
            elif key.endswith(".b") and value.dim() == 1:
                value = torch.from_numpy(rng.normal(0.0, 0.3, n).astype(np.float32))
            elif ".mix." in key and value.dim() == 2 and not key.endswith(".conv"):
                value = value * MIXER_SCALE[name] * (4.0 if key.endswith((".a1", ".a2", ".g")) else 1.0)
            elif ".mlp." in key and value.dim() == 2:
                value = value * 3.0
            elif key == "embed":
                value = value * 12.0                # the head is the table: logits of order one
            tensors[key] = value.to(torch.bfloat16)
    finally:
        handle.close()
    write_safetensors(directory / "model.safetensors", tensors, metadata={"format": "pt"})
    return directory


_models: dict = {}
_logits: dict = {}


def plain_model(directory):
    """(config.json as a dict, name -> float64 array)."""
    import json
    key = str(directory)
    if key not in _models:
        _models[key] = (json.loads((Path(directory) / "config.json").read_text()),
                        plain.read_safetensors(Path(directory) / "model.safetensors"))
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
    """Every place that came back against the plain implementation, by the root mean square of the difference over
    the vocabulary divided by the logits' own spread there (``relative``); a failure names the first wrong token and what
    is special about its place.  ``rounded`` (16-bit runs): a place's bar is ``tol`` or, where the model is touchy, three
    times what rounding the plain implementation's matrix products does there; and three places in a hundred may be over
    it: a linear attention's output at a sequence's first tokens is one q . k times v divided by its own root mean
    square, so where q . k is near zero any rounding turns its sign (the 32-bit run of the same plan has no such allowance)."""
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
