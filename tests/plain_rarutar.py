"""A plain, slow Rarutar decoder in numpy float64: one function per mechanism, whole sequences at once, no cache.

It shares nothing with the package (its own safetensors reader included) and is what the framework's kernels,
cache, state slots and step function are compared with.  Layers: layer norms with weight and bias before each
sublayer; mixers ``attention`` (chunked mask, a sink in the softmax, values that are the keys as projected, unit-norm
queries and keys, a gate per head), ``mamba2`` (short causal convolution, a state-space recurrence, a gated norm in
groups) and ``parallel`` (softmax attention over a sliding window beside gated linear attention, summed with two
scales); a clamped gated feed-forward; a head tied to the embedding table.
"""
from __future__ import annotations

import json
import math
import struct

import numpy as np


# ------------------------------------------------------------------------------------------------ files
def read_safetensors(path) -> dict:
    """name -> float64 (or int64) array of a safetensors file: 8-byte length, JSON header, data."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        raw, shape = data[lo:hi], info["shape"]
        if info["dtype"] == "BF16":
            bits = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
            out[name] = bits.view(np.float32).astype(np.float64).reshape(shape)
        elif info["dtype"] == "F32":
            out[name] = np.frombuffer(raw, dtype="<f4").astype(np.float64).reshape(shape)
        elif info["dtype"] == "F16":
            out[name] = np.frombuffer(raw, dtype="<f2").astype(np.float64).reshape(shape)
        elif info["dtype"] == "I32":
            out[name] = np.frombuffer(raw, dtype="<i4").astype(np.int64).reshape(shape)
        else:
            raise ValueError(f"{name}: dtype {info['dtype']}")
    return out


# ------------------------------------------------------------------------------------------------ small pieces
ROUND = None            # a function array -> array; set (see ``rounding``) to learn how far 16-bit matrix products move a result


def to_bfloat16(a):
    """Round to the nearest bfloat16 (ties to even), returned as float64."""
    bits = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    bits = (bits + 0x7FFF + ((bits >> 16) & 1)) & np.uint32(0xFFFF0000)
    return bits.view(np.float32).astype(np.float64)


class rounding:
    """``with rounding(to_bfloat16):`` every matrix product's input and output pass through the function."""

    def __init__(self, fn):
        self.fn = fn

    def __enter__(self):
        global ROUND
        self.before, ROUND = ROUND, self.fn

    def __exit__(self, *exc):
        global ROUND
        ROUND = self.before


def lin(x, weight):
    """W x for every row of x (weights are stored [out, in])."""
    if ROUND is None:
        return x @ weight.T
    return ROUND(ROUND(x) @ weight.T)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def layer_norm(x, w, b, eps):
    mean = x.mean(axis=-1, keepdims=True)
    var = ((x - mean) ** 2).mean(axis=-1, keepdims=True)
    return (x - mean) / np.sqrt(var + eps) * w + b


def rms_unit(x, eps):
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)


def rotary_frequencies(dims: int, base: float, scaling: dict | None):
    """(frequencies [dims / 2], factor on cos and sin)."""
    i = np.arange(dims // 2, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def where(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(where(float(scaling["fast"]))), 0)
    hi = min(math.ceil(where(float(scaling["slow"]))), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x, positions, rot: dict):
    """x [tokens, heads, dim]: the first rot['dims'] elements of each head turn, element i with element i + dims / 2."""
    dims = int(rot["dims"])
    if dims == 0:
        return x
    f, magnitude = rotary_frequencies(dims, float(rot["base"]), rot.get("scaling"))
    angle = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]
    cos, sin = (np.cos(angle) * magnitude)[:, None, :], (np.sin(angle) * magnitude)[:, None, :]
    half = dims // 2
    u, v = x[..., :half], x[..., half:dims]
    return np.concatenate([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], axis=-1)


def first_visible(kind: str, size: int, i: int) -> int:
    """The first position that a query at position i sees."""
    if kind == "window":
        return max(0, i - size + 1)
    if kind == "chunk":
        return (i // size) * size
    return 0


def masked_softmax_attention(q, k, v, scale, kind, size, sink=None, positions=None):
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H, dv]; query head h reads key/value head h // (H / G);
    ``sink`` [H] adds exp(sink_h) to head h's denominator."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]))
    positions = list(range(T)) if positions is None else positions
    for t in range(T):
        lo = first_visible(kind, size, positions[t])
        first = t - (positions[t] - lo)
        for h in range(H):
            g = h // (H // G)
            s = (k[first:t + 1, g] @ q[t, h]) * scale
            top = s.max() if sink is None else max(s.max(), sink[h])
            e = np.exp(s - top)
            denominator = e.sum() + (0.0 if sink is None else math.exp(sink[h] - top))
            out[t, h] = (e / denominator) @ v[first:t + 1, g]
    return out


# ------------------------------------------------------------------------------------------------ mixers
def gated_softmax_mixer(h, w, prefix, m, eps, kind, unit_norm, value_is_key, has_sink):
    """Softmax attention with grouped heads, a rotation over part of each head, a mask of ``kind`` and a gate per head."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = lin(h, w[prefix + "q"]).reshape(T, H, d)
    k = lin(h, w[prefix + "k"]).reshape(T, G, d)
    v = k.copy() if value_is_key else lin(h, w[prefix + "v"]).reshape(T, G, dv)
    positions = np.arange(T)
    q, k = rotate(q, positions, m["rot"]), rotate(k, positions, m["rot"])
    if unit_norm:
        q, k = rms_unit(q, eps), rms_unit(k, eps)
    sink = w[prefix + "sink"] if has_sink else None
    o = masked_softmax_attention(q, k, v, m["scale"], kind, m["mask"]["size"], sink)
    gate = sigmoid(lin(h, w[prefix + "g"]))                # [T, H]
    o = o * gate[:, :, None]
    return lin(o.reshape(T, H * dv), w[prefix + "o"])


def gated_linear_attention(h, w, prefix, m, eps, state=None):
    """S_t = diag(alpha_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t with a decay per key channel made from the input;
    each head's o is RMS-normed with a weight shared by the heads, then gated by silu(W_g h)."""
    T = h.shape[0]
    H, d, dv, tau = m["heads"], m["dim"], m["vdim"], float(m["tau"])
    q = lin(h, w[prefix + "q"]).reshape(T, H, d) * d ** -0.5
    k = lin(h, w[prefix + "k"]).reshape(T, H, d)
    v = lin(h, w[prefix + "v"]).reshape(T, H, dv)
    z = lin(lin(h, w[prefix + "a1"]), w[prefix + "a2"]) + w[prefix + "a2.b"]
    alpha = (sigmoid(z) ** (1.0 / tau)).reshape(T, H, d)
    S = np.zeros((H, d, dv)) if state is None else state
    o = np.zeros((T, H, dv))
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = np.einsum("hdv,hd->hv", S, q[t])
    o = rms_unit(o, eps) * w[prefix + "norm"]
    out = lin(o.reshape(T, H * dv) * silu(lin(h, w[prefix + "g"])), w[prefix + "o"])
    return out, S


def causal_conv(x, weight, bias):
    """x [T, C], weight [C, taps]: y_t = bias + sum_j weight[:, j] x_(t - (taps - 1 - j)), zeros before the start."""
    T, _ = x.shape
    taps = weight.shape[1]
    y = np.tile(bias, (T, 1)).astype(np.float64)
    for j in range(taps):
        back = taps - 1 - j
        if back < T:
            y[back:] += x[:T - back] * weight[:, j]
    return y


def mamba2_mixer(h, w, prefix, m, eps):
    T = h.shape[0]
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    row = lin(h, w[prefix + "in"])
    z, xbc, dt = row[:, :inner], row[:, inner:2 * inner + 2 * G * N], row[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w[prefix + "conv"], w[prefix + "conv.b"]))
    x = xbc[:, :inner].reshape(T, H, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + w[prefix + "dt_bias"])            # [T, H]
    A = -np.exp(w[prefix + "A_log"])
    S = np.zeros((H, N, P))
    y = np.zeros((T, H, P))
    for t in range(T):
        for head in range(H):
            g = head // (H // G)
            S[head] = math.exp(A[head] * dt[t, head]) * S[head] + dt[t, head] * np.outer(B[t, g], x[t, head])
            y[t, head] = S[head].T @ C[t, g] + w[prefix + "D"][head] * x[t, head]
    y = y.reshape(T, inner) * silu(z)
    parts = int(m["norm_groups"])
    y = rms_unit(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * w[prefix + "norm"]
    return lin(y, w[prefix + "o"])


def clamped_glu(h, w, prefix, mlp):
    limit = float(mlp["limit"])
    g = np.minimum(lin(h, w[prefix + "gate"]), limit)
    u = np.clip(lin(h, w[prefix + "up"]), -limit, limit)
    return lin(g * sigmoid(1.702 * g) * (u + 1.0), w[prefix + "down"])


# ------------------------------------------------------------------------------------------------ the model
def mixer_output(layer, h, w, prefix, eps):
    kind, m = layer["type"], layer["mixer"]
    if kind == "attention":
        return gated_softmax_mixer(h, w, prefix, m, eps, "chunk", unit_norm=True, value_is_key=True, has_sink=True)
    if kind == "mamba2":
        return mamba2_mixer(h, w, prefix, m, eps)
    if kind == "parallel":
        left = gated_softmax_mixer(h, w, prefix + "left.", m["left"], eps, "window", unit_norm=False, value_is_key=False,
                                   has_sink=False)
        right, _ = gated_linear_attention(h, w, prefix + "right.", m["right"], eps)
        return float(m["left_scale"]) * left + float(m["right_scale"]) * right
    raise ValueError(f"unknown layer type {kind}")


def forward(config: dict, w: dict, tokens, layers_out: list | None = None):
    """Logits [tokens, vocab] of one sequence from position 0; ``layers_out`` receives the stream after every layer."""
    eps = float(config["norm"]["eps"])
    x = w["embed"][np.asarray(tokens)] * float(config["embedding"]["scale"])
    for index, layer in enumerate(config["layers"]):
        p = f"l{index}."
        x = x + mixer_output(layer, layer_norm(x, w[p + "norm1"], w[p + "norm1.b"], eps), w, p + "mix.", eps)
        if layer.get("mlp") is not None:
            x = x + clamped_glu(layer_norm(x, w[p + "norm2"], w[p + "norm2.b"], eps), w, p + "mlp.", layer["mlp"])
        if layers_out is not None:
            layers_out.append(x.copy())
    x = layer_norm(x, w["final.norm"], w["final.norm.b"], eps)
    return lin(x, w["embed"])
