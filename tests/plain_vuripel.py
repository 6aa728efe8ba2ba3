"""A plain, slow Vuripel decoder in numpy float64: one function per mechanism, whole sequences at once, no cache.

It shares nothing with the package (its own safetensors reader included) and is what the framework's kernels, cache,
state slots and step function are compared with.  The model: a token embedding; layers in which the mixer and the
feed-forward read one RMS norm's output and are added to the stream together, followed by a per-layer token input;
three mixers (``mlstm``: a matrix memory with exponential gates and a running maximum; ``attention``: softmax attention
without positions, with capped scores, a sink per head and a gate per head; ``attention_2``: query/key norms, a partial
rotation, capped scores and a sliding window that keeps the first tokens); dense and routed feed-forwards; a span of
layers that runs several times with the same weights; a final norm and a head.
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
        elif info["dtype"] == "I32":
            out[name] = np.frombuffer(raw, dtype="<i4").astype(np.int64).reshape(shape)
        else:
            raise ValueError(f"{name}: dtype {info['dtype']}")
    return out


def read_model_folder(folder):
    with open(f"{folder}/config.json") as f:
        config = json.load(f)
    return config, read_safetensors(f"{folder}/model.safetensors")


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


def lin(x, weight, bias=None, exact=False):
    """W x (+ b) for every row of x (weights are stored [out, in]); ``exact``: never rounded (32-bit quantities)."""
    if ROUND is None or exact:
        y = x @ weight.T
        return y if bias is None else y + bias
    y = ROUND(x) @ weight.T
    return ROUND(y if bias is None else y + bias)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def log_sigmoid(z):
    return -(np.maximum(-z, 0.0) + np.log1p(np.exp(-np.abs(z))))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def gelu_erf(z):
    return 0.5 * z * (1.0 + np.vectorize(math.erf)(z / math.sqrt(2.0)))


def unit_rms(x, eps):
    """x divided by its root mean square over the last axis (eps inside the root)."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def rms_norm(x, weight, eps):
    return unit_rms(x, eps) * weight


def soft_cap(s, cap):
    return s if not cap else cap * np.tanh(s / cap)


# ------------------------------------------------------------------------------------------------ mixers
def exp_gated_memory(q, k, v, gi, gf, state=None, parts=None):
    """The recurrence alone: q, k [T, H, D] (q already scaled), v [T, H, V], log gates gi, gf [T, H].  ``state`` = (S [H, D, V],
    n [H, D], m [H]) to start from (zeros when None).  Returns o [T, H, V] and the state after the last token; a list given as
    ``parts`` receives what o is made of: S^T q [T, H, V], n . q [T, H] and m [T, H]."""
    T, H, D = q.shape
    V = v.shape[2]
    S, n, top = (np.zeros((H, D, V)), np.zeros((H, D)), np.zeros(H)) if state is None else (a.copy() for a in state)
    out, above, below, tops = np.zeros((T, H, V)), np.zeros((T, H, V)), np.zeros((T, H)), np.zeros((T, H))
    for head in range(H):
        for t in range(T):
            new_top = max(gf[t, head] + top[head], gi[t, head])
            keep, take = math.exp(gf[t, head] + top[head] - new_top), math.exp(gi[t, head] - new_top)
            S[head] = keep * S[head] + take * np.outer(k[t, head], v[t, head])
            n[head] = keep * n[head] + take * k[t, head]
            top[head] = new_top
            above[t, head], below[t, head], tops[t, head] = S[head].T @ q[t, head], n[head] @ q[t, head], new_top
            out[t, head] = above[t, head] / (max(abs(below[t, head]), math.exp(-new_top)) + 1e-6)
    if parts is not None:
        parts += [above, below, tops]
    return out, (S, n, top)


def log_gates(zi, zf, cap):
    """(log input gate, log forget gate) from the gate projections (biases added)."""
    if cap:
        zi, zf = cap * np.tanh(zi / cap), cap * np.tanh(zf / cap)
    return zi, log_sigmoid(zf)


def mlstm(h, w, p, m, eps):
    """The matrix memory: per head S (dim x vdim), n (dim) and a running maximum that starts at 0.
    Returns the mixer's output [tokens, width]."""
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = lin(h, w[p + "q"]).reshape(T, H, D) * D ** -0.5
    k = lin(h, w[p + "k"]).reshape(T, H, D)
    v = lin(h, w[p + "v"]).reshape(T, H, V)
    gi, gf = log_gates(lin(h, w[p + "i"], w[p + "i.b"], exact=True), lin(h, w[p + "f"], w[p + "f.b"], exact=True), m.get("gate_cap"))
    out, _ = exp_gated_memory(q, k, v, gi, gf)
    out = unit_rms(out, eps).reshape(T, H * V) * w[p + "norm"] * sigmoid(lin(h, w[p + "g"]))
    return lin(out, w[p + "o"])


def rotate_half(x, positions, base, dims):
    """x [tokens, heads, dim]: the first ``dims`` elements of each head turn, element i paired with i + dims / 2."""
    if not dims:
        return x
    half = dims // 2
    freq = base ** (-2.0 * np.arange(half) / dims)
    angle = positions[:, None].astype(np.float64) * freq[None, :]
    cos, sin = np.cos(angle)[:, None, :], np.sin(angle)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return np.concatenate([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], axis=-1)


def visible(i, j, mask):
    """Whether the query at position i sees the key at position j."""
    if j > i:
        return False
    if mask is None:
        return True
    return i - j < mask["size"] or j < mask.get("keep_first", 0)


def softmax_attention(q, k, v, scale, cap, mask, sink):
    """q [T, H, D], k [T, G, D], v [T, G, V] -> [T, H, V]; ``sink`` [H] or None joins every denominator."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]))
    for head in range(H):
        g = head // (H // G)
        for i in range(T):
            js = [j for j in range(i + 1) if visible(i, j, mask)]
            s = soft_cap((k[js, g] @ q[i, head]) * scale, cap)
            top = max(s.max(), sink[head]) if sink is not None else s.max()
            e = np.exp(s - top)
            total = e.sum() + (math.exp(sink[head] - top) if sink is not None else 0.0)
            out[i, head] = (e / total) @ v[js, g]
    return out


def attention(h, w, p, m):
    """No positions; capped scores; a sink per head; a gate per head."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = lin(h, w[p + "q"], w[p + "q.b"]).reshape(T, H, D)
    k = lin(h, w[p + "k"], w[p + "k.b"]).reshape(T, G, D)
    v = lin(h, w[p + "v"], w[p + "v.b"]).reshape(T, G, V)
    out = softmax_attention(q, k, v, m["scale"], m.get("softcap"), None, w[p + "sink"])
    out = out * sigmoid(lin(h, w[p + "g"]))[:, :, None]
    return lin(out.reshape(T, H * V), w[p + "o"])


def attention_2(h, w, p, m, positions, eps):
    """Query and key norms, a partial rotation, capped scores, a sliding window that keeps the first tokens."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_norm(lin(h, w[p + "q"], w[p + "q.b"]).reshape(T, H, D), w[p + "q.norm"], eps)
    k = rms_norm(lin(h, w[p + "k"], w[p + "k.b"]).reshape(T, G, D), w[p + "k.norm"], eps)
    v = lin(h, w[p + "v"], w[p + "v.b"]).reshape(T, G, V)
    rot = m.get("rot") or {"base": 10000.0, "dims": 0}
    q, k = rotate_half(q, positions, rot["base"], rot["dims"]), rotate_half(k, positions, rot["base"], rot["dims"])
    out = softmax_attention(q, k, v, m["scale"], m.get("softcap"), m.get("mask"), None)
    return lin(out.reshape(T, H * V), w[p + "o"])


# ------------------------------------------------------------------------------------------------ feed-forwards
def dense_mlp(h, w, p):
    return lin(gelu_tanh(lin(h, w[p + "gate"])) * lin(h, w[p + "up"]), w[p + "down"])


def route(h, w, p, router):
    """(chosen experts [T, top], their weights [T, top]): softmax scores, only the best groups' experts, not renormalized."""
    z = lin(h, w[p + "router"], exact=True)
    s = np.exp(z - z.max(axis=-1, keepdims=True))
    s = s / s.sum(axis=-1, keepdims=True)
    E, top = router["experts"], router["top"]
    groups = router.get("groups") or {"count": 1, "keep": 1}
    size = E // groups["count"]
    ids, weights = np.zeros((h.shape[0], top), dtype=np.int64), np.zeros((h.shape[0], top))
    for t in range(h.shape[0]):
        best = s[t].reshape(groups["count"], size).max(axis=1)
        kept = sorted(range(groups["count"]), key=lambda g: (-best[g], g))[:groups["keep"]]
        allowed = [e for e in range(E) if e // size in kept]
        chosen = sorted(allowed, key=lambda e: (-s[t, e], e))[:top]
        ids[t], weights[t] = chosen, s[t, chosen]
    return ids, weights


def moe_mlp(h, w, p, mlp):
    ids, weights = route(h, w, p, mlp["router"])
    out = np.zeros((h.shape[0], w[p + "e0.down"].shape[0]))
    for t in range(h.shape[0]):
        for e, weight in zip(ids[t], weights[t]):
            out[t] += weight * lin(gelu_erf(lin(h[t:t + 1], w[f"{p}e{e}.up"])), w[f"{p}e{e}.down"])[0]
    if mlp.get("shared"):
        shared = lin(gelu_erf(lin(h, w[p + "shared.up"])), w[p + "shared.down"])
        out += shared * sigmoid(lin(h, w[p + "shared.sg"], exact=True))
    return out


def token_side(x, w, p, part, eps):
    """The per-layer token input: y = proj(gelu_tanh(gate x) * e), x + y / rms(y) * norm."""
    y = lin(gelu_tanh(lin(x, w[p + "gate"])) * part, w[p + "proj"])
    return x + rms_norm(y, w[p + "norm"], eps)


# ------------------------------------------------------------------------------------------------ the model
def run_order(config):
    """(layer, pass number or None, first of its pass) for every layer run."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, None, False) for i in range(n)]
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, None, False) for i in range(start)]
    for t in range(times):
        order += [(i, t, i == start) for i in range(start, stop)]
    return order + [(i, None, False) for i in range(stop, n)]


def layer_forward(x, config, w, index, tokens, positions):
    layer, eps, p = config["layers"][index], config["norm"]["eps"], f"l{index}."
    h = rms_norm(x, w[p + "norm1"], eps)
    kind, m = layer["type"], layer["mixer"]
    if kind == "mlstm":
        y = mlstm(h, w, p + "mix.", m, eps)
    elif kind == "attention":
        y = attention(h, w, p + "mix.", m)
    elif kind == "attention_2":
        y = attention_2(h, w, p + "mix.", m, positions, eps)
    else:
        raise ValueError(kind)
    mlp = layer.get("mlp")
    if mlp is not None:
        y = y + (dense_mlp(h, w, p + "mlp.") if mlp["kind"] == "dense" else moe_mlp(h, w, p + "mlp.", mlp))
    x = x + y
    side = config.get("token_side")
    if side:
        d = side["dim"]
        x = token_side(x, w, p + "side.", w["side.embed"][tokens][:, index * d:(index + 1) * d], eps)
    return x


def forward(config, w, tokens, return_layers=False):
    """Logits [tokens, vocab] of one sequence from position 0 (and the stream after every layer run)."""
    tokens = np.asarray(tokens, dtype=np.int64)
    positions = np.arange(len(tokens))
    x = w["embed"][tokens]
    first = x.copy()
    after = []
    for index, number, begins in run_order(config):
        if begins:
            if number > 0:
                x = x + first
            x = x + w["loop.step"][number]
        x = layer_forward(x, config, w, index, tokens, positions)
        after.append(x.copy())
    logits = lin(rms_norm(x, w["final.norm"], config["norm"]["eps"]), w["head"])
    return (logits, np.stack(after)) if return_layers else logits
