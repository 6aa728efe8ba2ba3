"""Rarutar's configuration and its place in the registries, and the plain implementation's pieces against direct
arithmetic (no GPU)."""
import copy
import math

import numpy as np
import pytest

import plain_rarutar as plain
import rarutar_helpers as rh
from sprout_lm_b200.config import ConfigError, RarutarConfig, parse_config, registered_architectures
from sprout_lm_b200.models.decoder import DecoderModel


def test_registered_and_round_trip():
    assert "Rarutar" in registered_architectures()
    for raw, _, _ in rh.CONFIGS.values():
        config = parse_config(raw)
        assert isinstance(config, RarutarConfig)
        assert parse_config(config.to_dict()) == config
        assert config.to_dict()["layers"] == raw["layers"]


def test_model_spec_follows_the_file():
    spec = parse_config(rh.A).model_spec()
    assert [layer.mixer.kind for layer in spec.layers] == ["parallel_mixers", "selective_state_space", "multimap_attention",
                                                           "selective_state_space"]
    assert [layer.feed_forward.kind for layer in spec.layers] == ["clamped_glu_mlp", "none", "clamped_glu_mlp", "clamped_glu_mlp"]
    assert [len(layer.norms) for layer in spec.layers] == [2, 1, 2, 2]
    assert spec.embedding.params["scale"] == 1.7 and spec.head.params["tied_to"] == "embed"
    left, right = spec.layers[0].mixer.params["mixers"]
    assert left.kind == "multimap_attention" and right.kind == "gated_linear_attention"
    assert left.params["mask"] == ("window", 5) and not left.params["sink"] and left.params["unit_norm_eps"] == 0.0
    assert left.params["position"].params["scaling"] == {"factor": 4.0, "original": 16.0, "fast": 4.0, "slow": 1.0}
    assert spec.layers[0].mixer.params["scales"] == (1.3, 0.4)
    chunked = spec.layers[2].mixer.params
    assert chunked["mask"] == ("chunk", 7) and chunked["sink"] and chunked["value_from_key"] and chunked["unit_norm_eps"] == 1e-5
    assert chunked["position"].params["scaling"] is None and chunked["position"].params["dims"] == 12
    model = DecoderModel(spec)
    caches = model.cache_specs()
    assert caches[0].kind == "window" and caches[0].window == 5 and caches[0].kv_heads == 3 and caches[0].head_dim == 8 \
        and caches[0].value_dim == 12
    assert caches[1] is None and caches[3] is None and caches[2].kind == "full" and caches[2].value_dim == 12
    states = model.state_specs()
    assert states[0].shape == (1, 12, 8) and states[2] is None
    assert [s.shape for s in states[1]] == [(1, 3 * 8 + 2 * 1 * 5), (3, 5, 8)]           # the convolution's inputs, then S
    assert [s.shape for s in states[3]] == [(3, 4 * 6 + 2 * 4 * 16), (4, 16, 6)]
    names = {decl.name: decl.shape for decl in model.tensor_decls()}
    assert names["embed"] == (211, 40) and names["final.norm.b"] == (40,) and "lm_head" not in names
    assert names["l0.mix.left.q"] == (24, 40) and names["l0.mix.left.v"] == (36, 40) and names["l0.mix.left.g"] == (3, 40)
    assert names["l0.mix.right.a1"] == (5, 40) and names["l0.mix.right.a2"] == (12, 5) and names["l0.mix.right.a2.b"] == (12,)
    assert names["l0.mix.right.norm"] == (8,) and "l0.mix.left.sink" not in names
    assert names["l1.mix.in"] == (2 * 24 + 2 * 5 + 3, 40) and names["l1.mix.conv"] == (34, 2) and "l1.norm2" not in names
    assert names["l2.mix.k"] == (24, 40) and "l2.mix.v" not in names and names["l2.mix.sink"] == (4,)
    assert names["l3.mix.norm"] == (24,) and names["l3.mix.D"] == (4,) and names["l3.mlp.down"] == (40, 32)


@pytest.mark.parametrize("edit, text", [
    (lambda c: c["layers"][2]["mixer"].__setitem__("heads", 5), "multiple of kv_heads"),
    (lambda c: c["layers"][2]["mixer"]["rot"].__setitem__("dims", 14), "rot.dims"),
    (lambda c: c["layers"][2]["mixer"]["rot"].__setitem__("dims", 5), "rot.dims"),
    (lambda c: c["layers"][2]["mixer"].__setitem__("vdim", 8), "values are the keys"),
    (lambda c: c["layers"][2]["mixer"].pop("mask"), "mask"),
    (lambda c: c["layers"][2]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"]["scaling"].pop("slow"), "slow"),
    (lambda c: c["layers"][0]["mixer"].pop("right"), "left and right"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("left_scale", "x"), "left_scale"),
    (lambda c: c["layers"][0]["mixer"]["right"].__setitem__("tau", 0), "tau"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("groups", 2), "multiple of groups"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("norm_groups", 5), "norm_groups"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("conv", 1), "conv"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "moe"), "dense"),
    (lambda c: c["layers"][0]["mlp"].pop("limit"), "limit"),
    (lambda c: c["layers"][0].__setitem__("type", "window"), "type"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c["embedding"].pop("scale"), "embedding.scale"),
    (lambda c: c.pop("width"), "width"),
    (lambda c: c.__setitem__("layers", []), "layers"),
])
def test_refusals(edit, text):
    raw = copy.deepcopy(rh.A)
    edit(raw)
    with pytest.raises(ConfigError, match=text):
        parse_config(raw)


def test_rotary_tables_of_the_package_are_the_plain_frequencies():
    """The stretched frequencies and the factor on cos and sin, for ramps that start inside, before and after the table."""
    from types import SimpleNamespace
    from sprout_lm_b200.config.specs import PartSpec
    from sprout_lm_b200.parts import build_part
    for dims, base, scaling in [(16, 3000.0, None), (8, 100.0, (4.0, 16, 4.0, 1.0)), (32, 8000.0, (8.0, 64, 16.0, 1.0)),
                                (6, 700.0, (16.0, 32, 8.0, 2.0)), (2, 20.0, (2.0, 8, 2.0, 0.5)), (12, 50.0, (3.0, 4096, 1.0, 1.0))]:
        rot = rh.rot(base, dims, scaling)
        part = build_part("position", PartSpec("rope_yarn", {"dims": dims, "theta": base, "max_positions": 40,
                                                               "scaling": rot.get("scaling")}), "")
        cos, sin = part.rotary_tables(SimpleNamespace(device="cpu"))
        f, magnitude = plain.rotary_frequencies(dims, base, rot.get("scaling"))
        angle = np.arange(40)[:, None] * f[None, :]
        assert np.abs(cos.numpy() - np.cos(angle) * magnitude).max() < 1e-6
        assert np.abs(sin.numpy() - np.sin(angle) * magnitude).max() < 1e-6


def test_plain_mechanisms_agree_with_their_definitions():
    """The oracle's own pieces against direct arithmetic on tiny inputs."""
    rng = np.random.default_rng(0)
    x, w, b = rng.normal(2.0, 1.0, size=(3, 6)), rng.normal(size=6), rng.normal(size=6)
    assert np.allclose(plain.layer_norm(x, w, b, 1e-5), (x - x.mean(-1, keepdims=True)) / np.sqrt(x.var(-1, keepdims=True) + 1e-5) * w + b)
    assert np.allclose(plain.rms_unit(x, 1e-3), x / np.sqrt((x ** 2).mean(-1, keepdims=True) + 1e-3))
    # rotation: position 0 is the identity, a pair turns by its angle, the tail passes
    v = rng.normal(size=(2, 1, 8))
    turned = plain.rotate(v, [0, 3], {"base": 100.0, "dims": 4})
    assert np.allclose(turned[0], v[0]) and np.allclose(turned[1, 0, 4:], v[1, 0, 4:])
    angle = 3 * 100.0 ** (-2.0 / 4)
    assert np.isclose(turned[1, 0, 1], v[1, 0, 1] * np.cos(angle) - v[1, 0, 3] * np.sin(angle))
    assert np.isclose(turned[1, 0, 3], v[1, 0, 3] * np.cos(angle) + v[1, 0, 1] * np.sin(angle))
    # stretched frequencies: below the ramp untouched, above it divided by the factor
    f, magnitude = plain.rotary_frequencies(8, 100.0, {"factor": 4.0, "original": 16, "fast": 4.0, "slow": 1.0})
    lo = max(math.floor(8 * math.log(16 / (2 * math.pi * 4.0)) / (2 * math.log(100.0))), 0)
    hi = min(math.ceil(8 * math.log(16 / (2 * math.pi * 1.0)) / (2 * math.log(100.0))), 7)
    plainf = 100.0 ** (-2.0 * np.arange(4) / 8)
    assert np.isclose(f[lo], plainf[lo]) and np.allclose(f[hi:], plainf[hi:] / 4.0) and np.isclose(magnitude, 0.1 * math.log(4.0) + 1)
    # masks
    assert [plain.first_visible("window", 3, i) for i in range(6)] == [0, 0, 0, 1, 2, 3]
    assert [plain.first_visible("chunk", 3, i) for i in range(7)] == [0, 0, 0, 3, 3, 3, 6]
    # a sink takes its share: with equal scores s over n keys, the weights are e^s / (n e^s + e^sink)
    q, k = np.zeros((4, 1, 2)), np.zeros((4, 1, 2))
    val = rng.normal(size=(4, 1, 3))
    out = plain.masked_softmax_attention(q, k, val, 1.0, "chunk", 8, sink=np.array([math.log(2.0)]))
    assert np.allclose(out[3, 0], val[:4, 0].sum(axis=0) / (4 + 2.0))
    out = plain.masked_softmax_attention(q, k, val, 1.0, "window", 2)
    assert np.allclose(out[3, 0], val[2:4, 0].mean(axis=0))
    # gated linear attention in closed form: o_t = sum_j (prod_{j<s<=t} alpha_s) * k_j (q_t . ) v_j, per key channel
    T, d, dv = 5, 3, 2
    h = rng.normal(size=(T, 4))
    wts = {"p.q": rng.normal(size=(d, 4)), "p.k": rng.normal(size=(d, 4)), "p.v": rng.normal(size=(dv, 4)), "p.g": rng.normal(size=(dv, 4)),
           "p.a1": rng.normal(size=(2, 4)), "p.a2": rng.normal(size=(d, 2)), "p.a2.b": rng.normal(size=d), "p.norm": rng.normal(size=dv),
           "p.o": np.eye(dv)}
    got, _ = plain.gated_linear_attention(h, wts, "p.", {"heads": 1, "dim": d, "vdim": dv, "tau": 3.0}, 1e-6)
    alpha = plain.sigmoid(h @ wts["p.a1"].T @ wts["p.a2"].T + wts["p.a2.b"]) ** (1 / 3.0)
    qv, kv, vv = h @ wts["p.q"].T * d ** -0.5, h @ wts["p.k"].T, h @ wts["p.v"].T
    o = sum(((np.prod(alpha[j + 1:T], axis=0) * kv[j]) @ qv[T - 1]) * vv[j] for j in range(T))
    want = o / np.sqrt((o ** 2).mean() + 1e-6) * wts["p.norm"] * plain.silu(h[T - 1] @ wts["p.g"].T)
    assert np.allclose(got[T - 1], want)
    # the convolution: the last column is the current token's
    xs = rng.normal(size=(4, 2))
    cw, cb = rng.normal(size=(2, 3)), rng.normal(size=2)
    y = plain.causal_conv(xs, cw, cb)
    assert np.allclose(y[0], cb + cw[:, 2] * xs[0]) and np.allclose(y[3], cb + cw[:, 0] * xs[1] + cw[:, 1] * xs[2] + cw[:, 2] * xs[3])
    # the feed-forward clamps the gate from above only, the other factor on both sides
    m = {"f.gate": np.array([[1.0], [1.0]]), "f.up": np.array([[1.0], [-1.0]]), "f.down": np.eye(2)}
    out = plain.clamped_glu(np.array([[5.0]]), m, "f.", {"limit": 2.0})
    assert np.allclose(out[0], [2.0 * plain.sigmoid(1.702 * 2.0) * 3.0, 2.0 * plain.sigmoid(1.702 * 2.0) * -1.0])
    out = plain.clamped_glu(np.array([[-5.0]]), m, "f.", {"limit": 2.0})
    assert np.allclose(out[0], [-5.0 * plain.sigmoid(1.702 * -5.0) * -1.0, -5.0 * plain.sigmoid(1.702 * -5.0) * 3.0])


def test_the_plain_state_space_in_closed_form():
    """y_t = sum_j exp(A sum_{j<s<=t} dt_s) dt_j (C_t . B_j) x_j + D x_t on a model of one head without a convolution's memory."""
    rng = np.random.default_rng(3)
    T, P, N, width = 6, 2, 3, 5
    m = {"heads": 1, "vdim": P, "state": N, "groups": 1, "conv": 2, "norm_groups": 1}
    channels = P + 2 * N
    conv = np.zeros((channels, 2))
    conv[:, 1] = 1.0                                                     # only the current token's tap
    w = {"p.in": rng.normal(size=(2 * P + 2 * N + 1, width)), "p.conv": conv, "p.conv.b": np.zeros(channels),
         "p.dt_bias": np.array([0.3]), "p.A_log": np.array([-0.5]), "p.D": np.array([0.7]), "p.norm": rng.normal(size=P), "p.o": np.eye(P)}
    h = rng.normal(size=(T, width))
    got = plain.mamba2_mixer(h, w, "p.", m, 1e-6)
    row = h @ w["p.in"].T
    z, xbc, dt = row[:, :P], plain.silu(row[:, P:P + channels]), plain.softplus(row[:, -1] + 0.3)
    x, B, C = xbc[:, :P], xbc[:, P:P + N], xbc[:, P + N:]
    A = -math.exp(-0.5)
    t = T - 1
    y = sum(math.exp(A * dt[j + 1:t + 1].sum()) * dt[j] * (C[t] @ B[j]) * x[j] for j in range(T)) + 0.7 * x[t]
    y = y * plain.silu(z[t])
    want = y / np.sqrt((y ** 2).mean() + 1e-6) * w["p.norm"]
    assert np.allclose(got[t], want)
