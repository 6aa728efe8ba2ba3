"""Vuripel's configuration and its place in the registries, the cache manager's kept first pages, and the plain
implementation's pieces against direct arithmetic (no GPU)."""
import copy
import math

import numpy as np
import pytest

import plain_vuripel as plain
import vuripel_helpers as vh
from sprout_lm_b200.cache.manager import CacheManager, GroupSpec
from sprout_lm_b200.config import ConfigError, VuripelConfig, parse_config, registered_architectures
from sprout_lm_b200.models.decoder import DecoderModel


def test_registered_and_round_trip():
    assert "Vuripel" in registered_architectures()
    for raw, _, _ in vh.CONFIGS.values():
        config = parse_config(raw)
        assert isinstance(config, VuripelConfig)
        assert parse_config(config.to_dict()) == config
        assert config.to_dict() == raw


def test_model_spec_follows_the_file():
    spec = parse_config(vh.A).model_spec()
    assert [layer.block for layer in spec.layers] == ["parallel_residual"] * 4
    assert [layer.mixer.kind for layer in spec.layers] == ["multimap_attention", "exp_gated_matrix_memory", "multimap_attention",
                                                           "exp_gated_matrix_memory"]
    assert [layer.feed_forward.kind for layer in spec.layers] == ["gated_mlp", "routed_experts", "none", "gated_mlp"]
    assert all(len(layer.norms) == 1 for layer in spec.layers)
    windowed = spec.layers[0].mixer.params
    assert windowed["mask"] == ("window", 5, 2) and windowed["softcap"] == 2.0 and windowed["qk_norm_eps"] == 1e-5
    assert windowed["bias"] and not windowed["sink"] and not windowed["gate"] and windowed["position"].params["dims"] == 4
    full = spec.layers[2].mixer.params
    assert full["mask"] is None and full["sink"] and full["gate"] and full["bias"] and full["qk_norm_eps"] == 0.0
    assert full["position"].kind == "none" and full["softcap"] == 1.2 and full["scale"] == 0.9
    assert spec.layers[1].mixer.params["gate_cap"] == 3.0 and spec.layers[3].mixer.params["gate_cap"] is None
    routed = spec.layers[1].feed_forward.params
    assert routed["groups"] == (3, 1) and routed["top"] == 2 and not routed["renormalize"] and not routed["correction"]
    assert routed["expert_kind"] == "plain" and routed["shared_ff"] == 12 and routed["shared_gate"]
    side = [layer.options["side"].params for layer in spec.layers]
    assert [s["first"] for s in side] == [0, 6, 12, 18] and [s["declares_table"] for s in side] == [True, False, False, False]
    # layers 1 and 2 run three times: every run has a cache slot and a state entry of its own
    assert [(c.layer, c.cache) for c in spec.order] == [(0, 0), (1, 1), (2, 2), (1, 4), (2, 5), (1, 6), (2, 7), (3, 3)]
    assert spec.stream.kind == "loop_restart" and spec.stream.params["starts"] == (1, 3, 5)
    model = DecoderModel(spec)
    caches = model.cache_specs()
    assert (caches[0].kind, caches[0].window, caches[0].keep_first) == ("window", 5, 2) and caches[0].value_dim == 12
    assert caches[1] is None and caches[4] is None and caches[6] is None and caches[3] is None
    assert all(caches[i].kind == "full" and caches[i].kv_heads == 2 and caches[i].head_dim == 12 for i in (2, 5, 7))
    states = model.state_specs()
    assert [s.shape for s in states[1]] == [(3, 12, 8), (3,)] and [s.shape for s in states[3]] == [(1, 20, 24), (1,)]
    assert states[0] is None and states[2] is None and states[5] is None and states[7] is None
    assert [s.shape for s in states[4]] == [(3, 12, 8), (3,)] and [s.shape for s in states[6]] == [(3, 12, 8), (3,)]
    names = {decl.name: decl.shape for decl in model.tensor_decls()}
    assert names["embed"] == (203, 40) and names["head"] == (203, 40) and names["loop.step"] == (3, 40)
    assert names["side.embed"] == (203, 24) and names["l2.side.gate"] == (6, 40) and names["l2.side.proj"] == (40, 6)
    assert names["l0.mix.q"] == (24, 40) and names["l0.mix.q.b"] == (24,) and names["l0.mix.v.b"] == (36,)
    assert names["l0.mix.q.norm"] == (8,) and names["l0.mix.k.norm"] == (8,) and "l0.mix.sink" not in names
    assert names["l2.mix.sink"] == (4,) and names["l2.mix.g"] == (4, 40) and "l2.mix.q.norm" not in names
    assert names["l1.mix.i"] == (3, 40) and names["l1.mix.f.b"] == (3,) and names["l1.mix.norm"] == (21,)
    assert names["l1.mlp.router"] == (6, 40) and names["l1.mlp.e5.up"] == (20, 40) and "l1.mlp.e0.gate" not in names
    assert names["l1.mlp.shared.sg"] == (1, 40) and names["l1.mlp.shared.down"] == (40, 12) and "l1.mlp.correction" not in names
    assert "l2.mlp.gate" not in names and names["l3.mlp.gate"] == (27, 40)


def test_a_model_without_loop_or_token_input():
    spec = parse_config(vh.B).model_spec()
    assert spec.stream is None and all("side" not in layer.options for layer in spec.layers)
    assert [(c.layer, c.cache, c.state) for c in spec.order] == [(i, i, None) for i in range(5)]
    assert spec.layers[3].mixer.params["mask"] is None and spec.layers[3].mixer.params["position"].kind == "none"
    assert spec.layers[1].mixer.params["mask"] == ("window", 33, 0)
    assert spec.layers[0].feed_forward.params["groups"] is None and spec.layers[0].feed_forward.params["shared_ff"] is None
    names = {decl.name for decl in DecoderModel(spec).tensor_decls()}
    assert "loop.step" not in names and "side.embed" not in names and "l0.mlp.shared.sg" not in names


@pytest.mark.parametrize("edit, text", [
    (lambda c: c["layers"][0]["mixer"].__setitem__("heads", 4), "multiple of kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 10), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["mask"].__setitem__("size", 0), "mask.size"),
    (lambda c: c["layers"][0]["mixer"]["mask"].__setitem__("keep_first", -1), "keep_first"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].__setitem__("count", 4), "groups"),
    (lambda c: c["layers"][1]["mlp"]["router"].__setitem__("top", 3), "groups"),
    (lambda c: c["layers"][1].__setitem__("type", "mamba2"), "type"),
    (lambda c: c["layers"][3]["mlp"].__setitem__("kind", "sparse"), "kind"),
    (lambda c: c["loop"].__setitem__("stop", 5), "loop"),
    (lambda c: c["loop"].__setitem__("times", 0), "loop"),
    (lambda c: c["norm"].__setitem__("eps", 0), "eps"),
    (lambda c: c["token_side"].__setitem__("dim", 0), "token_side"),
    (lambda c: c.__setitem__("vocab", 0), "vocab"),
])
def test_refusals(edit, text):
    raw = copy.deepcopy(vh.A)
    edit(raw)
    with pytest.raises(ConfigError, match=text):
        parse_config(raw)


def test_window_group_keeps_the_first_pages():
    """A window group with kept first positions gives back the pages between them and the window, never theirs."""
    manager = CacheManager([GroupSpec("w", "window", window=10, keep_first=5, slots=(0,)), GroupSpec("f", "full", slots=(1,))],
                           num_pages=16, page_tokens=4, prefix_caching=False)
    seq = manager.create()
    for upto in range(4, 44, 4):
        assert manager.reserve(seq, upto)
    seq.length = 40
    assert manager.trim(seq) == 5                       # pages 2 .. 6: positions 8 .. 27 (the next query sees from 31 on)
    assert [page >= 0 for page in seq.tables[0]] == [True, True] + [False] * 5 + [True] * 3
    assert all(page >= 0 for page in seq.tables[1])
    manager.release(seq)
    manager.check_invariants()
    assert manager.free_pages(0) == 16 and manager.free_pages(1) == 16
    with pytest.raises(Exception):
        GroupSpec("x", "full", keep_first=3)


# ------------------------------------------------------------------------------------------------ the plain pieces
def test_plain_pieces_against_direct_arithmetic():
    assert plain.gelu_tanh(np.array([1.0]))[0] == pytest.approx(0.8411919906082768)
    assert plain.gelu_erf(np.array([1.0]))[0] == pytest.approx(0.8413447460685429)
    assert plain.log_sigmoid(np.array([0.0, 40.0, -40.0])) == pytest.approx([-math.log(2), 0.0, -40.0], abs=1e-12)
    assert plain.soft_cap(np.array([100.0]), 5.0)[0] == pytest.approx(5.0) and plain.soft_cap(np.array([3.0]), None)[0] == 3.0
    # a window of 3 that keeps the first 2: position 6 sees 0, 1, 4, 5, 6
    mask = {"size": 3, "keep_first": 2}
    assert [j for j in range(8) if plain.visible(6, j, mask)] == [0, 1, 4, 5, 6]
    # one head, one step from zero: S = e^(i - m) k v^T with m = max(f, i); the normaliser decides the output's size
    q, k, v = np.array([[[2.0, 0.0]]]), np.array([[[1.0, 3.0]]]), np.array([[[5.0, 7.0, 9.0]]])
    out, (S, n, top) = plain.exp_gated_memory(q, k, v, np.array([[1.5]]), np.array([[-0.2]]))
    assert top[0] == 1.5 and S[0] == pytest.approx(np.outer(k[0, 0], v[0, 0])) and n[0] == pytest.approx(k[0, 0])
    assert out[0, 0] == pytest.approx(2.0 * v[0, 0] / (2.0 + 1e-6))
    # a small input gate: the running maximum stays at f + 0, and exp(-m) bounds the denominator from below
    out, (_, _, top) = plain.exp_gated_memory(q, k, v, np.array([[-3.0]]), np.array([[-0.5]]))
    scale = math.exp(-3.0 + 0.5)
    assert top[0] == -0.5 and out[0, 0] == pytest.approx(scale * 2.0 * v[0, 0] / (max(scale * 2.0, math.exp(0.5)) + 1e-6))
    # the sink takes weight and has no value
    one = plain.softmax_attention(np.ones((1, 1, 2)), np.ones((1, 1, 2)), np.array([[[4.0]]]), 1.0, None, None, np.array([2.0]))
    assert one[0, 0, 0] == pytest.approx(4.0 * 0.5)
    # routing: groups (0,1) (2,3) (4,5); the best two groups are those of experts 4 and 1; experts 2, 3 cannot be taken
    w = {"r.router": np.eye(6)}
    ids, weights = plain.route(np.array([[0.1, 2.0, 1.9, 1.8, 3.0, -1.0]]), w, "r.", {"experts": 6, "top": 3, "groups": {"count": 3, "keep": 2}})
    assert list(ids[0]) == [4, 1, 0] and weights[0].sum() < 1.0


def test_run_order_of_the_plain_model():
    assert plain.run_order(vh.A) == [(0, None, False), (1, 0, True), (2, 0, False), (1, 1, True), (2, 1, False), (1, 2, True),
                                     (2, 2, False), (3, None, False)]
    assert plain.run_order(vh.B) == [(i, None, False) for i in range(5)]
