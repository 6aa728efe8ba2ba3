"""Vuripel on the GPU against the plain implementation: every mechanism alone (with inputs made so that a fault shows),
then whole models under every way of cutting the work, through the step function, the trace replay program and the
scheduler."""
import copy
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import helpers
import plain_vuripel as plain
import vuripel_helpers as vh

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 6e-5, "bfloat16": 6e-2}       # of the logits' spread over the vocabulary at that place (vuripel_helpers.relative)


def rounded(array, dtype):
    """float32 values that ``dtype`` holds exactly."""
    return torch.from_numpy(np.asarray(array, dtype=np.float32)).to(DTYPES[dtype]).float()


def dev(array, dtype=None):
    t = array if isinstance(array, torch.Tensor) else torch.from_numpy(np.ascontiguousarray(array))
    return (t.to(DTYPES[dtype]) if dtype else t).to(DEV)


def ints(values):
    return torch.tensor(list(values), dtype=torch.int32, device=DEV)


def f64(t):
    return t.numpy().astype(np.float64)


def new_status():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


# =============================================================================== mechanisms alone
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_row_kernels(dtype):
    """Activations (gated and not), the gated token row, the normed sum, the passes' vector, the gated sum."""
    from sprout_lm_b200 import kernels
    rng = np.random.default_rng(0)
    tol = 4e-6 if dtype == "float32" else 2e-2
    acts = {"silu": lambda z: z * plain.sigmoid(z), "gelu_tanh": plain.gelu_tanh, "gelu_erf": plain.gelu_erf}
    for ff in (19, 64, 7):
        rows = rounded(rng.normal(0, 2.0, size=(6, 2 * ff + 3)), dtype)
        for name, fn in acts.items():
            out = torch.empty(6, ff, dtype=DTYPES[dtype], device=DEV)
            kernels.unit_act(dev(rows, dtype), out, name, gated=True)
            want = fn(f64(rows)[:, :ff]) * f64(rows)[:, ff:2 * ff]
            assert (np.abs(out.float().cpu().numpy() - want) <= tol * (1 + np.abs(want))).all(), (name, ff)
            kernels.unit_act(dev(rows, dtype)[:, 2:2 + ff], out, name, gated=False)
            assert (np.abs(out.float().cpu().numpy() - fn(f64(rows)[:, 2:2 + ff])) <= tol * (1 + np.abs(f64(rows)[:, 2:2 + ff]))).all(), (name, ff)
    # the two forms of gelu differ by more than the bar somewhere: a mix-up would show
    z = np.linspace(-3, 3, 61)
    assert np.abs(plain.gelu_tanh(z) - plain.gelu_erf(z)).max() > 2e-4
    status = new_status()
    table = rounded(rng.normal(size=(23, 30)), dtype)
    z = rounded(rng.normal(0, 1.5, size=(5, 9)), dtype)
    tokens = [22, 0, 7, 7, 13]
    out = torch.empty(5, 6, dtype=DTYPES[dtype], device=DEV)
    kernels.side_gate(dev(z, dtype)[:, :6], dev(table, dtype), 12, ints(tokens), out, status)
    want = plain.gelu_tanh(f64(z)[:, :6]) * f64(table)[tokens][:, 12:18]
    assert np.abs(out.float().cpu().numpy() - want).max() <= tol * 4 and int(status.item()) == 0
    kernels.side_gate(dev(z, dtype)[:, :6], dev(table, dtype), 12, ints([1, 2, 23, 3, 4]), out, status)
    assert int(status.item()) == 2                                           # a token beyond the table is flagged, not read
    status.zero_()
    # the whole per-layer token input in one launch, for a handful of tokens
    for width, dim in ((40, 6), (128, 16), (200, 24)):
        x = rng.normal(0, 2.0, size=(5, width)).astype(np.float32)
        parts = {"s.gate": rounded(rng.normal(0, 0.3, size=(dim, width)), dtype), "s.proj": rounded(rng.normal(0, 0.3, size=(width, dim)), dtype)}
        gain = rng.normal(1.0, 0.3, size=width).astype(np.float32)
        wide = rounded(rng.normal(size=(23, 3 * dim)), dtype)
        got = dev(x.copy())
        kernels.side_input_few(got, dev(parts["s.gate"], dtype), dev(parts["s.proj"], dtype), dev(gain), dev(wide, dtype), dim, ints(tokens),
                               1e-5, status)
        w = {key: f64(value) for key, value in parts.items()} | {"s.norm": gain.astype(np.float64)}
        want = plain.token_side(x.astype(np.float64), w, "s.", f64(wide)[tokens][:, dim:2 * dim], 1e-5)
        assert np.abs(got.cpu().numpy() - want).max() <= (2e-5 if dtype == "float32" else 5e-2), (width, dim)
    status.zero_()
    # a gate per row on an activation
    rows = rounded(rng.normal(0, 2.0, size=(6, 20)), dtype)
    logits = rng.normal(0, 2.0, size=(6, 2)).astype(np.float32)
    out = torch.empty(6, 20, dtype=DTYPES[dtype], device=DEV)
    kernels.unit_act(dev(rows, dtype), out, "gelu_erf", gated=False, row_logits=dev(logits)[:, 1:])
    want = plain.gelu_erf(f64(rows)) * plain.sigmoid(logits[:, 1:].astype(np.float64))
    assert (np.abs(out.float().cpu().numpy() - want) <= tol * (1 + np.abs(want))).all()
    if dtype == "bfloat16":
        return
    for width in (40, 257, 1030):
        x = rng.normal(size=(4, width)).astype(np.float32)
        y = rng.normal(0, 3.0, size=(4, width)).astype(np.float32)
        w = rng.normal(1.0, 0.3, size=width).astype(np.float32)
        got = dev(x.copy())
        kernels.rms_add(dev(y), dev(w), got, 1e-5)
        assert np.abs(got.cpu().numpy() - (x + plain.rms_norm(y.astype(np.float64), w, 1e-5))).max() <= 4e-6
        got, vec = dev(x.copy()), rng.normal(size=width).astype(np.float32)
        kernels.add_rows(got, dev(vec))
        assert np.abs(got.cpu().numpy() - (x + vec)).max() <= 1e-6
        kernels.add_rows(got, dev(vec), other=dev(y))
        assert np.abs(got.cpu().numpy() - (x + 2 * vec.astype(np.float64) + y)).max() <= 2e-6
        got, logits = dev(x.copy()), rng.normal(0, 2.0, size=(4, 3)).astype(np.float32)
        kernels.gated_rows_add(got, dev(y), dev(logits)[:, 1:2])
        assert np.abs(got.cpu().numpy() - (x + plain.sigmoid(logits[:, 1:2].astype(np.float64)) * y)).max() <= 4e-6
        narrow = kernels.narrow_rows(dev(x))
        assert torch.equal(narrow.cpu(), torch.from_numpy(x).to(torch.bfloat16))


def test_gated_gelu_in_the_products_epilogue():
    """The dense feed-forward's first product with the tanh form of gelu on its accumulators (gate and up rows interleaved
    in blocks of 8), for few tokens (weights on the MMA's rows) and many (tokens on them), beside silu."""
    from sprout_lm_b200 import kernels
    from sprout_lm_b200.parts.mlp import interleave_gate_up
    rng = np.random.default_rng(6)
    status = new_status()
    for tokens, width, ff in ((5, 64, 48), (70, 128, 160), (300, 64, 256), (33, 40, 56)):
        a = rounded(rng.normal(size=(tokens, width)), "bfloat16")
        gate, up = rounded(rng.normal(0, 0.3, size=(ff, width)), "bfloat16"), rounded(rng.normal(0, 0.3, size=(ff, width)), "bfloat16")
        fused = dev(interleave_gate_up(gate, up, 8), "bfloat16")
        for name, fn in (("gelu_tanh", plain.gelu_tanh), ("silu", lambda z: z * plain.sigmoid(z))):
            out = torch.empty(tokens, ff, dtype=torch.bfloat16, device=DEV)
            kernels.gemm_bf16(dev(a, "bfloat16"), fused, out, status, swiglu=True, gate_activation=name)
            want = fn(f64(a) @ f64(gate).T) * (f64(a) @ f64(up).T)
            assert (np.abs(out.float().cpu().numpy() - want) <= 1e-2 * (1 + np.abs(want))).all(), (tokens, width, ff, name)
    assert int(status.item()) == 0


def _memory_inputs(rng, lengths, H, D, V, cap):
    """Projections and gate inputs per request; the forget gates run from fast to very slow, the input gates are wide, so
    the running maximum moves, and some steps push it far up."""
    out = []
    for n in lengths:
        zi = rng.normal(0, 2.0, size=(n, H)) + (rng.random(size=(n, H)) < 0.05) * 9.0
        zf = rng.normal(0, 1.0, size=(n, H)) + np.linspace(0.0, 6.0, H)[None, :]
        out.append({"q": rng.normal(size=(n, H, D)), "k": rng.normal(size=(n, H, D)), "v": rng.normal(size=(n, H, V)),
                    "zi": zi, "zf": zf})
    for r in out:
        for key in r:
            r[key] = r[key].astype(np.float32).astype(np.float64)
    return out


def _run_memory(kernels, requests, pieces, slots, state, H, D, V, cap, bias_i, bias_f):
    """One step: request r brings tokens pieces[r] = (from, to).  Returns per request o [tokens, H, V] and n . q, m."""
    status = new_status()
    cols = state[0].shape[-1]
    cat = lambda key, width: np.concatenate([requests[r][key][a:b].reshape(b - a, width) for r, (a, b) in pieces.items()])
    counts = [b - a for a, b in pieces.values()]
    rows = np.concatenate([cat("q", H * D), cat("k", H * D), cat("v", H * V), cat("zi", H), cat("zf", H)], axis=1).astype(np.float32)
    rows = dev(rows)
    q_start = ints(np.concatenate([[0], np.cumsum(counts)]))
    ctx = SimpleNamespace(q_start=q_start, max_q_len=max(counts))
    slot_ids = ints([slots[r] for r in pieces])
    at = 2 * H * D + H * V
    a, c, m = kernels.exp_gates(rows[:, at:at + H], rows[:, at + H:at + 2 * H], dev(bias_i), dev(bias_f), cap or 0.0, ctx, state[1],
                                slot_ids, status)
    o = torch.empty(rows.shape[0], H * cols, dtype=torch.float32, device=DEV)
    kernels.gated_scan(rows[:, :H * D], rows[:, H * D:2 * H * D], rows[:, 2 * H * D:at], None, None, ctx,
                       SimpleNamespace(buffer=state[0], slots=slot_ids), o, H, H, D, cols, status, q_scale=D ** -0.5, given=(a, c),
                       ones_col=True)
    assert int(status.item()) == 0
    return o.cpu().numpy().reshape(-1, H, cols), m.cpu().numpy(), counts


@pytest.mark.parametrize("sizes", [(3, 12, 7, 6.0), (1, 20, 20, None), (2, 64, 64, 12.0), (2, 16, 33, 10.0), (5, 8, 48, 3.0)])
def test_matrix_memory_whole_portions_and_single_tokens(sizes):
    """Gates, scan and normaliser against the recurrence in float64: requests of unequal length in one batch (long ones
    walk chunks side by side), then the same requests in portions of changing size from states that are not zero, in
    other slots that were used before, then token by token."""
    from sprout_lm_b200 import kernels
    H, D, V, cap = sizes
    rng = np.random.default_rng(H * 100 + D)
    lengths = [300, 1, 129, 64, 5]
    requests = dict(enumerate(_memory_inputs(rng, lengths, H, D, V, cap)))
    bias_i, bias_f = rng.normal(0, 0.5, size=H).astype(np.float32), rng.uniform(0.0, 3.0, size=H).astype(np.float32)
    cols = (V + 1 + 3) // 4 * 4
    want = {}
    for r, item in requests.items():
        gi, gf = plain.log_gates(item["zi"] + bias_i, item["zf"] + bias_f, cap)
        parts = []
        _, (S, n, top) = plain.exp_gated_memory(item["q"] * D ** -0.5, item["k"], item["v"], gi, gf, parts=parts)
        want[r] = (np.concatenate([parts[0], parts[1][:, :, None], parts[2][:, :, None]], axis=2), S, n, top)   # [S^T q | n . q | m]

    def fresh(slots_total):
        # slots hold rubbish from earlier use; a request's slot is zeroed when it takes it, as the cache manager does
        return (torch.full((slots_total, H, D, cols), 7.0, dtype=torch.float32, device=DEV),
                torch.full((slots_total, H), -3.0, dtype=torch.float32, device=DEV))

    def check(state, slots, got_o, label):
        for r, (o, S, n, top) in want.items():
            scale = max(1.0, np.abs(o).max())
            assert np.abs(got_o[r] - o).max() <= 2e-4 * scale, (label, r, np.abs(got_o[r] - o).max())
            memory = state[0][slots[r]].cpu().numpy()
            big = max(1.0, np.abs(S).max())
            assert np.abs(memory[:, :, :V] - S).max() <= 1e-4 * big and np.abs(memory[:, :, V] - n).max() <= 1e-4 * big, (label, r)
            assert np.abs(state[1][slots[r]].cpu().numpy() - top).max() <= 1e-4, (label, r)

    # all at once
    state, slots = fresh(6), {0: 4, 1: 0, 2: 5, 3: 2, 4: 1}
    for s in slots.values():
        state[0][s].zero_(); state[1][s].zero_()
    o, m, counts = _run_memory(kernels, requests, {r: (0, n) for r, n in enumerate(lengths)}, slots, state, H, D, V, cap, bias_i, bias_f)
    got, at = {}, 0
    for r, n in enumerate(lengths):
        got[r] = _parts(o[at:at + n], m[at:at + n], V)
        at += n
    check(state, slots, got, "whole")
    # portions of changing size, several requests per step, from the states the steps before left
    state, slots = fresh(5), {0: 1, 1: 3, 2: 0, 3: 4, 4: 2}
    for s in slots.values():
        state[0][s].zero_(); state[1][s].zero_()
    sizes_cycle, done, got, k = (17, 2, 131, 1, 64, 3, 128), {r: 0 for r in requests}, {r: [] for r in requests}, 0
    while any(done[r] < lengths[r] for r in requests):
        pieces = {}
        for r in requests:
            if done[r] < lengths[r] and (r + k) % 3 != 0:
                n = min(sizes_cycle[(k + r) % len(sizes_cycle)], lengths[r] - done[r])
                pieces[r] = (done[r], done[r] + n)
        k += 1
        if not pieces:
            continue
        o, m, counts = _run_memory(kernels, requests, pieces, slots, state, H, D, V, cap, bias_i, bias_f)
        at = 0
        for r, (a, b) in pieces.items():
            got[r].append(_parts(o[at:at + b - a], m[at:at + b - a], V))
            at += b - a
            done[r] = b
    check(state, slots, {r: np.concatenate(parts) for r, parts in got.items()}, "portions")
    # token by token (the two short requests and the start of a long one)
    state, slots = fresh(3), {1: 2, 4: 0, 3: 1}
    for s in slots.values():
        state[0][s].zero_(); state[1][s].zero_()
    got = {r: [] for r in slots}
    for t in range(40):
        pieces = {r: (t, t + 1) for r in slots if t < lengths[r]}
        o, m, _ = _run_memory(kernels, requests, pieces, slots, state, H, D, V, cap, bias_i, bias_f)
        for i, r in enumerate(pieces):
            got[r].append(_parts(o[i:i + 1], m[i:i + 1], V))
    for r in slots:
        n = min(40, lengths[r])
        assert np.abs(np.concatenate(got[r]) - want[r][0][:n]).max() <= 2e-4 * max(1.0, np.abs(want[r][0]).max()), ("single", r)


def _parts(o, m, V):
    """The scan's rows and the running maxima side by side: [S^T q | n . q | m] per head."""
    return np.concatenate([o[:, :, :V + 1], m[:, :, None]], axis=2)


def _normalised(o, m, V):
    """What exp_memory_out does before its norm: o / (max(|n . q|, exp(-m)) + 1e-6)."""
    return o[:, :, :V] / (np.maximum(np.abs(o[:, :, V]), np.exp(-m.astype(np.float64))) + 1e-6)[:, :, None]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_matrix_memory_output(dtype):
    """The denominator from the normaliser and the running maximum, the norm per head, the weight, the sigmoid gate."""
    from sprout_lm_b200 import kernels
    rng = np.random.default_rng(3)
    for H, V in ((3, 7), (2, 64), (1, 20)):
        cols = (V + 1 + 3) // 4 * 4
        o = rng.normal(size=(9, H, cols)).astype(np.float32)
        o[:, :, V] *= np.array([1e-3, 1.0, 30.0])[rng.integers(0, 3, size=(9, H))]       # normalisers below and above exp(-m)
        m = rng.normal(0, 2.0, size=(9, H)).astype(np.float32)
        gate = rounded(rng.normal(0, 2.0, size=(9, H * V + 5)), dtype)
        weight = rng.normal(1.0, 0.3, size=H * V).astype(np.float32)
        out = torch.empty(9, H * V, dtype=DTYPES[dtype], device=DEV)
        gates = {"float32": [dev(gate)], "bfloat16": [dev(gate), dev(gate, dtype)]}[dtype]
        for g in gates:
            kernels.exp_memory_out(dev(o.reshape(9, -1)), dev(m), g[:, 2:2 + H * V], dev(weight), out, H, V, 1e-5, 1.5)
            want = plain.unit_rms(_normalised(o.astype(np.float64), m, V), 1e-5).reshape(9, H * V) * weight \
                * plain.sigmoid(f64(gate)[:, 2:2 + H * V]) * 1.5
            assert np.abs(out.float().cpu().numpy() - want).max() <= (1e-5 if dtype == "float32" else 3e-2)


def _tables(dims, base):
    from sprout_lm_b200.config.specs import PartSpec
    from sprout_lm_b200.parts import build_part
    if not dims:
        return None, None
    part = build_part("position", PartSpec("rope_yarn", {"dims": dims, "theta": base, "max_positions": 2048, "scaling": None}), "")
    return part.rotary_tables(SimpleNamespace(device=DEV))


# (heads, kv heads, dim, vdim, rotated, page, window or None, kept first, cap, sink and gate, query/key norm)
ATTENTION_CASES = [
    (3, 3, 8, 12, 4, 16, 5, 2, 7.0, False, True),
    (4, 2, 12, 6, 0, 8, None, 0, 4.0, True, False),
    (4, 1, 16, 24, 16, 8, 33, 0, 30.0, False, True),
    (6, 2, 8, 8, 2, 8, 9, 11, 0.0, False, True),
    (4, 2, 32, 64, 32, 16, 70, 3, 20.0, False, True),
    (8, 2, 64, 128, 0, 16, None, 0, 25.0, True, False),
    (4, 1, 64, 64, 48, 16, 100, 17, 40.0, False, True),
    (8, 1, 64, 64, 32, 16, 130, 70, 45.0, True, True),
    (2, 2, 128, 128, 64, 32, 1, 1, 15.0, False, False),
]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", ATTENTION_CASES)
def test_capped_attention_with_kept_first_positions(dtype, case):
    """Norm before the rotation, rotation, append and attention together: capped scores, a window that keeps the first
    positions, sinks and gates; contexts on both sides of page, window, kept-range and 64-key borders; portions of queries
    and single queries; pages in shuffled order."""
    from sprout_lm_b200 import kernels
    H, G, dim, vdim, rotated, page, window, keep, cap, sink_gate, qk_norm = case
    rng = np.random.default_rng(sum(x or 0 for x in case[:8]))
    cos, sin = _tables(rotated, 300.0)
    mask = None if window is None else ("window", window, keep)
    plain_mask = None if window is None else {"size": window, "keep_first": keep}
    edges = sorted({1, 2, keep, keep + 1, page, page + 1, 63, 64, 65, 127, 129, 200} | ({window - 1, window, window + 1, window + keep,
                   window + keep + 1, 2 * window + 3} if window else set()))
    contexts = [n for n in edges if n >= 1][:14]
    q_lens = [min(n, q) for n, q in zip(contexts, (1, 1, 2, 1, 5, 1, 17, 1, 64, 1, 3, 1, 40, 1))]
    pages_per = [-(-n // page) for n in contexts]
    total = sum(pages_per) + 3
    order = rng.permutation(total)[:sum(pages_per)]
    table = np.full((len(contexts), max(pages_per)), -1, dtype=np.int32)
    at = 0
    for r, n in enumerate(pages_per):
        table[r, :n] = order[at:at + n]
        at += n
    k_cache = torch.full((total, G, page, dim), float("nan"), dtype=DTYPES[dtype], device=DEV)
    v_cache = torch.full((total, G, page, vdim), float("nan"), dtype=DTYPES[dtype], device=DEV)
    status = new_status()
    qw = rng.normal(1.0, 0.4, size=dim).astype(np.float32) if qk_norm else None
    kw = rng.normal(1.0, 0.4, size=dim).astype(np.float32) if qk_norm else None
    sink = rng.uniform(-1.0, 3.0, size=H).astype(np.float32) if sink_gate else None
    scale = 1.7 / np.sqrt(dim) * (3.0 if cap else 1.0)                    # with a cap, scores that reach into its bend
    wants, q_rows, gate_rows, starts = [], [], [], [0]
    for r, (n, ql) in enumerate(zip(contexts, q_lens)):
        q = rounded(rng.normal(size=(n, H, dim)), dtype)
        k = rounded(rng.normal(size=(n, G, dim)), dtype)
        v = rounded(rng.normal(size=(n, G, vdim)), dtype)
        gate = rounded(rng.normal(0, 2.0, size=(n, H)), dtype)
        rows = torch.cat([q.reshape(n, -1), k.reshape(n, -1), v.reshape(n, -1)], dim=1)
        rows = dev(rows, dtype)
        kernels.rope_maps_append(rows, ints(range(n)), ints([r] * n), dev(table), cos, sin, k_cache, v_cache, H, G, 1, dim, vdim, page,
                                 True, status, q_weight=None if qw is None else dev(qw), k_weight=None if kw is None else dev(kw),
                                 weight_eps=1e-5)
        q_rows.append(rows[n - ql:, :H * dim])
        gate_rows.append(gate[n - ql:])
        starts.append(starts[-1] + ql)
        pq, pk = f64(q), f64(k)
        if qk_norm:
            pq, pk = plain.rms_norm(pq, qw, 1e-5), plain.rms_norm(pk, kw, 1e-5)
        pos = np.arange(n)
        pq, pk = plain.rotate_half(pq, pos, 300.0, rotated), plain.rotate_half(pk, pos, 300.0, rotated)
        o = plain.softmax_attention(pq, pk, f64(v), scale, cap or None, plain_mask, sink)
        if sink_gate:
            o = o * plain.sigmoid(f64(gate))[:, :, None]
        wants.append(o[n - ql:].reshape(ql, H * vdim))
    assert int(status.item()) == 0
    q_all = torch.cat(q_rows).contiguous()
    gates = dev(torch.cat(gate_rows), dtype) if sink_gate else None
    positions = np.concatenate([np.arange(n - ql, n) for n, ql in zip(contexts, q_lens)])
    seq_of = np.concatenate([[r] * ql for r, ql in enumerate(q_lens)])
    view = SimpleNamespace(k=k_cache, v=v_cache, block_table=dev(table), page_tokens=page, write=False)
    want = np.concatenate(wants)
    tol = 3e-5 if dtype == "float32" else 8e-2        # 16 bits: the queries and keys are rounded after norm and rotation, the scores are large

    def run(sel, max_q_len, planned):
        """The requests ``sel`` as one batch."""
        rows = np.concatenate([np.arange(starts[r], starts[r + 1]) for r in sel])
        ctx = SimpleNamespace(q_start=ints(np.concatenate([[0], np.cumsum([q_lens[r] for r in sel])])), positions=ints(positions[rows]),
                              seq_of_token=ints([sel.index(r) for r in seq_of[rows]]), max_q_len=max_q_len, planned_context=planned,
                              max_context=max(contexts))
        part = SimpleNamespace(k=k_cache, v=v_cache, block_table=view.block_table[torch.tensor(sel, device=DEV)].contiguous(),
                               page_tokens=page, write=False)
        out = torch.empty(len(rows), H * vdim, dtype=DTYPES[dtype], device=DEV)
        kernels.multimap_attention(q_all[rows].contiguous(), part, ctx, out, H, G, 1, dim, vdim, scale, 0.0, 0.0, 1.0, status, mask=mask,
                                   sink=None if sink is None else dev(sink), gate=None if gates is None else gates[rows].contiguous(),
                                   softcap=cap)
        err = np.abs(out.float().cpu().numpy() - want[rows]).max()
        assert err <= tol, (sel, err)
    everyone = list(range(len(contexts)))
    run(everyone, max(q_lens), max(contexts))                               # portions beside single queries
    singles = [r for r in everyone if q_lens[r] == 1]
    run(singles, 1, max(contexts[r] for r in singles))                      # a step of single tokens, its keys divided among CTAs
    run(singles[-1:], 1, contexts[singles[-1]])
    assert int(status.item()) == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_one_key_decides(dtype):
    """Where random numbers would hide a fault: one key's score stands out, far back among hundreds, just inside and just
    outside the window, among the kept first positions and right after them, in a prompt portion and in a single-token step;
    and a sink that takes nearly all the weight."""
    from sprout_lm_b200 import kernels
    H, G, dim, vdim, page, window, keep = 4, 2, 64, 64, 16, 70, 5
    rng = np.random.default_rng(9)
    n = 333
    status = new_status()
    table = rng.permutation(40)[:21].astype(np.int32).reshape(1, 21)
    for place, seen in ((n - 1 - 69, True), (n - 1 - 70, False), (4, True), (5, False), (0, True), (n - 1, True), (n - 64, True)):
        k = rng.normal(0, 0.05, size=(n, G, dim))
        v = rng.normal(0, 1.0, size=(n, G, vdim))
        q = rng.normal(0, 0.05, size=(n, H, dim))
        direction = rng.normal(size=dim)
        direction /= np.linalg.norm(direction)
        k[place] = direction * 6.0
        q[n - 1] = direction * 6.0                                          # score 36 * scale at one key, near zero elsewhere
        q_t, k_t, v_t = rounded(q, dtype), rounded(k, dtype), rounded(v, dtype)
        k_cache = torch.zeros((40, G, page, dim), dtype=DTYPES[dtype], device=DEV)
        v_cache = torch.zeros((40, G, page, vdim), dtype=DTYPES[dtype], device=DEV)
        rows = dev(torch.cat([q_t.reshape(n, -1), k_t.reshape(n, -1), v_t.reshape(n, -1)], dim=1), dtype)
        kernels.rope_maps_append(rows, ints(range(n)), ints([0] * n), dev(table), None, None, k_cache, v_cache, H, G, 1, dim, vdim, page,
                                 True, status)
        view = SimpleNamespace(k=k_cache, v=v_cache, block_table=dev(table), page_tokens=page, write=False)
        for q_len in (1, 23):
            ctx = SimpleNamespace(q_start=ints([0, q_len]), positions=ints(range(n - q_len, n)), seq_of_token=ints([0] * q_len),
                                  max_q_len=q_len, planned_context=n, max_context=n)
            out = torch.empty(q_len, H * vdim, dtype=DTYPES[dtype], device=DEV)
            kernels.multimap_attention(rows[n - q_len:, :H * dim], view, ctx, out, H, G, 1, dim, vdim, 0.5, 0.0, 0.0, 1.0, status,
                                       mask=("window", window, keep), softcap=30.0)
            last = out[-1].float().cpu().numpy().reshape(H, vdim)
            chosen = f64(v_t)[place]                                          # [G, vdim]
            near = all(np.abs(last[h] - chosen[h // 2]).max() < 0.08 for h in range(H))
            assert near == seen, (place, q_len, seen)
        # without the cap the key would dominate even more; with a tiny cap it would not at all
        want = plain.softmax_attention(f64(q_t), f64(k_t), f64(v_t), 0.5, 30.0, {"size": window, "keep_first": keep}, None)[-1]
        assert np.abs(last - want).max() <= (3e-5 if dtype == "float32" else 4e-2)
    # a sink far above every score: the output is almost nothing; far below: as if it were not there
    for level, share in ((30.0, 0.0), (-30.0, 1.0)):
        ctx = SimpleNamespace(q_start=ints([0, 1]), positions=ints([n - 1]), seq_of_token=ints([0]), max_q_len=1, planned_context=n,
                              max_context=n)
        out = torch.empty(1, H * vdim, dtype=DTYPES[dtype], device=DEV)
        sink = torch.full((H,), level, dtype=torch.float32, device=DEV)
        kernels.multimap_attention(rows[n - 1:, :H * dim], view, ctx, out, H, G, 1, dim, vdim, 0.5, 0.0, 0.0, 1.0, status, sink=sink,
                                   softcap=20.0)
        want = plain.softmax_attention(f64(q_t), f64(k_t), f64(v_t), 0.5, 20.0, None, np.full(H, level))[-1]
        assert np.abs(out.float().cpu().numpy().reshape(H, vdim) - want).max() <= (3e-5 if dtype == "float32" else 4e-2)
        assert (np.abs(want).max() < 1e-3) == (share == 0.0)
    assert int(status.item()) == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_grouped_routing_and_plain_experts(dtype):
    """The router's choice among the best groups with weights that are the scores, the gate beside the router, and the
    experts' two products with the exact gelu: few tokens and many, sizes the tensor-core products take and sizes they do
    not, one expert per token and several."""
    from sprout_lm_b200 import kernels
    rng = np.random.default_rng(4)
    cases = [(40, 6, 2, (3, 2), 20, 5), (64, 8, 3, (4, 2), 16, 300), (128, 8, 2, (4, 2), 32, 70), (64, 4, 1, None, 24, 9),
             (72, 12, 4, (3, 1), 40, 130), (64, 16, 2, (2, 1), 64, 3)]
    for width, experts, top, groups, ff, tokens in cases:
        h = rounded(rng.normal(size=(tokens, width)), dtype)
        router = rng.normal(0, 0.4, size=(experts + 1, width)).astype(np.float32)
        w = {"m.router": router[:experts].astype(np.float64)}
        want_ids, want_w = plain.route(f64(h), w, "m.", {"experts": experts, "top": top,
                                                         "groups": None if groups is None else {"count": groups[0], "keep": groups[1]}})
        ids = torch.empty((tokens, top), dtype=torch.int32, device=DEV)
        weights = torch.empty((tokens, top), dtype=torch.float32, device=DEV)
        counts = torch.zeros(experts, dtype=torch.int32, device=DEV)
        extra = torch.empty((tokens, 1), dtype=torch.float32, device=DEV)
        kernels.moe_route(dev(h, dtype), dev(router), None, ids, weights, counts, experts, top, 1.0, groups=groups, renormalize=False,
                          extra_out=extra)
        assert np.array_equal(ids.cpu().numpy(), want_ids), (width, experts)
        assert np.abs(weights.cpu().numpy() - want_w).max() <= 2e-6
        assert np.abs(extra.cpu().numpy()[:, 0] - f64(h) @ router[experts].astype(np.float64)).max() <= 2e-5
        if groups is not None and groups[1] < top and tokens >= 50:       # the best `top` groups always hold the `top` best experts
            free_ids, _ = plain.route(f64(h), w, "m.", {"experts": experts, "top": top})
            assert not np.array_equal(free_ids, want_ids)                   # the groups do forbid some choices
        # the experts
        up = rounded(rng.normal(0, 0.3, size=(experts, ff, width)), dtype)
        down = rounded(rng.normal(0, 0.3, size=(experts, width, ff)), dtype)
        offsets = torch.zeros(experts + 1, dtype=torch.int32, device=DEV)
        order = torch.empty(tokens * top, dtype=torch.int32, device=DEV)
        place_of = torch.empty(tokens * top, dtype=torch.int32, device=DEV)
        kernels.moe_arrange(ids, counts, offsets, order, place_of, experts)
        act = torch.empty((tokens * top, ff), dtype=DTYPES[dtype], device=DEV)
        rows = torch.empty((tokens * top, width), dtype=torch.float32, device=DEV)
        kernels.moe_experts(dev(h, dtype), order, offsets, dev(up, dtype), dev(down, dtype), act, rows, experts, top, 0.0, 0.0)
        y = torch.zeros((tokens, width), dtype=torch.float32, device=DEV)
        kernels.moe_combine(y, dev(h, dtype), ids, weights, place_of, rows, top)
        want = np.zeros((tokens, width))
        for t in range(tokens):
            for e, weight in zip(want_ids[t], want_w[t]):
                want[t] += weight * (plain.gelu_erf(f64(h)[t] @ f64(up)[e].T) @ f64(down)[e].T)
        err = np.abs(y.cpu().numpy() - want).max()
        assert err <= (3e-5 if dtype == "float32" else 3e-2) * max(1.0, np.abs(want).max()), (width, experts, tokens, err)


# =============================================================================== whole models
@pytest.fixture(scope="module")
def model_dirs(tmp_path_factory):
    base = tmp_path_factory.mktemp("vuripel")
    return {name: vh.make_model_dir(base, name) for name in vh.CONFIGS}


def make_requests(name, seed, lengths):
    vocab = vh.CONFIGS[name][0]["vocab"]
    rng = np.random.default_rng(seed)
    return {f"r{i}": helpers.random_tokens(rng, n, vocab) for i, n in enumerate(lengths)}


def make_runner(model_dir, dtype, pages, page_tokens, requests=4):
    from sprout_lm_b200.engine.step import ModelRunner
    from sprout_lm_b200.models import load_model
    model = load_model(model_dir, dtype=DTYPES[dtype])
    return ModelRunner(model, num_pages=pages, page_tokens=page_tokens, max_requests=requests, prefix_caching=False)


def test_layers_one_by_one(model_dirs):
    """The stream after every layer run in 32-bit (a looped layer counts each time), so that a fault names its layer."""
    from sprout_lm_b200.engine.batch import StepEntry
    for name, directory in model_dirs.items():
        config, tensors = vh.plain_model(directory)
        tokens = make_requests(name, 1, [41])["r0"]
        runner = make_runner(directory, "float32", 8, vh.CONFIGS[name][2])
        seen = []
        for block in runner.model.blocks:
            def wrapped(x, *args, _inner=block.forward, **more):
                _inner(x, *args, **more)
                seen.append(x.clone())
            block.forward = wrapped
        seq = runner.new_sequence()
        assert runner.reserve(seq, len(tokens))
        runner.step([StepEntry(seq, tokens, [0])])
        _, want = plain.forward(config, tensors, tokens, return_layers=True)
        assert len(seen) == len(want) == len(plain.run_order(config))
        for i, (got, expected) in enumerate(zip(seen, want)):
            assert np.abs(got.cpu().numpy() - expected).max() <= 3e-5 * max(1.0, np.abs(expected).max()), (name, "layer run", i)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_all_cuttings_in_process(model_dirs, name, dtype):
    """Whole, tail decoded token by token (110 tokens: every window of the models passes over decoded tokens), portions
    down to two tokens, mixed batches with pages and state slots used again: against the plain implementation, and in 32-bit
    equal to one another to rounding."""
    page = vh.CONFIGS[name][2]
    requests = make_requests(name, 11, [5, 17, 33, 70, 150, 1, 40])
    rng = np.random.default_rng(5)
    plans = {
        "whole": helpers.plan_whole(requests),
        "tail": helpers.plan_tail_decode(requests, tail=110),
        "portions": helpers.plan_portions(requests),
        "mixed": helpers.plan_mixed(requests, rng),
    }
    results = {}
    for label, plan in plans.items():
        budget = helpers.live_token_budget(plan, requests)
        runner = make_runner(model_dirs[name], dtype, budget // page, page, requests=4)
        got = results[label] = helpers.run_plan_in_process(runner, plan)
        assert len(got) == sum(len(t) for t in requests.values())
        worst = vh.compare(model_dirs[name], requests, got, TOL[dtype], f"{name}/{dtype}/{label}", page, rounded=dtype == "bfloat16")
        print(f"{name}/{dtype}/{label}: worst difference {worst:.2e}")
        runner.manager.check_invariants()
        for pool in runner.manager.pools:
            assert len(pool.free) == pool.num_pages                                           # every page came back
        assert len(runner.manager._free_state) == 4                                           # and every state slot
    if dtype == "float32":
        for label in ("tail", "portions", "mixed"):
            for place, row in results["whole"].items():
                assert np.abs(row - results[label][place]).max() <= 1e-4 * max(1.0, np.abs(row).max()), \
                    f"{name}: {label} differs from whole at {place}"


def test_long_context_and_long_decoding(model_dirs):
    """A prompt of several hundred tokens in uneven portions, then 140 tokens decoded one by one, in both dtypes: the slow
    forget gates' states, windows that are no multiple of a page, kept first pages beside pages given back, keys many pages
    back in the layers that see everything."""
    for name, page, pages in (("B", 8, 90), ("C", 16, 45)):
        requests = make_requests(name, 21, [670])
        plan = helpers.plan_portions(requests, sizes=(130, 2, 127, 3, 64, 100, 2, 97, 5) + (1,) * 140)
        for dtype in ("float32", "bfloat16"):
            runner = make_runner(model_dirs[name], dtype, pages, page)
            got = helpers.run_plan_in_process(runner, plan)
            vh.compare(model_dirs[name], requests, got, TOL[dtype], f"long/{name}/{dtype}", page, rounded=dtype == "bfloat16")


def test_a_lost_state_a_dropped_sink_or_a_shifted_window_shows(model_dirs):
    """The test models are made so that each mechanism matters: the same tokens after another prefix, weights without the
    sinks, windows and kept ranges one token off, a missing cap, a pass without its vector or without the embedding added
    again, a missing token row and a router without its groups all move the logits by far more than the bar."""
    name = "A"
    tokens = make_requests(name, 31, [60])["r0"]
    full = vh.plain_logits(model_dirs[name], tokens)
    tail_alone = vh.plain_logits(model_dirs[name], tokens[30:])
    bar = 3 * TOL["bfloat16"]

    def moved(other, places=slice(None)):
        """The largest change at any place: a fault is found if one place is over the bar."""
        return max(vh.relative(a, b) for a, b in zip(other, full[places]))
    assert moved(tail_alone, slice(30, None)) > bar
    config, tensors = vh.plain_model(model_dirs[name])

    def with_tensors(change):
        return plain.forward(config, {k: change(k, v) for k, v in tensors.items()}, tokens)
    assert moved(with_tensors(lambda k, v: np.full_like(v, -30.0) if k.endswith(".sink") else v)) > bar
    assert moved(with_tensors(lambda k, v: np.zeros_like(v) if k == "loop.step" else v)) > bar
    assert moved(with_tensors(lambda k, v: np.zeros_like(v) if k == "side.embed" else v)) > bar
    assert moved(with_tensors(lambda k, v: np.zeros_like(v) if k.endswith(".mix.f.b") else v)) > bar
    assert moved(with_tensors(lambda k, v: np.zeros_like(v) if k.endswith((".q.b", ".k.b", ".v.b")) else v)) > bar
    assert moved(with_tensors(lambda k, v: np.ones_like(v) if k.endswith((".q.norm", ".k.norm")) else v)) > bar
    edits = [lambda c: c["layers"][0]["mixer"]["mask"].__setitem__("size", 6),
             lambda c: c["layers"][0]["mixer"]["mask"].__setitem__("keep_first", 3),
             lambda c: c["layers"][0]["mixer"]["mask"].__setitem__("keep_first", 0),
             lambda c: c["layers"][0]["mixer"].__setitem__("softcap", None),
             lambda c: c["layers"][2]["mixer"].__setitem__("softcap", None),
             lambda c: c["layers"][1]["mixer"].__setitem__("gate_cap", None),
             lambda c: c["layers"][1]["mlp"]["router"].__setitem__("groups", None),
             lambda c: c["layers"][1]["mlp"].__setitem__("shared", None),
             lambda c: c["loop"].__setitem__("times", 2),
             lambda c: c.__setitem__("loop", None)]
    for number, edit in enumerate(edits):
        changed = copy.deepcopy(config)
        edit(changed)
        assert moved(plain.forward(changed, tensors, tokens)) > bar, number
    # the embedding's output joins every later pass: a model whose later passes start from the stream alone differs
    original = plain.forward

    def run_without_restart(cfg, w, toks):
        toks = np.asarray(toks)
        x = w["embed"][toks]
        for index, number, begins in plain.run_order(cfg):
            if begins:
                x = x + w["loop.step"][number]
            x = plain.layer_forward(x, cfg, w, index, toks, np.arange(len(toks)))
        return plain.lin(plain.rms_norm(x, w["final.norm"], cfg["norm"]["eps"]), w["head"])
    assert moved(run_without_restart(config, tensors, tokens)) > bar and original is plain.forward


def test_trace_replay_program(model_dirs, tmp_path):
    """bin/trace_run picks the model class by config.json and replays a mixed plan with four state slots."""
    name = "B"
    requests = make_requests(name, 13, [9, 40, 70, 23, 31, 12])
    plan = helpers.plan_mixed(requests, np.random.default_rng(2))
    budget = helpers.live_token_budget(plan, requests)
    vocab = vh.CONFIGS[name][0]["vocab"]
    for dtype in ("float32", "bfloat16"):
        got = helpers.run_plan_with_trace_run(model_dirs[name], dtype, plan, tmp_path / dtype, budget, vocab=vocab)
        vh.compare(model_dirs[name], requests, got, TOL[dtype], f"trace/{dtype}", 16, rounded=dtype == "bfloat16")


@pytest.mark.parametrize("name", ["A", "C"])
def test_greedy_generation_through_the_scheduler(model_dirs, name):
    """generate(): continuous batching, chunked prefill and captured decode steps; in 32-bit the tokens are the plain
    implementation's, in bfloat16 every token is within bfloat16's reach of the plain choice."""
    from sprout_lm_b200 import generate, load_model
    config, tensors = vh.plain_model(model_dirs[name])
    rng = np.random.default_rng(7)
    prompts = [helpers.random_tokens(rng, n, config["vocab"]) for n in (3, 19, 44)]
    new_tokens = 12
    for dtype in ("float32", "bfloat16"):
        model = load_model(model_dirs[name], dtype=dtype)
        results = generate(model, prompts, max_new_tokens=new_tokens, ignore_eos=True)
        for prompt, result in zip(prompts, results):
            assert len(result["output"]) == new_tokens
            history = list(prompt)
            for token in result["output"]:
                row = plain.forward(config, tensors, history)[-1]
                spread = float(np.sqrt(np.mean((row - row.mean()) ** 2)))
                assert row[token] >= row.max() - (1e-4 if dtype == "float32" else 4 * TOL["bfloat16"]) * spread, (name, dtype, len(history))
                history.append(token)


def test_scheduler_under_page_pressure(model_dirs):
    """A pool smaller than the requests together: a preempted request gives its state slot back and recomputes its state
    from the start; the greedy tokens stay the plain implementation's."""
    from sprout_lm_b200 import EngineOptions, generate, load_model
    name = "A"
    config, _ = vh.plain_model(model_dirs[name])
    rng = np.random.default_rng(8)
    prompts = [helpers.random_tokens(rng, n, config["vocab"]) for n in (30, 41, 26, 35)]
    model = load_model(model_dirs[name], dtype="float32")
    options = EngineOptions(block_size=8, num_blocks=14, max_sequences=4, max_batch_tokens=24, prefill_chunk_size=7)
    results = generate(model, prompts, max_new_tokens=10, ignore_eos=True, options=options)
    for prompt, result in zip(prompts, results):
        assert result["output"] == vh.plain_greedy(model_dirs[name], prompt, 10)
