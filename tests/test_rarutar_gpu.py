"""Rarutar on the GPU against the plain implementation: every mechanism alone (with inputs made so that a fault
shows), then whole models under every way of cutting the work, through the step function, the trace replay program
and the scheduler."""
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import helpers
import plain_rarutar as plain
import rarutar_helpers as rh

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 6e-5, "bfloat16": 6e-2}       # of the logits' spread over the vocabulary at that place (rarutar_helpers.relative)


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


# =============================================================================== mechanisms alone
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layernorm_with_bias_and_scaled_embedding(dtype):
    from sprout_lm_b200 import kernels
    rng = np.random.default_rng(0)
    tol = 4e-6 if dtype == "float32" else 4e-2
    for width in (40, 257, 1030, 128, 768):
        x = rng.normal(3.0, 2.0, size=(5, width)).astype(np.float32)         # a mean far from zero: the deviations matter
        w, b = rng.normal(1.0, 0.3, size=width).astype(np.float32), rng.normal(0.0, 1.0, size=width).astype(np.float32)
        out = torch.empty(5, width, dtype=DTYPES[dtype], device=DEV)
        kernels.layernorm(dev(x), dev(w), out, 1e-5, bias=dev(b))
        assert np.abs(out.float().cpu().numpy() - plain.layer_norm(x.astype(np.float64), w, b, 1e-5)).max() <= tol
        picked = torch.empty(2, width, dtype=DTYPES[dtype], device=DEV)
        kernels.layernorm(dev(x), dev(w), picked, 1e-5, rows=ints([3, 0]), bias=dev(b))
        assert torch.equal(picked, out[[3, 0]])
    table = rounded(rng.normal(size=(19, 24)), "bfloat16")
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    x = torch.empty(4, 24, dtype=torch.float32, device=DEV)
    kernels.embed(dev(table, dtype), ints([3, 18, 0, 3]), x, status, scale=1.7)
    assert np.abs(x.cpu().numpy() - f64(table)[[3, 18, 0, 3]] * 1.7).max() <= 1e-6 and int(status.item()) == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_clamped_gated_activation(dtype):
    from sprout_lm_b200 import kernels
    rng = np.random.default_rng(1)
    tol = 4e-6 if dtype == "float32" else 3e-2
    for ff, limit in ((19, 0.8), (64, 2.5), (7, 1.0)):
        gate_up = rounded(rng.normal(0, 2.0, size=(6, 2 * ff)), dtype)        # values on both sides of every limit
        act = torch.empty(6, ff, dtype=DTYPES[dtype], device=DEV)
        kernels.glu_clamped(dev(gate_up, dtype), act, limit, 1.702)
        g = np.minimum(f64(gate_up)[:, :ff], limit)                            # from above only
        u = np.clip(f64(gate_up)[:, ff:], -limit, limit)
        assert np.abs(act.float().cpu().numpy() - g * plain.sigmoid(1.702 * g) * (u + 1)).max() <= tol * 4
        assert (f64(gate_up)[:, :ff] < -limit).any() and (f64(gate_up)[:, ff:] < -limit).any()


def _fill_cache(kernels, dtype, contexts, G, dim, vdim, page, tables, rng, unit_eps, value_from_key, keys=None, values=None):
    """Append every request's keys and values through the kernel, into shuffled pages.  Returns the cache view, the
    projected keys [r][S, G, dim] and values [r][S, G, vdim] as the dtype holds them."""
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
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    cos, sin = tables
    all_k, all_v = [], []
    for r, n in enumerate(contexts):
        k = rounded(rng.normal(0, 1.0, size=(n, G, dim)) if keys is None else keys[r], dtype)
        v = k if value_from_key else rounded(rng.normal(0, 1.0, size=(n, G, vdim)) if values is None else values[r], dtype)
        all_k.append(f64(k))
        all_v.append(f64(v))
        parts = [torch.zeros(n, dim), k.reshape(n, -1)] + ([] if value_from_key else [v.reshape(n, -1)])
        kernels.rope_maps_append(dev(torch.cat(parts, dim=1), dtype), ints(range(n)), ints([r] * n), dev(table), cos, sin, k_cache,
                                 v_cache, 1, G, 1, dim, vdim, page, True, status, unit_eps=unit_eps, value_from_key=value_from_key)
    assert int(status.item()) == 0
    view = SimpleNamespace(k=k_cache, v=v_cache, block_table=dev(table), page_tokens=page, write=False)
    return view, all_k, all_v, status


def _rotary(dims, base, scaling=None):
    from sprout_lm_b200.config.specs import PartSpec
    from sprout_lm_b200.parts import build_part
    if not dims:
        return (None, None), rh.rot(base, 0)
    rot = rh.rot(base, dims, scaling)
    part = build_part("position", PartSpec("rope_yarn", {"dims": dims, "theta": base, "max_positions": 2048, "scaling": rot.get("scaling")}), "")
    return part.rotary_tables(SimpleNamespace(device=DEV)), rot


# (heads, kv heads, dim, vdim, rotated, page, mask, scaling, the values are the keys with unit-norm vectors and a sink)
ATTENTION_CASES = [
    (6, 2, 16, 24, 8, 16, ("window", 21), (4.0, 64, 8.0, 1.0), False),
    (3, 3, 8, 8, 4, 8, ("chunk", 8), None, True),
    (2, 1, 12, 12, 12, 16, ("chunk", 37), None, True),
    (8, 4, 32, 64, 16, 16, ("window", 64), (8.0, 128, 16.0, 2.0), False),
    (8, 2, 64, 64, 32, 16, ("chunk", 100), None, True),
    (6, 3, 64, 32, 64, 16, ("window", 130), (8.0, 256, 32.0, 1.0), False),
    (4, 2, 64, 128, 32, 16, ("window", 70), None, False),
    (4, 4, 32, 32, 0, 8, ("chunk", 64), None, True),
    (2, 1, 8, 300, 4, 16, ("window", 1), None, False),
    (4, 1, 128, 128, 64, 32, ("chunk", 129), None, True),
]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", ATTENTION_CASES)
def test_masked_attention_over_pages(dtype, case):
    """Rotation (stretched or not), unit norm, append and attention together under a window or chunks, with sinks and
    gates: contexts on both sides of page, window, chunk and 64-key borders, portions of queries and single queries,
    pages in shuffled order."""
    from sprout_lm_b200 import kernels
    H, G, dim, vdim, rotated, page, mask, scaling, chunked = case
    rng = np.random.default_rng(sum(case[:6]))
    tables, rot = _rotary(rotated, 300.0, scaling)
    unit_eps = 1e-5 if chunked else 0.0
    size = mask[1]
    contexts = sorted({1, 2, page - 1, page, page + 1, size, size + 1, max(1, size - 1), 2 * size, 2 * size + 1, 63, 64, 65, 129, 257, 300})
    view, keys, values, status = _fill_cache(kernels, dtype, contexts, G, dim, vdim, page, tables, rng, unit_eps, chunked)
    # unit-norm vectors have length sqrt(dim): the scale keeps the scores' spread near 2, where bfloat16 keys still tell
    # the weights apart by rounding alone
    scale, out_scale = 0.3 if not chunked else min(2.0, 16.0 / dim), 0.6
    tol = 4e-5 if dtype == "float32" else 4e-2
    wanted = [min(n, 5) for n in contexts]
    wanted[-3], wanted[-2], wanted[-1] = min(contexts[-3], 70), 40, 150
    positions, seqs = [], []
    for r, n in enumerate(contexts):
        positions += list(range(n - wanted[r], n))
        seqs += [r] * wanted[r]
    T = len(positions)
    q = rounded(rng.normal(0, 1.0, size=(T, H, dim)), dtype)
    gate = rounded(rng.normal(0, 2.0, size=(T, H)), dtype)
    pad = (-(H * dim + H)) % 8
    rows = dev(torch.cat([q.reshape(T, -1), gate, torch.zeros(T, pad)], dim=1), dtype)
    kernels.rope_maps_append(rows, ints(positions), ints(seqs), view.block_table, tables[0], tables[1], None, None, H, G, 1, dim,
                             vdim, page, False, status, unit_eps=unit_eps, value_from_key=chunked)
    sink = rng.uniform(-1.0, 2.0, size=H).astype(np.float32) if chunked else None
    starts = np.concatenate([[0], np.cumsum(wanted)])
    ctx = SimpleNamespace(positions=ints(positions), seq_of_token=ints(seqs), q_start=ints(starts), max_q_len=max(wanted))
    out = torch.empty(T, H * vdim, dtype=DTYPES[dtype], device=DEV)
    gate_view = rows[:, H * dim:H * dim + H]
    kernels.multimap_attention(rows[:, :H * dim], view, ctx, out, H, G, 1, dim, vdim, scale, 0.0, 0.0, out_scale, status, mask=mask,
                               sink=None if sink is None else dev(sink), gate=gate_view)
    got = out.float().cpu().numpy().reshape(T, H, vdim)
    # the same with single tokens only (every request's last position): the step a decoding batch makes
    last = [int(starts[r + 1]) - 1 for r in range(len(contexts))]
    single = SimpleNamespace(positions=ints([positions[i] for i in last]), seq_of_token=ints(range(len(contexts))),
                             q_start=ints(range(len(contexts) + 1)), max_q_len=1, max_context=max(contexts))
    rows1 = rows[last].contiguous()
    out1 = torch.empty(len(contexts), H * vdim, dtype=DTYPES[dtype], device=DEV)
    kernels.multimap_attention(rows1[:, :H * dim], view, single, out1, H, G, 1, dim, vdim, scale, 0.0, 0.0, out_scale, status, mask=mask,
                               sink=None if sink is None else dev(sink), gate=rows1[:, H * dim:H * dim + H])
    got1 = out1.float().cpu().numpy().reshape(len(contexts), H, vdim)
    assert int(status.item()) == 0
    at = 0
    for r, n in enumerate(contexts):
        count = wanted[r]
        pos = list(range(n - count, n))
        qr = plain.rotate(f64(q[at:at + count]), pos, rot)
        kr = plain.rotate(keys[r], list(range(n)), rot)
        if chunked:
            qr, kr = plain.rms_unit(qr, unit_eps), plain.rms_unit(kr, unit_eps)
        # the plain function takes whole sequences: queries at every position, of which the last ``count`` are the step's
        q_all = np.zeros((n, H, dim))
        q_all[n - count:] = qr
        want = plain.masked_softmax_attention(q_all, kr, values[r], scale, mask[0], size, sink)[n - count:]
        want = want * plain.sigmoid(f64(gate[at:at + count]))[:, :, None] * out_scale
        assert np.abs(got[at:at + count] - want).max() <= tol, (n, np.abs(got[at:at + count] - want).max())
        assert np.abs(got1[r] - want[-1]).max() <= tol, (n, "single token", np.abs(got1[r] - want[-1]).max())
        at += count


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", [("window", 16, 24, 21, 16), ("chunk", 16, 16, 37, 16), ("window", 64, 64, 64, 16), ("chunk", 64, 64, 100, 16),
                                  ("window", 32, 40, 130, 8), ("chunk", 128, 128, 129, 32)])
def test_attention_sees_the_edge_key_and_not_the_one_beyond(dtype, case):
    """One key far back is made to stand out (its score dwarfs the others, its value is large).  Placed on the first
    visible position it decides the output; placed one position earlier it must not be seen at all.  Single queries and
    queries inside a portion, contexts of several hundred keys over shuffled pages."""
    from sprout_lm_b200 import kernels
    kind, dim, vdim, size, page = case
    H = G = 2
    chunked = kind == "chunk"
    if chunked:
        vdim = dim
    rng = np.random.default_rng(size)
    tables, rot = _rotary(0, 100.0)
    contexts = [size + 40, 2 * size + 3, 300, 3 * size, size]
    inside, outside = [], []
    keys = []
    direction = rng.normal(size=dim)
    direction /= np.linalg.norm(direction)
    for r, n in enumerate(contexts):
        k = rng.normal(0, 0.3, size=(n, G, dim))
        first = plain.first_visible(kind, size, n - 1)
        target = first if r % 2 == 0 else first - 1            # even requests: just inside; odd ones: just outside
        if target >= 0:
            k[target] = direction * 6.0
        (inside if r % 2 == 0 else outside).append(r)
        keys.append(k)
    values = None if chunked else [rng.normal(0, 1.0, size=(n, G, vdim)) + 8.0 * (np.arange(n) == (plain.first_visible(kind, size, n - 1) - (r % 2)))[:, None, None]
                                   for r, n in enumerate(contexts)]
    view, keys_r, values_r, status = _fill_cache(kernels, dtype, contexts, G, dim, vdim, page, tables, rng, 0.0, chunked, keys=keys, values=values)
    tol = 4e-5 if dtype == "float32" else 6e-2
    for portion in (1, 7):
        positions, seqs, starts = [], [], [0]
        for r, n in enumerate(contexts):
            count = min(portion, n)
            positions += list(range(n - count, n))
            seqs += [r] * count
            starts.append(starts[-1] + count)
        T = len(positions)
        q = rounded(np.tile(direction * 6.0, (T, H, 1)) + rng.normal(0, 0.05, size=(T, H, dim)), dtype)
        ctx = SimpleNamespace(positions=ints(positions), seq_of_token=ints(seqs), q_start=ints(starts), max_q_len=portion, max_context=max(contexts))
        out = torch.empty(T, H * vdim, dtype=DTYPES[dtype], device=DEV)
        sink = np.zeros(H, dtype=np.float32) if chunked else None
        kernels.multimap_attention(dev(q.reshape(T, -1), dtype), view, ctx, out, H, G, 1, dim, vdim, 1.0, 0.0, 0.0, 1.0, status, mask=(kind, size),
                                   sink=None if sink is None else dev(sink))
        got = out.float().cpu().numpy().reshape(T, H, vdim)
        for r, n in enumerate(contexts):
            count = starts[r + 1] - starts[r]
            q_all = np.zeros((n, H, dim))
            q_all[n - count:] = f64(q[starts[r]:starts[r + 1]])
            want = plain.masked_softmax_attention(q_all, keys_r[r], values_r[r], 1.0, kind, size, sink)[n - count:]
            assert np.abs(got[starts[r]:starts[r + 1]] - want).max() <= tol * max(1.0, np.abs(want).max()), (kind, n, portion)
            first = plain.first_visible(kind, size, n - 1)
            if r in inside or first == 0:
                continue
            # the case shows something: with the key one place further in, the last query's output would be another one
            moved = keys_r[r].copy()
            moved[first] = moved[first - 1]
            vals = values_r[r].copy() if not chunked else moved
            if not chunked:
                vals[first] = vals[first - 1]
            other = plain.masked_softmax_attention(q_all, moved, vals, 1.0, kind, size, sink)[-1]
            assert np.abs(other - want[-1]).max() > 20 * tol
    assert int(status.item()) == 0


def _scan_ctx(batch):
    starts = np.concatenate([[0], np.cumsum([rows.shape[0] for _, rows in batch])])
    return SimpleNamespace(q_start=ints(starts), max_q_len=max(rows.shape[0] for _, rows in batch)), starts


def _run_mixer(part, batch, state_buffers, width, dtype):
    """batch [(slot, h rows)] through a recurrent mixer's forward -> its contribution to the stream per entry."""
    from sprout_lm_b200.parts.base import StateView
    ctx, starts = _scan_ctx(batch)
    h = torch.cat([rows for _, rows in batch])
    x = torch.zeros(h.shape[0], width, dtype=torch.float32, device=DEV)
    part.forward(dev(h, dtype), x, ctx, None, StateView(state_buffers, ints([slot for slot, _ in batch])))
    got = x.cpu().numpy()
    return [got[starts[i]:starts[i + 1]] for i in range(len(batch))]


def _cut_three_ways(run, zero, inputs, wants, tol, cuts=(0, 2, 9, 10, 33)):
    """Requests 0 and 1 whole in one batch (slots 2 and 0); then slot 2 is used again by request 2 in portions beside
    request 3 token by token in slot 1."""
    zero(2); zero(0)
    got = run([(2, inputs[0]), (0, inputs[1])])
    for i in (0, 1):
        assert np.abs(got[i] - wants[i]).max() <= tol * max(1.0, np.abs(wants[i]).max()), ("whole", i)
    zero(2); zero(1)
    pieces = {2: [], 3: []}
    for step in range(inputs[3].shape[0]):
        batch = []
        if step + 1 < len(cuts):
            batch.append((2, inputs[2][cuts[step]:cuts[step + 1]]))
        batch.append((1, inputs[3][step:step + 1]))
        got = run(batch)
        if len(batch) == 2:
            pieces[2].append(got[0])
        pieces[3].append(got[-1])
    for i in (2, 3):
        assert np.abs(np.concatenate(pieces[i]) - wants[i]).max() <= tol * max(1.0, np.abs(wants[i]).max()), ("cut", i)


def _plain_scan(q, k, v, a, c, S, skip):
    """S_t = diag(a_t) S_(t-1) + (c_t k_t) v_t^T, o_t = S_t^T q_t + skip v_t for one head in float64; returns (o, S)."""
    out = np.zeros((q.shape[0], v.shape[1]))
    for t in range(q.shape[0]):
        S = a[t][:, None] * S + np.outer(c[t] * k[t], v[t])
        out[t] = S.T @ q[t] + skip * v[t]
    return out, S


# (heads, groups, dim, value dim, decay per head)
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("sizes", [(3, 3, 24, 40, False), (2, 2, 128, 64, False), (4, 2, 16, 24, True), (2, 1, 64, 130, True), (1, 1, 520, 8, False),
                                   (2, 2, 200, 36, False), (2, 1, 136, 12, True), (1, 1, 5, 3, False)])
def test_gated_scan_in_chunks(dtype, sizes, monkeypatch):
    """Long portions walked as chunks side by side: requests of 300, 1, 129, 64 and 191 tokens in one batch (a last chunk
    of one token, of a full chunk, requests of one chunk beside them), from states that are not zero, decays from very
    fast to nearly one; against the recurrence in float64 and, in 32-bit, against the single walk of the same kernel."""
    from sprout_lm_b200 import kernels
    heads, groups, dim, vdim, per_head = sizes
    rng = np.random.default_rng(dim + vdim)
    lengths = [300, 1, 129, 64, 191]
    total = sum(lengths)
    q = rounded(rng.normal(0, 1.0, size=(total, groups * dim)), dtype)
    k = rounded(rng.normal(0, 1.0, size=(total, groups * dim)), dtype)
    v = rounded(rng.normal(0, 1.0, size=(total, heads * vdim)), dtype)
    z = rounded(rng.normal(0, 2.0, size=(total, heads if per_head else heads * dim)), dtype)
    bias = rounded(rng.uniform(-3.0, 1.0, size=heads) if per_head else rng.permutation(np.linspace(-3.0, 8.0, heads * dim)), "float32")
    a_log = rounded(np.linspace(-5.0, 0.5, heads), "float32")
    skip = rounded(rng.uniform(0.3, 1.5, size=heads), "float32")
    tau, q_scale = 3.0, 0.5
    start = rounded(rng.normal(0, 1.0, size=(6, heads, dim, vdim)), "float32")
    slots = [4, 0, 5, 2, 1]
    zf, bf = f64(z), f64(bias)
    if per_head:
        step = np.logaddexp(0.0, zf + bf)                                     # [tokens, heads]
        decay = np.repeat(np.exp(-np.exp(f64(a_log)) * step)[:, :, None], dim, axis=2)
    else:
        step = np.ones((total, heads))
        decay = (1.0 / (1.0 + np.exp(-(zf + bf))) ** (1.0 / tau)).reshape(total, heads, dim)
    want, want_state, at = np.zeros((total, heads * vdim)), f64(start).copy(), 0
    for n, slot in zip(lengths, slots):
        for h in range(heads):
            g = h // (heads // groups)
            rows = slice(at, at + n)
            o, S = _plain_scan(f64(q)[rows, g * dim:(g + 1) * dim] * q_scale, f64(k)[rows, g * dim:(g + 1) * dim], f64(v)[rows, h * vdim:(h + 1) * vdim],
                               decay[rows, h], step[rows, h], want_state[slot, h], float(skip[h]) if per_head else 0.0)
            want[rows, h * vdim:(h + 1) * vdim], want_state[slot, h] = o, S
        at += n
    ctx = SimpleNamespace(q_start=ints(np.concatenate([[0], np.cumsum(lengths)])), max_q_len=max(lengths))
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    results = {}
    for form in ("chunks", "whole"):
        monkeypatch.setenv("SPROUT_GATED_SCAN", form)
        state = SimpleNamespace(buffer=dev(start, "float32").clone(), slots=ints(slots))
        out = torch.full((total, heads * vdim), float("nan"), device=DEV)
        before = kernels.LAUNCHES
        kernels.gated_scan(dev(q, dtype), dev(k, dtype), dev(v, dtype), dev(z, dtype), dev(bias, "float32"), ctx, state, out, heads, groups, dim, vdim,
                           status, per_head=per_head, tau=tau, q_scale=q_scale, a_log=dev(a_log, "float32") if per_head else None,
                           skip=dev(skip, "float32") if per_head else None)
        assert kernels.LAUNCHES - before == (4 if form == "chunks" else 1)
        results[form] = (out.cpu().numpy(), state.buffer.cpu().numpy())
        for got, expected in zip(results[form], (want, want_state)):
            assert np.abs(got - expected).max() <= 2e-5 * max(1.0, np.abs(expected).max()), (form, np.abs(got - expected).max())
        assert np.array_equal(results[form][1][3], f64(start)[3].astype(np.float32))        # a slot of no request stays as it was
    assert int(status.item()) == 0


# (heads, dim, value dim, tau, inner size of the decay, width)
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("sizes", [(3, 8, 20, 4.0, 5, 40), (1, 24, 8, 1.0, 3, 24), (4, 32, 64, 16.0, 8, 64), (2, 16, 130, 9.0, 7, 48),
                                   (2, 64, 40, 2.0, 16, 64), (1, 128, 64, 8.0, 4, 32), (3, 64, 128, 5.0, 6, 72), (1, 520, 24, 3.0, 4, 32)])
def test_gated_linear_attention_part(dtype, sizes):
    """The whole mixer against the plain one: decays per key channel from very fast to nearly 1, whole against portions
    against token by token, slots given back and used again, the final state."""
    from sprout_lm_b200.config.specs import PartSpec
    from sprout_lm_b200.parts import Runtime, WeightSource, build_part
    heads, dim, vdim, tau, rank, width = sizes
    rng = np.random.default_rng(heads * 7 + dim)
    qk, vw = heads * dim, heads * vdim
    weights = {"m.q": rng.normal(0, width ** -0.5, size=(qk, width)), "m.k": rng.normal(0, width ** -0.5, size=(qk, width)),
               "m.v": rng.normal(0, width ** -0.5, size=(vw, width)), "m.g": rng.normal(0, 2 * width ** -0.5, size=(vw, width)),
               "m.a1": rng.normal(0, width ** -0.5, size=(rank, width)), "m.a2": rng.normal(0, 2.0 * rank ** -0.5, size=(qk, rank)),
               "m.a2.b": rng.permutation(np.linspace(-2.0, 7.0, qk)), "m.norm": rng.normal(1.0, 0.3, size=vdim),
               "m.o": rng.normal(0, vw ** -0.5, size=(width, vw))}
    stored = {k: rounded(v, "bfloat16") for k, v in weights.items()}
    weights = {k: f64(v) for k, v in stored.items()}
    part = build_part("mixer", PartSpec("gated_linear_attention", {"hidden_size": width, "heads": heads, "dim": dim, "value_dim": vdim,
                                                                   "tau": tau, "eps": 1e-5, "out_scale": 0.7}), "m.")
    runtime = Runtime(DEV, DTYPES[dtype])
    part.load(WeightSource(lambda name: stored[name], runtime))
    m = {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}
    inputs = [rounded(rng.normal(0, 1.0, size=(n, width)), dtype) for n in (70, 1, 33, 150)]
    plain_out = [plain.gated_linear_attention(f64(h), weights, "m.", m, 1e-5) for h in inputs]
    wants = [0.7 * out for out, _ in plain_out]
    state = torch.full((3, heads, dim, vdim), float("nan"), device=DEV)
    tol = 3e-5 if dtype == "float32" else 5e-2
    _cut_three_ways(lambda batch: _run_mixer(part, batch, state, width, dtype), lambda slot: state[slot].zero_(), inputs, wants, tol)
    final = plain_out[3][1]
    assert np.abs(state[1].cpu().numpy() - final).max() <= tol * max(1.0, np.abs(final).max())
    assert int(runtime.status.item()) == 0


# (heads, value dim, state, groups, taps, norm parts, width)
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("sizes", [(3, 8, 5, 1, 2, 3, 40), (4, 6, 16, 4, 4, 1, 24), (2, 24, 12, 2, 3, 4, 64), (4, 32, 64, 2, 4, 4, 64),
                                   (2, 64, 128, 1, 4, 2, 48), (6, 20, 16, 3, 5, 5, 40), (1, 130, 8, 1, 2, 1, 32)])
def test_selective_state_space_part(dtype, sizes):
    """The whole mixer against the plain one: steps from tiny to large, rates from slow to fast, groups shared by
    several heads, a convolution whose memory is longer than a portion, slots used again."""
    from sprout_lm_b200.config.specs import PartSpec
    from sprout_lm_b200.parts import Runtime, WeightSource, build_part
    heads, vdim, n_state, groups, taps, norm_groups, width = sizes
    rng = np.random.default_rng(heads * 11 + vdim)
    inner = heads * vdim
    channels = inner + 2 * groups * n_state
    weights = {"m.in": rng.normal(0, 1.5 * width ** -0.5, size=(inner + channels + heads, width)), "m.conv": rng.normal(0, 0.6, size=(channels, taps)),
               "m.conv.b": rng.normal(0, 0.3, size=channels), "m.dt_bias": rng.uniform(-3.0, 1.0, size=heads),
               "m.A_log": rng.permutation(np.linspace(-5.0, 0.5, heads)), "m.D": rng.uniform(0.3, 1.5, size=heads),
               "m.norm": rng.normal(1.0, 0.3, size=inner), "m.o": rng.normal(0, inner ** -0.5, size=(width, inner))}
    stored = {k: rounded(v, "bfloat16") for k, v in weights.items()}
    weights = {k: f64(v) for k, v in stored.items()}
    part = build_part("mixer", PartSpec("selective_state_space", {"hidden_size": width, "heads": heads, "value_dim": vdim, "state": n_state,
                                                                  "groups": groups, "taps": taps, "norm_groups": norm_groups, "eps": 1e-5}), "m.")
    runtime = Runtime(DEV, DTYPES[dtype])
    part.load(WeightSource(lambda name: stored[name], runtime))
    m = {"heads": heads, "vdim": vdim, "state": n_state, "groups": groups, "conv": taps, "norm_groups": norm_groups}
    inputs = [rounded(rng.normal(0, 1.0, size=(n, width)), dtype) for n in (70, 1, 33, 150)]
    wants = [plain.mamba2_mixer(f64(h), weights, "m.", m, 1e-5) for h in inputs]
    conv_state = torch.full((3, taps - 1, channels), float("nan"), device=DEV)
    scan_state = torch.full((3, heads, n_state, vdim), float("nan"), device=DEV)

    def zero(slot):
        conv_state[slot].zero_(); scan_state[slot].zero_()
    tol = 3e-5 if dtype == "float32" else 6e-2
    _cut_three_ways(lambda batch: _run_mixer(part, batch, (conv_state, scan_state), width, dtype), zero, inputs, wants, tol)
    assert int(runtime.status.item()) == 0


# =============================================================================== whole models
@pytest.fixture(scope="module")
def model_dirs(tmp_path_factory):
    base = tmp_path_factory.mktemp("rarutar")
    return {name: rh.make_model_dir(base, name) for name in rh.CONFIGS}


def make_requests(name, seed, lengths):
    vocab = rh.CONFIGS[name][0]["vocab"]
    rng = np.random.default_rng(seed)
    return {f"r{i}": helpers.random_tokens(rng, n, vocab) for i, n in enumerate(lengths)}


def make_runner(model_dir, dtype, pages, page_tokens, requests=4):
    from sprout_lm_b200.engine.step import ModelRunner
    from sprout_lm_b200.models import load_model
    model = load_model(model_dir, dtype=DTYPES[dtype])
    return ModelRunner(model, num_pages=pages, page_tokens=page_tokens, max_requests=requests, prefix_caching=False)


def test_layers_one_by_one(model_dirs):
    """The stream after every layer in 32-bit, so that a fault names its layer."""
    from sprout_lm_b200.engine.batch import StepEntry
    for name, directory in model_dirs.items():
        config, tensors = rh.plain_model(directory)
        tokens = make_requests(name, 1, [41])["r0"]
        runner = make_runner(directory, "float32", 8, rh.CONFIGS[name][2])
        seen = []
        for block in runner.model.blocks:
            def wrapped(x, *args, _inner=block.forward, **more):
                _inner(x, *args, **more)
                seen.append(x.clone())
            block.forward = wrapped
        seq = runner.new_sequence()
        assert runner.reserve(seq, len(tokens))
        runner.step([StepEntry(seq, tokens, [0])])
        want = []
        plain.forward(config, tensors, tokens, layers_out=want)
        assert len(seen) == len(want)
        for i, (got, expected) in enumerate(zip(seen, want)):
            assert np.abs(got.cpu().numpy() - expected).max() <= 3e-5 * max(1.0, np.abs(expected).max()), (name, "layer", i)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_all_cuttings_in_process(model_dirs, name, dtype):
    """Whole, tail decoded token by token (80 tokens: every window and chunk of the models passes over decoded tokens),
    portions down to two tokens, mixed batches with pages and state slots used again: against the plain
    implementation, and in 32-bit equal to one another to rounding."""
    page = rh.CONFIGS[name][2]
    requests = make_requests(name, 11, [5, 17, 33, 70, 150, 1, 40])
    rng = np.random.default_rng(5)
    plans = {
        "whole": helpers.plan_whole(requests),
        "tail": helpers.plan_tail_decode(requests, tail=80),
        "portions": helpers.plan_portions(requests),
        "mixed": helpers.plan_mixed(requests, rng),
    }
    results = {}
    for label, plan in plans.items():
        budget = helpers.live_token_budget(plan, requests)
        runner = make_runner(model_dirs[name], dtype, budget // page, page, requests=4)
        got = results[label] = helpers.run_plan_in_process(runner, plan)
        assert len(got) == sum(len(t) for t in requests.values())
        worst = rh.compare(model_dirs[name], requests, got, TOL[dtype], f"{name}/{dtype}/{label}", page, rounded=dtype == "bfloat16")
        print(f"{name}/{dtype}/{label}: worst difference {worst:.2e}")
        runner.manager.check_invariants()
        assert len(runner.manager.pools[0].free) == runner.manager.pools[0].num_pages        # every page came back
        assert len(runner.manager._free_state) == 4                                           # and every state slot
    if dtype == "float32":
        for label in ("tail", "portions", "mixed"):
            for place, row in results["whole"].items():
                assert np.abs(row - results[label][place]).max() <= 2e-5, f"{name}: {label} differs from whole at {place}"


def test_long_context_and_long_decoding(model_dirs):
    """A prompt of several hundred tokens in uneven portions, then 140 tokens decoded one by one, in both dtypes: the
    slow decays' states, windows and chunks that are no multiple of a page, and keys many pages back."""
    for name, page, pages in (("B", 8, 90), ("C", 16, 45)):
        requests = make_requests(name, 21, [670])
        plan = helpers.plan_portions(requests, sizes=(130, 2, 127, 3, 64, 100, 2, 97, 5) + (1,) * 140)
        for dtype in ("float32", "bfloat16"):
            runner = make_runner(model_dirs[name], dtype, pages, page)
            got = helpers.run_plan_in_process(runner, plan)
            rh.compare(model_dirs[name], requests, got, TOL[dtype], f"long/{name}/{dtype}", page, rounded=dtype == "bfloat16")


def test_a_lost_state_a_dropped_sink_or_a_shifted_window_shows(model_dirs):
    """The test models are made so that each mechanism matters: the same tokens after another prefix, weights without
    the sinks, and windows or chunks one token off all move the logits by far more than the bar."""
    import copy
    name = "A"
    tokens = make_requests(name, 31, [60])["r0"]
    full = rh.plain_logits(model_dirs[name], tokens)
    tail_alone = rh.plain_logits(model_dirs[name], tokens[30:])
    bar = 3 * TOL["bfloat16"]

    def moved(other, places=slice(None)):
        """The largest change at any place: a fault is found if one place is over the bar."""
        return max(rh.relative(a, b) for a, b in zip(other, full[places]))
    assert moved(tail_alone, slice(30, None)) > bar
    config, tensors = rh.plain_model(model_dirs[name])
    no_sink = {k: (np.full_like(v, -30.0) if k.endswith(".sink") else v) for k, v in tensors.items()}
    assert moved(plain.forward(config, no_sink, tokens)) > bar
    for index, path in ((0, ("mixer", "left", "mask")), (2, ("mixer", "mask"))):
        shifted = copy.deepcopy(config)
        node = shifted["layers"][index]
        for key in path:
            node = node[key]
        node["size"] += 1
        assert moved(plain.forward(shifted, tensors, tokens)) > bar, path


def test_trace_replay_program(model_dirs, tmp_path):
    """bin/trace_run picks the model class by config.json and replays a mixed plan with four state slots."""
    name = "B"
    requests = make_requests(name, 13, [9, 40, 70, 23, 31, 12])
    plan = helpers.plan_mixed(requests, np.random.default_rng(2))
    budget = helpers.live_token_budget(plan, requests)
    vocab = rh.CONFIGS[name][0]["vocab"]
    for dtype in ("float32", "bfloat16"):
        got = helpers.run_plan_with_trace_run(model_dirs[name], dtype, plan, tmp_path / dtype, budget, vocab=vocab)
        rh.compare(model_dirs[name], requests, got, TOL[dtype], f"trace/{dtype}", 16, rounded=dtype == "bfloat16")


@pytest.mark.parametrize("name", ["A", "C"])
def test_greedy_generation_through_the_scheduler(model_dirs, name):
    """generate(): continuous batching, chunked prefill and captured decode steps; in 32-bit the tokens are the
    plain implementation's, in bfloat16 every token is within bfloat16's reach of the plain choice."""
    from sprout_lm_b200 import generate, load_model
    config, tensors = rh.plain_model(model_dirs[name])
    rng = np.random.default_rng(7)
    prompts = [helpers.random_tokens(rng, n, config["vocab"]) for n in (3, 19, 44)]
    new_tokens = 12
    for dtype in ("float32", "bfloat16"):
        model = load_model(model_dirs[name], dtype=dtype)
        results = generate(model, prompts, max_new_tokens=new_tokens, ignore_eos=True)
        for prompt, result in zip(prompts, results):
            assert len(result["output"]) == new_tokens
            if dtype == "float32":
                assert result["output"] == rh.plain_greedy(model_dirs[name], prompt, new_tokens)
                continue
            history = list(prompt)
            for token in result["output"]:
                row = plain.forward(config, tensors, history)[-1]
                assert row[token] >= row.max() - 4 * TOL["bfloat16"], (name, len(history), token)
                history.append(token)


def test_scheduler_under_page_pressure(model_dirs):
    """A pool smaller than the requests together: a preempted request gives its state slot back and recomputes its
    state from the start; the greedy tokens stay the plain implementation's."""
    from sprout_lm_b200 import EngineOptions, generate, load_model
    name = "A"
    config, _ = rh.plain_model(model_dirs[name])
    rng = np.random.default_rng(8)
    prompts = [helpers.random_tokens(rng, n, config["vocab"]) for n in (30, 41, 26, 35)]
    model = load_model(model_dirs[name], dtype="float32")
    options = EngineOptions(block_size=8, num_blocks=14, max_sequences=4, max_batch_tokens=24, prefill_chunk_size=7)
    results = generate(model, prompts, max_new_tokens=10, ignore_eos=True, options=options)
    for prompt, result in zip(prompts, results):
        assert result["output"] == rh.plain_greedy(model_dirs[name], prompt, 10)
