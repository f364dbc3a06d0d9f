"""Babotar on the GPU against the plain float64 implementation (``tests/plain/babotar_plain.py``): each mechanism's kernels
alone, then whole models under every way of cutting and batching their requests, through the engine's own step function,
cache manager, scheduler and entry point. Sizes are the tests' own (``babotar_util.CONFIGS``)."""
import numpy as np
import pytest
import torch

import conftest
from plain import babotar_plain as plain
import babotar_util as bu
import zurerax_util as zu

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

# bfloat16 against float64: the recurrences carry every rounding of their inputs forward, and the models' logits have a
# spread near one, so the bound is on the worst row's mean error and on the worst element, relative to the spread.
BF16_REL_MAX, BF16_REL_MEAN = 0.4, 0.08


def assert_logits_close(got, want, dtype, what=""):
    if dtype == "float32":
        return conftest.assert_logits_close(got, want, dtype, what)
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape and np.isfinite(got).all(), what
    diff, spread = np.abs(got - want), want.std()
    assert diff.max() <= BF16_REL_MAX * spread, f"{what}: worst element {diff.max():.3e} > {BF16_REL_MAX} x spread {spread:.3e}"
    assert diff.mean(1).max() <= BF16_REL_MEAN * spread, f"{what}: worst row's mean {diff.mean(1).max():.3e} (spread {spread:.3e})"


def _i32(values):
    return torch.tensor(values, dtype=torch.int32, device=DEV)


def _f32(a):
    return torch.tensor(np.asarray(a, dtype=np.float32), device=DEV)


def _status():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


def _rounded(a, dtype):
    """``a`` as float64, rounded to ``dtype`` first, so that kernel and plain implementation start from the same numbers."""
    return torch.tensor(np.asarray(a), dtype=torch.float32).to(dtype).double().numpy()


class _Pages:
    """A paged cache for a few requests whose pages lie scattered and interleaved in the pool."""

    def __init__(self, lengths, G, D, V, page, dtype, seed=0):
        rng = np.random.default_rng(seed)
        need = [-(-n // page) for n in lengths]
        order = rng.permutation(sum(need) + 3)
        self.page, self.tables, at = page, [], 0
        for k in need:
            self.tables.append([int(p) for p in order[at:at + k]])
            at += k
        self.width = max(need)
        self.k = torch.zeros((sum(need) + 3, G, page, D), dtype=dtype, device=DEV)
        self.v = torch.zeros((sum(need) + 3, G, page, V), dtype=dtype, device=DEV)

    def row(self, seq):
        return self.tables[seq] + [-1] * (self.width - len(self.tables[seq]))

    def slot(self, seq, pos):
        return self.tables[seq][pos // self.page] * self.page + pos % self.page


def _step_meta(step, at):
    """Device metadata of one step of (request, rows) entries (None: a padding sequence of one row)."""
    row_seq, positions, first, start, row = [], [], [], [], 0
    for s, e in enumerate(step):
        first.append(row)
        if e is None:
            start.append(-1); row_seq.append(s); positions.append(-1); row += 1
            continue
        start.append(at[e[0]])
        row_seq += [s] * e[1]
        positions += [at[e[0]] + i for i in range(e[1])]
        row += e[1]
    first.append(row)
    return row, _i32(row_seq), _i32(positions), _i32(first), _i32(start)


def _cuts(lengths, rng, tail=True):
    """Steps that bring every request in: portions of changing sizes side by side (down to one and two rows), then (``tail``)
    the last third of each request token by token, all requests in one step, finished ones as padding sequences."""
    at, steps = [0] * len(lengths), []
    stop = [n - (n // 3 if tail else 0) for n in lengths]
    while any(a < s for a, s in zip(at, stop)):
        step = []
        for r in range(len(lengths)):
            if at[r] < stop[r] and rng.random() < 0.8:
                k = min(int(rng.choice([1, 2, 3, 15, 16, 17, 40, 64, 70])), stop[r] - at[r])
                step.append((r, k))
                at[r] += k
        if step:
            steps.append(step)
    while any(a < n for a, n in zip(at, lengths)):
        steps.append([(r, 1) if at[r] < lengths[r] else None for r in range(len(lengths))])
        for r in range(len(lengths)):
            at[r] += at[r] < lengths[r]
    return steps


def _gather(step, at, rows_in, width):
    n = sum(1 if e is None else e[1] for e in step)
    x, row = np.zeros((n, width)), 0
    for e in step:
        if e is None:
            row += 1
            continue
        x[row:row + e[1]] = rows_in[e[0]][at[e[0]]:at[e[0]] + e[1]]
        row += e[1]
    return x


def _scatter(step, at, out, got):
    row = 0
    for e in step:
        if e is None:
            row += 1
            continue
        got[e[0]][at[e[0]]:at[e[0]] + e[1]] = out[row:row + e[1]]
        row += e[1]
        at[e[0]] += e[1]


# ---------------------------------------------------------------------------------------------- each mechanism alone
def test_learned_positions_join_the_embedding():
    from glassbox_b200 import kernels
    rng = np.random.default_rng(0)
    for dtype in (torch.float32, torch.bfloat16):
        table, pos_table = _f32(rng.standard_normal((37, 50))).to(dtype), _f32(rng.standard_normal((23, 50))).to(dtype)
        tokens, positions = [5, 36, 0, 7, 7], [0, 22, -1, 3, 4]
        x, status = torch.full((5, 50), 9.0, device=DEV), _status()
        kernels.embed_positions(table, pos_table, _i32(tokens), _i32(positions), x, status)
        want = table.float()[tokens] + pos_table.float()[[max(p, 0) for p in positions]]
        want[2] = 0.0                                            # a padding row is cleared
        assert torch.equal(x, want) and int(status.item()) == 0
        kernels.embed_positions(table, pos_table, _i32([1]), _i32([23]), x[:1], status)      # a position past the table
        assert int(status.item()) == 4


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("taps, C", [(1, 33), (2, 50), (3, 64), (5, 7), (4, 300)])
def test_input_convolution_carries_its_last_inputs(dtype, taps, C):
    """h + conv(h) for requests that arrive in portions of one, two and many rows, beside padding sequences; the slots of other
    requests stay as they were."""
    from glassbox_b200 import kernels
    rng = np.random.default_rng(taps * 100 + C)
    lengths = [67, 1, 9, 30]
    rows_in = [_rounded(rng.standard_normal((n, C)), dtype) for n in lengths]
    w = _rounded(rng.standard_normal((C, taps)) * 0.5, dtype)
    off, slots = 3, [4, 0, 2, 5]
    state = torch.zeros((7, off + max(taps - 1, 1) * C + 2), device=DEV)
    state[[1, 3, 6]] = 7.0
    state[:, :off] = 7.0
    got, at, status = [np.zeros((n, C)) for n in lengths], [0] * len(lengths), _status()
    for step in _cuts(lengths, rng):
        n, row_seq, positions, first, start = _step_meta(step, at)
        x = _f32(_gather(step, at, rows_in, C)).to(dtype)
        y = torch.zeros_like(x)
        seq_slots = _i32([0 if e is None else slots[e[0]] for e in step])
        single = all(e is None or e[1] == 1 for e in step)          # (then the same launch moves the last inputs up)
        kernels.residual_conv(x, _f32(w), y, state, off, row_seq, positions, first, start, seq_slots, True, status, single_rows=single)
        _scatter(step, at, y.float().cpu().numpy(), got)
    assert int(status.item()) == 0
    assert bool((state[[1, 3, 6]] == 7.0).all()) and bool((state[:, :off] == 7.0).all()) and bool((state[:, off + max(taps - 1, 1) * C:] == (
        torch.tensor([0, 7, 0, 7, 0, 0, 7], device=DEV)[:, None])).all())
    for r, n in enumerate(lengths):
        want = rows_in[r] + plain.causal_conv(rows_in[r], w)
        tol = 1e-5 if dtype == torch.float32 else 0.02
        np.testing.assert_allclose(got[r], want, atol=tol * max(1.0, np.abs(want).max()), err_msg=f"request {r}")


def test_gelu_gated_unit_and_weighted_sum():
    from glassbox_b200 import kernels
    rng = np.random.default_rng(3)
    for n, ff in [(1, 1), (7, 11), (33, 64)]:
        gu = rng.standard_normal((n, 2 * ff)) * 2.5
        for dtype, tol in ((torch.float32, 1e-6), (torch.bfloat16, 0.01)):
            act = torch.zeros((n, ff), dtype=dtype, device=DEV)
            kernels.gelu_glu(_f32(gu), act)
            np.testing.assert_allclose(act.float().cpu().numpy(), plain.gelu_tanh(gu[:, :ff]) * gu[:, ff:], atol=tol * 8, rtol=tol)
    a, b, out = rng.standard_normal((5, 9)), rng.standard_normal((5, 9)), rng.standard_normal((5, 9))
    o = _f32(out)
    kernels.scaled_sum(_f32(a), _f32(b), 0.6, -1.5, o, accumulate=True)
    np.testing.assert_allclose(o.cpu().numpy(), out + 0.6 * a - 1.5 * b, atol=1e-6)
    kernels.scaled_sum(_f32(a), _f32(b), 0.6, -1.5, o, accumulate=False)
    np.testing.assert_allclose(o.cpu().numpy(), 0.6 * a - 1.5 * b, atol=1e-6)


@pytest.mark.parametrize("n, ff, d", [(1, 64, 128), (8, 48, 72), (64, 256, 128), (65, 64, 128), (300, 136, 64), (2048, 512, 256)])
def test_gelu_gated_unit_in_a_products_epilogue(n, ff, d):
    """The two products of a feed-forward's first half with gelu_tanh(gate) * up formed from their float32 sums, in the kernel
    for few rows (the weights streamed once) and in the tile kernel."""
    from glassbox_b200 import kernels
    rng = np.random.default_rng(n + ff)
    bf = lambda a: _f32(a).to(torch.bfloat16)
    h, w = bf(rng.standard_normal((n, d))), bf(rng.standard_normal((2 * ff, d)) * 2.0 / np.sqrt(d))
    z = h.float().cpu().numpy().astype(np.float64) @ w.float().cpu().numpy().astype(np.float64).T
    want = plain.gelu_tanh(z[:, :ff]) * z[:, ff:]
    limit, slope = kernels.GELU_UNIT
    ran = 0
    if kernels.gemm_stream_supported(h, w) and ff % 16 == 0:
        act = torch.zeros((n, ff), dtype=torch.bfloat16, device=DEV)
        kernels.gemm_stream_unit(h, w, None, limit, slope, act)
        np.testing.assert_allclose(act.float().cpu().numpy(), want, atol=2e-2, rtol=1e-2)
        ran += 1
    act = torch.zeros((n, ff), dtype=torch.bfloat16, device=DEV)
    if kernels.gemm_tc_supported(h, w, act):
        status = _status()
        kernels.gemm_tc_unit(h, w, None, limit, slope, act, status)
        assert int(status.item()) == 0
        np.testing.assert_allclose(act.float().cpu().numpy(), want, atol=2e-2, rtol=1e-2)
        ran += 1
    assert ran >= 1


def _identity_rows(pieces):
    """{name: rows of an identity matrix} that pick the named parts of a stacked row apart."""
    eye, out, at = np.eye(sum(n for _, n in pieces)), {}, 0
    for name, n in pieces:
        out[name] = eye[at:at + n]
        at += n
    return out


@pytest.mark.parametrize("H, D, V", [(3, 10, 6), (4, 64, 64), (1, 8, 1), (2, 128, 64), (2, 7, 33), (2, 200, 16), (5, 32, 128)])
def test_lightning_recurrence_norm_and_gate(H, D, V):
    """The recurrence with a fixed decay per head (one, zero and between), SiLU on its inputs, the joint norm and the gate,
    for requests in portions and single tokens with the state carried in slots."""
    from glassbox_b200 import kernels
    rng = np.random.default_rng(H * 100 + D)
    decay = ([1.0, 0.0, 0.5, 0.97, 0.999] * 2)[:H]
    m = {"heads": H, "dim": D, "vdim": V, "decay": decay}
    W = _identity_rows([("q", H * D), ("k", H * D), ("v", H * V), ("g", H * V)])
    W.update({"o": np.eye(H * V), "norm": 1 + 0.3 * rng.standard_normal(H * V)})
    cols = 2 * H * D + 2 * H * V
    lengths = [90, 1, 23]
    rows_in = [_rounded(rng.standard_normal((n, cols)), torch.float32) for n in lengths]
    slots = [2, 0, 3]
    state = torch.zeros((5, H * D * V + 5), device=DEV)
    state[[1, 4]] = 3.0
    got, at, status, used = [np.zeros((n, H * V)) for n in lengths], [0] * len(lengths), _status(), set()
    for step in _cuts(lengths, rng):
        n, row_seq, positions, first, start = _step_meta(step, at)
        proj = _f32(_gather(step, at, rows_in, cols))
        o = torch.zeros((n, H * V), device=DEV)
        att = torch.zeros((n, H * V), device=DEV)
        seq_slots = _i32([0 if e is None else slots[e[0]] for e in step])
        single = all(e is None or e[1] == 1 for e in step)
        run = kernels.decay_linear_attention_decode if single and kernels.channel_delta_decode_supported(D, V) else kernels.decay_linear_attention
        used.add(run.__name__)
        run(proj[:, :2 * H * D + H * V], _f32(decay), state, o, first, start, seq_slots, H, D, V, True, status)
        kernels.gated_head_norm(o, proj[:, 2 * H * D + H * V:], _f32(W["norm"]), att, 1, 1e-5)
        _scatter(step, at, att.cpu().numpy(), got)
    assert int(status.item()) == 0 and bool((state[[1, 4]] == 3.0).all())
    assert ("decay_linear_attention_decode" in used) == (D <= 128 and V <= 128) and "decay_linear_attention" in used
    for r in range(len(lengths)):
        want = plain.lightning(rows_in[r], W, "", m, 1e-5)
        np.testing.assert_allclose(got[r], want, atol=3e-5 * max(1.0, np.abs(want).max()), rtol=1e-4, err_msg=f"request {r}")


@pytest.mark.parametrize("H, D, V", [(3, 10, 6), (4, 64, 64), (2, 128, 128), (2, 40, 70), (1, 200, 16)])
def test_lightning_over_long_portions_in_pieces(H, D, V):
    """Long portions cut into pieces that walk side by side and are chained afterwards equal the walk over the whole portion:
    requests of unequal length side by side, a padding sequence between them, portions that end inside a piece, a state carried
    in from an earlier step and out to a later one, decays of one, zero and between."""
    from glassbox_b200 import kernels
    rng = np.random.default_rng(H * 100 + D)
    decay = ([1.0, 0.0, 0.5, 0.97, 0.999] * 2)[:H]
    m = {"heads": H, "dim": D, "vdim": V, "decay": decay}
    W = _identity_rows([("q", H * D), ("k", H * D), ("v", H * V), ("g", H * V)])
    W.update({"o": np.eye(H * V), "norm": np.ones(H * V)})
    cols = 2 * H * D + 2 * H * V
    lengths = [700, 130, 3, 515]
    rows_in = [_rounded(rng.standard_normal((n, cols)), torch.float32) for n in lengths]
    rows_in = [np.concatenate([r[:, :2 * H * D + H * V], np.full((len(r), H * V), 30.0)], 1) for r in rows_in]      # (gate wide open)
    slots = [2, 0, 3, 5]
    state = torch.zeros((7, H * D * V), device=DEV)
    state[[1, 4, 6]] = 3.0
    steps = [[(0, 5), (3, 129)], [(0, 400), None, (1, 130), (2, 3), (3, 386)], [(0, 295), None]]
    got, at, status = [np.zeros((n, H * V)) for n in lengths], [0] * len(lengths), _status()
    for step in steps:
        n, row_seq, positions, first, start = _step_meta(step, at)
        proj = _f32(_gather(step, at, rows_in, cols))
        o = torch.full((n, H * V), float("nan"), device=DEV)
        seq_slots = _i32([0 if e is None else slots[e[0]] for e in step])
        piece_rows = [128, 192, 320][n % 3]                           # (another length of the pieces at every step)
        pieces = kernels.linear_pieces_needed(n, len(step), piece_rows)
        meta = torch.zeros(4 * pieces + 2 * len(step) + 1, dtype=torch.int32, device=DEV)
        piece_state = torch.full((pieces, H * D * V), float("nan"), device=DEV)
        kernels.decay_linear_attention_pieces(proj[:, :2 * H * D + H * V], _f32(decay), state, o, first, start, seq_slots, H, D, V, True,
                                              status, meta, piece_state, piece_rows=piece_rows)
        _scatter(step, at, o.cpu().numpy(), got)
    assert int(status.item()) == 0 and bool((state[[1, 4, 6]] == 3.0).all())
    for r in range(len(lengths)):
        q = plain.silu(rows_in[r][:, :H * D]).reshape(-1, H, D)
        k = plain.silu(rows_in[r][:, H * D:2 * H * D]).reshape(-1, H, D)
        v = plain.silu(rows_in[r][:, 2 * H * D:2 * H * D + H * V]).reshape(-1, H, V)
        want = np.zeros((lengths[r], H, V))
        for h in range(H):
            S = np.zeros((D, V))
            for t in range(lengths[r]):
                S = decay[h] * S + np.outer(k[t, h], v[t, h])
                want[t, h] = S.T @ q[t, h]
        np.testing.assert_allclose(got[r], want.reshape(lengths[r], -1), atol=1e-4 * max(1.0, np.abs(want).max()), rtol=2e-4,
                                   err_msg=f"request {r}")


def test_lightning_in_closed_form():
    """Inputs whose SiLU is known: with q = k = a constant vector and v constant, o_t = |k|^2 v sum_j decay^(t - j)."""
    from glassbox_b200 import kernels
    H, D, V, T = 2, 4, 3, 40
    decay = [0.5, 1.0]
    x = np.zeros((T, 2 * H * D + H * V))
    x[:, :2 * H * D] = 1.0
    x[:, 2 * H * D:] = 2.0
    s1, s2 = 1.0 / (1.0 + np.exp(-1.0)), 2.0 / (1.0 + np.exp(-2.0))
    state, o = torch.zeros((1, H * D * V), device=DEV), torch.zeros((T, H * V), device=DEV)
    kernels.decay_linear_attention(_f32(x), _f32(decay), state, o, _i32([0, T]), _i32([0]), _i32([0]), H, D, V, True, _status())
    got = o.cpu().numpy().reshape(T, H, V)
    for t in range(T):
        for h, g in enumerate(decay):
            np.testing.assert_allclose(got[t, h], D * s1 * s1 * s2 * sum(g ** (t - j) for j in range(t + 1)), rtol=2e-5)


@pytest.mark.parametrize("H, G, D, V, taps", [(4, 2, 12, 6, 4), (4, 2, 64, 64, 4), (1, 1, 8, 1, 1), (2, 1, 128, 128, 2), (3, 1, 9, 7, 3),
                                              (2, 2, 20, 130, 2)])
def test_gated_delta_rule_with_one_decay_per_head(H, G, D, V, taps):
    """Convolutions, unit vectors, one decay per head and token, the recurrence, the per-head norm and the silu gate: prompt
    portions on the walking kernel, single tokens on the decoding kernel, states and last inputs carried in slots."""
    from glassbox_b200 import kernels
    rng = np.random.default_rng(H * 100 + D + taps)
    m = {"heads": H, "kv_heads": G, "dim": D, "vdim": V, "conv": taps}
    conv_cols = 2 * G * D + H * V
    W = _identity_rows([("q", G * D), ("k", G * D), ("v", H * V), ("a", H), ("b", H), ("g", H * V)])
    W.update({"o": np.eye(H * V), "norm": 1 + 0.3 * rng.standard_normal(V), "A_log": rng.uniform(-2, 0.5, H), "dt_bias": rng.standard_normal(H),
              "q.conv": rng.standard_normal((G * D, taps)) * 0.6, "k.conv": rng.standard_normal((G * D, taps)) * 0.6,
              "v.conv": rng.standard_normal((H * V, taps)) * 0.6})
    W = {k: _rounded(v, torch.float32) for k, v in W.items()}
    conv = _f32(np.concatenate([W["q.conv"], W["k.conv"], W["v.conv"]], 0))
    cols = conv_cols + 2 * H + H * V
    lengths = [70, 1, 26]
    rows_in = [_rounded(rng.standard_normal((n, cols)) * 1.5, torch.float32) for n in lengths]
    slots = [1, 3, 0]
    numbers = H * D * V
    state = torch.zeros((4, numbers + max(taps - 1, 0) * conv_cols), device=DEV)
    state[2] = 5.0
    got, at, status = [np.zeros((n, H * V)) for n in lengths], [0] * len(lengths), _status()
    used_decode = False
    for step in _cuts(lengths, rng):
        n, row_seq, positions, first, start = _step_meta(step, at)
        proj = _f32(_gather(step, at, rows_in, cols))
        seq_slots = _i32([0 if e is None else slots[e[0]] for e in step])
        qkv = torch.zeros((n, conv_cols), device=DEV)
        kernels.short_conv(proj[:, :conv_cols], conv, qkv, state, numbers, row_seq, positions, first, start, seq_slots, True, status)
        a, b, g = proj[:, conv_cols:conv_cols + H], proj[:, conv_cols + H:conv_cols + 2 * H], proj[:, conv_cols + 2 * H:]
        att = torch.zeros((n, H * V), device=DEV)
        single = all(e is None or e[1] == 1 for e in step)
        if single and kernels.channel_delta_decode_supported(D, V):
            used_decode = True
            kernels.channel_delta_decode(qkv, b, a, _f32(W["dt_bias"]), _f32(W["A_log"]), state, g, _f32(W["norm"]), 1e-5, att, first, start,
                                         seq_slots, H, G, D, V, True, status, decay_per_head=True, gate_silu=True)
        else:
            o = torch.zeros((n, H * V), device=DEV)
            kernels.channel_delta(qkv, b, a, _f32(W["dt_bias"]), _f32(W["A_log"]), state, o, first, start, seq_slots, H, G, D, V, True,
                                  status, decay_per_head=True)
            kernels.gated_head_norm(o, g, _f32(W["norm"]), att, H, 1e-5, gate_silu=True)
        _scatter(step, at, att.cpu().numpy(), got)
    assert int(status.item()) == 0 and bool((state[2] == 5.0).all()) and used_decode == (V <= 128)
    for r in range(len(lengths)):
        want = plain.gated_delta(rows_in[r], W, "", m, 1e-5)
        np.testing.assert_allclose(got[r], want, atol=1e-4 * max(1.0, np.abs(want).max()), rtol=2e-4, err_msg=f"request {r}")


# ------------------------------------------------------------------------------ attention whose heads exchange their weights
ATTENTION_PATHS = [("rows", torch.float32), ("rows", torch.bfloat16), ("fast", torch.bfloat16), ("fast", torch.float32)]


def _attend(kernels, how, q, wide, cache, tables, row_seq, positions, first, start, longest, single, common):
    """``how`` "rows": the one-warp-per-(row, head) kernel; "fast": what the mixer picks for a bfloat16 step (single tokens
    the decoding kernel, portions the tensor-core tiles), where its head sizes have such a kernel."""
    from glassbox_b200.parts import talking_attention as ta
    if how == "fast":
        picked = ta.pick_kernel(q.dtype, single, common["heads"], common["kv_heads"], common["dim"], common["vdim"], common["value_heads"])
        if picked == "decode":
            # another number of shares of the keys at every step; the mix then merges the shares
            n, shares = q.shape[0], [1, 3, 2, 5, 16][int(positions.max().item()) % 5]
            if shares == 1:
                return kernels.talking_attention_decode(q, wide, cache.k, cache.v, tables, row_seq, positions, **common)
            parts = torch.full((shares * n, wide.shape[1]), float("nan"), device=DEV)
            ml = torch.full((shares * n, common["heads"] * 2), float("nan"), device=DEV)
            kernels.talking_attention_decode(q, parts, cache.k, cache.v, tables, row_seq, positions, shares=shares, ml=ml, **common)
            return parts, ml, shares
        if picked == "tiles":
            return kernels.talking_attention_tiles(q, wide, cache.k, cache.v, tables, first, start, longest, **common)
    kernels.talking_attention_rows(q, wide, cache.k, cache.v, tables, row_seq, positions, **common)


def _run_left_steps(kernels, how, steps, lengths, rows_in, m, W, cache, dtype, talk=True):
    """Biases, rotation and cache write, attention over every key/value head's values, the mix of the heads: step by step."""
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    from glassbox_b200.parts.rope import rotary_table
    from glassbox_b200.config.specs import RopeRescaleSpec
    rot_dims, table = 0, None
    if m.get("rot") is not None:
        r = m["rot"]
        sc = r.get("scaling")
        rescale = RopeRescaleSpec(sc["factor"], sc["original"], sc["fast"], sc["slow"]) if sc else None
        rot_dims, table = r["dims"], rotary_table(r["base"], r["dims"], 512, rescale).to(DEV)
    bias = _f32(np.concatenate([W["q.b"], W["k.b"], W["v.b"]]))
    status = _status()
    got, at = [np.zeros((n, H * V)) for n in lengths], [0] * len(lengths)
    VG = G if talk else 1
    common = dict(heads=H, kv_heads=G, dim=D, vdim=V, value_heads=VG, page_size=cache.page, scale=m["scale"], softcap=m.get("softcap"),
                  unit_sink=True, window=None, status=status)
    for step in steps:
        n, row_seq, positions, first, start = _step_meta(step, at)
        proj = _f32(_gather(step, at, rows_in, (H + G) * D + G * V))
        slots, row = [-1] * n, 0
        for e in step:
            if e is not None:
                slots[row:row + e[1]] = [cache.slot(e[0], at[e[0]] + i) for i in range(e[1])]
            row += 1 if e is None else e[1]
        q = torch.zeros((n, H * D), dtype=dtype, device=DEV)
        kernels.bias_rope_write(proj, bias, table, positions, _i32(slots), q, cache.k, cache.v, H, G, D, V, rot_dims, cache.page, True, status)
        tables = _i32([[-1] * cache.width if e is None else cache.row(e[0]) for e in step])
        wide = torch.full((n, H * VG * V), float("nan"), device=DEV)
        single = all(e is None or e[1] == 1 for e in step)
        shared = _attend(kernels, how, q, wide, cache, tables, row_seq, positions, first, start, max(e[1] for e in step if e), single, common)
        att = torch.zeros((n, H * V), dtype=dtype, device=DEV)
        if shared is not None:
            kernels.talk_combine(shared[0], _f32(W["talk"]) if talk else None, att, positions, H, G, V, VG, shares=shared[2], ml=shared[1])
        else:
            kernels.talk_combine(wide, _f32(W["talk"]) if talk else None, att, positions, H, G, V, VG)
        _scatter(step, at, att.float().cpu().numpy(), got)
    assert int(status.item()) == 0
    return got


def _left_by_identity(H, G, D, V, rng, rotation, softcap, scale):
    m = bu.left(H, G, D, V, rotation, softcap, scale)
    W = _identity_rows([("q", H * D), ("k", G * D), ("v", G * V)])
    W.update({"o": np.eye(H * V), "q.b": rng.standard_normal(H * D) * 0.5, "k.b": rng.standard_normal(G * D) * 0.5,
              "v.b": rng.standard_normal(G * V) * 0.5, "talk": np.eye(H) + rng.standard_normal((H, H)) * 0.4})
    return m, {k: _rounded(v, torch.float32) for k, v in W.items()}


@pytest.mark.parametrize("how, dtype", ATTENTION_PATHS)
@pytest.mark.parametrize("H, G, D, V, rot_dims, scaling, cap", [
    (6, 2, 20, 12, 12, (4.0, 64, 8.0, 2.0), 5.0), (4, 4, 16, 24, 16, None, 2.0), (8, 2, 64, 64, 64, (8.0, 128, 16.0, 1.0), 30.0),
    (4, 1, 128, 64, 128, None, None), (1, 1, 8, 1, 2, (2.0, 8, 2.0, 1.0), None), (3, 1, 10, 7, 6, (3.0, 32, 4.0, 1.0), 4.0),
    (4, 4, 32, 32, 0, None, 10.0), (16, 4, 64, 64, 32, None, 50.0), (2, 2, 128, 128, 64, None, None), (8, 4, 32, 128, 16, None, 6.0),
    (6, 6, 16, 128, 0, None, None)])
def test_talking_attention_kernels(how, dtype, H, G, D, V, rot_dims, scaling, cap):
    """Three requests of unequal length whose pages lie interleaved, brought in by portions and single tokens, against the
    plain mixer over each whole request."""
    from glassbox_b200 import kernels
    rng = np.random.default_rng(H * 1000 + D)
    rotation = bu.rot(rot_dims, 300.0, scaling) if rot_dims else None
    m, W = _left_by_identity(H, G, D, V, rng, rotation, cap, 1.3 * D ** -0.5)
    lengths = [131, 1, 50]
    rows_in = [_rounded(rng.standard_normal((n, (H + G) * D + G * V)), torch.float32) for n in lengths]
    cache = _Pages(lengths, G, D, V, 16, dtype, seed=D)
    got = _run_left_steps(kernels, how, _cuts(lengths, rng), lengths, rows_in, m, W, cache, dtype)
    for r in range(len(lengths)):
        want = plain.talking_softmax_attention(rows_in[r], W, "", m)
        if dtype == torch.float32:
            np.testing.assert_allclose(got[r], want, atol=3e-5, rtol=1e-4, err_msg=f"request {r}")
        else:
            assert np.abs(got[r] - want).max() <= 0.04 * max(1.0, np.abs(want).max()), f"request {r}"


@pytest.mark.parametrize("how, dtype", ATTENTION_PATHS)
@pytest.mark.parametrize("back", [0, 1, 15, 16, 17, 31, 32, 33, 63, 64, 65, 127, 128, 129, 300])
def test_a_marked_key_decides(how, dtype, back):
    """One key ``back`` tokens behind the query (at page borders, tile borders, far away, the query itself, the first token)
    has a score far above the others': the output is that key's value. Every key's value names its position. In a prompt's
    portion and for a single token."""
    from glassbox_b200 import kernels
    H, G, D, V, T = 4, 2, 32, 32, 330
    rng = np.random.default_rng(back)
    m, W = _left_by_identity(H, G, D, V, rng, None, None, 1.0)
    for k in ("q.b", "k.b", "v.b"):
        W[k][:] = 0.0
    W["talk"] = np.eye(H)
    x = np.zeros((T, (H + G) * D + G * V))
    x[:, H * D:(H + G) * D] = _rounded(rng.standard_normal((T, G * D)) * 0.1, dtype)
    values = np.zeros((T, G, V))
    for t in range(T):
        values[t, :, t % V] = 1.0 + t // V                      # position t <-> (channel, height)
    x[:, (H + G) * D:] = values.reshape(T, -1)
    marked = T - 1 - back
    x[marked, H * D:(H + G) * D] = 0.0
    x[marked, H * D] = x[marked, H * D + D] = 8.0               # the marked key, in both key heads
    x[T - 1, :H * D] = 0.0
    x[T - 1, 0:H * D:D] = 8.0                                   # the last query asks for it: score 64 against ~0
    for tail in (False, True):
        cache = _Pages([T], G, D, V, 16, dtype, seed=back)
        steps = [[(0, T - 1)], [(0, 1)]] if tail else [[(0, 100)], [(0, T - 100)]]
        got = _run_left_steps(kernels, how, steps, [T], [x], m, W, cache, dtype)[0][T - 1].reshape(H, V)
        want = np.zeros(V)
        want[marked % V] = 1.0 + marked // V
        np.testing.assert_allclose(got, np.tile(want, (H, 1)), atol=2e-2 if dtype == torch.bfloat16 else 1e-4,
                                   err_msg=f"key {back} back, {'single token' if tail else 'portion'}")


@pytest.mark.parametrize("how, dtype", ATTENTION_PATHS)
def test_unit_sink_cap_and_mix_in_closed_form(how, dtype):
    """Equal scores: n visible keys weigh 1 / (n + 1) each, the missing share is the sink's. A cap below the raw scores makes
    unequal keys nearly equal. A mixing matrix that swaps two heads gives each the other's weights on its OWN values."""
    from glassbox_b200 import kernels
    H, G, D, V, T = 2, 2, 16, 16, 40
    rng = np.random.default_rng(1)
    m, W = _left_by_identity(H, G, D, V, rng, None, None, 1.0)
    for k in ("q.b", "k.b", "v.b"):
        W[k][:] = 0.0
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
    x = np.zeros((T, (H + G) * D + G * V))
    x[:, (H + G) * D:] = _rounded(rng.standard_normal((T, G * V)), dtype)
    v = x[:, (H + G) * D:].reshape(T, G, V)
    W["talk"] = np.eye(H)
    cache = _Pages([T], G, D, V, 16, dtype)
    got = _run_left_steps(kernels, how, [[(0, 17)], [(0, 1)], [(0, T - 18)]], [T], [x], m, W, cache, dtype)[0].reshape(T, H, V)
    for t in (0, 1, 16, 17, T - 1):
        np.testing.assert_allclose(got[t], v[:t + 1].sum(0) / (t + 2), atol=tol, err_msg=f"equal scores, row {t}")
    # head 0 looks at key 3 alone (score 30), head 1 at key 5 alone; swapped weights: head 0 gets key 5 of its own values
    x2 = x.copy()
    x2[3, H * D] = x2[5, H * D + D + 1] = 6.0
    x2[T - 1, 0], x2[T - 1, D + 1] = 5.0, 5.0
    W["talk"] = np.array([[0.0, 1.0], [1.0, 0.0]])
    cache = _Pages([T], G, D, V, 16, dtype)
    got = _run_left_steps(kernels, how, [[(0, T - 1)], [(0, 1)]], [T], [x2], m, W, cache, dtype)[0].reshape(T, H, V)
    np.testing.assert_allclose(got[T - 1, 0], v[5, 0], atol=tol * 3)
    np.testing.assert_allclose(got[T - 1, 1], v[3, 1], atol=tol * 3)
    # raw scores 30 (key 3) and 60 (key 7) under a cap of 0.1: every key weighs exp(+-0.1) at most
    x3 = x.copy()
    x3[3, H * D], x3[7, H * D] = 6.0, 12.0
    x3[T - 1, 0] = 5.0
    W["talk"] = np.eye(H)
    m3 = dict(m, softcap=0.1)
    cache = _Pages([T], G, D, V, 16, dtype)
    got = _run_left_steps(kernels, how, [[(0, T)]], [T], [x3], m3, W, cache, dtype)[0].reshape(T, H, V)
    e = np.ones(T)
    e[3], e[7] = np.exp(0.1 * np.tanh(300.0)), np.exp(0.1 * np.tanh(600.0))
    np.testing.assert_allclose(got[T - 1, 0], (e[:, None] * v[:, 0]).sum(0) / (1.0 + e.sum()), atol=tol)


def test_heads_that_do_not_talk_read_their_own_values_only():
    from glassbox_b200 import kernels
    rng = np.random.default_rng(2)
    H, G, D, V = 4, 2, 16, 8
    m, W = _left_by_identity(H, G, D, V, rng, bu.rot(8, 100.0), 3.0, 0.4)
    W["talk"] = np.eye(H)
    lengths = [40, 7]
    rows_in = [_rounded(rng.standard_normal((n, (H + G) * D + G * V)), torch.float32) for n in lengths]
    for talk in (True, False):
        cache = _Pages(lengths, G, D, V, 16, torch.float32)
        got = _run_left_steps(kernels, "rows", _cuts(lengths, rng), lengths, rows_in, m, W, cache, torch.float32, talk=talk)
        for r in range(len(lengths)):
            np.testing.assert_allclose(got[r], plain.talking_softmax_attention(rows_in[r], W, "", m), atol=3e-5, rtol=1e-4)


# ------------------------------------------------------------------------------------------------------ whole models
_MODELS = {}


def _model(name, tmp_path_factory, seed=21):
    key = (name, seed)
    if key not in _MODELS:
        cfg = bu.CONFIGS[name]()
        tensors = bu.random_weights(cfg, seed)
        folder = bu.write_model(str(tmp_path_factory.mktemp(f"bb_{name}_{seed}")), cfg, tensors)
        _MODELS[key] = (cfg, bu.as_float64(tensors), folder, {})
    return _MODELS[key]


def _want(model, tokens):
    cfg, W, _, memo = model
    key = tuple(tokens)
    if key not in memo:
        memo[key] = plain.forward(cfg, W, list(tokens))
    return memo[key]


def _tokens(cfg, n, seed):
    return [int(t) for t in np.random.default_rng(seed).integers(0, cfg["vocab"], n)]


def _engine(folder, dtype, **kw):
    from glassbox_b200.engine.engine import Engine
    args = dict(cache_tokens=512, page_size=16, max_batch_tokens=256, max_requests=4)
    args.update(kw)
    return Engine(folder, dtype, **args)


@pytest.mark.parametrize("name", ["odd", "plain"])
def test_every_layer_of_a_short_request(name, tmp_path_factory):
    """The summed residual streams after every layer, in float32, against the plain ones: the first layer that differs
    names itself. (A layer leaves its last branch to be folded into the streams by the next reader; the test folds it.)"""
    cfg, W, folder, _ = _model(name, tmp_path_factory)
    eng = _engine(folder, "float32", use_graphs=False)
    toks = _tokens(cfg, 29, 4)
    layers = []
    plain.forward(cfg, W, toks, layers)
    from glassbox_b200.engine.engine import StepEntry
    eng.add_request("r", [])
    seen, S, d = [], eng.config.residual_streams, cfg["width"]

    def tapped(layer):
        inner = layer.forward

        def forward(ctx, xs, *args, **kw):
            inner(ctx, xs, *args, **kw)
            y, mix, write = ctx.pending_fold
            x = xs[:len(toks)].view(len(toks), S, d).double()
            new = torch.einsum("st,nsd->ntd", mix.double(), x) + write.double()[None, :, None] * y[:len(toks)].double()[:, None, :]
            seen.append(new.sum(1).cpu().numpy())
        return forward
    for layer in eng.model.layers:
        layer.forward = tapped(layer)
    try:
        eng.step([StepEntry("r", toks, [len(toks) - 1])])
    finally:
        for layer in eng.model.layers:
            del layer.forward
    assert len(seen) == len(cfg["layers"])
    for i, (a, b) in enumerate(zip(seen, layers)):
        np.testing.assert_allclose(a, b, atol=3e-4, rtol=1e-4, err_msg=f"after layer {i}")


@pytest.mark.parametrize("name, dtype", [(n, "float32") for n in sorted(bu.CONFIGS)] + [("odd", "bfloat16"), ("even", "bfloat16")])
def test_whole_prompt_and_token_by_token(name, dtype, tmp_path_factory):
    model = _model(name, tmp_path_factory)
    cfg, _, folder, _ = model
    eng = _engine(folder, dtype)
    for n, seed in [(1, 1), (2, 2), (3, 6), (77, 3)]:                # the first tokens of a sequence; past several pages
        toks = _tokens(cfg, n, seed)
        want = _want(model, toks)
        got = zu.run_schedule(eng, {"r": toks}, [[("r", n)]])["r"]
        assert_logits_close(got, want, dtype, f"{name} whole {n}")
        got = zu.run_schedule(eng, {"r": toks}, [[("r", 1)] for _ in range(n)])["r"]
        assert_logits_close(got, want, dtype, f"{name} token by token {n}")


def test_sizes_that_fit_no_vector_width_run_in_bfloat16_too(tmp_path_factory):
    model = _model("ragged", tmp_path_factory)
    cfg, _, folder, _ = model
    eng = _engine(folder, "bfloat16")
    toks = _tokens(cfg, 41, 5)
    want = _want(model, toks)
    whole = zu.run_schedule(eng, {"r": toks}, [[("r", 41)]])["r"]
    cut = zu.run_schedule(eng, {"r": toks}, [[("r", 17)], [("r", 2)], [("r", 21)], [("r", 1)]])["r"]
    assert_logits_close(whole, want, "bfloat16", "ragged whole")
    assert_logits_close(cut, want, "bfloat16", "ragged cut")


@pytest.mark.parametrize("name", ["odd", "even", "ones"])
def test_portions_of_every_size(name, tmp_path_factory):
    model = _model(name, tmp_path_factory)
    cfg, _, folder, _ = model
    eng = _engine(folder, "float32")
    toks = _tokens(cfg, 83, 7)
    want = _want(model, toks)
    for sizes in ([2] * 41 + [1], [3, 2, 16, 1, 15, 17, 2, 2, 25], [16, 16, 16, 16, 16, 3], [31, 2, 33, 17], [1, 82]):
        assert sum(sizes) == len(toks)
        got = zu.run_schedule(eng, {"r": toks}, [[("r", k)] for k in sizes])["r"]
        assert_logits_close(got, want, "float32", f"{name} portions {sizes[:4]}...")


@pytest.mark.parametrize("name, dtype", [("odd", "float32"), ("even", "float32"), ("plain", "float32"), ("even", "bfloat16")])
def test_mixed_batches_equal_each_request_alone(name, dtype, tmp_path_factory):
    """Unequal requests side by side, portions beside single tokens, requests that sit out a step, more requests than
    slots over time and a pool that only holds what is live: slots and pages are freed and used again."""
    model = _model(name, tmp_path_factory)
    cfg, _, folder, _ = model
    eng = _engine(folder, dtype, cache_tokens=192, max_requests=3)
    reqs = {"a": _tokens(cfg, 70, 11), "b": _tokens(cfg, 9, 12), "c": _tokens(cfg, 33, 13), "d": _tokens(cfg, 50, 14),
            "e": _tokens(cfg, 1, 15), "f": _tokens(cfg, 18, 16)}
    schedule = [[("a", 30), ("b", 2)], [("b", 1), ("a", 2), ("c", 16)], [("a", 1), ("b", 1), ("c", 1)],
                [("c", 16), ("b", 5)],                              # b and c end: their slots and pages go back
                [("a", 1)], [("d", 20), ("a", 2)], [("e", 1), ("d", 1), ("a", 1)], [("d", 29), ("a", 1)],
                [("f", 2), ("a", 1)], [("f", 16), ("a", 25)]] + [[("a", 1)]] * 6
    want = {k: _want(model, v) for k, v in reqs.items()}
    got = zu.run_schedule(eng, reqs, schedule)
    for k in reqs:
        assert_logits_close(got[k], want[k], dtype, f"{name} mixed, request {k}")
    eng.cache.check_invariants()
    assert len(eng.cache.free_slots) == eng.cache.max_requests


def test_long_decoding_replays_recorded_steps(tmp_path_factory):
    """Two requests decode for more than two hundred steps: the steps run as recorded graphs, the states, the last inputs of
    every convolution and the pages carry from one replay to the next."""
    model = _model("even", tmp_path_factory)
    cfg, _, folder, _ = model
    eng = _engine(folder, "float32", cache_tokens=512, max_requests=2)
    a, b = _tokens(cfg, 250, 31), _tokens(cfg, 226, 32)
    schedule = [[("a", 20)], [("b", 3)]] + [[("a", 1), ("b", 1)]] * 216 + [[("a", 14), ("b", 7)]]
    got = zu.run_schedule(eng, {"a": a, "b": b}, schedule)
    assert eng.graph_replays > 150
    assert_logits_close(got["a"], _want(model, a), "float32", "long decoding a")
    assert_logits_close(got["b"], _want(model, b), "float32", "long decoding b")
    eng.cache.check_invariants()


def test_a_slot_and_its_pages_that_are_used_again(tmp_path_factory):
    model = _model("odd", tmp_path_factory)
    cfg, _, folder, _ = model
    eng = _engine(folder, "float32", max_requests=1, cache_tokens=64)
    for seed in (41, 42, 43):
        toks = _tokens(cfg, 40, seed)
        got = zu.run_schedule(eng, {"r": toks}, [[("r", 25)], [("r", 15)]])["r"]
        assert_logits_close(got, _want(model, toks), "float32", f"slot reuse {seed}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(dtype, tmp_path_factory):
    import glassbox_b200
    model = _model("even", tmp_path_factory, seed=5)
    cfg, W, folder, _ = model
    llm = glassbox_b200.load(folder, dtype, blocks=64, budget=32, max_seqs=3, prefix_cache=True)
    prompts = [_tokens(cfg, 37, 51), _tokens(cfg, 5, 52), _tokens(cfg, 70, 53), _tokens(cfg, 1, 54)]
    outs = llm.generate(prompts, max_tokens=10)
    for p, out in zip(prompts, outs):
        seq = list(p)
        assert len(out) == 10
        for i, tok in enumerate(out):
            logits = plain.forward(cfg, W, seq)[-1]
            best = int(np.argmax(logits))
            if dtype == "bfloat16" and tok != best:
                top2 = np.sort(logits)[-2:]
                assert logits[tok] >= top2[1] - 0.3 * logits.std(), f"token {i}: {tok} is not near the best"
                break                                                # rounding chose the runner-up: the texts part ways
            assert tok == best, f"{dtype} prompt of {len(p)}: token {i} is {tok}, plain says {best}"
            seq.append(tok)


def test_a_trace_replayed_from_the_command_line(tmp_path_factory, tmp_path):
    """``bin/trace_run`` as a user runs it: steps on standard input, logits in files; four live requests at most in a pool that
    holds only what is live, portions beside single tokens, requests that end and others that take their slots and pages."""
    import json
    import os
    import subprocess
    import sys
    from replay_util import TRACE_RUN, live_tokens_needed
    model = _model("odd", tmp_path_factory)
    cfg, _, folder, _ = model
    reqs = {"a": _tokens(cfg, 150, 61), "b": _tokens(cfg, 40, 62), "c": _tokens(cfg, 66, 63), "d": _tokens(cfg, 9, 64), "e": _tokens(cfg, 70, 65)}
    plan = [[("a", 64), ("b", 2)], [("a", 3), ("b", 1), ("c", 29)], [("a", 1), ("b", 16), ("c", 1), ("d", 2)],
            [("a", 16), ("b", 21), ("c", 36), ("d", 7)], [("a", 1), ("e", 64)], [("a", 64), ("e", 2)], [("a", 1), ("e", 4)]]
    at, steps = {k: 0 for k in reqs}, []
    for i, step in enumerate(plan):
        entries, end = [], []
        for rid, k in step:
            entries.append({"id": rid, "tokens": reqs[rid][at[rid]:at[rid] + k], "want": list(range(k))})
            at[rid] += k
            if at[rid] == len(reqs[rid]):
                end.append(rid)
        steps.append({"step": i, "entries": entries, "end": end})
    assert at == {k: len(v) for k, v in reqs.items()}
    out = str(tmp_path / "out")
    os.makedirs(out)
    proc = subprocess.run([sys.executable, TRACE_RUN, "--model", folder, "--dtype", "float32", "--out", out, "--max-tokens",
                           str(live_tokens_needed(steps))], input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True,
                          text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-3000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done ")] == [f"done {i}" for i in range(len(plan))]
    got = {k: [] for k in reqs}
    for i, step in enumerate(plan):
        rows = np.fromfile(os.path.join(out, f"{i}.f32"), dtype="<f4").reshape(-1, cfg["vocab"])
        row = 0
        for rid, k in step:
            got[rid].append(rows[row:row + k])
            row += k
        assert row == len(rows)
    for rid in reqs:
        assert_logits_close(np.concatenate(got[rid], 0), _want(model, reqs[rid]), "float32", f"replayed request {rid}")
