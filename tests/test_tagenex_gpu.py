"""Tagenex on the GPU against the plain float64 implementation (``tests/plain/tagenex_plain.py``): each mechanism's
kernel alone, then whole models under every way of cutting and batching their requests, through the engine's own step
function, cache manager, scheduler and entry point. Sizes are the tests' own (``tagenex_util.CONFIGS``)."""
import numpy as np
import pytest
import torch

import conftest
from plain import tagenex_plain as plain
import tagenex_util as tu
import zurerax_util as zu

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

# bfloat16 against float64: a handful of roundings per branch, each branch normed to unit size before it is added, so that
# a branch's rounding does not shrink with the branch; and where two router logits lie closer than the rounding of the
# router's input, bfloat16 picks another expert than float64 and that token's logits differ by a discrete amount. So the
# bound holds for nine rows in ten and for the median row. Faults in which key, value or expert a bfloat16 kernel reads are
# caught by the crafted tests below and by the float32 runs of the same code, which are held to 1e-4.
BF16_REL_MAX, BF16_REL_MEAN, BF16_ROWS_OFF = 0.25, 0.03, 0.1


def assert_logits_close(got, want, dtype, what=""):
    if dtype == "float32":
        return conftest.assert_logits_close(got, want, dtype, what)
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, f"{what}: shape {got.shape} != {want.shape}"
    assert np.isfinite(got).all(), f"{what}: not finite"
    diff, spread = np.abs(got - want), want.std()
    off = diff.max(1) > BF16_REL_MAX * spread
    assert off.sum() <= max(1, BF16_ROWS_OFF * len(off)), \
        f"{what}: {int(off.sum())} of {len(off)} rows differ by more than {BF16_REL_MAX} x spread {spread:.3e} (worst {diff.max():.3e})"
    assert np.median(diff.mean(1)) <= BF16_REL_MEAN * spread, \
        f"{what}: the median row's mean abs diff {np.median(diff.mean(1)):.3e} > {BF16_REL_MEAN} x spread {spread:.3e}"


def _i32(values):
    return torch.tensor(values, dtype=torch.int32, device=DEV)


def _f32(a):
    return torch.tensor(np.asarray(a, dtype=np.float32), device=DEV)


def _status():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


class _PagedRequests:
    """A paged cache for a few requests whose pages lie scattered and interleaved in the pool."""

    def __init__(self, lengths, G, D, V, page, dtype, seed=0):
        rng = np.random.default_rng(seed)
        self.page, self.G = page, G
        need = [-(-n // page) for n in lengths]
        order = rng.permutation(sum(need) + 3)
        self.tables, at = [], 0
        for k in need:
            self.tables.append([int(p) for p in order[at:at + k]])
            at += k
        self.pages = sum(need) + 3
        self.width = max(need)
        self.k = torch.zeros((self.pages, G, page, D), dtype=dtype, device=DEV)
        self.v = torch.zeros((self.pages, G, page, V), dtype=dtype, device=DEV)

    def row(self, seq):
        return self.tables[seq] + [-1] * (self.width - len(self.tables[seq]))

    def table(self, seqs):
        return _i32([self.row(s) for s in seqs])

    def slot(self, seq, pos):
        return self.tables[seq][pos // self.page] * self.page + pos % self.page

    def put(self, seq, pos, k=None, v=None):
        pg, off = self.tables[seq][pos // self.page], pos % self.page
        if k is not None:
            self.k[pg, :, off] = torch.as_tensor(k, dtype=self.k.dtype)
        if v is not None:
            self.v[pg, :, off] = torch.as_tensor(v, dtype=self.v.dtype)


def _mixer_by_identity(H, G, D, V, scale, window, rng):
    """A plain mixer whose projections pick the parts of a stacked row [q | k | v | gate logits] apart, with random
    per-head numbers; returns (config dict, float64 tensors)."""
    cols = (H + G) * D + G * V + H
    eye = np.eye(cols)
    m = {"heads": H, "kv_heads": G, "dim": D, "vdim": V, "scale": scale}
    if window:
        m["mask"] = {"size": window}
    W = {"q": eye[:H * D], "k": eye[H * D:(H + G) * D], "v": eye[(H + G) * D:(H + G) * D + G * V], "g": eye[(H + G) * D + G * V:],
         "o": np.eye(H * V), "q.norm": 1 + 0.3 * rng.standard_normal(D), "k.norm": 1 + 0.3 * rng.standard_normal(D),
         "r1": rng.uniform(0.1, 1.0, H), "r2": rng.uniform(0.05, 2.0, H), "sink": rng.standard_normal(H) * 1.5,
         "vmix": np.array(rng.uniform(0.2, 0.7))}
    return m, W


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


def _run_mixer_steps(kernels, how, steps, lengths, rows_in, m, W, cache, dtype, eps, first_values=None, keep_values=False):
    """Norm, value mixing and cache write, then attention with its gate, step by step; returns the outputs per request (and
    the float32 values each row kept, if asked for). ``how``: "rows", "decode" (single-token steps take the decode kernel,
    others the row kernel), "split" (single-token steps take the split-key tensor-core kernel, with another split count,
    block size and warp count at every step), "tiles" or "flash" (the tcgen05 kernel)."""
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    window, page = (m["mask"]["size"] if "mask" in m else None), cache.page
    gate_col = (H + G) * D + G * V
    status = _status()
    got = [np.zeros((n, H * V)) for n in lengths]
    kept = [np.zeros((n, G * V)) for n in lengths]
    at = [0] * len(lengths)
    common = dict(r1=_f32(W["r1"]), r2=_f32(W["r2"]), sink=_f32(W["sink"]), heads=H, kv_heads=G, dim=D, vdim=V, page_size=page,
                  scale=m["scale"], window=window, status=status)
    for step in steps:
        n, row_seq, positions, first, start = _step_meta(step, at)
        x, slots, vin = np.zeros((n, gate_col + H)), [-1] * n, np.zeros((n, G * V))
        row = 0
        for e in step:
            if e is None:
                row += 1
                continue
            r, k = e
            x[row:row + k] = rows_in[r][at[r]:at[r] + k]
            if first_values is not None:
                vin[row:row + k] = first_values[r][at[r]:at[r] + k]
            slots[row:row + k] = [cache.slot(r, at[r] + i) for i in range(k)]
            row += k
        proj = _f32(x)
        q = torch.zeros((n, H * D), dtype=dtype, device=DEV)
        out = torch.zeros((n, H * V), dtype=dtype, device=DEV)
        vout = torch.zeros((n, G * V), dtype=torch.float32, device=DEV)
        kernels.qk_norm_rope_write(proj[:, :gate_col], _f32(W["q.norm"]), _f32(W["k.norm"]), None, positions, _i32(slots), q, cache.k,
                                   cache.v, H, G, D, V, 0, eps, page, True, status,
                                   values_out=vout if first_values is None else None,
                                   values_in=_f32(vin) if first_values is not None else None,
                                   value_mix=_f32(W["vmix"]).reshape(()) if first_values is not None else None)
        tables = _i32([[-1] * cache.width if e is None else cache.row(e[0]) for e in step])
        gate = proj[:, gate_col:]
        single = all(e is None or e[1] == 1 for e in step)
        if how == "flash":
            kernels.attention_prefill_tc(q, out, cache.k, cache.v, tables, first, start, max(e[1] for e in step if e), H, G, D, page,
                                         m["scale"], window, status, sink_terms=(common["r1"], common["r2"], common["sink"], gate))
        elif how == "tiles":
            kernels.sink_attention_tiles(q, out, cache.k, cache.v, tables, first, start, max(e[1] for e in step if e), gate=gate, **common)
        elif how == "split" and single:
            plans = [(1, 0, 4), (3, 16, 4), (2, 16, 8), (2, 0, 8), (5, 0, 4)] if D == 64 else [(1, 0, 4), (3, 0, 4), (2, 0, 4)]
            splits, block_keys, warps = plans[sum(at) % len(plans)]
            part_acc = torch.full((n, H * warps * splits * D), float("nan"), device=DEV)
            part_ml = torch.full((n, H * warps * splits * 2), float("nan"), device=DEV)
            counters = torch.zeros(n * G, dtype=torch.int32, device=DEV)
            kernels.attention_decode_mma(q, out, cache.k, cache.v, tables, row_seq, positions, H, G, D, page, m["scale"], window,
                                         splits, part_acc, part_ml, counters, status, block_keys, warps,
                                         sink_terms=(common["r1"], common["r2"], common["sink"], gate))
            assert int(counters.abs().sum().item()) == 0
        elif how == "decode" and single and kernels.sink_attention_decode_supported(dtype, V):
            kernels.sink_attention_decode(q, out, cache.k, cache.v, tables, row_seq, positions, gate=gate, **common)
        else:
            kernels.sink_attention_rows(q, out, cache.k, cache.v, tables, row_seq, positions, gate=gate, **common)
        o, vo, row = out.float().cpu().numpy(), vout.cpu().numpy(), 0
        for e in step:
            if e is None:
                row += 1
                continue
            r, k = e
            got[r][at[r]:at[r] + k] = o[row:row + k]
            kept[r][at[r]:at[r] + k] = vo[row:row + k]
            row += k
            at[r] += k
    assert int(status.item()) == 0
    return (got, kept) if keep_values else got


# ---------------------------------------------------------------------------------------------- each mechanism alone
@pytest.mark.parametrize("n, d", [(1, 50), (5, 56), (70, 128), (3, 257)])
def test_branch_norm_joins_the_residual(n, d):
    """x += w * y / rms(y), with a bias added to y first and the new rows copied in the activation dtype."""
    from glassbox_b200 import kernels
    rng = np.random.default_rng(n * d)
    y, x, w, b = rng.standard_normal((n, d)) * 3, rng.standard_normal((n, d)), 1 + 0.2 * rng.standard_normal(d), rng.standard_normal(d)
    for bias in (None, b):
        for copy_dtype in (None, torch.bfloat16, torch.float32):
            xs, ys = _f32(x), _f32(y)
            copy = torch.zeros((n, d), dtype=copy_dtype, device=DEV) if copy_dtype else None
            kernels.rmsnorm_add(ys, _f32(w), xs, 1e-5, bias=_f32(bias) if bias is not None else None, copy=copy)
            want = x + plain.rms_unit(y + (bias if bias is not None else 0.0), w, 1e-5)
            np.testing.assert_allclose(xs.cpu().numpy(), want, atol=2e-5, rtol=1e-5)
            np.testing.assert_array_equal(ys.cpu().numpy(), y.astype(np.float32))          # the branch itself is left alone
            if copy is not None:
                assert torch.equal(copy, xs.to(copy_dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n, ff, limit", [(1, 1, 1.0), (7, 11, 0.75), (33, 64, 2.0), (4, 200, 7.0)])
def test_clamped_gated_unit(dtype, n, ff, limit):
    """Inputs far beyond the limit on both sides: the gate is cut from above only, the other branch on both sides."""
    from glassbox_b200 import kernels
    rng = np.random.default_rng(ff)
    gu, b = rng.standard_normal((n, 2 * ff)) * 2 * limit, rng.standard_normal(2 * ff)
    gu[0, 0], gu[0, ff] = -5 * limit, -5 * limit                # a gate far below -limit stays as it is
    for bias in (None, b):
        x = _f32(gu)
        act = torch.zeros((n, ff), dtype=dtype, device=DEV)
        kernels.clamped_glu(x, _f32(bias) if bias is not None else None, limit, plain.SLOPE, act)
        z = gu + (bias if bias is not None else 0.0)
        want = plain.gated_unit(z[:, :ff], z[:, ff:], limit)
        if dtype == torch.float32:
            np.testing.assert_allclose(act.cpu().numpy(), want, atol=1e-5, rtol=1e-5)
        else:
            np.testing.assert_allclose(act.float().cpu().numpy(), want, atol=1e-2 * max(1.0, limit * limit), rtol=1e-2)
    assert plain.gated_unit(np.array(-5.0), np.array(0.0), 1.0) < 0 and plain.gated_unit(np.array(9.0), np.array(9.0), 1.0) == \
        plain.gated_unit(np.array(1.0), np.array(1.0), 1.0)


@pytest.mark.parametrize("n, ff, d, limit", [(1, 64, 128, 2.0), (8, 48, 72, 0.75), (64, 256, 128, 7.0), (65, 64, 128, 1.0),
                                            (300, 136, 64, 1.5), (2048, 512, 256, 3.0)])
def test_clamped_gated_unit_in_a_products_epilogue(n, ff, d, limit):
    """The two products of a dense feed-forward's first half with the unit formed from their float32 sums, in the kernel for
    few rows (the weights streamed once) and in the tile kernel, with and without biases."""
    from glassbox_b200 import kernels
    rng = np.random.default_rng(n + ff)
    bf = lambda a: _f32(a).to(torch.bfloat16)
    h, w, b = bf(rng.standard_normal((n, d))), bf(rng.standard_normal((2 * ff, d)) * 2.0 * limit / np.sqrt(d)), rng.standard_normal(2 * ff)
    z = h.float().cpu().numpy().astype(np.float64) @ w.float().cpu().numpy().astype(np.float64).T
    ran = 0
    for bias in (None, b):
        zz = z + (_f32(bias).cpu().numpy().astype(np.float64) if bias is not None else 0.0)
        want = plain.gated_unit(zz[:, :ff], zz[:, ff:], limit)
        bias_dev = _f32(bias) if bias is not None else None
        if kernels.gemm_stream_supported(h, w) and ff % 16 == 0:
            act = torch.zeros((n, ff), dtype=torch.bfloat16, device=DEV)
            kernels.gemm_stream_unit(h, w, bias_dev, limit, plain.SLOPE, act)
            np.testing.assert_allclose(act.float().cpu().numpy(), want, atol=1e-2 * max(1.0, limit * limit), rtol=1e-2)
            ran += 1
        act = torch.zeros((n, ff), dtype=torch.bfloat16, device=DEV)
        if kernels.gemm_tc_supported(h, w, act):
            status = _status()
            kernels.gemm_tc_unit(h, w, bias_dev, limit, plain.SLOPE, act, status)
            assert int(status.item()) == 0
            np.testing.assert_allclose(act.float().cpu().numpy(), want, atol=1e-2 * max(1.0, limit * limit), rtol=1e-2)
            ran += 1
    assert ran >= 2


@pytest.mark.parametrize("E, top, d", [(6, 2, 56), (12, 3, 128), (5, 1, 33), (1, 1, 32), (8, 8, 40), (64, 5, 72)])
@pytest.mark.parametrize("n", [9, 300])                        # (300: the form that takes several rows per block)
def test_router_softmax_over_the_chosen(E, top, d, n):
    from glassbox_b200 import kernels
    rng = np.random.default_rng(E * 100 + top)
    h = _f32(rng.standard_normal((n, d))).to(torch.bfloat16)
    Wr, b = rng.standard_normal((E, d)) / np.sqrt(d) * 2, rng.standard_normal(E) * 0.7
    W = {"router": _f32(Wr).cpu().numpy().astype(np.float64), "router.b": _f32(b).cpu().numpy().astype(np.float64)}
    order, weight = plain.route(h.float().cpu().numpy().astype(np.float64), W, "", {"router": {"top": top}})
    choice = torch.zeros((n, top), dtype=torch.int32, device=DEV)
    wgt = torch.zeros((n, top), dtype=torch.float32, device=DEV)
    for x in (h, h.float()):
        kernels.moe_route(x, _f32(Wr), None, None, _i32(list(range(n))), top, 1, 1, 1.0, choice, wgt, None, router_bias=_f32(b),
                          softmax_chosen=True)
        c, w = choice.cpu().numpy(), wgt.cpu().numpy()
        np.testing.assert_allclose(w.sum(1), 1.0, atol=1e-5)
        for r in range(n):
            assert sorted(c[r]) == sorted(order[r]), f"row {r}"
            got = dict(zip(c[r].tolist(), w[r].tolist()))
            for e, a in zip(order[r], weight[r]):
                assert abs(got[int(e)] - a) < 2e-5


def test_router_on_crafted_logits():
    """Logits set by hand through a one-hot input: equal logits go to the lowest index; the bias alone can decide; a
    logit far above the others takes nearly all the weight but the others keep theirs (no renormalising tricks); padding
    rows (position -1) are left alone."""
    from glassbox_b200 import kernels
    E, d, top = 6, 8, 3
    Wr = np.zeros((E, d))
    Wr[:, 0] = [1.0, 3.0, 3.0, 2.0, 3.0, 0.0]                   # three equal largest: 1, 2, 4 win over 3
    Wr[:, 1] = [0.0, 0.0, 0.0, 0.0, 0.0, 0.0]                   # all equal before the bias
    Wr[:, 2] = [9.0, 0.0, 1.0, 0.0, 0.5, 0.0]
    b = np.array([0.0, 0.0, 0.0, 0.0, 0.0, 0.5])
    h = np.zeros((4, d)); h[0, 0] = h[1, 1] = h[2, 2] = 1.0; h[3, 0] = 1.0
    choice = torch.full((4, top), -7, dtype=torch.int32, device=DEV)
    wgt = torch.full((4, top), -7.0, dtype=torch.float32, device=DEV)
    kernels.moe_route(_f32(h), _f32(Wr), None, None, _i32([0, 1, 2, -1]), top, 1, 1, 1.0, choice, wgt, None, router_bias=_f32(b),
                      softmax_chosen=True)
    c, w = choice.cpu().numpy(), wgt.cpu().numpy()
    assert sorted(c[0]) == [1, 2, 4] and np.allclose(w[0], 1 / 3, atol=1e-6)
    assert sorted(c[1]) == [0, 1, 5]                             # 5 by its bias, then the lowest indices among equals
    got = dict(zip(c[1].tolist(), w[1].tolist()))
    z = np.exp([0.5, 0.0, 0.0]); z /= z.sum()
    assert abs(got[5] - z[0]) < 1e-6 and abs(got[0] - z[1]) < 1e-6
    assert sorted(c[2]) == [0, 2, 4]
    got = dict(zip(c[2].tolist(), w[2].tolist()))
    z = np.exp(np.array([9.0, 1.0, 0.5]) - 9.0); z /= z.sum()
    np.testing.assert_allclose([got[0], got[2], got[4]], z, atol=1e-6)
    assert (c[3] == -7).all() or (w[3] == 0).all()               # a padding row takes part in nothing


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("E, top, ff, d, limit", [(6, 2, 24, 56, 0.75), (4, 3, 11, 50, 2.5), (8, 2, 64, 128, 1.0), (1, 1, 8, 32, 1.0)])
def test_gated_experts_and_their_sum(dtype, E, top, ff, d, limit):
    """The routed feed-forward as the engine runs it for a few rows, against the plain one."""
    from glassbox_b200 import kernels
    rng = np.random.default_rng(E + ff)
    n = 7
    bf = lambda a: _f32(a).to(torch.bfloat16).float().cpu().numpy().astype(np.float64)
    h = bf(rng.standard_normal((n, d)))
    W = {"router": bf(rng.standard_normal((E, d)) * 2 / np.sqrt(d)), "router.b": bf(rng.standard_normal(E) * 0.7)}
    for e in range(E):
        W[f"e{e}.gate"], W[f"e{e}.up"] = bf(rng.standard_normal((ff, d)) * 1.5 / np.sqrt(d)), bf(rng.standard_normal((ff, d)) * 1.5 / np.sqrt(d))
        W[f"e{e}.down"] = bf(rng.standard_normal((d, ff)) / np.sqrt(ff))
    mlp = {"router": {"experts": E, "top": top}, "expert": {"ff": ff, "limit": limit}}
    want = plain.moe_ff(h, W, "", mlp)
    # unit f of an expert reads rows 2f (gate) and 2f + 1 (up) of the stacked parameter
    up = np.stack([np.stack([W[f"e{e}.gate"], W[f"e{e}.up"]], 1).reshape(2 * ff, d) for e in range(E)]).reshape(E * 2 * ff, d)
    down = np.concatenate([W[f"e{e}.down"] for e in range(E)])
    positions = _i32(list(range(n)))
    choice = torch.zeros((n, top), dtype=torch.int32, device=DEV)
    wgt = torch.zeros((n, top), dtype=torch.float32, device=DEV)
    hd = _f32(h).to(dtype)
    kernels.moe_route(hd, _f32(W["router"]), None, None, positions, top, 1, 1, 1.0, choice, wgt, None, router_bias=_f32(W["router.b"]),
                      softmax_chosen=True)
    act = torch.zeros((n, top * ff), dtype=torch.float32, device=DEV)
    pair = torch.zeros((n, top * d), dtype=torch.float32, device=DEV)
    kernels.moe_expert_halves(hd, _f32(up).to(dtype), _f32(down).to(dtype), E, choice, positions, act, pair, unit=(limit, plain.SLOPE))
    out = _f32(rng.standard_normal((n, d)))
    before = out.cpu().numpy().astype(np.float64)
    kernels.moe_combine(pair, wgt, None, None, positions, out, True)
    np.testing.assert_allclose(out.cpu().numpy() - before, want, atol=3e-5 if dtype == torch.float32 else 3e-2 * max(1.0, np.abs(want).max()),
                               rtol=1e-5 if dtype == torch.float32 else 2e-2)


@pytest.mark.parametrize("E, top, ff, d, n, limit", [(8, 2, 64, 128, 300, 1.0), (12, 4, 40, 72, 77, 0.5), (3, 3, 136, 64, 129, 3.0)])
def test_grouped_gated_experts_equal_the_row_form(E, top, ff, d, n, limit):
    """Many rows in bfloat16: the pairs sorted by expert and multiplied on the tensor cores give what the row form gives."""
    from glassbox_b200 import kernels
    if not kernels.moe_grouped_supported(torch.bfloat16, d, ff):
        pytest.skip("no grouped kernel for these sizes")
    rng = np.random.default_rng(n)
    h = _f32(rng.standard_normal((n, d))).to(torch.bfloat16)
    up = _f32(rng.standard_normal((E * 2 * ff, d)) * 1.5 / np.sqrt(d)).to(torch.bfloat16)
    down = _f32(rng.standard_normal((E * d, ff)) / np.sqrt(ff)).to(torch.bfloat16)
    choice = _i32([list(rng.permutation(E)[:top]) for _ in range(n)])
    pos = list(range(n)); pos[5] = pos[n - 1] = -1               # padding rows take part in nothing
    positions = _i32(pos)
    act32 = torch.zeros((n, top * ff), dtype=torch.float32, device=DEV)
    pair_rows = torch.zeros((n, top * d), dtype=torch.float32, device=DEV)
    kernels.moe_expert_halves(h, up, down, E, choice, positions, act32, pair_rows, unit=(limit, plain.SLOPE))
    tables = torch.zeros(2 * (E + 1) + n * top, dtype=torch.int32, device=DEV)
    act = torch.zeros((n, top * ff), dtype=torch.bfloat16, device=DEV)
    pair = torch.zeros((n, top * d), dtype=torch.float32, device=DEV)
    kernels.moe_experts_grouped(h, up, down, E, choice, positions, tables, act, pair, unit=(limit, plain.SLOPE))
    live = [r for r in range(n) if pos[r] >= 0]
    a, b = pair[live].cpu().numpy(), pair_rows[live].cpu().numpy()
    assert np.abs(a - b).max() <= 0.03 * max(1.0, np.abs(b).max())


# ------------------------------------------------------------------------------------ the attention kernels alone
def _plain_mixer(rows_in, m, W, eps, first_values=None):
    out, kept = plain.attention(rows_in, W, "", dict(m, v_mix=first_values is not None), eps,
                                None if first_values is None else first_values.reshape(len(rows_in), m["kv_heads"], m["vdim"]))
    return out, kept.reshape(len(rows_in), -1)


def _cuts(lengths, how, rng):
    """Steps that bring every request in: prompt portions of changing sizes side by side, then single tokens ("decode":
    and "split": the last third of each request token by token, all requests in one step)."""
    at, steps = [0] * len(lengths), []
    stop = [n - (n // 3 if how in ("decode", "split") else 0) for n in lengths]
    while any(a < s for a, s in zip(at, stop)):
        step = []
        for r, n in enumerate(lengths):
            if at[r] < stop[r] and rng.random() < 0.8:
                k = min(int(rng.choice([1, 2, 3, 15, 16, 17, 40, 64, 70])), stop[r] - at[r])
                step.append((r, k))
                at[r] += k
        if step:
            steps.append(step)
    while any(a < n for a, n in zip(at, lengths)):
        step = [(r, 1) if at[r] < lengths[r] else None for r in range(len(lengths))]     # finished requests: padding rows
        for r in range(len(lengths)):
            at[r] += at[r] < lengths[r]
        steps.append(step)
    return steps


@pytest.mark.parametrize("how, dtype", [("rows", torch.float32), ("decode", torch.float32), ("rows", torch.bfloat16),
                                        ("decode", torch.bfloat16), ("tiles", torch.bfloat16), ("split", torch.bfloat16),
                                        ("flash", torch.bfloat16)])
@pytest.mark.parametrize("H, G, D, V, window", [(6, 2, 20, 12, 7), (4, 4, 16, 32, 19), (8, 2, 64, 64, 33), (4, 2, 128, 64, 48),
                                                (2, 1, 32, 128, None), (1, 1, 8, 8, 1), (3, 1, 10, 7, 5), (4, 1, 64, 32, 100),
                                                (16, 1, 16, 16, 20), (6, 3, 128, 128, None), (5, 5, 32, 32, 17), (12, 2, 64, 64, 60)])
def test_sink_attention_kernels(how, dtype, H, G, D, V, window):
    """Norm, cache write and attention for three requests of unequal length whose pages lie interleaved, brought in by
    portions and single tokens, against the plain mixer over each whole request."""
    from glassbox_b200 import kernels
    if how == "tiles" and not kernels.sink_attention_tiles_supported(dtype, D, V):
        pytest.skip("no tile kernel for these head sizes")
    if how == "split" and not (D == V and kernels.attention_decode_mma_supported(dtype, H, G, D, 16)):
        pytest.skip("no split-key kernel for these head sizes")
    if how == "flash" and not (D == V and kernels.lib().gb_attention_prefill_tc_supported(H, G, D, 16)):
        pytest.skip("no tcgen05 flash kernel for these head sizes")
    rng = np.random.default_rng(H * 1000 + D)
    m, W = _mixer_by_identity(H, G, D, V, 1.3 * D ** -0.5, window, rng)
    lengths = [131, 1, 50]
    cols = (H + G) * D + G * V + H
    rows_in = [rng.standard_normal((n, cols)) for n in lengths]
    if dtype == torch.bfloat16:
        rows_in = [_f32(r).cpu().numpy().astype(np.float64) for r in rows_in]
    cache = _PagedRequests(lengths, G, D, V, 16, dtype, seed=D)
    got = _run_mixer_steps(kernels, how, _cuts(lengths, how, rng), lengths, rows_in, m, W, cache, dtype, 1e-5)
    for r, n in enumerate(lengths):
        want, _ = _plain_mixer(rows_in[r], m, W, 1e-5)
        if dtype == torch.float32:
            np.testing.assert_allclose(got[r], want, atol=2e-5, rtol=1e-4, err_msg=f"request {r}")
        else:
            assert np.abs(got[r] - want).max() <= 0.04 * max(1.0, np.abs(want).max()), f"request {r}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_values_are_mixed_before_they_are_cached(dtype):
    """A source layer hands its values on in float32; a mixing layer stores (1 - lambda) v + lambda v_source and attends
    over that, in prompts and for single tokens."""
    from glassbox_b200 import kernels
    rng = np.random.default_rng(5)
    H, G, D, V = 4, 2, 16, 32
    m, W = _mixer_by_identity(H, G, D, V, 0.3, 9, rng)
    lengths = [37, 20]
    cols = (H + G) * D + G * V + H
    rows_in = [_f32(rng.standard_normal((n, cols))).cpu().numpy().astype(np.float64) for n in lengths]
    steps = [[(0, 17), (1, 2)], [(0, 1), (1, 1)], [(1, 16), (0, 2)], [(0, 17), (1, 1)]]
    cache = _PagedRequests(lengths, G, D, V, 16, dtype, seed=1)
    _, source = _run_mixer_steps(kernels, "rows", steps, lengths, rows_in, m, W, cache, dtype, 1e-5, keep_values=True)
    for r in range(2):                               # the source's values leave as float32, not as the cache's rounding
        np.testing.assert_allclose(source[r], rows_in[r][:, (H + G) * D:(H + G) * D + G * V], rtol=1e-6)
    other = [rng.standard_normal((n, G * V)) for n in lengths]
    other = [_f32(o).cpu().numpy().astype(np.float64) for o in other]
    cache = _PagedRequests(lengths, G, D, V, 16, dtype, seed=2)
    got = _run_mixer_steps(kernels, "decode", steps, lengths, rows_in, m, W, cache, dtype, 1e-5, first_values=other)
    lam = float(_f32(W["vmix"]).cpu())
    for r, n in enumerate(lengths):
        want, kept = _plain_mixer(rows_in[r], m, dict(W, vmix=np.array(lam)), 1e-5, first_values=other[r])
        tol = 2e-5 if dtype == torch.float32 else 0.03
        assert np.abs(got[r] - want).max() <= tol * max(1.0, np.abs(want).max())
        stored = np.stack([cache.v[cache.tables[r][p // 16], :, p % 16].float().cpu().numpy().reshape(-1) for p in range(n)])
        assert np.abs(stored - kept).max() <= (1e-6 if dtype == torch.float32 else 0.01) * max(1.0, np.abs(kept).max())


def _marked_rows(T, H, G, D, V, marked, rng):
    """Rows [q | k | v | gate logits] in which every query points along the first axis and every key is orthogonal to it,
    but the keys at the ``marked`` positions, which point along it too: a query gives a marked key the score D * scale and
    every other key about nothing, so that whether a marked key is seen decides the output. Values are far apart."""
    q = np.zeros((T, H, D)); q[:, :, 0] = 1.0
    q += 0.01 * rng.standard_normal((T, H, D))
    k = rng.standard_normal((T, G, D)); k[:, :, 0] = 0.0
    for j in marked:
        k[j] = 0.0
        k[j, :, 0] = 1.0
    v = rng.standard_normal((T, G, V))
    for j in marked:
        v[j] += 6.0 * np.sign(rng.standard_normal((G, V)))
    gate = rng.standard_normal((T, H))
    return np.concatenate([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1), gate], 1)


@pytest.mark.parametrize("how, dtype", [("rows", torch.float32), ("decode", torch.float32), ("decode", torch.bfloat16),
                                        ("tiles", torch.bfloat16), ("split", torch.bfloat16), ("flash", torch.bfloat16)])
@pytest.mark.parametrize("window", [1, 2, 16, 19, 64, 65, 128, 129, None])
def test_a_marked_key_decides_at_the_windows_edge(how, dtype, window):
    """One key whose score stands out, placed at page borders and elsewhere; queries that see it as the oldest key of
    their window and queries one token later, which must not; without a window, a marked key hundreds of tokens back. The
    sink is large enough to take most of the weight where no marked key is visible, so that leaving it out shows too."""
    from glassbox_b200 import kernels
    rng = np.random.default_rng(window or 0)
    H, G, D, V, T = 4, 2, 32, 32, 330
    if how == "flash":                      # (built for this head size; its tiles are 128 rows by 128 keys)
        D = V = 64
    marked = [0, 15, 16, 31, 47, 48, 100, 128, 200]
    m, W = _mixer_by_identity(H, G, D, V, 0.5, window, rng)
    W["q.norm"], W["k.norm"] = np.ones(D), np.ones(D)
    W["sink"] = np.full(H, 4.0)
    rows = _f32(_marked_rows(T, H, G, D, V, marked, rng)).cpu().numpy().astype(np.float64)
    want, _ = _plain_mixer(rows, m, W, 1e-6)
    # the plain output itself tells the two sides of an edge apart: sure that the test can fail
    if window is not None and window > 1:
        i = 200 + window - 1                     # the last marked key is the oldest that row i sees; row i + 1 sees none
        gate = plain.logistic(rows[:, -H:])
        inside, outside = (np.abs(want[r].reshape(H, V) / gate[r][:, None]).max() for r in (i, i + 1))
        assert inside > 3.0 and outside < 2.0
    cut = 180 if how in ("decode", "split") else T
    if how in ("tiles", "flash"):
        steps = [[(0, 70)], [(0, 2)], [(0, 58)], [(0, 64)], [(0, 136)]]
    else:
        steps = [[(0, cut)]] if cut < T else [[(0, 33)], [(0, 150)], [(0, 147)]]
    steps += [[(0, 1)] for _ in range(T - cut)]
    cache = _PagedRequests([T], G, D, V, 16, dtype, seed=3)
    got = _run_mixer_steps(kernels, how, steps, [T], [rows], m, W, cache, dtype, 1e-6)[0]
    tol = 3e-5 if dtype == torch.float32 else 0.03
    worst = np.abs(got - want).max(1)
    assert worst.max() <= tol * max(1.0, np.abs(want).max()), f"row {int(worst.argmax())} differs by {worst.max():.3e}"


def test_sink_and_bias_are_each_optional_and_each_counts():
    """Equal scores by construction (scale 0): the weights are then known in closed form. Without bias and sink the output is
    the mean of the visible values; the sink adds exp(sink) to the denominator, once, unscaled; the bias weighs a key at
    distance k by (1 + r2 k)^(-r1)."""
    from glassbox_b200 import kernels
    H, G, D, V, T, window = 2, 1, 16, 32, 40, 12
    rng = np.random.default_rng(9)
    rows = rng.standard_normal((T, (H + G) * D + G * V + H))
    v = rows[:, (H + G) * D:(H + G) * D + G * V]
    r1, r2, sink = np.array([1.0, 0.5]), np.array([1.0, 3.0]), np.array([np.log(3.0), -1.0])
    for use_bias, use_sink, how in [(False, False, "rows"), (True, False, "rows"), (False, True, "decode"), (True, True, "decode"),
                                    (True, True, "rows")]:
        status = _status()
        cache = _PagedRequests([T], G, D, V, 16, torch.float32)
        q = torch.zeros((T, H * D), dtype=torch.float32, device=DEV)
        kernels.qk_norm_rope_write(_f32(rows[:, :(H + G) * D + G * V]), None, None, None, _i32(list(range(T))),
                                   _i32([cache.slot(0, p) for p in range(T)]), q, cache.k, cache.v, H, G, D, V, 0, 0.0, 16, True, status)
        out = torch.zeros((T, H * V), dtype=torch.float32, device=DEV)
        fn = kernels.sink_attention_decode if how == "decode" else kernels.sink_attention_rows
        fn(q, out, cache.k, cache.v, cache.table([0] * T) if how == "decode" else cache.table([0]),
           _i32(list(range(T)) if how == "decode" else [0] * T), _i32(list(range(T))), r1=_f32(r1) if use_bias else None,
           r2=_f32(r2) if use_bias else None, sink=_f32(sink) if use_sink else None, gate=None, heads=H, kv_heads=G, dim=D, vdim=V,
           page_size=16, scale=0.0, window=window, status=status)
        assert int(status.item()) == 0
        got = out.cpu().numpy().reshape(T, H, V)
        for i in (0, 1, 11, 12, 30):
            js = np.arange(max(0, i - window + 1), i + 1)
            for h in range(H):
                w = (1.0 + r2[h] * (i - js)) ** (-r1[h]) if use_bias else np.ones(len(js))
                den = w.sum() + (np.exp(sink[h]) if use_sink else 0.0)
                np.testing.assert_allclose(got[i, h], (w[:, None] * v[js]).sum(0) / den, atol=2e-5, rtol=1e-4)


# ------------------------------------------------------------------------------------------- whole models
_MODELS = {}


def _model(name, tmp_path_factory, seed=21):
    key = (name, seed)
    if key not in _MODELS:
        cfg = tu.CONFIGS[name]()
        tensors = tu.random_weights(cfg, seed)
        folder = tu.write_model(str(tmp_path_factory.mktemp(f"tx_{name}_{seed}")), cfg, tensors)
        _MODELS[key] = (cfg, tu.as_float64(tensors), folder, {})
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


def test_every_layer_of_a_short_request(tmp_path_factory):
    """The residual stream after every layer, in float32, against the plain one: the first layer that differs names itself."""
    model = _model("odd", tmp_path_factory)
    cfg, W, folder, _ = model
    eng = _engine(folder, "float32")
    toks = _tokens(cfg, 29, 4)
    _, layers = plain.forward(cfg, W, toks, keep_layers=True)
    from glassbox_b200.engine.engine import StepEntry
    eng.add_request("r", [])
    seen = []

    def tapped(layer):
        inner = layer.forward

        def forward(ctx, x, *args, **kw):
            inner(ctx, x, *args, **kw)
            seen.append(x[:len(toks)].float().cpu().numpy().copy())
        return forward
    for layer in eng.model.layers:
        layer.forward = tapped(layer)
    try:
        eng.step([StepEntry("r", toks, [len(toks) - 1])])
    finally:
        for layer in eng.model.layers:
            del layer.forward
    eng.free_request("r")
    assert len(seen) == len(cfg["layers"])
    for i, (a, b) in enumerate(zip(seen, layers)):
        np.testing.assert_allclose(a, b, atol=2e-4, rtol=1e-4, err_msg=f"after layer {i}")


@pytest.mark.parametrize("name, dtype", [(n, "float32") for n in sorted(tu.CONFIGS)] + [("odd", "bfloat16"), ("even", "bfloat16")])
def test_whole_prompt_and_token_by_token(name, dtype, tmp_path_factory):
    model = _model(name, tmp_path_factory)
    cfg, _, folder, _ = model
    eng = _engine(folder, dtype)
    for n, seed in [(1, 1), (2, 2), (3, 6), (77, 3)]:                # the first tokens of a sequence; past every window and page
        toks = _tokens(cfg, n, seed)
        want = _want(model, toks)
        got = zu.run_schedule(eng, {"r": toks}, [[("r", n)]])["r"]
        assert_logits_close(got, want, dtype, f"{name} whole {n}")
        got = zu.run_schedule(eng, {"r": toks}, [[("r", 1)] for _ in range(n)])["r"]
        assert_logits_close(got, want, dtype, f"{name} token by token {n}")


def test_sizes_that_fit_no_vector_width_run_in_bfloat16_too(tmp_path_factory):
    """Odd row lengths in bfloat16: rows that start on two-byte boundaries only. Every kernel must take the shapes, read no
    neighbour's numbers, and cutting the prompt must change nothing beyond rounding."""
    model = _model("ragged", tmp_path_factory)
    cfg, _, folder, _ = model
    eng = _engine(folder, "bfloat16")
    toks = _tokens(cfg, 41, 5)
    want = _want(model, toks)
    whole = zu.run_schedule(eng, {"r": toks}, [[("r", 41)]])["r"]
    cut = zu.run_schedule(eng, {"r": toks}, [[("r", 17)], [("r", 2)], [("r", 21)], [("r", 1)]])["r"]
    assert np.isfinite(whole).all()
    assert np.median(np.abs(whole - want).mean(1)) <= 0.06 * want.std()
    assert np.median(np.abs(whole - cut).mean(1)) <= 0.04 * want.std()


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


def test_windows_pass_over_decoded_tokens_in_a_pool_of_few_pages(tmp_path_factory):
    """Two requests decode far past every window of the model in a pool that could not hold one of them whole if no page
    ever came back: pages behind the windows are freed and used again while the requests live, and the decode steps run
    as recorded graphs."""
    model = _model("even", tmp_path_factory)
    cfg, _, folder, _ = model
    eng = _engine(folder, "float32", cache_tokens=448, max_requests=2)
    a, b = _tokens(cfg, 260, 31), _tokens(cfg, 236, 32)
    schedule = [[("a", 20)], [("b", 3)]] + [[("a", 1), ("b", 1)]] * 226 + [[("a", 14), ("b", 7)]]
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
    outs = llm.generate(prompts, max_tokens=12)
    for p, out in zip(prompts, outs):
        seq = list(p)
        assert len(out) == 12
        for i, tok in enumerate(out):
            logits = plain.forward(cfg, W, seq)[-1]
            best = int(np.argmax(logits))
            if dtype == "bfloat16" and tok != best:
                top2 = np.sort(logits)[-2:]
                assert logits[tok] >= top2[1] - 0.3 * logits.std(), f"token {i}: {tok} is not near the best"
                break                                                # rounding chose the runner-up: the texts part ways
            assert tok == best, f"{dtype} prompt of {len(p)}: token {i} is {tok}, plain says {best}"
            seq.append(tok)
