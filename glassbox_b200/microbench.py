"""Times single kernels on SmolLM2 shapes with CUDA events, inside a CUDA graph (no launch overhead),
over operands that rotate through more memory than L2 holds.

    python -m glassbox_b200.microbench gemm_stream [135m|360m|1.7b ...]   weight-streaming GEMM, 1..64 rows
    python -m glassbox_b200.microbench gemm_tc                           tcgen05 GEMM against torch.matmul
    python -m glassbox_b200.microbench attention_decode [batch ...]      paged decode attention at context 4096
    python -m glassbox_b200.microbench attention_splits HEADS KV_HEADS BATCH [CONTEXT]
                                                                         the large-batch decode attention at 1 to 6 splits
    python -m glassbox_b200.microbench attention_prefill                 flash attention, one 2048-token prompt
    python -m glassbox_b200.microbench float32                           the 32-bit path's kernels: FMA GEMM, decode and rows attention
    python -m glassbox_b200.microbench small                             embedding, RMSNorm, rotation + cache write, SwiGLU, sampling
    python -m glassbox_b200.microbench decode_program [batch ...]        a decode step as a kernel chain and as a persistent kernel
    python -m glassbox_b200.microbench layer_gemms [rows ...]            the four products of a decode layer as the layer runs them
    python -m glassbox_b200.microbench latent_attention                  attention over a latent cache (prompt and decoding) beside
                                                                         grouped-query attention of like size
    python -m glassbox_b200.microbench delta_rule                        the delta-rule recurrence over a prompt and for single tokens
    python -m glassbox_b200.microbench lonorax                           Lonorax's kernels, each beside its like kernel: sigmoid attention
                                                                         (window 1024) beside grouped-query attention with the same
                                                                         window; the grouped experts' products beside a dense product of
                                                                         as many multiply-adds; minGRU beside the delta rule; the streams'
                                                                         row kernel beside RMSNorm
    python -m glassbox_b200.microbench tagenex                           Tagenex's kernels, each beside its like kernel: sink attention
                                                                         with a distance bias and a gate (window 1024) beside
                                                                         grouped-query attention with the same window; q/k norm + value
                                                                         mixing + cache write beside rotation + cache write; the branch
                                                                         norm into the residual beside RMSNorm; the clamped gated unit in
                                                                         a product's epilogue beside SwiGLU in the same product; the
                                                                         routed clamped experts beside a dense product of as many
                                                                         multiply-adds; the router
    python -m glassbox_b200.microbench babotar                           Babotar's kernels, each beside its like kernel: talking-heads
                                                                         attention, lightning attention and the delta rule with one decay
                                                                         per head, the input convolution, the GELU unit in the products

Prints one line per case: microseconds and GB/s or TFLOP/s of the algorithmic bytes or flops. With ``--once`` after
the case's name every kernel is launched exactly once and nothing is timed: the form in which a profiler captures one
launch of each kernel.
"""
from __future__ import annotations

import sys

import torch

from . import kernels

DEV = "cuda:0"
L2_BYTES = 126e6

#: (name, output rows N, K, gated) of the per-layer matrices and the head
FAMILIES = {
    "135m": [("qkv", 960, 576, False), ("o", 576, 576, False), ("gate_up", 1536, 576, True), ("down", 576, 1536, False),
             ("head", 49152, 576, False)],
    "360m": [("qkv", 1600, 960, False), ("o", 960, 960, False), ("gate_up", 2560, 960, True), ("down", 960, 2560, False),
             ("head", 49152, 960, False)],
    "1.7b": [("qkv", 6144, 2048, False), ("o", 2048, 2048, False), ("gate_up", 8192, 2048, True),
             ("down", 2048, 8192, False), ("head", 49152, 2048, False)],
}


ONCE = False


def graph_time(fn, reps: int = 12, outer: int = 5) -> float:
    """Mean microseconds of one ``fn()`` among ``reps`` captured in a graph that is replayed ``outer`` times."""
    fn()
    torch.cuda.synchronize()
    if ONCE:
        return float("nan")
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(reps):
            fn()
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(outer):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (reps * outer)


def _rotating(rows: int, k: int):
    """Enough copies of a [rows, k] bfloat16 matrix that consecutive calls never find theirs in L2."""
    n = max(2, min(12, int(3 * L2_BYTES / (rows * k * 2)) + 1))
    return [(torch.randn(rows, k, device=DEV) * 0.05).bfloat16() for _ in range(n)]


def bench_gemm_stream(families) -> None:
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for fam in families or list(FAMILIES):
        for name, n, k, gated in FAMILIES[fam]:
            rows = 2 * n if gated else n
            ws = _rotating(rows, k)
            for m in (1, 8, 16, 32, 64):
                a = torch.randn(m, k, device=DEV).bfloat16()
                c = torch.empty(m, n, device=DEV, dtype=torch.bfloat16 if gated else torch.float32)
                turn = [0]

                def stream():
                    kernels.gemm_stream(a, ws[turn[0] % len(ws)], c, gated=gated)
                    turn[0] += 1

                def tiles():
                    w = ws[turn[0] % len(ws)]
                    kernels.gemm_tc_gated(a, w, c, status) if gated else kernels.gemm_tc(a, w, c, False, status)
                    turn[0] += 1

                t = graph_time(stream)
                line = f"{fam} {name:8s} {rows:6d} x {k:5d} rows {m:3d}: stream {t:7.1f} us {rows * k * 2 / t / 1e3:6.0f} GB/s"
                if m >= 16 and kernels.gemm_tc_supported(a, ws[0], c):
                    line += f" | tcgen05 {graph_time(tiles):7.1f} us"
                print(line, flush=True)
    kernels.check_status(status)


def bench_gemm_tc() -> None:
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for name, m, n, k in [("135m qkv", 2048, 960, 576), ("135m o", 2048, 576, 576), ("135m gate_up", 2048, 3072, 576),
                          ("135m down", 2048, 576, 1536), ("360m qkv", 2048, 1600, 960), ("360m o", 2048, 960, 960),
                          ("360m gate_up", 2048, 5120, 960), ("360m down", 2048, 960, 2560),
                          ("1.7b qkv", 2048, 6144, 2048), ("1.7b gate_up", 2048, 16384, 2048),
                          ("1.7b down", 2048, 2048, 8192), ("square", 8192, 8192, 8192)]:
        a = torch.randn(m, k, device=DEV).bfloat16()
        w = torch.randn(n, k, device=DEV).bfloat16()
        c = torch.empty(m, n, device=DEV).bfloat16()
        t = graph_time(lambda: kernels.gemm_tc(a, w, c, False, status), reps=6)
        t2 = graph_time(lambda: torch.matmul(a, w.T, out=c), reps=6)
        fl = 2.0 * m * n * k
        print(f"{name:13s} {m} x {n} x {k}: tcgen05 {t:8.1f} us {fl / t / 1e6:7.1f} TFLOP/s | torch.matmul {t2:8.1f} us "
              f"{fl / t2 / 1e6:7.1f} TFLOP/s", flush=True)
    kernels.check_status(status)


def bench_attention_decode(batches, nh: int = 9, nkv: int = 3, ctx: int = 4096, sweep: bool = False) -> None:
    """The planner's variant for each batch; with ``sweep`` the four-warp, 16-key variant at 1 to 6 splits as well."""
    hd, ps = 64, 16
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for m in batches or (1, 8, 64):
        per = ctx // ps
        kc = torch.randn(m * per + 4, nkv, ps, hd, device=DEV).bfloat16()
        vc = torch.randn_like(kc)
        tables = torch.arange(m * per, dtype=torch.int32, device=DEV).view(m, per).contiguous()
        row_seq = torch.arange(m, dtype=torch.int32, device=DEV)
        pos = torch.full((m,), ctx - 1, dtype=torch.int32, device=DEV)
        q = torch.randn(m, nh * hd, device=DEV).bfloat16()
        o = torch.empty_like(q)
        plans = [kernels.decode_mma_plan(m, nkv, hd, ctx)] + ([(s, 16, 4) for s in range(1, 7)] if sweep else [])
        for splits, block_keys, warps in plans:
            pa = torch.empty(m * nh * warps * splits * hd, device=DEV)
            pm = torch.empty(m * nh * warps * splits * 2, device=DEV)
            cn = torch.zeros(m * nkv, dtype=torch.int32, device=DEV)
            t = graph_time(lambda: kernels.attention_decode_mma(q, o, kc, vc, tables, row_seq, pos, nh, nkv, hd, ps, hd ** -0.5,
                                                                None, splits, pa, pm, cn, status, block_keys, warps))
            nbytes = m * ctx * nkv * hd * 2 * 2
            print(f"attention_decode_mma heads {nh}/{nkv} batch {m:3d} ctx {ctx} splits {splits} keys/iteration {block_keys or 32} "
                  f"warps {warps}: {t:7.1f} us {nbytes / t / 1e3:6.0f} GB/s", flush=True)
    kernels.check_status(status)


def bench_attention_prefill() -> None:
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for nh, nkv, hd, t_len, ps in [(9, 3, 64, 2048, 16), (15, 5, 64, 2048, 16), (32, 32, 64, 2048, 16), (32, 32, 64, 8192, 16),
                                   (32, 32, 64, 8192, 128)]:
        per = t_len // ps
        kc = torch.randn(per + 2, nkv, ps, hd, device=DEV).bfloat16()
        vc = torch.randn_like(kc)
        tables = torch.arange(per, dtype=torch.int32, device=DEV).view(1, per).contiguous()
        first = torch.tensor([0, t_len], dtype=torch.int32, device=DEV)
        start = torch.zeros(1, dtype=torch.int32, device=DEV)
        q = torch.randn(t_len, nh * hd, device=DEV).bfloat16()
        o = torch.empty_like(q)
        fl = 2.0 * t_len * t_len * nh * hd   # QK^T and PV over the causal half
        for name, fn in (("mma.sync", kernels.attention_prefill), ("tcgen05", kernels.attention_prefill_tc)):
            t = graph_time(lambda: fn(q, o, kc, vc, tables, first, start, t_len, nh, nkv, hd, ps, hd ** -0.5, None, status),
                           reps=6)
            print(f"attention_prefill {name:8s} heads {nh}/{nkv} x {hd}, {t_len} tokens, page {ps}: {t:7.1f} us {fl / t / 1e6:6.1f} TFLOP/s",
                  flush=True)
    kernels.check_status(status)


def bench_latent_attention() -> None:
    """Latent attention (heads x (64 + rotated), latent 128) beside grouped-query attention with as many heads of size 64:
    one 2,048-token prompt, and decoding at context 4,096."""
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ps, c = 16, 128
    for H, r, nkv in [(16, 32, 4), (32, 64, 8)]:
        w = c + r
        t_len = 2048
        per = t_len // ps
        cache = torch.randn(per + 2, 1, ps, w, device=DEV).bfloat16()
        tables = torch.arange(per, dtype=torch.int32, device=DEV).view(1, per).contiguous()
        first = torch.tensor([0, t_len], dtype=torch.int32, device=DEV)
        start = torch.zeros(1, dtype=torch.int32, device=DEV)
        pos = torch.arange(t_len, dtype=torch.int32, device=DEV)
        sink = torch.zeros(H, device=DEV)
        q = torch.randn(t_len, H * w, device=DEV).bfloat16()
        o = torch.empty(t_len, H * c, device=DEV).bfloat16()
        t = graph_time(lambda: kernels.latent_attention_mma(q, o, cache, tables, first, start, pos, sink, H, c, r, ps, w ** -0.5, None,
                                                            status, max_rows_per_seq=t_len), reps=6)
        fl = 1.0 * t_len * t_len * H * (w + c)           # scores over c + r and values over c, the causal half
        print(f"latent_attention prompt  heads {H} latent {c}+{r}, {t_len} tokens: {t:7.1f} us {fl / t / 1e6:6.1f} TFLOP/s", flush=True)
        hd = 64
        kc = torch.randn(per + 2, nkv, ps, hd, device=DEV).bfloat16()
        vc = torch.randn_like(kc)
        q2 = torch.randn(t_len, H * hd, device=DEV).bfloat16()
        o2 = torch.empty_like(q2)
        t = graph_time(lambda: kernels.attention_prefill_tc(q2, o2, kc, vc, tables, first, start, t_len, H, nkv, hd, ps, hd ** -0.5,
                                                            None, status), reps=6)
        fl = 2.0 * t_len * t_len * H * hd
        print(f"   grouped-query prompt  heads {H}/{nkv} x {hd} (tcgen05), {t_len} tokens: {t:7.1f} us {fl / t / 1e6:6.1f} TFLOP/s", flush=True)
        ctx = 4096
        for m in (1, 8, 64):
            per = ctx // ps
            cache = torch.randn(m * per + 4, 1, ps, w, device=DEV).bfloat16()
            tables = torch.arange(m * per, dtype=torch.int32, device=DEV).view(m, per).contiguous()
            first = torch.arange(m + 1, dtype=torch.int32, device=DEV)
            pos = torch.full((m,), ctx - 1, dtype=torch.int32, device=DEV)
            q = torch.randn(m, H * w, device=DEV).bfloat16()
            o = torch.empty(m, H * c, device=DEV).bfloat16()
            splits = kernels.latent_decode_splits(m, H, ctx)
            po, pm = torch.empty(m, H * splits * c, device=DEV), torch.empty(m, H * splits * 2, device=DEV)
            t = graph_time(lambda: kernels.latent_attention_mma(q, o, cache, tables, first, pos, pos, sink, H, c, r, ps, w ** -0.5,
                                                                None, status, decode=True, splits=splits, part_o=po, part_ml=pm))
            nbytes = m * ctx * w * 2
            print(f"latent_attention decode  heads {H} latent {c}+{r} batch {m:3d} ctx {ctx} shares {splits:2d}: {t:7.1f} us "
                  f"{nbytes / t / 1e3:6.0f} GB/s", flush=True)
            kc = torch.randn(m * per + 4, nkv, ps, hd, device=DEV).bfloat16()
            vc = torch.randn_like(kc)
            row_seq = torch.arange(m, dtype=torch.int32, device=DEV)
            q2 = torch.randn(m, H * hd, device=DEV).bfloat16()
            o2 = torch.empty_like(q2)
            sp, block_keys, warps = kernels.decode_mma_plan(m, nkv, hd, ctx)
            pa = torch.empty(m * H * warps * sp * hd, device=DEV)
            pm2 = torch.empty(m * H * warps * sp * 2, device=DEV)
            cn = torch.zeros(m * nkv, dtype=torch.int32, device=DEV)
            t = graph_time(lambda: kernels.attention_decode_mma(q2, o2, kc, vc, tables, row_seq, pos, H, nkv, hd, ps, hd ** -0.5, None,
                                                                sp, pa, pm2, cn, status, block_keys, warps))
            nbytes = m * ctx * nkv * hd * 2 * 2
            print(f"   grouped-query decode  heads {H}/{nkv} x {hd} batch {m:3d} ctx {ctx}: {t:7.1f} us {nbytes / t / 1e3:6.0f} GB/s", flush=True)
    kernels.check_status(status)


def bench_delta_rule() -> None:
    """The recurrence with key and value size 128: a 2,048-token prompt (a chain of 2,048 dependent updates per column of S),
    and single tokens for 1, 8 and 64 requests (S read and written once: bytes / time)."""
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    dk = dv = 128
    for H in (8, 16):
        for n, S in ((2048, 1), (1, 1), (8, 8), (64, 64)):
            per = n // S
            qkv = torch.randn(n, 2 * H * dk + H * dv, device=DEV)
            beta, a, gate = torch.randn(n, H, device=DEV), torch.randn(n, H * dk, device=DEV), torch.randn(n, H * dv, device=DEV)
            dt, al, w = torch.randn(H * dk, device=DEV), torch.zeros(H, device=DEV), torch.ones(dv, device=DEV)
            copies = max(1, int(2 * L2_BYTES / (S * H * dk * dv * 4)))            # rotate through more state than L2 holds
            states = [torch.zeros(S, H * dk * dv, device=DEV) for _ in range(min(copies, 8))]
            first = torch.arange(0, n + 1, per, dtype=torch.int32, device=DEV)
            start = torch.zeros(S, dtype=torch.int32, device=DEV)
            slots = torch.arange(S, dtype=torch.int32, device=DEV)
            turn = [0]
            if per == 1:
                att = torch.empty(n, H * dv, device=DEV).bfloat16()

                def fn():
                    turn[0] += 1
                    kernels.channel_delta_decode(qkv, beta, a, dt, al, states[turn[0] % len(states)], gate, w, 1e-6, att, first, start,
                                                 slots, H, H, dk, dv, True, status)
                t = graph_time(fn)
                nbytes = 2.0 * S * H * dk * dv * 4
                print(f"delta_rule single tokens heads {H} x {dk} x {dv}, {S:2d} requests: {t:7.1f} us {nbytes / t / 1e3:6.0f} GB/s", flush=True)
            else:
                out = torch.empty(n, H * dv, device=DEV)
                t = graph_time(lambda: kernels.channel_delta(qkv, beta, a, dt, al, states[0], out, first, start, slots, H, H, dk, dv,
                                                             True, status), reps=3)
                print(f"delta_rule prompt heads {H} x {dk} x {dv}, {n} tokens: {t:7.1f} us = {t / n:5.3f} us per token "
                      f"({6.0 * n * H * dk * dv / t / 1e6:5.2f} TFLOP/s)", flush=True)
    kernels.check_status(status)


def bench_lonorax() -> None:
    """Each kernel of the Lonorax path beside the like kernel of the other paths, at the sizes of the width-1024 and
    width-2048 models that ``bench.py --workload lonorax`` runs."""
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ps, hd, window, t_len = 16, 64, 1024, 2048
    for H, G in ((16, 4), (32, 8)):
        per = t_len // ps
        kc = torch.randn(per + 2, G, ps, hd, device=DEV).bfloat16()
        vc = torch.randn_like(kc)
        tables = torch.arange(per, dtype=torch.int32, device=DEV).view(1, per).contiguous()
        first = torch.tensor([0, t_len], dtype=torch.int32, device=DEV)
        start = torch.zeros(1, dtype=torch.int32, device=DEV)
        q = torch.randn(t_len, H * hd, device=DEV).bfloat16()
        o = torch.empty_like(q)
        bias = torch.full((H,), -2.0, device=DEV)
        # multiply-adds over the keys a row sees: rows below the window see all earlier keys, the others `window`
        seen = sum(min(p + 1, window) for p in range(t_len))
        fl = 2.0 * seen * H * (hd + hd)
        t = graph_time(lambda: kernels.sigmoid_attention_tiles(q, o, kc, vc, tables, first, start, t_len, bias, H, G, hd, hd, ps,
                                                               hd ** -0.5, window, status), reps=6)
        print(f"sigmoid_attention prompt heads {H}/{G} x {hd}, window {window}, {t_len} tokens: {t:7.1f} us {fl / t / 1e6:6.1f} TFLOP/s", flush=True)
        for name, fn in (("mma.sync", kernels.attention_prefill), ("tcgen05", kernels.attention_prefill_tc)):
            t = graph_time(lambda: fn(q, o, kc, vc, tables, first, start, t_len, H, G, hd, ps, hd ** -0.5, window, status), reps=6)
            print(f"   grouped-query prompt ({name}) the same heads and window: {t:7.1f} us {fl / t / 1e6:6.1f} TFLOP/s", flush=True)
        ctx = 4096
        for m in (1, 8, 64):
            per = ctx // ps
            kc = torch.randn(m * per + 4, G, ps, hd, device=DEV).bfloat16()
            vc = torch.randn_like(kc)
            tables = torch.arange(m * per, dtype=torch.int32, device=DEV).view(m, per).contiguous()
            row_seq = torch.arange(m, dtype=torch.int32, device=DEV)
            pos = torch.full((m,), ctx - 1, dtype=torch.int32, device=DEV)
            q = torch.randn(m, H * hd, device=DEV).bfloat16()
            o = torch.empty_like(q)
            nbytes = m * window * G * hd * 2 * 2
            t = graph_time(lambda: kernels.sigmoid_attention_decode(q, o, kc, vc, tables, row_seq, pos, bias, H, G, hd, hd, ps, hd ** -0.5,
                                                                    window, status))
            print(f"sigmoid_attention decode heads {H}/{G} x {hd} batch {m:3d} window {window}: {t:7.1f} us {nbytes / t / 1e3:6.0f} GB/s", flush=True)
            sp, block_keys, warps = kernels.decode_mma_plan(m, G, hd, window)
            pa = torch.empty(m * H * warps * sp * hd, device=DEV)
            pm = torch.empty(m * H * warps * sp * 2, device=DEV)
            cn = torch.zeros(m * G, dtype=torch.int32, device=DEV)
            t = graph_time(lambda: kernels.attention_decode_mma(q, o, kc, vc, tables, row_seq, pos, H, G, hd, ps, hd ** -0.5, window,
                                                                sp, pa, pm, cn, status, block_keys, warps))
            print(f"   grouped-query decode the same heads and window: {t:7.1f} us {nbytes / t / 1e3:6.0f} GB/s", flush=True)
    # the routed experts: 16 experts, two per token, beside the dense product of as many multiply-adds (the shared expert's)
    for d, ff in ((1024, 1024), (2048, 2048)):
        E, top = 16, 2
        for n in (2048, 64, 8):
            h = (torch.randn(n, d, device=DEV) * 0.5).bfloat16()
            ups = [(torch.randn(E * ff, d, device=DEV) * 0.03).bfloat16() for _ in range(3)]
            downs = [(torch.randn(E * d, ff, device=DEV) * 0.03).bfloat16() for _ in range(3)]
            choice = torch.stack([torch.randperm(E, device=DEV)[:top] for _ in range(n)]).int().contiguous()
            positions = torch.arange(n, dtype=torch.int32, device=DEV)
            pair = torch.empty(n, top * d, device=DEV)
            turn = [0]
            fl = 2.0 * n * top * 2 * d * ff
            if n > 16:
                tabs = torch.zeros(2 * (E + 1) + n * top, dtype=torch.int32, device=DEV)
                act = torch.empty(n, top * ff, device=DEV).bfloat16()

                def fn():
                    turn[0] += 1
                    kernels.moe_experts_grouped(h, ups[turn[0] % 3], downs[turn[0] % 3], E, choice, positions, tabs, act, pair)
            else:
                act = torch.empty(n, top * ff, device=DEV)

                def fn():
                    turn[0] += 1
                    kernels.moe_expert_halves(h, ups[turn[0] % 3], downs[turn[0] % 3], E, choice, positions, act, pair)
            t = graph_time(fn, reps=6)
            used = min(E, n * top) * 2 * d * ff * 2          # bytes of the experts that any row chose (at most all)
            print(f"routed experts {E} x ({d} -> {ff} -> {d}), {top} per token, {n:4d} rows: {t:7.1f} us {fl / t / 1e6:6.1f} TFLOP/s "
                  f"{used / t / 1e3:6.0f} GB/s of chosen weights", flush=True)
            w1 = _rotating(2 * ff, d)
            w2 = _rotating(d, 2 * ff)
            a1 = torch.empty(n, 2 * ff, device=DEV).bfloat16()
            out = torch.empty(n, d, device=DEV)

            def dense():
                turn[0] += 1
                if n > 64:
                    kernels.gemm_tc(h, w1[turn[0] % len(w1)], a1, False, status, relu2=True)
                    kernels.gemm_tc(a1, w2[turn[0] % len(w2)], out, False, status)
                else:
                    kernels.gemm_stream(h, w1[turn[0] % len(w1)], a1, relu2=True)
                    kernels.gemm_stream(a1, w2[turn[0] % len(w2)], out)
            t = graph_time(dense, reps=6)
            print(f"   dense squared-ReLU feed-forward {d} -> {2 * ff} -> {d} (as many multiply-adds), {n:4d} rows: {t:7.1f} us "
                  f"{fl / t / 1e6:6.1f} TFLOP/s {2 * 2 * d * ff * 2 / t / 1e3:6.0f} GB/s", flush=True)
    # minGRU: the scan over a prompt (reads the float32 projections twice, writes the gated output) and for single tokens
    for width in (2048, 4096):
        for n, S in ((2048, 1), (64, 64)):
            proj = torch.randn(n, 3 * width, device=DEV)
            bz, bx = torch.randn(width, device=DEV), torch.randn(width, device=DEV)
            state = torch.zeros(S, width, device=DEV)
            out = torch.empty(n, width, device=DEV).bfloat16()
            per = n // S
            first = torch.arange(0, n + 1, per, dtype=torch.int32, device=DEV)
            start = torch.zeros(S, dtype=torch.int32, device=DEV)
            slots = torch.arange(S, dtype=torch.int32, device=DEV)
            t = graph_time(lambda: kernels.mingru_scan(proj, bz, bx, state, 0, out, first, start, slots, width, True, status, max_rows=per),
                           reps=6)
            nbytes = n * width * (3 * 4 + 2)
            print(f"mingru width {width}, {S} requests x {per} rows: {t:7.1f} us {nbytes / t / 1e3:6.0f} GB/s (projections once + output)", flush=True)
    # the streams' row kernel (fold + read + layer norm over four streams) beside RMSNorm over one row
    for d in (1024, 2048):
        for n in (2048, 8):
            S = 4
            xs = torch.randn(n, S * d, device=DEV)
            y = torch.randn(n, d, device=DEV)
            mix, write, read = torch.eye(S, device=DEV).contiguous(), torch.ones(S, device=DEV), torch.full((S,), 0.25, device=DEV)
            w, b = torch.ones(d, device=DEV), torch.zeros(d, device=DEV)
            h = torch.empty(n, d, device=DEV).bfloat16()
            positions = torch.arange(n, dtype=torch.int32, device=DEV)
            t = graph_time(lambda: kernels.streams_step(xs, S, fold=(y, mix, write), read=read, norm=(w, b, 1e-6), h=h, positions=positions))
            nbytes = n * d * (2 * S * 4 + 4 + 2)
            print(f"streams fold + read + layer norm, {S} streams x {d}, {n:4d} rows: {t:7.1f} us {nbytes / t / 1e3:6.0f} GB/s", flush=True)
            x = torch.randn(n, d, device=DEV)
            t = graph_time(lambda: kernels.rmsnorm(x, w, h, 1e-6))
            print(f"   RMSNorm {d}, {n:4d} rows: {t:7.1f} us {n * d * 6 / t / 1e3:6.0f} GB/s", flush=True)
    kernels.check_status(status)


def bench_tagenex() -> None:
    """Each kernel of the Tagenex path beside the like kernel of the Llama path, at the sizes of the width-1024 and width-2048
    models that ``bench.py --workload tagenex`` runs."""
    from .parts.rope import rotary_table
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ps, hd, window, t_len = 16, 64, 1024, 2048
    for H, G in ((16, 4), (32, 8)):
        per = t_len // ps
        kc = torch.randn(per + 2, G, ps, hd, device=DEV).bfloat16()
        vc = torch.randn_like(kc)
        tables = torch.arange(per, dtype=torch.int32, device=DEV).view(1, per).contiguous()
        first = torch.tensor([0, t_len], dtype=torch.int32, device=DEV)
        start = torch.zeros(1, dtype=torch.int32, device=DEV)
        q = torch.randn(t_len, H * hd, device=DEV).bfloat16()
        o = torch.empty_like(q)
        r1, r2, sink = torch.full((H,), 0.5, device=DEV), torch.full((H,), 0.3, device=DEV), torch.zeros(H, device=DEV)
        gate = torch.randn(t_len, H, device=DEV)
        own = dict(r1=r1, r2=r2, sink=sink, heads=H, kv_heads=G, dim=hd, vdim=hd, page_size=ps, scale=hd ** -0.5, window=window,
                   status=status)
        seen = sum(min(p + 1, window) for p in range(t_len))
        fl = 2.0 * seen * H * (hd + hd)
        t = graph_time(lambda: kernels.sink_attention_tiles(q, o, kc, vc, tables, first, start, t_len, gate=gate, **own), reps=6)
        print(f"sink_attention prompt (mma.sync tiles) heads {H}/{G} x {hd}, window {window}, {t_len} tokens: {t:7.1f} us "
              f"{fl / t / 1e6:6.1f} TFLOP/s", flush=True)
        t = graph_time(lambda: kernels.attention_prefill_tc(q, o, kc, vc, tables, first, start, t_len, H, G, hd, ps, hd ** -0.5, window,
                                                            status, sink_terms=(r1, r2, sink, gate)), reps=6)
        print(f"sink_attention prompt (tcgen05) the same: {t:7.1f} us {fl / t / 1e6:6.1f} TFLOP/s", flush=True)
        for name, fn in (("mma.sync", kernels.attention_prefill), ("tcgen05", kernels.attention_prefill_tc)):
            t = graph_time(lambda: fn(q, o, kc, vc, tables, first, start, t_len, H, G, hd, ps, hd ** -0.5, window, status), reps=6)
            print(f"   grouped-query prompt ({name}) the same heads and window: {t:7.1f} us {fl / t / 1e6:6.1f} TFLOP/s", flush=True)
        # q/k norm, value mixing and the cache write from the float32 sums, beside rotation + cache write from bfloat16 sums
        for n in (t_len, 8):
            cols = (H + 2 * G) * hd
            proj = torch.randn(n, cols, device=DEV)
            pos = torch.arange(n, dtype=torch.int32, device=DEV)
            qn, kn = torch.ones(hd, device=DEV), torch.ones(hd, device=DEV)
            src, lam = torch.randn(n, G * hd, device=DEV), torch.full((), 0.4, device=DEV)
            qo = torch.empty(n, H * hd, device=DEV).bfloat16()
            t = graph_time(lambda: kernels.qk_norm_rope_write(proj, qn, kn, None, pos, pos, qo, kc, vc, H, G, hd, hd, 0, 1e-6, ps, True,
                                                              status, values_in=src, value_mix=lam))
            nbytes = n * (cols * 4 + G * hd * 4 + cols * 2)
            print(f"q/k norm + value mix + cache write heads {H}/{G}, {n:4d} rows: {t:6.1f} us {nbytes / t / 1e3:6.0f} GB/s", flush=True)
            qkv = torch.randn(n, cols, device=DEV).bfloat16()
            rope = rotary_table(10000.0, hd, 8192).to(DEV)
            t = graph_time(lambda: kernels.rope_kv_write(qkv, rope, pos, pos, kc, vc, H, G, hd, hd, ps, True, status))
            print(f"   rotation + cache write, {n:4d} rows: {t:6.1f} us {n * cols * 2 * 2 / t / 1e3:6.0f} GB/s", flush=True)
        ctx = 4096
        for m in (1, 8, 64):
            per = ctx // ps
            kc = torch.randn(m * per + 4, G, ps, hd, device=DEV).bfloat16()
            vc = torch.randn_like(kc)
            tables = torch.arange(m * per, dtype=torch.int32, device=DEV).view(m, per).contiguous()
            row_seq = torch.arange(m, dtype=torch.int32, device=DEV)
            pos = torch.full((m,), ctx - 1, dtype=torch.int32, device=DEV)
            q = torch.randn(m, H * hd, device=DEV).bfloat16()
            o = torch.empty_like(q)
            gate = torch.randn(m, H, device=DEV)
            nbytes = m * window * G * hd * 2 * 2
            t = graph_time(lambda: kernels.sink_attention_decode(q, o, kc, vc, tables, row_seq, pos, gate=gate, **own))
            print(f"sink_attention decode (warps share a row's keys) heads {H}/{G} x {hd} batch {m:3d} window {window}: {t:7.1f} us "
                  f"{nbytes / t / 1e3:6.0f} GB/s", flush=True)
            sp, block_keys, warps = kernels.decode_mma_plan(m, G, hd, window)
            pa = torch.empty(m * H * warps * sp * hd, device=DEV)
            pm = torch.empty(m * H * warps * sp * 2, device=DEV)
            cn = torch.zeros(m * G, dtype=torch.int32, device=DEV)
            t = graph_time(lambda: kernels.attention_decode_mma(q, o, kc, vc, tables, row_seq, pos, H, G, hd, ps, hd ** -0.5, window,
                                                                sp, pa, pm, cn, status, block_keys, warps,
                                                                sink_terms=(r1, r2, sink, gate)))
            print(f"sink_attention decode (split keys, tensor cores) the same: {t:7.1f} us {nbytes / t / 1e3:6.0f} GB/s", flush=True)
            sp, block_keys, warps = kernels.decode_mma_plan(m, G, hd, window)
            pa = torch.empty(m * H * warps * sp * hd, device=DEV)
            pm = torch.empty(m * H * warps * sp * 2, device=DEV)
            cn = torch.zeros(m * G, dtype=torch.int32, device=DEV)
            t = graph_time(lambda: kernels.attention_decode_mma(q, o, kc, vc, tables, row_seq, pos, H, G, hd, ps, hd ** -0.5, window,
                                                                sp, pa, pm, cn, status, block_keys, warps))
            print(f"   grouped-query decode the same heads and window: {t:7.1f} us {nbytes / t / 1e3:6.0f} GB/s", flush=True)
    # the branch norm into the residual (reads branch and residual, writes the residual and its bfloat16 copy) beside RMSNorm
    for d in (1024, 2048):
        for n in (2048, 8):
            y, x, w = torch.randn(n, d, device=DEV), torch.randn(n, d, device=DEV), torch.ones(d, device=DEV)
            h = torch.empty(n, d, device=DEV).bfloat16()
            t = graph_time(lambda: kernels.rmsnorm_add(y, w, x, 1e-6, copy=h))
            print(f"branch norm into the residual {d}, {n:4d} rows: {t:6.1f} us {n * d * 14 / t / 1e3:6.0f} GB/s", flush=True)
            t = graph_time(lambda: kernels.rmsnorm(x, w, h, 1e-6))
            print(f"   RMSNorm {d}, {n:4d} rows: {t:6.1f} us {n * d * 6 / t / 1e3:6.0f} GB/s", flush=True)
    # the dense feed-forward's first half with the clamped unit in the epilogue, beside the same product with SwiGLU
    for d, ff in ((1024, 4096), (2048, 8192)):
        for n in (2048, 64, 8):
            h = (torch.randn(n, d, device=DEV) * 0.5).bfloat16()
            ws = _rotating(2 * ff, d)
            bias = torch.randn(2 * ff, device=DEV) * 0.1
            act = torch.empty(n, ff, device=DEV).bfloat16()
            turn = [0]

            def unit():
                turn[0] += 1
                w = ws[turn[0] % len(ws)]
                (kernels.gemm_tc_unit(h, w, bias, 7.0, 1.702, act, status) if n > 64 else kernels.gemm_stream_unit(h, w, bias, 7.0, 1.702, act))

            def swiglu():
                turn[0] += 1
                w = ws[turn[0] % len(ws)]
                (kernels.gemm_tc_gated(h, w, act, status) if n > 64 else kernels.gemm_stream(h, w, act, gated=True))
            fl, nb = 2.0 * n * 2 * ff * d, 2 * ff * d * 2
            for name, fn in (("clamped unit", unit), ("   SwiGLU", swiglu)):
                t = graph_time(fn, reps=6)
                print(f"{name} in the epilogue of {d} -> 2 x {ff}, {n:4d} rows: {t:7.1f} us {fl / t / 1e6:6.1f} TFLOP/s {nb / t / 1e3:6.0f} GB/s", flush=True)
    # the router and the routed clamped experts: 16 experts, four per token, beside a dense feed-forward of as many multiply-adds
    for d, ff in ((1024, 1024), (2048, 2048)):
        E, top = 16, 4
        for n in (2048, 64, 8):
            h = (torch.randn(n, d, device=DEV) * 0.5).bfloat16()
            wr, br = torch.randn(E, d, device=DEV) * 0.05, torch.zeros(E, device=DEV)
            positions = torch.arange(n, dtype=torch.int32, device=DEV)
            choice = torch.empty(n, top, dtype=torch.int32, device=DEV)
            weight = torch.empty(n, top, device=DEV)
            t = graph_time(lambda: kernels.moe_route(h, wr, None, None, positions, top, 1, 1, 1.0, choice, weight, None, router_bias=br,
                                                     softmax_chosen=True))
            print(f"router {E} experts, {top} per token, width {d}, {n:4d} rows: {t:6.1f} us {(n * d * 2 + E * d * 4) / t / 1e3:6.0f} GB/s", flush=True)
            ups = [(torch.randn(E * 2 * ff, d, device=DEV) * 0.03).bfloat16() for _ in range(3)]
            downs = [(torch.randn(E * d, ff, device=DEV) * 0.03).bfloat16() for _ in range(3)]
            pair = torch.empty(n, top * d, device=DEV)
            turn = [0]
            fl = 2.0 * n * top * 3 * d * ff
            if n > 16:
                tabs = torch.zeros(2 * (E + 1) + n * top, dtype=torch.int32, device=DEV)
                act = torch.empty(n, top * ff, device=DEV).bfloat16()

                def fn():
                    turn[0] += 1
                    kernels.moe_experts_grouped(h, ups[turn[0] % 3], downs[turn[0] % 3], E, choice, positions, tabs, act, pair, unit=(7.0, 1.702))
            else:
                act = torch.empty(n, top * ff, device=DEV)

                def fn():
                    turn[0] += 1
                    kernels.moe_expert_halves(h, ups[turn[0] % 3], downs[turn[0] % 3], E, choice, positions, act, pair, unit=(7.0, 1.702))
            t = graph_time(fn, reps=6)
            used = int(choice.unique().numel()) * 3 * d * ff * 2       # bytes of the experts that any row chose
            print(f"routed clamped experts {E} x ({d} -> 2 x {ff} -> {d}), {top} per token, {n:4d} rows: {t:7.1f} us {fl / t / 1e6:6.1f} TFLOP/s "
                  f"{used / t / 1e3:6.0f} GB/s of chosen weights", flush=True)
            dff = top * ff
            w1, w2 = _rotating(2 * dff, d), _rotating(d, dff)
            a1 = torch.empty(n, dff, device=DEV).bfloat16()
            out = torch.empty(n, d, device=DEV)

            def dense():
                turn[0] += 1
                if n > 64:
                    kernels.gemm_tc_gated(h, w1[turn[0] % len(w1)], a1, status)
                    kernels.gemm_tc(a1, w2[turn[0] % len(w2)], out, False, status)
                else:
                    kernels.gemm_stream(h, w1[turn[0] % len(w1)], a1, gated=True)
                    kernels.gemm_stream(a1, w2[turn[0] % len(w2)], out)
            t = graph_time(dense, reps=6)
            print(f"   dense SwiGLU feed-forward {d} -> 2 x {dff} -> {d} (as many multiply-adds), {n:4d} rows: {t:7.1f} us "
                  f"{fl / t / 1e6:6.1f} TFLOP/s {3 * d * dff * 2 / t / 1e3:6.0f} GB/s", flush=True)
    kernels.check_status(status)


def bench_babotar() -> None:
    """Each kernel of the Babotar path beside the like kernel of the closest path, at the sizes of the width-1024 and
    width-2048 models that ``bench.py --workload babotar`` runs."""
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ps, hd, t_len, ctx = 16, 64, 2048, 4096
    for H, G in ((16, 4), (32, 8)):
        per = t_len // ps
        kc = torch.randn(per + 2, G, ps, hd, device=DEV).bfloat16()
        vc = torch.randn_like(kc)
        tables = torch.arange(per, dtype=torch.int32, device=DEV).view(1, per).contiguous()
        first = torch.tensor([0, t_len], dtype=torch.int32, device=DEV)
        start = torch.zeros(1, dtype=torch.int32, device=DEV)
        pos = torch.arange(t_len, dtype=torch.int32, device=DEV)
        q = torch.randn(t_len, H * hd, device=DEV).bfloat16()
        o = torch.empty_like(q)
        wide = torch.empty(t_len, H * G * hd, device=DEV)
        talk = torch.eye(H, device=DEV) + 0.1 * torch.randn(H, H, device=DEV)
        own = dict(heads=H, kv_heads=G, dim=hd, vdim=hd, value_heads=G, page_size=ps, scale=hd ** -0.5, softcap=30.0, unit_sink=True,
                   window=None, status=status)
        seen = t_len * (t_len + 1) // 2
        fl_own, fl_like = 2.0 * seen * H * (hd + G * hd), 2.0 * seen * H * (hd + hd)
        t = graph_time(lambda: kernels.talking_attention_tiles(q, wide, kc, vc, tables, first, start, t_len, **own), reps=4)
        print(f"talking_attention prompt (mma.sync tiles, every head over {G} value heads) heads {H}/{G} x {hd}, {t_len} tokens: {t:7.1f} us "
              f"{fl_own / t / 1e6:6.1f} TFLOP/s", flush=True)
        t = graph_time(lambda: kernels.talk_combine(wide, talk, o, pos, H, G, hd, G), reps=4)
        print(f"   mix of the heads, {t_len} rows: {t:7.1f} us {(wide.numel() * 4 + o.numel() * 2) / t / 1e3:6.0f} GB/s", flush=True)
        for name, fn in (("mma.sync", kernels.attention_prefill), ("tcgen05", kernels.attention_prefill_tc)):
            t = graph_time(lambda: fn(q, o, kc, vc, tables, first, start, t_len, H, G, hd, ps, hd ** -0.5, None, status), reps=4)
            print(f"   grouped-query prompt ({name}) the same heads: {t:7.1f} us {fl_like / t / 1e6:6.1f} TFLOP/s", flush=True)
        cols = (H + 2 * G) * hd
        from .parts.rope import rotary_table
        rope = rotary_table(10000.0, hd, 8192).to(DEV)
        for n in (t_len, 8):
            proj, bias = torch.randn(n, cols, device=DEV), torch.randn(cols, device=DEV)
            qo = torch.empty(n, H * hd, device=DEV).bfloat16()
            p = pos[:n]
            t = graph_time(lambda: kernels.bias_rope_write(proj, bias, rope, p, p, qo, kc, vc, H, G, hd, hd, hd, ps, True, status))
            print(f"bias + rotation + cache write heads {H}/{G}, {n:4d} rows: {t:6.1f} us {n * cols * 6 / t / 1e3:6.0f} GB/s", flush=True)
            qkv = torch.randn(n, cols, device=DEV).bfloat16()
            t = graph_time(lambda: kernels.rope_kv_write(qkv, rope, p, p, kc, vc, H, G, hd, hd, ps, True, status))
            print(f"   rotation + cache write, {n:4d} rows: {t:6.1f} us {n * cols * 4 / t / 1e3:6.0f} GB/s", flush=True)
        for m in (1, 8, 64):
            per = ctx // ps
            kd = torch.randn(m * per + 4, G, ps, hd, device=DEV).bfloat16()
            vd = torch.randn_like(kd)
            tb = torch.arange(m * per, dtype=torch.int32, device=DEV).view(m, per).contiguous()
            row_seq = torch.arange(m, dtype=torch.int32, device=DEV)
            pd = torch.full((m,), ctx - 1, dtype=torch.int32, device=DEV)
            qd = torch.randn(m, H * hd, device=DEV).bfloat16()
            od = torch.empty_like(qd)
            wd = torch.empty(m, H * G * hd, device=DEV)
            nbytes = m * ctx * G * hd * 2 * 2
            shares = kernels.talking_decode_shares(m, H, G, hd, G, ctx)
            wd = torch.empty(shares * m, H * G * hd, device=DEV)
            mld = torch.empty(shares * m, H * 2, device=DEV)
            t = graph_time(lambda: kernels.talking_attention_decode(qd, wd, kd, vd, tb, row_seq, pd, shares=shares, ml=mld, **own))
            t2 = graph_time(lambda: kernels.talk_combine(wd, talk, od, pd, H, G, hd, G, shares=shares, ml=mld))
            print(f"talking_attention decode heads {H}/{G} x {hd} batch {m:3d} context {ctx}, {shares:2d} shares: {t:7.1f} us "
                  f"{nbytes / t / 1e3:6.0f} GB/s (the cache once); merge + mix of the heads {t2:6.1f} us", flush=True)
            sp, block_keys, warps = kernels.decode_mma_plan(m, G, hd, ctx)
            pa = torch.empty(m * H * warps * sp * hd, device=DEV)
            pm = torch.empty(m * H * warps * sp * 2, device=DEV)
            cn = torch.zeros(m * G, dtype=torch.int32, device=DEV)
            t = graph_time(lambda: kernels.attention_decode_mma(qd, od, kd, vd, tb, row_seq, pd, H, G, hd, ps, hd ** -0.5, None, sp, pa, pm,
                                                                cn, status, block_keys, warps))
            print(f"   grouped-query decode (split keys) the same: {t:7.1f} us {nbytes / t / 1e3:6.0f} GB/s", flush=True)
    # the recurrences: lightning attention and the delta rule with one decay per head, key and value size 128
    dk = dv = 128
    for H in (8, 16):
        for n, S in ((2048, 1), (1, 1), (8, 8), (64, 64)):
            per = n // S
            qkv = torch.randn(n, 2 * H * dk + H * dv, device=DEV)
            decay = torch.full((H,), 0.97, device=DEV)
            first = torch.arange(0, n + 1, per, dtype=torch.int32, device=DEV)
            start = torch.zeros(S, dtype=torch.int32, device=DEV)
            slots = torch.arange(S, dtype=torch.int32, device=DEV)
            copies = max(1, int(2 * L2_BYTES / (S * H * dk * dv * 4)))
            states = [torch.zeros(S, H * dk * dv, device=DEV) for _ in range(min(copies, 8))]
            out = torch.empty(n, H * dv, device=DEV)
            turn = [0]

            def lightning():
                turn[0] += 1
                run = kernels.decay_linear_attention_decode if per == 1 else kernels.decay_linear_attention
                run(qkv, decay, states[turn[0] % len(states)], out, first, start, slots, H, dk, dv, True, status)
            t = graph_time(lightning, reps=3 if per > 1 else 12)
            beta, a, gate = torch.randn(n, H, device=DEV), torch.randn(n, H, device=DEV), torch.randn(n, H * dv, device=DEV)
            dt, al, w = torch.randn(H, device=DEV), torch.zeros(H, device=DEV), torch.ones(dv, device=DEV)
            if per == 1:
                att = torch.empty(n, H * dv, device=DEV).bfloat16()

                def delta():
                    turn[0] += 1
                    kernels.channel_delta_decode(qkv, beta, a, dt, al, states[turn[0] % len(states)], gate, w, 1e-6, att, first, start,
                                                 slots, H, H, dk, dv, True, status, decay_per_head=True, gate_silu=True)
                t2 = graph_time(delta)
                nbytes = 2.0 * S * H * dk * dv * 4
                print(f"lightning single tokens heads {H} x {dk} x {dv}, {S:2d} requests: {t:7.1f} us {nbytes / t / 1e3:6.0f} GB/s; "
                      f"delta rule (one decay per head, decoding form): {t2:7.1f} us {nbytes / t2 / 1e3:6.0f} GB/s", flush=True)
            else:
                t2 = graph_time(lambda: kernels.channel_delta(qkv, beta, a, dt, al, states[0], out, first, start, slots, H, H, dk, dv, True,
                                                              status, decay_per_head=True), reps=3)
                piece_rows = kernels.linear_piece_rows(n, H, dk, dv) or kernels.LINEAR_PIECE_ROWS
                pieces = kernels.linear_pieces_needed(n, S, piece_rows)
                meta = torch.zeros(4 * pieces + 2 * S + 1, dtype=torch.int32, device=DEV)
                piece_state = torch.empty(pieces, H * dk * dv, device=DEV)
                t3 = graph_time(lambda: kernels.decay_linear_attention_pieces(qkv, decay, states[0], out, first, start, slots, H, dk, dv, True,
                                                                              status, meta, piece_state, piece_rows=piece_rows), reps=3)
                print(f"lightning prompt heads {H} x {dk} x {dv}, {n} tokens: one walk {t:7.1f} us = {t / n:5.3f} us per token, in pieces of "
                      f"{piece_rows} {t3:7.1f} us; delta rule (one decay per head): {t2:7.1f} us = {t2 / n:5.3f} us per token", flush=True)
    # the convolution on the mixers' input and the gated GELU unit in the products' epilogues
    for d, ff in ((1024, 4096), (2048, 8192)):
        for n in (2048, 64, 8):
            x = torch.randn(n, d, device=DEV).bfloat16()
            y = torch.empty_like(x)
            w = torch.randn(d, 4, device=DEV)
            state = torch.zeros(1, 3 * d, device=DEV)
            row_seq = torch.zeros(n, dtype=torch.int32, device=DEV)
            pos = torch.arange(n, dtype=torch.int32, device=DEV)
            first = torch.tensor([0, n], dtype=torch.int32, device=DEV)
            zero = torch.zeros(1, dtype=torch.int32, device=DEV)
            t = graph_time(lambda: kernels.residual_conv(x, w, y, state, 0, row_seq, pos, first, zero, zero, True, status))
            print(f"input convolution (4 taps, two launches) {n:4d} rows x {d}: {t:6.1f} us {n * d * 4 / t / 1e3:6.0f} GB/s", flush=True)
            ws = _rotating(2 * ff, d)
            act = torch.empty(n, ff, device=DEV).bfloat16()
            turn = [0]
            for unit, args in (("gelu", kernels.GELU_UNIT), ("clamped", (7.0, 1.702))):
                def fn():
                    turn[0] += 1
                    wm = ws[turn[0] % len(ws)]
                    if n > kernels.STREAM_MAX_ROWS:
                        kernels.gemm_tc_unit(x, wm, None, args[0], args[1], act, status)
                    else:
                        kernels.gemm_stream_unit(x, wm, None, args[0], args[1], act)
                t = graph_time(fn)
                print(f"gated unit ({unit}) in the product's epilogue {n:4d} rows, {d} -> 2 x {ff}: {t:7.1f} us "
                      f"{2.0 * n * d * 2 * ff / t / 1e6:7.1f} TFLOP/s {2 * ff * d * 2 / t / 1e3:6.0f} GB/s", flush=True)
    kernels.check_status(status)


def bench_float32() -> None:
    """The kernels of the true 32-bit path at SmolLM2-135M shapes: FMA products for a 2,048-token prompt and for 8
    decoded rows, split-key decode attention and one-warp-per-row attention over a float32 cache."""
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for name, m, n, k in [("135m qkv, 2048 rows", 2048, 960, 576), ("135m gate/up, 2048 rows", 2048, 3072, 576),
                          ("135m down, 2048 rows", 2048, 576, 1536), ("135m qkv, 8 rows", 8, 960, 576),
                          ("135m head, 8 rows", 8, 49152, 576)]:
        a, w, c = torch.randn(m, k, device=DEV), torch.randn(n, k, device=DEV), torch.empty(m, n, device=DEV)
        t = graph_time(lambda: kernels.gemm_simt(a, w, c), reps=6)
        print(f"gemm_simt {name:24s} {m} x {n} x {k}: {t:8.1f} us {2.0 * m * n * k / t / 1e6:6.2f} TFLOP/s "
              f"{(m * k + n * k + m * n) * 4 / t / 1e3:6.0f} GB/s", flush=True)
    nh, nkv, hd, ps, ctx = 9, 3, 64, 16, 4096
    for m in (1, 8):
        per = ctx // ps
        kc = torch.randn(m * per + 4, nkv, ps, hd, device=DEV)
        vc = torch.randn_like(kc)
        tables = torch.arange(m * per, dtype=torch.int32, device=DEV).view(m, per).contiguous()
        row_seq = torch.arange(m, dtype=torch.int32, device=DEV)
        pos = torch.full((m,), ctx - 1, dtype=torch.int32, device=DEV)
        q = torch.randn(m, nh * hd, device=DEV)
        o = torch.empty_like(q)
        splits = kernels.decode_splits(m, nh, nkv, ctx)
        pa, pm = torch.empty(m * nh * splits * hd, device=DEV), torch.empty(m * nh * splits * 2, device=DEV)
        cn = torch.zeros(m * nh, dtype=torch.int32, device=DEV)
        nbytes = m * ctx * nkv * hd * 4 * 2
        t = graph_time(lambda: kernels.attention_decode(q, o, kc, vc, tables, row_seq, pos, nh, nkv, hd, ps, hd ** -0.5, None,
                                                        splits, pa, pm, cn, status))
        print(f"attention_decode (float32) batch {m} ctx {ctx} splits {splits}: {t:7.1f} us {nbytes / t / 1e3:6.0f} GB/s", flush=True)
        t = graph_time(lambda: kernels.attention_rows(q, o, kc, vc, tables, row_seq, pos, nh, nkv, hd, ps, hd ** -0.5, None, status))
        print(f"attention_rows   (float32) batch {m} ctx {ctx}: {t:7.1f} us {nbytes / t / 1e3:6.0f} GB/s", flush=True)
    kernels.check_status(status)


def bench_small() -> None:
    """The element-wise kernels and the sampling kernel at SmolLM2-135M sizes, for a 2,048-token prompt and for 8 rows."""
    from .parts.rope import rotary_table
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    d, inter, vocab, nh, nkv, hd, ps = 576, 1536, 49152, 9, 3, 64, 16
    table = (torch.randn(vocab, d, device=DEV) * 0.02).bfloat16()
    gain = torch.ones(d, device=DEV)
    rope = rotary_table(100000.0, hd, 8192).to(DEV)
    for n in (2048, 8):
        tokens = torch.randint(0, vocab, (n,), dtype=torch.int32, device=DEV)
        x = torch.empty(n, d, device=DEV)
        h = torch.empty(n, d, device=DEV, dtype=torch.bfloat16)
        t = graph_time(lambda: kernels.embed(table, tokens, x, status))
        print(f"embed            {n:5d} rows x {d}: {t:6.1f} us {n * d * 6 / t / 1e3:6.0f} GB/s", flush=True)
        t = graph_time(lambda: kernels.rmsnorm(x, gain, h, 1e-5))
        print(f"rmsnorm          {n:5d} rows x {d}: {t:6.1f} us {n * d * 6 / t / 1e3:6.0f} GB/s", flush=True)
        qkv = torch.randn(n, (nh + 2 * nkv) * hd, device=DEV).bfloat16()
        kc = torch.zeros(n // ps + 2, nkv, ps, hd, device=DEV, dtype=torch.bfloat16)
        vc = torch.zeros_like(kc)
        pos = torch.arange(n, dtype=torch.int32, device=DEV)
        t = graph_time(lambda: kernels.rope_kv_write(qkv, rope, pos, pos, kc, vc, nh, nkv, hd, hd, ps, True, status))
        print(f"rope_kv_write    {n:5d} rows: {t:6.1f} us {n * (nh + 2 * nkv) * hd * 2 * 2 / t / 1e3:6.0f} GB/s", flush=True)
        gu = torch.randn(n, 2 * inter, device=DEV).bfloat16()
        act = torch.empty(n, inter, device=DEV, dtype=torch.bfloat16)
        t = graph_time(lambda: kernels.swiglu(gu, act))
        print(f"swiglu           {n:5d} rows x {inter}: {t:6.1f} us {n * inter * 6 / t / 1e3:6.0f} GB/s", flush=True)
    for rows in (1, 8, 64):
        logits = torch.randn(rows, vocab, device=DEV)
        out = torch.empty(rows, dtype=torch.int32, device=DEV)
        temp = torch.full((rows,), 0.8, device=DEV)
        unif = torch.rand(rows, device=DEV)
        t = graph_time(lambda: kernels.sample(logits, out))
        t2 = graph_time(lambda: kernels.sample(logits, out, temp, unif))
        print(f"sample           {rows:3d} rows x {vocab}: greedy {t:6.1f} us {rows * vocab * 4 / t / 1e3:6.0f} GB/s | temperature "
              f"{t2:6.1f} us {rows * vocab * 4 * 3 / t2 / 1e3:6.0f} GB/s (three passes)", flush=True)
    kernels.check_status(status)


def bench_decode_program(batches) -> None:
    """A decode step of SmolLM2-135M shapes at context 4096: as the chain of kernels in a CUDA graph, and as a decode
    program run by the persistent kernel, shared by operations and by rows; for the programs also where the time goes
    (clock values that the first block notes for each operation: its own share of the work including the wait for the
    operation before, and the arrival at the barrier behind it), averaged over the layers."""
    import shutil
    import tempfile

    import numpy as np

    from . import write_random_model
    from .engine.engine import Engine, StepEntry
    from .models.llama import make_llama_raw_config
    shape = dict(num_hidden_layers=30, hidden_size=576, num_attention_heads=9, num_key_value_heads=3, intermediate_size=1536,
                 vocab_size=49152, rope_theta=100000.0, rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=8192)
    ctx_len, steps = 4096, 48
    tmp = tempfile.mkdtemp(prefix="glassbox_b200_microbench_")
    try:
        write_random_model(tmp, make_llama_raw_config(**shape), 0, torch.bfloat16)
        rng = np.random.default_rng(0)
        for batch in batches or (1, 8):
            for label, how in (("kernel chain", None), ("program, by operations", kernels.BY_OPERATIONS),
                               ("program, by rows", kernels.BY_ROWS)):
                kernels.PROGRAM_HOW = how if how is not None else kernels.BY_ROWS
                eng = Engine(tmp, "bfloat16", cache_tokens=batch * (ctx_len + 64), max_batch_tokens=2048, max_requests=batch + 2,
                             use_programs=how is not None)
                for i in range(batch):
                    eng.add_request(i)
                    toks = rng.integers(0, shape["vocab_size"], size=ctx_len - steps - 8)
                    for j in range(0, len(toks), 2048):
                        eng.step([StepEntry(i, toks[j:j + 2048].tolist(), [])])
                flags = [1] * batch

                def one():
                    eng.step([StepEntry(i, [5], [0]) for i in range(batch)], sampling=flags)
                for _ in range(4):
                    one()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(steps):
                    one()
                e1.record()
                torch.cuda.synchronize()
                line = f"135m batch {batch} context {ctx_len} {label:24s}: {e0.elapsed_time(e1) / steps:7.4f} ms per step"
                if how is not None:     # one more step outside the graphs, traced
                    eng.use_graphs = False
                    eng.ctx.program.trace_next = True
                    one()
                    torch.cuda.synchronize()
                    n, trace, _ = max(eng.ctx.program.traces, key=lambda t: t[0])
                    t = trace.cpu().numpy().reshape(2, n, 4).astype(np.float64)[0] / 1965.0     # microseconds at 1,965 MHz
                    k = (n // 5) * 5
                    parts = []
                    for j, name in enumerate(("qkv", "attention", "o", "gate/up", "down")):
                        sel = t[j:k:5]
                        parts.append(f"{name} {np.mean(sel[:, 2] - sel[:, 0]):.1f}+{np.mean((sel[:, 3] - sel[:, 2])[:-1]):.1f}")
                    line += f" | per operation, us (work + arrival), {n} operations: " + ", ".join(parts)
                print(line, flush=True)
                del eng
    finally:
        shutil.rmtree(tmp, ignore_errors=True)


def bench_layer_gemms(rows) -> None:
    """The four products of one SmolLM2-135M decode layer with what the layer folds into them: the norm on the way in,
    rotation and cache write on the way out of QKV, SwiGLU, the residual additions; each alone (back to back in a
    graph, cold weights) and the four in a row."""
    from .parts.rope import rotary_table
    st = torch.zeros(1, dtype=torch.int32, device=DEV)
    d, inter, nh, nkv, hd, ps = 576, 1536, 9, 3, 64, 16
    for m in rows or (1, 8, 16):
        res = torch.randn(m, d, device=DEV)
        gain = torch.ones(d, device=DEV)
        xb = torch.randn(m, d, device=DEV).bfloat16()
        wq, wo, wg, wd = _rotating(960, d), _rotating(d, d), _rotating(2 * inter, d), _rotating(d, inter)
        qkv = torch.empty(m, 960, device=DEV, dtype=torch.bfloat16)
        act = torch.empty(m, inter, device=DEV, dtype=torch.bfloat16)
        table = rotary_table(1e5, hd, 8192).to(DEV)
        pos = torch.full((m,), 4000, dtype=torch.int32, device=DEV)
        slots = torch.arange(m, dtype=torch.int32, device=DEV) * ps
        kc = torch.zeros(m + 2, nkv, ps, hd, device=DEV, dtype=torch.bfloat16)
        vc = torch.zeros_like(kc)
        turn = [0]

        def nxt(ws):
            turn[0] += 1
            return ws[turn[0] % len(ws)]

        def qkv_full():
            kernels.gemm_stream_qkv(res, nxt(wq), qkv, table, pos, slots, kc, vc, nh, nkv, hd, ps, True, st, norm=(gain, 1e-5))

        def layer():
            qkv_full()
            kernels.gemm_stream(qkv[:, :d], nxt(wo), res, True)
            kernels.gemm_stream(res, nxt(wg), act, gated=True, norm=(gain, 1e-5))
            kernels.gemm_stream(act, nxt(wd), res, True)

        t = [graph_time(lambda: kernels.gemm_stream(xb, nxt(wq), qkv)),
             graph_time(lambda: kernels.gemm_stream(res, nxt(wq), qkv, norm=(gain, 1e-5))),
             graph_time(qkv_full),
             graph_time(lambda: kernels.gemm_stream(xb, nxt(wo), res, True)),
             graph_time(lambda: kernels.gemm_stream(xb, nxt(wg), act, gated=True)),
             graph_time(lambda: kernels.gemm_stream(res, nxt(wg), act, gated=True, norm=(gain, 1e-5))),
             graph_time(lambda: kernels.gemm_stream(act, nxt(wd), res, True)),
             graph_time(layer, reps=8)]
        print(f"rows {m:2d}: qkv {t[0]:.2f} us, + norm {t[1]:.2f}, + rotation and cache write {t[2]:.2f} | o + residual {t[3]:.2f} | "
              f"gate/up + SwiGLU {t[4]:.2f}, + norm {t[5]:.2f} | down + residual {t[6]:.2f} | the four in a row {t[7]:.2f}", flush=True)
    kernels.check_status(st)


CASES = ("gemm_stream", "gemm_tc", "attention_decode", "attention_splits", "attention_prefill", "float32", "small", "decode_program", "layer_gemms", "latent_attention", "delta_rule", "lonorax", "tagenex", "babotar")


def main(argv) -> int:
    global ONCE
    if "--once" in argv:
        ONCE = True
        argv = [a for a in argv if a != "--once"]
    if not argv or argv[0] not in CASES or (argv[0] == "attention_splits" and len(argv) < 4):
        print(__doc__)
        return 2
    torch.cuda.set_device(0)
    kernels.lib()
    if argv[0] == "gemm_stream":
        bench_gemm_stream(argv[1:])
    elif argv[0] == "gemm_tc":
        bench_gemm_tc()
    elif argv[0] == "attention_decode":
        bench_attention_decode([int(x) for x in argv[1:]])
    elif argv[0] == "attention_splits":
        nh, nkv, m = (int(x) for x in argv[1:4])
        bench_attention_decode([m], nh, nkv, int(argv[4]) if len(argv) > 4 else 4096, sweep=True)
    elif argv[0] == "float32":
        bench_float32()
    elif argv[0] == "small":
        bench_small()
    elif argv[0] == "decode_program":
        bench_decode_program([int(x) for x in argv[1:]])
    elif argv[0] == "layer_gemms":
        bench_layer_gemms([int(x) for x in argv[1:]])
    elif argv[0] == "latent_attention":
        bench_latent_attention()
    elif argv[0] == "delta_rule":
        bench_delta_rule()
    elif argv[0] == "lonorax":
        bench_lonorax()
    elif argv[0] == "tagenex":
        bench_tagenex()
    elif argv[0] == "babotar":
        bench_babotar()
    else:
        bench_attention_prefill()
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
