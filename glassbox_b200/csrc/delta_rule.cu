// A gated delta-rule mixer with one decay per head and key channel, and the short causal convolutions in front of it.
//
// Per head the state S is a [dk, dv] matrix of float32 that lives in the request's state slot. For each token, in order:
//     S <- diag(g) S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
// with g = exp(-exp(A_log) * softplus(a + dt_bias)) per key channel, beta = sigmoid(b), q and k unit vectors
// (x / sqrt(sum x^2 + 1e-6)) and q also times dk^(-1/2). Everything here is float32.
//
//   gb_short_conv        y[t, c] = silu(sum_j w[c, j] x[t - (taps-1) + j, c]), inputs before a portion's first row come
//                        from the request's state slot (zeros for a fresh request)
//   gb_short_conv_state  afterwards: the last taps-1 inputs of each request go to its slot
//   gb_channel_delta     the recurrence over runs of tokens; columns of S are independent, so a head is shared between
//                        blocks by columns
//   gb_channel_delta_decode  the recurrence for steps of single tokens, with the read-out's norm and gate, and (fused
//                        form) the convolutions and the low-rank products of the decay and the gate
#include "common.cuh"

// ----------------------------------------------------------------------------------------------
// Short convolution + SiLU. x: float32 [n, ldx] (channels 0..C-1), w: float32 [C, taps] (last column is the current
// token's), state: float32, per slot `state_stride` numbers of which [taps-1, C] from `state_off` on (oldest first).
// One thread per (row, channel).
// ----------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) short_conv_kernel(const float* __restrict__ x, long long ldx, const float* __restrict__ w,
                                                         float* __restrict__ y, long long ldy, const float* __restrict__ state,
                                                         long long state_stride, long long state_off, const int* __restrict__ row_seq,
                                                         const int* __restrict__ positions, const int* __restrict__ seq_first_row,
                                                         const int* __restrict__ seq_slots, int n, int C, int taps, int num_slots,
                                                         int* __restrict__ status) {
    gb_pdl_launch_dependents();
    gb_pdl_wait();
    const int row = blockIdx.x;
    const int ch = blockIdx.y * blockDim.x + threadIdx.x;
    if (row >= n || ch >= C) return;
    if (positions[row] < 0) return;
    const int seq = row_seq[row];
    const int r0 = seq_first_row[seq];
    const int slot = seq_slots[seq];
    if (slot < 0 || slot >= num_slots) {
        atomicOr(status, GB_STATUS_BAD_SLOT);
        return;
    }
    const float* st = state + (size_t)slot * state_stride + state_off;
    float acc = 0.f;
    for (int j = 0; j < taps; ++j) {
        const int src = row - (taps - 1) + j;     // the row that holds this tap's input, if it is of this portion
        float v;
        if (src >= r0) v = x[(size_t)src * ldx + ch];
        else v = st[(size_t)(taps - 1 - (r0 - src)) * C + ch];     // r0 - src inputs back from the portion's start
        acc = fmaf(w[(size_t)ch * taps + j], v, acc);
    }
    y[(size_t)row * ldy + ch] = acc / (1.0f + expf(-acc));
}

// One thread per (sequence, channel): shift what the slot holds by the portion's length and append the portion's last inputs.
__global__ void __launch_bounds__(256) short_conv_state_kernel(const float* __restrict__ x, long long ldx, float* __restrict__ state,
                                                               long long state_stride, long long state_off,
                                                               const int* __restrict__ seq_first_row, const int* __restrict__ seq_start_pos,
                                                               const int* __restrict__ seq_slots, int S, int C, int taps, int num_slots) {
    gb_pdl_launch_dependents();
    gb_pdl_wait();
    const int seq = blockIdx.x;
    const int ch = blockIdx.y * blockDim.x + threadIdx.x;
    if (seq >= S || ch >= C) return;
    if (seq_start_pos[seq] < 0) return;
    const int slot = seq_slots[seq];
    if (slot < 0 || slot >= num_slots) return;
    const int r0 = seq_first_row[seq], len = seq_first_row[seq + 1] - r0;
    float* st = state + (size_t)slot * state_stride + state_off;
    const int keep = taps - 1;
    for (int i = 0; i < keep; ++i) {      // increasing i: a kept value moves to a lower index than any still to be read
        const int p = len - keep + i;      // index within the portion
        st[(size_t)i * C + ch] = p >= 0 ? x[(size_t)(r0 + p) * ldx + ch] : st[(size_t)(i + len) * C + ch];
    }
}

GB_EXPORT int gb_short_conv(const float* x, long long ldx, const float* w, float* y, long long ldy, float* state,
                            long long state_stride, long long state_off, const int* row_seq, const int* positions,
                            const int* seq_first_row, const int* seq_start_pos, const int* seq_slots, int n, int S, int C, int taps,
                            int num_slots, int update_state, int* status, cudaStream_t stream) {
    GB_REQUIRE(n >= 0 && S >= 0 && C > 0 && taps >= 1 && taps <= 64, "gb_short_conv: bad sizes (taps %d)", taps);
    if (n == 0 || S == 0) return 0;
    dim3 grid(n, gb_ceil_div(C, 256));
    gb_launch(GB_PDL_ELEMENTWISE, short_conv_kernel, grid, dim3(256), 0, stream, x, ldx, w, y, ldy, (const float*)state, state_stride,
              state_off, row_seq, positions, seq_first_row, seq_slots, n, C, taps, num_slots, status);
    int rc = gb_check_launch("gb_short_conv");
    if (rc || !update_state || taps == 1) return rc;
    dim3 grid2(S, gb_ceil_div(C, 256));
    gb_launch(GB_PDL_ELEMENTWISE, short_conv_state_kernel, grid2, dim3(256), 0, stream, x, ldx, state, state_stride, state_off,
              seq_first_row, seq_start_pos, seq_slots, S, C, taps, num_slots);
    return gb_check_launch("gb_short_conv_state");
}

// ----------------------------------------------------------------------------------------------
// The recurrence. Grid (sequences of the step, heads, column blocks); four walking warps and eight staging warps.
//
// Walkers: a thread owns DPT rows of one column of S in registers: lane = column * NS + split, so the NS splits of a
// column are neighbouring lanes and the two reductions over the key dimension are shuffles. Per token the chain that
// cannot be shortened is: decay, dot with k, reduce, u, update; the read-out's own reduction is put off by one token
// and rides in the same shuffle rounds as the next token's dot product, and the next token's decays and keys are read
// from shared memory while those rounds are under way.
// Stagers: meanwhile the other eight warps prepare the next TC tokens in the second shared-memory buffer: every load
// of a batch is asked for before the first is used (instructions issue in order: a loop that uses each value as it
// arrives pays the trip to memory once per round), decays are evaluated (exp(-r * softplus(z)) = exp(-r * log(1 + e^z))
// with the hardware's exponential and logarithm, whose absolute error of about 1e-7 in the exponent is far below the
// float32 rounding of the state), then one warp per token sums the squares of q and k. The unit vectors are never
// formed: 1/|q| and 1/|k| are two numbers per token that the walkers apply to their sums.
// ----------------------------------------------------------------------------------------------
constexpr int CD_GROUP = 128, CD_STAGERS = 256, CD_THREADS = CD_GROUP + CD_STAGERS;   // walkers first, then stagers
constexpr float CD_UNIT_EPS = 1e-6f;

struct ChannelDeltaArgs {
    const float* qkv;       // [n, ldq]: q (kvh * dk), k (kvh * dk), v (heads * dv), after convolution and SiLU
    long long ldq;
    const float* beta;      // [n, ldb]: logits of beta, one per head
    long long ldb;
    const float* a;         // [n, lda]: decay logits before the bias, heads * dk
    long long lda;
    const float* dt_bias;   // [heads * dk]
    const float* a_log;     // [heads]
    float* state;           // per slot `state_stride` numbers; S is [heads, dk, dv] at the start
    long long state_stride;
    float* out;             // [n, heads * dv]: o before its norm
    const int* seq_first_row;
    const int* seq_start_pos;
    const int* seq_slots;
    int heads, kv_heads, dk, dv, ns, tc, num_slots, write_state;
    int* status;
    int decay_channels;     // dk: a decay per head and key channel (a, dt_bias: heads * dk); 1: one per head (a, dt_bias: heads)
    int flags;              // CD_* below
};
// CD_SILU_INPUTS: q, k and v pass SiLU as they are read (a mixer without convolutions in front).
// CD_PLAIN: linear attention with a fixed decay per head, S <- decay_h S + k v^T, o = S^T q: no beta, no correction towards
//           the value, no unit vectors, no factor on q; `a_log` then holds the decays themselves, a, beta and dt_bias are not read.
// CD_GATE_SILU: the decoding form's output gate is silu(gate) instead of sigmoid(gate).
// CD_NO_NORM: the decoding form leaves the read-out as it is (float32, no norm, no gate), for a norm that spans the heads.
enum { CD_SILU_INPUTS = 1, CD_PLAIN = 2, CD_GATE_SILU = 4, CD_NO_NORM = 8 };
__device__ __forceinline__ float cd_silu(float v) { return v / (1.0f + expf(-v)); }

template <int DPT, int NS>
__global__ void __launch_bounds__(CD_THREADS) channel_delta_kernel(ChannelDeltaArgs p) {
    extern __shared__ __align__(16) float cd_smem[];
    gb_pdl_launch_dependents();
    gb_pdl_wait();
    const int seq = blockIdx.x, head = blockIdx.y;
    if (p.seq_start_pos[seq] < 0) return;
    const int slot = p.seq_slots[seq];
    if (slot < 0 || slot >= p.num_slots) {
        if (threadIdx.x == 0) atomicOr(p.status, GB_STATUS_BAD_SLOT);
        return;
    }
    const int r0 = p.seq_first_row[seq], r1 = p.seq_first_row[seq + 1];
    const int TC = p.tc, dk = p.dk, dv = p.dv;
    constexpr int cols = CD_GROUP / NS;                    // columns of S per block
    const bool walker = threadIdx.x < CD_GROUP;
    const int wt = walker ? threadIdx.x : threadIdx.x - CD_GROUP;     // index within the group
    const int kvh = head / (p.heads / p.kv_heads);
    constexpr int PAD = DPT + 4;                           // a split's numbers start 16-byte aligned, on other banks than its neighbours'
    constexpr int row_w = NS * PAD, Dp = NS * DPT;         // Dp: the key size rounded up (a power of two)
    const int dp_shift = 31 - __clz(Dp), cols_shift = 31 - __clz(cols);
    const int per_token = 3 * row_w + cols + 4;
    const int buf_floats = TC * per_token;
    // one buffer: q [TC][row_w], k [TC][row_w], g [TC][row_w], v [TC][cols], scalars [TC][4] = (beta, 1/|q| / sqrt(dk), 1/|k|, -)
    const int n_chunks = (r1 - r0 + TC - 1) / TC;
    const bool plain = p.flags & CD_PLAIN, silu_in = p.flags & CD_SILU_INPUTS;
    const float decay_rate = plain ? 0.f : expf(p.a_log[head]);
    const float fixed_decay = plain ? p.a_log[head] : 1.f;
    const float q_scale = plain ? 1.0f : 1.0f / sqrtf((float)dk);
    const float corr = plain ? 0.f : 1.f;               // how much of S^T k is taken off the value
    const int dc = p.decay_channels;

    auto stage = [&](int chunk) {
        float* buf = cd_smem + (size_t)(chunk & 1) * buf_floats;
        float* qs = buf, *ks = qs + (size_t)TC * row_w, *gs = ks + (size_t)TC * row_w, *vs = gs + (size_t)TC * row_w;
        float* sc = vs + (size_t)TC * cols;
        const int c0 = r0 + chunk * TC;
        const int nt = min(TC, r1 - c0);
        const int total = nt * Dp;
        // everything the chunk needs from memory is asked for before anything is used
        const int vidx = wt, vt_ = vidx >> cols_shift, vcl = vidx & (cols - 1), vcc = blockIdx.z * cols + vcl;
        float vv = 0.f, bb = 0.f;
        if (vidx < nt * cols && vcc < dv) {
            vv = p.qkv[(size_t)(c0 + vt_) * p.ldq + (size_t)2 * p.kv_heads * dk + (size_t)head * dv + vcc];
            if (silu_in) vv = cd_silu(vv);
        }
        if (wt < nt && !plain) bb = p.beta[(size_t)(c0 + wt) * p.ldb + head];
        constexpr int U = 8;
        for (int base = wt; base < total; base += CD_STAGERS * U) {
            float qv[U], kv[U], zv[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int idx = base + u * CD_STAGERS;
                const int t = idx >> dp_shift, d = idx & (Dp - 1);
                qv[u] = kv[u] = 0.f;
                zv[u] = -1e30f;
                if (idx < total && d < dk) {
                    const size_t row = (size_t)(c0 + t);
                    qv[u] = p.qkv[row * p.ldq + (size_t)kvh * dk + d];
                    kv[u] = p.qkv[row * p.ldq + (size_t)(p.kv_heads + kvh) * dk + d];
                    if (!plain) {
                        const size_t ai = (size_t)head * dc + (dc > 1 ? d : 0);
                        zv[u] = p.a[row * p.lda + ai] + p.dt_bias[ai];
                    }
                    if (silu_in) { qv[u] = cd_silu(qv[u]); kv[u] = cd_silu(kv[u]); }
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int idx = base + u * CD_STAGERS;
                if (idx < total) {
                    const int t = idx >> dp_shift, d = idx & (Dp - 1);
                    const int at = t * row_w + (d / DPT) * PAD + d % DPT;
                    const float sp = zv[u] > 15.f ? zv[u] : __logf(1.0f + __expf(zv[u]));     // (padding channels: sp = 0, g = 1)
                    qs[at] = qv[u];
                    ks[at] = kv[u];
                    gs[at] = (plain && d < dk) ? fixed_decay : __expf(-decay_rate * sp);
                }
            }
        }
        if (vidx < nt * cols) vs[vidx] = vv;
        for (int idx = wt + CD_STAGERS; idx < nt * cols; idx += CD_STAGERS) {     // (more than 256 values: few splits, many columns)
            const int t = idx >> cols_shift, cl = idx & (cols - 1);
            const int cc = blockIdx.z * cols + cl;
            float val = cc < dv ? p.qkv[(size_t)(c0 + t) * p.ldq + (size_t)2 * p.kv_heads * dk + (size_t)head * dv + cc] : 0.f;
            vs[idx] = silu_in ? cd_silu(val) : val;
        }
        if (wt < nt) sc[wt * 4] = plain ? 1.0f : 1.0f / (1.0f + __expf(-bb));
        asm volatile("bar.sync 1, 256;" ::: "memory");         // the stagers among themselves
        const int lane = wt & 31;
        for (int t = wt >> 5; t < nt; t += CD_STAGERS / 32) {
            float sq = 0.f, sk = 0.f;
            for (int d = lane; d < dk; d += 32) {
                const int at = t * row_w + (d / DPT) * PAD + d % DPT;
                sq = fmaf(qs[at], qs[at], sq);
                sk = fmaf(ks[at], ks[at], sk);
            }
            sq = gb_warp_sum(sq);
            sk = gb_warp_sum(sk);
            if (lane == 0) {
                sc[t * 4 + 1] = plain ? 1.0f : q_scale / sqrtf(sq + CD_UNIT_EPS);
                sc[t * 4 + 2] = plain ? 1.0f : 1.0f / sqrtf(sk + CD_UNIT_EPS);
            }
        }
    };

    // walkers: their part of S
    const int split = wt % NS, col_local = wt / NS;
    const int col = blockIdx.z * cols + col_local;
    const bool live = walker && col < dv;
    float S[DPT];
    float* sbase = p.state + (size_t)slot * p.state_stride + (size_t)head * dk * dv;
    if (walker) {
#pragma unroll
        for (int i = 0; i < DPT; ++i) {
            const int d = split * DPT + i;
            S[i] = (live && d < dk) ? sbase[(size_t)d * dv + col] : 0.f;
        }
    }
    float o_part = 0.f;          // the read-out of the token before, not yet summed over the splits
    long long o_row = -1;

    if (!walker) stage(0);
    __syncthreads();
    for (int chunk = 0; chunk < n_chunks; ++chunk) {
        if (!walker) {
            if (chunk + 1 < n_chunks) stage(chunk + 1);
        } else {
            const float* buf = cd_smem + (size_t)(chunk & 1) * buf_floats;
            const float* qs = buf, *ks = qs + (size_t)TC * row_w, *gs = ks + (size_t)TC * row_w, *vs = gs + (size_t)TC * row_w;
            const float* sc = vs + (size_t)TC * cols;
            const int c0 = r0 + chunk * TC;
            const int nt = min(TC, r1 - c0);
            // the decays and keys of the token after this one are asked for while this token's sums travel the lanes
            constexpr bool AHEAD = DPT <= 16;              // (with 32 rows per thread the registers do not reach)
            float4 gn[DPT / 4], kn[DPT / 4];
            if (AHEAD) {
#pragma unroll
                for (int i = 0; i < DPT / 4; ++i) {
                    gn[i] = reinterpret_cast<const float4*>(gs + split * PAD)[i];
                    kn[i] = reinterpret_cast<const float4*>(ks + split * PAD)[i];
                }
            }
            for (int t = 0; t < nt; ++t) {
                if (!AHEAD) {
#pragma unroll
                    for (int i = 0; i < DPT / 4; ++i) {
                        gn[i] = reinterpret_cast<const float4*>(gs + t * row_w + split * PAD)[i];
                        kn[i] = reinterpret_cast<const float4*>(ks + t * row_w + split * PAD)[i];
                    }
                }
                const float4* q4 = reinterpret_cast<const float4*>(qs + t * row_w + split * PAD);
                const float4 scal = *reinterpret_cast<const float4*>(sc + t * 4);      // beta, 1/|q| / sqrt(dk), 1/|k|
                const float vt = vs[t * cols + col_local];
                float4 qv[DPT / 4];
                float kk[DPT];
                float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
                for (int i = 0; i < DPT / 4; ++i) {
                    const float4 g = gn[i], k = kn[i];
                    qv[i] = q4[i];
                    kk[4 * i] = k.x; kk[4 * i + 1] = k.y; kk[4 * i + 2] = k.z; kk[4 * i + 3] = k.w;
                    S[4 * i] *= g.x; S[4 * i + 1] *= g.y; S[4 * i + 2] *= g.z; S[4 * i + 3] *= g.w;
                    a0 = fmaf(S[4 * i], k.x, a0);
                    a1 = fmaf(S[4 * i + 1], k.y, a1);
                    a2 = fmaf(S[4 * i + 2], k.z, a2);
                    a3 = fmaf(S[4 * i + 3], k.w, a3);
                }
                if (AHEAD && t + 1 < nt) {
#pragma unroll
                    for (int i = 0; i < DPT / 4; ++i) {
                        gn[i] = reinterpret_cast<const float4*>(gs + (t + 1) * row_w + split * PAD)[i];
                        kn[i] = reinterpret_cast<const float4*>(ks + (t + 1) * row_w + split * PAD)[i];
                    }
                }
                float sk = (a0 + a1) + (a2 + a3);
#pragma unroll
                for (int o = 1; o < NS; o <<= 1) {       // this token's dot product and the last token's read-out, together
                    sk += __shfl_xor_sync(0xffffffffu, sk, o);
                    o_part += __shfl_xor_sync(0xffffffffu, o_part, o);
                }
                if (o_row >= 0 && split == 0 && live) p.out[(size_t)o_row * p.heads * dv + (size_t)head * dv + col] = o_part;
                const float u = scal.x * (vt - corr * scal.z * sk) * scal.z;     // beta (v - S^T k), times 1/|k| for the update below
                a0 = a1 = a2 = a3 = 0.f;
#pragma unroll
                for (int i = 0; i < DPT / 4; ++i) {
                    const float4 q = qv[i];
                    S[4 * i] = fmaf(kk[4 * i], u, S[4 * i]);
                    S[4 * i + 1] = fmaf(kk[4 * i + 1], u, S[4 * i + 1]);
                    S[4 * i + 2] = fmaf(kk[4 * i + 2], u, S[4 * i + 2]);
                    S[4 * i + 3] = fmaf(kk[4 * i + 3], u, S[4 * i + 3]);
                    a0 = fmaf(S[4 * i], q.x, a0);
                    a1 = fmaf(S[4 * i + 1], q.y, a1);
                    a2 = fmaf(S[4 * i + 2], q.z, a2);
                    a3 = fmaf(S[4 * i + 3], q.w, a3);
                }
                o_part = ((a0 + a1) + (a2 + a3)) * scal.y;
                o_row = c0 + t;
            }
        }
        __syncthreads();
    }
    if (walker) {
#pragma unroll
        for (int o = 1; o < NS; o <<= 1) o_part += __shfl_xor_sync(0xffffffffu, o_part, o);
        if (o_row >= 0 && split == 0 && live) p.out[(size_t)o_row * p.heads * dv + (size_t)head * dv + col] = o_part;
        if (p.write_state) {
#pragma unroll
            for (int i = 0; i < DPT; ++i) {
                const int d = split * DPT + i;
                if (live && d < dk) sbase[(size_t)d * dv + col] = S[i];
            }
        }
    }
}

GB_EXPORT int gb_channel_delta(const float* qkv, long long ldq, const float* beta, long long ldb, const float* a, long long lda,
                               const float* dt_bias, const float* a_log, float* state, long long state_stride, float* out,
                               const int* seq_first_row, const int* seq_start_pos, const int* seq_slots, int S, int heads,
                               int kv_heads, int dk, int dv, int num_slots, int write_state, int* status, int decay_channels,
                               int flags, cudaStream_t stream) {
    GB_REQUIRE(S >= 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0, "gb_channel_delta: heads %d must be a multiple of key heads %d",
               heads, kv_heads);
    GB_REQUIRE(decay_channels == 1 || decay_channels == dk, "gb_channel_delta: %d decays per head (one, or one per key channel)",
               decay_channels);
    GB_REQUIRE(dk > 0 && dk <= 1024 && dv > 0, "gb_channel_delta: a key size of %d is outside 1..1024", dk);
    if (S == 0) return 0;
    const int dpt = dk <= 128 ? 16 : 32;
    int ns = 1;
    while (ns * dpt < dk) ns *= 2;
    const int cols = CD_GROUP / ns;
    const int per_token = (3 * ns * (dpt + 4) + cols + 4) * (int)sizeof(float);
    int tc = (64 * 1024) / (2 * per_token);      // two buffers
    if (tc > 16) tc = 16;
    if (tc < 1) tc = 1;
    ChannelDeltaArgs p = {qkv, ldq, beta, ldb, a, lda, dt_bias, a_log, state, state_stride, out, seq_first_row, seq_start_pos,
                          seq_slots, heads, kv_heads, dk, dv, ns, tc, num_slots, write_state, status, decay_channels, flags};
    dim3 grid(S, heads, gb_ceil_div(dv, cols));
    const size_t smem = (size_t)2 * tc * per_token;
    bool launched = false;
#define CD_CASE(D, N)                                                                                              \
    if (!launched && dpt == D && ns == N) {                                                                        \
        static bool raised = false;                                                                                \
        if (!raised) {                                                                                             \
            cudaFuncSetAttribute(channel_delta_kernel<D, N>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024); \
            raised = true;                                                                                         \
        }                                                                                                          \
        gb_launch(GB_PDL_ATTENTION, channel_delta_kernel<D, N>, grid, dim3(CD_THREADS), smem, stream, p);          \
        launched = true;                                                                                           \
    }
    CD_CASE(16, 1) CD_CASE(16, 2) CD_CASE(16, 4) CD_CASE(16, 8) CD_CASE(32, 8) CD_CASE(32, 16) CD_CASE(32, 32)
#undef CD_CASE
    GB_REQUIRE(launched, "gb_channel_delta: no kernel for a key size of %d", dk);
    return gb_check_launch("gb_channel_delta");
}

// ----------------------------------------------------------------------------------------------
// Linear attention with a FIXED decay per head over long portions, cut into pieces. With g constant the state after a piece
// is g^L S_start + B, where B (the piece's own sum of g^(L-1-j) k_j v_j^T) does not depend on S_start, and a token's read-out
// is its read-out from a zero state at the piece's start plus g^(i+1) q^T S_start (i its index in the piece). So the pieces of
// a request walk side by side, each from zero (the kernel above, one "sequence" per piece, into a scratch state per piece),
// a second kernel chains the pieces' states (an element of S per thread: S_start of every piece replaces its B, the request's
// slot receives the last), and a third adds q^T S_start to the read-outs as a small float32 product per piece. The chain of
// dependent updates is one piece long instead of one portion long. Float32 throughout; only the order of the sums differs
// from the walk over the whole portion.
// ----------------------------------------------------------------------------------------------
// meta: piece_first_row [P + 1] | piece_start [P] (0, or -1 for an unused piece) | piece_slot [P] (= its index) | piece_seq [P] |
//       seq_piece_lo [S] | seq_piece_hi [S] (a request's pieces; empty for a padding sequence)
__global__ void lin_pieces_plan_kernel(const int* __restrict__ seq_first_row, const int* __restrict__ seq_start_pos, int S, int P,
                                       int piece_len, int* __restrict__ meta) {
    gb_pdl_launch_dependents();
    gb_pdl_wait();
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    int* first = meta, *start = meta + P + 1, *slot = start + P, *pseq = slot + P, *piece_lo = pseq + P, *piece_hi = piece_lo + S;
    int p = 0, last_row = 0;
    for (int s = 0; s < S; ++s) {
        const int r0 = seq_first_row[s], r1 = seq_first_row[s + 1];
        const int p_before = p;
        if (r1 > r0) last_row = r1;
        // the pieces tile the step's rows: a padding sequence's rows are one unused piece
        const bool live = seq_start_pos[s] >= 0;
        for (int r = r0; r < r1 && p < P; r += live ? piece_len : r1 - r0) {
            first[p] = r;
            start[p] = live ? 0 : -1;
            slot[p] = p;
            pseq[p] = s;
            ++p;
        }
        piece_lo[s] = live ? p_before : p;       // (a padding sequence's piece belongs to no request)
        piece_hi[s] = p;
    }
    for (int i = p; i < P; ++i) { first[i] = last_row; start[i] = -1; slot[i] = i; pseq[i] = 0; }
    first[P] = last_row;
}

// the rows of piece p end where piece p + 1 begins
__device__ __forceinline__ int lin_piece_end(const int* __restrict__ meta, int P, const int* __restrict__ seq_first_row, int p) {
    return meta[p + 1];
}

__global__ void __launch_bounds__(256) lin_chain_kernel(const int* __restrict__ meta, int P, const int* __restrict__ seq_first_row,
                                                        const int* __restrict__ seq_start_pos, const int* __restrict__ seq_slots,
                                                        const float* __restrict__ decay, float* __restrict__ piece_state,
                                                        float* __restrict__ state, long long state_stride, int S, int heads, int numbers,
                                                        int num_slots, int write_state) {
    gb_pdl_launch_dependents();
    gb_pdl_wait();
    const int seq = blockIdx.x, head = blockIdx.y;
    const int e = blockIdx.z * 256 + threadIdx.x;           // an element of the head's S
    if (seq >= S || e >= numbers || seq_start_pos[seq] < 0) return;
    const int slot = seq_slots[seq];
    if (slot < 0 || slot >= num_slots) return;
    const int* first = meta, *piece_lo = meta + 4 * P + 1, *piece_hi = piece_lo + S;
    float* mine = state + (size_t)slot * state_stride + (size_t)head * numbers + e;
    float s = *mine;
    const float g = decay[head];
    // eight pieces at a time: their own sums and lengths are all asked for before the chain through them starts
    for (int p0 = piece_lo[seq]; p0 < piece_hi[seq]; p0 += 8) {
        float own[8], f[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int p = min(p0 + u, piece_hi[seq] - 1);
            own[u] = piece_state[((size_t)p * heads + head) * numbers + e];
            f[u] = powf(g, (float)(lin_piece_end(meta, P, seq_first_row, p) - first[p]));
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            if (p0 + u >= piece_hi[seq]) break;
            piece_state[((size_t)(p0 + u) * heads + head) * numbers + e] = s;      // the state this piece starts from
            s = fmaf(f[u], s, own[u]);
        }
    }
    if (write_state) *mine = s;
}

constexpr int LC_ROWS = 128, LC_COLS = 64, LC_K = 32;

__global__ void __launch_bounds__(256) lin_carry_kernel(const float* __restrict__ qkv, long long ldq, const int* __restrict__ meta, int P,
                                                        const int* __restrict__ seq_first_row, const float* __restrict__ decay,
                                                        const float* __restrict__ piece_state, float* __restrict__ out, int heads, int dk,
                                                        int dv, int piece_len, int silu_in) {
    __shared__ float qs[LC_ROWS][LC_K + 1];
    __shared__ float ss[LC_K][LC_COLS];
    gb_pdl_launch_dependents();
    gb_pdl_wait();
    const int p = blockIdx.x, head = blockIdx.y, c0 = blockIdx.z * LC_COLS;
    const int* first = meta, *start = meta + P + 1;
    if (start[p] < 0) return;
    const int r0 = first[p], rows = lin_piece_end(meta, P, seq_first_row, p) - r0;
    const float* S0 = piece_state + ((size_t)p * heads + head) * dk * dv;
    const float g = decay[head];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;          // 16 x 16 threads: 4 columns x 8 rows each
    for (int rb = 0; rb < rows; rb += LC_ROWS) {
        float acc[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
        for (int k0 = 0; k0 < dk; k0 += LC_K) {
            __syncthreads();
            for (int idx = threadIdx.x; idx < LC_ROWS * LC_K; idx += 256) {
                const int r = idx / LC_K, d = idx % LC_K;
                float v = 0.f;
                if (rb + r < rows && k0 + d < dk) {
                    v = qkv[(size_t)(r0 + rb + r) * ldq + (size_t)head * dk + k0 + d];
                    if (silu_in) v = cd_silu(v);
                }
                qs[r][d] = v;
            }
            for (int idx = threadIdx.x; idx < LC_K * LC_COLS; idx += 256) {
                const int d = idx / LC_COLS, c = idx % LC_COLS;
                ss[d][c] = (k0 + d < dk && c0 + c < dv) ? S0[(size_t)(k0 + d) * dv + c0 + c] : 0.f;
            }
            __syncthreads();
#pragma unroll 4
            for (int d = 0; d < LC_K; ++d) {
                const float4 sv = *reinterpret_cast<const float4*>(&ss[d][tx * 4]);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float qv = qs[ty * 8 + i][d];
                    acc[i][0] = fmaf(qv, sv.x, acc[i][0]);
                    acc[i][1] = fmaf(qv, sv.y, acc[i][1]);
                    acc[i][2] = fmaf(qv, sv.z, acc[i][2]);
                    acc[i][3] = fmaf(qv, sv.w, acc[i][3]);
                }
            }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int r = rb + ty * 8 + i;
            if (r >= rows) continue;
            const float f = powf(g, (float)(r + 1));
            float* dst = out + (size_t)(r0 + r) * heads * dv + (size_t)head * dv + c0 + tx * 4;
#pragma unroll
            for (int c = 0; c < 4; ++c)
                if (c0 + tx * 4 + c < dv) dst[c] = fmaf(f, acc[i][c], dst[c]);
        }
    }
}

// meta: int32 [4 * P + 2 * S + 1]; piece_state: float32 [P, heads * dk * dv]. P must be at least n / piece_len + S.
GB_EXPORT int gb_decay_linear_pieces(const float* qkv, long long ldq, const float* decay, float* state, long long state_stride, float* out,
                                     const int* seq_first_row, const int* seq_start_pos, const int* seq_slots, int S, int n, int heads,
                                     int dk, int dv, int num_slots, int write_state, int* status, int silu_in, int piece_len, int P,
                                     int* meta, float* piece_state, cudaStream_t stream) {
    GB_REQUIRE(S >= 0 && n >= 0 && heads > 0 && dk > 0 && dk <= 1024 && dv > 0 && piece_len >= 16, "gb_decay_linear_pieces: bad sizes");
    GB_REQUIRE(P >= n / piece_len + S && meta && piece_state, "gb_decay_linear_pieces: %d pieces are too few for %d rows of %d requests",
               P, n, S);
    if (S == 0 || n == 0) return 0;
    const size_t numbers = (size_t)dk * dv;
    if (cudaMemsetAsync(piece_state, 0, (size_t)P * heads * numbers * sizeof(float), stream) != cudaSuccess)
        GB_REQUIRE(false, "gb_decay_linear_pieces: clearing the pieces' states failed");
    gb_launch(GB_PDL_ELEMENTWISE, lin_pieces_plan_kernel, dim3(1), dim3(32), 0, stream, seq_first_row, seq_start_pos, S, P, piece_len, meta);
    int rc = gb_check_launch("gb_decay_linear_pieces (plan)");
    if (rc) return rc;
    const int* first = meta, *start = meta + P + 1, *slot = start + P;
    rc = gb_channel_delta(qkv, ldq, nullptr, 0, nullptr, 0, nullptr, decay, piece_state, (long long)(heads * numbers), out, first, start, slot,
                          P, heads, heads, dk, dv, P, 1, status, 1, CD_PLAIN | (silu_in ? CD_SILU_INPUTS : 0), stream);
    if (rc) return rc;
    gb_launch(GB_PDL_ELEMENTWISE, lin_chain_kernel, dim3(S, heads, gb_ceil_div((long long)numbers, 256)), dim3(256), 0, stream,
              (const int*)meta, P, seq_first_row, seq_start_pos, seq_slots, decay, piece_state, state, state_stride, S, heads, (int)numbers,
              num_slots, write_state);
    rc = gb_check_launch("gb_decay_linear_pieces (chain)");
    if (rc) return rc;
    gb_launch(GB_PDL_ELEMENTWISE, lin_carry_kernel, dim3(P, heads, gb_ceil_div(dv, LC_COLS)), dim3(256), 0, stream, qkv, ldq,
              (const int*)meta, P, seq_first_row, decay, (const float*)piece_state, out, heads, dk, dv, piece_len, silu_in);
    return gb_check_launch("gb_decay_linear_pieces (carry)");
}

// ----------------------------------------------------------------------------------------------
// The same recurrence for steps in which every request brings ONE token (decoding): the work is reading and writing
// S once, so the layout is chosen for that. One block per (request, head), eight warps; warp w owns rows
// 16 w .. 16 w + 15 of S and lane l the columns l, l + 32, l + 64, l + 96: every load and store of a warp is a row
// segment of 128 contiguous bytes, and all 64 loads of a thread are asked for before anything else happens. The two
// sums over the key dimension cross the warps through shared memory. The read-out's norm and gate are applied here
// too (the block holds the whole head): the output is the mixer's activation, ready for its output projection.
// Key and value sizes up to 128.
// ----------------------------------------------------------------------------------------------
// What the fused form reads instead of finished q, k, v, decay logits and gate logits: the stacked projection's raw row
// (q | k | v channels before their convolutions, then the low-rank inputs of the decay and of the gate), the
// convolutions' weights and last inputs, and the two second-level matrices.
struct DeltaDecodeFusion {
    const float* proj;       // [n, ldp]
    long long ldp;
    const float* conv_w;     // [channels, taps]
    long long conv_state_off;
    int taps, channels, a1_at, ra, rg;      // the gate's low-rank input follows the decay's
    const void* w_a2;        // [heads * dk, ra]
    const void* w_g2;        // [heads * dv, rg]
};
constexpr int CD_MAX_LOW_RANK = 512;        // ra + rg

template <typename TW>
__device__ __forceinline__ float cd_dot_row(const TW* __restrict__ w, const float* __restrict__ x, int n) {
    float acc = 0.f;
    for (int i = 0; i < n; ++i) acc = fmaf(gb_to_float(w[i]), x[i], acc);
    return acc;
}
template <>
__device__ __forceinline__ float cd_dot_row<__nv_bfloat16>(const __nv_bfloat16* __restrict__ w, const float* __restrict__ x, int n) {
    float a0 = 0.f, a1 = 0.f;
    int i = 0;
    if ((((uintptr_t)w) & 15) == 0) {
        for (; i + 8 <= n; i += 8) {        // eight weights per load
            const uint4 v = *reinterpret_cast<const uint4*>(w + i);
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                a0 = fmaf(__low2float(h[j]), x[i + 2 * j], a0);
                a1 = fmaf(__high2float(h[j]), x[i + 2 * j + 1], a1);
            }
        }
    }
    for (; i < n; ++i) a0 = fmaf(__bfloat162float(w[i]), x[i], a0);
    return a0 + a1;
}

// One causal convolution output for a single new token: the slot's taps - 1 last inputs, then the token's own.
__device__ __forceinline__ float cd_conv_one(const DeltaDecodeFusion& f, const float* __restrict__ st, size_t row, int ch) {
    float acc = f.conv_w[(size_t)ch * f.taps + f.taps - 1] * f.proj[row * f.ldp + ch];
    for (int j = 0; j < f.taps - 1; ++j) acc = fmaf(f.conv_w[(size_t)ch * f.taps + j], st[(size_t)j * f.channels + ch], acc);
    return acc / (1.0f + expf(-acc));
}

// FUSED: the convolutions of q, k, v (reading the slot's last inputs; the shift is left to the kernel that follows)
// and the two low-rank second-level products are computed here, from the stacked projection's row.
template <typename T, typename TW, bool FUSED>
__global__ void __launch_bounds__(256) channel_delta_decode_kernel(ChannelDeltaArgs p, const float* __restrict__ gate, long long ldg,
                                                                   const float* __restrict__ norm_w, float eps, T* __restrict__ att,
                                                                   DeltaDecodeFusion f) {
    __shared__ float qs[128], ks[128], gs[128], part[8][128], ovec[128], red[16], vsm[128], gsm[128];
    __shared__ float lr[FUSED ? CD_MAX_LOW_RANK : 1];
    gb_pdl_launch_dependents();
    gb_pdl_wait();
    const int seq = blockIdx.x, head = blockIdx.y;
    if (p.seq_start_pos[seq] < 0) return;
    const int slot = p.seq_slots[seq];
    if (slot < 0 || slot >= p.num_slots) {
        if (threadIdx.x == 0) atomicOr(p.status, GB_STATUS_BAD_SLOT);
        return;
    }
    const size_t row = (size_t)p.seq_first_row[seq];
    const int dk = p.dk, dv = p.dv;
    const bool plain = p.flags & CD_PLAIN, silu_in = p.flags & CD_SILU_INPUTS;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
    const int kvh = head / (p.heads / p.kv_heads);
    float* sbase = p.state + (size_t)slot * p.state_stride + (size_t)head * dk * dv;
    float S[16][4];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const int d = warp * 16 + i;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int col = lane + 32 * c;
            S[i][c] = (d < dk && col < dv) ? sbase[(size_t)d * dv + col] : 0.f;
        }
    }
    // the token's vectors: thread d takes key channel d
    float qv = 0.f, kv = 0.f, zv = -1e30f;
    float vt[4];
    if (FUSED) {
        for (int i = tid; i < f.ra + f.rg; i += 256) lr[i] = f.proj[row * f.ldp + f.a1_at + i];
        __syncthreads();
        const float* st = p.state + (size_t)slot * p.state_stride + f.conv_state_off;
        if (tid < dk) {
            qv = cd_conv_one(f, st, row, kvh * dk + tid);
            kv = cd_conv_one(f, st, row, (p.kv_heads + kvh) * dk + tid);
            zv = cd_dot_row(reinterpret_cast<const TW*>(f.w_a2) + ((size_t)head * dk + tid) * f.ra, lr, f.ra) +
                 p.dt_bias[(size_t)head * dk + tid];
        } else if (tid >= 128 && tid - 128 < dv) {      // the other half of the block: values and gate logits
            const int j = tid - 128;
            vsm[j] = cd_conv_one(f, st, row, 2 * p.kv_heads * dk + head * dv + j);
            gsm[j] = cd_dot_row(reinterpret_cast<const TW*>(f.w_g2) + ((size_t)head * dv + j) * f.rg, lr + f.ra, f.rg);
        }
    } else {
        if (tid < dk) {
            const size_t ai = (size_t)head * p.decay_channels + (p.decay_channels > 1 ? tid : 0);
            qv = p.qkv[row * p.ldq + (size_t)kvh * dk + tid];
            kv = p.qkv[row * p.ldq + (size_t)(p.kv_heads + kvh) * dk + tid];
            if (!plain) zv = p.a[row * p.lda + ai] + p.dt_bias[ai];
            if (silu_in) { qv = cd_silu(qv); kv = cd_silu(kv); }
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int col = lane + 32 * c;
            vt[c] = col < dv ? p.qkv[row * p.ldq + (size_t)2 * p.kv_heads * dk + (size_t)head * dv + col] : 0.f;
            if (silu_in) vt[c] = cd_silu(vt[c]);
        }
    }
    const float beta = plain ? 1.0f : 1.0f / (1.0f + __expf(-p.beta[row * p.ldb + head]));
    if (tid < 128) {
        const float sp = zv > 15.f ? zv : __logf(1.0f + __expf(zv));
        qs[tid] = qv;
        ks[tid] = kv;
        gs[tid] = plain ? (tid < dk ? p.a_log[head] : 1.0f) : __expf(-expf(p.a_log[head]) * sp);
        const float sq = gb_warp_sum(qv * qv), sk = gb_warp_sum(kv * kv);
        if (lane == 0) { red[warp] = sq; red[4 + warp] = sk; }
    }
    __syncthreads();
    if (FUSED) {
#pragma unroll
        for (int c = 0; c < 4; ++c) vt[c] = lane + 32 * c < dv ? vsm[lane + 32 * c] : 0.f;
    }
    const float iq = plain ? 1.0f : 1.0f / sqrtf((float)dk) / sqrtf(red[0] + red[1] + red[2] + red[3] + CD_UNIT_EPS);
    const float ik = plain ? 1.0f : 1.0f / sqrtf(red[4] + red[5] + red[6] + red[7] + CD_UNIT_EPS);
    const float corr = plain ? 0.f : 1.f;               // how much of S^T k is taken off the value
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const float g = gs[warp * 16 + i], k = ks[warp * 16 + i];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            S[i][c] *= g;
            acc[c] = fmaf(S[i][c], k, acc[c]);
        }
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) part[warp][lane + 32 * c] = acc[c];
    __syncthreads();
    float u[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        const int col = lane + 32 * c;
        float sk = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) sk += part[w][col];
        u[c] = beta * (vt[c] - corr * ik * sk) * ik;
        acc[c] = 0.f;
    }
    __syncthreads();           // everyone has read the first sums before the second ones overwrite them
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const float k = ks[warp * 16 + i], q = qs[warp * 16 + i];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            S[i][c] = fmaf(k, u[c], S[i][c]);
            acc[c] = fmaf(S[i][c], q, acc[c]);
        }
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) part[warp][lane + 32 * c] = acc[c];
    if (p.write_state) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int d = warp * 16 + i;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int col = lane + 32 * c;
                if (d < dk && col < dv) sbase[(size_t)d * dv + col] = S[i][c];
            }
        }
    }
    __syncthreads();
    if (tid < 128) {
        float o = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) o += part[w][tid];
        o = tid < dv ? o * iq : 0.f;
        ovec[tid] = o;
        const float ss = gb_warp_sum(o * o);
        if (lane == 0) red[8 + warp] = ss;
    }
    __syncthreads();
    if (p.flags & CD_NO_NORM) {
        if (tid < dv) p.out[row * p.heads * dv + (size_t)head * dv + tid] = ovec[tid];
    } else if (tid < dv) {
        const float s = 1.0f / sqrtf((red[8] + red[9] + red[10] + red[11]) / (float)dv + eps);
        const float gl = FUSED ? gsm[tid] : gate[row * ldg + (size_t)head * dv + tid];
        const float sig = (p.flags & CD_GATE_SILU) ? cd_silu(gl) : 1.0f / (1.0f + expf(-gl));
        att[row * p.heads * dv + (size_t)head * dv + tid] = gb_from_float<T>(ovec[tid] * s * norm_w[tid] * sig);
    }
}

GB_EXPORT int gb_channel_delta_decode_supported(int dk, int dv) { return dk > 0 && dk <= 128 && dv > 0 && dv <= 128; }

// Every sequence of the step brings exactly one row. att: [n, heads * dv] in `att_dtype`, the gated and normed read-out.
// With proj != nullptr the fused form runs: qkv, a and gate are not read; the convolutions (without the shift of the
// slot's last inputs: gb_short_conv_state does that afterwards) and the low-rank products are computed in the kernel
// from the stacked projection `proj` (columns: conv channels, then at `a1_at` the decay's and the gate's low-rank inputs).
GB_EXPORT int gb_channel_delta_decode(const float* qkv, long long ldq, const float* beta, long long ldb, const float* a, long long lda,
                                      const float* dt_bias, const float* a_log, float* state, long long state_stride,
                                      const float* gate, long long ldg, const float* norm_w, float eps, void* att, int att_dtype,
                                      const int* seq_first_row, const int* seq_start_pos, const int* seq_slots, int S, int heads,
                                      int kv_heads, int dk, int dv, int num_slots, int write_state, int* status,
                                      const float* proj, long long ldp, const float* conv_w, long long conv_state_off, int taps,
                                      int a1_at, int ra, int rg, const void* w_a2, const void* w_g2, int w_dtype,
                                      int decay_channels, int flags, cudaStream_t stream) {
    GB_REQUIRE(decay_channels == 1 || decay_channels == dk, "gb_channel_delta_decode: %d decays per head", decay_channels);
    GB_REQUIRE(proj == nullptr || (decay_channels == dk && flags == 0), "gb_channel_delta_decode: the fused form wants a decay per key "
               "channel and no flags");
    GB_REQUIRE(!(flags & CD_NO_NORM) || att_dtype == GB_F32, "gb_channel_delta_decode: a read-out without its norm is float32");
    GB_REQUIRE(S >= 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0, "gb_channel_delta_decode: heads %d must be a multiple of "
               "key heads %d", heads, kv_heads);
    GB_REQUIRE(gb_channel_delta_decode_supported(dk, dv), "gb_channel_delta_decode: key size %d and value size %d must be at most 128", dk, dv);
    const bool fused = proj != nullptr;
    GB_REQUIRE(!fused || (ra > 0 && rg > 0 && ra + rg <= CD_MAX_LOW_RANK && taps >= 1 && conv_w && w_a2 && w_g2),
               "gb_channel_delta_decode: the fused form takes low ranks up to %d in all", CD_MAX_LOW_RANK);
    if (S == 0) return 0;
    ChannelDeltaArgs p = {qkv, ldq, beta, ldb, a, lda, dt_bias, a_log, state, state_stride, nullptr, seq_first_row, seq_start_pos,
                          seq_slots, heads, kv_heads, dk, dv, 0, 0, num_slots, write_state, status, decay_channels, flags};
    if (flags & CD_NO_NORM) p.out = (float*)att;
    DeltaDecodeFusion f = {proj, ldp, conv_w, conv_state_off, taps, 2 * kv_heads * dk + heads * dv, a1_at, ra, rg, w_a2, w_g2};
    dim3 grid(S, heads);
#define CDD_LAUNCH(T, TW, F) gb_launch(GB_PDL_ATTENTION, channel_delta_decode_kernel<T, TW, F>, grid, dim3(256), 0, stream, p, gate, ldg, \
                                        norm_w, eps, (T*)att, f)
    if (att_dtype != GB_F32 && att_dtype != GB_BF16) GB_REQUIRE(false, "gb_channel_delta_decode: unsupported output dtype %d", att_dtype);
    if (!fused) {
        if (att_dtype == GB_F32) CDD_LAUNCH(float, float, false);
        else CDD_LAUNCH(__nv_bfloat16, float, false);
    } else if (w_dtype == GB_F32) {
        if (att_dtype == GB_F32) CDD_LAUNCH(float, float, true);
        else CDD_LAUNCH(__nv_bfloat16, float, true);
    } else if (w_dtype == GB_BF16) {
        if (att_dtype == GB_F32) CDD_LAUNCH(float, __nv_bfloat16, true);
        else CDD_LAUNCH(__nv_bfloat16, __nv_bfloat16, true);
    } else {
        GB_REQUIRE(false, "gb_channel_delta_decode: unsupported weight dtype %d", w_dtype);
    }
#undef CDD_LAUNCH
    return gb_check_launch("gb_channel_delta_decode");
}

// The shift-and-append of the convolutions' last inputs alone (after a kernel that computed the convolutions itself).
GB_EXPORT int gb_short_conv_state(const float* x, long long ldx, float* state, long long state_stride, long long state_off,
                                  const int* seq_first_row, const int* seq_start_pos, const int* seq_slots, int S, int C, int taps,
                                  int num_slots, cudaStream_t stream) {
    GB_REQUIRE(S >= 0 && C > 0 && taps >= 1 && taps <= 64, "gb_short_conv_state: bad sizes (taps %d)", taps);
    if (S == 0 || taps == 1) return 0;
    dim3 grid(S, gb_ceil_div(C, 256));
    gb_launch(GB_PDL_ELEMENTWISE, short_conv_state_kernel, grid, dim3(256), 0, stream, x, ldx, state, state_stride, state_off,
              seq_first_row, seq_start_pos, seq_slots, S, C, taps, num_slots);
    return gb_check_launch("gb_short_conv_state");
}

// ----------------------------------------------------------------------------------------------
// A causal convolution added to its own input: y[t, c] = x[t, c] + sum_j w[c, j] x[t - (taps-1) + j, c] along each request's
// rows, x and y in the activation dtype, sums in float32. Inputs from before a portion's first row come from the request's
// slot (float32, [taps-1, C] from `state_off` on, oldest first; zeros for a fresh request); afterwards the slot keeps the
// portion's last taps-1 inputs. x and y must be different buffers (a row reads the rows before it).
// ----------------------------------------------------------------------------------------------
template <typename T, typename TW>
__global__ void __launch_bounds__(256) residual_conv_kernel(const T* __restrict__ x, const TW* __restrict__ w, T* __restrict__ y,
                                                            const float* __restrict__ state, long long state_stride, long long state_off,
                                                            const int* __restrict__ row_seq, const int* __restrict__ positions,
                                                            const int* __restrict__ seq_first_row, const int* __restrict__ seq_slots,
                                                            int n, int C, int taps, int num_slots, int shift_here,
                                                            int* __restrict__ status) {
    gb_pdl_launch_dependents();
    gb_pdl_wait();
    const int row = blockIdx.x;
    const int ch = blockIdx.y * blockDim.x + threadIdx.x;
    if (row >= n || ch >= C) return;
    if (positions[row] < 0) return;
    const int seq = row_seq[row];
    const int r0 = seq_first_row[seq];
    const int slot = seq_slots[seq];
    if (slot < 0 || slot >= num_slots) {
        atomicOr(status, GB_STATUS_BAD_SLOT);
        return;
    }
    float* st = const_cast<float*>(state) + (size_t)slot * state_stride + state_off;
    float acc = 0.f;
    for (int j = 0; j < taps; ++j) {
        const int src = row - (taps - 1) + j;
        const float v = src >= r0 ? gb_to_float(x[(size_t)src * C + ch]) : st[(size_t)(taps - 1 - (r0 - src)) * C + ch];
        acc = fmaf(gb_to_float(w[(size_t)ch * taps + j]), v, acc);
    }
    const float own = gb_to_float(x[(size_t)row * C + ch]);
    y[(size_t)row * C + ch] = gb_from_float<T>(own + acc);
    if (shift_here) {
        // every request brings one row: this thread is the only reader of its channel's last inputs, so it moves them up itself
        for (int i = 0; i + 2 < taps; ++i) st[(size_t)i * C + ch] = st[(size_t)(i + 1) * C + ch];
        if (taps > 1) st[(size_t)(taps - 2) * C + ch] = own;
    }
}

template <typename T>
__global__ void __launch_bounds__(256) residual_conv_state_kernel(const T* __restrict__ x, float* __restrict__ state, long long state_stride,
                                                                  long long state_off, const int* __restrict__ seq_first_row,
                                                                  const int* __restrict__ seq_start_pos, const int* __restrict__ seq_slots,
                                                                  int S, int C, int taps, int num_slots) {
    gb_pdl_launch_dependents();
    gb_pdl_wait();
    const int seq = blockIdx.x;
    const int ch = blockIdx.y * blockDim.x + threadIdx.x;
    if (seq >= S || ch >= C) return;
    if (seq_start_pos[seq] < 0) return;
    const int slot = seq_slots[seq];
    if (slot < 0 || slot >= num_slots) return;
    const int r0 = seq_first_row[seq], len = seq_first_row[seq + 1] - r0;
    float* st = state + (size_t)slot * state_stride + state_off;
    const int keep = taps - 1;
    for (int i = 0; i < keep; ++i) {      // increasing i: a kept value moves to a lower index than any still to be read
        const int p = len - keep + i;
        st[(size_t)i * C + ch] = p >= 0 ? gb_to_float(x[(size_t)(r0 + p) * C + ch]) : st[(size_t)(i + len) * C + ch];
    }
}

template <typename T, typename TW>
static int residual_conv_launch(const void* x, const void* w, void* y, float* state, long long state_stride, long long state_off,
                                const int* row_seq, const int* positions, const int* seq_first_row, const int* seq_start_pos,
                                const int* seq_slots, int n, int S, int C, int taps, int num_slots, int update_state, int* status,
                                cudaStream_t stream) {
    // update_state 2: every request brings exactly one row, and the kernel that reads the last inputs also moves them up
    dim3 grid(n, gb_ceil_div(C, 256));
    gb_launch(GB_PDL_ELEMENTWISE, residual_conv_kernel<T, TW>, grid, dim3(256), 0, stream, (const T*)x, (const TW*)w, (T*)y,
              (const float*)state, state_stride, state_off, row_seq, positions, seq_first_row, seq_slots, n, C, taps, num_slots,
              update_state == 2 ? 1 : 0, status);
    int rc = gb_check_launch("gb_residual_conv");
    if (rc || update_state != 1 || taps == 1) return rc;
    dim3 grid2(S, gb_ceil_div(C, 256));
    gb_launch(GB_PDL_ELEMENTWISE, residual_conv_state_kernel<T>, grid2, dim3(256), 0, stream, (const T*)x, state, state_stride, state_off,
              seq_first_row, seq_start_pos, seq_slots, S, C, taps, num_slots);
    return gb_check_launch("gb_residual_conv (state)");
}

GB_EXPORT int gb_residual_conv(const void* x, int dtype, const void* w, int w_dtype, void* y, float* state, long long state_stride,
                               long long state_off, const int* row_seq, const int* positions, const int* seq_first_row,
                               const int* seq_start_pos, const int* seq_slots, int n, int S, int C, int taps, int num_slots,
                               int update_state, int* status, cudaStream_t stream) {
    GB_REQUIRE(n >= 0 && S >= 0 && C > 0 && taps >= 1 && taps <= 64 && x != y, "gb_residual_conv: bad sizes (taps %d)", taps);
    if (n == 0 || S == 0) return 0;
#define RC_ARGS x, w, y, state, state_stride, state_off, row_seq, positions, seq_first_row, seq_start_pos, seq_slots, n, S, C, taps, \
                num_slots, update_state, status, stream
    if (dtype == GB_F32 && w_dtype == GB_F32) return residual_conv_launch<float, float>(RC_ARGS);
    if (dtype == GB_BF16 && w_dtype == GB_BF16) return residual_conv_launch<__nv_bfloat16, __nv_bfloat16>(RC_ARGS);
    if (dtype == GB_BF16 && w_dtype == GB_F32) return residual_conv_launch<__nv_bfloat16, float>(RC_ARGS);
#undef RC_ARGS
    GB_REQUIRE(false, "gb_residual_conv: unsupported dtypes %d / %d", dtype, w_dtype);
}
