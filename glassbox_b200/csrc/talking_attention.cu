// Softmax attention whose heads exchange their weights after the softmax ("talking heads"), over the paged cache.
//
// For a row at position p of its request, query head g and a key at position j <= p (inside the window, if there is one):
//     s_j = q_g . k_j * scale;   s_j <- cap * tanh(s_j / cap)  (cap > 0)
//     w_g(j) = exp(s_j) / (unit + sum_j' exp(s_j'))             unit = 1: a key of score 0 that has no value; unit = 0: none
// and head h's output is sum_j (sum_g talk[h, g] w_g(j)) v_c(h)(j), c(h) the key/value head of h. Because the mix is linear,
//     out_h = sum_g talk[h, g] * O[g, c(h)],      O[g, c] = sum_j w_g(j) v_c(j):
// every query head's weights are applied to the values of ALL key/value heads in one pass with the usual running maximum
// (the attention kernels below, which leave O as float32 [n, heads, kv heads, vdim]), and a small kernel mixes the results
// (talk_combine). The sink's share is never mixed: it has no value. Scores, weights, sums and the mix are float32.
//
//   bias_rope_write        from the float32 sums of the stacked projection q | k | v: biases, rotation of the leading
//                          channels (channel i with channel i + rot/2, a (cos, sin) table per position), q into the query
//                          buffer, k and v into the paged cache at each row's slot
//   talking_attention_rows one warp per (row, head), any row, both dtypes
//   talking_attention_decode  single decoded tokens: a block of 8 warps per (row, heads of a group, share of the keys)
//   talking_attention_tiles   prompt portions in bfloat16 on the tensor cores (mma.sync), 64 rows x one head per block
//   talk_combine           the mix of the heads' results (and the merge of the shares of the keys, if there are several)
#include "common.cuh"
#include "paged_rows.cuh"

constexpr int TK_WARPS = 4;
constexpr int TK_MAX_WIDE = 2048;        // kv heads * vdim at most

__device__ __forceinline__ float tk_cap(float s, float cap, float inv_cap) { return cap > 0.f ? cap * tanhf(s * inv_cap) : s; }

// ----------------------------------------------------------------------------------------------
// One thread per (row, head slot, channel pair or single channel). Heads 0..H-1 are queries, H..H+G-1 keys, then G values.
// ----------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) bias_rope_write_kernel(const float* __restrict__ qkv, long long ld, const float* __restrict__ bias,
                                                              const float* __restrict__ cos_sin, int max_position,
                                                              const int* __restrict__ positions, const int* __restrict__ slots,
                                                              T* __restrict__ q_out, T* __restrict__ kcache, T* __restrict__ vcache,
                                                              int n, int H, int G, int D, int V, int rot, int page_size,
                                                              long long num_slots, int write_kv, int* __restrict__ status) {
    gb_pdl_launch_dependents();
    gb_pdl_wait();
    const int row = blockIdx.x;
    if (row >= n) return;
    const int pos = positions[row];
    if (pos < 0) return;
    if (rot > 0 && pos >= max_position) {
        if (threadIdx.x == 0) atomicOr(status, GB_STATUS_BAD_POSITION);
        return;
    }
    const long long slot = slots[row];
    const bool slot_ok = slot >= 0 && slot < num_slots;
    if (write_kv && !slot_ok && threadIdx.x == 0) atomicOr(status, GB_STATUS_BAD_SLOT);
    const float* src = qkv + (size_t)row * ld;
    const int half = rot / 2;
    const int qk_cols = (H + G) * D, total = qk_cols + G * V;
    const long long page = slot / page_size, off = slot % page_size;
    for (int c = threadIdx.x; c < total; c += blockDim.x) {
        float val = src[c] + (bias ? bias[c] : 0.f);
        if (c < qk_cols) {
            const int head = c / D, i = c % D;
            if (i < rot) {
                const int pair = i < half ? i : i - half;
                const int other = i < half ? c + half : c - half;
                const float ov = src[other] + (bias ? bias[other] : 0.f);
                const float cs = cos_sin[((size_t)pos * half + pair) * 2], sn = cos_sin[((size_t)pos * half + pair) * 2 + 1];
                // (u, v) -> (u cos - v sin, v cos + u sin)
                val = i < half ? val * cs - ov * sn : val * cs + ov * sn;
            }
            if (head < H) q_out[((size_t)row * H + head) * D + i] = gb_from_float<T>(val);
            else if (write_kv && slot_ok) kcache[((page * G + (head - H)) * page_size + off) * D + i] = gb_from_float<T>(val);
        } else if (write_kv && slot_ok) {
            const int head = (c - qk_cols) / V, i = (c - qk_cols) % V;
            vcache[((page * G + head) * page_size + off) * V + i] = gb_from_float<T>(val);
        }
    }
}

GB_EXPORT int gb_bias_rope_write(const float* qkv, long long ld, const float* bias, const float* cos_sin, int max_position,
                                 const int* positions, const int* slots, void* q_out, void* kcache, void* vcache, int dtype, int n,
                                 int H, int G, int D, int V, int rot, int page_size, long long num_slots, int write_kv, int* status,
                                 cudaStream_t stream) {
    GB_REQUIRE(n >= 0 && H > 0 && G > 0 && D > 0 && V > 0 && rot >= 0 && rot <= D && rot % 2 == 0,
               "gb_bias_rope_write: bad sizes (rot %d of %d)", rot, D);
    GB_REQUIRE(rot == 0 || cos_sin != nullptr, "gb_bias_rope_write: a rotation needs its table");
    if (n == 0) return 0;
    if (dtype == GB_F32)
        gb_launch(GB_PDL_ELEMENTWISE, bias_rope_write_kernel<float>, dim3(n), dim3(256), 0, stream, qkv, ld, bias, cos_sin, max_position,
                  positions, slots, (float*)q_out, (float*)kcache, (float*)vcache, n, H, G, D, V, rot, page_size, num_slots, write_kv, status);
    else if (dtype == GB_BF16)
        gb_launch(GB_PDL_ELEMENTWISE, bias_rope_write_kernel<__nv_bfloat16>, dim3(n), dim3(256), 0, stream, qkv, ld, bias, cos_sin,
                  max_position, positions, slots, (__nv_bfloat16*)q_out, (__nv_bfloat16*)kcache, (__nv_bfloat16*)vcache, n, H, G, D, V, rot,
                  page_size, num_slots, write_kv, status);
    else
        GB_REQUIRE(false, "gb_bias_rope_write: unsupported dtype %d", dtype);
    return gb_check_launch("gb_bias_rope_write");
}

// ----------------------------------------------------------------------------------------------
// One warp per (row, head): 32 keys at a time from the first visible one, a lane per key for the scores, a lane per
// channel of the wide value row (VG key/value heads x V channels) for the sums. NC = ceil(VG * V / 32) rounded up.
// out: float32 [n, H, VG, V]. VG is G (every head's values) or 1 (the head's own key/value head only).
// ----------------------------------------------------------------------------------------------
template <typename T, int NC>
__global__ void __launch_bounds__(TK_WARPS * 32) talking_attention_rows_kernel(
    const T* __restrict__ q, float* __restrict__ out, const T* __restrict__ kcache, const T* __restrict__ vcache,
    const int* __restrict__ block_tables, int max_pages, const int* __restrict__ row_seq, const int* __restrict__ positions,
    int n, int H, int G, int D, int V, int VG, int page_size, long long num_pages, float scale, float cap, float unit, int window,
    int* __restrict__ status) {
    __shared__ float qs[TK_WARPS][SA_MAX_DIM];
    gb_pdl_launch_dependents();
    gb_pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long task = (long long)blockIdx.x * TK_WARPS + warp;
    if (task >= (long long)n * H) return;
    const int row = (int)(task / H), head = (int)(task % H);
    const int g = head / (H / G);
    const int pos = positions[row];
    if (pos < 0) return;
    if (pos / page_size >= max_pages) {
        if (lane == 0) atomicOr(status, GB_STATUS_BAD_POSITION);
        return;
    }
    const int* table = block_tables + (size_t)row_seq[row] * max_pages;
    const T* qrow = q + ((size_t)row * H + head) * D;
    for (int i = lane; i < D; i += 32) qs[warp][i] = gb_to_float(qrow[i]);
    __syncwarp();
    const float inv_cap = cap > 0.f ? 1.0f / cap : 0.f;
    const int first = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;
    const int wide = VG * V;
    // the unit in the denominator is exp(0 - m): the running maximum starts at its score
    float m = unit > 0.f ? 0.f : -INFINITY, l = unit > 0.f ? unit : 0.f;
    float acc[NC];
    int voff[NC];          // where this lane's channel j lies within a key's values: head * page_size * V + channel
#pragma unroll
    for (int j = 0; j < NC; ++j) {
        acc[j] = 0.f;
        const int i = lane + 32 * j;
        const int c = VG == 1 ? g : i / V;
        voff[j] = i < wide ? c * page_size * V + i % V : -1;
    }
    for (int base = first; base <= pos; base += 32) {
        const int key = base + lane;
        float s = -INFINITY;
        long long at = -1;                   // page * G * page_size + offset of this lane's key
        if (key <= pos) {
            const long long page = table[key / page_size];
            if (page < 0 || page >= num_pages) {
                atomicOr(status, GB_STATUS_BAD_SLOT);
            } else {
                at = page * G * page_size + key % page_size;
                s = tk_cap(sa_dot<T>(qs[warp], kcache + (at + (long long)g * page_size) * D, D) * scale, cap, inv_cap);
            }
        }
        const float m_new = fmaxf(m, gb_warp_max(s));
        if (m_new == -INFINITY) continue;
        const float corr = expf(m - m_new);
        const float p = at >= 0 ? expf(s - m_new) : 0.f;
        l = l * corr + gb_warp_sum(p);
        m = m_new;
#pragma unroll
        for (int j = 0; j < NC; ++j) acc[j] *= corr;
        const int count = min(32, pos - base + 1);
        for (int t = 0; t < count; ++t) {
            const float pt = __shfl_sync(0xffffffffu, p, t);
            const long long vr = __shfl_sync(0xffffffffu, at, t);
            if (vr < 0) continue;
            const T* vp = vcache + vr * V;
#pragma unroll
            for (int j = 0; j < NC; ++j)
                if (voff[j] >= 0) acc[j] = fmaf(pt, gb_to_float(vp[voff[j]]), acc[j]);
        }
    }
    const float f = l > 0.f ? 1.0f / l : 0.f;
    float* orow = out + ((size_t)row * H + head) * wide;
#pragma unroll
    for (int j = 0; j < NC; ++j) {
        const int i = lane + 32 * j;
        if (i < wide) orow[i] = acc[j] * f;
    }
}

#define TK_COMMON_CHECKS(name)                                                                                                          \
    GB_REQUIRE(n >= 0 && H > 0 && G > 0 && H % G == 0, name ": heads %d must be a multiple of kv heads %d", H, G);                      \
    GB_REQUIRE(D > 0 && D <= SA_MAX_DIM && V > 0 && V <= SA_MAX_DIM, name ": head sizes %d / %d are outside 1..%d", D, V, SA_MAX_DIM);  \
    GB_REQUIRE((VG == G || VG == 1) && VG * V <= TK_MAX_WIDE, name ": %d value heads of %d channels are more than %d numbers", VG, V,   \
               TK_MAX_WIDE);                                                                                                            \
    GB_REQUIRE(page_size > 0 && max_pages > 0 && window >= 0, name ": bad page geometry or window");

GB_EXPORT int gb_talking_attention_rows(const void* q, float* out, int dtype, const void* kcache, const void* vcache,
                                        const int* block_tables, int max_pages, const int* row_seq, const int* positions, int n, int H,
                                        int G, int D, int V, int VG, int page_size, long long num_pages, float scale, float cap,
                                        float unit, int window, int* status, cudaStream_t stream) {
    TK_COMMON_CHECKS("gb_talking_attention_rows")
    if (n == 0) return 0;
    const int blocks = gb_ceil_div((long long)n * H, TK_WARPS);
    int nc = 1;
    while (nc * 32 < VG * V) nc *= 2;
#define TK_ROWS(T, N)                                                                                                                   \
    gb_launch(GB_PDL_ATTENTION, talking_attention_rows_kernel<T, N>, dim3(blocks), dim3(TK_WARPS * 32), 0, stream, (const T*)q, out,    \
              (const T*)kcache, (const T*)vcache, block_tables, max_pages, row_seq, positions, n, H, G, D, V, VG, page_size, num_pages, \
              scale, cap, unit, window, status)
#define TK_ROWS_NC(T)                                                                                                                   \
    switch (nc) {                                                                                                                       \
        case 1: TK_ROWS(T, 1); break;                                                                                                   \
        case 2: TK_ROWS(T, 2); break;                                                                                                   \
        case 4: TK_ROWS(T, 4); break;                                                                                                   \
        case 8: TK_ROWS(T, 8); break;                                                                                                   \
        case 16: TK_ROWS(T, 16); break;                                                                                                 \
        case 32: TK_ROWS(T, 32); break;                                                                                                 \
        default: TK_ROWS(T, 64); break;                                                                                                 \
    }
    if (dtype == GB_F32) { TK_ROWS_NC(float) }
    else if (dtype == GB_BF16) { TK_ROWS_NC(__nv_bfloat16) }
    else GB_REQUIRE(false, "gb_talking_attention_rows: unsupported dtype %d", dtype);
#undef TK_ROWS_NC
#undef TK_ROWS
    return gb_check_launch("gb_talking_attention_rows");
}

// ----------------------------------------------------------------------------------------------
// Single decoded tokens: one block of 8 warps per (row, R query heads of one key/value group, share of the row's keys). The
// block's keys are taken 32 at a time by its warps in turn (warp w the chunks w, w + 8, ...): a lane reads "its" key once and
// dots it with the R queries; then the wide value rows of the 32 keys pass KB at a time, a lane per channel: the KB rows'
// loads are all asked for before the first is used (instructions issue in order: a loop that uses each row as it arrives
// pays the trip to memory once per key), each value multiplied into the R heads' sums. Every warp keeps a running maximum
// and a denominator per head of its own; the warps meet in shared memory (fixed order). With one share per row the unit of
// the denominator joins there and the result is final; with several, every share leaves its sums, its maximum and its
// denominator (part: [shares][n][H][wide], ml: [shares][n][H][2]) and talk_combine merges the shares on its way. The order of
// a row's sums depends on its position, the window and the number of shares. R * NC <= 32 (NC = 32-channel pieces of the wide
// value row).
// ----------------------------------------------------------------------------------------------
constexpr int TKD_WARPS = 8;

// NC consecutive bfloat16 channels of a value row as 32-bit words, in the widest pieces their alignment allows
template <int NC>
__device__ __forceinline__ void tkd_load_words(const __nv_bfloat16* __restrict__ p, unsigned (&w)[NC / 2]) {
    if constexpr (NC % 8 == 0) {
#pragma unroll
        for (int i = 0; i < NC / 8; ++i) {
            const uint4 v = reinterpret_cast<const uint4*>(p)[i];
            w[4 * i] = v.x; w[4 * i + 1] = v.y; w[4 * i + 2] = v.z; w[4 * i + 3] = v.w;
        }
    } else if constexpr (NC % 4 == 0) {
#pragma unroll
        for (int i = 0; i < NC / 4; ++i) {
            const uint2 v = reinterpret_cast<const uint2*>(p)[i];
            w[2 * i] = v.x; w[2 * i + 1] = v.y;
        }
    } else {
#pragma unroll
        for (int i = 0; i < NC / 2; ++i) w[i] = reinterpret_cast<const unsigned*>(p)[i];
    }
}

// VEC (bfloat16, wide == 32 * NC, V a multiple of NC): a lane owns the NC consecutive channels lane * NC .. of the wide value
// row and reads them with one to three loads per key; otherwise lane l owns the channels l, l + 32, ... and reads them one by one.
template <typename T, int R, int NC, bool VEC>
__global__ void __launch_bounds__(TKD_WARPS * 32) talking_attention_decode_kernel(
    const T* __restrict__ q, float* __restrict__ out, float* __restrict__ ml, const T* __restrict__ kcache, const T* __restrict__ vcache,
    const int* __restrict__ block_tables, int max_pages, const int* __restrict__ row_seq, const int* __restrict__ positions,
    int n, int H, int G, int D, int V, int VG, int page_size, long long num_pages, float scale, float cap, float unit, int window,
    int shares, int col_blocks, int* __restrict__ status) {
    constexpr int KB = (NC > 8 && !VEC) ? 4 : 8;       // value rows in flight together
    __shared__ float qs[R * SA_MAX_DIM];
    __shared__ float part[TKD_WARPS][R][NC * 32 + 2];
    gb_pdl_launch_dependents();
    gb_pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // a wide value row of more than 256 channels is cut into column blocks of 256 (each forms the scores again: a key row is
    // an eighth of a value row's bytes), so that R heads' sums of a block's columns fit a thread's registers
    const int row = blockIdx.x, head0 = blockIdx.y * R, share = blockIdx.z / col_blocks, cb = blockIdx.z % col_blocks;
    if (row >= n) return;
    const int g = head0 / (H / G);
    const int pos = positions[row];
    if (pos < 0) return;
    if (pos / page_size >= max_pages) {
        if (threadIdx.x == 0) atomicOr(status, GB_STATUS_BAD_POSITION);
        return;
    }
    const int* table = block_tables + (size_t)row_seq[row] * max_pages;
    for (int i = threadIdx.x; i < R * D; i += TKD_WARPS * 32) qs[i] = gb_to_float(q[((size_t)row * H + head0) * D + i]);
    __syncthreads();
    const float inv_cap = cap > 0.f ? 1.0f / cap : 0.f;
    const int first = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;
    // this block's share of the visible keys: whole chunks of 32, the same count for every share but the last
    const int chunks = (pos - first) / 32 + 1, per_share = (chunks + shares - 1) / shares;
    const int c_lo = share * per_share, c_hi = min(chunks, c_lo + per_share);
    const int wide = VG * V, bw = wide / col_blocks, col0 = cb * bw;
    float m[R], l[R], acc[R][NC];
    int voff[NC];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        m[r] = -INFINITY;
        l[r] = 0.f;
#pragma unroll
        for (int j = 0; j < NC; ++j) acc[r][j] = 0.f;
    }
#pragma unroll
    for (int j = 0; j < NC; ++j) {
        const int il = VEC ? lane * NC + j : lane + 32 * j, i = col0 + il;
        const int c = VG == 1 ? g : i / V;
        voff[j] = il < bw ? c * page_size * V + i % V : 0;           // (lanes past the block's columns read a channel they never store)
    }
    for (int chunk = c_lo + warp; chunk < c_hi; chunk += TKD_WARPS) {
        const int base = first + chunk * 32, key = base + lane;
        float s[R];
#pragma unroll
        for (int r = 0; r < R; ++r) s[r] = -INFINITY;
        long long at = -1;
        if (key <= pos) {
            const long long page = table[key / page_size];
            if (page < 0 || page >= num_pages) {
                atomicOr(status, GB_STATUS_BAD_SLOT);
            } else {
                at = page * G * page_size + key % page_size;
                sad_dots<T, R>(qs, kcache + (at + (long long)g * page_size) * D, D, s);
#pragma unroll
                for (int r = 0; r < R; ++r) s[r] = tk_cap(s[r] * scale, cap, inv_cap);
            }
        }
        float p[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const float m_new = fmaxf(m[r], gb_warp_max(s[r]));
            const float corr = m_new == -INFINITY ? 1.f : expf(m[r] - m_new);
            p[r] = at >= 0 ? expf(s[r] - m_new) : 0.f;
            l[r] = l[r] * corr + gb_warp_sum(p[r]);
            m[r] = m_new;
#pragma unroll
            for (int j = 0; j < NC; ++j) acc[r][j] *= corr;
        }
        // a key that cannot be read has weight 0; its loads go to the first row of the pool instead
        const long long safe = at >= 0 ? at : 0;
#pragma unroll 1
        for (int t0 = 0; t0 < 32; t0 += KB) {
            if (base + t0 > pos) break;
            if constexpr (VEC) {
                unsigned raw[KB][NC / 2];
#pragma unroll
                for (int u = 0; u < KB; ++u)
                    tkd_load_words<NC>(reinterpret_cast<const __nv_bfloat16*>(vcache) + __shfl_sync(0xffffffffu, safe, t0 + u) * V + voff[0],
                                       raw[u]);
#pragma unroll
                for (int u = 0; u < KB; ++u) {
                    float pt[R];
#pragma unroll
                    for (int r = 0; r < R; ++r) pt[r] = __shfl_sync(0xffffffffu, p[r], t0 + u);
#pragma unroll
                    for (int j2 = 0; j2 < NC / 2; ++j2) {
                        const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw[u][j2]));
#pragma unroll
                        for (int r = 0; r < R; ++r) {
                            acc[r][2 * j2] = fmaf(pt[r], v.x, acc[r][2 * j2]);
                            acc[r][2 * j2 + 1] = fmaf(pt[r], v.y, acc[r][2 * j2 + 1]);
                        }
                    }
                }
            } else {
                float val[KB][NC];
#pragma unroll
                for (int u = 0; u < KB; ++u) {
                    const T* vp = vcache + __shfl_sync(0xffffffffu, safe, t0 + u) * V;
#pragma unroll
                    for (int j = 0; j < NC; ++j) val[u][j] = gb_to_float(vp[voff[j]]);
                }
#pragma unroll
                for (int u = 0; u < KB; ++u) {
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        const float pt = __shfl_sync(0xffffffffu, p[r], t0 + u);
#pragma unroll
                        for (int j = 0; j < NC; ++j) acc[r][j] = fmaf(pt, val[u][j], acc[r][j]);
                    }
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
#pragma unroll
        for (int j = 0; j < NC; ++j) part[warp][r][VEC ? lane * NC + j : lane + 32 * j] = acc[r][j];
        if (lane == 0) {
            part[warp][r][NC * 32] = m[r];
            part[warp][r][NC * 32 + 1] = l[r];
        }
    }
    __syncthreads();
    const bool final_ = shares == 1;
    for (int idx = threadIdx.x; idx < R * bw; idx += TKD_WARPS * 32) {
        const int r = idx / bw, i = idx % bw;
        float top = (final_ && unit > 0.f) ? 0.f : -INFINITY;
#pragma unroll
        for (int w = 0; w < TKD_WARPS; ++w) top = fmaxf(top, part[w][r][NC * 32]);
        float den = (final_ && unit > 0.f) ? unit * expf(-top) : 0.f, sum = 0.f;
        if (top > -INFINITY) {
#pragma unroll
            for (int w = 0; w < TKD_WARPS; ++w) {
                const float mw = part[w][r][NC * 32];
                const float f = mw == -INFINITY ? 0.f : expf(mw - top);
                den = fmaf(part[w][r][NC * 32 + 1], f, den);
                sum = fmaf(part[w][r][i], f, sum);
            }
        }
        const size_t at = ((size_t)share * n + row) * H + head0 + r;
        if (final_) {
            out[at * wide + col0 + i] = den > 0.f ? sum / den : 0.f;
        } else {
            out[at * wide + col0 + i] = sum;
            if (i == 0 && cb == 0) {
                ml[at * 2] = top;
                ml[at * 2 + 1] = den;
            }
        }
    }
}

GB_EXPORT int gb_talking_attention_decode_plan(int H, int G, int V, int VG) {
    // column blocks * 10000 + heads per block * 100 + pieces: a wide row that is a multiple of 256 channels goes in column blocks
    // of 256; heads per block: the largest of 8, 4, 2, 1 that divides the group and keeps R * NC within 32; 0: no kernel
    const int wide = VG * V;
    const int col_blocks = (wide > 256 && wide % 256 == 0) ? wide / 256 : 1;
    const int bw = wide / col_blocks;
    int nc = 1;
    while (nc < 8 && nc * 32 < bw) nc *= 2;
    if (nc * 32 < bw) nc = bw <= 384 ? 12 : 16;
    if (nc * 32 < bw) return 0;
    for (int r = 8; r >= 1; r /= 2)
        if ((H / G) % r == 0 && r * nc <= 32) return col_blocks * 10000 + r * 100 + nc;
    return 0;
}

// shares > 1: out is [shares][n][H][wide] and ml [shares][n][H][2], for talk_combine to merge; shares == 1: out is final
GB_EXPORT int gb_talking_attention_decode(const void* q, float* out, float* ml, int dtype, const void* kcache, const void* vcache,
                                          const int* block_tables, int max_pages, const int* row_seq, const int* positions, int n, int H,
                                          int G, int D, int V, int VG, int page_size, long long num_pages, float scale, float cap,
                                          float unit, int window, int shares, int* status, cudaStream_t stream) {
    TK_COMMON_CHECKS("gb_talking_attention_decode")
    const int plan = gb_talking_attention_decode_plan(H, G, V, VG);
    GB_REQUIRE(plan > 0, "gb_talking_attention_decode: %d value heads of %d channels are not built", VG, V);
    GB_REQUIRE(shares >= 1 && shares <= 64 && (shares == 1 || ml != nullptr), "gb_talking_attention_decode: %d shares", shares);
    if (n == 0) return 0;
    const int col_blocks = plan / 10000, R = plan % 10000 / 100, nc = plan % 100;
    const dim3 grid(n, H / R, shares * col_blocks);
    // (the vector form: bfloat16, a wide row of exactly 32 * nc channels, a lane's nc channels inside one value head)
    const bool vec = dtype == GB_BF16 && VG * V == 32 * nc * col_blocks && nc % 2 == 0 && V % nc == 0;
#define TKD_LAUNCH(T, RR, N, VV)                                                                                                        \
    gb_launch(GB_PDL_ATTENTION, talking_attention_decode_kernel<T, RR, N, VV>, grid, dim3(TKD_WARPS * 32), 0, stream, (const T*)q, out, \
              ml, (const T*)kcache, (const T*)vcache, block_tables, max_pages, row_seq, positions, n, H, G, D, V, VG, page_size,        \
              num_pages, scale, cap, unit, window, shares, col_blocks, status)
#define TKD_CASE(T, RR, N)                                                                                                             \
    if (R == RR && nc == N) {                                                                                                          \
        if (sizeof(T) == 2 && N % 2 == 0 && vec) TKD_LAUNCH(T, RR, (N % 2 == 0 ? N : 2), (sizeof(T) == 2));                            \
        else TKD_LAUNCH(T, RR, N, false);                                                                                              \
        launched = true;                                                                                                               \
    }
#define TKD_ALL(T)                                                                                                                      \
    TKD_CASE(T, 1, 1) TKD_CASE(T, 1, 2) TKD_CASE(T, 1, 4) TKD_CASE(T, 1, 8) TKD_CASE(T, 1, 12) TKD_CASE(T, 1, 16)                       \
    TKD_CASE(T, 2, 1) TKD_CASE(T, 2, 2) TKD_CASE(T, 2, 4) TKD_CASE(T, 2, 8) TKD_CASE(T, 2, 12) TKD_CASE(T, 2, 16)                       \
    TKD_CASE(T, 4, 1) TKD_CASE(T, 4, 2) TKD_CASE(T, 4, 4) TKD_CASE(T, 4, 8)                                                            \
    TKD_CASE(T, 8, 1) TKD_CASE(T, 8, 2) TKD_CASE(T, 8, 4)
    bool launched = false;
    if (dtype == GB_F32) { TKD_ALL(float) }
    else if (dtype == GB_BF16) { TKD_ALL(__nv_bfloat16) }
    else GB_REQUIRE(false, "gb_talking_attention_decode: unsupported dtype %d", dtype);
#undef TKD_ALL
#undef TKD_CASE
#undef TKD_LAUNCH
    GB_REQUIRE(launched, "gb_talking_attention_decode: no kernel for %d heads a block and %d pieces", R, nc);
    return gb_check_launch("gb_talking_attention_decode");
}

// ----------------------------------------------------------------------------------------------
// Prompt portions in bfloat16 on the tensor cores. One block = 64 rows of one request x one query head x VC columns of the
// wide value row (the values of all key/value heads side by side; blockIdx.z picks the columns, and every such block forms
// the head's scores again). The keys any row of the tile can see pass in 64-key tiles through shared memory (cp.async, two
// buffers, pages through the block table); S = Q K^T and O += P V with mma.sync m16n8k16, P from the score fragments in
// registers, float32 online softmax in the base-2 domain whose maximum starts at the unit's score (0). Four warps, 16 rows
// each. The float32 results go to out[row, head, z * VC ..].
// ----------------------------------------------------------------------------------------------
constexpr int TKT_BM = 64, TKT_BN = 64;
constexpr float TK_LOG2E = 1.4426950408889634f;

template <int D, int VC>
__global__ void __launch_bounds__(128) talking_attention_tiles_kernel(
    const __nv_bfloat16* __restrict__ q, float* __restrict__ out, const __nv_bfloat16* __restrict__ kcache,
    const __nv_bfloat16* __restrict__ vcache, const int* __restrict__ block_tables, int max_pages, const int* __restrict__ seq_first_row,
    const int* __restrict__ seq_start_pos, int num_seqs, int tiles_per_seq, int H, int G, int V, int VG, int page_size,
    long long num_pages, float scale, float cap, float unit, int window, int* __restrict__ status) {
    constexpr int LDK = D + 8, LDV = VC + 8;          // rows padded by 16 bytes: ldmatrix meets no bank twice
    extern __shared__ __align__(16) unsigned char tkt_smem[];
    __nv_bfloat16* sq = reinterpret_cast<__nv_bfloat16*>(tkt_smem);             // [64][LDK]
    __nv_bfloat16* sk = sq + TKT_BM * LDK;                                        // [2][64][LDK]
    __nv_bfloat16* sv = sk + 2 * TKT_BN * LDK;                                    // [2][64][LDV]
    gb_pdl_launch_dependents();
    gb_pdl_wait();
    const int seq = blockIdx.x / tiles_per_seq, tile = blockIdx.x % tiles_per_seq, head = blockIdx.y, col0 = blockIdx.z * VC;
    if (seq >= num_seqs) return;
    const int start = seq_start_pos[seq];
    if (start < 0) return;
    const int r0 = seq_first_row[seq], len = seq_first_row[seq + 1] - r0;
    if (tile * TKT_BM >= len) return;
    const int rows = min(TKT_BM, len - tile * TKT_BM);
    const int row0 = r0 + tile * TKT_BM, p_lo = start + tile * TKT_BM, p_hi = p_lo + rows - 1;
    if (p_hi / page_size >= max_pages) {
        if (threadIdx.x == 0) atomicOr(status, GB_STATUS_BAD_POSITION);
        return;
    }
    const int k_lo = (window > 0 && p_lo + 1 > window) ? p_lo + 1 - window : 0;
    const int g = head / (H / G);
    const int wide = VG * V;
    const int* table = block_tables + (size_t)seq * max_pages;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    for (int chunk = tid; chunk < TKT_BM * (D / 8); chunk += 128) {
        const int r = chunk / (D / 8), c = (chunk % (D / 8)) * 8;
        sat_cp16(sq + r * LDK + c, q + ((size_t)(row0 + (r < rows ? r : 0)) * H + head) * D + c, r < rows);
    }
    auto stage = [&](int buf, int kb) {
        // two threads per key: one page look-up each, then half of the key's 16-byte pieces (key row, then the value columns)
        constexpr int CPK = (D + VC) / 8;
        const int key = tid >> 1, kk = kb + key;
        long long page = kk <= p_hi ? table[kk / page_size] : -1;
        if (kk <= p_hi && (page < 0 || page >= num_pages)) {
            atomicOr(status, GB_STATUS_BAD_SLOT);
            page = -1;
        }
        const long long at = page < 0 ? 0 : page * G * page_size + kk % page_size;
#pragma unroll
        for (int i = 0; i < CPK / 2; ++i) {
            const int c = ((tid & 1) * (CPK / 2) + i) * 8;
            if (c < D) {
                sat_cp16(sk + (buf * TKT_BN + key) * LDK + c, kcache + (at + (long long)g * page_size) * D + c, page >= 0);
            } else {
                const int w = col0 + (c - D);                           // column of the wide value row
                const int vh = VG == 1 ? g : w / V;
                sat_cp16(sv + (buf * TKT_BN + key) * LDV + (c - D), vcache + (at + (long long)vh * page_size) * V + w % V, page >= 0);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    const int n_tiles = (p_hi - k_lo) / TKT_BN + 1;
    stage(0, k_lo);                                   // (one group holds Q and the first keys)
    unsigned qf[D / 16][4];
    float o[VC / 8][4];
#pragma unroll
    for (int j = 0; j < VC / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    const float unit2 = unit > 0.f ? 0.f : -INFINITY;                                 // the unit's score, 0, in the base-2 domain
    const float inv_cap = cap > 0.f ? 1.0f / cap : 0.f, cap2 = cap * TK_LOG2E, scale2 = scale * TK_LOG2E;
    const int my_pos0 = p_lo + warp * 16 + (lane >> 2), my_pos1 = my_pos0 + 8;       // positions of this thread's two rows
    float mrow[2] = {unit2, unit2}, lrow[2] = {0.f, 0.f};                             // (a thread's share of the denominator)
    for (int t = 0; t < n_tiles; ++t) {
        const int kb = k_lo + t * TKT_BN, buf = t & 1;
        if (t + 1 < n_tiles) {
            stage(buf ^ 1, kb + TKT_BN);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        if (t == 0) {
#pragma unroll
            for (int kd = 0; kd < D / 16; ++kd) {
                const unsigned addr = (unsigned)__cvta_generic_to_shared(sq + (warp * 16 + (lane & 15)) * LDK + kd * 16 + (lane >> 4) * 8);
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                             : "=r"(qf[kd][0]), "=r"(qf[kd][1]), "=r"(qf[kd][2]), "=r"(qf[kd][3]) : "r"(addr));
            }
        }
        // a warp whose rows lie wholly before this tile's first key or (with a window) wholly behind its last visible one
        // still walks the barriers, but skips the arithmetic
        const int w_lo = p_lo + warp * 16, w_hi = w_lo + 15;
        const bool any = kb <= w_hi && (window <= 0 || kb + TKT_BN - 1 > w_lo - window) && warp * 16 < rows;
        if (any) {
            float s[TKT_BN / 8][4];
#pragma unroll
            for (int j = 0; j < TKT_BN / 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
            const __nv_bfloat16* kt = sk + buf * TKT_BN * LDK;
#pragma unroll
            for (int kd = 0; kd < D / 16; ++kd) {
#pragma unroll
                for (int j2 = 0; j2 < TKT_BN / 16; ++j2) {
                    unsigned b0, b1_, b2_, b3;
                    const int nrow = j2 * 16 + (lane & 7) + ((lane >> 4) << 3), kcol = kd * 16 + ((lane >> 3) & 1) * 8;
                    const unsigned addr = (unsigned)__cvta_generic_to_shared(kt + nrow * LDK + kcol);
                    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(b0), "=r"(b1_), "=r"(b2_), "=r"(b3) : "r"(addr));
                    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                                 : "+f"(s[2 * j2][0]), "+f"(s[2 * j2][1]), "+f"(s[2 * j2][2]), "+f"(s[2 * j2][3])
                                 : "r"(qf[kd][0]), "r"(qf[kd][1]), "r"(qf[kd][2]), "r"(qf[kd][3]), "r"(b0), "r"(b1_));
                    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                                 : "+f"(s[2 * j2 + 1][0]), "+f"(s[2 * j2 + 1][1]), "+f"(s[2 * j2 + 1][2]), "+f"(s[2 * j2 + 1][3])
                                 : "r"(qf[kd][0]), "r"(qf[kd][1]), "r"(qf[kd][2]), "r"(qf[kd][3]), "r"(b2_), "r"(b3));
                }
            }
            // capped scores in the base-2 domain; the causal edge and the window per element, except in tiles that every row
            // of the warp sees whole (most of them); then the rows' maxima (a row lies in the four lanes of a quad)
            const bool whole = kb + TKT_BN - 1 <= w_lo && (window <= 0 || w_hi - kb < window) && w_hi <= p_hi;
            float mx[2] = {mrow[0], mrow[1]};
#pragma unroll
            for (int j = 0; j < TKT_BN / 8; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = kb + j * 8 + (lane & 3) * 2 + (e & 1);
                    const int pos = e < 2 ? my_pos0 : my_pos1;
                    float v = cap > 0.f ? cap2 * tanhf(s[j][e] * scale * inv_cap) : s[j][e] * scale2;
                    if (!whole) {
                        const bool sees = key <= pos && (window <= 0 || pos - key < window) && pos <= p_hi;
                        v = sees ? v : -INFINITY;
                    }
                    s[j][e] = v;
                    mx[e >> 1] = fmaxf(mx[e >> 1], v);
                }
            }
            float corr[2];
#pragma unroll
            for (int hrow = 0; hrow < 2; ++hrow) {
                mx[hrow] = fmaxf(mx[hrow], __shfl_xor_sync(0xffffffffu, mx[hrow], 1));
                mx[hrow] = fmaxf(mx[hrow], __shfl_xor_sync(0xffffffffu, mx[hrow], 2));
                corr[hrow] = mx[hrow] == -INFINITY ? 1.f : exp2f(mrow[hrow] - mx[hrow]);
                mrow[hrow] = mx[hrow];
                lrow[hrow] *= corr[hrow];
            }
            const float sub0 = mx[0] == -INFINITY ? 0.f : mx[0], sub1 = mx[1] == -INFINITY ? 0.f : mx[1];
#pragma unroll
            for (int j = 0; j < VC / 8; ++j) {
                o[j][0] *= corr[0]; o[j][1] *= corr[0];
                o[j][2] *= corr[1]; o[j][3] *= corr[1];
            }
            unsigned pf[TKT_BN / 16][4];
#pragma unroll
            for (int j = 0; j < TKT_BN / 8; ++j) {
                float p[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) p[e] = exp2f(s[j][e] - (e < 2 ? sub0 : sub1));
                // the denominator sums what the products use: the weights as rounded to bfloat16
                const __nv_bfloat162 lo = __floats2bfloat162_rn(p[0], p[1]), hi = __floats2bfloat162_rn(p[2], p[3]);
                const float2 flo = __bfloat1622float2(lo), fhi = __bfloat1622float2(hi);
                lrow[0] += flo.x + flo.y;
                lrow[1] += fhi.x + fhi.y;
                pf[j >> 1][(j & 1) * 2] = *reinterpret_cast<const unsigned*>(&lo);
                pf[j >> 1][(j & 1) * 2 + 1] = *reinterpret_cast<const unsigned*>(&hi);
            }
            const __nv_bfloat16* vt = sv + buf * TKT_BN * LDV;
#pragma unroll
            for (int kk = 0; kk < TKT_BN / 16; ++kk) {
#pragma unroll
                for (int n2 = 0; n2 < VC / 16; ++n2) {
                    unsigned b0, b1_, b2_, b3;
                    const int krow = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, ncol = n2 * 16 + (lane >> 4) * 8;
                    const unsigned addr = (unsigned)__cvta_generic_to_shared(vt + krow * LDV + ncol);
                    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(b0), "=r"(b1_), "=r"(b2_), "=r"(b3) : "r"(addr));
                    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                                 : "+f"(o[2 * n2][0]), "+f"(o[2 * n2][1]), "+f"(o[2 * n2][2]), "+f"(o[2 * n2][3])
                                 : "r"(pf[kk][0]), "r"(pf[kk][1]), "r"(pf[kk][2]), "r"(pf[kk][3]), "r"(b0), "r"(b1_));
                    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                                 : "+f"(o[2 * n2 + 1][0]), "+f"(o[2 * n2 + 1][1]), "+f"(o[2 * n2 + 1][2]), "+f"(o[2 * n2 + 1][3])
                                 : "r"(pf[kk][0]), "r"(pf[kk][1]), "r"(pf[kk][2]), "r"(pf[kk][3]), "r"(b2_), "r"(b3));
                }
            }
        }
        __syncthreads();          // everyone is done with this buffer before the round after next overwrites it
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        float den = lrow[half];
        den += __shfl_xor_sync(0xffffffffu, den, 1);
        den += __shfl_xor_sync(0xffffffffu, den, 2);
        if (unit > 0.f) den += unit * exp2f(unit2 - mrow[half]);          // (the maximum started at the unit's score: at most 1)
        const int r = warp * 16 + (lane >> 2) + half * 8;
        if (r >= rows) continue;
        const float f = den > 0.f ? 1.0f / den : 0.f;
        float* dst = out + ((size_t)(row0 + r) * H + head) * wide + col0;
#pragma unroll
        for (int j = 0; j < VC / 8; ++j)
            *reinterpret_cast<float2*>(dst + j * 8 + (lane & 3) * 2) = make_float2(o[j][half * 2] * f, o[j][half * 2 + 1] * f);
    }
}

// the columns of the wide value row that one block takes: the largest of 128, 64, 32 that divides the row; 0: no kernel
GB_EXPORT int gb_talking_attention_tiles_columns(int D, int V, int VG) {
    if (!(D == 32 || D == 64 || D == 96 || D == 128) || V % 8) return 0;
    const int wide = VG * V;
    for (int vc = 128; vc >= 32; vc /= 2)
        if (wide % vc == 0) return vc;
    return 0;
}

template <int D, int VC>
static int tkt_launch(const void* q, float* out, const void* kcache, const void* vcache, const int* block_tables, int max_pages,
                      const int* seq_first_row, const int* seq_start_pos, int num_seqs, int tiles_per_seq, int H, int G, int V, int VG,
                      int page_size, long long num_pages, float scale, float cap, float unit, int window, int* status,
                      cudaStream_t stream) {
    const size_t smem = ((size_t)3 * TKT_BM * (D + 8) + (size_t)2 * TKT_BN * (VC + 8)) * 2;
    cudaFuncSetAttribute(talking_attention_tiles_kernel<D, VC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    gb_launch(GB_PDL_ATTENTION, talking_attention_tiles_kernel<D, VC>, dim3(num_seqs * tiles_per_seq, H, VG * V / VC), dim3(128), smem,
              stream, (const __nv_bfloat16*)q, out, (const __nv_bfloat16*)kcache, (const __nv_bfloat16*)vcache, block_tables, max_pages,
              seq_first_row, seq_start_pos, num_seqs, tiles_per_seq, H, G, V, VG, page_size, num_pages, scale, cap, unit, window, status);
    return gb_check_launch("gb_talking_attention_tiles");
}

GB_EXPORT int gb_talking_attention_tiles(const void* q, float* out, const void* kcache, const void* vcache, const int* block_tables,
                                         int max_pages, const int* seq_first_row, const int* seq_start_pos, int num_seqs,
                                         int max_rows_per_seq, int H, int G, int D, int V, int VG, int page_size, long long num_pages,
                                         float scale, float cap, float unit, int window, int* status, cudaStream_t stream) {
    const int n = num_seqs;
    TK_COMMON_CHECKS("gb_talking_attention_tiles")
    const int vc = gb_talking_attention_tiles_columns(D, V, VG);
    GB_REQUIRE(vc > 0 && max_rows_per_seq > 0, "gb_talking_attention_tiles: head sizes %d / %d x %d are not built", D, V, VG);
    if (num_seqs == 0) return 0;
    const int tiles = gb_ceil_div(max_rows_per_seq, TKT_BM);
#define TKT_CASE(DD, VV)                                                                                                             \
    if (D == DD && vc == VV)                                                                                                          \
        return tkt_launch<DD, VV>(q, out, kcache, vcache, block_tables, max_pages, seq_first_row, seq_start_pos, num_seqs, tiles, H, G, \
                                  V, VG, page_size, num_pages, scale, cap, unit, window, status, stream);
    TKT_CASE(32, 32) TKT_CASE(32, 64) TKT_CASE(32, 128) TKT_CASE(64, 32) TKT_CASE(64, 64) TKT_CASE(64, 128) TKT_CASE(96, 32)
    TKT_CASE(96, 64) TKT_CASE(96, 128) TKT_CASE(128, 32) TKT_CASE(128, 64) TKT_CASE(128, 128)
#undef TKT_CASE
    GB_REQUIRE(false, "gb_talking_attention_tiles: head sizes %d / %d are not built", D, vc);
}

// ----------------------------------------------------------------------------------------------
// The mix: att[row, h, :] = sum_g talk[h, g] * O[row, g, c(h), :] (talk == nullptr: O[row, h, c(h) or 0, :] as it is).
// shares > 1: O arrives in shares of the keys (o: [shares][n][H][wide] unnormalised sums, ml: [shares][n][H][2] each share's
// maximum and denominator); the weights that merge them (and the unit of the denominator) are formed per (row, head) first.
// One block per (row, key/value head c): it brings every head's result over c's values into shared memory once (merging the
// shares on the way) and forms the outputs of the query heads whose key/value head is c.
// ----------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) talk_combine_kernel(const float* __restrict__ o, const float* __restrict__ ml,
                                                           const float* __restrict__ talk, T* __restrict__ att,
                                                           const int* __restrict__ positions, int n, int H, int G, int V, int VG, int shares,
                                                           float unit) {
    extern __shared__ float tkc_smem[];
    float* rows = tkc_smem;                  // [H][V]: head g's merged result over this block's value head
    float* factor = rows + (size_t)H * V;    // [H][shares]: a share's weight in head g's merged softmax
    gb_pdl_launch_dependents();
    gb_pdl_wait();
    const int row = blockIdx.x, c = blockIdx.y;
    if (row >= n || positions[row] < 0) return;
    const int wide = VG * V, per = H / G;
    // without a mix only the heads of this group are read, each over its own values
    const int g_lo = talk ? 0 : c * per, g_hi = talk ? H : (c + 1) * per;
    const size_t col0 = VG == 1 ? 0 : (size_t)c * V;
    if (shares > 1) {
        for (int g = g_lo + threadIdx.x; g < g_hi; g += 256) {
            float top = unit > 0.f ? 0.f : -INFINITY;
            for (int z = 0; z < shares; ++z) top = fmaxf(top, ml[(((size_t)z * n + row) * H + g) * 2]);
            float den = unit > 0.f ? unit * expf(-top) : 0.f;
            for (int z = 0; z < shares; ++z) {
                const float mz = ml[(((size_t)z * n + row) * H + g) * 2];
                const float f = mz == -INFINITY ? 0.f : expf(mz - top);
                den = fmaf(ml[(((size_t)z * n + row) * H + g) * 2 + 1], f, den);
                factor[g * shares + z] = f;
            }
            const float inv = den > 0.f ? 1.0f / den : 0.f;
            for (int z = 0; z < shares; ++z) factor[g * shares + z] *= inv;
        }
        __syncthreads();
    }
    // (with few rows the channels of a value head are cut over blockIdx.z, so that the merge has blocks enough)
    const int cw = (V + gridDim.z - 1) / gridDim.z, ch_lo = blockIdx.z * cw, ch_n = max(0, min(V, ch_lo + cw) - ch_lo);
    for (int t = threadIdx.x; t < (g_hi - g_lo) * ch_n; t += 256) {
        const int g = g_lo + t / ch_n, ch = ch_lo + t % ch_n, idx = g * V + ch;
        float v;
        if (shares > 1) {
            float a0 = 0.f, a1 = 0.f;
            int z = 0;
            for (; z + 2 <= shares; z += 2) {
                a0 = fmaf(factor[g * shares + z], o[(((size_t)z * n + row) * H + g) * wide + col0 + ch], a0);
                a1 = fmaf(factor[g * shares + z + 1], o[(((size_t)(z + 1) * n + row) * H + g) * wide + col0 + ch], a1);
            }
            if (z < shares) a0 = fmaf(factor[g * shares + z], o[(((size_t)z * n + row) * H + g) * wide + col0 + ch], a0);
            v = a0 + a1;
        } else {
            v = o[((size_t)row * H + g) * wide + col0 + ch];
        }
        rows[idx] = v;
    }
    __syncthreads();
    for (int t = threadIdx.x; t < per * ch_n; t += 256) {
        const int h = c * per + t / ch_n, ch = ch_lo + t % ch_n;
        float acc;
        if (talk) {
            float a0 = 0.f, a1 = 0.f;
            int g = 0;
            for (; g + 2 <= H; g += 2) {
                a0 = fmaf(talk[h * H + g], rows[g * V + ch], a0);
                a1 = fmaf(talk[h * H + g + 1], rows[(g + 1) * V + ch], a1);
            }
            if (g < H) a0 = fmaf(talk[h * H + g], rows[g * V + ch], a0);
            acc = a0 + a1;
        } else {
            acc = rows[h * V + ch];
        }
        att[((size_t)row * H + h) * V + ch] = gb_from_float<T>(acc);
    }
}

template <typename T>
static int tkc_launch(const float* o, const float* ml, const float* talk, void* att, const int* positions, int n, int H, int G, int V,
                      int VG, int shares, float unit, cudaStream_t stream) {
    const size_t smem = ((size_t)H * V + (size_t)H * shares) * sizeof(float);
    GB_REQUIRE(smem <= 200 * 1024, "gb_talk_combine: %d heads of %d channels in %d shares do not fit a block's shared memory", H, V, shares);
    if (smem > 48 * 1024) cudaFuncSetAttribute(talk_combine_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    const int cuts = (long long)n * G >= 296 ? 1 : (int)min((long long)gb_ceil_div(V, 16), (long long)gb_ceil_div(296, (long long)n * G));
    gb_launch(GB_PDL_ELEMENTWISE, talk_combine_kernel<T>, dim3(n, G, cuts), dim3(256), smem, stream, o, ml, talk, (T*)att, positions, n, H, G,
              V, VG, shares, unit);
    return gb_check_launch("gb_talk_combine");
}

GB_EXPORT int gb_talk_combine(const float* o, const float* ml, const float* talk, void* att, int dtype, const int* positions, int n, int H,
                              int G, int V, int VG, int shares, float unit, cudaStream_t stream) {
    GB_REQUIRE(n >= 0 && H > 0 && G > 0 && H % G == 0 && V > 0 && (VG == G || VG == 1), "gb_talk_combine: bad sizes");
    GB_REQUIRE(talk == nullptr || VG == G, "gb_talk_combine: mixing the heads needs every head's values");
    GB_REQUIRE(shares >= 1 && (shares == 1 || ml != nullptr), "gb_talk_combine: %d shares of %d heads", shares, H);
    if (n == 0) return 0;
    if (dtype == GB_F32) return tkc_launch<float>(o, ml, talk, att, positions, n, H, G, V, VG, shares, unit, stream);
    if (dtype == GB_BF16) return tkc_launch<__nv_bfloat16>(o, ml, talk, att, positions, n, H, G, V, VG, shares, unit, stream);
    GB_REQUIRE(false, "gb_talk_combine: unsupported dtype %d", dtype);
}
