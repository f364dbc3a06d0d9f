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
//   talking_attention_decode  single decoded tokens: a block of 8 warps per (row, head), the warps take the keys in turn
//   talking_attention_tiles   prompt portions in bfloat16 on the tensor cores (mma.sync), 64 rows x one head per block
//   talk_combine           the mix of the heads' results
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
// The mix: att[row, h, :] = sum_g talk[h, g] * O[row, g, c(h), :] (talk == nullptr: O[row, h, c(h) or 0, :] as it is).
// One thread per (row, h, channel).
// ----------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) talk_combine_kernel(const float* __restrict__ o, const float* __restrict__ talk, T* __restrict__ att,
                                                           const int* __restrict__ positions, int n, int H, int G, int V, int VG) {
    gb_pdl_launch_dependents();
    gb_pdl_wait();
    const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    if (i >= (long long)n * H * V) return;
    const int ch = (int)(i % V), h = (int)((i / V) % H), row = (int)(i / ((long long)V * H));
    if (positions[row] < 0) return;
    const int c = VG == 1 ? 0 : h / (H / G);
    const float* src = o + (size_t)row * H * VG * V + (size_t)c * V + ch;
    float acc;
    if (talk == nullptr) {
        acc = src[(size_t)h * VG * V];
    } else {
        acc = 0.f;
        for (int g = 0; g < H; ++g) acc = fmaf(talk[h * H + g], src[(size_t)g * VG * V], acc);
    }
    att[i] = gb_from_float<T>(acc);
}

GB_EXPORT int gb_talk_combine(const float* o, const float* talk, void* att, int dtype, const int* positions, int n, int H, int G, int V,
                              int VG, cudaStream_t stream) {
    GB_REQUIRE(n >= 0 && H > 0 && G > 0 && H % G == 0 && V > 0 && (VG == G || VG == 1), "gb_talk_combine: bad sizes");
    GB_REQUIRE(talk == nullptr || VG == G, "gb_talk_combine: mixing the heads needs every head's values");
    if (n == 0) return 0;
    const int blocks = gb_ceil_div((long long)n * H * V, 256);
    if (dtype == GB_F32)
        gb_launch(GB_PDL_ELEMENTWISE, talk_combine_kernel<float>, dim3(blocks), dim3(256), 0, stream, o, talk, (float*)att, positions, n, H, G,
                  V, VG);
    else if (dtype == GB_BF16)
        gb_launch(GB_PDL_ELEMENTWISE, talk_combine_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, o, talk, (__nv_bfloat16*)att,
                  positions, n, H, G, V, VG);
    else
        GB_REQUIRE(false, "gb_talk_combine: unsupported dtype %d", dtype);
    return gb_check_launch("gb_talk_combine");
}
