// Softmax attention over the paged cache whose positions enter as a bias on the distance, with a sink in the denominator
// and a gate on the output. For a row at position p of its request and a key at position j <= p:
//     s_j = q . k_j * scale - r1[head] * ln(1 + r2[head] * (p - j))                 (r1 == nullptr: no bias)
//     w_j = exp(s_j - m) / (sum_j' exp(s_j' - m) + exp(sink[head] - m))             (sink == nullptr: a plain softmax)
//     out = sum_j w_j v_j * sigmoid(gate[row, head])                                (gate == nullptr: no gate)
// The sink has no key and no value: it only takes its share of the weights. The row sees keys max(0, p - window + 1) .. p
// (window 0: all of them). Query heads share key/value heads in groups; the key size (dim) and the value size (vdim) may
// differ. Distances, logarithms, scores, weights, sums and the gate are float32. gate holds logits, float32 [n, ld_gate].
//
//   sink_attention_rows    one warp per (row, head), any row (prompt portion or single token), both dtypes: 32 keys at a
//                          time from the first visible one, a lane per key for the scores, a lane per channel for the sum,
//                          a running maximum that starts at the sink's logit.
//   sink_attention_decode  single decoded tokens: a block of 8 warps per (row, head or four heads of a group).
//   sink_attention_tiles   prompt portions in bfloat16 on the tensor cores.
#include "common.cuh"
#include "paged_rows.cuh"

constexpr int SK_WARPS = 4;

// what is taken off the score of a key `dist` tokens back
__device__ __forceinline__ float sk_distance_bias(float r1, float r2, int dist) { return r1 * log1pf(r2 * (float)dist); }

__device__ __forceinline__ float sk_sigmoid(float v) { return 1.0f / (1.0f + expf(-v)); }

template <typename T>
__global__ void __launch_bounds__(SK_WARPS * 32) sink_attention_rows_kernel(
    const T* __restrict__ q, T* __restrict__ out, const T* __restrict__ kcache, const T* __restrict__ vcache,
    const int* __restrict__ block_tables, int max_pages, const int* __restrict__ row_seq, const int* __restrict__ positions,
    const float* __restrict__ r1, const float* __restrict__ r2, const float* __restrict__ sink, const float* __restrict__ gate,
    long long ld_gate, int n, int H, int G, int D, int V, int page_size, long long num_pages, float scale, int window,
    int* __restrict__ status) {
    __shared__ float qs[SK_WARPS][SA_MAX_DIM];
    gb_pdl_launch_dependents();
    gb_pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long task = (long long)blockIdx.x * SK_WARPS + warp;
    if (task >= (long long)n * H) return;
    const int row = (int)(task / H), head = (int)(task % H);
    const int g = head / (H / G);
    const int pos = positions[row];
    if (pos < 0) return;
    if (pos / page_size >= max_pages) {      // a position the block table does not reach: reported, the row reads nothing
        if (lane == 0) atomicOr(status, GB_STATUS_BAD_POSITION);
        return;
    }
    const int* table = block_tables + (size_t)row_seq[row] * max_pages;
    const T* qrow = q + ((size_t)row * H + head) * D;
    for (int i = lane; i < D; i += 32) qs[warp][i] = gb_to_float(qrow[i]);
    __syncwarp();
    const float b1 = r1 ? r1[head] : 0.f, b2 = r1 ? r2[head] : 0.f;
    const int first = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;
    // the sink starts the running maximum and the denominator: exp(sink - m) with m = sink
    float m = sink ? sink[head] : -INFINITY, l = sink ? 1.f : 0.f;
    float acc[SA_MAX_DIM / 32];
#pragma unroll
    for (int j = 0; j < SA_MAX_DIM / 32; ++j) acc[j] = 0.f;
    for (int base = first; base <= pos; base += 32) {
        const int key = base + lane;
        float s = -INFINITY;
        long long at = -1;                   // (page * G + g) * page_size + offset of this lane's key
        if (key <= pos) {
            const long long page = table[key / page_size];
            if (page < 0 || page >= num_pages) {
                atomicOr(status, GB_STATUS_BAD_SLOT);
            } else {
                at = (page * G + g) * page_size + key % page_size;
                s = sa_dot<T>(qs[warp], kcache + at * D, D) * scale;
                if (r1) s -= sk_distance_bias(b1, b2, pos - key);
            }
        }
        const float m_new = fmaxf(m, gb_warp_max(s));
        if (m_new == -INFINITY) continue;    // (nothing readable so far and no sink)
        const float corr = expf(m - m_new);  // (m = -inf: 0)
        const float p = at >= 0 ? expf(s - m_new) : 0.f;
        l = l * corr + gb_warp_sum(p);
        m = m_new;
#pragma unroll
        for (int j = 0; j < SA_MAX_DIM / 32; ++j) acc[j] *= corr;
        const int count = min(32, pos - base + 1);
        for (int t = 0; t < count; ++t) {
            const float pt = __shfl_sync(0xffffffffu, p, t);
            const long long vr = __shfl_sync(0xffffffffu, at, t);
            if (vr < 0) continue;
            const T* vp = vcache + vr * V;
#pragma unroll
            for (int j = 0; j < SA_MAX_DIM / 32; ++j) {
                const int i = lane + 32 * j;
                if (i < V) acc[j] = fmaf(pt, gb_to_float(vp[i]), acc[j]);
            }
        }
    }
    float f = l > 0.f ? 1.0f / l : 0.f;
    if (gate) f *= sk_sigmoid(gate[(size_t)row * ld_gate + head]);
    T* orow = out + ((size_t)row * H + head) * V;
#pragma unroll
    for (int j = 0; j < SA_MAX_DIM / 32; ++j) {
        const int i = lane + 32 * j;
        if (i < V) orow[i] = gb_from_float<T>(acc[j] * f);
    }
}

#define SK_COMMON_CHECKS(name)                                                                                                          \
    GB_REQUIRE(n >= 0 && H > 0 && G > 0 && H % G == 0, name ": heads %d must be a multiple of kv heads %d", H, G);                      \
    GB_REQUIRE(D > 0 && D <= SA_MAX_DIM && V > 0 && V <= SA_MAX_DIM, name ": head sizes %d / %d are outside 1..%d", D, V, SA_MAX_DIM);  \
    GB_REQUIRE(page_size > 0 && max_pages > 0 && window >= 0, name ": bad page geometry or window");                                    \
    GB_REQUIRE((r1 == nullptr) == (r2 == nullptr), name ": the distance bias needs both of its numbers per head");                      \
    GB_REQUIRE(gate == nullptr || ld_gate >= H, name ": rows of gate logits are too short");

GB_EXPORT int gb_sink_attention_rows(const void* q, void* out, int dtype, const void* kcache, const void* vcache, const int* block_tables,
                                     int max_pages, const int* row_seq, const int* positions, const float* r1, const float* r2,
                                     const float* sink, const float* gate, long long ld_gate, int n, int H, int G, int D, int V,
                                     int page_size, long long num_pages, float scale, int window, int* status, cudaStream_t stream) {
    SK_COMMON_CHECKS("gb_sink_attention_rows")
    if (n == 0) return 0;
    const int blocks = gb_ceil_div((long long)n * H, SK_WARPS);
    if (dtype == GB_F32)
        gb_launch(GB_PDL_ATTENTION, sink_attention_rows_kernel<float>, dim3(blocks), dim3(SK_WARPS * 32), 0, stream, (const float*)q,
                  (float*)out, (const float*)kcache, (const float*)vcache, block_tables, max_pages, row_seq, positions, r1, r2, sink, gate,
                  ld_gate, n, H, G, D, V, page_size, num_pages, scale, window, status);
    else if (dtype == GB_BF16)
        gb_launch(GB_PDL_ATTENTION, sink_attention_rows_kernel<__nv_bfloat16>, dim3(blocks), dim3(SK_WARPS * 32), 0, stream,
                  (const __nv_bfloat16*)q, (__nv_bfloat16*)out, (const __nv_bfloat16*)kcache, (const __nv_bfloat16*)vcache, block_tables,
                  max_pages, row_seq, positions, r1, r2, sink, gate, ld_gate, n, H, G, D, V, page_size, num_pages, scale, window, status);
    else
        GB_REQUIRE(false, "gb_sink_attention_rows: unsupported dtype %d", dtype);
    return gb_check_launch("gb_sink_attention_rows");
}

// ----------------------------------------------------------------------------------------------
// Single decoded tokens: one block of 8 warps per (row, R heads of one key/value group). The warps take the row's visible
// keys 32 at a time in turn (warp w the chunks w, w + 8, ...). Per chunk a lane first looks up the page of "its" key; then
// the value rows of all 32 keys are asked for in 16-byte pieces (LPK lanes cover one key's row, and all LPK such loads are
// in flight together, before the scores exist: their addresses need only the page table); then the lane's key row is read
// whole and dotted with the R queries, the distance bias taken off. Every warp keeps a running maximum and a denominator
// per head of its own; a lane sums its 16-byte piece of channels over its keys. At the end the lanes that hold the same
// channels add up (shuffles), then the warps meet in shared memory, where their maxima, the sink's logit and the gate join
// (fixed order). The order of a row's sums depends on its position and the window alone. A value row must be 64, 128, 256
// or 512 bytes.
// ----------------------------------------------------------------------------------------------
constexpr int SKD_WARPS = 8;

template <typename T, int LPK, int R>
__global__ void __launch_bounds__(SKD_WARPS * 32) sink_attention_decode_kernel(
    const T* __restrict__ q, T* __restrict__ out, const T* __restrict__ kcache, const T* __restrict__ vcache,
    const int* __restrict__ block_tables, int max_pages, const int* __restrict__ row_seq, const int* __restrict__ positions,
    const float* __restrict__ r1, const float* __restrict__ r2, const float* __restrict__ sink, const float* __restrict__ gate,
    long long ld_gate, int n, int H, int G, int D, int V, int page_size, long long num_pages, float scale, int window,
    int* __restrict__ status) {
    constexpr int PN = SadPiece<T>::N;          // channels in a 16-byte piece
    constexpr int KPI = 32 / LPK;               // keys that one warp-wide load fetches
    __shared__ __align__(16) float qs[R * SA_MAX_DIM];        // the R heads' queries, D apart
    __shared__ float part[SKD_WARPS][R * SA_MAX_DIM / (R > 2 ? 2 : 1)];      // (R > 2 only with value rows of up to 128 channels)
    __shared__ float part_m[SKD_WARPS][R], part_l[SKD_WARPS][R];
    gb_pdl_launch_dependents();
    gb_pdl_wait();
    const int row = blockIdx.x, head = blockIdx.y * R;        // R consecutive heads of one key/value group
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (row >= n) return;
    const int pos = positions[row];
    if (pos < 0) return;
    if (pos / page_size >= max_pages) {
        if (threadIdx.x == 0) atomicOr(status, GB_STATUS_BAD_POSITION);
        return;
    }
    const int g = head / (H / G);
    const int* table = block_tables + (size_t)row_seq[row] * max_pages;
    const T* qrow = q + ((size_t)row * H + head) * D;
    for (int i = threadIdx.x; i < R * D; i += SKD_WARPS * 32) qs[i] = gb_to_float(qrow[i]);
    __syncthreads();
    float b1[R], b2[R], m[R], l[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        b1[r] = r1 ? r1[head + r] : 0.f;
        b2[r] = r1 ? r2[head + r] : 0.f;
        m[r] = -INFINITY;
        l[r] = 0.f;
    }
    const int first = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;
    const int chunks = (pos - first) / 32 + 1;
    const int sub = lane / LPK, piece = lane % LPK;     // this lane holds piece `piece` of the keys sub, sub + KPI, ...
    float acc[R][PN];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int c = 0; c < PN; ++c) acc[r][c] = 0.f;
    for (int c = warp; c < chunks; c += SKD_WARPS) {
        const int key = first + c * 32 + lane;
        long long at = -1;
        if (key <= pos) {
            const long long page = table[key / page_size];
            if (page < 0 || page >= num_pages) atomicOr(status, GB_STATUS_BAD_SLOT);
            else at = (page * G + g) * page_size + key % page_size;
        }
        uint4 raw[LPK];
#pragma unroll
        for (int r = 0; r < LPK; ++r) {
            const long long vr = __shfl_sync(0xffffffffu, at, r * KPI + sub);
            raw[r] = vr >= 0 ? *reinterpret_cast<const uint4*>(vcache + vr * V + piece * PN) : make_uint4(0u, 0u, 0u, 0u);
        }
        float s[R], p[R];
#pragma unroll
        for (int r = 0; r < R; ++r) s[r] = -INFINITY;
        if (at >= 0) {
            sad_dots<T, R>(qs, kcache + at * D, D, s);
#pragma unroll
            for (int r = 0; r < R; ++r) {
                s[r] *= scale;
                if (r1) s[r] -= sk_distance_bias(b1[r], b2[r], pos - key);
            }
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const float m_new = fmaxf(m[r], gb_warp_max(s[r]));
            const bool none = m_new == -INFINITY;                 // (warp-uniform: every key of the chunk was unreadable)
            const float corr = none ? 1.f : expf(m[r] - m_new);
            p[r] = (at >= 0 && !none) ? expf(s[r] - m_new) : 0.f;
            l[r] = l[r] * corr + p[r];                            // (this lane's keys only; the lanes add up at the end)
            m[r] = m_new;
#pragma unroll
            for (int e = 0; e < PN; ++e) acc[r][e] *= corr;
        }
#pragma unroll
        for (int v = 0; v < LPK; ++v) {
            float f[PN];
            SadPiece<T>::unpack(raw[v], f);
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const float pt = __shfl_sync(0xffffffffu, p[r], v * KPI + sub);
#pragma unroll
                for (int e = 0; e < PN; ++e) acc[r][e] = fmaf(pt, f[e], acc[r][e]);
            }
        }
    }
    // lanes with the same piece hold sums over different keys: add them (fixed order), then the warps
#pragma unroll
    for (int o = LPK; o < 32; o <<= 1)
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int e = 0; e < PN; ++e) acc[r][e] += __shfl_xor_sync(0xffffffffu, acc[r][e], o);
#pragma unroll
    for (int r = 0; r < R; ++r) l[r] = gb_warp_sum(l[r]);
    if (sub == 0) {
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int e = 0; e < PN; ++e) part[warp][r * V + piece * PN + e] = acc[r][e];
    }
    if (lane == 0) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            part_m[warp][r] = m[r];
            part_l[warp][r] = l[r];
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < R * V; i += SKD_WARPS * 32) {      // (the R heads' outputs are neighbours: head * V + channel)
        const int r = i / V;
        float top = sink ? sink[head + r] : -INFINITY;
#pragma unroll
        for (int w = 0; w < SKD_WARPS; ++w) top = fmaxf(top, part_m[w][r]);
        float t = 0.f, den = sink ? expf(sink[head + r] - top) : 0.f;
#pragma unroll
        for (int w = 0; w < SKD_WARPS; ++w) {
            const float c = part_m[w][r] == -INFINITY ? 0.f : expf(part_m[w][r] - top);
            t = fmaf(part[w][i], c, t);
            den = fmaf(part_l[w][r], c, den);
        }
        float f = den > 0.f ? 1.0f / den : 0.f;
        if (gate) f *= sk_sigmoid(gate[(size_t)row * ld_gate + head + r]);
        out[((size_t)row * H + head) * V + i] = gb_from_float<T>(t * f);
    }
}

// 1 if the decode kernel takes value rows of this many bytes
GB_EXPORT int gb_sink_attention_decode_supported(int value_row_bytes) {
    return value_row_bytes == 64 || value_row_bytes == 128 || value_row_bytes == 256 || value_row_bytes == 512 ? 1 : 0;
}

template <typename T>
static int skd_launch(const void* q, void* out, const void* kcache, const void* vcache, const int* block_tables, int max_pages,
                      const int* row_seq, const int* positions, const float* r1, const float* r2, const float* sink, const float* gate,
                      long long ld_gate, int n, int H, int G, int D, int V, int page_size, long long num_pages, float scale, int window,
                      int* status, cudaStream_t stream) {
    const int lpk = V * (int)sizeof(T) / 16;
    // With enough (row, key/value head) pairs to fill the GPU, the query heads of a group go four at a time through one
    // block, which then reads the group's keys and values once for the four; with few rows every head gets its own block.
    const int group = H / G;
    const bool together = group % 4 == 0 && V <= 128 && lpk <= 16 && (long long)n * (H / 4) >= 148;
#define SKD_CASE(L, RR)                                                                                                                  \
    if (lpk == L && (together ? 4 : 1) == RR)                                                                                            \
        gb_launch(GB_PDL_ATTENTION, sink_attention_decode_kernel<T, L, RR>, dim3(n, H / RR), dim3(SKD_WARPS * 32), 0, stream,            \
                  (const T*)q, (T*)out, (const T*)kcache, (const T*)vcache, block_tables, max_pages, row_seq, positions, r1, r2, sink,   \
                  gate, ld_gate, n, H, G, D, V, page_size, num_pages, scale, window, status);
    SKD_CASE(4, 1) SKD_CASE(8, 1) SKD_CASE(16, 1) SKD_CASE(32, 1) SKD_CASE(4, 4) SKD_CASE(8, 4) SKD_CASE(16, 4)
#undef SKD_CASE
    return gb_check_launch("gb_sink_attention_decode");
}

GB_EXPORT int gb_sink_attention_decode(const void* q, void* out, int dtype, const void* kcache, const void* vcache,
                                       const int* block_tables, int max_pages, const int* row_seq, const int* positions, const float* r1,
                                       const float* r2, const float* sink, const float* gate, long long ld_gate, int n, int H, int G,
                                       int D, int V, int page_size, long long num_pages, float scale, int window, int* status,
                                       cudaStream_t stream) {
    SK_COMMON_CHECKS("gb_sink_attention_decode")
    GB_REQUIRE(dtype == GB_F32 || dtype == GB_BF16, "gb_sink_attention_decode: unsupported dtype %d", dtype);
    GB_REQUIRE(gb_sink_attention_decode_supported(V * (dtype == GB_F32 ? 4 : 2)),
               "gb_sink_attention_decode: value size %d is not built (a value row must be 64, 128, 256 or 512 bytes)", V);
    GB_REQUIRE(((uintptr_t)vcache & 15) == 0, "gb_sink_attention_decode: the value cache must be 16-byte aligned");
    if (n == 0) return 0;
    if (dtype == GB_F32)
        return skd_launch<float>(q, out, kcache, vcache, block_tables, max_pages, row_seq, positions, r1, r2, sink, gate, ld_gate, n, H, G,
                                 D, V, page_size, num_pages, scale, window, status, stream);
    return skd_launch<__nv_bfloat16>(q, out, kcache, vcache, block_tables, max_pages, row_seq, positions, r1, r2, sink, gate, ld_gate, n,
                                     H, G, D, V, page_size, num_pages, scale, window, status, stream);
}

// ----------------------------------------------------------------------------------------------
// Prompt portions in bfloat16 on the tensor cores. A block is 64 consecutive rows of one request x one head; its 4 warps
// own 16 rows each. The keys any of the 64 rows can see, first_position - window + 1 .. last_position, pass in tiles of 64
// through shared memory (cp.async, two buffers, each key's row found through the block table): S = Q K^T with mma.sync
// m16n8k16; in float32 and in the base-2 domain t = S * (scale * log2 e) - r1 * log2(1 + r2 * distance), the window and the
// causal edge per element, a running maximum per row that starts at the sink's logit, weights 2^(t - m) rounded to
// bfloat16 as the A operand of O += P V (float32 sums), O rescaled when the maximum moves. At the end the sink's share
// joins the denominator and the gate multiplies the row. Head sizes 32, 64 or 128 for keys and for values.
// ----------------------------------------------------------------------------------------------
constexpr int SKT_BM = 64, SKT_BN = 64;
constexpr float SK_LOG2E = 1.4426950408889634f;

template <int D, int V>
__global__ void __launch_bounds__(128) sink_attention_tiles_kernel(
    const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ kcache,
    const __nv_bfloat16* __restrict__ vcache, const int* __restrict__ block_tables, int max_pages, const int* __restrict__ seq_first_row,
    const int* __restrict__ seq_start_pos, const float* __restrict__ r1, const float* __restrict__ r2, const float* __restrict__ sink,
    const float* __restrict__ gate, long long ld_gate, int num_seqs, int tiles_per_seq, int H, int G, int page_size, long long num_pages,
    float scale, int window, int* __restrict__ status) {
    constexpr int LDK = D + 8, LDV = V + 8;          // rows padded by 16 bytes: ldmatrix meets no bank twice
    extern __shared__ __align__(16) unsigned char skt_smem[];
    __nv_bfloat16* sq = reinterpret_cast<__nv_bfloat16*>(skt_smem);             // [64][LDK]
    __nv_bfloat16* sk = sq + SKT_BM * LDK;                                        // [2][64][LDK]
    __nv_bfloat16* sv = sk + 2 * SKT_BN * LDK;                                    // [2][64][LDV]
    gb_pdl_launch_dependents();
    gb_pdl_wait();
    const int seq = blockIdx.x / tiles_per_seq, tile = blockIdx.x % tiles_per_seq, head = blockIdx.y;
    if (seq >= num_seqs) return;
    const int start = seq_start_pos[seq];
    if (start < 0) return;
    const int r0 = seq_first_row[seq], len = seq_first_row[seq + 1] - r0;
    if (tile * SKT_BM >= len) return;
    const int rows = min(SKT_BM, len - tile * SKT_BM);
    const int row0 = r0 + tile * SKT_BM, p_lo = start + tile * SKT_BM, p_hi = p_lo + rows - 1;
    if (p_hi / page_size >= max_pages) {
        if (threadIdx.x == 0) atomicOr(status, GB_STATUS_BAD_POSITION);
        return;
    }
    const int k_lo = (window > 0 && p_lo + 1 > window) ? p_lo + 1 - window : 0;
    const int g = head / (H / G);
    const int* table = block_tables + (size_t)seq * max_pages;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // Q tile
    for (int chunk = tid; chunk < SKT_BM * (D / 8); chunk += 128) {
        const int r = chunk / (D / 8), c = (chunk % (D / 8)) * 8;
        sat_cp16(sq + r * LDK + c, q + ((size_t)(row0 + (r < rows ? r : 0)) * H + head) * D + c, r < rows);
    }
    auto stage = [&](int buf, int kb) {
        // two threads per key: one page look-up each, then half of the key's 16-byte pieces (key row, then value row)
        constexpr int CPK = (D + V) / 8;
        const int key = tid >> 1, kk = kb + key;
        long long page = kk <= p_hi ? table[kk / page_size] : -1;
        if (kk <= p_hi && (page < 0 || page >= num_pages)) {
            atomicOr(status, GB_STATUS_BAD_SLOT);
            page = -1;
        }
        const long long at = page < 0 ? 0 : (page * G + g) * page_size + kk % page_size;
#pragma unroll
        for (int i = 0; i < CPK / 2; ++i) {
            const int c = ((tid & 1) * (CPK / 2) + i) * 8;
            if (c < D) sat_cp16(sk + (buf * SKT_BN + key) * LDK + c, kcache + at * D + c, page >= 0);
            else sat_cp16(sv + (buf * SKT_BN + key) * LDV + (c - D), vcache + at * V + (c - D), page >= 0);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    const int n_tiles = (p_hi - k_lo) / SKT_BN + 1;
    stage(0, k_lo);                                   // (one group holds Q and the first keys)
    unsigned qf[D / 16][4];
    float o[V / 8][4];
#pragma unroll
    for (int j = 0; j < V / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    const float b1 = r1 ? r1[head] : 0.f, b2 = r1 ? r2[head] : 0.f;
    const float sink2 = sink ? sink[head] * SK_LOG2E : -INFINITY;                     // the sink's logit in the base-2 domain
    const float scale2 = scale * SK_LOG2E;
    const int my_pos0 = p_lo + warp * 16 + (lane >> 2), my_pos1 = my_pos0 + 8;       // positions of this thread's two rows
    float mrow[2] = {sink2, sink2}, lrow[2] = {0.f, 0.f};                             // (a thread's share of the denominator)
    // The bias depends on the distance alone, and a tile of 64 rows x 64 keys holds 127 distances: one logarithm per thread
    // and tile instead of one per score. sbias[i] belongs to the distance (p_lo - kb) + i - 63, which is row - key + 63
    // counted inside the tile; distances below zero (keys that no row of theirs sees) count as zero.
    __shared__ float sbias[128];
    const float* my_bias = sbias + 63 + warp * 16 + (lane >> 2) - (lane & 3) * 2;
    for (int t = 0; t < n_tiles; ++t) {
        const int kb = k_lo + t * SKT_BN, buf = t & 1;
        if (r1) sbias[tid] = b1 * log2f(fmaf(b2, (float)max(p_lo - kb + tid - 63, 0), 1.0f));   // (read after the barrier below)
        if (t + 1 < n_tiles) {
            stage(buf ^ 1, kb + SKT_BN);
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
        const bool any = kb <= w_hi && (window <= 0 || kb + SKT_BN - 1 > w_lo - window) && warp * 16 < rows;
        if (any) {
            float s[SKT_BN / 8][4];
#pragma unroll
            for (int j = 0; j < SKT_BN / 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
            const __nv_bfloat16* kt = sk + buf * SKT_BN * LDK;
#pragma unroll
            for (int kd = 0; kd < D / 16; ++kd) {
#pragma unroll
                for (int j2 = 0; j2 < SKT_BN / 16; ++j2) {
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
            // base-2 logits with the distance bias; the causal edge and the window per element, except in tiles that every
            // row of the warp sees whole (most of them); then the rows' maxima (a row lies in the four lanes of a quad)
            const bool whole = kb + SKT_BN - 1 <= w_lo && (window <= 0 || w_hi - kb < window) && w_hi <= p_hi;
            float mx[2] = {mrow[0], mrow[1]};
#pragma unroll
            for (int j = 0; j < SKT_BN / 8; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = kb + j * 8 + (lane & 3) * 2 + (e & 1);
                    const int pos = e < 2 ? my_pos0 : my_pos1;
                    float v = s[j][e] * scale2;
                    if (r1) v -= my_bias[(e >> 1) * 8 - j * 8 - (e & 1)];
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
                // (a row that has seen nothing yet and has no sink keeps -inf: its weights are zeros, not NaNs)
                corr[hrow] = mx[hrow] == -INFINITY ? 1.f : exp2f(mrow[hrow] - mx[hrow]);
                mrow[hrow] = mx[hrow];
                lrow[hrow] *= corr[hrow];
            }
            const float sub0 = mx[0] == -INFINITY ? 0.f : mx[0], sub1 = mx[1] == -INFINITY ? 0.f : mx[1];
#pragma unroll
            for (int j = 0; j < V / 8; ++j) {
                o[j][0] *= corr[0]; o[j][1] *= corr[0];
                o[j][2] *= corr[1]; o[j][3] *= corr[1];
            }
            unsigned pf[SKT_BN / 16][4];
#pragma unroll
            for (int j = 0; j < SKT_BN / 8; ++j) {
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
            const __nv_bfloat16* vt = sv + buf * SKT_BN * LDV;
#pragma unroll
            for (int kk = 0; kk < SKT_BN / 16; ++kk) {
#pragma unroll
                for (int n2 = 0; n2 < V / 16; ++n2) {
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
        if (sink) den += exp2f(sink2 - mrow[half]);          // (the maximum started at the sink's logit: at most 1)
        const int r = warp * 16 + (lane >> 2) + half * 8;
        if (r >= rows) continue;
        float f = den > 0.f ? 1.0f / den : 0.f;
        if (gate) f *= sk_sigmoid(gate[(size_t)(row0 + r) * ld_gate + head]);
        __nv_bfloat16* dst = out + ((size_t)(row0 + r) * H + head) * V;
#pragma unroll
        for (int j = 0; j < V / 8; ++j)
            *reinterpret_cast<__nv_bfloat162*>(dst + j * 8 + (lane & 3) * 2) = __floats2bfloat162_rn(o[j][half * 2] * f, o[j][half * 2 + 1] * f);
    }
}

GB_EXPORT int gb_sink_attention_tiles_supported(int D, int V) {
    return (D == 32 || D == 64 || D == 128) && (V == 32 || V == 64 || V == 128) ? 1 : 0;
}

template <int D, int V>
static int skt_launch(const void* q, void* out, const void* kcache, const void* vcache, const int* block_tables, int max_pages,
                      const int* seq_first_row, const int* seq_start_pos, const float* r1, const float* r2, const float* sink,
                      const float* gate, long long ld_gate, int num_seqs, int tiles_per_seq, int H, int G, int page_size,
                      long long num_pages, float scale, int window, int* status, cudaStream_t stream) {
    const size_t smem = ((size_t)3 * SKT_BM * (D + 8) + (size_t)2 * SKT_BN * (V + 8)) * 2;
    cudaFuncSetAttribute(sink_attention_tiles_kernel<D, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    gb_launch(GB_PDL_ATTENTION, sink_attention_tiles_kernel<D, V>, dim3(num_seqs * tiles_per_seq, H), dim3(128), smem, stream,
              (const __nv_bfloat16*)q, (__nv_bfloat16*)out, (const __nv_bfloat16*)kcache, (const __nv_bfloat16*)vcache, block_tables,
              max_pages, seq_first_row, seq_start_pos, r1, r2, sink, gate, ld_gate, num_seqs, tiles_per_seq, H, G, page_size, num_pages,
              scale, window, status);
    return gb_check_launch("gb_sink_attention_tiles");
}

GB_EXPORT int gb_sink_attention_tiles(const void* q, void* out, const void* kcache, const void* vcache, const int* block_tables,
                                      int max_pages, const int* seq_first_row, const int* seq_start_pos, const float* r1, const float* r2,
                                      const float* sink, const float* gate, long long ld_gate, int num_seqs, int max_rows_per_seq, int H,
                                      int G, int D, int V, int page_size, long long num_pages, float scale, int window, int* status,
                                      cudaStream_t stream) {
    const int n = num_seqs;
    SK_COMMON_CHECKS("gb_sink_attention_tiles")
    GB_REQUIRE(gb_sink_attention_tiles_supported(D, V), "gb_sink_attention_tiles: head sizes %d / %d are not built", D, V);
    GB_REQUIRE(max_rows_per_seq > 0, "gb_sink_attention_tiles: bad sizes");
    if (num_seqs == 0) return 0;
    const int tiles = gb_ceil_div(max_rows_per_seq, SKT_BM);
#define SKT_CASE(DD, VV)                                                                                                              \
    if (D == DD && V == VV)                                                                                                           \
        return skt_launch<DD, VV>(q, out, kcache, vcache, block_tables, max_pages, seq_first_row, seq_start_pos, r1, r2, sink, gate,   \
                                  ld_gate, num_seqs, tiles, H, G, page_size, num_pages, scale, window, status, stream);
    SKT_CASE(32, 32) SKT_CASE(32, 64) SKT_CASE(32, 128) SKT_CASE(64, 32) SKT_CASE(64, 64) SKT_CASE(64, 128) SKT_CASE(128, 32)
    SKT_CASE(128, 64) SKT_CASE(128, 128)
#undef SKT_CASE
    GB_REQUIRE(false, "gb_sink_attention_tiles: head sizes %d / %d are not built", D, V);
}
