// Attention without a softmax over the paged cache: the weight of a visible key is sigmoid(q.k * scale + bias[head]),
// on its own, not normalised over the keys; out = sum over visible keys of weight * v. A row at position p of its request
// sees keys max(0, p - window + 1) .. p (window 0: all of them). Query heads share key/value heads in groups. The key
// size (dim) and the value size (vdim) may differ. Scores, weights and sums are float32.
//
//   qk_norm_rope_write   per row: RMS norm of every query and key head over dim (one gain for all query heads, one for
//                        all key heads, eps inside the root), rotation of the first `rot` channels in neighbouring pairs
//                        (2i, 2i+1) by the angle float32(position) * inv_freq[i], q to the query buffer, k and v into the
//                        cache at the row's slot. Input: the float32 sums of the stacked projection q | k | v. Optionally
//                        the values are mixed on the way: values_in given, v <- (1 - lambda) v + lambda values_in[row]
//                        (lambda one float32 number on the device); values_out given, it receives the row's (mixed) v.
//   sigmoid_attention_rows  one warp per (row, head), any row (prompt portion or single token), both dtypes: 32 keys at a
//                        time from the first visible one, a lane per key for the scores, a lane per channel for the sum.
#include "common.cuh"
#include "paged_rows.cuh"

constexpr int SA_WARPS = 4;

template <typename T>
__global__ void __launch_bounds__(512) qk_norm_rope_write_kernel(
    const float* __restrict__ qkv, long long ld, const float* __restrict__ q_gain, const float* __restrict__ k_gain,
    const float* __restrict__ inv_freq, const int* __restrict__ positions, const int* __restrict__ slots, T* __restrict__ q_out,
    T* __restrict__ kcache, T* __restrict__ vcache, int n, int H, int G, int D, int V, int rot, float eps, int page_size,
    long long num_slots, int write_kv, int* __restrict__ status, float* __restrict__ values_out, const float* __restrict__ values_in,
    long long ld_values, const float* __restrict__ value_mix) {
    gb_pdl_launch_dependents();
    gb_pdl_wait();
    const int row = blockIdx.x;
    if (row >= n) return;
    const int pos = positions[row];
    if (pos < 0) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const float* src = qkv + (size_t)row * ld;
    long long slot = slots[row];
    bool store = write_kv != 0;
    if (store && (slot < 0 || slot >= num_slots)) {
        if (threadIdx.x == 0) atomicOr(status, GB_STATUS_BAD_SLOT);
        store = false;
    }
    const long long page = slot / page_size;
    const int off = (int)(slot % page_size);
    const int pairs = D / 2;          // (an odd last channel is handled apart)
    for (int head = warp; head < H + G; head += warps) {
        const bool is_q = head < H;
        if (!is_q && !store) continue;
        const float* x = src + (size_t)head * D;     // q heads, then k heads: contiguous in the stacked row
        const float* gain = is_q ? q_gain : k_gain;      // nullptr: the heads are not normed
        float r = 1.f;
        if (gain != nullptr) {
            float ss = 0.f;
            for (int i = lane; i < D; i += 32) ss = fmaf(x[i], x[i], ss);
            ss = gb_warp_sum(ss);
            r = 1.0f / sqrtf(ss / (float)D + eps);
        }
        T* dst = is_q ? q_out + ((size_t)row * H + head) * D
                      : kcache + ((page * G + (head - H)) * page_size + off) * D;
        for (int i = lane; i < pairs; i += 32) {
            float a = x[2 * i] * r, c = x[2 * i + 1] * r;
            if (gain != nullptr) {
                a *= gain[2 * i];
                c *= gain[2 * i + 1];
            }
            if (2 * i + 1 < rot) {
                float sn, cs;
                sincosf((float)pos * inv_freq[i], &sn, &cs);
                const float ra = a * cs - c * sn, rc = c * cs + a * sn;
                a = ra;
                c = rc;
            }
            dst[2 * i] = gb_from_float<T>(a);
            dst[2 * i + 1] = gb_from_float<T>(c);
        }
        if ((D & 1) && lane == 0) dst[D - 1] = gb_from_float<T>(x[D - 1] * r * (gain ? gain[D - 1] : 1.f));
    }
    if (store || values_out != nullptr) {
        const float* v = src + (size_t)(H + G) * D;
        const float lam = values_in != nullptr ? *value_mix : 0.f;
        for (int idx = threadIdx.x; idx < G * V; idx += blockDim.x) {
            const int g = idx / V, i = idx % V;
            float val = v[idx];
            if (values_in != nullptr) val = (1.0f - lam) * val + lam * values_in[(size_t)row * ld_values + idx];
            if (values_out != nullptr) values_out[(size_t)row * ld_values + idx] = val;
            if (store) vcache[((page * G + g) * page_size + off) * V + i] = gb_from_float<T>(val);
        }
    }
}

GB_EXPORT int gb_qk_norm_rope_write(const float* qkv, long long ld, const float* q_gain, const float* k_gain, const float* inv_freq,
                                    const int* positions, const int* slots, void* q_out, void* kcache, void* vcache, int dtype, int n,
                                    int H, int G, int D, int V, int rot, float eps, int page_size, long long num_slots, int write_kv,
                                    int* status, float* values_out, const float* values_in, long long ld_values,
                                    const float* value_mix, cudaStream_t stream) {
    GB_REQUIRE(n >= 0 && H > 0 && G > 0 && D > 0 && V > 0, "gb_qk_norm_rope_write: bad sizes");
    GB_REQUIRE(values_in == nullptr || value_mix != nullptr, "gb_qk_norm_rope_write: values to mix in need their weight");
    GB_REQUIRE((values_in == nullptr && values_out == nullptr) || ld_values >= (long long)G * V, "gb_qk_norm_rope_write: rows of values are too short");
    GB_REQUIRE(rot >= 0 && rot % 2 == 0 && rot <= D, "gb_qk_norm_rope_write: %d rotated channels of %d", rot, D);
    GB_REQUIRE(rot == 0 || inv_freq != nullptr, "gb_qk_norm_rope_write: a rotation needs its frequencies");
    if (n == 0) return 0;
    const dim3 block(32 * (H + G < 4 ? 4 : (H + G > 16 ? 16 : H + G)));      // a warp per head, up to 16 at a time
    if (dtype == GB_F32)
        gb_launch(GB_PDL_ELEMENTWISE, qk_norm_rope_write_kernel<float>, dim3(n), block, 0, stream, qkv, ld, q_gain, k_gain, inv_freq,
                  positions, slots, (float*)q_out, (float*)kcache, (float*)vcache, n, H, G, D, V, rot, eps, page_size, num_slots,
                  write_kv, status, values_out, values_in, ld_values, value_mix);
    else if (dtype == GB_BF16)
        gb_launch(GB_PDL_ELEMENTWISE, qk_norm_rope_write_kernel<__nv_bfloat16>, dim3(n), block, 0, stream, qkv, ld, q_gain, k_gain,
                  inv_freq, positions, slots, (__nv_bfloat16*)q_out, (__nv_bfloat16*)kcache, (__nv_bfloat16*)vcache, n, H, G, D, V,
                  rot, eps, page_size, num_slots, write_kv, status, values_out, values_in, ld_values, value_mix);
    else
        GB_REQUIRE(false, "gb_qk_norm_rope_write: unsupported dtype %d", dtype);
    return gb_check_launch("gb_qk_norm_rope_write");
}

template <typename T>
__global__ void __launch_bounds__(SA_WARPS * 32) sigmoid_attention_rows_kernel(
    const T* __restrict__ q, T* __restrict__ out, const T* __restrict__ kcache, const T* __restrict__ vcache,
    const int* __restrict__ block_tables, int max_pages, const int* __restrict__ row_seq, const int* __restrict__ positions,
    const float* __restrict__ head_bias, int n, int H, int G, int D, int V, int page_size, long long num_pages, float scale,
    int window, int* __restrict__ status) {
    __shared__ float qs[SA_WARPS][SA_MAX_DIM];
    gb_pdl_launch_dependents();
    gb_pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long task = (long long)blockIdx.x * SA_WARPS + warp;
    if (task >= (long long)n * H) return;
    const int row = (int)(task / H), head = (int)(task % H);
    const int g = head / (H / G);
    int pos = positions[row];
    if (pos < 0) return;
    if (pos / page_size >= max_pages) {      // a position the block table does not reach: reported, the row reads nothing
        if (lane == 0) atomicOr(status, GB_STATUS_BAD_POSITION);
        return;
    }
    const int* table = block_tables + (size_t)row_seq[row] * max_pages;
    const T* qrow = q + ((size_t)row * H + head) * D;
    for (int i = lane; i < D; i += 32) qs[warp][i] = gb_to_float(qrow[i]);
    __syncwarp();
    const float bias = head_bias ? head_bias[head] : 0.f;
    const int first = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;
    float acc[SA_MAX_DIM / 32];
#pragma unroll
    for (int j = 0; j < SA_MAX_DIM / 32; ++j) acc[j] = 0.f;
    for (int base = first; base <= pos; base += 32) {
        const int key = base + lane;
        float p = 0.f;
        long long at = -1;                   // (page * G + g) * page_size + offset of this lane's key
        if (key <= pos) {
            const long long page = table[key / page_size];
            if (page < 0 || page >= num_pages) {
                atomicOr(status, GB_STATUS_BAD_SLOT);
            } else {
                at = (page * G + g) * page_size + key % page_size;
                const float s = sa_dot<T>(qs[warp], kcache + at * D, D) * scale + bias;
                p = 1.0f / (1.0f + expf(-s));
            }
        }
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
    T* orow = out + ((size_t)row * H + head) * V;
#pragma unroll
    for (int j = 0; j < SA_MAX_DIM / 32; ++j) {
        const int i = lane + 32 * j;
        if (i < V) orow[i] = gb_from_float<T>(acc[j]);
    }
}

GB_EXPORT int gb_sigmoid_attention_rows(const void* q, void* out, int dtype, const void* kcache, const void* vcache,
                                        const int* block_tables, int max_pages, const int* row_seq, const int* positions,
                                        const float* head_bias, int n, int H, int G, int D, int V, int page_size, long long num_pages,
                                        float scale, int window, int* status, cudaStream_t stream) {
    GB_REQUIRE(n >= 0 && H > 0 && G > 0 && H % G == 0, "gb_sigmoid_attention_rows: heads %d must be a multiple of kv heads %d", H, G);
    GB_REQUIRE(D > 0 && D <= SA_MAX_DIM && V > 0 && V <= SA_MAX_DIM, "gb_sigmoid_attention_rows: head sizes %d / %d are outside 1..%d",
               D, V, SA_MAX_DIM);
    GB_REQUIRE(page_size > 0 && max_pages > 0 && window >= 0, "gb_sigmoid_attention_rows: bad page geometry or window");
    if (n == 0) return 0;
    const int blocks = gb_ceil_div((long long)n * H, SA_WARPS);
    if (dtype == GB_F32)
        gb_launch(GB_PDL_ATTENTION, sigmoid_attention_rows_kernel<float>, dim3(blocks), dim3(SA_WARPS * 32), 0, stream, (const float*)q,
                  (float*)out, (const float*)kcache, (const float*)vcache, block_tables, max_pages, row_seq, positions, head_bias, n, H,
                  G, D, V, page_size, num_pages, scale, window, status);
    else if (dtype == GB_BF16)
        gb_launch(GB_PDL_ATTENTION, sigmoid_attention_rows_kernel<__nv_bfloat16>, dim3(blocks), dim3(SA_WARPS * 32), 0, stream,
                  (const __nv_bfloat16*)q, (__nv_bfloat16*)out, (const __nv_bfloat16*)kcache, (const __nv_bfloat16*)vcache, block_tables,
                  max_pages, row_seq, positions, head_bias, n, H, G, D, V, page_size, num_pages, scale, window, status);
    else
        GB_REQUIRE(false, "gb_sigmoid_attention_rows: unsupported dtype %d", dtype);
    return gb_check_launch("gb_sigmoid_attention_rows");
}

// ----------------------------------------------------------------------------------------------
// Single decoded tokens: one block of 8 warps per (row, head). The warps take the row's visible keys 32 at a time in turn
// (warp w the chunks w, w + 8, ...). Per chunk a lane first looks up the page of "its" key; then the value rows of all 32
// keys are asked for in 16-byte pieces (LPK lanes cover one key's row, so a warp-wide load fetches 32 / LPK keys, and all
// LPK such loads are in flight together, before the scores exist: their addresses need only the page table); then the
// lane's key row is read whole and dotted with the query, the weight sigmoid(score) formed in float32 and handed to the
// lanes that hold that key's values. A lane sums its 16-byte piece of channels over its keys; at the end the lanes that
// hold the same channels add up (shuffles), then the warps (shared memory, fixed order). The order of a row's sums
// depends on its position and the window alone. A value row must be 64, 128, 256 or 512 bytes.
// ----------------------------------------------------------------------------------------------
constexpr int SAD_WARPS = 8;

template <typename T, int LPK, int R>
__global__ void __launch_bounds__(SAD_WARPS * 32) sigmoid_attention_decode_kernel(
    const T* __restrict__ q, T* __restrict__ out, const T* __restrict__ kcache, const T* __restrict__ vcache,
    const int* __restrict__ block_tables, int max_pages, const int* __restrict__ row_seq, const int* __restrict__ positions,
    const float* __restrict__ head_bias, int n, int H, int G, int D, int V, int page_size, long long num_pages, float scale,
    int window, int* __restrict__ status) {
    constexpr int PN = SadPiece<T>::N;          // channels in a 16-byte piece
    constexpr int KPI = 32 / LPK;               // keys that one warp-wide load fetches
    __shared__ __align__(16) float qs[R * SA_MAX_DIM];        // the R heads' queries, D apart
    __shared__ float part[SAD_WARPS][R * SA_MAX_DIM / (R > 2 ? 2 : 1)];      // (R > 2 only with value rows of up to 128 channels)
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
    for (int i = threadIdx.x; i < R * D; i += SAD_WARPS * 32) qs[i] = gb_to_float(qrow[i]);
    __syncthreads();
    float bias[R];
#pragma unroll
    for (int r = 0; r < R; ++r) bias[r] = head_bias ? head_bias[head + r] : 0.f;
    const int first = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;
    const int chunks = (pos - first) / 32 + 1;
    const int sub = lane / LPK, piece = lane % LPK;     // this lane holds piece `piece` of the keys sub, sub + KPI, ...
    float acc[R][PN];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int c = 0; c < PN; ++c) acc[r][c] = 0.f;
    for (int c = warp; c < chunks; c += SAD_WARPS) {
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
        float p[R];
#pragma unroll
        for (int r = 0; r < R; ++r) p[r] = 0.f;
        if (at >= 0) {
            float sc[R];
            sad_dots<T, R>(qs, kcache + at * D, D, sc);
#pragma unroll
            for (int r = 0; r < R; ++r) p[r] = 1.0f / (1.0f + expf(-(sc[r] * scale + bias[r])));
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
    if (sub == 0) {
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int e = 0; e < PN; ++e) part[warp][r * V + piece * PN + e] = acc[r][e];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < R * V; i += SAD_WARPS * 32) {      // (the R heads' outputs are neighbours: head * V + channel)
        float t = 0.f;
#pragma unroll
        for (int w = 0; w < SAD_WARPS; ++w) t += part[w][i];
        out[((size_t)row * H + head) * V + i] = gb_from_float<T>(t);
    }
}

// 1 if the decode kernel takes value rows of this many bytes
GB_EXPORT int gb_sigmoid_attention_decode_supported(int value_row_bytes) {
    return value_row_bytes == 64 || value_row_bytes == 128 || value_row_bytes == 256 || value_row_bytes == 512 ? 1 : 0;
}

template <typename T>
static int sad_launch(const void* q, void* out, const void* kcache, const void* vcache, const int* block_tables, int max_pages,
                      const int* row_seq, const int* positions, const float* head_bias, int n, int H, int G, int D, int V, int page_size,
                      long long num_pages, float scale, int window, int* status, cudaStream_t stream) {
    const int lpk = V * (int)sizeof(T) / 16;
    // With enough (row, key/value head) pairs to fill the GPU, the query heads of a group go four at a time through one
    // block, which then reads the group's keys and values once for the four; with few rows every head gets its own block.
    const int group = H / G;
    const bool together = group % 4 == 0 && V <= 128 && lpk <= 16 && (long long)n * (H / 4) >= 148;
#define SAD_CASE(L, RR)                                                                                                                  \
    if (lpk == L && (together ? 4 : 1) == RR)                                                                                            \
        gb_launch(GB_PDL_ATTENTION, sigmoid_attention_decode_kernel<T, L, RR>, dim3(n, H / RR), dim3(SAD_WARPS * 32), 0, stream,         \
                  (const T*)q, (T*)out, (const T*)kcache, (const T*)vcache, block_tables, max_pages, row_seq, positions, head_bias, n, H, \
                  G, D, V, page_size, num_pages, scale, window, status);
    SAD_CASE(4, 1) SAD_CASE(8, 1) SAD_CASE(16, 1) SAD_CASE(32, 1) SAD_CASE(4, 4) SAD_CASE(8, 4) SAD_CASE(16, 4)
#undef SAD_CASE
    return gb_check_launch("gb_sigmoid_attention_decode");
}

GB_EXPORT int gb_sigmoid_attention_decode(const void* q, void* out, int dtype, const void* kcache, const void* vcache,
                                          const int* block_tables, int max_pages, const int* row_seq, const int* positions,
                                          const float* head_bias, int n, int H, int G, int D, int V, int page_size, long long num_pages,
                                          float scale, int window, int* status, cudaStream_t stream) {
    GB_REQUIRE(n >= 0 && H > 0 && G > 0 && H % G == 0, "gb_sigmoid_attention_decode: heads %d must be a multiple of kv heads %d", H, G);
    GB_REQUIRE(dtype == GB_F32 || dtype == GB_BF16, "gb_sigmoid_attention_decode: unsupported dtype %d", dtype);
    GB_REQUIRE(D > 0 && D <= SA_MAX_DIM && V > 0 && V <= SA_MAX_DIM && gb_sigmoid_attention_decode_supported(V * (dtype == GB_F32 ? 4 : 2)),
               "gb_sigmoid_attention_decode: head sizes %d / %d are not built (a value row must be 64, 128, 256 or 512 bytes)", D, V);
    GB_REQUIRE(page_size > 0 && max_pages > 0 && window >= 0, "gb_sigmoid_attention_decode: bad page geometry or window");
    GB_REQUIRE(((uintptr_t)vcache & 15) == 0, "gb_sigmoid_attention_decode: the value cache must be 16-byte aligned");
    if (n == 0) return 0;
    if (dtype == GB_F32)
        return sad_launch<float>(q, out, kcache, vcache, block_tables, max_pages, row_seq, positions, head_bias, n, H, G, D, V, page_size,
                                 num_pages, scale, window, status, stream);
    return sad_launch<__nv_bfloat16>(q, out, kcache, vcache, block_tables, max_pages, row_seq, positions, head_bias, n, H, G, D, V,
                                     page_size, num_pages, scale, window, status, stream);
}

// ----------------------------------------------------------------------------------------------
// Prompt portions in bfloat16 on the tensor cores. A block is 64 consecutive rows of one request x one head; its 4 warps
// own 16 rows each. The keys any of the 64 rows can see, first_position - window + 1 .. last_position, pass in tiles of 64
// through shared memory (cp.async, two buffers, each key's row found through the block table): S = Q K^T with mma.sync
// m16n8k16, weights sigmoid(S * scale + bias) in float32 with the window and the causal edge applied per element, rounded
// to bfloat16 as the A operand of O += P V (float32 sums). No running maximum, no rescaling: a key's weight does not depend
// on the other keys. Head sizes 32, 64 or 128 for keys and for values, in any combination.
// ----------------------------------------------------------------------------------------------
constexpr int SAT_BM = 64, SAT_BN = 64;

template <int D, int V>
__global__ void __launch_bounds__(128) sigmoid_attention_tiles_kernel(
    const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ kcache,
    const __nv_bfloat16* __restrict__ vcache, const int* __restrict__ block_tables, int max_pages, const int* __restrict__ seq_first_row,
    const int* __restrict__ seq_start_pos, const float* __restrict__ head_bias, int num_seqs, int tiles_per_seq, int H, int G,
    int page_size, long long num_pages, float scale, int window, int* __restrict__ status) {
    constexpr int LDK = D + 8, LDV = V + 8;          // rows padded by 16 bytes: ldmatrix meets no bank twice
    extern __shared__ __align__(16) unsigned char sat_smem[];
    __nv_bfloat16* sq = reinterpret_cast<__nv_bfloat16*>(sat_smem);             // [64][LDK]
    __nv_bfloat16* sk = sq + SAT_BM * LDK;                                        // [2][64][LDK]
    __nv_bfloat16* sv = sk + 2 * SAT_BN * LDK;                                    // [2][64][LDV]
    gb_pdl_launch_dependents();
    gb_pdl_wait();
    const int seq = blockIdx.x / tiles_per_seq, tile = blockIdx.x % tiles_per_seq, head = blockIdx.y;
    if (seq >= num_seqs) return;
    const int start = seq_start_pos[seq];
    if (start < 0) return;
    const int r0 = seq_first_row[seq], len = seq_first_row[seq + 1] - r0;
    if (tile * SAT_BM >= len) return;
    const int rows = min(SAT_BM, len - tile * SAT_BM);
    const int row0 = r0 + tile * SAT_BM, p_lo = start + tile * SAT_BM, p_hi = p_lo + rows - 1;
    if (p_hi / page_size >= max_pages) {
        if (threadIdx.x == 0) atomicOr(status, GB_STATUS_BAD_POSITION);
        return;
    }
    const int k_lo = (window > 0 && p_lo + 1 > window) ? p_lo + 1 - window : 0;
    const int g = head / (H / G);
    const int* table = block_tables + (size_t)seq * max_pages;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // Q tile
    for (int chunk = tid; chunk < SAT_BM * (D / 8); chunk += 128) {
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
            if (c < D) sat_cp16(sk + (buf * SAT_BN + key) * LDK + c, kcache + at * D + c, page >= 0);
            else sat_cp16(sv + (buf * SAT_BN + key) * LDV + (c - D), vcache + at * V + (c - D), page >= 0);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    const int n_tiles = (p_hi - k_lo) / SAT_BN + 1;
    stage(0, k_lo);                                   // (one group holds Q and the first keys)
    unsigned qf[D / 16][4];
    float o[V / 8][4];
#pragma unroll
    for (int j = 0; j < V / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    const float bias = head_bias ? head_bias[head] : 0.f;
    const int my_pos0 = p_lo + warp * 16 + (lane >> 2), my_pos1 = my_pos0 + 8;       // positions of this thread's two rows
    for (int t = 0; t < n_tiles; ++t) {
        const int kb = k_lo + t * SAT_BN, buf = t & 1;
        if (t + 1 < n_tiles) {
            stage(buf ^ 1, kb + SAT_BN);
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
        const bool any = kb <= w_hi && (window <= 0 || kb + SAT_BN - 1 > w_lo - window) && warp * 16 < rows;
        if (any) {
            float s[SAT_BN / 8][4];
#pragma unroll
            for (int j = 0; j < SAT_BN / 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
            const __nv_bfloat16* kt = sk + buf * SAT_BN * LDK;
#pragma unroll
            for (int kd = 0; kd < D / 16; ++kd) {
#pragma unroll
                for (int j2 = 0; j2 < SAT_BN / 16; ++j2) {
                    unsigned b0, b1, b2, b3;
                    const int nrow = j2 * 16 + (lane & 7) + ((lane >> 4) << 3), kcol = kd * 16 + ((lane >> 3) & 1) * 8;
                    const unsigned addr = (unsigned)__cvta_generic_to_shared(kt + nrow * LDK + kcol);
                    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3) : "r"(addr));
                    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                                 : "+f"(s[2 * j2][0]), "+f"(s[2 * j2][1]), "+f"(s[2 * j2][2]), "+f"(s[2 * j2][3])
                                 : "r"(qf[kd][0]), "r"(qf[kd][1]), "r"(qf[kd][2]), "r"(qf[kd][3]), "r"(b0), "r"(b1));
                    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                                 : "+f"(s[2 * j2 + 1][0]), "+f"(s[2 * j2 + 1][1]), "+f"(s[2 * j2 + 1][2]), "+f"(s[2 * j2 + 1][3])
                                 : "r"(qf[kd][0]), "r"(qf[kd][1]), "r"(qf[kd][2]), "r"(qf[kd][3]), "r"(b2), "r"(b3));
                }
            }
            // weights: float32 sigmoid; the causal edge and the window per element, except in tiles that every row of the
            // warp sees whole (most of them)
            const bool whole = kb + SAT_BN - 1 <= w_lo && (window <= 0 || w_hi - kb < window) && w_hi <= p_hi;
            const float c1 = -scale * 1.4426950408889634f, c0 = -bias * 1.4426950408889634f;     // exp(-(s * scale + bias)) = 2^(s c1 + c0)
            unsigned pf[SAT_BN / 16][4];
#pragma unroll
            for (int j = 0; j < SAT_BN / 8; ++j) {
                float p[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    p[e] = __fdividef(1.0f, 1.0f + exp2f(fmaf(s[j][e], c1, c0)));      // (rounded to bfloat16 next)
                    if (!whole) {
                        const int key = kb + j * 8 + (lane & 3) * 2 + (e & 1);
                        const int pos = e < 2 ? my_pos0 : my_pos1;
                        const bool sees = key <= pos && (window <= 0 || pos - key < window) && pos <= p_hi;
                        p[e] = sees ? p[e] : 0.f;
                    }
                }
                const __nv_bfloat162 lo = __floats2bfloat162_rn(p[0], p[1]), hi = __floats2bfloat162_rn(p[2], p[3]);
                pf[j >> 1][(j & 1) * 2] = *reinterpret_cast<const unsigned*>(&lo);
                pf[j >> 1][(j & 1) * 2 + 1] = *reinterpret_cast<const unsigned*>(&hi);
            }
            const __nv_bfloat16* vt = sv + buf * SAT_BN * LDV;
#pragma unroll
            for (int kk = 0; kk < SAT_BN / 16; ++kk) {
#pragma unroll
                for (int n2 = 0; n2 < V / 16; ++n2) {
                    unsigned b0, b1, b2, b3;
                    const int krow = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, ncol = n2 * 16 + (lane >> 4) * 8;
                    const unsigned addr = (unsigned)__cvta_generic_to_shared(vt + krow * LDV + ncol);
                    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3) : "r"(addr));
                    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                                 : "+f"(o[2 * n2][0]), "+f"(o[2 * n2][1]), "+f"(o[2 * n2][2]), "+f"(o[2 * n2][3])
                                 : "r"(pf[kk][0]), "r"(pf[kk][1]), "r"(pf[kk][2]), "r"(pf[kk][3]), "r"(b0), "r"(b1));
                    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                                 : "+f"(o[2 * n2 + 1][0]), "+f"(o[2 * n2 + 1][1]), "+f"(o[2 * n2 + 1][2]), "+f"(o[2 * n2 + 1][3])
                                 : "r"(pf[kk][0]), "r"(pf[kk][1]), "r"(pf[kk][2]), "r"(pf[kk][3]), "r"(b2), "r"(b3));
                }
            }
        }
        __syncthreads();          // everyone is done with this buffer before the round after next overwrites it
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = warp * 16 + (lane >> 2) + half * 8;
        if (r >= rows) continue;
        __nv_bfloat16* dst = out + ((size_t)(row0 + r) * H + head) * V;
#pragma unroll
        for (int j = 0; j < V / 8; ++j)
            *reinterpret_cast<__nv_bfloat162*>(dst + j * 8 + (lane & 3) * 2) = __floats2bfloat162_rn(o[j][half * 2], o[j][half * 2 + 1]);
    }
}

GB_EXPORT int gb_sigmoid_attention_tiles_supported(int D, int V) {
    return (D == 32 || D == 64 || D == 128) && (V == 32 || V == 64 || V == 128) ? 1 : 0;
}

template <int D, int V>
static int sat_launch(const void* q, void* out, const void* kcache, const void* vcache, const int* block_tables, int max_pages,
                      const int* seq_first_row, const int* seq_start_pos, const float* head_bias, int num_seqs, int tiles_per_seq, int H,
                      int G, int page_size, long long num_pages, float scale, int window, int* status, cudaStream_t stream) {
    const size_t smem = ((size_t)3 * SAT_BM * (D + 8) + (size_t)2 * SAT_BN * (V + 8)) * 2;
    cudaFuncSetAttribute(sigmoid_attention_tiles_kernel<D, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    gb_launch(GB_PDL_ATTENTION, sigmoid_attention_tiles_kernel<D, V>, dim3(num_seqs * tiles_per_seq, H), dim3(128), smem, stream,
              (const __nv_bfloat16*)q, (__nv_bfloat16*)out, (const __nv_bfloat16*)kcache, (const __nv_bfloat16*)vcache, block_tables,
              max_pages, seq_first_row, seq_start_pos, head_bias, num_seqs, tiles_per_seq, H, G, page_size, num_pages, scale, window,
              status);
    return gb_check_launch("gb_sigmoid_attention_tiles");
}

GB_EXPORT int gb_sigmoid_attention_tiles(const void* q, void* out, const void* kcache, const void* vcache, const int* block_tables,
                                         int max_pages, const int* seq_first_row, const int* seq_start_pos, const float* head_bias,
                                         int num_seqs, int max_rows_per_seq, int H, int G, int D, int V, int page_size, long long num_pages,
                                         float scale, int window, int* status, cudaStream_t stream) {
    GB_REQUIRE(gb_sigmoid_attention_tiles_supported(D, V), "gb_sigmoid_attention_tiles: head sizes %d / %d are not built", D, V);
    GB_REQUIRE(num_seqs >= 0 && H > 0 && G > 0 && H % G == 0 && page_size > 0 && max_pages > 0 && window >= 0 && max_rows_per_seq > 0,
               "gb_sigmoid_attention_tiles: bad sizes");
    if (num_seqs == 0) return 0;
    const int tiles = gb_ceil_div(max_rows_per_seq, SAT_BM);
#define SAT_CASE(DD, VV)                                                                                                         \
    if (D == DD && V == VV)                                                                                                      \
        return sat_launch<DD, VV>(q, out, kcache, vcache, block_tables, max_pages, seq_first_row, seq_start_pos, head_bias, num_seqs, \
                                  tiles, H, G, page_size, num_pages, scale, window, status, stream);
    SAT_CASE(32, 32) SAT_CASE(32, 64) SAT_CASE(32, 128) SAT_CASE(64, 32) SAT_CASE(64, 64) SAT_CASE(64, 128) SAT_CASE(128, 32)
    SAT_CASE(128, 64) SAT_CASE(128, 128)
#undef SAT_CASE
    GB_REQUIRE(false, "gb_sigmoid_attention_tiles: head sizes %d / %d are not built", D, V);
}
