// A routed feed-forward (mixture of experts) with sigmoid scores, a choice bias and a limit to the best groups of experts.
//
//   moe_route        per row: logits = W_router h in float32 (h in the activation dtype), scores s = sigmoid(logits);
//                    experts are chosen by s + correction, the weights use s alone. The experts form `groups` equal runs of
//                    neighbours; a run's score is the sum of its two largest choice scores (its only one, if it has one
//                    member); only experts of the `keep` best runs can be chosen, the others count as minus infinity. The
//                    `top` largest are taken (among equals the lowest index), each with the weight s * route_scale, not
//                    renormalised. Also the gate of a shared expert, sigmoid(w_gate . h), one number per row.
//                    With softmax_chosen the scores are the logits themselves (plus a stored bias per expert), the `top`
//                    largest are taken and their weights are the softmax over the chosen logits alone.
//                    An expert is either W_down relu(W_up h)^2 or (UNIT) W_down unit(W_gate h, W_up h) with the clamped
//                    gated unit g * sigmoid(slope g) * (u + 1), g = min(gate, limit), u = clamp(up, -limit, limit); its
//                    up matrix then holds gate row f and up row f as rows 2f and 2f + 1.
//   moe_expert_rows  one block per (row, chosen expert): act = relu(W_up[e] h)^2 in shared memory, then W_down[e] act,
//                    written as float32 per (row, choice). Reads the two matrices of one expert once per block: the
//                    form for few rows (decoding), and the float32 path's form for any number.
//   moe_combine      out[row] (+)= sum_k weight[row, k] * pair[row, k] + gate[row] * shared[row]; a fixed order of sums.
#include "common.cuh"

#include <math.h>

constexpr int MOE_MAX_EXPERTS = 512;
constexpr int MOE_ROUTE_THREADS = 1024;      // at most; the launch takes a warp per expert (and one for the shared gate)

__device__ __forceinline__ float moe_sigmoid(float v) { return 1.0f / (1.0f + expf(-v)); }

// sum over K of w[k] * x[k]; x float32 in shared memory, w a row of a matrix in global memory; all lanes get the sum
template <typename T>
__device__ __forceinline__ float moe_warp_dot(const T* __restrict__ w, const float* __restrict__ x, int K, int lane);

template <>
__device__ __forceinline__ float moe_warp_dot<float>(const float* __restrict__ w, const float* __restrict__ x, int K, int lane) {
    float d = 0.f;
    if (K % 4 == 0 && ((uintptr_t)w & 15) == 0) {
#pragma unroll 4
        for (int i = lane * 4; i < K; i += 128) {
            const float4 v = *reinterpret_cast<const float4*>(w + i);
            d = fmaf(v.x, x[i], d); d = fmaf(v.y, x[i + 1], d); d = fmaf(v.z, x[i + 2], d); d = fmaf(v.w, x[i + 3], d);
        }
    } else {
        for (int i = lane; i < K; i += 32) d = fmaf(w[i], x[i], d);
    }
    return gb_warp_sum(d);
}

template <>
__device__ __forceinline__ float moe_warp_dot<__nv_bfloat16>(const __nv_bfloat16* __restrict__ w, const float* __restrict__ x, int K,
                                                             int lane) {
    float d = 0.f;
    if (K % 8 == 0 && ((uintptr_t)w & 15) == 0) {
#pragma unroll 4
        for (int i = lane * 8; i < K; i += 256) {
            const uint4 raw = *reinterpret_cast<const uint4*>(w + i);
            const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                const float2 f = __bfloat1622float2(p[t]);
                d = fmaf(f.x, x[i + 2 * t], d);
                d = fmaf(f.y, x[i + 2 * t + 1], d);
            }
        }
    } else {
        for (int i = lane; i < K; i += 32) d = fmaf(__bfloat162float(w[i]), x[i], d);
    }
    return gb_warp_sum(d);
}

// index of the largest of v[0 .. count) (lowest index among equals) over a warp; every lane gets it; -1 if all are -inf
__device__ __forceinline__ int moe_warp_argmax(const float* v, int count, int lane) {
    float best = -INFINITY;
    int at = -1;
    for (int i = lane; i < count; i += 32) {
        const float c = v[i];
        if (c > best) { best = c; at = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oa = __shfl_xor_sync(0xffffffffu, at, o);
        if (oa >= 0 && (at < 0 || ob > best || (ob == best && oa < at))) { best = ob; at = oa; }
    }
    return at;
}

// The choice for one row, by one warp: `score`, `choice` (score + correction), `run_score` and `kept` are the row's arrays.
__device__ __forceinline__ void moe_choose(const float* score, float* choice, float* run_score, unsigned char* kept, int E, int top,
                                           int groups, int keep, float route_scale, int* choice_out, float* weight_out, int lane,
                                           bool softmax_chosen = false) {
    if (groups > 1 && keep < groups) {
        const int per = E / groups;
        for (int g = lane; g < groups; g += 32) {
            float a = -INFINITY, b = -INFINITY;          // the two largest of the run
            for (int i = 0; i < per; ++i) {
                const float c = choice[g * per + i];
                if (c > a) { b = a; a = c; } else if (c > b) { b = c; }
            }
            run_score[g] = per > 1 ? a + b : a;
            kept[g] = 0;
        }
        __syncwarp();
        for (int k = 0; k < keep; ++k) {
            const int g = moe_warp_argmax(run_score, groups, lane);
            __syncwarp();
            if (lane == 0 && g >= 0) { run_score[g] = -INFINITY; kept[g] = 1; }
            __syncwarp();
        }
        for (int e = lane; e < E; e += 32)
            if (!kept[e / per]) choice[e] = -INFINITY;
        __syncwarp();
    }
    // The chosen values wait in the row's run_score (its use above is over) and reach global memory once, at the end: a
    // store and a load of the same address per choice would put a trip to memory into each turn of this chain.
    for (int k = 0; k < top; ++k) {
        const int e = moe_warp_argmax(choice, E, lane);
        __syncwarp();
        if (lane == 0) {
            choice_out[k] = e;                                               // -1: fewer experts could be chosen than `top`
            run_score[k] = e >= 0 ? score[e] * route_scale : (softmax_chosen ? -INFINITY : 0.f);
            if (e >= 0) choice[e] = -INFINITY;
        }
        __syncwarp();
    }
    if (lane == 0) {
        if (softmax_chosen) {
            // run_score holds the chosen logits, the largest first: softmax over them alone
            const float m = run_score[0];
            float sum = 0.f;
            for (int k = 0; k < top; ++k) {
                const float w = run_score[k] > -INFINITY ? expf(run_score[k] - m) : 0.f;
                run_score[k] = w;
                sum += w;
            }
            const float inv = 1.0f / sum;
            for (int k = 0; k < top; ++k) weight_out[k] = run_score[k] * inv;
        } else {
            for (int k = 0; k < top; ++k) weight_out[k] = run_score[k];
        }
    }
}

// RB rows per block: a warp per expert (and one for the shared gate) reads its row of the router matrix once and dots it
// with the block's RB rows; then a warp per row chooses. RB = 1 for a handful of rows (shortest chain), 8 for many (the
// router matrix is read an eighth as often). EMAX bounds the experts (the arrays' size).
template <typename T, int RB, int EMAX>
__global__ void __launch_bounds__(RB > 1 ? MOE_ROUTE_THREADS / 2 : MOE_ROUTE_THREADS) moe_route_kernel(
    const T* __restrict__ h, int d, const float* __restrict__ w_router, const float* __restrict__ correction,
    const float* __restrict__ w_gate, const int* __restrict__ positions, int n, int E, int top, int groups, int keep,
    float route_scale, int* __restrict__ choice_out, float* __restrict__ weight_out, float* __restrict__ gate_out,
    const float* __restrict__ router_bias, int softmax_chosen) {
    extern __shared__ __align__(16) float moe_smem[];
    float* hx = moe_smem;                       // RB rows of d numbers (rows start 16-byte aligned: ldh is a multiple of 4)
    const int ldh = (d + 3) & ~3;
    __shared__ float score[RB][EMAX], choice[RB][EMAX], run_score[RB][EMAX];
    __shared__ unsigned char kept[RB][EMAX];
    gb_pdl_launch_dependents();
    gb_pdl_wait();
    const int row0 = blockIdx.x * RB;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = (int)(blockDim.x >> 5);
    bool any = false;
#pragma unroll
    for (int r = 0; r < RB; ++r) {
        const int row = row0 + r;
        const bool live = row < n && positions[row] >= 0;
        any = any || live;
        const T* src = h + (size_t)(live ? row : 0) * d;
        for (int i = threadIdx.x; i < d; i += blockDim.x) hx[r * ldh + i] = live ? gb_to_float(src[i]) : 0.f;
    }
    if (!any) return;
    __syncthreads();
    for (int e = warp; e < E + (w_gate ? 1 : 0); e += warps) {
        const float* wrow = e < E ? w_router + (size_t)e * d : w_gate;
        float acc[RB];
#pragma unroll
        for (int r = 0; r < RB; ++r) acc[r] = 0.f;
        if (d % 4 == 0 && ((uintptr_t)wrow & 15) == 0) {
#pragma unroll 4
            for (int i = lane * 4; i < d; i += 128) {
                const float4 v = *reinterpret_cast<const float4*>(wrow + i);
#pragma unroll
                for (int r = 0; r < RB; ++r) {
                    const float4 x = *reinterpret_cast<const float4*>(hx + r * ldh + i);
                    acc[r] = fmaf(v.x, x.x, acc[r]); acc[r] = fmaf(v.y, x.y, acc[r]);
                    acc[r] = fmaf(v.z, x.z, acc[r]); acc[r] = fmaf(v.w, x.w, acc[r]);
                }
            }
        } else {
            for (int i = lane; i < d; i += 32) {
                const float v = wrow[i];
#pragma unroll
                for (int r = 0; r < RB; ++r) acc[r] = fmaf(v, hx[r * ldh + i], acc[r]);
            }
        }
#pragma unroll
        for (int r = 0; r < RB; ++r) {
            const float z = gb_warp_sum(acc[r]);
            const int row = row0 + r;
            if (lane == 0 && row < n && positions[row] >= 0) {
                const float sg = moe_sigmoid(z);
                if (e < E && softmax_chosen) {
                    score[r][e] = choice[r][e] = z + (router_bias ? router_bias[e] : 0.f);
                } else if (e < E) {
                    score[r][e] = sg;
                    choice[r][e] = sg + (correction ? correction[e] : 0.f);
                } else {
                    gate_out[row] = sg;
                }
            }
        }
    }
    __syncthreads();
    for (int r = warp; r < RB; r += warps) {
        const int row = row0 + r;
        if (row < n && positions[row] >= 0)
            moe_choose(score[r], choice[r], run_score[r], kept[r], E, top, groups, keep, softmax_chosen ? 1.0f : route_scale,
                       choice_out + (size_t)row * top, weight_out + (size_t)row * top, lane, softmax_chosen != 0);
    }
}

template <typename T, int RB, int EMAX>
static void moe_route_launch(const void* h, int d, const float* w_router, const float* correction, const float* w_gate,
                             const int* positions, int n, int E, int top, int groups, int keep, float route_scale, int* choice_out,
                             float* weight_out, float* gate_out, const float* router_bias, int softmax_chosen, cudaStream_t stream) {
    const size_t smem = (size_t)RB * ((d + 3) & ~3) * 4;
    int warps = E + (w_gate ? 1 : 0);
    const int most = (RB > 1 ? MOE_ROUTE_THREADS / 2 : MOE_ROUTE_THREADS) / 32, least = RB > 4 ? RB : 4;
    warps = warps < least ? least : (warps > most ? most : warps);
    if (smem > 32 * 1024) cudaFuncSetAttribute(moe_route_kernel<T, RB, EMAX>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    gb_launch(GB_PDL_ELEMENTWISE, moe_route_kernel<T, RB, EMAX>, dim3(gb_ceil_div(n, RB)), dim3(32 * warps), smem, stream, (const T*)h, d,
              w_router, correction, w_gate, positions, n, E, top, groups, keep, route_scale, choice_out, weight_out, gate_out, router_bias,
              softmax_chosen);
}

GB_EXPORT int gb_moe_route(const void* h, int h_dtype, int d, const float* w_router, const float* correction, const float* w_gate,
                           const int* positions, int n, int E, int top, int groups, int keep, float route_scale, int* choice_out,
                           float* weight_out, float* gate_out, const float* router_bias, int softmax_chosen, cudaStream_t stream) {
    GB_REQUIRE(!softmax_chosen || (groups == 1 && correction == nullptr), "gb_moe_route: softmax over the chosen logits goes with neither groups nor a correction");
    GB_REQUIRE(n >= 0 && d > 0 && E > 0 && E <= MOE_MAX_EXPERTS && top > 0 && top <= E, "gb_moe_route: bad sizes (experts %d, top %d)", E,
               top);
    GB_REQUIRE(groups >= 1 && E % groups == 0 && keep >= 1 && keep <= groups, "gb_moe_route: %d experts in %d groups, %d kept", E, groups,
               keep);
    GB_REQUIRE((size_t)d * 4 <= 160 * 1024, "gb_moe_route: a row of %d numbers does not fit shared memory", d);
    GB_REQUIRE(w_gate == nullptr || gate_out != nullptr, "gb_moe_route: a gate needs its output");
    GB_REQUIRE(h_dtype == GB_F32 || h_dtype == GB_BF16, "gb_moe_route: unsupported dtype %d", h_dtype);
    if (n == 0) return 0;
    // eight rows per block when there are many rows, the experts are few enough for the block's arrays and eight rows fit
    const bool many = n > 256 && E <= 128 && (size_t)8 * ((d + 3) & ~3) * 4 <= 160 * 1024;      // (below: too few blocks to fill the GPU)
#define MOE_ROUTE_GO(T)                                                                                                              \
    if (many)                                                                                                                        \
        moe_route_launch<T, 8, 128>(h, d, w_router, correction, w_gate, positions, n, E, top, groups, keep, route_scale, choice_out,  \
                                    weight_out, gate_out, router_bias, softmax_chosen, stream);                                      \
    else                                                                                                                             \
        moe_route_launch<T, 1, MOE_MAX_EXPERTS>(h, d, w_router, correction, w_gate, positions, n, E, top, groups, keep, route_scale,  \
                                                choice_out, weight_out, gate_out, router_bias, softmax_chosen, stream);
    if (h_dtype == GB_F32) { MOE_ROUTE_GO(float) } else { MOE_ROUTE_GO(__nv_bfloat16) }
#undef MOE_ROUTE_GO
    return gb_check_launch("gb_moe_route");
}

// ----------------------------------------------------------------------------------------------
// One block per (row, choice k): pair[row, k, :] = W_down[e] relu(W_up[e] h[row])^2, e = choice[row, k].
// w_up [E * ff, d], w_down [E * d, ff] (the experts' matrices stacked by rows).
// ----------------------------------------------------------------------------------------------
constexpr int MOE_ROWS_THREADS = 256;

template <typename T>
__global__ void __launch_bounds__(MOE_ROWS_THREADS) moe_expert_rows_kernel(
    const T* __restrict__ h, int d, const T* __restrict__ w_up, const T* __restrict__ w_down, int ff, const int* __restrict__ choice,
    const int* __restrict__ positions, int n, int E, int top, float* __restrict__ pair) {
    extern __shared__ __align__(16) float moe_smem[];
    float* hx = moe_smem;            // d
    float* act = moe_smem + ((d + 3) & ~3);     // ff
    gb_pdl_launch_dependents();
    gb_pdl_wait();
    const int row = blockIdx.x, k = blockIdx.y;
    if (row >= n || positions[row] < 0) return;
    const int e = choice[(size_t)row * top + k];
    float* dst = pair + ((size_t)row * top + k) * d;
    if (e < 0 || e >= E) {
        for (int i = threadIdx.x; i < d; i += MOE_ROWS_THREADS) dst[i] = 0.f;
        return;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const T* src = h + (size_t)row * d;
    for (int i = threadIdx.x; i < d; i += MOE_ROWS_THREADS) hx[i] = gb_to_float(src[i]);
    __syncthreads();
    const T* up = w_up + (size_t)e * ff * d;
    for (int f = warp; f < ff; f += MOE_ROWS_THREADS / 32) {
        const float a = fmaxf(moe_warp_dot<T>(up + (size_t)f * d, hx, d, lane), 0.f);
        if (lane == 0) act[f] = a * a;
    }
    __syncthreads();
    const T* down = w_down + (size_t)e * d * ff;
    for (int c = warp; c < d; c += MOE_ROWS_THREADS / 32) {
        const float o = moe_warp_dot<T>(down + (size_t)c * ff, act, ff, lane);
        if (lane == 0) dst[c] = o;
    }
}

GB_EXPORT int gb_moe_expert_rows(const void* h, int dtype, int d, const void* w_up, const void* w_down, int ff, const int* choice,
                                 const int* positions, int n, int E, int top, float* pair, cudaStream_t stream) {
    GB_REQUIRE(n >= 0 && d > 0 && ff > 0 && E > 0 && top > 0, "gb_moe_expert_rows: bad sizes");
    const size_t smem = ((size_t)((d + 3) & ~3) + ff) * 4;
    GB_REQUIRE(smem <= 200 * 1024, "gb_moe_expert_rows: a row of %d and %d hidden numbers do not fit shared memory", d, ff);
    if (n == 0) return 0;
    dim3 grid(n, top);
    if (dtype == GB_F32) {
        if (smem > 32 * 1024) cudaFuncSetAttribute(moe_expert_rows_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        gb_launch(GB_PDL_GEMM, moe_expert_rows_kernel<float>, grid, dim3(MOE_ROWS_THREADS), smem, stream, (const float*)h, d,
                  (const float*)w_up, (const float*)w_down, ff, choice, positions, n, E, top, pair);
    } else if (dtype == GB_BF16) {
        if (smem > 32 * 1024)
            cudaFuncSetAttribute(moe_expert_rows_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        gb_launch(GB_PDL_GEMM, moe_expert_rows_kernel<__nv_bfloat16>, grid, dim3(MOE_ROWS_THREADS), smem, stream, (const __nv_bfloat16*)h,
                  d, (const __nv_bfloat16*)w_up, (const __nv_bfloat16*)w_down, ff, choice, positions, n, E, top, pair);
    } else {
        GB_REQUIRE(false, "gb_moe_expert_rows: unsupported dtype %d", dtype);
    }
    return gb_check_launch("gb_moe_expert_rows");
}

// ----------------------------------------------------------------------------------------------
// out[row, :] (+)= sum_k weight[row, k] * pair[row, k, :] + gate[row] * shared[row, :]
// ----------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) moe_combine_kernel(const float* __restrict__ pair, const float* __restrict__ weight, int top,
                                                          const float* __restrict__ shared, long long lds, const float* __restrict__ gate,
                                                          const int* __restrict__ positions, float* __restrict__ out, long long ldo,
                                                          int n, int d, int accumulate) {
    gb_pdl_launch_dependents();
    gb_pdl_wait();
    const int row = blockIdx.x;
    if (row >= n || positions[row] < 0) return;
    const float g = gate ? gate[row] : 1.f;
    for (int j = threadIdx.x; j < d; j += blockDim.x) {
        float a = 0.f;
        for (int k = 0; k < top; ++k) a = fmaf(weight[(size_t)row * top + k], pair[((size_t)row * top + k) * d + j], a);
        if (shared) a = fmaf(g, shared[(size_t)row * lds + j], a);
        float* o = out + (size_t)row * ldo + j;
        *o = accumulate ? *o + a : a;
    }
}

GB_EXPORT int gb_moe_combine(const float* pair, const float* weight, int top, const float* shared, long long lds, const float* gate,
                             const int* positions, float* out, long long ldo, int n, int d, int accumulate, cudaStream_t stream) {
    GB_REQUIRE(n >= 0 && d > 0 && top > 0, "gb_moe_combine: bad sizes");
    if (n == 0) return 0;
    gb_launch(GB_PDL_ELEMENTWISE, moe_combine_kernel, dim3(n), dim3(256), 0, stream, pair, weight, top, shared, lds, gate, positions, out,
              ldo, n, d, accumulate);
    return gb_check_launch("gb_moe_combine");
}

// ----------------------------------------------------------------------------------------------
// The two halves of moe_expert_rows as kernels of their own, many blocks per (row, choice): the form for a handful of rows
// (decoding), where one block per pair would leave most of the GPU idle. act float32 [n * top, ff].
//   up:   act[pair, f]  = relu(W_up[e][f, :] . h[row])^2         grid (pairs, ceil(ff / 8)), a warp per f
//   down: pair[pair, c] = W_down[e][c, :] . act[pair, :]         grid (pairs, ceil(d / 8)), a warp per c
// ----------------------------------------------------------------------------------------------
template <typename T, bool UP>
__global__ void __launch_bounds__(256) moe_half_rows_kernel(const void* __restrict__ in_, long long ld_in, const T* __restrict__ w, int N,
                                                            int K, const int* __restrict__ choice, const int* __restrict__ positions,
                                                            int n, int E, int top, float* __restrict__ out, long long ld_out,
                                                            int unit, float limit, float slope) {
    extern __shared__ __align__(16) float moe_smem[];
    float* x = moe_smem;       // K numbers: the row h (UP) or the pair's activations (DOWN)
    const int pair = blockIdx.x, row = pair / top;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int c = blockIdx.y * 8 + warp;
    gb_pdl_launch_dependents();
    gb_pdl_wait();                // (the choice is the router kernel's output: nothing of it may be read before this)
    const int e = (row < n && positions[row] >= 0) ? choice[pair] : -2;
    // (with the gated unit an expert has 2N rows: output c reads its gate row 2c and its up row 2c + 1)
    const T* wrow = (e >= 0 && e < E && c < N) ? w + ((size_t)e * N + c) * K * (UP && unit ? 2 : 1) : nullptr;
    if (e == -2) return;
    if (e < 0 || e >= E) {
        if (c < N && lane == 0) out[(size_t)pair * ld_out + c] = 0.f;
        return;
    }
    if (UP) {
        const T* src = (const T*)in_ + (size_t)row * ld_in;
        for (int i = threadIdx.x; i < K; i += 256) x[i] = gb_to_float(src[i]);
    } else {
        const float* src = (const float*)in_ + (size_t)pair * ld_in;
        for (int i = threadIdx.x; i < K; i += 256) x[i] = src[i];
    }
    __syncthreads();
    if (wrow == nullptr) return;
    float v = moe_warp_dot<T>(wrow, x, K, lane);
    if (UP && unit) {
        v = gb_clamped_unit(v, moe_warp_dot<T>(wrow + K, x, K, lane), limit, slope);
    } else if (UP) {
        v = fmaxf(v, 0.f);
        v *= v;
    }
    if (lane == 0) out[(size_t)pair * ld_out + c] = v;
}

template <typename T>
static int moe_half_rows_launch(const void* h, int d, const T* w_up, const T* w_down, int ff, const int* choice, const int* positions,
                                int n, int E, int top, float* act, float* pair, int unit, float limit, float slope, cudaStream_t stream) {
    const size_t smem_up = (size_t)d * 4, smem_down = (size_t)ff * 4;
    if (smem_up > 32 * 1024)
        cudaFuncSetAttribute(moe_half_rows_kernel<T, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_up);
    if (smem_down > 32 * 1024)
        cudaFuncSetAttribute(moe_half_rows_kernel<T, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_down);
    gb_launch(GB_PDL_GEMM, moe_half_rows_kernel<T, true>, dim3(n * top, gb_ceil_div(ff, 8)), dim3(256), smem_up, stream, h, (long long)d,
              w_up, ff, d, choice, positions, n, E, top, act, (long long)ff, unit, limit, slope);
    int rc = gb_check_launch("gb_moe_expert_halves (up)");
    if (rc) return rc;
    gb_launch(GB_PDL_GEMM, moe_half_rows_kernel<T, false>, dim3(n * top, gb_ceil_div(d, 8)), dim3(256), smem_down, stream,
              (const void*)act, (long long)ff, w_down, d, ff, choice, positions, n, E, top, pair, (long long)d, 0, 0.f, 0.f);
    return gb_check_launch("gb_moe_expert_halves (down)");
}

GB_EXPORT int gb_moe_expert_halves(const void* h, int dtype, int d, const void* w_up, const void* w_down, int ff, const int* choice,
                                   const int* positions, int n, int E, int top, float* act, float* pair, int unit, float limit, float slope,
                                   cudaStream_t stream) {
    GB_REQUIRE(n >= 0 && d > 0 && ff > 0 && E > 0 && top > 0, "gb_moe_expert_halves: bad sizes");
    GB_REQUIRE((size_t)d * 4 <= 200 * 1024 && (size_t)ff * 4 <= 200 * 1024, "gb_moe_expert_halves: rows of %d / %d numbers do not fit", d, ff);
    if (n == 0) return 0;
    if (dtype == GB_F32)
        return moe_half_rows_launch<float>(h, d, (const float*)w_up, (const float*)w_down, ff, choice, positions, n, E, top, act, pair, unit,
                                           limit, slope, stream);
    if (dtype == GB_BF16)
        return moe_half_rows_launch<__nv_bfloat16>(h, d, (const __nv_bfloat16*)w_up, (const __nv_bfloat16*)w_down, ff, choice, positions,
                                                   n, E, top, act, pair, unit, limit, slope, stream);
    GB_REQUIRE(false, "gb_moe_expert_halves: unsupported dtype %d", dtype);
}

// ----------------------------------------------------------------------------------------------
// Many rows (prompt portions, large batches), bfloat16: the (row, choice) pairs are sorted by expert, and the experts'
// products run as ONE grouped product per half on the tensor cores.
//   moe_sort            one block: counts per expert, where each expert's pairs start (offsets [E + 1]), where its 64-row
//                       tiles start (tile_start [E + 1]), and sorted[slot] = pair. The order of an expert's pairs is not
//                       fixed from run to run; no result depends on it (a pair's numbers do not depend on its slot).
//   moe_grouped_gemm    a block = 64 slots of one expert x 128 outputs, 8 warps of mma.sync m16n8k16 (bf16, float32 sums),
//                       operands staged by cp.async in a ring of three buffers of 64 columns. UP: rows of h gathered by pair, epilogue relu^2, act
//                       [slot, ff] bfloat16. DOWN: rows of act, float32 out scattered to pair[pair, :].
// ----------------------------------------------------------------------------------------------
constexpr int MG_BM = 64, MG_BN = 128, MG_BK = 64, MG_STAGES = 3;
constexpr int MG_LD = MG_BK + 8;             // (rows padded by 16 bytes: ldmatrix meets no bank twice)
constexpr int MG_SMEM = MG_STAGES * (MG_BM + MG_BN) * MG_LD * 2;
constexpr int MG_THREADS = 256;

__global__ void __launch_bounds__(1024) moe_sort_kernel(const int* __restrict__ choice, const int* __restrict__ positions, int n, int E,
                                                        int top, int* __restrict__ offsets, int* __restrict__ tile_start,
                                                        int* __restrict__ sorted) {
    __shared__ int count[MOE_MAX_EXPERTS], cursor[MOE_MAX_EXPERTS];
    gb_pdl_launch_dependents();
    gb_pdl_wait();
    for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
    __syncthreads();
    const int pairs = n * top;
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = positions[p / top] >= 0 ? choice[p] : -1;
        if (e >= 0 && e < E) atomicAdd(&count[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0, tiles = 0;
        for (int e = 0; e < E; ++e) {
            offsets[e] = at;
            tile_start[e] = tiles;
            cursor[e] = at;
            at += count[e];
            tiles += (count[e] + MG_BM - 1) / MG_BM;
        }
        offsets[E] = at;
        tile_start[E] = tiles;
    }
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = positions[p / top] >= 0 ? choice[p] : -1;
        if (e >= 0 && e < E) sorted[atomicAdd(&cursor[e], 1)] = p;
    }
}

__device__ __forceinline__ void mg_cp_async16(void* smem, const void* gmem, bool valid) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    const int bytes = valid ? 16 : 0;        // 0: the 16 bytes are filled with zeros, nothing is read
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(bytes));
}

template <bool UP>
__global__ void __launch_bounds__(MG_THREADS) moe_grouped_gemm_kernel(const __nv_bfloat16* __restrict__ A, long long lda,
                                                               const __nv_bfloat16* __restrict__ W, int N, int K,
                                                               const int* __restrict__ sorted, const int* __restrict__ offsets,
                                                               const int* __restrict__ tile_start, int E, int top,
                                                               void* __restrict__ C, long long ldc, int unit, float limit,
                                                               float slope) {
    extern __shared__ __align__(16) unsigned char mg_smem[];
    __nv_bfloat16* sa = reinterpret_cast<__nv_bfloat16*>(mg_smem);                 // [stages][BM][LD]
    __nv_bfloat16* sb = sa + MG_STAGES * MG_BM * MG_LD;                            // [stages][BN][LD]
    __shared__ int src_row[MG_BM];           // where each slot's input row is (UP: the token's row; DOWN: the slot), -1: none
    __shared__ int dst_row[MG_BM];           // where its output goes (UP: the slot; DOWN: the pair)
    gb_pdl_launch_dependents();
    gb_pdl_wait();
    const int tile = blockIdx.x;
    if (tile >= tile_start[E]) return;
    int lo = 0, hi = E;                      // the expert whose tiles hold this one: the last e with tile_start[e] <= tile
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (tile_start[mid] <= tile) lo = mid; else hi = mid;
    }
    const int e = lo;
    const int m0 = offsets[e] + (tile - tile_start[e]) * MG_BM, m_end = offsets[e + 1];
    const int n0 = blockIdx.y * MG_BN;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid < MG_BM) {
        const int slot = m0 + tid;
        const bool live = slot < m_end;
        const int pair = live ? sorted[slot] : -1;
        src_row[tid] = !live ? -1 : (UP ? pair / top : slot);
        dst_row[tid] = !live ? -1 : (UP ? slot : pair);
    }
    __syncthreads();
    const __nv_bfloat16* Wb = W + (size_t)e * N * K;
    const int steps = (K + MG_BK - 1) / MG_BK;
    // staging: rows of BK = 64 columns are 8 chunks of 16 bytes; 256 threads take 2 chunks of A and 4 of W each
    auto stage = [&](int st) {
        if (st < steps) {
            const int buf = st % MG_STAGES, k0 = st * MG_BK;
#pragma unroll
            for (int i = 0; i < (MG_BM * 8) / MG_THREADS; ++i) {
                const int chunk = tid + i * MG_THREADS, r = chunk >> 3, c = (chunk & 7) * 8;
                const int ar = src_row[r];
                const bool ka = k0 + c < K;
                mg_cp_async16(sa + (buf * MG_BM + r) * MG_LD + c, A + (size_t)(ar < 0 ? 0 : ar) * lda + (ka ? k0 + c : 0), ar >= 0 && ka);
            }
#pragma unroll
            for (int i = 0; i < (MG_BN * 8) / MG_THREADS; ++i) {
                const int chunk = tid + i * MG_THREADS, r = chunk >> 3, c = (chunk & 7) * 8;
                const int br = n0 + r;
                const bool ka = k0 + c < K;
                mg_cp_async16(sb + (buf * MG_BN + r) * MG_LD + c, Wb + (size_t)(br < N ? br : 0) * K + (ka ? k0 + c : 0), br < N && ka);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");      // (a group per round, empty past the end: the count stays in step)
    };
    const int wm = (warp >> 2) * 32, wn = (warp & 3) * 32;       // this warp's 32 x 32 piece of the tile (8 warps: 2 x 4)
    float acc[2][4][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int t = 0; t < 4; ++t) acc[i][j][t] = 0.f;
#pragma unroll
    for (int st = 0; st < MG_STAGES - 1; ++st) stage(st);
    for (int s = 0; s < steps; ++s) {
        asm volatile("cp.async.wait_group %0;" ::"n"(MG_STAGES - 2) : "memory");
        __syncthreads();                     // round s has landed for everyone, and everyone is done with round s - 1's buffer
        stage(s + MG_STAGES - 1);
        const __nv_bfloat16* ta = sa + (s % MG_STAGES) * MG_BM * MG_LD;
        const __nv_bfloat16* tb = sb + (s % MG_STAGES) * MG_BN * MG_LD;
#pragma unroll
        for (int kk = 0; kk < MG_BK; kk += 16) {
            unsigned a[2][4], b[4][2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const unsigned addr = (unsigned)__cvta_generic_to_shared(ta + (wm + i * 16 + (lane & 15)) * MG_LD + kk + (lane >> 4) * 8);
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                             : "=r"(a[i][0]), "=r"(a[i][1]), "=r"(a[i][2]), "=r"(a[i][3]) : "r"(addr));
            }
#pragma unroll
            for (int j = 0; j < 2; ++j) {      // two 8-column tiles of W per ldmatrix.x4: rows n, columns k
                const int nrow = wn + j * 16 + (lane & 7) + ((lane >> 4) << 3), kcol = kk + ((lane >> 3) & 1) * 8;
                const unsigned addr = (unsigned)__cvta_generic_to_shared(tb + nrow * MG_LD + kcol);
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                             : "=r"(b[2 * j][0]), "=r"(b[2 * j][1]), "=r"(b[2 * j + 1][0]), "=r"(b[2 * j + 1][1]) : "r"(addr));
            }
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                                 : "+f"(acc[i][j][0]), "+f"(acc[i][j][1]), "+f"(acc[i][j][2]), "+f"(acc[i][j][3])
                                 : "r"(a[i][0]), "r"(a[i][1]), "r"(a[i][2]), "r"(a[i][3]), "r"(b[j][0]), "r"(b[j][1]));
        }
    }
    // epilogue: thread holds rows (lane / 4) and (lane / 4 + 8) of each 16-row tile, columns 2 * (lane % 4), + 1
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r = wm + i * 16 + (lane >> 2) + half * 8;
            const int out_row = dst_row[r];
            if (out_row < 0) continue;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int col = n0 + wn + j * 8 + (lane & 3) * 2;
                float v0 = acc[i][j][half * 2], v1 = acc[i][j][half * 2 + 1];
                if (UP && unit) {
                    // neighbouring outputs are the gate sum and the up sum of one unit: N / 2 units per row
                    if (col + 1 < N) ((__nv_bfloat16*)C)[(size_t)out_row * ldc + (col >> 1)] = __float2bfloat16_rn(gb_clamped_unit(v0, v1, limit, slope));
                } else if (UP) {
                    v0 = fmaxf(v0, 0.f); v0 *= v0;
                    v1 = fmaxf(v1, 0.f); v1 *= v1;
                    __nv_bfloat16* o = (__nv_bfloat16*)C + (size_t)out_row * ldc + col;
                    if (col + 1 < N && (ldc & 1) == 0) *reinterpret_cast<__nv_bfloat162*>(o) = __floats2bfloat162_rn(v0, v1);
                    else {
                        if (col < N) o[0] = __float2bfloat16_rn(v0);
                        if (col + 1 < N) o[1] = __float2bfloat16_rn(v1);
                    }
                } else {
                    float* o = (float*)C + (size_t)out_row * ldc + col;
                    if (col < N) o[0] = v0;
                    if (col + 1 < N) o[1] = v1;
                }
            }
        }
}

GB_EXPORT int gb_moe_sort(const int* choice, const int* positions, int n, int E, int top, int* offsets, int* tile_start, int* sorted,
                          cudaStream_t stream) {
    GB_REQUIRE(n >= 0 && E > 0 && E <= MOE_MAX_EXPERTS && top > 0, "gb_moe_sort: bad sizes");
    if (n == 0) return 0;
    gb_launch(GB_PDL_ELEMENTWISE, moe_sort_kernel, dim3(1), dim3(1024), 0, stream, choice, positions, n, E, top, offsets, tile_start, sorted);
    return gb_check_launch("gb_moe_sort");
}

// 1 if the grouped tensor-core products take these sizes (rows of 16-byte pieces)
GB_EXPORT int gb_moe_grouped_supported(int d, int ff) { return d % 8 == 0 && ff % 8 == 0 ? 1 : 0; }

GB_EXPORT int gb_moe_grouped_gemm(const void* a, long long lda, const void* w, int N, int K, const int* sorted, const int* offsets,
                                  const int* tile_start, int E, int top, int pairs, void* c, long long ldc, int up, int unit, float limit,
                                  float slope, cudaStream_t stream) {
    GB_REQUIRE(!unit || (up && N % 2 == 0), "gb_moe_grouped_gemm: the gated unit belongs to the up half and needs pairs of rows");
    GB_REQUIRE(N > 0 && K > 0 && K % 8 == 0 && lda % 8 == 0 && pairs >= 0, "gb_moe_grouped_gemm: rows must be whole 16-byte pieces (K=%d)", K);
    GB_REQUIRE(((uintptr_t)a & 15) == 0 && ((uintptr_t)w & 15) == 0, "gb_moe_grouped_gemm: operands must be 16-byte aligned");
    if (pairs == 0) return 0;
    dim3 grid(gb_ceil_div(pairs, MG_BM) + E, gb_ceil_div(N, MG_BN));      // (at most this many tiles: blocks beyond the last return)
    cudaFuncSetAttribute(moe_grouped_gemm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, MG_SMEM);
    cudaFuncSetAttribute(moe_grouped_gemm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, MG_SMEM);
    if (up)
        gb_launch(GB_PDL_GEMM, moe_grouped_gemm_kernel<true>, grid, dim3(MG_THREADS), MG_SMEM, stream, (const __nv_bfloat16*)a, lda,
                  (const __nv_bfloat16*)w, N, K, sorted, offsets, tile_start, E, top, c, ldc, unit, limit, slope);
    else
        gb_launch(GB_PDL_GEMM, moe_grouped_gemm_kernel<false>, grid, dim3(MG_THREADS), MG_SMEM, stream, (const __nv_bfloat16*)a, lda,
                  (const __nv_bfloat16*)w, N, K, sorted, offsets, tile_start, E, top, c, ldc, 0, 0.f, 0.f);
    return gb_check_launch("gb_moe_grouped_gemm");
}
