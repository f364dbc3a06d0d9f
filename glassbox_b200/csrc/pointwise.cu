// Small row-wise and element-wise kernels for layers that norm a branch before it joins the residual stream, for
// activations other than SwiGLU, and for a scaled head:
//   rmsnorm_add   x[r, :] += gain * y[r, :] / sqrt(mean(y[r, :]^2) + eps)   (float32 throughout); optionally y + bias in the
//                 place of y, and a copy of the new x[r, :] in the activation dtype
//   cast_rows     out[r, :] = x[rows[r], :] in the activation dtype
//   add_bias      y[r, :] += bias
//   clamped_glu   act[r, f] = g * sigmoid(slope * g) * (u + 1), g = min(gate + b, limit), u = clamp(up + b, -limit, limit)
//   relu2         out = max(in, 0)^2
//   scale         t *= s
//   gated_head_norm  out[r, h, :] = w * o[r, h, :] / sqrt(mean_v(o[r, h, :]^2) + eps) * sigmoid(gate[r, h, :])  (or * silu(gate))
//   gelu_glu      act[r, f] = gelu_tanh(gate[r, f]) * up[r, f]
//   scaled_sum    out (+)= a * x + b * y
#include "common.cuh"

// ----------------------------------------------------------------------------------------------
// A branch's output y (float32) is normalised and added into the residual x (float32). One block per row.
// ----------------------------------------------------------------------------------------------
template <int THREADS, typename T>
__global__ void __launch_bounds__(THREADS) rmsnorm_add_kernel(const float* __restrict__ y, long long ldy,
                                                              const float* __restrict__ gain, float* __restrict__ x,
                                                              long long ldx, int n, int d, float eps,
                                                              const float* __restrict__ bias, T* __restrict__ copy) {
    gb_pdl_launch_dependents();
    gb_pdl_wait();
    const int r = blockIdx.x;
    if (r >= n) return;
    const float* src = y + (size_t)r * ldy;
    float* dst = x + (size_t)r * ldx;
    __shared__ float partial[THREADS / 32];
    __shared__ float total;
    constexpr int VMAX = 4;
    const bool quick = d % 4 == 0 && d <= THREADS * 4 * VMAX && ((uintptr_t)src & 15) == 0 && ((uintptr_t)dst & 15) == 0 &&
                       ((uintptr_t)gain & 15) == 0 && ((uintptr_t)bias & 15) == 0;
    T* cp = copy ? copy + (size_t)r * d : nullptr;
    float4 v[VMAX], o[VMAX];
    float ss = 0.f;
    if (quick) {
#pragma unroll
        for (int i = 0; i < VMAX; ++i) {
            const int j = (i * THREADS + threadIdx.x) * 4;
            v[i] = j < d ? *reinterpret_cast<const float4*>(src + j) : make_float4(0.f, 0.f, 0.f, 0.f);
            o[i] = j < d ? *reinterpret_cast<const float4*>(dst + j) : make_float4(0.f, 0.f, 0.f, 0.f);
            if (bias != nullptr && j < d) {
                const float4 b = *reinterpret_cast<const float4*>(bias + j);
                v[i].x += b.x; v[i].y += b.y; v[i].z += b.z; v[i].w += b.w;
            }
        }
#pragma unroll
        for (int i = 0; i < VMAX; ++i) {
            ss = fmaf(v[i].x, v[i].x, ss); ss = fmaf(v[i].y, v[i].y, ss);
            ss = fmaf(v[i].z, v[i].z, ss); ss = fmaf(v[i].w, v[i].w, ss);
        }
    } else {
        for (int j = threadIdx.x; j < d; j += THREADS) {
            const float t = src[j] + (bias ? bias[j] : 0.f);
            ss = fmaf(t, t, ss);
        }
    }
    ss = gb_warp_sum(ss);
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
#pragma unroll
        for (int w = 0; w < THREADS / 32; ++w) t += partial[w];
        total = 1.0f / sqrtf(t / (float)d + eps);
    }
    __syncthreads();
    const float s = total;
    if (quick) {
#pragma unroll
        for (int i = 0; i < VMAX; ++i) {
            const int j = (i * THREADS + threadIdx.x) * 4;
            if (j < d) {
                const float4 g = *reinterpret_cast<const float4*>(gain + j);
                float4 w;
                w.x = o[i].x + g.x * (v[i].x * s);
                w.y = o[i].y + g.y * (v[i].y * s);
                w.z = o[i].z + g.z * (v[i].z * s);
                w.w = o[i].w + g.w * (v[i].w * s);
                *reinterpret_cast<float4*>(dst + j) = w;
                if (cp != nullptr) {
                    cp[j] = gb_from_float<T>(w.x); cp[j + 1] = gb_from_float<T>(w.y);
                    cp[j + 2] = gb_from_float<T>(w.z); cp[j + 3] = gb_from_float<T>(w.w);
                }
            }
        }
    } else {
        for (int j = threadIdx.x; j < d; j += THREADS) {
            const float w = dst[j] + gain[j] * ((src[j] + (bias ? bias[j] : 0.f)) * s);
            dst[j] = w;
            if (cp != nullptr) cp[j] = gb_from_float<T>(w);
        }
    }
}

// bias (optional, float32 [d]) is added to y first; copy (optional, [n, d] of dtype copy_dtype) receives the new x
GB_EXPORT int gb_rmsnorm_add(const float* y, long long ldy, const float* gain, float* x, long long ldx, int n, int d,
                             float eps, const float* bias, void* copy, int copy_dtype, cudaStream_t stream) {
    GB_REQUIRE(n >= 0 && d > 0, "gb_rmsnorm_add: bad sizes n=%d d=%d", n, d);
    GB_REQUIRE(copy == nullptr || copy_dtype == GB_F32 || copy_dtype == GB_BF16, "gb_rmsnorm_add: unsupported dtype %d", copy_dtype);
    if (n == 0) return 0;
    if (copy != nullptr && copy_dtype == GB_BF16)
        gb_launch(GB_PDL_ELEMENTWISE, rmsnorm_add_kernel<128, __nv_bfloat16>, dim3(n), dim3(128), 0, stream, y, ldy, gain, x, ldx, n, d,
                  eps, bias, (__nv_bfloat16*)copy);
    else
        gb_launch(GB_PDL_ELEMENTWISE, rmsnorm_add_kernel<128, float>, dim3(n), dim3(128), 0, stream, y, ldy, gain, x, ldx, n, d, eps,
                  bias, (float*)copy);
    return gb_check_launch("gb_rmsnorm_add");
}

// ----------------------------------------------------------------------------------------------
// out[r, :] = x[rows ? rows[r] : r, :], float32 -> the activation dtype (a branch that reads the residual as it is).
// ----------------------------------------------------------------------------------------------
template <typename T>
__global__ void cast_rows_kernel(const float* __restrict__ x, long long ldx, const int* __restrict__ rows, T* __restrict__ out, int n,
                                 int d) {
    gb_pdl_launch_dependents();
    gb_pdl_wait();
    const long long total = (long long)n * d;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const int r = (int)(idx / d), j = (int)(idx % d);
        const int src = rows ? rows[r] : r;
        out[idx] = gb_from_float<T>(src >= 0 ? x[(size_t)src * ldx + j] : 0.f);
    }
}

GB_EXPORT int gb_cast_rows(const float* x, long long ldx, const int* rows, void* out, int dtype, int n, int d, cudaStream_t stream) {
    GB_REQUIRE(n >= 0 && d > 0, "gb_cast_rows: bad sizes n=%d d=%d", n, d);
    if (n == 0) return 0;
    long long total = (long long)n * d;
    int blocks = (int)((total + 255) / 256);
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (dtype == GB_F32)
        gb_launch(GB_PDL_ELEMENTWISE, cast_rows_kernel<float>, dim3(blocks), dim3(256), 0, stream, x, ldx, rows, (float*)out, n, d);
    else if (dtype == GB_BF16)
        gb_launch(GB_PDL_ELEMENTWISE, cast_rows_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, x, ldx, rows,
                  (__nv_bfloat16*)out, n, d);
    else
        GB_REQUIRE(false, "gb_cast_rows: unsupported dtype %d", dtype);
    return gb_check_launch("gb_cast_rows");
}

// ----------------------------------------------------------------------------------------------
// y[r, :] += bias (float32): a product's bias where no later kernel takes it along.
// ----------------------------------------------------------------------------------------------
__global__ void add_bias_kernel(float* __restrict__ y, long long ldy, const float* __restrict__ bias, int n, int d) {
    gb_pdl_launch_dependents();
    gb_pdl_wait();
    const long long total = (long long)n * d;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const int r = (int)(idx / d), j = (int)(idx % d);
        y[(size_t)r * ldy + j] += bias[j];
    }
}

GB_EXPORT int gb_add_bias(float* y, long long ldy, const float* bias, int n, int d, cudaStream_t stream) {
    GB_REQUIRE(n >= 0 && d > 0, "gb_add_bias: bad sizes n=%d d=%d", n, d);
    if (n == 0) return 0;
    long long total = (long long)n * d;
    int blocks = (int)((total + 255) / 256);
    if (blocks > 148 * 16) blocks = 148 * 16;
    gb_launch(GB_PDL_ELEMENTWISE, add_bias_kernel, dim3(blocks), dim3(256), 0, stream, y, ldy, bias, n, d);
    return gb_check_launch("gb_add_bias");
}

// ----------------------------------------------------------------------------------------------
// The clamped gated unit, from the sums of the stacked gate | up product (row r: ff gate sums, then ff up sums):
// g = min(gate + b_gate, limit), u = clamp(up + b_up, -limit, limit), act = g * sigmoid(slope * g) * (u + 1), in float32.
// ----------------------------------------------------------------------------------------------
template <typename TI, typename T>
__global__ void clamped_glu_kernel(const TI* __restrict__ gate_up, long long ld, const float* __restrict__ bias, float limit,
                                   float slope, T* __restrict__ act, int n, int ff) {
    gb_pdl_launch_dependents();
    gb_pdl_wait();
    const long long total = (long long)n * ff;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const int r = (int)(idx / ff), f = (int)(idx % ff);
        const TI* row = gate_up + (size_t)r * ld;
        act[idx] = gb_from_float<T>(gb_clamped_unit(gb_to_float(row[f]) + (bias ? bias[f] : 0.f),
                                                   gb_to_float(row[ff + f]) + (bias ? bias[ff + f] : 0.f), limit, slope));
    }
}

GB_EXPORT int gb_clamped_glu(const void* gate_up, int in_dtype, long long ld, const float* bias, float limit, float slope, void* act,
                             int dtype, int n, int ff, cudaStream_t stream) {
    GB_REQUIRE(n >= 0 && ff > 0 && limit > 0.f, "gb_clamped_glu: bad sizes n=%d ff=%d limit=%g", n, ff, (double)limit);
    if (n == 0) return 0;
    long long total = (long long)n * ff;
    int blocks = (int)((total + 255) / 256);
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (in_dtype == GB_F32 && dtype == GB_F32)
        gb_launch(GB_PDL_ELEMENTWISE, clamped_glu_kernel<float, float>, dim3(blocks), dim3(256), 0, stream, (const float*)gate_up, ld,
                  bias, limit, slope, (float*)act, n, ff);
    else if (in_dtype == GB_F32 && dtype == GB_BF16)
        gb_launch(GB_PDL_ELEMENTWISE, clamped_glu_kernel<float, __nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (const float*)gate_up,
                  ld, bias, limit, slope, (__nv_bfloat16*)act, n, ff);
    else if (in_dtype == GB_BF16 && dtype == GB_BF16)
        gb_launch(GB_PDL_ELEMENTWISE, clamped_glu_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(blocks), dim3(256), 0, stream,
                  (const __nv_bfloat16*)gate_up, ld, bias, limit, slope, (__nv_bfloat16*)act, n, ff);
    else
        GB_REQUIRE(false, "gb_clamped_glu: unsupported dtypes %d -> %d", in_dtype, dtype);
    return gb_check_launch("gb_clamped_glu");
}

// ----------------------------------------------------------------------------------------------
// Squared ReLU.
// ----------------------------------------------------------------------------------------------
template <typename T>
__global__ void relu2_kernel(const T* __restrict__ in, T* __restrict__ out, long long total) {
    gb_pdl_launch_dependents();
    gb_pdl_wait();
    long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    for (; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const float v = fmaxf(gb_to_float(in[idx]), 0.f);
        out[idx] = gb_from_float<T>(v * v);
    }
}

GB_EXPORT int gb_relu2(const void* in, void* out, int dtype, long long total, cudaStream_t stream) {
    GB_REQUIRE(total >= 0, "gb_relu2: bad size");
    if (total == 0) return 0;
    int blocks = (int)((total + 255) / 256);
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (dtype == GB_F32)
        gb_launch(GB_PDL_ELEMENTWISE, relu2_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)in, (float*)out, total);
    else if (dtype == GB_BF16)
        gb_launch(GB_PDL_ELEMENTWISE, relu2_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (const __nv_bfloat16*)in,
                  (__nv_bfloat16*)out, total);
    else
        GB_REQUIRE(false, "gb_relu2: unsupported dtype %d", dtype);
    return gb_check_launch("gb_relu2");
}

// ----------------------------------------------------------------------------------------------
// t *= s (float32): a head whose logits carry a constant factor.
// ----------------------------------------------------------------------------------------------
__global__ void scale_kernel(float* __restrict__ t, long long total, float s) {
    gb_pdl_launch_dependents();
    gb_pdl_wait();
    long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    for (; idx < total; idx += (long long)gridDim.x * blockDim.x) t[idx] *= s;
}

GB_EXPORT int gb_scale(float* t, long long total, float s, cudaStream_t stream) {
    GB_REQUIRE(total >= 0, "gb_scale: bad size");
    if (total == 0) return 0;
    int blocks = (int)((total + 255) / 256);
    if (blocks > 148 * 16) blocks = 148 * 16;
    gb_launch(GB_PDL_ELEMENTWISE, scale_kernel, dim3(blocks), dim3(256), 0, stream, t, total, s);
    return gb_check_launch("gb_scale");
}

// ----------------------------------------------------------------------------------------------
// Per-head RMS norm of a mixer's read-out with an output gate: one warp per (row, head).
// o float32 [n, heads * v]; gate float32 (row stride ldg), logits of the gate; w float32 [v] shared by heads.
// ----------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128) gated_head_norm_kernel(const float* __restrict__ o, const float* __restrict__ gate,
                                                              long long ldg, const float* __restrict__ w, T* __restrict__ out,
                                                              int n, int heads, int v, float eps, int gate_silu) {
    gb_pdl_launch_dependents();
    gb_pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long task = (long long)blockIdx.x * 4 + warp;
    if (task >= (long long)n * heads) return;
    const int row = (int)(task / heads), head = (int)(task % heads);
    const float* src = o + ((size_t)row * heads + head) * v;
    const float* g = gate + (size_t)row * ldg + (size_t)head * v;
    T* dst = out + ((size_t)row * heads + head) * v;
    float ss = 0.f;
    for (int j = lane; j < v; j += 32) ss = fmaf(src[j], src[j], ss);
    ss = gb_warp_sum(ss);
    const float s = 1.0f / sqrtf(ss / (float)v + eps);
    for (int j = lane; j < v; j += 32) {
        const float sig = 1.0f / (1.0f + expf(-g[j]));
        dst[j] = gb_from_float<T>(src[j] * s * w[j] * (gate_silu ? g[j] * sig : sig));
    }
}

// The same for long rows (a norm that spans all heads): one block per (row, head), the sum of squares meets in shared memory.
template <typename T>
__global__ void __launch_bounds__(256) gated_head_norm_wide_kernel(const float* __restrict__ o, const float* __restrict__ gate,
                                                                   long long ldg, const float* __restrict__ w, T* __restrict__ out,
                                                                   int n, int heads, int v, float eps, int gate_silu) {
    __shared__ float partial[8];
    gb_pdl_launch_dependents();
    gb_pdl_wait();
    const int row = blockIdx.x / heads, head = blockIdx.x % heads;
    const float* src = o + ((size_t)row * heads + head) * v;
    const float* g = gate + (size_t)row * ldg + (size_t)head * v;
    T* dst = out + ((size_t)row * heads + head) * v;
    float ss = 0.f;
    for (int j = threadIdx.x; j < v; j += 256) ss = fmaf(src[j], src[j], ss);
    ss = gb_warp_sum(ss);
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = ss;
    __syncthreads();
    ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += partial[i];
    const float s = 1.0f / sqrtf(ss / (float)v + eps);
    for (int j = threadIdx.x; j < v; j += 256) {
        const float sig = 1.0f / (1.0f + expf(-g[j]));
        dst[j] = gb_from_float<T>(src[j] * s * w[j] * (gate_silu ? g[j] * sig : sig));
    }
}

GB_EXPORT int gb_gated_head_norm(const float* o, const float* gate, long long ldg, const float* w, void* out, int out_dtype,
                                 int n, int heads, int v, float eps, int gate_silu, cudaStream_t stream) {
    GB_REQUIRE(n >= 0 && heads > 0 && v > 0, "gb_gated_head_norm: bad sizes");
    if (n == 0) return 0;
    if (v > 256) {
        if (out_dtype == GB_F32)
            gb_launch(GB_PDL_ELEMENTWISE, gated_head_norm_wide_kernel<float>, dim3(n * heads), dim3(256), 0, stream, o, gate, ldg, w,
                      (float*)out, n, heads, v, eps, gate_silu);
        else if (out_dtype == GB_BF16)
            gb_launch(GB_PDL_ELEMENTWISE, gated_head_norm_wide_kernel<__nv_bfloat16>, dim3(n * heads), dim3(256), 0, stream, o, gate, ldg, w,
                      (__nv_bfloat16*)out, n, heads, v, eps, gate_silu);
        else
            GB_REQUIRE(false, "gb_gated_head_norm: unsupported output dtype %d", out_dtype);
        return gb_check_launch("gb_gated_head_norm");
    }
    const int blocks = gb_ceil_div((long long)n * heads, 4);
    if (out_dtype == GB_F32)
        gb_launch(GB_PDL_ELEMENTWISE, gated_head_norm_kernel<float>, dim3(blocks), dim3(128), 0, stream, o, gate, ldg, w, (float*)out, n,
                  heads, v, eps, gate_silu);
    else if (out_dtype == GB_BF16)
        gb_launch(GB_PDL_ELEMENTWISE, gated_head_norm_kernel<__nv_bfloat16>, dim3(blocks), dim3(128), 0, stream, o, gate, ldg, w,
                  (__nv_bfloat16*)out, n, heads, v, eps, gate_silu);
    else
        GB_REQUIRE(false, "gb_gated_head_norm: unsupported output dtype %d", out_dtype);
    return gb_check_launch("gb_gated_head_norm");
}

// ----------------------------------------------------------------------------------------------
// The gated unit whose gate passes the tanh form of GELU: act[r, f] = 0.5 g (1 + tanh(sqrt(2/pi) (g + 0.044715 g^3))) * u with
// g = gate_up[r, f], u = gate_up[r, ff + f]; float32 arithmetic, any input and output dtype.
// ----------------------------------------------------------------------------------------------
template <typename TI, typename TO>
__global__ void __launch_bounds__(256) gelu_glu_kernel(const TI* __restrict__ gate_up, long long ld, TO* __restrict__ act, int n, int ff) {
    gb_pdl_launch_dependents();
    gb_pdl_wait();
    const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    if (i >= (long long)n * ff) return;
    const int r = (int)(i / ff), f = (int)(i % ff);
    const float g = gb_to_float(gate_up[(size_t)r * ld + f]), u = gb_to_float(gate_up[(size_t)r * ld + ff + f]);
    act[i] = gb_from_float<TO>(gb_gelu_tanh(g) * u);
}

GB_EXPORT int gb_gelu_glu(const void* gate_up, int in_dtype, long long ld, void* act, int out_dtype, int n, int ff, cudaStream_t stream) {
    GB_REQUIRE(n >= 0 && ff > 0 && ld >= 2 * ff, "gb_gelu_glu: bad sizes");
    if (n == 0) return 0;
    const int blocks = gb_ceil_div((long long)n * ff, 256);
    if (in_dtype == GB_F32 && out_dtype == GB_F32)
        gb_launch(GB_PDL_ELEMENTWISE, gelu_glu_kernel<float, float>, dim3(blocks), dim3(256), 0, stream, (const float*)gate_up, ld, (float*)act, n, ff);
    else if (in_dtype == GB_F32 && out_dtype == GB_BF16)
        gb_launch(GB_PDL_ELEMENTWISE, gelu_glu_kernel<float, __nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (const float*)gate_up, ld,
                  (__nv_bfloat16*)act, n, ff);
    else if (in_dtype == GB_BF16 && out_dtype == GB_BF16)
        gb_launch(GB_PDL_ELEMENTWISE, gelu_glu_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(blocks), dim3(256), 0, stream,
                  (const __nv_bfloat16*)gate_up, ld, (__nv_bfloat16*)act, n, ff);
    else
        GB_REQUIRE(false, "gb_gelu_glu: unsupported dtypes %d -> %d", in_dtype, out_dtype);
    return gb_check_launch("gb_gelu_glu");
}

// ----------------------------------------------------------------------------------------------
// out[r, :] (+)= a * x[r, :] + b * y[r, :]: two branches that share an input join with a weight each. Float32.
// ----------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) scaled_sum_kernel(const float* __restrict__ x, const float* __restrict__ y, float a, float b,
                                                         float* __restrict__ out, long long count, int accumulate) {
    gb_pdl_launch_dependents();
    gb_pdl_wait();
    const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    if (i >= count) return;
    const float v = fmaf(a, x[i], b * y[i]);
    out[i] = accumulate ? out[i] + v : v;
}

GB_EXPORT int gb_scaled_sum(const float* x, const float* y, float a, float b, float* out, long long count, int accumulate,
                            cudaStream_t stream) {
    GB_REQUIRE(count >= 0, "gb_scaled_sum: bad size");
    if (count == 0) return 0;
    gb_launch(GB_PDL_ELEMENTWISE, scaled_sum_kernel, dim3(gb_ceil_div(count, 256)), dim3(256), 0, stream, x, y, a, b, out, count, accumulate);
    return gb_check_launch("gb_scaled_sum");
}
