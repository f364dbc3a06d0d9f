// Pieces shared by the attention kernels that walk a paged cache row by row (one lane per key, float32 arithmetic): dot
// products of a query in shared memory with a cached key row, 16-byte pieces of a value row as floats, and the 16-byte
// asynchronous copy that stages tiles.
#pragma once
#include "common.cuh"

constexpr int SA_MAX_DIM = 256;      // largest key or value size of these kernels

// q . k over D channels; q in shared memory as float32, k a row of the cache.
template <typename T>
__device__ __forceinline__ float sa_dot(const float* __restrict__ q, const T* __restrict__ k, int D);

template <>
__device__ __forceinline__ float sa_dot<float>(const float* __restrict__ q, const float* __restrict__ k, int D) {
    float d = 0.f;
    if (D % 4 == 0 && ((uintptr_t)k & 15) == 0) {
#pragma unroll 8
        for (int i = 0; i < D; i += 4) {
            const float4 kv = *reinterpret_cast<const float4*>(k + i);
            d = fmaf(q[i], kv.x, d); d = fmaf(q[i + 1], kv.y, d); d = fmaf(q[i + 2], kv.z, d); d = fmaf(q[i + 3], kv.w, d);
        }
    } else {
        for (int i = 0; i < D; ++i) d = fmaf(q[i], k[i], d);
    }
    return d;
}

template <>
__device__ __forceinline__ float sa_dot<__nv_bfloat16>(const float* __restrict__ q, const __nv_bfloat16* __restrict__ k, int D) {
    float d = 0.f;
    if (D % 8 == 0 && ((uintptr_t)k & 15) == 0) {
#pragma unroll 8
        for (int i = 0; i < D; i += 8) {
            const uint4 raw = *reinterpret_cast<const uint4*>(k + i);
            const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                const float2 f = __bfloat1622float2(p[t]);
                d = fmaf(q[i + 2 * t], f.x, d);
                d = fmaf(q[i + 2 * t + 1], f.y, d);
            }
        }
    } else {
        for (int i = 0; i < D; ++i) d = fmaf(q[i], __bfloat162float(k[i]), d);
    }
    return d;
}

template <typename T> struct SadPiece;                 // 16 bytes of a value row as floats
template <> struct SadPiece<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void unpack(const uint4& raw, float (&f)[4]) {
        f[0] = __uint_as_float(raw.x); f[1] = __uint_as_float(raw.y); f[2] = __uint_as_float(raw.z); f[3] = __uint_as_float(raw.w);
    }
};
template <> struct SadPiece<__nv_bfloat16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void unpack(const uint4& raw, float (&f)[8]) {
        const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            const float2 v = __bfloat1622float2(p[t]);
            f[2 * t] = v.x;
            f[2 * t + 1] = v.y;
        }
    }
};

// NP 16-byte pieces of a key row against the same channels of R queries (q rows D apart): all loads first, then the sums
template <typename T, int R, int NP>
__device__ __forceinline__ void sad_dot_pieces(const float* __restrict__ q, int D, const T* __restrict__ k, float (&out)[R]) {
    constexpr int PN = SadPiece<T>::N;
    uint4 raw[NP];
#pragma unroll
    for (int c = 0; c < NP; ++c) raw[c] = *reinterpret_cast<const uint4*>(k + c * PN);
#pragma unroll
    for (int c = 0; c < NP; ++c) {
        float f[PN];
        SadPiece<T>::unpack(raw[c], f);
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int e = 0; e < PN; ++e) out[r] = fmaf(q[r * D + c * PN + e], f[e], out[r]);
    }
}

// q . k for R query heads at once (q: R rows of D floats in shared memory), the key row read once
template <typename T, int R>
__device__ __forceinline__ void sad_dots(const float* __restrict__ q, const T* __restrict__ k, int D, float (&out)[R]) {
#pragma unroll
    for (int r = 0; r < R; ++r) out[r] = 0.f;
    constexpr int PN = SadPiece<T>::N;
    if (D % PN == 0 && ((uintptr_t)k & 15) == 0) {
        // a key row's loads are the critical path of a chunk: eight 16-byte pieces in flight together, then four, then single
        int i = 0;
        for (; i + 8 * PN <= D; i += 8 * PN) sad_dot_pieces<T, R, 8>(q + i, D, k + i, out);
        for (; i + 4 * PN <= D; i += 4 * PN) sad_dot_pieces<T, R, 4>(q + i, D, k + i, out);
        for (; i < D; i += PN) sad_dot_pieces<T, R, 1>(q + i, D, k + i, out);
    } else {
        for (int i = 0; i < D; ++i) {
            const float kv = gb_to_float(k[i]);
#pragma unroll
            for (int r = 0; r < R; ++r) out[r] = fmaf(q[r * D + i], kv, out[r]);
        }
    }
}

__device__ __forceinline__ void sat_cp16(void* smem, const void* gmem, bool valid) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(bytes));
}

