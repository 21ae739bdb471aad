// Embedding gather, RMSNorm (optionally of selected rows) and the residual sum.
// RMSNorm follows tinyinfer/csrc/rmsnorm.cu:22-50 of the reference: sum of squares, rsqrt and
// the product w * x * inv all in float32, one rounding at the store.
#include "common.cuh"

// ------------------------------------------------------------------ embedding
template <typename T>
__global__ void embedding_kernel(T* __restrict__ out, const T* __restrict__ table,
                                 const int* __restrict__ ids, int hidden, int vocab) {
    ti_grid_launch_dependents();
    ti_grid_wait();
    const int t = blockIdx.x;
    const int id = ids[t];
    const bool ok = id >= 0 && id < vocab;
    const T* src = table + (size_t)(ok ? id : 0) * hidden;
    T* dst = out + (size_t)t * hidden;
    constexpr int VEC = 16 / sizeof(T);
    if (hidden % VEC == 0) {
        const uint4* s4 = reinterpret_cast<const uint4*>(src);
        uint4* d4 = reinterpret_cast<uint4*>(dst);
        for (int i = threadIdx.x; i < hidden / VEC; i += blockDim.x)
            d4[i] = ok ? s4[i] : make_uint4(0, 0, 0, 0);
    } else {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = ok ? src[i] : from_f32<T>(0.f);
    }
}

TI_API int ti_embedding(void* out, const void* table, const int* ids, int num_tokens, int hidden,
                        int vocab, int dtype, cudaStream_t stream) {
    TI_REQUIRE(num_tokens >= 0 && hidden > 0 && vocab > 0, "embedding: bad sizes");
    if (num_tokens == 0) return 0;
    const int threads = hidden >= 2048 ? 256 : 128;
    if (dtype == TI_F32)
        ti_launch(embedding_kernel<float>, num_tokens, threads, 0, stream, (float*)out, (const float*)table, ids, hidden, vocab);
    else if (dtype == TI_BF16)
        ti_launch(embedding_kernel<__nv_bfloat16>, num_tokens, threads, 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)table, ids, hidden, vocab);
    else TI_REQUIRE(false, "embedding: unknown dtype %d", dtype);
    TI_CHECK_LAUNCH("embedding");
    return 0;
}

// ------------------------------------------------------------------ token ids that never visit the host
// ids[dst_rows[i]] = src[src_rows[i]] for every i with dst_rows[i] >= 0: the tokens a step sampled become the
// next step's inputs on the device, so the next step can be launched before the host has seen them.
__global__ void feed_tokens_kernel(int* __restrict__ ids, const int* __restrict__ dst_rows,
                                   const int* __restrict__ src_rows, const int* __restrict__ src, int n) {
    ti_grid_launch_dependents();
    ti_grid_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        const int d = dst_rows[i];
        if (d >= 0) ids[d] = src[src_rows[i]];
    }
}

TI_API int ti_feed_tokens(int* ids, const int* dst_rows, const int* src_rows, const int* src, int n, cudaStream_t stream) {
    TI_REQUIRE(n >= 0, "feed_tokens: bad size");
    if (n == 0) return 0;
    ti_launch(feed_tokens_kernel, (n + 127) / 128, 128, 0, stream, ids, dst_rows, src_rows, src, n);
    TI_CHECK_LAUNCH("feed_tokens");
    return 0;
}

// ------------------------------------------------------------------ rmsnorm
// One block per output row. rows == nullptr: output row r is input row r; else input row rows[r].
// General form: two passes over the row.
template <typename T>
__global__ void rmsnorm_kernel(T* __restrict__ out, const T* __restrict__ x,
                               const float* __restrict__ w, const int* __restrict__ rows,
                               int size, float eps) {
    __shared__ float red[33];
    ti_grid_launch_dependents();
    ti_grid_wait();
    const int r = blockIdx.x;
    const T* src = x + (size_t)(rows ? rows[r] : r) * size;
    T* dst = out + (size_t)r * size;
    float ss = 0.f;
    for (int i = threadIdx.x; i < size; i += blockDim.x) {
        const float v = to_f32(src[i]);
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)size + eps);
    for (int i = threadIdx.x; i < size; i += blockDim.x)
        dst[i] = from_f32<T>(w[i] * to_f32(src[i]) * inv);
}

// Rows of up to 8192 elements whose length is a multiple of the 16-byte vector: the row is read
// once with 16-byte loads and kept in registers between the sum and the scaling.
template <typename T, int PER_THREAD>
__global__ void __launch_bounds__(1024) rmsnorm_vec_kernel(T* __restrict__ out, const T* __restrict__ x,
                                                            const float* __restrict__ w, const int* __restrict__ rows,
                                                            int size, float eps) {
    constexpr int VEC = 16 / sizeof(T);
    __shared__ float red[33];
    ti_grid_launch_dependents();
    const int nvec = size / VEC;
    float wv[PER_THREAD][VEC];
#pragma unroll
    for (int k = 0; k < PER_THREAD; ++k) {           // the weight does not depend on earlier kernels
        const int v = threadIdx.x + k * blockDim.x;
        if (v < nvec) {
#pragma unroll
            for (int i = 0; i < VEC; i += 4) {
                const float4 f = *reinterpret_cast<const float4*>(w + (size_t)v * VEC + i);
                wv[k][i] = f.x; wv[k][i + 1] = f.y; wv[k][i + 2] = f.z; wv[k][i + 3] = f.w;
            }
        }
    }
    ti_grid_wait();
    const int r = blockIdx.x;
    const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(rows ? rows[r] : r) * size);
    uint4* dst = reinterpret_cast<uint4*>(out + (size_t)r * size);
    float xv[PER_THREAD][VEC];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < PER_THREAD; ++k) {
        const int v = threadIdx.x + k * blockDim.x;
        if (v < nvec) {
            const uint4 q = src[v];
            const T* e = reinterpret_cast<const T*>(&q);
#pragma unroll
            for (int i = 0; i < VEC; ++i) {
                xv[k][i] = to_f32(e[i]);
                ss += xv[k][i] * xv[k][i];
            }
        }
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)size + eps);
#pragma unroll
    for (int k = 0; k < PER_THREAD; ++k) {
        const int v = threadIdx.x + k * blockDim.x;
        if (v < nvec) {
            uint4 q;
            T* e = reinterpret_cast<T*>(&q);
#pragma unroll
            for (int i = 0; i < VEC; ++i) e[i] = from_f32<T>(wv[k][i] * xv[k][i] * inv);
            dst[v] = q;
        }
    }
}

template <typename T>
static int launch_rmsnorm(void* out, const void* x, const float* weight, const int* rows, int num_rows, int size,
                          float eps, cudaStream_t stream) {
    constexpr int VEC = 16 / sizeof(T);
    const bool aligned = size % VEC == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)out & 15) == 0 && ((uintptr_t)weight & 15) == 0;
    if (aligned && size / VEC <= 2048) {
        const int nvec = size / VEC;
        const int per = nvec <= 1024 ? 1 : 2;
        int threads = ((nvec + per - 1) / per + 31) / 32 * 32;
        if (per == 1)
            ti_launch(rmsnorm_vec_kernel<T, 1>, num_rows, threads, 0, stream, (T*)out, (const T*)x, weight, rows, size, eps);
        else
            ti_launch(rmsnorm_vec_kernel<T, 2>, num_rows, threads, 0, stream, (T*)out, (const T*)x, weight, rows, size, eps);
    } else {
        int threads = 32;
        while (threads < 512 && threads * 4 < size) threads <<= 1;
        ti_launch(rmsnorm_kernel<T>, num_rows, threads, 0, stream, (T*)out, (const T*)x, weight, rows, size, eps);
    }
    return 0;
}

TI_API int ti_rmsnorm(void* out, const void* x, const float* weight, const int* rows, int num_rows,
                      int size, float eps, int dtype, cudaStream_t stream) {
    TI_REQUIRE(num_rows >= 0 && size > 0, "rmsnorm: bad sizes");
    if (num_rows == 0) return 0;
    if (dtype == TI_F32) launch_rmsnorm<float>(out, x, weight, rows, num_rows, size, eps, stream);
    else if (dtype == TI_BF16) launch_rmsnorm<__nv_bfloat16>(out, x, weight, rows, num_rows, size, eps, stream);
    else TI_REQUIRE(false, "rmsnorm: unknown dtype %d", dtype);
    TI_CHECK_LAUNCH("rmsnorm");
    return 0;
}

// ------------------------------------------------------------------ residual sum
template <typename T>
__global__ void add_kernel(T* __restrict__ out, const T* __restrict__ a, const T* __restrict__ b, size_t n) {
    ti_grid_launch_dependents();
    ti_grid_wait();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        out[i] = from_f32<T>(to_f32(a[i]) + to_f32(b[i]));
}

TI_API int ti_add(void* out, const void* a, const void* b, long long n, int dtype, cudaStream_t stream) {
    TI_REQUIRE(n >= 0, "add: bad size");
    if (n == 0) return 0;
    const int threads = 256;
    const int blocks = (int)((n + threads - 1) / threads < 148 * 16 ? (n + threads - 1) / threads : 148 * 16);
    if (dtype == TI_F32)
        ti_launch(add_kernel<float>, blocks, threads, 0, stream, (float*)out, (const float*)a, (const float*)b, (size_t)n);
    else if (dtype == TI_BF16)
        ti_launch(add_kernel<__nv_bfloat16>, blocks, threads, 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)a, (const __nv_bfloat16*)b, (size_t)n);
    else TI_REQUIRE(false, "add: unknown dtype %d", dtype);
    TI_CHECK_LAUNCH("add");
    return 0;
}
