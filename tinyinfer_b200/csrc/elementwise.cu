// Embedding gather, RMSNorm (optionally of selected rows) and the residual sum.
// RMSNorm follows tinyinfer/csrc/rmsnorm.cu:22-50 of the reference: sum of squares, rsqrt and
// the product w * x * inv all in float32, one rounding at the store.
#include "common.cuh"

// ------------------------------------------------------------------ embedding
template <typename T>
__global__ void embedding_kernel(T* __restrict__ out, const T* __restrict__ table,
                                 const int* __restrict__ ids, int hidden, int vocab) {
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
        embedding_kernel<float><<<num_tokens, threads, 0, stream>>>((float*)out, (const float*)table, ids, hidden, vocab);
    else if (dtype == TI_BF16)
        embedding_kernel<__nv_bfloat16><<<num_tokens, threads, 0, stream>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)table, ids, hidden, vocab);
    else TI_REQUIRE(false, "embedding: unknown dtype %d", dtype);
    TI_CHECK_LAUNCH("embedding");
    return 0;
}

// ------------------------------------------------------------------ rmsnorm
// One block per output row. rows == nullptr: output row r is input row r; else input row rows[r].
template <typename T>
__global__ void rmsnorm_kernel(T* __restrict__ out, const T* __restrict__ x,
                               const float* __restrict__ w, const int* __restrict__ rows,
                               int size, float eps) {
    __shared__ float red[33];
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

TI_API int ti_rmsnorm(void* out, const void* x, const float* weight, const int* rows, int num_rows,
                      int size, float eps, int dtype, cudaStream_t stream) {
    TI_REQUIRE(num_rows >= 0 && size > 0, "rmsnorm: bad sizes");
    if (num_rows == 0) return 0;
    int threads = 32;
    while (threads < 512 && threads * 4 < size) threads <<= 1;
    if (dtype == TI_F32)
        rmsnorm_kernel<float><<<num_rows, threads, 0, stream>>>((float*)out, (const float*)x, weight, rows, size, eps);
    else if (dtype == TI_BF16)
        rmsnorm_kernel<__nv_bfloat16><<<num_rows, threads, 0, stream>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)x, weight, rows, size, eps);
    else TI_REQUIRE(false, "rmsnorm: unknown dtype %d", dtype);
    TI_CHECK_LAUNCH("rmsnorm");
    return 0;
}

// ------------------------------------------------------------------ residual sum
template <typename T>
__global__ void add_kernel(T* __restrict__ out, const T* __restrict__ a, const T* __restrict__ b, size_t n) {
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
        add_kernel<float><<<blocks, threads, 0, stream>>>((float*)out, (const float*)a, (const float*)b, (size_t)n);
    else if (dtype == TI_BF16)
        add_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)a, (const __nv_bfloat16*)b, (size_t)n);
    else TI_REQUIRE(false, "add: unknown dtype %d", dtype);
    TI_CHECK_LAUNCH("add");
    return 0;
}
