// Paged causal attention for any head size, page size and window, in float32 arithmetic.
// It serves the 32-bit path and every bfloat16 shape the tensor-core kernels refuse.
// One block per (token, query head); keys lo..pos of the token's own request are read from the
// pages named by its block table (the step's own keys were appended before this runs, as in
// tinyinfer/layers/attention.py:455-465). Scores (q.k)*scale, running max from -inf, sum and
// output in float32 (tinyinfer/csrc/flash_decoding.cu:124-147,334); GQA head map
// kv = q_head / (Hq / Hkv) (flash_decoding.cu:54-55).
#include "common.cuh"

constexpr int AG_THREADS = 128;
constexpr int AG_MAX_D = 256;

template <typename T>
__global__ void __launch_bounds__(AG_THREADS) attention_generic_kernel(
    T* __restrict__ out, const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
    const int* __restrict__ positions, const int* __restrict__ token_seq,
    const int* __restrict__ block_table, int max_blocks, int hq, int hkv, int d, int page_size,
    int num_pages, float scale, int window, int* __restrict__ status) {
    __shared__ float qs[AG_MAX_D];
    __shared__ float p[AG_THREADS];
    __shared__ long long row_off[AG_THREADS];
    __shared__ float red[33];
    ti_grid_launch_dependents();
    ti_grid_wait();
    const int tid = threadIdx.x;
    const int h = blockIdx.x, t = blockIdx.y;
    const int pos = positions[t];
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int kvh = h / (hq / hkv);
    const int* table = block_table + (size_t)token_seq[t] * max_blocks;
    const T* qrow = q + ((size_t)t * hq + h) * d;
    for (int i = tid; i < d; i += AG_THREADS) qs[i] = to_f32(qrow[i]);
    __syncthreads();

    float acc0 = 0.f, acc1 = 0.f, m = -INFINITY, l = 0.f;
    for (int tile0 = lo; tile0 <= pos; tile0 += AG_THREADS) {
        const int j = tile0 + tid;
        float s = -INFINITY;
        long long off = -1;
        if (j <= pos) {
            const int logical = j / page_size;
            const int page = logical < max_blocks ? table[logical] : -1;
            if (page >= 0 && page < num_pages) {
                off = (((long long)page * hkv + kvh) * page_size + j % page_size) * d;
                const T* krow = k_cache + off;
                float dot = 0.f;
                for (int i = 0; i < d; ++i) dot = fmaf(qs[i], to_f32(krow[i]), dot);
                s = dot * scale;
            } else if (status) {
                atomicExch(status, 2);                 // a visible key without a page
            }
        }
        const float tile_max = block_max(s, red);
        const float m_new = fmaxf(m, tile_max);
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        const float pj = (s == -INFINITY) ? 0.f : expf(s - m_new);
        p[tid] = pj;
        row_off[tid] = off;
        const float tile_sum = block_sum(pj, red);      // also orders the writes of p and row_off
        l = l * corr + tile_sum;
        acc0 *= corr;
        acc1 *= corr;
        m = m_new;
        const int n = min(AG_THREADS, pos + 1 - tile0);
        if (tid < d) {
            for (int jj = 0; jj < n; ++jj) {
                const long long o = row_off[jj];
                if (o < 0) continue;
                const float pv = p[jj];
                acc0 = fmaf(pv, to_f32(v_cache[o + tid]), acc0);
                if (tid + AG_THREADS < d) acc1 = fmaf(pv, to_f32(v_cache[o + tid + AG_THREADS]), acc1);
            }
        }
        __syncthreads();
    }
    T* orow = out + ((size_t)t * hq + h) * d;
    const float inv = l > 0.f ? 1.f / l : 0.f;
    if (tid < d) orow[tid] = from_f32<T>(acc0 * inv);
    if (tid + AG_THREADS < d) orow[tid + AG_THREADS] = from_f32<T>(acc1 * inv);
}

TI_API int ti_attention_generic(
    void* out, const void* q, const void* kv_cache, const int* positions, const int* token_seq,
    const int* block_table, int max_blocks, int num_tokens, int hq, int hkv, int d, int page_size,
    int num_pages, float scale, int window, int* status, int dtype, cudaStream_t stream) {
    TI_REQUIRE(d > 0 && d <= AG_MAX_D, "attention: head_dim %d not in 1..%d", d, AG_MAX_D);
    TI_REQUIRE(hq > 0 && hkv > 0 && hq % hkv == 0, "attention: %d query heads do not group over %d kv heads", hq, hkv);
    TI_REQUIRE(page_size > 0 && num_tokens >= 0 && window >= 0, "attention: bad sizes");
    TI_REQUIRE(num_tokens <= 65535, "attention: more than 65535 tokens in one step");
    if (num_tokens == 0) return 0;
    const size_t v_off = (size_t)num_pages * hkv * page_size * d;
    dim3 grid(hq, num_tokens);
    if (dtype == TI_F32) {
        const float* kc = (const float*)kv_cache;
        ti_launch(attention_generic_kernel<float>, grid, AG_THREADS, 0, stream,
            (float*)out, (const float*)q, kc, kc + v_off, positions, token_seq, block_table, max_blocks, hq, hkv,
            d, page_size, num_pages, scale, window, status);
    } else if (dtype == TI_BF16) {
        const __nv_bfloat16* kc = (const __nv_bfloat16*)kv_cache;
        ti_launch(attention_generic_kernel<__nv_bfloat16>, grid, AG_THREADS, 0, stream,
            (__nv_bfloat16*)out, (const __nv_bfloat16*)q, kc, kc + v_off, positions, token_seq, block_table,
            max_blocks, hq, hkv, d, page_size, num_pages, scale, window, status);
    } else TI_REQUIRE(false, "attention: unknown dtype %d", dtype);
    TI_CHECK_LAUNCH("attention_generic");
    return 0;
}
