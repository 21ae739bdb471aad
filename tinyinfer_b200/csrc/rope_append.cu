// Fused per-head RMSNorm of q and k, half-split rotary embedding, and the write of k and v into
// the pages of the cache. One warp handles one head of one token.
// Formulas of the reference: norm before rotation, v untouched (tinyinfer/models/qwen3.py:116-122);
// angle = float(position) * inv_freq[j], out[j] = x[j] cos - x[j+half] sin,
// out[j+half] = x[j+half] cos + x[j] sin (tinyinfer/csrc/rope.cu:31-74); the rotated k is what is
// cached (tinyinfer/layers/attention.py:455-465). All arithmetic in float32, one rounding at the store.
//
// Where the angles come from and which features are paired is data, so that another position encoding
// needs no other kernel: the angle of pair j at position p is p * inv_freq[j], or, if a table is given,
// cos = table[p][j] and sin = table[p][rotary_dim / 2 + j] (float32 [table_positions, rotary_dim]: any
// encoding whose angles depend on the position alone, scaled or learned). The pair is (j, j + rotary_dim/2)
// (half-split, the reference's) or, with `interleaved`, (2j, 2j + 1). A position beyond the table, like a
// token without a page, sets the status word and writes nothing.
#include "common.cuh"

constexpr int RA_WARPS = 4;
constexpr int RA_MAX_D = 256;

template <typename T>
__global__ void qk_norm_rope_append_kernel(
    T* __restrict__ q_out, const T* __restrict__ qkv, T* __restrict__ k_cache, T* __restrict__ v_cache,
    const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
    const float* __restrict__ inv_freq, const float* __restrict__ table, int table_positions, int interleaved,
    int rotary_dim,
    const int* __restrict__ positions, const int* __restrict__ token_seq,
    const int* __restrict__ block_table, int max_blocks,
    int hq, int hkv, int d, int page_size, int num_pages, int* __restrict__ status) {
    __shared__ float buf[RA_WARPS][RA_MAX_D];
    ti_grid_launch_dependents();
    ti_grid_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = blockIdx.x * RA_WARPS + warp;
    const int t = blockIdx.y;
    const int heads_total = hq + 2 * hkv;
    if (head >= heads_total) return;
    const bool is_q = head < hq;
    const bool is_k = !is_q && head < hq + hkv;
    if (!is_q && k_cache == nullptr) return;           // an entry that only reads the cache
    const T* src = qkv + ((size_t)t * heads_total + head) * d;
    float* x = buf[warp];

    float ss = 0.f;
    for (int i = lane; i < d; i += 32) {
        const float v = to_f32(src[i]);
        x[i] = v;
        ss += v * v;
    }
    const float* w = is_q ? q_w : (is_k ? k_w : nullptr);
    if (w != nullptr) {
        ss = warp_sum(ss);
        const float inv = rsqrtf(ss / (float)d + eps);
        for (int i = lane; i < d; i += 32) x[i] = w[i] * x[i] * inv;
    }
    __syncwarp();

    T* dst;
    if (is_q) {
        dst = q_out + ((size_t)t * hq + head) * d;
    } else {
        const int pos = positions[t];
        const int logical = pos / page_size;
        const int page = logical < max_blocks ? block_table[(size_t)token_seq[t] * max_blocks + logical] : -1;
        if (page < 0 || page >= num_pages) {
            if (lane == 0 && status) atomicExch(status, 1);   // a token without a page: never write
            return;
        }
        const int kvh = is_k ? head - hq : head - hq - hkv;
        T* base = is_k ? k_cache : v_cache;
        dst = base + (((size_t)page * hkv + kvh) * page_size + pos % page_size) * d;
    }

    if ((is_q || is_k) && (inv_freq != nullptr || table != nullptr)) {
        const int half = rotary_dim >> 1;
        const int pos = positions[t];
        if (table != nullptr && (pos < 0 || pos >= table_positions)) {
            if (lane == 0 && status) atomicExch(status, 4);   // a position the table does not reach
            return;
        }
        const float pos_f = (float)pos;
        for (int i = lane; i < d; i += 32) {
            float o;
            if (i < rotary_dim) {
                const int j = interleaved ? (i >> 1) : (i < half ? i : i - half);
                const bool first = interleaved ? !(i & 1) : i < half;
                const int other = interleaved ? (i ^ 1) : (i < half ? i + half : i - half);
                float s, c;
                if (table != nullptr) {
                    c = table[(size_t)pos * rotary_dim + j];
                    s = table[(size_t)pos * rotary_dim + half + j];
                } else {
                    sincosf(pos_f * inv_freq[j], &s, &c);
                }
                o = first ? x[i] * c - x[other] * s : x[i] * c + x[other] * s;
            } else {
                o = x[i];
            }
            dst[i] = from_f32<T>(o);
        }
    } else {
        for (int i = lane; i < d; i += 32) dst[i] = from_f32<T>(x[i]);
    }
}

// Head sizes 64 and 128 with the rotation over the whole head (or none): a lane owns D / 32
// neighbouring features, loads and stores them as one vector, and gets its rotation partner from the
// lane 16 further on (half-split: the feature D / 2 away) or from its own vector (interleaved pairs).
template <typename T, int D, int HPW>
__global__ void __launch_bounds__(RA_WARPS * 32) qk_norm_rope_append_vec_kernel(
    T* __restrict__ q_out, const T* __restrict__ qkv, T* __restrict__ k_cache, T* __restrict__ v_cache,
    const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
    const float* __restrict__ inv_freq, const float* __restrict__ table, int table_positions, int interleaved,
    const int* __restrict__ positions, const int* __restrict__ token_seq,
    const int* __restrict__ block_table, int max_blocks,
    int hq, int hkv, int page_size, int num_pages, int* __restrict__ status) {
    constexpr int VEC = D / 32;
    struct alignas(sizeof(T) * VEC) Pack { T e[VEC]; };
    __shared__ float cos_sh[D / 2], sin_sh[D / 2];
    ti_grid_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head0 = (blockIdx.x * RA_WARPS + warp) * HPW;        // a warp takes HPW heads of the token
    const int t = blockIdx.y;
    const int heads_total = hq + 2 * hkv;
    // The angles of a token are the same for all its heads: the block works them out once (sincosf is
    // most of this kernel's arithmetic), from the step's positions, which were on the device before the
    // step's first kernel began, so this happens before the wait for the kernel ahead.
    const int pos = positions[t];
    const bool rotate = inv_freq != nullptr || table != nullptr;
    if (table != nullptr && (pos < 0 || pos >= table_positions)) {
        if (threadIdx.x == 0 && status) atomicExch(status, 4);      // a position the table does not reach
        return;
    }
    if (rotate && threadIdx.x < D / 2 && blockIdx.x * RA_WARPS * HPW < hq + hkv) {
        if (table != nullptr) {
            cos_sh[threadIdx.x] = table[(size_t)pos * D + threadIdx.x];
            sin_sh[threadIdx.x] = table[(size_t)pos * D + D / 2 + threadIdx.x];
        } else {
            sincosf((float)pos * inv_freq[threadIdx.x], &sin_sh[threadIdx.x], &cos_sh[threadIdx.x]);
        }
    }
    __syncthreads();
    if (head0 >= heads_total) return;
    // The page of the token's keys and values, for a warp that has a key or value head: block tables and
    // token_seq are inputs of the step like the positions, so the two dependent loads happen before the wait.
    int page = -2;
    if (k_cache != nullptr && head0 + HPW > hq) {
        const int logical = pos / page_size;
        page = logical < max_blocks ? block_table[(size_t)token_seq[t] * max_blocks + logical] : -1;
    }
    ti_grid_wait();
    // all of the warp's loads first: with many tokens the kernel lives on the bytes it has in flight
    Pack in[HPW];
    bool live[HPW];
#pragma unroll
    for (int hh = 0; hh < HPW; ++hh) {
        const int head = head0 + hh;
        live[hh] = head < heads_total && (head < hq || k_cache != nullptr);
        if (live[hh]) in[hh] = *reinterpret_cast<const Pack*>(qkv + ((size_t)t * heads_total + head) * D + lane * VEC);
    }
#pragma unroll
    for (int hh = 0; hh < HPW; ++hh) {
        if (!live[hh]) continue;
        const int head = head0 + hh;
        const bool is_q = head < hq;
        const bool is_k = !is_q && head < hq + hkv;
        const float* w = is_q ? q_w : (is_k ? k_w : nullptr);
        float x[VEC];
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
            x[i] = to_f32(in[hh].e[i]);
            ss += x[i] * x[i];
        }
        if (w != nullptr) {
            ss = warp_sum(ss);
            const float inv = rsqrtf(ss / (float)D + eps);
#pragma unroll
            for (int i = 0; i < VEC; ++i) x[i] = w[lane * VEC + i] * x[i] * inv;
        }
        if ((is_q || is_k) && rotate && !interleaved) {
#pragma unroll
            for (int i = 0; i < VEC; ++i) {
                const float other = __shfl_xor_sync(0xffffffffu, x[i], 16);
                const float sn = sin_sh[(lane & 15) * VEC + i], cs = cos_sh[(lane & 15) * VEC + i];
                x[i] = lane < 16 ? x[i] * cs - other * sn : x[i] * cs + other * sn;
            }
        } else if ((is_q || is_k) && rotate) {
#pragma unroll
            for (int i = 0; i < VEC; i += 2) {
                const int j = (lane * VEC + i) >> 1;
                const float sn = sin_sh[j], cs = cos_sh[j];
                const float a = x[i], b = x[i + 1];
                x[i] = a * cs - b * sn;
                x[i + 1] = b * cs + a * sn;
            }
        }
        T* dst;
        if (is_q) {
            dst = q_out + ((size_t)t * hq + head) * D;
        } else {
            if (page < 0 || page >= num_pages) {
                if (lane == 0 && status) atomicExch(status, 1);
                return;
            }
            const int kvh = is_k ? head - hq : head - hq - hkv;
            dst = (is_k ? k_cache : v_cache) + (((size_t)page * hkv + kvh) * page_size + pos % page_size) * D;
        }
        Pack o;
#pragma unroll
        for (int i = 0; i < VEC; ++i) o.e[i] = from_f32<T>(x[i]);
        *reinterpret_cast<Pack*>(dst + lane * VEC) = o;
    }
}

template <typename T>
static void launch_rope(T* q_out, const T* qkv, T* kc, size_t v_off, const float* q_norm_w, const float* k_norm_w,
                        float eps, const float* inv_freq, const float* table, int table_positions, int interleaved,
                        int rotary_dim, const int* positions, const int* token_seq,
                        const int* block_table, int max_blocks, int num_tokens, int hq, int hkv, int d, int page_size,
                        int num_pages, int* status, cudaStream_t stream) {
    dim3 grid((hq + 2 * hkv + RA_WARPS - 1) / RA_WARPS, num_tokens);
    T* vc = kc ? kc + v_off : nullptr;
    const bool whole = (inv_freq == nullptr && table == nullptr) || rotary_dim == d;
    // a warp takes one head of a token when tokens are few (a decode step wants the kernel short),
    // four when they are many (more bytes in flight per warp)
    const bool many = num_tokens >= 256;
    const dim3 grid4((hq + 2 * hkv + 4 * RA_WARPS - 1) / (4 * RA_WARPS), num_tokens);
#define TI_ROPE_ARGS q_out, qkv, kc, vc, q_norm_w, k_norm_w, eps, inv_freq, table, table_positions, interleaved, \
                     positions, token_seq, block_table, max_blocks, \
                     hq, hkv, page_size, num_pages, status
    if (whole && d == 128 && many)
        ti_launch(qk_norm_rope_append_vec_kernel<T, 128, 4>, grid4, RA_WARPS * 32, 0, stream, TI_ROPE_ARGS);
    else if (whole && d == 128)
        ti_launch(qk_norm_rope_append_vec_kernel<T, 128, 1>, grid, RA_WARPS * 32, 0, stream, TI_ROPE_ARGS);
    else if (whole && d == 64 && many)
        ti_launch(qk_norm_rope_append_vec_kernel<T, 64, 4>, grid4, RA_WARPS * 32, 0, stream, TI_ROPE_ARGS);
    else if (whole && d == 64)
        ti_launch(qk_norm_rope_append_vec_kernel<T, 64, 1>, grid, RA_WARPS * 32, 0, stream, TI_ROPE_ARGS);
#undef TI_ROPE_ARGS
    else
        ti_launch(qk_norm_rope_append_kernel<T>, grid, RA_WARPS * 32, 0, stream, q_out, qkv, kc, vc, q_norm_w, k_norm_w,
                  eps, inv_freq, table, table_positions, interleaved, rotary_dim, positions, token_seq, block_table,
                  max_blocks, hq, hkv, d, page_size, num_pages, status);
}

// inv_freq (float32 [rotary_dim / 2]) or cos_sin_table (float32 [table_positions, rotary_dim], cosines then
// sines of a position's rotary_dim / 2 angles) or neither (no rotation); interleaved: pairs (2j, 2j + 1)
// instead of (j, j + rotary_dim / 2).
TI_API int ti_qk_norm_rope_append(
    void* q_out, const void* qkv, void* kv_cache, const float* q_norm_w, const float* k_norm_w, float eps,
    const float* inv_freq, const float* cos_sin_table, int table_positions, int interleaved,
    int rotary_dim, const int* positions, const int* token_seq,
    const int* block_table, int max_blocks, int num_tokens, int hq, int hkv, int d, int page_size,
    int num_pages, int* status, int dtype, cudaStream_t stream) {
    TI_REQUIRE(d > 0 && d <= RA_MAX_D, "qk_norm_rope_append: head_dim %d not in 1..%d", d, RA_MAX_D);
    TI_REQUIRE(rotary_dim >= 0 && rotary_dim <= d && rotary_dim % 2 == 0,
               "qk_norm_rope_append: rotary_dim %d must be even and at most head_dim %d", rotary_dim, d);
    TI_REQUIRE(hq > 0 && hkv > 0 && page_size > 0 && num_tokens >= 0, "qk_norm_rope_append: bad sizes");
    TI_REQUIRE(inv_freq == nullptr || cos_sin_table == nullptr, "qk_norm_rope_append: inverse frequencies or a table, not both");
    TI_REQUIRE(cos_sin_table == nullptr || table_positions > 0, "qk_norm_rope_append: a table needs its number of positions");
    TI_REQUIRE(num_tokens <= 65535, "qk_norm_rope_append: more than 65535 tokens in one step");
    if (num_tokens == 0) return 0;
    const size_t v_off = (size_t)num_pages * hkv * page_size * d;
    if (dtype == TI_F32)
        launch_rope<float>((float*)q_out, (const float*)qkv, (float*)kv_cache, v_off, q_norm_w, k_norm_w, eps, inv_freq,
                           cos_sin_table, table_positions, interleaved, rotary_dim, positions, token_seq, block_table, max_blocks, num_tokens, hq, hkv, d, page_size,
                           num_pages, status, stream);
    else if (dtype == TI_BF16)
        launch_rope<__nv_bfloat16>((__nv_bfloat16*)q_out, (const __nv_bfloat16*)qkv, (__nv_bfloat16*)kv_cache, v_off,
                                   q_norm_w, k_norm_w, eps, inv_freq, cos_sin_table, table_positions, interleaved,
                                   rotary_dim, positions, token_seq, block_table,
                                   max_blocks, num_tokens, hq, hkv, d, page_size, num_pages, status, stream);
    else TI_REQUIRE(false, "qk_norm_rope_append: unknown dtype %d", dtype);
    TI_CHECK_LAUNCH("qk_norm_rope_append");
    return 0;
}
