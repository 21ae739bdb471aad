// Token choice from rows of float32 logits: greedy argmax, or temperature scaling, an optional
// top-k threshold and Gumbel-max (tinyinfer/layers/sampler.py:42-43 greedy with the first index
// winning ties; :59-63 scaled = logits / T, values below the k-th largest masked, ties at the
// threshold kept; :69-72 argmax(scaled + G), G = -log(-log(U))).
// U does not come from a global generator: element i of a row draws word i % 4 of the
// Philox-4x32-10 block with counter (i / 4, step, stream, 0) and key (seed), so a row's token
// depends only on (seed, stream, step) and its logits, whatever else is in the batch.
#include "common.cuh"

constexpr int SP_THREADS = 256;      // argmax parts, nll
constexpr int SK_THREADS = 1024;     // the one-block-per-row sampling kernel: a row is 150 thousand logits

__device__ __forceinline__ uint4 philox4x32_10(uint4 c, uint2 k) {
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const unsigned hi0 = __umulhi(0xD2511F53u, c.x), lo0 = 0xD2511F53u * c.x;
        const unsigned hi1 = __umulhi(0xCD9E8D57u, c.z), lo1 = 0xCD9E8D57u * c.z;
        c = make_uint4(hi1 ^ c.y ^ k.x, lo1, hi0 ^ c.w ^ k.y, lo0);
        k.x += 0x9E3779B9u;
        k.y += 0xBB67AE85u;
    }
    return c;
}
__device__ __forceinline__ float philox_uniform(unsigned word) {   // in (0, 1), exact in float32
    return ((float)(word >> 9) + 0.5f) * (1.0f / 8388608.0f);
}
__device__ __forceinline__ unsigned order_key(float v) {           // larger float -> larger key
    const unsigned b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

struct Best { float v; int i; };
__device__ __forceinline__ Best better(Best a, Best b) {
    if (b.i < 0) return a;
    if (a.i < 0) return b;
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}
__device__ __forceinline__ Best block_best(Best x, Best* sh) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best y;
        y.v = __shfl_xor_sync(0xffffffffu, x.v, o);
        y.i = __shfl_xor_sync(0xffffffffu, x.i, o);
        x = better(x, y);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) sh[warp] = x;
    __syncthreads();
    if (warp == 0) {
        Best y = lane < SP_THREADS / 32 ? sh[lane] : Best{0.f, -1};
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            Best z;
            z.v = __shfl_xor_sync(0xffffffffu, y.v, o);
            z.i = __shfl_xor_sync(0xffffffffu, y.i, o);
            y = better(y, z);
        }
        if (lane == 0) sh[0] = y;
    }
    __syncthreads();
    return sh[0];
}

// Block-wide best for blocks of NT threads.
template <int NT>
__device__ __forceinline__ Best block_best_n(Best x, Best* sh) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best y;
        y.v = __shfl_xor_sync(0xffffffffu, x.v, o);
        y.i = __shfl_xor_sync(0xffffffffu, x.i, o);
        x = better(x, y);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) sh[warp] = x;
    __syncthreads();
    if (warp == 0) {
        Best y = lane < NT / 32 ? sh[lane] : Best{0.f, -1};
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            Best z;
            z.v = __shfl_xor_sync(0xffffffffu, y.v, o);
            z.i = __shfl_xor_sync(0xffffffffu, y.i, o);
            y = better(y, z);
        }
        if (lane == 0) sh[0] = y;
    }
    __syncthreads();
    return sh[0];
}

// Calls f(value, index) for every logit of the row, four at a time where the row allows it.
template <typename F>
__device__ __forceinline__ void for_each_logit(const float* x, int vocab, F f) {
    if ((((uintptr_t)x) & 15) == 0 && (vocab & 3) == 0) {
        for (int i = threadIdx.x * 4; i < vocab; i += SK_THREADS * 4) {
            const float4 v = *reinterpret_cast<const float4*>(x + i);
            f(v.x, i); f(v.y, i + 1); f(v.z, i + 2); f(v.w, i + 3);
        }
    } else {
        for (int i = threadIdx.x; i < vocab; i += SK_THREADS) f(x[i], i);
    }
}

__global__ void __launch_bounds__(SK_THREADS) sample_kernel(
    int* __restrict__ out, const float* __restrict__ logits, int vocab,
    const float* __restrict__ temperature, const int* __restrict__ topk, const int* __restrict__ greedy,
    const long long* __restrict__ seed, const int* __restrict__ stream_id, const int* __restrict__ step,
    const int* __restrict__ extra, int num_extra) {
    __shared__ Best sh_best[SK_THREADS / 32];
    __shared__ unsigned hist[256];
    __shared__ unsigned sel_prefix, sel_remaining;
    ti_grid_launch_dependents();
    ti_grid_wait();
    const int row = blockIdx.x, tid = threadIdx.x;
    if (row == 0 && tid < num_extra) out[gridDim.x + tid] = extra[tid];   // words that ride home with the tokens
    const float* x = logits + (size_t)row * vocab;

    if (greedy == nullptr || greedy[row]) {
        Best b{0.f, -1};
        for_each_logit(x, vocab, [&](float v, int i) { if (v == v) b = better(b, Best{v, i}); });
        b = block_best_n<SK_THREADS>(b, sh_best);
        if (tid == 0) out[row] = b.i < 0 ? 0 : b.i;
        return;
    }

    const float temp = temperature[row];
    const int k = topk[row];
    unsigned threshold = 0u;                              // keys below it are masked
    if (k > 0 && k < vocab) {
        // radix select of the k-th largest key, one byte per pass from the top
        if (tid == 0) { sel_prefix = 0u; sel_remaining = (unsigned)k; }
        for (int pass = 0; pass < 4; ++pass) {
            const int shift = 24 - 8 * pass;
            if (tid < 256) hist[tid] = 0u;
            __syncthreads();
            const unsigned prefix = sel_prefix;
            const unsigned mask = pass == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
            for_each_logit(x, vocab, [&](float raw, int) {
                const float v = raw / temp;
                if (v == v) {
                    const unsigned key = order_key(v);
                    if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 0xFFu], 1u);
                }
            });
            __syncthreads();
            if (tid == 0) {
                unsigned remaining = sel_remaining;
                int b = 255;
                for (; b > 0; --b) {
                    if (hist[b] >= remaining) break;
                    remaining -= hist[b];
                }
                sel_prefix = prefix | ((unsigned)b << shift);
                sel_remaining = remaining;
            }
            __syncthreads();
        }
        threshold = sel_prefix;
    }

    const uint2 key2 = make_uint2((unsigned)(seed[row] & 0xFFFFFFFFll), (unsigned)((unsigned long long)seed[row] >> 32));
    const unsigned c1 = (unsigned)step[row], c2 = (unsigned)stream_id[row];
    Best b{0.f, -1};
    const bool vec = (((uintptr_t)x) & 15) == 0 && (vocab & 3) == 0;
    for (int blk = tid; blk * 4 < vocab; blk += SK_THREADS) {
        float vals[4];
        if (vec) {
            const float4 q = *reinterpret_cast<const float4*>(x + blk * 4);
            vals[0] = q.x; vals[1] = q.y; vals[2] = q.z; vals[3] = q.w;
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) vals[j] = blk * 4 + j < vocab ? x[blk * 4 + j] : -INFINITY;
        }
        bool any = false;
        float sc[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            sc[j] = vals[j] / temp;
            const bool keep = blk * 4 + j < vocab && sc[j] == sc[j] && sc[j] != -INFINITY && order_key(sc[j]) >= threshold;
            if (!keep) sc[j] = -INFINITY;
            any |= keep;
        }
        if (!any) continue;                               // the random block is only drawn where something survives
        const uint4 r = philox4x32_10(make_uint4((unsigned)blk, c1, c2, 0u), key2);
        const unsigned words[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (sc[j] == -INFINITY) continue;
            const float g = -logf(-logf(philox_uniform(words[j])));
            b = better(b, Best{sc[j] + g, blk * 4 + j});
        }
    }
    b = block_best_n<SK_THREADS>(b, sh_best);
    if (tid == 0) out[row] = b.i < 0 ? 0 : b.i;
}

// greedy == nullptr: every row is an argmax and the other per-row arrays are not read.
// extra / num_extra: device words (the kernels' status words, say) copied to out[num_rows ...] so that
// one device-to-host copy brings them home with the tokens; out then has num_rows + num_extra entries.
TI_API int ti_sample(int* out, const float* logits, int num_rows, int vocab, const float* temperature,
                     const int* topk, const int* greedy, const long long* seed, const int* stream_id,
                     const int* step, const int* extra, int num_extra, cudaStream_t stream) {
    TI_REQUIRE(num_rows >= 0 && vocab > 0, "sample: bad sizes");
    TI_REQUIRE(num_extra >= 0 && num_extra <= 32 && (num_extra == 0 || extra != nullptr), "sample: bad extra words");
    if (num_rows == 0) return 0;
    ti_launch(sample_kernel, num_rows, SK_THREADS, 0, stream, out, logits, vocab, temperature, topk, greedy, seed, stream_id, step,
              extra, num_extra);
    TI_CHECK_LAUNCH("sample");
    return 0;
}

// ------------------------------------------------------------------ argmax over many blocks
// A row of 150 thousand logits is too long for one block: AM_PARTS blocks each scan a slice and
// leave their best in scratch; the block that arrives last (a counter per row, left at zero again)
// picks among the parts. Ties go to the lowest index at both levels.
constexpr int AM_PARTS = 32;

__global__ void __launch_bounds__(SP_THREADS) argmax_parts_kernel(
    int* __restrict__ out, const float* __restrict__ logits, int vocab, float* __restrict__ part_val,
    int* __restrict__ part_idx, int* __restrict__ counters, const int* __restrict__ extra, int num_extra) {
    __shared__ Best sh_best[SP_THREADS / 32];
    __shared__ int last_sh;
    ti_grid_launch_dependents();
    ti_grid_wait();
    const int part = blockIdx.x, row = blockIdx.y, tid = threadIdx.x;
    if (part == 0 && row == 0 && tid < num_extra) out[gridDim.y + tid] = extra[tid];
    const float* x = logits + (size_t)row * vocab;
    const int chunk = ((vocab + AM_PARTS - 1) / AM_PARTS + 3) & ~3;
    const int begin = part * chunk, end = min(vocab, begin + chunk);
    Best b{0.f, -1};
    if ((((uintptr_t)x) & 15) == 0 && (vocab & 3) == 0) {
        for (int i = begin + tid * 4; i < end; i += SP_THREADS * 4) {
            const float4 v = *reinterpret_cast<const float4*>(x + i);
            if (v.x == v.x) b = better(b, Best{v.x, i});
            if (v.y == v.y) b = better(b, Best{v.y, i + 1});
            if (v.z == v.z) b = better(b, Best{v.z, i + 2});
            if (v.w == v.w) b = better(b, Best{v.w, i + 3});
        }
    } else {
        for (int i = begin + tid; i < end; i += SP_THREADS) {
            const float v = x[i];
            if (v == v) b = better(b, Best{v, i});
        }
    }
    b = block_best(b, sh_best);
    if (tid == 0) {
        part_val[row * AM_PARTS + part] = b.v;
        part_idx[row * AM_PARTS + part] = b.i;
        __threadfence();
        const int arrived = atomicAdd(counters + row, 1);
        last_sh = arrived == AM_PARTS - 1;
        if (last_sh) counters[row] = 0;
    }
    __syncthreads();
    if (!last_sh) return;
    __threadfence();
    Best m{0.f, -1};
    if (tid < AM_PARTS) m = Best{__ldcg(part_val + row * AM_PARTS + tid), __ldcg(part_idx + row * AM_PARTS + tid)};
    m = block_best(m, sh_best);
    if (tid == 0) out[row] = m.i < 0 ? 0 : m.i;
}

TI_API int ti_argmax_parts() { return AM_PARTS; }

// part_val / part_idx: scratch of num_rows * ti_argmax_parts() entries; counters: num_rows zeroed ints
// (left zeroed). Calls that share them must be ordered on one stream. extra / num_extra: as in ti_sample.
TI_API int ti_argmax(int* out, const float* logits, int num_rows, int vocab, float* part_val, int* part_idx,
                     int* counters, const int* extra, int num_extra, cudaStream_t stream) {
    TI_REQUIRE(num_rows >= 0 && num_rows <= 65535 && vocab > 0, "argmax: bad sizes");
    TI_REQUIRE(num_extra >= 0 && num_extra <= 32 && (num_extra == 0 || extra != nullptr), "argmax: bad extra words");
    if (num_rows == 0) return 0;
    ti_launch(argmax_parts_kernel, dim3(AM_PARTS, num_rows), SP_THREADS, 0, stream, out, logits, vocab, part_val,
              part_idx, counters, extra, num_extra);
    TI_CHECK_LAUNCH("argmax");
    return 0;
}

// ------------------------------------------------------------------ negative log-likelihood
// nll[row] = logsumexp(logits[row]) - logits[row][token[row]] in float32
// (tinyinfer/layers/sampler.py:82-86 of the reference): what the perplexity statistic sums.
__global__ void __launch_bounds__(SP_THREADS) nll_kernel(float* __restrict__ out, const float* __restrict__ logits,
                                                         const int* __restrict__ tokens, int vocab) {
    __shared__ float red[33];
    ti_grid_launch_dependents();
    ti_grid_wait();
    const int row = blockIdx.x;
    const float* x = logits + (size_t)row * vocab;
    float mx = -INFINITY;
    for (int i = threadIdx.x; i < vocab; i += SP_THREADS) mx = fmaxf(mx, x[i]);
    mx = block_max(mx, red);
    float sum = 0.f;
    for (int i = threadIdx.x; i < vocab; i += SP_THREADS) sum += expf(x[i] - mx);
    sum = block_sum(sum, red);
    if (threadIdx.x == 0) {
        const int t = tokens[row];
        out[row] = (t >= 0 && t < vocab) ? mx + logf(sum) - x[t] : 0.f;
    }
}

TI_API int ti_token_nll(float* out, const float* logits, const int* tokens, int num_rows, int vocab, cudaStream_t stream) {
    TI_REQUIRE(num_rows >= 0 && vocab > 0, "token_nll: bad sizes");
    if (num_rows == 0) return 0;
    ti_launch(nll_kernel, num_rows, SP_THREADS, 0, stream, out, logits, tokens, vocab);
    TI_CHECK_LAUNCH("token_nll");
    return 0;
}
