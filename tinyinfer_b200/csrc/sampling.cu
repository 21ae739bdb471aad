// Token choice from rows of float32 logits: greedy argmax, or temperature scaling, an optional
// top-k threshold and Gumbel-max (tinyinfer/layers/sampler.py:42-43 greedy with the first index
// winning ties; :59-63 scaled = logits / T, values below the k-th largest masked, ties at the
// threshold kept; :69-72 argmax(scaled + G), G = -log(-log(U))).
// U does not come from a global generator: element i of a row draws word i % 4 of the
// Philox-4x32-10 block with counter (i / 4, step, stream, 0) and key (seed), so a row's token
// depends only on (seed, stream, step) and its logits, whatever else is in the batch.
#include "common.cuh"

constexpr int SP_THREADS = 256;      // argmax parts, nll

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

// Calls f(value, index) for the logits [begin, end) of the row (begin a multiple of 4), four at a time where
// the row allows it. NT threads.
template <int NT, typename F>
__device__ __forceinline__ void for_each_logit(const float* x, int vocab, int begin, int end, F f) {
    if ((((uintptr_t)x) & 15) == 0 && (vocab & 3) == 0) {
        for (int i = begin + threadIdx.x * 4; i < end; i += NT * 4) {
            const float4 v = *reinterpret_cast<const float4*>(x + i);
            f(v.x, i); f(v.y, i + 1); f(v.z, i + 2); f(v.w, i + 3);
        }
    } else {
        for (int i = begin + threadIdx.x; i < end; i += NT) f(x[i], i);
    }
}

// Radix select, one byte per pass from the top: the k-th largest of the keys that `each` hands out (it calls
// its argument once per key; every thread of the block calls select_kth with the same k). 0 if k <= 0.
// hist: 256 shared words; sel: 2 shared words. The counts of a pass go into the histogram warp by warp: lanes
// that hold the same byte count themselves once together (most logits share their sign and exponent, so a
// plain atomic per key would make a warp wait for itself 32 times over); the bin that holds the k-th largest
// is found by the first warp together (a suffix sum over lanes of eight bins each), not by one thread.
// One pass: sel[0] holds the bytes found so far (from the top), sel[1] which of the keys that begin with them,
// counted from the largest, is looked for; afterwards one byte more and the rank among those.
template <typename Each>
__device__ __forceinline__ void radix_pass(int pass, unsigned* hist, unsigned* sel, Each each) {
    {
        const int shift = 24 - 8 * pass;
        for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0u;
        __syncthreads();
        const unsigned prefix = sel[0];
        const unsigned mask = pass == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
        each([&](unsigned key) {
            if ((key & mask) == prefix) {
                const unsigned bin = (key >> shift) & 0xFFu;
                const unsigned same = __match_any_sync(__activemask(), bin);
                if ((threadIdx.x & 31) == (unsigned)(__ffs(same) - 1)) atomicAdd(&hist[bin], (unsigned)__popc(same));
            }
        });
        __syncthreads();
        if (threadIdx.x < 32) {
            const int lane = threadIdx.x;
            unsigned mine[8], sum = 0u;
#pragma unroll
            for (int i = 0; i < 8; ++i) { mine[i] = hist[8 * lane + i]; sum += mine[i]; }
            unsigned above = sum;                                  // keys in this lane's bins and all higher ones
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const unsigned v = __shfl_down_sync(0xffffffffu, above, off);
                if (lane + off < 32) above += v;
            }
            const unsigned remaining = sel[1];
            // the highest lane whose bins, with all above them, reach the k-th largest; lane 0 if none does
            const unsigned reach = __ballot_sync(0xffffffffu, above >= remaining);
            const int owner = reach ? 31 - __clz(reach) : 0;
            if (lane == owner) {
                unsigned left = remaining - (above - sum);         // still to find inside this lane's bins
                int b = 7;
                if (reach) {
                    for (; b > 0; --b) {
                        if (mine[b] >= left) break;
                        left -= mine[b];
                    }
                } else {
                    b = 0;                                         // fewer keys than k: bin 0, as the plain walk does
                    left = remaining;
                    for (int i = 255; i > 0; --i) left -= hist[i];
                }
                sel[0] = prefix | ((unsigned)(8 * lane + b) << shift);
                sel[1] = left;
            }
        }
        __syncthreads();
    }
}
template <typename Each>
__device__ __forceinline__ unsigned select_kth(int k, unsigned* hist, unsigned* sel, Each each) {
    if (k <= 0) return 0u;
    if (threadIdx.x == 0) { sel[0] = 0u; sel[1] = (unsigned)k; }
    for (int pass = 0; pass < 4; ++pass) radix_pass(pass, hist, sel, each);
    return sel[0];
}

__device__ __forceinline__ float key_value(unsigned key) {          // the inverse of order_key
    return __uint_as_float((key & 0x80000000u) ? (key & 0x7FFFFFFFu) : ~key);
}
__device__ __forceinline__ float gumbel(int index, unsigned c1, unsigned c2, uint2 key2) {
    const uint4 r = philox4x32_10(make_uint4((unsigned)(index >> 2), c1, c2, 0u), key2);
    const unsigned words[4] = {r.x, r.y, r.z, r.w};
    return -logf(-logf(philox_uniform(words[index & 3])));
}

// Gumbel-max over the logits [begin, end) of a row whose scaled value's key is at least `threshold`.
template <int NT>
__device__ __forceinline__ Best gumbel_best(const float* x, int vocab, int begin, int end, float temp, unsigned threshold,
                                            unsigned c1, unsigned c2, uint2 key2) {
    Best b{0.f, -1};
    const bool vec = (((uintptr_t)x) & 15) == 0 && (vocab & 3) == 0;
    for (int blk = (begin >> 2) + threadIdx.x; blk * 4 < end; blk += NT) {
        float vals[4];
        if (vec) {
            const float4 q = *reinterpret_cast<const float4*>(x + blk * 4);
            vals[0] = q.x; vals[1] = q.y; vals[2] = q.z; vals[3] = q.w;
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) vals[j] = blk * 4 + j < end ? x[blk * 4 + j] : -INFINITY;
        }
        bool any = false;
        float sc[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            sc[j] = vals[j] / temp;
            const bool keep = blk * 4 + j < end && sc[j] == sc[j] && sc[j] != -INFINITY && order_key(sc[j]) >= threshold;
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
    return b;
}

// A row of 150 thousand logits is too long for one block, and a Gumbel draw costs a Philox block and two
// logarithms: SMP_PARTS blocks each take a slice of the row and the block that arrives last (a counter per
// row, left at zero again) finishes it.
//   greedy, or temperature without top-k: a part leaves its best (scaled logit + Gumbel noise for the
//       latter) and the last block picks among the parts: the argmax of a row is the best of its slices' best.
//   top-k with k <= SMP_CAP: a part finds the k-th largest scaled logit OF ITS SLICE and leaves every logit of
//       the slice that is at least that (its key and index). Every logit among the row's k largest, ties with
//       the k-th included, is among those; the last block selects the k-th largest of the at most SMP_PARTS *
//       SMP_CAP candidates, which is the row's, and draws among the candidates that reach it. The noise
//       of a logit depends on its index alone, so the token is the one a scan of the whole row would give.
//   larger k, or more than SMP_CAP candidates in a slice (hundreds of equal logits): the last block scans the
//       whole row itself.
constexpr int SMP_PARTS = 16;
constexpr int SMP_THREADS = 256;
constexpr int SMP_CAP = 256;

__global__ void __launch_bounds__(SMP_THREADS) sample_parts_kernel(
    int* __restrict__ out, const float* __restrict__ logits, int vocab,
    const float* __restrict__ temperature, const int* __restrict__ topk, const int* __restrict__ greedy,
    const long long* __restrict__ seed, const int* __restrict__ stream_id, const int* __restrict__ step,
    float* __restrict__ part_val, int* __restrict__ part_idx, unsigned* __restrict__ cand_key,
    int* __restrict__ cand_idx, int* __restrict__ cand_cnt, int* __restrict__ counters,
    const int* __restrict__ extra, int num_extra) {
    __shared__ Best sh_best[SMP_THREADS / 32];
    __shared__ unsigned hist[256];
    __shared__ unsigned sel[2];
    __shared__ int count_sh, aside_sh, last_sh;
    __shared__ unsigned keys_sh[SMP_PARTS * SMP_CAP];
    __shared__ int idx_sh[SMP_PARTS * SMP_CAP];
    ti_grid_launch_dependents();
    ti_grid_wait();
    const int part = blockIdx.x, row = blockIdx.y, tid = threadIdx.x;
    if (part == 0 && row == 0 && tid < num_extra) out[gridDim.y + tid] = extra[tid];   // words that ride home with the tokens
    const float* x = logits + (size_t)row * vocab;
    const int chunk = ((vocab + SMP_PARTS - 1) / SMP_PARTS + 3) & ~3;
    const int begin = min(vocab, part * chunk), end = min(vocab, begin + chunk);
    const bool is_greedy = greedy == nullptr || greedy[row];
    const float temp = is_greedy ? 1.f : temperature[row];
    const int k = is_greedy ? 0 : topk[row];
    const bool top = k > 0 && k < vocab;
    const uint2 key2 = is_greedy ? make_uint2(0u, 0u)
                                 : make_uint2((unsigned)(seed[row] & 0xFFFFFFFFll), (unsigned)((unsigned long long)seed[row] >> 32));
    const unsigned c1 = is_greedy ? 0u : (unsigned)step[row], c2 = is_greedy ? 0u : (unsigned)stream_id[row];

    Best b{0.f, -1};
    if (is_greedy) {
        for_each_logit<SMP_THREADS>(x, vocab, begin, end, [&](float v, int i) { if (v == v) b = better(b, Best{v, i}); });
    } else if (!top) {
        b = gumbel_best<SMP_THREADS>(x, vocab, begin, end, temp, 0u, c1, c2, key2);
    } else if (k <= SMP_CAP) {
        // The slice's k-th largest scaled logit. The first byte from a scan of the slice; then the logits that share
        // that byte with it (a few hundred of some ten thousand, as a rule) are set aside in shared memory, those
        // above it are candidates already, and the other three bytes come from what was set aside: two scans of
        // the slice, each with its division, instead of five.
        auto slice_keys = [&](auto count) {
            for_each_logit<SMP_THREADS>(x, vocab, begin, end, [&](float raw, int) {
                const float v = raw / temp;
                if (v == v) count(order_key(v));
            });
        };
        unsigned* ck = cand_key + ((size_t)row * SMP_PARTS + part) * SMP_CAP;
        int* ci = cand_idx + ((size_t)row * SMP_PARTS + part) * SMP_CAP;
        if (tid == 0) { sel[0] = 0u; sel[1] = (unsigned)k; count_sh = 0; aside_sh = 0; }
        radix_pass(0, hist, sel, slice_keys);               // (its first barrier also publishes the words just set)
        const unsigned first_byte = sel[0] >> 24;
        constexpr int ASIDE = SMP_PARTS * SMP_CAP;          // the candidate arrays of the last block: free until then
        for_each_logit<SMP_THREADS>(x, vocab, begin, end, [&](float raw, int i) {
            const float v = raw / temp;
            if (v == v) {
                const unsigned key = order_key(v);
                if ((key >> 24) > first_byte) {
                    const int at = atomicAdd(&count_sh, 1);
                    if (at < SMP_CAP) { ck[at] = key; ci[at] = i; }
                } else if ((key >> 24) == first_byte) {
                    const int at = atomicAdd(&aside_sh, 1);
                    if (at < ASIDE) { keys_sh[at] = key; idx_sh[at] = i; }
                }
            }
        });
        __syncthreads();
        const int aside = aside_sh;
        if (aside <= ASIDE) {
            const int above = count_sh;                     // logits above the first byte's bin: all among the k largest
            const unsigned local = select_kth(k - above, hist, sel, [&](auto count) {
                for (int i = tid; i < aside; i += SMP_THREADS) count(keys_sh[i]);
            });
            for (int i = tid; i < aside; i += SMP_THREADS) {
                if (keys_sh[i] >= local) {
                    const int at = atomicAdd(&count_sh, 1);
                    if (at < SMP_CAP) { ck[at] = keys_sh[i]; ci[at] = idx_sh[i]; }
                }
            }
        } else {
            // more logits share the first byte than shared memory holds: the other bytes from scans of the slice
            if (tid == 0) count_sh = 0;
            for (int pass = 1; pass < 4; ++pass) radix_pass(pass, hist, sel, slice_keys);
            const unsigned local = sel[0];
            for_each_logit<SMP_THREADS>(x, vocab, begin, end, [&](float raw, int i) {
                const float v = raw / temp;
                if (v == v && order_key(v) >= local) {
                    const int at = atomicAdd(&count_sh, 1);
                    if (at < SMP_CAP) { ck[at] = order_key(v); ci[at] = i; }
                }
            });
        }
        __syncthreads();
        if (tid == 0) cand_cnt[row * SMP_PARTS + part] = count_sh <= SMP_CAP ? count_sh : -1;
    }
    if (is_greedy || !top) {
        b = block_best_n<SMP_THREADS>(b, sh_best);
        if (tid == 0) { part_val[row * SMP_PARTS + part] = b.v; part_idx[row * SMP_PARTS + part] = b.i; }
    }
    __syncthreads();                                      // every thread's candidates are written
    if (tid == 0) {
        __threadfence();
        const int arrived = atomicAdd(counters + row, 1);
        last_sh = arrived == SMP_PARTS - 1;
        if (last_sh) counters[row] = 0;
    }
    __syncthreads();
    if (!last_sh) return;
    __threadfence();

    Best m{0.f, -1};
    if (is_greedy || !top) {
        if (tid < SMP_PARTS) m = Best{__ldcg(part_val + row * SMP_PARTS + tid), __ldcg(part_idx + row * SMP_PARTS + tid)};
    } else {
        // all parts' counts in one trip, then all candidates in one
        __shared__ int start_sh[SMP_PARTS + 1];
        if (tid == 0) {
            int n[SMP_PARTS];
#pragma unroll
            for (int pp = 0; pp < SMP_PARTS; ++pp) n[pp] = k > SMP_CAP ? -1 : __ldcg(cand_cnt + row * SMP_PARTS + pp);
            int total0 = 0;
            bool over = false;
#pragma unroll
            for (int pp = 0; pp < SMP_PARTS; ++pp) {
                start_sh[pp] = total0;
                if (n[pp] < 0) over = true; else total0 += n[pp];
            }
            start_sh[SMP_PARTS] = over ? -1 : total0;
        }
        __syncthreads();
        const int total = start_sh[SMP_PARTS];
        const bool whole = total < 0;
        if (!whole) {
            for (int i = tid; i < SMP_PARTS * SMP_CAP; i += SMP_THREADS) {
                const int pp = i / SMP_CAP, at = i % SMP_CAP;
                if (at < start_sh[pp + 1 < SMP_PARTS ? pp + 1 : SMP_PARTS] - start_sh[pp]) {
                    keys_sh[start_sh[pp] + at] = __ldcg(cand_key + ((size_t)row * SMP_PARTS + pp) * SMP_CAP + at);
                    idx_sh[start_sh[pp] + at] = __ldcg(cand_idx + ((size_t)row * SMP_PARTS + pp) * SMP_CAP + at);
                }
            }
        }
        __syncthreads();
        if (whole) {
            // the plain way: select over the whole row, then draw over the whole row
            const unsigned threshold = select_kth(k, hist, sel, [&](auto count) {
                for_each_logit<SMP_THREADS>(x, vocab, 0, vocab, [&](float raw, int) {
                    const float v = raw / temp;
                    if (v == v) count(order_key(v));
                });
            });
            m = gumbel_best<SMP_THREADS>(x, vocab, 0, vocab, temp, threshold, c1, c2, key2);
        } else {
            const unsigned threshold = select_kth(k, hist, sel, [&](auto count) {
                for (int i = tid; i < total; i += SMP_THREADS) count(keys_sh[i]);
            });
            for (int i = tid; i < total; i += SMP_THREADS) {
                const float sc = key_value(keys_sh[i]);
                if (keys_sh[i] >= threshold && sc != -INFINITY)
                    m = better(m, Best{sc + gumbel(idx_sh[i], c1, c2, key2), idx_sh[i]});
            }
        }
    }
    m = block_best_n<SMP_THREADS>(m, sh_best);
    if (tid == 0) out[row] = m.i < 0 ? 0 : m.i;
}

TI_API int ti_sample_parts() { return SMP_PARTS; }
TI_API int ti_sample_candidates() { return SMP_CAP; }

// greedy == nullptr: every row is an argmax and the other per-row arrays are not read.
// Scratch: part_val / part_idx of num_rows * ti_sample_parts() entries, cand_key / cand_idx of num_rows *
// ti_sample_parts() * ti_sample_candidates(), cand_cnt of num_rows * ti_sample_parts(), counters: num_rows
// zeroed ints (left zeroed). Calls that share them must be ordered on one stream.
// extra / num_extra: device words (the kernels' status words, say) copied to out[num_rows ...] so that
// one device-to-host copy brings them home with the tokens; out then has num_rows + num_extra entries.
TI_API int ti_sample(int* out, const float* logits, int num_rows, int vocab, const float* temperature,
                     const int* topk, const int* greedy, const long long* seed, const int* stream_id,
                     const int* step, float* part_val, int* part_idx, unsigned* cand_key, int* cand_idx, int* cand_cnt,
                     int* counters, const int* extra, int num_extra, cudaStream_t stream) {
    TI_REQUIRE(num_rows >= 0 && num_rows <= 65535 && vocab > 0, "sample: bad sizes");
    TI_REQUIRE(num_extra >= 0 && num_extra <= 32 && (num_extra == 0 || extra != nullptr), "sample: bad extra words");
    if (num_rows == 0) return 0;
    ti_launch(sample_parts_kernel, dim3(SMP_PARTS, num_rows), SMP_THREADS, 0, stream, out, logits, vocab, temperature, topk,
              greedy, seed, stream_id, step, part_val, part_idx, cand_key, cand_idx, cand_cnt, counters, extra, num_extra);
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
