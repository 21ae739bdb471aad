// Causal paged attention for portions of prompts on the tcgen05 tensor cores (bfloat16, head sizes
// 64 and 128). One CTA owns 128 consecutive query tokens of one request and one query head:
//
//   warp 0      TMA: the query tile once, then key/value tiles of 128 keys from the pages (the cached
//               prefix and the portion itself, through the block table) into a 2-stage ring;
//   warp 1      one thread issues the MMAs: S = Q K^T (128 x 128, fp32 in tensor memory, two buffers so
//               that the scores of tile j+1 are computed while tile j is in the softmax), then
//               O_j = P V (P from shared memory, V straight from the page layout as an MN-major operand);
//   warps 2..9  softmax: two threads share a query row (its tensor-memory lane), each half of the keys
//               and of the output features; they read the scores with tcgen05.ld, mask by assignment,
//               keep the running maximum (from -inf) and sum in float32, write P as bfloat16 into the
//               swizzled operand tile, and fold every O_j into their float32 output row in registers
//               with the usual rescaling.
//
// It replaces what the reference does with a gather on the host and a scalar FlashAttention kernel
// (tinyinfer/layers/attention.py:60-81, tinyinfer/csrc/flash_attention.cu:5-234). Every mbarrier wait
// is bounded (status word, abort flag, tensor memory freed on the common exit). Value rows that no
// query of the CTA may see are zeroed in shared memory before the second product, so pages that
// were never written or were given back cannot leak NaNs through 0 * NaN.
#include "sm100_ptx.cuh"

namespace {

constexpr int QM = 128;              // query rows per CTA = accumulator lanes
constexpr int KT = 128;              // keys per tile
constexpr int KV_STAGES = 2;
constexpr int PF_THREADS = 320;      // TMA warp, MMA warp, eight softmax warps

struct PrefillParams {
    __nv_bfloat16* out;              // [T, Hq * D]
    const int* tiles;                // int4 {request index, first flat row, rows (<= 128), first position}
    const int* block_table;
    int max_blocks, hq, hkv, page_size, num_pages, window;
    int halves;                      // 1: a tile entry has up to 256 rows and two CTAs take 128 each
    int splits, split_keys;          // > 1: CTA z of a tile takes keys z * split_keys .. (a multiple of 128) and leaves a partial
    float* part_o;                   // [128-row tile][split][head][row][D] unnormalised outputs
    float* part_ml;                  // [128-row tile][split][head][row][2] maximum (log2 domain) and sum
    float scale_log2;
    int* status;
};

template <int D>
struct PfSmem {
    static constexpr int HALVES = D / 64;
    static constexpr int Q_BYTES = HALVES * QM * 128;
    static constexpr int KV_TILE = HALVES * KT * 128;         // keys OR values of a tile
    static constexpr int STAGE = 2 * KV_TILE;
    static constexpr int P_BYTES = (KT / 64) * QM * 128;
    static constexpr int BYTES = 1024 + Q_BYTES + KV_STAGES * STAGE + P_BYTES + 256;
    static constexpr int TMEM_COLS = 512;                     // S0 at 0, S1 at 128, O_j at 256
};

__device__ __forceinline__ float ex2(float x) {          // 2^x, flushing; inputs are <= 0 or -inf
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

template <int D>
__global__ void __launch_bounds__(PF_THREADS, 1)
prefill_attention_tc_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap kv_map,
                            const PrefillParams p) {
    using S = PfSmem<D>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* q_tile = smem;
    uint8_t* kv_ring = smem + S::Q_BYTES;
    uint8_t* p_tile = kv_ring + KV_STAGES * S::STAGE;
    uint64_t* bars = reinterpret_cast<uint64_t*>(p_tile + S::P_BYTES);
    const uint32_t bar0 = smem_u32(bars);
    // barriers: q_full, kv_full[2], kv_empty[2], s_full[2], s_empty[2], p_full, o_full
    const uint32_t q_full = bar0;
    auto kv_full = [&](int s) { return bar0 + 8u * (1 + s); };
    auto kv_empty = [&](int s) { return bar0 + 8u * (3 + s); };
    auto s_full = [&](int b) { return bar0 + 8u * (5 + b); };
    auto s_empty = [&](int b) { return bar0 + 8u * (7 + b); };
    const uint32_t p_full = bar0 + 8u * 9, o_full = bar0 + 8u * 10;
    __shared__ uint32_t tmem_base_sh;
    __shared__ float max_xch[2][2][QM];      // [tile parity][column half][row]: row maxima of the halves
    __shared__ float sum_xch[2][QM];
    __shared__ int abort_sh;
    volatile int* abort_flag = &abort_sh;

    ti_grid_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        abort_sh = 0;
        mbar_init(q_full, 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(kv_full(s), 1);
            mbar_init(kv_empty(s), 1);
            mbar_init(s_full(s), 1);
            mbar_init(s_empty(s), 8);
        }
        mbar_init(p_full, 8);
        mbar_init(o_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(&tmem_base_sh, S::TMEM_COLS);
    tmem_fence_before();
    __syncthreads();
    tmem_fence_after();
    const uint32_t tmem_base = tmem_base_sh;
    ti_grid_wait();                                     // q, the pages and the tables come from earlier kernels

    // heads along x, tiles (longest key range first) along y: CTAs are handed out x first, so every head of
    // the longest tile starts before any shorter tile does
    const int4 td = reinterpret_cast<const int4*>(p.tiles)[p.halves ? blockIdx.y >> 1 : blockIdx.y];
    const int half_off = p.halves ? (blockIdx.y & 1) * QM : 0;
    const int seq = td.x, row0 = td.y + half_off, pos0 = td.w + half_off;
    const int nrows = min(td.z - half_off, QM);
    const int head = blockIdx.x;
    const int kvh = head / (p.hq / p.hkv);
    const int hi = pos0 + nrows;                                   // one past the last key any query sees
    const int lo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0; // first key the first query sees
    // With a split of the keys (few query tiles behind long prefixes: too few CTAs otherwise) this CTA takes the
    // key tiles of its share only and leaves an unnormalised partial result for the merge kernel.
    int tile0 = lo / KT, tile1 = (hi + KT - 1) / KT;
    if (p.splits > 1) {
        tile0 = max(tile0, (int)blockIdx.z * (p.split_keys / KT));
        tile1 = min(tile1, ((int)blockIdx.z + 1) * (p.split_keys / KT));
    }
    const int num_tiles = tile1 - tile0;
    const int* table = p.block_table + (size_t)seq * p.max_blocks;

    if (nrows <= 0 || num_tiles <= 0) {
        // the second half of an entry of at most 128 rows, or a share of the keys this tile has none of:
        // nothing to do but the common exit
    } else if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        // A tile is KT / piece_rows pieces (a piece lies in one page) x head halves x (keys, values): up to
        // 32 copies. Each lane issues one of them, so that a tile is on its way in one round instead of
        // one copy after the other; lane 0 waits for the stage and arms its barrier.
        if (lane == 0) {
            mbar_expect_tx(q_full, S::Q_BYTES);
#pragma unroll
            for (int hh = 0; hh < S::HALVES; ++hh)
                tma_load_2d(smem_u32(q_tile) + hh * (QM * 128), &q_map, q_full, head * D + hh * 64, row0);
        }
        const int piece_rows = p.page_size < 64 ? p.page_size : 64;
        const int num_copies = (KT / piece_rows) * S::HALVES * 2;
        const int my_piece = lane / (S::HALVES * 2), my_half = (lane >> 1) % S::HALVES, my_kv = lane & 1;
        auto page_of_tile = [&](int j) {                            // this lane's page of tile j, read ahead of its use
            const int logical = ((tile0 + j) * KT + my_piece * piece_rows) / p.page_size;
            const int page = (j < num_tiles && lane < num_copies && logical < p.max_blocks) ? table[logical] : -1;
            return page >= p.num_pages ? -1 : page;                 // never written, or given back by a window
        };
        int page_next = page_of_tile(0);
        for (int j = 0; j < num_tiles; ++j) {
            const int s = j % KV_STAGES;
            const int page = page_next;
            page_next = page_of_tile(j + 1);
            int ok = 1;
            if (lane == 0) ok = mbar_wait(kv_empty(s), ((j / KV_STAGES) & 1u) ^ 1u, abort_flag, p.status, 31) ? 1 : 0;
            if (!__shfl_sync(0xffffffffu, ok, 0)) break;
            const int tok = (tile0 + j) * KT + my_piece * piece_rows;
            const uint32_t copies = __popc(__ballot_sync(0xffffffffu, page >= 0));
            if (lane == 0) mbar_expect_tx(kv_full(s), copies * (uint32_t)piece_rows * 128u);
            __syncwarp();
            if (page >= 0) {
                const int row = ((my_kv * p.num_pages + page) * p.hkv + kvh) * p.page_size + tok % p.page_size;
                const uint32_t dst = smem_u32(kv_ring + s * S::STAGE) + my_kv * S::KV_TILE + my_half * (KT * 128) +
                                     my_piece * piece_rows * 128;
                tma_load_2d(dst, &kv_map, kv_full(s), my_half * 64, row);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_s = make_idesc(QM, KT);               // S = Q K^T: both operands K-major
            constexpr uint32_t idesc_o = make_idesc(QM, D, true);          // O = P V: V is MN-major (features contiguous)
            // the descriptors are made once (this one thread's instructions are what the tensor cores wait for
            // between products): a k step is an addition to them, in the descriptors' 16-byte units
            const uint64_t q_desc = make_sw128_desc(smem_u32(q_tile)), p_desc = make_sw128_desc(smem_u32(p_tile));
            static_assert(KV_STAGES == 2, "the descriptors below are picked for two stages");
            uint64_t k_desc[KV_STAGES], v_desc[KV_STAGES];
#pragma unroll
            for (int st = 0; st < KV_STAGES; ++st) {
                k_desc[st] = make_sw128_desc(smem_u32(kv_ring + st * S::STAGE));
                v_desc[st] = make_sw128_desc_mn(smem_u32(kv_ring + st * S::STAGE) + S::KV_TILE, KT * 128, 1024);
            }
            bool ok = mbar_wait(q_full, 0, abort_flag, p.status, 32);
            auto issue_s = [&](int j) {                                    // scores of tile j into buffer j % 2
                const int s = j % KV_STAGES, b = j & 1;
                if (!mbar_wait(kv_full(s), (j / KV_STAGES) & 1u, abort_flag, p.status, 33)) return false;
                if (!mbar_wait(s_empty(b), ((j >> 1) & 1u) ^ 1u, abort_flag, p.status, 34)) return false;
                tmem_fence_after();
                const uint64_t kd = s == 0 ? k_desc[0] : k_desc[KV_STAGES - 1];
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    const uint64_t off = (uint64_t)(((ks >> 2) * (QM * 128) + (ks & 3) * 32) >> 4);   // half, then 32 bytes a step
                    umma_bf16(tmem_base + b * KT, q_desc + off, kd + off, idesc_s, ks > 0 ? 1u : 0u);
                }
                umma_commit(s_full(b));
                return true;
            };
            if (ok && num_tiles > 0) ok = issue_s(0);
            for (int j = 0; j < num_tiles && ok; ++j) {
                if (j + 1 < num_tiles) ok = issue_s(j + 1);
                if (!ok) break;
                if (!mbar_wait(p_full, j & 1u, abort_flag, p.status, 35)) { ok = false; break; }
                tmem_fence_after();
                const int s = j % KV_STAGES;
                const uint64_t vd = s == 0 ? v_desc[0] : v_desc[KV_STAGES - 1];
#pragma unroll
                for (int ks = 0; ks < KT / 16; ++ks) {
                    // A: 16 keys = 32 bytes along the swizzled row of P; B: 16 key rows of V = 2048 bytes
                    const uint64_t aoff = (uint64_t)(((ks >> 2) * (QM * 128) + (ks & 3) * 32) >> 4);
                    umma_bf16(tmem_base + 2 * KT, p_desc + aoff, vd + (uint64_t)(ks * 128), idesc_o, ks > 0 ? 1u : 0u);
                }
                umma_commit(o_full);             // O_j is complete (and P and this stage have been read)
                umma_commit(kv_empty(s));
            }
        }
    } else {
        // ------------------------------------------------------------ softmax and output (warps 2..9)
        // Two warps share a quarter of the rows (their tensor-memory lanes) and split the columns:
        // `half` 0 owns keys 0..63 of every tile and output features 0..D/2-1, half 1 the rest.
        // The row maximum goes through shared memory once per tile; the row sums meet at the end.
        const int lane_group = warp & 3;
        const int half = (warp - 2) >> 2;
        const int r = lane_group * 32 + lane;                          // query row of the tile = tensor-memory lane
        const uint32_t lane_addr = tmem_base + ((uint32_t)(lane_group * 32) << 16);
        const int qpos = pos0 + r;
        const int etid = threadIdx.x - 64;                             // 0..255 among the softmax threads
        constexpr int KH = KT / 2, DH = D / 2;                         // this thread's share of keys and features
        float o[DH];
#pragma unroll
        for (int i = 0; i < DH; ++i) o[i] = 0.f;
        float m_run = -INFINITY, l_run = 0.f;
        bool ok = true;
        for (int j = 0; j < num_tiles && ok; ++j) {
            const int b = j & 1, s = j % KV_STAGES;
            const int tk0 = (tile0 + j) * KT;
            if (!mbar_wait(s_full(b), (j >> 1) & 1u, abort_flag, p.status, 36)) { ok = false; break; }
            tmem_fence_after();
            // Columns of this tile the row may see: kmin < column <= kmax (tile-local). A chunk of 32
            // columns inside that range needs no per-element test, one outside it no arithmetic at all.
            const int kmax = qpos - tk0;
            const int kmin = p.window > 0 ? qpos - p.window - tk0 : -1;
            // the same bounds for the warp's first and last row: the choice per chunk must be the
            // same for the whole warp, because tcgen05.ld is a warp-wide instruction
            const int wmax0 = pos0 + lane_group * 32 - tk0, wmax1 = wmax0 + 31;
            const int wmin0 = p.window > 0 ? wmax0 - p.window : -1, wmin1 = p.window > 0 ? wmax1 - p.window : -1;
            float v[32];
            // pass 1: the row maximum of the visible scores (raw; the scale is positive)
            float mx = -INFINITY;
#pragma unroll
            for (int cc = 0; cc < KH; cc += 32) {
                const int c = half * KH + cc;
                if (c > wmax1 || c + 31 <= wmin0) continue;
                tmem_ld32(lane_addr + b * KT + c, v);
                if (c + 31 <= wmax0 && c > wmin1) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) mx = fmaxf(mx, v[i]);
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) mx = fmaxf(mx, (c + i <= kmax && c + i > kmin) ? v[i] : -INFINITY);
                }
            }
            max_xch[b][half][r] = mx;
            asm volatile("bar.sync %0, 64;" ::"r"(1 + lane_group) : "memory");     // the two warps of this row quarter
            mx = fmaxf(mx, max_xch[b][half ^ 1][r]);
            const float m_new = fmaxf(m_run, mx * p.scale_log2);
            const float m_use = m_new == -INFINITY ? 0.f : m_new;
            const float corr = ex2(m_run - m_use);
            m_run = m_new;
            // fold the previous tile's product into the output row, rescaled for the new maximum;
            // this also means P and the O buffer of tensor memory are free again
            if (j > 0) {
                if (!mbar_wait(o_full, (j - 1) & 1u, abort_flag, p.status, 37)) { ok = false; break; }
                tmem_fence_after();
#pragma unroll
                for (int c = 0; c < DH; c += 32) {
                    tmem_ld32(lane_addr + 2 * KT + half * DH + c, v);
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[c + i] = (o[c + i] + v[i]) * corr;
                }
            }
            l_run *= corr;
            // value rows no query may see: zero them once the tile has landed (first and last tiles only)
            if (tk0 < lo || tk0 + KT > hi) {
                if (!mbar_wait(kv_full(s), (j / KV_STAGES) & 1u, abort_flag, p.status, 38)) { ok = false; break; }
                uint8_t* v_tile = kv_ring + s * S::STAGE + S::KV_TILE;
                for (int idx = etid; idx < KT * (D / 8); idx += 256) {
                    const int row = idx / (D / 8), chunk = idx % (D / 8);
                    if (row >= lo - tk0 && row < hi - tk0) continue;
                    *reinterpret_cast<uint4*>(v_tile + (chunk >> 3) * (KT * 128) + row * 128 + (((chunk & 7) ^ (row & 7)) << 4)) =
                        make_uint4(0, 0, 0, 0);
                }
            }
            // pass 2: probabilities, their sum, and P as the bfloat16 operand tile (row r, 128-byte swizzle)
#pragma unroll
            for (int cc = 0; cc < KH; cc += 32) {
                const int c = half * KH + cc;
                const bool none = c > wmax1 || c + 31 <= wmin0;
                if (none) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = 0.f;
                } else {
                    tmem_ld32(lane_addr + b * KT + c, v);
                    if (c + 31 <= wmax0 && c > wmin1) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            v[i] = ex2(fmaf(v[i], p.scale_log2, -m_use));
                            l_run += v[i];
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            v[i] = (c + i <= kmax && c + i > kmin) ? ex2(fmaf(v[i], p.scale_log2, -m_use)) : 0.f;
                            l_run += v[i];
                        }
                    }
                }
#pragma unroll
                for (int q8 = 0; q8 < 4; ++q8) {                     // 8 keys = one 16-byte chunk
                    const int chunk = ((c & 63) >> 3) + q8;
                    uint4 w;
                    w.x = pack2(v[q8 * 8], v[q8 * 8 + 1]);
                    w.y = pack2(v[q8 * 8 + 2], v[q8 * 8 + 3]);
                    w.z = pack2(v[q8 * 8 + 4], v[q8 * 8 + 5]);
                    w.w = pack2(v[q8 * 8 + 6], v[q8 * 8 + 7]);
                    *reinterpret_cast<uint4*>(p_tile + (c >> 6) * (QM * 128) + r * 128 + ((chunk ^ (r & 7)) << 4)) = w;
                }
            }
            tmem_fence_before();
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // P and the zeroed rows are read by the MMA
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(s_empty(b));
                mbar_arrive(p_full);
            }
        }
        if (ok && num_tiles > 0) {
            if (mbar_wait(o_full, (num_tiles - 1) & 1u, abort_flag, p.status, 39)) {
                tmem_fence_after();
                float v[32];
                sum_xch[half][r] = l_run;
                asm volatile("bar.sync %0, 64;" ::"r"(1 + lane_group) : "memory");
                const float l_all = l_run + sum_xch[half ^ 1][r];
                const float inv = l_all > 0.f ? 1.f / l_all : 0.f;
                __nv_bfloat16* dst = p.out + ((size_t)(row0 + r) * p.hq + head) * D + half * DH;
                const size_t part = (((size_t)blockIdx.y * p.splits + blockIdx.z) * p.hq + head) * QM + r;
                if (p.splits > 1 && half == 0 && r < nrows)
                    *reinterpret_cast<float2*>(p.part_ml + part * 2) = make_float2(m_run, l_all);
#pragma unroll
                for (int c = 0; c < DH; c += 32) {
                    tmem_ld32(lane_addr + 2 * KT + half * DH + c, v);
                    if (p.splits > 1) {
                        if (r < nrows) {
                            float4* po = reinterpret_cast<float4*>(p.part_o + part * D + half * DH + c);
#pragma unroll
                            for (int q4 = 0; q4 < 8; ++q4)
                                po[q4] = make_float4(o[c + q4 * 4] + v[q4 * 4], o[c + q4 * 4 + 1] + v[q4 * 4 + 1],
                                                     o[c + q4 * 4 + 2] + v[q4 * 4 + 2], o[c + q4 * 4 + 3] + v[q4 * 4 + 3]);
                        }
                    } else if (r < nrows) {
#pragma unroll
                        for (int q8 = 0; q8 < 4; ++q8) {
                            uint4 w;
                            w.x = pack2((o[c + q8 * 8] + v[q8 * 8]) * inv, (o[c + q8 * 8 + 1] + v[q8 * 8 + 1]) * inv);
                            w.y = pack2((o[c + q8 * 8 + 2] + v[q8 * 8 + 2]) * inv, (o[c + q8 * 8 + 3] + v[q8 * 8 + 3]) * inv);
                            w.z = pack2((o[c + q8 * 8 + 4] + v[q8 * 8 + 4]) * inv, (o[c + q8 * 8 + 5] + v[q8 * 8 + 5]) * inv);
                            w.w = pack2((o[c + q8 * 8 + 6] + v[q8 * 8 + 6]) * inv, (o[c + q8 * 8 + 7] + v[q8 * 8 + 7]) * inv);
                            *reinterpret_cast<uint4*>(dst + c + q8 * 8) = w;
                        }
                    }
                }
            }
        }
    }

    // ---------------------------------------------------------------- common exit
    tmem_fence_before();
    __syncthreads();
    if (warp == 1) {
        tmem_fence_after();
        tmem_dealloc(tmem_base, S::TMEM_COLS);
    }
}

// Merges the partial results of a split of the keys: one block per (query row of a tile, head), one thread
// per feature, the shares in key order. A share the tile has no keys in was not computed and is not read.
template <int D>
__global__ void prefill_merge_kernel(const PrefillParams p) {
    ti_grid_launch_dependents();
    ti_grid_wait();
    const int slot = blockIdx.x / QM, r = blockIdx.x % QM, head = blockIdx.y, d = threadIdx.x;
    const int4 td = reinterpret_cast<const int4*>(p.tiles)[p.halves ? slot >> 1 : slot];
    const int half_off = p.halves ? (slot & 1) * QM : 0;
    const int row0 = td.y + half_off, pos0 = td.w + half_off;
    const int nrows = min(td.z - half_off, QM);
    if (r >= nrows) return;
    const int hi = pos0 + nrows;
    const int lo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
    const int tile0 = lo / KT, tile1 = (hi + KT - 1) / KT, per = p.split_keys / KT;
    float m_run = -INFINITY, acc = 0.f, l_all = 0.f;
    for (int z = tile0 / per; z < p.splits && z * per < tile1; ++z) {
        const size_t part = (((size_t)slot * p.splits + z) * p.hq + head) * QM + r;
        const float2 ml = __ldcg(reinterpret_cast<const float2*>(p.part_ml + part * 2));
        const float ov = __ldcg(p.part_o + part * D + d);
        const float m_new = fmaxf(m_run, ml.x);
        const float m_use = m_new == -INFINITY ? 0.f : m_new;
        const float keep = ex2(m_run - m_use), f = ex2(ml.x - m_use);      // 0 while nothing has been merged yet
        acc = acc * keep + f * ov;
        l_all = l_all * keep + f * ml.y;
        m_run = m_new;
    }
    p.out[((size_t)(row0 + r) * p.hq + head) * D + d] = __float2bfloat16_rn(l_all > 0.f ? acc / l_all : 0.f);
}

}  // namespace

TI_API int ti_attention_prefill_tile_rows() { return QM; }

// Prefill attention on tcgen05. `tiles`: num_tiles int4 {request index in the step, first flat row,
// rows (<= 128), position of the first row}, every tile inside one request's portion. q [T, Hq, D],
// out [T, Hq * D], kv_cache [2, num_pages, Hkv, page_size, D]; page_size 16, 32 or a multiple of 64.
// With `halves` a tile entry has up to 256 rows (the form the two-tile kernel takes) and two CTAs take
// 128 rows each: for steps whose entries are too few to fill the machine with one CTA each.
// splits > 1: the keys are shared out too, split_keys (a multiple of 128) to a CTA, for few query tiles behind long
// prefixes; the partial results go through `scratch` (scratch_floats >= ti_attention_prefill_scratch_floats(...))
// and a second kernel merges them in key order.
TI_API long long ti_attention_prefill_scratch_floats(int num_tiles, int halves, int splits, int hq, int d) {
    return (long long)num_tiles * (halves ? 2 : 1) * splits * hq * QM * (d + 2);
}
TI_API int ti_attention_prefill_tc_bf16(void* out, const void* q, const void* kv_cache, const int* tiles, int num_tiles,
                                        int num_tokens, const int* block_table, int max_blocks, int hq, int hkv, int d,
                                        int page_size, int num_pages, float scale, int window, int halves, int splits,
                                        int split_keys, float* scratch, long long scratch_floats, int* status,
                                        cudaStream_t stream) {
    TI_REQUIRE(splits >= 1 && splits <= 65535, "attention_prefill_tc: %d shares of the keys", splits);
    TI_REQUIRE(splits == 1 || (split_keys > 0 && split_keys % KT == 0 && scratch != nullptr &&
                               scratch_floats >= ti_attention_prefill_scratch_floats(num_tiles, halves, splits, hq, d)),
               "attention_prefill_tc: a split of the keys needs shares of a multiple of %d keys and %lld floats of scratch",
               KT, ti_attention_prefill_scratch_floats(num_tiles, halves, splits, hq, d));
    TI_REQUIRE(d == 64 || d == 128, "attention_prefill_tc: head_dim %d is not 64 or 128", d);
    TI_REQUIRE(hq > 0 && hkv > 0 && hq % hkv == 0, "attention_prefill_tc: bad head counts");
    TI_REQUIRE(num_tiles <= 32767, "attention_prefill_tc: more than 32767 tiles in one step");
    TI_REQUIRE(page_size == 16 || page_size == 32 || page_size % 64 == 0, "attention_prefill_tc: page size %d", page_size);
    TI_REQUIRE(num_tiles >= 0 && num_tokens > 0, "attention_prefill_tc: bad sizes");
    if (num_tiles == 0) return 0;
    CUtensorMap q_map, kv_map;
    if (!ti_get_bf16_map(q, num_tokens, hq * d, QM, &q_map)) return -1;
    if (!ti_get_bf16_map(kv_cache, 2ll * num_pages * hkv * page_size, d, page_size < 64 ? page_size : 64, &kv_map)) return -1;
    PrefillParams p;
    p.out = (__nv_bfloat16*)out; p.tiles = tiles; p.block_table = block_table; p.max_blocks = max_blocks;
    p.hq = hq; p.hkv = hkv; p.page_size = page_size; p.num_pages = num_pages; p.window = window;
    p.scale_log2 = scale * 1.4426950408889634f; p.status = status; p.halves = halves ? 1 : 0;
    const int slots = halves ? 2 * num_tiles : num_tiles;
    p.splits = splits; p.split_keys = split_keys;
    p.part_o = scratch; p.part_ml = scratch ? scratch + (long long)slots * splits * hq * QM * d : nullptr;
    dim3 grid(hq, slots, splits);
    if (d == 128) {
        static bool once = false;
        if (!once) {
            cudaError_t e = cudaFuncSetAttribute(prefill_attention_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, PfSmem<128>::BYTES);
            TI_REQUIRE(e == cudaSuccess, "attention_prefill_tc: shared memory: %s", cudaGetErrorString(e));
            once = true;
        }
        ti_launch(prefill_attention_tc_kernel<128>, grid, PF_THREADS, PfSmem<128>::BYTES, stream, q_map, kv_map, p);
    } else {
        static bool once = false;
        if (!once) {
            cudaError_t e = cudaFuncSetAttribute(prefill_attention_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, PfSmem<64>::BYTES);
            TI_REQUIRE(e == cudaSuccess, "attention_prefill_tc: shared memory: %s", cudaGetErrorString(e));
            once = true;
        }
        ti_launch(prefill_attention_tc_kernel<64>, grid, PF_THREADS, PfSmem<64>::BYTES, stream, q_map, kv_map, p);
    }
    TI_CHECK_LAUNCH("attention_prefill_tc");
    if (splits > 1) {
        if (d == 128) ti_launch(prefill_merge_kernel<128>, dim3(slots * QM, hq), 128, 0, stream, p);
        else ti_launch(prefill_merge_kernel<64>, dim3(slots * QM, hq), 64, 0, stream, p);
        TI_CHECK_LAUNCH("attention_prefill_merge");
    }
    return 0;
}
