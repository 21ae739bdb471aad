// bfloat16 paged attention for single decoded tokens, head sizes 64 and 128: a split-KV kernel
// (FlashDecoding: tinyinfer/csrc/flash_decoding.cu:17-336 of the reference, here batched over requests
// in ONE launch, with the query heads of a kv head sharing one read of its keys and values).
//
// Keys and values come straight from the pages: a warp of its own issues TMA tile copies
// (64 keys x 64 features, 128-byte swizzle) into a 3-stage ring guarded by mbarriers; four warps
// consume them with ldmatrix + mma.sync.m16n8k16 (bf16 in, float32 out): a decoded token has at most
// 16 query rows per kv head, far too few for a 128-row tcgen05 tile, and the kernel is bound by HBM,
// not by the tensor pipe. Scores, running maximum (from -inf), sums and outputs are float32;
// probabilities are rounded to bfloat16 for the second product. Masked scores are assigned -inf
// (never added), and value rows that no query of the CTA may see are zeroed in shared memory, so
// stale or unwritten pages cannot leak NaNs.
//
// The work is shared out evenly: all key tiles of the step, in the order (request, kv head, tile), are
// cut into as many equal runs as there are CTAs (at least four tiles, 256 keys, a run), so that every
// CTA streams the same number of bytes whatever the mix of context lengths; a run that crosses from one
// (request, kv head) into the next makes a part of each. A pair that lies inside one run is finished
// there. Of a pair that several CTAs share, each writes its partial result (unnormalised output, maximum,
// sum) to float32 scratch and a second kernel merges the pair's parts, in key order. Where the cuts fall
// depends on the batch, so a request's result depends on what else is in the batch by float32 rounding
// of the merge, and by nothing else.
// (Prompt portions: attention_prefill_tcgen05.cu.)
#include "sm100_ptx.cuh"

namespace {

constexpr int TK = 64;            // keys per tile
constexpr int MIN_RUN_TILES = 4;  // fewest key tiles of a CTA's run: a part pays about 52 keys' worth of time beyond its keys
constexpr int STAGES = 3;        // stages of the ring of key/value tiles (decode with one CTA an SM: twice as many)
constexpr int CONSUMER_THREADS = 128;
constexpr int THREADS = CONSUMER_THREADS + 32;

struct AttnParams {
    __nv_bfloat16* out;            // [T, Hq * D]
    const __nv_bfloat16* q;        // [T, Hq, D]
    float* part_o;                 // [part slots][query heads of a kv head][D]
    float* part_ml;                // [part slots][query heads of a kv head][2]
    const int* rows;               // flat token rows of the decoded tokens
    const int* positions;
    const int* token_seq;
    const int* block_table;
    int max_blocks, hq, hkv, page_size, num_pages, window, num_rows;
    int num_ctas;                  // CTAs of the split kernel: the runs are cut for this many
    float scale_log2;              // softmax scale times log2(e)
    int* status;
};

__device__ __forceinline__ void ldmatrix_x4(uint32_t* r, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t* r, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
// Byte offset of (row, 16-byte chunk) inside a tile of 64-feature halves, each [TK][128 B] swizzled.
__device__ __forceinline__ uint32_t tile_off(int row, int chunk) {
    return (uint32_t)((chunk >> 3) * (TK * 128) + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
}

template <int D>
struct Smem {
    static constexpr int HALVES = D / 64;
    static constexpr int TILE_BYTES = HALVES * TK * 128;      // keys OR values of one tile
    static constexpr int STAGE_BYTES = 2 * TILE_BYTES;
    // 1 KB to align the ring, the ring, its barriers, and the merge buffer [4 warps][query heads of a kv head <= 16]
    // [D + 2] floats; slim: a warp finishes a quarter of the features and gets the other three warps' partials of
    // them, [4 warps][3][query heads][D / 4 + 2] floats
    static int decode_bytes(int group, int stages = STAGES, bool slim = false) {
        return 1024 + stages * STAGE_BYTES + 128 + (slim ? 4 * 3 * group * (D / 4 + 2) * 4 : 4 * group * (D + 2) * 4);
    }
};

// Issues the copies of tile `t` (keys t*TK .. t*TK+63 of the request) into a stage. Pieces whose
// page the request does not hold (never written, or given back by a window) are skipped.
template <int D>
__device__ __forceinline__ void load_tile(const CUtensorMap* map, const AttnParams& p, const int* table, int kvh,
                                          int t, uint32_t stage_addr, uint32_t bar) {
    using S = Smem<D>;
    const int piece_rows = p.page_size < TK ? p.page_size : TK;
    const int pieces = TK / piece_rows;
    int pages[4];                                   // page_size >= 16, so at most four pieces
    uint32_t bytes = 0;
    for (int i = 0; i < pieces; ++i) {
        const int tok = t * TK + i * piece_rows;
        const int logical = tok / p.page_size;
        int page = logical < p.max_blocks ? table[logical] : -1;
        if (page >= p.num_pages) page = -1;
        pages[i] = page;
        if (page >= 0) bytes += (uint32_t)piece_rows * 128u * S::HALVES * 2u;
    }
    mbar_expect_tx(bar, bytes);
    for (int i = 0; i < pieces; ++i) {
        if (pages[i] < 0) continue;
        const int tok = t * TK + i * piece_rows;
        const int off = tok % p.page_size;
        const int krow = (pages[i] * p.hkv + kvh) * p.page_size + off;
        const int vrow = ((p.num_pages + pages[i]) * p.hkv + kvh) * p.page_size + off;
#pragma unroll
        for (int hh = 0; hh < S::HALVES; ++hh) {
            const uint32_t dst = stage_addr + hh * (TK * 128) + i * piece_rows * 128;
            tma_load_2d(dst, map, bar, hh * 64, krow);
            tma_load_2d(dst + S::TILE_BYTES, map, bar, hh * 64, vrow);
        }
    }
}

// Zeroes the value rows of a tile outside [keep_lo, keep_hi) (tile-local key indices): no query of
// this CTA may see them and what the stage holds there may be stale or unwritten. Called by the
// `nthreads` threads that will read the tile, `tid` being the caller's index among them.
template <int D>
__device__ __forceinline__ void zero_value_rows(uint8_t* v_tile, int keep_lo, int keep_hi, int tid, int nthreads,
                                                int row_begin, int row_end) {
    constexpr int CHUNKS = D / 8;
    for (int idx = tid; idx < (row_end - row_begin) * CHUNKS; idx += nthreads) {
        const int row = row_begin + idx / CHUNKS, chunk = idx % CHUNKS;
        if (row >= keep_lo && row < keep_hi) continue;
        *reinterpret_cast<uint4*>(v_tile + tile_off(row, chunk)) = make_uint4(0, 0, 0, 0);
    }
}

// ------------------------------------------------------------------------------------ decode
// Key tiles a decoded row has to read: those from the one its window (if any) begins in to its last.
struct RowTiles { int n, lo_tile, lo, ctx, row; };
__device__ __forceinline__ RowTiles row_tiles(const AttnParams& p, int r) {
    RowTiles t;
    t.row = p.rows[r];
    t.ctx = p.positions[t.row] + 1;
    t.lo = p.window > 0 ? max(0, t.ctx - p.window) : 0;
    t.lo_tile = t.lo / TK;
    t.n = (t.ctx + TK - 1) / TK - t.lo_tile;
    return t;
}
// Tiles per run for `total` tiles (all kv heads) on `ctas` CTAs. (The tiles of a step are counted in 32 bits: a
// step with 2^31 of them, 137 G keys, is refused with a status word. Divisions of 64-bit counts in every part's
// walk were a measurable share of a short kernel.)
__device__ __forceinline__ int run_tiles(int total, int ctas) {
    const int per = (int)(((unsigned)total + (unsigned)ctas - 1u) / (unsigned)ctas);
    return per < MIN_RUN_TILES ? MIN_RUN_TILES : per;
}
// All tiles of the step for all kv heads, or -1 if they cannot be counted in 32 bits.
__device__ __forceinline__ int all_tiles_of(int per_head, int hkv) {
    const long long all = (long long)per_head * hkv;
    return all < (1ll << 31) - 65536 ? (int)all : -1;
}
// Sum over the block of `mine` (all of it) and over the threads before this one. NT threads, all call it.
template <int NT>
__device__ __forceinline__ void block_scan(int mine, int* warp_sums /* [NT / 32] shared */, int& before, int& total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int incl = mine;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += v;
    }
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    before = incl - mine;
    total = 0;
#pragma unroll
    for (int w = 0; w < NT / 32; ++w) {
        if (w < warp) before += warp_sums[w];
        total += warp_sums[w];
    }
}

// A CTA's walk over the parts of its run: the loading warp and the consumers step through the same parts.
struct Part { int r, row, kvh, tile0, tile1, tile_new, k_begin, k_end, slot, pair, cta0, cta1; };   // tile_new: the tile of the row's own token; cta0..cta1: the CTAs whose runs hold the pair's tiles
struct RunWalk {
    int cur, end, base;            // global tile indices; base: that of (row r, kv head 0, its first tile)
    int r, per;
    RowTiles rt;
    __device__ __forceinline__ bool next(const AttnParams& p, Part& part) {
        if (cur >= end) return false;
        while (cur - base >= p.hkv * rt.n) {                   // on to the next decoded row
            base += p.hkv * rt.n;
            rt = row_tiles(p, ++r);
        }
        const int off = cur - base;
        const int kvh = off / rt.n, tl = off % rt.n;
        const int cnt = min(rt.n - tl, end - cur);
        part.r = r; part.row = rt.row; part.kvh = kvh;
        part.tile0 = rt.lo_tile + tl; part.tile1 = part.tile0 + cnt;
        part.tile_new = (rt.ctx - 1) / TK;
        part.k_begin = max(rt.lo, part.tile0 * TK);
        part.k_end = min(rt.ctx, part.tile1 * TK);
        part.pair = r * p.hkv + kvh;
        part.slot = (int)blockIdx.x + part.pair;               // CTA and pair both only grow along the walk: no two parts share a slot
        const int first = base + kvh * rt.n;                   // the pair's first tile
        part.cta0 = first / per;
        part.cta1 = (first + rt.n - 1) / per;
        cur += cnt;
        return true;
    }
};

// Persistent: every CTA takes one run of key tiles (see the head of the file) and walks over its parts;
// the loading warp runs ahead into the next part while the consumers merge and write the current one,
// so HBM does not idle at part boundaries. `rows`, `positions`, `token_seq`, the block tables and every key
// tile but a row's last are read BEFORE the wait for the kernels ahead in the stream: they are inputs of the
// step or older than it, never written by the kernels that lead up to this one.
// NS: stages of the ring. Three with two or more CTAs an SM; where the merge buffer of many query heads a kv
// head leaves room for one CTA only, six, so that an SM has as many bytes on their way as with two CTAs.
// SLIM: the merge of the four warps at the end of a part through a buffer of three quarters the size, which lets
// two CTAs of 8 or 9 query heads a kv head (head size 128) share an SM (32 requests x 8,192 keys, 64 query heads
// over 8: 193 -> 170 us); with fewer query heads, where two CTAs fit anyway, the whole buffer's merge is shorter
// (8 x 4,096 keys, 32 over 8: 26.9 us against 30.0).
template <int D, int NS, bool SLIM>
__global__ void __launch_bounds__(THREADS) decode_attention_kernel(const __grid_constant__ CUtensorMap kv_map,
                                                                   const AttnParams p) {
    using S = Smem<D>;
    constexpr int STAGES = NS;                             // hides the file's constant in this kernel
    constexpr int LDW = D + 2;                             // whole merge buffer row: D outputs, maximum, sum
    constexpr int OWN = D / 4, NB_OWN = OWN / 8;           // slim: features (and 8-wide blocks of them) a warp finishes
    constexpr int LD = OWN + 2;                            // slim merge buffer row: a warp's partial of OWN features, its maximum, its sum
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * S::STAGE_BYTES);
    float* mbuf = reinterpret_cast<float*>(smem + STAGES * S::STAGE_BYTES + 128);   // [4 warps][group][LDW], slim: [4 owners][3 others][group][LD]
    const uint32_t bar0 = smem_u32(bars);
    __shared__ int abort_sh;
    __shared__ int warp_sums[THREADS / 32];
    __shared__ int start_sh[2];                            // first row of this CTA's run, tiles (per kv head) before it
    volatile int* abort_flag = &abort_sh;

    ti_grid_launch_dependents();
    const int group = p.hq / p.hkv;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        abort_sh = 0;
        for (int s = 0; s < STAGES; ++s) { mbar_init(bar0 + 8u * s, 1); mbar_init(bar0 + 8u * (STAGES + s), 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // ---- this CTA's run: every thread adds up the tiles of a stretch of rows, a scan gives the total and
    // what lies before each stretch, and the thread whose stretch holds the run's first tile says where
    const int stretch = (p.num_rows + THREADS - 1) / THREADS;
    const int my_r0 = min(p.num_rows, (int)threadIdx.x * stretch), my_r1 = min(p.num_rows, my_r0 + stretch);
    int mine = 0;
    for (int r = my_r0; r < my_r1; ++r) mine += row_tiles(p, r).n;
    int before, total;
    block_scan<THREADS>(mine, warp_sums, before, total);
    const int all_tiles = all_tiles_of(total, p.hkv);
    if (all_tiles < 0) {                                   // more tiles than 32 bits count: refused, loudly
        if (threadIdx.x == 0 && p.status) atomicExch(p.status, 23);
        return;
    }
    const int per = run_tiles(all_tiles, p.num_ctas);
    const long long run_begin_ll = (long long)blockIdx.x * per;
    const int run_begin = run_begin_ll < all_tiles ? (int)run_begin_ll : all_tiles;
    const int run_end = min(all_tiles, run_begin + per);
    if (run_begin < all_tiles && run_begin >= before * p.hkv && run_begin < (before + mine) * p.hkv) {
        int acc = before;
        for (int r = my_r0; r < my_r1; ++r) {
            const int n = row_tiles(p, r).n;
            if (run_begin < (acc + n) * p.hkv) { start_sh[0] = r; start_sh[1] = acc; break; }
            acc += n;
        }
    }
    __syncthreads();
    if (run_begin >= all_tiles) return;                    // more CTAs than runs
    RunWalk walk;
    walk.cur = run_begin; walk.end = run_end; walk.r = start_sh[0]; walk.per = per;
    walk.base = start_sh[1] * p.hkv;
    walk.rt = row_tiles(p, walk.r);

    if (warp == 4) {
        // The kernel just before wrote this step's keys and values: for a decoded row that is its own token, in
        // the row's last tile. Every other tile is older than the step, so the ring is filled with such tiles
        // BEFORE the wait for that kernel (block tables and token_seq are inputs of the step, like positions),
        // and HBM is busy while the kernels ahead drain.
        if (lane == 0) {
            uint32_t n = 0;
            bool ok = true, waited = false;
            Part it;
            while (ok && walk.next(p, it)) {
                const int* table = p.block_table + (size_t)p.token_seq[it.row] * p.max_blocks;
                for (int t = it.tile0; t < it.tile1; ++t, ++n) {
                    if (!waited && (n >= STAGES || t == it.tile_new)) { ti_grid_wait(); waited = true; }
                    const int s = n % STAGES;
                    if (!mbar_wait(bar0 + 8u * (STAGES + s), ((n / STAGES) & 1u) ^ 1u, abort_flag, p.status, 21)) { ok = false; break; }
                    load_tile<D>(&kv_map, p, table, it.kvh, t, smem_u32(smem + s * S::STAGE_BYTES), bar0 + 8u * s);
                }
            }
        }
        return;
    }

    // ---- consumers: the 16 rows of the MMA are the query heads of one kv head (rows >= group are zero)
    ti_grid_wait();                                        // q comes from the kernel before
    const int g = lane >> 2, c = (lane & 3) * 2;
    const int id = lane >> 3, rr = lane & 7;
    uint32_t n = 0;
    Part item;
    while (walk.next(p, item)) {
        uint32_t qa[D / 16][4];
        {
            const __nv_bfloat16* q0 = p.q + ((size_t)item.row * p.hq + (size_t)item.kvh * group) * D;
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                qa[ks][0] = g < group ? *reinterpret_cast<const uint32_t*>(q0 + (size_t)g * D + ks * 16 + c) : 0u;
                qa[ks][1] = g + 8 < group ? *reinterpret_cast<const uint32_t*>(q0 + (size_t)(g + 8) * D + ks * 16 + c) : 0u;
                qa[ks][2] = g < group ? *reinterpret_cast<const uint32_t*>(q0 + (size_t)g * D + ks * 16 + c + 8) : 0u;
                qa[ks][3] = g + 8 < group ? *reinterpret_cast<const uint32_t*>(q0 + (size_t)(g + 8) * D + ks * 16 + c + 8) : 0u;
            }
        }
        float o[D / 8][4];
#pragma unroll
        for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
        float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
        const int k_begin = item.k_begin, k_end = item.k_end;

        for (int t = item.tile0; t < item.tile1; ++t, ++n) {
            const int s = n % STAGES;
            if (!mbar_wait(bar0 + 8u * s, (n / STAGES) & 1u, abort_flag, p.status, 22)) return;
            uint8_t* k_tile = smem + s * S::STAGE_BYTES;
            uint8_t* v_tile = k_tile + S::TILE_BYTES;
            const int w0 = warp * 16;                         // this warp's 16 keys of the tile
            const int tok0 = t * TK + w0;
            if (tok0 < k_end && tok0 + 16 > k_begin) {
                float sc[2][4] = {};
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    uint32_t b[4];
                    const int krow = w0 + (id >> 1) * 8 + rr;
                    ldmatrix_x4(b, smem_u32(k_tile) + tile_off(krow, ks * 2 + (id & 1)));
                    mma_bf16(sc[0], qa[ks], b[0], b[1]);
                    mma_bf16(sc[1], qa[ks], b[2], b[3]);
                }
                float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
                for (int nb = 0; nb < 2; ++nb)
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int tok = tok0 + nb * 8 + c + (j & 1);
                        const float v = (tok >= k_begin && tok < k_end) ? sc[nb][j] * p.scale_log2 : -INFINITY;
                        sc[nb][j] = v;
                        mx[j >> 1] = fmaxf(mx[j >> 1], v);
                    }
                float corr[2], m_use[2];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
                    mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
                    const float m_new = fmaxf(m_run[h], mx[h]);
                    m_use[h] = m_new == -INFINITY ? 0.f : m_new;
                    corr[h] = exp2f(m_run[h] - m_use[h]);
                    m_run[h] = m_new;
                    l_run[h] *= corr[h];
                }
#pragma unroll
                for (int nb = 0; nb < 2; ++nb)
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float pv = exp2f(sc[nb][j] - m_use[j >> 1]);
                        sc[nb][j] = pv;
                        l_run[j >> 1] += pv;
                    }
                uint32_t pa[4] = {pack_bf16(sc[0][0], sc[0][1]), pack_bf16(sc[0][2], sc[0][3]),
                                  pack_bf16(sc[1][0], sc[1][1]), pack_bf16(sc[1][2], sc[1][3])};
                if (tok0 < k_begin || tok0 + 16 > k_end) {    // warp-local: only this warp reads these rows
                    zero_value_rows<D>(v_tile, k_begin - t * TK, k_end - t * TK, lane, 32, w0, w0 + 16);
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // a later TMA copy overwrites these rows
                    __syncwarp();
                }
#pragma unroll
                for (int nb = 0; nb < D / 8; nb += 2) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        o[nb][j] *= corr[j >> 1];
                        o[nb + 1][j] *= corr[j >> 1];
                    }
                    uint32_t b[4];
                    const int vrow = w0 + (id & 1) * 8 + rr;
                    ldmatrix_x4_trans(b, smem_u32(v_tile) + tile_off(vrow, nb + (id >> 1)));
                    mma_bf16(o[nb], pa, b[0], b[1]);
                    mma_bf16(o[nb + 1], pa, b[2], b[3]);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar0 + 8u * (STAGES + s));
        }

        if constexpr (!SLIM) {
            // ---- merge the four warps (each saw a quarter of the keys) and write the part's partial.
            // Only the rows that are real query heads travel through shared memory.
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
                l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");       // the previous item's merge buffer has been read
#pragma unroll
            for (int nb = 0; nb < D / 8; ++nb) {
                float* base = mbuf + ((size_t)warp * group) * LDW + nb * 8 + c;
                if (g < group) { base[(size_t)g * LDW] = o[nb][0]; base[(size_t)g * LDW + 1] = o[nb][1]; }
                if (g + 8 < group) { base[(size_t)(g + 8) * LDW] = o[nb][2]; base[(size_t)(g + 8) * LDW + 1] = o[nb][3]; }
            }
            if ((lane & 3) == 0) {
                if (g < group) {
                    mbuf[((size_t)warp * group + g) * LDW + D] = m_run[0];
                    mbuf[((size_t)warp * group + g) * LDW + D + 1] = l_run[0];
                }
                if (g + 8 < group) {
                    mbuf[((size_t)warp * group + g + 8) * LDW + D] = m_run[1];
                    mbuf[((size_t)warp * group + g + 8) * LDW + D + 1] = l_run[1];
                }
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            for (int idx = threadIdx.x; idx < group * D; idx += CONSUMER_THREADS) {
                const int hrow = idx / D, d = idx % D;
                float mw[4], m_all = -INFINITY;
#pragma unroll
                for (int w4 = 0; w4 < 4; ++w4) { mw[w4] = mbuf[((size_t)w4 * group + hrow) * LDW + D]; m_all = fmaxf(m_all, mw[w4]); }
                const float m_use = m_all == -INFINITY ? 0.f : m_all;
                float acc = 0.f, l_all = 0.f;
#pragma unroll
                for (int w4 = 0; w4 < 4; ++w4) {
                    const float f = exp2f(mw[w4] - m_use);
                    acc += f * mbuf[((size_t)w4 * group + hrow) * LDW + d];
                    l_all += f * mbuf[((size_t)w4 * group + hrow) * LDW + D + 1];
                }
                if (item.cta0 == item.cta1) {                      // the pair lies inside this run: this is its result
                    p.out[((size_t)item.row * p.hq + (size_t)item.kvh * group + hrow) * D + d] =
                        __float2bfloat16_rn(l_all > 0.f ? acc / l_all : 0.f);
                } else {
                    const size_t slot = (size_t)item.slot * group + hrow;
                    __stcg(p.part_o + slot * D + d, acc);
                    if (d == 0) __stcg(reinterpret_cast<float2*>(p.part_ml + slot * 2), make_float2(m_all, l_all));
                }
            }
        } else {
        // ---- merge the four warps (each saw a quarter of the keys) and write the part's partial: warp w
        // finishes features [w OWN, (w + 1) OWN) and gets the other warps' partials of them through shared
        // memory, in the layout of the MMA's accumulator (a lane reads what it would hold itself). Only the
        // rows that are real query heads travel. The four partials are added in the order of the warps.
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
            l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");       // the previous item's merge buffer has been read
#pragma unroll
        for (int nb = 0; nb < D / 8; ++nb) {
            const int owner = nb / NB_OWN;
            if (owner == warp) continue;
            const int from = warp < owner ? warp : warp - 1;   // this warp's place among the owner's three others
            float* base = mbuf + ((size_t)(owner * 3 + from) * group) * LD + (nb % NB_OWN) * 8 + c;
            if (g < group) { base[(size_t)g * LD] = o[nb][0]; base[(size_t)g * LD + 1] = o[nb][1]; }
            if (g + 8 < group) { base[(size_t)(g + 8) * LD] = o[nb][2]; base[(size_t)(g + 8) * LD + 1] = o[nb][3]; }
        }
        if ((lane & 3) == 0) {
#pragma unroll
            for (int owner = 0; owner < 4; ++owner) {
                if (owner == warp) continue;
                const int from = warp < owner ? warp : warp - 1;
                float* ml = mbuf + ((size_t)(owner * 3 + from) * group) * LD + OWN;
                if (g < group) { ml[(size_t)g * LD] = m_run[0]; ml[(size_t)g * LD + 1] = l_run[0]; }
                if (g + 8 < group) { ml[(size_t)(g + 8) * LD] = m_run[1]; ml[(size_t)(g + 8) * LD + 1] = l_run[1]; }
            }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int hrow = g + 8 * h;
            if (hrow >= group) continue;
            // the four warps' maxima and sums, in the order of the warps (this warp's own from its registers)
            const float* others = mbuf + ((size_t)(warp * 3) * group + hrow) * LD;
            float mw[4], lw[4], m_all = -INFINITY;
#pragma unroll
            for (int w4 = 0; w4 < 4; ++w4) {
                const int from = w4 < warp ? w4 : w4 - 1;
                mw[w4] = w4 == warp ? m_run[h] : others[(size_t)from * group * LD + OWN];
                lw[w4] = w4 == warp ? l_run[h] : others[(size_t)from * group * LD + OWN + 1];
                m_all = fmaxf(m_all, mw[w4]);
            }
            const float m_use = m_all == -INFINITY ? 0.f : m_all;
            float f[4], l_all = 0.f;
#pragma unroll
            for (int w4 = 0; w4 < 4; ++w4) { f[w4] = exp2f(mw[w4] - m_use); l_all += f[w4] * lw[w4]; }
            const float inv = l_all > 0.f ? 1.f / l_all : 0.f;
#pragma unroll
            for (int nb = 0; nb < D / 8; ++nb) {               // every block, so that the accumulator's index is a constant
                if (nb / NB_OWN != warp) continue;
                const int nbo = nb % NB_OWN, d = nb * 8 + c;
                float a0 = 0.f, a1 = 0.f;
#pragma unroll
                for (int w4 = 0; w4 < 4; ++w4) {
                    const int from = w4 < warp ? w4 : w4 - 1;
                    const float x0 = w4 == warp ? o[nb][2 * h] : others[(size_t)from * group * LD + nbo * 8 + c];
                    const float x1 = w4 == warp ? o[nb][2 * h + 1] : others[(size_t)from * group * LD + nbo * 8 + c + 1];
                    a0 += f[w4] * x0;
                    a1 += f[w4] * x1;
                }
                if (item.cta0 == item.cta1) {                  // the pair lies inside this run: this is its result
                    *reinterpret_cast<__nv_bfloat162*>(p.out + ((size_t)item.row * p.hq + (size_t)item.kvh * group + hrow) * D + d) =
                        __floats2bfloat162_rn(a0 * inv, a1 * inv);
                } else {
                    const size_t slot = (size_t)item.slot * group + hrow;
                    __stcg(reinterpret_cast<float2*>(p.part_o + slot * D + d), make_float2(a0, a1));
                }
            }
            if (item.cta0 != item.cta1 && warp == 0 && (lane & 3) == 0)
                __stcg(reinterpret_cast<float2*>(p.part_ml + ((size_t)item.slot * group + hrow) * 2), make_float2(m_all, l_all));
        }
        }   // SLIM
    }
}

// The pairs that several CTAs share: one block per (decode row, query head), one thread per feature, merges
// the pair's parts in key order (a pair that lay inside one run was finished there: its blocks leave at
// once). The block works out which CTAs' runs hold the pair the way the split kernel does, before it waits
// for that kernel. The partials of eight parts are requested together and folded into a running maximum,
// sum and output. (Merging inside the split kernel, by the CTA that counts itself in last, was slower by
// 3 to 5 us at 1 to 8 long requests: while the kernel streams, the release that publishes a CTA's
// partials waits microseconds for its stores.)
template <int D>
__global__ void decode_merge_kernel(const AttnParams p) {
    __shared__ int warp_sums[D / 32];
    ti_grid_launch_dependents();
    const int r = blockIdx.x, h = blockIdx.y, d = threadIdx.x;
    int mine = 0, mine_before = 0;
    for (int r2 = d; r2 < p.num_rows; r2 += D) {
        const int n = row_tiles(p, r2).n;
        mine += n;
        if (r2 < r) mine_before += n;
    }
    int skip, total, tiles_before;
    block_scan<D>(mine, warp_sums, skip, total);
    __syncthreads();
    block_scan<D>(mine_before, warp_sums, skip, tiles_before);
    const RowTiles rt = row_tiles(p, r);
    const int group = p.hq / p.hkv, kvh = h / group, hrow = h % group;
    const int all_tiles = all_tiles_of(total, p.hkv);
    if (all_tiles < 0) return;                             // the split kernel has said so
    const int per = run_tiles(all_tiles, p.num_ctas);
    const int first = tiles_before * p.hkv + kvh * rt.n;                                   // the pair's tiles, globally
    const int c0 = first / per, c1 = (first + rt.n - 1) / per;
    if (c0 == c1) return;
    const int pair = r * p.hkv + kvh;
    ti_grid_wait();
    float m_run = -INFINITY, acc = 0.f, l_all = 0.f;
    for (int cb = c0; cb <= c1; cb += 8) {
        float ms[8], ls[8], os[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const bool in = cb + j <= c1;
            const size_t slot = (size_t)(cb + j + pair) * group + hrow;
            const float2 ml = in ? __ldcg(reinterpret_cast<const float2*>(p.part_ml + slot * 2)) : make_float2(-INFINITY, 0.f);
            ms[j] = ml.x;
            ls[j] = ml.y;
            os[j] = in ? __ldcg(p.part_o + slot * D + d) : 0.f;
        }
        float m_new = m_run;
#pragma unroll
        for (int j = 0; j < 8; ++j) m_new = fmaxf(m_new, ms[j]);
        const float m_use = m_new == -INFINITY ? 0.f : m_new;
        const float keep = exp2f(m_run - m_use);          // 0 while nothing has been merged yet
        acc *= keep;
        l_all *= keep;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float f = exp2f(ms[j] - m_use);          // 0 for a part that is not there
            acc += f * os[j];
            l_all += f * ls[j];
        }
        m_run = m_new;
    }
    p.out[((size_t)rt.row * p.hq + h) * D + d] = __float2bfloat16_rn(l_all > 0.f ? acc / l_all : 0.f);
}

template <typename K>
int set_smem(K kernel, int bytes, const char* name) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) { ti_set_error("%s: cannot get %d bytes of shared memory: %s", name, bytes, cudaGetErrorString(e)); return (int)e; }
    return 0;
}

int check_shape(int hq, int hkv, int d, int page_size, const char* name) {
    TI_REQUIRE(d == 64 || d == 128, "%s: head_dim %d is not 64 or 128", name, d);
    TI_REQUIRE(hq > 0 && hkv > 0 && hq % hkv == 0 && hq / hkv <= 16, "%s: %d query heads over %d kv heads (at most 16 per kv head)", name, hq, hkv);
    TI_REQUIRE(page_size >= 16 && ((page_size < TK && TK % page_size == 0) || page_size % TK == 0),
               "%s: page size %d must be 16, 32 or a multiple of 64", name, page_size);
    return 0;
}

}  // namespace

// 1 if the tensor-core attention kernels take these sizes.
TI_API int ti_attention_bf16_supported(int hq, int hkv, int d, int page_size) {
    return (d == 64 || d == 128) && hq > 0 && hkv > 0 && hq % hkv == 0 && hq / hkv <= 16 && page_size >= 16 &&
           ((page_size < TK && TK % page_size == 0) || page_size % TK == 0) ? 1 : 0;
}
namespace {
// Shared memory that decode_attention_kernel<128, 3, false> (which 0), <64, 3, false> (which 1), <128, 6, false> (which 2)
// or <128, 3, true> (which 3) was last allowed on the current device: the attribute is kept per device, so the record
// is too. nullptr: no current device.
int* configured_bytes(int which) {
    constexpr int MAX_DEVICES = 64;
    static int bytes[4][MAX_DEVICES] = {};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return nullptr;
    return &bytes[which][dev];
}

// The form of the decode kernel at head size 128: 0, three stages and the whole merge buffer, two CTAs an SM;
// 1, three stages and the slim buffer where that still lets two CTAs share an SM; 2, one CTA an SM with six stages.
int decode_form(int group) {
    if (Smem<128>::decode_bytes(group) <= 113 * 1024) return 0;
    if (Smem<128>::decode_bytes(group, STAGES, true) <= 113 * 1024) return 1;
    return 2;
}
// CTAs of the decode kernel that run side by side.
int decode_slots(int d, int group) {
    if (d == 128) return ti_sm_count() * (decode_form(group) == 2 ? 1 : 2);
    const int bytes = Smem<64>::decode_bytes(group);
    return ti_sm_count() * (bytes <= 56 * 1024 ? 4 : (bytes <= 75 * 1024 ? 3 : 2));
}
}  // namespace

// CTAs the decode kernel is launched with for num_rows requests of at most max_context keys each: those
// that run side by side, or fewer when there are not four key tiles for each. A function of its arguments
// alone, so a captured launch and the scratch sized for it agree.
TI_API int ti_attention_decode_ctas(int num_rows, int hq, int hkv, int d, int max_context, int window) {
    if (num_rows <= 0 || hkv <= 0 || hq % hkv != 0 || (d != 64 && d != 128) || max_context <= 0) return 1;
    const long long visible = window > 0 && window + TK < max_context ? window + TK : max_context;
    const long long runs = ((long long)num_rows * hkv * ((visible + TK - 1) / TK) + MIN_RUN_TILES - 1) / MIN_RUN_TILES;
    // Seven eighths of the CTAs that would run side by side, where two and more share an SM: every SM still streams,
    // and the free places let the CTAs of the kernel behind (the output projection) move in and ask for their
    // weights while this kernel drains (decode step, Qwen3-8B sizes: batch 8 3.84 -> 3.79 ms, batch 64 9.65 -> 9.46,
    // Qwen3-32B sizes 2 % as well; three quarters of them and fifteen sixteenths both gain less).
    const int side_by_side = decode_slots(d, hq / hkv);
    const int slots = side_by_side >= 2 * ti_sm_count() ? side_by_side * 7 / 8 : side_by_side;
    return (int)(runs < slots ? (runs < 1 ? 1 : runs) : slots);
}
// Floats of scratch that ti_attention_decode_bf16 needs for these arguments: a part slot per CTA and per
// (request, kv head), each the query heads of a kv head times head_dim + 2.
TI_API long long ti_attention_decode_scratch_floats(int num_rows, int hq, int hkv, int d, int max_context, int window) {
    if (hkv <= 0) return 0;
    const long long slots = (long long)ti_attention_decode_ctas(num_rows, hq, hkv, d, max_context, window) + (long long)num_rows * hkv;
    return slots * (hq / hkv) * (d + 2);
}

// Decode: `rows` lists the flat rows of the step whose request brings exactly one token. `scratch`: float32,
// scratch_floats >= ti_attention_decode_scratch_floats(same arguments), else the call is refused. max_context:
// an upper bound of the rows' contexts (it only sizes the launch: a longer context is computed all the same,
// on the CTAs there are). `rows`, `positions`, `token_seq`, `block_table` and the keys and values of all
// positions before each row's own are read before the kernels wait for the work ahead of them in the stream:
// they must be complete when the call is made, not results of the kernels launched just before (those may
// write q and the keys and values at the rows' own positions). Calls that share the scratch must not overlap.
TI_API int ti_attention_decode_bf16(void* out, const void* q, const void* kv_cache, float* scratch, long long scratch_floats,
                                    const int* rows, int num_rows, const int* positions, const int* token_seq,
                                    const int* block_table, int max_blocks, int hq, int hkv, int d, int page_size,
                                    int num_pages, float scale, int window, int max_context, int* status,
                                    cudaStream_t stream) {
    if (check_shape(hq, hkv, d, page_size, "attention_decode")) return -1;
    TI_REQUIRE(num_rows >= 0 && num_rows <= 65535 && max_context > 0, "attention_decode: bad sizes");
    if (num_rows == 0) return 0;
    const int group = hq / hkv;
    const int ctas = ti_attention_decode_ctas(num_rows, hq, hkv, d, max_context, window);
    const long long slots = (long long)ctas + (long long)num_rows * hkv;
    TI_REQUIRE(slots * group * (d + 2) <= scratch_floats,
               "attention_decode: %d rows x %d kv heads on %d CTAs need %lld floats of scratch, %lld given",
               num_rows, hkv, ctas, slots * group * (d + 2), scratch_floats);
    CUtensorMap map;
    if (!ti_get_bf16_map(kv_cache, 2ll * num_pages * hkv * page_size, d, page_size < TK ? page_size : TK, &map)) return -1;
    AttnParams p;
    p.out = (__nv_bfloat16*)out; p.q = (const __nv_bfloat16*)q;
    p.part_o = scratch; p.part_ml = scratch + slots * group * d;
    p.rows = rows; p.positions = positions; p.token_seq = token_seq; p.block_table = block_table;
    p.max_blocks = max_blocks; p.hq = hq; p.hkv = hkv; p.page_size = page_size; p.num_pages = num_pages;
    p.window = window; p.scale_log2 = scale * 1.4426950408889634f; p.status = status;
    p.num_rows = num_rows; p.num_ctas = ctas;
    if (d == 128 && decode_form(group) == 2) {
        const int bytes = Smem<128>::decode_bytes(group, 2 * STAGES);
        int* configured = configured_bytes(2);
        TI_REQUIRE(configured != nullptr, "attention_decode: no current device");
        if (*configured < bytes) { if (set_smem(decode_attention_kernel<128, 2 * STAGES, false>, bytes, "attention_decode")) return -1; *configured = bytes; }
        ti_launch(decode_attention_kernel<128, 2 * STAGES, false>, ctas, THREADS, bytes, stream, map, p);
        TI_CHECK_LAUNCH("attention_decode");
        ti_launch(decode_merge_kernel<128>, dim3(num_rows, hq), 128, 0, stream, p);
    } else if (d == 128 && decode_form(group) == 1) {
        const int bytes = Smem<128>::decode_bytes(group, STAGES, true);
        int* configured = configured_bytes(3);
        TI_REQUIRE(configured != nullptr, "attention_decode: no current device");
        if (*configured < bytes) { if (set_smem(decode_attention_kernel<128, STAGES, true>, bytes, "attention_decode")) return -1; *configured = bytes; }
        ti_launch(decode_attention_kernel<128, STAGES, true>, ctas, THREADS, bytes, stream, map, p);
        TI_CHECK_LAUNCH("attention_decode");
        ti_launch(decode_merge_kernel<128>, dim3(num_rows, hq), 128, 0, stream, p);
    } else if (d == 128) {
        const int bytes = Smem<128>::decode_bytes(group);
        int* configured = configured_bytes(0);
        TI_REQUIRE(configured != nullptr, "attention_decode: no current device");
        if (*configured < bytes) { if (set_smem(decode_attention_kernel<128, STAGES, false>, bytes, "attention_decode")) return -1; *configured = bytes; }
        ti_launch(decode_attention_kernel<128, STAGES, false>, ctas, THREADS, bytes, stream, map, p);
        TI_CHECK_LAUNCH("attention_decode");
        ti_launch(decode_merge_kernel<128>, dim3(num_rows, hq), 128, 0, stream, p);
    } else {
        const int bytes = Smem<64>::decode_bytes(group);
        int* configured = configured_bytes(1);
        TI_REQUIRE(configured != nullptr, "attention_decode: no current device");
        if (*configured < bytes) { if (set_smem(decode_attention_kernel<64, STAGES, false>, bytes, "attention_decode")) return -1; *configured = bytes; }
        ti_launch(decode_attention_kernel<64, STAGES, false>, ctas, THREADS, bytes, stream, map, p);
        TI_CHECK_LAUNCH("attention_decode");
        ti_launch(decode_merge_kernel<64>, dim3(num_rows, hq), 64, 0, stream, p);
    }
    TI_CHECK_LAUNCH("attention_decode_merge");
    return 0;
}

// ------------------------------------------------------------------------------------------------
// A decode-attention entry point that allocates nothing (declared in tinyinfer_b200_noalloc.h; the
// reference has no counterpart). It is ti_attention_decode_bf16 with the split partials kept in a
// fixed array inside this library instead of a buffer the caller allocates.
//
// Who needs it: code that runs where device allocation is off limits. A plugin called from inside
// another runtime's stream callback or graph-capture region, a serving loop that has handed all free
// memory to its cache and must not grow, or a host that forbids cudaMalloc after start-up for
// latency reasons can still call this: it issues kernel launches only.
//
// The array is `static __device__`: every GPU that loads this library holds TI_NOALLOC_SCRATCH_FLOATS
// floats (8 MB) of it until the process exits. In host code the array's name is only a stand-in, not
// a device address, so the first call on each device looks the address up with
// cudaGetSymbolAddress while that device is current and keeps it; the same call may make the driver
// load this library's code and array onto the device and raises the kernel's shared-memory limit there.
// That first call should be made at start-up, before any stream capture begins and before allocation
// becomes off limits. All calls on a device share the array: two calls that overlap on
// the GPU (different streams, no ordering) race on it. Nothing in it needs clearing between calls:
// every word the merge kernel reads was written by the split kernel of the same call.
constexpr long long TI_NOALLOC_SCRATCH_FLOATS = 2ll * 1024 * 1024;
static __device__ __align__(256) float g_noalloc_decode_scratch[TI_NOALLOC_SCRATCH_FLOATS];

TI_API long long ti_attention_decode_noalloc_capacity() { return TI_NOALLOC_SCRATCH_FLOATS; }

TI_API int ti_attention_decode_bf16_noalloc(void* out, const void* q, const void* kv_cache, const int* rows,
                                            int num_rows, const int* positions, const int* token_seq,
                                            const int* block_table, int max_blocks, int hq, int hkv, int d,
                                            int page_size, int num_pages, float scale, int window, int max_context,
                                            int* status, cudaStream_t stream) {
    constexpr int MAX_DEVICES = 64;
    static float* scratch_of_device[MAX_DEVICES] = {};
    TI_REQUIRE(num_rows >= 0 && max_context > 0 && hq > 0 && hkv > 0 && d > 0, "attention_decode_noalloc: bad sizes");
    const long long need = ti_attention_decode_scratch_floats(num_rows, hq, hkv, d, max_context, window);
    TI_REQUIRE(need <= TI_NOALLOC_SCRATCH_FLOATS,
               "attention_decode_noalloc: %d rows x %d kv heads x %d query heads each x (%d + 2) need %lld floats, the "
               "built-in scratch has %lld; use ti_attention_decode_bf16 with a buffer of your own",
               num_rows, hkv, hq / hkv, d, need, TI_NOALLOC_SCRATCH_FLOATS);
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    TI_REQUIRE(e == cudaSuccess && dev >= 0 && dev < MAX_DEVICES, "attention_decode_noalloc: no current device (%s)",
               cudaGetErrorString(e));
    if (scratch_of_device[dev] == nullptr) {
        float* ptr = nullptr;
        e = cudaGetSymbolAddress((void**)&ptr, g_noalloc_decode_scratch);
        TI_REQUIRE(e == cudaSuccess && ptr != nullptr, "attention_decode_noalloc: cudaGetSymbolAddress failed: %s",
                   cudaGetErrorString(e));
        scratch_of_device[dev] = ptr;
    }
    return ti_attention_decode_bf16(out, q, kv_cache, scratch_of_device[dev], TI_NOALLOC_SCRATCH_FLOATS, rows, num_rows,
                                    positions, token_seq, block_table, max_blocks, hq, hkv, d, page_size, num_pages,
                                    scale, window, max_context, status, stream);
}
