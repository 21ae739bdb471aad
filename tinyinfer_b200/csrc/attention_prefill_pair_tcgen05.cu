// Causal paged attention for portions of prompts on the tcgen05 tensor cores (bfloat16, head sizes 64
// and 128), two query tiles a CTA. One CTA owns up to 256 consecutive query tokens of one request and
// one query head, as tiles A (rows 0..127) and B (rows 128..255). Both read the same keys and values, so
// a key tile is fetched once for 256 queries, and while one tile's scores are in the softmax the
// tensor cores work on the other tile's products: the softmax of a tile costs about twice what its two
// products cost, and with one tile a CTA the tensor cores waited for it most of the time.
//
//   warp 0        TMA: both query tiles once, then K_j, V_j, K_j+1, ... tiles of 128 keys from the pages
//                 (through the block table) into a ring of four buffers;
//   warp 1        one thread issues the MMAs, whichever is ready next: S_X = Q_X K_j^T (128 x 128, fp32 in
//                 tensor memory) and O_X += P_X V_j, X = A, B. P is read from TENSOR MEMORY (it is written
//                 over the first 64 columns of S_X, two bfloat16 a column), V straight from the page layout
//                 as an MN-major operand. O_X accumulates in tensor memory over all key tiles;
//   warps 2..5    softmax of tile A, warps 6..9 of tile B: a thread owns a query row (its tensor-memory
//                 lane). The row's 128 scores come to registers in one trip (tcgen05.ld), are masked by
//                 assignment, and with a reference maximum m (from -inf) and the sum in float32 go back
//                 as P = 2^(s - m) in bfloat16 (tcgen05.st); nothing is exchanged between threads. The
//                 reference moves only when the row maximum has grown by more than 8 (a factor 256:
//                 bfloat16 and float32 hold that with ease); then, and only then, the rows of O_X in
//                 tensor memory are multiplied by 2^(m_old - m_new). At the end O_X / sum is stored.
//
// Clock stamps taken inside the kernel (8,192 tokens, a tile of 128 keys for both query tiles every 4,200
// cycles): a tile's softmax takes 2,200 cycles (scores in 90, maxima 280, exponentials 1,300 against 1,024
// at the rate of the XU pipe, P out and fenced 300), its two products 1,100 (1,024 at the tensor rate), and
// 400 go by before the issuing thread notices that P is there (a look at an mbarrier whose phase is not
// complete costs it that much). The two tiles run out of step by themselves. Those figures are from before
// the issuing thread's descriptors were made once instead of per MMA: its own instructions were a good part
// of the 1,100 (8,192 tokens 560 -> 530 us). Tried on this form, none
// faster: the issuing thread watching plain counters instead of mbarriers (the tiles then fall into step:
// both in their exponentials, then both waiting for products), P handed over in two halves, turns of the
// two tiles at the exponentials, an issuing warp per tile (polling, or sleeping on its barriers with its
// descriptors made once: 682 us; the products of two issuing threads share the tensor pipe, those of one take
// turns at it), sleeping between polls; and
// steps of 64 keys with two score buffers a query tile, so that the next scores are ready before a step's
// softmax ends (8,192 tokens 753 us against 560: the score products of 64 keys take in 192 bytes of
// operands a cycle from shared memory, which gives 128, and every step pays its hand-overs twice); and a
// share of the exponentials as a polynomial of degree 5 on the FMA pipe (every fourth: 547 us, every
// eighth: 576, every second: 690; the softmax warps are short of issue slots as much as of the XU pipe).
//
// Masked scores never reach an exponential (P is assigned 0 there), rows of V that no query of the CTA
// may see are zeroed in shared memory before the second product (pages never written or given back cannot
// leak NaNs through 0 * NaN), and every mbarrier wait is bounded (status word, abort flag, tensor memory
// freed on the common exit). The formulas are those of attention_prefill_tcgen05.cu; it replaces what the
// reference does with a gather on the host and a scalar FlashAttention kernel
// (tinyinfer/layers/attention.py:60-81, tinyinfer/csrc/flash_attention.cu:5-234).
#include "sm100_ptx.cuh"

namespace {

constexpr int QM = 128;              // query rows per tile = accumulator lanes
constexpr int KT = 128;              // keys per tile
constexpr int NBUF = 4;              // ring of key OR value tiles
constexpr int PP_THREADS = 320;      // TMA warp, MMA warp, four softmax warps per query tile (a thread a row)
constexpr float RESCALE_STEP = 8.f;  // the reference maximum follows the row maximum in steps of at least this (log2)

struct PairParams {
    __nv_bfloat16* out;              // [T, Hq * D]
    const int* tiles;                // int4 {request index, first flat row, rows (<= 256), first position}
    const int* block_table;
    int max_blocks, hq, hkv, page_size, num_pages, window;
    float scale_log2;
    int* status;
};

template <int D>
struct PpSmem {
    static constexpr int HALVES = D / 64;
    static constexpr int Q_BYTES = HALVES * QM * 128;          // one query tile
    static constexpr int KV_TILE = HALVES * KT * 128;          // keys OR values of a tile
    static constexpr int BYTES = 1024 + 2 * Q_BYTES + NBUF * KV_TILE + 256;
    // tensor memory: S_A at 0, S_B at 128 (P_X over columns 0..31 and 64..95 of S_X), O_A at 256, O_B at 256 + D
    static constexpr int TMEM_COLS = 512;
};

__device__ __forceinline__ float ex2(float x) {          // 2^x, flushing; inputs are finite or -inf
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
// D += A B with A in tensor memory (rows on the lanes, two bfloat16 of k a column), B from shared memory.
__device__ __forceinline__ void umma_bf16_tmem_a(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_ld32_nowait(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

template <int D>
__global__ void __launch_bounds__(PP_THREADS, 1)
prefill_attention_pair_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap kv_map,
                              const PairParams p) {
    using S = PpSmem<D>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* q_tiles = smem;                                   // A, then B
    uint8_t* kv_ring = smem + 2 * S::Q_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(kv_ring + NBUF * S::KV_TILE);
    const uint32_t bar0 = smem_u32(bars);
    // barriers: q_full, kv_full[NBUF], kv_empty[NBUF], s_full[2], p_full[2], o_full[2]
    const uint32_t q_full = bar0;
    auto kv_full = [&](int b) { return bar0 + 8u * (1 + b); };
    auto kv_empty = [&](int b) { return bar0 + 8u * (1 + NBUF + b); };
    auto s_full = [&](int x) { return bar0 + 8u * (1 + 2 * NBUF + x); };
    auto p_full = [&](int x) { return bar0 + 8u * (3 + 2 * NBUF + x); };
    auto o_full = [&](int x) { return bar0 + 8u * (5 + 2 * NBUF + x); };
    __shared__ uint32_t tmem_base_sh;
    __shared__ int abort_sh;
    volatile int* abort_flag = &abort_sh;

    ti_grid_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        abort_sh = 0;
        mbar_init(q_full, 1);
        for (int b = 0; b < NBUF; ++b) { mbar_init(kv_full(b), 1); mbar_init(kv_empty(b), 1); }
        for (int x = 0; x < 2; ++x) { mbar_init(s_full(x), 1); mbar_init(p_full(x), 4); mbar_init(o_full(x), 1); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(&tmem_base_sh, S::TMEM_COLS);
    tmem_fence_before();
    __syncthreads();
    tmem_fence_after();
    const uint32_t tmem_base = tmem_base_sh;
    ti_grid_wait();                                     // q, the pages and the tables come from earlier kernels

    // heads along x, tiles (longest key range first) along y: CTAs are handed out x first, so every head of
    // the longest tile starts before any shorter tile does, and the short ones fill in behind
    const int4 td = reinterpret_cast<const int4*>(p.tiles)[blockIdx.y];
    const int seq = td.x, row0 = td.y, nrows = td.z, pos0 = td.w;
    const int head = blockIdx.x;
    const int kvh = head / (p.hq / p.hkv);
    const int* table = p.block_table + (size_t)seq * p.max_blocks;
    // Key tiles each query tile needs: tile X holds rows X*128 .. of the block; its first query sees keys from
    // lo_x on, its last query keys below hi_x. The CTA walks over the union; a tile outside X's range is
    // not multiplied for X.
    int t0x[2], t1x[2];
#pragma unroll
    for (int x = 0; x < 2; ++x) {
        const int rows_x = min(QM, nrows - x * QM);
        if (rows_x <= 0) { t0x[x] = 0; t1x[x] = 0; continue; }
        const int first = pos0 + x * QM, hi_x = first + rows_x;
        const int lo_x = p.window > 0 ? max(0, first - p.window + 1) : 0;
        t0x[x] = lo_x / KT;
        t1x[x] = (hi_x + KT - 1) / KT;
    }
    const bool has_b = t1x[1] > t0x[1];
    const int tmin = has_b ? min(t0x[0], t0x[1]) : t0x[0], tmax = has_b ? max(t1x[0], t1x[1]) : t1x[0];
    const int lo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;   // first key any query of the CTA sees
    const int hi = pos0 + nrows;                                     // one past the last

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            mbar_expect_tx(q_full, (has_b ? 2u : 1u) * S::Q_BYTES);
#pragma unroll
            for (int hh = 0; hh < S::HALVES; ++hh) {
                tma_load_2d(smem_u32(q_tiles) + hh * (QM * 128), &q_map, q_full, head * D + hh * 64, row0);
                if (has_b)
                    tma_load_2d(smem_u32(q_tiles) + S::Q_BYTES + hh * (QM * 128), &q_map, q_full, head * D + hh * 64, row0 + QM);
            }
        }
        // Load number i is K of tile tmin + i / 2 (i even) or V of it (i odd), into buffer i % NBUF. A tile is
        // KT / piece_rows pieces (a piece lies in one page) x head halves: up to 16 copies, one a lane.
        const int piece_rows = p.page_size < 64 ? p.page_size : 64;
        const int num_copies = (KT / piece_rows) * S::HALVES;
        const int my_piece = lane / S::HALVES, my_half = lane % S::HALVES;
        const int num_loads = 2 * (tmax - tmin);
        for (int i = 0; i < num_loads; ++i) {
            const int j = tmin + (i >> 1), is_v = i & 1, b = i % NBUF;
            const int tok = j * KT + my_piece * piece_rows;
            const int logical = tok / p.page_size;
            int page = (lane < num_copies && logical < p.max_blocks) ? table[logical] : -1;
            if (page >= p.num_pages) page = -1;                     // never written, or given back by a window
            int ok = 1;
            if (lane == 0) ok = mbar_wait(kv_empty(b), ((i / NBUF) & 1u) ^ 1u, abort_flag, p.status, 41) ? 1 : 0;
            if (!__shfl_sync(0xffffffffu, ok, 0)) break;
            const uint32_t copies = __popc(__ballot_sync(0xffffffffu, page >= 0));
            if (lane == 0) mbar_expect_tx(kv_full(b), copies * (uint32_t)piece_rows * 128u);
            __syncwarp();
            if (page >= 0) {
                const int row = ((is_v * p.num_pages + page) * p.hkv + kvh) * p.page_size + tok % p.page_size;
                const uint32_t dst = smem_u32(kv_ring + b * S::KV_TILE) + my_half * (KT * 128) + my_piece * piece_rows * 128;
                tma_load_2d(dst, &kv_map, kv_full(b), my_half * 64, row);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_s = make_idesc(QM, KT);               // S = Q K^T: both operands K-major
            constexpr uint32_t idesc_o = make_idesc(QM, D, true);          // O = P V: V is MN-major (features contiguous)
            bool ok = mbar_wait(q_full, 0, abort_flag, p.status, 42);
            int js[2] = {t0x[0], t0x[1]}, jp[2] = {t0x[0], t0x[1]};        // next S and next P V to issue, per query tile
            uint32_t spins = 0;
            unsigned long long idle_since = 0;
            auto users = [&](int j) { return (j >= t0x[0] && j < t1x[0] ? 1 : 0) + (j >= t0x[1] && j < t1x[1] ? 1 : 0); };
            auto issued = [&](const int* next, int j) { return (j >= t0x[0] && j < t1x[0] && next[0] > j ? 1 : 0) +
                                                               (j >= t0x[1] && j < t1x[1] && next[1] > j ? 1 : 0); };
            // This one thread's instructions are what the tensor cores wait for between products (a descriptor made
            // from an address costs it as much as the MMA it describes costs the tensor pipe), so the descriptors
            // of the two query tiles and of the four key/value buffers are made once: a k step then is an addition.
            const uint64_t q_desc[2] = {make_sw128_desc(smem_u32(q_tiles)), make_sw128_desc(smem_u32(q_tiles) + S::Q_BYTES)};
            uint64_t k_desc[NBUF], v_desc[NBUF];
#pragma unroll
            for (int b = 0; b < NBUF; ++b) {
                k_desc[b] = make_sw128_desc(smem_u32(kv_ring + b * S::KV_TILE));
                v_desc[b] = make_sw128_desc_mn(smem_u32(kv_ring + b * S::KV_TILE), KT * 128, 1024);
            }
            auto pick = [&](const uint64_t* d, int b) { return b == 0 ? d[0] : (b == 1 ? d[1] : (b == 2 ? d[2] : d[3])); };
            while (ok && (jp[0] < t1x[0] || jp[1] < t1x[1])) {
                bool moved = false;
#pragma unroll
                for (int x = 0; x < 2; ++x) {
                    const uint32_t s_tmem = tmem_base + x * KT, o_tmem = tmem_base + 2 * KT + x * D;
                    if (jp[x] < js[x]) {                                   // P V of tile jp: P written, V landed
                        const int j = jp[x], li = 2 * (j - tmin) + 1, b = li % NBUF;
                        if (mbar_test_wait(p_full(x), (j - t0x[x]) & 1u) && mbar_test_wait(kv_full(b), (li / NBUF) & 1u)) {
                            tmem_fence_after();
                            const uint64_t vd = pick(v_desc, b);
                            // A: 16 keys = 8 columns of packed bfloat16 pairs (P lies over the first 64 of the
                            // tile's 128 score columns); B: 16 key rows of V = 2048 bytes further on (128 in the
                            // descriptor's 16-byte units)
                            umma_bf16_tmem_a(o_tmem, s_tmem, vd, idesc_o, j > t0x[x] ? 1u : 0u);
#pragma unroll
                            for (int ks = 1; ks < KT / 16; ++ks)
                                umma_bf16_tmem_a(o_tmem, s_tmem + ks * 8, vd + (uint64_t)(ks * 128), idesc_o, 1u);
                            umma_commit(o_full(x));
                            ++jp[x];
                            if (issued(jp, j) == users(j)) umma_commit(kv_empty(b));   // both tiles have read these values
                            moved = true;
                        }
                    }
                    if (js[x] < t1x[x] && js[x] == jp[x]) {                // S of the next tile: behind the P V before it
                        const int j = js[x], li = 2 * (j - tmin), b = li % NBUF;
                        if (mbar_test_wait(kv_full(b), (li / NBUF) & 1u)) {
                            tmem_fence_after();
                            const uint64_t kd = pick(k_desc, b), qd = q_desc[x];
#pragma unroll
                            for (int ks = 0; ks < D / 16; ++ks) {
                                // half of the head, then 32 bytes a step: in the descriptor's 16-byte units
                                const uint64_t off = (uint64_t)(((ks >> 2) * (QM * 128) + (ks & 3) * 32) >> 4);
                                umma_bf16(s_tmem, qd + off, kd + off, idesc_s, ks > 0 ? 1u : 0u);
                            }
                            umma_commit(s_full(x));
                            ++js[x];
                            if (issued(js, j) == users(j)) umma_commit(kv_empty(b));   // both tiles have read these keys
                            moved = true;
                        }
                    }
                }
                if (moved) { spins = 0; idle_since = 0; continue; }
                if ((++spins & 1023u) == 0u) {
                    if (idle_since == 0) idle_since = global_ns();
                    if (*abort_flag) ok = false;
                    else if (global_ns() - idle_since > TI_WAIT_NS) {
                        *abort_flag = 1;
                        if (p.status) atomicExch(p.status, 43);
                        ok = false;
                    }
                }
            }
        }
    } else {
        // ------------------------------------------------------------ softmax and output (warps 2..9)
        // A thread owns a query row (its tensor-memory lane): the whole row of 128 scores comes to registers in
        // one trip, nothing is exchanged with other threads, and P goes back in one.
        const int x = (warp - 2) >> 2;                                  // query tile of this warp
        const int lane_group = warp & 3;                                // tensor-memory lanes this warp may touch
        const int r = lane_group * 32 + lane;                           // query row of the tile = tensor-memory lane
        const int num_x = t1x[x] - t0x[x];
        const int first_pos = pos0 + x * QM;
        const int qpos = first_pos + r;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(lane_group * 32) << 16);
        const uint32_t s_tmem = lane_addr + x * KT, o_tmem = lane_addr + 2 * KT + x * D;
        const int gtid = threadIdx.x - 64 - x * 128;                    // 0..127 among this tile's softmax threads
        float m_ref = -INFINITY, l_run = 0.f;
        bool ok = true;
        for (int i = 0; i < num_x && ok; ++i) {
            const int j = t0x[x] + i;
            const int tk0 = j * KT;
            if (!mbar_wait(s_full(x), i & 1u, abort_flag, p.status, 44)) { ok = false; break; }
            tmem_fence_after();
            // columns of this tile the row may see: kmin < column <= kmax (tile-local)
            const int kmax = qpos - tk0;
            const int kmin = p.window > 0 ? qpos - p.window - tk0 : -1;
            const bool all_seen = KT - 1 <= kmax && kmin < 0;
            uint32_t sr[KT];
#pragma unroll
            for (int cc = 0; cc < KT; cc += 32) tmem_ld32_nowait(s_tmem + cc, sr + cc);
            tmem_wait_ld();
            // the row's maximum (of the visible scores), four chains side by side
            float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            if (all_seen) {
#pragma unroll
                for (int k = 0; k < KT; k += 8)
#pragma unroll
                    for (int u = 0; u < 4; ++u)
                        m4[u] = fmax3(m4[u], __uint_as_float(sr[k + 2 * u]), __uint_as_float(sr[k + 2 * u + 1]));
            } else {
#pragma unroll
                for (int k = 0; k < KT; ++k) {
                    if (!(k <= kmax && k > kmin)) sr[k] = 0xff800000u;             // -inf: masked by assignment
                    m4[k & 3] = fmaxf(m4[k & 3], __uint_as_float(sr[k]));
                }
            }
            const float mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])) * p.scale_log2;   // the scale is positive
            // The reference maximum moves only when the row's maximum has outgrown it by RESCALE_STEP.
            const bool move = mx > m_ref + RESCALE_STEP || (m_ref == -INFINITY && mx > -INFINITY);
            const float m_new = move ? mx : m_ref;
            const float m_old = m_ref;
            m_ref = m_new;
            const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
            // P = 2^(s * scale - m) (a masked score is -inf: exactly 0), its sum, and P as packed bfloat16 over the
            // first 64 score columns of the tile
            // Sixteen exponentials are issued before the first of them is used: a warp is alone on its scheduler
            // while the other tile is in its products, and an ex2 takes tens of cycles to come back.
            float l4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int k0 = 0; k0 < KT; k0 += 16) {
#pragma unroll
                for (int u = 0; u < 16; ++u)
                    sr[k0 + u] = __float_as_uint(ex2(fmaf(__uint_as_float(sr[k0 + u]), p.scale_log2, -m_use)));
#pragma unroll
                for (int u = 0; u < 16; u += 2) {
                    const float a = __uint_as_float(sr[k0 + u]), b = __uint_as_float(sr[k0 + u + 1]);
                    l4[(u >> 1) & 3] += a + b;
                    sr[(k0 + u) >> 1] = pack2(a, b);
                }
            }
            l_run = l_run * (move ? ex2(m_old - m_new) : 1.f) + ((l4[0] + l4[1]) + (l4[2] + l4[3]));   // m_old = -inf: l_run is 0
            tmem_st32(s_tmem, sr);
            tmem_st32(s_tmem + 32, sr + 32);
            // (after P is on its way, so that the row of scores and the row of O never share the registers)
            if (i > 0 && __any_sync(0xffffffffu, move)) {
                // the rows of O so far carry the old reference: O *= 2^(m_ref - m_new), once P V of the tile before is in
                if (!mbar_wait(o_full(x), (i - 1) & 1u, abort_flag, p.status, 45)) { ok = false; break; }
                tmem_fence_after();
                const float f = move ? ex2(m_old - m_new) : 1.f;               // m_ref = -inf: O and l are 0, f = 0 is right
                uint32_t orow[32];
#pragma unroll
                for (int c = 0; c < D; c += 32) {
                    tmem_ld32_nowait(o_tmem + c, orow);
                    tmem_wait_ld();
#pragma unroll
                    for (int k = 0; k < 32; ++k) orow[k] = __float_as_uint(__uint_as_float(orow[k]) * f);
                    tmem_st32(o_tmem + c, orow);
                }
            }
            tmem_wait_st();
            // value rows no query of the CTA may see: zero them once the tile has landed (first and last tiles only)
            if (tk0 < lo || tk0 + KT > hi) {
                const int li = 2 * (j - tmin) + 1, b = li % NBUF;
                if (!mbar_wait(kv_full(b), (li / NBUF) & 1u, abort_flag, p.status, 46)) { ok = false; break; }
                uint8_t* v_tile = kv_ring + b * S::KV_TILE;
                for (int idx = gtid; idx < KT * (D / 8); idx += 128) {
                    const int row = idx / (D / 8), chunk = idx % (D / 8);
                    if (row >= lo - tk0 && row < hi - tk0) continue;
                    *reinterpret_cast<uint4*>(v_tile + (chunk >> 3) * (KT * 128) + row * 128 + (((chunk & 7) ^ (row & 7)) << 4)) =
                        make_uint4(0, 0, 0, 0);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the zeroed rows are read by the MMA
            }
            tmem_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full(x));
        }
        if (ok && num_x > 0) {
            if (mbar_wait(o_full(x), (num_x - 1) & 1u, abort_flag, p.status, 47)) {
                tmem_fence_after();
                const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
                const int rows_x = min(QM, nrows - x * QM);
                __nv_bfloat16* dst = p.out + ((size_t)(row0 + x * QM + r) * p.hq + head) * D;
                uint32_t orow[32];
#pragma unroll
                for (int c = 0; c < D; c += 32) {
                    tmem_ld32_nowait(o_tmem + c, orow);
                    tmem_wait_ld();
                    if (r < rows_x) {
#pragma unroll
                        for (int q8 = 0; q8 < 4; ++q8) {
                            uint4 w;
                            w.x = pack2(__uint_as_float(orow[q8 * 8]) * inv, __uint_as_float(orow[q8 * 8 + 1]) * inv);
                            w.y = pack2(__uint_as_float(orow[q8 * 8 + 2]) * inv, __uint_as_float(orow[q8 * 8 + 3]) * inv);
                            w.z = pack2(__uint_as_float(orow[q8 * 8 + 4]) * inv, __uint_as_float(orow[q8 * 8 + 5]) * inv);
                            w.w = pack2(__uint_as_float(orow[q8 * 8 + 6]) * inv, __uint_as_float(orow[q8 * 8 + 7]) * inv);
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

}  // namespace

TI_API int ti_attention_prefill_pair_rows() { return 2 * QM; }

// Prefill attention on tcgen05, two query tiles a CTA. `tiles`: num_tiles int4 {request index in the step,
// first flat row, rows (<= 256), position of the first row}, every tile inside one request's portion.
// q [T, Hq, D], out [T, Hq * D], kv_cache [2, num_pages, Hkv, page_size, D]; page_size 16, 32 or a multiple of 64.
TI_API int ti_attention_prefill_pair_bf16(void* out, const void* q, const void* kv_cache, const int* tiles, int num_tiles,
                                          int num_tokens, const int* block_table, int max_blocks, int hq, int hkv, int d,
                                          int page_size, int num_pages, float scale, int window, int* status,
                                          cudaStream_t stream) {
    TI_REQUIRE(d == 64 || d == 128, "attention_prefill_pair: head_dim %d is not 64 or 128", d);
    TI_REQUIRE(hq > 0 && hkv > 0 && hq % hkv == 0, "attention_prefill_pair: bad head counts");
    TI_REQUIRE(num_tiles <= 65535, "attention_prefill_pair: more than 65535 tiles in one step");
    TI_REQUIRE(page_size == 16 || page_size == 32 || page_size % 64 == 0, "attention_prefill_pair: page size %d", page_size);
    TI_REQUIRE(num_tiles >= 0 && num_tokens > 0, "attention_prefill_pair: bad sizes");
    if (num_tiles == 0) return 0;
    CUtensorMap q_map, kv_map;
    if (!ti_get_bf16_map(q, num_tokens, hq * d, QM, &q_map)) return -1;
    if (!ti_get_bf16_map(kv_cache, 2ll * num_pages * hkv * page_size, d, page_size < 64 ? page_size : 64, &kv_map)) return -1;
    PairParams p;
    p.out = (__nv_bfloat16*)out; p.tiles = tiles; p.block_table = block_table; p.max_blocks = max_blocks;
    p.hq = hq; p.hkv = hkv; p.page_size = page_size; p.num_pages = num_pages; p.window = window;
    p.scale_log2 = scale * 1.4426950408889634f; p.status = status;
    dim3 grid(hq, num_tiles);
    if (d == 128) {
        static bool once = false;
        if (!once) {
            cudaError_t e = cudaFuncSetAttribute(prefill_attention_pair_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, PpSmem<128>::BYTES);
            TI_REQUIRE(e == cudaSuccess, "attention_prefill_pair: shared memory: %s", cudaGetErrorString(e));
            once = true;
        }
        ti_launch(prefill_attention_pair_kernel<128>, grid, PP_THREADS, PpSmem<128>::BYTES, stream, q_map, kv_map, p);
    } else {
        static bool once = false;
        if (!once) {
            cudaError_t e = cudaFuncSetAttribute(prefill_attention_pair_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, PpSmem<64>::BYTES);
            TI_REQUIRE(e == cudaSuccess, "attention_prefill_pair: shared memory: %s", cudaGetErrorString(e));
            once = true;
        }
        ti_launch(prefill_attention_pair_kernel<64>, grid, PP_THREADS, PpSmem<64>::BYTES, stream, q_map, kv_map, p);
    }
    TI_CHECK_LAUNCH("attention_prefill_pair");
    return 0;
}
