// bfloat16 matrix product y[M,N] = x[M,K] . w[N,K]^T on the 5th-generation tensor cores of
// sm_100a: operands staged in shared memory by TMA (128-byte swizzle, no multicast), one elected
// thread issuing tcgen05.mma, float32 accumulators in tensor memory, read back with tcgen05.ld for
// the epilogue. The kernel is persistent (one CTA per SM walks over output tiles) and warp
// specialised: warp 0 loads, warp 1 issues the MMAs, warps 2..5 run the epilogue of tile i while
// the MMAs of tile i+1 fill the other half of tensor memory.
//
// Two orientations share the code. "Rows" are the 128 accumulator lanes, "cols" the BN columns:
//   tokens on the lanes (many tokens):  rows = tokens of x, cols = output features of w; tiles of
//       128 x 256 (or 128 x 128), and of 256 x 256 for very large steps (two accumulators of one tile);
//       with few tiles and 130 to 700 tokens the k loops are cut and the units of a tile add their
//       partial sums up together, each its share of the columns;
//   weights on the lanes (M <= 128, gated form M <= 64): rows = output features of w, cols = tokens of x
//       (padded to BN), so a decode step streams every weight once with full 128-row MMAs; the k
//       loops are cut to fill the SMs; up to 15 tokens the last unit of a tile adds the partial sums
//       up, from 16 tokens on the units of a tile do so together, each its share of the tokens.
// Epilogues, all on the float32 accumulators with one rounding: + bias[n], + residual[m,n],
// float32 output (logits), the gated form out[m,j] = silu(x.w[j]) * (x.w[J+j]) of the
// reference's MLP kernel (tinyinfer/csrc/mlp.cu:116-141), and the two halves of an RMSNorm that is
// spread over the products around it (see GemmParams). A row's result does not depend on
// which other rows share its tile: every output element is one k loop in a fixed order, or a
// fixed number of partial k loops added in a fixed order.
//
// Every wait is bounded: those on mbarriers, and the one where the units of a tile wait for each other
// on a counter in global memory (about two seconds, by the SM's clock). A wait that runs out sets
// *status, raises the CTA's abort flag, and all warps fall through to the common exit, where tensor
// memory is freed.
#include "sm100_ptx.cuh"
#include <type_traits>

namespace {

constexpr int BM = 128;          // accumulator lanes = rows of the "rows" operand per tile
constexpr int BK = 64;           // bf16 elements per 128-byte swizzled row
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 192;
constexpr int SMEM_BUDGET = 212 * 1024;

struct GemmParams {
    void* out;
    const float* bias;
    const __nv_bfloat16* residual;
    int M, N, K;            // problem: out is [M, N] (gated: N = J, w has 2J rows)
    int rows_total;         // extent of the rows operand that tiles walk over
    int cols_total;         // extent of the cols operand
    int gated, out_f32, swap;
    int splits;             // the k range of a tile is cut into this many work units
    int share_sum;          // weights on the lanes, splits > 1: every unit of a tile adds up its share of the
                            // tokens once all units have arrived (all units run at once), not the last alone
    float* partials;        // [tile][split][col][128] float32 scratch for splits > 1
    int* counters;          // [tile] arrivals; zero before the launch and again after it
    // Weights on the lanes only: an RMSNorm spread over two products. The product that makes a residual
    // stream x also stores x * g (g: the weights of the norm that follows, rounded to bfloat16 like x) and,
    // per 128 outputs and token, the sum of squares of x as rounded (emit_*). The product behind the norm
    // reads x * g as its input and multiplies every output row by rsqrt(mean(x^2) + eps) (scale_*): the
    // norm kernel between the two, and the hop it costs in a decode step, are gone.
    const float* emit_g;            // [N] or null
    __nv_bfloat16* emit_xg;         // [M, N]
    float* emit_sums;               // [row tiles][M]
    const float* scale_sums;        // [scale_parts][M] or null
    int scale_parts, scale_dim;     // the rows of x had scale_dim elements
    float scale_eps;
    int* status;
};

__device__ __forceinline__ float silu_mul(float g, float u) { return (g / (1.f + __expf(-g))) * u; }

// TM: accumulators of 128 rows a tile holds. 1: tiles of 128 x BN with two accumulators in tensor memory,
// so that the epilogue of a tile overlaps the MMAs of the next. 2 (only with BN = 256, many tokens): tiles of
// 256 x 256, both accumulators belong to one tile and every tile of w is used by two MMAs: an SM takes in
// about 64 bytes a cycle from L2, and a 128 x 256 tile needs 48 KB for 512 cycles of MMAs (it waits for
// its operands a third of the time), a 256 x 256 tile 64 KB for 1024 cycles.
template <int BN, int TM = 1>
struct Cfg {
    static_assert(TM == 1 || (TM == 2 && BN == 256), "tall tiles are 256 x 256");
    static constexpr int STAGE_BYTES = (TM * BM + BN) * BK * 2;
    static constexpr int TMEM_COLS = TM == 2 ? 512 : (2 * BN < 32 ? 32 : 2 * BN);   // two accumulators; a power of two
    static constexpr int EXCH_FLOATS = BN <= 64 ? 64 * 17 + 2 : 2;   // swapped gated epilogue (BN <= 64): 16 tokens at a time; + one word
    // small-batch tiles (BN <= 64) take half an SM's shared memory, so that two CTAs share an SM: one
    // streams weights while the other reduces and stores, and the next kernel's CTAs can move in early
    static constexpr int CTAS_PER_SM = BN <= 64 ? 2 : 1;
    static constexpr int BUDGET = (TM == 2 ? 216 * 1024 : SMEM_BUDGET / CTAS_PER_SM) - EXCH_FLOATS * 4;
    static constexpr int STAGES = (BUDGET / STAGE_BYTES) > 12 ? 12 : (BUDGET / STAGE_BYTES);
    static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + EXCH_FLOATS * 4 + 256;
    static_assert(STAGES >= 2, "too little shared memory for a pipeline");
    static_assert(CTAS_PER_SM * (SMEM_BYTES + 1024) <= 227 * 1024, "the CTAs of an SM do not fit its shared memory");
};

// SWAP: weights on the lanes (a compile-time choice, so that a decode step's kernels carry none of the code for many tokens).
template <int BN, int TM, bool SWAP>
__global__ void __launch_bounds__(NUM_THREADS, Cfg<BN, TM>::CTAS_PER_SM)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_rows, const __grid_constant__ CUtensorMap map_cols,
                    const GemmParams p) {
    using C = Cfg<BN, TM>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* stages = smem;
    float* exch = reinterpret_cast<float*>(smem + C::STAGES * C::STAGE_BYTES);
    uint64_t* bars = reinterpret_cast<uint64_t*>(exch + C::EXCH_FLOATS);
    // barrier layout: full[STAGES], empty[STAGES], acc_full[2], acc_empty[2]
    const uint32_t bar0 = smem_u32(bars);
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (C::STAGES + s); };
    auto acc_full_bar = [&](int a) { return bar0 + 8u * (2 * C::STAGES + a); };
    auto acc_empty_bar = [&](int a) { return bar0 + 8u * (2 * C::STAGES + 2 + a); };
    __shared__ uint32_t tmem_base_sh;
    __shared__ int abort_sh;
    __shared__ float row_scale_sh[128];     // scale_*: 1 / rms of every token of the tile (1 if no scale)
    volatile int* abort_flag = &abort_sh;

    ti_grid_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // tiles: gated normal tiles hold BN/2 gate and BN/2 up columns; gated swapped tiles 64 + 64 rows
    const int rows_per_tile = (p.gated && SWAP) ? BM / 2 : TM * BM;
    const int cols_per_tile = (p.gated && !SWAP) ? BN / 2 : BN;
    const int row_tiles = (p.rows_total + rows_per_tile - 1) / rows_per_tile;
    const int col_tiles = (p.cols_total + cols_per_tile - 1) / cols_per_tile;
    const int num_tiles = row_tiles * col_tiles;
    const int num_kb = (p.K + BK - 1) / BK;
    const int num_units = num_tiles * p.splits;     // unit = tile * splits + split: a tile's splits run side by side
    // A CTA's i-th piece of work: k blocks kb0 .. kb1 of a tile, as part `split` of `nsplits` parts of the tile.
    // (32-bit arithmetic: splits x k blocks of a tile stays far below 2^31; with 64-bit divisions here the loading
    // thread, whose work per unit is on a decode step's critical path, made the step 1 % slower.)
    struct Work { int tile, split, nsplits, kb0, kb1; };
    auto work_at = [&](int i, Work& w) -> bool {
        const int unit = (int)blockIdx.x + i * (int)gridDim.x;
        if (unit >= num_units) return false;
        w.tile = unit / p.splits; w.split = unit % p.splits; w.nsplits = p.splits;
        w.kb0 = w.split * num_kb / p.splits;
        w.kb1 = (w.split + 1) * num_kb / p.splits;
        return true;
    };

    // a thread a barrier (up to 28 of them: one thread alone spent a third of a microsecond of every launch here)
    if (threadIdx.x == 0) abort_sh = 0;
    if (threadIdx.x < 2 * C::STAGES + 4) {
        const int b = threadIdx.x;                       // full[STAGES], empty[STAGES], acc_full[2], acc_empty[2]
        mbar_init(bar0 + 8u * b, b >= 2 * C::STAGES + 2 ? 4 : 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_base_sh)), "r"((uint32_t)C::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tmem_fence_before();
    __syncthreads();
    tmem_fence_after();
    const uint32_t tmem_base = tmem_base_sh;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            // The copies of one k block of the tile whose first row and column are r0 and c0: `rows_side` /
            // `cols_side` pick the operand(s) to load. (This thread's work per k block is on the critical
            // path of a decode step: what depends on the unit alone is worked out once per unit.)
            auto issue = [&](int r0, int c0, int kb, int s, bool rows_side, bool cols_side) {
                const uint32_t a_dst = smem_u32(stages + s * C::STAGE_BYTES);
                const uint32_t b_dst = a_dst + TM * BM * BK * 2;      // tall tiles: one copy of 256 rows
                if (rows_side) {
                    tma_load_2d(a_dst, &map_rows, full_bar(s), kb * BK, r0);
                    if (p.gated && SWAP)            // 64 gate rows, then 64 up rows
                        tma_load_2d(a_dst + (BM / 2) * BK * 2, &map_rows, full_bar(s), kb * BK, p.N + r0);
                }
                if (cols_side) {
                    tma_load_2d(b_dst, &map_cols, full_bar(s), kb * BK, c0);
                    if (p.gated && !SWAP)           // BN/2 gate rows, then BN/2 up rows
                        tma_load_2d(b_dst + (BN / 2) * BK * 2, &map_cols, full_bar(s), kb * BK, p.N + c0);
                }
            };
            auto unit_range = [&](int i, int& r0, int& c0, int& kb0, int& kb1) -> bool {
                Work w;
                if (!work_at(i, w)) return false;
                r0 = (w.tile % row_tiles) * rows_per_tile;
                c0 = (w.tile / row_tiles) * cols_per_tile;
                kb0 = w.kb0; kb1 = w.kb1;
                return true;
            };
            // Before waiting for the kernels ahead of this one in the stream: the weights do not
            // depend on them, so their copies for the first ring of stages start right away and
            // HBM stays busy while the previous kernel drains. The activations follow after the wait.
            const bool weights_are_rows = SWAP;
            uint32_t pre = 0;
            for (int i = 0; pre < (uint32_t)C::STAGES; ++i) {
                int r0, c0, kb0, kb1;
                if (!unit_range(i, r0, c0, kb0, kb1)) break;
                for (int kb = kb0; kb < kb1 && pre < (uint32_t)C::STAGES; ++kb, ++pre) {
                    mbar_expect_tx(full_bar(pre), C::STAGE_BYTES);
                    issue(r0, c0, kb, pre, weights_are_rows, !weights_are_rows);
                }
            }
            ti_grid_wait();
            uint32_t it = 0;
            bool ok = true;
            for (int i = 0; ok; ++i) {
                int r0, c0, kb0, kb1;
                if (!unit_range(i, r0, c0, kb0, kb1)) break;
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = it % C::STAGES;
                    if (it < pre) {                   // its weights are already on their way
                        issue(r0, c0, kb, s, !weights_are_rows, weights_are_rows);
                        continue;
                    }
                    const uint32_t ph = (it / C::STAGES) & 1u;
                    if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, p.status, 11)) { ok = false; break; }
                    mbar_expect_tx(full_bar(s), C::STAGE_BYTES);
                    issue(r0, c0, kb, s, true, true);
                }
            }
            // After an abort, give the copies this CTA still has in flight time to land (they take
            // microseconds) before shared memory is given up: a bounded wait of one millisecond.
            if (!ok) {
                const unsigned long long t0 = global_ns();
                while (global_ns() - t0 < 1000000ull) {}
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(BM, BN);
            uint32_t it = 0, tile_i = 0;
            bool ok = true;
            Work wk;
            for (; ok && work_at((int)tile_i, wk); ++tile_i) {
                const int kb0 = wk.kb0, kb1 = wk.kb1;
                // tall tiles own all of tensor memory: one accumulator buffer, a phase per tile
                const uint32_t as = TM == 2 ? 0u : (tile_i & 1u), aph = TM == 2 ? (tile_i & 1u) : ((tile_i >> 1) & 1u);
                if (!mbar_wait(acc_empty_bar(as), aph ^ 1u, abort_flag, p.status, 12)) { ok = false; break; }
                tmem_fence_after();
                const uint32_t d_tmem = tmem_base + as * BN;
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = it % C::STAGES;
                    const uint32_t ph = (it / C::STAGES) & 1u;
                    if (!mbar_wait(full_bar(s), ph, abort_flag, p.status, 13)) { ok = false; break; }
                    tmem_fence_after();
                    const uint32_t a_addr = smem_u32(stages + s * C::STAGE_BYTES);
                    const uint64_t adesc = make_sw128_desc(a_addr);
                    const uint64_t bdesc = make_sw128_desc(a_addr + TM * BM * BK * 2);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        // 16 bf16 = 32 bytes along K inside the 128-byte swizzled row: +2 in 16-byte units
                        umma_bf16(d_tmem, adesc + 2u * k, bdesc + 2u * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
                        if constexpr (TM == 2)      // rows 128..255 of the tile: 16 KB further in the stage, next 256 columns
                            umma_bf16(d_tmem + BN, make_sw128_desc(a_addr + BM * BK * 2) + 2u * k, bdesc + 2u * k, idesc,
                                      (kb > kb0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(empty_bar(s));           // the stage is free once these MMAs have read it
                }
                if (ok) umma_commit(acc_full_bar(as));   // the accumulator is complete
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..5)
        ti_grid_wait();                                  // residual, scratch and out belong to earlier kernels until now
        const int lane_group = warp & 3;                 // the 32 accumulator lanes this warp may read
        const int row_in_tile = lane_group * 32 + lane;
        uint32_t tile_i = 0;
        bool ok = true;
        if (SWAP) {                                    // tokens are columns: at most BN <= 128 of them, one column tile
            float sc = 1.f;
            if (p.scale_sums != nullptr && row_in_tile < p.M) {
                float ss = 0.f;
                for (int part = 0; part < p.scale_parts; ++part) ss += p.scale_sums[(size_t)part * p.M + row_in_tile];
                sc = rsqrtf(ss / (float)p.scale_dim + p.scale_eps);
            }
            row_scale_sh[row_in_tile] = sc;
            asm volatile("bar.sync 1, 128;" ::: "memory");
        }
        Work wk;
        for (; ok && work_at((int)tile_i, wk); ++tile_i) {
            const int tile = wk.tile, split = wk.split, nsplits = wk.nsplits;
            const int rt = tile % row_tiles, ct = tile / row_tiles;
            const int r0 = rt * rows_per_tile, c0 = ct * cols_per_tile;
            const uint32_t as = TM == 2 ? 0u : (tile_i & 1u), aph = TM == 2 ? (tile_i & 1u) : ((tile_i >> 1) & 1u);
            if (!mbar_wait(acc_full_bar(as), aph, abort_flag, p.status, 14)) { ok = false; break; }
            tmem_fence_after();
            const uint32_t t_addr0 = tmem_base + as * BN + ((uint32_t)(lane_group * 32) << 16);
            const uint32_t t_addr = t_addr0;
            float v[16], u[16];
            bool released = false;
            // Split k range: every unit leaves its partial accumulator in scratch; the unit that
            // arrives last sums all partials of the tile in split order (so the result does not
            // depend on who was last) and runs the epilogue.
            float* tile_partials = nullptr;
            if (nsplits > 1 && SWAP) {
                tile_partials = p.partials + (size_t)tile * nsplits * BN * BM;
                float* mine = tile_partials + (size_t)split * BN * BM + row_in_tile;
                for (int c = 0; c < BN; c += 16) {
                    tmem_ld16(t_addr + c, v);
#pragma unroll
                    for (int i = 0; i < 16; ++i) __stcg(mine + (size_t)(c + i) * BM, v[i]);
                }
                tmem_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(acc_empty_bar(as));
                released = true;
                // Publish, then count: the barrier orders every thread's stores before thread 64's count,
                // which releases them (cumulative, GPU scope) and acquires what the units before it
                // released; after the barrier behind it every thread may read the other units' partials
                // (from L2, never from L1). One acquire-release atomic took 0.3 to 0.4 us less per
                // product than a fence on either side of a relaxed one.
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (threadIdx.x == 64) {
                    int arrived;
                    asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(arrived) : "l"(p.counters + tile) : "memory");
                    if (p.share_sum) {
                        // every unit of the tile takes a share of the sum: wait for the others (they all
                        // run at once: the host launches one CTA per unit, no more than fit the SMs)
                        arrived = nsplits - 1;
                        const long long t_start = clock64();
                        for (uint32_t spin = 1; *reinterpret_cast<volatile int*>(p.counters + tile) < nsplits; ++spin) {
                            __nanosleep(64);
                            if ((spin & 63u) == 0u && (*abort_flag || clock64() - t_start > 4000000000ll)) { arrived = -1; break; }
                        }
                    } else if (arrived == nsplits - 1) {
                        p.counters[tile] = 0;     // leave the counter ready for the next launch
                    }
                    if (p.share_sum) __threadfence();          // after the wait: the other units' partials may be read
                    *reinterpret_cast<volatile int*>(&exch[C::EXCH_FLOATS - 1]) = arrived;
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                const int arrived = *reinterpret_cast<volatile int*>(&exch[C::EXCH_FLOATS - 1]);
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (arrived < 0) {                                 // a unit of the tile never came: give up, loudly
                    *abort_flag = 1;
                    if (p.status && threadIdx.x == 64) atomicExch(p.status, 16);
                    ok = false;
                    break;
                }
                if (arrived != nsplits - 1) continue;
                // Swapped (the products of a decode step): the four warps share the columns (tokens), a
                // lane takes four consecutive rows (output features). So every load is 16 bytes and a
                // warp reads a whole column of a partial at once; the partials of several columns and
                // of all splits are in flight together and are added in split order. Gated: lanes 0..15
                // hold gate rows j.., lanes 16..31 the up rows of the same outputs, which reach the
                // gate's lanes by a shuffle.
                if (SWAP && (p.N & 3) == 0 &&
                    (p.gated ? ((uintptr_t)p.out & 7) == 0
                             : ((uintptr_t)p.out & 15) == 0 && ((uintptr_t)p.residual & 7) == 0 && ((uintptr_t)p.bias & 15) == 0)) {
                    const int n0 = r0 + 4 * (p.gated ? (lane & 15) : lane);
                    const bool n_ok = n0 < p.N;                        // N is a multiple of 4: all four rows or none
                    float4 b4 = make_float4(0.f, 0.f, 0.f, 0.f), g4 = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (p.bias && n_ok) b4 = *reinterpret_cast<const float4*>(p.bias + n0);
                    if (p.emit_g && n_ok) g4 = *reinterpret_cast<const float4*>(p.emit_g + n0);
                    const int cols_real = min(BN, p.M - c0);
                    // the tokens this unit finishes: all of them, or with a shared sum those with
                    // token mod splits == split
                    const int col_first = p.share_sum ? split : 0, col_step = p.share_sum ? nsplits : 1;
                    auto wide = [&](auto cols_tag, auto splits_tag) {
                        constexpr int G = decltype(cols_tag)::value, SP = decltype(splits_tag)::value;
                        for (int g0 = col_first + lane_group * col_step; g0 < cols_real; g0 += 4 * G * col_step) {
                            float4 acc[G];
                            uint2 res[G];
                            float sq[G];
#pragma unroll
                            for (int i = 0; i < G; ++i) sq[i] = 0.f;
#pragma unroll
                            for (int i = 0; i < G; ++i) {
                                acc[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                                res[i] = make_uint2(0u, 0u);
                                const int col = g0 + 4 * i * col_step;
                                if (p.residual && n_ok && col < cols_real)
                                    res[i] = *reinterpret_cast<const uint2*>(p.residual + (size_t)(c0 + col) * p.N + n0);
                            }
                            for (int sp0 = 0; sp0 < nsplits; sp0 += SP) {
                                float4 part[SP][G];
#pragma unroll
                                for (int sp = 0; sp < SP; ++sp) {
#pragma unroll
                                    for (int i = 0; i < G; ++i) {
                                        const int col = g0 + 4 * i * col_step;
                                        const bool in = sp0 + sp < nsplits && col < cols_real;
                                        part[sp][i] = in ? __ldcg(reinterpret_cast<const float4*>(
                                                               tile_partials + ((size_t)(sp0 + sp) * BN + col) * BM + 4 * lane))
                                                         : make_float4(0.f, 0.f, 0.f, 0.f);
                                    }
                                }
#pragma unroll
                                for (int sp = 0; sp < SP; ++sp) {
#pragma unroll
                                    for (int i = 0; i < G; ++i) {
                                        acc[i].x += part[sp][i].x; acc[i].y += part[sp][i].y;
                                        acc[i].z += part[sp][i].z; acc[i].w += part[sp][i].w;
                                    }
                                }
                            }
                            if (p.gated) {
#pragma unroll
                                for (int i = 0; i < G; ++i) {
                                    const int col = g0 + 4 * i * col_step;              // the same for the whole warp
                                    float4 up;
                                    up.x = __shfl_xor_sync(0xffffffffu, acc[i].x, 16); up.y = __shfl_xor_sync(0xffffffffu, acc[i].y, 16);
                                    up.z = __shfl_xor_sync(0xffffffffu, acc[i].z, 16); up.w = __shfl_xor_sync(0xffffffffu, acc[i].w, 16);
                                    if (lane >= 16 || !n_ok || col >= cols_real) continue;
                                    const float sc = row_scale_sh[col];                 // gate and up alike
                                    __nv_bfloat162 lo2 = __floats2bfloat162_rn(silu_mul(acc[i].x * sc, up.x * sc), silu_mul(acc[i].y * sc, up.y * sc));
                                    __nv_bfloat162 hi2 = __floats2bfloat162_rn(silu_mul(acc[i].z * sc, up.z * sc), silu_mul(acc[i].w * sc, up.w * sc));
                                    uint2 o2;
                                    o2.x = *reinterpret_cast<uint32_t*>(&lo2);
                                    o2.y = *reinterpret_cast<uint32_t*>(&hi2);
                                    *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.out) + (size_t)(c0 + col) * p.N + n0) = o2;
                                }
                                continue;
                            }
#pragma unroll
                            for (int i = 0; i < G; ++i) {
                                const int col = g0 + 4 * i * col_step;
                                if (!n_ok || col >= cols_real) continue;
                                const __nv_bfloat162* r2 = reinterpret_cast<const __nv_bfloat162*>(&res[i]);
                                const float2 ra = __bfloat1622float2(r2[0]), rb = __bfloat1622float2(r2[1]);
                                const float sc = row_scale_sh[col];
                                const float4 v4 = make_float4(acc[i].x * sc + b4.x + ra.x, acc[i].y * sc + b4.y + ra.y,
                                                              acc[i].z * sc + b4.z + rb.x, acc[i].w * sc + b4.w + rb.y);
                                const size_t idx = (size_t)(c0 + col) * p.N + n0;
                                if (p.out_f32) {
                                    *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + idx) = v4;
                                } else {
                                    uint2 o2;
                                    __nv_bfloat162 lo2 = __floats2bfloat162_rn(v4.x, v4.y), hi2 = __floats2bfloat162_rn(v4.z, v4.w);
                                    o2.x = *reinterpret_cast<uint32_t*>(&lo2);
                                    o2.y = *reinterpret_cast<uint32_t*>(&hi2);
                                    *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.out) + idx) = o2;
                                    if (p.emit_g != nullptr) {           // x * g of the rounded x, and the squares of x
                                        const float2 xa = __bfloat1622float2(lo2), xb = __bfloat1622float2(hi2);
                                        sq[i] = xa.x * xa.x + xa.y * xa.y + xb.x * xb.x + xb.y * xb.y;
                                        __nv_bfloat162 ga = __floats2bfloat162_rn(xa.x * g4.x, xa.y * g4.y);
                                        __nv_bfloat162 gb = __floats2bfloat162_rn(xb.x * g4.z, xb.y * g4.w);
                                        uint2 e2;
                                        e2.x = *reinterpret_cast<uint32_t*>(&ga);
                                        e2.y = *reinterpret_cast<uint32_t*>(&gb);
                                        *reinterpret_cast<uint2*>(p.emit_xg + idx) = e2;
                                    }
                                }
                            }
                            if (p.emit_g != nullptr) {
                                // the warp holds all 128 outputs of the tile for this token
#pragma unroll
                                for (int i = 0; i < G; ++i) {
                                    const int col = g0 + 4 * i * col_step;                  // the same for the whole warp
                                    if (col >= cols_real) continue;
                                    float t = sq[i];
#pragma unroll
                                    for (int off = 16; off > 0; off >>= 1) t += __shfl_xor_sync(0xffffffffu, t, off);
                                    if (lane == 0) p.emit_sums[(size_t)rt * p.M + c0 + col] = t;
                                }
                            }
                        }
                    };
                    // two columns and eight splits a trip to L2, whatever the number of splits (one form: see the note on the kernel's length below)
                    wide(std::integral_constant<int, 2>{}, std::integral_constant<int, 8>{});
                    if (p.share_sum) {
                        // second arrival: when every unit has read what it needs, the last one clears the counter
                        asm volatile("bar.sync 1, 128;" ::: "memory");
                        if (threadIdx.x == 64) {
                            if (atomicAdd(p.counters + tile, 1) == 2 * nsplits - 1) p.counters[tile] = 0;
                        }
                    }
                    continue;
                }
            }
            // The last arriver's sum on the path of odd sizes (the 16-byte path above takes the sizes of real
            // models): the partials of 16 columns and of two splits are requested together, 32 independent
            // loads, then added in split order. Kept short on purpose: with three forms of it (64 loads each, by
            // number of splits) the kernel for 16 tokens was 143 KB of code and every decode product paid for
            // fetching it (8 x 6144 x 4096: 11.4 -> 10.5 us with 75 KB). Swapped tiles skip the columns beyond
            // the last token: nothing of them is stored.
            auto sum_group = [&](int c, float* dst, auto cols_tag, auto splits_tag) {
                constexpr int COLS = decltype(cols_tag)::value, SPLITS = decltype(splits_tag)::value;
#pragma unroll
                for (int i0 = 0; i0 < 16; i0 += COLS) {
                    float acc[COLS];
#pragma unroll
                    for (int i = 0; i < COLS; ++i) acc[i] = 0.f;
                    if (!SWAP || c0 + c + i0 < p.M) {
                        for (int sp0 = 0; sp0 < nsplits; sp0 += SPLITS) {
                            float part[SPLITS][COLS];
#pragma unroll
                            for (int sp = 0; sp < SPLITS; ++sp) {
                                const bool in = sp0 + sp < nsplits;
                                const float* src = tile_partials + (size_t)(in ? sp0 + sp : 0) * BN * BM + row_in_tile;
#pragma unroll
                                for (int i = 0; i < COLS; ++i) part[sp][i] = in ? __ldcg(src + (size_t)(c + i0 + i) * BM) : 0.f;
                            }
#pragma unroll
                            for (int sp = 0; sp < SPLITS; ++sp) {
#pragma unroll
                                for (int i = 0; i < COLS; ++i) acc[i] += part[sp][i];
                            }
                        }
                    }
#pragma unroll
                    for (int i = 0; i < COLS; ++i) dst[i0 + i] = acc[i];
                }
            };
            auto load_chunk = [&](int c, float* dst) {
                if (nsplits > 1) {       // (one form for every number of splits: this is the path of odd sizes, and the kernel's code is long as it is)
                    sum_group(c, dst, std::integral_constant<int, 16>{}, std::integral_constant<int, 2>{});
                } else {
                    tmem_ld16(t_addr + c, dst);
                }
            };
            // bias, residual and store of 16 consecutive outputs of row m (tokens on the lanes, not gated)
            auto finish16 = [&](int m, int n0, float* v) {
                const size_t base = (size_t)m * p.N + n0;
                const bool full16 = n0 + 16 <= p.N;
                if (p.bias) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) if (n0 + i < p.N) v[i] += p.bias[n0 + i];
                }
                if (p.residual) {
                    if (full16 && (base & 7) == 0) {
                        const uint4* r4 = reinterpret_cast<const uint4*>(p.residual + base);
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const uint4 q = r4[h];
                            const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const float2 f = __bfloat1622float2(b2[i]);
                                v[h * 8 + 2 * i] += f.x;
                                v[h * 8 + 2 * i + 1] += f.y;
                            }
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 16; ++i) if (n0 + i < p.N) v[i] += __bfloat162float(p.residual[base + i]);
                    }
                }
                if (p.out_f32) {
                    float* o = reinterpret_cast<float*>(p.out) + base;
                    if (full16 && (base & 3) == 0) {
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            reinterpret_cast<float4*>(o)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
                    } else {
#pragma unroll
                        for (int i = 0; i < 16; ++i) if (n0 + i < p.N) o[i] = v[i];
                    }
                } else {
                    __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + base;
                    if (full16 && (base & 7) == 0) {
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            uint4 q;
                            __nv_bfloat162* b2 = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
                            for (int i = 0; i < 4; ++i) b2[i] = __floats2bfloat162_rn(v[h * 8 + 2 * i], v[h * 8 + 2 * i + 1]);
                            reinterpret_cast<uint4*>(o)[h] = q;
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 16; ++i) if (n0 + i < p.N) o[i] = __float2bfloat16_rn(v[i]);
                    }
                }
            };
            if (!SWAP && p.splits > 1) {
                // Tokens on the lanes with a cut k loop (few tiles, many tokens): every unit of a tile
                // leaves its partial accumulator in scratch, waits until the other units of the tile have
                // done so (they all run at once: the host launches one CTA per unit and no more units than
                // SMs), then adds up and finishes its share of the columns, every 16-column chunk c with
                // c mod splits == split, in split order. The sum is spread over the units instead of being
                // left to the last one.
                // scratch layout [split][column / 4][row][4 columns]: the 32 lanes of a warp (32 rows) write and
                // read 512 consecutive bytes with every 16-byte access
                float4* tile_part = reinterpret_cast<float4*>(p.partials + (size_t)tile * p.splits * BM * BN);
                float4* mine = tile_part + (size_t)split * (BN / 4) * BM + row_in_tile;
                for (int c = 0; c < BN; c += 16) {
                    tmem_ld16(t_addr0 + c, v);
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        __stcg(mine + (size_t)(c / 4 + q) * BM, make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]));
                }
                tmem_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(acc_empty_bar(as));
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (threadIdx.x == 64) {
                    __threadfence();
                    atomicAdd(p.counters + tile, 1);
                    int all_there = 1;
                    const long long t_start = clock64();
                    for (uint32_t spin = 1; *reinterpret_cast<volatile int*>(p.counters + tile) < p.splits; ++spin) {
                        __nanosleep(100);
                        if ((spin & 63u) == 0u && (*abort_flag || clock64() - t_start > 4000000000ll)) { all_there = 0; break; }
                    }
                    __threadfence();
                    *reinterpret_cast<volatile int*>(&exch[C::EXCH_FLOATS - 1]) = all_there;
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                const int all_there = *reinterpret_cast<volatile int*>(&exch[C::EXCH_FLOATS - 1]);
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (!all_there) {                                  // a unit of the tile never came: give up, loudly
                    *abort_flag = 1;
                    if (p.status && threadIdx.x == 64) atomicExch(p.status, 15);
                    ok = false;
                    break;
                }
                const int m = r0 + row_in_tile;
                for (int ch = split; ch < BN / 16; ch += p.splits) {
                    const int n0 = c0 + ch * 16;
                    if (n0 >= p.N) break;
#pragma unroll
                    for (int i = 0; i < 16; ++i) v[i] = 0.f;
                    for (int sp0 = 0; sp0 < p.splits; sp0 += 4) {
                        float4 part[4][4];
#pragma unroll
                        for (int sp = 0; sp < 4; ++sp) {
                            const bool in = sp0 + sp < p.splits;
                            const float4* src = tile_part + ((size_t)(in ? sp0 + sp : 0) * (BN / 4) + ch * 4) * BM + row_in_tile;
#pragma unroll
                            for (int q = 0; q < 4; ++q) part[sp][q] = in ? __ldcg(src + (size_t)q * BM) : make_float4(0.f, 0.f, 0.f, 0.f);
                        }
#pragma unroll
                        for (int sp = 0; sp < 4; ++sp) {
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                v[4 * q] += part[sp][q].x; v[4 * q + 1] += part[sp][q].y;
                                v[4 * q + 2] += part[sp][q].z; v[4 * q + 3] += part[sp][q].w;
                            }
                        }
                    }
                    if (m < p.M) finish16(m, n0, v);
                }
                // second arrival: when every unit has read what it needs, the last one clears the counter
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (threadIdx.x == 64) {
                    if (atomicAdd(p.counters + tile, 1) == 2 * p.splits - 1) p.counters[tile] = 0;
                }
                continue;
            }
            if (!SWAP) {
              for (int hm = 0; hm < TM; ++hm) {                 // the tile's accumulators of 128 rows, one after the other
                const uint32_t t_addr = t_addr0 + hm * BN;
                const int m = r0 + hm * BM + row_in_tile;
                const bool row_ok = m < p.M;
                if (!p.gated) {
                    for (int c = 0; c < BN; c += 16) {
                        tmem_ld16(t_addr + c, v);
                        const int n0 = c0 + c;
                        if (!row_ok || n0 >= p.N) continue;
                        finish16(m, n0, v);
                    }
                } else {
                    // columns [0, BN/2) hold the gate, [BN/2, BN) the up projection of the same outputs
                    for (int c = 0; c < BN / 2; c += 16) {
                        tmem_ld16(t_addr + c, v);
                        tmem_ld16(t_addr + BN / 2 + c, u);
                        const int j0 = c0 + c;
                        if (!row_ok || j0 >= p.N) continue;
                        __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + (size_t)m * p.N + j0;
#pragma unroll
                        for (int i = 0; i < 16; ++i) v[i] = silu_mul(v[i], u[i]);
                        if (j0 + 16 <= p.N && (((size_t)m * p.N + j0) & 7) == 0) {
#pragma unroll
                            for (int h = 0; h < 2; ++h) {
                                uint4 q;
                                __nv_bfloat162* b2 = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
                                for (int i = 0; i < 4; ++i) b2[i] = __floats2bfloat162_rn(v[h * 8 + 2 * i], v[h * 8 + 2 * i + 1]);
                                reinterpret_cast<uint4*>(o)[h] = q;
                            }
                        } else {
#pragma unroll
                            for (int i = 0; i < 16; ++i) if (j0 + i < p.N) o[i] = __float2bfloat16_rn(v[i]);
                        }
                    }
                }
              }
            } else {
                // swapped: this thread owns output feature n, the columns are tokens
                if (!p.gated) {
                    const int n = r0 + row_in_tile;
                    const bool n_ok = n < p.N;
                    const float b = (p.bias && n_ok) ? p.bias[n] : 0.f;
                    for (int c = 0; c < BN; c += 16) {
                        // the residual may be the output itself: all of it is read before anything is stored,
                        // and the reads are in flight together with those of the partials
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const int m = c0 + c + i;
                            u[i] = (p.residual && n_ok && m < p.M) ? __bfloat162float(p.residual[(size_t)m * p.N + n]) : 0.f;
                        }
                        load_chunk(c, v);
                        if (!n_ok) continue;
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const int m = c0 + c + i;
                            if (m < p.M) {
                                const float val = v[i] * row_scale_sh[c + i] + b + u[i];
                                const size_t idx = (size_t)m * p.N + n;
                                if (p.out_f32) reinterpret_cast<float*>(p.out)[idx] = val;
                                else reinterpret_cast<__nv_bfloat16*>(p.out)[idx] = __float2bfloat16_rn(val);
                            }
                        }
                    }
                } else {
                    // lanes 0..63 hold gate rows j0..j0+63, lanes 64..127 the matching up rows:
                    // the up half goes through shared memory to the threads that hold the gate
                    const bool is_up = row_in_tile >= 64;
                    const int jj = row_in_tile & 63;
                    for (int c = 0; c < BN; c += 16) {
                        load_chunk(c, v);
#pragma unroll
                        for (int i = 0; i < 16; ++i) v[i] *= row_scale_sh[c + i];        // gate and up alike
                        if (is_up) {
#pragma unroll
                            for (int i = 0; i < 16; ++i) exch[jj * 17 + i] = v[i];
                        }
                        asm volatile("bar.sync 1, 128;" ::: "memory");
                        if (!is_up) {
                            const int j = r0 + jj;
                            if (j < p.N) {
#pragma unroll
                                for (int i = 0; i < 16; ++i) {
                                    const int m = c0 + c + i;
                                    if (m >= p.M) break;
                                    reinterpret_cast<__nv_bfloat16*>(p.out)[(size_t)m * p.N + j] =
                                        __float2bfloat16_rn(silu_mul(v[i], exch[jj * 17 + i]));
                                }
                            }
                        }
                        asm volatile("bar.sync 1, 128;" ::: "memory");
                    }
                }
            }
            if (!released) {
                tmem_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(acc_empty_bar(as));   // this half of tensor memory may be overwritten
            }
        }
    }

    // ---------------------------------------------------------------- common exit
    tmem_fence_before();
    __syncthreads();
    if (warp == 1) {
        tmem_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)C::TMEM_COLS) : "memory");
    }
}

// ---------------------------------------------------------------------------- host side
// How many work units to cut a tile's k range into, so that the units fill the SMs evenly:
// a decode step is bound by how fast all SMs together can stream the weights, and 32 or 48 tiles
// leave most of the 148 SMs idle. Needs scratch for the partial sums.
// share_sum: the units of a tile add up together (see GemmParams), so the sum costs little and as many
// units as run side by side pay (measured at 64 tokens, 4096 x 4096: 9 cuts 12.6 us, 4 cuts 15.1 us,
// 4 cuts added up by the last unit alone 17.9 us).
int choose_splits(int tiles, int num_kb, int bn, long long workspace_floats, int num_counters, bool share_sum) {
    if (tiles > num_counters) return 1;
    const int per_sm = bn <= 64 ? 2 : 1;                  // Cfg<BN>::CTAS_PER_SM
    const int sms = ti_sm_count() * per_sm;               // CTAs that run side by side
    if (tiles * 2 >= sms) return 1;                       // every SM has a tile: cutting them only adds the merge
    if (share_sum) {
        int s = sms / tiles;
        s = s < 12 ? s : 12;
        s = s < num_kb / 4 ? s : num_kb / 4;
        while (s > 1 && (long long)tiles * s * bn * BM > workspace_floats) --s;
        return s > 1 ? s : 1;
    }
    int best = 1;
    double best_eff = 0.0;
    for (int s = 1; s <= 8; ++s) {
        if (s > 1 && (num_kb / s < 4 || (long long)tiles * s * bn * BM > workspace_floats)) break;
        // partial sums must stay small beside the weights, unless the tiles alone leave most SMs idle
        if (s > 1 && s * bn * 40 > num_kb * BK && (tiles * 2 >= sms || s > 4)) break;
        const long long units = (long long)tiles * s;
        const double eff = (double)units / (double)(((units + sms - 1) / sms) * sms);
        if (eff > best_eff + 0.04) { best_eff = eff; best = s; }
    }
    return best;
}

template <int BN, int TM = 1, bool SWAP = false>
int launch(const CUtensorMap& rows_map, const CUtensorMap& cols_map, const GemmParams& p, int num_tiles, cudaStream_t stream) {
    using C = Cfg<BN, TM>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, TM, SWAP>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
        if (e != cudaSuccess) { ti_set_error("gemm_tcgen05: cannot get %d bytes of shared memory: %s", C::SMEM_BYTES, cudaGetErrorString(e)); return (int)e; }
        configured = true;
    }
    num_tiles *= p.splits;
    const int slots = ti_sm_count() * C::CTAS_PER_SM;
    const int grid = num_tiles < slots ? num_tiles : slots;
    ti_launch(gemm_tcgen05_kernel<BN, TM, SWAP>, grid, NUM_THREADS, C::SMEM_BYTES, stream, rows_map, cols_map, p);
    TI_CHECK_LAUNCH("gemm_tcgen05");
    return 0;
}

}  // namespace

// 1 if ti_gemm_bf16 takes this shape (K a multiple of 8 so that rows start on 16-byte boundaries).
TI_API int ti_gemm_bf16_supported(int M, int N, int K) { return (M > 0 && N > 0 && K > 0 && K % 8 == 0) ? 1 : 0; }

// y = x . w^T in bfloat16 with float32 accumulation. gated: w is [2N, K] (gate rows, then up rows),
// out [M, N] = silu(x.gate) * (x.up). out_f32: out is float32. status: device word set if a wait ran out.
// workspace / counters: float32 scratch and zeroed int32 words for the split-k path of small M (may be
// null: then no tile is split). Calls that share them must be ordered on one stream.
struct NormLink {                  // an RMSNorm spread over two products (see GemmParams)
    const float* scale_sums = nullptr;
    int scale_parts = 0, scale_dim = 0;
    float scale_eps = 0.f;
    const float* emit_g = nullptr;
    void* emit_xg = nullptr;
    float* emit_sums = nullptr;
    int* emitted_parts = nullptr;  // host: how many parts of emit_sums were written (0: this shape cannot)
};

static int gemm_entry(void* out, const void* x, const void* w, const float* bias, const void* residual,
                      int M, int N, int K, int gated, int out_f32, float* workspace, long long workspace_floats,
                      int* counters, int num_counters, const NormLink& link, int* status, cudaStream_t stream);

TI_API int ti_gemm_bf16(void* out, const void* x, const void* w, const float* bias, const void* residual,
                        int M, int N, int K, int gated, int out_f32, float* workspace, long long workspace_floats,
                        int* counters, int num_counters, int* status, cudaStream_t stream) {
    return gemm_entry(out, x, w, bias, residual, M, N, K, gated, out_f32, workspace, workspace_floats, counters,
                      num_counters, NormLink(), status, stream);
}

// The same product for at most 64 tokens as one half of an RMSNorm spread over two products.
// scale_sums (may be null): x holds rows of scale_dim elements times the norm's weights, NOT divided by their
// rms; scale_sums [scale_parts][M] are partial sums of squares of the rows before the weights; every output
// row is multiplied by rsqrt(sum / scale_dim + scale_eps) (before bias and residual).
// emit_g (may be null): the weights [N] of the norm that follows this product; emit_xg [M, N] receives
// out * emit_g (of out as rounded to bfloat16), emit_sums [ceil(N / 128)][M] the sums of squares of out per
// 128 outputs; *emitted_parts says how many parts were written, 0 if this shape does not take the path
// that can (then the caller runs the norm kernel).
TI_API int ti_gemm_bf16_linked(void* out, const void* x, const void* w, const float* bias, const void* residual,
                               int M, int N, int K, int gated, float* workspace, long long workspace_floats,
                               int* counters, int num_counters, const float* scale_sums, int scale_parts,
                               int scale_dim, float scale_eps, const float* emit_g, void* emit_xg, float* emit_sums,
                               int* emitted_parts, int* status, cudaStream_t stream) {
    NormLink link;
    link.scale_sums = scale_sums; link.scale_parts = scale_parts; link.scale_dim = scale_dim; link.scale_eps = scale_eps;
    link.emit_g = emit_g; link.emit_xg = emit_xg; link.emit_sums = emit_sums; link.emitted_parts = emitted_parts;
    return gemm_entry(out, x, w, bias, residual, M, N, K, gated, 0, workspace, workspace_floats, counters,
                      num_counters, link, status, stream);
}

// The pair form (gemm_pair_tcgen05.cu): two CTAs a 256 x 256 tile.
TI_API int ti_gemm_pair_bf16(void* out, const void* x, const void* w, const float* bias, const void* residual,
                             int M, int N, int K, int gated, int out_f32, int* status, cudaStream_t stream);
static int g_pair_form = 1;      // 0: never, 1: where it was measured to be faster
// Whether ti_gemm_bf16 may hand steps of many tokens to the pair form (for measurements; the default is yes).
TI_API void ti_gemm_set_pair_form(int mode) { g_pair_form = mode; }

static int gemm_entry(void* out, const void* x, const void* w, const float* bias, const void* residual,
                      int M, int N, int K, int gated, int out_f32, float* workspace, long long workspace_floats,
                      int* counters, int num_counters, const NormLink& link, int* status, cudaStream_t stream) {
    if (link.emitted_parts) *link.emitted_parts = 0;
    // Many tokens: the pair form, from 512 tokens on where its 256 x 256 tiles are at least 48 (measured on a
    // B200 at Qwen3-8B's widths: 768 to 8,192 tokens 6 to 17 % faster for all four products of a layer; at
    // 512 tokens faster with 48 tiles and more, slower with 32, where the one-CTA form cuts its k loops; at
    // 384 tokens and fewer slower, half of a second row of tiles being empty).
    if (g_pair_form && M >= 512 && K % 8 == 0 && (gated ? 2 * N : N) >= 256 && link.scale_sums == nullptr &&
        link.emit_g == nullptr && ((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0) {
        const long long pair_tiles = (long long)((M + 255) / 256) * ((N + (gated ? 127 : 255)) / (gated ? 128 : 256));
        if (pair_tiles >= 48)
            return ti_gemm_pair_bf16(out, x, w, bias, residual, M, N, K, gated, out_f32, status, stream);
    }
    TI_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm_bf16: bad sizes M=%d N=%d K=%d", M, N, K);
    TI_REQUIRE(link.scale_sums == nullptr || (M <= 64 && link.scale_parts > 0 && link.scale_dim > 0),
               "gemm_bf16: rows can be scaled by their rms for at most 64 tokens");
    TI_REQUIRE(K % 8 == 0, "gemm_bf16: K=%d is not a multiple of 8 (rows must start on 16-byte boundaries)", K);
    TI_REQUIRE(!(gated && (bias || residual || out_f32)), "gemm_bf16: the gated form takes no bias, residual or float32 output");
    TI_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0, "gemm_bf16: operands must be 16-byte aligned");
    if (M == 0) return 0;
    GemmParams p;
    p.out = out; p.bias = bias; p.residual = (const __nv_bfloat16*)residual;
    p.M = M; p.N = N; p.K = K; p.gated = gated; p.out_f32 = out_f32; p.status = status;
    p.splits = 1; p.share_sum = 0; p.partials = workspace; p.counters = counters;
    p.scale_sums = link.scale_sums; p.scale_parts = link.scale_parts; p.scale_dim = link.scale_dim;
    p.scale_eps = link.scale_eps;
    p.emit_g = nullptr; p.emit_xg = nullptr; p.emit_sums = nullptr;
    const int w_rows = gated ? 2 * N : N;
    CUtensorMap rows_map, cols_map;
    // Up to 128 tokens the weights go on the 128 accumulator lanes and the tokens on the columns: with
    // so few tokens the other orientation has one row of tiles, too few for 148 SMs, and no way to
    // cut their k loops. (The gated form keeps its 64-column limit; it has tiles enough. Beyond 128
    // tokens the partial sums of the cut k loops cost more than the idle SMs: measured.)
    if (M <= 64 || (!gated && M <= 128 && workspace && counters)) {
        p.swap = 1;
        p.rows_total = N; p.cols_total = M;
        const int bn = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128));
        if (!ti_get_bf16_map(w, w_rows, K, gated ? BM / 2 : BM, &rows_map)) return -1;
        if (!ti_get_bf16_map(x, M, K, bn, &cols_map)) return -1;
        const int tiles = (N + (gated ? 64 : 128) - 1) / (gated ? 64 : 128);
        // From 16 tokens on the sum over the cut k loops is shared out among the units of a tile (the
        // last unit alone makes a trip to L2 per few tokens, one after the other; up to 8 tokens that is
        // one trip and sharing only adds the wait: measured). Needs every unit running at once, and the
        // 16-byte path of the sum.
        const bool may_share = M >= 16 && (N & 3) == 0 &&
                               (gated ? ((uintptr_t)out & 7) == 0
                                      : ((uintptr_t)out & 15) == 0 && ((uintptr_t)residual & 7) == 0 && ((uintptr_t)bias & 15) == 0);
        if (workspace && counters)
            p.splits = choose_splits(tiles, (K + BK - 1) / BK, bn, workspace_floats, num_counters, may_share);
        if (may_share && p.splits > 1 && (long long)tiles * p.splits <= (long long)ti_sm_count() * (bn <= 64 ? 2 : 1))
            p.share_sum = 1;
        // the scaled rows and the sums are written by the last unit of a cut k loop, on its 16-byte path
        if (link.emit_g && link.emit_xg && link.emit_sums && !gated && !out_f32 && p.splits > 1 && (N & 3) == 0 &&
            ((uintptr_t)out & 15) == 0 && ((uintptr_t)residual & 7) == 0 && ((uintptr_t)bias & 15) == 0 &&
            ((uintptr_t)link.emit_g & 15) == 0 && ((uintptr_t)link.emit_xg & 7) == 0) {
            p.emit_g = link.emit_g; p.emit_xg = (__nv_bfloat16*)link.emit_xg; p.emit_sums = link.emit_sums;
            if (link.emitted_parts) *link.emitted_parts = tiles;
        }
        if (bn == 16) return launch<16, 1, true>(rows_map, cols_map, p, tiles, stream);
        if (bn == 32) return launch<32, 1, true>(rows_map, cols_map, p, tiles, stream);
        if (bn == 64) return launch<64, 1, true>(rows_map, cols_map, p, tiles, stream);
        return launch<128, 1, true>(rows_map, cols_map, p, tiles, stream);
    }
    p.swap = 0;
    p.rows_total = M; p.cols_total = N;
    if (!ti_get_bf16_map(x, M, K, BM, &rows_map)) return -1;
    const int row_tiles = (M + BM - 1) / BM;
    // 256 columns a tile, unless the output is narrow or, with so few tiles that half the SMs would
    // have none, twice as many tiles of 128 columns finish sooner (a tile of half the width does not
    // run faster per k step, but twice as many SMs work)
    bool wide = (gated ? 2 * N : N) >= 256;
    if (wide) {
        const int cpt256 = gated ? 128 : 256;
        const long long tiles256 = (long long)row_tiles * ((N + cpt256 - 1) / cpt256);
        // Few tiles, many tokens (about 130 to 700 of them): the k loops are cut so that as many units as
        // there are SMs run at once, and the units of a tile add their partial sums up together.
        const int sms = ti_sm_count(), num_kb = (K + BK - 1) / BK;
        if (!gated && workspace && counters && tiles256 <= num_counters && tiles256 * 2 <= sms) {
            int cut = (int)(sms / tiles256);
            cut = cut < 8 ? cut : 8;
            cut = cut < num_kb / 8 ? cut : num_kb / 8;
            while (cut > 1 && tiles256 * cut * BM * 256 > workspace_floats) --cut;
            if (cut > 1) {
                p.splits = cut;
                if (!ti_get_bf16_map(w, w_rows, K, 256, &cols_map)) return -1;
                return launch<256>(rows_map, cols_map, p, (int)tiles256, stream);
            }
        }
        if (tiles256 * 2 <= sms) wide = false;
    }
    if (wide) {
        if (!ti_get_bf16_map(w, w_rows, K, gated ? 128 : 256, &cols_map)) return -1;
        const int cpt = gated ? 128 : 256;
        const long long col_tiles = (N + cpt - 1) / cpt;
        // 256 x 256 tiles if they finish sooner: a wave of them was measured to take 1.77 times a wave of
        // 128 x 256 tiles (twice the MMAs for 4/3 of the operand bytes, but three stages of 64 KB keep
        // fewer bytes in flight than four of 48 KB, and no epilogue runs behind the next tile's MMAs).
        // Inside a prefill step they paid from about 3,000 tokens on (4,096 tokens: 7.5 % off the step;
        // 2,048 tokens: 2 % on, although the products alone were faster), hence the lower bound.
        const int sms = ti_sm_count();
        const long long tall_tiles = (long long)((M + 2 * BM - 1) / (2 * BM)) * col_tiles;
        const long long waves = (row_tiles * col_tiles + sms - 1) / sms, tall_waves = (tall_tiles + sms - 1) / sms;
        const bool tall = M >= 3072 && tall_waves * 177 < waves * 100;
        if (tall) {
            if (!ti_get_bf16_map(x, M, K, 2 * BM, &rows_map)) return -1;
            return launch<256, 2>(rows_map, cols_map, p, (int)tall_tiles, stream);
        }
        return launch<256>(rows_map, cols_map, p, row_tiles * ((N + cpt - 1) / cpt), stream);
    }
    if (!ti_get_bf16_map(w, w_rows, K, gated ? 64 : 128, &cols_map)) return -1;
    const int cpt = gated ? 64 : 128;
    return launch<128>(rows_map, cols_map, p, row_tiles * ((N + cpt - 1) / cpt), stream);
}
