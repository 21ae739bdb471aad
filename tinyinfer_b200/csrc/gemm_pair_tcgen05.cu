// bfloat16 matrix product y[M,N] = x[M,K] . w[N,K]^T for many tokens, in the pair form of the 5th-generation
// tensor cores (tcgen05.mma.cta_group::2): a cluster of two CTAs on the two SMs of a TPC computes one
// 256 x 256 output tile. Each CTA holds 128 of the tile's 256 token rows (its own A operand) and HALF of the
// tile's 256 weight rows (its half of the B operand); the MMA, issued by one thread of the even CTA, reads
// both halves of B across the pair and writes rows 0..127 of the accumulator into the even CTA's tensor
// memory and rows 128..255 into the odd one's. A CTA so takes in 32 KB of operands per 64-wide k block
// for 512 cycles of MMAs, where a lone CTA with a 128 x 256 tile takes in 48 KB: an SM gets about
// 64 bytes a cycle from L2, and that, not the tensor pipe, bounds the one-CTA form (gemm_tcgen05.cu).
//
//   warp 0 (both CTAs)   TMA: its 128 rows of x and its 128 rows of w per k block into a ring of six stages;
//                        the copies of BOTH CTAs complete on the even CTA's barrier (no multicast: every CTA
//                        loads what it alone holds). Weights of the first ring are requested before the wait
//                        for the kernels ahead in the stream.
//   warp 1 (even CTA)    one thread issues the MMAs (256 x 256 x 16) and commits to the barriers of both CTAs
//                        (tcgen05.commit with multicast): stage free, accumulator full.
//   warps 2..5 (both)    epilogue of tile i from one half of tensor memory while the MMAs of tile i+1 fill
//                        the other: + bias[n], + residual[m,n], float32 output, or the gated form
//                        out[m,j] = silu(x.w[j]) * (x.w[J+j]) (the even CTA's half of B holds 128 gate rows, the
//                        odd one's the 128 up rows of the same outputs). All on the float32 accumulators,
//                        one rounding. They tell the even CTA's MMA thread when their half is read.
//
// A row's result does not depend on which other rows share its tile: every output element is one k loop in
// a fixed order. Every wait is bounded (status word, abort flag); the two CTAs leave together (cluster
// barrier) and free their tensor memory on the common exit. The formulas are those of gemm_tcgen05.cu
// (tinyinfer/csrc/mlp.cu:116-141 for the gated form).
#include "sm100_ptx.cuh"

namespace {

constexpr int BM = 128;              // rows of x a CTA holds = its accumulator lanes
constexpr int BN = 256;              // columns of the pair's tile
constexpr int BK = 64;               // bf16 elements per 128-byte swizzled row
constexpr int STAGES = 6;
constexpr int STAGE_BYTES = (BM + BN / 2) * BK * 2;          // 32 KB: 128 rows of x, 128 rows of w
constexpr int NUM_THREADS = 192;
constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + 256;

struct PairGemmParams {
    void* out;
    const float* bias;
    const __nv_bfloat16* residual;
    int M, N, K;                     // out is [M, N] (gated: N = J, w has 2J rows)
    int gated, out_f32;
    int* status;
};

__device__ __forceinline__ float silu_mul(float g, float u) { return (g / (1.f + __expf(-g))) * u; }
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_id_x() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%clusterid.x;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t num_clusters_x() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%nclusterid.x;" : "=r"(r));
    return r;
}
// The address, in the cluster's window, of this shared-memory address in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// A TMA copy into this CTA's shared memory whose bytes are counted on a barrier of the pair's even CTA.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrives, once the MMAs issued so far are done, on the barrier at this offset in BOTH CTAs of the pair.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"((unsigned short)3) : "memory");
}
// 32 columns of this warp's 32 accumulator lanes into registers; the values are there after tmem_ld_wait().
__device__ __forceinline__ void tmem_ld32_issue(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_in_cluster_window) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_in_cluster_window) : "memory");
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, const PairGemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* stages = smem;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
    // barrier layout: full[STAGES] (used in the even CTA), empty[STAGES], acc_full[2], acc_empty[2] (even CTA)
    const uint32_t bar0 = smem_u32(bars);
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES + s); };
    auto acc_full_bar = [&](int a) { return bar0 + 8u * (2 * STAGES + a); };
    auto acc_empty_bar = [&](int a) { return bar0 + 8u * (2 * STAGES + 2 + a); };
    __shared__ uint32_t tmem_base_sh;
    __shared__ int abort_sh;
    volatile int* abort_flag = &abort_sh;

    ti_grid_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();
    const int cols_per_tile = p.gated ? BN / 2 : BN;
    const int row_tiles = (p.M + 2 * BM - 1) / (2 * BM);
    const int col_tiles = (p.N + cols_per_tile - 1) / cols_per_tile;
    const int num_tiles = row_tiles * col_tiles;
    const int num_kb = (p.K + BK - 1) / BK;
    const int first_tile = (int)cluster_id_x(), tile_step = (int)num_clusters_x();

    if (threadIdx.x == 0) {
        abort_sh = 0;
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(acc_full_bar(a), 1); mbar_init(acc_empty_bar(a), 8); }   // four warps of each CTA
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {        // one warp of EACH CTA of the pair takes part in the allocation
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_base_sh)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tmem_fence_before();
    __syncthreads();
    cluster_sync_all();                                  // the other CTA's barriers and tensor memory are there too
    tmem_fence_after();
    const uint32_t tmem_base = tmem_base_sh;

    // tile -> first token row of the PAIR's tile, first output column
    auto tile_origin = [&](int tile, int& r0, int& c0) {
        r0 = (tile % row_tiles) * (2 * BM);
        c0 = (tile / row_tiles) * cols_per_tile;
    };

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (both CTAs)
        if (lane == 0) {
            const uint32_t full0 = map_to_cta(bar0, 0);                  // the even CTA's full[0]
            auto issue_w = [&](int c0, int kb, int s) {
                // this CTA's half of the tile's weight rows: plain, rows c0 + 128 rank ..; gated, the even CTA takes
                // the 128 gate rows c0 .., the odd one the 128 up rows N + c0 ..
                const int row = p.gated ? (rank == 0 ? c0 : p.N + c0) : c0 + (int)rank * (BN / 2);
                tma_load_2d_pair(smem_u32(stages + s * STAGE_BYTES) + BM * BK * 2, &map_w, full0 + 8u * s, kb * BK, row);
            };
            auto issue_x = [&](int r0, int kb, int s) {
                tma_load_2d_pair(smem_u32(stages + s * STAGE_BYTES), &map_x, full0 + 8u * s, kb * BK, r0 + (int)rank * BM);
            };
            // Before waiting for the kernels ahead of this one in the stream: the weights do not depend on
            // them. The even CTA announces the bytes of both CTAs' copies of a stage.
            uint32_t pre = 0;
            for (int tile = first_tile; tile < num_tiles && pre < (uint32_t)STAGES; tile += tile_step) {
                int r0, c0;
                tile_origin(tile, r0, c0);
                for (int kb = 0; kb < num_kb && pre < (uint32_t)STAGES; ++kb, ++pre) {
                    if (rank == 0) mbar_expect_tx(full_bar(pre), 2 * STAGE_BYTES);
                    issue_w(c0, kb, pre);
                }
            }
            ti_grid_wait();
            uint32_t it = 0;
            bool ok = true;
            for (int tile = first_tile; tile < num_tiles && ok; tile += tile_step) {
                int r0, c0;
                tile_origin(tile, r0, c0);
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (it < pre) { issue_x(r0, kb, s); continue; }      // its weights are already on their way
                    if (!mbar_wait(empty_bar(s), ((it / STAGES) & 1u) ^ 1u, abort_flag, p.status, 61)) { ok = false; break; }
                    if (rank == 0) mbar_expect_tx(full_bar(s), 2 * STAGE_BYTES);
                    issue_x(r0, kb, s);
                    issue_w(c0, kb, s);
                }
            }
            if (!ok) {       // give the copies still in flight time to land before shared memory is given up
                const unsigned long long t0 = global_ns();
                while (global_ns() - t0 < 1000000ull) {}
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (even CTA)
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = make_idesc(2 * BM, BN);
            uint32_t it = 0, tile_i = 0;
            bool ok = true;
            for (int tile = first_tile; tile < num_tiles && ok; tile += tile_step, ++tile_i) {
                const uint32_t as = tile_i & 1u, aph = (tile_i >> 1) & 1u;
                if (!mbar_wait(acc_empty_bar(as), aph ^ 1u, abort_flag, p.status, 62)) { ok = false; break; }
                tmem_fence_after();
                const uint32_t d_tmem = tmem_base + as * BN;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait(full_bar(s), (it / STAGES) & 1u, abort_flag, p.status, 63)) { ok = false; break; }
                    tmem_fence_after();
                    const uint32_t a_addr = smem_u32(stages + s * STAGE_BYTES);
                    const uint64_t adesc = make_sw128_desc(a_addr);
                    const uint64_t bdesc = make_sw128_desc(a_addr + BM * BK * 2);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k)
                        umma_bf16_pair(d_tmem, adesc + 2u * k, bdesc + 2u * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    umma_commit_pair(empty_bar(s));          // the stage is free, in both CTAs, once these MMAs have read it
                }
                if (ok) umma_commit_pair(acc_full_bar(as));  // the accumulator is complete, in both CTAs
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
        ti_grid_wait();                                  // residual and out belong to earlier kernels until now
        const int lane_group = warp & 3;                 // the 32 accumulator lanes this warp may read
        const int row_in_tile = lane_group * 32 + lane;
        const uint32_t acc_empty0 = map_to_cta(acc_empty_bar(0), 0);
        // bias, residual and store of 16 consecutive outputs n0.. of token row m (the general path: ragged edges,
        // float32 output, rows that do not start on 16-byte boundaries)
        auto finish16 = [&](int m, int n0, float* v) {
            const size_t base = (size_t)m * p.N + n0;
            if (p.bias) {
#pragma unroll
                for (int i = 0; i < 16; ++i) if (n0 + i < p.N) v[i] += p.bias[n0 + i];
            }
            if (p.residual) {
#pragma unroll
                for (int i = 0; i < 16; ++i) if (n0 + i < p.N) v[i] += __bfloat162float(p.residual[base + i]);
            }
            if (p.out_f32) {
                float* o = reinterpret_cast<float*>(p.out) + base;
                if (n0 + 16 <= p.N && (base & 3) == 0) {
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        reinterpret_cast<float4*>(o)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
                } else {
#pragma unroll
                    for (int i = 0; i < 16; ++i) if (n0 + i < p.N) o[i] = v[i];
                }
            } else {
                __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + base;
                if (n0 + 16 <= p.N && (base & 7) == 0) {
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
        uint32_t tile_i = 0;
        bool ok = true;
        for (int tile = first_tile; tile < num_tiles && ok; tile += tile_step, ++tile_i) {
            int r0, c0;
            tile_origin(tile, r0, c0);
            const uint32_t as = tile_i & 1u, aph = (tile_i >> 1) & 1u;
            if (!mbar_wait(acc_full_bar(as), aph, abort_flag, p.status, 64)) { ok = false; break; }
            tmem_fence_after();
            const uint32_t t_addr = tmem_base + as * BN + ((uint32_t)(lane_group * 32) << 16);
            const int m = r0 + (int)rank * BM + row_in_tile;
            const bool row_ok = m < p.M;
            // 64 columns at a time: two tensor-memory loads and the row's residual are asked for together and
            // waited for once (the epilogue of a pair's last tile has no MMAs to hide behind: every wait of it
            // is the kernel's time)
            if (!p.gated) {
                for (int c = 0; c < BN; c += 64) {
                    uint32_t r[64];
                    tmem_ld32_issue(t_addr + c, r);
                    tmem_ld32_issue(t_addr + c + 32, r + 32);
                    const int n0 = c0 + c;
                    const size_t base = (size_t)m * p.N + n0;
                    const bool whole = row_ok && !p.out_f32 && n0 + 64 <= p.N && (base & 7) == 0;
                    uint4 res[8];
                    if (whole && p.residual) {
#pragma unroll
                        for (int i = 0; i < 8; ++i) res[i] = reinterpret_cast<const uint4*>(p.residual + base)[i];
                    }
                    tmem_ld_wait();
                    float* v = reinterpret_cast<float*>(r);
                    if (whole) {
                        if (p.bias) {
#pragma unroll
                            for (int i = 0; i < 64; ++i) v[i] += p.bias[n0 + i];
                        }
                        uint4* o = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.out) + base);
#pragma unroll
                        for (int h = 0; h < 8; ++h) {
                            uint4 q;
                            __nv_bfloat162* b2 = reinterpret_cast<__nv_bfloat162*>(&q);
                            if (p.residual) {
                                const __nv_bfloat162* r2 = reinterpret_cast<const __nv_bfloat162*>(&res[h]);
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    const float2 f = __bfloat1622float2(r2[i]);
                                    b2[i] = __floats2bfloat162_rn(v[h * 8 + 2 * i] + f.x, v[h * 8 + 2 * i + 1] + f.y);
                                }
                            } else {
#pragma unroll
                                for (int i = 0; i < 4; ++i) b2[i] = __floats2bfloat162_rn(v[h * 8 + 2 * i], v[h * 8 + 2 * i + 1]);
                            }
                            o[h] = q;
                        }
                    } else if (row_ok) {
#pragma unroll
                        for (int g = 0; g < 4; ++g)
                            if (n0 + 16 * g < p.N) finish16(m, n0 + 16 * g, v + 16 * g);
                    }
                }
            } else {
                // columns [0, 128) hold the gate, [128, 256) the up projection of the same outputs
                for (int c = 0; c < BN / 2; c += 32) {
                    uint32_t rg[32], ru[32];
                    tmem_ld32_issue(t_addr + c, rg);
                    tmem_ld32_issue(t_addr + BN / 2 + c, ru);
                    tmem_ld_wait();
                    const int j0 = c0 + c;
                    if (!row_ok || j0 >= p.N) continue;
                    float* v = reinterpret_cast<float*>(rg);
                    const float* u = reinterpret_cast<const float*>(ru);
                    __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + (size_t)m * p.N + j0;
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = silu_mul(v[i], u[i]);
                    if (j0 + 32 <= p.N && (((size_t)m * p.N + j0) & 7) == 0) {
#pragma unroll
                        for (int h = 0; h < 4; ++h) {
                            uint4 q;
                            __nv_bfloat162* b2 = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
                            for (int i = 0; i < 4; ++i) b2[i] = __floats2bfloat162_rn(v[h * 8 + 2 * i], v[h * 8 + 2 * i + 1]);
                            reinterpret_cast<uint4*>(o)[h] = q;
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i) if (j0 + i < p.N) o[i] = __float2bfloat16_rn(v[i]);
                    }
                }
            }
            tmem_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(acc_empty0 + 8u * as);   // this half of tensor memory may be overwritten
        }
    }

    // ---------------------------------------------------------------- common exit
    tmem_fence_before();
    __syncthreads();
    cluster_sync_all();                  // nobody leaves while the other CTA's MMAs still read its shared memory or write its tensor memory
    if (warp == 1) {
        tmem_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

}  // namespace

// 1 if ti_gemm_pair_bf16 takes this shape.
TI_API int ti_gemm_pair_supported(int M, int N, int K, int gated) {
    return (M > 0 && N > 0 && K > 0 && K % 8 == 0 && (gated ? 2 * N : N) >= 256) ? 1 : 0;
}

// y = x . w^T in bfloat16 with float32 accumulation, in the pair form; for steps of many tokens. gated: w is
// [2N, K] (gate rows, then up rows), out [M, N] = silu(x.gate) * (x.up). out_f32: out is float32.
// status: device word set if a wait ran out.
TI_API int ti_gemm_pair_bf16(void* out, const void* x, const void* w, const float* bias, const void* residual,
                             int M, int N, int K, int gated, int out_f32, int* status, cudaStream_t stream) {
    TI_REQUIRE(ti_gemm_pair_supported(M, N, K, gated), "gemm_pair: shape %d x %d x %d not supported", M, N, K);
    TI_REQUIRE(!(gated && (bias || residual || out_f32)), "gemm_pair: the gated form takes no bias, residual or float32 output");
    CUtensorMap map_x, map_w;
    if (!ti_get_bf16_map(x, M, K, BM, &map_x)) return -1;
    if (!ti_get_bf16_map(w, gated ? 2 * N : N, K, BN / 2, &map_w)) return -1;
    PairGemmParams p;
    p.out = out; p.bias = bias; p.residual = (const __nv_bfloat16*)residual;
    p.M = M; p.N = N; p.K = K; p.gated = gated; p.out_f32 = out_f32; p.status = status;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        TI_REQUIRE(e == cudaSuccess, "gemm_pair: cannot get %d bytes of shared memory: %s", SMEM_BYTES, cudaGetErrorString(e));
        configured = true;
    }
    const int cols_per_tile = gated ? BN / 2 : BN;
    const long long tiles = (long long)((M + 2 * BM - 1) / (2 * BM)) * ((N + cols_per_tile - 1) / cols_per_tile);
    const int pairs = ti_sm_count() / 2;
    const int clusters = (int)(tiles < pairs ? tiles : pairs);
    ti_launch(gemm_pair_kernel, 2 * clusters, NUM_THREADS, SMEM_BYTES, stream, map_x, map_w, p);
    TI_CHECK_LAUNCH("gemm_pair");
    return 0;
}
