// bfloat16 matrix product y[M,N] = x[M,K] . w[N,K]^T on the 5th-generation tensor cores of
// sm_100a: operands staged in shared memory by TMA (128-byte swizzle, no multicast), one elected
// thread issuing tcgen05.mma, float32 accumulators in tensor memory, read back with tcgen05.ld for
// the epilogue. The kernel is persistent (one CTA per SM walks over output tiles) and warp
// specialised: warp 0 loads, warp 1 issues the MMAs, warps 2..5 run the epilogue of tile i while
// the MMAs of tile i+1 fill the other half of tensor memory.
//
// Two orientations share the code. "Rows" are the 128 accumulator lanes, "cols" the BN columns:
//   normal (many tokens):  rows = tokens of x, cols = output features of w;
//   swapped (M <= 64):     rows = output features of w, cols = tokens of x (padded to BN), so a
//                          decode step streams every weight once with full 128-row MMAs.
// Epilogues, all on the float32 accumulators with one rounding: + bias[n], + residual[m,n],
// float32 output (logits), and the gated form out[m,j] = silu(x.w[j]) * (x.w[J+j]) of the
// reference's MLP kernel (tinyinfer/csrc/mlp.cu:116-141). A row's result does not depend on
// which other rows share its tile: every output element is one fixed-order k loop.
//
// Every wait on an mbarrier is bounded; a wait that runs out sets *status, raises the CTA's abort
// flag, and all warps fall through to the common exit, where tensor memory is freed.
#include "common.cuh"
#include <cuda.h>
#include <mutex>
#include <unordered_map>

namespace {

constexpr int BM = 128;          // accumulator lanes = rows of the "rows" operand per tile
constexpr int BK = 64;           // bf16 elements per 128-byte swizzled row
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 192;
constexpr int SMEM_BUDGET = 200 * 1024;
constexpr unsigned long long WAIT_NS = 2000000000ull;   // a wait gives up after two seconds

struct GemmParams {
    void* out;
    const float* bias;
    const __nv_bfloat16* residual;
    int M, N, K;            // problem: out is [M, N] (gated: N = J, w has 2J rows)
    int rows_total;         // extent of the rows operand that tiles walk over
    int cols_total;         // extent of the cols operand
    int gated, out_f32, swap;
    int* status;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait. Returns false if the CTA is aborting or the wait ran out (then it raises the abort).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
    for (uint32_t i = 1;; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 255u) == 0u) {
            if (*abort_flag) return false;
            if (global_ns() - t0 > WAIT_NS) {
                *abort_flag = 1;
                if (status) atomicExch(status, code);
                return false;
            }
        }
    }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
// Shared-memory operand descriptor: K-major tile of rows x 64 bf16, 128-byte swizzle; rows are
// 128 bytes apart, groups of 8 rows 1024 bytes apart.
__device__ __forceinline__ uint64_t make_sw128_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;                 // leading byte offset: not used by swizzled K-major tiles
    d |= (uint64_t)(1024 >> 4) << 32;       // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                 // descriptor version of sm_100
    d |= (uint64_t)2 << 61;                 // SWIZZLE_128B
    return d;
}
// Instruction descriptor: bf16 x bf16 -> f32, both operands K-major, M x N tile.
__host__ __device__ constexpr uint32_t make_idesc(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ float silu_mul(float g, float u) { return (g / (1.f + __expf(-g))) * u; }

template <int BN>
struct Cfg {
    static constexpr int STAGE_BYTES = (BM + BN) * BK * 2;
    static constexpr int STAGES = (SMEM_BUDGET / STAGE_BYTES) > 12 ? 12 : (SMEM_BUDGET / STAGE_BYTES);
    static constexpr int TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;        // two accumulators; a power of two
    static constexpr int EXCH_FLOATS = 64 * (BN + 1);                   // swapped gated epilogue only
    static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + EXCH_FLOATS * 4 + 256;
};

template <int BN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_rows, const __grid_constant__ CUtensorMap map_cols,
                    const GemmParams p) {
    using C = Cfg<BN>;
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
    volatile int* abort_flag = &abort_sh;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // tiles: gated normal tiles hold BN/2 gate and BN/2 up columns; gated swapped tiles 64 + 64 rows
    const int rows_per_tile = (p.gated && p.swap) ? BM / 2 : BM;
    const int cols_per_tile = (p.gated && !p.swap) ? BN / 2 : BN;
    const int row_tiles = (p.rows_total + rows_per_tile - 1) / rows_per_tile;
    const int col_tiles = (p.cols_total + cols_per_tile - 1) / cols_per_tile;
    const int num_tiles = row_tiles * col_tiles;
    const int num_kb = (p.K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        abort_sh = 0;
        for (int s = 0; s < C::STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(acc_full_bar(a), 1); mbar_init(acc_empty_bar(a), 4); }
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
            uint32_t it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                const int rt = tile % row_tiles, ct = tile / row_tiles;
                const int r0 = rt * rows_per_tile, c0 = ct * cols_per_tile;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % C::STAGES;
                    const uint32_t ph = (it / C::STAGES) & 1u;
                    if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, p.status, 11)) { ok = false; break; }
                    const uint32_t a_dst = smem_u32(stages + s * C::STAGE_BYTES);
                    const uint32_t b_dst = a_dst + BM * BK * 2;
                    mbar_expect_tx(full_bar(s), C::STAGE_BYTES);
                    if (p.gated && p.swap) {          // 64 gate rows, then 64 up rows
                        tma_load_2d(a_dst, &map_rows, full_bar(s), kb * BK, r0);
                        tma_load_2d(a_dst + (BM / 2) * BK * 2, &map_rows, full_bar(s), kb * BK, p.N + r0);
                    } else {
                        tma_load_2d(a_dst, &map_rows, full_bar(s), kb * BK, r0);
                    }
                    if (p.gated && !p.swap) {         // BN/2 gate rows, then BN/2 up rows
                        tma_load_2d(b_dst, &map_cols, full_bar(s), kb * BK, c0);
                        tma_load_2d(b_dst + (BN / 2) * BK * 2, &map_cols, full_bar(s), kb * BK, p.N + c0);
                    } else {
                        tma_load_2d(b_dst, &map_cols, full_bar(s), kb * BK, c0);
                    }
                }
            }
            // On the way out no copy of this CTA may still be in flight: every stage it armed is
            // either consumed (normal end: the MMA warp waited on it) or awaited here, bounded.
            if (!ok) {
                for (int s = 0; s < C::STAGES; ++s) {
                    const unsigned long long t0 = global_ns();
                    const uint32_t armed = it > (uint32_t)s ? ((it - 1 - s) / C::STAGES) & 1u : 2u;
                    if (armed == 2u) continue;
                    while (!mbar_try_wait(full_bar((it - 1 - s) % C::STAGES), armed) && global_ns() - t0 < 1000000ull) {}
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(BM, BN);
            uint32_t it = 0, tile_i = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++tile_i) {
                const uint32_t as = tile_i & 1u, aph = (tile_i >> 1) & 1u;
                if (!mbar_wait(acc_empty_bar(as), aph ^ 1u, abort_flag, p.status, 12)) { ok = false; break; }
                tmem_fence_after();
                const uint32_t d_tmem = tmem_base + as * BN;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % C::STAGES;
                    const uint32_t ph = (it / C::STAGES) & 1u;
                    if (!mbar_wait(full_bar(s), ph, abort_flag, p.status, 13)) { ok = false; break; }
                    tmem_fence_after();
                    const uint32_t a_addr = smem_u32(stages + s * C::STAGE_BYTES);
                    const uint64_t adesc = make_sw128_desc(a_addr);
                    const uint64_t bdesc = make_sw128_desc(a_addr + BM * BK * 2);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        // 16 bf16 = 32 bytes along K inside the 128-byte swizzled row: +2 in 16-byte units
                        umma_bf16(d_tmem, adesc + 2u * k, bdesc + 2u * k, idesc, (kb | k) != 0 ? 1u : 0u);
                    }
                    umma_commit(empty_bar(s));           // the stage is free once these MMAs have read it
                }
                if (ok) umma_commit(acc_full_bar(as));   // the accumulator is complete
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..5)
        const int lane_group = warp & 3;                 // the 32 accumulator lanes this warp may read
        const int row_in_tile = lane_group * 32 + lane;
        uint32_t tile_i = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++tile_i) {
            const int rt = tile % row_tiles, ct = tile / row_tiles;
            const int r0 = rt * rows_per_tile, c0 = ct * cols_per_tile;
            const uint32_t as = tile_i & 1u, aph = (tile_i >> 1) & 1u;
            if (!mbar_wait(acc_full_bar(as), aph, abort_flag, p.status, 14)) { ok = false; break; }
            tmem_fence_after();
            const uint32_t t_addr = tmem_base + as * BN + ((uint32_t)(lane_group * 32) << 16);
            float v[16], u[16];
            if (!p.swap) {
                const int m = r0 + row_in_tile;
                const bool row_ok = m < p.M;
                if (!p.gated) {
                    for (int c = 0; c < BN; c += 16) {
                        tmem_ld16(t_addr + c, v);
                        const int n0 = c0 + c;
                        if (!row_ok || n0 >= p.N) continue;
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
            } else {
                // swapped: this thread owns output feature n, the columns are tokens
                if (!p.gated) {
                    const int n = r0 + row_in_tile;
                    const bool n_ok = n < p.N;
                    const float b = (p.bias && n_ok) ? p.bias[n] : 0.f;
                    for (int c = 0; c < BN; c += 16) {
                        tmem_ld16(t_addr + c, v);
                        if (!n_ok) continue;
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const int m = c0 + c + i;
                            if (m >= p.M) break;
                            float val = v[i] + b;
                            const size_t idx = (size_t)m * p.N + n;
                            if (p.residual) val += __bfloat162float(p.residual[idx]);
                            if (p.out_f32) reinterpret_cast<float*>(p.out)[idx] = val;
                            else reinterpret_cast<__nv_bfloat16*>(p.out)[idx] = __float2bfloat16_rn(val);
                        }
                    }
                } else {
                    // lanes 0..63 hold gate rows j0..j0+63, lanes 64..127 the matching up rows:
                    // the up half goes through shared memory to the threads that hold the gate
                    const bool is_up = row_in_tile >= 64;
                    const int jj = row_in_tile & 63;
                    for (int c = 0; c < BN; c += 16) {
                        tmem_ld16(t_addr + c, v);
                        if (is_up) {
#pragma unroll
                            for (int i = 0; i < 16; ++i) exch[jj * (BN + 1) + c + i] = v[i];
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
                                        __float2bfloat16_rn(silu_mul(v[i], exch[jj * (BN + 1) + c + i]));
                                }
                            }
                        }
                        asm volatile("bar.sync 1, 128;" ::: "memory");
                    }
                }
            }
            tmem_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty_bar(as));   // this half of tensor memory may be overwritten
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
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    });
    return fn;
}

struct MapKey {
    const void* ptr; int rows, k, box_rows;
    bool operator==(const MapKey& o) const { return ptr == o.ptr && rows == o.rows && k == o.k && box_rows == o.box_rows; }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        return std::hash<const void*>()(k.ptr) ^ (size_t)k.rows * 1000003u ^ (size_t)k.k * 10007u ^ (size_t)k.box_rows;
    }
};

// A tensor map of a row-major [rows, k] bf16 matrix, boxes of box_rows x 64, 128-byte swizzle.
bool get_map(const void* ptr, int rows, int k, int box_rows, CUtensorMap* out) {
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    const MapKey key{ptr, rows, k, box_rows};
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return true; }
    EncodeTiledFn fn = encode_fn();
    if (!fn) { ti_set_error("gemm_tcgen05: cuTensorMapEncodeTiled is not available from this driver"); return false; }
    cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)k * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUtensorMap m;
    CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { ti_set_error("gemm_tcgen05: cuTensorMapEncodeTiled failed (%d) for [%d, %d] box %d", (int)r, rows, k, box_rows); return false; }
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, m);
    *out = m;
    return true;
}

int sm_count() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    }
    return n;
}

template <int BN>
int launch(const CUtensorMap& rows_map, const CUtensorMap& cols_map, const GemmParams& p, int num_tiles, cudaStream_t stream) {
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<BN>::SMEM_BYTES);
        if (e != cudaSuccess) { ti_set_error("gemm_tcgen05: cannot get %d bytes of shared memory: %s", Cfg<BN>::SMEM_BYTES, cudaGetErrorString(e)); return (int)e; }
        configured = true;
    }
    const int grid = num_tiles < sm_count() ? num_tiles : sm_count();
    gemm_tcgen05_kernel<BN><<<grid, NUM_THREADS, Cfg<BN>::SMEM_BYTES, stream>>>(rows_map, cols_map, p);
    TI_CHECK_LAUNCH("gemm_tcgen05");
    return 0;
}

}  // namespace

// 1 if ti_gemm_bf16 takes this shape (K a multiple of 8 so that rows start on 16-byte boundaries).
TI_API int ti_gemm_bf16_supported(int M, int N, int K) { return (M > 0 && N > 0 && K > 0 && K % 8 == 0) ? 1 : 0; }

// y = x . w^T in bfloat16 with float32 accumulation. gated: w is [2N, K] (gate rows, then up rows),
// out [M, N] = silu(x.gate) * (x.up). out_f32: out is float32. status: device word set if a wait ran out.
TI_API int ti_gemm_bf16(void* out, const void* x, const void* w, const float* bias, const void* residual,
                        int M, int N, int K, int gated, int out_f32, int* status, cudaStream_t stream) {
    TI_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm_bf16: bad sizes M=%d N=%d K=%d", M, N, K);
    TI_REQUIRE(K % 8 == 0, "gemm_bf16: K=%d is not a multiple of 8 (rows must start on 16-byte boundaries)", K);
    TI_REQUIRE(!(gated && (bias || residual || out_f32)), "gemm_bf16: the gated form takes no bias, residual or float32 output");
    TI_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0, "gemm_bf16: operands must be 16-byte aligned");
    if (M == 0) return 0;
    GemmParams p;
    p.out = out; p.bias = bias; p.residual = (const __nv_bfloat16*)residual;
    p.M = M; p.N = N; p.K = K; p.gated = gated; p.out_f32 = out_f32; p.status = status;
    const int w_rows = gated ? 2 * N : N;
    CUtensorMap rows_map, cols_map;
    if (M <= 64) {
        // swapped: weights on the 128 accumulator lanes, tokens on the columns
        p.swap = 1;
        p.rows_total = N; p.cols_total = M;
        const int bn = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
        if (!get_map(w, w_rows, K, gated ? BM / 2 : BM, &rows_map)) return -1;
        if (!get_map(x, M, K, bn, &cols_map)) return -1;
        const int tiles = (N + (gated ? 64 : 128) - 1) / (gated ? 64 : 128);
        if (bn == 16) return launch<16>(rows_map, cols_map, p, tiles, stream);
        if (bn == 32) return launch<32>(rows_map, cols_map, p, tiles, stream);
        return launch<64>(rows_map, cols_map, p, tiles, stream);
    }
    p.swap = 0;
    p.rows_total = M; p.cols_total = N;
    if (!get_map(x, M, K, BM, &rows_map)) return -1;
    const int row_tiles = (M + BM - 1) / BM;
    const bool wide = (gated ? 2 * N : N) >= 256;
    if (wide) {
        if (!get_map(w, w_rows, K, gated ? 128 : 256, &cols_map)) return -1;
        const int cpt = gated ? 128 : 256;
        return launch<256>(rows_map, cols_map, p, row_tiles * ((N + cpt - 1) / cpt), stream);
    }
    if (!get_map(w, w_rows, K, gated ? 64 : 128, &cols_map)) return -1;
    const int cpt = gated ? 64 : 128;
    return launch<128>(rows_map, cols_map, p, row_tiles * ((N + cpt - 1) / cpt), stream);
}
