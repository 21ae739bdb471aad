// PTX helpers shared by the sm_100a kernels: mbarriers with bounded waits, TMA tile loads,
// and the lazily resolved cuTensorMapEncodeTiled entry point.
#pragma once
#include "common.cuh"
#include <cuda.h>

constexpr unsigned long long TI_WAIT_NS = 2000000000ull;   // a wait gives up after two seconds

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
            if (global_ns() - t0 > TI_WAIT_NS) {
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

// ---------------------------------------------------------------------------- host side
typedef CUresult (*TiEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
TiEncodeTiledFn ti_encode_tiled_fn();
// A tensor map of a row-major [rows, cols] bf16 matrix (cols * 2 bytes a multiple of 16), boxes of
// box_rows x 64 elements, 128-byte swizzle, zero fill outside. Cached by (ptr, rows, cols, box_rows).
bool ti_get_bf16_map(const void* ptr, long long rows, int cols, int box_rows, CUtensorMap* out);
int ti_sm_count();
