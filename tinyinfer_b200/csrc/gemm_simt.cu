// y[M,N] = x[M,K] . w[N,K]^T with float32 FMA accumulation in a fixed k order: the true 32-bit
// matrix product of the engine (no tensor cores, no reduced-precision mode), also the fallback
// for bfloat16 shapes the tcgen05 kernels refuse. Epilogues: + bias[n], + residual[m,n], or the
// gated form out[m,j] = silu(x.w[j]) * (x.w[J+j]) on the float32 accumulators
// (tinyinfer/csrc/mlp.cu:116-141; silu(g) = g / (1 + exp(-g)), tinyinfer/csrc/utils.h:76-78).
// A row's result does not depend on which other rows share its tile.
#include "common.cuh"

constexpr int GS_BM = 64, GS_BN = 64, GS_BK = 16, GS_THREADS = 256;

template <typename T, typename OutT, bool GATED>
__global__ void __launch_bounds__(GS_THREADS) gemm_simt_kernel(
    OutT* __restrict__ out, const T* __restrict__ x, const T* __restrict__ w,
    const float* __restrict__ bias, const T* __restrict__ residual, int M, int N, int K, int gate_rows) {
    __shared__ float As[GS_BK][GS_BM + 4];
    __shared__ float Bs[GS_BK][GS_BN + 4];
    __shared__ float Cs[GATED ? GS_BK : 1][GS_BN + 4];
    ti_grid_launch_dependents();
    ti_grid_wait();
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;          // 16 x 16 threads, 4 x 4 outputs each
    const int m0 = blockIdx.y * GS_BM, n0 = blockIdx.x * GS_BN;
    float acc[4][4] = {}, acc2[GATED ? 4 : 1][4] = {};

    for (int k0 = 0; k0 < K; k0 += GS_BK) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int idx = tid + r * GS_THREADS;      // 0..1023
            const int row = idx >> 4, col = idx & 15;
            const int k = k0 + col;
            const int m = m0 + row, n = n0 + row;
            As[col][row] = (m < M && k < K) ? to_f32(x[(size_t)m * K + k]) : 0.f;
            Bs[col][row] = (n < N && k < K) ? to_f32(w[(size_t)n * K + k]) : 0.f;
            if constexpr (GATED) Cs[col][row] = (n < N && k < K) ? to_f32(w[(size_t)(gate_rows + n) * K + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GS_BK; ++kk) {
            float a[4], b[4], c[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
            if constexpr (GATED) {
#pragma unroll
                for (int j = 0; j < 4; ++j) c[j] = Cs[kk][tx * 4 + j];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
                    if constexpr (GATED) acc2[i][j] = fmaf(a[i], c[j], acc2[i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if constexpr (GATED) {
                v = (v / (1.f + expf(-v))) * acc2[i][j];
            } else {
                if (bias) v += bias[n];
                if (residual) v += to_f32(residual[(size_t)m * N + n]);
            }
            out[(size_t)m * N + n] = from_f32<OutT>(v);
        }
    }
}

// out_f32 != 0: the result is stored as float32 whatever the input dtype (logits).
// gated != 0: w is [2N, K], rows 0..N-1 the gate and N..2N-1 the up projection; out is [M, N].
TI_API int ti_gemm_simt(void* out, const void* x, const void* w, const float* bias, const void* residual,
                        int M, int N, int K, int gated, int out_f32, int dtype, cudaStream_t stream) {
    TI_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm: bad sizes M=%d N=%d K=%d", M, N, K);
    TI_REQUIRE(!(gated && (bias || residual || out_f32)), "gemm: the gated form takes no bias, residual or float32 output");
    if (M == 0) return 0;
    dim3 grid((N + GS_BN - 1) / GS_BN, (M + GS_BM - 1) / GS_BM);
    TI_REQUIRE(grid.y <= 65535, "gemm: too many rows");
    if (dtype == TI_F32) {
        if (gated)
            ti_launch(gemm_simt_kernel<float, float, true>, grid, GS_THREADS, 0, stream, (float*)out, (const float*)x, (const float*)w, nullptr, nullptr, M, N, K, N);
        else
            ti_launch(gemm_simt_kernel<float, float, false>, grid, GS_THREADS, 0, stream, (float*)out, (const float*)x, (const float*)w, bias, (const float*)residual, M, N, K, 0);
    } else if (dtype == TI_BF16) {
        typedef __nv_bfloat16 B;
        if (gated)
            ti_launch(gemm_simt_kernel<B, B, true>, grid, GS_THREADS, 0, stream, (B*)out, (const B*)x, (const B*)w, nullptr, nullptr, M, N, K, N);
        else if (out_f32)
            ti_launch(gemm_simt_kernel<B, float, false>, grid, GS_THREADS, 0, stream, (float*)out, (const B*)x, (const B*)w, bias, (const B*)residual, M, N, K, 0);
        else
            ti_launch(gemm_simt_kernel<B, B, false>, grid, GS_THREADS, 0, stream, (B*)out, (const B*)x, (const B*)w, bias, (const B*)residual, M, N, K, 0);
    } else TI_REQUIRE(false, "gemm: unknown dtype %d", dtype);
    TI_CHECK_LAUNCH("gemm_simt");
    return 0;
}
