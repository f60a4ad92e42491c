// The true 32-bit matrix product: C = epilogue(A[M,K] . W[N,K]^T + bias), plain FMA on
// CUDA cores, no tensor cores and no reduced-precision mode.  Each output element is
// accumulated by one thread over k = 0..K-1 in ascending order, so a row's result does
// not depend on how many other rows are in the batch.
#include "common.cuh"

namespace {
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

__global__ void __launch_bounds__(256)
gemm_f32_kernel(float* __restrict__ c, const float* __restrict__ a, const float* __restrict__ w,
                const float* __restrict__ bias, const float* __restrict__ resid, int m, int n,
                int k, long lda, long ldw, long ldc, int act) {
    __shared__ float as[BK][BM + 1];
    __shared__ float ws[BK][BN + 1];
    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < k; k0 += BK) {
        // 64 rows x 16 k = 1024 elements per tile, 4 per thread
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int e = tid + i * 256;
            const int r = e / BK, kk = e % BK;
            const int gm = m0 + r, gn = n0 + r, gk = k0 + kk;
            as[kk][r] = (gm < m && gk < k) ? a[(size_t)gm * lda + gk] : 0.0f;
            ws[kk][r] = (gn < n && gk < k) ? w[(size_t)gn * ldw + gk] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float av[TM], wv[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) av[i] = as[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) wv[j] = ws[kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int gm = m0 + ty * TM + i;
        if (gm >= m) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int gn = n0 + tx * TN + j;
            if (gn >= n) continue;
            float v = acc[i][j];
            if (bias) v += bias[gn];
            v = prb_activate(v, act);
            if (resid) v += resid[(size_t)gm * ldc + gn];
            c[(size_t)gm * ldc + gn] = v;
        }
    }
}
}  // namespace

PRB_API int prb_gemm_f32(float* c, const float* a, const float* w, const float* bias,
                         const float* resid, int m, int n, int k, long lda, long ldw, long ldc,
                         int act, cudaStream_t stream) {
    if (m <= 0 || n <= 0) return 0;
    if (k <= 0) return PRB_E_SIZE;
    dim3 grid((n + BN - 1) / BN, (m + BM - 1) / BM);
    if (grid.y > 65535) return PRB_E_SIZE;
    gemm_f32_kernel<<<grid, 256, 0, stream>>>(c, a, w, bias, resid, m, n, k, lda, ldw, ldc, act);
    PRB_LAUNCH_CHECK();
    return 0;
}
