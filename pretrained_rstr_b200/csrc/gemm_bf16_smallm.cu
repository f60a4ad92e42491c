// Decode-time matrix product: few rows (M <= 64 tokens), bandwidth bound.
//
//     C[M,N] = act(X[M,K] . W[N,K]^T + bias[N]) (+ resid[M,N])
//     with X = A (bfloat16), or X = LayerNorm(R) rounded to bfloat16 (R float32 [M,K]),
//     the norm fused into the product's prologue.
//
// The weights are streamed once from HBM straight into tensor-core operand registers:
// with the roles swapped (C^T = W . X^T) a 16-row strip of W is the A operand of
// mma.sync.m16n8k16 and the tokens are the N dimension.  A thread loads 16 contiguous
// bytes of a W row per step; the k index inside an MMA is only a summation index, so the
// 8 elements of a load are spread over two MMAs in the order they arrive and the X
// fragments are read with the same permutation -- no shared-memory staging of W, no
// transposition.  One CTA owns 16 output features for all tokens; its 8 warps split K
// (steps of 32, round robin) and their partial sums are added in warp order through
// shared memory, so a result does not depend on the batch.  X comes from shared memory
// (after the fused LayerNorm) or from global memory (L2) directly.
// float32: statistics of the norm, accumulation, bias, activation, residual.
#include "gemm_smallm.cuh"

namespace {
using namespace smallm;

template <int MT, bool LN, typename O>
__global__ void __launch_bounds__(THREADS)
gemm_smallm_kernel(Args a) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    float* red = reinterpret_cast<float*>(smem_raw);                      // [8][16][8*MT]
    __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(red + WARPS * ROWS * 8 * MT);
    prb_grid_launch_dependents();                  // the next kernel may start its own prefetch
    Prefetch pf;
    prefetch(a, blockIdx.x, pf);
    // The weights above do not depend on the previous kernel; everything below does.
    prb_grid_wait();
    if constexpr (LN) norm_rows<MT>(a, xs);
    strip<MT, LN, O>(a, blockIdx.x, red, xs, pf);
}

template <int MT, bool LN, typename O>
int launch_smallm(Args a, cudaStream_t stream) {
    a.xs_pitch = LN ? norm_pitch(a.k) : a.k;
    const size_t smem = smem_bytes(MT, LN, a.k);
    if (smem > 220 * 1024) return PRB_E_SIZE;
    static size_t configured = 0;
    if (smem > 48 * 1024 && smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_smallm_kernel<MT, LN, O>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = smem;
    }
    const int grid = (a.n + ROWS - 1) / ROWS;
    cudaError_t e = prb_launch_dependent(gemm_smallm_kernel<MT, LN, O>, dim3(grid), dim3(THREADS),
                                         smem, stream, a);
    if (e != cudaSuccess) return (int)e;
    return 0;
}

template <bool LN, typename O>
int dispatch_mt(const Args& a, cudaStream_t stream) {
    if (a.m <= 8) return launch_smallm<1, LN, O>(a, stream);
    if (a.m <= 16) return launch_smallm<2, LN, O>(a, stream);
    if (a.m <= 32) return launch_smallm<4, LN, O>(a, stream);
    return launch_smallm<8, LN, O>(a, stream);
}
}  // namespace

PRB_API int prb_gemm_smallm_max_rows() { return 64; }
PRB_API int prb_gemm_smallm_max_norm_width() { return LN_MAX_K; }

// Argument check shared with the decode program; 0 when the kernel takes these sizes.
int prb_gemm_smallm_check(const void* x, const float* xf, const float* gamma, const float* beta,
                          const void* w, int m, int n, int k, long ldx, long ldw) {
    if (m > 64 || k <= 0 || n <= 0) return PRB_E_SIZE;
    if (k % 8 != 0 || ldw % 8 != 0 || ((uintptr_t)w) % 16 != 0) return PRB_E_ALIGN;
    if (xf != nullptr) {
        if (k > LN_MAX_K) return PRB_E_SIZE;
        if (ldx % 4 != 0 || ((uintptr_t)xf) % 16 != 0 || ((uintptr_t)gamma) % 16 != 0 ||
            (beta && ((uintptr_t)beta) % 16 != 0))
            return PRB_E_ALIGN;
    } else {
        if (x == nullptr) return PRB_E_ARG;
        if (ldx % 8 != 0 || ((uintptr_t)x) % 16 != 0) return PRB_E_ALIGN;
    }
    return 0;
}

// x: bfloat16 [M,K] (xf null), or xf: float32 [M,K] to be LayerNorm-ed first with gamma, beta
// (may be null) and eps.  m <= 64, k % 8 == 0, pitches multiples of 8 (4 for xf).
// kv_width > 0: the product is a fused QKV projection and its key and value columns are
// also written to the paged cache at slots[token] (the cache has the output's element type).
PRB_API int prb_gemm_smallm(void* out, const void* x, const float* xf, const float* gamma,
                            const float* beta, float eps, const void* w, const float* bias,
                            const float* resid, int m, int n, int k, long ldx, long ldw, long ldc,
                            int act, int out_dtype, void* k_pages, void* v_pages,
                            const int* slots, int q_width, int kv_width, int head_dim,
                            int page_size, int num_pages, int* status, cudaStream_t stream) {
    if (m <= 0 || n <= 0) return 0;
    const int bad = prb_gemm_smallm_check(x, xf, gamma, beta, w, m, n, k, ldx, ldw);
    if (bad) return bad;
    Args a;
    a.out = out;
    a.x = (const __nv_bfloat16*)x;
    a.xf = xf;
    a.gamma = gamma;
    a.beta = beta;
    a.eps = eps;
    a.w = (const __nv_bfloat16*)w;
    a.bias = bias;
    a.resid = resid;
    a.m = m; a.n = n; a.k = k;
    a.ldx = ldx; a.ldw = ldw; a.ldc = ldc;
    a.act = act;
    a.xs_pitch = k;
    if (kv_width > 0) {
        if (head_dim <= 0 || kv_width % head_dim != 0 || page_size <= 0 || q_width < 0 ||
            q_width + 2 * kv_width != n || k_pages == nullptr || v_pages == nullptr ||
            slots == nullptr)
            return PRB_E_ARG;
    }
    a.k_pages = k_pages; a.v_pages = v_pages; a.slots = slots;
    a.q_width = q_width; a.kv_width = kv_width; a.head_dim = head_dim;
    a.page_size = page_size; a.num_pages = num_pages; a.status = status;
    const bool ln = xf != nullptr;
    if (out_dtype == PRB_F32)
        return ln ? dispatch_mt<true, float>(a, stream) : dispatch_mt<false, float>(a, stream);
    if (out_dtype == PRB_BF16)
        return ln ? dispatch_mt<true, __nv_bfloat16>(a, stream)
                  : dispatch_mt<false, __nv_bfloat16>(a, stream);
    return PRB_E_DTYPE;
}
