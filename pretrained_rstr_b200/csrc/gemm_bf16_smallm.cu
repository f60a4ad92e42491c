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
#include "common.cuh"

namespace {
constexpr int SM_THREADS = 256;
constexpr int SM_WARPS = 8;
constexpr int ROWS = 16;            // output features per CTA
constexpr int KSTEP = 32;
constexpr int LN_MAX_K = 2048;      // fused norm keeps a row in registers: 16 float4 per lane

__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 v;      // weights are read once: do not keep them in L1
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

template <int MT, bool LN, typename O>
__global__ void __launch_bounds__(SM_THREADS)
gemm_smallm_kernel(O* __restrict__ out, const __nv_bfloat16* __restrict__ x,
                   const float* __restrict__ xf, const float* __restrict__ gamma,
                   const float* __restrict__ beta, float eps,
                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ bias,
                   const float* __restrict__ resid, int m, int n, int k, long ldx, long ldw,
                   long ldc, int act, int xs_pitch) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    float* red = reinterpret_cast<float*>(smem_raw);                      // [8][16][8*MT]
    __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(red + SM_WARPS * ROWS * 8 * MT);
    constexpr int MP = 8 * MT;      // padded token count

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, q = lane & 3;        // MMA group (row / token) and quad index
    const int n0 = blockIdx.x * ROWS;
    prb_grid_launch_dependents();                  // the next kernel may start its own prefetch

    // ---- stream the 16 weight rows; this warp takes k-steps warp, warp+8, ...
    // (the first loads are issued before the norm so that they overlap it)
    float acc[MT][4];
#pragma unroll
    for (int i = 0; i < MT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.0f;
    const int steps = (k + KSTEP - 1) / KSTEP;
    const int r0 = n0 + g, r1 = n0 + g + 8;
    const bool row0_ok = r0 < n, row1_ok = r1 < n;
    const __nv_bfloat16* w0 = w + (size_t)(row0_ok ? r0 : 0) * ldw;
    const __nv_bfloat16* w1 = w + (size_t)(row1_ok ? r1 : 0) * ldw;

    constexpr int PF = 4;                          // steps of weights in flight per warp
    uint4 wa[PF], wb[PF];
#pragma unroll
    for (int p = 0; p < PF; ++p) {
        const int kk = (warp + p * SM_WARPS) * KSTEP + q * 8;
        const bool ok = kk < k;
        wa[p] = (ok && row0_ok) ? ldg_stream(w0 + kk) : make_uint4(0, 0, 0, 0);
        wb[p] = (ok && row1_ok) ? ldg_stream(w1 + kk) : make_uint4(0, 0, 0, 0);
    }
    // The weights above do not depend on the previous kernel; everything below does.
    prb_grid_wait();
    if constexpr (LN) {
        // ---- fused LayerNorm of the M rows into shared memory (bfloat16)
        const int nvec = k / 4;                   // float4 per row
        for (int t = warp; t < MP; t += SM_WARPS) {
            __nv_bfloat16* dst = xs + (size_t)t * xs_pitch;
            if (t >= m) {
                for (int i = lane; i < k / 2; i += 32)
                    reinterpret_cast<uint32_t*>(dst)[i] = 0u;
                continue;
            }
            const float4* src = reinterpret_cast<const float4*>(xf + (size_t)t * ldx);
            float4 v[LN_MAX_K / 128];
            float s = 0.0f;
#pragma unroll
            for (int i = 0; i < LN_MAX_K / 128; ++i) {
                const int idx = lane + 32 * i;
                v[i] = idx < nvec ? src[idx] : make_float4(0.f, 0.f, 0.f, 0.f);
                s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
            }
            const float mean = prb_warp_sum(s) / (float)k;
            float sq = 0.0f;
#pragma unroll
            for (int i = 0; i < LN_MAX_K / 128; ++i) {
                if (lane + 32 * i < nvec) {
                    const float a = v[i].x - mean, b = v[i].y - mean, c = v[i].z - mean,
                                d = v[i].w - mean;
                    sq += (a * a + b * b) + (c * c + d * d);
                }
            }
            const float inv = 1.0f / sqrtf(prb_warp_sum(sq) / (float)k + eps);
#pragma unroll
            for (int i = 0; i < LN_MAX_K / 128; ++i) {
                const int idx = lane + 32 * i;
                if (idx < nvec) {
                    const float4 gm = reinterpret_cast<const float4*>(gamma)[idx];
                    float4 bt = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (beta) bt = reinterpret_cast<const float4*>(beta)[idx];
                    const __nv_bfloat162 lo = __floats2bfloat162_rn(
                        (v[i].x - mean) * inv * gm.x + bt.x, (v[i].y - mean) * inv * gm.y + bt.y);
                    const __nv_bfloat162 hi = __floats2bfloat162_rn(
                        (v[i].z - mean) * inv * gm.z + bt.z, (v[i].w - mean) * inv * gm.w + bt.w);
                    uint2 pk;
                    pk.x = *reinterpret_cast<const uint32_t*>(&lo);
                    pk.y = *reinterpret_cast<const uint32_t*>(&hi);
                    *reinterpret_cast<uint2*>(dst + idx * 4) = pk;
                }
            }
        }
        __syncthreads();
    }

    for (int s0 = warp; s0 < steps; s0 += SM_WARPS * PF) {
#pragma unroll
        for (int p = 0; p < PF; ++p) {
            const int s = s0 + p * SM_WARPS;
            if (s >= steps) break;
            const uint4 a = wa[p], b = wb[p];
            {   // refill this slot with the step PF rounds ahead
                const int kk = (s + PF * SM_WARPS) * KSTEP + q * 8;
                const bool ok = kk < k;
                wa[p] = (ok && row0_ok) ? ldg_stream(w0 + kk) : make_uint4(0, 0, 0, 0);
                wb[p] = (ok && row1_ok) ? ldg_stream(w1 + kk) : make_uint4(0, 0, 0, 0);
            }
            const int kx = s * KSTEP + q * 8;      // this thread's 8 k indices of the step
            const bool kok = kx < k;
#pragma unroll
            for (int nt = 0; nt < MT; ++nt) {
                uint4 xv = make_uint4(0, 0, 0, 0);
                const int tok = nt * 8 + g;
                if constexpr (LN) {
                    if (kok) xv = *reinterpret_cast<const uint4*>(xs + (size_t)tok * xs_pitch + kx);
                } else {
                    if (kok && tok < m)
                        xv = *reinterpret_cast<const uint4*>(x + (size_t)tok * ldx + kx);
                }
                // elements 0..3 of each load feed the first MMA, 4..7 the second
                mma16816(acc[nt], a.x, b.x, a.y, b.y, xv.x, xv.y);
                mma16816(acc[nt], a.z, b.z, a.w, b.w, xv.z, xv.w);
            }
        }
    }
    // ---- add the warps' partial sums in warp order
    // acc[nt][0,1]: feature g, tokens nt*8 + q*2 + {0,1}; acc[nt][2,3]: feature g + 8
#pragma unroll
    for (int nt = 0; nt < MT; ++nt) {
        float* base = red + ((size_t)warp * ROWS) * MP + nt * 8 + q * 2;
        base[(size_t)g * MP] = acc[nt][0];
        base[(size_t)g * MP + 1] = acc[nt][1];
        base[(size_t)(g + 8) * MP] = acc[nt][2];
        base[(size_t)(g + 8) * MP + 1] = acc[nt][3];
    }
    __syncthreads();
    for (int e = threadIdx.x; e < ROWS * MP; e += SM_THREADS) {
        const int tok = e / ROWS, r = e % ROWS;    // consecutive threads: consecutive features
        const int col = n0 + r;
        if (tok >= m || col >= n) continue;
        float v = 0.0f;
#pragma unroll
        for (int wv = 0; wv < SM_WARPS; ++wv) v += red[((size_t)wv * ROWS + r) * MP + tok];
        if (bias) v += bias[col];
        v = prb_activate(v, act);
        if (resid) v += resid[(size_t)tok * ldc + col];
        out[(size_t)tok * ldc + col] = prb_from_float<O>(v);
    }
}

template <int MT, bool LN, typename O>
int launch_smallm(O* out, const __nv_bfloat16* x, const float* xf, const float* gamma,
                  const float* beta, float eps, const __nv_bfloat16* w, const float* bias,
                  const float* resid, int m, int n, int k, long ldx, long ldw, long ldc, int act,
                  cudaStream_t stream) {
    // row pitch of the normalised activations: words per row = 16 mod 32 (conflict-free)
    int pitch = k;
    if (LN) {
        const int words = k / 2;
        pitch = k + 2 * ((16 - (words % 32) + 32) % 32);
    }
    const size_t smem = (size_t)SM_WARPS * ROWS * 8 * MT * sizeof(float) +
                        (LN ? (size_t)8 * MT * pitch * 2 : 0);
    if (smem > 220 * 1024) return PRB_E_SIZE;
    static size_t configured = 0;
    if (smem > 48 * 1024 && smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_smallm_kernel<MT, LN, O>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = smem;
    }
    const int grid = (n + ROWS - 1) / ROWS;
    cudaError_t e = prb_launch_dependent(gemm_smallm_kernel<MT, LN, O>, dim3(grid),
                                         dim3(SM_THREADS), smem, stream, out, x, xf, gamma, beta,
                                         eps, w, bias, resid, m, n, k, ldx, ldw, ldc, act, pitch);
    if (e != cudaSuccess) return (int)e;
    return 0;
}

template <bool LN, typename O>
int dispatch_mt(O* out, const __nv_bfloat16* x, const float* xf, const float* gamma,
                const float* beta, float eps, const __nv_bfloat16* w, const float* bias,
                const float* resid, int m, int n, int k, long ldx, long ldw, long ldc, int act,
                cudaStream_t stream) {
#define PRB_SM(MT_) \
    launch_smallm<MT_, LN, O>(out, x, xf, gamma, beta, eps, w, bias, resid, m, n, k, ldx, ldw, ldc, act, stream)
    if (m <= 8) return PRB_SM(1);
    if (m <= 16) return PRB_SM(2);
    if (m <= 32) return PRB_SM(4);
    return PRB_SM(8);
#undef PRB_SM
}
}  // namespace

PRB_API int prb_gemm_smallm_max_rows() { return 64; }
PRB_API int prb_gemm_smallm_max_norm_width() { return LN_MAX_K; }

// x: bfloat16 [M,K] (xf null), or xf: float32 [M,K] to be LayerNorm-ed first with gamma, beta
// (may be null) and eps.  m <= 64, k % 8 == 0, pitches multiples of 8 (4 for xf).
PRB_API int prb_gemm_smallm(void* out, const void* x, const float* xf, const float* gamma,
                            const float* beta, float eps, const void* w, const float* bias,
                            const float* resid, int m, int n, int k, long ldx, long ldw, long ldc,
                            int act, int out_dtype, cudaStream_t stream) {
    if (m <= 0 || n <= 0) return 0;
    if (m > 64 || k <= 0) return PRB_E_SIZE;
    if (k % 8 != 0 || ldw % 8 != 0 || ((uintptr_t)w) % 16 != 0) return PRB_E_ALIGN;
    const bool ln = xf != nullptr;
    if (ln) {
        if (k > LN_MAX_K) return PRB_E_SIZE;
        if (ldx % 4 != 0 || ((uintptr_t)xf) % 16 != 0 || ((uintptr_t)gamma) % 16 != 0 ||
            (beta && ((uintptr_t)beta) % 16 != 0))
            return PRB_E_ALIGN;
    } else {
        if (x == nullptr) return PRB_E_ARG;
        if (ldx % 8 != 0 || ((uintptr_t)x) % 16 != 0) return PRB_E_ALIGN;
    }
    const __nv_bfloat16* xb = (const __nv_bfloat16*)x;
    const __nv_bfloat16* wb = (const __nv_bfloat16*)w;
    if (out_dtype == PRB_F32) {
        return ln ? dispatch_mt<true, float>((float*)out, xb, xf, gamma, beta, eps, wb, bias, resid,
                                             m, n, k, ldx, ldw, ldc, act, stream)
                  : dispatch_mt<false, float>((float*)out, xb, xf, gamma, beta, eps, wb, bias,
                                              resid, m, n, k, ldx, ldw, ldc, act, stream);
    }
    if (out_dtype == PRB_BF16) {
        return ln ? dispatch_mt<true, __nv_bfloat16>((__nv_bfloat16*)out, xb, xf, gamma, beta, eps,
                                                     wb, bias, resid, m, n, k, ldx, ldw, ldc, act,
                                                     stream)
                  : dispatch_mt<false, __nv_bfloat16>((__nv_bfloat16*)out, xb, xf, gamma, beta,
                                                      eps, wb, bias, resid, m, n, k, ldx, ldw, ldc,
                                                      act, stream);
    }
    return PRB_E_DTYPE;
}
