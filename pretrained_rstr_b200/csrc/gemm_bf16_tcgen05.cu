// bfloat16 matrix product on the 5th-generation tensor cores with a fused epilogue:
//
//     C[M,N] = act(A[M,K] . W[N,K]^T + bias[N]) (+ resid[M,N])
//
// A and W are bfloat16 with K contiguous ("K-major"), accumulation is float32 in tensor
// memory (TMEM), C is bfloat16 or float32, bias and resid are float32.
//
// Persistent CTAs (one per SM) walk 128 x BN tiles of C; the accumulator alternates
// between two TMEM buffers so that a tile's epilogue overlaps the next tile's main loop.
// Warp roles:
//   warp 0  producer: one thread issues TMA loads (cp.async.bulk.tensor, 128-byte swizzle)
//           of a 128 x 64 tile of A and a BN x 64 tile of W per pipeline stage;
//   warp 1  allocates TMEM; one thread issues tcgen05.mma (M=128, N=BN, K=16, four per
//           stage) and commits each stage back to the producer through an mbarrier;
//   warps 2-9  epilogue: tcgen05.ld the accumulator (one row per thread, two warps per
//           32-lane quarter taking alternate 32-column chunks), add bias, apply the
//           activation, add the residual, store.
// Rows of A beyond M, rows of W beyond N and the K tail are zero-filled by TMA; stores
// are masked.  K and the row pitches must be multiples of 8 elements (TMA needs 16-byte
// strides); other sizes are refused with PRB_E_ALIGN, never computed wrongly.
// No TMA load uses cluster multicast.  Every mbarrier wait is bounded: on a timeout the
// kernel records PRB_S_WAIT_TIMEOUT in the status word, skips the remaining work,
// waits (bounded) for its loads in flight, frees its TMEM and returns.
#include <cuda.h>
#include <cudaTypedefs.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "tcgen05.cuh"
#include "tensor_map.cuh"

namespace {

constexpr int BM = 128;
constexpr int BK = 64;             // 64 bf16 = 128 bytes = one swizzle atom row
constexpr int UMMA_K = 16;
constexpr int GEMM_THREADS = 320;     // producer warp, MMA warp, 8 epilogue warps

using namespace tc5;

template <int BN> struct TileCfg {
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int STAGES = (192 * 1024) / STAGE_BYTES > 8 ? 8 : (192 * 1024) / STAGE_BYTES;
    static constexpr int TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;      // two accumulators
    static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + 1024 /*align*/ + 256;
};


// tanh-form GELU as u * sigmoid(2z), z = sqrt(2/pi) (u + 0.044715 u^3): no cancellation in
// the negative tail, relative error of the fast exp and divide about 1e-6.
__device__ __forceinline__ float gelu_tanh_fast(float u) {
    const float z2 = 1.5957691216057308f * (u + 0.044715f * u * u * u);   // 2z
    return __fdividef(u, 1.0f + __expf(-z2));
}
__device__ __forceinline__ float epilogue_act(float x, int act) {
    if (act == PRB_ACT_GELU_TANH) return gelu_tanh_fast(x);
    if (act == PRB_ACT_NONE) return x;
    return prb_activate(x, act);
}

// Persistent kernel: each CTA walks tiles blockIdx.x, blockIdx.x + gridDim.x, ... (tiles
// that share a W tile are neighbours, so they run at the same time and share it in L2).
// The producer runs ahead across tile borders; the accumulator alternates between two
// TMEM buffers, so the epilogue of one tile overlaps the main loop of the next.
template <int BN, typename O>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                 O* __restrict__ c, const float* __restrict__ bias,
                 const float* __restrict__ resid, int m, int n, int k, long ldc, int act,
                 int* status) {
    using Cfg = TileCfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    // tiles need 1024-byte alignment for the 128-byte swizzle
    uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* tiles = smem;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)Cfg::STAGES * Cfg::STAGE_BYTES);
    uint64_t* full_bar = bars;                       // [STAGES]  TMA -> MMA
    uint64_t* empty_bar = bars + Cfg::STAGES;        // [STAGES]  MMA -> TMA
    uint64_t* tfull_bar = bars + 2 * Cfg::STAGES;    // [2]       MMA -> epilogue
    uint64_t* tempty_bar = tfull_bar + 2;            // [2]       epilogue -> MMA
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
    volatile int* failed = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m_tiles = (m + BM - 1) / BM, n_tiles = (n + BN - 1) / BN;
    const int total_tiles = m_tiles * n_tiles;
    const int k_blocks = (k + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < Cfg::STAGES; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&tfull_bar[a]), 1);
            mbar_init(smem_u32(&tempty_bar[a]), 8);      // one arrival per epilogue warp
        }
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(tmem_slot)),
                     "r"((uint32_t)Cfg::TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ producer
        if (lane == 0) {
            int it = 0;                               // k-blocks issued so far, over all tiles
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const int m0 = (tile % m_tiles) * BM, n0 = (tile / m_tiles) * BN;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % Cfg::STAGES;
                    ok = mbar_wait(smem_u32(&empty_bar[s]), ((it / Cfg::STAGES) & 1) ^ 1, failed);
                    if (!ok) {
                        prb_set_status(status, PRB_S_WAIT_TIMEOUT, 1, blockIdx.x, it);
                        break;
                    }
                    const uint32_t fb = smem_u32(&full_bar[s]);
                    mbar_expect_tx(fb, Cfg::STAGE_BYTES);
                    uint8_t* stage = tiles + (size_t)s * Cfg::STAGE_BYTES;
                    tma_load_2d(smem_u32(stage), &map_a, fb, kb * BK, m0);
                    tma_load_2d(smem_u32(stage + Cfg::A_BYTES), &map_w, fb, kb * BK, n0);
                }
            }
            if (!ok) {
                // wait (bounded) for loads still in flight before the CTA may exit
                const int first = it > Cfg::STAGES ? it - Cfg::STAGES : 0;
                for (int j = first; j < it; ++j) {
                    const uint32_t fb = smem_u32(&full_bar[j % Cfg::STAGES]);
                    for (uint32_t i = 0; i < WAIT_LIMIT; ++i)
                        if (mbar_try_wait(fb, (j / Cfg::STAGES) & 1)) break;
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(BM, BN);
            int it = 0, local = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++local) {
                const int acc = local & 1;
                // the epilogue must have drained this accumulator (two tiles ago)
                ok = mbar_wait(smem_u32(&tempty_bar[acc]), ((local >> 1) & 1) ^ 1, failed);
                if (!ok) {
                    prb_set_status(status, PRB_S_WAIT_TIMEOUT, 4, blockIdx.x, local);
                    break;
                }
                tcgen05_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % Cfg::STAGES;
                    ok = mbar_wait(smem_u32(&full_bar[s]), (it / Cfg::STAGES) & 1, failed);
                    if (!ok) {
                        prb_set_status(status, PRB_S_WAIT_TIMEOUT, 2, blockIdx.x, it);
                        break;
                    }
                    tcgen05_fence_after();
                    const uint32_t a_addr = smem_u32(tiles + (size_t)s * Cfg::STAGE_BYTES);
                    const uint64_t a_desc = make_smem_desc(a_addr);
                    const uint64_t b_desc = make_smem_desc(a_addr + Cfg::A_BYTES);
#pragma unroll
                    for (int kk = 0; kk < BK / UMMA_K; ++kk) {
                        // 16 elements = 32 bytes further inside the swizzle atom: +2 (16-byte units)
                        umma_bf16(d_tmem, a_desc + (uint64_t)(kk * 2), b_desc + (uint64_t)(kk * 2),
                                  idesc, (kb > 0 || kk > 0) ? 1u : 0u);
                    }
                    umma_commit(smem_u32(&empty_bar[s]));   // frees the stage when the MMAs retire
                }
                if (ok) umma_commit(smem_u32(&tfull_bar[acc]));   // accumulator complete
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue
        const int quarter = warp & 3;                       // TMEM lanes this warp may read
        const int half = (warp - 2) >> 2;                   // two warps share a quarter: even / odd chunks
        const bool vec_ok = ((ldc * (long)sizeof(O)) % 16 == 0) && (((uintptr_t)c) % 16 == 0) &&
                            (resid == nullptr ||
                             (((ldc * 4) % 16 == 0) && (((uintptr_t)resid) % 16 == 0)));
        int local = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++local) {
            const int m0 = (tile % m_tiles) * BM, n0 = (tile / m_tiles) * BN;
            const int acc = local & 1;
            const int row = m0 + quarter * 32 + lane;
            ok = mbar_wait(smem_u32(&tfull_bar[acc]), (local >> 1) & 1, failed);
            if (!ok && lane == 0) prb_set_status(status, PRB_S_WAIT_TIMEOUT, 3, blockIdx.x, local);
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok) break;
            tcgen05_fence_after();
            if (half * 32 >= BN || n0 + half * 32 >= n) {      // nothing to read for this warp
                if (lane == 0) mbar_arrive(smem_u32(&tempty_bar[acc]));
                continue;
            }
#pragma unroll 1
            for (int c0 = half * 32; c0 < BN; c0 += 64) {
                if (n0 + c0 >= n) break;                    // uniform across the warp
                uint32_t r[32];
                tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) +
                                  (uint32_t)(acc * BN + c0), r);
                if (c0 + 64 >= BN || n0 + c0 + 64 >= n) {
                    // this warp's last read of the accumulator: hand it back before the stores
                    tcgen05_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&tempty_bar[acc]));
                }
                if (row >= m) continue;
                const int ncol = n0 + c0;
                const int n_valid = (n - ncol) < 32 ? (n - ncol) : 32;
                O* crow = c + (size_t)row * ldc + ncol;
                const float* rrow = resid ? resid + (size_t)row * ldc + ncol : nullptr;
                if (vec_ok && n_valid == 32) {
#pragma unroll
                    for (int j = 0; j < 32; j += 8) {
                        float v[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(r[j + e]);
                        if (bias) {
                            const float4 b0 = __ldg(reinterpret_cast<const float4*>(bias + ncol + j));
                            const float4 b1 = __ldg(reinterpret_cast<const float4*>(bias + ncol + j + 4));
                            v[0] += b0.x; v[1] += b0.y; v[2] += b0.z; v[3] += b0.w;
                            v[4] += b1.x; v[5] += b1.y; v[6] += b1.z; v[7] += b1.w;
                        }
#pragma unroll
                        for (int e = 0; e < 8; ++e) v[e] = epilogue_act(v[e], act);
                        if (rrow) {
                            const float4 q0 = *reinterpret_cast<const float4*>(rrow + j);
                            const float4 q1 = *reinterpret_cast<const float4*>(rrow + j + 4);
                            v[0] += q0.x; v[1] += q0.y; v[2] += q0.z; v[3] += q0.w;
                            v[4] += q1.x; v[5] += q1.y; v[6] += q1.z; v[7] += q1.w;
                        }
                        if constexpr (sizeof(O) == 4) {
                            *reinterpret_cast<float4*>(crow + j) = make_float4(v[0], v[1], v[2], v[3]);
                            *reinterpret_cast<float4*>(crow + j + 4) = make_float4(v[4], v[5], v[6], v[7]);
                        } else {
                            uint4 u;
                            u.x = pack2(v[0], v[1]); u.y = pack2(v[2], v[3]);
                            u.z = pack2(v[4], v[5]); u.w = pack2(v[6], v[7]);
                            *reinterpret_cast<uint4*>(crow + j) = u;
                        }
                    }
                } else {
                    // tail columns or unaligned rows (e.g. a vocabulary that is odd): one by one
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        if (j < n_valid) {
                            float x = __uint_as_float(r[j]);
                            if (bias) x += __ldg(bias + ncol + j);
                            x = epilogue_act(x, act);
                            if (rrow) x += rrow[j];
                            crow[j] = prb_from_float<O>(x);
                        }
                    }
                }
            }
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                     "r"((uint32_t)Cfg::TMEM_COLS)
                     : "memory");
    }
}

// ------------------------------------------------------------------ host side
using tmap::get_map;

template <int BN, typename O>
int launch(const CUtensorMap& ma, const CUtensorMap& mw, O* c, const float* bias,
           const float* resid, int m, int n, int k, long ldc, int act, int* status,
           cudaStream_t stream) {
    using Cfg = TileCfg<BN>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_bf16_kernel<BN, O>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)Cfg::SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    static int sm_count = 0;
    if (sm_count == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
            sm_count <= 0)
            sm_count = 148;
    }
    const long tiles = (long)((n + BN - 1) / BN) * ((m + BM - 1) / BM);
    const int grid = (int)(tiles < sm_count ? tiles : sm_count);
    gemm_bf16_kernel<BN, O><<<grid, GEMM_THREADS, Cfg::SMEM, stream>>>(ma, mw, c, bias, resid, m,
                                                                       n, k, ldc, act, status);
    PRB_LAUNCH_CHECK();
    return 0;
}

}  // namespace

// tile_n: 0 = choose (by M and N), or one of 32, 64, 128, 256.
PRB_API int prb_gemm_bf16(void* c, const void* a, const void* w, const float* bias,
                          const float* resid, int m, int n, int k, long lda, long ldw, long ldc,
                          int act, int out_dtype, int tile_n, int* status, cudaStream_t stream) {
    if (m <= 0 || n <= 0) return 0;
    if (k <= 0) return PRB_E_SIZE;
    if (k % 8 != 0 || lda % 8 != 0 || ldw % 8 != 0 || ((uintptr_t)a) % 16 != 0 ||
        ((uintptr_t)w) % 16 != 0)
        return PRB_E_ALIGN;
    if (tile_n == 0) {
        // fewest rounds of tiles over the SMs, weighted by tile width plus a fixed cost
        const long mt = (m + BM - 1) / BM;
        long best = -1;
        for (int bn = 256; bn >= 32; bn /= 2) {
            const long tiles = mt * ((n + bn - 1) / bn);
            const long rounds = (tiles + 147) / 148;
            const long cost = rounds * (bn + 64);
            if (best < 0 || cost < best) { best = cost; tile_n = bn; }
        }
    }
    if (tile_n != 32 && tile_n != 64 && tile_n != 128 && tile_n != 256) return PRB_E_ARG;
    CUtensorMap ma, mw;
    int r = get_map(a, m, k, lda, BM, &ma);
    if (r) return r;
    r = get_map(w, n, k, ldw, tile_n, &mw);
    if (r) return r;
#define PRB_GO(BN_)                                                                              \
    (out_dtype == PRB_F32                                                                        \
         ? launch<BN_, float>(ma, mw, (float*)c, bias, resid, m, n, k, ldc, act, status, stream) \
         : launch<BN_, __nv_bfloat16>(ma, mw, (__nv_bfloat16*)c, bias, resid, m, n, k, ldc, act, \
                                      status, stream))
    if (out_dtype != PRB_F32 && out_dtype != PRB_BF16) return PRB_E_DTYPE;
    switch (tile_n) {
        case 32: return PRB_GO(32);
        case 64: return PRB_GO(64);
        case 128: return PRB_GO(128);
        default: return PRB_GO(256);
    }
#undef PRB_GO
}
