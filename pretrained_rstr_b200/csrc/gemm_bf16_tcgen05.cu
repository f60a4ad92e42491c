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
#include <type_traits>
#include <unordered_map>

#include "common.cuh"
#include "tcgen05.cuh"
#include "tensor_map.cuh"

#ifdef PRB_TRACE
__device__ unsigned long long g_gemm_trace[256 * 8];
#define GT(slot)                                                                      \
    do {                                                                              \
        if (lane == 0 && blockIdx.x < 256) {                                          \
            unsigned long long t__;                                                   \
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t__));                   \
            g_gemm_trace[blockIdx.x * 8 + (slot)] = t__;                              \
        }                                                                             \
    } while (0)
PRB_API int prb_gemm_bf16_trace(unsigned long long* host, int n) {
    return (int)cudaMemcpyFromSymbol(host, g_gemm_trace, sizeof(unsigned long long) * n);
}
// cycles one role of a CTA spent in a kind of work: [0] producer waiting for a free stage,
// [1] producer issuing loads, [2] MMA thread waiting for a full stage, [3] MMA thread issuing
__device__ long long g_gemm_cycles[256 * 4];
PRB_API int prb_gemm_bf16_cycles(long long* host, int n) {
    return (int)cudaMemcpyFromSymbol(host, g_gemm_cycles, sizeof(long long) * n);
}
#define GC_BEGIN long long gc_t__ = clock64(), gc_a__ = 0, gc_b__ = 0
#define GC_A do { const long long n__ = clock64(); gc_a__ += n__ - gc_t__; gc_t__ = n__; } while (0)
#define GC_B do { const long long n__ = clock64(); gc_b__ += n__ - gc_t__; gc_t__ = n__; } while (0)
#define GC_END(slot)                                                                  \
    do {                                                                              \
        if (blockIdx.x < 256) {                                                       \
            g_gemm_cycles[blockIdx.x * 4 + (slot)] = gc_a__;                          \
            g_gemm_cycles[blockIdx.x * 4 + (slot) + 1] = gc_b__;                      \
        }                                                                             \
    } while (0)
#else
#define GT(slot)
#define GC_BEGIN
#define GC_A
#define GC_B
#define GC_END(slot)
#endif

namespace {

constexpr int BM = 128;
constexpr int BK = 64;             // 64 bf16 = 128 bytes = one swizzle atom row
constexpr int UMMA_K = 16;
constexpr int GEMM_THREADS = 320;     // producer warp, MMA warp, 8 epilogue warps

using namespace tc5;

template <int BN, bool PAIR = false> struct TileCfg {
    static_assert(BN % 32 == 0 && BN >= 32 && BN <= 256, "tile width: a multiple of 32 up to 256");
    static constexpr int A_BYTES = BM * BK * 2;
    // (a CTA of a pair loads its 128 rows of A and its half of the tile's rows of W)
    static constexpr int B_BYTES = (PAIR ? BN / 2 : BN) * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int STAGES = (176 * 1024) / STAGE_BYTES > 8 ? 8 : (176 * 1024) / STAGE_BYTES;
    // two accumulators, each at a power-of-two column offset (tensor memory is allocated in
    // powers of two)
    static constexpr int ACC_STRIDE = BN <= 32 ? 32 : BN <= 64 ? 64 : BN <= 128 ? 128 : 256;
    static constexpr int TMEM_COLS = 2 * ACC_STRIDE;
    // per epilogue warp a staging tile of 32 rows x 128 bytes of finished output (after the
    // stages, so that it is 1024-byte aligned as the 128-byte swizzle wants)
    static constexpr int STG_BYTES = 32 * 128;
    static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + 1024 /*align*/ + 256 +
                                   (size_t)8 * STG_BYTES;
};


// Optional scatter of output columns into the paged cache (a fused QKV product whose output
// has the cache's element type: columns [q_width, q_width + kv_width) are keys, the next
// kv_width are values; slots[row] is the token's cache slot, -1 = none).  kv_width == 0: off.
struct Scatter {
    void* k_pages;                  // [pages][kv heads][page_size][head_dim]
    void* v_pages;
    const int* slots;
    int q_width, kv_width, head_dim, page_size, num_pages;
    int only_cache;                 // key and value columns go to the cache alone, not to the output
};

// Where `count` consecutive output columns starting at `col` (inside one head) of the token
// with cache slot `slot` go; null when they are not key or value columns or there is no slot.
template <typename O>
__device__ __forceinline__ O* scatter_dst(const Scatter& sc, int col, int slot, int row,
                                          int* status) {
    if (sc.kv_width == 0 || col < sc.q_width || slot < 0) return nullptr;
    const int page = slot / sc.page_size, off = slot - page * sc.page_size;
    if (page >= sc.num_pages) {
        prb_set_status(status, PRB_S_SLOT_RANGE, row, slot, sc.num_pages);
        return nullptr;
    }
    int cc = col - sc.q_width;
    O* pages = reinterpret_cast<O*>(cc < sc.kv_width ? sc.k_pages : sc.v_pages);
    if (cc >= sc.kv_width) cc -= sc.kv_width;
    const int h = cc / sc.head_dim, d = cc - h * sc.head_dim;
    const int kv_heads = sc.kv_width / sc.head_dim;
    return pages + (((size_t)page * kv_heads + h) * sc.page_size + off) * sc.head_dim + d;
}

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

__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float ld_cluster_f32(uint32_t local_addr, int rank) {
    uint32_t raddr;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(raddr) : "r"(local_addr), "r"(rank));
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(raddr) : "memory");
    return v;
}

__device__ __forceinline__ uint32_t cluster_addr(uint32_t local_addr, int rank) {
    uint32_t raddr;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(raddr) : "r"(local_addr), "r"(rank));
    return raddr;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar)
                 : "memory");
}

// Persistent kernel: each CTA walks tiles blockIdx.x, blockIdx.x + gridDim.x, ... (tiles
// that share a W tile are neighbours, so they run at the same time and share it in L2).
// The producer runs ahead across tile borders; the accumulator alternates between two
// TMEM buffers, so the epilogue of one tile overlaps the main loop of the next.
//
// PAIR: the two CTAs of a cluster share a 256 x BN tile (tcgen05.mma.cta_group::2).  Each
// loads its own 128 rows of A and its own half of the tile's rows of W with plain TMA loads
// (no multicast) that count on the even CTA's barrier; the even CTA's MMA thread issues one
// instruction for both, whose operands are read from both CTAs' shared memory and whose
// result lands in both CTAs' tensor memory; its commits arrive on both CTAs' barriers
// (tcgen05.commit ... multicast::cluster).  Each CTA finishes its own 128 rows.  A CTA thus
// takes in half the bytes of W per multiply-add: the main loop of a 128 x 128 tile is bound
// by what one SM can take in from the L2, not by its tensor core.
template <int BN, typename O, bool PAIR>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                 O* __restrict__ c, const float* __restrict__ bias,
                 const float* __restrict__ resid, int m, int n, int k, long ldc, int act,
                 int* status, Scatter sc) {
    using Cfg = TileCfg<BN, PAIR>;
    extern __shared__ uint8_t smem_raw[];
    // tiles need 1024-byte alignment for the 128-byte swizzle
    uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* tiles = smem;
    uint8_t* staging = smem + (size_t)Cfg::STAGES * Cfg::STAGE_BYTES;      // [8][32][128]
    uint64_t* bars = reinterpret_cast<uint64_t*>(staging + (size_t)8 * Cfg::STG_BYTES);
    uint64_t* full_bar = bars;                       // [STAGES]  TMA -> MMA
    uint64_t* empty_bar = bars + Cfg::STAGES;        // [STAGES]  MMA -> TMA
    uint64_t* tfull_bar = bars + 2 * Cfg::STAGES;    // [2]       MMA -> epilogue
    uint64_t* tempty_bar = tfull_bar + 2;            // [2]       epilogue -> MMA
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
    volatile int* failed = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (warp == 0) GT(0);
    prb_grid_launch_dependents();     // the next kernel may set itself up while this one runs
    // A walker is a CTA, or the pair of CTAs of a cluster; it owns tiles of TM rows.
    constexpr int TM = PAIR ? 2 * BM : BM;
    const int rank = PAIR ? (int)(blockIdx.x & 1) : 0;              // CTA of the pair (cluster of 2 along x)
    const int walker = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
    const int walkers = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
    const int m_tiles = (m + TM - 1) / TM, n_tiles = (n + BN - 1) / BN;
    const int total_tiles = m_tiles * n_tiles;
    const int k_blocks = (k + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < Cfg::STAGES; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&tfull_bar[a]), 1);
            // one arrival per epilogue warp (of both CTAs, on the even CTA's barrier, in a pair)
            mbar_init(smem_u32(&tempty_bar[a]), PAIR ? 16 : 8);
        }
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        if constexpr (PAIR) {
            // one warp of each CTA of the pair, the same shared-memory offset in both
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                             smem_u32(tmem_slot)),
                         "r"((uint32_t)Cfg::TMEM_COLS)
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                             smem_u32(tmem_slot)),
                         "r"((uint32_t)Cfg::TMEM_COLS)
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if constexpr (PAIR) cluster_sync_all();           // the peer's barriers exist before anything arrives on them
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (warp == 0) GT(1);
    // barriers and tensor memory are set up; everything below reads what earlier kernels wrote
    prb_grid_wait();

    if (warp == 0) {
        // ------------------------------------------------------------ producer
        // The whole warp walks the loop and waits; one elected lane issues.  (With the loop
        // inside "if (lane == 0)" the warp is divergent for its whole life, and the copy and
        // MMA instructions, whose operands live in uniform registers, measured three times
        // as slow to issue.)
        int it = 0;                                   // k-blocks issued so far, over all tiles
        bool ok = true;
        GC_BEGIN;
        for (int tile = walker; tile < total_tiles && ok; tile += walkers) {
            const int m0 = (tile % m_tiles) * TM + rank * BM;
            const int n0 = (tile / m_tiles) * BN + (PAIR ? rank * (BN / 2) : 0);
            for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                const int s = it % Cfg::STAGES;
                ok = mbar_wait_warp(smem_u32(&empty_bar[s]), ((it / Cfg::STAGES) & 1) ^ 1, failed);
                if (!ok) {
                    if (lane == 0) prb_set_status(status, PRB_S_WAIT_TIMEOUT, 1, blockIdx.x, it);
                    break;
                }
                GC_A;
                const uint32_t fb = smem_u32(&full_bar[s]);
                const uint32_t stage = smem_u32(tiles + (size_t)s * Cfg::STAGE_BYTES);
                if (elect_one()) {
                    if constexpr (PAIR) {
                        // both CTAs' bytes count on the even CTA's barrier, which its own
                        // producer arms for both; the odd CTA only loads
                        if (rank == 0) mbar_expect_tx(fb, 2 * Cfg::STAGE_BYTES);
                        tma_load_2d_pair(stage, &map_a, fb, kb * BK, m0);
                        tma_load_2d_pair(stage + Cfg::A_BYTES, &map_w, fb, kb * BK, n0);
                    } else {
                        mbar_expect_tx(fb, Cfg::STAGE_BYTES);
                        tma_load_2d(stage, &map_a, fb, kb * BK, m0);
                        tma_load_2d(stage + Cfg::A_BYTES, &map_w, fb, kb * BK, n0);
                    }
                }
                __syncwarp();
                GC_B;
            }
        }
        if (lane == 0) GC_END(0);
        if (!ok && lane == 0) {
            // wait (bounded) for loads still in flight before the CTA may exit (the odd
            // CTA of a pair cannot see the barrier they count on: it gives them time)
            if (PAIR && rank != 0) {
                for (int i = 0; i < 1000; ++i) __nanosleep(1000);
            } else {
                const int first = it > Cfg::STAGES ? it - Cfg::STAGES : 0;
                for (int j = first; j < it; ++j) {
                    const uint32_t fb = smem_u32(&full_bar[j % Cfg::STAGES]);
                    for (uint32_t i = 0; i < WAIT_LIMIT; ++i)
                        if (mbar_try_wait(fb, (j / Cfg::STAGES) & 1)) break;
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------------------------------------------------- MMA issuer
        if (rank == 0) {
            constexpr uint32_t idesc = make_idesc(TM, BN);
            int it = 0, local = 0;
            bool ok = true;
            GC_BEGIN;
            for (int tile = walker; tile < total_tiles && ok; tile += walkers, ++local) {
                const int acc = local & 1;
                // the epilogue must have drained this accumulator (two tiles ago)
                ok = mbar_wait_warp(smem_u32(&tempty_bar[acc]), ((local >> 1) & 1) ^ 1, failed);
                if (!ok) {
                    if (lane == 0) prb_set_status(status, PRB_S_WAIT_TIMEOUT, 4, blockIdx.x, local);
                    break;
                }
                tcgen05_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * Cfg::ACC_STRIDE);
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % Cfg::STAGES;
                    ok = mbar_wait_warp(smem_u32(&full_bar[s]), (it / Cfg::STAGES) & 1, failed);
                    if (!ok) {
                        if (lane == 0) prb_set_status(status, PRB_S_WAIT_TIMEOUT, 2, blockIdx.x, it);
                        break;
                    }
                    tcgen05_fence_after();
                    GC_A;
                    if (it == 0) GT(2);
                    const uint32_t a_addr = smem_u32(tiles + (size_t)s * Cfg::STAGE_BYTES);
                    const uint64_t a_desc = make_smem_desc(a_addr);
                    const uint64_t b_desc = make_smem_desc(a_addr + Cfg::A_BYTES);
                    if (elect_one()) {
#pragma unroll
                        for (int kk = 0; kk < BK / UMMA_K; ++kk) {
                            // 16 elements = 32 bytes further inside the swizzle atom: +2 (16-byte units)
                            if constexpr (PAIR)
                                umma_bf16_pair(d_tmem, a_desc + (uint64_t)(kk * 2),
                                               b_desc + (uint64_t)(kk * 2), idesc,
                                               (kb > 0 || kk > 0) ? 1u : 0u);
                            else
                                umma_bf16(d_tmem, a_desc + (uint64_t)(kk * 2), b_desc + (uint64_t)(kk * 2),
                                          idesc, (kb > 0 || kk > 0) ? 1u : 0u);
                        }
                        // frees the stage (in both CTAs of a pair) when the MMAs retire
                        if constexpr (PAIR) umma_commit_pair(smem_u32(&empty_bar[s]));
                        else umma_commit(smem_u32(&empty_bar[s]));
                    }
                    __syncwarp();
                    GC_B;
                }
                if (ok && elect_one()) {                          // accumulator complete
                    if constexpr (PAIR) umma_commit_pair(smem_u32(&tfull_bar[acc]));
                    else umma_commit(smem_u32(&tfull_bar[acc]));
                }
                __syncwarp();
                if (local == 0) GT(3);
            }
            if (lane == 0) GC_END(2);
        }
    } else {
        // ------------------------------------------------------------ epilogue
        // Per chunk of 32 columns a warp reads 32 accumulator rows from tensor memory, one row
        // per thread, and writes them as they are into its staging tile (32 rows x 128 bytes,
        // the eight 16-byte pieces of a row XORed with the row index: no bank conflicts either
        // way).  Then it reads the tile the other way round, four whole rows per instruction
        // (eight lanes a row, four columns a lane): there it adds bias, applies the
        // activation, adds the residual, converts and stores, so that every global access
        // covers whole 128-byte (float32) or 64-byte (bfloat16) runs of a row.  A lane's four
        // columns are the same for all rows of a chunk: its bias and residual values are
        // requested a chunk ahead, before the accumulator is waited for.
        const int quarter = warp & 3;                       // TMEM lanes this warp may read
        const int half = (warp - 2) >> 2;                   // two warps share a quarter: even / odd chunks
        constexpr bool F32 = sizeof(O) == 4;
        constexpr int CH = 32;                              // columns per chunk
        const bool vec_ok = ((ldc * (long)sizeof(O)) % 16 == 0) && (((uintptr_t)c) % 16 == 0) &&
                            (((uintptr_t)bias) % 16 == 0) &&
                            (resid == nullptr ||
                             (((ldc * 4) % 16 == 0) && (((uintptr_t)resid) % 16 == 0)));
        uint8_t* warp_stage = staging + (size_t)(warp - 2) * Cfg::STG_BYTES;
        uint8_t* my_stage = warp_stage + (size_t)lane * 128;         // this thread's row
        const int rd_row = lane >> 3, rd_piece = lane & 7;           // the way back: row within four, piece
        float4 pb;                                          // prefetched bias of the lane's four columns
        float4 pr[F32 ? 8 : 1];                             // prefetched residual (float32 output)
        auto prefetch = [&](int row0, int ncol) {
            // (pieces the fast path will not use, or that do not exist, read as zero)
            const int col = ncol + rd_piece * 4;
            const bool there = vec_ok && col + 4 <= n;
            pb = (there && bias != nullptr) ? __ldg(reinterpret_cast<const float4*>(bias + col))
                                            : make_float4(0.f, 0.f, 0.f, 0.f);
            if constexpr (F32) {
#pragma unroll
                for (int it = 0; it < 8; ++it) {
                    const int rr = row0 + it * 4 + rd_row;
                    pr[it] = (there && resid != nullptr && rr < m)
                                 ? *reinterpret_cast<const float4*>(resid + (size_t)rr * ldc + col)
                                 : make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
        };
        // where in a page array the rows this lane stores on the way back begin (element
        // offset of head 0, dimension 0 of the token's slot; -1: no slot), worked out once
        // per tile, for the next tile while this one's last chunk is on its way out
        long slot_at[(!F32) ? 8 : 1];
        auto find_slots = [&](int first_row) {
            if constexpr (!F32) {
                if (sc.kv_width != 0) {
                    const int kv_heads = sc.kv_width / sc.head_dim;
#pragma unroll
                    for (int it = 0; it < 8; ++it) {
                        const int rr = first_row + it * 4 + rd_row;
                        const int slot = rr < m ? sc.slots[rr] : -1;
                        slot_at[it] = -1;
                        if (slot >= 0) {
                            const int page = slot / sc.page_size, off = slot - page * sc.page_size;
                            if (page >= sc.num_pages)
                                prb_set_status(status, PRB_S_SLOT_RANGE, rr, slot, sc.num_pages);
                            else
                                slot_at[it] = ((long)page * kv_heads * sc.page_size + off) * sc.head_dim;
                        }
                    }
                }
            }
        };
        int local = 0;
        bool ok = true;
        // the accumulator is handed back on the barrier the MMA thread waits on: this CTA's,
        // or the even CTA's of a pair
        uint32_t tempty_addr[2] = {smem_u32(&tempty_bar[0]), smem_u32(&tempty_bar[1])};
        if constexpr (PAIR) {
            tempty_addr[0] = cluster_addr(tempty_addr[0], 0);
            tempty_addr[1] = cluster_addr(tempty_addr[1], 0);
        }
        auto hand_back = [&](int acc) {
            if constexpr (PAIR) mbar_arrive_cluster(tempty_addr[acc]);
            else mbar_arrive(tempty_addr[acc]);
        };
        auto tile_m0 = [&](int t) { return (t % m_tiles) * TM + rank * BM; };
        if (walker < total_tiles && half * CH < BN) {
            prefetch(tile_m0(walker) + quarter * 32, (walker / m_tiles) * BN + half * CH);
            find_slots(tile_m0(walker) + quarter * 32);
        }
        for (int tile = walker; tile < total_tiles && ok; tile += walkers, ++local) {
            const int m0 = tile_m0(tile), n0 = (tile / m_tiles) * BN;
            const int acc = local & 1;
            const int row0 = m0 + quarter * 32;
            const int row = row0 + lane;
            ok = mbar_wait(smem_u32(&tfull_bar[acc]), (local >> 1) & 1, failed);
            if (!ok && lane == 0) prb_set_status(status, PRB_S_WAIT_TIMEOUT, 3, blockIdx.x, local);
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok) break;
            tcgen05_fence_after();
            if (warp == 2 && local == 0) GT(4);
            const int nt = tile + walkers;                  // this CTA's next tile
            if (half * CH >= BN || n0 + half * CH >= n) {   // nothing to read for this warp
                if (lane == 0) hand_back(acc);
                if (nt < total_tiles && half * CH < BN)
                    prefetch(tile_m0(nt) + quarter * 32, (nt / m_tiles) * BN + half * CH);
                continue;
            }
            // (the cache rows of this tile were looked up before the accumulator was waited for)
#pragma unroll 1
            for (int c0 = half * CH; c0 < BN; c0 += 2 * CH) {
                if (n0 + c0 >= n) break;                    // uniform across the warp
                const int ncol = n0 + c0;
                uint32_t r[32];
                tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) +
                                  (uint32_t)(acc * Cfg::ACC_STRIDE + c0), r);
                const bool last_chunk = c0 + 2 * CH >= BN || n0 + c0 + 2 * CH >= n;
                if (last_chunk) {
                    // this warp's last read of the accumulator: hand it back before the stores
                    tcgen05_fence_before();
                    __syncwarp();
                    if (lane == 0) hand_back(acc);
                }
                const int n_valid = (n - ncol) < CH ? (n - ncol) : CH;
                if (vec_ok && n_valid % 4 == 0) {
                    __syncwarp();                        // the tile's last readers are done
#pragma unroll
                    for (int q = 0; q < 8; ++q)
                        *reinterpret_cast<uint4*>(my_stage + ((q ^ (lane & 7)) << 4)) =
                            make_uint4(r[4 * q], r[4 * q + 1], r[4 * q + 2], r[4 * q + 3]);
                    __syncwarp();
                    // what this chunk needs has been requested before; keep it and request the
                    // next chunk's (of this tile, or the first of the CTA's next tile)
                    const float4 b_now = pb;
                    float4 r_now[F32 ? 8 : 1];
#pragma unroll
                    for (int it = 0; it < (F32 ? 8 : 1); ++it) r_now[it] = pr[it];
                    if (!last_chunk) prefetch(row0, ncol + 2 * CH);
                    else if (nt < total_tiles)
                        prefetch(tile_m0(nt) + quarter * 32, (nt / m_tiles) * BN + half * CH);
                    const int col = ncol + rd_piece * 4;
                    // key or value columns: the page array and the offset of the lane's four
                    // columns (inside one head: head sizes are multiples of 8) within a slot
                    O* pages = nullptr;
                    long head_at = 0;
                    if constexpr (!F32) {
                        if (sc.kv_width != 0 && col >= sc.q_width) {
                            int cc = col - sc.q_width;
                            pages = reinterpret_cast<O*>(cc < sc.kv_width ? sc.k_pages : sc.v_pages);
                            if (cc >= sc.kv_width) cc -= sc.kv_width;
                            const int h = cc / sc.head_dim;
                            head_at = (long)h * sc.page_size * sc.head_dim + (cc - h * sc.head_dim);
                        }
                    }
                    // (the activation is chosen outside the loop: chosen per element, its branches
                    // were most of the epilogue's time, a lone warp having nothing to hide them with)
                    auto way_back = [&](auto kind) {
                        constexpr int KIND = decltype(kind)::value;
#pragma unroll
                        for (int it = 0; it < 8; ++it) {
                            const int tr = it * 4 + rd_row;           // row of the tile
                            const float4 a4 = *reinterpret_cast<const float4*>(
                                warp_stage + tr * 128 + ((rd_piece ^ (tr & 7)) << 4));
                            float v0 = a4.x + b_now.x, v1 = a4.y + b_now.y, v2 = a4.z + b_now.z,
                                  v3 = a4.w + b_now.w;
                            if constexpr (KIND == 1) {
                                v0 = gelu_tanh_fast(v0); v1 = gelu_tanh_fast(v1);
                                v2 = gelu_tanh_fast(v2); v3 = gelu_tanh_fast(v3);
                            } else if constexpr (KIND == 2) {
                                v0 = prb_activate(v0, act); v1 = prb_activate(v1, act);
                                v2 = prb_activate(v2, act); v3 = prb_activate(v3, act);
                            }
                            if (row0 + tr < m) {
                                const size_t off = (size_t)(row0 + tr) * ldc + col;
                                if constexpr (F32) {
                                    *reinterpret_cast<float4*>(reinterpret_cast<float*>(c) + off) =
                                        make_float4(v0 + r_now[it].x, v1 + r_now[it].y,
                                                    v2 + r_now[it].z, v3 + r_now[it].w);
                                } else {
                                    const uint2 u = make_uint2(pack2(v0, v1), pack2(v2, v3));
                                    if (pages == nullptr || !sc.only_cache)
                                        *reinterpret_cast<uint2*>(c + off) = u;
                                    if (pages != nullptr && slot_at[it] >= 0)
                                        *reinterpret_cast<uint2*>(pages + slot_at[it] + head_at) = u;
                                }
                            }
                        }
                    };
                    if (rd_piece * 4 < n_valid) {
                        if (act == PRB_ACT_NONE) way_back(std::integral_constant<int, 0>{});
                        else if (act == PRB_ACT_GELU_TANH) way_back(std::integral_constant<int, 1>{});
                        else way_back(std::integral_constant<int, 2>{});
                    }
                } else {
                    // tail columns or unaligned rows (e.g. a vocabulary that is odd): one by one
                    O* crow = c + (size_t)row * ldc + ncol;
                    const float* rrow = resid ? resid + (size_t)row * ldc + ncol : nullptr;
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        if (j < n_valid && row < m) {
                            float x = __uint_as_float(r[j]);
                            if (bias) x += __ldg(bias + ncol + j);
                            x = epilogue_act(x, act);
                            if (rrow) x += rrow[j];
                            crow[j] = prb_from_float<O>(x);
                            if (sc.kv_width != 0 && ncol + j >= sc.q_width) {
                                O* dst = scatter_dst<O>(sc, ncol + j, sc.slots[row], row, status);
                                if (dst) *dst = prb_from_float<O>(x);
                            }
                        }
                    }
                    if (!last_chunk) prefetch(row0, ncol + 2 * CH);
                    else if (nt < total_tiles)
                        prefetch(tile_m0(nt) + quarter * 32, (nt / m_tiles) * BN + half * CH);
                }
            }
            if (nt < total_tiles) find_slots(tile_m0(nt) + quarter * 32);
            if (warp == 2 && local == 0) GT(5);
        }
        if (warp == 2) GT(6);
    }
    tcgen05_fence_before();
    __syncthreads();
    // neither CTA of a pair leaves (or frees tensor memory) while the other may still read its
    // shared memory, write its tensor memory or arrive on its barriers
    if constexpr (PAIR) cluster_sync_all();
    if (warp == 0) GT(7);
    if (warp == 1) {
        tcgen05_fence_after();
        if constexpr (PAIR)
            asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                         "r"((uint32_t)Cfg::TMEM_COLS)
                         : "memory");
        else
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                         "r"((uint32_t)Cfg::TMEM_COLS)
                         : "memory");
    }
}

// ---------------------------------------------------------------- split-K variant
// For products with too few output tiles to fill the SMs (a few hundred rows into a narrow
// output): the reduction dimension of a tile is split over the S CTAs of a thread-block
// cluster.  CTA r multiplies k-blocks [r * per, (r + 1) * per) into tensor memory, copies its
// 128 x BN float32 partial tile into its shared memory (over the stage ring, which is free by
// then), and after a cluster barrier every CTA finishes 128 / S rows: it sums their partial
// values over the cluster in rank order through distributed shared memory, adds bias, applies
// the activation, adds the residual and stores.  A second cluster barrier keeps every CTA's
// shared memory alive until its peers have read it.
template <int BN, int S, typename O>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_splitk_kernel(const __grid_constant__ CUtensorMap map_a,
                        const __grid_constant__ CUtensorMap map_w, O* __restrict__ c,
                        const float* __restrict__ bias, const float* __restrict__ resid, int m,
                        int n, int k, long ldc, int act, int* status) {
    using Cfg = TileCfg<BN>;
    constexpr int PP = BN + 1;                       // pitch of the partial tile (words)
    static_assert((size_t)BM * PP * 4 <= (size_t)Cfg::STAGES * Cfg::STAGE_BYTES,
                  "the partial tile must fit over the stage ring");
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* tiles = smem;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)Cfg::STAGES * Cfg::STAGE_BYTES);
    uint64_t* full_bar = bars;                       // [STAGES]  TMA -> MMA
    uint64_t* empty_bar = bars + Cfg::STAGES;        // [STAGES]  MMA -> TMA
    uint64_t* tfull_bar = bars + 2 * Cfg::STAGES;    // accumulator complete
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tfull_bar + 1);
    volatile int* failed = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float* part = reinterpret_cast<float*>(tiles);   // [BM][PP], after the main loop

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    prb_grid_launch_dependents();
    const int rank = (int)(blockIdx.x % S);          // clusters are S consecutive CTAs of x
    const int tile = (int)(blockIdx.x / S);
    const int m_tiles = (m + BM - 1) / BM;
    const int m0 = (tile % m_tiles) * BM, n0 = (tile / m_tiles) * BN;
    const int k_blocks = (k + BK - 1) / BK;
    const int per = (k_blocks + S - 1) / S;
    const int kb0 = rank * per;
    const int kb1 = kb0 + per < k_blocks ? kb0 + per : k_blocks;
    const int n_kb = kb1 > kb0 ? kb1 - kb0 : 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < Cfg::STAGES; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        mbar_init(smem_u32(tfull_bar), 1);
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(tmem_slot)),
                     "r"((uint32_t)Cfg::ACC_STRIDE)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    prb_grid_wait();

    // Rows rank * RPC .. of the tile are finished here; a warp takes every eighth of them, a
    // lane every 32nd column.  Their bias and residual values do not depend on the product:
    // they are requested before the cluster barrier, so their latency is off the path.
    constexpr int RPC = BM / S, CPL = BN / 32, RPW = (RPC + 7) / 8;
    float pre_b[CPL], pre_r[RPW][CPL];
    if (warp >= 2) {
#pragma unroll
        for (int j = 0; j < CPL; ++j) {
            const int col = n0 + j * 32 + lane;
            pre_b[j] = (bias && col < n) ? __ldg(bias + col) : 0.0f;
#pragma unroll
            for (int i = 0; i < RPW; ++i) {
                const int row = m0 + rank * RPC + (warp - 2) + 8 * i;
                pre_r[i][j] = (resid && col < n && row < m && (warp - 2) + 8 * i < RPC)
                                  ? resid[(size_t)row * ldc + col] : 0.0f;
            }
        }
    }
    if (warp == 0) {
        // (whole warps walk the loops, one elected lane issues: see the kernel above)
        bool ok = true;
        int it = 0;
        for (; it < n_kb; ++it) {
            const int s = it % Cfg::STAGES;
            ok = mbar_wait_warp(smem_u32(&empty_bar[s]), ((it / Cfg::STAGES) & 1) ^ 1, failed);
            if (!ok) {
                if (lane == 0) prb_set_status(status, PRB_S_WAIT_TIMEOUT, 21, blockIdx.x, it);
                break;
            }
            const uint32_t fb = smem_u32(&full_bar[s]);
            const uint32_t stage = smem_u32(tiles + (size_t)s * Cfg::STAGE_BYTES);
            if (elect_one()) {
                mbar_expect_tx(fb, Cfg::STAGE_BYTES);
                tma_load_2d(stage, &map_a, fb, (kb0 + it) * BK, m0);
                tma_load_2d(stage + Cfg::A_BYTES, &map_w, fb, (kb0 + it) * BK, n0);
            }
            __syncwarp();
        }
        if (!ok && lane == 0) {
            const int first = it > Cfg::STAGES ? it - Cfg::STAGES : 0;
            for (int j = first; j < it; ++j) {
                const uint32_t fb = smem_u32(&full_bar[j % Cfg::STAGES]);
                for (uint32_t i = 0; i < WAIT_LIMIT; ++i)
                    if (mbar_try_wait(fb, (j / Cfg::STAGES) & 1)) break;
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        constexpr uint32_t idesc = make_idesc(BM, BN);
        bool ok = true;
        for (int it = 0; it < n_kb; ++it) {
            const int s = it % Cfg::STAGES;
            ok = mbar_wait_warp(smem_u32(&full_bar[s]), (it / Cfg::STAGES) & 1, failed);
            if (!ok) {
                if (lane == 0) prb_set_status(status, PRB_S_WAIT_TIMEOUT, 22, blockIdx.x, it);
                break;
            }
            tcgen05_fence_after();
            const uint32_t a_addr = smem_u32(tiles + (size_t)s * Cfg::STAGE_BYTES);
            const uint64_t a_desc = make_smem_desc(a_addr);
            const uint64_t b_desc = make_smem_desc(a_addr + Cfg::A_BYTES);
            if (elect_one()) {
#pragma unroll
                for (int kk = 0; kk < BK / UMMA_K; ++kk)
                    umma_bf16(tmem_base, a_desc + (uint64_t)(kk * 2), b_desc + (uint64_t)(kk * 2),
                              idesc, (it > 0 || kk > 0) ? 1u : 0u);
                umma_commit(smem_u32(&empty_bar[s]));
            }
            __syncwarp();
        }
        if (ok && elect_one()) {
            if (n_kb > 0) umma_commit(smem_u32(tfull_bar));
            else mbar_arrive(smem_u32(tfull_bar));       // nothing to wait for
        }
        __syncwarp();
    } else {
        // the accumulator, one row per thread, into the partial tile
        const int quarter = warp & 3, half = (warp - 2) >> 2;
        bool ok = mbar_wait(smem_u32(tfull_bar), 0, failed);
        if (!ok && lane == 0) prb_set_status(status, PRB_S_WAIT_TIMEOUT, 23, blockIdx.x, warp);
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        tcgen05_fence_after();
        float* prow = part + (size_t)(quarter * 32 + lane) * PP;
        for (int c0 = half * 32; c0 < BN; c0 += 64) {
            uint32_t r[32];
            if (ok && n_kb > 0) {
                tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, r);
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) r[j] = 0u;
            }
#pragma unroll
            for (int j = 0; j < 32; ++j) prow[c0 + j] = __uint_as_float(r[j]);
        }
        tcgen05_fence_before();
    }
    __syncwarp();
    cluster_sync_all();                               // every CTA's partial tile is in place
    if (warp >= 2) {
        const uint32_t part_addr = smem_u32(part);
#pragma unroll
        for (int i = 0; i < RPW; ++i) {
            const int rr = (warp - 2) + 8 * i;
            const int trow = rank * RPC + rr, row = m0 + trow;
            if (rr >= RPC || row >= m) break;         // uniform across the warp
            float v[CPL][S];
#pragma unroll
            for (int j = 0; j < CPL; ++j)
#pragma unroll
                for (int s = 0; s < S; ++s)
                    v[j][s] = ld_cluster_f32(part_addr + (uint32_t)(trow * PP + j * 32 + lane) * 4, s);
#pragma unroll
            for (int j = 0; j < CPL; ++j) {
                const int col = n0 + j * 32 + lane;
                if (col >= n) continue;
                float x = v[j][0];
#pragma unroll
                for (int s = 1; s < S; ++s) x += v[j][s];           // in rank order
                x = epilogue_act(x + pre_b[j], act) + pre_r[i][j];
                c[(size_t)row * ldc + col] = prb_from_float<O>(x);
            }
        }
    }
    __syncwarp();
    cluster_sync_all();                               // the partial tiles have been read
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                     "r"((uint32_t)Cfg::ACC_STRIDE)
                     : "memory");
    }
}

// ------------------------------------------------------------------ host side
using tmap::get_map;

template <int BN, typename O>
int launch(const CUtensorMap& ma, const CUtensorMap& mw, O* c, const float* bias,
           const float* resid, int m, int n, int k, long ldc, int act, int* status,
           const Scatter& sc, cudaStream_t stream) {
    using Cfg = TileCfg<BN>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_bf16_kernel<BN, O, false>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)Cfg::SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int sm_count = prb_sm_count();
    const long tiles = (long)((n + BN - 1) / BN) * ((m + BM - 1) / BM);
    const int grid = (int)(tiles < sm_count ? tiles : sm_count);
    cudaError_t le = prb_launch_dependent(gemm_bf16_kernel<BN, O, false>, dim3(grid),
                                          dim3(GEMM_THREADS), Cfg::SMEM, stream, ma, mw, c, bias,
                                          resid, m, n, k, ldc, act, status, sc);
    if (le != cudaSuccess) return (int)le;
    return 0;
}

// CTA pairs on 256 x BN tiles: clusters of two CTAs, as many as tiles or as pairs of SMs.
template <int BN, typename O>
int launch_pair(const CUtensorMap& ma, const CUtensorMap& mw, O* c, const float* bias,
                const float* resid, int m, int n, int k, long ldc, int act, int* status,
                const Scatter& sc, cudaStream_t stream) {
    using Cfg = TileCfg<BN, true>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_bf16_kernel<BN, O, true>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)Cfg::SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const long tiles = (long)((n + BN - 1) / BN) * ((m + 2 * BM - 1) / (2 * BM));
    const long pairs = prb_sm_count() / 2;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(2 * (tiles < pairs ? tiles : pairs)));
    cfg.blockDim = dim3(GEMM_THREADS);
    cfg.dynamicSmemBytes = Cfg::SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = prb_pdl_enabled() ? 1 : 0;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = 2;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    cudaError_t le = cudaLaunchKernelEx(&cfg, gemm_bf16_kernel<BN, O, true>, ma, mw, c, bias, resid,
                                        m, n, k, ldc, act, status, sc);
    if (le != cudaSuccess) return (int)le;
    return 0;
}

template <int BN, int S, typename O>
int launch_splitk(const CUtensorMap& ma, const CUtensorMap& mw, O* c, const float* bias,
                  const float* resid, int m, int n, int k, long ldc, int act, int* status,
                  cudaStream_t stream) {
    using Cfg = TileCfg<BN>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_bf16_splitk_kernel<BN, S, O>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)Cfg::SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const long tiles = (long)((n + BN - 1) / BN) * ((m + BM - 1) / BM);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(tiles * S));
    cfg.blockDim = dim3(GEMM_THREADS);
    cfg.dynamicSmemBytes = Cfg::SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = prb_pdl_enabled() ? 1 : 0;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = S;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    cudaError_t le = cudaLaunchKernelEx(&cfg, gemm_bf16_splitk_kernel<BN, S, O>, ma, mw, c, bias,
                                        resid, m, n, k, ldc, act, status);
    if (le != cudaSuccess) return (int)le;
    return 0;
}
}  // namespace

namespace {
int gemm_bf16_entry(void* c, const void* a, const void* w, const float* bias, const float* resid,
                    int m, int n, int k, long lda, long ldw, long ldc, int act, int out_dtype,
                    int tile_n, int* status, const Scatter& sc, cudaStream_t stream) {
    if (m <= 0 || n <= 0) return 0;
    if (k <= 0) return PRB_E_SIZE;
    if (k % 8 != 0 || lda % 8 != 0 || ldw % 8 != 0 || ((uintptr_t)a) % 16 != 0 ||
        ((uintptr_t)w) % 16 != 0)
        return PRB_E_ALIGN;
    // forced: tile width in the low half, cluster size of the split-K variant in bits 16 to
    // 23, bit 24 for CTA pairs
    int pair = (tile_n >> 24) & 1;
    int split = (tile_n >> 16) & 0xff;
    tile_n &= 0xffff;
    if (tile_n == 0) {
        // The CTA with the most tiles sets the time.  A tile's main loop is bound by the
        // bytes its SM takes in (128 + width rows of 128 bytes per block of 64 along K), its
        // epilogue by the bytes it loads and stores (measured: a 128-column float32 tile with
        // residual costs what 11 blocks of the main loop do, a bfloat16 tile half of that);
        // all but a CTA's last epilogue hide behind the next tile's main loop.
        const long mt = (m + BM - 1) / BM;
        const long kb = (k + BK - 1) / BK;
        const long per_col = out_dtype == PRB_F32 ? 23 : 12;
        long best = -1;
        const long sms = prb_sm_count();
        for (int bn = 256; bn >= 32; bn -= 32) {
            const long tiles = mt * ((n + bn - 1) / bn);
            const long rounds = (tiles + sms - 1) / sms;
            const long main_loop = kb * (128 + bn) + 400, epilogue = per_col * bn;
            const long cost = (rounds - 1) * (main_loop > epilogue ? main_loop : epilogue) +
                              main_loop + epilogue;
            if (best < 0 || cost < best) { best = cost; tile_n = bn; split = 0; }
        }
        // Few tiles and a long reduction: the k-blocks of a tile over a cluster of CTAs, which
        // costs the partial tiles' way through shared memory and two cluster barriers, while a
        // CTA finishes only its share of the tile's rows (constants fitted to measurements at
        // 128 to 1,024 rows, N = 768 and 1,600, K = 768 to 6,400).
        if (sc.kv_width == 0) {
            for (int bn = 256; bn >= 64; bn -= 64) {
                const long tiles = mt * ((n + bn - 1) / bn);
                for (int sp = 2; sp <= (bn > 128 ? 2 : 8); sp *= 2) {
                    const long per = (kb + sp - 1) / sp;
                    if (tiles * sp > sms || per * (sp - 1) >= kb || per < 2) continue;
                    // (the partial tiles' way through shared memory grows with their width)
                    const long exchange = bn > 128 ? 300 + 6 * bn : 700;
                    const long cost = per * (128 + bn) + 400 + exchange + per_col * bn / 2;
                    if (cost < best) { best = cost; tile_n = bn; split = sp; }
                }
            }
        }
        // Pairs of CTAs on 256-row tiles take in half the bytes of W per multiply-add, which
        // is what bounds the main loop once every SM is loading; they cost a cluster's set-up
        // and need enough 256-row tiles to go round.  Times in nanoseconds, fitted to
        // measurements at K = 768 to 6,400 (a k-block of a single CTA: 190 + width, of a
        // pair: 230 + width / 2; an epilogue: 1,900 + 14.5 a column, a quarter more with an
        // activation): pairs win at GPT-2 XL's widths and beyond, not at GPT-2 small's.
        if (split == 0 && kb >= 16) {
            const double act_factor = (act == PRB_ACT_NONE) ? 1.0 : 1.25;
            auto model = [&](long tiles, long walkers, double per_kb, double setup, int bn) {
                const double rounds = (double)((tiles + walkers - 1) / walkers);
                const double main_loop = kb * per_kb, epilogue = (1900.0 + 14.5 * bn) * act_factor;
                return setup + (rounds - 1) * (main_loop > epilogue ? main_loop : epilogue) +
                       main_loop + epilogue;
            };
            const double single = model(mt * ((n + tile_n - 1) / tile_n), sms, 190.0 + tile_n, 1300.0, tile_n);
            double best_pair = single * 0.95;
            const long mt2 = (m + 2 * BM - 1) / (2 * BM);
            for (int bn = 256; bn >= 128; bn -= 64) {
                const double t = model(mt2 * ((n + bn - 1) / bn), sms / 2, 230.0 + bn / 2.0, 1900.0, bn);
                if (t < best_pair) { best_pair = t; tile_n = bn; pair = 1; }
            }
        }
    }
    if (split != 0 && (sc.kv_width != 0 || (split != 2 && split != 4 && split != 8) ||
                       (tile_n != 64 && tile_n != 128 && !(split == 2 && (tile_n == 192 || tile_n == 256))) ||
                       (((k + BK - 1) / BK + split - 1) / split) * (split - 1) >= (k + BK - 1) / BK))
        return PRB_E_ARG;
    if (tile_n < 32 || tile_n > 256 || tile_n % 32 != 0) return PRB_E_ARG;
    if (pair && (split != 0 || tile_n % 64 != 0)) return PRB_E_ARG;
    CUtensorMap ma, mw;
    int r = get_map(a, m, k, lda, BM, &ma);
    if (r) return r;
    r = get_map(w, n, k, ldw, pair ? tile_n / 2 : tile_n, &mw);
    if (r) return r;
#define PRB_GO(BN_)                                                                              \
    (out_dtype == PRB_F32                                                                        \
         ? launch<BN_, float>(ma, mw, (float*)c, bias, resid, m, n, k, ldc, act, status, sc, \
                              stream)                                                            \
         : launch<BN_, __nv_bfloat16>(ma, mw, (__nv_bfloat16*)c, bias, resid, m, n, k, ldc,  \
                                      act, status, sc, stream))
    if (out_dtype != PRB_F32 && out_dtype != PRB_BF16) return PRB_E_DTYPE;
#define PRB_GO_PAIR(BN_)                                                                         \
    (out_dtype == PRB_F32                                                                        \
         ? launch_pair<BN_, float>(ma, mw, (float*)c, bias, resid, m, n, k, ldc, act,        \
                                   status, sc, stream)                                           \
         : launch_pair<BN_, __nv_bfloat16>(ma, mw, (__nv_bfloat16*)c, bias, resid, m, n, k,  \
                                           ldc, act, status, sc, stream))
    if (pair) {
        switch (tile_n) {
            case 64: return PRB_GO_PAIR(64);
            case 128: return PRB_GO_PAIR(128);
            case 192: return PRB_GO_PAIR(192);
            default: return PRB_GO_PAIR(256);
        }
    }
#undef PRB_GO_PAIR
#define PRB_GO_SPLIT(BN_, S_)                                                                    \
    (out_dtype == PRB_F32                                                                        \
         ? launch_splitk<BN_, S_, float>(ma, mw, (float*)c, bias, resid, m, n, k, ldc, act,      \
                                         status, stream)                                         \
         : launch_splitk<BN_, S_, __nv_bfloat16>(ma, mw, (__nv_bfloat16*)c, bias, resid, m, n, k, \
                                                 ldc, act, status, stream))
    if (split != 0) {
        if (tile_n == 192) return PRB_GO_SPLIT(192, 2);
        if (tile_n == 256) return PRB_GO_SPLIT(256, 2);
        if (tile_n == 64)
            return split == 2 ? PRB_GO_SPLIT(64, 2) : split == 4 ? PRB_GO_SPLIT(64, 4) : PRB_GO_SPLIT(64, 8);
        return split == 2 ? PRB_GO_SPLIT(128, 2) : split == 4 ? PRB_GO_SPLIT(128, 4) : PRB_GO_SPLIT(128, 8);
    }
#undef PRB_GO_SPLIT
    switch (tile_n) {
        case 32: return PRB_GO(32);
        case 64: return PRB_GO(64);
        case 96: return PRB_GO(96);
        case 128: return PRB_GO(128);
        case 160: return PRB_GO(160);
        case 192: return PRB_GO(192);
        case 224: return PRB_GO(224);
        default: return PRB_GO(256);
    }
#undef PRB_GO
}
}  // namespace

// tile_n: 0 = choose (by M, N, K and the output type), or a multiple of 32 up to 256; with a
// cluster size of 2, 4 or 8 in bits 16 to 23, the split-K variant at tile width 64 or 128
// (cluster size 2: also 192 and 256);
// with bit 24, CTA pairs on 256-row tiles at tile width 64, 128, 192 or 256.
PRB_API int prb_gemm_bf16(void* c, const void* a, const void* w, const float* bias,
                          const float* resid, int m, int n, int k, long lda, long ldw, long ldc,
                          int act, int out_dtype, int tile_n, int* status, cudaStream_t stream) {
    Scatter sc = {};
    return gemm_bf16_entry(c, a, w, bias, resid, m, n, k, lda, ldw, ldc, act, out_dtype, tile_n,
                           status, sc, stream);
}

// The same product whose key and value columns (a fused QKV projection: n = q_width + 2 *
// kv_width) are also written to the paged cache at slots[row]; the cache has the output's
// element type and head_dim is a multiple of 8.
PRB_API int prb_gemm_bf16_scatter(void* c, const void* a, const void* w, const float* bias, int m,
                                  int n, int k, long lda, long ldw, long ldc, int act,
                                  int out_dtype, void* k_pages, void* v_pages, const int* slots,
                                  int q_width, int kv_width, int head_dim, int page_size,
                                  int num_pages, int only_cache, int* status, cudaStream_t stream) {
    if (head_dim <= 0 || head_dim % 8 != 0 || kv_width <= 0 || kv_width % head_dim != 0 ||
        page_size <= 0 || q_width < 0 || q_width % 8 != 0 || q_width + 2 * kv_width != n ||
        k_pages == nullptr || v_pages == nullptr || slots == nullptr)
        return PRB_E_ARG;
    if (((uintptr_t)k_pages) % 16 != 0 || ((uintptr_t)v_pages) % 16 != 0) return PRB_E_ALIGN;
    Scatter sc = {k_pages, v_pages, slots, q_width, kv_width, head_dim, page_size, num_pages,
                  only_cache ? 1 : 0};
    return gemm_bf16_entry(c, a, w, bias, nullptr, m, n, k, lda, ldw, ldc, act, out_dtype, 0,
                           status, sc, stream);
}
