// Matrix product for a few dozen rows (17..64 tokens: decoding a large batch) with the
// reduction dimension split over a thread-block cluster:
//
//     C[M,N] = act(A[M,K] . W[N,K]^T + bias[N]) (+ resid[M,N]),   M <= 64, K % 64 == 0
//
// With so few rows a product has too few output tiles to fill the GPU when every tile walks
// all of K (N = 768: 12 tiles of 64 columns), and what bounds a tile is the bytes its SM
// takes in.  Here a cluster of S CTAs shares one tile of NB output columns: CTA r multiplies
// the r-th part of K (A and W slices come by TMA through a ring of shared-memory stages,
// 128-byte swizzle, mma.sync m16n8k16 with ldmatrix), keeps its partial tile in shared
// memory, and after a cluster barrier every CTA sums, in rank order, the rows r, r + S, ...
// of all partial tiles through distributed shared memory and runs the epilogue for them
// (bias, activation, residual, store).  S depends on K and N only, and a row's sum is
// taken in a fixed order, so a row's result does not depend on the batch.
// No TMA load uses cluster multicast.  Every mbarrier wait is bounded: on a timeout the
// kernel records PRB_S_WAIT_TIMEOUT, stores nothing, waits (bounded) for its copies in
// flight and leaves through the same cluster barriers as its peers.
#include "common.cuh"
#include "tensor_map.cuh"

#ifdef PRB_TRACE
__device__ unsigned long long g_midm_trace[512 * 8];
#define MT_TRACE(slot)                                                                \
    do {                                                                              \
        const int cta__ = blockIdx.z * gridDim.x + blockIdx.x;                        \
        if (threadIdx.x == 0 && cta__ < 512) {                                        \
            unsigned long long t__;                                                   \
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t__));                   \
            g_midm_trace[cta__ * 8 + (slot)] = t__;                                   \
        }                                                                             \
    } while (0)
PRB_API int prb_gemm_midm_trace(unsigned long long* host, int n) {
    return (int)cudaMemcpyFromSymbol(host, g_midm_trace, sizeof(unsigned long long) * n);
}
#else
#define MT_TRACE(slot)
#endif

namespace {
constexpr int THREADS = 256;
constexpr int WARPS = 8;
constexpr int MROWS = 64;           // token rows of a tile (rows beyond M are zero)
constexpr int KC = 2;               // 64-column slabs per stage
constexpr int STAGES = 4;
constexpr uint32_t WAIT_LIMIT = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* failed) {
    for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 255u) == 255u && *failed) return false;
    }
    *failed = 1;
    return false;
}
// x is always 0 (a slab is 64 elements wide), so the 16-byte rule on x holds.
__device__ __forceinline__ void tma_load_slabs(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                               int row, int slab) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4, %5}], [%2];" ::"r"(dst),
        "l"(map), "r"(bar), "r"(0), "r"(row), "r"(slab)
        : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
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

struct Args {
    void* c;
    const float* bias;
    const float* resid;
    int m, n, k;
    long ldc;
    int act;
    int splits;                     // CTAs of a cluster (grid z)
    int* status;
};

// Address of the 16-byte piece `piece` (0..7) of row `row` in a slab of [rows][64] bfloat16
// written by TMA with the 128-byte swizzle (slab base 1024-byte aligned).
__device__ __forceinline__ uint32_t swz(uint32_t slab, int row, int piece) {
    return slab + (uint32_t)row * 128 + (uint32_t)((piece ^ (row & 7)) << 4);
}

template <int NB, typename O>
__global__ void __launch_bounds__(THREADS)
gemm_midm_kernel(Args a, const __grid_constant__ CUtensorMap map_a,
                 const __grid_constant__ CUtensorMap map_w) {
    constexpr int NT = NB / 16;                       // 8-column MMA tiles per warp: 2 or 4
    constexpr uint32_t A_BYTES = KC * MROWS * 128, W_BYTES = KC * NB * 128;
    constexpr uint32_t STAGE_BYTES = A_BYTES + W_BYTES;
    constexpr int PP = NB + 1;                        // pitch of the partial tile (floats)
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t ring = smem_u32(smem);
    float* part = reinterpret_cast<float*>(smem + STAGES * STAGE_BYTES);       // [64][PP]
    uint64_t* bars = reinterpret_cast<uint64_t*>(part + MROWS * PP + 1);
    bars = reinterpret_cast<uint64_t*>(((uintptr_t)bars + 7) & ~(uintptr_t)7);
    volatile int* failed = reinterpret_cast<volatile int*>(bars + 2 * STAGES);
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * NB;
    const int rank = blockIdx.z, S = a.splits;
    // this CTA's part of K, in slabs of 64
    const int slabs = a.k / 64;
    const int slab_lo = (int)((long)slabs * rank / S), slab_hi = (int)((long)slabs * (rank + 1) / S);
    const int items = (slab_hi - slab_lo + KC - 1) / KC;

    MT_TRACE(0);
    prb_grid_launch_dependents();
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, WARPS);
        }
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    auto issue_w = [&](int i) {
        const int st = i % STAGES;
        mbar_expect_tx(full0 + 8 * st, STAGE_BYTES);
        tma_load_slabs(ring + st * STAGE_BYTES + A_BYTES, &map_w, full0 + 8 * st, n0,
                       slab_lo + i * KC);
    };
    auto issue_a = [&](int i) {
        const int st = i % STAGES;
        tma_load_slabs(ring + st * STAGE_BYTES, &map_a, full0 + 8 * st, 0, slab_lo + i * KC);
    };
    // The weights do not depend on the previous kernel; the activations do.
    const int first = min(STAGES, items);
    if (threadIdx.x == 0)
        for (int i = 0; i < first; ++i) issue_w(i);
    prb_grid_wait();
    if (threadIdx.x == 0)
        for (int i = 0; i < first; ++i) issue_a(i);

    // warp -> 16 token rows (mt) and NB/2 columns (nh)
    const int mt = warp & 3, nh = warp >> 2;
    float acc[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.0f;
    int issued = first;
    bool alive = true;
    for (int i = 0; i < items; ++i) {
        const int st = i % STAGES;
        if (alive && threadIdx.x == 0 && i >= 1 && i - 1 + STAGES < items) {
            const int pi = i - 1;
            if (mbar_wait(empty0 + 8 * (pi % STAGES), (uint32_t)(pi / STAGES) & 1u, failed)) {
                issue_w(pi + STAGES);
                issue_a(pi + STAGES);
                issued = pi + STAGES + 1;
            }
        }
        if (alive) alive = mbar_wait(full0 + 8 * st, (uint32_t)(i / STAGES) & 1u, failed);
        if (i == 0) MT_TRACE(1);
        if (i == items - 1) MT_TRACE(2);
        if (alive) {
            const uint32_t abase = ring + st * STAGE_BYTES, wbase = abase + A_BYTES;
            // slabs of this stage that lie inside this CTA's part of K (a copy may have run
            // past it into the next CTA's slabs; those are simply not multiplied)
            const int valid = min(KC, slab_hi - (slab_lo + i * KC));
            for (int sl = 0; sl < valid; ++sl) {
                const uint32_t aslab = abase + sl * (MROWS * 128), wslab = wbase + sl * (NB * 128);
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) {          // four k-steps of 16 in a slab
                    uint32_t af[4];
                    ldmatrix_x4(af, swz(aslab, mt * 16 + (lane & 15), kk * 2 + (lane >> 4)));
#pragma unroll
                    for (int np = 0; np < NT / 2; ++np) {     // two 8-column tiles per ldmatrix
                        uint32_t bf[4];
                        const int nrow = nh * (NB / 2) + np * 16 + ((lane >> 4) << 3) + (lane & 7);
                        ldmatrix_x4(bf, swz(wslab, nrow, kk * 2 + ((lane >> 3) & 1)));
                        mma16816(acc[2 * np], af, bf[0], bf[1]);
                        mma16816(acc[2 * np + 1], af, bf[2], bf[3]);
                    }
                }
            }
            if (i + STAGES < items) {
                __syncwarp();
                if (lane == 0) mbar_arrive(empty0 + 8 * st);
            }
        }
    }
    MT_TRACE(3);
    // ---- this CTA's partial tile -> shared memory
    {
        const int g = lane >> 2, q = lane & 3;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const int col = nh * (NB / 2) + nt * 8 + q * 2;
            float* p0 = part + (size_t)(mt * 16 + g) * PP + col;
            float* p1 = part + (size_t)(mt * 16 + g + 8) * PP + col;
            p0[0] = acc[nt][0]; p0[1] = acc[nt][1];
            p1[0] = acc[nt][2]; p1[1] = acc[nt][3];
        }
    }
    __syncthreads();
    const bool bad_here = *failed != 0;
    if (bad_here && threadIdx.x == 0) {
        prb_set_status(a.status, PRB_S_WAIT_TIMEOUT, blockIdx.x, rank, 0);
        for (int i = max(0, issued - STAGES); i < issued; ++i) {
            const uint32_t bar = full0 + 8 * (i % STAGES);
            const uint32_t parity = (uint32_t)(i / STAGES) & 1u;
            for (uint32_t w = 0; w < WAIT_LIMIT; ++w)
                if (mbar_try_wait(bar, parity)) break;
        }
        part[MROWS * PP] = 1.0f;                          // peers see that this part is missing
    } else if (threadIdx.x == 0) {
        part[MROWS * PP] = 0.0f;
    }
    MT_TRACE(4);
    cluster_sync_all();                                   // every CTA's partial tile is in place
    MT_TRACE(5);
    // ---- rows rank, rank + S, ...: sum over the cluster in rank order, epilogue, store
    bool any_bad = false;
    for (int r = 0; r < S; ++r) any_bad |= ld_cluster_f32(smem_u32(part + MROWS * PP), r) != 0.0f;
    if (!any_bad) {
        O* out = reinterpret_cast<O*>(a.c);
        constexpr int RPP = THREADS / NB;                 // rows per pass
        const int col = threadIdx.x % NB, rsub = threadIdx.x / NB;
        const int gcol = n0 + col;
        const float bias = (a.bias && gcol < a.n) ? a.bias[gcol] : 0.0f;
        for (int row = rank + rsub * S; row < a.m && row < MROWS; row += RPP * S) {
            const uint32_t addr = smem_u32(part + (size_t)row * PP + col);
            float pv[8];                                  // all requested before any is used
#pragma unroll
            for (int r = 0; r < 8; ++r) pv[r] = r < S ? ld_cluster_f32(addr, r) : 0.0f;
            float v = 0.0f;
#pragma unroll
            for (int r = 0; r < 8; ++r) v += pv[r];
            if (gcol < a.n) {
                v = prb_activate(v + bias, a.act);
                if (a.resid) v += a.resid[(size_t)row * a.ldc + gcol];
                out[(size_t)row * a.ldc + gcol] = prb_from_float<O>(v);
            }
        }
    }
    MT_TRACE(6);
    cluster_sync_all();                                   // the partial tiles have been read
    MT_TRACE(7);
}

template <int NB, typename O>
int launch_midm(const Args& a, const CUtensorMap& ma, const CUtensorMap& mw, cudaStream_t stream) {
    constexpr size_t smem = 1024 + (size_t)STAGES * KC * (MROWS + NB) * 128 +
                            (size_t)(MROWS * (NB + 1) + 2) * 4 + 16 + 2 * STAGES * 8 + 16;
    static bool configured = false;
    if (!configured) {
        cudaFuncSetAttribute(gemm_midm_kernel<NB, O>, cudaFuncAttributePreferredSharedMemoryCarveout,
                             cudaSharedmemCarveoutMaxShared);
        cudaError_t e = cudaFuncSetAttribute(gemm_midm_kernel<NB, O>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((a.n + NB - 1) / NB, 1, a.splits);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = prb_pdl_enabled() ? 1 : 0;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = 1;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = (unsigned)a.splits;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_midm_kernel<NB, O>, a, ma, mw);
    if (e != cudaSuccess) return (int)e;
    return 0;
}
}  // namespace

// 1 when the kernel takes these sizes (else the caller uses another product kernel).
PRB_API int prb_gemm_midm_supports(int m, int n, int k) {
    return m >= 1 && m <= MROWS && n >= 1 && k >= 64 && k % 64 == 0 ? 1 : 0;
}

// a: bfloat16 [M,K]; w: bfloat16 [N,K]; c: bfloat16 or float32 [M,N] (resid float32, may
// alias c).  M <= 64, K a multiple of 64, pitches multiples of 8 elements.
PRB_API int prb_gemm_midm(void* c, const void* a, const void* w, const float* bias,
                          const float* resid, int m, int n, int k, long lda, long ldw, long ldc,
                          int act, int out_dtype, int* status, cudaStream_t stream) {
    if (m <= 0 || n <= 0) return 0;
    if (!prb_gemm_midm_supports(m, n, k)) return PRB_E_SIZE;
    if (lda % 8 != 0 || ldw % 8 != 0 || ((uintptr_t)a) % 16 != 0 || ((uintptr_t)w) % 16 != 0)
        return PRB_E_ALIGN;
    if (out_dtype != PRB_F32 && out_dtype != PRB_BF16) return PRB_E_DTYPE;
    // Tile width and cluster size from N and K only.  All CTAs should run at once (one per
    // SM with 64-column tiles, two with 32-column tiles); within that, the split that gives
    // an SM the fewest bytes to take in (its CTAs' slices of A and W) wins.
    const int slabs = k / 64;
    const int sms = prb_sm_count();
    int nb = 32, splits = 1;
    long best = -1;
    for (int cand = 64; cand >= 32; cand /= 2) {
        const int tiles = (n + cand - 1) / cand;
        const int slots = sms * (cand == 64 ? 1 : 2);
        int s = slots / tiles;
        if (s > 8) s = 8;
        if (s > slabs / 2) s = slabs / 2;
        if (s < 1) s = 1;
        const long per_cta = (long)(MROWS + cand) * 2 * ((long)k / s);
        const long ctas = (long)tiles * s;
        const long per_sm = per_cta * ((ctas + sms - 1) / sms);
        if (best < 0 || per_sm < best) { best = per_sm; nb = cand; splits = s; }
    }
    CUtensorMap ma, mw;
    int rc = tmap::slab_map(a, m, k, lda, MROWS, KC, &ma);
    if (rc) return rc;
    if ((rc = tmap::slab_map(w, n, k, ldw, nb, KC, &mw)) != 0) return rc;
    Args args{c, bias, resid, m, n, k, ldc, act, splits, status};
    if (nb == 64)
        return out_dtype == PRB_F32 ? launch_midm<64, float>(args, ma, mw, stream)
                                    : launch_midm<64, __nv_bfloat16>(args, ma, mw, stream);
    return out_dtype == PRB_F32 ? launch_midm<32, float>(args, ma, mw, stream)
                                : launch_midm<32, __nv_bfloat16>(args, ma, mw, stream);
}
