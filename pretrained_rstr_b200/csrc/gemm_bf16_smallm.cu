// Decode-time matrix product: few rows (M <= 64 tokens), bandwidth bound.
//
//     C[M,N] = act(X[M,K] . W[N,K]^T + bias[N]) (+ resid[M,N])
//     with X = A (bfloat16), or X = LayerNorm(R) rounded to bfloat16 (R float32 [M,K]),
//     the norm fused into the product's prologue.
//
// With the roles swapped (C^T = W . X^T) a 16-row strip of W is the A operand of
// mma.sync.m16n8k16 and the tokens are the N dimension.  One CTA owns 16 output features
// for all tokens; its 8 warps split K (steps of 32, round robin) and their partial sums are
// added in warp order through shared memory, so a result does not depend on the batch.
// The k index inside an MMA is only a summation index, so a thread's 16 contiguous bytes of
// a W row are spread over two MMAs in the order they lie and the X fragments are read with
// the same permutation: no transposition anywhere.
// float32: statistics of the norm, accumulation, bias, activation, residual.
//
// Two kernels:
//  * M <= 16 and K a multiple of 64: the weights (and the tokens' activations) come to
//    shared memory by TMA (cp.async.bulk.tensor over a tensor map that views the matrix as
//    slabs of 64 columns; one copy per 16-row strip and K piece, completion on an
//    mbarrier) through a ring of buffers that runs across the strips a CTA owns.  The
//    first weight copies are issued before the wait on the previous kernel, and the fused
//    LayerNorm runs while they fly.  No copy uses cluster multicast.  Every mbarrier wait
//    is bounded: on a timeout the kernel records PRB_S_WAIT_TIMEOUT, stores nothing more,
//    waits (bounded) for its copies in flight and returns.
//  * otherwise (16 < M <= 64, other K): weights straight from global memory into operand
//    registers (gemm_smallm.cuh), four k-steps in flight per warp.
#include "gemm_smallm.cuh"
#include "tensor_map.cuh"

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
    static bool carved = false;
    if (!carved) {      // several CTAs per SM need the large shared-memory carve-out
        cudaFuncSetAttribute(gemm_smallm_kernel<MT, LN, O>,
                             cudaFuncAttributePreferredSharedMemoryCarveout,
                             cudaSharedmemCarveoutMaxShared);
        carved = true;
    }
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

// ------------------------------------------------------- M <= 16, K % 64 == 0: TMA ring
namespace stream {
using namespace smallm;
constexpr int MAX_STAGES = 8;
constexpr int MAX_CTAS_PER_SM = 2;
constexpr uint32_t WAIT_LIMIT = 1u << 22;

// How a launch cuts its work: every CTA takes the strips blockIdx.x + j * grid, each strip
// in `chunks` pieces of `kc` K elements (kc / 64 slabs of 64), which go round a ring of
// `stages` shared-memory buffers, so that the copies of the next pieces (of this strip and
// the next) are in flight while a piece is multiplied.  One TMA copy brings the 16 weight
// rows of a piece, one more the tokens' activations; a slab lands as [rows][64] with the
// 128-byte swizzle.
struct Geometry {
    int kc, chunks, stages;
    int early;      // ring buffers whose weight copies start before the previous kernel is done
};
struct Plan {
    Geometry geo;
    int grid;
    size_t smem;
};

// Tuning knobs (0 = the built-in choice): K elements per piece, CTAs per SM, ring depth,
// shared-memory budget of a CTA in KB.
int g_tune[5] = {0, 0, 0, 0, 0};   // [4]: ring buffers filled before the wait on the previous kernel

inline int sm_count() { return prb_sm_count(); }

__host__ __device__ inline size_t stage_size(int mp, bool ln, int kc) {
    return (size_t)(kc / 64) * (ROWS * 128 + (ln ? 0 : mp * 128));
}

inline Plan make_plan(int mt, bool ln, int n, int k) {
    const int mp = 8 * mt;
    const size_t fixed = (size_t)WARPS * ROWS * mp * sizeof(float) + 256 + 1024 +
                         (ln ? (size_t)mp * norm_pitch(k) * 2 + (size_t)2 * k * sizeof(float) : 0);
    const size_t sm_bytes = 224 * 1024;                // shared memory of an SM that CTAs can share
    Plan p;
    Geometry& g = p.geo;
    const int strips = (n + ROWS - 1) / ROWS;
    const int sms = sm_count();
    const int max_stages = g_tune[2] > 0 && g_tune[2] < MAX_STAGES ? g_tune[2] : MAX_STAGES;
    // Pieces as large as possible (a whole strip when a copy can hold it); as many CTAs per
    // SM as still leaves each a ring of two pieces (or all its work), because what limits a
    // short streaming kernel is the bytes in flight; the strips are then dealt out evenly.
    const int cand[] = {k, 2048, 1024, 512, 256, 128, 64};
    for (int c = 0; c < 7; ++c) {
        g.kc = cand[c];
        if (g_tune[0] > 0) g.kc = g_tune[0];
        if (g.kc > k) g.kc = k;
        if (g.kc > 64 * 256) continue;                 // a copy takes at most 256 slabs
        g.chunks = (k + g.kc - 1) / g.kc;
        const size_t stage = stage_size(mp, ln, g.kc);
        for (int per_sm = (g_tune[1] > 0 ? g_tune[1] : MAX_CTAS_PER_SM); per_sm >= 1; --per_sm) {
            size_t budget = g_tune[3] > 0 ? (size_t)g_tune[3] * 1024 : sm_bytes / per_sm - 1024;
            if (budget > 216 * 1024) budget = 216 * 1024;    // a CTA's own limit
            if (fixed + stage > budget) continue;
            const int slots = sms * per_sm;
            const int per = (strips + slots - 1) / slots;
            const int items = g.chunks * per;
            int fit = (int)((budget - fixed) / stage);
            if (fit > max_stages) fit = max_stages;
            g.stages = fit < items ? fit : items;
            if (g.stages < items && g.stages < 2 && !(g_tune[0] > 0 && per_sm == 1)) continue;
            p.grid = (strips + per - 1) / per;
            p.smem = fixed + (size_t)g.stages * stage;
            return p;
        }
        if (g_tune[0] > 0) break;
    }
    // nothing fits (a very wide K with many rows): smallest pieces, one CTA per SM
    g.kc = 64;
    g.chunks = k / 64;
    g.stages = 1;
    const int per = (strips + sms - 1) / sms;
    p.grid = (strips + per - 1) / per;
    p.smem = fixed + stage_size(mp, ln, 64);
    return p;
}
// How many ring buffers' weight copies start before the wait on the previous kernel.  All of
// them, except with the norm fused: the norm's own loads (every CTA reads the same rows) then
// come back behind whatever weights the SM has in flight, and nothing is multiplied before
// the norm is done.  With one buffer before and the others after the norm, GPT-2 XL's fc at 8
// rows (three strips a CTA) takes 9.7 us instead of 11.0 us, its qkv 9.1 instead of 9.9 us.
inline Plan finish_plan(Plan p, bool ln) {
    p.geo.early = ln ? 1 : p.geo.stages;
    if (g_tune[4] > 0 && g_tune[4] < p.geo.stages) p.geo.early = g_tune[4];
    if (g_tune[4] < 0) p.geo.early = 0;
    return p;
}

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
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "r"(addr));
    return v;
}

#ifdef PRB_TRACE
__device__ unsigned long long g_trace[1024 * 8];
#define TRACE(slot)                                                                   \
    do {                                                                              \
        if (threadIdx.x == 0 && blockIdx.x < 1024) {                                  \
            unsigned long long t__;                                                   \
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t__));                   \
            g_trace[blockIdx.x * 8 + (slot)] = t__;                                   \
        }                                                                             \
    } while (0)
#else
#define TRACE(slot)
#endif

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
    asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
}

// LayerNorm of the M rows of xf into shared memory as bfloat16 (rows beyond M are zero),
// one warp per row, gamma and beta already in shared memory (`gb`: gamma[k], beta[k]; the
// caller has waited for them and the barrier at the end publishes the rows).
template <int MT>
__device__ __forceinline__ void norm_rows_staged(const Args& a, __nv_bfloat16* xs, const float* gb) {
    constexpr int MP = 8 * MT;
    static_assert(MP % WARPS == 0 && MP / WARPS <= 2, "one or two rows per warp");
    constexpr int R = MP / WARPS;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k = a.k;
    // rows warp, warp + 8: those beyond M (or gathered from outside the input) are zero
    const float* xrow[R];
    __nv_bfloat16* dst[R];
    int live = 0;
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int t = warp + r * WARPS;
        dst[r] = xs + (size_t)t * a.xs_pitch;
        xrow[r] = t < a.m ? norm_source(a, t) : nullptr;
        if (xrow[r] != nullptr) {
            ++live;
        } else {
            for (int i = lane; i < k / 2; i += 32) reinterpret_cast<uint32_t*>(dst[r])[i] = 0u;
        }
    }
    if (live == R) {
        norm_rows_any<R>(xrow, dst, gb, k, a.beta != nullptr, a.eps);
    } else if (live > 0) {
#pragma unroll
        for (int r = 0; r < R; ++r)
            if (xrow[r] != nullptr) norm_row_any(xrow[r], dst[r], gb, k, a.beta != nullptr, a.eps);
    }
    __syncthreads();
}


template <int MT, bool LN, typename O>
__global__ void __launch_bounds__(THREADS)
gemm_stream_kernel(Args a, Geometry geo, const __grid_constant__ CUtensorMap map_w,
                   const __grid_constant__ CUtensorMap map_x) {
    constexpr int MP = 8 * MT;
    extern __shared__ __align__(128) uint8_t smem_raw[];
    float* red = reinterpret_cast<float*>(smem_raw);                         // [8][16][MP]
    uint64_t* bars = reinterpret_cast<uint64_t*>(red + WARPS * ROWS * MP);    // full[], empty[]
    volatile int* failed = reinterpret_cast<volatile int*>(bars + 2 * MAX_STAGES);
    uint8_t* after = reinterpret_cast<uint8_t*>(bars) + 256;
    float* gb = reinterpret_cast<float*>(after);                             // LN only: gamma, beta
    __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(after + (LN ? (size_t)2 * a.k * 4 : 0));
    uint8_t* ring = reinterpret_cast<uint8_t*>(xs) + (LN ? (size_t)MP * a.xs_pitch * 2 : 0);
    const uint32_t stage_base = (smem_u32(ring) + 1023u) & ~1023u;            // swizzle atoms
    const uint32_t slabs = (uint32_t)geo.kc / 64;
    const uint32_t w_bytes = slabs * ROWS * 128, x_bytes = LN ? 0u : slabs * MP * 128;
    const uint32_t stage_bytes = w_bytes + x_bytes;
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + MAX_STAGES);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, q = lane & 3;
    const int k = a.k, m = a.m, n = a.n;
    const int strips = (n + ROWS - 1) / ROWS;
    const int mine = (strips - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;   // my strips
    const int items = mine * geo.chunks;

    TRACE(0);
    prb_grid_launch_dependents();                  // the next kernel may start its own copies
    if constexpr (LN) {
        // the norm's parameters come first: they are needed early and are not in any cache
        const uint32_t gdst = smem_u32(gb);
        for (int i = threadIdx.x; i < a.k / 4; i += THREADS) {
            cp_async16(gdst + i * 16, a.gamma + i * 4);
            if (a.beta) cp_async16(gdst + (a.k + i * 4) * 4, a.beta + i * 4);
        }
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < geo.stages; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, WARPS);
        }
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    // item i = (my strip i / chunks, piece i % chunks) -> ring buffer i % stages
    auto issue_weights = [&](int i) {
        const int st = i % geo.stages;
        const int n0 = ((int)blockIdx.x + (i / geo.chunks) * (int)gridDim.x) * ROWS;
        mbar_expect_tx(full0 + 8 * st, stage_bytes);
        tma_load_slabs(stage_base + st * stage_bytes, &map_w, full0 + 8 * st, n0,
                       (i % geo.chunks) * (int)slabs);
    };
    auto issue_tokens = [&](int i) {
        if constexpr (!LN) {
            const int st = i % geo.stages;
            tma_load_slabs(stage_base + st * stage_bytes + w_bytes, &map_x, full0 + 8 * st, 0,
                           (i % geo.chunks) * (int)slabs);
        }
    };
    // The weights do not depend on the previous kernel; everything else does.
    const int first = min(geo.stages, items), early = min(geo.early, first);
    if (threadIdx.x == 0)
        for (int i = 0; i < early; ++i) issue_weights(i);
    prb_grid_wait();
    if (threadIdx.x == 0)
        for (int i = 0; i < early; ++i) issue_tokens(i);
    TRACE(1);
    if constexpr (LN) {
        cp_async_wait_all();
        __syncthreads();
        TRACE(2);
        norm_rows_staged<MT>(a, xs, gb);
    }
    if (threadIdx.x == 0)
        for (int i = early; i < first; ++i) {
            issue_weights(i);
            issue_tokens(i);
        }
    TRACE(4);

    // Four accumulators per token group (first / second MMA of a step, even / odd turn of
    // the warp) keep the MMAs independent of one another; they are added in a fixed order.
    float acc[MT][4][4];
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.0f;
    int issued = first;                            // items whose copies were started (thread 0)
    bool alive = true;
    O* out = reinterpret_cast<O*>(a.out);
    // this thread's 16-byte pieces of a slab row: logical piece 4 * (step & 1) + q of rows g,
    // g + 8 (and of token rows g, g + 8), swizzled with the row
    const uint32_t row_off = (uint32_t)g * 128;
    // the epilogue's element of this thread (ROWS * MP <= THREADS): its bias and residual are
    // fetched when a strip begins
    const int e_tok = threadIdx.x / ROWS, e_r = threadIdx.x % ROWS;
    float e_bias = 0.0f, e_resid = 0.0f;
    for (int i = 0; i < items; ++i) {
        const int st = i % geo.stages;
        const int c = i % geo.chunks;
        if (c == 0) {
            const int col = ((int)blockIdx.x + (i / geo.chunks) * (int)gridDim.x) * ROWS + e_r;
            // plain loads from addresses that are always valid (a word of shared memory when
            // there is nothing to fetch): nothing waits for them before the epilogue
            const bool mine_e = e_tok < m && col < n;
            const float* bp = (a.bias && mine_e) ? a.bias + col : red;
            const float* rp = (a.resid && mine_e) ? a.resid + (size_t)e_tok * a.ldc + col : red;
            e_bias = *bp;
            e_resid = *rp;
        }
        // refill the buffer of the item before, once every warp has released it
        if (alive && threadIdx.x == 0 && i >= 1 && i - 1 + geo.stages < items) {
            const int pi = i - 1;
            if (mbar_wait(empty0 + 8 * (pi % geo.stages), (uint32_t)(pi / geo.stages) & 1u, failed)) {
                issue_weights(pi + geo.stages);
                issue_tokens(pi + geo.stages);
                issued = pi + geo.stages + 1;
            }
        }
        // After a wait gave up nothing more is multiplied or stored, but every warp still
        // walks all items so that the CTA's barriers stay matched.
        if (i == 0) TRACE(3);
        if (alive) alive = mbar_wait(full0 + 8 * st, (uint32_t)(i / geo.stages) & 1u, failed);
        if (i == 0) TRACE(5);
        const int k0 = c * geo.kc;
        const int steps = min(geo.kc, k - k0) / KSTEP;
        const uint32_t wbase = stage_base + st * stage_bytes;
        const uint32_t xbase = wbase + w_bytes;
        auto one_step = [&](int s, int turn) {
            const uint32_t piece = (uint32_t)(((4 * (s & 1) + q) ^ g) << 4);
            const uint32_t wslab = wbase + (uint32_t)(s >> 1) * (ROWS * 128) + row_off + piece;
            const uint4 wa = lds128(wslab), wb = lds128(wslab + 8 * 128);
#pragma unroll
            for (int nt = 0; nt < MT; ++nt) {
                uint4 xv;
                if constexpr (LN) {
                    xv = *reinterpret_cast<const uint4*>(xs + (size_t)(nt * 8 + g) * a.xs_pitch + k0 +
                                                         s * KSTEP + q * 8);
                } else {
                    xv = lds128(xbase + (uint32_t)(s >> 1) * (MP * 128) + nt * 8 * 128 + row_off + piece);
                }
                // elements 0..3 of each load feed the first MMA, 4..7 the second
                mma16816(acc[nt][2 * turn], wa.x, wb.x, wa.y, wb.y, xv.x, xv.y);
                mma16816(acc[nt][2 * turn + 1], wa.z, wb.z, wa.w, wb.w, xv.z, xv.w);
            }
        };
        if (alive) {
            int s = warp;
            for (; s + WARPS < steps; s += 2 * WARPS) {
                one_step(s, 0);
                one_step(s + WARPS, 1);
            }
            if (s < steps) one_step(s, 0);
        }
        if (alive && i + geo.stages < items) {     // the buffer will be used again
            __syncwarp();
            if (lane == 0) mbar_arrive(empty0 + 8 * st);
        }
        if (c != geo.chunks - 1) continue;
        if (i == geo.chunks - 1) TRACE(6);

        // ---- the strip is complete: add the warps' partial sums in warp order
        // acc[nt][0,1]: feature g, tokens nt*8 + q*2 + {0,1}; acc[nt][2,3]: feature g + 8
#pragma unroll
        for (int nt = 0; nt < MT; ++nt) {
            float* base = red + ((size_t)warp * ROWS) * MP + nt * 8 + q * 2;
            float sum[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                sum[j] = (acc[nt][0][j] + acc[nt][1][j]) + (acc[nt][2][j] + acc[nt][3][j]);
                acc[nt][0][j] = acc[nt][1][j] = acc[nt][2][j] = acc[nt][3][j] = 0.0f;
            }
            base[(size_t)g * MP] = sum[0];
            base[(size_t)g * MP + 1] = sum[1];
            base[(size_t)(g + 8) * MP] = sum[2];
            base[(size_t)(g + 8) * MP + 1] = sum[3];
        }
        __syncthreads();
        const int n0 = ((int)blockIdx.x + (i / geo.chunks) * (int)gridDim.x) * ROWS;
        const int col = n0 + e_r;
        if (!*failed && threadIdx.x < ROWS * MP && e_tok < m && col < n) {
            const int tok = e_tok, r = e_r;            // consecutive threads: consecutive features
            float v = 0.0f;
#pragma unroll
            for (int wv = 0; wv < WARPS; ++wv) v += red[((size_t)wv * ROWS + r) * MP + tok];
            if (a.bias) v += e_bias;
            v = prb_activate(v, a.act);
            if (a.resid) v += e_resid;
            const O o = prb_from_float<O>(v);
            out[(size_t)tok * a.ldc + col] = o;
            if (a.kv_width > 0 && col >= a.q_width) {
                // this column is a key or value element of token `tok`: also to its cache slot
                const int slot = a.slots[tok];
                if (slot >= 0) {
                    const int page = slot / a.page_size, off = slot - page * a.page_size;
                    if (page >= a.num_pages) {
                        prb_set_status(a.status, PRB_S_SLOT_RANGE, tok, slot, a.num_pages);
                    } else {
                        int cc = col - a.q_width;
                        O* pages = reinterpret_cast<O*>(cc < a.kv_width ? a.k_pages : a.v_pages);
                        if (cc >= a.kv_width) cc -= a.kv_width;
                        const int h = cc / a.head_dim, d = cc - h * a.head_dim;
                        const int kv_heads = a.kv_width / a.head_dim;
                        pages[(((size_t)page * kv_heads + h) * a.page_size + off) * a.head_dim + d] = o;
                    }
                }
            }
        }
        __syncthreads();                           // `red` is free for the next strip
    }
    __syncthreads();
    TRACE(7);
    if (*failed) {
        // A wait gave up.  Record it; copies already started must land before the CTA's
        // shared memory is given back.
        if (threadIdx.x == 0) {
            prb_set_status(a.status, PRB_S_WAIT_TIMEOUT, blockIdx.x, 0, 0);
            for (int i = max(0, issued - geo.stages); i < issued; ++i) {
                const uint32_t bar = full0 + 8 * (i % geo.stages);
                const uint32_t parity = (uint32_t)(i / geo.stages) & 1u;
                for (uint32_t w = 0; w < WAIT_LIMIT; ++w)
                    if (mbar_try_wait(bar, parity)) break;
            }
        }
    }
}

// Sizes this kernel takes; anything else goes to the register-prefetch kernel.
inline bool takes(const Args& a) {
    return a.m <= 16 && a.k % 64 == 0 && a.ldw % 8 == 0 && (a.xf != nullptr || a.ldx % 8 == 0);
}

template <int MT, bool LN, typename O>
int launch_stream(Args a, cudaStream_t stream) {
    constexpr int MP = 8 * MT;
    a.xs_pitch = LN ? norm_pitch(a.k) : a.k;
    const Plan p = finish_plan(make_plan(MT, LN, a.n, a.k), LN);
    if (p.smem > 220 * 1024) return PRB_E_SIZE;
    CUtensorMap map_w, map_x;
    const int slabs = p.geo.kc / 64;
    int rc = tmap::slab_map(a.w, a.n, a.k, a.ldw, ROWS, slabs, &map_w);
    if (rc) return rc;
    if (LN) map_x = map_w;
    else if ((rc = tmap::slab_map(a.x, a.m, a.k, a.ldx, MP, slabs, &map_x)) != 0) return rc;
    static bool carved = false;
    if (!carved) {      // several CTAs per SM need the large shared-memory carve-out
        cudaFuncSetAttribute(gemm_stream_kernel<MT, LN, O>,
                             cudaFuncAttributePreferredSharedMemoryCarveout,
                             cudaSharedmemCarveoutMaxShared);
        carved = true;
    }
    static size_t configured = 0;
    if (p.smem > 48 * 1024 && p.smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_stream_kernel<MT, LN, O>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)p.smem);
        if (e != cudaSuccess) return (int)e;
        configured = p.smem;
    }
    cudaError_t e = prb_launch_dependent(gemm_stream_kernel<MT, LN, O>, dim3(p.grid), dim3(THREADS),
                                         p.smem, stream, a, p.geo, map_w, map_x);
    if (e != cudaSuccess) return (int)e;
    return 0;
}
}  // namespace stream

template <bool LN, typename O>
int dispatch_mt(const Args& a, cudaStream_t stream) {
    if (stream::takes(a))
        return a.m <= 8 ? stream::launch_stream<1, LN, O>(a, stream)
                        : stream::launch_stream<2, LN, O>(a, stream);
    if (a.m <= 8) return launch_smallm<1, LN, O>(a, stream);
    if (a.m <= 16) return launch_smallm<2, LN, O>(a, stream);
    if (a.m <= 32) return launch_smallm<4, LN, O>(a, stream);
    return launch_smallm<8, LN, O>(a, stream);
}
}  // namespace

PRB_API int prb_gemm_smallm_max_rows() { return 64; }
#ifdef PRB_TRACE
PRB_API int prb_gemm_smallm_trace(unsigned long long* host, int n) {
    return (int)cudaMemcpyFromSymbol(host, stream::g_trace, sizeof(unsigned long long) * n);
}
#endif
PRB_API int prb_gemm_smallm_tune(int kc, int ctas_per_sm, int stages, int budget_kb, int early) {
    stream::g_tune[0] = kc; stream::g_tune[1] = ctas_per_sm;
    stream::g_tune[2] = stages; stream::g_tune[3] = budget_kb; stream::g_tune[4] = early;
    return 0;
}
PRB_API int prb_gemm_smallm_max_norm_width() { return LN_MAX_K; }

// Argument check; 0 when the kernel takes these sizes.
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

// x: bfloat16 [M,K] (xf null), or xf: float32 rows to be LayerNorm-ed first with gamma, beta
// (may be null) and eps: row t of the product from row xf_rows[t] of xf's xf_rows_in rows
// (xf_rows null: from row t).  m <= 64, k % 8 == 0, pitches multiples of 8 (4 for xf).
// kv_width > 0: the product is a fused QKV projection and its key and value columns are
// also written to the paged cache at slots[token] (the cache has the output's element type).
PRB_API int prb_gemm_smallm(void* out, const void* x, const float* xf, const int* xf_rows,
                            int xf_rows_in, const float* gamma,
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
    a.xf_rows = xf != nullptr ? xf_rows : nullptr;
    a.xf_rows_in = xf_rows_in;
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
