// A whole decode step as ONE persistent kernel.
//
// A decode step of a small model is a chain of about sixty short, dependent operations
// (norm + projection, attention, projection, ...).  Launched one by one, even as a CUDA graph
// with programmatic dependent launch, each costs its launch gap, the latency of its first
// reads from HBM and the round trips of its dependent reads; together several times the
// work.  Here the step's operations are recorded once as a list of `Op` records in device
// memory (a "program"), and one cooperative kernel with one CTA per SM interprets the list.
// What makes it fast is that nothing that does not depend on the chain is waited for:
//
//  * every CTA knows, from the list alone, which weights and which cached keys and values it
//    will need for the operation after the next, and asks for them (TMA into shared memory)
//    as soon as its share of the current operation is done, before it waits for the others;
//  * the grid-wide barrier between operations is split into an arrival and a wait, with those
//    requests in between; it is a counter in global memory, about 1.3 us a round on a B200;
//  * after the barrier an operation only reads the activations the previous one wrote
//    (from the L2), multiplies from shared memory and writes its own.
//
// Shared memory: an area for the running product's activations (normalised rows), and an
// arena in which consecutive operations' regions (weights; key and value rings) lie at
// opposite ends, so that an operation's region is free for the operation after the next as
// soon as this CTA has finished with it.
//
// The products are the decode-time products of gemm_bf16_smallm.cu (a 16-row strip of W is
// the A operand of mma.sync.m16n8k16, tokens are N, the 8 warps split K and are added in warp
// order, optional fused LayerNorm, bias, activation, residual, scatter of keys and values to
// the paged cache); attention is the ring kernel's own device code (attention_decode_ring.cuh);
// embedding and the norm of the wanted rows are the device functions of elementwise.cuh.
//
// Limits: up to 8 tokens a step, reductions that are multiples of 64, head size 64.  A step
// that does not fit is refused when it is recorded and runs as separate kernels instead.
//
// Every wait is bounded.  A CTA that gives up raises a flag in global memory that all
// spinning CTAs poll, records PRB_S_WAIT_TIMEOUT, waits (bounded) for its own copies in
// flight, and every CTA leaves the kernel.
#include <vector>

#include "attention_decode_ring.cuh"
#include "elementwise.cuh"
#include "gemm_smallm.cuh"
#include "tensor_map.cuh"

int prb_gemm_smallm_check(const void* x, const float* xf, const float* gamma, const float* beta,
                          const void* w, int m, int n, int k, long ldx, long ldw);

#ifdef PRB_TRACE
// device-side timestamps (thread 0 of every CTA), per operation: its turn begins, its share
// is done (arrival), the requests for the operation after the next are out, the wait is over
__device__ unsigned long long g_prog_trace[128 * 160 * 8];
#define PROG_TRACE(op, slot)                                                          \
    do {                                                                              \
        if (threadIdx.x == 0 && (op) < 128 && blockIdx.x < 160) {                     \
            unsigned long long t__;                                                   \
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t__));                   \
            g_prog_trace[((op) * 160 + blockIdx.x) * 8 + (slot)] = t__;               \
        }                                                                             \
    } while (0)
PRB_API int prb_program_trace(unsigned long long* host, int n) {
    return (int)cudaMemcpyFromSymbol(host, g_prog_trace, sizeof(unsigned long long) * n);
}
__device__ int g_prog_op = 0;     // (the operation that runs: where gemm_run's stamps go)
#define GEMM_TRACE(slot) PROG_TRACE(g_prog_op_local, slot)
#else
#define PROG_TRACE(op, slot)
#define GEMM_TRACE(slot)
#endif

namespace {
using smallm::KSTEP;
using smallm::ROWS;
using smallm::WARPS;
constexpr int PROG_THREADS = 256;
constexpr int MP = 8;                          // token rows of a product (padded)
constexpr int MAX_ROWS = 8;
constexpr int GEMM_STAGES = 8;                 // most ring buffers of a product
constexpr unsigned SPIN_LIMIT = 1u << 22;
constexpr uint32_t WAIT_LIMIT = 1u << 22;
constexpr size_t SMEM_TOTAL = 211 * 1024;      // dynamic shared memory of the kernel
constexpr size_t MAX_KC = 3072;                // most K elements of a ring item (96 KB of weights)
constexpr size_t CHUNK_KC = 2048;              // K elements of an item when a strip is cut up

enum OpType : int { OP_END = 0, OP_EMBED = 1, OP_NORM = 2, OP_GEMM = 3, OP_ATTN = 4 };

struct alignas(64) Op {
    CUtensorMap map_a;          // GEMM: the weights as 64-column slabs; ATTN: the keys
    CUtensorMap map_b;          // ATTN: the values
    int type;
    int units;                  // EMBED / NORM: rows; GEMM: 16-row strips
    int flags;                  // GEMM: bit 0 fused norm, bit 1 float32 output; NORM: bit 1
                                // float32 output; EMBED: bit 1 float32 tables
    int kc, chunks, stages;     // GEMM: K elements per ring item, items per strip, ring buffers
    int region_bytes;           // what the operation keeps in the arena
    int x_bytes;                // what it needs in the activation area
    union {
        smallm::Args gemm;
        ring::RingArgs attn;
        elementwise::EmbedArgs embed;
        elementwise::NormArgs norm;
    };
};

struct Program {
    std::vector<Op> ops;
    size_t x_bytes = 0;          // activation area (the largest any operation needs)
    bool laid_out = false;
};

// ------------------------------------------------------------------ small device helpers
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* failed) {
    for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
        if (ring::mbar_try_wait(bar, parity)) return true;
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
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
    asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
}

// ---- the grid-wide barrier, in two halves.  bar[0]: arrivals so far; bar[1]: somebody gave up.
__device__ __forceinline__ void grid_arrive(unsigned* bar) {
    __syncthreads();                               // the CTA's writes come before thread 0's release
    if (threadIdx.x == 0) asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(bar) : "memory");
}
__device__ __forceinline__ bool grid_wait(unsigned* bar, unsigned target, int* sh_flag, int* status,
                                          int op_index) {
    if (threadIdx.x == 0) {
        int ok = 1;
        for (unsigned spins = 0;; ++spins) {
            unsigned v;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(bar) : "memory");
            if (v >= target) break;
            if ((spins & 63u) == 63u || spins > SPIN_LIMIT) {
                unsigned failed;
                asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(failed) : "l"(bar + 1) : "memory");
                if (failed != 0u || spins > SPIN_LIMIT) {
                    if (failed == 0u) {
                        atomicExch(&bar[1], 1u);
                        prb_set_status(status, PRB_S_WAIT_TIMEOUT, 9, (int)blockIdx.x, op_index);
                    }
                    ok = 0;
                    break;
                }
            }
        }
        __threadfence();
        *sh_flag = ok;
    }
    __syncthreads();
    return *sh_flag != 0;
}

// What a product keeps per side of the arena.
struct GemmBars {
    unsigned long long full[GEMM_STAGES];
    unsigned long long empty[GEMM_STAGES];
    int valid;                  // how many of each hold a valid (idle) barrier object
};

__device__ __forceinline__ int my_strips(const Op& op) {
    return (op.units - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
}
__device__ __forceinline__ uint32_t item_bytes(const Op& op) { return (uint32_t)(op.kc / 64) * ROWS * 128; }
__device__ __forceinline__ uint32_t gb_bytes(const Op& op) {     // gamma and beta, ahead of the weights
    return (op.flags & 1) ? (((uint32_t)op.gemm.k * 8u + 1023u) & ~1023u) : 0u;
}

// Item i of this CTA = (its strip i / chunks, piece i % chunks) -> ring buffer i % stages.
// (`op`: the copy in shared memory; `map`: the tensor map, which has to stay in global memory.)
__device__ __forceinline__ void gemm_issue(const Op& op, const CUtensorMap* map, uint32_t region,
                                           GemmBars& gb, int i) {
    const int st = i % op.stages;
    const int n0 = ((int)blockIdx.x + (i / op.chunks) * (int)gridDim.x) * ROWS;
    const uint32_t full = smem_u32(&gb.full[st]);
    ring::mbar_expect_tx(full, item_bytes(op));
    tma_load_slabs(region + gb_bytes(op) + st * item_bytes(op), map, full, n0,
                   (i % op.chunks) * (op.kc / 64));
}

// Before the operation's turn: barriers, the norm's parameters, the first ring buffers.
__device__ __noinline__ void gemm_prefetch(const Op& op, const CUtensorMap* map, uint32_t region,
                                              GemmBars& gb) {
    const int items = my_strips(op) * op.chunks;
    if (items <= 0) return;
    if (op.flags & 1) {
        const smallm::Args& a = op.gemm;
        for (int i = threadIdx.x; i < a.k / 4; i += PROG_THREADS) {
            cp_async16(region + i * 16, a.gamma + i * 4);
            if (a.beta) cp_async16(region + (a.k + i * 4) * 4, a.beta + i * 4);
        }
    }
    if (threadIdx.x == 0) {
        // (an mbarrier object is invalidated before its memory takes a new one)
        for (int s = 0; s < gb.valid; ++s) {
            ring::mbar_inval(smem_u32(&gb.full[s]));
            ring::mbar_inval(smem_u32(&gb.empty[s]));
        }
        for (int s = 0; s < op.stages; ++s) {
            ring::mbar_init(smem_u32(&gb.full[s]), 1);
            ring::mbar_init(smem_u32(&gb.empty[s]), WARPS);
        }
        gb.valid = op.stages;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        // (generic-proxy reads of the region by an earlier operation come before these copies)
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        const int first = min(op.stages, items);
        for (int i = 0; i < first; ++i) gemm_issue(op, map, region, gb, i);
    }
}

// The rows the product multiplies, as bfloat16 in shared memory (rows beyond M are zero):
// LayerNorm of the float32 rows, or the bfloat16 rows as they are.  One warp per row.
__device__ __noinline__ void stage_rows(const Op& op, __nv_bfloat16* xs, const float* gb) {
    const smallm::Args& a = op.gemm;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k = a.k;
    const int pitch = smallm::norm_pitch(k);
    for (int t = warp; t < MP; t += WARPS) {
        __nv_bfloat16* dst = xs + (size_t)t * pitch;
        if (t >= a.m) {
            for (int i = lane; i < k / 2; i += 32) reinterpret_cast<uint32_t*>(dst)[i] = 0u;
            continue;
        }
        if (!(op.flags & 1)) {
            const uint4* src = reinterpret_cast<const uint4*>(a.x + (size_t)t * a.ldx);
            for (int i = lane; i < k / 8; i += 32) reinterpret_cast<uint4*>(dst)[i] = __ldcg(src + i);
            continue;
        }
        smallm::norm_row_any(a.xf + (size_t)t * a.ldx, dst, gb, k, a.beta != nullptr, a.eps);
    }
}

// The operation's turn: everything another CTA wrote is visible.
__device__ __noinline__ void gemm_run(const Op& op, const CUtensorMap* map, uint32_t region,
                                         GemmBars& gb, __nv_bfloat16* xs, float* red,
                                         volatile int* failed, int g_prog_op_local = 0) {
    const smallm::Args& a = op.gemm;
    const int mine = my_strips(op);
    const int op_stages = op.stages, op_chunks = op.chunks, op_kc = op.kc;
    const int items = mine * op_chunks;
    if (items <= 0) return;                          // (uniform in the CTA)
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, q = lane & 3;
    const int k = a.k, m = a.m, n = a.n;
    const int pitch = smallm::norm_pitch(k);
    if (op.flags & 1) cp_async_wait_all();           // this thread's pieces of gamma and beta
    __syncthreads();
    stage_rows(op, xs, reinterpret_cast<const float*>(__cvta_shared_to_generic(region)));
    __syncthreads();
    GEMM_TRACE(4);

    const uint32_t wregion = region + gb_bytes(op);
    const uint32_t ibytes = item_bytes(op);
    float acc[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f;
    bool alive = true;
    const bool f32_out = (op.flags & 2) != 0;
    const uint32_t row_off = (uint32_t)g * 128;
    const int e_tok = threadIdx.x / ROWS, e_r = threadIdx.x % ROWS;     // the epilogue's element
    float e_bias = 0.0f, e_resid = 0.0f;
    for (int i = 0; i < items; ++i) {
        const int st = i % op_stages;
        const int c = i % op_chunks;
        if (c == 0) {
            const int col = ((int)blockIdx.x + (i / op_chunks) * (int)gridDim.x) * ROWS + e_r;
            const bool mine_e = threadIdx.x < ROWS * MP && e_tok < m && col < n;
            e_bias = (a.bias && mine_e) ? a.bias[col] : 0.0f;
            e_resid = (a.resid && mine_e) ? __ldcg(a.resid + (size_t)e_tok * a.ldc + col) : 0.0f;
        }
        // refill the buffer of the item before, once every warp has released it
        if (alive && threadIdx.x == 0 && i >= 1 && i - 1 + op_stages < items) {
            const int pi = i - 1;
            if (mbar_wait(smem_u32(&gb.empty[pi % op_stages]), (uint32_t)(pi / op_stages) & 1u, failed))
                gemm_issue(op, map, region, gb, pi + op_stages);
        }
        if (alive) alive = mbar_wait(smem_u32(&gb.full[st]), (uint32_t)(i / op_stages) & 1u, failed);
        if (i == 0) GEMM_TRACE(5);
        const int k0 = c * op_kc;
        const int steps = min(op_kc, k - k0) / KSTEP;
        const uint32_t wbase = wregion + st * ibytes;
        auto one_step = [&](int s, int turn) {
            const uint32_t piece = (uint32_t)(((4 * (s & 1) + q) ^ g) << 4);
            const uint32_t wslab = wbase + (uint32_t)(s >> 1) * (ROWS * 128) + row_off + piece;
            const uint4 wa = lds128(wslab), wb = lds128(wslab + 8 * 128);
            const uint4 xv = *reinterpret_cast<const uint4*>(xs + (size_t)g * pitch + k0 + s * KSTEP + q * 8);
            // elements 0..3 of each load feed the first MMA, 4..7 the second
            smallm::mma16816(acc[2 * turn], wa.x, wb.x, wa.y, wb.y, xv.x, xv.y);
            smallm::mma16816(acc[2 * turn + 1], wa.z, wb.z, wa.w, wb.w, xv.z, xv.w);
        };
        if (alive) {
            int s = warp;
            for (; s + WARPS < steps; s += 2 * WARPS) {
                one_step(s, 0);
                one_step(s + WARPS, 1);
            }
            if (s < steps) one_step(s, 0);
        }
        if (alive && i + op_stages < items) {        // the buffer will be used again
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&gb.empty[st]));
        }
        if (c != op_chunks - 1) continue;
        if (i == op_chunks - 1) GEMM_TRACE(6);
        // ---- the strip is complete: add the warps' partial sums in warp order
        {
            float* base = red + ((size_t)warp * ROWS) * MP + q * 2;
            float sum[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                sum[j] = (acc[0][j] + acc[1][j]) + (acc[2][j] + acc[3][j]);
                acc[0][j] = acc[1][j] = acc[2][j] = acc[3][j] = 0.0f;
            }
            base[(size_t)g * MP] = sum[0];
            base[(size_t)g * MP + 1] = sum[1];
            base[(size_t)(g + 8) * MP] = sum[2];
            base[(size_t)(g + 8) * MP + 1] = sum[3];
        }
        __syncthreads();
        const int n0 = ((int)blockIdx.x + (i / op_chunks) * (int)gridDim.x) * ROWS;
        const int col = n0 + e_r;
        if (!*failed && threadIdx.x < ROWS * MP && e_tok < m && col < n) {
            const int tok = e_tok, r = e_r;
            float v = 0.0f;
#pragma unroll
            for (int wv = 0; wv < WARPS; ++wv) v += red[((size_t)wv * ROWS + r) * MP + tok];
            if (a.bias) v += e_bias;
            v = prb_activate(v, a.act);
            if (a.resid) v += e_resid;
            const __nv_bfloat16 o16 = __float2bfloat16_rn(v);
            if (f32_out) reinterpret_cast<float*>(a.out)[(size_t)tok * a.ldc + col] = v;
            else reinterpret_cast<__nv_bfloat16*>(a.out)[(size_t)tok * a.ldc + col] = o16;
            if (a.kv_width > 0 && col >= a.q_width) {
                // this column is a key or value element of token `tok`: also to its cache slot
                const int slot = a.slots[tok];
                if (slot >= 0) {
                    const int page = slot / a.page_size, off = slot - page * a.page_size;
                    if (page >= a.num_pages) {
                        prb_set_status(a.status, PRB_S_SLOT_RANGE, tok, slot, a.num_pages);
                    } else {
                        int cc = col - a.q_width;
                        void* pages = cc < a.kv_width ? a.k_pages : a.v_pages;
                        if (cc >= a.kv_width) cc -= a.kv_width;
                        const int h = cc / a.head_dim, d = cc - h * a.head_dim;
                        const int kv_heads = a.kv_width / a.head_dim;
                        const size_t at = (((size_t)page * kv_heads + h) * a.page_size + off) * a.head_dim + d;
                        if (f32_out) reinterpret_cast<float*>(pages)[at] = v;
                        else reinterpret_cast<__nv_bfloat16*>(pages)[at] = o16;
                    }
                }
            }
        }
        __syncthreads();                             // `red` is free for the next strip
        if (i == op_chunks - 1) GEMM_TRACE(7);
    }
}

// What a plan of attention units was made for (made once per step if nothing changes).
struct PlanKey {
    const int* token_list;
    const int* token_count;
    const int* positions;
    const int* seq_of_token;
    int n_list, n_heads, window, valid;
};

__global__ void __launch_bounds__(PROG_THREADS, 1)
decode_program_kernel(const Op* __restrict__ ops, int n_ops, unsigned* bar, int* status,
                      int x_area) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    __shared__ float red[WARPS * ROWS * MP];
    __shared__ ring::Shared ring_sh;
    __shared__ GemmBars gbars[2];
    __shared__ PlanKey plan_key;
    __shared__ Op sop[3];                           // the running operation and the two after it
    __shared__ float scratch[32];
    __shared__ int sh_flag;
    __shared__ int gemm_failed;

    // the activation area, then the arena; regions of even operations at its bottom, of odd
    // ones at its top
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
    __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(base_ptr);
    float* row = reinterpret_cast<float*>(base_ptr);
    const uint32_t arena0 = base + (uint32_t)x_area;
    const uint32_t arena1 = (smem_u32(smem_raw) + (uint32_t)SMEM_TOTAL) & ~1023u;
    auto region_of = [&](int i) {
        return (i & 1) ? ((arena1 - (uint32_t)sop[i % 3].region_bytes) & ~1023u) : arena0;
    };
    if (threadIdx.x == 0) {
        plan_key.valid = 0;
        gemm_failed = 0;
        gbars[0].valid = gbars[1].valid = 0;
    }
    if (threadIdx.x < ring::RING_WARPS) ring_sh.bars_valid[threadIdx.x] = 0;
    __syncthreads();

    auto prefetch = [&](int i) {
        if (i >= n_ops) return;
        // the record itself first, into shared memory: after a barrier nothing of it has to
        // come from the L2 again
        {
            const uint4* src = reinterpret_cast<const uint4*>(ops + i);
            uint4* dst = reinterpret_cast<uint4*>(&sop[i % 3]);
            for (int w = threadIdx.x; w < (int)(sizeof(Op) / 16); w += PROG_THREADS) dst[w] = src[w];
        }
        __syncthreads();
        const Op& op = sop[i % 3];
        if (op.type == OP_GEMM) {
            gemm_prefetch(op, &ops[i].map_a, region_of(i), gbars[i & 1]);
        } else if (op.type == OP_ATTN) {
            const ring::RingArgs& a = op.attn;
            const bool same = plan_key.valid && plan_key.token_list == a.token_list &&
                              plan_key.token_count == a.token_count && plan_key.positions == a.positions &&
                              plan_key.seq_of_token == a.seq_of_token && plan_key.n_list == a.n_list &&
                              plan_key.n_heads == a.n_heads && plan_key.window == a.window;
            __syncthreads();
            if (!same) {
                ring::plan(a, ring_sh);
                if (threadIdx.x == 0)
                    plan_key = PlanKey{a.token_list, a.token_count, a.positions, a.seq_of_token,
                                       a.n_list, a.n_heads, a.window, 1};
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            ring::early(a, &ops[i].map_a, &ops[i].map_b, ring_sh, region_of(i), (int)gridDim.x,
                        (int)blockIdx.x);
        }
    };
    auto drain = [&]() {
        // somebody gave up: wait (bounded) for this CTA's own copies in flight before leaving
        if (threadIdx.x == 0) {
            for (int side = 0; side < 2; ++side)
                for (int s = 0; s < gbars[side].valid; ++s)
                    for (uint32_t w = 0; w < (1u << 14); ++w)
                        if (ring::mbar_try_wait(smem_u32(&gbars[side].full[s]), 0) ||
                            ring::mbar_try_wait(smem_u32(&gbars[side].full[s]), 1)) break;
        }
        __syncthreads();
    };

    unsigned epoch = 0;
    prefetch(0);
    prefetch(1);
    for (int i = 0; i < n_ops; ++i) {
        const Op& op = sop[i % 3];
        const int type = op.type, units = op.units, flags = op.flags;
        PROG_TRACE(i, 0);
        switch (type) {
            case OP_EMBED:
                for (int vb = blockIdx.x; vb < units; vb += gridDim.x) {
                    if (flags & 2) elementwise::embed_token<float>(op.embed, vb);
                    else elementwise::embed_token<__nv_bfloat16>(op.embed, vb);
                }
                break;
            case OP_NORM:
                for (int vb = blockIdx.x; vb < units; vb += gridDim.x) {
                    if (flags & 2) elementwise::layernorm_row<float>(op.norm, vb, row, scratch);
                    else elementwise::layernorm_row<__nv_bfloat16>(op.norm, vb, row, scratch);
                    __syncthreads();
                }
                break;
            case OP_GEMM:
                gemm_run(op, &ops[i].map_a, region_of(i), gbars[i & 1], xs, red, &gemm_failed, i);
                break;
            case OP_ATTN:
                ring::late(op.attn, &ops[i].map_a, &ops[i].map_b, ring_sh, region_of(i), (int)gridDim.x,
                           (int)blockIdx.x);
                break;
            default:
                break;
        }
        if (gemm_failed) {
            if (threadIdx.x == 0) {
                prb_set_status(status, PRB_S_WAIT_TIMEOUT, 10, (int)blockIdx.x, i);
                atomicExch(&bar[1], 1u);
            }
            drain();
            return;
        }
        if (i + 1 >= n_ops) break;
        grid_arrive(bar);                            // this CTA's share of operation i is done
        PROG_TRACE(i, 1);
        prefetch(i + 2);                             // its region is free: the operation after the next
        PROG_TRACE(i, 2);
        epoch += 1;
        if (!grid_wait(bar, epoch * gridDim.x, &sh_flag, status, i)) {
            drain();
            return;
        }
        PROG_TRACE(i, 3);
    }
}

size_t max_size(size_t a, size_t b) { return a > b ? a : b; }
size_t round_up(size_t v, size_t to) { return (v + to - 1) / to * to; }

// Sizes of the regions so that consecutive operations fit the arena together; false if the
// program cannot run as one kernel.
bool lay_out(Program& p) {
    p.x_bytes = 0;
    for (Op& op : p.ops) p.x_bytes = max_size(p.x_bytes, (size_t)op.x_bytes);
    p.x_bytes = round_up(p.x_bytes, 1024);
    if (p.x_bytes + 2048 > SMEM_TOTAL) return false;
    const size_t arena = SMEM_TOTAL - 1024 - p.x_bytes - 1024;       // (alignment at both ends)
    auto gemm_region = [](const Op& op, int stages) {
        const size_t gb = (op.flags & 1) ? round_up((size_t)op.gemm.k * 8, 1024) : 0;
        return gb + (size_t)stages * (op.kc / 64) * ROWS * 128;
    };
    const int sms = prb_sm_count();
    for (Op& op : p.ops) {
        if (op.type != OP_GEMM) continue;
        const int items = ((op.units + sms - 1) / sms) * op.chunks;
        op.stages = items < GEMM_STAGES ? items : GEMM_STAGES;
        while (op.stages > 1 && gemm_region(op, op.stages) > 100 * 1024) --op.stages;
        op.region_bytes = (int)round_up(gemm_region(op, op.stages), 1024);
    }
    for (size_t i = 0; i + 1 < p.ops.size(); ++i) {
        Op& a = p.ops[i];
        Op& b = p.ops[i + 1];
        if (a.type == OP_ATTN && b.type == OP_ATTN) return false;    // they share their barriers
        while ((size_t)a.region_bytes + (size_t)b.region_bytes > arena) {
            Op* shrink = nullptr;                     // the product with more buffers gives one up
            if (a.type == OP_GEMM && a.stages > 1) shrink = &a;
            if (b.type == OP_GEMM && b.stages > 1 && (!shrink || b.stages > a.stages)) shrink = &b;
            if (!shrink) return false;
            --shrink->stages;
            shrink->region_bytes = (int)round_up(gemm_region(*shrink, shrink->stages), 1024);
        }
    }
    // (a region shrunk for its right-hand neighbour still fits beside its left-hand one)
    for (const Op& op : p.ops)
        if ((size_t)op.region_bytes > arena) return false;
    p.laid_out = true;
    return true;
}
}  // namespace

// ---------------------------------------------------------------- building a program
PRB_API int prb_program_max_rows() { return MAX_ROWS; }

PRB_API void* prb_program_new(int max_rows) {
    if (max_rows > MAX_ROWS) return nullptr;
    return new Program();
}
PRB_API void prb_program_free(void* handle) { delete static_cast<Program*>(handle); }
PRB_API int prb_program_length(void* handle) { return (int)static_cast<Program*>(handle)->ops.size(); }
PRB_API long prb_program_bytes(void* handle) {
    return (long)(static_cast<Program*>(handle)->ops.size() * sizeof(Op));
}

PRB_API int prb_program_add_embed(void* handle, float* out, const int* tokens, const int* positions,
                                  const void* wte, const void* wpe, int n_tokens, int width,
                                  int vocab, int n_positions, int table_dtype, int* status) {
    Program* p = static_cast<Program*>(handle);
    if (table_dtype != PRB_F32 && table_dtype != PRB_BF16) return PRB_E_DTYPE;
    Op op{};
    op.type = OP_EMBED;
    op.units = n_tokens;
    op.flags = table_dtype == PRB_F32 ? 2 : 0;
    op.embed = elementwise::EmbedArgs{out, tokens, positions, wte, wpe, n_tokens, width, vocab,
                                      n_positions, status};
    p->ops.push_back(op);
    return 0;
}

PRB_API int prb_program_add_norm(void* handle, void* out, const float* x, const float* gamma,
                                 const float* beta, const int* rows, int n_rows, int n_rows_in,
                                 int width, float eps, int out_dtype, int* status) {
    Program* p = static_cast<Program*>(handle);
    if (out_dtype != PRB_F32 && out_dtype != PRB_BF16) return PRB_E_DTYPE;
    if (width <= 0 || (size_t)width * 4 > 64 * 1024) return PRB_E_SIZE;
    Op op{};
    op.type = OP_NORM;
    op.units = n_rows;
    op.flags = out_dtype == PRB_F32 ? 2 : 0;
    op.x_bytes = width * (int)sizeof(float);
    op.norm = elementwise::NormArgs{out, x, gamma, beta, rows, n_rows, n_rows_in, width, eps, status};
    p->ops.push_back(op);
    return 0;
}

PRB_API int prb_program_add_gemm(void* handle, void* out, const void* x, const float* xf,
                                 const float* gamma, const float* beta, float eps, const void* w,
                                 const float* bias, const float* resid, int m, int n, int k,
                                 long ldx, long ldw, long ldc, int act, int out_dtype,
                                 void* k_pages, void* v_pages, const int* slots, int q_width,
                                 int kv_width, int head_dim, int page_size, int num_pages,
                                 int* status) {
    Program* p = static_cast<Program*>(handle);
    if (out_dtype != PRB_F32 && out_dtype != PRB_BF16) return PRB_E_DTYPE;
    if (m > MAX_ROWS || k % 64 != 0) return PRB_E_SIZE;
    const int bad = prb_gemm_smallm_check(x, xf, gamma, beta, w, m, n, k, ldx, ldw);
    if (bad) return bad;
    const bool ln = xf != nullptr;
    Op op{};
    op.type = OP_GEMM;
    op.units = (n + ROWS - 1) / ROWS;
    op.flags = (ln ? 1 : 0) | (out_dtype == PRB_F32 ? 2 : 0);
    op.kc = (size_t)k <= MAX_KC ? k : (int)CHUNK_KC;
    op.chunks = (k + op.kc - 1) / op.kc;
    op.x_bytes = MP * smallm::norm_pitch(k) * 2;
    smallm::Args a;
    a.out = out; a.x = (const __nv_bfloat16*)x; a.xf = xf; a.gamma = gamma; a.beta = beta;
    a.eps = eps; a.w = (const __nv_bfloat16*)w; a.bias = bias; a.resid = resid;
    a.m = m; a.n = n; a.k = k; a.ldx = ldx; a.ldw = ldw; a.ldc = ldc; a.act = act;
    a.xs_pitch = smallm::norm_pitch(k);
    if (kv_width > 0 && (head_dim <= 0 || kv_width % head_dim != 0 || page_size <= 0 ||
                         q_width + 2 * kv_width != n || !k_pages || !v_pages || !slots))
        return PRB_E_ARG;
    a.k_pages = k_pages; a.v_pages = v_pages; a.slots = slots;
    a.q_width = q_width; a.kv_width = kv_width; a.head_dim = head_dim;
    a.page_size = page_size; a.num_pages = num_pages; a.status = status;
    op.gemm = a;
    const int rc = tmap::slab_map(w, n, k, ldw, ROWS, op.kc / 64, &op.map_a);
    if (rc) return rc;
    p->ops.push_back(op);
    return 0;
}

PRB_API int prb_program_add_attention_ring(void* handle, void* out, long out_stride, const void* q,
                                           long q_stride, const void* k_pages, const void* v_pages,
                                           const int* block_table, const int* seq_of_token,
                                           const int* positions, const int* token_list,
                                           const int* token_count, int n_list, int n_heads,
                                           int kv_heads, int head_dim, int page_size, int max_pages,
                                           int num_pages, float scale, int window, int new_keys,
                                           const void* k_new, const void* v_new, long kv_stride,
                                           float* workspace, int* counters, int* status) {
    Program* p = static_cast<Program*>(handle);
    Op op{};
    op.type = OP_ATTN;
    const int rc = ring::check_and_maps(q, q_stride, out, out_stride, k_pages, v_pages, n_list, n_heads,
                                        kv_heads, head_dim, page_size, num_pages, new_keys, k_new,
                                        v_new, kv_stride, &op.map_a, &op.map_b);
    if (rc) return rc;
    ring::RingArgs a;
    a.out = (__nv_bfloat16*)out; a.out_stride = out_stride;
    a.q = (const __nv_bfloat16*)q; a.q_stride = q_stride;
    a.block_table = block_table; a.seq_of_token = seq_of_token; a.positions = positions;
    a.token_list = token_list; a.token_count = token_count;
    a.n_list = n_list; a.n_heads = n_heads; a.kv_heads = kv_heads; a.page_size = page_size;
    a.max_pages = max_pages; a.num_pages = num_pages; a.scale = scale; a.window = window;
    a.k_new = (const __nv_bfloat16*)k_new; a.v_new = (const __nv_bfloat16*)v_new; a.kv_stride = kv_stride;
    a.new_keys = new_keys; a.workspace = workspace; a.counters = counters; a.status = status;
    a.stages = 2;                                    // 8 warps x 2 buffers x 8 KB
    op.attn = a;
    op.region_bytes = (PROG_THREADS / 32) * a.stages * 2 * ring::TILE;
    p->ops.push_back(op);
    return 0;
}

// Lay the program out and copy it to `device_ops` (at least prb_program_bytes bytes).
// PRB_E_SIZE: the step does not fit one kernel.
PRB_API int prb_program_upload(void* handle, void* device_ops, cudaStream_t stream) {
    Program* p = static_cast<Program*>(handle);
    if (p->ops.empty()) return PRB_E_ARG;
    if (!lay_out(*p)) return PRB_E_SIZE;
    cudaError_t e = cudaMemcpyAsync(device_ops, p->ops.data(), p->ops.size() * sizeof(Op),
                                    cudaMemcpyHostToDevice, stream);
    if (e != cudaSuccess) return (int)e;
    e = cudaStreamSynchronize(stream);                 // the vector may be freed afterwards
    return e == cudaSuccess ? 0 : (int)e;
}

// Run an uploaded program: `barrier` is 2 x uint32 of scratch (zeroed here, on the stream).
PRB_API int prb_program_run(void* handle, const void* device_ops, unsigned* barrier, int* status,
                            cudaStream_t stream) {
    Program* p = static_cast<Program*>(handle);
    if (!p->laid_out) return PRB_E_ARG;
    const Op* ops = static_cast<const Op*>(device_ops);
    int n = (int)p->ops.size();
    static int grid = 0;
    if (grid == 0) {
        cudaError_t e = cudaFuncSetAttribute(decode_program_kernel,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)SMEM_TOTAL);
        if (e != cudaSuccess) return (int)e;
        int per_sm = 0;
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_program_kernel,
                                                          PROG_THREADS, SMEM_TOTAL);
        if (e != cudaSuccess) return (int)e;
        if (per_sm < 1) return PRB_E_SIZE;
        grid = prb_sm_count();                           // one CTA per SM, all co-resident
    }
    cudaError_t e = cudaMemsetAsync(barrier, 0, 2 * sizeof(unsigned), stream);
    if (e != cudaSuccess) return (int)e;
    int x_area = (int)p->x_bytes;
    void* args[] = {(void*)&ops, (void*)&n, (void*)&barrier, (void*)&status, (void*)&x_area};
    e = cudaLaunchCooperativeKernel((void*)decode_program_kernel, dim3(grid), dim3(PROG_THREADS),
                                    args, SMEM_TOTAL, stream);
    if (e != cudaSuccess) return (int)e;
    return 0;
}
