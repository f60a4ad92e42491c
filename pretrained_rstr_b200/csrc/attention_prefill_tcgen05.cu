// Causal attention for prompt portions over the paged bfloat16 cache on the 5th-generation
// tensor cores, flash style: scores live in tensor memory and registers, never in global
// memory.  Head size 64, pages of a multiple of 64 positions.
//
// One CTA takes up to 128 consecutive query tokens of one request for one head and walks
// the keys in blocks of 64 absolute positions (boundaries at multiples of 64, so a row's
// summation order depends on its own position only).  Warp roles:
//   warp 0     producer: TMA loads of the query tile (once) and of a block's keys and
//              values (two 64 x 64 boxes of the cache, found through the block table) into
//              a ring of shared-memory stages;
//   warp 1     allocates tensor memory; one thread issues tcgen05.mma:
//              S = Q K^T (128 x 64, K = 64) into one of two score buffers, and, once the
//              softmax warps have written P, O += P V (128 x 64, K = 64 keys, V as an
//              MN-major operand straight from its [key][dim] rows);
//   warps 2-9  softmax: two threads per query row, each with 32 of a block's 64 scores and
//              32 of the 64 output dims: read the scores from tensor memory, scale, mask
//              (causal, window, rows beyond the tile), keep the running maximum and sum in
//              float32, write P (bfloat16, only as an MMA operand) to shared memory in the
//              swizzled operand layout (two buffers take turns).  The output rows
//              accumulate in tensor memory over all blocks; a row's reference maximum moves
//              only in large steps, and only then are its output values rescaled there.
// The score MMA of block j+1 is issued before the softmax of block j is waited for, so the
// tensor cores and the softmax warps overlap.
//
// Key parts: a tile late in a long prompt walks many blocks one after the other while the
// CTAs of early tiles have long finished.  With part_blocks > 0 a (tile, head) is taken by
// as many CTAs (grid z) as its keys have chunks of part_blocks blocks (chunk borders at
// absolute positions; a CTA whose z has no chunk leaves at once).  A tile with one chunk is
// stored as before.  Otherwise every CTA writes its maximum, sum and output rows (float32)
// to a workspace and counts itself in; the one that finds itself last merges all parts in
// chunk order and stores the rows, so the result does not depend on who came last.  No TMA load uses cluster multicast.  Every
// mbarrier wait is bounded: on a timeout the kernel records PRB_S_WAIT_TIMEOUT, stores
// nothing more, waits (bounded) for its loads in flight, frees its tensor memory and
// returns.
#include "common.cuh"
#include "tcgen05.cuh"
#include "tensor_map.cuh"

#ifdef PRB_TRACE
__device__ unsigned long long g_pf_trace[64 * 16];
#define PF_TRACE(j, slot)                                                             \
    do {                                                                              \
        if (blockIdx.x == 0 && blockIdx.y == 0 && lane == 0 && (j) < 64) {            \
            unsigned long long t__;                                                   \
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t__));                   \
            g_pf_trace[(j) * 16 + (slot)] = t__;                                      \
        }                                                                             \
    } while (0)
// per CTA (linear block index): start, -, first scores seen, last block done, end, key blocks, SM
__device__ unsigned long long g_pf_cta[8192 * 8];
#define PF_CTA(slot, value)                                                           \
    do {                                                                              \
        const unsigned id__ = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x; \
        if (id__ < 8192) g_pf_cta[id__ * 8 + (slot)] = (value);                        \
    } while (0)
__device__ __forceinline__ unsigned long long pf_now() {
    unsigned long long t__;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t__));
    return t__;
}
PRB_API int prb_attention_prefill_tc_cta_trace(unsigned long long* host, int n) {
    return (int)cudaMemcpyFromSymbol(host, g_pf_cta, sizeof(unsigned long long) * n);
}
PRB_API int prb_attention_prefill_tc_trace(unsigned long long* host, int n) {
    return (int)cudaMemcpyFromSymbol(host, g_pf_trace, sizeof(unsigned long long) * n);
}
#else
#define PF_TRACE(j, slot)
#define PF_CTA(slot, value)
#endif

namespace {
using namespace tc5;

constexpr int QT = 128;             // queries per CTA
constexpr int KB = 64;              // keys per block
constexpr int DH = 64;              // head size
constexpr int STAGES = 3;           // ring of key/value blocks
constexpr int THREADS = 320;        // producer, MMA issuer, eight softmax warps
constexpr int Q_BYTES = QT * DH * 2, P_BYTES = QT * KB * 2;
constexpr int K_BYTES = KB * DH * 2, V_BYTES = KB * DH * 2;
constexpr int STAGE_BYTES = K_BYTES + V_BYTES;
constexpr int TMEM_COLS = 256;      // two score buffers and the output rows, 64 columns each
constexpr size_t SMEM_BYTES = 1024 + Q_BYTES + 2 * P_BYTES + STAGES * STAGE_BYTES + 256 + 4 * QT * 4;
constexpr float RESCALE_STEP = 8.0f;   // a row's reference maximum moves only by more than this (log2 units)

constexpr int MAX_PARTS = 16;       // most chunks of keys one (tile, head) may have

struct Params {
    float* part_o;                  // [(tile * heads + head) * max_parts + part][DH][QT]
    float* part_ml;                 // [...][QT][2]: maximum (log2 units) and sum of a row
    int* part_count;                // [tile * heads + head], zero before and after
    int part_blocks;                // blocks per chunk; 0: one CTA per (tile, head)
    // Work items (optional; else a CTA's tile and chunk are its grid indices x and z): item i
    // is tile item_tile[i] as a whole (item_part[i] < 0) or its chunk item_part[i], whose
    // partial result goes to slot item_slot[i] of the workspace (the chunks of a tile have
    // consecutive slots, chunk 0 first); the chunk size is read from the device.
    const int* item_tile;
    const int* item_part;
    const int* item_slot;
    const int* item_count;          // null: every CTA of the grid has an item
    const int* part_blocks_dev;
    __nv_bfloat16* out;
    long out_stride;
    const int* block_table;
    const int* positions;
    const int* tile_req;
    const int* tile_row0;
    const int* tile_rows;
    const int* tile_count;
    int n_heads, kv_heads, page_size, max_pages, num_pages;
    float scale;
    int window;
    int* status;
};

// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp writes lane (base + i).
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]),
        "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
        "r"(r[30]), "r"(r[31])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c,
                                             uint32_t d) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d)
                 : "memory");
}

// 2^x by the hardware approximation (relative error about 2^-22; 2^-inf = 0)
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__global__ void __launch_bounds__(THREADS, 2)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q,
                            const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, Params p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* q_s = smem;
    uint8_t* p_s = smem + Q_BYTES;
    uint8_t* ring = p_s + 2 * P_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(ring + STAGES * STAGE_BYTES);
    uint64_t* kv_full = bars;                  // [STAGES] TMA -> MMA
    uint64_t* kv_empty = bars + STAGES;        // [STAGES] MMA -> TMA
    uint64_t* s_full = bars + 2 * STAGES;      // [2] scores ready
    uint64_t* q_full = s_full + 2;
    uint64_t* p_full = q_full + 1;             // P written (one arrival per softmax warp)
    uint64_t* o_full = p_full + 1;             // O_blk ready
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_full + 1);
    volatile int* failed = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* is_last = reinterpret_cast<volatile int*>(tmem_slot + 2);
    float* xmax = reinterpret_cast<float*>(bars + 32);     // [2 blocks][2 halves][QT]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    prb_grid_launch_dependents();     // the next kernel may set itself up while this one runs

    const bool listed = p.item_tile != nullptr;
    int item, chunk_z = (int)blockIdx.z, part_blocks = p.part_blocks, slot_base = 0;
    bool whole = part_blocks <= 0;
    if (listed) {
        // the host's list: longest first, only items that have work.  The grid is (heads,
        // items): CTAs are placed in the order of their linear index, heads fastest, so the
        // longest items of all heads come first.
        const int n_listed = p.item_count != nullptr ? *p.item_count : (int)gridDim.y;
        const int li = (int)blockIdx.y;
        if (li >= n_listed) {
            prb_grid_wait();          // a kernel is complete only when those before it are
            return;
        }
        item = p.item_tile[li];
        chunk_z = p.item_part[li];
        whole = chunk_z < 0;
        part_blocks = whole ? 0 : *p.part_blocks_dev;
        slot_base = whole ? 0 : p.item_slot[li] - chunk_z;
        if (!whole && part_blocks <= 0) {
            if (threadIdx.x == 0) prb_set_status(p.status, PRB_S_POSITION_RANGE, item, chunk_z, part_blocks);
            prb_grid_wait();
            return;
        }
    } else {
        // the longest tiles (late query positions) first
        const int n_items = p.tile_count != nullptr ? *p.tile_count : (int)gridDim.x;
        if ((int)blockIdx.x >= n_items) {
            prb_grid_wait();
            return;
        }
        item = n_items - 1 - blockIdx.x;
    }
    const int h = listed ? (int)blockIdx.x : (int)blockIdx.y;
    const int b = p.tile_req[item];
    const int row0 = p.tile_row0[item];
    const int rows = p.tile_rows[item];
    const int pos0 = p.positions[row0];
    const int pos_last = pos0 + rows - 1;
    if (b < 0 || rows <= 0 || rows > QT || pos0 < 0 || pos_last >= p.max_pages * p.page_size) {
        if (threadIdx.x == 0) prb_set_status(p.status, PRB_S_POSITION_RANGE, row0, pos0, rows);
        prb_grid_wait();
        return;
    }
    const int hk = h / (p.n_heads / p.kv_heads);
    const int* table = p.block_table + (size_t)b * p.max_pages;
    const int lo_all = (p.window > 0 && pos0 - p.window + 1 > 0) ? pos0 - p.window + 1 : 0;
    int blk_first = lo_all / KB, blk_last = pos_last / KB;
    int n_parts = 1;
    if (!whole) {
        // chunk (first chunk + z) of the tile's keys
        const int chunk0 = blk_first / part_blocks;
        n_parts = blk_last / part_blocks - chunk0 + 1;
        if ((!listed && n_parts > (int)gridDim.z) || n_parts > MAX_PARTS) {
            if (threadIdx.x == 0 && chunk_z == 0)
                prb_set_status(p.status, PRB_S_POSITION_RANGE, row0, pos_last, n_parts);
            prb_grid_wait();
            return;
        }
        if (chunk_z >= n_parts) {
            prb_grid_wait();
            return;
        }
        const int lo = (chunk0 + chunk_z) * part_blocks;
        if (lo > blk_first) blk_first = lo;
        if (lo + part_blocks - 1 < blk_last) blk_last = lo + part_blocks - 1;
    }
    const int n_blocks = blk_last - blk_first + 1;
#ifdef PRB_TRACE
    if (threadIdx.x == 0) {
        unsigned smid;
        asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
        PF_CTA(0, pf_now()); PF_CTA(5, (unsigned long long)n_blocks); PF_CTA(6, (unsigned long long)smid);
    }
#endif

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&kv_full[s]), 1);
            mbar_init(smem_u32(&kv_empty[s]), 1);
        }
        mbar_init(smem_u32(&s_full[0]), 1);
        mbar_init(smem_u32(&s_full[1]), 1);
        mbar_init(smem_u32(q_full), 1);
        mbar_init(smem_u32(p_full), 8);
        mbar_init(smem_u32(o_full), 1);
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(tmem_slot)),
                     "r"((uint32_t)TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // set up; the queries, keys and values below were written by the kernels before
    prb_grid_wait();

    if (warp == 0) {
        // ------------------------------------------------------------ producer
        // (The whole warp walks the loop and waits; one elected lane issues: inside
        // "if (lane == 0)" the warp would be divergent for its whole life and the copy and MMA
        // instructions, whose operands live in uniform registers, issue several times slower.)
        const uint32_t qb = smem_u32(q_full);
        if (elect_one()) {
            mbar_expect_tx(qb, Q_BYTES);
            tma_load_2d(smem_u32(q_s), &map_q, qb, h * DH, row0);
        }
        __syncwarp();
        bool ok = true;
        int j = 0;
        for (; j < n_blocks && ok; ++j) {
            const int st = j % STAGES;
            ok = mbar_wait_warp(smem_u32(&kv_empty[st]), ((j / STAGES) & 1) ^ 1, failed);
            if (!ok) {
                if (lane == 0) prb_set_status(p.status, PRB_S_WAIT_TIMEOUT, 11, blockIdx.x, j);
                break;
            }
            const int key0 = (blk_first + j) * KB;
            const int page = table[key0 / p.page_size];
            const uint32_t fb = smem_u32(&kv_full[st]);
            if (page < 0 || page >= p.num_pages) {
                // recorded; the block's buffer keeps what it held and the result of the
                // tile is not to be used
                if (lane == 0) {
                    prb_set_status(p.status, PRB_S_PAGE_RANGE, row0, key0, page);
                    mbar_arrive(fb);
                }
                __syncwarp();
                continue;
            }
            const int crow = (page * p.kv_heads + hk) * p.page_size + key0 % p.page_size;
            const uint32_t stage = smem_u32(ring + (size_t)st * STAGE_BYTES);
            if (elect_one()) {
                mbar_expect_tx(fb, STAGE_BYTES);
                tma_load_2d(stage, &map_k, fb, 0, crow);
                tma_load_2d(stage + K_BYTES, &map_v, fb, 0, crow);
            }
            __syncwarp();
        }
        if (!ok && lane == 0) {
            // wait (bounded) for loads still in flight before the CTA may exit
            for (uint32_t i = 0; i < WAIT_LIMIT; ++i)
                if (mbar_try_wait(smem_u32(q_full), 0)) break;
            const int first = j > STAGES ? j - STAGES : 0;
            for (int jj = first; jj < j; ++jj) {
                const uint32_t fb = smem_u32(&kv_full[jj % STAGES]);
                for (uint32_t i = 0; i < WAIT_LIMIT; ++i)
                    if (mbar_try_wait(fb, (jj / STAGES) & 1)) break;
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------------------------------------------------- MMA issuer
        constexpr uint32_t idesc_s = make_idesc(QT, KB);          // Q, K: both K-major
        constexpr uint32_t idesc_o = make_idesc_b_mn(QT, DH);     // P K-major, V MN-major
        const uint64_t q_desc = make_smem_desc(smem_u32(q_s));
        auto issue_scores = [&](int j) {
            const uint8_t* stage = ring + (size_t)(j % STAGES) * STAGE_BYTES;
            const uint64_t k_desc = make_smem_desc(smem_u32(stage));
            const uint32_t d = tmem_base + (uint32_t)((j & 1) * KB);
            if (elect_one()) {
#pragma unroll
                for (int kk = 0; kk < DH / 16; ++kk)
                    umma_bf16(d, q_desc + (uint64_t)(kk * 2), k_desc + (uint64_t)(kk * 2), idesc_s,
                              kk > 0 ? 1u : 0u);
                umma_commit(smem_u32(&s_full[j & 1]));
            }
            __syncwarp();
        };
        bool ok = mbar_wait_warp(smem_u32(q_full), 0, failed);
        if (ok) ok = mbar_wait_warp(smem_u32(&kv_full[0]), 0, failed);
        if (ok) {
            tcgen05_fence_after();
            issue_scores(0);
        }
        for (int j = 0; j < n_blocks && ok; ++j) {
            if (j + 1 < n_blocks) {
                ok = mbar_wait_warp(smem_u32(&kv_full[(j + 1) % STAGES]), ((j + 1) / STAGES) & 1, failed);
                if (!ok) break;
                tcgen05_fence_after();
                issue_scores(j + 1);
            }
            PF_TRACE(j, 8);
            ok = mbar_wait_warp(smem_u32(p_full), j & 1, failed);
            if (!ok) break;
            PF_TRACE(j, 9);
            tcgen05_fence_after();
            const uint8_t* stage = ring + (size_t)(j % STAGES) * STAGE_BYTES;
            const uint32_t v_addr = smem_u32(stage + K_BYTES);
            const uint64_t pj_desc = make_smem_desc(smem_u32(p_s + (size_t)(j & 1) * P_BYTES));
            const uint32_t d = tmem_base + 2 * KB;
            if (elect_one()) {
#pragma unroll
                for (int kk = 0; kk < KB / 16; ++kk) {
                    // 16 keys further: two 8-row groups of 1024 bytes; O accumulates over blocks
                    umma_bf16(d, pj_desc + (uint64_t)(kk * 2), make_smem_desc(v_addr + kk * 2048),
                              idesc_o, (j > 0 || kk > 0) ? 1u : 0u);
                }
                umma_commit(smem_u32(o_full));
                umma_commit(smem_u32(&kv_empty[j % STAGES]));     // frees the stage
            }
            __syncwarp();
            PF_TRACE(j, 10);
        }
        if (!ok && lane == 0) prb_set_status(p.status, PRB_S_WAIT_TIMEOUT, 12, blockIdx.x, 0);
    } else {
        // ------------------------------------------------------------- softmax
        // Two threads per query row: warps 2-5 take key columns 0-31 of a block and output
        // dims 0-31, warps 6-9 the other halves; the two meet only for the row maximum of a
        // block (through shared memory and a barrier of their 64 threads) and, at the end,
        // for the row sum.
        const int quarter = warp & 3;                   // TMEM lanes this warp may read
        const int half = (warp - 2) >> 2;               // which 32 columns / dims
        const int r = quarter * 32 + lane;              // query row of this thread
        const int qpos = pos0 + r;
        const bool row_ok = r < rows;
        const float sl2 = p.scale * 1.4426950408889634f;   // scores are handled in log2 units
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
        const uint32_t p_row = smem_u32(p_s) + (uint32_t)r * 128;
        constexpr int HC = KB / 2, HD = DH / 2;
        float m_run = -INFINITY, l_run = 0.0f;
        bool ok = true;
        for (int j = 0; j < n_blocks; ++j) {
            // After a wait gave up the warp still walks every block, without waiting or
            // touching tensor memory, so that the barriers of its thread pairs stay matched.
            if (warp == 2) PF_TRACE(j, 0);
            if (ok) {
                ok = mbar_wait(smem_u32(&s_full[j & 1]), (j >> 1) & 1, failed);
                ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            }
            if (warp == 2) PF_TRACE(j, 1);
#ifdef PRB_TRACE
            if (warp == 2 && lane == 0 && j == 0) PF_CTA(2, pf_now());
#endif
            uint32_t sr[HC];
            if (ok) {
                tcgen05_fence_after();
                tmem_ld_32x32(lane_addr + (uint32_t)((j & 1) * KB + half * HC), sr);
                if (warp == 2 && sr[0] != 0x12345u) PF_TRACE(j, 2);
            } else {
#pragma unroll
                for (int c = 0; c < HC; ++c) sr[c] = 0u;
            }
            const int key0 = (blk_first + j) * KB + half * HC;
            const bool need_mask = !row_ok || p.window > 0 || key0 + HC - 1 > qpos;
            if (need_mask) {
#pragma unroll
                for (int c = 0; c < HC; ++c) {
                    const int jk = key0 + c;
                    const bool vis = row_ok && jk <= qpos && (p.window <= 0 || jk > qpos - p.window);
                    if (!vis) sr[c] = 0xff800000u;            // -inf
                }
            }
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int c = 0; c < HC; c += 4) {
#pragma unroll
                for (int e = 0; e < 4; ++e) mx4[e] = fmaxf(mx4[e], __uint_as_float(sr[c + e]));
            }
            const float mx_own = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            // the row maximum of the block: both halves
            xmax[((j & 1) * 2 + half) * QT + r] = mx_own;
            asm volatile("bar.sync %0, 64;" ::"r"(quarter + 1) : "memory");
            const float mx = fmaxf(mx_own, xmax[((j & 1) * 2 + (half ^ 1)) * QT + r]) * sl2;
            if (warp == 2 && mx != 1.2345f) PF_TRACE(j, 3);
            // The reference maximum of a row moves only when the block's maximum exceeds it by
            // more than RESCALE_STEP (softmax does not depend on the reference; exponents stay
            // below 2^RESCALE_STEP), so the output row in tensor memory is rarely rescaled.
            float m_new = m_run;
            if (m_run == -INFINITY || mx > m_run + RESCALE_STEP) m_new = mx;
            const bool rescale = m_run != -INFINITY && m_new != m_run;
            const float corr = rescale ? fast_exp2(m_run - m_new) : 1.0f;
            m_run = m_new;
            const float neg_m = (m_new == -INFINITY) ? 0.0f : -m_new;   // all masked: exp2(-inf) = 0
            uint32_t pk[HC / 2];
            float rs0 = 0.0f, rs1 = 0.0f;
#pragma unroll
            for (int c = 0; c < HC; c += 2) {
                const float p0 = fast_exp2(fmaf(__uint_as_float(sr[c]), sl2, neg_m));
                const float p1 = fast_exp2(fmaf(__uint_as_float(sr[c + 1]), sl2, neg_m));
                rs0 += p0;
                rs1 += p1;
                pk[c >> 1] = pack2(p0, p1);
            }
            l_run = l_run * corr + (rs0 + rs1);
            if (warp == 2 && l_run != 1.2345f) PF_TRACE(j, 4);
            // the product of the block before has retired: its P buffer's twin is free and the
            // output rows may be touched
            if (ok && j >= 1) {
                ok = mbar_wait(smem_u32(o_full), (j - 1) & 1, failed);
                ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                if (ok) tcgen05_fence_after();
            }
            if (warp == 2) PF_TRACE(j, 5);
            if (ok && __any_sync(0xffffffffu, rescale)) {
                uint32_t ob[HD];
                tmem_ld_32x32(lane_addr + (uint32_t)(2 * KB + half * HD), ob);
#pragma unroll
                for (int i = 0; i < HD; ++i) ob[i] = __float_as_uint(__uint_as_float(ob[i]) * corr);
                tmem_st_32x32(lane_addr + (uint32_t)(2 * KB + half * HD), ob);
            }
            // Keys after the tile's last query position (the rest of the request's last page)
            // hold whatever the page's earlier owner left there.  Their weights are zero, but
            // zero times a NaN or an infinity is a NaN: their value rows are cleared before
            // the product reads them (whole 128-byte rows, so the swizzle does not matter).
            const int first_stale = pos_last + 1 - (blk_first + j) * KB;    // key row within the block
            if (ok && first_stale < KB) {
                const uint32_t v_tile = smem_u32(ring + (size_t)(j % STAGES) * STAGE_BYTES + K_BYTES);
                const int t = (warp - 2) * 32 + lane;
                for (int piece = (first_stale < 0 ? 0 : first_stale) * 8 + t; piece < KB * 8; piece += 256)
                    st_shared_v4(v_tile + (uint32_t)piece * 16, 0u, 0u, 0u, 0u);
            }
            // 16-byte pieces of row r, swizzled with the row as TMA would have placed them
            const uint32_t p_dst = p_row + (uint32_t)((j & 1) * P_BYTES);
#pragma unroll
            for (int c = 0; c < HC / 8; ++c)
                st_shared_v4(p_dst + (uint32_t)(((half * 4 + c) ^ (r & 7)) << 4), pk[4 * c], pk[4 * c + 1],
                             pk[4 * c + 2], pk[4 * c + 3]);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(p_full));
            if (warp == 2) PF_TRACE(j, 6);
        }
#ifdef PRB_TRACE
        if (warp == 2 && lane == 0) PF_CTA(3, pf_now());
#endif
        // the row sum: both halves (every thread of the pair reaches this barrier)
        xmax[half * QT + r] = l_run;
        asm volatile("bar.sync %0, 64;" ::"r"(quarter + 1) : "memory");
        const float l_all = half == 0 ? l_run + xmax[QT + r] : xmax[r] + l_run;
        if (ok) {
            ok = mbar_wait(smem_u32(o_full), (n_blocks - 1) & 1, failed);
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        }
        __nv_bfloat16* dst = p.out + (size_t)(row0 + r) * p.out_stride + (size_t)h * DH + half * HD;
        auto store_row = [&](const float (&o)[HD], float inv) {
#pragma unroll
            for (int c = 0; c < HD; c += 8) {
                uint4 v;
                v.x = pack2(o[c] * inv, o[c + 1] * inv);
                v.y = pack2(o[c + 2] * inv, o[c + 3] * inv);
                v.z = pack2(o[c + 4] * inv, o[c + 5] * inv);
                v.w = pack2(o[c + 6] * inv, o[c + 7] * inv);
                *reinterpret_cast<uint4*>(dst + c) = v;
            }
        };
        float o_own[HD];
        if (ok) {
            tcgen05_fence_after();
            uint32_t ob[HD];
            tmem_ld_32x32(lane_addr + (uint32_t)(2 * KB + half * HD), ob);
            tcgen05_fence_before();
#pragma unroll
            for (int i = 0; i < HD; ++i) o_own[i] = __uint_as_float(ob[i]);
        } else {
#pragma unroll
            for (int i = 0; i < HD; ++i) o_own[i] = 0.0f;
        }
        if (n_parts == 1) {
            if (ok && row_ok) store_row(o_own, l_all > 0.0f ? 1.0f / l_all : 0.0f);
        } else {
            // this CTA's part: rows as [dim][row], so that a warp's 32 rows are one line
            // listed items: the tile's chunks lie in consecutive slots from slot_base on;
            // else (tile, head) units of gridDim.z slots each
            const size_t unit = listed ? (size_t)slot_base * p.n_heads + h : (size_t)item * p.n_heads + h;
            const size_t stride = listed ? (size_t)p.n_heads : 1;
            const size_t slot = listed ? (size_t)(slot_base + chunk_z) * p.n_heads + h
                                       : unit * gridDim.z + chunk_z;
            float* po = p.part_o + slot * (size_t)(DH * QT) + (size_t)(half * HD) * QT + r;
#pragma unroll
            for (int i = 0; i < HD; ++i) __stcg(po + (size_t)i * QT, o_own[i]);
            if (half == 0)
                __stcg(reinterpret_cast<float2*>(p.part_ml + slot * (size_t)(2 * QT)) + r,
                       make_float2(ok ? m_run : -INFINITY, ok ? l_all : 0.0f));
            __threadfence();
            asm volatile("bar.sync 5, 256;" ::: "memory");
            if (warp == 2 && lane == 0) {
                const int before = atomicAdd(p.part_count + unit, 1);
                const int last = before == n_parts - 1 ? 1 : 0;
                if (last) p.part_count[unit] = 0;              // left zero for the next launch
                *is_last = last;
            }
            asm volatile("bar.sync 5, 256;" ::: "memory");
            if (*is_last) {
                __threadfence();
                const size_t slot0 = listed ? unit : unit * gridDim.z;
                float ms[MAX_PARTS], m_all = -INFINITY;
                for (int s = 0; s < n_parts; ++s) {
                    ms[s] = __ldcg(p.part_ml + (slot0 + s * stride) * (size_t)(2 * QT) + 2 * r);
                    m_all = fmaxf(m_all, ms[s]);
                }
                float acc[HD], l_sum = 0.0f;
#pragma unroll
                for (int i = 0; i < HD; ++i) acc[i] = 0.0f;
                for (int s = 0; s < n_parts; ++s) {          // in chunk order
                    const float wgt = ms[s] == -INFINITY ? 0.0f : fast_exp2(ms[s] - m_all);
                    l_sum = fmaf(wgt, __ldcg(p.part_ml + (slot0 + s * stride) * (size_t)(2 * QT) + 2 * r + 1), l_sum);
                    const float* src = p.part_o + (slot0 + s * stride) * (size_t)(DH * QT) + (size_t)(half * HD) * QT + r;
#pragma unroll
                    for (int i = 0; i < HD; ++i) acc[i] = fmaf(wgt, __ldcg(src + (size_t)i * QT), acc[i]);
                }
                if (row_ok) store_row(acc, l_sum > 0.0f ? 1.0f / l_sum : 0.0f);
            }
        }
        if (!ok && lane == 0) prb_set_status(p.status, PRB_S_WAIT_TIMEOUT, 13, blockIdx.x, warp);
#ifdef PRB_TRACE
        if (warp == 2 && lane == 0) PF_CTA(4, pf_now());
#endif
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                     "r"((uint32_t)TMEM_COLS)
                     : "memory");
    }
}
}  // namespace

// Queries per tile of the work list this kernel takes.
PRB_API int prb_attention_prefill_tc_tile() { return QT; }

// 1 when the tensor-memory kernel takes this head size and page size, else 0.
PRB_API int prb_attention_prefill_tc_supports(int head_dim, int page_size) {
    return head_dim == DH && page_size > 0 && page_size % KB == 0 ? 1 : 0;
}

// Work list as prb_attention_prefill, with tiles of up to 128 rows.  part_blocks > 0: the
// keys of a tile in chunks of part_blocks * 64 positions, a CTA each, at most max_parts (up
// to 16) per tile; part_o: float32 [n_tiles * n_heads * max_parts * 64 * 128], part_ml:
// float32 [n_tiles * n_heads * max_parts * 256], part_count: int32 [n_tiles * n_heads], zero.  q: bfloat16 rows of
// q_stride elements, q_rows of them (head h at columns [h*64, h*64+64)); out likewise.
PRB_API int prb_attention_prefill_tc(void* out, long out_stride, const void* q, long q_stride,
                                     int q_rows, const void* k_pages, const void* v_pages,
                                     const int* block_table, const int* positions,
                                     const int* tile_req, const int* tile_row0,
                                     const int* tile_rows, const int* tile_count, int n_tiles,
                                     int n_heads, int kv_heads, int head_dim, int page_size,
                                     int max_pages, int num_pages, float scale, int window,
                                     int part_blocks, int max_parts, float* part_o,
                                     float* part_ml, int* part_count, const int* item_tile,
                                     const int* item_part, const int* item_slot,
                                     const int* item_count, const int* part_blocks_dev,
                                     int n_items, int* status, cudaStream_t stream) {
    if (n_tiles <= 0) return 0;
    const bool listed = item_tile != nullptr;
    if (listed && (n_items <= 0 || item_part == nullptr || item_slot == nullptr ||
                   part_blocks_dev == nullptr || part_o == nullptr || part_ml == nullptr ||
                   part_count == nullptr))
        return PRB_E_ARG;
    if (part_blocks < 0 || (part_blocks > 0 && (max_parts < 1 || max_parts > MAX_PARTS ||
                                                part_o == nullptr || part_ml == nullptr ||
                                                part_count == nullptr)))
        return PRB_E_ARG;
    if (!prb_attention_prefill_tc_supports(head_dim, page_size) || n_heads <= 0 || kv_heads <= 0 ||
        n_heads % kv_heads != 0 || n_heads > 65535 || q_rows <= 0)
        return PRB_E_SIZE;
    if (q_stride % 8 != 0 || out_stride % 8 != 0 || ((uintptr_t)q) % 16 != 0 ||
        ((uintptr_t)out) % 16 != 0 || ((uintptr_t)k_pages) % 16 != 0 ||
        ((uintptr_t)v_pages) % 16 != 0)
        return PRB_E_ALIGN;
    CUtensorMap map_q, map_k, map_v;
    int rc = tmap::get_map(q, q_rows, (long)n_heads * DH, q_stride, QT, &map_q);
    if (rc) return rc;
    const long cache_rows = (long)num_pages * kv_heads * page_size;
    if ((rc = tmap::get_map(k_pages, cache_rows, DH, DH, KB, &map_k)) != 0) return rc;
    if ((rc = tmap::get_map(v_pages, cache_rows, DH, DH, KB, &map_v)) != 0) return rc;
    static bool configured = false;
    if (!configured) {
        cudaFuncSetAttribute(attention_prefill_tc_kernel,
                             cudaFuncAttributePreferredSharedMemoryCarveout,
                             cudaSharedmemCarveoutMaxShared);
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_tc_kernel,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    Params p;
    p.part_o = part_o; p.part_ml = part_ml; p.part_count = part_count; p.part_blocks = part_blocks;
    p.item_tile = item_tile; p.item_part = item_part; p.item_slot = item_slot;
    p.item_count = item_count; p.part_blocks_dev = part_blocks_dev;
    p.out = (__nv_bfloat16*)out; p.out_stride = out_stride;
    p.block_table = block_table; p.positions = positions;
    p.tile_req = tile_req; p.tile_row0 = tile_row0; p.tile_rows = tile_rows;
    p.tile_count = tile_count;
    p.n_heads = n_heads; p.kv_heads = kv_heads; p.page_size = page_size;
    p.max_pages = max_pages; p.num_pages = num_pages; p.scale = scale; p.window = window;
    p.status = status;
    if (listed && n_items > 65535) return PRB_E_SIZE;
    dim3 grid(listed ? n_heads : n_tiles, listed ? n_items : n_heads,
              (!listed && part_blocks > 0) ? max_parts : 1);
    cudaError_t le = prb_launch_maybe_early(prb_small_ctas_early(), attention_prefill_tc_kernel, grid,
                                            dim3(THREADS), SMEM_BYTES, stream, map_q, map_k, map_v, p);
    if (le != cudaSuccess) return (int)le;
    return 0;
}
