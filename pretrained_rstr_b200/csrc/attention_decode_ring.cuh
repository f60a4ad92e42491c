// Decode attention by persistent CTAs whose warps stream keys and values through private
// rings of shared-memory buffers (TMA tile copies, 128-byte swizzle, no multicast) and
// multiply them with mma.sync: the device functions of the kernel in
// attention_decode_ring.cu, where the method is described.
//
// Three phases, each called by every thread of the CTA:
//   plan()   the step's description -> units per token and their running sum, in shared memory
//            (depends only on what was on the device before the step began);
//   early()  every warp works out its run of units and requests as many of them as it has ring
//            buffers, except units that hold rows the step itself writes when those rows are
//            not handed over beside the queries (also independent of the step's kernels);
//   late()   after the dependency has resolved: queries, the step's own rows, scores, values,
//            the merge inside the CTA and across CTAs.
#pragma once
#include "common.cuh"
#include "tensor_map.cuh"

#ifndef RING_TRACE
#define RING_TRACE(slot)
#endif

namespace ring {
constexpr int RING_WARPS = 8;                 // most warps of a CTA (a launch may use fewer)
constexpr int RING_THREADS = RING_WARPS * 32;
constexpr int UNIT = 32;                      // keys per unit
constexpr int DH = 64;                        // head size: one 128-byte swizzled box per row
constexpr int ROW = DH * 2;                   // bytes of a row
constexpr int TILE = UNIT * ROW;              // bytes of a unit's keys (and of its values)
constexpr int MAX_LIST = 256;                 // most single tokens of a launch
constexpr int MAX_STAGES = 4;
constexpr int PART = DH + 4;                  // floats of a partial state: values, maximum, sum
constexpr uint32_t RING_WAIT_LIMIT = 1u << 22;

struct RingArgs {
    __nv_bfloat16* out;
    long out_stride;
    const __nv_bfloat16* q;
    long q_stride;
    const int* block_table;
    const int* seq_of_token;
    const int* positions;
    const int* token_list;
    const int* token_count;
    int n_list, n_heads, kv_heads, page_size, max_pages, num_pages;
    float scale;
    int window;
    int new_keys;                   // a token's last `new_keys` visible positions may have been
                                    // written by the step itself
    // The step's own keys and values as the product before this kernel left them beside the
    // queries (row t of k_new / v_new: token t's keys / values, kv_heads * 64 wide), or null.
    // With them no unit has to wait for the cache rows the step appended: the whole unit is
    // requested early and those rows are put in from here once the dependency has resolved.
    const __nv_bfloat16* k_new;
    const __nv_bfloat16* v_new;
    long kv_stride;
    float* workspace;               // [(CTAs + n_list * n_heads)][PART] float32
    int* counters;                  // [n_list * n_heads] int32, zero; left zero
    int stages;                     // ring buffers per warp
    int* status;
};

// What the phases share, in the CTA's shared memory.
struct Shared {
    int cum[MAX_LIST + 1];          // units before each place of the token list
    int span_t[MAX_LIST], span_b[MAX_LIST], span_pos[MAX_LIST];   // token, request, position
    int n;                          // places of the token list in use
    int warp_tot[RING_WARPS];
    unsigned long long bars[RING_WARPS * MAX_STAGES];
    unsigned bad_mask[RING_WARPS];  // units (of a warp's first 32) with a page outside the pool
    int bars_valid[RING_WARPS];     // barriers of each warp that hold a valid object (0 at first:
                                    // whoever owns this struct clears it once, before early())
    // what a warp leaves for the merge: the state of the first and of the last (token, head)
    // of its run (the ones other warps may share), and which they are
    float edge_state[RING_WARPS][2][PART];
    int edge_pair[RING_WARPS][2];   // idx * heads + h, or -1
};

// The kernel's stages are inlined into their caller: called out of line (tried: a third less
// code) every launch was 6 us slower, which is what the calls' register traffic costs a kernel
// whose whole life is a dozen microseconds.
#define RING_FN __device__ __forceinline__

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
// An mbarrier object must be invalidated before its memory takes a new one.
__device__ __forceinline__ void mbar_inval(uint32_t bar) {
    asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
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
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < RING_WAIT_LIMIT; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
// Rows `row` .. of the cache seen as a matrix of 64 columns; x is always 0, so the 16-byte
// rule on the innermost coordinate holds.
__device__ __forceinline__ void tma_rows(uint32_t dst, const CUtensorMap* map, uint32_t bar, int row) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4}], [%2];" ::"r"(dst), "l"(map), "r"(bar), "r"(0), "r"(row)
        : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
// D += A . B where only row 0 of A is a query (its rows 8..15 are zero: a1 = a3 = 0)
__device__ __forceinline__ void mma_row(float (&d)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float x, float y) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(x, y);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// Where a token's keys are: request, position, first and number of 32-key blocks.
struct TokenSpan {
    int t, b, pos, lo, first_blk, n_blk;
};
__device__ __forceinline__ void span_blocks(const RingArgs& a, TokenSpan& s) {
    s.lo = (a.window > 0 && s.pos - a.window + 1 > 0) ? s.pos - a.window + 1 : 0;
    s.first_blk = s.lo / UNIT;
    s.n_blk = s.pos / UNIT - s.first_blk + 1;
}
__device__ __forceinline__ TokenSpan token_span(const RingArgs& a, int idx, int n) {
    TokenSpan s{-1, -1, 0, 0, 0, 0};
    if (idx >= n) return s;
    s.t = a.token_list ? a.token_list[idx] : idx;
    s.b = a.seq_of_token[s.t];
    if (s.b < 0) return s;
    s.pos = a.positions[s.t];
    if (s.pos < 0 || s.pos >= a.max_pages * a.page_size) {
        prb_set_status(a.status, PRB_S_POSITION_RANGE, s.t, s.pos, 0);
        s.b = -1;
        return s;
    }
    span_blocks(a, s);
    return s;
}

// A partial state as the merges see it: lane l holds output dimensions 2 l, 2 l + 1.
struct Partial {
    float m, l, o0, o1;
};
__device__ __forceinline__ void merge_into(Partial& acc, float m2, float l2, float a0, float a1) {
    const float mn = fmaxf(acc.m, m2);
    const float c1 = (acc.m == -INFINITY) ? 0.0f : __expf(acc.m - mn);
    const float c2 = (m2 == -INFINITY) ? 0.0f : __expf(m2 - mn);
    acc.l = acc.l * c1 + l2 * c2;
    acc.o0 = acc.o0 * c1 + a0 * c2;
    acc.o1 = acc.o1 * c1 + a1 * c2;
    acc.m = mn;
}

// ---- plan: units per token and their running sum.  Ends with a barrier of the CTA.
RING_FN void plan(const RingArgs& a, Shared& sh) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_warps = (int)blockDim.x >> 5;
    int n = a.n_list;
    if (a.token_count != nullptr) n = min(n, *a.token_count);
    int run = 0;
    for (int base = 0; base < n; base += (int)blockDim.x) {
        const TokenSpan s = token_span(a, base + (int)threadIdx.x, n);
        if (base + (int)threadIdx.x < n) {
            sh.span_t[base + threadIdx.x] = s.t;
            sh.span_b[base + threadIdx.x] = s.b;
            sh.span_pos[base + threadIdx.x] = s.pos;
        }
        const int mine = s.b >= 0 ? s.n_blk * a.n_heads : 0;
        int incl = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += v;
        }
        if (lane == 31) sh.warp_tot[warp] = incl;
        __syncthreads();
        int before = 0, total = 0;
        for (int w = 0; w < n_warps; ++w) {
            const int c = sh.warp_tot[w];
            if (w < warp) before += c;
            total += c;
        }
        if (base + (int)threadIdx.x < n) sh.cum[base + threadIdx.x] = run + before + incl - mine;
        run += total;
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        sh.cum[n] = run;
        sh.n = n;
    }
    __syncthreads();
}

// A warp's share of the launch.  Runs of `per` units each: CTA c's warp w is worker
// c * wpc + w and takes units [worker * per, worker * per + per), so that the warps that share
// a (token, head) are mostly warps of one CTA.  With few units the runs are a unit long and
// only `wpc` warps of every CTA have one, so that the work is spread over all SMs.
struct Run {
    long per, wpc, gw;
    int u_begin, u_end;
};
RING_FN Run my_run(const Shared& sh, int n_ctas, int cta) {
    const int warp = threadIdx.x >> 5, n_warps = (int)blockDim.x >> 5;
    Run r;
    const long total_units = sh.cum[sh.n];
    const long workers = (long)n_ctas * n_warps;
    r.per = total_units > 0 ? (total_units + workers - 1) / workers : 1;
    const long busy = (total_units + r.per - 1) / r.per;         // workers that have a run
    r.wpc = min((long)n_warps, max(1L, (busy + n_ctas - 1) / (long)n_ctas));
    r.gw = (long)cta * r.wpc + warp;
    const bool has_run = warp < r.wpc && r.gw < busy;
    r.u_begin = has_run ? (int)(r.gw * r.per) : 0;
    r.u_end = has_run ? (int)min(total_units, r.gw * r.per + r.per) : 0;
    return r;
}

// A lane's own unit of a batch of 32 units.
struct LaneUnit {
    int idx, h, blk;            // place in the token list, head, absolute 32-key block
    int pos, lo, t;
    bool late;                  // holds rows the step itself may have written (and they are not
                                // handed over beside the queries)
    bool bad;                   // a page of it lies outside the pool
    int pages[4];               // its pages (one when the page holds 32 keys or more)
    int rows;                   // rows to copy: up to the end of the last page it touches
};
// Which unit it is: from shared memory only.
RING_FN LaneUnit decode_unit(const RingArgs& a, const Shared& sh, int u, int u_end) {
    LaneUnit lu;
    lu.idx = -1;
    lu.h = lu.blk = lu.pos = lu.lo = lu.t = 0;
    lu.late = lu.bad = false;
    lu.rows = 0;
    lu.pages[0] = lu.pages[1] = lu.pages[2] = lu.pages[3] = -1;
    if (u >= u_end) return lu;
    int lo_i = 0, hi_i = sh.n;                       // largest idx with cum[idx] <= u
    while (hi_i - lo_i > 1) {
        const int mid = (lo_i + hi_i) >> 1;
        if (sh.cum[mid] <= u) lo_i = mid; else hi_i = mid;
    }
    TokenSpan s{sh.span_t[lo_i], sh.span_b[lo_i], sh.span_pos[lo_i], 0, 0, 0};
    span_blocks(a, s);
    const int r = u - sh.cum[lo_i];
    lu.idx = lo_i;
    lu.h = r / s.n_blk;
    lu.blk = s.first_blk + r % s.n_blk;
    lu.pos = s.pos; lu.lo = s.lo; lu.t = s.t;
    lu.late = a.k_new == nullptr && lu.blk * UNIT + UNIT > s.pos - a.new_keys + 1;
    return lu;
}
// Its pages, from the block table.
RING_FN void unit_pages(const RingArgs& a, const Shared& sh, LaneUnit& lu) {
    if (lu.idx < 0) return;
    const int k0 = lu.blk * UNIT;
    const int last_key = min(k0 + UNIT - 1, lu.pos);
    const int* table = a.block_table + (size_t)sh.span_b[lu.idx] * a.max_pages;
    if (a.page_size >= UNIT) {
        lu.pages[0] = table[k0 / a.page_size];
        lu.rows = UNIT;
        if (lu.pages[0] < 0 || lu.pages[0] >= a.num_pages) lu.bad = true;
    } else {
        const int fit = UNIT / a.page_size;          // 2 or 4 pages to a unit
        const int used = (last_key - k0) / a.page_size + 1;
        lu.rows = used * a.page_size;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            lu.pages[i] = (i < fit && i < used) ? table[k0 / a.page_size + i] : -1;
            if (i < used && (lu.pages[i] < 0 || lu.pages[i] >= a.num_pages)) lu.bad = true;
        }
    }
    if (lu.bad) prb_set_status(a.status, PRB_S_PAGE_RANGE, lu.t, k0, lu.pages[0]);
}
// This lane starts the copies of its unit into ring buffer `slot` of its warp.
RING_FN void issue_unit(const RingArgs& a, const CUtensorMap* map_k,
                                           const CUtensorMap* map_v, const LaneUnit& lu,
                                           uint32_t ring0, uint32_t bar0, int slot) {
    const uint32_t bar = bar0 + 8 * slot;
    if (lu.bad) {                                    // nothing to copy: the unit counts as masked
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
        return;
    }
    const uint32_t kd = ring0 + slot * 2 * TILE, vd = kd + TILE;
    const int hk = lu.h / (a.n_heads / a.kv_heads);
    mbar_expect_tx(bar, 2u * lu.rows * ROW);
    if (a.page_size >= UNIT) {
        const int row = (lu.pages[0] * a.kv_heads + hk) * a.page_size + (lu.blk * UNIT) % a.page_size;
        tma_rows(kd, map_k, bar, row);
        tma_rows(vd, map_v, bar, row);
    } else {
        const int used = lu.rows / a.page_size;
        for (int i = 0; i < used; ++i) {
            const int row = (lu.pages[i] * a.kv_heads + hk) * a.page_size;
            tma_rows(kd + i * a.page_size * ROW, map_k, bar, row);
            tma_rows(vd + i * a.page_size * ROW, map_v, bar, row);
        }
    }
}
// Where a warp's ring lies: `ring_base` is a shared-memory address on a 1,024-byte boundary
// (the swizzle is a function of the address), with blockDim.x / 32 * stages * 8 KB behind it.
__device__ __forceinline__ uint32_t warp_ring(uint32_t ring_base, int stages) {
    return ring_base + (uint32_t)(threadIdx.x >> 5) * stages * 2 * TILE;
}

// ---- early: request what does not depend on the step's kernels.  `n_ctas`, `cta`: how many
// CTAs share the launch and which one this is.
RING_FN void early(const RingArgs& a, const CUtensorMap* map_k,
                                      const CUtensorMap* map_v, Shared& sh, uint32_t ring_base,
                                      int n_ctas, int cta) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int stages = a.stages;
    if (lane == 0) {
        // (an earlier call in the same kernel has left valid, idle barriers behind)
        for (int s = 0; s < sh.bars_valid[warp]; ++s) mbar_inval(smem_addr(&sh.bars[warp * MAX_STAGES + s]));
        for (int s = 0; s < stages; ++s) mbar_init(smem_addr(&sh.bars[warp * MAX_STAGES + s]), 1);
        sh.bars_valid[warp] = stages;
        sh.edge_pair[warp][0] = sh.edge_pair[warp][1] = -1;
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    __syncwarp();
    const Run r = my_run(sh, n_ctas, cta);
    const uint32_t ring0 = warp_ring(ring_base, stages);
    const uint32_t bar0 = smem_addr(&sh.bars[warp * MAX_STAGES]);
    LaneUnit mine = decode_unit(a, sh, r.u_begin + lane, r.u_end);
    if (lane < stages) unit_pages(a, sh, mine);
    const unsigned bad = __ballot_sync(0xffffffffu, mine.bad);
    if (lane == 0) sh.bad_mask[warp] = bad;
    if (lane < stages && mine.idx >= 0 && !mine.late) issue_unit(a, map_k, map_v, mine, ring0, bar0, lane);
}

// ---- late: everything that needs the step's queries (and its own keys and values).
RING_FN void late(const RingArgs& a, const CUtensorMap* map_k,
                                     const CUtensorMap* map_v, Shared& sh, uint32_t ring_base,
                                     int n_ctas, int cta) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_warps = (int)blockDim.x >> 5;
    const int stages = a.stages;
    const Run r = my_run(sh, n_ctas, cta);
    const int u_begin = r.u_begin, u_end = r.u_end;
    const uint32_t ring0 = warp_ring(ring_base, stages);
    const uint32_t bar0 = smem_addr(&sh.bars[warp * MAX_STAGES]);
    const int hpg = a.n_heads / a.kv_heads;          // query heads per key/value head
    auto cta_of = [&](long u) { return (u / r.per) / r.wpc; };   // the CTA whose warps hold unit u

    // the lanes' units again (from shared memory), the pages of those still to be requested
    LaneUnit mine = decode_unit(a, sh, u_begin + lane, u_end);
    {
        const unsigned bad = sh.bad_mask[warp];
        if (lane < stages) mine.bad = (bad >> lane) & 1u;
        const bool need_pages = mine.idx >= 0 && (lane >= stages || mine.late);
        if (need_pages) unit_pages(a, sh, mine);
        if (lane < stages && mine.idx >= 0 && mine.late) issue_unit(a, map_k, map_v, mine, ring0, bar0, lane);
    }
    LaneUnit ahead = mine;                           // the 32 units after them, once decoded
    bool ahead_ready = false;
    int batch0 = u_begin;                            // first unit of `mine`

    // ---- walk the run.  The query is row 0 of a 16-row tile, so the lanes 0..3 (row group 0
    // of the tensor-core fragments) hold what counts: lane c of them the scores of keys
    // 8 j + 2 c, + 1 of a unit and the output dimensions 8 j + 2 c, + 1.
    const int qd = lane & 3;
    const bool row0 = lane < 4;
    float m = -INFINITY, l = 0.0f;
    float o[8][4];                                   // [dimension tile][fragment]; [j][0], [j][1] count
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f;
    uint32_t qa[4][2];                               // the query as A fragments, per 16 dimensions
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) qa[ks][0] = qa[ks][1] = 0u;
    int cur_idx = -1, cur_h = -1, cur_t = 0, cur_n_blk = 0;
    int pairs_done = 0;                              // (token, head)s this warp has left behind
    bool alive = true;

    // The running state is complete as far as this warp goes.  If the whole (token, head) lies
    // in this warp's run it is written out; otherwise it is left in shared memory for the merge
    // (only the first and the last (token, head) of a run can be shared with other warps).
    auto finish_pair = [&]() {
        const long p_u0 = (long)sh.cum[cur_idx] + (long)cur_h * cur_n_blk, p_u1 = p_u0 + cur_n_blk;
        if (p_u0 >= u_begin && p_u1 <= u_end) {
            const float inv = l > 0.0f ? 1.0f / l : 0.0f;
            __nv_bfloat16* head_out = a.out + (size_t)cur_t * a.out_stride + (size_t)cur_h * DH;
            if (row0) {
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    *reinterpret_cast<__nv_bfloat162*>(head_out + 8 * j + 2 * qd) =
                        __floats2bfloat162_rn(o[j][0] * inv, o[j][1] * inv);
            }
        } else {
            float* st = sh.edge_state[warp][pairs_done == 0 ? 0 : 1];
            if (row0) {
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    *reinterpret_cast<float2*>(st + 8 * j + 2 * qd) = make_float2(o[j][0], o[j][1]);
            }
            if (lane == 0) {
                st[DH] = m;
                st[DH + 1] = l;
                sh.edge_pair[warp][pairs_done == 0 ? 0 : 1] = cur_idx * a.n_heads + cur_h;
            }
        }
        ++pairs_done;
    };

#pragma unroll 1
    for (int u = u_begin; u < u_end && alive; ++u) {
        if (u - batch0 >= 32) {                      // on to the next 32 units (decoded when the
            mine = ahead;                            // first of them was requested)
            batch0 += 32;
            ahead_ready = false;
        }
        const int rel = u - batch0;                  // which lane decoded this unit
        const int slot = (u - u_begin) % stages;
        const uint32_t parity = (uint32_t)((u - u_begin) / stages) & 1u;
        const int idx = __shfl_sync(0xffffffffu, mine.idx, rel);
        const int h = __shfl_sync(0xffffffffu, mine.h, rel);
        const int blk = __shfl_sync(0xffffffffu, mine.blk, rel);
        const int pos = __shfl_sync(0xffffffffu, mine.pos, rel);
        const int lo = __shfl_sync(0xffffffffu, mine.lo, rel);
        const int t = __shfl_sync(0xffffffffu, mine.t, rel);
        const int bad = __shfl_sync(0xffffffffu, mine.bad ? 1 : 0, rel);
        if (idx != cur_idx || h != cur_h) {
            if (cur_idx >= 0) finish_pair();
            cur_idx = idx; cur_h = h; cur_t = t;
            TokenSpan s{t, sh.span_b[idx], pos, 0, 0, 0};
            span_blocks(a, s);
            cur_n_blk = s.n_blk;
            m = -INFINITY; l = 0.0f;
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f;
            // this pair's query as A fragments: row 0 only, so only lanes 0..3 hold any of it
            const uint32_t* qp = reinterpret_cast<const uint32_t*>(
                a.q + (size_t)t * a.q_stride + (size_t)h * DH);
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                qa[ks][0] = row0 ? qp[8 * ks + qd] : 0u;          // dimensions 16 ks + 2 c, + 1
                qa[ks][1] = row0 ? qp[8 * ks + 4 + qd] : 0u;      // dimensions 16 ks + 8 + 2 c, + 1
            }
        }
        if (!mbar_wait_bounded(bar0 + 8 * slot, parity)) {
            if (lane == 0) prb_set_status(a.status, PRB_S_WAIT_TIMEOUT, 32, cta, u);
            alive = false;
            break;
        }
        if (u == u_begin) RING_TRACE(4);
        const uint32_t kd = ring0 + slot * 2 * TILE, vd = kd + TILE;
        if (a.k_new != nullptr && !bad && (blk + 1) * UNIT > pos - a.new_keys + 1) {
            // rows of this unit that the step itself appended: lanes 8 j .. 8 j + 7 bring the
            // row of position pos - j, if token t - j is that position of the same request
            const int j = lane >> 3, c = lane & 7;
            const int key = pos - j;
            const int src = idx - j;                 // its place in the token list
            if (j < a.new_keys && key >= blk * UNIT && key < (blk + 1) * UNIT && key >= lo && src >= 0 &&
                sh.span_t[src] == t - j && sh.span_b[src] == sh.span_b[idx] && sh.span_pos[src] == key) {
                const int hk = h / hpg, rr = key - blk * UNIT;
                const size_t off = (size_t)(t - j) * a.kv_stride + (size_t)hk * DH + c * 8;
                const uint4 kk = *reinterpret_cast<const uint4*>(a.k_new + off);
                const uint4 vv = *reinterpret_cast<const uint4*>(a.v_new + off);
                const uint32_t dst = (uint32_t)rr * ROW + (uint32_t)((c ^ (rr & 7)) << 4);
                asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(kd + dst), "r"(kk.x), "r"(kk.y), "r"(kk.z), "r"(kk.w) : "memory");
                asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(vd + dst), "r"(vv.x), "r"(vv.y), "r"(vv.z), "r"(vv.w) : "memory");
            }
            __syncwarp();
        }
        // a masked key's values must be finite: what an earlier owner of the page left there is
        // zeroed (lane j looks after row j) before it is multiplied by a zero weight
        {
            const int key = blk * UNIT + lane;
            if (bad || key < lo || key > pos) {
#pragma unroll
                for (int c = 0; c < 8; ++c)
                    asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(vd + lane * ROW + c * 16), "r"(0u) : "memory");
            }
        }
        // ---- scores S = q . K^T: key tiles of 8 (B fragments straight from the rows of the
        // swizzled tile), 16 dimensions a step
        float sc[4][4];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.0f;
        {
            const int rr = lane & 7, mi = lane >> 3; // this lane gives the address of row rr of matrix mi
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) {
                const uint32_t rowaddr = kd + (uint32_t)(8 * nt + rr) * ROW;
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    uint32_t b[4];                   // 16-byte pieces 4 half + 0..3 of the 8 rows
                    ldmatrix_x4(rowaddr + (uint32_t)(((4 * half + mi) ^ rr) << 4), b);
                    mma_row(sc[nt], qa[2 * half][0], qa[2 * half][1], b[0], b[1]);
                    mma_row(sc[nt], qa[2 * half + 1][0], qa[2 * half + 1][1], b[2], b[3]);
                }
            }
        }
        // ---- softmax over the unit's keys (row 0: lanes 0..3), running maximum and sum
        float um = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int key = blk * UNIT + 8 * nt + 2 * qd + e;
                const bool seen = row0 && !bad && key >= lo && key <= pos;
                sc[nt][e] = seen ? sc[nt][e] * a.scale : -INFINITY;
                um = fmaxf(um, sc[nt][e]);
            }
        um = fmaxf(um, __shfl_xor_sync(0xffffffffu, um, 1));
        um = fmaxf(um, __shfl_xor_sync(0xffffffffu, um, 2));
        const float m_new = fmaxf(m, um);
        float corr = 1.0f, ps = 0.0f;
        uint32_t pa[2][2];                           // the weights as A fragments, per 16 keys
        {
            float pv[4][2];
#pragma unroll
            for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    pv[nt][e] = (m_new > -INFINITY && sc[nt][e] > -INFINITY) ? __expf(sc[nt][e] - m_new) : 0.0f;
                    ps += pv[nt][e];
                }
            if (m_new > -INFINITY) corr = (m == -INFINITY) ? 0.0f : __expf(m - m_new);
            pa[0][0] = pack_bf16(pv[0][0], pv[0][1]);
            pa[0][1] = pack_bf16(pv[1][0], pv[1][1]);
            pa[1][0] = pack_bf16(pv[2][0], pv[2][1]);
            pa[1][1] = pack_bf16(pv[3][0], pv[3][1]);
        }
        ps += __shfl_xor_sync(0xffffffffu, ps, 1);
        ps += __shfl_xor_sync(0xffffffffu, ps, 2);
        l = l * corr + ps;
        m = m_new;
        __syncwarp();                                 // the zeroed value rows are in place
        // ---- O = O * corr + P . V: dimension tiles of 8, 16 keys a step (B fragments by
        // transposing loads from the rows of the value tile)
#pragma unroll
        for (int j = 0; j < 8; ++j) { o[j][0] *= corr; o[j][1] *= corr; }
        {
            const int rr = lane & 7, mi = lane >> 3;
#pragma unroll
            for (int ks = 0; ks < 2; ++ks)
#pragma unroll
                for (int jp = 0; jp < 4; ++jp) {     // dimension tiles 2 jp, 2 jp + 1
                    // matrices: (keys 16 ks + 0..7, piece 2 jp), (keys + 8.., piece 2 jp),
                    //           (keys 16 ks + 0..7, piece 2 jp + 1), (keys + 8.., piece 2 jp + 1)
                    const int key_row = 16 * ks + 8 * (mi & 1) + rr;
                    const int piece = 2 * jp + (mi >> 1);
                    uint32_t b[4];
                    ldmatrix_x4_trans(vd + (uint32_t)key_row * ROW + (uint32_t)((piece ^ (key_row & 7)) << 4), b);
                    mma_row(o[2 * jp], pa[ks][0], pa[ks][1], b[0], b[1]);
                    mma_row(o[2 * jp + 1], pa[ks][0], pa[ks][1], b[2], b[3]);
                }
        }
        __syncwarp();                                 // every lane has read the buffer
        // ---- the buffer is free: the unit `stages` ahead takes it
        const int nu = u + stages;
        if (nu < u_end) {
            // (generic-proxy accesses to the buffer come before the copy engine's writes)
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            if (nu - batch0 < 32) {
                if (lane == nu - batch0) issue_unit(a, map_k, map_v, mine, ring0, bar0, slot);
            } else {
                if (!ahead_ready) {
                    ahead = decode_unit(a, sh, batch0 + 32 + lane, u_end);
                    unit_pages(a, sh, ahead);
                    ahead_ready = true;
                }
                if (lane == nu - batch0 - 32) issue_unit(a, map_k, map_v, ahead, ring0, bar0, slot);
            }
        }
    }
    if (alive && cur_idx >= 0) finish_pair();
    if (!alive) {
        // a wait gave up: wait once more, bounded, for this warp's own copies in flight
        for (int s = 0; s < stages; ++s)
            for (uint32_t i = 0; i < (1u << 16); ++i)
                if (mbar_try_wait(bar0 + 8 * s, 0) || mbar_try_wait(bar0 + 8 * s, 1)) break;
    }
    RING_TRACE(5);
    __syncthreads();                                  // every warp's edge states are in place

    // ---- merge.  The edge states of the CTA's warps, in warp order, form chains of the same
    // (token, head); the warp that holds a chain's first state merges it.  A chain that is the
    // whole (token, head) is written out; otherwise it goes to the workspace, and the last CTA
    // of that (token, head) to arrive merges the CTAs' states in CTA order.
#pragma unroll 1
    for (int e = 0; e < 2; ++e) {
        const int pair = sh.edge_pair[warp][e];
        if (pair < 0) continue;
        bool first = true;                            // no earlier state of this pair in the CTA?
        if (e == 1 && sh.edge_pair[warp][0] == pair) first = false;
        if (first && warp > 0 && (sh.edge_pair[warp - 1][1] == pair ||
                                  (sh.edge_pair[warp - 1][1] < 0 && sh.edge_pair[warp - 1][0] == pair)))
            first = false;
        if (!first) continue;
        Partial acc{-INFINITY, 0.0f, 0.0f, 0.0f};
        bool go = true;
#pragma unroll 1
        for (int w = warp; w < n_warps && go; ++w)
#pragma unroll 1
            for (int e2 = (w == warp ? e : 0); e2 < 2; ++e2) {
                if (sh.edge_pair[w][e2] != pair) {
                    // a warp's second slot may be empty (its run was one (token, head) long)
                    if (sh.edge_pair[w][e2] < 0 && e2 == 1) continue;
                    go = false;
                    break;
                }
                const float* st = sh.edge_state[w][e2];
                merge_into(acc, st[DH], st[DH + 1], st[2 * lane], st[2 * lane + 1]);
            }
        const int idx = pair / a.n_heads, h = pair - idx * a.n_heads;
        TokenSpan s{sh.span_t[idx], sh.span_b[idx], sh.span_pos[idx], 0, 0, 0};
        span_blocks(a, s);
        const long p_u0 = (long)sh.cum[idx] + (long)h * s.n_blk, p_u1 = p_u0 + s.n_blk;
        const long fc = cta_of(p_u0), lc = cta_of(p_u1 - 1);
        __nv_bfloat16* dst = a.out + (size_t)s.t * a.out_stride + (size_t)h * DH + 2 * lane;
        if (fc == lc) {
            const float inv = acc.l > 0.0f ? 1.0f / acc.l : 0.0f;
            *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(acc.o0 * inv, acc.o1 * inv);
            continue;
        }
        float* part = a.workspace + (size_t)(cta + pair) * PART;
        *reinterpret_cast<float2*>(part + 2 * lane) = make_float2(acc.o0, acc.o1);
        if (lane == 0) { part[DH] = acc.m; part[DH + 1] = acc.l; }
        __threadfence();
        __syncwarp();
        int last = 0;
        if (lane == 0) last = atomicAdd(&a.counters[pair], 1) == (int)(lc - fc) ? 1 : 0;
        last = __shfl_sync(0xffffffffu, last, 0);
        if (!last) continue;
        __threadfence();
        // the CTAs' states in CTA order (= block order); all loads first, then the sums
        Partial tot{-INFINITY, 0.0f, 0.0f, 0.0f};
#pragma unroll 1
        for (long c0 = fc; c0 <= lc; c0 += 4) {
            float pm[4], pl[4];
            float2 po[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float* pw = a.workspace + (size_t)(min(c0 + j, lc) + pair) * PART;
                pm[j] = __ldcg(pw + DH);
                pl[j] = __ldcg(pw + DH + 1);
                po[j] = __ldcg(reinterpret_cast<const float2*>(pw + 2 * lane));
            }
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (c0 + j <= lc) merge_into(tot, pm[j], pl[j], po[j].x, po[j].y);
        }
        const float inv = tot.l > 0.0f ? 1.0f / tot.l : 0.0f;
        *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(tot.o0 * inv, tot.o1 * inv);
        if (lane == 0) a.counters[pair] = 0;
    }
    RING_TRACE(6);
}

// Host side: checks and the two tensor maps (the cache as a matrix of 64 columns; a copy
// brings the rows of a unit, or of a page where pages are shorter than a unit).
inline int supports(int head_dim, int page_size) {
    return head_dim == DH &&
           (page_size == 8 || page_size == 16 || (page_size >= 32 && page_size % 32 == 0));
}
inline int check_and_maps(const void* q, long q_stride, const void* out, long out_stride,
                          const void* k_pages, const void* v_pages, int n_list, int n_heads,
                          int kv_heads, int head_dim, int page_size, int num_pages, int new_keys,
                          const void* k_new, const void* v_new, long kv_stride,
                          CUtensorMap* mk, CUtensorMap* mv) {
    if (!supports(head_dim, page_size) || n_heads <= 0 || kv_heads <= 0 || n_heads % kv_heads != 0 ||
        n_list > MAX_LIST || new_keys < 1 || new_keys > 4 ||
        (long)num_pages * kv_heads * page_size > 0x7fffffffL)
        return PRB_E_SIZE;
    if (q_stride % 8 != 0 || ((uintptr_t)q) % 16 != 0 || ((uintptr_t)k_pages) % 16 != 0 ||
        ((uintptr_t)v_pages) % 16 != 0 || ((uintptr_t)out) % 4 != 0 || out_stride % 2 != 0 ||
        ((k_new != nullptr) != (v_new != nullptr)) ||
        (k_new != nullptr && (kv_stride % 8 != 0 || ((uintptr_t)k_new) % 16 != 0 || ((uintptr_t)v_new) % 16 != 0)))
        return PRB_E_ALIGN;
    const long cache_rows = (long)num_pages * kv_heads * page_size;
    const int box_rows = page_size >= UNIT ? UNIT : page_size;
    int rc = tmap::get_map(k_pages, cache_rows, DH, DH, box_rows, mk);
    if (rc) return rc;
    return tmap::get_map(v_pages, cache_rows, DH, DH, box_rows, mv);
}
}  // namespace ring
