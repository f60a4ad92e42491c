// Decode attention over the paged bfloat16 cache, second kernel: persistent CTAs whose warps
// each stream their share of the keys and values through a private ring of shared-memory
// buffers filled by bulk copies (cp.async.bulk, no multicast).
//
// Why a second kernel.  A decode step is a chain of short dependent kernels, and what a
// decode attention launch costs is not its bytes but its latencies in a row: wait for the
// QKV product, read the step's description, read the block table, ask HBM for the first
// keys, score them, merge.  Almost none of that depends on the QKV product: every key and
// value that was cached before this step, the block tables and the positions are there
// before the step begins.  So this kernel is launched early (programmatic dependent launch),
// one CTA per SM, reads the description, divides the work, and has its bulk copies of all
// OLD keys and values in flight or landed before the product it depends on has finished.
// After the dependency resolves it fetches the queries and the few rows the step itself
// appended, and computes from shared memory.
//
// Work.  A unit is 32 consecutive key positions [32 i, 32 i + 32) of one (token, head): one
// key per lane.  Units are numbered token by token, head by head, block by block; the G * 8
// warps of the grid take equal contiguous runs of that numbering, so a warp walks consecutive
// blocks of the same (token, head) and keeps a running softmax state (maximum, sum, weighted
// values, all float32) in registers.  Where a (token, head) is shared by several warps each
// writes its partial state to the workspace and counts itself in; the last one merges the
// partial states in warp order, which is block order.  Nobody waits for anybody: the only
// waits are on a warp's own copies, and they are bounded.
//
// Scores are (q . k) * scale in float32; keys outside [lo, pos] are masked by selection, and
// the value rows of masked keys are zeroed in shared memory before they are multiplied by a
// zero weight, so that whatever a page's earlier owner left there cannot reach the output.
//
// Limits: head size 64, page sizes 8, 16 or a multiple of 32.  Other sizes are refused
// (the caller uses the register-batch kernel of attention_decode.cu).
#include "common.cuh"

namespace {
constexpr int RING_THREADS = 256;
constexpr int RING_WARPS = RING_THREADS / 32;
constexpr int UNIT = 32;                      // keys per unit, one per lane
constexpr int MAX_LIST = 1024;                // most single tokens of a launch
constexpr int MAX_STAGES = 4;
constexpr uint32_t RING_WAIT_LIMIT = 1u << 22;

struct RingArgs {
    __nv_bfloat16* out;
    long out_stride;
    const __nv_bfloat16* q;
    long q_stride;
    const __nv_bfloat16* k_pages;
    const __nv_bfloat16* v_pages;
    const int* block_table;
    const int* seq_of_token;
    const int* positions;
    const int* token_list;
    const int* token_count;
    int n_list, n_heads, kv_heads, page_size, max_pages, num_pages;
    float scale;
    int window;
    int new_keys;                   // a token's last `new_keys` visible positions may have been
                                    // written by the step itself: fetched after the dependency
    float* workspace;               // [(workers + n_list * n_heads)][DH + 4] float32
    int* counters;                  // [n_list * n_heads] int32, zero; left zero
    int stages;
    int* status;
};

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
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
__device__ __forceinline__ void bulk_copy(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
        "l"(src), "r"(bytes), "r"(bar)
        : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ float dot8(const uint4& a, const uint4& b) {
    const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&b);
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 fa = __bfloat1622float2(pa[i]), fb = __bfloat1622float2(pb[i]);
        s = fmaf(fa.x, fb.x, s);
        s = fmaf(fa.y, fb.y, s);
    }
    return s;
}

// Where a token's keys are: request, position, first and number of 32-key blocks.
struct TokenSpan {
    int t, b, pos, lo, first_blk, n_blk;
};
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
    s.lo = (a.window > 0 && s.pos - a.window + 1 > 0) ? s.pos - a.window + 1 : 0;
    s.first_blk = s.lo / UNIT;
    s.n_blk = s.pos / UNIT - s.first_blk + 1;
    return s;
}

template <int DH>
__global__ void __launch_bounds__(RING_THREADS, 1)
attention_decode_ring_kernel(RingArgs a) {
    constexpr int CH = DH / 8;                      // 16-byte pieces of a row
    constexpr int DPL = DH / 32;                    // output dimensions per lane
    constexpr int ROW = DH * 2;                     // bytes of a row
    constexpr int TILE = UNIT * ROW;                // bytes of a unit's keys (and of its values)
    extern __shared__ __align__(128) unsigned char ring_raw[];
    __shared__ int cum[MAX_LIST + 1];               // units before each place of the token list
    __shared__ int warp_tot[RING_WARPS];
    __shared__ __align__(8) unsigned long long bars[RING_WARPS * MAX_STAGES];
    __shared__ __align__(16) __nv_bfloat16 q_sh[RING_WARPS][DH];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    prb_grid_launch_dependents();                   // the next kernel may set itself up

    // ---- the step's description (it was copied to the device before the step's first
    // kernel): units per token, and their running sum
    int n = a.n_list;
    if (a.token_count != nullptr) n = min(n, *a.token_count);
    {
        int run = 0;                                // units before this thread's chunk so far
        for (int base = 0; base < n; base += RING_THREADS) {
            const TokenSpan s = token_span(a, base + (int)threadIdx.x, n);
            const int mine = s.b >= 0 ? s.n_blk * a.n_heads : 0;
            int incl = mine;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += v;
            }
            if (lane == 31) warp_tot[warp] = incl;
            __syncthreads();
            int before = 0, total = 0;
#pragma unroll
            for (int w = 0; w < RING_WARPS; ++w) {
                const int c = warp_tot[w];
                if (w < warp) before += c;
                total += c;
            }
            if (base + (int)threadIdx.x < n) cum[base + threadIdx.x] = run + before + incl - mine;
            run += total;
            __syncthreads();
        }
        if (threadIdx.x == 0) cum[n] = run;
    }
    const int stages = a.stages;
    if (lane == 0)
        for (int s = 0; s < stages; ++s) mbar_init(smem_addr(&bars[warp * MAX_STAGES + s]), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    __syncthreads();

    // Runs of `per` units each, dealt to workers 0, 1, 2, ...; consecutive workers are warps of
    // different CTAs, so that a launch with few units is spread over all SMs.
    const long total_units = cum[n];
    const long workers = (long)gridDim.x * RING_WARPS;
    const long per = (total_units + workers - 1) / workers;
    const long gw = (long)warp * gridDim.x + blockIdx.x;
    const long run0 = gw * per;
    const int u_begin = (int)(run0 < total_units ? run0 : total_units);
    const int u_end = (int)(run0 + per < total_units ? run0 + per : total_units);
    if (u_begin >= u_end) {                          // nothing for this warp
        prb_grid_wait();
        return;
    }
    auto worker_of = [&](long u) { return u / per; };   // the warp whose run holds unit u

    unsigned char* my_ring = ring_raw + (size_t)warp * stages * 2 * TILE;
    const uint32_t ring0 = smem_addr(my_ring);
    const uint32_t bar0 = smem_addr(&bars[warp * MAX_STAGES]);
    const int hpg = a.n_heads / a.kv_heads;          // query heads per key/value head

    // ---- a lane's own unit of the current batch of 32 units: decoded once, then its copies
    // are issued by that lane when the unit's ring buffer is free
    struct LaneUnit {
        int idx, h, blk;            // place in the token list, head, absolute 32-key block
        int b, pos, lo, t;
        bool late;                  // holds rows the step itself may have written
        bool bad;                   // a page of it lies outside the pool
        int pages[4];               // its pages (one when the page holds 32 keys or more)
        int rows;                   // rows to copy: up to the end of the last page it touches
    };
    auto decode = [&](int u) {
        LaneUnit lu;
        lu.idx = -1;
        if (u >= u_end) return lu;
        int lo_i = 0, hi_i = n;                      // largest idx with cum[idx] <= u
        while (hi_i - lo_i > 1) {
            const int mid = (lo_i + hi_i) >> 1;
            if (cum[mid] <= u) lo_i = mid; else hi_i = mid;
        }
        const TokenSpan s = token_span(a, lo_i, n);
        const int r = u - cum[lo_i];
        lu.idx = lo_i;
        lu.h = r / s.n_blk;
        lu.blk = s.first_blk + r % s.n_blk;
        lu.b = s.b; lu.pos = s.pos; lu.lo = s.lo; lu.t = s.t;
        const int k0 = lu.blk * UNIT;
        lu.late = k0 + UNIT > s.pos - a.new_keys + 1;
        lu.bad = false;
        const int last_key = min(k0 + UNIT - 1, s.pos);
        const int* table = a.block_table + (size_t)s.b * a.max_pages;
        if (a.page_size >= UNIT) {
            lu.pages[0] = table[k0 / a.page_size];
            lu.pages[1] = lu.pages[2] = lu.pages[3] = -1;
            lu.rows = UNIT;
            if (lu.pages[0] < 0 || lu.pages[0] >= a.num_pages) lu.bad = true;
        } else {
            const int per = UNIT / a.page_size;      // 2 or 4 pages to a unit
            const int used = (last_key - k0) / a.page_size + 1;
            lu.rows = used * a.page_size;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                lu.pages[i] = (i < per && i < used) ? table[k0 / a.page_size + i] : -1;
                if (i < used && (lu.pages[i] < 0 || lu.pages[i] >= a.num_pages)) lu.bad = true;
            }
        }
        if (lu.bad) prb_set_status(a.status, PRB_S_PAGE_RANGE, s.t, k0, lu.pages[0]);
        return lu;
    };
    auto issue = [&](const LaneUnit& lu, int slot) {  // this lane starts the copies of its unit
        const uint32_t bar = bar0 + 8 * slot;
        if (lu.bad) {                                // nothing to copy: the unit counts as masked
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
            return;
        }
        const uint32_t kd = ring0 + slot * 2 * TILE, vd = kd + TILE;
        const int hk = lu.h / hpg;
        mbar_expect_tx(bar, 2u * lu.rows * ROW);
        if (a.page_size >= UNIT) {
            const size_t row = (((size_t)lu.pages[0] * a.kv_heads + hk) * a.page_size +
                                (lu.blk * UNIT) % a.page_size) * DH;
            bulk_copy(kd, a.k_pages + row, UNIT * ROW, bar);
            bulk_copy(vd, a.v_pages + row, UNIT * ROW, bar);
        } else {
            const int used = lu.rows / a.page_size;
            for (int i = 0; i < used; ++i) {
                const size_t row = (((size_t)lu.pages[i] * a.kv_heads + hk) * a.page_size) * DH;
                bulk_copy(kd + i * a.page_size * ROW, a.k_pages + row, a.page_size * ROW, bar);
                bulk_copy(vd + i * a.page_size * ROW, a.v_pages + row, a.page_size * ROW, bar);
            }
        }
    };

    // ---- before the dependency: every old unit that has a ring buffer is requested
    LaneUnit mine = decode(u_begin + lane);          // units u_begin .. u_begin + 31
    LaneUnit ahead = mine;                           // the 32 units after them, once decoded
    bool ahead_ready = false;
    int batch0 = u_begin;                            // first unit of `mine`
    if (lane < stages && mine.idx >= 0 && !mine.late) issue(mine, lane);
    prb_grid_wait();
    if (lane < stages && mine.idx >= 0 && mine.late) issue(mine, lane);

    // ---- walk the run
    float m = -INFINITY, l = 0.0f, o[DPL];
#pragma unroll
    for (int i = 0; i < DPL; ++i) o[i] = 0.0f;
    int cur_idx = -1, cur_h = -1;                    // the (token, head) of the running state
    int cur_t = 0, cur_first_blk = 0, cur_n_blk = 0;
    bool alive = true;

    auto finish_pair = [&]() {
        // the running state belongs to (cur_idx, cur_h): is the pair all ours?
        const long p_u0 = (long)cum[cur_idx] + (long)cur_h * cur_n_blk, p_u1 = p_u0 + cur_n_blk;
        const long fw = worker_of(p_u0), lw = worker_of(p_u1 - 1);
        __nv_bfloat16* dst = a.out + (size_t)cur_t * a.out_stride + (size_t)cur_h * DH + lane * DPL;
        if (fw == lw) {
            const float inv = l > 0.0f ? 1.0f / l : 0.0f;
#pragma unroll
            for (int i = 0; i < DPL; i += 2)
                *reinterpret_cast<__nv_bfloat162*>(dst + i) = __floats2bfloat162_rn(o[i] * inv, o[i + 1] * inv);
            return;
        }
        const long pair = (long)cur_idx * a.n_heads + cur_h;
        float* part = a.workspace + (size_t)(gw + pair) * (DH + 4);
#pragma unroll
        for (int i = 0; i < DPL; ++i) part[lane * DPL + i] = o[i];
        if (lane == 0) { part[DH] = m; part[DH + 1] = l; }
        __threadfence();
        __syncwarp();
        int last = 0;
        if (lane == 0) last = atomicAdd(&a.counters[pair], 1) == (int)(lw - fw) ? 1 : 0;
        last = __shfl_sync(0xffffffffu, last, 0);
        if (!last) return;
        __threadfence();
        // merge the partial states in warp order (= block order)
        float mg = -INFINITY;
        for (long w = fw; w <= lw; ++w)
            mg = fmaxf(mg, __ldcg(a.workspace + (size_t)(w + pair) * (DH + 4) + DH));
        float lg = 0.0f, og[DPL];
#pragma unroll
        for (int i = 0; i < DPL; ++i) og[i] = 0.0f;
        for (long w = fw; w <= lw; ++w) {
            const float* pw = a.workspace + (size_t)(w + pair) * (DH + 4);
            const float mw = __ldcg(pw + DH);
            const float c = (mw == -INFINITY) ? 0.0f : __expf(mw - mg);
            lg += __ldcg(pw + DH + 1) * c;
#pragma unroll
            for (int i = 0; i < DPL; ++i) og[i] += __ldcg(pw + lane * DPL + i) * c;
        }
        const float inv = lg > 0.0f ? 1.0f / lg : 0.0f;
#pragma unroll
        for (int i = 0; i < DPL; i += 2)
            *reinterpret_cast<__nv_bfloat162*>(dst + i) = __floats2bfloat162_rn(og[i] * inv, og[i + 1] * inv);
        if (lane == 0) a.counters[pair] = 0;
    };

    for (int u = u_begin; u < u_end && alive; ++u) {
        if (u - batch0 >= 32) {                      // on to the next 32 units (decoded when the
            mine = ahead;                            // first of them was requested)
            batch0 += 32;
            ahead_ready = false;
        }
        const int rel = u - batch0;                  // which lane decoded this unit
        const int slot = (u - u_begin) % stages;
        const uint32_t parity = (uint32_t)((u - u_begin) / stages) & 1u;
        // the unit's description, from the lane that holds it
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
            const TokenSpan s = token_span(a, idx, n);
            cur_first_blk = s.first_blk; cur_n_blk = s.n_blk;
            m = -INFINITY; l = 0.0f;
#pragma unroll
            for (int i = 0; i < DPL; ++i) o[i] = 0.0f;
            // this pair's query (bfloat16, 16 bytes per lane) into the warp's shared row
            if (lane < CH) {
                const uint4 qv = *reinterpret_cast<const uint4*>(
                    a.q + (size_t)t * a.q_stride + (size_t)h * DH + lane * 8);
                *reinterpret_cast<uint4*>(&q_sh[warp][lane * 8]) = qv;
            }
            __syncwarp();
        }
        if (!mbar_wait_bounded(bar0 + 8 * slot, parity)) {
            if (lane == 0) prb_set_status(a.status, PRB_S_WAIT_TIMEOUT, 32, (int)blockIdx.x, u);
            alive = false;
            break;
        }
        const uint32_t kd = ring0 + slot * 2 * TILE, vd = kd + TILE;
        const int key = blk * UNIT + lane;           // this lane's key position
        const bool seen = !bad && key >= lo && key <= pos;
        // ---- score: q . k over the row, pieces taken in an order rotated by the lane so
        // that the 32 rows are read without bank conflicts
        float sc = 0.0f;
        const uint32_t krow = kd + lane * ROW, qrow = smem_addr(&q_sh[warp][0]);
#pragma unroll
        for (int c = 0; c < CH; ++c) {
            const int piece = (c + lane) & (CH - 1);
            sc += dot8(lds128(krow + piece * 16), lds128(qrow + piece * 16));
        }
        sc = seen ? sc * a.scale : -INFINITY;
        if (!seen) {                                  // a masked key's values must be finite: zero
#pragma unroll
            for (int c = 0; c < CH; ++c)
                asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(vd + lane * ROW + c * 16), "r"(0u) : "memory");
        }
        float um = sc;
#pragma unroll
        for (int s2 = 16; s2 > 0; s2 >>= 1) um = fmaxf(um, __shfl_xor_sync(0xffffffffu, um, s2));
        const float m_new = fmaxf(m, um);
        float p = 0.0f, corr = 1.0f;
        if (m_new > -INFINITY) {
            p = seen ? __expf(sc - m_new) : 0.0f;
            corr = (m == -INFINITY) ? 0.0f : __expf(m - m_new);
        }
        float ps = p;
#pragma unroll
        for (int s2 = 16; s2 > 0; s2 >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, s2);
        l = l * corr + ps;
        m = m_new;
        __syncwarp();                                 // the zeroed value rows are in place
        // ---- weighted values: this lane's DPL output dimensions over the 32 keys, in key order
#pragma unroll
        for (int i = 0; i < DPL; ++i) o[i] *= corr;
        const uint32_t vcol = vd + lane * DPL * 2;
#pragma unroll 8
        for (int j = 0; j < UNIT; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            if constexpr (DPL == 2) {
                uint32_t raw;
                asm volatile("ld.shared.u32 %0, [%1];" : "=r"(raw) : "r"(vcol + j * ROW));
                const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw));
                o[0] = fmaf(pj, f.x, o[0]);
                o[1] = fmaf(pj, f.y, o[1]);
            } else {
                uint2 raw;
                asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(raw.x), "=r"(raw.y) : "r"(vcol + j * ROW));
                const float2 f0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
                const float2 f1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
                o[0] = fmaf(pj, f0.x, o[0]);
                o[1] = fmaf(pj, f0.y, o[1]);
                o[2] = fmaf(pj, f1.x, o[2]);
                o[3] = fmaf(pj, f1.y, o[3]);
            }
        }
        __syncwarp();                                 // every lane has read the buffer
        // ---- the buffer is free: the unit `stages` ahead takes it
        const int nu = u + stages;
        if (nu < u_end) {
            // (generic-proxy accesses to the buffer come before the copy engine's writes)
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            if (nu - batch0 < 32) {
                if (lane == nu - batch0) issue(mine, slot);
            } else {
                if (!ahead_ready) {
                    ahead = decode(batch0 + 32 + lane);
                    ahead_ready = true;
                }
                if (lane == nu - batch0 - 32) issue(ahead, slot);
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
}

template <int DH>
int launch_ring(const RingArgs& a, int grid, cudaStream_t stream) {
    const size_t smem = (size_t)RING_WARPS * a.stages * 2 * UNIT * DH * 2;
    static size_t configured = 0;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_decode_ring_kernel<DH>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = smem;
    }
    cudaError_t e = prb_launch_dependent(attention_decode_ring_kernel<DH>, dim3(grid),
                                         dim3(RING_THREADS), smem, stream, a);
    return e == cudaSuccess ? 0 : (int)e;
}
}  // namespace

// Whether the kernel takes these sizes.
PRB_API int prb_attention_decode_ring_supports(int head_dim, int page_size) {
    return head_dim == 64 &&
           (page_size == 8 || page_size == 16 || (page_size >= 32 && page_size % 32 == 0));
}

// Floats of workspace a launch of up to n_list tokens needs.
PRB_API long prb_attention_decode_ring_workspace(int n_list, int n_heads, int head_dim) {
    return ((long)prb_sm_count() * RING_WARPS + (long)n_list * n_heads) * (head_dim + 4);
}

// new_keys: how many of a token's last visible positions the step itself may have written
// (the most tokens a request brings to this kernel in one step).  stages: ring buffers per
// warp (2 to 4; 0 = the kernel's choice).  workspace: prb_attention_decode_ring_workspace
// floats; counters: n_list * n_heads int32, zero (left zero).
PRB_API int prb_attention_decode_ring(void* out, long out_stride, const void* q, long q_stride,
                                      const void* k_pages, const void* v_pages,
                                      const int* block_table, const int* seq_of_token,
                                      const int* positions, const int* token_list,
                                      const int* token_count, int n_list, int n_heads,
                                      int kv_heads, int head_dim, int page_size, int max_pages,
                                      int num_pages, float scale, int window, int new_keys,
                                      float* workspace, int* counters, int stages,
                                      int max_context, int* status, cudaStream_t stream) {
    if (n_list <= 0) return 0;
    if (!prb_attention_decode_ring_supports(head_dim, page_size) || n_heads <= 0 || kv_heads <= 0 ||
        n_heads % kv_heads != 0 || n_list > MAX_LIST || new_keys < 1 || stages < 0 ||
        stages > MAX_STAGES || stages == 1)
        return PRB_E_SIZE;
    if (q_stride % 8 != 0 || ((uintptr_t)q) % 16 != 0 || ((uintptr_t)k_pages) % 16 != 0 ||
        ((uintptr_t)v_pages) % 16 != 0 || ((uintptr_t)out) % 4 != 0 || out_stride % 2 != 0)
        return PRB_E_ALIGN;
    RingArgs a;
    a.out = (__nv_bfloat16*)out; a.out_stride = out_stride;
    a.q = (const __nv_bfloat16*)q; a.q_stride = q_stride;
    a.k_pages = (const __nv_bfloat16*)k_pages; a.v_pages = (const __nv_bfloat16*)v_pages;
    a.block_table = block_table; a.seq_of_token = seq_of_token; a.positions = positions;
    a.token_list = token_list; a.token_count = token_count;
    a.n_list = n_list; a.n_heads = n_heads; a.kv_heads = kv_heads; a.page_size = page_size;
    a.max_pages = max_pages; a.num_pages = num_pages; a.scale = scale; a.window = window;
    a.new_keys = new_keys; a.workspace = workspace; a.counters = counters; a.status = status;
    const int sms = prb_sm_count();
    // Ring depth: with a short run per warp two buffers hold all of it and leave shared memory
    // for the next kernel's early CTAs; longer runs stream, and bytes in flight are what counts.
    const long units = (long)n_list * n_heads * ((max_context > 0 ? max_context : page_size * max_pages) / UNIT + 1);
    const long per_warp = (units + (long)sms * RING_WARPS - 1) / ((long)sms * RING_WARPS);
    int st = stages > 0 ? stages : (per_warp <= 2 ? 2 : 3);
    if ((size_t)RING_WARPS * st * 2 * UNIT * head_dim * 2 > 200 * 1024) st = 2;
    a.stages = st;
    return launch_ring<64>(a, sms, stream);
}
