// Decode attention over the paged bfloat16 cache: one query row per (token, head), keys
// split into fixed ranges of absolute positions so that a single token still fills the
// GPU, partial results merged in split order.
//
// Grid (token list, head, split).  Split s owns positions [s*split, (s+1)*split), split a
// multiple of 128 keys and of the page size chosen per launch (fewer, longer splits when
// there are many (token, head) pairs), so what a split sums and in which order depends only on
// the token's own visible range [lo, pos], never on the batch.  Each warp takes the
// keys of the split in turn, 32/LPK keys per load (LPK lanes share one key row, 16 bytes
// each), keeps a running maximum and sum (online softmax, float32) and accumulates
// weighted values; warps are merged through shared memory, splits through a float32
// workspace: the last CTA of a (token, head) to finish merges all of its splits in
// order s = first..last (a counter in scratch memory tells which CTA is last, and is
// reset by it).  Softmax statistics and all sums are float32.
//
// Scratch: workspace [tokens, heads, max_splits, head_dim + 4] float32 and counters
// [tokens * heads] int32 (zero before the first launch; the kernel leaves them zero).
//
// The unit of work (one token, one head, one split) is a device function of its own; the
// kernels of attention_decode.cu call it.
#pragma once
#include "common.cuh"

#ifndef DEC_TRACE
#define DEC_TRACE(slot)
#endif

namespace decode_attn {
constexpr int SPLIT = 128;          // granule of the split size (keys); a multiple of the page size
constexpr int MAX_SPLIT_PAGES = 128; // most pages one split may span
constexpr int MAX_DH = 256;

struct Args {
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
    int n_heads, kv_heads, head_dim, page_size, max_pages, num_pages;
    float scale;
    int window;
    float* workspace;
    int* counters;
    int max_splits;
    int split;                      // keys per split: a multiple of SPLIT
    int* status;
};

__device__ __forceinline__ float dot8(const uint4& a, const float* q) {
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&a);
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(p[i]);
        s = fmaf(f.x, q[2 * i], s);
        s = fmaf(f.y, q[2 * i + 1], s);
    }
    return s;
}

// Shared memory of one unit; the caller provides it.
template <int NW> struct Shared {
    float m[NW], l[NW];
    float o[NW][MAX_DH];
    int last;
    int pages[MAX_SPLIT_PAGES];     // pages of this split
    float part_o[MAX_DH];           // this split's result, read by the cluster's first CTA
    float part_ml[2];
};

// Streaming variant (long splits, many units): keys and values of a split come in blocks of
// 64 positions by bulk copies (cp.async.bulk, whole runs of a page's rows; no multicast) into
// a ring of shared-memory stages, signalled by mbarriers, so that two blocks are in flight
// while the warps score a third; the register-batch variant has at most one batch in flight
// while it scores.  The keys go to the same (warp, lane) in the same order, so both variants
// give the same bits.
constexpr int STREAM_KEYS = 64;     // keys per block
constexpr int STREAM_STAGES = 3;
constexpr uint32_t STREAM_WAIT_LIMIT = 1u << 22;
struct StreamState {
    unsigned long long full[STREAM_STAGES];       // mbarriers: a block has landed
    unsigned long long empty[STREAM_STAGES];      //            all warps have read it
    int bad[STREAM_STAGES];                       // the block names a page outside the pool
    int failed;                                   // a wait gave up
    unsigned char* ring;                          // [stages][K | V][64 keys * head_dim * 2 bytes]
};
__device__ __forceinline__ uint32_t st_smem(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void st_mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void st_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void st_mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool st_mbar_try_wait(uint32_t bar, uint32_t parity) {
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
// Bounded wait; false when it gave up or another thread of the CTA already had.
__device__ __forceinline__ bool st_mbar_wait(uint32_t bar, uint32_t parity, volatile int* failed) {
    for (uint32_t i = 0; i < STREAM_WAIT_LIMIT; ++i) {
        if (st_mbar_try_wait(bar, parity)) return true;
        if ((i & 255u) == 255u && *failed) return false;
    }
    *failed = 1;
    return false;
}
__device__ __forceinline__ void st_bulk_copy(uint32_t dst, const void* src, uint32_t bytes,
                                             uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
        "l"(src), "r"(bytes), "r"(bar)
        : "memory");
}
__device__ __forceinline__ uint4 st_ld_shared_v4(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

// Thread-block cluster helpers (the splits of one (token, head) form a cluster).
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float ld_cluster_f32(const float* local, int rank) {
    const uint32_t laddr = (uint32_t)__cvta_generic_to_shared(local);
    uint32_t raddr;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(raddr) : "r"(laddr), "r"(rank));
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(raddr) : "memory");
    return v;
}

// The cluster's first CTA merges the splits s_first..s_last in split order, reading each
// split's (maximum, sum, weighted values) from that CTA's shared memory; the arithmetic is
// that of the workspace merge.
template <int NW>
__device__ __forceinline__ void merge_cluster(const Args& a, int t, int h, int s_first, int s_last,
                                              Shared<NW>& sh) {
    __nv_bfloat16* o = a.out + (size_t)t * a.out_stride + (size_t)h * a.head_dim;
    float mg = -INFINITY;
    for (int ss = s_first; ss <= s_last; ++ss) mg = fmaxf(mg, ld_cluster_f32(&sh.part_ml[0], ss));
    float lg = 0.0f;
    for (int ss = s_first; ss <= s_last; ++ss) {
        const float ms = ld_cluster_f32(&sh.part_ml[0], ss);
        lg += ld_cluster_f32(&sh.part_ml[1], ss) * ((ms == -INFINITY) ? 0.0f : __expf(ms - mg));
    }
    for (int d = threadIdx.x; d < a.head_dim; d += (NW * 32)) {
        float od = 0.0f;
        for (int ss = s_first; ss <= s_last; ++ss) {
            const float ms = ld_cluster_f32(&sh.part_ml[0], ss);
            od += ld_cluster_f32(&sh.part_o[d], ss) * ((ms == -INFINITY) ? 0.0f : __expf(ms - mg));
        }
        o[d] = __float2bfloat16_rn(lg > 0.0f ? od / lg : 0.0f);
    }
}

// One (token list place idx, head h, split s).  LPK lanes share a key row (head_dim <= 8 *
// LPK); NW warps of the CTA take part; barriers inside are reached by all of them or none.
// UB: keys per thread in a register batch (4: most bytes in flight per thread; 2: fewer
// registers, so more CTAs per SM when there are many units).
// CLUSTER: the launch put the max_splits CTAs of a (token, head) into one thread-block
// cluster (split s = rank s): partial results are exchanged through distributed shared
// memory and merged by the cluster's first CTA instead of going through the workspace and
// a counter.  Every CTA of the cluster then reaches the two cluster barriers, also those
// whose split holds no visible key.
// STREAM: the keys come through the shared-memory ring of `stream` (no window; head_dim up
// to 128).
template <int LPK, int NW, int UB = 4, bool CLUSTER = false, bool STREAM = false>
__device__ __forceinline__ void unit(const Args& a, int idx, int h, int s, Shared<NW>& sh,
                                     StreamState* stream = nullptr) {
    float* sh_m = sh.m;
    float* sh_l = sh.l;
    float (*sh_o)[MAX_DH] = sh.o;
    int* sh_pages = sh.pages;
    int& sh_last = sh.last;
    constexpr int KPW = 32 / LPK;                 // keys per warp per load

    DEC_TRACE(0);
    if (a.token_count != nullptr && idx >= *a.token_count) return;
    const int t = a.token_list ? a.token_list[idx] : idx;
    const int b = a.seq_of_token[t];
    if (b < 0) return;
    const int pos = a.positions[t];
    if (pos < 0 || pos >= a.max_pages * a.page_size) {
        if (threadIdx.x == 0 && s == 0) prb_set_status(a.status, PRB_S_POSITION_RANGE, t, pos, 0);
        return;
    }
    const int lo = (a.window > 0 && pos - a.window + 1 > 0) ? pos - a.window + 1 : 0;
    const int s_first = lo / a.split, s_last = pos / a.split;
    if (s_last >= a.max_splits) {                   // the launch does not cover this context
        if (threadIdx.x == 0 && s == 0) prb_set_status(a.status, PRB_S_POSITION_RANGE, t, pos, a.max_splits);
        return;
    }
    const int n_splits = s_last - s_first + 1;
    if (s < s_first || s > s_last) {
        if constexpr (CLUSTER) {
            if (n_splits > 1) {
                cluster_sync_all();                  // the partial results are in place
                if (s == 0) {                        // (a window has moved past split 0)
                    merge_cluster<NW>(a, t, h, s_first, s_last, sh);
                }
                cluster_sync_all();                  // they have been read
            }
        }
        return;
    }
    const int k_begin = max(lo, s * a.split), k_end = min(pos + 1, (s + 1) * a.split);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane % LPK;                   // which 16-byte piece of the row
    const int kslot = lane / LPK;                 // which key of the warp's load
    const int hk = h / (a.n_heads / a.kv_heads);
    const int* table = a.block_table + (size_t)b * a.max_pages;
    const bool piece_ok = sub * 8 < a.head_dim;

    // this lane's 8 query dims; scores are (q . k) * scale as in the formula
    float qf[8];
    {
        const __nv_bfloat16* qp = a.q + (size_t)t * a.q_stride + (size_t)h * a.head_dim + sub * 8;
#pragma unroll
        for (int i = 0; i < 8; ++i) qf[i] = piece_ok ? __bfloat162float(qp[i]) : 0.0f;
    }
    float m = -INFINITY, l = 0.0f;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.0f;

    // page ids of this split, once
    const int first_page = (s * a.split) / a.page_size;
    for (int i = threadIdx.x; i < a.split / a.page_size; i += (NW * 32))
        sh_pages[i] = (first_page + i < a.max_pages) ? table[first_page + i] : -1;
    if constexpr (STREAM) {
        if (threadIdx.x == 0) {
            for (int i = 0; i < STREAM_STAGES; ++i) {
                st_mbar_init(st_smem(&stream->full[i]), 1);
                st_mbar_init(st_smem(&stream->empty[i]), NW);
            }
            stream->failed = 0;
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        }
    }
    __syncthreads();
    DEC_TRACE(1);

    // Keys k_begin + warp*KPW + kslot, stepping NW*KPW, in batches of UB per thread.  Two
    // batches of registers take turns: the loads of the next batch are issued before the
    // current one is scored, so some are always in flight.
    constexpr int BATCH = NW * KPW * UB;
    struct Batch {
        uint4 k[UB], v[UB];
        bool ok[UB];
    };
    auto load = [&](int base, Batch& bt) {
#pragma unroll
        for (int u = 0; u < UB; ++u) {
            const int j = base + u * NW * KPW + kslot;
            bt.ok[u] = false;
            bt.k[u] = make_uint4(0, 0, 0, 0);
            bt.v[u] = make_uint4(0, 0, 0, 0);
            if (j < k_end) {
                const int page = sh_pages[j / a.page_size - first_page];
                if (page < 0 || page >= a.num_pages) {
                    prb_set_status(a.status, PRB_S_PAGE_RANGE, t, j, page);
                } else {
                    bt.ok[u] = true;
                    if (piece_ok) {
                        const size_t row =
                            (((size_t)page * a.kv_heads + hk) * a.page_size + (j % a.page_size)) *
                                a.head_dim + sub * 8;
                        bt.k[u] = *reinterpret_cast<const uint4*>(a.k_pages + row);
                        bt.v[u] = *reinterpret_cast<const uint4*>(a.v_pages + row);
                    }
                }
            }
        }
    };
    auto score_key = [&](const uint4& kk, const uint4& vv, bool ok) {
        {
            float part = dot8(kk, qf);
            // every lane takes part in the reduction over the LPK pieces of a key row
#pragma unroll
            for (int o = LPK / 2; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
            const float sc = ok ? part * a.scale : -INFINITY;
            // online softmax per key slot (each group of LPK lanes has its own running state)
            const float m_new = fmaxf(m, sc);
            if (m_new > -INFINITY) {
                const float corr = (m == -INFINITY) ? 0.0f : __expf(m - m_new);
                const float p = (sc == -INFINITY) ? 0.0f : __expf(sc - m_new);
                l = l * corr + p;
                const __nv_bfloat162* vp = reinterpret_cast<const __nv_bfloat162*>(&vv);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 f = __bfloat1622float2(vp[i]);
                    acc[2 * i] = fmaf(p, f.x, acc[2 * i] * corr);
                    acc[2 * i + 1] = fmaf(p, f.y, acc[2 * i + 1] * corr);
                }
                m = m_new;
            }
        }
    };
    auto score = [&](const Batch& bt) {
#pragma unroll
        for (int u = 0; u < UB; ++u) score_key(bt.k[u], bt.v[u], bt.ok[u]);
    };
    if constexpr (STREAM) {
        const int row_bytes = a.head_dim * 2;
        const uint32_t ring = st_smem(stream->ring);
        const uint32_t stage_bytes = 2u * STREAM_KEYS * row_bytes;
        const int n_blk = (k_end - k_begin + STREAM_KEYS - 1) / STREAM_KEYS;
        volatile int* failed = &stream->failed;
        // thread 0: the copies of block `blk` (its stage is free)
        auto issue = [&](int blk) {
            const int st = blk % STREAM_STAGES;
            const int j0 = k_begin + blk * STREAM_KEYS;
            const int cnt = min(STREAM_KEYS, k_end - j0);
            const uint32_t fb = st_smem(&stream->full[st]);
            bool bad = false;
            for (int j = j0; j < j0 + cnt; j += a.page_size - j % a.page_size) {
                const int page = sh_pages[j / a.page_size - first_page];
                if (page < 0 || page >= a.num_pages) {
                    prb_set_status(a.status, PRB_S_PAGE_RANGE, t, j, page);
                    bad = true;
                }
            }
            stream->bad[st] = bad ? 1 : 0;
            if (bad) {                             // nothing is copied; the block counts as masked
                st_mbar_arrive(fb);
                return;
            }
            st_mbar_expect_tx(fb, 2u * cnt * row_bytes);
            const uint32_t kd = ring + st * stage_bytes, vd = kd + STREAM_KEYS * row_bytes;
            for (int j = j0; j < j0 + cnt;) {
                const int off = j % a.page_size;
                const int n = min(a.page_size - off, j0 + cnt - j);
                const int page = sh_pages[j / a.page_size - first_page];
                const size_t row = (((size_t)page * a.kv_heads + hk) * a.page_size + off) * a.head_dim;
                st_bulk_copy(kd + (j - j0) * row_bytes, a.k_pages + row, n * row_bytes, fb);
                st_bulk_copy(vd + (j - j0) * row_bytes, a.v_pages + row, n * row_bytes, fb);
                j += n;
            }
        };
        int issued = 0;
        if (threadIdx.x == 0)
            for (; issued < STREAM_STAGES && issued < n_blk; ++issued) issue(issued);
        bool ok = true;
        int blk = 0;
        for (; blk < n_blk && ok; ++blk) {
            const int st = blk % STREAM_STAGES;
            // the stage of the block before is free once all warps have passed it: refill it
            if (threadIdx.x == 0 && blk >= 1 && issued < n_blk) {
                const int prev = (blk - 1) % STREAM_STAGES;
                if (st_mbar_wait(st_smem(&stream->empty[prev]), ((blk - 1) / STREAM_STAGES) & 1, failed)) {
                    issue(issued);
                    ++issued;
                }
            }
            ok = st_mbar_wait(st_smem(&stream->full[st]), (blk / STREAM_STAGES) & 1, failed);
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok) break;
            const bool bad = stream->bad[st] != 0;
            const int j0 = k_begin + blk * STREAM_KEYS;
            const uint32_t kd = ring + st * stage_bytes, vd = kd + STREAM_KEYS * row_bytes;
#pragma unroll
            for (int u = 0; u < STREAM_KEYS / (NW * KPW); ++u) {
                const int jj = u * NW * KPW + warp * KPW + kslot;      // key within the block
                const bool key_ok = j0 + jj < k_end && !bad;
                uint4 kk = make_uint4(0, 0, 0, 0), vv = make_uint4(0, 0, 0, 0);
                if (key_ok && piece_ok) {
                    kk = st_ld_shared_v4(kd + jj * row_bytes + sub * 16);
                    vv = st_ld_shared_v4(vd + jj * row_bytes + sub * 16);
                }
                score_key(kk, vv, key_ok);
            }
            if (blk == 0 && m != 1234.5f) { DEC_TRACE(2); }
            __syncwarp();
            if (lane == 0) st_mbar_arrive(st_smem(&stream->empty[st]));
        }
        if (!ok && lane == 0) prb_set_status(a.status, PRB_S_WAIT_TIMEOUT, 31, idx, blk);
        __syncthreads();
        if (threadIdx.x == 0 && *failed) {
            // wait (bounded) for the copies still in flight before the CTA may leave
            for (int b2 = blk; b2 < issued; ++b2) {
                const uint32_t fb = st_smem(&stream->full[b2 % STREAM_STAGES]);
                for (uint32_t i = 0; i < STREAM_WAIT_LIMIT; ++i)
                    if (st_mbar_try_wait(fb, (b2 / STREAM_STAGES) & 1)) break;
            }
        }
    } else {
        Batch b0, b1;
        int base = k_begin + warp * KPW;           // the same for the whole warp
        load(base, b0);
        load(base + BATCH, b1);                    // keys beyond the split are not fetched
        bool first_batch = true;
        while (base < k_end) {
            score(b0);
            if (first_batch && m != 1234.5f) { DEC_TRACE(2); first_batch = false; }
            base += BATCH;
            if (base >= k_end) break;
            load(base + BATCH, b0);
            score(b1);
            base += BATCH;
            if (base >= k_end) break;
            load(base + BATCH, b1);
        }
    }
    if (m != 1234.5f) { DEC_TRACE(3); }
    // merge the KPW key slots of the warp (fixed butterfly order)
#pragma unroll
    for (int o = LPK; o < 32; o <<= 1) {
        const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
        const float l2 = __shfl_xor_sync(0xffffffffu, l, o);
        const float mn = fmaxf(m, m2);
        const float c1 = (m == -INFINITY) ? 0.0f : __expf(m - mn);
        const float c2 = (m2 == -INFINITY) ? 0.0f : __expf(m2 - mn);
        l = l * c1 + l2 * c2;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float a2 = __shfl_xor_sync(0xffffffffu, acc[i], o);
            acc[i] = acc[i] * c1 + a2 * c2;
        }
        m = mn;
    }
    if (kslot == 0 && piece_ok) {
#pragma unroll
        for (int i = 0; i < 8; ++i) sh_o[warp][sub * 8 + i] = acc[i];
    }
    if (lane == 0) { sh_m[warp] = m; sh_l[warp] = l; }
    __syncthreads();

    // merge warps in order 0..3; thread d owns output dimension d (and d + 128)
    float mt = -INFINITY;
#pragma unroll
    for (int w = 0; w < NW; ++w) mt = fmaxf(mt, sh_m[w]);
    float lt = 0.0f;
    float cw[NW];
#pragma unroll
    for (int w = 0; w < NW; ++w) {
        cw[w] = (sh_m[w] == -INFINITY) ? 0.0f : __expf(sh_m[w] - mt);
        lt += sh_l[w] * cw[w];
    }
    const size_t pair = (size_t)idx * a.n_heads + h;       // scratch is indexed by list place
    float* ws = a.workspace + (pair * a.max_splits + s) * (size_t)(a.head_dim + 4);
    __nv_bfloat16* o = a.out + (size_t)t * a.out_stride + (size_t)h * a.head_dim;
    for (int d = threadIdx.x; d < a.head_dim; d += (NW * 32)) {
        float od = 0.0f;
#pragma unroll
        for (int w = 0; w < NW; ++w) od += sh_o[w][d] * cw[w];
        if (n_splits == 1) o[d] = __float2bfloat16_rn(lt > 0.0f ? od / lt : 0.0f);
        else if constexpr (CLUSTER) sh.part_o[d] = od;
        else ws[d] = od;
    }
    if constexpr (CLUSTER) {
        if (threadIdx.x == 0) { sh.part_ml[0] = mt; sh.part_ml[1] = lt; }
    }
    DEC_TRACE(4);
    if (n_splits == 1) return;
    if constexpr (CLUSTER) {
        cluster_sync_all();                          // every split's partial result is in place
        if (s == 0) merge_cluster<NW>(a, t, h, s_first, s_last, sh);
        cluster_sync_all();                          // they have been read: CTAs may leave
        return;
    }
    if (threadIdx.x == 0) { ws[a.head_dim] = mt; ws[a.head_dim + 1] = lt; }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int done = atomicAdd(&a.counters[pair], 1);
        sh_last = (done == n_splits - 1) ? 1 : 0;
    }
    __syncthreads();
    DEC_TRACE(5);
    if (!sh_last) return;
    __threadfence();
    // last CTA of this (token, head): merge the splits in order
    const float* wbase = a.workspace + pair * a.max_splits * (size_t)(a.head_dim + 4);
    constexpr int FAST = 8;                       // splits merged from registers
    if (n_splits <= FAST && a.head_dim <= NW * 32) {
        // everything a thread needs is fetched at once (one round trip to the L2), then
        // combined in split order exactly as in the general loop below
        const int d = threadIdx.x;
        float ms[FAST], ls[FAST], os[FAST];
#pragma unroll
        for (int j = 0; j < FAST; ++j) {
            const bool on = j < n_splits;
            const float* w = wbase + (size_t)(s_first + (on ? j : 0)) * (a.head_dim + 4);
            ms[j] = __ldcg(w + a.head_dim);
            ls[j] = __ldcg(w + a.head_dim + 1);
            os[j] = __ldcg(w + (d < a.head_dim ? d : 0));
            if (!on) ms[j] = -INFINITY;
        }
        float mg = -INFINITY;
#pragma unroll
        for (int j = 0; j < FAST; ++j) mg = fmaxf(mg, ms[j]);
        float lg = 0.0f, od = 0.0f;
#pragma unroll
        for (int j = 0; j < FAST; ++j) {
            if (j < n_splits) {
                const float c = (ms[j] == -INFINITY) ? 0.0f : __expf(ms[j] - mg);
                lg += ls[j] * c;
                od += os[j] * c;
            }
        }
        if (d < a.head_dim) o[d] = __float2bfloat16_rn(lg > 0.0f ? od / lg : 0.0f);
    } else {
        float mg = -INFINITY;
        for (int ss = s_first; ss <= s_last; ++ss)
            mg = fmaxf(mg, __ldcg(wbase + (size_t)ss * (a.head_dim + 4) + a.head_dim));
        float lg = 0.0f;
        for (int ss = s_first; ss <= s_last; ++ss) {
            const float* w = wbase + (size_t)ss * (a.head_dim + 4);
            const float ms = __ldcg(w + a.head_dim);
            lg += __ldcg(w + a.head_dim + 1) * ((ms == -INFINITY) ? 0.0f : __expf(ms - mg));
        }
        for (int d = threadIdx.x; d < a.head_dim; d += (NW * 32)) {
            float od = 0.0f;
            for (int ss = s_first; ss <= s_last; ++ss) {
                const float* w = wbase + (size_t)ss * (a.head_dim + 4);
                const float ms = __ldcg(w + a.head_dim);
                od += __ldcg(w + d) * ((ms == -INFINITY) ? 0.0f : __expf(ms - mg));
            }
            o[d] = __float2bfloat16_rn(lg > 0.0f ? od / lg : 0.0f);
        }
    }
    if (threadIdx.x == 0) a.counters[pair] = 0;
    DEC_TRACE(6);
}
}  // namespace decode_attn
