// Decode attention over the paged bfloat16 cache: one query row per (token, head), keys
// split into fixed ranges of absolute positions so that a single token still fills the
// GPU, partial results merged in split order.
//
// The unit of work is one (token, head, split) and is done by ONE WARP, with no shared
// memory and no block-wide barrier: warps of a CTA work on different units at the same
// time, which is what hides the latency of these short dependent chains.  Split s owns
// positions [s*SPLIT, (s+1)*SPLIT), so what a split sums and
// in which order depends only on the token's own visible range [lo, pos], never on the
// batch.  LPK lanes share a key row (16 bytes each), so a warp reads 32/LPK keys per load;
// eight loads of keys and of values are in flight before the first is used.  Each group
// of LPK lanes keeps a running maximum and sum (online softmax, float32) and weighted
// values; the groups are merged by a butterfly, splits through a float32 workspace: the
// last warp of a (token, head) to finish merges all of its splits in order s =
// first..last (a counter in scratch memory tells which warp is last, and is reset by
// it).  Softmax statistics and all sums are float32.
//
// Scratch: workspace [list places, heads, max_splits, head_dim + 4] float32 (a split's
// values, then its maximum and sum; the pitch keeps 16-byte alignment) and counters
// [list places * heads] int32 (zero before the first launch; left zero).
//
// The unit is a device function so that the stand-alone kernel (attention_decode.cu) and
// the whole-step decode program (decode_program.cu) run the very same code.
#pragma once
#include "common.cuh"

namespace decode_attn {
constexpr int SPLIT = 32;           // keys per split: one round of loads per warp
constexpr int MAX_DH = 256;
constexpr int UNROLL = 8;           // loads in flight per lane (keys and values each)

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

// One (token-list place idx, head h, split s), run by one whole warp.  LPK lanes share a
// key row (head_dim <= 8 * LPK).
template <int LPK>
__device__ __forceinline__ void warp_unit(const Args& a, int idx, int h, int s) {
    constexpr int KPW = 32 / LPK;                 // keys per warp per load
    constexpr unsigned FULL = 0xffffffffu;
    if (a.token_count != nullptr && idx >= *a.token_count) return;
    const int t = a.token_list ? a.token_list[idx] : idx;
    const int b = a.seq_of_token[t];
    if (b < 0) return;
    const int pos = a.positions[t];
    const int lane = threadIdx.x & 31;
    if (pos < 0 || pos >= a.max_pages * a.page_size) {
        if (lane == 0 && s == 0) prb_set_status(a.status, PRB_S_POSITION_RANGE, t, pos, 0);
        return;
    }
    const int lo = (a.window > 0 && pos - a.window + 1 > 0) ? pos - a.window + 1 : 0;
    const int s_first = lo / SPLIT, s_last = pos / SPLIT;
    if (s_last >= a.max_splits) {                   // the launch does not cover this context
        if (lane == 0 && s == 0) prb_set_status(a.status, PRB_S_POSITION_RANGE, t, pos, a.max_splits);
        return;
    }
    if (s < s_first || s > s_last) return;
    const int n_splits = s_last - s_first + 1;
    const int k_begin = max(lo, s * SPLIT), k_end = min(pos + 1, (s + 1) * SPLIT);

    const int sub = lane % LPK;                   // which 16-byte piece of the row
    const int kslot = lane / LPK;                 // which key of the warp's load
    const int hk = h / (a.n_heads / a.kv_heads);
    const bool piece_ok = sub * 8 < a.head_dim;

    // page ids of this split: lane i holds the i-th page the split touches (page_size >= 8,
    // so at most SPLIT / 8 + 1 pages)
    const int first_page = (s * SPLIT) / a.page_size;
    const int pages_in_split = (s * SPLIT + SPLIT - 1) / a.page_size - first_page + 1;
    int my_page = -1;
    if (lane < pages_in_split && first_page + lane < a.max_pages)
        my_page = a.block_table[(size_t)b * a.max_pages + first_page + lane];

    // this lane's 8 query dims; scores are (q . k) * scale as in the formula
    float qf[8];
    {
        const __nv_bfloat16* qp = a.q + (size_t)t * a.q_stride + (size_t)h * a.head_dim + sub * 8;
        uint4 raw = make_uint4(0, 0, 0, 0);
        if (piece_ok) raw = *reinterpret_cast<const uint4*>(qp);
        const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(p2[i]);
            qf[2 * i] = f.x;
            qf[2 * i + 1] = f.y;
        }
    }
    float m = -INFINITY, l = 0.0f;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.0f;

    for (int base = k_begin; base < k_end; base += KPW * UNROLL) {      // warp-uniform
        uint4 kraw[UNROLL], vraw[UNROLL];
        bool ok[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int j = base + u * KPW + kslot;
            const int jj = j < k_end ? j : k_end - 1;
            // every lane takes part in the shuffle, also those whose key is out of range
            const int page = __shfl_sync(FULL, my_page, jj / a.page_size - first_page);
            ok[u] = false;
            kraw[u] = make_uint4(0, 0, 0, 0);
            vraw[u] = make_uint4(0, 0, 0, 0);
            if (j < k_end) {
                if (page < 0 || page >= a.num_pages) {
                    prb_set_status(a.status, PRB_S_PAGE_RANGE, t, j, page);
                } else {
                    ok[u] = true;
                    if (piece_ok) {
                        const size_t row =
                            (((size_t)page * a.kv_heads + hk) * a.page_size + (j % a.page_size)) *
                                a.head_dim + sub * 8;
                        kraw[u] = *reinterpret_cast<const uint4*>(a.k_pages + row);
                        vraw[u] = *reinterpret_cast<const uint4*>(a.v_pages + row);
                    }
                }
            }
        }
        // scores of the UNROLL keys of this lane group, then one softmax update for all
        float sc[UNROLL];
        float m_new = m;
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            float part = dot8(kraw[u], qf);
#pragma unroll
            for (int o = LPK / 2; o > 0; o >>= 1) part += __shfl_xor_sync(FULL, part, o);
            sc[u] = ok[u] ? part * a.scale : -INFINITY;
            m_new = fmaxf(m_new, sc[u]);
        }
        if (m_new > -INFINITY) {
            const float corr = (m == -INFINITY) ? 0.0f : __expf(m - m_new);
            l *= corr;
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] *= corr;
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                const float p = (sc[u] == -INFINITY) ? 0.0f : __expf(sc[u] - m_new);
                l += p;
                const __nv_bfloat162* vp = reinterpret_cast<const __nv_bfloat162*>(&vraw[u]);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 f = __bfloat1622float2(vp[i]);
                    acc[2 * i] = fmaf(p, f.x, acc[2 * i]);
                    acc[2 * i + 1] = fmaf(p, f.y, acc[2 * i + 1]);
                }
            }
            m = m_new;
        }
    }
    // merge the KPW key slots of the warp (fixed butterfly order); afterwards every lane
    // holds the split's result for its 8 dimensions
#pragma unroll
    for (int o = LPK; o < 32; o <<= 1) {
        const float m2 = __shfl_xor_sync(FULL, m, o);
        const float l2 = __shfl_xor_sync(FULL, l, o);
        const float mn = fmaxf(m, m2);
        const float c1 = (m == -INFINITY) ? 0.0f : __expf(m - mn);
        const float c2 = (m2 == -INFINITY) ? 0.0f : __expf(m2 - mn);
        l = l * c1 + l2 * c2;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float a2 = __shfl_xor_sync(FULL, acc[i], o);
            acc[i] = acc[i] * c1 + a2 * c2;
        }
        m = mn;
    }
    __nv_bfloat16* o = a.out + (size_t)t * a.out_stride + (size_t)h * a.head_dim;
    if (n_splits == 1) {
        if (kslot == 0 && piece_ok) {
            const float inv = l > 0.0f ? 1.0f / l : 0.0f;
            uint4 pk;
            __nv_bfloat162 p0 = __floats2bfloat162_rn(acc[0] * inv, acc[1] * inv);
            __nv_bfloat162 p1 = __floats2bfloat162_rn(acc[2] * inv, acc[3] * inv);
            __nv_bfloat162 p2 = __floats2bfloat162_rn(acc[4] * inv, acc[5] * inv);
            __nv_bfloat162 p3 = __floats2bfloat162_rn(acc[6] * inv, acc[7] * inv);
            pk.x = *reinterpret_cast<uint32_t*>(&p0);
            pk.y = *reinterpret_cast<uint32_t*>(&p1);
            pk.z = *reinterpret_cast<uint32_t*>(&p2);
            pk.w = *reinterpret_cast<uint32_t*>(&p3);
            *reinterpret_cast<uint4*>(o + sub * 8) = pk;
        }
        return;
    }
    // several splits: park this one in the workspace, the last warp to arrive merges them
    const size_t pair = (size_t)idx * a.n_heads + h;       // scratch is indexed by list place
    const size_t stride = (size_t)(a.head_dim + 4);      // keeps every split 16-byte aligned
    float* ws = a.workspace + (pair * a.max_splits + s) * stride;
    if (kslot == 0 && piece_ok) {
        *reinterpret_cast<float4*>(ws + sub * 8) = make_float4(acc[0], acc[1], acc[2], acc[3]);
        *reinterpret_cast<float4*>(ws + sub * 8 + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
    }
    if (lane == 0) {
        ws[a.head_dim] = m;
        ws[a.head_dim + 1] = l;
    }
    __threadfence();
    __syncwarp();
    int last = 0;
    if (lane == 0) last = (atomicAdd(&a.counters[pair], 1) == n_splits - 1) ? 1 : 0;
    last = __shfl_sync(FULL, last, 0);
    if (!last) return;
    __threadfence();
    // Merge: rounds of up to 32 splits, one split per lane for the statistics, then every
    // lane sums its dimensions over the round's splits (weights passed by shuffle).
    const float* wbase = a.workspace + pair * a.max_splits * stride;
    float mg = -INFINITY, lg = 0.0f;
    float od[MAX_DH / 32];
#pragma unroll
    for (int i = 0; i < MAX_DH / 32; ++i) od[i] = 0.0f;
    for (int r0 = s_first; r0 <= s_last; r0 += 32) {
        const int ss = r0 + lane;
        const bool have = ss <= s_last;
        const float* w = wbase + (size_t)(have ? ss : s_last) * stride;
        const float ms = have ? __ldcg(w + a.head_dim) : -INFINITY;
        const float ls = have ? __ldcg(w + a.head_dim + 1) : 0.0f;
        float mr = ms;
#pragma unroll
        for (int o2 = 16; o2 > 0; o2 >>= 1) mr = fmaxf(mr, __shfl_xor_sync(FULL, mr, o2));
        const float mn = fmaxf(mg, mr);
        const float keep = (mg == -INFINITY) ? 0.0f : __expf(mg - mn);
        const float cs = (ms == -INFINITY) ? 0.0f : __expf(ms - mn);     // this lane's split
        float lsum = ls * cs;
#pragma unroll
        for (int o2 = 16; o2 > 0; o2 >>= 1) lsum += __shfl_xor_sync(FULL, lsum, o2);
        lg = lg * keep + lsum;
        const int in_round = min(32, s_last - r0 + 1);
#pragma unroll
        for (int i = 0; i < MAX_DH / 32; ++i) {
            const int d = lane + 32 * i;
            float sum = od[i] * keep;
            const bool mine = d < a.head_dim;        // the shuffles below are done by every lane
#pragma unroll 8
            for (int j = 0; j < in_round; ++j) {
                const float cj = __shfl_sync(FULL, cs, j);
                const float wv = mine ? __ldcg(wbase + (size_t)(r0 + j) * stride + d) : 0.0f;
                sum = fmaf(cj, wv, sum);
            }
            od[i] = sum;
        }
        mg = mn;
    }
    const float inv = lg > 0.0f ? 1.0f / lg : 0.0f;
#pragma unroll
    for (int i = 0; i < MAX_DH / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < a.head_dim) o[d] = __float2bfloat16_rn(od[i] * inv);
    }
    if (lane == 0) a.counters[pair] = 0;
}

// Units of a launch are numbered (place * n_heads + head) * max_splits + split.
template <int LPK>
__device__ __forceinline__ void warp_unit_flat(const Args& a, int unit) {
    const int per_place = a.n_heads * a.max_splits;
    const int idx = unit / per_place, rem = unit - idx * per_place;
    const int h = rem / a.max_splits, s = rem - h * a.max_splits;
    warp_unit<LPK>(a, idx, h, s);
}
}  // namespace decode_attn
