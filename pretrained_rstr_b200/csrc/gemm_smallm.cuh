// Decode-time matrix product: few rows (M <= 64 tokens), bandwidth bound.
//
//     C[M,N] = act(X[M,K] . W[N,K]^T + bias[N]) (+ resid[M,N])
//     with X = A (bfloat16), or X = LayerNorm(R) rounded to bfloat16 (R float32 [M,K]),
//     the norm fused into the product's prologue.
//
// The weights are streamed once from HBM straight into tensor-core operand registers:
// with the roles swapped (C^T = W . X^T) a 16-row strip of W is the A operand of
// mma.sync.m16n8k16 and the tokens are the N dimension.  A thread loads 16 contiguous
// bytes of a W row per step; the k index inside an MMA is only a summation index, so the
// 8 elements of a load are spread over two MMAs in the order they arrive and the X
// fragments are read with the same permutation -- no shared-memory staging of W, no
// transposition.  One CTA owns 16 output features for all tokens; its 8 warps split K
// (steps of 32, round robin) and their partial sums are added in warp order through
// shared memory, so a result does not depend on the batch.  X comes from shared memory
// (after the fused LayerNorm) or from global memory (L2) directly.
// float32: statistics of the norm, accumulation, bias, activation, residual.
//
// The pieces the kernels of gemm_bf16_smallm.cu are made of.
#pragma once
#include "common.cuh"

namespace smallm {
constexpr int THREADS = 256;
constexpr int WARPS = 8;
constexpr int ROWS = 16;            // output features per strip
constexpr int KSTEP = 32;
constexpr int LN_MAX_K = 2048;      // fused norm keeps a row in registers: 16 float4 per lane
constexpr int PF = 4;               // k-steps of weights in flight per warp

struct Args {
    void* out;
    const __nv_bfloat16* x;         // bfloat16 [M,K], or null when xf is given
    const float* xf;                // float32 rows to be normalised first, or null
    const int* xf_rows;             // which row of xf output row t is made of (null: row t)
    int xf_rows_in;                 // rows xf holds (the gathered indices are checked against it)
    const float* gamma;
    const float* beta;
    float eps;
    const __nv_bfloat16* w;         // [N,K]
    const float* bias;
    const float* resid;
    int m, n, k;
    long ldx, ldw, ldc;
    int act;
    int xs_pitch;                   // row pitch (elements) of the normalised rows in shared memory
    // Optional scatter of output columns into the paged cache (a fused QKV product: columns
    // [q_width, q_width + kv_width) are keys, the next kv_width are values).  kv_width == 0: off.
    void* k_pages;                  // [pages][kv heads][page_size][head_dim], element type of out
    void* v_pages;
    const int* slots;               // cache slot of each token, -1 = none
    int q_width, kv_width, head_dim, page_size, num_pages;
    int* status;
};

struct Prefetch {
    uint4 wa[PF], wb[PF];
};

// The float32 row that output row t is normalised from; null (and recorded in the status
// word) when a gathered index lies outside xf.  The same answer in every lane of a warp.
__device__ __forceinline__ const float* norm_source(const Args& a, int t) {
    if (a.xf_rows == nullptr) return a.xf + (size_t)t * a.ldx;
    const int src = a.xf_rows[t];
    if (src < 0 || src >= a.xf_rows_in) {
        if ((threadIdx.x & 31) == 0) prb_set_status(a.status, PRB_S_ROW_RANGE, t, src, a.xf_rows_in);
        return nullptr;
    }
    return a.xf + (size_t)src * a.ldx;
}

// row pitch of the normalised activations: words per row = 16 mod 32 (conflict-free reads)
__host__ __device__ inline int norm_pitch(int k) {
    const int words = k / 2;
    return k + 2 * ((16 - (words % 32) + 32) % 32);
}
__host__ __device__ inline size_t smem_bytes(int mt, bool ln, int k) {
    return (size_t)WARPS * ROWS * 8 * mt * sizeof(float) + (ln ? (size_t)8 * mt * norm_pitch(k) * 2 : 0);
}

// LayerNorm of R float32 rows of k elements into bfloat16, by one warp: the rows' loads are
// all requested before the first sum, so that two rows cost one round trip to the L2, not
// two (a CTA of eight warps norms sixteen rows in the time of eight).  A row is held in NV
// float4 per lane; the caller picks the smallest instance that holds it, so that a short row
// does not issue the (predicated-off) instructions of a long one.  Mean first, then the
// centred squares from the registers, both float32 and both summed in a fixed order: a row's
// result does not depend on R.
// gb: gamma [k] then beta [k] (if has_beta), anywhere (shared memory in both callers).
template <int NV, int R>
__device__ __forceinline__ void norm_rows_of_warp(const float* const (&xrow)[R],
                                                  __nv_bfloat16* const (&dst)[R], const float* gb,
                                                  int k, bool has_beta, float eps) {
    const int lane = threadIdx.x & 31;
    const int nvec = k / 4;
    float4 v[R][NV];
    float s[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const float4* src = reinterpret_cast<const float4*>(xrow[r]);
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int idx = lane + 32 * i;
            v[r][i] = idx < nvec ? __ldcg(src + idx) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    float mean[R], inv[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        s[r] = 0.0f;
#pragma unroll
        for (int i = 0; i < NV; ++i) s[r] += (v[r][i].x + v[r][i].y) + (v[r][i].z + v[r][i].w);
        mean[r] = prb_warp_sum(s[r]) / (float)k;
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        float sq = 0.0f;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            if (lane + 32 * i < nvec) {
                const float c0 = v[r][i].x - mean[r], c1 = v[r][i].y - mean[r],
                            c2 = v[r][i].z - mean[r], c3 = v[r][i].w - mean[r];
                sq += (c0 * c0 + c1 * c1) + (c2 * c2 + c3 * c3);
            }
        }
        inv[r] = 1.0f / sqrtf(prb_warp_sum(sq) / (float)k + eps);
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int idx = lane + 32 * i;
        if (idx < nvec) {
            const float4 gm = reinterpret_cast<const float4*>(gb)[idx];
            float4 bt = make_float4(0.f, 0.f, 0.f, 0.f);
            if (has_beta) bt = reinterpret_cast<const float4*>(gb + k)[idx];
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const __nv_bfloat162 lo =
                    __floats2bfloat162_rn((v[r][i].x - mean[r]) * inv[r] * gm.x + bt.x,
                                          (v[r][i].y - mean[r]) * inv[r] * gm.y + bt.y);
                const __nv_bfloat162 hi =
                    __floats2bfloat162_rn((v[r][i].z - mean[r]) * inv[r] * gm.z + bt.z,
                                          (v[r][i].w - mean[r]) * inv[r] * gm.w + bt.w);
                uint2 pk;
                pk.x = *reinterpret_cast<const uint32_t*>(&lo);
                pk.y = *reinterpret_cast<const uint32_t*>(&hi);
                *reinterpret_cast<uint2*>(dst[r] + idx * 4) = pk;
            }
        }
    }
}

// The instance for rows of k elements (k a multiple of 4, at most LN_MAX_K).  Two long rows
// together would not fit a lane's registers: they go one after the other.
template <int R>
__device__ __forceinline__ void norm_rows_any(const float* const (&xrow)[R],
                                              __nv_bfloat16* const (&dst)[R], const float* gb, int k,
                                              bool has_beta, float eps) {
    const int iters = (k / 4 + 31) / 32;
    if (iters <= 2) norm_rows_of_warp<2, R>(xrow, dst, gb, k, has_beta, eps);
    else if (iters <= 6) norm_rows_of_warp<6, R>(xrow, dst, gb, k, has_beta, eps);
    else if (iters <= 8) norm_rows_of_warp<8, R>(xrow, dst, gb, k, has_beta, eps);
    else {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const float* const one_x[1] = {xrow[r]};
            __nv_bfloat16* const one_d[1] = {dst[r]};
            norm_rows_of_warp<LN_MAX_K / 128, 1>(one_x, one_d, gb, k, has_beta, eps);
        }
    }
}
__device__ __forceinline__ void norm_row_any(const float* xrow, __nv_bfloat16* dst, const float* gb,
                                             int k, bool has_beta, float eps) {
    const float* const one_x[1] = {xrow};
    __nv_bfloat16* const one_d[1] = {dst};
    norm_rows_any<1>(one_x, one_d, gb, k, has_beta, eps);
}

__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 v;      // weights are read once: do not keep them in L1
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// Issue this warp's first PF weight loads of `strip` (they depend on nothing but the
// weights, so they may be issued before a wait on the previous kernel or phase).
__device__ __forceinline__ void prefetch(const Args& a, int strip, Prefetch& pf) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, q = lane & 3;
    const int r0 = strip * ROWS + g, r1 = r0 + 8;
    const bool row0_ok = r0 < a.n, row1_ok = r1 < a.n;
    const __nv_bfloat16* w0 = a.w + (size_t)(row0_ok ? r0 : 0) * a.ldw;
    const __nv_bfloat16* w1 = a.w + (size_t)(row1_ok ? r1 : 0) * a.ldw;
#pragma unroll
    for (int p = 0; p < PF; ++p) {
        const int kk = (warp + p * WARPS) * KSTEP + q * 8;
        const bool ok = kk < a.k;
        pf.wa[p] = (ok && row0_ok) ? ldg_stream(w0 + kk) : make_uint4(0, 0, 0, 0);
        pf.wb[p] = (ok && row1_ok) ? ldg_stream(w1 + kk) : make_uint4(0, 0, 0, 0);
    }
}

// LayerNorm of the M rows of xf into shared memory as bfloat16 (rows beyond M are zero).
// All threads of the CTA take part; ends with a barrier.
template <int MT>
__device__ __forceinline__ void norm_rows(const Args& a, __nv_bfloat16* xs) {
    constexpr int MP = 8 * MT;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k = a.k, nvec = a.k / 4;            // float4 per row
    for (int t = warp; t < MP; t += WARPS) {
        __nv_bfloat16* dst = xs + (size_t)t * a.xs_pitch;
        const float* xrow = t < a.m ? norm_source(a, t) : nullptr;
        if (xrow == nullptr) {
            for (int i = lane; i < k / 2; i += 32) reinterpret_cast<uint32_t*>(dst)[i] = 0u;
            continue;
        }
        const float4* src = reinterpret_cast<const float4*>(xrow);
        float4 v[LN_MAX_K / 128];
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < LN_MAX_K / 128; ++i) {
            const int idx = lane + 32 * i;
            v[i] = idx < nvec ? src[idx] : make_float4(0.f, 0.f, 0.f, 0.f);
            s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
        }
        const float mean = prb_warp_sum(s) / (float)k;
        float sq = 0.0f;
#pragma unroll
        for (int i = 0; i < LN_MAX_K / 128; ++i) {
            if (lane + 32 * i < nvec) {
                const float c0 = v[i].x - mean, c1 = v[i].y - mean, c2 = v[i].z - mean,
                            c3 = v[i].w - mean;
                sq += (c0 * c0 + c1 * c1) + (c2 * c2 + c3 * c3);
            }
        }
        const float inv = 1.0f / sqrtf(prb_warp_sum(sq) / (float)k + a.eps);
#pragma unroll
        for (int i = 0; i < LN_MAX_K / 128; ++i) {
            const int idx = lane + 32 * i;
            if (idx < nvec) {
                const float4 gm = reinterpret_cast<const float4*>(a.gamma)[idx];
                float4 bt = make_float4(0.f, 0.f, 0.f, 0.f);
                if (a.beta) bt = reinterpret_cast<const float4*>(a.beta)[idx];
                const __nv_bfloat162 lo = __floats2bfloat162_rn(
                    (v[i].x - mean) * inv * gm.x + bt.x, (v[i].y - mean) * inv * gm.y + bt.y);
                const __nv_bfloat162 hi = __floats2bfloat162_rn(
                    (v[i].z - mean) * inv * gm.z + bt.z, (v[i].w - mean) * inv * gm.w + bt.w);
                uint2 pk;
                pk.x = *reinterpret_cast<const uint32_t*>(&lo);
                pk.y = *reinterpret_cast<const uint32_t*>(&hi);
                *reinterpret_cast<uint2*>(dst + idx * 4) = pk;
            }
        }
    }
    __syncthreads();
}

// One 16-feature strip for all tokens: stream the rest of the weights (the first PF steps
// are in `pf`), multiply, add the warps' partial sums in warp order, epilogue.  Ends with a
// barrier, so `red` may be reused at once.
template <int MT, bool LN, typename O>
__device__ __forceinline__ void strip(const Args& a, int strip_index, float* red,
                                      const __nv_bfloat16* xs, Prefetch& pf) {
    constexpr int MP = 8 * MT;      // padded token count
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, q = lane & 3;        // MMA group (row / token) and quad index
    const int n0 = strip_index * ROWS;
    const int k = a.k, m = a.m, n = a.n;
    float acc[MT][4];
#pragma unroll
    for (int i = 0; i < MT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.0f;
    const int steps = (k + KSTEP - 1) / KSTEP;
    const int r0 = n0 + g, r1 = n0 + g + 8;
    const bool row0_ok = r0 < n, row1_ok = r1 < n;
    const __nv_bfloat16* w0 = a.w + (size_t)(row0_ok ? r0 : 0) * a.ldw;
    const __nv_bfloat16* w1 = a.w + (size_t)(row1_ok ? r1 : 0) * a.ldw;

    for (int s0 = warp; s0 < steps; s0 += WARPS * PF) {
#pragma unroll
        for (int p = 0; p < PF; ++p) {
            const int s = s0 + p * WARPS;
            if (s >= steps) break;
            const uint4 wa = pf.wa[p], wb = pf.wb[p];
            {   // refill this slot with the step PF rounds ahead
                const int kk = (s + PF * WARPS) * KSTEP + q * 8;
                const bool ok = kk < k;
                pf.wa[p] = (ok && row0_ok) ? ldg_stream(w0 + kk) : make_uint4(0, 0, 0, 0);
                pf.wb[p] = (ok && row1_ok) ? ldg_stream(w1 + kk) : make_uint4(0, 0, 0, 0);
            }
            const int kx = s * KSTEP + q * 8;      // this thread's 8 k indices of the step
            const bool kok = kx < k;
#pragma unroll
            for (int nt = 0; nt < MT; ++nt) {
                uint4 xv = make_uint4(0, 0, 0, 0);
                const int tok = nt * 8 + g;
                if constexpr (LN) {
                    if (kok) xv = *reinterpret_cast<const uint4*>(xs + (size_t)tok * a.xs_pitch + kx);
                } else {
                    if (kok && tok < m)
                        xv = *reinterpret_cast<const uint4*>(a.x + (size_t)tok * a.ldx + kx);
                }
                // elements 0..3 of each load feed the first MMA, 4..7 the second
                mma16816(acc[nt], wa.x, wb.x, wa.y, wb.y, xv.x, xv.y);
                mma16816(acc[nt], wa.z, wb.z, wa.w, wb.w, xv.z, xv.w);
            }
        }
    }
    // ---- add the warps' partial sums in warp order
    // acc[nt][0,1]: feature g, tokens nt*8 + q*2 + {0,1}; acc[nt][2,3]: feature g + 8
#pragma unroll
    for (int nt = 0; nt < MT; ++nt) {
        float* base = red + ((size_t)warp * ROWS) * MP + nt * 8 + q * 2;
        base[(size_t)g * MP] = acc[nt][0];
        base[(size_t)g * MP + 1] = acc[nt][1];
        base[(size_t)(g + 8) * MP] = acc[nt][2];
        base[(size_t)(g + 8) * MP + 1] = acc[nt][3];
    }
    __syncthreads();
    O* out = reinterpret_cast<O*>(a.out);
    for (int e = threadIdx.x; e < ROWS * MP; e += THREADS) {
        const int tok = e / ROWS, r = e % ROWS;    // consecutive threads: consecutive features
        const int col = n0 + r;
        if (tok >= m || col >= n) continue;
        float v = 0.0f;
#pragma unroll
        for (int wv = 0; wv < WARPS; ++wv) v += red[((size_t)wv * ROWS + r) * MP + tok];
        if (a.bias) v += a.bias[col];
        v = prb_activate(v, a.act);
        if (a.resid) v += a.resid[(size_t)tok * a.ldc + col];
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
                    int c = col - a.q_width;
                    O* pages = reinterpret_cast<O*>(c < a.kv_width ? a.k_pages : a.v_pages);
                    if (c >= a.kv_width) c -= a.kv_width;
                    const int h = c / a.head_dim, d = c - h * a.head_dim;
                    const int kv_heads = a.kv_width / a.head_dim;
                    pages[(((size_t)page * kv_heads + h) * a.page_size + off) * a.head_dim + d] = o;
                }
            }
        }
    }
    __syncthreads();
}
}  // namespace smallm
