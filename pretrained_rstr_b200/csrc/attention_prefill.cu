// Causal attention for prompt portions over the paged bfloat16 cache, flash style:
// scores are never written to memory.  One CTA takes 64 consecutive query tokens of one
// request for one head (warp groups of 4 warps x 16 rows) and walks the keys in tiles of 64 absolute
// positions (tile boundaries at multiples of 64, independent of where the portion
// starts, so a row's summation order depends on its own position only).  Per tile:
// S = Q K^T on tensor cores (bf16 inputs, float32 accumulate), scale, mask (causal,
// window, request length), online softmax in float32, P (rounded to bf16 as an MMA
// operand only) times V accumulated in float32.  Keys and values are fetched through
// the block table with cp.async, double buffered, so later portions see earlier pages.
//
// This first tensor-core version uses mma.sync m16n8k16; it is the kernel a tcgen05
// version has to beat.  Head sizes: multiples of 16 up to 256 (template instances).
#include "common.cuh"

namespace {
constexpr int QT = 64;              // queries per CTA
constexpr int LIST_TILE = 128;      // queries per item of the work list
constexpr int KT = 64;              // keys per tile
constexpr int PADE = 8;             // row padding in elements (16 bytes): conflict-free ldmatrix

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
    const int bytes = valid ? 16 : 0;      // src-size 0: the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&p);
}

__device__ __forceinline__ void group_sync(int group) {
    // barrier of the 128 threads of one warp group (ids 1.. leave 0 to __syncthreads)
    asm volatile("bar.sync %0, 128;" ::"r"(group + 1) : "memory");
}

// G warp groups of four warps share the key tiles of one 64-query tile: group g takes
// tiles first+g, first+g+G, ... with its own running softmax state and its own buffers,
// and the groups' results are merged (in group order) at the end.  The kernel lasts as
// long as its longest chain of key tiles, and this divides that chain by G.
template <int DH, int G>
__global__ void __launch_bounds__(128 * G)
attention_prefill_kernel(__nv_bfloat16* __restrict__ out, long out_stride,
                         const __nv_bfloat16* __restrict__ q, long q_stride,
                         const __nv_bfloat16* __restrict__ k_pages,
                         const __nv_bfloat16* __restrict__ v_pages,
                         const int* __restrict__ block_table, const int* __restrict__ positions,
                         const int* __restrict__ tile_req, const int* __restrict__ tile_row0,
                         const int* __restrict__ tile_rows, const int* __restrict__ tile_count,
                         int n_heads, int kv_heads, int page_size, int max_pages, int num_pages,
                         float scale, int window, int* status) {
    constexpr int PITCH = DH + PADE;
    constexpr int CHUNKS = DH / 8;                 // 16-byte pieces per row
    constexpr int GROUP_ELEMS = (QT + 4 * KT) * PITCH;
    extern __shared__ __align__(16) uint8_t smem_raw[];
    const int group = threadIdx.x >> 7, tid = threadIdx.x & 127;
    __nv_bfloat16* base = reinterpret_cast<__nv_bfloat16*>(smem_raw) + (size_t)group * GROUP_ELEMS;
    __nv_bfloat16* qs = base;                      // [QT][PITCH]       (a copy per group)
    __nv_bfloat16* ks = qs + QT * PITCH;           // [2][KT][PITCH]
    __nv_bfloat16* vs = ks + 2 * KT * PITCH;       // [2][KT][PITCH]

    // the longest tiles (late query positions) first
    // a work item is a tile of up to LIST_TILE rows; two CTAs take its halves
    const int n_items = tile_count != nullptr ? *tile_count : (int)gridDim.x / (LIST_TILE / QT);
    const int which = blockIdx.x / (LIST_TILE / QT), half = blockIdx.x % (LIST_TILE / QT);
    if (which >= n_items) return;
    const int item = n_items - 1 - which;
    const int h = blockIdx.y;
    const int b = tile_req[item];
    const int item_rows = tile_rows[item];         // valid queries of the item (1..LIST_TILE)
    if (item_rows > 0 && item_rows <= half * QT) return;
    const int row0 = tile_row0[item] + half * QT;  // first token row of this CTA
    const int rows = min(QT, item_rows - half * QT);
    const int pos0 = positions[row0];
    const int pos_last = pos0 + rows - 1;
    if (b < 0 || item_rows <= 0 || item_rows > LIST_TILE || pos0 < 0 ||
        pos_last >= max_pages * page_size) {
        if (threadIdx.x == 0) prb_set_status(status, PRB_S_POSITION_RANGE, row0, pos0, rows);
        return;
    }
    const int hk = h / (n_heads / kv_heads);
    const int* table = block_table + (size_t)b * max_pages;
    const int warp = tid >> 5, lane = tid & 31;    // warp within the group
    const int lo_all = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
    const int tile_first = lo_all / KT, tile_last = pos_last / KT;

    // ---- Q tile -> this group's shared memory (rows beyond `rows` are zero)
    for (int c = tid; c < QT * CHUNKS; c += 128) {
        const int r = c / CHUNKS, piece = c % CHUNKS;
        const bool valid = r < rows;
        const __nv_bfloat16* src = q + (size_t)(row0 + (valid ? r : 0)) * q_stride +
                                   (size_t)h * DH + piece * 8;
        cp_async16(qs + r * PITCH + piece * 8, src, valid);
    }
    auto load_kv = [&](int tile, int buf) {
        __nv_bfloat16* kd = ks + buf * KT * PITCH;
        __nv_bfloat16* vd = vs + buf * KT * PITCH;
        for (int c = tid; c < KT * CHUNKS; c += 128) {
            const int r = c / CHUNKS, piece = c % CHUNKS;
            const int j = tile * KT + r;
            bool valid = j >= lo_all && j <= pos_last;
            size_t off = 0;
            if (valid) {
                const int page = table[j / page_size];
                if (page < 0 || page >= num_pages) {
                    prb_set_status(status, PRB_S_PAGE_RANGE, row0, j, page);
                    valid = false;
                } else {
                    off = (((size_t)page * kv_heads + hk) * page_size + (j % page_size)) * DH +
                          piece * 8;
                }
            }
            cp_async16(kd + r * PITCH + piece * 8, k_pages + off, valid);
            cp_async16(vd + r * PITCH + piece * 8, v_pages + off, valid);
        }
    };
    const int my_first = tile_first + group;
    if (my_first <= tile_last) load_kv(my_first, 0);
    cp_async_commit();

    float o[DH / 8][4];
#pragma unroll
    for (int i = 0; i < DH / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
    const int qr = warp * 16 + (lane >> 2);        // this thread's first query row in the tile
    const int qpos[2] = {pos0 + qr, pos0 + qr + 8};
    const bool qvalid[2] = {qr < rows, qr + 8 < rows};
    const float sl2 = scale * 1.4426950408889634f;  // scores are handled in log2 units
    const int warp_pos_min = pos0 + warp * 16;

    int it = 0;
    for (int tile = my_first; tile <= tile_last; tile += G, ++it) {
        const int buf = it & 1;
        if (tile + G <= tile_last) {
            load_kv(tile + G, buf ^ 1);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        group_sync(group);
        const __nv_bfloat16* kb = ks + buf * KT * PITCH;
        const __nv_bfloat16* vb = vs + buf * KT * PITCH;

        // ---- S = Q K^T for this warp's 16 rows x 64 keys
        float s[KT / 8][4];
#pragma unroll
        for (int i = 0; i < KT / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f;
#pragma unroll
        for (int kk = 0; kk < DH / 16; ++kk) {
            uint32_t a[4];
            ldmatrix_x4(a, qs + (warp * 16 + (lane & 15)) * PITCH + kk * 16 + (lane >> 4) * 8);
#pragma unroll
            for (int nt = 0; nt < KT / 16; ++nt) {
                uint32_t bfr[4];
                const int mi = lane >> 3, r = lane & 7;
                ldmatrix_x4(bfr, kb + (nt * 16 + (mi >> 1) * 8 + r) * PITCH + kk * 16 + (mi & 1) * 8);
                mma_bf16(s[2 * nt], a, bfr[0], bfr[1]);
                mma_bf16(s[2 * nt + 1], a, bfr[2], bfr[3]);
            }
        }
        // ---- scale, mask, online softmax (two rows per thread); a tile whose keys all lie
        // at or before the warp's first query needs no mask
        const bool need_mask = window > 0 || tile * KT + KT - 1 > warp_pos_min || rows < QT;
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < KT / 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int rr = e >> 1;
                float v = s[nt][e] * sl2;
                if (need_mask) {
                    const int j = tile * KT + nt * 8 + (lane & 3) * 2 + (e & 1);
                    const bool vis = qvalid[rr] && j <= qpos[rr] &&
                                     (window <= 0 || j > qpos[rr] - window);
                    v = vis ? v : -INFINITY;
                }
                s[nt][e] = v;
                mx[rr] = fmaxf(mx[rr], v);
            }
        }
        float corr[2];
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
            mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 1));
            mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 2));
            const float m_new = fmaxf(m_run[rr], mx[rr]);
            corr[rr] = (m_run[rr] == -INFINITY) ? 0.0f : exp2f(m_run[rr] - m_new);
            m_run[rr] = m_new;
        }
        float rs[2] = {0.0f, 0.0f};
#pragma unroll
        for (int nt = 0; nt < KT / 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int rr = e >> 1;
                const float p = (s[nt][e] == -INFINITY) ? 0.0f : exp2f(s[nt][e] - m_run[rr]);
                s[nt][e] = p;
                rs[rr] += p;
            }
        }
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) l_run[rr] = l_run[rr] * corr[rr] + rs[rr];
#pragma unroll
        for (int i = 0; i < DH / 8; ++i) {
            o[i][0] *= corr[0]; o[i][1] *= corr[0];
            o[i][2] *= corr[1]; o[i][3] *= corr[1];
        }
        // ---- O += P V
#pragma unroll
        for (int kk = 0; kk < KT / 16; ++kk) {
            uint32_t a[4];
            a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
            a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
            a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int dt = 0; dt < DH / 16; ++dt) {
                uint32_t bfr[4];
                const int mi = lane >> 3, r = lane & 7;
                ldmatrix_x4_trans(bfr, vb + (kk * 16 + (mi & 1) * 8 + r) * PITCH + dt * 16 +
                                            (mi >> 1) * 8);
                mma_bf16(o[2 * dt], a, bfr[0], bfr[1]);
                mma_bf16(o[2 * dt + 1], a, bfr[2], bfr[3]);
            }
        }
        group_sync(group);    // the group is done with this buffer before it is refilled
    }
    cp_async_wait<0>();       // a group without tiles still has its Q copies in flight

    // ---- merge the groups (in order 1, 2, ...) into group 0, through shared memory
    if constexpr (G > 1) {
        constexpr int PER_THREAD = DH / 2 + 4;     // o values, then m and l of two rows
        float* mine = reinterpret_cast<float*>(base) + (size_t)tid * PER_THREAD;
        group_sync(group);
        if (group > 0) {
#pragma unroll
            for (int i = 0; i < DH / 8; ++i) {
                mine[4 * i] = o[i][0]; mine[4 * i + 1] = o[i][1];
                mine[4 * i + 2] = o[i][2]; mine[4 * i + 3] = o[i][3];
            }
            mine[DH / 2] = m_run[0]; mine[DH / 2 + 1] = m_run[1];
            mine[DH / 2 + 2] = l_run[0]; mine[DH / 2 + 3] = l_run[1];
        }
        __syncthreads();
        if (group > 0) return;
#pragma unroll
        for (int g = 1; g < G; ++g) {
            const float* other = reinterpret_cast<const float*>(
                                     reinterpret_cast<__nv_bfloat16*>(smem_raw) + (size_t)g * GROUP_ELEMS) +
                                 (size_t)tid * PER_THREAD;
            float c_me[2], c_ot[2];
#pragma unroll
            for (int rr = 0; rr < 2; ++rr) {
                const float mo = other[DH / 2 + rr];
                const float mn = fmaxf(m_run[rr], mo);
                c_me[rr] = (m_run[rr] == -INFINITY) ? 0.0f : exp2f(m_run[rr] - mn);
                c_ot[rr] = (mo == -INFINITY) ? 0.0f : exp2f(mo - mn);
                l_run[rr] = l_run[rr] * c_me[rr] + other[DH / 2 + 2 + rr] * c_ot[rr];
                m_run[rr] = mn;
            }
#pragma unroll
            for (int i = 0; i < DH / 8; ++i) {
                o[i][0] = o[i][0] * c_me[0] + other[4 * i] * c_ot[0];
                o[i][1] = o[i][1] * c_me[0] + other[4 * i + 1] * c_ot[0];
                o[i][2] = o[i][2] * c_me[1] + other[4 * i + 2] * c_ot[1];
                o[i][3] = o[i][3] * c_me[1] + other[4 * i + 3] * c_ot[1];
            }
        }
    }
    // ---- normalise and store
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        l_run[rr] += __shfl_xor_sync(0xffffffffu, l_run[rr], 1);
        l_run[rr] += __shfl_xor_sync(0xffffffffu, l_run[rr], 2);
    }
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        if (!qvalid[rr]) continue;
        const float inv = l_run[rr] > 0.0f ? 1.0f / l_run[rr] : 0.0f;
        __nv_bfloat16* dst = out + (size_t)(row0 + qr + rr * 8) * out_stride + (size_t)h * DH;
#pragma unroll
        for (int i = 0; i < DH / 8; ++i) {
            const __nv_bfloat162 p = __floats2bfloat162_rn(o[i][2 * rr] * inv, o[i][2 * rr + 1] * inv);
            *reinterpret_cast<__nv_bfloat162*>(dst + i * 8 + (lane & 3) * 2) = p;
        }
    }
}

template <int DH>
int launch_prefill(void* out, long out_stride, const void* q, long q_stride, const void* k_pages,
                   const void* v_pages, const int* block_table, const int* positions,
                   const int* tile_req, const int* tile_row0, const int* tile_rows,
                   const int* tile_count, int n_tiles, int n_heads, int kv_heads, int page_size,
                   int max_pages, int num_pages, float scale, int window, int* status,
                   cudaStream_t stream) {
    constexpr int G = DH <= 128 ? 2 : 1;           // warp groups (shared memory allows two)
    constexpr size_t smem = (size_t)G * (QT + 4 * KT) * (DH + PADE) * 2;
    static bool configured = false;
    if (!configured) {      // several CTAs per SM need the large shared-memory carve-out
        cudaFuncSetAttribute(attention_prefill_kernel<DH, G>,
                             cudaFuncAttributePreferredSharedMemoryCarveout,
                             cudaSharedmemCarveoutMaxShared);
        if (smem > 48 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel<DH, G>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
        }
    }
    configured = true;
    dim3 grid(n_tiles * (LIST_TILE / QT), n_heads);
    attention_prefill_kernel<DH, G><<<grid, 128 * G, smem, stream>>>(
        (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)q, q_stride,
        (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages, block_table, positions,
        tile_req, tile_row0, tile_rows, tile_count, n_heads, kv_heads, page_size, max_pages,
        num_pages, scale, window, status);
    PRB_LAUNCH_CHECK();
    return 0;
}
}  // namespace

PRB_API int prb_attention_prefill_tile() { return LIST_TILE; }

// 1 when this head size has a tensor-core instance, else 0.
PRB_API int prb_attention_prefill_supports(int head_dim) {
    return (head_dim % 16 == 0 && head_dim >= 16 && head_dim <= 128) || head_dim == 256 ? 1 : 0;
}

// Work list: tile i covers token rows [tile_row0[i], tile_row0[i] + tile_rows[i]) (at most
// 64, all of request tile_req[i], consecutive positions).  tile_count may be null.
PRB_API int prb_attention_prefill(void* out, long out_stride, const void* q, long q_stride,
                                  const void* k_pages, const void* v_pages,
                                  const int* block_table, const int* positions,
                                  const int* tile_req, const int* tile_row0, const int* tile_rows,
                                  const int* tile_count, int n_tiles, int n_heads, int kv_heads,
                                  int head_dim, int page_size, int max_pages, int num_pages,
                                  float scale, int window, int* status, cudaStream_t stream) {
    if (n_tiles <= 0) return 0;
    if (n_heads <= 0 || kv_heads <= 0 || n_heads % kv_heads != 0 || page_size <= 0 ||
        n_heads > 65535)
        return PRB_E_SIZE;
    if (!prb_attention_prefill_supports(head_dim)) return PRB_E_SIZE;
    if (q_stride % 8 != 0 || out_stride % 2 != 0 || ((uintptr_t)q) % 16 != 0 ||
        ((uintptr_t)k_pages) % 16 != 0 || ((uintptr_t)v_pages) % 16 != 0 ||
        ((uintptr_t)out) % 4 != 0)
        return PRB_E_ALIGN;
#define PRB_PF(D)                                                                              \
    case D:                                                                                    \
        return launch_prefill<D>(out, out_stride, q, q_stride, k_pages, v_pages, block_table,  \
                                 positions, tile_req, tile_row0, tile_rows, tile_count,        \
                                 n_tiles, n_heads, kv_heads, page_size, max_pages, num_pages,  \
                                 scale, window, status, stream)
    switch (head_dim) {
        PRB_PF(16); PRB_PF(32); PRB_PF(48); PRB_PF(64); PRB_PF(80); PRB_PF(96); PRB_PF(112);
        PRB_PF(128); PRB_PF(256);
        default: return PRB_E_SIZE;
    }
#undef PRB_PF
}
