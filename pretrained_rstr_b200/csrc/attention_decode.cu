// Decode attention over the paged bfloat16 cache: one query row per (token, head), keys
// split into fixed ranges of absolute positions so that a single token still fills the
// GPU, partial results merged in split order.
//
// Grid (token list, head, split).  Split s owns positions [s*SPLIT, (s+1)*SPLIT), a
// multiple of the page size, so what a split sums and in which order depends only on
// the token's own visible range [lo, pos], never on the batch.  Each warp takes the
// keys of the split in turn, 32/LPK keys per load (LPK lanes share one key row, 16 bytes
// each), keeps a running maximum and sum (online softmax, float32) and accumulates
// weighted values; warps are merged through shared memory, splits through a float32
// workspace: the last CTA of a (token, head) to finish merges all of its splits in
// order s = first..last (a counter in scratch memory tells which CTA is last, and is
// reset by it).  Softmax statistics and all sums are float32.
//
// Scratch: workspace [tokens, heads, max_splits, head_dim + 2] float32 and counters
// [tokens * heads] int32 (zero before the first launch; the kernel leaves them zero).
#include "common.cuh"

namespace {
constexpr int DEC_THREADS = 128;
constexpr int DEC_WARPS = DEC_THREADS / 32;
constexpr int SPLIT = 128;          // keys per split
constexpr int MAX_DH = 256;

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

template <int LPK>   // lanes per key row: 2, 4, 8, 16 or 32 (head_dim <= 8 * LPK)
__global__ void __launch_bounds__(DEC_THREADS)
attention_decode_kernel(__nv_bfloat16* __restrict__ out, long out_stride,
                        const __nv_bfloat16* __restrict__ q, long q_stride,
                        const __nv_bfloat16* __restrict__ k_pages,
                        const __nv_bfloat16* __restrict__ v_pages,
                        const int* __restrict__ block_table, const int* __restrict__ seq_of_token,
                        const int* __restrict__ positions, const int* __restrict__ token_list,
                        const int* __restrict__ token_count, int n_heads, int kv_heads,
                        int head_dim, int page_size, int max_pages, int num_pages, float scale,
                        int window, float* __restrict__ workspace, int* __restrict__ counters,
                        int max_splits, int* status) {
    constexpr int KPW = 32 / LPK;                 // keys per warp per load
    __shared__ float sh_m[DEC_WARPS], sh_l[DEC_WARPS];
    __shared__ float sh_o[DEC_WARPS][MAX_DH];
    __shared__ int sh_last;
    __shared__ int sh_pages[SPLIT / 8];          // pages of this split (page_size >= 8)

    prb_grid_launch_dependents();
    prb_grid_wait();
    const int idx = blockIdx.x;
    if (token_count != nullptr && idx >= *token_count) return;
    const int t = token_list ? token_list[idx] : idx;
    const int h = blockIdx.y, s = blockIdx.z;
    const int b = seq_of_token[t];
    if (b < 0) return;
    const int pos = positions[t];
    if (pos < 0 || pos >= max_pages * page_size) {
        if (threadIdx.x == 0 && s == 0) prb_set_status(status, PRB_S_POSITION_RANGE, t, pos, 0);
        return;
    }
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int s_first = lo / SPLIT, s_last = pos / SPLIT;
    if (s_last >= max_splits) {                   // the launch does not cover this context
        if (threadIdx.x == 0 && s == 0) prb_set_status(status, PRB_S_POSITION_RANGE, t, pos, max_splits);
        return;
    }
    if (s < s_first || s > s_last) return;
    const int n_splits = s_last - s_first + 1;
    const int k_begin = max(lo, s * SPLIT), k_end = min(pos + 1, (s + 1) * SPLIT);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane % LPK;                   // which 16-byte piece of the row
    const int kslot = lane / LPK;                 // which key of the warp's load
    const int hk = h / (n_heads / kv_heads);
    const int* table = block_table + (size_t)b * max_pages;
    const bool piece_ok = sub * 8 < head_dim;

    // this lane's 8 query dims; scores are (q . k) * scale as in the formula
    float qf[8];
    {
        const __nv_bfloat16* qp = q + (size_t)t * q_stride + (size_t)h * head_dim + sub * 8;
#pragma unroll
        for (int i = 0; i < 8; ++i) qf[i] = piece_ok ? __bfloat162float(qp[i]) : 0.0f;
    }
    float m = -INFINITY, l = 0.0f;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.0f;

    // page ids of this split, once
    const int first_page = (s * SPLIT) / page_size;
    for (int i = threadIdx.x; i < SPLIT / page_size; i += DEC_THREADS)
        sh_pages[i] = (first_page + i < max_pages) ? table[first_page + i] : -1;
    __syncthreads();

    // keys k_begin + warp*KPW + kslot, stepping DEC_WARPS*KPW; UNROLL steps' loads are
    // issued before any of them is used
    constexpr int UNROLL = 8;
    for (int base = k_begin + warp * KPW; base < k_end; base += DEC_WARPS * KPW * UNROLL) {
        uint4 kraw[UNROLL], vraw[UNROLL];
        bool ok[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int j = base + u * DEC_WARPS * KPW + kslot;
            ok[u] = false;
            kraw[u] = make_uint4(0, 0, 0, 0);
            vraw[u] = make_uint4(0, 0, 0, 0);
            if (j < k_end) {
                const int page = sh_pages[j / page_size - first_page];
                if (page < 0 || page >= num_pages) {
                    prb_set_status(status, PRB_S_PAGE_RANGE, t, j, page);
                } else {
                    ok[u] = true;
                    if (piece_ok) {
                        const size_t row =
                            (((size_t)page * kv_heads + hk) * page_size + (j % page_size)) *
                                head_dim + sub * 8;
                        kraw[u] = *reinterpret_cast<const uint4*>(k_pages + row);
                        vraw[u] = *reinterpret_cast<const uint4*>(v_pages + row);
                    }
                }
            }
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            float part = dot8(kraw[u], qf);
            // every lane takes part in the reduction over the LPK pieces of a key row
#pragma unroll
            for (int o = LPK / 2; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
            const float sc = ok[u] ? part * scale : -INFINITY;
            // online softmax per key slot (each group of LPK lanes has its own running state)
            const float m_new = fmaxf(m, sc);
            if (m_new > -INFINITY) {
                const float corr = (m == -INFINITY) ? 0.0f : __expf(m - m_new);
                const float p = (sc == -INFINITY) ? 0.0f : __expf(sc - m_new);
                l = l * corr + p;
                const __nv_bfloat162* vp = reinterpret_cast<const __nv_bfloat162*>(&vraw[u]);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 f = __bfloat1622float2(vp[i]);
                    acc[2 * i] = fmaf(p, f.x, acc[2 * i] * corr);
                    acc[2 * i + 1] = fmaf(p, f.y, acc[2 * i + 1] * corr);
                }
                m = m_new;
            }
        }
    }
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
    for (int w = 0; w < DEC_WARPS; ++w) mt = fmaxf(mt, sh_m[w]);
    float lt = 0.0f;
    float cw[DEC_WARPS];
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) {
        cw[w] = (sh_m[w] == -INFINITY) ? 0.0f : __expf(sh_m[w] - mt);
        lt += sh_l[w] * cw[w];
    }
    const size_t pair = (size_t)idx * n_heads + h;       // scratch is indexed by list place
    float* ws = workspace + (pair * max_splits + s) * (size_t)(head_dim + 2);
    __nv_bfloat16* o = out + (size_t)t * out_stride + (size_t)h * head_dim;
    for (int d = threadIdx.x; d < head_dim; d += DEC_THREADS) {
        float od = 0.0f;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) od += sh_o[w][d] * cw[w];
        if (n_splits == 1) o[d] = __float2bfloat16_rn(lt > 0.0f ? od / lt : 0.0f);
        else ws[d] = od;
    }
    if (n_splits == 1) return;
    if (threadIdx.x == 0) { ws[head_dim] = mt; ws[head_dim + 1] = lt; }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int done = atomicAdd(&counters[pair], 1);
        sh_last = (done == n_splits - 1) ? 1 : 0;
    }
    __syncthreads();
    if (!sh_last) return;
    __threadfence();
    // last CTA of this (token, head): merge the splits in order
    const float* wbase = workspace + pair * max_splits * (size_t)(head_dim + 2);
    float mg = -INFINITY;
    for (int ss = s_first; ss <= s_last; ++ss)
        mg = fmaxf(mg, __ldcg(wbase + (size_t)ss * (head_dim + 2) + head_dim));
    float lg = 0.0f;
    for (int ss = s_first; ss <= s_last; ++ss) {
        const float* w = wbase + (size_t)ss * (head_dim + 2);
        const float ms = __ldcg(w + head_dim);
        lg += __ldcg(w + head_dim + 1) * ((ms == -INFINITY) ? 0.0f : __expf(ms - mg));
    }
    for (int d = threadIdx.x; d < head_dim; d += DEC_THREADS) {
        float od = 0.0f;
        for (int ss = s_first; ss <= s_last; ++ss) {
            const float* w = wbase + (size_t)ss * (head_dim + 2);
            const float ms = __ldcg(w + head_dim);
            od += __ldcg(w + d) * ((ms == -INFINITY) ? 0.0f : __expf(ms - mg));
        }
        o[d] = __float2bfloat16_rn(lg > 0.0f ? od / lg : 0.0f);
    }
    if (threadIdx.x == 0) counters[pair] = 0;
}
}  // namespace

PRB_API int prb_attention_decode_split() { return SPLIT; }

// workspace: float32 [n_list, n_heads, max_splits, head_dim + 2]; counters: int32
// [n_list * n_heads], zero; both indexed by the place in the token list.  token_list/token_count may be null (all
// tokens 0..n_list-1).  max_splits >= ceil(max context / SPLIT).
PRB_API int prb_attention_decode(void* out, long out_stride, const void* q, long q_stride,
                                 const void* k_pages, const void* v_pages, const int* block_table,
                                 const int* seq_of_token, const int* positions,
                                 const int* token_list, const int* token_count, int n_list,
                                 int n_heads, int kv_heads, int head_dim, int page_size,
                                 int max_pages, int num_pages, float scale, int window,
                                 float* workspace, int* counters, int max_splits, int* status,
                                 cudaStream_t stream) {
    if (n_list <= 0) return 0;
    if (n_heads <= 0 || kv_heads <= 0 || n_heads % kv_heads != 0 || head_dim <= 0 ||
        head_dim % 8 != 0 || head_dim > MAX_DH || page_size < 8 || SPLIT % page_size != 0 ||
        max_splits <= 0 || max_splits > 65535 || n_heads > 65535)
        return PRB_E_SIZE;
    if (q_stride % 8 != 0 || ((uintptr_t)q) % 16 != 0 || ((uintptr_t)k_pages) % 16 != 0 ||
        ((uintptr_t)v_pages) % 16 != 0)
        return PRB_E_ALIGN;
    dim3 grid(n_list, n_heads, max_splits);
    const int pieces = head_dim / 8;
#define PRB_DEC(L)                                                                             \
    e = prb_launch_dependent(attention_decode_kernel<L>, grid, dim3(DEC_THREADS), 0, stream,   \
        (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)q, q_stride,                    \
        (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages, block_table,             \
        seq_of_token, positions, token_list, token_count, n_heads, kv_heads, head_dim,         \
        page_size, max_pages, num_pages, scale, window, workspace, counters, max_splits, status)
    cudaError_t e;
    if (pieces <= 2) PRB_DEC(2);
    else if (pieces <= 4) PRB_DEC(4);
    else if (pieces <= 8) PRB_DEC(8);
    else if (pieces <= 16) PRB_DEC(16);
    else PRB_DEC(32);
#undef PRB_DEC
    if (e != cudaSuccess) return (int)e;
    return 0;
}

// ---------------------------------------------------------------------------------
// Entry point that allocates nothing (declared in attention_decode_noalloc.h).
//
// Some programs that load this library may not allocate device memory at all: a host
// whose allocator owns the whole GPU and hands nothing to third parties, a plugin that
// runs inside someone else's process under a fixed memory budget, or a caller in a
// context where an allocation would synchronise the device or fail.  For them the split
// workspace and the per-(token, head) counters of the decode attention kernel live in
// two file-scope device arrays of fixed size instead of caller-provided buffers.  Every
// GPU that loads the library holds these arrays (a little over 4 MiB) until the process
// exits, whether or not the entry point is ever called.
//
// In host code `noalloc_workspace` and `noalloc_counters` are only stand-ins for the
// device arrays, not device addresses; the addresses are asked for with
// cudaGetSymbolAddress once per device, with that device current, by the first call on
// that device.  That first call should therefore come before any stream capture.
//
// All calls share the two arrays and the arrays keep what the last call left in them.
// The counters have to be zero when the kernel starts, so every call clears the part it
// is going to use (an asynchronous memset on the caller's stream, ordered before the
// kernel).  Two calls whose kernels overlap on the GPU (different streams, or graph
// branches that run side by side) race on the arrays and give wrong results: keep calls
// to this entry point ordered one after the other.
constexpr long NOALLOC_WS_FLOATS = 1L << 20;     // 4 MiB of float32 partial results
constexpr int NOALLOC_COUNTERS = 1 << 14;        // 64 KiB of int32 counters
constexpr int NOALLOC_MAX_DEVICES = 64;

static __device__ __align__(256) float noalloc_workspace[NOALLOC_WS_FLOATS];
static __device__ __align__(256) int noalloc_counters[NOALLOC_COUNTERS];

namespace {
struct NoAllocDevice {
    bool ready = false;
    float* workspace = nullptr;
    int* counters = nullptr;
};
NoAllocDevice noalloc_devices[NOALLOC_MAX_DEVICES];
}  // namespace

// Largest sizes the entry point takes: floats of workspace (n_list * n_heads * max_splits
// * (head_dim + 2) must not exceed it) and counters (n_list * n_heads).
PRB_API void prb_attention_decode_noalloc_limits(long* workspace_floats, int* counters) {
    if (workspace_floats) *workspace_floats = NOALLOC_WS_FLOATS;
    if (counters) *counters = NOALLOC_COUNTERS;
}

// Same computation and arguments as prb_attention_decode, without the scratch pointers.
// Returns PRB_E_SIZE (-3) when the launch would need more scratch than the fixed arrays
// hold, a positive cudaError_t if the set-up or the launch failed, 0 otherwise.
PRB_API int prb_attention_decode_noalloc(void* out, long out_stride, const void* q, long q_stride,
                                         const void* k_pages, const void* v_pages,
                                         const int* block_table, const int* seq_of_token,
                                         const int* positions, const int* token_list,
                                         const int* token_count, int n_list, int n_heads,
                                         int kv_heads, int head_dim, int page_size, int max_pages,
                                         int num_pages, float scale, int window, int max_splits,
                                         int* status, cudaStream_t stream) {
    if (n_list <= 0) return 0;
    if (n_heads <= 0 || head_dim <= 0 || max_splits <= 0) return PRB_E_SIZE;
    const long need_ws = (long)n_list * n_heads * max_splits * (head_dim + 2);
    const long need_counters = (long)n_list * n_heads;
    if (need_ws > NOALLOC_WS_FLOATS || need_counters > NOALLOC_COUNTERS) return PRB_E_SIZE;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= NOALLOC_MAX_DEVICES) return PRB_E_ARG;
    NoAllocDevice& d = noalloc_devices[dev];
    if (!d.ready) {
        // once per device, with that device current: the device addresses of the arrays
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, noalloc_workspace);
        if (e != cudaSuccess) return (int)e;
        d.workspace = static_cast<float*>(p);
        e = cudaGetSymbolAddress(&p, noalloc_counters);
        if (e != cudaSuccess) return (int)e;
        d.counters = static_cast<int*>(p);
        d.ready = true;
    }
    // the counters must start at zero, whatever an earlier call left behind
    e = cudaMemsetAsync(d.counters, 0, (size_t)need_counters * sizeof(int), stream);
    if (e != cudaSuccess) return (int)e;
    return prb_attention_decode(out, out_stride, q, q_stride, k_pages, v_pages, block_table,
                                seq_of_token, positions, token_list, token_count, n_list, n_heads,
                                kv_heads, head_dim, page_size, max_pages, num_pages, scale, window,
                                d.workspace, d.counters, max_splits, status, stream);
}
