// Memory-bound kernels of the step: embedding + position gather, LayerNorm, bias /
// activation / residual epilogue, cache append, page copy.  All statistics and sums in
// 32-bit; element types of tables, activations and the cache are template parameters.
#include <cstdlib>
#include "elementwise.cuh"

// Programmatic dependent launch is on unless switched off (for measurements).
static int g_pdl = 1;
int prb_pdl_enabled() { return g_pdl; }
PRB_API void prb_set_pdl(int on) { g_pdl = on ? 1 : 0; }
int prb_sm_count() {
    static int counts[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 1;
    if (counts[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 1;
        counts[dev] = n;
    }
    return counts[dev];
}
PRB_API int prb_device_sm_count() { return prb_sm_count(); }
int prb_small_ctas_early() {
    static const int on = [] { const char* e = getenv("PRB200_EARLY_SMALL"); return e ? atoi(e) : 0; }();
    return on;
}

// ------------------------------------------------------------------ embedding
template <typename W>
__global__ void embed_kernel(elementwise::EmbedArgs a) {
    elementwise::embed_token<W>(a, blockIdx.x);
}

PRB_API int prb_embed(float* out, const int* tokens, const int* positions, const void* wte,
                      const void* wpe, int n_tokens, int width, int vocab, int n_positions,
                      int table_dtype, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (width <= 0 || vocab <= 0) return PRB_E_SIZE;
    const int threads = width >= 256 ? 256 : ((width + 31) / 32) * 32;
    elementwise::EmbedArgs a{out, tokens, positions, wte, wpe, n_tokens, width, vocab,
                             n_positions, status};
    if (table_dtype == PRB_F32)
        embed_kernel<float><<<n_tokens, threads, 0, stream>>>(a);
    else if (table_dtype == PRB_BF16)
        embed_kernel<__nv_bfloat16><<<n_tokens, threads, 0, stream>>>(a);
    else
        return PRB_E_DTYPE;
    PRB_LAUNCH_CHECK();
    return 0;
}

// ------------------------------------------------------------------ LayerNorm
// rows: optional gather (out row r reads x row rows[r]).
template <typename O>
__global__ void layernorm_kernel(elementwise::NormArgs a) {
    extern __shared__ float row[];
    __shared__ float scratch[32];
    elementwise::layernorm_row<O>(a, blockIdx.x, row, scratch);
}

// Rows that fit a warp's registers (width <= 1024, a multiple of 4): one warp per row, four
// rows per CTA, 16-byte loads, statistics by shuffles only.  Same two-pass formula.
template <typename O>
__global__ void __launch_bounds__(128)
layernorm_warp_kernel(elementwise::NormArgs a) {
    const int r = blockIdx.x * 4 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    prb_grid_launch_dependents();
    prb_grid_wait();
    if (r >= a.n_rows) return;
    O* out = reinterpret_cast<O*>(a.out) + (size_t)r * a.width;
    const int src = a.rows ? a.rows[r] : r;
    if (src < 0 || src >= a.n_rows_in) {
        if (lane == 0) prb_set_status(a.status, PRB_S_ROW_RANGE, r, src, a.n_rows_in);
        for (int i = lane; i < a.width; i += 32) out[i] = prb_from_float<O>(0.0f);
        return;
    }
    const int nvec = a.width / 4;
    const float4* x4 = reinterpret_cast<const float4*>(a.x + (size_t)src * a.width);
    float4 v[8];
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int idx = lane + 32 * i;
        v[i] = idx < nvec ? x4[idx] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    // gamma and beta are asked for before the statistics are reduced, not after: the row's
    // way through the kernel is one memory round trip long instead of two
    const float4* g4 = reinterpret_cast<const float4*>(a.gamma);
    const float4* b4 = reinterpret_cast<const float4*>(a.beta);
    float4 g[8], b[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int idx = lane + 32 * i;
        g[i] = idx < nvec ? __ldg(g4 + idx) : make_float4(0.f, 0.f, 0.f, 0.f);
        b[i] = (idx < nvec && a.beta) ? __ldg(b4 + idx) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    const float mean = prb_warp_sum(s) / (float)a.width;
    float q = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        if (lane + 32 * i < nvec) {
            const float c0 = v[i].x - mean, c1 = v[i].y - mean, c2 = v[i].z - mean,
                        c3 = v[i].w - mean;
            q += (c0 * c0 + c1 * c1) + (c2 * c2 + c3 * c3);
        }
    }
    const float inv = 1.0f / sqrtf(prb_warp_sum(q) / (float)a.width + a.eps);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int idx = lane + 32 * i;
        if (idx < nvec) {
            const float y0 = (v[i].x - mean) * inv * g[i].x + b[i].x, y1 = (v[i].y - mean) * inv * g[i].y + b[i].y;
            const float y2 = (v[i].z - mean) * inv * g[i].z + b[i].z, y3 = (v[i].w - mean) * inv * g[i].w + b[i].w;
            if constexpr (sizeof(O) == 4) {
                *reinterpret_cast<float4*>(out + idx * 4) = make_float4(y0, y1, y2, y3);
            } else {
                const __nv_bfloat162 lo = __floats2bfloat162_rn(y0, y1), hi = __floats2bfloat162_rn(y2, y3);
                uint2 pk;
                pk.x = *reinterpret_cast<const uint32_t*>(&lo);
                pk.y = *reinterpret_cast<const uint32_t*>(&hi);
                *reinterpret_cast<uint2*>(out + idx * 4) = pk;
            }
        }
    }
}

PRB_API int prb_layernorm(void* out, const float* x, const float* gamma, const float* beta,
                          const int* rows, int n_rows, int n_rows_in, int width, float eps,
                          int out_dtype, int* status, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (width <= 0 || (size_t)width * 4 > 200 * 1024) return PRB_E_SIZE;
    if (out_dtype != PRB_F32 && out_dtype != PRB_BF16) return PRB_E_DTYPE;
    elementwise::NormArgs a{out, x, gamma, beta, rows, n_rows, n_rows_in, width, eps, status};
    const bool aligned = ((uintptr_t)x) % 16 == 0 && ((uintptr_t)out) % 16 == 0 &&
                         ((uintptr_t)gamma) % 16 == 0 && (!beta || ((uintptr_t)beta) % 16 == 0);
    if (width % 4 == 0 && width <= 1024 && aligned && n_rows >= 16) {
        const int blocks = (n_rows + 3) / 4;
        cudaError_t e = out_dtype == PRB_F32
            ? prb_launch_maybe_early(prb_small_ctas_early(), layernorm_warp_kernel<float>,
                                     dim3(blocks), dim3(128), 0, stream, a)
            : prb_launch_maybe_early(prb_small_ctas_early(), layernorm_warp_kernel<__nv_bfloat16>,
                                     dim3(blocks), dim3(128), 0, stream, a);
        if (e != cudaSuccess) return (int)e;
        return 0;
    }
    const int threads = width >= 256 ? 256 : ((width + 31) / 32) * 32;
    const size_t smem = (size_t)width * sizeof(float);
    // (few rows: the norm of the wanted rows before the head; launched the plain way, which
    // keeps the head's product from starting its copies while the last layer still runs)
    if (out_dtype == PRB_F32) {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(layernorm_kernel<float>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        layernorm_kernel<float><<<n_rows, threads, smem, stream>>>(a);
    } else {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(layernorm_kernel<__nv_bfloat16>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        layernorm_kernel<__nv_bfloat16><<<n_rows, threads, smem, stream>>>(a);
    }
    PRB_LAUNCH_CHECK();
    return 0;
}

// -------------------------------------------------- bias + activation + residual
// out[m,n] = act(in[m,n] + bias[n]) (+ resid[m,n]); sums in 32-bit.
template <typename I, typename O>
__global__ void bias_act_kernel(O* __restrict__ out, const I* __restrict__ in,
                                const float* __restrict__ bias, const float* __restrict__ resid,
                                size_t total, int n, int act) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    float v = prb_to_float<I>(in[i]);
    if (bias) v += bias[i % n];
    v = prb_activate(v, act);
    if (resid) v += resid[i];
    out[i] = prb_from_float<O>(v);
}

PRB_API int prb_bias_act(void* out, const void* in, const float* bias, const float* resid, int m,
                         int n, int act, int in_dtype, int out_dtype, cudaStream_t stream) {
    if (m <= 0 || n <= 0) return 0;
    const size_t total = (size_t)m * n;
    const int threads = 256;
    const unsigned blocks = (unsigned)((total + threads - 1) / threads);
#define PRB_BA(I, O)                                                                        \
    bias_act_kernel<I, O><<<blocks, threads, 0, stream>>>((O*)out, (const I*)in, bias, resid, \
                                                          total, n, act)
    if (in_dtype == PRB_F32 && out_dtype == PRB_F32) PRB_BA(float, float);
    else if (in_dtype == PRB_BF16 && out_dtype == PRB_F32) PRB_BA(__nv_bfloat16, float);
    else if (in_dtype == PRB_BF16 && out_dtype == PRB_BF16) PRB_BA(__nv_bfloat16, __nv_bfloat16);
    else if (in_dtype == PRB_F32 && out_dtype == PRB_BF16) PRB_BA(float, __nv_bfloat16);
    else return PRB_E_DTYPE;
#undef PRB_BA
    PRB_LAUNCH_CHECK();
    return 0;
}

// --------------------------------------------------------------- cache append
template <typename T>
__global__ void kv_append_kernel(elementwise::AppendArgs a) {
    prb_grid_launch_dependents();
    prb_grid_wait();
    elementwise::append_token<T>(a, blockIdx.x);
}

PRB_API int prb_kv_append(void* k_pages, void* v_pages, const void* k_src, const void* v_src,
                          long src_stride, const int* slots, int n_tokens, int kv_heads,
                          int head_dim, int page_size, int num_pages, int dtype, int* status,
                          cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (kv_heads <= 0 || head_dim <= 0 || page_size <= 0) return PRB_E_SIZE;
    const int row = kv_heads * head_dim;
    const int threads = row >= 256 ? 256 : ((row + 31) / 32) * 32;
    elementwise::AppendArgs a{k_pages, v_pages, k_src, v_src, src_stride, slots, n_tokens,
                              kv_heads, head_dim, page_size, num_pages, status};
    cudaError_t e;
    if (dtype == PRB_F32)
        e = prb_launch_dependent(kv_append_kernel<float>, dim3(n_tokens), dim3(threads), 0, stream, a);
    else if (dtype == PRB_BF16)
        e = prb_launch_dependent(kv_append_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), 0,
                                 stream, a);
    else
        return PRB_E_DTYPE;
    if (e != cudaSuccess) return (int)e;
    return 0;
}

// ------------------------------------------------------------------ page copy
// Copy-on-write (page_pool.clj:892-900): page src -> page dst in every pool of a group.
// A group's storage is [pools][num_pages][page_bytes]; bytes are moved as 16-byte words.
__global__ void copy_pages_kernel(uint4* __restrict__ base, const int* __restrict__ pairs,
                                  int n_pairs, size_t page_words, size_t pool_words,
                                  int num_pages, int* status) {
    const int pair = blockIdx.x, pool = blockIdx.y;
    if (pair >= n_pairs) return;
    const int src = pairs[2 * pair], dst = pairs[2 * pair + 1];
    if (src < 0 || src >= num_pages || dst < 0 || dst >= num_pages) {
        if (threadIdx.x == 0) prb_set_status(status, PRB_S_PAGE_RANGE, pair, src, dst);
        return;
    }
    const uint4* s = base + pool * pool_words + (size_t)src * page_words;
    uint4* d = base + pool * pool_words + (size_t)dst * page_words;
    for (size_t i = threadIdx.x; i < page_words; i += blockDim.x) d[i] = s[i];
}

PRB_API int prb_copy_pages(void* base, const int* pairs, int n_pairs, long page_bytes,
                           int n_pools, int num_pages, int* status, cudaStream_t stream) {
    if (n_pairs <= 0) return 0;
    if (page_bytes % 16 != 0 || ((uintptr_t)base) % 16 != 0) return PRB_E_ALIGN;
    const size_t page_words = (size_t)page_bytes / 16;
    dim3 grid(n_pairs, n_pools);
    copy_pages_kernel<<<grid, 256, 0, stream>>>((uint4*)base, pairs, n_pairs, page_words,
                                                page_words * (size_t)num_pages, num_pages, status);
    PRB_LAUNCH_CHECK();
    return 0;
}


// ------------------------------------------------------------------ token feedback
// A step that was launched before the step before it had reported its chosen tokens names
// them by place: token id -(k + 1) stands for prev[k], the k-th token the sampling kernel
// chose last.  This kernel puts the ids in (before the step's first kernel reads them).
namespace {
__global__ void resolve_tokens_kernel(int* __restrict__ tokens, int n, const int* __restrict__ prev,
                                      int n_prev, int* status) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= n) return;
    const int v = tokens[t];
    if (v >= 0) return;
    const int k = -v - 1;
    if (k >= n_prev) {
        prb_set_status(status, PRB_S_ROW_RANGE, t, k, n_prev);
        tokens[t] = 0;
        return;
    }
    tokens[t] = prev[k];
}
}  // namespace

// ---------------------------------------------- a step's words in and out without copy engines
// A small step's description (a kilobyte or so) and its result (a few dozen words) cross the
// bus inside kernels, which read and write pinned host memory directly: between a copy and a
// kernel, and more so between two copies, the stream pays microseconds of hand-over that a
// kernel after a kernel does not (measured between two decode steps: sample, 2.3 us, copy out
// 2.6 us, 10.5 us, copy in 1.1 us, 1.7 us, resolve).
//
// prb_fetch_step: dev[i] = host[i] for i < words, and, like prb_resolve_tokens, token ids below
// zero among words [tokens_at, tokens_at + n_tokens) are replaced by prev[-id - 1].
// prb_publish_result: host[i] = dev[i] for i < words, visible to the host once the kernel
// has completed.  Both take the DEVICE address of pinned host memory
// (prb_host_device_address; null if the memory cannot be reached from kernels: the caller
// then copies).
namespace {
// (at most FETCH_PER_THREAD words per thread: the host words are requested before the wait on
// the kernel before, whose chosen ids only the replacement needs)
constexpr int FETCH_THREADS = 256, FETCH_PER_THREAD = 4;
__global__ void __launch_bounds__(FETCH_THREADS)
fetch_step_kernel(int* __restrict__ dev, const int* __restrict__ host, int words,
                  int tokens_at, int n_tokens, const int* __restrict__ prev,
                  int n_prev, int* status) {
    prb_grid_launch_dependents();
    const int first = blockIdx.x * blockDim.x + threadIdx.x, stride = gridDim.x * blockDim.x;
    int v[FETCH_PER_THREAD];
#pragma unroll
    for (int j = 0; j < FETCH_PER_THREAD; ++j) {
        const int i = first + j * stride;
        v[j] = i < words ? host[i] : 0;
    }
    prb_grid_wait();
#pragma unroll
    for (int j = 0; j < FETCH_PER_THREAD; ++j) {
        const int i = first + j * stride;
        if (i >= words) continue;
        int x = v[j];
        if (prev != nullptr && x < 0 && i >= tokens_at && i < tokens_at + n_tokens) {
            const int k = -x - 1;
            if (k >= n_prev) {
                prb_set_status(status, PRB_S_ROW_RANGE, i - tokens_at, k, n_prev);
                x = 0;
            } else {
                x = prev[k];
            }
        }
        dev[i] = x;
    }
}
__global__ void publish_result_kernel(int* __restrict__ host, const int* __restrict__ dev, int words) {
    for (int i = threadIdx.x; i < words; i += blockDim.x) host[i] = dev[i];
}
}  // namespace

PRB_API void* prb_host_device_address(void* host_ptr) {
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, host_ptr) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    if (attr.type != cudaMemoryTypeHost) return nullptr;
    return attr.devicePointer;
}

PRB_API int prb_fetch_step(int* dev, const int* host_dev_address, int words, int tokens_at,
                           int n_tokens, const int* prev, int n_prev, int* status,
                           cudaStream_t stream) {
    if (words <= 0) return 0;
    if (dev == nullptr || host_dev_address == nullptr) return PRB_E_ARG;
    // one word per thread up to 2,048 words (8 blocks); beyond, up to FETCH_PER_THREAD words
    // per thread over 8 blocks or as many as that needs
    int blocks = (words + FETCH_THREADS - 1) / FETCH_THREADS;
    if (blocks > 8) {
        blocks = (words + FETCH_THREADS * FETCH_PER_THREAD - 1) / (FETCH_THREADS * FETCH_PER_THREAD);
        if (blocks < 8) blocks = 8;
    }
    cudaError_t e = prb_launch_dependent(fetch_step_kernel, dim3(blocks), dim3(FETCH_THREADS), 0, stream,
                                         dev, host_dev_address, words, tokens_at, n_tokens, prev,
                                         n_prev, status);
    return e == cudaSuccess ? 0 : (int)e;
}

PRB_API int prb_publish_result(int* host_dev_address, const int* dev, int words, cudaStream_t stream) {
    if (words <= 0) return 0;
    if (dev == nullptr || host_dev_address == nullptr) return PRB_E_ARG;
    publish_result_kernel<<<1, 128, 0, stream>>>(host_dev_address, dev, words);
    PRB_LAUNCH_CHECK();
    return 0;
}

PRB_API int prb_resolve_tokens(int* tokens, int n, const int* prev, int n_prev, int* status,
                               cudaStream_t stream) {
    if (n <= 0) return 0;
    resolve_tokens_kernel<<<(n + 127) / 128, 128, 0, stream>>>(tokens, n, prev, n_prev, status);
    PRB_LAUNCH_CHECK();
    return 0;
}
