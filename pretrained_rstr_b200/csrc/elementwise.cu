// Memory-bound kernels of the step: embedding + position gather, LayerNorm, bias /
// activation / residual epilogue, cache append, page copy.  All statistics and sums in
// 32-bit; element types of tables, activations and the cache are template parameters.
#include "common.cuh"

// Programmatic dependent launch is on unless switched off (for measurements).
static int g_pdl = 1;
int prb_pdl_enabled() { return g_pdl; }
PRB_API void prb_set_pdl(int on) { g_pdl = on ? 1 : 0; }

// ------------------------------------------------------------------ embedding
// x[t,:] = wte[token[t],:] (+ wpe[position[t],:])          (gpt2.clj:49-62)
template <typename W>
__global__ void embed_kernel(float* __restrict__ out, const int* __restrict__ tokens,
                             const int* __restrict__ positions, const W* __restrict__ wte,
                             const W* __restrict__ wpe, int n_tokens, int width, int vocab,
                             int n_positions, int* status) {
    const int t = blockIdx.x;
    if (t >= n_tokens) return;
    const int tok = tokens[t];
    const int pos = positions[t];
    bool ok = true;
    if (tok < 0 || tok >= vocab) {
        if (threadIdx.x == 0) prb_set_status(status, PRB_S_TOKEN_RANGE, t, tok, vocab);
        ok = false;
    }
    if (wpe != nullptr && (pos < 0 || pos >= n_positions)) {
        if (threadIdx.x == 0) prb_set_status(status, PRB_S_POSITION_RANGE, t, pos, n_positions);
        ok = false;
    }
    float* o = out + (size_t)t * width;
    if (!ok) {
        for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = 0.0f;
        return;
    }
    const W* e = wte + (size_t)tok * width;
    if (wpe != nullptr) {
        const W* p = wpe + (size_t)pos * width;
        for (int i = threadIdx.x; i < width; i += blockDim.x)
            o[i] = prb_to_float<W>(e[i]) + prb_to_float<W>(p[i]);
    } else {
        for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = prb_to_float<W>(e[i]);
    }
}

PRB_API int prb_embed(float* out, const int* tokens, const int* positions, const void* wte,
                      const void* wpe, int n_tokens, int width, int vocab, int n_positions,
                      int table_dtype, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (width <= 0 || vocab <= 0) return PRB_E_SIZE;
    const int threads = width >= 256 ? 256 : ((width + 31) / 32) * 32;
    if (table_dtype == PRB_F32)
        embed_kernel<float><<<n_tokens, threads, 0, stream>>>(
            out, tokens, positions, (const float*)wte, (const float*)wpe, n_tokens, width, vocab,
            n_positions, status);
    else if (table_dtype == PRB_BF16)
        embed_kernel<__nv_bfloat16><<<n_tokens, threads, 0, stream>>>(
            out, tokens, positions, (const __nv_bfloat16*)wte, (const __nv_bfloat16*)wpe,
            n_tokens, width, vocab, n_positions, status);
    else
        return PRB_E_DTYPE;
    PRB_LAUNCH_CHECK();
    return 0;
}

// ------------------------------------------------------------------ LayerNorm
// y = (x - mean) / sqrt(var + eps) * gamma + beta, biased variance, per row
// (gpt2.clj:152; formula asr/moonshine.clj:87-104).  Two passes over a row held in
// shared memory; the reduction tree depends on the width only.
// rows: optional gather (out row r reads x row rows[r]).
template <typename O>
__global__ void layernorm_kernel(O* __restrict__ out, const float* __restrict__ x,
                                 const float* __restrict__ gamma, const float* __restrict__ beta,
                                 const int* __restrict__ rows, int n_rows, int n_rows_in,
                                 int width, float eps, int* status) {
    extern __shared__ float row[];
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    if (r >= n_rows) return;
    int src = rows ? rows[r] : r;
    if (src < 0 || src >= n_rows_in) {
        if (threadIdx.x == 0) prb_set_status(status, PRB_S_ROW_RANGE, r, src, n_rows_in);
        for (int i = threadIdx.x; i < width; i += blockDim.x)
            out[(size_t)r * width + i] = prb_from_float<O>(0.0f);
        return;
    }
    const float* xr = x + (size_t)src * width;
    float s = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = xr[i];
        row[i] = v;
        s += v;
    }
    const float mean = prb_block_sum(s, scratch) / (float)width;
    float q = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float c = row[i] - mean;
        q += c * c;
    }
    const float var = prb_block_sum(q, scratch) / (float)width;
    const float inv = 1.0f / sqrtf(var + eps);
    O* o = out + (size_t)r * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float y = (row[i] - mean) * inv * gamma[i] + (beta ? beta[i] : 0.0f);
        o[i] = prb_from_float<O>(y);
    }
}

PRB_API int prb_layernorm(void* out, const float* x, const float* gamma, const float* beta,
                          const int* rows, int n_rows, int n_rows_in, int width, float eps,
                          int out_dtype, int* status, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (width <= 0 || (size_t)width * 4 > 200 * 1024) return PRB_E_SIZE;
    const int threads = width >= 256 ? 256 : ((width + 31) / 32) * 32;
    const size_t smem = (size_t)width * sizeof(float);
    if (out_dtype == PRB_F32) {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(layernorm_kernel<float>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        layernorm_kernel<float><<<n_rows, threads, smem, stream>>>(
            (float*)out, x, gamma, beta, rows, n_rows, n_rows_in, width, eps, status);
    } else if (out_dtype == PRB_BF16) {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(layernorm_kernel<__nv_bfloat16>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        layernorm_kernel<__nv_bfloat16><<<n_rows, threads, smem, stream>>>(
            (__nv_bfloat16*)out, x, gamma, beta, rows, n_rows, n_rows_in, width, eps, status);
    } else {
        return PRB_E_DTYPE;
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
// New keys and values of the step go to their slots (paged_append.clj:44-57: slot =
// page * page_size + offset; -1 = skip).  Page layout: [page][kv head][offset][head dim].
template <typename T>
__global__ void kv_append_kernel(T* __restrict__ k_pages, T* __restrict__ v_pages,
                                 const T* __restrict__ k_src, const T* __restrict__ v_src,
                                 long src_stride, const int* __restrict__ slots, int n_tokens,
                                 int kv_heads, int head_dim, int page_size, int num_pages,
                                 int* status) {
    prb_grid_launch_dependents();
    prb_grid_wait();
    const int t = blockIdx.x;
    if (t >= n_tokens) return;
    const int slot = slots[t];
    if (slot < 0) return;
    const int page = slot / page_size, off = slot - page * page_size;
    if (page >= num_pages) {
        if (threadIdx.x == 0) prb_set_status(status, PRB_S_SLOT_RANGE, t, slot, num_pages);
        return;
    }
    const int row = kv_heads * head_dim;
    for (int i = threadIdx.x; i < row; i += blockDim.x) {
        const int h = i / head_dim, d = i - h * head_dim;
        const size_t dst = (((size_t)page * kv_heads + h) * page_size + off) * head_dim + d;
        k_pages[dst] = k_src[(size_t)t * src_stride + i];
        v_pages[dst] = v_src[(size_t)t * src_stride + i];
    }
}

PRB_API int prb_kv_append(void* k_pages, void* v_pages, const void* k_src, const void* v_src,
                          long src_stride, const int* slots, int n_tokens, int kv_heads,
                          int head_dim, int page_size, int num_pages, int dtype, int* status,
                          cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (kv_heads <= 0 || head_dim <= 0 || page_size <= 0) return PRB_E_SIZE;
    const int row = kv_heads * head_dim;
    const int threads = row >= 256 ? 256 : ((row + 31) / 32) * 32;
    cudaError_t e;
    if (dtype == PRB_F32)
        e = prb_launch_dependent(kv_append_kernel<float>, dim3(n_tokens), dim3(threads), 0, stream,
                                 (float*)k_pages, (float*)v_pages, (const float*)k_src,
                                 (const float*)v_src, src_stride, slots, n_tokens, kv_heads,
                                 head_dim, page_size, num_pages, status);
    else if (dtype == PRB_BF16)
        e = prb_launch_dependent(kv_append_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), 0,
                                 stream, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages,
                                 (const __nv_bfloat16*)k_src, (const __nv_bfloat16*)v_src,
                                 src_stride, slots, n_tokens, kv_heads, head_dim, page_size,
                                 num_pages, status);
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
