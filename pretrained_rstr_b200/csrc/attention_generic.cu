// Attention over the paged cache, any sizes, 32-bit arithmetic throughout: the kernel of
// the true 32-bit path, and the plain twin the tensor-core kernels are checked against.
//
// One block per (token, query head).  Token t of request b at position p sees the keys
// at positions lo..p of the same request (lo = 0, or p - window + 1 with a window),
// found through the request's block table:
//     s_j = (q . k_j) * scale;  w_j = exp(s_j - max s);  out = sum_j w_j v_j / sum_j w_j
// (scale: decoder.clj:56; visibility: paged_decoder.clj:166-177; 32-bit accumulators:
// paged_attention.clj:225).  Reduction orders depend on (p - lo, head size) only, never
// on what else is in the batch.
#include "common.cuh"

namespace {
constexpr int ATT_THREADS = 128;

template <typename T>
__global__ void __launch_bounds__(ATT_THREADS)
attention_generic_kernel(T* __restrict__ out, long out_stride, const T* __restrict__ q,
                         long q_stride, const T* __restrict__ k_pages,
                         const T* __restrict__ v_pages, const int* __restrict__ block_table,
                         const int* __restrict__ seq_of_token, const int* __restrict__ positions,
                         int n_tokens, int n_heads, int kv_heads, int head_dim, int page_size,
                         int max_pages, int num_pages, int max_context, float scale, int window,
                         int* status) {
    extern __shared__ float smem[];
    __shared__ float scratch[32];
    float* qs = smem;                       // [head_dim]
    float* part = smem + head_dim;          // [ATT_THREADS] partial outputs
    float* scores = part + ATT_THREADS;     // [max_context]

    const int t = blockIdx.x, h = blockIdx.y;
    if (t >= n_tokens) return;
    const int b = seq_of_token[t];
    const int pos = positions[t];
    T* o = out + (size_t)t * out_stride + (size_t)h * head_dim;
    if (b < 0) {                            // padding token
        for (int d = threadIdx.x; d < head_dim; d += blockDim.x) o[d] = prb_from_float<T>(0.0f);
        return;
    }
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int n = pos - lo + 1;
    if (pos < 0 || n > max_context || pos >= max_pages * page_size) {
        if (threadIdx.x == 0) prb_set_status(status, PRB_S_POSITION_RANGE, t, pos, max_context);
        for (int d = threadIdx.x; d < head_dim; d += blockDim.x) o[d] = prb_from_float<T>(0.0f);
        return;
    }
    const int hk = h / (n_heads / kv_heads);
    const int* table = block_table + (size_t)b * max_pages;
    const T* qp = q + (size_t)t * q_stride + (size_t)h * head_dim;
    for (int d = threadIdx.x; d < head_dim; d += blockDim.x) qs[d] = prb_to_float<T>(qp[d]);
    __syncthreads();

    // scores
    float mx = -INFINITY;
    bool bad = false;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int j = lo + i;
        const int page = table[j / page_size];
        float s = -INFINITY;
        if (page < 0 || page >= num_pages) {
            bad = true;
            prb_set_status(status, PRB_S_PAGE_RANGE, t, j, page);
        } else {
            const T* kp = k_pages +
                (((size_t)page * kv_heads + hk) * page_size + (j % page_size)) * head_dim;
            float acc = 0.0f;
            for (int d = 0; d < head_dim; ++d) acc = fmaf(qs[d], prb_to_float<T>(kp[d]), acc);
            s = acc * scale;
        }
        scores[i] = s;
        mx = fmaxf(mx, s);
    }
    mx = prb_block_max(mx, scratch);
    float sum = 0.0f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float s = scores[i];
        const float w = (s == -INFINITY) ? 0.0f : expf(s - mx);
        scores[i] = w;
        sum += w;
    }
    sum = prb_block_sum(sum, scratch);     // also orders the writes to scores[]
    __syncthreads();
    (void)bad;

    // weighted values: thread (g, d) sums keys i = g, g + G, ... for dimension d
    const int dpad = head_dim;             // threads per key group
    const int groups = ATT_THREADS / dpad > 0 ? ATT_THREADS / dpad : 1;
    for (int d0 = 0; d0 < head_dim; d0 += ATT_THREADS) {
        const int d = d0 + (threadIdx.x % (dpad < ATT_THREADS ? dpad : ATT_THREADS));
        const int g = (dpad < ATT_THREADS) ? threadIdx.x / dpad : 0;
        float acc = 0.0f;
        if (d < head_dim && g < groups) {
            for (int i = g; i < n; i += groups) {
                const float w = scores[i];
                if (w != 0.0f) {
                    const int j = lo + i;
                    const int page = table[j / page_size];
                    const T* vp = v_pages +
                        (((size_t)page * kv_heads + hk) * page_size + (j % page_size)) * head_dim;
                    acc = fmaf(w, prb_to_float<T>(vp[d]), acc);
                }
            }
        }
        part[threadIdx.x] = acc;
        __syncthreads();
        if (d < head_dim && g == 0) {
            float total = 0.0f;
            for (int gg = 0; gg < groups; ++gg) {
                const int idx = gg * dpad + (d - d0);
                if (idx < ATT_THREADS) total += part[idx];
            }
            o[d] = prb_from_float<T>(sum > 0.0f ? total / sum : 0.0f);
        }
        __syncthreads();
    }
}
}  // namespace

PRB_API int prb_attention_generic(void* out, long out_stride, const void* q, long q_stride,
                                  const void* k_pages, const void* v_pages,
                                  const int* block_table, const int* seq_of_token,
                                  const int* positions, int n_tokens, int n_heads, int kv_heads,
                                  int head_dim, int page_size, int max_pages, int num_pages,
                                  int max_context, float scale, int window, int dtype,
                                  int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (n_heads <= 0 || kv_heads <= 0 || n_heads % kv_heads != 0 || head_dim <= 0 ||
        page_size <= 0 || max_pages <= 0 || max_context <= 0)
        return PRB_E_SIZE;
    if (n_heads > 65535) return PRB_E_SIZE;
    const size_t smem = (size_t)(head_dim + ATT_THREADS + max_context) * sizeof(float);
    if (smem > 200 * 1024) return PRB_E_SIZE;
    dim3 grid(n_tokens, n_heads);
    if (dtype == PRB_F32) {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(attention_generic_kernel<float>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        attention_generic_kernel<float><<<grid, ATT_THREADS, smem, stream>>>(
            (float*)out, out_stride, (const float*)q, q_stride, (const float*)k_pages,
            (const float*)v_pages, block_table, seq_of_token, positions, n_tokens, n_heads,
            kv_heads, head_dim, page_size, max_pages, num_pages, max_context, scale, window, status);
    } else if (dtype == PRB_BF16) {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(attention_generic_kernel<__nv_bfloat16>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        attention_generic_kernel<__nv_bfloat16><<<grid, ATT_THREADS, smem, stream>>>(
            (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)q, q_stride,
            (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages, block_table,
            seq_of_token, positions, n_tokens, n_heads, kv_heads, head_dim, page_size, max_pages,
            num_pages, max_context, scale, window, status);
    } else {
        return PRB_E_DTYPE;
    }
    PRB_LAUNCH_CHECK();
    return 0;
}
