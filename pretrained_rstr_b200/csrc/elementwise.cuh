// Units of work of the memory-bound kernels (elementwise.cu) as device functions.
#pragma once
#include "common.cuh"

namespace elementwise {

struct EmbedArgs {
    float* out;
    const int* tokens;
    const int* positions;
    const void* wte;
    const void* wpe;
    int n_tokens, width, vocab, n_positions;
    int* status;
};

// x[t,:] = wte[token[t],:] (+ wpe[position[t],:])          (gpt2.clj:49-62)
template <typename W>
__device__ __forceinline__ void embed_token(const EmbedArgs& a, int t) {
    if (t >= a.n_tokens) return;
    const W* wte = reinterpret_cast<const W*>(a.wte);
    const W* wpe = reinterpret_cast<const W*>(a.wpe);
    const int tok = a.tokens[t];
    const int pos = a.positions[t];
    bool ok = true;
    if (tok < 0 || tok >= a.vocab) {
        if (threadIdx.x == 0) prb_set_status(a.status, PRB_S_TOKEN_RANGE, t, tok, a.vocab);
        ok = false;
    }
    if (wpe != nullptr && (pos < 0 || pos >= a.n_positions)) {
        if (threadIdx.x == 0) prb_set_status(a.status, PRB_S_POSITION_RANGE, t, pos, a.n_positions);
        ok = false;
    }
    float* o = a.out + (size_t)t * a.width;
    if (!ok) {
        for (int i = threadIdx.x; i < a.width; i += blockDim.x) o[i] = 0.0f;
        return;
    }
    const W* e = wte + (size_t)tok * a.width;
    if (wpe != nullptr) {
        const W* p = wpe + (size_t)pos * a.width;
        for (int i = threadIdx.x; i < a.width; i += blockDim.x)
            o[i] = prb_to_float<W>(e[i]) + prb_to_float<W>(p[i]);
    } else {
        for (int i = threadIdx.x; i < a.width; i += blockDim.x) o[i] = prb_to_float<W>(e[i]);
    }
}

struct NormArgs {
    void* out;
    const float* x;
    const float* gamma;
    const float* beta;
    const int* rows;
    int n_rows, n_rows_in, width;
    float eps;
    int* status;
};

// y = (x - mean) / sqrt(var + eps) * gamma + beta, biased variance, one row
// (gpt2.clj:152; formula asr/moonshine.clj:87-104).  Two passes over the row held in
// shared memory (`row`: width floats, `scratch`: 32 floats); the reduction tree depends
// on the width and the block size only.  Reached by all threads of the CTA.
template <typename O>
__device__ __forceinline__ void layernorm_row(const NormArgs& a, int r, float* row, float* scratch) {
    if (r >= a.n_rows) return;
    O* out = reinterpret_cast<O*>(a.out);
    const int width = a.width;
    int src = a.rows ? a.rows[r] : r;
    if (src < 0 || src >= a.n_rows_in) {
        if (threadIdx.x == 0) prb_set_status(a.status, PRB_S_ROW_RANGE, r, src, a.n_rows_in);
        for (int i = threadIdx.x; i < width; i += blockDim.x)
            out[(size_t)r * width + i] = prb_from_float<O>(0.0f);
        return;
    }
    const float* xr = a.x + (size_t)src * width;
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
    const float inv = 1.0f / sqrtf(var + a.eps);
    O* o = out + (size_t)r * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float y = (row[i] - mean) * inv * a.gamma[i] + (a.beta ? a.beta[i] : 0.0f);
        o[i] = prb_from_float<O>(y);
    }
}

struct AppendArgs {
    void* k_pages;
    void* v_pages;
    const void* k_src;
    const void* v_src;
    long src_stride;
    const int* slots;
    int n_tokens, kv_heads, head_dim, page_size, num_pages;
    int* status;
};

// New keys and values of the step go to their slots (paged_append.clj:44-57: slot =
// page * page_size + offset; -1 = skip).  Page layout: [page][kv head][offset][head dim].
template <typename T>
__device__ __forceinline__ void append_token(const AppendArgs& a, int t) {
    if (t >= a.n_tokens) return;
    const int slot = a.slots[t];
    if (slot < 0) return;
    const int page = slot / a.page_size, off = slot - page * a.page_size;
    if (page >= a.num_pages) {
        if (threadIdx.x == 0) prb_set_status(a.status, PRB_S_SLOT_RANGE, t, slot, a.num_pages);
        return;
    }
    T* k_pages = reinterpret_cast<T*>(a.k_pages);
    T* v_pages = reinterpret_cast<T*>(a.v_pages);
    const T* k_src = reinterpret_cast<const T*>(a.k_src);
    const T* v_src = reinterpret_cast<const T*>(a.v_src);
    const int rowlen = a.kv_heads * a.head_dim;
    for (int i = threadIdx.x; i < rowlen; i += blockDim.x) {
        const int h = i / a.head_dim, d = i - h * a.head_dim;
        const size_t dst = (((size_t)page * a.kv_heads + h) * a.page_size + off) * a.head_dim + d;
        k_pages[dst] = k_src[(size_t)t * a.src_stride + i];
        v_pages[dst] = v_src[(size_t)t * a.src_stride + i];
    }
}
}  // namespace elementwise
