// Token choice from 32-bit logits rows: greedy, or top-k -> temperature softmax ->
// nucleus cut -> multinomial draw, in the order of the reference's sampler
// (src/pretrained/sampling.clj:31-64).  One block per row.
//
// Greedy: the first maximum wins, so ties go to the lowest id, and a NaN wins over
// every number (gpt2.clj:264-270; decoder_gpu.clj:68-70).
//
// Sampling: the k candidates are found in descending order (equal logits: lower id
// first, as sampling.clj:14-29 leaves them), then one thread does the remaining
// arithmetic in double precision and in the reference's order of operations.  Draws
// come from a per-request 48-bit linear congruential generator with the constants of
// java.util.Random (sampling.clj:43, 61 draws from java.util.Random(seed)); its state
// lives in the request's state slot, so a request's draws do not depend on the batch.
#include "common.cuh"

namespace {
constexpr int SAMPLE_THREADS = 1024;
constexpr int MAX_TOP_K = 1024;

struct Best {
    float v;
    int i;
};

// order: NaN first, then larger value, then lower index
__device__ __forceinline__ bool better(float v, int i, float bv, int bi) {
    if (bi < 0) return true;
    const bool vn = isnan(v), bn = isnan(bv);
    if (vn || bn) return vn && (!bn || i < bi);
    return v > bv || (v == bv && i < bi);
}

__device__ __forceinline__ Best block_best(Best b, Best* sh) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, b.v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, b.i, o);
        if (oi >= 0 && better(ov, oi, b.v, b.i)) { b.v = ov; b.i = oi; }
    }
    __syncthreads();
    if (lane == 0) sh[warp] = b;
    __syncthreads();
    Best r = (lane < (int)(blockDim.x >> 5)) ? sh[lane] : Best{0.0f, -1};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, r.v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, r.i, o);
        if (oi >= 0 && better(ov, oi, r.v, r.i)) { r.v = ov; r.i = oi; }
    }
    return r;   // identical in every thread of every warp
}

__device__ __forceinline__ unsigned long long lcg_next(unsigned long long* s, int bits) {
    *s = (*s * 0x5DEECE66DULL + 0xBULL) & ((1ULL << 48) - 1);
    return *s >> (48 - bits);
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(int* __restrict__ out, const float* __restrict__ logits, long row_stride, int vocab,
              const float* __restrict__ temperature, const int* __restrict__ top_k,
              const float* __restrict__ top_p, const long long* __restrict__ seeds,
              const int* __restrict__ fresh, const int* __restrict__ slots,
              unsigned long long* __restrict__ rng_states, int n_rows) {
    __shared__ Best sh[32];
    __shared__ int cand_id[MAX_TOP_K];
    __shared__ float cand_v[MAX_TOP_K];
    const int r = blockIdx.x;
    if (r >= n_rows) return;
    const float* row = logits + (size_t)r * row_stride;
    const float temp = temperature ? temperature[r] : 0.0f;

    if (!(temp > 0.0f)) {
        Best b{0.0f, -1};
        const int bd = blockDim.x;
        for (int i = threadIdx.x; i < vocab; i += 4 * bd) {        // four loads in flight
            const int i1 = i + bd, i2 = i + 2 * bd, i3 = i + 3 * bd;
            const float v0 = row[i];
            const float v1 = i1 < vocab ? row[i1] : 0.0f;
            const float v2 = i2 < vocab ? row[i2] : 0.0f;
            const float v3 = i3 < vocab ? row[i3] : 0.0f;
            if (better(v0, i, b.v, b.i)) { b.v = v0; b.i = i; }
            if (i1 < vocab && better(v1, i1, b.v, b.i)) { b.v = v1; b.i = i1; }
            if (i2 < vocab && better(v2, i2, b.v, b.i)) { b.v = v2; b.i = i2; }
            if (i3 < vocab && better(v3, i3, b.v, b.i)) { b.v = v3; b.i = i3; }
        }
        b = block_best(b, sh);
        if (threadIdx.x == 0) out[r] = b.i;
        return;
    }

    int k = top_k[r];
    if (k > vocab) k = vocab;
    if (k > MAX_TOP_K) k = MAX_TOP_K;
    if (k < 1) k = 1;
    // k rounds: the best element that comes after the previous pick in (value desc, id asc)
    float pv = 0.0f;
    int pi = -1;
    for (int round = 0; round < k; ++round) {
        Best b{0.0f, -1};
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
            float v = row[i];
            if (isnan(v)) v = -INFINITY;
            if (pi >= 0 && !(v < pv || (v == pv && i > pi))) continue;
            if (b.i < 0 || v > b.v || (v == b.v && i < b.i)) { b.v = v; b.i = i; }
        }
        b = block_best(b, sh);
        if (threadIdx.x == 0) { cand_id[round] = b.i; cand_v[round] = b.v; }
        pv = b.v;
        pi = b.i;
        if (pi < 0) { k = round; break; }
    }
    __syncthreads();
    if (threadIdx.x != 0) return;
    if (k == 0) { out[r] = 0; return; }

    const double t = (double)temp;
    const double p = (double)top_p[r];
    const double mx = (double)cand_v[0] / t;
    // probabilities are recomputed where needed instead of stored: k <= 1024 exps
    double psum = 0.0;
    for (int j = 0; j < k; ++j) psum += exp((double)cand_v[j] / t - mx);
    int cut = k;
    double c = 0.0;
    for (int j = 0; j < k; ++j) {
        c += exp((double)cand_v[j] / t - mx) / psum;
        if (c >= p) { cut = j + 1; break; }
    }
    double tot = 0.0;
    for (int j = 0; j < cut; ++j) tot += exp((double)cand_v[j] / t - mx);

    unsigned long long* state = rng_states + slots[r];
    unsigned long long s = *state;
    if (fresh[r]) s = ((unsigned long long)seeds[r] ^ 0x5DEECE66DULL) & ((1ULL << 48) - 1);
    const unsigned long long hi = lcg_next(&s, 26), lo = lcg_next(&s, 27);
    *state = s;
    const double u = (double)((hi << 27) + lo) * (1.0 / 9007199254740992.0);
    const double draw = u * tot;
    double acc = 0.0;
    int pick = cand_id[cut - 1];
    for (int j = 0; j < cut; ++j) {
        acc += exp((double)cand_v[j] / t - mx);
        if (acc >= draw || j == cut - 1) { pick = cand_id[j]; break; }
    }
    out[r] = pick;
}
}  // namespace

PRB_API int prb_sample_max_top_k() { return MAX_TOP_K; }

// temperature == nullptr: every row is greedy and the remaining pointers are unused.
PRB_API int prb_sample(int* out, const float* logits, long row_stride, int vocab,
                       const float* temperature, const int* top_k, const float* top_p,
                       const long long* seeds, const int* fresh, const int* slots,
                       unsigned long long* rng_states, int n_rows, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (vocab <= 0) return PRB_E_SIZE;
    sample_kernel<<<n_rows, SAMPLE_THREADS, 0, stream>>>(out, logits, row_stride, vocab,
                                                         temperature, top_k, top_p, seeds, fresh,
                                                         slots, rng_states, n_rows);
    PRB_LAUNCH_CHECK();
    return 0;
}
