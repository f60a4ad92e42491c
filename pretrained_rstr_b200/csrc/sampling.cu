// Token choice from 32-bit logits rows: greedy, or top-k -> temperature softmax ->
// nucleus cut -> multinomial draw, in the order of the reference's sampler
// (src/pretrained/sampling.clj:31-64).  One block per row.
//
// Greedy: the first maximum wins, so ties go to the lowest id, and a NaN wins over
// every number (gpt2.clj:264-270; decoder_gpu.clj:68-70).
//
// Sampling: the k largest logits are selected in a few passes over the row, whatever k is:
// a radix select on an order-preserving 32-bit key (three passes of 11, 11 and 10 bits with
// shared-memory histograms) finds the key of the k-th largest logit, one more pass collects
// everything above it and, of the logits equal to it, the lowest ids; the candidates are
// then sorted (larger logit first, equal logits: lower id first, as sampling.clj:14-29
// leaves them) by a bitonic sort in shared memory.  The exponentials are computed one per
// thread in double precision; one thread then does the sums, the nucleus cut and the draw
// in the reference's order of operations.  Draws come from a per-request 48-bit linear
// congruential generator with the constants of java.util.Random (sampling.clj:43, 61 draws
// from java.util.Random(seed)); its state lives in the request's state slot, so a request's
// draws do not depend on the batch.  A NaN or -infinity logit counts as a candidate of weight
// zero (the reference's search skips it and leaves its candidate slot at id 0; the two differ
// only when k exceeds the number of finite logits of a row).
#include <cstdlib>

#include "common.cuh"

namespace {
constexpr int SAMPLE_THREADS = 1024;
constexpr int MAX_TOP_K = 1024;
constexpr int HIST_COPIES = 4;        // private copies of the histogram (fewer collisions)
constexpr int CAND_CAP = 4096;        // candidates the fast path sorts (8 bytes each)
static_assert(CAND_CAP * 8 >= HIST_COPIES * 2048 * 4, "the histograms share the candidates' memory");

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

// Order-preserving key of a logit: larger logit, larger key.  NaN counts as -infinity (as in
// the candidate search of the reference's sampler a NaN never beats a number) and -0 as +0.
__device__ __forceinline__ unsigned sample_key(float v) {
    if (isnan(v)) v = -INFINITY;
    v += 0.0f;
    const unsigned u = __float_as_uint(v);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float sample_value(unsigned key) {
    return __uint_as_float((key & 0x80000000u) ? (key & 0x7fffffffu) : ~key);
}

// Visit every logit of a row once: f(index, value).  The row's start need not be aligned
// (rows of an odd vocabulary are not): up to three leading elements and the tail are read one
// by one, the rest as 16-byte loads, four of them in flight per thread, because what such a
// pass costs is the round trips to the L2, not the bytes.
template <typename F>
__device__ __forceinline__ void for_each_logit(const float* __restrict__ row, int vocab, F f) {
    const int head = min(vocab, (int)((4u - (unsigned)(((uintptr_t)row >> 2) & 3u)) & 3u));
    const int nvec = (vocab - head) >> 2;
    const int tail0 = head + 4 * nvec;
    if ((int)threadIdx.x < head) f((int)threadIdx.x, row[threadIdx.x]);
    if ((int)threadIdx.x < vocab - tail0) f(tail0 + (int)threadIdx.x, row[tail0 + threadIdx.x]);
    const float4* vec = reinterpret_cast<const float4*>(row + head);
    const int bd = blockDim.x;
    for (int j = threadIdx.x; j < nvec; j += 4 * bd) {
        const int j1 = j + bd, j2 = j + 2 * bd, j3 = j + 3 * bd;
        const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
        const float4 v0 = vec[j];
        const float4 v1 = j1 < nvec ? vec[j1] : z;
        const float4 v2 = j2 < nvec ? vec[j2] : z;
        const float4 v3 = j3 < nvec ? vec[j3] : z;
        const int b0 = head + 4 * j;
        f(b0, v0.x); f(b0 + 1, v0.y); f(b0 + 2, v0.z); f(b0 + 3, v0.w);
        if (j1 < nvec) { const int b = head + 4 * j1; f(b, v1.x); f(b + 1, v1.y); f(b + 2, v1.z); f(b + 3, v1.w); }
        if (j2 < nvec) { const int b = head + 4 * j2; f(b, v2.x); f(b + 1, v2.y); f(b + 2, v2.z); f(b + 3, v2.w); }
        if (j3 < nvec) { const int b = head + 4 * j3; f(b, v3.x); f(b + 1, v3.y); f(b + 2, v3.z); f(b + 3, v3.w); }
    }
}

__device__ __forceinline__ unsigned long long lcg_next(unsigned long long* s, int bits) {
    *s = (*s * 0x5DEECE66DULL + 0xBULL) & ((1ULL << 48) - 1);
    return *s >> (48 - bits);
}

// What a CTA that samples a row keeps in shared memory.
struct SampleShared {
    Best best[32];
    // histograms of the exact selection; else the candidates (64-bit sort keys: the logit's
    // order-preserving key above, 0x7fffffff - id below, so that one compare orders by larger
    // logit first, then lower id) and, behind them, their exponentials
    alignas(16) unsigned char work[CAND_CAP * sizeof(unsigned long long) + MAX_TOP_K * sizeof(double)];
    int pick[8];          // [0..2] radix select, [3..4] its collect counters, [5] candidates, [6] bound
    int warp_count[32];
    double psum;
    int ids[MAX_TOP_K];
    int last;
};

__device__ __forceinline__ int clamp_top_k(int k, int vocab) {
    if (k > vocab) k = vocab;
    if (k > MAX_TOP_K) k = MAX_TOP_K;
    return k < 1 ? 1 : k;
}
__device__ __forceinline__ unsigned long long candidate(unsigned key, int id) {
    return ((unsigned long long)key << 32) | (unsigned)(0x7fffffff - id);
}

// Bitonic sort of cand[0, count) in shared memory: larger key first, equal keys: lower id
// first (one 64-bit compare does both); entries beyond `count` are padded below every key.
__device__ __forceinline__ void sort_descending(unsigned long long* cand, int count) {
    int n2 = 1;
    while (n2 < count) n2 <<= 1;
    __syncthreads();
    for (int i = count + threadIdx.x; i < n2; i += blockDim.x) cand[i] = 0ULL;
    __syncthreads();
    for (int size = 2; size <= n2; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            for (int i = threadIdx.x; i < n2 / 2; i += blockDim.x) {
                const int lo = 2 * i - (i & (stride - 1));      // pairs (lo, lo + stride)
                const int hi = lo + stride;
                const bool descending = (lo & size) == 0;
                const unsigned long long x = cand[lo], y = cand[hi];
                if ((x < y) == descending) { cand[lo] = y; cand[hi] = x; }
            }
            __syncthreads();
        }
    }
}

// Order cand[0, count) (larger key first, equal keys: lower id first) by counting, for every
// entry, the entries that come before it: no barriers inside, `count` broadcast reads per
// entry.  The ordered entries go to `sorted` (another part of shared memory).
__device__ __forceinline__ void rank_sort(const unsigned long long* cand, int count,
                                          unsigned long long* sorted) {
    __syncthreads();
    for (int t = threadIdx.x; t < count; t += blockDim.x) {
        const unsigned long long mine = cand[t];
        int before = 0;
        for (int j = 0; j < count; ++j) before += cand[j] > mine ? 1 : 0;
        sorted[before] = mine;                                 // entries are distinct
    }
    __syncthreads();
}

// Too many logits at or above the bound (long runs of equal logits, a large k): the exact key
// of the k-th largest by radix select over the whole row, then exactly k candidates in
// cand[0, k).  By all threads of the CTA.
__device__ __forceinline__ void select_exactly(SampleShared& ss, const float* __restrict__ row,
                                               int vocab, int k) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    unsigned long long* cand = reinterpret_cast<unsigned long long*>(ss.work);
    int* pick_sh = ss.pick;
    int* warp_count = ss.warp_count;
    __syncthreads();
    // ---- the key of the k-th largest logit, most significant bits first
    unsigned* hist = reinterpret_cast<unsigned*>(ss.work);               // [HIST_COPIES][2048]
    unsigned prefix = 0u, decided = 0u;
    int need = k;                        // how many of the logits under the current prefix are taken
    unsigned equal_count = 0u;           // logits whose key equals the k-th largest's
#pragma unroll 1
    for (int pass = 0; pass < 3; ++pass) {
        const int shift = pass == 0 ? 21 : pass == 1 ? 10 : 0;
        const unsigned bins = pass == 2 ? 1024u : 2048u;
        for (unsigned i = threadIdx.x; i < HIST_COPIES * 2048u; i += blockDim.x) hist[i] = 0u;
        __syncthreads();
        unsigned* mine = hist + (warp % HIST_COPIES) * 2048;
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
            const unsigned key = sample_key(row[i]);
            if ((key & decided) == prefix) atomicAdd(&mine[(key >> shift) & (bins - 1u)], 1u);
        }
        __syncthreads();
        for (unsigned i = threadIdx.x; i < bins; i += blockDim.x) {
            unsigned c = hist[i];
#pragma unroll
            for (int j = 1; j < HIST_COPIES; ++j) c += hist[j * 2048 + i];
            hist[i] = c;
        }
        __syncthreads();
        if (warp == 0) {
            // lane l owns bins [hi - per, hi) counted from the top; find where the count of
            // larger keys passes `need`
            const int per = (int)bins / 32;
            const int top = (int)bins - lane * per;             // exclusive upper bin of this lane
            unsigned mine_sum = 0u;
            for (int j = 1; j <= per; ++j) mine_sum += hist[top - j];
            unsigned incl = mine_sum;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const unsigned v = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += v;
            }
            const unsigned above = incl - mine_sum;             // keys in bins above this lane's
            if (above < (unsigned)need && incl >= (unsigned)need) {
                unsigned seen = above;
                for (int j = 1; j <= per; ++j) {
                    const unsigned c = hist[top - j];
                    if (seen + c >= (unsigned)need) {
                        pick_sh[0] = top - j;                   // the bin of the k-th largest
                        pick_sh[1] = need - (int)seen;          // still to take inside it
                        pick_sh[2] = (int)c;
                        break;
                    }
                    seen += c;
                }
            }
        }
        __syncthreads();
        prefix |= (unsigned)pick_sh[0] << shift;
        decided |= (bins - 1u) << shift;
        need = pick_sh[1];
        equal_count = (unsigned)pick_sh[2];
        __syncthreads();
    }
    const unsigned kth = prefix;                       // key of the k-th largest logit
    const int n_greater = k - need;                    // logits strictly above it

    // ---- collect: everything above, and `need` of the equal ones, lowest ids first
    __syncthreads();
    if (threadIdx.x == 0) { pick_sh[3] = 0; pick_sh[4] = 0; }
    __syncthreads();
    const bool all_equal_taken = equal_count == (unsigned)need;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const unsigned key = sample_key(row[i]);
        if (key > kth) {
            const int slot = atomicAdd(&pick_sh[3], 1);
            cand[slot] = candidate(key, i);
        } else if (key == kth && all_equal_taken) {
            const int slot = n_greater + atomicAdd(&pick_sh[4], 1);
            cand[slot] = candidate(key, i);
        }
    }
    if (!all_equal_taken) {
        // more equal logits than are wanted: the lowest ids, found in id order
        int base = 0;
        for (int start = 0; start < vocab && base < need; start += blockDim.x) {
            const int i = start + threadIdx.x;
            const bool hit = i < vocab && sample_key(row[i]) == kth;
            const unsigned ballot = __ballot_sync(0xffffffffu, hit);
            if (lane == 0) warp_count[warp] = __popc(ballot);
            __syncthreads();
            int before = 0, total = 0;
            for (int w = 0; w < (int)(blockDim.x >> 5); ++w) {
                const int c = warp_count[w];
                if (w < warp) before += c;
                total += c;
            }
            const int rank = base + before + __popc(ballot & ((1u << lane) - 1u));
            if (hit && rank < need) cand[n_greater + rank] = candidate(kth, i);
            base += total;
            __syncthreads();
        }
    }
}

// From n_cand candidates in cand[0, n_cand) (all of the k largest among them) to the row's
// token: order them, exponentials, sums, nucleus cut, draw.  By all threads of the CTA, which
// come back at different places (thread 0 last, after it has stored out[r]).
__device__ __forceinline__ void
finish_row(SampleShared& ss, int n_cand, int k, float temp, int r, int* __restrict__ out,
           const float* __restrict__ top_p, const long long* __restrict__ seeds,
           const int* __restrict__ fresh, const int* __restrict__ slots,
           unsigned long long* __restrict__ rng_states) {
    unsigned long long* cand = reinterpret_cast<unsigned long long*>(ss.work);
    // ---- order the candidates
    // (few candidates: by counting ranks, no barriers; many: a bitonic sort, whose work grows
    // with n log^2 n instead of n^2)
    unsigned long long* sorted = cand + CAND_CAP / 2;               // second half of the buffer
    if (n_cand <= 256) {
        rank_sort(cand, n_cand, sorted);
    } else {
        sort_descending(cand, n_cand);
        sorted = cand;
    }
    __syncthreads();
    double* e = reinterpret_cast<double*>(ss.work + CAND_CAP * sizeof(unsigned long long));     // [MAX_TOP_K]
    const double t = (double)temp;
    {
        const double mx = (double)sample_value((unsigned)(sorted[0] >> 32)) / t;
        for (int j = threadIdx.x; j < k; j += blockDim.x)
            e[j] = exp((double)sample_value((unsigned)(sorted[j] >> 32)) / t - mx);
    }
    __syncthreads();
    // The sums are the reference's, term by term in its order (one thread); what does not
    // depend on the order is done by all: the quotients e / sum.  The sum of the first `cut`
    // terms and the running sum of the draw are partial sums of the same series, so they are
    // kept from the first loop instead of being added up again.
    double* part = reinterpret_cast<double*>(ss.work);   // [k] partial sums (the candidates' keys are
    int* ids_sh = ss.ids;                                //      not needed any more: ids are kept here)
    for (int j = threadIdx.x; j < k; j += blockDim.x)
        ids_sh[j] = 0x7fffffff - (int)(unsigned)(sorted[j] & 0xffffffffULL);
    __syncthreads();
    if (threadIdx.x == 0) {
        double acc0 = 0.0;
        for (int j = 0; j < k; ++j) { acc0 += e[j]; part[j] = acc0; }
        ss.psum = acc0;
    }
    __syncthreads();
    const double psum = ss.psum;
    for (int j = threadIdx.x; j < k; j += blockDim.x) e[j] = e[j] / psum;
    __syncthreads();
    if (threadIdx.x != 0) return;

    const double p = (double)top_p[r];
    int cut = k;
    double c = 0.0;
    for (int j = 0; j < k; ++j) {
        c += e[j];
        if (c >= p) { cut = j + 1; break; }
    }
    const double tot = part[cut - 1];

    unsigned long long* state = rng_states + slots[r];
    unsigned long long s = *state;
    if (fresh[r]) s = ((unsigned long long)seeds[r] ^ 0x5DEECE66DULL) & ((1ULL << 48) - 1);
    const unsigned long long hi = lcg_next(&s, 26), lo = lcg_next(&s, 27);
    *state = s;
    const double u = (double)((hi << 27) + lo) * (1.0 / 9007199254740992.0);
    const double draw = u * tot;
    int pick = ids_sh[cut - 1];
    for (int j = 0; j < cut; ++j) {
        if (part[j] >= draw || j == cut - 1) { pick = ids_sh[j]; break; }
    }
    out[r] = pick;
}

// One row by one CTA: the CTA's threads come back from here at different places (thread 0 last).
__device__ __forceinline__ void
sample_row(SampleShared& ss, int* __restrict__ out, const float* __restrict__ logits, long row_stride,
           int vocab, const float* __restrict__ temperature, const int* __restrict__ top_k,
           const float* __restrict__ top_p, const long long* __restrict__ seeds,
           const int* __restrict__ fresh, const int* __restrict__ slots,
           unsigned long long* __restrict__ rng_states, int n_rows) {
    const int r = blockIdx.x;
    if (r >= n_rows) return;
    const float* row = logits + (size_t)r * row_stride;
    const float temp = temperature ? temperature[r] : 0.0f;

    if (!(temp > 0.0f)) {
        Best b{0.0f, -1};
        for_each_logit(row, vocab, [&](int i, float v) {
            if (better(v, i, b.v, b.i)) { b.v = v; b.i = i; }
        });
        b = block_best(b, ss.best);
        if (threadIdx.x == 0) out[r] = b.i;
        return;
    }
    const int k = clamp_top_k(top_k[r], vocab);
    unsigned long long* cand = reinterpret_cast<unsigned long long*>(ss.work);   // [CAND_CAP]
    int* pick_sh = ss.pick;

    // ---- a bound first: the k-th largest of the threads' own maxima.  At least k logits are
    // that large, so every one of the k largest is; usually not many more are.
    {
        unsigned best = 0u;
        for_each_logit(row, vocab, [&](int, float v) { best = max(best, sample_key(v)); });
        // (made distinct by the thread's number, so that exactly one entry has each rank)
        cand[threadIdx.x] = ((unsigned long long)best << 32) | (unsigned)(blockDim.x - 1 - threadIdx.x);
        // (ordered by a bitonic sort, 55 exchanges a thread: counting every maximum's rank
        // against all the others was 1,024 compares a thread and half the kernel's time)
        sort_descending(cand, (int)blockDim.x);
        if (threadIdx.x == 0) pick_sh[6] = (int)(cand[k - 1] >> 32);
        __syncthreads();
    }
    const unsigned bound = (unsigned)pick_sh[6];
    if (threadIdx.x == 0) pick_sh[5] = 0;
    __syncthreads();
    for_each_logit(row, vocab, [&](int i, float v) {
        const unsigned key = sample_key(v);
        if (key >= bound) {
            const int slot = atomicAdd(&pick_sh[5], 1);
            if (slot < CAND_CAP) cand[slot] = candidate(key, i);
        }
    });
    __syncthreads();
    int n_cand = pick_sh[5];
    if (n_cand > CAND_CAP) {
        select_exactly(ss, row, vocab, k);
        n_cand = k;
    }
    finish_row(ss, n_cand, k, temp, r, out, top_p, seeds, fresh, slots, rng_states);
}

// Where the chosen ids go besides `out`: the last CTA of the launch to finish copies `words`
// int32 words from `src` (the ids and, behind them, the step's status words, which every
// earlier kernel of the stream has finished writing) to `host`, the device address of a
// pinned host buffer, so that no kernel or copy of its own stands between a step's last
// kernel and the host's read.  counter: one int32, zero between launches.
struct Publish {
    int* host;
    const int* src;
    int words;
    int* counter;
};

// Scratch of the launch that gives a row to several CTAs, in a workspace the caller owns
// (one per sampler, so that two engines of a process do not meet in it): int32 words.
constexpr int WS_MAX_ROWS = 64, WS_PARTS = 8;
constexpr int WS_COUNTER = 0;                                   // the launch's counter (Publish::counter)
constexpr int WS_PARTIAL = 4;                                   // [rows][parts] Best (2 words)
constexpr int WS_WORDS = WS_PARTIAL + 2 * WS_MAX_ROWS * WS_PARTS;

// Greedy rows only, few of them: a row's vocabulary in ARGMAX_PARTS slices, a CTA each (one CTA
// a row spends its time on the round trips of 50 loads per thread in a row: 9 us for 8 rows of
// 50,257); the launch's last CTA takes, per row, the best of the slices' bests (`better` is a
// total order: the same id as one pass over the row) and publishes like the kernel below.
constexpr int ARGMAX_PARTS = WS_PARTS, ARGMAX_THREADS = 256;

__global__ void __launch_bounds__(ARGMAX_THREADS)
argmax_parts_kernel(int* __restrict__ out, const float* __restrict__ logits, long row_stride,
                    int vocab, int n_rows, int* __restrict__ ws, Publish pub) {
    __shared__ Best sh[32];
    __shared__ int last_sh;
    Best* partial = reinterpret_cast<Best*>(ws + WS_PARTIAL);
    prb_grid_launch_dependents();      // the next step's description may be fetched meanwhile
    const int r = blockIdx.y, part = blockIdx.x;
    const int chunk = (((vocab + ARGMAX_PARTS - 1) / ARGMAX_PARTS) + 3) & ~3;
    const int begin = min(vocab, part * chunk), len = min(vocab - begin, chunk);
    Best b{0.0f, -1};
    for_each_logit(logits + (size_t)r * row_stride + begin, len, [&](int i, float v) {
        if (better(v, begin + i, b.v, b.i)) { b.v = v; b.i = begin + i; }
    });
    b = block_best(b, sh);
    if (threadIdx.x == 0) {
        partial[r * ARGMAX_PARTS + part] = b;
        __threadfence();
        last_sh = atomicAdd(pub.counter, 1) == (int)(gridDim.x * gridDim.y) - 1 ? 1 : 0;
    }
    __syncthreads();
    if (!last_sh) return;
    __threadfence();
    // Where the ids are the first words of what is published (the engine's layout), a row's id
    // goes to the host as it is found; the words behind the ids are copied beside that.
    const bool ids_first = pub.host != nullptr && pub.src == out;
    for (int row = threadIdx.x; row < n_rows; row += blockDim.x) {
        const Best* src = &partial[row * ARGMAX_PARTS];
        float cv[ARGMAX_PARTS];
        int ci[ARGMAX_PARTS];
#pragma unroll
        for (int p = 0; p < ARGMAX_PARTS; ++p) {       // all slices' bests in one round trip
            cv[p] = __ldcg(&src[p].v);
            ci[p] = __ldcg(&src[p].i);
        }
        Best t{0.0f, -1};
#pragma unroll
        for (int p = 0; p < ARGMAX_PARTS; ++p)
            if (ci[p] >= 0 && better(cv[p], ci[p], t.v, t.i)) { t.v = cv[p]; t.i = ci[p]; }
        out[row] = t.i;
        if (ids_first && row < pub.words) pub.host[row] = t.i;
    }
    if (threadIdx.x == 0) *pub.counter = 0;
    if (pub.host == nullptr) return;
    if (ids_first) {
        for (int i = n_rows + threadIdx.x; i < pub.words; i += blockDim.x)
            pub.host[i] = __ldcg(pub.src + i);
        return;
    }
    __syncthreads();                   // the ids above may be among the words published
    for (int i = threadIdx.x; i < pub.words; i += blockDim.x) pub.host[i] = __ldcg(pub.src + i);
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(int* __restrict__ out, const float* __restrict__ logits, long row_stride, int vocab,
              const float* __restrict__ temperature, const int* __restrict__ top_k,
              const float* __restrict__ top_p, const long long* __restrict__ seeds,
              const int* __restrict__ fresh, const int* __restrict__ slots,
              unsigned long long* __restrict__ rng_states, int n_rows, Publish pub) {
    __shared__ SampleShared ss;
    prb_grid_launch_dependents();      // the next step's description may be fetched meanwhile
    sample_row(ss, out, logits, row_stride, vocab, temperature, top_k, top_p, seeds, fresh, slots,
               rng_states, n_rows);
    if (pub.host == nullptr) return;
    __shared__ int last_sh;
    __syncthreads();                   // thread 0 has stored this row's id
    if (threadIdx.x == 0) {
        __threadfence();
        last_sh = atomicAdd(pub.counter, 1) == (int)gridDim.x - 1 ? 1 : 0;
    }
    __syncthreads();
    if (!last_sh) return;
    __threadfence();
    for (int i = threadIdx.x; i < pub.words; i += blockDim.x) pub.host[i] = __ldcg(pub.src + i);
    if (threadIdx.x == 0) *pub.counter = 0;
    // (the host reads after an event recorded behind this launch has completed: the end of
    // the kernel makes the words visible, no fence of its own is needed)
}
}  // namespace

PRB_API int prb_sample_max_top_k() { return MAX_TOP_K; }
// int32 words of the workspace prb_sample may be given (zero at first; left as it needs them).
PRB_API int prb_sample_workspace_words() { return WS_WORDS; }

// Switch for measurements: PRB200_SAMPLE_SPLIT=0 keeps greedy rows on one CTA each too.
static int sample_split_off() {
    static const int off = [] { const char* e = getenv("PRB200_SAMPLE_SPLIT"); return e && atoi(e) == 0 ? 1 : 0; }();
    return off;
}

// temperature == nullptr: every row is greedy and the remaining pointers are unused.
// workspace (may be null): prb_sample_workspace_words() int32 words, 8-byte aligned, zero before
// the first call, one per stream of calls; with it, a launch of up to 64 greedy rows gives
// every row to several CTAs.  publish_host (may be null; needs the workspace): see Publish.
PRB_API int prb_sample(int* out, const float* logits, long row_stride, int vocab,
                       const float* temperature, const int* top_k, const float* top_p,
                       const long long* seeds, const int* fresh, const int* slots,
                       unsigned long long* rng_states, int n_rows, int* publish_host,
                       const int* publish_src, int publish_words, int* workspace,
                       cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (vocab <= 0) return PRB_E_SIZE;
    Publish pub{publish_host, publish_src, publish_words, workspace ? workspace + WS_COUNTER : nullptr};
    if (publish_host != nullptr && (publish_src == nullptr || workspace == nullptr || publish_words <= 0))
        return PRB_E_ARG;
    if (workspace != nullptr && ((uintptr_t)workspace) % 8 != 0) return PRB_E_ALIGN;
    const bool several = workspace != nullptr && n_rows <= WS_MAX_ROWS && vocab >= 64 * WS_PARTS &&
                         !sample_split_off();
    if (temperature == nullptr && several) {
        argmax_parts_kernel<<<dim3(ARGMAX_PARTS, n_rows), ARGMAX_THREADS, 0, stream>>>(
            out, logits, row_stride, vocab, n_rows, workspace, pub);
        PRB_LAUNCH_CHECK();
        return 0;
    }
    // (Rows that sample stay one CTA a row.  Two launches of eight CTAs a row, the first for a
    // bound from the slices' group maxima, the second collecting candidates for the row's last
    // CTA to finish, were built and gave the same tokens; alone they took 26.0 us for 8 rows of
    // 50,257 with k = 40 against 23.7 us, 40.2 against 24.5 us for 64 rows; inside a decode step
    // they won at 8 requests, 0.428 against 0.436 ms, and lost at 1 and at 16.)
    sample_kernel<<<n_rows, SAMPLE_THREADS, 0, stream>>>(out, logits, row_stride, vocab,
                                                         temperature, top_k, top_p, seeds, fresh,
                                                         slots, rng_states, n_rows, pub);
    PRB_LAUNCH_CHECK();
    return 0;
}
