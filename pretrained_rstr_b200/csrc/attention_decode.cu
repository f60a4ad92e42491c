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
// Scratch: workspace [tokens, heads, max_splits, head_dim + 4] float32 and counters
// [tokens * heads] int32 (zero before the first launch; the kernel leaves them zero).
#ifdef PRB_TRACE
__device__ unsigned long long g_dec_trace[4096 * 8];
#define DEC_TRACE(slot)                                                               \
    do {                                                                              \
        const int cta__ = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x; \
        if (threadIdx.x == 0 && cta__ < 4096) {                                       \
            unsigned long long t__;                                                   \
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t__));                   \
            g_dec_trace[cta__ * 8 + (slot)] = t__;                                    \
        }                                                                             \
    } while (0)
#endif
#include <cstdlib>
#include <mutex>
#include "attention_decode.cuh"

namespace {
using namespace decode_attn;
constexpr int DEC_THREADS = 128;
constexpr int DEC_WARPS = DEC_THREADS / 32;

// LPK: lanes per key row: 2, 4, 8, 16 or 32 (head_dim <= 8 * LPK).  Two instances per LPK:
// batches of four keys per thread at four CTAs per SM, and batches of two at six CTAs per
// SM for launches with more CTAs than four per SM hold at once.  Both sum in the same order.
template <int LPK, int UB, int MIN_CTAS, bool CLUSTER>
__global__ void __launch_bounds__(DEC_THREADS, MIN_CTAS)
attention_decode_kernel(Args a) {
    __shared__ Shared<DEC_WARPS> sh;
    prb_grid_launch_dependents();
    prb_grid_wait();
    unit<LPK, DEC_WARPS, UB, CLUSTER>(a, blockIdx.x, blockIdx.y, blockIdx.z, sh);
}

// The streaming variant: one more template of the same unit, with the ring in dynamic shared
// memory (3 stages x (keys + values) x 64 positions x head_dim x 2 bytes: 48 KB at head size
// 64, four CTAs per SM).
template <int LPK, bool CLUSTER>
__global__ void __launch_bounds__(DEC_THREADS, 1)
attention_decode_stream_kernel(Args a) {
    extern __shared__ __align__(128) unsigned char stream_ring[];
    __shared__ Shared<DEC_WARPS> sh;
    __shared__ StreamState st;
    prb_grid_launch_dependents();
    prb_grid_wait();
    if (threadIdx.x == 0) st.ring = stream_ring;
    unit<LPK, DEC_WARPS, 2, CLUSTER, true>(a, blockIdx.x, blockIdx.y, blockIdx.z, sh, &st);
}

// Whether the kernel may be placed on the SMs before its predecessor has ended.  Off, by
// measurement: GPT-2 small with 8 requests takes 0.467 ms a step with it and 0.430 ms
// without.  The likely cause: CTAs that are placed one by one, as the CTAs of the QKV product
// leave, fill the first free SMs to their limit and leave the last ones half empty, and the
// kernel lasts as long as its fullest SM.  PRB200_DECODE_EARLY=1 turns it on for measurements.
static int decode_early() {
    static const int on = [] { const char* e = getenv("PRB200_DECODE_EARLY"); return e ? atoi(e) : 0; }();
    return on;
}

// Launch (the kernel itself lets its successor start early) and, for `cluster_z` > 1, the
// CTAs of a (token, head) (grid z) as one thread-block cluster.
template <typename K>
cudaError_t launch_decode(K kernel, dim3 grid, int cluster_z, cudaStream_t stream, const Args& a,
                          size_t dynamic_smem = 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(DEC_THREADS);
    cfg.dynamicSmemBytes = dynamic_smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = prb_pdl_enabled() && decode_early() ? 1 : 0;
    cfg.numAttrs = 1;
    if (cluster_z > 1) {
        attr[1].id = cudaLaunchAttributeClusterDimension;
        attr[1].val.clusterDim.x = 1;
        attr[1].val.clusterDim.y = 1;
        attr[1].val.clusterDim.z = (unsigned)cluster_z;
        cfg.numAttrs = 2;
    }
    cfg.attrs = attr;
    return cudaLaunchKernelEx(&cfg, kernel, a);
}
}  // namespace

PRB_API int prb_attention_decode_split() { return SPLIT; }
PRB_API int prb_attention_decode_max_split_pages() { return MAX_SPLIT_PAGES; }

// Switch (for measurements): 0 = splits always merge through the workspace.
// Switch (for measurements): -1 = the streaming variant where it is chosen, 0 = never,
// 1 = wherever it applies.
static int g_decode_stream = -1;
static int prb_decode_stream() { return g_decode_stream; }
PRB_API void prb_attention_decode_set_stream(int mode) { g_decode_stream = mode; }
static int g_decode_clusters = 1;
static int prb_decode_clusters() { return g_decode_clusters; }
PRB_API void prb_attention_decode_set_clusters(int on) { g_decode_clusters = on ? 1 : 0; }
#ifdef PRB_TRACE
PRB_API int prb_attention_decode_trace(unsigned long long* host, int n) {
    return (int)cudaMemcpyFromSymbol(host, g_dec_trace, sizeof(unsigned long long) * n);
}
#endif

// workspace: float32 [n_list, n_heads, max_splits, head_dim + 4]; counters: int32
// [n_list * n_heads], zero; both indexed by the place in the token list.  token_list/token_count may be null (all
// tokens 0..n_list-1).  split_keys: keys per split (a multiple of 128 and of the page size);
// max_splits >= ceil(max context / split_keys).
PRB_API int prb_attention_decode(void* out, long out_stride, const void* q, long q_stride,
                                 const void* k_pages, const void* v_pages, const int* block_table,
                                 const int* seq_of_token, const int* positions,
                                 const int* token_list, const int* token_count, int n_list,
                                 int n_heads, int kv_heads, int head_dim, int page_size,
                                 int max_pages, int num_pages, float scale, int window,
                                 float* workspace, int* counters, int max_splits,
                                 int split_keys, int* status, cudaStream_t stream) {
    if (n_list <= 0) return 0;
    if (n_heads <= 0 || kv_heads <= 0 || n_heads % kv_heads != 0 || head_dim <= 0 ||
        head_dim % 8 != 0 || head_dim > MAX_DH || page_size < 8 || SPLIT % page_size != 0 ||
        split_keys < SPLIT || split_keys % SPLIT != 0 || split_keys / page_size > MAX_SPLIT_PAGES ||
        max_splits <= 0 || max_splits > 65535 || n_heads > 65535)
        return PRB_E_SIZE;
    if (q_stride % 8 != 0 || ((uintptr_t)q) % 16 != 0 || ((uintptr_t)k_pages) % 16 != 0 ||
        ((uintptr_t)v_pages) % 16 != 0 || ((uintptr_t)workspace) % 16 != 0)
        return PRB_E_ALIGN;
    dim3 grid(n_list, n_heads, max_splits);
    const int pieces = head_dim / 8;
    Args a;
    a.out = (__nv_bfloat16*)out; a.out_stride = out_stride;
    a.q = (const __nv_bfloat16*)q; a.q_stride = q_stride;
    a.k_pages = (const __nv_bfloat16*)k_pages; a.v_pages = (const __nv_bfloat16*)v_pages;
    a.block_table = block_table; a.seq_of_token = seq_of_token; a.positions = positions;
    a.token_list = token_list; a.token_count = token_count;
    a.n_heads = n_heads; a.kv_heads = kv_heads; a.head_dim = head_dim; a.page_size = page_size;
    a.max_pages = max_pages; a.num_pages = num_pages; a.scale = scale; a.window = window;
    a.workspace = workspace; a.counters = counters; a.max_splits = max_splits;
    a.split = split_keys; a.status = status;
    // more CTAs than fit at four per SM: the leaner instance, six per SM; two to eight
    // splits: the CTAs of a (token, head) form a cluster and merge through shared memory
    const bool many = (long)n_list * n_heads * max_splits > 4L * prb_sm_count();
    const bool cluster = max_splits >= 2 && max_splits <= 8 && prb_decode_clusters();
#define PRB_DEC(L)                                                                               \
    do {                                                                                         \
        if (cluster)                                                                             \
            e = many ? launch_decode(attention_decode_kernel<L, 2, 6, true>, grid, max_splits,   \
                                     stream, a)                                                  \
                     : launch_decode(attention_decode_kernel<L, 4, 4, true>, grid, max_splits,   \
                                     stream, a);                                                 \
        else                                                                                     \
            e = many ? launch_decode(attention_decode_kernel<L, 2, 6, false>, grid, 1, stream, a) \
                     : launch_decode(attention_decode_kernel<L, 4, 4, false>, grid, 1, stream,   \
                                     a);                                                         \
    } while (0)
    cudaError_t e;
    // Long splits and more units than run at once: the streaming variant.
    const size_t ring_bytes = (size_t)STREAM_STAGES * 2 * STREAM_KEYS * head_dim * 2;
    const int stream_mode = prb_decode_stream();
    const bool use_stream = window <= 0 && head_dim <= 128 &&
                            (stream_mode == 1 || (stream_mode < 0 && many && split_keys >= 512));
    if (use_stream) {
#define PRB_DEC_STREAM(L)                                                                        \
    do {                                                                                         \
        auto kern = cluster ? attention_decode_stream_kernel<L, true>                            \
                            : attention_decode_stream_kernel<L, false>;                          \
        static bool configured[2] = {false, false};                                              \
        if (!configured[cluster ? 1 : 0]) {                                                      \
            cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout,           \
                                 cudaSharedmemCarveoutMaxShared);                                \
            e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,          \
                                     (int)((size_t)STREAM_STAGES * 2 * STREAM_KEYS * (L * 8) * 2)); \
            if (e != cudaSuccess) return (int)e;                                                 \
            configured[cluster ? 1 : 0] = true;                                                  \
        }                                                                                        \
        e = launch_decode(kern, grid, cluster ? max_splits : 1, stream, a, ring_bytes);          \
    } while (0)
        if (pieces <= 2) PRB_DEC_STREAM(2);
        else if (pieces <= 4) PRB_DEC_STREAM(4);
        else if (pieces <= 8) PRB_DEC_STREAM(8);
        else PRB_DEC_STREAM(16);
#undef PRB_DEC_STREAM
        if (e != cudaSuccess) return (int)e;
        return 0;
    }
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
std::mutex noalloc_setup_lock;          // two host threads may make the first call together
}  // namespace

// Largest sizes the entry point takes: floats of workspace (n_list * n_heads * max_splits
// * (head_dim + 4) must not exceed it) and counters (n_list * n_heads).
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
                                         int split_keys, int* status, cudaStream_t stream) {
    if (n_list <= 0) return 0;
    if (n_heads <= 0 || head_dim <= 0 || max_splits <= 0) return PRB_E_SIZE;
    const long need_ws = (long)n_list * n_heads * max_splits * (head_dim + 4);
    const long need_counters = (long)n_list * n_heads;
    if (need_ws > NOALLOC_WS_FLOATS || need_counters > NOALLOC_COUNTERS) return PRB_E_SIZE;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= NOALLOC_MAX_DEVICES) return PRB_E_ARG;
    NoAllocDevice& d = noalloc_devices[dev];
    {
        std::lock_guard<std::mutex> guard(noalloc_setup_lock);
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
    }
    // the counters must start at zero, whatever an earlier call left behind
    e = cudaMemsetAsync(d.counters, 0, (size_t)need_counters * sizeof(int), stream);
    if (e != cudaSuccess) return (int)e;
    return prb_attention_decode(out, out_stride, q, q_stride, k_pages, v_pages, block_table,
                                seq_of_token, positions, token_list, token_count, n_list, n_heads,
                                kv_heads, head_dim, page_size, max_pages, num_pages, scale, window,
                                d.workspace, d.counters, max_splits, split_keys, status, stream);
}
