// Decode attention over the paged bfloat16 cache, second kernel: persistent CTAs whose warps
// each stream their share of the keys and values through a private ring of shared-memory
// buffers filled by TMA tile copies (cp.async.bulk.tensor with the 128-byte swizzle, no
// multicast) and multiply them on the tensor cores (mma.sync: one query row is a sixteenth
// of a tile, but thirty-two instructions replace a thousand).
//
// Why a second kernel.  A decode step is a chain of short dependent kernels, and what a
// decode attention launch costs is not its bytes but its latencies in a row: wait for the
// QKV product, read the step's description, read the block table, ask HBM for the first
// keys, score them, merge.  Almost none of that depends on the QKV product: every key and
// value that was cached before this step, the block tables and the positions are there
// before the step begins.  So this kernel is launched early (programmatic dependent launch),
// one CTA per SM, reads the description, divides the work, and has its copies of all OLD
// keys and values in flight or landed before the product it depends on has finished.  After
// the dependency resolves it fetches the queries and the few rows the step itself appended,
// and computes from shared memory.
//
// Work.  A unit is 32 consecutive key positions [32 i, 32 i + 32) of one (token, head).
// Units are numbered token by token, head by head, block by block; the warps of the grid
// (CTA by CTA, warp by warp) take equal contiguous runs of that numbering, so a warp walks
// consecutive blocks of the same (token, head) and keeps a running softmax state (maximum,
// sum, weighted values, all float32) in registers.  Where a (token, head) is shared by
// several warps of a CTA their partial states meet in shared memory and one warp merges them
// in warp order, which is block order; where it is shared by several CTAs each writes its
// merged state to the workspace and counts itself in, and the last one merges the CTAs'
// states in CTA order.  No CTA waits for another: the only waits are on a warp's own copies
// (bounded) and the CTA's own barrier.
//
// Scores are (q . k) * scale in float32; keys outside [lo, pos] are masked by selection, and
// the value rows of masked keys are zeroed in shared memory before they are multiplied by a
// zero weight, so that whatever a page's earlier owner left there cannot reach the output.
//
// Limits: head size 64, page sizes 8, 16 or a multiple of 32.  Other sizes are refused
// (the caller uses the register-batch kernel of attention_decode.cu).
#ifdef PRB_TRACE
// device-side timestamps of one launch (thread 0 of every CTA): start, work divided, first
// copies requested, dependency resolved, first buffer landed, run done, end
#include <cuda_runtime.h>
__device__ unsigned long long g_ring_trace[256 * 8];
#define RING_TRACE(slot)                                                              \
    do {                                                                              \
        if (threadIdx.x == 0 && blockIdx.x < 256) {                                   \
            unsigned long long t__;                                                   \
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t__));                   \
            g_ring_trace[blockIdx.x * 8 + (slot)] = t__;                              \
        }                                                                             \
    } while (0)
#endif
#include "attention_decode_ring.cuh"

#ifdef PRB_TRACE
PRB_API int prb_attention_decode_ring_trace(unsigned long long* host, int n) {
    return (int)cudaMemcpyFromSymbol(host, g_ring_trace, sizeof(unsigned long long) * n);
}
#endif

namespace {
using namespace ring;

__global__ void __launch_bounds__(RING_THREADS, 2)
attention_decode_ring_kernel(RingArgs a, const __grid_constant__ CUtensorMap map_k,
                             const __grid_constant__ CUtensorMap map_v) {
    extern __shared__ __align__(128) unsigned char ring_raw[];
    __shared__ Shared sh;
    RING_TRACE(0);
    prb_grid_launch_dependents();                   // the next kernel may set itself up
    const uint32_t ring_base = (smem_addr(ring_raw) + 1023u) & ~1023u;
    if (threadIdx.x < RING_WARPS) sh.bars_valid[threadIdx.x] = 0;
    plan(a, sh);
    RING_TRACE(1);
    early(a, &map_k, &map_v, sh, ring_base, (int)gridDim.x, (int)blockIdx.x);
    RING_TRACE(2);
    prb_grid_wait();
    RING_TRACE(3);
    late(a, &map_k, &map_v, sh, ring_base, (int)gridDim.x, (int)blockIdx.x);
}

int launch_ring(const RingArgs& a, const CUtensorMap& mk, const CUtensorMap& mv, int grid, int warps,
                cudaStream_t stream) {
    const size_t smem = (size_t)warps * a.stages * 2 * TILE + 1024;      // (+ alignment of the tiles)
    static size_t configured = 0;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_decode_ring_kernel,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = smem;
    }
    cudaError_t e = prb_launch_dependent(attention_decode_ring_kernel, dim3(grid), dim3(32 * warps),
                                         smem, stream, a, mk, mv);
    return e == cudaSuccess ? 0 : (int)e;
}
}  // namespace

// Warps per CTA and buffers per warp, forced (for measurements; 0, 0: the kernel's choice).
static int g_ring_warps = 0, g_ring_stages = 0;
PRB_API int prb_attention_decode_ring_tune(int warps, int stages) {
    if (warps == 0 && stages == 0) { g_ring_warps = g_ring_stages = 0; return 0; }
    if (warps < 1 || warps > RING_WARPS || stages < 2 || stages > MAX_STAGES ||
        (size_t)warps * stages * 2 * TILE > 200 * 1024)
        return PRB_E_SIZE;
    g_ring_warps = warps;
    g_ring_stages = stages;
    return 0;
}

// Whether the kernel takes these sizes.
PRB_API int prb_attention_decode_ring_supports(int head_dim, int page_size) {
    return ring::supports(head_dim, page_size);
}

PRB_API int prb_attention_decode_ring_max_list() { return MAX_LIST; }

// Whether this kernel is the faster one for a launch of n_list tokens over contexts of up to
// max_context keys; the split-key kernel of attention_decode.cu is the other.  Measured inside
// whole decode steps (ms a step, split-key / ring; n_list is the capacity the step's graph
// was made for, so 24 requests run as 32 and 48 as 64).  GPT-2 small, 12 heads: 1 request 0.372
// / 0.364 at context 256 and 0.366 / 0.366 at 1,000; 8 requests 0.358 / 0.391 (500) and 0.417 /
// 0.437 (1,000); 12 requests 0.540 / 0.524 and 16 requests 0.545 / 0.544 (1,000), 16 requests
// 0.502 / 0.507 (320) and 0.561 / 0.541 (576); 32 requests 0.586 / 0.578 (250), 0.691 / 0.660
// (320), 0.821 / 0.717 (576), 0.884 / 0.776 (1,000); 24 as 32: 0.709 / 0.726; 40: 0.875 / 0.859;
// 48: 0.881 / 0.895; 56: 1.121 / 0.947; 64 requests 0.620 / 0.646 (250), 0.719 / 0.730 (320),
// 0.899 / 0.858 (576), 1.140 / 0.992 (1,000).  Medium, 16 heads: 16 requests 1.360 / 1.305
// (1,000); 32 requests 1.633 / 1.487 (250).  XL, 25 heads: 8 requests 2.55 / 2.75 (1,000); 16
// requests 3.99 / 3.80 (1,000) and 2.80 / 2.83 (250).
// The ring wins where many (token, head) pairs have long contexts (its warps stream long runs,
// the other kernel's CTAs walk their keys one batch after the other), in the middle range at
// every context, and at a single request with a short context (everything it reads is
// requested before the dependency resolves and one CTA holds a whole pair).
PRB_API int prb_attention_decode_ring_prefers(int n_list, int n_heads, int max_context) {
    const long pairs = (long)n_list * n_heads;
    const long sms = prb_sm_count();
    if (pairs >= 4 * sms) return max_context > 512;
    if (pairs >= 2 * sms) return 1;
    if (pairs >= sms) return n_list >= 16 && max_context > 512;
    return pairs * 8 <= sms && max_context <= 512;
}

// Floats of workspace a launch of up to n_list tokens needs.
PRB_API long prb_attention_decode_ring_workspace(int n_list, int n_heads, int head_dim) {
    return ((long)prb_sm_count() + (long)n_list * n_heads) * (head_dim + 4);
}

// new_keys: how many of a token's last visible positions the step itself may have written
// (the most tokens a request brings to this kernel in one step, at most 4).  k_new / v_new:
// the step's own keys and values, row t for token t (null: the kernel reads them from the
// cache after the dependency has resolved).  stages: ring buffers per
// warp (2 to 4; 0 = the kernel's choice).  workspace: prb_attention_decode_ring_workspace
// floats; counters: n_list * n_heads int32, zero (left zero).  The cache must be contiguous.
PRB_API int prb_attention_decode_ring(void* out, long out_stride, const void* q, long q_stride,
                                      const void* k_pages, const void* v_pages,
                                      const int* block_table, const int* seq_of_token,
                                      const int* positions, const int* token_list,
                                      const int* token_count, int n_list, int n_heads,
                                      int kv_heads, int head_dim, int page_size, int max_pages,
                                      int num_pages, float scale, int window, int new_keys,
                                      const void* k_new, const void* v_new, long kv_stride,
                                      float* workspace, int* counters, int stages,
                                      int max_context, int* status, cudaStream_t stream) {
    if (n_list <= 0) return 0;
    if (stages < 0 || stages > MAX_STAGES || stages == 1) return PRB_E_SIZE;
    CUtensorMap mk, mv;
    const int rc = check_and_maps(q, q_stride, out, out_stride, k_pages, v_pages, n_list, n_heads,
                                  kv_heads, head_dim, page_size, num_pages, new_keys, k_new, v_new,
                                  kv_stride, &mk, &mv);
    if (rc) return rc;
    RingArgs a;
    a.out = (__nv_bfloat16*)out; a.out_stride = out_stride;
    a.q = (const __nv_bfloat16*)q; a.q_stride = q_stride;
    a.block_table = block_table; a.seq_of_token = seq_of_token; a.positions = positions;
    a.token_list = token_list; a.token_count = token_count;
    a.n_list = n_list; a.n_heads = n_heads; a.kv_heads = kv_heads; a.page_size = page_size;
    a.max_pages = max_pages; a.num_pages = num_pages; a.scale = scale; a.window = window;
    a.k_new = (const __nv_bfloat16*)k_new; a.v_new = (const __nv_bfloat16*)v_new; a.kv_stride = kv_stride;
    a.new_keys = new_keys; a.workspace = workspace; a.counters = counters; a.status = status;
    const int sms = prb_sm_count();
    // Warps and ring depth: 8 warps x 2 buffers (128 KB).  The CTAs of this kernel are meant
    // to sit on the SMs beside those of the product before it (about 48 KB of shared memory
    // each) while that still runs, and to leave room for the product after it; with up to two
    // units per warp the buffers hold everything a warp will ever read, requested before the
    // dependency resolves (a third unit follows when the first has been read).  Longer runs
    // stream through the same two buffers: a third buffer per warp (most bytes in flight)
    // measured slower alone at every size (64 requests x 12 heads at 1,000 keys: 43.9 against
    // 42.8 us) and more so inside a step, where its 192 KB leave the next kernel no room
    // (GPT-2 small, 64 requests: 1.021 against 0.992 ms a step; XL: 7.43 against 7.24 ms).
    int warps = 8, st = 2;
    if (stages > 0) { st = stages; warps = (size_t)stages * 8 * 2 * TILE > 200 * 1024 ? 6 : 8; }
    if (stages == 0 && g_ring_warps > 0) { warps = g_ring_warps; st = g_ring_stages; }
    a.stages = st;
    return launch_ring(a, mk, mv, sms, warps, stream);
}
