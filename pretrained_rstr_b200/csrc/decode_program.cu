// A whole decode step as ONE persistent kernel.
//
// A decode step of a small model is a chain of about a hundred short, dependent
// operations (norm + projection, cache append, attention, projection, ...), each a few
// microseconds of latency and far from any throughput limit; launched one by one their
// launch and drain gaps add up to several times the work.  Here the step's operations
// are recorded once as a list of `Op` records in device memory (a "program"), and one
// cooperative kernel with one CTA per SM interprets the list: every CTA takes the
// operation's units of work blockIdx.x, blockIdx.x + gridDim.x, ..., then all CTAs meet
// at a grid-wide barrier.  The weights of the next product are requested *before* the
// barrier, so their HBM latency is hidden behind it.
//
// The units of work are the very device functions of the stand-alone kernels
// (gemm_smallm.cuh, attention_decode.cuh, elementwise.cuh), so results are identical to
// launching those kernels one after the other.
//
// The grid barrier is a counter in global memory (zeroed by a memset that precedes the
// launch).  Its spin is bounded: if a CTA gives up it raises a flag that every CTA polls,
// records PRB_S_WAIT_TIMEOUT in the status word, and all CTAs leave the kernel.
#include <vector>

#include "attention_decode.cuh"
#include "elementwise.cuh"
#include "gemm_smallm.cuh"

int prb_gemm_smallm_check(const void* x, const float* xf, const float* gamma, const float* beta,
                          const void* w, int m, int n, int k, long ldx, long ldw);

namespace {
constexpr int PROG_THREADS = 256;
constexpr int PROG_WARPS = PROG_THREADS / 32;
constexpr unsigned SPIN_LIMIT = 1u << 21;

enum OpType : int { OP_END = 0, OP_EMBED = 1, OP_NORM = 2, OP_GEMM = 3, OP_APPEND = 4, OP_ATTN = 5 };

struct alignas(16) Op {
    int type;
    int units;          // virtual blocks of this operation
    int flags;          // GEMM: bit 0 fused norm, bit 1 float32 output; NORM: bit 1 float32 output;
                        // ATTN: lanes per key row; EMBED/APPEND: bit 1 float32 tables / cache
    int aux;            // ATTN: heads * splits per token-list place
    union {
        smallm::Args gemm;
        decode_attn::Args attn;
        elementwise::EmbedArgs embed;
        elementwise::NormArgs norm;
        elementwise::AppendArgs append;
    };
};

struct Program {
    std::vector<Op> ops;
    int mt = 1;                  // 8-token tiles of the products (1, 2, 4, 8)
    size_t smem = 0;             // dynamic shared memory the interpreter needs
};

__device__ __forceinline__ bool grid_barrier(unsigned* bar, unsigned& epoch, int* sh_flag,
                                             int* status, int op_index) {
    __syncthreads();
    epoch += 1;
    if (threadIdx.x == 0) {
        const unsigned target = epoch * gridDim.x;
        __threadfence();                                   // publish this CTA's writes
        atomicAdd(&bar[0], 1u);
        int ok = 1;
        for (unsigned spins = 0;; ++spins) {
            unsigned v, failed;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(bar) : "memory");
            if (v >= target) break;
            asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(failed) : "l"(bar + 1) : "memory");
            if (failed != 0u || spins > SPIN_LIMIT) {
                if (failed == 0u) {
                    atomicExch(&bar[1], 1u);
                    prb_set_status(status, PRB_S_WAIT_TIMEOUT, 9, (int)blockIdx.x, op_index);
                }
                ok = 0;
                break;
            }
            __nanosleep(32);
        }
        __threadfence();
        *sh_flag = ok;
    }
    __syncthreads();
    return *sh_flag != 0;
}

template <int MT, bool LN, typename O>
__device__ __forceinline__ void run_gemm(const smallm::Args& a, int units, float* red,
                                         __nv_bfloat16* xs, smallm::Prefetch& pf, bool have_pf) {
    if ((int)blockIdx.x >= units) return;                  // uniform in the CTA
    if (!have_pf) smallm::prefetch(a, blockIdx.x, pf);
    if constexpr (LN) smallm::norm_rows<MT>(a, xs);
    for (int vb = blockIdx.x; vb < units; vb += gridDim.x) {
        if (vb != (int)blockIdx.x) smallm::prefetch(a, vb, pf);
        smallm::strip<MT, LN, O>(a, vb, red, xs, pf);
    }
}

template <int LPK>
__device__ __forceinline__ void run_attn(const decode_attn::Args& a, int units, int per_place,
                                         decode_attn::Shared<PROG_WARPS>& sh) {
    for (int vb = blockIdx.x; vb < units; vb += gridDim.x) {
        const int idx = vb / per_place, rem = vb - idx * per_place;
        const int h = rem / a.max_splits, s = rem - h * a.max_splits;
        decode_attn::unit<LPK, PROG_WARPS>(a, idx, h, s, sh);
        __syncthreads();
    }
}

template <int MT>
__global__ void __launch_bounds__(PROG_THREADS, 1)
decode_program_kernel(const Op* __restrict__ ops, int n_ops, unsigned* bar, int* status) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    __shared__ decode_attn::Shared<PROG_WARPS> attn_sh;
    __shared__ float scratch[32];
    __shared__ int sh_flag;
    float* red = reinterpret_cast<float*>(smem_raw);                       // [8][16][8*MT]
    __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(red + smallm::WARPS * smallm::ROWS * 8 * MT);
    float* row = reinterpret_cast<float*>(smem_raw);                       // norm rows reuse it

    unsigned epoch = 0;
    smallm::Prefetch pf;
    bool have_pf = false;
    for (int i = 0; i < n_ops; ++i) {
        const Op& op = ops[i];
        const int type = op.type, units = op.units, flags = op.flags;
        switch (type) {
            case OP_EMBED:
                for (int vb = blockIdx.x; vb < units; vb += gridDim.x) {
                    if (flags & 2) elementwise::embed_token<float>(op.embed, vb);
                    else elementwise::embed_token<__nv_bfloat16>(op.embed, vb);
                }
                break;
            case OP_NORM:
                for (int vb = blockIdx.x; vb < units; vb += gridDim.x) {
                    if (flags & 2) elementwise::layernorm_row<float>(op.norm, vb, row, scratch);
                    else elementwise::layernorm_row<__nv_bfloat16>(op.norm, vb, row, scratch);
                    __syncthreads();
                }
                break;
            case OP_GEMM:
                if (flags & 1) {
                    if (flags & 2) run_gemm<MT, true, float>(op.gemm, units, red, xs, pf, have_pf);
                    else run_gemm<MT, true, __nv_bfloat16>(op.gemm, units, red, xs, pf, have_pf);
                } else {
                    if (flags & 2) run_gemm<MT, false, float>(op.gemm, units, red, xs, pf, have_pf);
                    else run_gemm<MT, false, __nv_bfloat16>(op.gemm, units, red, xs, pf, have_pf);
                }
                break;
            case OP_APPEND:
                for (int vb = blockIdx.x; vb < units; vb += gridDim.x) {
                    if (flags & 2) elementwise::append_token<float>(op.append, vb);
                    else elementwise::append_token<__nv_bfloat16>(op.append, vb);
                }
                break;
            case OP_ATTN:
                switch (flags) {
                    case 2: run_attn<2>(op.attn, units, op.aux, attn_sh); break;
                    case 4: run_attn<4>(op.attn, units, op.aux, attn_sh); break;
                    case 8: run_attn<8>(op.attn, units, op.aux, attn_sh); break;
                    case 16: run_attn<16>(op.attn, units, op.aux, attn_sh); break;
                    default: run_attn<32>(op.attn, units, op.aux, attn_sh); break;
                }
                break;
            default:
                break;
        }
        if (i + 1 >= n_ops) break;
        // ask for the next product's first weights now: they do not depend on this phase
        const Op& next = ops[i + 1];
        have_pf = false;
        if (next.type == OP_GEMM && (int)blockIdx.x < next.units) {
            smallm::prefetch(next.gemm, blockIdx.x, pf);
            have_pf = true;
        }
        if (!grid_barrier(bar, epoch, &sh_flag, status, i)) return;
    }
}

size_t max_size(size_t a, size_t b) { return a > b ? a : b; }

template <int MT>
int launch_program(const Op* ops, int n_ops, size_t smem, unsigned* bar, int* status,
                   cudaStream_t stream) {
    static int grid = 0;
    static size_t configured = 0;
    if (smem > configured) {
        if (smem > 48 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(decode_program_kernel<MT>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 (int)smem);
            if (e != cudaSuccess) return (int)e;
        }
        int dev = 0, sms = 0, per_sm = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
            return PRB_E_ARG;
        cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(
            &per_sm, decode_program_kernel<MT>, PROG_THREADS, smem);
        if (e != cudaSuccess) return (int)e;
        if (per_sm < 1) return PRB_E_SIZE;
        grid = sms;                                      // one CTA per SM, all co-resident
        configured = smem;
    }
    cudaError_t e = cudaMemsetAsync(bar, 0, 2 * sizeof(unsigned), stream);
    if (e != cudaSuccess) return (int)e;
    void* args[] = {(void*)&ops, (void*)&n_ops, (void*)&bar, (void*)&status};
    e = cudaLaunchCooperativeKernel((void*)decode_program_kernel<MT>, dim3(grid),
                                    dim3(PROG_THREADS), args, smem, stream);
    if (e != cudaSuccess) return (int)e;
    return 0;
}
}  // namespace

// ---------------------------------------------------------------- building a program
PRB_API void* prb_program_new(int max_rows) {
    Program* p = new Program();
    p->mt = max_rows <= 8 ? 1 : max_rows <= 16 ? 2 : max_rows <= 32 ? 4 : 8;
    p->smem = smallm::smem_bytes(p->mt, false, 0);
    return p;
}
PRB_API void prb_program_free(void* handle) { delete static_cast<Program*>(handle); }
PRB_API int prb_program_length(void* handle) { return (int)static_cast<Program*>(handle)->ops.size(); }
PRB_API long prb_program_bytes(void* handle) {
    return (long)(static_cast<Program*>(handle)->ops.size() * sizeof(Op));
}

PRB_API int prb_program_add_embed(void* handle, float* out, const int* tokens, const int* positions,
                                  const void* wte, const void* wpe, int n_tokens, int width,
                                  int vocab, int n_positions, int table_dtype, int* status) {
    Program* p = static_cast<Program*>(handle);
    if (table_dtype != PRB_F32 && table_dtype != PRB_BF16) return PRB_E_DTYPE;
    Op op{};
    op.type = OP_EMBED;
    op.units = n_tokens;
    op.flags = table_dtype == PRB_F32 ? 2 : 0;
    op.embed = elementwise::EmbedArgs{out, tokens, positions, wte, wpe, n_tokens, width, vocab,
                                      n_positions, status};
    p->ops.push_back(op);
    return 0;
}

PRB_API int prb_program_add_norm(void* handle, void* out, const float* x, const float* gamma,
                                 const float* beta, const int* rows, int n_rows, int n_rows_in,
                                 int width, float eps, int out_dtype, int* status) {
    Program* p = static_cast<Program*>(handle);
    if (out_dtype != PRB_F32 && out_dtype != PRB_BF16) return PRB_E_DTYPE;
    if (width <= 0 || (size_t)width * 4 > 200 * 1024) return PRB_E_SIZE;
    Op op{};
    op.type = OP_NORM;
    op.units = n_rows;
    op.flags = out_dtype == PRB_F32 ? 2 : 0;
    op.norm = elementwise::NormArgs{out, x, gamma, beta, rows, n_rows, n_rows_in, width, eps, status};
    p->smem = max_size(p->smem, (size_t)width * sizeof(float));
    p->ops.push_back(op);
    return 0;
}

PRB_API int prb_program_add_gemm(void* handle, void* out, const void* x, const float* xf,
                                 const float* gamma, const float* beta, float eps, const void* w,
                                 const float* bias, const float* resid, int m, int n, int k,
                                 long ldx, long ldw, long ldc, int act, int out_dtype,
                                 void* k_pages, void* v_pages, const int* slots, int q_width,
                                 int kv_width, int head_dim, int page_size, int num_pages,
                                 int* status) {
    Program* p = static_cast<Program*>(handle);
    if (out_dtype != PRB_F32 && out_dtype != PRB_BF16) return PRB_E_DTYPE;
    if (m > 8 * p->mt) return PRB_E_SIZE;
    const int bad = prb_gemm_smallm_check(x, xf, gamma, beta, w, m, n, k, ldx, ldw);
    if (bad) return bad;
    const bool ln = xf != nullptr;
    const size_t smem = smallm::smem_bytes(p->mt, ln, k);
    if (smem > 200 * 1024) return PRB_E_SIZE;
    Op op{};
    op.type = OP_GEMM;
    op.units = (n + smallm::ROWS - 1) / smallm::ROWS;
    op.flags = (ln ? 1 : 0) | (out_dtype == PRB_F32 ? 2 : 0);
    smallm::Args a;
    a.out = out; a.x = (const __nv_bfloat16*)x; a.xf = xf; a.gamma = gamma; a.beta = beta;
    a.eps = eps; a.w = (const __nv_bfloat16*)w; a.bias = bias; a.resid = resid;
    a.m = m; a.n = n; a.k = k; a.ldx = ldx; a.ldw = ldw; a.ldc = ldc; a.act = act;
    a.xs_pitch = ln ? smallm::norm_pitch(k) : k;
    if (kv_width > 0 && (head_dim <= 0 || kv_width % head_dim != 0 || page_size <= 0 ||
                         q_width + 2 * kv_width != n || !k_pages || !v_pages || !slots))
        return PRB_E_ARG;
    a.k_pages = k_pages; a.v_pages = v_pages; a.slots = slots;
    a.q_width = q_width; a.kv_width = kv_width; a.head_dim = head_dim;
    a.page_size = page_size; a.num_pages = num_pages; a.status = status;
    op.gemm = a;
    p->smem = max_size(p->smem, smem);
    p->ops.push_back(op);
    return 0;
}

PRB_API int prb_program_add_append(void* handle, void* k_pages, void* v_pages, const void* k_src,
                                   const void* v_src, long src_stride, const int* slots,
                                   int n_tokens, int kv_heads, int head_dim, int page_size,
                                   int num_pages, int dtype, int* status) {
    Program* p = static_cast<Program*>(handle);
    if (dtype != PRB_F32 && dtype != PRB_BF16) return PRB_E_DTYPE;
    if (kv_heads <= 0 || head_dim <= 0 || page_size <= 0) return PRB_E_SIZE;
    Op op{};
    op.type = OP_APPEND;
    op.units = n_tokens;
    op.flags = dtype == PRB_F32 ? 2 : 0;
    op.append = elementwise::AppendArgs{k_pages, v_pages, k_src, v_src, src_stride, slots, n_tokens,
                                        kv_heads, head_dim, page_size, num_pages, status};
    p->ops.push_back(op);
    return 0;
}

PRB_API int prb_program_add_attention(void* handle, void* out, long out_stride, const void* q,
                                      long q_stride, const void* k_pages, const void* v_pages,
                                      const int* block_table, const int* seq_of_token,
                                      const int* positions, const int* token_list,
                                      const int* token_count, int n_list, int n_heads,
                                      int kv_heads, int head_dim, int page_size, int max_pages,
                                      int num_pages, float scale, int window, float* workspace,
                                      int* counters, int max_splits, int split_keys,
                                      int* status) {
    Program* p = static_cast<Program*>(handle);
    if (n_heads <= 0 || kv_heads <= 0 || n_heads % kv_heads != 0 || head_dim <= 0 ||
        head_dim % 8 != 0 || head_dim > decode_attn::MAX_DH || page_size < 8 ||
        decode_attn::SPLIT % page_size != 0 || max_splits <= 0 || split_keys < decode_attn::SPLIT ||
        split_keys % decode_attn::SPLIT != 0 ||
        split_keys / page_size > decode_attn::MAX_SPLIT_PAGES)
        return PRB_E_SIZE;
    if (q_stride % 8 != 0 || ((uintptr_t)q) % 16 != 0 ||
        ((uintptr_t)out) % 4 != 0 || ((uintptr_t)k_pages) % 16 != 0 ||
        ((uintptr_t)v_pages) % 16 != 0)
        return PRB_E_ALIGN;
    Op op{};
    op.type = OP_ATTN;
    op.units = n_list * n_heads * max_splits;
    op.aux = n_heads * max_splits;
    const int pieces = head_dim / 8;
    op.flags = pieces <= 2 ? 2 : pieces <= 4 ? 4 : pieces <= 8 ? 8 : pieces <= 16 ? 16 : 32;
    decode_attn::Args a;
    a.out = (__nv_bfloat16*)out; a.out_stride = out_stride;
    a.q = (const __nv_bfloat16*)q; a.q_stride = q_stride;
    a.k_pages = (const __nv_bfloat16*)k_pages; a.v_pages = (const __nv_bfloat16*)v_pages;
    a.block_table = block_table; a.seq_of_token = seq_of_token; a.positions = positions;
    a.token_list = token_list; a.token_count = token_count;
    a.n_heads = n_heads; a.kv_heads = kv_heads; a.head_dim = head_dim; a.page_size = page_size;
    a.max_pages = max_pages; a.num_pages = num_pages; a.scale = scale; a.window = window;
    a.workspace = workspace; a.counters = counters; a.max_splits = max_splits;
    a.split = split_keys; a.status = status;
    op.attn = a;
    p->ops.push_back(op);
    return 0;
}

// Copy the recorded operations to `device_ops` (at least prb_program_bytes bytes).
PRB_API int prb_program_upload(void* handle, void* device_ops, cudaStream_t stream) {
    Program* p = static_cast<Program*>(handle);
    if (p->ops.empty()) return PRB_E_ARG;
    cudaError_t e = cudaMemcpyAsync(device_ops, p->ops.data(), p->ops.size() * sizeof(Op),
                                    cudaMemcpyHostToDevice, stream);
    if (e != cudaSuccess) return (int)e;
    e = cudaStreamSynchronize(stream);                 // the vector may be freed afterwards
    return e == cudaSuccess ? 0 : (int)e;
}

// Run an uploaded program: `barrier` is 2 x uint32 of scratch (zeroed here, on the stream).
PRB_API int prb_program_run(void* handle, const void* device_ops, unsigned* barrier, int* status,
                            cudaStream_t stream) {
    Program* p = static_cast<Program*>(handle);
    const Op* ops = static_cast<const Op*>(device_ops);
    const int n = (int)p->ops.size();
    switch (p->mt) {
        case 1: return launch_program<1>(ops, n, p->smem, barrier, status, stream);
        case 2: return launch_program<2>(ops, n, p->smem, barrier, status, stream);
        case 4: return launch_program<4>(ops, n, p->smem, barrier, status, stream);
        default: return launch_program<8>(ops, n, p->smem, barrier, status, stream);
    }
}
