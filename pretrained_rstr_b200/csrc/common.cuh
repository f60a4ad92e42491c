// Shared helpers of the sm_100a kernels: element types, the status word, launch checks.
//
// Every exported function is `extern "C"`, takes raw device pointers, explicit sizes
// and the stream to launch on, allocates nothing, and returns 0 or a negative code
// (see PRB_E_*) for arguments it refuses; a CUDA launch error is returned as the
// positive cudaError_t value.  Kernels never trap: an index that is out of range is
// recorded in the status word (first error wins) and the access is skipped.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define PRB_API extern "C" __attribute__((visibility("default")))

// argument errors (host side)
#define PRB_E_DTYPE (-2)     // unknown element type code
#define PRB_E_SIZE (-3)      // a size the kernel does not take
#define PRB_E_ALIGN (-4)     // a pointer or stride that is not aligned as required
#define PRB_E_ARG (-5)       // any other bad argument

// element type codes shared with Python
#define PRB_F32 0
#define PRB_BF16 1

// status word codes (device side); status[0] = code, status[1..3] = details
#define PRB_S_OK 0
#define PRB_S_TOKEN_RANGE 1      // token id outside the vocabulary
#define PRB_S_POSITION_RANGE 2   // position outside the position table / cache
#define PRB_S_SLOT_RANGE 3       // cache slot outside the pool
#define PRB_S_PAGE_RANGE 4       // block-table entry outside the pool or missing
#define PRB_S_WAIT_TIMEOUT 5     // a bounded wait on a barrier gave up
#define PRB_S_ROW_RANGE 6        // a row index outside its tensor

__device__ __forceinline__ void prb_set_status(int* status, int code, int a, int b, int c) {
    if (status == nullptr) return;
    if (atomicCAS(status, PRB_S_OK, code) == PRB_S_OK) {
        status[1] = a;
        status[2] = b;
        status[3] = c;
    }
}

template <typename T> __device__ __forceinline__ float prb_to_float(T v);
template <> __device__ __forceinline__ float prb_to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float prb_to_float<__nv_bfloat16>(__nv_bfloat16 v) {
    return __bfloat162float(v);
}
template <typename T> __device__ __forceinline__ T prb_from_float(float v);
template <> __device__ __forceinline__ float prb_from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 prb_from_float<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

__device__ __forceinline__ float prb_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float prb_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide sum with a fixed reduction tree (result identical for identical inputs,
// whatever else runs on the GPU).  `scratch` holds at least 32 floats.
__device__ __forceinline__ float prb_block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = prb_warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = (lane < nwarps) ? scratch[lane] : 0.0f;
    r = prb_warp_sum(r);
    return r;
}
__device__ __forceinline__ float prb_block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = prb_warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = (lane < nwarps) ? scratch[lane] : -INFINITY;
    r = prb_warp_max(r);
    return r;
}

// activation codes
#define PRB_ACT_NONE 0
#define PRB_ACT_GELU_TANH 1
#define PRB_ACT_GELU_ERF 2
#define PRB_ACT_RELU 3

__device__ __forceinline__ float prb_activate(float u, int act) {
    switch (act) {
        case PRB_ACT_GELU_TANH: {
            const float c = 0.7978845608028654f;  // sqrt(2/pi)
            return 0.5f * u * (1.0f + tanhf(c * (u + 0.044715f * u * u * u)));
        }
        case PRB_ACT_GELU_ERF:
            return 0.5f * u * (1.0f + erff(u * 0.7071067811865476f));
        case PRB_ACT_RELU:
            return fmaxf(u, 0.0f);
        default:
            return u;
    }
}

// Programmatic dependent launch.  A kernel launched with prb_launch_dependent may start
// while its predecessor in the stream is still running; everything it does before
// prb_grid_wait() must not depend on the predecessor (prefetching weights, reading the
// step's metadata).  Every thread calls prb_grid_wait() before it reads or writes
// anything another kernel of the step produces or consumes, and before it exits, so
// that completion of a kernel implies completion of all kernels before it.
__device__ __forceinline__ void prb_grid_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void prb_grid_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
int prb_pdl_enabled();

// Streaming multiprocessors of the current device (asked once per device); every heuristic
// that sizes a grid or counts waves takes the number from here.
int prb_sm_count();

// Kernels of many small CTAs (norms, attention) are not placed early: their CTAs would fill
// the few SMs that the predecessor leaves free, several to an SM, instead of spreading
// over all of them when it has ended, and then run at the pace of those SMs (measured: a
// prompt step of 256 to 1,024 tokens is 6 % slower with them placed early).  They still
// call prb_grid_launch_dependents(), so that a successor of one CTA per SM sets itself up
// while they run.  prb_small_ctas_early() is the switch for measurements.
int prb_small_ctas_early();

template <typename... KArgs, typename... Args>
inline cudaError_t prb_launch_maybe_early(bool early, void (*kernel)(KArgs...), dim3 grid,
                                          dim3 block, size_t smem, cudaStream_t stream,
                                          Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = early && prb_pdl_enabled() ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

template <typename... KArgs, typename... Args>
inline cudaError_t prb_launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block,
                                        size_t smem, cudaStream_t stream, Args... args) {
    return prb_launch_maybe_early(true, kernel, grid, block, smem, stream, args...);
}

#define PRB_LAUNCH_CHECK()                               \
    do {                                                 \
        cudaError_t e__ = cudaGetLastError();            \
        if (e__ != cudaSuccess) return (int)e__;         \
    } while (0)
