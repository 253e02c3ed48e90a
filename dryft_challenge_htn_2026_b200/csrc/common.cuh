// Shared device helpers of the sm_100a kernels: element types, reductions, launch with
// programmatic dependent launch (PDL), and the page layout of the key/value cache.
//
// Every kernel file builds into a shared object of its own with plain C entry points
// (loaded with ctypes); entry points return the cudaError_t of the launch as an int.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

typedef __nv_bfloat16 bf16;

// Tokens per cache page. A page of one kv head is a contiguous [PAGE, head_dim] tile.
#define DK_PAGE 64

#define DK_EXPORT extern "C" __attribute__((visibility("default")))

__device__ __forceinline__ float to_f(float x) { return x; }
__device__ __forceinline__ float to_f(bf16 x) { return __bfloat162float(x); }
template <typename T> __device__ __forceinline__ T from_f(float x);
template <> __device__ __forceinline__ float from_f<float>(float x) { return x; }
template <> __device__ __forceinline__ bf16 from_f<bf16>(float x) { return __float2bfloat16_rn(x); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result. `red` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();  // red may still be read from an earlier call
    if (lane == 0) red[w] = v;
    __syncthreads();
    if (w == 0) {
        float t = lane < nw ? red[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

// Programmatic dependent launch. A kernel launched with the attribute may start while its
// predecessor in the stream drains; pdl_wait() blocks until the predecessor has finished and its
// writes are visible, so nothing the predecessor (or any earlier kernel) wrote may be read, and
// nothing may be written, before it. Without the attribute both are no-ops.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// The kernel after this one may be launched once every block of this one has called this (or has
// left). Most kernels call it after their wait, so at most one kernel runs ahead. The short kernels
// that stand directly before a streaming kernel of a decode step (the norms, the merge of the
// attention parts and the embedding before a product; the rotation before decode attention) call
// it before their wait: the streaming kernel's blocks then come in as soon as the SMs have room
// and fill their rings while the kernel before the short one is still at work. That is safe
// because every kernel waits before it reads or writes anything that another kernel of the step
// writes (a wait returns only when the kernel before has finished, which in turn has waited for
// the one before it), and what a streaming kernel does before its wait reads only what no kernel
// of the step writes: weights; positions, page ids and the cache pages of older tokens.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;"); }

// Cache policy for what a decode step reads exactly once (weights, the keys and values of a sequence):
// first in line to leave the L2, so that gigabytes of them streaming through do not push out the few
// megabytes that the kernels of a step hand to one another (the residual stream, partial sums, q).
__device__ __forceinline__ uint64_t l2_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}

static int g_pdl = 0;
DK_EXPORT void dk_set_pdl(int on) { g_pdl = on; }

template <typename... KArgs, typename... Args>
static inline int dk_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                            Args... args) {
    if (grid.x == 0 || grid.y == 0 || grid.z == 0) return 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_pdl ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return (int)e;
    }
    return 0;
}

// Address of (page, kv head, slot in page) in a store laid out [pages, n_kv, DK_PAGE, hd].
__device__ __forceinline__ size_t kv_offset(int page, int n_kv, int kvh, int in_page, int hd) {
    return (((size_t)page * n_kv + kvh) * DK_PAGE + in_page) * (size_t)hd;
}

DK_EXPORT const char* dk_error_string(int e) { return cudaGetErrorString((cudaError_t)e); }
