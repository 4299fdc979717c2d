// Shared helpers of the kuiperllama_b200 kernels (sm_100a).
//
// Every kernel file exports plain C entry points that take raw device pointers, sizes and
// a cudaStream_t, allocate nothing and return 0 or an error code; the Python side
// (csrc/ops.py) checks shapes and types before it calls them.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define KL_API extern "C" __attribute__((visibility("default")))

// Return codes of the C entry points.
enum : int {
    KL_OK = 0,
    KL_ERR_BAD_DTYPE = -1,      // a dtype code the kernel has no instance for
    KL_ERR_BAD_SIZE = -2,       // a size the kernel refuses (message printed to stderr)
    KL_ERR_BAD_ALIGN = -3,      // a pointer or stride that is not aligned as the kernel needs
    KL_ERR_DEVICE_STATUS = -4,  // a kernel reported through its status word (bounded wait ran out)
    KL_ERR_SETUP = -5,          // a driver or runtime call at set-up failed
};

// dtype codes shared with csrc/ops.py
enum : int { KL_F32 = 0, KL_BF16 = 1 };

#define KL_LAUNCH_CHECK()                                  \
    do {                                                   \
        cudaError_t e__ = cudaGetLastError();              \
        if (e__ != cudaSuccess) return (int)e__;           \
    } while (0)

#define KL_CUDA(call)                                      \
    do {                                                   \
        cudaError_t e__ = (call);                          \
        if (e__ != cudaSuccess) return (int)e__;           \
    } while (0)

namespace kl {

typedef __nv_bfloat16 bf16;

// Programmatic dependent launch.  Every kernel of this package is launched with the
// programmatic-stream-serialization attribute (unless KL_PDL=0 is in the environment): it may
// start while the kernel before it in the stream is still running.  A kernel therefore calls
// pdl_wait() before it reads anything another kernel wrote or writes anything at all; what it
// does before that (barrier set-up, tensor-memory allocation, loads of weights, which no
// kernel writes) overlaps the tail of its predecessor.  pdl_launch_dependents() at the top
// lets the next kernel in the stream do the same with this one.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

inline bool pdl_enabled() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("KL_PDL");
        v = (e != nullptr && e[0] == '0') ? 0 : 1;
    }
    return v != 0;
}

// Launch on `stream`; a failure is left for cudaGetLastError (KL_LAUNCH_CHECK).  `cluster_x` > 1
// launches thread-block clusters of that many CTAs along x (the grid's x must be a multiple of it).
template <typename... KArgs, typename... Args>
inline void launch_kernel_clustered(void (*kernel)(KArgs...), int cluster_x, dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    Args&&... args) {
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (pdl_enabled()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cluster_x > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = (unsigned)cluster_x;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = 1;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
template <typename... KArgs, typename... Args>
inline void launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
    launch_kernel_clustered(kernel, 1, grid, block, smem, stream, static_cast<Args&&>(args)...);
}

// Streaming multiprocessors of the current device (asked of the driver once per device; 0 on error).
inline int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
        cached[dev] = n;
    }
    return cached[dev];
}

// Grid of a grid-stride kernel over `items`: enough CTAs of `threads` for all of them, at most
// `per_sm` for every multiprocessor of the device.
inline int strided_grid(size_t items, int threads, int per_sm) {
    const size_t need = (items + threads - 1) / threads;
    const size_t cap = (size_t)(sm_count() > 0 ? sm_count() : 1) * per_sm;
    return (int)(need < cap ? need : cap);
}

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

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

// Sum over a CTA whose size is a multiple of 32 (at most 1024 threads).  Every thread gets
// the result.  `scratch` holds 33 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();                       // scratch may still be read from an earlier call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// Paged cache addressing.  One cache entry (one execution of a layer) stores keys (or
// values) as [n_pages][kv_heads][PAGE][head_dim]; a sequence's logical block b lives in page
// block_table[slot * blocks_per_seq + b].
constexpr int PAGE = 64;

__device__ __forceinline__ size_t cache_row_offset(const int* __restrict__ block_table, int blocks_per_seq,
                                                   int slot, int pos, int kv_head, int kv_heads, int head_dim) {
    const int page = block_table[(size_t)slot * blocks_per_seq + (pos / PAGE)];
    return (((size_t)page * kv_heads + kv_head) * PAGE + (pos % PAGE)) * (size_t)head_dim;
}

}  // namespace kl
