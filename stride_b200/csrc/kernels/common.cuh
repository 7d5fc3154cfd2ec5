// Shared helpers of the sm_100a kernels: element types, conversions, reductions
// and the launch-status convention.
//
// Every exported launcher is `extern "C"`, takes raw device pointers, sizes and
// a stream, validates its sizes on the host and returns 0 or a negative code
// (-1 bad argument, -2 unsupported size) or a positive cudaError_t. Nothing here
// allocates device memory.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdlib>

#define STRIDE_DTYPE_F32 0
#define STRIDE_DTYPE_BF16 1

#define STRIDE_BAD_ARGUMENT (-1)
#define STRIDE_UNSUPPORTED (-2)

#define STRIDE_LAUNCH_STATUS() static_cast<int>(cudaPeekAtLastError())

namespace stride {

// ------------------------------------------------ programmatic dependent launch
// Every kernel of the package is launched with the attribute that lets it start
// while the kernel before it on the stream is still finishing. A kernel calls
// pdl_trigger() at once (the next kernel may then be scheduled as soon as SMs
// have room) and pdl_wait() before it reads or writes anything another kernel
// touches; pdl_wait() returns when the kernel before it has completed and its
// writes are visible. What a kernel does before pdl_wait() overlaps the tail of
// its predecessor: block start-up, barrier and tensor-memory set-up, and, in the
// matrix products, the first TMA loads of the weights. Launched without the
// attribute (STRIDE_B200_PDL=0), both calls do nothing.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

inline bool pdl_enabled() {
    static const bool on = [] {
        const char* e = getenv("STRIDE_B200_PDL");
        return !(e && e[0] == '0');
    }();
    return on;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// The same for a kernel whose CTAs form clusters of `cluster_z` along z (CTAs of a cluster run at the same time on
// SMs of one GPC and can write into one another's shared memory).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_clusters(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, int cluster_z,
                                   Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = static_cast<unsigned>(cluster_z);
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ------------------------------------------------------------------ thread-block clusters
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// The barrier of the cluster, in two halves: every thread of every CTA arrives; a thread that waits goes on when all
// have (or have exited). What a thread wrote before it arrived, also into another CTA's shared memory, is visible to
// the threads that waited.
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire;" ::: "memory"); }
// Four floats into the shared memory of CTA `rank` of the cluster, at the place that `local` names in this CTA's.
__device__ __forceinline__ void store_cluster_f4(uint32_t local, uint32_t rank, float a, float b, float c, float d) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
    asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(remote), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// Two floats, the same way.
__device__ __forceinline__ void store_cluster_f2(uint32_t local, uint32_t rank, float a, float b) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
    asm volatile("st.shared::cluster.v2.f32 [%0], {%1, %2};" ::"r"(remote), "f"(a), "f"(b) : "memory");
}

__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T>
__device__ __forceinline__ T from_f32(float x);
template <>
__device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

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

// Sum over a block of up to 1024 threads; every thread gets the result. The
// order of the additions depends only on the block size.
__device__ __forceinline__ float block_sum(float v, float* scratch /* >= 32 floats */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float total = 0.f;
    for (int w = 0; w < nwarps; ++w) total += scratch[w];
    return total;
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float total = scratch[0];
    for (int w = 1; w < nwarps; ++w) total = fmaxf(total, scratch[w]);
    return total;
}

}  // namespace stride
