// Shared helpers of the kernels: storage types, conversions, reductions, error codes.
//
// Every kernel keeps its arithmetic in float32 and converts only at loads and
// stores, as the reference's fp16 kernels do (src/qwen_kernels.cu:2-3, :10-11);
// the storage type here is bfloat16 or float32, chosen by the launcher's
// `dtype` argument (0 = float32, 1 = bfloat16).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>

#define KVB_API extern "C" __attribute__((visibility("default")))

// Return codes of the launchers (0 = launched; CUDA errors are returned as positive codes).
#define KVB_OK 0
#define KVB_ERR_DTYPE (-1)
#define KVB_ERR_SHAPE (-2)
#define KVB_ERR_ALIGN (-3)
#define KVB_ERR_LIMIT (-4)

// Bits of the device-side error word that kernels set instead of touching bad memory.
#define KVB_DEV_BAD_TOKEN 1   // a token id outside the vocabulary
#define KVB_DEV_BAD_PAGE 2    // a needed key or value lies in a page the block table does not hold
#define KVB_DEV_BAD_POS 4     // a position beyond the rotation table

enum { KVB_F32 = 0, KVB_BF16 = 1 };

typedef __nv_bfloat16 bf16;

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<bf16>(bf16 v) { return __bfloat162float(v); }

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

// Sum over the block in a fixed order (warp shuffles, then the warps' partials one by
// one), so a row's result does not depend on what else the launch holds.
// `scratch` holds at least 33 floats.  All threads receive the result.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
        for (int w = 0; w < nwarps; ++w) t += scratch[w];
        scratch[32] = t;
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
    if (threadIdx.x == 0) {
        float t = -FLT_MAX;
        for (int w = 0; w < nwarps; ++w) t = fmaxf(t, scratch[w]);
        scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// Programmatic dependent launch: a kernel launched with `kvb_launch` may be placed on the SMs while the
// kernel before it in the stream is still running; everything it does before `pdl_wait()` (parameter reads,
// prefetching weights, which no kernel writes) overlaps the predecessor's tail, and `pdl_wait()` returns only
// when the predecessor has completed and its writes are visible.  `pdl_launch_dependents()` lets the successor
// be placed as soon as every block of this kernel has started.  Kernels launched the ordinary way see both as
// no-ops.  KVB_PDL=0 in the environment turns the attribute off.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Thread-block clusters: a barrier over the cluster's blocks, and reads of another block's shared memory.
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// Split form: every block arrives when it starts and waits just before it first touches another block's shared
// memory - by then the others have long arrived, and all are known to be running.
__device__ __forceinline__ void cluster_arrive_started() { asm volatile("barrier.cluster.arrive.relaxed.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void cluster_wait_started() { asm volatile("barrier.cluster.wait.aligned;\n" ::: "memory"); }
__device__ __forceinline__ uint32_t peer_smem(const void* mine, uint32_t rank) {
    uint32_t out;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(out) : "r"((uint32_t)__cvta_generic_to_shared(mine)), "r"(rank));
    return out;
}
__device__ __forceinline__ float2 peer_ld2(uint32_t addr) {
    float2 v;
    asm volatile("ld.shared::cluster.v2.f32 {%0,%1}, [%2];\n" : "=f"(v.x), "=f"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ void peer_st4(uint32_t addr, const float4& v) {
    asm volatile("st.shared::cluster.v4.f32 [%0], {%1,%2,%3,%4};\n" ::"r"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
__device__ __forceinline__ void peer_st2(uint32_t addr, const float2& v) {
    asm volatile("st.shared::cluster.v2.f32 [%0], {%1,%2};\n" ::"r"(addr), "f"(v.x), "f"(v.y) : "memory");
}
__device__ __forceinline__ float4 peer_ld4(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0,%1,%2,%3}, [%4];\n" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}

#include <stdlib.h>
static inline bool kvb_pdl_enabled() {
    static int enabled = -1;
    if (enabled < 0) {
        const char* v = getenv("KVB_PDL");
        enabled = (v && v[0] == '0') ? 0 : 1;
    }
    return enabled == 1;
}

template <typename... KArgs, typename... Args>
static inline cudaError_t kvb_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                     Args... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = kvb_pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&config, kernel, static_cast<KArgs>(args)...);
}

// The same with thread-block clusters of `cluster_x` blocks along x (the grid's x must be a multiple of it).
template <typename... KArgs, typename... Args>
static inline cudaError_t kvb_launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, unsigned cluster_x, size_t smem,
                                             cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[2];
    attribute[0].id = cudaLaunchAttributeClusterDimension;
    attribute[0].val.clusterDim.x = cluster_x;
    attribute[0].val.clusterDim.y = 1;
    attribute[0].val.clusterDim.z = 1;
    attribute[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = kvb_pdl_enabled() ? 2 : 1;
    return cudaLaunchKernelEx(&config, kernel, static_cast<KArgs>(args)...);
}

// The number of SMs of the current device, asked once.
static inline int kvb_sm_count() {
    static int count = 0;
    if (count == 0) {
        int device = 0, found = 0;
        if (cudaGetDevice(&device) == cudaSuccess &&
            cudaDeviceGetAttribute(&found, cudaDevAttrMultiProcessorCount, device) == cudaSuccess && found > 0)
            count = found;
        else
            return 1;
    }
    return count;
}

static inline int kvb_launch_status() {
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? KVB_OK : (int)e;
}

#ifdef KVB_TRACE
// Debug builds only (-DKVB_TRACE): nanosecond time stamps of the phases of every block of the module's last
// kernel, slot i of block b at [b * 8 + i]; read back with kvb_trace_read.
__device__ long long kvb_trace_buf[8192 * 8];
__device__ __forceinline__ long long trace_now() {
    long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define TRACE(i)                                                                                              \
    if (threadIdx.x == 0) {                                                                                   \
        const int cta = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;                       \
        if (cta < 8192) kvb_trace_buf[cta * 8 + (i)] = trace_now();                                           \
    }
KVB_API int kvb_trace_read(long long* host, int count) {
    return (int)cudaMemcpyFromSymbol(host, kvb_trace_buf, sizeof(long long) * count);
}
#else
#define TRACE(i)
#endif
