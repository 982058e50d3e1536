// Shared helpers for the sm_100a kernels: element types, loads and stores that
// widen to float, block reductions with a fixed order, and the error word.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

// Element type codes passed through the C interface.
#define SS_F32 0
#define SS_BF16 1

// Bits of the device error word that kernels set instead of trapping.
#define SS_ERR_TOKEN_RANGE 1   // a token id outside [0, vocab)
#define SS_ERR_SLOT_RANGE 2    // a cache slot outside the pool
#define SS_ERR_PAGE_RANGE 4    // a block-table entry outside the pool
#define SS_ERR_WAIT_LIMIT 8    // a bounded wait gave up

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_float<bf16>(float v) { return __float2bfloat16_rn(v); }

// A vector weight may be stored in 32-bit even when activations are bfloat16.
template <typename T>
__device__ __forceinline__ float load_vec(const void* base, int64_t i, int is_f32) {
    return is_f32 ? reinterpret_cast<const float*>(base)[i]
                  : to_float(reinterpret_cast<const T*>(base)[i]);
}

// silu(gate) * up, formed in float32.  FAST (the bfloat16 kernels): the approximate exponential and division,
// whose error (about 2^-21) is far below the rounding of the result to bfloat16; every bfloat16 kernel that forms
// this product uses the same expression, so a value does not depend on which of them ran.
template <bool FAST>
__device__ __forceinline__ float silu_mul(float g, float u) {
    return FAST ? __fdividef(g, 1.0f + __expf(-g)) * u : g / (1.0f + expf(-g)) * u;
}

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

// Sum over the block; every thread gets the result.  The order of additions
// depends on blockDim only, never on what else is in the batch.
__device__ __forceinline__ float block_sum(float v, float* scratch /* >= 33 floats */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
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

#define SS_LAUNCH_CHECK() (int)cudaGetLastError()

// ---------------------------------------------------------------- per-device set-up
// A kernel's opt-in to more than 48 KB of dynamic shared memory (cudaFuncSetAttribute) holds for one device
// only, so it is remembered per device, not per process.  Two host threads that make their first call on a device
// at the same moment both do the (idempotent) opt-in; nothing else is shared.
#define SS_MAX_DEVICES 64
struct SsPerDevice {
    unsigned char done[SS_MAX_DEVICES];
};

static inline int ss_current_device() {
    int dev = -1;
    return (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < SS_MAX_DEVICES) ? dev : -1;
}

template <typename K>
static inline int ss_opt_in_smem(K kernel, int bytes, SsPerDevice& state) {
    const int dev = ss_current_device();
    if (dev < 0) return (int)cudaErrorInvalidDevice;
    if (!state.done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        if (e != cudaSuccess) return (int)e;
        state.done[dev] = 1;
    }
    return 0;
}

// Streaming multiprocessors of the current device (asked once per device).
static inline int ss_sm_count() {
    static int count[SS_MAX_DEVICES];
    const int dev = ss_current_device();
    if (dev < 0) return 1;
    if (count[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n < 1) n = 1;
        count[dev] = n;
    }
    return count[dev];
}

// ---------------------------------------------------------------- programmatic dependent launch
// Kernels are launched so that the next kernel in the stream may start while this one is still running
// (cudaLaunchAttributeProgrammaticStreamSerialization).  A kernel calls pdl_launch_dependents() as early
// as it likes and must call pdl_wait() before it reads anything an earlier kernel wrote and before it
// writes anything an earlier kernel may still read; until then it may only touch constants (weights).
// In a decode step this lets a matrix product stream its weights while the small kernel before it runs.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

inline int& ss_pdl_flag() {
    static int enabled = 1;
    return enabled;
}

template <typename... KArgs, typename... Args>
static inline void ss_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                             Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ss_pdl_flag() ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// The same with the blocks along grid.z grouped into thread-block clusters of `cluster_z` (2..8): the blocks of
// a cluster run at the same time and can read one another's shared memory.
template <typename... KArgs, typename... Args>
static inline void ss_launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                     int cluster_z, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = cluster_z;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ss_pdl_flag() ? 2 : 1;
    cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Blocks along grid.x grouped into clusters of `cluster_x`.
template <typename... KArgs, typename... Args>
static inline void ss_launch_cluster_x(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                       int cluster_x, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cluster_x;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ss_pdl_flag() ? 2 : 1;
    cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

__device__ __forceinline__ void cluster_sync_all() {
    __syncwarp();
    asm volatile("barrier.cluster.arrive.release;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
}
// The barrier before a block of a cluster leaves: every block has finished READING the others' shared memory (its
// loads have returned: their values have been used).  Nothing written is handed over here, so the arrival need not
// wait for the thread's stores to global memory to be acknowledged, which a releasing arrival does (about a
// microsecond behind the output stores of a product's epilogue).
__device__ __forceinline__ void cluster_sync_before_exit() {
    __syncwarp();
    asm volatile("barrier.cluster.arrive.relaxed;" ::: "memory");
    asm volatile("barrier.cluster.wait;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// four floats (16-byte aligned) at the same shared-memory offset in block `rank` of this cluster
__device__ __forceinline__ float4 ld_cluster_f32x4(const float* local, uint32_t rank) {
    uint32_t addr = (uint32_t)__cvta_generic_to_shared(local), remote;
    float4 v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t cluster_size() {
    uint32_t n;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(n));
    return n;
}
// 64-bit word at the same shared-memory offset in block `rank` of this cluster
__device__ __forceinline__ unsigned long long ld_cluster_u64(const unsigned long long* local, uint32_t rank) {
    uint32_t addr = (uint32_t)__cvta_generic_to_shared(local), remote;
    unsigned long long v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
    asm volatile("ld.shared::cluster.u64 %0, [%1];" : "=l"(v) : "r"(remote) : "memory");
    return v;
}
// float at the same shared-memory offset in block `rank` of this cluster
__device__ __forceinline__ float ld_cluster_f32(const float* local, uint32_t rank) {
    uint32_t addr = (uint32_t)__cvta_generic_to_shared(local), remote;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    return v;
}
