// Shared helpers of the sm_100a kernels: element types, conversions, reductions
// and the C calling convention of the library.
//
// Every exported function is `extern "C" int sb_<name>(..., cudaStream_t stream)`.
// It validates its arguments on the host, launches on `stream`, and returns 0 or a
// non-zero code: a cudaError_t from the launch, or SB_ERR_ARG (a size the kernel
// does not take; the text is in sb_last_error()).  Nothing allocates device memory;
// scratch buffers are passed in by the caller.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define SB_F32 0
#define SB_BF16 1
#define SB_ERR_ARG 100001

extern "C" const char* sb_last_error();
void sb_set_error(const char* fmt, ...);

#define SB_REQUIRE(cond, ...)                                   \
    do {                                                         \
        if (!(cond)) {                                           \
            sb_set_error(__VA_ARGS__);                           \
            return SB_ERR_ARG;                                   \
        }                                                        \
    } while (0)

#define SB_LAUNCH_CHECK()                                        \
    do {                                                         \
        cudaError_t e__ = cudaGetLastError();                    \
        if (e__ != cudaSuccess) {                                \
            sb_set_error("%s", cudaGetErrorString(e__));         \
            return (int)e__;                                     \
        }                                                        \
        return 0;                                                \
    } while (0)

namespace sb {

// Programmatic dependent launch.  Every kernel of the library is launched with the
// "programmatic stream serialization" attribute: it may start while the kernel before it
// in the stream is still running.  `pdl_launch_dependents()` lets the NEXT kernel start
// its own prologue; `pdl_wait()` returns once every earlier kernel has completed and its
// writes are visible.  Before pdl_wait() a kernel touches only memory no kernel of the
// step writes (weights, gains, tables of constants) and its own shared/tensor memory;
// it reads activations and writes anything global only after it.
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

bool pdl_enabled();    // host: false when SOCRATES_PDL=0

// Host: one flag per device, for set-up that the runtime keeps per device (a kernel's opt-in to
// large dynamic shared memory above all).  `flag()` is the current device's flag.  What such
// set-up caches beside the flag (SM counts) assumes that the devices of a process are alike.
struct OncePerDevice {
    bool done[64] = {};
    bool& flag() {
        int dev = 0;
        cudaGetDevice(&dev);
        return done[dev & 63];
    }
};

template <typename... KArgs, typename... Args>
inline cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
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
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// The same for a kernel whose blocks form clusters of `cluster` blocks (the grid a multiple of it in each dim).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                  dim3 cluster, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cluster.x;
    attr[0].val.clusterDim.y = cluster.y;
    attr[0].val.clusterDim.z = cluster.z;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

__device__ __forceinline__ float to_float(float x) { return x; }
__device__ __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_float(float x);
template <> __device__ __forceinline__ float from_float<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float x) {
    return __float2bfloat16_rn(x);
}

// 16-byte vector of T: 4 floats or 8 bf16.
template <typename T> struct Vec16;
template <> struct Vec16<float> {
    static constexpr int N = 4;
    float4 raw;
    __device__ __forceinline__ void load(const float* p) { raw = *reinterpret_cast<const float4*>(p); }
    __device__ __forceinline__ float get(int i) const { return reinterpret_cast<const float*>(&raw)[i]; }
};
template <> struct Vec16<__nv_bfloat16> {
    static constexpr int N = 8;
    uint4 raw;
    __device__ __forceinline__ void load(const __nv_bfloat16* p) { raw = *reinterpret_cast<const uint4*>(p); }
    __device__ __forceinline__ float get(int i) const {
        return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(&raw)[i]);
    }
};

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

// Sum over a block of up to 1024 threads; every thread gets the result.
// `scratch` is 33 floats of shared memory.  The order of additions is fixed.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
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

}  // namespace sb
