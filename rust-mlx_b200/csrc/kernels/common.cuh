// Shared helpers of the kernels: element types, loads and stores through float,
// fixed-order reductions, and the error channel of the C entry points.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define RMX_API extern "C" __attribute__((visibility("default")))

// dtype codes of the C interface
enum { RMX_F32 = 0, RMX_BF16 = 1 };

// Every entry point returns 0 or a negative code and leaves a message for rmx_last_error().
void rmx_set_error(const char* fmt, ...);
#define RMX_FAIL(...)                 \
    do {                              \
        rmx_set_error(__VA_ARGS__);   \
        return -1;                    \
    } while (0)
#define RMX_REQUIRE(cond, ...)        \
    do {                              \
        if (!(cond)) RMX_FAIL(__VA_ARGS__); \
    } while (0)
#define RMX_CHECK_LAUNCH(name)                                              \
    do {                                                                    \
        cudaError_t e__ = cudaGetLastError();                               \
        if (e__ != cudaSuccess) RMX_FAIL("%s: launch failed: %s", name, cudaGetErrorString(e__)); \
    } while (0)

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Butterfly reductions: every lane ends with the same value, formed in the same order
// whatever the data, so a row's result does not depend on what else is in the batch.
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

// Sum over a block of up to 1024 threads; `scratch` holds 32 floats.  Warps are added in
// index order by every thread alike.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    v = warp_sum(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float total = 0.f;
    for (int w = 0; w < nwarps; ++w) total += scratch[w];
    return total;
}

// Programmatic dependent launch.  Every kernel here lets its dependents go first thing (before its own wait): the
// kernel after it then takes its place and does what needs no input (a product fetches its first weight tiles) while
// this kernel still waits for the one before, so that the prologues of up to three kernels run ahead of the data.
// A dependent's wait returns only when this kernel has completed, which it cannot before its own wait has returned,
// so waiting for the kernel before covers the ones before that too.
// A kernel that is launched as a dependent of the one before it may start
// (and do what does not need that kernel's results, such as fetching weights) once every block of that
// kernel has called this or has ended.  It has no effect when the next kernel is launched the usual way.
__device__ __forceinline__ void allow_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }
// The other half: a kernel launched as a programmatic dependent waits here until the kernels before it on the
// stream have completed and their writes are visible.  Launched the usual way, it returns at once.
__device__ __forceinline__ void wait_for_prior_kernels() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }

// Whether kernels are launched as programmatic dependents (their blocks may take their places on the SMs while the
// kernel before them drains; each waits for it with wait_for_prior_kernels() before touching memory).
bool rmx_dependent_launch_enabled();

#include <utility>
// Launch `kernel` as a programmatic dependent of the work before it on the stream (or the usual way when that is
// switched off).  The kernel must call wait_for_prior_kernels() before it reads or writes global memory.
template <typename... KArgs, typename... Args>
cudaError_t launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = rmx_dependent_launch_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(std::forward<Args>(args))...);
}
// A kernel function's attributes (its limit of dynamic shared memory) are kept per device.  True the first time it
// is asked for `seen` with the current device, so that each entry point raises its kernel's limit once on every device.
inline bool rmx_first_on_device(bool (&seen)[64]) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return true;
    if (seen[dev]) return false;
    seen[dev] = true;
    return true;
}
#define RMX_CHECK_LAUNCHED(err, name)                                                     \
    do {                                                                                  \
        cudaError_t e__ = (err);                                                          \
        if (e__ != cudaSuccess) RMX_FAIL("%s: launch failed: %s", name, cudaGetErrorString(e__)); \
    } while (0)
