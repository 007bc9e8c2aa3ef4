// Shared helpers for the engine's CUDA kernels (sm_100a).
//
// Every exported launcher is `extern "C"`, takes raw device pointers plus a `cudaStream_t` and returns a
// status: 0 on success, a negative CVB_E_* code when it refuses its arguments (the Python wrapper turns the
// code into an exception with the text from cvb_error_string), or the positive cudaError_t of a failed launch.
// Activations come in two element types selected by an integer code: 0 = float (the true 32-bit path),
// 1 = __nv_bfloat16.  All arithmetic between loads and stores is float; `rnd<T>` rounds to the activation
// type and back where the reference rounds (kernels/fused_ops.cu:27).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#define CVB_OK 0
#define CVB_E_DTYPE (-1)      // element type code is neither 0 (float) nor 1 (bf16)
#define CVB_E_SIZE (-2)       // a size is zero/negative where it must be positive, or beyond a kernel's limit
#define CVB_E_ALIGN (-3)      // a pointer or row length breaks the kernel's alignment rule
#define CVB_E_SHAPE (-4)      // sizes are inconsistent with one another (heads vs groups, rotary width, ...)
#define CVB_E_UNSUPPORTED (-5)  // this specialised kernel does not cover the configuration; use the general one
#define CVB_E_SCRATCH (-6)    // scratch memory is missing or too small

#define CVB_DTYPE_F32 0
#define CVB_DTYPE_BF16 1

namespace cvb {

__device__ __forceinline__ float to_float(float x) { return x; }
__device__ __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_float(float x);
template <> __device__ __forceinline__ float from_float<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

// Round to the activation type and come back: identity in the 32-bit path.
template <typename T> __device__ __forceinline__ float rnd(float x) { return to_float(from_float<T>(x)); }

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

// Sum over the block; every thread receives the result.  `scratch` holds at least 32 floats.  The partial
// sums are added in warp order so that the result does not depend on scheduling.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    v = warp_sum(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = (blockDim.x + 31) >> 5;
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = 0.f;
    for (int i = 0; i < n_warps; ++i) r += scratch[i];
    __syncthreads();
    return r;
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
    v = warp_max(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = (blockDim.x + 31) >> 5;
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = scratch[0];
    for (int i = 1; i < n_warps; ++i) r = fmaxf(r, scratch[i]);
    __syncthreads();
    return r;
}

// Programmatic dependent launch.  Most kernels of the package start with pdl_trigger() (the next kernel in the stream
// may be scheduled as soon as all blocks of this one have started) and pdl_wait() (blocks until the kernels before this
// one have completed and their writes are visible).  Nothing that depends on an earlier kernel's output is read, and
// nothing is written, before pdl_wait(); a kernel may fetch weights before it.  This hides launch gaps between the short
// kernels of eagerly launched steps (prompt portions).  Launched through launch_kernel, a kernel does not take the
// attribute while a CUDA graph is being captured: measured on a B200, a decode step replayed from a graph in which every
// kernel had a programmatic edge ran 8 % slower than with plain edges, because blocks that arrive early land unevenly
// on SMs that the kernel in front still occupies.  The kernels of the decode chain (gemv_bf16.cu: gemv_stream_kernel;
// attention_bf16.cu: the fused decode attention) are written for such edges and take them inside graphs too, through
// launch_kernel_dependent: one block per SM, at most half an SM's shared memory, the trigger placed where the successor's
// early work does not get in the way.  Both instructions do nothing in a kernel that was launched without the attribute.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

inline bool pdl_enabled() {
    static const bool on = [] { const char* e = getenv("CVB_NO_PDL"); return !(e && e[0] == '1'); }();
    return on;
}

template <typename... KArgs, typename... Args>
inline void launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 0;
    if (pdl_enabled()) {
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(stream, &cap) == cudaSuccess && cap == cudaStreamCaptureStatusNone) cfg.numAttrs = 1;
    }
    cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// The same launch with the attribute decided by the caller: kernels written for a chain of dependent launches (they ask
// for what depends on no kernel before griddepcontrol.wait, and size their blocks so that the blocks of two neighbouring
// kernels share an SM evenly) take it inside captured graphs as well.
template <typename... KArgs, typename... Args>
inline void launch_kernel_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, bool dependent,
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
    cfg.numAttrs = (dependent && pdl_enabled()) ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

inline int launch_status() {
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? CVB_OK : static_cast<int>(e);
}

}  // namespace cvb

// Dispatch on the element type code.  `CALL` is a macro taking the C++ type.
#define CVB_DISPATCH_DTYPE(code, CALL)                       \
    do {                                                     \
        if ((code) == CVB_DTYPE_F32) { CALL(float); }        \
        else if ((code) == CVB_DTYPE_BF16) { CALL(__nv_bfloat16); } \
        else return CVB_E_DTYPE;                             \
    } while (0)
