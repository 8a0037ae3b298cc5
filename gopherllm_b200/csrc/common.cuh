// Shared declarations of the sm_100a kernels.
//
// Every launcher is an extern "C" function that takes raw device pointers, sizes
// and the CUDA stream, launches on that stream, allocates nothing and returns 0
// or a negative error code (see gl_error_string in the Python wrapper).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define GL_API extern "C" __attribute__((visibility("default")))

// element types of buffers passed by void*
enum GlDtype { GL_F32 = 0, GL_BF16 = 1 };

// activation applied in an epilogue
enum GlAct { GL_ACT_NONE = 0, GL_ACT_GELU_TANH = 1, GL_ACT_GELU_ERF = 2, GL_ACT_RELU = 3 };

// error codes
enum GlError {
    GL_OK = 0,
    GL_ERR_DTYPE = -1,      // combination of element types not built
    GL_ERR_SHAPE = -2,      // a size the kernel does not take
    GL_ERR_ALIGN = -3,      // a pointer or stride not aligned as required
    GL_ERR_LAUNCH = -4,     // cudaGetLastError() after the launch was not success
    GL_ERR_SMEM = -5,       // shared memory need exceeds the device limit
    GL_ERR_DRIVER = -6,     // a driver entry point could not be obtained or failed
    GL_ERR_SCRATCH = -7,    // the call needs more scratch than a built-in array holds
};

// tokens of the cache that share one page
#define GL_PAGE 64

// Programmatic dependent launch.  A kernel launched through gl_launch may begin while the
// kernel before it in the stream is still finishing: blocks are scheduled and run up to
// gl_grid_wait(), which returns once every kernel it depends on has completed and its writes
// are visible.  Everything a kernel reads from or writes to memory that an earlier kernel
// touches must therefore come after gl_grid_wait(); only constants of the launch (weights,
// barrier set-up) may come before.  gl_grid_launch_dependents() lets the next kernel start
// being scheduled.  Both are no-ops in a kernel launched the ordinary way.
static int gl_pdl = 1;
GL_API void gl_set_pdl(int on) { gl_pdl = on; }

#ifdef __CUDACC__
__device__ __forceinline__ void gl_grid_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void gl_grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
static int gl_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                     int cluster_x, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (gl_pdl) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cluster_x > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = cluster_x;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = 1;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    if (cudaLaunchKernelEx(&cfg, kernel, args...) != cudaSuccess) {
        cudaGetLastError();
        return -4;
    }
    return 0;
}
#endif

// A build with -DGL_DEBUG_BOUNDS checks the indices that kernels take from memory (token ids, page
// numbers, positions within a page table) before they use them.  A bad index is recorded (which kind,
// its value, the limit it broke, how many were seen) in a word the host reads, and the access is made at
// index 0 instead: the kernel runs on with a wrong result and an error on record, it never traps and
// never touches memory outside its buffers.  The host checks the same things before a step is launched;
// this is the second net, for an index that a kernel or a caller of the C entry points got wrong.
enum GlBoundsKind { GL_BAD_TOKEN = 1, GL_BAD_PAGE = 2, GL_BAD_POSITION = 3, GL_BAD_ROW = 4 };
#if defined(GL_DEBUG_BOUNDS) && defined(__CUDACC__)
__device__ int gl_bounds_word[4];      // [0] kind of the first bad index (0: none), [1] its value, [2] the limit, [3] how many
__device__ __forceinline__ int gl_checked(int v, int limit, int kind) {
    if ((unsigned)v < (unsigned)limit) return v;
    if (atomicCAS(&gl_bounds_word[0], 0, kind) == 0) { gl_bounds_word[1] = v; gl_bounds_word[2] = limit; }
    atomicAdd(&gl_bounds_word[3], 1);
    return 0;
}
// out4 receives the four words; clear sets them back to zero.  -1 if they could not be read.
GL_API int gl_bounds_status(int* out4, int clear) {
    if (cudaMemcpyFromSymbol(out4, gl_bounds_word, 4 * sizeof(int)) != cudaSuccess) return -1;
    if (clear && out4[0] != 0) {
        const int zero[4] = {0, 0, 0, 0};
        if (cudaMemcpyToSymbol(gl_bounds_word, zero, sizeof(zero)) != cudaSuccess) return -1;
    }
    return 0;
}
#else
#define gl_checked(v, limit, kind) (v)
#endif

static inline int gl_check_launch() {
    return cudaGetLastError() == cudaSuccess ? GL_OK : GL_ERR_LAUNCH;
}

__device__ __forceinline__ float gl_load(const float* p) { return *p; }
__device__ __forceinline__ float gl_load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void gl_store(float* p, float v) { *p = v; }
__device__ __forceinline__ void gl_store(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ float gl_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float gl_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Activations in 32-bit.  gelu "tanh form" is x*sigmoid(2*sqrt(2/pi)*(x+0.044715x^3)),
// the form the reference evaluates (fastmath.go:138-141); the erf form is
// 0.5*x*(1+erf(x/sqrt(2))) (bert.go:742-744).
// For results that are rounded to bfloat16 right away: the tanh form through the hardware's
// tanh.approx (relative error about 2^-11, below bfloat16's 2^-9 rounding).
__device__ __forceinline__ float gl_activate_bf16_grade(float x, int act) {
    if (act == GL_ACT_GELU_TANH) {
        float th;
        const float u = 0.7978845608028654f * x * fmaf(0.044715f * x, x, 1.0f);
        asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(u));
        const float hx = 0.5f * x;
        return fmaf(hx, th, hx);
    }
    if (act == GL_ACT_GELU_ERF) return 0.5f * x * (1.0f + erff(x * 0.70710678118654752440f));
    if (act == GL_ACT_RELU) return fmaxf(x, 0.0f);
    return x;
}

template <bool EXACT>
__device__ __forceinline__ float gl_activate(float x, int act) {
    switch (act) {
        case GL_ACT_GELU_TANH: {
            const float z = 1.5957691216057308f * (x + 0.044715f * x * x * x);
            const float e = EXACT ? expf(-z) : __expf(-z);
            return x / (1.0f + e);
        }
        case GL_ACT_GELU_ERF:
            return 0.5f * x * (1.0f + erff(x * 0.70710678118654752440f));
        case GL_ACT_RELU:
            return fmaxf(x, 0.0f);
        default:
            return x;
    }
}
