// TMA (cp.async.bulk.tensor) and mbarrier helpers for sm_100a, and the host side
// of tensor maps.  Loads here never use cluster multicast.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"

// ---------------------------------------------------------------------------
// host: tensor maps for row-major bf16 matrices [rows, cols], 128-byte swizzle
// ---------------------------------------------------------------------------
typedef CUresult (*gl_encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                       const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                       CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                       CUtensorMapFloatOOBfill);

static gl_encode_tiled_fn gl_get_encode() {
    static gl_encode_tiled_fn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (gl_encode_tiled_fn)p;
        else
            cudaGetLastError();
    }
    return fn;
}

// A box of box_rows x box_cols elements over a row-major matrix of bf16 (elem_bytes 2) or f32 (4)
// whose rows lie pitch_elems apart (0: cols).  The box's row (box_cols * elem_bytes = 128, 64 or 32
// bytes) is the swizzle span.  Elements outside the matrix read as zero and are not written.
static int gl_make_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols,
                       uint32_t box_rows, uint32_t box_cols, uint32_t elem_bytes, uint64_t pitch_elems = 0) {
    gl_encode_tiled_fn enc = gl_get_encode();
    if (!enc) return GL_ERR_DRIVER;
    const uint64_t pitch = pitch_elems ? pitch_elems : cols;       // elements between rows
    if (((uintptr_t)base & 15) || (pitch * elem_bytes) % 16) return GL_ERR_ALIGN;
    const uint32_t row_bytes = box_cols * elem_bytes;              // the swizzle span is the box's row
    const CUtensorMapSwizzle swz = row_bytes >= 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                                 : row_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                                 : row_bytes == 32 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_NONE;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {pitch * elem_bytes};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2,
                     const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? GL_OK : GL_ERR_DRIVER;
}

// Tensor maps of long-lived matrices (weights) are encoded once and kept.
struct GlMapKey {
    const void* base; uint64_t rows, cols, pitch; uint32_t box_rows, box_cols, elem_bytes;
    bool operator==(const GlMapKey& o) const {
        return base == o.base && rows == o.rows && cols == o.cols && pitch == o.pitch && box_rows == o.box_rows &&
               box_cols == o.box_cols && elem_bytes == o.elem_bytes;
    }
};
struct GlMapKeyHash {
    size_t operator()(const GlMapKey& k) const {
        size_t h = (size_t)k.base;
        h ^= k.rows * 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
        h ^= (k.cols + 31 * k.pitch) * 0xC2B2AE3D27D4EB4Full + (h << 6) + (h >> 2);
        h ^= ((size_t)k.box_rows << 32 | k.box_cols) + k.elem_bytes + (h << 6) + (h >> 2);
        return h;
    }
};
static int gl_cached_map(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols,
                         uint32_t box_rows, uint32_t box_cols, uint32_t elem_bytes, uint64_t pitch_elems = 0) {
    static std::unordered_map<GlMapKey, CUtensorMap, GlMapKeyHash> cache;
    static std::mutex mu;
    GlMapKey key{base, rows, cols, pitch_elems, box_rows, box_cols, elem_bytes};
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it == cache.end()) {
        CUtensorMap m;
        int rc = gl_make_map(&m, base, rows, cols, box_rows, box_cols, elem_bytes, pitch_elems);
        if (rc != GL_OK) return rc;
        if (cache.size() > 4096) cache.clear();
        it = cache.emplace(key, m).first;
    }
    memcpy(out, &it->second, sizeof(CUtensorMap));
    return GL_OK;
}
static int gl_cached_map_bf16(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols,
                              uint32_t box_rows, uint32_t box_cols) {
    return gl_cached_map(out, base, rows, cols, box_rows, box_cols, 2);
}

// ---------------------------------------------------------------------------
// device
// ---------------------------------------------------------------------------
#ifdef __CUDACC__
// A wait that ran out sets this word; launchers expose it to the host.
__device__ int gl_wait_failed = 0;

// The word as the host sees it: 1 if a bounded wait of this library ran out since the word was last
// cleared (what that launch computed, and everything computed from it, is invalid), -1 if the word
// could not be read.  ``clear`` sets it back to 0 once read.  The copy waits for the device.
GL_API int gl_wait_status(int clear) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, gl_wait_failed, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0 && clear) {
        const int zero = 0;
        if (cudaMemcpyToSymbol(gl_wait_failed, &zero, sizeof(int)) != cudaSuccess) return -1;
    }
    return v;
}

#ifndef GL_SPIN_LIMIT
#define GL_SPIN_LIMIT (1u << 22)      // tries before a wait gives up (each try may itself sleep briefly)
#endif

__device__ __forceinline__ unsigned gl_smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned bar, unsigned parity) {
    unsigned ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// the same question without waiting at all
__device__ __forceinline__ bool mbar_test(unsigned bar, unsigned parity) {
    unsigned ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: false (and the failure word set) if the phase never completed.
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity) {
    for (unsigned i = 0; i < GL_SPIN_LIMIT; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    atomicExch(&gl_wait_failed, 1);
    return false;
}
// 2-D tile load: x is the inner (contiguous) coordinate in elements and must be a multiple
// of 8 for 16-bit types (a TMA copy starts on a 16-byte boundary); y is the row.
__device__ __forceinline__ void tma_load_2d(unsigned dst, const CUtensorMap* map, int x, int y, unsigned bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
// Tile in shared memory added onto a tile of a 32-bit tensor in global memory (elements
// outside the tensor are skipped); completion is tracked by the thread's bulk-copy groups.
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* map, int x, int y, unsigned src) {
    asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%1, %2}], [%3];"
                 ::"l"(map), "r"(x), "r"(y), "r"(src) : "memory");
}
// Tile in shared memory written to a tile of a tensor in global memory (elements outside the
// tensor are skipped).
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, int x, int y, unsigned src) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];"
                 ::"l"(map), "r"(x), "r"(y), "r"(src) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// until the shared-memory sources of all but the newest n groups have been read
template <int N>
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait() { asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
#endif
