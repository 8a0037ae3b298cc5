// Device helpers shared by the decode attention kernel and the fused decode layer: the rotation of a
// head's 16-byte chunks as they are loaded from the projection's output, and thin wrappers of the
// warp-level matrix instructions both kernels use for their small products.
#pragma once

#include "common.cuh"

// One 16-byte chunk (8 dims starting at dim 8 c) of a head of the projection's output for token b,
// rotated if it lies in the rotary part and scaled: the arithmetic of qkv_cache_bf16_kernel.
__device__ __forceinline__ uint4 ad_rotated_chunk(const __nv_bfloat16* head, int c, int half, const float* cs, const float* sn, float sc) {
    const uint4 raw = *(const uint4*)(head + c * 8);
    float v[8];
    {
        const __nv_bfloat162* p2 = (const __nv_bfloat162*)&raw;
#pragma unroll
        for (int e = 0; e < 4; ++e) { const float2 f = __bfloat1622float2(p2[e]); v[2 * e] = f.x; v[2 * e + 1] = f.y; }
    }
    const int hc = half >> 3;
    if (cs && c < 2 * hc) {
        const bool low = c < hc;
        const uint4 praw = *(const uint4*)(head + (low ? c + hc : c - hc) * 8);
        const __nv_bfloat162* q2 = (const __nv_bfloat162*)&praw;
        const float* csp = cs + (low ? c : c - hc) * 8;
        const float* snp = sn + (low ? c : c - hc) * 8;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(q2[e]);
            const float pw[2] = {f.x, f.y};
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                const float co = csp[2 * e + k], si = snp[2 * e + k];
                v[2 * e + k] = low ? v[2 * e + k] * co - pw[k] * si : pw[k] * si + v[2 * e + k] * co;
            }
        }
    }
    uint4 out;
    __nv_bfloat162 p0 = __floats2bfloat162_rn(v[0] * sc, v[1] * sc), p1 = __floats2bfloat162_rn(v[2] * sc, v[3] * sc);
    __nv_bfloat162 p2 = __floats2bfloat162_rn(v[4] * sc, v[5] * sc), p3 = __floats2bfloat162_rn(v[6] * sc, v[7] * sc);
    out.x = *(unsigned*)&p0; out.y = *(unsigned*)&p1; out.z = *(unsigned*)&p2; out.w = *(unsigned*)&p3;
    return out;
}

__device__ __forceinline__ unsigned ad_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ad_ldm4(unsigned addr, unsigned (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ad_ldm4t(unsigned addr, unsigned (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ad_mma(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

