// Prefill attention: runs of many new tokens against the paged bfloat16 cache
// (their own keys included), causal, with an optional window.
//
// A block takes 64 consecutive query rows of one (sequence, head); each of its 4
// warps owns 16 rows.  Key/value pages (64 positions, contiguous per head) stream
// through shared memory with cp.async, two pages in flight.  Scores and the
// output are mma.sync.m16n8k16 products with 32-bit accumulators; the maximum,
// the sum and the rescaling of the running softmax are 32-bit.  Rows past a
// sequence's length are zero-filled on load, so stale cache contents cannot
// reach a product.  The head size is a compile-time constant (GL_HEAD_DIM).
#include "common.cuh"

#ifndef GL_HEAD_DIM
#error "compile with -DGL_HEAD_DIM=<head size>: this file is built once per head size a model uses, and knows none itself"
#endif
static_assert(GL_HEAD_DIM % 16 == 0 && GL_HEAD_DIM >= 16 && GL_HEAD_DIM <= 256, "head size: 16..256 in steps of 16");

#define AP_HD GL_HEAD_DIM
#define AP_BM 64
#define AP_THREADS 128
#define AP_KS (AP_HD / 16)            // k-steps of the score product
#define AP_NT (AP_HD / 8)             // 8-wide column tiles of the output
#define AP_CHUNKS (AP_HD / 8)         // 16-byte chunks per row
#define AP_ROW (AP_HD * 2 + 16)       // padded row: 8 consecutive rows fall in distinct banks
#define AP_TILE (64 * AP_ROW)

struct AttnArgs {
    const void* q;            // [T, nH*hd] bf16, already scaled
    void* out;                // [T, nH*hd] bf16
    const void* k_cache;      // [pages, nKV, GL_PAGE, hd] bf16
    const void* v_cache;
    const int* seq_qstart;    // [B]
    const int* seq_qlen;      // [B]
    const int* seq_ctx;       // [B]
    const int* pages;         // [B, max_pages]
    int B, nH, nKV, hd, max_pages, window, max_qlen;
    float score_scale;
};

__device__ __forceinline__ unsigned ap_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ap_cp16(unsigned dst, const void* src, int bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void ap_commit() { asm volatile("cp.async.commit_group;"); }
template <int N>
__device__ __forceinline__ void ap_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }
__device__ __forceinline__ void ap_ldm4(unsigned addr, unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ap_ldm4t(unsigned addr, unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ap_mma(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned ap_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *(unsigned*)&v;
}

// rows [0, n_valid) of a page tile (or of the query tile) to padded shared memory; the rest is zero
__device__ __forceinline__ void ap_load_rows(unsigned dst, const __nv_bfloat16* src, size_t src_row_stride, int n_valid) {
    for (int i = threadIdx.x; i < 64 * AP_CHUNKS; i += AP_THREADS) {
        const int r = i / AP_CHUNKS, c = i - r * AP_CHUNKS;
        const bool ok = r < n_valid;
        ap_cp16(dst + r * AP_ROW + c * 16, ok ? (const void*)(src + (size_t)r * src_row_stride + c * 8) : (const void*)src,
                ok ? 16 : 0);
    }
}

__global__ void __launch_bounds__(AP_THREADS)
attn_prefill_kernel(AttnArgs a) {
    extern __shared__ __align__(16) unsigned char smem[];
    const unsigned sQ = ap_smem(smem);
    const unsigned sK[2] = {sQ + AP_TILE, sQ + 3 * AP_TILE};
    const unsigned sV[2] = {sQ + 2 * AP_TILE, sQ + 4 * AP_TILE};
    const int b = blockIdx.z, h = blockIdx.y;
    const int qlen = a.seq_qlen[b];
    const int n_qtiles = (qlen + AP_BM - 1) / AP_BM;
    const int qt = n_qtiles - 1 - (int)blockIdx.x;           // longest rows first
    if (qt < 0) return;
    const int ctx = a.seq_ctx[b], qstart = a.seq_qstart[b];
    const int q0 = qt * AP_BM;
    const int rows = min(AP_BM, qlen - q0);
    const int g = h / (a.nH / a.nKV);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int grp = lane >> 2, t = lane & 3;
    const int p_first = ctx + q0, p_last = ctx + q0 + rows - 1;
    const int lo_first = (a.window > 0 && p_first - a.window + 1 > 0) ? p_first - a.window + 1 : 0;
    const int page_begin = lo_first / GL_PAGE, page_end = p_last / GL_PAGE + 1;
    const int* pg = a.pages + (size_t)b * a.max_pages;
    const __nv_bfloat16* K = (const __nv_bfloat16*)a.k_cache;
    const __nv_bfloat16* V = (const __nv_bfloat16*)a.v_cache;
    const size_t head_off = (size_t)g * GL_PAGE * AP_HD, page_stride = (size_t)a.nKV * GL_PAGE * AP_HD;
    const int total = ctx + qlen;

    // the query tile, then the first page
    ap_load_rows(sQ, (const __nv_bfloat16*)a.q + ((size_t)(qstart + q0) * a.nH + h) * AP_HD, (size_t)a.nH * AP_HD, rows);
    {
        const size_t off = (size_t)pg[page_begin] * page_stride + head_off;
        const int nv = min(GL_PAGE, total - page_begin * GL_PAGE);
        ap_load_rows(sK[0], K + off, AP_HD, nv);
        ap_load_rows(sV[0], V + off, AP_HD, nv);
    }
    ap_commit();

    unsigned qf[AP_KS][4];
    float o[AP_NT][4];
#pragma unroll
    for (int i = 0; i < AP_NT; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[i][e] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const float LOG2E = 1.4426950408889634f;
    const int r_lo = warp * 16 + grp, r_hi = r_lo + 8;        // this thread's two rows inside the tile
    const int pos_lo = p_first + r_lo, pos_hi = p_first + r_hi;
    const int wlo_lo = (a.window > 0 && pos_lo - a.window + 1 > 0) ? pos_lo - a.window + 1 : 0;
    const int wlo_hi = (a.window > 0 && pos_hi - a.window + 1 > 0) ? pos_hi - a.window + 1 : 0;

    for (int p = page_begin; p < page_end; ++p) {
        const int st = (p - page_begin) & 1;
        if (p + 1 < page_end) {
            const size_t off = (size_t)pg[p + 1] * page_stride + head_off;
            const int nv = min(GL_PAGE, total - (p + 1) * GL_PAGE);
            ap_load_rows(sK[st ^ 1], K + off, AP_HD, nv);
            ap_load_rows(sV[st ^ 1], V + off, AP_HD, nv);
        }
        ap_commit();
        ap_wait<1>();
        __syncthreads();
        if (p == page_begin) {
#pragma unroll
            for (int kk = 0; kk < AP_KS; ++kk) {
                const int r = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                const int c = kk * 2 + (lane >> 4);
                ap_ldm4(sQ + r * AP_ROW + c * 16, qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3]);
            }
        }
        const int j0 = p * GL_PAGE;
        // a warp whose rows all lie before this page has nothing to do here (causal)
        const bool warp_active = j0 <= p_first + warp * 16 + 15;
        if (warp_active) {
            float s[8][4];
#pragma unroll
            for (int j = 0; j < 8; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
#pragma unroll
            for (int kk = 0; kk < AP_KS; ++kk) {
#pragma unroll
                for (int j = 0; j < 8; j += 2) {
                    unsigned b0, b1, b2, b3;
                    const int r = j * 8 + ((lane >> 4) & 1) * 8 + (lane & 7);
                    const int c = kk * 2 + ((lane >> 3) & 1);
                    ap_ldm4(sK[st] + r * AP_ROW + c * 16, b0, b1, b2, b3);
                    ap_mma(s[j], qf[kk], b0, b1);
                    ap_mma(s[j + 1], qf[kk], b2, b3);
                }
            }
            // mask: a row at position x sees keys max(0, x-window+1) .. x
            const bool need_mask = (j0 + GL_PAGE - 1 > p_first + warp * 16) || (a.window > 0 && j0 < wlo_hi + 8);
            if (need_mask) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int key = j0 + j * 8 + 2 * t + (e & 1);
                        const int pos = (e < 2) ? pos_lo : pos_hi;
                        const int wl = (e < 2) ? wlo_lo : wlo_hi;
                        if (key > pos || key < wl) s[j][e] = -INFINITY;
                    }
                }
            }
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                mx[0] = fmaxf(mx[0], fmaxf(s[j][0], s[j][1]));
                mx[1] = fmaxf(mx[1], fmaxf(s[j][2], s[j][3]));
            }
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
                mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
            }
            float corr[2], mu[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const float m_new = fmaxf(m_run[i], mx[i]);
                mu[i] = (m_new == -INFINITY) ? 0.f : m_new * LOG2E;
                corr[i] = exp2f(m_run[i] * LOG2E - mu[i]);       // m_run = -inf gives 0
                m_run[i] = m_new;
                l_run[i] *= corr[i];
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                s[j][0] = exp2f(s[j][0] * LOG2E - mu[0]);
                s[j][1] = exp2f(s[j][1] * LOG2E - mu[0]);
                s[j][2] = exp2f(s[j][2] * LOG2E - mu[1]);
                s[j][3] = exp2f(s[j][3] * LOG2E - mu[1]);
                l_run[0] += s[j][0] + s[j][1];
                l_run[1] += s[j][2] + s[j][3];
            }
#pragma unroll
            for (int i = 0; i < AP_NT; ++i) {
                o[i][0] *= corr[0]; o[i][1] *= corr[0];
                o[i][2] *= corr[1]; o[i][3] *= corr[1];
            }
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                unsigned pa[4];
                pa[0] = ap_pack(s[2 * kk][0], s[2 * kk][1]);
                pa[1] = ap_pack(s[2 * kk][2], s[2 * kk][3]);
                pa[2] = ap_pack(s[2 * kk + 1][0], s[2 * kk + 1][1]);
                pa[3] = ap_pack(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
                for (int dn = 0; dn < AP_NT; dn += 2) {
                    unsigned b0, b1, b2, b3;
                    const int r = kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
                    const int c = dn + (lane >> 4);
                    ap_ldm4t(sV[st] + r * AP_ROW + c * 16, b0, b1, b2, b3);
                    ap_mma(o[dn], pa, b0, b1);
                    ap_mma(o[dn + 1], pa, b2, b3);
                }
            }
        }
        __syncthreads();
    }
    ap_wait<0>();
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
    }
    const float inv_lo = l_run[0] > 0.f ? 1.f / l_run[0] : 0.f;
    const float inv_hi = l_run[1] > 0.f ? 1.f / l_run[1] : 0.f;
    __nv_bfloat16* O = (__nv_bfloat16*)a.out;
#pragma unroll
    for (int i = 0; i < AP_NT; ++i) {
        const int d = i * 8 + 2 * t;
        if (r_lo < rows)
            *(unsigned*)(O + ((size_t)(qstart + q0 + r_lo) * a.nH + h) * AP_HD + d) = ap_pack(o[i][0] * inv_lo, o[i][1] * inv_lo);
        if (r_hi < rows)
            *(unsigned*)(O + ((size_t)(qstart + q0 + r_hi) * a.nH + h) * AP_HD + d) = ap_pack(o[i][2] * inv_hi, o[i][3] * inv_hi);
    }
}

GL_API int gl_attention_prefill_head_dim() { return AP_HD; }

GL_API int gl_attention_prefill(const AttnArgs* args, cudaStream_t stream) {
    const AttnArgs& a = *args;
    if (a.B <= 0 || a.max_qlen <= 0) return GL_OK;
    if (a.hd != AP_HD || a.nH <= 0 || a.nKV <= 0 || a.nH % a.nKV) return GL_ERR_SHAPE;
    if (a.B > 65535 || a.nH > 65535 || a.score_scale != 1.0f) return GL_ERR_SHAPE;
    const size_t smem = 5 * (size_t)AP_TILE;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(attn_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
            cudaGetLastError();
            return GL_ERR_SMEM;
        }
        configured = true;
    }
    dim3 grid((a.max_qlen + AP_BM - 1) / AP_BM, a.nH, a.B);
    attn_prefill_kernel<<<grid, AP_THREADS, smem, stream>>>(a);
    return gl_check_launch();
}
