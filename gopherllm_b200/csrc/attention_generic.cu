// Attention over the paged cache with 32-bit arithmetic, for any head size and
// any element type: the kernel of the 32-bit path and the one the fast kernels
// are checked against.
//
// One warp owns one query row (token, head); the warps of a block are
// consecutive tokens of one sequence and share the key/value tiles they stage
// in shared memory.  Scores, the running maximum, the sum and the output
// accumulate in 32-bit (the reference: model.go:3346-3366, 3801-3855; it makes
// two passes, this one rescales on the fly, which differs by rounding only).
// A query at position p sees keys lo..p, lo = 0 or p-window+1
// (model.go:2707-2710); nothing else masks.
#include "common.cuh"

struct AttnArgs {
    const void* q;            // [T, nH*hd] activation type, already scaled
    void* out;                // [T, nH*hd] activation type
    const void* k_cache;      // [pages, nKV, GL_PAGE, hd] cache type
    const void* v_cache;
    const int* seq_qstart;    // [B] row of each sequence's first token
    const int* seq_qlen;      // [B] tokens of each sequence in this step
    const int* seq_ctx;       // [B] positions cached before this step
    const int* pages;         // [B, max_pages]
    int B, nH, nKV, hd, max_pages, window, max_qlen;
    float score_scale;
    int n_pages;              // pages of the cache entry (read by builds that check indices; 0: unknown)
};

#define AG_ROWS 8

template <typename TA, typename TC, int NACC>
__global__ void __launch_bounds__(AG_ROWS * 32)
attn_generic_kernel(AttnArgs a) {
    extern __shared__ float smem[];
    const int hd = a.hd, ks = hd + 1;
    float* Ks = smem;                       // [GL_PAGE][hd+1]
    float* Vs = Ks + GL_PAGE * ks;          // [GL_PAGE][hd]
    float* Qs = Vs + GL_PAGE * hd;          // [AG_ROWS][hd]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = blockIdx.z, h = blockIdx.y;
    const int qlen = a.seq_qlen[b];
    const int row0 = blockIdx.x * AG_ROWS;
    if (row0 >= qlen) return;
    const int ctx = a.seq_ctx[b];
    const int total = ctx + qlen;
    const int g = h / (a.nH / a.nKV);
    const int idx = row0 + warp;
    const bool live = idx < qlen;
    const int p = ctx + idx;                               // this row's position
    const int lo = (a.window > 0 && p - a.window + 1 > 0) ? p - a.window + 1 : 0;
    const int rows_here = min(AG_ROWS, qlen - row0);
    const int p_first = ctx + row0, p_last = ctx + row0 + rows_here - 1;
    const int lo_cta = (a.window > 0 && p_first - a.window + 1 > 0) ? p_first - a.window + 1 : 0;

    float* qv = Qs + warp * hd;
    if (live) {
        const TA* qsrc = (const TA*)a.q + ((size_t)(a.seq_qstart[b] + idx) * a.nH + h) * hd;
        for (int d = lane; d < hd; d += 32) qv[d] = gl_load(qsrc + d) * a.score_scale;
    }
    float acc[NACC];
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;

    const int* pg = a.pages + (size_t)b * a.max_pages;
    for (int page_i = lo_cta / GL_PAGE; page_i <= p_last / GL_PAGE; ++page_i) {
        const int page = gl_checked(pg[gl_checked(page_i, a.max_pages, GL_BAD_POSITION)], a.n_pages > 0 ? a.n_pages : 0x7fffffff, GL_BAD_PAGE);
        const TC* kp = (const TC*)a.k_cache + ((size_t)page * a.nKV + g) * GL_PAGE * hd;
        const TC* vp = (const TC*)a.v_cache + ((size_t)page * a.nKV + g) * GL_PAGE * hd;
        const int j0 = page_i * GL_PAGE;
        __syncthreads();
        for (int e = threadIdx.x; e < GL_PAGE * hd; e += blockDim.x) {
            const int r = e / hd, d = e - r * hd;
            const bool ok = j0 + r < total;       // rows past the sequence were never written
            Ks[r * ks + d] = ok ? gl_load(kp + e) : 0.f;
            Vs[r * hd + d] = ok ? gl_load(vp + e) : 0.f;
        }
        __syncthreads();
        if (!live) continue;
#pragma unroll 1
        for (int half = 0; half < GL_PAGE / 32; ++half) {
            const int jj = half * 32 + lane, j = j0 + jj;
            const bool ok = j >= lo && j <= p;
            float s = -INFINITY;
            if (ok) {
                const float* kr = Ks + jj * ks;
                float d0 = 0.f;
                for (int d = 0; d < hd; ++d) d0 = fmaf(qv[d], kr[d], d0);
                s = d0;
            }
            const float m_new = fmaxf(m, gl_warp_max(s));
            if (m_new == -INFINITY) continue;
            const float pj = ok ? expf(s - m_new) : 0.f;
            const float corr = expf(m - m_new);            // m = -inf gives 0
            l = l * corr + gl_warp_sum(pj);
            m = m_new;
#pragma unroll
            for (int i = 0; i < NACC; ++i) acc[i] *= corr;
            const float* vr = Vs + half * 32 * hd;
            for (int k = 0; k < 32; ++k) {
                const float pk = __shfl_sync(0xffffffffu, pj, k);
#pragma unroll
                for (int i = 0; i < NACC; ++i) {
                    const int d = lane + 32 * i;
                    if (d < hd) acc[i] = fmaf(pk, vr[k * hd + d], acc[i]);
                }
            }
        }
    }
    if (!live) return;
    const float inv = l > 0.f ? 1.0f / l : 0.f;
    TA* o = (TA*)a.out + ((size_t)(a.seq_qstart[b] + idx) * a.nH + h) * hd;
#pragma unroll
    for (int i = 0; i < NACC; ++i) {
        const int d = lane + 32 * i;
        if (d < hd) gl_store(o + d, acc[i] * inv);
    }
}

template <typename TA, typename TC, int NACC>
static int launch_generic(const AttnArgs& a, cudaStream_t stream) {
    const size_t smem = ((size_t)GL_PAGE * (a.hd + 1) + (size_t)GL_PAGE * a.hd + (size_t)AG_ROWS * a.hd) * sizeof(float);
    auto kern = attn_generic_kernel<TA, TC, NACC>;
    if (smem > 48 * 1024) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
            cudaGetLastError();
            return GL_ERR_SMEM;
        }
    }
    dim3 grid((a.max_qlen + AG_ROWS - 1) / AG_ROWS, a.nH, a.B);
    kern<<<grid, AG_ROWS * 32, smem, stream>>>(a);
    return gl_check_launch();
}

template <typename TA, typename TC>
static int dispatch_generic(const AttnArgs& a, cudaStream_t stream) {
    switch ((a.hd + 31) / 32) {
        case 1: return launch_generic<TA, TC, 1>(a, stream);
        case 2: return launch_generic<TA, TC, 2>(a, stream);
        case 3: return launch_generic<TA, TC, 3>(a, stream);
        case 4: return launch_generic<TA, TC, 4>(a, stream);
        case 5: return launch_generic<TA, TC, 5>(a, stream);
        case 6: return launch_generic<TA, TC, 6>(a, stream);
        case 7: return launch_generic<TA, TC, 7>(a, stream);
        case 8: return launch_generic<TA, TC, 8>(a, stream);
        default: return GL_ERR_SHAPE;
    }
}

GL_API int gl_attention_generic(const AttnArgs* args, int act_dtype, int cache_dtype, cudaStream_t stream) {
    const AttnArgs& a = *args;
    if (a.B <= 0 || a.max_qlen <= 0) return GL_OK;
    if (a.hd <= 0 || a.hd > 256 || a.nH <= 0 || a.nKV <= 0 || a.nH % a.nKV) return GL_ERR_SHAPE;
    if (a.B > 65535 || a.nH > 65535) return GL_ERR_SHAPE;
    if (act_dtype == GL_F32 && cache_dtype == GL_F32) return dispatch_generic<float, float>(a, stream);
    if (act_dtype == GL_BF16 && cache_dtype == GL_BF16) return dispatch_generic<__nv_bfloat16, __nv_bfloat16>(a, stream);
    return GL_ERR_DTYPE;
}
