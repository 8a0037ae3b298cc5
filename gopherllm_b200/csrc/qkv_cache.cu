// What happens between the QKV product and attention, in one pass over the
// projected rows: optional per-head norm of q and k, rotary position encoding,
// the query scale, and the write of k and v into the paged cache.
//
// Order as in the reference: bias (already in the product's epilogue), head
// norm, rotation, then the query scale (model.go:2677-2706, forward_batch.go:446-469);
// keys are cached rotated and unscaled (model.go:1466-1487).
#include "common.cuh"

// cos/sin of angle float(pos) * inv_freq[i]; the product is taken in 32-bit and
// the functions in 64-bit, as the reference does (model.go:3041-3046).
__global__ void rope_table_kernel(const int* pos, const float* __restrict__ inv_freq,
                                  float* __restrict__ cosv, float* __restrict__ sinv, int T, int half) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    gl_grid_launch_dependents();
    gl_grid_wait();
    if (i >= T * half) return;
    const int t = i / half, p = i % half;
    const float a = (float)pos[t] * inv_freq[p];
    double s, c;
    sincos((double)a, &s, &c);
    cosv[i] = (float)c;
    sinv[i] = (float)s;
}

GL_API int gl_rope_table(const int* pos, const float* inv_freq, float* cosv, float* sinv,
                         int T, int half, cudaStream_t stream) {
    if (T <= 0 || half <= 0) return GL_OK;
    const int n = T * half;
    return gl_launch(rope_table_kernel, dim3((n + 127) / 128), dim3(128), 0, stream, 1, pos, inv_freq, cosv, sinv, T, half);
}

struct QkvCacheArgs {
    const void* qkv;          // [T, (nH + 2 nKV) * hd], activation type
    void* q_out;              // [T, nH * hd], activation type
    void* k_cache;            // this cache entry's keys   [pages, nKV, GL_PAGE, hd], cache type
    void* v_cache;            // this cache entry's values
    const float* cosv;        // [T, half] or null
    const float* sinv;
    const float* q_gamma;     // [hd] or null: per-head norm of q
    const float* q_beta;      // [hd] or null
    const float* k_gamma;
    const float* k_beta;
    const int* tok_seq;       // [T] sequence of each token
    const int* tok_pos;       // [T] absolute position of each token
    const int* pages;         // [B, max_pages] page ids of each sequence
    int T, nH, nKV, hd, half, max_pages;
    int interleaved, norm_rms, write_kv;
    float eps, q_scale;
    int n_pages;              // pages of the cache entry (read by builds that check indices; 0: unknown)
};

template <typename TA, typename TC>
__global__ void qkv_cache_kernel(QkvCacheArgs a) {
    extern __shared__ float smem[];
    gl_grid_launch_dependents();
    gl_grid_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads = a.nH + 2 * a.nKV;
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
    if (item >= (long long)a.T * heads) return;
    const int t = (int)(item / heads), j = (int)(item % heads);
    const int kind = j < a.nH ? 0 : (j < a.nH + a.nKV ? 1 : 2);   // q, k, v
    if (kind != 0 && !a.write_kv) return;
    const int hd = a.hd;
    float* v = smem + warp * hd;
    const TA* src = (const TA*)a.qkv + (size_t)t * heads * hd + (size_t)j * hd;
    for (int d = lane; d < hd; d += 32) v[d] = gl_load(src + d);
    __syncwarp();

    const float* gamma = kind == 0 ? a.q_gamma : a.k_gamma;
    const float* beta = kind == 0 ? a.q_beta : a.k_beta;
    if (kind != 2 && gamma) {
        float mean = 0.f;
        if (!a.norm_rms) {
            float s = 0.f;
            for (int d = lane; d < hd; d += 32) s += v[d];
            mean = gl_warp_sum(s) / (float)hd;
        }
        float q = 0.f;
        for (int d = lane; d < hd; d += 32) { const float c = v[d] - mean; q += c * c; }
        const float var = gl_warp_sum(q) / (float)hd;
        const float inv = (float)(1.0 / sqrt((double)(var + a.eps)));
        for (int d = lane; d < hd; d += 32) {
            float y = (v[d] - mean) * inv * gamma[d];
            if (beta) y += beta[d];
            v[d] = y;
        }
        __syncwarp();
    }
    if (kind != 2 && a.half > 0 && a.cosv) {
        const float* cs = a.cosv + (size_t)t * a.half;
        const float* sn = a.sinv + (size_t)t * a.half;
        for (int i = lane; i < a.half; i += 32) {
            const int i0 = a.interleaved ? 2 * i : i;
            const int i1 = a.interleaved ? 2 * i + 1 : i + a.half;
            const float c = cs[i], s = sn[i];
            const float u = v[i0], w = v[i1];
            v[i0] = u * c - w * s;
            v[i1] = u * s + w * c;
        }
        __syncwarp();
    }
    if (kind == 0) {
        TA* dst = (TA*)a.q_out + (size_t)t * a.nH * hd + (size_t)j * hd;
        for (int d = lane; d < hd; d += 32) gl_store(dst + d, v[d] * a.q_scale);
    } else {
        const int head = kind == 1 ? j - a.nH : j - a.nH - a.nKV;
        const int pos = a.tok_pos[t];
        const int slot = gl_checked(pos / GL_PAGE, a.max_pages, GL_BAD_POSITION);
        const int page = gl_checked(a.pages[(size_t)a.tok_seq[t] * a.max_pages + slot], a.n_pages > 0 ? a.n_pages : 0x7fffffff, GL_BAD_PAGE);
        TC* base = (TC*)(kind == 1 ? a.k_cache : a.v_cache);
        TC* dst = base + (((size_t)page * a.nKV + head) * GL_PAGE + (pos % GL_PAGE)) * hd;
        for (int d = lane; d < hd; d += 32) gl_store(dst + d, v[d]);
    }
}

// The same for bfloat16 rows and cache without a head norm, one 16-byte chunk (8 dims) of a head at a
// time: the chunk and, inside the rotary part, its partner chunk are loaded with 16-byte loads and the
// result leaves with one 16-byte store.  One block per token, its threads over the token's chunks: what
// depends on the token alone (position, page, angle rows) is looked up once, and a chunk's place costs
// one 32-bit division (a flat index over all tokens cost three 64-bit ones a chunk and made the kernel
// instruction-bound).  Needs the head size and the rotary half to be multiples of 8 and split-half pairing.
__global__ void __launch_bounds__(256)
qkv_cache_bf16_kernel(QkvCacheArgs a) {
    gl_grid_launch_dependents();
    gl_grid_wait();
    const unsigned chunks = a.hd >> 3, heads = a.nH + 2 * a.nKV;
    const unsigned hc = a.half >> 3;                          // chunks in one half of the rotary part
    const int t = blockIdx.x;
    const unsigned n = (a.write_kv ? heads : (unsigned)a.nH) * chunks;
    const __nv_bfloat16* row = (const __nv_bfloat16*)a.qkv + (size_t)t * heads * a.hd;
    const float* cs_row = a.cosv ? a.cosv + (size_t)t * a.half : nullptr;
    const float* sn_row = a.sinv ? a.sinv + (size_t)t * a.half : nullptr;
    const int pos = a.tok_pos[t];
    const int slot = gl_checked(pos / GL_PAGE, a.max_pages, GL_BAD_POSITION);
    const size_t cache_row = a.write_kv
        ? ((size_t)gl_checked(a.pages[(size_t)a.tok_seq[t] * a.max_pages + slot], a.n_pages > 0 ? a.n_pages : 0x7fffffff, GL_BAD_PAGE)
           * a.nKV * GL_PAGE + (pos % GL_PAGE)) * a.hd : 0;
    for (unsigned i = threadIdx.x; i < n; i += blockDim.x) {
        const unsigned j = i / chunks, c = i - j * chunks;
        const int kind = j < (unsigned)a.nH ? 0 : (j < (unsigned)(a.nH + a.nKV) ? 1 : 2);
        const __nv_bfloat16* src = row + (size_t)j * a.hd;
        const uint4 raw = *(const uint4*)(src + c * 8);
        float v[8];
        {
            const __nv_bfloat162* p2 = (const __nv_bfloat162*)&raw;
#pragma unroll
            for (int e = 0; e < 4; ++e) { const float2 f = __bfloat1622float2(p2[e]); v[2 * e] = f.x; v[2 * e + 1] = f.y; }
        }
        if (kind != 2 && cs_row && c < 2 * hc) {
            const bool low = c < hc;                             // this chunk holds u (first half) or w (second half)
            const uint4 praw = *(const uint4*)(src + (low ? c + hc : c - hc) * 8);
            const __nv_bfloat162* q2 = (const __nv_bfloat162*)&praw;
            const float* cs = cs_row + (low ? c : c - hc) * 8;
            const float* sn = sn_row + (low ? c : c - hc) * 8;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __bfloat1622float2(q2[e]);
                const float pw[2] = {f.x, f.y};
#pragma unroll
                for (int k = 0; k < 2; ++k) {
                    const float co = cs[2 * e + k], si = sn[2 * e + k];
                    // u' = u cos - w sin ;  w' = u sin + w cos
                    v[2 * e + k] = low ? v[2 * e + k] * co - pw[k] * si : pw[k] * si + v[2 * e + k] * co;
                }
            }
        }
        const float sc = kind == 0 ? a.q_scale : 1.0f;
        uint4 out;
        {
            __nv_bfloat162 p0 = __floats2bfloat162_rn(v[0] * sc, v[1] * sc), p1 = __floats2bfloat162_rn(v[2] * sc, v[3] * sc);
            __nv_bfloat162 p2 = __floats2bfloat162_rn(v[4] * sc, v[5] * sc), p3 = __floats2bfloat162_rn(v[6] * sc, v[7] * sc);
            out.x = *(unsigned*)&p0; out.y = *(unsigned*)&p1; out.z = *(unsigned*)&p2; out.w = *(unsigned*)&p3;
        }
        if (kind == 0) {
            *(uint4*)((__nv_bfloat16*)a.q_out + ((size_t)t * a.nH + j) * a.hd + c * 8) = out;
        } else {
            const unsigned head = kind == 1 ? j - a.nH : j - a.nH - a.nKV;
            __nv_bfloat16* base = (__nv_bfloat16*)(kind == 1 ? a.k_cache : a.v_cache);
            *(uint4*)(base + cache_row + (size_t)head * GL_PAGE * a.hd + c * 8) = out;
        }
    }
}

GL_API int gl_qkv_cache(const QkvCacheArgs* args, int act_dtype, int cache_dtype, cudaStream_t stream) {
    const QkvCacheArgs& a = *args;
    if (a.T <= 0) return GL_OK;
    if (a.hd <= 0 || a.nH <= 0 || a.nKV <= 0 || 2 * a.half > a.hd) return GL_ERR_SHAPE;
    if (act_dtype == GL_BF16 && cache_dtype == GL_BF16 && !a.q_gamma && !a.k_gamma && !a.interleaved &&
        a.hd % 8 == 0 && a.half % 8 == 0 &&
        !(((uintptr_t)a.qkv | (uintptr_t)a.q_out | (uintptr_t)a.k_cache | (uintptr_t)a.v_cache) & 15)) {
        return gl_launch(qkv_cache_bf16_kernel, dim3((unsigned)a.T), dim3(256), 0, stream, 1, a);
    }
    const int warps = 4;
    const long long items = (long long)a.T * (a.nH + 2 * a.nKV);
    const unsigned blocks = (unsigned)((items + warps - 1) / warps);
    const size_t smem = (size_t)warps * a.hd * sizeof(float);
    const dim3 g(blocks), b(warps * 32);
    if (act_dtype == GL_F32 && cache_dtype == GL_F32) return gl_launch(qkv_cache_kernel<float, float>, g, b, smem, stream, 1, a);
    if (act_dtype == GL_BF16 && cache_dtype == GL_BF16)
        return gl_launch(qkv_cache_kernel<__nv_bfloat16, __nv_bfloat16>, g, b, smem, stream, 1, a);
    if (act_dtype == GL_BF16 && cache_dtype == GL_F32) return gl_launch(qkv_cache_kernel<__nv_bfloat16, float>, g, b, smem, stream, 1, a);
    if (act_dtype == GL_F32 && cache_dtype == GL_BF16) return gl_launch(qkv_cache_kernel<float, __nv_bfloat16>, g, b, smem, stream, 1, a);
    return GL_ERR_DTYPE;
}
