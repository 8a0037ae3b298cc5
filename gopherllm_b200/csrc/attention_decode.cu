// Decode attention: one new token per sequence against its cached keys and
// values, bandwidth-bound, so the work is cut over (sequence, key/value head,
// split of the sequence's pages) to fill the machine, and merged afterwards.
//
// A block streams its pages through shared memory with cp.async (16-byte copies,
// AD_STAGES pages in flight).  Inside a page each of the 4 warps owns 16 of the 64
// keys and runs a softmax of its own over them: scores are one mma.sync.m16n8k16
// chain (keys as the 16-row operand, the up to 8 query heads that share the
// key/value head as the 8 columns), maximum, sum and rescaling are 32-bit, and the
// weighted values are a second chain (values transposed by ldmatrix as the 16-row
// operand) into 32-bit accumulators.  The warps never wait for one another inside
// the loop except at the barrier that hands a page buffer back; their four partial
// softmaxes are merged at the end.  With one split the block writes the result
// itself.  Up to 8 splits form a thread-block cluster and merge through distributed
// shared memory; more splits (or a caller that passes scratch) write (max, sum,
// unnormalised output) to scratch and a second kernel merges them.  The head size is a compile-time constant (GL_HEAD_DIM, a
// multiple of 16).
#include "common.cuh"
#include <cooperative_groups.h>
namespace cg = cooperative_groups;

#ifndef GL_HEAD_DIM
#error "compile with -DGL_HEAD_DIM=<head size>: this file is built once per head size a model uses, and knows none itself"
#endif
static_assert(GL_HEAD_DIM % 16 == 0 && GL_HEAD_DIM >= 16 && GL_HEAD_DIM <= 256, "head size: 16..256 in steps of 16");

#define AD_THREADS 128
#define AD_HD GL_HEAD_DIM
#define AD_KS (AD_HD / 16)                          // 16-wide steps along the head size
#define AD_CHUNKS (AD_HD / 8)                       // 16-byte chunks per row
#define AD_ROW (AD_HD * 2 + 16)                     // padded row in bytes: conflict-free ldmatrix
#define AD_TILE (GL_PAGE * AD_ROW)                  // one page of K (or V) for one head
#ifndef AD_STAGES
#define AD_STAGES 2                                 // pages of K and V in flight per block
#endif
#define AD_MAXG 8                                   // query heads per key/value head (the 8 columns of the MMA)

#define GL_DECODE_ARGS_DEFINED      // (attention_decode_static.h declares the same layout for C hosts)
struct DecodeArgs {
    const __nv_bfloat16* q;      // [B, nH*hd], scaled
    __nv_bfloat16* out;          // [B, nH*hd]
    const __nv_bfloat16* k_cache;// [pages, nKV, GL_PAGE, hd]
    const __nv_bfloat16* v_cache;
    const int* seq_ctx;          // [B] positions cached before this step (the new token sits at seq_ctx[b])
    const int* pages;            // [B, max_pages]
    float* part_o;               // [B, nH, splits, hd] scratch
    float* part_ml;              // [B, nH, splits, 2]  scratch
    int B, nH, nKV, max_pages, window, splits;
};

// Queries, and the new token's key and value, straight from the projection's output: with qkv set the
// kernel rotates and scales the queries itself as it loads them (DecodeArgs.q is not read), and the block
// that owns the sequence's last page rotates the new key, writes it and the new value into the cache
// (write_kv) and into its own copy of the page.  Split-half pairing of the rotary dims, bfloat16, no
// per-head norm: what the separate kernel does for those cases, with the same arithmetic.  A record of
// its own, so that DecodeArgs stays what callers of the other entry points compiled against.
struct DecodeQkv {
    const __nv_bfloat16* qkv;    // [B, (nH + 2 nKV) * hd] or null
    const float* cosv;           // [B, half] or null (no rotation)
    const float* sinv;
    int half;                    // pairs of rotary dims (a multiple of 8)
    int write_kv;
    float q_scale;
};

#include "decode_common.cuh"

__device__ __forceinline__ void ad_cp16(unsigned dst, const void* src, int bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void ad_commit() { asm volatile("cp.async.commit_group;"); }
template <int N>
__device__ __forceinline__ void ad_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }
// rows [0, n_valid) of a page (64 rows of hd bf16, contiguous) to padded rows; the rest is zero,
// so that what an earlier sequence left in the page cannot reach a product
__device__ __forceinline__ void ad_load_page(unsigned dst, const __nv_bfloat16* src, int n_valid) {
    // 64 * hd / 8 chunks over 128 threads: hd / 16 chunks a thread, at fixed (row, column) places
#pragma unroll
    for (int j = 0; j < AD_KS; ++j) {
        const int i = threadIdx.x + j * AD_THREADS;
        const int r = i / AD_CHUNKS, c = i - r * AD_CHUNKS;
        const bool ok = r < n_valid;
        ad_cp16(dst + r * AD_ROW + c * 16, ok ? (const void*)((const unsigned char*)src + (size_t)i * 16) : (const void*)src,
                ok ? 16 : 0);
    }
}

// CLUSTER: the splits of one (sequence, key/value head) are the blocks of a cluster
template <bool CLUSTER>
__global__ void __launch_bounds__(AD_THREADS)
attn_decode_kernel(DecodeArgs a, DecodeQkv x) {
    extern __shared__ __align__(16) unsigned char smem[];
    // stage s: keys at 2 s AD_TILE, values one tile further; then per-warp scratch
    const unsigned sbase = ad_smem(smem);
    __nv_bfloat16* pw = (__nv_bfloat16*)(smem + 2 * AD_STAGES * AD_TILE);      // [4 warps][8 heads][16 keys]
    float* mrg = (float*)(smem + 2 * AD_STAGES * AD_TILE + 4 * 8 * 16 * 2);    // [4][8][2] then [4][hd][G]

    const int split = blockIdx.x, g = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int grp = lane >> 2, t = lane & 3;
    gl_grid_launch_dependents();
    gl_grid_wait();
    const int G = a.nH / a.nKV;                          // query heads of this key/value head (<= 8)
    const int pos = a.seq_ctx[b];                        // the query's position; keys lo..pos
    const int lo = (a.window > 0 && pos - a.window + 1 > 0) ? pos - a.window + 1 : 0;
    const int first_page = lo / GL_PAGE, n_pages = pos / GL_PAGE + 1 - first_page;
    const int per = (n_pages + a.splits - 1) / a.splits;
    const int p_begin = first_page + split * per;
    const int p_end = min(first_page + n_pages, p_begin + per);
    const int* pg = a.pages + (size_t)b * a.max_pages;
    const size_t head_off = (size_t)g * GL_PAGE * AD_HD;
    const size_t page_stride = (size_t)a.nKV * GL_PAGE * AD_HD;

    // the first pages are under way before anything else is fetched
#pragma unroll
    for (int s = 0; s < AD_STAGES - 1; ++s) {
        const int p = p_begin + s;
        if (p < p_end) {
            const int nv = min(GL_PAGE, pos + 1 - p * GL_PAGE);
            ad_load_page(sbase + 2 * s * AD_TILE, a.k_cache + (size_t)pg[p] * page_stride + head_off, nv);
            ad_load_page(sbase + (2 * s + 1) * AD_TILE, a.v_cache + (size_t)pg[p] * page_stride + head_off, nv);
        }
        ad_commit();
    }
    // the queries as the 8-column operand: column = head within the group, rows = head dims
    unsigned qb[AD_KS][2];
    const size_t qkv_row = (size_t)(a.nH + 2 * a.nKV) * AD_HD;
    if (x.qkv) {
        // rotated and scaled here: the group's query heads through this block's corner of shared memory
        __nv_bfloat16* qs = (__nv_bfloat16*)mrg;                       // [G][hd], free until the merge
        const float* cs = x.cosv ? x.cosv + (size_t)b * x.half : nullptr;
        const float* sn = x.sinv ? x.sinv + (size_t)b * x.half : nullptr;
        for (int i = tid; i < G * AD_CHUNKS; i += AD_THREADS) {
            const int hq = i / AD_CHUNKS, c = i - hq * AD_CHUNKS;
            const __nv_bfloat16* head = x.qkv + (size_t)b * qkv_row + ((size_t)g * G + hq) * AD_HD;
            *(uint4*)(qs + hq * AD_HD + c * 8) = ad_rotated_chunk(head, c, x.half, cs, sn, x.q_scale);
        }
        __syncthreads();
        const __nv_bfloat16* qh = qs + grp * AD_HD;
#pragma unroll
        for (int kk = 0; kk < AD_KS; ++kk) {
            qb[kk][0] = grp < G ? *(const unsigned*)(qh + kk * 16 + 2 * t) : 0u;
            qb[kk][1] = grp < G ? *(const unsigned*)(qh + kk * 16 + 8 + 2 * t) : 0u;
        }
        __syncthreads();
    } else {
        const __nv_bfloat16* qh = a.q + ((size_t)b * a.nH + (size_t)g * G + grp) * AD_HD;
#pragma unroll
        for (int kk = 0; kk < AD_KS; ++kk) {
            qb[kk][0] = grp < G ? *(const unsigned*)(qh + kk * 16 + 2 * t) : 0u;
            qb[kk][1] = grp < G ? *(const unsigned*)(qh + kk * 16 + 8 + 2 * t) : 0u;
        }
    }
    float o[AD_KS][4];                                   // [d tile][d g | g+8, head 2t | 2t+1]
#pragma unroll
    for (int i = 0; i < AD_KS; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[i][e] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};      // heads 2t, 2t+1; this warp's keys only
    const float LOG2E = 1.4426950408889634f;

    for (int p = p_begin; p < p_end; ++p) {
        const int st = (p - p_begin) % AD_STAGES;
        ad_wait<AD_STAGES - 2>();
        __syncthreads();                                 // page p has landed; the stage read last time is free
        {
            const int pn = p + AD_STAGES - 1, sn = (pn - p_begin) % AD_STAGES;
            if (pn < p_end) {
                const int nv = min(GL_PAGE, pos + 1 - pn * GL_PAGE);
                ad_load_page(sbase + 2 * sn * AD_TILE, a.k_cache + (size_t)pg[pn] * page_stride + head_off, nv);
                ad_load_page(sbase + (2 * sn + 1) * AD_TILE, a.v_cache + (size_t)pg[pn] * page_stride + head_off, nv);
            }
            ad_commit();
        }
        const unsigned Ks = sbase + 2 * st * AD_TILE, Vs = Ks + AD_TILE;
        if (x.qkv && x.write_kv && p == pos / GL_PAGE) {
            // the new token's key (rotated) and value: into the cache for the steps to come, and over
            // the row of this block's copy of the page that the copy from the cache brought stale
            if (tid < 2 * AD_CHUNKS) {
                const int c = tid % AD_CHUNKS, is_v = tid / AD_CHUNKS, r = pos % GL_PAGE;
                const __nv_bfloat16* head = x.qkv + (size_t)b * qkv_row + ((size_t)a.nH + (size_t)is_v * a.nKV + g) * AD_HD;
                const float* cs = (!is_v && x.cosv) ? x.cosv + (size_t)b * x.half : nullptr;
                const float* sn = (!is_v && x.sinv) ? x.sinv + (size_t)b * x.half : nullptr;
                const uint4 val = ad_rotated_chunk(head, c, is_v ? 0 : x.half, cs, sn, 1.0f);
                *(uint4*)(smem + (2 * st + is_v) * AD_TILE + r * AD_ROW + c * 16) = val;
                __nv_bfloat16* cache = (__nv_bfloat16*)(is_v ? a.v_cache : a.k_cache);
                *(uint4*)(cache + (size_t)pg[p] * page_stride + head_off + (size_t)r * AD_HD + c * 8) = val;
            }
            __syncthreads();
        }
        const int j0 = p * GL_PAGE + warp * 16;          // this warp's first key
        if (j0 > pos) continue;                          // all of this warp's keys lie past the sequence
        // scores: [16 keys] x [8 heads]
        float s4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int kk = 0; kk < AD_KS; ++kk) {
            unsigned af[4];
            const int r = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
            const int c = kk * 2 + (lane >> 4);
            ad_ldm4(Ks + r * AD_ROW + c * 16, af);
            ad_mma(s4, af, qb[kk][0], qb[kk][1]);
        }
        {
            const int k_lo = j0 + grp, k_hi = k_lo + 8;
            if (k_lo > pos || k_lo < lo) { s4[0] = -INFINITY; s4[1] = -INFINITY; }
            if (k_hi > pos || k_hi < lo) { s4[2] = -INFINITY; s4[3] = -INFINITY; }
        }
        float mx[2] = {fmaxf(s4[0], s4[2]), fmaxf(s4[1], s4[3])};
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 4));
            mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 8));
            mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 16));
        }
        float corr[2], mu[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const float m_new = fmaxf(m_run[i], mx[i]);
            mu[i] = (m_new == -INFINITY) ? 0.f : m_new * LOG2E;
            corr[i] = exp2f(m_run[i] * LOG2E - mu[i]);    // m_run = -inf gives 0
            m_run[i] = m_new;
        }
        const float p0 = exp2f(s4[0] * LOG2E - mu[0]), p1 = exp2f(s4[1] * LOG2E - mu[1]);
        const float p2 = exp2f(s4[2] * LOG2E - mu[0]), p3 = exp2f(s4[3] * LOG2E - mu[1]);
        l_run[0] = l_run[0] * corr[0] + p0 + p2;         // summed over the 8 key lanes at the end
        l_run[1] = l_run[1] * corr[1] + p1 + p3;
        // weights to the 8-column operand layout: through this warp's [head][key] corner of shared memory
        __nv_bfloat16* pm = pw + warp * 128;
        __syncwarp();
        pm[(2 * t) * 16 + grp] = __float2bfloat16_rn(p0);
        pm[(2 * t + 1) * 16 + grp] = __float2bfloat16_rn(p1);
        pm[(2 * t) * 16 + grp + 8] = __float2bfloat16_rn(p2);
        pm[(2 * t + 1) * 16 + grp + 8] = __float2bfloat16_rn(p3);
        __syncwarp();
        const unsigned pb0 = *(const unsigned*)(pm + grp * 16 + 2 * t);
        const unsigned pb1 = *(const unsigned*)(pm + grp * 16 + 8 + 2 * t);
#pragma unroll
        for (int dt = 0; dt < AD_KS; ++dt) {
            o[dt][0] *= corr[0]; o[dt][1] *= corr[1]; o[dt][2] *= corr[0]; o[dt][3] *= corr[1];
            unsigned vf[4];
            const int r = warp * 16 + (lane >> 4) * 8 + (lane & 7);
            const int c = dt * 2 + ((lane >> 3) & 1);
            ad_ldm4t(Vs + r * AD_ROW + c * 16, vf);
            ad_mma(o[dt], vf, pb0, pb1);
        }
    }
    ad_wait<0>();
    // the sums over this warp's key lanes
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 4);
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 8);
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 16);
    }
    // merge the four warps: (max, sum) per head, then the outputs rescaled to the common maximum
    float* ml_w = mrg;                                   // [4][8][2]
    float* o_w = mrg + 64;                               // [4][hd][G]
    float* fin_o = o_w + 4 * AD_HD * G;                  // [G][hd] this split's result, for the cluster merge
    float* fin_ml = fin_o + G * AD_HD;                   // [G][2]
    __syncthreads();
    if (grp == 0) {
        ml_w[(warp * 8 + 2 * t) * 2] = m_run[0];     ml_w[(warp * 8 + 2 * t) * 2 + 1] = l_run[0];
        ml_w[(warp * 8 + 2 * t + 1) * 2] = m_run[1]; ml_w[(warp * 8 + 2 * t + 1) * 2 + 1] = l_run[1];
    }
#pragma unroll
    for (int dt = 0; dt < AD_KS; ++dt) {
        float* ow = o_w + ((size_t)warp * AD_HD + dt * 16 + grp) * G + 2 * t;
        if (2 * t < G) { ow[0] = o[dt][0]; ow[8 * G] = o[dt][2]; }             // d and d + 8
        if (2 * t + 1 < G) { ow[1] = o[dt][1]; ow[8 * G + 1] = o[dt][3]; }
    }
    __syncthreads();
    for (int i = tid; i < G * AD_HD; i += AD_THREADS) {
        const int hq = i / AD_HD, d = i - hq * AD_HD;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) m = fmaxf(m, ml_w[(w * 8 + hq) * 2]);
        float ov = 0.f, l = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float mw = ml_w[(w * 8 + hq) * 2];
            if (mw == -INFINITY) continue;
            const float f = exp2f((mw - m) * LOG2E);
            ov = fmaf(f, o_w[((size_t)w * AD_HD + d) * G + hq], ov);
            l = fmaf(f, ml_w[(w * 8 + hq) * 2 + 1], l);
        }
        const int h = g * G + hq;
        if (a.splits == 1) {
            a.out[((size_t)b * a.nH + h) * AD_HD + d] = __float2bfloat16_rn(l > 0.f ? ov / l : 0.f);
        } else if (CLUSTER) {
            fin_o[i] = ov;
            if (d == 0) { fin_ml[2 * hq] = m; fin_ml[2 * hq + 1] = l; }
        } else {
            a.part_o[(((size_t)b * a.nH + h) * a.splits + split) * AD_HD + d] = ov;
            if (d == 0) {
                float* ml = a.part_ml + (((size_t)b * a.nH + h) * a.splits + split) * 2;
                ml[0] = m;
                ml[1] = l;
            }
        }
    }
    if (CLUSTER) {
        // the splits meet in distributed shared memory; block r finishes every S-th output, in rank order
        cg::cluster_group cluster = cg::this_cluster();
        const int S = (int)cluster.num_blocks(), rank = (int)cluster.block_rank();
        cluster.sync();
        for (int i = tid * S + rank; i < G * AD_HD; i += AD_THREADS * S) {
            const int hq = i / AD_HD, d = i - hq * AD_HD;
            float m = -INFINITY;
            for (int s = 0; s < S; ++s) m = fmaxf(m, cluster.map_shared_rank(fin_ml, s)[2 * hq]);
            float ov = 0.f, l = 0.f;
            for (int s = 0; s < S; ++s) {
                const float* pml = cluster.map_shared_rank(fin_ml, s);
                const float ms = pml[2 * hq];
                if (ms == -INFINITY) continue;
                const float f = exp2f((ms - m) * LOG2E);
                ov = fmaf(f, cluster.map_shared_rank(fin_o, s)[i], ov);
                l = fmaf(f, pml[2 * hq + 1], l);
            }
            a.out[((size_t)b * a.nH + g * G + hq) * AD_HD + d] = __float2bfloat16_rn(l > 0.f ? ov / l : 0.f);
        }
        cluster.sync();
    }
}

// out = sum_s exp(m_s - m) o_s / sum_s exp(m_s - m) l_s over the splits, in split order
__global__ void attn_decode_merge_kernel(DecodeArgs a) {
    const int h = blockIdx.x, b = blockIdx.y;
    gl_grid_launch_dependents();
    gl_grid_wait();
    const float* ml = a.part_ml + ((size_t)b * a.nH + h) * a.splits * 2;
    const float* po = a.part_o + ((size_t)b * a.nH + h) * a.splits * AD_HD;
    float m = -INFINITY;
    for (int s = 0; s < a.splits; ++s) m = fmaxf(m, ml[2 * s]);
    for (int d = threadIdx.x; d < AD_HD; d += blockDim.x) {
        float o = 0.f, l = 0.f;
        for (int s = 0; s < a.splits; ++s) {
            const float ms = ml[2 * s];
            if (ms == -INFINITY) continue;
            const float w = exp2f((ms - m) * 1.4426950408889634f);
            o = fmaf(w, po[s * AD_HD + d], o);
            l = fmaf(w, ml[2 * s + 1], l);
        }
        a.out[((size_t)b * a.nH + h) * AD_HD + d] = __float2bfloat16_rn(l > 0.f ? o / l : 0.f);
    }
}

static size_t decode_smem(int G) {
    return 2 * AD_STAGES * (size_t)AD_TILE + 4 * 8 * 16 * 2 + sizeof(float) * (64 + 5 * (size_t)AD_HD * G + 2 * G);
}

static int launch_decode(const DecodeArgs& a, const DecodeQkv& x, cudaStream_t stream) {
    static bool configured = false;
    const size_t smem = decode_smem(a.nH / a.nKV);
    if (!configured) {
        if (cudaFuncSetAttribute(attn_decode_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)decode_smem(AD_MAXG)) != cudaSuccess ||
            cudaFuncSetAttribute(attn_decode_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)decode_smem(AD_MAXG)) != cudaSuccess) {
            cudaGetLastError();
            return GL_ERR_SMEM;
        }
        configured = true;
    }
    const dim3 grid(a.splits, a.nKV, a.B);
    if (a.splits > 1 && a.splits <= 8 && !a.part_o)
        return gl_launch(attn_decode_kernel<true>, grid, dim3(AD_THREADS), smem, stream, a.splits, a, x);
    return gl_launch(attn_decode_kernel<false>, grid, dim3(AD_THREADS), smem, stream, 1, a, x);
}

GL_API int gl_attention_decode_head_dim() { return AD_HD; }

// scratch floats needed for B sequences, nH heads and a number of splits
GL_API long long gl_attention_decode_scratch(int B, int nH, int splits) {
    return splits > 1 ? (long long)B * nH * splits * (AD_HD + 2) : 0;
}

static int decode_checked(const DecodeArgs& a, const DecodeQkv& x, cudaStream_t stream);

GL_API int gl_attention_decode(const DecodeArgs* args, cudaStream_t stream) {
    const DecodeQkv none = {nullptr, nullptr, nullptr, 0, 0, 1.0f};
    return decode_checked(*args, none, stream);
}

// the same with the queries and the new key and value taken from the projection's output
GL_API int gl_attention_decode_qkv(const DecodeArgs* args, const DecodeQkv* extra, cudaStream_t stream) {
    const DecodeQkv& x = *extra;
    if (!x.qkv || x.half < 0 || x.half % 8 || 2 * x.half > AD_HD || (x.half > 0 && (!x.cosv || !x.sinv))) return GL_ERR_SHAPE;
    if (((uintptr_t)x.qkv | (uintptr_t)args->k_cache | (uintptr_t)args->v_cache) & 15) return GL_ERR_ALIGN;
    return decode_checked(*args, x, stream);
}

static int decode_checked(const DecodeArgs& a, const DecodeQkv& x, cudaStream_t stream) {
    if (a.B <= 0) return GL_OK;
    if (a.nH <= 0 || a.nKV <= 0 || a.nH % a.nKV || a.nH / a.nKV > AD_MAXG) return GL_ERR_SHAPE;
    if (a.splits < 1 || a.B > 65535 || a.nKV > 65535) return GL_ERR_SHAPE;
    if (a.splits > 8 && (!a.part_o || !a.part_ml)) return GL_ERR_SHAPE;     // more than a cluster holds: scratch
    if ((a.part_o == nullptr) != (a.part_ml == nullptr)) return GL_ERR_SHAPE;
    const int rc = launch_decode(a, x, stream);
    if (rc != GL_OK) return rc;
    if (a.splits > 1 && a.part_o) {
        return gl_launch(attn_decode_merge_kernel, dim3(a.nH, a.B), dim3(AD_HD >= 128 ? 128 : 64), 0, stream, 1, a);
    }
    return GL_OK;
}

// ---------------------------------------------------------------------------
// The same decode attention for callers that must not allocate device memory.
// See attention_decode_static.h for who that is and what the limits are.
// ---------------------------------------------------------------------------
#include "attention_decode_static.h"

// Scratch for the splits' partial results, resident in every GPU context that
// loads this library until the process exits.
static __device__ __align__(256) float gl_decode_static_scratch[GL_DECODE_STATIC_SCRATCH_FLOATS];

#define GL_DECODE_STATIC_MAX_DEVICES 64
// device address of the array, per device; written once per device with a value that is the same
// whichever thread writes it, so first calls from two threads need no lock
static float* gl_decode_static_ptr[GL_DECODE_STATIC_MAX_DEVICES];

GL_API long long gl_attention_decode_static_capacity() { return GL_DECODE_STATIC_SCRATCH_FLOATS; }

GL_API int gl_attention_decode_static(const DecodeArgs* args, cudaStream_t stream) {
    if (!args) return GL_ERR_SHAPE;
    DecodeArgs a = *args;
    if (a.B <= 0) return GL_OK;
    if (a.splits < 1 || a.nH <= 0) return GL_ERR_SHAPE;
    const long long need = gl_attention_decode_scratch(a.B, a.nH, a.splits);
    if (need > (long long)GL_DECODE_STATIC_SCRATCH_FLOATS) return GL_ERR_SCRATCH;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= GL_DECODE_STATIC_MAX_DEVICES) {
        cudaGetLastError();
        return GL_ERR_DRIVER;
    }
    if (!gl_decode_static_ptr[dev]) {
        // In host code the array's name is only a handle; the address a kernel can use is
        // looked up once per device, with that device current.
        float* p = nullptr;
        if (cudaGetSymbolAddress((void**)&p, gl_decode_static_scratch) != cudaSuccess || !p) {
            cudaGetLastError();
            return GL_ERR_DRIVER;
        }
        gl_decode_static_ptr[dev] = p;
    }
    // Every (sequence, head, split) cell that the merge reads is written by the first kernel of
    // the same call, empty splits included, so nothing has to be cleared between calls.
    a.part_o = gl_decode_static_ptr[dev];
    a.part_ml = gl_decode_static_ptr[dev] + (size_t)a.B * a.nH * a.splits * AD_HD;
    return gl_attention_decode(&a, stream);
}
