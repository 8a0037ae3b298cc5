// Prefill attention on the 5th-generation tensor cores: runs of new tokens against the
// paged bfloat16 cache (their own keys included), causal, with an optional window.
//
// A block takes 256 consecutive query rows of one (sequence, head) as two tiles of 128 and
// walks the keys a page (64) at a time.  One warp feeds shared memory by TMA: the query tiles
// once, then key pages and value pages, each in a ring of its own, several pages ahead.  Each
// tile has a thread of its own that issues tcgen05.mma: scores S = Q K^T (M 128, N 64) into
// one of the tile's two score buffers in tensor memory, two pages ahead of the rows, and
// O += P V (M 128, N = head size, the values MN-major straight from the cache layout).  The
// two tiles drift apart freely: while one tile's rows go through the softmax, the tensor
// core works for the other.  Eight warps own one query row
// per thread (four warps a tile): they read a row of scores from tensor memory, mask, keep
// the running maximum and sum in 32-bit, and write the weights as bfloat16 back into tensor
// memory over the scores they came from; the second product reads its 16-row operand from
// there, which spares shared-memory bandwidth and a proxy fence.  The output accumulates in
// tensor memory over all keys; it is rescaled there only when a row's maximum has grown by
// more than 2^8 since the last rescaling.  Since a row lives in one thread, maxima and sums
// need no shuffles.
//
// One thread issues a tcgen05.mma about every 59 clocks at best, whatever its N, so the kernel
// issues few, wide ones: one per 16 dims of the head for the scores, one per 16 keys for the
// output, over the whole head size.
//
// The head size is a compile-time constant (GL_HEAD_DIM, a multiple of 16 up to 128).  For
// queries and keys it is cut into pieces of 64, 32 and 16 dims, each a tile with a swizzle
// of its own row width; values lie in 64-dim tiles of 128-byte rows (what a tile has beyond
// the head size is filled with zeros by TMA and never read).
// Every wait is bounded; a block whose wait runs out records it, leaves its loops, frees its
// tensor memory and returns.
#include "common.cuh"
#include "tma.cuh"
#include "tcgen05.cuh"

#ifndef GL_HEAD_DIM
#error "compile with -DGL_HEAD_DIM=<head size>: this file is built once per head size a model uses, and knows none itself"
#endif
static_assert(GL_HEAD_DIM % 16 == 0 && GL_HEAD_DIM >= 16 && GL_HEAD_DIM <= 128, "head size: 16..128 in steps of 16");
static_assert(GL_PAGE == 64, "a step is one page of 64 keys");

#define AT_HD GL_HEAD_DIM
#define AT_BM 128                 // query rows of a tile
#define AT_THREADS 352
#define AT_TMEM_COLS 512

// pieces of the head size for queries and keys: widths 64, 64, 32, 16 as far as they fit
struct AtSeg { int off, width; };
__host__ __device__ constexpr int at_nseg() { return (AT_HD / 64) + ((AT_HD % 64) >= 32 ? 1 : 0) + ((AT_HD % 32) >= 16 ? 1 : 0); }
__host__ __device__ constexpr AtSeg at_seg(int i) {
    int off = 0, idx = 0;
    for (int k = 0; k < AT_HD / 64; ++k) { if (idx == i) return AtSeg{off, 64}; off += 64; ++idx; }
    if ((AT_HD % 64) >= 32) { if (idx == i) return AtSeg{off, 32}; off += 32; ++idx; }
    if ((AT_HD % 32) >= 16) { if (idx == i) return AtSeg{off, 16}; off += 16; ++idx; }
    return AtSeg{0, 0};
}
// byte offset of piece i inside a tile of `rows` rows (each piece 1024-byte aligned)
__host__ __device__ constexpr int at_seg_base(int i, int rows) {
    int b = 0;
    for (int k = 0; k < i; ++k) b += ((rows * at_seg(k).width * 2 + 1023) / 1024) * 1024;
    return b;
}
#define AT_NSEG at_nseg()
#define AT_Q_BYTES at_seg_base(AT_NSEG, AT_BM)           // a query tile
#define AT_K_BYTES at_seg_base(AT_NSEG, GL_PAGE)         // a page of keys
#define AT_VATOMS ((AT_HD + 63) / 64)
#define AT_VATOM_BYTES (GL_PAGE * 128)                   // 64 keys x 64 dims
#define AT_V_BYTES (AT_VATOMS * AT_VATOM_BYTES)          // a page of values
// Pages in flight in each ring: as many as fit beside the two query tiles.
__host__ __device__ constexpr int at_stages() {
    int n = (227 * 1024 - 2048 - 2 * AT_Q_BYTES) / (AT_K_BYTES + AT_V_BYTES);
    return n > 8 ? 8 : n;
}
#define AT_STAGES at_stages()
static_assert(AT_STAGES >= 4, "shared memory holds too few key/value pages");

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

struct AttnMaps { CUtensorMap q[4], k[4], v; };

__device__ __forceinline__ float at_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__global__ void __launch_bounds__(AT_THREADS, 1)
attn_prefill_tc_kernel(AttnArgs a, const __grid_constant__ AttnMaps maps) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ unsigned tmem_slot;
    __shared__ volatile int failed;
    unsigned char* smem = smem_raw + ((1024u - (gl_smem_u32(smem_raw) & 1023u)) & 1023u);
    const unsigned base = gl_smem_u32(smem);
    const unsigned sQ = base;                                          // [2] query tiles
    const unsigned sK = sQ + 2 * AT_Q_BYTES;                           // [AT_STAGES] key pages
    const unsigned sV = sK + AT_STAGES * AT_K_BYTES;                   // [AT_STAGES] value pages
    const unsigned bars = sV + AT_STAGES * AT_V_BYTES;
    const unsigned bar_q = bars;
    const unsigned bar_kf = bars + 8, bar_ke = bar_kf + 8 * AT_STAGES;
    const unsigned bar_vf = bar_ke + 8 * AT_STAGES, bar_ve = bar_vf + 8 * AT_STAGES;
    const unsigned bar_t = bar_ve + 8 * AT_STAGES;     // per tile: scores full [2], weights full [2], product done, output full
#define BAR_SF(t, i) (bar_t + 64 * (t) + 8 * (i))
#define BAR_PF(t, i) (bar_t + 64 * (t) + 16 + 8 * (i))
#define BAR_PD(t) (bar_t + 64 * (t) + 32)
#define BAR_OF(t) (bar_t + 64 * (t) + 40)

    // Blocks are numbered with the position of their rows in the sequence as the slowest index, from
    // the far end: the blocks with the most keys to walk start first, whatever their sequence and head.
    const int h = blockIdx.x % a.nH, b = (blockIdx.x / a.nH) % a.B;
    const int qlen = a.seq_qlen[b];
    const int qt = (a.max_qlen + 2 * AT_BM - 1) / (2 * AT_BM) - 1 - (int)(blockIdx.x / (a.nH * a.B));
    if (qt * 2 * AT_BM >= qlen) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ctx = a.seq_ctx[b], qstart = a.seq_qstart[b];
    const int q0 = qt * 2 * AT_BM;
    const int rows_all = min(2 * AT_BM, qlen - q0);
    const int g = h / (a.nH / a.nKV);
    const int total = ctx + qlen;
    const int p_first = ctx + q0;
    const int lo_first = (a.window > 0 && p_first - a.window + 1 > 0) ? p_first - a.window + 1 : 0;
    const int page_begin = lo_first / GL_PAGE;
    // pages each tile needs: from the block's first page to the page of the tile's last row
    const int n0 = (p_first + min(AT_BM, rows_all) - 1) / GL_PAGE + 1 - page_begin;
    const int n1 = rows_all > AT_BM ? (p_first + rows_all - 1) / GL_PAGE + 1 - page_begin : 0;
    const int n_max = max(n0, n1);
    const int* pg = a.pages + (size_t)b * a.max_pages;

    if (threadIdx.x == 0) {
        failed = 0;
        mbar_init(bar_q, 1);
        for (int s = 0; s < AT_STAGES; ++s) {
            mbar_init(bar_kf + 8 * s, 1); mbar_init(bar_ke + 8 * s, 2);     // both issuers release a page
            mbar_init(bar_vf + 8 * s, 1); mbar_init(bar_ve + 8 * s, 2);
        }
        for (int t = 0; t < 2; ++t) {
            for (int i = 0; i < 2; ++i) { mbar_init(BAR_SF(t, i), 1); mbar_init(BAR_PF(t, i), 4); }
            mbar_init(BAR_PD(t), 1); mbar_init(BAR_OF(t), 1);
        }
        mbar_fence_init();
    }
    if (warp == 8) tmem_alloc(gl_smem_u32(&tmem_slot), AT_TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem = tmem_slot;
    gl_grid_launch_dependents();                          // launched programmatically: everything read or written
    gl_grid_wait();                                       // comes after the kernel before
    // tile t: score buffers at columns 256 t and 256 t + 64 (the weights of a page overwrite the first
    // 32 columns of its scores, two a column), output at 256 t + 128

    if (warp == 8) {
        // ---- TMA producer ------------------------------------------------------
        if (lane == 0) {
            mbar_expect_tx(bar_q, 2 * AT_BM * AT_HD * 2);
#pragma unroll
            for (int t = 0; t < 2; ++t)
#pragma unroll
                for (int s = 0; s < AT_NSEG; ++s)
                    tma_load_2d(sQ + t * AT_Q_BYTES + at_seg_base(s, AT_BM), &maps.q[s], h * AT_HD + at_seg(s).off,
                                qstart + q0 + t * AT_BM, bar_q);
            for (int j = 0; j < n_max && !failed; ++j) {
                const int st = j % AT_STAGES;
                const unsigned par = ((j / AT_STAGES) - 1) & 1;
                const int row = (pg[page_begin + j] * a.nKV + g) * GL_PAGE;
                if (j >= AT_STAGES && !mbar_wait(bar_ke + 8 * st, par)) { failed = 1; break; }
                mbar_expect_tx(bar_kf + 8 * st, GL_PAGE * AT_HD * 2);
#pragma unroll
                for (int s = 0; s < AT_NSEG; ++s)
                    tma_load_2d(sK + st * AT_K_BYTES + at_seg_base(s, GL_PAGE), &maps.k[s], at_seg(s).off, row, bar_kf + 8 * st);
                if (j >= AT_STAGES && !mbar_wait(bar_ve + 8 * st, par)) { failed = 1; break; }
                mbar_expect_tx(bar_vf + 8 * st, AT_V_BYTES);                       // zero fill counts
#pragma unroll
                for (int c = 0; c < AT_VATOMS; ++c)
                    tma_load_2d(sV + st * AT_V_BYTES + c * AT_VATOM_BYTES, &maps.v, 64 * c, row, bar_vf + 8 * st);
            }
        }
    } else if (warp == 9 || warp == 10) {
        // ---- MMA issuers: one thread a tile ----------------------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc_s = umma_idesc_bf16(GL_PAGE, 0);
            constexpr uint32_t idesc_o = umma_idesc_bf16(AT_HD, 1);
            const int t = warp - 9;
            const int nt = t ? n1 : n0;
            auto issue_scores = [&](int j) {                  // S_j = Q K_j^T into score buffer j & 1
                const int st = j % AT_STAGES;
                bool first = true;
#pragma unroll
                for (int s = 0; s < AT_NSEG; ++s) {
                    const int rb = at_seg(s).width * 2;       // row bytes of this piece
                    const uint64_t dq = umma_tile_desc(sQ + t * AT_Q_BYTES + at_seg_base(s, AT_BM), rb);
                    const uint64_t dk = umma_tile_desc(sK + st * AT_K_BYTES + at_seg_base(s, GL_PAGE), rb);
#pragma unroll
                    for (int k = 0; k < at_seg(s).width / 16; ++k) {
                        umma_bf16(tmem + 256 * t + 64 * (j & 1), dq + 2 * k, dk + 2 * k, idesc_s, first ? 0u : 1u);
                        first = false;
                    }
                }
                umma_commit(BAR_SF(t, j & 1));
                umma_commit(bar_ke + 8 * st);                 // this tile is done with the key page (the other arrives too)
            };
            bool ok = nt == 0 || mbar_wait(bar_q, 0);
            for (int j = 0; ok && j < 2 && j < nt; ++j) {    // scores run two pages ahead of the output product
                ok = mbar_wait(bar_kf + 8 * (j % AT_STAGES), (j / AT_STAGES) & 1);
                if (ok) { tc_fence_after(); issue_scores(j); }
            }
            for (int j = 0; ok && j < nt && !failed; ++j) {
                const int st = j % AT_STAGES;
                ok = mbar_wait(BAR_PF(t, j & 1), (j >> 1) & 1) && mbar_wait(bar_vf + 8 * st, (j / AT_STAGES) & 1);
                if (!ok) break;
                tc_fence_after();
                // O += P_j V_j: 16 keys a step, 8 columns of P (two bf16 each), 16 rows down V's tiles
                const uint64_t dv = umma_smem_desc(sV + st * AT_V_BYTES, AT_VATOM_BYTES, 1024, 2);
#pragma unroll
                for (int k = 0; k < GL_PAGE / 16; ++k)
                    umma_bf16_tmem_a(tmem + 256 * t + 128, tmem + 256 * t + 64 * (j & 1) + 8 * k,
                                     dv + (uint64_t)((16 * 128) >> 4) * k, idesc_o, (j | k) ? 1u : 0u);
                umma_commit(BAR_PD(t));
                if (j == nt - 1) umma_commit(BAR_OF(t));
                umma_commit(bar_ve + 8 * st);                 // this tile is done with the value page
                // S_{j+2} overwrites S_j and P_j: the rows have read the one and written the other, and the
                // product above, issued earlier by this thread, reads its operand first
                if (j + 2 < nt) {
                    ok = mbar_wait(bar_kf + 8 * ((j + 2) % AT_STAGES), ((j + 2) / AT_STAGES) & 1);
                    if (!ok) break;
                    tc_fence_after();
                    issue_scores(j + 2);
                }
            }
            // pages this tile does not need still wait for its word before they go back to the producer;
            // a page counts only once it has been loaded, so that no word lands in an earlier round of its ring slot
            for (int j = nt; ok && j < n_max && !failed; ++j) {
                const int st = j % AT_STAGES;
                ok = mbar_wait(bar_kf + 8 * st, (j / AT_STAGES) & 1);
                if (ok) mbar_arrive(bar_ke + 8 * st);
                ok = ok && mbar_wait(bar_vf + 8 * st, (j / AT_STAGES) & 1);
                if (ok) mbar_arrive(bar_ve + 8 * st);
            }
            if (!ok) failed = 1;
        }
    } else if (warp < 8) {
        // ---- softmax and output: warps 0..7, one query row per thread -------------------
        const int t = warp >> 2, quarter = warp & 3;
        const int r = quarter * 32 + lane;                                  // row inside the tile
        const int rows = min(AT_BM, rows_all - t * AT_BM);                  // valid rows of this tile (may be <= 0)
        const int pos = p_first + t * AT_BM + r;
        const int wlo = (a.window > 0 && pos - a.window + 1 > 0) ? pos - a.window + 1 : 0;
        const unsigned lane_off = (unsigned)(quarter * 32) << 16;
        const unsigned tS = tmem + 256 * t + lane_off, tO = tS + 128;
        const int nt = t ? n1 : n0;
        const float LOG2E = 1.4426950408889634f;
        float m_run = -INFINITY, l_run = 0.f;
        bool alive = true;
        for (int j = 0; j < nt; ++j) {
            const int st = j % AT_STAGES;
            const int j0 = (page_begin + j) * GL_PAGE;
            bool ok = mbar_wait(BAR_SF(t, j & 1), (j >> 1) & 1);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) { failed = 1; alive = false; break; }
            tc_fence_after();
            float sc[GL_PAGE];
            {
                unsigned (&su)[GL_PAGE] = reinterpret_cast<unsigned (&)[GL_PAGE]>(sc);
                tmem_ld32_issue(tS + 64 * (j & 1), *reinterpret_cast<unsigned (*)[32]>(&su[0]));
                tmem_ld32_issue(tS + 64 * (j & 1) + 32, *reinterpret_cast<unsigned (*)[32]>(&su[32]));
                tmem_ld_wait();
            }
            if (j0 + GL_PAGE - 1 > pos || j0 < wlo) {                       // a row at x sees keys max(0, x-window+1)..x
#pragma unroll
                for (int i = 0; i < GL_PAGE; ++i)
                    if (j0 + i > pos || j0 + i < wlo) sc[i] = -INFINITY;
            }
            float mx8[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) mx8[i] = sc[i];
#pragma unroll
            for (int i = 8; i < GL_PAGE; i += 8)
#pragma unroll
                for (int k = 0; k < 8; ++k) mx8[k] = fmaxf(mx8[k], sc[i + k]);
            const float mx = fmaxf(fmaxf(fmaxf(mx8[0], mx8[1]), fmaxf(mx8[2], mx8[3])), fmaxf(fmaxf(mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7])));
            // The exponent's reference is the row's maximum as of the last rescaling: the output in
            // tensor memory is rescaled only when some row of the warp has outgrown it by 2^8, so that
            // weights stay below 256 and most pages cost no pass over the output.
            const float m_new = fmaxf(m_run, mx);
            const bool outgrown = (m_new - m_run) * LOG2E > 8.f;           // -inf to finite: yes; -inf to -inf: no
            const bool rescale = __any_sync(0xffffffffu, outgrown);
            float corr = 1.f;
            if (rescale && m_new != -INFINITY) {
                corr = at_exp2((m_run - m_new) * LOG2E);                    // m_run = -inf gives 0
                m_run = m_new;
            }
            const float mu = (m_run == -INFINITY) ? 0.f : m_run * LOG2E;
            if (rescale && j >= 1) {
                ok = mbar_wait(BAR_PD(t), (j - 1) & 1);                     // the products so far are complete
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) { failed = 1; alive = false; break; }
                tc_fence_after();
#pragma unroll
                for (int c = 0; c < AT_HD; c += 16) {
                    unsigned t16[16];
                    tmem_ld16(tO + c, t16);
#pragma unroll
                    for (int i = 0; i < 16; ++i) t16[i] = __float_as_uint(__uint_as_float(t16[i]) * corr);
                    tmem_st16(tO + c, t16);
                }
            }
            // weights as bfloat16 over the first half of the scores they came from, two a column
            float ps4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int c = 0; c < GL_PAGE; c += 32) {
                unsigned pk[16];
#pragma unroll
                for (int i = 0; i < 32; i += 4) {
                    const float e0 = at_exp2(fmaf(sc[c + i], LOG2E, -mu)), e1 = at_exp2(fmaf(sc[c + i + 1], LOG2E, -mu));
                    const float e2 = at_exp2(fmaf(sc[c + i + 2], LOG2E, -mu)), e3 = at_exp2(fmaf(sc[c + i + 3], LOG2E, -mu));
                    ps4[0] += e0; ps4[1] += e1; ps4[2] += e2; ps4[3] += e3;
                    __nv_bfloat162 p0 = __floats2bfloat162_rn(e0, e1), p1 = __floats2bfloat162_rn(e2, e3);
                    pk[i / 2] = *(unsigned*)&p0; pk[i / 2 + 1] = *(unsigned*)&p1;
                }
                tmem_st16(tS + 64 * (j & 1) + c / 2, pk);
            }
            l_run = l_run * corr + ((ps4[0] + ps4[1]) + (ps4[2] + ps4[3]));
            // rows of the page past the sequence were never written: they must not reach the product
            // (both tiles may clear the same rows; they write the same zeros)
            if (j0 + GL_PAGE > total) {
                ok = mbar_wait(bar_vf + 8 * st, (j / AT_STAGES) & 1);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) { failed = 1; alive = false; break; }
                const int n_valid = total - j0;
#pragma unroll
                for (int c = 0; c < AT_VATOMS; ++c) {
                    unsigned char* vt = smem + (sV - base) + st * AT_V_BYTES + c * AT_VATOM_BYTES;
                    for (int i = n_valid * 8 + r; i < GL_PAGE * 8; i += 128)
                        *(uint4*)(vt + i * 16) = make_uint4(0, 0, 0, 0);
                }
                fence_proxy_async();
            }
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(BAR_PF(t, j & 1));
        }
        if (alive && nt > 0) {
            bool ok = mbar_wait(BAR_OF(t), 0);
            ok = __all_sync(0xffffffffu, ok);
            if (ok) {
                tc_fence_after();
                const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
                __nv_bfloat16* dst = (__nv_bfloat16*)a.out + ((size_t)(qstart + q0 + t * AT_BM + r) * a.nH + h) * AT_HD;
#pragma unroll
                for (int c = 0; c < AT_HD; c += 16) {
                    unsigned t16[16];
                    tmem_ld16(tO + c, t16);
                    if (r < rows) {
                        uint4 pk[2];
                        unsigned* pw = (unsigned*)pk;
#pragma unroll
                        for (int i = 0; i < 16; i += 2) {
                            __nv_bfloat162 v2 = __floats2bfloat162_rn(__uint_as_float(t16[i]) * inv, __uint_as_float(t16[i + 1]) * inv);
                            pw[i / 2] = *(unsigned*)&v2;
                        }
                        *(uint4*)(dst + c) = pk[0];
                        *(uint4*)(dst + c + 8) = pk[1];
                    }
                }
            } else {
                failed = 1;
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 8) {
        tc_fence_after();
        tmem_dealloc(tmem, AT_TMEM_COLS);
    }
    if (threadIdx.x == 0 && failed) atomicExch(&gl_wait_failed, 1);
}

static size_t at_smem() {
    return 2 * (size_t)AT_Q_BYTES + AT_STAGES * ((size_t)AT_K_BYTES + AT_V_BYTES) + 512 + 1024;
}

GL_API int gl_attention_prefill_tc_head_dim() { return AT_HD; }



GL_API int gl_attention_prefill_tc_wait_failed() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, gl_wait_failed, sizeof(int)) != cudaSuccess) return -1;
    return v;
}

// n_tokens: rows of q; n_pages: pages of the cache entry
GL_API int gl_attention_prefill_tc(const AttnArgs* args, int n_tokens, int n_pages, cudaStream_t stream) {
    const AttnArgs& a = *args;
    if (a.B <= 0 || a.max_qlen <= 0) return GL_OK;
    if (a.hd != AT_HD || a.nH <= 0 || a.nKV <= 0 || a.nH % a.nKV) return GL_ERR_SHAPE;
    if (a.score_scale != 1.0f) return GL_ERR_SHAPE;
    if (((uintptr_t)a.q | (uintptr_t)a.out | (uintptr_t)a.k_cache | (uintptr_t)a.v_cache) & 15) return GL_ERR_ALIGN;
    const size_t smem = at_smem();
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
            cudaGetLastError();
            return GL_ERR_SMEM;
        }
        configured = true;
    }
    AttnMaps maps;
    const uint64_t kv_rows = (uint64_t)n_pages * a.nKV * GL_PAGE;
    for (int s = 0; s < AT_NSEG; ++s) {
        const int w = at_seg(s).width;
        int rc = gl_cached_map(&maps.q[s], a.q, (uint64_t)n_tokens, (uint64_t)a.nH * AT_HD, AT_BM, w, 2);
        if (rc != GL_OK) return rc;
        rc = gl_cached_map(&maps.k[s], a.k_cache, kv_rows, AT_HD, GL_PAGE, w, 2);
        if (rc != GL_OK) return rc;
    }
    {   // values: 64 dims a box; what a box has beyond the head size reads as zero
        int rc = gl_cached_map(&maps.v, a.v_cache, kv_rows, AT_HD, GL_PAGE, 64, 2);
        if (rc != GL_OK) return rc;
    }
    const long long blocks = (long long)((a.max_qlen + 2 * AT_BM - 1) / (2 * AT_BM)) * a.nH * a.B;
    if (blocks > 0x7fffffffLL) return GL_ERR_SHAPE;
    if (gl_launch(attn_prefill_tc_kernel, dim3((unsigned)blocks), dim3(AT_THREADS), smem, stream, 1, a, maps) != 0) return GL_ERR_LAUNCH;
    return GL_OK;
}
