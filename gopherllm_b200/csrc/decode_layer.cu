// One decode step of one parallel block (norm -> attention and feed-forward side by side -> sum onto
// the residual stream) as ONE kernel, for a few tokens (one per sequence, at most 64).
//
// With few tokens a layer is a stream of bytes: its four weight matrices, read once, and the cached
// keys and values of the live sequences.  Run as separate kernels (norm, projection, attention,
// feed-forward, last products) every one of them pays its own start and finish, a few microseconds
// against 5 to 30 of streaming, and HBM idles in between.  Here a layer is one persistent kernel: a
// block on every SM (a cooperative launch), each block two halves of six warps that share nothing but
// the launch and a tensor-memory allocation (a kernel that allocates tensor memory gets one block an
// SM, so what would be two blocks is two halves of one).  A half has two warps that do nothing but
// issue TMA loads into its ring of stages (20 to 32 KB each), in the order the half will need them,
// and four warps that consume the stages.  The loads of a phase do not wait for the phase before it
// to end: weights and old cache pages depend on nothing this kernel computes, so the ring keeps
// filling while the block waits at a barrier.
//
// Measured on Phi-2's sizes (148 SMs): 64 tokens over 2,040 cached positions take 267 us a layer, the
// layer's 1.5 GB read once at 5.6 TB/s (attention alone at 6.0); a step's barriers (about 3 us each)
// hide behind the ring's prefetch only in part.  From 17 tokens on this kernel is faster than the
// separate kernels, below that slower (they run four blocks an SM on two streams); the caller chooses.
//
// Phases, separated by barriers over the whole grid (an arrival counter and a generation word in
// global memory; every wait is bounded and a wait that runs out sets the library's failure word):
//   0  the norm of the M rows of the residual stream, one row a block               -> xn   (bf16)
//   1  [q,k,v | up] = xn · [Wqkv | Wup]ᵀ + bias (activation on the up part)          -> qkv, h
//   2  attention of every sequence's new token over its cache: rotation and scale of q, the new
//      token's rotated key and its value written to the cache, softmax in 32-bit    -> o
//   3  x += h · Wdownᵀ + o · Woutᵀ + both biases (one product over the joined K, the down part
//      first: it needs nothing of phase 2, so only the blocks that hold chunks of the out part
//      wait for the barrier behind phase 2)                                          -> x   (f32)
//
// Work is cut so that every block streams the same number of bytes whatever the sizes are: a product
// is a line of (128-row tile, 64-k chunk) units, tile-major, and block c takes units [c*per, (c+1)*per)
// (whole tiles where that keeps nine blocks in ten busy; in phase 3, while there are no more tiles than
// blocks, whole blocks to a tile, each with an equal share of the down part's and of the out part's
// chunks); the two halves of a block split each of its runs of chunks in two.  Attention is a line of
// (sequence, key/value head, page) units cut over the halves in the same way.
//
// The products run on tcgen05: the 128 weight rows of a tile are the M of the instruction, the tokens
// (padded to 16, 32 or 64) its N, the accumulator lies in tensor memory; one thread issues the four
// products of a stage and their completion frees the stage, so the consuming warps do nothing per stage
// and read the accumulators once per tile: both halves', added as they are read.  A tile that spans
// several blocks: each writes its partial sums to scratch and counts itself in; when all have, every
// one of them finishes an equal share of the
// tile's tokens, adding the partials in the order of the blocks, so the result does not depend on
// timing and no block is left to add up a whole tile alone.  A sequence's head that spans several
// blocks is merged by whichever arrives last, again in the blocks' order.  Softmax, norm and the
// residual sum are 32-bit.
#include "common.cuh"
#include "tma.cuh"
#include "tcgen05.cuh"
#include "decode_common.cuh"

#ifndef GL_HEAD_DIM
#error "compile with -DGL_HEAD_DIM=<head size>: this file is built once per head size a model uses, and knows none itself"
#endif
static_assert(GL_HEAD_DIM % 16 == 0 && GL_HEAD_DIM >= 16 && GL_HEAD_DIM <= 128, "head size: 16..128 in steps of 16");

#define DL_HD GL_HEAD_DIM
#define DL_KS (DL_HD / 16)            // 16-wide steps along the head size
#define DL_CHUNKS (DL_HD / 8)         // 16-byte chunks per row of a page
#define DL_ROWB (DL_HD * 2)           // bytes per row of a page in shared memory (as TMA leaves it)
#define DL_THREADS 192                // four consuming warps and two loading warps
#define DL_CONS 128
#define DL_WBYTES 16384               // 128 weight rows x 64 k
#define DL_BK 64
#define DL_ROWS 128
#define DL_PAGE_BYTES (GL_PAGE * DL_ROWB)   // the keys or the values of one page of one head
// Rows of a whole number of 128 bytes (head sizes 64 and 128) would put the eight rows of an ldmatrix on
// the same banks: such pages are brought in as tiles of 64 dims with the 128-byte swizzle (one copy per
// tile), and every access goes through dl_page_off.  Other row lengths spread over the banks by themselves.
#define DL_PAGE_SWIZZLED ((DL_ROWB % 128) == 0)
#define DL_PAGE_TILES (DL_PAGE_SWIZZLED ? DL_HD / 64 : 1)
#define DL_MAXG 8                     // query heads per key/value head
#define DL_MAXB 64                    // sequences (= tokens) per step
#define DL_GEN 32                     // the barrier's generation word, a cache line away from its arrival count
#define DL_SYNC_HEAD 64               // ints of sync before the per-tile counters

// What the host hands over (plain pointers and sizes; ctypes fills it in).
struct DecodeLayerArgs {
    float* x;                          // [M, D] the residual stream, updated in place
    const float* norm_g;               // [D]
    const float* norm_b;               // [D] or null
    const void* w_qkv;                 // [Nqkv, D] bf16, rows q, k, v
    const float* b_qkv;                // [Nqkv] or null
    const void* w_up;                  // [I, D] bf16
    const float* b_up;                 // [I] or null
    const void* w_out;                 // [D, nH*hd] bf16
    const float* b_out;                // [D] or null
    const void* w_down;                // [D, I] bf16
    const float* b_down;               // [D] or null
    void* k_cache;                     // [pages, nKV, 64, hd] bf16
    void* v_cache;
    const int* pages;                  // [M, max_pages]
    const int* seq_ctx;                // [M] positions cached before this step
    const float* cosv;                 // [M, half] or null
    const float* sinv;
    void* xn;                          // [M, D] bf16       (work buffers, the caller's)
    void* qkv;                         // [M, Nqkv] bf16
    void* o;                           // [M, nH*hd] bf16
    void* h;                           // [M, I] bf16
    float* scratch;                    // gl_decode_layer_sizes() floats
    int* sync;                         // gl_decode_layer_sizes() ints, zero when first used, left zero by every call
    int M, D, I, nH, nKV, half, max_pages, n_pages, window, act, rms, write_kv;
    float eps, q_scale;
};

// What the kernel gets.
struct LayerArgs {
    CUtensorMap w_qkv, w_up, w_out, w_down;     // boxes of 128 rows x 64 k, 128-byte swizzle
    CUtensorMap a_xn, a_o, a_h;                 // boxes of BN rows x 64 k
    CUtensorMap k_pages, v_pages;               // [pages*nKV*64, hd], boxes of 64 x hd, no swizzle
    DecodeLayerArgs p;
    float *scratch1, *scratchA, *scratch3;
    int *cnt1, *cntA, *cnt3;                    // blocks that have delivered their part of a tile / of a sequence's head
    int *done1, *done3;                         // blocks that have finished their share of a tile
    unsigned* gridbar;                          // [0..2] arrivals at the kernel's three barriers, [DL_GEN] generation
    int Nqkv, No;
    int tiles_q, tiles_u, kc1, per1, maxseg1;
    int tiles3, kc3a, kc3, per3, maxseg3, s3;    // s3: blocks to a tile in phase 3, 0 for the cut along the line
    int maxsegA, stages;
    int stage_bytes;                            // a weight tile and its activations, or a page of keys and its values; a multiple of 1024
    int half_bytes;                             // shared memory of one half of a block
};

// ---------------------------------------------------------------------------
// small device helpers
// ---------------------------------------------------------------------------
__device__ __forceinline__ unsigned dl_ld_acquire(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// the four consuming warps of one half of a block (the halves have a barrier each: 1 and 2)
__device__ __forceinline__ void dl_cons_sync(int id) { asm volatile("bar.sync %0, 128;" ::"r"(id) : "memory"); }
__device__ __forceinline__ void dl_fence_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

// One block's arrival at barrier k of the kernel (0, 1, 2); the last of n to arrive clears the count
// and opens the next generation.  Each barrier of a kernel has an arrival count of its own: a block with
// no work in a phase may count itself in for the next barrier while a slow block is still on its way to
// this one, and must not be taken for one of this one's arrivals.
__device__ __forceinline__ void dl_grid_arrive(unsigned* bar0, int k, unsigned n) {
    unsigned* bar = bar0 + k;
    __threadfence();
    const unsigned prev = atomicAdd(bar, 1u);
    if (prev == n - 1) {
        *(volatile unsigned*)bar = 0u;                     // ordered before the next line by its release
        asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(bar0 + DL_GEN) : "memory");
    }
}
// Wait until the barrier's generation has reached `target` (bounded: false and the failure word on time-out).
__device__ __forceinline__ bool dl_grid_wait(const unsigned* bar, unsigned target) {
    for (unsigned i = 0; i < GL_SPIN_LIMIT; ++i) {
        if ((int)(dl_ld_acquire(bar + DL_GEN) - target) >= 0) return true;
    }
    atomicExch(&gl_wait_failed, 1);
    return false;
}

// What this thread wrote to global memory, made visible to the other blocks' loads, TMA's included: TMA
// reads through the async proxy, and writes made through the generic proxy reach it only past a proxy
// fence on the writer's side (the reader's side orders its own accesses, not the writer's).
__device__ __forceinline__ void dl_publish() {
    dl_fence_async_all();
    __threadfence();
}

// byte offset of 16-byte chunk cc of row r of a page of keys or values in shared memory
__device__ __forceinline__ int dl_page_off(int r, int cc) {
    if (DL_PAGE_SWIZZLED) return (cc >> 3) * (GL_PAGE * 128) + r * 128 + (((cc & 7) ^ (r & 7)) << 4);
    return r * DL_ROWB + cc * 16;
}

__device__ __forceinline__ float dl_cons_sum(float v, float* red, int tid, int bar_id) {   // sum over the 128 consuming threads
    v = gl_warp_sum(v);
    dl_cons_sync(bar_id);
    if ((tid & 31) == 0) red[tid >> 5] = v;
    dl_cons_sync(bar_id);
    return (red[0] + red[1]) + (red[2] + red[3]);
}

// What the finished sums of one weight row of a tile become: tokens m0 .. m0+NE-1 (those below `mend`) with
// sums v[e].  phase 1: bias, activation on the up part, bfloat16 into qkv or h.  phase 3: both biases and
// the residual, 32-bit, onto x.  Everything the row needs from memory is loaded before the first store, so
// the loads overlap.  The threads of a warp hold neighbouring weight rows: a store of theirs is one line.
// `b` is the row's bias (dl_row_bias), which the caller asks for before the sums are ready.
__device__ __forceinline__ float dl_row_bias(const LayerArgs& a, int phase, int tile, int nl) {
    const DecodeLayerArgs& p = a.p;
    if (phase == 1) {
        const bool up = tile >= a.tiles_q;
        const int n = (up ? tile - a.tiles_q : tile) * DL_ROWS + nl;
        const float* bias = up ? p.b_up : p.b_qkv;
        return (bias && n < (up ? p.I : a.Nqkv)) ? bias[n] : 0.f;
    }
    const int n = tile * DL_ROWS + nl;
    if (n >= p.D) return 0.f;
    return (p.b_out ? p.b_out[n] : 0.f) + (p.b_down ? p.b_down[n] : 0.f);
}

// `xs_pre`: the residual values of phase 3 where the caller asked for them ahead of the sums (else they are
// read here).
template <int NE>
__device__ __forceinline__ void dl_finish_rows(const LayerArgs& a, int phase, int tile, int nl, int m0, int mend,
                                               const float (&v)[NE], float b, const float* xs_pre = nullptr) {
    const DecodeLayerArgs& p = a.p;
    if (phase == 1) {
        const bool up = tile >= a.tiles_q;
        const int n = (up ? tile - a.tiles_q : tile) * DL_ROWS + nl;
        const int N = up ? p.I : a.Nqkv;
        if (n >= N) return;
        __nv_bfloat16* out = (__nv_bfloat16*)(up ? p.h : p.qkv);
        // (the kind of activation is chosen once, outside the loop over the tokens: chosen per element, with
        // the erf form among the choices, it cost a tile of 64 tokens 1.5 us more; the bfloat16-grade forms
        // will do, since the result is rounded to bfloat16 at once)
        auto rows = [&](auto act) {
#pragma unroll
            for (int e = 0; e < NE; ++e)
                if (m0 + e < mend) out[(size_t)(m0 + e) * N + n] = __float2bfloat16_rn(act(v[e] + b));
        };
        const int kind = up ? p.act : GL_ACT_NONE;
        if (kind == GL_ACT_GELU_TANH) rows([](float w) { return gl_activate_bf16_grade(w, GL_ACT_GELU_TANH); });
        else if (kind == GL_ACT_GELU_ERF) rows([](float w) { return gl_activate_bf16_grade(w, GL_ACT_GELU_ERF); });
        else if (kind == GL_ACT_RELU) rows([](float w) { return fmaxf(w, 0.0f); });
        else rows([](float w) { return w; });
    } else {
        const int n = tile * DL_ROWS + nl;
        if (n >= p.D) return;
        float xs[NE];
#pragma unroll
        for (int e = 0; e < NE; ++e)
            xs[e] = xs_pre ? xs_pre[e] : (m0 + e < mend ? __ldcg(p.x + (size_t)(m0 + e) * p.D + n) : 0.f);
#pragma unroll
        for (int e = 0; e < NE; ++e)
            if (m0 + e < mend) p.x[(size_t)(m0 + e) * p.D + n] = xs[e] + (v[e] + b);
    }
}

// ---------------------------------------------------------------------------
// the kernel
// ---------------------------------------------------------------------------
template <int BN>                                         // the tokens, padded: 16, 32 or 64
__global__ void __launch_bounds__(2 * DL_THREADS, 1)
decode_layer_kernel(const __grid_constant__ LayerArgs a) {
    extern __shared__ unsigned char smem_raw[];
    const DecodeLayerArgs& p = a.p;
    constexpr unsigned A_BYTES = BN * 128;
    constexpr unsigned GEMM_TX = DL_WBYTES + A_BYTES;
    constexpr unsigned PAGE_TX = 2 * DL_PAGE_BYTES;       // a page's keys and its values share a stage
    constexpr unsigned TMEM_COLS = BN < 32 ? 32 : BN;
    const int NS = a.stages;
    const unsigned DL_STAGE = (unsigned)a.stage_bytes;
    // A kernel that allocates tensor memory gets one block an SM, so a block is two halves of six warps that
    // share nothing but the launch and the allocation: each has its own ring, barriers, work and number c.
    const int half = threadIdx.x / DL_THREADS;
    unsigned char* smem0 = smem_raw + ((1024u - (gl_smem_u32(smem_raw) & 1023u)) & 1023u);
    unsigned char* smem = smem0 + (size_t)half * a.half_bytes;
    const unsigned base = gl_smem_u32(smem);
    const unsigned full0 = base + NS * DL_STAGE, empty0 = full0 + 8 * NS;
    const unsigned acc_bar = empty0 + 8 * NS;             // the accumulator of a run of chunks is complete
    unsigned* tmem_slot = (unsigned*)(smem0 + NS * DL_STAGE + 16 * NS + 8);      // in the first half's part
    unsigned char* misc = smem + NS * DL_STAGE + 16 * NS + 16;
    int* s_off = (int*)misc;                              // [MAXB + 1] first unit of each sequence in phase 2
    int* s_first = s_off + DL_MAXB + 1;                   // [MAXB] first page each sequence reads
    int* s_n = s_first + DL_MAXB;                         // [MAXB] pages each sequence reads
    int* s_flag = s_n + DL_MAXB;                          // [7] (200 ints so far: what follows stays 16-byte aligned)
    float* red = (float*)(s_flag + 7);                    // [4]
    __nv_bfloat16* pw = (__nv_bfloat16*)(red + 4);        // [4 warps][8 heads][16 keys]
    float* mrg = (float*)(pw + 4 * 8 * 16);               // [64] + [4][hd][G] (+ the queries before that)

    const int tid = threadIdx.x - half * DL_THREADS, lane = tid & 31, warp = tid >> 5;
    const int bar_id = 1 + half;
    auto cons_sync = [&]() { dl_cons_sync(bar_id); };
    const int grp = lane >> 2, t = lane & 3;
    const int c = 2 * blockIdx.x + half, GC = 2 * gridDim.x;
    const int G = p.nH / p.nKV;
    const unsigned gen0 = dl_ld_acquire(a.gridbar + DL_GEN);   // read before this block arrives anywhere

    if (tid == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 4);                 // four warps let go of a page; a product's stage gets four commits
        }
        mbar_init(acc_bar, 1);
        mbar_fence_init();
        int off = 0;
        for (int b = 0; b < p.M; ++b) {
            const int pos = p.seq_ctx[b];
            const int lo = (p.window > 0 && pos - p.window + 1 > 0) ? pos - p.window + 1 : 0;
            s_off[b] = off;
            s_first[b] = lo / GL_PAGE;
            s_n[b] = pos / GL_PAGE + 1 - lo / GL_PAGE;
            off += s_n[b] * p.nKV;
        }
        s_off[p.M] = off;
    }
    __syncwarp();
    if (threadIdx.x < 32) tmem_alloc(gl_smem_u32(tmem_slot), 2 * TMEM_COLS);      // both halves' accumulators
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem = *tmem_slot + half * TMEM_COLS;
    // the sequence whose units hold unit L of the attention's line: the last b with s_off[b] <= L
    auto seq_of = [&](int L) {
        int lo = 0, hi = p.M - 1;
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (s_off[mid] <= L) lo = mid; else hi = mid - 1;
        }
        return lo;
    };
    const int totalA = s_off[p.M];
    const int perA = (totalA + GC - 1) / GC;
    const int a0 = min(totalA, c * perA), a1 = min(totalA, a0 + perA);
    const int total1 = (a.tiles_q + a.tiles_u) * a.kc1, total3 = a.tiles3 * a.kc3;
    // the products are cut over the launched blocks; the two halves of a block share every run of chunks
    const int cb = blockIdx.x;
    const int g10 = min(total1, cb * a.per1), g11 = min(total1, g10 + a.per1);
    const int g30 = min(total3, cb * a.per3), g31 = min(total3, g30 + a.per3);
    // A run: the chunks of one tile that lie with this block, as two ranges [c1, c1+n1) and [c2, c2+n2) of the
    // tile's chunks, taken one after the other; `nseg` blocks hold chunks of the tile and this one is number
    // `ord` among them.  The loading warps and the consuming warps walk the same runs.
    //   phase 1, and phase 3 when it has more tiles than there are blocks: the block's stretch [L0, L1) of the
    //   line of (tile, chunk) units, cut where a tile ends.
    //   phase 3 otherwise: s3 blocks to a tile, each with an equal share of the down product's chunks and an
    //   equal share of the out product's; so what has to wait for attention is spread over all blocks.
    auto for_runs = [&](int phase, auto&& f) {
        if (phase == 3 && a.s3 > 0) {
            if (cb < a.tiles3 * a.s3) {
                const int S = a.s3, tile = cb / S, sh = cb - tile * S;
                const int kd = a.kc3a, ko = a.kc3 - a.kc3a;
                const int d0 = sh * kd / S, d1 = (sh + 1) * kd / S, o0 = sh * ko / S, o1 = (sh + 1) * ko / S;
                f(tile, d0, d1 - d0, kd + o0, o1 - o0, S, sh);
            }
            return;
        }
        const int kc = phase == 1 ? a.kc1 : a.kc3, per = phase == 1 ? a.per1 : a.per3;
        int L = phase == 1 ? g10 : g30;
        const int L1 = phase == 1 ? g11 : g31;
        while (L < L1) {
            const int tile = L / kc, ch0 = L - tile * kc;
            const int ch1 = min(kc, ch0 + (L1 - L));
            const int first = (tile * kc) / per, last = (tile * kc + kc - 1) / per;
            f(tile, ch0, ch1 - ch0, 0, 0, last - first + 1, cb - first);
            L += ch1 - ch0;
        }
    };
    // the part [q0, q1) of a run's n chunks that this half takes: the first half (rounded up) or the rest
    auto my_part = [&](int n, int& q0, int& q1) {
        const int mid = (n + 1) / 2;
        q0 = half ? mid : 0;
        q1 = half ? n : mid;
    };
    bool dead = false;                                    // a wait ran out: go through the motions, wait for nothing

    if (warp >= 4) {
        // =====================================================================================
        // The two loading warps: every load of the layer, in the order the consumers take them.  One
        // thread issues a TMA copy every hundred clocks or so, which would set the pace of a block that
        // loads with one thread; so the loads are shared.  Warp 4 brings the weight tiles and the
        // pages of keys, warp 5 the activations that go with the weight tiles (they exist only once a
        // barrier has been passed, so it is also the one that waits for barriers) and the pages of
        // values, behind the keys in the same stage.  Both walk the same sequence of stages; warp 4
        // announces a stage's byte count, warp 5's share included.
        // =====================================================================================
        const bool second = warp == 5;
        int slot = 0, lap = 0;                            // the ring's cursor: the next stage, laps so far
        auto advance = [&]() { if (++slot == NS) { slot = 0; ++lap; } };
        auto acquire = [&]() {                            // lane 0: the cursor's stage is free again
            if (lap >= 1 && !dead)
                if (!mbar_wait(empty0 + 8 * slot, (lap - 1) & 1)) dead = true;
        };
        // The loads of a product: run by run (the chunks of one tile that lie with this block), this half's
        // share of each.
        bool have_o = false;
        auto gemm_loads = [&](int phase, unsigned gen_target) {
            bool waited = false;
            for_runs(phase, [&](int tile, int c1, int n1, int c2, int n2, int, int) {
                if (second && lane == 0 && !waited) {     // the activations exist once every block has arrived
                    if (!dead && !dl_grid_wait(a.gridbar, gen_target)) dead = true;
                    dl_fence_async_all();
                    waited = true;
                }
                int q0, q1;
                my_part(n1 + n2, q0, q1);
                for (int q = q0; q < q1; ++q) {
                    if (lane == 0) {
                        const int ch = q < n1 ? c1 + q : c2 + (q - n1);
                        const CUtensorMap* map;
                        int xk, wy;
                        if (phase == 1) {
                            const bool up = tile >= a.tiles_q;
                            map = second ? &a.a_xn : (up ? &a.w_up : &a.w_qkv);
                            wy = second ? 0 : (up ? tile - a.tiles_q : tile) * DL_ROWS;
                            xk = ch * DL_BK;
                        } else {
                            const bool down = ch < a.kc3a;
                            map = second ? (down ? &a.a_h : &a.a_o) : (down ? &a.w_down : &a.w_out);
                            wy = second ? 0 : tile * DL_ROWS;
                            xk = (down ? ch : ch - a.kc3a) * DL_BK;
                            if (second && !down && !have_o) {            // attention's output: every block past phase 2
                                if (!dead && !dl_grid_wait(a.gridbar, gen0 + 3)) dead = true;
                                dl_fence_async_all();
                                have_o = true;
                            }
                        }
                        acquire();
                        const unsigned sb = base + slot * DL_STAGE, bar = full0 + 8 * slot;
                        if (!second) {
                            mbar_expect_tx(bar, GEMM_TX); // the activations count too; they may even land first
                            tma_load_2d(sb, map, xk, wy, bar);
                        } else {
                            tma_load_2d(sb + DL_WBYTES, map, xk, 0, bar);
                        }
                    }
                    advance();
                }
            });
        };

        gemm_loads(1, gen0 + 1);
        // pages of keys (warp 4) and values (warp 5): they depend on nothing this kernel computes
        {
            const CUtensorMap* pmap = second ? &a.v_pages : &a.k_pages;
            int L = a0;
            while (L < a1) {
                const int b = seq_of(L);
                const int nb = s_n[b];
                const int g = (L - s_off[b]) / nb, pi = (L - s_off[b]) - g * nb;
                const int cnt = min(nb - pi, a1 - L);
                for (int j0 = 0; j0 < cnt; j0 += 32) {
                    const int mine = j0 + lane;
                    const int pg = mine < cnt ? gl_checked(p.pages[(size_t)b * p.max_pages + gl_checked(s_first[b] + pi + mine, p.max_pages, GL_BAD_POSITION)],
                                                           p.n_pages, GL_BAD_PAGE) : 0;
                    const int n = min(32, cnt - j0);
                    for (int j = 0; j < n; ++j) {
                        const int id = __shfl_sync(0xffffffffu, pg, j);
                        const int row = (id * p.nKV + g) * GL_PAGE;
                        if (lane == 0) {
                            acquire();
                            if (!second) mbar_expect_tx(full0 + 8 * slot, PAGE_TX);
#pragma unroll
                            for (int pt = 0; pt < DL_PAGE_TILES; ++pt)
                                tma_load_2d(base + slot * DL_STAGE + (second ? DL_PAGE_BYTES : 0) + pt * (GL_PAGE * 128), pmap,
                                            pt * 64, row, full0 + 8 * slot);
                        }
                        advance();
                    }
                }
                L += cnt;
            }
        }
        gemm_loads(3, gen0 + 2);        // h exists since the barrier behind phase 1
        return;
    }

    // =========================================================================================
    // the consuming warps
    // =========================================================================================
    int slot = 0, lap = 0;                               // the ring's cursor: the stage consumed next, laps so far
    auto advance = [&]() { if (++slot == NS) { slot = 0; ++lap; } };
    auto advance_by = [&](int n) { slot += n; lap += slot / NS; slot %= NS; };
    auto full_wait = [&](int s_, int lap_) {
        if (!dead && !mbar_wait(full0 + 8 * s_, lap_ & 1)) dead = true;
    };
    auto release = [&](int s_) {                         // this warp is done with the stage
        __syncwarp();
        if (lane == 0) mbar_arrive(empty0 + 8 * s_);
    };

    // ---- phase 0: the norm, a row a block; the row is read once and kept in registers -----------------
    for (int r = c; r < p.M; r += GC) {
        const float* xr = p.x + (size_t)r * p.D;
        constexpr int NV = 8;                             // 4-wide pieces a thread keeps: rows up to 4096 wide
        const int n4 = p.D / 4;                           // (D is a multiple of 8)
        float4 v[NV], g4[NV], b4[NV];
        const bool fits = n4 <= NV * DL_CONS;
        float s = 0.f;
        if (fits) {
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                const int j = tid + i * DL_CONS;
                const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
                v[i] = j < n4 ? *(const float4*)(xr + 4 * j) : zero;
                g4[i] = j < n4 ? *(const float4*)(p.norm_g + 4 * j) : zero;
                b4[i] = (j < n4 && p.norm_b) ? *(const float4*)(p.norm_b + 4 * j) : zero;
            }
#pragma unroll
            for (int i = 0; i < NV; ++i) s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
        } else {
            for (int d = tid; d < p.D; d += DL_CONS) s += xr[d];
        }
        const float mean = p.rms ? 0.f : dl_cons_sum(s, red, tid, bar_id) / (float)p.D;
        float q = 0.f;
        if (fits) {
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                if (tid + i * DL_CONS < n4) {
                    const float a0 = v[i].x - mean, a1 = v[i].y - mean, a2 = v[i].z - mean, a3 = v[i].w - mean;
                    q += (a0 * a0 + a1 * a1) + (a2 * a2 + a3 * a3);
                }
            }
        } else {
            for (int d = tid; d < p.D; d += DL_CONS) { const float w = xr[d] - mean; q += w * w; }
        }
        const float var = dl_cons_sum(q, red, tid, bar_id) / (float)p.D;
        const float inv = (float)(1.0 / sqrt((double)(var + p.eps)));
        __nv_bfloat16* o = (__nv_bfloat16*)p.xn + (size_t)r * p.D;
        if (fits) {
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                const int j = tid + i * DL_CONS;
                if (j < n4) {
                    const float4 gg = g4[i], bb = b4[i];
                    const __nv_bfloat162 lo2 = __floats2bfloat162_rn((v[i].x - mean) * inv * gg.x + bb.x, (v[i].y - mean) * inv * gg.y + bb.y);
                    const __nv_bfloat162 hi2 = __floats2bfloat162_rn((v[i].z - mean) * inv * gg.z + bb.z, (v[i].w - mean) * inv * gg.w + bb.w);
                    uint2 pk;
                    pk.x = *(const unsigned*)&lo2;
                    pk.y = *(const unsigned*)&hi2;
                    *(uint2*)(o + 4 * j) = pk;
                }
            }
        } else {
            for (int d = tid; d < p.D; d += DL_CONS) {
                float w = (xr[d] - mean) * inv * p.norm_g[d];
                if (p.norm_b) w += p.norm_b[d];
                o[d] = __float2bfloat16_rn(w);
            }
        }
    }
    dl_publish();
    cons_sync();
    if (tid == 0) dl_grid_arrive(a.gridbar, 0, GC);

    // ---- a product: this block's runs of (tile, chunk) units --------------------------------------
    // A run is the chunks of one tile that lie with this block; each half of the block takes half of them,
    // with an accumulator of its own.  One thread of a half issues its products: D[128 weight rows, BN
    // tokens] += W[128, 16] · X[BN, 16]ᵀ, four to a stage, and commits them to the stage's barrier (four
    // times: the barrier counts four arrivals, as many as the warps that let go of a page), and at the end
    // of the run to the half's acc_bar.  Then the consuming threads of both halves read both accumulators
    // out of tensor memory and add them: each thread one weight row (a warp may touch one quarter of the
    // lanes only: the one its number within the block gives), each half one half of the tokens.
    unsigned acc_parity = 0;
    const int quarter = (threadIdx.x >> 5) & 3;
    const int nl = quarter * 32 + lane;                   // this thread's weight row within a tile
    const unsigned acc_bar_other = acc_bar + (half ? -a.half_bytes : a.half_bytes);
    const unsigned tmem_pair = *tmem_slot;                // the first half's accumulator; the second's lies TMEM_COLS on
    auto both_sync = [&]() { asm volatile("bar.sync 3, 256;" ::: "memory"); };      // the consuming warps of both halves
    auto gemm_phase = [&](int phase, int maxseg, float* scratch, int* cnt, int* done) {
        constexpr int SZ = BN * DL_ROWS;                  // floats of one partial tile, [token][weight row]
        constexpr int CH = BN / 2;                        // tokens this half finishes
        constexpr uint32_t idesc = umma_idesc_bf16(BN, 0);
        int pend_tile[2], pend_nseg[2], pend_ord[2], npend = 0;      // tiles this block shares with others
        for_runs(phase, [&](int tile, int, int n1, int, int n2, int nseg, int ord) {
            int q0, q1;
            my_part(n1 + n2, q0, q1);
            const int n_my = q1 - q0;
            // (asked for now, while the products run: a layer's biases are cold in a decode step)
            const float row_bias = nseg == 1 ? dl_row_bias(a, phase, tile, nl) : 0.f;
            if (warp == 0) {
                if (lane == 0) {
                    int s_ = slot, l_ = lap;
                    for (int i = 0; i < n_my; ++i) {
                        full_wait(s_, l_);
                        tc_fence_after();
                        if (!dead) {
                            const unsigned sb = base + s_ * DL_STAGE;
                            const uint64_t da = umma_tile_desc(sb, 128), db = umma_tile_desc(sb + DL_WBYTES, 128);
#pragma unroll
                            for (int k = 0; k < DL_BK / 16; ++k)     // 32 bytes further along the swizzled row per K 16
                                umma_bf16(tmem, da + 2 * k, db + 2 * k, idesc, i != 0 || k != 0);
                        }
#pragma unroll
                        for (int k = 0; k < 4; ++k) umma_commit(empty0 + 8 * s_);    // free once the products have read it
                        if (++s_ == NS) { s_ = 0; ++l_; }
                    }
                    umma_commit(acc_bar);
                }
                __syncwarp();
            }
            advance_by(n_my);
            if (!dead && !mbar_wait(acc_bar, acc_parity)) dead = true;
            if (!dead && !mbar_wait(acc_bar_other, acc_parity)) dead = true;
            acc_parity ^= 1u;
            tc_fence_after();
            const bool two = n1 + n2 > 1;                 // a run of one chunk leaves the second half's accumulator unused
            {
                unsigned r0[CH], r1[CH];
                const unsigned t0 = tmem_pair + ((unsigned)(quarter * 32) << 16) + half * CH;
                if constexpr (CH == 32) { tmem_ld32(t0, r0); if (two) tmem_ld32(t0 + TMEM_COLS, r1); }
                else if constexpr (CH == 16) { tmem_ld16(t0, r0); if (two) tmem_ld16(t0 + TMEM_COLS, r1); }
                else { tmem_ld8(t0, r0); if (two) tmem_ld8(t0 + TMEM_COLS, r1); }
                float v[CH];
#pragma unroll
                for (int e = 0; e < CH; ++e) v[e] = __uint_as_float(r0[e]) + (two ? __uint_as_float(r1[e]) : 0.f);
                if (nseg == 1) {
                    dl_finish_rows<CH>(a, phase, tile, nl, half * CH, p.M, v, row_bias);
                } else {
                    float* mine = scratch + ((size_t)tile * maxseg + ord) * SZ;
#pragma unroll
                    for (int e = 0; e < CH; ++e) __stcg(mine + (half * CH + e) * DL_ROWS + nl, v[e]);
                    __threadfence();
                }
            }
            tc_fence_before();
            both_sync();                                  // nobody still reads the accumulators the next run overwrites
            if (nseg > 1) {
                if (threadIdx.x == 0) atomicAdd(cnt + tile, 1);
                pend_tile[npend] = tile; pend_nseg[npend] = nseg; pend_ord[npend] = ord;
                ++npend;
            }
        });
        // The shared tiles: once every block of a tile has delivered its part, this block finishes its share of
        // the tile's tokens (each half one half of the share), adding the parts in the blocks' order.  Every
        // block delivers all its parts before it waits for anyone's, and all blocks are resident, so the waits end.
        for (int q = 0; q < npend; ++q) {
            const int tile = pend_tile[q], nseg = pend_nseg[q], ord = pend_ord[q];
            const float row_bias = dl_row_bias(a, phase, tile, nl);      // (under the wait for the other blocks)
            if (threadIdx.x == 0 && !dead) {
                bool ok = false;
                for (unsigned i = 0; i < GL_SPIN_LIMIT && !ok; ++i) ok = (int)dl_ld_acquire((const unsigned*)cnt + tile) >= nseg;
                if (!ok) { atomicExch(&gl_wait_failed, 1); dead = true; }
            }
            both_sync();
            __threadfence();
            const float* part = scratch + (size_t)tile * maxseg * SZ;
            const int s0 = ord * p.M / nseg, s1 = (ord + 1) * p.M / nseg;        // the block's share of the tokens
            const int smid = s0 + (s1 - s0 + 1) / 2;
            const int r0 = half ? smid : s0, r1 = half ? s1 : smid;
            for (int m0 = r0; m0 < r1; m0 += 8) {
                float v[8], xs[8];
                {                                         // the residual values, asked for ahead of the blocks' parts
                    const int n = tile * DL_ROWS + nl;
#pragma unroll
                    for (int e = 0; e < 8; ++e)
                        xs[e] = (phase == 3 && n < p.D && m0 + e < r1) ? __ldcg(p.x + (size_t)(m0 + e) * p.D + n) : 0.f;
                }
#pragma unroll
                for (int e = 0; e < 8; ++e) v[e] = 0.f;
                for (int sg0 = 0; sg0 < nseg; sg0 += 4) {            // four blocks' parts asked for before the first is added
                    float t4[4][8];
#pragma unroll
                    for (int u = 0; u < 4; ++u)
#pragma unroll
                        for (int e = 0; e < 8; ++e)
                            t4[u][e] = (sg0 + u < nseg && m0 + e < r1) ? __ldcg(part + (size_t)(sg0 + u) * SZ + (m0 + e) * DL_ROWS + nl) : 0.f;
#pragma unroll
                    for (int u = 0; u < 4; ++u)
#pragma unroll
                        for (int e = 0; e < 8; ++e) v[e] += t4[u][e];
                }
                dl_finish_rows<8>(a, phase, tile, nl, m0, r1, v, row_bias, xs);
            }
            both_sync();
            if (threadIdx.x == 0 && atomicAdd(done + tile, 1) == nseg - 1) {     // the last to finish leaves both as the next call expects them
                cnt[tile] = 0;
                done[tile] = 0;
            }
        }
    };

    // ---- phase 1 --------------------------------------------------------------------------------
    gemm_phase(1, a.maxseg1, a.scratch1, a.cnt1, a.done1);
    dl_publish();
    cons_sync();
    if (tid == 0) {
        dl_grid_arrive(a.gridbar, 1, GC);
        dl_grid_wait(a.gridbar, gen0 + 2);                           // everyone's q, k, v are written
    }
    cons_sync();

    // ---- phase 2: attention over this block's run of (sequence, head, page) units -----------------
    {
        const float LOG2E = 1.4426950408889634f;
        const size_t qkv_row = (size_t)a.Nqkv;
        const size_t page_stride = (size_t)p.nKV * GL_PAGE * DL_HD;
        const int OSZ = G * DL_HD + 2 * G;                // floats of one partial result
        int L = a0;
        while (L < a1) {
            const int b = seq_of(L);
            const int nb = s_n[b];
            const int g = (L - s_off[b]) / nb, pi0 = (L - s_off[b]) - g * nb;
            const int cnt = min(nb - pi0, a1 - L);
            const int pos = p.seq_ctx[b];
            const int lo = (p.window > 0 && pos - p.window + 1 > 0) ? pos - p.window + 1 : 0;
            const size_t head_off = (size_t)g * GL_PAGE * DL_HD;
            const __nv_bfloat16* qkv_b = (const __nv_bfloat16*)p.qkv + (size_t)b * qkv_row;
            const float* cs = p.cosv ? p.cosv + (size_t)b * p.half : nullptr;
            const float* sn = p.sinv ? p.sinv + (size_t)b * p.half : nullptr;
            // the group's queries, rotated and scaled, as the 8-column operand
            unsigned qb[DL_KS][2];
            {
                cons_sync();                           // the merge of the segment before is over
                __nv_bfloat16* qs = (__nv_bfloat16*)mrg;
                for (int i = tid; i < G * DL_CHUNKS; i += DL_CONS) {
                    const int hq = i / DL_CHUNKS, cc = i - hq * DL_CHUNKS;
                    const __nv_bfloat16* head = qkv_b + ((size_t)g * G + hq) * DL_HD;
                    *(uint4*)(qs + hq * DL_HD + cc * 8) = ad_rotated_chunk(head, cc, p.half, cs, sn, p.q_scale);
                }
                cons_sync();
                const __nv_bfloat16* qh = qs + grp * DL_HD;
#pragma unroll
                for (int kk = 0; kk < DL_KS; ++kk) {
                    qb[kk][0] = grp < G ? *(const unsigned*)(qh + kk * 16 + 2 * t) : 0u;
                    qb[kk][1] = grp < G ? *(const unsigned*)(qh + kk * 16 + 8 + 2 * t) : 0u;
                }
                cons_sync();
            }
            float o[DL_KS][4];
#pragma unroll
            for (int i = 0; i < DL_KS; ++i)
#pragma unroll
                for (int e = 0; e < 4; ++e) o[i][e] = 0.f;
            float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

            for (int pi = pi0; pi < pi0 + cnt; ++pi) {
                const int pabs = s_first[b] + pi;         // the page's number within the sequence
                const int slotP = slot, lapP = lap;       // the page's keys, and its values behind them
                advance();
                full_wait(slotP, lapP);
                const unsigned Ks = base + slotP * DL_STAGE, Vs = Ks + DL_PAGE_BYTES;
                if (pabs == pos / GL_PAGE) {
                    // The sequence's last page.  The new token's key (rotated) and value go into the cache
                    // for the steps to come and over the stale row of this block's copy; rows past the
                    // sequence are cleared in the copy of the values, so that what an earlier sequence
                    // left there cannot reach a product (their weights are zero, but 0 * NaN is not).
                    const int r = pos % GL_PAGE;
                    unsigned char* sK = smem + slotP * DL_STAGE;
                    unsigned char* sV = sK + DL_PAGE_BYTES;
                    if (p.write_kv && tid < 2 * DL_CHUNKS) {
                        const int cc = tid % DL_CHUNKS, is_v = tid / DL_CHUNKS;
                        const __nv_bfloat16* head = qkv_b + ((size_t)p.nH + (size_t)is_v * p.nKV + g) * DL_HD;
                        const uint4 val = ad_rotated_chunk(head, cc, is_v ? 0 : p.half, is_v ? nullptr : cs,
                                                           is_v ? nullptr : sn, 1.0f);
                        *(uint4*)((is_v ? sV : sK) + dl_page_off(r, cc)) = val;
                        const int id = gl_checked(p.pages[(size_t)b * p.max_pages + gl_checked(pabs, p.max_pages, GL_BAD_POSITION)], p.n_pages, GL_BAD_PAGE);
                        __nv_bfloat16* cache = (__nv_bfloat16*)(is_v ? p.v_cache : p.k_cache);
                        *(uint4*)(cache + (size_t)id * page_stride + head_off + (size_t)r * DL_HD + cc * 8) = val;
                    }
                    for (int i = tid; i < (GL_PAGE - 1 - r) * DL_CHUNKS; i += DL_CONS)
                        *(uint4*)(sV + dl_page_off(r + 1 + i / DL_CHUNKS, i % DL_CHUNKS)) = make_uint4(0u, 0u, 0u, 0u);
                    fence_proxy_async();                  // these writes before the stage's next load
                    cons_sync();
                }
                const int j0 = pabs * GL_PAGE + warp * 16;            // this warp's first key
                if (j0 <= pos) {
                    float s4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                    for (int kk = 0; kk < DL_KS; ++kk) {
                        unsigned af[4];
                        const int r = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                        const int cc = kk * 2 + (lane >> 4);
                        ad_ldm4(Ks + dl_page_off(r, cc), af);
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
                        corr[i] = exp2f(m_run[i] * LOG2E - mu[i]);
                        m_run[i] = m_new;
                    }
                    const float p0 = exp2f(s4[0] * LOG2E - mu[0]), p1 = exp2f(s4[1] * LOG2E - mu[1]);
                    const float p2 = exp2f(s4[2] * LOG2E - mu[0]), p3 = exp2f(s4[3] * LOG2E - mu[1]);
                    l_run[0] = l_run[0] * corr[0] + p0 + p2;
                    l_run[1] = l_run[1] * corr[1] + p1 + p3;
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
                    for (int dt = 0; dt < DL_KS; ++dt) {
                        o[dt][0] *= corr[0]; o[dt][1] *= corr[1]; o[dt][2] *= corr[0]; o[dt][3] *= corr[1];
                        unsigned vf[4];
                        const int r = warp * 16 + (lane >> 4) * 8 + (lane & 7);
                        const int cc = dt * 2 + ((lane >> 3) & 1);
                        ad_ldm4t(Vs + dl_page_off(r, cc), vf);
                        ad_mma(o[dt], vf, pb0, pb1);
                    }
                }
                release(slotP);
            }
            // the sums over this warp's key lanes, then the four warps' results at a common maximum
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 4);
                l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 8);
                l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 16);
            }
            float* ml_w = mrg;                            // [4][8][2]
            float* o_w = mrg + 64;                        // [4][hd][G]
            cons_sync();
            if (grp == 0) {
                ml_w[(warp * 8 + 2 * t) * 2] = m_run[0];     ml_w[(warp * 8 + 2 * t) * 2 + 1] = l_run[0];
                ml_w[(warp * 8 + 2 * t + 1) * 2] = m_run[1]; ml_w[(warp * 8 + 2 * t + 1) * 2 + 1] = l_run[1];
            }
#pragma unroll
            for (int dt = 0; dt < DL_KS; ++dt) {
                float* ow = o_w + ((size_t)warp * DL_HD + dt * 16 + grp) * G + 2 * t;
                if (2 * t < G) { ow[0] = o[dt][0]; ow[8 * G] = o[dt][2]; }
                if (2 * t + 1 < G) { ow[1] = o[dt][1]; ow[8 * G + 1] = o[dt][3]; }
            }
            cons_sync();
            // which blocks hold pages of this (sequence, head), and this block's number among them
            const int Ls = s_off[b] + g * nb;
            const int first = Ls / perA, last = (Ls + nb - 1) / perA;
            const int nseg = last - first + 1, ord = c - first;
            float* part = a.scratchA + ((size_t)(b * p.nKV + g) * a.maxsegA) * OSZ;
            __nv_bfloat16* out = (__nv_bfloat16*)p.o;
            for (int i = tid; i < G * DL_HD; i += DL_CONS) {
                const int hq = i / DL_HD, d = i - hq * DL_HD;
                float m = -INFINITY;
#pragma unroll
                for (int w = 0; w < 4; ++w) m = fmaxf(m, ml_w[(w * 8 + hq) * 2]);
                float ov = 0.f, l = 0.f;
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    const float mw = ml_w[(w * 8 + hq) * 2];
                    if (mw == -INFINITY) continue;
                    const float f = exp2f((mw - m) * LOG2E);
                    ov = fmaf(f, o_w[((size_t)w * DL_HD + d) * G + hq], ov);
                    l = fmaf(f, ml_w[(w * 8 + hq) * 2 + 1], l);
                }
                if (nseg == 1) {
                    out[((size_t)b * p.nH + g * G + hq) * DL_HD + d] = __float2bfloat16_rn(l > 0.f ? ov / l : 0.f);
                } else {
                    float* mine = part + (size_t)ord * OSZ;
                    __stcg(mine + i, ov);
                    if (d == 0) { __stcg(mine + G * DL_HD + 2 * hq, m); __stcg(mine + G * DL_HD + 2 * hq + 1, l); }
                }
            }
            if (nseg > 1) {
                __threadfence();
                cons_sync();
                if (tid == 0) s_flag[0] = (atomicAdd(a.cntA + b * p.nKV + g, 1) == nseg - 1) ? 1 : 0;
                cons_sync();
                if (s_flag[0]) {                          // the last to arrive merges the parts, in the blocks' order
                    __threadfence();
                    for (int i = tid; i < G * DL_HD; i += DL_CONS) {
                        const int hq = i / DL_HD, d = i - hq * DL_HD;
                        float m = -INFINITY;
                        for (int s = 0; s < nseg; ++s) m = fmaxf(m, __ldcg(part + (size_t)s * OSZ + G * DL_HD + 2 * hq));
                        float ov = 0.f, l = 0.f;
                        for (int s = 0; s < nseg; ++s) {
                            const float ms = __ldcg(part + (size_t)s * OSZ + G * DL_HD + 2 * hq);
                            if (ms == -INFINITY) continue;
                            const float f = exp2f((ms - m) * LOG2E);
                            ov = fmaf(f, __ldcg(part + (size_t)s * OSZ + i), ov);
                            l = fmaf(f, __ldcg(part + (size_t)s * OSZ + G * DL_HD + 2 * hq + 1), l);
                        }
                        out[((size_t)b * p.nH + g * G + hq) * DL_HD + d] = __float2bfloat16_rn(l > 0.f ? ov / l : 0.f);
                    }
                    if (tid == 0) a.cntA[b * p.nKV + g] = 0;
                }
            }
            L += cnt;
        }
    }
    dl_publish();
    cons_sync();
    if (tid == 0) dl_grid_arrive(a.gridbar, 2, GC);

    // ---- phase 3 (its activations are loaded once every block has arrived above) ------------------
    gemm_phase(3, a.maxseg3, a.scratch3, a.cnt3, a.done3);
    tc_fence_before();
    both_sync();                                          // the consuming warps of both halves are done with tensor memory
    if (threadIdx.x < 32) {
        tc_fence_after();
        tmem_dealloc(tmem, 2 * TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------
// host
// ---------------------------------------------------------------------------
static int dl_plain_map(CUtensorMap* map, const void* base, uint64_t rows, uint32_t cols) {
    gl_encode_tiled_fn enc = gl_get_encode();
    if (!enc) return GL_ERR_DRIVER;
    if (((uintptr_t)base & 15) || (cols * 2) % 16) return GL_ERR_ALIGN;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    cuuint32_t box[2] = {DL_PAGE_SWIZZLED ? 64u : cols, GL_PAGE};       // (swizzled pages: a tile of 64 dims a copy)
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, DL_PAGE_SWIZZLED ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? GL_OK : GL_ERR_DRIVER;
}

static size_t dl_misc_bytes(int G) {
    return sizeof(int) * (3 * DL_MAXB + 1 + 7) + sizeof(float) * 4 + 4 * 8 * 16 * 2 +
           sizeof(float) * (64 + 4 * (size_t)DL_HD * G) + 64;
}

struct DlPlan { int blocks, stages, stage_bytes, half_bytes; size_t smem; };   // blocks: halves, two to a launched block


template <int BN>
static int dl_plan_for(int G, DlPlan* out) {
    static int sms = 0, per_sm[DL_MAXG + 1] = {0};
    static size_t smem_for[DL_MAXG + 1] = {0}, half_for[DL_MAXG + 1] = {0};
    static int stages_for[DL_MAXG + 1] = {0};
    if (!sms) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (sms <= 0) sms = 148;
    }
    // a stage holds a weight tile with its activations or a page of keys with its values, whichever is larger
    const size_t gemm_bytes = DL_WBYTES + (size_t)BN * 128, page_bytes = 2 * (size_t)DL_PAGE_BYTES;
    const size_t stage = ((gemm_bytes > page_bytes ? gemm_bytes : page_bytes) + 1023) / 1024 * 1024;
    if (!per_sm[G]) {
        // two halves a block, a block an SM: as many stages as half an SM's shared memory holds beside the rest
        const size_t budget = 113 * 1024, misc = (dl_misc_bytes(G) + 16 + 1023) / 1024 * 1024;
        int stages = (int)((budget - misc) / (stage + 16));
        if (stages > 16) stages = 16;
        if (stages < 3) return GL_ERR_SMEM;
        const size_t half_bytes = ((size_t)stages * (stage + 16) + misc + 1023) / 1024 * 1024;
        const size_t smem = 2 * half_bytes + 1024;
        if (cudaFuncSetAttribute(decode_layer_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
            cudaGetLastError();
            return GL_ERR_SMEM;
        }
        int n = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, decode_layer_kernel<BN>, 2 * DL_THREADS, smem) != cudaSuccess || n < 1) {
            cudaGetLastError();
            return GL_ERR_SMEM;
        }
        per_sm[G] = 2;
        smem_for[G] = smem;
        half_for[G] = half_bytes;
        stages_for[G] = stages;
    }
    out->blocks = sms * per_sm[G];
    out->stages = stages_for[G];
    out->stage_bytes = (int)stage;
    out->smem = smem_for[G];
    out->half_bytes = (int)half_for[G];
    return GL_OK;
}

static int dl_plan(int M, int G, DlPlan* out) {
    if (M <= 16) return dl_plan_for<16>(G, out);
    if (M <= 32) return dl_plan_for<32>(G, out);
    return dl_plan_for<64>(G, out);
}

static int dl_check(const DecodeLayerArgs& p) {
    if (p.M <= 0 || p.M > DL_MAXB || p.D <= 0 || p.I <= 0 || p.nH <= 0 || p.nKV <= 0) return GL_ERR_SHAPE;
    if (p.nH % p.nKV || p.nH / p.nKV > DL_MAXG) return GL_ERR_SHAPE;
    if (p.D % 8 || p.I % 8 || (p.nH * DL_HD) % 8) return GL_ERR_SHAPE;            // 16-byte row pitches for TMA
    if (p.half < 0 || p.half % 8 || 2 * p.half > DL_HD || (p.half > 0 && (!p.cosv || !p.sinv))) return GL_ERR_SHAPE;
    if (p.max_pages <= 0 || p.n_pages <= 0) return GL_ERR_SHAPE;
    return GL_OK;
}

struct DlCut { int tiles_q, tiles_u, kc1, per1, maxseg1, tiles3, kc3a, kc3, per3, maxseg3, s3, maxsegA; };

// blocks: launched blocks, which share the products; halves: two to a block, which share the attention
static void dl_cut(const DecodeLayerArgs& p, int blocks, int halves, DlCut* k) {
    const int Nqkv = (p.nH + 2 * p.nKV) * DL_HD, No = p.nH * DL_HD;
    k->tiles_q = (Nqkv + DL_ROWS - 1) / DL_ROWS;
    k->tiles_u = (p.I + DL_ROWS - 1) / DL_ROWS;
    k->kc1 = (p.D + DL_BK - 1) / DL_BK;
    const long long t1 = (long long)(k->tiles_q + k->tiles_u) * k->kc1;
    k->per1 = (int)((t1 + blocks - 1) / blocks);
    {
        // whole tiles to a block, where that keeps seven blocks in ten busy: a tile then ends in the
        // block that began it, without the detour through scratch and the wait for the blocks it shares
        // the tile with, which cost more than idle blocks do (Phi-1.5's 112 tiles on 148 SMs: 64 tokens of
        // 2,048 positions 5.36 ms a step cut along the line, 5.16 with whole tiles)
        const long long tiles = k->tiles_q + k->tiles_u, each = (tiles + blocks - 1) / blocks;
        if (tiles * 10 >= (long long)blocks * each * 7) k->per1 = (int)(each * k->kc1);
    }
    k->maxseg1 = (k->kc1 - 1) / k->per1 + 2;
    k->tiles3 = (p.D + DL_ROWS - 1) / DL_ROWS;
    k->kc3a = (p.I + DL_BK - 1) / DL_BK;                  // the down product's chunks come first in the joined K
    k->kc3 = k->kc3a + (No + DL_BK - 1) / DL_BK;
    const long long t3 = (long long)k->tiles3 * k->kc3;
    k->per3 = (int)((t3 + blocks - 1) / blocks);
    {
        const long long each = (k->tiles3 + blocks - 1) / blocks;
        if ((long long)k->tiles3 * 10 >= (long long)blocks * each * 9) k->per3 = (int)(each * k->kc3);
    }
    k->maxseg3 = (k->kc3 - 1) / k->per3 + 2;
    k->s3 = 0;
    if (k->tiles3 <= blocks) {                            // whole blocks to a tile, each with a share of both products
        k->s3 = blocks / k->tiles3;
        if (k->s3 > k->kc3a) k->s3 = k->kc3a;             // (a share is at least one chunk of the down product)
        if (k->s3 < 1) k->s3 = 1;
        k->maxseg3 = k->s3;
    }
    k->maxsegA = (p.max_pages < halves ? p.max_pages : halves) + 1;
}

// floats of scratch and ints of sync a call with these sizes needs
GL_API int gl_decode_layer_sizes(const DecodeLayerArgs* args, long long* scratch_floats, long long* sync_ints) {
    const DecodeLayerArgs& p = *args;
    int rc = dl_check(p);
    if (rc != GL_OK) return rc;
    DlPlan plan;
    rc = dl_plan(p.M, p.nH / p.nKV, &plan);
    if (rc != GL_OK) return rc;
    DlCut k;
    dl_cut(p, plan.blocks / 2, plan.blocks, &k);
    const int G = p.nH / p.nKV;
    const long long mrows = p.M <= 16 ? 16 : p.M <= 32 ? 32 : 64;
    *scratch_floats = (long long)(k.tiles_q + k.tiles_u) * k.maxseg1 * mrows * DL_ROWS +
                      (long long)k.tiles3 * k.maxseg3 * mrows * DL_ROWS +
                      (long long)p.M * p.nKV * k.maxsegA * (G * DL_HD + 2 * G);
    *sync_ints = DL_SYNC_HEAD + 2 * ((long long)(k.tiles_q + k.tiles_u) + k.tiles3) + (long long)DL_MAXB * p.nKV;
    return GL_OK;
}

GL_API int gl_decode_layer_head_dim() { return DL_HD; }

template <int BN>
static int dl_launch(const DecodeLayerArgs& p, const DlPlan& plan, const DlCut& k, cudaStream_t stream) {
    LayerArgs a;
    memset(&a, 0, sizeof(a));
    a.p = p;
    a.Nqkv = (p.nH + 2 * p.nKV) * DL_HD;
    a.No = p.nH * DL_HD;
    int rc;
    if ((rc = gl_cached_map_bf16(&a.w_qkv, p.w_qkv, (uint64_t)a.Nqkv, (uint64_t)p.D, DL_ROWS, DL_BK)) != GL_OK) return rc;
    if ((rc = gl_cached_map_bf16(&a.w_up, p.w_up, (uint64_t)p.I, (uint64_t)p.D, DL_ROWS, DL_BK)) != GL_OK) return rc;
    if ((rc = gl_cached_map_bf16(&a.w_out, p.w_out, (uint64_t)p.D, (uint64_t)a.No, DL_ROWS, DL_BK)) != GL_OK) return rc;
    if ((rc = gl_cached_map_bf16(&a.w_down, p.w_down, (uint64_t)p.D, (uint64_t)p.I, DL_ROWS, DL_BK)) != GL_OK) return rc;
    if ((rc = gl_cached_map_bf16(&a.a_xn, p.xn, (uint64_t)p.M, (uint64_t)p.D, BN, DL_BK)) != GL_OK) return rc;
    if ((rc = gl_cached_map_bf16(&a.a_o, p.o, (uint64_t)p.M, (uint64_t)a.No, BN, DL_BK)) != GL_OK) return rc;
    if ((rc = gl_cached_map_bf16(&a.a_h, p.h, (uint64_t)p.M, (uint64_t)p.I, BN, DL_BK)) != GL_OK) return rc;
    const uint64_t kv_rows = (uint64_t)p.n_pages * p.nKV * GL_PAGE;
    if ((rc = dl_plain_map(&a.k_pages, p.k_cache, kv_rows, DL_HD)) != GL_OK) return rc;
    if ((rc = dl_plain_map(&a.v_pages, p.v_cache, kv_rows, DL_HD)) != GL_OK) return rc;
    a.tiles_q = k.tiles_q; a.tiles_u = k.tiles_u; a.kc1 = k.kc1; a.per1 = k.per1; a.maxseg1 = k.maxseg1;
    a.tiles3 = k.tiles3; a.kc3a = k.kc3a; a.kc3 = k.kc3; a.per3 = k.per3; a.maxseg3 = k.maxseg3; a.s3 = k.s3;
    a.maxsegA = k.maxsegA;
    a.stages = plan.stages;
    a.stage_bytes = plan.stage_bytes;
    a.half_bytes = plan.half_bytes;
    const size_t sz = (size_t)BN * DL_ROWS;
    a.scratch1 = p.scratch;
    a.scratch3 = a.scratch1 + (size_t)(k.tiles_q + k.tiles_u) * k.maxseg1 * sz;
    a.scratchA = a.scratch3 + (size_t)k.tiles3 * k.maxseg3 * sz;
    a.gridbar = (unsigned*)p.sync;
    a.cnt1 = p.sync + DL_SYNC_HEAD;
    a.cnt3 = a.cnt1 + k.tiles_q + k.tiles_u;
    a.done1 = a.cnt3 + k.tiles3;
    a.done3 = a.done1 + k.tiles_q + k.tiles_u;
    a.cntA = a.done3 + k.tiles3;

    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)plan.blocks / 2);
    cfg.blockDim = dim3(2 * DL_THREADS);
    cfg.dynamicSmemBytes = plan.smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;          // every block resident at once: they wait for one another
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, decode_layer_kernel<BN>, a) != cudaSuccess) {
        cudaGetLastError();
        return GL_ERR_LAUNCH;
    }
    return GL_OK;
}

// One layer's decode step.  The calls of a device share `sync` (and usually the work buffers): they
// must follow one another on a stream, never overlap.
GL_API int gl_decode_layer(const DecodeLayerArgs* args, cudaStream_t stream) {
    const DecodeLayerArgs& p = *args;
    int rc = dl_check(p);
    if (rc != GL_OK) return rc;
    const uintptr_t al = (uintptr_t)p.w_qkv | (uintptr_t)p.w_up | (uintptr_t)p.w_out | (uintptr_t)p.w_down |
                         (uintptr_t)p.k_cache | (uintptr_t)p.v_cache | (uintptr_t)p.xn | (uintptr_t)p.qkv |
                         (uintptr_t)p.o | (uintptr_t)p.h;
    if (al & 15) return GL_ERR_ALIGN;
    DlPlan plan;
    rc = dl_plan(p.M, p.nH / p.nKV, &plan);
    if (rc != GL_OK) return rc;
    DlCut k;
    dl_cut(p, plan.blocks / 2, plan.blocks, &k);
    if (p.M <= 16) return dl_launch<16>(p, plan, k, stream);
    if (p.M <= 32) return dl_launch<32>(p, plan, k, stream);
    return dl_launch<64>(p, plan, k, stream);
}
