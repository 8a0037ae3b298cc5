// One decode step of one parallel block (norm -> attention and feed-forward side by side -> sum onto
// the residual stream) as ONE kernel, for a few tokens (one per sequence, at most 64).
//
// With few tokens a layer is a stream of bytes: its four weight matrices, read once, and the cached
// keys and values of the live sequences.  Run as separate kernels (norm, projection, attention,
// feed-forward, last products) every one of them pays its own start and finish, a few microseconds
// against 5 to 30 of streaming, and HBM idles in between.  Here a layer is one persistent kernel:
// as many blocks as the machine holds at once (a cooperative launch), each with two warps that do
// nothing but issue TMA loads into a ring of stages (10 to 16 KB each), in the order the block will
// need them, and four warps that consume the stages.  The loads of a phase do not wait for the phase
// before it to end: weights and old cache pages depend on nothing this kernel computes, so the ring
// keeps filling while the block waits at a barrier.
//
// Measured on Phi-2's sizes (148 SMs, two blocks each): the phases stream at about 5.2 TB/s whatever
// the ring's depth (3 to 10 stages), the shape of the weight boxes (64 rows of 128 bytes, or 8 KB in
// one piece) and the work of the consuming warps (none at all gives the same time); a step's barriers
// (about 3 us each) hide behind the ring's prefetch only in part, and every (sequence, head) or tile
// that spans two blocks costs its finisher a few microseconds.  At 33 to 64 tokens a step is 3 to 6 %
// faster than the separate kernels; below that the separate kernels, four blocks an SM and two
// streams, are 10 to 20 % faster, so the caller takes this kernel for more than 32 tokens only.
//
// Phases, separated by barriers over the whole grid (an arrival counter and a generation word in
// global memory; every wait is bounded and a wait that runs out sets the library's failure word):
//   0  the norm of the M rows of the residual stream, one row a block               -> xn   (bf16)
//   1  [q,k,v | up] = xn · [Wqkv | Wup]ᵀ + bias (activation on the up part)          -> qkv, h
//   2  attention of every sequence's new token over its cache: rotation and scale of q, the new
//      token's rotated key and its value written to the cache, softmax in 32-bit    -> o
//   3  x += o · Woutᵀ + h · Wdownᵀ + both biases (one product over the joined K)      -> x   (f32)
//
// Work is cut so that every block streams the same number of bytes whatever the sizes are: a product
// is a line of (64-row tile, 64-k chunk) units, tile-major, and block c takes units [c*per, (c+1)*per);
// attention is a line of (sequence, key/value head, page) units cut the same way.  A tile (or a
// sequence's head) that spans several blocks is finished by whichever of them arrives last: each
// writes its partial result to scratch and counts itself in; the last one adds the partials in the
// order of the blocks, so the result does not depend on who that was.  Products run on mma.sync
// m16n8k16 with the weight rows as the 16-row operand (the step is bound by HBM, not by the tensor
// pipe); softmax, norm and the residual sum are 32-bit.
#include "common.cuh"
#include "tma.cuh"
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
#define DL_WBYTES 8192                // 64 weight rows x 64 k
#define DL_BK 64
#define DL_ROWS 64
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
    CUtensorMap w_qkv, w_up, w_out, w_down;     // boxes of 64 rows x 64 k, 128-byte swizzle
    CUtensorMap a_xn, a_o, a_h;                 // boxes of MT*8 rows x 64 k
    CUtensorMap k_pages, v_pages;               // [pages*nKV*64, hd], boxes of 64 x hd, no swizzle
    DecodeLayerArgs p;
    float *scratch1, *scratchA, *scratch3;
    int *cnt1, *cntA, *cnt3;
    unsigned* gridbar;                          // [0..2] arrivals at the kernel's three barriers, [DL_GEN] generation
    int Nqkv, No;
    int tiles_q, tiles_u, kc1, per1, maxseg1;
    int tiles3, kc3a, kc3, per3, maxseg3;
    int maxsegA, stages;
    int stage_bytes;                            // a weight tile and its activations, or one page of keys or values; a multiple of 1024
};

// ---------------------------------------------------------------------------
// small device helpers
// ---------------------------------------------------------------------------
__device__ __forceinline__ unsigned dl_ld_acquire(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void dl_cons_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
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

__device__ __forceinline__ int dl_swz(int r, int c) { return r * 128 + ((c ^ (r & 7)) << 4); }
__device__ __forceinline__ void dl_ldm2(unsigned addr, unsigned& r0, unsigned& r1) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}

__device__ __forceinline__ float dl_cons_sum(float v, float* red) {        // sum over the 128 consuming threads
    v = gl_warp_sum(v);
    dl_cons_sync();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    dl_cons_sync();
    return (red[0] + red[1]) + (red[2] + red[3]);
}

// What the finished elements of one column of a tile become: rows m[e] with sums v[e].  phase 1: bias,
// activation on the up part, bfloat16 into qkv or h.  phase 3: both biases and the residual, 32-bit, onto x.
// Everything a column needs from memory is loaded before the first store, so the loads overlap.
template <int NE>
__device__ __forceinline__ void dl_finish_col(const LayerArgs& a, int phase, int tile, int nl, const int (&m)[NE],
                                              const float (&v)[NE]) {
    const DecodeLayerArgs& p = a.p;
    if (phase == 1) {
        const bool up = tile >= a.tiles_q;
        const int n = (up ? tile - a.tiles_q : tile) * DL_ROWS + nl;
        const int N = up ? p.I : a.Nqkv;
        if (n >= N) return;
        const float* bias = up ? p.b_up : p.b_qkv;
        const float b = bias ? bias[n] : 0.f;
        __nv_bfloat16* out = (__nv_bfloat16*)(up ? p.h : p.qkv);
#pragma unroll
        for (int e = 0; e < NE; ++e) {
            if (m[e] >= p.M) continue;
            float w = v[e] + b;
            if (up) w = gl_activate<false>(w, p.act);
            out[(size_t)m[e] * N + n] = __float2bfloat16_rn(w);
        }
    } else {
        const int n = tile * DL_ROWS + nl;
        if (n >= p.D) return;
        const float b = (p.b_out ? p.b_out[n] : 0.f) + (p.b_down ? p.b_down[n] : 0.f);
        float xs[NE];
#pragma unroll
        for (int e = 0; e < NE; ++e) xs[e] = m[e] < p.M ? __ldcg(p.x + (size_t)m[e] * p.D + n) : 0.f;
#pragma unroll
        for (int e = 0; e < NE; ++e)
            if (m[e] < p.M) p.x[(size_t)m[e] * p.D + n] = xs[e] + (v[e] + b);
    }
}

// ---------------------------------------------------------------------------
// the kernel
// ---------------------------------------------------------------------------
template <int MT>
__global__ void __launch_bounds__(DL_THREADS, 2)
decode_layer_kernel(const __grid_constant__ LayerArgs a) {
    extern __shared__ unsigned char smem_raw[];
    const DecodeLayerArgs& p = a.p;
    constexpr unsigned A_BYTES = MT * 8 * 128;
    constexpr unsigned GEMM_TX = DL_WBYTES + A_BYTES;
    constexpr unsigned PAGE_TX = GL_PAGE * DL_ROWB;
    const int NS = a.stages;
    const unsigned DL_STAGE = (unsigned)a.stage_bytes;
    unsigned char* smem = smem_raw + ((1024u - (gl_smem_u32(smem_raw) & 1023u)) & 1023u);
    const unsigned base = gl_smem_u32(smem);
    const unsigned full0 = base + NS * DL_STAGE, empty0 = full0 + 8 * NS;
    unsigned char* misc = smem + NS * DL_STAGE + 16 * NS;
    int* s_off = (int*)misc;                              // [MAXB + 1] first unit of each sequence in phase 2
    int* s_first = s_off + DL_MAXB + 1;                   // [MAXB] first page each sequence reads
    int* s_n = s_first + DL_MAXB;                         // [MAXB] pages each sequence reads
    int* s_flag = s_n + DL_MAXB;                          // [7] (200 ints so far: what follows stays 16-byte aligned)
    float* red = (float*)(s_flag + 7);                    // [4]
    __nv_bfloat16* pw = (__nv_bfloat16*)(red + 4);        // [4 warps][8 heads][16 keys]
    float* mrg = (float*)(pw + 4 * 8 * 16);               // [64] + [4][hd][G] (+ the queries before that)

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int grp = lane >> 2, t = lane & 3;
    const int c = blockIdx.x, GC = gridDim.x;
    const int G = p.nH / p.nKV;
    const unsigned gen0 = dl_ld_acquire(a.gridbar + DL_GEN);   // read before this block arrives anywhere

    if (tid == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 4);
        }
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
    __syncthreads();
    const int totalA = s_off[p.M];
    const int perA = (totalA + GC - 1) / GC;
    const int a0 = min(totalA, c * perA), a1 = min(totalA, a0 + perA);
    const int total1 = (a.tiles_q + a.tiles_u) * a.kc1, total3 = a.tiles3 * a.kc3;
    const int g10 = min(total1, c * a.per1), g11 = min(total1, g10 + a.per1);
    const int g30 = min(total3, c * a.per3), g31 = min(total3, g30 + a.per3);
    bool dead = false;                                    // a wait ran out: go through the motions, wait for nothing

    if (warp >= 4) {
        // =====================================================================================
        // The two loading warps: every load of the layer, in the order the consumers take them.  One
        // thread issues a TMA copy every hundred clocks or so, which would set the pace of a block that
        // loads with one thread; so the loads are shared.  Warp 4 brings the weight tiles and the
        // pages of keys, warp 5 the activations that go with the weight tiles (they exist only once a
        // barrier has been passed, so it is also the one that waits for barriers) and the pages of
        // values.  Both walk the same sequence of stages; a stage's byte count is announced by warp 4
        // for the products and by each warp for its own pages.
        // =====================================================================================
        const bool second = warp == 5;
        int slot = 0, lap = 0;                            // the ring's cursor: the next stage, laps so far
        auto advance = [&]() { if (++slot == NS) { slot = 0; ++lap; } };
        auto acquire = [&]() {                            // lane 0: the cursor's stage is free again
            if (lap >= 1 && !dead)
                if (!mbar_wait(empty0 + 8 * slot, (lap - 1) & 1)) dead = true;
        };
        // The loads of a product, unit by unit.  What changes from one unit to the next is kept in a few
        // registers (the map, the coordinates) and recomputed only where a tile or the second product begins.
        auto gemm_loads = [&](int phase, int L0, int L1, int kc, unsigned gen_target) {
            if (L1 <= L0) return;
            int tile = L0 / kc, ch = L0 - tile * kc;
            const CUtensorMap* map;
            int xk, wy;
            auto settle = [&]() {                         // map and coordinates of unit (tile, ch)
                if (phase == 1) {
                    const bool up = tile >= a.tiles_q;
                    map = second ? &a.a_xn : (up ? &a.w_up : &a.w_qkv);
                    wy = second ? 0 : (up ? tile - a.tiles_q : tile) * DL_ROWS;
                    xk = ch * DL_BK;
                } else {
                    const bool down = ch >= a.kc3a;
                    map = second ? (down ? &a.a_h : &a.a_o) : (down ? &a.w_down : &a.w_out);
                    wy = second ? 0 : tile * DL_ROWS;
                    xk = (down ? ch - a.kc3a : ch) * DL_BK;
                }
            };
            settle();
            if (second && lane == 0) {                    // the activations exist once every block has arrived
                if (!dead && !dl_grid_wait(a.gridbar, gen_target)) dead = true;
                dl_fence_async_all();
            }
            for (int L = L0; L < L1; ++L) {
                if (lane == 0) {
                    acquire();
                    const unsigned sb = base + slot * DL_STAGE, bar = full0 + 8 * slot;
                    if (!second) {
                        mbar_expect_tx(bar, GEMM_TX);     // the activations count too; they may even land first
                        tma_load_2d(sb, map, xk, wy, bar);
                    } else {
                        tma_load_2d(sb + DL_WBYTES, map, xk, 0, bar);
                    }
                }
                advance();
                ++ch;
                xk += DL_BK;
                if (ch == kc) { ch = 0; ++tile; settle(); }
                else if (phase == 3 && ch == a.kc3a) settle();
            }
        };

        gemm_loads(1, g10, g11, a.kc1, gen0 + 1);
        // pages of keys (warp 4) and values (warp 5): they depend on nothing this kernel computes
        {
            const CUtensorMap* pmap = second ? &a.v_pages : &a.k_pages;
            int L = a0;
            while (L < a1) {
                int b = 0;
                while (b + 1 < p.M && s_off[b + 1] <= L) ++b;
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
                        if (second) advance();            // a page's keys fill one stage, its values the next
                        if (lane == 0) {
                            acquire();
                            mbar_expect_tx(full0 + 8 * slot, PAGE_TX);
                            tma_load_2d(base + slot * DL_STAGE, pmap, 0, row, full0 + 8 * slot);
                        }
                        advance();
                        if (!second) advance();
                    }
                }
                L += cnt;
            }
        }
        gemm_loads(3, g30, g31, a.kc3, gen0 + 3);
        return;
    }

    // =========================================================================================
    // the consuming warps
    // =========================================================================================
    int slot = 0, lap = 0;                               // the ring's cursor: the stage consumed next, laps so far
    auto advance = [&]() { if (++slot == NS) { slot = 0; ++lap; } };
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
        const float mean = p.rms ? 0.f : dl_cons_sum(s, red) / (float)p.D;
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
        const float var = dl_cons_sum(q, red) / (float)p.D;
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
    dl_cons_sync();
    if (tid == 0) dl_grid_arrive(a.gridbar, 0, GC);

    // ---- a product: this block's run of (tile, chunk) units -------------------------------------
    auto gemm_phase = [&](int phase, int L0, int L1, int kc, int per, int maxseg, float* scratch, int* cnt) {
        int L = L0;
        while (L < L1) {
            const int tile = L / kc, ch0 = L - tile * kc;
            const int ch1 = min(kc, ch0 + (L1 - L));
            float acc[MT][4], acc2[MT <= 2 ? MT : 1][4];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[mt][e] = 0.f;
#pragma unroll
            for (int mt = 0; mt < (MT <= 2 ? MT : 1); ++mt)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc2[mt][e] = 0.f;
            for (int ch = ch0; ch < ch1; ++ch) {
                full_wait(slot, lap);
                const unsigned sb = base + slot * DL_STAGE;
                // every fragment of the stage is asked for before the first product needs one, and the
                // products of even and odd k-steps go to accumulators of their own: the warp's chain of
                // dependent instructions per stage is two loads and two products long, not eight and four
                unsigned af[DL_BK / 16][4];
#pragma unroll
                for (int kk = 0; kk < DL_BK / 16; ++kk) {
                    const int r = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                    const int cc = kk * 2 + (lane >> 4);
                    ad_ldm4(sb + dl_swz(r, cc), af[kk]);
                }
                if constexpr (MT <= 2) {
                    unsigned bfr[DL_BK / 16][MT][2];
#pragma unroll
                    for (int kk = 0; kk < DL_BK / 16; ++kk)
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt) {
                            const int r = mt * 8 + (lane & 7);
                            const int cc = kk * 2 + ((lane >> 3) & 1);
                            dl_ldm2(sb + DL_WBYTES + dl_swz(r, cc), bfr[kk][mt][0], bfr[kk][mt][1]);
                        }
#pragma unroll
                    for (int kk = 0; kk < DL_BK / 16; ++kk)
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt)
                            ad_mma((kk & 1) ? acc2[mt] : acc[mt], af[kk], bfr[kk][mt][0], bfr[kk][mt][1]);
                } else {
#pragma unroll
                    for (int kk = 0; kk < DL_BK / 16; ++kk) {
                        unsigned bfr[MT][2];
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt) {
                            const int r = mt * 8 + (lane & 7);
                            const int cc = kk * 2 + ((lane >> 3) & 1);
                            dl_ldm2(sb + DL_WBYTES + dl_swz(r, cc), bfr[mt][0], bfr[mt][1]);
                        }
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt) ad_mma(acc[mt], af[kk], bfr[mt][0], bfr[mt][1]);
                    }
                }
                release(slot);
                advance();
            }
            if constexpr (MT <= 2) {
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) acc[mt][e] += acc2[mt][e];
            }
            // the tile's chunks lie with blocks first..last; this block is number `ord` among them
            const int first = (tile * kc) / per, last = (tile * kc + kc - 1) / per;
            const int nseg = last - first + 1, ord = c - first;
            if (nseg == 1) {
                // straight from the accumulators: this thread holds rows 2t, 2t+1 (+8 mt) of two columns
                int mrow[2 * MT];
                float v0[2 * MT], v1[2 * MT];
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    mrow[2 * mt] = mt * 8 + 2 * t;       mrow[2 * mt + 1] = mt * 8 + 2 * t + 1;
                    v0[2 * mt] = acc[mt][0];              v0[2 * mt + 1] = acc[mt][1];
                    v1[2 * mt] = acc[mt][2];              v1[2 * mt + 1] = acc[mt][3];
                }
                dl_finish_col<2 * MT>(a, phase, tile, warp * 16 + grp, mrow, v0);
                dl_finish_col<2 * MT>(a, phase, tile, warp * 16 + grp + 8, mrow, v1);
            } else {
                constexpr int SZ = MT * 8 * DL_ROWS;
                float* mine = scratch + ((size_t)tile * maxseg + ord) * SZ;
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        __stcg(mine + (mt * 8 + 2 * t + (e & 1)) * DL_ROWS + warp * 16 + grp + (e >> 1) * 8, acc[mt][e]);
                __threadfence();
                dl_cons_sync();
                if (tid == 0) s_flag[0] = (atomicAdd(cnt + tile, 1) == nseg - 1) ? 1 : 0;
                dl_cons_sync();
                if (s_flag[0]) {                          // the last to arrive adds the partial tiles, in the blocks' order
                    __threadfence();
                    const float* part = scratch + (size_t)tile * maxseg * SZ;
                    // this thread: column tid % 64, rows tid / 64 + 2 j
                    int mrow[MT * 4];
                    float v[MT * 4];
#pragma unroll
                    for (int j = 0; j < MT * 4; ++j) { mrow[j] = 2 * j + (tid >> 6); v[j] = 0.f; }
                    for (int sg = 0; sg < nseg; ++sg) {
#pragma unroll
                        for (int j = 0; j < MT * 4; ++j) v[j] += __ldcg(part + (size_t)sg * SZ + tid + j * DL_CONS);
                    }
                    dl_finish_col<MT * 4>(a, phase, tile, tid & 63, mrow, v);
                    if (tid == 0) cnt[tile] = 0;          // as the next call expects to find it
                }
            }
            L += ch1 - ch0;
        }
    };

    // ---- phase 1 --------------------------------------------------------------------------------
    gemm_phase(1, g10, g11, a.kc1, a.per1, a.maxseg1, a.scratch1, a.cnt1);
    dl_publish();
    dl_cons_sync();
    if (tid == 0) {
        dl_grid_arrive(a.gridbar, 1, GC);
        dl_grid_wait(a.gridbar, gen0 + 2);                           // everyone's q, k, v are written
    }
    dl_cons_sync();

    // ---- phase 2: attention over this block's run of (sequence, head, page) units -----------------
    {
        const float LOG2E = 1.4426950408889634f;
        const size_t qkv_row = (size_t)a.Nqkv;
        const size_t page_stride = (size_t)p.nKV * GL_PAGE * DL_HD;
        const int OSZ = G * DL_HD + 2 * G;                // floats of one partial result
        int L = a0;
        while (L < a1) {
            int b = 0;
            while (b + 1 < p.M && s_off[b + 1] <= L) ++b;
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
                dl_cons_sync();                           // the merge of the segment before is over
                __nv_bfloat16* qs = (__nv_bfloat16*)mrg;
                for (int i = tid; i < G * DL_CHUNKS; i += DL_CONS) {
                    const int hq = i / DL_CHUNKS, cc = i - hq * DL_CHUNKS;
                    const __nv_bfloat16* head = qkv_b + ((size_t)g * G + hq) * DL_HD;
                    *(uint4*)(qs + hq * DL_HD + cc * 8) = ad_rotated_chunk(head, cc, p.half, cs, sn, p.q_scale);
                }
                dl_cons_sync();
                const __nv_bfloat16* qh = qs + grp * DL_HD;
#pragma unroll
                for (int kk = 0; kk < DL_KS; ++kk) {
                    qb[kk][0] = grp < G ? *(const unsigned*)(qh + kk * 16 + 2 * t) : 0u;
                    qb[kk][1] = grp < G ? *(const unsigned*)(qh + kk * 16 + 8 + 2 * t) : 0u;
                }
                dl_cons_sync();
            }
            float o[DL_KS][4];
#pragma unroll
            for (int i = 0; i < DL_KS; ++i)
#pragma unroll
                for (int e = 0; e < 4; ++e) o[i][e] = 0.f;
            float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

            for (int pi = pi0; pi < pi0 + cnt; ++pi) {
                const int pabs = s_first[b] + pi;         // the page's number within the sequence
                const int slotK = slot, lapK = lap;
                advance();
                const int slotV = slot, lapV = lap;
                advance();
                full_wait(slotK, lapK);
                full_wait(slotV, lapV);
                const unsigned Ks = base + slotK * DL_STAGE, Vs = base + slotV * DL_STAGE;
                if (pabs == pos / GL_PAGE) {
                    // The sequence's last page.  The new token's key (rotated) and value go into the cache
                    // for the steps to come and over the stale row of this block's copy; rows past the
                    // sequence are cleared in the copy of the values, so that what an earlier sequence
                    // left there cannot reach a product (their weights are zero, but 0 * NaN is not).
                    const int r = pos % GL_PAGE;
                    unsigned char* sK = smem + slotK * DL_STAGE;
                    unsigned char* sV = smem + slotV * DL_STAGE;
                    if (p.write_kv && tid < 2 * DL_CHUNKS) {
                        const int cc = tid % DL_CHUNKS, is_v = tid / DL_CHUNKS;
                        const __nv_bfloat16* head = qkv_b + ((size_t)p.nH + (size_t)is_v * p.nKV + g) * DL_HD;
                        const uint4 val = ad_rotated_chunk(head, cc, is_v ? 0 : p.half, is_v ? nullptr : cs,
                                                           is_v ? nullptr : sn, 1.0f);
                        *(uint4*)((is_v ? sV : sK) + r * DL_ROWB + cc * 16) = val;
                        const int id = gl_checked(p.pages[(size_t)b * p.max_pages + gl_checked(pabs, p.max_pages, GL_BAD_POSITION)], p.n_pages, GL_BAD_PAGE);
                        __nv_bfloat16* cache = (__nv_bfloat16*)(is_v ? p.v_cache : p.k_cache);
                        *(uint4*)(cache + (size_t)id * page_stride + head_off + (size_t)r * DL_HD + cc * 8) = val;
                    }
                    for (int i = tid; i < (GL_PAGE - 1 - r) * DL_CHUNKS; i += DL_CONS)
                        *(uint4*)(sV + (r + 1) * DL_ROWB + i * 16) = make_uint4(0u, 0u, 0u, 0u);
                    fence_proxy_async();                  // these writes before the stage's next load
                    dl_cons_sync();
                }
                const int j0 = pabs * GL_PAGE + warp * 16;            // this warp's first key
                if (j0 <= pos) {
                    float s4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                    for (int kk = 0; kk < DL_KS; ++kk) {
                        unsigned af[4];
                        const int r = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                        const int cc = kk * 2 + (lane >> 4);
                        ad_ldm4(Ks + r * DL_ROWB + cc * 16, af);
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
                        ad_ldm4t(Vs + r * DL_ROWB + cc * 16, vf);
                        ad_mma(o[dt], vf, pb0, pb1);
                    }
                }
                release(slotK);
                release(slotV);
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
            dl_cons_sync();
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
            dl_cons_sync();
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
                dl_cons_sync();
                if (tid == 0) s_flag[0] = (atomicAdd(a.cntA + b * p.nKV + g, 1) == nseg - 1) ? 1 : 0;
                dl_cons_sync();
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
    dl_cons_sync();
    if (tid == 0) dl_grid_arrive(a.gridbar, 2, GC);

    // ---- phase 3 (its activations are loaded once every block has arrived above) ------------------
    gemm_phase(3, g30, g31, a.kc3, a.per3, a.maxseg3, a.scratch3, a.cnt3);
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
    cuuint32_t box[2] = {cols, GL_PAGE};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? GL_OK : GL_ERR_DRIVER;
}

static size_t dl_misc_bytes(int G) {
    return sizeof(int) * (3 * DL_MAXB + 1 + 7) + sizeof(float) * 4 + 4 * 8 * 16 * 2 +
           sizeof(float) * (64 + 4 * (size_t)DL_HD * G) + 64;
}

struct DlPlan { int blocks, stages, stage_bytes; size_t smem; };


template <int MT>
static int dl_plan_for(int G, DlPlan* out) {
    static int sms = 0, per_sm[DL_MAXG + 1] = {0};
    static size_t smem_for[DL_MAXG + 1] = {0};
    static int stages_for[DL_MAXG + 1] = {0};
    if (!sms) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (sms <= 0) sms = 148;
    }
    // a stage holds a weight tile with its activations or a page of keys or values, whichever is larger
    const size_t gemm_bytes = DL_WBYTES + (size_t)MT * 8 * 128, page_bytes = (size_t)GL_PAGE * DL_ROWB;
    const size_t stage = ((gemm_bytes > page_bytes ? gemm_bytes : page_bytes) + 1023) / 1024 * 1024;
    if (!per_sm[G]) {
        // two blocks an SM: as many stages as half an SM's shared memory holds beside the rest
        const size_t budget = 113 * 1024, misc = dl_misc_bytes(G) + 1024;
        int stages = (int)((budget - misc) / (stage + 16));
        if (stages > 16) stages = 16;
        if (stages < 3) return GL_ERR_SMEM;
        const size_t smem = (size_t)stages * (stage + 16) + misc;
        if (cudaFuncSetAttribute(decode_layer_kernel<MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
            cudaGetLastError();
            return GL_ERR_SMEM;
        }
        int n = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, decode_layer_kernel<MT>, DL_THREADS, smem) != cudaSuccess || n < 1) {
            cudaGetLastError();
            return GL_ERR_SMEM;
        }
        per_sm[G] = n > 2 ? 2 : n;
        smem_for[G] = smem;
        stages_for[G] = stages;
    }
    out->blocks = sms * per_sm[G];
    out->stages = stages_for[G];
    out->stage_bytes = (int)stage;
    out->smem = smem_for[G];
    return GL_OK;
}

static int dl_plan(int M, int G, DlPlan* out) {
    if (M <= 8) return dl_plan_for<1>(G, out);
    if (M <= 16) return dl_plan_for<2>(G, out);
    if (M <= 32) return dl_plan_for<4>(G, out);
    return dl_plan_for<8>(G, out);
}

static int dl_check(const DecodeLayerArgs& p) {
    if (p.M <= 0 || p.M > DL_MAXB || p.D <= 0 || p.I <= 0 || p.nH <= 0 || p.nKV <= 0) return GL_ERR_SHAPE;
    if (p.nH % p.nKV || p.nH / p.nKV > DL_MAXG) return GL_ERR_SHAPE;
    if (p.D % 8 || p.I % 8 || (p.nH * DL_HD) % 8) return GL_ERR_SHAPE;            // 16-byte row pitches for TMA
    if (p.half < 0 || p.half % 8 || 2 * p.half > DL_HD || (p.half > 0 && (!p.cosv || !p.sinv))) return GL_ERR_SHAPE;
    if (p.max_pages <= 0 || p.n_pages <= 0) return GL_ERR_SHAPE;
    return GL_OK;
}

struct DlCut { int tiles_q, tiles_u, kc1, per1, maxseg1, tiles3, kc3a, kc3, per3, maxseg3, maxsegA; };

static void dl_cut(const DecodeLayerArgs& p, int blocks, DlCut* k) {
    const int Nqkv = (p.nH + 2 * p.nKV) * DL_HD, No = p.nH * DL_HD;
    k->tiles_q = (Nqkv + DL_ROWS - 1) / DL_ROWS;
    k->tiles_u = (p.I + DL_ROWS - 1) / DL_ROWS;
    k->kc1 = (p.D + DL_BK - 1) / DL_BK;
    const long long t1 = (long long)(k->tiles_q + k->tiles_u) * k->kc1;
    k->per1 = (int)((t1 + blocks - 1) / blocks);
    {
        // whole tiles to a block, where that keeps nine blocks in ten busy: a tile then ends in the
        // block that began it, without the detour through scratch
        const long long tiles = k->tiles_q + k->tiles_u, each = (tiles + blocks - 1) / blocks;
        if (tiles * 10 >= (long long)blocks * each * 9) k->per1 = (int)(each * k->kc1);
    }
    k->maxseg1 = (k->kc1 - 1) / k->per1 + 2;
    k->tiles3 = (p.D + DL_ROWS - 1) / DL_ROWS;
    k->kc3a = (No + DL_BK - 1) / DL_BK;
    k->kc3 = k->kc3a + (p.I + DL_BK - 1) / DL_BK;
    const long long t3 = (long long)k->tiles3 * k->kc3;
    k->per3 = (int)((t3 + blocks - 1) / blocks);
    {
        const long long each = (k->tiles3 + blocks - 1) / blocks;
        if ((long long)k->tiles3 * 10 >= (long long)blocks * each * 9) k->per3 = (int)(each * k->kc3);
    }
    k->maxseg3 = (k->kc3 - 1) / k->per3 + 2;
    k->maxsegA = (p.max_pages < blocks ? p.max_pages : blocks) + 1;
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
    dl_cut(p, plan.blocks, &k);
    const int G = p.nH / p.nKV;
    const long long mrows = p.M <= 8 ? 8 : p.M <= 16 ? 16 : p.M <= 32 ? 32 : 64;
    *scratch_floats = (long long)(k.tiles_q + k.tiles_u) * k.maxseg1 * mrows * DL_ROWS +
                      (long long)k.tiles3 * k.maxseg3 * mrows * DL_ROWS +
                      (long long)p.M * p.nKV * k.maxsegA * (G * DL_HD + 2 * G);
    *sync_ints = DL_SYNC_HEAD + (long long)(k.tiles_q + k.tiles_u) + k.tiles3 + (long long)DL_MAXB * p.nKV;
    return GL_OK;
}

GL_API int gl_decode_layer_head_dim() { return DL_HD; }

template <int MT>
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
    if ((rc = gl_cached_map_bf16(&a.a_xn, p.xn, (uint64_t)p.M, (uint64_t)p.D, MT * 8, DL_BK)) != GL_OK) return rc;
    if ((rc = gl_cached_map_bf16(&a.a_o, p.o, (uint64_t)p.M, (uint64_t)a.No, MT * 8, DL_BK)) != GL_OK) return rc;
    if ((rc = gl_cached_map_bf16(&a.a_h, p.h, (uint64_t)p.M, (uint64_t)p.I, MT * 8, DL_BK)) != GL_OK) return rc;
    const uint64_t kv_rows = (uint64_t)p.n_pages * p.nKV * GL_PAGE;
    if ((rc = dl_plain_map(&a.k_pages, p.k_cache, kv_rows, DL_HD)) != GL_OK) return rc;
    if ((rc = dl_plain_map(&a.v_pages, p.v_cache, kv_rows, DL_HD)) != GL_OK) return rc;
    a.tiles_q = k.tiles_q; a.tiles_u = k.tiles_u; a.kc1 = k.kc1; a.per1 = k.per1; a.maxseg1 = k.maxseg1;
    a.tiles3 = k.tiles3; a.kc3a = k.kc3a; a.kc3 = k.kc3; a.per3 = k.per3; a.maxseg3 = k.maxseg3;
    a.maxsegA = k.maxsegA;
    a.stages = plan.stages;
    a.stage_bytes = plan.stage_bytes;
    const size_t sz = (size_t)MT * 8 * DL_ROWS;
    a.scratch1 = p.scratch;
    a.scratch3 = a.scratch1 + (size_t)(k.tiles_q + k.tiles_u) * k.maxseg1 * sz;
    a.scratchA = a.scratch3 + (size_t)k.tiles3 * k.maxseg3 * sz;
    a.gridbar = (unsigned*)p.sync;
    a.cnt1 = p.sync + DL_SYNC_HEAD;
    a.cnt3 = a.cnt1 + k.tiles_q + k.tiles_u;
    a.cntA = a.cnt3 + k.tiles3;

    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)plan.blocks);
    cfg.blockDim = dim3(DL_THREADS);
    cfg.dynamicSmemBytes = plan.smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;          // every block resident at once: they wait for one another
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, decode_layer_kernel<MT>, a) != cudaSuccess) {
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
    dl_cut(p, plan.blocks, &k);
    if (p.M <= 8) return dl_launch<1>(p, plan, k, stream);
    if (p.M <= 16) return dl_launch<2>(p, plan, k, stream);
    if (p.M <= 32) return dl_launch<4>(p, plan, k, stream);
    return dl_launch<8>(p, plan, k, stream);
}
