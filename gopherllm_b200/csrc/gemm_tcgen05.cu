// out[M,N] = act(A[M,K] · W[N,K]ᵀ + bias) + add0 + add1 for many rows, bfloat16,
// on the 5th-generation tensor cores.
//
// A persistent kernel, one block per SM, walks the 128 x BN output tiles.  Warp 0
// feeds shared memory by TMA (128-byte swizzled boxes of 64 k, several stages
// ahead); one thread of warp 1 issues tcgen05.mma (M 128, N BN, K 16, both
// operands K-major from shared memory, accumulator in tensor memory) and hands
// stages back through tcgen05.commit; warps 2..5 read a finished accumulator out
// of tensor memory (tcgen05.ld, one row per thread), apply bias, activation and
// the residual additions in 32-bit and store.  Two accumulators alternate, so the
// epilogue of one tile runs under the products of the next; to stay under them it must
// not wait on memory or queue behind the operand traffic, so the bias of a tile is fetched
// before its accumulator is ready and results leave by TMA from a swizzled patch in shared
// memory: a plain tile store, or, for a product that is added onto its own output (out =
// out + product, the residual stream), TMA's add-reduction, which loads nothing.  Rows and columns
// outside the matrices are zero-filled by TMA and masked at the store.
//
// Every wait on an mbarrier is bounded; if one runs out the block records it,
// leaves its loops, frees its tensor memory and returns.
#include <type_traits>

#include "common.cuh"
#include "tma.cuh"
#include "tcgen05.cuh"

#define TG_BM 128
#define TG_BK 64
#define TG_THREADS 192

struct GemmArgs {
    const void* a;        // [M, K] bf16
    const void* w;        // [N, K] bf16
    const float* bias;    // [N] or null
    const float* add0;    // [M, N] or null
    const float* add1;    // [M, N] or null
    void* out;            // [M, N] f32 or bf16
    int M, N, K, act;
    // a second product summed into the same tile (out = act(a w^T + a2 w2^T + bias + bias2) + ...): two
    // branches that end on the same rows and columns cost one epilogue.  The second product starts on a
    // k-block of its own (what the first one's last block lacks is zero-filled by TMA).
    const void* a2;       // [M, K2] bf16 or null
    const void* w2;       // [N, K2] bf16
    const float* bias2;   // [N] or null
    int K2;
    // a second set of columns from the same rows (outB = actB(a wB^T + biasB)): two branches that start
    // from the same input run as one grid, whose tiles fill the SMs' waves together.  Only with tile
    // stores (no tensors to add), without a second product and without cut tiles.
    const void* wB;       // [NB, K] bf16 or null
    const float* biasB;   // [NB] or null
    void* outB;           // [M, NB], the type of out
    int NB, actB;
};

// The work of one block: whole output tiles taken round-robin, or (split) an equal share of all
// (tile, k-block) units in tile order, which cuts tiles where shares meet.  A cut tile is finished by
// two or more blocks, each adding its part onto the output, so split work needs the add-reduction
// epilogue and no activation; the part that starts at k-block 0 carries the bias.
struct TgWork {
    long long u, end;
    int tile, step, n_tiles, k_blocks, split;
    __device__ TgWork(int n_tiles_, int k_blocks_, int split_) : n_tiles(n_tiles_), k_blocks(k_blocks_), split(split_) {
        const long long units = (long long)n_tiles * k_blocks;
        u = units * blockIdx.x / gridDim.x;
        end = units * (blockIdx.x + 1) / gridDim.x;
        tile = blockIdx.x;
        step = gridDim.x;
    }
    __device__ bool next(int& t, int& kb0, int& kb1) {
        if (!split) {
            if (tile >= n_tiles) return false;
            t = tile; kb0 = 0; kb1 = k_blocks;
            tile += step;
            return true;
        }
        if (u >= end) return false;
        t = (int)(u / k_blocks);
        kb0 = (int)(u % k_blocks);
        const long long left = end - u;
        kb1 = (left < k_blocks - kb0) ? kb0 + (int)left : k_blocks;
        u += kb1 - kb0;
        return true;
    }
};

// Tile number -> (row tile, column tile).  Tiles are numbered group by group: a group is `group` row tiles
// by all column tiles, row tile fastest.  Blocks work on neighbouring numbers at the same time, so within a
// group they share one weight tile and a few activation tiles, and the group's activations stay in L2
// while the weights stream past; without groups (all row tiles fastest) a matrix of activations larger
// than L2 would come from memory once per column tile.
__device__ __forceinline__ void tg_tile_coords(int tile, int tiles_m, int tiles_n_all, int group, int& mt, int& nt) {
    const int per_group = group * tiles_n_all;
    const int g = tile / per_group, r = tile - g * per_group;
    const int rows = min(group, tiles_m - g * group);
    nt = r / rows;
    mt = g * group + (r - nt * rows);
}

// K-major operand tile of 128-byte rows (64 bf16 of K), 128-byte swizzle
__device__ __forceinline__ uint64_t umma_desc(unsigned smem_addr) { return umma_tile_desc(smem_addr, 128); }
__host__ __device__ constexpr uint32_t umma_idesc(int bn) { return umma_idesc_bf16(bn, 0); }

// MT: 128-row sub-tiles of a block's tile (1 or 2).  With 2, the block's two products of a k-step share
// the weight tile in shared memory, which cuts the operand bytes pulled from L2 per flop: at these tile
// sizes L2 bandwidth, not the tensor pipe, sets the pace.  The accumulators then fill tensor memory
// (no second set), so a tile's epilogue is not hidden behind the next tile's products.
template <int BN, int STAGES, typename TO, int MT>
__global__ void __launch_bounds__(TG_THREADS, 1)
gemm_tcgen05_kernel(GemmArgs g, const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                    const __grid_constant__ CUtensorMap map_a2, const __grid_constant__ CUtensorMap map_w2,
                    const __grid_constant__ CUtensorMap map_out, const __grid_constant__ CUtensorMap map_wB,
                    const __grid_constant__ CUtensorMap map_outB, int out_mode, int split, int group) {
    extern __shared__ unsigned char smem_raw[];
    constexpr int A_BYTES = MT * TG_BM * 128, B_BYTES = BN * 128, STAGE = A_BYTES + B_BYTES;
    constexpr int NBUF = 2 * MT * BN <= 512 ? 2 : 1;                                      // accumulator sets
    static_assert(MT * BN <= 512, "the accumulators of a tile must fit tensor memory");
    constexpr unsigned TMEM_COLS = NBUF * MT * BN <= 128 ? 128 : (NBUF * MT * BN <= 256 ? 256 : 512);   // a power of two
    __shared__ unsigned tmem_base_slot;
    __shared__ volatile int failed;

    unsigned char* smem = smem_raw + ((1024u - (gl_smem_u32(smem_raw) & 1023u)) & 1023u);
    const unsigned base = gl_smem_u32(smem);
    const unsigned bar_full = base + STAGES * STAGE;          // [STAGES]; the barriers own 1024 bytes
    const unsigned bar_empty = bar_full + 8 * STAGES;         // [STAGES]
    const unsigned bar_tfull = bar_empty + 8 * STAGES;        // [2] accumulator ready for the epilogue
    const unsigned bar_tempty = bar_tfull + 16;               // [2] accumulator drained
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_m = (g.M + MT * TG_BM - 1) / (MT * TG_BM), tiles_n = (g.N + BN - 1) / BN;
    const int tiles_n_all = tiles_n + (g.wB ? (g.NB + BN - 1) / BN : 0);            // the second set's tiles follow the first's
    const int n_tiles = tiles_m * tiles_n_all;
    const int k1_blocks = (g.K + TG_BK - 1) / TG_BK;                   // k-blocks of the first product
    const int k_blocks = k1_blocks + (g.a2 ? (g.K2 + TG_BK - 1) / TG_BK : 0);

    if (threadIdx.x == 0) {
        failed = 0;
        for (int s = 0; s < STAGES; ++s) { mbar_init(bar_full + 8 * s, 1); mbar_init(bar_empty + 8 * s, 1); }
        for (int b = 0; b < NBUF; ++b) { mbar_init(bar_tfull + 8 * b, 1); mbar_init(bar_tempty + 8 * b, 4); }
        mbar_fence_init();
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(gl_smem_u32(&tmem_base_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_base = tmem_base_slot;
    // launched programmatically: set up while the kernel before still runs, read and write after it
    gl_grid_launch_dependents();
    gl_grid_wait();

    if (warp == 0) {
        // ---- TMA producer -------------------------------------------------
        if (lane == 0) {
            int it = 0, tile, kb0, kb1;
            TgWork work(n_tiles, k_blocks, split);
            while (!failed && work.next(tile, kb0, kb1)) {
                int mt, nt;
                tg_tile_coords(tile, tiles_m, tiles_n_all, group, mt, nt);
                const bool fork = nt >= tiles_n;
                const int m0 = mt * MT * TG_BM, n0 = (nt - (fork ? tiles_n : 0)) * BN;
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (it >= STAGES && !mbar_wait(bar_empty + 8 * s, ((it / STAGES) - 1) & 1)) { failed = 1; break; }
                    const unsigned sb = base + s * STAGE;
                    mbar_expect_tx(bar_full + 8 * s, STAGE);
                    const bool second = kb >= k1_blocks;
                    const CUtensorMap* ma = second ? &map_a2 : &map_a;
                    const CUtensorMap* mw = fork ? &map_wB : (second ? &map_w2 : &map_w);
                    const int k0 = (second ? kb - k1_blocks : kb) * TG_BK;
#pragma unroll
                    for (int i = 0; i < MT; ++i)
                        tma_load_2d(sb + i * TG_BM * 128, ma, k0, m0 + i * TG_BM, bar_full + 8 * s);
                    tma_load_2d(sb + A_BYTES, mw, k0, n0, bar_full + 8 * s);
                }
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer ------------------------------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc(BN);
            int it = 0, local = 0, tile, kb0, kb1;
            TgWork work(n_tiles, k_blocks, split);
            for (; !failed && work.next(tile, kb0, kb1); ++local) {
                const int buf = local % NBUF, use = local / NBUF;
                if (use >= 1 && !mbar_wait(bar_tempty + 8 * buf, (use - 1) & 1)) { failed = 1; break; }
                tc_fence_after();
                const unsigned d = tmem_base + buf * MT * BN;
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait(bar_full + 8 * s, (it / STAGES) & 1)) { failed = 1; break; }
                    tc_fence_after();
                    const unsigned sb = base + s * STAGE;
                    const uint64_t db = umma_desc(sb + A_BYTES);
#pragma unroll
                    for (int i = 0; i < MT; ++i) {
                        const uint64_t da = umma_desc(sb + i * TG_BM * 128);
#pragma unroll
                        for (int k = 0; k < TG_BK / 16; ++k)     // 32 bytes further along the swizzled row per K 16
                            umma_bf16(d + i * BN, da + 2 * k, db + 2 * k, idesc, kb != kb0 || k != 0);
                    }
                    umma_commit(bar_empty + 8 * s);          // the stage is free once these products have read it
                }
                if (failed) break;
                umma_commit(bar_tfull + 8 * buf);            // the accumulator is complete
            }
        }
    } else {
        // ---- epilogue: warps 2..5, each on the tensor-memory lanes of its quarter -----
        // A thread reads one accumulator row (32 columns at a time); the warp turns the 32 x 32
        // patch round in shared memory so that each store (and each load of the tensors to add)
        // covers 32 consecutive columns of one row.
        const int quarter = warp & 3;
        // per warp: a 32 x 32 patch of 32-bit values (4 KB, 1024-byte aligned for the swizzled
        // TMA reduction; read back with a 33-float pitch view for the plain store) and the tile's bias
        unsigned char* epi = smem + STAGES * STAGE + 1024;               // barriers live in the first 1024 bytes
        float* patch = (float*)(epi + (warp - 2) * 5120);                // 5 KB apart: every patch starts on a 1024-byte boundary
        float* bias_s = (float*)(epi + 4 * 5120) + (warp - 2) * BN;
        const unsigned patch_u32 = gl_smem_u32(patch);
        int local = 0, tile, kb0, kb1;
        TO* O = (TO*)g.out;
        TgWork work(n_tiles, k_blocks, split);
        for (; work.next(tile, kb0, kb1); ++local) {
            const int buf = local % NBUF, use = local / NBUF;
            int mt, nt;
            tg_tile_coords(tile, tiles_m, tiles_n_all, group, mt, nt);
            const bool fork = nt >= tiles_n;
            const int m0 = mt * MT * TG_BM, n0 = (nt - (fork ? tiles_n : 0)) * BN;
            const int N = fork ? g.NB : g.N, act = fork ? g.actB : g.act;
            const float* bias = fork ? g.biasB : g.bias;
            const CUtensorMap* mo = fork ? &map_outB : &map_out;
            // before the accumulator is ready: this tile's bias into shared memory
            __syncwarp();
            for (int j = lane; j < BN; j += 32) {
                float bv = 0.f;
                if (kb0 == 0 && n0 + j < N) {
                    if (bias) bv = bias[n0 + j];
                    if (g.bias2) bv += g.bias2[n0 + j];
                }
                bias_s[j] = bv;
            }
            bool ok = mbar_wait(bar_tfull + 8 * buf, use & 1);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) { failed = 1; break; }
            tc_fence_after();
            // The activation is a constant inside the loops (one copy of them per kind): a tile's kind is
            // known only at run time, and a choice per element would put a chain of branches into every value.
            auto store_tile = [&](auto act_c) {
            constexpr int ACT = decltype(act_c)::value;
#pragma unroll 1
            for (int sub = 0; sub < MT; ++sub) {
            const int mrow0 = m0 + sub * TG_BM + quarter * 32;
            const unsigned trow = tmem_base + (buf * MT + sub) * BN + ((unsigned)(quarter * 32) << 16);
            // out_mode 1: tile store by TMA; 2: add-reduction by TMA; 0: element-wise (any alignment,
            // tensors to add that are not the output)
            constexpr int CW = sizeof(TO) == 4 ? 32 : 64;              // columns per 128-byte patch row
            if (out_mode != 0) {
#pragma unroll 1
                for (int c = 0; c < BN; c += CW) {
                    unsigned r[32], r2[32];
                    tmem_ld32(trow + c, r);
                    if (CW == 64) tmem_ld32(trow + c + 32, r2);
                    if (lane == 0) bulk_wait_read<0>();                  // the patch's last copy has been read
                    __syncwarp();
#pragma unroll
                    for (int q = 0; q < 8; ++q) {                        // 16-byte chunks, swizzled as TMA expects
                        uint4 pk;
                        if (CW == 32) {
                            pk.x = __float_as_uint(gl_activate<false>(__uint_as_float(r[4 * q + 0]) + bias_s[c + 4 * q + 0], ACT));
                            pk.y = __float_as_uint(gl_activate<false>(__uint_as_float(r[4 * q + 1]) + bias_s[c + 4 * q + 1], ACT));
                            pk.z = __float_as_uint(gl_activate<false>(__uint_as_float(r[4 * q + 2]) + bias_s[c + 4 * q + 2], ACT));
                            pk.w = __float_as_uint(gl_activate<false>(__uint_as_float(r[4 * q + 3]) + bias_s[c + 4 * q + 3], ACT));
                        } else {
                            float v[8];
#pragma unroll
                            for (int e = 0; e < 8; ++e) {
                                const unsigned raw = q < 4 ? r[8 * q + e] : r2[8 * (q - 4) + e];
                                v[e] = gl_activate_bf16_grade(__uint_as_float(raw) + bias_s[c + 8 * q + e], ACT);
                            }
                            __nv_bfloat162 p0 = __floats2bfloat162_rn(v[0], v[1]), p1 = __floats2bfloat162_rn(v[2], v[3]);
                            __nv_bfloat162 p2 = __floats2bfloat162_rn(v[4], v[5]), p3 = __floats2bfloat162_rn(v[6], v[7]);
                            pk.x = *(unsigned*)&p0; pk.y = *(unsigned*)&p1; pk.z = *(unsigned*)&p2; pk.w = *(unsigned*)&p3;
                        }
                        *(uint4*)((unsigned char*)patch + lane * 128 + ((q ^ (lane & 7)) << 4)) = pk;
                    }
                    fence_proxy_async();
                    __syncwarp();
                    if (lane == 0 && mrow0 < g.M && n0 + c < N) {
                        if (out_mode == 2) tma_reduce_add_2d(mo, n0 + c, mrow0, patch_u32);
                        else tma_store_2d(mo, n0 + c, mrow0, patch_u32);
                        bulk_commit();
                    }
                }
            } else {
#pragma unroll 1
                for (int c = 0; c < BN; c += 32) {
                    unsigned r[32];
                    tmem_ld32(trow + c, r);
                    __syncwarp();
#pragma unroll
                    for (int j = 0; j < 32; ++j) patch[lane * 33 + j] = __uint_as_float(r[j]);
                    __syncwarp();
                    const int n = n0 + c + lane;
                    if (n < N) {              // (element-wise results are never of a second set: N is g.N here)
                        const float bv = bias_s[c + lane];
                        const int rows_here = min(32, g.M - mrow0);
#pragma unroll 4
                        for (int rr = 0; rr < rows_here; ++rr) {
                            float v = gl_activate<false>(patch[rr * 33 + lane] + bv, ACT);
                            const size_t o = (size_t)(mrow0 + rr) * g.N + n;
                            if (g.add0) v += g.add0[o];
                            if (g.add1) v += g.add1[o];
                            gl_store(O + o, v);
                        }
                    }
                }
            }
            }
            };
            switch (act) {
                case GL_ACT_GELU_TANH: store_tile(std::integral_constant<int, GL_ACT_GELU_TANH>{}); break;
                case GL_ACT_GELU_ERF: store_tile(std::integral_constant<int, GL_ACT_GELU_ERF>{}); break;
                case GL_ACT_RELU: store_tile(std::integral_constant<int, GL_ACT_RELU>{}); break;
                default: store_tile(std::integral_constant<int, GL_ACT_NONE>{}); break;
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_tempty + 8 * buf);
        }
        if (lane == 0) bulk_wait<0>();           // every reduction of this thread has reached memory
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
    if (threadIdx.x == 0 && failed) atomicExch(&gl_wait_failed, 1);
}

template <int BN, int STAGES, int MT>
static constexpr size_t tg_smem() {
    // stages, 1024 bytes of barriers, the epilogue warps' patches and bias rows, room to align the start
    return (size_t)STAGES * (MT * TG_BM * 128 + BN * 128) + 1024 + 4 * 5120 + 4 * BN * 4 + 1024;
}

// 0 (the default) never cuts tiles: inside a model step, where the products run back to back at the
// power limit, cutting gained nothing measurable, and whole tiles keep the sums in one order.  1 cuts
// whenever the epilogue allows; -1 cuts when whole tiles would leave more than 8% of the SMs' slots empty
// (alone and from a cold L2 that took a 2048 x 2560 x 10240 product from 142 to 120 us).
static int tg_split_mode = 0;
GL_API void gl_gemm_tcgen05_set_split(int mode) { tg_split_mode = mode; }

template <int BN, int STAGES, typename TO, int MT = 1>
static int launch_tg(const GemmArgs& g, cudaStream_t stream) {
    constexpr size_t smem = tg_smem<BN, STAGES, MT>();
    static_assert(smem <= 227 * 1024, "shared memory of a block");
    static bool configured = false;
    static int sms = 0;
    if (!configured) {
        if (cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, STAGES, TO, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem) != cudaSuccess) {
            cudaGetLastError();
            return GL_ERR_SMEM;
        }
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (sms <= 0) sms = 148;
        configured = true;
    }
    CUtensorMap map_a, map_w;
    int rc = gl_cached_map_bf16(&map_a, g.a, (uint64_t)g.M, (uint64_t)g.K, TG_BM, TG_BK);
    if (rc != GL_OK) return rc;
    rc = gl_cached_map_bf16(&map_w, g.w, (uint64_t)g.N, (uint64_t)g.K, BN, TG_BK);
    if (rc != GL_OK) return rc;
    CUtensorMap map_a2 = map_a, map_w2 = map_w;
    if (g.a2) {
        rc = gl_cached_map_bf16(&map_a2, g.a2, (uint64_t)g.M, (uint64_t)g.K2, TG_BM, TG_BK);
        if (rc != GL_OK) return rc;
        rc = gl_cached_map_bf16(&map_w2, g.w2, (uint64_t)g.N, (uint64_t)g.K2, BN, TG_BK);
        if (rc != GL_OK) return rc;
    }
    // How results leave: by TMA when the output's rows are whole 16-byte units and nothing has to be
    // loaded: a plain store when nothing is added, an add-reduction for out = out + product (add0
    // is the output itself, 32-bit); otherwise element by element.
    int out_mode = 0;
    CUtensorMap map_out = map_a;
    GemmArgs ga = g;
    const bool aligned = (g.N * sizeof(TO)) % 16 == 0 && ((uintptr_t)g.out & 15) == 0;
    if (aligned && !g.add0 && !g.add1) {
        out_mode = 1;
    } else if (aligned && sizeof(TO) == 4 && g.add0 == (const float*)g.out && !g.add1) {
        out_mode = 2;
        ga.add0 = nullptr;
    }
    if (out_mode != 0) {
        rc = gl_cached_map(&map_out, g.out, (uint64_t)g.M, (uint64_t)g.N, 32, sizeof(TO) == 4 ? 32 : 64, (uint32_t)sizeof(TO));
        if (rc != GL_OK) return rc;
    }
    CUtensorMap map_wB = map_w, map_outB = map_out;
    if (g.wB) {
        if (out_mode != 1 || g.a2 || (g.NB * sizeof(TO)) % 16 || ((uintptr_t)g.outB & 15)) return GL_ERR_SHAPE;
        rc = gl_cached_map_bf16(&map_wB, g.wB, (uint64_t)g.NB, (uint64_t)g.K, BN, TG_BK);
        if (rc != GL_OK) return rc;
        rc = gl_cached_map(&map_outB, g.outB, (uint64_t)g.M, (uint64_t)g.NB, 32, sizeof(TO) == 4 ? 32 : 64, (uint32_t)sizeof(TO));
        if (rc != GL_OK) return rc;
    }
    const int tiles = ((g.M + MT * TG_BM - 1) / (MT * TG_BM)) * ((g.N + BN - 1) / BN + (g.wB ? (g.NB + BN - 1) / BN : 0));
    // Tiles that fill the SMs unevenly are cut where the blocks' equal shares meet, if the epilogue can
    // add parts onto the output and every share still holds a fair run of k-blocks.
    const int k_blocks = (g.K + TG_BK - 1) / TG_BK + (g.a2 ? (g.K2 + TG_BK - 1) / TG_BK : 0);
    const int waves = (tiles + sms - 1) / sms;
    const bool uneven = tiles % sms != 0 && (long long)tiles * 100 < (long long)waves * sms * 92;
    // (alone it pays only for a long K: a cut tile costs a second add-reduction of its 32-bit patch)
    const bool can_split = out_mode == 2 && g.act == GL_ACT_NONE && (long long)tiles * k_blocks >= 8LL * sms;
    // (with few rows the tiles are fewer than the SMs: equal shares then whatever the mode when under 70 %
    // of the SMs would have a tile, since part of the machine would otherwise stream all the weights)
    const int split = can_split && (tg_split_mode > 0 || (tg_split_mode < 0 && uneven && k_blocks >= 64) || tiles * 10 < sms * 7);
    const int grid = split ? sms : (tiles < sms ? tiles : sms);
    // row tiles of a group: as many as keep the group's activations (all of K) within 28 MB
    const long long a_tile_bytes = (long long)MT * TG_BM * (g.K + (g.a2 ? g.K2 : 0)) * 2;
    int group = (int)((28LL << 20) / a_tile_bytes);
    group = group < 1 ? 1 : group;
    if (gl_launch(gemm_tcgen05_kernel<BN, STAGES, TO, MT>, dim3(grid), dim3(TG_THREADS), smem, stream, 1, ga, map_a, map_w, map_a2, map_w2,
                  map_out, map_wB, map_outB, out_mode, split, group) != 0)
        return GL_ERR_LAUNCH;
    return GL_OK;
}

template <typename TO>
static int dispatch_bn(const GemmArgs& g, int bn, cudaStream_t stream) {
    if (bn == 256) return launch_tg<256, 4, TO>(g, stream);
    if (bn == 192) return launch_tg<192, 5, TO>(g, stream);
    if (bn == 128) return launch_tg<128, 6, TO>(g, stream);
    if (bn == 64) return launch_tg<64, 8, TO>(g, stream);
    if (bn == 160 && sizeof(TO) == 4) return launch_tg<160, 5, TO>(g, stream);    // 160 is no multiple of 64: 32-bit outputs only
    // 1000 + width: tiles of 256 rows
    if (bn == 1256) return launch_tg<256, 3, TO, 2>(g, stream);
    if (bn == 1192) return launch_tg<192, 3, TO, 2>(g, stream);
    if (bn == 1160 && sizeof(TO) == 4) return launch_tg<160, 3, TO, 2>(g, stream);
    return GL_ERR_SHAPE;
}

GL_API int gl_gemm_tcgen05_wait_failed() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, gl_wait_failed, sizeof(int)) != cudaSuccess) return -1;
    return v;
}

// bn: tile width 64, 128 or 256; 0 lets the launcher choose
GL_API int gl_gemm_tcgen05(const GemmArgs* args, int out_dtype, int bn, cudaStream_t stream) {
    const GemmArgs& g = *args;
    if (g.M <= 0 || g.N <= 0) return GL_OK;
    if (g.K <= 0 || g.K % 8) return GL_ERR_SHAPE;
    if (((uintptr_t)g.a | (uintptr_t)g.w) & 15) return GL_ERR_ALIGN;
    if (g.a2) {
        // the second product starts on a k-block of its own: a partial last block of the first would
        // be padded with zeros by TMA, which is fine, but K2 still needs whole 16-byte rows
        if (!g.w2 || g.K2 <= 0 || g.K2 % 8) return GL_ERR_SHAPE;
        if (((uintptr_t)g.a2 | (uintptr_t)g.w2) & 15) return GL_ERR_ALIGN;
    }
    if (g.wB) {
        if (g.NB <= 0 || !g.outB || g.a2 || g.add0 || g.add1) return GL_ERR_SHAPE;
        if ((uintptr_t)g.wB & 15) return GL_ERR_ALIGN;
    }
    if (bn == 0) {
        // A tile's time goes with the operand bytes it pulls from L2, about (128 + width); the
        // grid runs in waves of one tile per SM, and the last wave counts whole.
        static int sms = 0;
        if (!sms) {
            int dev = 0;
            cudaGetDevice(&dev);
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
            if (sms <= 0) sms = 148;
        }
        const int tm = (g.M + TG_BM - 1) / TG_BM;
        long best = -1;
        const int cands[5] = {256, 192, 160, 128, 64};
        for (int i = 0; i < 5; ++i) {
            const int c = cands[i];
            if (c == 160 && out_dtype != GL_F32) continue;
            const int tiles = tm * ((g.N + c - 1) / c + (g.wB ? (g.NB + c - 1) / c : 0));
            long cost = (long)((tiles + sms - 1) / sms) * (TG_BM + c) * 1000;
            // Fewer tiles than 70 % of the SMs, added onto a 32-bit output: launch_tg cuts them into equal
            // shares of (tile, k-block) units, so there are no waves; an SM's share of the operand bytes
            // counts, plus the add-reduction of its part of a tile, which grows with the tile's width
            // (measured at 2560 x 12800: 128 rows 19 us at width 128 against 22 at 64 and 25 at 256;
            // 256 rows 26 against 37 and 28; 512 rows 39 at width 256 against 43 at 128).
            const long k_blocks = (g.K + TG_BK - 1) / TG_BK + (g.a2 ? (g.K2 + TG_BK - 1) / TG_BK : 0);
            if (out_dtype == GL_F32 && g.add0 == (const float*)g.out && !g.add1 && g.act == GL_ACT_NONE && !g.wB &&
                tiles * 10 < sms * 7 && (long)tiles * k_blocks >= 8L * sms)
                cost = (long)tiles * (TG_BM + c) * 1000 / sms + 150L * c;
            if (best < 0 || cost < best) { best = cost; bn = c; }
        }
        // A long product added onto its 32-bit output, many rows, few columns (the second feed-forward
        // product): tiles of 256 x 160 when one wave of them covers the output.  Two products of a
        // k-step then share the weight tile (81 instead of 112 bytes from L2 per clock of tensor work);
        // measured 108 against 127 us at 2048 x 2560 x 10240.  Shorter products gain nothing from it.
        const int big_tiles = ((g.M + 255) / 256) * ((g.N + 159) / 160);
        if (out_dtype == GL_F32 && g.add0 == (const float*)g.out && !g.add1 && g.K + (g.a2 ? g.K2 : 0) >= 5120 &&
            big_tiles <= sms && big_tiles * 10 >= sms * 7)      // (fewer would leave SMs idle, or cut tiles into costly parts)
            bn = 1160;
    }
    if (out_dtype == GL_F32) return dispatch_bn<float>(g, bn, stream);
    if (out_dtype == GL_BF16) return dispatch_bn<__nv_bfloat16>(g, bn, stream);
    return GL_ERR_DTYPE;
}
