// out[M,N] = act(A[M,K] · W[N,K]ᵀ + bias) + add0 + add1 for 17 to 64 rows (tokens), bfloat16, on the
// 5th-generation tensor cores with the product turned round: the WEIGHTS are the 128-row operand of
// tcgen05.mma, the tokens its N (32 or 64).
//
// With a few dozen tokens a product is still a stream of weights, but the tokens' tile is no longer
// small beside the weights' tile: the mma.sync kernel for few rows fetches 64 tokens x 64 k (8 KB, from
// L2) for every 64 weight rows x 64 k (8 KB, from HBM), and the L2's traffic, not HBM, sets its pace
// (batch 64 ran at a third of the HBM rate).  Here a block owns 128 weight rows, so the tokens' tile is
// fetched half as often per weight byte; one thread issues the products, the accumulator (128 weight
// rows x tokens, 32-bit) lives in tensor memory, and the warps that would have issued ldmatrix and mma
// do nothing until the epilogue.  Weights and tokens arrive by TMA (128-byte swizzled boxes of 64 k),
// the weights' first stages before the kernel waits for the one before it.
//
// To fill the SMs when N is small, K is cut over the blocks of a thread-block cluster (up to 16); the
// partial tiles meet in distributed shared memory and each block finishes its share of the tile's weight
// rows, adding the parts in rank order, so the result does not depend on timing.  A second product may
// be summed into the same output (K is then the joined length, the first K a multiple of 64).
// Every wait on an mbarrier is bounded; if one runs out the block records it and goes on to the end
// without waiting again (the cluster's barriers still have to be met).
#include <cooperative_groups.h>

#include "common.cuh"
#include "tma.cuh"
#include "tcgen05.cuh"
namespace cg = cooperative_groups;

#define GS_ROWS 128          // weight rows per block
#define GS_BK 64             // k per stage
#define GS_THREADS 192       // loading warp, issuing warp, four epilogue warps
#define GS_WBYTES (GS_ROWS * 128)

struct GemmArgs {
    const void* a;        // [M, K] bf16
    const void* w;        // [N, K] bf16
    const float* bias;    // [N] or null
    const float* add0;    // [M, N] or null
    const float* add1;    // [M, N] or null
    void* out;            // [M, N] f32 or bf16
    int M, N, K, act;
    const void* a2;       // [M, K2] bf16 or null: a second product summed into the same output
    const void* w2;       // [N, K2] bf16
    const float* bias2;   // [N] or null
    int K2;
};

template <int BN, int STAGES, typename TO>
__global__ void __launch_bounds__(GS_THREADS)
gemm_stream_kernel(GemmArgs g, int k_per_block, const __grid_constant__ CUtensorMap map_w,
                   const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w2,
                   const __grid_constant__ CUtensorMap map_a2) {
    extern __shared__ unsigned char smem_raw[];
    constexpr int A_BYTES = BN * 128, STAGE = GS_WBYTES + A_BYTES;
    constexpr unsigned TMEM_COLS = BN <= 32 ? 32 : 64;
    static_assert(BN * GS_ROWS * 4 <= STAGES * STAGE, "the reduction tile reuses the stages");
    __shared__ unsigned tmem_slot;
    __shared__ volatile int failed;
    cg::cluster_group cluster = cg::this_cluster();
    const int S = (int)cluster.num_blocks(), rank = (int)cluster.block_rank();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.y * GS_ROWS;
    const int k1 = g.K, k_all = g.K + (g.a2 ? g.K2 : 0);
    const int kb = blockIdx.x * k_per_block;
    const int ke = min(k_all, kb + k_per_block);
    const int iters = ke > kb ? (ke - kb + GS_BK - 1) / GS_BK : 0;
    unsigned char* smem = smem_raw + ((1024u - (gl_smem_u32(smem_raw) & 1023u)) & 1023u);
    const unsigned base = gl_smem_u32(smem);
    const unsigned bar_full = base + STAGES * STAGE, bar_empty = bar_full + 8 * STAGES, bar_done = bar_empty + 8 * STAGES;

    if (threadIdx.x == 0) {
        failed = 0;
        for (int s = 0; s < STAGES; ++s) { mbar_init(bar_full + 8 * s, 1); mbar_init(bar_empty + 8 * s, 1); }
        mbar_init(bar_done, 1);
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc(gl_smem_u32(&tmem_slot), TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem = tmem_slot;
    gl_grid_launch_dependents();

    if (warp == 0) {
        // ---- loads: the weights of the first stages before this kernel waits for the one before it ----
        if (lane == 0) {
            auto load_w = [&](int it) {
                const int s = it % STAGES, k = kb + it * GS_BK;
                mbar_expect_tx(bar_full + 8 * s, STAGE);             // the tokens' tile counts too
                if (k < k1) tma_load_2d(base + s * STAGE, &map_w, k, n0, bar_full + 8 * s);
                else tma_load_2d(base + s * STAGE, &map_w2, k - k1, n0, bar_full + 8 * s);
            };
            auto load_a = [&](int it) {
                const int s = it % STAGES, k = kb + it * GS_BK;
                if (k < k1) tma_load_2d(base + s * STAGE + GS_WBYTES, &map_a, k, 0, bar_full + 8 * s);
                else tma_load_2d(base + s * STAGE + GS_WBYTES, &map_a2, k - k1, 0, bar_full + 8 * s);
            };
            const int head = iters < STAGES ? iters : STAGES;
            for (int it = 0; it < head; ++it) load_w(it);
            gl_grid_wait();
            for (int it = 0; it < head; ++it) load_a(it);
            for (int it = head; it < iters && !failed; ++it) {
                if (!mbar_wait(bar_empty + 8 * (it % STAGES), ((it / STAGES) - 1) & 1)) { failed = 1; break; }
                load_w(it);
                load_a(it);
            }
        }
    } else if (warp == 1) {
        // ---- products: one thread, D[128 weight rows, BN tokens] += W[128, 16] · X[BN, 16]ᵀ per k-step ----
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16(BN, 0);
            for (int it = 0; it < iters && !failed; ++it) {
                const int s = it % STAGES;
                if (!mbar_wait(bar_full + 8 * s, (it / STAGES) & 1)) { failed = 1; break; }
                tc_fence_after();
                const uint64_t da = umma_tile_desc(base + s * STAGE, 128), db = umma_tile_desc(base + s * STAGE + GS_WBYTES, 128);
#pragma unroll
                for (int k = 0; k < GS_BK / 16; ++k)                 // 32 bytes further along the swizzled row per K 16
                    umma_bf16(tmem, da + 2 * k, db + 2 * k, idesc, it != 0 || k != 0);
                umma_commit(bar_empty + 8 * s);                      // the stage is free once these products have read it
            }
            umma_commit(bar_done);                                   // the accumulator is complete
        }
    }
    // ---- everyone: the partial tile to shared memory as tile[token][weight row] (the stages are free) ----
    if (warp >= 2) gl_grid_wait();
    float* tile = (float*)smem;
    if (warp >= 2) {
        bool ok = iters == 0 || mbar_wait(bar_done, 0);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) failed = 1;
        tc_fence_after();
        const int quarter = warp & 3;                                // the tensor-memory lanes this warp may read
        const int nl = quarter * 32 + lane;                          // this thread's weight row within the tile
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
            unsigned r[32];
            if (iters > 0) tmem_ld32(tmem + ((unsigned)(quarter * 32) << 16) + c, r);
#pragma unroll
            for (int j = 0; j < 32; ++j) tile[(c + j) * GS_ROWS + nl] = iters > 0 ? __uint_as_float(r[j]) : 0.f;
        }
        tc_fence_before();
    }
    cluster.sync();
    // this block finishes weight rows [lo, hi) of the tile, summing the blocks' parts in rank order
    const int lo = rank * GS_ROWS / S, hi = (rank + 1) * GS_ROWS / S, cnt = hi - lo;
    TO* O = (TO*)g.out;
    // (four elements a thread at a time, everything they need from the peers' tiles and from memory asked for
    // before the first of them is stored: an element finished on its own would wait out a trip to a peer's
    // shared memory and one to L2 before the next could start)
    const int total = g.M * cnt;
    for (int i0 = threadIdx.x; i0 < total; i0 += 4 * GS_THREADS) {
        float v[4], b[4], a0[4], a1[4];
        size_t o[4];
        bool ok[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = i0 + u * GS_THREADS;
            const int m = i / cnt, nl = lo + (i - m * cnt), n = n0 + nl;
            ok[u] = i < total && n < g.N;
            o[u] = (size_t)m * g.N + n;
            v[u] = 0.f; b[u] = 0.f; a0[u] = 0.f; a1[u] = 0.f;
            if (ok[u]) {
                for (int s = 0; s < S; ++s) v[u] += cluster.map_shared_rank(tile, s)[m * GS_ROWS + nl];
                if (g.bias) b[u] = g.bias[n];
                if (g.bias2) b[u] += g.bias2[n];
                if (g.add0) a0[u] = g.add0[o[u]];
                if (g.add1) a1[u] = g.add1[o[u]];
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (ok[u]) gl_store(O + o[u], gl_activate<false>(v[u] + b[u], g.act) + a0[u] + a1[u]);
    }
    cluster.sync();                                                  // nobody leaves while a peer may still read its tile
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, TMEM_COLS);
    }
    if (threadIdx.x == 0 && failed) atomicExch(&gl_wait_failed, 1);
}

template <int BN, int STAGES>
static constexpr size_t gs_smem() {
    return (size_t)STAGES * (GS_WBYTES + BN * 128) + 8 * (2 * STAGES + 1) + 1024;
}

template <int BN, int STAGES, typename TO>
static int gs_launch(const GemmArgs& g, int S, cudaStream_t stream) {
    constexpr size_t smem = gs_smem<BN, STAGES>();
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(gemm_stream_kernel<BN, STAGES, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess ||
            cudaFuncSetAttribute(gemm_stream_kernel<BN, STAGES, TO>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) {
            cudaGetLastError();
            return GL_ERR_SMEM;
        }
        configured = true;
    }
    const int k_all = g.K + (g.a2 ? g.K2 : 0);
    const int k_per_block = ((k_all + S - 1) / S + GS_BK - 1) / GS_BK * GS_BK;
    CUtensorMap map_w, map_a;
    int rc = gl_cached_map_bf16(&map_w, g.w, (uint64_t)g.N, (uint64_t)g.K, GS_ROWS, GS_BK);
    if (rc != GL_OK) return rc;
    rc = gl_cached_map_bf16(&map_a, g.a, (uint64_t)g.M, (uint64_t)g.K, BN, GS_BK);
    if (rc != GL_OK) return rc;
    CUtensorMap map_w2 = map_w, map_a2 = map_a;
    if (g.a2) {
        rc = gl_cached_map_bf16(&map_w2, g.w2, (uint64_t)g.N, (uint64_t)g.K2, GS_ROWS, GS_BK);
        if (rc != GL_OK) return rc;
        rc = gl_cached_map_bf16(&map_a2, g.a2, (uint64_t)g.M, (uint64_t)g.K2, BN, GS_BK);
        if (rc != GL_OK) return rc;
    }
    const dim3 grid(S, (g.N + GS_ROWS - 1) / GS_ROWS, 1);
    if (grid.y > 65535) return GL_ERR_SHAPE;
    if (gl_launch(gemm_stream_kernel<BN, STAGES, TO>, grid, dim3(GS_THREADS), smem, stream, S, g, k_per_block, map_w, map_a, map_w2, map_a2) != 0)
        return GL_ERR_LAUNCH;
    return GL_OK;
}

template <typename TO>
static int gs_dispatch(const GemmArgs& g, int S, cudaStream_t stream) {
    // four stages of 20 or 24 KB: two blocks fit an SM, so one's epilogue runs under the other's stream
    if (g.M <= 32) return gs_launch<32, 4, TO>(g, S, stream);
    return gs_launch<64, 4, TO>(g, S, stream);
}

// split_k: 0 lets the launcher choose; else 1..16 blocks of a cluster share K
GL_API int gl_gemm_stream(const GemmArgs* args, int out_dtype, int split_k, cudaStream_t stream) {
    const GemmArgs& g = *args;
    if (g.M <= 0 || g.N <= 0) return GL_OK;
    if (g.M > 64 || g.K <= 0 || g.K % 8) return GL_ERR_SHAPE;
    if (((uintptr_t)g.a | (uintptr_t)g.w) & 15) return GL_ERR_ALIGN;
    if (g.a2) {
        if (!g.w2 || g.K2 <= 0 || g.K2 % 8 || g.K % GS_BK) return GL_ERR_SHAPE;     // a stage lies in one product
        if (((uintptr_t)g.a2 | (uintptr_t)g.w2) & 15) return GL_ERR_ALIGN;
    }
    int S = split_k;
    if (S == 0) {
        static int sms = 0;
        if (!sms) {
            int dev = 0;
            cudaGetDevice(&dev);
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
            if (sms <= 0) sms = 148;
        }
        // the number of parts that fills most of the resident slots (two an SM) in one wave, while
        // every part keeps at least four stages of K
        const int tiles = (g.N + GS_ROWS - 1) / GS_ROWS, slots = 2 * sms;
        const int chunks = (g.K + GS_BK - 1) / GS_BK + (g.a2 ? (g.K2 + GS_BK - 1) / GS_BK : 0);
        S = 1;
        for (int s = 2; s <= 16; ++s)
            if ((long long)tiles * s <= slots && chunks / s >= 4) S = s;
    }
    if (S < 1 || S > 16) return GL_ERR_SHAPE;
    if (out_dtype == GL_F32) return gs_dispatch<float>(g, S, stream);
    if (out_dtype == GL_BF16) return gs_dispatch<__nv_bfloat16>(g, S, stream);
    return GL_ERR_DTYPE;
}
