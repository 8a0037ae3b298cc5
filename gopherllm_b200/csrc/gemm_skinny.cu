// out[M,N] = act(A[M,K] · W[N,K]ᵀ + bias) + add0 + add1 for few rows (M <= 64), bfloat16.
//
// With few tokens a product is a stream of weights: every weight is read once
// and the machine is bound by HBM, so what counts is bytes in flight.  A block
// owns 64 weight rows and a range of K.  Weights and activations arrive in
// shared memory by TMA (cp.async.bulk.tensor, 64 k per stage, 128-byte swizzle so
// that ldmatrix reads without bank conflicts; one thread issues, an mbarrier per
// stage counts the bytes), several stages ahead, and the product is turned round
// for mma.sync.m16n8k16: the weight rows are the 16-row operand, the tokens the
// 8-column operand.  Rows and columns outside the matrices read as zero.
//
// To fill 148 SMs when N is small, K is cut over the blocks of a thread-block
// cluster; the partial tiles meet in distributed shared memory, each block
// reducing and finishing (bias, activation, residual adds) its share of the
// tile's columns in rank order, so the result does not depend on timing.
#include "common.cuh"
#include "tma.cuh"
#include <cooperative_groups.h>
namespace cg = cooperative_groups;

#define SK_ROWS 64          // weight rows per block
#define SK_BK 64            // k per pipeline stage (128 bytes per row)
#define SK_THREADS 128

struct GemmArgs {
    const void* a;        // [M, K] bf16
    const void* w;        // [N, K] bf16
    const float* bias;    // [N] or null
    const float* add0;    // [M, N] or null
    const float* add1;    // [M, N] or null
    void* out;            // [M, N] f32 or bf16
    int M, N, K, act;
    // a second product summed into the same output (out = act(a w^T + a2 w2^T + bias + bias2) + ...):
    // K is then the joined length K1 + K2, with K1 a multiple of the stage's 64
    const void* a2;       // [M, K2] bf16 or null
    const void* w2;       // [N, K2] bf16
    const float* bias2;   // [N] or null
    int K2;
};

__device__ __forceinline__ void ldmatrix_x4(unsigned addr, unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x2(unsigned addr, unsigned& r0, unsigned& r1) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// byte offset of 16-byte chunk c of row r in a tile of 128-byte rows
__device__ __forceinline__ int swz(int r, int c) { return r * 128 + ((c ^ (r & 7)) << 4); }

template <int MT, int STAGES, typename TO>
__global__ void __launch_bounds__(SK_THREADS)
gemm_skinny_kernel(GemmArgs g, int k_per_block, const __grid_constant__ CUtensorMap map_w,
                   const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w2,
                   const __grid_constant__ CUtensorMap map_a2) {
    extern __shared__ unsigned char smem_raw[];
    constexpr int W_BYTES = SK_ROWS * 128, A_BYTES = MT * 8 * 128, STAGE = W_BYTES + A_BYTES;
    constexpr int LD = SK_ROWS + 1;
    cg::cluster_group cluster = cg::this_cluster();
    const int S = (int)cluster.num_blocks(), rank = (int)cluster.block_rank();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.y * SK_ROWS;
    const int k1 = g.K, k_all = g.K + (g.a2 ? g.K2 : 0);       // the first product's K, the joined K
    const int kb = blockIdx.x * k_per_block;
    const int ke = min(k_all, kb + k_per_block);
    const int iters = ke > kb ? (ke - kb + SK_BK - 1) / SK_BK : 0;
    // stages start on a 1024-byte boundary (the swizzle pattern repeats every 8 rows of 128 bytes)
    unsigned char* smem = smem_raw + ((1024u - (gl_smem_u32(smem_raw) & 1023u)) & 1023u);
    const unsigned base = gl_smem_u32(smem);
    const unsigned bars = base + STAGES * STAGE;            // one 8-byte mbarrier per stage

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) mbar_init(bars + 8 * s, 1);
        mbar_fence_init();
    }
    __syncthreads();
    auto load_w = [&](int it) {                               // one thread: the stage's weights
        const unsigned sb = base + (it % STAGES) * STAGE, bar = bars + 8 * (it % STAGES);
        mbar_expect_tx(bar, STAGE);                           // the activations of the stage count too
        const int k = kb + it * SK_BK;
        if (k < k1) tma_load_2d(sb, &map_w, k, n0, bar);
        else tma_load_2d(sb, &map_w2, k - k1, n0, bar);
    };
    auto load_a = [&](int it) {                               // one thread: the stage's activations
        const unsigned sb = base + (it % STAGES) * STAGE, bar = bars + 8 * (it % STAGES);
        const int k = kb + it * SK_BK;
        if (k < k1) tma_load_2d(sb + W_BYTES, &map_a, k, 0, bar);
        else tma_load_2d(sb + W_BYTES, &map_a2, k - k1, 0, bar);
    };

    float acc[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[mt][e] = 0.f;

    // The weights do not depend on the kernel before this one: their first stages are under way
    // before this kernel waits for it.  The activations and everything written come after.
    gl_grid_launch_dependents();
    if (tid == 0)
        for (int s = 0; s < STAGES - 1 && s < iters; ++s) load_w(s);
    // What the epilogue adds is asked for now, not when the sums are ready: the biases (this thread
    // finishes elements of one column only, since the threads of a block are a multiple of the columns a
    // block finishes) before the wait, the residual values behind it.  In a decode step both are cold or
    // far, and their trip would otherwise follow the products instead of running under them.
    const int cnt = SK_ROWS / S;
    const int my_n = n0 + rank * cnt + tid % cnt;
    float my_bias = 0.f;
    if (my_n < g.N) {
        if (g.bias) my_bias = g.bias[my_n];
        if (g.bias2) my_bias += g.bias2[my_n];
    }
    gl_grid_wait();
    if (tid == 0)
        for (int s = 0; s < STAGES - 1 && s < iters; ++s) load_a(s);
    constexpr int EARLY = MT <= 2 ? MT * 4 : 1;               // elements a thread finishes at most (few rows only)
    float early0[EARLY], early1[EARLY];
    if constexpr (MT <= 2) {
#pragma unroll
        for (int e = 0; e < EARLY; ++e) {
            const int i = tid + e * SK_THREADS, m = i / cnt;
            const bool ok = i < MT * 8 * cnt && m < g.M && my_n < g.N;
            early0[e] = (ok && g.add0) ? g.add0[(size_t)m * g.N + my_n] : 0.f;
            early1[e] = (ok && g.add1) ? g.add1[(size_t)m * g.N + my_n] : 0.f;
        }
    }
    for (int it = 0; it < iters; ++it) {
        if (!mbar_wait(bars + 8 * (it % STAGES), (it / STAGES) & 1)) break;
        __syncthreads();                                      // everyone is done with the stage refilled next
        if (tid == 0 && it + STAGES - 1 < iters) { load_w(it + STAGES - 1); load_a(it + STAGES - 1); }
        const unsigned sb = base + (it % STAGES) * STAGE;
        // a stage's fragments are asked for ahead of the products that need them (the weights' for the
        // whole stage, the tokens' for a k-step at a time): a warp that loaded and multiplied in turn
        // would wait out a shared-memory round trip before every product
        unsigned af[SK_BK / 16][4];
#pragma unroll
        for (int kk = 0; kk < SK_BK / 16; ++kk) {
            const int r = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
            const int c = kk * 2 + (lane >> 4);
            ldmatrix_x4(sb + swz(r, c), af[kk][0], af[kk][1], af[kk][2], af[kk][3]);
        }
#pragma unroll
        for (int kk = 0; kk < SK_BK / 16; ++kk) {
            unsigned bf[MT][2];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                const int r = mt * 8 + (lane & 7);
                const int c = kk * 2 + ((lane >> 3) & 1);
                ldmatrix_x2(sb + W_BYTES + swz(r, c), bf[mt][0], bf[mt][1]);
            }
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
                mma_bf16(acc[mt], af[kk][0], af[kk][1], af[kk][2], af[kk][3], bf[mt][0], bf[mt][1]);
        }
    }
    __syncthreads();
    // partial tile to shared memory (the pipeline's buffers are free now): tile[m][n_local]
    float* tile = (float*)smem;
    {
        const int grp = lane >> 2, t = lane & 3;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            const int m = mt * 8 + 2 * t, nl = warp * 16 + grp;
            tile[m * LD + nl] = acc[mt][0];
            tile[(m + 1) * LD + nl] = acc[mt][1];
            tile[m * LD + nl + 8] = acc[mt][2];
            tile[(m + 1) * LD + nl + 8] = acc[mt][3];
        }
    }
    cluster.sync();
    // this block finishes columns [rank*cnt, (rank+1)*cnt) of the tile, summing the blocks in rank order
    TO* O = (TO*)g.out;
    const int nl = my_n - n0;
#pragma unroll 1
    for (int e = 0; e * SK_THREADS + tid < MT * 8 * cnt; ++e) {
        const int m = (tid + e * SK_THREADS) / cnt;
        if (m >= g.M || my_n >= g.N) continue;
        float v = 0.f;
        for (int s = 0; s < S; ++s) {
            const float* peer = cluster.map_shared_rank(tile, s);
            v += peer[m * LD + nl];
        }
        v = gl_activate<false>(v + my_bias, g.act);
        const size_t o = (size_t)m * g.N + my_n;
        if constexpr (MT <= 2) {
            // (indexed with a compile-time number below: the array stays in registers)
            float a0 = 0.f, a1 = 0.f;
#pragma unroll
            for (int q = 0; q < EARLY; ++q)
                if (q == e) { a0 = early0[q]; a1 = early1[q]; }
            v = (v + a0) + a1;
        } else {
            if (g.add0) v += g.add0[o];
            if (g.add1) v += g.add1[o];
        }
        gl_store(O + o, v);
    }
    cluster.sync();       // nobody leaves while a peer may still read its tile
}

template <int MT, int STAGES>
static constexpr size_t skinny_smem() {
    // stages + barriers + room to align the start; the reduction tile reuses the stages
    return (size_t)STAGES * (SK_ROWS * 128 + MT * 8 * 128) + 8 * STAGES + 1024;
}
static_assert(4 * (SK_ROWS * 128 + 8 * 8 * 128) >= 8 * 8 * (SK_ROWS + 1) * 4, "reduction tile fits the stages");

template <int MT, int STAGES, typename TO>
static int launch_skinny(const GemmArgs& g, int S, cudaStream_t stream) {
    constexpr size_t smem = skinny_smem<MT, STAGES>();
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(gemm_skinny_kernel<MT, STAGES, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem) != cudaSuccess) {
            cudaGetLastError();
            return GL_ERR_SMEM;
        }
        configured = true;
    }
    const int k_all = g.K + (g.a2 ? g.K2 : 0);
    const int k_per_block = ((k_all + S - 1) / S + SK_BK - 1) / SK_BK * SK_BK;
    CUtensorMap map_w, map_a;
    int rc = gl_cached_map_bf16(&map_w, g.w, (uint64_t)g.N, (uint64_t)g.K, SK_ROWS, SK_BK);
    if (rc != GL_OK) return rc;
    rc = gl_cached_map_bf16(&map_a, g.a, (uint64_t)g.M, (uint64_t)g.K, MT * 8, SK_BK);
    if (rc != GL_OK) return rc;
    CUtensorMap map_w2 = map_w, map_a2 = map_a;
    if (g.a2) {
        rc = gl_cached_map_bf16(&map_w2, g.w2, (uint64_t)g.N, (uint64_t)g.K2, SK_ROWS, SK_BK);
        if (rc != GL_OK) return rc;
        rc = gl_cached_map_bf16(&map_a2, g.a2, (uint64_t)g.M, (uint64_t)g.K2, MT * 8, SK_BK);
        if (rc != GL_OK) return rc;
    }
    const dim3 grid(S, (g.N + SK_ROWS - 1) / SK_ROWS, 1);
    if (grid.y > 65535) return GL_ERR_SHAPE;
    if (gl_launch(gemm_skinny_kernel<MT, STAGES, TO>, grid, dim3(SK_THREADS), smem, stream, S, g, k_per_block, map_w, map_a, map_w2, map_a2) != 0)
        return GL_ERR_LAUNCH;
    return GL_OK;
}

// blocks of one SM that fit by shared memory, for each M bucket
static int blocks_per_sm(int M) {
    const size_t smem = M <= 8 ? skinny_smem<1, 6>() : M <= 16 ? skinny_smem<2, 6>()
                      : M <= 32 ? skinny_smem<4, 5>() : skinny_smem<8, 4>();
    const int n = (int)((227 * 1024) / (smem + 1024));
    return n < 1 ? 1 : (n > 8 ? 8 : n);
}

template <typename TO>
static int dispatch_m(const GemmArgs& g, int S, cudaStream_t stream) {
    if (g.M <= 8) return launch_skinny<1, 6, TO>(g, S, stream);
    if (g.M <= 16) return launch_skinny<2, 6, TO>(g, S, stream);
    if (g.M <= 32) return launch_skinny<4, 5, TO>(g, S, stream);
    return launch_skinny<8, 4, TO>(g, S, stream);
}

// 1 if a bounded wait of this library ever ran out (the result of that launch is invalid)
GL_API int gl_gemm_skinny_wait_failed() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, gl_wait_failed, sizeof(int)) != cudaSuccess) return -1;
    return v;
}

// split_k: 0 lets the launcher choose; else 1, 2, 4 or 8 blocks of a cluster share K
GL_API int gl_gemm_skinny(const GemmArgs* args, int out_dtype, int split_k, cudaStream_t stream) {
    const GemmArgs& g = *args;
    if (g.M <= 0 || g.N <= 0) return GL_OK;
    if (g.M > 64 || g.K <= 0 || g.K % 8) return GL_ERR_SHAPE;
    if (((uintptr_t)g.a | (uintptr_t)g.w) & 15) return GL_ERR_ALIGN;
    if (g.a2) {
        if (!g.w2 || g.K2 <= 0 || g.K2 % 8 || g.K % SK_BK) return GL_ERR_SHAPE;    // a stage lies in one product
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
        // as many blocks as are resident at once, while every block keeps a few stages of K
        const int tiles = (g.N + SK_ROWS - 1) / SK_ROWS;
        const int slots = sms * blocks_per_sm(g.M);
        S = 1;
        const int k_all = g.K + (g.a2 ? g.K2 : 0);
        while (S < 8 && tiles * S * 2 <= slots && k_all / (S * 2) >= 4 * SK_BK) S *= 2;
    }
    if (S != 1 && S != 2 && S != 4 && S != 8) return GL_ERR_SHAPE;
    if (out_dtype == GL_F32) return dispatch_m<float>(g, S, stream);
    if (out_dtype == GL_BF16) return dispatch_m<__nv_bfloat16>(g, S, stream);
    return GL_ERR_DTYPE;
}
