// out[M,N] = act(A[M,K] · W[N,K]ᵀ + bias) + add0 + add1 for few rows (M <= 64), bfloat16.
//
// With few tokens a product is a stream of weights: every weight is read once
// and the machine is bound by HBM.  The kernel therefore turns the product
// round: the weight rows are the 16-row operand of mma.sync.m16n8k16 and the
// tokens the 8-column operand, and each thread fetches its fragments straight
// from global memory with 16-byte loads (8 consecutive k for one row).  Because
// both operands are indexed by the same k, taking the same 8 consecutive k for
// slots {2t,2t+1,2t+8,2t+9} of two successive MMAs in both operands is only a
// renaming of k and leaves the sum unchanged.
//
// A block is 4 warps x 16 weight rows.  To fill 148 SMs when N is small, K is cut
// over the blocks of a thread-block cluster; the partial tiles meet in
// distributed shared memory, each block reducing and finishing (bias,
// activation, residual adds) its share of the tile's columns in a fixed order,
// so the result does not depend on timing.
#include "common.cuh"
#include <cooperative_groups.h>
namespace cg = cooperative_groups;

#define SK_ROWS 64          // weight rows per block
#define SK_THREADS 128
#define SK_UNROLL 4         // k-steps of 32 whose weight loads are issued together

struct GemmArgs {
    const void* a;        // [M, K] bf16
    const void* w;        // [N, K] bf16
    const float* bias;    // [N] or null
    const float* add0;    // [M, N] or null
    const float* add1;    // [M, N] or null
    void* out;            // [M, N] f32 or bf16
    int M, N, K, act;
};

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ void mma_bf16(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int MT, typename TO>
__global__ void __launch_bounds__(SK_THREADS)
gemm_skinny_kernel(GemmArgs g, int k_per_block) {
    extern __shared__ float tile[];                       // [MT*8][SK_ROWS + 1]
    constexpr int LD = SK_ROWS + 1;
    cg::cluster_group cluster = cg::this_cluster();
    const int S = (int)cluster.num_blocks();
    const int rank = (int)cluster.block_rank();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int grp = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.y * SK_ROWS;
    const int kb = blockIdx.x * k_per_block;
    const int ke = min(g.K, kb + k_per_block);
    const __nv_bfloat16* W = (const __nv_bfloat16*)g.w;
    const __nv_bfloat16* A = (const __nv_bfloat16*)g.a;
    const int r0 = min(n0 + warp * 16 + grp, g.N - 1), r1 = min(n0 + warp * 16 + grp + 8, g.N - 1);
    const __nv_bfloat16* w0 = W + (size_t)r0 * g.K;
    const __nv_bfloat16* w1 = W + (size_t)r1 * g.K;
    const __nv_bfloat16* arow[MT];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) arow[mt] = A + (size_t)min(mt * 8 + grp, g.M - 1) * g.K;

    float acc[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[mt][e] = 0.f;

    const uint4 zero = make_uint4(0, 0, 0, 0);
    for (int k0 = kb; k0 < ke; k0 += 32 * SK_UNROLL) {
        uint4 wa[SK_UNROLL], wb[SK_UNROLL];
#pragma unroll
        for (int u = 0; u < SK_UNROLL; ++u) {
            const int kk = k0 + 32 * u + 8 * t;
            const bool ok = kk < ke;
            wa[u] = ok ? ldg_stream(w0 + kk) : zero;
            wb[u] = ok ? ldg_stream(w1 + kk) : zero;
        }
#pragma unroll
        for (int u = 0; u < SK_UNROLL; ++u) {
            const int kk = k0 + 32 * u + 8 * t;
            const bool ok = kk < ke;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                const uint4 x = ok ? *(const uint4*)(arow[mt] + kk) : zero;
                mma_bf16(acc[mt], wa[u].x, wb[u].x, wa[u].y, wb[u].y, x.x, x.y);
                mma_bf16(acc[mt], wa[u].z, wb[u].z, wa[u].w, wb[u].w, x.z, x.w);
            }
        }
    }
    // partial tile to shared memory: tile[m][n_local]
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        const int m = mt * 8 + 2 * t, nl = warp * 16 + grp;
        tile[m * LD + nl] = acc[mt][0];
        tile[(m + 1) * LD + nl] = acc[mt][1];
        tile[m * LD + nl + 8] = acc[mt][2];
        tile[(m + 1) * LD + nl + 8] = acc[mt][3];
    }
    cluster.sync();
    // this block finishes columns [rank*cnt, (rank+1)*cnt) of the tile, summing the blocks in rank order
    const int cnt = SK_ROWS / S;
    TO* O = (TO*)g.out;
    for (int i = threadIdx.x; i < MT * 8 * cnt; i += SK_THREADS) {
        const int m = i / cnt, nl = rank * cnt + (i - m * cnt);
        const int n = n0 + nl;
        if (m >= g.M || n >= g.N) continue;
        float v = 0.f;
        for (int s = 0; s < S; ++s) {
            const float* peer = cluster.map_shared_rank(tile, s);
            v += peer[m * LD + nl];
        }
        if (g.bias) v += g.bias[n];
        v = gl_activate<false>(v, g.act);
        const size_t o = (size_t)m * g.N + n;
        if (g.add0) v += g.add0[o];
        if (g.add1) v += g.add1[o];
        gl_store(O + o, v);
    }
    cluster.sync();       // nobody leaves while a peer may still read its tile
}

template <int MT, typename TO>
static int launch_skinny(const GemmArgs& g, int S, cudaStream_t stream) {
    const int k_per_block = ((g.K + S - 1) / S + 31) / 32 * 32;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(S, (g.N + SK_ROWS - 1) / SK_ROWS, 1);
    cfg.blockDim = dim3(SK_THREADS, 1, 1);
    cfg.dynamicSmemBytes = (size_t)MT * 8 * (SK_ROWS + 1) * sizeof(float);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = S;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cfg.gridDim.y > 65535) return GL_ERR_SHAPE;
    if (cudaLaunchKernelEx(&cfg, gemm_skinny_kernel<MT, TO>, g, k_per_block) != cudaSuccess) {
        cudaGetLastError();
        return GL_ERR_LAUNCH;
    }
    return GL_OK;
}

template <typename TO>
static int dispatch_m(const GemmArgs& g, int S, cudaStream_t stream) {
    if (g.M <= 8) return launch_skinny<1, TO>(g, S, stream);
    if (g.M <= 16) return launch_skinny<2, TO>(g, S, stream);
    if (g.M <= 32) return launch_skinny<4, TO>(g, S, stream);
    return launch_skinny<8, TO>(g, S, stream);
}

// split_k: 0 lets the launcher choose; else 1, 2, 4 or 8 blocks of a cluster share K
GL_API int gl_gemm_skinny(const GemmArgs* args, int out_dtype, int split_k, cudaStream_t stream) {
    const GemmArgs& g = *args;
    if (g.M <= 0 || g.N <= 0) return GL_OK;
    if (g.M > 64 || g.K <= 0 || g.K % 8) return GL_ERR_SHAPE;
    if (((uintptr_t)g.a | (uintptr_t)g.w) & 15) return GL_ERR_ALIGN;
    int S = split_k;
    if (S == 0) {
        const int tiles = (g.N + SK_ROWS - 1) / SK_ROWS;
        S = 1;
        while (S < 8 && tiles * S * 4 < 2400 && g.K / (S * 2) >= 256) S *= 2;
    }
    if (S != 1 && S != 2 && S != 4 && S != 8) return GL_ERR_SHAPE;
    if (out_dtype == GL_F32) return dispatch_m<float>(g, S, stream);
    if (out_dtype == GL_BF16) return dispatch_m<__nv_bfloat16>(g, S, stream);
    return GL_ERR_DTYPE;
}
