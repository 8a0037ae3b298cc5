// out[M,N] = act(A[M,K] · W[N,K]ᵀ + bias[N]) + add0[M,N] + add1[M,N]
//
// The plain matrix product: 32-bit FMA on CUDA cores, every element type, every
// size.  It is the whole 32-bit path (no tensor-core mode of reduced precision
// is ever used there) and the product every faster kernel is checked against.
// Each output element sums over k in ascending order whatever M, N or the tile
// it falls in, so a row's result does not depend on what else is in the batch
// (the reference's product is a per-row dot, simd.go:188-196).
#include "common.cuh"

#define SG_BM 64
#define SG_BN 64
#define SG_BK 16

struct GemmArgs {
    const void* a;        // [M, K]
    const void* w;        // [N, K]
    const float* bias;    // [N] or null
    const float* add0;    // [M, N] or null, 32-bit
    const float* add1;    // [M, N] or null, 32-bit
    void* out;            // [M, N]
    int M, N, K, act;
};

template <typename TA, typename TW, typename TO>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(GemmArgs g) {
    __shared__ float As[SG_BK][SG_BM + 4];
    __shared__ float Ws[SG_BK][SG_BN + 4];
    const TA* A = (const TA*)g.a;
    const TW* W = (const TW*)g.w;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * SG_BM, n0 = blockIdx.x * SG_BN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < g.K; k0 += SG_BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int e = tid + i * 256, r = e >> 4, c = e & 15;
            const int k = k0 + c;
            float va = 0.f, vw = 0.f;
            if (k < g.K) {
                if (m0 + r < g.M) va = gl_load(A + (size_t)(m0 + r) * g.K + k);
                if (n0 + r < g.N) vw = gl_load(W + (size_t)(n0 + r) * g.K + k);
            }
            As[c][r] = va;
            Ws[c][r] = vw;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < SG_BK; ++kk) {
            float av[4], wv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) av[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) wv[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
    TO* O = (TO*)g.out;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= g.M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= g.N) continue;
            float v = acc[i][j];
            if (g.bias) v += g.bias[n];
            v = gl_activate<true>(v, g.act);
            const size_t o = (size_t)m * g.N + n;
            if (g.add0) v += g.add0[o];
            if (g.add1) v += g.add1[o];
            gl_store(O + o, v);
        }
    }
}

template <typename TA, typename TW, typename TO>
static int launch_simt(const GemmArgs& g, cudaStream_t stream) {
    dim3 grid((g.N + SG_BN - 1) / SG_BN, (g.M + SG_BM - 1) / SG_BM);
    if (grid.y > 65535) return GL_ERR_SHAPE;
    gemm_simt_kernel<TA, TW, TO><<<grid, 256, 0, stream>>>(g);
    return gl_check_launch();
}

template <typename TA, typename TW>
static int dispatch_out(const GemmArgs& g, int out_dtype, cudaStream_t stream) {
    if (out_dtype == GL_F32) return launch_simt<TA, TW, float>(g, stream);
    if (out_dtype == GL_BF16) return launch_simt<TA, TW, __nv_bfloat16>(g, stream);
    return GL_ERR_DTYPE;
}

GL_API int gl_gemm_simt(const GemmArgs* args, int a_dtype, int w_dtype, int out_dtype, cudaStream_t stream) {
    const GemmArgs& g = *args;
    if (g.M <= 0 || g.N <= 0) return GL_OK;
    if (g.K <= 0) return GL_ERR_SHAPE;
    if (a_dtype == GL_F32 && w_dtype == GL_F32) return dispatch_out<float, float>(g, out_dtype, stream);
    if (a_dtype == GL_BF16 && w_dtype == GL_BF16) return dispatch_out<__nv_bfloat16, __nv_bfloat16>(g, out_dtype, stream);
    if (a_dtype == GL_BF16 && w_dtype == GL_F32) return dispatch_out<__nv_bfloat16, float>(g, out_dtype, stream);
    if (a_dtype == GL_F32 && w_dtype == GL_BF16) return dispatch_out<float, __nv_bfloat16>(g, out_dtype, stream);
    return GL_ERR_DTYPE;
}
