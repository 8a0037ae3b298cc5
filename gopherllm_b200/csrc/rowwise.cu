// Row-wise kernels: embedding gather and normalisation.
//
// The residual stream is 32-bit in every mode; the norm writes the activation
// type of the mode (32-bit or bfloat16) that the matrix products read.
#include "common.cuh"

// ---------------------------------------------------------------------------
// Embedding: out[t, :] = scale * table[tokens[t], :]          (model.go:2642-2651)
// ---------------------------------------------------------------------------
template <typename TW>
__global__ void embed_kernel(const TW* __restrict__ table, const int* __restrict__ tokens,
                             float* __restrict__ out, int D, int V, float scale) {
    const int t = blockIdx.x;
    int tok = tokens[t];
    // ids are checked on the host; a bad id must still not read outside the table
    tok = tok < 0 ? 0 : (tok >= V ? V - 1 : tok);
    const TW* row = table + (size_t)tok * D;
    float* o = out + (size_t)t * D;
    for (int d = threadIdx.x; d < D; d += blockDim.x) o[d] = gl_load(row + d) * scale;
}

GL_API int gl_embed(const void* table, int table_dtype, const int* tokens, float* out,
                    int T, int D, int V, float scale, cudaStream_t stream) {
    if (T <= 0) return GL_OK;
    if (D <= 0 || V <= 0) return GL_ERR_SHAPE;
    const int threads = D >= 1024 ? 256 : 128;
    if (table_dtype == GL_F32)
        embed_kernel<float><<<T, threads, 0, stream>>>((const float*)table, tokens, out, D, V, scale);
    else if (table_dtype == GL_BF16)
        embed_kernel<__nv_bfloat16><<<T, threads, 0, stream>>>((const __nv_bfloat16*)table, tokens, out, D, V, scale);
    else
        return GL_ERR_DTYPE;
    return gl_check_launch();
}

// ---------------------------------------------------------------------------
// Normalisation of selected rows of a 32-bit matrix.
//   layernorm: mean, biased variance over the row, y = (x-mean)*rsqrt(var+eps)*g + b
//              (bert.go:748-776; the reference takes 1/sqrt in 64-bit, so does this)
//   rmsnorm:   y = x * rsqrt(mean(x^2)+eps) * g            (model.go:2949-2981)
// rows == nullptr: row r of the output comes from row r of x; else from x[rows[r]].
// ---------------------------------------------------------------------------
__device__ __forceinline__ float block_sum(float v, float* red) {
    v = gl_warp_sum(v);
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
    __syncthreads();
    if (lane == 0) red[w] = v;
    __syncthreads();
    float s = 0.f;
    for (int i = 0; i < nw; ++i) s += red[i];   // same order in every thread
    return s;
}

template <typename TO>
__global__ void norm_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                            const float* __restrict__ gamma, const float* __restrict__ beta,
                            TO* __restrict__ out, int D, float eps, int rms) {
    __shared__ float red[32];
    const int r = blockIdx.x;
    const float* xr = x + (size_t)(rows ? rows[r] : r) * D;
    TO* o = out + (size_t)r * D;
    float mean = 0.f;
    if (!rms) {
        float s = 0.f;
        for (int d = threadIdx.x; d < D; d += blockDim.x) s += xr[d];
        mean = block_sum(s, red) / (float)D;
    }
    float q = 0.f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        const float c = xr[d] - mean;
        q += c * c;
    }
    const float var = block_sum(q, red) / (float)D;
    const float inv = (float)(1.0 / sqrt((double)(var + eps)));
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float y = (xr[d] - mean) * inv * gamma[d];
        if (beta) y += beta[d];
        gl_store(o + d, y);
    }
}

GL_API int gl_norm(const float* x, const int* rows, const float* gamma, const float* beta,
                   void* out, int out_dtype, int R, int D, float eps, int rms,
                   cudaStream_t stream) {
    if (R <= 0) return GL_OK;
    if (D <= 0) return GL_ERR_SHAPE;
    const int threads = D >= 2048 ? 512 : (D >= 512 ? 256 : 128);
    if (out_dtype == GL_F32)
        norm_kernel<float><<<R, threads, 0, stream>>>(x, rows, gamma, beta, (float*)out, D, eps, rms);
    else if (out_dtype == GL_BF16)
        norm_kernel<__nv_bfloat16><<<R, threads, 0, stream>>>(x, rows, gamma, beta, (__nv_bfloat16*)out, D, eps, rms);
    else
        return GL_ERR_DTYPE;
    return gl_check_launch();
}

// ---------------------------------------------------------------------------
// Feeding a decode step's choices back on the device: the sampled token becomes
// the next input, positions and cached lengths move on by one, and the choice is
// appended to a history so that several steps can run without the host.
// ---------------------------------------------------------------------------
__global__ void advance_kernel(int* tokens, int* tok_pos, int* seq_ctx, const int* sampled,
                               int* history, int* counter, int B, int max_steps) {
    const int b = threadIdx.x;
    const int i = counter[0];
    if (b < B) {
        const int t = sampled[b];
        if (i < max_steps) history[(size_t)i * B + b] = t;
        tokens[b] = t;
        tok_pos[b] += 1;
        seq_ctx[b] += 1;
    }
    __syncthreads();
    if (b == 0) counter[0] = i + 1;
}

GL_API int gl_advance_decode(int* tokens, int* tok_pos, int* seq_ctx, const int* sampled,
                             int* history, int* counter, int B, int max_steps, cudaStream_t stream) {
    if (B <= 0) return GL_OK;
    if (B > 1024) return GL_ERR_SHAPE;
    advance_kernel<<<1, ((B + 31) / 32) * 32, 0, stream>>>(tokens, tok_pos, seq_ctx, sampled, history, counter, B, max_steps);
    return gl_check_launch();
}
