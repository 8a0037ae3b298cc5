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
    gl_grid_launch_dependents();
    gl_grid_wait();
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
        return gl_launch(embed_kernel<float>, dim3(T), dim3(threads), 0, stream, 1, (const float*)table, tokens, out, D, V, scale);
    if (table_dtype == GL_BF16)
        return gl_launch(embed_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, 1,
                         (const __nv_bfloat16*)table, tokens, out, D, V, scale);
    return GL_ERR_DTYPE;
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

// NV: values of the row each thread keeps in registers (the row is read once when it fits)
template <typename TO, int NV>
__global__ void norm_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                            const float* __restrict__ gamma, const float* __restrict__ beta,
                            TO* __restrict__ out, int D, float eps, int rms) {
    __shared__ float red[32];
    __shared__ float s_inv;
    const int r = blockIdx.x;
    gl_grid_launch_dependents();
    gl_grid_wait();
    const float* xr = x + (size_t)(rows ? rows[r] : r) * D;
    TO* o = out + (size_t)r * D;
    float v[NV > 0 ? NV : 1];
    if (NV > 0) {
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int d = threadIdx.x + i * blockDim.x;
            v[i] = d < D ? xr[d] : 0.f;
        }
    }
    float mean = 0.f;
    if (!rms) {
        float s = 0.f;
        if (NV > 0) {
#pragma unroll
            for (int i = 0; i < NV; ++i) s += v[i];
        } else {
            for (int d = threadIdx.x; d < D; d += blockDim.x) s += xr[d];
        }
        mean = block_sum(s, red) / (float)D;
    }
    float q = 0.f;
    if (NV > 0) {
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const float c = (threadIdx.x + i * blockDim.x < D) ? v[i] - mean : 0.f;
            q += c * c;
        }
    } else {
        for (int d = threadIdx.x; d < D; d += blockDim.x) { const float c = xr[d] - mean; q += c * c; }
    }
    const float var = block_sum(q, red) / (float)D;
    // one thread takes the reciprocal square root in 64-bit, as the reference does (bert.go:764)
    if (threadIdx.x == 0) s_inv = (float)(1.0 / sqrt((double)(var + eps)));
    __syncthreads();
    const float inv = s_inv;
    if (NV > 0) {
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int d = threadIdx.x + i * blockDim.x;
            if (d < D) {
                float y = (v[i] - mean) * inv * gamma[d];
                if (beta) y += beta[d];
                gl_store(o + d, y);
            }
        }
    } else {
        for (int d = threadIdx.x; d < D; d += blockDim.x) {
            float y = (xr[d] - mean) * inv * gamma[d];
            if (beta) y += beta[d];
            gl_store(o + d, y);
        }
    }
}

template <typename TO>
static int launch_norm(const float* x, const int* rows, const float* gamma, const float* beta, TO* out,
                       int R, int D, float eps, int rms, cudaStream_t stream) {
    const int threads = D >= 2048 ? 512 : (D >= 512 ? 256 : 128);
    const int per = (D + threads - 1) / threads;
    if (per <= 2) return gl_launch(norm_kernel<TO, 2>, dim3(R), dim3(threads), 0, stream, 1, x, rows, gamma, beta, out, D, eps, rms);
    if (per <= 4) return gl_launch(norm_kernel<TO, 4>, dim3(R), dim3(threads), 0, stream, 1, x, rows, gamma, beta, out, D, eps, rms);
    if (per <= 8) return gl_launch(norm_kernel<TO, 8>, dim3(R), dim3(threads), 0, stream, 1, x, rows, gamma, beta, out, D, eps, rms);
    if (per <= 16) return gl_launch(norm_kernel<TO, 16>, dim3(R), dim3(threads), 0, stream, 1, x, rows, gamma, beta, out, D, eps, rms);
    return gl_launch(norm_kernel<TO, 0>, dim3(R), dim3(threads), 0, stream, 1, x, rows, gamma, beta, out, D, eps, rms);
}

GL_API int gl_norm(const float* x, const int* rows, const float* gamma, const float* beta,
                   void* out, int out_dtype, int R, int D, float eps, int rms,
                   cudaStream_t stream) {
    if (R <= 0) return GL_OK;
    if (D <= 0) return GL_ERR_SHAPE;
    if (out_dtype == GL_F32) return launch_norm<float>(x, rows, gamma, beta, (float*)out, R, D, eps, rms, stream);
    if (out_dtype == GL_BF16) return launch_norm<__nv_bfloat16>(x, rows, gamma, beta, (__nv_bfloat16*)out, R, D, eps, rms, stream);
    return GL_ERR_DTYPE;
}

// ---------------------------------------------------------------------------
// Feeding a decode step's choices back on the device: the sampled token becomes
// the next input, positions and cached lengths move on by one, and the choice is
// appended to a history so that several steps can run without the host.
// ---------------------------------------------------------------------------
__global__ void advance_kernel(int* tokens, int* tok_pos, int* seq_ctx, const int* sampled,
                               int* history, int* counter, int B, int max_steps) {
    const int b = threadIdx.x;
    gl_grid_launch_dependents();
    gl_grid_wait();
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
    return gl_launch(advance_kernel, dim3(1), dim3(((B + 31) / 32) * 32), 0, stream, 1, tokens, tok_pos, seq_ctx, sampled,
                     history, counter, B, max_steps);
}
