// Row-wise kernels: embedding gather and normalisation.
//
// The residual stream is 32-bit in every mode; the norm writes the activation
// type of the mode (32-bit or bfloat16) that the matrix products read.
#include "common.cuh"

// ---------------------------------------------------------------------------
// Embedding: out[t, :] = scale * table[tokens[t], :]          (model.go:2642-2651)
// ---------------------------------------------------------------------------
// (tokens, index, x below: what an earlier kernel of the step wrote is not declared restrict: loads through a
// const restrict pointer count as loads of memory nobody writes, which the compiler may move above the wait)
template <typename TW>
__global__ void embed_kernel(const TW* __restrict__ table, const int* tokens,
                             float* __restrict__ out, int D, int V, float scale) {
    const int t = blockIdx.x;
    gl_grid_launch_dependents();
    gl_grid_wait();
    int tok = gl_checked(tokens[t], V, GL_BAD_TOKEN);
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
// A second table added onto the residual stream: out[t, :] += table[index[t], :].  Learned
// absolute positions are added once, before the first layer (model.go:2648-2651).
// ---------------------------------------------------------------------------
template <typename TW>
__global__ void add_rows_kernel(const TW* __restrict__ table, const int* index,
                                float* __restrict__ out, int D, int N) {
    const int t = blockIdx.x;
    gl_grid_launch_dependents();
    gl_grid_wait();
    int i = gl_checked(index[t], N, GL_BAD_ROW);
    i = i < 0 ? 0 : (i >= N ? N - 1 : i);        // checked on the host; never read outside the table
    const TW* row = table + (size_t)i * D;
    float* o = out + (size_t)t * D;
    for (int d = threadIdx.x; d < D; d += blockDim.x) o[d] += gl_load(row + d);
}

GL_API int gl_add_rows(const void* table, int table_dtype, const int* index, float* out,
                       int T, int D, int N, cudaStream_t stream) {
    if (T <= 0) return GL_OK;
    if (D <= 0 || N <= 0) return GL_ERR_SHAPE;
    const int threads = D >= 1024 ? 256 : 128;
    if (table_dtype == GL_F32)
        return gl_launch(add_rows_kernel<float>, dim3(T), dim3(threads), 0, stream, 1, (const float*)table, index, out, D, N);
    if (table_dtype == GL_BF16)
        return gl_launch(add_rows_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, 1,
                         (const __nv_bfloat16*)table, index, out, D, N);
    return GL_ERR_DTYPE;
}

// ---------------------------------------------------------------------------
// Logits in place: x <- x * scale, then x <- cap * tanh(x / cap) if cap > 0 (the reference's
// LogitScale and final soft cap, model.go:2555-2564).  32-bit throughout.
// ---------------------------------------------------------------------------
__global__ void scale_softcap_kernel(float* __restrict__ x, size_t n, float scale, float cap) {
    gl_grid_launch_dependents();
    gl_grid_wait();
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        float v = x[i] * scale;
        if (cap > 0.f) v = cap * tanhf(v / cap);
        x[i] = v;
    }
}

GL_API int gl_scale_softcap(float* x, long long n, float scale, float cap, cudaStream_t stream) {
    if (n <= 0) return GL_OK;
    const int threads = 256;
    const long long want = (n + threads - 1) / threads;
    const int blocks = (int)(want > 4096 ? 4096 : want);
    return gl_launch(scale_softcap_kernel, dim3(blocks), dim3(threads), 0, stream, 1, x, (size_t)n, scale, cap);
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
__global__ void norm_kernel(const float* x, const int* __restrict__ rows,
                            const float* __restrict__ gamma, const float* __restrict__ beta,
                            TO* __restrict__ out, int D, float eps, int rms) {
    __shared__ float red[32];
    __shared__ float s_inv;
    const int r = blockIdx.x;
    gl_grid_launch_dependents();
    // The norm's own vectors do not depend on the kernel before this one: they are asked for before this
    // kernel waits for it.  In a decode step they are cold (a layer's vectors are read once a step, with
    // gigabytes in between), and fetched at the end their trip to memory would stand between two products.
    float gv[NV > 0 ? NV : 1], bv[NV > 0 ? NV : 1];
    if (NV > 0) {
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int d = threadIdx.x + i * blockDim.x;
            gv[i] = d < D ? gamma[d] : 0.f;
            bv[i] = (d < D && beta) ? beta[d] : 0.f;
        }
    }
    gl_grid_wait();
    // (x is what the kernel before this one wrote: it is read with loads that the compiler may not move
    // above the wait.  Declared const and restrict, a pointer's loads count as loads of memory that nobody
    // writes, and those may be issued together with the loads above.)
    const float* xr = x + (size_t)(rows ? rows[r] : r) * D;
    TO* o = out + (size_t)r * D;
    float v[NV > 0 ? NV : 1];
    if (NV > 0) {
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int d = threadIdx.x + i * blockDim.x;
            v[i] = d < D ? __ldcg(xr + d) : 0.f;
        }
    }
    float mean = 0.f;
    if (!rms) {
        float s = 0.f;
        if (NV > 0) {
#pragma unroll
            for (int i = 0; i < NV; ++i) s += v[i];
        } else {
            for (int d = threadIdx.x; d < D; d += blockDim.x) s += __ldcg(xr + d);
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
        for (int d = threadIdx.x; d < D; d += blockDim.x) { const float c = __ldcg(xr + d) - mean; q += c * c; }
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
            if (d < D) gl_store(o + d, (v[i] - mean) * inv * gv[i] + bv[i]);
        }
    } else {
        for (int d = threadIdx.x; d < D; d += blockDim.x) {
            float y = (__ldcg(xr + d) - mean) * inv * gamma[d];
            if (beta) y += beta[d];
            gl_store(o + d, y);
        }
    }
}

// One warp per row, for many rows: the row lives in registers as NV4 float4 per lane, the
// statistics need warp shuffles only, loads and stores are 16 bytes (D a multiple of 4).
template <typename TO, int NV4>
__global__ void __launch_bounds__(256)
norm_warp_kernel(const float* x, const int* __restrict__ rows, const float* __restrict__ gamma,
                 const float* __restrict__ beta, TO* __restrict__ out, int R, int D, float eps, int rms) {
    gl_grid_launch_dependents();
    gl_grid_wait();
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= R) return;
    const float4* xr = (const float4*)(x + (size_t)(rows ? rows[r] : r) * D);
    const int n4 = D >> 2;
    float4 v[NV4];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < NV4; ++i) {
        const int k = lane + 32 * i;
        v[i] = k < n4 ? xr[k] : make_float4(0.f, 0.f, 0.f, 0.f);
        s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    }
    const float mean = rms ? 0.f : gl_warp_sum(s) / (float)D;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < NV4; ++i) {
        if (lane + 32 * i < n4) {
            const float a = v[i].x - mean, b = v[i].y - mean, c = v[i].z - mean, d = v[i].w - mean;
            q += (a * a + b * b) + (c * c + d * d);
        }
    }
    const float var = gl_warp_sum(q) / (float)D;
    float inv = 0.f;
    if (lane == 0) inv = (float)(1.0 / sqrt((double)(var + eps)));
    inv = __shfl_sync(0xffffffffu, inv, 0);
    const float4* g4 = (const float4*)gamma;
    const float4* b4 = (const float4*)beta;
#pragma unroll
    for (int i = 0; i < NV4; ++i) {
        const int k = lane + 32 * i;
        if (k < n4) {
            const float4 g = g4[k];
            float4 y;
            y.x = (v[i].x - mean) * inv * g.x; y.y = (v[i].y - mean) * inv * g.y;
            y.z = (v[i].z - mean) * inv * g.z; y.w = (v[i].w - mean) * inv * g.w;
            if (beta) { const float4 b = b4[k]; y.x += b.x; y.y += b.y; y.z += b.z; y.w += b.w; }
            if constexpr (sizeof(TO) == 4) {
                ((float4*)(out + (size_t)r * D))[k] = y;
            } else {
                __nv_bfloat162 p0 = __floats2bfloat162_rn(y.x, y.y), p1 = __floats2bfloat162_rn(y.z, y.w);
                uint2 pk;
                pk.x = *(unsigned*)&p0; pk.y = *(unsigned*)&p1;
                ((uint2*)(out + (size_t)r * D))[k] = pk;
            }
        }
    }
}

template <typename TO, int NV4>
static int launch_norm_warp(const float* x, const int* rows, const float* gamma, const float* beta, TO* out,
                            int R, int D, float eps, int rms, cudaStream_t stream) {
    return gl_launch(norm_warp_kernel<TO, NV4>, dim3((R + 7) / 8), dim3(256), 0, stream, 1, x, rows, gamma, beta, out, R, D, eps, rms);
}

template <typename TO>
static int launch_norm(const float* x, const int* rows, const float* gamma, const float* beta, TO* out,
                       int R, int D, float eps, int rms, cudaStream_t stream) {
    const bool vec = D % 4 == 0 && !(((uintptr_t)x | (uintptr_t)out | (uintptr_t)gamma | (uintptr_t)beta) & 15);
    // (the 32-bit path keeps one kernel for every row count, so that a row's result never depends
    // on how many rows come with it)
    if (sizeof(TO) == 2 && R >= 256 && vec && D <= 4096) {
        const int n = (D / 4 + 31) / 32;
        if (n <= 4) return launch_norm_warp<TO, 4>(x, rows, gamma, beta, out, R, D, eps, rms, stream);
        if (n <= 8) return launch_norm_warp<TO, 8>(x, rows, gamma, beta, out, R, D, eps, rms, stream);
        if (n <= 16) return launch_norm_warp<TO, 16>(x, rows, gamma, beta, out, R, D, eps, rms, stream);
        if (n <= 24) return launch_norm_warp<TO, 24>(x, rows, gamma, beta, out, R, D, eps, rms, stream);
        return launch_norm_warp<TO, 32>(x, rows, gamma, beta, out, R, D, eps, rms, stream);
    }
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
