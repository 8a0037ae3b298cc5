// Decode attention: one new token per sequence against its cached keys and
// values, bandwidth-bound, so the work is cut over (sequence, key/value head,
// split of the sequence's pages) to fill the machine, and merged afterwards.
//
// A block streams its pages through shared memory with cp.async (16-byte
// copies, two pages in flight), scores 64 keys at a time, keeps a running
// maximum and sum in 32-bit and accumulates the weighted values in 32-bit
// registers.  Splits write (max, sum, unnormalised output) to scratch and a
// second kernel merges them; with one split the block writes the result itself.
// The head size is a compile-time constant (GL_HEAD_DIM, a multiple of 16).
#include "common.cuh"
#include <cuda_pipeline.h>

#ifndef GL_HEAD_DIM
#define GL_HEAD_DIM 80
#endif
static_assert(GL_HEAD_DIM % 16 == 0 && GL_HEAD_DIM >= 16 && GL_HEAD_DIM <= 256, "head size: 16..256 in steps of 16");

#define AD_THREADS 128
#define AD_HD GL_HEAD_DIM
#define AD_CHUNKS (AD_HD / 8)                       // 16-byte chunks per row
#define AD_ROW (AD_HD * 2 + 16)                     // padded row in bytes: conflict-free 16-byte reads
#define AD_TILE (GL_PAGE * AD_ROW)                  // one page of K (or V) for one head
#define AD_KG (AD_THREADS / AD_CHUNKS)              // key groups in the value pass
#define AD_MAXG 8                                   // query heads per key/value head handled at once

struct DecodeArgs {
    const __nv_bfloat16* q;      // [B, nH*hd], scaled
    __nv_bfloat16* out;          // [B, nH*hd]
    const __nv_bfloat16* k_cache;// [pages, nKV, GL_PAGE, hd]
    const __nv_bfloat16* v_cache;
    const int* seq_ctx;          // [B] positions cached before this step (the new token sits at seq_ctx[b])
    const int* pages;            // [B, max_pages]
    float* part_o;               // [B, nH, splits, hd] scratch
    float* part_ml;              // [B, nH, splits, 2]  scratch
    int B, nH, nKV, max_pages, window, splits;
};

__device__ __forceinline__ void load_page(unsigned char* dst, const __nv_bfloat16* src) {
    // 64 rows of hd bf16, contiguous in global memory, to padded rows in shared memory
    for (int i = threadIdx.x; i < GL_PAGE * AD_CHUNKS; i += AD_THREADS) {
        const int r = i / AD_CHUNKS, c = i - r * AD_CHUNKS;
        __pipeline_memcpy_async(dst + r * AD_ROW + c * 16, (const unsigned char*)src + (size_t)i * 16, 16);
    }
}

// GM: compile-time bound on the query heads per key/value head (1, 2, 4 or 8), so that the
// per-head accumulators stay in registers
template <int GM>
__global__ void __launch_bounds__(AD_THREADS)
attn_decode_kernel(DecodeArgs a) {
    extern __shared__ __align__(16) unsigned char smem[];
    unsigned char* Kt[2] = {smem, smem + 2 * AD_TILE};
    unsigned char* Vt[2] = {smem + AD_TILE, smem + 3 * AD_TILE};
    float* qs = (float*)(smem + 4 * AD_TILE);            // [G][hd]
    float* ps = qs + GM * AD_HD;                         // [G][64] scores, then weights
    float* red = ps + GM * GL_PAGE;                      // [G][4] warp maxima, [G][4] warp sums
    float* osum = red + GM * 8;                     // [KG][hd] final reduction, one head at a time

    const int split = blockIdx.x, g = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int G = a.nH / a.nKV;                          // query heads of this key/value head (<= AD_MAXG)
    const int pos = a.seq_ctx[b];                        // the query's position; keys lo..pos
    const int lo = (a.window > 0 && pos - a.window + 1 > 0) ? pos - a.window + 1 : 0;
    const int first_page = lo / GL_PAGE, n_pages = pos / GL_PAGE + 1 - first_page;
    const int per = (n_pages + a.splits - 1) / a.splits;
    const int p_begin = first_page + split * per;
    const int p_end = min(first_page + n_pages, p_begin + per);
    const int* pg = a.pages + (size_t)b * a.max_pages;
    const size_t head_off = (size_t)g * GL_PAGE * AD_HD;
    const size_t page_stride = (size_t)a.nKV * GL_PAGE * AD_HD;

    for (int i = tid; i < G * AD_HD; i += AD_THREADS) {
        const int h = g * G + i / AD_HD;
        qs[i] = __bfloat162float(a.q[((size_t)b * a.nH + h) * AD_HD + (i % AD_HD)]);
    }
    float acc[GM][8];
    float m_run[GM], l_run[GM];
#pragma unroll
    for (int q = 0; q < GM; ++q) {
        m_run[q] = -INFINITY; l_run[q] = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[q][e] = 0.f;
    }
    const int my_chunk = tid % AD_CHUNKS, my_kg = tid / AD_CHUNKS;   // value pass: my 8 dims, my keys
    const bool v_active = my_kg < AD_KG;

    if (p_begin < p_end) {
        load_page(Kt[0], a.k_cache + (size_t)pg[p_begin] * page_stride + head_off);
        load_page(Vt[0], a.v_cache + (size_t)pg[p_begin] * page_stride + head_off);
    }
    __pipeline_commit();
    for (int p = p_begin; p < p_end; ++p) {
        const int st = (p - p_begin) & 1;
        if (p + 1 < p_end) {
            load_page(Kt[st ^ 1], a.k_cache + (size_t)pg[p + 1] * page_stride + head_off);
            load_page(Vt[st ^ 1], a.v_cache + (size_t)pg[p + 1] * page_stride + head_off);
        }
        __pipeline_commit();
        __pipeline_wait_prior(1);
        __syncthreads();
        const int j0 = p * GL_PAGE;
        const int n_valid = min(GL_PAGE, pos + 1 - j0);          // rows past the sequence were never written
        // scores: thread = (key, half of the head dims); the two halves meet by shuffle
        {
            const int key = tid >> 1, half = tid & 1;
            const unsigned char* kr = Kt[st] + key * AD_ROW + half * AD_HD;   // hd/2 elements = hd bytes
            const bool ok = key < n_valid && j0 + key >= lo;
#pragma unroll
            for (int q = 0; q < GM; ++q) {
                if (q >= G) break;
                float s = 0.f;
                if (ok) {
                    const float* qv = qs + q * AD_HD + half * (AD_HD / 2);
#pragma unroll
                    for (int c = 0; c < AD_HD / 16; ++c) {
                        const uint4 raw = *(const uint4*)(kr + c * 16);
                        const __nv_bfloat162* k2 = (const __nv_bfloat162*)&raw;
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float2 kf = __bfloat1622float2(k2[e]);
                            s = fmaf(qv[c * 8 + 2 * e], kf.x, s);
                            s = fmaf(qv[c * 8 + 2 * e + 1], kf.y, s);
                        }
                    }
                }
                s += __shfl_xor_sync(0xffffffffu, s, 1);
                s = ok ? s : -INFINITY;
                if (half == 0) ps[q * GL_PAGE + key] = s;
                const float wm = gl_warp_max(s);
                if (lane == 0) red[q * 8 + warp] = wm;
            }
        }
        __syncthreads();
        // running maximum and sum; weights replace scores
#pragma unroll
        for (int q = 0; q < GM; ++q) {
            if (q >= G) break;
            const float pm = fmaxf(fmaxf(red[q * 8], red[q * 8 + 1]), fmaxf(red[q * 8 + 2], red[q * 8 + 3]));
            const float m_new = fmaxf(m_run[q], pm);
            const float corr = (m_new == -INFINITY) ? 1.f : __expf(m_run[q] - m_new);
            float w = 0.f;
            if (tid < GL_PAGE) {
                const float s = ps[q * GL_PAGE + tid];
                w = (s == -INFINITY) ? 0.f : __expf(s - m_new);
                ps[q * GL_PAGE + tid] = w;
            }
            const float ws = gl_warp_sum(w);
            if (lane == 0) red[q * 8 + 4 + warp] = ws;
            m_run[q] = m_new;
            l_run[q] *= corr;
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[q][e] *= corr;
        }
        __syncthreads();
#pragma unroll
        for (int q = 0; q < GM; ++q)
            if (q < G) l_run[q] += red[q * 8 + 4] + red[q * 8 + 5];           // only warps 0 and 1 hold keys
        // values: thread = (8 dims, every AD_KG-th key)
        if (v_active) {
            for (int j = my_kg; j < n_valid; j += AD_KG) {
                const uint4 raw = *(const uint4*)(Vt[st] + j * AD_ROW + my_chunk * 16);
                const __nv_bfloat162* v2 = (const __nv_bfloat162*)&raw;
                float vf[8];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 f = __bfloat1622float2(v2[e]);
                    vf[2 * e] = f.x; vf[2 * e + 1] = f.y;
                }
#pragma unroll
                for (int q = 0; q < GM; ++q) {
                    if (q >= G) break;
                    const float w = ps[q * GL_PAGE + j];
#pragma unroll
                    for (int e = 0; e < 8; ++e) acc[q][e] = fmaf(w, vf[e], acc[q][e]);
                }
            }
        }
        __syncthreads();
    }
    __pipeline_wait_prior(0);

    // sum the key groups, one query head at a time, and write the split's result
#pragma unroll
    for (int q = 0; q < GM; ++q) {
        if (q >= G) break;
        __syncthreads();
        if (v_active) {
#pragma unroll
            for (int e = 0; e < 8; ++e) osum[my_kg * AD_HD + my_chunk * 8 + e] = acc[q][e];
        }
        __syncthreads();
        const int h = g * G + q;
        for (int d = tid; d < AD_HD; d += AD_THREADS) {
            float o = 0.f;
            for (int kg = 0; kg < AD_KG; ++kg) o += osum[kg * AD_HD + d];
            if (a.splits == 1) {
                const float inv = l_run[q] > 0.f ? 1.f / l_run[q] : 0.f;
                a.out[((size_t)b * a.nH + h) * AD_HD + d] = __float2bfloat16_rn(o * inv);
            } else {
                a.part_o[(((size_t)b * a.nH + h) * a.splits + split) * AD_HD + d] = o;
            }
        }
        if (a.splits > 1 && tid == 0) {
            float* ml = a.part_ml + (((size_t)b * a.nH + h) * a.splits + split) * 2;
            ml[0] = m_run[q];
            ml[1] = l_run[q];
        }
    }
}

// out = sum_s exp(m_s - m) o_s / sum_s exp(m_s - m) l_s over the splits, in split order
__global__ void attn_decode_merge_kernel(DecodeArgs a) {
    const int h = blockIdx.x, b = blockIdx.y;
    const float* ml = a.part_ml + ((size_t)b * a.nH + h) * a.splits * 2;
    const float* po = a.part_o + ((size_t)b * a.nH + h) * a.splits * AD_HD;
    float m = -INFINITY;
    for (int s = 0; s < a.splits; ++s) m = fmaxf(m, ml[2 * s]);
    for (int d = threadIdx.x; d < AD_HD; d += blockDim.x) {
        float o = 0.f, l = 0.f;
        for (int s = 0; s < a.splits; ++s) {
            const float ms = ml[2 * s];
            if (ms == -INFINITY) continue;
            const float w = __expf(ms - m);
            o = fmaf(w, po[s * AD_HD + d], o);
            l = fmaf(w, ml[2 * s + 1], l);
        }
        a.out[((size_t)b * a.nH + h) * AD_HD + d] = __float2bfloat16_rn(l > 0.f ? o / l : 0.f);
    }
}

static size_t decode_smem(int gm) {
    return 4 * (size_t)AD_TILE + sizeof(float) * ((size_t)gm * AD_HD + gm * GL_PAGE + gm * 8 + (size_t)AD_KG * AD_HD);
}

template <int GM>
static int launch_decode(const DecodeArgs& a, cudaStream_t stream) {
    static bool configured = false;
    const size_t smem = decode_smem(GM);
    if (!configured) {
        if (cudaFuncSetAttribute(attn_decode_kernel<GM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
            cudaGetLastError();
            return GL_ERR_SMEM;
        }
        configured = true;
    }
    dim3 grid(a.splits, a.nKV, a.B);
    attn_decode_kernel<GM><<<grid, AD_THREADS, smem, stream>>>(a);
    return GL_OK;
}

GL_API int gl_attention_decode_head_dim() { return AD_HD; }

// scratch floats needed for B sequences, nH heads and a number of splits
GL_API long long gl_attention_decode_scratch(int B, int nH, int splits) {
    return splits > 1 ? (long long)B * nH * splits * (AD_HD + 2) : 0;
}

GL_API int gl_attention_decode(const DecodeArgs* args, cudaStream_t stream) {
    const DecodeArgs& a = *args;
    if (a.B <= 0) return GL_OK;
    if (a.nH <= 0 || a.nKV <= 0 || a.nH % a.nKV || a.nH / a.nKV > AD_MAXG) return GL_ERR_SHAPE;
    if (a.splits < 1 || a.B > 65535 || a.nKV > 65535) return GL_ERR_SHAPE;
    if (a.splits > 1 && (!a.part_o || !a.part_ml)) return GL_ERR_SHAPE;
    const int G = a.nH / a.nKV;
    int rc;
    if (G == 1) rc = launch_decode<1>(a, stream);
    else if (G == 2) rc = launch_decode<2>(a, stream);
    else if (G <= 4) rc = launch_decode<4>(a, stream);
    else rc = launch_decode<8>(a, stream);
    if (rc != GL_OK) return rc;
    if (a.splits > 1) {
        dim3 mg(a.nH, a.B);
        attn_decode_merge_kernel<<<mg, AD_HD >= 128 ? 128 : 64, 0, stream>>>(a);
    }
    return gl_check_launch();
}

// ---------------------------------------------------------------------------
// The same decode attention for callers that must not allocate device memory.
// See attention_decode_static.h for who that is and what the limits are.
// ---------------------------------------------------------------------------
#include "attention_decode_static.h"

// Scratch for the splits' partial results, resident in every GPU context that
// loads this library until the process exits.
static __device__ __align__(256) float gl_decode_static_scratch[GL_DECODE_STATIC_SCRATCH_FLOATS];

#define GL_DECODE_STATIC_MAX_DEVICES 64
static float* gl_decode_static_ptr[GL_DECODE_STATIC_MAX_DEVICES];   // device address of the array, per device

GL_API long long gl_attention_decode_static_capacity() { return GL_DECODE_STATIC_SCRATCH_FLOATS; }

GL_API int gl_attention_decode_static(const DecodeArgs* args, cudaStream_t stream) {
    if (!args) return GL_ERR_SHAPE;
    DecodeArgs a = *args;
    if (a.B <= 0) return GL_OK;
    if (a.splits < 1 || a.nH <= 0) return GL_ERR_SHAPE;
    const long long need = gl_attention_decode_scratch(a.B, a.nH, a.splits);
    if (need > (long long)GL_DECODE_STATIC_SCRATCH_FLOATS) return GL_ERR_SCRATCH;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= GL_DECODE_STATIC_MAX_DEVICES) {
        cudaGetLastError();
        return GL_ERR_DRIVER;
    }
    if (!gl_decode_static_ptr[dev]) {
        // In host code the array's name is only a handle; the address a kernel can use is
        // looked up once per device, with that device current.
        float* p = nullptr;
        if (cudaGetSymbolAddress((void**)&p, gl_decode_static_scratch) != cudaSuccess || !p) {
            cudaGetLastError();
            return GL_ERR_DRIVER;
        }
        gl_decode_static_ptr[dev] = p;
    }
    // Every (sequence, head, split) cell that the merge reads is written by the first kernel of
    // the same call, empty splits included, so nothing has to be cleared between calls.
    a.part_o = gl_decode_static_ptr[dev];
    a.part_ml = gl_decode_static_ptr[dev] + (size_t)a.B * a.nH * a.splits * AD_HD;
    return gl_attention_decode(&a, stream);
}
