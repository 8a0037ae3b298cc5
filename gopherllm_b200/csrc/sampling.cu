// Sampling of one token per row of logits, one block per row.
//
// The pipeline is the reference's (sampling.go:1-15, 81-130): repeat penalty on
// the tokens of the recent window, then greedy argmax when the temperature is
// (near) zero or top-k is 1; else softmax with temperature over the top-k
// candidates (or over the whole row), min-p, top-p, and one draw from a
// xorshift64 generator kept per row (sampling.go:25-42).  Non-finite logits
// count as -inf everywhere.  Logits are not modified: the row is copied to a
// scratch row first.
#include "common.cuh"
#include <float.h>

#define SM_THREADS 1024
#define SM_KMAX 1024
#define SM_WINDOW 64

struct SampleArgs {
    const float* logits;      // [B, V]
    float* work;              // [B, V] scratch
    const int* state_row;     // [B] row of recent/recent_n/rng that logits row b uses, or null (= b)
    int* recent;              // [*, SM_WINDOW] most recent tokens, oldest first; the choice is appended
    int* recent_n;            // [*] how many of them are valid
    unsigned long long* rng;  // [*] generator state, advanced by one draw when a draw is made
    int* out;                 // [B] chosen token
    float* sort_key;          // [B, vpad] scratch for the whole-row nucleus, or null
    int* sort_idx;            // [B, vpad]
    int B, V, vpad;           // vpad: a power of two >= V
    int top_k;                // <= 0: all tokens
    float temperature, top_p, min_p, repeat_penalty;
};

__device__ __forceinline__ bool finite_bits(float v) {
    return (__float_as_uint(v) & 0x7f800000u) != 0x7f800000u;
}
__device__ __forceinline__ unsigned ordered_key(float v) {
    const unsigned u = __float_as_uint(v);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float rng_next(unsigned long long* st) {
    unsigned long long s = *st;
    s ^= s << 13; s ^= s >> 7; s ^= s << 17;
    *st = s;
    return (float)(s >> 40) / 16777216.0f;
}

// the chosen token: written out and pushed onto the row's window of recent tokens
// (the reference appends every emitted token and keeps the last 64, runtime.go:1088-1093)
__device__ void finish(const SampleArgs& a, int b, int row, int token) {
    a.out[b] = token;
    int* rc = a.recent + (size_t)row * SM_WINDOW;
    int n = a.recent_n[row];
    if (n >= SM_WINDOW) {
        for (int k = 1; k < SM_WINDOW; ++k) rc[k - 1] = rc[k];
        n = SM_WINDOW - 1;
    }
    rc[n] = token;
    a.recent_n[row] = n + 1;
}

// (value, index) argmax with the lowest index among equal values
__device__ void block_argmax(float v, int i, float* sv, int* si, float* ov, int* oi) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float v2 = __shfl_xor_sync(0xffffffffu, v, o);
        const int i2 = __shfl_xor_sync(0xffffffffu, i, o);
        if (v2 > v || (v2 == v && i2 < i)) { v = v2; i = i2; }
    }
    __syncthreads();
    if (lane == 0) { sv[w] = v; si[w] = i; }
    __syncthreads();
    if (threadIdx.x == 0) {
        float bv = sv[0]; int bi = si[0];
        for (int k = 1; k < SM_THREADS / 32; ++k)
            if (sv[k] > bv || (sv[k] == bv && si[k] < bi)) { bv = sv[k]; bi = si[k]; }
        *ov = bv; *oi = bi;
    }
    __syncthreads();
}

// inclusive block scan of one float per thread; returns this thread's prefix and the total
__device__ float block_scan(float v, float* sw, float* total) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float t = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += t;
    }
    __syncthreads();
    if (lane == 31) sw[w] = v;
    __syncthreads();
    if (w == 0) {
        float t = sw[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float u = __shfl_up_sync(0xffffffffu, t, o);
            if (lane >= o) t += u;
        }
        sw[lane] = t;
    }
    __syncthreads();
    const float before = w > 0 ? sw[w - 1] : 0.f;
    *total = sw[31];
    return v + before;
}

__global__ void __launch_bounds__(SM_THREADS)
sample_kernel(SampleArgs a) {
    __shared__ float s_f[32];
    __shared__ int s_i[32];
    __shared__ float s_best;
    __shared__ int s_besti;
    __shared__ unsigned s_hist[256];
    __shared__ unsigned s_prefix, s_need, s_ngt, s_eq;
    __shared__ float c_val[SM_KMAX];
    __shared__ int c_idx[SM_KMAX];
    __shared__ int s_found;

    const int b = blockIdx.x, tid = threadIdx.x, V = a.V;
    gl_grid_launch_dependents();
    gl_grid_wait();
    const int row = a.state_row ? a.state_row[b] : b;
    const float* src = a.logits + (size_t)b * V;
    float* w = a.work + (size_t)b * V;

    // 1. copy, with every non-finite value as -inf; then the repeat penalty, once per
    //    occurrence in the window and in window order (sampling.go:136-153)
    // 2. the row's maximum, lowest index first (sampling.go:399-418)
    float bv = -INFINITY; int bi = 0x7fffffff;
    const bool vec4 = (V & 3) == 0 && (((uintptr_t)src | (uintptr_t)w) & 15) == 0;
    if ((a.temperature < 1e-6f || a.top_k == 1) && a.repeat_penalty == 1.0f) {
        // greedy without a penalty needs only the maximum: one pass over the logits, no copy
        if (vec4) {
            const float4* s4 = (const float4*)src;
            for (int i = tid; i < (V >> 2); i += SM_THREADS) {
                const float4 q = s4[i];
                const float e[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float v = finite_bits(e[k]) ? e[k] : -INFINITY;
                    if (v > bv) { bv = v; bi = 4 * i + k; }        // indices only grow inside a thread
                }
            }
        } else {
            for (int i = tid; i < V; i += SM_THREADS) {
                const float v0 = src[i];
                const float v = finite_bits(v0) ? v0 : -INFINITY;
                if (v > bv) { bv = v; bi = i; }
            }
        }
    } else {
        if (vec4) {
            const float4* s4 = (const float4*)src;
            float4* w4 = (float4*)w;
            for (int i = tid; i < (V >> 2); i += SM_THREADS) {
                float4 q = s4[i];
                q.x = finite_bits(q.x) ? q.x : -INFINITY; q.y = finite_bits(q.y) ? q.y : -INFINITY;
                q.z = finite_bits(q.z) ? q.z : -INFINITY; q.w = finite_bits(q.w) ? q.w : -INFINITY;
                w4[i] = q;
            }
        } else {
            for (int i = tid; i < V; i += SM_THREADS) {
                const float v = src[i];
                w[i] = finite_bits(v) ? v : -INFINITY;
            }
        }
        __syncthreads();
        if (tid == 0 && a.repeat_penalty != 1.0f) {
            const int n = min(a.recent_n[row], SM_WINDOW);
            const int* rc = a.recent + (size_t)row * SM_WINDOW;
            for (int k = 0; k < n; ++k) {
                const int t = rc[k];
                if (t < 0 || t >= V) continue;
                const float v = w[t];
                if (!finite_bits(v)) w[t] = -INFINITY;
                else if (v > 0.f) w[t] = v / a.repeat_penalty;
                else w[t] = v * a.repeat_penalty;
            }
        }
        __syncthreads();
        for (int i = tid; i < V; i += SM_THREADS) {
            const float v = w[i];
            if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
        }
    }
    block_argmax(bv, bi, s_f, s_i, &s_best, &s_besti);
    const float vmax = s_best;
    const int imax = s_besti;
    const bool greedy = a.temperature < 1e-6f || a.top_k == 1 || vmax == -INFINITY;
    if (greedy) {
        if (tid == 0) finish(a, b, row, (vmax == -INFINITY) ? 0 : imax);
        return;
    }
    const float inv_temp = 1.0f / a.temperature;

    if (a.top_k > 0 && a.top_k < V) {
        // 3. top-k by (value descending, index ascending): radix select of the k-th
        //    largest key, then an ordered gather (sampling.go:234-255 keeps the same set)
        const unsigned k = (unsigned)a.top_k;
        if (tid == 0) { s_prefix = 0; s_need = k; }
        __syncthreads();
        for (int shift = 24; shift >= 0; shift -= 8) {
            for (int i = tid; i < 256; i += SM_THREADS) s_hist[i] = 0;
            __syncthreads();
            const unsigned prefix = s_prefix;
            const unsigned mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
            for (int i = tid; i < V; i += SM_THREADS) {
                const unsigned key = ordered_key(w[i]);
                if ((key & mask) == prefix) atomicAdd(&s_hist[(key >> shift) & 255u], 1u);
            }
            __syncthreads();
            if (tid == 0) {
                unsigned need = s_need;
                int bin = 255;
                for (; bin > 0; --bin) {
                    if (s_hist[bin] >= need) break;
                    need -= s_hist[bin];
                }
                s_need = need;
                s_prefix = prefix | ((unsigned)bin << shift);
            }
            __syncthreads();
        }
        const unsigned kth = s_prefix;          // key of the k-th largest element
        const unsigned need_eq = s_need;        // how many elements equal to it belong to the set
        if (tid == 0) { s_ngt = 0; s_eq = 0; }
        for (int i = tid; i < SM_KMAX; i += SM_THREADS) { c_val[i] = -INFINITY; c_idx[i] = 0x7fffffff; }
        __syncthreads();
        for (int base = 0; base < V; base += SM_THREADS) {
            const int i = base + tid;
            float v = 0.f; unsigned key = 0; bool eq = false;
            if (i < V) {
                v = w[i];
                key = ordered_key(v);
                if (key > kth) {
                    const unsigned slot = atomicAdd(&s_ngt, 1u);
                    c_val[k - 1 - slot] = v;          // filled from the back; sorted below
                    c_idx[k - 1 - slot] = i;
                }
                eq = key == kth;
            }
            // elements equal to the k-th key enter in index order until the set is full
            const unsigned bal = __ballot_sync(0xffffffffu, eq);
            const int lane = tid & 31, wp = tid >> 5;
            __syncthreads();
            if (lane == 0) s_i[wp] = __popc(bal);
            __syncthreads();
            unsigned before = s_eq;
            for (int q = 0; q < wp; ++q) before += (unsigned)s_i[q];
            const unsigned mine = before + __popc(bal & ((1u << lane) - 1u));
            if (eq && mine < need_eq) { c_val[mine] = v; c_idx[mine] = i; }
            __syncthreads();
            if (tid == 0) {
                unsigned tot = 0;
                for (int q = 0; q < SM_THREADS / 32; ++q) tot += (unsigned)s_i[q];
                s_eq += tot;
            }
            __syncthreads();
        }
        // bitonic sort of the candidates, value descending then index ascending
        int kp = 1;
        while (kp < (int)k) kp <<= 1;
        for (int size = 2; size <= kp; size <<= 1) {
            for (int stride = size >> 1; stride > 0; stride >>= 1) {
                __syncthreads();
                for (int t = tid; t < kp / 2; t += SM_THREADS) {
                    const int lo = 2 * t - (t & (stride - 1));
                    const int hi = lo + stride;
                    const bool up = (lo & size) == 0;      // "up" here means best first
                    const float v0 = c_val[lo], v1 = c_val[hi];
                    const int i0 = c_idx[lo], i1 = c_idx[hi];
                    const bool first_better = v0 > v1 || (v0 == v1 && i0 < i1);
                    if (first_better != up) {
                        c_val[lo] = v1; c_val[hi] = v0;
                        c_idx[lo] = i1; c_idx[hi] = i0;
                    }
                }
            }
        }
        __syncthreads();
        // probabilities exp((l - l_max)/T), evaluated in 64-bit as the reference does
        // (sampling.go:259-262); the sums below run in candidate order in 32-bit
        const float top = c_val[0];
        __syncthreads();
        for (int i = tid; i < (int)k; i += SM_THREADS)
            c_val[i] = (float)exp((double)((c_val[i] - top) * inv_temp));
        __syncthreads();
        if (tid == 0) {
            const int n = (int)k;
            float sum = 0.f;
            for (int i = 0; i < n; ++i) sum += c_val[i];
            int token = c_idx[0];
            if (sum > 0.f) {
                int cutoff = n;
                float kept = sum;
                if (a.min_p > 0.f) {
                    const float thr = a.min_p * c_val[0];
                    float s = 0.f;
                    for (int i = 0; i < n; ++i) {
                        if (i > 0 && c_val[i] < thr) { cutoff = i; break; }
                        s += c_val[i];
                    }
                    sum = s; kept = s;
                }
                if (a.top_p < 1.0f) {
                    const float target = a.top_p * sum;
                    float cs = 0.f;
                    for (int i = 0; i < cutoff; ++i) {
                        cs += c_val[i];
                        if (cs > target) { cutoff = i + 1; break; }
                    }
                    kept = cs;
                }
                if (kept > 0.f) {
                    unsigned long long st = a.rng[row];
                    const float r = rng_next(&st) * kept;
                    a.rng[row] = st;
                    float cs = 0.f;
                    token = c_idx[cutoff - 1];
                    for (int i = 0; i < cutoff; ++i) {
                        cs += c_val[i];
                        if (cs > r) { token = c_idx[i]; break; }
                    }
                }
            }
            finish(a, b, row, token);
        }
        return;
    }

    // 4. whole row: weights exp((l - l_max)/T), normalised, inverse CDF (sampling.go:98-129, 156-166)
    float part = 0.f;
    for (int i = tid; i < V; i += SM_THREADS) {
        const float p = (float)exp((double)((w[i] - vmax) * inv_temp));
        w[i] = p;
        part += p;
    }
    float sum;
    block_scan(part, s_f, &sum);
    __syncthreads();
    if (!(sum > 0.f) || !finite_bits(sum)) {
        if (tid == 0) finish(a, b, row, imax);
        return;
    }
    if (a.top_p < 1.0f || a.min_p > 0.f) {
        // 5. nucleus over the whole row (sampleTopPFromWeights, sampling.go:171-228): candidates are
        //    the weights >= 1e-5 of the largest (all of them if that set holds less than top_p of the
        //    mass), sorted by weight descending then index ascending; min-p and top-p cut the sorted
        //    list; one draw over what is kept.
        float* ck = a.sort_key + (size_t)b * a.vpad;
        int* ci = a.sort_idx + (size_t)b * a.vpad;
        float mxp = 0.f;
        for (int i = tid; i < V; i += SM_THREADS) mxp = fmaxf(mxp, w[i]);
        int dummy;
        block_argmax(mxp, tid, s_f, s_i, &s_best, &dummy);
        const float thr = s_best * 1e-5f;
        if (tid == 0) { s_ngt = 0; }
        __syncthreads();
        float kpart = 0.f;
        for (int i = tid; i < V; i += SM_THREADS) {
            const float p = w[i];
            if (p >= thr) {
                const unsigned slot = atomicAdd(&s_ngt, 1u);
                ck[slot] = p; ci[slot] = i;
                kpart += p;
            }
        }
        float kept_sum;
        block_scan(kpart, s_f, &kept_sum);
        __syncthreads();
        int n_c = (int)s_ngt;
        if (kept_sum < a.top_p * sum) {                  // too little mass: every token is a candidate
            for (int i = tid; i < V; i += SM_THREADS) { ck[i] = w[i]; ci[i] = i; }
            n_c = V;
        }
        int np = 1;
        while (np < n_c) np <<= 1;
        for (int i = n_c + tid; i < np; i += SM_THREADS) { ck[i] = -1.f; ci[i] = 0x7fffffff; }
        // bitonic sort in global memory (the row's candidates stay in L2), best first
        for (int size = 2; size <= np; size <<= 1) {
            for (int stride = size >> 1; stride > 0; stride >>= 1) {
                __syncthreads();
                for (int t = tid; t < np / 2; t += SM_THREADS) {
                    const int lo_i = 2 * t - (t & (stride - 1)), hi_i = lo_i + stride;
                    const bool up = (lo_i & size) == 0;
                    const float v0 = ck[lo_i], v1 = ck[hi_i];
                    const int i0 = ci[lo_i], i1 = ci[hi_i];
                    const bool first_better = v0 > v1 || (v0 == v1 && i0 < i1);
                    if (first_better != up) { ck[lo_i] = v1; ck[hi_i] = v0; ci[lo_i] = i1; ci[hi_i] = i0; }
                }
            }
        }
        __syncthreads();
        // min-p: the list ends before the first weight below min_p * best; its mass is the new total
        int cutoff = n_c;
        float total = sum;
        if (a.min_p > 0.f) {
            const float mthr = a.min_p * ck[0];
            if (tid == 0) s_found = n_c;
            __syncthreads();
            for (int i = tid; i < n_c; i += SM_THREADS)
                if (i > 0 && ck[i] < mthr) atomicMin(&s_found, i);
            __syncthreads();
            cutoff = s_found;
            float mpart = 0.f;
            for (int i = tid; i < cutoff; i += SM_THREADS) mpart += ck[i];
            block_scan(mpart, s_f, &total);
            __syncthreads();
        }
        // top-p: the shortest prefix whose mass exceeds top_p * total
        const float target = a.top_p * total;
        if (tid == 0) { s_found = 0x7fffffff; s_besti = 0; }
        __syncthreads();
        float carry = 0.f, kept = 0.f;
        for (int base = 0; base < cutoff; base += SM_THREADS) {
            const int i = base + tid;
            const float p = i < cutoff ? ck[i] : 0.f;
            float tot;
            const float incl = block_scan(p, s_f, &tot) + carry;
            if (i < cutoff && incl > target) { atomicMin(&s_found, i); s_besti = 1; }
            carry += tot;
            __syncthreads();
            if (s_besti) break;
        }
        __syncthreads();
        if (s_found != 0x7fffffff) cutoff = s_found + 1;
        // the kept mass: the running sum up to the cut
        {
            float kp = 0.f;
            for (int i = tid; i < cutoff; i += SM_THREADS) kp += ck[i];
            block_scan(kp, s_f, &kept);
            __syncthreads();
        }
        if (!(kept > 0.f) || !finite_bits(kept)) {
            if (tid == 0) finish(a, b, row, imax);
            return;
        }
        if (tid == 0) {
            unsigned long long st = a.rng[row];
            s_best = rng_next(&st) * kept;
            a.rng[row] = st;
            s_found = cutoff - 1;
            s_besti = 0;
        }
        __syncthreads();
        const float rr = s_best;
        carry = 0.f;
        for (int base = 0; base < cutoff; base += SM_THREADS) {
            const int i = base + tid;
            const float p = i < cutoff ? ck[i] : 0.f;
            float tot;
            const float incl = block_scan(p, s_f, &tot) + carry;
            if (i < cutoff && incl > rr) { atomicMin(&s_found, i); s_besti = 1; }
            carry += tot;
            __syncthreads();
            if (s_besti) break;
        }
        __syncthreads();
        if (tid == 0) finish(a, b, row, ci[s_found]);
        return;
    }
    float r = 0.f;
    if (tid == 0) {
        unsigned long long st = a.rng[row];
        s_best = rng_next(&st);
        a.rng[row] = st;
        s_found = V - 1;
        s_besti = 0;
    }
    __syncthreads();
    r = s_best;
    float carry = 0.f;
    for (int base = 0; base < V; base += SM_THREADS) {
        const int i = base + tid;
        const float p = i < V ? w[i] / sum : 0.f;
        float tot;
        const float incl = block_scan(p, s_f, &tot) + carry;
        if (i < V && incl > r) atomicMin(&s_found, i);
        if (i < V && incl > r) s_besti = 1;
        carry += tot;
        __syncthreads();
        if (s_besti) break;
    }
    __syncthreads();
    if (tid == 0) finish(a, b, row, s_found);
}

GL_API int gl_sample(const SampleArgs* args, cudaStream_t stream) {
    const SampleArgs& a = *args;
    if (a.B <= 0) return GL_OK;
    if (a.V <= 0) return GL_ERR_SHAPE;
    const bool greedy = a.temperature < 1e-6f || a.top_k == 1;
    if (!greedy) {
        if (a.top_k > SM_KMAX && a.top_k < a.V) return GL_ERR_SHAPE;
        const bool whole_row = !(a.top_k > 0 && a.top_k < a.V);
        if (whole_row && (a.top_p < 1.0f || a.min_p > 0.f) && (!a.sort_key || !a.sort_idx || a.vpad < a.V))
            return GL_ERR_SHAPE;
    }
    return gl_launch(sample_kernel, dim3(a.B), dim3(SM_THREADS), 0, stream, 1, a);
}
