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
    float* sort_key;          // unused (the whole-row nucleus once sorted its candidates here); kept for the layout
    int* sort_idx;            // unused
    int B, V, vpad;           // vpad: unused
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


// ---------------------------------------------------------------------------
// Helpers of the whole-row nucleus: mass in fixed point, prefixes of the order
// "weight descending, index ascending" found without sorting.
// ---------------------------------------------------------------------------
#define SM_FIX 17592186044416.0          /* 2^44: weights are <= 1, a row has < 2^19 of them */
// a weight (0 <= p <= 1) in units of 2^-44, from its bits: integer work only, one such conversion per
// element and pass adds up (64-bit floating point is slow on this part)
__device__ __forceinline__ unsigned long long to_fixed(float p) {
    const unsigned u = __float_as_uint(p);
    const int e = (int)((u >> 23) & 255u);
    const unsigned long long m = (u & 0x7fffffu) | (e ? 0x800000u : 0u);
    const int sh = (e ? e : 1) - 106;                     // 2^(e-127) * m * 2^-23 * 2^44
    if (sh >= 0) return m << sh;
    return sh > -64 ? m >> (-sh) : 0ull;
}
__device__ __forceinline__ unsigned long long to_fixed_sum(float p) {       // a sum of weights: may exceed 1
    const double v = (double)p * SM_FIX;
    return v <= 0.0 ? 0ull : (unsigned long long)v;
}
__device__ __forceinline__ float from_fixed(unsigned long long v) { return (float)((double)v / SM_FIX); }

// f(i, w[i]) for every element of the row that falls to this thread, eight loads under way at a time: a
// loop that loads, then adds to a histogram, then loads again waits out a trip to L2 per element
template <typename F>
__device__ __forceinline__ void for_row(const float* w, int V, F f) {
    for (int base = threadIdx.x; base < V; base += SM_THREADS * 8) {
        float v[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const int i = base + k * SM_THREADS;
            v[k] = i < V ? w[i] : 0.f;
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const int i = base + k * SM_THREADS;
            if (i < V) f(i, v[k]);
        }
    }
}

// sum of one 64-bit integer per thread; every thread gets the total
__device__ unsigned long long block_sum_u64(unsigned long long v, unsigned long long* sw) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) sw[w] = v;
    __syncthreads();
    unsigned long long t = 0;
    for (int k = 0; k < SM_THREADS / 32; ++k) t += sw[k];
    __syncthreads();
    return t;
}

// A prefix of the order: every weight whose bits exceed `key`, and the first `among` (by index) of the
// weights whose bits equal it; `mass` is the prefix's mass.  found false: no prefix's mass exceeds the goal.
struct Boundary { unsigned key; unsigned among; unsigned long long mass; bool found; };
struct SelectShared { unsigned prefix; unsigned long long above; int bin; int found; unsigned rank; int token; };

// The shortest prefix (in the order above) of the candidates (weights >= low; with `within`, only the
// elements of that prefix) whose mass exceeds `goal`.  hist: [32 warps][256] 64-bit words.
__device__ Boundary select_prefix(const float* w, int V, float low, const Boundary* within, unsigned long long goal,
                                  unsigned long long* hist, unsigned long long* s_u64, SelectShared* sh) {
    const int tid = threadIdx.x, lane = tid & 31, wp = tid >> 5;
    Boundary out;
    out.found = false; out.key = 0; out.among = 0; out.mass = 0;
    if (tid == 0) { sh->prefix = 0; sh->above = 0; sh->found = 1; }
    __syncthreads();
    for (int shift = 24; shift >= 0; shift -= 8) {
        for (int i = tid; i < 32 * 256; i += SM_THREADS) hist[i] = 0;
        __syncthreads();
        const unsigned prefix = sh->prefix;
        const unsigned mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
        unsigned long long* mine = hist + wp * 256;
        const unsigned wkey = within ? within->key : 0u;
        for_row(w, V, [&](int, float pv) {
            const unsigned key = __float_as_uint(pv);
            if (pv < low || (key & mask) != prefix) return;
            if (within && key <= wkey) return;                   // what lies at the prefix's own boundary is added below
            // (one histogram per warp.  Adding the lanes' mass together first, where they hit the same
            // bin, was tried and is slower: 230 against 165 us a row, the shuffles cost more than the
            // collisions they avoid.)
            atomicAdd(mine + ((key >> shift) & 255u), to_fixed(pv));
        });
        __syncthreads();
        // the boundary weight of `within`: its first `among` elements count, as one lump in their bin
        if (within && tid == 0 && (within->key & mask) == prefix && __uint_as_float(within->key) >= low)
            hist[(within->key >> shift) & 255u] += (unsigned long long)within->among * to_fixed(__uint_as_float(within->key));
        __syncthreads();
        unsigned long long t = 0;                                 // the 32 warps' histograms into the first
        if (tid < 256)
            for (int k = 0; k < 32; ++k) t += hist[k * 256 + tid];
        __syncthreads();
        if (tid < 256) hist[tid] = t;
        __syncthreads();
        if (tid == 0) {
            unsigned long long above = sh->above;
            int bin = 255;
            for (; bin >= 0; --bin) {
                if (above + hist[bin] > goal) break;
                above += hist[bin];
            }
            sh->bin = bin;
            if (bin >= 0) { sh->above = above; sh->prefix = prefix | ((unsigned)bin << shift); }
            else sh->found = 0;
        }
        __syncthreads();
        if (!sh->found) return out;
    }
    // all 32 bits are known: how many of the equal weights it takes to pass the goal
    const unsigned key = sh->prefix;
    const unsigned long long each = to_fixed(__uint_as_float(key)), above = sh->above;
    const unsigned long long n = each > 0 ? (goal - above) / each + 1 : 1;
    out.found = true;
    out.key = key;
    out.among = (unsigned)n;
    out.mass = above + n * each;
    (void)lane; (void)wp; (void)s_u64;
    return out;
}

// index of the e-th (1-based, by index ascending) weight whose bits equal `key`; each thread takes a run of
// consecutive indices, so the equals before a thread's run are one scan away
__device__ int kth_equal(const float* w, int V, unsigned key, unsigned e, float* s_f, SelectShared* sh) {
    const int tid = threadIdx.x;
    const int per = (V + SM_THREADS - 1) / SM_THREADS;
    const int i0 = min(V, tid * per), i1 = min(V, i0 + per);
    int mine = 0;
    for (int b0 = i0; b0 < i1; b0 += 8) {
        float v[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = b0 + k < i1 ? w[b0 + k] : 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) mine += (b0 + k < i1 && __float_as_uint(v[k]) == key) ? 1 : 0;
    }
    if (tid == 0) sh->token = -1;
    float total;
    const int upto = (int)block_scan((float)mine, s_f, &total);        // counts are far below 2^24: exact in float
    __syncthreads();
    const int before = upto - mine;
    if ((unsigned)before < e && e <= (unsigned)upto) {
        int seen = before;
        for (int i = i0; i < i1; ++i)
            if (__float_as_uint(w[i]) == key && (unsigned)(++seen) == e) { sh->token = i; break; }
    }
    __syncthreads();
    int token = sh->token;
    __syncthreads();
    if (token < 0) {
        // fewer than e equals (cannot happen for a boundary that select_prefix returned): the last of them
        int last = -1;
        for (int i = i0; i < i1; ++i) if (__float_as_uint(w[i]) == key) last = i;
        atomicMax(&sh->token, last);
        __syncthreads();
        token = max(sh->token, 0);
    }
    return token;
}

// the candidate that sorts last: the smallest weight >= low, the highest index among equals
__device__ int last_candidate(const float* w, int V, float low, float* s_f, int* s_i, SelectShared* sh) {
    const int tid = threadIdx.x;
    float mn = INFINITY;
    for (int i = tid; i < V; i += SM_THREADS) { const float pv = w[i]; if (pv >= low) mn = fminf(mn, pv); }
    float bv; int bi;
    block_argmax(-mn, tid, s_f, s_i, &bv, &bi);                  // (thread 0 publishes through the two words below)
    __syncthreads();
    if (tid == 0) { sh->rank = __float_as_uint(-bv); sh->token = -1; }
    __syncthreads();
    const unsigned key = sh->rank;
    int last = -1;
    for (int i = tid; i < V; i += SM_THREADS) if (__float_as_uint(w[i]) == key) last = max(last, i);
    atomicMax(&sh->token, last);
    __syncthreads();
    return max(sh->token, 0);
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
    __shared__ unsigned long long s_u64[32];
    __shared__ SelectShared s_sel_obj;
    SelectShared* s_sel = &s_sel_obj;
    extern __shared__ unsigned long long hist[];          // [32][256], the whole-row nucleus only

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
        for_row(w, V, [&](int i, float v) {
            if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
        });
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
            // (eight loads under way per thread: a loop that loads, counts and loads again waits out a trip
            // to L2 per element, 50 of them a pass)
            for_row(w, V, [&](int, float pv) {
                const unsigned key = ordered_key(pv);
                if ((key & mask) == prefix) atomicAdd(&s_hist[(key >> shift) & 255u], 1u);
            });
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
        // what lies above the k-th key goes in as it comes (filled from the back; sorted below), and the
        // elements equal to it are counted: eight loads under way per thread, no barrier inside
        for_row(w, V, [&](int i, float v) {
            const unsigned key = ordered_key(v);
            if (key > kth) {
                const unsigned slot = atomicAdd(&s_ngt, 1u);
                c_val[k - 1 - slot] = v;
                c_idx[k - 1 - slot] = i;
            } else if (key == kth) {
                atomicAdd(&s_eq, 1u);
            }
        });
        __syncthreads();
        const unsigned n_eq = s_eq;
        __syncthreads();
        if (tid == 0) s_eq = 0;
        __syncthreads();
        if (n_eq <= need_eq) {
            // every element equal to the k-th key belongs to the set: their order is the sort's business
            for_row(w, V, [&](int i, float v) {
                if (ordered_key(v) == kth) {
                    const unsigned slot = atomicAdd(&s_eq, 1u);
                    c_val[slot] = v;
                    c_idx[slot] = i;
                }
            });
        } else {
            // more equals than places (ties at the set's edge): they enter in index order until the set is full
            for (int base = 0; base < V; base += SM_THREADS) {
                const int i = base + tid;
                float v = 0.f; bool eq = false;
                if (i < V) {
                    v = w[i];
                    eq = ordered_key(v) == kth;
                }
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
                if (s_eq >= need_eq) break;                // (the same for every thread: read behind the barrier)
            }
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
        // 5. nucleus over the whole row (sampleTopPFromWeights, sampling.go:171-228).  The reference sorts
        //    the candidates (the weights >= 1e-5 of the largest; all of them if that set holds less than
        //    top_p of the mass) by weight descending then index ascending, cuts the list at the first
        //    weight below min_p times the best and at the shortest prefix whose mass exceeds top_p times
        //    the total, and draws from what is kept.  A prefix of that order is "every weight above some
        //    value, and the first few, by index, of the weights equal to it", so nothing is sorted here:
        //    the value is found digit by digit (four passes of 256-bin histograms of mass over the bits
        //    of the weights), once for the cut and once for the draw.  Mass is added up in 64-bit fixed
        //    point, so the sums do not depend on the order of the additions.
        float mxp = 0.f;
        for_row(w, V, [&](int, float pv) { mxp = fmaxf(mxp, pv); });
        block_argmax(mxp, tid, s_f, s_i, &s_best, &s_besti);
        const float best = s_best;
        const float thr = best * 1e-5f;
        // the candidates: weights >= thr if they carry top_p of the mass, else all
        unsigned long long part_fx = 0;
        for_row(w, V, [&](int, float pv) { if (pv >= thr) part_fx += to_fixed(pv); });
        const float kept_sum = from_fixed(block_sum_u64(part_fx, s_u64));
        float low = (kept_sum < a.top_p * sum) ? 0.f : thr;          // weights below `low` are not candidates
        // min-p: the list ends before the first weight below min_p * best; its mass is the new total
        float total = sum;
        if (a.min_p > 0.f) {
            low = fmaxf(low, a.min_p * best);
            unsigned long long m_fx = 0;
            for_row(w, V, [&](int, float pv) { if (pv >= low) m_fx += to_fixed(pv); });
            total = from_fixed(block_sum_u64(m_fx, s_u64));
        }
        // top-p: the shortest prefix whose mass exceeds top_p * total
        const float target = a.top_p * total;
        Boundary cut = select_prefix(w, V, low, nullptr, to_fixed_sum(target), hist, s_u64, s_sel);
        float kept;
        if (cut.found) {
            kept = from_fixed(cut.mass);
        } else {                                                      // never exceeded: everything is kept
            unsigned long long m_fx = 0;
            for_row(w, V, [&](int, float pv) { if (pv >= low) m_fx += to_fixed(pv); });
            kept = from_fixed(block_sum_u64(m_fx, s_u64));
        }
        if (!(kept > 0.f) || !finite_bits(kept)) {
            if (tid == 0) finish(a, b, row, imax);
            return;
        }
        if (tid == 0) {
            unsigned long long st = a.rng[row];
            s_best = rng_next(&st) * kept;
            a.rng[row] = st;
        }
        __syncthreads();
        const float rr = s_best;
        // the draw: the first element of the kept prefix, in the same order, whose running mass exceeds rr
        Boundary pick = select_prefix(w, V, low, cut.found ? &cut : nullptr, to_fixed_sum(rr), hist, s_u64, s_sel);
        int token;
        if (pick.found) token = kth_equal(w, V, pick.key, pick.among, s_f, s_sel);
        else if (cut.found) token = kth_equal(w, V, cut.key, cut.among, s_f, s_sel);     // the list's last element
        else token = last_candidate(w, V, low, s_f, s_i, s_sel);
        if (tid == 0) finish(a, b, row, token);
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
    size_t smem = 0;
    if (!greedy) {
        if (a.top_k > SM_KMAX && a.top_k < a.V) return GL_ERR_SHAPE;
        const bool whole_row = !(a.top_k > 0 && a.top_k < a.V);
        if (whole_row && (a.top_p < 1.0f || a.min_p > 0.f)) {
            // the nucleus over the whole row keeps a histogram of mass per warp
            smem = 32 * 256 * sizeof(unsigned long long);
            static bool configured = false;
            if (!configured) {
                if (cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
                    cudaGetLastError();
                    return GL_ERR_SMEM;
                }
                configured = true;
            }
        }
    }
    return gl_launch(sample_kernel, dim3(a.B), dim3(SM_THREADS), smem, stream, 1, a);
}
