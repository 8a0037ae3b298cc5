// out[M,N] = act(A[M,K] · W[N,K]ᵀ + bias) + add0 + add1 for many rows, bfloat16,
// on the 5th-generation tensor cores.
//
// A persistent kernel, one block per SM, walks the 128 x BN output tiles.  Warp 0
// feeds shared memory by TMA (128-byte swizzled boxes of 64 k, several stages
// ahead); one thread of warp 1 issues tcgen05.mma (M 128, N BN, K 16, both
// operands K-major from shared memory, accumulator in tensor memory) and hands
// stages back through tcgen05.commit; warps 2..5 read a finished accumulator out
// of tensor memory (tcgen05.ld, one row per thread), apply bias, activation and
// the residual additions in 32-bit and store.  Two accumulators alternate, so the
// epilogue of one tile runs under the products of the next.  Rows and columns
// outside the matrices are zero-filled by TMA and masked at the store.
//
// Every wait on an mbarrier is bounded; if one runs out the block records it,
// leaves its loops, frees its tensor memory and returns.
#include "common.cuh"
#include "tma.cuh"

#define TG_BM 128
#define TG_BK 64
#define TG_THREADS 192

struct GemmArgs {
    const void* a;        // [M, K] bf16
    const void* w;        // [N, K] bf16
    const float* bias;    // [N] or null
    const float* add0;    // [M, N] or null
    const float* add1;    // [M, N] or null
    void* out;            // [M, N] f32 or bf16
    int M, N, K, act;
};

// shared-memory matrix descriptor: K-major tile of 128-byte rows, 128-byte swizzle,
// 8-row groups 1024 bytes apart, descriptor version 1 (sm_100)
__device__ __forceinline__ uint64_t umma_desc(unsigned smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);          // start address, 16-byte units
    d |= (uint64_t)1 << 16;                               // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;                     // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                               // version
    d |= (uint64_t)2 << 61;                               // SWIZZLE_128B
    return d;
}
// instruction descriptor: bf16 x bf16 -> f32, A and B K-major, M 128, N bn
__host__ __device__ constexpr uint32_t umma_idesc(int bn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(TG_BM >> 4) << 24);
}
__device__ __forceinline__ void umma_bf16(unsigned tmem_d, uint64_t da, uint64_t db, uint32_t idesc, unsigned accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                 " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n}"
                 ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void umma_commit(unsigned bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld32(unsigned taddr, unsigned (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
                 "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

template <int BN, int STAGES, typename TO>
__global__ void __launch_bounds__(TG_THREADS, 1)
gemm_tcgen05_kernel(GemmArgs g, const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w) {
    extern __shared__ unsigned char smem_raw[];
    constexpr int A_BYTES = TG_BM * 128, B_BYTES = BN * 128, STAGE = A_BYTES + B_BYTES;
    constexpr unsigned TMEM_COLS = 2 * BN >= 32 ? 2 * BN : 32;     // a power of two: BN is 64, 128 or 256
    __shared__ unsigned tmem_base_slot;
    __shared__ volatile int failed;

    unsigned char* smem = smem_raw + ((1024u - (gl_smem_u32(smem_raw) & 1023u)) & 1023u);
    const unsigned base = gl_smem_u32(smem);
    const unsigned bar_full = base + STAGES * STAGE;          // [STAGES]
    const unsigned bar_empty = bar_full + 8 * STAGES;         // [STAGES]
    const unsigned bar_tfull = bar_empty + 8 * STAGES;        // [2] accumulator ready for the epilogue
    const unsigned bar_tempty = bar_tfull + 16;               // [2] accumulator drained
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_m = (g.M + TG_BM - 1) / TG_BM, tiles_n = (g.N + BN - 1) / BN;
    const int n_tiles = tiles_m * tiles_n;
    const int k_blocks = (g.K + TG_BK - 1) / TG_BK;

    if (threadIdx.x == 0) {
        failed = 0;
        for (int s = 0; s < STAGES; ++s) { mbar_init(bar_full + 8 * s, 1); mbar_init(bar_empty + 8 * s, 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(bar_tfull + 8 * b, 1); mbar_init(bar_tempty + 8 * b, 4); }
        mbar_fence_init();
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(gl_smem_u32(&tmem_base_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_base = tmem_base_slot;

    if (warp == 0) {
        // ---- TMA producer -------------------------------------------------
        if (lane == 0) {
            int it = 0;
            for (int tile = blockIdx.x; tile < n_tiles && !failed; tile += gridDim.x) {
                const int m0 = (tile % tiles_m) * TG_BM, n0 = (tile / tiles_m) * BN;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (it >= STAGES && !mbar_wait(bar_empty + 8 * s, ((it / STAGES) - 1) & 1)) { failed = 1; break; }
                    const unsigned sb = base + s * STAGE;
                    mbar_expect_tx(bar_full + 8 * s, STAGE);
                    tma_load_2d(sb, &map_a, kb * TG_BK, m0, bar_full + 8 * s);
                    tma_load_2d(sb + A_BYTES, &map_w, kb * TG_BK, n0, bar_full + 8 * s);
                }
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer ------------------------------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc(BN);
            int it = 0, local = 0;
            for (int tile = blockIdx.x; tile < n_tiles && !failed; tile += gridDim.x, ++local) {
                const int buf = local & 1;
                if (local >= 2 && !mbar_wait(bar_tempty + 8 * buf, ((local >> 1) - 1) & 1)) { failed = 1; break; }
                tc_fence_after();
                const unsigned d = tmem_base + buf * BN;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait(bar_full + 8 * s, (it / STAGES) & 1)) { failed = 1; break; }
                    tc_fence_after();
                    const unsigned sb = base + s * STAGE;
                    const uint64_t da = umma_desc(sb), db = umma_desc(sb + A_BYTES);
#pragma unroll
                    for (int k = 0; k < TG_BK / 16; ++k)     // 32 bytes further along the swizzled row per K 16
                        umma_bf16(d, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
                    umma_commit(bar_empty + 8 * s);          // the stage is free once these products have read it
                }
                if (failed) break;
                umma_commit(bar_tfull + 8 * buf);            // the accumulator is complete
            }
        }
    } else {
        // ---- epilogue: warps 2..5, each on the tensor-memory lanes of its quarter -----
        const int quarter = warp & 3;
        int local = 0;
        TO* O = (TO*)g.out;
        for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++local) {
            const int buf = local & 1;
            const int m0 = (tile % tiles_m) * TG_BM, n0 = (tile / tiles_m) * BN;
            bool ok = mbar_wait(bar_tfull + 8 * buf, (local >> 1) & 1);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) { failed = 1; break; }
            tc_fence_after();
            const int m = m0 + quarter * 32 + lane;
            const unsigned trow = tmem_base + buf * BN + ((unsigned)(quarter * 32) << 16);
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                unsigned r[32];
                tmem_ld32(trow + c, r);
                if (m < g.M) {
                    const int nb = n0 + c;
                    const size_t o = (size_t)m * g.N + nb;
                    const bool full = nb + 32 <= g.N && (g.N & 7) == 0;
                    float v[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        v[j] = __uint_as_float(r[j]);
                        if (g.bias && nb + j < g.N) v[j] += g.bias[nb + j];
                        v[j] = gl_activate<false>(v[j], g.act);
                    }
                    if (full) {
                        if (g.add0) {
#pragma unroll
                            for (int j = 0; j < 32; j += 4) {
                                const float4 t = *(const float4*)(g.add0 + o + j);
                                v[j] += t.x; v[j + 1] += t.y; v[j + 2] += t.z; v[j + 3] += t.w;
                            }
                        }
                        if (g.add1) {
#pragma unroll
                            for (int j = 0; j < 32; j += 4) {
                                const float4 t = *(const float4*)(g.add1 + o + j);
                                v[j] += t.x; v[j + 1] += t.y; v[j + 2] += t.z; v[j + 3] += t.w;
                            }
                        }
                        if constexpr (sizeof(TO) == 4) {
#pragma unroll
                            for (int j = 0; j < 32; j += 4)
                                *(float4*)((float*)O + o + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; j += 8) {
                                uint4 pk;
                                __nv_bfloat162 p0 = __floats2bfloat162_rn(v[j], v[j + 1]);
                                __nv_bfloat162 p1 = __floats2bfloat162_rn(v[j + 2], v[j + 3]);
                                __nv_bfloat162 p2 = __floats2bfloat162_rn(v[j + 4], v[j + 5]);
                                __nv_bfloat162 p3 = __floats2bfloat162_rn(v[j + 6], v[j + 7]);
                                pk.x = *(unsigned*)&p0; pk.y = *(unsigned*)&p1; pk.z = *(unsigned*)&p2; pk.w = *(unsigned*)&p3;
                                *(uint4*)((__nv_bfloat16*)O + o + j) = pk;
                            }
                        }
                    } else {
                        for (int j = 0; j < 32 && nb + j < g.N; ++j) {
                            float y = v[j];
                            if (g.add0) y += g.add0[o + j];
                            if (g.add1) y += g.add1[o + j];
                            gl_store(O + o + j, y);
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_tempty + 8 * buf);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
    if (threadIdx.x == 0 && failed) atomicExch(&gl_wait_failed, 1);
}

template <int BN, int STAGES>
static constexpr size_t tg_smem() {
    return (size_t)STAGES * (TG_BM * 128 + BN * 128) + 8 * (2 * STAGES + 4) + 1024;
}

template <int BN, int STAGES, typename TO>
static int launch_tg(const GemmArgs& g, cudaStream_t stream) {
    constexpr size_t smem = tg_smem<BN, STAGES>();
    static bool configured = false;
    static int sms = 0;
    if (!configured) {
        if (cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, STAGES, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem) != cudaSuccess) {
            cudaGetLastError();
            return GL_ERR_SMEM;
        }
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (sms <= 0) sms = 148;
        configured = true;
    }
    CUtensorMap map_a, map_w;
    int rc = gl_cached_map_bf16(&map_a, g.a, (uint64_t)g.M, (uint64_t)g.K, TG_BM, TG_BK);
    if (rc != GL_OK) return rc;
    rc = gl_cached_map_bf16(&map_w, g.w, (uint64_t)g.N, (uint64_t)g.K, BN, TG_BK);
    if (rc != GL_OK) return rc;
    const int tiles = ((g.M + TG_BM - 1) / TG_BM) * ((g.N + BN - 1) / BN);
    const int grid = tiles < sms ? tiles : sms;
    gemm_tcgen05_kernel<BN, STAGES, TO><<<grid, TG_THREADS, smem, stream>>>(g, map_a, map_w);
    return gl_check_launch();
}

template <typename TO>
static int dispatch_bn(const GemmArgs& g, int bn, cudaStream_t stream) {
    if (bn == 256) return launch_tg<256, 4, TO>(g, stream);
    if (bn == 128) return launch_tg<128, 6, TO>(g, stream);
    if (bn == 64) return launch_tg<64, 8, TO>(g, stream);
    return GL_ERR_SHAPE;
}

GL_API int gl_gemm_tcgen05_wait_failed() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, gl_wait_failed, sizeof(int)) != cudaSuccess) return -1;
    return v;
}

// bn: tile width 64, 128 or 256; 0 lets the launcher choose
GL_API int gl_gemm_tcgen05(const GemmArgs* args, int out_dtype, int bn, cudaStream_t stream) {
    const GemmArgs& g = *args;
    if (g.M <= 0 || g.N <= 0) return GL_OK;
    if (g.K <= 0 || g.K % 8) return GL_ERR_SHAPE;
    if (((uintptr_t)g.a | (uintptr_t)g.w) & 15) return GL_ERR_ALIGN;
    if (bn == 0) {
        // the widest tile whose last wave is not mostly idle
        int sms = 148;
        const int tm = (g.M + TG_BM - 1) / TG_BM;
        double best = 1e30;
        const int cands[3] = {256, 128, 64};
        for (int i = 0; i < 3; ++i) {
            const int c = cands[i];
            const int tiles = tm * ((g.N + c - 1) / c);
            const int waves = (tiles + sms - 1) / sms;
            const double cost = (double)waves * c * (c == 256 ? 1.0 : c == 128 ? 1.3 : 2.0);
            if (cost < best) { best = cost; bn = c; }
        }
    }
    if (out_dtype == GL_F32) return dispatch_bn<float>(g, bn, stream);
    if (out_dtype == GL_BF16) return dispatch_bn<__nv_bfloat16>(g, bn, stream);
    return GL_ERR_DTYPE;
}
