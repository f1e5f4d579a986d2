// E2M1 weights x batched activations on the 5th-generation tensor cores
// (tcgen05, sm_100a) for batch 9..64.
//
// The format's scales are fp16 per (row, 32-code group), which the hardware
// block-scale formats (UE8M0 / UE4M3) cannot represent, so each 32-code group
// is one K = 32 MMA (kind::f8f6f4: A = E2M1 weights, B = E4M3 activations)
// into its own fp32 accumulator columns in tensor memory; the epilogue warps
// read the accumulators back with tcgen05.ld and apply the group's fp16 scale
// in fp32 on the CUDA cores (B/32 FMAs per weight).  The activation is held
// exactly enough by a sum of E4M3 terms (2 terms = all 8 significant bits of a
// bf16 input; 3 terms = 12 bits for fp16/fp32 inputs or a rotated activation):
// the terms share one accumulator, i.e. they extend K, not N.
//
// Roles (256 threads, one persistent CTA per SM): warp 0 copies weight tiles
// (cp.async, 8 bytes = 16 codes into the low half of each 16-byte chunk, the
// padded FP4 layout the MMA reads), warp 1 copies the pre-quantised activation
// tiles, warp 2 issues the MMAs, warp 3 owns the tensor-memory allocation,
// warps 4-7 are the epilogue (one accumulator lane = one weight row each).
// Every wait on an mbarrier is bounded: on expiry the kernel raises a status
// word, leaves its loops, frees tensor memory and returns.
#include "common.cuh"
#include <cuda_fp8.h>

namespace jqtc {

constexpr int kThreads = 256;
constexpr int kTileM = 128;
constexpr int kHeaderBytes = 512;      // workspace: int status, int exponent[64]
constexpr uint32_t kSpinLimit = 1u << 22;

template <int BN>
struct Cfg {
    static constexpr int G = (256 / BN) < 8 ? (256 / BN) : 8;  // 32-code groups per stage (and per accumulator buffer)
    static constexpr int SK = G * 32;                          // codes of K per stage
    static constexpr int A_BYTES = 2 * G * kTileM * 16;        // padded FP4: 16 codes per 16-byte chunk
    static constexpr int ACC_COLS = G * BN;                    // fp32 accumulator columns per buffer
    static constexpr int TMEM_COLS = 2 * ACC_COLS < 32 ? 32 : 2 * ACC_COLS;
};

template <int BN, int TERMS>
__host__ __device__ constexpr int b_bytes() { return TERMS * Cfg<BN>::G * 2 * BN * 16; }

template <int BN, int TERMS>
__host__ __device__ constexpr int stages() {
    // as many stages as fit in ~200 KB, at most 6
    return (200 * 1024) / (Cfg<BN>::A_BYTES + b_bytes<BN, TERMS>()) > 6 ? 6 : (200 * 1024) / (Cfg<BN>::A_BYTES + b_bytes<BN, TERMS>());
}

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("{ .reg .b64 t; mbarrier.arrive.shared::cta.b64 t, [%0]; }" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: false (and the CTA-wide error flag raised) when it gives up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *err) {
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        if (mbar_try(bar, parity)) return true;
        if (*err) return false;
        if (i > 32) __nanosleep(128);
    }
    *err = JQ_ERR_TIMEOUT;
    return false;
}

__device__ __forceinline__ void cp_async8(uint32_t dst, const void *src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
// the mbarrier receives this thread's arrival once all its earlier cp.async have landed
__device__ __forceinline__ void cp_async_arrive(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}

// K-major, no swizzle: 8 rows x 16 bytes are contiguous (128 B); lbo = byte
// distance between the two 16-byte K chunks of one MMA, sbo = distance
// between 8-row groups.  Bits 46-47 = 1 (descriptor version of sm_100).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = 0;
    d |= (uint64_t)((addr >> 4) & 0x3fffu);
    d |= (uint64_t)((lbo >> 4) & 0x3fffu) << 16;
    d |= (uint64_t)((sbo >> 4) & 0x3fffu) << 32;
    d |= (uint64_t)1 << 46;
    return d;
}

// kind::f8f6f4 instruction descriptor: D = fp32, A = E2M1 (5), B = E4M3 (0), both K-major.
__host__ __device__ constexpr uint32_t instr_desc(int M, int N) {
    return (1u << 4) | (5u << 7) | (0u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

__device__ __forceinline__ void mma_f8f6f4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{ .reg .pred p; setp.ne.b32 p, %4, 0;\n"
                 "  tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p; }"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

template <int N>
__device__ __forceinline__ void tmem_ld(uint32_t taddr, float (&v)[N]);
template <>
__device__ __forceinline__ void tmem_ld<16>(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// ---- activation preparation -----------------------------------------------------
// x[B,K] -> (rotate) -> u = x * 2^-e with max|u| < 256 -> t1 = e4m3(u),
// t2 = e4m3(u - t1), t3 = e4m3(u - t1 - t2) -> bytes in the smem-ready layout
// [stage][term][group][chunk][column][16].  Columns >= B are zero.  One block
// per column.
__device__ __forceinline__ int tc_exponent(float amax, bool had) {
    uint32_t bits = __float_as_uint(amax);
    int field = (bits >> 23) & 0xff;
    if (field == 0xff || (bits & 0x7fffffffu) == 0) return 0;
    int e = field - 127 - (had ? 3 : 7);
    return max(-100, min(100, e));
}

__device__ __forceinline__ float e4m3_round(float v, uint8_t &byte) {
    const __nv_fp8_storage_t s = __nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
    byte = (uint8_t)s;
    const __half_raw h = __nv_cvt_fp8_to_halfraw(s, __NV_E4M3);
    return __half2float(__half(h));
}

template <int BN, int TERMS>
__global__ void __launch_bounds__(256) tc_prepare_kernel(const void *__restrict__ x, int B, int K, int had, int x_dtype,
                                                          unsigned char *__restrict__ ws) {
    constexpr int G = Cfg<BN>::G, SK = Cfg<BN>::SK;
    __shared__ float sred[8];
    __shared__ int sexp;
    const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    unsigned char *xq = ws + kHeaderBytes;
    int *hdr = reinterpret_cast<int *>(ws);
    if (b == 0 && tid == 0) hdr[0] = 0;  // status word
    const bool live = b < B;
    float m = 0.f;
    if (live)
        for (int k = tid; k < K; k += 256) m = fmaxf(m, fabsf(jq::load_act(x, (size_t)b * K + k, x_dtype)));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) sred[warp] = m;
    __syncthreads();
    if (tid == 0) {
        float mm = 0.f;
        for (int w = 0; w < 8; ++w) mm = fmaxf(mm, sred[w]);
        sexp = tc_exponent(mm, had != 0);
        if (live) hdr[1 + b] = sexp;
    }
    __syncthreads();
    const float down = __uint_as_float((uint32_t)(127 - sexp) << 23);
    // one warp per 128 consecutive k (a Hadamard block when rotating); lane holds 4 consecutive k
    for (int blk = warp; blk * 128 < K; blk += 8) {
        float v[4];
        const int k0 = blk * 128 + lane * 4;
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] = live ? jq::load_act(x, (size_t)b * K + k0 + j, x_dtype) * down : 0.f;
        if (had) jq::fwht128_warp(v, lane);
        uint32_t packed[TERMS];
#pragma unroll
        for (int t = 0; t < TERMS; ++t) packed[t] = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float r = v[j];
#pragma unroll
            for (int t = 0; t < TERMS; ++t) {
                uint8_t byte;
                const float q = e4m3_round(r, byte);
                r = r - q;
                packed[t] |= (uint32_t)byte << (8 * j);
            }
        }
        const int st = k0 / SK, kk = k0 % SK, g = kk >> 5, ch = (kk >> 4) & 1, off = kk & 15;
#pragma unroll
        for (int t = 0; t < TERMS; ++t) {
            const size_t idx = ((((size_t)(st * TERMS + t) * G + g) * 2 + ch) * BN + b) * 16 + off;
            *reinterpret_cast<uint32_t *>(xq + idx) = packed[t];
        }
    }
}

// ---- main kernel ------------------------------------------------------------------
struct TcArgs {
    const uint8_t *qw;
    const __half *scales;
    const float *bias;
    void *y;
    unsigned char *ws;
    int N, K, B, y_dtype;
};

template <int BN, int TERMS>
__global__ void __launch_bounds__(kThreads, 1) gemm_e2m1_tc_kernel(TcArgs a) {
    using C = Cfg<BN>;
    constexpr int G = C::G, SK = C::SK, S = stages<BN, TERMS>();
    constexpr int A_BYTES = C::A_BYTES, B_BYTES = b_bytes<BN, TERMS>();
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ __align__(8) uint64_t bars[2 * 6 + 4];
    __shared__ uint32_t s_tmem;
    __shared__ int s_err;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t smem_base = (smem_u32(smem) + 127u) & ~127u;
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[6]);
    const uint32_t tfull0 = smem_u32(&bars[12]), tempty0 = smem_u32(&bars[14]);
    volatile int *err = &s_err;

    if (tid == 0) {
        s_err = 0;
        for (int s = 0; s < S; ++s) {
            mbar_init(full0 + 8 * s, 64);   // 32 lanes of each producer warp, arriving through cp.async completion
            mbar_init(empty0 + 8 * s, 1);   // one tcgen05.commit
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(tfull0 + 8 * i, 1);   // one tcgen05.commit
            mbar_init(tempty0 + 8 * i, 4);  // one arrival per epilogue warp
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // the upper 8 bytes of every FP4 chunk are padding that no copy writes: keep them defined
    for (uint32_t i = tid; i < (uint32_t)(S * (A_BYTES + B_BYTES)) / 16; i += kThreads)
        asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(smem_base + i * 16), "r"(0u) : "memory");
    if (warp == 3) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(C::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;

    const int ntiles = (a.N + kTileM - 1) / kTileM;
    const int nst = a.K / SK;           // stages per row tile
    const int ldw = a.K >> 1;           // bytes per packed row (K % 32 == 0 here)
    const int ngroups = a.K >> 5;
    const unsigned char *xq = a.ws + kHeaderBytes;

    if (warp == 0) {
        // ---- weight producer: lane = row inside a 32-row block
        uint32_t it = 0;
        for (int tile = blockIdx.x; tile < ntiles && !*err; tile += gridDim.x) {
            for (int st = 0; st < nst; ++st, ++it) {
                const int s = it % S;
                if (!mbar_wait(empty0 + 8 * s, ((it / S) & 1) ^ 1, err)) break;
                const uint32_t dstA = smem_base + s * (A_BYTES + B_BYTES);
#pragma unroll
                for (int rb = 0; rb < 4; ++rb) {
                    const int r = rb * 32 + lane;
                    const int row = min(tile * kTileM + r, a.N - 1);
                    const uint8_t *src = a.qw + (size_t)row * ldw + (size_t)st * (SK / 2);
#pragma unroll
                    for (int c = 0; c < 2 * G; ++c) cp_async8(dstA + c * (kTileM * 16) + r * 16, src + c * 8);
                }
                cp_async_arrive(full0 + 8 * s);
            }
        }
    } else if (warp == 1) {
        // ---- activation producer: the stage's tile is one contiguous block of the prepared buffer
        uint32_t it = 0;
        for (int tile = blockIdx.x; tile < ntiles && !*err; tile += gridDim.x) {
            for (int st = 0; st < nst; ++st, ++it) {
                const int s = it % S;
                if (!mbar_wait(empty0 + 8 * s, ((it / S) & 1) ^ 1, err)) break;
                const uint32_t dstB = smem_base + s * (A_BYTES + B_BYTES) + A_BYTES;
                const unsigned char *src = xq + (size_t)st * B_BYTES;
                for (int i = lane; i < B_BYTES / 16; i += 32) cp_async16(dstB + i * 16, src + (size_t)i * 16);
                cp_async_arrive(full0 + 8 * s);
            }
        }
    } else if (warp == 2) {
        // ---- MMA issuer (one thread)
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc(kTileM, BN);
            uint32_t it = 0;
            for (int tile = blockIdx.x; tile < ntiles && !*err; tile += gridDim.x) {
                for (int st = 0; st < nst; ++st, ++it) {
                    const int s = it % S, ab = it & 1;
                    if (!mbar_wait(tempty0 + 8 * ab, ((it >> 1) & 1) ^ 1, err)) break;  // accumulator buffer drained
                    if (!mbar_wait(full0 + 8 * s, (it / S) & 1, err)) break;            // tiles landed
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    tc_fence_after();
                    const uint32_t sa = smem_base + s * (A_BYTES + B_BYTES), sb = sa + A_BYTES;
#pragma unroll
                    for (int g = 0; g < G; ++g) {
                        const uint64_t ad = smem_desc(sa + g * (2 * kTileM * 16), kTileM * 16, 128);
#pragma unroll
                        for (int t = 0; t < TERMS; ++t) {
                            const uint64_t bd = smem_desc(sb + (t * G + g) * (2 * BN * 16), BN * 16, 128);
                            mma_f8f6f4(tmem + ab * C::ACC_COLS + g * BN, ad, bd, idesc, t > 0 ? 1u : 0u);
                        }
                    }
                    mma_commit(empty0 + 8 * s);    // smem stage reusable once these MMAs have read it
                    mma_commit(tfull0 + 8 * ab);   // accumulators of this stage complete
                }
            }
        }
    } else if (warp >= 4) {
        // ---- epilogue: thread = one accumulator lane = one weight row of the tile
        const int q = warp & 3;                // tensor-memory lane quarter this warp may touch
        const int r = q * 32 + lane;
        const int *hdr = reinterpret_cast<const int *>(a.ws);
        uint32_t it = 0;
        for (int tile = blockIdx.x; tile < ntiles && !*err; tile += gridDim.x) {
            const int row = tile * kTileM + r;
            const int rowc = min(row, a.N - 1);
            float acc[BN];
#pragma unroll
            for (int b = 0; b < BN; ++b) acc[b] = 0.f;
            bool ok = true;
            for (int st = 0; st < nst; ++st, ++it) {
                const int ab = it & 1;
                // this row's G scales of the stage (contiguous fp16)
                float sc[G];
                {
                    const __half *sp = a.scales + (size_t)rowc * ngroups + (size_t)st * G;
#pragma unroll
                    for (int g = 0; g < G; ++g) sc[g] = __half2float(sp[g]);
                }
                ok = __all_sync(0xffffffffu, mbar_wait(tfull0 + 8 * ab, (it >> 1) & 1, err));  // warp-uniform outcome
                if (!ok) break;
                tc_fence_after();
#pragma unroll
                for (int g = 0; g < G; ++g) {
#pragma unroll
                    for (int c0 = 0; c0 < BN; c0 += 16) {
                        float d[16];
                        tmem_ld<16>(tmem + ((uint32_t)(q * 32) << 16) + ab * C::ACC_COLS + g * BN + c0, d);
#pragma unroll
                        for (int i = 0; i < 16; ++i) acc[c0 + i] = fmaf(d[i], sc[g], acc[c0 + i]);
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(tempty0 + 8 * ab);
            }
            if (!ok) break;
            if (row < a.N) {
                const float bias = a.bias ? a.bias[row] : 0.f;
#pragma unroll
                for (int b = 0; b < BN; ++b) {
                    if (b < a.B) {
                        const float up = __uint_as_float((uint32_t)(127 + hdr[1 + b]) << 23);
                        jq::store_out(a.y, (size_t)b * a.N + row, fmaf(acc[b], up, bias), a.y_dtype);
                    }
                }
            }
        }
    }

    // ---- teardown: drain this thread's copies, publish the status, free tensor memory
    asm volatile("cp.async.wait_all;" ::: "memory");
    tc_fence_before();
    __syncthreads();
    if (tid == 0 && s_err) atomicExch(reinterpret_cast<int *>(a.ws), s_err);
    if (warp == 3) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(C::TMEM_COLS) : "memory");
    }
}

template <int BN, int TERMS>
static size_t tc_ws_bytes(int K) { return (size_t)kHeaderBytes + (size_t)TERMS * K * BN; }

template <int BN, int TERMS>
static int launch_tc(const TcArgs &a, const void *x, int had, int x_dtype, cudaStream_t st) {
    using C = Cfg<BN>;
    if (a.K % C::SK) return JQ_ERR_UNSUPPORTED;
    constexpr int S = stages<BN, TERMS>();
    static_assert(S >= 2 && S <= 6, "stage count");
    const size_t smem = (size_t)S * (C::A_BYTES + b_bytes<BN, TERMS>()) + 128;
    tc_prepare_kernel<BN, TERMS><<<BN, 256, 0, st>>>(x, a.B, a.K, had, x_dtype, a.ws);
    int s = jq_launch_status();
    if (s) return s;
    auto kern = gemm_e2m1_tc_kernel<BN, TERMS>;
    JQ_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int ntiles = (a.N + kTileM - 1) / kTileM;
    int grid = jq_sm_count();
    if (grid > ntiles) grid = ntiles;
    kern<<<grid, kThreads, smem, st>>>(a);
    return jq_launch_status();
}

}  // namespace jqtc

using namespace jqtc;

static int tc_bn(int B) { return B <= 16 ? 16 : (B <= 32 ? 32 : 64); }
// bf16 has 8 significant bits = two E4M3 terms exactly; anything else gets three
static int tc_terms(int had, int x_dtype) { return (!had && x_dtype == JQ_BF16) ? 2 : 3; }

size_t jq_tc_workspace_bytes(int K, int B) {
    if (B < 1 || B > 64 || K <= 0) return 0;
    return (size_t)kHeaderBytes + (size_t)3 * K * tc_bn(B);
}

extern "C" int jq_gemm_e2m1_tc(const void *qweight, const void *scales, const void *x, const float *bias, void *y,
                               int N, int K, int B, int g, int had_block, int x_dtype, int y_dtype, void *workspace,
                               size_t workspace_bytes, jq_stream_t stream) {
    if (!qweight || !scales || !x || !y || !workspace) return JQ_ERR_NULL_PTR;
    if (N <= 0 || K <= 0 || B < 1) return JQ_ERR_BAD_SHAPE;
    if (B > 64 || g != 32) return JQ_ERR_UNSUPPORTED;
    if (had_block != 0 && had_block != 128) return JQ_ERR_UNSUPPORTED;
    if (K % 256 || (had_block && K % 128)) return JQ_ERR_UNSUPPORTED;
    if (x_dtype < 0 || x_dtype > 2 || y_dtype < 0 || y_dtype > 2) return JQ_ERR_BAD_DTYPE;
    if (!jq_aligned16(qweight) || !jq_aligned16(scales) || !jq_aligned16(workspace)) return JQ_ERR_BAD_ALIGN;
    if (workspace_bytes < jq_tc_workspace_bytes(K, B)) return JQ_ERR_WORKSPACE;
    TcArgs a{reinterpret_cast<const uint8_t *>(qweight), reinterpret_cast<const __half *>(scales), bias, y,
             reinterpret_cast<unsigned char *>(workspace), N, K, B, y_dtype};
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const int bn = tc_bn(B), terms = tc_terms(had_block, x_dtype);
    if (bn == 16) return terms == 2 ? launch_tc<16, 2>(a, x, had_block, x_dtype, st) : launch_tc<16, 3>(a, x, had_block, x_dtype, st);
    if (bn == 32) return terms == 2 ? launch_tc<32, 2>(a, x, had_block, x_dtype, st) : launch_tc<32, 3>(a, x, had_block, x_dtype, st);
    return terms == 2 ? launch_tc<64, 2>(a, x, had_block, x_dtype, st) : launch_tc<64, 3>(a, x, had_block, x_dtype, st);
}

// Status word of the last jq_gemm_e2m1_tc call that used this workspace
// (0 = fine, JQ_ERR_TIMEOUT if a device-side wait gave up).  Synchronises the stream.
extern "C" int jq_tc_status(const void *workspace, jq_stream_t stream) {
    if (!workspace) return JQ_ERR_NULL_PTR;
    int v = 0;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    JQ_CUDA_TRY(cudaMemcpyAsync(&v, workspace, sizeof(int), cudaMemcpyDeviceToHost, st));
    JQ_CUDA_TRY(cudaStreamSynchronize(st));
    return v;
}
