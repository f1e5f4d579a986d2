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

constexpr int kPrefetch = 12;   // stages of weights requested into L2 ahead of the shared-memory ring
constexpr int kThreads = 512;   // warps 0-3 producers, 4-7 MMA issuers (4 owns tensor memory), 8-15 epilogue
constexpr int kMmaWarps = 2;   // issuer w owns accumulator buffer w and the stages it = w, w+2, ... (warps 6, 7 idle)   // 4 service warps + 8 epilogue warps
constexpr int kTileM = 128;
constexpr int kHeaderBytes = 512;      // workspace: int status, int exponent[64]
constexpr uint32_t kSpinLimit = 1u << 22;

template <int BN, int TERMS>
struct Cfg {
    static constexpr int G = 8;                                // 32-code groups per shared-memory stage
    static constexpr int SK = G * 32;                          // codes of K per stage
    // padded FP4: 16 codes per 16-byte chunk; one chunk column = 128 rows x 16 B, plus 16 B so that the 16
    // lanes that copy one row's 16 chunks do not all hit the same shared-memory bank
    static constexpr int A_CHUNK = kTileM * 16 + 16;
    static constexpr int A_BYTES = 2 * G * A_CHUNK;
    // The issue rate of tcgen05.mma from one thread (~70 clk each, whatever N is) bounds the kernel, so as
    // few MMAs per group as possible: while TERMS x BN <= 48 columns the E4M3 terms sit side by side in N
    // (one MMA per group, the epilogue adds the term columns); beyond that they extend K (TERMS MMAs).
    static constexpr int TN = (TERMS * BN <= 48) ? TERMS : 1;  // terms laid out along N
    static constexpr int TK = TERMS / TN;                      // terms accumulated along K
    static constexpr int NW = TN * BN;                         // MMA N
    static constexpr int B_BYTES = G * TK * 2 * NW * 16;       // [group][k-term][chunk][n-term * BN + column][16 B]
    static constexpr int GA_ = 256 / NW;                       // groups whose accumulators fit one 256-column buffer
    static constexpr int GA = GA_ >= G ? G : (GA_ >= 4 ? 4 : (GA_ >= 2 ? 2 : 1));
    static constexpr int ROUNDS = G / GA;                      // accumulator rounds per stage
    static constexpr int TMEM_COLS = 512;
};

constexpr int kScaleBytes = kTileM * 16;  // per stage: 16 bytes (up to 8 fp16 group scales) per weight row

template <int BN, int TERMS>
__host__ __device__ constexpr int stage_bytes() { return Cfg<BN, TERMS>::A_BYTES + Cfg<BN, TERMS>::B_BYTES + kScaleBytes; }

template <int BN, int TERMS>
__host__ __device__ constexpr int stages() {
    // as many stages as fit in ~200 KB, at most 6
    return (200 * 1024) / stage_bytes<BN, TERMS>() > 6 ? 6 : (200 * 1024) / stage_bytes<BN, TERMS>();
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
// Bounded wait: false (and the CTA-wide error flag raised) when it gives up, after kSpinLimit polls or
// ~0.25 s of SM clock, whichever comes first.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *err) {
    const long long t0 = clock64();
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        if (mbar_try(bar, parity)) return true;
        if (*err) return false;
        if (i > 8192) {
            __nanosleep(64);  // back off only when the wait is clearly long: a sleeping waiter wakes late
            if (clock64() - t0 > 500000000LL) break;
        }
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

// tcgen05.ld of N consecutive fp32 columns of this thread's lane; the data is valid after tmem_wait()
template <int N>
__device__ __forceinline__ void tmem_ld(uint32_t taddr, uint32_t (&r)[N]);
template <>
__device__ __forceinline__ void tmem_ld<8>(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr));
}
template <>
__device__ __forceinline__ void tmem_ld<16>(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr));
}
template <>
__device__ __forceinline__ void tmem_ld<32>(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---- activation preparation -----------------------------------------------------
// x[B,K] -> (rotate) -> u = x * 2^-e with max|u| < 256 -> t1 = e4m3(u),
// t2 = e4m3(u - t1), t3 = e4m3(u - t1 - t2) -> bytes in the smem-ready layout
// [stage][group][k-term][chunk][n-term * BN + column][16] (see Cfg).  Columns >= B
// are zero.  One block per column.
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
    using C = Cfg<BN, TERMS>;
    constexpr int G = C::G, SK = C::SK;
    __shared__ float sred[8];
    __shared__ int sexp;
    const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    unsigned char *xq = ws + kHeaderBytes;
    int *hdr = reinterpret_cast<int *>(ws);
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
            const int tk = t / C::TN, tn = t % C::TN;
            const size_t idx = (((((size_t)st * G + g) * C::TK + tk) * 2 + ch) * C::NW + tn * BN + b) * 16 + off;
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
    int kparts;     // K is cut into this many equal parts, one work item per (row tile, part)
    float *parts;   // [kparts][B][N] fp32 partial outputs when kparts > 1
};

template <int BN, int TERMS>
__global__ void __launch_bounds__(kThreads, 1) gemm_e2m1_tc_kernel(TcArgs a) {
    using C = Cfg<BN, TERMS>;
    constexpr int G = C::G, SK = C::SK, S = stages<BN, TERMS>(), NW = C::NW, GA = C::GA, ROUNDS = C::ROUNDS, TK = C::TK, TN = C::TN;
    constexpr int A_BYTES = C::A_BYTES, B_BYTES = C::B_BYTES, STAGE = stage_bytes<BN, TERMS>();
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
            mbar_init(full0 + 8 * s, 128);  // 32 lanes of each of the 4 producer warps, arriving through cp.async completion
            mbar_init(empty0 + 8 * s, 8);   // the 8 epilogue warps, once the stage's last accumulator round is complete
                                            // (that implies its MMAs have read the stage; the warps have read the scales)
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(tfull0 + 8 * i, 1);   // one tcgen05.commit
            mbar_init(tempty0 + 8 * i, 8);  // one arrival per epilogue warp
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // the upper 8 bytes of every FP4 chunk are padding that no copy writes: keep them defined
    for (uint32_t i = tid; i < (uint32_t)(S * STAGE) / 16; i += kThreads)
        asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(smem_base + i * 16), "r"(0u) : "memory");
    if (warp == 4) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(C::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;

    const int ntiles = (a.N + kTileM - 1) / kTileM;
    const int nst = (a.K / SK) / a.kparts;   // stages per work item
    const int nitems = ntiles * a.kparts;    // item = tile * kparts + part
    const int ldw = a.K >> 1;                // bytes per packed row (K % 32 == 0 here)
    const int ngroups = a.K >> 5;
    const unsigned char *xq = a.ws + kHeaderBytes;

    if (warp < 4) {
        // ---- producers, four warps of 32 weight rows each.  16 lanes copy the 16 chunks (8 B) of one row's
        //      stage slice, so global reads coalesce; two rows per instruction.  Each warp also copies a
        //      quarter of the activation tile and its rows' group scales.
        uint32_t it = 0;
        const int c = lane & 15, rsub = lane >> 4;
        for (int item = blockIdx.x; item < nitems && !*err; item += gridDim.x) {
            const int tile = item / a.kparts, part = item % a.kparts;
            const bool full_tile = tile * kTileM + kTileM <= a.N;
            for (int st = 0; st < nst; ++st, ++it) {
                const int s = it % S;
                if (!mbar_wait(empty0 + 8 * s, ((it / S) & 1) ^ 1, err)) break;
                const uint32_t sa = smem_base + s * STAGE;
                uint32_t dst = sa + c * C::A_CHUNK + (warp * 32 + rsub) * 16;
                const size_t koff = (size_t)(part * nst + st) * (SK / 2) + c * 8;
                if (c < 2 * G) {
                    if (full_tile) {
                        const uint8_t *src = a.qw + (size_t)(tile * kTileM + warp * 32 + rsub) * ldw + koff;
                        const size_t step = (size_t)2 * ldw;
#pragma unroll 8
                        for (int rr = 0; rr < 16; ++rr) { cp_async8(dst, src); dst += 32; src += step; }
                    } else {
#pragma unroll 4
                        for (int rr = 0; rr < 16; ++rr) {
                            const int row = min(tile * kTileM + warp * 32 + rr * 2 + rsub, a.N - 1);
                            cp_async8(dst, a.qw + (size_t)row * ldw + koff);
                            dst += 32;
                        }
                    }
                }
                // a quarter of the stage's activation tile (one contiguous block of the prepared buffer)
                {
                    const unsigned char *src = xq + (size_t)(part * nst + st) * B_BYTES;
                    for (int i = warp * 32 + lane; i < B_BYTES / 16; i += 128) cp_async16(sa + A_BYTES + i * 16, src + (size_t)i * 16);
                }
                // this warp's 32 rows' group scales: G fp16 per row, to 16 bytes per row
                {
                    const int r = warp * 32 + lane;
                    const int row = min(tile * kTileM + r, a.N - 1);
                    const __half *sp = a.scales + (size_t)row * ngroups + (size_t)(part * nst + st) * G;
                    if (G == 8) cp_async16(sa + A_BYTES + B_BYTES + r * 16, sp);
                    else cp_async8(sa + A_BYTES + B_BYTES + r * 16, sp);
                }
                cp_async_arrive(full0 + 8 * s);
            }
        }
    } else if (warp < 4 + kMmaWarps) {
        // ---- MMA issuers: one thread in each of four warps; issuer w takes the stages it = w, w+4, ...
        //      Per stage an issuer spends ~0.7 us in serial latencies (two mbarrier waits, the tcgen05.mma
        //      issue itself at ~100 clk per instruction whatever its size, the commit); four issuers working on
        //      different stages overlap them.  Accumulator buffers and barrier phases follow the global stage
        //      and round counters, so the issuers need no ordering among themselves.
        const int w = warp - 4;
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc(kTileM, NW);
            uint32_t it = 0;
            for (int item = blockIdx.x; item < nitems && !*err; item += gridDim.x) {
                for (int st = 0; st < nst && !*err; ++st, ++it) {
                    if ((int)(it % kMmaWarps) != w) continue;
                    const int s = it % S;
                    const int ab = it & 1;                 // == w: this issuer's accumulator buffer
                    uint32_t pa = (it >> 1) * ROUNDS;      // rounds this buffer has seen so far
                    if (!mbar_wait(full0 + 8 * s, (it / S) & 1, err)) break;            // tiles landed
                    const uint32_t sa = smem_base + s * STAGE, sb = sa + A_BYTES;
#pragma unroll
                    for (int rd = 0; rd < ROUNDS; ++rd, ++pa) {
                        if (!mbar_wait(tempty0 + 8 * ab, (pa & 1) ^ 1, err)) break;  // accumulator buffer drained
                        tc_fence_after();
#pragma unroll
                        for (int gg = 0; gg < GA; ++gg) {
                            const int g = rd * GA + gg;
                            const uint64_t ad = smem_desc(sa + g * (2 * C::A_CHUNK), C::A_CHUNK, 128);
#pragma unroll
                            for (int tk = 0; tk < TK; ++tk) {
                                const uint64_t bd = smem_desc(sb + (g * TK + tk) * (2 * NW * 16), NW * 16, 128);
                                mma_f8f6f4(tmem + ab * 256 + gg * NW, ad, bd, idesc, tk > 0 ? 1u : 0u);
                            }
                        }
                        mma_commit(tfull0 + 8 * ab);   // this round's accumulators complete
                    }
                }
            }
        }
    } else if (warp >= 8) {
        // ---- epilogue, 8 warps: thread = one accumulator lane (weight row) x one half of the batch columns.
        //      The read of group g+1 from tensor memory is in flight while group g is scaled and added.
        const int q = warp & 3;                // tensor-memory lane quarter this warp may touch
        const int h = (warp - 8) >> 2;         // which half of the columns
        constexpr int CH = BN / 2;
        const int r = q * 32 + lane;
        const int *hdr = reinterpret_cast<const int *>(a.ws);
        uint32_t it = 0;
        for (int item = blockIdx.x; item < nitems && !*err; item += gridDim.x) {
            const int tile = item / a.kparts, part = item % a.kparts;
            const int row = tile * kTileM + r;
            float acc[CH];
#pragma unroll
            for (int b = 0; b < CH; ++b) acc[b] = 0.f;
            bool ok = true;
            for (int st = 0; st < nst && ok; ++st, ++it) {
                const int s = it % S, ab = it & 1;     // the stage's accumulator buffer (its issuer's)
                uint32_t pa = (it >> 1) * ROUNDS;
                float sc[G];  // this row's G scales of the stage, staged in shared memory by the producer
#pragma unroll
                for (int rd = 0; rd < ROUNDS; ++rd, ++pa) {
                    ok = __all_sync(0xffffffffu, mbar_wait(tfull0 + 8 * ab, pa & 1, err));  // warp-uniform outcome
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t tbase = tmem + ((uint32_t)(q * 32) << 16) + ab * 256 + h * CH;
                    uint32_t d[2][TN][CH];
#pragma unroll
                    for (int tn = 0; tn < TN; ++tn) tmem_ld<CH>(tbase + tn * BN, d[0][tn]);
                    if (rd == 0) {
                        // tfull of the first round implies the stage's copies have landed (the MMA thread saw 'full')
                        const uint32_t sp = smem_base + s * STAGE + A_BYTES + B_BYTES + r * 16;
                        uint32_t w[4];
                        if (G == 8) asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]) : "r"(sp));
                        else asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(w[0]), "=r"(w[1]) : "r"(sp));
#pragma unroll
                        for (int g = 0; g < G; ++g)
                            sc[g] = __half2float(__ushort_as_half((uint16_t)((g & 1) ? (w[g >> 1] >> 16) : (w[g >> 1] & 0xffffu))));
                    }
                    if (rd == ROUNDS - 1) {
                        __syncwarp();
                        if (lane == 0) mbar_arrive(empty0 + 8 * s);  // all MMAs of the stage are done and its scales are in registers
                    }
                    tmem_wait();
#pragma unroll
                    for (int gg = 0; gg < GA; ++gg) {
                        if (gg + 1 < GA) {
#pragma unroll
                            for (int tn = 0; tn < TN; ++tn) tmem_ld<CH>(tbase + (gg + 1) * NW + tn * BN, d[(gg + 1) & 1][tn]);
                        }
                        const float sg = sc[rd * GA + gg];
#pragma unroll
                        for (int i = 0; i < CH; ++i) {
                            float v = __uint_as_float(d[gg & 1][0][i]);
#pragma unroll
                            for (int tn = 1; tn < TN; ++tn) v += __uint_as_float(d[gg & 1][tn][i]);
                            acc[i] = fmaf(v, sg, acc[i]);
                        }
                        if (gg + 1 < GA) tmem_wait();
                    }
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(tempty0 + 8 * ab);
                }
            }
            if (!ok) break;
            if (row < a.N) {
                const float bias = (a.bias && a.kparts == 1) ? a.bias[row] : 0.f;
#pragma unroll
                for (int i = 0; i < CH; ++i) {
                    const int b = h * CH + i;
                    if (b < a.B) {
                        const float up = __uint_as_float((uint32_t)(127 + hdr[1 + b]) << 23);
                        const float v = fmaf(acc[i], up, bias);
                        if (a.kparts == 1) jq::store_out(a.y, (size_t)b * a.N + row, v, a.y_dtype);
                        else a.parts[((size_t)part * a.B + b) * a.N + row] = v;
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
    if (warp == 4) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(C::TMEM_COLS) : "memory");
    }
}

// y[b][n] = sum_p parts[p][b][n] + bias[n]
__global__ void __launch_bounds__(256) tc_reduce_kernel(const float *__restrict__ parts, int np, int B, int N,
                                                        const float *__restrict__ bias, void *__restrict__ y, int y_dtype) {
    const long long total = (long long)B * N;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        float acc = 0.f;
        for (int p = 0; p < np; ++p) acc += parts[(size_t)p * total + i];
        if (bias) acc += bias[i % N];
        jq::store_out(y, (size_t)i, acc, y_dtype);
    }
}

constexpr int kMaxKParts = 8;

template <int BN, int TERMS>
static int launch_tc(TcArgs a, const void *x, int had, int x_dtype, cudaStream_t st) {
    using C = Cfg<BN, TERMS>;
    if (a.K % C::SK) return JQ_ERR_UNSUPPORTED;
    // enough work items for every SM: cut K while the stage count divides evenly
    {
        const int ntiles_ = (a.N + kTileM - 1) / kTileM, nst_all = a.K / C::SK, sms = jq_sm_count();
        int kp = 1;
        while (kp < kMaxKParts && ntiles_ * kp < sms && nst_all % (kp * 2) == 0 && nst_all / (kp * 2) >= 4) kp *= 2;
        a.kparts = kp;
        a.parts = reinterpret_cast<float *>(a.ws + kHeaderBytes + ((size_t)3 * a.K * BN + 255) / 256 * 256);
    }
    constexpr int S = stages<BN, TERMS>();
    static_assert(S >= 2 && S <= 6, "stage count");
    const size_t smem = (size_t)S * stage_bytes<BN, TERMS>() + 128;
    tc_prepare_kernel<BN, TERMS><<<BN, 256, 0, st>>>(x, a.B, a.K, had, x_dtype, a.ws);
    int s = jq_launch_status();
    if (s) return s;
    auto kern = gemm_e2m1_tc_kernel<BN, TERMS>;
    JQ_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int nitems = ((a.N + kTileM - 1) / kTileM) * a.kparts;
    int grid = jq_sm_count();
    if (grid > nitems) grid = nitems;
    kern<<<grid, kThreads, smem, st>>>(a);
    s = jq_launch_status();
    if (s || a.kparts == 1) return s;
    const long long total = (long long)a.B * a.N;
    int blocks = (int)((total + 255) / 256);
    if (blocks > jq_sm_count() * 8) blocks = jq_sm_count() * 8;
    tc_reduce_kernel<<<blocks, 256, 0, st>>>(a.parts, a.kparts, a.B, a.N, a.bias, a.y, a.y_dtype);
    return jq_launch_status();
}

}  // namespace jqtc

using namespace jqtc;

static int tc_bn(int B) { return B <= 16 ? 16 : (B <= 32 ? 32 : 64); }
// bf16 has 8 significant bits = two E4M3 terms exactly; anything else gets three
static int tc_terms(int had, int x_dtype) { return (!had && x_dtype == JQ_BF16) ? 2 : 3; }

// header | prepared activation (3 terms x K x columns) | split-K partials
size_t jq_tc_workspace_bytes(int N, int K, int B) {
    if (B < 1 || B > 64 || K <= 0 || N <= 0) return 0;
    const size_t xq = ((size_t)3 * K * tc_bn(B) + 255) / 256 * 256;
    return (size_t)kHeaderBytes + xq + (size_t)kMaxKParts * B * N * sizeof(float);
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
    if (workspace_bytes < jq_tc_workspace_bytes(N, K, B)) return JQ_ERR_WORKSPACE;
    TcArgs a{reinterpret_cast<const uint8_t *>(qweight), reinterpret_cast<const __half *>(scales), bias, y,
             reinterpret_cast<unsigned char *>(workspace), N, K, B, y_dtype, 1, nullptr};
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const int bn = tc_bn(B), terms = tc_terms(had_block, x_dtype);
    if (bn == 16) return terms == 2 ? launch_tc<16, 2>(a, x, had_block, x_dtype, st) : launch_tc<16, 3>(a, x, had_block, x_dtype, st);
    if (bn == 32) return terms == 2 ? launch_tc<32, 2>(a, x, had_block, x_dtype, st) : launch_tc<32, 3>(a, x, had_block, x_dtype, st);
    return terms == 2 ? launch_tc<64, 2>(a, x, had_block, x_dtype, st) : launch_tc<64, 3>(a, x, had_block, x_dtype, st);
}

// A decode step's worth of batched layers in one host call: the launches of every problem are enqueued
// back to back on the stream, sharing one workspace (stream order keeps them apart).
extern "C" int jq_gemm_e2m1_tc_multi(const jq_problem *problems_host, int n, int B, int x_dtype, int y_dtype,
                                     void *workspace, size_t workspace_bytes, jq_stream_t stream) {
    if (!problems_host || !workspace) return JQ_ERR_NULL_PTR;
    if (n <= 0) return JQ_ERR_BAD_SHAPE;
    for (int i = 0; i < n; ++i) {
        const jq_problem &p = problems_host[i];
        if (p.ldy != 0 && p.ldy != p.N) return JQ_ERR_UNSUPPORTED;
        int st = jq_gemm_e2m1_tc(p.qweight, p.scales, p.x, p.bias, p.y, p.N, p.K, B, p.g, p.had_block, x_dtype, y_dtype,
                                 workspace, workspace_bytes, stream);
        if (st) return st;
    }
    return JQ_OK;
}

// Status word of the jq_gemm_e2m1_tc calls that used this workspace since it was last read: 0 = fine,
// JQ_ERR_TIMEOUT if a device-side wait gave up in any of them (kernels only raise the word, they never reset
// it; this call clears it after reading).  The word must be zero before the workspace's first use.
// Synchronises the stream.
extern "C" int jq_tc_status(const void *workspace, jq_stream_t stream) {
    if (!workspace) return JQ_ERR_NULL_PTR;
    int v = 0;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    JQ_CUDA_TRY(cudaMemcpyAsync(&v, workspace, sizeof(int), cudaMemcpyDeviceToHost, st));
    JQ_CUDA_TRY(cudaStreamSynchronize(st));
    if (v) JQ_CUDA_TRY(cudaMemsetAsync(const_cast<void *>(workspace), 0, sizeof(int), st));
    return v;
}

// ---- bounded-wait self test ------------------------------------------------------
// One CTA waits, with the same bounded wait the pipeline uses, on an mbarrier
// that nothing ever arrives on.  The wait has to give up, raise the status
// word and let the kernel return; the device stays usable.  (This is how the
// failure path is exercised without faulting or hanging a GPU.)
namespace jqtc {
__global__ void __launch_bounds__(64) bounded_wait_selftest_kernel(int *status, uint32_t limit) {
    __shared__ __align__(8) uint64_t bar;
    __shared__ int s_err;
    if (threadIdx.x == 0) {
        s_err = 0;
        mbar_init(smem_u32(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    volatile int *err = &s_err;
    bool ok = true;
    if (threadIdx.x == 32) {          // one waiter; nobody arrives
        ok = false;
        for (uint32_t i = 0; i < limit; ++i) {
            if (mbar_try(smem_u32(&bar), 0)) { ok = true; break; }
            if (i > 64) __nanosleep(64);
        }
        if (!ok) *err = JQ_ERR_TIMEOUT;
    }
    __syncthreads();
    if (threadIdx.x == 0) *status = s_err;
}
}  // namespace jqtc

extern "C" int jq_selftest_bounded_wait(int *status_dev, unsigned int polls, jq_stream_t stream) {
    if (!status_dev) return JQ_ERR_NULL_PTR;
    if (polls == 0 || polls > (1u << 20)) return JQ_ERR_BAD_SHAPE;   // at most ~0.1 s of polling
    jqtc::bounded_wait_selftest_kernel<<<1, 64, 0, reinterpret_cast<cudaStream_t>(stream)>>>(status_dev, polls);
    return jq_launch_status();
}
