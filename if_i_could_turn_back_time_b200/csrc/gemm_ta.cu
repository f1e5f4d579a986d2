// Packed 4-bit weights x activations on the 5th-generation tensor cores with
// the decoded weights handed over in tensor memory (tcgen05, sm_100a).
//
// One persistent CTA per SM works through 128-row tiles of the weight matrices.
// A decode thread owns one weight row of the tile (= one tensor-memory lane)
// and one half of the 256-code steps of that row:
//   * the packed codes of a warp's 32 rows arrive by TMA (cp.async.bulk.tensor,
//     one 32-row x 128-byte box per step with the 128-byte swizzle, completion
//     counted on an mbarrier), so that every lane reads its own row without
//     bank conflicts;
//   * GF4: a byte (two codes) indexes the row's 256-entry table of fp16 pairs,
//     built once per tile in a shared-memory column that only this lane's bank
//     serves (one conflict-free 32-bit lookup per two codes, the address formed
//     by one dp4a); E2M1: cvt.rn.f16x2.e2m1x2 per byte, times the group's fp16
//     scale in fp16x2;
//   * the fp16 values go to tensor memory with tcgen05.st as the A operand
//     (M = 128 rows, K = 16 per instruction) of tcgen05.mma kind::f16; the B
//     operand is the prepared activation (rotated, normalised by a power of
//     two, fp16, in the K-major core-matrix layout) that each MMA-issuing
//     thread streams from global memory into a ring of its own, one 128-code
//     chunk per bulk copy;
//   * GF4 keeps one fp32 accumulator per 128-code scale group in tensor memory;
//     the thread reads its row's sums back with tcgen05.ld and applies the
//     group's fp16 scale in fp32, so every product and every scale stays exact
//     (the results differ from the FMA kernels only in summation order).
//     E2M1 folds the scale into the fp16 weight (one rounding per weight) and
//     accumulates the whole row in one accumulator per issuing thread.
// The multiply-accumulate work thus costs the CUDA cores nothing, whatever the
// batch (up to 64 columns per pass), and the lookups are halved.
//
// Every wait on an mbarrier is bounded: on expiry the CTA raises a status word
// in the workspace, all roles leave their loops, tensor memory is freed and
// the kernel returns.  Nothing traps or spins without a limit.
#include "common.cuh"
#include <cuda.h>
#include <mutex>
#include <string.h>

namespace jqta {

constexpr int kDecodeWarps = 8;              // warps 0-3: first half of the steps, warps 4-7: second half
constexpr int kTileM = 128;
constexpr int kWStage = 32 * 128;            // bytes of a weight stage: 32 rows x 128 bytes (256 codes), swizzled by TMA
constexpr int kXMaxStages = 8;               // stages of an MMA issuer's activation ring, at most
constexpr int kTabBytes = 4 * 256 * 128;     // GF4: 256 entries x 32 lanes x 4 bytes per 32-row quarter
constexpr uint32_t kSpinLimit = 1u << 22;
constexpr int kHeaderBytes = 1024;           // workspace: int status

struct TaProblem {
    const uint8_t *qw;
    const __half *scales;
    const __half *codebook;
    const void *x;          // activations [B, K] as the caller gave them
    const float *bias;
    void *y;
    __half *xprep;          // prepared activation: [K / 8][B rows][8 halves]
    float *xscale;          // [B] 2^e of each batch row (the power of two taken out before rounding to fp16)
    int N, K, g, had;
    int ldw;                // bytes between packed rows
    int lds;                // scales between rows
    int ldy;                // outputs between batch rows
    int tile0;              // first tile of this problem in the launch's tile sequence
};

struct PeerInfo {
    int n;
    long long delta[8];
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("{ .reg .b64 t; mbarrier.arrive.shared::cta.b64 t, [%0]; }" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("{ .reg .b64 t; mbarrier.arrive.expect_tx.shared::cta.b64 t, [%0], %1; }" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: false (and the CTA-wide error flag raised) when it gives up, after kSpinLimit polls or
// about 0.25 s of SM clock, whichever comes first; also false as soon as another thread has raised the flag.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *err) {
    if (mbar_try(bar, parity)) return true;
    const long long t0 = clock64();
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        if (mbar_try(bar, parity)) return true;
        if (*err) return false;
        if (i > 8192) {
            __nanosleep(64);
            if (clock64() - t0 > 500000000LL) break;
        }
    }
    *err = JQ_ERR_TIMEOUT;
    return false;
}
// global -> shared bulk copy (16-byte aligned, a multiple of 16 bytes); its bytes are counted on the mbarrier
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// 2-D tiled TMA load: box at (x bytes, y rows) of the tensor map -> shared memory; x must be a multiple of 16
__device__ __forceinline__ void tma_2d_g2s(uint32_t dst, const void *tmap, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(tmap), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void tma_2d_prefetch_l2(const void *tmap, int x, int y) {
    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global [%0, {%1, %2}];" ::"l"(tmap), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// K-major operand in shared memory without swizzle: 8 rows x 16 bytes are contiguous; lbo = bytes between
// the two 16-byte K chunks of one MMA, sbo = bytes between 8-row groups (bits 46-47 = 1: sm_100 descriptor).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = 0;
    d |= (uint64_t)((addr >> 4) & 0x3fffu);
    d |= (uint64_t)((lbo >> 4) & 0x3fffu) << 16;
    d |= (uint64_t)((sbo >> 4) & 0x3fffu) << 32;
    d |= (uint64_t)1 << 46;
    return d;
}
// kind::f16 instruction descriptor: D = fp32, A = B = fp16, both K-major
__host__ __device__ constexpr uint32_t idesc_f16(int M, int N) {
    return (1u << 4) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
// D[128 x N] (+)= A[128 x 16] (tensor memory) . B[N x 16]^T (shared memory)
__device__ __forceinline__ void mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{ .reg .pred p; setp.ne.b32 p, %4, 0;\n"
                 "  tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p; }"
                 ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr));
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t dp4a_u(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// Programmatic dependent launch: the main kernels are launched while the activation preparation in front of them
// is still running; everything they do before pdl_wait() (barrier set-up, problem look-ups, the first weight boxes)
// overlaps it, everything that reads the prepared activation comes after.  Without the launch attribute both are
// no-ops.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// e with amax * 2^-e below 2^15 after the rotation's worst-case growth (the rule of the GEMV kernels)
__device__ __forceinline__ int act_exponent(float amax, bool had) {
    uint32_t bits = __float_as_uint(amax);
    int field = (bits >> 23) & 0xff;
    if (field == 0xff || (bits & 0x7fffffffu) == 0) return 0;
    int e = field - 127 - (had ? 10 : 14);
    return max(-100, min(100, e));
}

// ---- activation preparation -----------------------------------------------------
// One block per (problem, batch row): x -> (x 2^-e) -> block Hadamard -> fp16, written as
// [8-code piece][batch row][8 halves].  Copied to shared memory as it is, this is the K-major operand
// layout of the MMA with a piece stride of 16 B bytes: row n of piece c sits at (c B + n) 16 bytes.  The MMA
// always reads 16 rows; rows >= B are whatever follows (the next pieces), and their accumulator columns
// are never read.
// The second pass is a chain of load -> rotate -> store per 128-element block and warp, and its latency is what a
// decode step waits for before the main kernel can start.  With one or two batch rows there are few blocks: 32 warps
// each (K = 11008: 3 rounds instead of 11; 4.5 us less per 7B-shaped step).  With many batch rows 8 warps per block
// keep more rows resident per SM.
template <int kPrepThreads>
__global__ void __launch_bounds__(kPrepThreads) ta_prepare_kernel(const TaProblem *probs, TaProblem single, int B,
                                                                   int x_dtype) {
    constexpr int kWarps = kPrepThreads / 32;
    __shared__ float sred[kWarps];
    __shared__ int sexp;
    pdl_launch_dependents();
    const int pi = blockIdx.x / B, b = blockIdx.x % B;
    const TaProblem p = probs ? probs[pi] : single;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float m = 0.f;
    for (int k = tid; k < p.K; k += kPrepThreads) m = fmaxf(m, fabsf(jq::load_act(p.x, (size_t)b * p.K + k, x_dtype)));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) sred[warp] = m;
    __syncthreads();
    if (warp == 0) {
        float mm = lane < kWarps ? sred[lane] : 0.f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, o));
        if (lane == 0) {
            sexp = act_exponent(mm, p.had != 0);
            p.xscale[b] = __uint_as_float((uint32_t)(127 + sexp) << 23);
        }
    }
    __syncthreads();
    const float down = __uint_as_float((uint32_t)(127 - sexp) << 23);
    for (int blk = warp; blk * 128 < p.K; blk += kWarps) {
        float v[4];
        const int k0 = blk * 128 + lane * 4;
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] = jq::load_act(p.x, (size_t)b * p.K + k0 + j, x_dtype) * down;
        if (p.had) jq::fwht128_warp(v, lane);
        __half2 h01 = __floats2half2_rn(v[0], v[1]), h23 = __floats2half2_rn(v[2], v[3]);
        const size_t off = (((size_t)blk * 16 + (lane >> 1)) * B + b) * 8 + (lane & 1) * 4;
        *reinterpret_cast<uint2 *>(p.xprep + off) =
            make_uint2(*reinterpret_cast<uint32_t *>(&h01), *reinterpret_cast<uint32_t *>(&h23));
    }
}

// ---- main kernel --------------------------------------------------------------------
// Roles of a CTA (12 warps): warps 0-7 decode (warp = 32-row quarter q of the tile x half h of the 256-code
// steps of a row: step sg belongs to half sg & 1); lane 0 of warps 8-11 issues MMAs (two issuers per half:
// a thread cannot issue a tcgen05.mma more often than every 50 clocks, threads of different warps can) and
// streams the prepared activation of its own groups; warp 11 also owns the tensor-memory allocation.  The
// two halves are independent pipelines that meet at the end of a tile.
//
// Tensor-memory columns: kRing slots per half of 64 columns each for the A operand (one 128-code group);
// GF4 adds NB accumulator columns to every slot (one accumulator per group: the group's fp16 scale is
// applied in fp32 after tcgen05.ld), E2M1 has one accumulator of NB columns per issuer for the whole row
// (its scales are folded into the fp16 weights).  The second half's sums reach the first half's threads at
// the end of a tile through NB more columns (GF4) or through shared memory (E2M1, which needs all 512
// columns at 32 and 64 rows).
//
// Where the time goes (clock64 counters per role, 11008 x 4096 GF4 and 8192 x 8192 E2M1, 16 batch rows): the
// decode threads are busy decoding for about 60 % of a tile (GF4: the shared-memory pipe, 80 wavefronts per
// 128 codes of 32 rows, is 3/4 full while they do; E2M1: about 230 instructions per 128 codes and thread),
// the rest goes to the table build, the accumulator read-back and the end of the tile; neither the weight
// ring nor the activation rings are waited for (deepening the weight ring to four stages changed nothing).
// The MMA issuers are single lanes running dependent scalar code beside two decode warps: while they still
// divided their ring positions out of counters they were the bottleneck of E2M1 (busy 89 % of the time, half
// of it bookkeeping; with the MMAs left out the kernel ran 17 % faster); with the positions carried along
// E2M1 runs at that decode bound, and GF4's issuers idle 3/4 of the time.
constexpr int kTaThreads = 12 * 32;
template <int FMT, int NB>
struct Cols {
    static constexpr bool kGf4 = FMT == JQ_FMT_GF4;
    // MMA issuers per half.  One thread issues a tcgen05.mma every 50 clocks at best, whatever N up to 32 and
    // whatever the accumulator; threads of different warps issue in parallel.  At N = 64 two issuers already
    // saturate the pipe's arithmetic.
    static constexpr int kIssuers = (!kGf4 && NB == 64) ? 1 : 2;
    static constexpr int kRing = 3;                                // groups a half may have in flight
    static constexpr int kSlot = 64 + (kGf4 ? NB : 0);
    static constexpr int kAcc = 2 * kRing * kSlot;                 // E2M1: accumulator of (half h, issuer i) at kAcc + (h * kIssuers + i) * NB
    // GF4 hands the second half's sums to the first half's threads through NB more columns; E2M1 needs all 512
    // columns at 32 and 64 rows and uses shared memory for that (GF4 has none to spare)
    static constexpr int kExchange = kAcc;
    static_assert(kGf4 ? kExchange + NB <= 512 : kAcc + 2 * kIssuers * NB <= 512, "tensor memory");
};

template <int FMT>
struct Smem {
    static constexpr bool kGf4 = FMT == JQ_FMT_GF4;
    static constexpr int kTab = 0;
    static constexpr int kWRing = kGf4 ? kTabBytes : 0;
    static constexpr int kSW = 2;       // stages of a decode warp's weight ring (four did not change anything: the ring is not what the decode threads wait for)
    static constexpr int kXRing = kWRing + kDecodeWarps * kSW * kWStage;
    static constexpr int kXBytes = kGf4 ? 32 * 1024 : 96 * 1024;    // E2M1 has no tables: three stages of 64 batch rows per issuer
    static constexpr int kExch = kXRing + kXBytes + 512;            // + what the MMA reads past the last chunk (rows >= B)
    static constexpr int kExchBytes = kGf4 ? 0 : 2 * kTileM * 64 * 4;   // E2M1: second half's sums, [tile parity][batch row][tile row] fp32
    static constexpr int kBars = kExch + kExchBytes;
    static constexpr int kNumBars = kDecodeWarps * 4 + 4 * 3 + 2 * 4 * kXMaxStages + 4;   // weights, A full, MMAs done, x full/free per issuer, quarter sync
    static constexpr int kBytes = kBars + kNumBars * 8 + 1024;      // + slack for the 1 KB alignment of the base (TMA swizzle)
};

// geometry of an issuer's activation ring for a batch of B rows: a stage is one group (128 codes), 256 B bytes
struct XGeom {
    int chunk, ring, nstages, lag;
    __host__ __device__ XGeom(int B, int ring_bytes) {
        chunk = 256 * B;
        ring = ring_bytes;
        nstages = ring_bytes / chunk < kXMaxStages ? ring_bytes / chunk : kXMaxStages;
        lag = nstages > 2 ? 2 : 1;      // a stage is refilled this many groups after the MMAs that read it were issued
    }
};

template <int FMT, int NB>
__global__ void __launch_bounds__(kTaThreads, 1) gemm_ta_kernel(const TaProblem *probs, const CUtensorMap *maps,
                                                                const __grid_constant__ TaProblem single,
                                                                const __grid_constant__ CUtensorMap single_map, int nprob,
                                                                const int *tile_start, const int *cta_first,
                                                                int B, int y_dtype, PeerInfo peers, int *status) {
    using C = Cols<FMT, NB>;
    using S = Smem<FMT>;
    constexpr bool kGf4 = FMT == JQ_FMT_GF4;
    constexpr int kRing = C::kRing;
    constexpr int kSW = S::kSW;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ uint32_t s_tmem;
    __shared__ int s_err;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bars = sbase + S::kBars;
    auto wbar = [&](int w, int s) { return bars + 8u * (w * kSW + s); };
    auto abar = [&](int h, int s) { return bars + 8u * (kDecodeWarps * kSW + h * 3 + s); };
    auto dbar = [&](int h, int s) { return bars + 8u * (kDecodeWarps * kSW + 6 + h * 3 + s); };
    auto xbar = [&](int iss, int s) { return bars + 8u * (kDecodeWarps * kSW + 12 + iss * kXMaxStages + s); };           // issuer's stage filled
    auto xebar = [&](int iss, int s) { return bars + 8u * (kDecodeWarps * kSW + 12 + (4 + iss) * kXMaxStages + s); };    // its MMAs have read it
    auto qbar = [&](int q) { return bars + 8u * (kDecodeWarps * kSW + 12 + 8 * kXMaxStages + q); };
    volatile int *err = &s_err;
    const XGeom xg(B, S::kXBytes / (2 * C::kIssuers));

    if (tid == 0) {
        s_err = 0;
        for (int w = 0; w < kDecodeWarps; ++w)
            for (int s = 0; s < kSW; ++s) mbar_init(wbar(w, s), 1);     // one arrive.expect_tx per fill
        for (int h = 0; h < 2; ++h)
            for (int s = 0; s < 3; ++s) {
                mbar_init(abar(h, s), 128);                             // the 128 decode threads of the half
                mbar_init(dbar(h, s), 1);                               // one tcgen05.commit
            }
        for (int i = 0; i < 4; ++i)
            for (int s = 0; s < kXMaxStages; ++s) { mbar_init(xbar(i, s), 1); mbar_init(xebar(i, s), 1); }
        for (int q = 0; q < 4; ++q) mbar_init(qbar(q), 64);             // the two warps that share a quarter of the rows
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 11) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;

    // this CTA's tiles
    int tile_lo, tile_hi;
    if (nprob == 0) {   // one problem, passed by value: an even split of its tiles
        const int nt = (single.N + kTileM - 1) / kTileM;
        tile_lo = (int)((long long)nt * blockIdx.x / gridDim.x);
        tile_hi = (int)((long long)nt * (blockIdx.x + 1) / gridDim.x);
    } else {
        tile_lo = cta_first[blockIdx.x];
        tile_hi = cta_first[blockIdx.x + 1];
    }
    // Problems change rarely along a CTA's tile sequence: every walker keeps what it needs of its current
    // problem in registers and goes back to global memory only for a tile beyond that problem's last one.
    auto problem_at = [&](int &pi, int &t_end, int tile, TaProblem &p) {
        if (nprob == 0) { p = single; t_end = 0x7fffffff; return; }
        if (t_end < 0) {
            // first look-up of a walker: bisect (a step's list can hold hundreds of problems, and a scan from the
            // first one is a chain of dependent global loads, 0.2 us each, in front of the last CTAs' first tile)
            int lo = 0, hi = nprob - 1;
            while (lo < hi) {
                const int mid = (lo + hi + 1) >> 1;
                if (tile_start[mid] <= tile) lo = mid; else hi = mid - 1;
            }
            pi = lo;
        } else {
            while (pi + 1 < nprob && tile_start[pi + 1] <= tile) ++pi;
        }
        p = probs[pi];
        t_end = tile_start[pi + 1];
    };

    if (warp < kDecodeWarps) {
        // =============================== decode threads ===============================
        const int q = warp & 3, h = warp >> 2;
        const int r = q * 32 + lane;                       // row of the tile = tensor-memory lane
        const uint32_t lane_t = tmem + ((uint32_t)(q * 32) << 16);
        const uint32_t tcol = sbase + S::kTab + q * (256 * 128) + lane * 4;   // GF4: entry e of this row at tcol + 128 e
        const uint32_t wring = sbase + S::kWRing + warp * (kSW * kWStage);     // + stage * kWStage; 1 KB aligned
        // 16-byte piece c of this lane's row sits at piece c ^ (lane & 7) of the row (128-byte swizzle)
        const uint32_t lrow = lane * 128, lkey = (lane & 7) << 4;

        // ---- producer side of the weight ring: the (tile, step) whose box is requested next
        int i_tile = tile_lo, i_pi = 0, i_tend = -1, i_j = 0, i_n = 0, i_x = 0, i_y = 0, i_tile0 = 0, i_steps = 0, i_stage = 0;
        const void *i_map = nullptr;
        auto i_open = [&]() {
            while (i_tile < tile_hi) {
                if (i_tile >= i_tend) {
                    TaProblem p;
                    problem_at(i_pi, i_tend, i_tile, p);
                    i_steps = ((p.K >> 8) - h + 1) >> 1;
                    i_tile0 = p.tile0;
                    i_map = nprob ? &maps[i_pi] : &single_map;
                }
                i_n = i_steps;
                i_x = h * 128;
                i_y = (i_tile - i_tile0) * kTileM + q * 32;     // rows past N read as zeros
                i_j = 0;
                if (i_n > 0) return;
                ++i_tile;
            }
        };
        auto issue = [&]() {
            if (i_tile < tile_hi) {
                if (lane == 0) {
                    const uint32_t bar = wbar(warp, i_stage);
                    mbar_expect_tx(bar, kWStage);
                    tma_2d_g2s(wring + i_stage * kWStage, i_map, i_x, i_y, bar);
                }
                i_x += 256;
                if (++i_j == i_n) { ++i_tile; i_open(); }
            }
            i_stage = (i_stage + 1 == kSW) ? 0 : i_stage + 1;
        };
        i_open();
#pragma unroll
        for (int s = 0; s < kSW; ++s) issue();

        // ---- per-row side data one tile ahead: GF4 codebook row
        int f_pi = 0, f_tend = -1, f_tile0 = 0, f_N = 1;
        const __half *f_cb = nullptr;
        uint4 cb0 = make_uint4(0, 0, 0, 0), cb1 = cb0;
        auto fetch_codebook = [&](int tile) {
            if (kGf4 && tile < tile_hi) {
                if (tile >= f_tend) {
                    TaProblem p;
                    problem_at(f_pi, f_tend, tile, p);
                    f_tile0 = p.tile0; f_N = p.N; f_cb = p.codebook;
                }
                const int row = min((tile - f_tile0) * kTileM + r, f_N - 1);
                const uint4 *src = reinterpret_cast<const uint4 *>(f_cb + (size_t)row * 16);
                cb0 = __ldg(src);
                cb1 = __ldg(src + 1);
            }
        };

        // ---- consumer state
        uint32_t wcount = 0;        // weight stages consumed so far
        uint32_t t_h = 0;           // groups this half has handed to the MMA so far
        uint32_t t_fold = 0;        // groups whose slot has been released (GF4: folded into acc) so far
        uint32_t qcount = 0;        // quarter syncs so far
        unsigned short raw_q[3] = {0, 0, 0};   // GF4: fp16 scales (bits) of the groups in flight, by slot
        float acc[NB];
        bool have_prev = false;     // a finished tile waiting for its last group and its outputs
        float prev_bias = 0.f;
        int prev_row = 0, prev_N = 0, prev_ldy = 0;
        void *prev_y = nullptr;
        float prev_xs[(NB + 31) / 32];   // lane l holds 2^e of batch rows l, l + 32 (loaded at the start of the tile)

        uint32_t fin_count = 0;     // finished tiles so far (parity picks the E2M1 exchange buffer)
        int pend_slot = -1;         // slot of the group whose tensor-memory stores are issued but not yet handed over
        auto hand_over = [&]() {
            if (pend_slot >= 0) {
                tmem_wait_st();
                tc_fence_before();
                mbar_arrive(abar(h, (uint32_t)pend_slot));
                pend_slot = -1;
            }
        };
        auto quarter_sync = [&]() -> bool {
            mbar_arrive(qbar(q));
            const bool ok = mbar_wait(qbar(q), qcount & 1, err);
            ++qcount;
            return ok;
        };
        // release the oldest slot in flight: wait for its group's MMAs; GF4 folds the group's accumulator (scaled)
        auto fold_one = [&]() -> bool {
            const uint32_t s = t_fold % kRing;
            const bool ok = __all_sync(0xffffffffu, mbar_wait(dbar(h, s), (t_fold / kRing) & 1, err));
            if (!ok) return false;
            if constexpr (kGf4) {
                tc_fence_after();
                unsigned short raw = raw_q[0];
#pragma unroll
                for (int i = 1; i < kRing; ++i) raw = (s == (uint32_t)i) ? raw_q[i] : raw;
                const float sc = __half2float(__ushort_as_half(raw));
#pragma unroll
                for (int c = 0; c < NB; c += 16) {
                    uint32_t d[16];
                    tmem_ld16(lane_t + (h * kRing + s) * C::kSlot + 64 + c, d);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 16; ++i) acc[c + i] = fmaf(__uint_as_float(d[i]), sc, acc[c + i]);
                }
            }
            ++t_fold;
            return true;
        };
        // outputs of the finished tile: the second half hands its sums over through tensor memory
        auto finish_prev = [&]() -> bool {
            if (!have_prev) return true;
            while (t_fold < t_h)
                if (!fold_one()) return false;
            if constexpr (!kGf4) {          // the accumulators of the half's issuers hold the whole row between them
                tc_fence_after();
#pragma unroll
                for (int c = 0; c < NB; c += 16) {
#pragma unroll
                    for (int is = 0; is < C::kIssuers; ++is) {
                        uint32_t d[16];
                        tmem_ld16(lane_t + C::kAcc + (h * C::kIssuers + is) * NB + c, d);
                        tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 16; ++i) acc[c + i] = is ? acc[c + i] + __uint_as_float(d[i]) : __uint_as_float(d[i]);
                    }
                }
            }
            // E2M1: two buffers by tile parity, so that the second half (which does not meet the first again until
            // the end of the next tile) never overwrites sums that are still to be read; column b of the buffer is
            // 128 consecutive floats, one per tile row: conflict-free for a warp
            float *exch = reinterpret_cast<float *>(smem_raw + (sbase - smem_u32(smem_raw)) + S::kExch) +
                          (fin_count & 1) * (kTileM * 64) + r;
            ++fin_count;
            if (h == 1) {
                if constexpr (kGf4) {
#pragma unroll
                    for (int c = 0; c < NB; c += 16) {
                        uint32_t v[16];
#pragma unroll
                        for (int i = 0; i < 16; ++i) v[i] = __float_as_uint(acc[c + i]);
                        tmem_st16(lane_t + C::kExchange + c, v);
                    }
                    tmem_wait_st();
                } else {
#pragma unroll
                    for (int b = 0; b < NB; ++b)
                        exch[b * kTileM] = acc[b];
                }
            }
            tc_fence_before();
            if (!quarter_sync()) return false;
            if (h == 0) {
                tc_fence_after();
                const bool live = prev_row < prev_N;
#pragma unroll
                for (int c = 0; c < NB; c += 16) {
                    uint32_t v[16];
                    if constexpr (kGf4) {
                        tmem_ld16(lane_t + C::kExchange + c, v);
                        tmem_wait_ld();
                    } else {
#pragma unroll
                        for (int i = 0; i < 16; ++i) v[i] = __float_as_uint(exch[(c + i) * kTileM]);
                    }
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const int b = c + i;
                        const float xs_b = __shfl_sync(0xffffffffu, prev_xs[b >> 5], b & 31);
                        acc[b] = fmaf(acc[b] + __uint_as_float(v[i]), xs_b, prev_bias);
                    }
                }
                if (live) {
                    for (int cpy = 0; cpy < peers.n; ++cpy) {
                        char *yb = reinterpret_cast<char *>(prev_y) + jq::peer_offset(peers.delta, cpy);
#pragma unroll
                        for (int b = 0; b < NB; ++b)
                            if (b < B) jq::store_out(yb, (size_t)b * prev_ldy + prev_row, acc[b], y_dtype);
                    }
                }
                tc_fence_before();
            }
            have_prev = false;
            return true;
        };

        // scales of one 256-code step of a row: E2M1 eight fp16 (16 bytes), GF4 one fp16 per 128 * 2^k codes (.x, .y)
        auto load_scales = [&](const unsigned short *srow, int sg, int gshift) -> uint4 {
            if constexpr (kGf4)
                return make_uint4(__ldg(srow + ((2 * sg) >> gshift)), __ldg(srow + ((2 * sg + 1) >> gshift)), 0, 0);
            else
                return __ldg(reinterpret_cast<const uint4 *>(srow + sg * 8));
        };

        int c_pi = 0, c_tend = -1;
        TaProblem p = single;
        fetch_codebook(tile_lo);
        pdl_wait();                 // from here on the prepared activation and its row factors are read
        bool ok = true;
        for (int tile = tile_lo; tile < tile_hi && ok; ++tile) {
            if (tile >= c_tend) problem_at(c_pi, c_tend, tile, p);
            const int row_raw = (tile - p.tile0) * kTileM + r;
            const int row = min(row_raw, p.N - 1);
            const int nsteps = ((p.K >> 8) - h + 1) >> 1;
            const unsigned short *srow = reinterpret_cast<const unsigned short *>(p.scales) + (size_t)row * p.lds;
            const int gshift = kGf4 ? 31 - __clz(p.g >> 7) : 0;   // GF4: log2 of the 128-code groups per scale
            uint4 sc_nxt = load_scales(srow, h, gshift);          // in flight during the table build / the previous tile's outputs
            if constexpr (kGf4) {
                // ---- the pair table of this row (this thread fills the entries whose second code is in its half)
                if (!(ok = quarter_sync())) break;      // both warps are done with the previous tile's lookups
                const uint32_t c[8] = {cb0.x, cb0.y, cb0.z, cb0.w, cb1.x, cb1.y, cb1.z, cb1.w};
                uint32_t ch[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) ch[i] = h ? c[4 + i] : c[i];
                const uint32_t tb = tcol + h * (128 * 128);
#pragma unroll
                for (int i = 0; i < 8; ++i)
#pragma unroll
                    for (int lo = 0; lo < 16; ++lo) {
                        const uint32_t e = __byte_perm(c[lo >> 1], ch[i >> 1],
                                                       ((lo & 1) ? 0x32u : 0x10u) | (((i & 1) ? 0x76u : 0x54u) << 8));
                        asm volatile("st.shared.u32 [%0], %1;" ::"r"(tb + (i * 16 + lo) * 128), "r"(e) : "memory");
                    }
                fetch_codebook(tile + 1);
            }
            // the previous tile's last groups have had the table build to finish; its sync also publishes the table
            const bool had_prev = have_prev;
            if (!(ok = finish_prev())) break;
            if (kGf4 && !had_prev) { if (!(ok = quarter_sync())) break; }
#pragma unroll
            for (int b = 0; b < NB; ++b) acc[b] = 0.f;

            float xs_next[(NB + 31) / 32];
#pragma unroll
            for (int i = 0; i < (NB + 31) / 32; ++i) xs_next[i] = (lane + 32 * i < B) ? p.xscale[lane + 32 * i] : 0.f;
            for (int j = 0; j < nsteps && ok; ++j) {
                const int stage = wcount % kSW;
                ok = __all_sync(0xffffffffu, mbar_wait(wbar(warp, stage), (wcount / kSW) & 1, err));
                if (!ok) break;
                ++wcount;
                const uint32_t slot = wring + stage * kWStage + lrow;
                // the step's scales were loaded a step ahead; the next step's start their way now
                const uint4 sc_cur = sc_nxt;
                if (j + 1 < nsteps) sc_nxt = load_scales(srow, 2 * (j + 1) + h, gshift);
#pragma unroll
                for (int gi = 0; gi < 2; ++gi) {
                    // this group's scales: GF4 one fp16 (per 128 * 2^k codes), E2M1 four (one per 32 codes)
                    const unsigned short scale_raw = (unsigned short)(gi ? sc_cur.y : sc_cur.x);
                    const uint2 sc4 = gi ? make_uint2(sc_cur.z, sc_cur.w) : make_uint2(sc_cur.x, sc_cur.y);
                    // slot t % kRing is free once group t - kRing has been released
                    if (t_h - t_fold == (uint32_t)kRing && !(ok = fold_one())) break;
                    const uint32_t t = t_h, s = t % kRing;
                    const uint32_t a_t = lane_t + (h * kRing + s) * C::kSlot;
                    uint4 w4[4];
#pragma unroll
                    for (int part = 0; part < 4; ++part) w4[part] = lds128(slot + (((gi * 4 + part) << 4) ^ lkey));
                    // 32 codes (four words) -> 16 fp16 pairs
                    auto decode16 = [&](int part, uint32_t (&v)[16]) {
#pragma unroll
                        for (int wi = 0; wi < 4; ++wi) {
                            const uint32_t w = wi == 0 ? w4[part].x : (wi == 1 ? w4[part].y : (wi == 2 ? w4[part].z : w4[part].w));
                            if constexpr (kGf4) {
#pragma unroll
                                for (int bj = 0; bj < 4; ++bj) v[wi * 4 + bj] = lds32(dp4a_u(w, 0x80u << (8 * bj), tcol));
                            } else {
                                // E2M1: the group scale folded into the fp16 weight (one rounding per weight)
                                const uint32_t sh = part == 0 ? (sc4.x & 0xffffu) : (part == 1 ? (sc4.x >> 16) : (part == 2 ? (sc4.y & 0xffffu) : (sc4.y >> 16)));
                                const uint32_t s2 = sh * 0x00010001u;
                                uint32_t hh[4];
                                asm("{ .reg .b8 b0, b1, b2, b3; mov.b32 {b0, b1, b2, b3}, %4;\n"
                                    "  cvt.rn.f16x2.e2m1x2 %0, b0; cvt.rn.f16x2.e2m1x2 %1, b1;\n"
                                    "  cvt.rn.f16x2.e2m1x2 %2, b2; cvt.rn.f16x2.e2m1x2 %3, b3; }"
                                    : "=r"(hh[0]), "=r"(hh[1]), "=r"(hh[2]), "=r"(hh[3]) : "r"(w));
#pragma unroll
                                for (int bj = 0; bj < 4; ++bj)
                                    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(v[wi * 4 + bj]) : "r"(hh[bj]), "r"(s2));
                            }
                        }
                    };
                    // the decode of the next 32 codes is issued before the previous 16 pairs are stored, and the
                    // previous group is handed to the MMA issuer only once this group's first lookups are under way
                    // (its tensor-memory stores have had that long to land)
                    uint32_t va[16], vb[16];
                    decode16(0, va);
                    decode16(1, vb);
                    hand_over();
                    tmem_st16(a_t, va);
                    decode16(2, va);
                    tmem_st16(a_t + 16, vb);
                    decode16(3, vb);
                    tmem_st16(a_t + 32, va);
                    tmem_st16(a_t + 48, vb);
                    pend_slot = (int)s;
                    ++t_h;
#pragma unroll
                    for (int i = 0; i < kRing; ++i) raw_q[i] = (s == (uint32_t)i) ? scale_raw : raw_q[i];
                }
                if (!ok) break;
                __syncwarp();                           // every lane has read its row of the stage
                fence_async_smem();
                issue();                                // refill the stage just read
            }
            hand_over();
            have_prev = true;
            prev_bias = (p.bias && row_raw < p.N) ? p.bias[row_raw] : 0.f;
            prev_row = row_raw; prev_N = p.N; prev_ldy = p.ldy; prev_y = p.y;
#pragma unroll
            for (int i = 0; i < (NB + 31) / 32; ++i) prev_xs[i] = xs_next[i];
        }
        if (ok) ok = finish_prev();
    } else {
        // =============================== MMA issuers ===============================
        // Warps 8, 9: half 0, 1; warps 10, 11: a second issuer per half (kIssuers == 2).  With two issuers a half's
        // groups alternate between them (the first group of every 256-code step to one, the second to the other).
        // Every issuer owns a ring of activation stages (one 128-code group each) that it fills itself, so the
        // only thing it ever waits for besides the decode threads is its own earlier work.
        const int h = (warp - 8) & 1, sub = (warp - 8) >> 1, iss = warp - 8;
        if (lane == 0 && sub < C::kIssuers) {
            constexpr uint32_t idesc = idesc_f16(kTileM, NB);
            constexpr int kPer = 2 / C::kIssuers;       // groups of a step this issuer takes
            const uint32_t lbo = (uint32_t)B * 16;
            const uint32_t ring = sbase + S::kXRing + iss * xg.ring;
            // two walks over the same sequence of groups: the loads run ahead of the MMAs
            struct Walk { int tile, pi, t_end, nsg, sg, k; const unsigned char *xp; };
            auto open_tile = [&](Walk &w) {
                while (w.tile < tile_hi) {
                    if (w.tile >= w.t_end) {
                        TaProblem p;
                        problem_at(w.pi, w.t_end, w.tile, p);
                        w.nsg = p.K >> 8;
                        w.xp = reinterpret_cast<const unsigned char *>(p.xprep);
                    }
                    w.sg = h; w.k = 0;
                    if (w.sg < w.nsg) return;
                    ++w.tile;
                }
            };
            auto advance = [&](Walk &w) {
                if (++w.k == kPer) { w.k = 0; w.sg += 2; }
                if (w.sg >= w.nsg) { ++w.tile; open_tile(w); }
            };
            Walk ld = {tile_lo, 0, -1, 0, 0, 0, nullptr};
            open_tile(ld);
            Walk mm = ld;
            // The issuing thread is a single lane running dependent scalar code on a scheduler it shares with two
            // decode warps, so every instruction of this loop costs several clocks: ring positions and parities
            // are carried along instead of being divided out of counters, and the operand descriptor is formed
            // once per group.
            uint32_t ld_s = 0;                          // stage the next load goes to
            auto load_next = [&]() {
                if (ld.tile < tile_hi) {
                    const int G = 2 * ld.sg + (C::kIssuers == 2 ? sub : ld.k);
                    mbar_expect_tx(xbar(iss, ld_s), xg.chunk);
                    bulk_g2s(ring + ld_s * xg.chunk, ld.xp + (size_t)G * xg.chunk, xg.chunk, xbar(iss, ld_s));
                    advance(ld);
                }
                ld_s = (ld_s + 1 == (uint32_t)xg.nstages) ? 0 : ld_s + 1;
            };
            pdl_wait();
            for (int i = 0; i < xg.nstages; ++i) load_next();
            bool ok = true;
            uint32_t cs = 0, cpar = 0;                  // stage and phase parity of the group being multiplied
            uint32_t rs = 0, rpar = 0;                  // stage and phase parity of the group whose stage is refilled next
            uint32_t slot = (uint32_t)sub % kRing, spar = 0;   // A slot of this issuer's next group (the half's group count t = kIssuers n + sub)
            const uint32_t desc_step = (2 * lbo) >> 4;  // descriptor address field per K = 16 slice
            for (uint32_t n = 0; mm.tile < tile_hi && ok; ++n) {
                // the stage whose MMAs were issued xg.lag groups ago is free by now: refill it
                if (n >= (uint32_t)xg.lag) {
                    if (!(ok = mbar_wait(xebar(iss, rs), rpar, err))) break;
                    load_next();
                    if (++rs == (uint32_t)xg.nstages) { rs = 0; rpar ^= 1; }
                }
                if (!(ok = mbar_wait(xbar(iss, cs), cpar, err))) break;
                if (!(ok = mbar_wait(abar(h, slot), spar, err))) break;
                tc_fence_after();
                const uint32_t a_t = tmem + (h * kRing + slot) * C::kSlot;
                const uint32_t d_t = kGf4 ? a_t + 64 : tmem + C::kAcc + (h * C::kIssuers + sub) * NB;
                const uint64_t desc0 = smem_desc(ring + cs * xg.chunk, lbo, 128);
                const bool first = mm.sg == h && mm.k == 0;                // E2M1: this issuer's first group of the tile
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    mma_f16_ts(d_t, a_t + 8 * i, desc0 + (uint64_t)(i * desc_step), idesc, kGf4 ? (i > 0) : (i > 0 || !first));
                mma_commit(dbar(h, slot));
                mma_commit(xebar(iss, cs));
                if (++cs == (uint32_t)xg.nstages) { cs = 0; cpar ^= 1; }
                slot += C::kIssuers;
                if (slot >= (uint32_t)kRing) { slot -= kRing; spar ^= 1; }
                advance(mm);
            }
        }
    }

    // ---- teardown
    if (*err) {   // a wait gave up: let the copies still in flight land before the CTA's shared memory goes away
        for (int i = 0; i < 400; ++i) __nanosleep(256);
    }
    tc_fence_before();
    __syncthreads();
    if (tid == 0 && s_err) atomicExch(status, s_err);
    if (warp == 11) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
    }
}

// ---- GF4, batch 1 on the CUDA cores (the template also covers two rows, where the tensor-memory kernel is faster) ----
// Same tiles, same TMA weight ring, same per-row pair tables as the tensor-memory kernel above, but the
// multiply-accumulate stays in the decode threads: lane = weight row, so all lanes of a warp need the same
// activation values, which they read as broadcast 16-byte shared-memory loads (one wavefront per eight
// codes) from the prepared activation of the whole problem, and a looked-up pair feeds two
// fma.rn.f32.f16 (fp16 x fp16 exact, fp32 accumulation).  Per 128-code group the partial sum is scaled by
// the group's fp16 scale in fp32.  At batch 1 this costs about 2.2 instructions and 0.75 shared-memory
// wavefronts per code, where one 16-bit lookup per code costs 1.2 wavefronts; the tensor pipe, whose
// K = 16 instructions have a floor of about 45 clocks whatever the batch, is not involved.
// Per code a lane receives 2 bytes of looked-up pairs, 0.5 of packed weights and 2 of activations through
// the shared-memory pipe (128 bytes per clock and SM).  A variant whose lanes carry two rows each and read
// the activations once for both (8 warps instead of 16, same tables and ring) was slower: 950 against 1022
// tokens/s on the 7B-shaped stack.
constexpr int kLutQuarters = 2;                      // 32-row sets of a tile (each has its own pair table)
constexpr int kLutTileM = 32 * kLutQuarters;
constexpr int kLutSplit = 8;                         // warps that share a row set, each taking every 8th 256-code step
constexpr int kLutWarps = kLutQuarters * kLutSplit;
constexpr int kLutThreads = kLutWarps * 32;
constexpr int kLutStage = kWStage;                   // a weight stage: 32 rows x 128 bytes (two 128-code groups), 128-byte swizzle
constexpr int kLutSW = 2;                            // stages per warp (16 warps x 2 x 4 KB: this TMA pattern streams at 6.5 TB/s when
                                                     // nothing else limits it; 64-byte boxes four deep reached only 4.3 TB/s)
struct LutSmem {
    static constexpr int kTab = 0;
    static constexpr int kWRing = kTab + kLutQuarters * 256 * 128;
    static constexpr int kX = kWRing + kLutWarps * kLutSW * kLutStage;   // prepared activation of the current problem
    static constexpr int kXBytes = 24 * 1024;
    static constexpr int kPart = kX + kXBytes;                           // partial sums of the other warps of a row set, two tiles
    static constexpr int kBars = kPart + 2 * (kLutSplit - 1) * kLutTileM * 2 * 4;
    static constexpr int kNumBars = kLutWarps * kLutSW + kLutQuarters + 2;   // weights, row-set sync, x free / x full
    static constexpr int kBytes = kBars + kNumBars * 8 + 1024;
};

// acc0 += lo(w) * lo(x), acc1 += hi(w) * hi(x): fp16 operands, exact products, fp32 accumulation
__device__ __forceinline__ void fma_pair(float &acc0, float &acc1, uint32_t w, uint32_t x) {
    asm("{ .reg .b16 wl, wh, xl, xh; mov.b32 {wl, wh}, %2; mov.b32 {xl, xh}, %3;\n"
        "  fma.rn.f32.f16 %0, wl, xl, %0; fma.rn.f32.f16 %1, wh, xh, %1; }"
        : "+f"(acc0), "+f"(acc1) : "r"(w), "r"(x));
}

template <int B>
__global__ void __launch_bounds__(kLutThreads, 1) gf4_lut2_kernel(const TaProblem *probs, const CUtensorMap *maps,
                                                                  const __grid_constant__ TaProblem single,
                                                                  const __grid_constant__ CUtensorMap single_map,
                                                                  int nprob, const int *tile_start, const int *cta_first,
                                                                  int y_dtype, PeerInfo peers, int *status) {
    using S = LutSmem;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ int s_err;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char *sgen = smem_raw + (sbase - smem_u32(smem_raw));
    const uint32_t bars = sbase + S::kBars;
    auto wbar = [&](int w, int s) { return bars + 8u * (w * kLutSW + s); };
    auto qbar = [&](int q) { return bars + 8u * (kLutWarps * kLutSW + q); };
    const uint32_t xfree = bars + 8u * (kLutWarps * kLutSW + kLutQuarters), xfull = xfree + 8;
    volatile int *err = &s_err;
    if (tid == 0) {
        s_err = 0;
        for (int w = 0; w < kLutWarps; ++w)
            for (int s = 0; s < kLutSW; ++s) mbar_init(wbar(w, s), 1);
        for (int q = 0; q < kLutQuarters; ++q) mbar_init(qbar(q), 32 * kLutSplit);
        mbar_init(xfree, kLutThreads);
        mbar_init(xfull, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    int tile_lo, tile_hi;
    if (nprob == 0) {
        const int nt = (single.N + kLutTileM - 1) / kLutTileM;
        tile_lo = (int)((long long)nt * blockIdx.x / gridDim.x);
        tile_hi = (int)((long long)nt * (blockIdx.x + 1) / gridDim.x);
    } else {
        tile_lo = cta_first[blockIdx.x];
        tile_hi = cta_first[blockIdx.x + 1];
    }
    // Problems change rarely along a CTA's tile sequence, so every walker keeps its current problem's fields
    // in registers and goes back to global memory only when a tile lies beyond that problem's last tile.
    auto problem_at = [&](int &pi, int &t_end, int tile, TaProblem &p) {
        if (nprob == 0) { p = single; t_end = 0x7fffffff; return; }
        if (t_end < 0) {
            // first look-up of a walker: bisect (a step's list can hold hundreds of problems, and a scan from the
            // first one is a chain of dependent global loads, 0.2 us each, in front of the last CTAs' first tile)
            int lo = 0, hi = nprob - 1;
            while (lo < hi) {
                const int mid = (lo + hi + 1) >> 1;
                if (tile_start[mid] <= tile) lo = mid; else hi = mid - 1;
            }
            pi = lo;
        } else {
            while (pi + 1 < nprob && tile_start[pi + 1] <= tile) ++pi;
        }
        p = probs[pi];
        t_end = tile_start[pi + 1];
    };

    const int q = warp % kLutQuarters, h = warp / kLutQuarters;   // row set of the tile, which groups (g % kLutSplit == h)
    const int r = q * 32 + lane;
    const uint32_t tcol = sbase + S::kTab + q * (256 * 128) + lane * 4;
    const uint32_t wring = sbase + S::kWRing + warp * (kLutSW * kLutStage);
    // 16-byte piece c of this lane's row sits at piece c ^ (lane & 7) of the row (128-byte swizzle)
    const uint32_t lrow = lane * 128, lkey = (lane & 7) << 4;
    const uint32_t xs_u = sbase + S::kX;

    // ---- producer side of the weight ring: steps of this warp are 256 codes each (steps h, h + 8, ... of a row)
    int i_tile = tile_lo, i_pi = 0, i_tend = -1, i_j = 0, i_n = 0, i_x = 0, i_y = 0, i_tile0 = 0, i_steps = 0, i_stage = 0;
    const void *i_map = nullptr;
    auto i_open = [&]() {   // position on step 0 of tile i_tile
        while (i_tile < tile_hi) {
            if (i_tile >= i_tend) {
                TaProblem p;
                problem_at(i_pi, i_tend, i_tile, p);
                i_steps = ((p.K >> 8) - h + kLutSplit - 1) / kLutSplit;
                i_tile0 = p.tile0;
                i_map = nprob ? &maps[i_pi] : &single_map;
            }
            i_n = i_steps;
            i_x = h * 128;
            i_y = (i_tile - i_tile0) * kLutTileM + q * 32;     // rows past N read as zeros
            i_j = 0;
            if (i_n > 0) return;
            ++i_tile;
        }
    };
    auto issue = [&]() {
        if (i_tile < tile_hi) {
            if (lane == 0) {
                const uint32_t bar = wbar(warp, i_stage);
                mbar_expect_tx(bar, kLutStage);
                tma_2d_g2s(wring + i_stage * kLutStage, i_map, i_x, i_y, bar);
            }
            i_x += 128 * kLutSplit;
            if (++i_j == i_n) { ++i_tile; i_open(); }
        }
        i_stage = (i_stage + 1 == kLutSW) ? 0 : i_stage + 1;
    };
    i_open();
#pragma unroll
    for (int s = 0; s < kLutSW; ++s) issue();

    uint32_t wcount = 0, qcount = 0, xcount = 0;
    // ---- the codebook of this lane's row, one tile ahead
    int f_pi = 0, f_tend = -1, f_tile0 = 0, f_N = 1;
    const __half *f_cb = nullptr;
    uint4 cb0 = make_uint4(0, 0, 0, 0), cb1 = cb0;
    auto fetch_codebook = [&](int tile) {
        if (tile < tile_hi) {
            if (tile >= f_tend) {
                TaProblem p;
                problem_at(f_pi, f_tend, tile, p);
                f_tile0 = p.tile0; f_N = p.N; f_cb = p.codebook;
            }
            const int row = min((tile - f_tile0) * kLutTileM + r, f_N - 1);
            const uint4 *src = reinterpret_cast<const uint4 *>(f_cb + (size_t)row * 16);
            cb0 = __ldg(src);
            cb1 = __ldg(src + 1);
        }
    };
    auto quarter_sync = [&]() -> bool {
        mbar_arrive(qbar(q));
        const bool ok = mbar_wait(qbar(q), qcount & 1, err);
        ++qcount;
        return ok;
    };

    // ---- a finished tile whose outputs are written after the next row-set sync (first warp of the row set)
    float *part_s = reinterpret_cast<float *>(sgen + S::kPart);      // [2 parities][kLutSplit - 1][kLutTileM][2]
    constexpr int kPartStride = (kLutSplit - 1) * kLutTileM * 2;
    bool have_prev = false;
    float prev_acc[B], prev_xsc[B], prev_bias = 0.f;
    int prev_row = 0, prev_N = 0, prev_ldy = 0;
    void *prev_y = nullptr;
    auto write_prev = [&](int parity) {
        if (have_prev && h == 0 && prev_row < prev_N) {
            const float *ps = part_s + parity * kPartStride;
#pragma unroll
            for (int b = 0; b < B; ++b) {
                float v = prev_acc[b];
#pragma unroll
                for (int hh = 1; hh < kLutSplit; ++hh) v += ps[((hh - 1) * kLutTileM + r) * 2 + b];
                const float o = fmaf(v, prev_xsc[b], prev_bias);
                jq::store_out_copies(prev_y, peers.delta, peers.n, (size_t)b * prev_ldy + prev_row, o, y_dtype);
            }
        }
        have_prev = false;
    };

    int c_pi = 0, c_tend = -1, x_pi = -1;
    TaProblem p = single;
    fetch_codebook(tile_lo);
    pdl_wait();                     // from here on the prepared activation and its row factors are read
    bool ok = true;
    int tparity = 0;
    for (int tile = tile_lo; tile < tile_hi && ok; ++tile, tparity ^= 1) {
        if (tile >= c_tend) problem_at(c_pi, c_tend, tile, p);
        const int row_raw = (tile - p.tile0) * kLutTileM + r;
        const int row = min(row_raw, p.N - 1);
        // ---- a new problem: its prepared activation replaces the previous one in shared memory
        if (c_pi != x_pi) {
            mbar_arrive(xfree);                                      // this thread no longer reads the old activation
            if (tid == 0) {
                if ((ok = mbar_wait(xfree, xcount & 1, err))) {
                    const uint32_t bytes = (uint32_t)p.K * B * 2;
                    fence_async_smem();
                    mbar_expect_tx(xfull, bytes);
                    bulk_g2s(xs_u, p.xprep, bytes, xfull);
                }
            }
            ok = mbar_wait(xfull, xcount & 1, err);
            ++xcount;
            x_pi = c_pi;
            if (!ok) break;
        }
        // ---- row-set sync: the previous tile's lookups are over (its table may go) and its partial sums are visible
        if (!(ok = quarter_sync())) break;
        write_prev(tparity ^ 1);
        // ---- the pair table of this row: this thread fills the entries whose second code is 2 h or 2 h + 1
        {
            const uint32_t c[8] = {cb0.x, cb0.y, cb0.z, cb0.w, cb1.x, cb1.y, cb1.z, cb1.w};
            uint32_t ch = c[0];                                      // the pair register holding entries 2 h, 2 h + 1
#pragma unroll
            for (int hh = 1; hh < kLutSplit; ++hh) ch = (h == hh) ? c[hh] : ch;
            const uint32_t tb = tcol + h * (32 * 128);
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int lo = 0; lo < 16; ++lo) {
                    const uint32_t e = __byte_perm(c[lo >> 1], ch,
                                                   ((lo & 1) ? 0x32u : 0x10u) | (((i & 1) ? 0x76u : 0x54u) << 8));
                    asm volatile("st.shared.u32 [%0], %1;" ::"r"(tb + (i * 16 + lo) * 128), "r"(e) : "memory");
                }
        }
        fetch_codebook(tile + 1);
        float acc[B], xsc[B];
#pragma unroll
        for (int b = 0; b < B; ++b) {
            acc[b] = 0.f;
            xsc[b] = p.xscale[b];                                    // in flight during the tile, needed at its end
        }
        const float bias = (p.bias && row_raw < p.N) ? p.bias[row_raw] : 0.f;
        const int nsteps = ((p.K >> 8) - h + kLutSplit - 1) / kLutSplit;
        const unsigned short *srow = reinterpret_cast<const unsigned short *>(p.scales) + (size_t)row * p.lds;
        const int gshift = 31 - __clz(p.g >> 7);
        if (!(ok = quarter_sync())) break;                           // the table is complete
        for (int j = 0; j < nsteps && ok; ++j) {
            const int stage = wcount % kLutSW;
            ok = __all_sync(0xffffffffu, mbar_wait(wbar(warp, stage), (wcount / kLutSW) & 1, err));
            if (!ok) break;
            ++wcount;
            const uint32_t slot = wring + stage * kLutStage + lrow;
#pragma unroll
            for (int gi = 0; gi < 2; ++gi) {
            const int grp = 2 * (kLutSplit * j + h) + gi;
            const unsigned short scale_raw = __ldg(srow + (grp >> gshift));
            const uint32_t xg0 = xs_u + (uint32_t)grp * (256 * B);   // the group's activations: [16 pieces][B][16 bytes]
            float part[B][4];
#pragma unroll
            for (int b = 0; b < B; ++b) part[b][0] = part[b][1] = part[b][2] = part[b][3] = 0.f;
#pragma unroll
            for (int pc = 0; pc < 4; ++pc) {                         // 32 codes
                const uint4 w4 = lds128(slot + (((gi * 4 + pc) << 4) ^ lkey));
#pragma unroll
                for (int wi = 0; wi < 4; ++wi) {                     // 8 codes
                    const uint32_t w = wi == 0 ? w4.x : (wi == 1 ? w4.y : (wi == 2 ? w4.z : w4.w));
                    uint32_t v[4];
#pragma unroll
                    for (int bj = 0; bj < 4; ++bj) v[bj] = lds32(dp4a_u(w, 0x80u << (8 * bj), tcol));
#pragma unroll
                    for (int b = 0; b < B; ++b) {
                        const uint4 xv = lds128(xg0 + (uint32_t)(((pc * 4 + wi) * B + b) * 16));
                        fma_pair(part[b][0], part[b][1], v[0], xv.x);
                        fma_pair(part[b][2], part[b][3], v[1], xv.y);
                        fma_pair(part[b][0], part[b][1], v[2], xv.z);
                        fma_pair(part[b][2], part[b][3], v[3], xv.w);
                    }
                }
            }
            const float sc = __half2float(__ushort_as_half(scale_raw));
#pragma unroll
            for (int b = 0; b < B; ++b)
                acc[b] = fmaf((part[b][0] + part[b][1]) + (part[b][2] + part[b][3]), sc, acc[b]);
            }
            __syncwarp();
            fence_async_smem();
            issue();
        }
        if (!ok) break;
        // ---- the other warps of the row set park their sums; the first keeps what it needs for the outputs
        if (h > 0) {
            float *ps = part_s + tparity * kPartStride;
#pragma unroll
            for (int b = 0; b < B; ++b) ps[((h - 1) * kLutTileM + r) * 2 + b] = acc[b];
        } else {
#pragma unroll
            for (int b = 0; b < B; ++b) { prev_acc[b] = acc[b]; prev_xsc[b] = xsc[b]; }
            prev_bias = bias; prev_row = row_raw; prev_N = p.N; prev_ldy = p.ldy; prev_y = p.y;
        }
        have_prev = true;
    }
    if (ok && have_prev && (ok = quarter_sync())) write_prev(tparity ^ 1);
    if (*err) {
        for (int i = 0; i < 400; ++i) __nanosleep(256);
    }
    __syncthreads();
    if (tid == 0 && s_err) atomicExch(status, s_err);
}


}  // namespace jqta

using namespace jqta;

// ---- host side -------------------------------------------------------------------
// plan layout: 12 ints [magic, n, grid, NB, tensor-map offset (bytes), B, fmt, problem offset (bytes),
// largest K, 0, 0, 0],
// tile_start[n + 1], cta_first[grid + 1], padding to 64 bytes, TaProblem[n], padding to 64 bytes, CUtensorMap[n]
static const int kTaMagic = 0x4a515441;
// fixed time per tile / per problem of the partition's cost model, in codes of one row.  Swept on the 7B-shaped
// GF4 step (us per step on one GPU / for an eighth of it): bytes only 940 / 150.5; 384, 2048: 921.5 / 143.0;
// 768, 4096: 910.1 / 141.3; 1408, 6144: 900.1 / 140.1; 2304, 8192: 943.3 / 143.9.
static const double kTileCost = 1408, kProblemCost = 6144;
static const int kTaHeader = 12;

// MMA N: GF4 keeps one accumulator per group and slot (up to 16 columns); E2M1 one per half (up to 64)
static int ta_cols(int fmt, int B) {
    if (B <= 16) return 16;
    if (fmt == JQ_FMT_E2M1) return B <= 32 ? 32 : (B <= 64 ? 64 : 0);
    return 0;
}

static bool ta_use_lut(int B, int maxK);
static size_t ta_align(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Tensor map over the packed rows of one matrix: bytes [N rows][ldw], boxes of 32 rows x 128 bytes with the
// 128-byte swizzle; rows past N read as zeros.  The driver entry point is looked up once (no link-time
// dependency on the driver library).
typedef CUresult (*ta_encode_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                 const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static ta_encode_fn ta_encoder() {
    static ta_encode_fn fn = nullptr;
    static bool tried = false;
    static std::mutex mu;
    std::lock_guard<std::mutex> lk(mu);
    if (!tried) {
        tried = true;
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) == cudaSuccess &&
            qr == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<ta_encode_fn>(p);
    }
    return fn;
}
static int ta_encode_map(CUtensorMap *out, const void *qw, int N, int ldw) {
    ta_encode_fn enc = ta_encoder();
    if (!enc) return JQ_ERR_UNSUPPORTED;
    const cuuint64_t dims[2] = {(cuuint64_t)ldw, (cuuint64_t)N};
    const cuuint64_t strides[1] = {(cuuint64_t)ldw};
    const cuuint32_t box[2] = {128, 32};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(qw), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? JQ_OK : JQ_ERR_CUDA_BASE - (int)cudaErrorInvalidValue;
}

static bool ta_shape_ok(int fmt, int N, int K, int g, int had) {
    if (N <= 0 || K < 512 || K % 256) return false;
    if (had != 0 && had != 128) return false;
    if (fmt == JQ_FMT_GF4) {
        const int gq = g >> 7;
        return g >= 128 && g % 128 == 0 && (gq & (gq - 1)) == 0 && K % g == 0;
    }
    return fmt == JQ_FMT_E2M1 && g == 32;
}

// batch 1 runs on the CUDA cores when the prepared activation of one problem fits its shared-memory buffer
// (K up to 12288); from two rows on the tensor-memory kernel is faster (decode7b: 1800 against 1090 tokens/s)
static bool ta_use_lut(int B, int maxK) { return B == 1 && (size_t)maxK * 2 <= (size_t)LutSmem::kXBytes; }

extern "C" size_t jq_ta_workspace_bytes(const jq_problem *ph, int n, int B) {
    if (!ph || n <= 0 || B < 1 || B > 64) return 0;
    size_t total = kHeaderBytes;
    for (int i = 0; i < n; ++i) total += 256 + ta_align((size_t)ph[i].K * B * 2, 128);
    return total;
}

extern "C" size_t jq_ta_plan_bytes(int n) {
    if (n <= 0) return 0;
    return ta_align(ta_align(((size_t)kTaHeader + (size_t)(n + 1) + (size_t)jq_sm_count() + 1) * sizeof(int), 64) +
                        (size_t)n * sizeof(TaProblem), 64) + (size_t)n * sizeof(CUtensorMap);
}

static int ta_fill_problem(TaProblem &t, int fmt, const jq_problem &p, unsigned char *ws, size_t &off, int B) {
    if (!p.qweight || !p.x || !p.y || !p.scales) return JQ_ERR_NULL_PTR;
    if (fmt == JQ_FMT_GF4 && !p.codebook) return JQ_ERR_NULL_PTR;
    if (!ta_shape_ok(fmt, p.N, p.K, p.g, p.had_block)) return JQ_ERR_UNSUPPORTED;
    if (!jq_aligned16(p.qweight) || (fmt == JQ_FMT_GF4 && !jq_aligned16(p.codebook)) ||
        (reinterpret_cast<uintptr_t>(p.scales) & (fmt == JQ_FMT_E2M1 ? 15u : 1u)))
        return JQ_ERR_BAD_ALIGN;
    t.qw = reinterpret_cast<const uint8_t *>(p.qweight);
    t.scales = reinterpret_cast<const __half *>(p.scales);
    t.codebook = reinterpret_cast<const __half *>(p.codebook);
    t.x = p.x;
    t.bias = p.bias;
    t.y = p.y;
    t.xscale = reinterpret_cast<float *>(ws + off);
    off += 256;   // up to 64 batch rows
    t.xprep = reinterpret_cast<__half *>(ws + off);
    off += ta_align((size_t)p.K * B * 2, 128);
    t.N = p.N; t.K = p.K; t.g = p.g; t.had = p.had_block;
    t.ldw = p.K >> 1;
    t.lds = p.K / p.g;
    t.ldy = p.ldy > 0 ? p.ldy : p.N;
    t.tile0 = 0;
    return JQ_OK;
}

extern "C" int jq_ta_plan(int fmt, const jq_problem *ph, int n, int B, void *workspace_dev, size_t workspace_bytes,
                          void *plan_host, size_t plan_bytes) {
    if (!ph || !plan_host || !workspace_dev) return JQ_ERR_NULL_PTR;
    if (n <= 0 || B < 1) return JQ_ERR_BAD_SHAPE;
    if ((fmt != JQ_FMT_GF4 && fmt != JQ_FMT_E2M1) || !ta_cols(fmt, B)) return JQ_ERR_UNSUPPORTED;
    if (plan_bytes < jq_ta_plan_bytes(n) || workspace_bytes < jq_ta_workspace_bytes(ph, n, B)) return JQ_ERR_WORKSPACE;
    if (reinterpret_cast<uintptr_t>(workspace_dev) & 127u) return JQ_ERR_BAD_ALIGN;
    const int grid = jq_sm_count();
    int *h = reinterpret_cast<int *>(plan_host);
    int *tile_start = h + kTaHeader, *cta_first = tile_start + n + 1;
    const size_t poff = ta_align(((size_t)kTaHeader + (n + 1) + grid + 1) * sizeof(int), 64);
    const size_t moff = ta_align(poff + (size_t)n * sizeof(TaProblem), 64);
    TaProblem *tp = reinterpret_cast<TaProblem *>(reinterpret_cast<unsigned char *>(plan_host) + poff);
    unsigned char *maps = reinterpret_cast<unsigned char *>(plan_host) + moff;
    size_t off = kHeaderBytes;
    double total = 0;
    int maxK = 0;
    for (int i = 0; i < n; ++i) maxK = ph[i].K > maxK ? ph[i].K : maxK;
    const bool lut = fmt == JQ_FMT_GF4 && ta_use_lut(B, maxK);
    const int tile_m = lut ? kLutTileM : kTileM;
    tile_start[0] = 0;
    for (int i = 0; i < n; ++i) {
        int st = ta_fill_problem(tp[i], fmt, ph[i], reinterpret_cast<unsigned char *>(workspace_dev), off, B);
        if (st) return st;
        CUtensorMap tm;
        st = ta_encode_map(&tm, ph[i].qweight, ph[i].N, ph[i].K >> 1);
        if (st) return st;
        memcpy(maps + (size_t)i * sizeof(CUtensorMap), &tm, sizeof(CUtensorMap));
        const int tiles = (ph[i].N + tile_m - 1) / tile_m;
        tp[i].tile0 = tile_start[i];
        tile_start[i + 1] = tile_start[i] + tiles;
        total += (double)tiles * (ph[i].K + kTileCost) + kProblemCost;
    }
    // contiguous tile ranges of (nearly) equal cost: cut where the running cost passes c * total / grid.  A tile
    // costs its packed bytes plus a fixed part (table build, two syncs, outputs), a problem's first tile also the
    // switch of the activation buffer: with bytes alone a CTA of short rows ran 10 % longer than one of long rows.
    int cta = 0;
    double acc = 0;
    cta_first[0] = 0;
    for (int i = 0; i < n; ++i)
        for (int t = tile_start[i]; t < tile_start[i + 1]; ++t) {
            const double c = ph[i].K + kTileCost + (t == tile_start[i] ? kProblemCost : 0);
            while (cta + 1 < grid && acc + 0.5 * c >= total * (cta + 1) / grid) cta_first[++cta] = t;
            acc += c;
        }
    while (cta < grid) cta_first[++cta] = tile_start[n];
    h[0] = kTaMagic; h[1] = n; h[2] = grid; h[3] = ta_cols(fmt, B); h[4] = (int)moff; h[5] = B; h[6] = fmt; h[7] = (int)poff;
    h[8] = maxK; h[9] = h[10] = h[11] = 0;
    return JQ_OK;
}

// launch configuration of a main kernel: allowed to start while the preparation kernel in front of it still runs
static void ta_pdl_config(cudaLaunchConfig_t &cfg, cudaLaunchAttribute *attr, int grid, int threads, int smem, cudaStream_t st) {
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = (size_t)smem;
    cfg.stream = st;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
}

template <int FMT, int NB>
static int ta_launch(const TaProblem *probs_dev, const CUtensorMap *maps_dev, const TaProblem &single,
                     const CUtensorMap &single_map, int nprob, const int *tile_start,
                     const int *cta_first, int grid, int B, int x_dtype, int y_dtype, const jqta::PeerInfo &peers,
                     int *status, cudaStream_t st) {
    const int nblk = (nprob ? nprob : 1) * B;
    if (B <= 2) ta_prepare_kernel<1024><<<nblk, 1024, 0, st>>>(probs_dev, single, B, x_dtype);
    else ta_prepare_kernel<256><<<nblk, 256, 0, st>>>(probs_dev, single, B, x_dtype);
    int s = jq_launch_status();
    if (s) return s;
    auto kern = gemm_ta_kernel<FMT, NB>;
    constexpr int smem = Smem<FMT>::kBytes;
    static_assert(smem <= 227 * 1024, "shared memory");
    JQ_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    ta_pdl_config(cfg, attr, grid, kTaThreads, smem, st);
    JQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, probs_dev, maps_dev, single, single_map, nprob, tile_start, cta_first, B, y_dtype,
                                   peers, status));
    return jq_launch_status();
}

template <int B>
static int lut2_launch(const TaProblem *probs_dev, const CUtensorMap *maps_dev, const TaProblem &single,
                       const CUtensorMap &single_map, int nprob, const int *tile_start, const int *cta_first, int grid,
                       int x_dtype, int y_dtype, const jqta::PeerInfo &peers, int *status, cudaStream_t st) {
    const int nblk = (nprob ? nprob : 1) * B;
    if (B <= 2) ta_prepare_kernel<1024><<<nblk, 1024, 0, st>>>(probs_dev, single, B, x_dtype);
    else ta_prepare_kernel<256><<<nblk, 256, 0, st>>>(probs_dev, single, B, x_dtype);
    int s = jq_launch_status();
    if (s) return s;
    auto kern = gf4_lut2_kernel<B>;
    constexpr int smem = LutSmem::kBytes;
    static_assert(smem <= 227 * 1024, "shared memory");
    JQ_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    ta_pdl_config(cfg, attr, grid, kLutThreads, smem, st);
    JQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, probs_dev, maps_dev, single, single_map, nprob, tile_start, cta_first, y_dtype,
                                   peers, status));
    return jq_launch_status();
}

static int ta_dispatch(int fmt, int nb, int maxK, const TaProblem *probs_dev, const CUtensorMap *maps_dev, const TaProblem &single,
                       const CUtensorMap &single_map, int nprob,
                       const int *tile_start, const int *cta_first, int grid, int B, int x_dtype, int y_dtype,
                       const jqta::PeerInfo &peers, int *status, cudaStream_t st) {
#define JQ_TA_ARGS probs_dev, maps_dev, single, single_map, nprob, tile_start, cta_first, grid, B, x_dtype, y_dtype, peers, status, st
    if (fmt == JQ_FMT_GF4) {
        if (ta_use_lut(B, maxK)) {
            return lut2_launch<1>(probs_dev, maps_dev, single, single_map, nprob, tile_start, cta_first, grid, x_dtype, y_dtype, peers, status, st);
        }
        if (nb == 16) return ta_launch<JQ_FMT_GF4, 16>(JQ_TA_ARGS);
        return JQ_ERR_UNSUPPORTED;
    }
    if (nb == 16) return ta_launch<JQ_FMT_E2M1, 16>(JQ_TA_ARGS);
    if (nb == 32) return ta_launch<JQ_FMT_E2M1, 32>(JQ_TA_ARGS);
    if (nb == 64) return ta_launch<JQ_FMT_E2M1, 64>(JQ_TA_ARGS);
#undef JQ_TA_ARGS
    return JQ_ERR_UNSUPPORTED;
}

extern "C" int jq_gemm_ta_grouped(const void *plan_host, const void *plan_dev, void *workspace_dev, int x_dtype,
                                  int y_dtype, int npeer, const int64_t *peer_delta, jq_stream_t stream) {
    if (!plan_host || !plan_dev || !workspace_dev || !peer_delta) return JQ_ERR_NULL_PTR;
    if (npeer < 1 || npeer > 8) return JQ_ERR_BAD_SHAPE;
    if (x_dtype < 0 || x_dtype > 2 || y_dtype < 0 || y_dtype > 2) return JQ_ERR_BAD_DTYPE;
    const int *h = reinterpret_cast<const int *>(plan_host);
    if (h[0] != kTaMagic) return JQ_ERR_BAD_SHAPE;
    jqta::PeerInfo peers;
    peers.n = npeer;
    for (int i = 0; i < 8; ++i) peers.delta[i] = i < npeer ? (long long)peer_delta[i] : 0;
    const int n = h[1], grid = h[2];
    const int *d = reinterpret_cast<const int *>(plan_dev);
    const TaProblem *probs = reinterpret_cast<const TaProblem *>(reinterpret_cast<const unsigned char *>(plan_dev) + h[7]);
    const CUtensorMap *maps = reinterpret_cast<const CUtensorMap *>(reinterpret_cast<const unsigned char *>(plan_dev) + h[4]);
    if (reinterpret_cast<uintptr_t>(maps) & 63u) return JQ_ERR_BAD_ALIGN;
    TaProblem none{};
    CUtensorMap nomap{};
    return ta_dispatch(h[6], h[3], h[8], probs, maps, none, nomap, n, d + kTaHeader, d + kTaHeader + n + 1, grid, h[5], x_dtype, y_dtype,
                       peers, reinterpret_cast<int *>(workspace_dev), reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int jq_gemm_ta(int fmt, const void *qweight, const void *scales, const void *codebook, const void *x,
                          const float *bias, void *y, int N, int K, int B, int g, int had_block, int x_dtype,
                          int y_dtype, void *workspace, size_t workspace_bytes, jq_stream_t stream) {
    if (!workspace) return JQ_ERR_NULL_PTR;
    if (B < 1) return JQ_ERR_BAD_SHAPE;
    if ((fmt != JQ_FMT_GF4 && fmt != JQ_FMT_E2M1) || !ta_cols(fmt, B)) return JQ_ERR_UNSUPPORTED;
    if (x_dtype < 0 || x_dtype > 2 || y_dtype < 0 || y_dtype > 2) return JQ_ERR_BAD_DTYPE;
    if (reinterpret_cast<uintptr_t>(workspace) & 127u) return JQ_ERR_BAD_ALIGN;
    jq_problem p{};
    p.qweight = qweight; p.scales = scales; p.codebook = codebook; p.x = x; p.bias = bias; p.y = y;
    p.N = N; p.K = K; p.g = g; p.had_block = had_block;
    if (workspace_bytes < jq_ta_workspace_bytes(&p, 1, B)) return JQ_ERR_WORKSPACE;
    TaProblem t;
    size_t off = kHeaderBytes;
    int st = ta_fill_problem(t, fmt, p, reinterpret_cast<unsigned char *>(workspace), off, B);
    if (st) return st;
    CUtensorMap tm;
    st = ta_encode_map(&tm, qweight, N, K >> 1);
    if (st) return st;
    jqta::PeerInfo peers;
    peers.n = 1;
    for (int i = 0; i < 8; ++i) peers.delta[i] = 0;
    int grid = jq_sm_count();
    const int tile_m = (fmt == JQ_FMT_GF4 && ta_use_lut(B, K)) ? kLutTileM : kTileM;
    const int tiles = (N + tile_m - 1) / tile_m;
    if (grid > tiles) grid = tiles;
    return ta_dispatch(fmt, ta_cols(fmt, B), K, nullptr, nullptr, t, tm, 0, nullptr, nullptr, grid, B, x_dtype, y_dtype, peers,
                       reinterpret_cast<int *>(workspace), reinterpret_cast<cudaStream_t>(stream));
}

// The status word is sticky: kernels only ever raise it.  Reading it synchronises the stream; clear != 0
// also resets it (stream-ordered) after the read.
extern "C" int jq_ta_status(void *workspace, int clear, jq_stream_t stream) {
    if (!workspace) return JQ_ERR_NULL_PTR;
    int v = 0;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    JQ_CUDA_TRY(cudaMemcpyAsync(&v, workspace, sizeof(int), cudaMemcpyDeviceToHost, st));
    JQ_CUDA_TRY(cudaStreamSynchronize(st));
    if (clear && v) JQ_CUDA_TRY(cudaMemsetAsync(workspace, 0, sizeof(int), st));
    return v;
}

// ---- bounded-wait self test ------------------------------------------------------
// One CTA waits, the way the pipelines above wait, on an mbarrier that nothing ever arrives on.  The wait
// has to give up after the given number of polls, raise the status word and let the kernel return; the
// device stays usable.  (This is how the failure path is exercised without faulting or hanging a GPU.)
namespace jqta {
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
    if (threadIdx.x == 32) {          // one waiter; nobody arrives
        bool ok = false;
        for (uint32_t i = 0; i < limit; ++i) {
            if (mbar_try(smem_u32(&bar), 0)) { ok = true; break; }
            if (i > 64) __nanosleep(64);
        }
        if (!ok) *err = JQ_ERR_TIMEOUT;
    }
    __syncthreads();
    if (threadIdx.x == 0) *status = s_err;
}
}  // namespace jqta

extern "C" int jq_selftest_bounded_wait(int *status_dev, unsigned int polls, jq_stream_t stream) {
    if (!status_dev) return JQ_ERR_NULL_PTR;
    if (polls == 0 || polls > (1u << 20)) return JQ_ERR_BAD_SHAPE;   // at most ~0.1 s of polling
    jqta::bounded_wait_selftest_kernel<<<1, 64, 0, reinterpret_cast<cudaStream_t>(stream)>>>(status_dev, polls);
    return jq_launch_status();
}
