// Fused 4-bit dequantise + GEMV for B200 (sm_100a), batch 1..8.
//
// Data path: packed weight rows stream from HBM exactly once (cp.async into
// per-thread or per-warp shared-memory rings, or straight into registers); the
// activation is rotated (block Hadamard), normalised by a power of two and
// rounded to fp16 once per CTA into shared memory; E2M1 nibbles are converted
// two at a time by the sm_100a cvt.rn.f16x2.e2m1x2 instruction, GF4 nibbles
// index per-row 16-entry fp16 tables in shared memory; products fp16 x fp16
// are exact in fp32 and accumulated in fp32; group scales are applied in fp32.
// Row loops (run_rows picks one per problem):
//   cta_rows            batch 1 (and any shape the others do not take): one FMA
//                       per code (fma.rn.f32.f16), warp = T rows x all of K
//   cta_rows_gf4_direct GF4 batch 1: the same with rows loaded to registers
//   cta_rows_mma        E2M1 batch 2..8: dot products on mma.sync.m16n8k16
//   cta_rows_mma_gf4    GF4 batch 3..8: per-lane table columns + the same MMA
//   rows_k_tiled        grouped launches whose batch x K exceeds shared memory
#include "common.cuh"

namespace jq {

struct GemvProblem {
    const uint8_t *qw;
    const __half *scales;
    const __half *codebook;
    const void *x;
    const float *bias;
    void *y;
    int N, K, g, had;
    // leading dimensions, so that a K-tile of a wider matrix is itself a problem
    int ldw;        // bytes between packed rows
    int lds;        // scales between rows
    int ldx;        // activations between batch rows
    const void *x_full;  // whole activation rows (x_full[b*ldx + k], k < K_full): the normalisation sees all of K
    int K_full;
    int ldy;        // outputs between batch rows (N, or the unsharded N when this is a row shard)
    int npeer;      // copies of every output element to write (1 = only the local buffer)
    long long peer_delta[8];  // byte offsets from this rank's output buffer to each copy's buffer (peer GPUs)
};

__host__ __device__ inline void finish_problem(GemvProblem &p) {
    p.ldw = jq_row_stride_codes(p.K) >> 1;
    p.lds = p.g ? p.K / p.g : 0;
    p.ldx = p.K;
    p.x_full = p.x;
    p.K_full = p.K;
    p.ldy = p.N;
    p.npeer = 1;
    p.peer_delta[0] = 0;
}

constexpr int kThreads = 512;
constexpr int kWarps = kThreads / 32;

constexpr int kRowsE2m1 = 4, kRowsGf4 = 4;   // rows a warp carries at once in the FMA row loops, batch <= 2
constexpr int kMmaMinB = 2;                  // E2M1 batches from here up to 8 use the m16n8k16 row loop when the problem allows
constexpr int kMmaMinBGf4 = 3;               // GF4: from 3 rows (at 2 the FMA loop's shared tables are faster)
template <int FMT, int B>
struct Tile {
    // rows a warp carries at once in the FMA row loops; bounded by registers and by the ring's shared memory
    static constexpr int T = (B <= 2) ? (FMT == JQ_FMT_GF4 ? kRowsGf4 : kRowsE2m1) : (B <= 4 ? 2 : 1);
    // both formats have an MMA row loop for batches (GF4 from 3 rows: at 2 the FMA loop's shared tables are faster)
    static constexpr bool kMma = B >= (FMT == JQ_FMT_GF4 ? kMmaMinBGf4 : kMmaMinB);
    // rows of a row group, the unit in which work is handed to warps (and planned on the host)
    static constexpr int R = kMma ? 16 : T;
};
constexpr int kXPad = 32;  // halves between batch rows of the plain activation layout beyond xs_halves(K)

// halves of shared memory one batch row of the activation occupies
__host__ __device__ inline int xs_halves(int K) { return (jq_row_stride_codes(K) + 1023) / 1024 * 1024; }

// position of code k inside the lane-interleaved activation layout: the
// 16-byte piece j of 32-code chunk c sits at ((c/32*4 + j)*32 + c%32), so the
// 32 lanes of a warp, holding consecutive chunks, read consecutive 16-byte
// words (conflict-free LDS.128).
__device__ __forceinline__ int xs_pos(int k) {
    int c = k >> 5, i = c >> 5, l = c & 31, j = (k >> 3) & 3, e = k & 7;
    return (((i * 4 + j) * 32 + l) << 3) + e;
}

// e with amax * 2^-e below 2^15 after the rotation's worst-case growth:
// exponent field - 127 - (10 with rotation, 14 without), clamped to +-100.
__device__ __forceinline__ int act_exponent(float amax, bool had) {
    uint32_t bits = __float_as_uint(amax);
    int field = (bits >> 23) & 0xff;
    if (field == 0xff || (bits & 0x7fffffffu) == 0) return 0;
    int e = field - 127 - (had ? 10 : 14);
    return max(-100, min(100, e));
}

// CTA prologue: x[B,K] -> rotated, normalised fp16 in shared memory.
// sred: kWarps floats of scratch; sexp: B ints (the exponents, kept for the epilogue).
// plain: position of code k is k and batch rows are xs_halves(K) + kXPad halves
// apart (the m16n8k16 row loop); otherwise the lane-interleaved layout above.
template <int B>
__device__ void stage_activation(const GemvProblem &p, int x_dtype, __half *xs, float *sred, int *sexp, bool plain = false,
                                 bool keep_exponents = false) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int K = p.K, XS = xs_halves(K);
    const int XSB = plain ? XS + kXPad : XS;
    for (int b = 0; b < B && !keep_exponents; ++b) {   // (a later K tile of the same rows: sexp[] is already right)
        float m = 0.f;
        for (int k = tid; k < p.K_full; k += kThreads) m = fmaxf(m, fabsf(load_act(p.x_full, (size_t)b * p.ldx + k, x_dtype)));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (lane == 0) sred[warp] = m;
        __syncthreads();
        if (tid == 0) {
            float mm = 0.f;
            for (int w = 0; w < kWarps; ++w) mm = fmaxf(mm, sred[w]);
            sexp[b] = act_exponent(mm, p.had != 0);
        }
        __syncthreads();
    }
    for (int b = 0; b < B; ++b) {
        const float down = __uint_as_float((uint32_t)(127 - sexp[b]) << 23);  // 2^-e
        __half *xb = xs + (size_t)b * XSB;
        if (p.had) {
            for (int blk = warp; blk * 128 < K; blk += kWarps) {
                float v[4];
                const int k0 = blk * 128 + lane * 4;
#pragma unroll
                for (int j = 0; j < 4; ++j) v[j] = load_act(p.x, (size_t)b * p.ldx + k0 + j, x_dtype) * down;
                fwht128_warp(v, lane);
                __half2 h01 = __floats2half2_rn(v[0], v[1]), h23 = __floats2half2_rn(v[2], v[3]);
                uint2 pk = make_uint2(*reinterpret_cast<uint32_t *>(&h01), *reinterpret_cast<uint32_t *>(&h23));
                *reinterpret_cast<uint2 *>(xb + (plain ? k0 : xs_pos(k0))) = pk;
            }
        } else {
            for (int k = tid; k < K; k += kThreads)
                xb[plain ? k : xs_pos(k)] = __float2half_rn(load_act(p.x, (size_t)b * p.ldx + k, x_dtype) * down);
        }
        for (int k = K + tid; k < XS; k += kThreads) xb[plain ? k : xs_pos(k)] = __float2half_rn(0.f);
    }
    __syncthreads();
}

// ---- asynchronous per-thread prefetch ring ------------------------------------
// Every thread copies exactly the 16-byte weight chunks (and the 4-byte scale
// pairs) it will consume itself, with cp.async, DEPTH stages ahead, into
// shared-memory slots only it reads.  No barrier of any kind guards the ring:
// cp.async.wait_group orders a thread's own copies before its own loads.
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void *src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
// src_bytes < size: the rest of the destination is filled with zeros (0 = nothing is read)
__device__ __forceinline__ void cp_async16_z(uint32_t dst, const void *src, uint32_t src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async4_z(uint32_t dst, const void *src, uint32_t src_bytes) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
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
__device__ __forceinline__ uint16_t lds16(uint32_t a) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(a));
    return v;
}
// Eight E2M1 codes (one 32-bit word) times eight fp16 activations (x: four
// half2), accumulated into two fp32 partial sums.  One asm block so that the
// byte and half-word unpacking stays register sub-addressing instead of
// shift/mask instructions: 4 cvt + 8 fma per word.
__device__ __forceinline__ void dot8_e2m1(uint32_t word, const uint4 &x, float &p0, float &p1) {
    asm("{ .reg .b8 b0, b1, b2, b3; .reg .b32 h0, h1, h2, h3;\n"
        "  .reg .b16 wl0, wh0, wl1, wh1, wl2, wh2, wl3, wh3, xl0, xh0, xl1, xh1, xl2, xh2, xl3, xh3;\n"
        "  mov.b32 {b0, b1, b2, b3}, %2;\n"
        "  cvt.rn.f16x2.e2m1x2 h0, b0; cvt.rn.f16x2.e2m1x2 h1, b1;\n"
        "  cvt.rn.f16x2.e2m1x2 h2, b2; cvt.rn.f16x2.e2m1x2 h3, b3;\n"
        "  mov.b32 {wl0, wh0}, h0; mov.b32 {wl1, wh1}, h1; mov.b32 {wl2, wh2}, h2; mov.b32 {wl3, wh3}, h3;\n"
        "  mov.b32 {xl0, xh0}, %3; mov.b32 {xl1, xh1}, %4; mov.b32 {xl2, xh2}, %5; mov.b32 {xl3, xh3}, %6;\n"
        "  fma.rn.f32.f16 %0, wl0, xl0, %0; fma.rn.f32.f16 %1, wh0, xh0, %1;\n"
        "  fma.rn.f32.f16 %0, wl1, xl1, %0; fma.rn.f32.f16 %1, wh1, xh1, %1;\n"
        "  fma.rn.f32.f16 %0, wl2, xl2, %0; fma.rn.f32.f16 %1, wh2, xh2, %1;\n"
        "  fma.rn.f32.f16 %0, wl3, xl3, %0; fma.rn.f32.f16 %1, wh3, xh3, %1; }"
        : "+f"(p0), "+f"(p1)
        : "r"(word), "r"(x.x), "r"(x.y), "r"(x.z), "r"(x.w));
}

// Same for B > 1: the four converted half2 are produced once and reused.
__device__ __forceinline__ void cvt8_e2m1(uint32_t word, uint32_t (&h)[4]) {
    asm("{ .reg .b8 b0, b1, b2, b3; mov.b32 {b0, b1, b2, b3}, %4;\n"
        "  cvt.rn.f16x2.e2m1x2 %0, b0; cvt.rn.f16x2.e2m1x2 %1, b1;\n"
        "  cvt.rn.f16x2.e2m1x2 %2, b2; cvt.rn.f16x2.e2m1x2 %3, b3; }"
        : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3])
        : "r"(word));
}
__device__ __forceinline__ void dot8_h2(const uint32_t (&h)[4], const uint4 &x, float &p0, float &p1) {
    asm("{ .reg .b16 wl0, wh0, wl1, wh1, wl2, wh2, wl3, wh3, xl0, xh0, xl1, xh1, xl2, xh2, xl3, xh3;\n"
        "  mov.b32 {wl0, wh0}, %2; mov.b32 {wl1, wh1}, %3; mov.b32 {wl2, wh2}, %4; mov.b32 {wl3, wh3}, %5;\n"
        "  mov.b32 {xl0, xh0}, %6; mov.b32 {xl1, xh1}, %7; mov.b32 {xl2, xh2}, %8; mov.b32 {xl3, xh3}, %9;\n"
        "  fma.rn.f32.f16 %0, wl0, xl0, %0; fma.rn.f32.f16 %1, wh0, xh0, %1;\n"
        "  fma.rn.f32.f16 %0, wl1, xl1, %0; fma.rn.f32.f16 %1, wh1, xh1, %1;\n"
        "  fma.rn.f32.f16 %0, wl2, xl2, %0; fma.rn.f32.f16 %1, wh2, xh2, %1;\n"
        "  fma.rn.f32.f16 %0, wl3, xl3, %0; fma.rn.f32.f16 %1, wh3, xh3, %1; }"
        : "+f"(p0), "+f"(p1)
        : "r"(h[0]), "r"(h[1]), "r"(h[2]), "r"(h[3]), "r"(x.x), "r"(x.y), "r"(x.z), "r"(x.w));
}

// Eight GF4 codes times B x eight activations.  The row's 16-entry fp16 table
// sits at byte offset rb (a multiple of 32 below 256) of a 256-byte aligned
// block tb of shared memory, so a lookup address is tb with its low byte
// replaced by rb | 2 * nibble: two shifts and two LOP3 put the eight doubled
// nibbles (OR-ed with rb) into the bytes of two registers, one PRMT per code
// splices a byte into the address, a 16-bit shared load fetches the entry,
// and it feeds the mixed-precision FMA as a 16-bit register (no repacking).
template <int B>
__device__ __forceinline__ void dot8_gf4(uint32_t word, uint32_t tb, uint32_t rb4, const uint4 (&x)[B], float (&part)[B][2]) {
    uint32_t m0, m1;  // bytes: 2 * nibbles {0,2,4,6} | rb  and  2 * nibbles {1,3,5,7} | rb
    asm("lop3.b32 %0, %1, 0x1e1e1e1e, %2, 0xea;" : "=r"(m0) : "r"(word << 1), "r"(rb4));  // (a & b) | c
    asm("lop3.b32 %0, %1, 0x1e1e1e1e, %2, 0xea;" : "=r"(m1) : "r"(word >> 3), "r"(rb4));
#pragma unroll
    for (int bb = 0; bb < 4; ++bb) {
        const uint32_t o0 = __byte_perm(m0, tb, 0x7650 + bb), o1 = __byte_perm(m1, tb, 0x7650 + bb);
        uint16_t w0, w1;
        asm volatile("ld.shared.u16 %0, [%1];" : "=h"(w0) : "r"(o0));
        asm volatile("ld.shared.u16 %0, [%1];" : "=h"(w1) : "r"(o1));
#pragma unroll
        for (int b = 0; b < B; ++b) {
            const uint32_t xx = bb == 0 ? x[b].x : (bb == 1 ? x[b].y : (bb == 2 ? x[b].z : x[b].w));
            asm("{ .reg .b16 xl, xh; mov.b32 {xl, xh}, %4;\n"
                "  fma.rn.f32.f16 %0, %2, xl, %0; fma.rn.f32.f16 %1, %3, xh, %1; }"
                : "+f"(part[b][0]), "+f"(part[b][1])
                : "h"(w0), "h"(w1), "r"(xx));
        }
    }
}

template <int FMT, int B, int DEPTH>
struct Ring {
    static constexpr int T = Tile<FMT, B>::T;                       // rows per stage
    static constexpr int kSlots = DEPTH * T;                   // 16-byte slots per thread
    static constexpr int kWBytes = kSlots * kThreads * 16;     // weight ring
    static constexpr int kSBytes = kSlots * kThreads * 4;      // scale-pair ring
    static constexpr int kTabBytes = kWarps * DEPTH * 256 + 256;  // GF4 codebooks: a 256-byte aligned block per warp and row group
    static constexpr int kBytes = kWBytes + kSBytes + kTabBytes;
};

// All row groups [rg_lo, rg_hi) of one problem, by one CTA.  Warp w takes the
// row groups rg_lo + w, rg_lo + w + kWarps, ...; a row group is T adjacent rows.
// Everything that is constant over a row group (row pointers, scale-pair
// parity) is computed once per row group, so that a stage costs little beyond
// its copies, its shared loads and the dot products themselves.
// End of a row group: reduce the T x B partial sums over the warp, write the
// outputs (and their copies into peer buffers), clear the accumulators.
template <int T, int B>
__device__ __forceinline__ void finish_rows(const GemvProblem &p, int crg, float (&acc)[T][B], int lane, const int *sexp,
                                            int y_dtype) {
    const int N = p.N;
#pragma unroll
    for (int r = 0; r < T; ++r)
#pragma unroll
        for (int b = 0; b < B; ++b) acc[r][b] = warp_sum(acc[r][b]);
    // every lane holds every sum: lane (copy c, row r) = c * T + r writes row r into copy c of the
    // output (copy 0 is the local buffer; further copies are peer GPUs' buffers, written over NVLink)
    {
        const int r_l = lane % T, c_l = lane / T;
        const int row = crg * T + r_l;
        if (c_l < p.npeer && row < N) {
            const float bias = p.bias ? p.bias[row] : 0.f;
            long long delta = 0;     // selected with constant indices: a variable index would put the problem in local memory
#pragma unroll
            for (int c = 0; c < 8; ++c) delta = (c == c_l) ? p.peer_delta[c] : delta;
            void *yc = reinterpret_cast<char *>(p.y) + delta;
#pragma unroll
            for (int b = 0; b < B; ++b) {
                float v = 0.f;
#pragma unroll
                for (int r = 0; r < T; ++r) v = (r == r_l) ? acc[r][b] : v;
                const float up = __uint_as_float((uint32_t)(127 + sexp[b]) << 23);  // 2^e
                store_out(yc, (size_t)b * p.ldy + row, fmaf(v, up, bias), y_dtype);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < T; ++r)
#pragma unroll
        for (int b = 0; b < B; ++b) acc[r][b] = 0.f;
}

// FAST (the caller checked fast_scales(p)): group scales exist and are fetched
// as aligned fp16 pairs by cp.async; the ragged end of a row is handled by
// zero-filling copies instead of branches (zero codes and zero scales times
// the zero-padded activation add nothing), so a stage has no data-dependent
// control flow.
__device__ __forceinline__ bool fast_scales(const GemvProblem &p) {
    const int gq = p.g >> 5;
    return p.g && (gq & (gq - 1)) == 0 && p.g <= 512 && (((size_t)p.N * p.lds) & 1) == 0 &&
           (reinterpret_cast<uintptr_t>(p.scales) & 3u) == 0;
}

template <int FMT, int B, int DEPTH, bool FAST>
__device__ void cta_rows(const GemvProblem &p, int rg_lo, int rg_hi, const __half *xs, const int *sexp,
                         unsigned char *ring_base, int y_dtype) {
    using R_ = Ring<FMT, B, DEPTH>;
    constexpr int T = R_::T;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int K = p.K, N = p.N, XS = xs_halves(K);
    const int stride_b = p.ldw;
    const int nchunks = jq_row_stride_codes(K) >> 5;
    const int nit = (nchunks + 31) >> 5;
    const int ngroups = p.lds;
    const int gq = p.g >> 5;                             // chunks per scale group
    const bool gpow2 = p.g && (gq & (gq - 1)) == 0;
    const int gshift = p.g ? (31 - __clz(gq)) : 0;
    // Fast scale path: 4-byte cp.async of the aligned fp16 pair holding this
    // lane's scale.  Needs a power-of-two group of at most 512 codes (so the
    // pair pointer advances by a constant, 4-byte-multiple step per stage), an
    // even element count (the pair never crosses the end) and an aligned base.
    const bool scale_async = FAST || (p.g && gpow2 && p.g <= 512 && (((size_t)N * ngroups) & 1) == 0 &&
                                      (reinterpret_cast<uintptr_t>(p.scales) & 3u) == 0);
    const int sadv = scale_async ? (2048 / p.g) : 0;     // bytes the pair pointer moves per stage (32 chunks)
    const int g_lane = p.g ? (gpow2 ? (lane >> gshift) : (lane * 32) / p.g) : 0;  // group of chunk `lane`

    const uint32_t wring = smem_u32(ring_base) + tid * 16;
    const uint32_t sring = smem_u32(ring_base + R_::kWBytes) + tid * 4;
    const uint32_t tabs = ((smem_u32(ring_base + R_::kWBytes + R_::kSBytes) + 255u) & ~255u) + warp * (DEPTH * 256);
    const uint32_t xs_u = smem_u32(xs) + lane * 16;

    const int first = rg_lo + warp;
    const int nrg = first < rg_hi ? (rg_hi - first + kWarps - 1) / kWarps : 0;
    const int total = nrg * nit;

    // ---- producer state ----
    int is = 0, ii = 0, irg = first, islot = 0, itab = 0;
    const uint8_t *wptr[T];
    const char *sptr[T];
    auto issue = [&]() {
        if (is < total) {
            if (ii == 0) {
#pragma unroll
                for (int r = 0; r < T; ++r) {
                    const int row = min(irg * T + r, N - 1);
                    wptr[r] = p.qw + (size_t)row * stride_b + lane * 16;
                    if (scale_async)
                        sptr[r] = reinterpret_cast<const char *>(p.scales) + (((size_t)row * ngroups + g_lane) & ~(size_t)1) * 2;
                }
                if (FMT == JQ_FMT_GF4) {
                    __syncwarp();  // nobody still reads the table buffer being replaced
                    if (lane < T * 2) {
                        const int row = min(irg * T + (lane >> 1), N - 1);
                        cp_async16(tabs + itab * 256 + lane * 16, p.codebook + (size_t)row * 16 + (lane & 1) * 8);
                    }
                }
            }
            if (FAST) {
                const uint32_t live = (lane + 32 * ii < nchunks) ? 1u : 0u;
#pragma unroll
                for (int r = 0; r < T; ++r) {
                    cp_async16_z(wring + (islot * T + r) * (kThreads * 16), wptr[r], live * 16u);
                    cp_async4_z(sring + (islot * T + r) * (kThreads * 4), sptr[r], live * 4u);
                }
            } else if (lane + 32 * ii < nchunks) {
#pragma unroll
                for (int r = 0; r < T; ++r) {
                    cp_async16(wring + (islot * T + r) * (kThreads * 16), wptr[r]);
                    if (scale_async) cp_async4(sring + (islot * T + r) * (kThreads * 4), sptr[r]);
                }
            }
#pragma unroll
            for (int r = 0; r < T; ++r) {
                wptr[r] += 512;
                if (scale_async) sptr[r] += sadv;
            }
            if (++ii == nit) { ii = 0; irg += kWarps; itab = (itab + 1 == DEPTH) ? 0 : itab + 1; }
        }
        ++is;
        islot = (islot + 1 == DEPTH) ? 0 : islot + 1;
        cp_async_commit();
    };

#pragma unroll
    for (int d = 0; d < DEPTH - 1; ++d) issue();

    float acc[T][B];
#pragma unroll
    for (int r = 0; r < T; ++r)
#pragma unroll
        for (int b = 0; b < B; ++b) acc[r][b] = 0.f;

    // ---- consumer state ----
    int ci = 0, crg = first, cslot = 0, ctab = 0;
    uint32_t sel[T];  // byte-permute selectors picking this lane's fp16 out of the copied pair
    for (int s = 0; s < total; ++s) {
        issue();
        cp_async_wait<DEPTH - 1>();
        if (ci == 0) {
            if (FMT == JQ_FMT_GF4) __syncwarp();  // the codebooks were copied by other lanes
            if (scale_async) {
#pragma unroll
                for (int r = 0; r < T; ++r) {
                    const int row = min(crg * T + r, N - 1);
                    sel[r] = ((row & ngroups & 1) ^ (g_lane & 1)) ? 0x4432u : 0x4410u;
                }
            }
        }
        const int c = lane + 32 * ci;
        if (FAST || c < nchunks) {
            uint4 w[T];
            float sc[T];
            float part[T][B][2];
#pragma unroll
            for (int r = 0; r < T; ++r) {
                w[r] = lds128(wring + (cslot * T + r) * (kThreads * 16));
                sc[r] = 1.f;
                if (FAST || p.g) {
                    uint32_t hb;
                    if (FAST || scale_async) {
                        hb = __byte_perm(lds32(sring + (cslot * T + r) * (kThreads * 4)), 0, sel[r]);
                    } else {
                        const int row = min(crg * T + r, N - 1);
                        const int gi = gpow2 ? (c >> gshift) : (c * 32) / p.g;
                        hb = reinterpret_cast<const uint16_t *>(p.scales)[(size_t)row * ngroups + gi];
                    }
                    sc[r] = __half2float(__ushort_as_half((uint16_t)hb));
                }
#pragma unroll
                for (int b = 0; b < B; ++b) part[r][b][0] = part[r][b][1] = 0.f;
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                uint4 xv[B];  // the 8 activations of 16-byte piece q, per batch row
#pragma unroll
                for (int b = 0; b < B; ++b) xv[b] = lds128(xs_u + (uint32_t)(b * XS + (((ci * 4 + q) * 32) << 3)) * 2);
#pragma unroll
                for (int r = 0; r < T; ++r) {
                    const uint32_t word = q == 0 ? w[r].x : (q == 1 ? w[r].y : (q == 2 ? w[r].z : w[r].w));
                    if (FMT == JQ_FMT_GF4) {
                        dot8_gf4<B>(word, tabs + ctab * 256, 0x20202020u * r, xv, part[r]);
                    } else if (B == 1) {
                        dot8_e2m1(word, xv[0], part[r][0][0], part[r][0][1]);
                    } else {
                        uint32_t h[4];
                        cvt8_e2m1(word, h);
#pragma unroll
                        for (int b = 0; b < B; ++b) dot8_h2(h, xv[b], part[r][b][0], part[r][b][1]);
                    }
                }
            }
#pragma unroll
            for (int r = 0; r < T; ++r)
#pragma unroll
                for (int b = 0; b < B; ++b) acc[r][b] = fmaf(part[r][b][0] + part[r][b][1], sc[r], acc[r][b]);
        }
        cslot = (cslot + 1 == DEPTH) ? 0 : cslot + 1;
        if (++ci == nit) {
            finish_rows<T, B>(p, crg, acc, lane, sexp, y_dtype);
            ci = 0;
            crg += kWarps;
            ctab = (ctab + 1 == DEPTH) ? 0 : ctab + 1;
        }
    }
    cp_async_wait<0>();
}

// GF4, groups present, batch 1..2: the shared-memory path is the bottleneck of
// this format (one 16-bit table load per code), so the packed rows do not pass
// through shared memory at all: every thread loads the 16 bytes (and the one
// scale) it will consume one stage ahead into registers.  A stage of four rows
// lasts longer than a DRAM round trip, so one stage in flight per thread (32 KB
// per SM) is enough to cover the latency.  Only the per-row tables go through
// shared memory (cp.async by the first 2T lanes, one 256-byte block per row
// group, DEPTH blocks per warp).
template <int B, int DEPTH>
__device__ void cta_rows_gf4_direct(const GemvProblem &p, int rg_lo, int rg_hi, const __half *xs, const int *sexp,
                                    unsigned char *ring_base, int y_dtype) {
    using R_ = Ring<JQ_FMT_GF4, B, DEPTH>;
    constexpr int T = R_::T;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int K = p.K, N = p.N, XS = xs_halves(K);
    const int stride_b = p.ldw;
    const int nchunks = jq_row_stride_codes(K) >> 5;
    const int nit = (nchunks + 31) >> 5;
    const int ngroups = p.lds;
    const int gshift = 31 - __clz(p.g >> 5);
    const int g_lane = lane >> gshift;                   // group of chunk `lane` within a stage
    const int sadv = 1024 / p.g;                         // scales a stage advances by
    const uint32_t tabs = ((smem_u32(ring_base + R_::kWBytes + R_::kSBytes) + 255u) & ~255u) + warp * (DEPTH * 256);
    const uint32_t xs_u = smem_u32(xs) + lane * 16;

    const int first = rg_lo + warp;
    const int nrg = first < rg_hi ? (rg_hi - first + kWarps - 1) / kWarps : 0;
    const int total = nrg * nit;

    // ---- producer state: the stage whose loads are issued next ----
    int is = 0, ii = 0, irg = first, itab = 0;
    const uint8_t *wptr[T];
    const __half *sptr[T];
    auto fetch = [&](uint4 (&wn)[T], uint32_t (&sn)[T]) {
        if (is < total) {
            if (ii == 0) {
#pragma unroll
                for (int r = 0; r < T; ++r) {
                    const int row = min(irg * T + r, N - 1);
                    wptr[r] = p.qw + (size_t)row * stride_b + lane * 16;
                    sptr[r] = p.scales + (size_t)row * ngroups + g_lane;
                }
                __syncwarp();  // nobody still reads the table block being replaced
                if (lane < T * 2) {
                    const int row = min(irg * T + (lane >> 1), N - 1);
                    cp_async16(tabs + itab * 256 + lane * 16, p.codebook + (size_t)row * 16 + (lane & 1) * 8);
                }
                cp_async_commit();
            }
            const bool live = lane + 32 * ii < nchunks;
#pragma unroll
            for (int r = 0; r < T; ++r) {
                wn[r] = make_uint4(0u, 0u, 0u, 0u);
                sn[r] = 0u;
                if (live) {
                    wn[r] = ldg_stream_u4(wptr[r]);
                    sn[r] = __ldg(reinterpret_cast<const unsigned short *>(sptr[r]));
                }
                wptr[r] += 512;
                sptr[r] += sadv;
            }
            if (++ii == nit) { ii = 0; irg += kWarps; itab = (itab + 1 == DEPTH) ? 0 : itab + 1; }
        }
        ++is;
    };

    float acc[T][B];
#pragma unroll
    for (int r = 0; r < T; ++r)
#pragma unroll
        for (int b = 0; b < B; ++b) acc[r][b] = 0.f;

    // ---- consumer state ----
    int ci = 0, crg = first, ctab = 0;
    auto consume = [&](const uint4 (&w)[T], const uint32_t (&sn)[T]) {
        if (ci == 0) {
            cp_async_wait<0>();  // this row group's tables (copied by the first lanes one stage ago)
            __syncwarp();
        }
        float part[T][B][2];
#pragma unroll
        for (int r = 0; r < T; ++r)
#pragma unroll
            for (int b = 0; b < B; ++b) part[r][b][0] = part[r][b][1] = 0.f;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            uint4 xv[B];
#pragma unroll
            for (int b = 0; b < B; ++b) xv[b] = lds128(xs_u + (uint32_t)(b * XS + (((ci * 4 + q) * 32) << 3)) * 2);
#pragma unroll
            for (int r = 0; r < T; ++r) {
                const uint32_t word = q == 0 ? w[r].x : (q == 1 ? w[r].y : (q == 2 ? w[r].z : w[r].w));
                dot8_gf4<B>(word, tabs + ctab * 256, 0x20202020u * r, xv, part[r]);
            }
        }
#pragma unroll
        for (int r = 0; r < T; ++r) {
            const float sc = __half2float(__ushort_as_half((unsigned short)sn[r]));
#pragma unroll
            for (int b = 0; b < B; ++b) acc[r][b] = fmaf(part[r][b][0] + part[r][b][1], sc, acc[r][b]);
        }
        if (++ci == nit) {
            finish_rows<T, B>(p, crg, acc, lane, sexp, y_dtype);
            ci = 0;
            crg += kWarps;
            ctab = (ctab + 1 == DEPTH) ? 0 : ctab + 1;
        }
    };

    uint4 wa[T], wb[T];
    uint32_t sa[T], sb[T];
    fetch(wa, sa);
    for (int s = 0; s < total; s += 2) {
        fetch(wb, sb);
        consume(wa, sa);
        fetch(wa, sa);
        if (s + 1 < total) consume(wb, sb);
    }
    cp_async_wait<0>();
}

// ---- E2M1, batch 2..8: the dot products on mma.sync.m16n8k16 ---------------------
// With more than one batch row the FMA loops above pay one FMA per code and
// batch row and become issue bound.  Here a warp owns 16 rows; the decoded fp16
// weights are the A operand (16 rows x 16 codes) and the staged fp16 activation
// the B operand (16 codes x 8 batch columns) of the legacy warp-level MMA, which
// costs one instruction per 256 codes whatever the batch (up to 8).  Products
// fp16 x fp16 and the fp32 accumulation stay as in the FMA loops.  The group
// scale (one per row and 32 codes) cannot enter the MMA, so every 32-code chunk
// (two MMAs) starts from a zero accumulator and is folded into the running sum
// with one fp32 FMA per output.  Thread (g = lane / 4, t = lane % 4) feeds rows
// g and g + 8 with the 8 codes of 32-bit word t of the chunk and batch column g
// with the matching 8 activations; it ends up with the finished sums of rows
// g, g + 8 x batch columns 2t, 2t + 1: no reduction across lanes at all.
//
// Staging: a stage is 16 rows x 8 chunks (128 bytes per row), copied with four
// 16-byte cp.async per lane into a per-warp slot whose 16-byte columns are
// XOR-swizzled by the row so that the fragment reads (one 32-bit word per lane)
// hit 32 different banks; the stage's 16 x 8 scales follow with one more copy
// by the first 16 lanes.  Lanes consume what other lanes copied, so one
// __syncwarp per stage orders the ring; nothing spins.
constexpr int kMmaStageBytes = 16 * 128 + 16 * 16;  // weights + scales

template <int DEPTH>
struct MmaRing {
    static constexpr int kCombBytes = 2 * kWarps * 32 * 16;   // partial sums of K parts: two rounds x warps x lanes x 4 floats
    static constexpr int kBytes = kWarps * DEPTH * kMmaStageBytes + kCombBytes + 128;  // + slack to start at a 128-byte boundary
};

// GF4: the same slots, plus 2 KB of lookup table per warp (two warps share a
// 4 KB aligned block, see cta_rows_mma_gf4).
template <int DEPTH>
struct MmaRingGf4 {
    static constexpr int kTabBytes = (kWarps / 2) * 4096 + 4096;   // + slack to start at a 4 KB boundary
    static constexpr int kBytes = MmaRing<DEPTH>::kBytes + kTabBytes;
};

// The problem suits the MMA row loop.  E2M1: one scale per 32-code chunk, whole
// 8-chunk stages, 16-byte aligned scale rows.  GF4: 128-code groups (two per
// stage and row, copied as one aligned fp16 pair), 16-byte aligned codebooks.
template <int FMT>
__host__ __device__ inline bool mma_ok_raw(int g, int K, const void *scales, const void *codebook) {
    if (FMT == JQ_FMT_E2M1) return g == 32 && (K & 255) == 0 && (reinterpret_cast<uintptr_t>(scales) & 15u) == 0;
    return g == 128 && (K & 255) == 0 && (reinterpret_cast<uintptr_t>(scales) & 3u) == 0 &&
           (reinterpret_cast<uintptr_t>(codebook) & 15u) == 0;
}
template <int FMT>
__device__ __forceinline__ bool mma_ok(const GemvProblem &p) {
    return mma_ok_raw<FMT>(p.g, p.K, p.scales, p.codebook) && (FMT == JQ_FMT_E2M1 ? (p.lds & 7) == 0 : (p.lds & 1) == 0);
}

// K parts a row group is cut into (a function of K alone, so that every launch
// and every row shard of a matrix sums in the same order): 16 rows x all of K
// is a coarse unit of work for 16 warps per SM, and a row group's parts run on
// adjacent warps in the same round.
__host__ __device__ inline int mma_ksplit_log2(int K) {
    const int nit = K >> 8;
    return (nit >= 8 && (nit & 3) == 0) ? 2 : ((nit >= 4 && (nit & 1) == 0) ? 1 : 0);
}

__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1, const float (&c)[4]) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
}

// End of a task of the MMA row loops.  acc = this K part's sums of rows g, g + 8
// x batch columns 2t, 2t + 1 (g = lane / 4, t = lane % 4).  The parts of a row
// group are joined in part order, then the first part's warp writes the outputs
// (or, in a K-tiled launch, adds them to the chunk's table in shared memory).
template <int B>
__device__ __forceinline__ void mma_task_end(const GemvProblem &p, float (&acc)[4], int ctask, int ksh, int &cpar,
                                             float4 *comb, const int *sexp, int y_dtype, float *partial,
                                             int partial_rg0, bool partial_first) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int ks = 1 << ksh, N = p.N;
    // acc = this K part's sums of rows g, g + 8 x batch columns 2t, 2t + 1
    bool writer = true;
    if (ks > 1) {
        // the parts of a row group sit on ks adjacent warps in the same round: all but the first
        // park their sums in shared memory (two alternating sets, so that a set is never rewritten
        // before its reader has passed the next round's barrier), the first adds them in part order
        writer = (warp & (ks - 1)) == 0;
        float4 *mine = comb + (cpar * kWarps + warp) * 32 + lane;
        if (!writer) *mine = make_float4(acc[0], acc[1], acc[2], acc[3]);
        asm volatile("bar.sync %0, %1;" ::"r"(1 + (warp >> ksh)), "r"(ks * 32) : "memory");
        if (writer) {
            for (int q = 1; q < ks; ++q) {
                const float4 o = mine[q * 32];
                acc[0] += o.x; acc[1] += o.y; acc[2] += o.z; acc[3] += o.w;
            }
        }
        cpar ^= 1;
    }
    if (writer && partial) {
        // one K tile of several: the sums go to the chunk's [row][batch] table in shared memory
        const int rg = ctask >> ksh;
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int b = 2 * t + j;
                if (b < B) {
                    float *dst = partial + ((rg - partial_rg0) * 16 + g + 8 * h) * B + b;
                    *dst = partial_first ? acc[2 * h + j] : *dst + acc[2 * h + j];
                }
            }
    } else if (writer) {
        const int rg = ctask >> ksh;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = rg * 16 + g + 8 * h;
            if (row < N) {
                const float bias = p.bias ? p.bias[row] : 0.f;
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int b = 2 * t + j;
                    if (b < B) {
                        const float up = __uint_as_float((uint32_t)(127 + sexp[b]) << 23);  // 2^e
                        const float v = fmaf(acc[2 * h + j], up, bias);
                        store_out_copies(p.y, p.peer_delta, p.npeer, (size_t)b * p.ldy + row, v, y_dtype);
                    }
                }
            }
        }
    }
}

template <int B, int DEPTH>
__device__ void cta_rows_mma(const GemvProblem &p, int rg_lo, int rg_hi, const __half *xs, const int *sexp,
                             unsigned char *ring_base, int y_dtype, float *partial = nullptr, int partial_rg0 = 0,
                             bool partial_first = true) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int N = p.N, XSB = xs_halves(p.K) + kXPad;
    const int nit = p.K >> 8;                            // stages (8 chunks of 32 codes) per row
    // 128-byte aligned slots (a stage is a multiple of 128 bytes), so that bits 4..6 of a row's address are free
    const uint32_t ring = ((smem_u32(ring_base) + 127u) & ~127u) + warp * (DEPTH * kMmaStageBytes);
    // producer addressing: copy i of a stage moves chunk (lane & 7) of row (lane >> 3) + 4 i
    const int prow = lane >> 3, pch = lane & 7;
    // consumer addressing: chunk c of row g sits in 16-byte column c ^ g, i.e. at (base | g << 4) ^ (c << 4)
    const uint32_t cw = ring + g * 128 + (g << 4) + t * 4;           // ^ (c << 4); + 1024 for row g + 8
    const uint32_t cs = ring + 2048 + g * 16;                        // scales of row g; + 128 for row g + 8
    // batch columns beyond B read batch row B - 1: their outputs are never stored
    const uint32_t xs_u = smem_u32(xs) + (uint32_t)(min(g, B - 1) * XSB + t * 8) * 2;

    // a task = (row group, K part); part q of a row group covers stages [q nitp, (q + 1) nitp)
    const int ksh = mma_ksplit_log2(p.K), ks = 1 << ksh, nitp = nit >> ksh;
    const int first = (rg_lo << ksh) + warp, task_end = rg_hi << ksh;
    const int ntask = first < task_end ? (task_end - first + kWarps - 1) / kWarps : 0;
    const int total = ntask * nitp;
    float4 *comb = reinterpret_cast<float4 *>(ring_base + (MmaRing<DEPTH>::kBytes - MmaRing<DEPTH>::kCombBytes));

    // ---- producer state ----
    int is = 0, ii = 0, itask = first, islot = 0;
    const uint8_t *wptr[4];
    const __half *sptr = nullptr;
    auto issue = [&]() {
        if (is < total) {
            if (ii == 0) {
                const int rg = itask >> ksh, part = itask & (ks - 1);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int row = min(rg * 16 + 4 * i + prow, N - 1);
                    wptr[i] = p.qw + (size_t)row * p.ldw + (part * nitp * 8 + pch) * 16;
                }
                sptr = p.scales + (size_t)min(rg * 16 + (lane & 15), N - 1) * p.lds + part * nitp * 8;
            }
            const uint32_t slot = islot * kMmaStageBytes;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                // row 4 i + prow: its swizzle key is (row & 7) = (4 i + prow) & 7
                const uint32_t key = (uint32_t)((4 * i + prow) & 7);
                cp_async16(ring + slot + (4 * i + prow) * 128 + ((pch ^ key) << 4), wptr[i]);
                wptr[i] += 128;
            }
            if (lane < 16) cp_async16(ring + slot + 2048 + lane * 16, sptr);
            sptr += 8;
            if (++ii == nitp) { ii = 0; itask += kWarps; }
        }
        ++is;
        islot = (islot + 1 == DEPTH) ? 0 : islot + 1;
        cp_async_commit();
    };

#pragma unroll
    for (int d = 0; d < DEPTH - 1; ++d) issue();

    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    const float zero[4] = {0.f, 0.f, 0.f, 0.f};
    int ci = 0, ctask = first, cslot = 0, cpar = 0;
    for (int s = 0; s < total; ++s) {
        cp_async_wait<DEPTH - 2>();   // this thread's copies of stage s have landed
        __syncwarp();                 // ... and everyone's; everyone has also finished reading stage s - 1
        issue();                      // refills the slot of stage s - 1
        const uint32_t slot = cslot * kMmaStageBytes;
        const uint4 sa = lds128(cs + slot), sb = lds128(cs + slot + 128);   // 8 scales of rows g and g + 8
        const uint32_t xbase = xs_u + (uint32_t)(((ctask & (ks - 1)) * nitp + ci) * 256) * 2;
        const uint32_t cwslot = cw + slot;
#pragma unroll
        for (int c2 = 0; c2 < 4; ++c2) {
            const uint32_t pa = c2 == 0 ? sa.x : (c2 == 1 ? sa.y : (c2 == 2 ? sa.z : sa.w));
            const uint32_t pb = c2 == 0 ? sb.x : (c2 == 1 ? sb.y : (c2 == 2 ? sb.z : sb.w));
            const float2 fa = __half22float2(*reinterpret_cast<const __half2 *>(&pa));
            const float2 fb = __half22float2(*reinterpret_cast<const __half2 *>(&pb));
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int c = 2 * c2 + j;
                const uint32_t a = cwslot ^ (uint32_t)(c << 4);
                const uint32_t wa = lds32(a), wb = lds32(a + 1024);
                const uint4 xv = lds128(xbase + c * 64);
                uint32_t ha[4], hb[4];
                cvt8_e2m1(wa, ha);
                cvt8_e2m1(wb, hb);
                float d[4];
                mma16816(d, ha[0], hb[0], ha[1], hb[1], xv.x, xv.y, zero);
                mma16816(d, ha[2], hb[2], ha[3], hb[3], xv.z, xv.w, d);
                const float sca = j ? fa.y : fa.x, scb = j ? fb.y : fb.x;
                acc[0] = fmaf(d[0], sca, acc[0]);
                acc[1] = fmaf(d[1], sca, acc[1]);
                acc[2] = fmaf(d[2], scb, acc[2]);
                acc[3] = fmaf(d[3], scb, acc[3]);
            }
        }
        cslot = (cslot + 1 == DEPTH) ? 0 : cslot + 1;
        if (++ci == nitp) {
            mma_task_end<B>(p, acc, ctask, ksh, cpar, comb, sexp, y_dtype, partial, partial_rg0, partial_first);
            acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
            ci = 0;
            ctask += kWarps;
        }
    }
    cp_async_wait<0>();
}

// ---- GF4, batch 2..8: table lookups feeding mma.sync.m16n8k16 --------------------
// Same tasks, ring, fragments and task end as cta_rows_mma; what differs is the
// decode.  In the MMA layout the 32 lanes of a lookup instruction belong to 8
// different rows, so a shared 32-byte table per row would collide in the banks.
// Instead every lane owns one 4-byte column of a [16 entries][32 lanes] table:
// the word of entry e holds {codebook[row g][e], codebook[row g + 8][e]} of the
// lane's own two rows (the 4 lanes of a row hold identical copies).  A lookup
// never leaves the lane's own bank: conflict-free whatever the codes.  Entries
// are 256 bytes apart (two warps interleave their 128-byte halves in a 4 KB
// aligned block), so the entry index is bits 8..11 of the address and one PRMT
// splices a nibble (OR-ed with the block's address bits 12..15) into byte 1.
// The table is rebuilt per task from codebook rows prefetched into registers a
// task ahead.  Group scales (128 codes = 4 chunks) are applied after four
// chunks' MMAs, not after each.
__device__ __forceinline__ void gf4_lookup8(uint32_t w, uint32_t tb, uint32_t hb4, uint32_t (&h)[4]) {
    uint32_t m0, m1;  // bytes: nibbles {0,2,4,6} | hb  and  nibbles {1,3,5,7} | hb
    asm("lop3.b32 %0, %1, 0x0f0f0f0f, %2, 0xea;" : "=r"(m0) : "r"(w), "r"(hb4));       // (a & b) | c
    asm("lop3.b32 %0, %1, 0x0f0f0f0f, %2, 0xea;" : "=r"(m1) : "r"(w >> 4), "r"(hb4));
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint32_t a0 = __byte_perm(m0, tb, 0x7604 | (j << 4)), a1 = __byte_perm(m1, tb, 0x7604 | (j << 4));
        uint32_t v0, v1;
        asm volatile("ld.shared.u16 %0, [%1];" : "=r"(v0) : "r"(a0));
        asm volatile("ld.shared.u16 %0, [%1];" : "=r"(v1) : "r"(a1));
        asm("mad.lo.u32 %0, %1, 65536, %2;" : "=r"(h[j]) : "r"(v1), "r"(v0));   // pack on the FMA pipe
    }
}

template <int B, int DEPTH>
__device__ void cta_rows_mma_gf4(const GemvProblem &p, int rg_lo, int rg_hi, const __half *xs, const int *sexp,
                                 unsigned char *ring_base, int y_dtype, float *partial = nullptr, int partial_rg0 = 0,
                                 bool partial_first = true) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int N = p.N, XSB = xs_halves(p.K) + kXPad;
    const int nit = p.K >> 8;                            // stages (8 chunks of 32 codes = 2 scale groups) per row
    const uint32_t ring = ((smem_u32(ring_base) + 127u) & ~127u) + warp * (DEPTH * kMmaStageBytes);
    const int prow = lane >> 3, pch = lane & 7;
    const uint32_t cw = ring + g * 128 + (g << 4) + t * 4;           // ^ (c << 4); + 1024 for row g + 8
    const uint32_t cs = ring + 2048 + g * 4;                         // scale pair of row g; + 32 for row g + 8
    const uint32_t xs_u = smem_u32(xs) + (uint32_t)(min(g, B - 1) * XSB + t * 8) * 2;
    float4 *comb = reinterpret_cast<float4 *>(ring_base + (MmaRing<DEPTH>::kBytes - MmaRing<DEPTH>::kCombBytes));
    // this lane's table column: entry e at tcol + 256 e, row g in the low half, row g + 8 in the high half
    const uint32_t tcol = ((smem_u32(ring_base) + MmaRing<DEPTH>::kBytes + 4095u) & ~4095u) + (warp >> 1) * 4096 +
                          (warp & 1) * 128 + lane * 4;
    const uint32_t hb4 = ((tcol >> 8) & 0xf0u) * 0x01010101u;

    const int ksh = mma_ksplit_log2(p.K), ks = 1 << ksh, nitp = nit >> ksh;
    const int first = (rg_lo << ksh) + warp, task_end = rg_hi << ksh;
    const int ntask = first < task_end ? (task_end - first + kWarps - 1) / kWarps : 0;
    const int total = ntask * nitp;

    // ---- producer state ----
    int is = 0, ii = 0, itask = first, islot = 0;
    const uint8_t *wptr[4];
    const __half *sptr = nullptr;
    auto issue = [&]() {
        if (is < total) {
            if (ii == 0) {
                const int rg = itask >> ksh, part = itask & (ks - 1);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int row = min(rg * 16 + 4 * i + prow, N - 1);
                    wptr[i] = p.qw + (size_t)row * p.ldw + (part * nitp * 8 + pch) * 16;
                }
                sptr = p.scales + (size_t)min(rg * 16 + (lane & 15), N - 1) * p.lds + part * nitp * 2;
            }
            const uint32_t slot = islot * kMmaStageBytes;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t key = (uint32_t)((4 * i + prow) & 7);
                cp_async16(ring + slot + (4 * i + prow) * 128 + ((pch ^ key) << 4), wptr[i]);
                wptr[i] += 128;
            }
            if (lane < 16) cp_async4(ring + slot + 2048 + lane * 4, sptr);
            sptr += 2;
            if (++ii == nitp) { ii = 0; itask += kWarps; }
        }
        ++is;
        islot = (islot + 1 == DEPTH) ? 0 : islot + 1;
        cp_async_commit();
    };

    // codebook rows g and g + 8 of a task's row group, as 2 x 2 16-byte halves
    uint4 cb[4];
    auto fetch_tables = [&](int task) {
        if (task < task_end) {
            const int rg = task >> ksh;
            const uint4 *ra = reinterpret_cast<const uint4 *>(p.codebook + (size_t)min(rg * 16 + g, N - 1) * 16);
            const uint4 *rb = reinterpret_cast<const uint4 *>(p.codebook + (size_t)min(rg * 16 + g + 8, N - 1) * 16);
            cb[0] = __ldg(ra); cb[1] = __ldg(ra + 1); cb[2] = __ldg(rb); cb[3] = __ldg(rb + 1);
        }
    };
    auto build_tables = [&]() {
        const uint32_t a[8] = {cb[0].x, cb[0].y, cb[0].z, cb[0].w, cb[1].x, cb[1].y, cb[1].z, cb[1].w};
        const uint32_t b[8] = {cb[2].x, cb[2].y, cb[2].z, cb[2].w, cb[3].x, cb[3].y, cb[3].z, cb[3].w};
#pragma unroll
        for (int e2 = 0; e2 < 8; ++e2) {
            // entries 2 e2 and 2 e2 + 1: {row g, row g + 8} pairs
            const uint32_t lo = __byte_perm(a[e2], b[e2], 0x5410), hi = __byte_perm(a[e2], b[e2], 0x7632);
            asm volatile("st.shared.u32 [%0], %1;" ::"r"(tcol + (2 * e2) * 256), "r"(lo) : "memory");
            asm volatile("st.shared.u32 [%0], %1;" ::"r"(tcol + (2 * e2 + 1) * 256), "r"(hi) : "memory");
        }
    };

#pragma unroll
    for (int d = 0; d < DEPTH - 1; ++d) issue();
    fetch_tables(first);

    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    const float zero[4] = {0.f, 0.f, 0.f, 0.f};
    int ci = 0, ctask = first, cslot = 0, cpar = 0;
    for (int s = 0; s < total; ++s) {
        if (ci == 0) {
            build_tables();                    // own column only: no other lane reads it
            fetch_tables(ctask + kWarps);      // the next task's rows, in flight during this task
        }
        cp_async_wait<DEPTH - 2>();   // this thread's copies of stage s have landed
        __syncwarp();                 // ... and everyone's; everyone has also finished reading stage s - 1
        issue();                      // refills the slot of stage s - 1
        const uint32_t slot = cslot * kMmaStageBytes;
        const uint32_t pa = lds32(cs + slot), pb = lds32(cs + slot + 32);   // 2 scales of rows g and g + 8
        const float2 fa = __half22float2(*reinterpret_cast<const __half2 *>(&pa));
        const float2 fb = __half22float2(*reinterpret_cast<const __half2 *>(&pb));
        const uint32_t xbase = xs_u + (uint32_t)(((ctask & (ks - 1)) * nitp + ci) * 256) * 2;
        const uint32_t cwslot = cw + slot;
#pragma unroll
        for (int hs = 0; hs < 2; ++hs) {       // the stage's two scale groups
            float d[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int c = 4 * hs + j;
                const uint32_t a = cwslot ^ (uint32_t)(c << 4);
                const uint32_t wa = lds32(a), wb = lds32(a + 1024);
                const uint4 xv = lds128(xbase + c * 64);
                uint32_t ha[4], hb[4];
                gf4_lookup8(wa, tcol, hb4, ha);
                gf4_lookup8(wb, tcol + 2, hb4, hb);
                if (j == 0) mma16816(d, ha[0], hb[0], ha[1], hb[1], xv.x, xv.y, zero);
                else mma16816(d, ha[0], hb[0], ha[1], hb[1], xv.x, xv.y, d);
                mma16816(d, ha[2], hb[2], ha[3], hb[3], xv.z, xv.w, d);
            }
            const float sca = hs ? fa.y : fa.x, scb = hs ? fb.y : fb.x;
            acc[0] = fmaf(d[0], sca, acc[0]);
            acc[1] = fmaf(d[1], sca, acc[1]);
            acc[2] = fmaf(d[2], scb, acc[2]);
            acc[3] = fmaf(d[3], scb, acc[3]);
        }
        cslot = (cslot + 1 == DEPTH) ? 0 : cslot + 1;
        if (++ci == nitp) {
            mma_task_end<B>(p, acc, ctask, ksh, cpar, comb, sexp, y_dtype, partial, partial_rg0, partial_first);
            acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
            ci = 0;
            ctask += kWarps;
        }
    }
    cp_async_wait<0>();
}

constexpr int kGf4DirectMaxB = 1;   // GF4 batches up to here load the packed rows straight to registers
// the row loop that suits the problem (uniform over the CTA)
template <int FMT, int B, int DEPTH>
__device__ __forceinline__ void run_rows(const GemvProblem &p, int rg_lo, int rg_hi, const __half *xs, const int *sexp,
                                         unsigned char *ring_base, int y_dtype) {
    if constexpr (Tile<FMT, B>::kMma) {
        if (mma_ok<FMT>(p)) {
            if constexpr (FMT == JQ_FMT_GF4) cta_rows_mma_gf4<B, DEPTH>(p, rg_lo, rg_hi, xs, sexp, ring_base, y_dtype);
            else cta_rows_mma<B, DEPTH>(p, rg_lo, rg_hi, xs, sexp, ring_base, y_dtype);
            return;
        }
    }
    // the FMA loops count row groups of Tile::T rows
    constexpr int kSub = Tile<FMT, B>::R / Tile<FMT, B>::T;
    rg_lo *= kSub;
    rg_hi *= kSub;
    if (fast_scales(p)) {
        if constexpr (FMT == JQ_FMT_GF4 && B <= kGf4DirectMaxB)
            cta_rows_gf4_direct<B, DEPTH>(p, rg_lo, rg_hi, xs, sexp, ring_base, y_dtype);
        else
            cta_rows<FMT, B, DEPTH, true>(p, rg_lo, rg_hi, xs, sexp, ring_base, y_dtype);
    } else {
        cta_rows<FMT, B, DEPTH, false>(p, rg_lo, rg_hi, xs, sexp, ring_base, y_dtype);
    }
}

// shared memory of the row loops a kernel instance may run: the larger ring,
// the wider activation rows
template <int FMT, int B, int DEPTH>
__host__ __device__ constexpr int ring_bytes() {
    constexpr int mma = FMT == JQ_FMT_GF4 ? MmaRingGf4<DEPTH>::kBytes : MmaRing<DEPTH>::kBytes;
    return (Tile<FMT, B>::kMma && mma > Ring<FMT, B, DEPTH>::kBytes) ? mma : Ring<FMT, B, DEPTH>::kBytes;
}
template <int FMT, int B>
__host__ __device__ inline int xs_stride(int K) { return xs_halves(K) + (Tile<FMT, B>::kMma ? kXPad : 0); }

struct SmemLayout {
    __half *xs;
    float *sred;
    int *sexp;
    unsigned char *ring;
};

constexpr int kSmallBytes = 128;  // reduction scratch (kWarps floats) + exponents (8 ints), with padding
// xhalves: halves of the activation region (the small arrays sit behind it)
template <int FMT, int B, int DEPTH>
__device__ __forceinline__ SmemLayout carve(unsigned char *smem, int xhalves) {
    SmemLayout L;
    L.ring = smem;  // 16-byte aligned slots first
    // (the activation directly behind the ring: with the small arrays in between the GF4 batch-1 loop
    // measured 3.5 % slower)
    L.xs = reinterpret_cast<__half *>(smem + ring_bytes<FMT, B, DEPTH>());
    L.sred = reinterpret_cast<float *>(L.xs + ((xhalves + 7) & ~7));
    L.sexp = reinterpret_cast<int *>(L.sred + kWarps);
    return L;
}

// B x K halves do not fit in the activation region (xcap halves): the CTA walks
// its row groups in chunks and, per chunk, the K range in tiles.  Each tile's
// activation is staged in the first half of the region, the chunk's partial
// sums (fp32, [row][batch]) live in the rest and are turned into outputs after
// the last tile.  The normalisation exponent is that of the whole row, so the
// tiles add up in one scale.
template <int FMT, int B, int DEPTH>
__device__ void rows_k_tiled(const GemvProblem &p, int rg_lo, int rg_hi, const SmemLayout &L, int xcap, int x_dtype,
                             int y_dtype) {
    const int tileK = ((xcap / 2) / B - kXPad) / 1024 * 1024;
    const int xuse = (B * (tileK + kXPad) + 7) & ~7;              // halves, keeps the partial sums 16-byte aligned
    float *partial = reinterpret_cast<float *>(L.xs + xuse);
    const int chunk = ((xcap - xuse) / 2) / (16 * B);             // row groups whose partial sums fit
    if (tileK < 1024 || chunk < 1) return;                        // (the host never launches such a case)
    const size_t xe = x_dtype == JQ_F32 ? 4 : 2;
    for (int c0 = rg_lo; c0 < rg_hi; c0 += chunk) {
        const int c1 = min(rg_hi, c0 + chunk);
        for (int k0 = 0; k0 < p.K; k0 += tileK) {
            GemvProblem q = p;
            q.K = min(tileK, p.K - k0);
            q.qw = p.qw + (k0 >> 1);
            q.scales = p.scales + k0 / p.g;
            q.x = reinterpret_cast<const char *>(p.x) + (size_t)k0 * xe;
            __syncthreads();  // the previous tile's activation is no longer read
            stage_activation<B>(q, x_dtype, L.xs, L.sred, L.sexp, true, !(c0 == rg_lo && k0 == 0));
            if constexpr (FMT == JQ_FMT_GF4)
                cta_rows_mma_gf4<B, DEPTH>(q, c0, c1, L.xs, L.sexp, L.ring, y_dtype, partial, c0, k0 == 0);
            else
                cta_rows_mma<B, DEPTH>(q, c0, c1, L.xs, L.sexp, L.ring, y_dtype, partial, c0, k0 == 0);
        }
        __syncthreads();
        for (int i = threadIdx.x; i < (c1 - c0) * 16 * B; i += kThreads) {
            const int row = c0 * 16 + i / B, b = i % B;
            if (row < p.N) {
                const float up = __uint_as_float((uint32_t)(127 + L.sexp[b]) << 23);  // 2^e
                const float v = fmaf(partial[i], up, p.bias ? p.bias[row] : 0.f);
                store_out_copies(p.y, p.peer_delta, p.npeer, (size_t)b * p.ldy + row, v, y_dtype);
            }
        }
    }
}

template <int FMT, int B, int DEPTH>
__global__ void __launch_bounds__(kThreads, 1) gemv_kernel(GemvProblem p, int x_dtype, int y_dtype) {
    extern __shared__ __align__(16) unsigned char smem[];
    const SmemLayout L = carve<FMT, B, DEPTH>(smem, B * xs_stride<FMT, B>(p.K));
    stage_activation<B>(p, x_dtype, L.xs, L.sred, L.sexp, Tile<FMT, B>::kMma && mma_ok<FMT>(p));
    constexpr int T = Tile<FMT, B>::R;
    const long long nrg = (p.N + T - 1) / T;
    const int lo = (int)(nrg * blockIdx.x / gridDim.x), hi = (int)(nrg * (blockIdx.x + 1) / gridDim.x);
    run_rows<FMT, B, DEPTH>(p, lo, hi, L.xs, L.sexp, L.ring, y_dtype);
}

struct PeerInfo {
    int n;
    long long delta[8];
};

// Grouped launch: the concatenated row-group space of all problems is split
// into contiguous, byte-balanced CTA ranges on the host (cta_first[]); a CTA
// re-stages the activation whenever it crosses into the next problem.  With
// peers.n > 1 every output element is also stored into the same offset of the
// peers' output buffers (the all-gather of a row-sharded layer, fused into the
// epilogue as plain stores over NVLink).
template <int FMT, int B, int DEPTH>
__global__ void __launch_bounds__(kThreads, 1) gemv_grouped_kernel(const jq_problem *probs, int nprob,
                                                                     const int *rg_start, const int *cta_first,
                                                                     int xcap, int x_dtype, int y_dtype, PeerInfo peers) {
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ int s_prob;
    const SmemLayout L = carve<FMT, B, DEPTH>(smem, xcap);
    int rg = cta_first[blockIdx.x];
    const int rg_end = cta_first[blockIdx.x + 1];
    int pi = -1;
    while (rg < rg_end) {
        if (threadIdx.x == 0) {
            int q = pi;
            if (q < 0) {
                // the CTA's first problem: bisect (a scan from problem 0 is a chain of dependent global loads,
                // 0.2 us each, that the CTAs of the last problems would pay before their first row)
                int lo = 0, hi = nprob - 1;
                while (lo < hi) {
                    const int mid = (lo + hi + 1) >> 1;
                    if (rg_start[mid] <= rg) lo = mid; else hi = mid - 1;
                }
                q = lo;
            } else {
                while (q + 1 < nprob && rg_start[q + 1] <= rg) ++q;
            }
            s_prob = q;
        }
        __syncthreads();
        pi = s_prob;
        const jq_problem jp = probs[pi];
        GemvProblem p;
        p.qw = reinterpret_cast<const uint8_t *>(jp.qweight);
        p.scales = reinterpret_cast<const __half *>(jp.scales);
        p.codebook = reinterpret_cast<const __half *>(jp.codebook);
        p.x = jp.x; p.bias = jp.bias; p.y = jp.y;
        p.N = jp.N; p.K = jp.K; p.g = jp.g; p.had = jp.had_block;
        finish_problem(p);
        if (jp.ldy > 0) p.ldy = jp.ldy;
        p.npeer = peers.n;
#pragma unroll
        for (int i = 0; i < 8; ++i) p.peer_delta[i] = peers.delta[i];
        const int base = rg_start[pi];
        const int lim = min(rg_end, rg_start[pi + 1]);
        bool tiled = false;
        if constexpr (Tile<FMT, B>::kMma) tiled = B * xs_stride<FMT, B>(p.K) > xcap && mma_ok<FMT>(p);
        if (!tiled) {
            stage_activation<B>(p, x_dtype, L.xs, L.sred, L.sexp, Tile<FMT, B>::kMma && mma_ok<FMT>(p));
            run_rows<FMT, B, DEPTH>(p, rg - base, lim - base, L.xs, L.sexp, L.ring, y_dtype);
        } else if constexpr (Tile<FMT, B>::kMma) {
            rows_k_tiled<FMT, B, DEPTH>(p, rg - base, lim - base, L, xcap, x_dtype, y_dtype);
        }
        rg = lim;
        __syncthreads();  // all warps done with xs before the next problem restages it
    }
}

template <int FMT, int B, int DEPTH>
static size_t gemv_smem_bytes(int K) {
    return (size_t)ring_bytes<FMT, B, DEPTH>() + (size_t)B * xs_stride<FMT, B>(K) * 2 + kSmallBytes;
}

}  // namespace jq

using namespace jq;

static int validate_problem(int fmt, const void *qw, const void *scales, const void *codebook, const void *x,
                            const void *y, int N, int K, int g, int had) {
    if (!qw || !x || !y) return JQ_ERR_NULL_PTR;
    if (fmt == JQ_FMT_GF4 && !codebook) return JQ_ERR_NULL_PTR;
    if (N <= 0 || K <= 0) return JQ_ERR_BAD_SHAPE;
    if (fmt == JQ_FMT_E2M1 && g == 0) return JQ_ERR_BAD_SHAPE;
    if (g < 0 || (g && (g % 32 || K % g))) return JQ_ERR_BAD_SHAPE;
    if (g && !scales) return JQ_ERR_NULL_PTR;
    if (had != 0 && had != 128) return JQ_ERR_UNSUPPORTED;
    if (had && K % had) return JQ_ERR_BAD_SHAPE;
    if (!jq_aligned16(qw)) return JQ_ERR_BAD_ALIGN;
    // codebook rows (32 bytes) are fetched with 16-byte copies; a base that is not 16-byte aligned would fault
    if (codebook && !jq_aligned16(codebook)) return JQ_ERR_BAD_ALIGN;
    if (scales && (reinterpret_cast<uintptr_t>(scales) & 1u)) return JQ_ERR_BAD_ALIGN;
    return JQ_OK;
}

static bool dtype_ok(int d) { return d == JQ_F32 || d == JQ_F16 || d == JQ_BF16; }

static const size_t kMaxSmem = 227 * 1024 - 64;  // dynamic part: the grouped kernel also has a few static bytes

template <int FMT, int B, int DEPTH>
static int launch_gemv_d(const GemvProblem &p, int x_dtype, int y_dtype, cudaStream_t st) {
    const size_t smem = gemv_smem_bytes<FMT, B, DEPTH>(p.K);
    if (smem > kMaxSmem) return JQ_ERR_UNSUPPORTED;
    auto kern = gemv_kernel<FMT, B, DEPTH>;
    JQ_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int row_groups = (p.N + Tile<FMT, B>::R - 1) / Tile<FMT, B>::R;
    int grid = jq_sm_count();  // one persistent CTA per SM; a small matrix still spreads over all of them
    if (grid > row_groups) grid = row_groups;
    kern<<<grid, kThreads, smem, st>>>(p, x_dtype, y_dtype);
    return jq_launch_status();
}

// deepest prefetch ring that fits beside the staged activation
template <int FMT, int B>
static int launch_gemv(const GemvProblem &p, int x_dtype, int y_dtype, cudaStream_t st) {
    if (gemv_smem_bytes<FMT, B, 4>(p.K) <= kMaxSmem) return launch_gemv_d<FMT, B, 4>(p, x_dtype, y_dtype, st);
    if constexpr (Tile<FMT, B>::kMma)
        if (gemv_smem_bytes<FMT, B, 3>(p.K) <= kMaxSmem) return launch_gemv_d<FMT, B, 3>(p, x_dtype, y_dtype, st);
    return launch_gemv_d<FMT, B, 2>(p, x_dtype, y_dtype, st);
}

template <int FMT, int B>
static bool gemv_fits(int K) { return gemv_smem_bytes<FMT, B, 2>(K) <= kMaxSmem; }

template <int FMT>
static bool gemv_fits_b(int B, int K) {
    switch (B) {
        case 1: return gemv_fits<FMT, 1>(K); case 2: return gemv_fits<FMT, 2>(K); case 3: return gemv_fits<FMT, 3>(K);
        case 4: return gemv_fits<FMT, 4>(K); case 5: return gemv_fits<FMT, 5>(K); case 6: return gemv_fits<FMT, 6>(K);
        case 7: return gemv_fits<FMT, 7>(K); case 8: return gemv_fits<FMT, 8>(K); default: return false;
    }
}

template <int FMT>
static int dispatch_gemv_one(const GemvProblem &p, int B, int x_dtype, int y_dtype, cudaStream_t st);

namespace jq {
// y[b][n] = sum_t part[t][b][n] + bias[n], cast to the output type.
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float *__restrict__ part, int nt, int B, int N,
                                                            const float *__restrict__ bias, void *__restrict__ y,
                                                            int y_dtype) {
    const long long total = (long long)B * N;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        float acc = 0.f;
        for (int t = 0; t < nt; ++t) acc += part[(size_t)t * total + i];
        if (bias) acc += bias[i % N];
        store_out(y, (size_t)i, acc, y_dtype);
    }
}
}  // namespace jq

// K-tile (codes) used when a batch's staged activation does not fit in shared
// memory: the largest multiple of 1024 codes that fits, 0 if even that fails.
template <int FMT>
static int splitk_tile(int B, int K, int g) {
    int tile = 0;
    for (int t = 1024; t < K; t += 1024) {
        if (!gemv_fits_b<FMT>(B, t)) break;
        if (g == 0 || t % g == 0) tile = t;
    }
    return tile;
}

// A batch whose staged activation does not fit in shared memory runs as
// split-K: one launch per K-tile writes fp32 partial outputs into the caller's
// workspace ([tiles][B][N] floats) and a small kernel sums them.  Without a
// workspace it falls back to several launches over sub-batches (which re-reads
// the weights once per sub-batch).
template <int FMT>
static int dispatch_gemv(const GemvProblem &p, int B, int x_dtype, int y_dtype, void *ws, size_t ws_bytes,
                         cudaStream_t st) {
    if (B > 8) return JQ_ERR_UNSUPPORTED;
    if (gemv_fits_b<FMT>(B, p.K)) return dispatch_gemv_one<FMT>(p, B, x_dtype, y_dtype, st);
    const size_t xe = x_dtype == JQ_F32 ? 4 : 2, ye = y_dtype == JQ_F32 ? 4 : 2;
    const int tile = splitk_tile<FMT>(B, p.K, p.g);
    if (tile > 0 && ws) {
        const int nt = (p.K + tile - 1) / tile;
        const size_t need = (size_t)nt * B * p.N * sizeof(float);
        if (ws_bytes < need) return JQ_ERR_WORKSPACE;
        if (reinterpret_cast<uintptr_t>(ws) & 15u) return JQ_ERR_BAD_ALIGN;
        for (int t = 0; t < nt; ++t) {
            const int k0 = t * tile;
            GemvProblem q = p;
            q.K = p.K - k0 < tile ? p.K - k0 : tile;
            q.qw = p.qw + (k0 >> 1);
            q.scales = p.g ? p.scales + k0 / p.g : nullptr;
            q.x = reinterpret_cast<const char *>(p.x) + (size_t)k0 * xe;
            q.bias = nullptr;
            q.y = reinterpret_cast<float *>(ws) + (size_t)t * B * p.N;
            int st_ = dispatch_gemv_one<FMT>(q, B, x_dtype, JQ_F32, st);
            if (st_) return st_;
        }
        const long long total = (long long)B * p.N;
        int blocks = (int)((total + 255) / 256);
        if (blocks > jq_sm_count() * 8) blocks = jq_sm_count() * 8;
        splitk_reduce_kernel<<<blocks, 256, 0, st>>>(reinterpret_cast<const float *>(ws), nt, B, p.N, p.bias, p.y, y_dtype);
        return jq_launch_status();
    }
    int bc = B;
    while (bc > 1 && !gemv_fits_b<FMT>(bc, p.K)) --bc;
    if (!gemv_fits_b<FMT>(bc, p.K)) return JQ_ERR_UNSUPPORTED;
    for (int b0 = 0; b0 < B; b0 += bc) {
        GemvProblem q = p;
        const int nb = B - b0 < bc ? B - b0 : bc;
        q.x = reinterpret_cast<const char *>(p.x) + (size_t)b0 * p.ldx * xe;
        q.x_full = reinterpret_cast<const char *>(p.x_full) + (size_t)b0 * p.ldx * xe;
        q.y = reinterpret_cast<char *>(p.y) + (size_t)b0 * p.N * ye;
        int st_ = dispatch_gemv_one<FMT>(q, nb, x_dtype, y_dtype, st);
        if (st_) return st_;
    }
    return JQ_OK;
}

extern "C" size_t jq_workspace_bytes(int op, int N, int K, int B) {
    if (op != JQ_OP_GEMV || N <= 0 || K <= 0 || B <= 0 || B > 8) return 0;
    if (gemv_fits_b<JQ_FMT_E2M1>(B, K) && gemv_fits_b<JQ_FMT_GF4>(B, K)) return 0;
    int tile = splitk_tile<JQ_FMT_E2M1>(B, K, 0);
    const int tile2 = splitk_tile<JQ_FMT_GF4>(B, K, 0);
    if (tile2 < tile) tile = tile2;
    if (tile <= 0) return 0;
    // (a group size that does not divide the tile shrinks it; such calls answer
    // JQ_ERR_WORKSPACE and the caller may retry without a workspace)
    const int nt = (K + tile - 1) / tile;
    return (size_t)nt * B * N * sizeof(float);
}

template <int FMT>
static int dispatch_gemv_one(const GemvProblem &p, int B, int x_dtype, int y_dtype, cudaStream_t st) {
    switch (B) {
        case 1: return launch_gemv<FMT, 1>(p, x_dtype, y_dtype, st);
        case 2: return launch_gemv<FMT, 2>(p, x_dtype, y_dtype, st);
        case 3: return launch_gemv<FMT, 3>(p, x_dtype, y_dtype, st);
        case 4: return launch_gemv<FMT, 4>(p, x_dtype, y_dtype, st);
        case 5: return launch_gemv<FMT, 5>(p, x_dtype, y_dtype, st);
        case 6: return launch_gemv<FMT, 6>(p, x_dtype, y_dtype, st);
        case 7: return launch_gemv<FMT, 7>(p, x_dtype, y_dtype, st);
        case 8: return launch_gemv<FMT, 8>(p, x_dtype, y_dtype, st);
        default: return JQ_ERR_UNSUPPORTED;
    }
}

extern "C" int jq_gemv_e2m1(const void *qweight, const void *scales, const void *x, const float *bias, void *y,
                            int N, int K, int B, int g, int had_block, int x_dtype, int y_dtype, void *workspace,
                            size_t workspace_bytes, jq_stream_t stream) {
    int st = validate_problem(JQ_FMT_E2M1, qweight, scales, nullptr, x, y, N, K, g, had_block);
    if (st) return st;
    if (B < 1) return JQ_ERR_BAD_SHAPE;
    if (!dtype_ok(x_dtype) || !dtype_ok(y_dtype)) return JQ_ERR_BAD_DTYPE;
    GemvProblem p{reinterpret_cast<const uint8_t *>(qweight), reinterpret_cast<const __half *>(scales), nullptr, x,
                  bias, y, N, K, g, had_block};
    finish_problem(p);
    return dispatch_gemv<JQ_FMT_E2M1>(p, B, x_dtype, y_dtype, workspace, workspace_bytes,
                                      reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int jq_gemv_gf4(const void *qweight, const void *scales, const void *codebook, const void *x,
                           const float *bias, void *y, int N, int K, int B, int g, int had_block, int x_dtype,
                           int y_dtype, void *workspace, size_t workspace_bytes, jq_stream_t stream) {
    int st = validate_problem(JQ_FMT_GF4, qweight, scales, codebook, x, y, N, K, g, had_block);
    if (st) return st;
    if (B < 1) return JQ_ERR_BAD_SHAPE;
    if (!dtype_ok(x_dtype) || !dtype_ok(y_dtype)) return JQ_ERR_BAD_DTYPE;
    GemvProblem p{reinterpret_cast<const uint8_t *>(qweight), reinterpret_cast<const __half *>(scales),
                  reinterpret_cast<const __half *>(codebook), x, bias, y, N, K, g, had_block};
    finish_problem(p);
    return dispatch_gemv<JQ_FMT_GF4>(p, B, x_dtype, y_dtype, workspace, workspace_bytes,
                                     reinterpret_cast<cudaStream_t>(stream));
}

// ---- grouped launch ---------------------------------------------------------
// plan layout (ints): [magic, n, grid, maxK, R, B, fmt, maxK_whole] rg_start[n+1] cta_first[grid+1]
// (maxK_whole: the largest K among problems whose activation must be staged whole, i.e. that the K-tiled
// MMA row loop cannot take)
static const int kPlanMagic = 0x4a51504c;
static const int kPlanHeader = 8;

extern "C" size_t jq_grouped_plan_bytes(int n) {
    if (n < 0) return 0;
    return ((size_t)kPlanHeader + (size_t)(n + 1) + (size_t)jq_sm_count() + 1) * sizeof(int);
}

template <int FMT>
static int tile_rows_f(int B) {
    switch (B) {
        case 1: return Tile<FMT, 1>::R; case 2: return Tile<FMT, 2>::R; case 3: return Tile<FMT, 3>::R;
        case 4: return Tile<FMT, 4>::R; case 5: return Tile<FMT, 5>::R; case 6: return Tile<FMT, 6>::R;
        case 7: return Tile<FMT, 7>::R; case 8: return Tile<FMT, 8>::R; default: return 0;
    }
}

static int tile_rows(int fmt, int B) {
    return fmt == JQ_FMT_GF4 ? tile_rows_f<JQ_FMT_GF4>(B) : tile_rows_f<JQ_FMT_E2M1>(B);
}

extern "C" int jq_grouped_plan(int fmt, const jq_problem *ph, int n, int B, void *plan_host, size_t plan_bytes) {
    if (!ph || !plan_host) return JQ_ERR_NULL_PTR;
    if (n <= 0) return JQ_ERR_BAD_SHAPE;
    if (fmt != JQ_FMT_E2M1 && fmt != JQ_FMT_GF4) return JQ_ERR_UNSUPPORTED;
    const int R = tile_rows(fmt, B);
    if (!R) return JQ_ERR_UNSUPPORTED;
    if (plan_bytes < jq_grouped_plan_bytes(n)) return JQ_ERR_WORKSPACE;
    const int grid = jq_sm_count();  // one persistent CTA per SM
    int *h = reinterpret_cast<int *>(plan_host);
    int *rg_start = h + kPlanHeader, *cta_first = rg_start + n + 1;
    int maxK = 0, maxK_whole = 0;
    double total = 0;
    rg_start[0] = 0;
    const bool mma_fmt = B >= (fmt == JQ_FMT_GF4 ? kMmaMinBGf4 : kMmaMinB);
    for (int i = 0; i < n; ++i) {
        int st = validate_problem(fmt, ph[i].qweight, ph[i].scales, ph[i].codebook, ph[i].x, ph[i].y, ph[i].N,
                                  ph[i].K, ph[i].g, ph[i].had_block);
        if (st) return st;
        const long long groups = ((long long)ph[i].N + R - 1) / R;
        if (rg_start[i] + groups > 0x7fffffffLL) return JQ_ERR_BAD_SHAPE;
        rg_start[i + 1] = rg_start[i] + (int)groups;
        total += (double)groups * ph[i].K;
        maxK = ph[i].K > maxK ? ph[i].K : maxK;
        const bool tileable = mma_fmt && (fmt == JQ_FMT_E2M1
                                              ? mma_ok_raw<JQ_FMT_E2M1>(ph[i].g, ph[i].K, ph[i].scales, ph[i].codebook)
                                              : mma_ok_raw<JQ_FMT_GF4>(ph[i].g, ph[i].K, ph[i].scales, ph[i].codebook));
        if (!tileable && ph[i].K > maxK_whole) maxK_whole = ph[i].K;
    }
    // contiguous CTA ranges of (nearly) equal packed bytes: cut every total/grid
    // units of row-groups * K while walking the problems in order
    const double per = total / grid;
    int cta = 0;
    double acc = 0;
    cta_first[0] = 0;
    for (int i = 0; i < n; ++i) {
        const int groups = rg_start[i + 1] - rg_start[i];
        const double w = (double)ph[i].K;
        int done = 0;
        while (done < groups) {
            if (cta + 1 >= grid) { done = groups; break; }
            const double room = per * (cta + 1) - acc;
            int take = (int)(room / w + 0.5);
            if (take < 1) take = 1;
            if (take >= groups - done) {  // the cut lies beyond this problem
                acc += (double)(groups - done) * w;
                done = groups;
                break;
            }
            done += take;
            acc += (double)take * w;
            ++cta;
            cta_first[cta] = rg_start[i] + done;
        }
    }
    for (int c = cta + 1; c <= grid; ++c) cta_first[c] = rg_start[n];
    h[0] = kPlanMagic; h[1] = n; h[2] = grid; h[3] = maxK; h[4] = R; h[5] = B; h[6] = fmt; h[7] = maxK_whole;
    return JQ_OK;
}

template <int FMT, int B, int DEPTH>
static int launch_grouped_d(const jq_problem *pd, const int *plan_host, const int *plan_dev, int x_dtype, int y_dtype,
                            const PeerInfo &peers, cudaStream_t st) {
    const int n = plan_host[1], grid = plan_host[2], maxK = plan_host[3];
    size_t smem = gemv_smem_bytes<FMT, B, DEPTH>(maxK);
    if (smem > kMaxSmem) {
        // K-tiled problems: all the shared memory there is; the kernel splits the activation region
        if (!Tile<FMT, B>::kMma || gemv_smem_bytes<FMT, B, DEPTH>(plan_host[7]) > kMaxSmem) return JQ_ERR_UNSUPPORTED;
        smem = kMaxSmem;
    }
    const int xcap = (int)((smem - ring_bytes<FMT, B, DEPTH>() - kSmallBytes) / 2);  // halves for the activation
    auto kern = gemv_grouped_kernel<FMT, B, DEPTH>;
    JQ_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<grid, kThreads, smem, st>>>(pd, n, plan_dev + kPlanHeader, plan_dev + kPlanHeader + n + 1, xcap, x_dtype, y_dtype, peers);
    return jq_launch_status();
}

constexpr int kTiledDepth = 2;   // stages of the ring in a K-tiled launch: larger K tiles beat a deeper ring (decode70b, batch 8: 1142 vs 888 tok/s)
template <int FMT, int B>
static int launch_grouped(const jq_problem *pd, const int *plan_host, const int *plan_dev, int x_dtype, int y_dtype,
                          const PeerInfo &peers, cudaStream_t st) {
    if (gemv_smem_bytes<FMT, B, 4>(plan_host[3]) <= kMaxSmem)
        return launch_grouped_d<FMT, B, 4>(pd, plan_host, plan_dev, x_dtype, y_dtype, peers, st);
    if constexpr (Tile<FMT, B>::kMma) {
        if (gemv_smem_bytes<FMT, B, 3>(plan_host[3]) <= kMaxSmem)
            return launch_grouped_d<FMT, B, 3>(pd, plan_host, plan_dev, x_dtype, y_dtype, peers, st);
        // the largest K does not fit even with two stages: K-tiled MMA row loop, if a K tile of
        // at least 1024 codes and one row group of partial sums fit and every problem that cannot be tiled fits
        // whole.  (Where two stages untiled fit they are faster than three stages tiled: 3.6 vs 3.1 TB/s at
        // 16 x 8192 x 8192, batch 8.)
        if (gemv_smem_bytes<FMT, B, 2>(plan_host[3]) > kMaxSmem) {
            constexpr int TD = kTiledDepth;
            const long long xcap = ((long long)kMaxSmem - ring_bytes<FMT, B, TD>() - kSmallBytes) / 2;
            const long long tileK = ((xcap / 2) / B - kXPad) / 1024 * 1024;
            if (tileK >= 1024 && (xcap - B * (tileK + kXPad) - 8) / 2 / (16 * B) >= 1 &&
                gemv_smem_bytes<FMT, B, TD>(plan_host[7]) <= kMaxSmem)
                return launch_grouped_d<FMT, B, TD>(pd, plan_host, plan_dev, x_dtype, y_dtype, peers, st);
        }
    }
    return launch_grouped_d<FMT, B, 2>(pd, plan_host, plan_dev, x_dtype, y_dtype, peers, st);
}

template <int FMT>
static int dispatch_grouped(int B, const jq_problem *pd, const int *ph, const int *pdv, int xd, int yd,
                            const PeerInfo &peers, cudaStream_t st) {
    switch (B) {
        case 1: return launch_grouped<FMT, 1>(pd, ph, pdv, xd, yd, peers, st);
        case 2: return launch_grouped<FMT, 2>(pd, ph, pdv, xd, yd, peers, st);
        case 3: return launch_grouped<FMT, 3>(pd, ph, pdv, xd, yd, peers, st);
        case 4: return launch_grouped<FMT, 4>(pd, ph, pdv, xd, yd, peers, st);
        case 5: return launch_grouped<FMT, 5>(pd, ph, pdv, xd, yd, peers, st);
        case 6: return launch_grouped<FMT, 6>(pd, ph, pdv, xd, yd, peers, st);
        case 7: return launch_grouped<FMT, 7>(pd, ph, pdv, xd, yd, peers, st);
        case 8: return launch_grouped<FMT, 8>(pd, ph, pdv, xd, yd, peers, st);
        default: return JQ_ERR_UNSUPPORTED;
    }
}

extern "C" int jq_gemv_grouped_peers(const jq_problem *problems_dev, const void *plan_host, const void *plan_dev,
                                     int x_dtype, int y_dtype, int npeer, const int64_t *peer_delta,
                                     jq_stream_t stream);

extern "C" int jq_gemv_grouped(const jq_problem *problems_dev, const void *plan_host, const void *plan_dev,
                               int x_dtype, int y_dtype, jq_stream_t stream) {
    const int64_t zero = 0;
    return jq_gemv_grouped_peers(problems_dev, plan_host, plan_dev, x_dtype, y_dtype, 1, &zero, stream);
}

extern "C" int jq_gemv_grouped_peers(const jq_problem *problems_dev, const void *plan_host, const void *plan_dev,
                                     int x_dtype, int y_dtype, int npeer, const int64_t *peer_delta,
                                     jq_stream_t stream) {
    if (!problems_dev || !plan_host || !plan_dev || !peer_delta) return JQ_ERR_NULL_PTR;
    if (npeer < 1 || npeer > 8) return JQ_ERR_BAD_SHAPE;
    PeerInfo peers;
    peers.n = npeer;
    for (int i = 0; i < 8; ++i) peers.delta[i] = i < npeer ? (long long)peer_delta[i] : 0;
    const int *ph = reinterpret_cast<const int *>(plan_host);
    if (ph[0] != kPlanMagic) return JQ_ERR_BAD_SHAPE;
    if (!dtype_ok(x_dtype) || !dtype_ok(y_dtype)) return JQ_ERR_BAD_DTYPE;
    const int B = ph[5], fmt = ph[6];
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const int *pdv = reinterpret_cast<const int *>(plan_dev);
    if (fmt == JQ_FMT_E2M1) return dispatch_grouped<JQ_FMT_E2M1>(B, problems_dev, ph, pdv, x_dtype, y_dtype, peers, st);
    return dispatch_grouped<JQ_FMT_GF4>(B, problems_dev, ph, pdv, x_dtype, y_dtype, peers, st);
}

// ---- allocation-free entry point ---------------------------------------------
// Split-K partial outputs for callers that can neither allocate device memory
// nor lend a workspace (allocator hooks, fixed-footprint real-time loops): the
// scratch is this file-scope device array.  In host code the symbol is only a
// stand-in for the device object, so its device address is fetched once per
// device with cudaGetSymbolAddress and that pointer is what the kernels get.
static __device__ __align__(256) unsigned char jq_noalloc_scratch[JQ_NOALLOC_SCRATCH_BYTES];

#include <mutex>
static int noalloc_scratch_address(void **out) {
    static void *addr[64];
    static bool known[64];
    static std::mutex mu;
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return JQ_ERR_CUDA_BASE - (int)e;
    if (dev < 0 || dev >= 64) return JQ_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lk(mu);
    if (!known[dev]) {
        void *p = nullptr;
        e = cudaGetSymbolAddress(&p, jq_noalloc_scratch);  // the current device's copy of the array
        if (e != cudaSuccess) return JQ_ERR_CUDA_BASE - (int)e;
        if (!p) return JQ_ERR_NULL_PTR;
        addr[dev] = p;
        known[dev] = true;
    }
    *out = addr[dev];
    return JQ_OK;
}

template <int FMT>
static int gemv_noalloc(const GemvProblem &p, int B, int x_dtype, int y_dtype, cudaStream_t st) {
    if (B > 8) return JQ_ERR_UNSUPPORTED;
    if (gemv_fits_b<FMT>(B, p.K)) return dispatch_gemv<FMT>(p, B, x_dtype, y_dtype, nullptr, 0, st);  // no scratch needed
    const int tile = splitk_tile<FMT>(B, p.K, p.g);
    if (tile <= 0) return JQ_ERR_UNSUPPORTED;
    const size_t nt = (size_t)((p.K + tile - 1) / tile);
    if (nt * (size_t)B * (size_t)p.N * sizeof(float) > (size_t)JQ_NOALLOC_SCRATCH_BYTES) return JQ_ERR_SCRATCH_LIMIT;
    void *scratch = nullptr;
    int s = noalloc_scratch_address(&scratch);
    if (s) return s;
    return dispatch_gemv<FMT>(p, B, x_dtype, y_dtype, scratch, JQ_NOALLOC_SCRATCH_BYTES, st);
}

extern "C" int jq_gemv_noalloc(int fmt, const void *qweight, const void *scales, const void *codebook, const void *x,
                               const float *bias, void *y, int N, int K, int B, int g, int had_block, int x_dtype,
                               int y_dtype, jq_stream_t stream) {
    if (fmt != JQ_FMT_E2M1 && fmt != JQ_FMT_GF4) return JQ_ERR_UNSUPPORTED;
    int st = validate_problem(fmt, qweight, scales, fmt == JQ_FMT_GF4 ? codebook : nullptr, x, y, N, K, g, had_block);
    if (st) return st;
    if (B < 1) return JQ_ERR_BAD_SHAPE;
    if (!dtype_ok(x_dtype) || !dtype_ok(y_dtype)) return JQ_ERR_BAD_DTYPE;
    GemvProblem p{reinterpret_cast<const uint8_t *>(qweight), reinterpret_cast<const __half *>(scales),
                  fmt == JQ_FMT_GF4 ? reinterpret_cast<const __half *>(codebook) : nullptr, x, bias, y, N, K, g,
                  had_block};
    finish_problem(p);
    cudaStream_t cs = reinterpret_cast<cudaStream_t>(stream);
    return fmt == JQ_FMT_GF4 ? gemv_noalloc<JQ_FMT_GF4>(p, B, x_dtype, y_dtype, cs)
                             : gemv_noalloc<JQ_FMT_E2M1>(p, B, x_dtype, y_dtype, cs);
}
