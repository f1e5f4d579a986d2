// Fused 4-bit dequantise + GEMV for B200 (sm_100a), batch 1..8, CUDA cores.
//
// Data path: packed weight rows stream from HBM with 128-bit no-allocate
// loads (each byte is read exactly once); the activation is rotated (block
// Hadamard), normalised by a power of two and rounded to fp16 once per CTA
// into shared memory; E2M1 nibbles are converted two at a time by the sm_100a
// cvt.rn.f16x2.e2m1x2 instruction, GF4 nibbles index a per-row 16-entry fp16
// table in shared memory; products fp16 x fp16 are exact in fp32 and are
// accumulated with the mixed-precision fma.rn.f32.f16; group scales are
// applied in fp32 per 32-code chunk; rows are reduced with warp shuffles.
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
};

constexpr int kThreads = 512;
constexpr int kWarps = kThreads / 32;

template <int B>
struct Tile {
    // rows a warp carries at once; bounded by registers
    static constexpr int R = (B <= 2) ? 4 : (B <= 4 ? 2 : 1);
};

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
template <int B>
__device__ void stage_activation(const GemvProblem &p, int x_dtype, __half *xs, float *sred, int *sexp) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int K = p.K, XS = xs_halves(K);
    for (int b = 0; b < B; ++b) {
        float m = 0.f;
        for (int k = tid; k < K; k += kThreads) m = fmaxf(m, fabsf(load_act(p.x, (size_t)b * K + k, x_dtype)));
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
        __half *xb = xs + (size_t)b * XS;
        if (p.had) {
            for (int blk = warp; blk * 128 < K; blk += kWarps) {
                float v[4];
                const int k0 = blk * 128 + lane * 4;
#pragma unroll
                for (int j = 0; j < 4; ++j) v[j] = load_act(p.x, (size_t)b * K + k0 + j, x_dtype) * down;
                fwht128_warp(v, lane);
                __half2 h01 = __floats2half2_rn(v[0], v[1]), h23 = __floats2half2_rn(v[2], v[3]);
                uint2 pk = make_uint2(*reinterpret_cast<uint32_t *>(&h01), *reinterpret_cast<uint32_t *>(&h23));
                *reinterpret_cast<uint2 *>(xb + xs_pos(k0)) = pk;
            }
        } else {
            for (int k = tid; k < K; k += kThreads)
                xb[xs_pos(k)] = __float2half_rn(load_act(p.x, (size_t)b * K + k, x_dtype) * down);
        }
        for (int k = K + tid; k < XS; k += kThreads) xb[xs_pos(k)] = __float2half_rn(0.f);
    }
    __syncthreads();
}

// One warp, R rows starting at row0, full K.  tab: R*16 halves of per-warp
// shared memory (GF4 tables).
template <int FMT, int B, int R>
__device__ __forceinline__ void warp_rows(const GemvProblem &p, int row0, const __half *xs, const int *sexp,
                                          __half *tab, int y_dtype) {
    const int lane = threadIdx.x & 31;
    const int K = p.K, N = p.N, XS = xs_halves(K);
    const int stride_b = jq_row_stride_codes(K) >> 1;  // bytes per packed row
    const int nchunks = jq_row_stride_codes(K) >> 5;
    const int ngroups = p.g ? K / p.g : 0;
    float acc[R][B];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int b = 0; b < B; ++b) acc[r][b] = 0.f;

    int rows[R];
#pragma unroll
    for (int r = 0; r < R; ++r) rows[r] = min(row0 + r, N - 1);

    if (FMT == JQ_FMT_GF4) {
        __syncwarp();
        if (lane < R * 8) {
            const int r = lane >> 3;
            reinterpret_cast<uint32_t *>(tab)[lane] =
                reinterpret_cast<const uint32_t *>(p.codebook + (size_t)rows[r] * 16)[lane & 7];
        }
        __syncwarp();
    }

    for (int c = lane; c < nchunks; c += 32) {
        uint4 w[R];
        float sc[R];
#pragma unroll
        for (int r = 0; r < R; ++r) w[r] = ldg_stream_u4(p.qw + (size_t)rows[r] * stride_b + (size_t)c * 16);
#pragma unroll
        for (int r = 0; r < R; ++r) {
            if (p.g) {
                int gi = min((c * 32) / p.g, ngroups - 1);
                sc[r] = __half2float(p.scales[(size_t)rows[r] * ngroups + gi]);
            } else {
                sc[r] = 1.f;
            }
        }
        const int i = c >> 5;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            uint4 xv[B];
#pragma unroll
            for (int b = 0; b < B; ++b)
                xv[b] = *reinterpret_cast<const uint4 *>(xs + (size_t)b * XS + (((i * 4 + q) * 32 + lane) << 3));
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const uint32_t word = q == 0 ? w[r].x : (q == 1 ? w[r].y : (q == 2 ? w[r].z : w[r].w));
                float part[B];
#pragma unroll
                for (int b = 0; b < B; ++b) part[b] = 0.f;
#pragma unroll
                for (int bb = 0; bb < 4; ++bb) {
                    uint16_t w0, w1;
                    if (FMT == JQ_FMT_E2M1) {
                        uint32_t h2 = e2m1x2_to_h2((word >> (8 * bb)) & 0xffu);
                        w0 = h2_lo(h2);
                        w1 = h2_hi(h2);
                    } else {
                        const uint16_t *t = reinterpret_cast<const uint16_t *>(tab) + r * 16;
                        w0 = t[(word >> (8 * bb)) & 0xfu];
                        w1 = t[(word >> (8 * bb + 4)) & 0xfu];
                    }
#pragma unroll
                    for (int b = 0; b < B; ++b) {
                        const uint32_t xx = bb == 0 ? xv[b].x : (bb == 1 ? xv[b].y : (bb == 2 ? xv[b].z : xv[b].w));
                        fma_h(part[b], w0, h2_lo(xx));
                        fma_h(part[b], w1, h2_hi(xx));
                    }
                }
#pragma unroll
                for (int b = 0; b < B; ++b) acc[r][b] = fmaf(part[b], sc[r], acc[r][b]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int b = 0; b < B; ++b) acc[r][b] = warp_sum(acc[r][b]);
    if (lane == 0) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            if (row0 + r < N) {
                const float bias = p.bias ? p.bias[row0 + r] : 0.f;
#pragma unroll
                for (int b = 0; b < B; ++b) {
                    const float up = __uint_as_float((uint32_t)(127 + sexp[b]) << 23);  // 2^e
                    store_out(p.y, (size_t)b * N + row0 + r, fmaf(acc[r][b], up, bias), y_dtype);
                }
            }
        }
    }
}

template <int FMT, int B>
__global__ void __launch_bounds__(kThreads) gemv_kernel(GemvProblem p, int x_dtype, int y_dtype) {
    extern __shared__ __align__(16) unsigned char smem[];
    constexpr int R = Tile<B>::R;
    const int XS = xs_halves(p.K);
    __half *xs = reinterpret_cast<__half *>(smem);
    __half *tabs = xs + (size_t)B * XS;                     // kWarps * R * 16 halves
    float *sred = reinterpret_cast<float *>(tabs + kWarps * R * 16);
    int *sexp = reinterpret_cast<int *>(sred + kWarps);

    stage_activation<B>(p, x_dtype, xs, sred, sexp);

    const int warp = threadIdx.x >> 5;
    const int total_warps = gridDim.x * kWarps;
    const int ngroups_rows = (p.N + R - 1) / R;
    for (int rg = blockIdx.x * kWarps + warp; rg < ngroups_rows; rg += total_warps)
        warp_rows<FMT, B, R>(p, rg * R, xs, sexp, tabs + warp * R * 16, y_dtype);
}

// Grouped launch: the concatenated row space of all problems is split into
// contiguous, byte-balanced CTA ranges on the host (cta_first[]: first global
// row-group of each CTA, in units of R rows); a CTA re-stages the activation
// whenever it crosses into the next problem.
template <int FMT, int B>
__global__ void __launch_bounds__(kThreads) gemv_grouped_kernel(const jq_problem *probs, int nprob,
                                                                  const int *rg_start, const int *cta_first,
                                                                  int x_dtype, int y_dtype) {
    extern __shared__ __align__(16) unsigned char smem[];
    constexpr int R = Tile<B>::R;
    __shared__ int s_prob;
    const int warp = threadIdx.x >> 5;
    int rg = cta_first[blockIdx.x];
    const int rg_end = cta_first[blockIdx.x + 1];
    int pi = 0;
    while (rg < rg_end) {
        if (threadIdx.x == 0) {
            int q = pi;
            while (q + 1 < nprob && rg_start[q + 1] <= rg) ++q;
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
        const int XS = xs_halves(p.K);
        __half *xs = reinterpret_cast<__half *>(smem);
        __half *tabs = xs + (size_t)B * XS;
        float *sred = reinterpret_cast<float *>(tabs + kWarps * R * 16);
        int *sexp = reinterpret_cast<int *>(sred + kWarps);
        stage_activation<B>(p, x_dtype, xs, sred, sexp);
        const int base = rg_start[pi];
        const int lim = min(rg_end, rg_start[pi + 1]);
        for (int t = rg + warp; t < lim; t += kWarps)
            warp_rows<FMT, B, R>(p, (t - base) * R, xs, sexp, tabs + warp * R * 16, y_dtype);
        rg = lim;
        __syncthreads();  // all warps done with xs before the next problem restages it
    }
}

template <int B>
static size_t gemv_smem_bytes(int K) {
    return (size_t)B * xs_halves(K) * 2 + (size_t)kWarps * Tile<B>::R * 16 * 2 + kWarps * 4 + 8 * 4;
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
    if (codebook && (reinterpret_cast<uintptr_t>(codebook) & 3u)) return JQ_ERR_BAD_ALIGN;
    if (scales && (reinterpret_cast<uintptr_t>(scales) & 1u)) return JQ_ERR_BAD_ALIGN;
    return JQ_OK;
}

static bool dtype_ok(int d) { return d == JQ_F32 || d == JQ_F16 || d == JQ_BF16; }

static const size_t kMaxSmem = 227 * 1024;

template <int FMT, int B>
static int launch_gemv(const GemvProblem &p, int x_dtype, int y_dtype, cudaStream_t st) {
    const size_t smem = gemv_smem_bytes<B>(p.K);
    if (smem > kMaxSmem) return JQ_ERR_UNSUPPORTED;
    auto kern = gemv_kernel<FMT, B>;
    JQ_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int sms = jq_sm_count();
    const int per_sm = smem * 2 + 2048 <= kMaxSmem ? 2 : 1;
    const int row_groups = (p.N + Tile<B>::R - 1) / Tile<B>::R;
    int grid = sms * per_sm;
    const int need = (row_groups + kWarps - 1) / kWarps;
    if (grid > need) grid = need;
    kern<<<grid, kThreads, smem, st>>>(p, x_dtype, y_dtype);
    return jq_launch_status();
}

template <int FMT>
static int dispatch_gemv(const GemvProblem &p, int B, int x_dtype, int y_dtype, cudaStream_t st) {
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
    (void)workspace; (void)workspace_bytes;
    int st = validate_problem(JQ_FMT_E2M1, qweight, scales, nullptr, x, y, N, K, g, had_block);
    if (st) return st;
    if (B < 1) return JQ_ERR_BAD_SHAPE;
    if (!dtype_ok(x_dtype) || !dtype_ok(y_dtype)) return JQ_ERR_BAD_DTYPE;
    GemvProblem p{reinterpret_cast<const uint8_t *>(qweight), reinterpret_cast<const __half *>(scales), nullptr, x,
                  bias, y, N, K, g, had_block};
    return dispatch_gemv<JQ_FMT_E2M1>(p, B, x_dtype, y_dtype, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int jq_gemv_gf4(const void *qweight, const void *scales, const void *codebook, const void *x,
                           const float *bias, void *y, int N, int K, int B, int g, int had_block, int x_dtype,
                           int y_dtype, void *workspace, size_t workspace_bytes, jq_stream_t stream) {
    (void)workspace; (void)workspace_bytes;
    int st = validate_problem(JQ_FMT_GF4, qweight, scales, codebook, x, y, N, K, g, had_block);
    if (st) return st;
    if (B < 1) return JQ_ERR_BAD_SHAPE;
    if (!dtype_ok(x_dtype) || !dtype_ok(y_dtype)) return JQ_ERR_BAD_DTYPE;
    GemvProblem p{reinterpret_cast<const uint8_t *>(qweight), reinterpret_cast<const __half *>(scales),
                  reinterpret_cast<const __half *>(codebook), x, bias, y, N, K, g, had_block};
    return dispatch_gemv<JQ_FMT_GF4>(p, B, x_dtype, y_dtype, reinterpret_cast<cudaStream_t>(stream));
}

// ---- grouped launch ---------------------------------------------------------
// plan layout (ints): [magic, n, grid, maxK, R, B, fmt, 0] rg_start[n+1] cta_first[grid+1]
static const int kPlanMagic = 0x4a51504c;
static const int kPlanHeader = 8;

extern "C" size_t jq_grouped_plan_bytes(int n) {
    if (n < 0) return 0;
    return ((size_t)kPlanHeader + (size_t)(n + 1) + (size_t)jq_sm_count() * 2 + 1) * sizeof(int);
}

template <int B>
static int plan_rows() { return Tile<B>::R; }

static int tile_rows(int B) {
    switch (B) {
        case 1: return plan_rows<1>(); case 2: return plan_rows<2>(); case 3: return plan_rows<3>();
        case 4: return plan_rows<4>(); case 5: return plan_rows<5>(); case 6: return plan_rows<6>();
        case 7: return plan_rows<7>(); case 8: return plan_rows<8>(); default: return 0;
    }
}

extern "C" int jq_grouped_plan(int fmt, const jq_problem *ph, int n, int B, void *plan_host, size_t plan_bytes) {
    if (!ph || !plan_host) return JQ_ERR_NULL_PTR;
    if (n <= 0) return JQ_ERR_BAD_SHAPE;
    if (fmt != JQ_FMT_E2M1 && fmt != JQ_FMT_GF4) return JQ_ERR_UNSUPPORTED;
    const int R = tile_rows(B);
    if (!R) return JQ_ERR_UNSUPPORTED;
    if (plan_bytes < jq_grouped_plan_bytes(n)) return JQ_ERR_WORKSPACE;
    const int grid = jq_sm_count() * 2;
    int *h = reinterpret_cast<int *>(plan_host);
    int *rg_start = h + kPlanHeader, *cta_first = rg_start + n + 1;
    int maxK = 0;
    double total = 0;
    rg_start[0] = 0;
    for (int i = 0; i < n; ++i) {
        int st = validate_problem(fmt, ph[i].qweight, ph[i].scales, ph[i].codebook, ph[i].x, ph[i].y, ph[i].N,
                                  ph[i].K, ph[i].g, ph[i].had_block);
        if (st) return st;
        const long long groups = ((long long)ph[i].N + R - 1) / R;
        if (rg_start[i] + groups > 0x7fffffffLL) return JQ_ERR_BAD_SHAPE;
        rg_start[i + 1] = rg_start[i] + (int)groups;
        total += (double)groups * ph[i].K;
        maxK = ph[i].K > maxK ? ph[i].K : maxK;
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
    h[0] = kPlanMagic; h[1] = n; h[2] = grid; h[3] = maxK; h[4] = R; h[5] = B; h[6] = fmt; h[7] = 0;
    return JQ_OK;
}

template <int FMT, int B>
static int launch_grouped(const jq_problem *pd, const int *plan_host, const int *plan_dev, int x_dtype, int y_dtype,
                          cudaStream_t st) {
    const int n = plan_host[1], grid = plan_host[2], maxK = plan_host[3];
    const size_t smem = gemv_smem_bytes<B>(maxK);
    if (smem * 2 + 2048 > kMaxSmem) return JQ_ERR_UNSUPPORTED;
    auto kern = gemv_grouped_kernel<FMT, B>;
    JQ_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<grid, kThreads, smem, st>>>(pd, n, plan_dev + kPlanHeader, plan_dev + kPlanHeader + n + 1, x_dtype, y_dtype);
    return jq_launch_status();
}

template <int FMT>
static int dispatch_grouped(int B, const jq_problem *pd, const int *ph, const int *pdv, int xd, int yd, cudaStream_t st) {
    switch (B) {
        case 1: return launch_grouped<FMT, 1>(pd, ph, pdv, xd, yd, st);
        case 2: return launch_grouped<FMT, 2>(pd, ph, pdv, xd, yd, st);
        case 3: return launch_grouped<FMT, 3>(pd, ph, pdv, xd, yd, st);
        case 4: return launch_grouped<FMT, 4>(pd, ph, pdv, xd, yd, st);
        case 5: return launch_grouped<FMT, 5>(pd, ph, pdv, xd, yd, st);
        case 6: return launch_grouped<FMT, 6>(pd, ph, pdv, xd, yd, st);
        case 7: return launch_grouped<FMT, 7>(pd, ph, pdv, xd, yd, st);
        case 8: return launch_grouped<FMT, 8>(pd, ph, pdv, xd, yd, st);
        default: return JQ_ERR_UNSUPPORTED;
    }
}

extern "C" int jq_gemv_grouped(const jq_problem *problems_dev, const void *plan_host, const void *plan_dev,
                               int x_dtype, int y_dtype, jq_stream_t stream) {
    if (!problems_dev || !plan_host || !plan_dev) return JQ_ERR_NULL_PTR;
    const int *ph = reinterpret_cast<const int *>(plan_host);
    if (ph[0] != kPlanMagic) return JQ_ERR_BAD_SHAPE;
    if (!dtype_ok(x_dtype) || !dtype_ok(y_dtype)) return JQ_ERR_BAD_DTYPE;
    const int B = ph[5], fmt = ph[6];
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const int *pdv = reinterpret_cast<const int *>(plan_dev);
    if (fmt == JQ_FMT_E2M1) return dispatch_grouped<JQ_FMT_E2M1>(B, problems_dev, ph, pdv, x_dtype, y_dtype, st);
    return dispatch_grouped<JQ_FMT_GF4>(B, problems_dev, ph, pdv, x_dtype, y_dtype, st);
}
