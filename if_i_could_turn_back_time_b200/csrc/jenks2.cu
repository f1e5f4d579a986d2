// Two-class Jenks natural break of an ascending-sorted array in O(n).
//
// The reference evaluates, for every candidate break i, the within-class sum
// of squared deviations var[i] = SSD(v[0..i)) + SSD(v[i..n)) with two serial
// loops per thread, O(n^2) in total
// (Python_Jenks_Test/Jenks_Tests/cuda_helpers.py:151-184; native twin
// CUDA_C_Code/include/layers.h:2423-2562), then takes the first argmin on the
// host (cuda_helpers.py:387).  With prefix sums S1[i] = sum v, S2[i] = sum v^2,
//     var[i] = (S2[i] - S1[i]^2 / i) + ((S2[n]-S2[i]) - (S1[n]-S1[i])^2 / (n-i))
// (first term 0 at i = 0), which is one pass.  Sums are float64: a three-phase
// scan (per-block scan, scan of block totals, per-element evaluation fused
// with a block-level first-argmin), then a single-block final argmin.
#include "common.cuh"

namespace jq2 {

constexpr int kBlock = 256;
constexpr int kPerThread = 8;
constexpr int kChunk = kBlock * kPerThread;  // elements per block

struct D2 { double a, b; };

__device__ __forceinline__ D2 warp_scan_incl(D2 v, int lane) {
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        double a = __shfl_up_sync(0xffffffffu, v.a, o), b = __shfl_up_sync(0xffffffffu, v.b, o);
        if (lane >= o) { v.a += a; v.b += b; }
    }
    return v;
}

// exclusive prefix (within the block) of this thread's chunk total; total of the block to `tot`
__device__ __forceinline__ D2 block_scan_excl(D2 mine, D2 *sm, D2 &tot) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    D2 inc = warp_scan_incl(mine, lane);
    if (lane == 31) sm[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        D2 w = lane < kBlock / 32 ? sm[lane] : D2{0.0, 0.0};
        D2 wi = warp_scan_incl(w, lane);
        if (lane < kBlock / 32) sm[lane] = D2{wi.a - w.a, wi.b - w.b};  // exclusive warp offsets
        if (lane == kBlock / 32 - 1) sm[kBlock / 32] = wi;              // block total
    }
    __syncthreads();
    tot = sm[kBlock / 32];
    D2 off = sm[warp];
    return D2{off.a + inc.a - mine.a, off.b + inc.b - mine.b};
}

// phase 1: block totals of (v, v^2)
__global__ void __launch_bounds__(kBlock) block_totals(const float *__restrict__ v, long long n, D2 *__restrict__ totals) {
    __shared__ D2 sm[kBlock / 32 + 1];
    const long long base = (long long)blockIdx.x * kChunk + (long long)threadIdx.x * kPerThread;
    D2 mine{0.0, 0.0};
#pragma unroll
    for (int j = 0; j < kPerThread; ++j)
        if (base + j < n) { const double x = (double)v[base + j]; mine.a += x; mine.b += x * x; }
    D2 tot;
    (void)block_scan_excl(mine, sm, tot);
    if (threadIdx.x == 0) totals[blockIdx.x] = tot;
}

// phase 2: exclusive scan of the block totals in place (single block); grand total to totals[nblocks]
__global__ void __launch_bounds__(kBlock) scan_totals(D2 *totals, int nblocks) {
    __shared__ D2 sm[kBlock / 32 + 1];
    D2 carry{0.0, 0.0};
    for (int base = 0; base < nblocks; base += kBlock) {
        const int i = base + threadIdx.x;
        D2 mine = i < nblocks ? totals[i] : D2{0.0, 0.0};
        D2 tot;
        D2 ex = block_scan_excl(mine, sm, tot);
        if (i < nblocks) totals[i] = D2{carry.a + ex.a, carry.b + ex.b};
        carry.a += tot.a; carry.b += tot.b;
        __syncthreads();
    }
    if (threadIdx.x == 0) totals[nblocks] = carry;
}

struct Best { double var; long long idx; };

__device__ __forceinline__ Best better(Best x, Best y) {  // smaller var, then smaller index
    return (y.var < x.var || (y.var == x.var && y.idx < x.idx)) ? y : x;
}

// phase 3: var[i] for every i and the block's first argmin
__global__ void __launch_bounds__(kBlock) eval_breaks(const float *__restrict__ v, long long n, const D2 *__restrict__ totals,
                                                      int nblocks, double *__restrict__ var_out, Best *__restrict__ block_best) {
    __shared__ D2 sm[kBlock / 32 + 1];
    __shared__ Best sb[kBlock / 32];
    const long long base = (long long)blockIdx.x * kChunk + (long long)threadIdx.x * kPerThread;
    double x[kPerThread];
    D2 mine{0.0, 0.0};
#pragma unroll
    for (int j = 0; j < kPerThread; ++j) {
        x[j] = base + j < n ? (double)v[base + j] : 0.0;
        mine.a += x[j]; mine.b += x[j] * x[j];
    }
    D2 tot;
    D2 ex = block_scan_excl(mine, sm, tot);
    const D2 boff = totals[blockIdx.x], all = totals[nblocks];
    double s1 = boff.a + ex.a, s2 = boff.b + ex.b;  // sums over v[0..i)
    Best best{1.7976931348623157e308, 0x7fffffffffffffffLL};
#pragma unroll
    for (int j = 0; j < kPerThread; ++j) {
        const long long i = base + j;
        if (i < n) {
            const double lo = i > 0 ? s2 - s1 * s1 / (double)i : 0.0;
            const double r1 = all.a - s1, r2 = all.b - s2;
            const double var = lo + (r2 - r1 * r1 / (double)(n - i));
            if (var_out) var_out[i] = var;
            best = better(best, Best{var, i});
        }
        s1 += x[j]; s2 += x[j] * x[j];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best y{__shfl_xor_sync(0xffffffffu, best.var, o), __shfl_xor_sync(0xffffffffu, best.idx, o)};
        best = better(best, y);
    }
    if ((threadIdx.x & 31) == 0) sb[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
        Best b = sb[0];
        for (int w = 1; w < kBlock / 32; ++w) b = better(b, sb[w]);
        block_best[blockIdx.x] = b;
    }
}

// phase 4: final argmin, goodness of variance fit; out[0] = break index, out[1] = min var, out[2] = GVF
__global__ void __launch_bounds__(kBlock) final_break(const Best *__restrict__ block_best, int nblocks, const D2 *__restrict__ totals,
                                                      long long n, double *__restrict__ out) {
    __shared__ Best sb[kBlock];
    Best b{1.7976931348623157e308, 0x7fffffffffffffffLL};
    for (int i = threadIdx.x; i < nblocks; i += kBlock) b = better(b, block_best[i]);
    sb[threadIdx.x] = b;
    __syncthreads();
    for (int s = kBlock / 2; s > 0; s >>= 1) {
        if (threadIdx.x < s) sb[threadIdx.x] = better(sb[threadIdx.x], sb[threadIdx.x + s]);
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        const D2 all = totals[nblocks];
        const double ssd_total = all.b - all.a * all.a / (double)n;  // sum (v - mean)^2
        out[0] = (double)sb[0].idx;
        out[1] = sb[0].var;
        out[2] = (ssd_total - sb[0].var) / (ssd_total + 1e-8);       // as cuda_helpers.py:393
    }
}

}  // namespace jq2

using namespace jq2;

static size_t jenks2_ws(long long n) {
    const long long nb = (n + kChunk - 1) / kChunk;
    return (size_t)(nb + 1) * sizeof(D2) + (size_t)nb * sizeof(Best) + 64;
}

extern "C" size_t jq_jenks2_workspace_bytes(long long n) { return n > 0 ? jenks2_ws(n) : 0; }

extern "C" int jq_jenks2_break(const float *sorted, long long n, double *var_or_null, double *out3, void *workspace,
                               size_t workspace_bytes, jq_stream_t stream) {
    if (!sorted || !out3 || !workspace) return JQ_ERR_NULL_PTR;
    if (n <= 0 || n > (1LL << 40)) return JQ_ERR_BAD_SHAPE;
    if (workspace_bytes < jenks2_ws(n)) return JQ_ERR_WORKSPACE;
    if (!jq_aligned16(workspace)) return JQ_ERR_BAD_ALIGN;
    const long long nb = (n + kChunk - 1) / kChunk;
    if (nb > 0x7fffffffLL) return JQ_ERR_BAD_SHAPE;
    D2 *totals = reinterpret_cast<D2 *>(workspace);
    Best *bests = reinterpret_cast<Best *>(totals + nb + 1);
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    block_totals<<<(int)nb, kBlock, 0, st>>>(sorted, n, totals);
    scan_totals<<<1, kBlock, 0, st>>>(totals, (int)nb);
    eval_breaks<<<(int)nb, kBlock, 0, st>>>(sorted, n, totals, (int)nb, var_or_null, bests);
    final_break<<<1, kBlock, 0, st>>>(bests, (int)nb, totals, n, out3);
    return jq_launch_status();
}
