// Device-side GF4 packer: per-row 16-class Jenks natural breaks on the GPU,
// bit-identical to the host packer (pack_host.cpp) and to the CPU oracle.
//
// One CTA per row at a time (persistent CTAs stride over the rows):
//   1. group scales (fp16_rn of the group absmax) and u = w / scale into shared memory;
//   2. bitonic sort of u in shared memory (padded with +inf to a power of two);
//   3. run-length compression to (distinct value, multiplicity);
//   4. float64 prefix sums, sequential in index order (the summation order is
//      part of the format contract: codebooks must come out bit-identical);
//   5. the dynamic programme over 16 classes in its divide-and-conquer form
//      (the left-most optimal split is monotone in the prefix length): the
//      recursion is walked level by level, one warp per node, lanes striding
//      over the node's candidate range, then a warp-wide (value, index) minimum
//      with the smaller index winning ties -- the same candidates and the same
//      tie rule as the host's depth-first walk;
//   6. back-track, class means -> fp16 codebook, codes by comparing each u with
//      the classes' upper bounds, nibbles packed 8 per thread.
// The objective is the k-class form of the one the reference evaluates for two
// classes (Python_Jenks_Test/Jenks_Tests/cuda_helpers.py:151-184).
#include "common.cuh"
#include <cfloat>

namespace jqg {

constexpr int kThreads = 1024;
constexpr int kWarps = kThreads / 32;
constexpr int kClasses = 16;

struct Node { int lo, hi, olo, ohi; };

struct RowWs {            // per-CTA scratch in global memory, sized for mcap = padded K
    double *uv;           // [mcap]   distinct values
    int *cnt;             // [mcap]   multiplicities
    double *P1, *P2, *C;  // [mcap+1] prefix sums
    double *prev, *cur;   // [mcap+1]
    int *arg;             // [17][mcap+1]
    Node *nodes[2];       // [mcap + 2] each: the non-empty intervals of one recursion level
};

__host__ __device__ inline size_t ws_bytes_per_cta(int mcap) {
    const size_t m1 = (size_t)mcap + 1;
    const size_t raw = sizeof(double) * mcap + sizeof(int) * (size_t)mcap + 5 * sizeof(double) * m1 +
                       sizeof(int) * 17 * m1 + 2 * sizeof(Node) * ((size_t)mcap + 2);
    return (raw + 255) / 256 * 256;   // every CTA's slice starts 256-byte aligned (it begins with doubles)
}

__device__ inline RowWs carve_ws(unsigned char *base, int mcap) {
    RowWs w;
    const size_t m1 = (size_t)mcap + 1;
    unsigned char *p = base;
    w.uv = reinterpret_cast<double *>(p); p += sizeof(double) * mcap;
    w.P1 = reinterpret_cast<double *>(p); p += sizeof(double) * m1;
    w.P2 = reinterpret_cast<double *>(p); p += sizeof(double) * m1;
    w.C = reinterpret_cast<double *>(p); p += sizeof(double) * m1;
    w.prev = reinterpret_cast<double *>(p); p += sizeof(double) * m1;
    w.cur = reinterpret_cast<double *>(p); p += sizeof(double) * m1;
    w.nodes[0] = reinterpret_cast<Node *>(p); p += sizeof(Node) * ((size_t)mcap + 2);
    w.nodes[1] = reinterpret_cast<Node *>(p); p += sizeof(Node) * ((size_t)mcap + 2);
    w.cnt = reinterpret_cast<int *>(p); p += sizeof(int) * (size_t)mcap;
    w.arg = reinterpret_cast<int *>(p);
    return w;
}

__device__ __forceinline__ double seg_cost(const RowWs &w, int a, int b) {
    const double d1 = __dsub_rn(w.P1[b], w.P1[a]);
    const double d2 = __dsub_rn(w.P2[b], w.P2[a]);
    const double c = __dsub_rn(w.C[b], w.C[a]);
    const double sq = __dmul_rn(d1, d1);
    const double q = __ddiv_rn(sq, c);
    return __dsub_rn(d2, q);
}

__global__ void __launch_bounds__(kThreads, 1) pack_gf4_kernel(const float *__restrict__ W, int N, int K, int g,
                                                                uint8_t *__restrict__ qw, __half *__restrict__ scales,
                                                                __half *__restrict__ codebook, unsigned char *__restrict__ ws,
                                                                int npad) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float *sv = reinterpret_cast<float *>(smem_raw);   // npad floats: the row being sorted
    __shared__ int s_m, s_ke, s_zero, s_breaks[kClasses + 1];
    __shared__ float s_upper[kClasses];                // largest value of each class
    __shared__ int s_scan[kWarps + 1];
    __shared__ int s_nn[2];                            // node counts of the current and next recursion level
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const RowWs w = carve_ws(ws + (size_t)blockIdx.x * ws_bytes_per_cta(npad), npad);
    const int G = g ? K / g : 0;
    const int stride_b = jq_row_stride_codes(K) >> 1;

    for (int row = blockIdx.x; row < N; row += gridDim.x) {
        const float *wr = W + (size_t)row * K;
        // ---- 1. scales and normalised values
        if (g) {
            for (int gi = warp; gi < G; gi += kWarps) {
                float amax = 0.f;
                for (int k = lane; k < g; k += 32) amax = fmaxf(amax, fabsf(wr[gi * g + k]));
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
                __half hs = __float2half_rn(amax);
                float s = __half2float(hs);
                if (amax == 0.f || s == 0.f || isinf(s) || isnan(s)) { hs = __float2half_rn(1.0f); s = 1.0f; }
                if (lane == 0) scales[(size_t)row * G + gi] = hs;
                for (int k = lane; k < g; k += 32) sv[gi * g + k] = __fdiv_rn(wr[gi * g + k], s);
            }
        } else {
            for (int k = tid; k < K; k += kThreads) sv[k] = wr[k];
        }
        for (int k = K + tid; k < npad; k += kThreads) sv[k] = __int_as_float(0x7f800000);  // +inf padding sorts last
        __syncthreads();
        // ---- 2. bitonic sort, ascending
        for (int size = 2; size <= npad; size <<= 1) {
            for (int stride = size >> 1; stride > 0; stride >>= 1) {
                for (int i = tid; i < npad / 2; i += kThreads) {
                    const int lo = 2 * i - (i & (stride - 1));
                    const int hi = lo + stride;
                    const bool up = (lo & size) == 0;
                    const float a = sv[lo], b = sv[hi];
                    if ((a > b) == up) { sv[lo] = b; sv[hi] = a; }
                }
                __syncthreads();
            }
        }
        // ---- 3. run-length compression of sv[0..K) into (uv, cnt)
        {
            // each thread owns a contiguous slice; head = first element of a run
            const int per = (K + kThreads - 1) / kThreads;
            const int b0 = min(tid * per, K), b1 = min(b0 + per, K);
            int heads = 0;
            for (int i = b0; i < b1; ++i) heads += (i == 0 || sv[i] != sv[i - 1]) ? 1 : 0;
            // block exclusive scan of heads
            int inc = heads;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) { int t = __shfl_up_sync(0xffffffffu, inc, o); if (lane >= o) inc += t; }
            if (lane == 31) s_scan[warp] = inc;
            __syncthreads();
            if (warp == 0) {
                int v = lane < kWarps ? s_scan[lane] : 0, vi = v;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) { int t = __shfl_up_sync(0xffffffffu, vi, o); if (lane >= o) vi += t; }
                if (lane < kWarps) s_scan[lane] = vi - v;
                if (lane == kWarps - 1) s_scan[kWarps] = vi;
            }
            __syncthreads();
            int pos = s_scan[warp] + inc - heads;   // index of this slice's first head
            if (tid == 0) s_m = s_scan[kWarps];
            // heads write their value; run lengths follow from the next head's position
            for (int i = b0; i < b1; ++i) {
                if (i == 0 || sv[i] != sv[i - 1]) {
                    w.uv[pos] = (double)sv[i] + 0.0;   // -0.0 and +0.0 are one value: +0.0
                    w.cnt[pos] = i;                     // start index for now
                    ++pos;
                }
            }
            __syncthreads();
            const int m = s_m;
            for (int t = tid; t < m; t += kThreads) {
                const int start = w.cnt[t];
                const int next = t + 1 < m ? w.cnt[t + 1] : K;
                // cannot overwrite cnt[t] before the neighbour read it: stash in prev (as int bits are not needed yet)
                w.prev[t] = (double)(next - start);
            }
            __syncthreads();
            for (int t = tid; t < m; t += kThreads) w.cnt[t] = (int)w.prev[t];
            __syncthreads();
        }
        const int m = s_m;
        const int ke = m < kClasses ? m : kClasses;
        // ---- 4. sequential float64 prefix sums
        if (tid == 0) {
            double p1 = 0.0, p2 = 0.0, c = 0.0;
            w.P1[0] = 0.0; w.P2[0] = 0.0; w.C[0] = 0.0;
#pragma unroll 4
            for (int t = 0; t < m; ++t) {
                const double v = w.uv[t], n = (double)w.cnt[t];
                const double cv = __dmul_rn(n, v);
                const double cvv = __dmul_rn(cv, v);
                p1 = __dadd_rn(p1, cv); p2 = __dadd_rn(p2, cvv); c = __dadd_rn(c, n);
                w.P1[t + 1] = p1; w.P2[t + 1] = p2; w.C[t + 1] = c;
            }
            s_ke = ke;
        }
        __syncthreads();
        // ---- 5. dynamic programme
        for (int i = tid; i <= m; i += kThreads) { w.prev[i] = i >= 1 ? seg_cost(w, 0, i) : DBL_MAX; w.cur[i] = DBL_MAX; }
        __syncthreads();
        double *prev = w.prev, *cur = w.cur;
        for (int j = 2; j <= ke; ++j) {
            for (int i = tid; i <= m; i += kThreads) cur[i] = DBL_MAX;
            if (tid == 0) {
                w.nodes[0][0] = (j == ke) ? Node{m, m, j - 1, m - 1} : Node{j, m, j - 1, m - 1};
                s_nn[0] = 1; s_nn[1] = 0;
            }
            __syncthreads();
            int buf = 0;
            while (true) {
                const Node *in = w.nodes[buf];
                Node *out = w.nodes[buf ^ 1];
                const int nn = s_nn[buf];
                for (int q = warp; q < nn; q += kWarps) {
                    const Node nd = in[q];   // never empty: only non-empty intervals are queued
                    const int mid = (nd.lo + nd.hi) >> 1;
                    const int t0 = max(nd.olo, j - 1), t1 = min(mid - 1, nd.ohi);
                    double best = DBL_MAX;
                    int bt = 0x7fffffff;
                    for (int t = t0 + lane; t <= t1; t += 32) {
                        const double c = __dadd_rn(prev[t], seg_cost(w, t, mid));
                        if (c < best) { best = c; bt = t; }   // ascending t per lane: first minimum of the lane
                    }
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) {
                        const double ob = __shfl_xor_sync(0xffffffffu, best, o);
                        const int ot = __shfl_xor_sync(0xffffffffu, bt, o);
                        if (ob < best || (ob == best && ot < bt)) { best = ob; bt = ot; }
                    }
                    if (bt == 0x7fffffff) bt = t0;            // empty range or all DBL_MAX: the host keeps t0
                    if (lane == 0) {
                        cur[mid] = best;
                        w.arg[(size_t)j * (m + 1) + mid] = bt;
                        if (nd.lo <= mid - 1) out[atomicAdd(&s_nn[buf ^ 1], 1)] = Node{nd.lo, mid - 1, nd.olo, bt};
                        if (mid + 1 <= nd.hi) out[atomicAdd(&s_nn[buf ^ 1], 1)] = Node{mid + 1, nd.hi, bt, nd.ohi};
                    }
                }
                __syncthreads();
                const int next = s_nn[buf ^ 1];
                __syncthreads();
                if (tid == 0) s_nn[buf] = 0;   // becomes the "next" counter after the swap
                buf ^= 1;
                __syncthreads();
                if (next == 0) break;
            }
            double *tswap = prev; prev = cur; cur = tswap;
            __syncthreads();
        }
        // ---- 6. back-track, codebook, class upper bounds
        if (tid == 0) {
            s_breaks[ke] = m;
            for (int j = ke; j >= 2; --j) s_breaks[j - 1] = w.arg[(size_t)j * (m + 1) + s_breaks[j]];
            s_breaks[0] = 0;
            // index of the distinct value 0.0 (m if the row has no exact zero)
            int lo = 0, hi = m;
            while (lo < hi) {
                const int mid = (lo + hi) >> 1;
                if (w.uv[mid] < 0.0) lo = mid + 1; else hi = mid;
            }
            s_zero = (lo < m && w.uv[lo] == 0.0) ? lo : m;
        }
        __syncthreads();
        if (tid < kClasses) {
            const int c = tid < ke ? tid : ke - 1;
            const int a = s_breaks[c], b = s_breaks[c + 1];
            double mean = __ddiv_rn(__dsub_rn(w.P1[b], w.P1[a]), __dsub_rn(w.C[b], w.C[a]));
            if (s_zero >= a && s_zero < b) mean = 0.0;   // the class holding an exact zero is pinned to 0 (as the host packer)
            codebook[(size_t)row * kClasses + tid] = __double2half(mean);
            s_upper[tid] = tid < ke ? (float)w.uv[b - 1] : __int_as_float(0x7f800000);
        }
        __syncthreads();
        // codes: class = number of class upper bounds below the value
        const int words = stride_b >> 2;
        for (int wi = tid; wi < words; wi += kThreads) {
            uint32_t word = 0;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const int k = wi * 8 + e;
                if (k < K) {
                    float u = wr[k];
                    if (g) {
                        float s = __half2float(scales[(size_t)row * G + k / g]);
                        u = __fdiv_rn(u, s);
                    }
                    int c = 0;
#pragma unroll
                    for (int q = 0; q < kClasses - 1; ++q) c += (u > s_upper[q]) ? 1 : 0;
                    word |= (uint32_t)c << (4 * e);
                }
            }
            reinterpret_cast<uint32_t *>(qw + (size_t)row * stride_b)[wi] = word;
        }
        __syncthreads();
    }
}

}  // namespace jqg

static int next_pow2(int v) { int p = 1; while (p < v) p <<= 1; return p; }

extern "C" size_t jq_pack_gf4_workspace_bytes(int K) {
    if (K <= 0) return 0;
    return jqg::ws_bytes_per_cta(next_pow2(K)) * (size_t)jq_sm_count();
}

extern "C" int jq_pack_gf4(const float *W, int N, int K, int g, void *qweight, void *scales, void *codebook,
                           void *workspace, size_t workspace_bytes, jq_stream_t stream) {
    if (!W || !qweight || !codebook || !workspace) return JQ_ERR_NULL_PTR;
    if (N <= 0 || K <= 0 || g < 0 || (g && (g % 32 || K % g))) return JQ_ERR_BAD_SHAPE;
    if (g && !scales) return JQ_ERR_NULL_PTR;
    const int npad = next_pow2(K);
    const size_t smem = (size_t)npad * sizeof(float);
    if (smem > 200 * 1024) return JQ_ERR_UNSUPPORTED;   // rows longer than 51200 values
    if (workspace_bytes < jq_pack_gf4_workspace_bytes(K)) return JQ_ERR_WORKSPACE;
    if ((reinterpret_cast<uintptr_t>(workspace) & 255u) || !jq_aligned16(qweight) || (reinterpret_cast<uintptr_t>(W) & 3u))
        return JQ_ERR_BAD_ALIGN;
    auto kern = jqg::pack_gf4_kernel;
    JQ_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    int grid = jq_sm_count();
    if (grid > N) grid = N;
    kern<<<grid, jqg::kThreads, smem, reinterpret_cast<cudaStream_t>(stream)>>>(
        W, N, K, g, reinterpret_cast<uint8_t *>(qweight), reinterpret_cast<__half *>(scales),
        reinterpret_cast<__half *>(codebook), reinterpret_cast<unsigned char *>(workspace), npad);
    return jq_launch_status();
}
