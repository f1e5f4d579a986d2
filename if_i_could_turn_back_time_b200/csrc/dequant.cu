// Packed 4-bit -> dense fp32 (bit-exact: one fp32 multiply per weight), and
// the stand-alone block Hadamard rotation.
#include "common.cuh"

namespace jq {

__constant__ float kE2M1[16] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f,
                                -0.f, -0.5f, -1.f, -1.5f, -2.f, -3.f, -4.f, -6.f};

// One thread per 32-bit word (8 codes).  Rows of the packed matrix are
// stride/8 words; the dense output has no padding.
template <int FMT>
__global__ void __launch_bounds__(256) dequant_kernel(const uint32_t *__restrict__ qw, const __half *__restrict__ scales,
                                                       const __half *__restrict__ codebook, float *__restrict__ out,
                                                       int N, int K, int g) {
    const int words_per_row = jq_row_stride_codes(K) >> 3;
    const long long total = (long long)N * words_per_row;
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const int n = (int)(idx / words_per_row), wi = (int)(idx % words_per_row);
        const int k0 = wi * 8;
        if (k0 >= K) continue;
        const uint32_t word = qw[idx];
        float s = 1.f;
        if (g) s = __half2float(scales[(size_t)n * (K / g) + k0 / g]);  // g % 32 == 0: one group per word
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint32_t c = (word >> (4 * j)) & 0xfu;
            float t;
            if (FMT == JQ_FMT_E2M1) t = kE2M1[c];
            else t = __half2float(codebook[(size_t)n * 16 + c]);
            v[j] = g ? __fmul_rn(t, s) : t;
        }
        float *o = out + (size_t)n * K + k0;
        if (k0 + 8 <= K && ((reinterpret_cast<uintptr_t>(o) & 15u) == 0)) {
            reinterpret_cast<float4 *>(o)[0] = make_float4(v[0], v[1], v[2], v[3]);
            reinterpret_cast<float4 *>(o)[1] = make_float4(v[4], v[5], v[6], v[7]);
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (k0 + j < K) o[j] = v[j];
        }
    }
}

// One warp per 128-block.
__global__ void __launch_bounds__(256) fwht_kernel(const void *__restrict__ x, float *__restrict__ y, long long nblocks,
                                                    int x_dtype) {
    const int lane = threadIdx.x & 31;
    const long long warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
    const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
    for (long long blk = warp; blk < nblocks; blk += nwarps) {
        float v[4];
        const size_t k0 = (size_t)blk * 128 + lane * 4;
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] = load_act(x, k0 + j, x_dtype);
        fwht128_warp(v, lane);
        *reinterpret_cast<float4 *>(y + k0) = make_float4(v[0], v[1], v[2], v[3]);
    }
}

}  // namespace jq

using namespace jq;

static int dequant_common(int fmt, const void *qw, const void *scales, const void *codebook, float *out, int N, int K,
                          int g, jq_stream_t stream) {
    if (!qw || !out) return JQ_ERR_NULL_PTR;
    if (fmt == JQ_FMT_GF4 && !codebook) return JQ_ERR_NULL_PTR;
    if (N <= 0 || K <= 0) return JQ_ERR_BAD_SHAPE;
    if (fmt == JQ_FMT_E2M1 && g == 0) return JQ_ERR_BAD_SHAPE;
    if (g < 0 || (g && (g % 32 || K % g))) return JQ_ERR_BAD_SHAPE;
    if (g && !scales) return JQ_ERR_NULL_PTR;
    if (!jq_aligned16(qw)) return JQ_ERR_BAD_ALIGN;
    if (reinterpret_cast<uintptr_t>(out) & 3u) return JQ_ERR_BAD_ALIGN;
    const long long total = (long long)N * (jq_row_stride_codes(K) >> 3);
    long long blocks = (total + 255) / 256;
    const long long cap = (long long)jq_sm_count() * 16;
    if (blocks > cap) blocks = cap;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (fmt == JQ_FMT_E2M1)
        dequant_kernel<JQ_FMT_E2M1><<<(int)blocks, 256, 0, st>>>(reinterpret_cast<const uint32_t *>(qw),
                                                                 reinterpret_cast<const __half *>(scales), nullptr, out,
                                                                 N, K, g);
    else
        dequant_kernel<JQ_FMT_GF4><<<(int)blocks, 256, 0, st>>>(reinterpret_cast<const uint32_t *>(qw),
                                                                reinterpret_cast<const __half *>(scales),
                                                                reinterpret_cast<const __half *>(codebook), out, N, K,
                                                                g);
    return jq_launch_status();
}

extern "C" int jq_dequant_e2m1(const void *qweight, const void *scales, float *out, int N, int K, int g,
                               jq_stream_t stream) {
    return dequant_common(JQ_FMT_E2M1, qweight, scales, nullptr, out, N, K, g, stream);
}

extern "C" int jq_dequant_gf4(const void *qweight, const void *scales, const void *codebook, float *out, int N, int K,
                              int g, jq_stream_t stream) {
    return dequant_common(JQ_FMT_GF4, qweight, scales, codebook, out, N, K, g, stream);
}

extern "C" int jq_fwht_block(const void *x, float *y, int B, int K, int block, int x_dtype, jq_stream_t stream) {
    if (!x || !y) return JQ_ERR_NULL_PTR;
    if (B <= 0 || K <= 0) return JQ_ERR_BAD_SHAPE;
    if (block != 128) return JQ_ERR_UNSUPPORTED;
    if (K % block) return JQ_ERR_BAD_SHAPE;
    if (x_dtype != JQ_F32 && x_dtype != JQ_F16 && x_dtype != JQ_BF16) return JQ_ERR_BAD_DTYPE;
    if (!jq_aligned16(y)) return JQ_ERR_BAD_ALIGN;
    const long long nblocks = (long long)B * (K / 128);
    long long blocks = (nblocks + 7) / 8;
    const long long cap = (long long)jq_sm_count() * 8;
    if (blocks > cap) blocks = cap;
    fwht_kernel<<<(int)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(x, y, nblocks, x_dtype);
    return jq_launch_status();
}
