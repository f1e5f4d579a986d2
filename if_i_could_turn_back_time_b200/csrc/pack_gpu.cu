// Device-side packer for the E2M1 format: fp32 weights -> packed codes + fp16
// group scales, bit-identical to the host packer (pack_host.cpp).  Replaces
// the grid construction of QuantLinear.__init__
// (Python_Jenks_Test/Jenks_Tests/Quantization_Experiments/layers.py:22-26) for
// weights that already live on the GPU.
#include "common.cuh"

namespace jqp {

// nearest E2M1 code, ties to the even mantissa bit, saturating; never code 8
__device__ __forceinline__ uint32_t e2m1_code(float u) {
    const float a = fabsf(u);
    int idx;
    if (a <= 0.25f) idx = 0;
    else if (a < 0.75f) idx = 1;
    else if (a <= 1.25f) idx = 2;
    else if (a < 1.75f) idx = 3;
    else if (a <= 2.5f) idx = 4;
    else if (a < 3.5f) idx = 5;
    else if (a <= 5.0f) idx = 6;
    else idx = 7;
    return (u < 0.f && idx != 0) ? (uint32_t)idx + 8u : (uint32_t)idx;
}

// one thread per 32-code slice of a group; a group of g codes is g/32 adjacent threads of one warp
__global__ void __launch_bounds__(256) pack_e2m1_kernel(const float *__restrict__ W, int N, int K, int g,
                                                         uint8_t *__restrict__ qw, __half *__restrict__ scales) {
    const int slices_per_row = K >> 5, per_group = g >> 5;
    const long long total = (long long)N * slices_per_row;
    const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    const bool live = idx < total;
    const int n = live ? (int)(idx / slices_per_row) : 0, sl = live ? (int)(idx % slices_per_row) : 0;
    float v[32];
    float amax = 0.f;
    if (live) {
        const float4 *src = reinterpret_cast<const float4 *>(W + (size_t)n * K + (size_t)sl * 32);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float4 t = src[j];
            v[4 * j] = t.x; v[4 * j + 1] = t.y; v[4 * j + 2] = t.z; v[4 * j + 3] = t.w;
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) amax = fmaxf(amax, fabsf(v[j]));
    }
    // group maximum over the per_group adjacent lanes (per_group is a power of two <= 32 here)
    for (int o = 1; o < per_group; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if (!live) return;
    __half hs = __float2half_rn(__fdiv_rn(amax, 6.0f));
    float s = __half2float(hs);
    if (amax == 0.f || s == 0.f) { hs = __float2half_rn(1.0f); s = 1.0f; }
    if (isinf(s)) { hs = __ushort_as_half((unsigned short)0x7bffu); s = 65504.0f; }   // absmax / 6 beyond fp16: largest finite scale, codes saturate
    if ((sl % per_group) == 0) scales[(size_t)n * (K / g) + sl / per_group] = hs;
    uint32_t words[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        uint32_t w = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) w |= e2m1_code(__fdiv_rn(v[8 * q + j], s)) << (4 * j);
        words[q] = w;
    }
    *reinterpret_cast<uint4 *>(qw + (size_t)n * (K >> 1) + (size_t)sl * 16) = make_uint4(words[0], words[1], words[2], words[3]);
}

}  // namespace jqp

extern "C" int jq_pack_e2m1(const float *W, int N, int K, int g, void *qweight, void *scales, jq_stream_t stream) {
    if (!W || !qweight || !scales) return JQ_ERR_NULL_PTR;
    if (N <= 0 || K <= 0 || g <= 0 || g % 32 || K % g) return JQ_ERR_BAD_SHAPE;
    const int per_group = g >> 5;
    if (per_group > 32 || (per_group & (per_group - 1))) return JQ_ERR_UNSUPPORTED;  // group within one warp
    if ((K >> 5) % per_group) return JQ_ERR_BAD_SHAPE;
    if (!jq_aligned16(W) || !jq_aligned16(qweight)) return JQ_ERR_BAD_ALIGN;
    const long long total = (long long)N * (K >> 5);
    const long long blocks = (total + 255) / 256;
    if (blocks > 0x7fffffffLL) return JQ_ERR_BAD_SHAPE;
    jqp::pack_e2m1_kernel<<<(int)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        W, N, K, g, reinterpret_cast<uint8_t *>(qweight), reinterpret_cast<__half *>(scales));
    return jq_launch_status();
}
