// Shared device/host helpers for libjq (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include "../../include/jq.h"

#define JQ_SM_COUNT_FALLBACK 148

#define JQ_CUDA_TRY(expr)                                     \
    do {                                                      \
        cudaError_t _e = (expr);                              \
        if (_e != cudaSuccess) return JQ_ERR_CUDA_BASE - (int)_e; \
    } while (0)

// Right after a launch: the thread's last CUDA error, read and thereby cleared.  CUDA has one slot per thread,
// so an earlier unread asynchronous error of the process lands here too (stated in jq.h).
static inline int jq_launch_status() {
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? JQ_OK : JQ_ERR_CUDA_BASE - (int)e;
}

static inline bool jq_aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Number of SMs of the current device (cached per device id).
int jq_sm_count();

__host__ __device__ static inline int jq_row_stride_codes(int K) { return (K + 31) / 32 * 32; }

namespace jq {

// 16-byte streaming load that bypasses L1 allocation: packed weights are read
// exactly once.
__device__ __forceinline__ uint4 ldg_stream_u4(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::128B.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// Two E2M1 codes (one byte, low nibble first) -> half2, exact.
__device__ __forceinline__ uint32_t e2m1x2_to_h2(uint32_t byte) {
    uint32_t h2;
    asm("{ .reg .b8 lo, hi; .reg .b16 t; cvt.u16.u32 t, %1; mov.b16 {lo, hi}, t; cvt.rn.f16x2.e2m1x2 %0, lo; }"
        : "=r"(h2)
        : "r"(byte));
    return h2;
}

// acc += a * b with a, b fp16 (exact product) and fp32 accumulation.
__device__ __forceinline__ void fma_h(float &acc, uint16_t a, uint16_t b) {
    asm("fma.rn.f32.f16 %0, %1, %2, %0;" : "+f"(acc) : "h"(a), "h"(b));
}

__device__ __forceinline__ uint16_t h2_lo(uint32_t v) { return (uint16_t)(v & 0xffffu); }
__device__ __forceinline__ uint16_t h2_hi(uint32_t v) { return (uint16_t)(v >> 16); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float load_act(const void *x, size_t i, int dtype) {
    if (dtype == JQ_F32) return reinterpret_cast<const float *>(x)[i];
    if (dtype == JQ_F16) return __half2float(reinterpret_cast<const __half *>(x)[i]);
    return __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(x)[i]);
}

__device__ __forceinline__ void store_out(void *y, size_t i, float v, int dtype) {
    if (dtype == JQ_F32) reinterpret_cast<float *>(y)[i] = v;
    else if (dtype == JQ_F16) reinterpret_cast<__half *>(y)[i] = __float2half_rn(v);
    else reinterpret_cast<__nv_bfloat16 *>(y)[i] = __float2bfloat16_rn(v);
}

// The same element of n <= 8 copies of the output (this rank's buffer and its peers'), copy c at byte offset
// delta[c] from y.  The offset is picked with constant indices: indexing the array with a variable would make
// the compiler keep it (and the structure around it) in local memory.
template <class Delta>
__device__ __forceinline__ long long peer_offset(const Delta &delta, int c) {
    long long d = delta[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) d = (i == c) ? delta[i] : d;
    return d;
}
template <class Delta>
__device__ __forceinline__ void store_out_copies(void *y, const Delta &delta, int n, size_t i, float v, int dtype) {
    for (int c = 0; c < n; ++c) store_out(reinterpret_cast<char *>(y) + peer_offset(delta, c), i, v, dtype);
}

// In-warp orthonormal Hadamard of one 128-block: lane holds elements
// 4*lane .. 4*lane+3.  Stage order (strides 1,2,4,..,64) and the a+b / a-b
// slot convention are part of the format contract: fp32 results must be
// reproducible bit for bit.
__device__ __forceinline__ void fwht128_warp(float (&v)[4], int lane) {
    float a0 = v[0] + v[1], a1 = v[0] - v[1], a2 = v[2] + v[3], a3 = v[2] - v[3];  // stride 1
    v[0] = a0 + a2; v[2] = a0 - a2; v[1] = a1 + a3; v[3] = a1 - a3;              // stride 2
#pragma unroll
    for (int m = 1; m < 32; m <<= 1) {  // strides 4..64 live across lanes
        const bool high = (lane & m) != 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float o = __shfl_xor_sync(0xffffffffu, v[j], m);
            v[j] = high ? (o - v[j]) : (v[j] + o);
        }
    }
    const float s = 0.08838834764831845f;
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = v[j] * s;
}

}  // namespace jq
