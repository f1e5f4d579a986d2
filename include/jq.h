/* jq.h -- C ABI of libjq.so: packed 4-bit (E2M1 / GF4) dequantise-and-multiply
 * for NVIDIA B200 (sm_100a).
 *
 * The library slots in under the quantized-Linear forward of
 * jvap2/If_I_could_turn_back_time, replacing the per-call
 *     W_bar = mask * s * (Q + Theta);  y = F.linear(x, W_bar, bias)
 * of Python_Jenks_Test/Jenks_Tests/Quantization_Experiments/layers.py:33-38
 * (and the same F.linear boundary at Quantization_Experiments/brecq.py:321-329)
 * by one fused kernel over packed weights.  The reference has no native code
 * on this path; its only native boundary is a torch C++ extension
 * (Python_Jenks_Test/Jenks_Tests/cuda_helpers.py:186-211).  Conventions here:
 *
 *   - plain C types only; every function returns an int status, 0 = JQ_OK,
 *     negative = error (jq_strerror gives the text); nothing calls exit(),
 *     throws, resets the device or synchronises it;
 *   - the caller owns every buffer; device pointers are raw addresses
 *     (tensor.data_ptr()); the library allocates no device memory and keeps
 *     no reference after return;
 *   - work is enqueued on the CUDA stream passed in (a cudaStream_t cast to
 *     void*; NULL is the legacy default stream) and returns immediately;
 *   - arguments are validated on the host before anything is launched.
 *
 * Formats.  qweight is uint8 [N, stride/2] row-major, stride = K rounded up to
 * a multiple of 32 codes (rows are 16-byte multiples); byte j of a row holds
 * code 2j in bits 3:0 and code 2j+1 in bits 7:4; padding codes are 0.
 *   E2M1: code = s e1 e0 m, magnitudes {0,.5,1,1.5,2,3,4,6}; scales are fp16
 *         [N, K/g]; w = fp32(value(code)) * fp32(scale).
 *   GF4 : code indexes codebook fp16 [N,16] (ascending per row); scales are
 *         fp16 [N, K/g] or absent (g = 0); w = fp32(codebook[n][code]) *
 *         fp32(scale)   (or just fp32(codebook[n][code]) when g = 0).
 * g is 0 (GF4 only) or a multiple of 32 that divides K.
 * Alignment: qweight and codebook 16 bytes (rows are 16- / 32-byte multiples, so
 * every row slice of an aligned matrix qualifies), scales 2 bytes; anything
 * else is refused with JQ_ERR_BAD_ALIGN before a launch.
 */
#ifndef JQ_H_
#define JQ_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define JQ_VERSION 100

/* status codes */
#define JQ_OK 0
#define JQ_ERR_NULL_PTR (-1)
#define JQ_ERR_BAD_SHAPE (-2)
#define JQ_ERR_BAD_ALIGN (-3)
#define JQ_ERR_BAD_DTYPE (-4)
#define JQ_ERR_UNSUPPORTED (-5)
#define JQ_ERR_WORKSPACE (-6)
#define JQ_ERR_TIMEOUT (-7)
#define JQ_ERR_NOMEM (-8)
#define JQ_ERR_SCRATCH_LIMIT (-9)
#define JQ_ERR_CUDA_BASE (-1000) /* JQ_ERR_CUDA_BASE - cudaError_t */
/* A launching entry point reads the calling thread's last CUDA error right after its launch (cudaGetLastError:
 * reading clears it).  CUDA keeps one such slot per thread, so an asynchronous error left there earlier by other
 * code of the process, and not yet read by it, is reported by -- and attributed to -- the next libjq launch; a
 * caller that mixes libraries should read cudaGetLastError() itself before calling in if it needs to tell the two
 * apart.  A non-sticky error never outlives the call that reports it. */

/* element types of activations / outputs */
#define JQ_F32 0
#define JQ_F16 1
#define JQ_BF16 2

/* weight formats */
#define JQ_FMT_E2M1 0
#define JQ_FMT_GF4 1

/* ops for jq_workspace_bytes */
#define JQ_OP_GEMV 0
#define JQ_OP_GROUPED 2

typedef void *jq_stream_t;

/* Library version (JQ_VERSION of the build).  No reference counterpart. */
int jq_version(void);

/* Text for a status code; never NULL.  Replaces the bool HandleCUDAError +
 * exit(1) convention of CUDA_C_Code/include/GPUErrors.cu:3-12. */
const char *jq_strerror(int status);

/* Dequantise a packed matrix to dense fp32 out[N,K] (row-major, no padding).
 * Bit-exact: one fp32 multiply per weight.  Replaces the elementwise
 * "mask * s * (Q + Theta)" materialisation of
 * Quantization_Experiments/layers.py:37 and QuantLinear.commit (:39-45). */
int jq_dequant_e2m1(const void *qweight, const void *scales, float *out,
                    int N, int K, int g, jq_stream_t stream);
int jq_dequant_gf4(const void *qweight, const void *scales_or_null, const void *codebook,
                   float *out, int N, int K, int g, jq_stream_t stream);

/* Orthonormal block Walsh-Hadamard rotation of x[B,K] (x_dtype) into fp32
 * y[B,K]; block must be 128 and divide K.  Fixed butterfly order (strides
 * 1,2,..,64, a+b low / a-b high, then one multiply by fp32(1/sqrt(128))), so
 * results are reproducible bit for bit.  No reference counterpart (the
 * reference has no rotation); it is the stand-alone form of the prologue
 * fused into jq_gemv_*. */
int jq_fwht_block(const void *x, float *y, int B, int K, int block, int x_dtype,
                  jq_stream_t stream);

/* y[B,N] = rotate(x)[B,K] . W_hat[N,K]^T + bias, W_hat never materialised.
 * Replaces F.linear(x, W_bar, bias) at Quantization_Experiments/layers.py:38
 * (and :35) for 1 <= B <= 8.  x is row-major [B,K] of x_dtype, y row-major
 * [B,N] of y_dtype, bias fp32 [N] or NULL.  had_block is 0 (no rotation) or
 * 128 (K % 128 == 0).  The rotated activation is rounded to fp16 after an
 * exact power-of-two normalisation per batch row; products are exact and
 * accumulated in fp32 (batch 1 and GF4: fma.rn.f32.f16 on the CUDA cores; E2M1
 * with 32-code groups, K % 256 == 0 and 2 <= B <= 8: the same products on
 * mma.sync.m16n8k16, one instruction per 256 codes whatever B).  workspace may
 * be NULL when jq_workspace_bytes says 0. */
int jq_gemv_e2m1(const void *qweight, const void *scales, const void *x,
                 const float *bias_or_null, void *y, int N, int K, int B, int g,
                 int had_block, int x_dtype, int y_dtype, void *workspace,
                 size_t workspace_bytes, jq_stream_t stream);
int jq_gemv_gf4(const void *qweight, const void *scales_or_null, const void *codebook,
                const void *x, const float *bias_or_null, void *y, int N, int K, int B,
                int g, int had_block, int x_dtype, int y_dtype, void *workspace,
                size_t workspace_bytes, jq_stream_t stream);

/* The same operator for callers that must not allocate device memory and
 * have no buffer of their own to lend as a workspace: code running inside a
 * memory-pool callback or an allocator hook, a real-time loop whose memory was
 * fixed at start-up, a host that only hands this library the tensors of the
 * layer.  Such a caller cannot call cudaMalloc (it may deadlock on the
 * allocator it is being called from, or break a latency or footprint
 * guarantee) and cannot size a torch workspace either.  When the batch needs
 * the split-K path (B x K too large to stage in shared memory), this entry
 * keeps the fp32 partial outputs in a fixed array compiled into the library
 * (JQ_NOALLOC_SCRATCH_BYTES, 8 MiB per GPU, held from library load to
 * process exit) instead of a caller workspace.  fmt is JQ_FMT_E2M1 or
 * JQ_FMT_GF4 (codebook NULL for E2M1); the other arguments are those of
 * jq_gemv_*.  It has no counterpart in the reference.
 *   - Limit: tiles * B * N * 4 bytes must fit the array, otherwise
 *     JQ_ERR_SCRATCH_LIMIT is returned and nothing is launched.
 *   - The first call on each device looks up the array's device address
 *     (a driver query, not an allocation); make that first call outside any
 *     stream capture.
 *   - All calls on a device share the one array.  Every word a call reads
 *     from it was written earlier in the same call, so nothing has to be
 *     cleared between calls; but two calls whose kernels may overlap on the
 *     GPU (different streams, no ordering) race on it.  Serialise them.
 *   - No cudaMalloc, cudaFree or allocating library routine is called. */
#define JQ_NOALLOC_SCRATCH_BYTES (8u << 20)
int jq_gemv_noalloc(int fmt, const void *qweight, const void *scales_or_null,
                    const void *codebook_or_null, const void *x, const float *bias_or_null,
                    void *y, int N, int K, int B, int g, int had_block, int x_dtype,
                    int y_dtype, jq_stream_t stream);

/* Self test of the failure path of the kernels' device-side waits: one CTA
 * polls (at most `polls` times, <= 2^20) an mbarrier that nothing arrives on,
 * gives up, and writes JQ_ERR_TIMEOUT to *status_dev (device int).  Nothing
 * traps or hangs; the context stays usable.  No reference counterpart (the
 * reference's native code calls exit(1) on any CUDA error,
 * CUDA_C_Code/include/layers.h:1195-1199). */
int jq_selftest_bounded_wait(int *status_dev, unsigned int polls, jq_stream_t stream);

/* One entry of a grouped launch: an independent GEMV problem. */
typedef struct jq_problem {
    const void *qweight;
    const void *scales;    /* NULL when g == 0 */
    const void *codebook;  /* NULL for E2M1 */
    const void *x;
    const float *bias;     /* NULL for none */
    void *y;
    int32_t N, K, g, had_block;
    int32_t ldy;           /* outputs between batch rows of y; 0 means N.  A row shard of a wider layer sets
                              this to the unsharded N and points y at its first row's column. */
    int32_t reserved[3];   /* must be 0 */
} jq_problem;

/* Grouped launch: n independent GEMVs (same format, batch B and dtypes) in
 * ONE launch of persistent CTAs that walk the concatenated row space of all
 * problems; used for a decode step's layer set, where one launch per matrix
 * would be bound by launch latency.  Two phases:
 *   jq_grouped_plan   (host only, once per layer set) validates the problems
 *       and writes a partition plan of jq_grouped_plan_bytes(n) bytes into
 *       plan_host; the caller copies those bytes to the device (plan_dev);
 *   jq_gemv_grouped   enqueues the launch; it reads a few ints of plan_host
 *       on the host, touches no device memory on the host side and does not
 *       synchronise.
 * problems_dev is a DEVICE array of the same n jq_problem given to the plan.
 * No reference counterpart: the reference runs one F.linear per layer
 * (Python_Jenks_Test/Jenks_Tests/QuantNetworkTest.py:236-238). */
size_t jq_grouped_plan_bytes(int n);
int jq_grouped_plan(int fmt, const jq_problem *problems_host, int n, int B, void *plan_host,
                    size_t plan_bytes);
int jq_gemv_grouped(const jq_problem *problems_dev, const void *plan_host, const void *plan_dev,
                    int x_dtype, int y_dtype, jq_stream_t stream);

/* The grouped launch with the all-gather of a row-sharded layer fused into
 * its epilogue: every output element is stored at the same byte offset into
 * npeer (<= 8) output buffers, the local one (peer_delta 0) and those of the
 * peer GPUs (peer_delta[i] = peer buffer base - local buffer base, from
 * symmetric / peer-mapped memory), as plain stores over NVLink; no loads from
 * peer memory, no multicast.  The caller still has to order the ranks (a
 * barrier after the launch) before anyone reads the gathered outputs.  The
 * reference has no multi-device path
 * (Python_Jenks_Test/Jenks_Tests/QuantNetworkTest.py:19 picks one device). */
int jq_gemv_grouped_peers(const jq_problem *problems_dev, const void *plan_host,
                          const void *plan_dev, int x_dtype, int y_dtype, int npeer,
                          const int64_t *peer_delta, jq_stream_t stream);

/* The TMA-fed kernels (B200 tensor memory).  Same operator as jq_gemv_gf4 /
 * jq_gemv_e2m1, i.e. the F.linear(x, W_bar, bias) of
 * Quantization_Experiments/layers.py:38, for K % 256 == 0, K >= 512,
 * qweight / codebook / E2M1 scales 16-byte aligned, and
 *   fmt GF4,  group sizes of 128 * 2^k, 1 <= B <= 16;
 *   fmt E2M1, group size 32,            1 <= B <= 64.
 * The packed rows arrive by 2-D tiled TMA (32-row x 128-byte boxes, 128-byte
 * swizzle), a decode thread owns one weight row of a 128-row tile.
 *   GF4: a byte of packed codes indexes a 256-entry table of fp16 pairs that is
 *        built per tile in shared memory, one bank column per weight row, so
 *        two codes cost one conflict-free lookup.  Every weight and every scale
 *        stays exact; only the fp32 summation order differs from jq_gemv_gf4.
 *        B == 1 (K <= 12288): the decode threads also multiply (fma.rn.f32.f16,
 *        fp32 accumulation), reading the prepared activation by broadcast
 *        shared-memory loads.  Otherwise the fp16 values go to tensor memory
 *        (tcgen05.st) as the A operand of tcgen05.mma kind::f16, one fp32
 *        accumulator per 128-code group, read back (tcgen05.ld) and scaled by
 *        the group's fp16 scale in fp32.
 *   E2M1: cvt.rn.f16x2.e2m1x2 per byte, then the group's fp16 scale is
 *        multiplied in with mul.rn.f16x2 -- ONE fp16 rounding per weight that
 *        jq_gemv_e2m1 does not have (its weights are exact): the results of the
 *        two entry points differ by up to about 2^-11 relative per weight, well
 *        inside the 1e-3 gate of the operator, and the dequantised matrix
 *        (jq_dequant_e2m1) remains the exact one.  The whole row accumulates in
 *        tensor memory (fp32).
 * A launch is preceded by a small kernel that rotates, normalises and rounds
 * the activation to fp16 once per problem (not once per CTA).  The workspace
 * (128-byte aligned, jq_ta_workspace_bytes) holds that prepared activation and
 * a status word at offset 0, which must be zero before the first use and is
 * only ever raised by the kernels: every device-side wait is bounded (2^22
 * polls or about 0.25 s); one that gives up leaves JQ_ERR_TIMEOUT there, the
 * CTA's roles leave their loops, free tensor memory and the kernel returns
 * early with y partly written.  The word is sticky across launches;
 * jq_ta_status reads it (synchronising the stream) and, with clear != 0,
 * resets it.  Grouped form: jq_ta_plan (host only) validates the problems,
 * creates their tensor maps and writes jq_ta_plan_bytes(n) bytes that the
 * caller copies to the device (64-byte aligned); jq_gemm_ta_grouped enqueues
 * the two launches, with the peer-store all-gather of jq_gemv_grouped_peers
 * when npeer > 1.  problems_host[i].K alone is read by jq_ta_workspace_bytes.
 * Unsupported shapes return JQ_ERR_UNSUPPORTED, misaligned pointers
 * JQ_ERR_BAD_ALIGN; nothing is launched then. */
size_t jq_ta_workspace_bytes(const jq_problem *problems_host, int n, int B);
size_t jq_ta_plan_bytes(int n);
int jq_ta_plan(int fmt, const jq_problem *problems_host, int n, int B, void *workspace_dev,
               size_t workspace_bytes, void *plan_host, size_t plan_bytes);
int jq_gemm_ta_grouped(const void *plan_host, const void *plan_dev, void *workspace_dev,
                       int x_dtype, int y_dtype, int npeer, const int64_t *peer_delta,
                       jq_stream_t stream);
int jq_gemm_ta(int fmt, const void *qweight, const void *scales, const void *codebook,
               const void *x, const float *bias_or_null, void *y, int N, int K, int B, int g,
               int had_block, int x_dtype, int y_dtype, void *workspace, size_t workspace_bytes,
               jq_stream_t stream);
int jq_ta_status(void *workspace, int clear, jq_stream_t stream);

/* Bytes of caller-provided device scratch an op needs for these sizes. */
size_t jq_workspace_bytes(int op, int N, int K, int B);

/* Two-class Jenks natural break of an ascending-sorted fp32 array (device),
 * O(n) with float64 prefix sums.  Replaces the O(n^2) kernel
 * jenks_optimization_cuda of Python_Jenks_Test/Jenks_Tests/cuda_helpers.py:151-211
 * and the host argmin / GVF of its wrapper Linear_Mask (:378-395).
 * var_or_null (device, n doubles) receives var[i] = SSD(v[:i]) + SSD(v[i:])
 * when given; out3 (device, 3 doubles) receives {break index (first argmin),
 * min var, GVF = (SSD_total - min var) / (SSD_total + 1e-8)}. */
size_t jq_jenks2_workspace_bytes(long long n);
int jq_jenks2_break(const float *sorted, long long n, double *var_or_null, double *out3,
                    void *workspace, size_t workspace_bytes, jq_stream_t stream);

/* E2M1 packer on the device: W fp32 [N,K] (device) -> qweight, scales (device),
 * bit-identical to jq_pack_e2m1_host.  g must be 32 * a power of two <= 1024.
 * Same reference counterpart as the host packers below. */
int jq_pack_e2m1(const float *W, int N, int K, int g, void *qweight, void *scales,
                 jq_stream_t stream);

/* GF4 packer on the device (per-row 16-class Jenks natural breaks, one CTA per
 * row), bit-identical to jq_pack_gf4_host; rows up to 51200 values.  scales
 * may be NULL when g == 0.  workspace: jq_pack_gf4_workspace_bytes(K) bytes. */
size_t jq_pack_gf4_workspace_bytes(int K);
int jq_pack_gf4(const float *W, int N, int K, int g, void *qweight, void *scales_or_null,
                void *codebook, void *workspace, size_t workspace_bytes, jq_stream_t stream);

/* ---- host-side packers (CPU, multi-threaded; one-off, not the hot path) ----
 * Replace the grid/scale construction of QuantLinear.__init__
 * (Quantization_Experiments/layers.py:22-26) for the packed formats.  All
 * pointers are HOST memory.  W is fp32 [N,K] row-major.  qweight receives
 * [N, stride/2] bytes, scales fp16 bits [N, K/g], codebook fp16 bits [N,16].
 * threads <= 0 means "all hardware threads". */
int jq_pack_e2m1_host(const float *W, int N, int K, int g, uint8_t *qweight,
                      uint16_t *scales, int threads);
/* GF4: per-row 16-class Jenks natural breaks (the k-class form of the
 * objective in Python_Jenks_Test/Jenks_Tests/cuda_helpers.py:151-184) on the
 * group-normalised row; g = 0 means no scales (Jenks on the raw row). */
int jq_pack_gf4_host(const float *W, int N, int K, int g, uint8_t *qweight,
                     uint16_t *scales_or_null, uint16_t *codebook, int threads);
/* In-place right-multiplication of W[N,K] by blockdiag(H_128/sqrt(128)) in
 * fp32 (the offline weight-side rotation paired with had_block = 128). */
int jq_rotate_weights_host(float *W, int N, int K, int block, int threads);

#ifdef __cplusplus
}
#endif
#endif /* JQ_H_ */
