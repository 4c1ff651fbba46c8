/*
 * cfk_b200.h — C ABI of libcfk_b200.so (sm_100a flash-attention forward + GEMM).
 *
 * Every entry point takes plain pointers and sizes, returns an int status (0 = success) and
 * never throws, exits or synchronises the device unless its comment says so.  Buffers belong to
 * the caller; the library allocates one 256-byte status block per device on first use and
 * nothing else.  Kernels are enqueued on the stream that is passed in.
 *
 * The reference project has no FFI: its "API" is the templated host launchers inside each
 * program.  Each function below names the launcher it replaces (paths inside the reference).
 */
#ifndef CFK_B200_H_
#define CFK_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* cfk_stream_t; /* == cudaStream_t */

enum cfk_dtype { CFK_FP16 = 0, CFK_BF16 = 1, CFK_E4M3 = 2, CFK_FP32 = 3 };

enum cfk_status {
  CFK_OK = 0,
  CFK_ERR_INVALID_ARG = 1,   /* null pointer, non-positive size, misaligned pointer or stride */
  CFK_ERR_UNSUPPORTED = 2,   /* a shape / type combination no kernel was built for */
  CFK_ERR_DESCRIPTOR = 3,    /* the driver refused a TMA descriptor */
  CFK_ERR_LAUNCH = 4,        /* cudaFuncSetAttribute / launch failed; see cfk_last_cuda_error */
  CFK_ERR_NO_DRIVER = 5,     /* no CUDA driver / device */
  CFK_ERR_DEVICE_WAIT = 6,   /* a bounded wait inside a kernel gave up; see cfk_device_status */
  CFK_ERR_TOO_LARGE = 7      /* the call needs more scratch than a fixed-capacity entry point holds */
};

/*
 * Flash-attention forward:  O = softmax(Q K^T * softmax_scale [causal mask]) V.
 *
 * Replaces fmhaForwardDevice<PrecType,Gemm2Type,SoftType,OutputType,HEADDIM>(SEQLEN, KEYLEN,
 * NUMHEADS, BATCH, Q, K, V, S, O, miOut, sPrimeOut, iterations, scale, stream)
 * (src/fmha-pipeline/fmha_forward.cu:86-93) and the legacy fmhaForwardDevice<PrecType,AccumType,
 * HEADDIM> (src/fmha/fmha_forward.cu:425-430).  Differences a caller must know:
 *   - softmax_scale is the plain factor (e.g. 1/sqrt(D)); the reference passes it pre-multiplied
 *     by log2(e) (src/fmha-pipeline/fmha_forward.cu:452-454).  include/cfk_compat.hpp converts.
 *   - the S x S debug matrix of the reference (argument S) is not produced.
 *   - additions: causal flag, bf16, log-sum-exp output, per-tensor e4m3 de-scale factors,
 *     explicit strides.  Mixed operand formats in one MMA (fp16 P with bf16 V) are not possible:
 *     the hardware rejects them as an illegal instruction.
 * Tensors are [batch][seq][head][head_dim] with head_dim contiguous (the reference's layout,
 * fmha_forward.cu:151-152).  A stride of 0 means "packed".  Strides are in elements; every
 * stride times the element size must be a multiple of 16 bytes and every base pointer 16-byte
 * aligned.  head_dim must be 64, 128 or 256.  Accumulation and softmax are fp32.
 */
typedef struct cfk_fmha_args {
  int dtype;      /* cfk_dtype of Q, K and V: FP16, BF16 or E4M3 */
  int out_dtype;  /* cfk_dtype of O: FP16 or BF16 */
  int p_split_keys; /* P (unnormalised probabilities) is rounded to the input type before P*V, as the
                       reference does (fmha_consumer.h:54).  bf16 only: 256-row query blocks whose first
                       row sees fewer keys than this keep P as a two-term bf16 sum (hi + lo, two MMAs),
                       because with few keys bf16's 8-bit rounding of P is not averaged out.
                       -1 = default (1024), 0 = never.  Ignored for fp16 / e4m3. */
  int batch, heads, seqlen_q, seqlen_kv, head_dim;
  const void* q;
  const void* k;
  const void* v;
  void* o;
  float* lse;     /* optional, [batch][heads][seqlen_q]: ln(sum_j exp(scale * q.k_j)) */
  float* mi;      /* optional, reference's miOut: row maximum in the log2 domain */
  float* sprime;  /* optional, reference's sPrimeOut: sum_j 2^(x_j - mi), not inverted */
  int64_t q_stride[3]; /* batch, seq, head (elements); all 0 = packed */
  int64_t k_stride[3];
  int64_t v_stride[3];
  int64_t o_stride[3];
  float softmax_scale;
  int causal;     /* key j visible to query i iff j <= i + (seqlen_kv - seqlen_q) */
  float q_descale, k_descale, v_descale; /* multiply the stored values to get real ones; use 1 for 16-bit */
  int iterations; /* number of back-to-back launches (the reference's loop, fmha_forward.cu:375-382) */
  int v_fp16;     /* e4m3 inputs only: 1 = V is fp16 (strides in fp16 elements) and P is rounded to fp16, while Q and K
                     are e4m3: what the reference runs for --prec-type=2 unless it is built with GEMM2FP8
                     (src/fmha-pipeline/fmha_forward.cu:446-450).  Head dimensions 64 and 128.  0 = V has the type
                     of Q and K. */
  void* s_dump;   /* optional, debugging only: [batch][heads][seqlen_q][seqlen_kv], the reference's S of a COPYOUTMM0
                     build (fmha_consumer.h:31-42): Q K^T before the softmax scale and before masking, rounded to the
                     input type (fp16 for e4m3 inputs, in stored units).  Key tiles a causal mask skips are not
                     written.  Slows the kernel down. */
} cfk_fmha_args;

int cfk_fmha_forward(const cfk_fmha_args* args, cfk_stream_t stream);

/*
 * The same forward pass for callers that are not allowed to allocate device memory.  (This entry point
 * has no counterpart in the reference, whose launchers never allocate because they keep no device state.)
 *
 * cfk_fmha_forward obtains its 256-byte status block with cudaMalloc the first time a device is used,
 * which also synchronises the device.  That rules it out in a server that has given all of HBM to its
 * own pool (even 256 bytes can fail or fragment there), in latency-bound loops that cannot take the
 * device-wide synchronisation, and wherever allocation after start-up is forbidden.  This variant
 * runs the same kernels with that scratch in a fixed 256-byte array inside the library image (one copy
 * per GPU that loads the library, held until the process exits) and calls no allocating routine.
 *   - Arguments, checks, kernels and results are those of cfk_fmha_forward.
 *   - The first call on a device looks up the array's device address; make it before any capture starts.
 *   - The array is shared by all calls on a device and keeps the last call's contents; the status word is
 *     cleared on `stream` before the launches.  Calls whose kernels overlap on the GPU race on it.
 *   - A build whose kernels need more scratch than the array holds is refused with CFK_ERR_TOO_LARGE.
 *   - iterations == 0 launches nothing: it waits for `stream` and returns CFK_ERR_DEVICE_WAIT if the status
 *     word left by the preceding call is non-zero (cfk_device_status reads the allocated block only).
 *   - Because every call clears the word on entry, a wait that gave up inside call N is forgotten by call
 *     N + 1: a caller that wants to know puts an iterations == 0 query between the two (it synchronises
 *     `stream`).  A launch that finds the word set does nothing, so without the query the outputs of call N
 *     may be partly unwritten and nothing says so.
 */
int cfk_fmha_forward_static(const cfk_fmha_args* args, cfk_stream_t stream);

/*
 * GEMM:  C[m,n] = alpha * sum_k A[m,k] * B[n,k] + beta * C[m,n], fp32 accumulation, batched over L.
 *
 * Replaces gemm<TA,TB,TC,Alpha,Beta>(m, n, k, alpha, A, ldA, B, ldB, beta, C, ldC, A_out, B_out,
 * L, stream) (src/cute-gemm-tma-gma/gemm.cu:336-339).  A is M x K row-major, B is N x K row-major
 * (i.e. column-major K x N), both K-contiguous, as the reference builds them (gemm.cu:366-379); C is
 * column-major with leading dimension M by default (gemm.cu:388-389) or row-major with leading
 * dimension N.  Unlike the reference, alpha and beta are honoured and the accumulator is fp32.
 * K must be a multiple of 8 and M, N multiples of 8; pointers 16-byte aligned.
 */
typedef struct cfk_gemm_args {
  int dtype;      /* FP16 or BF16 for A, B and C; FP32: fp32 A, B and C with the products taken in tf32, the
                     reference's fp32 GEMM type (src/cute-gemm-tma-gma/gemm.cu:355-356, 677-678) */
  int m, n, k, l;
  const void* a;
  const void* b;
  void* c;
  float alpha, beta;
  int c_row_major; /* 0: column-major (reference), 1: row-major */
  int iterations;
  const void* c_src; /* optional: when non-null the beta term reads this matrix (layout of c) and c is only written,
                        D = alpha A B + beta C with separate C and D (src/cutlass-gemm/gemm.cu:316-323) */
} cfk_gemm_args;

int cfk_gemm(const cfk_gemm_args* args, cfk_stream_t stream);

/*
 * Device-side random fills, element i depends only on (seed, first_index + i).
 * Replaces cfk::initialize_rand / initialize_const (include/utils/random.hpp:20-50).
 * kind 0: N(0,1); kind 1: U[-1,1]; kind 2: constant `value`.  The result is value * scale
 * rounded to `dtype`.  kind 3: integers, U[-1,1] * scale rounded to nearest (the integer-valued operands of
 * src/cutlass-gemm/gemm.cu:268-293).
 */
int cfk_fill(void* dst, int dtype, int64_t n, uint64_t seed, int64_t first_index, int kind, float scale,
             float value, cfk_stream_t stream);

/* Element-wise conversion on the device between FP32 and any cfk_dtype (either side may be FP32). */
int cfk_convert(const void* src, int src_dtype, void* dst, int dst_dtype, int64_t n, float scale,
                cfk_stream_t stream);

/*
 * Reads (and clears) the status word of the current device.  Synchronises the device.
 * 0 = no kernel wait gave up; otherwise the code tells which wait did (1xx FMHA, 2xx GEMM).
 */
int cfk_device_status(int* code_out);

/* Text of the last CUDA runtime error seen by this library on the calling thread ("" if none). */
const char* cfk_last_cuda_error(void);

/*
 * Tuning knobs, process-wide; the defaults are the values measured best on B200 and a negative value
 * restores the default.  No counterpart in the reference, whose knobs are compile-time macros
 * (src/fmha-pipeline/shared_storage.h:3-32).
 *   CFK_TUNE_FMHA_EXP_EMU   0..3: of every four pairs of softmax exponentials, how many are evaluated
 *                           with a cubic on the FMA pipe instead of the special-function unit.  -1 (default):
 *                           by input type and head dimension, the measured best.
 *   CFK_TUNE_FMHA_GROUP_MB  causal only: heads are scheduled in groups whose K and V total at most
 *                           this many MiB (so they share L2), heaviest query blocks first.
 *   CFK_TUNE_FMHA_KERNEL    which FMHA kernel runs: 0 one CTA per 256 query rows (two 128-row tiles side by side);
 *                           1 pairs of CTAs (two SMs per 256 rows, tcgen05 cta_group::2; 16-bit inputs with head
 *                           dimension 128 only, other shapes run kernel 0); 2 a persistent grid whose CTAs take one
 *                           128-row tile at a time, with the scores double-buffered, both softmax warpgroups on the
 *                           two halves of the same key tile and a correction warpgroup (head dimensions 64 and 128).
 *   CFK_TUNE_FMHA_GRID      kernel 2: CTAs of the persistent grid; 0 = one per SM.  Never more than work items.
 *   CFK_TUNE_FMHA_SCHED     kernel 0 at head dimension 128: how the two query tiles of a CTA use tensor memory.
 *                           0: each has a score buffer and writes its probabilities over it; 1: they take turns on
 *                           one score buffer and keep their probabilities in buffers of their own, so that no
 *                           Q K^T waits for a P V; -1 (default): by input type, the measured best.
 */
enum cfk_tunable { CFK_TUNE_FMHA_EXP_EMU = 0, CFK_TUNE_FMHA_GROUP_MB = 1, CFK_TUNE_FMHA_KERNEL = 2, CFK_TUNE_FMHA_GRID = 3,
                   CFK_TUNE_FMHA_SCHED = 4, CFK_TUNE_COUNT = 5 };
int cfk_set_tunable(int which, int value);
int cfk_get_tunable(int which); /* -1 for an unknown knob */

/* Library version, e.g. 100 = 0.1.0. */
int cfk_version(void);

/*
 * Tensor-core ceiling probe: one CTA per SM issues `groups` x 4 tcgen05.mma 128 x 256 x (32 bytes of K) on random
 * operands resident in shared memory; *flops_out receives the floating-point operations of the launch, so that the
 * caller, timing the stream, gets the dense UMMA rate of `dtype` (FP16, BF16 or E4M3) at the clocks of its own run.
 * Used by bench.py for the e4m3 roofline denominator, for which no library GEMM figure exists.  No counterpart in
 * the reference.
 */
int cfk_umma_peak(int dtype, int groups, double* flops_out, cfk_stream_t stream);

/*
 * Failure-path self-test: launches one warp that waits, through the kernels' own bounded wait with a limit of
 * `limit_ms` (1..1000), on a barrier nothing arrives on.  The wait gives up and records code 901 in the status
 * word; cfk_device_status then returns CFK_ERR_DEVICE_WAIT with that code, and FMHA / GEMM launches enqueued
 * before the word is read do nothing.  Nothing traps or faults.  No counterpart in the reference, whose kernels
 * wait without a limit.
 */
int cfk_selftest_wait_gives_up(int limit_ms, cfk_stream_t stream);
/* The same wait, reporting into the fixed scratch array of cfk_fmha_forward_static instead of the allocated
 * status block (and allocating nothing): makes that entry point's status query return CFK_ERR_DEVICE_WAIT once,
 * so its failure path can be tested.  No counterpart in the reference. */
int cfk_selftest_wait_gives_up_static(int limit_ms, cfk_stream_t stream);

/*
 * Single-CTA UMMA self-test used by the GPU test-suite to prove each operand-descriptor form
 * (K-major / MN-major shared-memory operands, A from tensor memory, 16-bit and e4m3 kinds) against
 * a CPU product.  D[128][n] (fp32, row-major) = A[128][k] * B, where B is [n][k] (b_mn_major = 0)
 * or [k][n] (b_mn_major = 1).  k * elem_size must be 128; n is 64 or 128.  a_from_tmem routes A
 * through tensor memory.  a_fmt / b_fmt are cfk_dtype codes and must be equal: one MMA instruction
 * takes both operands in one format, and a mixed pair is refused with CFK_ERR_UNSUPPORTED before any
 * launch.  The descriptor fields of B are the ones the kernels use; the caller cannot override them.
 * No counterpart in the reference.
 */
int cfk_selftest_umma(const void* a, const void* b, float* d, int n, int a_fmt, int b_fmt, int b_mn_major,
                      int a_from_tmem, cfk_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* CFK_B200_H_ */
