// Host-side launch plumbing for the FMHA kernel family: what the reference does inside
// fmhaForwardDevice after it has built its layouts (kernel choice, shared-memory attribute, grid,
// `iterations` back-to-back launches: src/fmha-pipeline/fmha_forward.cu:294-382).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include "../../include/cfk_b200.h"
#include "fmha_params.h"

namespace cfk {

struct FmhaLaunch {
  CUtensorMap tm_q, tm_k, tm_v, tm_o;
  CUtensorMap tm_k_half, tm_v_half;   // CTA-pair kernel: boxes of 64 keys x all columns / 128 keys x one 64-column span
  int variant;                        // 0 one CTA per 256 query rows, 1 CTA pairs, 2 persistent, one tile per CTA (see cfk_b200.h)
  int grid_ctas;                      // variant 2: CTAs of the persistent grid (0 = one per SM)
  FmhaParams p;
  int iterations;
  int exp_emu;   // 0..3: share (in quarters) of the exponentials computed on the FMA pipe
  cudaStream_t stream;
};

// One function per built (input type, P type, head dim) combination; each lives in its own
// translation unit so the combinations compile in parallel.
int fmha_launch_f16_f16_64(const FmhaLaunch&);
int fmha_launch_f16_f16_128(const FmhaLaunch&);
int fmha_launch_bf16_bf16_64(const FmhaLaunch&);
int fmha_launch_bf16_bf16_128(const FmhaLaunch&);
int fmha_launch_e4m3_f16_64(const FmhaLaunch&);    // Q, K e4m3; V, P fp16
int fmha_launch_e4m3_f16_128(const FmhaLaunch&);
int fmha_launch_e4m3_e4m3_64(const FmhaLaunch&);
int fmha_launch_e4m3_e4m3_128(const FmhaLaunch&);
int fmha_launch_hd256_f16(const FmhaLaunch&);    // head dimension 256: tm_k / tm_v boxes are 128 keys x 128 columns,
int fmha_launch_hd256_bf16(const FmhaLaunch&);   // p.nqblk counts 128-row blocks
int fmha_launch_hd256_e4m3(const FmhaLaunch&);
int fmha_launch_persist_f16_f16_64(const FmhaLaunch&);    // variant 2: p.nqblk counts 128-row blocks
int fmha_launch_persist_f16_f16_128(const FmhaLaunch&);
int fmha_launch_persist_bf16_bf16_64(const FmhaLaunch&);
int fmha_launch_persist_bf16_bf16_128(const FmhaLaunch&);
int fmha_launch_persist_e4m3_f16_64(const FmhaLaunch&);
int fmha_launch_persist_e4m3_f16_128(const FmhaLaunch&);
int fmha_launch_persist_e4m3_e4m3_64(const FmhaLaunch&);
int fmha_launch_persist_e4m3_e4m3_128(const FmhaLaunch&);
int fmha_launch_pair_f16(const FmhaLaunch&);
int fmha_launch_pair_bf16(const FmhaLaunch&);

int fmha_dispatch(int dtype, int p_dtype, int head_dim, const FmhaLaunch& L);

// Checks the arguments of a call and fills the launch (descriptors, parameters, kernel choice) except for
// FmhaParams::status and the stream.  Returns a cfk status code.
int fmha_prepare(const struct ::cfk_fmha_args* a, FmhaLaunch* out, int* p_dtype);

}  // namespace cfk
