// Launch of one CTA-pair FMHA instantiation (included by the fmha_inst_pair_*.cu files only).
#pragma once
#include "fmha_fwd_pair_sm100.cuh"
#include "fmha_launch.h"
#include "host_util.h"

namespace cfk {

template <int DT, int EMU, bool DUMP = false>
int fmha_launch_pair_e(const FmhaLaunch& L) {
  using C = FmhaPairCfg<DT>;
  auto kern = fmha_fwd_pair_kernel<DT, EMU, DUMP>;
  static thread_local int attr_set_for_device = -1;
  int dev = 0;
  if (note_cuda(cudaGetDevice(&dev), "cudaGetDevice") != cudaSuccess) return CFK_ERR_NO_DRIVER;
  if (attr_set_for_device != dev) {
    if (note_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES),
                  "cudaFuncSetAttribute(fmha pair smem)") != cudaSuccess)
      return CFK_ERR_LAUNCH;
    attr_set_for_device = dev;
  }
  const long long items = (long long)L.p.nqblk * L.p.H * L.p.B;     // 256-row blocks, one per pair
  if (2 * items > 0x7fffffffLL) return CFK_ERR_UNSUPPORTED;
  const dim3 grid((unsigned)(2 * items), 1, 1);   // two CTAs (one cluster) per item
  for (int it = 0; it < L.iterations; ++it)
    kern<<<grid, C::NTHREADS, C::SMEM_BYTES, L.stream>>>(L.tm_q, L.tm_k_half, L.tm_v_half, L.tm_o, L.p);
  return note_cuda(cudaGetLastError(), "fmha pair launch") == cudaSuccess ? CFK_OK : CFK_ERR_LAUNCH;
}

template <int DT>
int fmha_launch_pair_t(const FmhaLaunch& L) {
  if (L.p.s_dump) return fmha_launch_pair_e<DT, 0, true>(L);   // debugging build: raw scores are written too
  switch (L.exp_emu) {
    case 0: return fmha_launch_pair_e<DT, 0>(L);
    case 1: return fmha_launch_pair_e<DT, 1>(L);
    case 2: return fmha_launch_pair_e<DT, 2>(L);
    default: return fmha_launch_pair_e<DT, 3>(L);
  }
}

}  // namespace cfk
