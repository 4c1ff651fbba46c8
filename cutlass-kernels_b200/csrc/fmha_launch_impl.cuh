// Launch of one FMHA kernel instantiation (included by the fmha_inst_*.cu files only).
#pragma once
#include "fmha_fwd_sm100.cuh"
#include "fmha_launch.h"
#include "host_util.h"

namespace cfk {

template <int DT, int PT, int HD, int EMU, bool DUMP = false>
int fmha_launch_e(const FmhaLaunch& L) {
  using C = FmhaCfg<DT, PT, HD>;
  auto kern = fmha_fwd_kernel<DT, PT, HD, EMU, DUMP>;
  static thread_local int attr_set_for_device = -1;
  int dev = 0;
  if (note_cuda(cudaGetDevice(&dev), "cudaGetDevice") != cudaSuccess) return CFK_ERR_NO_DRIVER;
  if (attr_set_for_device != dev) {
    if (note_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES),
                  "cudaFuncSetAttribute(fmha smem)") != cudaSuccess)
      return CFK_ERR_LAUNCH;
    attr_set_for_device = dev;
  }
  const dim3 grid((unsigned)((long long)L.p.nqblk * L.p.H * L.p.B), 1, 1);
  for (int it = 0; it < L.iterations; ++it) {
    kern<<<grid, C::NTHREADS, C::SMEM_BYTES, L.stream>>>(L.tm_q, L.tm_k, L.tm_v, L.tm_o, L.p);
  }
  return note_cuda(cudaGetLastError(), "fmha launch") == cudaSuccess ? CFK_OK : CFK_ERR_LAUNCH;
}

template <int DT, int PT, int HD>
int fmha_launch_t(const FmhaLaunch& L) {
  if (L.p.s_dump) return fmha_launch_e<DT, PT, HD, 0, true>(L);   // debugging build: raw scores are written too
  switch (L.exp_emu) {
    case 0: return fmha_launch_e<DT, PT, HD, 0>(L);
    case 1: return fmha_launch_e<DT, PT, HD, 1>(L);
    case 2: return fmha_launch_e<DT, PT, HD, 2>(L);
    default: return fmha_launch_e<DT, PT, HD, 3>(L);
  }
}

}  // namespace cfk
