// Launch of one instantiation of the persistent one-tile-per-CTA FMHA kernel (included by the fmha_inst_persist_*.cu
// files only).
#pragma once
#include "fmha_fwd_persist_sm100.cuh"
#include "fmha_launch.h"
#include "host_util.h"

namespace cfk {

template <int DT, int PT, int HD, int EMU, bool DUMP = false>
int fmha_launch_persist_e(const FmhaLaunch& L) {
  using C = FmhaPersistCfg<DT, PT, HD>;
  auto kern = fmha_fwd_persist_kernel<DT, PT, HD, EMU, DUMP>;
  static thread_local int attr_set_for_device = -1;
  static thread_local int sm_count = 0;
  int dev = 0;
  if (note_cuda(cudaGetDevice(&dev), "cudaGetDevice") != cudaSuccess) return CFK_ERR_NO_DRIVER;
  if (attr_set_for_device != dev) {
    if (note_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES),
                  "cudaFuncSetAttribute(fmha persist smem)") != cudaSuccess)
      return CFK_ERR_LAUNCH;
    if (note_cuda(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev),
                  "cudaDeviceGetAttribute(sm count)") != cudaSuccess || sm_count <= 0)
      return CFK_ERR_LAUNCH;
    attr_set_for_device = dev;
  }
  // Persistent grid: one CTA per SM (a CTA takes a whole SM's shared and tensor memory), or the number the caller
  // set; never more CTAs than work items.
  const long long items = (long long)L.p.nqblk * L.p.H * L.p.B;
  long long ctas = L.grid_ctas > 0 ? L.grid_ctas : sm_count;
  if (ctas > items) ctas = items;
  const dim3 grid((unsigned)ctas, 1, 1);
  for (int it = 0; it < L.iterations; ++it)
    kern<<<grid, C::NTHREADS, C::SMEM_BYTES, L.stream>>>(L.tm_q, L.tm_k, L.tm_v, L.tm_o, L.p);
  return note_cuda(cudaGetLastError(), "fmha persist launch") == cudaSuccess ? CFK_OK : CFK_ERR_LAUNCH;
}

template <int DT, int PT, int HD>
int fmha_launch_persist_t(const FmhaLaunch& L) {
  if (L.p.s_dump) return fmha_launch_persist_e<DT, PT, HD, 0, true>(L);   // debugging build: raw scores are written too
  switch (L.exp_emu) {
    case 0: return fmha_launch_persist_e<DT, PT, HD, 0>(L);
    case 1: return fmha_launch_persist_e<DT, PT, HD, 1>(L);
    case 2: return fmha_launch_persist_e<DT, PT, HD, 2>(L);
    default: return fmha_launch_persist_e<DT, PT, HD, 3>(L);
  }
}

}  // namespace cfk
