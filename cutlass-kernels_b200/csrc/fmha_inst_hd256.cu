// FMHA forward, head dimension 256, fp16, bf16 and e4m3 inputs (P rounded to the input type).
#include "fmha_fwd_hd256_sm100.cuh"
#include "fmha_launch.h"
#include "host_util.h"

namespace cfk {

template <int DT, int EMU, bool DUMP = false>
static int launch_hd256_e(const FmhaLaunch& L) {
  using C = FmhaHd256Cfg<DT>;
  auto kern = fmha_fwd_hd256_kernel<DT, EMU, DUMP>;
  static thread_local int attr_set_for_device = -1;
  int dev = 0;
  if (note_cuda(cudaGetDevice(&dev), "cudaGetDevice") != cudaSuccess) return CFK_ERR_NO_DRIVER;
  if (attr_set_for_device != dev) {
    if (note_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES),
                  "cudaFuncSetAttribute(fmha hd256 smem)") != cudaSuccess)
      return CFK_ERR_LAUNCH;
    attr_set_for_device = dev;
  }
  const dim3 grid((unsigned)((long long)L.p.nqblk * L.p.H * L.p.B), 1, 1);   // 128-row blocks
  for (int it = 0; it < L.iterations; ++it)
    kern<<<grid, C::NTHREADS, C::SMEM_BYTES, L.stream>>>(L.tm_q, L.tm_k, L.tm_v, L.tm_o, L.p);
  return note_cuda(cudaGetLastError(), "fmha hd256 launch") == cudaSuccess ? CFK_OK : CFK_ERR_LAUNCH;
}

template <int DT>
static int launch_hd256_t(const FmhaLaunch& L) {
  if (L.p.s_dump) return launch_hd256_e<DT, 0, true>(L);   // debugging build: raw scores are written too
  switch (L.exp_emu) {
    case 0: return launch_hd256_e<DT, 0>(L);
    case 1: return launch_hd256_e<DT, 1>(L);
    case 2: return launch_hd256_e<DT, 2>(L);
    default: return launch_hd256_e<DT, 3>(L);
  }
}

int fmha_launch_hd256_f16(const FmhaLaunch& L) { return launch_hd256_t<kDtF16>(L); }
int fmha_launch_hd256_bf16(const FmhaLaunch& L) { return launch_hd256_t<kDtBF16>(L); }
int fmha_launch_hd256_e4m3(const FmhaLaunch& L) { return launch_hd256_t<kDtE4M3>(L); }

}  // namespace cfk
