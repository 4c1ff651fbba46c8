// Chooses the FMHA instantiation for (input type, P type, head dimension); the reference does this
// with compile-time macros and a switch in main (src/fmha-pipeline/fmha_forward.cu:744-791).
#include "fmha_launch.h"
#include "host_util.h"

namespace cfk {

int fmha_dispatch(int dtype, int p_dtype, int head_dim, const FmhaLaunch& L) {
  if (head_dim == 256) {
    if (dtype == CFK_FP16 && p_dtype == CFK_FP16) return fmha_launch_hd256_f16(L);
    if (dtype == CFK_BF16 && p_dtype == CFK_BF16) return fmha_launch_hd256_bf16(L);
    if (dtype == CFK_E4M3 && p_dtype == CFK_E4M3) return fmha_launch_hd256_e4m3(L);
    return CFK_ERR_UNSUPPORTED;
  }
  if (L.variant == 2) {
    if (dtype == CFK_FP16 && p_dtype == CFK_FP16)
      return head_dim == 64 ? fmha_launch_persist_f16_f16_64(L) : fmha_launch_persist_f16_f16_128(L);
    if (dtype == CFK_BF16 && p_dtype == CFK_BF16)
      return head_dim == 64 ? fmha_launch_persist_bf16_bf16_64(L) : fmha_launch_persist_bf16_bf16_128(L);
    if (dtype == CFK_E4M3 && p_dtype == CFK_FP16)
      return head_dim == 64 ? fmha_launch_persist_e4m3_f16_64(L) : fmha_launch_persist_e4m3_f16_128(L);
    if (dtype == CFK_E4M3 && p_dtype == CFK_E4M3)
      return head_dim == 64 ? fmha_launch_persist_e4m3_e4m3_64(L) : fmha_launch_persist_e4m3_e4m3_128(L);
    return CFK_ERR_UNSUPPORTED;
  }
  if (L.variant == 1 && head_dim == 128 && dtype == p_dtype && (dtype == CFK_FP16 || dtype == CFK_BF16))
    return dtype == CFK_FP16 ? fmha_launch_pair_f16(L) : fmha_launch_pair_bf16(L);
  if (dtype == CFK_FP16 && p_dtype == CFK_FP16)
    return head_dim == 64 ? fmha_launch_f16_f16_64(L) : fmha_launch_f16_f16_128(L);
  if (dtype == CFK_BF16 && p_dtype == CFK_BF16)
    return head_dim == 64 ? fmha_launch_bf16_bf16_64(L) : fmha_launch_bf16_bf16_128(L);
  if (dtype == CFK_E4M3 && p_dtype == CFK_FP16)
    return head_dim == 64 ? fmha_launch_e4m3_f16_64(L) : head_dim == 128 ? fmha_launch_e4m3_f16_128(L) : CFK_ERR_UNSUPPORTED;
  if (dtype == CFK_E4M3 && p_dtype == CFK_E4M3)
    return head_dim == 64 ? fmha_launch_e4m3_e4m3_64(L) : head_dim == 128 ? fmha_launch_e4m3_e4m3_128(L) : CFK_ERR_UNSUPPORTED;
  return CFK_ERR_UNSUPPORTED;
}

}  // namespace cfk
