// FMHA forward instantiation: Q and K e4m3, V fp16 and P rounded to fp16 (the reference's FP8 mode without GEMM2FP8),
// head dimension 64.
#include "fmha_launch_impl.cuh"
namespace cfk {
int fmha_launch_e4m3_f16_64(const FmhaLaunch& L) { return fmha_launch_t<kDtE4M3, kDtF16, 64>(L); }
}  // namespace cfk
