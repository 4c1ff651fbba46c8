// Persistent one-tile-per-CTA FMHA forward instantiation: Q and K e4m3, V fp16 and P rounded to fp16, head dimension 64.
#include "fmha_launch_persist_impl.cuh"
namespace cfk {
int fmha_launch_persist_e4m3_f16_64(const FmhaLaunch& L) { return fmha_launch_persist_t<kDtE4M3, kDtF16, 64>(L); }
}  // namespace cfk
