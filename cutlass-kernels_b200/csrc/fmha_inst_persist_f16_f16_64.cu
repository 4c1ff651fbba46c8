// Persistent one-tile-per-CTA FMHA forward instantiation: inputs f16, P rounded to f16, head dimension 64.
#include "fmha_launch_persist_impl.cuh"
namespace cfk {
int fmha_launch_persist_f16_f16_64(const FmhaLaunch& L) { return fmha_launch_persist_t<kDtF16, kDtF16, 64>(L); }
}  // namespace cfk
