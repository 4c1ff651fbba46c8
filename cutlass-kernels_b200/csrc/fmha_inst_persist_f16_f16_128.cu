// Persistent one-tile-per-CTA FMHA forward instantiation: inputs f16, P rounded to f16, head dimension 128.
#include "fmha_launch_persist_impl.cuh"
namespace cfk {
int fmha_launch_persist_f16_f16_128(const FmhaLaunch& L) { return fmha_launch_persist_t<kDtF16, kDtF16, 128>(L); }
}  // namespace cfk
