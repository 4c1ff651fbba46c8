// Persistent one-tile-per-CTA FMHA forward instantiation: inputs bf16, P rounded to bf16, head dimension 64.
#include "fmha_launch_persist_impl.cuh"
namespace cfk {
int fmha_launch_persist_bf16_bf16_64(const FmhaLaunch& L) { return fmha_launch_persist_t<kDtBF16, kDtBF16, 64>(L); }
}  // namespace cfk
