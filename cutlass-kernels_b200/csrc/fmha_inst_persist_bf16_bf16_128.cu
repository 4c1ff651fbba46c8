// Persistent one-tile-per-CTA FMHA forward instantiation: inputs bf16, P rounded to bf16, head dimension 128.
#include "fmha_launch_persist_impl.cuh"
namespace cfk {
int fmha_launch_persist_bf16_bf16_128(const FmhaLaunch& L) { return fmha_launch_persist_t<kDtBF16, kDtBF16, 128>(L); }
}  // namespace cfk
