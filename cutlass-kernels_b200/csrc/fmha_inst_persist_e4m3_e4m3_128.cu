// Persistent one-tile-per-CTA FMHA forward instantiation: inputs e4m3, P rounded to e4m3, head dimension 128.
#include "fmha_launch_persist_impl.cuh"
namespace cfk {
int fmha_launch_persist_e4m3_e4m3_128(const FmhaLaunch& L) { return fmha_launch_persist_t<kDtE4M3, kDtE4M3, 128>(L); }
}  // namespace cfk
