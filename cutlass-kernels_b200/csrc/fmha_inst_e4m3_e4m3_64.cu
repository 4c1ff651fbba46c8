// FMHA forward instantiation: inputs e4m3, P rounded to e4m3, head dimension 64 (64-byte rows, 64-byte swizzle).
#include "fmha_launch_impl.cuh"
namespace cfk {
int fmha_launch_e4m3_e4m3_64(const FmhaLaunch& L) { return fmha_launch_t<kDtE4M3, kDtE4M3, 64>(L); }
}  // namespace cfk
