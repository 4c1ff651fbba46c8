// FMHA forward on CTA pairs: inputs bf16, P rounded to bf16, head dimension 128.
#include "fmha_launch_pair_impl.cuh"
namespace cfk {
int fmha_launch_pair_bf16(const FmhaLaunch& L) { return fmha_launch_pair_t<kDtBF16>(L); }
}  // namespace cfk
