// FMHA forward on CTA pairs: inputs fp16, P rounded to fp16, head dimension 128.
#include "fmha_launch_pair_impl.cuh"
namespace cfk {
int fmha_launch_pair_f16(const FmhaLaunch& L) { return fmha_launch_pair_t<kDtF16>(L); }
}  // namespace cfk
