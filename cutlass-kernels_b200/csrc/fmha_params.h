// Kernel parameter block and status codes of the FMHA kernel family (host and device).
#pragma once

namespace cfk {

constexpr int kDtF16 = 0, kDtBF16 = 1, kDtE4M3 = 2;

// Where a bounded wait gave up (stored in the status word).
constexpr int kErrFmhaQFull = 101, kErrFmhaKvFull = 102, kErrFmhaKvEmpty = 103, kErrFmhaSFull = 104,
              kErrFmhaPFull = 105, kErrFmhaOFull = 106, kErrFmhaOStaged = 107, kErrFmhaSFree = 108,
              kErrFmhaPvDone = 109, kErrFmhaMaxPub = 110, kErrFmhaPvDone256 = 111, kErrFmhaRowMax = 112,
              kErrFmhaSRead = 113, kErrFmhaOFree = 115, kErrFmhaStats = 117, kErrFmhaCorrPv = 118;

struct FmhaParams {
  int B, H, Sq, Skv;
  int causal;        // key j visible to query i iff j <= i + (Skv - Sq)
  int out_bf16;      // output element type: 0 fp16, 1 bf16
  int nqblk;         // number of query blocks (256 rows each; 128 for the kernels with one query tile per CTA)
  int group;         // (batch, head) pairs scheduled side by side (their K and V share L2)
  int sched;         // d = 128: 1 = one S buffer shared by the two query tiles, P in buffers of its own; 0 = P over S
  int split_keys;    // bf16: CTAs whose first row sees fewer keys than this keep P as hi + lo (0 = never)
  float scale_log2;  // softmax_scale * log2(e) * q_descale * k_descale
  float out_scale;   // v_descale
  float* lse;        // optional [B][H][Sq]: natural-log sum of exp of the scaled scores
  float* mi;         // optional [B][H][Sq]: row maximum in the log2 domain
  float* sprime;     // optional [B][H][Sq]: sum of 2^(x - mi), not inverted
  void* s_dump;      // optional debug output [B][H][Sq][Skv]: raw Q K^T (16-bit); see cfk_b200.h
  int s_dump_bf16;   // element type of s_dump: 0 fp16, 1 bf16
  int* status;       // device status word
};

}  // namespace cfk
