// Host-side helpers shared by the C-ABI translation units: TMA descriptor encoding through the
// driver entry point (no link-time libcuda dependency), the per-device status block, and error text.
// The reference builds its TMA descriptors with CuTe's make_tma_copy inside each launcher
// (src/fmha-pipeline/fmha_forward.cu:144-252, src/cute-gemm-tma-gma/gemm.cu:363-384).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/cfk_b200.h"

namespace cfk {

// Records the text of a CUDA runtime error for cfk_last_cuda_error(); returns its argument.
cudaError_t note_cuda(cudaError_t e, const char* what);

// Device pointer to the 256-byte status block of the current device (int[64]; word 0 is the status
// word the kernels write).  nullptr (and *err set) if there is no usable device.
int* device_status_block(int* err);

// Device address of the fixed scratch array that cfk_fmha_forward_static uses (fmha_static.cu); allocates nothing.
int* static_scratch_for_current_device(int* err);

inline int dtype_size(int dt) { return dt == CFK_E4M3 ? 1 : (dt == CFK_FP32 ? 4 : 2); }

// Generic tiled descriptor.  dims/box are innermost first; strides_bytes has rank-1 entries.
// Returns CFK_OK, CFK_ERR_NO_DRIVER or CFK_ERR_DESCRIPTOR.
int encode_tiled(CUtensorMap* map, int dtype, int rank, const void* base, const uint64_t* dims,
                 const uint64_t* strides_bytes, const uint32_t* box, int swizzle_bytes /* 128, 64 or 0 */);

// [batch][seq][head][d] tensor (element strides sb, ss, sh; d contiguous) seen as the 5-D tensor
// {128-byte span, seq, spans per row, head, batch}; a box is {span, box_rows, all spans, 1, 1}, so
// one copy lands in shared memory as [span][row][128 B] with the 128-byte swizzle applied.  Rows of 64 bytes
// (e4m3, d = 64) are a single 64-byte span with the 64-byte swizzle.
int encode_bshd(CUtensorMap* map, int dtype, const void* base, int batch, int seq, int heads, int d, int64_t sb,
                int64_t ss, int64_t sh, int box_rows, int box_spans = 0 /* 0 = all spans of a row */);

}  // namespace cfk
