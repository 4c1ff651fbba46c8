// cfk_fmha_forward_static: the FMHA forward for callers that must not allocate device memory.
//
// The ordinary entry point keeps its scratch (the status block that the kernels' bounded waits report
// into) in memory it obtains with cudaMalloc the first time a device is used, which also synchronises
// that device.  Some callers cannot afford either: serving loops that have handed all of HBM to their
// own pool (so even a 256-byte cudaMalloc can fail or fragment), latency-bound loops that cannot take a
// device-wide synchronisation, and hosts that forbid allocation after start-up.  For them the same kernels run here with the scratch
// in a fixed array that is part of the library image.  No counterpart in the reference.
#include <mutex>

#include "fmha_launch.h"
#include "host_util.h"

namespace cfk {

// The scratch itself: 256 bytes per GPU that loads the library, held until the process exits.  Word 0 is
// the status word; profiling builds keep their cycle counters in the words after it.  In host code this
// name is only a stand-in for the symbol, never a device address: the address comes from
// cudaGetSymbolAddress below.
constexpr int kStaticScratchInts = 64;
static __device__ __align__(256) int g_fmha_static_scratch[kStaticScratchInts];

// Scratch one call needs, in ints: the status block the kernels address through FmhaParams::status.
#ifdef CFK_FMHA_PROFILE
constexpr int kFmhaScratchInts = 8 + 2 * 12;   // status word, padding, twelve 64-bit cycle counters
#else
constexpr int kFmhaScratchInts = 1;
#endif

static std::mutex g_static_mu;
static int* g_static_addr[64] = {nullptr};

// Device address of the array on the current device; resolved once per device, with that device current.
// (Not static: the bounded-wait self-test can be pointed at this array, see cfk_selftest_wait_gives_up_static.)
int* static_scratch_for_current_device(int* err) {
  int dev = -1;
  if (note_cuda(cudaGetDevice(&dev), "cudaGetDevice") != cudaSuccess || dev < 0 || dev >= 64) {
    *err = CFK_ERR_NO_DRIVER;
    return nullptr;
  }
  std::lock_guard<std::mutex> lk(g_static_mu);
  if (!g_static_addr[dev]) {
    void* ptr = nullptr;
    if (note_cuda(cudaGetSymbolAddress(&ptr, g_fmha_static_scratch), "cudaGetSymbolAddress(static scratch)") !=
            cudaSuccess || !ptr) {
      *err = CFK_ERR_NO_DRIVER;
      return nullptr;
    }
    g_static_addr[dev] = static_cast<int*>(ptr);
  }
  return g_static_addr[dev];
}

}  // namespace cfk

using namespace cfk;

// Same arguments, checks, kernels and results as cfk_fmha_forward; differences:
//   * nothing is allocated: no cudaMalloc / cudaFree / allocating library call, here or in what it calls;
//   * the first call on a device resolves the address of the static array (cudaGetSymbolAddress); make
//     that first call before any stream capture begins;
//   * the array is shared by every call on that device and keeps the previous call's contents, so the
//     status word is cleared on `stream` before the launches; two calls whose kernels overlap on the GPU
//     (different streams) race on it and may hide or misattribute a wait that gave up;
//   * a call whose scratch need exceeds the array (kStaticScratchInts ints; only special builds need more
//     than one word) is refused with CFK_ERR_TOO_LARGE and nothing is launched;
//   * iterations == 0 launches nothing: it waits for `stream` and returns CFK_ERR_DEVICE_WAIT if the status
//     word left by the preceding call is non-zero (cfk_device_status only sees the allocated block).
extern "C" int cfk_fmha_forward_static(const cfk_fmha_args* a, cfk_stream_t stream) {
  FmhaLaunch L;
  int pdt = 0;
  const int rc = fmha_prepare(a, &L, &pdt);   // host-side only: checks, descriptors, parameters
  if (rc != CFK_OK) return rc;

  if (kFmhaScratchInts > kStaticScratchInts) {
    (void)note_cuda(cudaErrorInvalidValue, "cfk_fmha_forward_static: this build needs more scratch than the static "
                                          "array holds (kFmhaScratchInts > kStaticScratchInts)");
    return CFK_ERR_TOO_LARGE;
  }

  int err = CFK_OK;
  int* status = static_scratch_for_current_device(&err);
  if (!status) return err;
  const cudaStream_t st = (cudaStream_t)stream;

  if (a->iterations == 0) {   // query: what did the preceding call leave in the status word?
    if (note_cuda(cudaStreamSynchronize(st), "cudaStreamSynchronize") != cudaSuccess) return CFK_ERR_LAUNCH;
    int code = 0;
    if (note_cuda(cudaMemcpy(&code, status, sizeof(int), cudaMemcpyDeviceToHost), "cudaMemcpy(static status)") !=
        cudaSuccess)
      return CFK_ERR_LAUNCH;
    return code == 0 ? CFK_OK : CFK_ERR_DEVICE_WAIT;
  }

  L.p.status = status;
  L.stream = st;
  // The status word must start at zero: a launch that finds it set does nothing.
  if (note_cuda(cudaMemsetAsync(status, 0, sizeof(int) * kFmhaScratchInts, st), "cudaMemsetAsync(static status)") !=
      cudaSuccess)
    return CFK_ERR_LAUNCH;
  return fmha_dispatch(a->dtype, pdt, a->head_dim, L);
}
