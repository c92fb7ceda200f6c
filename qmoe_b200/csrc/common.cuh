// Shared declarations of the sm_100a kernels behind the C ABI in include/qmoe_sub1.h.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#include <mutex>

#include "qmoe_sub1.h"

namespace qmoe {

// ---- error plumbing -------------------------------------------------------------------------
void set_error(const char *fmt, ...);
int cuda_fail(cudaError_t e, const char *what);

#define QMOE_CUDA(call)                                   \
  do {                                                    \
    cudaError_t e__ = (call);                             \
    if (e__ != cudaSuccess) return qmoe::cuda_fail(e__, #call); \
  } while (0)

#define QMOE_REQUIRE(cond, msg)                           \
  do {                                                    \
    if (!(cond)) {                                        \
      qmoe::set_error("%s: %s", __func__, msg);           \
      return QMOE_ERR_INVALID_ARG;                        \
    }                                                     \
  } while (0)

struct DeviceGuard {
  int prev = -1;
  bool ok = false;
  explicit DeviceGuard(int device) {
    if (cudaGetDevice(&prev) != cudaSuccess) return;
    if (prev != device && cudaSetDevice(device) != cudaSuccess) return;
    ok = true;
  }
  ~DeviceGuard() {
    if (ok && prev >= 0) cudaSetDevice(prev);
  }
};

int sm_count(int device);

// One mutex for every "first call on a device" set-up step of the library (kernel attributes, the
// SM count, the sticky status word): entry points may be called from several host threads.
std::mutex &setup_mutex();

// Sticky per-device status word of the tensor-core tile kernels: incremented (never cleared by a
// launch) whenever a bounded wait gave up.  Allocated and zeroed on first use; read and optionally
// reset through qmoe_moe_tile_timeouts().  nullptr if the allocation failed.
int *tile_status_word(int device);

// Event timing of the grouped launches (qmoe_profile_enable): returns true and four fresh events
// when the next grouped call should be timed.
bool profile_begin(int device, cudaEvent_t **events);

// Every kernel launch of the library goes through QMOE_LAUNCH so that qmoe_launch_count() is exact.
void count_launch();
#define QMOE_LAUNCH(kernel, grid, block, smem, stream, ...) \
  do {                                                      \
    kernel<<<grid, block, smem, stream>>>(__VA_ARGS__);     \
    qmoe::count_launch();                                   \
  } while (0)

// ---- derived decoder table -------------------------------------------------------------------
// The reference table `dec` (sub1.py:60-72) spends 8 bytes per code on a dense list of 2-bit
// digits.  Every entry of the standard dictionary has at most three non-zero digits, so the
// kernels use a 4-byte sparse form built once per device from `dec`:
//   byte 0   bits 0..3  length of the code in pairs (1..14; 0 in the null entry)
//            bits 4..6  bit 4+k set: the k-th non-zero is digit 2 (row max); clear: digit 1 (row min)
//            bit 7      the entry does not fit this form (more than three non-zeros or a malformed
//                       word) and is decoded from `dec` digit by digit instead
//   byte 1+k position (0..27) of the k-th non-zero inside the code, or 0x80 when there is none
constexpr uint32_t kEntryNull = 0x80808000u;   // covers nothing, contributes nothing
constexpr uint32_t kEntryDense = 0x80808080u;  // "decode me from dec"

struct SparseTable {
  const uint32_t *entries = nullptr;  // uint32[65536] on the device
  bool conforming = false;            // no entry needs the digit-by-digit path
};

// Returns the cached sparse table for (device, dec pointer), building it on `stream` on first use.
int get_sparse_table(const int32_t *dec_dev, int device, cudaStream_t stream, SparseTable *out);

}  // namespace qmoe
