// pqhsa_scan_scores_static: approximate logits of every indexed key for a batch of
// query rows, for callers that may not allocate device memory.
//
// Who that is: an attention backend running inside an inference server is handed its
// query, its KV pages and a preallocated output by the server, which has already given
// every spare byte of the GPU to the KV cache; a cudaMalloc at that point can fail, or
// stall the whole process behind a device-wide synchronisation.  The same holds for a C
// host that only owns the buffers it was passed.  Such a caller cannot supply the scratch
// buffer that pqhsa_scan_scores needs for the per-query tables.
//
// Here the tables live in a fixed array inside the library image instead.  Nothing is
// allocated or freed; the price is a size limit (PQHSA_STATIC_MAX_ROWS query rows per
// call) and about 0.7 MB of device memory held by every GPU that loads the library until
// the process exits.
#include <string.h>

#include "common.cuh"

namespace pqhsa {

constexpr int kStaticMaxRows = PQHSA_STATIC_MAX_ROWS;
constexpr size_t align256(size_t v) { return (v + 255) / 256 * 256; }
// regions, in order: tables, list scores, histogram origin/width, threshold, arrival counters, row counters
constexpr size_t kOffLut = 0;
constexpr size_t kOffListScores = kOffLut + align256((size_t)kStaticMaxRows * kM * kC * sizeof(float));
constexpr size_t kOffRowBin = kOffListScores + align256((size_t)kStaticMaxRows * kLMax * sizeof(float));
constexpr size_t kOffRowTau = kOffRowBin + align256((size_t)kStaticMaxRows * 2 * sizeof(float));
constexpr size_t kOffTicket = kOffRowTau + align256((size_t)kStaticMaxRows * sizeof(float));
constexpr size_t kOffRowInfo = kOffTicket + align256((size_t)2 * kStaticMaxRows * sizeof(int32_t));  // int32 [S, 2], S <= rows
constexpr size_t kStaticBytes = kOffRowInfo + align256((size_t)kStaticMaxRows * kRI * sizeof(int32_t));

// The scratch itself.  In host code this name is only a handle for the runtime, not a device
// address: the address is asked for once per device below and that pointer is what the kernels get.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticBytes];

constexpr int kMaxDevices = 64;
static void* g_scratch_ptr[kMaxDevices] = {};

// Device address of the scratch on the current device (looked up on the first call per device).
static int static_scratch(void** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices)
    return set_error(PQHSA_E_CUDA, "cannot identify the current device");
  if (g_scratch_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess || ptr == nullptr)
      return set_error(PQHSA_E_CUDA, "cudaGetSymbolAddress(static scratch): %s", cudaGetErrorString(e));
    g_scratch_ptr[dev] = ptr;
  }
  *out = g_scratch_ptr[dev];
  return PQHSA_OK;
}

}  // namespace pqhsa

using namespace pqhsa;

extern "C" int pqhsa_scan_scores_static(const pqhsa_params* p, float* scores, void* stream) {
  if (int rc = check_params(p, false, false, false)) return rc;
  if (!p->q) return set_error(PQHSA_E_NULL, "q is null");
  if (!scores) return set_error(PQHSA_E_NULL, "scores is null");
  const long long rows = (long long)p->num_streams * p->group;
  if (rows > kStaticMaxRows)
    return set_error(PQHSA_E_CAPACITY,
                     "%lld query rows exceed the %d rows the built-in scratch holds: use pqhsa_scan_scores "
                     "with a caller-owned workspace",
                     rows, kStaticMaxRows);
  void* base = nullptr;
  if (int rc = static_scratch(&base)) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  // The table kernel keeps two arrival counters per stream, int32 [S, 2], that it expects at zero.  This
  // entry point appends and encodes nothing, so today's kernels never count on them; they are cleared
  // all the same, so that the call does not depend on what an earlier one left in the shared array.
  if (cudaMemsetAsync(static_cast<char*>(base) + kOffTicket, 0, (size_t)2 * p->num_streams * sizeof(int32_t), st) !=
      cudaSuccess)
    return check_launch("static scratch: clearing the arrival counters");
  pqhsa_params q = *p;
  q.workspace = base;
  q.workspace_bytes = kStaticBytes;
  pqhsa_ws_layout w;
  memset(&w, 0, sizeof(w));
  w.total_bytes = kStaticBytes;
  w.lut = kOffLut;
  w.pair_tab = (size_t)-1;  // only the full scan reads pair tables
  w.norm_pend = (size_t)-1;
  w.list_scores = kOffListScores;
  w.row_bin = (size_t)-1;  // ... and thresholds
  w.row_tau = kOffRowTau;
  w.ticket = kOffTicket;
  w.row_info = kOffRowInfo;
  if (int rc = launch_lut_build(q, w, nullptr, st)) return rc;
  return launch_scan(q, w, scores, st);
}
