// extern "C" entry points of libpqhsa_b200: validation, workspace layout and
// the launch sequences.  No allocation, no synchronisation, no exceptions.
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include "common.cuh"

namespace pqhsa {

static thread_local char g_err[512] = "";

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int check_launch(const char* what) {
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(PQHSA_E_CUDA, "%s: %s", what, cudaGetErrorString(e));
  return PQHSA_OK;
}

static int g_sm_count = 0;
int sm_count() {
  if (g_sm_count == 0) {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    g_sm_count = n;
  }
  return g_sm_count;
}

static inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

static int topk_capacity(const pqhsa_params* p) {
  long long k = p->topk_fixed > 0 ? p->topk_fixed : 0;
  if (p->top_fraction >= 0.0) k = (long long)((double)p->slot_capacity * p->top_fraction) + 8;
  if (k > p->slot_capacity) k = p->slot_capacity;
  if (k < 8) k = 8;
  return (int)align_up((size_t)k, 8);
}

void layout_of(const pqhsa_params* p, pqhsa_ws_layout* o) {
  memset(o, 0, sizeof(*o));
  const size_t S = (size_t)p->num_streams, G = (size_t)p->group, R = S * G;
  const size_t cap = (size_t)p->slot_capacity;
  o->kcap = topk_capacity(p);
  o->tail_cap = (int32_t)align_up((size_t)(p->tail_capacity > 0 ? p->tail_capacity : 8), 8);
  o->chunks = (int32_t)((p->max_full + o->kcap + kChunk - 1) / kChunk);
  // The selection of a row is done by one CTA when the candidates a row can reasonably have (about 1.7 K; allowed
  // for here: 2 K + 1024) fit the registers of its 1024 threads - 8 per thread (parts = 1) or 16 (parts = -1) -
  // whatever the number of rows: measured, one CTA per row beats the shared form even with 16 rows on 148 SMs.  A
  // still larger K is shared by `parts` CTAs (a power of two): enough of them to fill the GPU, and enough that a
  // part's candidate list (`seg` entries, a quarter more than an even share of the candidates) fits in shared memory.
  {
    const size_t ccap = cap < (size_t)2 * o->kcap + 2048 ? cap : (size_t)2 * o->kcap + 2048;
    const size_t want = (size_t)2 * o->kcap + 1024;
    int parts = want <= 8192 ? 1 : (want <= 16384 ? -1 : 2);
    if (parts == 2)
      while (parts < 16 && (R * parts < 296 || ccap * 5 / 4 > (size_t)parts * 8192)) parts *= 2;
    o->parts = parts;
    o->seg = parts < 2 ? 8 : (int32_t)align_up(ccap * 5 / (4 * (size_t)parts) + 32, 8);
  }
  const size_t nparts = o->parts < 2 ? 1 : (size_t)o->parts;
  const size_t nrec = R * nparts * (size_t)o->seg;
  size_t off = 0;
  auto take = [&](size_t bytes) {
    const size_t at = off;
    off = align_up(off + bytes, 256);
    return at;
  };
  o->lut = take(S * G * kM * kC * sizeof(float));
  o->list_scores = take(S * G * kLMax * sizeof(float));
  o->pair_tab = take(S * G * 1024 * sizeof(float));
  o->row_bin = take(R * 2 * sizeof(float));
  o->row_tau = take(R * sizeof(float));
  o->ticket = take(2 * S * sizeof(int32_t));
  o->norm_pend = take(S * sizeof(float));
  o->unit_max = take(R * (size_t)p->unit_capacity * sizeof(float));
  o->unit_sum = take(R * (size_t)p->unit_capacity * sizeof(float));
  o->tail_logit = take(R * (size_t)o->tail_cap * sizeof(float));
  o->row_info = take(R * kRI * sizeof(int32_t));
  o->hitmap = take(R * (size_t)p->unit_capacity * (kUnit / 32) * sizeof(uint32_t));
  o->cand_key = take(nrec * sizeof(uint32_t));
  o->cand_rec = take(nrec * 4 * sizeof(int32_t));
  o->cand_bin = take(nrec * sizeof(uint16_t));
  o->part_hist = take(R * nparts * (PQHSA_SELECT_BINS + 4) * sizeof(uint32_t));
  o->part_cnt = take(R * nparts * sizeof(int32_t));
  o->sel_slot = take(R * (size_t)o->kcap * sizeof(int32_t));
  o->sel_off = take(R * (size_t)o->kcap * sizeof(int64_t));
  o->partial = take(R * (size_t)(o->chunks + kBgParts) * kPartial * sizeof(float));
  o->row_ticket = take(R * sizeof(int32_t));
  o->work_counter = take(2 * sizeof(unsigned long long));
  o->combine_ticket = take(sizeof(int32_t));
  o->total_bytes = off;
}

int check_params(const pqhsa_params* p, bool need_ws, bool need_kv, bool need_io) {
  if (p == nullptr) return set_error(PQHSA_E_NULL, "params is null");
  if (p->abi_version != PQHSA_ABI_VERSION)
    return set_error(PQHSA_E_SHAPE, "abi_version %d, library speaks %d", p->abi_version, PQHSA_ABI_VERSION);
  if (p->dtype < PQHSA_F32 || p->dtype > PQHSA_F16) return set_error(PQHSA_E_DTYPE, "unknown dtype %d", p->dtype);
  if (p->head_dim != kD) return set_error(PQHSA_E_SHAPE, "head_dim must be %d, got %d", kD, p->head_dim);
  if (p->group != 1 && p->group != 2 && p->group != 4 && p->group != 8)
    return set_error(PQHSA_E_SHAPE, "group must be 1, 2, 4 or 8, got %d", p->group);
  if (p->num_streams <= 0) return set_error(PQHSA_E_SHAPE, "num_streams must be positive");
  if (p->num_lists <= 0 || p->num_lists > kLMax)
    return set_error(PQHSA_E_SHAPE, "num_lists must be in 1..%d, got %d", kLMax, p->num_lists);
  if (p->slot_capacity <= 0 || p->slot_capacity % 8 != 0)
    return set_error(PQHSA_E_SHAPE, "slot_capacity must be a positive multiple of 8, got %d", p->slot_capacity);
  if (p->slot_capacity > (1 << 22)) return set_error(PQHSA_E_SHAPE, "slot_capacity %d exceeds %d", p->slot_capacity, 1 << 22);
  if (p->unit_capacity < p->num_lists + p->slot_capacity / kUnit)
    return set_error(PQHSA_E_SHAPE, "unit_capacity %d < num_lists + slot_capacity/%d", p->unit_capacity, kUnit);
  if (p->unit_capacity > 65535) return set_error(PQHSA_E_SHAPE, "unit_capacity %d does not fit 16 bits", p->unit_capacity);
  if (p->max_slots < 0 || p->max_slots > p->slot_capacity)
    return set_error(PQHSA_E_SHAPE, "max_slots %d outside 0..slot_capacity", p->max_slots);
  if (p->sink_tokens < 0 || p->local_window < 0 || p->max_full < 0)
    return set_error(PQHSA_E_SHAPE, "sink_tokens, local_window and max_full must be non-negative");
  if (p->tail_capacity < 0 || p->tail_capacity > p->slot_capacity)
    return set_error(PQHSA_E_SHAPE, "tail_capacity %d outside 0..slot_capacity", p->tail_capacity);
  if (!p->codes || !p->norms || !p->list_ids || !p->slot_pos || !p->slot_unit || !p->unit_off || !p->unit_list ||
      !p->coarse || !p->codebooks || !p->vmeans || !p->state || !p->norm_max)
    return set_error(PQHSA_E_NULL, "an index pool pointer is null");
  if (need_kv) {
    if (!p->k_base || !p->v_base) return set_error(PQHSA_E_NULL, "k_base / v_base is null");
    if (p->block_table != nullptr && (p->block_size <= 0 || p->max_blocks <= 0))
      return set_error(PQHSA_E_SHAPE, "paged cache needs positive block_size and max_blocks");
    const int64_t row_align = p->dtype == PQHSA_F32 ? 4 : 8;
    if (p->stride_block % row_align || p->stride_head % row_align || p->stride_row % row_align)
      return set_error(PQHSA_E_SHAPE, "KV strides must keep rows 16-byte aligned");
    if (((uintptr_t)p->k_base | (uintptr_t)p->v_base) & 15)
      return set_error(PQHSA_E_SHAPE, "k_base / v_base must be 16-byte aligned");
  }
  if (p->peer_world > 1) {
    if (!p->peer_out || !p->peer_gather || !p->peer_seq)
      return set_error(PQHSA_E_NULL, "peer_out / peer_gather / peer_seq is null with peer_world > 1");
    if (p->peer_rank < 0 || p->peer_rank >= p->peer_world || p->peer_world > 32)
      return set_error(PQHSA_E_SHAPE, "peer_rank %d / peer_world %d out of range", p->peer_rank, p->peer_world);
    if (p->peer_wait_polls < 0) return set_error(PQHSA_E_SHAPE, "peer_wait_polls must be non-negative");
  }
  if (need_io) {
    if (!p->q || !p->out) return set_error(PQHSA_E_NULL, "q / out is null");
    if (((uintptr_t)p->q | (uintptr_t)p->out) & 15) return set_error(PQHSA_E_SHAPE, "q / out must be 16-byte aligned");
  }
  if (need_ws) {
    {
      pqhsa_ws_layout w;
      layout_of(p, &w);
      if (w.chunks + kBgParts > kD)
        return set_error(PQHSA_E_SHAPE, "%d partials per query row exceed %d: lower max_full or the top-k", w.chunks + kBgParts, kD);
    }
    if (!p->workspace) return set_error(PQHSA_E_WORKSPACE, "workspace is null");
    if ((uintptr_t)p->workspace & 255) return set_error(PQHSA_E_WORKSPACE, "workspace must be 256-byte aligned");
    pqhsa_ws_layout w;
    layout_of(p, &w);
    if (p->workspace_bytes < w.total_bytes)
      return set_error(PQHSA_E_WORKSPACE, "workspace has %zu bytes, %zu needed", p->workspace_bytes, w.total_bytes);
  }
  return PQHSA_OK;
}

}  // namespace pqhsa

using namespace pqhsa;

extern "C" {

int pqhsa_abi_version(void) { return PQHSA_ABI_VERSION; }

const char* pqhsa_last_error_string(void) { return g_err; }

size_t pqhsa_workspace_bytes(const pqhsa_params* p) {
  if (p == nullptr) return 0;
  pqhsa_ws_layout w;
  layout_of(p, &w);
  return w.total_bytes;
}

int pqhsa_workspace_layout(const pqhsa_params* p, pqhsa_ws_layout* out) {
  if (p == nullptr || out == nullptr) return set_error(PQHSA_E_NULL, "null argument");
  layout_of(p, out);
  return PQHSA_OK;
}

int pqhsa_lut_build(const pqhsa_params* p, void* stream) {
  if (int rc = check_params(p, true, false, false)) return rc;
  if (!p->q) return set_error(PQHSA_E_NULL, "q is null");
  pqhsa_ws_layout w;
  layout_of(p, &w);
  return launch_lut_build(*p, w, nullptr, (cudaStream_t)stream);
}

int pqhsa_scan_select(const pqhsa_params* p, void* stream) {
  if (int rc = check_params(p, true, true, false)) return rc;
  pqhsa_ws_layout w;
  layout_of(p, &w);
  if (int rc = launch_scan(*p, w, nullptr, (cudaStream_t)stream)) return rc;
  return launch_select(*p, w, (cudaStream_t)stream);
}

int pqhsa_attend_merge(const pqhsa_params* p, void* stream) {
  if (int rc = check_params(p, true, true, true)) return rc;
  pqhsa_ws_layout w;
  layout_of(p, &w);
  if (int rc = launch_attend(*p, w, (cudaStream_t)stream)) return rc;
  return launch_merge(*p, w, (cudaStream_t)stream);
}

int pqhsa_decode_step(const pqhsa_params* p, void* stream) {
  if (int rc = check_params(p, true, true, true)) return rc;
  pqhsa_ws_layout w;
  layout_of(p, &w);
  cudaStream_t st = (cudaStream_t)stream;
  if (int rc = launch_lut_build(*p, w, nullptr, st)) return rc;
  if (int rc = launch_scan(*p, w, nullptr, st)) return rc;
  if (int rc = launch_select(*p, w, st)) return rc;
  if (int rc = launch_attend(*p, w, st)) return rc;
  return launch_merge(*p, w, st);
}

int pqhsa_decode_step_append(const pqhsa_params* p, const void* new_k, const void* new_v, const int32_t* enc_count,
                             int32_t uniform_count, void* stream) {
  if (int rc = check_params(p, true, true, true)) return rc;
  if ((new_k == nullptr) != (new_v == nullptr)) return set_error(PQHSA_E_NULL, "new_k and new_v go together");
  if (((uintptr_t)new_k | (uintptr_t)new_v) & 15) return set_error(PQHSA_E_SHAPE, "new_k / new_v must be 16-byte aligned");
  if (uniform_count < 0) return set_error(PQHSA_E_SHAPE, "uniform_count must be non-negative");
  const bool encode = enc_count != nullptr || uniform_count > 0;
  if (encode && (!p->vsum || !p->vcnt)) return set_error(PQHSA_E_NULL, "vsum / vcnt is null");
  pqhsa_ws_layout w;
  layout_of(p, &w);
  cudaStream_t st = (cudaStream_t)stream;
  StepAppend ap = {new_k, new_v, enc_count, uniform_count};
  if (new_k != nullptr && encode && p->local_window == 0) {
    // the key to encode may be the row written in this very step: keep the two in order
    if (int rc = launch_append_kv(*p, new_k, new_v, st)) return rc;
    if (int rc = launch_append_encode(*p, enc_count, uniform_count, st)) return rc;
    if (int rc = launch_lut_build(*p, w, nullptr, st)) return rc;
  } else {
    if (int rc = launch_lut_build(*p, w, &ap, st)) return rc;
  }
  if (int rc = launch_scan(*p, w, nullptr, st)) return rc;
  if (int rc = launch_select(*p, w, st)) return rc;
  if (int rc = launch_attend(*p, w, st)) return rc;
  return launch_merge(*p, w, st);
}

__global__ void __launch_bounds__(256) copy16_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src, size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) dst[i] = src[i];
}

int pqhsa_copy_small(void* dst, const void* src, size_t bytes, void* stream) {
  if (!dst || !src) return set_error(PQHSA_E_NULL, "dst / src is null");
  if ((bytes & 15) || (((uintptr_t)dst | (uintptr_t)src) & 15))
    return set_error(PQHSA_E_SHAPE, "pqhsa_copy_small needs 16-byte aligned pointers and a multiple of 16 bytes");
  if (bytes == 0) return PQHSA_OK;
  const size_t n = bytes / 16;
  const unsigned grid = (unsigned)((n + 255) / 256 < 1024 ? (n + 255) / 256 : 1024);
  copy16_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(static_cast<uint4*>(dst), static_cast<const uint4*>(src), n);
  return check_launch("copy_small");
}

__global__ void __launch_bounds__(32) empty_kernel() {}

int pqhsa_launch_empty(int32_t count, void* stream) {
  if (count < 0 || count > 64) return set_error(PQHSA_E_SHAPE, "count %d out of range", (int)count);
  for (int i = 0; i < count; ++i) empty_kernel<<<1, 32, 0, (cudaStream_t)stream>>>();
  return check_launch("launch_empty");
}

int pqhsa_wait_peers(const pqhsa_params* p, void* stream) {
  if (p == nullptr) return set_error(PQHSA_E_NULL, "params is null");
  if (p->peer_world <= 1) return PQHSA_OK;
  if (!p->peer_out || !p->peer_gather || !p->peer_seq)
    return set_error(PQHSA_E_NULL, "peer_out / peer_gather / peer_seq is null");
  if (p->num_streams <= 0 || (p->group != 1 && p->group != 2 && p->group != 4 && p->group != 8))
    return set_error(PQHSA_E_SHAPE, "num_streams %d / group %d out of range", p->num_streams, p->group);
  if (p->peer_rank < 0 || p->peer_rank >= p->peer_world || p->peer_world > 32)
    return set_error(PQHSA_E_SHAPE, "peer_rank %d / peer_world %d out of range", p->peer_rank, p->peer_world);
  return launch_wait_peers(*p, (cudaStream_t)stream);
}

int pqhsa_run_stage(const pqhsa_params* p, int stage, void* stream) {
  const bool kv = stage >= PQHSA_STAGE_SELECT;
  if (int rc = check_params(p, true, kv, stage >= PQHSA_STAGE_ATTEND)) return rc;
  if (stage == PQHSA_STAGE_LUT && !p->q) return set_error(PQHSA_E_NULL, "q is null");
  pqhsa_ws_layout w;
  layout_of(p, &w);
  cudaStream_t st = (cudaStream_t)stream;
  switch (stage) {
    case PQHSA_STAGE_LUT: return launch_lut_build(*p, w, nullptr, st);
    case PQHSA_STAGE_SCAN: return launch_scan(*p, w, nullptr, st);
    case PQHSA_STAGE_SELECT: return launch_select(*p, w, st);
    case PQHSA_STAGE_ATTEND: return launch_attend(*p, w, st);
    case PQHSA_STAGE_MERGE: return launch_merge(*p, w, st);
    default: return set_error(PQHSA_E_SHAPE, "unknown stage %d", stage);
  }
}

int pqhsa_compact(const pqhsa_params* p, int32_t* error, void* stream) {
  if (int rc = check_params(p, false, false, false)) return rc;
  if (!error) return set_error(PQHSA_E_NULL, "error flag is null");
  if (!p->slot_unit || !p->unit_off || !p->unit_list) return set_error(PQHSA_E_NULL, "unit arrays are null");
  return launch_compact(*p, error, (cudaStream_t)stream);
}

int pqhsa_append_kv(const pqhsa_params* p, const void* new_k, const void* new_v, void* stream) {
  if (int rc = check_params(p, false, true, false)) return rc;
  if (!new_k || !new_v) return set_error(PQHSA_E_NULL, "new_k / new_v is null");
  return launch_append_kv(*p, new_k, new_v, (cudaStream_t)stream);
}

int pqhsa_append_encode(const pqhsa_params* p, const int32_t* enc_count, int32_t uniform_count, void* stream) {
  if (int rc = check_params(p, false, true, false)) return rc;
  if (!p->vsum || !p->vcnt) return set_error(PQHSA_E_NULL, "vsum / vcnt is null");
  if (enc_count == nullptr && uniform_count < 0) return set_error(PQHSA_E_SHAPE, "uniform_count must be >= 0");
  if (enc_count == nullptr && uniform_count == 0) return PQHSA_OK;
  return launch_append_encode(*p, enc_count, uniform_count, (cudaStream_t)stream);
}

static int encode_bulk_checked(const void* keys, int64_t stream_stride, int32_t num_streams, int32_t n, int32_t dtype,
                               const void* coarse, int32_t num_lists, const void* codebooks, uint32_t* codes, void* norms,
                               uint16_t* list_ids, bool lists_given, void* stream) {
  if (!keys || !coarse || !codebooks || !codes || !norms || !list_ids) return set_error(PQHSA_E_NULL, "null argument");
  if (dtype < PQHSA_F32 || dtype > PQHSA_F16) return set_error(PQHSA_E_DTYPE, "unknown dtype %d", dtype);
  if (num_streams <= 0 || num_streams > 65535) return set_error(PQHSA_E_SHAPE, "num_streams must be in 1..65535");
  if (n < 0 || stream_stride < (int64_t)n * kD) return set_error(PQHSA_E_SHAPE, "need n >= 0 and stream_stride >= n * %d", kD);
  if (num_lists < 1 || num_lists > kLMax) return set_error(PQHSA_E_SHAPE, "num_lists must be in 1..%d, got %d", kLMax, num_lists);
  const int64_t esz = dtype == PQHSA_F32 ? 4 : 2;
  if (((uintptr_t)keys | (uintptr_t)coarse | (uintptr_t)codebooks) & 15 || (stream_stride * esz) & 15)
    return set_error(PQHSA_E_SHAPE, "keys, coarse and codebooks must be 16-byte aligned");
  if (n == 0) return PQHSA_OK;
  return launch_encode_bulk(keys, stream_stride, num_streams, n, dtype, coarse, num_lists, codebooks, codes, norms,
                            list_ids, lists_given, (cudaStream_t)stream);
}

int pqhsa_encode_bulk(const void* keys, int64_t stream_stride, int32_t num_streams, int32_t n, int32_t dtype,
                      const void* coarse, int32_t num_lists, const void* codebooks, uint32_t* codes, void* norms,
                      uint16_t* list_ids, void* stream) {
  return encode_bulk_checked(keys, stream_stride, num_streams, n, dtype, coarse, num_lists, codebooks, codes, norms,
                             list_ids, false, stream);
}

int pqhsa_encode_bulk_assigned(const void* keys, int64_t stream_stride, int32_t num_streams, int32_t n, int32_t dtype,
                               const void* coarse, int32_t num_lists, const void* codebooks, const uint16_t* list_ids,
                               uint32_t* codes, void* norms, void* stream) {
  return encode_bulk_checked(keys, stream_stride, num_streams, n, dtype, coarse, num_lists, codebooks, codes, norms,
                             const_cast<uint16_t*>(list_ids), true, stream);
}

int pqhsa_cluster_order(const uint16_t* ids, int32_t num_sets, int32_t n, int32_t k, int32_t* order, int32_t* start,
                        void* stream) {
  if (!ids || !order || !start) return set_error(PQHSA_E_NULL, "null argument");
  if (num_sets <= 0 || n < 0) return set_error(PQHSA_E_SHAPE, "need num_sets > 0 and n >= 0");
  if (k < 1 || k > kLMax) return set_error(PQHSA_E_SHAPE, "k must be in 1..%d, got %d", kLMax, k);
  return launch_cluster_order(ids, num_sets, n, k, order, start, (cudaStream_t)stream);
}

int pqhsa_cluster_sums(const void* rows, int32_t dtype, int64_t stream_stride, int32_t row_stride, int32_t width,
                       int32_t num_streams, int32_t groups, int32_t n, int32_t k, const int32_t* order,
                       const int32_t* start, float* sums, void* stream) {
  if (!rows || !order || !start || !sums) return set_error(PQHSA_E_NULL, "null argument");
  if (dtype < PQHSA_F32 || dtype > PQHSA_F16) return set_error(PQHSA_E_DTYPE, "unknown dtype %d", dtype);
  if (width < 1 || width > 128 || 128 % width) return set_error(PQHSA_E_SHAPE, "width must divide 128, got %d", width);
  if (num_streams <= 0 || groups <= 0 || (int64_t)num_streams * groups > 65535)
    return set_error(PQHSA_E_SHAPE, "need 1 <= num_streams * groups <= 65535");
  if (n < 0 || k < 1 || row_stride < groups * width || stream_stride < (int64_t)n * row_stride)
    return set_error(PQHSA_E_SHAPE, "need n >= 0, k >= 1, row_stride >= groups * width, stream_stride >= n * row_stride");
  return launch_cluster_sums(rows, dtype, stream_stride, row_stride, width, num_streams, groups, n, k, order, start, sums,
                             (cudaStream_t)stream);
}

int pqhsa_subspace_assign(const float* rows, int64_t stream_stride, const float* books, int32_t num_streams, int32_t n,
                          uint16_t* ids, void* stream) {
  if (!rows || !books || !ids) return set_error(PQHSA_E_NULL, "null argument");
  if (num_streams <= 0 || num_streams > 65535) return set_error(PQHSA_E_SHAPE, "num_streams must be in 1..65535");
  if (n < 0 || stream_stride < (int64_t)n * kD) return set_error(PQHSA_E_SHAPE, "need n >= 0 and stream_stride >= n * %d", kD);
  if (((uintptr_t)rows & 15) || (stream_stride & 3)) return set_error(PQHSA_E_SHAPE, "rows must be 16-byte aligned");
  if (n == 0) return PQHSA_OK;
  return launch_subspace_assign(rows, stream_stride, books, num_streams, n, ids, (cudaStream_t)stream);
}

int pqhsa_scan_scores(const pqhsa_params* p, float* scores, void* stream) {
  if (int rc = check_params(p, true, false, false)) return rc;
  if (!scores) return set_error(PQHSA_E_NULL, "scores is null");
  pqhsa_ws_layout w;
  layout_of(p, &w);
  return launch_scan(*p, w, scores, (cudaStream_t)stream);
}

int pqhsa_topk_radix(const float* scores, int32_t rows, int32_t n, int64_t row_stride, int32_t k, int32_t* out_idx,
                     float* out_val, void* stream) {
  if (!scores || !out_idx || !out_val) return set_error(PQHSA_E_NULL, "null argument");
  if (rows <= 0 || n < 0 || k < 0 || k > n || row_stride < n)
    return set_error(PQHSA_E_SHAPE, "need rows > 0, 0 <= k <= n <= row_stride");
  if (k == 0) return PQHSA_OK;
  return launch_topk(scores, rows, n, row_stride, k, out_idx, out_val, (cudaStream_t)stream);
}

}  // extern "C"
