// Exact top-K selection from the scan's histogram and bin array, without the
// logits ever being stored (the reference materialises [H, G, N] fp16 scores and
// runs aten topk over them: benchmarks/e2e_pq_param_sweep.py:212-217, :6642).
//
//   threshold : per query row, walk the 4096-bin histogram from the top to the
//               bin b* where the count reaches K; bins above b* are selected
//               outright (fewer than K slots), b* itself is ambiguous.  Also
//               folds the per-unit maxima into the row's max approximate logit.
//   collect   : one pass over the uint16 bin array; compacts slots with
//               bin > b* into sel_slot and slots with bin == b* into cand_slot.
//   finish    : re-scores the candidates from their codes (bit-identical to the
//               scan) and takes the exact best K - #above by (logit desc, slot
//               asc) with a block radix select.
//
// Because logit -> bin is monotone, the result is exactly the K largest logits.
#include "common.cuh"
#include "radix_select.cuh"

namespace pqhsa {

constexpr int kThrThreads = 512;      // 8 bins per thread
constexpr int kColThreads = 512;      // 8 slots per thread
constexpr int kColSlots = kColThreads * 8;
constexpr int kFinThreads = 512;
constexpr int kFinCache = 8192;       // candidate keys cached in shared memory

__global__ void __launch_bounds__(kThrThreads) threshold_kernel(
    const uint32_t* __restrict__ hist, int32_t* __restrict__ row_info, const float* __restrict__ unit_max,
    const float* __restrict__ tail_logit, const int32_t* __restrict__ state, float* __restrict__ row_amax, int G,
    int ucap, int tail_cap) {
  __shared__ uint32_t wsum[kThrThreads / 32];
  __shared__ float wmax[kThrThreads / 32];
  const int row = blockIdx.x, s = row / G;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int32_t* ri = row_info + (size_t)row * kRI;
  const int K = ri[PQHSA_RI_K];

  // row max of the approximate logits
  {
    const int32_t* st = state + (size_t)s * kST;
    const int n_units = st[PQHSA_ST_N_UNITS], n_tail = st[PQHSA_ST_N_TAIL];
    float m = kNegInf;
    for (int u = tid; u < n_units; u += kThrThreads) m = fmaxf(m, unit_max[(size_t)row * ucap + u]);
    for (int t = tid; t < n_tail; t += kThrThreads) m = fmaxf(m, tail_logit[(size_t)row * tail_cap + t]);
    m = warp_max(m);
    if (lane == 0) wmax[warp] = m;
    __syncthreads();
    if (tid == 0) {
      float mm = wmax[0];
      for (int i = 1; i < kThrThreads / 32; ++i) mm = fmaxf(mm, wmax[i]);
      row_amax[row] = mm;
    }
  }
  if (K <= 0) return;  // uniform per block

  // thread j owns the 8 bins just below 4096 - 8j, i.e. ascending j walks down from the top
  const uint32_t* h = hist + (size_t)row * kBins;
  const int top = kBins - 8 * tid;  // bins top-1 ... top-8
  const uint4 lo4 = *reinterpret_cast<const uint4*>(h + top - 8);
  const uint4 hi4 = *reinterpret_cast<const uint4*>(h + top - 4);
  const uint32_t c[8] = {hi4.w, hi4.z, hi4.y, hi4.x, lo4.w, lo4.z, lo4.y, lo4.x};  // c[j] = count of bin top-1-j
  uint32_t sum = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) sum += c[j];
  uint32_t incl = sum;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t v = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += v;
  }
  if (lane == 31) wsum[warp] = incl;
  __syncthreads();
  uint32_t before = 0;
  for (int i = 0; i < warp; ++i) before += wsum[i];
  incl += before;
  const uint32_t excl = incl - sum;
  const uint32_t need = (uint32_t)K;
  if (excl < need && need <= incl) {
    uint32_t cum = excl;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (cum < need && need <= cum + c[j]) {
        ri[PQHSA_RI_THR_BIN] = top - 1 - j;
        ri[PQHSA_RI_ABOVE] = (int)cum;
      }
      cum += c[j];
    }
  }
}

__global__ void __launch_bounds__(kColThreads) collect_kernel(const uint16_t* __restrict__ bins,
                                                              int32_t* __restrict__ row_info,
                                                              int32_t* __restrict__ sel_slot,
                                                              int32_t* __restrict__ cand_slot, int cap, int kcap) {
  __shared__ uint32_t wtot[kColThreads / 32];
  __shared__ uint32_t base_sh[2];
  const int row = blockIdx.y;
  int32_t* ri = row_info + (size_t)row * kRI;
  const int n = ri[PQHSA_RI_N], K = ri[PQHSA_RI_K], thr = ri[PQHSA_RI_THR_BIN];
  const int cta0 = blockIdx.x * kColSlots;
  if (K <= 0 || cta0 >= n) return;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int base = cta0 + tid * 8;
  uint32_t b[8];
  if (base < n) {
    const uint4 v = *reinterpret_cast<const uint4*>(bins + (size_t)row * cap + base);
    b[0] = v.x & 0xffffu; b[1] = v.x >> 16; b[2] = v.y & 0xffffu; b[3] = v.y >> 16;
    b[4] = v.z & 0xffffu; b[5] = v.z >> 16; b[6] = v.w & 0xffffu; b[7] = v.w >> 16;
  }
  uint32_t sel_mask = 0, cand_mask = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    if (base + j < n) {
      if ((int)b[j] > thr) sel_mask |= 1u << j;
      else if ((int)b[j] == thr) cand_mask |= 1u << j;
    }
  }
  // packed counts: selected in the low half, candidates in the high half (8 * 512 < 65536)
  const uint32_t mine = (uint32_t)__popc(sel_mask) | ((uint32_t)__popc(cand_mask) << 16);
  uint32_t incl = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t v = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += v;
  }
  if (lane == 31) wtot[warp] = incl;
  __syncthreads();
  uint32_t before = 0, total = 0;
  for (int i = 0; i < kColThreads / 32; ++i) {
    if (i < warp) before += wtot[i];
    total += wtot[i];
  }
  if (tid == 0) {
    base_sh[0] = (total & 0xffffu) ? (uint32_t)atomicAdd(&ri[PQHSA_RI_NSEL], (int)(total & 0xffffu)) : 0u;
    base_sh[1] = (total >> 16) ? (uint32_t)atomicAdd(&ri[PQHSA_RI_NCAND], (int)(total >> 16)) : 0u;
  }
  __syncthreads();
  const uint32_t excl = before + incl - mine;
  uint32_t so = base_sh[0] + (excl & 0xffffu);
  uint32_t co = base_sh[1] + (excl >> 16);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    if (sel_mask & (1u << j)) {
      if (so < (uint32_t)kcap) sel_slot[(size_t)row * kcap + so] = base + j;
      ++so;
    } else if (cand_mask & (1u << j)) {
      cand_slot[(size_t)row * cap + co] = base + j;
      ++co;
    }
  }
}

struct FinishArgs {
  const uint32_t* codes;
  const void* norms;
  const uint16_t* list_ids;
  const float* lut;
  const float* list_scores;
  int32_t* row_info;
  int32_t* sel_slot;
  const int32_t* cand_slot;
  int G, cap, kcap;
};

template <typename E>
__global__ void __launch_bounds__(kFinThreads) finish_kernel(const FinishArgs a) {
  __shared__ float lut_s[kM * kC];
  __shared__ RadixShared rsh;
  __shared__ int emit_count;
  extern __shared__ uint32_t key_cache[];  // kFinCache keys
  const int row = blockIdx.x, s = row / a.G;
  const int tid = threadIdx.x;
  int32_t* ri = a.row_info + (size_t)row * kRI;
  const int K = ri[PQHSA_RI_K];
  if (K <= 0) return;
  const int above = ri[PQHSA_RI_ABOVE];
  const int C = ri[PQHSA_RI_NCAND];
  const int r = K - above;  // 1 <= r <= C by construction of the threshold bin
  int32_t* sel = a.sel_slot + (size_t)row * a.kcap;
  const int32_t* cand = a.cand_slot + (size_t)row * a.cap;
  if (r >= C) {  // the whole bin is taken
    for (int i = tid; i < C; i += kFinThreads)
      if (above + i < a.kcap) sel[above + i] = cand[i];
    if (tid == 0) ri[PQHSA_RI_NSEL] = above + C;
    return;
  }
  if (tid < kM * kC) lut_s[tid] = a.lut[(size_t)row * kM * kC + tid];
  if (tid == 0) emit_count = 0;
  __syncthreads();
  const uint32_t* codes = a.codes + (size_t)s * a.cap;
  const E* norms = static_cast<const E*>(a.norms) + (size_t)s * a.cap;
  const uint16_t* lids = a.list_ids + (size_t)s * a.cap;
  const float* lsc = a.list_scores + (size_t)row * kLMax;
  auto rescore = [&](int i) -> uint32_t {
    const int slot = cand[i];
    const float x = finish_logit(pq_sum_row(lut_s, __ldg(codes + slot)), __ldg(lsc + lids[slot]), to_f(norms[slot]));
    return float_key(x);
  };
  const bool cached = C <= kFinCache;
  if (cached) {
    for (int i = tid; i < C; i += kFinThreads) key_cache[i] = rescore(i);
    __syncthreads();
  }
  auto key = [&](int i) -> uint32_t { return cached ? key_cache[i] : rescore(i); };
  uint32_t T;
  int t;
  block_radix_threshold<kFinThreads>(key, C, r, rsh, T, t);
  // ties at T: take the t smallest slots
  auto tie_key = [&](int i) -> uint32_t { return key(i) == T ? ~(uint32_t)cand[i] : 0u; };
  uint32_t T2;
  int t2;
  block_radix_threshold<kFinThreads>(tie_key, C, t, rsh, T2, t2);
  for (int i = tid; i < C; i += kFinThreads) {
    const uint32_t k = key(i);
    if (k > T || (k == T && ~(uint32_t)cand[i] >= T2)) {
      const int o = above + atomicAdd(&emit_count, 1);
      if (o < a.kcap) sel[o] = cand[i];
    }
  }
  __syncthreads();
  if (tid == 0) ri[PQHSA_RI_NSEL] = above + emit_count;
}

int launch_select(const pqhsa_params& p, const pqhsa_ws_layout& w, cudaStream_t st) {
  char* ws = static_cast<char*>(p.workspace);
  const int R = p.num_streams * p.group;
  int32_t* row_info = reinterpret_cast<int32_t*>(ws + w.row_info);
  threshold_kernel<<<R, kThrThreads, 0, st>>>(
      reinterpret_cast<const uint32_t*>(ws + w.hist), row_info, reinterpret_cast<const float*>(ws + w.unit_max),
      reinterpret_cast<const float*>(ws + w.tail_logit), static_cast<const int32_t*>(p.state),
      reinterpret_cast<float*>(ws + w.row_amax), p.group, p.unit_capacity, w.tail_cap);
  if (int rc = check_launch("threshold")) return rc;
  if (p.max_slots > 0) {
    const dim3 grid((p.max_slots + kColSlots - 1) / kColSlots, R);
    collect_kernel<<<grid, kColThreads, 0, st>>>(reinterpret_cast<const uint16_t*>(ws + w.bins), row_info,
                                                 reinterpret_cast<int32_t*>(ws + w.sel_slot),
                                                 reinterpret_cast<int32_t*>(ws + w.cand_slot), p.slot_capacity,
                                                 w.kcap);
    if (int rc = check_launch("collect")) return rc;
  }
  FinishArgs a;
  a.codes = static_cast<const uint32_t*>(p.codes);
  a.norms = p.norms;
  a.list_ids = static_cast<const uint16_t*>(p.list_ids);
  a.lut = reinterpret_cast<const float*>(ws + w.lut);
  a.list_scores = reinterpret_cast<const float*>(ws + w.list_scores);
  a.row_info = row_info;
  a.sel_slot = reinterpret_cast<int32_t*>(ws + w.sel_slot);
  a.cand_slot = reinterpret_cast<const int32_t*>(ws + w.cand_slot);
  a.G = p.group;
  a.cap = p.slot_capacity;
  a.kcap = w.kcap;
  PQHSA_DISPATCH_E(p.dtype, finish_kernel<E><<<R, kFinThreads, kFinCache * sizeof(uint32_t), st>>>(a));
  return check_launch("finish");
}

}  // namespace pqhsa
