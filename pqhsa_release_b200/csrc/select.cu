// Exact top-K selection among the scan's candidates (the reference runs aten
// topk over a materialised [H, G, N] score tensor:
// benchmarks/e2e_pq_param_sweep.py:212-217, :6642; here the scores never
// leave the chip except for the ~2K candidates per row).
//
// One CTA per query row.  The scan left one bit per (row, slot): the key's
// approximate logit reached the row's threshold.  The CTA turns the set bits into
// a candidate list in shared memory and scores the candidates again from their
// codes (bit-identical to the scan, a few thousand gathers that hit the L2 the
// scan just filled).  If at least K turned up, the K best of them ARE the K best
// of all N keys, and a block radix select picks them by (logit desc, slot asc).
// Otherwise - the threshold estimate was too high, probability ~1e-9 at the
// default margin - the same select runs over all N slots: slow, exact, and
// flagged in row_info.
//
// For every selected key the kernel then
//   * resolves the element offset of its K/V row in the (paged) cache, so the
//     attend kernel starts its gather from one dependent load, and
//   * removes the key from the approximate side of the softmax: exactly the
//     term the scan added for it is subtracted from its unit's exp-sum (a
//     selected tail slot has its stored logit set to -inf).  This is the
//     "- old_exact_exp" of pq_hsa/attention/sparse_attention.py:985-1009, done
//     per unit so that no cancellation error is left behind.
#include "common.cuh"
#include "radix_select.cuh"

namespace pqhsa {

constexpr int kFinThreads = 1024;
constexpr int kFinPer = 8;  // candidates per thread held in registers on the normal path
constexpr int kCandCap = 16384;  // candidates listed in shared memory; more than that selects from all keys
constexpr int kSlotBits = 22;    // a list entry is slot | list << 22

struct FinishArgs {
  const uint32_t* codes;
  const void* norms;
  const uint16_t* list_ids;
  const uint16_t* slot_unit;
  const int32_t* unit_off;
  const uint16_t* unit_list;
  const int32_t* slot_pos;
  const int32_t* state;
  const float* lut;
  const float* list_scores;
  int32_t* row_info;
  const uint32_t* hitmap;
  int32_t* sel_slot;
  long long* sel_off;
  const float* unit_max;
  float* unit_sum;
  float* tail_logit;
  KvAddr kv;
  int G, cap, ucap, tail_cap, kcap;
  double top_fraction;
  int topk_fixed;
};

template <typename E>
__global__ void __launch_bounds__(kFinThreads) finish_kernel(const FinishArgs a) {
  extern __shared__ uint32_t cslot[];  // [kCandCap] candidates as slot | list << kSlotBits, then their units
  uint16_t* cunit = reinterpret_cast<uint16_t*>(cslot + kCandCap);
  __shared__ float lut_s[kM * kC];
  __shared__ float lsc_s[kLMax];
  __shared__ RadixShared rsh;
  __shared__ RadixShared2 rsh2;
  __shared__ int emit_count;
  __shared__ int wtot[kFinThreads / 32];
  const int row = blockIdx.x, s = row / a.G;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int32_t* ri = a.row_info + (size_t)row * kRI;
  const int32_t* st = a.state + (size_t)s * kST;
  const int n_sorted = st[PQHSA_ST_N_SORTED], n_tail = st[PQHSA_ST_N_TAIL], n_units = st[PQHSA_ST_N_UNITS];
  const int N = n_sorted + n_tail;
  const int K = resolve_topk(N, a.top_fraction, a.topk_fixed);
  if (K <= 0) {
    if (threadIdx.x == 0) {
      ri[PQHSA_RI_K] = 0;
      ri[PQHSA_RI_N] = N;
      ri[PQHSA_RI_NCAND] = 0;
      ri[PQHSA_RI_NSEL] = 0;
      ri[PQHSA_RI_FALLBACK] = 0;
    }
    return;
  }
  const int req = st[PQHSA_ST_REQ], head = st[PQHSA_ST_KV_HEAD];
  const uint32_t* codes = a.codes + (size_t)s * a.cap;
  const E* norms = static_cast<const E*>(a.norms) + (size_t)s * a.cap;
  const uint16_t* lids = a.list_ids + (size_t)s * a.cap;
  const int32_t* uoff = a.unit_off + (size_t)s * (a.ucap + 1);
  const uint16_t* ulist = a.unit_list + (size_t)s * a.ucap;

  if (tid < kM * kC) lut_s[tid] = a.lut[(size_t)row * kM * kC + tid];
  if (tid < kLMax) lsc_s[tid] = a.list_scores[(size_t)row * kLMax + tid];
  if (tid == 0) emit_count = 0;

  // ---- the set bits of the row's hit words become a candidate list ----
  // A thread owns the words tid, tid + 1024, ...; the first kWords of them stay in registers together
  // with their units' first slot and list, requested in the same round trip.
  const uint32_t* hm = a.hitmap + (size_t)row * a.ucap * (kUnit / 32);
  const int nw = (n_units + (n_tail + kUnit - 1) / kUnit) * (kUnit / 32);
  constexpr int kWords = 8;
  uint32_t wbits[kWords];
  int wfirst[kWords];
  uint32_t wlist[kWords];
  int mine = 0;
#pragma unroll
  for (int j = 0; j < kWords; ++j) {
    const int w = tid + j * kFinThreads;
    wbits[j] = 0u;
    wfirst[j] = 0;
    wlist[j] = 0xFFFFu;
    if (w < nw) {
      const int u = w / (kUnit / 32), it = w % (kUnit / 32);
      wbits[j] = hm[w];
      if (u < n_units) {
        wfirst[j] = uoff[u] + it * 32;
        wlist[j] = ulist[u];
      } else {
        wfirst[j] = n_sorted + (u - n_units) * kUnit + it * 32;
      }
    }
  }
#pragma unroll
  for (int j = 0; j < kWords; ++j) mine += __popc(wbits[j]);
  for (int w = tid + kWords * kFinThreads; w < nw; w += kFinThreads) mine += __popc(hm[w]);
  int incl = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int v = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += v;
  }
  if (lane == 31) wtot[warp] = incl;
  __syncthreads();
  int before = 0, C = 0;
#pragma unroll
  for (int w = 0; w < kFinThreads / 32; ++w) {
    const int v = wtot[w];
    before += w < warp ? v : 0;
    C += v;
  }
  const int ncand = C;
  const bool fallback = C < K || C > kCandCap;
  if (!fallback) {
    int o = before + incl - mine;
    auto expand = [&](uint32_t bits, int first, uint32_t l, int u) {
      while (bits) {
        const int slot = first + __ffs((int)bits) - 1;
        bits &= bits - 1u;
        cslot[o] = (uint32_t)slot | ((l != 0xFFFFu ? l : (uint32_t)lids[slot]) << kSlotBits);
        cunit[o] = (uint16_t)u;
        ++o;
      }
    };
#pragma unroll
    for (int j = 0; j < kWords; ++j) expand(wbits[j], wfirst[j], wlist[j], (tid + j * kFinThreads) / (kUnit / 32));
    for (int w = tid + kWords * kFinThreads; w < nw; w += kFinThreads) {
      const int u = w / (kUnit / 32), it = w % (kUnit / 32);
      const bool sorted = u < n_units;
      expand(hm[w], (sorted ? uoff[u] : n_sorted + (u - n_units) * kUnit) + it * 32, sorted ? (uint32_t)ulist[u] : 0xFFFFu, u);
    }
  } else {
    C = N;
  }
  __syncthreads();

  constexpr uint32_t kSlotMask = (1u << kSlotBits) - 1u;
  auto slot_of = [&](int i) -> int { return fallback ? i : (int)(cslot[i] & kSlotMask); };
  auto logit_of = [&](int i) -> float {
    const int slot = slot_of(i);
    const int l = fallback ? (int)lids[slot] : (int)(cslot[i] >> kSlotBits);
    return finish_logit(pq_sum_row(lut_s, __ldg(codes + slot)), lsc_s[l], to_f(norms[slot]));
  };
  auto key = [&](int i) -> uint32_t { return float_key(logit_of(i)); };
  int32_t* sel = a.sel_slot + (size_t)row * a.kcap;
  long long* soff = a.sel_off + (size_t)row * a.kcap;
  const bool take_all = K >= C;
  uint32_t T = 0u, T2 = 0u;
  int t = 0;
  bool regs_path = false;
  if (!fallback && C <= kFinThreads * kFinPer) {
    // normal path: the candidates sit in registers, kFinPer per thread
    uint32_t kreg[kFinPer];
    int sreg[kFinPer];
    // four candidates per thread at a time: their gathers (code, norm) travel together, then the arithmetic
#pragma unroll
    for (int j0 = 0; j0 < kFinPer; j0 += 4) {
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        kreg[j0 + jj] = 0u;
        sreg[j0 + jj] = 0;
      }
      if (j0 * kFinThreads >= C) continue;  // block-uniform: rounds past the list cost nothing
      uint32_t code[4], ent[4];
      float kn[4];
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const int i = (j0 + jj) * kFinThreads + tid;
        ent[jj] = i < C ? cslot[i] : 0xFFFFFFFFu;
        code[jj] = 0u;
        kn[jj] = 0.f;
        if (i < C) {
          sreg[j0 + jj] = (int)(ent[jj] & kSlotMask);
          code[jj] = __ldg(codes + sreg[j0 + jj]);
          kn[jj] = to_f(norms[sreg[j0 + jj]]);
        }
      }
#pragma unroll
      for (int jj = 0; jj < 4; ++jj)
        if (ent[jj] != 0xFFFFFFFFu)
          kreg[j0 + jj] = float_key(finish_logit(pq_sum_row(lut_s, code[jj]), lsc_s[ent[jj] >> kSlotBits], kn[jj]));
    }
    if (!take_all) {
      const int ties = block_radix_threshold_regs<kFinThreads, kFinPer>(kreg, K, rsh2, T, t);
      if (ties != t) {  // more keys tie at the K-th value than fit: lowest slots first
        auto tie_key = [&](int i) -> uint32_t { return key(i) == T ? ~(uint32_t)slot_of(i) : 0u; };
        int t2;
        block_radix_threshold<kFinThreads>(tie_key, C, t, rsh, T2, t2);
      }
    }
    // Emit: a taken key gets its place in the selection (one shared-memory atomic per warp), the
    // element offset of its K/V row, and leaves the approximate side of the softmax - its unit's
    // exp-sum loses exactly the term the scan added (a tail slot's stored logit becomes -inf).
    const size_t sb = (size_t)s * a.cap;
#pragma unroll
    for (int j0 = 0; j0 < kFinPer; j0 += 4) {
      if (j0 * kFinThreads >= C) break;  // block-uniform
      int o[4], pos[4], u[4];
      float um[4];
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const int j = j0 + jj;
        const uint32_t k = kreg[j];
        const bool take = k != 0u && (take_all || k > T || (k == T && ~(uint32_t)sreg[j] >= T2));
        const unsigned m = __ballot_sync(0xffffffffu, take);
        int base = 0;
        if (m != 0u && lane == 0) base = atomicAdd(&emit_count, __popc(m));
        base = __shfl_sync(0xffffffffu, base, 0) + __popc(m & ((1u << lane) - 1u));
        o[jj] = take && base < a.kcap ? base : -1;
        pos[jj] = 0;
        u[jj] = 0;
        um[jj] = 0.f;
        if (o[jj] >= 0) {
          pos[jj] = a.slot_pos[sb + sreg[j]];
          const int i = j * kFinThreads + tid;
          u[jj] = cunit[i];
          if (sreg[j] < n_sorted) um[jj] = a.unit_max[(size_t)row * a.ucap + u[jj]];
        }
      }
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const int j = j0 + jj;
        if (o[jj] < 0) continue;
        sel[o[jj]] = sreg[j];
        soff[o[jj]] = a.kv.offset(req, head, pos[jj]);
        if (sreg[j] < n_sorted)
          atomicAdd(a.unit_sum + (size_t)row * a.ucap + u[jj], -unit_term(key_float(kreg[j]), unit_ref(um[jj])));
        else
          a.tail_logit[(size_t)row * a.tail_cap + (sreg[j] - n_sorted)] = kNegInf;
      }
    }
    regs_path = true;
  } else {
    // all N keys (the threshold estimate failed) or an oversized candidate list: keys are
    // recomputed on every pass
    if (!take_all) {
      const int ties = block_radix_threshold<kFinThreads>(key, C, K, rsh, T, t);
      if (ties != t) {
        auto tie_key = [&](int i) -> uint32_t { return key(i) == T ? ~(uint32_t)slot_of(i) : 0u; };
        int t2;
        block_radix_threshold<kFinThreads>(tie_key, C, t, rsh, T2, t2);
      }
    }
    for (int i = tid; i < C; i += kFinThreads) {
      const uint32_t k = take_all ? 1u : key(i);
      const int slot = slot_of(i);
      if (take_all || k > T || (k == T && ~(uint32_t)slot >= T2)) {
        const int o = atomicAdd(&emit_count, 1);
        if (o < a.kcap) {
          sel[o] = slot;
          soff[o] = (long long)__float_as_uint(logit_of(i));
        }
      }
    }
  }
  __syncthreads();
  const int nsel = regs_path ? 0 : min(emit_count, a.kcap);  // the register path has finished its keys already
  // pass 2: four selected keys per thread at a time, every level of dependent loads issued
  // together: slot -> (position, unit) -> (cache offset, unit max) -> stores
  constexpr int kB = 4;
  const size_t sbase = (size_t)s * a.cap;
  for (int base = 0; base < nsel; base += kFinThreads * kB) {
    int slot[kB], pos[kB], u[kB];
    float x[kB], um[kB];
    bool ok[kB];
#pragma unroll
    for (int j = 0; j < kB; ++j) {
      const int o = base + j * kFinThreads + tid;
      ok[j] = o < nsel;
      slot[j] = ok[j] ? sel[o] : 0;
      x[j] = ok[j] ? __uint_as_float((uint32_t)soff[o]) : 0.f;
    }
#pragma unroll
    for (int j = 0; j < kB; ++j) {
      pos[j] = ok[j] ? a.slot_pos[sbase + slot[j]] : 0;
      u[j] = (ok[j] && slot[j] < n_sorted) ? a.slot_unit[sbase + slot[j]] : 0;
    }
#pragma unroll
    for (int j = 0; j < kB; ++j) um[j] = (ok[j] && slot[j] < n_sorted) ? a.unit_max[(size_t)row * a.ucap + u[j]] : 0.f;
#pragma unroll
    for (int j = 0; j < kB; ++j) {
      if (!ok[j]) continue;
      soff[base + j * kFinThreads + tid] = a.kv.offset(req, head, pos[j]);
      if (slot[j] < n_sorted)
        atomicAdd(a.unit_sum + (size_t)row * a.ucap + u[j], -unit_term(x[j], unit_ref(um[j])));
      else
        a.tail_logit[(size_t)row * a.tail_cap + (slot[j] - n_sorted)] = kNegInf;
    }
  }
  if (tid == 0) {
    ri[PQHSA_RI_K] = K;
    ri[PQHSA_RI_N] = N;
    ri[PQHSA_RI_NCAND] = ncand;
    ri[PQHSA_RI_NSEL] = emit_count;
    ri[PQHSA_RI_FALLBACK] = fallback ? 1 : 0;
  }
}

int launch_select(const pqhsa_params& p, const pqhsa_ws_layout& w, cudaStream_t st) {
  char* ws = static_cast<char*>(p.workspace);
  const int R = p.num_streams * p.group;
  FinishArgs a;
  a.codes = static_cast<const uint32_t*>(p.codes);
  a.norms = p.norms;
  a.list_ids = static_cast<const uint16_t*>(p.list_ids);
  a.slot_unit = static_cast<const uint16_t*>(p.slot_unit);
  a.slot_pos = static_cast<const int32_t*>(p.slot_pos);
  a.state = static_cast<const int32_t*>(p.state);
  a.lut = reinterpret_cast<const float*>(ws + w.lut);
  a.list_scores = reinterpret_cast<const float*>(ws + w.list_scores);
  a.row_info = reinterpret_cast<int32_t*>(ws + w.row_info);
  a.hitmap = reinterpret_cast<const uint32_t*>(ws + w.hitmap);
  a.unit_off = static_cast<const int32_t*>(p.unit_off);
  a.unit_list = static_cast<const uint16_t*>(p.unit_list);
  a.sel_slot = reinterpret_cast<int32_t*>(ws + w.sel_slot);
  a.sel_off = reinterpret_cast<long long*>(ws + w.sel_off);
  a.unit_max = reinterpret_cast<const float*>(ws + w.unit_max);
  a.unit_sum = reinterpret_cast<float*>(ws + w.unit_sum);
  a.tail_logit = reinterpret_cast<float*>(ws + w.tail_logit);
  a.kv = make_kvaddr(p);
  a.G = p.group;
  a.cap = p.slot_capacity;
  a.ucap = p.unit_capacity;
  a.tail_cap = w.tail_cap;
  a.kcap = w.kcap;
  a.top_fraction = p.top_fraction;
  a.topk_fixed = p.topk_fixed;
  const size_t smem = (size_t)kCandCap * (sizeof(uint32_t) + sizeof(uint16_t));
  PQHSA_DISPATCH_E(p.dtype, {
    auto kern = finish_kernel<E>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return check_launch("finish: shared memory opt-in");
    kern<<<R, kFinThreads, smem, st>>>(a);
  });
  return check_launch("finish");
}

}  // namespace pqhsa
