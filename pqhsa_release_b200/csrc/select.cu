// Exact top-K selection among the scan's candidates (the reference runs aten
// topk over a materialised [H, G, N] score tensor:
// benchmarks/e2e_pq_param_sweep.py:212-217, :6642; here the scores never
// leave the chip except for the ~2K candidates per row).
//
// The scan left one bit per (row, slot): the key's approximate logit reached the
// row's threshold tau.  The selection is two launches, each with `parts` CTAs per
// query row so that the GPU is full whatever the row count is; a CTA never waits
// for another one (the second launch starts when the first has ended).
//
// cand_kernel.  The hit words of a row are dealt out to its CTAs word by word.  A
// CTA turns its set bits into a candidate list in shared memory, scores the
// candidates again from their codes (bit-identical to the scan; a few thousand
// gathers that hit the L2 the scan just filled) and writes one record per
// candidate - logit key, slot, token position, the term the scan added to the
// unit's exp-sum for it, unit - plus a histogram of its candidates over
// PQHSA_SELECT_BINS linear bins between tau and an upper companion tau_hi placed by
// the threshold kernel (one more bin holds everything above).
//
// emit_kernel.  Every CTA of a row adds up the row's partial histograms and walks
// them from the top: the bin in which the count reaches K is the boundary bin.
// Candidates above it are selected outright; of the boundary bin's few members the
// best `need` are taken by (logit desc, slot asc) - by rank counting when there
// are at most 256 of them, by a block radix select otherwise.  A CTA emits the
// selected candidates of its own part: place in the selection, element offset of the
// K/V row in the (paged) cache, and removal from the approximate side of the
// softmax - exactly the term the scan added is subtracted from the unit's exp-sum
// (a selected tail slot has its stored logit set to -inf).  This is the
// "- old_exact_exp" of pq_hsa/attention/sparse_attention.py:985-1009, done per unit
// so that no cancellation error is left behind.
//
// If fewer than K candidates turned up (the threshold estimate was too high,
// probability ~1e-9 at the default margin), a part overflowed its list, or the
// boundary bin holds more than 2048 keys, the first CTA of the row selects from all
// N slots with a block radix select over recomputed logits: slow, exact, and
// flagged in row_info.
#include "common.cuh"
#include "radix_select.cuh"

namespace pqhsa {

constexpr int kSelThreads = 256;
constexpr int kSelBins = PQHSA_SELECT_BINS;
constexpr int kSelHist = kSelBins + 4;  // bins, the bin above them, padding to 16 bytes
constexpr int kBoundPer = 8;
constexpr int kBoundCap = kSelThreads * kBoundPer;  // boundary keys resolved in shared memory
constexpr int kSlotBits = 22;                       // a list entry is slot | list << 22
constexpr uint32_t kSlotMask = (1u << kSlotBits) - 1u;

struct SelectArgs {
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
  const float* row_bin;
  int32_t* row_info;
  const uint32_t* hitmap;
  uint32_t* cand_key;
  int32_t* cand_slot;
  int32_t* cand_pos;
  float* cand_term;
  uint16_t* cand_unit;
  uint32_t* part_hist;
  int32_t* part_cnt;
  int32_t* sel_slot;
  long long* sel_off;
  const float* unit_max;
  float* unit_sum;
  float* tail_logit;
  KvAddr kv;
  int G, cap, ucap, tail_cap, kcap, parts, seg;
  double top_fraction;
  int topk_fixed;
};

// bin of a candidate: linear in the logit between the row's threshold (lo) and its upper companion;
// kSelBins = above it.  inv_w == 0 (no range known) puts everything into bin 0.  Monotone in the logit.
__device__ __forceinline__ int cand_bin(float logit, float lo, float inv_w) {
  if (inv_w == 0.f) return 0;
  const float t = __fmul_rn(__fsub_rn(logit, lo), inv_w);
  int b = __float2int_rd(t);
  b = b < 0 ? 0 : b;
  return b > kSelBins ? kSelBins : b;
}

// The words of a row's hit map are dealt out so that word `it` of unit u goes to part (u + it) mod parts:
// full units spread their four words, units of a few slots (only word 0 populated) spread by unit.
__device__ __forceinline__ bool word_of_part(int u, int it, int part, int parts) { return ((u + it) & (parts - 1)) == part; }

template <typename E>
__global__ void __launch_bounds__(kSelThreads) cand_kernel(const SelectArgs a) {
  extern __shared__ __align__(16) unsigned char sel_smem[];
  uint32_t* cslot = reinterpret_cast<uint32_t*>(sel_smem);       // [seg] slot | list << kSlotBits
  uint16_t* cunit = reinterpret_cast<uint16_t*>(cslot + a.seg);  // [seg]
  __shared__ float lut_s[kM * kC];
  __shared__ float lsc_s[kLMax];
  __shared__ uint32_t hist[kSelHist];
  __shared__ int wtot[kSelThreads / 32];
  const int P = a.parts;
  const int row = blockIdx.x / P, part = blockIdx.x % P, s = row / a.G;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int32_t* st = a.state + (size_t)s * kST;
  const int n_sorted = st[PQHSA_ST_N_SORTED], n_tail = st[PQHSA_ST_N_TAIL], n_units = st[PQHSA_ST_N_UNITS];
  const int N = n_sorted + n_tail;
  const int K = resolve_topk(N, a.top_fraction, a.topk_fixed);
  int32_t* pcnt = a.part_cnt + (size_t)row * P + part;
  if (K <= 0) {
    if (tid == 0) *pcnt = 0;
    return;
  }
  const uint32_t* codes = a.codes + (size_t)s * a.cap;
  const E* norms = static_cast<const E*>(a.norms) + (size_t)s * a.cap;
  const uint16_t* lids = a.list_ids + (size_t)s * a.cap;
  const int32_t* spos = a.slot_pos + (size_t)s * a.cap;
  const int32_t* uoff = a.unit_off + (size_t)s * (a.ucap + 1);
  const uint16_t* ulist = a.unit_list + (size_t)s * a.ucap;
  const float* umax = a.unit_max + (size_t)row * a.ucap;
  const uint32_t* hm = a.hitmap + (size_t)row * a.ucap * (kUnit / 32);
  const float lo = a.row_bin[2 * row], inv_w = a.row_bin[2 * row + 1];

  if (tid < kM * kC) lut_s[tid] = a.lut[(size_t)row * kM * kC + tid];
  for (int i = tid; i < kLMax; i += kSelThreads) lsc_s[i] = a.list_scores[(size_t)row * kLMax + i];
  for (int i = tid; i < kSelHist; i += kSelThreads) hist[i] = 0u;

  // ---- pass 1: how many candidates this thread's words hold ----
  const int n_all = n_units + (n_tail + kUnit - 1) / kUnit;  // sorted units, then 128-slot chunks of the tail
  int mine = 0;
  for (int u = tid; u < n_all; u += kSelThreads) {
#pragma unroll
    for (int it = 0; it < kUnit / 32; ++it)
      if (word_of_part(u, it, part, P)) mine += __popc(__ldg(hm + (size_t)u * (kUnit / 32) + it));
  }
  int incl = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int v = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += v;
  }
  if (lane == 31) wtot[warp] = incl;
  __syncthreads();  // also: tables, list scores and the cleared histogram are in place
  int before = 0, C = 0;
#pragma unroll
  for (int w = 0; w < kSelThreads / 32; ++w) {
    const int v = wtot[w];
    before += w < warp ? v : 0;
    C += v;
  }
  if (C > a.seg) {  // more candidates than this part can list: the row is selected from all keys
    if (tid == 0) *pcnt = C;
    return;
  }
  // ---- pass 2: the set bits become list entries (the words are read again: L1 / L2 hits) ----
  {
    int o = before + incl - mine;
    for (int u = tid; u < n_all; u += kSelThreads) {
      const bool sorted = u < n_units;
      int first0 = 0;
      uint32_t l = 0xFFFFu;
      bool have = false;
#pragma unroll
      for (int it = 0; it < kUnit / 32; ++it) {
        if (!word_of_part(u, it, part, P)) continue;
        uint32_t bits = __ldg(hm + (size_t)u * (kUnit / 32) + it);
        if (bits == 0u) continue;
        if (!have) {
          have = true;
          if (sorted) {
            first0 = uoff[u];
            l = ulist[u];
          } else {
            first0 = n_sorted + (u - n_units) * kUnit;
          }
        }
        while (bits) {
          const int slot = first0 + it * 32 + __ffs((int)bits) - 1;
          bits &= bits - 1u;
          cslot[o] = (uint32_t)slot | ((sorted ? l : (uint32_t)lids[slot]) << kSlotBits);
          cunit[o] = (uint16_t)u;
          ++o;
        }
      }
    }
  }
  __syncthreads();

  // ---- the candidates are scored again, four per thread at a time: their gathers travel together ----
  const size_t rec0 = ((size_t)row * P + part) * a.seg;
  for (int i0 = 0; i0 < C; i0 += 4 * kSelThreads) {
    uint32_t ent[4], code[4];
    float kn[4], um[4];
    int pos[4], un[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int i = i0 + j * kSelThreads + tid;
      ent[j] = i < C ? cslot[i] : 0xFFFFFFFFu;
      code[j] = 0u;
      kn[j] = 0.f;
      um[j] = 0.f;
      pos[j] = 0;
      un[j] = 0;
      if (i < C) {
        const int slot = (int)(ent[j] & kSlotMask);
        un[j] = cunit[i];
        code[j] = __ldg(codes + slot);
        kn[j] = to_f(norms[slot]);
        pos[j] = spos[slot];
        if (slot < n_sorted) um[j] = umax[un[j]];
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int i = i0 + j * kSelThreads + tid;
      if (i >= C) continue;
      const int slot = (int)(ent[j] & kSlotMask);
      const float x = finish_logit(pq_sum_row(lut_s, code[j]), lsc_s[ent[j] >> kSlotBits], kn[j]);
      atomicAdd(&hist[cand_bin(x, lo, inv_w)], 1u);
      a.cand_key[rec0 + i] = float_key(x);
      a.cand_slot[rec0 + i] = slot;
      a.cand_pos[rec0 + i] = pos[j];
      a.cand_term[rec0 + i] = slot < n_sorted ? unit_term(x, unit_ref(um[j])) : 0.f;
      a.cand_unit[rec0 + i] = (uint16_t)un[j];
    }
  }
  __syncthreads();
  uint32_t* ph = a.part_hist + ((size_t)row * P + part) * kSelHist;
  for (int i = tid; i < kSelHist; i += kSelThreads) ph[i] = hist[i];
  if (tid == 0) *pcnt = C;
}

struct EmitShared {
  int bstar, above, nb;  // boundary bin, candidates in the bins above it, candidates in it
  int total, overflow;
  int top;               // candidates in the bin above the linear ones
  int bcount;            // boundary keys collected so far
  int emit_count;        // this CTA's selected candidates placed so far
  int base_above;        // selected candidates above the boundary in the parts before this one
  int base_bound;        // taken boundary keys in the parts before this one (radix path)
  uint32_t wsum[kSelThreads / 32];
};

template <typename E>
__global__ void __launch_bounds__(kSelThreads) emit_kernel(const SelectArgs a) {
  extern __shared__ __align__(16) unsigned char sel_smem[];
  uint32_t* bkey = reinterpret_cast<uint32_t*>(sel_smem);  // [kBoundCap] boundary keys: logit key,
  uint32_t* bslot = bkey + kBoundCap;                      //   slot,
  uint32_t* bref = bslot + kBoundCap;                      //   part << 24 | index in the part's list
  __shared__ RadixShared rsh;
  __shared__ RadixShared2 rsh2;
  __shared__ EmitShared es;
  __shared__ float lut_s[kM * kC];
  __shared__ float lsc_s[kLMax];
  const int P = a.parts;
  const int row = blockIdx.x / P, part = blockIdx.x % P, s = row / a.G;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int32_t* ri = a.row_info + (size_t)row * kRI;
  const int32_t* st = a.state + (size_t)s * kST;
  const int n_sorted = st[PQHSA_ST_N_SORTED], n_tail = st[PQHSA_ST_N_TAIL];
  const int N = n_sorted + n_tail;
  const int K = resolve_topk(N, a.top_fraction, a.topk_fixed);
  if (K <= 0) {
    if (part == 0 && tid == 0) {
      ri[PQHSA_RI_K] = 0;
      ri[PQHSA_RI_N] = N;
      ri[PQHSA_RI_NCAND] = 0;
      ri[PQHSA_RI_NSEL] = 0;
      ri[PQHSA_RI_FALLBACK] = 0;
    }
    return;
  }
  const int req = st[PQHSA_ST_REQ], head = st[PQHSA_ST_KV_HEAD];
  const float lo = a.row_bin[2 * row], inv_w = a.row_bin[2 * row + 1];
  const uint32_t* ph = a.part_hist + (size_t)row * P * kSelHist;
  const int32_t* pc = a.part_cnt + (size_t)row * P;
  int32_t* sel = a.sel_slot + (size_t)row * a.kcap;
  long long* soff = a.sel_off + (size_t)row * a.kcap;
  float* usum = a.unit_sum + (size_t)row * a.ucap;
  float* tlog = a.tail_logit + (size_t)row * a.tail_cap;

  // ---- the row's histogram, walked from the top ----
  // thread t owns the bins 4 (255 - t) .. 4 (255 - t) + 3, highest first, so that ascending t descends
  const int b0 = 4 * (kSelThreads - 1 - tid);
  uint32_t c[4] = {0u, 0u, 0u, 0u};
  if (tid == 0) {
    es.bstar = -2;
    es.above = 0;
    es.nb = 0;
    es.bcount = 0;
    es.emit_count = 0;
    es.base_above = 0;
    es.base_bound = 0;
  }
  if (warp == 0) {
    int cnt = 0, top = 0;
    if (lane < P) {
      cnt = pc[lane];
      top = (int)ph[(size_t)lane * kSelHist + kSelBins];
    }
    const int over = __any_sync(0xffffffffu, cnt > a.seg);
    const int tot = __reduce_add_sync(0xffffffffu, cnt);
    const int tops = __reduce_add_sync(0xffffffffu, over ? 0 : top);
    if (lane == 0) {
      es.total = tot;
      es.overflow = over;
      es.top = tops;
    }
  }
  __syncthreads();
  const int C = es.total;
  bool fallback = es.overflow != 0 || C < K;
  if (!fallback) {
    for (int pp = 0; pp < P; ++pp) {
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(ph + (size_t)pp * kSelHist + b0));
      c[3] += v.x;  // c[0] is the highest of the four bins
      c[2] += v.y;
      c[1] += v.z;
      c[0] += v.w;
    }
    const uint32_t sum = c[0] + c[1] + c[2] + c[3];
    uint32_t incl = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    if (lane == 31) es.wsum[warp] = incl;
    __syncthreads();
    uint32_t before = (uint32_t)es.top;
    for (int w = 0; w < warp; ++w) before += es.wsum[w];
    incl += before;
    const uint32_t excl = incl - sum, need = (uint32_t)K;
    if (tid == 0 && (uint32_t)es.top >= need) {
      es.bstar = kSelBins;
      es.above = 0;
      es.nb = es.top;
    }
    if (excl < need && need <= incl) {
      uint32_t cum = excl;
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        if (cum < need && need <= cum + c[b]) {
          es.bstar = b0 + 3 - b;
          es.above = (int)cum;
          es.nb = (int)c[b];
        }
        cum += c[b];
      }
    }
    __syncthreads();
  }
  int bstar = es.bstar, above = es.above, nb = es.nb;
  int need = K - above;  // boundary keys to take, 1 .. nb
  if (!fallback && need == nb) {
    // the whole boundary bin is taken: nothing to resolve
    bstar -= 1;
    above += nb;
    need = 0;
    nb = 0;
  }
  if (!fallback && nb > kBoundCap) fallback = true;

  // one selected candidate of this part: its place in the selection, the offset of its K/V row, and its
  // removal from the approximate side of the softmax
  const size_t rec0 = ((size_t)row * P + part) * a.seg;
  auto emit = [&](int i, int o) {
    if (o >= a.kcap) return;
    const int slot = a.cand_slot[rec0 + i];
    sel[o] = slot;
    soff[o] = a.kv.offset(req, head, a.cand_pos[rec0 + i]);
    if (slot < n_sorted)
      atomicAdd(usum + a.cand_unit[rec0 + i], -a.cand_term[rec0 + i]);
    else
      tlog[slot - n_sorted] = kNegInf;
  };

  if (!fallback) {
    // ---- selected candidates above the boundary in the parts before this one ----
    if (part > 0) {
      uint32_t v = 0;
      for (int pp = 0; pp < part; ++pp) {
        const uint4 h = __ldg(reinterpret_cast<const uint4*>(ph + (size_t)pp * kSelHist + b0));
        v += (b0 + 0 > bstar ? h.x : 0u) + (b0 + 1 > bstar ? h.y : 0u) + (b0 + 2 > bstar ? h.z : 0u) +
             (b0 + 3 > bstar ? h.w : 0u);
        if (tid == 0 && kSelBins > bstar) v += ph[(size_t)pp * kSelHist + kSelBins];
      }
      v = __reduce_add_sync(0xffffffffu, v);
      if (lane == 0 && v != 0u) atomicAdd(&es.base_above, (int)v);
    }
    // ---- the boundary bin's keys, from all parts ----
    if (need > 0) {
      for (int pp = 0; pp < P; ++pp) {
        const int cnt = pc[pp];
        const size_t r0 = ((size_t)row * P + pp) * a.seg;
        for (int i = tid; i < cnt; i += kSelThreads) {
          const uint32_t k = a.cand_key[r0 + i];
          if (cand_bin(key_float(k), lo, inv_w) == bstar) {
            const int o = atomicAdd(&es.bcount, 1);
            if (o < kBoundCap) {
              bkey[o] = k;
              bslot[o] = (uint32_t)a.cand_slot[r0 + i];
              bref[o] = ((uint32_t)pp << 24) | (uint32_t)i;
            }
          }
        }
      }
    }
    __syncthreads();
    const int base_above = es.base_above;
    // ---- candidates of this part above the boundary ----
    {
      const int cnt = pc[part];
      for (int i0 = 0; i0 < cnt; i0 += kSelThreads) {
        const int i = i0 + tid;
        const bool take = i < cnt && cand_bin(key_float(a.cand_key[rec0 + i]), lo, inv_w) > bstar;
        const unsigned m = __ballot_sync(0xffffffffu, take);
        int base = 0;
        if (m != 0u && lane == 0) base = atomicAdd(&es.emit_count, __popc(m));
        base = __shfl_sync(0xffffffffu, base, 0) + __popc(m & ((1u << lane) - 1u));
        if (take) emit(i, base_above + base);
      }
    }
    // ---- the boundary: the best `need` of its nb keys by (logit desc, slot asc) ----
    if (need > 0) {
      if (nb <= kSelThreads) {
        // rank counting: key i is taken if fewer than `need` keys beat it; its rank is its place
        if (tid < nb) {
          const uint32_t k = bkey[tid], sl = bslot[tid];
          int rank = 0;
          for (int j = 0; j < nb; ++j) {
            const uint32_t kj = bkey[j], sj = bslot[j];
            rank += (kj > k || (kj == k && sj < sl)) ? 1 : 0;
          }
          if (rank < need && (int)(bref[tid] >> 24) == part) emit((int)(bref[tid] & 0xFFFFFFu), above + rank);
        }
      } else {
        uint32_t kreg[kBoundPer];
#pragma unroll
        for (int j = 0; j < kBoundPer; ++j) {
          const int i = j * kSelThreads + tid;
          kreg[j] = i < nb ? bkey[i] : 0u;
        }
        uint32_t T = 0u, T2 = 0u;
        int t = 0;
        const int ties = block_radix_threshold_regs<kSelThreads, kBoundPer>(kreg, need, rsh2, T, t);
        if (ties != t) {  // more keys tie at the boundary value than fit: lowest slots first
          auto tie_key = [&](int i) -> uint32_t { return bkey[i] == T ? ~bslot[i] : 0u; };
          int t2;
          block_radix_threshold<kSelThreads>(tie_key, nb, t, rsh, T2, t2);
        }
        // taken keys of the parts before this one come first
        int mine_before = 0;
        bool take[kBoundPer];
#pragma unroll
        for (int j = 0; j < kBoundPer; ++j) {
          const int i = j * kSelThreads + tid;
          take[j] = false;
          if (i < nb) {
            const uint32_t k = kreg[j];
            const bool tk = k > T || (k == T && ~bslot[i] >= T2);
            const int owner = (int)(bref[i] >> 24);
            take[j] = tk && owner == part;
            mine_before += (tk && owner < part) ? 1 : 0;
          }
        }
        mine_before = __reduce_add_sync(0xffffffffu, mine_before);
        if (lane == 0 && mine_before != 0) atomicAdd(&es.base_bound, mine_before);
        __syncthreads();
        if (tid == 0) es.emit_count = 0;
        __syncthreads();
        const int bb = above + es.base_bound;
#pragma unroll
        for (int j = 0; j < kBoundPer; ++j) {
          const unsigned m = __ballot_sync(0xffffffffu, take[j]);
          int base = 0;
          if (m != 0u && lane == 0) base = atomicAdd(&es.emit_count, __popc(m));
          base = __shfl_sync(0xffffffffu, base, 0) + __popc(m & ((1u << lane) - 1u));
          if (take[j]) emit((int)(bref[j * kSelThreads + tid] & 0xFFFFFFu), bb + base);
        }
      }
    }
    if (part == 0 && tid == 0) {
      ri[PQHSA_RI_K] = K;
      ri[PQHSA_RI_N] = N;
      ri[PQHSA_RI_NCAND] = C;
      ri[PQHSA_RI_NSEL] = K;
      ri[PQHSA_RI_FALLBACK] = 0;
    }
    return;
  }

  // ---- fallback: the first CTA of the row selects from all N slots, logits recomputed on every pass ----
  if (part != 0) return;
  const uint32_t* codes = a.codes + (size_t)s * a.cap;
  const E* norms = static_cast<const E*>(a.norms) + (size_t)s * a.cap;
  const uint16_t* lids = a.list_ids + (size_t)s * a.cap;
  if (tid < kM * kC) lut_s[tid] = a.lut[(size_t)row * kM * kC + tid];
  for (int i = tid; i < kLMax; i += kSelThreads) lsc_s[i] = a.list_scores[(size_t)row * kLMax + i];
  if (tid == 0) es.emit_count = 0;
  __syncthreads();
  auto logit_of = [&](int slot) -> float {
    return finish_logit(pq_sum_row(lut_s, __ldg(codes + slot)), lsc_s[lids[slot]], to_f(norms[slot]));
  };
  auto key = [&](int i) -> uint32_t { return float_key(logit_of(i)); };
  const bool take_all = K >= N;
  uint32_t T = 0u, T2 = 0u;
  int t = 0;
  if (!take_all) {
    const int ties = block_radix_threshold<kSelThreads>(key, N, K, rsh, T, t);
    if (ties != t) {
      auto tie_key = [&](int i) -> uint32_t { return key(i) == T ? ~(uint32_t)i : 0u; };
      int t2;
      block_radix_threshold<kSelThreads>(tie_key, N, t, rsh, T2, t2);
    }
  }
  const size_t sb = (size_t)s * a.cap;
  for (int slot = tid; slot < N; slot += kSelThreads) {
    const float x = logit_of(slot);
    const uint32_t k = float_key(x);
    if (take_all || k > T || (k == T && ~(uint32_t)slot >= T2)) {
      const int o = atomicAdd(&es.emit_count, 1);
      if (o < a.kcap) {
        sel[o] = slot;
        soff[o] = a.kv.offset(req, head, a.slot_pos[sb + slot]);
        if (slot < n_sorted) {
          const int u = a.slot_unit[sb + slot];
          atomicAdd(usum + u, -unit_term(x, unit_ref(a.unit_max[(size_t)row * a.ucap + u])));
        } else {
          tlog[slot - n_sorted] = kNegInf;
        }
      }
    }
  }
  __syncthreads();
  if (tid == 0) {
    ri[PQHSA_RI_K] = K;
    ri[PQHSA_RI_N] = N;
    ri[PQHSA_RI_NCAND] = C;
    ri[PQHSA_RI_NSEL] = es.emit_count;
    ri[PQHSA_RI_FALLBACK] = 1;
  }
}

int launch_select(const pqhsa_params& p, const pqhsa_ws_layout& w, cudaStream_t st) {
  char* ws = static_cast<char*>(p.workspace);
  const int R = p.num_streams * p.group;
  SelectArgs a;
  a.codes = static_cast<const uint32_t*>(p.codes);
  a.norms = p.norms;
  a.list_ids = static_cast<const uint16_t*>(p.list_ids);
  a.slot_unit = static_cast<const uint16_t*>(p.slot_unit);
  a.slot_pos = static_cast<const int32_t*>(p.slot_pos);
  a.state = static_cast<const int32_t*>(p.state);
  a.lut = reinterpret_cast<const float*>(ws + w.lut);
  a.list_scores = reinterpret_cast<const float*>(ws + w.list_scores);
  a.row_bin = reinterpret_cast<const float*>(ws + w.row_bin);
  a.row_info = reinterpret_cast<int32_t*>(ws + w.row_info);
  a.hitmap = reinterpret_cast<const uint32_t*>(ws + w.hitmap);
  a.unit_off = static_cast<const int32_t*>(p.unit_off);
  a.unit_list = static_cast<const uint16_t*>(p.unit_list);
  a.cand_key = reinterpret_cast<uint32_t*>(ws + w.cand_key);
  a.cand_slot = reinterpret_cast<int32_t*>(ws + w.cand_slot);
  a.cand_pos = reinterpret_cast<int32_t*>(ws + w.cand_pos);
  a.cand_term = reinterpret_cast<float*>(ws + w.cand_term);
  a.cand_unit = reinterpret_cast<uint16_t*>(ws + w.cand_unit);
  a.part_hist = reinterpret_cast<uint32_t*>(ws + w.part_hist);
  a.part_cnt = reinterpret_cast<int32_t*>(ws + w.part_cnt);
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
  a.parts = w.parts;
  a.seg = w.seg;
  a.top_fraction = p.top_fraction;
  a.topk_fixed = p.topk_fixed;
  const size_t smem_a = (size_t)w.seg * (sizeof(uint32_t) + sizeof(uint16_t));
  const size_t smem_b = (size_t)kBoundCap * 3 * sizeof(uint32_t);
  const unsigned grid = (unsigned)(R * w.parts);
  PQHSA_DISPATCH_E(p.dtype, {
    auto ka = cand_kernel<E>;
    auto kb = emit_kernel<E>;
    if (cudaFuncSetAttribute(ka, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_a) != cudaSuccess ||
        cudaFuncSetAttribute(kb, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_b) != cudaSuccess)
      return check_launch("select: shared memory opt-in");
    ka<<<grid, kSelThreads, smem_a, st>>>(a);
    kb<<<grid, kSelThreads, smem_b, st>>>(a);
  });
  return check_launch("select");
}

}  // namespace pqhsa
