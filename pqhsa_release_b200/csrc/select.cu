// Exact top-K selection among the scan's candidates (the reference runs aten
// topk over a materialised [H, G, N] score tensor:
// benchmarks/e2e_pq_param_sweep.py:212-217, :6642; here the scores never
// leave the chip except for the ~2K candidates per row).
//
// The scan left one bit per (row, slot): the key's approximate logit reached the
// row's threshold tau.  Two forms, chosen by K:
//
// 2 K + 1024 <= 8192 - row_select_kernel, one CTA of 1024 threads per row (end of this
// file): the row's candidates (about 1.7 K) stay in the CTA's registers and never
// leave the SM.  Measured, this is the faster form even with 16 rows on 148 SMs.
//
// A larger K (c4: 5243 of 262144 keys) - two launches with `parts` CTAs per row,
// each with its share of the candidates in shared memory; a CTA never waits for
// another one (the second launch starts when the first has ended):
//
// cand_kernel.  The hit words of a row are dealt out to its CTAs word by word.  A
// CTA tabulates its words (bits, first slot, list, candidates listed before) in
// shared memory; candidate i is then the (i - offset)-th set bit of the word a
// binary search over the offsets finds, so every thread gets an even share of the
// candidates whatever the words look like.  The candidates are scored again from
// their codes (bit-identical to the scan; a few thousand gathers that hit the L2
// the scan just filled) and one record per candidate is written - logit key, bin,
// and (slot, token position, the term the scan added to the unit's exp-sum for it,
// unit) - plus a histogram of the part's candidates over PQHSA_SELECT_BINS linear
// bins between tau and an upper companion tau_hi placed by the threshold kernel
// (one more bin holds everything above).
//
// emit_kernel.  Every CTA of a row adds up the row's partial histograms and walks
// them from the top: the bin in which the count reaches K is the boundary bin.
// One pass over the bins of all the row's candidates (eight to a 16-byte load)
// collects the boundary bin's few members and emits this part's candidates above
// it; of the boundary members the best `need` are taken by (logit desc, slot asc) -
// by rank counting when there are at most 256 of them, by a block radix select
// otherwise.  Emitting a candidate = its place in the selection, the element
// offset of its K/V row in the (paged) cache, and its removal from the approximate
// side of the softmax: exactly the term the scan added is subtracted from the
// unit's exp-sum (a selected tail slot has its stored logit set to -inf).  This is
// the "- old_exact_exp" of pq_hsa/attention/sparse_attention.py:985-1009, done per
// unit so that no cancellation error is left behind.
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
constexpr int kSelWords = 8;                        // hit words a thread holds at a time
constexpr int kSelBatch = 8;                        // candidates a thread holds at a time
constexpr int kSelVecs = 4;                         // 8-candidate bin vectors a thread holds at a time

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
  int4* cand_rec;      // (slot, token position, exp-sum term as float bits, unit)
  uint16_t* cand_bin;
  uint32_t* part_hist;
  int32_t* part_cnt;
  int32_t* sel_slot;
  long long* sel_off;
  const float* unit_max;
  float* unit_sum;
  float* tail_logit;
  KvAddr kv;
  int G, cap, ucap, tail_cap, kcap, parts, seg;
  int wcap;  // hit words one part can hold: its share of the unit capacity
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
// A part enumerates its words by an index k: with parts <= 4 every unit gives it 4 / parts words, with
// more parts every run of `parts` units gives it four.
__device__ __forceinline__ int part_word_count(int parts, int n_all) {
  return parts <= 4 ? n_all * (4 / parts) : ((n_all + parts - 1) / parts) * 4;
}
__device__ __forceinline__ bool part_word(int k, int parts, int part, int n_all, int& u, int& it) {
  if (parts <= 4) {
    const int lm = parts == 1 ? 2 : (parts == 2 ? 1 : 0);  // log2(4 / parts): no integer division in the loops
    u = k >> lm;
    it = ((part - u) & (parts - 1)) + parts * (k & ((1 << lm) - 1));
  } else {
    u = parts * (k >> 2) + ((part - (k & 3)) & (parts - 1));
    it = k & 3;
  }
  return u < n_all;
}

// position of the n-th (0-based) set bit of `bits` (n < popc(bits))
__device__ __forceinline__ int nth_set_bit(uint32_t bits, int n) {
  int pos = 0;
#pragma unroll
  for (int w = 16; w >= 1; w >>= 1) {
    const int c = __popc(bits & ((1u << w) - 1u));
    if (n >= c) {
      n -= c;
      bits >>= w;
      pos += w;
    }
  }
  return pos;
}

template <typename E>
__global__ void __launch_bounds__(kSelThreads, 4) cand_kernel(const SelectArgs a) {
  // per hit word of this part: candidates listed before it, its bits, its first slot, its list (0xFFFF: tail)
  extern __shared__ __align__(16) unsigned char sel_smem[];
  uint32_t* woff = reinterpret_cast<uint32_t*>(sel_smem);
  uint32_t* wbits = woff + a.wcap;
  int32_t* wfirst = reinterpret_cast<int32_t*>(wbits + a.wcap);
  uint16_t* wlist = reinterpret_cast<uint16_t*>(wfirst + a.wcap);
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

  // ---- the part's hit words, kSelWords consecutive ones per thread: bits, first slot and list go to shared
  // memory together with the number of candidates listed before the word ----
  const int n_all = n_units + (n_tail + kUnit - 1) / kUnit;  // sorted units, then 128-slot chunks of the tail
  const int nwp = min(part_word_count(P, n_all), a.wcap);
  int C = 0;  // candidates so far (all rounds)
  for (int k0 = 0; k0 < nwp; k0 += kSelWords * kSelThreads) {
    uint32_t b[kSelWords], l[kSelWords];
    int first[kSelWords];
#pragma unroll
    for (int j = 0; j < kSelWords; ++j) {
      const int k = k0 + tid * kSelWords + j;
      int u, it;
      b[j] = 0u;
      l[j] = 0xFFFFu;
      first[j] = 0;
      if (k < nwp && part_word(k, P, part, n_all, u, it)) {
        b[j] = __ldg(hm + (size_t)u * (kUnit / 32) + it);
        if (u < n_units) {
          first[j] = uoff[u] + it * 32;
          l[j] = ulist[u];
        } else {
          first[j] = n_sorted + (u - n_units) * kUnit + it * 32;
        }
      }
    }
    int mine = 0;
#pragma unroll
    for (int j = 0; j < kSelWords; ++j) mine += __popc(b[j]);
    int incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    __syncthreads();  // wtot of the previous round has been read
    if (lane == 31) wtot[warp] = incl;
    __syncthreads();
    int before = 0, total = 0;
#pragma unroll
    for (int w = 0; w < kSelThreads / 32; ++w) {
      const int v = wtot[w];
      before += w < warp ? v : 0;
      total += v;
    }
    int o = C + before + incl - mine;
#pragma unroll
    for (int j = 0; j < kSelWords; ++j) {
      const int k = k0 + tid * kSelWords + j;
      if (k < nwp) {
        woff[k] = (uint32_t)o;
        wbits[k] = b[j];
        wfirst[k] = first[j];
        wlist[k] = (uint16_t)l[j];
      }
      o += __popc(b[j]);
    }
    C += total;
  }
  __syncthreads();  // the word table, the tables, the list scores and the cleared histogram are in place
  if (C > a.seg) {  // more candidates than this part can list: the row is selected from all keys
    if (tid == 0) *pcnt = C;
    return;
  }

  // ---- candidate i (a thread takes i = tid, tid + 256, ...: an even share whatever the words look like) is the
  // (i - woff[w])-th set bit of the last word w whose offset does not exceed i; kSelBatch candidates per thread
  // are scored again at a time, so that their gathers travel together ----
  const size_t rec0 = ((size_t)row * P + part) * a.seg;
  for (int i0 = 0; i0 < C; i0 += kSelBatch * kSelThreads) {
    uint32_t code[kSelBatch];
    float kn[kSelBatch], um[kSelBatch];
    int slot[kSelBatch], pos[kSelBatch], un[kSelBatch], li[kSelBatch];
#pragma unroll
    for (int j = 0; j < kSelBatch; ++j) {
      slot[j] = -1;
      code[j] = 0u;
      kn[j] = 0.f;
      um[j] = 0.f;
      pos[j] = 0;
      un[j] = 0;
      li[j] = 0;
      if (i0 + j * kSelThreads >= C) continue;  // block-uniform: slots past the list cost nothing
      const int i = i0 + j * kSelThreads + tid;
      if (i < C) {
        int lo_w = 0, hi_w = nwp;  // first word whose offset exceeds i
        while (lo_w < hi_w) {
          const int mid = (lo_w + hi_w) >> 1;
          if (woff[mid] <= (uint32_t)i) lo_w = mid + 1; else hi_w = mid;
        }
        const int w = lo_w - 1;
        int u, it;
        part_word(w, P, part, n_all, u, it);
        slot[j] = wfirst[w] + nth_set_bit(wbits[w], i - (int)woff[w]);
        un[j] = u;
        li[j] = wlist[w];
        code[j] = __ldg(codes + slot[j]);
        kn[j] = to_f(norms[slot[j]]);
        pos[j] = spos[slot[j]];
        if (li[j] == 0xFFFF) li[j] = lids[slot[j]];  // a tail slot carries its own list
        else um[j] = umax[u];
      }
    }
#pragma unroll
    for (int j = 0; j < kSelBatch; ++j) {
      if (i0 + j * kSelThreads >= C) continue;  // block-uniform
      const int i = i0 + j * kSelThreads + tid;
      if (i >= C) continue;
      const float x = finish_logit(pq_sum_row(lut_s, code[j]), lsc_s[li[j]], kn[j]);
      const int bin = cand_bin(x, lo, inv_w);
      atomicAdd(&hist[bin], 1u);
      const float term = slot[j] < n_sorted ? unit_term(x, unit_ref(um[j])) : 0.f;
      a.cand_key[rec0 + i] = float_key(x);
      a.cand_bin[rec0 + i] = (uint16_t)bin;
      a.cand_rec[rec0 + i] = make_int4(slot[j], pos[j], __float_as_int(term), un[j]);
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
  int pcnt[16];          // candidates listed by part q
  int vpref[17];         // 8-candidate vectors of the parts before part q
  uint32_t wsum[kSelThreads / 32];
};

template <typename E>
__global__ void __launch_bounds__(kSelThreads, 4) emit_kernel(const SelectArgs a) {
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
    {
      const int nv = (lane < P && !over) ? (cnt + 7) >> 3 : 0;
      int incl = nv;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
      }
      if (lane < 16) es.pcnt[lane] = lane < P ? cnt : 0;
      if (lane <= 16) es.vpref[lane] = incl - nv;  // lanes >= P hold the total
    }
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

  // one selected candidate of this part: its place in the selection, the offset of its K/V row, and its removal from
  // the approximate side of the softmax
  const size_t rec0 = ((size_t)row * P + part) * a.seg;
  auto emit_rec = [&](const int4& r, int o) {  // r = (slot, token position, term, unit)
    if (o >= a.kcap) return;
    sel[o] = r.x;
    soff[o] = a.kv.offset(req, head, r.y);
    if (r.x < n_sorted)
      atomicAdd(usum + r.w, -__int_as_float(r.z));
    else
      tlog[r.x - n_sorted] = kNegInf;
  };
  auto emit = [&](int i, int o) { emit_rec(__ldg(a.cand_rec + rec0 + i), o); };

  if (!fallback) {
    // ---- selected candidates above the boundary in the parts before this one (the histograms again: L1 hits) ----
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
    __syncthreads();
    const int base_above = es.base_above;
    // ---- one pass over the bins of all the row's candidates, eight to a 16-byte vector, the parts' lists walked as
    // one sequence with kSelVecs vectors per thread in flight: members of the boundary bin are collected from every
    // part; candidates of this part above the boundary are placed (one shared-memory atomic per warp) and emitted ----
    {
      const int VT = es.vpref[P];
      for (int g0 = 0; g0 < VT; g0 += kSelVecs * kSelThreads) {
        uint4 w[kSelVecs];
        int vpp[kSelVecs], vidx[kSelVecs];
#pragma unroll
        for (int j = 0; j < kSelVecs; ++j) {
          vpp[j] = -1;
          vidx[j] = 0;
          w[j] = make_uint4(0u, 0u, 0u, 0u);
          if (g0 + j * kSelThreads >= VT) continue;  // block-uniform
          const int g = g0 + j * kSelThreads + tid;
          if (g < VT) {
            int pp = 0;
            for (int q = 1; q < P; ++q) pp += g >= es.vpref[q] ? 1 : 0;
            vpp[j] = pp;
            vidx[j] = g - es.vpref[pp];
            w[j] = __ldg(reinterpret_cast<const uint4*>(a.cand_bin + ((size_t)row * P + pp) * a.seg) + vidx[j]);
          }
        }
#pragma unroll
        for (int j = 0; j < kSelVecs; ++j) {
          if (g0 + j * kSelThreads >= VT) continue;  // block-uniform
          unsigned mask = 0u;
          if (vpp[j] >= 0) {
            const int cnt = es.pcnt[vpp[j]];
            const uint32_t ww[4] = {w[j].x, w[j].y, w[j].z, w[j].w};
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              const int bin = (int)((ww[e >> 1] >> (16 * (e & 1))) & 0xFFFFu);
              const int i = vidx[j] * 8 + e;
              if (i < cnt) {
                if (need > 0 && bin == bstar) {
                  const int o = atomicAdd(&es.bcount, 1);
                  if (o < kBoundCap) bref[o] = ((uint32_t)vpp[j] << 24) | (uint32_t)i;
                }
                if (bin > bstar && vpp[j] == part) mask |= 1u << e;
              }
            }
          }
          if (__ballot_sync(0xffffffffu, mask != 0u) == 0u) continue;  // warp-uniform
          const int mine = __popc(mask);
          int incl = mine;
#pragma unroll
          for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += t;
          }
          int base = 0;
          if (lane == 31) base = atomicAdd(&es.emit_count, incl);
          int o = base_above + __shfl_sync(0xffffffffu, base, 31) + incl - mine;
          // the records of four finds at a time are requested together
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            int4 r[4];
#pragma unroll
            for (int e = 0; e < 4; ++e)
              if ((mask >> (4 * h + e)) & 1u) r[e] = __ldg(a.cand_rec + rec0 + vidx[j] * 8 + 4 * h + e);
#pragma unroll
            for (int e = 0; e < 4; ++e)
              if ((mask >> (4 * h + e)) & 1u) emit_rec(r[e], o++);
          }
        }
      }
    }
    if (need > 0) {
      __syncthreads();
      // the boundary members' keys and slots (ties are broken towards the lower slot)
      for (int i = tid; i < nb; i += kSelThreads) {
        const size_t at = ((size_t)row * P + (bref[i] >> 24)) * a.seg + (bref[i] & 0xFFFFFFu);
        bkey[i] = __ldg(a.cand_key + at);
        bslot[i] = (uint32_t)__ldg(a.cand_rec + at).x;
      }
      __syncthreads();
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

// ---- one CTA per query row --------------------------------------------------------------------------
// A row's selection stays in one CTA of 1024 threads, and nothing is written to or read back from global memory in
// between.
//   1. A thread takes 8 consecutive hit words (two 16-byte loads) and a block prefix sum says how many candidates are
//      listed before each word.
//   2. Candidate i belongs to the last non-empty word whose offset does not exceed i: such a word writes (its index,
//      its offset) at its offset into an array over the candidates and a prefix maximum carries the pair forward.
//      Every candidate finds its word, and its rank inside the word, with one shared-memory load, and the threads get
//      even shares (i = tid, tid + 1024, ...) whatever the bits look like.  The array is all the shared memory the
//      kernel needs (32 KB, whatever the context length); the word's bits, first slot and list come back out of L2.
//   3. The candidates are scored again (bit-identical to the scan), at most 8 per thread in registers, with the token
//      position each one would be gathered from; a block radix select over the register-resident keys finds the K-th
//      largest (ties to the lower slot); the CTA emits.
// More than 8192 candidates, or fewer than K (the threshold estimate failed): the same select over all N slots with the
// keys recomputed on every pass - slow, exact, flagged.
constexpr int kRowThreads = 1024;
// Candidates per thread held in registers: 8 (up to 8192 candidates; their token positions are fetched together
// with their codes) or, for a larger K, 16 (up to 16384; positions are fetched for the selected ones only).
// THREADS: 1024, or 512 for rows with at most 4096 candidates when there are more rows than SMs - two CTAs fit an SM
// then, and the rows' latency chains overlap instead of queueing in waves.
template <int PER, int THREADS> struct RowShape {
  static constexpr int kPer = PER;
  static constexpr int kCap = THREADS * PER;   // more candidates than that select from all keys
  static constexpr int kIdxBits = (PER == 8 ? 13 : 14) - (THREADS == 512 ? 1 : 0);  // bits of a candidate index
  static constexpr bool kPositionsEarly = PER == 8;
  static constexpr int kBinsPer = kSelBins / THREADS;  // histogram bins a thread walks
  static_assert(THREADS == 1024 || THREADS == 512, "thread count");
  static_assert(kCap == 1 << kIdxBits, "candidate index bits");
  static_assert(kBinsPer * THREADS == kSelBins, "bins per thread");
};
constexpr int kRowWords = 8;                        // consecutive hit words per thread and round

constexpr int kRowBoundary = 256;  // members of the boundary bin ranked against each other
static_assert(kSelHist + kRowBoundary <= kRadixBins2, "the boundary members' slots sit behind the bins");
struct RowBoundary {
  int bin, above, members, count, tie;
  uint32_t T, T2;
};

struct RowShared {
  float lut[kM * kC];
  float lsc[kLMax];
  int wtot[kRowThreads / 32];
  int emit_count;
};

template <typename E, int PER, int THREADS>
__global__ void __launch_bounds__(THREADS, 1024 / THREADS) row_select_kernel(const SelectArgs a) {
  using RS = RowShape<PER, THREADS>;
  constexpr int kRowThreads = THREADS;  // shadows the default above
  constexpr int kRowPer = RS::kPer, kRowCandCap = RS::kCap, kRowIdxBits = RS::kIdxBits;
  // candidate -> (word + 1) << 13 | offset of the word's first candidate
  extern __shared__ __align__(16) uint32_t owner[];  // [kRowCandCap]
  __shared__ RowShared sh;
  __shared__ RadixShared rsh;
  __shared__ RadixShared2 rsh2;
  __shared__ RowBoundary bnd;
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
  const int32_t* spos = a.slot_pos + (size_t)s * a.cap;
  const int32_t* uoff = a.unit_off + (size_t)s * (a.ucap + 1);
  const uint16_t* ulist = a.unit_list + (size_t)s * a.ucap;
  const float* umax = a.unit_max + (size_t)row * a.ucap;

  if (tid < kM * kC) sh.lut[tid] = a.lut[(size_t)row * kM * kC + tid];
  if (tid < kLMax) sh.lsc[tid] = a.list_scores[(size_t)row * kLMax + tid];
  if (tid == 0) sh.emit_count = 0;
  const float blo = a.row_bin[2 * row], binv = a.row_bin[2 * row + 1];  // the selection's bins (0, 0: none)
#pragma unroll
  for (int j = 0; j < kRowPer / 4; ++j) reinterpret_cast<uint4*>(owner)[j * kRowThreads + tid] = make_uint4(0u, 0u, 0u, 0u);

  // ---- 1. candidates before every hit word ----
  const uint32_t* hm = a.hitmap + (size_t)row * a.ucap * (kUnit / 32);
  const int nw = (n_units + (n_tail + kUnit - 1) / kUnit) * (kUnit / 32);
  int C = 0;  // candidates so far (all rounds)
  for (int k0 = 0; k0 < nw; k0 += kRowWords * kRowThreads) {
    const int kb = k0 + tid * kRowWords;  // this thread's words kb .. kb + 7
    uint32_t b[kRowWords];
#pragma unroll
    for (int j = 0; j < kRowWords; ++j) b[j] = 0u;
    if (kb < nw) {  // the hit map of a row is a whole number of 16-byte word quadruples
      const uint4 q0 = __ldg(reinterpret_cast<const uint4*>(hm + kb));
      b[0] = q0.x; b[1] = q0.y; b[2] = q0.z; b[3] = q0.w;
      if (kb + 4 < nw) {
        const uint4 q1 = __ldg(reinterpret_cast<const uint4*>(hm + kb + 4));
        b[4] = q1.x; b[5] = q1.y; b[6] = q1.z; b[7] = q1.w;
      }
    }
    int mine = 0;
#pragma unroll
    for (int j = 0; j < kRowWords; ++j) mine += __popc(b[j]);
    int incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    __syncthreads();  // the previous round's totals have been read; first round: the array is clear
    if (lane == 31) sh.wtot[warp] = incl;
    __syncthreads();
    int wt = lane < kRowThreads / 32 ? sh.wtot[lane] : 0;  // every warp scans the warps' totals
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, wt, o);
      if (lane >= o) wt += v;
    }
    const int total = __shfl_sync(0xffffffffu, wt, 31);
    const int before = __shfl_sync(0xffffffffu, wt, warp) - __shfl_sync(0xffffffffu, incl, 31);
    int o = C + before + incl - mine;
#pragma unroll
    for (int j = 0; j < kRowWords; ++j) {
      if (b[j] != 0u && o < kRowCandCap) owner[o] = ((uint32_t)(kb + j + 1) << kRowIdxBits) | (uint32_t)o;
      o += __popc(b[j]);
    }
    C += total;
  }
  const int ncand = C;
  const bool fallback = C < K || C > kRowCandCap || nw >= (1 << (32 - kRowIdxBits)) - 1;
  if (fallback) C = N;
  // ---- 2. candidate -> word: prefix maximum, a warp over a contiguous stretch of the array ----
  if (!fallback) {
    __syncthreads();
    const int per = (C + kRowThreads - 1) / kRowThreads;  // <= kRowPer rounds of 32 per warp
    const int base = warp * per * 32;
    uint32_t v[kRowPer];
    uint32_t carry = 0u;
#pragma unroll
    for (int j = 0; j < kRowPer; ++j) {
      v[j] = 0u;
      if (j >= per) continue;  // block-uniform
      uint32_t x = owner[base + j * 32 + lane];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const uint32_t y = __shfl_up_sync(0xffffffffu, x, o);
        if (lane >= o) x = max(x, y);
      }
      x = max(x, carry);
      carry = __shfl_sync(0xffffffffu, x, 31);
      v[j] = x;
    }
    if (lane == 0) sh.wtot[warp] = (int)carry;
    __syncthreads();
    const uint32_t prev = __reduce_max_sync(0xffffffffu, lane < warp ? (uint32_t)sh.wtot[lane] : 0u);
#pragma unroll
    for (int j = 0; j < kRowPer; ++j) {
      if (j >= per) continue;  // block-uniform
      owner[base + j * 32 + lane] = max(v[j], prev);
    }
  }
  __syncthreads();

  // slot, list and unit of candidate i (normal path) / slot i (fallback)
  auto locate = [&](int i, int& slot, int& list, int& unit) {
    if (fallback) {
      slot = i;
      list = lids[i];
      unit = 0;
      return;
    }
    const uint32_t ow = owner[i];
    const int w = (int)(ow >> kRowIdxBits) - 1, rank = i - (int)(ow & (kRowCandCap - 1));
    unit = w >> 2;
    const uint32_t bits = __ldg(hm + w);
    int first;
    list = -1;
    if (unit < n_units) {
      first = __ldg(uoff + unit);
      list = __ldg(ulist + unit);
    } else {
      first = n_sorted + (unit - n_units) * kUnit;
    }
    slot = first + (w & 3) * 32 + nth_set_bit(bits, rank);
    if (list < 0) list = lids[slot];  // a tail slot carries its own list
  };
  auto logit_at = [&](int slot, int list) -> float {
    return finish_logit(pq_sum_row(sh.lut, __ldg(codes + slot)), sh.lsc[list], to_f(norms[slot]));
  };
  auto key = [&](int i) -> uint32_t {
    int slot, list, unit;
    locate(i, slot, list, unit);
    return float_key(logit_at(slot, list));
  };
  int32_t* sel = a.sel_slot + (size_t)row * a.kcap;
  long long* soff = a.sel_off + (size_t)row * a.kcap;
  const bool take_all = K >= C;
  uint32_t T = 0u, T2 = 0u;
  int t = 0, tie_group = 0;
  const size_t sb = (size_t)s * a.cap;
  if (!fallback) {
    // ---- 3. the candidates sit in registers, kRowPer per thread; their gathers travel four at a time ----
    uint32_t kreg[kRowPer];
    int sreg[kRowPer], preg[RS::kPositionsEarly ? kRowPer : 1];
#pragma unroll
    for (int j0 = 0; j0 < kRowPer; j0 += 4) {
      uint32_t code[4];
      int list[4];
      float kn[4];
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const int j = j0 + jj, i = j * kRowThreads + tid;
        kreg[j] = 0u;
        sreg[j] = -1;
        if constexpr (RS::kPositionsEarly) preg[j] = 0;
        code[jj] = 0u;
        list[jj] = 0;
        kn[jj] = 0.f;
        if (j * kRowThreads >= C) continue;  // block-uniform: slots past the list cost nothing
        if (i < C) {
          int unit;
          locate(i, sreg[j], list[jj], unit);
          code[jj] = __ldg(codes + sreg[j]);
          kn[jj] = to_f(norms[sreg[j]]);
          if constexpr (RS::kPositionsEarly) preg[j] = __ldg(spos + sreg[j]);
        }
      }
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const int j = j0 + jj;
        if (j * kRowThreads >= C) continue;  // block-uniform
        if (sreg[j] >= 0) kreg[j] = float_key(finish_logit(pq_sum_row(sh.lut, code[jj]), sh.lsc[list[jj]], kn[jj]));
      }
    }
    if (!take_all) {
      // The K-th largest lies, as a rule, between the row's threshold and its upper companion (both from the sample):
      // one histogram pass over the kSelBins bins between them (and one bin above) finds the boundary bin, whose few
      // members are ranked against each other by (logit desc, slot asc).  No bins, or a crowded boundary bin: the
      // block radix select over the keys.
      bool done = false;
      if (binv != 0.f) {  // block-uniform
        uint32_t* hist = rsh2.hist;              // [kSelHist]
        uint32_t* bkey = rsh.hist;               // [kRowBoundary] keys of the boundary bin's members
        uint32_t* bslot = rsh2.hist + kSelHist;  // [kRowBoundary] ... their slots
        for (int i = tid; i < kSelHist; i += kRowThreads) hist[i] = 0u;
        if (tid == 0) {
          bnd.count = 0;
          bnd.tie = 0;
        }
        __syncthreads();
#pragma unroll
        for (int j = 0; j < kRowPer; ++j)
          if (kreg[j] != 0u) atomicAdd(&hist[cand_bin(key_float(kreg[j]), blo, binv)], 1u);
        __syncthreads();
        // walk from the top: thread t owns the bins kSelBins - t * kBinsPer downwards (all threads: bins kSelBins .. 1);
        // the last thread also bin 0
        constexpr int kBinsPer = RS::kBinsPer;
        uint32_t bv[kBinsPer], val = 0u;
#pragma unroll
        for (int b = 0; b < kBinsPer; ++b) {
          bv[b] = hist[kSelBins - tid * kBinsPer - b];
          val += bv[b];
        }
        uint32_t incl = val;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const uint32_t v = __shfl_up_sync(0xffffffffu, incl, o);
          if (lane >= o) incl += v;
        }
        if (lane == 31) rsh2.wtot[warp] = incl;
        __syncthreads();
        incl += __reduce_add_sync(0xffffffffu, lane < warp ? rsh2.wtot[lane] : 0u);
        const uint32_t need_k = (uint32_t)K;
        uint32_t run = incl - val;  // candidates in the bins above this thread's
#pragma unroll
        for (int b = 0; b < kBinsPer; ++b) {
          if (run < need_k && need_k <= run + bv[b]) {
            bnd.bin = kSelBins - tid * kBinsPer - b;
            bnd.above = (int)run;
            bnd.members = (int)bv[b];
          }
          run += bv[b];
        }
        if (tid == kRowThreads - 1 && incl < need_k) {
          bnd.bin = 0;
          bnd.above = (int)incl;
          bnd.members = (int)hist[0];
        }
        __syncthreads();
        const int bstar = bnd.bin, need = K - bnd.above, nb = bnd.members;
        if (nb <= kRowBoundary) {  // block-uniform
#pragma unroll
          for (int j = 0; j < kRowPer; ++j)
            if (kreg[j] != 0u && cand_bin(key_float(kreg[j]), blo, binv) == bstar) {
              const int at = atomicAdd(&bnd.count, 1);
              bkey[at] = kreg[j];
              bslot[at] = (uint32_t)sreg[j];
            }
          __syncthreads();
          if (tid < nb) {
            const uint32_t mk = bkey[tid], ms = bslot[tid];
            int rank = 0, eq = 0, eq_after = 0;
            for (int i = 0; i < nb; ++i) {
              const uint32_t ok = bkey[i], os = bslot[i];
              rank += (ok > mk || (ok == mk && os < ms)) ? 1 : 0;
              eq += ok == mk ? 1 : 0;
              eq_after += (ok == mk && os > ms) ? 1 : 0;
            }
            if (rank == need - 1) {  // the last key taken: everything better than it goes, equal logits up to its slot
              bnd.T = mk;
              bnd.T2 = ~ms;
              bnd.tie = eq_after > 0 ? eq : 0;
            }
          }
          __syncthreads();
          T = bnd.T;
          T2 = bnd.T2;
          tie_group = bnd.tie;
          done = true;
        }
      }
      if (!done) {
        __syncthreads();
        const int ties = block_radix_threshold_regs<kRowThreads, kRowPer>(kreg, K, rsh2, T, t);
        if (ties != t) {  // more keys tie at the K-th value than fit (equal code, list and norm): lowest slots first
          uint32_t tk[kRowPer];
#pragma unroll
          for (int j = 0; j < kRowPer; ++j) tk[j] = (kreg[j] == T && kreg[j] != 0u) ? ~(uint32_t)sreg[j] : 0u;
          int t2;
          block_radix_threshold_regs<kRowThreads, kRowPer>(tk, t, rsh2, T2, t2);
          tie_group = ties;
        }
      }
    }
    // Emit: a taken key gets its place in the selection (one shared-memory atomic per warp), the
    // element offset of its K/V row, and leaves the approximate side of the softmax - its unit's
    // exp-sum loses exactly the term the scan added (a tail slot's stored logit becomes -inf).
#pragma unroll
    for (int j0 = 0; j0 < kRowPer; j0 += 4) {
      int o[4], un[4], pos[4];
      float um[4];
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const int j = j0 + jj;
        o[jj] = -1;
        un[jj] = 0;
        pos[jj] = 0;
        um[jj] = 0.f;
        if (j * kRowThreads >= C) continue;  // block-uniform
        const uint32_t k = kreg[j];
        const bool take = k != 0u && (take_all || k > T || (k == T && ~(uint32_t)sreg[j] >= T2));
        const unsigned m = __ballot_sync(0xffffffffu, take);
        int base = 0;
        if (m != 0u && lane == 0) base = atomicAdd(&sh.emit_count, __popc(m));
        base = __shfl_sync(0xffffffffu, base, 0) + __popc(m & ((1u << lane) - 1u));
        o[jj] = take && base < a.kcap ? base : -1;
        if (o[jj] >= 0) {
          if constexpr (RS::kPositionsEarly) pos[jj] = preg[j]; else pos[jj] = __ldg(spos + sreg[j]);
          if (sreg[j] < n_sorted) {
            un[jj] = ((int)(owner[j * kRowThreads + tid] >> kRowIdxBits) - 1) >> 2;
            um[jj] = umax[un[jj]];
          }
        }
      }
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const int j = j0 + jj;
        if (o[jj] < 0) continue;
        sel[o[jj]] = sreg[j];
        soff[o[jj]] = a.kv.offset(req, head, pos[jj]);
        if (sreg[j] < n_sorted)
          atomicAdd(a.unit_sum + (size_t)row * a.ucap + un[jj], -unit_term(key_float(kreg[j]), unit_ref(um[jj])));
        else
          a.tail_logit[(size_t)row * a.tail_cap + (sreg[j] - n_sorted)] = kNegInf;
      }
    }
  } else {
    // all N keys: the keys are recomputed on every pass
    if (!take_all) {
      const int ties = block_radix_threshold<kRowThreads>(key, C, K, rsh, T, t);
      if (ties != t) {
        auto tie_key = [&](int i) -> uint32_t { return key(i) == T ? ~(uint32_t)i : 0u; };
        int t2;
        block_radix_threshold<kRowThreads>(tie_key, C, t, rsh, T2, t2);
        tie_group = ties;
      }
    }
    for (int slot = tid; slot < C; slot += kRowThreads) {
      const float x = logit_at(slot, lids[slot]);
      const uint32_t k = float_key(x);
      if (take_all || k > T || (k == T && ~(uint32_t)slot >= T2)) {
        const int o = atomicAdd(&sh.emit_count, 1);
        if (o < a.kcap) {
          sel[o] = slot;
          soff[o] = a.kv.offset(req, head, a.slot_pos[sb + slot]);
          if (slot < n_sorted) {
            const int u = a.slot_unit[sb + slot];
            atomicAdd(a.unit_sum + (size_t)row * a.ucap + u, -unit_term(x, unit_ref(umax[u])));
          } else {
            a.tail_logit[(size_t)row * a.tail_cap + (slot - n_sorted)] = kNegInf;
          }
        }
      }
    }
  }
  __syncthreads();
  if (tid == 0) {
    ri[PQHSA_RI_K] = K;
    ri[PQHSA_RI_N] = N;
    ri[PQHSA_RI_NCAND] = ncand;
    ri[PQHSA_RI_NSEL] = sh.emit_count;
    ri[PQHSA_RI_FALLBACK] = fallback ? 1 : 0;
    ri[PQHSA_RI_TIES] = tie_group;
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
  a.cand_rec = reinterpret_cast<int4*>(ws + w.cand_rec);
  a.cand_bin = reinterpret_cast<uint16_t*>(ws + w.cand_bin);
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
  a.wcap = w.parts <= 4 ? p.unit_capacity * (4 / w.parts) : ((p.unit_capacity + w.parts - 1) / w.parts) * 4;
  const size_t smem_a = (size_t)a.wcap * (3 * sizeof(uint32_t) + sizeof(uint16_t));
  const size_t smem_b = (size_t)kBoundCap * 3 * sizeof(uint32_t);
  if (w.parts == 1 || w.parts == -1) {
    // one CTA per row: 8 candidates per thread, or 16 for a larger K (parts == -1)
    PQHSA_DISPATCH_E(p.dtype, {
      if (w.parts == 1 && R > sm_count() && 2 * w.kcap + 1024 <= RowShape<8, 512>::kCap) {
        // more rows than SMs and few candidates per row: half-size CTAs, two to an SM
        row_select_kernel<E, 8, 512><<<R, 512, RowShape<8, 512>::kCap * sizeof(uint32_t), st>>>(a);
      } else if (w.parts == 1) {
        row_select_kernel<E, 8, kRowThreads><<<R, kRowThreads, RowShape<8, kRowThreads>::kCap * sizeof(uint32_t), st>>>(a);
      } else {
        auto kern = row_select_kernel<E, 16, kRowThreads>;
        constexpr int smem = RowShape<16, kRowThreads>::kCap * (int)sizeof(uint32_t);
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
          return check_launch("select: shared memory opt-in");
        kern<<<R, kRowThreads, smem, st>>>(a);
      }
    });
    return check_launch("select");
  }
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
