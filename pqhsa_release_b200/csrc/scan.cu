// 4-bit code scan: streams packed codes and norms once per KV head and scores
// them for all G query rows of the head.
//
//   logit[g][n] = (sum_m lut[g][m][nibble_m(n)] + list_scores[g][list(n)]) * |k_n|
//
// (pq_hsa/kernels/lut_scan.py:92-114 + pq_hsa/index/ivfpq.py:1084-1118; the
// production kernel it replaces is pq_hsa/kernels/triton_lut_scan_h20.py:1197-1291.)
//
// Work split.  The sorted region of a stream is cut into units of at most 128
// consecutive slots of ONE list, so the list score is a warp-uniform register
// and the per-list log-sum-exp is a warp reduction with no atomics.  A persistent
// grid (one CTA per SM) shares the units out.  With few streams every CTA stays
// inside one stream (a stream's CTAs split its units evenly), because entering a
// stream - 128 KB of tables, list scores, headers - costs about as much as 40
// units of scanning.  With many streams all units of all streams form one global
// sequence and the CTAs take equal shares of it, so ragged contexts balance by
// themselves and a CTA may run across stream boundaries.  Inside a
// stream the sequence is a stride permutation of the units, so every CTA gets
// units from all over the stream (lists with many candidates do not pile up on one
// CTA).  The unit headers of a share are staged in shared memory; a warp takes one
// unit at a time, lanes take consecutive slots (coalesced 4-byte code and 2-byte
// norm loads), and the loads of a warp's next unit are issued before the current
// one is scored.  Slots of the unsorted tail carry their own list id and are
// scored in the same launch; their logits are kept individually.
//
// The scan is bound by instruction issue, not HBM (8 bytes per key against G sums
// of 8 table entries), so the inner loop is built to be short:
//   * the 8 nibble tables are folded into 4 byte-pair tables (256 entries of
//     min(G,4) floats) when a CTA enters a stream, replicated so that lane j of a
//     quarter warp reads replica j: every LDS.128 hits distinct banks whatever the
//     codes are - 4 conflict-free 16-byte lookups per key (128 KB of tables);
//     G = 8 runs two such passes;
//   * the rows of a pass are carried as packed f32x2 values (add / mul / fma on
//     two rows per instruction, same IEEE rounding as the scalar form);
//   * the unit maximum is one redux.sync.max.f32 per row;
//   * candidates (logit >= the row's threshold) are marked in a bit map: one vote per
//     row and 32 slots, taken only in units whose maximum reaches the threshold (the
//     others store zero words); the 4 words of a (row, unit) are one 16-byte store.
//
// Outputs per query row: per-unit (max, sum exp) - a unit's logits stay in
// registers and the sum is taken against the unit's final maximum, so every key
// contributes exactly unit_term(logit, reference) and the selection kernel can
// remove a selected key again without cancellation error - the tail logits, and
// the hit bits.  The logits themselves are never written; the separate dump
// kernel writes all of them for tests and the stand-alone scoring entry point.
#include "common.cuh"

namespace pqhsa {

constexpr int kScanThreads = 1024;  // 32 warps of 64 registers: the loop is issue-bound and needs the warps
constexpr int kHdr = 512;     // unit headers staged in shared memory at a time
constexpr int kSegCost = 48;  // cost of entering a stream, in units of scanning work (share balancing)
constexpr int kIter = kUnit / 32;

template <int G> struct PairShape {
  static constexpr int GP = G < 4 ? G : 4;      // rows per pass = floats per lookup vector
  static constexpr int NP = G / GP;             // passes
  static constexpr int REP = 32 / GP;           // replicas
  static constexpr int kFloats = 4 * 256 * 32;  // 4 pair tables x 256 entries x REP x GP = 128 KB
};

struct ScanArgs {
  const uint32_t* codes;
  const void* norms;
  const uint16_t* list_ids;
  const int32_t* unit_off;
  const uint16_t* unit_list;
  const int32_t* state;
  const float* lut;
  const float* pair_tab;
  const float* list_scores;
  const float* row_tau;
  uint32_t* hitmap;
  float* unit_max;
  float* unit_sum;
  float* tail_logit;
  float* dump;
  int S, G, cap, ucap, tail_cap;
};

__device__ __forceinline__ float redux_max(float v) {
  float r;
  asm volatile("redux.sync.max.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(v));
  return r;
}

// Sum GP values across the warp: each halving step exchanges half of the values, so 4
// values cost 6 shuffles instead of 20.  Afterwards the lanes of group j = lane / (32 / GP)
// hold the total of value j.
template <int GP>
__device__ __forceinline__ float warp_sum_multi(const float (&v)[GP], int lane) {
  if constexpr (GP == 4) {
    const bool hi = lane & 16;
    float k0 = hi ? v[2] : v[0], k1 = hi ? v[3] : v[1];
    const float s0 = hi ? v[0] : v[2], s1 = hi ? v[1] : v[3];
    k0 += __shfl_xor_sync(0xffffffffu, s0, 16);
    k1 += __shfl_xor_sync(0xffffffffu, s1, 16);
    const bool h2 = lane & 8;
    float k = h2 ? k1 : k0;
    const float s = h2 ? k0 : k1;
    k += __shfl_xor_sync(0xffffffffu, s, 8);
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) k += __shfl_xor_sync(0xffffffffu, k, o);
    return k;  // lanes 0-7: value 0, 8-15: value 1, 16-23: value 2, 24-31: value 3
  } else if constexpr (GP == 2) {
    const bool hi = lane & 16;
    float k = hi ? v[1] : v[0];
    const float s = hi ? v[0] : v[1];
    k += __shfl_xor_sync(0xffffffffu, s, 16);
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) k += __shfl_xor_sync(0xffffffffu, k, o);
    return k;  // lanes 0-15: value 0, 16-31: value 1
  } else {
    float k = v[0];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) k += __shfl_xor_sync(0xffffffffu, k, o);
    return k;
  }
}

// logits of one key for the GP rows of a pass, from the replicated pair tables
template <int GP>
__device__ __forceinline__ void score_key(const float* __restrict__ mytab, uint32_t code, const float (&ls)[GP],
                                          float kn, float (&x)[GP]) {
  const float* p0 = mytab + ((code & 255u) << 5);
  const float* p1 = mytab + 8192 + (((code >> 8) & 255u) << 5);
  const float* p2 = mytab + 16384 + (((code >> 16) & 255u) << 5);
  const float* p3 = mytab + 24576 + ((code >> 24) << 5);
  if constexpr (GP == 4) {
    const float4 t0 = *reinterpret_cast<const float4*>(p0), t1 = *reinterpret_cast<const float4*>(p1);
    const float4 t2 = *reinterpret_cast<const float4*>(p2), t3 = *reinterpret_cast<const float4*>(p3);
    float2 a = __fadd2_rn(make_float2(t0.x, t0.y), make_float2(t1.x, t1.y));
    float2 b = __fadd2_rn(make_float2(t0.z, t0.w), make_float2(t1.z, t1.w));
    a = __fadd2_rn(a, make_float2(t2.x, t2.y));
    b = __fadd2_rn(b, make_float2(t2.z, t2.w));
    a = __fadd2_rn(a, make_float2(t3.x, t3.y));
    b = __fadd2_rn(b, make_float2(t3.z, t3.w));
    a = __fmul2_rn(__fadd2_rn(a, make_float2(ls[0], ls[1])), make_float2(kn, kn));
    b = __fmul2_rn(__fadd2_rn(b, make_float2(ls[2], ls[3])), make_float2(kn, kn));
    x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y;
  } else if constexpr (GP == 2) {
    const float2 t0 = *reinterpret_cast<const float2*>(p0), t1 = *reinterpret_cast<const float2*>(p1);
    const float2 t2 = *reinterpret_cast<const float2*>(p2), t3 = *reinterpret_cast<const float2*>(p3);
    float2 a = __fadd2_rn(__fadd2_rn(__fadd2_rn(t0, t1), t2), t3);
    a = __fmul2_rn(__fadd2_rn(a, make_float2(ls[0], ls[1])), make_float2(kn, kn));
    x[0] = a.x; x[1] = a.y;
  } else {
    const float a = __fadd_rn(__fadd_rn(__fadd_rn(*p0, *p1), *p2), *p3);
    x[0] = finish_logit(a, ls[0], kn);
  }
}

template <typename E> struct ScanRing {
  static constexpr int kCodeBytes = (kUnit / 4 + 1) * 16;                                  // 128 codes + alignment slack
  static constexpr int kNormBytes = (kUnit * (int)sizeof(E) / 16 + 1) * 16;                // 128 norms + slack
  static constexpr int kStageBytes = kCodeBytes + kNormBytes;
  static constexpr int kDepth = 2;  // units per warp in the ring: one being scored, one in flight
};

// ALIGNED: few streams (at most a warp's worth and a quarter of the grid): every CTA works inside ONE stream, so it
// pays for one set of tables, list scores and headers; stream s gets 1 + floor(units_s * (grid - streams) / units)
// CTAs, which split its units evenly.  Every warp works the split out for itself from the counters (no barrier).
// Otherwise: equal shares of the global unit sequence, a CTA may run across stream boundaries.
template <typename E, int G, int T, bool ALIGNED>
__global__ void __launch_bounds__(T, 1) scan_kernel(const ScanArgs a) {
  using PS = PairShape<G>;
  using RG = ScanRing<E>;
  constexpr int GP = PS::GP;
  constexpr int W = T / 32;
  constexpr int D = RG::kDepth;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* tab = reinterpret_cast<float*>(smem_raw);                              // pair tables, replicated
  float* lsc_s = tab + PS::kFloats;                                             // [kLMax][GP] list scores of the pass
  int4* hdr = reinterpret_cast<int4*>(lsc_s + kLMax * GP);                      // [kHdr] (first slot, slots, list, unit)
  unsigned char* ring = reinterpret_cast<unsigned char*>(hdr + kHdr);           // [W][D] codes + norms of units in flight
  __shared__ long long s_red[32];
  __shared__ int s_pref[T], s_ut[T], s_first;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  unsigned char* wring = ring + (size_t)warp * D * RG::kStageBytes;

  // Length of a stream on the axis the shares are cut from: its units plus kSegCost, the price (in
  // units of scanning work) of entering a stream - tables, list scores, headers.  A CTA whose share
  // runs across the start of a stream pays for a second entry and gets that many units less.
  auto units_of = [&](int s) -> int {
    const int32_t* st = a.state + (size_t)s * kST;
    const int u = st[PQHSA_ST_N_UNITS] + (st[PQHSA_ST_N_TAIL] + kUnit - 1) / kUnit;
    return u > 0 ? u + kSegCost : 0;
  };

  // ---- the units [u0, u1) of stream s (u_tot units in all) ----
  auto scan_stream = [&](const int s, const int u0, const int u1, const int u_tot) {
        const int32_t* st = a.state + (size_t)s * kST;
        const int n_sorted = st[PQHSA_ST_N_SORTED], n_tail = st[PQHSA_ST_N_TAIL], n_units = st[PQHSA_ST_N_UNITS];
        const uint32_t* codes = a.codes + (size_t)s * a.cap;
        const E* norms = static_cast<const E*>(a.norms) + (size_t)s * a.cap;
        const uint16_t* lids = a.list_ids + (size_t)s * a.cap;
        const int32_t* uoff = a.unit_off + (size_t)s * (a.ucap + 1);
        const uint16_t* ulist = a.unit_list + (size_t)s * a.ucap;
        // first slot of unit u (sorted units, then 128-slot chunks of the tail); also valid for u = u_tot
        auto unit_first = [&](int u) -> int {
          return u < n_units ? uoff[u] : n_sorted + min((u - n_units) * kUnit, n_tail);
        };
        // Position x of the stream's share sequence is unit (x * stride) mod u_tot, stride a prime that
        // does not divide u_tot: a bijection that hands every CTA units from all over the stream.  Lists
        // with many candidates would otherwise all fall to the one CTA that owns their range.
        int stride = 127;
        if (u_tot % stride == 0) stride = 131;
        if (u_tot % stride == 0) stride = 137;
        if (u_tot % stride == 0) stride = 139;  // 127 x 131 x 137 exceeds any unit count, so one of the four fits

#pragma unroll 1
        for (int pass = 0; pass < PS::NP; ++pass) {
          const int row0 = s * G + pass * GP;  // first query row of this pass
          __syncthreads();                     // tables, list scores and headers of the previous pass are done with
          for (int i = tid; i < GP * kLMax; i += T)  // [g][l] in global memory -> [l][g] here
            lsc_s[(i % kLMax) * GP + i / kLMax] = a.list_scores[(size_t)row0 * kLMax + i];
          // Pair tables of the pass (made by the table kernel), replicated:
          // tab[((p * 256 + byte) * REP + rep) * GP + g].  Consecutive threads write consecutive
          // GP-float vectors (conflict-free stores); the REP threads of an entry read the same vector.
          {
            const float* src = a.pair_tab + (size_t)(s * PS::NP + pass) * (4 * 256 * GP);
#pragma unroll
            for (int i = tid; i < 4 * 256 * PS::REP; i += T) {
              const int e = i / PS::REP;
              if constexpr (GP == 4) {
                reinterpret_cast<float4*>(tab)[i] = __ldg(reinterpret_cast<const float4*>(src) + e);
              } else if constexpr (GP == 2) {
                reinterpret_cast<float2*>(tab)[i] = __ldg(reinterpret_cast<const float2*>(src) + e);
              } else {
                tab[i] = __ldg(src + e);
              }
            }
          }
          const float* mytab = tab + (lane & (PS::REP - 1)) * GP;
          float tau[GP];
#pragma unroll
          for (int g = 0; g < GP; ++g) tau[g] = a.row_tau[row0 + g];

          for (int h0 = u0; h0 < u1; h0 += kHdr) {
            const int cnt = min(kHdr, u1 - h0);
            __syncthreads();  // the previous header chunk is done with
            for (int i = tid; i < cnt; i += T) {
              const int u = (int)(((long long)(h0 + i) * stride) % u_tot);  // position in the share -> unit
              const int lo = unit_first(u);
              hdr[i] = make_int4(lo, unit_first(u + 1) - lo, u < n_units ? (int)ulist[u] : 0xFFFF, u);
            }
            __syncthreads();  // headers, tables and list scores are in place

            // A warp's units: i = warp, warp + W, ...  Their codes and norms travel through a ring of D
            // stages per warp, filled by 16-byte asynchronous copies issued D - 1 units ahead; a copy
            // starts at the 16-byte boundary below the unit's first element.
            auto request = [&](int i) {
              if (i < cnt) {
                const int4 h = hdr[i];
                unsigned char* stg = wring + (size_t)((i / W) % D) * RG::kStageBytes;
                const int c0 = h.x & ~3;                                  // codes: 4 per 16 bytes
                const int cch = (h.x + h.y - c0 + 3) >> 2;                // at most 33 chunks
                if (lane < cch) cp_async16(stg + lane * 16, codes + c0 + lane * 4);
                if (lane == 0 && cch > 32) cp_async16(stg + 32 * 16, codes + c0 + 32 * 4);
                constexpr int kPer = 16 / (int)sizeof(E);                 // norms per 16 bytes
                const int n0 = h.x & ~(kPer - 1);
                const int nch = (h.x + h.y - n0 + kPer - 1) / kPer;
                if (lane < nch) cp_async16(stg + RG::kCodeBytes + lane * 16, norms + n0 + lane * kPer);
                if (lane == 0 && nch > 32) cp_async16(stg + RG::kCodeBytes + 32 * 16, norms + n0 + 32 * kPer);
              }
              cp_async_commit();  // one group per request, empty or not: the wait below counts groups
            };
#pragma unroll
            for (int d = 0; d < D - 1; ++d) request(warp + d * W);
            for (int i = warp; i < cnt; i += W) {
              request(i + (D - 1) * W);
              cp_async_wait<D - 1>();
              __syncwarp();
              const int4 cur = hdr[i];
              const int lo = cur.x, n = cur.y, u = cur.w;
              const unsigned char* stg = wring + (size_t)((i / W) % D) * RG::kStageBytes;
              const uint32_t* cs = reinterpret_cast<const uint32_t*>(stg) + (lo & 3) + lane;
              const E* ns = reinterpret_cast<const E*>(stg + RG::kCodeBytes) + (lo & (16 / (int)sizeof(E) - 1)) + lane;
              if (cur.z != 0xFFFF) {
                float ls[GP];
                if constexpr (GP == 4) {
                  const float4 v = *reinterpret_cast<const float4*>(lsc_s + cur.z * 4);
                  ls[0] = v.x; ls[1] = v.y; ls[2] = v.z; ls[3] = v.w;
                } else if constexpr (GP == 2) {
                  const float2 v = *reinterpret_cast<const float2*>(lsc_s + cur.z * 2);
                  ls[0] = v.x; ls[1] = v.y;
                } else {
                  ls[0] = lsc_s[cur.z];
                }
                float xs[kIter][GP];
#pragma unroll
                for (int it = 0; it < kIter; ++it) {
                  if ((it + 1) * 32 <= n) {  // warp-uniform: every lane has a key
                    score_key<GP>(mytab, cs[it * 32], ls, to_f(ns[it * 32]), xs[it]);
                  } else if (it * 32 < n) {  // warp-uniform: the ragged end (the ring holds stale bytes there)
                    score_key<GP>(mytab, cs[it * 32], ls, to_f(ns[it * 32]), xs[it]);
                    if (it * 32 + lane >= n) {
#pragma unroll
                      for (int g = 0; g < GP; ++g) xs[it][g] = kNegInf;
                    }
                  } else {
#pragma unroll
                    for (int g = 0; g < GP; ++g) xs[it][g] = kNegInf;
                  }
                }
                // unit maximum per row (one redux each)
                float mg[GP];
#pragma unroll
                for (int g = 0; g < GP; ++g) {
                  float mx = xs[0][g];
#pragma unroll
                  for (int it = 1; it < kIter; ++it) mx = fmaxf(mx, xs[it][g]);
                  mg[g] = redux_max(mx);
                }
                // candidates: one vote per row and 32 slots, only where the unit maximum reaches the threshold
                // (padding lanes are excluded by index: the threshold may be -inf); the 4 words of a row and unit are one 16-byte store
#pragma unroll
                for (int g = 0; g < GP; ++g) {
                  unsigned m[kIter];
#pragma unroll
                  for (int it = 0; it < kIter; ++it) m[it] = 0u;
                  if (mg[g] >= tau[g]) {  // warp-uniform
#pragma unroll
                    for (int it = 0; it < kIter; ++it)
                      m[it] = __ballot_sync(0xffffffffu, it * 32 + lane < n && xs[it][g] >= tau[g]);
                  }
                  if (lane == 0)
                    *reinterpret_cast<uint4*>(a.hitmap + ((size_t)(row0 + g) * a.ucap + u) * kIter) =
                        make_uint4(m[0], m[1], m[2], m[3]);
                }
                // the sum of unit_term(logit, reference of the unit maximum); -inf contributes 0
                float sm[GP];
                if constexpr (GP >= 2) {
#pragma unroll
                  for (int g = 0; g < GP; g += 2) {
                    const float2 ref = make_float2(unit_ref(mg[g]), unit_ref(mg[g + 1]));
                    float2 acc = make_float2(0.f, 0.f);
#pragma unroll
                    for (int it = 0; it < kIter; ++it) {
                      const float2 t =
                          __ffma2_rn(make_float2(xs[it][g], xs[it][g + 1]), make_float2(kLog2e, kLog2e), ref);
                      acc = __fadd2_rn(acc, make_float2(ex2(t.x), ex2(t.y)));
                    }
                    sm[g] = acc.x;
                    sm[g + 1] = acc.y;
                  }
                } else {
                  const float ref = unit_ref(mg[0]);
                  sm[0] = 0.f;
#pragma unroll
                  for (int it = 0; it < kIter; ++it) sm[0] += unit_term(xs[it][0], ref);
                }
                const float sred = warp_sum_multi<GP>(sm, lane);
                if ((lane & (32 / GP - 1)) == 0) {
                  const int g = lane / (32 / GP);
                  float mine = mg[0];
#pragma unroll
                  for (int gg = 1; gg < GP; ++gg)
                    if (gg == g) mine = mg[gg];
                  a.unit_max[(size_t)(row0 + g) * a.ucap + u] = mine;
                  a.unit_sum[(size_t)(row0 + g) * a.ucap + u] = sred;
                }
              } else {
                // a chunk of the unsorted tail: every slot has its own list; logits are kept one by one
#pragma unroll
                for (int it = 0; it < kIter; ++it) {
                  if (it * 32 < n) {  // warp-uniform
                    const bool valid = it * 32 + lane < n;
                    const int slot = lo + (valid ? it * 32 + lane : 0);
                    const int l = lids[slot];
                    float ls[GP], x[GP];
#pragma unroll
                    for (int g = 0; g < GP; ++g) ls[g] = lsc_s[l * GP + g];
                    score_key<GP>(mytab, cs[it * 32], ls, to_f(ns[it * 32]), x);
#pragma unroll
                    for (int g = 0; g < GP; ++g) {
                      if (valid) a.tail_logit[(size_t)(row0 + g) * a.tail_cap + (slot - n_sorted)] = x[g];
                      const unsigned m = __ballot_sync(0xffffffffu, valid && x[g] >= tau[g]);
                      if (lane == 0) a.hitmap[((size_t)(row0 + g) * a.ucap + u) * kIter + it] = m;
                    }
                  } else if (lane < GP) {
                    a.hitmap[((size_t)(row0 + lane) * a.ucap + u) * kIter + it] = 0u;
                  }
                }
              }
              __syncwarp();  // every lane is done with this stage before a later request refills it
            }
            cp_async_wait<0>();
          }
        }
  };

  if constexpr (ALIGNED) {
    int cost = 0;  // lane s: units of stream s
    if (lane < a.S) {
      const int32_t* st = a.state + (size_t)lane * kST;
      cost = st[PQHSA_ST_N_UNITS] + (st[PQHSA_ST_N_TAIL] + kUnit - 1) / kUnit;
    }
    const int total = (int)__reduce_add_sync(0xffffffffu, (unsigned)cost);
    const int live = __popc(__ballot_sync(0xffffffffu, cost > 0));
    if (total == 0) return;
    const int ctas = cost > 0 ? 1 + (int)((long long)cost * ((int)gridDim.x - live) / total) : 0;
    int incl = ctas;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    const int b = blockIdx.x;
    const unsigned owner = __ballot_sync(0xffffffffu, incl - ctas <= b && b < incl);
    if (owner == 0u) return;  // a spare CTA
    const int s = __ffs(owner) - 1;
    const int j = b - __shfl_sync(0xffffffffu, incl - ctas, s), n = __shfl_sync(0xffffffffu, ctas, s);
    const int c = __shfl_sync(0xffffffffu, cost, s);
    const int u0 = (int)((long long)c * j / n), u1 = (int)((long long)c * (j + 1) / n);
    if (u0 < u1) scan_stream(s, u0, u1, c);
  } else {
  // total number of units (all streams), one load per thread
  long long part = 0;
  for (int s = tid; s < a.S; s += T) part += units_of(s);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
  if (lane == 0) s_red[warp] = part;
  __syncthreads();
  long long total = 0;
#pragma unroll
  for (int w = 0; w < W; ++w) total += s_red[w];
  // this CTA's share [g0, g1) of the global unit sequence
  const long long g0 = total * blockIdx.x / gridDim.x, g1 = total * (blockIdx.x + 1) / gridDim.x;
  if (g0 >= g1) return;

  long long carry = 0;  // global index of the first unit of stream `base`
  for (int base = 0; base < a.S && carry < g1; base += T) {
    // exclusive prefix of the unit counts of streams base .. base + T - 1
    const int ut = base + tid < a.S ? units_of(base + tid) : 0;
    int incl = ut;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    __syncthreads();  // s_red, s_pref, s_ut, s_first of the previous round are no longer read
    if (lane == 31) s_red[warp] = incl;
    if (tid == 0) s_first = 0;
    __syncthreads();
    int woff = 0, ctot = 0;
#pragma unroll
    for (int w = 0; w < W; ++w) {
      const int v = (int)s_red[w];
      woff += w < warp ? v : 0;
      ctot += v;
    }
    const int excl = woff + incl - ut;
    s_pref[tid] = excl;
    s_ut[tid] = ut;
    if (ut > 0 && carry + excl <= g0 && g0 < carry + excl + ut) s_first = tid;  // the stream holding g0
    __syncthreads();
    if (carry + ctot > g0) {
      const int tend = min(T, a.S - base);
      for (int t = s_first; t < tend; ++t) {
        const long long sb = carry + s_pref[t];
        const int len = s_ut[t];  // units + kSegCost
        if (sb >= g1) break;
        if (len == 0 || sb + len <= g0) continue;
        const int s = base + t;
        const int u_tot = len - kSegCost;
        const int u0 = max((int)((sb > g0 ? sb : g0) - sb) - kSegCost, 0);
        const int u1 = max((int)((sb + len < g1 ? sb + len : g1) - sb) - kSegCost, 0);
        if (u0 >= u1) continue;

        scan_stream(s, u0, u1, u_tot);
      }
    }
    carry += ctot;
  }
  }
}

// All logits of all slots, fp32 [R, cap]: same arithmetic (pq_sum_row / finish_logit) as the
// scan, one thread per slot.  Not on the decode path.
template <typename E>
__global__ void __launch_bounds__(256) scan_dump_kernel(const ScanArgs a) {
  extern __shared__ float lut_d[];  // [G][128]
  const int s = blockIdx.y, tid = threadIdx.x;
  for (int i = tid; i < a.G * kM * kC; i += 256) lut_d[i] = a.lut[(size_t)s * a.G * kM * kC + i];
  __syncthreads();
  const int32_t* st = a.state + (size_t)s * kST;
  const int n = st[PQHSA_ST_N_SORTED] + st[PQHSA_ST_N_TAIL];
  const int slot = blockIdx.x * 256 + tid;
  if (slot >= n) return;
  const uint32_t code = __ldg(a.codes + (size_t)s * a.cap + slot);
  const float kn = to_f(static_cast<const E*>(a.norms)[(size_t)s * a.cap + slot]);
  const int l = a.list_ids[(size_t)s * a.cap + slot];
  for (int g = 0; g < a.G; ++g) {
    const int row = s * a.G + g;
    a.dump[(size_t)row * a.cap + slot] =
        finish_logit(pq_sum_row(lut_d + g * kM * kC, code), __ldg(a.list_scores + (size_t)row * kLMax + l), kn);
  }
}

template <typename E, int G, int T>
static int launch_scan_t(const pqhsa_params& p, const ScanArgs& a, cudaStream_t st) {
  const long long units_hi = (long long)p.num_streams * (p.num_lists + p.max_slots / kUnit + 2);
  long long ctas = sm_count();
  if (ctas > units_hi) ctas = units_hi;
  if (ctas < 1) ctas = 1;
  const bool aligned = p.num_streams <= 32 && 4LL * p.num_streams <= ctas;
  using PS = PairShape<G>;
  const size_t smem = PS::kFloats * sizeof(float) + (size_t)kLMax * PS::GP * sizeof(float) + (size_t)kHdr * sizeof(int4) +
                      (size_t)(T / 32) * ScanRing<E>::kDepth * ScanRing<E>::kStageBytes;
  auto kern = aligned ? scan_kernel<E, G, T, true> : scan_kernel<E, G, T, false>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    return check_launch("scan: shared memory opt-in");
  kern<<<(unsigned)ctas, T, smem, st>>>(a);
  return check_launch("scan");
}

int launch_scan(const pqhsa_params& p, const pqhsa_ws_layout& w, float* dump, cudaStream_t st) {
  char* ws = static_cast<char*>(p.workspace);
  ScanArgs a;
  a.codes = static_cast<const uint32_t*>(p.codes);
  a.norms = p.norms;
  a.list_ids = static_cast<const uint16_t*>(p.list_ids);
  a.unit_off = static_cast<const int32_t*>(p.unit_off);
  a.unit_list = static_cast<const uint16_t*>(p.unit_list);
  a.state = static_cast<const int32_t*>(p.state);
  a.lut = reinterpret_cast<const float*>(ws + w.lut);
  a.pair_tab = reinterpret_cast<const float*>(ws + w.pair_tab);
  a.list_scores = reinterpret_cast<const float*>(ws + w.list_scores);
  a.row_tau = reinterpret_cast<const float*>(ws + w.row_tau);
  a.hitmap = reinterpret_cast<uint32_t*>(ws + w.hitmap);
  a.unit_max = reinterpret_cast<float*>(ws + w.unit_max);
  a.unit_sum = reinterpret_cast<float*>(ws + w.unit_sum);
  a.tail_logit = reinterpret_cast<float*>(ws + w.tail_logit);
  a.dump = dump;
  a.S = p.num_streams;
  a.G = p.group;
  a.cap = p.slot_capacity;
  a.ucap = p.unit_capacity;
  a.tail_cap = w.tail_cap;
  if (dump != nullptr) {
    if (p.max_slots == 0) return PQHSA_OK;
    const dim3 grid((p.max_slots + 255) / 256, p.num_streams);
    const size_t smem = (size_t)p.group * kM * kC * sizeof(float);
    PQHSA_DISPATCH_E(p.dtype, scan_dump_kernel<E><<<grid, 256, smem, st>>>(a));
    return check_launch("scan_dump");
  }
  PQHSA_DISPATCH_E(p.dtype, PQHSA_DISPATCH_G(p.group, return (launch_scan_t<E, G, kScanThreads>(p, a, st))));
  return PQHSA_OK;
}

}  // namespace pqhsa
