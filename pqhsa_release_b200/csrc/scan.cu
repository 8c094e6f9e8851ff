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
// and the per-list log-sum-exp is a warp reduction with no atomics.  All units
// of all streams form one global sequence; a persistent grid (one CTA per SM)
// takes equal contiguous shares of it, so ragged contexts balance by
// themselves.  A warp takes one unit at a time; lanes take consecutive slots
// (coalesced 4-byte code and 2-byte norm loads, all of a unit in flight at once).
// Slots of the unsorted tail carry their own list id and are scored in the same
// launch; their logits are kept individually.
//
// Table lookups.  The scan is bound by shared-memory bandwidth, not HBM: a key
// needs its G sums of 8 table entries.  The kernel therefore folds the 8 nibble
// tables into 4 byte-pair tables (256 entries of min(G,4) floats) when it enters
// a stream, and replicates them so that lane j of a quarter warp reads replica
// j: every LDS.128 hits distinct banks whatever the codes are.  4 conflict-free
// 16-byte lookups per key = 64 B of shared-memory traffic per key for 4 rows;
// G = 8 runs two such passes.  (128 KB of tables per CTA.)
//
// Outputs per query row: per-unit (max, sum exp) - a unit's logits stay in
// registers, the sum is taken against the unit's final maximum, so every key
// contributes exactly unit_term(logit, max) and the selection kernel can remove
// a selected key again without cancellation error - the tail logits, and the
// candidates (slot, logit) with logit >= the row's threshold.  Candidates are
// compacted per warp: ballot + prefix count into a warp-private shared-memory
// buffer, written out with one global atomic per 64 candidates.  The logits
// themselves are never written.  Dump mode writes all fp32 logits instead
// (tests / stand-alone scoring).
#include "common.cuh"

namespace pqhsa {

constexpr int kScanThreads = 1024;
constexpr int kScanWarps = kScanThreads / 32;
constexpr int kWStage = 64;  // staged candidates per warp and row
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
  const float* list_scores;
  const float* row_tau;
  int32_t* row_info;
  int32_t* cand_slot;
  float* cand_logit;
  float* unit_max;
  float* unit_sum;
  float* tail_logit;
  float* dump;
  int S, cap, ucap, tail_cap, ccap;
};

// Reduce GP values across the warp: each halving step exchanges half of the
// values, so 4 values cost 6 shuffles instead of 20.  Afterwards the lanes of
// group j = lane / (32 / GP) hold the total of value j.
template <int GP, bool MAX>
__device__ __forceinline__ float warp_reduce_multi(float (&v)[GP], int lane) {
  auto op = [](float a, float b) { return MAX ? fmaxf(a, b) : a + b; };
  if constexpr (GP == 4) {
    const bool hi = lane & 16;
    float k0 = hi ? v[2] : v[0], k1 = hi ? v[3] : v[1];
    const float s0 = hi ? v[0] : v[2], s1 = hi ? v[1] : v[3];
    k0 = op(k0, __shfl_xor_sync(0xffffffffu, s0, 16));
    k1 = op(k1, __shfl_xor_sync(0xffffffffu, s1, 16));
    const bool h2 = lane & 8;
    float k = h2 ? k1 : k0;
    const float s = h2 ? k0 : k1;
    k = op(k, __shfl_xor_sync(0xffffffffu, s, 8));
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) k = op(k, __shfl_xor_sync(0xffffffffu, k, o));
    return k;  // lanes 0-7: value 0, 8-15: value 1, 16-23: value 2, 24-31: value 3
  } else if constexpr (GP == 2) {
    const bool hi = lane & 16;
    float k = hi ? v[1] : v[0];
    const float s = hi ? v[0] : v[1];
    k = op(k, __shfl_xor_sync(0xffffffffu, s, 16));
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) k = op(k, __shfl_xor_sync(0xffffffffu, k, o));
    return k;  // lanes 0-15: value 0, 16-31: value 1
  } else {
    float k = v[0];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) k = op(k, __shfl_xor_sync(0xffffffffu, k, o));
    return k;
  }
}

template <int GP>
__device__ __forceinline__ void pair_lookup(const float* __restrict__ base, uint32_t code, float (&acc)[GP]) {
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    const uint32_t byte = (code >> (8 * p)) & 255u;
    const float* src = base + (p * 256 + byte) * 32;
    float t[GP];
    if constexpr (GP == 4) {
      const float4 v = *reinterpret_cast<const float4*>(src);
      t[0] = v.x; t[1] = v.y; t[2] = v.z; t[3] = v.w;
    } else if constexpr (GP == 2) {
      const float2 v = *reinterpret_cast<const float2*>(src);
      t[0] = v.x; t[1] = v.y;
    } else {
      t[0] = *src;
    }
#pragma unroll
    for (int g = 0; g < GP; ++g) acc[g] = (p == 0) ? t[g] : __fadd_rn(acc[g], t[g]);
  }
}

template <typename E, int G, bool DUMP>
__global__ void __launch_bounds__(kScanThreads, 1) scan_kernel(const ScanArgs a) {
  using PS = PairShape<G>;
  constexpr int GP = PS::GP;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* tab = reinterpret_cast<float*>(smem_raw);                         // pair tables
  int2* stage = reinterpret_cast<int2*>(tab + PS::kFloats);                // [warps][GP][kWStage] (slot, logit bits)
  __shared__ float lut_s[GP][kM * kC];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int2* wstage = stage + (size_t)warp * GP * kWStage;

  // this CTA's share [g0, g1) of the global unit sequence; streams are walked in order
  long long total = 0;
  for (int s = 0; s < a.S; ++s) {
    const int32_t* st = a.state + (size_t)s * kST;
    total += st[PQHSA_ST_N_UNITS] + (st[PQHSA_ST_N_TAIL] + kUnit - 1) / kUnit;
  }
  const long long g0 = total * blockIdx.x / gridDim.x, g1 = total * (blockIdx.x + 1) / gridDim.x;
  if (g0 >= g1) return;

  long long sbase = 0;  // global index of the first unit of stream s
  for (int s = 0; s < a.S && sbase < g1; ++s) {
    const int32_t* st = a.state + (size_t)s * kST;
    const int n_sorted = st[PQHSA_ST_N_SORTED], n_tail = st[PQHSA_ST_N_TAIL], n_units = st[PQHSA_ST_N_UNITS];
    const int u_tot = n_units + (n_tail + kUnit - 1) / kUnit;
    const long long lo_g = sbase > g0 ? sbase : g0;
    const long long hi_g = sbase + u_tot < g1 ? sbase + u_tot : g1;
    const int u0 = (int)(lo_g - sbase), u1 = (int)(hi_g - sbase);
    sbase += u_tot;
    if (u0 >= u1) continue;

    const uint32_t* codes = a.codes + (size_t)s * a.cap;
    const E* norms = static_cast<const E*>(a.norms) + (size_t)s * a.cap;
    const uint16_t* lids = a.list_ids + (size_t)s * a.cap;

#pragma unroll 1
    for (int pass = 0; pass < PS::NP; ++pass) {
      const int row0 = s * G + pass * GP;  // first query row of this pass
      __syncthreads();                     // the previous tables are no longer in use
      for (int i = tid; i < GP * kM * kC; i += kScanThreads)
        lut_s[i / (kM * kC)][i % (kM * kC)] = a.lut[(size_t)row0 * kM * kC + i];
      __syncthreads();
      // pair tables, replicated: tab[((p * 256 + byte) * REP + rep) * GP + g]
      {
        const int e = tid;  // 4 * 256 entries, one per thread
        const int p = e >> 8;
        const uint32_t byte = e & 255;
        float v[GP];
#pragma unroll
        for (int g = 0; g < GP; ++g) v[g] = pair_entry(lut_s[g], p, byte);
        float* dst = tab + (size_t)e * 32;
#pragma unroll
        for (int rep = 0; rep < PS::REP; ++rep)
#pragma unroll
          for (int g = 0; g < GP; ++g) dst[rep * GP + g] = v[g];
      }
      __syncthreads();

      float tau[GP];
      int cnt[GP];  // staged candidates of this warp, warp-uniform
#pragma unroll
      for (int g = 0; g < GP; ++g) {
        tau[g] = DUMP ? 0.f : a.row_tau[row0 + g];
        cnt[g] = 0;
      }
      const float* lsc = a.list_scores + (size_t)row0 * kLMax;
      const float* mytab = tab + (lane & (PS::REP - 1)) * GP;

      auto flush = [&](int g) {
        __syncwarp();  // the staged entries of all lanes are visible
        int base = 0;
        if (lane == 0) base = atomicAdd(a.row_info + (size_t)(row0 + g) * kRI + PQHSA_RI_NCAND, cnt[g]);
        base = __shfl_sync(0xffffffffu, base, 0);
        for (int i = lane; i < cnt[g]; i += 32) {
          if (base + i < a.ccap) {
            const int2 e = wstage[g * kWStage + i];
            a.cand_slot[(size_t)(row0 + g) * a.ccap + base + i] = e.x;
            a.cand_logit[(size_t)(row0 + g) * a.ccap + base + i] = __int_as_float(e.y);
          }
        }
        __syncwarp();
        cnt[g] = 0;
      };

      for (int u = u0 + warp; u < u1; u += kScanWarps) {
        const bool sorted = u < n_units;
        int lo, hi, l = 0;
        if (sorted) {
          lo = a.unit_off[(size_t)s * (a.ucap + 1) + u];
          hi = a.unit_off[(size_t)s * (a.ucap + 1) + u + 1];
          l = a.unit_list[(size_t)s * a.ucap + u];
        } else {
          lo = n_sorted + (u - n_units) * kUnit;
          hi = min(lo + kUnit, n_sorted + n_tail);
        }
        // all loads of the unit first
        uint32_t code[kIter];
        float kn[kIter];
        int lid[kIter];
#pragma unroll
        for (int it = 0; it < kIter; ++it) {
          const int slot = lo + it * 32 + lane;
          code[it] = 0u;
          kn[it] = 0.f;
          lid[it] = l;
          if (slot < hi) {
            code[it] = __ldg(codes + slot);
            kn[it] = to_f(norms[slot]);
            if (!sorted) lid[it] = lids[slot];
          }
        }
        float ls[GP];
#pragma unroll
        for (int g = 0; g < GP; ++g) ls[g] = __ldg(lsc + g * kLMax + l);

        float xs[kIter][GP];
#pragma unroll
        for (int it = 0; it < kIter; ++it) {
          const int slot = lo + it * 32 + lane;
          const bool valid = slot < hi;
          float acc[GP];
          pair_lookup<GP>(mytab, code[it], acc);
#pragma unroll
          for (int g = 0; g < GP; ++g) {
            const float bias = sorted ? ls[g] : __ldg(lsc + g * kLMax + lid[it]);
            const float x = finish_logit(acc[g], bias, kn[it]);
            xs[it][g] = valid ? x : kNegInf;
            if constexpr (DUMP) {
              if (valid) a.dump[(size_t)(row0 + g) * a.cap + slot] = x;
            } else {
              if (!sorted && valid) a.tail_logit[(size_t)(row0 + g) * a.tail_cap + (slot - n_sorted)] = x;
              const bool pass_tau = valid && x >= tau[g];
              const unsigned m = __ballot_sync(0xffffffffu, pass_tau);
              if (m) {
                const int n_new = __popc(m);
                if (cnt[g] + n_new > kWStage) flush(g);
                if (pass_tau)
                  wstage[g * kWStage + cnt[g] + __popc(m & ((1u << lane) - 1u))] = make_int2(slot, __float_as_int(x));
                cnt[g] += n_new;
              }
            }
          }
        }
        if constexpr (!DUMP) {
          if (sorted) {
            float mx[GP];
#pragma unroll
            for (int g = 0; g < GP; ++g) {
              mx[g] = xs[0][g];
#pragma unroll
              for (int it = 1; it < kIter; ++it) mx[g] = fmaxf(mx[g], xs[it][g]);
            }
            const float mred = warp_reduce_multi<GP, true>(mx, lane);
            float sm[GP];
#pragma unroll
            for (int g = 0; g < GP; ++g) {
              const float mg = __shfl_sync(0xffffffffu, mred, g * (32 / GP));
              sm[g] = 0.f;
#pragma unroll
              for (int it = 0; it < kIter; ++it) sm[g] += unit_term(xs[it][g], mg);  // -inf contributes 0
            }
            const float sred = warp_reduce_multi<GP, false>(sm, lane);
            if ((lane & (32 / GP - 1)) == 0) {
              const int g = lane / (32 / GP);
              a.unit_max[(size_t)(row0 + g) * a.ucap + u] = mred;
              a.unit_sum[(size_t)(row0 + g) * a.ucap + u] = sred;
            }
          }
        }
      }
      if constexpr (!DUMP) {
        __syncwarp();
#pragma unroll
        for (int g = 0; g < GP; ++g)
          if (cnt[g]) flush(g);
      }
    }
  }
}

template <typename E, int G, bool DUMP>
static int launch_scan_t(const pqhsa_params& p, const ScanArgs& a, cudaStream_t st) {
  using PS = PairShape<G>;
  const size_t smem = PS::kFloats * sizeof(float) + (size_t)kScanWarps * PS::GP * kWStage * sizeof(int2);
  auto kern = scan_kernel<E, G, DUMP>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    return check_launch("scan: shared memory opt-in");
  const long long units_hi = (long long)p.num_streams * (p.num_lists + p.max_slots / kUnit + 2);
  long long ctas = sm_count();
  if (ctas > units_hi) ctas = units_hi;
  if (ctas < 1) ctas = 1;
  kern<<<(unsigned)ctas, kScanThreads, smem, st>>>(a);
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
  a.list_scores = reinterpret_cast<const float*>(ws + w.list_scores);
  a.row_tau = reinterpret_cast<const float*>(ws + w.row_tau);
  a.row_info = reinterpret_cast<int32_t*>(ws + w.row_info);
  a.cand_slot = reinterpret_cast<int32_t*>(ws + w.cand_slot);
  a.cand_logit = reinterpret_cast<float*>(ws + w.cand_logit);
  a.unit_max = reinterpret_cast<float*>(ws + w.unit_max);
  a.unit_sum = reinterpret_cast<float*>(ws + w.unit_sum);
  a.tail_logit = reinterpret_cast<float*>(ws + w.tail_logit);
  a.dump = dump;
  a.S = p.num_streams;
  a.cap = p.slot_capacity;
  a.ucap = p.unit_capacity;
  a.tail_cap = w.tail_cap;
  a.ccap = w.ccap;
  if (dump != nullptr) {
    PQHSA_DISPATCH_E(p.dtype, PQHSA_DISPATCH_G(p.group, return (launch_scan_t<E, G, true>(p, a, st))));
  } else {
    PQHSA_DISPATCH_E(p.dtype, PQHSA_DISPATCH_G(p.group, return (launch_scan_t<E, G, false>(p, a, st))));
  }
  return PQHSA_OK;
}

}  // namespace pqhsa
