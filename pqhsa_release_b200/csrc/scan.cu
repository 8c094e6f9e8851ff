// 4-bit code scan: streams packed codes and norms once per KV head and scores
// them for all G query rows of the head.
//
//   logit[g][n] = (sum_m lut[g][m][nibble_m(n)] + list_scores[g][list(n)]) * |k_n|
//
// (pq_hsa/kernels/lut_scan.py:92-114 + pq_hsa/index/ivfpq.py:1084-1118; the
// production kernel it replaces is pq_hsa/kernels/triton_lut_scan_h20.py:1197-1291.)
//
// Layout and work split.  The sorted region of a stream is cut into units of at
// most 128 consecutive slots of ONE list, so the list score is a warp-uniform
// register and the per-list log-sum-exp is a warp reduction with no atomics.  A
// warp takes one unit at a time; lanes take consecutive slots (coalesced 4-byte
// code and 2-byte norm loads).  Slots of the unsorted tail carry their own list
// id and are scored in the same launch; their logits are kept individually.
//
// Table lookups.  The 8x16 table of the G rows lives in shared memory as
// vectors of W = min(G, 4) floats, replicated 32 / W times so that lane j of a
// quarter (half, full) warp reads replica j: every LDS.128 (.64, .32) then hits
// distinct banks whatever the codes are, i.e. the scan runs at the shared-memory
// bandwidth of G*32 bytes per key with no bank conflicts.
//
// Outputs per query row (select mode): the 12-bit histogram bin of every slot
// (uint16, dense), the row's bin histogram (shared-memory atomics, flushed once
// per CTA), per-unit (max, sum exp) and the tail logits.  The logits themselves
// are never written.  A unit's <= 4 logits per lane stay in registers, so the sum
// is taken against the unit's final maximum: each key contributes exactly
// unit_term(logit, max), which the attend kernel can reproduce bit for bit when
// it removes a selected key from its unit (no cancellation error).  Dump mode writes the fp32 logits instead (tests, and the
// stand-alone scoring entry point).
#include "common.cuh"

namespace pqhsa {

constexpr int kScanThreads = 512;

template <int G> struct LutShape {
  static constexpr int W = G < 4 ? G : 4;       // floats per lookup vector
  static constexpr int P = G / W;               // planes (lookups per table entry)
  static constexpr int REP = 32 / W;            // replicas
  static constexpr int kFloats = P * kM * kC * 32;  // = P * 4096
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
  uint16_t* bins;
  uint32_t* hist;
  float* unit_max;
  float* unit_sum;
  float* tail_logit;
  float* dump;
  const float* row_bin;
  int cap, ucap, tail_cap;
};

template <int G>
__device__ __forceinline__ void lookup_all(const float* __restrict__ lutrep, uint32_t code, int lane,
                                           float (&acc)[G]) {
  using S = LutShape<G>;
  const int rep = lane & (S::REP - 1);
#pragma unroll
  for (int m = 0; m < kM; ++m) {
    const int entry = m * kC + ((code >> (4 * m)) & 15u);
#pragma unroll
    for (int pl = 0; pl < S::P; ++pl) {
      const float* src = lutrep + (((pl * kM * kC + entry) * S::REP + rep) * S::W);
      float t[S::W];
      if constexpr (S::W == 4) {
        const float4 v = *reinterpret_cast<const float4*>(src);
        t[0] = v.x; t[1] = v.y; t[2] = v.z; t[3] = v.w;
      } else if constexpr (S::W == 2) {
        const float2 v = *reinterpret_cast<const float2*>(src);
        t[0] = v.x; t[1] = v.y;
      } else {
        t[0] = *src;
      }
#pragma unroll
      for (int w = 0; w < S::W; ++w) {
        const int g = pl * S::W + w;
        acc[g] = (m == 0) ? t[w] : __fadd_rn(acc[g], t[w]);
      }
    }
  }
}

template <typename E, int G, bool DUMP>
__global__ void __launch_bounds__(kScanThreads) scan_kernel(const ScanArgs a) {
  using S = LutShape<G>;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* lutrep = reinterpret_cast<float*>(smem_raw);
  uint32_t* shist = reinterpret_cast<uint32_t*>(lutrep + S::kFloats);

  const int s = blockIdx.y;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int32_t* st = a.state + (size_t)s * kST;
  const int n_sorted = st[PQHSA_ST_N_SORTED], n_tail = st[PQHSA_ST_N_TAIL], n_units = st[PQHSA_ST_N_UNITS];
  const int u_tot = n_units + (n_tail + kUnit - 1) / kUnit;
  const int u0 = (int)((long long)u_tot * blockIdx.x / gridDim.x);
  const int u1 = (int)((long long)u_tot * (blockIdx.x + 1) / gridDim.x);
  if (u0 >= u1) return;

  // replicated table: [plane][entry][replica][w]
  for (int i = tid; i < S::kFloats; i += kScanThreads) {
    const int w = i % S::W;
    const int entry = (i / (S::W * S::REP)) % (kM * kC);
    const int pl = i / (S::W * S::REP * kM * kC);
    lutrep[i] = a.lut[((size_t)s * G + pl * S::W + w) * (kM * kC) + entry];
  }
  if constexpr (!DUMP) {
    uint4* h4 = reinterpret_cast<uint4*>(shist);
    for (int i = tid; i < G * kBins / 4; i += kScanThreads) h4[i] = make_uint4(0u, 0u, 0u, 0u);
  }
  __syncthreads();

  const uint32_t* codes = a.codes + (size_t)s * a.cap;
  const E* norms = static_cast<const E*>(a.norms) + (size_t)s * a.cap;
  const float* lsc = a.list_scores + (size_t)s * G * kLMax;

  for (int u = u0 + warp; u < u1; u += kScanThreads / 32) {
    if (u < n_units) {
      const int lo = a.unit_off[(size_t)s * (a.ucap + 1) + u];
      const int hi = a.unit_off[(size_t)s * (a.ucap + 1) + u + 1];
      const int l = a.unit_list[(size_t)s * a.ucap + u];
      float ls[G], lo_b[G], iw_b[G];
#pragma unroll
      for (int g = 0; g < G; ++g) {
        ls[g] = __ldg(lsc + g * kLMax + l);
        if constexpr (!DUMP) {
          lo_b[g] = a.row_bin[((size_t)s * G + g) * 2];
          iw_b[g] = a.row_bin[((size_t)s * G + g) * 2 + 1];
        }
      }
      constexpr int kIter = kUnit / 32;
      float xs[kIter][G];
#pragma unroll
      for (int it = 0; it < kIter; ++it) {
        const int slot = lo + it * 32 + lane;
        if (slot < hi) {
          const uint32_t code = __ldg(codes + slot);
          const float kn = to_f(norms[slot]);
          float acc[G];
          lookup_all<G>(lutrep, code, lane, acc);
#pragma unroll
          for (int g = 0; g < G; ++g) {
            const float x = finish_logit(acc[g], ls[g], kn);
            xs[it][g] = x;
            if constexpr (DUMP) {
              a.dump[((size_t)s * G + g) * a.cap + slot] = x;
            } else {
              const int b = logit_bin(x, lo_b[g], iw_b[g]);
              a.bins[((size_t)s * G + g) * a.cap + slot] = (uint16_t)b;
              atomicAdd(&shist[g * kBins + b], 1u);
            }
          }
        } else {
#pragma unroll
          for (int g = 0; g < G; ++g) xs[it][g] = kNegInf;
        }
      }
      if constexpr (!DUMP) {
#pragma unroll
        for (int g = 0; g < G; ++g) {
          float mx = xs[0][g];
#pragma unroll
          for (int it = 1; it < kIter; ++it) mx = fmaxf(mx, xs[it][g]);
          mx = warp_max(mx);
          float sm = 0.f;
#pragma unroll
          for (int it = 0; it < kIter; ++it) sm += unit_term(xs[it][g], mx);  // -inf contributes 0
          sm = warp_sum(sm);
          if (lane == 0) {
            a.unit_max[((size_t)s * G + g) * a.ucap + u] = mx;
            a.unit_sum[((size_t)s * G + g) * a.ucap + u] = sm;
          }
        }
      }
    } else {
      // a chunk of the unsorted tail: every slot has its own list
      const uint16_t* lids = a.list_ids + (size_t)s * a.cap;
      const int t0 = (u - n_units) * kUnit;
      const int t1 = min(t0 + kUnit, n_tail);
      for (int t = t0 + lane; t < t1; t += 32) {
        const int slot = n_sorted + t;
        const uint32_t code = __ldg(codes + slot);
        const float kn = to_f(norms[slot]);
        const int l = lids[slot];
        float acc[G];
        lookup_all<G>(lutrep, code, lane, acc);
#pragma unroll
        for (int g = 0; g < G; ++g) {
          const float x = finish_logit(acc[g], __ldg(lsc + g * kLMax + l), kn);
          if constexpr (DUMP) {
            a.dump[((size_t)s * G + g) * a.cap + slot] = x;
          } else {
            const int b = logit_bin(x, a.row_bin[((size_t)s * G + g) * 2], a.row_bin[((size_t)s * G + g) * 2 + 1]);
            a.bins[((size_t)s * G + g) * a.cap + slot] = (uint16_t)b;
            atomicAdd(&shist[g * kBins + b], 1u);
            a.tail_logit[((size_t)s * G + g) * a.tail_cap + t] = x;
          }
        }
      }
    }
  }

  if constexpr (!DUMP) {
    __syncthreads();
    for (int i = tid; i < G * kBins; i += kScanThreads) {
      const uint32_t v = shist[i];
      if (v) atomicAdd(a.hist + (size_t)s * G * kBins + i, v);
    }
  }
}

static int g_sm_count = 0;
int sm_count() {
  if (g_sm_count == 0) {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    g_sm_count = n;
  }
  return g_sm_count;
}

template <typename E, int G, bool DUMP>
static int launch_scan_t(const pqhsa_params& p, const ScanArgs& a, cudaStream_t st) {
  using S = LutShape<G>;
  const size_t smem = S::kFloats * sizeof(float) + (DUMP ? 0 : (size_t)G * kBins * sizeof(uint32_t));
  auto kern = scan_kernel<E, G, DUMP>;
  if (smem > 48 * 1024) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return check_launch("scan: shared memory opt-in");
  }
  const int per_sm = smem > 110 * 1024 ? 1 : 2;
  const int units_hi = p.num_lists + p.max_slots / kUnit + 1;
  int ctas = (sm_count() * per_sm + p.num_streams - 1) / p.num_streams;
  ctas = ctas > units_hi ? units_hi : ctas;
  ctas = ctas < 1 ? 1 : ctas;
  kern<<<dim3(ctas, p.num_streams), kScanThreads, smem, st>>>(a);
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
  a.bins = reinterpret_cast<uint16_t*>(ws + w.bins);
  a.hist = reinterpret_cast<uint32_t*>(ws + w.hist);
  a.unit_max = reinterpret_cast<float*>(ws + w.unit_max);
  a.unit_sum = reinterpret_cast<float*>(ws + w.unit_sum);
  a.tail_logit = reinterpret_cast<float*>(ws + w.tail_logit);
  a.dump = dump;
  a.cap = p.slot_capacity;
  a.ucap = p.unit_capacity;
  a.tail_cap = w.tail_cap;
  a.row_bin = reinterpret_cast<const float*>(ws + w.row_bin);
  if (dump != nullptr) {
    PQHSA_DISPATCH_E(p.dtype, PQHSA_DISPATCH_G(p.group, return (launch_scan_t<E, G, true>(p, a, st))));
  } else {
    PQHSA_DISPATCH_E(p.dtype, PQHSA_DISPATCH_G(p.group, return (launch_scan_t<E, G, false>(p, a, st))));
  }
  return PQHSA_OK;
}

}  // namespace pqhsa
