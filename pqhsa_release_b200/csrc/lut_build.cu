// First kernel of a decode step: per-query, per-head table construction and the
// candidate-threshold estimate, optionally fused with the step's token append (raw K/V row
// write) and the incremental encode of the key that left the local window.  The CTAs of a
// stream take roles by blockIdx.y - tables, list scores (64 lists each), encode - and run
// side by side; nobody changes a stream counter before every CTA of the stream has arrived,
// so all roles see the same state.
//
// For every stream s and query row g:
//   lut[s][g][m][c]      = scale * <q_g restricted to subspace m, codebooks[s][m][c]>
//   list_scores[s][g][l] = scale * <q_g, coarse[s][l]>
// The reference normalises q, scores, and multiplies |q| back
// (pq_hsa/index/ivfpq.py:1061-1118); production folds |q| and the softmax scale
// into the tables (benchmarks/e2e_pq_param_sweep.py:228-249,
// pq_hsa/kernels/cuda/pq_fused_h20.cu:2975-3051), as is done here, in fp32.
//
// Threshold estimate.  The exact top-K needs the K-th largest of N logits, which
// is not known before the scan.  The CTA of a stream that finishes last (arrival
// counter, no waiting) scores a stratified sample of 4096 slots of the
// list-sorted region, histograms the sample per row and takes as threshold tau
// the logit below which all but r sample keys lie, r = f n + margin * sqrt(f n) + 1
// with f = K / N.  The scan then keeps only keys with logit >= tau as candidates
// (about 2 K of them) and the selection kernel takes the exact top K among them.
// tau is only a filter: if fewer than K candidates turn up (probability ~1e-9 at
// the default margin of 6 sigma) the selection kernel falls back to all keys, so
// the result is exact either way.
#include "encode.cuh"

namespace pqhsa {

constexpr int kLutThreads = 512;
constexpr int kListsPerCta = 64;  // 16 warps x 4 lists

struct LutArgs {
  const void* q;
  const void* codebooks;
  const void* coarse;
  int32_t* state;
  const float* norm_max;
  const uint32_t* codes;
  const void* norms;
  const uint16_t* list_ids;
  const int4* sample;  // [S, kSample] (code, norm as float bits, list, slot) of the stratified sample, or null
  float* lut;
  float* pair_tab;  // [S, G / GP, 4, 256, GP] byte-pair sums of the tables for the scan, GP = min(G, 4); or null
  float* list_scores;
  int32_t* row_info;
  float* row_bin;
  float* row_tau;
  int32_t* ticket;
  int num_lists, cap;
  float scale;
  double top_fraction;
  int topk_fixed;
  float fixed_lo, fixed_inv_w, margin;
  // fused append (all null / 0 when the kernel only builds tables)
  void* k_base;
  void* v_base;
  const void* new_k;
  const void* new_v;
  KvAddr kv;
  int list_ctas;  // CTAs per stream with the list-score role
  int encode;     // 1: one more CTA per stream encodes enc.enc_count[s] / enc.uniform_count keys
  EncodeArgs enc;
};

template <typename E, int G>
__global__ void __launch_bounds__(kLutThreads) lut_build_kernel(const LutArgs a) {
  extern __shared__ uint32_t hist[];  // [G][kBins], used by the last CTA of a stream only
  __shared__ float qs[G][kD];
  __shared__ float sub_max[G][kM];
  __shared__ float lut_s[G][kM * kC];
  __shared__ uint32_t wsum[kLutThreads / 32];
  __shared__ int is_last;
  __shared__ float bin_s[G][2];
  const int s = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const E* q = static_cast<const E*>(a.q);
  const bool append = a.new_k != nullptr;
  const int seq_old = a.state[(size_t)s * kST + PQHSA_ST_SEQ_LEN];

  if ((int)blockIdx.y > a.list_ctas) {
    // encode role: the token just appended counts as part of the stream
    const int n_tail = encode_tokens<E, kLutThreads>(a.enc, s, seq_old + (append ? 1 : 0));
    if (tid == 0) a.state[(size_t)s * kST + PQHSA_ST_N_TAIL] = n_tail;
  } else {
    for (int i = tid; i < G * kD; i += kLutThreads) qs[i / kD][i % kD] = to_f(q[(size_t)s * G * kD + i]) * a.scale;
    __syncthreads();
  }

  if (blockIdx.y == 0) {
    if (a.sample != nullptr) {  // the last CTA of the stream will want the sample: start it towards L2
      const char* sp = reinterpret_cast<const char*>(a.sample + (size_t)s * kSample) + (size_t)tid * 128;
      asm volatile("prefetch.global.L2 [%0];" ::"l"(sp));
    }
    if (append && tid < 2 * kD / 8) {
      // the step's K/V row, 16 bytes per thread (elements are 2 or 4 bytes: 8 or 4 per vector)
      constexpr int kVec = 16 / (int)sizeof(E);
      const int32_t* st = a.state + (size_t)s * kST;
      const long long off = a.kv.offset(st[PQHSA_ST_REQ], st[PQHSA_ST_KV_HEAD], seq_old);
      for (int i = tid; i < 2 * kD / kVec; i += 2 * kD / 8) {
        const bool isv = i >= kD / kVec;
        const int e = (isv ? i - kD / kVec : i) * kVec;
        const E* src = static_cast<const E*>(isv ? a.new_v : a.new_k) + (size_t)s * kD + e;
        E* dst = static_cast<E*>(isv ? a.v_base : a.k_base) + off + e;
        *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
      }
    }
    if (tid < kM * kC) {
      const int m = tid / kC;
      const E* cw = static_cast<const E*>(a.codebooks) + ((size_t)s * kM * kC + tid) * kSub;
      float w[kSub];
      {
        float x[8], y[8];
        load8(cw, x);
        load8(cw + 8, y);
#pragma unroll
        for (int d = 0; d < 8; ++d) { w[d] = x[d]; w[8 + d] = y[d]; }
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float acc = 0.f;
#pragma unroll
        for (int d = 0; d < kSub; ++d) acc = fmaf(qs[g][m * kSub + d], w[d], acc);
        a.lut[((size_t)s * G + g) * kM * kC + tid] = acc;
        lut_s[g][tid] = acc;
        float mx = fabsf(acc);  // max over the 16 code words of this subspace (16 consecutive lanes)
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        if ((tid & (kC - 1)) == 0) sub_max[g][m] = mx;
      }
    }
    __syncthreads();
    if (a.pair_tab != nullptr) {
      // the scan looks codes up a byte (two subspaces) at a time: entry (p, byte) = lut[2p][byte & 15] + lut[2p+1][byte >> 4]
      constexpr int GP = G < 4 ? G : 4;
      float* dst = a.pair_tab + (size_t)s * G * 1024;
      for (int i = tid; i < G * 1024; i += kLutThreads) {
        const int pass = i / (1024 * GP), rem = i % (1024 * GP);
        const int e = rem / GP, g = rem % GP;
        dst[i] = pair_entry(lut_s[pass * GP + g], e >> 8, (uint32_t)(e & 255));
      }
    }
    if (tid < G) {
      // |logit| <= (scale |q| max_l |c_l| + sum_m max_c |lut[m][c]|) * max |k|, |c_l| <= 1: the part
      // that does not depend on the norms is parked here; the last CTA multiplies max |k| in
      // (the encode role may still be raising it)
      float qq = 0.f, pm = 0.f;
      for (int d = 0; d < kD; ++d) qq = fmaf(qs[tid][d], qs[tid][d], qq);
#pragma unroll
      for (int m = 0; m < kM; ++m) pm += sub_max[tid][m];
      a.row_bin[((size_t)s * G + tid) * 2] = sqrtf(qq) + pm;
    }
  } else if ((int)blockIdx.y <= a.list_ctas) {
    // list scores: one warp per list, a lane owns 4 dims
    const int l0 = (blockIdx.y - 1) * kListsPerCta;
    float qr[G][4];
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
      for (int d = 0; d < 4; ++d) qr[g][d] = qs[g][lane * 4 + d];
    const E* coarse = static_cast<const E*>(a.coarse) + (size_t)s * a.num_lists * kD;
    constexpr int kPerWarp = kListsPerCta / (kLutThreads / 32);
    float c[kPerWarp][4];
#pragma unroll
    for (int i = 0; i < kPerWarp; ++i) {
      const int l = l0 + warp * kPerWarp + i;
      if (l < a.num_lists) load4(coarse + (size_t)l * kD + lane * 4, c[i]);
    }
#pragma unroll
    for (int i = 0; i < kPerWarp; ++i) {
      const int l = l0 + warp * kPerWarp + i;
      if (l >= a.num_lists) break;
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float acc = c[i][0] * qr[g][0];
        acc = fmaf(c[i][1], qr[g][1], acc);
        acc = fmaf(c[i][2], qr[g][2], acc);
        acc = fmaf(c[i][3], qr[g][3], acc);
        acc = warp_sum(acc);
        if (lane == 0) a.list_scores[((size_t)s * G + g) * kLMax + l] = acc;
      }
    }
  }

  // ---- the CTA of this stream that arrives last places the candidate thresholds ----
  // (the barrier makes the CTA's stores visible to thread 0, whose fence then publishes them
  //  device-wide before the ticket; the last CTA reads the others' results through L2)
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    const int t = atomicAdd(a.ticket + s, 1);
    is_last = (t == (int)gridDim.y - 1);
    if (is_last) {
      __threadfence();
      a.ticket[s] = 0;  // ready for the next launch
    }
  }
  __syncthreads();
  if (!is_last) return;

  // every CTA of the stream is done: counters may change now; what other CTAs wrote is read through L2
  int32_t* st = a.state + (size_t)s * kST;
  if (append && tid == 0) st[PQHSA_ST_SEQ_LEN] = seq_old + 1;
  const int n_sorted = st[PQHSA_ST_N_SORTED];
  const int n = n_sorted + __ldcg(st + PQHSA_ST_N_TAIL);
  const int K = resolve_topk(n, a.top_fraction, a.topk_fixed);
  if (tid < G) {
    float lo = a.fixed_lo, inv_w = a.fixed_inv_w;
    if (!(a.fixed_inv_w > 0.f)) {
      const float bound = __ldcg(a.row_bin + ((size_t)s * G + tid) * 2) * __ldcg(a.norm_max + s) * 1.0001f;
      lo = -bound;
      inv_w = bound > 1e-30f ? (float)(kBins / 2) / bound : 1.f;
    }
    a.row_bin[((size_t)s * G + tid) * 2] = lo;
    a.row_bin[((size_t)s * G + tid) * 2 + 1] = inv_w;
    bin_s[tid][0] = lo;
    bin_s[tid][1] = inv_w;
    int32_t* ri = a.row_info + ((size_t)s * G + tid) * kRI;
    ri[PQHSA_RI_K] = K;
    ri[PQHSA_RI_N] = n;
    ri[PQHSA_RI_NCAND] = 0;
    ri[PQHSA_RI_NSEL] = 0;
    ri[PQHSA_RI_FALLBACK] = 0;
  }
  const int ns = min(kSample, n_sorted);
  const float expect = n > 0 ? (float)K / (float)n * (float)ns : 0.f;
  const float margin = a.margin != 0.f ? a.margin : 6.f;
  const int r = (int)ceilf(expect + margin * sqrtf(expect) + 1.f);
  if (K == 0 || n_sorted <= kSample || r >= ns || r < 1) {
    // nothing to select, or a context so short that every key is a candidate
    if (tid < G) a.row_tau[(size_t)s * G + tid] = (K == 0) ? __builtin_huge_valf() : kNegInf;
    return;
  }
  for (int i = tid; i < G * kM * kC; i += kLutThreads)
    lut_s[i / (kM * kC)][i % (kM * kC)] = __ldcg(a.lut + (size_t)s * G * kM * kC + i);
  for (int i = tid; i < G * kBins; i += kLutThreads) hist[i] = 0u;
  __syncthreads();
  float lo[G], iw[G];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    lo[g] = bin_s[g][0];
    iw[g] = bin_s[g][1];
  }
  const uint32_t* codes = a.codes + (size_t)s * a.cap;
  const E* norms = static_cast<const E*>(a.norms) + (size_t)s * a.cap;
  const uint16_t* lids = a.list_ids + (size_t)s * a.cap;
  // the 4096 / 512 = 8 samples of a thread: all index loads first, then all list scores
  constexpr int kPer = kSample / kLutThreads;
  uint32_t code[kPer];
  float kn[kPer];
  int li[kPer];
  if (a.sample != nullptr) {
    const int4* rec = a.sample + (size_t)s * kSample;  // the same slots, gathered when the layout was made
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
      const int4 v = __ldg(rec + tid + j * kLutThreads);
      code[j] = (uint32_t)v.x;
      kn[j] = __int_as_float(v.y);
      li[j] = v.z;
    }
  } else {
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
      const int i = tid + j * kLutThreads;
      const int slot = (int)((long long)(i < ns ? i : 0) * n_sorted / ns);
      code[j] = __ldg(codes + slot);
      kn[j] = to_f(norms[slot]);
      li[j] = lids[slot];
    }
  }
  float lsv[kPer][G];
#pragma unroll
  for (int j = 0; j < kPer; ++j)
#pragma unroll
    for (int g = 0; g < G; ++g) lsv[j][g] = __ldcg(a.list_scores + ((size_t)s * G + g) * kLMax + li[j]);
#pragma unroll
  for (int j = 0; j < kPer; ++j) {
    if (tid + j * kLutThreads < ns) {
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float x = finish_logit(pq_sum_row(lut_s[g], code[j]), lsv[j][g], kn[j]);
        atomicAdd(&hist[g * kBins + logit_bin(x, lo[g], iw[g])], 1u);
      }
    }
  }
  __syncthreads();
  // All rows at once: row g is walked by kLutThreads / G threads, thread j of a row owns the
  // kBins / (kLutThreads / G) bins just below 4096 - j * that; find the bin where the count
  // from the top reaches r.
  constexpr int kTPR = kLutThreads / G;  // threads per row (a multiple of 32)
  constexpr int kBPT = kBins / kTPR;     // bins per thread
  const int g = tid / kTPR, j = tid % kTPR;
  const uint32_t* h = hist + g * kBins;
  const int top = kBins - kBPT * j;
  uint32_t sum = 0;
#pragma unroll 8
  for (int b = 0; b < kBPT; ++b) sum += h[top - 1 - b];
  uint32_t incl = sum;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t v = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += v;
  }
  if (lane == 31) wsum[warp] = incl;
  __syncthreads();
  uint32_t before = 0;
  for (int i = g * (kTPR / 32); i < warp; ++i) before += wsum[i];
  incl += before;
  const uint32_t excl = incl - sum, need = (uint32_t)r;
  if (excl < need && need <= incl) {
    uint32_t cum = excl;
    float lo_g = lo[0], iw_g = iw[0];
#pragma unroll
    for (int gg = 1; gg < G; ++gg)
      if (gg == g) { lo_g = lo[gg]; iw_g = iw[gg]; }
    for (int b = top - 1; b >= top - kBPT; --b) {
      const uint32_t c = h[b];
      if (cum < need && need <= cum + c) {
        // one bin of slack for the rounding of the edge; bins 0 and 1 mean "everything"
        a.row_tau[(size_t)s * G + g] = b <= 1 ? kNegInf : lo_g + (float)(b - 1) / iw_g;
      }
      cum += c;
    }
  }
}

template <typename E, int G>
static int launch_lut_build_t(const pqhsa_params& p, const pqhsa_ws_layout& w, const StepAppend* ap, cudaStream_t st) {
  char* ws = static_cast<char*>(p.workspace);
  LutArgs a;
  a.q = p.q;
  a.codebooks = p.codebooks;
  a.coarse = p.coarse;
  a.state = static_cast<int32_t*>(p.state);
  a.norm_max = static_cast<const float*>(p.norm_max);
  a.codes = static_cast<const uint32_t*>(p.codes);
  a.norms = p.norms;
  a.list_ids = static_cast<const uint16_t*>(p.list_ids);
  a.lut = reinterpret_cast<float*>(ws + w.lut);
  a.pair_tab = w.pair_tab == (size_t)-1 ? nullptr : reinterpret_cast<float*>(ws + w.pair_tab);
  a.list_scores = reinterpret_cast<float*>(ws + w.list_scores);
  a.row_info = reinterpret_cast<int32_t*>(ws + w.row_info);
  a.row_bin = reinterpret_cast<float*>(ws + w.row_bin);
  a.row_tau = reinterpret_cast<float*>(ws + w.row_tau);
  a.ticket = reinterpret_cast<int32_t*>(ws + w.ticket);
  a.num_lists = p.num_lists;
  a.cap = p.slot_capacity;
  a.scale = p.scale;
  a.top_fraction = p.top_fraction;
  a.topk_fixed = p.topk_fixed;
  a.fixed_lo = p.hist_lo;
  a.fixed_inv_w = p.hist_inv_width;
  a.margin = p.select_margin;
  a.sample = static_cast<const int4*>(p.sample);
  a.list_ctas = (p.num_lists + kListsPerCta - 1) / kListsPerCta;
  a.k_base = const_cast<void*>(p.k_base);
  a.v_base = const_cast<void*>(p.v_base);
  a.kv = make_kvaddr(p);
  a.new_k = ap ? ap->new_k : nullptr;
  a.new_v = ap ? ap->new_v : nullptr;
  a.encode = (ap && (ap->enc_count != nullptr || ap->uniform_count > 0)) ? 1 : 0;
  a.enc = make_encode_args(p, ap ? ap->enc_count : nullptr, ap ? ap->uniform_count : 0);
  const size_t smem = (size_t)G * kBins * sizeof(uint32_t);
  auto kern = lut_build_kernel<E, G>;
  if (smem > 40 * 1024) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return check_launch("lut_build: shared memory opt-in");
  }
  const dim3 grid(p.num_streams, 1 + a.list_ctas + a.encode);
  kern<<<grid, kLutThreads, smem, st>>>(a);
  return check_launch("lut_build");
}

int launch_lut_build(const pqhsa_params& p, const pqhsa_ws_layout& w, const StepAppend* ap, cudaStream_t st) {
  PQHSA_DISPATCH_E(p.dtype, PQHSA_DISPATCH_G(p.group, return (launch_lut_build_t<E, G>(p, w, ap, st))));
  return PQHSA_OK;
}

}  // namespace pqhsa
