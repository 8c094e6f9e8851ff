// First two kernels of a decode step.
//
// lut_build_kernel: per-query, per-head table construction, optionally fused with the step's token
// append (raw K/V row write) and the incremental encode of the key that left the local window.  The
// CTAs of a stream take roles by blockIdx.y - list scores for 64 lists each (they also share out the
// byte-pair tables; the first one writes the K/V row), encode - and run side by side; the stream's
// length and its norm bound change once all of them are done (arrival counter, no waiting), the tail
// count is written by the encode CTA, which is the only one that reads it after the start.
//
// For every stream s and query row g:
//   lut[s][g][m][c]      = scale * <q_g restricted to subspace m, codebooks[s][m][c]>
//   list_scores[s][g][l] = scale * <q_g, coarse[s][l]>
// The reference normalises q, scores, and multiplies |q| back
// (pq_hsa/index/ivfpq.py:1061-1118); production folds |q| and the softmax scale
// into the tables (benchmarks/e2e_pq_param_sweep.py:228-249,
// pq_hsa/kernels/cuda/pq_fused_h20.cu:2975-3051), as is done here, in fp32.
// The 8 nibble tables are also folded into the 4 byte-pair tables the scan looks codes up in.
//
// Threshold estimate.  The exact top-K needs the K-th largest of N logits, which is not
// known before the scan.  A stratified sample of 4096 slots of the list-sorted region
// (contiguous records made when the layout was made) is scored by the list CTAs - each the
// sample keys of its own lists, whose scores it has just computed - and their logits go to
// the rows' sample arrays.
//
// tau_kernel (second launch, one CTA per query row) histograms the row's sample logits over their
// own range, walks the histogram from the top and takes as threshold tau the logit below which all
// but r sample keys lie, r = f n + margin * sqrt(f n) + 1 with f = K / N, and as its upper
// companion tau_hi the logit that only f n - margin * sqrt(f n) - 1 sample keys exceed.  The scan
// marks the keys with logit >= tau (about 1.7 K of them); the selection bins them between tau and
// tau_hi, where the K-th largest lies.  Both are only filters: if fewer than K candidates turn up
// (probability ~1e-9 at the default margin of 6 sigma) the selection falls back to all keys, and a
// K-th largest outside [tau, tau_hi] only makes the boundary bin larger, so the result is exact
// either way.
#include "encode.cuh"

namespace pqhsa {

constexpr int kLutThreads = 256;
constexpr int kLutWarps = kLutThreads / 32;
constexpr int kListsPerCta = 64;  // 8 warps x 8 lists: 8 list CTAs + 1 encode CTA per stream at 512 lists
constexpr int kTauThreads = 256;

struct LutArgs {
  const void* q;
  const int32_t* io_map;  // [S] block of q a stream reads, or null: block s
  const void* codebooks;
  const void* coarse;
  int32_t* state;
  const float* norm_max;
  const uint32_t* codes;
  const void* norms;
  const uint16_t* list_ids;
  const int4* sample;  // [S, kSample] (code, norm as float bits, list, slot) of the stratified sample, or null
  const int32_t* sample_start;  // [S, kLMax + 1] first sample record of every list
  float* slog;         // [R, kSample] logits of the sample keys, or null: no threshold wanted
  float* norm_max_rw;
  float* lut;
  float* pair_tab;  // [S, G / GP, 4, 256, GP] byte-pair sums of the tables for the scan, GP = min(G, 4); or null
  float* list_scores;
  float* row_bin;
  float* row_tau;
  int32_t* ticket;
  float2* enc_best;  // [S, 16] nearest list of the key being encoded among each list CTA's lists: (distance, list as int bits)
  int num_lists, cap, G;
  float scale;
  double top_fraction;
  int topk_fixed;
  float margin;
  // fused append (all null / 0 when the kernel only builds tables)
  void* k_base;
  void* v_base;
  const void* new_k;
  const void* new_v;
  KvAddr kv;
  int bump;       // 1: no row is written but the length of a live stream advances (the caller stored the row)
  int list_ctas;  // CTAs per stream with the list-score role
  int encode;     // 1: one more CTA per stream encodes enc.enc_count[s] / enc.uniform_count keys
  EncodeArgs enc;
};

// Sums 32 values per lane across the warp; lane j returns the total of v[j].  Each step exchanges one
// half of the remaining values with the lane `o` away and keeps the other half.
__device__ __forceinline__ float warp_reduce_scatter32(float (&v)[32], int lane) {
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) {
    const bool up = (lane & o) != 0;
#pragma unroll
    for (int i = 0; i < o; ++i) {  // o values stay after this step
      const float keep = up ? v[i + o] : v[i];
      const float send = up ? v[i] : v[i + o];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, o);
    }
  }
  return v[0];
}

template <typename E, int G>
__global__ void __launch_bounds__(kLutThreads, 2) lut_build_kernel(const LutArgs a) {
  __shared__ float qs[G][kD];
  __shared__ float lut_s[G][kM * kC];
  __shared__ float lsc_s[G][kListsPerCta];
  __shared__ EncodeShared<kLutThreads> esh;
  __shared__ int last_list_s;
  const int s = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const E* q = static_cast<const E*>(a.q);
  const bool append = a.new_k != nullptr;
  int32_t* st = a.state + (size_t)s * kST;
  const int seq_old = st[PQHSA_ST_SEQ_LEN];
  const int n_sorted = st[PQHSA_ST_N_SORTED];
  const bool sampling = a.slog != nullptr && n_sorted > kSample;  // shorter streams: every key is a candidate
  const bool is_encode = (int)blockIdx.y >= a.list_ctas;
  const bool bump = a.bump != 0 && seq_old > 0;
  // One key to encode (the usual decode step): the list CTAs share the nearest-list search - each over the lists
  // whose scores it computes anyway - and the one that arrives last among them finishes the key.  More keys: the
  // encode CTA takes them one after the other.
  const int want = a.encode ? (a.enc.enc_count ? a.enc.enc_count[s] : a.enc.uniform_count) : 0;
  const bool shared_encode = want == 1;

  if (is_encode && shared_encode) {
    // nothing to do here: the list CTAs encode the key
  } else if (is_encode) {
    // encode role.  Only tokens that were in the cache when the kernel started are encoded: the row
    // another CTA of this launch is writing is not read (a row the caller stored before the call
    // counts).  A larger norm is parked in norm_pend and folded into norm_max by the last CTA, like
    // the length.
    if (tid == 0) a.enc.norm_max[s] = a.norm_max[s];
    __syncthreads();
    const int n_tail = encode_tokens<E, kLutThreads>(a.enc, s, seq_old + (bump ? 1 : 0));
    if (tid == 0) st[PQHSA_ST_N_TAIL] = n_tail;
  } else {
    const int l0 = blockIdx.y * kListsPerCta;
    // requested before anything else is looked at: this warp's centroid rows (a lane owns 4 dims) ...
    const E* coarse = static_cast<const E*>(a.coarse) + (size_t)s * a.num_lists * kD;
    constexpr int kPerWarp = kListsPerCta / kLutWarps;
    float c[kPerWarp][4];
#pragma unroll
    for (int i = 0; i < kPerWarp; ++i) {
      const int l = l0 + warp * kPerWarp + i;
#pragma unroll
      for (int d = 0; d < 4; ++d) c[i][d] = 0.f;
      if (l < a.num_lists) load4(coarse + (size_t)l * kD + lane * 4, c[i]);
    }
    // ... the thread's code word ...
    float w[kSub];
    if (tid < kM * kC) {
      const E* cw = static_cast<const E*>(a.codebooks) + ((size_t)s * kM * kC + tid) * kSub;
      float x[8], y[8];
      load8(cw, x);
      load8(cw + 8, y);
#pragma unroll
      for (int d = 0; d < 8; ++d) { w[d] = x[d]; w[8 + d] = y[d]; }
    }
    // ... and this CTA's slice of the stream's sample records (sorted by list)
    int i0 = 0, i1 = 0;
    if (sampling && a.sample != nullptr) {
      const int32_t* ss = a.sample_start + (size_t)s * (kLMax + 1);
      i0 = ss[min(l0, a.num_lists)];
      i1 = ss[min(l0 + kListsPerCta, a.num_lists)];
    }
    const int qb = a.io_map != nullptr ? a.io_map[s] : s;  // negative: the stream is idle this step
    for (int i = tid; i < G * kD; i += kLutThreads)
      qs[i / kD][i % kD] = qb >= 0 ? to_f(q[(size_t)qb * G * kD + i]) * a.scale : 0.f;
    __syncthreads();
    // the tables (every list CTA: it scores its share of the sample with them)
    if (tid < kM * kC) {
      const int m = tid / kC;
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float acc = 0.f;
#pragma unroll
        for (int d = 0; d < kSub; ++d) acc = fmaf(qs[g][m * kSub + d], w[d], acc);
        if (blockIdx.y == 0) a.lut[((size_t)s * G + g) * kM * kC + tid] = acc;
        lut_s[g][tid] = acc;
      }
    }
    if (blockIdx.y == 0 && append && tid >= kM * kC && tid < kM * kC + 2 * kD / 8) {
      // the step's K/V row, 16 bytes per thread (elements are 2 or 4 bytes: 8 or 4 per vector)
      constexpr int kVec = 16 / (int)sizeof(E);
      const long long off = a.kv.offset(st[PQHSA_ST_REQ], st[PQHSA_ST_KV_HEAD], seq_old);
      for (int i = tid - kM * kC; i < 2 * kD / kVec; i += 2 * kD / 8) {
        const bool isv = i >= kD / kVec;
        const int e = (isv ? i - kD / kVec : i) * kVec;
        const E* src = static_cast<const E*>(isv ? a.new_v : a.new_k) + (size_t)s * kD + e;
        E* dst = static_cast<E*>(isv ? a.v_base : a.k_base) + off + e;
        *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
      }
    }
    // list scores: one warp per list, kPerWarp x G partial dot products per lane; 32 of them at a time
    // are summed across the warp with 31 shuffles (halving exchange: lane j ends up with the total of
    // value j) instead of 5 per value
    float qr[G][4];
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
      for (int d = 0; d < 4; ++d) qr[g][d] = qs[g][lane * 4 + d];
    constexpr int kVals = kPerWarp * G;
#pragma unroll
    for (int b0 = 0; b0 < kVals; b0 += 32) {
      float v[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int idx = b0 + j;
        v[j] = 0.f;
        if (idx < kVals) {
          const int i = idx / G, g = idx % G;
          float acc = c[i][0] * qr[g][0];
          acc = fmaf(c[i][1], qr[g][1], acc);
          acc = fmaf(c[i][2], qr[g][2], acc);
          v[j] = fmaf(c[i][3], qr[g][3], acc);
        }
      }
      const float tot = warp_reduce_scatter32(v, lane);
      const int idx = b0 + lane;
      if (idx < kVals) {
        const int i = idx / G, g = idx % G;
        const int l = l0 + warp * kPerWarp + i;
        if (l < a.num_lists) {
          a.list_scores[((size_t)s * G + g) * kLMax + l] = tot;
          lsc_s[g][l - l0] = tot;
        }
      }
    }
    __syncthreads();  // tables and list scores of this CTA are in shared memory
    if (a.pair_tab != nullptr) {
      // the scan looks codes up a byte (two subspaces) at a time: entry (p, byte) = lut[2p][byte & 15] +
      // lut[2p+1][byte >> 4]; the list CTAs of a stream write equal shares of the G x 1024 entries
      constexpr int GP = G < 4 ? G : 4;
      float* dst = a.pair_tab + (size_t)s * G * 1024;
      const int per = (G * 1024 + a.list_ctas - 1) / a.list_ctas;
      const int e1 = min(G * 1024, ((int)blockIdx.y + 1) * per);
      for (int i = blockIdx.y * per + tid; i < e1; i += kLutThreads) {
        const int pass = i / (1024 * GP), rem = i % (1024 * GP);
        const int e = rem / GP, g = rem % GP;
        dst[i] = pair_entry(lut_s[pass * GP + g], e >> 8, (uint32_t)(e & 255));
      }
    }
    // the sample keys of this CTA's lists are scored (same arithmetic as the scan)
    for (int i = i0 + tid; i < i1; i += kLutThreads) {
      const int4 v = __ldg(a.sample + (size_t)s * kSample + i);
      const uint32_t code = (uint32_t)v.x;
      const float kn = __int_as_float(v.y);
      const int l = v.z - l0;
#pragma unroll
      for (int g = 0; g < G; ++g)
        a.slog[((size_t)s * G + g) * kSample + i] = finish_logit(pq_sum_row(lut_s[g], code), lsc_s[g][l], kn);
    }
    if (shared_encode) {
      // the key that leaves the local window: position, slot, and whether it can be taken at all (never a token
      // that is not in the cache, never beyond the pool) - the same tests as encode_tokens
      const int n_tail_old = st[PQHSA_ST_N_TAIL];
      const int seq_lim = seq_old + (bump ? 1 : 0);
      const int pos = min(a.enc.sink, seq_lim) + n_sorted + n_tail_old, slot = n_sorted + n_tail_old;
      const bool valid = pos < seq_lim && slot < a.enc.cap && n_tail_old < a.enc.tail_cap;
      if (valid) {  // uniform over the CTA (and over the stream's CTAs)
        const int nl = st[PQHSA_ST_N_LISTS];
        const long long off = a.enc.kv.offset(st[PQHSA_ST_REQ], st[PQHSA_ST_KV_HEAD], pos);
        float vval = 0.f;
        if (tid < kD) vval = to_f(static_cast<const E*>(a.enc.v_base)[off + tid]);
        const float nrm = enc_direction<E, kLutThreads>(static_cast<const E*>(a.enc.k_base), off, esh);
        float bd;
        int bl;
        enc_nearest_list<E, kLutThreads>(coarse, l0, l0 + kListsPerCta, nl, esh, bd, bl);
        if (tid == 0) {
          a.enc_best[(size_t)s * 16 + blockIdx.y] = make_float2(bd, __int_as_float(bl));
          __threadfence();
          const int t = atomicAdd(a.ticket + 2 * s, 1);
          last_list_s = (t == a.list_ctas - 1);
          if (last_list_s) a.ticket[2 * s] = 0;  // ready for the next launch
        }
        __syncthreads();
        if (last_list_s) {
          if (tid == 0) {
            float d0 = __builtin_huge_valf();
            int lw = 0;
            for (int y = 0; y < a.list_ctas; ++y) {  // ascending list ranges: strict < keeps the lowest index on ties
              const float2 b = __ldcg(a.enc_best + (size_t)s * 16 + y);
              if (y * kListsPerCta < nl && b.x < d0) {
                d0 = b.x;
                lw = __float_as_int(b.y);
              }
            }
            esh.list_sh = lw;
            a.enc.norm_max[s] = a.norm_max[s];  // the pending norm bound starts from the stream's
          }
          __syncthreads();
          enc_finish<E, kLutThreads>(a.enc, s, slot, pos, esh.list_sh, nrm, vval, w, esh);
          if (tid == 0) st[PQHSA_ST_N_TAIL] = n_tail_old + 1;
        }
      }
    }
  }

  // ---- counters: the CTA of the stream that arrives last of all.  Every CTA of the stream is then done
  // reading the length: the token written above now counts, a larger norm becomes the stream's bound ----
  if (!append && !a.encode && !bump) return;
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    const int t = atomicAdd(a.ticket + 2 * s + 1, 1);
    if (t == (int)gridDim.y - 1) {
      a.ticket[2 * s + 1] = 0;
      if (append || bump) st[PQHSA_ST_SEQ_LEN] = seq_old + 1;
      if (a.encode) {
        const float pend = __ldcg(a.enc.norm_max + s);
        if (pend > a.norm_max[s]) a.norm_max_rw[s] = pend;
      }
    }
  }
}

// One CTA per query row: the candidate threshold tau and the upper end tau_hi of the selection's bins from
// the row's sample logits (see the file comment).  Runs after lut_build_kernel has ended, so the stream
// counters are final.
template <typename E>
__global__ void __launch_bounds__(kTauThreads) tau_kernel(const LutArgs a) {
  __shared__ uint32_t hist[kBins];
  __shared__ uint32_t wsum[kTauThreads / 32], wmin[kTauThreads / 32], wmax[kTauThreads / 32];
  __shared__ float lut_s[kM * kC];
  __shared__ int bin_lo, bin_hi;
  const int row = blockIdx.x, s = row / a.G;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int32_t* st = a.state + (size_t)s * kST;
  const int n_sorted = st[PQHSA_ST_N_SORTED], n_tail = st[PQHSA_ST_N_TAIL];
  const int n = n_sorted + n_tail;
  const int K = resolve_topk(n, a.top_fraction, a.topk_fixed);
  const int ns = min(kSample, n_sorted);
  const float expect = n > 0 ? (float)K / (float)n * (float)ns : 0.f;
  const float margin = a.margin != 0.f ? a.margin : 6.f;
  const int r = (int)ceilf(expect + margin * sqrtf(expect) + 1.f);
  const int r_hi = (int)floorf(expect - fabsf(margin) * sqrtf(expect)) - 1;
  const bool trivial = K == 0 || n_sorted <= kSample || r >= ns || r < 1;
  if (trivial) {
    // nothing to select, or so few keys (or so large a fraction) that every key is a candidate
    if (tid == 0) {
      a.row_tau[row] = (K == 0) ? __builtin_huge_valf() : kNegInf;
      a.row_bin[2 * row] = 0.f;
      a.row_bin[2 * row + 1] = 0.f;
    }
    return;
  }
  constexpr int kVPT = kSample / kTauThreads;  // sample logits per thread
  constexpr int kBPT = kBins / kTauThreads;    // bins per thread
  uint32_t key[kVPT];
  if (a.sample != nullptr) {
    const float* slog = a.slog + (size_t)row * kSample;
#pragma unroll
    for (int i = 0; i < kVPT; ++i) key[i] = float_key(__ldcg(slog + tid + i * kTauThreads));
  } else {
    // no sample records: the sample slots are gathered from the index and scored here
    if (tid < kM * kC) lut_s[tid] = a.lut[(size_t)row * kM * kC + tid];
    __syncthreads();
    const uint32_t* codes = a.codes + (size_t)s * a.cap;
    const E* norms = static_cast<const E*>(a.norms) + (size_t)s * a.cap;
    const uint16_t* lids = a.list_ids + (size_t)s * a.cap;
#pragma unroll
    for (int i = 0; i < kVPT; ++i) {
      const int slot = (int)((long long)(tid + i * kTauThreads) * n_sorted / ns);
      key[i] = float_key(finish_logit(pq_sum_row(lut_s, __ldg(codes + slot)),
                                      a.list_scores[(size_t)row * kLMax + lids[slot]], to_f(norms[slot])));
    }
  }
  uint32_t mn = key[0], mx = key[0];
#pragma unroll
  for (int i = 1; i < kVPT; ++i) {
    mn = min(mn, key[i]);
    mx = max(mx, key[i]);
  }
  mn = __reduce_min_sync(0xffffffffu, mn);
  mx = __reduce_max_sync(0xffffffffu, mx);
  if (lane == 0) {
    wmin[warp] = mn;
    wmax[warp] = mx;
  }
  for (int i = tid; i < kBins; i += kTauThreads) hist[i] = 0u;
  if (tid == 0) {
    bin_lo = -1;
    bin_hi = -1;
  }
  __syncthreads();
#pragma unroll
  for (int w = 0; w < kTauThreads / 32; ++w) {
    mn = min(mn, wmin[w]);
    mx = max(mx, wmax[w]);
  }
  // linear bins over the row's own range [min, max]
  const float lo = key_float(mn), hi = key_float(mx);
  const float inv_w = hi > lo ? (float)kBins / (hi - lo) : 1.f;
#pragma unroll
  for (int i = 0; i < kVPT; ++i) atomicAdd(&hist[logit_bin(key_float(key[i]), lo, inv_w)], 1u);
  __syncthreads();
  const int top = kBins - kBPT * tid;  // thread j owns the kBPT bins just below
  uint32_t c[kBPT], sum = 0;
#pragma unroll
  for (int b = 0; b < kBPT; ++b) {
    c[b] = hist[top - 1 - b];
    sum += c[b];
  }
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
  // the bin in which the count from the top reaches r (threshold) and r_hi (upper companion)
  const uint32_t needs[2] = {(uint32_t)r, (uint32_t)max(r_hi, 0)};
#pragma unroll
  for (int which = 0; which < 2; ++which) {
    const uint32_t need = needs[which];
    if (need >= 1u && excl < need && need <= incl) {
      uint32_t cum = excl;
#pragma unroll
      for (int b = 0; b < kBPT; ++b) {
        if (cum < need && need <= cum + c[b]) {
          if (which == 0) bin_lo = top - 1 - b; else bin_hi = top - 1 - b;
        }
        cum += c[b];
      }
    }
  }
  __syncthreads();
  if (tid == 0) {
    // one bin of slack for the rounding of the edges; bins 0 and 1 mean "everything"
    const bool all = bin_lo <= 1;
    const float tau = all ? kNegInf : lo + (float)(bin_lo - 1) / inv_w;
    const float tau_hi = bin_hi < 0 ? hi : lo + (float)(bin_hi + 2) / inv_w;
    a.row_tau[row] = tau;
    a.row_bin[2 * row] = all ? 0.f : tau;
    a.row_bin[2 * row + 1] = (!all && tau_hi > tau) ? (float)PQHSA_SELECT_BINS / (tau_hi - tau) : 0.f;
  }
}

static void fill_lut_args(const pqhsa_params& p, const pqhsa_ws_layout& w, const StepAppend* ap, LutArgs& a) {
  char* ws = static_cast<char*>(p.workspace);
  a.q = p.q;
  a.io_map = p.io_map;
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
  a.row_bin = reinterpret_cast<float*>(ws + w.row_bin);
  a.row_tau = reinterpret_cast<float*>(ws + w.row_tau);
  a.ticket = reinterpret_cast<int32_t*>(ws + w.ticket);
  a.enc_best = w.enc_best == (size_t)-1 ? nullptr : reinterpret_cast<float2*>(ws + w.enc_best);
  a.num_lists = p.num_lists;
  a.cap = p.slot_capacity;
  a.G = p.group;
  a.scale = p.scale;
  a.top_fraction = p.top_fraction;
  a.topk_fixed = p.topk_fixed;
  a.margin = p.select_margin;
  a.sample = static_cast<const int4*>(p.sample);
  a.sample_start = static_cast<const int32_t*>(p.sample_start);
  a.slog = w.slog == (size_t)-1 ? nullptr : reinterpret_cast<float*>(ws + w.slog);
  a.norm_max_rw = static_cast<float*>(p.norm_max);
  a.list_ctas = (p.num_lists + kListsPerCta - 1) / kListsPerCta;
  a.k_base = const_cast<void*>(p.k_base);
  a.v_base = const_cast<void*>(p.v_base);
  a.kv = make_kvaddr(p);
  a.new_k = ap ? ap->new_k : nullptr;
  a.new_v = ap ? ap->new_v : nullptr;
  a.bump = (ap && ap->new_k == nullptr && p.external_append != 0) ? 1 : 0;
  a.encode = (ap && (ap->enc_count != nullptr || ap->uniform_count > 0)) ? 1 : 0;
  a.enc = make_encode_args(p, ap ? ap->enc_count : nullptr, ap ? ap->uniform_count : 0);
  a.enc.norm_max = w.norm_pend == (size_t)-1 ? nullptr : reinterpret_cast<float*>(ws + w.norm_pend);
}

template <typename E, int G>
static int launch_lut_build_t(const pqhsa_params& p, const LutArgs& a, cudaStream_t st) {
  const dim3 grid(p.num_streams, a.list_ctas + a.encode);
  lut_build_kernel<E, G><<<grid, kLutThreads, 0, st>>>(a);
  if (int rc = check_launch("lut_build")) return rc;
  if (a.slog == nullptr) return PQHSA_OK;  // tables only: no threshold wanted
  tau_kernel<E><<<p.num_streams * p.group, kTauThreads, 0, st>>>(a);
  return check_launch("tau");
}

int launch_lut_build(const pqhsa_params& p, const pqhsa_ws_layout& w, const StepAppend* ap, cudaStream_t st) {
  LutArgs a;
  fill_lut_args(p, w, ap, a);
  PQHSA_DISPATCH_E(p.dtype, PQHSA_DISPATCH_G(p.group, return (launch_lut_build_t<E, G>(p, a, st))));
  return PQHSA_OK;
}

}  // namespace pqhsa
