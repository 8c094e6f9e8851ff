// First kernel of a decode step.
//
// lut_build_kernel: per-query-row table construction and threshold estimate, optionally fused with the step's
// token append (raw K/V row write) and the incremental encode of the key that left the local window.  The CTAs
// of a stream take roles by blockIdx.y - the encode CTA first (the longest chain of the kernel), then one CTA per
// query row - and run side by side without waiting for one another: a row CTA needs nothing from the others.  The
// stream's length and its norm bound change once all of them are done (arrival counter), the tail count is written
// by the encode CTA at its very end.
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
// A row CTA streams the stream's centroid rows (128 KB at 512 lists in 16-bit elements) and then the sample
// records (64 KB) through a ring of three 32 KB stages in shared memory with 16-byte asynchronous copies, three
// chunks in flight: the list scores are computed from the stage (two threads per centroid row, pieces placed so
// that the reads are free of bank conflicts) and kept in shared memory, the sample keys are scored from them
// as their chunks land, and their logits never leave the registers.  The G row CTAs of a stream read the same
// rows: one of them brings them in from HBM, the others find them in L2.
//
// Threshold estimate.  The exact top-K needs the K-th largest of N logits, which is not
// known before the scan.  A stratified sample of 4096 slots of the list-sorted region
// (contiguous records made when the layout was made) is scored by the row's CTA, which histograms
// the logits over their own range, walks the histogram from the top and takes as threshold tau the
// logit below which all but r sample keys lie, r = f n + margin * sqrt(f n) + 1 with f = K / N, and as its
// upper companion tau_hi the logit that only f n - margin * sqrt(f n) - 1 sample keys exceed.  The scan
// marks the keys with logit >= tau (about 1.7 K of them); the selection bins them between tau and
// tau_hi, where the K-th largest lies.  Both are only filters: if fewer than K candidates turn up
// (probability ~1e-9 at the default margin of 6 sigma) the selection falls back to all keys, and a
// K-th largest outside [tau, tau_hi] only makes the boundary bin larger, so the result is exact
// either way.
//
// tau_kernel (a second launch, only for an index without sample records) gathers and scores the sample slots
// itself, one CTA per query row.
#include "encode.cuh"

namespace pqhsa {

constexpr int kLutThreads = 256;
constexpr int kLutWarps = kLutThreads / 32;
constexpr int kRingStages = 3;
constexpr int kStageBytes = 32768;

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
  int encode;     // 1: one more CTA per stream encodes enc.enc_count[s] / enc.uniform_count keys
  EncodeArgs enc;
};

// Scratch of the threshold placement of one row by one CTA of kLutThreads threads.
struct TauScratch {
  uint32_t hist[kBins];
  uint32_t wsum[kLutWarps], wmin[kLutWarps], wmax[kLutWarps];
  int bin_lo, bin_hi;
};
constexpr int kTauPer = kSample / kLutThreads;  // sample logits per thread

// Thresholds of a row from the kSample sample logits its CTA holds in registers (as ordered keys): a 2048-bin histogram
// over the sample's own range is walked from the top; tau is the lower edge of the bin where the count reaches r (one
// bin of slack), tau_hi the upper edge of the bin where it reaches r_hi.  n = the stream's key count this step.  All
// threads of the CTA call.
__device__ __forceinline__ void place_thresholds(const LutArgs& a, int row, int n_sorted, int n,
                                                 const uint32_t (&key)[kTauPer], TauScratch& sh) {
  constexpr int kBPT = kBins / kLutThreads;  // bins per thread
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int K = resolve_topk(n, a.top_fraction, a.topk_fixed);
  const int ns = min(kSample, n_sorted);
  const float expect = n > 0 ? (float)K / (float)n * (float)ns : 0.f;
  const float margin = a.margin != 0.f ? a.margin : 6.f;
  const int r = (int)ceilf(expect + margin * sqrtf(expect) + 1.f);
  const int r_hi = (int)floorf(expect - fabsf(margin) * sqrtf(expect)) - 1;
  if (K == 0 || r >= ns || r < 1) {
    // nothing to select, or so large a fraction that every key is a candidate
    if (tid == 0) {
      a.row_tau[row] = (K == 0) ? __builtin_huge_valf() : kNegInf;
      a.row_bin[2 * row] = 0.f;
      a.row_bin[2 * row + 1] = 0.f;
    }
    return;
  }
  uint32_t mn = key[0], mx = key[0];
#pragma unroll
  for (int i = 1; i < kTauPer; ++i) {
    mn = min(mn, key[i]);
    mx = max(mx, key[i]);
  }
  mn = __reduce_min_sync(0xffffffffu, mn);
  mx = __reduce_max_sync(0xffffffffu, mx);
  if (lane == 0) {
    sh.wmin[warp] = mn;
    sh.wmax[warp] = mx;
  }
  for (int i = tid; i < kBins; i += kLutThreads) sh.hist[i] = 0u;
  if (tid == 0) {
    sh.bin_lo = -1;
    sh.bin_hi = -1;
  }
  __syncthreads();
  mn = __reduce_min_sync(0xffffffffu, sh.wmin[lane & (kLutWarps - 1)]);
  mx = __reduce_max_sync(0xffffffffu, sh.wmax[lane & (kLutWarps - 1)]);
  // linear bins over the row's own range [min, max]
  const float lo = key_float(mn), hi = key_float(mx);
  const float inv_w = hi > lo ? (float)kBins / (hi - lo) : 1.f;
#pragma unroll
  for (int i = 0; i < kTauPer; ++i) atomicAdd(&sh.hist[logit_bin(key_float(key[i]), lo, inv_w)], 1u);
  __syncthreads();
  const int top = kBins - kBPT * tid;  // thread j owns the kBPT bins just below
  uint32_t c[kBPT], sum = 0;
#pragma unroll
  for (int b = 0; b < kBPT; ++b) {
    c[b] = sh.hist[top - 1 - b];
    sum += c[b];
  }
  uint32_t incl = sum;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t v = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += v;
  }
  if (lane == 31) sh.wsum[warp] = incl;
  __syncthreads();
  incl += __reduce_add_sync(0xffffffffu, lane < warp ? sh.wsum[lane & (kLutWarps - 1)] : 0u);
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
          if (which == 0) sh.bin_lo = top - 1 - b; else sh.bin_hi = top - 1 - b;
        }
        cum += c[b];
      }
    }
  }
  __syncthreads();
  if (tid == 0) {
    // one bin of slack for the rounding of the edges; bins 0 and 1 mean "everything"
    const bool all = sh.bin_lo <= 1;
    const float tau = all ? kNegInf : lo + (float)(sh.bin_lo - 1) / inv_w;
    const float tau_hi = sh.bin_hi < 0 ? hi : lo + (float)(sh.bin_hi + 2) / inv_w;
    a.row_tau[row] = tau;
    a.row_bin[2 * row] = all ? 0.f : tau;
    a.row_bin[2 * row + 1] = (!all && tau_hi > tau) ? (float)PQHSA_SELECT_BINS / (tau_hi - tau) : 0.f;
  }
}

// 16 bytes of a centroid row as floats
template <typename E> struct Piece {
  static constexpr int kDims = 16 / (int)sizeof(E);
  static __device__ __forceinline__ void unpack(const uint4& r, float (&v)[kDims]) {
    if constexpr (sizeof(E) == 2) {
      unpack8(r, static_cast<const E*>(nullptr), v);
    } else {
      v[0] = __uint_as_float(r.x);
      v[1] = __uint_as_float(r.y);
      v[2] = __uint_as_float(r.z);
      v[3] = __uint_as_float(r.w);
    }
  }
};

struct LutShared {
  float q[kD];  // the query row times the softmax scale
  float lut[kM * kC];
  float lsc[kLMax];
  TauScratch tau;
};

template <typename E>
__global__ void __launch_bounds__(kLutThreads, 2) lut_build_kernel(const LutArgs a) {
  extern __shared__ __align__(16) unsigned char ring[];  // kRingStages x kStageBytes
  __shared__ LutShared sh;
  const int s = blockIdx.x, G = a.G;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const bool append = a.new_k != nullptr;
  int32_t* st = a.state + (size_t)s * kST;
  const int seq_old = st[PQHSA_ST_SEQ_LEN];
  const int n_sorted = st[PQHSA_ST_N_SORTED];
  const int n_tail_old = st[PQHSA_ST_N_TAIL];  // the encode CTA rewrites it at its very end
  const bool is_encode = a.encode != 0 && blockIdx.y == 0;  // first in launch order: the longest chain of the kernel
  const bool bump = a.bump != 0 && seq_old > 0;
  const int want = a.encode ? (a.enc.enc_count ? a.enc.enc_count[s] : a.enc.uniform_count) : 0;

  if (is_encode) {
    // encode role.  Only tokens that were in the cache when the kernel started are encoded: the row
    // another CTA of this launch is writing is not read (a row the caller stored before the call
    // counts).  A larger norm is parked in norm_pend and folded into norm_max by the last CTA, like
    // the length.
    if (tid == 0) a.enc.norm_max[s] = a.norm_max[s];
    __syncthreads();
    const int n_tail = encode_tokens<E, kLutThreads>(a.enc, s, seq_old + (bump ? 1 : 0));
    if (tid == 0) st[PQHSA_ST_N_TAIL] = n_tail;
  } else {
    const int g = (int)blockIdx.y - a.encode, row = s * G + g;
    const bool want_tau = a.slog != nullptr && a.sample != nullptr;
    const bool sampling = want_tau && n_sorted > kSample;  // shorter streams: every key is a candidate
    // ---- the stream of 32 KB chunks through the ring: the centroid rows, then the sample records ----
    constexpr int kRowBytes = kD * (int)sizeof(E);
    constexpr int kPPR = kRowBytes / 16;           // 16-byte pieces per centroid row
    constexpr int kLPS = kStageBytes / kRowBytes;  // centroid rows per chunk
    constexpr int kPPT = kPPR / 2;                 // pieces per thread: two threads share a row, one the even pieces, one the odd
    constexpr int kDPP = Piece<E>::kDims;
    constexpr int kRecPerChunk = kStageBytes / 16;
    constexpr int kSampleChunks = kSample / kRecPerChunk;
    static_assert(2 * kLPS <= kLutThreads && kSample % kRecPerChunk == 0 && kRecPerChunk % kLutThreads == 0, "chunk shape");
    const unsigned char* coarse = static_cast<const unsigned char*>(a.coarse) + (size_t)s * a.num_lists * kRowBytes;
    const int4* sample = a.sample + (size_t)s * kSample;
    const int nc = (a.num_lists + kLPS - 1) / kLPS;
    const int total = nc + (sampling ? kSampleChunks : 0);
    auto issue = [&](int c) {
      if (c < total) {
        unsigned char* stage = ring + (size_t)(c % kRingStages) * kStageBytes;
        if (c < nc) {
          // piece P of the chunk's row l sits at piece slot P ^ ((l & 3) << 1) of the row: the eight threads of a
          // quarter warp (four rows, even and odd pieces) then read eight different 16-byte bank groups
          const int rows = min(kLPS, a.num_lists - c * kLPS);
          const unsigned char* src = coarse + (size_t)c * kStageBytes;
          for (int i = tid; i < rows * kPPR; i += kLutThreads) {
            const int l = i / kPPR, P = i % kPPR;
            cp_async16(stage + l * kRowBytes + ((P ^ ((l & 3) << 1)) << 4), src + (size_t)i * 16);
          }
        } else {
          const int4* src = sample + (size_t)(c - nc) * kRecPerChunk;
          for (int i = tid; i < kRecPerChunk; i += kLutThreads) cp_async16(stage + i * 16, src + i);
        }
      }
      cp_async_commit();  // one group per chunk slot, empty or not: the waits count groups
    };
#pragma unroll
    for (int c = 0; c < kRingStages; ++c) issue(c);
    // ---- the row's tables while the first chunks travel ----
    float w[kSub];
    if (tid < kM * kC) {
      const E* cw = static_cast<const E*>(a.codebooks) + ((size_t)s * kM * kC + tid) * kSub;
      float x[8], y[8];
      load8(cw, x);
      load8(cw + 8, y);
#pragma unroll
      for (int d = 0; d < 8; ++d) { w[d] = x[d]; w[8 + d] = y[d]; }
    }
    const int qb = a.io_map != nullptr ? a.io_map[s] : s;  // negative: the stream is idle this step
    if (tid < kD) sh.q[tid] = qb >= 0 ? to_f(static_cast<const E*>(a.q)[((size_t)qb * G + g) * kD + tid]) * a.scale : 0.f;
    if (g == 0 && append && tid >= kM * kC && tid < kM * kC + 2 * kD / 8) {
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
    __syncthreads();
    if (tid < kM * kC) {
      const int m = tid / kC;
      float acc = 0.f;
#pragma unroll
      for (int d = 0; d < kSub; ++d) acc = fmaf(sh.q[m * kSub + d], w[d], acc);
      a.lut[(size_t)row * kM * kC + tid] = acc;
      sh.lut[tid] = acc;
    }
    // this thread's half of the query row: the dims of the even (h = 0) or odd (h = 1) pieces of a centroid row
    const int h = tid & 1, ll = tid >> 1;
    float qh[kD / 2];
#pragma unroll
    for (int k = 0; k < kPPT; ++k)
#pragma unroll
      for (int e = 0; e < kDPP; ++e) qh[k * kDPP + e] = sh.q[(2 * k + h) * kDPP + e];
    __syncthreads();
    if (a.pair_tab != nullptr) {
      // the scan looks codes up a byte (two subspaces) at a time: entry (p, byte) = lut[2p][byte & 15] +
      // lut[2p+1][byte >> 4], the rows of a group of min(G, 4) interleaved
      const int GP = G < 4 ? G : 4;
      float* dst = a.pair_tab + (size_t)s * G * 1024 + (size_t)(g / GP) * 1024 * GP + (g % GP);
      for (int e = tid; e < 1024; e += kLutThreads) dst[(size_t)e * GP] = pair_entry(sh.lut, e >> 8, (uint32_t)(e & 255));
    }
    // ---- list scores: two threads per centroid row of the chunk ----
    for (int c = 0; c < nc; ++c) {
      cp_async_wait<kRingStages - 1>();
      __syncthreads();  // every thread's pieces of chunk c have landed
      const unsigned char* stage = ring + (size_t)(c % kRingStages) * kStageBytes;
      const int l = c * kLPS + ll;
      const bool valid = ll < kLPS && l < a.num_lists;
      float dot = 0.f;
      if (valid) {
        const unsigned char* rowp = stage + ll * kRowBytes;
        const int sw = (ll & 3) << 1;
#pragma unroll
        for (int k = 0; k < kPPT; ++k) {
          float cv[kDPP];
          Piece<E>::unpack(*reinterpret_cast<const uint4*>(rowp + (((2 * k + h) ^ sw) << 4)), cv);
#pragma unroll
          for (int e = 0; e < kDPP; ++e) dot = fmaf(cv[e], qh[k * kDPP + e], dot);
        }
      }
      dot += __shfl_xor_sync(0xffffffffu, dot, 1);
      if (valid && h == 0) {
        sh.lsc[l] = dot;
        a.list_scores[(size_t)row * kLMax + l] = dot;
      }
      __syncthreads();  // the stage is free again
      issue(c + kRingStages);
    }
    // ---- the sample keys are scored (same arithmetic as the scan) and the thresholds placed ----
    if (sampling) {
      constexpr int kPer = kRecPerChunk / kLutThreads;
      uint32_t key[kSampleChunks * kPer];
#pragma unroll
      for (int j = 0; j < kSampleChunks; ++j) {
        cp_async_wait<kRingStages - 1>();
        __syncthreads();  // the chunk has landed; the first time round also: all list scores are in shared memory
        const int4* rec = reinterpret_cast<const int4*>(ring + (size_t)((nc + j) % kRingStages) * kStageBytes);
#pragma unroll
        for (int i = 0; i < kPer; ++i) {
          const int4 v = rec[tid + i * kLutThreads];
          key[j * kPer + i] = float_key(finish_logit(pq_sum_row(sh.lut, (uint32_t)v.x), sh.lsc[v.z], __int_as_float(v.y)));
        }
        __syncthreads();
        issue(nc + j + kRingStages);
      }
      // the encode role may still be running: its effect on the key count follows from the counters as they
      // were when the kernel started (tau is only a filter: the selection takes K from the final counters)
      int added = 0;
      if (a.encode) {
        const int seq_new = seq_old + ((append || bump) ? 1 : 0);
        const int room_seq = seq_new - (min(a.enc.sink, seq_new) + n_sorted + n_tail_old);
        added = max(0, min(min(want, room_seq), min(a.enc.cap - (n_sorted + n_tail_old), a.enc.tail_cap - n_tail_old)));
      }
      place_thresholds(a, row, n_sorted, n_sorted + n_tail_old + added, key, sh.tau);
    } else if (want_tau && tid == 0) {
      // so few keys that every key is a candidate (or nothing to select)
      const int K = resolve_topk(n_sorted + n_tail_old, a.top_fraction, a.topk_fixed);
      a.row_tau[row] = (K == 0) ? __builtin_huge_valf() : kNegInf;
      a.row_bin[2 * row] = 0.f;
      a.row_bin[2 * row + 1] = 0.f;
    }
    cp_async_wait<0>();
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

// One CTA per query row, for an index without sample records: the sample slots are gathered from the index, scored,
// and the thresholds placed as above.  Runs after lut_build_kernel has ended, so the stream counters are final.
template <typename E>
__global__ void __launch_bounds__(kLutThreads) tau_kernel(const LutArgs a) {
  __shared__ TauScratch tsh;
  __shared__ float lut_s[kM * kC];
  const int row = blockIdx.x, s = row / a.G;
  const int tid = threadIdx.x;
  const int32_t* st = a.state + (size_t)s * kST;
  const int n_sorted = st[PQHSA_ST_N_SORTED], n_tail = st[PQHSA_ST_N_TAIL];
  const int n = n_sorted + n_tail;
  if (n_sorted <= kSample) {
    // so few keys that every key is a candidate (or nothing to select)
    if (tid == 0) {
      a.row_tau[row] = resolve_topk(n, a.top_fraction, a.topk_fixed) == 0 ? __builtin_huge_valf() : kNegInf;
      a.row_bin[2 * row] = 0.f;
      a.row_bin[2 * row + 1] = 0.f;
    }
    return;
  }
  if (tid < kM * kC) lut_s[tid] = a.lut[(size_t)row * kM * kC + tid];
  __syncthreads();
  const uint32_t* codes = a.codes + (size_t)s * a.cap;
  const E* norms = static_cast<const E*>(a.norms) + (size_t)s * a.cap;
  const uint16_t* lids = a.list_ids + (size_t)s * a.cap;
  uint32_t key[kTauPer];
#pragma unroll
  for (int i = 0; i < kTauPer; ++i) {
    const int slot = (int)((long long)(tid + i * kLutThreads) * n_sorted / kSample);
    key[i] = float_key(finish_logit(pq_sum_row(lut_s, __ldg(codes + slot)),
                                    a.list_scores[(size_t)row * kLMax + lids[slot]], to_f(norms[slot])));
  }
  place_thresholds(a, row, n_sorted, n, key, tsh);
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

template <typename E>
static int launch_lut_build_t(const pqhsa_params& p, const LutArgs& a, cudaStream_t st) {
  const dim3 grid(p.num_streams, p.group + a.encode);
  constexpr size_t smem = (size_t)kRingStages * kStageBytes;
  auto kern = lut_build_kernel<E>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    return check_launch("lut_build: shared memory opt-in");
  kern<<<grid, kLutThreads, smem, st>>>(a);
  if (int rc = check_launch("lut_build")) return rc;
  if (a.slog == nullptr || a.sample != nullptr) return PQHSA_OK;  // no threshold wanted, or placed by the first kernel
  tau_kernel<E><<<p.num_streams * p.group, kLutThreads, 0, st>>>(a);
  return check_launch("tau");
}

int launch_lut_build(const pqhsa_params& p, const pqhsa_ws_layout& w, const StepAppend* ap, cudaStream_t st) {
  LutArgs a;
  fill_lut_args(p, w, ap, a);
  PQHSA_DISPATCH_E(p.dtype, return (launch_lut_build_t<E>(p, a, st)));
  return PQHSA_OK;
}

}  // namespace pqhsa
