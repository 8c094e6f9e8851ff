// First kernel of a decode step.
//
// lut_build_kernel: per-query-row table construction and threshold estimate, optionally fused with the step's
// token append (raw K/V row write) and the incremental encode of the key that left the local window.  The grid is
// made of thread block clusters of G CTAs (G = query rows per stream).  Encode clusters come first in launch order
// (the longest chain of the kernel; one CTA per stream), then one cluster per stream whose CTA j serves query row j.
// No CTA waits for a CTA outside its cluster.  The stream's length and its norm bound change once all CTAs of the
// stream are done (arrival counter), the tail count is written by the encode CTA at its very end.
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
// A CTA's data comes through a ring of three 32 KB stages in shared memory, filled by 16-byte asynchronous copies
// with three chunks in flight: CTA j of a row cluster streams the j-th share of the stream's centroid rows, scores
// them against all G query rows and stores row g's scores into the shared memory of CTA g (distributed shared memory)
// - the centroid rows cross from L2 to an SM once, not G times - and, behind them, the stream's sample records
// (64 KB), which it scores for its own row after the cluster's barrier, when all list scores of the row have
// arrived; the sample logits never leave the registers.  With 512 lists, 16-bit elements and G = 4 the three chunks
// (32 KB of centroids, 64 KB of sample records) are all asked for when the CTA starts.  The small loads a CTA's first
// steps depend on (query rows, code words, counters, the key row to encode) are issued before the bulk copies: a
// load issued behind 96 KB of copies waits for them.
//
// Threshold estimate.  The exact top-K needs the K-th largest of N logits, which is not
// known before the scan.  A stratified sample of 4096 slots of the list-sorted region
// (contiguous records made when the layout was made) is scored by the row's CTA, which histograms the top of
// the sample over its own range, walks the histogram from the top and takes as threshold tau the
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
#include <cooperative_groups.h>

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
  int want_tau;        // 1: thresholds wanted
  float* norm_max_rw;
  float* lut;
  float* pair_tab;  // [S, G / GP, 4, 256, GP] byte-pair sums of the tables for the scan, GP = min(G, 4); or null
  float* list_scores;
  float* row_bin;
  float* row_tau;
  int32_t* ticket;
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
  int enc_layers; // grid rows of encode clusters (G streams each) in front of the row clusters
  int num_streams;
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
// over the top of the sample's range is walked from the top; tau is the lower edge of the bin where the count reaches r (one
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
  // Only the top r sample keys matter.  The smallest of the threads' largest keys is at most the 256th largest of
  // the sample, the smallest of their second largest at most the 512th: with r within that, the histogram covers
  // only [that key, max] - a few hundred keys spread over all bins instead of 4096 piled up in the middle ones.
  uint32_t m1 = 0u, m2 = 0u, mn = key[0];
#pragma unroll
  for (int i = 0; i < kTauPer; ++i) {
    const uint32_t k = key[i];
    m2 = max(m2, min(m1, k));
    m1 = max(m1, k);
    mn = min(mn, k);
  }
  const bool restricted = r <= 2 * kLutThreads;
  uint32_t cut = r <= kLutThreads ? m1 : (restricted ? m2 : mn);
  uint32_t mx = m1;
  cut = __reduce_min_sync(0xffffffffu, cut);
  mx = __reduce_max_sync(0xffffffffu, mx);
  if (lane == 0) {
    sh.wmin[warp] = cut;
    sh.wmax[warp] = mx;
  }
  for (int i = tid; i < kBins; i += kLutThreads) sh.hist[i] = 0u;
  if (tid == 0) {
    sh.bin_lo = -1;
    sh.bin_hi = -1;
  }
  __syncthreads();
  cut = __reduce_min_sync(0xffffffffu, sh.wmin[lane & (kLutWarps - 1)]);
  mx = __reduce_max_sync(0xffffffffu, sh.wmax[lane & (kLutWarps - 1)]);
  // linear bins over [cut, max]
  const float lo = key_float(cut), hi = key_float(mx);
  const float inv_w = hi > lo ? (float)kBins / (hi - lo) : 1.f;
#pragma unroll
  for (int i = 0; i < kTauPer; ++i)
    if (key[i] >= cut) atomicAdd(&sh.hist[logit_bin(key_float(key[i]), lo, inv_w)], 1u);
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
    // one bin of slack for the rounding of the edges; bins 0 and 1 of the full range mean "everything"
    const bool all = !restricted && sh.bin_lo <= 1;
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

// The ring: chunk c of a CTA's data stream goes to stage c % kRingStages, three chunks in flight.  A centroid chunk is
// kLPS rows as they lie in memory; a sample chunk is kRecPerChunk records.
template <typename E> struct Ring {
  static constexpr int kRowBytes = kD * (int)sizeof(E);
  static constexpr int kLPS = kStageBytes / kRowBytes;  // centroid rows per chunk
  static constexpr int kRecPerChunk = kStageBytes / 16;
  static constexpr int kSampleChunks = kSample / kRecPerChunk;
  static_assert(kSample % kRecPerChunk == 0 && kRecPerChunk % kLutThreads == 0 && kLPS % kLutWarps == 0, "chunk shape");

  static __device__ __forceinline__ unsigned char* stage(unsigned char* ring, int c) {
    return ring + (size_t)(c % kRingStages) * kStageBytes;
  }
  // The encode role reads a centroid row with 4 lanes, 32 dims each, 16 bytes at a time: with the pieces of a row
  // permuted like this the 8 lanes of a quarter warp (two rows) read 8 different 16-byte bank groups (16-bit elements).
  static constexpr int kPPR = kRowBytes / 16;            // 16-byte pieces per centroid row
  static constexpr int kPPL = 32 * (int)sizeof(E) / 16;  // pieces per lane
  static __device__ __forceinline__ int slot(int row, int piece) {
    return piece ^ ((((piece / kPPL) >> 1) & 1) << 1) ^ (row & 1);
  }
  // `rows` centroid rows from src -> the stage of chunk c, pieces permuted; all threads call; one group per call
  static __device__ __forceinline__ void issue_rows(unsigned char* ring, int c, const unsigned char* src, int rows) {
    unsigned char* dst = stage(ring, c);
    for (int i = threadIdx.x; i < rows * kPPR; i += kLutThreads) {
      const int l = i / kPPR, P = i % kPPR;
      cp_async16(dst + l * kRowBytes + (slot(l, P) << 4), src + (size_t)i * 16);
    }
    cp_async_commit();
  }
  // `bytes` (a multiple of 16, at most a stage) from src -> the stage of chunk c; all threads call; one group per call
  static __device__ __forceinline__ void issue(unsigned char* ring, int c, const void* src, int bytes) {
    unsigned char* dst = stage(ring, c);
    const unsigned char* from = static_cast<const unsigned char*>(src);
    for (int i = threadIdx.x * 16; i < bytes; i += kLutThreads * 16) cp_async16(dst + i, from + i);
    cp_async_commit();
  }
};

template <int G> struct LutShared {
  float q[G][kD];  // the stream's query rows times the softmax scale
  float lut[kM * kC];
  float lsc[kLMax];  // this CTA's row: filled by all CTAs of the cluster
  TauScratch tau;
};

// The G row CTAs of a stream form a thread block cluster.  CTA j of the cluster
//   - brings in the j-th share of the stream's centroid rows and scores them against all G query rows (one warp per
//     row of centroids, a lane 4 dims), storing row g's scores into the shared memory of CTA g (distributed shared
//     memory) and into the workspace for the scan: the centroid rows cross from L2 to an SM once, not G times;
//   - after the cluster's barrier holds all list scores of query row j: it builds row j's tables, scores the sample
//     records for row j as their chunks land and places row j's thresholds.
// Encode CTAs come first in launch order, G streams to a cluster (they do not use the barrier).
template <typename E, int G>
__global__ void __launch_bounds__(kLutThreads, 2) lut_build_kernel(const LutArgs a) {
  using R = Ring<E>;
  namespace cg = cooperative_groups;
  extern __shared__ __align__(16) unsigned char ring[];  // kRingStages x kStageBytes
  __shared__ LutShared<G> sh;
  __shared__ EncodeShared<kLutThreads> esh;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int j = blockIdx.x;  // rank in the cluster (the grid is one cluster wide)
  const bool append = a.new_k != nullptr;
  const bool is_encode = (int)blockIdx.y < a.enc_layers;
  const int s = is_encode ? (int)blockIdx.y * G + j : (int)blockIdx.y - a.enc_layers;
  if (s >= a.num_streams) return;  // an encode cluster's spare CTA
  const unsigned char* coarse = static_cast<const unsigned char*>(a.coarse) + (size_t)s * a.num_lists * R::kRowBytes;
  int32_t* st = a.state + (size_t)s * kST;

  if (is_encode) {
    // encode role.  Only tokens that were in the cache when the kernel started are encoded: the row
    // another CTA of this launch is writing is not read (a row the caller stored before the call
    // counts).  A larger norm is parked in norm_pend and folded into norm_max by the last CTA, like
    // the length.  The first key's nearest list is searched in the centroid rows as they come through the
    // ring (asked for before anything else is looked at); further keys of the same step (a catch-up) read them
    // again from L2.
    const int nc = (a.num_lists + R::kLPS - 1) / R::kLPS;
    const int seq_old = st[PQHSA_ST_SEQ_LEN];
    const int n_sorted = st[PQHSA_ST_N_SORTED];
    int n_tail = st[PQHSA_ST_N_TAIL];
    const int want = a.enc.enc_count ? a.enc.enc_count[s] : a.enc.uniform_count;
    const bool bump = a.bump != 0 && seq_old > 0;
    const int seq_lim = seq_old + (bump ? 1 : 0);
    const int nl = st[PQHSA_ST_N_LISTS];
    const int req = st[PQHSA_ST_REQ], head = st[PQHSA_ST_KV_HEAD];
    const int sink_end = min(a.enc.sink, seq_lim);
    const E* kb = static_cast<const E*>(a.enc.k_base);
    const E* vb = static_cast<const E*>(a.enc.v_base);
    const E* books = static_cast<const E*>(a.enc.codebooks) + (size_t)s * kM * kC * kSub;
    // The first key's rows are asked for before the 96 KB of centroid rows: a load issued behind those waits for them.
    float k0 = 0.f, v0 = 0.f;
    {
      const int pos = sink_end + n_sorted + n_tail;
      if (want > 0 && pos < seq_lim && tid < kD) {
        const long long off = a.enc.kv.offset(req, head, pos);
        k0 = to_f(kb[off + tid]);
        v0 = to_f(vb[off + tid]);
      }
    }
#pragma unroll
    for (int c = 0; c < kRingStages; ++c) {
      const int rows = min(R::kLPS, a.num_lists - c * R::kLPS);
      R::issue_rows(ring, c, coarse + (size_t)c * kStageBytes, max(rows, 0));
    }
    if (tid == 0) a.enc.norm_max[s] = a.norm_max[s];
    for (int it = 0; it < want; ++it) {
      const int pos = sink_end + n_sorted + n_tail, slot = n_sorted + n_tail;
      // never index a token that is not in the cache, never overrun the pool
      if (pos >= seq_lim || slot >= a.enc.cap || n_tail >= a.enc.tail_cap) break;
      const long long off = a.enc.kv.offset(req, head, pos);
      float kval = k0, vval = v0;
      if (it > 0 && tid < kD) {
        kval = to_f(kb[off + tid]);
        vval = to_f(vb[off + tid]);
      }
      const float nrm = enc_direction<kLutThreads>(kval, esh);
      float bd;
      int lid;
      if (it == 0) {
        // argmin_l |u - c_l|^2 over the ring, 4 lanes per row and 32 dims per lane as in enc_nearest_list: the row's
        // distance is (p0 + p1) + (p2 + p3), so both searches agree to the bit
        const int sub = tid & 3, grp = tid >> 2;
        float uq[32];
#pragma unroll
        for (int d = 0; d < 32; ++d) uq[d] = esh.unit[sub * 32 + d];
        bd = __builtin_huge_valf();
        lid = 0;
        for (int c = 0; c < nc; ++c) {
          cp_async_wait<kRingStages - 1>();
          __syncthreads();  // every thread's pieces of chunk c have landed
          const unsigned char* stg = R::stage(ring, c);
          for (int l0 = 0; l0 < R::kLPS; l0 += kLutThreads / 4) {
            const int ll = l0 + grp, l = c * R::kLPS + ll;
            const bool valid = ll < R::kLPS && l < nl;
            float dist = 0.f;
            if (valid) {
              const unsigned char* rowp = stg + (size_t)ll * R::kRowBytes;
#pragma unroll
              for (int v = 0; v < R::kPPL; ++v) {
                float cv[Piece<E>::kDims];
                Piece<E>::unpack(*reinterpret_cast<const uint4*>(rowp + (R::slot(ll, sub * R::kPPL + v) << 4)), cv);
#pragma unroll
                for (int e = 0; e < Piece<E>::kDims; ++e) {
                  const float df = uq[v * Piece<E>::kDims + e] - cv[e];
                  dist = fmaf(df, df, dist);
                }
              }
            }
            dist += __shfl_xor_sync(0xffffffffu, dist, 1);
            dist += __shfl_xor_sync(0xffffffffu, dist, 2);
            if (valid && dist < bd) {  // l ascends within a thread, so strict < keeps the lowest index on ties
              bd = dist;
              lid = l;
            }
          }
          __syncthreads();  // the stage is free again
          const int cn = c + kRingStages;
          const int rows = min(R::kLPS, a.num_lists - cn * R::kLPS);
          R::issue_rows(ring, cn, coarse + (size_t)cn * kStageBytes, max(rows, 0));
        }
        enc_best_of_cta<kLutThreads>(bd, lid, esh);
      } else {
        enc_nearest_list<E, kLutThreads>(static_cast<const E*>(a.enc.coarse) + (size_t)s * a.num_lists * kD, 0, nl, nl, esh, bd, lid);
      }
      if (tid == 0) esh.list_sh = lid;
      __syncthreads();
      float cwv[kSub];
      if (tid < kM * kC) {
        float x[8], y[8];
        load8(books + (size_t)tid * kSub, x);
        load8(books + (size_t)tid * kSub + 8, y);
#pragma unroll
        for (int d = 0; d < 8; ++d) { cwv[d] = x[d]; cwv[8 + d] = y[d]; }
      }
      enc_finish<E, kLutThreads>(a.enc, s, slot, pos, esh.list_sh, nrm, vval, cwv, esh);
      ++n_tail;
    }
    cp_async_wait<0>();
    if (tid == 0) st[PQHSA_ST_N_TAIL] = n_tail;
  } else {
    cg::cluster_group cluster = cg::this_cluster();
    const int row = s * G + j;
    // ---- this CTA's data stream: its share of the centroid rows, then the sample records; asked for first ----
    const int share = ((a.num_lists + G - 1) / G + kLutWarps - 1) / kLutWarps * kLutWarps;  // rows per CTA, whole warps
    const int l_begin = min(j * share, a.num_lists), l_end = min(l_begin + share, a.num_lists);
    const int nmy = (l_end - l_begin + R::kLPS - 1) / R::kLPS;
    const bool want_tau = a.want_tau != 0 && a.sample != nullptr;
    const int4* sample = a.sample + (size_t)s * kSample;
    const int total = nmy + (want_tau ? R::kSampleChunks : 0);
    auto issue = [&](int c) {  // one group per call, empty or not: the waits count groups
      if (c < nmy) {
        const int rows = min(R::kLPS, l_end - l_begin - c * R::kLPS);
        R::issue(ring, c, coarse + (size_t)(l_begin + c * R::kLPS) * R::kRowBytes, rows * R::kRowBytes);
      } else if (c < total) {
        R::issue(ring, c, sample + (size_t)(c - nmy) * R::kRecPerChunk, kStageBytes);
      } else {
        cp_async_commit();
      }
    };
    // ---- inputs: asked for before the bulk copies (a load issued behind 96 KB of copies waits for them) ----
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
    // the stream counters: wanted after the cluster barrier, asked for now
    const int seq_old = st[PQHSA_ST_SEQ_LEN];
    const int n_sorted = st[PQHSA_ST_N_SORTED];
    const int n_tail_old = st[PQHSA_ST_N_TAIL];  // the encode CTA rewrites it at its very end (a later value shifts n by one)
    constexpr int kQPer = (G * kD + kLutThreads - 1) / kLutThreads;
    float qv[kQPer];
#pragma unroll
    for (int i = 0; i < kQPer; ++i) {
      const int e = tid + i * kLutThreads;
      qv[i] = (qb >= 0 && e < G * kD) ? to_f(static_cast<const E*>(a.q)[(size_t)qb * G * kD + e]) * a.scale : 0.f;
    }
#pragma unroll
    for (int c = 0; c < kRingStages; ++c) issue(c);
#pragma unroll
    for (int i = 0; i < kQPer; ++i) {
      const int e = tid + i * kLutThreads;
      if (e < G * kD) sh.q[e / kD][e % kD] = qv[i];
    }
    __syncthreads();
    // ---- row j's tables ----
    if (tid < kM * kC) {
      const int m = tid / kC;
      float acc = 0.f;
#pragma unroll
      for (int d = 0; d < kSub; ++d) acc = fmaf(sh.q[j][m * kSub + d], w[d], acc);
      a.lut[(size_t)row * kM * kC + tid] = acc;
      sh.lut[tid] = acc;
    }
    float qr[G][4];  // a lane's 4 dims of every query row
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
      for (int d = 0; d < 4; ++d) qr[g][d] = sh.q[g][lane * 4 + d];
    __syncthreads();
    if (a.pair_tab != nullptr) {
      // the scan looks codes up a byte (two subspaces) at a time: entry (p, byte) = lut[2p][byte & 15] +
      // lut[2p+1][byte >> 4], the rows of a group of min(G, 4) interleaved
      constexpr int GP = G < 4 ? G : 4;
      float* dst = a.pair_tab + (size_t)s * G * 1024 + (size_t)(j / GP) * 1024 * GP + (j % GP);
      for (int e = tid; e < 1024; e += kLutThreads) dst[(size_t)e * GP] = pair_entry(sh.lut, e >> 8, (uint32_t)(e & 255));
    }
    if (j == 0 && append && tid < 2 * kD / 8) {
      // the step's K/V row, 16 bytes per thread (elements are 2 or 4 bytes: 8 or 4 per vector)
      constexpr int kVec = 16 / (int)sizeof(E);
      const long long off = a.kv.offset(st[PQHSA_ST_REQ], st[PQHSA_ST_KV_HEAD], seq_old);
      for (int i = tid; i < 2 * kD / kVec; i += 2 * kD / 8) {
        const bool isv = i >= kD / kVec;
        const int e = (isv ? i - kD / kVec : i) * kVec;
        const E* src = static_cast<const E*>(isv ? a.new_v : a.new_k) + (size_t)s * kD + e;
        E* dst = static_cast<E*>(isv ? a.v_base : a.k_base) + off + e;
        *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
      }
    }
    // ---- list scores of this CTA's centroid rows against all G query rows: one warp per centroid row, 32 / G of
    // them at a time; the 32 partial dot products per lane are summed across the warp with 31 shuffles (halving
    // exchange: lane i ends up with the total of value i) instead of 5 per value ----
    constexpr int kPerWarp = R::kLPS / kLutWarps;                       // centroid rows of a chunk per warp
    constexpr int kLR = (32 / G) < kPerWarp ? 32 / G : kPerWarp;        // ... and per round
    float* const lsc_dst = cluster.map_shared_rank(sh.lsc, lane % G);   // the shared memory of the CTA of row lane % G
    for (int c = 0; c < nmy; ++c) {
      cp_async_wait<kRingStages - 1>();
      __syncthreads();  // every thread's pieces of chunk c have landed
      const unsigned char* stg = R::stage(ring, c);
      for (int r0 = 0; r0 < kPerWarp; r0 += kLR) {
        float v[32];
#pragma unroll
        for (int i = kLR * G; i < 32; ++i) v[i] = 0.f;
#pragma unroll
        for (int i = 0; i < kLR; ++i) {
          const int ll = warp * kPerWarp + r0 + i;
          float cv[4];
          if constexpr (sizeof(E) == 2) {
            const uint2 raw = *reinterpret_cast<const uint2*>(stg + (size_t)ll * R::kRowBytes + lane * 8);
            unpack4(raw, static_cast<const E*>(nullptr), cv);
          } else {
            const float4 raw = *reinterpret_cast<const float4*>(stg + (size_t)ll * R::kRowBytes + lane * 16);
            cv[0] = raw.x; cv[1] = raw.y; cv[2] = raw.z; cv[3] = raw.w;
          }
#pragma unroll
          for (int g = 0; g < G; ++g) {
            float acc = cv[0] * qr[g][0];
            acc = fmaf(cv[1], qr[g][1], acc);
            acc = fmaf(cv[2], qr[g][2], acc);
            v[i * G + g] = fmaf(cv[3], qr[g][3], acc);
          }
        }
        const float tot = warp_reduce_scatter32(v, lane);
        const int l = l_begin + c * R::kLPS + warp * kPerWarp + r0 + lane / G;
        if (lane < kLR * G && l < l_end) {
          a.list_scores[((size_t)s * G + lane % G) * kLMax + l] = tot;
          lsc_dst[l] = tot;
        }
      }
      __syncthreads();  // the stage is free again
      issue(c + kRingStages);
    }
    cluster.sync();  // all list scores of row j are in this CTA's shared memory
    // ---- the sample keys are scored (same arithmetic as the scan) and the thresholds placed ----
    if (want_tau && n_sorted > kSample) {
      constexpr int kPer = R::kRecPerChunk / kLutThreads;
      uint32_t key[R::kSampleChunks * kPer];
#pragma unroll
      for (int c2 = 0; c2 < R::kSampleChunks; ++c2) {
        cp_async_wait<kRingStages - 1>();
        __syncthreads();  // the chunk has landed
        const int4* rec = reinterpret_cast<const int4*>(R::stage(ring, nmy + c2));
#pragma unroll
        for (int i = 0; i < kPer; ++i) {
          const int4 v = rec[tid + i * kLutThreads];
          key[c2 * kPer + i] = float_key(finish_logit(pq_sum_row(sh.lut, (uint32_t)v.x), sh.lsc[v.z], __int_as_float(v.y)));
        }
        __syncthreads();
        issue(nmy + c2 + kRingStages);
      }
      // the encode role may still be running: its effect on the key count follows from the counters as they
      // were when the kernel started (tau is only a filter: the selection takes K from the final counters)
      int added = 0;
      if (a.encode) {
        const bool bump = a.bump != 0 && seq_old > 0;
        const int want = a.enc.enc_count ? a.enc.enc_count[s] : a.enc.uniform_count;
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
  const int seq_was = st[PQHSA_ST_SEQ_LEN];  // unchanged until the last CTA of the stream gets here
  const bool bump = a.bump != 0 && seq_was > 0;
  if (!append && !a.encode && !bump) return;
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    const int t = atomicAdd(a.ticket + 2 * s + 1, 1);
    if (t == G + (a.encode ? 1 : 0) - 1) {
      a.ticket[2 * s + 1] = 0;
      if (append || bump) st[PQHSA_ST_SEQ_LEN] = seq_was + 1;
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
  a.row_bin = w.row_bin == (size_t)-1 ? nullptr : reinterpret_cast<float*>(ws + w.row_bin);
  a.row_tau = reinterpret_cast<float*>(ws + w.row_tau);
  a.ticket = reinterpret_cast<int32_t*>(ws + w.ticket);
  a.num_lists = p.num_lists;
  a.cap = p.slot_capacity;
  a.G = p.group;
  a.scale = p.scale;
  a.top_fraction = p.top_fraction;
  a.topk_fixed = p.topk_fixed;
  a.margin = p.select_margin;
  a.sample = static_cast<const int4*>(p.sample);
  a.want_tau = w.row_bin == (size_t)-1 ? 0 : 1;
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

template <typename E, int G>
static int launch_lut_build_t(const pqhsa_params& p, LutArgs& a, cudaStream_t st) {
  a.num_streams = p.num_streams;
  a.enc_layers = a.encode ? (p.num_streams + G - 1) / G : 0;
  constexpr size_t smem = (size_t)kRingStages * kStageBytes;
  auto kern = lut_build_kernel<E, G>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    return check_launch("lut_build: shared memory opt-in");
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(G, p.num_streams + a.enc_layers);
  cfg.blockDim = dim3(kLutThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;  // the G row CTAs of a stream share their list scores
  attr.val.clusterDim.x = G;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, kern, (const LutArgs)a) != cudaSuccess) return check_launch("lut_build");
  if (int rc = check_launch("lut_build")) return rc;
  if (!a.want_tau || a.sample != nullptr) return PQHSA_OK;  // no threshold wanted, or placed by the first kernel
  tau_kernel<E><<<p.num_streams * p.group, kLutThreads, 0, st>>>(a);
  return check_launch("tau");
}

int launch_lut_build(const pqhsa_params& p, const pqhsa_ws_layout& w, const StepAppend* ap, cudaStream_t st) {
  LutArgs a;
  fill_lut_args(p, w, ap, a);
  PQHSA_DISPATCH_E(p.dtype, PQHSA_DISPATCH_G(p.group, return (launch_lut_build_t<E, G>(p, a, st))));
  return PQHSA_OK;
}

}  // namespace pqhsa
