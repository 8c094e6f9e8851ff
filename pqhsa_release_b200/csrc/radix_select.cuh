// Block-wide exact radix selection over 32-bit keys (4 passes of 8 bits).
// Shared by the selection kernel of the decode step and by the stand-alone
// top-k entry point.  Counterpart of the two-pass 16-bit radix select of
// pq_hsa/kernels/cuda/pq_fused_h20.cu:3624-3688, widened to the fp32 key.
#pragma once

#include "common.cuh"

namespace pqhsa {

struct RadixShared {
  uint32_t hist[256];
  uint32_t prefix;
  uint32_t mask;
  int remaining;
  int count;
};

// Among n items with keys key(i) (i in [0, n)), find T and t such that
// {key > T} plus t items of {key == T} are exactly the r largest (1 <= r <= n;
// items whose key is 0 never take part and must number at most n - r).
// Returns the number of items with key == T (so t == return value means the
// whole tie group is taken).  All threads of the block must call it; results are
// returned to every thread.
template <int THREADS, typename KeyFn>
__device__ int block_radix_threshold(KeyFn key, int n, int r, RadixShared& sh, uint32_t& T, int& t) {
  const int tid = threadIdx.x, lane = tid & 31;
  __syncthreads();
  if (tid == 0) {
    sh.prefix = 0u;
    sh.mask = 0u;
    sh.remaining = r;
    sh.count = 0;
  }
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = tid; i < 256; i += THREADS) sh.hist[i] = 0u;
    __syncthreads();
    const uint32_t prefix = sh.prefix, mask = sh.mask;
    const int n_round = (n + THREADS - 1) / THREADS * THREADS;
    for (int i = tid; i < n_round; i += THREADS) {
      uint32_t digit = 256u + lane;  // unique per lane: never matches, never counted
      if (i < n) {
        const uint32_t k = key(i);
        if (k != 0u && (k & mask) == prefix) digit = (k >> shift) & 255u;
      }
      // one shared-memory atomic per distinct digit in the warp
      const unsigned peers = __match_any_sync(0xffffffffu, digit);
      if (digit < 256u && lane == __ffs(peers) - 1) atomicAdd(&sh.hist[digit], (uint32_t)__popc(peers));
    }
    __syncthreads();
    if (tid < 32) {
      // lane j owns digits 255-8j .. 248-8j; find where the count from the top reaches `remaining`
      uint32_t local[8];
      uint32_t sum = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        local[j] = sh.hist[255 - (lane * 8 + j)];
        sum += local[j];
      }
      uint32_t incl = sum;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const uint32_t v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
      }
      const uint32_t excl = incl - sum;
      const uint32_t need = (uint32_t)sh.remaining;
      __syncwarp();  // every lane has read `remaining` before one of them updates it
      if (excl < need && need <= incl) {
        uint32_t cum = excl;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (cum < need && need <= cum + local[j]) {
            sh.prefix = prefix | ((uint32_t)(255 - (lane * 8 + j)) << shift);
            sh.mask = mask | (255u << shift);
            sh.remaining = (int)(need - cum);
            sh.count = (int)local[j];
          }
          cum += local[j];
        }
      }
    }
    __syncthreads();
  }
  T = sh.prefix;
  t = sh.remaining;
  const int ties = sh.count;
  __syncthreads();
  return ties;
}

}  // namespace pqhsa

namespace pqhsa {

// ---- register-resident variant ------------------------------------------------
// The same selection for at most THREADS * PER items held PER per thread in
// registers (key 0 = no item).  Candidate logits lie in a narrow band, so the
// keys share their high bits: the common prefix is skipped (block min / max) and
// the remaining bits are resolved in 11-bit digits with plain shared-memory
// atomics - usually two passes, no warp-match, no re-reading of the keys.
constexpr int kRadixBins2 = 2048;
struct RadixShared2 {
  uint32_t hist[kRadixBins2];
  uint32_t wtot[32];
  uint32_t wmin[32], wmax[32];
  uint32_t prefix;
  int remaining;
  int count;
};

template <int THREADS, int PER>
__device__ int block_radix_threshold_regs(const uint32_t (&key)[PER], int r, RadixShared2& sh, uint32_t& T, int& t) {
  static_assert(kRadixBins2 % THREADS == 0 && THREADS % 32 == 0 && THREADS <= 1024, "thread count");
  constexpr int BPT = kRadixBins2 / THREADS;
  constexpr int NW = THREADS / 32;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  uint32_t mn = 0xffffffffu, mx = 0u;
  int have = 0;
#pragma unroll
  for (int j = 0; j < PER; ++j)
    if (key[j] != 0u) {
      mn = min(mn, key[j]);
      mx = max(mx, key[j]);
      ++have;
    }
  mn = __reduce_min_sync(0xffffffffu, mn);
  mx = __reduce_max_sync(0xffffffffu, mx);
  have = __reduce_add_sync(0xffffffffu, have);
  __syncthreads();
  if (lane == 0) {
    sh.wmin[warp] = mn;
    sh.wmax[warp] = mx;
    sh.wtot[warp] = (uint32_t)have;
  }
  __syncthreads();
  mn = __reduce_min_sync(0xffffffffu, lane < NW ? sh.wmin[lane] : 0xffffffffu);
  mx = __reduce_max_sync(0xffffffffu, lane < NW ? sh.wmax[lane] : 0u);
  const int total = __reduce_add_sync(0xffffffffu, lane < NW ? (int)sh.wtot[lane] : 0);
  const uint32_t diff = mn ^ mx;
  int hb = diff ? 32 - __clz(diff) : 0;  // number of low bits that vary
  uint32_t prefix = hb >= 32 ? 0u : (mx >> hb) << hb;
  int remaining = r, count = total;
  while (hb > 0) {
    const int w = hb < 11 ? hb : 11, shift = hb - w;
    const uint32_t dmask = (1u << w) - 1u;
    __syncthreads();
#pragma unroll
    for (int b = 0; b < BPT; ++b) sh.hist[tid * BPT + b] = 0u;
    __syncthreads();
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const uint32_t k = key[j];
      const bool match = k != 0u && (hb >= 32 || (k >> hb) == (prefix >> hb));
      if (match) atomicAdd(&sh.hist[(k >> shift) & dmask], 1u);
    }
    __syncthreads();
    // thread j owns the BPT bins just below 2048 - BPT * j: ascending j walks down from the top
    const int top = kRadixBins2 - BPT * tid;
    uint32_t c[BPT], sum = 0;
#pragma unroll
    for (int b = 0; b < BPT; ++b) {
      c[b] = sh.hist[top - 1 - b];
      sum += c[b];
    }
    uint32_t incl = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    if (lane == 31) sh.wtot[warp] = incl;
    __syncthreads();
    incl += __reduce_add_sync(0xffffffffu, lane < warp ? sh.wtot[lane] : 0u);
    const uint32_t excl = incl - sum, need = (uint32_t)remaining;
    if (excl < need && need <= incl) {
      uint32_t cum = excl;
#pragma unroll
      for (int b = 0; b < BPT; ++b) {
        if (cum < need && need <= cum + c[b]) {
          sh.prefix = prefix | ((uint32_t)(top - 1 - b) << shift);
          sh.remaining = (int)(need - cum);
          sh.count = (int)c[b];
        }
        cum += c[b];
      }
    }
    __syncthreads();
    prefix = sh.prefix;
    remaining = sh.remaining;
    count = sh.count;
    hb = shift;
  }
  T = prefix;
  t = remaining;
  return count;
}

}  // namespace pqhsa
