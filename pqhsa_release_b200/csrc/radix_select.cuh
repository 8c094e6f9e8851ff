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
