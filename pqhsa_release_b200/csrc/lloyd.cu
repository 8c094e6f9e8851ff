// The Lloyd steps of the index build (pq_hsa/index/kmeans.py:195-224, pq_hsa/index/pq.py:81-94) and the per-list
// value sums (pq_hsa/attention/kv_cache.py:688-728) on the device, with results that do not depend on the order in
// which CTAs run.
//
// The reference updates centroids with `index_add_(0, assignments, vectors)`: on a CPU that is one fp32 addition
// per key and column, in the order of the keys.  A device scatter with atomics gives sums that change from run to
// run, and with them the centroids, the lists of keys near a boundary and the whole index.  Here a step is
//   1. cluster_order_kernel: a stable counting sort of the keys of a stream by cluster - which key sits at place j
//      when the keys are ordered by (cluster, key index) - and the first place of every cluster;
//   2. cluster_sums_kernel: one thread per (cluster, column) adds the cluster's rows in that order, one rounded fp32
//      addition per key: the sums a single CPU thread gets from the same assignments, bit for bit;
// and the assignment of the code-word training is subspace_assign_kernel (the coarse assignment is the bulk
// encode kernel's).  Dividing by the counts, re-seeding empty clusters and rounding to the storage type are small
// tensor operations on [streams, clusters, width] and stay with the caller.
#include "common.cuh"

namespace pqhsa {

constexpr int kOrdThreads = 1024;
constexpr int kOrdWarps = kOrdThreads / 32;  // with at most 512 clusters: 32 x 512 counters, 64 KB of shared memory

// Stable counting sort by cluster id, one CTA per key set.  Warp w owns a contiguous range of the keys; a table
// [warp][cluster] first counts the range's keys per cluster, then holds the place of the range's next key of the
// cluster.  Inside a range the keys are placed 32 at a time: keys of the same cluster in a batch find each other
// with match.any and take consecutive places in lane order.  No barrier in the placement loop.
__global__ void __launch_bounds__(kOrdThreads) cluster_order_kernel(const uint16_t* __restrict__ ids, int n, int k,
                                                                     int32_t* __restrict__ order,
                                                                     int32_t* __restrict__ start) {
  extern __shared__ int ord_tab[];  // [kOrdWarps][k]
  __shared__ int wtot[kOrdWarps];
  const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint16_t* id = ids + (size_t)t * n;
  int32_t* ord = order + (size_t)t * n;
  int32_t* st = start + (size_t)t * (k + 1);
  const int per = (n + kOrdThreads - 1) / kOrdThreads * 32;  // keys per warp, a multiple of 32
  const int lo = min(n, warp * per), hi = min(n, lo + per);
  for (int i = tid; i < kOrdWarps * k; i += kOrdThreads) ord_tab[i] = 0;
  __syncthreads();
  int* mine = ord_tab + warp * k;
  for (int i = lo + lane; i < hi; i += 32) atomicAdd(&mine[min((int)id[i], k - 1)], 1);  // integer counts: any order
  __syncthreads();
  // thread c: keys of cluster c, the clusters' first places (prefix sum over the clusters), then the first place of
  // every warp's keys of the cluster (prefix sum over the warps)
  int total = 0;
  if (tid < k) {
    for (int w = 0; w < kOrdWarps; ++w) total += ord_tab[w * k + tid];
  }
  int all;
  int run = block_exscan(total, wtot, &all);
  if (tid < k) {
    st[tid] = run;
    for (int w = 0; w < kOrdWarps; ++w) {
      const int v = ord_tab[w * k + tid];
      ord_tab[w * k + tid] = run;
      run += v;
    }
  }
  if (tid == 0) st[k] = n;
  __syncthreads();
  for (int i0 = lo; i0 < hi; i0 += 32) {
    const int i = i0 + lane;
    const bool live = i < hi;
    const int c = live ? min((int)id[i], k - 1) : 0x10000 + lane;  // idle lanes match nobody
    const unsigned peers = __match_any_sync(0xffffffffu, c);
    const int rank = __popc(peers & ((1u << lane) - 1u));
    int base = 0;
    if (live) base = mine[c];
    __syncwarp();  // every peer has read the place before the first of them moves it on
    if (live && rank == 0) mine[c] = base + __popc(peers);
    __syncwarp();
    if (live) ord[base + rank] = i;
  }
}

// Sums of the rows of every cluster, added in the order of the keys.  rows: E [streams][n] rows of row_stride
// elements; key set t = group * streams + stream sums the columns [group * width, (group + 1) * width) of its
// stream's rows.  128 threads: 128 / width clusters per CTA, a thread per column.
template <typename E>
__global__ void __launch_bounds__(128) cluster_sums_kernel(const E* __restrict__ rows, long long stream_stride,
                                                            int row_stride, int width, int streams, int n, int k,
                                                            const int32_t* __restrict__ order,
                                                            const int32_t* __restrict__ start,
                                                            float* __restrict__ sums) {
  const int t = blockIdx.y, s = t % streams, group = t / streams;
  const int c = blockIdx.x * (128 / width) + (int)threadIdx.x / width, col = (int)threadIdx.x % width;
  if (c >= k) return;
  const E* base = rows + (size_t)s * stream_stride + group * width + col;
  const int32_t* ord = order + (size_t)t * n;
  const int p1 = start[(size_t)t * (k + 1) + c + 1];
  int p = start[(size_t)t * (k + 1) + c];
  float acc = 0.f;
  // Batches of U rows, two batches of row loads and the places of a third in flight; the additions stay one after
  // the other.  A chain is latency-bound (one thread per cluster and column), so what counts is loads in flight.
  constexpr int U = 32;
  const int nb = (p1 - p) / U;
  int idx[U];
  E v[U];
  if (nb > 0) {
#pragma unroll
    for (int u = 0; u < U; ++u) idx[u] = ord[p + u];
#pragma unroll
    for (int u = 0; u < U; ++u) v[u] = base[(size_t)idx[u] * row_stride];
    if (nb > 1) {
#pragma unroll
      for (int u = 0; u < U; ++u) idx[u] = ord[p + U + u];
    }
  }
  for (int bt = 0; bt < nb; ++bt) {
    E w[U];
    if (bt + 1 < nb) {
#pragma unroll
      for (int u = 0; u < U; ++u) w[u] = base[(size_t)idx[u] * row_stride];
    }
    if (bt + 2 < nb) {
#pragma unroll
      for (int u = 0; u < U; ++u) idx[u] = ord[p + (bt + 2) * U + u];
    }
#pragma unroll
    for (int u = 0; u < U; ++u) acc = __fadd_rn(acc, to_f(v[u]));
    if (bt + 1 < nb) {
#pragma unroll
      for (int u = 0; u < U; ++u) v[u] = w[u];
    }
  }
  p += nb * U;
  for (; p < p1; ++p) acc = __fadd_rn(acc, to_f(base[(size_t)ord[p] * row_stride]));
  sums[((size_t)t * k + c) * width + col] = acc;
}

// Nearest code word of every residual in each of the 8 subspaces, for the Lloyd steps of the code-word training:
// argmin_c (|c|^2 - 2 x.c), the form of pq_hsa/index/kmeans.py:108-131, first minimum on ties.  rows: float
// [streams][n][128]; books: float [streams][8][16][16]; ids: u16 [8][streams][n].  One key per thread; a subspace's
// 64-byte pieces of 256 keys are read coalesced into a padded tile (rows of 20 words: the 16-byte reads of eight
// consecutive keys fall into different banks).
constexpr int kSaKeys = 256;
constexpr int kSaRow = 20;

__global__ void __launch_bounds__(kSaKeys) subspace_assign_kernel(const float* __restrict__ rows, long long stream_stride,
                                                                   const float* __restrict__ books, int streams, int n,
                                                                   uint16_t* __restrict__ ids) {
  __shared__ __align__(16) float cb[kM * kC * 16];
  __shared__ float csq[kM * kC];
  __shared__ __align__(16) float tile[kSaKeys * kSaRow];
  const int s = blockIdx.y, k0 = blockIdx.x * kSaKeys, tid = threadIdx.x;
  for (int i = tid; i < kM * kC * 16; i += kSaKeys) cb[i] = books[(size_t)s * kM * kC * 16 + i];
  __syncthreads();
  if (tid < kM * kC) {
    float q = 0.f;
#pragma unroll
    for (int d = 0; d < 16; ++d) q = fmaf(cb[tid * 16 + d], cb[tid * 16 + d], q);
    csq[tid] = q;
  }
  const float* src = rows + (size_t)s * stream_stride + (size_t)k0 * kD;
  for (int m = 0; m < kM; ++m) {
    __syncthreads();  // the previous subspace's tile has been read; first round: csq is in place
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int e = r * kSaKeys + tid, key = e >> 2, part = e & 3;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (k0 + key < n) v = __ldg(reinterpret_cast<const float4*>(src + (size_t)key * kD + m * 16 + part * 4));
      *reinterpret_cast<float4*>(tile + key * kSaRow + part * 4) = v;
    }
    __syncthreads();
    float x[16];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float4 v = *reinterpret_cast<const float4*>(tile + tid * kSaRow + j * 4);
      x[4 * j] = v.x; x[4 * j + 1] = v.y; x[4 * j + 2] = v.z; x[4 * j + 3] = v.w;
    }
    int best = 0;
    float bs = INFINITY;
#pragma unroll 4
    for (int c = 0; c < kC; ++c) {
      const float* w = cb + (m * kC + c) * 16;  // the same address in every lane: a broadcast
      float dot = 0.f;
#pragma unroll
      for (int d = 0; d < 16; ++d) dot = fmaf(x[d], w[d], dot);
      const float sc = fmaf(-2.f, dot, csq[m * kC + c]);
      if (sc < bs) {  // a NaN score never wins: such a key stays with code word 0
        bs = sc;
        best = c;
      }
    }
    if (k0 + tid < n) ids[((size_t)m * streams + s) * n + k0 + tid] = (uint16_t)best;
  }
}

int launch_cluster_order(const uint16_t* ids, int sets, int n, int k, int32_t* order, int32_t* start, cudaStream_t st) {
  const size_t smem = (size_t)kOrdWarps * k * sizeof(int);
  if (cudaFuncSetAttribute(cluster_order_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    return check_launch("cluster_order: shared memory opt-in");
  cluster_order_kernel<<<sets, kOrdThreads, smem, st>>>(ids, n, k, order, start);
  return check_launch("cluster_order");
}

int launch_cluster_sums(const void* rows, int dtype, long long stream_stride, int row_stride, int width, int streams,
                        int groups, int n, int k, const int32_t* order, const int32_t* start, float* sums,
                        cudaStream_t st) {
  const dim3 grid((k + 128 / width - 1) / (128 / width), streams * groups);
  PQHSA_DISPATCH_E(dtype, {
    cluster_sums_kernel<E><<<grid, 128, 0, st>>>(static_cast<const E*>(rows), stream_stride, row_stride, width, streams,
                                                 n, k, order, start, sums);
  });
  return check_launch("cluster_sums");
}

int launch_subspace_assign(const float* rows, long long stream_stride, const float* books, int streams, int n,
                           uint16_t* ids, cudaStream_t st) {
  const dim3 grid((n + kSaKeys - 1) / kSaKeys, streams);
  subspace_assign_kernel<<<grid, kSaKeys, 0, st>>>(rows, stream_stride, books, streams, n, ids);
  return check_launch("subspace_assign");
}

}  // namespace pqhsa
