// Bulk encode against fixed codebooks: every key of [S, N, 128] is split into norm and
// direction, assigned to its nearest list and residual-encoded to 8 nibbles.  This is the
// "assign + encode every key" pass that ends an index build (pq_hsa/index/ivfpq.py:275-348)
// and a codebook-moving refresh (:647-707), and IVFPQIndex.add (:598-645) for a large batch.
//
// The arithmetic is the incremental encoder's (encode.cuh), value for value: the squared norm
// is four 32-dim butterfly sums added left to right, a list distance is
// (p0 + p1) + (p2 + p3) with p_q the fmaf chain of (u_d - c_d)^2 over dims 32q .. 32q+31, a
// code-word distance is one fmaf chain over its 16 dims, and ties go to the lower index.  A key
// encoded here and the same key encoded by pqhsa_append_encode get the same list, code and norm.
//
// Shape of the work: N x L x 128 subtract-and-fma pairs per stream (fp32 pipe bound), the
// code-word search is 1/32 of that.  One CTA takes 128 keys; their directions stay in shared
// memory, dimension-major, while the stream's centroids pass through a second shared tile 64
// lists at a time.  A thread owns a 4-key x 8-list block of distances, so three 16-byte
// shared loads feed 32 subtract-fma pairs.
//
// GIVEN: the lists are an input (the caller kept them from an earlier pass against the same centroids, as the index
// build does once its code words are trained); the search is skipped and only norm, residual and code remain.
#include "common.cuh"

namespace pqhsa {

#ifndef PQHSA_BULK_NJ
#define PQHSA_BULK_NJ 2
#endif
constexpr int kBulkLists = 64;     // lists per centroid tile
constexpr int kBulkThreads = 256;

struct BulkArgs {
  const void* keys;
  long long stream_stride;  // elements between the first keys of two streams
  const void* coarse;
  const void* codebooks;
  uint32_t* codes;
  void* norms;
  uint16_t* list_ids;  // written, or read when the lists are given
  int n, num_lists;
};

// rows [row0, row0 + 64) of a row-major [rows, 128] matrix of E -> dst[d][r] as fp32; rows at or
// beyond `rows` read as zero.  Lane -> row, so the transposed stores hit 32 different banks.
template <typename E>
__device__ __forceinline__ void load_tile_transposed(const E* src, int row0, int rows, float (*dst)[kBulkLists]) {
  constexpr int kPer = 16 / (int)sizeof(E);  // elements per 16-byte vector
  constexpr int kVec = kD / kPer;            // vectors per row
  for (int i = threadIdx.x; i < kBulkLists * kVec; i += kBulkThreads) {
    const int r = i % kBulkLists, j = i / kBulkLists;
    float v[kPer];
    if (row0 + r < rows) {
      const uint4 raw = __ldg(reinterpret_cast<const uint4*>(src + (size_t)(row0 + r) * kD) + j);
      if constexpr (sizeof(E) == 2) {
        unpack8(raw, static_cast<const E*>(nullptr), v);
      } else {
        v[0] = __uint_as_float(raw.x);
        v[1] = __uint_as_float(raw.y);
        v[2] = __uint_as_float(raw.z);
        v[3] = __uint_as_float(raw.w);
      }
    } else {
#pragma unroll
      for (int d = 0; d < kPer; ++d) v[d] = 0.f;
    }
#pragma unroll
    for (int d = 0; d < kPer; ++d) dst[j * kPer + d][r] = v[d];
  }
}

// NJ = blocks of 4 lists per thread.  A warp spans 16 / NJ threads along the lists of a tile and
// 2 NJ threads along the keys; a thread owns 4 keys x 4 NJ lists; a CTA takes 64 NJ keys.
template <typename E, int NJ, bool GIVEN>
__global__ void __launch_bounds__(kBulkThreads, 2) encode_bulk_kernel(const BulkArgs a) {
  constexpr int kBulkKeys = 64 * NJ;
  constexpr int kTx = 16 / NJ;  // threads of a warp along the lists
  extern __shared__ __align__(16) float bulk_smem[];
  float (*U)[kBulkKeys] = reinterpret_cast<float (*)[kBulkKeys]>(bulk_smem);                    // directions, then residuals
  float (*C)[kBulkLists] = reinterpret_cast<float (*)[kBulkLists]>(bulk_smem + kD * kBulkKeys);  // centroid tile, then code words
  __shared__ float nrm_sh[kBulkKeys];
  __shared__ int list_sh[kBulkKeys];
  __shared__ uint32_t code_sh[kBulkKeys];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int s = blockIdx.y, key0 = blockIdx.x * kBulkKeys;
  const E* keys = static_cast<const E*>(a.keys) + (size_t)s * a.stream_stride;
  const E* coarse = static_cast<const E*>(a.coarse) + (size_t)s * a.num_lists * kD;
  const E* books = static_cast<const E*>(a.codebooks) + (size_t)s * kM * kC * kSub;

  // ---- norm and direction: a warp per key, lane -> dims lane, lane + 32, ...
  for (int k = warp; k < kBulkKeys; k += kBulkThreads / 32) {
    const int n = key0 + k;
    float kv[4], tot = 0.f;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      kv[q] = n < a.n ? to_f(keys[(size_t)n * kD + q * 32 + lane]) : 0.f;
      tot += warp_sum(kv[q] * kv[q]);
    }
    const float nrm = fmaxf(sqrtf(tot), 1e-12f);
#pragma unroll
    for (int q = 0; q < 4; ++q) U[q * 32 + lane][k] = kv[q] / nrm;
    if (lane == 0) {
      nrm_sh[k] = nrm;
      code_sh[k] = 0u;
    }
  }

  if constexpr (GIVEN) {
    if (tid < kBulkKeys)
      list_sh[tid] = key0 + tid < a.n ? min((int)a.list_ids[(size_t)s * a.n + key0 + tid], a.num_lists - 1) : 0;
  } else {
  // ---- nearest list
  const int tx = lane % kTx, ty = warp * (32 / kTx) + lane / kTx;  // lists 4 tx (+ 4 kTx jb) .., keys 4 ty ..
  float bd[4];
  int bl[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    bd[i] = __builtin_huge_valf();
    bl[i] = 0;  // stays in range when every distance is NaN (a key row holding NaN or Inf): argmin then gives list 0
  }
  for (int l0 = 0; l0 < a.num_lists; l0 += kBulkLists) {
    __syncthreads();  // U written (first pass) / the previous tile has been read
    load_tile_transposed<E>(coarse, l0, a.num_lists, C);
    __syncthreads();
    float half01[4][4 * NJ], dist[4][4 * NJ];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float acc[4][4 * NJ];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4 * NJ; ++j) acc[i][j] = 0.f;
#pragma unroll 4
      for (int d = q * 32; d < q * 32 + 32; ++d) {
        const float4 u = *reinterpret_cast<const float4*>(&U[d][4 * ty]);
        const float uu[4] = {u.x, u.y, u.z, u.w};
        float cc[4 * NJ];
#pragma unroll
        for (int jb = 0; jb < NJ; ++jb) {
          const float4 c = *reinterpret_cast<const float4*>(&C[d][4 * tx + 4 * kTx * jb]);
          cc[4 * jb] = c.x;
          cc[4 * jb + 1] = c.y;
          cc[4 * jb + 2] = c.z;
          cc[4 * jb + 3] = c.w;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4 * NJ; ++j) {
            const float df = __fsub_rn(uu[i], cc[j]);
            acc[i][j] = __fmaf_rn(df, df, acc[i][j]);
          }
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4 * NJ; ++j) {
          if (q == 0) half01[i][j] = acc[i][j];
          if (q == 1) half01[i][j] = __fadd_rn(half01[i][j], acc[i][j]);
          if (q == 2) dist[i][j] = acc[i][j];
          if (q == 3) dist[i][j] = __fadd_rn(half01[i][j], __fadd_rn(dist[i][j], acc[i][j]));
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4 * NJ; ++j) {
        const int l = l0 + 4 * tx + 4 * kTx * (j >> 2) + (j & 3);  // ascending within a thread: strict < keeps the lowest index
        if (l < a.num_lists && dist[i][j] < bd[i]) {
          bd[i] = dist[i][j];
          bl[i] = l;
        }
      }
  }
  // best over the threads that share a key: tx is the low bits of the lane
#pragma unroll
  for (int i = 0; i < 4; ++i) {
#pragma unroll
    for (int o = 1; o < kTx; o <<= 1) {
      const float od = __shfl_xor_sync(0xffffffffu, bd[i], o);
      const int ol = __shfl_xor_sync(0xffffffffu, bl[i], o);
      if (od < bd[i] || (od == bd[i] && ol < bl[i])) {
        bd[i] = od;
        bl[i] = ol;
      }
    }
    if (tx == 0) list_sh[4 * ty + i] = bl[i];
  }
  }
  __syncthreads();  // the lists and (lists given: no tile loop before this) the directions are in place

  // ---- residuals in place of the directions, code words into the centroid tile
  // lane -> key: the shared accesses touch 32 banks; the centroid rows come from L2
  {
    const int k = tid % kBulkKeys;
    const E* crow = coarse + (size_t)list_sh[k] * kD;
    constexpr int kPer = 16 / (int)sizeof(E);
    if (key0 + k < a.n) {
      for (int v = tid / kBulkKeys; v < kD / kPer; v += kBulkThreads / kBulkKeys) {
        const uint4 raw = __ldg(reinterpret_cast<const uint4*>(crow) + v);
        float c[kPer];
        if constexpr (sizeof(E) == 2) {
          unpack8(raw, static_cast<const E*>(nullptr), c);
        } else {
          c[0] = __uint_as_float(raw.x);
          c[1] = __uint_as_float(raw.y);
          c[2] = __uint_as_float(raw.z);
          c[3] = __uint_as_float(raw.w);
        }
#pragma unroll
        for (int d = 0; d < kPer; ++d) U[v * kPer + d][k] = __fsub_rn(U[v * kPer + d][k], c[d]);
      }
    }
  }
  float* cw = &C[0][0];  // [m][c][16]
  for (int i = tid; i < kM * kC * kSub; i += kBulkThreads) cw[i] = to_f(books[i]);
  __syncthreads();

  // ---- nearest code word per subspace: thread -> (key, subspace), 2 NJ subspaces each
  constexpr int kKeyGroups = kBulkThreads / kBulkKeys;
#pragma unroll 1
  for (int h = 0; h < kM / kKeyGroups; ++h) {
    const int k = tid % kBulkKeys, m = tid / kBulkKeys + kKeyGroups * h;
    float r[kSub];
#pragma unroll
    for (int d = 0; d < kSub; ++d) r[d] = U[m * kSub + d][k];
    float best = __builtin_huge_valf();
    int bc = 0;
    for (int c = 0; c < kC; ++c) {
      const float4* w4 = reinterpret_cast<const float4*>(cw + (m * kC + c) * kSub);
      float dist = 0.f;
#pragma unroll
      for (int v = 0; v < kSub / 4; ++v) {
        const float4 w = w4[v];
        const float ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int d = 0; d < 4; ++d) {
          const float df = __fsub_rn(r[4 * v + d], ww[d]);
          dist = __fmaf_rn(df, df, dist);
        }
      }
      if (dist < best) {
        best = dist;
        bc = c;
      }
    }
    atomicOr(&code_sh[k], (uint32_t)bc << (4 * m));
  }
  __syncthreads();

  if (tid < kBulkKeys && key0 + tid < a.n) {
    const size_t o = (size_t)s * a.n + key0 + tid;
    a.codes[o] = code_sh[tid];
    static_cast<E*>(a.norms)[o] = from_f<E>(nrm_sh[tid]);
    if constexpr (!GIVEN) a.list_ids[o] = (uint16_t)list_sh[tid];
  }
}

int launch_encode_bulk(const void* keys, long long stream_stride, int streams, int n, int dtype, const void* coarse,
                       int num_lists, const void* codebooks, uint32_t* codes, void* norms, uint16_t* list_ids,
                       bool lists_given, cudaStream_t st) {
  BulkArgs a;
  a.keys = keys;
  a.stream_stride = stream_stride;
  a.coarse = coarse;
  a.codebooks = codebooks;
  a.codes = codes;
  a.norms = norms;
  a.list_ids = list_ids;
  a.n = n;
  a.num_lists = num_lists;
  constexpr int NJ = PQHSA_BULK_NJ;
  constexpr int kKeys = 64 * NJ;
  const dim3 grid((n + kKeys - 1) / kKeys, streams);
  constexpr int kSmem = kD * (kKeys + kBulkLists) * (int)sizeof(float);  // above the default limit
  PQHSA_DISPATCH_E(dtype, {
    auto kern = lists_given ? encode_bulk_kernel<E, NJ, true> : encode_bulk_kernel<E, NJ, false>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem) != cudaSuccess)
      return check_launch("encode_bulk: shared memory opt-in");
    kern<<<grid, kBulkThreads, kSmem, st>>>(a);
  });
  return check_launch("encode_bulk");
}

}  // namespace pqhsa
