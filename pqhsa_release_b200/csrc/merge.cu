// Per-list log-sum-exp background and the final three-source softmax merge.
//
//   mass[g][l] = sum over the UNSELECTED keys n of list l of exp(approx[g][n] - M)
//   denom[g]   = sum_l mass[g][l] + sum_{sink, local, selected} exp(exact - M)
//   out[g]     = (sum exp(exact - M) v + sum_l mass[g][l] * vmean[l]) / denom[g]
//
// with M the maximum over all sources: the centroid-mode merge of
// pq_hsa/attention/sparse_attention.py:887-1012 (there the selected keys'
// approximate mass is added and subtracted again; here the attend kernel has
// already taken each selected key out of its unit's sum).  It replaces
// pq_attend_bg and pq_attend_reduce_mw
// (pq_hsa/kernels/cuda/pq_fused_h20.cu:2150-2402) and takes the list-space form
// of the background argued for at :2043-2058: the value means of a stream are
// read once for all G rows.
//
// One CTA per stream.  The per-unit (max, sum) pairs are folded into list
// masses in shared memory (a list owns a few consecutive units), the tail logits
// are scattered with shared-memory float atomics, then a [G x L] x [L x 128]
// product with the value means and the split-K partials of the exact part
// finish the rows.  Exponents are base 2: exp(x - M) = 2^(x * log2e - M2), the
// fused multiply-add keeps the difference accurate for large logits.
#include "common.cuh"

namespace pqhsa {

constexpr int kMrgThreads = 512;

struct MergeArgs {
  void* out;
  const void* vmeans;
  const uint16_t* list_ids;
  const uint16_t* unit_list;
  const int32_t* state;
  const int32_t* row_info;
  const float* row_amax;
  const float* unit_max;
  const float* unit_sum;
  const float* tail_logit;
  const float* partial;
  int cap, ucap, tail_cap, chunks, sink, num_lists;
};

template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* sh) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int i = 0; i < THREADS / 32; ++i) t += sh[i];
  return t;
}

template <typename E, int G>
__global__ void __launch_bounds__(kMrgThreads) merge_kernel(const MergeArgs a) {
  __shared__ float mass[G][kLMax];
  __shared__ float red[kMrgThreads / 32];
  __shared__ float sM[G], sden[G];
  __shared__ float part[kMrgThreads / kD][G][kD];
  const int s = blockIdx.x, tid = threadIdx.x;
  const int32_t* st = a.state + (size_t)s * kST;
  const int n_sorted = st[PQHSA_ST_N_SORTED], n_tail = st[PQHSA_ST_N_TAIL], n_units = st[PQHSA_ST_N_UNITS];
  const int seq_len = st[PQHSA_ST_SEQ_LEN];
  const int sink_end = min(a.sink, seq_len);
  const int F = sink_end + max(seq_len - (sink_end + n_sorted + n_tail), 0);

  for (int i = tid; i < G * kLMax; i += kMrgThreads) (&mass[0][0])[i] = 0.f;

  int nchunks[G];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const int row = s * G + g;
    const int K = a.row_info[(size_t)row * kRI + PQHSA_RI_K];
    nchunks[g] = (F + K + kChunk - 1) / kChunk;
    // M2 = max(max approximate logit, max exact logit) in the base-2 domain
    float m = a.row_amax[row] * kLog2e;
    for (int c = 0; c < nchunks[g]; ++c) m = fmaxf(m, a.partial[((size_t)row * a.chunks + c) * kPartial]);
    if (tid == 0) sM[g] = m;
  }
  __syncthreads();

#pragma unroll
  for (int g = 0; g < G; ++g) {
    const int row = s * G + g;
    const float M = sM[g];
    float approx = 0.f;
    for (int u = tid; u < n_units; u += kMrgThreads) {
      const float v = a.unit_sum[(size_t)row * a.ucap + u] * ex2(fmaf(a.unit_max[(size_t)row * a.ucap + u], kLog2e, -M));
      atomicAdd(&mass[g][a.unit_list[(size_t)s * a.ucap + u]], v);
      approx += v;
    }
    for (int t = tid; t < n_tail; t += kMrgThreads) {
      const float x = a.tail_logit[(size_t)row * a.tail_cap + t];
      if (x != kNegInf) {  // -inf marks a selected tail slot
        const float v = ex2(fmaf(x, kLog2e, -M));
        atomicAdd(&mass[g][a.list_ids[(size_t)s * a.cap + n_sorted + t]], v);
        approx += v;
      }
    }
    float exact = 0.f;
    for (int c = tid; c < nchunks[g]; c += kMrgThreads) {
      const float* pp = a.partial + ((size_t)row * a.chunks + c) * kPartial;
      exact += pp[1] * ex2(pp[0] - M);
    }
    const float tot_approx = block_sum<kMrgThreads>(approx, red);
    const float tot_exact = block_sum<kMrgThreads>(exact, red);
    if (tid == 0) sden[g] = fmaxf(tot_approx + tot_exact, 1.17549435e-38f);
  }
  __syncthreads();

  // background product and exact accumulators: thread = (slice, dim)
  const int d = tid & (kD - 1), slice = tid / kD;
  constexpr int kSlices = kMrgThreads / kD;
  float accg[G];
#pragma unroll
  for (int g = 0; g < G; ++g) accg[g] = 0.f;
  const E* vm = static_cast<const E*>(a.vmeans) + (size_t)s * a.num_lists * kD;
  for (int l = slice; l < a.num_lists; l += kSlices) {
    const float v = to_f(vm[(size_t)l * kD + d]);
#pragma unroll
    for (int g = 0; g < G; ++g) accg[g] = fmaf(mass[g][l], v, accg[g]);
  }
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const int row = s * G + g;
    const float M = sM[g];
    for (int c = slice; c < nchunks[g]; c += kSlices) {
      const float* pp = a.partial + ((size_t)row * a.chunks + c) * kPartial;
      accg[g] = fmaf(pp[2 + d], ex2(pp[0] - M), accg[g]);
    }
    part[slice][g][d] = accg[g];
  }
  __syncthreads();
  for (int i = tid; i < G * kD; i += kMrgThreads) {
    const int g = i / kD, dd = i % kD;
    float v = 0.f;
#pragma unroll
    for (int sl = 0; sl < kSlices; ++sl) v += part[sl][g][dd];
    static_cast<E*>(a.out)[((size_t)s * G + g) * kD + dd] = from_f<E>(v / sden[g]);
  }
}

template <typename E, int G>
static int launch_merge_t(const pqhsa_params& p, const MergeArgs& a, cudaStream_t st) {
  merge_kernel<E, G><<<p.num_streams, kMrgThreads, 0, st>>>(a);
  return check_launch("merge");
}

int launch_merge(const pqhsa_params& p, const pqhsa_ws_layout& w, cudaStream_t st) {
  char* ws = static_cast<char*>(p.workspace);
  MergeArgs a;
  a.out = p.out;
  a.vmeans = p.vmeans;
  a.list_ids = static_cast<const uint16_t*>(p.list_ids);
  a.unit_list = static_cast<const uint16_t*>(p.unit_list);
  a.state = static_cast<const int32_t*>(p.state);
  a.row_info = reinterpret_cast<const int32_t*>(ws + w.row_info);
  a.row_amax = reinterpret_cast<const float*>(ws + w.row_amax);
  a.unit_max = reinterpret_cast<const float*>(ws + w.unit_max);
  a.unit_sum = reinterpret_cast<const float*>(ws + w.unit_sum);
  a.tail_logit = reinterpret_cast<const float*>(ws + w.tail_logit);
  a.partial = reinterpret_cast<const float*>(ws + w.partial);
  a.cap = p.slot_capacity;
  a.ucap = p.unit_capacity;
  a.tail_cap = w.tail_cap;
  a.chunks = w.chunks;
  a.sink = p.sink_tokens;
  a.num_lists = p.num_lists;
  PQHSA_DISPATCH_E(p.dtype, PQHSA_DISPATCH_G(p.group, return (launch_merge_t<E, G>(p, a, st))));
  return PQHSA_OK;
}

}  // namespace pqhsa
