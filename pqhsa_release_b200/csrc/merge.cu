// Per-list log-sum-exp background and the final three-source softmax merge.
//
//   mass[l] = sum over the UNSELECTED keys n of list l of exp(approx[n] - M)
//   denom   = sum_l mass[l] + sum_{sink, local, selected} exp(exact - M)
//   out     = (sum exp(exact - M) v + sum_l mass[l] * vmean[l]) / denom
//
// with M the maximum over all sources: the centroid-mode merge of
// pq_hsa/attention/sparse_attention.py:887-1012 (there the selected keys'
// approximate mass is added and subtracted again; here the selection kernel has
// already taken each selected key out of its unit's sum).  It replaces
// pq_attend_bg and pq_attend_reduce_mw
// (pq_hsa/kernels/cuda/pq_fused_h20.cu:2150-2402) in the list-space form of the
// background argued for at :2043-2058.
//
// One CTA per query row.  The value-mean rows of the stream are requested first
// (they depend on nothing), then the per-unit (max, sum) pairs are folded into
// list masses in shared memory (a list owns a few consecutive units), the tail
// logits are scattered with shared-memory float atomics, and the
// [L] x [L x 128] product plus the split-K partials of the exact part finish the
// row.  Exponents are base 2: exp(x - M) = 2^(x * log2e - M2); the fused
// multiply-add keeps the difference accurate for large logits.
#include "common.cuh"

namespace pqhsa {

constexpr int kMrgThreads = 512;
constexpr int kMrgWarps = kMrgThreads / 32;
constexpr int kListGroups = kMrgThreads / 16;  // 16 threads x 8 dims cover one value-mean row
constexpr int kVmIter = kLMax / kListGroups;   // rows per thread

struct MergeArgs {
  void* out;
  const void* vmeans;
  const uint16_t* list_ids;
  const uint16_t* unit_list;
  const int32_t* state;
  const int32_t* row_info;
  const float* unit_max;
  const float* unit_sum;
  const float* tail_logit;
  const float* partial;
  int G, cap, ucap, tail_cap, chunks, sink, num_lists;
};

__device__ __forceinline__ float block_reduce(float v, float* sh, bool is_max) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = is_max ? warp_max(v) : warp_sum(v);
  __syncthreads();
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  float t = sh[0];
#pragma unroll
  for (int i = 1; i < kMrgWarps; ++i) t = is_max ? fmaxf(t, sh[i]) : t + sh[i];
  return t;
}

template <typename E> struct VmRaw;  // 8 elements of a value-mean row
template <> struct VmRaw<float> { float4 a, b; };
template <> struct VmRaw<__nv_bfloat16> { uint4 a; };
template <> struct VmRaw<__half> { uint4 a; };
__device__ __forceinline__ void vm_load(const float* p, VmRaw<float>& r) {
  r.a = __ldg(reinterpret_cast<const float4*>(p));
  r.b = __ldg(reinterpret_cast<const float4*>(p) + 1);
}
__device__ __forceinline__ void vm_load(const __nv_bfloat16* p, VmRaw<__nv_bfloat16>& r) {
  r.a = __ldg(reinterpret_cast<const uint4*>(p));
}
__device__ __forceinline__ void vm_load(const __half* p, VmRaw<__half>& r) { r.a = __ldg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ void vm_cvt(const VmRaw<float>& r, float (&v)[8]) {
  v[0] = r.a.x; v[1] = r.a.y; v[2] = r.a.z; v[3] = r.a.w; v[4] = r.b.x; v[5] = r.b.y; v[6] = r.b.z; v[7] = r.b.w;
}
__device__ __forceinline__ void vm_cvt(const VmRaw<__nv_bfloat16>& r, float (&v)[8]) {
  unpack8(r.a, static_cast<const __nv_bfloat16*>(nullptr), v);
}
__device__ __forceinline__ void vm_cvt(const VmRaw<__half>& r, float (&v)[8]) {
  unpack8(r.a, static_cast<const __half*>(nullptr), v);
}

template <typename E>
__global__ void __launch_bounds__(kMrgThreads) merge_kernel(const MergeArgs a) {
  __shared__ float mass[kLMax];
  __shared__ float red[kMrgWarps];
  __shared__ float part[kListGroups][kD];
  const int row = blockIdx.x, s = row / a.G, tid = threadIdx.x;
  const int32_t* st = a.state + (size_t)s * kST;
  const StreamGeom geo = stream_geom(st, a.sink);
  const int K = a.row_info[(size_t)row * kRI + PQHSA_RI_K];
  const int nchunks = (geo.full + K + kChunk - 1) / kChunk;

  // value-mean rows of this thread: list = lg + kListGroups * i, dims d8*8 .. d8*8+7
  const int d8 = tid & 15, lg = tid >> 4;
  const E* vm = static_cast<const E*>(a.vmeans) + (size_t)s * a.num_lists * kD + d8 * 8;
  VmRaw<E> vr[kVmIter / 2];
#pragma unroll
  for (int i = 0; i < kVmIter / 2; ++i) {
    const int l = lg + kListGroups * i;
    if (l < a.num_lists) vm_load(vm + (size_t)l * kD, vr[i]);
  }
  for (int i = tid; i < kLMax; i += kMrgThreads) mass[i] = 0.f;

  // M2 = max(max approximate logit, max exact logit) in the base-2 domain
  const float* umax = a.unit_max + (size_t)row * a.ucap;
  const float* usum = a.unit_sum + (size_t)row * a.ucap;
  const float* tl = a.tail_logit + (size_t)row * a.tail_cap;
  const float* pp = a.partial + (size_t)row * a.chunks * kPartial;
  float m = kNegInf;
  for (int u = tid; u < geo.n_units; u += kMrgThreads) m = fmaxf(m, umax[u]);
  for (int t = tid; t < geo.n_tail; t += kMrgThreads) m = fmaxf(m, tl[t]);
  m *= kLog2e;
  for (int c = tid; c < nchunks; c += kMrgThreads) m = fmaxf(m, pp[(size_t)c * kPartial]);
  const float M = block_reduce(m, red, true);  // also orders the zeroing of mass before the atomics

  float tot = 0.f;
  for (int u = tid; u < geo.n_units; u += kMrgThreads) {
    const float v = usum[u] * ex2(fmaf(umax[u], kLog2e, -M));
    atomicAdd(&mass[a.unit_list[(size_t)s * a.ucap + u]], v);
    tot += v;
  }
  for (int t = tid; t < geo.n_tail; t += kMrgThreads) {
    const float x = tl[t];
    if (x != kNegInf) {  // -inf marks a selected tail slot
      const float v = ex2(fmaf(x, kLog2e, -M));
      atomicAdd(&mass[a.list_ids[(size_t)s * a.cap + geo.n_sorted + t]], v);
      tot += v;
    }
  }
  for (int c = tid; c < nchunks; c += kMrgThreads) tot += pp[(size_t)c * kPartial + 1] * ex2(pp[(size_t)c * kPartial] - M);
  const float denom = fmaxf(block_reduce(tot, red, false), 1.17549435e-38f);  // the syncs inside publish mass[]

  // background: sum_l mass[l] * vmean[l][:]
  float acc[8];
#pragma unroll
  for (int d = 0; d < 8; ++d) acc[d] = 0.f;
#pragma unroll
  for (int i = 0; i < kVmIter / 2; ++i) {
    const int l = lg + kListGroups * i;
    if (l < a.num_lists) {
      float v[8];
      vm_cvt(vr[i], v);
      const float w = mass[l];
#pragma unroll
      for (int d = 0; d < 8; ++d) acc[d] = fmaf(w, v[d], acc[d]);
    }
  }
#pragma unroll
  for (int i = kVmIter / 2; i < kVmIter; ++i) {
    const int l = lg + kListGroups * i;
    if (l < a.num_lists) vm_load(vm + (size_t)l * kD, vr[i - kVmIter / 2]);
  }
#pragma unroll
  for (int i = kVmIter / 2; i < kVmIter; ++i) {
    const int l = lg + kListGroups * i;
    if (l < a.num_lists) {
      float v[8];
      vm_cvt(vr[i - kVmIter / 2], v);
      const float w = mass[l];
#pragma unroll
      for (int d = 0; d < 8; ++d) acc[d] = fmaf(w, v[d], acc[d]);
    }
  }
#pragma unroll
  for (int d = 0; d < 8; ++d) part[lg][d8 * 8 + d] = acc[d];
  __syncthreads();
  // fold the list groups, add the exact part: thread = (quarter, dim)
  const int d = tid & (kD - 1), qtr = tid / kD;
  constexpr int kQ = kMrgThreads / kD;
  float v = 0.f;
  for (int j = qtr; j < kListGroups; j += kQ) v += part[j][d];
  for (int c = qtr; c < nchunks; c += kQ) v = fmaf(pp[(size_t)c * kPartial + 2 + d], ex2(pp[(size_t)c * kPartial] - M), v);
  __syncthreads();
  part[qtr][d] = v;
  __syncthreads();
  if (tid < kD) {
    float o = part[0][tid];
#pragma unroll
    for (int j = 1; j < kQ; ++j) o += part[j][tid];
    static_cast<E*>(a.out)[(size_t)row * kD + tid] = from_f<E>(o / denom);
  }
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
  a.unit_max = reinterpret_cast<const float*>(ws + w.unit_max);
  a.unit_sum = reinterpret_cast<const float*>(ws + w.unit_sum);
  a.tail_logit = reinterpret_cast<const float*>(ws + w.tail_logit);
  a.partial = reinterpret_cast<const float*>(ws + w.partial);
  a.G = p.group;
  a.cap = p.slot_capacity;
  a.ucap = p.unit_capacity;
  a.tail_cap = w.tail_cap;
  a.chunks = w.chunks;
  a.sink = p.sink_tokens;
  a.num_lists = p.num_lists;
  const int R = p.num_streams * p.group;
  PQHSA_DISPATCH_E(p.dtype, merge_kernel<E><<<R, kMrgThreads, 0, st>>>(a));
  return check_launch("merge");
}

}  // namespace pqhsa
