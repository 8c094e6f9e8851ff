// Appending decoded tokens: the raw K/V row write and the incremental encode
// of keys that have left the local window into the IVF-PQ index.
//
// append_kv      replaces pq_append_prep (pq_hsa/kernels/cuda/pq_fused_h20.cu:2888-2922).
// append_encode  mirrors IVFPQIndex.add with fixed codebooks
//                (pq_hsa/index/ivfpq.py:598-645): |k| and direction
//                (:1052-1059), nearest list by Euclidean distance (:1001-1005),
//                residual (:1012-1016), nearest code word per subspace
//                (pq_hsa/index/pq.py:97-115), nibble packing
//                (pq_hsa/index/packing.py:6-34); and the running per-list value
//                mean of pq_hsa/attention/kv_cache.py:730-776.
// All arithmetic is fp32 on the stored element values; ties go to the lower
// index as torch.argmin does.
#include "encode.cuh"

namespace pqhsa {

constexpr int kEncThreads = 256;

template <typename E>
__global__ void __launch_bounds__(kD) append_kv_kernel(E* __restrict__ kb, E* __restrict__ vb, KvAddr kv,
                                                       int32_t* __restrict__ state, const E* __restrict__ nk,
                                                       const E* __restrict__ nv) {
  const int s = blockIdx.x;
  int32_t* st = state + (size_t)s * kST;
  const int pos = st[PQHSA_ST_SEQ_LEN];
  const long long off = kv.offset(st[PQHSA_ST_REQ], st[PQHSA_ST_KV_HEAD], pos);
  kb[off + threadIdx.x] = nk[(size_t)s * kD + threadIdx.x];
  vb[off + threadIdx.x] = nv[(size_t)s * kD + threadIdx.x];
  __syncthreads();
  if (threadIdx.x == 0) st[PQHSA_ST_SEQ_LEN] = pos + 1;
}

template <typename E>
__global__ void __launch_bounds__(kEncThreads) append_encode_kernel(const EncodeArgs a) {
  const int s = blockIdx.x;
  int32_t* st = a.state + (size_t)s * kST;
  const int n_tail = encode_tokens<E, kEncThreads>(a, s, st[PQHSA_ST_SEQ_LEN]);
  if (threadIdx.x == 0) st[PQHSA_ST_N_TAIL] = n_tail;
}

int launch_append_kv(const pqhsa_params& p, const void* k, const void* v, cudaStream_t st) {
  PQHSA_DISPATCH_E(p.dtype, append_kv_kernel<E><<<p.num_streams, kD, 0, st>>>(
      static_cast<E*>(const_cast<void*>(p.k_base)), static_cast<E*>(const_cast<void*>(p.v_base)), make_kvaddr(p),
      static_cast<int32_t*>(p.state), static_cast<const E*>(k), static_cast<const E*>(v)));
  return check_launch("append_kv");
}

int launch_append_encode(const pqhsa_params& p, const int32_t* cnt, int32_t uni, cudaStream_t st) {
  const EncodeArgs a = make_encode_args(p, cnt, uni);
  PQHSA_DISPATCH_E(p.dtype, append_encode_kernel<E><<<p.num_streams, kEncThreads, 0, st>>>(a));
  return check_launch("append_encode");
}

}  // namespace pqhsa
