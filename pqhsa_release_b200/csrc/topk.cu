// Stand-alone exact top-k over rows of fp32 scores (one CTA per row, radix
// select on the order-preserving 32-bit key, ties towards the lower index).
// Same selection rule as the fused path; counterpart of pq_topk_radix
// (pq_hsa/kernels/cuda/pq_fused_h20.cu:3624-3688) and of torch.topk as used at
// pq_hsa/attention/sparse_attention.py:661-666.
#include "common.cuh"
#include "radix_select.cuh"

namespace pqhsa {

constexpr int kTopkThreads = 1024;

__global__ void __launch_bounds__(kTopkThreads) topk_kernel(const float* __restrict__ scores, int n, long long stride,
                                                            int k, int32_t* __restrict__ out_idx,
                                                            float* __restrict__ out_val) {
  __shared__ RadixShared rsh;
  __shared__ int emit_count;
  const float* row = scores + (size_t)blockIdx.x * stride;
  const int tid = threadIdx.x;
  if (tid == 0) emit_count = 0;
  auto key = [&](int i) -> uint32_t { return float_key(__ldg(row + i)); };
  uint32_t T = 0u, T2 = 0u;
  int t = 0;
  const bool take_all = k >= n;
  if (!take_all) {
    const int ties = block_radix_threshold<kTopkThreads>(key, n, k, rsh, T, t);
    if (ties != t) {
      auto tie_key = [&](int i) -> uint32_t { return key(i) == T ? ~(uint32_t)i : 0u; };
      int t2;
      block_radix_threshold<kTopkThreads>(tie_key, n, t, rsh, T2, t2);
    }
  }
  __syncthreads();
  for (int i = tid; i < n; i += kTopkThreads) {
    const float v = __ldg(row + i);
    const uint32_t kk = float_key(v);
    if (take_all || kk > T || (kk == T && ~(uint32_t)i >= T2)) {
      const int o = atomicAdd(&emit_count, 1);
      if (o < k) {
        out_idx[(size_t)blockIdx.x * k + o] = i;
        out_val[(size_t)blockIdx.x * k + o] = v;
      }
    }
  }
}

int launch_topk(const float* scores, int rows, int n, int64_t stride, int k, int32_t* oi, float* ov, cudaStream_t st) {
  topk_kernel<<<rows, kTopkThreads, 0, st>>>(scores, n, (long long)stride, k, oi, ov);
  return check_launch("topk_radix");
}

}  // namespace pqhsa
