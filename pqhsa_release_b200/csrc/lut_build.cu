// Per-query, per-head table construction (first kernel of a decode step).
//
// For every stream s and query row g:
//   lut[s][g][m][c]      = scale * <q_g restricted to subspace m, codebooks[s][m][c]>
//   list_scores[s][g][l] = scale * <q_g, coarse[s][l]>
// The reference normalises q, scores, and multiplies |q| back
// (pq_hsa/index/ivfpq.py:1061-1118); production folds |q| and the softmax scale
// into the tables (benchmarks/e2e_pq_param_sweep.py:228-249,
// pq_hsa/kernels/cuda/pq_fused_h20.cu:2975-3051), as is done here, in fp32.
//
// The same launch clears the per-step selection histogram and row counters,
// resolves K for every row from the device-side slot counts, and sizes the
// row's histogram bins from a bound on |logit|:
//   |logit| <= (scale |q| max_l |c_l| + sum_m max_c |lut[m][c]|) * max |k|,  |c_l| <= 1
// (centroids are means of unit vectors).  The bound only sets the resolution of
// the histogram; the selection is exact whatever it is.
#include "common.cuh"

namespace pqhsa {

constexpr int kLutThreads = 256;
constexpr int kListsPerCta = 64;  // 8 warps x 8 lists

template <typename E, int G>
__global__ void __launch_bounds__(kLutThreads) lut_build_kernel(
    const E* __restrict__ q, const E* __restrict__ codebooks, const E* __restrict__ coarse,
    const int32_t* __restrict__ state, const float* __restrict__ norm_max, float* __restrict__ lut,
    float* __restrict__ list_scores, uint32_t* __restrict__ hist, int32_t* __restrict__ row_info,
    float* __restrict__ row_bin, int num_lists, float scale, double top_fraction, int topk_fixed, float fixed_lo,
    float fixed_inv_w) {
  __shared__ float qs[G][kD];
  __shared__ float sub_max[G][kM];
  const int s = blockIdx.x;
  const int tid = threadIdx.x;
  for (int i = tid; i < G * kD; i += kLutThreads) qs[i / kD][i % kD] = to_f(q[(size_t)s * G * kD + i]) * scale;
  __syncthreads();

  // clear this stream's share of the histogram: G rows x 4096 bins
  {
    uint4* h4 = reinterpret_cast<uint4*>(hist + (size_t)s * G * kBins);
    const int total4 = G * kBins / 4;
    for (int i = blockIdx.y * kLutThreads + tid; i < total4; i += gridDim.y * kLutThreads)
      h4[i] = make_uint4(0u, 0u, 0u, 0u);
  }

  if (blockIdx.y == 0) {
    if (tid < kM * kC) {
      const int m = tid / kC;
      const E* cw = codebooks + ((size_t)s * kM * kC + tid) * kSub;
      float w[kSub];
      {
        float a[8], b[8];
        load8(cw, a);
        load8(cw + 8, b);
#pragma unroll
        for (int d = 0; d < 8; ++d) { w[d] = a[d]; w[8 + d] = b[d]; }
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float acc = 0.f;
#pragma unroll
        for (int d = 0; d < kSub; ++d) acc = fmaf(qs[g][m * kSub + d], w[d], acc);
        lut[((size_t)s * G + g) * kM * kC + tid] = acc;
        float mx = fabsf(acc);  // max over the 16 code words of this subspace (16 consecutive lanes)
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        if ((tid & (kC - 1)) == 0) sub_max[g][m] = mx;
      }
    }
    __syncthreads();
    if (tid < G) {
      const int32_t* st = state + (size_t)s * kST;
      const int n = st[PQHSA_ST_N_SORTED] + st[PQHSA_ST_N_TAIL];
      int32_t* ri = row_info + ((size_t)s * G + tid) * kRI;
      ri[PQHSA_RI_K] = resolve_topk(n, top_fraction, topk_fixed);
      ri[PQHSA_RI_THR_BIN] = kBins;
      ri[PQHSA_RI_ABOVE] = 0;
      ri[PQHSA_RI_NSEL] = 0;
      ri[PQHSA_RI_NCAND] = 0;
      ri[PQHSA_RI_N] = n;
      float lo = fixed_lo, inv_w = fixed_inv_w;
      if (!(fixed_inv_w > 0.f)) {
        float qq = 0.f, pm = 0.f;
        for (int d = 0; d < kD; ++d) qq = fmaf(qs[tid][d], qs[tid][d], qq);
#pragma unroll
        for (int m = 0; m < kM; ++m) pm += sub_max[tid][m];
        const float bound = (sqrtf(qq) + pm) * norm_max[s] * 1.0001f;
        lo = -bound;
        inv_w = bound > 1e-30f ? (float)(kBins / 2) / bound : 1.f;
      }
      row_bin[((size_t)s * G + tid) * 2] = lo;
      row_bin[((size_t)s * G + tid) * 2 + 1] = inv_w;
    }
    return;
  }

  // list scores: one warp per list, a lane owns 4 dims
  const int warp = tid >> 5, lane = tid & 31;
  const int l0 = (blockIdx.y - 1) * kListsPerCta;
  float qr[G][4];
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int d = 0; d < 4; ++d) qr[g][d] = qs[g][lane * 4 + d];
  for (int i = warp; i < kListsPerCta; i += kLutThreads / 32) {
    const int l = l0 + i;
    if (l >= num_lists) break;
    float c[4];
    load4(coarse + ((size_t)s * num_lists + l) * kD + lane * 4, c);
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float acc = c[0] * qr[g][0];
      acc = fmaf(c[1], qr[g][1], acc);
      acc = fmaf(c[2], qr[g][2], acc);
      acc = fmaf(c[3], qr[g][3], acc);
      acc = warp_sum(acc);
      if (lane == 0) list_scores[((size_t)s * G + g) * kLMax + l] = acc;
    }
  }
}

template <typename E, int G>
static int launch_lut_build_t(const pqhsa_params& p, const pqhsa_ws_layout& w, cudaStream_t st) {
  char* ws = static_cast<char*>(p.workspace);
  const dim3 grid(p.num_streams, 1 + (p.num_lists + kListsPerCta - 1) / kListsPerCta);
  lut_build_kernel<E, G><<<grid, kLutThreads, 0, st>>>(
      static_cast<const E*>(p.q), static_cast<const E*>(p.codebooks), static_cast<const E*>(p.coarse),
      static_cast<const int32_t*>(p.state), static_cast<const float*>(p.norm_max),
      reinterpret_cast<float*>(ws + w.lut), reinterpret_cast<float*>(ws + w.list_scores),
      reinterpret_cast<uint32_t*>(ws + w.hist), reinterpret_cast<int32_t*>(ws + w.row_info),
      reinterpret_cast<float*>(ws + w.row_bin), p.num_lists, p.scale, p.top_fraction, p.topk_fixed, p.hist_lo,
      p.hist_inv_width);
  return check_launch("lut_build");
}

int launch_lut_build(const pqhsa_params& p, const pqhsa_ws_layout& w, cudaStream_t st) {
  PQHSA_DISPATCH_E(p.dtype, PQHSA_DISPATCH_G(p.group, return (launch_lut_build_t<E, G>(p, w, st))));
  return PQHSA_OK;
}

}  // namespace pqhsa
