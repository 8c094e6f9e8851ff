// Exact attention over sink + local-window rows and the selected keys, read in
// place from the (paged or contiguous) KV cache: split-K partials.
//
// Replaces pq_attend_partial_nw(_paged)_kernel
// (pq_hsa/kernels/cuda/pq_fused_h20.cu:1225-1753); the arithmetic is the
// full_logits / exact_retrieval_logits part of
// pq_hsa/attention/sparse_attention.py:807-857.
//
// This is the HBM-bound kernel of the step: K + F random 256-byte K rows and V
// rows per query row.  Work item = (query row, chunk of 128 entries); entry e of
// a row is the e-th row of [sink | local | selected].  A persistent grid sized to
// the resident CTA count strides over the items.  Inside a CTA each of the 4
// warps owns 32 entries:
//   1. lane-parallel: entry -> element offset of its K/V row (computed for sink
//      and local rows, read from sel_off for selected rows - one dependent load);
//   2. half-warp per row: 16 lanes x 16 bytes cover one 256-byte bf16 row
//      (2 x 16 bytes per lane for fp32); four row pairs (8 K rows + 8 V rows)
//      are requested before the first is consumed;
//   3. online softmax in the base-2 domain per half-warp; halves and warps are
//      merged at the end and one (max, sum, acc[128]) partial is written.
#include "common.cuh"

namespace pqhsa {

constexpr int kAttThreads = 128;
constexpr int kAttWarps = kAttThreads / 32;
constexpr int kAttUnroll = 4;  // row pairs in flight per warp
static_assert(kAttWarps * 32 == kChunk, "one entry per lane and chunk");

struct AttendArgs {
  const void* q;
  const void* k_base;
  const void* v_base;
  KvAddr kv;
  const int32_t* state;
  const int32_t* row_info;
  const long long* sel_off;
  float* partial;
  int R, G, kcap, chunks, sink;
  float scale;
};

template <typename E> struct RawRow;  // 8 elements of a K/V row as loaded
template <> struct RawRow<float> { float4 a, b; };
template <> struct RawRow<__nv_bfloat16> { uint4 a; };
template <> struct RawRow<__half> { uint4 a; };

__device__ __forceinline__ void ld_row(const float* p, RawRow<float>& r) {
  r.a = __ldg(reinterpret_cast<const float4*>(p));
  r.b = __ldg(reinterpret_cast<const float4*>(p) + 1);
}
__device__ __forceinline__ void ld_row(const __nv_bfloat16* p, RawRow<__nv_bfloat16>& r) {
  r.a = __ldg(reinterpret_cast<const uint4*>(p));
}
__device__ __forceinline__ void ld_row(const __half* p, RawRow<__half>& r) {
  r.a = __ldg(reinterpret_cast<const uint4*>(p));
}
__device__ __forceinline__ void zero_row(RawRow<float>& r) { r.a = make_float4(0, 0, 0, 0); r.b = r.a; }
__device__ __forceinline__ void zero_row(RawRow<__nv_bfloat16>& r) { r.a = make_uint4(0, 0, 0, 0); }
__device__ __forceinline__ void zero_row(RawRow<__half>& r) { r.a = make_uint4(0, 0, 0, 0); }
__device__ __forceinline__ void cvt_row(const RawRow<float>& r, float (&v)[8]) {
  v[0] = r.a.x; v[1] = r.a.y; v[2] = r.a.z; v[3] = r.a.w; v[4] = r.b.x; v[5] = r.b.y; v[6] = r.b.z; v[7] = r.b.w;
}
__device__ __forceinline__ void cvt_row(const RawRow<__nv_bfloat16>& r, float (&v)[8]) {
  unpack8(r.a, static_cast<const __nv_bfloat16*>(nullptr), v);
}
__device__ __forceinline__ void cvt_row(const RawRow<__half>& r, float (&v)[8]) {
  unpack8(r.a, static_cast<const __half*>(nullptr), v);
}

template <typename E>
__global__ void __launch_bounds__(kAttThreads, 6) attend_kernel(const AttendArgs a) {
  __shared__ float wm[kAttWarps], wl[kAttWarps];
  __shared__ float wacc[kAttWarps][kD];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int half = lane >> 4, l16 = lane & 15;
  const E* kb = static_cast<const E*>(a.k_base);
  const E* vb = static_cast<const E*>(a.v_base);
  const long long items = (long long)a.R * a.chunks;

  for (long long item = blockIdx.x; item < items; item += gridDim.x) {
    const int c = (int)(item / a.R);
    const int row = (int)(item % a.R);
    const int s = row / a.G;
    const int32_t* st = a.state + (size_t)s * kST;
    const StreamGeom geo = stream_geom(st, a.sink);
    const int F = geo.full;
    const int K = a.row_info[(size_t)row * kRI + PQHSA_RI_K];
    const int total = F + K;
    if (c * kChunk >= total) continue;  // uniform per block

    // 1. element offset of this lane's entry
    const int e = c * kChunk + warp * 32 + lane;
    long long off = 0;
    if (e < total) {
      if (e < F) {
        const int pos = e < geo.sink_end ? e : geo.retr_end + (e - geo.sink_end);
        off = a.kv.offset(st[PQHSA_ST_REQ], st[PQHSA_ST_KV_HEAD], pos);
      } else {
        off = a.sel_off[(size_t)row * a.kcap + (e - F)];
      }
    }
    // query slice of this lane, pre-multiplied by scale * log2(e)
    float qv[8];
    load8(static_cast<const E*>(a.q) + (size_t)row * kD + l16 * 8, qv);
#pragma unroll
    for (int d = 0; d < 8; ++d) qv[d] *= a.scale * kLog2e;

    // 2.+3. half-warp per row, kAttUnroll row pairs in flight
    float m = kNegInf, l = 0.f, acc[8];
#pragma unroll
    for (int d = 0; d < 8; ++d) acc[d] = 0.f;
    const int n_here = min(32, total - (c * kChunk + warp * 32));  // entries of this warp (may be <= 0)
    for (int i = 0; i < 16 && 2 * i < n_here; i += kAttUnroll) {
      RawRow<E> kr[kAttUnroll], vr[kAttUnroll];
      bool ok[kAttUnroll];
#pragma unroll
      for (int u = 0; u < kAttUnroll; ++u) {
        const int src = 2 * (i + u) + half;
        const long long o = __shfl_sync(0xffffffffu, off, src & 31) + l16 * 8;
        ok[u] = (i + u) < 16 && src < n_here;
        if (ok[u]) {
          ld_row(kb + o, kr[u]);
          ld_row(vb + o, vr[u]);
        } else {
          zero_row(kr[u]);
          zero_row(vr[u]);
        }
      }
      float x[kAttUnroll];
#pragma unroll
      for (int u = 0; u < kAttUnroll; ++u) {
        float kf[8];
        cvt_row(kr[u], kf);
        float d0 = kf[0] * qv[0];
#pragma unroll
        for (int d = 1; d < 8; ++d) d0 = fmaf(kf[d], qv[d], d0);
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) d0 += __shfl_xor_sync(0xffffffffu, d0, o);
        x[u] = ok[u] ? d0 : kNegInf;
      }
      float mx = m;
#pragma unroll
      for (int u = 0; u < kAttUnroll; ++u) mx = fmaxf(mx, x[u]);
      if (mx != kNegInf) {
        const float corr = ex2(m - mx);  // m == -inf gives 0
        l *= corr;
#pragma unroll
        for (int d = 0; d < 8; ++d) acc[d] *= corr;
#pragma unroll
        for (int u = 0; u < kAttUnroll; ++u) {
          const float pe = ex2(x[u] - mx);
          float vf[8];
          cvt_row(vr[u], vf);
          l += pe;
#pragma unroll
          for (int d = 0; d < 8; ++d) acc[d] = fmaf(pe, vf[d], acc[d]);
        }
        m = mx;
      }
    }
    // merge the two half-warps
    {
      const float mo = __shfl_xor_sync(0xffffffffu, m, 16);
      const float lo = __shfl_xor_sync(0xffffffffu, l, 16);
      const float mn = fmaxf(m, mo);
      const float cs = (m == kNegInf) ? 0.f : ex2(m - mn);
      const float co = (mo == kNegInf) ? 0.f : ex2(mo - mn);
      l = l * cs + lo * co;
#pragma unroll
      for (int d = 0; d < 8; ++d) {
        const float ao = __shfl_xor_sync(0xffffffffu, acc[d], 16);
        acc[d] = acc[d] * cs + ao * co;
      }
      m = mn;
    }
    __syncthreads();  // the previous item's partial has been written out
    if (half == 0) {
#pragma unroll
      for (int d = 0; d < 8; ++d) wacc[warp][l16 * 8 + d] = acc[d];
      if (l16 == 0) {
        wm[warp] = m;
        wl[warp] = l;
      }
    }
    __syncthreads();
    {
      float M = wm[0];
#pragma unroll
      for (int w = 1; w < kAttWarps; ++w) M = fmaxf(M, wm[w]);
      float L = 0.f, A = 0.f;
#pragma unroll
      for (int w = 0; w < kAttWarps; ++w) {
        const float f = (wm[w] == kNegInf) ? 0.f : ex2(wm[w] - M);
        L = fmaf(wl[w], f, L);
        A = fmaf(wacc[w][tid], f, A);
      }
      float* out = a.partial + ((size_t)row * a.chunks + c) * kPartial;
      out[2 + tid] = A;
      if (tid == 0) {
        out[0] = M;  // base-2 domain: scale * log2(e) * q.k
        out[1] = L;
      }
    }
  }
}

template <typename E>
static int launch_attend_t(const AttendArgs& a, cudaStream_t st) {
  static int per_sm = 0;  // resident CTAs per SM of this instantiation
  if (per_sm == 0) {
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, attend_kernel<E>, kAttThreads, 0) != cudaSuccess || n < 1)
      n = 4;
    per_sm = n;
  }
  const long long items = (long long)a.R * a.chunks;
  long long grid = (long long)sm_count() * per_sm;
  if (grid > items) grid = items;
  if (grid < 1) grid = 1;
  attend_kernel<E><<<(unsigned)grid, kAttThreads, 0, st>>>(a);
  return check_launch("attend");
}

int launch_attend(const pqhsa_params& p, const pqhsa_ws_layout& w, cudaStream_t st) {
  char* ws = static_cast<char*>(p.workspace);
  AttendArgs a;
  a.q = p.q;
  a.k_base = p.k_base;
  a.v_base = p.v_base;
  a.kv = make_kvaddr(p);
  a.state = static_cast<const int32_t*>(p.state);
  a.row_info = reinterpret_cast<const int32_t*>(ws + w.row_info);
  a.sel_off = reinterpret_cast<const long long*>(ws + w.sel_off);
  a.partial = reinterpret_cast<float*>(ws + w.partial);
  a.R = p.num_streams * p.group;
  a.G = p.group;
  a.kcap = w.kcap;
  a.chunks = w.chunks;
  a.sink = p.sink_tokens;
  a.scale = p.scale;
  PQHSA_DISPATCH_E(p.dtype, return (launch_attend_t<E>(a, st)));
  return PQHSA_OK;
}

}  // namespace pqhsa
