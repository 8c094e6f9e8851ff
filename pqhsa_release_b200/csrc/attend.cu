// Exact attention over sink + local-window rows and the selected keys, read in
// place from the (paged or contiguous) KV cache: split-K partials.
//
// Replaces pq_attend_partial_nw(_paged)_kernel
// (pq_hsa/kernels/cuda/pq_fused_h20.cu:1225-1753); the arithmetic is the
// full_logits / exact_retrieval_logits part of
// pq_hsa/attention/sparse_attention.py:807-857.
//
// Work item = (query row, chunk of 256 entries); entry e of a row is the e-th
// row of [sink | local | selected].  A persistent grid strides over the items.
// Inside a CTA each of the 8 warps owns 32 entries:
//   1. lane-parallel: entry -> token position -> cache offset.  A selected entry
//      also leaves the approximate side of the softmax here: its logit is
//      re-scored from the code (bit-identical to the scan) and exactly the term
//      the scan added for it is subtracted from its unit's exp-sum (a selected
//      tail slot has its stored logit set to -inf).  This is the
//      "- old_exact_exp" of pq_hsa/attention/sparse_attention.py:985-1009,
//      done per unit so that no cancellation error is left behind;
//   2. half-warp per K/V row: 16 lanes x 16 bytes cover one 256-byte bf16 row
//      (2 x 16 bytes per lane for fp32), four row pairs (8 K rows + 8 V rows)
//      are in flight per warp before the first is consumed;
//   3. online softmax in the base-2 domain per half-warp, halves and warps are
//      merged at the end and one (max, sum, acc[128]) partial is written.
#include "common.cuh"

namespace pqhsa {

constexpr int kAttThreads = 256;
constexpr int kAttWarps = kAttThreads / 32;
constexpr int kAttUnroll = 4;  // row pairs in flight per warp

struct AttendArgs {
  const void* q;
  const void* k_base;
  const void* v_base;
  KvAddr kv;
  const uint32_t* codes;
  const void* norms;
  const uint16_t* list_ids;
  const uint16_t* slot_unit;
  const int32_t* slot_pos;
  const int32_t* state;
  const float* lut;
  const float* list_scores;
  const int32_t* row_info;
  const int32_t* sel_slot;
  const float* unit_max;
  float* unit_sum;
  float* tail_logit;
  float* partial;
  int R, G, cap, ucap, tail_cap, kcap, chunks, sink;
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
  const uint32_t w[4] = {r.a.x, r.a.y, r.a.z, r.a.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
__device__ __forceinline__ void cvt_row(const RawRow<__half>& r, float (&v)[8]) {
  const uint32_t w[4] = {r.a.x, r.a.y, r.a.z, r.a.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}

template <typename E>
__global__ void __launch_bounds__(kAttThreads, 2) attend_kernel(const AttendArgs a) {
  __shared__ float lut_s[kM * kC];
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
    const int n_sorted = st[PQHSA_ST_N_SORTED];
    const int n_idx = n_sorted + st[PQHSA_ST_N_TAIL];
    const int seq_len = st[PQHSA_ST_SEQ_LEN];
    const int sink_end = min(a.sink, seq_len);
    const int retr_end = sink_end + n_idx;
    const int F = sink_end + max(seq_len - retr_end, 0);
    const int K = a.row_info[(size_t)row * kRI + PQHSA_RI_K];
    const int total = F + K;
    if (c * kChunk >= total) continue;  // uniform per block
    const int req = st[PQHSA_ST_REQ], head = st[PQHSA_ST_KV_HEAD];

    __syncthreads();  // previous item's shared memory is free
    if (tid < kM * kC) lut_s[tid] = a.lut[(size_t)row * kM * kC + tid];
    __syncthreads();

    // query slice of this lane, pre-multiplied by scale * log2(e)
    float qv[8];
    load8(static_cast<const E*>(a.q) + (size_t)row * kD + l16 * 8, qv);
#pragma unroll
    for (int d = 0; d < 8; ++d) qv[d] *= a.scale * kLog2e;

    // 1. entry metadata, one entry per lane
    const int e = c * kChunk + warp * 32 + lane;
    long long off = 0;
    if (e < total) {
      int pos;
      if (e < F) {
        pos = e < sink_end ? e : retr_end + (e - sink_end);
      } else {
        const int slot = a.sel_slot[(size_t)row * a.kcap + (e - F)];
        pos = a.slot_pos[(size_t)s * a.cap + slot];
        if (slot < n_sorted) {
          const uint32_t code = __ldg(a.codes + (size_t)s * a.cap + slot);
          const int lid = a.list_ids[(size_t)s * a.cap + slot];
          const int u = a.slot_unit[(size_t)s * a.cap + slot];
          const float kn = to_f(static_cast<const E*>(a.norms)[(size_t)s * a.cap + slot]);
          const float x = finish_logit(pq_sum_row(lut_s, code), __ldg(a.list_scores + (size_t)row * kLMax + lid), kn);
          atomicAdd(a.unit_sum + (size_t)row * a.ucap + u, -unit_term(x, a.unit_max[(size_t)row * a.ucap + u]));
        } else {
          a.tail_logit[(size_t)row * a.tail_cap + (slot - n_sorted)] = kNegInf;
        }
      }
      off = a.kv.offset(req, head, pos);
    }

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
    if (half == 0) {
#pragma unroll
      for (int d = 0; d < 8; ++d) wacc[warp][l16 * 8 + d] = acc[d];
      if (l16 == 0) {
        wm[warp] = m;
        wl[warp] = l;
      }
    }
    __syncthreads();
    if (tid < kD) {
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

int sm_count();

int launch_attend(const pqhsa_params& p, const pqhsa_ws_layout& w, cudaStream_t st) {
  char* ws = static_cast<char*>(p.workspace);
  AttendArgs a;
  a.q = p.q;
  a.k_base = p.k_base;
  a.v_base = p.v_base;
  a.kv = make_kvaddr(p);
  a.codes = static_cast<const uint32_t*>(p.codes);
  a.norms = p.norms;
  a.list_ids = static_cast<const uint16_t*>(p.list_ids);
  a.slot_unit = static_cast<const uint16_t*>(p.slot_unit);
  a.slot_pos = static_cast<const int32_t*>(p.slot_pos);
  a.state = static_cast<const int32_t*>(p.state);
  a.lut = reinterpret_cast<const float*>(ws + w.lut);
  a.list_scores = reinterpret_cast<const float*>(ws + w.list_scores);
  a.row_info = reinterpret_cast<const int32_t*>(ws + w.row_info);
  a.sel_slot = reinterpret_cast<const int32_t*>(ws + w.sel_slot);
  a.unit_max = reinterpret_cast<const float*>(ws + w.unit_max);
  a.unit_sum = reinterpret_cast<float*>(ws + w.unit_sum);
  a.tail_logit = reinterpret_cast<float*>(ws + w.tail_logit);
  a.partial = reinterpret_cast<float*>(ws + w.partial);
  a.R = p.num_streams * p.group;
  a.G = p.group;
  a.cap = p.slot_capacity;
  a.ucap = p.unit_capacity;
  a.tail_cap = w.tail_cap;
  a.kcap = w.kcap;
  a.chunks = w.chunks;
  a.sink = p.sink_tokens;
  a.scale = p.scale;
  const long long items = (long long)a.R * a.chunks;
  long long grid = (long long)sm_count() * 4;
  if (grid > items) grid = items;
  if (grid < 1) grid = 1;
  PQHSA_DISPATCH_E(p.dtype, attend_kernel<E><<<(unsigned)grid, kAttThreads, 0, st>>>(a));
  return check_launch("attend");
}

}  // namespace pqhsa
