// Exact attention over sink + local-window rows and the selected keys, read in
// place from the (paged or contiguous) KV cache, the per-list background of the
// unselected keys, and the merge of all of it into one softmax.
//
// Replaces pq_attend_partial_nw(_paged)_kernel
// (pq_hsa/kernels/cuda/pq_fused_h20.cu:1225-1753); the arithmetic is the
// full_logits / exact_retrieval_logits part of
// pq_hsa/attention/sparse_attention.py:807-857.
//
// This is the HBM-bound kernel of the step: K + F random 256-byte K rows and V
// rows per query row.  Work item = (query row, chunk of 128 entries); entry e of
// a row is the e-th row of [sink | local | selected].  A persistent grid sized to
// the resident CTA count draws the items from a counter.  Inside a CTA each of the 4
// warps owns 32 entries:
//   1. lane-parallel: entry -> element offset of its K/V row (computed for sink
//      and local rows, read from sel_off for selected rows - one dependent load);
//   2. half-warp per row: 16 lanes x 16 bytes cover one 256-byte bf16 row
//      (2 x 16 bytes per lane for fp32); four row pairs (8 K rows + 8 V rows)
//      are requested before the first is consumed;
//   3. online softmax in the base-2 domain per half-warp; halves and warps are
//      merged at the end and one (max, sum, acc[128]) partial is written.
//
// Background.  One to five more items per query row turn the scan's per-unit (max, sum exp)
// pairs - selected keys already taken out by the selection kernel - and the tail logits into
// list masses and multiply them with the lists' value means ([1 x L] x [L x 128]): partials of
// the same form.  This is the centroid-mode background of
// pq_hsa/attention/sparse_attention.py:887-1012 in the list-space form argued for at
// pq_hsa/kernels/cuda/pq_fused_h20.cu:2043-2058 (it replaces pq_attend_bg, :2150-2242).
// Items are handed out by an atomic counter, background items first.
//
// Merge.  combine_kernel folds a row's partials - out = sum_p acc_p 2^(m_p - M) /
// sum_p l_p 2^(m_p - M) - and writes the output row (pq_attend_reduce_mw, :2244-2402); with
// several GPUs it also sends the rank's rows to the peers.
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
  float* partial;  // [R, chunks + kBgParts, kPartial]: the exact chunks, then the background parts
  int R, G, kcap, chunks, sink;
  float scale;
  // background and merge
  void* out;
  const void* vmeans;
  const uint16_t* list_ids;
  const uint16_t* unit_list;
  const float* unit_max;
  const float* unit_sum;
  const float* tail_logit;
  // output exchange between GPUs (peer_world <= 1: none)
  void* const* peer_out;
  int32_t* peer_seq;
  int32_t* combine_ticket;
  int peer_world, peer_rank;
  int32_t* row_ticket;  // [R], zero between launches
  unsigned long long* work_counter;  // [2]: next item, CTAs that have left; zero between launches
  int cap, ucap, tail_cap, num_lists;
  int bg_parts;  // background items per query row in this launch (1 .. kBgParts)
  // Kept last: measured, the gather kernel compiles to 78 registers and runs 9 % faster than with this pointer
  // next to q (same source otherwise).
  const int32_t* io_map;  // [S] block of q / out of a stream, or null: block s
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

constexpr int kBgGroups = kAttThreads / 16;  // 16 threads x 8 dims cover one value-mean row

// One of the background partials of a query row (all kAttThreads threads): list masses from the
// per-unit (max, sum) pairs of a share of the row's units - consecutive units, hence a contiguous
// range of lists - times those lists' value means.  The unselected keys of the unsorted tail, whose
// lists are arbitrary, are a part of their own (range = all lists, lists without mass are skipped);
// with a single unit part they ride along with it.
template <typename E>
__device__ __forceinline__ void background_item(const AttendArgs& a, int row, int s, int part, const StreamGeom& geo,
                                                float* pout, float* mass, float (*gacc)[kD], float* red) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float* umax = a.unit_max + (size_t)row * a.ucap;
  const float* usum = a.unit_sum + (size_t)row * a.ucap;
  const float* tl = a.tail_logit + (size_t)row * a.tail_cap;
  const uint16_t* ulist = a.unit_list + (size_t)s * a.ucap;
  const uint16_t* tlist = a.list_ids + (size_t)s * a.cap + geo.n_sorted;
  // unit parts 0 .. bg_units - 1; the tail rides with part 0 when there is one unit part, else it is a part of its own
  const int bg_units = a.bg_parts > 1 ? a.bg_parts - 1 : 1;
  const bool unit_part = part < bg_units;
  const int u_lo = unit_part ? (int)((long long)geo.n_units * part / bg_units) : 0;
  const int u_hi = unit_part ? (int)((long long)geo.n_units * (part + 1) / bg_units) : 0;
  const int n_tail = (a.bg_parts == 1 || !unit_part) ? geo.n_tail : 0;
  int l_lo = u_lo < u_hi ? (int)ulist[u_lo] : 0, l_hi = u_lo < u_hi ? (int)ulist[u_hi - 1] + 1 : 0;
  if (n_tail > 0) {
    l_lo = 0;
    l_hi = a.num_lists;
  }
  for (int i = l_lo + tid; i < l_hi; i += kAttThreads) mass[i] = 0.f;
  // reference of the partial: the largest unit maximum / tail logit of the part, base-2 domain
  float m = kNegInf;
  for (int u = u_lo + tid; u < u_hi; u += kAttThreads) m = fmaxf(m, umax[u]);
  for (int t = tid; t < n_tail; t += kAttThreads) m = fmaxf(m, tl[t]);
  m = warp_max(m * kLog2e);
  __syncthreads();  // also: the previous item is done with the shared arrays, mass[] is zero
  if (lane == 0) red[warp] = m;
  __syncthreads();
  float M = red[0];
#pragma unroll
  for (int w = 1; w < kAttWarps; ++w) M = fmaxf(M, red[w]);
  float tot = 0.f;
  if (M != kNegInf) {
    for (int u = u_lo + tid; u < u_hi; u += kAttThreads) {
      const float v = usum[u] * ex2(fmaf(umax[u], kLog2e, -M));
      atomicAdd(&mass[ulist[u]], v);
      tot += v;
    }
    for (int t = tid; t < n_tail; t += kAttThreads) {
      const float x = tl[t];
      if (x != kNegInf) {  // -inf marks a selected tail slot
        const float v = ex2(fmaf(x, kLog2e, -M));
        atomicAdd(&mass[tlist[t]], v);
        tot += v;
      }
    }
  }
  tot = warp_sum(tot);
  __syncthreads();  // red[] has been read; mass[] is complete after the next barrier
  if (lane == 0) red[warp] = tot;
  __syncthreads();
  float L = 0.f;
#pragma unroll
  for (int w = 0; w < kAttWarps; ++w) L += red[w];
  // sum_l mass[l] * vmean[l][:]: list = l_lo + lg + kBgGroups * i, dims d8*8 .. d8*8+7, 8 rows in flight
  const int d8 = tid & 15, lg = tid >> 4;
  const E* vm = static_cast<const E*>(a.vmeans) + (size_t)s * a.num_lists * kD + d8 * 8;
  float acc[8];
#pragma unroll
  for (int d = 0; d < 8; ++d) acc[d] = 0.f;
  for (int l0 = l_lo + lg; l0 < l_hi; l0 += kBgGroups * 8) {
    RawRow<E> vr[8];
    float w[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int l = l0 + kBgGroups * i;
      w[i] = l < l_hi ? mass[l] : 0.f;
      if (w[i] != 0.f) ld_row(vm + (size_t)l * kD, vr[i]); else zero_row(vr[i]);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float v[8];
      cvt_row(vr[i], v);
#pragma unroll
      for (int d = 0; d < 8; ++d) acc[d] = fmaf(w[i], v[d], acc[d]);
    }
  }
#pragma unroll
  for (int d = 0; d < 8; ++d) gacc[lg][d8 * 8 + d] = acc[d];
  __syncthreads();
  float o = gacc[0][tid];
#pragma unroll
  for (int j = 1; j < kBgGroups; ++j) o += gacc[j][tid];
  pout[2 + tid] = o;
  if (tid == 0) {
    pout[0] = M;
    pout[1] = L;
  }
}

// MAPPED: the streams' query blocks are looked up in io_map (a separate instantiation, so that the plain case keeps
// its address arithmetic free of the lookup).
template <typename E, bool MAPPED>
__global__ void __launch_bounds__(kAttThreads, 6) attend_kernel(const AttendArgs a) {
  __shared__ float wm[kAttWarps], wl[kAttWarps];
  __shared__ float wacc[kAttWarps][kD];
  __shared__ float mass[kLMax];
  __shared__ float gacc[kBgGroups][kD];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int half = lane >> 4, l16 = lane & 15;
  const E* kb = static_cast<const E*>(a.k_base);
  const E* vb = static_cast<const E*>(a.v_base);
  const int slots = a.chunks + kBgParts;  // partial slots per row (a.bg_parts of the background slots are used)
  const long long items = (long long)a.R * (a.chunks + a.bg_parts);

  // Items are handed out by a counter (a CTA that drew a long item draws fewer): first the rows'
  // background items (long dependent chains), then the chunks row by row, so that rows finish - and
  // get merged - one after the other instead of all at the very end.  A CTA asks for its next item
  // before it works on the current one.
  __shared__ long long item_s;
  if (tid == 0) item_s = (long long)atomicAdd(a.work_counter, 1ull);
  __syncthreads();
  long long item = item_s;
  while (item < items) {
    __syncthreads();  // everybody has read item_s
    long long nxt = 0;
    if (tid == 0) nxt = (long long)atomicAdd(a.work_counter, 1ull);  // used at the end of the item: the round trip is hidden
    const bool is_bg = item < (long long)a.R * a.bg_parts;
    const int row = (int)(item % a.R);
    const int c = is_bg ? a.chunks + (int)(item / a.R) : (int)(item / a.R) - a.bg_parts;
    const int s = row / a.G;
    const int32_t* st = a.state + (size_t)s * kST;
    const StreamGeom geo = stream_geom(st, a.sink);
    const int F = geo.full;
    const int K = a.row_info[(size_t)row * kRI + PQHSA_RI_K];
    const int total = F + K;
    const int nchunks = (total + kChunk - 1) / kChunk;
    float* pout = a.partial + ((size_t)row * slots + c) * kPartial;
    if (c < a.chunks && c >= nchunks) {  // uniform per block: an empty chunk
      if (tid == 0) {
        pout[0] = kNegInf;
        pout[1] = 0.f;
        item_s = nxt;
      }
      __syncthreads();
      item = item_s;
      continue;
    }

    if (c >= a.chunks) {
      background_item<E>(a, row, s, c - a.chunks, geo, pout, mass, gacc, wm);
    } else {

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
    if constexpr (MAPPED) {
      const int qb = a.io_map[s];  // negative: idle stream (it has no entries either)
      if (qb >= 0) {
        load8(static_cast<const E*>(a.q) + ((size_t)qb * a.G + (row - s * a.G)) * kD + l16 * 8, qv);
      } else {
#pragma unroll
        for (int d = 0; d < 8; ++d) qv[d] = 0.f;
      }
    } else {
      load8(static_cast<const E*>(a.q) + (size_t)row * kD + l16 * 8, qv);
    }
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
      {
        // the lane's share of the four dot products, then their sums over the 16 lanes of the half-warp:
        // a halving exchange (lane bits 3, 2 pick which product a lane ends up with) and a broadcast -
        // 9 shuffles instead of 16
        static_assert(kAttUnroll == 4, "the reduction below is written for four rows");
        float dp[kAttUnroll];
#pragma unroll
        for (int u = 0; u < kAttUnroll; ++u) {
          float kf[8];
          cvt_row(kr[u], kf);
          // two dims per instruction (packed f32x2 multiply-add)
          float2 d2 = __fmul2_rn(make_float2(kf[0], kf[1]), make_float2(qv[0], qv[1]));
#pragma unroll
          for (int d = 2; d < 8; d += 2) d2 = __ffma2_rn(make_float2(kf[d], kf[d + 1]), make_float2(qv[d], qv[d + 1]), d2);
          dp[u] = d2.x + d2.y;
        }
        const bool b3 = (lane & 8) != 0, b2 = (lane & 4) != 0;
        const float e0 = (b3 ? dp[2] : dp[0]) + __shfl_xor_sync(0xffffffffu, b3 ? dp[0] : dp[2], 8);
        const float e1 = (b3 ? dp[3] : dp[1]) + __shfl_xor_sync(0xffffffffu, b3 ? dp[1] : dp[3], 8);
        float f = (b2 ? e1 : e0) + __shfl_xor_sync(0xffffffffu, b2 ? e0 : e1, 4);
        f += __shfl_xor_sync(0xffffffffu, f, 2);
        f += __shfl_xor_sync(0xffffffffu, f, 1);  // lanes with (bit 3, bit 2) = (u >> 1, u & 1) hold product u
#pragma unroll
        for (int u = 0; u < kAttUnroll; ++u) {
          const float d0 = __shfl_sync(0xffffffffu, f, (lane & 16) | ((u >> 1) << 3) | ((u & 1) << 2));
          x[u] = ok[u] ? d0 : kNegInf;
        }
      }
      float mx = m;
#pragma unroll
      for (int u = 0; u < kAttUnroll; ++u) mx = fmaxf(mx, x[u]);
      if (mx != kNegInf) {
        const float corr = ex2(m - mx);  // m == -inf gives 0
        l *= corr;
        const float2 c2 = make_float2(corr, corr);
#pragma unroll
        for (int d = 0; d < 8; d += 2) {
          const float2 t = __fmul2_rn(make_float2(acc[d], acc[d + 1]), c2);
          acc[d] = t.x;
          acc[d + 1] = t.y;
        }
#pragma unroll
        for (int u = 0; u < kAttUnroll; ++u) {
          const float pe = ex2(x[u] - mx);
          const float2 p2 = make_float2(pe, pe);
          float vf[8];
          cvt_row(vr[u], vf);
          l += pe;
#pragma unroll
          for (int d = 0; d < 8; d += 2) {
            const float2 t = __ffma2_rn(make_float2(vf[d], vf[d + 1]), p2, make_float2(acc[d], acc[d + 1]));
            acc[d] = t.x;
            acc[d + 1] = t.y;
          }
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
      pout[2 + tid] = A;
      if (tid == 0) {
        pout[0] = M;  // base-2 domain: scale * log2(e) * q.k
        pout[1] = L;
      }
    }
    }  // chunk item

    if (tid == 0) item_s = nxt;
    __syncthreads();
    item = item_s;
  }
  // the CTA that leaves last puts the counters back to zero for the next launch
  if (tid == 0) {
    __threadfence();
    if (atomicAdd(a.work_counter + 1, 1ull) == (unsigned long long)gridDim.x - 1) {
      a.work_counter[0] = 0ull;
      a.work_counter[1] = 0ull;
    }
  }
}

// A flagged word: 8 bytes stored and loaded as one transaction (the data and the step count that says it is there).
__device__ __forceinline__ void store_flagged(uint2* p, uint32_t data, uint32_t flag) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(data), "r"(flag) : "memory");
}
__device__ __forceinline__ uint2 load_flagged(const uint2* p) {
  uint2 v;
  asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}

// One CTA per query row folds the row's partials (exact chunks + background) into the output row:
// out = sum_p acc_p 2^(m_p - M) / sum_p l_p 2^(m_p - M)  (pq_attend_reduce_mw,
// pq_hsa/kernels/cuda/pq_fused_h20.cu:2244-2402).  Thread d owns output dim d.  Everything a thread needs
// of 32 partials - their (max, sum) pairs, which every thread of a warp reads from the same
// addresses, and its own dim of their accumulators - is requested at once: one round trip per 32 partials, no barrier.
template <typename E>
__global__ void __launch_bounds__(kD) combine_kernel(const AttendArgs a) {
  const int row = blockIdx.x, tid = threadIdx.x;
  const int slots = a.chunks + a.bg_parts;  // <= kD, checked with the parameters; empty chunks carry (-inf, 0)
  const float* pp = a.partial + (size_t)row * (a.chunks + kBgParts) * kPartial;
  // 32 partials at a time, all of a batch requested at once (one round trip per batch; c2 has 27 partials per row,
  // a row of 5243 selected keys 47); the batches are folded into a running (max, sum, acc)
  constexpr int kBatch = 32;
  float M = kNegInf, L = 0.f, A = 0.f;
  for (int p0 = 0; p0 < slots; p0 += kBatch) {
    float m[kBatch], l[kBatch], v[kBatch];
#pragma unroll
    for (int p = 0; p < kBatch; ++p) {
      m[p] = kNegInf;
      l[p] = 0.f;
      v[p] = 0.f;
      if (p0 + p < slots) {
        m[p] = __ldcg(pp + (size_t)(p0 + p) * kPartial);
        l[p] = __ldcg(pp + (size_t)(p0 + p) * kPartial + 1);
        v[p] = __ldcg(pp + (size_t)(p0 + p) * kPartial + 2 + tid);
      }
    }
    float Mb = m[0];
#pragma unroll
    for (int p = 1; p < kBatch; ++p) Mb = fmaxf(Mb, m[p]);
    if (Mb == kNegInf) continue;  // a batch of empty chunks
    const float Mn = fmaxf(M, Mb);
    const float fo = (M == kNegInf) ? 0.f : ex2(M - Mn);
    L *= fo;
    A *= fo;
#pragma unroll
    for (int p = 0; p < kBatch; ++p) {
      const float f = (m[p] == kNegInf) ? 0.f : ex2(m[p] - Mn);
      L = fmaf(l[p], f, L);
      A = fmaf(v[p], f, A);
    }
    M = Mn;
  }
  const E res = from_f<E>(A / fmaxf(L, 1.17549435e-38f));
  {
    const int s = row / a.G;
    const int ob = a.io_map != nullptr ? a.io_map[s] : s;  // negative: idle stream, nothing to write
    if (ob >= 0) static_cast<E*>(a.out)[((size_t)ob * a.G + (row - s * a.G)) * kD + tid] = res;
  }
  if (a.peer_world > 1) {
    // Every CTA sends its own row to every rank as flagged words: 8-byte stores (4 bytes of the row, the step
    // count) into peer memory over NVLink.  A word arrives whole, so the receiver needs no fence and no flag
    // besides it, and nobody waits here.  The CTA that arrives last at the ticket counts the step.
    __shared__ __align__(16) E row_s[kD];
    const int seq0 = a.peer_seq[0];  // steps before this one: only the last CTA changes it, after all have read it
    row_s[tid] = res;
    __syncthreads();
    constexpr int kWords = kD * (int)sizeof(E) / 4;  // flagged words per row
    const uint32_t* row_w = reinterpret_cast<const uint32_t*>(row_s);
    const size_t at = (((size_t)(seq0 & 1) * a.peer_world + a.peer_rank) * a.R + row) * kWords;
    for (int w = tid; w < kWords; w += kD) {
      const uint32_t payload = row_w[w];
      for (int r = 0; r < a.peer_world; ++r)
        store_flagged(static_cast<uint2*>(a.peer_out[r]) + at + w, payload, (uint32_t)(seq0 + 1));
    }
    __syncthreads();  // every thread has read the step count
    if (tid == 0) {
      const int t = atomicAdd(a.combine_ticket, 1);
      if (t == (int)gridDim.x - 1) {
        a.combine_ticket[0] = 0;
        a.peer_seq[0] = seq0 + 1;
      }
    }
  }
}

// Receiving side: one thread per flagged word of this step's parity.  It polls its word (bounded: `polls` polls
// about 100 ns apart) until the word carries the step count, then stores the 4 bytes into the gathered rows.  When a
// wait runs out the error flag is set, the word is skipped and the thread returns.
__global__ void __launch_bounds__(256) wait_peers_kernel(const uint2* const* peer_out, int rank, uint32_t* gather,
                                                         int32_t* peer_seq, long long words, int polls) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= words) return;
  const uint2* recv = peer_out[rank];  // this rank's own receive buffer
  const int target = peer_seq[0];  // counted by the combine kernel of this step, which ran before on this stream
  const size_t at = (size_t)((target - 1) & 1) * (size_t)words + (size_t)i;
  for (int it = 0; it < polls; ++it) {
    const uint2 w = load_flagged(recv + at);
    if ((int)w.y == target) {
      gather[at] = w.x;
      return;
    }
    __nanosleep(100);
  }
  peer_seq[1] = 1;
}

template <typename E, bool MAPPED>
static int launch_attend_t(const AttendArgs& a, bool combine, cudaStream_t st) {
  static int per_sm = 0;  // resident CTAs per SM of this instantiation
  if (per_sm == 0) {
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, attend_kernel<E, MAPPED>, kAttThreads, 0) != cudaSuccess || n < 1)
      n = 4;
    per_sm = n;
  }
  const long long items = (long long)a.R * (a.chunks + a.bg_parts);
  long long grid = (long long)sm_count() * per_sm;
  if (grid > items) grid = items;
  if (grid < 1) grid = 1;
  if (combine) {
    combine_kernel<E><<<(unsigned)a.R, kD, 0, st>>>(a);
    return check_launch("combine");
  }
  attend_kernel<E, MAPPED><<<(unsigned)grid, kAttThreads, 0, st>>>(a);
  return check_launch("attend");
}

static int launch_attend_or_combine(const pqhsa_params& p, const pqhsa_ws_layout& w, bool combine, cudaStream_t st) {
  char* ws = static_cast<char*>(p.workspace);
  AttendArgs a;
  a.q = p.q;
  a.io_map = p.io_map;
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
  a.out = p.out;
  a.vmeans = p.vmeans;
  a.list_ids = static_cast<const uint16_t*>(p.list_ids);
  a.unit_list = static_cast<const uint16_t*>(p.unit_list);
  a.unit_max = reinterpret_cast<const float*>(ws + w.unit_max);
  a.unit_sum = reinterpret_cast<const float*>(ws + w.unit_sum);
  a.tail_logit = reinterpret_cast<const float*>(ws + w.tail_logit);
  a.peer_out = static_cast<void* const*>(p.peer_out);
  a.peer_seq = static_cast<int32_t*>(p.peer_seq);
  a.combine_ticket = reinterpret_cast<int32_t*>(ws + w.combine_ticket);
  a.peer_world = p.peer_world;
  a.peer_rank = p.peer_rank;
  a.row_ticket = reinterpret_cast<int32_t*>(ws + w.row_ticket);
  a.work_counter = reinterpret_cast<unsigned long long*>(ws + w.work_counter);
  a.cap = p.slot_capacity;
  a.ucap = p.unit_capacity;
  a.tail_cap = w.tail_cap;
  a.num_lists = p.num_lists;
  // Few rows: the background of a row is a long chain and would be the kernel's critical path, so it is cut
  // into parts.  Many rows: the parts only add items, and one item per row hides behind the chunk items.
  a.bg_parts = a.R >= 96 ? 1 : kBgParts;  // kBgParts - 1 unit parts + the tail part
  if (a.io_map != nullptr) {
    PQHSA_DISPATCH_E(p.dtype, return (launch_attend_t<E, true>(a, combine, st)));
  }
  PQHSA_DISPATCH_E(p.dtype, return (launch_attend_t<E, false>(a, combine, st)));
  return PQHSA_OK;
}

int launch_attend(const pqhsa_params& p, const pqhsa_ws_layout& w, cudaStream_t st) {
  return launch_attend_or_combine(p, w, false, st);
}
int launch_wait_peers(const pqhsa_params& p, cudaStream_t st) {
  const size_t esz = p.dtype == PQHSA_F32 ? 4 : 2;
  const long long words = (long long)p.peer_world * p.num_streams * p.group * (long long)(kD * esz / 4);
  wait_peers_kernel<<<(unsigned)((words + 255) / 256), 256, 0, st>>>(
      static_cast<const uint2* const*>(p.peer_out), p.peer_rank, static_cast<uint32_t*>(p.peer_gather),
      static_cast<int32_t*>(p.peer_seq), words, p.peer_wait_polls > 0 ? p.peer_wait_polls : (1 << 22));
  return check_launch("wait_peers");
}

int launch_merge(const pqhsa_params& p, const pqhsa_ws_layout& w, cudaStream_t st) {
  return launch_attend_or_combine(p, w, true, st);
}

}  // namespace pqhsa
