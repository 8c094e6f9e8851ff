// Incremental encode of keys that have left the local window (shared by the stand-alone
// append_encode kernel and the fused first kernel of a decode step).
//
// Mirrors IVFPQIndex.add with fixed codebooks (pq_hsa/index/ivfpq.py:598-645): |k| and
// direction (:1052-1059), nearest list by Euclidean distance (:1001-1005), residual
// (:1012-1016), nearest code word per subspace (pq_hsa/index/pq.py:97-115), nibble packing
// (pq_hsa/index/packing.py:6-34); and the running per-list value mean of
// pq_hsa/attention/kv_cache.py:730-776.  All arithmetic is fp32 on the stored element
// values; ties go to the lower index as torch.argmin does.
#pragma once
#include "common.cuh"

namespace pqhsa {

struct EncodeArgs {
  uint32_t* codes;
  void* norms;
  uint16_t* list_ids;
  int32_t* slot_pos;
  const void* coarse;
  const void* codebooks;
  void* vmeans;
  float* vsum;
  int32_t* vcnt;
  int32_t* state;
  float* norm_max;
  const void* k_base;
  const void* v_base;
  KvAddr kv;
  const int32_t* enc_count;
  int uniform_count, cap, tail_cap, num_lists, sink;
};

inline EncodeArgs make_encode_args(const pqhsa_params& p, const int32_t* cnt, int32_t uni) {
  EncodeArgs a;
  a.codes = static_cast<uint32_t*>(const_cast<void*>(p.codes));
  a.norms = const_cast<void*>(p.norms);
  a.list_ids = static_cast<uint16_t*>(const_cast<void*>(p.list_ids));
  a.slot_pos = static_cast<int32_t*>(const_cast<void*>(p.slot_pos));
  a.coarse = p.coarse;
  a.codebooks = p.codebooks;
  a.vmeans = const_cast<void*>(p.vmeans);
  a.vsum = static_cast<float*>(p.vsum);
  a.vcnt = static_cast<int32_t*>(p.vcnt);
  a.state = static_cast<int32_t*>(p.state);
  a.norm_max = static_cast<float*>(p.norm_max);
  a.k_base = p.k_base;
  a.v_base = p.v_base;
  a.kv = make_kvaddr(p);
  a.enc_count = cnt;
  a.uniform_count = uni;
  a.cap = p.slot_capacity;
  a.tail_cap = p.tail_capacity;
  a.num_lists = p.num_lists;
  a.sink = p.sink_tokens;
  return a;
}

// Shared-memory scratch of the encode steps of one CTA of THREADS threads.
template <int THREADS> struct EncodeShared {
  float unit[kD];
  float resid[kD];
  float red[THREADS / 32];
  float best_d[THREADS / 32];
  int best_l[THREADS / 32];
  uint32_t code_sh;
  int list_sh;
};

// Step 1: |k| (clamped at 1e-12) of the key row whose element tid this thread holds in kval (tid < 128; 0 otherwise),
// its unit direction into sh.unit.  All threads of the CTA call; all get the norm.  The squared norm is four 32-dim
// butterfly sums added left to right.
template <int THREADS>
__device__ __forceinline__ float enc_direction(float kval, EncodeShared<THREADS>& sh) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float sq = warp_sum(kval * kval);
  __syncthreads();
  if (lane == 0) sh.red[warp] = sq;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < THREADS / 32; ++i) tot += sh.red[i];
  const float nrm = fmaxf(sqrtf(tot), 1e-12f);
  if (tid < kD) sh.unit[tid] = kval / nrm;
  __syncthreads();
  return nrm;
}
template <typename E, int THREADS>
__device__ __forceinline__ float enc_direction(const E* __restrict__ kb, long long off, EncodeShared<THREADS>& sh) {
  return enc_direction<THREADS>(threadIdx.x < kD ? to_f(kb[off + threadIdx.x]) : 0.f, sh);
}

// The best (distance, then lower list index) of the threads' candidates over the CTA; all threads call, the result is
// valid in thread 0.
template <int THREADS>
__device__ __forceinline__ void enc_best_of_cta(float& bd, int& bl, EncodeShared<THREADS>& sh) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float od = __shfl_xor_sync(0xffffffffu, bd, o);
    const int ol = __shfl_xor_sync(0xffffffffu, bl, o);
    if (od < bd || (od == bd && ol < bl)) {
      bd = od;
      bl = ol;
    }
  }
  if (lane == 0) {
    sh.best_d[warp] = bd;
    sh.best_l[warp] = bl;
  }
  __syncthreads();
  if (tid == 0) {
    for (int i = 1; i < THREADS / 32; ++i)
      if (sh.best_d[i] < bd || (sh.best_d[i] == bd && sh.best_l[i] < bl)) {
        bd = sh.best_d[i];
        bl = sh.best_l[i];
      }
  }
  __syncthreads();  // best_d / best_l may be rewritten by the next call
}

// Step 2: nearest of the lists [l_begin, l_end) (clipped to [0, nl)) to sh.unit: argmin_l |u - c_l|^2 with ties to the
// lower index, as torch.argmin.  4 lanes per list (32 dims each, kept as raw 16-byte vectors), THREADS / 4 lists per
// pass, kBatch passes of loads in flight.  A list's distance is (p0 + p1) + (p2 + p3), p_q the fmaf chain of
// (u_d - c_d)^2 over dims 32q .. 32q+31 - the same value whichever CTA computes it, so the search can be split over
// CTAs by list range and the partial winners merged.  All threads call; the result is valid in thread 0.
template <typename E, int THREADS>
__device__ __forceinline__ void enc_nearest_list(const E* __restrict__ coarse, int l_begin, int l_end, int nl,
                                                 EncodeShared<THREADS>& sh, float& out_d, int& out_l) {
  const int tid = threadIdx.x;
  const int sub = tid & 3, grp = tid >> 2;  // groups of 4 lanes
  constexpr int kGroups = THREADS / 4;
  constexpr int kVecs = 32 * (int)sizeof(E) / 16;  // 16-byte vectors per 32 dims
  constexpr int kBatch = sizeof(E) == 2 ? 4 : 2;   // lists per thread in flight
  l_end = min(l_end, nl);
  uint4 raw[kBatch][kVecs];
  auto load_batch = [&](int l0) {
#pragma unroll
    for (int h = 0; h < kBatch; ++h) {
      const int l = l0 + h * kGroups + grp;
      if (l < l_end) {
        const uint4* src = reinterpret_cast<const uint4*>(coarse + (size_t)l * kD + sub * 32);
#pragma unroll
        for (int j = 0; j < kVecs; ++j) raw[h][j] = __ldg(src + j);
      }
    }
  };
  load_batch(l_begin);
  float bd = __builtin_huge_valf();
  int bl = 0;  // stays in range when every distance is NaN (a key row holding NaN or Inf): argmin then gives list 0
  float uq[32];
#pragma unroll
  for (int d = 0; d < 32; ++d) uq[d] = sh.unit[sub * 32 + d];
  for (int l0 = l_begin; l0 < l_end; l0 += kBatch * kGroups) {
    if (l0 > l_begin) load_batch(l0);
#pragma unroll
    for (int h = 0; h < kBatch; ++h) {
      const int l = l0 + h * kGroups + grp;
      float dist = 0.f;
      if (l < l_end) {
#pragma unroll
        for (int j = 0; j < kVecs; ++j) {
          if constexpr (sizeof(E) == 2) {
            float c8[8];
            unpack8(raw[h][j], static_cast<const E*>(nullptr), c8);
#pragma unroll
            for (int d = 0; d < 8; ++d) {
              const float df = uq[j * 8 + d] - c8[d];
              dist = fmaf(df, df, dist);
            }
          } else {
            const float c4[4] = {__uint_as_float(raw[h][j].x), __uint_as_float(raw[h][j].y),
                                 __uint_as_float(raw[h][j].z), __uint_as_float(raw[h][j].w)};
#pragma unroll
            for (int d = 0; d < 4; ++d) {
              const float df = uq[j * 4 + d] - c4[d];
              dist = fmaf(df, df, dist);
            }
          }
        }
      }
      dist += __shfl_xor_sync(0xffffffffu, dist, 1);
      dist += __shfl_xor_sync(0xffffffffu, dist, 2);
      if (l < l_end && dist < bd) {  // l ascends within a thread, so strict < keeps the lowest index on ties
        bd = dist;
        bl = l;
      }
    }
  }
  enc_best_of_cta<THREADS>(bd, bl, sh);
  out_d = bd;
  out_l = bl;
}

// Step 3: residual against the winning list, nearest code word per subspace (thread (m, c) for tid < 128 holds code
// word c of subspace m in cwv), the slot's index entry, and the running value mean of the list (vval = this thread's
// element of the value row, tid < 128).  All threads call.
template <typename E, int THREADS>
__device__ __forceinline__ void enc_finish(const EncodeArgs& a, int s, int slot, int pos, int lid, float nrm, float vval,
                                           const float (&cwv)[kSub], EncodeShared<THREADS>& sh) {
  const int tid = threadIdx.x;
  const E* coarse = static_cast<const E*>(a.coarse) + (size_t)s * a.num_lists * kD;
  if (tid == 0) sh.code_sh = 0u;
  if (tid < kD) sh.resid[tid] = sh.unit[tid] - to_f(coarse[(size_t)lid * kD + tid]);
  __syncthreads();
  if (tid < kM * kC) {
    const int m = tid / kC, c = tid % kC;
    float dist = 0.f;
#pragma unroll
    for (int d = 0; d < kSub; ++d) {
      const float df = sh.resid[m * kSub + d] - cwv[d];
      dist = fmaf(df, df, dist);
    }
    int bc = c;
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) {
      const float od = __shfl_xor_sync(0xffffffffu, dist, o);
      const int oc = __shfl_xor_sync(0xffffffffu, bc, o);
      if (od < dist || (od == dist && oc < bc)) {
        dist = od;
        bc = oc;
      }
    }
    if (c == 0) atomicOr(&sh.code_sh, (uint32_t)bc << (4 * m));
  }
  __syncthreads();
  if (tid == 0) {
    a.codes[(size_t)s * a.cap + slot] = sh.code_sh;
    static_cast<E*>(a.norms)[(size_t)s * a.cap + slot] = from_f<E>(nrm);
    a.list_ids[(size_t)s * a.cap + slot] = (uint16_t)lid;
    a.slot_pos[(size_t)s * a.cap + slot] = pos;
    const float stored = to_f(from_f<E>(nrm));
    if (stored > a.norm_max[s]) a.norm_max[s] = stored;
  }
  // running value mean of the list
  if (tid < kD) {
    const size_t vi = ((size_t)s * a.num_lists + lid) * kD + tid;
    const float nsum = a.vsum[vi] + vval;
    const int ncnt = a.vcnt[(size_t)s * a.num_lists + lid] + 1;
    a.vsum[vi] = nsum;
    static_cast<E*>(a.vmeans)[vi] = from_f<E>(nsum / (float)ncnt);
  }
  __syncthreads();
  if (tid == 0) a.vcnt[(size_t)s * a.num_lists + lid] += 1;
  __syncthreads();
}

// Encodes the next `count` tokens after the indexed region of stream s (all threads of the CTA
// take part; THREADS is the CTA size, a multiple of 128 and at least 128).  seq_len is the
// stream's length including any token appended in the same launch.  Returns the new tail count
// (the caller stores it).
template <typename E, int THREADS>
__device__ __forceinline__ int encode_tokens(const EncodeArgs& a, const int s, const int seq_len) {
  __shared__ EncodeShared<THREADS> sh;
  const int tid = threadIdx.x;
  const int32_t* st = a.state + (size_t)s * kST;
  const int count = a.enc_count ? a.enc_count[s] : a.uniform_count;
  const int n_sorted = st[PQHSA_ST_N_SORTED];
  int n_tail = st[PQHSA_ST_N_TAIL];
  const int nl = st[PQHSA_ST_N_LISTS];
  const int req = st[PQHSA_ST_REQ], head = st[PQHSA_ST_KV_HEAD];
  const int sink_end = min(a.sink, seq_len);
  const E* coarse = static_cast<const E*>(a.coarse) + (size_t)s * a.num_lists * kD;
  const E* books = static_cast<const E*>(a.codebooks) + (size_t)s * kM * kC * kSub;
  const E* kb = static_cast<const E*>(a.k_base);
  const E* vb = static_cast<const E*>(a.v_base);
  float cwv[kSub];
  if (tid < kM * kC) {
    float x[8], y[8];
    load8(books + (size_t)tid * kSub, x);
    load8(books + (size_t)tid * kSub + 8, y);
#pragma unroll
    for (int d = 0; d < 8; ++d) { cwv[d] = x[d]; cwv[8 + d] = y[d]; }
  }
  if (count > 0) {
    // the centroid rows are wanted two dependent loads from now (key row, then its direction): ask L2 for them already
    const char* cb = reinterpret_cast<const char*>(coarse);
    const size_t bytes = (size_t)nl * kD * sizeof(E);
    for (size_t o = (size_t)tid * 128; o < bytes; o += (size_t)THREADS * 128)
      asm volatile("prefetch.global.L2 [%0];" ::"l"(cb + o));
  }
  for (int it = 0; it < count; ++it) {
    const int pos = sink_end + n_sorted + n_tail;
    const int slot = n_sorted + n_tail;
    // never index a token that is not in the cache, never overrun the pool
    if (pos >= seq_len || slot >= a.cap || n_tail >= a.tail_cap) break;
    const long long off = a.kv.offset(req, head, pos);
    float vval = 0.f;
    if (tid < kD) vval = to_f(vb[off + tid]);
    const float nrm = enc_direction<E, THREADS>(kb, off, sh);
    float bd;
    int lid;
    enc_nearest_list<E, THREADS>(coarse, 0, nl, nl, sh, bd, lid);
    if (tid == 0) sh.list_sh = lid;
    __syncthreads();
    lid = sh.list_sh;
    enc_finish<E, THREADS>(a, s, slot, pos, lid, nrm, vval, cwv, sh);
    ++n_tail;
  }
  return n_tail;
}

}  // namespace pqhsa
