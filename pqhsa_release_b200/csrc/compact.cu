// Folding the unsorted tail of a stream back into its list-sorted region, on the device and in place.
//
// The sorted region keeps the keys of a list together, in token order inside the list (the reference's CSR order,
// pq_hsa/index/ivfpq.py:864-882); keys encoded since then sit in the tail in arrival order.  The reference rebuilds
// its snapshot with a stable argsort over all list ids after a flush (benchmarks/e2e_pq_param_sweep.py:4163-4363,
// :3246-3256).  No sort is needed: a tail key of list l goes to the end of l's segment, and l's segment moves up by
// the number of tail keys in the lists below l.
//
// One CTA of 1024 threads per stream, nothing but its own shared memory as scratch:
//   1. the tail records are stashed in shared memory (the moving segments will run over them) and counted per list;
//      the old segment sizes come from the scan units;
//   2. prefix sums over the lists: old starts, shifts, new starts, units per list;
//   3. a tail key's place inside its list = the number of earlier tail keys of the same list (they arrived in
//      token order);
//   4. the segments move up, the last list first, a chunk of 1024 slots at a time through registers (read,
//      barrier, write, barrier): a segment only ever runs over slots whose keys have moved already;
//   5. the tail keys drop into the gaps; scan units, the slots' unit ids, the sample records and the counters are
//      rebuilt.
// The result is the layout a stable sort by (list, token position) gives, bit for bit.
#include "common.cuh"

namespace pqhsa {

constexpr int kCompThreads = 1024;
constexpr int kCompTail = PQHSA_COMPACT_MAX_TAIL;  // tail slots one call can fold in

struct CompactArgs {
  uint32_t* codes;
  void* norms;
  uint16_t* list_ids;
  int32_t* slot_pos;
  uint16_t* slot_unit;
  int32_t* unit_off;
  uint16_t* unit_list;
  int4* sample;  // or null
  int32_t* state;
  int32_t* error;  // [1]: set to 1 if a stream could not be compacted (tail too long, too many units)
  int cap, ucap;
};

struct CompactShared {
  int tail_cnt[kLMax];   // tail keys per list; later: start of the list's new segment
  int old_cnt[kLMax];    // keys of the list in the sorted region
  int old_start[kLMax];
  int shift[kLMax];      // tail keys in the lists below
  int ubase[kLMax];      // first unit of the list in the new layout
  int wtot[kCompThreads / 32];
  int total_units;
};

template <typename E>
__global__ void __launch_bounds__(kCompThreads) compact_kernel(const CompactArgs a) {
  extern __shared__ __align__(16) unsigned char comp_smem[];
  int4* stash = reinterpret_cast<int4*>(comp_smem);  // [kCompTail] (code, token position, norm bits, list)
  __shared__ CompactShared sh;
  const int s = blockIdx.x, tid = threadIdx.x;
  int32_t* st = a.state + (size_t)s * kST;
  const int n_sorted = st[PQHSA_ST_N_SORTED], n_tail = st[PQHSA_ST_N_TAIL], n_units = st[PQHSA_ST_N_UNITS];
  if (n_tail == 0) return;
  const int n = n_sorted + n_tail;
  if (n_tail > kCompTail || n > a.cap) {
    if (tid == 0) *a.error = 1;
    return;
  }
  uint32_t* codes = a.codes + (size_t)s * a.cap;
  E* norms = static_cast<E*>(a.norms) + (size_t)s * a.cap;
  uint16_t* lids = a.list_ids + (size_t)s * a.cap;
  int32_t* spos = a.slot_pos + (size_t)s * a.cap;
  uint16_t* sunit = a.slot_unit + (size_t)s * a.cap;
  int32_t* uoff = a.unit_off + (size_t)s * (a.ucap + 1);
  uint16_t* ulist = a.unit_list + (size_t)s * a.ucap;

  // ---- 1. stash the tail, count it per list, and the old segments from the units ----
  for (int l = tid; l < kLMax; l += kCompThreads) {
    sh.tail_cnt[l] = 0;
    sh.old_cnt[l] = 0;
  }
  __syncthreads();
  for (int j = tid; j < n_tail; j += kCompThreads) {
    const int slot = n_sorted + j;
    const int l = lids[slot];
    uint32_t nb = 0u;
    if constexpr (sizeof(E) == 4) {
      nb = reinterpret_cast<const uint32_t*>(norms)[slot];
    } else {
      nb = reinterpret_cast<const uint16_t*>(norms)[slot];
    }
    stash[j] = make_int4((int)codes[slot], spos[slot], (int)nb, l);
    atomicAdd(&sh.tail_cnt[l], 1);
  }
  for (int u = tid; u < n_units; u += kCompThreads) atomicAdd(&sh.old_cnt[ulist[u]], uoff[u + 1] - uoff[u]);
  __syncthreads();
  // ---- 2. prefix sums over the lists ----
  const int my_tail = tid < kLMax ? sh.tail_cnt[tid] : 0, my_old = tid < kLMax ? sh.old_cnt[tid] : 0;
  int total;
  const int old_start = block_exscan(my_old, sh.wtot, &total);
  const int shift = block_exscan(my_tail, sh.wtot, &total);
  const int my_units = (my_old + my_tail + kUnit - 1) / kUnit;
  int total_units;
  const int ubase = block_exscan(my_units, sh.wtot, &total_units);
  if (total_units > a.ucap) {  // block-uniform; cannot happen with unit_capacity >= lists + cap / 128
    if (tid == 0) *a.error = 1;
    return;
  }
  if (tid < kLMax) {
    sh.old_start[tid] = old_start;
    sh.shift[tid] = shift;
    sh.ubase[tid] = ubase;
  }
  __syncthreads();
  // ---- 3. where the tail keys go: end of the list's old segment + earlier tail keys of the same list ----
  constexpr int kPer = kCompTail / kCompThreads;
  int dst[kPer];
#pragma unroll
  for (int k = 0; k < kPer; ++k) {
    const int j = tid + k * kCompThreads;
    dst[k] = -1;
    if (j < n_tail) {
      const int l = stash[j].w;
      int rank = 0;
      for (int i = 0; i < j; ++i) rank += stash[i].w == l ? 1 : 0;
      dst[k] = sh.old_start[l] + sh.shift[l] + sh.old_cnt[l] + rank;
    }
  }
  // ---- 4. the segments move up, last list first, 1024 slots at a time through registers ----
  for (int l = kLMax - 1; l >= 0; --l) {
    const int sft = sh.shift[l], cnt = sh.old_cnt[l];
    if (sft == 0) break;  // the lists below have no tail keys under them either
    if (cnt == 0) continue;
    const int a0 = sh.old_start[l];
    for (int hi = a0 + cnt; hi > a0; hi -= kCompThreads) {
      const int i = hi - kCompThreads + tid;  // this thread's slot of the chunk [hi - 1024, hi)
      const bool mine = i >= a0;
      uint32_t c = 0u;
      E nr = E();
      uint16_t li = 0;
      int32_t po = 0;
      if (mine) {
        c = codes[i];
        nr = norms[i];
        li = lids[i];
        po = spos[i];
      }
      __syncthreads();  // the chunk is in registers before anybody writes over it
      if (mine) {
        codes[i + sft] = c;
        norms[i + sft] = nr;
        lids[i + sft] = li;
        spos[i + sft] = po;
      }
      __syncthreads();
    }
  }
  // ---- 5. the tail keys drop into the gaps ----
#pragma unroll
  for (int k = 0; k < kPer; ++k) {
    if (dst[k] < 0) continue;
    const int4 r = stash[tid + k * kCompThreads];
    codes[dst[k]] = (uint32_t)r.x;
    spos[dst[k]] = r.y;
    if constexpr (sizeof(E) == 4) {
      reinterpret_cast<uint32_t*>(norms)[dst[k]] = (uint32_t)r.z;
    } else {
      reinterpret_cast<uint16_t*>(norms)[dst[k]] = (uint16_t)r.z;
    }
    lids[dst[k]] = (uint16_t)r.w;
  }
  // scan units of the new layout: list l owns units ubase[l] .., 128 slots each from its new start
  if (tid < kLMax) {
    const int start = old_start + shift;
    for (int k = 0; k < my_units; ++k) {
      uoff[ubase + k] = start + k * kUnit;
      ulist[ubase + k] = (uint16_t)tid;
    }
    sh.tail_cnt[tid] = start;  // from here on: the new start of the list
  }
  if (tid == 0) uoff[total_units] = n;
  __syncthreads();  // the moved keys and the new starts are visible to the CTA
  for (int i = tid; i < n; i += kCompThreads) {
    const int l = lids[i];
    sunit[i] = (uint16_t)(sh.ubase[l] + (i - sh.tail_cnt[l]) / kUnit);
  }
  // sample records of the new sorted region (streams with at most kSample sorted slots are never sampled)
  if (a.sample != nullptr && n > kSample) {
    int4* rec = a.sample + (size_t)s * kSample;
    for (int i = tid; i < kSample; i += kCompThreads) {
      const int j = (int)((long long)i * n / kSample);
      rec[i] = make_int4((int)codes[j], __float_as_int(to_f(norms[j])), (int)lids[j], j);
    }
  }
  if (tid == 0) {
    st[PQHSA_ST_N_SORTED] = n;
    st[PQHSA_ST_N_TAIL] = 0;
    st[PQHSA_ST_N_UNITS] = total_units;
  }
}

int launch_compact(const pqhsa_params& p, int32_t* error, cudaStream_t st) {
  CompactArgs a;
  a.codes = static_cast<uint32_t*>(const_cast<void*>(p.codes));
  a.norms = const_cast<void*>(p.norms);
  a.list_ids = static_cast<uint16_t*>(const_cast<void*>(p.list_ids));
  a.slot_pos = static_cast<int32_t*>(const_cast<void*>(p.slot_pos));
  a.slot_unit = static_cast<uint16_t*>(const_cast<void*>(p.slot_unit));
  a.unit_off = static_cast<int32_t*>(const_cast<void*>(p.unit_off));
  a.unit_list = static_cast<uint16_t*>(const_cast<void*>(p.unit_list));
  a.sample = static_cast<int4*>(const_cast<void*>(p.sample));
  a.state = static_cast<int32_t*>(p.state);
  a.error = error;
  a.cap = p.slot_capacity;
  a.ucap = p.unit_capacity;
  constexpr size_t smem = (size_t)kCompTail * sizeof(int4);
  PQHSA_DISPATCH_E(p.dtype, {
    auto kern = compact_kernel<E>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return check_launch("compact: shared memory opt-in");
    kern<<<p.num_streams, kCompThreads, smem, st>>>(a);
  });
  return check_launch("compact");
}

}  // namespace pqhsa
