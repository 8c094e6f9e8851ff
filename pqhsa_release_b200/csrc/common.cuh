// Shared device/host helpers of the PQ-HSA sm_100a decode kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "pqhsa.h"

namespace pqhsa {

constexpr int kD = PQHSA_HEAD_DIM;      // head dimension
constexpr int kM = PQHSA_SUBSPACES;     // PQ subspaces
constexpr int kC = PQHSA_CODES;         // code words per subspace
constexpr int kSub = kD / kM;           // dims per subspace
constexpr int kLMax = PQHSA_MAX_LISTS;  // IVF lists
constexpr int kUnit = PQHSA_UNIT_KEYS;  // slots per scan unit
constexpr int kBins = PQHSA_HIST_BINS;  // sample histogram bins
constexpr int kSample = PQHSA_SAMPLE_KEYS;
constexpr int kRI = PQHSA_RI_INTS;      // ints of row_info per row
constexpr int kST = PQHSA_STATE_INTS;   // ints of state per stream
constexpr int kChunk = 128;             // attend entries per split-K chunk
constexpr int kPartial = kD + 2;        // floats per split-K partial (max, sum, acc[D])
constexpr int kBgParts = 5;             // background partial slots per query row (4 unit parts + the tail)
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kNegInf = -__builtin_huge_valf();

// host-side error plumbing (abi.cu)
int set_error(int code, const char* fmt, ...);
int check_params(const pqhsa_params* p, bool need_ws, bool need_kv, bool need_io);
int check_launch(const char* what);
void layout_of(const pqhsa_params* p, pqhsa_ws_layout* o);
int sm_count();

// kernel launchers, one translation unit each; all return a pqhsa_status
// What the first kernel of a step does besides the tables when the token append is fused into it.
struct StepAppend {
  const void* new_k;         // E [S, 128] or null: no row is written and the length stays
  const void* new_v;
  const int32_t* enc_count;  // device int32 [S] or null
  int32_t uniform_count;     // keys to encode per stream when enc_count is null
};
int launch_lut_build(const pqhsa_params& p, const pqhsa_ws_layout& w, const StepAppend* ap, cudaStream_t st);
int launch_scan(const pqhsa_params& p, const pqhsa_ws_layout& w, float* dump, cudaStream_t st);
int launch_select(const pqhsa_params& p, const pqhsa_ws_layout& w, cudaStream_t st);
int launch_attend(const pqhsa_params& p, const pqhsa_ws_layout& w, cudaStream_t st);
int launch_merge(const pqhsa_params& p, const pqhsa_ws_layout& w, cudaStream_t st);
int launch_wait_peers(const pqhsa_params& p, cudaStream_t st);
int launch_append_kv(const pqhsa_params& p, const void* k, const void* v, cudaStream_t st);
int launch_append_encode(const pqhsa_params& p, const int32_t* cnt, int32_t uni, cudaStream_t st);
int launch_compact(const pqhsa_params& p, int32_t* error, cudaStream_t st);
int launch_encode_bulk(const void* keys, long long stream_stride, int streams, int n, int dtype, const void* coarse,
                       int num_lists, const void* codebooks, uint32_t* codes, void* norms, uint16_t* list_ids,
                       bool lists_given, cudaStream_t st);
int launch_topk(const float* scores, int rows, int n, int64_t stride, int k, int32_t* oi, float* ov,
                cudaStream_t st);
int launch_cluster_order(const uint16_t* ids, int sets, int n, int k, int32_t* order, int32_t* start, cudaStream_t st);
int launch_cluster_sums(const void* rows, int dtype, long long stream_stride, int row_stride, int width, int streams,
                        int groups, int n, int k, const int32_t* order, const int32_t* start, float* sums,
                        cudaStream_t st);
int launch_subspace_assign(const float* rows, long long stream_stride, const float* books, int streams, int n,
                           uint16_t* ids, cudaStream_t st);

#define PQHSA_DISPATCH_E(dtype, ...)                                   \
  switch (dtype) {                                                     \
    case PQHSA_F32: { using E = float; __VA_ARGS__; break; }           \
    case PQHSA_BF16: { using E = __nv_bfloat16; __VA_ARGS__; break; }  \
    case PQHSA_F16: { using E = __half; __VA_ARGS__; break; }          \
    default: return set_error(PQHSA_E_DTYPE, "unknown dtype %d", (int)(dtype)); \
  }

#define PQHSA_DISPATCH_G(group, ...)                                   \
  switch (group) {                                                     \
    case 1: { constexpr int G = 1; __VA_ARGS__; break; }               \
    case 2: { constexpr int G = 2; __VA_ARGS__; break; }               \
    case 4: { constexpr int G = 4; __VA_ARGS__; break; }               \
    case 8: { constexpr int G = 8; __VA_ARGS__; break; }               \
    default: return set_error(PQHSA_E_SHAPE, "unsupported group size %d", (int)(group)); \
  }

#ifdef __CUDACC__

// ---- element access ---------------------------------------------------
__device__ __forceinline__ float to_f(float v) { return v; }
__device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float to_f(__half v) { return __half2float(v); }

template <typename E> __device__ __forceinline__ E from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }

__device__ __forceinline__ void unpack8(const uint4& r, const __nv_bfloat16*, float (&v)[8]) {
  const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
__device__ __forceinline__ void unpack8(const uint4& r, const __half*, float (&v)[8]) {
  const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}

__device__ __forceinline__ void unpack4(const uint2& r, const __nv_bfloat16*, float (&v)[4]) {
  v[0] = __uint_as_float(r.x << 16); v[1] = __uint_as_float(r.x & 0xffff0000u);
  v[2] = __uint_as_float(r.y << 16); v[3] = __uint_as_float(r.y & 0xffff0000u);
}
__device__ __forceinline__ void unpack4(const uint2& r, const __half*, float (&v)[4]) {
  const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&r.x));
  const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&r.y));
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
__device__ __forceinline__ void unpack4(const uint2&, const float*, float (&)[4]) {}  // never called: floats come as float4

// 8 consecutive elements, 16-byte aligned
__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
  const float4 a = __ldg(reinterpret_cast<const float4*>(p));
  const float4 b = __ldg(reinterpret_cast<const float4*>(p) + 1);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&v)[8]) {
  unpack8(__ldg(reinterpret_cast<const uint4*>(p)), p, v);
}
__device__ __forceinline__ void load8(const __half* p, float (&v)[8]) {
  unpack8(__ldg(reinterpret_cast<const uint4*>(p)), p, v);
}
// 4 consecutive elements, 8-byte (2-byte types) or 16-byte (float) aligned
__device__ __forceinline__ void load4(const float* p, float (&v)[4]) {
  const float4 a = __ldg(reinterpret_cast<const float4*>(p));
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
}
__device__ __forceinline__ void load4(const __nv_bfloat16* p, float (&v)[4]) {
  const uint2 r = __ldg(reinterpret_cast<const uint2*>(p));
  v[0] = __uint_as_float(r.x << 16); v[1] = __uint_as_float(r.x & 0xffff0000u);
  v[2] = __uint_as_float(r.y << 16); v[3] = __uint_as_float(r.y & 0xffff0000u);
}
__device__ __forceinline__ void load4(const __half* p, float (&v)[4]) {
  const uint2 r = __ldg(reinterpret_cast<const uint2*>(p));
  const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&r.x));
  const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&r.y));
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ---- the approximate logit --------------------------------------------
// logit = (pq + list_score) * |k| with
//   pq = ((t0 + t1) + (t2 + t3)) + ... : (t_{2p} + t_{2p+1}) first, then the four
//        pair sums left to right,  t_m = lut[m][nibble_m]
// which is the subspace sum of pq_hsa/kernels/lut_scan.py:101-114 in the
// association order of the byte-pair tables
// (pq_hsa/kernels/triton_lut_scan_h20.py:127-171), then the list bias, then the
// norm (pq_hsa/index/ivfpq.py:1093-1118).  The scale and |q| are folded into
// lut and list_score.  Explicit rounding intrinsics (no contraction, no
// re-association) make every kernel that re-scores a slot reproduce the scan's
// value bit for bit.
__device__ __forceinline__ float finish_logit(float pq, float list_score, float knorm) {
  return __fmul_rn(__fadd_rn(pq, list_score), knorm);
}
__device__ __forceinline__ float pair_entry(const float* lut, int pair, uint32_t byte) {
  return __fadd_rn(lut[(2 * pair) * kC + (byte & 15u)], lut[(2 * pair + 1) * kC + (byte >> 4)]);
}
// lut: 128 floats [m][c] of one query row
__device__ __forceinline__ float pq_sum_row(const float* lut, uint32_t code) {
  float acc = pair_entry(lut, 0, code & 255u);
#pragma unroll
  for (int p = 1; p < kM / 2; ++p) acc = __fadd_rn(acc, pair_entry(lut, p, (code >> (8 * p)) & 255u));
  return acc;
}

// asynchronous 16-byte copies from global to shared memory (L2 only), in groups a thread can wait for
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Contribution of one key to the exp-sum of its scan unit, relative to the unit's maximum
// logit: 2^(logit * log2(e) + ref), ref = unit_ref(unit maximum), one fused multiply-add
// (the scan runs it on two rows at a time with the packed form, which rounds identically).
// The scan adds it and the selection subtracts it for a selected key: same inputs, same
// operations, so the removal is exact.
__device__ __forceinline__ float unit_ref(float unit_max) { return -__fmul_rn(unit_max, kLog2e); }
__device__ __forceinline__ float unit_term(float logit, float ref) { return ex2(__fmaf_rn(logit, kLog2e, ref)); }

// histogram bin of a logit: monotone non-decreasing in the logit
__device__ __forceinline__ int logit_bin(float logit, float lo, float inv_w) {
  const float t = __fmul_rn(__fsub_rn(logit, lo), inv_w);
  int b = __float2int_rd(t);
  b = b < 0 ? 0 : b;
  return b > kBins - 1 ? kBins - 1 : b;
}

// order-preserving 32-bit key of a float (larger float <=> larger key)
__device__ __forceinline__ uint32_t float_key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ float key_float(uint32_t k) {  // inverse of float_key
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

// K = min(max(ceil(N * fraction), 0), N) in double precision
// (pq_hsa/attention/sparse_attention.py:1779-1783); fraction < 0 selects the fixed count.
__device__ __forceinline__ int resolve_topk(int n, double fraction, int fixed) {
  if (n <= 0) return 0;
  long long k = fixed;
  if (fraction >= 0.0) k = (long long)ceil((double)n * fraction);
  if (k < 0) k = 0;
  if (k > n) k = n;
  return (int)k;
}

// address (in elements) of token `t` of request `req`, KV head `head`
struct KvAddr {
  const int32_t* block_table;
  int32_t max_blocks, block_size;
  int64_t stride_block, stride_head, stride_row;
  __device__ __forceinline__ int64_t offset(int req, int head, int t) const {
    int64_t blk = req, row = t;
    if (block_table != nullptr) {
      blk = __ldg(block_table + (int64_t)req * max_blocks + t / block_size);
      row = t % block_size;
    }
    return blk * stride_block + (int64_t)head * stride_head + row * stride_row;
  }
};
__host__ __device__ inline KvAddr make_kvaddr(const pqhsa_params& p) {
  KvAddr a;
  a.block_table = p.block_table;
  a.max_blocks = p.max_blocks;
  a.block_size = p.block_size;
  a.stride_block = p.stride_block;
  a.stride_head = p.stride_head;
  a.stride_row = p.stride_row;
  return a;
}

// geometry of the exact part of a stream, from its device counters
struct StreamGeom {
  int n_sorted, n_tail, n_units, seq_len, sink_end, retr_end, full;  // full = sink + local rows
};
__device__ __forceinline__ StreamGeom stream_geom(const int32_t* st, int sink) {
  StreamGeom g;
  g.n_sorted = st[PQHSA_ST_N_SORTED];
  g.n_tail = st[PQHSA_ST_N_TAIL];
  g.n_units = st[PQHSA_ST_N_UNITS];
  g.seq_len = st[PQHSA_ST_SEQ_LEN];
  g.sink_end = min(sink, g.seq_len);
  g.retr_end = g.sink_end + g.n_sorted + g.n_tail;
  g.full = g.sink_end + max(g.seq_len - g.retr_end, 0);
  return g;
}

// Exclusive prefix sum over the 1024 threads of a CTA (thread t holds value t; threads with nothing pass 0); all
// threads call.  Returns the exclusive sum; *total = the sum of all.  wtot: 32 ints of shared memory.
__device__ __forceinline__ int block_exscan(int v, int* wtot, int* total) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int x = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += x;
  }
  __syncthreads();  // wtot of an earlier call has been read
  if (lane == 31) wtot[warp] = incl;
  __syncthreads();
  int w = wtot[lane];  // 32 warps
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int x = __shfl_up_sync(0xffffffffu, w, o);
    if (lane >= o) w += x;
  }
  *total = __shfl_sync(0xffffffffu, w, 31);
  const int before = __shfl_sync(0xffffffffu, w, warp) - __shfl_sync(0xffffffffu, incl, 31);
  return before + incl - v;
}

#endif  // __CUDACC__

}  // namespace pqhsa
