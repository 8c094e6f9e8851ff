/*
 * pqhsa.h -- C ABI of the B200 (sm_100a) PQ-HSA per-step decode operator.
 *
 * Plain pointers and sizes only: no torch types, no exceptions, no allocation
 * and no host synchronisation inside any entry point.  Every function returns
 * 0 on success or a negative PQHSA_E_* code; pqhsa_last_error_string() gives
 * the text of the calling thread's last failure.  All work is enqueued on the
 * cudaStream_t handed in (passed as void* so that this header needs no CUDA
 * include), so a sequence of calls can be captured in a CUDA graph.
 *
 * The entry points replace the reference's torch-pybind FFI
 * (pq_hsa/kernels/cuda/pq_fused_h20.cu:3826-3839) and its Triton launchers for
 * the decode hot path.  Each declaration cites what it stands in for.
 */
#ifndef PQHSA_H_
#define PQHSA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PQHSA_ABI_VERSION 4

/* fixed shape of the index (pq_hsa/kernels/cuda/pq_fused_h20.cu:26-35 fixes the
 * same: 8 subspaces x 4 bits, at most 512 lists, head_dim 128) */
#define PQHSA_SUBSPACES 8
#define PQHSA_CODES 16
#define PQHSA_HEAD_DIM 128
#define PQHSA_MAX_LISTS 512
#define PQHSA_UNIT_KEYS 128     /* a scan unit = at most this many slots of one list */
#define PQHSA_COMPACT_MAX_TAIL 4096 /* tail slots per stream one pqhsa_compact call can fold in */
#define PQHSA_SAMPLE_KEYS 4096  /* keys scored per stream to place the candidate threshold */
#define PQHSA_HIST_BINS 2048    /* resolution of the sample histogram */
#define PQHSA_SELECT_BINS 1024  /* candidate bins between the threshold and its upper companion; one more above */

enum pqhsa_status {
  PQHSA_OK = 0,
  PQHSA_E_NULL = -1,        /* a required pointer is null */
  PQHSA_E_SHAPE = -2,       /* unsupported or inconsistent size */
  PQHSA_E_DTYPE = -3,       /* unknown element type */
  PQHSA_E_WORKSPACE = -4,   /* workspace missing, misaligned or too small */
  PQHSA_E_CUDA = -5,        /* a CUDA runtime call failed */
  PQHSA_E_CAPACITY = -6     /* index slots / tail / static scratch exhausted */
};

enum pqhsa_dtype { PQHSA_F32 = 0, PQHSA_BF16 = 1, PQHSA_F16 = 2 };

/* Per-stream counters kept ON THE DEVICE (int32[PQHSA_STATE_INTS] per stream),
 * so that append/encode and the decode step need no host round trip. */
enum pqhsa_state_slot {
  PQHSA_ST_N_SORTED = 0, /* slots in the list-sorted region                     */
  PQHSA_ST_N_TAIL = 1,   /* slots appended after it, in arrival order           */
  PQHSA_ST_SEQ_LEN = 2,  /* tokens of this request present in the KV cache      */
  PQHSA_ST_N_UNITS = 3,  /* scan units covering the sorted region               */
  PQHSA_ST_N_LISTS = 4,  /* IVF lists in use (min(num_lists, keys at build))    */
  PQHSA_ST_REQ = 5,      /* request index: row of block_table / batch index     */
  PQHSA_ST_KV_HEAD = 6,  /* KV head index inside the cache                      */
  PQHSA_ST_RESERVED = 7,
  PQHSA_STATE_INTS = 8
};

/*
 * One POD describes a batch of independent streams (stream = one request x one
 * KV head; its G query heads share the index).  E is the element type `dtype`
 * of q, K/V rows, output and of the float tensors of the index, as in the
 * reference where centroids, code words and norms take the key dtype
 * (pq_hsa/index/ivfpq.py:1052-1059, pq_hsa/index/kmeans.py:225).
 *
 * Index pool, S = num_streams, cap = slot_capacity (IVF-PQ layout of
 * pq_hsa/index/ivfpq.py:160-173 in the list-sorted snapshot form of
 * benchmarks/e2e_pq_param_sweep.py:4182-4305):
 *   codes     uint32 [S, cap]      8 nibbles, subspace s in bits 4s..4s+3
 *   norms     E      [S, cap]      |k|, clamped at 1e-12
 *   norm_max  float  [S]           upper bound of the stream's norms (sizes the sample histogram)
 *   list_ids  uint16 [S, cap]
 *   slot_pos  int32  [S, cap]      token position of the slot's key
 *   slot_unit uint16 [S, cap]      scan unit holding the slot (sorted region only)
 *   unit_off  int32  [S, unit_capacity + 1]   slot ranges of the scan units
 *   unit_list uint16 [S, unit_capacity]       list of each unit
 *   coarse    E      [S, num_lists, 128]      list centroids (unit-direction space)
 *   codebooks E      [S, 8, 16, 16]           residual code words
 *   vmeans    E      [S, num_lists, 128]      per-list mean value row
 *   vsum      float  [S, num_lists, 128]      running value sums   (append only)
 *   vcnt      int32  [S, num_lists]           running list counts  (append only)
 *   state     int32  [S, PQHSA_STATE_INTS]
 *
 * KV cache addressing for token t of request r, KV head h
 * (pq_hsa/kernels/cuda/pq_fused_h20.cu:879-903 supports the same two page
 * layouts; a contiguous [B, Hkv, S, D] cache is the block_table == NULL case):
 *   blk = block_table ? block_table[r * max_blocks + t / block_size] : r
 *   row = block_table ? t % block_size : t
 *   K   = k_base + blk * stride_block + h * stride_head + row * stride_row   (elements)
 *   V   = v_base + the same offset
 */
typedef struct pqhsa_params {
  int32_t abi_version;     /* PQHSA_ABI_VERSION */
  int32_t dtype;           /* enum pqhsa_dtype */
  int32_t num_streams;     /* S = requests x local KV heads */
  int32_t group;           /* G = query heads per KV head: 1, 2, 4 or 8 */
  int32_t head_dim;        /* 128 */
  int32_t num_lists;       /* row count of coarse / vmeans, <= 512 */
  int32_t slot_capacity;   /* cap, multiple of 8 */
  int32_t unit_capacity;   /* >= lists + cap / PQHSA_UNIT_KEYS */
  int32_t sink_tokens;
  int32_t local_window;
  int32_t max_slots;       /* host upper bound of n_sorted + n_tail over streams (grid sizing) */
  int32_t max_full;        /* capacity: sink + local rows of any stream never exceed it (fixes the layout) */
  int32_t topk_fixed;      /* used when top_fraction < 0 */
  int32_t tail_capacity;   /* most slots the unsorted tail may hold (fixes the workspace layout) */
  double top_fraction;     /* K = min(max(ceil(N * f), 0), N) in double, as
                              pq_hsa/attention/sparse_attention.py:1779-1783 */
  float scale;             /* softmax scale, 1/sqrt(D) unless the model says otherwise */
  float hist_lo;           /* sample histogram: bin = (logit - lo) * inv_width, clamped;          */
  float hist_inv_width;    /* inv_width <= 0 (default) sizes the bins per query row from a bound   */
                           /* on |logit|.  The selection is exact for any choice.                  */
  float select_margin;     /* standard deviations of head-room of the candidate threshold;         */
                           /* 0 = default (6).  Lower values only make the exact fallback likelier */

  const void *codes, *norms, *list_ids, *slot_pos, *slot_unit, *unit_off, *unit_list;
  const void *coarse, *codebooks, *vmeans;
  void *vsum, *vcnt, *state, *norm_max;
  const void *sample;      /* optional int32 [S, PQHSA_SAMPLE_KEYS, 4]: for sample i of a stream, the slot
                              j = floor(i * n_sorted / 4096) of its list-sorted region as (code, norm as float
                              bits, list id, j) - a contiguous copy of what the threshold estimate reads, to
                              be refreshed whenever the sorted region changes; NULL = gather from the index.
                              Only read for streams with more than PQHSA_SAMPLE_KEYS sorted slots. */

  const void *k_base, *v_base;
  const int32_t *block_table;
  int32_t max_blocks;
  int32_t block_size;
  int64_t stride_block, stride_head, stride_row;

  /* Output exchange between the GPUs of a node (all zero / NULL on one GPU).  With peer_world > 1 the
   * combine kernel also sends every output row to every rank as flagged words: 8-byte stores of (4 bytes of the
   * row, the step count), each of which arrives whole, so the receiver needs no fence and no separate flag.
   * Row r of this rank goes to words ((parity * peer_world + peer_rank) * R + r) * W .. + W of a rank's receive
   * buffer, W = 128 * sizeof(E) / 4 (parity = step count & 1: two buffers, so a rank that is one step ahead never
   * overwrites what a peer still reads).  pqhsa_wait_peers enqueues the receiving kernel: it waits for every
   * word of the step (bounded) and unpacks the rows into peer_gather.  All ranks must run the same sequence
   * of steps. */
  const void *peer_out;    /* device array of peer_world pointers: every rank's receive buffer,
                              uint32 [2, peer_world, R, W, 2], mapped into this process (peer memory) */
  void *peer_gather;       /* this rank's gathered rows: E [2, peer_world, R, 128] (parity, source rank, its rows) */
  void *peer_seq;          /* device int32 [2] of this rank: steps exchanged so far, error flag */
  int32_t peer_world;
  int32_t peer_rank;
  int32_t peer_wait_polls; /* polls (about 100 ns apart) a thread of pqhsa_wait_peers makes for its word before it gives
                              up; 0 = about half a second */
  int32_t external_append; /* 1: pqhsa_decode_step_append with new_k == NULL advances every live stream's length by
                              one without writing a row - the caller's own cache write (vLLM's
                              reshape_and_cache_flash) has already stored this step's K/V.  0: the length stays. */

  const void *q;           /* E [S, G, 128]: query heads h*G .. h*G+G-1 of KV head h */
  void *out;               /* E [S, G, 128] */
  const int32_t *io_map;   /* optional device int32 [S]: stream s reads its G query rows from block io_map[s] of q
                              and writes block io_map[s] of out (a block = G x 128 elements), so that streams can
                              keep their pool slot while the batch order of their requests changes from step to
                              step; negative = the stream is idle this step (nothing is read or written for
                              it).  NULL = block s.  The peer exchange sends rows in stream order either way. */
  void *workspace;         /* >= pqhsa_workspace_bytes(), 256-byte aligned */
  size_t workspace_bytes;
} pqhsa_params;

/* Byte offsets of the intermediate results inside the workspace, so that a
 * caller (or a parity test) can read them after the stream has been synchronised.
 * R = S * G query rows. */
typedef struct pqhsa_ws_layout {
  size_t total_bytes;
  size_t lut;          /* float  [S, G, 8, 16]   scale * <q_m, code word>                 */
  size_t list_scores;  /* float  [S, G, 512]     scale * <q, centroid>                    */
  size_t pair_tab;     /* float  [S, G/GP, 4, 256, GP], GP = min(G, 4): byte-pair sums of lut for the scan */
  size_t row_bin;      /* float  [R, 2]   origin (= row_tau) and 1 / width of the candidate bins of the selection
                          ((size_t)-1 in a hand-made layout: no thresholds wanted)       */
  size_t row_tau;      /* float  [R]      candidate threshold on the approximate logit     */
  size_t ticket;       /* int32  [S, 2]   arrival counters of the table kernel's CTAs (0 between launches) */
  size_t norm_pend;    /* float  [S]      norm of a key encoded in the current launch                    */
  size_t unit_max;     /* float  [R, unit_capacity]   per-unit max logit                   */
  size_t unit_sum;     /* float  [R, unit_capacity]   per-unit sum exp(logit - max), selected keys removed */
  size_t tail_logit;   /* float  [R, tail capacity]   logits of the unsorted tail (-inf once selected) */
  size_t row_info;     /* int32  [R, 8]   see enum pqhsa_row_info_slot                     */
  size_t hitmap;       /* uint32 [R, unit_capacity, 4]  bit b of word (u, i): slot first(u) + 32 i + b reached the threshold */
  size_t cand_key;     /* uint32 [R, parts, seg]  candidates of a row, listed by `parts` CTAs: order-preserving key of the logit */
  size_t cand_rec;     /* int32  [R, parts, seg, 4]  ... slot, token position, the term the scan added to the unit's
                                                     exp-sum (float bits), scan unit                 */
  size_t cand_bin;     /* uint16 [R, parts, seg]  ... bin between the threshold and its upper companion */
  size_t part_hist;    /* uint32 [R, parts, PQHSA_SELECT_BINS + 4]  candidates per bin and part        */
  size_t part_cnt;     /* int32  [R, parts]       candidates found by each part (> seg: overflow)      */
  size_t sel_slot;     /* int32  [R, kcap]  the K selected slots (unordered)               */
  size_t sel_off;      /* int64  [R, kcap]  element offset of their K/V rows in the cache  */
  size_t partial;      /* float  [R, chunks + 5, 130]  split-K partials (max, sum, acc): exact chunks, then up to 5 background parts */
  size_t row_ticket;   /* int32  [R]      finished items of the attend kernel per row (0 between launches) */
  size_t work_counter; /* uint64 [2]      work distribution of the attend kernel (0 between launches)      */
  size_t combine_ticket; /* int32 [1]     finished CTAs of the combine kernel (0 between launches)          */
  int32_t parts;       /* form of the selection: 1 = one CTA per query row with 8 candidates per thread (1024 threads;
                          512, two CTAs to an SM, when there are more rows than SMs and 2 kcap + 1024 <= 4096), -1 = one
                          CTA with 16 per thread (larger K), >= 2 = that many CTAs share a row (still larger K) */
  int32_t seg;         /* candidates one of them can list */
  int32_t kcap;        /* row stride of sel_* */
  int32_t tail_cap;    /* row stride of tail_logit */
  int32_t chunks;      /* split-K partials per row */
} pqhsa_ws_layout;

enum pqhsa_row_info_slot {
  PQHSA_RI_K = 0,        /* keys to select                                              */
  PQHSA_RI_N = 1,        /* indexed keys of the stream                                  */
  PQHSA_RI_NCAND = 2,    /* keys whose logit reached the candidate threshold            */
  PQHSA_RI_NSEL = 3,     /* keys selected (== K after the finish kernel)                */
  PQHSA_RI_FALLBACK = 4, /* 1 if the finish kernel had to select from all keys          */
  PQHSA_RI_TIES = 5,     /* size of the group of equal logits the K-th fell into, when only part of it
                            was taken (lowest slots first); 0 otherwise.  One CTA per row form only */
  PQHSA_RI_INTS = 8
};

int pqhsa_abi_version(void);

/* Text of the calling thread's last error ("" if none). */
const char* pqhsa_last_error_string(void);

/* Workspace size for `p` (ignores p->workspace*).  Replaces the function-static
 * scratch tensors of pq_fused_h20.cu:2610-2618; here the caller owns the memory. */
size_t pqhsa_workspace_bytes(const pqhsa_params* p);
int pqhsa_workspace_layout(const pqhsa_params* p, pqhsa_ws_layout* out);

/* (1) Per-query, per-head table construction: lut, its byte-pair form and
 * list_scores in the workspace, plus the per-row candidate threshold estimated
 * from a stratified sample of the stream's keys (p->sample, or gathered from the
 * index when that is NULL).  Replaces pq_lut_prep (pq_fused_h20.cu:2975-3051),
 * _build_pair_tables (pq_hsa/kernels/triton_lut_scan_h20.py:127-171) and
 * ProductQuantizer.compute_lut + the coarse bias (pq_hsa/index/pq.py:190-217,
 * pq_hsa/index/ivfpq.py:1179-1190).  The workspace must be all zero before its
 * first use (the kernels keep their counters in it and leave them at zero). */
int pqhsa_lut_build(const pqhsa_params* p, void* stream);

/* (2)+(3)+(5a) Code scan with per-unit log-sum-exp, one bit per (row, slot) for
 * "logit reached the threshold", and exact top-K selection among those slots.
 * Needs pqhsa_lut_build first.  Leaves sel_slot / sel_off / row_info / unit_*
 * in the workspace.  Replaces the pair-fused Triton scan
 * (pq_hsa/kernels/triton_lut_scan_h20.py:1197-1291), list_exp_sums_sorted
 * (pq_hsa/kernels/triton_lut_scan.py:424-514), pq_block_reduce
 * (pq_fused_h20.cu:3094) and aten topk + pq_cast_topk
 * (benchmarks/e2e_pq_param_sweep.py:212-217, pq_fused_h20.cu:3148).
 * Needs the KV binding (it resolves the selected rows' cache offsets). */
int pqhsa_scan_select(const pqhsa_params* p, void* stream);

/* (4)+(5b) Exact attention over sink, local window and the selected keys read in
 * place from the (paged) cache, background = per-list mass x list mean value,
 * one softmax; writes p->out.  Needs pqhsa_scan_select first.  Replaces
 * pq_attend_partial_nw(_paged) / pq_attend_bg / pq_attend_reduce_mw
 * (pq_fused_h20.cu:1225-1753, :2150-2402). */
int pqhsa_attend_merge(const pqhsa_params* p, void* stream);

/* The whole step: the three calls above in order.  Stands in for one replay of
 * the reference's per-layer CUDA graph body
 * (benchmarks/e2e_pq_param_sweep.py:6308-6969). */
int pqhsa_decode_step(const pqhsa_params* p, void* stream);

/* One kernel group of the step on its own, for per-kernel timing and profiling:
 * the same launches pqhsa_decode_step makes, in the same order. */
enum pqhsa_stage {
  PQHSA_STAGE_LUT = 0,      /* table construction + threshold estimate */
  PQHSA_STAGE_SCAN = 1,     /* code scan                               */
  PQHSA_STAGE_SELECT = 2,   /* exact selection among the candidates    */
  PQHSA_STAGE_ATTEND = 3,   /* exact attention partials (the gather) and the background partial */
  PQHSA_STAGE_MERGE = 4     /* fold of the partials into the output rows              */
};

/* A whole decode step including the token append, in the five launches of pqhsa_decode_step:
 *   pqhsa_append_kv(new_k, new_v) + pqhsa_append_encode(enc_count, uniform_count) + pqhsa_decode_step
 * with the row write, the encode and the table construction running side by side in the first
 * kernel (they touch disjoint data; the stream counters change once all three are done).  Same
 * results as the three calls in sequence.  new_k / new_v: E [S, 128], 16-byte aligned, or both
 * NULL when the caller's cache write already happened (no row is written, the length stays).
 * The per-layer step of the reference's decode loop (pq_append_prep + deferred incremental
 * encode + attention, benchmarks/e2e_pq_param_sweep.py:6308-6969). */
int pqhsa_decode_step_append(const pqhsa_params* p, const void* new_k, const void* new_v,
                             const int32_t* enc_count, int32_t uniform_count, void* stream);

int pqhsa_run_stage(const pqhsa_params* p, int stage, void* stream);

/* Copy `bytes` (a multiple of 16, both pointers 16-byte aligned) with a kernel instead of a copy-engine
 * transfer.  Meant for a step's inputs (queries, new K/V rows: tens of KB) sitting in pinned host memory
 * that is mapped into the device's address space: for such sizes a kernel reading over PCIe finishes
 * several microseconds before a cudaMemcpyAsync node would.  No counterpart in the reference (its inputs
 * are already on the device inside vLLM). */
int pqhsa_copy_small(void* dst, const void* src, size_t bytes, void* stream);

/* Launch `count` empty kernels (one warp each) on `stream`: the latency floor of a step's launches, timed by the
 * benchmark the same way as the step itself.  No counterpart in the reference. */
int pqhsa_launch_empty(int32_t count, void* stream);

/* Multi-GPU: enqueue the receiving side of the output exchange on `stream`.  One thread per flagged word of
 * this step's parity in this rank's receive buffer waits until the word carries this rank's step count and
 * stores its 4 bytes into peer_gather (the buffer of parity (steps - 1) & 1): when the kernel has ended, the
 * output rows of all ranks are there.  Every wait is bounded (peer_wait_polls); when one runs out,
 * peer_seq[1] is set to 1, the word is skipped and the kernel returns (the context stays usable).
 * Replaces the NCCL all-gather that would otherwise follow the step: the rows travel as plain
 * stores over NVLink from inside the combine kernel.  The reference has no counterpart (it runs
 * under vLLM's own tensor parallelism). */
int pqhsa_wait_peers(const pqhsa_params* p, void* stream);

/* Fold every stream's unsorted tail back into its list-sorted region, on the device and in place: the keys of a
 * list stay together in token order (the layout a stable sort by list gives), the scan units, the slots' unit
 * ids, the sample records and the counters N_SORTED / N_TAIL / N_UNITS are rebuilt.  One CTA per stream, no
 * scratch memory, no host round trip.  Streams with an empty tail are left alone.  A stream whose tail is longer
 * than PQHSA_COMPACT_MAX_TAIL (or whose units would not fit unit_capacity) is left as it is and `*error` (device
 * int32, caller-owned, not cleared by the call) is set to 1.  Replaces the snapshot rebuild after a flush
 * (benchmarks/e2e_pq_param_sweep.py:4163-4363: stable argsort over all list ids). */
int pqhsa_compact(const pqhsa_params* p, int32_t* error, void* stream);

/* Write one new K/V row per stream into the cache at position seq_len and bump
 * seq_len (contiguous or paged addressing as above).  new_k/new_v: E [S, 128].
 * Replaces pq_append_prep (pq_fused_h20.cu:2888-2922). */
int pqhsa_append_kv(const pqhsa_params* p, const void* new_k, const void* new_v, void* stream);

/* Incremental encode with fixed codebooks: for every stream, the next
 * enc_count[s] tokens after the indexed region (positions sink_end + N ...) are
 * read from the cache, split into norm and direction, assigned to the nearest
 * list, residual-encoded to 8 nibbles and appended to the tail; the list's
 * value sum / count / mean are updated.  enc_count: device int32 [S], or NULL
 * for `uniform_count` on every stream.  Mirrors IVFPQIndex.add
 * (pq_hsa/index/ivfpq.py:598-645) and the value-summary update
 * (pq_hsa/attention/kv_cache.py:730-764).  p->vsum / p->vcnt must be valid. */
int pqhsa_append_encode(const pqhsa_params* p, const int32_t* enc_count, int32_t uniform_count,
                        void* stream);

/* Bulk encode with fixed codebooks, outside any index pool: keys E [num_streams, n, 128]
 * (stream_stride elements from one stream's first key to the next's) are split into norm and
 * direction, assigned to the nearest of coarse E [num_streams, num_lists, 128] and
 * residual-encoded against codebooks E [num_streams, 8, 16, 16].  Writes, in the order of the
 * keys, codes u32 [num_streams, n] (subspace m = bits 4m..4m+3), norms E [num_streams, n] and
 * list_ids u16 [num_streams, n].  This is the assign-and-encode-every-key pass that ends
 * IVFPQIndex.build (pq_hsa/index/ivfpq.py:275-348) and the codebook-moving refresh
 * (:647-707), and IVFPQIndex.add (:598-645) for a large batch; same arithmetic as
 * pqhsa_append_encode, value for value.  The caller sorts the result into list order. */
int pqhsa_encode_bulk(const void* keys, int64_t stream_stride, int32_t num_streams, int32_t n, int32_t dtype,
                      const void* coarse, int32_t num_lists, const void* codebooks, uint32_t* codes, void* norms,
                      uint16_t* list_ids, void* stream);

/* The same with the lists given: list_ids u16 [num_streams, n] is read (a key's list from an earlier pass against the
 * same coarse centroids), the nearest-list search is skipped, and codes and norms come out as pqhsa_encode_bulk
 * writes them for those lists.  The index build uses it for its last pass, once the code words are trained
 * (pq_hsa/index/ivfpq.py:275-348: the lists are fixed before the code words are). */
int pqhsa_encode_bulk_assigned(const void* keys, int64_t stream_stride, int32_t num_streams, int32_t n, int32_t dtype,
                               const void* coarse, int32_t num_lists, const void* codebooks, const uint16_t* list_ids,
                               uint32_t* codes, void* norms, void* stream);

/* The Lloyd steps of the index build (pq_hsa/index/kmeans.py:195-224; code words: pq_hsa/index/pq.py:81-94) and
 * the per-list value sums (pq_hsa/attention/kv_cache.py:688-728), with results that do not depend on the order in
 * which thread blocks run.  The reference's update is `index_add_(0, assignments, vectors)`: on a CPU one fp32
 * addition per key and column in the order of the keys; the two calls below give exactly those sums.
 *
 * pqhsa_cluster_order: stable counting sort.  ids u16 [num_sets, n] hold a cluster id below k (1..PQHSA_MAX_LISTS)
 * per key; writes order int32 [num_sets, n] (order[j] = the key at place j when the keys are sorted by cluster and,
 * inside a cluster, by index) and start int32 [num_sets, k + 1] (first place of every cluster; start[k] = n).
 *
 * pqhsa_cluster_sums: rows E [num_streams][n] of row_stride elements (stream_stride elements from one stream's
 * first row to the next's); key set t = g * num_streams + s (g < groups) sums columns [g * width, (g + 1) * width)
 * of stream s's rows by the clusters of order / start [groups * num_streams, ...]; width divides 128.  Writes sums
 * float [groups * num_streams, k, width], every element the rows added one by one in the order of the keys. */
int pqhsa_cluster_order(const uint16_t* ids, int32_t num_sets, int32_t n, int32_t k, int32_t* order, int32_t* start,
                        void* stream);
int pqhsa_cluster_sums(const void* rows, int32_t dtype, int64_t stream_stride, int32_t row_stride, int32_t width,
                       int32_t num_streams, int32_t groups, int32_t n, int32_t k, const int32_t* order,
                       const int32_t* start, float* sums, void* stream);

/* The assignment of the code-word training: rows float [num_streams, n, 128] (residuals; stream_stride floats between
 * streams, 16-byte aligned), books float [num_streams, 8, 16, 16]; writes ids u16 [8, num_streams, n], the nearest
 * code word of every key in every subspace as argmin_c (|c|^2 - 2 x.c) (pq_hsa/index/kmeans.py:108-131), the first
 * minimum on ties. */
int pqhsa_subspace_assign(const float* rows, int64_t stream_stride, const float* books, int32_t num_streams, int32_t n,
                          uint16_t* ids, void* stream);

/* Test / inspection entry: approximate logits (scale * estimated q.k) of every
 * slot, float [R, cap], same arithmetic as the scan.  Counterpart of
 * score_packed_4bit_lut_multihead_list_bias
 * (pq_hsa/kernels/triton_lut_scan.py:1027-1104).  Needs pqhsa_lut_build first. */
int pqhsa_scan_scores(const pqhsa_params* p, float* scores, void* stream);

/* The same result as pqhsa_lut_build followed by pqhsa_scan_scores, for a caller that
 * cannot allocate device memory (an attention backend inside an inference server whose
 * free memory has all gone to the KV cache; a C host that owns only the buffers it was
 * handed).  It has no counterpart in the reference.  p->workspace is ignored: the
 * per-query tables go to a fixed array inside the library, so nothing is allocated or
 * freed, here or in any library routine.  Limits and rules:
 *   - at most PQHSA_STATIC_MAX_ROWS query rows (num_streams * group) per call, else
 *     PQHSA_E_CAPACITY; the array (~0.7 MB) stays resident on every GPU that loads the
 *     library until the process exits;
 *   - the first call on a device looks up the array's device address (a one-time set-up
 *     that talks to the CUDA runtime): make that first call before any stream capture;
 *   - every call uses the same array: calls whose kernels could overlap on the GPU
 *     (different streams, no ordering between them) race with each other.  The array keeps
 *     whatever the last call left; the counters that must start at zero are cleared on
 *     the stream at the start of each call.
 * scores: float [R, slot_capacity]; q, the index pool and max_slots as for pqhsa_scan_scores. */
#define PQHSA_STATIC_MAX_ROWS 256
int pqhsa_scan_scores_static(const pqhsa_params* p, float* scores, void* stream);

/* Stand-alone exact top-k of float rows: scores [rows, row_stride] (first n
 * valid) -> out_idx int32 [rows, k] (unordered) and out_val float [rows, k].
 * Ties at the k-th value are resolved towards the lower index.  Counterpart of
 * pq_topk_radix (pq_fused_h20.cu:3624-3688) / torch.topk. */
int pqhsa_topk_radix(const float* scores, int32_t rows, int32_t n, int64_t row_stride, int32_t k,
                     int32_t* out_idx, float* out_val, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* PQHSA_H_ */
