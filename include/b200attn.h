/* b200attn -- C ABI of the B200 (sm_100a) attention library.
 *
 * Every entry point takes plain pointers and sizes (no torch types), launches
 * asynchronously on the given CUDA stream, never allocates device memory and
 * never throws: it returns 0 or a negative b200attn_status.  All pointers are
 * device pointers that stay owned by the caller and must stay valid until the
 * stream has run the launch.  Strides are in ELEMENTS of the tensor's dtype;
 * the innermost (head_dim) stride is always 1.  Q, K, V and O share one
 * head_dim (the reference wrappers take a separate width for V,
 * flash_attn_decoding.py:233-236, but allocate O with Q's, flash_attn_triton.py:608).
 *
 * Threads and devices: calls are re-entrant and may come from any host
 * thread; the library keeps no state beyond read-only per-device facts looked
 * up once under std::call_once.  Every launcher checks, after its arguments,
 * that the current device is compute capability 10.x and answers
 * B200ATTN_ERR_DEVICE otherwise (the reference only probes for Hopper,
 * utils/utils.py:19-24).  B200ATTN_ASSUME_CC_MAJOR=<n> in the environment
 * replaces the probed major version, so that refusal can be exercised on a
 * machine whose GPUs are all sm_100.
 *
 * Device-side waits are bounded: a kernel whose wait on a copy or a product
 * gives up drains, returns normally and sets *status_word (where the argument
 * struct has one and it is not NULL); its outputs are then invalid.
 *
 * Each function names the reference interface (rookie-joe/TritonOps,
 * path:line inside that project) it stands in for.
 */
#ifndef B200ATTN_H_
#define B200ATTN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200ATTN_ABI_VERSION 1

typedef struct CUstream_st* b200attn_stream_t; /* == cudaStream_t */

typedef enum {
  B200ATTN_OK = 0,
  B200ATTN_ERR_NULL = -1,        /* a required pointer is NULL */
  B200ATTN_ERR_DTYPE = -2,       /* dtype is not F16 / BF16 */
  B200ATTN_ERR_HEAD_DIM = -3,    /* head_dim not in {32, 64, 96, 128} */
  B200ATTN_ERR_GQA = -4,         /* heads_q not a positive multiple of heads_kv */
  B200ATTN_ERR_ALIGN = -5,       /* base pointer not 16-byte aligned */
  B200ATTN_ERR_STRIDE = -6,      /* a stride is not a multiple of 8 elements (16 bytes) */
  B200ATTN_ERR_SHAPE = -7,       /* negative / zero / inconsistent sizes */
  B200ATTN_ERR_WORKSPACE = -8,   /* workspace missing or too small */
  B200ATTN_ERR_MODE = -9,        /* unknown sparsity mode or bad window / block parameters */
  B200ATTN_ERR_CUDA = -10,       /* a CUDA call failed (launch, tensor-map encode, ...) */
  B200ATTN_ERR_TOO_LARGE = -11,  /* problem exceeds a built-in limit */
  B200ATTN_ERR_DEVICE = -12      /* current device is not compute capability 10.x */
} b200attn_status;

typedef enum { B200ATTN_F16 = 0, B200ATTN_BF16 = 1, B200ATTN_F32 = 2 /* RMSNorm only */ } b200attn_dtype;

typedef enum {
  B200ATTN_DENSE = 0,       /* every (causally) visible key */
  B200ATTN_WINDOW = 1,      /* the reference's sparsity: local sliding window + global prefix */
  B200ATTN_BLOCK_LIST = 2   /* explicit sorted KV-block index lists */
} b200attn_sparsity;

/* ------------------------------------------------------------------------
 * Prefill (many query tokens per sequence).
 *
 * Logical tensors: q [batch, tokens, heads_q, head_dim], k/v [batch, tokens,
 * heads_kv, head_dim], o like q, lse fp32 [batch, tokens, heads_q].
 * Two addressing forms:
 *   packed varlen (the reference's): cu_seqlens != NULL, int32 [batch+1];
 *     sequence b owns token rows cu[b]..cu[b+1] of one [total_tokens, heads,
 *     head_dim] array; *_stride_b is ignored.
 *   fixed length: cu_seqlens == NULL; every sequence has `seqlen` tokens and
 *     starts at b * *_stride_b.
 * Query head h reads KV head h / (heads_q / heads_kv).
 * ---------------------------------------------------------------------- */
typedef struct {
  const void* q;
  const void* k;
  const void* v;
  void* o;
  float* lse;                 /* nullable */
  int32_t dtype;              /* b200attn_dtype */
  int32_t batch, heads_q, heads_kv, head_dim;
  int32_t seqlen;             /* fixed-length form: tokens per sequence */
  int32_t max_seqlen;         /* varlen form: upper bound on cu[b+1]-cu[b]; it sizes the grid, and a longer
                                 sequence is cut at ceil(max_seqlen / 256) * 256 tokens */
  int64_t total_tokens;       /* varlen form: rows in the packed arrays */
  const int32_t* cu_seqlens;  /* nullable, see above */
  int64_t q_stride_b, q_stride_t, q_stride_h;
  int64_t k_stride_b, k_stride_t, k_stride_h;
  int64_t v_stride_b, v_stride_t, v_stride_h;
  int64_t o_stride_b, o_stride_t, o_stride_h;
  int64_t lse_stride_b, lse_stride_t, lse_stride_h;
  float softmax_scale;        /* multiplies q.k before the softmax */
  int32_t scale_has_log2e;    /* 1: softmax_scale already contains log2(e), as the reference's sm_scale does */
  int32_t causal;             /* 1: key j visible to query i only if j <= i */
  int32_t lse_base2;          /* 1: store log2-domain LSE of the log2e-prescaled scores (reference), 0: natural log */
  /* sparsity (ignored by b200attn_prefill_fwd) */
  int32_t sparsity;           /* b200attn_sparsity */
  int32_t window_local;       /* WINDOW: i - j < window_local ... */
  int32_t window_global;      /* ... or j < window_global */
  const int32_t* block_idx;   /* BLOCK_LIST: int32 [batch, heads_q, n_qblocks, max_nnz], ascending, -1 padded */
  const int32_t* block_cnt;   /* BLOCK_LIST: int32 [batch, heads_q, n_qblocks] */
  int32_t block_size;         /* BLOCK_LIST: 64 */
  int32_t n_qblocks;          /* BLOCK_LIST: third extent of block_idx / block_cnt */
  int32_t max_nnz;            /* BLOCK_LIST: last extent of block_idx */
  int32_t* status_word;       /* nullable; device int set non-zero if a bounded device-side wait gave up */
} b200attn_prefill_args;

/* Dense causal / non-causal varlen GQA forward.  Replaces flash_attn_triton_fwd
 * (flash_attn_triton/flash_attn_triton.py:595-658) and its kernel (:52-180). */
int b200attn_prefill_fwd(const b200attn_prefill_args* args, b200attn_stream_t stream);

/* The same forward restricted to the query rows [row_begin, row_end) of every sequence: only
 * those rows of o and lse are written.  row_begin is a multiple of 256; row_end is a multiple of
 * 256 or reaches the end of the longest sequence (B200ATTN_ERR_SHAPE otherwise).  With causal = 1
 * the call reads no K / V row at or beyond row_end, so a caller whose sequence is still arriving
 * (from the host, from a peer) can attend to the rows that have landed while the next ones are on
 * their way; rows computed this way are bit-identical to those of the full call.  The reference
 * has no counterpart: its launcher (flash_attn_triton/flash_attn_triton.py:595-658) always covers
 * whole sequences.  tritonops_b200/host.py streams host buffers through it. */
int b200attn_prefill_fwd_rows(const b200attn_prefill_args* args, int32_t row_begin, int32_t row_end,
                              b200attn_stream_t stream);

/* Window-sparse (local + global) or block-list sparse forward.  Replaces the
 * launcher body at flash_attn_triton/flash_attn_sparse_attn_triton.py:237-326
 * and its kernel (:47-234), with the mask of the torch function at :422-433. */
int b200attn_sparse_prefill_fwd(const b200attn_prefill_args* args, b200attn_stream_t stream);

/* ------------------------------------------------------------------------
 * Decoding (one query token per sequence over a padded KV cache).
 *
 * q [batch, heads_q, head_dim], k_cache/v_cache [batch, capacity, heads_kv,
 * head_dim], o like q.  Lengths come from cu_seqlens (len_b = cu[b+1]-cu[b],
 * exactly the reference's use of it) or from seqlens (int32 [batch]); give
 * one of the two.  Split-KV: phase 1 writes fp32 partials into `workspace`,
 * phase 2 combines them by their log-sum-exp.
 * ---------------------------------------------------------------------- */
typedef struct {
  const void* q;
  const void* k_cache;
  const void* v_cache;
  void* o;
  int32_t dtype;
  int32_t batch, heads_q, heads_kv, head_dim;
  int32_t max_seqlen;         /* upper bound on the lengths (<= cache capacity); a longer length is cut there */
  const int32_t* cu_seqlens;  /* nullable */
  const int32_t* seqlens;     /* nullable */
  int64_t q_stride_b, q_stride_h;
  int64_t k_stride_b, k_stride_t, k_stride_h;
  int64_t v_stride_b, v_stride_t, v_stride_h;
  int64_t o_stride_b, o_stride_h;
  float softmax_scale;        /* natural scale, e.g. head_dim^-0.5 */
  int32_t chunk_tokens;       /* split size, multiple of 64; 0 = chosen from the problem size (128..8192) */
  /* sparsity (ignored by b200attn_decode_fwd) */
  int32_t sparsity;
  int32_t window_global;      /* WINDOW: key j visible iff j < window_global ... */
  int32_t window_local;       /* ... or j >= len - window_local */
  const int32_t* block_idx;   /* BLOCK_LIST: int32 [batch, heads_kv, max_sel] ascending, -1 padded */
  const int32_t* block_cnt;   /* BLOCK_LIST: nullable int32 [batch, heads_kv]; NULL = max_sel entries */
  int32_t block_size;         /* BLOCK_LIST: multiple of 16 */
  int32_t max_sel;
  void* workspace;
  size_t workspace_bytes;
  int32_t* status_word;       /* nullable; device int set to 1 if a bounded wait of the split kernel gave up
                                 (the chunks it could not finish count as empty) */
} b200attn_decode_args;

/* Bytes of scratch b200attn_decode_fwd / b200attn_sparse_decode_fwd need. */
size_t b200attn_decode_workspace_bytes(const b200attn_decode_args* args);

/* GQA split-KV decoding + LSE combine.  Replaces flash_attention_decoding
 * (flash_attn_triton/flash_attn_decoding.py:213-336) and its two kernels
 * (:9-122, :126-210). */
int b200attn_decode_fwd(const b200attn_decode_args* args, b200attn_stream_t stream);

/* Window (sink + recent) or block-list decoding.  Replaces
 * flash_attention_sparse_decoding (flash_attn_triton/flash_attn_decoding_sparse.py:222-365)
 * and its kernels (:10-127, :131-219). */
int b200attn_sparse_decode_fwd(const b200attn_decode_args* args, b200attn_stream_t stream);

/* Dense GQA decoding for callers that cannot allocate.  No counterpart in the
 * reference (its wrapper allocates three tensors per call,
 * flash_attn_decoding.py:249-261); this entry point exists for hosts where
 * nobody may call cudaMalloc when a request arrives: an inference server
 * that has already handed all free HBM to its KV-cache pool, a real-time loop
 * that must not hit the implicit device synchronisation of cudaMalloc/cudaFree,
 * or a plugin running inside another runtime's fixed arena.  Same arguments
 * and results as b200attn_decode_fwd, except that `workspace` and
 * `workspace_bytes` are ignored: the split-KV partials go to a fixed array of
 * B200ATTN_NOALLOC_SCRATCH_BYTES that is part of the library image, so every
 * GPU that loads the library carries those bytes until the process exits.
 *   - A problem whose b200attn_decode_workspace_bytes() exceeds that size is
 *     rejected with B200ATTN_ERR_TOO_LARGE (config 3, B=64 Hq=32 D=128 with
 *     8192-token caches, needs 4.0 MiB with the default split and fits).
 *   - The first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress, with that device current) and keeps it; make
 *     that first call before starting any stream capture.  No call allocates:
 *     no cudaMalloc, cudaFree or allocating library routine is used.
 *   - All calls on one device share the array and it keeps the previous
 *     call's contents.  Nothing in it has to start at zero (every partial a
 *     call reads was written by that same call), but two calls that overlap
 *     on the GPU -- different streams, or different host threads -- race on
 *     it: run them on one stream or order them with events. */
#define B200ATTN_NOALLOC_SCRATCH_BYTES (32u << 20)
int b200attn_decode_fwd_noalloc(const b200attn_decode_args* args, b200attn_stream_t stream);

/* ------------------------------------------------------------------------
 * Decoding over a paged KV cache.
 *
 * k_pages / v_pages are pools [num_pages, page_size, heads_kv, head_dim];
 * page_table[b][i] is the pool page that holds keys i*page_size .. of sequence
 * b (entries at or beyond ceil(len_b / page_size) are not read).  Pages must
 * follow one another in memory: *_stride_page == page_size * *_stride_t.
 * ---------------------------------------------------------------------- */
typedef struct {
  const void* q;               /* [batch, heads_q, head_dim] */
  const void* k_pages;
  const void* v_pages;
  void* o;                     /* like q */
  int32_t dtype;
  int32_t batch, heads_q, heads_kv, head_dim;
  int32_t page_size;           /* keys per page, a multiple of 16 */
  int32_t num_pages;           /* pages in the pool */
  int32_t max_pages_per_seq;   /* row length of page_table */
  int32_t max_seqlen;          /* upper bound on the lengths */
  const int32_t* page_table;   /* int32 [batch, max_pages_per_seq] */
  const int32_t* seqlens;      /* int32 [batch] */
  int64_t q_stride_b, q_stride_h;
  int64_t k_stride_page, k_stride_t, k_stride_h;
  int64_t v_stride_page, v_stride_t, v_stride_h;
  int64_t o_stride_b, o_stride_h;
  float softmax_scale;         /* natural scale */
  int32_t chunk_tokens;        /* as in b200attn_decode_args */
  void* workspace;
  size_t workspace_bytes;
  int32_t* status_word;        /* nullable; as in b200attn_decode_args */
} b200attn_paged_decode_args;

size_t b200attn_paged_decode_workspace_bytes(const b200attn_paged_decode_args* args);

/* GQA split-KV decoding whose keys are found through a page table; same
 * arithmetic as b200attn_decode_fwd on the equivalent padded cache.  The
 * reference has no paged form: its decoding kernels index one padded cache
 * per sequence (flash_attn_triton/flash_attn_decoding.py:62-69); here the row
 * of key t is looked up per page instead of being b * stride + t. */
int b200attn_paged_decode_fwd(const b200attn_paged_decode_args* args, b200attn_stream_t stream);

/* ------------------------------------------------------------------------
 * Block selection: building the block lists the BLOCK_LIST modes take, on the
 * device, with no host work between the producer of the pattern and the
 * attention launch.
 * ---------------------------------------------------------------------- */
typedef struct {
  int32_t* block_idx;          /* out int32 [batch, heads, n_qblocks, max_nnz], ascending, -1 padded */
  int32_t* block_cnt;          /* out int32 [batch, heads, n_qblocks] */
  int32_t batch, heads, n_qblocks, max_nnz;
  int32_t block_size;
  int32_t window_local, window_global;
} b200attn_window_blocks_prefill_args;

/* Upper bound on the blocks one query block can select (sizes max_nnz). */
int32_t b200attn_window_blocks_prefill_max_nnz(int32_t block_size, int32_t window_local, int32_t window_global,
                                               int32_t n_qblocks);

/* The block cover of the reference's window pattern for prefill: query block i
 * lists KV block j <= i iff some query of block i sees some key of block j
 * under "i_q - j_k < window_local or j_k < window_global"
 * (flash_attn_triton/flash_attn_sparse_attn_triton.py:125-129, 178-183 give
 * the same two key ranges per query tile).  Whole listed blocks are attended,
 * so the result is a superset of the exact window; B200ATTN_ERR_TOO_LARGE if a
 * row needs more than max_nnz entries. */
int b200attn_window_blocks_prefill(const b200attn_window_blocks_prefill_args* args, b200attn_stream_t stream);

typedef struct {
  int32_t* block_idx;          /* out int32 [batch, heads_kv, max_sel], ascending, -1 padded */
  int32_t* block_cnt;          /* out int32 [batch, heads_kv] */
  const int32_t* cu_seqlens;   /* nullable; give one of the two, as for decoding */
  const int32_t* seqlens;
  int32_t batch, heads_kv, max_sel;
  int32_t block_size;
  int32_t window_local, window_global;
} b200attn_window_blocks_decode_args;

/* The blocks that hold keys "j < window_global or j >= len - window_local" of
 * each sequence (flash_attn_triton/flash_attn_decoding_sparse.py:52-58, 82-85;
 * the wrapper's chunk count :256-266 is the same cover in units of
 * window_global).  Rows that would need more than max_sel entries keep the
 * first max_sel. */
int b200attn_window_blocks_decode(const b200attn_window_blocks_decode_args* args, b200attn_stream_t stream);

typedef struct {
  const float* scores;         /* fp32 [rows, n_blocks] block scores, larger = more important */
  int64_t score_stride_row;    /* elements between rows */
  const int32_t* n_valid;      /* nullable int32 [rows]: only blocks 0 .. n_valid-1 are candidates
                                  (causal prefill: query block + 1; decoding: ceil(len / block)) */
  int32_t rows, n_blocks;      /* n_blocks <= 8192 */
  int32_t top_k;               /* entries per output row */
  int32_t force_first;         /* this many leading candidate blocks are always taken (attention sinks) */
  int32_t force_last;          /* this many trailing candidate blocks are always taken (the diagonal / newest block) */
  int32_t* block_idx;          /* out int32 [rows, top_k], ascending, -1 padded */
  int32_t* block_cnt;          /* out int32 [rows] = min(top_k, candidates) */
} b200attn_topk_blocks_args;

/* Per row, the top_k highest-scoring candidate blocks, returned in ascending
 * block order as the BLOCK_LIST modes want them.  Ties go to the lower block
 * number and NaN scores rank last, so the result is a pure function of the
 * scores.  No counterpart in the reference, whose sparsity is fixed to the
 * window pattern (flash_attn_triton/flash_attn_decoding_sparse.py:82-85). */
int b200attn_topk_blocks(const b200attn_topk_blocks_args* args, b200attn_stream_t stream);

/* ------------------------------------------------------------------------
 * Dense prefill backward.  Tensors and addressing forms as in
 * b200attn_prefill_args; o and lse are the forward's outputs, d_o the
 * gradient of o; dq like q, dk / dv like k / v (the query heads of a GQA group
 * are summed into their KV head).  Workspace: fp32 dq accumulator + row sums.
 * ---------------------------------------------------------------------- */
typedef struct {
  const void* q;
  const void* k;
  const void* v;
  const void* o;
  const void* d_o;
  const float* lse;
  void* dq;
  void* dk;
  void* dv;
  int32_t dtype;
  int32_t batch, heads_q, heads_kv, head_dim;
  int32_t seqlen, max_seqlen;
  int64_t total_tokens;
  const int32_t* cu_seqlens;
  int64_t q_stride_b, q_stride_t, q_stride_h;
  int64_t k_stride_b, k_stride_t, k_stride_h;
  int64_t v_stride_b, v_stride_t, v_stride_h;
  int64_t o_stride_b, o_stride_t, o_stride_h;
  int64_t do_stride_b, do_stride_t, do_stride_h;
  int64_t dq_stride_b, dq_stride_t, dq_stride_h;
  int64_t dk_stride_b, dk_stride_t, dk_stride_h;
  int64_t dv_stride_b, dv_stride_t, dv_stride_h;
  int64_t lse_stride_b, lse_stride_t, lse_stride_h;
  float softmax_scale;
  int32_t scale_has_log2e;
  int32_t causal;
  int32_t lse_base2;           /* form of `lse`, as written by the forward */
  void* workspace;
  size_t workspace_bytes;
  int32_t* status_word;
} b200attn_prefill_bwd_args;

size_t b200attn_prefill_bwd_workspace_bytes(const b200attn_prefill_bwd_args* args);

/* dQ, dK, dV of the dense causal / non-causal forward.  Replaces
 * flash_attn_triton_bwd (flash_attn_triton/flash_attn_triton.py:661-813) and
 * its kernels (:184-592).  dK and dV are summed in a fixed order and repeat
 * bit for bit; dQ is summed in fp32 by reduce-adds whose order is not fixed
 * (the reference's separate dQ kernel, :255-410, is deterministic), so two
 * runs may differ in the last bit of the 16-bit result. */
int b200attn_prefill_bwd(const b200attn_prefill_bwd_args* args, b200attn_stream_t stream);

/* ------------------------------------------------------------------------
 * KV-cache glue (16-bit elements, head_dim a multiple of 8).
 * ---------------------------------------------------------------------- */
typedef struct {
  const void* packed;          /* [total_tokens, heads, head_dim] rows of all sequences */
  void* cache;                 /* [batch, capacity, heads, head_dim] */
  const int32_t* cu_seqlens;   /* int32 [batch+1] */
  int32_t batch, heads, head_dim, capacity;
  int64_t packed_stride_t, packed_stride_h;
  int64_t cache_stride_b, cache_stride_t, cache_stride_h;
  int32_t zero_pad;            /* 1: rows t >= len_b of the cache are set to zero */
} b200attn_kv_pack_args;

/* Packed varlen K (or V) rows -> padded cache: cache[b, t] = packed[cu[b] + t]
 * for t < len_b.  Replaces the Python copy loops of the reference's decoding
 * tests (flash_attn_triton/flash_attn_decoding.py:404-425). */
int b200attn_kv_pack_to_cache(const b200attn_kv_pack_args* args, b200attn_stream_t stream);

typedef struct {
  const void* new_k;           /* [batch, heads, head_dim] the token to append */
  const void* new_v;
  void* k_cache;               /* [batch, capacity, heads, head_dim] */
  void* v_cache;
  const int32_t* seqlens;      /* int32 [batch]: current lengths = write positions */
  int32_t batch, heads, head_dim, capacity;
  int64_t new_stride_b, new_stride_h;
  int64_t cache_stride_b, cache_stride_t, cache_stride_h;
} b200attn_kv_append_args;

/* One decoding step's new K/V rows written at position len_b of each sequence
 * (sequences already at capacity are skipped).  No counterpart function in the
 * reference, whose tests rebuild the whole cache instead
 * (flash_attn_triton/flash_attn_decoding_sparse.py:445-466). */
int b200attn_kv_append(const b200attn_kv_append_args* args, b200attn_stream_t stream);

/* ------------------------------------------------------------------------
 * RMSNorm over the last dimension of a [rows, dim] view (the op in front of the
 * QKV projection).  x / y / dy / dx share one dtype (F16, BF16 or F32); weight
 * and dweight have that dtype or F32.  Row strides are in elements, the inner
 * stride is 1.  Arithmetic is fp32.
 * ---------------------------------------------------------------------- */
typedef struct {
  const void* x;
  const void* weight;          /* [dim] */
  void* y;
  float* rstd;                 /* nullable; fp32 [rows] = (mean(x^2) + eps)^-1/2, needed by the backward */
  int32_t x_dtype, w_dtype;
  int64_t rows;
  int32_t dim;
  int64_t x_stride_row, y_stride_row;
  float eps;
} b200attn_rmsnorm_fwd_args;

/* y = x * rstd * weight.  Replaces RMSNormTritonFunction.forward and
 * rmsnorm_fwd_kernel (common/rms.py:221-290, :9-88). */
int b200attn_rmsnorm_fwd(const b200attn_rmsnorm_fwd_args* args, b200attn_stream_t stream);

typedef struct {
  const void* dy;
  const void* x;
  const void* weight;
  const float* rstd;           /* from the forward */
  void* dx;
  void* dweight;               /* [dim], overwritten */
  int32_t x_dtype, w_dtype;
  int64_t rows;
  int32_t dim;                 /* <= 16384 */
  int64_t dy_stride_row, x_stride_row, dx_stride_row;
  void* workspace;             /* fp32 partial sums of dweight */
  size_t workspace_bytes;
} b200attn_rmsnorm_bwd_args;

size_t b200attn_rmsnorm_bwd_workspace_bytes(const b200attn_rmsnorm_bwd_args* args);

/* dx and dweight.  Replaces RMSNormTritonFunction.backward and rmsnorm_bwd_kernel
 * (common/rms.py:292-355, :91-218); dweight is summed in a fixed order instead of
 * with atomics (:217), and the weights used inside the row sum are those of the
 * summed columns (the reference kernel takes another block's for dim > 128, :197-199). */
int b200attn_rmsnorm_bwd(const b200attn_rmsnorm_bwd_args* args, b200attn_stream_t stream);

/* Self-test of the bounded device-side wait the kernels use (every spin on an
 * mbarrier has a cycle budget; when it runs out the CTA raises an abort flag, all
 * its roles drain, the kernel returns normally and *status_word is set non-zero).
 * Launches one CTA that waits on a barrier nothing ever completes, with the given
 * budget in SM cycles (at most 1e8, about 50 ms).  Afterwards *status_word == 3 (the
 * waiting thread gave up, and a second thread's wait returned at once) and
 * *waited_cycles (nullable) holds how long the first wait lasted.  The reference has
 * no counterpart (Triton kernels do not wait on one another). */
int b200attn_selftest_bounded_wait(int32_t* status_word, int64_t budget_cycles, int64_t* waited_cycles,
                                   b200attn_stream_t stream);

/* Prefill needs no scratch; kept so callers can size buffers uniformly. */
size_t b200attn_prefill_workspace_bytes(const b200attn_prefill_args* args);

const char* b200attn_strerror(int status);
int b200attn_abi_version(void);
/* Number of kernels the last call on this thread launched (for accounting). */
int b200attn_last_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* B200ATTN_H_ */
