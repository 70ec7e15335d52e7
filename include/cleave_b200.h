/*
 * cleave_b200 - C ABI of the sm_100a kernel library behind Cleave's scheduled plans.
 *
 * The reference (nyu-systems/cleave) has no C FFI: a scheduled plan is turned into TileLang
 * source (python/cleave/codegen/__init__.py:24-48), JIT-compiled (python/cleave/runtime/compile.py:30-34)
 * and called as kernel(*tensors). Each entry point below is what such a compiled kernel object
 * binds to instead; the comment on every function names the reference kernel it replaces.
 *
 * Conventions
 *  - plain pointers and sizes only; all tensor pointers are DEVICE pointers, caller-owned,
 *    inputs are never written;
 *  - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream);
 *  - every launch function returns a cb200_status (0 = ok); nothing throws, nothing
 *    allocates device memory, nothing synchronises: a launch can be captured in a CUDA graph
 *    (the reference times kernels by graph replay, python/cleave/runtime/timer.py:14-108);
 *  - scratch ("workspace") is caller-owned; ask cb200_*_workspace_bytes() for the size. A
 *    workspace must be zero-filled once before its first use; every launch leaves it
 *    zero-filled where that matters, so it can be reused by the next launch on the same
 *    stream. Two launches that overlap on the GPU must not share a workspace;
 *  - a kernel that gives up a bounded wait records it in the first word of its workspace;
 *    cb200_workspace_status() reads it back (synchronises the stream).
 *  - storage dtypes are IEEE half (CB200_F16) or bfloat16 (CB200_BF16); accumulation, softmax
 *    and norm statistics are fp32.
 */
#ifndef CLEAVE_B200_H
#define CLEAVE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* 2: cb200_gemm_args and cb200_attn_prefill_args gained trailing fields (zero = the behaviour of version 1);
 *    new entry points cb200_matmul_matmul, cb200_matmul_rowsum, cb200_lora. A binding written against
 *    version 1 must zero-fill the longer structs. */
/* 3: cb200_workspace_status clears a reported fault; new cb200_workspace_reset,
 *    cb200_attn_decode_static_scratch_status, cb200_split_combine, cb200_attn_unnormalise, cb200_mla_prefill,
 *    cb200_gemm_plan;
 *    cb200_gemm_args gained
 *    the trailing field ldx (zero = the behaviour of version 2). */
/* 4: cb200_attn_prefill_ragged_args gained the trailing field num_kv_indices (zero = the behaviour of
 *    version 3); the paged MLA decode clips request ranges to num_kv_indices; new cb200_set_small_problem_limit. */
/* 5: cb200_gemm_args gained the trailing fields ldy, n_peers, y_peers (zero = the behaviour of version 4): a result
 *    with its own row pitch that the kernel also stores into the copies of peer GPUs; new cb200_peer_scatter_cols. */
#define CB200_VERSION 5

typedef enum {
  CB200_OK = 0,
  CB200_ERR_BAD_ARG = 1,       /* NULL pointer, non-positive extent, inconsistent shapes */
  CB200_ERR_UNSUPPORTED = 2,   /* shape / dtype outside what the kernels implement */
  CB200_ERR_ALIGNMENT = 3,     /* pointer or stride not 16-byte aligned */
  CB200_ERR_WORKSPACE = 4,     /* workspace NULL or too small */
  CB200_ERR_CUDA = 5,          /* a CUDA runtime / driver call failed (see cb200_last_cuda_error) */
  CB200_ERR_DEVICE_TIMEOUT = 6, /* a bounded device-side wait gave up (from cb200_workspace_status) */
  CB200_ERR_SCRATCH_LIMIT = 7   /* the problem needs more scratch than the built-in static array holds */
} cb200_status;

typedef enum { CB200_F16 = 0, CB200_BF16 = 1 } cb200_dtype;

int cb200_version(void);
const char* cb200_strerror(int status);
/* cudaError_t of the most recent failing CUDA call made by this library on this thread. */
int cb200_last_cuda_error(void);
/* Number of SMs of the current device (grid sizing is a multiple of it). */
int cb200_sm_count(void);
/* Copies the status word of `workspace` to the host after synchronising `stream`.
 * Returns CB200_OK, CB200_ERR_DEVICE_TIMEOUT or CB200_ERR_CUDA. A fault is reported once: the status word is
 * cleared before the function returns. The launch that faulted did not finish its items, so their arrival
 * counters are still dirty: zero the workspace (cb200_workspace_reset) before launching on it again. */
int cb200_workspace_status(const void* workspace, void* stream);
/* Zero-fills `workspace_bytes` bytes of `workspace` on `stream` (a cudaMemsetAsync; no synchronisation): the
 * state a workspace must be in before its first use and after a reported fault. */
int cb200_workspace_reset(void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------------------------
 * Decode attention, one query token per request: O = softmax(Q K^T * scale) V, plus the base-2
 * log-sum-exp. Query head h reads kv head h / (num_qo_heads / num_kv_heads)  (MHA, GQA, MQA).
 *
 * Replaces, for contiguous caches, the static split-KV pair
 *   tests/graph/handwritten/expected_kernels/{gqa,mha,mqa}_split_partial.py + mha_split_combine.py
 *   (operator: demo/attention.py:5-8, demo/{mha,gqa,mqa}_decode.py),
 * and, for paged caches, the paged decode kernels
 *   tests/graph/handwritten/expected_kernels/gqa_paged_decode_h32_kv8_d128_ps64.py  (slab, page 64)
 *   tests/graph/handwritten/expected_kernels/gqa_paged_decode_h32_kv{8,4}_d128_ps1.py (row gather)
 *   tests/graph/handwritten/expected_kernels/splitkv/gqa_paged_decode_*_splitkv8.py (split pair)
 *   built by python/cleave/dynamic/paging/builders/{slab,decode,combine}.py; argument order and
 *   meaning follow python/cleave/dynamic/reference.py:156-200.
 *
 * One persistent launch: KV tiles of 64 tokens are dealt evenly to one CTA per SM; a request
 * whose tiles span several CTAs is finished by the last CTA to arrive (fused log-sum-exp
 * combine, no second launch). Empty requests give out = 0, lse = -inf.
 * ---------------------------------------------------------------------------------------- */
typedef struct {
  const void* q;       /* (batch, num_qo_heads, head_dim) */
  const void* k_cache; /* paged: (num_pages, page_size, num_kv_heads, head_dim)
                          contiguous: (batch, num_kv_heads, kv_len, head_dim) */
  const void* v_cache; /* same layout as k_cache */
  const int32_t* kv_indptr;        /* (batch + 1), in pages; NULL selects contiguous caches */
  const int32_t* kv_indices;       /* (num_kv_indices) page ids */
  const int32_t* kv_last_page_len; /* (batch) tokens in each request's last page; may be NULL
                                      when page_size == 1 */
  void* out;  /* (batch, num_qo_heads, head_dim), storage dtype */
  float* lse; /* (batch, num_qo_heads) base-2 log-sum-exp; may be NULL */
  void* workspace;
  size_t workspace_bytes;
  int32_t batch;
  int32_t num_qo_heads;
  int32_t num_kv_heads;
  int32_t head_dim;       /* 64 or 128 */
  int32_t page_size;      /* paged only */
  int32_t num_pages;      /* paged only: pages in the pool */
  int32_t num_kv_indices; /* paged only: entries of kv_indices */
  int32_t kv_len;         /* contiguous only: tokens per request */
  int32_t q_rows;         /* query rows per head (S_Q of the static operator); 0 or 1 = decode */
  int32_t dtype;          /* cb200_dtype */
  int32_t max_ctas;       /* 0 = one CTA per SM; otherwise an upper bound on the grid */
  float sm_scale;
} cb200_attn_decode_args;

size_t cb200_attn_decode_workspace_bytes(const cb200_attn_decode_args* a);
int cb200_attn_decode(const cb200_attn_decode_args* a, void* stream);

/* ------------------------------------------------------------------------------------------
 * Fused dense contractions on the tcgen05 tensor cores. X is (m, k) row-major, W (and W1) are
 * (k, n) row-major, Y is (m, n) row-major; k and n must be multiples of 8.
 *   CB200_GEMM_MATMUL   Y = X @ W
 *       replaces tests/graph/handwritten/expected_kernels/matmul.py and the split-K pair
 *       matmul_splitk_partial.py + matmul_splitk_combine.py (operator demo/matmul.py:11-13)
 *   CB200_GEMM_RMSNORM  Y = (X * rsqrt(mean_k(X^2) + eps) [* gamma]) @ W, fp32 statistics
 *       replaces expected_kernels/rmsnorm_matmul.py and rmsnorm_matmul_split_{partial,combine}.py
 *       (operator demo/rmsnorm_matmul.py:11-13, python/cleave/frontend/composites.py:48-53);
 *       gamma (k) is an optional per-column weight of the normalised row, NULL = none
 *   CB200_GEMM_SWIGLU   Y = silu(X @ W) * (X @ W1)
 *       replaces expected_kernels/swiglu.py (operator demo/swiglu.py:6-10)
 * split_k is the plan's split factor (K chunks per output tile, e.g. 4, 8, 16); 0 lets the
 * library choose. The split-K combine is fused: one launch, partial tiles are summed in a fixed
 * order by the last CTA to arrive, so results are bit-stable for a given (shape, split, grid).
 * ---------------------------------------------------------------------------------------- */
typedef enum { CB200_GEMM_MATMUL = 0, CB200_GEMM_RMSNORM = 1, CB200_GEMM_SWIGLU = 2 } cb200_gemm_op;

typedef struct {
  const void* x;     /* (m, k) */
  const void* w;     /* (k, n) */
  const void* w1;    /* (k, n), SwiGLU only */
  const void* gamma; /* (k), RMSNorm only, may be NULL */
  void* y;           /* (m, n) */
  void* workspace;
  size_t workspace_bytes;
  int32_t m, n, k;
  int32_t op;       /* cb200_gemm_op */
  int32_t dtype;    /* cb200_dtype */
  int32_t split_k;  /* 0 = auto */
  int32_t max_ctas; /* 0 = one CTA per SM */
  float eps;        /* RMSNorm only */
  const void* addend; /* CB200_GEMM_MATMUL only, may be NULL: (m, n) in the storage dtype, Y = X @ W + addend
                         (added in fp32 in the epilogue; the low-rank term of cb200_lora) */
  int32_t dependent_launch; /* 0: the launch is ordered after the preceding kernel of the stream, as usual.
                               1: it may start while that kernel still runs and waits for it before reading any
                                  operand (set-up overlaps). 2: it waits only before reading `addend`. 3: it waits
                                  only before the first read of the second operand pair (x2, w2 below); a CTA whose
                                  share holds no K block of that pair never waits. cb200_lora streams W beside the
                                  rank-r product this way.
                               Contract of modes 2 and 3: every kernel of this library lets its successor start
                               before it has itself waited, so such a launch can run beside ANY kernel still in
                               flight on the stream, not only the one directly before it. X, W, Y's other inputs
                               and the workspace must therefore not be written, and the workspace not used at all,
                               by any kernel that may still be running when the launch is made; put an ordinary
                               launch (mode 0) before it, as cb200_lora does, and give it a workspace of its own. */
  /* Optional second operand pair, CB200_GEMM_MATMUL only (k2 = 0: none): Y = X @ W + X2 @ W2 [+ addend] in one
   * accumulator - the K blocks of X2 (m, k2) / W2 (k2, n) follow those of X / W. k2 a multiple of 8. */
  const void* x2;
  const void* w2;
  int32_t k2;
  int32_t ldx; /* CB200_GEMM_MATMUL only: elements between consecutive rows of X (0 = k, a dense matrix). A
                  multiple of 8. Lets a K slice of a wider matrix be the operand: the per-split products of the
                  two-stage split-K form are X[:, s K/S : (s+1) K/S] @ W[s K/S : (s+1) K/S, :]. */
  /* Version 5, trailing fields (zero = a dense local result, as before). A GEMM sharded along N over several GPUs
   * of one node whose every GPU wants the whole result (the reference has no multi-GPU path; this is the fused form
   * of "local product, then all-gather"): `y` points at this GPU's column slice inside its copy of the full result
   * (element [0, first own column]), `ldy` is the full row length in elements (a multiple of 8; the slice starts on
   * a multiple of 8 columns), and `y_peers[0 .. n_peers)` point at the same element of the other GPUs' copies
   * (peer-mapped device pointers: symmetric memory, CUDA IPC). The kernel writes every finished tile into its own
   * copy and, from four further warps, on into the peers' copies while it computes the next tile; nothing is
   * signalled: the caller orders the GPUs (a barrier) before any of them reads the result. Taken by the CTA-pair
   * kernel only (m >= 256, no split_k, max_ctas 0); CB200_ERR_UNSUPPORTED otherwise. */
  int32_t ldy;
  int32_t n_peers;      /* 0 .. 7 */
  void* y_peers[7];
} cb200_gemm_args;

size_t cb200_gemm_workspace_bytes(const cb200_gemm_args* a);
/* The plan the library would run for `a` (pointers are not read) and its cost model's estimate: the sm_100
 * counterpart of the score the reference's tile policy gives a candidate
 * (python/cleave/schedule/policy/default.py:1015-1110 scores tilings for sm_90 shared memory and wmma shapes).
 * A scheduler can rank split factors with it before anything is built. */
typedef struct {
  int32_t tile_m, tile_n; /* output tile of one CTA (128 x 128 / 128 x 256) or of a CTA pair (256 x 256) */
  int32_t split;          /* K parts per output tile that will really be used */
  int32_t kind;           /* 0 = whole tiles or a stream-K walk with a workspace fix-up, 1 = the K parts of a tile are
                             one thread-block cluster (reduced through distributed shared memory), 2 = CTA pairs */
  int32_t grid;           /* CTAs */
  float estimate_us;      /* the model's estimate for this plan */
} cb200_gemm_plan_info;
int cb200_gemm_plan(const cb200_gemm_args* a, cb200_gemm_plan_info* out);
/* K chunks per output tile the launch will use (the requested split clamped to the K extent). */
int cb200_gemm_effective_split(const cb200_gemm_args* a);
int cb200_gemm(const cb200_gemm_args* a, void* stream);

/* ------------------------------------------------------------------------------------------
 * MLA decode (absorbed latent): S = (Q_nope CKV^T + Q_pe KPE^T) * scale, O = softmax(S) CKV, plus
 * the base-2 log-sum-exp; ckv_dim = 512, kpe_dim = 64.
 *
 * Replaces the static MLA decode kernel of demo/mla_decode.py:8-13 (contiguous caches) and the
 * paged kernels tests/graph/handwritten/expected_kernels/mla_paged_decode_h16_ckv512_kpe64_ps1.py and
 * splitkv/mla_paged_decode_*_splitkv8.py (python/cleave/dynamic/paging/builders/mla.py); argument order
 * and meaning follow python/cleave/dynamic/reference.py:282-320. Paged caches hold one token per page.
 * ---------------------------------------------------------------------------------------- */
typedef enum { CB200_MLA_IMPL_AUTO = 0, CB200_MLA_IMPL_MMA_SYNC = 1, CB200_MLA_IMPL_TCGEN05 = 2 } cb200_mla_impl;

typedef struct {
  const void* q_nope;    /* (batch, num_heads, 512) */
  const void* q_pe;      /* (batch, num_heads, 64) */
  const void* ckv_cache; /* paged: (num_pages, 1, 512); contiguous: (batch, kv_len, 512) */
  const void* kpe_cache; /* paged: (num_pages, 1, 64);  contiguous: (batch, kv_len, 64) */
  const int32_t* kv_indptr;  /* (batch + 1), in tokens; NULL selects contiguous caches */
  const int32_t* kv_indices; /* (num_kv_indices) page ids */
  void* out;  /* (batch, num_heads, 512) */
  float* lse; /* (batch, num_heads) base 2, may be NULL */
  void* workspace;
  size_t workspace_bytes;
  int32_t batch;
  int32_t num_heads;
  int32_t ckv_dim;        /* 512 */
  int32_t kpe_dim;        /* 64 */
  int32_t page_size;      /* paged only: 1 */
  int32_t num_pages;      /* paged only */
  int32_t num_kv_indices; /* paged only */
  int32_t kv_len;         /* contiguous only */
  int32_t dtype;          /* cb200_dtype */
  int32_t max_ctas;       /* 0 = one CTA per SM */
  int32_t impl;           /* cb200_mla_impl: 0 = choose (tcgen05 kernels for contiguous caches with at least 64
                             heads and 512 tokens), 1 = mma.sync kernel, 2 = tcgen05 kernels (contiguous caches) */
  float sm_scale;
  /* Optional, paged only (NULL otherwise): request b reads kv_indices[kv_start[b] .. kv_start[b] + kv_lens[b])
   * instead of the range kv_indptr gives. Ranges may overlap: causal prefill
   * (mla_paged_prefill_causal_*, python/cleave/dynamic/reference.py:324-365) runs one request per query
   * token over the prefix of its sequence's pages that the end-aligned mask lets it see. */
  const int32_t* kv_start;
  const int32_t* kv_lens;
} cb200_mla_decode_args;

size_t cb200_mla_decode_workspace_bytes(const cb200_mla_decode_args* a);
int cb200_mla_decode(const cb200_mla_decode_args* a, void* stream);

/* ------------------------------------------------------------------------------------------
 * Unsplit attention with many query rows (the "prefill" shapes), tcgen05/TMEM kernel.
 *   O = softmax(sm_scale * Q K^T [+ causal mask]) V; query head h reads kv head h / (HQ / HKV).
 * Replaces the static unsplit attention kernels of demo/{mha,gqa,mqa}_prefill.py
 * (tests/graph/handwritten/expected_kernels/mha_bhsd.py); `causal` applies the end-aligned mask of
 * python/cleave/dynamic/reference.py:129-133 (query row r sees keys <= r + kv_len - q_len), the
 * mask of the paged and ragged prefill operators. head_dim 64 or 128. The workspace holds the status
 * word (cb200_workspace_status), the counter from which the kernel's persistent CTAs take their (head, query tile)
 * items (in the 256-byte header; it clears itself at the end of a launch, so the zero-fill before first use is
 * all the caller owes) and, with qk_norm, the normalised copy of K.
 * ---------------------------------------------------------------------------------------- */
typedef enum { CB200_SCORE_SOFTMAX = 0, CB200_SCORE_LINEAR = 1 } cb200_score_mode;

typedef struct {
  const void* q;   /* (num_qo_heads, q_len, head_dim) */
  const void* k;   /* (num_kv_heads, kv_len, head_dim) */
  const void* v;   /* (num_kv_heads, kv_len, head_dim) */
  void* out;       /* (num_qo_heads, q_len, head_dim) */
  float* lse;      /* (num_qo_heads, q_len) base 2, may be NULL */
  void* workspace;
  size_t workspace_bytes;
  int32_t num_qo_heads;
  int32_t num_kv_heads;
  int32_t q_len;
  int32_t kv_len;
  int32_t head_dim; /* 64 or 128 */
  int32_t dtype;    /* cb200_dtype */
  int32_t causal;   /* 0 = no mask, 1 = end-aligned causal mask (a row left without keys gives 0 and lse -inf) */
  float sm_scale;
  /* The fields below select two more operators of the same kernel; zero gives plain attention.
   * score_mode CB200_SCORE_LINEAR: O = (sm_scale * Q K^T) V without softmax - the operator
   *   (q @ k.mT) @ v of demo/matmul_matmul.py (sm_scale 1). The scores are rounded to the storage type
   *   before the second product, as a 16-bit tensor-core operand must be; lse is not written.
   * qk_norm 1: Q and K rows are RMS-normalised first, x * rsqrt(mean_d(x^2) + norm_eps) with fp32
   *   statistics - the operator of demo/qknorm.py. The query factor is taken from the resident query tile
   *   and folded into the score scale; K is normalised once by a pre-pass into the workspace, which
   *   then holds num_kv_heads * kv_len * head_dim * 2 more bytes (cb200_attn_prefill_workspace_bytes
   *   accounts for it). */
  int32_t score_mode; /* cb200_score_mode */
  int32_t qk_norm;
  float norm_eps;
} cb200_attn_prefill_args;

size_t cb200_attn_prefill_workspace_bytes(const cb200_attn_prefill_args* a);
int cb200_attn_prefill(const cb200_attn_prefill_args* a, void* stream);

/* Ragged and paged causal prefill: one (query range, key range) per request, token-major tensors.
 * Replaces gqa_ragged_prefill_causal_* (python/cleave/dynamic/paging/builders/ragged.py) and, with
 * kv_indices set, gqa_paged_prefill_causal_* (builders/prefill.py); argument order and meaning follow
 * python/cleave/dynamic/reference.py:204-278. A request with no query rows or no keys leaves its rows
 * of `out` zero and of `lse` -inf, as the reference's preallocation does; so does a row that the mask
 * leaves without keys. */
typedef struct {
  const void* q;             /* (total_q, num_qo_heads, head_dim) */
  const void* k;             /* ragged: (total_kv, num_kv_heads, head_dim); paged: cache (num_pages, 1, num_kv_heads, head_dim) */
  const void* v;             /* same shape as k */
  const int32_t* qo_indptr;  /* (batch + 1) device */
  const int32_t* kv_indptr;  /* (batch + 1) device: key offsets (ragged) or offsets into kv_indices (paged) */
  const int32_t* kv_indices; /* NULL = ragged; paged: page id of every key (one token per page), device */
  void* out;                 /* (total_q, num_qo_heads, head_dim) */
  float* lse;                /* (total_q, num_qo_heads) base 2, may be NULL */
  void* workspace;
  size_t workspace_bytes;
  int32_t batch;
  int32_t total_q;
  int32_t total_kv;          /* ragged: rows of k; paged: num_pages */
  int32_t num_qo_heads;
  int32_t num_kv_heads;
  int32_t head_dim; /* 64 or 128 */
  int32_t dtype;    /* cb200_dtype */
  int32_t causal;   /* 1 = end-aligned causal mask per request */
  float sm_scale;
  int32_t num_kv_indices; /* paged: entries of kv_indices; ranges of kv_indptr are clipped to it (0 = not stated, no clipping) */
} cb200_attn_prefill_ragged_args;

size_t cb200_attn_prefill_ragged_workspace_bytes(const cb200_attn_prefill_ragged_args* a);
int cb200_attn_prefill_ragged(const cb200_attn_prefill_ragged_args* a, void* stream);

/* ------------------------------------------------------------------------------------------
 * O = (Q K^T) V without softmax or scale; q (num_qo_heads, q_len, head_dim), k / v (num_kv_heads, kv_len,
 * head_dim), query head h uses kv head h / (HQ / HKV); head_dim 64 or 128. Replaces the fused kernel of
 * demo/matmul_matmul.py ((q @ k.mT) @ v). Two evaluation orders:
 *   CB200_MM_SCORES_FIRST  (Q K^T) V on the tcgen05 attention kernel (cb200_attn_prefill, linear scores);
 *   CB200_MM_CHAIN         Q (K^T V): T = K^T V (head_dim x head_dim per kv head, fp32 accumulation over
 *                          token chunks summed in a fixed order, stored in the storage dtype), then O = Q T.
 *                          2 (kv_len + g q_len) D^2 FLOPs per kv head instead of 4 g q_len kv_len D, every
 *                          input byte read once;
 *   CB200_MM_AUTO          the chain when it saves at least four times the FLOPs.
 * Both orders round one intermediate to the storage dtype (the scores, or T).
 * ---------------------------------------------------------------------------------------- */
typedef enum { CB200_MM_AUTO = 0, CB200_MM_SCORES_FIRST = 1, CB200_MM_CHAIN = 2 } cb200_mm_impl;

typedef struct {
  const void* q;
  const void* k;
  const void* v;
  void* out; /* (num_qo_heads, q_len, head_dim) */
  void* workspace;
  size_t workspace_bytes;
  int32_t num_qo_heads;
  int32_t num_kv_heads;
  int32_t q_len;
  int32_t kv_len;
  int32_t head_dim;
  int32_t dtype; /* cb200_dtype */
  int32_t impl;  /* cb200_mm_impl */
} cb200_matmul_matmul_args;

size_t cb200_matmul_matmul_workspace_bytes(const cb200_matmul_matmul_args* a);
/* 1 when the launch will use the chain order, 0 otherwise. */
int cb200_matmul_matmul_uses_chain(const cb200_matmul_matmul_args* a);
int cb200_matmul_matmul(const cb200_matmul_matmul_args* a, void* stream);

/* ------------------------------------------------------------------------------------------
 * Y = rowsum(X @ W): y[m] = sum_n (X @ W)[m, n]; X (m, k), W (k, n) row-major, y (m) = (m, 1); k and n
 * multiples of 8. Replaces the fused matmul + reduce kernel of demo/matmul_rowsum.py
 * ((x @ w).sum(-1, keepdim=True)). Computed as X @ (W 1): one pass over W for its fp32 row sums (k
 * floats in the workspace), one pass over X; the (m, n) product is never formed.
 * ---------------------------------------------------------------------------------------- */
typedef struct {
  const void* x; /* (m, k) */
  const void* w; /* (k, n) */
  void* y;       /* (m) */
  void* workspace;
  size_t workspace_bytes;
  int32_t m, n, k;
  int32_t dtype; /* cb200_dtype */
} cb200_matmul_rowsum_args;

size_t cb200_matmul_rowsum_workspace_bytes(const cb200_matmul_rowsum_args* a);
int cb200_matmul_rowsum(const cb200_matmul_rowsum_args* a, void* stream);

/* ------------------------------------------------------------------------------------------
 * LoRA: Y = X @ W + (X @ A) @ B; X (m, k), W (k, n), A (k, r), B (r, n), Y (m, n), all row-major in the
 * storage dtype; k, n and r multiples of 8. Replaces the fused kernel of demo/lora.py
 * (x @ w + (x @ a) @ b). Two launches of cb200_gemm on `stream`: T = X @ A (kept in the workspace in the
 * storage dtype), then Y = X @ W + T @ B as one product over the concatenated K (x2 / w2 of cb200_gemm_args),
 * launched so that it streams W while T is computed.
 * ---------------------------------------------------------------------------------------- */
typedef struct {
  const void* x; /* (m, k) */
  const void* w; /* (k, n) */
  const void* a; /* (k, r) */
  const void* b; /* (r, n) */
  void* y;       /* (m, n) */
  void* workspace;
  size_t workspace_bytes;
  int32_t m, n, k, r;
  int32_t dtype; /* cb200_dtype */
} cb200_lora_args;

size_t cb200_lora_workspace_bytes(const cb200_lora_args* a);
int cb200_lora(const cb200_lora_args* a, void* stream);

/* ------------------------------------------------------------------------------------------
 * Paged causal MLA prefill (absorbed latent), one token per page:
 *   S = (Q_nope CKV^T + Q_pe KPE^T) * scale under the end-aligned causal mask (query i of a request with q_len
 *   queries and kv_len keys sees keys <= i + kv_len - q_len), O = softmax(S) CKV, plus the base-2 log-sum-exp.
 * Rows without a visible key give 0 and -inf.
 *
 * Replaces tests/graph/handwritten/expected_kernels/mla_paged_prefill_causal_h16_ckv512_kpe64_ps1.py
 * (python/cleave/dynamic/paging/builders/mla.py:393); argument order and meaning follow
 * python/cleave/dynamic/reference.py:324-365. A query-tile kernel on tcgen05: 128 / num_heads consecutive query
 * tokens times their heads are the 128 rows of every MMA, so num_heads must divide 128. The workspace is the
 * 256-byte header: the status word (cb200_workspace_status) and, for batches of many short prompts, which run on
 * persistent CTAs, the counter their items are dealt from (it clears itself at the end of a launch; zero-fill the
 * workspace once before first use, as every workspace).
 * ---------------------------------------------------------------------------------------- */
typedef struct {
  const void* q_nope;    /* (total_q, num_heads, 512) */
  const void* q_pe;      /* (total_q, num_heads, 64) */
  const void* ckv_cache; /* (num_pages, 1, 512) */
  const void* kpe_cache; /* (num_pages, 1, 64) */
  const int32_t* qo_indptr;  /* (batch + 1) query-row offsets */
  const int32_t* kv_indptr;  /* (batch + 1) offsets into kv_indices */
  const int32_t* kv_indices; /* (num_kv_indices) page id per token */
  void* out;             /* (total_q, num_heads, 512) */
  float* lse;            /* (total_q, num_heads), may be NULL */
  void* workspace;
  size_t workspace_bytes;
  int32_t batch, total_q, num_heads, ckv_dim, kpe_dim, num_pages, num_kv_indices;
  int32_t dtype;         /* cb200_dtype */
  float sm_scale;
} cb200_mla_prefill_args;

size_t cb200_mla_prefill_workspace_bytes(const cb200_mla_prefill_args* a);
int cb200_mla_prefill(const cb200_mla_prefill_args* a, void* stream);

/* ------------------------------------------------------------------------------------------
 * The two-stage form of a split (compatibility with the reference's partial + combine kernel pairs; the
 * entry points above fuse the combine into the one launch and are what performance work should call).
 *
 * cb200_split_combine replaces the combine kernels
 *   tests/graph/handwritten/expected_kernels/matmul_splitk_combine.py   (Y = sum_s P[s])
 *   tests/graph/handwritten/expected_kernels/mha_split_combine.py       (O = sum_s O[s] / sum_s L[s], per row)
 * `num` is (outer, splits, inner) in the storage dtype, contiguous; `out` (outer, inner) receives the sum over
 * `splits` in fp32, rounded once. With `den` (den_outer rows of `splits` values, den_outer * den_inner = the
 * rows the quotient is taken over; den_inner is 1 for a per-row denominator) every sum is divided by the
 * matching denominator sum: element (o, i) by den row o (den_inner == 1) or by element (o, i) (den_inner ==
 * inner). No workspace.
 *
 * cb200_attn_unnormalise turns the normalised per-split results of cb200_attn_decode (out, base-2 lse) into
 * the partial results the reference's split partial kernels emit
 *   tests/graph/handwritten/expected_kernels/{gqa,mha,mqa}_split_partial.py:
 *   O[s] = sum_j exp(score_j + shift) v_j and L[s] = sum_j exp(score_j + shift) with the operator's fixed shift
 *   (demo/attention.py:5-8), i.e. O[s] = out * L[s], L[s] = 2^lse * e^shift. `out`, `lse` are laid out
 *   (kv_heads, splits, group) rows (the order cb200_attn_decode produces for a cache viewed as
 *   kv_heads * splits requests); o_part is (kv_heads * group, splits, head_dim), l_part (kv_heads * group, splits).
 * ---------------------------------------------------------------------------------------- */
typedef struct {
  const void* num;
  const void* den; /* may be NULL */
  void* out;
  int64_t outer, inner;
  int32_t splits;
  int32_t den_inner; /* 1 or inner; ignored without den */
  int32_t dtype;     /* cb200_dtype of num, den and out */
} cb200_split_combine_args;

int cb200_split_combine(const cb200_split_combine_args* a, void* stream);

typedef struct {
  const void* out;  /* (kv_heads * splits * group, head_dim), storage dtype */
  const float* lse; /* (kv_heads * splits * group), base 2 */
  void* o_part;     /* (kv_heads * group, splits, head_dim), storage dtype */
  void* l_part;     /* (kv_heads * group, splits), storage dtype */
  int32_t kv_heads, group, splits, head_dim;
  int32_t dtype;
  float shift; /* natural-log shift added to every score before exp (the demos use -50 / sqrt(d)) */
} cb200_attn_unnormalise_args;

int cb200_attn_unnormalise(const cb200_attn_unnormalise_args* a, void* stream);

/* ------------------------------------------------------------------------------------------
 * Decode attention for callers that cannot allocate device memory. (No counterpart in the
 * reference, whose wrappers always own a torch-allocated scratch buffer.)
 *
 * Who needs it: a host that runs inside someone else's memory plan - an inference server that
 * hands this library only the tensors it carved out of its own arena at start-up, a plugin
 * loaded by a runtime that forbids cudaMalloc after initialisation, or a process whose device
 * memory is fully committed to the KV cache. Such a caller has nowhere to get the split-KV
 * workspace from, so this variant keeps it inside the library: a 4 MiB array in the library's
 * device image (cb200_attn_decode_static_scratch_max_bytes()). Every GPU that loads the library
 * holds those 4 MiB until the process exits, whether or not this function is ever called.
 *
 * Same arguments and results as cb200_attn_decode; `workspace` / `workspace_bytes` are ignored.
 * The function calls no allocating routine. A problem whose scratch need
 * (cb200_attn_decode_workspace_bytes) exceeds the array is refused with CB200_ERR_SCRATCH_LIMIT;
 * on a 148-SM GPU that leaves room for about 430 000 (request, kv head) pairs.
 *
 * The first call on each device looks up the array's device address (one runtime query, with
 * that device current) and caches it; make that first call before starting any stream capture.
 * All calls on a device share the one array: each call clears the words it needs at zero on
 * `stream` before its kernel, and two calls that overlap on the GPU (different streams with no
 * ordering between them) race on it - keep them on one stream or order them with events.
 * ---------------------------------------------------------------------------------------- */
size_t cb200_attn_decode_static_scratch_max_bytes(void);
int cb200_attn_decode_static_scratch(const cb200_attn_decode_args* a, void* stream);
/* The status word of the built-in array after synchronising `stream` (the caller has no pointer to hand to
 * cb200_workspace_status): CB200_OK, or CB200_ERR_DEVICE_TIMEOUT if a bounded wait of the most recent call on
 * the current device gave up, in which case that call's outputs are not valid. Ask before the next call: every
 * call clears the word. Allocates nothing. */
int cb200_attn_decode_static_scratch_status(void* stream);

/* ------------------------------------------------------------------------------------------
 * The all-gather of an N-sharded GEMM for shapes whose product cb200_gemm does not send to the peers itself (the
 * y_peers fields need the CTA-pair kernel, m >= 256): the dense (m, n) block `src` of this GPU is copied to
 * `dsts[0 .. n_dst)` - element [0, first own column] of its own copy of the (m, ld_dst) result and of the peer GPUs'
 * copies (peer-mapped device pointers; `dsts` is a host array, n_dst <= 8). n and ld_dst multiples of 8, 16-bit
 * types. One kernel of plain stores on `stream`; nothing is signalled: put a barrier across the GPUs between this call
 * and the first read of the result. No counterpart in the reference (single-GPU).
 * ---------------------------------------------------------------------------------------- */
int cb200_peer_scatter_cols(const void* src, int m, int n, int ld_dst, void* const* dsts, int n_dst, int dtype,
                            void* stream);

/* ------------------------------------------------------------------------------------------
 * Causal prefill whose key window is far shorter than its run of query rows (a chunk with thousands of query tokens
 * and a page table of a few dozen entries: only the last min(q_len, kv_len) rows of a request see a key, all others
 * are 0 / -inf) is run by two light kernels - one CTA per row that sees a key, one warp per blind row - instead of
 * the tcgen05 kernels: cb200_attn_prefill_ragged (causal, ragged or paged) and cb200_mla_prefill take them when the
 * keys (num_kv_indices, or total_kv for ragged) number at most `tokens` (default 256) and the query rows at least
 * eight times the keys. 0 turns the kernels off. Returns the previous value. Process-wide and not synchronised:
 * set it before launching. No counterpart in the reference (its captured workloads are where such chunks come from:
 * python/cleave/dynamic/workloads.py).
 * ---------------------------------------------------------------------------------------- */
int cb200_set_small_problem_limit(int tokens);

#ifdef __cplusplus
}
#endif
#endif /* CLEAVE_B200_H */
