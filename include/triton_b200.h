/*
 * triton_b200 — C ABI of the B200 (sm_100a) kernel library.
 *
 * The reference (facebookexperimental/triton, TLX layer + triton_kernels) has no FFI: its
 * boundary is a set of Python functions that take torch tensors. Each entry point below is
 * what a ctypes/cffi binding for one of those functions calls; the comment on each names the
 * reference function it stands behind (path inside the reference project : line).
 *
 * Conventions
 *  - Plain pointers and sizes only. All data pointers are DEVICE pointers unless a name ends
 *    in `_host`. `stream` is a cudaStream_t passed as void* (NULL = default stream).
 *  - No entry point allocates device memory, creates streams or synchronises, except tb200_check
 *    and the set-up calls of the expert-parallel path (tb200_symm_alloc / _free / _open / _close).
 *    Outputs and workspaces are caller-owned. A few entry points take a HOST array of device
 *    pointers (one per rank); their comments say so.
 *  - Return value: 0 (TB200_OK) or a negative TB200_ERR_* code. Nothing throws.
 *  - Launches are asynchronous on `stream`. Device-side waits are bounded; a wait that gives
 *    up records a code in a per-device status word that tb200_check() reads and clears.
 *  - Thread safety: calls on different streams may be issued from different host threads.
 */
#ifndef TRITON_B200_H_
#define TRITON_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  TB200_OK = 0,
  TB200_ERR_BAD_ARG = -1,
  TB200_ERR_UNSUPPORTED = -2,
  TB200_ERR_CUDA = -3,
  TB200_ERR_TIMEOUT = -4,
  TB200_ERR_TMAP = -5,
  TB200_ERR_TOO_LARGE = -6
};

/* element types */
enum {
  TB200_BF16 = 0,
  TB200_F16 = 1,
  TB200_F32 = 2,
  TB200_E4M3 = 3,
  TB200_E5M2 = 4
};

/* ---------------------------------------------------------------- library ---------- */

int tb200_version(void);
const char* tb200_error_string(int code);
/* Synchronises `stream`, returns TB200_ERR_TIMEOUT if any kernel launched on this device
 * since the last check abandoned a wait (and clears the flag), else TB200_OK. */
int tb200_check(void* stream);
/* Raw status word of the current device without clearing it: 0, or (wait_code<<16)|block. */
int tb200_last_status_code(void);
/*
 * Self-test of the bounded-wait path (no counterpart in the reference, whose waits are unbounded
 * mbarrier.try_wait loops): launches one block whose thread 0 waits, with the wait routine every
 * kernel here uses, on an mbarrier that nothing completes, for at most limit_ns nanoseconds
 * (1 .. 1e9). When the limit runs out the thread records wait code 9 in the status word and the
 * block returns; no copy or MMA is in flight and nothing faults. After it, tb200_check() returns
 * TB200_ERR_TIMEOUT once and TB200_OK from then on. completed: optional device int that receives
 * 1 if the wait completed (it cannot) or 0 if it was abandoned.
 */
int tb200_selftest_wait(uint64_t limit_ns, int* completed, void* stream);

/* ---------------------------------------------------------------- dense GEMM ------- */

/*
 * C[M,N] = A[M,K] * B[K,N], fp32 accumulation in tensor memory.
 * Stands behind: third_party/tlx/tutorials/blackwell_gemm_ws.py:1486  matmul(a, b, config=None)
 *   (kernel matmul_kernel_tma_ws_blackwell :1168, split-K reduction _reduce_k_kernel :1098)
 * and, with dtype TB200_E4M3 and scale pointers, behind
 *   third_party/tlx/tutorials/blackwell_scaled_mm_ws.py:392  blackwell_scaled_mm_ws(..., scale_mode="tensorwise" | "rowwise").
 *
 * a_k_major = 1: A stored [M,K] with K contiguous (row-major), lda = elements between rows.
 * a_k_major = 0: A stored [K,M] with M contiguous (column-major A), lda = elements between k rows.
 * b_k_major = 1: B stored [N,K] with K contiguous (the reference's "B supplied transposed").
 * b_k_major = 0: B stored [K,N] with N contiguous (row-major B), ldb = elements between k rows.
 * 8-bit dtypes require both operands K-major.
 * Leading dimensions in bytes and base addresses must be multiples of 16.
 *
 * split_k: 0 = let the library choose, 1 = none, >1 = that many K partitions (clamped so that
 *   every partition is non-empty). When the effective value is >1, `workspace` must hold
 *   split_k*M*N floats (tb200_gemm_workspace_bytes gives the size for the choice the library
 *   would make); partial sums are kept in fp32 and reduced by a second kernel.
 * scale_a / scale_b: optional device pointers to one float each; the result is multiplied by
 *   (*scale_a)*(*scale_b) before the cast. NULL = 1.
 * out_dtype: TB200_BF16 or TB200_F16 (or TB200_F32).
 */
typedef struct {
  const void* a;
  const void* b;
  void* c;
  int64_t m, n, k;
  int64_t lda, ldb, ldc;
  int32_t in_dtype;
  int32_t out_dtype;
  int32_t a_k_major;
  int32_t b_k_major;
  int32_t split_k;
  int32_t block_n; /* 0 = choose; 64, 128 or 256 = one CTA per 128 x block_n tile; 512 = CTA pair per 256 x 256 tile; 1024 = CTA pair per 256 x 512 tile */
  void* workspace;
  size_t workspace_bytes;
  const float* scale_a;
  const float* scale_b;
  int32_t scale_mode; /* 0: scale_a / scale_b point to one float each (tensorwise); 1: rowwise, scale_a is float[M] (per row of A), scale_b float[N] (per row of B): C[m,n] = acc * scale_a[m] * scale_b[n] */
  int32_t reserved;
} tb200_gemm_args;

int tb200_gemm(const tb200_gemm_args* args, void* stream);
/* Bytes of workspace tb200_gemm needs for these args (0 when no split-K is used). */
size_t tb200_gemm_workspace_bytes(const tb200_gemm_args* args);
/* The tiling tb200_gemm takes for these args (no launch): out6 = {tile rows, tile columns, CTAs per tile (1 or 2),
 * split_k, ring stages, K elements per stage}. Stands behind get_heuristic_config,
 * third_party/tlx/tutorials/blackwell_gemm_ws.py:25-335 (which returns the reference kernel's config dict). */
int tb200_gemm_plan(const tb200_gemm_args* args, int32_t* out6);

/* ---------------------------------------------------------------- MXFP8 GEMM ------- */

/*
 * C[M,N] (bf16) = dq(A) * dq(B)^T with A [M,K] and B [N,K] contiguous float8_e4m3fn and one e8m0
 * scale per 1x32 block along K (value = element * 2^(scale - 127)), fp32 accumulation.
 * Stands behind: third_party/tlx/tutorials/blackwell_gemm_ws_mxfp8.py:1135
 *   matmul(a, b, a_scale, b_scale, config=None)   (kernel _gemm_mxfp8_ws_kernel :759).
 * a_scale / b_scale: rows*K/32 bytes each in the Blackwell 512-byte-atom order the reference
 *   reshapes to [1, rows/128, K/128, 2, 256] (:1038-1041): atom (row/128, k/128), byte
 *   (row%32)*16 + (row/32%4)*4 + (k/32)%4.
 * M, N and K must be multiples of 128 (as the reference asserts, :1167-1168); all four input
 * pointers 16-byte aligned. block_n: 0 = choose; 128 or 256 = one CTA per 128 x block_n tile;
 * 512 = CTA pair per 256 x 256 tile.
 */
typedef struct {
  const void* a;
  const void* b;
  const void* a_scale;
  const void* b_scale;
  void* c;
  int64_t m, n, k;
  int64_t ldc;
  int32_t block_n;
  int32_t reserved;
} tb200_gemm_mxfp8_args;

int tb200_gemm_mxfp8(const tb200_gemm_mxfp8_args* args, void* stream);

/*
 * Block-wise scaled FP8 GEMM: C[m,n] = sum over 128-wide K groups g of
 *   (A[m, g] . B[n, g]) * scale_a[m, g] * scale_b[n / 128, g].
 * Stands behind: third_party/tlx/tutorials/blackwell_scaled_mm_ws.py:392
 *   blackwell_scaled_mm_ws(a, b, scale_a, scale_b, ..., scale_mode="blockwise")  (promotion :300-341).
 * a [M, K], b [N, K] fp8 row-major (in_dtype TB200_E4M3 or TB200_E5M2); K % 128 == 0, N % 128 == 0;
 * scale_a: float, M-major ([K/128][M] in memory: element (m, g) at g * M + m);
 * scale_b: float [N/128][K/128] row-major; c [M, N] with row pitch ldc, out_dtype TB200_BF16, _F16 or _F32.
 */
typedef struct {
  const void* a;
  const void* b;
  void* c;
  const float* scale_a;
  const float* scale_b;
  int64_t m, n, k;
  int64_t ldc;
  int32_t in_dtype;
  int32_t out_dtype;
} tb200_gemm_fp8_blockwise_args;

int tb200_gemm_fp8_blockwise(const tb200_gemm_fp8_blockwise_args* args, void* stream);

/* ---------------------------------------------------------------- attention -------- */

/*
 * Flash-attention forward: o = softmax(q k^T * sm_scale [+ causal mask]) v, and optionally
 * lse[b,h,i] = log2(sum_j exp(s_ij)) with s the scaled (masked) scores, i.e. the reference's
 * M = m*sm_scale*log2(e) + log2(l).
 * Stands behind: third_party/tlx/tutorials/blackwell_fa_ws_pipelined_persistent.py:3491
 *   attention(q, k, v, sm_scale, causal, config=None)   (kernel _attn_fwd_ws :600, forward :3288).
 * q, o: [batch, heads, seq_q, head_dim] contiguous; k, v: [batch, heads, seq_kv, head_dim]
 * contiguous; dtype TB200_BF16 or TB200_F16; head_dim 64, 128 or 256; lse (may be NULL):
 * float [batch, heads, seq_q]. causal requires seq_q == seq_kv (as in the reference).
 * Any sequence length >= 1 is accepted (the tail is masked). Base pointers 16-byte aligned.
 */
typedef struct {
  const void* q;
  const void* k;
  const void* v;
  void* o;
  float* lse;
  int64_t batch, heads, seq_q, seq_kv;
  int32_t head_dim;
  int32_t dtype;
  int32_t causal;
  float sm_scale;
} tb200_attention_args;

int tb200_attention_fwd(const tb200_attention_args* args, void* stream);

/*
 * MXFP8 flash-attention forward: o = softmax(dq(q) dq(k)^T * sm_scale [+ causal mask]) dq(v) as bf16, with q, k, v
 * in e4m3 and one e8m0 scale per 32 values: q and k scaled along head_dim, v along the sequence (its transpose
 * [head_dim, seq] was quantised along seq); the probabilities are quantised inside the kernel (e4m3, one e8m0
 * scale per 32 keys of a row). lse as in tb200_attention_fwd (may be NULL).
 * Stands behind: third_party/tlx/tutorials/blackwell_fa_ws_pipelined_persistent_mxfp8.py:3374
 *   attention(q, k, v, q_scale, k_scale, v_scale, sm_scale, causal, config=None)   (kernel _attn_fwd_mxf8_ws :532).
 * q: [batch, heads, seq_q, 128] e4m3 contiguous; k, v: [batch, heads, seq_kv, 128]; o: bf16 [batch, heads, seq_q, 128].
 * Scales: uint8 e8m0 in 512-byte atoms [row % 32][row / 32 % 4][block % 4] (the "swizzled" / to_blocked order the
 * reference feeds its kernel, viewed there as [batch*heads, blocks, 1, 2, 256]):
 *   q_scale: [batch*heads][seq_q / 128] atoms, rows = the 128 query rows, blocks = the 4 groups of 32 along head_dim;
 *   k_scale: [batch*heads][seq_kv / 128] atoms, the same for the key rows;
 *   v_scale: [batch*heads][seq_kv / 128] atoms, rows = the 128 head-dim columns, blocks = the 4 groups of 32 keys.
 * head_dim 128; seq_q and seq_kv multiples of 128; causal requires seq_q == seq_kv. Pointers 16-byte aligned.
 */
typedef struct {
  const void* q;
  const void* k;
  const void* v;
  const void* q_scale;
  const void* k_scale;
  const void* v_scale;
  void* o;
  float* lse;
  int64_t batch, heads, seq_q, seq_kv;
  int32_t head_dim;
  int32_t causal;
  float sm_scale;
  int32_t reserved0;
} tb200_attention_mxfp8_args;

int tb200_attention_mxfp8_fwd(const tb200_attention_mxfp8_args* args, void* stream);

/*
 * Flash-attention backward: dq, dk, dv from q, k, v, the forward output o, its gradient d_o and
 * the base-2 log-sum-exp `lse` written by tb200_attention_fwd.
 * Stands behind: third_party/tlx/tutorials/blackwell_fa_ws_pipelined_persistent.py:3362
 *   _attention.backward (kernels _attn_bwd_preprocess :1252, _attn_bwd_ws :2442,
 *   _attn_bwd_dq_postprocess :1269).
 * Layouts as in the forward call; d_o and dq are shaped like q, dk and dv like k; all gradients are
 * written in `dtype` (the reference returns dq in fp32). head_dim 128 only. causal requires
 * seq_q == seq_kv. `workspace` (device memory, 16-byte aligned, at least
 * tb200_attention_bwd_workspace_bytes(args) bytes) holds the row sums of o * d_o and the fp32 dq
 * accumulator. Partial dq tiles of different key blocks are summed with floating-point atomics:
 * the last bits of dq can differ between two runs on the same inputs (as with the reference's
 * reduce-add); dk and dv are reproducible.
 */
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
  void* workspace;
  size_t workspace_bytes;
  int64_t batch, heads, seq_q, seq_kv;
  int32_t head_dim;
  int32_t dtype;
  int32_t causal;
  float sm_scale;
} tb200_attention_bwd_args;

size_t tb200_attention_bwd_workspace_bytes(const tb200_attention_bwd_args* args);
int tb200_attention_bwd(const tb200_attention_bwd_args* args, void* stream);

/* ---------------------------------------------------------------- MoE routing ------ */
/* Paths below are inside python/triton_kernels/triton_kernels/ of the reference. */

/*
 * Per-row top-k over n_cols expert logits.
 * Stands behind: topk.py:106 topk(x, k, apply_softmax=True, dim=1, y_indx=None, n_rows=None, ...)
 *   (kernel _topk_forward, topk_details/_topk_forward.py:87-147; torch twin topk_torch topk.py:144).
 * Selection: k largest per row, ties to the smaller column; values in descending order; softmax
 * (fp32) over the k selected values when apply_softmax. Rows in [n_rows, rows_alloc) get index -1,
 * values x[row, :k] and no mask bits, as the torch twin does.
 * x: [rows_alloc, n_cols] of dtype (F32/BF16/F16), row stride stride_x elements.
 * y_vals: same dtype [rows_alloc, k]; y_indx: int16 [rows_alloc, k]; both with row stride stride_y.
 * bitmatrix: uint32 words; word w of row r lives at r*bits_stride_row + w*bits_stride_word
 *   (the reference stores it transposed: bits_stride_row = 1).
 * use_provided_indx: y_indx is an input (values are gathered, the mask is built from it); a provided
 *   index outside [0, n_cols) is treated as "none": value 0, no mask bit.
 * n_cols <= 1024, k <= 32.
 */
typedef struct {
  const void* x;
  void* y_vals;
  void* y_indx;
  void* bitmatrix;
  int64_t rows_alloc, n_rows, n_cols;
  int64_t stride_x, stride_y;
  int64_t bits_stride_row, bits_stride_word;
  int32_t k;
  int32_t dtype;
  int32_t apply_softmax;
  int32_t use_provided_indx;
} tb200_topk_args;
int tb200_topk(const tb200_topk_args* args, void* stream);

/*
 * Expert histogram and the two index permutations of the routing bitmatrix.
 * Stands behind: tensor_details/bitmatrix.py:110 make_bitmatrix_metadata(nonzero_indx, bitmatrix)
 *   (torch twin make_bitmatrix_metadata_torch :157).
 * indx: [n_entries] expert index per (token, slot) in row-major order, int16 or int32, -1 = none.
 * col_sum int32[n_cols]; col_sorted_indx int32[n_entries]: entry ids grouped by expert, stable
 * ("combine" order); row_sorted_indx int32[n_entries]: position of each entry in that order
 * ("dispatch"); unused tail entries are -1. workspace: tb200_bitmatrix_metadata_workspace_bytes().
 */
typedef struct {
  const void* indx;
  int32_t* col_sum;
  int32_t* col_sorted_indx;
  int32_t* row_sorted_indx;
  void* workspace;
  size_t workspace_bytes;
  int64_t n_entries;
  int32_t n_cols;
  int32_t indx_is_int16;
} tb200_bitmatrix_metadata_args;
int tb200_bitmatrix_metadata(const tb200_bitmatrix_metadata_args* args, void* stream);
size_t tb200_bitmatrix_metadata_workspace_bytes(int64_t n_entries, int32_t n_cols);

/*
 * Same result as tb200_bitmatrix_metadata, but without a workspace argument: the scratch lives in
 * a fixed device array inside the library (about 1 MiB per GPU, resident until exit). This entry
 * point has no counterpart in the reference; it exists for callers that cannot allocate device
 * memory at call time and have none to lend — processes that freeze their GPU memory plan at
 * start-up, or runtimes that forbid cudaMalloc (a device-wide stall) on the request path.
 * Limit: ceil(n_entries / 1024) * n_cols + n_cols <= 263168 words (e.g. 262144 entries x 1024
 * columns = 263168, exactly the limit; or 61440 entries x 4096 columns = 249856); beyond that the
 * call returns TB200_ERR_TOO_LARGE and launches nothing. n_entries == 0 is accepted (col_sum is
 * zeroed). The first call on each device looks up the array's device address (make that call
 * outside stream capture); the address is cached per device ordinal and does not survive a
 * cudaDeviceReset of that device. Calls on the same GPU share the array: run them on one stream or
 * order them yourself — kernels of two calls that overlap in time corrupt each other's scratch.
 * No call here allocates or frees memory.
 */
int tb200_bitmatrix_metadata_static(const void* indx, int32_t indx_is_int16, int64_t n_entries, int32_t n_cols,
                                    int32_t* col_sum, int32_t* col_sorted_indx, int32_t* row_sorted_indx,
                                    void* stream);

/*
 * Ragged-tensor metadata for block sizes 16, 32, 64, 128.
 * Stands behind: tensor_details/ragged_tensor.py:183 make_ragged_tensor_metadata(slice_sizes, n_total_rows)
 *   (torch twin make_ragged_tensor_metadata_torch :217).
 * slice_offs int32[n_slices+1]; block_offs int32[4, n_slices+1]; block_schedule int32[4, max_n_blocks]
 * with entries (block_in_slice << 16) | slice, -1 padded. max_n_blocks is the caller's bound
 * (RaggedTensorMetadata.max_n_blocks, :79-81).
 */
typedef struct {
  const int32_t* slice_sizes;
  int32_t* slice_offs;
  int32_t* block_offs;
  int32_t* block_schedule;
  int32_t n_slices;
  int32_t max_n_blocks;
} tb200_ragged_metadata_args;
int tb200_ragged_metadata(const tb200_ragged_metadata_args* args, void* stream);

/*
 * Metadata of the ragged tensor that keeps slice i iff slice_map[i] != -1, renumbered to slice_map[i]; dropped
 * entries are compacted to the end as -1 and block_offs[s][number of kept slices] holds the number of kept
 * schedule entries. The expert-parallel layer uses it to turn the global metadata into that of a rank's experts.
 * Stands behind: tensor_details/ragged_tensor.py:348 remap_ragged_tensor_metadata(metadata, slice_map)
 *   (torch twin remap_ragged_tensor_metadata_torch :388-433). All arrays int32, shaped as in
 * tb200_ragged_metadata_args; the outputs must not alias the inputs.
 */
typedef struct {
  const int32_t* slice_sizes;
  const int32_t* slice_offs;
  const int32_t* block_offs;
  const int32_t* block_schedule;
  const int32_t* slice_map;
  int32_t* out_slice_sizes;
  int32_t* out_slice_offs;
  int32_t* out_block_offs;
  int32_t* out_block_schedule;
  int32_t n_slices;
  int32_t max_n_blocks;
} tb200_remap_ragged_metadata_args;
int tb200_remap_ragged_metadata(const tb200_remap_ragged_metadata_args* args, void* stream);

/*
 * y[t, :] = sum over the k slots of x[t, j, :] (optionally masked / scaled per (t, j)), fp32 sum.
 * Stands behind: reduce.py:1135 reduce(x, dim, mask=None, scale=None, ...) for the MoE combine
 *   `reduce(y.view(-1, k, d), dim=1)` (torch twin reduce_torch :1173).
 * x: [n_tokens, k, d] contiguous BF16/F16, d % 8 == 0; mask: uint8 [n_tokens, k] or NULL;
 * scale: float [n_tokens, k] or NULL; y: [n_tokens, d].
 */
typedef struct {
  const void* x;
  const uint8_t* mask;
  const float* scale;
  void* y;
  int64_t n_tokens;
  int64_t d;
  int32_t k;
  int32_t dtype;
  const int32_t* row_indx; /* optional int32 [n_tokens*k]: slot (t, j) reads row row_indx[t*k+j] of x (< 0 or >= x_rows = skip) */
  int64_t x_rows;          /* rows of x when row_indx is given; 0 = n_tokens * k */
} tb200_reduce_k_args;
int tb200_reduce_k(const tb200_reduce_k_args* args, void* stream);

/*
 * Row gather (scatter = 0: dst[i] = src[indx[i]]) or scatter (scatter = 1: dst[indx[i]] = src[i]) of
 * rows of row_bytes bytes (multiple of 16; pitches and bases 16-byte aligned). indexed_rows is the
 * number of rows of the indexed side (src when gathering, dst when scattering): an index outside
 * [0, indexed_rows) skips the row, so a corrupt index never becomes an out-of-bounds access.
 * Stands behind the local row moves around the expert-parallel exchange,
 * distributed.py:176-283 (convert_dp_to_ep / convert_ep_to_dp store rows at indexed positions).
 */
int tb200_move_rows(const void* src, int64_t src_pitch_bytes, void* dst, int64_t dst_pitch_bytes,
                    const int32_t* indx, int64_t n_indx, int64_t row_bytes, int32_t scatter, int64_t indexed_rows,
                    void* stream);

/* ---------------------------------------------------------------- expert-parallel exchange -------- */

/*
 * Symmetric buffers: every rank (one process per GPU) allocates one buffer of the same size, exports a
 * 64-byte CUDA IPC handle, exchanges the handles by any host-side means (the Python mirror uses
 * torch.distributed.all_gather) and opens its peers' handles; it then holds a device pointer to every
 * rank's buffer. Stands behind SymmetricMemoryPool._initialize, distributed_details/mesh.py:118-136
 * (symm_mem.empty + rendezvous in the reference). These five calls are set-up / tear-down: they are the
 * only calls of the library that allocate, free or synchronise the device.
 */
int tb200_symm_alloc(size_t bytes, void** ptr);              /* cudaMalloc + zero fill */
int tb200_symm_free(void* ptr);
int tb200_symm_export(const void* ptr, uint8_t* handle64);   /* handle of a tb200_symm_alloc buffer */
int tb200_symm_open(const uint8_t* handle64, void** peer_ptr);   /* maps a peer's buffer, enables peer access */
int tb200_symm_close(void* peer_ptr);

/*
 * Cross-GPU barrier on `stream` (hdl.barrier(channel) in the reference, mesh.py:130-136): one small kernel
 * in which rank r stores its next epoch into flag r of every rank's signal block (st.release.sys) and waits
 * until all `world` flags of its own block carry that epoch (ld.acquire.sys). signal_peers: HOST array of
 * `world` device pointers, entry j = the signal block of this channel inside rank j's symmetric buffer
 * (320 zero-initialised bytes, 16-byte aligned: uint32 flags[16] at byte 0, the owner's epoch at byte 256).
 * All ranks must call it the same number of times. Writes a rank made before the barrier (peer stores
 * included) are visible to kernels the others launch after it. The wait is bounded by limit_ns
 * (<= 30 s): when a peer does not arrive the kernel records wait code 10 and returns; tb200_check()
 * then reports TB200_ERR_TIMEOUT. Each rank must run on its own GPU.
 */
int tb200_symm_barrier(void* const* signal_peers, int32_t rank, int32_t world, uint64_t limit_ns, void* stream);

/*
 * Stores `bytes` (a multiple of 16, 16-byte aligned) of local memory to dst_peers[r] for every rank r: one rank's
 * part of an all-gather through symmetric buffers (dst_peers[r] = this rank's slot inside rank r's buffer). The
 * expert-parallel layer publishes its local top-k values and indices this way (topk(..., all_gather=True) in
 * the reference, topk.py:41-69, writes them into symmetric memory too). Follow with tb200_symm_barrier.
 */
int tb200_symm_put(const void* src, size_t bytes, void* const* dst_peers, int32_t world, void* stream);

/*
 * DP -> EP dispatch: for every local token t and slot j with expert e = expt_indx[token_offset + t, j] >= 0,
 * copies x[t, :] to row dispatch_indx[(token_offset + t) * k + j] of the buffer of rank expt_owner[e].
 * Stands behind _convert_dp_to_ep, distributed.py:136-173 (host convert_dp_to_ep :176-211).
 * expt_indx: GLOBAL [n_tokens_global, k] int16 or int32; dispatch_indx: global row_sorted_indx;
 * expt_owner: int32 [n_experts]; dst_peers: HOST array of `world` device pointers, each a
 * [dst_rows, row_bytes] buffer with pitch dst_pitch_bytes. Rows of 16-byte multiples, 16-byte aligned.
 */
typedef struct {
  const void* x;
  int64_t x_pitch_bytes;
  const void* expt_indx;
  const int32_t* dispatch_indx;
  const int32_t* expt_owner;
  void* const* dst_peers;
  int64_t dst_pitch_bytes;
  int64_t dst_rows;
  int64_t row_bytes;
  int64_t n_tokens_local;
  int64_t token_offset;
  int32_t k;
  int32_t n_experts;
  int32_t world;
  int32_t indx_is_int16;
} tb200_ep_dispatch_args;
int tb200_ep_dispatch(const tb200_ep_dispatch_args* args, void* stream);

/*
 * EP -> DP combine: for every expert-sorted row r whose entry = combine_indx[r] belongs to an expert this
 * rank owns, copies src[r, :] to row (entry % rows_per_rank) of the buffer of rank entry / rows_per_rank
 * (rows_per_rank = n_tokens_local * k). Stands behind _convert_ep_to_dp, distributed.py:217-254 (host
 * convert_ep_to_dp :257-283). tb200_moe_gemm does the same from its epilogue when given y_peers.
 */
typedef struct {
  const void* src;
  int64_t src_pitch_bytes;
  const void* expt_indx;
  const int32_t* combine_indx;
  const int32_t* expt_owner;
  void* const* dst_peers;
  int64_t dst_pitch_bytes;
  int64_t row_bytes;
  int64_t n_rows;
  int64_t rows_per_rank;
  int32_t n_experts;
  int32_t world;
  int32_t rank;
  int32_t indx_is_int16;
} tb200_ep_combine_args;
int tb200_ep_combine(const tb200_ep_combine_args* args, void* stream);

/*
 * dst[i] = src[indx[i]] when 0 <= indx[i] < src_rows, else a row of zeros: the rows tb200_moe_gemm would read through
 * gather_indx, written out in sorted order. For many rows the grouped GEMM is faster on rows gathered by this pass
 * (tiled TMA loads of A) than with its in-kernel gather (measured on the 16384-token MoE layer: 3.29 ms against
 * 3.90 ms); the host mirror of matmul.py:243 does so from 2048 sorted rows on. Same alignment rules as tb200_move_rows.
 * Stands behind the X.gather loads of python/triton_kernels/triton_kernels/matmul_details/_p_matmul.py.
 */
int tb200_gather_rows(const void* src, int64_t src_pitch_bytes, int64_t src_rows, void* dst, int64_t dst_pitch_bytes,
                      const int32_t* indx, int64_t n_indx, int64_t row_bytes, void* stream);

/*
 * out[r, j] = g * sigmoid(alpha * g) * (l + 1), g = a[r, 2j] (clamped to <= limit),
 * l = a[r, 2j+1] (clamped to [-limit, limit]) when has_limit.
 * Stands behind: swiglu.py swiglu(a, alpha, precision_config) (torch twin swiglu_torch :89-100).
 */
typedef struct {
  const void* a;
  void* out;
  int64_t rows, n_in;
  int64_t lda, ldo;
  float alpha, limit;
  int32_t has_limit;
  int32_t dtype;
} tb200_swiglu_args;
int tb200_swiglu(const tb200_swiglu_args* args, void* stream);

/* ---------------------------------------------------------------- MoE grouped GEMM - */

/*
 * Per-expert GEMM over expert-sorted rows with fused gather / bias / SwiGLU / gate scale / scatter:
 *   for r in [slice_offs[e], slice_offs[e+1]):
 *     acc = x[gather_indx[r], :] @ w[e] (+ bias[e]);  if swiglu: acc = swiglu(acc) (N -> N/2 columns)
 *     y[scatter_indx[r], :] = acc * gammas[r]          (scatter_indx[r] == -1: row dropped)
 * Stands behind: python/triton_kernels/triton_kernels/matmul.py:243
 *   matmul(a, b, bias, a_ragged_metadata, ..., gather_indx, scatter_indx, ..., gammas, ..., fused_activation)
 *   (kernel _p_matmul, matmul_details/_p_matmul.py:62; torch twin matmul_torch matmul.py:823).
 * x: [rows_x, k] row-major (ldx elements between rows), BF16/F16.
 * w: n_experts matrices, w_n_major = 1: [E, K, N] with N contiguous; 0: [E, N, K] with K contiguous.
 * bias: float [E, N] or NULL. gammas: float [R] or NULL. gather_indx / scatter_indx: int32 [R] or
 * NULL (identity). slice_offs: int32 [E+1]; block_schedule: the 128-row schedule of the ragged
 * metadata, int32 [n_sched], entries (block << 16) | expert or -1.
 * y: [rows_y, N or N/2], ldy elements between rows; rows that no sorted row maps to are untouched.
 * k % 8 == 0, ldx % 8 == 0 (and n % 8 == 0 when w_n_major); n even when swiglu.
 */
typedef struct {
  const void* x;
  const void* w;
  const float* bias;
  void* y;
  const int32_t* slice_offs;
  const int32_t* block_schedule;
  const int32_t* gather_indx;
  const int32_t* scatter_indx;
  const float* gammas;
  int64_t n_experts, k, n;
  int64_t rows_x, rows_y;
  int64_t ldx, ldy;
  int32_t n_sched;
  int32_t w_n_major;
  int32_t dtype;
  int32_t swiglu;
  float swiglu_alpha;
  float swiglu_limit;
  int32_t swiglu_has_limit;
  int32_t moe_tile_mode; /* 0 = choose; 1 = one CTA per 128-row block; 2 = CTA pair per two consecutive blocks */
  const int32_t* slice_sizes; /* optional int32 [E]: rows of expert e (needed for remapped metadata, whose slice_offs are not cumulative); NULL = slice_offs[e+1] - slice_offs[e] */
  /* Fused expert-parallel combine (the reference's fused-comm epilogue, matmul_details/_p_matmul.py:755-782):
   * with y_world > 0, y is ignored and the output row with index i (scatter_indx[r], or r) is stored to row
   * i % rows_per_peer of y_peers[i / rows_per_peer]; y_peers is a HOST array of y_world device pointers
   * (buffers of this and of other GPUs as tb200_symm_open maps them), each [rows_per_peer, N] with pitch ldy.
   * Plain stores; follow the call with tb200_symm_barrier before any rank reads its buffer. */
  void* const* y_peers;
  int64_t rows_per_peer;
  int32_t y_world;
  int32_t gammas_by_out_row; /* 1: the scale of sorted row r is gammas[i] with i its output index (scatter_indx[r], or r)
                                instead of gammas[r]: lets the top-k values [tokens, k] serve as gate weights as they are */
  /* Remaining epilogue terms of matmul.py:245-256, applied in the reference's order (_p_matmul.py:606-622):
   * acc = (acc + bias[e] * betas[r]) * out_alpha -> activation -> * gammas[r] -> + c_acc_in[row]. */
  const float* betas;     /* optional float [R]: per sorted row factor on the bias */
  const void* c_acc_in;   /* optional [rows_y, N or N/2] matrix of the output dtype added to the result (may be y itself);
                             not with scatter_indx or y_peers */
  int64_t ld_acc_in;      /* elements between rows of c_acc_in */
  float out_alpha;
  int32_t has_out_alpha;
  /* MX-quantised output (precision_config.c_mx_scale with the quantize_mxfp8 epilogue, matmul.py:362-366 and
   * matmul_details/_p_matmul.py:650-704): with y_mx_scale set, y is a matrix of y_mx_dtype (TB200_E4M3 /
   * TB200_E5M2; ldy in bytes), every 32 consecutive outputs of a row share the e8m0 scale
   * 2^ceil(log2(amax / max_finite)) written to y_mx_scale[row][col / 32] (ld_y_mx_scale bytes between rows) and the
   * values are output / scale rounded to nearest even. Not with c_acc_in or y_peers. */
  void* y_mx_scale;
  int64_t ld_y_mx_scale;
  int32_t y_mx_dtype;
  int32_t reserved0;
} tb200_moe_gemm_args;
int tb200_moe_gemm(const tb200_moe_gemm_args* args, void* stream);

/*
 * The same grouped GEMM with FP8 activations and MXFP4 weights (the configuration the reference's MoE
 * benchmark sweeps on Blackwell: x "fp8", w "mx4"):
 *     acc = x_scale * x[r, :] @ dequant(w[e]) (+ bias[e]);  swiglu / gammas / scatter as above.
 * Stands behind: python/triton_kernels/triton_kernels/matmul.py:243 called with an FP4 weight and
 *   PrecisionConfig(weight_scale=...) (weights prepared as in bench/bench_mlp.py:36-57).
 * x: [rows_x, k] TB200_E4M3 or TB200_E5M2, row-major (ldx bytes between rows, multiple of 16), rows sorted
 *    by expert (no gather index); x_scale: one float or NULL (1).
 * w: uint8, two e2m1 values per byte along K (even index in the low nibble), blocked as
 *    [E][ceil(N/256)][ceil(K/128)][256][64]: block (e, t, s) holds rows 256 t .. 256 t + 255 of expert e (zero
 *    rows past N) and values 128 s .. 128 s + 127 of each (zero codes past K); 32-byte aligned.
 * w_scale: uint8 e8m0, one per 32 values of K, per expert in 512-byte atoms
 *    [E][ceil(N/128)][ceil(K/128)][n%32][n/32%4][k/32%4]   (the layout tb200_gemm_mxfp8 uses for its scales; 127 past
 *    N and K).
 * k % 32 == 0 (whole scale blocks); n is free. Output TB200_BF16, TB200_F16, or TB200_E4M3 / TB200_E5M2 (round to nearest even,
 * saturating to the largest finite value: the conversion of the reference's kernels when the output tensor is
 * fp8, which is what matmul.py:243 allocates for fp8 activations unless precision_config.out_dtype says otherwise).
 * ldy in elements of the output type. Other fields as in tb200_moe_gemm_args.
 */
typedef struct {
  const void* x;
  const void* w;
  const void* w_scale;
  const float* x_scale;
  const float* bias;
  void* y;
  const int32_t* slice_offs;
  const int32_t* slice_sizes;
  const int32_t* block_schedule;
  const int32_t* scatter_indx;
  const float* gammas;
  int64_t n_experts, k, n;
  int64_t rows_x, rows_y;
  int64_t ldx, ldy;
  int32_t n_sched;
  int32_t x_dtype;
  int32_t out_dtype;
  int32_t swiglu;
  float swiglu_alpha;
  float swiglu_limit;
  int32_t swiglu_has_limit;
  int32_t block_rows; /* rows per entry of block_schedule: 0 or 128 = the 128-row schedule; 32 = the 32-row schedule (few rows per expert: operand roles swapped, weights on the MMA's M side) */
  /* MX-scaled activations (precision_config.a_mx_scale, matmul.py:309-334): uint8 e8m0, one per 32 values of K,
   * [rows_x][k/32] row-major with ld_x_mx_scale bytes between rows (multiple of 4, pointer 4-byte aligned);
   * NULL = the activations carry no block scales. */
  const void* x_mx_scale;
  int64_t ld_x_mx_scale;
  /* MX-quantised output (precision_config.c_mx_scale with the quantize_mxfp8 epilogue, matmul.py:362-366 and
   * matmul_details/_p_matmul.py:650-704): out_dtype TB200_E4M3 / TB200_E5M2, every 32 consecutive outputs of a
   * row share the e8m0 scale 2^ceil(log2(amax / max_finite)) written to y_mx_scale[row][col / 32]
   * (ld_y_mx_scale bytes between rows), values = round-to-nearest-even of output / scale. Not with swiglu on
   * the 32-row schedule (TB200_ERR_UNSUPPORTED: use the 128-row schedule). NULL = plain output. */
  void* y_mx_scale;
  int64_t ld_y_mx_scale;
  /* Flexpoint (precision_config.flex_ctx, matmul.py:116-121; numerics_details/flexpoint.py:133-188): device
   * scalars. w_flex_scale multiplies every accumulator like x_scale (rhs_data.scale; x_scale is lhs_data.scale).
   * y_expected_scale: the finished output is divided by it before the conversion (out_data.expected_scale),
   * clamped to the finite range of the output type first when flexpoint_saturate_inf is set.
   * y_actual_scale: max |output| * (1 / max_finite(output type)) + 1e-30 is folded in with an atomic max
   * (out_data.actual_scale; the caller zeroes it before the call). Ignored for an MX-quantised output. */
  const float* w_flex_scale;
  const float* y_expected_scale;
  float* y_actual_scale;
  int32_t flexpoint_saturate_inf;
  /* FP8 weights (the reference's float8 x float8 and float8 / mxfloat8 x mxfloat8 cases, tests/test_matmul.py:150,
   * 193,214,254): w_dtype TB200_E4M3 or TB200_E5M2 makes w a byte matrix [E][N][K] with K contiguous (16-byte
   * aligned, k % 16 == 0; n and k need not be multiples of 128). w_scale is then optional: NULL for plain fp8 weights
   * (their tensor-wide scale goes in w_flex_scale), or the e8m0 atoms described above with ceil(N/128) and ceil(K/128)
   * atoms per expert (bytes past N or K: 127) for MXFP8 weights; with x_mx_scale, ld_x_mx_scale >= 4 ceil(K/128).
   * The 128-row schedule only. 0 = packed MXFP4 weights as described above. */
  int32_t w_dtype;
} tb200_moe_gemm_mx4_args;
int tb200_moe_gemm_mx4(const tb200_moe_gemm_mx4_args* args, void* stream);

/*
 * Upcast of an MXFP4 weight (the blocked layout above) to a 16-bit matrix out[E][N][K], K contiguous - the
 * operand tb200_moe_gemm takes with w_n_major = 0. With 16-bit activations the reference multiplies by an
 * MXFP4 weight through tl.dot_scaled(x, None, "bf16", w, w_scales, "e2m1")
 * (python/triton_kernels/triton_kernels/matmul_details/_matmul.py:485-489), i.e. the weight upcast to bf16 and
 * the ordinary 16-bit MMA; this pass followed by tb200_moe_gemm is that product. Element values follow
 * numerics_details/mxfp.py upcast_from_mxfp_torch: e2m1 value * float(scale << 23), clamped to the finite range
 * of the output type, NaN kept.
 * w, w_scale: as in tb200_moe_gemm_mx4_args. out: n_experts * n * k elements of TB200_BF16 / TB200_F16,
 * 16-byte aligned. k % 128 == 0, n % 128 == 0.
 */
typedef struct {
  const void* w;
  const void* w_scale;
  void* out;
  int64_t n_experts, k, n;
  int32_t out_dtype;
} tb200_mxfp4_upcast_args;
int tb200_mxfp4_upcast(const tb200_mxfp4_upcast_args* args, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TRITON_B200_H_ */
