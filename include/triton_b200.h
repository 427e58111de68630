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
 *  - No entry point allocates device memory, creates streams or synchronises (except
 *    tb200_check and the *_host convenience calls). Outputs and workspaces are caller-owned.
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

/* ---------------------------------------------------------------- dense GEMM ------- */

/*
 * C[M,N] = A[M,K] * B[K,N], fp32 accumulation in tensor memory.
 * Stands behind: third_party/tlx/tutorials/blackwell_gemm_ws.py:1486  matmul(a, b, config=None)
 *   (kernel matmul_kernel_tma_ws_blackwell :1168, split-K reduction _reduce_k_kernel :1098)
 * and, with dtype TB200_E4M3 and scale pointers, behind
 *   third_party/tlx/tutorials/blackwell_scaled_mm_ws.py:392  blackwell_scaled_mm_ws(..., scale_mode="tensorwise").
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
  int32_t block_n; /* 0 = choose; 64, 128 or 256 = one CTA per 128 x block_n tile; 512 = CTA pair per 256 x 256 tile */
  void* workspace;
  size_t workspace_bytes;
  const float* scale_a;
  const float* scale_b;
} tb200_gemm_args;

int tb200_gemm(const tb200_gemm_args* args, void* stream);
/* Bytes of workspace tb200_gemm needs for these args (0 when no split-K is used). */
size_t tb200_gemm_workspace_bytes(const tb200_gemm_args* args);

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
 * pointers 16-byte aligned. block_n: 0 = choose, else 128 or 256.
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

/* ---------------------------------------------------------------- attention -------- */

/*
 * Flash-attention forward: o = softmax(q k^T * sm_scale [+ causal mask]) v, and optionally
 * lse[b,h,i] = log2(sum_j exp(s_ij)) with s the scaled (masked) scores, i.e. the reference's
 * M = m*sm_scale*log2(e) + log2(l).
 * Stands behind: third_party/tlx/tutorials/blackwell_fa_ws_pipelined_persistent.py:3491
 *   attention(q, k, v, sm_scale, causal, config=None)   (kernel _attn_fwd_ws :600, forward :3288).
 * q, o: [batch, heads, seq_q, head_dim] contiguous; k, v: [batch, heads, seq_kv, head_dim]
 * contiguous; dtype TB200_BF16 or TB200_F16; head_dim 64 or 128; lse (may be NULL):
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

#ifdef __cplusplus
}
#endif
#endif /* TRITON_B200_H_ */
