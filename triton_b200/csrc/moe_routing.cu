// MoE routing and combine kernels (integer index work, bit-exact against the reference's torch
// twins) plus the small elementwise kernels around the grouped GEMM.
//
//   topk_kernel               per-row top-k with softmax over the k values, int16 expert indices and
//                             the (row x expert) bitmatrix          <- _topk_forward, topk_details/_topk_forward.py:87-147
//   bitmatrix metadata (x3)   expert histogram, stable expert-sorted order ("combine" indices) and
//                             its inverse ("dispatch" indices)      <- sum_bitmatrix_rows + _bitmatrix_metadata_compute_stage1/2,
//                                                                      tensor_details/bitmatrix.py:43-150
//   ragged_metadata_kernel    slice offsets, per-block-size block offsets and block schedule
//                                                                   <- _ragged_tensor_metadata_memset/_compute, tensor_details/ragged_tensor.py:128-210
//   reduce_k_kernel           sum over the k expert slots of each token (optional mask / scale)
//                                                                   <- _reduce_forward, reduce.py:497-655
//   swiglu_kernel             standalone interleaved SwiGLU          <- _swiglu, swiglu_details/_swiglu.py:73-120
// (paths are inside python/triton_kernels/triton_kernels/ of the reference).
// These are HBM- or launch-bound integer/elementwise kernels: plain coalesced loads, no tensor cores.
#include <string.h>

#include <mutex>

#include "common.cuh"
#include "host_common.h"

namespace tb200 {

// ------------------------------------------------------------------------------------ top-k

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }

// One warp per row. Lane l holds columns l, l+32, ... (CPL of them). k rounds of "largest value,
// ties to the smaller column" give the selection already sorted the way the reference sorts it.
template <typename T, int CPL>
__global__ void topk_kernel(const T* __restrict__ x, long long stride_x, int rows_alloc, int n_rows, int n_cols, int k,
                            int apply_softmax, T* __restrict__ y_vals, int16_t* __restrict__ y_indx, long long stride_y,
                            uint32_t* __restrict__ bits, long long bits_stride_row, long long bits_stride_word,
                            int n_words, int use_provided_indx) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= rows_alloc) return;
  const int row = warp;
  const T* xr = x + (long long)row * stride_x;
  if (row >= n_rows) {
    // rows past the valid count: indices -1, values copied through, no mask bits
    for (int j = lane; j < k; j += 32) {
      y_vals[(long long)row * stride_y + j] = xr[j];
      if (!use_provided_indx) y_indx[(long long)row * stride_y + j] = -1;
    }
    if (lane < n_words) bits[(long long)row * bits_stride_row + lane * bits_stride_word] = 0u;
    return;
  }
  float v[CPL];
  bool taken[CPL];
#pragma unroll
  for (int i = 0; i < CPL; ++i) {
    const int c = lane + 32 * i;
    v[i] = c < n_cols ? to_f32<T>(xr[c]) : -INFINITY;
    taken[i] = c >= n_cols;
  }
  float my_val = 0.f;  // lane j keeps the j-th selected value / index (k <= 32)
  int my_idx = -1;
  if (use_provided_indx) {
    if (lane < k) {
      my_idx = y_indx[(long long)row * stride_y + lane];
      if (my_idx < 0 || my_idx >= n_cols) my_idx = -1;  // outside the row: no value, no mask bit
      my_val = my_idx >= 0 ? to_f32<T>(xr[my_idx]) : 0.f;
    }
  } else {
    for (int j = 0; j < k; ++j) {
      float best = -INFINITY;
      int best_c = 0x7fffffff;
#pragma unroll
      for (int i = 0; i < CPL; ++i) {
        const int c = lane + 32 * i;
        if (!taken[i] && (v[i] > best || (v[i] == best && c < best_c) || best_c == 0x7fffffff)) {
          best = v[i];
          best_c = c;
        }
      }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, off);
        const int oc = __shfl_xor_sync(0xffffffffu, best_c, off);
        if (oc != 0x7fffffff && (best_c == 0x7fffffff || ob > best || (ob == best && oc < best_c))) {
          best = ob;
          best_c = oc;
        }
      }
#pragma unroll
      for (int i = 0; i < CPL; ++i)
        if (lane + 32 * i == best_c) taken[i] = true;
      if (lane == j) {
        my_val = best;
        my_idx = best_c == 0x7fffffff ? -1 : best_c;
      }
    }
  }
  float out = my_val;
  if (apply_softmax) {
    float mx = lane < k ? my_val : -INFINITY;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    float e = lane < k ? expf(my_val - mx) : 0.f;
    float sum = e;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
    out = e / sum;
  }
  if (lane < k) {
    y_vals[(long long)row * stride_y + lane] = from_f32<T>(out);
    if (!use_provided_indx) y_indx[(long long)row * stride_y + lane] = (int16_t)my_idx;
  }
  uint32_t word = 0u;
  for (int j = 0; j < k; ++j) {
    const int idx = __shfl_sync(0xffffffffu, my_idx, j);
    if (idx >= 0 && (idx >> 5) == lane) word |= 1u << (idx & 31);
  }
  if (lane < n_words) bits[(long long)row * bits_stride_row + lane * bits_stride_word] = word;
}

// ------------------------------------------------------------------------- bitmatrix metadata

static constexpr int BM_BLOCK = 1024;  // entries per block

__device__ __forceinline__ int load_indx(const void* indx, int is16, long long i) {
  return is16 ? (int)reinterpret_cast<const int16_t*>(indx)[i] : reinterpret_cast<const int32_t*>(indx)[i];
}

// partial[b][c] = number of entries of block b that name column c
__global__ void bm_hist_kernel(const void* __restrict__ indx, int is16, long long n, int n_cols,
                               int* __restrict__ partial) {
  extern __shared__ int hist[];
  for (int c = threadIdx.x; c < n_cols; c += blockDim.x) hist[c] = 0;
  __syncthreads();
  const long long i = (long long)blockIdx.x * BM_BLOCK + threadIdx.x;
  if (i < n) {
    const int e = load_indx(indx, is16, i);
    if (e >= 0 && e < n_cols) atomicAdd(&hist[e], 1);
  }
  __syncthreads();
  for (int c = threadIdx.x; c < n_cols; c += blockDim.x) partial[(long long)blockIdx.x * n_cols + c] = hist[c];
}

// partial -> exclusive prefix over blocks; col_sum; col_offs = exclusive scan of col_sum.
// One block. A warp owns a column at a time: its lanes take 32 blocks per step and scan them with shuffles (a
// thread per column walking all blocks one after the other took 22 us for 64 blocks x 128 columns: every step is a
// dependent global load); warp 0 then scans the column sums the same way.
__global__ void bm_scan_kernel(int* __restrict__ partial, int n_blocks, int n_cols, int* __restrict__ col_sum,
                               int* __restrict__ col_offs) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  for (int c = warp; c < n_cols; c += nwarps) {
    int carry = 0;
    for (int b0 = 0; b0 < n_blocks; b0 += 32) {
      const int b = b0 + lane;
      const int v = b < n_blocks ? partial[(long long)b * n_cols + c] : 0;
      int incl = v;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += t;
      }
      if (b < n_blocks) partial[(long long)b * n_cols + c] = carry + incl - v;
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) col_sum[c] = carry;
  }
  __syncthreads();
  if (warp == 0) {
    int carry = 0;
    for (int c0 = 0; c0 < n_cols; c0 += 32) {
      const int c = c0 + lane;
      const int v = c < n_cols ? col_sum[c] : 0;
      int incl = v;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += t;
      }
      if (c < n_cols) col_offs[c] = carry + incl - v;
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
  }
}

// position of entry i in column-sorted order = col_offs[e] + (entries of column e before i)
__global__ void bm_rank_kernel(const void* __restrict__ indx, int is16, long long n, int n_cols,
                               const int* __restrict__ partial, const int* __restrict__ col_offs,
                               int* __restrict__ col_sorted, int* __restrict__ row_sorted) {
  extern __shared__ int counter[];
  for (int c = threadIdx.x; c < n_cols; c += blockDim.x) counter[c] = 0;
  __syncthreads();
  const long long i = (long long)blockIdx.x * BM_BLOCK + threadIdx.x;
  int e = -1;
  if (i < n) {
    e = load_indx(indx, is16, i);
    if (e >= n_cols) e = -1;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned peers = __match_any_sync(0xffffffffu, e);
  const int lane_rank = __popc(peers & ((1u << lane) - 1u));
  const int leader = __ffs(peers) - 1;
  int base = 0;
  for (int w = 0; w < BM_BLOCK / 32; ++w) {
    if (warp == w && e >= 0) {
      base = counter[e];
      __syncwarp(peers);
      if (lane == leader) counter[e] = base + __popc(peers);
    }
    __syncthreads();
  }
  if (e >= 0) {
    const int pos = col_offs[e] + partial[(long long)blockIdx.x * n_cols + e] + base + lane_rank;
    row_sorted[i] = pos;
    col_sorted[pos] = (int)i;
  }
}

// The same two steps for up to BM_SMALL_COLS columns (the expert counts of MoE layers), shaped for latency: the routing
// chain runs on every rank of an expert-parallel layer whatever the number of ranks. The scan spreads its columns
// over blocks (a warp per column); the rank kernel derives the column offsets from the column sums itself, counts
// per warp with match.any and prefixes the 32 warps' counts per column - three block barriers instead of one per
// warp - and also writes the -1 entries the caller would otherwise have to memset (rows that name no column, the
// tail of the column-sorted list).
static constexpr int BM_SMALL_COLS = 256;

__global__ void bm_scan_cols_kernel(int* __restrict__ partial, int n_blocks, int n_cols, int* __restrict__ col_sum) {
  const int lane = threadIdx.x & 31;
  const int c = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (c >= n_cols) return;
  int carry = 0;
  for (int b0 = 0; b0 < n_blocks; b0 += 32) {
    const int b = b0 + lane;
    const int v = b < n_blocks ? partial[(long long)b * n_cols + c] : 0;
    int incl = v;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off) incl += t;
    }
    if (b < n_blocks) partial[(long long)b * n_cols + c] = carry + incl - v;
    carry += __shfl_sync(0xffffffffu, incl, 31);
  }
  if (lane == 0) col_sum[c] = carry;
}

__global__ void bm_rank_small_kernel(const void* __restrict__ indx, int is16, long long n, int n_cols,
                                     const int* __restrict__ partial, const int* __restrict__ col_sum,
                                     int* __restrict__ col_sorted, int* __restrict__ row_sorted) {
  extern __shared__ int sm[];
  int* offs = sm;                  // [n_cols] exclusive scan of col_sum
  int* wc = sm + n_cols;           // [32][n_cols] per-warp counts, then their exclusive prefix over the warps
  __shared__ int warp_tot[BM_SMALL_COLS / 32];
  __shared__ int total_sh;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int j = threadIdx.x; j < 32 * n_cols; j += blockDim.x) wc[j] = 0;
  int v = 0, incl = 0;
  if (threadIdx.x < BM_SMALL_COLS) {
    v = threadIdx.x < n_cols ? col_sum[threadIdx.x] : 0;
    incl = v;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off) incl += t;
    }
    if (lane == 31) warp_tot[warp] = incl;
  }
  __syncthreads();
  if (threadIdx.x < BM_SMALL_COLS) {
    int base = 0;
    for (int w = 0; w < warp; ++w) base += warp_tot[w];
    if (threadIdx.x < n_cols) offs[threadIdx.x] = base + incl - v;
    if (threadIdx.x == BM_SMALL_COLS - 1) total_sh = base + incl;
  }
  const long long i = (long long)blockIdx.x * BM_BLOCK + threadIdx.x;
  int e = -1;
  if (i < n) {
    e = load_indx(indx, is16, i);
    if (e >= n_cols) e = -1;
  }
  const unsigned peers = __match_any_sync(0xffffffffu, e);
  const int lane_rank = __popc(peers & ((1u << lane) - 1u));
  if (e >= 0 && lane == __ffs(peers) - 1) wc[warp * n_cols + e] = __popc(peers);
  __syncthreads();
  if (threadIdx.x < n_cols) {
    int running = 0;
    for (int w = 0; w < 32; ++w) {
      const int t = wc[w * n_cols + threadIdx.x];
      wc[w * n_cols + threadIdx.x] = running;
      running += t;
    }
  }
  __syncthreads();
  if (i < n) {
    if (e >= 0) {
      const int pos = offs[e] + partial[(long long)blockIdx.x * n_cols + e] + wc[warp * n_cols + e] + lane_rank;
      row_sorted[i] = pos;
      col_sorted[pos] = (int)i;
    } else {
      row_sorted[i] = -1;
    }
  }
  if (blockIdx.x == 0)  // positions no entry maps to
    for (long long j = total_sh + threadIdx.x; j < n; j += blockDim.x) col_sorted[j] = -1;
}

// --------------------------------------------------------------------------- ragged metadata

// blockIdx.x == 0: slice_offs; blockIdx.x = 1 + s: block_offs[s] and block_schedule[s] for block
// size 16 << s. One thread block each; experts are walked in chunks of blockDim.x with a carry.
__global__ void ragged_metadata_kernel(const int* __restrict__ slice_sizes, int n_slices, int max_n_blocks,
                                       int* __restrict__ slice_offs, int* __restrict__ block_offs,
                                       int* __restrict__ block_schedule) {
  __shared__ int warp_sums[32];
  __shared__ int carry_s;
  const int which = blockIdx.x;
  const int log2bs = 4 + (which - 1);
  int* offs = which == 0 ? slice_offs : block_offs + (long long)(which - 1) * (n_slices + 1);
  int* sched = which == 0 ? nullptr : block_schedule + (long long)(which - 1) * max_n_blocks;
  if (threadIdx.x == 0) carry_s = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  for (int base = 0; base < n_slices; base += blockDim.x) {
    const int e = base + threadIdx.x;
    const int sz = e < n_slices ? slice_sizes[e] : 0;
    const int val = which == 0 ? sz : ((sz + (1 << log2bs) - 1) >> log2bs);
    int incl = val;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off) incl += t;
    }
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    int wprefix = 0;
    for (int w = 0; w < warp; ++w) wprefix += warp_sums[w];
    const int carry = carry_s;
    const int excl = carry + wprefix + incl - val;
    if (e < n_slices) {
      offs[e] = excl;
      if (sched) {
        for (int blk = 0; blk < val; ++blk)
          if (excl + blk < max_n_blocks) sched[excl + blk] = (blk << 16) | e;
      }
    }
    __syncthreads();
    if (threadIdx.x == blockDim.x - 1) carry_s = excl + val;
    __syncthreads();
    (void)nwarps;
  }
  if (threadIdx.x == 0) offs[n_slices] = carry_s;
}

// ---------------------------------------------------------------------- ragged metadata remap

// Stable compaction by a whole thread block: out[0..count) = val(i) for the i in [0, n) with keep(i), in order;
// out[count..out_len) = -1. Returns count to every thread. `scratch` holds 33 ints of shared memory.
template <typename KeepFn, typename ValFn>
__device__ int block_compact(int n, KeepFn keep, ValFn val, int* __restrict__ out, int out_len, int* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  __syncthreads();
  if (threadIdx.x == 0) scratch[32] = 0;
  __syncthreads();
  for (int base = 0; base < n; base += blockDim.x) {
    const int i = base + threadIdx.x;
    const bool k = i < n && keep(i);
    const unsigned ballot = __ballot_sync(0xffffffffu, k);
    if (lane == 0) scratch[warp] = __popc(ballot);
    __syncthreads();
    int before = scratch[32];
    for (int w = 0; w < warp; ++w) before += scratch[w];
    if (k) {
      const int pos = before + __popc(ballot & ((1u << lane) - 1u));
      if (pos < out_len) out[pos] = val(i);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int tot = scratch[32];
      for (int w = 0; w < nwarps; ++w) tot += scratch[w];
      scratch[32] = tot;
    }
    __syncthreads();
  }
  const int count = scratch[32];
  for (int j = count + threadIdx.x; j < out_len; j += blockDim.x) out[j] = -1;
  return count;
}

// Metadata of the ragged tensor that keeps slice i iff slice_map[i] != -1, renumbered to slice_map[i]
// (remap_ragged_tensor_metadata, tensor_details/ragged_tensor.py:348-381; torch twin :388-433). Block 0 compacts
// slice_sizes and slice_offs; block 1 + s compacts block_offs[s] and block_schedule[s], rewrites the slice id of
// every kept schedule entry and stores the number of kept entries behind the kept block offsets.
__global__ void remap_ragged_metadata_kernel(const int* __restrict__ slice_sizes, const int* __restrict__ slice_offs,
                                             const int* __restrict__ block_offs, const int* __restrict__ sched,
                                             const int* __restrict__ slice_map, int n_slices, int max_n_blocks,
                                             int* __restrict__ o_sizes, int* __restrict__ o_offs,
                                             int* __restrict__ o_block_offs, int* __restrict__ o_sched) {
  __shared__ int scratch[33];
  auto keep_slice = [&](int i) { return slice_map[i] != -1; };
  if (blockIdx.x == 0) {
    block_compact(n_slices, keep_slice, [&](int i) { return slice_sizes[i]; }, o_sizes, n_slices, scratch);
    block_compact(n_slices, keep_slice, [&](int i) { return slice_offs[i]; }, o_offs, n_slices + 1, scratch);
    return;
  }
  const int s = blockIdx.x - 1;
  const int* bo = block_offs + (long long)s * (n_slices + 1);
  const int* sc = sched + (long long)s * max_n_blocks;
  int* obo = o_block_offs + (long long)s * (n_slices + 1);
  int* osc = o_sched + (long long)s * max_n_blocks;
  const int n_keep = block_compact(n_slices, keep_slice, [&](int i) { return bo[i]; }, obo, n_slices + 1, scratch);
  const int n_sched = block_compact(
      max_n_blocks,
      [&](int i) {
        const int id = sc[i] & 0xFFFF;
        return id != 0xFFFF && id < n_slices && slice_map[id] != -1;
      },
      [&](int i) { return (int)((unsigned)sc[i] & 0xFFFF0000u) | slice_map[sc[i] & 0xFFFF]; }, osc, max_n_blocks,
      scratch);
  __syncthreads();
  if (threadIdx.x == 0) obo[n_keep] = n_sched;
}

// ------------------------------------------------------------------------------- k-way reduce

// y[t, d] = sum_j (mask[t, j] ? x[row(t, j), d] * scale[t, j] : 0), fp32 accumulation, 8 columns per
// thread; row(t, j) = row_indx[t*k + j] when an index is given (negative = skip), else t*k + j.
template <typename T>
__global__ void reduce_k_kernel(const T* __restrict__ x, const uint8_t* __restrict__ mask,
                                const float* __restrict__ scale, const int* __restrict__ row_indx,
                                T* __restrict__ y, long long n_tok, int k, int d, long long x_rows) {
  const int d8 = d >> 3;
  const long long total = n_tok * d8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / d8;
    const int c = (int)(i - t * d8) << 3;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < k; ++j) {
      if (mask && !mask[t * k + j]) continue;
      const float s = scale ? scale[t * k + j] : 1.f;
      long long row = t * k + j;
      if (row_indx) {
        row = row_indx[row];
        if (row < 0 || row >= x_rows) continue;
      }
      const uint4 raw = *reinterpret_cast<const uint4*>(x + (row * (long long)d + c));
      const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int u = 0; u < 8; ++u) acc[u] += to_f32<T>(e[u]) * s;
    }
    uint4 out;
    T* o = reinterpret_cast<T*>(&out);
#pragma unroll
    for (int u = 0; u < 8; ++u) o[u] = from_f32<T>(acc[u]);
    *reinterpret_cast<uint4*>(y + (t * (long long)d + c)) = out;
  }
}

// ---------------------------------------------------------------------------------- row mover

// gather: dst[i] = src[indx[i]];  scatter: dst[indx[i]] = src[i];  an index outside [0, indexed_rows)
// skips the row. One warp per row, 16 bytes per lane per step.
__global__ void move_rows_kernel(const uint8_t* __restrict__ src, long long src_pitch, uint8_t* __restrict__ dst,
                                 long long dst_pitch, const int* __restrict__ indx, long long n, int row_bytes,
                                 int scatter, long long indexed_rows) {
  const long long warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long i = warp; i < n; i += nwarps) {
    const int j = indx[i];
    if (j < 0 || j >= indexed_rows) continue;
    const uint8_t* s = src + (scatter ? i : (long long)j) * src_pitch;
    uint8_t* d = dst + (scatter ? (long long)j : i) * dst_pitch;
    for (int b = lane * 16; b < row_bytes; b += 512) *reinterpret_cast<uint4*>(d + b) = *reinterpret_cast<const uint4*>(s + b);
  }
}

// dst[i] = src[indx[i]] for 0 <= indx[i] < src_rows, else a row of zeros (what the grouped GEMM's own gather reads
// for such an index). One warp per row, two 16-byte copies per lane in flight.
__global__ void gather_rows_kernel(const uint8_t* __restrict__ src, long long src_pitch, int src_rows,
                                   uint8_t* __restrict__ dst, long long dst_pitch, const int* __restrict__ indx,
                                   long long n, int row_bytes) {
  const long long warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long i = warp; i < n; i += nwarps) {
    const int j = __ldg(indx + i);
    const bool valid = j >= 0 && j < src_rows;
    const uint8_t* s = src + (long long)(valid ? j : 0) * src_pitch;
    uint8_t* d = dst + i * dst_pitch;
    for (int b = lane * 16; b < row_bytes; b += 1024) {
      const bool second = b + 512 < row_bytes;
      uint4 v0 = make_uint4(0, 0, 0, 0), v1 = make_uint4(0, 0, 0, 0);
      if (valid) {
        v0 = __ldg(reinterpret_cast<const uint4*>(s + b));
        if (second) v1 = __ldg(reinterpret_cast<const uint4*>(s + b + 512));
      }
      *reinterpret_cast<uint4*>(d + b) = v0;
      if (second) *reinterpret_cast<uint4*>(d + b + 512) = v1;
    }
  }
}

// ------------------------------------------------------------------------------------ swiglu

__device__ __forceinline__ float swiglu_f(float g, float l, float alpha, float limit, int has_limit) {
  if (has_limit) {
    g = fminf(g, limit);
    l = fminf(fmaxf(l, -limit), limit);
  }
  return g / (1.f + __expf(-alpha * g)) * (l + 1.f);
}

template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ a, T* __restrict__ out, long long rows, int n_out, long long lda,
                              long long ldo, float alpha, float limit, int has_limit) {
  const long long total = rows * n_out;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / n_out;
    const int c = (int)(i - r * n_out);
    const float g = to_f32<T>(a[r * lda + 2 * c]);
    const float l = to_f32<T>(a[r * lda + 2 * c + 1]);
    out[r * ldo + c] = from_f32<T>(swiglu_f(g, l, alpha, limit, has_limit));
  }
}

template <typename T>
static int launch_topk(const tb200_topk_args* a, cudaStream_t stream) {
  const int n_words = (int)((a->n_cols + 31) / 32);
  const int cpl = (int)((a->n_cols + 31) / 32);
  const int threads = 256;
  const long long warps = a->rows_alloc;
  const int blocks = (int)((warps * 32 + threads - 1) / threads);
#define TB200_TOPK_CASE(C)                                                                                     \
  topk_kernel<T, C><<<blocks, threads, 0, stream>>>(                                                           \
      static_cast<const T*>(a->x), a->stride_x, (int)a->rows_alloc, (int)a->n_rows, (int)a->n_cols, a->k,      \
      a->apply_softmax, static_cast<T*>(a->y_vals), static_cast<int16_t*>(a->y_indx), a->stride_y,             \
      static_cast<uint32_t*>(a->bitmatrix), a->bits_stride_row, a->bits_stride_word, n_words, a->use_provided_indx)
  if (cpl <= 1) TB200_TOPK_CASE(1);
  else if (cpl <= 2) TB200_TOPK_CASE(2);
  else if (cpl <= 4) TB200_TOPK_CASE(4);
  else if (cpl <= 8) TB200_TOPK_CASE(8);
  else if (cpl <= 16) TB200_TOPK_CASE(16);
  else TB200_TOPK_CASE(32);
#undef TB200_TOPK_CASE
  return cuda_err(cudaGetLastError());
}

}  // namespace tb200

using namespace tb200;

extern "C" int tb200_topk(const tb200_topk_args* a, void* stream_) {
  if (!a || !a->x || !a->y_vals || !a->y_indx || !a->bitmatrix) return TB200_ERR_BAD_ARG;
  if (a->rows_alloc < 0 || a->n_rows < 0 || a->n_rows > a->rows_alloc) return TB200_ERR_BAD_ARG;
  if (a->n_cols <= 0 || a->n_cols > 1024 || a->k <= 0 || a->k > 32 || a->k > a->n_cols) return TB200_ERR_UNSUPPORTED;
  if (a->rows_alloc == 0) return TB200_OK;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  switch (a->dtype) {
    case TB200_F32: return launch_topk<float>(a, stream);
    case TB200_BF16: return launch_topk<__nv_bfloat16>(a, stream);
    case TB200_F16: return launch_topk<__half>(a, stream);
    default: return TB200_ERR_UNSUPPORTED;
  }
}

extern "C" size_t tb200_bitmatrix_metadata_workspace_bytes(int64_t n_entries, int32_t n_cols) {
  if (n_entries < 0 || n_cols <= 0) return 0;
  const long long n_blocks = (n_entries + BM_BLOCK - 1) / BM_BLOCK;
  return (size_t)(n_blocks * n_cols + n_cols) * sizeof(int);
}

namespace tb200 {
// Shared by the allocating-caller and the fixed-scratch entry points.
int bitmatrix_metadata_launch(const void* indx, int is16, long long n, int n_cols, int* col_sum, int* col_sorted,
                              int* row_sorted, int* scratch, cudaStream_t stream) {
  const int n_blocks = (int)((n + BM_BLOCK - 1) / BM_BLOCK);
  int* partial = scratch;
  int* col_offs = scratch + (long long)n_blocks * n_cols;
  if (n_cols <= BM_SMALL_COLS) {
    if (n_blocks > 0) bm_hist_kernel<<<n_blocks, BM_BLOCK, n_cols * sizeof(int), stream>>>(indx, is16, n, n_cols, partial);
    bm_scan_cols_kernel<<<(n_cols + 7) / 8, 256, 0, stream>>>(partial, n_blocks, n_cols, col_sum);
    if (n_blocks > 0)
      bm_rank_small_kernel<<<n_blocks, BM_BLOCK, 33 * n_cols * sizeof(int), stream>>>(indx, is16, n, n_cols, partial, col_sum,
                                                                                    col_sorted, row_sorted);
    return cuda_err(cudaGetLastError());
  }
  if (n > 0) {
    cudaError_t e = cudaMemsetAsync(col_sorted, 0xFF, (size_t)n * sizeof(int), stream);
    if (e != cudaSuccess) return TB200_ERR_CUDA;
    e = cudaMemsetAsync(row_sorted, 0xFF, (size_t)n * sizeof(int), stream);
    if (e != cudaSuccess) return TB200_ERR_CUDA;
  }
  if (n_blocks > 0) bm_hist_kernel<<<n_blocks, BM_BLOCK, n_cols * sizeof(int), stream>>>(indx, is16, n, n_cols, partial);
  bm_scan_kernel<<<1, 1024, 0, stream>>>(partial, n_blocks, n_cols, col_sum, col_offs);
  if (n_blocks > 0)
    bm_rank_kernel<<<n_blocks, BM_BLOCK, n_cols * sizeof(int), stream>>>(indx, is16, n, n_cols, partial, col_offs,
                                                                        col_sorted, row_sorted);
  return cuda_err(cudaGetLastError());
}
}  // namespace tb200

extern "C" int tb200_bitmatrix_metadata(const tb200_bitmatrix_metadata_args* a, void* stream_) {
  if (!a || !a->col_sum || (a->n_entries > 0 && (!a->indx || !a->col_sorted_indx || !a->row_sorted_indx)))
    return TB200_ERR_BAD_ARG;
  if (a->n_entries < 0 || a->n_cols <= 0 || a->n_cols > 8192) return TB200_ERR_UNSUPPORTED;
  if (a->n_entries > INT32_MAX) return TB200_ERR_UNSUPPORTED;
  const size_t need = tb200_bitmatrix_metadata_workspace_bytes(a->n_entries, a->n_cols);
  if (!a->workspace || a->workspace_bytes < need) return TB200_ERR_BAD_ARG;
  return bitmatrix_metadata_launch(a->indx, a->indx_is_int16, a->n_entries, a->n_cols, a->col_sum, a->col_sorted_indx,
                                   a->row_sorted_indx, static_cast<int*>(a->workspace),
                                   static_cast<cudaStream_t>(stream_));
}

// ------------------------------------------------------------------ fixed-scratch variant
// tb200_bitmatrix_metadata_static: the same three kernels as tb200_bitmatrix_metadata, with the
// per-block histograms and the column offsets kept in a device array that is part of this library
// instead of in a caller-provided workspace. It is for callers whose device memory is fully
// planned before they start calling into the library and who therefore have no buffer to lend and
// no permission to create one: a serving process that carves up the GPU at start-up and treats
// any later allocation as a fault, or a host runtime in which cudaMalloc (which stalls the whole
// device) is banned on the request path.
//
// Capacity: TB200_STATIC_SCRATCH_INTS 32-bit words (a little over 1 MiB). The array exists once per
// GPU that loads the library and stays resident until the process exits. A call needs
// ceil(n_entries / 1024) * n_cols + n_cols words; larger problems are refused with
// TB200_ERR_TOO_LARGE before anything is launched.
//
// `g_static_scratch` below is a device symbol. In host code that name is only a handle: taking
// its address on the host does not give a pointer a kernel can use. The device address is fetched
// once per device with cudaGetSymbolAddress (with that device current) and cached by device ordinal
// (the cached address does not survive a cudaDeviceReset of that device); this happens inside the
// first call made on each device, so make that first call outside of any stream capture. Nothing in the scratch has to start out as zero: every call overwrites the part it uses
// (histograms, then prefix sums) before reading it. All calls on one GPU share the one array, so
// two calls whose kernels may run at the same time (different streams) corrupt each other; issue
// them on one stream or order them with events.
#define TB200_STATIC_SCRATCH_INTS (256 * 1024 + 1024)
static __device__ __align__(256) int g_static_scratch[TB200_STATIC_SCRATCH_INTS];

namespace tb200 {
static int* g_static_scratch_ptr[64] = {};
static std::mutex g_static_scratch_mu;

// Device address of g_static_scratch on the current device (nullptr on failure).
static int* static_scratch_ptr() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(g_static_scratch_mu);
  if (!g_static_scratch_ptr[dev]) {
    int* ptr = nullptr;
    if (cudaGetSymbolAddress((void**)&ptr, g_static_scratch) != cudaSuccess) return nullptr;
    g_static_scratch_ptr[dev] = ptr;
  }
  return g_static_scratch_ptr[dev];
}
}  // namespace tb200

extern "C" int tb200_bitmatrix_metadata_static(const void* indx, int32_t indx_is_int16, int64_t n_entries,
                                               int32_t n_cols, int32_t* col_sum, int32_t* col_sorted_indx,
                                               int32_t* row_sorted_indx, void* stream_) {
  if (!col_sum || (n_entries > 0 && (!indx || !col_sorted_indx || !row_sorted_indx))) return TB200_ERR_BAD_ARG;
  if (n_entries < 0 || n_cols <= 0) return TB200_ERR_BAD_ARG;
  if (n_cols > 8192 || n_entries > INT32_MAX) return TB200_ERR_UNSUPPORTED;
  const long long n_blocks = (n_entries + BM_BLOCK - 1) / BM_BLOCK;
  if (n_blocks * n_cols + n_cols > (long long)TB200_STATIC_SCRATCH_INTS) return TB200_ERR_TOO_LARGE;
  int* scratch = static_scratch_ptr();
  if (!scratch) return TB200_ERR_CUDA;
  return bitmatrix_metadata_launch(indx, indx_is_int16, n_entries, n_cols, col_sum, col_sorted_indx, row_sorted_indx,
                                   scratch, static_cast<cudaStream_t>(stream_));
}

extern "C" int tb200_ragged_metadata(const tb200_ragged_metadata_args* a, void* stream_) {
  if (!a || !a->slice_sizes || !a->slice_offs || !a->block_offs || (a->max_n_blocks > 0 && !a->block_schedule))
    return TB200_ERR_BAD_ARG;
  if (a->n_slices <= 0 || a->max_n_blocks < 0) return TB200_ERR_BAD_ARG;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (a->max_n_blocks > 0) {
    cudaError_t e = cudaMemsetAsync(a->block_schedule, 0xFF, (size_t)4 * a->max_n_blocks * sizeof(int), stream);
    if (e != cudaSuccess) return TB200_ERR_CUDA;
  }
  ragged_metadata_kernel<<<5, 256, 0, stream>>>(a->slice_sizes, a->n_slices, a->max_n_blocks, a->slice_offs,
                                                a->block_offs, a->block_schedule);
  return cuda_err(cudaGetLastError());
}

extern "C" int tb200_remap_ragged_metadata(const tb200_remap_ragged_metadata_args* a, void* stream_) {
  if (!a || !a->slice_sizes || !a->slice_offs || !a->block_offs || !a->slice_map || !a->out_slice_sizes ||
      !a->out_slice_offs || !a->out_block_offs)
    return TB200_ERR_BAD_ARG;
  if (a->n_slices <= 0 || a->n_slices > 65535 || a->max_n_blocks < 0) return TB200_ERR_BAD_ARG;
  if (a->max_n_blocks > 0 && (!a->block_schedule || !a->out_block_schedule)) return TB200_ERR_BAD_ARG;
  remap_ragged_metadata_kernel<<<5, 1024, 0, static_cast<cudaStream_t>(stream_)>>>(
      a->slice_sizes, a->slice_offs, a->block_offs, a->block_schedule, a->slice_map, a->n_slices, a->max_n_blocks,
      a->out_slice_sizes, a->out_slice_offs, a->out_block_offs, a->out_block_schedule);
  return cuda_err(cudaGetLastError());
}

extern "C" int tb200_reduce_k(const tb200_reduce_k_args* a, void* stream_) {
  if (!a || !a->x || !a->y) return TB200_ERR_BAD_ARG;
  if (a->n_tokens < 0 || a->k <= 0 || a->d <= 0 || (a->d % 8)) return TB200_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(a->x) & 15) || (reinterpret_cast<uintptr_t>(a->y) & 15)) return TB200_ERR_BAD_ARG;
  if (a->n_tokens == 0) return TB200_OK;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const long long total = a->n_tokens * (a->d / 8);
  if (a->x_rows < 0) return TB200_ERR_BAD_ARG;
  const long long x_rows = a->x_rows > 0 ? a->x_rows : a->n_tokens * a->k;
  int sms = sm_count();
  if (sms <= 0) sms = 148;
  long long blocks = (total + 255) / 256;
  if (blocks > (long long)sms * 16) blocks = (long long)sms * 16;
  if (a->dtype == TB200_BF16)
    reduce_k_kernel<__nv_bfloat16><<<(int)blocks, 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(a->x), a->mask, a->scale, a->row_indx, static_cast<__nv_bfloat16*>(a->y),
        a->n_tokens, a->k, (int)a->d, x_rows);
  else if (a->dtype == TB200_F16)
    reduce_k_kernel<__half><<<(int)blocks, 256, 0, stream>>>(static_cast<const __half*>(a->x), a->mask, a->scale,
                                                            a->row_indx, static_cast<__half*>(a->y), a->n_tokens, a->k,
                                                            (int)a->d, x_rows);
  else
    return TB200_ERR_UNSUPPORTED;
  return cuda_err(cudaGetLastError());
}

extern "C" int tb200_move_rows(const void* src, int64_t src_pitch_bytes, void* dst, int64_t dst_pitch_bytes,
                               const int32_t* indx, int64_t n_indx, int64_t row_bytes, int32_t scatter,
                               int64_t indexed_rows, void* stream_) {
  if (n_indx < 0 || row_bytes < 0 || indexed_rows < 0) return TB200_ERR_BAD_ARG;
  if (n_indx == 0 || row_bytes == 0) return TB200_OK;
  if (!src || !dst || !indx) return TB200_ERR_BAD_ARG;
  if ((row_bytes % 16) || (src_pitch_bytes % 16) || (dst_pitch_bytes % 16) || row_bytes > INT32_MAX)
    return TB200_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(src) & 15) || (reinterpret_cast<uintptr_t>(dst) & 15)) return TB200_ERR_BAD_ARG;
  int sms = sm_count();
  if (sms <= 0) sms = 148;
  long long blocks = (n_indx + 7) / 8;  // 8 warps per block
  if (blocks > (long long)sms * 16) blocks = (long long)sms * 16;
  move_rows_kernel<<<(int)blocks, 256, 0, static_cast<cudaStream_t>(stream_)>>>(
      static_cast<const uint8_t*>(src), src_pitch_bytes, static_cast<uint8_t*>(dst), dst_pitch_bytes, indx, n_indx,
      (int)row_bytes, scatter ? 1 : 0, indexed_rows);
  return cuda_err(cudaGetLastError());
}

extern "C" int tb200_gather_rows(const void* src, int64_t src_pitch_bytes, int64_t src_rows, void* dst,
                                 int64_t dst_pitch_bytes, const int32_t* indx, int64_t n_indx, int64_t row_bytes,
                                 void* stream_) {
  if (n_indx < 0 || row_bytes < 0 || src_rows < 0 || src_rows > INT32_MAX) return TB200_ERR_BAD_ARG;
  if (n_indx == 0 || row_bytes == 0) return TB200_OK;
  if (!src || !dst || !indx) return TB200_ERR_BAD_ARG;
  if ((row_bytes % 16) || (src_pitch_bytes % 16) || (dst_pitch_bytes % 16) || row_bytes > INT32_MAX)
    return TB200_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(src) & 15) || (reinterpret_cast<uintptr_t>(dst) & 15)) return TB200_ERR_BAD_ARG;
  int sms = sm_count();
  if (sms <= 0) sms = 148;
  long long blocks = (n_indx + 7) / 8;  // 8 warps per block
  if (blocks > (long long)sms * 16) blocks = (long long)sms * 16;
  gather_rows_kernel<<<(int)blocks, 256, 0, static_cast<cudaStream_t>(stream_)>>>(
      static_cast<const uint8_t*>(src), src_pitch_bytes, (int)src_rows, static_cast<uint8_t*>(dst), dst_pitch_bytes, indx,
      n_indx, (int)row_bytes);
  return cuda_err(cudaGetLastError());
}

extern "C" int tb200_swiglu(const tb200_swiglu_args* a, void* stream_) {
  if (!a || !a->a || !a->out) return TB200_ERR_BAD_ARG;
  if (a->rows < 0 || a->n_in <= 0 || (a->n_in & 1)) return TB200_ERR_BAD_ARG;
  if (a->rows == 0) return TB200_OK;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int n_out = (int)(a->n_in / 2);
  const long long total = a->rows * n_out;
  int sms = sm_count();
  if (sms <= 0) sms = 148;
  long long blocks = (total + 255) / 256;
  if (blocks > (long long)sms * 16) blocks = (long long)sms * 16;
  if (a->dtype == TB200_BF16)
    swiglu_kernel<__nv_bfloat16><<<(int)blocks, 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(a->a), static_cast<__nv_bfloat16*>(a->out), a->rows, n_out, a->lda, a->ldo,
        a->alpha, a->limit, a->has_limit);
  else if (a->dtype == TB200_F16)
    swiglu_kernel<__half><<<(int)blocks, 256, 0, stream>>>(static_cast<const __half*>(a->a),
                                                          static_cast<__half*>(a->out), a->rows, n_out, a->lda, a->ldo,
                                                          a->alpha, a->limit, a->has_limit);
  else if (a->dtype == TB200_F32)
    swiglu_kernel<float><<<(int)blocks, 256, 0, stream>>>(static_cast<const float*>(a->a),
                                                         static_cast<float*>(a->out), a->rows, n_out, a->lda, a->ldo,
                                                         a->alpha, a->limit, a->has_limit);
  else
    return TB200_ERR_UNSUPPORTED;
  return cuda_err(cudaGetLastError());
}
