// Expert-parallel token exchange over NVLink by plain peer stores (one process per GPU):
//
//   symmetric buffers   each rank allocates one buffer, exports a CUDA IPC handle, opens the
//                       handles of its peers: after that every rank holds a device pointer to
//                       every rank's buffer                <- SymmetricMemoryPool, distributed_details/mesh.py:34-166
//   symm_barrier_kernel cross-GPU barrier: rank r stores an epoch into flag r of every peer and
//                       waits (bounded) until all of its own flags carry it   <- hdl.barrier(channel)
//   ep_dispatch_kernel  a rank's token rows -> row `dispatch[entry]` of the buffer of the rank
//                       that owns the entry's expert         <- _convert_dp_to_ep, distributed.py:136-173
//   ep_combine_kernel   expert-sorted output rows -> row (entry % rows_per_rank) of the rank
//                       that holds the token                 <- _convert_ep_to_dp, distributed.py:217-254
// (paths are inside python/triton_kernels/triton_kernels/ of the reference).
//
// Transport is `st.global` of 16 bytes per lane to addresses that CUDA IPC mapped from the peer GPU;
// no multimem, no multicast, no TMA on peer memory. The barrier's waits are bounded like every wait
// in this library: a rank that never arrives makes the others give up after the limit, record a
// code in the status word and return.
#include <string.h>

#include "common.cuh"
#include "host_common.h"

namespace tb200 {

static constexpr int EP_MAX_RANKS = 16;

struct PeerPtrs {
  void* p[EP_MAX_RANKS];
};

// ---------------------------------------------------------------------------------- barrier
// Signal block of a channel inside every rank's symmetric buffer: uint32 flags[EP_MAX_RANKS] at
// byte 0 (flag j is written by rank j only), the rank's own epoch counter at byte 256 (never
// written by a peer). Epochs only grow, so nothing has to be reset between barriers, and because
// the counter lives on the device the launch has no per-call host state.
__global__ void symm_barrier_kernel(PeerPtrs sig, int rank, int world, unsigned long long limit_ns, int* status) {
  __shared__ uint32_t epoch_s;
  uint32_t* own = static_cast<uint32_t*>(sig.p[rank]);
  if (threadIdx.x == 0) epoch_s = own[64] + 1u;
  __syncthreads();
  const uint32_t epoch = epoch_s;
  const int j = threadIdx.x;
  if (j < world) {
    // everything this GPU wrote before the barrier (peer stores of earlier kernels included) is
    // ordered before the flag by a system-scope release
    __threadfence_system();
    uint32_t* remote = static_cast<uint32_t*>(sig.p[j]) + rank;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
    const uint32_t* mine = own + j;
    uint64_t t0 = 0;
    uint32_t spins = 0;
    for (;;) {
      uint32_t v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
      if ((int32_t)(v - epoch) >= 0) break;
      if (((++spins) & 0x3f) == 0) {
        if (*reinterpret_cast<volatile int*>(status) != 0) break;
        const uint64_t now = globaltimer_ns();
        if (t0 == 0) {
          t0 = now;
        } else if (now - t0 > limit_ns) {
          atomicCAS(status, 0, (WAIT_PEER << 16) | (j & 0xffff));
          break;
        }
      }
    }
    __threadfence_system();
  }
  __syncthreads();
  if (threadIdx.x == 0) own[64] = epoch;
}

// ---------------------------------------------------------------------------------- dispatch
// One warp per local token: lanes 0..k-1 look up the token's k (expert, sorted position) pairs and
// turn them into destination row addresses; the row is then read once, 16 bytes per lane, and stored
// to each destination. Entries with expert -1 or a position outside the buffer are skipped.
__global__ void ep_dispatch_kernel(const uint8_t* __restrict__ x, long long x_pitch, const void* __restrict__ expt_indx,
                                   int is16, const int* __restrict__ dispatch, const int* __restrict__ owner,
                                   PeerPtrs dst, long long dst_pitch, long long dst_rows, int row_bytes,
                                   int n_tokens_local, long long token0, int k, int n_experts, int world) {
  const int lane = threadIdx.x & 31;
  const long long warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long t = warp; t < n_tokens_local; t += nwarps) {
    uint8_t* my_dst = nullptr;
    if (lane < k) {
      const long long entry = (token0 + t) * k + lane;
      const int e = is16 ? (int)static_cast<const int16_t*>(expt_indx)[entry] : static_cast<const int*>(expt_indx)[entry];
      if (e >= 0 && e < n_experts) {
        const int r = __ldg(owner + e);
        const int pos = __ldg(dispatch + entry);
        if (r >= 0 && r < world && pos >= 0 && pos < dst_rows)
          my_dst = static_cast<uint8_t*>(dst.p[r]) + (long long)pos * dst_pitch;
      }
    }
    const uint8_t* src = x + t * x_pitch;
    for (int b = lane * 16; b < row_bytes; b += 512) {
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(src + b));
      for (int j = 0; j < k; ++j) {
        uint8_t* d = reinterpret_cast<uint8_t*>(__shfl_sync(0xffffffffu, (unsigned long long)my_dst, j));
        if (d) *reinterpret_cast<uint4*>(d + b) = v;
      }
    }
  }
}

// ---------------------------------------------------------------------------------- combine
// One warp per expert-sorted row r: entry = combine[r] names the (token, slot) the row belongs to; the row
// is forwarded iff this rank owns the entry's expert, to row (entry % rows_per_rank) of the rank
// entry / rows_per_rank.
__global__ void ep_combine_kernel(const uint8_t* __restrict__ src, long long src_pitch, const void* __restrict__ expt_indx,
                                  int is16, const int* __restrict__ combine, const int* __restrict__ owner, PeerPtrs dst,
                                  long long dst_pitch, int row_bytes, long long n_rows, long long rows_per_rank,
                                  int n_experts, int world, int rank) {
  const int lane = threadIdx.x & 31;
  const long long warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long r = warp; r < n_rows; r += nwarps) {
    const int entry = __ldg(combine + r);
    if (entry < 0 || entry >= n_rows) continue;
    const int e = is16 ? (int)static_cast<const int16_t*>(expt_indx)[entry] : static_cast<const int*>(expt_indx)[entry];
    if (e < 0 || e >= n_experts || __ldg(owner + e) != rank) continue;
    const long long to = entry / rows_per_rank;
    if (to >= world) continue;
    uint8_t* d = static_cast<uint8_t*>(dst.p[to]) + (entry - to * rows_per_rank) * dst_pitch;
    const uint8_t* s = src + r * src_pitch;
    for (int b = lane * 16; b < row_bytes; b += 1024) {
      const bool second = b + 512 < row_bytes;
      const uint4 v0 = __ldg(reinterpret_cast<const uint4*>(s + b));
      uint4 v1 = make_uint4(0, 0, 0, 0);
      if (second) v1 = __ldg(reinterpret_cast<const uint4*>(s + b + 512));
      *reinterpret_cast<uint4*>(d + b) = v0;
      if (second) *reinterpret_cast<uint4*>(d + b + 512) = v1;
    }
  }
}

// ---------------------------------------------------------------------------------- put
// The same `bytes` of local memory stored to one destination per rank (a rank's block of an all-gather:
// destination r is this rank's slot inside rank r's buffer). 16 bytes per thread per step.
__global__ void symm_put_kernel(const uint4* __restrict__ src, long long n16, PeerPtrs dst, int world) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n16; i += (long long)gridDim.x * blockDim.x) {
    const uint4 v = __ldg(src + i);
    for (int r = 0; r < world; ++r) static_cast<uint4*>(dst.p[r])[i] = v;
  }
}

static bool fill_peers(PeerPtrs* out, void* const* peers, int world) {
  if (!peers || world < 1 || world > EP_MAX_RANKS) return false;
  memset(out, 0, sizeof(*out));
  for (int i = 0; i < world; ++i) {
    if (!peers[i] || (reinterpret_cast<uintptr_t>(peers[i]) & 15)) return false;
    out->p[i] = peers[i];
  }
  return true;
}

}  // namespace tb200

using namespace tb200;

extern "C" int tb200_symm_alloc(size_t bytes, void** ptr) {
  if (!ptr || bytes == 0) return TB200_ERR_BAD_ARG;
  void* p = nullptr;
  if (cudaMalloc(&p, bytes) != cudaSuccess) return TB200_ERR_CUDA;
  if (cudaMemset(p, 0, bytes) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) {
    cudaFree(p);
    return TB200_ERR_CUDA;
  }
  *ptr = p;
  return TB200_OK;
}

extern "C" int tb200_symm_free(void* ptr) {
  if (!ptr) return TB200_OK;
  return cuda_err(cudaFree(ptr));
}

extern "C" int tb200_symm_export(const void* ptr, uint8_t* handle64) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handles are exchanged as 64 bytes");
  if (!ptr || !handle64) return TB200_ERR_BAD_ARG;
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, const_cast<void*>(ptr)) != cudaSuccess) return TB200_ERR_CUDA;
  memcpy(handle64, &h, 64);
  return TB200_OK;
}

extern "C" int tb200_symm_open(const uint8_t* handle64, void** peer_ptr) {
  if (!handle64 || !peer_ptr) return TB200_ERR_BAD_ARG;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  void* p = nullptr;
  if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) return TB200_ERR_CUDA;
  *peer_ptr = p;
  return TB200_OK;
}

extern "C" int tb200_symm_close(void* peer_ptr) {
  if (!peer_ptr) return TB200_OK;
  return cuda_err(cudaIpcCloseMemHandle(peer_ptr));
}

extern "C" int tb200_symm_barrier(void* const* signal_peers, int32_t rank, int32_t world, uint64_t limit_ns, void* stream) {
  PeerPtrs sig;
  if (!fill_peers(&sig, signal_peers, world) || rank < 0 || rank >= world) return TB200_ERR_BAD_ARG;
  if (limit_ns == 0 || limit_ns > 30000000000ull) return TB200_ERR_BAD_ARG;
  int* status = status_ptr();
  if (!status) return TB200_ERR_CUDA;
  symm_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(sig, rank, world, limit_ns, status);
  return cuda_err(cudaGetLastError());
}

extern "C" int tb200_symm_put(const void* src, size_t bytes, void* const* dst_peers, int32_t world, void* stream) {
  PeerPtrs dst;
  if (!fill_peers(&dst, dst_peers, world) || !src || (bytes % 16) || (reinterpret_cast<uintptr_t>(src) & 15))
    return TB200_ERR_BAD_ARG;
  if (bytes == 0) return TB200_OK;
  const long long n16 = (long long)(bytes / 16);
  int sms = sm_count();
  if (sms <= 0) sms = 148;
  long long blocks = (n16 + 255) / 256;
  if (blocks > sms * 4) blocks = sms * 4;
  symm_put_kernel<<<(int)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const uint4*>(src), n16, dst,
                                                                           world);
  return cuda_err(cudaGetLastError());
}

static int ep_grid(long long rows, int sms) {
  long long blocks = (rows + 7) / 8;  // 8 warps per block
  if (blocks > (long long)sms * 8) blocks = (long long)sms * 8;
  return (int)(blocks < 1 ? 1 : blocks);
}

extern "C" int tb200_ep_dispatch(const tb200_ep_dispatch_args* a, void* stream) {
  if (!a || !a->x || !a->expt_indx || !a->dispatch_indx || !a->expt_owner) return TB200_ERR_BAD_ARG;
  PeerPtrs dst;
  if (!fill_peers(&dst, a->dst_peers, a->world)) return TB200_ERR_BAD_ARG;
  if (a->n_tokens_local < 0 || a->token_offset < 0 || a->k <= 0 || a->k > 32 || a->n_experts <= 0 || a->dst_rows < 0)
    return TB200_ERR_BAD_ARG;
  if (a->row_bytes <= 0 || (a->row_bytes % 16) || (a->x_pitch_bytes % 16) || (a->dst_pitch_bytes % 16) ||
      a->row_bytes > INT32_MAX || (reinterpret_cast<uintptr_t>(a->x) & 15))
    return TB200_ERR_BAD_ARG;
  if (a->n_tokens_local == 0) return TB200_OK;
  int sms = sm_count();
  if (sms <= 0) sms = 148;
  ep_dispatch_kernel<<<ep_grid(a->n_tokens_local, sms), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(a->x), a->x_pitch_bytes, a->expt_indx, a->indx_is_int16 ? 1 : 0, a->dispatch_indx,
      a->expt_owner, dst, a->dst_pitch_bytes, a->dst_rows, (int)a->row_bytes, (int)a->n_tokens_local, a->token_offset,
      a->k, a->n_experts, a->world);
  return cuda_err(cudaGetLastError());
}

extern "C" int tb200_ep_combine(const tb200_ep_combine_args* a, void* stream) {
  if (!a || !a->src || !a->expt_indx || !a->combine_indx || !a->expt_owner) return TB200_ERR_BAD_ARG;
  PeerPtrs dst;
  if (!fill_peers(&dst, a->dst_peers, a->world)) return TB200_ERR_BAD_ARG;
  if (a->n_rows < 0 || a->n_rows > INT32_MAX || a->rows_per_rank <= 0 || a->n_experts <= 0 || a->rank < 0 ||
      a->rank >= a->world)
    return TB200_ERR_BAD_ARG;
  if (a->row_bytes <= 0 || (a->row_bytes % 16) || (a->src_pitch_bytes % 16) || (a->dst_pitch_bytes % 16) ||
      a->row_bytes > INT32_MAX || (reinterpret_cast<uintptr_t>(a->src) & 15))
    return TB200_ERR_BAD_ARG;
  if (a->n_rows == 0) return TB200_OK;
  int sms = sm_count();
  if (sms <= 0) sms = 148;
  ep_combine_kernel<<<ep_grid(a->n_rows, sms), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(a->src), a->src_pitch_bytes, a->expt_indx, a->indx_is_int16 ? 1 : 0, a->combine_indx,
      a->expt_owner, dst, a->dst_pitch_bytes, (int)a->row_bytes, a->n_rows, a->rows_per_rank, a->n_experts, a->world,
      a->rank);
  return cuda_err(cudaGetLastError());
}
