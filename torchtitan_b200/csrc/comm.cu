// NVLink / NVSwitch peer-memory collectives for the sharded data-parallel runtime.
//
// Every rank owns a "symmetric heap" (one cudaMalloc arena exported with CUDA IPC and mapped by all
// peers of the node). Collectives are single kernels that read peers' memory directly:
//
//   all-gather    : pull each peer's bf16 parameter shard straight into the parameter-contiguous
//                   gathered buffer (no copy-in / copy-out, one launch for all parameters of a unit)
//   reduce-scatter: read this rank's slice of every peer's bf16 gradient staging buffer, add in fp32
//                   in rank order (deterministic) and write / accumulate the fp32 gradient shard --
//                   the cast and the accumulation are fused into the transfer, and bf16 crosses the
//                   wire instead of fp32
//
// Ordering between ranks uses version flags in the symmetric heap (st.release.sys / ld.acquire.sys).
// Waits are bounded: when a peer's flag does not arrive within the limit the kernel records
// {code, peer} in an error word and returns without touching the data. Plain ld/st over NVLink only
// (no multimem, no TMA multicast), so the kernels run on any number of GPUs.
//
// Replaces: NCCL all-gather / reduce-scatter plus FSDP2's copy-in, copy-out and cast kernels
// (torch/distributed/fsdp/_fully_shard/_fsdp_collectives.py) used by the reference.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "protocol.h"

namespace {

using tt::proto::now_ns;
using tt::proto::st_release_sys;

#ifndef TT_COMM_WAIT_NS
#define TT_COMM_WAIT_NS 20000000000ull  // 20 s: peers may legitimately lag by a whole (first) step
#endif
constexpr int kMaxPeers = 16;

__device__ int g_comm_error[4] = {0, 0, 0, 0};  // {code, peer, expected, seen}
__device__ unsigned long long g_comm_wait_ns = TT_COMM_WAIT_NS;  // settable: tt_comm_set_wait_ns

struct Peers {
  const void* ptr[kMaxPeers];   // base of the relevant buffer on each rank (mapped into this process)
  const int* flag[kMaxPeers];   // that rank's flag word for this unit
};

struct Seg {            // one parameter of a unit
  long long shard_off;  // element offset of the chunk in a rank's flat shard
  long long full_off;   // element offset of the whole parameter in the gathered / staging layout
  long long chunk;      // elements per rank chunk (unpadded rows * inner)
};

// Thread 0 of the block waits until every peer's flag >= expected; result broadcast through smem.
__device__ bool wait_peers(const Peers& peers, int world, int expected, int* ok_smem) {
  if (threadIdx.x == 0) {
    int ok = 1;
    const uint64_t t0 = now_ns();
    for (int r = 0; r < world && ok; ++r) {
      if (peers.flag[r] == nullptr) continue;
      int seen;
      if (!tt::proto::wait_flag_ge(peers.flag[r], expected, t0, g_comm_wait_ns, &seen)) {
        if (atomicCAS(&g_comm_error[0], 0, 1) == 0) {
          g_comm_error[1] = r; g_comm_error[2] = expected; g_comm_error[3] = seen;
        }
        ok = 0;
      }
    }
    *ok_smem = ok;
  }
  __syncthreads();
  return *ok_smem != 0;
}

__global__ void set_flag_kernel(int* flag, int value) {
  __threadfence_system();
  st_release_sys(flag, value);
}

// ---------------------------------------------------------------------------------- all-gather
// grid.x = blocks per (peer); grid.y = world. Block (bx, r) copies a strided share of peer r's chunks.
template <typename T>
__global__ void __launch_bounds__(512) allgather_pull_kernel(Peers peers, const Seg* __restrict__ segs, int nseg,
                                                             T* __restrict__ dst, int world, int my_rank,
                                                             int expected) {
  __shared__ int ok;
  if (!wait_peers(peers, world, expected, &ok)) return;
  const int r = (my_rank + 1 + blockIdx.y) % world;  // start with the next rank so peers are hit evenly
  const T* src = static_cast<const T*>(peers.ptr[r]);
  constexpr int VEC = 16 / sizeof(T);
  for (int s = 0; s < nseg; ++s) {
    const Seg sg = segs[s];
    const T* sp = src + sg.shard_off;
    T* dp = dst + sg.full_off + static_cast<long long>(r) * sg.chunk;
    const bool aligned = ((reinterpret_cast<uintptr_t>(sp) | reinterpret_cast<uintptr_t>(dp)) & 15) == 0;
    if (aligned) {
      const long long nvec = sg.chunk / VEC;
      const uint4* s4 = reinterpret_cast<const uint4*>(sp);
      uint4* d4 = reinterpret_cast<uint4*>(dp);
      long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
      const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
      // four independent 16-byte loads in flight per thread
      for (; i + 3 * stride < nvec; i += 4 * stride) {
        const uint4 a = s4[i], b = s4[i + stride], c = s4[i + 2 * stride], d = s4[i + 3 * stride];
        d4[i] = a; d4[i + stride] = b; d4[i + 2 * stride] = c; d4[i + 3 * stride] = d;
      }
      for (; i < nvec; i += stride) d4[i] = s4[i];
      if (blockIdx.x == 0)
        for (long long t = nvec * VEC + threadIdx.x; t < sg.chunk; t += blockDim.x) dp[t] = sp[t];
    } else {
      for (long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; t < sg.chunk;
           t += static_cast<long long>(gridDim.x) * blockDim.x)
        dp[t] = sp[t];
    }
  }
}

// ---------------------------------------------------------------------------------- reduce-scatter
// out[shard_off + i] (+)= sum_r bf16(peer_r.staging[full_off + my_rank * chunk + i]), fp32 accumulate.
__global__ void __launch_bounds__(512) reduce_scatter_pull_kernel(Peers peers, const Seg* __restrict__ segs, int nseg,
                                                                  float* __restrict__ out, int world, int my_rank,
                                                                  int expected, int accumulate) {
  __shared__ int ok;
  if (!wait_peers(peers, world, expected, &ok)) return;
  for (int s = 0; s < nseg; ++s) {
    const Seg sg = segs[s];
    const long long base = sg.full_off + static_cast<long long>(my_rank) * sg.chunk;
    float* o = out + sg.shard_off;
    bool aligned = ((reinterpret_cast<uintptr_t>(o) & 15) == 0) && (base % 8 == 0);
    const long long nvec = aligned ? sg.chunk / 8 : 0;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
      uint4 v[kMaxPeers];
#pragma unroll
      for (int r = 0; r < kMaxPeers; ++r)
        if (r < world) v[r] = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(peers.ptr[r]) + base)[i];
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
      for (int r = 0; r < kMaxPeers; ++r) {
        if (r < world) {
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[r]);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(h[e]);
            acc[2 * e] += f.x; acc[2 * e + 1] += f.y;
          }
        }
      }
      float4* o4 = reinterpret_cast<float4*>(o + i * 8);
      if (accumulate) {
        const float4 a = o4[0], b = o4[1];
        acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
        acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
      }
      o4[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
      o4[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
    }
    // tail (or the whole segment when unaligned)
    for (long long t = nvec * 8 + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; t < sg.chunk;
         t += static_cast<long long>(gridDim.x) * blockDim.x) {
      float a = 0.f;
      for (int r = 0; r < world; ++r) a += __bfloat162float(static_cast<const __nv_bfloat16*>(peers.ptr[r])[base + t]);
      o[t] = accumulate ? o[t] + a : a;
    }
  }
}

// Elementwise all-reduce (sum) of small fp32 vectors through peer reads (used for HSDP replicas and
// norm weights under tensor parallel); every rank reads all peers and keeps the full result.
__global__ void allreduce_pull_f32_kernel(Peers peers, float* __restrict__ out, long long n, int world, int expected) {
  __shared__ int ok;
  if (!wait_peers(peers, world, expected, &ok)) return;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float a = 0.f;
    for (int r = 0; r < world; ++r) a += static_cast<const float*>(peers.ptr[r])[i];
    out[i] = a;
  }
}

Peers make_peers(const void* const* ptrs, const int* const* flags, int world) {
  Peers p;
  for (int i = 0; i < kMaxPeers; ++i) {
    p.ptr[i] = i < world ? ptrs[i] : nullptr;
    p.flag[i] = (i < world && flags) ? flags[i] : nullptr;
  }
  return p;
}

}  // namespace

extern "C" {

// ---- symmetric heap (CUDA IPC) ------------------------------------------------------------------
int tt_ipc_alloc(void** out, long long bytes) { return cudaMalloc(out, static_cast<size_t>(bytes)) == cudaSuccess ? 0 : -1; }
int tt_ipc_free(void* p) { return cudaFree(p) == cudaSuccess ? 0 : -1; }
int tt_ipc_handle_size() { return static_cast<int>(sizeof(cudaIpcMemHandle_t)); }
int tt_ipc_get_handle(void* p, void* handle_out) {
  return cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t*>(handle_out), p) == cudaSuccess ? 0 : -1;
}
int tt_ipc_open(const void* handle, void** out) {
  cudaIpcMemHandle_t h = *static_cast<const cudaIpcMemHandle_t*>(handle);
  cudaError_t e = cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess);
  return e == cudaSuccess ? 0 : -static_cast<int>(e);
}
int tt_ipc_close(void* p) { return cudaIpcCloseMemHandle(p) == cudaSuccess ? 0 : -1; }
int tt_memset(void* p, int v, long long bytes, cudaStream_t st) {
  return cudaMemsetAsync(p, v, static_cast<size_t>(bytes), st) == cudaSuccess ? 0 : -1;
}

int tt_set_flag(int* flag, int value, cudaStream_t st) {
  set_flag_kernel<<<1, 1, 0, st>>>(flag, value);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// peer_ptrs[world]: each rank's flat bf16 (dtype 0) / fp32 (dtype 1) shard; peer_flags[world] may be null entries.
int tt_allgather_pull(const void* const* peer_ptrs, const int* const* peer_flags, const void* segs, int nseg, void* dst,
                      int world, int my_rank, int expected, int dtype, int blocks_per_peer, cudaStream_t st) {
  if (world > kMaxPeers) return -2;
  Peers p = make_peers(peer_ptrs, peer_flags, world);
  dim3 grid(blocks_per_peer > 0 ? blocks_per_peer : 8, world);
  if (dtype == 0)
    allgather_pull_kernel<__nv_bfloat16><<<grid, 512, 0, st>>>(p, static_cast<const Seg*>(segs), nseg,
                                                              static_cast<__nv_bfloat16*>(dst), world, my_rank, expected);
  else
    allgather_pull_kernel<float><<<grid, 512, 0, st>>>(p, static_cast<const Seg*>(segs), nseg, static_cast<float*>(dst),
                                                      world, my_rank, expected);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

int tt_reduce_scatter_pull(const void* const* peer_ptrs, const int* const* peer_flags, const void* segs, int nseg,
                           float* out, int world, int my_rank, int expected, int accumulate, int blocks,
                           cudaStream_t st) {
  if (world > kMaxPeers) return -2;
  Peers p = make_peers(peer_ptrs, peer_flags, world);
  reduce_scatter_pull_kernel<<<blocks > 0 ? blocks : 64, 512, 0, st>>>(p, static_cast<const Seg*>(segs), nseg, out, world,
                                                                      my_rank, expected, accumulate);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

int tt_allreduce_pull_f32(const void* const* peer_ptrs, const int* const* peer_flags, float* out, long long n, int world,
                          int expected, cudaStream_t st) {
  if (world > kMaxPeers) return -2;
  Peers p = make_peers(peer_ptrs, peer_flags, world);
  int blocks = static_cast<int>((n + 511) / 512);
  if (blocks > 64) blocks = 64;
  if (blocks < 1) blocks = 1;
  allreduce_pull_f32_kernel<<<blocks, 512, 0, st>>>(p, out, n, world, expected);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// Upper bound for waiting on peers' version flags (default 20 s).
int tt_comm_set_wait_ns(unsigned long long ns) {
  return cudaMemcpyToSymbol(g_comm_wait_ns, &ns, sizeof(ns)) == cudaSuccess ? 0 : -1;
}

// {code, peer, expected, seen}; code 1 = a peer's version flag did not arrive in time. Reading clears.
int tt_comm_error(int* out4) {
  int v[4] = {0, 0, 0, 0}, zero[4] = {0, 0, 0, 0};
  cudaMemcpyFromSymbol(v, g_comm_error, sizeof(v));
  if (v[0]) cudaMemcpyToSymbol(g_comm_error, zero, sizeof(zero));
  for (int i = 0; i < 4; ++i) out4[i] = v[i];
  return v[0];
}

}  // extern "C"

// ------------------------------------------------------------------------------------ RL weight sync
// Trainer -> generator replicas: every trainer rank casts the fp32 master shards it owns to bf16 and stores them straight
// into the parameter arenas of all generator replicas (peer-mapped), following a precomputed list of contiguous
// segments. One launch per sync per trainer rank; the arena version flag is published afterwards (tt_set_flag on the
// peer-mapped flag), and a generator waits for all trainer flags (tt_wait_flags, bounded) before it swaps arenas.
// Counterpart of get_weights (full tensors) + RPC + set_model_state_dict in the reference
// (torchtitan/experiments/rl/unified/actors/trainer.py:226-239, actors/generator.py:307-335).
namespace {

struct PushSeg {
  const float* src;     // fp32 source (this rank's shard of one parameter)
  long long dst_off;    // element offset in the bf16 arena
  long long n;          // elements
};

struct Arenas {
  __nv_bfloat16* base[kMaxPeers];
  int count;
};

__global__ void __launch_bounds__(256) push_cast_kernel(const PushSeg* __restrict__ segs, int nseg, Arenas dst) {
  // grid.y = segment, grid.x = blocks striding over the segment in 8-element (16-byte bf16) chunks
  for (int s = blockIdx.y; s < nseg; s += gridDim.y) {
    const PushSeg sg = segs[s];
    const bool vec = ((sg.dst_off & 7) == 0) && ((reinterpret_cast<uintptr_t>(sg.src) & 15) == 0);
    if (vec) {
      const long long n8 = sg.n / 8;
      for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8;
           i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const float4 a = reinterpret_cast<const float4*>(sg.src)[2 * i];
        const float4 b = reinterpret_cast<const float4*>(sg.src)[2 * i + 1];
        uint4 v;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
        h[0] = __floats2bfloat162_rn(a.x, a.y); h[1] = __floats2bfloat162_rn(a.z, a.w);
        h[2] = __floats2bfloat162_rn(b.x, b.y); h[3] = __floats2bfloat162_rn(b.z, b.w);
        for (int g = 0; g < dst.count; ++g) reinterpret_cast<uint4*>(dst.base[g] + sg.dst_off)[i] = v;
      }
      if (blockIdx.x == 0 && threadIdx.x < (sg.n & 7)) {
        const long long i = n8 * 8 + threadIdx.x;
        const __nv_bfloat16 v = __float2bfloat16(sg.src[i]);
        for (int g = 0; g < dst.count; ++g) dst.base[g][sg.dst_off + i] = v;
      }
    } else {
      for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < sg.n;
           i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const __nv_bfloat16 v = __float2bfloat16(sg.src[i]);
        for (int g = 0; g < dst.count; ++g) dst.base[g][sg.dst_off + i] = v;
      }
    }
  }
}

__global__ void wait_flags_kernel(Peers peers, int n, int expected) {
  __shared__ int ok;
  wait_peers(peers, n, expected, &ok);
}

}  // namespace

extern "C" {

// segs: device array of {const float* src, long long dst_off, long long n}; arenas: host array of peer-mapped bf16 arena
// base pointers (one per generator replica).
int tt_push_cast(const void* segs, int nseg, void* const* arenas, int n_arenas, cudaStream_t st) {
  if (nseg <= 0 || n_arenas <= 0) return 0;
  if (n_arenas > kMaxPeers) return -2;
  Arenas a;
  a.count = n_arenas;
  for (int i = 0; i < kMaxPeers; ++i) a.base[i] = i < n_arenas ? static_cast<__nv_bfloat16*>(arenas[i]) : nullptr;
  dim3 grid(32, nseg < 1024 ? nseg : 1024);
  push_cast_kernel<<<grid, 256, 0, st>>>(static_cast<const PushSeg*>(segs), nseg, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// Stream-ordered bounded wait until every flag >= expected (error word set on expiry, see tt_comm_error).
int tt_wait_flags(const int* const* flags, int n, int expected, cudaStream_t st) {
  if (n <= 0) return 0;
  if (n > kMaxPeers) return -2;
  Peers p;
  for (int i = 0; i < kMaxPeers; ++i) { p.ptr[i] = nullptr; p.flag[i] = i < n ? flags[i] : nullptr; }
  wait_flags_kernel<<<1, 32, 0, st>>>(p, n, expected);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // extern "C"
