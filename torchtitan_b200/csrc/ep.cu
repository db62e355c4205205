// Expert-parallel token exchange over NVLink peer memory: permute + all-to-all in one kernel, no host synchronisation.
//
// Every rank has sorted its (token, slot) pairs by global expert. Per MoE layer:
//   1. tt_ep_publish_counts : each rank stores its per-expert pair counts into slot [rank] of every peer's count table and
//                             raises that peer's flag for it (st.release.sys).
//   2. tt_ep_build_maps     : waits (bounded) for all peers' counts, then derives everything from the [ranks][experts]
//                             table, identically on every rank: for each of this rank's sorted rows the destination rank
//                             and the row inside that rank's expert-grouped receive buffer (groups padded to `align`
//                             rows, sources in rank order inside a group); for each receive row the source rank and sorted
//                             position it came from (the way back); the padded group offsets for the grouped GEMM; and it
//                             zero-fills the padding rows of the receive buffer.
//   3. tt_ep_push           : one warp per row copies the row (optionally gathered through an index, which fuses the
//                             permutation) straight into the destination rank's buffer with 16-byte stores; each CTA then
//                             bumps an arrival counter on every destination (system-scope atomic after a system fence).
//                             The same kernel runs the way back (expert outputs -> the source's sorted order) with the
//                             reverse maps, and both directions again for the gradients.
//   4. tt_ep_wait           : the consumer side waits (bounded) until the arrival counter reached W * CTAs * call count.
//
// Buffers are double-buffered by call parity: a rank sees a peer's pushes of call n + 1 only after that peer finished
// consuming call n (stream order on the peer), so buffer n % 2 is free again when call n + 2 starts.
// Rows that do not fit the fixed-capacity receive buffer are dropped and reported through the error word.
// Replaces: all_to_all_single of counts + device-to-host read of the split sizes + all_to_all_single of rows + the index
// permutation (torchtitan/distributed/expert_parallel.py:87-166) of the reference.

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace {

#ifndef TT_EP_WAIT_NS
#define TT_EP_WAIT_NS 20000000000ull   // 20 s: a peer may lag by a whole first step
#endif
constexpr int kMaxRanks = 16;
constexpr int kMaxExperts = 512;

__device__ int g_ep_error[4] = {0, 0, 0, 0};   // {code, detail, expected, seen}
__device__ unsigned long long g_ep_wait_ns = TT_EP_WAIT_NS;

__device__ __forceinline__ uint64_t now_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void set_error(int code, int detail, int expected, int seen) {
  if (atomicCAS(&g_ep_error[0], 0, code) == 0) {
    g_ep_error[1] = detail;
    g_ep_error[2] = expected;
    g_ep_error[3] = seen;
  }
}

struct PeerPtrs {
  void* p[kMaxRanks];
};

// counts [E] int64 of this rank -> tables[d][rank][e] on every rank d, then flags[d][rank] = version
__global__ void publish_counts_kernel(const long long* __restrict__ counts, PeerPtrs tables, PeerPtrs flags, int world,
                                      int rank, int E, int version) {
  for (int i = threadIdx.x; i < world * E; i += blockDim.x) {
    const int d = i / E, e = i - d * E;
    static_cast<int*>(tables.p[d])[rank * E + e] = static_cast<int>(counts[e]);
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < world) st_release_sys(static_cast<int*>(flags.p[threadIdx.x]) + rank, version);
}

// One CTA. Outputs (device): dst_rank / dst_row [n] for this rank's sorted rows, rev_rank / rev_row [cap] for its receive
// rows (-1 = padding or unused), offs [El] = inclusive padded group ends, info = {rows used in the receive buffer,
// rows expected from peers}.
__global__ void __launch_bounds__(256)
build_maps_kernel(const int* __restrict__ table, const int* __restrict__ flags, int world, int rank, int E, int El, int align,
                  int n, int cap, int version, int* __restrict__ dst_rank, int* __restrict__ dst_row,
                  int* __restrict__ rev_rank, int* __restrict__ rev_row, int* __restrict__ offs, int* __restrict__ info,
                  __nv_bfloat16* __restrict__ recv, int D, int report_overflow) {
  __shared__ int s_ok;
  __shared__ int s_dst_start[kMaxExperts];     // receive row (on the owner) where this rank's rows of expert e begin
  __shared__ int s_my_cum[kMaxExperts + 1];    // exclusive prefix of this rank's counts
  __shared__ int s_base[kMaxExperts];          // local experts: first row of the group
  __shared__ int s_size[kMaxExperts];          // local experts: real rows of the group
  __shared__ int s_red[256];
  if (threadIdx.x == 0) {
    int ok = 1;
    const uint64_t t0 = now_ns();
    for (int r = 0; r < world && ok; ++r) {
      int seen;
      while ((seen = ld_acquire_sys(flags + r)) < version) {
        if (now_ns() - t0 > g_ep_wait_ns) { set_error(1, r, version, seen); ok = 0; break; }
        __nanosleep(200);
      }
    }
    s_ok = ok;
  }
  __syncthreads();
  if (!s_ok) {
    if (threadIdx.x == 0) { info[0] = 0; info[1] = 0; }
    for (int i = threadIdx.x; i < El; i += blockDim.x) offs[i] = 0;
    for (int i = threadIdx.x; i < n; i += blockDim.x) dst_rank[i] = -1;
    for (int i = threadIdx.x; i < cap; i += blockDim.x) rev_rank[i] = -1;
    return;
  }
  // per owner rank d: padded bases of its local experts; every thread handles some (d, el) via a serial scan per d
  if (threadIdx.x < world) {
    const int d = threadIdx.x;
    int base = 0;
    for (int el = 0; el < El; ++el) {
      const int e = d * El + el;
      int total = 0, before = 0;
      for (int s = 0; s < world; ++s) {
        const int c = table[s * E + e];
        if (s < rank) before += c;
        total += c;
      }
      s_dst_start[e] = base + before;
      if (d == rank) { s_base[el] = base; s_size[el] = total; }
      base += (total + align - 1) / align * align;
    }
    if (d == rank) {
      int run = 0;
      for (int el = 0; el < El; ++el) { run = s_base[el] + (s_size[el] + align - 1) / align * align; offs[el] = min(run, cap); }
      info[0] = min(run, cap);
      // more rows than the buffer holds: an error in the fixed-capacity mode (they will be dropped); in the lossless
      // mode the host sees the same table and routes this call through the collectives, so nothing is lost
      if (run > cap && report_overflow) set_error(2, rank, cap, run);
    }
  }
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < E; ++e) { s_my_cum[e] = run; run += table[rank * E + e]; }
    s_my_cum[E] = run;
    if (run != n) set_error(3, rank, n, run);
  }
  __syncthreads();
  // forward map: sorted row j of this rank -> (owner, row)
  for (int j = threadIdx.x; j < n; j += blockDim.x) {
    int lo = 0, hi = E;                 // largest e with my_cum[e] <= j
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (s_my_cum[mid] <= j) lo = mid; else hi = mid;
    }
    // skip experts with no rows that share the same prefix value
    int e = lo;
    while (e + 1 < E && s_my_cum[e + 1] <= j) ++e;
    const int row = s_dst_start[e] + (j - s_my_cum[e]);
    dst_rank[j] = (j < s_my_cum[E] && row < cap) ? e / El : -1;
    dst_row[j] = row;
  }
  // reverse map + zero the padding rows of the receive buffer
  for (int r = threadIdx.x; r < cap; r += blockDim.x) rev_rank[r] = -1;
  __syncthreads();
  for (int el = 0; el < El; ++el) {
    const int e = rank * El + el;
    int seg = s_base[el];
    for (int s = 0; s < world; ++s) {
      const int c = table[s * E + e];
      // sorted position on rank s where its rows of expert e begin
      int src0 = 0;
      for (int e2 = threadIdx.x; e2 < e; e2 += blockDim.x) src0 += table[s * E + e2];
      // block-wide sum of src0
      s_red[threadIdx.x] = src0;
      __syncthreads();
      for (int o = 128; o > 0; o >>= 1) { if (threadIdx.x < o) s_red[threadIdx.x] += s_red[threadIdx.x + o]; __syncthreads(); }
      const int start = s_red[0];
      __syncthreads();
      for (int i = threadIdx.x; i < c; i += blockDim.x) {
        if (seg + i < cap) { rev_rank[seg + i] = s; rev_row[seg + i] = start + i; }
      }
      seg += c;
    }
    const int pad_end = min(s_base[el] + (s_size[el] + align - 1) / align * align, cap);
    const int pad_rows = max(pad_end - seg, 0);
    if (recv != nullptr) {
      const long long words = static_cast<long long>(pad_rows) * D / 8;
      uint4* z = reinterpret_cast<uint4*>(recv + static_cast<long long>(seg) * D);
      for (long long i = threadIdx.x; i < words; i += blockDim.x) z[i] = make_uint4(0, 0, 0, 0);
    }
  }
  if (threadIdx.x == 0) info[1] = info[0];
}

// One warp per input row. in_index (nullable): row i is read from in_rows[in_index[i]].
__global__ void __launch_bounds__(256)
push_kernel(const __nv_bfloat16* __restrict__ in_rows, const int* __restrict__ in_index, int n_in,
            const int* __restrict__ to_rank, const int* __restrict__ to_row, PeerPtrs bufs, PeerPtrs arrive, int world, int D,
            int cap_rows) {
  const int lane = threadIdx.x & 31, warps = (gridDim.x * blockDim.x) >> 5;
  const int n16 = D / 8;
  for (int i = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; i < n_in; i += warps) {
    const int d = to_rank[i];
    if (d < 0) continue;
    const int row = to_row[i];
    if (row < 0 || row >= cap_rows) continue;
    const long long src = in_index ? in_index[i] : i;
    const uint4* s = reinterpret_cast<const uint4*>(in_rows + src * D);
    uint4* t = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(bufs.p[d]) + static_cast<long long>(row) * D);
    for (int c = lane; c < n16; c += 32) t[c] = s[c];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < world) atomicAdd_system(static_cast<int*>(arrive.p[threadIdx.x]), 1);
}

__global__ void wait_kernel(const int* __restrict__ arrive, int target) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  const uint64_t t0 = now_ns();
  int seen;
  while ((seen = ld_acquire_sys(arrive)) < target) {
    if (now_ns() - t0 > g_ep_wait_ns) { set_error(4, 0, target, seen); return; }
    __nanosleep(200);
  }
}

}  // namespace

extern "C" {

// {code, detail, expected, seen}; reading clears. Codes: 1 counts of a peer missing, 2 receive capacity exceeded
// (rows dropped), 3 counts do not add up to the rows sent, 4 arrivals missing.
int tt_ep_error(int* out4) {
  int h[4];
  if (cudaMemcpyFromSymbol(h, g_ep_error, sizeof(h)) != cudaSuccess) return -1;
  for (int i = 0; i < 4; ++i) out4[i] = h[i];
  if (h[0]) {
    int z[4] = {0, 0, 0, 0};
    cudaMemcpyToSymbol(g_ep_error, z, sizeof(z));
  }
  return h[0] ? 1 : 0;
}

void tt_ep_set_wait_ns(unsigned long long ns) { cudaMemcpyToSymbol(g_ep_wait_ns, &ns, sizeof(ns)); }

int tt_ep_push_ctas() { return 148 * 2; }

int tt_ep_publish_counts(const long long* counts, void* const* tables, void* const* flags, int world, int rank, int E,
                         int version, cudaStream_t st) {
  if (world < 1 || world > kMaxRanks || E > kMaxExperts) return -6;
  PeerPtrs t, f;
  for (int r = 0; r < world; ++r) { t.p[r] = tables[r]; f.p[r] = flags[r]; }
  publish_counts_kernel<<<1, 256, 0, st>>>(counts, t, f, world, rank, E, version);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// report_overflow: 1 = rows beyond the capacity set error code 2 (they are dropped); 0 = the caller handles overflow itself.
int tt_ep_build_maps_opt(const int* table, const int* flags, int world, int rank, int E, int align, int n, int cap,
                         int version, int* dst_rank, int* dst_row, int* rev_rank, int* rev_row, int* offs, int* info,
                         void* recv, int D, int report_overflow, cudaStream_t st) {
  if (world < 1 || world > kMaxRanks || E > kMaxExperts || E % world || D % 8) return -6;
  build_maps_kernel<<<1, 256, 0, st>>>(table, flags, world, rank, E, E / world, align, n, cap, version, dst_rank, dst_row,
                                       rev_rank, rev_row, offs, info, static_cast<__nv_bfloat16*>(recv), D, report_overflow);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

int tt_ep_build_maps(const int* table, const int* flags, int world, int rank, int E, int align, int n, int cap, int version,
                     int* dst_rank, int* dst_row, int* rev_rank, int* rev_row, int* offs, int* info, void* recv, int D,
                     cudaStream_t st) {
  return tt_ep_build_maps_opt(table, flags, world, rank, E, align, n, cap, version, dst_rank, dst_row, rev_rank, rev_row, offs,
                              info, recv, D, 1, st);
}

int tt_ep_push(const void* in_rows, const int* in_index, int n_in, const int* to_rank, const int* to_row, void* const* bufs,
               void* const* arrive, int world, int D, int cap_rows, cudaStream_t st) {
  if (world < 1 || world > kMaxRanks || D % 8) return -6;
  PeerPtrs b, a;
  for (int r = 0; r < world; ++r) { b.p[r] = bufs[r]; a.p[r] = arrive[r]; }
  push_kernel<<<tt_ep_push_ctas(), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(in_rows), in_index, n_in, to_rank, to_row,
                                                 b, a, world, D, cap_rows);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

int tt_ep_wait(const int* arrive, int target, cudaStream_t st) {
  wait_kernel<<<1, 32, 0, st>>>(arrive, target);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // extern "C"
