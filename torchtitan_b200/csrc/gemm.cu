// bf16 GEMM on the 5th-generation tensor cores (tcgen05.mma, accumulators in TMEM), operands staged
// by TMA into 128-byte-swizzled shared memory.
//
//   C[M,N] (+)= A[M,K] * B[N,K]^T          (fp32 accumulate, bf16 or fp32 output)
//
// Each operand may be stored K-major (contraction dimension contiguous) or MN-major (stored
// transposed, [K, M] / [K, N]), which covers the three GEMMs of a linear layer without explicit
// transposes: forward (K,K), input gradient (A K-major, B MN-major), weight gradient (MN,MN).
//
// Structure: persistent CTAs (one per SM) walk a grouped tile order; warp 0 = TMA producer,
// warp 1 = UMMA issuer (a single elected thread), warp 2 owns the TMEM allocation, warps 4-7 =
// epilogue. A 4-stage (128x64 | 256x64) operand ring and two 256-column TMEM accumulators let the
// epilogue of tile i overlap the main loop of tile i+1. No cluster multicast is used anywhere, so
// the kernel is safe to run on any number of GPUs and with operands in peer memory.
//
// Replaces: cuBLAS/cuBLASLt calls behind nn.Linear in the reference (torchtitan/models/common/linear.py:14-56).
#include "ptx.cuh"

namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int STAGES = 4;
constexpr int UMMA_K = 16;
constexpr uint32_t A_STAGE_BYTES = BM * BK * 2;  // 16 KB
constexpr uint32_t B_STAGE_BYTES = BN * BK * 2;  // 32 KB
constexpr uint32_t TMEM_COLS = 512;
constexpr int NUM_THREADS = 256;
constexpr size_t SMEM_BYTES = 1024 /*align slack*/ + STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + 256;

__device__ int g_gemm_error = 0;

struct GemmArgs {
  int M, N, K;
  int tiles_m, tiles_n, k_iters;
  int a_mn, b_mn;       // operand stored MN-major (transposed) ?
  uint32_t idesc;
  void* C;
  long long ldc;
  int c_fp32;
  int accumulate;       // C = result + addend, where the addend is R when set and the previous content of C otherwise
  const void* R;        // bf16 [M, N] with row stride ldr (residual input of the layer); bf16 output only
  long long ldr;
  // fused all-gather variant: per n-tile readiness flags (nullptr = plain GEMM)
  const int* ready_flags;
  int ready_value;
  // fused all-gather (same launch): the last `copy_ctas` CTAs pull row panels of the gathered operand from the peers'
  // memory over NVLink into the local buffer and publish one flag per panel; the GEMM CTAs wait for the panel they need.
  int flags_by_m;       // ready_flags index = m-tile (A operand gathered) instead of n-tile (B operand gathered)
  int m_rot;            // tiles visit m-panels starting at this offset (the local shard first)
  int m_interleave;     // 1: visit the blocks round-robin (tile j of every block before tile j + 1 of any), which spreads the
                        // peer-bound stores of the fused reduce-scatter over the whole launch instead of its first part
  int m_block;          // m-tiles per ordering block: all tiles of one block are visited before the next block (the fused
                        // reduce-scatter sets it to the m-tiles per rank, so every peer-owned tile precedes the own ones)
  int copy_ctas;
  const void* gather_src[16];  // base of the gathered buffer on every rank (peer-mapped addresses)
  const int* gather_flag[16];  // rank r's "my slice is written" version flag
  void* gather_dst;            // local gathered buffer
  int* panel_ready;            // local flags, one per panel (same array as ready_flags)
  long long panel_bytes;
  int panels_per_rank, gather_world, gather_rank, gather_expected;
  // fused reduce-scatter (same launch): tiles whose rows another rank owns come first; their epilogue stores the bf16
  // partial into slot [this rank] of the owner's staging buffer (peer-mapped stores) and bumps the owner's counter for
  // (this rank, 128-row panel, 256-column tile). Tiles of this rank's own rows come last: their epilogue waits for the
  // peers' counters, adds the staged partials to the fp32 accumulator in rank order and writes the final rows.
  int rs_world, rs_rank;
  void* rs_stage[16];          // staging buffer [world][rows_per_rank][N] bf16 on every rank (peer-mapped)
  int* rs_count[16];           // counters [world][panels_per_rank][tiles of 256 columns] on every rank (peer-mapped)
  void* rs_out;                // local result [rows_per_rank, N] bf16
  int rs_rows_per_rank;
  int rs_tiles_n;              // 256-column tiles per row panel
  int rs_target;               // counter value that means "all 4 epilogue warps of this call have stored"
  int rs_skip_own;             // contribute only: tiles of this rank's own rows are not computed
  // 8-bit float operands (e4m3/e5m2, both K-major): `bk` contraction elements per stage (128 instead of 64) and an
  // epilogue that multiplies by the dequantisation scales: scale_mode 1 = one scale per tensor (pointers to scalars),
  // 2 = one per row of A and one per row of B (= output column).
  int fp8;
  int bk;
  int scale_mode;
  const float* scale_a;
  const float* scale_b;
};

__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int& tm, int& tn) {
  // grouped order: 8 m-tiles share the same sweep over n so concurrently running CTAs reuse
  // A row-panels and B column-panels out of L2
  constexpr int GROUP_M = 8;
  int per_group = GROUP_M * tiles_n;
  int g = t / per_group;
  int first_m = g * GROUP_M;
  int gm = min(tiles_m - first_m, GROUP_M);
  int r = t - g * per_group;
  tm = first_m + r % gm;
  tn = r / gm;
}

// Tile t of the persistent schedule -> (tm, tn): blocks of `m_block` m-tiles one after another, the grouped order inside
// a block, then the rotation.
__device__ __forceinline__ void tile_coords_p(const GemmArgs& p, int t, int& tm, int& tn) {
  int blk, local;
  if (p.m_interleave) {
    const int nblk = p.tiles_m / p.m_block;
    local = t / nblk;
    blk = t - local * nblk;
  } else {
    const int blk_tiles = p.m_block * p.tiles_n;
    blk = t / blk_tiles;
    local = t - blk * blk_tiles;
  }
  tile_coords(local, p.m_block, p.tiles_n, tm, tn);
  tm = (tm + blk * p.m_block + p.m_rot) % p.tiles_m;
}

// Write 32 consecutive accumulator columns of one output row (bf16 or fp32, optional C += ...).
// 8-bit float GEMMs: multiply the accumulators by the dequantisation scales (in place, before the store).
// `sa` is the row's scale (times the tensor scale of B in per-tensor mode), loaded once per tile row by the caller.
__device__ __forceinline__ void apply_scales(const GemmArgs& p, float sa, int col, uint32_t (&r)[32]) {
  if (p.scale_mode == 1) {
#pragma unroll
    for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * sa);
  } else if (col + 32 <= p.N && (reinterpret_cast<uintptr_t>(p.scale_b + col) & 15) == 0) {
#pragma unroll
    for (int j4 = 0; j4 < 8; ++j4) {
      const float4 sb = __ldg(reinterpret_cast<const float4*>(p.scale_b + col) + j4);
      r[4 * j4 + 0] = __float_as_uint(__uint_as_float(r[4 * j4 + 0]) * sa * sb.x);
      r[4 * j4 + 1] = __float_as_uint(__uint_as_float(r[4 * j4 + 1]) * sa * sb.y);
      r[4 * j4 + 2] = __float_as_uint(__uint_as_float(r[4 * j4 + 2]) * sa * sb.z);
      r[4 * j4 + 3] = __float_as_uint(__uint_as_float(r[4 * j4 + 3]) * sa * sb.w);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const float sb = (col + j < p.N) ? __ldg(p.scale_b + col + j) : 0.f;
      r[j] = __float_as_uint(__uint_as_float(r[j]) * sa * sb);
    }
  }
}

__device__ __forceinline__ void store_chunk_to(const GemmArgs& p, void* Cbase, int row, int col, const uint32_t (&r)[32]);

template <bool RS>
__device__ __forceinline__ void store_chunk(const GemmArgs& p, int row, int col, const uint32_t (&r)[32]) {
  if constexpr (RS) {
    // reduce-scatter epilogue: row -> (owner, row inside the owner's slice)
    const int owner = row / p.rs_rows_per_rank, local = row - owner * p.rs_rows_per_rank;
    if (owner != p.rs_rank) {
      store_chunk_to(p, p.rs_stage[owner], p.rs_rank * p.rs_rows_per_rank + local, col, r);   // slot of this rank
    } else {
      // own rows: add the peers' staged partials (the caller waited for their counters) and write the result
      float f[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) f[j] = 0.f;
      const bool full_chunk = (col + 32 <= p.N);
      for (int src = 0; src < p.rs_world; ++src) {
        if (src == p.rs_rank) {
#pragma unroll
          for (int j = 0; j < 32; ++j) f[j] += __uint_as_float(r[j]);
          continue;
        }
        const __nv_bfloat16* sp = static_cast<const __nv_bfloat16*>(p.rs_stage[p.rs_rank]) +
                                  (static_cast<long long>(src) * p.rs_rows_per_rank + local) * p.N + col;
        if (full_chunk) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint4 v = __ldcv(reinterpret_cast<const uint4*>(sp) + j);
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 x = __bfloat1622float2(h[e]);
              f[8 * j + 2 * e] += x.x;
              f[8 * j + 2 * e + 1] += x.y;
            }
          }
        } else {
          for (int j = 0; j < 32 && col + j < p.N; ++j) f[j] += __bfloat162float(sp[j]);
        }
      }
      uint32_t o[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) o[j] = __float_as_uint(f[j]);
      store_chunk_to(p, p.rs_out, local, col, o);
    }
  } else {
    store_chunk_to(p, p.C, row, col, r);
  }
}

__device__ __forceinline__ void store_chunk_to(const GemmArgs& p, void* Cbase, int row, int col, const uint32_t (&r)[32]) {
  const bool full_chunk = (col + 32 <= p.N);
        if (p.c_fp32) {
          float* dst = reinterpret_cast<float*>(Cbase) + static_cast<long long>(row) * p.ldc + col;
          if (full_chunk && (p.ldc % 4 == 0)) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              float4 v = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                     __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
              float4* q = reinterpret_cast<float4*>(dst) + j;
              if (p.accumulate) {
                float4 o = *q;
                v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
              }
              *q = v;
            }
          } else {
            for (int j = 0; j < 32 && col + j < p.N; ++j)
              dst[j] = __uint_as_float(r[j]) + (p.accumulate ? dst[j] : 0.f);
          }
        } else {
          __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(Cbase) + static_cast<long long>(row) * p.ldc + col;
          const __nv_bfloat16* add = p.R ? reinterpret_cast<const __nv_bfloat16*>(p.R) + static_cast<long long>(row) * p.ldr + col
                                         : dst;
          if (full_chunk && (p.ldc % 8 == 0) && (p.ldr % 8 == 0)) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4* q = reinterpret_cast<uint4*>(dst) + j;
              float f[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[8 * j + e]);
              if (p.accumulate) {
                uint4 o = *(reinterpret_cast<const uint4*>(add) + j);
                const __nv_bfloat162* ob = reinterpret_cast<const __nv_bfloat162*>(&o);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  float2 of = __bfloat1622float2(ob[e]);
                  f[2 * e] += of.x;
                  f[2 * e + 1] += of.y;
                }
              }
              uint4 v;
              v.x = tt::pack_bf16(f[0], f[1]);
              v.y = tt::pack_bf16(f[2], f[3]);
              v.z = tt::pack_bf16(f[4], f[5]);
              v.w = tt::pack_bf16(f[6], f[7]);
              *q = v;
            }
          } else {
            for (int j = 0; j < 32 && col + j < p.N; ++j) {
              float v = __uint_as_float(r[j]);
              if (p.accumulate) v += __bfloat162float(add[j]);
              dst[j] = __float2bfloat16(v);
            }
          }
        }
}

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(int* p, int v) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Reduce-scatter epilogue, once per (epilogue warp, output tile) before its stores. Rows owned by this rank: wait
// (bounded) until every peer's counter for this panel and column tile reached the target, so that their staged partials
// are visible. Returns false when the wait ran out (the error word is set; the tile's result is not meaningful).
__device__ __forceinline__ bool rs_begin(const GemmArgs& p, int first_row, int tn) {
  const int owner = first_row / p.rs_rows_per_rank;
  if (owner != p.rs_rank) return true;
  const int panel = (first_row - owner * p.rs_rows_per_rank) / BM;
  const int panels = p.rs_rows_per_rank / BM;
  const int lane = threadIdx.x & 31;
  int ok = 1;
  if (lane < p.rs_world && lane != p.rs_rank) {
    const int* c = p.rs_count[p.rs_rank] + (lane * panels + panel) * p.rs_tiles_n + tn;
    const uint64_t t0 = tt::globaltimer_ns();
    while (ld_acquire_sys(c) < p.rs_target) {
      if (tt::globaltimer_ns() - t0 > TT_WAIT_LIMIT_NS) { atomicCAS(&g_gemm_error, 0, 8); ok = 0; break; }
      __nanosleep(200);
    }
  }
  ok = __all_sync(0xffffffffu, ok);
  return ok != 0;
}

// ... and once after them. Rows owned by a peer: make the stores visible system-wide, then bump the owner's counter.
__device__ __forceinline__ void rs_end(const GemmArgs& p, int first_row, int tn) {
  const int owner = first_row / p.rs_rows_per_rank;
  if (owner == p.rs_rank) return;
  const int panel = (first_row - owner * p.rs_rows_per_rank) / BM;
  const int panels = p.rs_rows_per_rank / BM;
  __threadfence_system();
  __syncwarp();
  if ((threadIdx.x & 31) == 0)
    atomicAdd_system(p.rs_count[owner] + (p.rs_rank * panels + panel) * p.rs_tiles_n + tn, 1);
}

// Contribute-only launches leave out the tiles of this rank's own rows (all roles skip the same tiles).
__device__ __forceinline__ bool rs_skip_tile(const GemmArgs& p, int first_row) {
  return p.rs_skip_own && first_row / p.rs_rows_per_rank == p.rs_rank;
}

// Copy role of the fused all-gather GEMM. Copy CTA `c` handles panels c, c + copy_ctas, ... of a list that starts with
// the owner next to this rank, so that traffic is spread over the peers. A panel of the local slice needs no copy.
// One thread drives a ring of bulk copies through shared memory (peer memory -> smem -> local memory, GATHER_BUFS chunks
// of GATHER_CHUNK bytes in flight), which keeps far more bytes in flight per SM than register copies; plain (non-
// multicast) bulk loads. Bounded waits: on expiry the error word is set and the panel is left unpublished, which makes
// the consuming GEMM CTAs give up through their own bounded waits.
constexpr uint32_t GATHER_CHUNK = 32768;
constexpr int GATHER_BUFS = 5;   // 160 KB of the CTA's dynamic shared memory (+ barriers)

__device__ void gather_panels(const GemmArgs& p, int c, uint8_t* smem_raw) {
  const uint32_t base = (tt::smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bars = base + GATHER_BUFS * GATHER_CHUNK;
  auto bar = [&](int i) { return bars + 8u * i; };
  if (threadIdx.x != 0) return;           // a single thread issues everything
  for (int i = 0; i < GATHER_BUFS; ++i) tt::mbar_init(bar(i), 1);
  tt::mbar_fence_init();
  int abort_local = 0;
  uint32_t issued = 0;                    // chunks issued so far (ring position / phase)
  const int total = p.panels_per_rank * p.gather_world;
  const uint32_t chunks = static_cast<uint32_t>((p.panel_bytes + GATHER_CHUNK - 1) / GATHER_CHUNK);
  for (int i = c; i < total; i += p.copy_ctas) {
    const int hop = i / p.panels_per_rank;                       // 0 = local slice
    const int owner = (p.gather_rank + hop) % p.gather_world;
    const int panel = owner * p.panels_per_rank + i % p.panels_per_rank;
    if (hop != 0) {
      const uint64_t t0 = tt::globaltimer_ns();
      while (ld_acquire_sys(p.gather_flag[owner]) < p.gather_expected) {
        if (tt::globaltimer_ns() - t0 > TT_WAIT_LIMIT_NS) { atomicCAS(&g_gemm_error, 0, 6); return; }
        __nanosleep(500);
      }
      const uint8_t* src = static_cast<const uint8_t*>(p.gather_src[owner]) + panel * p.panel_bytes;
      uint8_t* dst = static_cast<uint8_t*>(p.gather_dst) + panel * p.panel_bytes;
      // software pipeline: loads run GATHER_BUFS - 1 chunks ahead of the stores
      uint32_t loaded = 0, stored = 0;
      const uint32_t first = issued;
      while (stored < chunks) {
        while (loaded < chunks && loaded - stored < GATHER_BUFS) {
          const uint32_t slot = (first + loaded) % GATHER_BUFS;
          // the bulk store that last read this slot must have finished reading shared memory
          if (first + loaded >= GATHER_BUFS) tt::bulk_store_wait_read<GATHER_BUFS - 1>();
          const long long off = static_cast<long long>(loaded) * GATHER_CHUNK;
          const uint32_t bytes = static_cast<uint32_t>(min(static_cast<long long>(GATHER_CHUNK), p.panel_bytes - off));
          tt::mbar_expect_tx(bar(slot), bytes);
          tt::bulk_load(base + slot * GATHER_CHUNK, src + off, bytes, bar(slot));
          ++loaded;
        }
        const uint32_t slot = (first + stored) % GATHER_BUFS;
        const uint32_t ph = ((first + stored) / GATHER_BUFS) & 1;
        if (!tt::mbar_wait(bar(slot), ph, &abort_local, &g_gemm_error, 7)) return;
        const long long off = static_cast<long long>(stored) * GATHER_CHUNK;
        const uint32_t bytes = static_cast<uint32_t>(min(static_cast<long long>(GATHER_CHUNK), p.panel_bytes - off));
        tt::fence_proxy_async();
        tt::bulk_store(dst + off, base + slot * GATHER_CHUNK, bytes);
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        ++stored;
      }
      issued = first + chunks;
      tt::bulk_store_wait_all();          // writes of this panel are complete before it is published
      __threadfence();
    }
    st_release_gpu(p.panel_ready + panel, p.ready_value);
  }
}

template <bool FP8, bool RS = false>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, GemmArgs p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (tt::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - tt::smem_u32(smem_raw));
  const uint32_t sA = base;
  const uint32_t sB = base + STAGES * A_STAGE_BYTES;
  const uint32_t bars = base + STAGES * (A_STAGE_BYTES + B_STAGE_BYTES);
  uint8_t* bars_gen = gen_base + STAGES * (A_STAGE_BYTES + B_STAGE_BYTES);
  // barrier layout (8 bytes each): full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2]
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bars + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bars + 8u * (2 * STAGES + 2 + a); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars_gen + 8 * (2 * STAGES + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars_gen + 8 * (2 * STAGES + 4) + 8);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int gemm_ctas = static_cast<int>(gridDim.x) - p.copy_ctas;

  if (static_cast<int>(blockIdx.x) >= gemm_ctas) {
    gather_panels(p, static_cast<int>(blockIdx.x) - gemm_ctas, smem_raw);
    return;
  }

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      tt::mbar_init(full_bar(s), 1);
      tt::mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      tt::mbar_init(tfull_bar(a), 1);
      tt::mbar_init(tempty_bar(a), 4);  // one arrival per epilogue warp
    }
    *abort_flag = 0;
    tt::mbar_fence_init();
    tt::tma_prefetch_desc(&tma_a);
    tt::tma_prefetch_desc(&tma_b);
  }
  if (warp == 2) {
    tt::tmem_alloc(tt::smem_u32(tmem_slot), TMEM_COLS);
    tt::tmem_relinquish();
  }
  tt::tc_fence_before();
  __syncthreads();
  tt::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (tt::elect_one()) {
      uint32_t it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gemm_ctas) {
        int tm, tn;
        tile_coords_p(p, t, tm, tn);
        if (RS && rs_skip_tile(p, tm * BM)) continue;
        if (p.ready_flags != nullptr) {
          // fused all-gather: wait until the copy CTAs have landed this n-tile of B locally
          uint64_t t0 = tt::globaltimer_ns();
          while (ld_acquire_gpu(p.ready_flags + (p.flags_by_m ? tm : tn)) < p.ready_value) {
            if (*abort_flag || tt::globaltimer_ns() - t0 > TT_WAIT_LIMIT_NS) {
              *abort_flag = 1;
              atomicCAS(&g_gemm_error, 0, 5);
              ok = false;
              break;
            }
            __nanosleep(200);
          }
          if (!ok) break;
          __threadfence();
        }
        for (int k = 0; k < p.k_iters; ++k, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!tt::mbar_wait(empty_bar(s), ph ^ 1, abort_flag, &g_gemm_error, 1)) { ok = false; break; }
          tt::mbar_expect_tx(full_bar(s), A_STAGE_BYTES + B_STAGE_BYTES);
          const uint32_t dA = sA + s * A_STAGE_BYTES, dB = sB + s * B_STAGE_BYTES;
          if (!p.a_mn) {
            tt::tma_load_2d(dA, &tma_a, full_bar(s), k * (FP8 ? 128 : BK), tm * BM);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tt::tma_load_2d(dA + j * (64 * BK * 2), &tma_a, full_bar(s), tm * BM + j * 64, k * BK);
          }
          if (!p.b_mn) {
            tt::tma_load_2d(dB, &tma_b, full_bar(s), k * (FP8 ? 128 : BK), tn * BN);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tt::tma_load_2d(dB + j * (64 * BK * 2), &tma_b, full_bar(s), tn * BN + j * 64, k * BK);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ UMMA issuer
    if (tt::elect_one()) {
      uint32_t it = 0, tile_it = 0;
      bool ok = true;
      // descriptor geometry per operand layout
      const uint32_t a_lbo = p.a_mn ? (64 * BK * 2) >> 4 : 1, b_lbo = p.b_mn ? (64 * BK * 2) >> 4 : 1;
      const uint32_t sbo = 1024 >> 4;
      const uint32_t a_kadv = p.a_mn ? (UMMA_K * 128) : (UMMA_K * 2);  // bytes per 16-wide k step
      const uint32_t b_kadv = p.b_mn ? (UMMA_K * 128) : (UMMA_K * 2);
      for (int t = blockIdx.x; t < num_tiles && ok; t += gemm_ctas, ++tile_it) {
        if (RS && p.rs_skip_own) {
          int tm, tn;
          tile_coords_p(p, t, tm, tn);
          if (rs_skip_tile(p, tm * BM)) { --tile_it; continue; }
        }
        const int acc = tile_it & 1;
        const uint32_t acc_ph = (tile_it >> 1) & 1;
        if (!tt::mbar_wait(tempty_bar(acc), acc_ph ^ 1, abort_flag, &g_gemm_error, 2)) break;
        tt::tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int k = 0; k < p.k_iters; ++k, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!tt::mbar_wait(full_bar(s), ph, abort_flag, &g_gemm_error, 3)) { ok = false; break; }
          tt::tc_fence_after();
          const uint32_t aA = sA + s * A_STAGE_BYTES, aB = sB + s * B_STAGE_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            const uint64_t ad = tt::umma_smem_desc(aA + kk * a_kadv, a_lbo, sbo);
            const uint64_t bd = tt::umma_smem_desc(aB + kk * b_kadv, b_lbo, sbo);
            if constexpr (FP8) tt::umma_f8_ss(d_tmem, ad, bd, p.idesc, (k | kk) != 0);
            else tt::umma_f16_ss(d_tmem, ad, bd, p.idesc, (k | kk) != 0);
          }
          tt::umma_commit(empty_bar(s));  // frees the stage once these UMMAs have read it
        }
        if (ok) tt::umma_commit(tfull_bar(acc));
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------ epilogue (TMEM -> registers -> global)
    const int ew = warp - 4;  // TMEM lanes [32*ew, 32*ew+32)
    uint32_t tile_it = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gemm_ctas, ++tile_it) {
      int tm, tn;
      tile_coords_p(p, t, tm, tn);
      if (RS && rs_skip_tile(p, tm * BM)) { --tile_it; continue; }
      const int acc = tile_it & 1;
      const uint32_t acc_ph = (tile_it >> 1) & 1;
      if (!tt::mbar_wait(tfull_bar(acc), acc_ph, abort_flag, &g_gemm_error, 4)) break;
      tt::tc_fence_after();
      const int row = tm * BM + ew * 32 + lane;
      const int n0 = tn * BN;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(ew * 32) << 16) + acc * BN;
      const bool row_ok = row < p.M;
      float sa = 1.f;
      if constexpr (FP8) {
        if (p.scale_mode == 1) sa = __ldg(p.scale_a) * __ldg(p.scale_b);
        else if (p.scale_mode == 2 && row_ok) sa = __ldg(p.scale_a + row);
      }
      if constexpr (RS) rs_begin(p, tm * BM, tn);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tt::tmem_ld_32x32(taddr + c * 32, r);
        tt::tc_wait_ld();
        const int col = n0 + c * 32;
        if (!row_ok || col >= p.N) continue;
        if constexpr (FP8) { if (p.scale_mode) apply_scales(p, sa, col, r); }
        store_chunk<RS>(p, row, col, r);
      }
      if constexpr (RS) rs_end(p, tm * BM, tn);
      tt::tc_fence_before();
      __syncwarp();
      if (lane == 0) tt::mbar_arrive(tempty_bar(acc));
    }
  }

  // ------------------------------------------------------------ teardown
  __syncthreads();
  if (*abort_flag) tt::abort_drain();
  if (warp == 2) {
    tt::tc_fence_after();
    tt::tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------------------------
// CTA-pair variant: two CTAs on neighbouring SMs share one 256x256 output tile. Each CTA stages its
// own 128 rows of A and *half* of the B tile; one UMMA (M = 256) issued by the leader reads both
// halves, so every CTA moves 32 KB instead of 48 KB per k-step from L2 and the ring gets 6 stages.
// Accumulators: each CTA's TMEM holds its 128 rows x 256 columns (two buffers).
namespace pair {
constexpr int TM = 256, TN = 256;
constexpr int PSTAGES = 6;
constexpr uint32_t PA_BYTES = 128 * BK * 2, PB_BYTES = 128 * BK * 2;  // per CTA per stage
constexpr size_t PSMEM_BYTES = 1024 + PSTAGES * (PA_BYTES + PB_BYTES) + 256;
// The fused reduce-scatter stages the rows it sends to a peer in shared memory (32 rows x 128 columns bf16 per epilogue
// warp, 16-byte columns XOR-swizzled by the row) so that every warp-wide store covers two whole 256-byte row segments:
// NVLink then carries full packets instead of one 16-byte write per lane.
constexpr uint32_t RS_STAGE_PER_WARP = 32 * 256;
constexpr size_t PSMEM_RS_BYTES = PSMEM_BYTES + 4 * RS_STAGE_PER_WARP;

template <bool FP8, bool RS = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, GemmArgs p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (tt::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - tt::smem_u32(smem_raw));
  const uint32_t sA = base, sB = base + PSTAGES * PA_BYTES;
  const uint32_t bars = base + PSTAGES * (PA_BYTES + PB_BYTES);
  uint8_t* bars_gen = gen_base + PSTAGES * (PA_BYTES + PB_BYTES);
  auto full_bar = [&](int s) { return bars + 8u * s; };                       // used in the leader only
  auto empty_bar = [&](int s) { return bars + 8u * (PSTAGES + s); };          // one per CTA
  auto tfull_bar = [&](int a) { return bars + 8u * (2 * PSTAGES + a); };      // one per CTA
  auto tempty_bar = [&](int a) { return bars + 8u * (2 * PSTAGES + 2 + a); }; // used in the leader only
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars_gen + 8 * (2 * PSTAGES + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars_gen + 8 * (2 * PSTAGES + 4) + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = tt::cluster_ctarank();  // 0 = leader
  const int num_tiles = p.tiles_m * p.tiles_n;  // in 256x256 tiles
  const int cluster_id = blockIdx.x >> 1;
  const int num_clusters = (static_cast<int>(gridDim.x) - p.copy_ctas) >> 1;   // clusters that multiply

  if (cluster_id >= num_clusters) {
    // fused all-gather: the trailing clusters only move data (both CTAs), see gather_panels
    gather_panels(p, static_cast<int>(blockIdx.x) - 2 * num_clusters, smem_raw);
    return;
  }

  if (threadIdx.x == 0) {
    for (int s = 0; s < PSTAGES; ++s) { tt::mbar_init(full_bar(s), 1); tt::mbar_init(empty_bar(s), 1); }
    for (int a = 0; a < 2; ++a) { tt::mbar_init(tfull_bar(a), 1); tt::mbar_init(tempty_bar(a), 8); }
    *abort_flag = 0;
    tt::mbar_fence_init();
    tt::tma_prefetch_desc(&tma_a);
    tt::tma_prefetch_desc(&tma_b);
  }
  if (warp == 2) { tt::tmem_alloc_pair(tt::smem_u32(tmem_slot), TMEM_COLS); tt::tmem_relinquish_pair(); }
  tt::tc_fence_before();
  tt::cluster_sync();  // barriers of both CTAs are initialised before anyone signals across
  tt::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (tt::elect_one()) {
      uint32_t it = 0;
      bool ok = true;
      for (int t = cluster_id; t < num_tiles && ok; t += num_clusters) {
        int tm, tn;
        tile_coords_p(p, t, tm, tn);
        if (RS && rs_skip_tile(p, tm * TM)) continue;
        const int m0 = tm * TM + rank * 128, n0 = tn * TN + rank * 128;
        if (p.ready_flags != nullptr) {
          // fused all-gather of A: this CTA's 128 rows are panel 2 * tm + rank
          const uint64_t t0 = tt::globaltimer_ns();
          while (ld_acquire_gpu(p.ready_flags + 2 * tm + static_cast<int>(rank)) < p.ready_value) {
            if (*abort_flag || tt::globaltimer_ns() - t0 > TT_WAIT_LIMIT_NS) {
              *abort_flag = 1;
              atomicCAS(&g_gemm_error, 0, 5);
              ok = false;
              break;
            }
            __nanosleep(200);
          }
          if (!ok) break;
        }
        for (int k = 0; k < p.k_iters; ++k, ++it) {
          const int s = it % PSTAGES;
          const uint32_t ph = (it / PSTAGES) & 1;
          if (!tt::mbar_wait(empty_bar(s), ph ^ 1, abort_flag, &g_gemm_error, 11)) { ok = false; break; }
          const uint32_t fb = tt::mapa(full_bar(s), 0);  // the leader's barrier collects both CTAs' bytes
          if (rank == 0) tt::mbar_expect_tx(full_bar(s), 2 * (PA_BYTES + PB_BYTES));
          const uint32_t dA = sA + s * PA_BYTES, dB = sB + s * PB_BYTES;
          if (!p.a_mn) {
            tt::tma_load_2d_pair(dA, &tma_a, fb, k * (FP8 ? 128 : BK), m0);
          } else {
#pragma unroll
            for (int j = 0; j < 2; ++j) tt::tma_load_2d_pair(dA + j * (64 * BK * 2), &tma_a, fb, m0 + j * 64, k * BK);
          }
          if (!p.b_mn) {
            tt::tma_load_2d_pair(dB, &tma_b, fb, k * (FP8 ? 128 : BK), n0);
          } else {
#pragma unroll
            for (int j = 0; j < 2; ++j) tt::tma_load_2d_pair(dB + j * (64 * BK * 2), &tma_b, fb, n0 + j * 64, k * BK);
          }
        }
      }
    }
  } else if (warp == 1 && rank == 0) {
    // ------------------------------------------------------------ UMMA issuer (leader CTA only)
    if (tt::elect_one()) {
      uint32_t it = 0, tile_it = 0;
      bool ok = true;
      const uint32_t a_lbo = p.a_mn ? (64 * BK * 2) >> 4 : 1, b_lbo = p.b_mn ? (64 * BK * 2) >> 4 : 1;
      const uint32_t sbo = 1024 >> 4;
      const uint32_t a_kadv = p.a_mn ? (UMMA_K * 128) : (UMMA_K * 2);
      const uint32_t b_kadv = p.b_mn ? (UMMA_K * 128) : (UMMA_K * 2);
      for (int t = cluster_id; t < num_tiles && ok; t += num_clusters, ++tile_it) {
        if (RS && p.rs_skip_own) {
          int tm, tn;
          tile_coords_p(p, t, tm, tn);
          if (rs_skip_tile(p, tm * TM)) { --tile_it; continue; }
        }
        const int acc = tile_it & 1;
        const uint32_t acc_ph = (tile_it >> 1) & 1;
        if (!tt::mbar_wait(tempty_bar(acc), acc_ph ^ 1, abort_flag, &g_gemm_error, 12)) break;
        tt::tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * TN;
        for (int k = 0; k < p.k_iters; ++k, ++it) {
          const int s = it % PSTAGES;
          const uint32_t ph = (it / PSTAGES) & 1;
          if (!tt::mbar_wait(full_bar(s), ph, abort_flag, &g_gemm_error, 13)) { ok = false; break; }
          tt::tc_fence_after();
          const uint32_t aA = sA + s * PA_BYTES, aB = sB + s * PB_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            const uint64_t ad = tt::umma_smem_desc(aA + kk * a_kadv, a_lbo, sbo);
            const uint64_t bd = tt::umma_smem_desc(aB + kk * b_kadv, b_lbo, sbo);
            if constexpr (FP8) tt::umma_f8_ss_pair(d_tmem, ad, bd, p.idesc, (k | kk) != 0);
            else tt::umma_f16_ss_pair(d_tmem, ad, bd, p.idesc, (k | kk) != 0);
          }
          tt::umma_commit_pair(empty_bar(s), 3);  // frees this stage in both CTAs
        }
        if (ok) tt::umma_commit_pair(tfull_bar(acc), 3);
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------ epilogue (both CTAs, own 128 rows)
    const int ew = warp - 4;
    uint32_t tile_it = 0;
    const uint32_t leader_tempty0 = tt::mapa(tempty_bar(0), 0), leader_tempty1 = tt::mapa(tempty_bar(1), 0);
    for (int t = cluster_id; t < num_tiles; t += num_clusters, ++tile_it) {
      int tm, tn;
      tile_coords_p(p, t, tm, tn);
      if (RS && rs_skip_tile(p, tm * TM)) { --tile_it; continue; }
      const int acc = tile_it & 1;
      const uint32_t acc_ph = (tile_it >> 1) & 1;
      if (!tt::mbar_wait(tfull_bar(acc), acc_ph, abort_flag, &g_gemm_error, 14)) break;
      tt::tc_fence_after();
      const int row = tm * TM + rank * 128 + ew * 32 + lane;
      const int n0 = tn * TN;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(ew * 32) << 16) + acc * TN;
      const bool row_ok = row < p.M;
      float sa = 1.f;
      if constexpr (FP8) {
        if (p.scale_mode == 1) sa = __ldg(p.scale_a) * __ldg(p.scale_b);
        else if (p.scale_mode == 2 && row_ok) sa = __ldg(p.scale_a + row);
      }
      if constexpr (RS) rs_begin(p, tm * TM + static_cast<int>(rank) * 128, tn);
      bool staged = false;
      if constexpr (RS) {
        const int first_row = tm * TM + static_cast<int>(rank) * 128;
        const int owner = first_row / p.rs_rows_per_rank;
        if (owner != p.rs_rank) {
          // rows of a peer: TMEM -> bf16 -> swizzled shared memory -> row-contiguous stores into the owner's staging slot
          staged = true;
          uint8_t* stg = bars_gen + 256 + ew * RS_STAGE_PER_WARP;
          const int local0 = first_row - owner * p.rs_rows_per_rank + ew * 32;   // first of this warp's 32 rows
          __nv_bfloat16* dst_base = static_cast<__nv_bfloat16*>(p.rs_stage[owner]) +
                                    (static_cast<long long>(p.rs_rank) * p.rs_rows_per_rank + local0) * p.N;
#pragma unroll 1
          for (int half = 0; half < 2; ++half) {
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
              uint32_t r[32];
              tt::tmem_ld_32x32(taddr + half * 128 + c * 32, r);
              tt::tc_wait_ld();
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                uint4 q;
                q.x = tt::pack_bf16(__uint_as_float(r[8 * v + 0]), __uint_as_float(r[8 * v + 1]));
                q.y = tt::pack_bf16(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3]));
                q.z = tt::pack_bf16(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5]));
                q.w = tt::pack_bf16(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7]));
                const int c16 = c * 4 + v;
                *reinterpret_cast<uint4*>(stg + lane * 256 + ((c16 ^ (lane & 7)) << 4)) = q;
              }
            }
            __syncwarp();
            const int c16 = lane & 15;
            const int gcol = n0 + half * 128 + c16 * 8;
#pragma unroll 4
            for (int r2 = 0; r2 < 16; ++r2) {
              const int rr = r2 * 2 + (lane >> 4);
              const uint4 q = *reinterpret_cast<const uint4*>(stg + rr * 256 + ((c16 ^ (rr & 7)) << 4));
              if (gcol < p.N) *reinterpret_cast<uint4*>(dst_base + static_cast<long long>(rr) * p.N + gcol) = q;
            }
            __syncwarp();
          }
        }
      }
      if (!staged) {
#pragma unroll 1
        for (int c = 0; c < TN / 32; ++c) {
          uint32_t r[32];
          tt::tmem_ld_32x32(taddr + c * 32, r);
          tt::tc_wait_ld();
          const int col = n0 + c * 32;
          if (!row_ok || col >= p.N) continue;
          if constexpr (FP8) { if (p.scale_mode) apply_scales(p, sa, col, r); }
          store_chunk<RS>(p, row, col, r);
        }
      }
      if constexpr (RS) rs_end(p, tm * TM + static_cast<int>(rank) * 128, tn);
      tt::tc_fence_before();
      __syncwarp();
      if (lane == 0) tt::mbar_arrive_cluster(acc ? leader_tempty1 : leader_tempty0);
    }
  }

  __syncthreads();
  if (*abort_flag) tt::abort_drain();
  tt::cluster_sync();  // nobody leaves while its partner may still touch its shared memory or TMEM
  if (warp == 2) { tt::tc_fence_after(); tt::tmem_dealloc_pair(tmem_base, TMEM_COLS); }
}
}  // namespace pair

int g_num_sms = 0;
bool g_pair_enabled = true;
int g_rs_interleave = -1;   // -1: by the burst estimate, 0 / 1: forced (tests)

void set_kernel_attrs() {
  cudaFuncSetAttribute(gemm_bf16_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(SMEM_BYTES));
  cudaFuncSetAttribute(gemm_bf16_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(SMEM_BYTES));
  cudaFuncSetAttribute(pair::gemm_bf16_pair_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(pair::PSMEM_BYTES));
  cudaFuncSetAttribute(pair::gemm_bf16_pair_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(pair::PSMEM_BYTES));
  cudaFuncSetAttribute(gemm_bf16_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(SMEM_BYTES));
  cudaFuncSetAttribute(pair::gemm_bf16_pair_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(pair::PSMEM_RS_BYTES));
}

}  // namespace

extern "C" {

// A: [M,K] (a_mn=0, row stride lda) or stored transposed [K,M] (a_mn=1). Same for B with N.
// Returns 0 on success, a negative number on invalid arguments / descriptor failures.
static int gemm_bf16_launch(const void* A, const void* B, void* C, int M, int N, int K, int a_mn, long long lda, int b_mn,
                            long long ldb, long long ldc, int c_fp32, int accumulate, const int* ready_flags, int ready_value,
                            int max_ctas, const void* R, long long ldr, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 8) || (ldb % 8)) return -2;  // TMA needs 16-byte row strides
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return -3;
  if (R && (c_fp32 || (reinterpret_cast<uintptr_t>(R) & 15) || (reinterpret_cast<uintptr_t>(C) & 15))) return -3;
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
    set_kernel_attrs();
  }
  // CTA-pair kernel for everything large enough to fill 256x256 tiles (no fused-gather flags there)
  const bool use_pair = g_pair_enabled && ready_flags == nullptr && M >= 256 && N >= 256;
  const int box_n = use_pair ? 128 : BN;
  CUtensorMap ta, tb;
  int rc;
  if (!a_mn) rc = tt::make_tmap_2d(&ta, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, lda, BM, BK);
  else       rc = tt::make_tmap_2d(&ta, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, M, lda, BK, 64);
  if (rc) return rc;
  if (!b_mn) rc = tt::make_tmap_2d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, ldb, box_n, BK);
  else       rc = tt::make_tmap_2d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, ldb, BK, 64);
  if (rc) return rc;
  GemmArgs p;
  p.M = M; p.N = N; p.K = K;
  p.k_iters = (K + BK - 1) / BK;
  p.a_mn = a_mn; p.b_mn = b_mn;
  p.C = C; p.ldc = ldc; p.c_fp32 = c_fp32; p.accumulate = accumulate; p.R = nullptr; p.ldr = 0;
  if (R) { p.accumulate = 1; p.R = R; p.ldr = ldr; }
  p.ready_flags = ready_flags; p.ready_value = ready_value;
  p.fp8 = 0; p.bk = BK; p.scale_mode = 0; p.scale_a = p.scale_b = nullptr;
  p.flags_by_m = 0; p.m_rot = 0; p.copy_ctas = 0; p.panel_ready = nullptr; p.rs_world = 0;
  int cap = (max_ctas > 0 && max_ctas < g_num_sms) ? max_ctas : g_num_sms;
  if (use_pair) {
    p.tiles_m = (M + pair::TM - 1) / pair::TM;
    p.m_block = p.tiles_m; p.m_interleave = 0;
    p.tiles_n = (N + pair::TN - 1) / pair::TN;
    p.idesc = tt::umma_idesc_bf16(pair::TM, pair::TN, a_mn, b_mn);
    int clusters = p.tiles_m * p.tiles_n;
    if (clusters > cap / 2) clusters = cap / 2;
    if (clusters < 1) clusters = 1;
    pair::gemm_bf16_pair_kernel<false><<<clusters * 2, NUM_THREADS, pair::PSMEM_BYTES, stream>>>(ta, tb, p);
  } else {
    p.tiles_m = (M + BM - 1) / BM;
    p.m_block = p.tiles_m; p.m_interleave = 0;
    p.tiles_n = (N + BN - 1) / BN;
    p.idesc = tt::umma_idesc_bf16(BM, BN, a_mn, b_mn);
    int grid = p.tiles_m * p.tiles_n;
    if (grid > cap) grid = cap;
    gemm_bf16_kernel<false><<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(ta, tb, p);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

int tt_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int a_mn, long long lda, int b_mn,
                 long long ldb, long long ldc, int c_fp32, int accumulate, const int* ready_flags, int ready_value,
                 int max_ctas, cudaStream_t stream) {
  return gemm_bf16_launch(A, B, C, M, N, K, a_mn, lda, b_mn, ldb, ldc, c_fp32, accumulate, ready_flags, ready_value, max_ctas,
                          nullptr, 0, stream);
}

// C[M,N] = A . B^T + R with R bf16 [M,N] (row stride ldr, 16-byte aligned): the residual connection of a transformer
// block folded into the epilogue of its output projection (saves the separate add: one read and one write of C).
int tt_gemm_bf16_res(const void* A, const void* B, void* C, const void* R, int M, int N, int K, int a_mn, long long lda,
                     int b_mn, long long ldb, long long ldc, long long ldr, cudaStream_t stream) {
  if (!R || (ldr % 8)) return -2;
  return gemm_bf16_launch(A, B, C, M, N, K, a_mn, lda, b_mn, ldb, ldc, 0, 0, nullptr, 0, 0, R, ldr, stream);
}

// C[M,N] = (A[M,K] . B[N,K]^T) * scales with 8-bit float operands (a_e5m2 / b_e5m2 select e5m2 instead of e4m3), both
// K-major with row strides lda / ldb in elements (multiples of 16), fp32 accumulation, C bf16 or fp32.
// scale_mode: 0 none, 1 per-tensor (scale_a, scale_b point to one float each), 2 per row of A / per row of B.
int tt_gemm_fp8(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb, long long ldc,
                int c_fp32, int a_e5m2, int b_e5m2, const float* scale_a, const float* scale_b, int scale_mode,
                cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 16) || (ldb % 16)) return -2;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return -3;
  if (scale_mode && (!scale_a || !scale_b)) return -5;
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
    set_kernel_attrs();
  }
  constexpr int BK8 = 128;  // one 128-byte swizzle row of 8-bit elements
  const bool use_pair = g_pair_enabled && M >= 256 && N >= 256;
  CUtensorMap ta, tb;
  int rc = tt::make_tmap_2d(&ta, A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, K, lda, BM, BK8);
  if (rc) return rc;
  rc = tt::make_tmap_2d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, K, ldb, use_pair ? 128 : BN, BK8);
  if (rc) return rc;
  GemmArgs p;
  p.M = M; p.N = N; p.K = K;
  p.k_iters = (K + BK8 - 1) / BK8;
  p.a_mn = 0; p.b_mn = 0;
  p.C = C; p.ldc = ldc; p.c_fp32 = c_fp32; p.accumulate = 0; p.R = nullptr; p.ldr = 0;
  p.ready_flags = nullptr; p.ready_value = 0;
  p.fp8 = 1; p.bk = BK8; p.scale_mode = scale_mode; p.scale_a = scale_a; p.scale_b = scale_b;
  p.flags_by_m = 0; p.m_rot = 0; p.copy_ctas = 0; p.panel_ready = nullptr; p.rs_world = 0;
  if (use_pair) {
    p.tiles_m = (M + pair::TM - 1) / pair::TM;
    p.m_block = p.tiles_m; p.m_interleave = 0;
    p.tiles_n = (N + pair::TN - 1) / pair::TN;
    p.idesc = tt::umma_idesc_f8(pair::TM, pair::TN, a_e5m2, b_e5m2);
    int clusters = p.tiles_m * p.tiles_n;
    if (clusters > g_num_sms / 2) clusters = g_num_sms / 2;
    pair::gemm_bf16_pair_kernel<true><<<clusters * 2, NUM_THREADS, pair::PSMEM_BYTES, stream>>>(ta, tb, p);
  } else {
    p.tiles_m = (M + BM - 1) / BM;
    p.m_block = p.tiles_m; p.m_interleave = 0;
    p.tiles_n = (N + BN - 1) / BN;
    p.idesc = tt::umma_idesc_f8(BM, BN, a_e5m2, b_e5m2);
    int grid = p.tiles_m * p.tiles_n;
    if (grid > g_num_sms) grid = g_num_sms;
    gemm_bf16_kernel<true><<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(ta, tb, p);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// Fused all-gather -> GEMM for sequence/tensor parallel: C[M,N] = A_full[M,K] . B[N,K]^T (or B stored [K,N] with b_mn)
// where A_full is the concatenation over `world` ranks of row slices of M/world rows. Every rank keeps a buffer of the
// full size at the same offset of its symmetric heap and has written its own slice; `peer_bufs[r]` is that buffer on rank
// r as mapped here, `peer_flags[r]` the version flag rank r sets once its slice is complete (>= expected).
// One launch: `copy_ctas` CTAs pull the remote slices panel by panel (128 rows) into `peer_bufs[rank]` while the
// remaining CTAs multiply, starting with the local panels; a tile waits only for its own panel.
// `panel_ready` is a local int array with M/128 entries; pass a `ready_value` larger than any used before.
int tt_gemm_allgather_a(const void* const* peer_bufs, const int* const* peer_flags, int world, int rank, int expected,
                        const void* B, void* C, int M, int N, int K, int b_mn, long long ldb, long long ldc, int c_fp32,
                        int* panel_ready, int ready_value, int copy_ctas, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (world < 1 || world > 16 || rank < 0 || rank >= world) return -6;
  if (M % (world * BM) || (K % 8) || (ldb % 8)) return -2;
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
    set_kernel_attrs();
  }
  void* A = const_cast<void*>(peer_bufs[rank]);
  // the CTA-pair kernel needs whole 256-row tiles inside one rank's slice
  const bool use_pair = g_pair_enabled && (M % (world * pair::TM) == 0) && N >= 256;
  CUtensorMap ta, tb;
  int rc = tt::make_tmap_2d(&ta, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, K, BM, BK);
  if (rc) return rc;
  if (!b_mn) rc = tt::make_tmap_2d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, ldb, use_pair ? 128 : BN, BK);
  else       rc = tt::make_tmap_2d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, ldb, BK, 64);
  if (rc) return rc;
  GemmArgs p;
  p.M = M; p.N = N; p.K = K;
  p.k_iters = (K + BK - 1) / BK;
  p.a_mn = 0; p.b_mn = b_mn;
  p.C = C; p.ldc = ldc; p.c_fp32 = c_fp32; p.accumulate = 0; p.R = nullptr; p.ldr = 0;
  p.fp8 = 0; p.bk = BK; p.scale_mode = 0; p.scale_a = p.scale_b = nullptr;
  p.ready_flags = panel_ready; p.ready_value = ready_value; p.panel_ready = panel_ready;
  p.flags_by_m = 1; p.rs_world = 0;
  p.panels_per_rank = M / BM / world;
  p.gather_world = world; p.gather_rank = rank; p.gather_expected = expected;
  p.gather_dst = A;
  p.panel_bytes = static_cast<long long>(BM) * K * 2;
  for (int r = 0; r < 16; ++r) { p.gather_src[r] = r < world ? peer_bufs[r] : nullptr; p.gather_flag[r] = r < world ? peer_flags[r] : nullptr; }
  if (copy_ctas < 2) copy_ctas = 2;
  copy_ctas &= ~1;
  if (copy_ctas > g_num_sms / 2) copy_ctas = (g_num_sms / 2) & ~1;
  p.copy_ctas = copy_ctas;
  // all CTAs must be co-resident (GEMM CTAs wait on flags written by copy CTAs): one CTA per SM, grid <= SM count
  if (use_pair) {
    p.tiles_m = M / pair::TM;
    p.m_block = p.tiles_m; p.m_interleave = 0;
    p.tiles_n = (N + pair::TN - 1) / pair::TN;
    p.idesc = tt::umma_idesc_bf16(pair::TM, pair::TN, 0, b_mn);
    p.m_rot = rank * (p.panels_per_rank / 2);
    int clusters = p.tiles_m * p.tiles_n;
    if (clusters > (g_num_sms - p.copy_ctas) / 2) clusters = (g_num_sms - p.copy_ctas) / 2;
    pair::gemm_bf16_pair_kernel<false><<<clusters * 2 + p.copy_ctas, NUM_THREADS, pair::PSMEM_BYTES, stream>>>(ta, tb, p);
  } else {
    p.tiles_m = M / BM;
    p.m_block = p.tiles_m; p.m_interleave = 0;
    p.tiles_n = (N + BN - 1) / BN;
    p.idesc = tt::umma_idesc_bf16(BM, BN, 0, b_mn);
    p.m_rot = rank * p.panels_per_rank;
    int gemm_ctas = p.tiles_m * p.tiles_n;
    if (gemm_ctas > g_num_sms - p.copy_ctas) gemm_ctas = g_num_sms - p.copy_ctas;
    gemm_bf16_kernel<false><<<gemm_ctas + p.copy_ctas, NUM_THREADS, SMEM_BYTES, stream>>>(ta, tb, p);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// Fused GEMM -> reduce-scatter for row-parallel layers: every rank computes the partial product P = A[M,K] . B[N,K]^T (or
// B stored [K,N] with b_mn) of its K-shard; rank r ends up with sum over ranks of P[r*M/world : (r+1)*M/world] in
// `out` [M/world, N] bf16. `stages[r]` / `counts[r]` are rank r's staging buffer ([world][M/world][N] bf16) and counters
// ([world][M/world/128][ceil(N/256)] int32, zero at allocation, never reset) as mapped here; `call_index` counts the
// calls made on these buffers (1, 2, ...) -- the same on every rank. Tiles owned by other ranks are computed first;
// `contribute_only` leaves this rank's own rows out (single-GPU emulation of several ranks, launch after launch).
int tt_gemm_reduce_scatter(const void* A, const void* B, void* const* stages, int* const* counts, void* out, int world,
                           int rank, int M, int N, int K, long long lda, int b_mn, long long ldb, int call_index,
                           int contribute_only, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (world < 1 || world > 16 || rank < 0 || rank >= world) return -6;
  if (M % (world * BM) || (N % 8) || (lda % 8) || (ldb % 8)) return -2;
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
    set_kernel_attrs();
  }
  const bool use_pair = g_pair_enabled && (M % (world * pair::TM) == 0) && N >= 256;
  CUtensorMap ta, tb;
  int rc = tt::make_tmap_2d(&ta, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, lda, BM, BK);
  if (rc) return rc;
  if (!b_mn) rc = tt::make_tmap_2d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, ldb, use_pair ? 128 : BN, BK);
  else       rc = tt::make_tmap_2d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, ldb, BK, 64);
  if (rc) return rc;
  GemmArgs p;
  p.M = M; p.N = N; p.K = K;
  p.k_iters = (K + BK - 1) / BK;
  p.a_mn = 0; p.b_mn = b_mn;
  p.C = nullptr; p.ldc = N; p.c_fp32 = 0; p.accumulate = 0; p.R = nullptr; p.ldr = 0;
  p.fp8 = 0; p.bk = BK; p.scale_mode = 0; p.scale_a = p.scale_b = nullptr;
  p.ready_flags = nullptr; p.ready_value = 0; p.panel_ready = nullptr; p.flags_by_m = 0;
  p.rs_world = world; p.rs_rank = rank; p.rs_out = out; p.rs_rows_per_rank = M / world;
  for (int r = 0; r < 16; ++r) { p.rs_stage[r] = r < world ? stages[r] : nullptr; p.rs_count[r] = r < world ? counts[r] : nullptr; }
  p.copy_ctas = 0;
  p.rs_skip_own = contribute_only;
  // Peer-owned tiles come first, so (world - 1) / world of the output crosses NVLink during the first part of the launch.
  // When that burst would need more than ~400 GB/s, interleave peer-owned and own tiles instead (own tile j then waits
  // for the peers' tile j, which they compute in the same round).
  {
    const double t_gemm = 2.0 * M * static_cast<double>(N) * K / 1.5e15;
    const double bytes = static_cast<double>(world - 1) / world * M * static_cast<double>(N) * 2.0;
    const bool burst = world > 1 && bytes / (t_gemm * (world - 1) / world) > 400e9;
    p.m_interleave = g_rs_interleave < 0 ? (burst ? 1 : 0) : g_rs_interleave;
  }
  p.rs_tiles_n = (N + 255) / 256;      // both tile kernels use 256 columns
  p.rs_target = call_index * 4;        // 4 epilogue warps store each (128-row panel, column tile)
  if (use_pair) {
    p.tiles_m = M / pair::TM;
    p.m_block = p.tiles_m;
    p.tiles_n = (N + pair::TN - 1) / pair::TN;
    p.idesc = tt::umma_idesc_bf16(pair::TM, pair::TN, 0, b_mn);
    p.m_block = p.tiles_m / world;
    p.m_rot = ((rank + 1) % world) * p.m_block;
    int clusters = p.tiles_m * p.tiles_n;
    if (clusters > g_num_sms / 2) clusters = g_num_sms / 2;
    pair::gemm_bf16_pair_kernel<false, true><<<clusters * 2, NUM_THREADS, pair::PSMEM_RS_BYTES, stream>>>(ta, tb, p);
  } else {
    p.tiles_m = M / BM;
    p.m_block = p.tiles_m;
    p.tiles_n = (N + BN - 1) / BN;
    p.idesc = tt::umma_idesc_bf16(BM, BN, 0, b_mn);
    p.m_block = p.tiles_m / world;
    p.m_rot = ((rank + 1) % world) * p.m_block;
    int gemm_ctas = p.tiles_m * p.tiles_n;
    if (gemm_ctas > g_num_sms) gemm_ctas = g_num_sms;
    gemm_bf16_kernel<false, true><<<gemm_ctas, NUM_THREADS, SMEM_BYTES, stream>>>(ta, tb, p);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// Tile order of the fused reduce-scatter: -1 = choose by the NVLink burst estimate, 0 = peer-owned tiles first, 1 =
// interleaved; for tests and benchmarks.
void tt_gemm_rs_set_interleave(int mode) { g_rs_interleave = mode; }

// Select between the single-CTA (0) and CTA-pair (1, default) tile kernels; for tests and benchmarks.
int tt_gemm_set_pair(int enabled) { g_pair_enabled = enabled != 0; return 0; }

// Error word written by kernels whose bounded waits expired (0 = none). Reading clears it.
int tt_gemm_error() {
  int v = 0, zero = 0;
  cudaMemcpyFromSymbol(&v, g_gemm_error, sizeof(int));
  if (v) cudaMemcpyToSymbol(g_gemm_error, &zero, sizeof(int));
  return v;
}

}  // extern "C"
