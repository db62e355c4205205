// Grouped bf16 GEMM for mixture-of-experts layers on tcgen05 tensor cores, group boundaries read on the device.
//
// Rows of the activation matrix are grouped by expert; `offs[g]` (int32, device memory) is the end row of group g
// (cumulative sum of the padded per-expert counts). Nothing about the split is known to the host, so routing never
// forces a device-to-host synchronisation.
//
//   mode 0  Y[r, :] = X[r, :] . W[g]^T            rows r of group g          (forward; input gradient with b_mn = 1)
//           X [R, K] K-major; W is [G, N, K] (b_mn = 0) or [G, K, N] (b_mn = 1); Y [R, N] bf16.
//           An output tile (128 rows x 256 columns) starts at the group's first row, so tiles never mix experts;
//           rows of a tile that lie beyond the group's end are computed and discarded.
//   mode 1  C[g] = A_g^T . B_g                     contraction over the rows of group g   (weight gradient)
//           A [R, M] (= dY), B [R, N] (= X), both row-major, so both operands are MN-major; C [G, M, N] bf16 / fp32.
//           Group sizes must be multiples of 64 (the contraction tile): the dispatcher pads groups with zero rows.
//           Empty groups are skipped: C must be zero-initialised by the caller.
//
// Same warp roles and mbarrier pipeline as gemm.cu (TMA producer / UMMA issuer / 4 epilogue warps, two TMEM accumulators
// so that the epilogue of one tile overlaps the main loop of the next); every wait is bounded.
// Replaces torch._grouped_mm (torchtitan/models/common/moe/moe.py:59-76).
#include "ptx.cuh"

namespace {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4, UMMA_K = 16;
constexpr uint32_t A_STAGE_BYTES = BM * BK * 2, B_STAGE_BYTES = BN * BK * 2;
constexpr uint32_t TMEM_COLS = 512;
constexpr int NUM_THREADS = 256;
constexpr int MAX_GROUPS = 1024;
constexpr size_t SMEM_BYTES = 1024 + STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + 256 + (MAX_GROUPS + 1) * 4;

__device__ int g_grouped_error = 0;

struct GArgs {
  int mode;            // 0: rows grouped, 1: contraction grouped
  int G;               // number of groups
  int M, N, K;         // mode 0: N, K per group (M unused); mode 1: M, N per group (K unused)
  int b_mn;            // mode 0 only: W stored [G, K, N]
  int tiles_n;         // mode 0: ceil(N / BN); mode 1: ceil(N / BN)
  int tiles_m;         // mode 1: ceil(M / BM)
  const int* offs;     // [G] cumulative group ends
  void* C;
  long long ldc;
  int c_fp32;
  uint32_t idesc;
};

struct Tile {
  int g, tm, tn;       // group, tile indices inside the group
  int row0, rows;      // first row of the group, rows in the group
};

// prefix[g] = number of tiles of groups < g (prefix[G] = total); built once per CTA
__device__ __forceinline__ void build_prefix(const GArgs& p, int* prefix) {
  if (threadIdx.x == 0) {
    int acc = 0, prev = 0;
    for (int g = 0; g < p.G; ++g) {
      prefix[g] = acc;
      const int end = __ldg(p.offs + g);
      const int rows = end - prev;
      prev = end;
      if (p.mode == 0) acc += ((rows + BM - 1) / BM) * p.tiles_n;
      else acc += rows > 0 ? p.tiles_m * p.tiles_n : 0;
    }
    prefix[p.G] = acc;
  }
}

__device__ __forceinline__ Tile locate(const GArgs& p, const int* prefix, int t) {
  int lo = 0, hi = p.G - 1;  // last g with prefix[g] <= t
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (prefix[mid] <= t) lo = mid; else hi = mid - 1;
  }
  // groups without tiles share their prefix with the next one: the search above lands on the last of equal entries
  Tile tl;
  tl.g = lo;
  const int end = __ldg(p.offs + lo);
  tl.row0 = lo > 0 ? __ldg(p.offs + lo - 1) : 0;
  tl.rows = end - tl.row0;
  const int r = t - prefix[lo];
  if (p.mode == 0) {
    const int tmg = (tl.rows + BM - 1) / BM;   // m fastest: concurrently running CTAs share one expert's weight panel
    tl.tm = r % tmg;
    tl.tn = r / tmg;
  } else {
    tl.tm = r % p.tiles_m;
    tl.tn = r / p.tiles_m;
  }
  return tl;
}

__device__ __forceinline__ void store32(const GArgs& p, long long row, int col, int col_end, const uint32_t (&r)[32]) {
  if (p.c_fp32) {
    float* dst = reinterpret_cast<float*>(p.C) + row * p.ldc + col;
    if (col + 32 <= col_end && (p.ldc % 4 == 0)) {
#pragma unroll
      for (int j = 0; j < 8; ++j)
        reinterpret_cast<float4*>(dst)[j] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                                        __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
    } else {
      for (int j = 0; j < 32 && col + j < col_end; ++j) dst[j] = __uint_as_float(r[j]);
    }
  } else {
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + row * p.ldc + col;
    if (col + 32 <= col_end && (p.ldc % 8 == 0)) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint4 v;
        v.x = tt::pack_bf16(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]));
        v.y = tt::pack_bf16(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
        v.z = tt::pack_bf16(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
        v.w = tt::pack_bf16(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
        reinterpret_cast<uint4*>(dst)[j] = v;
      }
    } else {
      for (int j = 0; j < 32 && col + j < col_end; ++j) dst[j] = __float2bfloat16(__uint_as_float(r[j]));
    }
  }
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, GArgs p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (tt::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - tt::smem_u32(smem_raw));
  const uint32_t sA = base, sB = base + STAGES * A_STAGE_BYTES;
  const uint32_t bars = base + STAGES * (A_STAGE_BYTES + B_STAGE_BYTES);
  uint8_t* bars_gen = gen + STAGES * (A_STAGE_BYTES + B_STAGE_BYTES);
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bars + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bars + 8u * (2 * STAGES + 2 + a); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars_gen + 8 * (2 * STAGES + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars_gen + 8 * (2 * STAGES + 4) + 8);
  int* prefix = reinterpret_cast<int*>(bars_gen + 256);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { tt::mbar_init(full_bar(s), 1); tt::mbar_init(empty_bar(s), 1); }
    for (int a = 0; a < 2; ++a) { tt::mbar_init(tfull_bar(a), 1); tt::mbar_init(tempty_bar(a), 4); }
    *abort_flag = 0;
    tt::mbar_fence_init();
    tt::tma_prefetch_desc(&tma_a);
    tt::tma_prefetch_desc(&tma_b);
  }
  build_prefix(p, prefix);
  if (warp == 2) { tt::tmem_alloc(tt::smem_u32(tmem_slot), TMEM_COLS); tt::tmem_relinquish(); }
  tt::tc_fence_before();
  __syncthreads();
  tt::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int num_tiles = prefix[p.G];

  if (warp == 0) {
    if (tt::elect_one()) {
      uint32_t it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const Tile tl = locate(p, prefix, t);
        const int k_iters = p.mode == 0 ? (p.K + BK - 1) / BK : tl.rows / BK;
        for (int k = 0; k < k_iters; ++k, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!tt::mbar_wait(empty_bar(s), ph ^ 1, abort_flag, &g_grouped_error, 1)) { ok = false; break; }
          tt::mbar_expect_tx(full_bar(s), A_STAGE_BYTES + B_STAGE_BYTES);
          const uint32_t dA = sA + s * A_STAGE_BYTES, dB = sB + s * B_STAGE_BYTES;
          if (p.mode == 0) {
            tt::tma_load_2d(dA, &tma_a, full_bar(s), k * BK, tl.row0 + tl.tm * BM);
            if (!p.b_mn) {
              tt::tma_load_2d(dB, &tma_b, full_bar(s), k * BK, tl.g * p.N + tl.tn * BN);
            } else {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j)
                tt::tma_load_2d(dB + j * (64 * BK * 2), &tma_b, full_bar(s), tl.tn * BN + j * 64, tl.g * p.K + k * BK);
            }
          } else {
            const int krow = tl.row0 + k * BK;
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tt::tma_load_2d(dA + j * (64 * BK * 2), &tma_a, full_bar(s), tl.tm * BM + j * 64, krow);
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tt::tma_load_2d(dB + j * (64 * BK * 2), &tma_b, full_bar(s), tl.tn * BN + j * 64, krow);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (tt::elect_one()) {
      uint32_t it = 0, tile_it = 0;
      bool ok = true;
      const int a_mn = p.mode == 1, b_mn = p.mode == 1 ? 1 : p.b_mn;
      const uint32_t a_lbo = a_mn ? (64 * BK * 2) >> 4 : 1, b_lbo = b_mn ? (64 * BK * 2) >> 4 : 1;
      const uint32_t sbo = 1024 >> 4;
      const uint32_t a_kadv = a_mn ? (UMMA_K * 128) : (UMMA_K * 2), b_kadv = b_mn ? (UMMA_K * 128) : (UMMA_K * 2);
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++tile_it) {
        const Tile tl = locate(p, prefix, t);
        const int k_iters = p.mode == 0 ? (p.K + BK - 1) / BK : tl.rows / BK;
        const int acc = tile_it & 1;
        const uint32_t acc_ph = (tile_it >> 1) & 1;
        if (!tt::mbar_wait(tempty_bar(acc), acc_ph ^ 1, abort_flag, &g_grouped_error, 2)) break;
        tt::tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int k = 0; k < k_iters; ++k, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!tt::mbar_wait(full_bar(s), ph, abort_flag, &g_grouped_error, 3)) { ok = false; break; }
          tt::tc_fence_after();
          const uint32_t aA = sA + s * A_STAGE_BYTES, aB = sB + s * B_STAGE_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk)
            tt::umma_f16_ss(d_tmem, tt::umma_smem_desc(aA + kk * a_kadv, a_lbo, sbo),
                            tt::umma_smem_desc(aB + kk * b_kadv, b_lbo, sbo), p.idesc, (k | kk) != 0);
          tt::umma_commit(empty_bar(s));
        }
        if (ok) tt::umma_commit(tfull_bar(acc));
      }
    }
  } else if (warp >= 4) {
    const int ew = warp - 4;
    uint32_t tile_it = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++tile_it) {
      const Tile tl = locate(p, prefix, t);
      const int acc = tile_it & 1;
      const uint32_t acc_ph = (tile_it >> 1) & 1;
      if (!tt::mbar_wait(tfull_bar(acc), acc_ph, abort_flag, &g_grouped_error, 4)) break;
      tt::tc_fence_after();
      const int r_in = tl.tm * BM + ew * 32 + lane;           // row inside the group (mode 0) / inside C[g] (mode 1)
      const bool row_ok = p.mode == 0 ? r_in < tl.rows : r_in < p.M;
      const long long row = p.mode == 0 ? static_cast<long long>(tl.row0) + r_in
                                        : static_cast<long long>(tl.g) * p.M + r_in;
      const int n0 = tl.tn * BN;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(ew * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tt::tmem_ld_32x32(taddr + c * 32, r);
        tt::tc_wait_ld();
        const int col = n0 + c * 32;
        if (!row_ok || col >= p.N) continue;
        store32(p, row, col, p.N, r);
      }
      tt::tc_fence_before();
      __syncwarp();
      if (lane == 0) tt::mbar_arrive(tempty_bar(acc));
    }
  }

  __syncthreads();
  if (*abort_flag) tt::abort_drain();
  if (warp == 2) { tt::tc_fence_after(); tt::tmem_dealloc(tmem_base, TMEM_COLS); }
}

// ------------------------------------------------------------------------------------------------
// CTA-pair form (cta_group::2): two CTAs on neighbouring SMs share one 256 x 256 output tile of a group. Each CTA stages
// its own 128 rows of A and its own half (128 columns) of the B tile, so every SM pulls 32 KB instead of 48 KB per K step
// through the L2-to-SM fabric, which is what bounds the single-CTA kernel; the leader issues M = 256 MMAs whose
// accumulator rows live in both CTAs' tensor memory. Same modes and group table as above; tiles are 256 rows.
namespace gpair {
constexpr int TM = 256, TN = 256, PSTAGES = 6;
constexpr uint32_t PA_BYTES = 128 * BK * 2, PB_BYTES = 128 * BK * 2;   // per CTA per stage
constexpr size_t PSMEM_BYTES = 1024 + PSTAGES * (PA_BYTES + PB_BYTES) + 256 + (MAX_GROUPS + 1) * 4;

__device__ __forceinline__ void build_prefix_pair(const GArgs& p, int* prefix) {
  if (threadIdx.x == 0) {
    int acc = 0, prev = 0;
    for (int g = 0; g < p.G; ++g) {
      prefix[g] = acc;
      const int end = __ldg(p.offs + g);
      const int rows = end - prev;
      prev = end;
      if (p.mode == 0) acc += ((rows + TM - 1) / TM) * p.tiles_n;
      else acc += rows > 0 ? p.tiles_m * p.tiles_n : 0;
    }
    prefix[p.G] = acc;
  }
}

__device__ __forceinline__ Tile locate_pair(const GArgs& p, const int* prefix, int t) {
  int lo = 0, hi = p.G - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (prefix[mid] <= t) lo = mid; else hi = mid - 1;
  }
  Tile tl;
  tl.g = lo;
  tl.row0 = lo > 0 ? __ldg(p.offs + lo - 1) : 0;
  tl.rows = __ldg(p.offs + lo) - tl.row0;
  const int r = t - prefix[lo];
  if (p.mode == 0) {
    const int tmg = (tl.rows + TM - 1) / TM;
    tl.tm = r % tmg;
    tl.tn = r / tmg;
  } else {
    tl.tm = r % p.tiles_m;
    tl.tn = r / p.tiles_m;
  }
  return tl;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
grouped_gemm_pair_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, GArgs p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (tt::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - tt::smem_u32(smem_raw));
  const uint32_t sA = base, sB = base + PSTAGES * PA_BYTES;
  const uint32_t bars = base + PSTAGES * (PA_BYTES + PB_BYTES);
  uint8_t* bars_gen = gen + PSTAGES * (PA_BYTES + PB_BYTES);
  auto full_bar = [&](int s) { return bars + 8u * s; };                        // used in the leader only
  auto empty_bar = [&](int s) { return bars + 8u * (PSTAGES + s); };           // one per CTA
  auto tfull_bar = [&](int a) { return bars + 8u * (2 * PSTAGES + a); };       // one per CTA
  auto tempty_bar = [&](int a) { return bars + 8u * (2 * PSTAGES + 2 + a); };  // used in the leader only
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars_gen + 8 * (2 * PSTAGES + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars_gen + 8 * (2 * PSTAGES + 4) + 8);
  int* prefix = reinterpret_cast<int*>(bars_gen + 256);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = tt::cluster_ctarank();  // 0 = leader
  const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < PSTAGES; ++s) { tt::mbar_init(full_bar(s), 1); tt::mbar_init(empty_bar(s), 1); }
    for (int a = 0; a < 2; ++a) { tt::mbar_init(tfull_bar(a), 1); tt::mbar_init(tempty_bar(a), 8); }
    *abort_flag = 0;
    tt::mbar_fence_init();
    tt::tma_prefetch_desc(&tma_a);
    tt::tma_prefetch_desc(&tma_b);
  }
  build_prefix_pair(p, prefix);
  if (warp == 2) { tt::tmem_alloc_pair(tt::smem_u32(tmem_slot), TMEM_COLS); tt::tmem_relinquish_pair(); }
  tt::tc_fence_before();
  __syncthreads();
  tt::cluster_sync();  // barriers of both CTAs are initialised before anyone signals across
  tt::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int num_tiles = prefix[p.G];          // both CTAs build the same table from the same offsets

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (tt::elect_one()) {
      uint32_t it = 0;
      bool ok = true;
      for (int t = cluster_id; t < num_tiles && ok; t += num_clusters) {
        const Tile tl = locate_pair(p, prefix, t);
        const int k_iters = p.mode == 0 ? (p.K + BK - 1) / BK : tl.rows / BK;
        const int m_off = tl.tm * TM + static_cast<int>(rank) * 128, n_off = tl.tn * TN + static_cast<int>(rank) * 128;
        for (int k = 0; k < k_iters; ++k, ++it) {
          const int s = it % PSTAGES;
          const uint32_t ph = (it / PSTAGES) & 1;
          if (!tt::mbar_wait(empty_bar(s), ph ^ 1, abort_flag, &g_grouped_error, 11)) { ok = false; break; }
          const uint32_t fb = tt::mapa(full_bar(s), 0);  // the leader's barrier collects both CTAs' bytes
          if (rank == 0) tt::mbar_expect_tx(full_bar(s), 2 * (PA_BYTES + PB_BYTES));
          const uint32_t dA = sA + s * PA_BYTES, dB = sB + s * PB_BYTES;
          if (p.mode == 0) {
            tt::tma_load_2d_pair(dA, &tma_a, fb, k * BK, tl.row0 + m_off);
            if (!p.b_mn) {
              tt::tma_load_2d_pair(dB, &tma_b, fb, k * BK, tl.g * p.N + n_off);
            } else {
#pragma unroll
              for (int j = 0; j < 2; ++j)
                tt::tma_load_2d_pair(dB + j * (64 * BK * 2), &tma_b, fb, n_off + j * 64, tl.g * p.K + k * BK);
            }
          } else {
            const int krow = tl.row0 + k * BK;
#pragma unroll
            for (int j = 0; j < 2; ++j) tt::tma_load_2d_pair(dA + j * (64 * BK * 2), &tma_a, fb, m_off + j * 64, krow);
#pragma unroll
            for (int j = 0; j < 2; ++j) tt::tma_load_2d_pair(dB + j * (64 * BK * 2), &tma_b, fb, n_off + j * 64, krow);
          }
        }
      }
    }
  } else if (warp == 1 && rank == 0) {
    // ------------------------------------------------------------ UMMA issuer (leader CTA only)
    if (tt::elect_one()) {
      uint32_t it = 0, tile_it = 0;
      bool ok = true;
      const int a_mn = p.mode == 1, b_mn = p.mode == 1 ? 1 : p.b_mn;
      const uint32_t a_lbo = a_mn ? (64 * BK * 2) >> 4 : 1, b_lbo = b_mn ? (64 * BK * 2) >> 4 : 1;
      const uint32_t sbo = 1024 >> 4;
      const uint32_t a_kadv = a_mn ? (UMMA_K * 128) : (UMMA_K * 2), b_kadv = b_mn ? (UMMA_K * 128) : (UMMA_K * 2);
      for (int t = cluster_id; t < num_tiles && ok; t += num_clusters, ++tile_it) {
        const Tile tl = locate_pair(p, prefix, t);
        const int k_iters = p.mode == 0 ? (p.K + BK - 1) / BK : tl.rows / BK;
        const int acc = tile_it & 1;
        const uint32_t acc_ph = (tile_it >> 1) & 1;
        if (!tt::mbar_wait(tempty_bar(acc), acc_ph ^ 1, abort_flag, &g_grouped_error, 12)) break;
        tt::tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * TN;
        for (int k = 0; k < k_iters; ++k, ++it) {
          const int s = it % PSTAGES;
          const uint32_t ph = (it / PSTAGES) & 1;
          if (!tt::mbar_wait(full_bar(s), ph, abort_flag, &g_grouped_error, 13)) { ok = false; break; }
          tt::tc_fence_after();
          const uint32_t aA = sA + s * PA_BYTES, aB = sB + s * PB_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk)
            tt::umma_f16_ss_pair(d_tmem, tt::umma_smem_desc(aA + kk * a_kadv, a_lbo, sbo),
                                 tt::umma_smem_desc(aB + kk * b_kadv, b_lbo, sbo), p.idesc, (k | kk) != 0);
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
      const Tile tl = locate_pair(p, prefix, t);
      const int acc = tile_it & 1;
      const uint32_t acc_ph = (tile_it >> 1) & 1;
      if (!tt::mbar_wait(tfull_bar(acc), acc_ph, abort_flag, &g_grouped_error, 14)) break;
      tt::tc_fence_after();
      const int r_in = tl.tm * TM + static_cast<int>(rank) * 128 + ew * 32 + lane;
      const bool row_ok = p.mode == 0 ? r_in < tl.rows : r_in < p.M;
      const long long row = p.mode == 0 ? static_cast<long long>(tl.row0) + r_in
                                        : static_cast<long long>(tl.g) * p.M + r_in;
      const int n0 = tl.tn * TN;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(ew * 32) << 16) + acc * TN;
#pragma unroll 1
      for (int c = 0; c < TN / 32; ++c) {
        uint32_t r[32];
        tt::tmem_ld_32x32(taddr + c * 32, r);
        tt::tc_wait_ld();
        const int col = n0 + c * 32;
        if (!row_ok || col >= p.N) continue;
        store32(p, row, col, p.N, r);
      }
      tt::tc_fence_before();
      __syncwarp();
      if (lane == 0) tt::mbar_arrive_cluster(acc ? leader_tempty1 : leader_tempty0);
    }
  }

  __syncthreads();
  if (*abort_flag) tt::abort_drain();
  tt::cluster_sync();  // nobody leaves while its partner may still touch its shared memory or tensor memory
  if (warp == 2) { tt::tc_fence_after(); tt::tmem_dealloc_pair(tmem_base, TMEM_COLS); }
}
}  // namespace gpair

bool g_attr = false;
bool g_grouped_pair = true;

void set_attrs() {
  if (g_attr) return;
  cudaFuncSetAttribute(grouped_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(SMEM_BYTES));
  cudaFuncSetAttribute(gpair::grouped_gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                       static_cast<int>(gpair::PSMEM_BYTES));
  g_attr = true;
}

}  // namespace

extern "C" {

// 0 forces the single-CTA kernel (tests, comparisons); 1 (default) lets shapes with N >= 256 use CTA pairs.
void tt_grouped_gemm_set_pair(int on) { g_grouped_pair = on != 0; }

// mode 0. X [R, K] bf16 (row stride ldx), W [G, N, K] (b_mn = 0) or [G, K, N] (b_mn = 1) contiguous bf16, Y [R, N] bf16
// (row stride ldy), offs int32 [G] on the device. K (and with b_mn, also N) must be a multiple of 8; with b_mn, K must
// be a multiple of 64. `max_tiles_m` bounds the grid only (any value >= 1 is correct).
int tt_grouped_gemm(const void* X, const void* W, void* Y, const int* offs, long long R, int G, int N, int K, int b_mn,
                    long long ldx, long long ldy, cudaStream_t st) {
  if (G < 1 || G > MAX_GROUPS || R <= 0) return G < 1 || G > MAX_GROUPS ? -2 : 0;
  if (K % 8 || N % 8 || (b_mn && K % BK)) return -3;
  set_attrs();
  const bool use_pair = g_grouped_pair && N >= 256 && R >= 256;
  CUtensorMap ta, tb;
  int rc = tt::make_tmap_2d(&ta, X, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, R, K, ldx, BM, BK);
  if (rc) return rc;
  if (!b_mn) rc = tt::make_tmap_2d(&tb, W, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, static_cast<uint64_t>(G) * N, K, K,
                                   use_pair ? 128 : BN, BK);
  else       rc = tt::make_tmap_2d(&tb, W, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, static_cast<uint64_t>(G) * K, N, N, BK, 64);
  if (rc) return rc;
  GArgs p{};
  p.mode = 0; p.G = G; p.N = N; p.K = K; p.b_mn = b_mn; p.tiles_n = (N + BN - 1) / BN; p.tiles_m = 0;
  p.offs = offs; p.C = Y; p.ldc = ldy; p.c_fp32 = 0;
  p.idesc = tt::umma_idesc_bf16(BM, BN, 0, b_mn);
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (use_pair) {
    p.idesc = tt::umma_idesc_bf16(gpair::TM, gpair::TN, 0, b_mn);
    const long long upper = ((R + gpair::TM - 1) / gpair::TM + G) * p.tiles_n;
    const int clusters = static_cast<int>(upper < sms / 2 ? upper : sms / 2);
    gpair::grouped_gemm_pair_kernel<<<clusters * 2, NUM_THREADS, gpair::PSMEM_BYTES, st>>>(ta, tb, p);
    return cudaGetLastError() == cudaSuccess ? 0 : -4;
  }
  const long long upper = ((R + BM - 1) / BM + G) * p.tiles_n;  // every group adds at most one partial tile
  const int grid = static_cast<int>(upper < sms ? upper : sms);
  grouped_gemm_kernel<<<grid, NUM_THREADS, SMEM_BYTES, st>>>(ta, tb, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// mode 1. A [R, M] bf16, B [R, N] bf16 (row-major, strides lda / ldb), C [G, M, N] contiguous (bf16, or fp32 when
// c_fp32), zero-initialised by the caller; every group size must be a multiple of 64.
int tt_grouped_gemm_wgrad(const void* A, const void* B, void* C, const int* offs, long long R, int G, int M, int N,
                          long long lda, long long ldb, int c_fp32, cudaStream_t st) {
  if (G < 1 || G > MAX_GROUPS) return -2;
  if (R <= 0) return 0;
  if (M % 8 || N % 8) return -3;
  set_attrs();
  CUtensorMap ta, tb;
  int rc = tt::make_tmap_2d(&ta, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, R, M, lda, BK, 64);
  if (rc) return rc;
  rc = tt::make_tmap_2d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, R, N, ldb, BK, 64);
  if (rc) return rc;
  GArgs p{};
  p.mode = 1; p.G = G; p.M = M; p.N = N; p.K = 0; p.b_mn = 1;
  p.tiles_m = (M + BM - 1) / BM; p.tiles_n = (N + BN - 1) / BN;
  p.offs = offs; p.C = C; p.ldc = N; p.c_fp32 = c_fp32;
  p.idesc = tt::umma_idesc_bf16(BM, BN, 1, 1);
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (g_grouped_pair && M >= 256 && N >= 256) {
    p.tiles_m = (M + gpair::TM - 1) / gpair::TM;
    p.idesc = tt::umma_idesc_bf16(gpair::TM, gpair::TN, 1, 1);
    const long long upper = static_cast<long long>(G) * p.tiles_m * p.tiles_n;
    const int clusters = static_cast<int>(upper < sms / 2 ? upper : sms / 2);
    gpair::grouped_gemm_pair_kernel<<<clusters * 2, NUM_THREADS, gpair::PSMEM_BYTES, st>>>(ta, tb, p);
    return cudaGetLastError() == cudaSuccess ? 0 : -4;
  }
  const long long upper = static_cast<long long>(G) * p.tiles_m * p.tiles_n;
  const int grid = static_cast<int>(upper < sms ? upper : sms);
  grouped_gemm_kernel<<<grid, NUM_THREADS, SMEM_BYTES, st>>>(ta, tb, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

int tt_grouped_gemm_error() {
  int v = 0, zero = 0;
  cudaMemcpyFromSymbol(&v, g_grouped_error, sizeof(int));
  if (v) cudaMemcpyToSymbol(g_grouped_error, &zero, sizeof(int));
  return v;
}

}  // extern "C"
