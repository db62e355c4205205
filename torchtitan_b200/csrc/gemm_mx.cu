// MXFP8 GEMM on the block-scaled tensor-core path: C[M,N] = A[M,K] . B[N,K]^T with e4m3 operands (both K-major) and one
// E8M0 scale per 32 consecutive K elements of every row of A and of B, applied by the MMA itself
// (tcgen05.mma.kind::mxf8f6f4.block_scale), fp32 accumulation in TMEM.
//
// One persistent CTA per SM, 128 x 256 output tiles, 128-wide K steps (one 128-byte swizzle row of 8-bit elements =
// four MMAs of K = 32):
//   warp 0   : producer. Per K step one TMA tile of A and of B plus the step's scale factors (three 512-byte bulk copies)
//   warp 1   : one elected thread copies the scale factors from shared memory to TMEM (tcgen05.cp 32x128b.warpx4) and
//              issues the MMAs; tcgen05.commit frees the stage and, after the last step, publishes the accumulator
//   warp 2   : TMEM allocation
//   warps 4-7: epilogue, TMEM -> registers -> global (bf16 or fp32)
// The accumulator is single-buffered (256 columns): the scale factors of the four stages take the columns after it.
//
// Scale-factor layout ("swizzled", produced by tt_mx_swizzle_scales): for every block of 128 rows and every K step
// (4 scales per row) one 512-byte chunk in which row r, scale j sits at byte (r % 32) * 16 + (r / 32) * 4 + j. The
// 32x128b.warpx4 copy puts the 16 bytes of source row i into four consecutive 32-bit TMEM columns of lanes i, i + 32,
// i + 64 and i + 96, so that row r of the tile finds its four scales in lane r, column r / 32, one byte each; the MMA for
// K sub-step j selects byte j through the scale-factor ids of the instruction descriptor.
//
// Every wait is bounded (see ptx.cuh); on expiry the CTA sets g_mx_error, drains and frees its TMEM.

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx.cuh"

namespace {

constexpr int BM = 128, BN = 256, BK = 128, STAGES = 4, UMMA_K = 32;
constexpr uint32_t A_STAGE = BM * BK;            // 16 KB
constexpr uint32_t B_STAGE = BN * BK;            // 32 KB
constexpr uint32_t SF_CHUNK = 512;               // scales of 128 rows x one K step
constexpr uint32_t SF_STAGE = 3 * SF_CHUNK;      // A, B rows 0..127, B rows 128..255
constexpr uint32_t ACC_COLS = 256, SF_COLS_PER_STAGE = 16, TMEM_COLS = 512;
constexpr int NUM_THREADS = 256;
constexpr size_t SMEM_BYTES = 1024 + STAGES * (A_STAGE + B_STAGE + SF_STAGE) + 256;
constexpr size_t SMEM_BYTES_GROUPED = SMEM_BYTES + (1024 + 1) * 4;   // + tiles-before-group table (MAX_GROUPS + 1 ints)

__device__ int g_mx_error = 0;

struct MxArgs {
  int M, N, K, k_iters, tiles_m, tiles_n;
  const uint8_t* sfa;   // [tiles_m][k_iters][512]
  const uint8_t* sfb;   // [2 * tiles_n][k_iters][512]
  void* C;
  long long ldc;
  int c_fp32;
};

// Grouped (mixture-of-experts) form: rows of the activation operand are grouped by expert, `offs[g]` (device memory) is
// the end row of group g. Every group starts at a multiple of 128 rows (the dispatcher pads), so a tile's scale chunks
// are whole chunks of the operand's scale array.
//   mode 0  Y[r, :] = X[r, :] . W_g^T for rows r of group g. A = X [R, K]. B is either the weights as [G * N, K]
//           (b_row_stride = N rows per group, b_k_stride = 0) or, for the input gradient, the transposed weights as
//           [N, G * K] (b_row_stride = 0, b_k_stride = K / 128 steps per group along the contraction).
//   mode 1  C_g = A[:, rows of g] . B[:, rows of g]^T, the weight gradient: A [M, R] and B [N, R] are the transposed
//           operands, the contraction runs over the group's rows; C is [G * M, N]. Empty groups get no tile.
constexpr int MAX_GROUPS = 1024;
struct MxGroups {
  int mode, G;
  const int* offs;
  int b_row_stride, b_k_stride;
  int a_kb4, b_kb4;      // K steps per row block in the scale arrays of A and B
  int b_row_blocks;      // 128-row blocks in B's scale array (the last one is reused for rows beyond it)
};

struct MxTile {
  int a_row, b_row, a_k0, b_k0, k_iters;
  long long c_row;       // first row of the tile in C
  long long c_row_end;   // rows of C at or beyond this are not written
  int c_col;
  bool ok;
};

__device__ __forceinline__ void mx_build_prefix(const MxArgs& p, const MxGroups& g, int* prefix) {
  if (threadIdx.x == 0) {
    int acc = 0, prev = 0;
    for (int i = 0; i < g.G; ++i) {
      prefix[i] = acc;
      const int end = __ldg(g.offs + i);
      const int rows = end - prev;
      prev = end;
      if (g.mode == 0) acc += ((rows + BM - 1) / BM) * p.tiles_n;
      else acc += rows > 0 ? p.tiles_m * p.tiles_n : 0;
    }
    prefix[g.G] = acc;
  }
}

template <bool GROUPED>
__device__ __forceinline__ MxTile mx_tile(const MxArgs& p, const MxGroups& g, const int* prefix, int t) {
  MxTile tl;
  if constexpr (!GROUPED) {
    const int tm = t % p.tiles_m, tn = t / p.tiles_m;
    tl.a_row = tm * BM; tl.b_row = tn * BN; tl.a_k0 = 0; tl.b_k0 = 0; tl.k_iters = p.k_iters;
    tl.c_row = tl.a_row; tl.c_row_end = p.M; tl.c_col = tl.b_row; tl.ok = true;
  } else {
    int lo = 0, hi = g.G - 1;                  // last group whose prefix is <= t (groups without tiles share a prefix
    while (lo < hi) {                          // with the next group: the search lands on the last of equal entries)
      const int mid = (lo + hi + 1) >> 1;
      if (prefix[mid] <= t) lo = mid; else hi = mid - 1;
    }
    const int row0 = lo > 0 ? __ldg(g.offs + lo - 1) : 0;
    const int rows = __ldg(g.offs + lo) - row0;
    const int r = t - prefix[lo];
    tl.ok = (row0 % BM) == 0 && (g.mode == 0 || (rows % BK) == 0);
    if (g.mode == 0) {
      const int tmg = (rows + BM - 1) / BM;    // m fastest: CTAs running together share one expert's weight panel
      const int tm = r % tmg, tn = r / tmg;
      tl.a_row = row0 + tm * BM; tl.a_k0 = 0;
      tl.b_row = lo * g.b_row_stride + tn * BN; tl.b_k0 = lo * g.b_k_stride;
      tl.k_iters = p.k_iters;
      tl.c_row = tl.a_row; tl.c_row_end = min(row0 + rows, p.M); tl.c_col = tn * BN;
    } else {
      const int tm = r % p.tiles_m, tn = r / p.tiles_m;
      tl.a_row = tm * BM; tl.b_row = tn * BN; tl.a_k0 = row0 / BK; tl.b_k0 = row0 / BK;
      tl.k_iters = rows / BK;
      tl.c_row = static_cast<long long>(lo) * p.M + tm * BM;
      tl.c_row_end = static_cast<long long>(lo) * p.M + p.M;
      tl.c_col = tn * BN;
    }
    if (!tl.ok) tl.k_iters = 0;
  }
  return tl;
}

// Shared-memory matrix descriptor without swizzle for the scale-factor chunk: 32 rows of 16 bytes, 8-row core matrices
// 128 bytes apart.
__device__ __forceinline__ uint64_t sf_smem_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3FFF);
  d |= static_cast<uint64_t>(128 >> 4) << 32;  // stride between 8-row groups
  d |= 1ull << 46;                             // descriptor version for sm_100
  return d;                                    // layout type 0: no swizzle
}

__device__ __forceinline__ void tmem_cp_sf(uint32_t taddr, uint64_t desc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
}

// Instruction descriptor: e4m3 x e4m3, both K-major, E8M0 scales, M = 128, N = 256; `j` selects the scale byte.
__device__ __forceinline__ uint32_t mx_idesc(int j) {
  return (static_cast<uint32_t>(j) << 4) | (static_cast<uint32_t>(BN >> 3) << 17) | (1u << 23) |
         (static_cast<uint32_t>(BM >> 4) << 24) | (static_cast<uint32_t>(j) << 29);
}

__device__ __forceinline__ void umma_mx_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sfa,
                                           uint32_t sfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
      : "memory");
}

// Write 32 consecutive accumulator columns of one output row (bf16 or fp32).
__device__ __forceinline__ void store_acc_chunk(const MxArgs& p, long long row, int col, const uint32_t (&r)[32]) {
  const bool full_chunk = col + 32 <= p.N;
  if (p.c_fp32) {
    float* dst = static_cast<float*>(p.C) + row * p.ldc + col;
    if (full_chunk && p.ldc % 4 == 0) {
#pragma unroll
      for (int j = 0; j < 8; ++j)
        reinterpret_cast<float4*>(dst)[j] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                                        __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
    } else {
      for (int j = 0; j < 32 && col + j < p.N; ++j) dst[j] = __uint_as_float(r[j]);
    }
  } else {
    __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.C) + row * p.ldc + col;
    if (full_chunk && p.ldc % 8 == 0) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint4 q;
        q.x = tt::pack_bf16(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]));
        q.y = tt::pack_bf16(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
        q.z = tt::pack_bf16(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
        q.w = tt::pack_bf16(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
        reinterpret_cast<uint4*>(dst)[j] = q;
      }
    } else {
      for (int j = 0; j < 32 && col + j < p.N; ++j) dst[j] = __float2bfloat16(__uint_as_float(r[j]));
    }
  }
}

template <bool GROUPED>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_mx_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, MxArgs p, MxGroups grp) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (tt::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - tt::smem_u32(smem_raw));
  const uint32_t sA = base;
  const uint32_t sB = sA + STAGES * A_STAGE;
  const uint32_t sSF = sB + STAGES * B_STAGE;
  const uint32_t bars = sSF + STAGES * SF_STAGE;
  uint8_t* bars_gen = gen_base + STAGES * (A_STAGE + B_STAGE + SF_STAGE);
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
  const uint32_t tfull_bar = bars + 8u * (2 * STAGES), tempty_bar = bars + 8u * (2 * STAGES + 1);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars_gen + 8 * (2 * STAGES + 2));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars_gen + 8 * (2 * STAGES + 2) + 8);
  int* prefix = reinterpret_cast<int*>(bars_gen + 256);     // grouped form only: tiles before each group

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if constexpr (GROUPED) mx_build_prefix(p, grp, prefix);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      tt::mbar_init(full_bar(s), 1);
      tt::mbar_init(empty_bar(s), 1);
    }
    tt::mbar_init(tfull_bar, 1);
    tt::mbar_init(tempty_bar, 4);  // one arrival per epilogue warp
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
  int num_tiles = p.tiles_m * p.tiles_n;
  if constexpr (GROUPED) num_tiles = prefix[grp.G];

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (tt::elect_one()) {
      uint32_t it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const MxTile tl = mx_tile<GROUPED>(p, grp, prefix, t);
        if (GROUPED && !tl.ok) atomicExch(&g_mx_error, 16);   // a group that does not start / end on a tile boundary
        const int a_kb4 = GROUPED ? grp.a_kb4 : p.k_iters, b_kb4 = GROUPED ? grp.b_kb4 : p.k_iters;
        const int brb0 = tl.b_row / 128;
        const int brb1 = (GROUPED && brb0 + 1 >= grp.b_row_blocks) ? brb0 : brb0 + 1;
        const uint8_t* ga = p.sfa + (static_cast<long long>(tl.a_row / 128) * a_kb4 + tl.a_k0) * SF_CHUNK;
        const uint8_t* gb0 = p.sfb + (static_cast<long long>(brb0) * b_kb4 + tl.b_k0) * SF_CHUNK;
        const uint8_t* gb1 = p.sfb + (static_cast<long long>(brb1) * b_kb4 + tl.b_k0) * SF_CHUNK;
        for (int k = 0; k < tl.k_iters; ++k, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!tt::mbar_wait(empty_bar(s), ph ^ 1, abort_flag, &g_mx_error, 1)) { ok = false; break; }
          tt::mbar_expect_tx(full_bar(s), A_STAGE + B_STAGE + SF_STAGE);
          tt::tma_load_2d(sA + s * A_STAGE, &tma_a, full_bar(s), (tl.a_k0 + k) * BK, tl.a_row);
          tt::tma_load_2d(sB + s * B_STAGE, &tma_b, full_bar(s), (tl.b_k0 + k) * BK, tl.b_row);
          const uint32_t sf = sSF + s * SF_STAGE;
          tt::bulk_load(sf, ga + static_cast<long long>(k) * SF_CHUNK, SF_CHUNK, full_bar(s));
          tt::bulk_load(sf + SF_CHUNK, gb0 + static_cast<long long>(k) * SF_CHUNK, SF_CHUNK, full_bar(s));
          tt::bulk_load(sf + 2 * SF_CHUNK, gb1 + static_cast<long long>(k) * SF_CHUNK, SF_CHUNK, full_bar(s));
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ scale-factor copies + MMAs
    if (tt::elect_one()) {
      uint32_t it = 0, tile_it = 0;
      bool ok = true;
      const uint32_t sbo = 1024 >> 4;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++tile_it) {
        const int k_iters = GROUPED ? mx_tile<GROUPED>(p, grp, prefix, t).k_iters : p.k_iters;
        if (!tt::mbar_wait(tempty_bar, (tile_it & 1) ^ 1, abort_flag, &g_mx_error, 2)) break;
        tt::tc_fence_after();
        for (int k = 0; k < k_iters; ++k, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!tt::mbar_wait(full_bar(s), ph, abort_flag, &g_mx_error, 3)) { ok = false; break; }
          tt::tc_fence_after();
          const uint32_t sf = sSF + s * SF_STAGE;
          const uint32_t t_sfa = tmem_base + ACC_COLS + s * SF_COLS_PER_STAGE, t_sfb = t_sfa + 4;
          tmem_cp_sf(t_sfa, sf_smem_desc(sf));
          tmem_cp_sf(t_sfb, sf_smem_desc(sf + SF_CHUNK));
          tmem_cp_sf(t_sfb + 4, sf_smem_desc(sf + 2 * SF_CHUNK));
          const uint32_t aA = sA + s * A_STAGE, aB = sB + s * B_STAGE;
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            const uint64_t ad = tt::umma_smem_desc(aA + kk * UMMA_K, 1, sbo);
            const uint64_t bd = tt::umma_smem_desc(aB + kk * UMMA_K, 1, sbo);
            // the byte of the scale column is carried both in the descriptor ids and in the top bits of the address
            umma_mx_ss(tmem_base, ad, bd, mx_idesc(kk), t_sfa + (static_cast<uint32_t>(kk) << 30),
                       t_sfb + (static_cast<uint32_t>(kk) << 30), (k | kk) != 0);
          }
          tt::umma_commit(empty_bar(s));
        }
        if (ok) tt::umma_commit(tfull_bar);
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------ epilogue
    const int ew = warp - 4;
    uint32_t tile_it = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++tile_it) {
      const MxTile tl = mx_tile<GROUPED>(p, grp, prefix, t);
      if (!tt::mbar_wait(tfull_bar, tile_it & 1, abort_flag, &g_mx_error, 4)) break;
      tt::tc_fence_after();
      const long long row = tl.c_row + ew * 32 + lane;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(ew * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tt::tmem_ld_32x32(taddr + c * 32, r);
        tt::tc_wait_ld();
        const int col = tl.c_col + c * 32;
        if (!tl.ok || row >= tl.c_row_end || col >= p.N) continue;
        store_acc_chunk(p, row, col, r);
      }
      tt::tc_fence_before();
      __syncwarp();
      if (lane == 0) tt::mbar_arrive(tempty_bar);
    }
  }

  __syncthreads();
  if (*abort_flag) tt::abort_drain();
  if (warp == 2) {
    tt::tc_fence_after();
    tt::tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------------------------
// CTA-pair variant (cta_group::2): two CTAs on neighbouring SMs share one 256 x 256 output tile. Each CTA stages its own
// 128 rows of A, *half* of the B tile and the scale factors it needs (its rows of A, all 256 columns of B), so every SM
// pulls 33.5 KB instead of 49.5 KB per K step through the L2-to-SM fabric, which is what bounds the single-CTA kernel.
// One elected thread of the leader issues the scale-factor copies (tcgen05.cp.cta_group::2 copies in both CTAs, each
// from its own shared memory) and the M = 256 MMAs; each CTA's TMEM holds its 128 rows x 256 columns of the accumulator.
// Scale factors travel as TMA tiles of the chunk array viewed as [chunks][128 x u32] (a bulk copy cannot credit the
// partner's barrier, the cta_group::2 tensor copy can). No cluster multicast anywhere.
namespace pairmx {
constexpr int PSTAGES = 6;
constexpr uint32_t PA = 128 * BK, PB = 128 * BK, PSF = 3 * SF_CHUNK;   // per CTA per stage
constexpr uint32_t STAGE_BYTES = PA + PB + PSF;
constexpr size_t PSMEM = 1024 + PSTAGES * STAGE_BYTES + 256;

__device__ __forceinline__ void tmem_cp_sf_pair(uint32_t taddr, uint64_t desc) {
  asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
}
__device__ __forceinline__ uint32_t mx_idesc_pair(int j) {   // M = 256 across the pair, N = 256
  return (static_cast<uint32_t>(j) << 4) | (static_cast<uint32_t>(256 >> 3) << 17) | (1u << 23) |
         (static_cast<uint32_t>(256 >> 4) << 24) | (static_cast<uint32_t>(j) << 29);
}
__device__ __forceinline__ void umma_mx_ss_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sfa,
                                                uint32_t sfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
      : "memory");
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm_mx_pair_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                    const __grid_constant__ CUtensorMap tma_sfa, const __grid_constant__ CUtensorMap tma_sfb, MxArgs p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (tt::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - tt::smem_u32(smem_raw));
  const uint32_t sA = base, sB = sA + PSTAGES * PA, sSF = sB + PSTAGES * PB;
  const uint32_t bars = sSF + PSTAGES * PSF;
  uint8_t* bars_gen = gen_base + PSTAGES * STAGE_BYTES;
  auto full_bar = [&](int s) { return bars + 8u * s; };                      // used in the leader only
  auto empty_bar = [&](int s) { return bars + 8u * (PSTAGES + s); };         // one per CTA
  const uint32_t tfull_bar = bars + 8u * (2 * PSTAGES);                      // one per CTA
  const uint32_t tempty_bar = bars + 8u * (2 * PSTAGES + 1);                 // used in the leader only
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars_gen + 8 * (2 * PSTAGES + 2));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars_gen + 8 * (2 * PSTAGES + 2) + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = tt::cluster_ctarank();   // 0 = leader
  const int num_tiles = p.tiles_m * p.tiles_n;   // in 256 x 256 tiles
  const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < PSTAGES; ++s) { tt::mbar_init(full_bar(s), 1); tt::mbar_init(empty_bar(s), 1); }
    tt::mbar_init(tfull_bar, 1);
    tt::mbar_init(tempty_bar, 8);                // four epilogue warps in each CTA
    *abort_flag = 0;
    tt::mbar_fence_init();
    tt::tma_prefetch_desc(&tma_a); tt::tma_prefetch_desc(&tma_b);
    tt::tma_prefetch_desc(&tma_sfa); tt::tma_prefetch_desc(&tma_sfb);
  }
  if (warp == 2) { tt::tmem_alloc_pair(tt::smem_u32(tmem_slot), TMEM_COLS); tt::tmem_relinquish_pair(); }
  tt::tc_fence_before();
  tt::cluster_sync();
  tt::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ producer (both CTAs)
    if (tt::elect_one()) {
      uint32_t it = 0;
      bool ok = true;
      for (int t = cluster_id; t < num_tiles && ok; t += num_clusters) {
        const int tm = t % p.tiles_m, tn = t / p.tiles_m;
        const int m0 = tm * 256 + rank * 128, n0 = tn * 256 + rank * 128;
        const int ca = (2 * tm + static_cast<int>(rank)) * p.k_iters;          // chunk rows of this CTA's A scales
        const int cb0 = (2 * tn) * p.k_iters, cb1 = (2 * tn + 1) * p.k_iters;  // both halves of the B scales
        for (int k = 0; k < p.k_iters; ++k, ++it) {
          const int s = it % PSTAGES;
          const uint32_t ph = (it / PSTAGES) & 1;
          if (!tt::mbar_wait(empty_bar(s), ph ^ 1, abort_flag, &g_mx_error, 11)) { ok = false; break; }
          const uint32_t fb = tt::mapa(full_bar(s), 0);   // the leader's barrier collects both CTAs' bytes
          if (rank == 0) tt::mbar_expect_tx(full_bar(s), 2 * STAGE_BYTES);
          tt::tma_load_2d_pair(sA + s * PA, &tma_a, fb, k * BK, m0);
          tt::tma_load_2d_pair(sB + s * PB, &tma_b, fb, k * BK, n0);
          const uint32_t sf = sSF + s * PSF;
          tt::tma_load_2d_pair(sf, &tma_sfa, fb, 0, ca + k);
          tt::tma_load_2d_pair(sf + SF_CHUNK, &tma_sfb, fb, 0, cb0 + k);
          tt::tma_load_2d_pair(sf + 2 * SF_CHUNK, &tma_sfb, fb, 0, cb1 + k);
        }
      }
    }
  } else if (warp == 1 && rank == 0) {
    // ------------------------------------------------------------ scale-factor copies + MMAs (leader only)
    if (tt::elect_one()) {
      uint32_t it = 0, tile_it = 0;
      bool ok = true;
      const uint32_t sbo = 1024 >> 4;
      for (int t = cluster_id; t < num_tiles && ok; t += num_clusters, ++tile_it) {
        if (!tt::mbar_wait(tempty_bar, (tile_it & 1) ^ 1, abort_flag, &g_mx_error, 12)) break;
        tt::tc_fence_after();
        for (int k = 0; k < p.k_iters; ++k, ++it) {
          const int s = it % PSTAGES;
          const uint32_t ph = (it / PSTAGES) & 1;
          if (!tt::mbar_wait(full_bar(s), ph, abort_flag, &g_mx_error, 13)) { ok = false; break; }
          tt::tc_fence_after();
          const uint32_t sf = sSF + s * PSF;
          const uint32_t t_sfa = tmem_base + ACC_COLS + s * SF_COLS_PER_STAGE, t_sfb = t_sfa + 4;
          tmem_cp_sf_pair(t_sfa, sf_smem_desc(sf));
          tmem_cp_sf_pair(t_sfb, sf_smem_desc(sf + SF_CHUNK));
          tmem_cp_sf_pair(t_sfb + 4, sf_smem_desc(sf + 2 * SF_CHUNK));
          const uint32_t aA = sA + s * PA, aB = sB + s * PB;
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            const uint64_t ad = tt::umma_smem_desc(aA + kk * UMMA_K, 1, sbo);
            const uint64_t bd = tt::umma_smem_desc(aB + kk * UMMA_K, 1, sbo);
            umma_mx_ss_pair(tmem_base, ad, bd, mx_idesc_pair(kk), t_sfa + (static_cast<uint32_t>(kk) << 30),
                            t_sfb + (static_cast<uint32_t>(kk) << 30), (k | kk) != 0);
          }
          tt::umma_commit_pair(empty_bar(s), 3);   // frees this stage in both CTAs
        }
        if (ok) tt::umma_commit_pair(tfull_bar, 3);
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------ epilogue (both CTAs, own 128 rows)
    const int ew = warp - 4;
    uint32_t tile_it = 0;
    const uint32_t leader_tempty = tt::mapa(tempty_bar, 0);
    for (int t = cluster_id; t < num_tiles; t += num_clusters, ++tile_it) {
      const int tm = t % p.tiles_m, tn = t / p.tiles_m;
      if (!tt::mbar_wait(tfull_bar, tile_it & 1, abort_flag, &g_mx_error, 14)) break;
      tt::tc_fence_after();
      const int row = tm * 256 + static_cast<int>(rank) * 128 + ew * 32 + lane;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(ew * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < 256 / 32; ++c) {
        uint32_t r[32];
        tt::tmem_ld_32x32(taddr + c * 32, r);
        tt::tc_wait_ld();
        const int col = tn * 256 + c * 32;
        if (row >= p.M || col >= p.N) continue;
        store_acc_chunk(p, row, col, r);
      }
      tt::tc_fence_before();
      __syncwarp();
      if (lane == 0) tt::mbar_arrive_cluster(leader_tempty);
    }
  }

  __syncthreads();
  if (*abort_flag) tt::abort_drain();
  tt::cluster_sync();   // nobody leaves while its partner may still touch its shared memory or TMEM
  if (warp == 2) { tt::tc_fence_after(); tt::tmem_dealloc_pair(tmem_base, TMEM_COLS); }
}
}  // namespace pairmx

// scales [R, KB] (row-major E8M0 bytes) -> chunks [ceil(R/128) rounded to row_blocks][kb4 = ceil(KB/4)][512]; missing rows
// and K blocks get exponent 127 (2^0), their data is zero-filled by TMA.
__global__ void mx_swizzle_scales_kernel(const uint8_t* __restrict__ s, int R, int KB, uint8_t* __restrict__ out,
                                         int row_blocks, int kb4) {
  const long long total = static_cast<long long>(row_blocks) * kb4 * SF_CHUNK;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int within = static_cast<int>(i % SF_CHUNK);
    const long long chunk = i / SF_CHUNK;
    const int ks = static_cast<int>(chunk % kb4);
    const int rb = static_cast<int>(chunk / kb4);
    const int j = within & 3, grp = (within >> 2) & 3, r32 = within >> 4;
    const int row = rb * 128 + grp * 32 + r32, kb = ks * 4 + j;
    out[i] = (row < R && kb < KB) ? s[static_cast<long long>(row) * KB + kb] : static_cast<uint8_t>(127);
  }
}

bool g_attr = false;
int g_sms = 0;
bool g_mx_pair = true;

}  // namespace

extern "C" {

// 0 forces the single-CTA kernel (tests, comparisons); 1 (default) lets large shapes use CTA pairs.
void tt_gemm_mx_set_pair(int on) { g_mx_pair = on != 0; }

int tt_gemm_mx_error() {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_mx_error, sizeof(int));
  if (v) {
    int z = 0;
    cudaMemcpyToSymbol(g_mx_error, &z, sizeof(int));
  }
  return v;
}

// Bytes of the swizzled scale buffer for `rows` rows (padded to a multiple of `row_pad`, 128 for A and 256 for B) and a
// contraction of K elements.
long long tt_mx_scales_bytes(int rows, int row_pad, int K) {
  const long long rb = (rows + row_pad - 1) / row_pad * (row_pad / 128);
  const long long kb4 = (K + BK - 1) / BK;
  return rb * kb4 * SF_CHUNK;
}

int tt_mx_swizzle_scales(const void* scales, int rows, int K, int row_pad, void* out, cudaStream_t st) {
  if (rows <= 0 || K <= 0) return 0;
  if (K % 32 || (row_pad != 128 && row_pad != 256)) return -2;
  const int KB = K / 32;
  const int rb = (rows + row_pad - 1) / row_pad * (row_pad / 128);
  const int kb4 = (K + BK - 1) / BK;
  const long long total = static_cast<long long>(rb) * kb4 * SF_CHUNK;
  long long g = (total + 255) / 256;
  if (g > 148 * 8) g = 148 * 8;
  mx_swizzle_scales_kernel<<<static_cast<int>(g), 256, 0, st>>>(static_cast<const uint8_t*>(scales), rows, KB,
                                                                 static_cast<uint8_t*>(out), rb, kb4);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// A [M,K], B [N,K] e4m3 (row strides lda / ldb bytes, multiples of 16); sfa / sfb in the swizzled layout (row_pad 128 /
// 256); C [M,N] bf16 or fp32.
int tt_gemm_mxfp8(const void* A, const void* B, const void* sfa, const void* sfb, void* C, int M, int N, int K,
                  long long lda, long long ldb, long long ldc, int c_fp32, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 16) || (ldb % 16) || (K % 32)) return -2;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) ||
      (reinterpret_cast<uintptr_t>(sfa) & 15) || (reinterpret_cast<uintptr_t>(sfb) & 15))
    return -3;
  if (!g_attr) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sms, cudaDevAttrMultiProcessorCount, dev);
    cudaFuncSetAttribute(gemm_mx_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(SMEM_BYTES));
    cudaFuncSetAttribute(gemm_mx_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(SMEM_BYTES_GROUPED));
    cudaFuncSetAttribute(pairmx::gemm_mx_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(pairmx::PSMEM));
    g_attr = true;
  }
  if (g_mx_pair && M >= 256 && N >= 256) {
    // CTA-pair tiles of 256 x 256. Needs the scale buffers padded to 256 rows (tt_mx_scales_bytes(rows, 256, K)).
    CUtensorMap ta, tb, tsa, tsb;
    int rc = tt::make_tmap_2d(&ta, A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, K, lda, 128, BK);
    if (rc) return rc;
    rc = tt::make_tmap_2d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, K, ldb, 128, BK);
    if (rc) return rc;
    MxArgs p;
    p.M = M; p.N = N; p.K = K;
    p.k_iters = (K + BK - 1) / BK;
    p.tiles_m = (M + 255) / 256;
    p.tiles_n = (N + 255) / 256;
    p.sfa = static_cast<const uint8_t*>(sfa);
    p.sfb = static_cast<const uint8_t*>(sfb);
    p.C = C; p.ldc = ldc; p.c_fp32 = c_fp32;
    // scale chunks as rows of 128 32-bit words
    rc = tt::make_tmap_2d(&tsa, sfa, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, static_cast<uint64_t>(2) * p.tiles_m * p.k_iters, 128, 128, 1,
                          128, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc) return rc;
    rc = tt::make_tmap_2d(&tsb, sfb, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, static_cast<uint64_t>(2) * p.tiles_n * p.k_iters, 128, 128, 1,
                          128, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc) return rc;
    int clusters = p.tiles_m * p.tiles_n;
    if (clusters > g_sms / 2) clusters = g_sms / 2;
    pairmx::gemm_mx_pair_kernel<<<clusters * 2, NUM_THREADS, pairmx::PSMEM, stream>>>(ta, tb, tsa, tsb, p);
    return cudaGetLastError() == cudaSuccess ? 0 : -4;
  }
  CUtensorMap ta, tb;
  int rc = tt::make_tmap_2d(&ta, A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, K, lda, BM, BK);
  if (rc) return rc;
  rc = tt::make_tmap_2d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, K, ldb, BN, BK);
  if (rc) return rc;
  MxArgs p;
  p.M = M; p.N = N; p.K = K;
  p.k_iters = (K + BK - 1) / BK;
  p.tiles_m = (M + BM - 1) / BM;
  p.tiles_n = (N + BN - 1) / BN;
  p.sfa = static_cast<const uint8_t*>(sfa);
  p.sfb = static_cast<const uint8_t*>(sfb);
  p.C = C; p.ldc = ldc; p.c_fp32 = c_fp32;
  int grid = p.tiles_m * p.tiles_n;
  if (grid > g_sms) grid = g_sms;
  gemm_mx_kernel<false><<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(ta, tb, p, MxGroups{});
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// Grouped MXFP8 GEMM with the group boundaries on the device (see MxGroups). `A` is [a_rows, a_cols] and `B` is
// [b_rows, b_cols] e4m3, both contiguous along the contraction, with swizzled scale arrays of a_rows / 128 and
// ceil(b_rows / 128) row blocks; all of a_rows, a_cols, b_cols and the group boundaries are multiples of 128.
//   mode 0: C [a_rows, N] rows grouped; `M` = a_rows, `K` = contraction per group; B rows of group g start at
//           g * b_row_stride, its contraction at g * b_k_stride elements.
//   mode 1: C [G * M, N]; contraction over the rows of group g (columns of A and B); the caller zero-fills C.
int tt_grouped_gemm_mxfp8(const void* A, const void* B, const void* sfa, const void* sfb, void* C, const int* offs, int mode,
                          int G, int M, int N, int K, long long a_rows, long long a_cols, long long b_rows, long long b_cols,
                          int b_row_stride, int b_k_stride, long long ldc, int c_fp32, cudaStream_t stream) {
  if (G <= 0 || a_rows <= 0 || N <= 0) return 0;
  if (G > MAX_GROUPS || (mode != 0 && mode != 1)) return -2;
  if ((a_rows % 128) || (a_cols % 128) || (b_cols % 128) || (b_row_stride % 128) || (b_k_stride % 128) || (K % 128)) return -2;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) ||
      (reinterpret_cast<uintptr_t>(sfa) & 15) || (reinterpret_cast<uintptr_t>(sfb) & 15))
    return -3;
  if (!g_attr) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sms, cudaDevAttrMultiProcessorCount, dev);
    cudaFuncSetAttribute(gemm_mx_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(SMEM_BYTES));
    cudaFuncSetAttribute(gemm_mx_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(SMEM_BYTES_GROUPED));
    cudaFuncSetAttribute(pairmx::gemm_mx_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(pairmx::PSMEM));
    g_attr = true;
  }
  CUtensorMap ta, tb;
  int rc = tt::make_tmap_2d(&ta, A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a_rows, a_cols, a_cols, BM, BK);
  if (rc) return rc;
  rc = tt::make_tmap_2d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, b_rows, b_cols, b_cols, BN, BK);
  if (rc) return rc;
  MxArgs p;
  p.M = M; p.N = N; p.K = K;
  p.k_iters = K / BK;
  p.tiles_m = (M + BM - 1) / BM;
  p.tiles_n = (N + BN - 1) / BN;
  p.sfa = static_cast<const uint8_t*>(sfa);
  p.sfb = static_cast<const uint8_t*>(sfb);
  p.C = C; p.ldc = ldc; p.c_fp32 = c_fp32;
  MxGroups g;
  g.mode = mode; g.G = G; g.offs = offs;
  g.b_row_stride = b_row_stride; g.b_k_stride = b_k_stride / BK;
  g.a_kb4 = static_cast<int>(a_cols / BK); g.b_kb4 = static_cast<int>(b_cols / BK);
  g.b_row_blocks = static_cast<int>((b_rows + 127) / 128);
  long long bound = mode == 0 ? (a_rows / BM + G) * p.tiles_n : static_cast<long long>(G) * p.tiles_m * p.tiles_n;
  int grid = bound < g_sms ? static_cast<int>(bound) : g_sms;
  if (grid < 1) grid = 1;
  gemm_mx_kernel<true><<<grid, NUM_THREADS, SMEM_BYTES_GROUPED, stream>>>(ta, tb, p, g);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // extern "C"
