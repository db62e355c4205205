// Causal / full / range-masked (document, sliding-window, fixed-block) softmax attention with grouped KV heads on
// tcgen05 tensor cores.
//
// Layout: q,o,dO,dq [B,Sq,H,D]; k,v,dk,dv [B,Sk,Hkv,D]; D = 128; lse, delta [B,H,Sq] fp32.
// All tiles are fetched with 3-D TMA descriptors (D, heads, B*S) straight from that layout, so no
// transposed copies of q/k/v exist anywhere.
//
// forward   (CTA = 128 query rows of one head, two CTAs per SM): S = Q K^T into TMEM, one softmax
//           thread per query row reads its row (no shuffles), P goes to shared memory as the A
//           operand of O += P V; O stays in TMEM and is rescaled only when the running maximum grew
//           by more than 2^8 (exact: the final division uses the same reference maximum).
// backward  is split into two kernels without atomics, so it is deterministic:
//           dkv kernel (CTA = 128 key rows of one KV head) loops over the query tiles and the query
//           heads of the group: S^T = K Q^T, dP^T = V dO^T, dV += P^T dO, dK += dS^T Q;
//           dq  kernel (CTA = 128 query rows) loops over key tiles: S, dP, dQ += dS K.
// Every mbarrier wait is bounded (see ptx.cuh).
//
// Replaces F.scaled_dot_product_attention (cuDNN / flash) used by the reference
// (torchtitan/models/common/attention.py:176-212).
#include "ptx.cuh"

namespace {

constexpr int D = 128;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

__device__ int g_attn_error = 0;

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct AttnArgs {
  int B, Sq, Sk, H, Hkv;
  int causal;
  float scale;          // softmax scale
  void* out;            // fwd: O bf16 ; dq kernel: dQ bf16 ; dkv kernel: dK bf16
  void* out2;           // dkv kernel: dV bf16
  float* lse;           // [B,H,Sq]
  const float* delta;   // [B,H,Sq]
  // Optional contiguous-range masks (need Sq == Sk): query i sees keys row_lo[b,i] <= k <= i, equivalently key k is
  // seen by queries k <= i <= col_hi[b,k]. Both arrays are non-decreasing along the sequence, which covers document
  // masks, sliding windows and fixed blocks. Tiles wholly outside the range are skipped.
  const int* row_lo;    // [B,Sq] or null
  const int* col_hi;    // [B,Sk] or null
  // Optional attention sinks (forward only): one learned logit per query head that joins the softmax denominator and
  // carries no value. The backward kernels need nothing extra: they rebuild the probabilities from lse, which includes
  // the sink.
  const float* sinks;   // [H] fp32 or null
};

// Write 64 fp32 values as one 128-byte bf16 row of a K-major, 128B-swizzled operand tile.
__device__ __forceinline__ void store_row_sw128(uint8_t* tile, int row, const float (&v)[64]) {
  uint8_t* r = tile + row * 128;
  const int x = row & 7;
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    uint4 q;
    q.x = tt::pack_bf16(v[8 * c + 0], v[8 * c + 1]);
    q.y = tt::pack_bf16(v[8 * c + 2], v[8 * c + 3]);
    q.z = tt::pack_bf16(v[8 * c + 4], v[8 * c + 5]);
    q.w = tt::pack_bf16(v[8 * c + 6], v[8 * c + 7]);
    *reinterpret_cast<uint4*>(r + ((c ^ x) << 4)) = q;
  }
}

// Write 32 fp32 values as one half (64 bytes) of a 128-byte bf16 row; half = 0 (cols 0..31) or 1.
__device__ __forceinline__ void store_halfrow_sw128(uint8_t* tile, int row, int half, const float (&v)[32]) {
  uint8_t* r = tile + row * 128;
  const int x = row & 7;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    uint4 q;
    q.x = tt::pack_bf16(v[8 * c + 0], v[8 * c + 1]);
    q.y = tt::pack_bf16(v[8 * c + 2], v[8 * c + 3]);
    q.z = tt::pack_bf16(v[8 * c + 4], v[8 * c + 5]);
    q.w = tt::pack_bf16(v[8 * c + 6], v[8 * c + 7]);
    *reinterpret_cast<uint4*>(r + (((half * 4 + c) ^ x) << 4)) = q;
  }
}

// 32 fp32 TMEM columns -> 32 bf16 written to a global row segment
__device__ __forceinline__ void store_out_32(__nv_bfloat16* dst, const uint32_t (&r)[32]) {
#pragma unroll
  for (int v4 = 0; v4 < 4; ++v4) {
    uint4 q;
    q.x = tt::pack_bf16(__uint_as_float(r[8 * v4 + 0]), __uint_as_float(r[8 * v4 + 1]));
    q.y = tt::pack_bf16(__uint_as_float(r[8 * v4 + 2]), __uint_as_float(r[8 * v4 + 3]));
    q.z = tt::pack_bf16(__uint_as_float(r[8 * v4 + 4]), __uint_as_float(r[8 * v4 + 5]));
    q.w = tt::pack_bf16(__uint_as_float(r[8 * v4 + 6]), __uint_as_float(r[8 * v4 + 7]));
    *reinterpret_cast<uint4*>(dst + v4 * 8) = q;
  }
}

// ---- UMMA helpers for the fixed tile shapes used here -------------------------------------------
// K-major operand made of two 64-wide halves along the contraction (head dim 128): rows x 128 bf16,
// half h at base + h * rows*128 bytes. Contraction step kk (16 wide), kk in [0, 8).
__device__ __forceinline__ uint64_t desc_kmajor_dh(uint32_t base, int rows, int kk) {
  return tt::umma_smem_desc(base + (kk >> 2) * rows * 128 + (kk & 3) * 32, 1, 64);
}
// K-major operand with a 64-wide contraction (one swizzle atom): step kk in [0, 4).
__device__ __forceinline__ uint64_t desc_kmajor_64(uint32_t base, int kk) {
  return tt::umma_smem_desc(base + kk * 32, 1, 64);
}
// MN-major operand: image is [krows rows][128 B] per 64-wide MN half; halves krows*128 bytes apart.
// Contraction step kk (16 rows each).
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t base, int krows, int kk) {
  return tt::umma_smem_desc(base + kk * 2048, (krows * 128) >> 4, 64);
}

constexpr uint32_t IDESC_128x64_KK = tt::umma_idesc_bf16(128, 64, 0, 0);
constexpr uint32_t IDESC_128x128_KM = tt::umma_idesc_bf16(128, 128, 0, 1);

// =================================================================================== forward
// Head dimensions are template parameters: DQK for queries / keys, DV for values and the output (128/128 Llama and
// Qwen, 64/64 GPT-OSS, 192/128 multi-head latent attention). An operand of width W lives in shared memory as W / 64
// chunks of [rows][128 bytes] (one 128-byte swizzle atom wide), chunk c holding elements 64c .. 64c + 63.
// smem: Q (DQK/64) x 16K | K 2 stages x (DQK/64) x 8K | V (DV/64) x 8K | barriers  (two CTAs per SM)
template <int DQK, int DV>
struct FwdLayout {
  static constexpr int QC = DQK / 64, VC = DV / 64;
  static constexpr uint32_t Q = 0, K = QC * 16384, KSTAGE = QC * 8192, V = K + 2 * KSTAGE, VBYTES = VC * 8192,
                            BAR = V + VBYTES;
  static constexpr size_t SMEM = 1024 + BAR + 256;
};

template <int DQK, int DV>
__global__ void __launch_bounds__(192, 2)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                const __grid_constant__ CUtensorMap tv, AttnArgs p) {
  using L = FwdLayout<DQK, DV>;
  constexpr uint32_t F_Q = L::Q, F_K = L::K, F_V = L::V, F_BAR = L::BAR;
  constexpr uint32_t IDESC_PV = tt::umma_idesc_bf16(128, DV, 0, 1);
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (tt::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (base - tt::smem_u32(smem_raw));
  const uint32_t bar0 = base + F_BAR;
  // barriers: 0 q_full | 1,2 k_full | 3,4 k_empty | 5 v_full | 7 v_empty | 9,10 s_full | 11 p_ready | 12 pv_done
  auto bar = [&](int i) { return bar0 + 8u * i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gbase + F_BAR + 8 * 13);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gbase + F_BAR + 8 * 13 + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = gridDim.x - 1 - blockIdx.x;  // heavy (late) causal tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.H / p.Hkv);
  const int q0 = qt * 128;
  const int off = p.Sk - p.Sq;  // query i attends keys <= i + off
  int n_kv = p.Sk / 64;
  if (p.causal) n_kv = min(n_kv, (q0 + 127 + off) / 64 + 1);
  // range mask: the first row of the tile has the smallest lower bound, earlier key tiles are skipped
  const int j0 = p.row_lo ? min(__ldg(p.row_lo + static_cast<long long>(b) * p.Sq + q0) / 64, n_kv) : 0;
  n_kv -= j0;  // from here on: number of key tiles visited, tile index j means key tile j0 + j

  if (threadIdx.x == 0) {
    for (int i = 0; i < 13; ++i) tt::mbar_init(bar(i), i == 11 ? 4 : 1);
    *abort_flag = 0;
    tt::mbar_fence_init();
    tt::tma_prefetch_desc(&tq); tt::tma_prefetch_desc(&tk); tt::tma_prefetch_desc(&tv);
  }
  if (warp == 1) { tt::tmem_alloc(tt::smem_u32(tmem_slot), 256); tt::tmem_relinquish(); }
  tt::tc_fence_before();
  __syncthreads();
  tt::tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tS = tmem, tO = tmem + 128;  // S buffers at cols 0 and 64, O at 128 .. 128 + DV

  if (warp == 0) {
    if (tt::elect_one()) {
      tt::mbar_expect_tx(bar(0), L::QC * 16384);
#pragma unroll
      for (int c = 0; c < L::QC; ++c) tt::tma_load_3d(base + F_Q + c * 16384, &tq, bar(0), c * 64, h, b * p.Sq + q0);
      auto load_k = [&](int j) -> bool {
        const int s = j & 1; const uint32_t ph = (j >> 1) & 1;
        if (!tt::mbar_wait(bar(3 + s), ph ^ 1, abort_flag, &g_attn_error, 11)) return false;
        tt::mbar_expect_tx(bar(1 + s), L::KSTAGE);
#pragma unroll
        for (int c = 0; c < L::QC; ++c)
          tt::tma_load_3d(base + F_K + s * L::KSTAGE + c * 8192, &tk, bar(1 + s), c * 64, hk, b * p.Sk + (j0 + j) * 64);
        return true;
      };
      bool ok = n_kv > 0 ? load_k(0) : true;
      for (int j = 0; j < n_kv && ok; ++j) {
        if (j + 1 < n_kv && !load_k(j + 1)) break;  // K runs one tile ahead of V
        if (!tt::mbar_wait(bar(7), (j & 1) ^ 1, abort_flag, &g_attn_error, 12)) break;
        tt::mbar_expect_tx(bar(5), L::VBYTES);
#pragma unroll
        for (int c = 0; c < L::VC; ++c) tt::tma_load_3d(base + F_V + c * 8192, &tv, bar(5), c * 64, hk, b * p.Sk + (j0 + j) * 64);
      }
    }
  } else if (warp == 1) {
    if (tt::elect_one()) {
      bool ok = tt::mbar_wait(bar(0), 0, abort_flag, &g_attn_error, 13);
      // descriptors are built once; an operand slice is one 32-bit add away (see tt::SmemDesc)
      const tt::SmemDesc dQ = tt::make_smem_desc(base + F_Q, 1, 64), dK0 = tt::make_smem_desc(base + F_K, 1, 64);
      const tt::SmemDesc dV = tt::make_smem_desc(base + F_V, (64 * 128) >> 4, 64);
      auto issue_s = [&](int j) {
        const int s = j & 1;
        const tt::SmemDesc kd = dK0.at(s * L::KSTAGE);
#pragma unroll
        for (int kk = 0; kk < DQK / 16; ++kk)
          tt::umma_f16_ss(tS + s * 64, dQ.at((kk >> 2) * 16384 + (kk & 3) * 32), kd.at((kk >> 2) * 8192 + (kk & 3) * 32),
                          IDESC_128x64_KK, kk != 0);
        tt::umma_commit(bar(9 + s));   // S ready
        tt::umma_commit(bar(3 + s));   // K stage free
      };
      if (ok && n_kv > 0) {
        ok = tt::mbar_wait(bar(1), 0, abort_flag, &g_attn_error, 14);
        if (ok) { tt::tc_fence_after(); issue_s(0); }
      }
      for (int j = 0; j < n_kv && ok; ++j) {
        if (j + 1 < n_kv) {
          const int s1 = (j + 1) & 1;
          if (!tt::mbar_wait(bar(1 + s1), ((j + 1) >> 1) & 1, abort_flag, &g_attn_error, 15)) break;
          tt::tc_fence_after();
          issue_s(j + 1);
        }
        const int s = j & 1;
        if (!tt::mbar_wait(bar(11), j & 1, abort_flag, &g_attn_error, 16)) break;
        if (!tt::mbar_wait(bar(5), j & 1, abort_flag, &g_attn_error, 17)) break;
        tt::tc_fence_after();
        const uint32_t acc0 = j != 0;
        // P (bf16) sits in the first 32 columns of the S buffer it was computed from: the A operand comes from tensor
        // memory, so neither the softmax warps' stores nor this MMA's A reads touch shared memory
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          tt::umma_f16_ts(tO, tS + s * 64 + kk * 8, dV.at(kk * 2048), IDESC_PV, kk ? 1u : acc0);
        tt::umma_commit(bar(12));      // O updated, P free
        tt::umma_commit(bar(7));       // V buffer free
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax: one thread per query row
    const int lg = warp & 3;                 // TMEM lane group of this warp
    const int row = lg * 32 + lane;          // query row inside the tile
    const uint32_t lane_off = static_cast<uint32_t>(lg * 32) << 16;
    const int qi = q0 + row;
    const float sc = p.scale * kLog2e;
    const int lo = p.row_lo ? __ldg(p.row_lo + static_cast<long long>(b) * p.Sq + qi) : 0;
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      const int s = j & 1;
      if (!tt::mbar_wait(bar(9 + s), (j >> 1) & 1, abort_flag, &g_attn_error, 18)) { ok = false; break; }
      tt::tc_fence_after();
      float x[64];
      {
        uint32_t r[32];
        tt::tmem_ld_32x32(tS + lane_off + s * 64, r);
        tt::tc_wait_ld();
#pragma unroll
        for (int e = 0; e < 32; ++e) x[e] = __uint_as_float(r[e]) * sc;
        tt::tmem_ld_32x32(tS + lane_off + s * 64 + 32, r);
        tt::tc_wait_ld();
#pragma unroll
        for (int e = 0; e < 32; ++e) x[32 + e] = __uint_as_float(r[e]) * sc;
      }
      const int kv0 = (j0 + j) * 64;
      if (p.causal && kv0 + 63 > q0 + off) {
#pragma unroll
        for (int e = 0; e < 64; ++e) if (kv0 + e > qi + off) x[e] = -INFINITY;
      }
      if (kv0 < lo) {
#pragma unroll
        for (int e = 0; e < 64; ++e) if (kv0 + e < lo) x[e] = -INFINITY;
      }
      float mx = x[0];
#pragma unroll
      for (int e = 1; e < 64; ++e) mx = fmaxf(mx, x[e]);
      // P buffer (and O) are free once the previous P*V has completed
      if (j > 0 && !tt::mbar_wait(bar(12), (j - 1) & 1, abort_flag, &g_attn_error, 19)) { ok = false; break; }
      tt::tc_fence_after();
      const bool first = (j == 0);
      const bool grow = !first && (mx > m_ref + 8.f);
      if (first) m_ref = mx;
      if (__any_sync(0xffffffffu, grow)) {
        const float m_new = fmaxf(m_ref, mx);
        // 1 when this row did not grow; a row that has seen only masked keys so far keeps m = -inf
        const float f = (m_new == -INFINITY) ? 1.f : fast_exp2(m_ref - m_new);
        m_ref = m_new;
        l *= f;
#pragma unroll 1
        for (int c = 0; c < DV / 16; ++c) {
          uint32_t r[16];
          tt::tmem_ld_32x16(tO + lane_off + c * 16, r);
          tt::tc_wait_ld();
#pragma unroll
          for (int e = 0; e < 16; ++e) r[e] = __float_as_uint(__uint_as_float(r[e]) * f);
          tt::tmem_st_32x16(tO + lane_off + c * 16, r);
        }
        tt::tc_wait_st();
      }
      float sum = 0.f;
      const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;  // all-masked row: exp2(-inf) = 0, not NaN
#pragma unroll
      for (int e = 0; e < 64; ++e) { x[e] = fast_exp2(x[e] - m_use); sum += x[e]; }
      l += sum;
      {
        // P as bf16 pairs over this row's S columns (the MMA reads it from there as its A operand)
        uint32_t pk[16];
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
#pragma unroll
          for (int e = 0; e < 16; ++e) pk[e] = tt::pack_bf16(x[hh * 32 + 2 * e], x[hh * 32 + 2 * e + 1]);
          tt::tmem_st_32x16(tS + lane_off + s * 64 + hh * 16, pk);
        }
        tt::tc_wait_st();
      }
      tt::tc_fence_before();
      __syncwarp();
      if (lane == 0) tt::mbar_arrive(bar(11));
    }
    if (ok && n_kv > 0) ok = tt::mbar_wait(bar(12), (n_kv - 1) & 1, abort_flag, &g_attn_error, 20);
    tt::tc_fence_after();
    if (ok) {
      float o_scale = 1.f;
      if (p.sinks != nullptr) {
        // fold exp(sink) into the running (max, sum): the accumulated O keeps its old reference, so it is rescaled
        // through `inv` below
        const float s2 = __ldg(p.sinks + h) * kLog2e;
        const float m_new = fmaxf(m_ref, s2);
        const float f = (m_ref == -INFINITY) ? 0.f : fast_exp2(m_ref - m_new);
        l = l * f + fast_exp2(s2 - m_new);
        o_scale = f;
        m_ref = m_new;
      }
      const float inv = (l > 0.f) ? o_scale / l : 0.f;
      __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.out) +
                            ((static_cast<long long>(b) * p.Sq + qi) * p.H + h) * DV;
#pragma unroll 1
      for (int c = 0; c < DV / 32; ++c) {
        uint32_t r[32];
        if (n_kv > 0) { tt::tmem_ld_32x32(tO + lane_off + c * 32, r); tt::tc_wait_ld(); }
        else {
#pragma unroll
          for (int e = 0; e < 32; ++e) r[e] = 0;
        }
#pragma unroll
        for (int v4 = 0; v4 < 4; ++v4) {
          uint4 q;
          q.x = tt::pack_bf16(__uint_as_float(r[8 * v4 + 0]) * inv, __uint_as_float(r[8 * v4 + 1]) * inv);
          q.y = tt::pack_bf16(__uint_as_float(r[8 * v4 + 2]) * inv, __uint_as_float(r[8 * v4 + 3]) * inv);
          q.z = tt::pack_bf16(__uint_as_float(r[8 * v4 + 4]) * inv, __uint_as_float(r[8 * v4 + 5]) * inv);
          q.w = tt::pack_bf16(__uint_as_float(r[8 * v4 + 6]) * inv, __uint_as_float(r[8 * v4 + 7]) * inv);
          *reinterpret_cast<uint4*>(orow + c * 32 + v4 * 8) = q;
        }
      }
      if (p.lse) p.lse[(static_cast<long long>(b) * p.H + h) * p.Sq + qi] = (l > 0.f) ? (m_ref + log2f(l)) * kLn2 : -INFINITY;
    }
    tt::tc_fence_before();
  }
  __syncthreads();
  if (*abort_flag) tt::abort_drain();
  if (warp == 1) { tt::tc_fence_after(); tt::tmem_dealloc(tmem, 256); }
}

// =================================================================================== backward: dQ
// CTA = 128 query rows. smem: Q (DQK/64) x 16K | dO (DV/64) x 16K | K/V ring NS x ((DQK/64) x 8K + (DV/64) x 8K) |
// dS 2 x 16K | barriers. A K/V stage is reloaded only after the dQ MMAs that read it have completed, so the ring must
// cover TMA latency plus one full step: three stages where they fit (two for the 192/128 head dimensions).
template <int DQK, int DV>
struct DqLayout {
  static constexpr int QC = DQK / 64, VC = DV / 64;
  static constexpr int NS = (QC * 16384 + VC * 16384 + 3 * (QC + VC) * 8192 + 32768 <= 220 * 1024) ? 3 : 2;
  static constexpr uint32_t Q = 0, DO = QC * 16384, KV = DO + VC * 16384, KBYTES = QC * 8192, STAGE = (QC + VC) * 8192,
                            DS = KV + NS * STAGE, BAR = DS + 32768;
  static constexpr size_t SMEM = 1024 + BAR + 256;
};
// barriers (sized for the largest ring)
constexpr int QB_QFULL = 0, QB_KVFULL = 1, QB_KVEMPTY = QB_KVFULL + 3, QB_SPFULL = QB_KVEMPTY + 3,
              QB_DSREADY = QB_SPFULL + 2, QB_DSFREE = QB_DSREADY + 2, QB_COUNT = QB_DSFREE + 2;

template <int DQK, int DV>
__global__ void __launch_bounds__(320, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tdo,
                   const __grid_constant__ CUtensorMap tk, const __grid_constant__ CUtensorMap tv, AttnArgs p) {
  using L = DqLayout<DQK, DV>;
  constexpr int Q_NS = L::NS;
  constexpr uint32_t Q_Q = L::Q, Q_DO = L::DO, Q_KV = L::KV, Q_DS = L::DS, Q_BAR = L::BAR;
  constexpr uint32_t IDESC_DQ = tt::umma_idesc_bf16(128, DQK, 0, 1);
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (tt::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (base - tt::smem_u32(smem_raw));
  const uint32_t bar0 = base + Q_BAR;
  auto bar = [&](int i) { return bar0 + 8u * i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gbase + Q_BAR + 8 * QB_COUNT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gbase + Q_BAR + 8 * QB_COUNT + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = gridDim.x - 1 - blockIdx.x;
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.H / p.Hkv);
  const int q0 = qt * 128;
  const int off = p.Sk - p.Sq;
  int n_kv = p.Sk / 64;
  if (p.causal) n_kv = min(n_kv, (q0 + 127 + off) / 64 + 1);
  const int j0 = p.row_lo ? min(__ldg(p.row_lo + static_cast<long long>(b) * p.Sq + q0) / 64, n_kv) : 0;
  n_kv -= j0;  // number of key tiles visited; tile index j means key tile j0 + j

  if (threadIdx.x == 0) {
    for (int i = 0; i < QB_COUNT; ++i) tt::mbar_init(bar(i), (i >= QB_DSREADY && i < QB_DSFREE) ? 8 : 1);
    *abort_flag = 0;
    tt::mbar_fence_init();
  }
  if (warp == 1) { tt::tmem_alloc(tt::smem_u32(tmem_slot), 512); tt::tmem_relinquish(); }
  tt::tc_fence_before();
  __syncthreads();
  tt::tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  // TMEM columns: S[2] at 0,64 | dP[2] at 128,192 | dQ at 256 .. 256 + DQK
  const uint32_t tS = tmem, tDP = tmem + 128, tDQ = tmem + 256;

  if (warp == 0) {
    if (tt::elect_one()) {
      tt::mbar_expect_tx(bar(QB_QFULL), (L::QC + L::VC) * 16384);
#pragma unroll
      for (int c = 0; c < L::QC; ++c) tt::tma_load_3d(base + Q_Q + c * 16384, &tq, bar(QB_QFULL), c * 64, h, b * p.Sq + q0);
#pragma unroll
      for (int c = 0; c < L::VC; ++c) tt::tma_load_3d(base + Q_DO + c * 16384, &tdo, bar(QB_QFULL), c * 64, h, b * p.Sq + q0);
      for (int j = 0; j < n_kv; ++j) {
        const int s = j % Q_NS; const uint32_t ph = (j / Q_NS) & 1;
        if (!tt::mbar_wait(bar(QB_KVEMPTY + s), ph ^ 1, abort_flag, &g_attn_error, 21)) break;
        const uint32_t kb = base + Q_KV + s * L::STAGE, vb = kb + L::KBYTES;
        tt::mbar_expect_tx(bar(QB_KVFULL + s), L::STAGE);
#pragma unroll
        for (int c = 0; c < L::QC; ++c) tt::tma_load_3d(kb + c * 8192, &tk, bar(QB_KVFULL + s), c * 64, hk, b * p.Sk + (j0 + j) * 64);
#pragma unroll
        for (int c = 0; c < L::VC; ++c) tt::tma_load_3d(vb + c * 8192, &tv, bar(QB_KVFULL + s), c * 64, hk, b * p.Sk + (j0 + j) * 64);
      }
    }
  } else if (warp == 1) {
    if (tt::elect_one()) {
      bool ok = tt::mbar_wait(bar(QB_QFULL), 0, abort_flag, &g_attn_error, 22);
      auto issue_sp = [&](int j) -> bool {
        const int s = j % Q_NS, t2 = j & 1;
        if (!tt::mbar_wait(bar(QB_KVFULL + s), (j / Q_NS) & 1, abort_flag, &g_attn_error, 23)) return false;
        tt::tc_fence_after();
        const uint32_t kb = base + Q_KV + s * L::STAGE, vb = kb + L::KBYTES;
#pragma unroll
        for (int kk = 0; kk < DQK / 16; ++kk)
          tt::umma_f16_ss(tS + t2 * 64, desc_kmajor_dh(base + Q_Q, 128, kk), desc_kmajor_dh(kb, 64, kk), IDESC_128x64_KK, kk != 0);
#pragma unroll
        for (int kk = 0; kk < DV / 16; ++kk)
          tt::umma_f16_ss(tDP + t2 * 64, desc_kmajor_dh(base + Q_DO, 128, kk), desc_kmajor_dh(vb, 64, kk), IDESC_128x64_KK, kk != 0);
        tt::umma_commit(bar(QB_SPFULL + t2));
        return true;
      };
      if (ok && n_kv > 0) ok = issue_sp(0);
      for (int j = 0; j < n_kv && ok; ++j) {
        if (j + 1 < n_kv && !issue_sp(j + 1)) break;
        const int s = j % Q_NS, t2 = j & 1;
        if (!tt::mbar_wait(bar(QB_DSREADY + t2), (j >> 1) & 1, abort_flag, &g_attn_error, 25)) break;
        tt::tc_fence_after();
        const uint32_t kb = base + Q_KV + s * L::STAGE;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          tt::umma_f16_ss(tDQ, desc_kmajor_64(base + Q_DS + t2 * 16384, kk), desc_mnmajor(kb, 64, kk), IDESC_DQ, (j | kk) != 0);
        tt::umma_commit(bar(QB_DSFREE + t2));   // dS buffer free, dQ step done
        tt::umma_commit(bar(QB_KVEMPTY + s));   // K/V stage free
      }
    }
  } else {
    // 8 softmax warps: lane group = warp & 3 (query row), column half = (warp - 2) >> 2
    const int lg = warp & 3, row = lg * 32 + lane, half = (warp - 2) >> 2;
    const uint32_t lane_off = static_cast<uint32_t>(lg * 32) << 16;
    const int qi = q0 + row;
    const long long stat = (static_cast<long long>(b) * p.H + h) * p.Sq + qi;
    const float lse2 = p.lse[stat] * kLog2e;
    const float dl = p.delta[stat];
    const float sc = p.scale * kLog2e;
    const int lo = p.row_lo ? __ldg(p.row_lo + static_cast<long long>(b) * p.Sq + qi) : 0;
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      const int t2 = j & 1;
      if (!tt::mbar_wait(bar(QB_SPFULL + t2), (j >> 1) & 1, abort_flag, &g_attn_error, 26)) { ok = false; break; }
      tt::tc_fence_after();
      float ds[32];
      const int kv0 = (j0 + j) * 64 + half * 32;
      {
        uint32_t rs[32], rp[32];
        tt::tmem_ld_32x32(tS + lane_off + t2 * 64 + half * 32, rs);
        tt::tmem_ld_32x32(tDP + lane_off + t2 * 64 + half * 32, rp);
        tt::tc_wait_ld();
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          float pr = fast_exp2(__uint_as_float(rs[e]) * sc - lse2);
          if ((p.causal && kv0 + e > qi + off) || kv0 + e < lo) pr = 0.f;
          ds[e] = pr * (__uint_as_float(rp[e]) - dl) * p.scale;
        }
      }
      if (j >= 2 && !tt::mbar_wait(bar(QB_DSFREE + t2), ((j - 2) >> 1) & 1, abort_flag, &g_attn_error, 27)) { ok = false; break; }
      store_halfrow_sw128(gbase + Q_DS + t2 * 16384, row, half, ds);
      tt::fence_proxy_async();
      tt::tc_fence_before();
      __syncwarp();
      if (lane == 0) tt::mbar_arrive(bar(QB_DSREADY + t2));
    }
    if (ok && n_kv > 0) ok = tt::mbar_wait(bar(QB_DSFREE + ((n_kv - 1) & 1)), ((n_kv - 1) >> 1) & 1, abort_flag, &g_attn_error, 28);
    tt::tc_fence_after();
    if (ok) {
      __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.out) + ((static_cast<long long>(b) * p.Sq + qi) * p.H + h) * DQK;
      constexpr int CH = DQK / 64;    // 32-column chunks per warp half
#pragma unroll 1
      for (int c = half * CH; c < half * CH + CH; ++c) {
        uint32_t r[32];
        if (n_kv > 0) { tt::tmem_ld_32x32(tDQ + lane_off + c * 32, r); tt::tc_wait_ld(); }
        else {
#pragma unroll
          for (int e = 0; e < 32; ++e) r[e] = 0;
        }
        store_out_32(orow + c * 32, r);
      }
    }
    tt::tc_fence_before();
  }
  __syncthreads();
  if (*abort_flag) tt::abort_drain();
  if (warp == 1) { tt::tc_fence_after(); tt::tmem_dealloc(tmem, 512); }
}

// =================================================================================== backward: dK, dV
// CTA = 128 key rows of one KV head; steps over (query head of the group, 64-row query tile).
// smem: K 32K | V 32K | Q/dO ring NS x (16K + 16K) | P^T 2x16K | dS^T 2x16K | barriers
// (per-query lse / delta are read straight from global memory: warp-uniform, L1-resident loads)
constexpr int K_NS = 3;
constexpr uint32_t K_K = 0, K_V = 32768, K_QDO = 65536, K_PT = K_QDO + K_NS * 32768, K_DST = K_PT + 32768,
                   K_BAR = K_DST + 32768;
constexpr size_t DKV_SMEM = 1024 + K_BAR + 256;
constexpr int KB_KVFULL = 0, KB_QFULL = 1, KB_QEMPTY = KB_QFULL + K_NS, KB_STFULL = KB_QEMPTY + K_NS,
              KB_PTREADY = KB_STFULL + 2, KB_PTFREE = KB_PTREADY + 2, KB_COUNT = KB_PTFREE + 2;

__global__ void __launch_bounds__(320, 1)
attn_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tdo,
                    const __grid_constant__ CUtensorMap tk, const __grid_constant__ CUtensorMap tv, AttnArgs p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (tt::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (base - tt::smem_u32(smem_raw));
  const uint32_t bar0 = base + K_BAR;
  auto bar = [&](int i) { return bar0 + 8u * i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gbase + K_BAR + 8 * KB_COUNT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gbase + K_BAR + 8 * KB_COUNT + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kt = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int G = p.H / p.Hkv;
  const int kv0 = kt * 128;
  const int off = p.Sk - p.Sq;
  const int nq_tiles = p.Sq / 64;
  int qt_first = 0;
  if (p.causal) { const int first_q = kv0 - off; qt_first = first_q > 0 ? first_q / 64 : 0; }
  // range mask: the last key of the tile is seen furthest; later query tiles are skipped
  int qt_end = nq_tiles;
  if (p.col_hi) qt_end = min(nq_tiles, __ldg(p.col_hi + static_cast<long long>(b) * p.Sk + kv0 + 127) / 64 + 1);
  const int per_head = qt_end > qt_first ? qt_end - qt_first : 0;
  const int n_steps = per_head * G;

  if (threadIdx.x == 0) {
    for (int i = 0; i < KB_COUNT; ++i) tt::mbar_init(bar(i), (i >= KB_PTREADY && i < KB_PTFREE) ? 8 : 1);
    *abort_flag = 0;
    tt::mbar_fence_init();
  }
  if (warp == 1) { tt::tmem_alloc(tt::smem_u32(tmem_slot), 512); tt::tmem_relinquish(); }
  tt::tc_fence_before();
  __syncthreads();
  tt::tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  // TMEM columns: S^T[2] at 0,64 | dP^T[2] at 128,192 | dV 256..383 | dK 384..511
  const uint32_t tST = tmem, tDPT = tmem + 128, tDV = tmem + 256, tDK = tmem + 384;

  if (warp == 0) {
    if (tt::elect_one()) {
      tt::mbar_expect_tx(bar(KB_KVFULL), 65536);
      tt::tma_load_3d(base + K_K, &tk, bar(KB_KVFULL), 0, hk, b * p.Sk + kv0);
      tt::tma_load_3d(base + K_K + 16384, &tk, bar(KB_KVFULL), 64, hk, b * p.Sk + kv0);
      tt::tma_load_3d(base + K_V, &tv, bar(KB_KVFULL), 0, hk, b * p.Sk + kv0);
      tt::tma_load_3d(base + K_V + 16384, &tv, bar(KB_KVFULL), 64, hk, b * p.Sk + kv0);
      for (int st = 0; st < n_steps; ++st) {
        const int s = st % K_NS; const uint32_t ph = (st / K_NS) & 1;
        const int h = hk * G + st / per_head, qt = qt_first + st % per_head;
        if (!tt::mbar_wait(bar(KB_QEMPTY + s), ph ^ 1, abort_flag, &g_attn_error, 31)) break;
        const uint32_t qb = base + K_QDO + s * 32768, dob = qb + 16384;
        tt::mbar_expect_tx(bar(KB_QFULL + s), 32768);
        tt::tma_load_3d(qb, &tq, bar(KB_QFULL + s), 0, h, b * p.Sq + qt * 64);
        tt::tma_load_3d(qb + 8192, &tq, bar(KB_QFULL + s), 64, h, b * p.Sq + qt * 64);
        tt::tma_load_3d(dob, &tdo, bar(KB_QFULL + s), 0, h, b * p.Sq + qt * 64);
        tt::tma_load_3d(dob + 8192, &tdo, bar(KB_QFULL + s), 64, h, b * p.Sq + qt * 64);
      }
    }
  } else if (warp == 1) {
    if (tt::elect_one()) {
      bool ok = tt::mbar_wait(bar(KB_KVFULL), 0, abort_flag, &g_attn_error, 32);
      auto issue_st = [&](int st) -> bool {
        const int s = st % K_NS, t2 = st & 1;
        if (!tt::mbar_wait(bar(KB_QFULL + s), (st / K_NS) & 1, abort_flag, &g_attn_error, 33)) return false;
        tt::tc_fence_after();
        const uint32_t qb = base + K_QDO + s * 32768, dob = qb + 16384;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          tt::umma_f16_ss(tST + t2 * 64, desc_kmajor_dh(base + K_K, 128, kk), desc_kmajor_dh(qb, 64, kk), IDESC_128x64_KK, kk != 0);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          tt::umma_f16_ss(tDPT + t2 * 64, desc_kmajor_dh(base + K_V, 128, kk), desc_kmajor_dh(dob, 64, kk), IDESC_128x64_KK, kk != 0);
        tt::umma_commit(bar(KB_STFULL + t2));
        return true;
      };
      if (ok && n_steps > 0) ok = issue_st(0);
      for (int st = 0; st < n_steps && ok; ++st) {
        if (st + 1 < n_steps && !issue_st(st + 1)) break;
        const int s = st % K_NS, t2 = st & 1;
        if (!tt::mbar_wait(bar(KB_PTREADY + t2), (st >> 1) & 1, abort_flag, &g_attn_error, 35)) break;
        tt::tc_fence_after();
        const uint32_t qb = base + K_QDO + s * 32768, dob = qb + 16384;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          tt::umma_f16_ss(tDV, desc_kmajor_64(base + K_PT + t2 * 16384, kk), desc_mnmajor(dob, 64, kk), IDESC_128x128_KM, (st | kk) != 0);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          tt::umma_f16_ss(tDK, desc_kmajor_64(base + K_DST + t2 * 16384, kk), desc_mnmajor(qb, 64, kk), IDESC_128x128_KM, (st | kk) != 0);
        tt::umma_commit(bar(KB_PTFREE + t2));   // P^T / dS^T buffers free
        tt::umma_commit(bar(KB_QEMPTY + s));    // Q / dO stage free
      }
    }
  } else {
    // 8 softmax warps: lane group = warp & 3 (key row), column half = (warp - 2) >> 2 (32 queries each)
    const int lg = warp & 3, row = lg * 32 + lane, half = (warp - 2) >> 2;
    const uint32_t lane_off = static_cast<uint32_t>(lg * 32) << 16;
    const int ki = kv0 + row;
    const float sc = p.scale * kLog2e;
    const int hi = p.col_hi ? __ldg(p.col_hi + static_cast<long long>(b) * p.Sk + ki) : 0x7fffffff;
    bool ok = true;
    for (int st = 0; st < n_steps; ++st) {
      const int t2 = st & 1;
      const int h = hk * G + st / per_head, qt = qt_first + st % per_head;
      const int qbase = qt * 64 + half * 32;
      const float* lse_g = p.lse + (static_cast<long long>(b) * p.H + h) * p.Sq + qbase;
      const float* dl_g = p.delta + (static_cast<long long>(b) * p.H + h) * p.Sq + qbase;
      if (!tt::mbar_wait(bar(KB_STFULL + t2), (st >> 1) & 1, abort_flag, &g_attn_error, 37)) { ok = false; break; }
      tt::tc_fence_after();
      float pt[32], dst[32];
      {
        uint32_t rs[32], rp[32];
        tt::tmem_ld_32x32(tST + lane_off + t2 * 64 + half * 32, rs);
        tt::tmem_ld_32x32(tDPT + lane_off + t2 * 64 + half * 32, rp);
        tt::tc_wait_ld();
#pragma unroll
        for (int e4 = 0; e4 < 8; ++e4) {
          const float4 l4 = __ldg(reinterpret_cast<const float4*>(lse_g) + e4);
          const float4 d4 = __ldg(reinterpret_cast<const float4*>(dl_g) + e4);
          const float ls[4] = {l4.x, l4.y, l4.z, l4.w}, dd[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int e = e4 * 4 + u;
            float pr = fast_exp2(__uint_as_float(rs[e]) * sc - ls[u] * kLog2e);
            if ((p.causal && ki > qbase + e + off) || qbase + e > hi) pr = 0.f;
            pt[e] = pr;
            dst[e] = pr * (__uint_as_float(rp[e]) - dd[u]) * p.scale;
          }
        }
      }
      if (st >= 2 && !tt::mbar_wait(bar(KB_PTFREE + t2), ((st - 2) >> 1) & 1, abort_flag, &g_attn_error, 36)) { ok = false; break; }
      store_halfrow_sw128(gbase + K_PT + t2 * 16384, row, half, pt);
      store_halfrow_sw128(gbase + K_DST + t2 * 16384, row, half, dst);
      tt::fence_proxy_async();
      tt::tc_fence_before();
      __syncwarp();
      if (lane == 0) tt::mbar_arrive(bar(KB_PTREADY + t2));
    }
    if (ok && n_steps > 0) ok = tt::mbar_wait(bar(KB_PTFREE + ((n_steps - 1) & 1)), ((n_steps - 1) >> 1) & 1, abort_flag, &g_attn_error, 38);
    tt::tc_fence_after();
    if (ok) {
      const long long o = ((static_cast<long long>(b) * p.Sk + ki) * p.Hkv + hk) * D;
      __nv_bfloat16* dk = reinterpret_cast<__nv_bfloat16*>(p.out) + o;
      __nv_bfloat16* dv = reinterpret_cast<__nv_bfloat16*>(p.out2) + o;
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        __nv_bfloat16* dstp = which ? dk : dv;
        const uint32_t t = which ? tDK : tDV;
#pragma unroll 1
        for (int c = half * 2; c < half * 2 + 2; ++c) {
          uint32_t r[32];
          if (n_steps > 0) { tt::tmem_ld_32x32(t + lane_off + c * 32, r); tt::tc_wait_ld(); }
          else {
#pragma unroll
            for (int e = 0; e < 32; ++e) r[e] = 0;
          }
          store_out_32(dstp + c * 32, r);
        }
      }
    }
    tt::tc_fence_before();
  }
  __syncthreads();
  if (*abort_flag) tt::abort_drain();
  if (warp == 1) { tt::tc_fence_after(); tt::tmem_dealloc(tmem, 512); }
}

// =================================================================================== backward: fused dK, dV and dQ
// One pass over the (key tile, query tile) pairs instead of two: the CTA of a key tile also forms that pair's share of
// dQ, so S^T and dP^T are computed once per pair (5 MMAs per pair instead of 4 + 3 in the two-kernel form above).
//   dQ^T[d, q] = K^T[d, keys] * dS^T[keys, q]      (A = the K tile read MN-major, B = the dS^T tile read MN-major)
// lands in TMEM with the head dimension on the lanes. Four drain warps move it through a 16 KB shared-memory staging
// tile ([32 queries][128 d] fp32, two halves per step) and add it to the fp32 dQ accumulator in global memory with bulk
// reduce-add copies (cp.reduce.async.bulk ... add.f32, one 512-byte row per copy): the memory system adds whole lines,
// which per-element atomics do far slower. The sum over key tiles is formed by those additions, in no fixed order: the
// low bits of dQ differ from run to run (the two-kernel form stays available for deterministic runs). A small kernel
// converts the accumulator to bf16 afterwards.
// S^T / dP^T are single-buffered in TMEM but released as soon as the softmax warps hold them in registers, so the
// MMAs of step st + 1 start while step st is still in the softmax. P^T is single-buffered in shared memory (its MMA,
// dV, is the first of a step's second group and frees it early); dS^T is double-buffered.
// smem: K 32K | V 32K | Q/dO ring 3 x 32K | P^T 16K | dQ staging 16K | dS^T 2 x 16K | barriers.
// TMEM columns: S^T 0..63 | dP^T 64..127 | dQ^T 128..191 | dV 256..383 | dK 384..511.
constexpr int FB_KVFULL = 0, FB_QFULL = 1, FB_QEMPTY = FB_QFULL + K_NS, FB_STFULL = FB_QEMPTY + K_NS,
              FB_STFREE = FB_STFULL + 1, FB_PTREADY = FB_STFREE + 1, FB_PTFREE = FB_PTREADY + 2,
              FB_DQFULL = FB_PTFREE + 2, FB_DQFREE = FB_DQFULL + 1, FB_PFREE = FB_DQFREE + 1, FB_COUNT = FB_PFREE + 1;
// Head dimensions are template parameters (see the forward kernel). WITH_DQ = false leaves dQ to the separate dQ kernel
// (used for the head dimensions other than 128, where dQ^T would need an MMA with M = 64 or 192): the kernel is then
// free of atomics, and the staging tile and the shared-memory P^T buffer are not allocated.
template <int DQK, int DV, bool WITH_DQ>
struct FusedLayout {
  static constexpr int QC = DQK / 64, VC = DV / 64;
  static constexpr uint32_t K = 0, V = QC * 16384, QDO = V + VC * 16384, DOOFF = QC * 8192, STAGE = (QC + VC) * 8192;
  static constexpr uint32_t EXTRA = WITH_DQ ? 32768 : 0;   // P^T buffer + dQ staging tile
  static constexpr int NS = (QDO + 3 * STAGE + EXTRA + 32768 <= 224 * 1024) ? 3 : 2;
  static constexpr uint32_t PT = QDO + NS * STAGE, DQS = PT + 16384, DST = PT + EXTRA, BAR = DST + 32768,
                            STAT = BAR + 256;   // per stage: 64 x (-lse * log2 e) then 64 x (-delta * scale), fp32
  static constexpr size_t SMEM = 1024 + STAT + NS * 512;
};
constexpr uint32_t IDESC_128x64_MM = tt::umma_idesc_bf16(128, 64, 1, 1);
constexpr int FUSED_THREADS = 448;   // TMA, MMA, 8 softmax warps, 4 drain warps

// Optional timeline probe (compiled only with -DTT_ATTN_TRACE): block (0,0,0) records the SM clock at a few points of
// steps [64, 72) into g_attn_trace[step - 64][slot].
#ifdef TT_ATTN_TRACE
__device__ long long g_attn_trace[8][16];
#define TT_TRACE(st, slot)                                                                                     \
  do {                                                                                                         \
    if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (st) >= 64 && (st) < 72 && (threadIdx.x & 31) == 0) \
      g_attn_trace[(st) - 64][slot] = clock64();                                                               \
  } while (0)
#else
#define TT_TRACE(st, slot) do {} while (0)
#endif

struct FusedExtra {
  const float* lse2;     // [B,H,Sq] -lse * log2(e)
  const float* delta_s;  // [B,H,Sq] -delta * scale
  float* dq_acc;         // [B,Sq,H,D] fp32, zero on entry
  int dq_mode;           // 0: tiled TMA reduce-add through shared memory; 1: one atomic add per element; 2: dQ dropped (timing aid)
  int a_tmem;            // 1: P^T and dS^T reach the dV / dK MMAs through tensor memory (no shared-memory reads for A)
};

// Tiled reduce-add of a shared-memory box into a 3-D fp32 tensor in global memory (one instruction per box).
__device__ __forceinline__ void tma_reduce_add_3d(const CUtensorMap* m, uint32_t src_smem, int c0, int c1, int c2) {
  asm volatile("cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(src_smem), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
// Two fp32 lanes per instruction (sm_100 packed math): halves the issue slots of the softmax arithmetic.
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
  unsigned long long d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d)
      : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)),
        "l"(*reinterpret_cast<unsigned long long*>(&c)));
  return *reinterpret_cast<float2*>(&d);
}
__device__ __forceinline__ float2 fmul2(float2 a, float2 b) {
  unsigned long long d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d)
      : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)));
  return *reinterpret_cast<float2*>(&d);
}
// 32 atomic adds, one query row apart (QS floats; 0 = the run-time stride): with a compile-time stride the offsets are
// immediates and no address arithmetic is issued.
template <int QS>
__device__ __forceinline__ void red_rows(float* dst, long long qstride, const uint32_t (&r)[32]) {
#pragma unroll
  for (int c = 0; c < 32; ++c) atomicAdd(dst + c * (QS ? static_cast<long long>(QS) : qstride), __uint_as_float(r[c]));
}

template <int DQK, int DV, bool WITH_DQ>
__global__ void __launch_bounds__(FUSED_THREADS, 1)
attn_bwd_fused_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tdo,
                      const __grid_constant__ CUtensorMap tk, const __grid_constant__ CUtensorMap tv,
                      const __grid_constant__ CUtensorMap tdq, AttnArgs p, FusedExtra x) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (tt::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (base - tt::smem_u32(smem_raw));
  using L = FusedLayout<DQK, DV, WITH_DQ>;
  constexpr int K_NS = L::NS;
  constexpr uint32_t K_K = L::K, K_V = L::V, K_QDO = L::QDO, K_PT = L::PT, K_DQS = L::DQS, K_DST = L::DST, K_BAR = L::BAR,
                     K_STAT = L::STAT;
  constexpr uint32_t IDESC_DV = tt::umma_idesc_bf16(128, DV, 0, 1), IDESC_DK = tt::umma_idesc_bf16(128, DQK, 0, 1);
  const bool a_tmem = !WITH_DQ || x.a_tmem;      // without the shared-memory P^T buffer the A operands must come from TMEM
  const uint32_t bar0 = base + K_BAR;
  auto bar = [&](int i) { return bar0 + 8u * i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gbase + K_BAR + 8 * FB_COUNT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gbase + K_BAR + 8 * FB_COUNT + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // the KV head is the fastest block index: under a causal mask the blocks run from the heaviest key tile (all
  // queries) to the lightest, over all heads, so the SMs finish close together
  const int hk = blockIdx.x, kt = blockIdx.y, b = blockIdx.z;
  const int G = p.H / p.Hkv;
  const int kv0 = kt * 128;
  const int off = p.Sk - p.Sq;
  const int nq_tiles = p.Sq / 64;
  int qt_first = 0;
  if (p.causal) { const int first_q = kv0 - off; qt_first = first_q > 0 ? first_q / 64 : 0; }
  int qt_end = nq_tiles;
  if (p.col_hi) qt_end = min(nq_tiles, __ldg(p.col_hi + static_cast<long long>(b) * p.Sk + kv0 + 127) / 64 + 1);
  const int per_head = qt_end > qt_first ? qt_end - qt_first : 0;
  const int n_steps = per_head * G;
  // step st <-> (query head h, query tile qt): every role walks the same sequence with counters (no divisions)
  int h = hk * G, qt = qt_first;
  auto next_step = [&]() { if (++qt == qt_end) { qt = qt_first; ++h; } };

  if (threadIdx.x == 0) {
    for (int i = 0; i < FB_COUNT; ++i) {
      uint32_t cnt = 1;
      if (i == FB_STFREE || (i >= FB_PTREADY && i < FB_PTFREE)) cnt = 8;   // one arrival per softmax warp
      if (i == FB_DQFREE) cnt = 4;                                         // one per drain warp
      tt::mbar_init(bar(i), cnt);
    }
    *abort_flag = 0;
    tt::mbar_fence_init();
  }
  if (warp == 1) { tt::tmem_alloc(tt::smem_u32(tmem_slot), 512); tt::tmem_relinquish(); }
  tt::tc_fence_before();
  __syncthreads();
  tt::tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  // with dQ: S^T 0 | dP^T 64 | dQ^T 128 | P^T 192 | dS^T 224 | dV 256 | dK 384; without: S^T 0 | dP^T 64 | P^T 128 |
  // dS^T 160 | dV 192 | dK 192 + DV (bf16 P^T / dS^T as A operands: 64 queries = 32 columns each)
  const uint32_t tST = tmem, tDPT = tmem + 64, tDQT = tmem + 128;
  const uint32_t tPT = tmem + (WITH_DQ ? 192 : 128), tDST = tPT + 32;
  const uint32_t tDV = tmem + (WITH_DQ ? 256 : 192), tDK = tDV + DV;

  if (warp == 0) {
    if (tt::elect_one()) {
      tt::mbar_expect_tx(bar(FB_KVFULL), (L::QC + L::VC) * 16384);
#pragma unroll
      for (int c = 0; c < L::QC; ++c) tt::tma_load_3d(base + K_K + c * 16384, &tk, bar(FB_KVFULL), c * 64, hk, b * p.Sk + kv0);
#pragma unroll
      for (int c = 0; c < L::VC; ++c) tt::tma_load_3d(base + K_V + c * 16384, &tv, bar(FB_KVFULL), c * 64, hk, b * p.Sk + kv0);
      for (int st = 0; st < n_steps; ++st, next_step()) {
        const int s = st % K_NS; const uint32_t ph = (st / K_NS) & 1;
        if (!tt::mbar_wait(bar(FB_QEMPTY + s), ph ^ 1, abort_flag, &g_attn_error, 41)) break;
        const uint32_t qb = base + K_QDO + s * L::STAGE, dob = qb + L::DOOFF;
        tt::mbar_expect_tx(bar(FB_QFULL + s), L::STAGE + 512);
        {
          // the 64 queries' softmax statistics ride on the same barrier (plain bulk copies, 256 bytes each)
          const long long so = (static_cast<long long>(b) * p.H + h) * p.Sq + qt * 64;
          tt::bulk_load(base + K_STAT + s * 512, x.lse2 + so, 256, bar(FB_QFULL + s));
          tt::bulk_load(base + K_STAT + s * 512 + 256, x.delta_s + so, 256, bar(FB_QFULL + s));
        }
#pragma unroll
        for (int c = 0; c < L::QC; ++c) tt::tma_load_3d(qb + c * 8192, &tq, bar(FB_QFULL + s), c * 64, h, b * p.Sq + qt * 64);
#pragma unroll
        for (int c = 0; c < L::VC; ++c) tt::tma_load_3d(dob + c * 8192, &tdo, bar(FB_QFULL + s), c * 64, h, b * p.Sq + qt * 64);
      }
    }
  } else if (warp == 1) {
    if (tt::elect_one()) {
      bool ok = tt::mbar_wait(bar(FB_KVFULL), 0, abort_flag, &g_attn_error, 42);
      // descriptors are built once; inside the loop an operand slice is one 32-bit add away (see tt::SmemDesc)
      const tt::SmemDesc dK_km = tt::make_smem_desc(base + K_K, 1, 64), dV_km = tt::make_smem_desc(base + K_V, 1, 64);
      const tt::SmemDesc dK_mn = tt::make_smem_desc(base + K_K, (128 * 128) >> 4, 64);
      const tt::SmemDesc dQ_km0 = tt::make_smem_desc(base + K_QDO, 1, 64);              // stage 0: Q; dO follows Q's chunks
      const tt::SmemDesc dQ_mn0 = tt::make_smem_desc(base + K_QDO, (64 * 128) >> 4, 64);
      const tt::SmemDesc dPT_km = tt::make_smem_desc(base + K_PT, 1, 64);
      const tt::SmemDesc dDS_km0 = tt::make_smem_desc(base + K_DST, 1, 64);
      const tt::SmemDesc dDS_mn0 = tt::make_smem_desc(base + K_DST, (128 * 128) >> 4, 64);
      // S^T and dP^T of step st; the TMEM buffers must have been read out by the softmax warps of step st - 1
      auto issue_st = [&](int st) -> bool {
        const int s = st % K_NS;
        if (!tt::mbar_wait(bar(FB_QFULL + s), (st / K_NS) & 1, abort_flag, &g_attn_error, 43)) return false;
        if (st > 0 && !tt::mbar_wait(bar(FB_STFREE), (st - 1) & 1, abort_flag, &g_attn_error, 44)) return false;
        tt::tc_fence_after();
        TT_TRACE(st, 0);   // S^T / dP^T issue begins
        const tt::SmemDesc q = dQ_km0.at(s * L::STAGE), dO = q.at(L::DOOFF);
        // K-major operands with two 64-wide halves of the head dimension: slice kk starts at
        // (kk >> 2) * rows * 128 + (kk & 3) * 32 bytes (rows = 128 for K / V, 64 for Q / dO)
#pragma unroll
        for (int kk = 0; kk < DQK / 16; ++kk)
          tt::umma_f16_ss(tST, dK_km.at((kk >> 2) * 16384 + (kk & 3) * 32), q.at((kk >> 2) * 8192 + (kk & 3) * 32),
                          IDESC_128x64_KK, kk != 0);
#pragma unroll
        for (int kk = 0; kk < DV / 16; ++kk)
          tt::umma_f16_ss(tDPT, dV_km.at((kk >> 2) * 16384 + (kk & 3) * 32), dO.at((kk >> 2) * 8192 + (kk & 3) * 32),
                          IDESC_128x64_KK, kk != 0);
        tt::umma_commit(bar(FB_STFULL));
        TT_TRACE(st, 1);   // S^T / dP^T issued
        return true;
      };
      if (ok && n_steps > 0) ok = issue_st(0);
      for (int st = 0; st < n_steps && ok; ++st) {
        if (st + 1 < n_steps && !issue_st(st + 1)) break;
        const int s = st % K_NS, t2 = st & 1;
        if (!tt::mbar_wait(bar(FB_PTREADY + t2), (st >> 1) & 1, abort_flag, &g_attn_error, 45)) break;
        tt::tc_fence_after();
        TT_TRACE(st, 2);   // P^T / dS^T seen ready
        const tt::SmemDesc q_mn = dQ_mn0.at(s * L::STAGE), dO_mn = q_mn.at(L::DOOFF);
        const tt::SmemDesc ds_km = dDS_km0.at(t2 * 16384), ds_mn = dDS_mn0.at(t2 * 16384);
        const uint32_t acc0 = st != 0;
        if (a_tmem) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            tt::umma_f16_ts(tDV, tPT + kk * 8, dO_mn.at(kk * 2048), IDESC_DV, kk ? 1u : acc0);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            tt::umma_f16_ts(tDK, tDST + kk * 8, q_mn.at(kk * 2048), IDESC_DK, kk ? 1u : acc0);
          tt::umma_commit(bar(FB_PFREE));       // P^T and dS^T (tensor memory) free for the next step's softmax
        } else {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            tt::umma_f16_ss(tDV, dPT_km.at(kk * 32), dO_mn.at(kk * 2048), IDESC_DV, kk ? 1u : acc0);
          tt::umma_commit(bar(FB_PFREE));       // P^T buffer free for the next step's softmax
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            tt::umma_f16_ss(tDK, ds_km.at(kk * 32), q_mn.at(kk * 2048), IDESC_DK, kk ? 1u : acc0);
        }
        if constexpr (WITH_DQ) {
          // dQ^T overwrites what the drain warps read for the previous step: wait for them as late as possible
          if (st > 0 && !tt::mbar_wait(bar(FB_DQFREE), (st - 1) & 1, abort_flag, &g_attn_error, 46)) break;
          tt::tc_fence_after();
          TT_TRACE(st, 3);   // dQ^T buffer seen free
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            tt::umma_f16_ss(tDQT, dK_mn.at(kk * 2048), ds_mn.at(kk * 2048), IDESC_128x64_MM, kk != 0);
          tt::umma_commit(bar(FB_DQFULL));      // dQ^T of this step complete
        }
        tt::umma_commit(bar(FB_PTFREE + t2));   // dS^T buffer free
        tt::umma_commit(bar(FB_QEMPTY + s));    // Q / dO stage free
        TT_TRACE(st, 4);   // second group issued
      }
    }
  } else if (warp < 10) {
    // 8 softmax warps: lane group = warp & 3 (key row), column half = (warp - 2) >> 2 (32 queries each)
    const int lg = warp & 3, row = lg * 32 + lane, half = (warp - 2) >> 2;
    const uint32_t lane_off = static_cast<uint32_t>(lg * 32) << 16;
    const int ki = kv0 + row;
    const float sc = p.scale * kLog2e;
    const int hi = p.col_hi ? __ldg(p.col_hi + static_cast<long long>(b) * p.Sk + ki) : 0x7fffffff;
    bool ok = true;
    const float2 sc2 = make_float2(sc, sc), scale2 = make_float2(p.scale, p.scale);
    for (int st = 0; st < n_steps; ++st, next_step()) {
      const int t2 = st & 1;
      const int qbase = qt * 64 + half * 32;
      // statistics of this step's queries: staged by the producer next to Q / dO (visible once S^T is: the MMA
      // warp waited for the stage's barrier before it issued S^T)
      const float4* lse_s = reinterpret_cast<const float4*>(gbase + K_STAT + (st % K_NS) * 512) + half * 8;
      const float4* dl_s = lse_s + 16;
      if (!tt::mbar_wait(bar(FB_STFULL), st & 1, abort_flag, &g_attn_error, 47)) { ok = false; break; }
      // the stage's own barrier completed before S^T was issued: this wait returns at once and orders the reads of
      // the bulk-copied statistics after the copies
      if (!tt::mbar_wait(bar(FB_QFULL + st % K_NS), (st / K_NS) & 1, abort_flag, &g_attn_error, 52)) { ok = false; break; }
      tt::tc_fence_after();
      if (warp == 2) TT_TRACE(st, 5);   // S^T seen complete
      uint32_t rs[32], rp[32];
      tt::tmem_ld_32x32(tST + lane_off + half * 32, rs);
      tt::tmem_ld_32x32(tDPT + lane_off + half * 32, rp);
      tt::tc_wait_ld();
      tt::tc_fence_before();
      __syncwarp();
      if (lane == 0) tt::mbar_arrive(bar(FB_STFREE));      // the next step's S^T / dP^T may overwrite TMEM now
      if (warp == 2) TT_TRACE(st, 6);   // TMEM read out
      // only tiles that touch the diagonal (or a range bound) need per-element masks: two versions of the loop
      const bool masked = (p.causal && kv0 + 127 > qt * 64 + off) || p.col_hi != nullptr;
      uint32_t pp[16], dd[16];   // packed bf16 pairs: P^T and dS^T of this thread's 32 queries
      if (!masked) {
#pragma unroll
        for (int e4 = 0; e4 < 8; ++e4) {
          const float4 l4 = lse_s[e4];   // -lse * log2(e)
          const float4 d4 = dl_s[e4];    // -delta * scale
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int e = e4 * 4 + 2 * u;
            const float2 xx = ffma2(make_float2(__uint_as_float(rs[e]), __uint_as_float(rs[e + 1])), sc2,
                                    u ? make_float2(l4.z, l4.w) : make_float2(l4.x, l4.y));
            const float2 pr = make_float2(fast_exp2(xx.x), fast_exp2(xx.y));
            const float2 tt2 = ffma2(make_float2(__uint_as_float(rp[e]), __uint_as_float(rp[e + 1])), scale2,
                                     u ? make_float2(d4.z, d4.w) : make_float2(d4.x, d4.y));
            const float2 ds = fmul2(pr, tt2);
            pp[2 * e4 + u] = tt::pack_bf16(pr.x, pr.y);
            dd[2 * e4 + u] = tt::pack_bf16(ds.x, ds.y);
          }
        }
      } else {
#pragma unroll
        for (int e4 = 0; e4 < 8; ++e4) {
          const float4 l4 = lse_s[e4];
          const float4 d4 = dl_s[e4];
          const float ls[4] = {l4.x, l4.y, l4.z, l4.w}, dl[4] = {d4.x, d4.y, d4.z, d4.w};
          float pr[4], ds[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int e = e4 * 4 + u;
            pr[u] = fast_exp2(fmaf(__uint_as_float(rs[e]), sc, ls[u]));
            if ((p.causal && ki > qbase + e + off) || qbase + e > hi) pr[u] = 0.f;
            ds[u] = pr[u] * fmaf(__uint_as_float(rp[e]), p.scale, dl[u]);
          }
          pp[2 * e4] = tt::pack_bf16(pr[0], pr[1]); pp[2 * e4 + 1] = tt::pack_bf16(pr[2], pr[3]);
          dd[2 * e4] = tt::pack_bf16(ds[0], ds[1]); dd[2 * e4 + 1] = tt::pack_bf16(ds[2], ds[3]);
        }
      }
      if (warp == 2) TT_TRACE(st, 7);   // arithmetic done
      if (st >= 1 && !tt::mbar_wait(bar(FB_PFREE), (st - 1) & 1, abort_flag, &g_attn_error, 51)) { ok = false; break; }
      if (st >= 2 && !tt::mbar_wait(bar(FB_PTFREE + t2), ((st - 2) >> 1) & 1, abort_flag, &g_attn_error, 48)) { ok = false; break; }
      {
        uint8_t* prow = gbase + K_PT + row * 128;
        uint8_t* drow = gbase + K_DST + t2 * 16384 + row * 128;
        const int xr = row & 7;
        if (a_tmem) {
          // A operands of dV / dK straight into tensor memory: this thread's key row = its lane, 32 queries = 16 columns
          tt::tmem_st_32x16(tPT + lane_off + half * 16, pp);
          tt::tmem_st_32x16(tDST + lane_off + half * 16, dd);
        }
        if (WITH_DQ || !a_tmem) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int chunk = ((half * 4 + c) ^ xr) << 4;
            if (!a_tmem) *reinterpret_cast<uint4*>(prow + chunk) = make_uint4(pp[4 * c], pp[4 * c + 1], pp[4 * c + 2], pp[4 * c + 3]);
            *reinterpret_cast<uint4*>(drow + chunk) = make_uint4(dd[4 * c], dd[4 * c + 1], dd[4 * c + 2], dd[4 * c + 3]);   // B operand of dQ^T
          }
        }
        if (a_tmem) tt::tc_wait_st();
      }
      tt::fence_proxy_async();
      tt::tc_fence_before();
      __syncwarp();
      if (lane == 0) tt::mbar_arrive(bar(FB_PTREADY + t2));
      if (warp == 2) TT_TRACE(st, 8);   // P^T / dS^T published
    }
    if (ok && n_steps > 0) ok = tt::mbar_wait(bar(FB_PTFREE + ((n_steps - 1) & 1)), ((n_steps - 1) >> 1) & 1, abort_flag, &g_attn_error, 49);
    tt::tc_fence_after();
    if (ok) {
      const long long orow = (static_cast<long long>(b) * p.Sk + ki) * p.Hkv + hk;
      __nv_bfloat16* dk = reinterpret_cast<__nv_bfloat16*>(p.out) + orow * DQK;
      __nv_bfloat16* dv = reinterpret_cast<__nv_bfloat16*>(p.out2) + orow * DV;
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        __nv_bfloat16* dstp = which ? dk : dv;
        const uint32_t t = which ? tDK : tDV;
        const int ch = (which ? DQK : DV) / 64;         // 32-column chunks per warp half
#pragma unroll 1
        for (int c = half * ch; c < half * ch + ch; ++c) {
          uint32_t r[32];
          if (n_steps > 0) { tt::tmem_ld_32x32(t + lane_off + c * 32, r); tt::tc_wait_ld(); }
          else {
#pragma unroll
            for (int e = 0; e < 32; ++e) r[e] = 0;
          }
          store_out_32(dstp + c * 32, r);
        }
      }
    }
    tt::tc_fence_before();
  } else if constexpr (WITH_DQ) {
    // 4 drain warps: lane = head-dim index d of dQ^T; add this step's [64 queries x 128 d] to the fp32 accumulator
    const int lg = warp & 3, d = lg * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(lg * 32) << 16;
    float* stage = reinterpret_cast<float*>(gbase + K_DQS);
    const uint32_t stage_u32 = base + K_DQS;
    const long long qstride = static_cast<long long>(p.H) * D;
    const bool issuer = (warp == 10) && lane == 0;   // issues (and tracks) the tiled reduce copies
    for (int st = 0; st < n_steps; ++st, next_step()) {
      if (!tt::mbar_wait(bar(FB_DQFULL), st & 1, abort_flag, &g_attn_error, 50)) break;
      tt::tc_fence_after();
      if (warp == 10) TT_TRACE(st, 9);   // dQ^T seen complete
      float* dst0 = x.dq_acc + ((static_cast<long long>(b) * p.Sq + qt * 64) * p.H + h) * D + d;
      uint32_t r0[32], r1[32];
      tt::tmem_ld_32x32(tDQT + lane_off, r0);
      tt::tmem_ld_32x32(tDQT + lane_off + 32, r1);
      tt::tc_wait_ld();
      tt::tc_fence_before();
      __syncwarp();
      if (lane == 0) tt::mbar_arrive(bar(FB_DQFREE));       // dQ^T is in registers: the next step's MMA may overwrite it
      if (warp == 10) TT_TRACE(st, 10);  // dQ^T read out
#pragma unroll
      for (int hq = 0; hq < 2; ++hq) {
        const uint32_t (&r)[32] = hq ? r1 : r0;
        if (x.dq_mode == 0) {
          if (issuer) tt::bulk_store_wait_read<0>();         // the previous half's copy has read the staging tile
          asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll
          for (int c = 0; c < 32; ++c) stage[c * D + d] = __uint_as_float(r[c]);
          tt::fence_proxy_async();
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (issuer) {
            tma_reduce_add_3d(&tdq, stage_u32, 0, h, b * p.Sq + qt * 64 + hq * 32);
            tt::tma_store_commit();
          }
        } else if (x.dq_mode == 1) {
          float* dst = dst0 + hq * 32 * qstride;
          if (p.H == 32) red_rows<32 * D>(dst, qstride, r);
          else if (p.H == 16) red_rows<16 * D>(dst, qstride, r);
          else if (p.H == 64) red_rows<64 * D>(dst, qstride, r);
          else red_rows<0>(dst, qstride, r);
        }
      }
      if (warp == 10) TT_TRACE(st, 11);  // dQ handed to the memory system
    }
    if (issuer) tt::bulk_store_wait_all();                  // all additions have been performed before the kernel ends
    tt::tc_fence_before();
  }
  __syncthreads();
  if (*abort_flag) tt::abort_drain();
  if (warp == 1) { tt::tc_fence_after(); tt::tmem_dealloc(tmem, 512); }
}

// -delta[b,h,s] * scale (delta = sum_d dO * O) and -lse * log2(e): the addends of the fused backward's two FMAs
template <int DVT>
__global__ void attn_prep_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout,
                                 const float* __restrict__ lse, float* __restrict__ lse2, float* __restrict__ delta_s,
                                 float* __restrict__ delta, float scale, int B, int S, int H) {
  constexpr int LPR = DVT / 8;       // lanes per (b, s, h) row, 8 elements each
  const long long row = static_cast<long long>(blockIdx.x) * (blockDim.x / LPR) + threadIdx.x / LPR;
  const int l = threadIdx.x % LPR;
  const long long rows = static_cast<long long>(B) * S * H;
  float acc = 0.f;
  if (row < rows) {
    const uint4 a = *reinterpret_cast<const uint4*>(o + row * DVT + l * 8);
    const uint4 c = *reinterpret_cast<const uint4*>(dout + row * DVT + l * 8);
    const __nv_bfloat162* ah = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* ch = reinterpret_cast<const __nv_bfloat162*>(&c);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 xx = __bfloat1622float2(ah[i]), y = __bfloat1622float2(ch[i]);
      acc += xx.x * y.x + xx.y * y.y;
    }
  }
#pragma unroll
  for (int o2 = LPR / 2; o2 > 0; o2 >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o2);
  if (row < rows && l == 0) {
    const int hh = static_cast<int>(row % H);
    const long long bs = row / H;
    const int s = static_cast<int>(bs % S);
    const long long bb = bs / S;
    const long long i = (bb * H + hh) * S + s;
    delta_s[i] = -acc * scale;
    lse2[i] = -lse[i] * kLog2e;
    if (delta != nullptr) delta[i] = acc;    // plain form for the separate dQ kernel
  }
}

// fp32 dQ accumulator -> bf16
__global__ void attn_dq_convert_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq, long long n8) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float4 a = reinterpret_cast<const float4*>(acc)[2 * i], c = reinterpret_cast<const float4*>(acc)[2 * i + 1];
    uint4 v;
    v.x = tt::pack_bf16(a.x, a.y); v.y = tt::pack_bf16(a.z, a.w);
    v.z = tt::pack_bf16(c.x, c.y); v.w = tt::pack_bf16(c.z, c.w);
    reinterpret_cast<uint4*>(dq)[i] = v;
  }
}

// delta[b,h,s] = sum_d dO * O
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout,
                                  float* __restrict__ delta, int B, int S, int H) {
  const long long row = static_cast<long long>(blockIdx.x) * (blockDim.x / 16) + threadIdx.x / 16;  // (b,s,h)
  const int l16 = threadIdx.x & 15;
  const long long rows = static_cast<long long>(B) * S * H;
  float acc = 0.f;
  if (row < rows) {
    const uint4 a = *reinterpret_cast<const uint4*>(o + row * D + l16 * 8);
    const uint4 c = *reinterpret_cast<const uint4*>(dout + row * D + l16 * 8);
    const __nv_bfloat162* ah = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* ch = reinterpret_cast<const __nv_bfloat162*>(&c);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 x = __bfloat1622float2(ah[i]), y = __bfloat1622float2(ch[i]);
      acc += x.x * y.x + x.y * y.y;
    }
  }
#pragma unroll
  for (int o2 = 8; o2 > 0; o2 >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o2);
  if (row < rows && l16 == 0) {
    const int hh = static_cast<int>(row % H);
    const long long bs = row / H;
    const int s = static_cast<int>(bs % S);
    const long long bb = bs / S;
    delta[(bb * H + hh) * S + s] = acc;
  }
}

// [B*S, heads, 128] bf16 viewed as a 3-D tensor (d, head, row); box = (64, 1, box_rows), 128B swizzle
int make_map(CUtensorMap* m, const void* ptr, long long rows, int heads, int box_rows, int Dh = D) {
  tt::EncodeTiledFn fn = tt::encode_tiled_fn();
  if (!fn) return -1;
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(Dh), static_cast<cuuint64_t>(heads), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(Dh) * 2, static_cast<cuuint64_t>(heads) * Dh * 2};
  cuuint32_t box[3] = {64, 1, static_cast<cuuint32_t>(box_rows)};
  cuuint32_t es[3] = {1, 1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, es,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -static_cast<int>(r) - 1000;
}

bool g_attr_set = false;
int g_dq_mode = 0;
int g_a_tmem = 1;
void set_attrs() {
  if (g_attr_set) return;
  cudaFuncSetAttribute(attn_fwd_kernel<128, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(FwdLayout<128, 128>::SMEM));
  cudaFuncSetAttribute(attn_fwd_kernel<64, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(FwdLayout<64, 64>::SMEM));
  cudaFuncSetAttribute(attn_fwd_kernel<192, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(FwdLayout<192, 128>::SMEM));
  cudaFuncSetAttribute(attn_bwd_dq_kernel<128, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(DqLayout<128, 128>::SMEM));
  cudaFuncSetAttribute(attn_bwd_dq_kernel<64, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(DqLayout<64, 64>::SMEM));
  cudaFuncSetAttribute(attn_bwd_dq_kernel<192, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(DqLayout<192, 128>::SMEM));
  cudaFuncSetAttribute(attn_bwd_dkv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(DKV_SMEM));
  cudaFuncSetAttribute(attn_bwd_fused_kernel<128, 128, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(FusedLayout<128, 128, true>::SMEM));
  cudaFuncSetAttribute(attn_bwd_fused_kernel<64, 64, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(FusedLayout<64, 64, false>::SMEM));
  cudaFuncSetAttribute(attn_bwd_fused_kernel<192, 128, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(FusedLayout<192, 128, false>::SMEM));
  g_attr_set = true;
}

// Head dimensions the kernels are instantiated for: (query/key, value) = (128,128), (64,64), (192,128).
bool dims_ok(int Dqk, int Dv) { return (Dqk == 128 && Dv == 128) || (Dqk == 64 && Dv == 64) || (Dqk == 192 && Dv == 128); }

int check_shapes(int Sq, int Sk, int H, int Hkv, int Dh, int Dv = -1) {
  if (!dims_ok(Dh, Dv < 0 ? Dh : Dv)) return -10;
  if (Sq % 128 || Sk % 128) return -11;
  if (Hkv <= 0 || H % Hkv) return -12;
  return 0;
}

}  // namespace

extern "C" {

// Shapes this build of the kernels accepts (0 = yes).
int tt_attn_supported(int Sq, int Sk, int H, int Hkv, int Dh) { return check_shapes(Sq, Sk, H, Hkv, Dh); }
int tt_attn_supported_dims(int Sq, int Sk, int H, int Hkv, int Dqk, int Dv) { return check_shapes(Sq, Sk, H, Hkv, Dqk, Dv); }

// row_lo (nullable, int32 [B,Sq], non-decreasing along the sequence, needs Sq == Sk): see AttnArgs.
int tt_attn_fwd_range(const void* q, const void* k, const void* v, void* o, float* lse, const int* row_lo, int B, int Sq,
                      int Sk, int H, int Hkv, int Dh, int causal, float scale, cudaStream_t st);

int tt_attn_fwd_sinks(const void* q, const void* k, const void* v, void* o, float* lse, const int* row_lo,
                      const float* sinks, int B, int Sq, int Sk, int H, int Hkv, int Dh, int causal, float scale,
                      cudaStream_t st);

int tt_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int Sq, int Sk, int H, int Hkv,
                int Dh, int causal, float scale, cudaStream_t st) {
  return tt_attn_fwd_range(q, k, v, o, lse, nullptr, B, Sq, Sk, H, Hkv, Dh, causal, scale, st);
}

int tt_attn_fwd_range(const void* q, const void* k, const void* v, void* o, float* lse, const int* row_lo, int B, int Sq,
                      int Sk, int H, int Hkv, int Dh, int causal, float scale, cudaStream_t st) {
  return tt_attn_fwd_sinks(q, k, v, o, lse, row_lo, nullptr, B, Sq, Sk, H, Hkv, Dh, causal, scale, st);
}

// sinks (nullable, fp32 [H]): per-head logit added to the softmax denominator; lse includes it.
// General form: separate head dimensions for queries / keys (Dqk) and values (Dv); see dims_ok for the supported pairs.
int tt_attn_fwd_dims(const void* q, const void* k, const void* v, void* o, float* lse, const int* row_lo,
                     const float* sinks, int B, int Sq, int Sk, int H, int Hkv, int Dqk, int Dv, int causal, float scale,
                     cudaStream_t st) {
  int rc = check_shapes(Sq, Sk, H, Hkv, Dqk, Dv);
  if (rc) return rc;
  if (row_lo && Sq != Sk) return -13;
  set_attrs();
  CUtensorMap tq, tk, tv;
  if ((rc = make_map(&tq, q, static_cast<long long>(B) * Sq, H, 128, Dqk))) return rc;
  if ((rc = make_map(&tk, k, static_cast<long long>(B) * Sk, Hkv, 64, Dqk))) return rc;
  if ((rc = make_map(&tv, v, static_cast<long long>(B) * Sk, Hkv, 64, Dv))) return rc;
  AttnArgs p{B, Sq, Sk, H, Hkv, causal, scale, o, nullptr, lse, nullptr, row_lo, nullptr, sinks};
  dim3 grid(Sq / 128, H, B);
  if (Dqk == 128) attn_fwd_kernel<128, 128><<<grid, 192, FwdLayout<128, 128>::SMEM, st>>>(tq, tk, tv, p);
  else if (Dqk == 64) attn_fwd_kernel<64, 64><<<grid, 192, FwdLayout<64, 64>::SMEM, st>>>(tq, tk, tv, p);
  else attn_fwd_kernel<192, 128><<<grid, 192, FwdLayout<192, 128>::SMEM, st>>>(tq, tk, tv, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

int tt_attn_fwd_sinks(const void* q, const void* k, const void* v, void* o, float* lse, const int* row_lo,
                      const float* sinks, int B, int Sq, int Sk, int H, int Hkv, int Dh, int causal, float scale,
                      cudaStream_t st) {
  return tt_attn_fwd_dims(q, k, v, o, lse, row_lo, sinks, B, Sq, Sk, H, Hkv, Dh, Dh, causal, scale, st);
}

// delta is scratch [B,H,Sq] fp32 written by the first launch and read by the other two.
int tt_attn_bwd_range(const void* q, const void* k, const void* v, const void* o, const void* dout, const float* lse,
                      float* delta, void* dq, void* dk, void* dv, const int* row_lo, const int* col_hi, int B, int Sq,
                      int Sk, int H, int Hkv, int Dh, int causal, float scale, cudaStream_t st);

int tt_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout, const float* lse,
                float* delta, void* dq, void* dk, void* dv, int B, int Sq, int Sk, int H, int Hkv, int Dh, int causal,
                float scale, cudaStream_t st) {
  return tt_attn_bwd_range(q, k, v, o, dout, lse, delta, dq, dk, dv, nullptr, nullptr, B, Sq, Sk, H, Hkv, Dh, causal,
                           scale, st);
}

// row_lo / col_hi: both null or both given (see AttnArgs).
int tt_attn_bwd_range(const void* q, const void* k, const void* v, const void* o, const void* dout, const float* lse,
                      float* delta, void* dq, void* dk, void* dv, const int* row_lo, const int* col_hi, int B, int Sq,
                      int Sk, int H, int Hkv, int Dh, int causal, float scale, cudaStream_t st) {
  int rc = check_shapes(Sq, Sk, H, Hkv, Dh);
  if (rc) return rc;
  if ((row_lo != nullptr) != (col_hi != nullptr)) return -14;
  if (row_lo && Sq != Sk) return -13;
  set_attrs();
  const long long rows = static_cast<long long>(B) * Sq * H;
  attn_delta_kernel<<<static_cast<unsigned>((rows + 15) / 16), 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(o), static_cast<const __nv_bfloat16*>(dout), delta, B, Sq, H);
  CUtensorMap tq128, tdo128, tk64, tv64, tq64, tdo64, tk128, tv128;
  if ((rc = make_map(&tq128, q, static_cast<long long>(B) * Sq, H, 128))) return rc;
  if ((rc = make_map(&tdo128, dout, static_cast<long long>(B) * Sq, H, 128))) return rc;
  if ((rc = make_map(&tk64, k, static_cast<long long>(B) * Sk, Hkv, 64))) return rc;
  if ((rc = make_map(&tv64, v, static_cast<long long>(B) * Sk, Hkv, 64))) return rc;
  if ((rc = make_map(&tq64, q, static_cast<long long>(B) * Sq, H, 64))) return rc;
  if ((rc = make_map(&tdo64, dout, static_cast<long long>(B) * Sq, H, 64))) return rc;
  if ((rc = make_map(&tk128, k, static_cast<long long>(B) * Sk, Hkv, 128))) return rc;
  if ((rc = make_map(&tv128, v, static_cast<long long>(B) * Sk, Hkv, 128))) return rc;
  AttnArgs pq{B, Sq, Sk, H, Hkv, causal, scale, dq, nullptr, const_cast<float*>(lse), delta, row_lo, col_hi, nullptr};
  attn_bwd_dq_kernel<128, 128><<<dim3(Sq / 128, H, B), 320, DqLayout<128, 128>::SMEM, st>>>(tq128, tdo128, tk64, tv64, pq);
  AttnArgs pk{B, Sq, Sk, H, Hkv, causal, scale, dk, dv, const_cast<float*>(lse), delta, row_lo, col_hi, nullptr};
  attn_bwd_dkv_kernel<<<dim3(Sk / 128, Hkv, B), 320, DKV_SMEM, st>>>(tq64, tdo64, tk128, tv128, pk);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// Debug / measurement knob: bits 0-1 = how the fused backward adds dQ (see FusedExtra::dq_mode; 2 drops dQ), bit 2 = feed
// P^T / dS^T to the dV / dK MMAs through tensor memory.
void tt_attn_set_dq_mode(int mode) { g_dq_mode = mode & 3; g_a_tmem = (mode >> 2) & 1; }

// Fused backward (see attn_bwd_fused_kernel). scratch: fp32 [2 * B*H*Sq] (written here); dq_acc: fp32 [B,Sq,H,D] that the
// caller has zeroed (on the same stream). dQ's low bits are not reproducible from run to run.
int tt_attn_bwd_fused(const void* q, const void* k, const void* v, const void* o, const void* dout, const float* lse,
                      float* scratch, float* dq_acc, void* dq, void* dk, void* dv, const int* row_lo, const int* col_hi,
                      int B, int Sq, int Sk, int H, int Hkv, int Dh, int causal, float scale, cudaStream_t st) {
  int rc = check_shapes(Sq, Sk, H, Hkv, Dh);
  if (rc) return rc;
  if ((row_lo != nullptr) != (col_hi != nullptr)) return -14;
  if (row_lo && Sq != Sk) return -13;
  set_attrs();
  const long long rows = static_cast<long long>(B) * Sq * H;
  float* lse2 = scratch;
  float* delta_s = scratch + rows;
  attn_prep_kernel<128><<<static_cast<unsigned>((rows + 15) / 16), 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(o), static_cast<const __nv_bfloat16*>(dout), lse, lse2, delta_s, nullptr, scale, B, Sq, H);
  CUtensorMap tq64, tdo64, tk128, tv128;
  if ((rc = make_map(&tq64, q, static_cast<long long>(B) * Sq, H, 64))) return rc;
  if ((rc = make_map(&tdo64, dout, static_cast<long long>(B) * Sq, H, 64))) return rc;
  if ((rc = make_map(&tk128, k, static_cast<long long>(B) * Sk, Hkv, 128))) return rc;
  if ((rc = make_map(&tv128, v, static_cast<long long>(B) * Sk, Hkv, 128))) return rc;
  AttnArgs pk{B, Sq, Sk, H, Hkv, causal, scale, dk, dv, const_cast<float*>(lse), nullptr, row_lo, col_hi, nullptr};
  FusedExtra x{lse2, delta_s, dq_acc, g_dq_mode, g_a_tmem};
  // the fp32 dQ accumulator as a 3-D tensor (d, head, row); box = (128, 1, 32) fp32 rows, no swizzle
  CUtensorMap tdq;
  {
    tt::EncodeTiledFn fn = tt::encode_tiled_fn();
    if (!fn) return -1;
    cuuint64_t dims[3] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(H), static_cast<cuuint64_t>(B) * Sq};
    cuuint64_t strides[2] = {static_cast<cuuint64_t>(D) * 4, static_cast<cuuint64_t>(H) * D * 4};
    cuuint32_t box[3] = {static_cast<cuuint32_t>(D), 1, 32};
    cuuint32_t es[3] = {1, 1, 1};
    CUresult r = fn(&tdq, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, dq_acc, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return -static_cast<int>(r) - 1000;
  }
  attn_bwd_fused_kernel<128, 128, true><<<dim3(Hkv, Sk / 128, B), FUSED_THREADS, FusedLayout<128, 128, true>::SMEM, st>>>(
      tq64, tdo64, tk128, tv128, tdq, pk, x);
  const long long n8 = rows * D / 8;
  long long cblocks = (n8 + 255) / 256;
  if (cblocks > 148 * 16) cblocks = 148 * 16;
  attn_dq_convert_kernel<<<static_cast<unsigned>(cblocks), 256, 0, st>>>(
      dq_acc, static_cast<__nv_bfloat16*>(dq), n8);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// Backward for the head dimensions other than 128 (see dims_ok): the key-tile kernel forms dK and dV (no dQ, no atomics),
// the query-tile kernel forms dQ. scratch: fp32 [3 * B*H*Sq] (written here). Deterministic.
int tt_attn_bwd_dims(const void* q, const void* k, const void* v, const void* o, const void* dout, const float* lse,
                     float* scratch, void* dq, void* dk, void* dv, const int* row_lo, const int* col_hi, int B, int Sq, int Sk,
                     int H, int Hkv, int Dqk, int Dv, int causal, float scale, cudaStream_t st) {
  int rc = check_shapes(Sq, Sk, H, Hkv, Dqk, Dv);
  if (rc) return rc;
  if (Dqk == 128) return -15;     // use tt_attn_bwd_fused / tt_attn_bwd_range
  if ((row_lo != nullptr) != (col_hi != nullptr)) return -14;
  if (row_lo && Sq != Sk) return -13;
  set_attrs();
  const long long rows = static_cast<long long>(B) * Sq * H;
  float* lse2 = scratch;
  float* delta_s = scratch + rows;
  float* delta = scratch + 2 * rows;
  if (Dv == 128) {
    attn_prep_kernel<128><<<static_cast<unsigned>((rows + 15) / 16), 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(o), static_cast<const __nv_bfloat16*>(dout), lse, lse2, delta_s, delta, scale, B, Sq, H);
  } else {
    attn_prep_kernel<64><<<static_cast<unsigned>((rows + 31) / 32), 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(o), static_cast<const __nv_bfloat16*>(dout), lse, lse2, delta_s, delta, scale, B, Sq, H);
  }
  CUtensorMap tq64, tdo64, tk128, tv128, tq128, tdo128, tk64, tv64;
  if ((rc = make_map(&tq64, q, static_cast<long long>(B) * Sq, H, 64, Dqk))) return rc;
  if ((rc = make_map(&tdo64, dout, static_cast<long long>(B) * Sq, H, 64, Dv))) return rc;
  if ((rc = make_map(&tk128, k, static_cast<long long>(B) * Sk, Hkv, 128, Dqk))) return rc;
  if ((rc = make_map(&tv128, v, static_cast<long long>(B) * Sk, Hkv, 128, Dv))) return rc;
  if ((rc = make_map(&tq128, q, static_cast<long long>(B) * Sq, H, 128, Dqk))) return rc;
  if ((rc = make_map(&tdo128, dout, static_cast<long long>(B) * Sq, H, 128, Dv))) return rc;
  if ((rc = make_map(&tk64, k, static_cast<long long>(B) * Sk, Hkv, 64, Dqk))) return rc;
  if ((rc = make_map(&tv64, v, static_cast<long long>(B) * Sk, Hkv, 64, Dv))) return rc;
  AttnArgs pk{B, Sq, Sk, H, Hkv, causal, scale, dk, dv, const_cast<float*>(lse), nullptr, row_lo, col_hi, nullptr};
  FusedExtra x{lse2, delta_s, nullptr, 2, 1};
  AttnArgs pq{B, Sq, Sk, H, Hkv, causal, scale, dq, nullptr, const_cast<float*>(lse), delta, row_lo, col_hi, nullptr};
  const dim3 gk(Hkv, Sk / 128, B), gq(Sq / 128, H, B);
  if (Dqk == 64) {
    attn_bwd_fused_kernel<64, 64, false><<<gk, FUSED_THREADS, FusedLayout<64, 64, false>::SMEM, st>>>(tq64, tdo64, tk128, tv128, tq64, pk, x);
    attn_bwd_dq_kernel<64, 64><<<gq, 320, DqLayout<64, 64>::SMEM, st>>>(tq128, tdo128, tk64, tv64, pq);
  } else {
    attn_bwd_fused_kernel<192, 128, false><<<gk, FUSED_THREADS, FusedLayout<192, 128, false>::SMEM, st>>>(tq64, tdo64, tk128, tv128, tq64, pk, x);
    attn_bwd_dq_kernel<192, 128><<<gq, 320, DqLayout<192, 128>::SMEM, st>>>(tq128, tdo128, tk64, tv64, pq);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

#ifdef TT_ATTN_TRACE
int tt_attn_trace(long long* out) { return cudaMemcpyFromSymbol(out, g_attn_trace, sizeof(long long) * 8 * 16) == cudaSuccess ? 0 : -1; }
#endif

int tt_attn_error() {
  int v = 0, zero = 0;
  cudaMemcpyFromSymbol(&v, g_attn_error, sizeof(int));
  if (v) cudaMemcpyToSymbol(g_attn_error, &zero, sizeof(int));
  return v;
}

}  // extern "C"
