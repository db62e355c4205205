// Dynamic float8 quantisation of bf16 matrices for the 8-bit GEMMs (e4m3 / e5m2 data, fp32 scales).
//
// A GEMM operand must be contiguous along the contraction dimension and carries one scale per tensor or one per
// non-contraction index. The operand is either the matrix as stored (contraction along the rows' contiguous dimension:
// "rows" kernels) or its transpose (contraction down the columns: "cols" kernels, which write the quantised transpose so
// that the result is again contiguous along the contraction). Every form reads the source twice (amax, then convert; the
// second read of a row-quantised matrix hits L1/L2) and writes one byte per element, instead of the dozen full-size
// fp32 temporaries of the elementwise definition.
//
// Scales: x ~= q * scale. Per tensor: scale = amax / fmax. Per row / column: scale = 2^ceil(log2(amax / fmax)), taken
// exactly from the float's exponent and mantissa bits. amax is clamped from below at 1e-12. Conversion divides by the
// scale, clamps to +-fmax and rounds to nearest even.

#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace {

constexpr float E4M3_MAX = 448.f;
constexpr float E5M2_MAX = 57344.f;
constexpr float AMAX_FLOOR = 1e-12f;

__device__ __forceinline__ float scale_from_amax(float amax, float fmax, int pow2) {
  const float v = fmaxf(amax, AMAX_FLOOR) / fmax;
  if (!pow2) return v;
  // 2^ceil(log2 v) for a positive normal float: bump the exponent when any mantissa bit is set
  uint32_t b = __float_as_uint(v);
  if (b & 0x007fffffu) b = (b & 0xff800000u) + 0x00800000u;
  return __uint_as_float(b);
}

template <bool E5M2>
__device__ __forceinline__ uint8_t to_fp8(float x, float scale, float fmax) {
  const float y = fminf(fmaxf(__fdiv_rn(x, scale), -fmax), fmax);
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(y, __NV_SATFINITE, E5M2 ? __NV_E5M2 : __NV_E4M3));
}

__device__ __forceinline__ float block_max(float v, float* s_red) {
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  const int w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  if ((threadIdx.x & 31) == 0) s_red[w] = v;
  __syncthreads();
  v = (threadIdx.x & 31) < nw ? s_red[threadIdx.x & 31] : 0.f;
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();
  return v;
}

// ------------------------------------------------------------------------------------------- rows
// One CTA per row: amax over the row, scale, convert. K % 8 == 0, ld % 8 == 0.
template <bool E5M2>
__global__ void __launch_bounds__(256)
quant_rows_kernel(const __nv_bfloat16* __restrict__ x, long long ld, int K, uint8_t* __restrict__ q,
                  float* __restrict__ scale_out, int pow2) {
  __shared__ float s_red[8];
  const long long row = blockIdx.x;
  const uint4* src = reinterpret_cast<const uint4*>(x + row * ld);
  const int n8 = K / 8;
  float mx = 0.f;
  for (int i = threadIdx.x; i < n8; i += blockDim.x) {
    const uint4 v = src[i];
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = __bfloat1622float2(h[e]);
      mx = fmaxf(mx, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
  }
  mx = block_max(mx, s_red);
  const float fmax = E5M2 ? E5M2_MAX : E4M3_MAX;
  const float scale = scale_from_amax(mx, fmax, pow2);
  if (threadIdx.x == 0) scale_out[row] = scale;
  uint2* dst = reinterpret_cast<uint2*>(q + row * static_cast<long long>(K));
  for (int i = threadIdx.x; i < n8; i += blockDim.x) {
    const uint4 v = src[i];
    const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(&v);
    uint8_t o[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = to_fp8<E5M2>(__bfloat162float(h[e]), scale, fmax);
    dst[i] = *reinterpret_cast<const uint2*>(o);
  }
}

// ------------------------------------------------------------------------------------------- amax of columns / of all
// Tile of 256 rows x 64 columns per CTA; column maxima merged with atomicMax on the float bits (values are >= 0).
__global__ void __launch_bounds__(256)
amax_cols_kernel(const __nv_bfloat16* __restrict__ x, long long ld, int M, int N, float* __restrict__ amax, int whole) {
  __shared__ float s_max[32][65];
  const int c8 = threadIdx.x & 7, rl = threadIdx.x >> 3;     // 8 column chunks of 8, 32 row lanes
  const int col = blockIdx.x * 64 + c8 * 8;
  const int row0 = blockIdx.y * 256;
  float mx[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) mx[e] = 0.f;
  if (col < N) {
    for (int r = row0 + rl; r < min(M, row0 + 256); r += 32) {
      const uint4 v = *reinterpret_cast<const uint4*>(x + r * ld + col);
      const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(&v);
#pragma unroll
      for (int e = 0; e < 8; ++e) mx[e] = fmaxf(mx[e], fabsf(__bfloat162float(h[e])));
    }
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) s_max[rl][c8 * 8 + e] = mx[e];
  __syncthreads();
  if (threadIdx.x < 64) {
    float m = 0.f;
    for (int r = 0; r < 32; ++r) m = fmaxf(m, s_max[r][threadIdx.x]);
    const int c = blockIdx.x * 64 + threadIdx.x;
    if (whole) {
      for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
      if ((threadIdx.x & 31) == 0) atomicMax(reinterpret_cast<int*>(amax), __float_as_int(m));
    } else if (c < N) {
      atomicMax(reinterpret_cast<int*>(amax) + c, __float_as_int(m));
    }
  }
}

__global__ void scale_from_amax_kernel(float* __restrict__ s, int n, float fmax, int pow2) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) s[i] = scale_from_amax(s[i], fmax, pow2);
}

// ------------------------------------------------------------------------------------------- convert with given scales
// Straight: q[m, k] = x[m, k] / scale[scale_per_row ? m : 0]; 8 elements per thread.
template <bool E5M2>
__global__ void __launch_bounds__(256)
cast_kernel(const __nv_bfloat16* __restrict__ x, long long ld, int M, int K, uint8_t* __restrict__ q,
            const float* __restrict__ scale, int scale_per_row) {
  const float fmax = E5M2 ? E5M2_MAX : E4M3_MAX;
  const int n8 = K / 8;
  const long long total = static_cast<long long>(M) * n8;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / n8;
    const int c = static_cast<int>(i - r * n8);
    const float sc = __ldg(scale + (scale_per_row ? r : 0));
    const uint4 v = *reinterpret_cast<const uint4*>(x + r * ld + c * 8);
    const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(&v);
    uint8_t o[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = to_fp8<E5M2>(__bfloat162float(h[e]), sc, fmax);
    *reinterpret_cast<uint2*>(q + r * static_cast<long long>(K) + c * 8) = *reinterpret_cast<const uint2*>(o);
  }
}

// Transposed: qT[n, m] = x[m, n] / scale[scale_per_col ? n : 0]. Tile of 128 rows (m) x 64 columns (n) through shared
// memory; every output row segment is 128 contiguous bytes. M % 16 == 0 (16-byte stores), N % 8 == 0.
template <bool E5M2>
__global__ void __launch_bounds__(256)
cast_transpose_kernel(const __nv_bfloat16* __restrict__ x, long long ld, int M, int N, uint8_t* __restrict__ qT,
                      const float* __restrict__ scale, int scale_per_col) {
  __shared__ uint8_t s_t[64][128 + 16];
  const float fmax = E5M2 ? E5M2_MAX : E4M3_MAX;
  const int n0 = blockIdx.x * 64, m0 = blockIdx.y * 128;
  const int c8 = threadIdx.x & 7, rl = threadIdx.x >> 3;
  const int col = n0 + c8 * 8;
  float sc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) sc[e] = (col + e < N) ? __ldg(scale + (scale_per_col ? col + e : 0)) : 1.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = rl + 32 * i;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (m0 + r < M && col < N) v = *reinterpret_cast<const uint4*>(x + (m0 + r) * ld + col);
    const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(&v);
#pragma unroll
    for (int e = 0; e < 8; ++e) s_t[c8 * 8 + e][r] = to_fp8<E5M2>(__bfloat162float(h[e]), sc[e], fmax);
  }
  __syncthreads();
  // 64 output rows x 128 bytes = 512 segments of 16 bytes, 2 per thread
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int seg = threadIdx.x + 256 * i;
    const int n = seg >> 3, part = seg & 7;
    if (n0 + n < N && m0 + part * 16 < M)
      *reinterpret_cast<uint4*>(qT + (n0 + n) * static_cast<long long>(M) + m0 + part * 16) =
          *reinterpret_cast<const uint4*>(&s_t[n][part * 16]);
  }
}

// ------------------------------------------------------------------------------------------- MXFP8
// e4m3 data with one E8M0 scale (biased exponent byte) per 32 consecutive elements of the contraction dimension.
// RCEIL: exponent = ceil(log2(amax / 448)), clamped to [-127, 127], so no element saturates.
__device__ __forceinline__ int mx_exponent(float amax) {
  const float v = fmaxf(amax, 448.f * 1.17549435e-38f * 0.5f) / 448.f;   // floor 2^-127 * 448, as the definition
  const uint32_t b = __float_as_uint(v);
  int e = static_cast<int>((b >> 23) & 0xff) - 127;
  if ((b >> 23) == 0) e = (b == 0x00400000u) ? -127 : -126;   // subnormal quotient: exactly 2^-127, or just above it
  else if (b & 0x007fffffu) e += 1;
  return max(-127, min(127, e));
}

// Where the scale of (row r, K block b) lives in the layout the block-scaled MMA wants (see gemm_mx.cu): one 512-byte
// chunk per 128 rows and per 4 K blocks; inside it row r, block j sits at byte (r % 32) * 16 + ((r / 32) % 4) * 4 + j.
// Writing this layout here saves the separate re-layout launch per operand.
__device__ __forceinline__ long long mx_swizzled_index(long long r, int b, int kb4) {
  return ((r >> 7) * kb4 + (b >> 2)) * 512 + (r & 31) * 16 + ((r >> 5) & 3) * 4 + (b & 3);
}

// Rows: one thread per 32-element block (64 bytes in, 32 bytes + 1 scale byte out). K % 32 == 0.
__global__ void __launch_bounds__(256)
mx_quant_rows_kernel(const __nv_bfloat16* __restrict__ x, long long ld, int M, int K, uint8_t* __restrict__ q,
                     uint8_t* __restrict__ scales, int kb4) {
  const int kb = K / 32;
  const long long total = static_cast<long long>(M) * kb;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / kb;
    const int b = static_cast<int>(i - r * kb);
    const uint4* src = reinterpret_cast<const uint4*>(x + r * ld + b * 32);
    uint4 v[4];
    float mx = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      v[j] = src[j];
      const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(&v[j]);
#pragma unroll
      for (int e = 0; e < 8; ++e) mx = fmaxf(mx, fabsf(__bfloat162float(h[e])));
    }
    const int ex = mx_exponent(mx);
    const float inv = exp2f(static_cast<float>(-ex));
    uint8_t o[32];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(&v[j]);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float y = fminf(fmaxf(__bfloat162float(h[e]) * inv, -E4M3_MAX), E4M3_MAX);
        o[8 * j + e] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(y, __NV_SATFINITE, __NV_E4M3));
      }
    }
    uint4* dst = reinterpret_cast<uint4*>(q + r * static_cast<long long>(K) + b * 32);
    dst[0] = *reinterpret_cast<const uint4*>(o);
    dst[1] = *reinterpret_cast<const uint4*>(o + 16);
    scales[kb4 ? mx_swizzled_index(r, b, kb4) : r * kb + b] = static_cast<uint8_t>(ex + 127);
  }
}

// Columns: qT [N, M] = transpose of x [M, N], blocks of 32 along M (the contraction of the transposed operand);
// scales [N, M/32]. Tile of 128 rows (m) x 64 columns (n): per column four 32-row blocks. M % 32 == 0, N % 8 == 0.
__global__ void __launch_bounds__(256)
mx_quant_cols_kernel(const __nv_bfloat16* __restrict__ x, long long ld, int M, int N, uint8_t* __restrict__ qT,
                     uint8_t* __restrict__ scales, int kb4) {
  __shared__ __nv_bfloat16 s_x[128][64 + 8];
  __shared__ uint8_t s_t[64][128 + 16];
  const int n0 = blockIdx.x * 64, m0 = blockIdx.y * 128;
  const int c8 = threadIdx.x & 7, rl = threadIdx.x >> 3;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = rl + 32 * i;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (m0 + r < M && n0 + c8 * 8 < N) v = *reinterpret_cast<const uint4*>(x + (m0 + r) * ld + n0 + c8 * 8);
    *reinterpret_cast<uint4*>(&s_x[r][c8 * 8]) = v;
  }
  __syncthreads();
  // thread -> (column n = tid % 64, 32-row block blk = tid / 64)
  const int n = threadIdx.x & 63, blk = threadIdx.x >> 6;
  float mx = 0.f;
#pragma unroll 8
  for (int r = 0; r < 32; ++r) mx = fmaxf(mx, fabsf(__bfloat162float(s_x[blk * 32 + r][n])));
  const int ex = mx_exponent(mx);
  const float inv = exp2f(static_cast<float>(-ex));
#pragma unroll 8
  for (int r = 0; r < 32; ++r) {
    const float y = fminf(fmaxf(__bfloat162float(s_x[blk * 32 + r][n]) * inv, -E4M3_MAX), E4M3_MAX);
    s_t[n][blk * 32 + r] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(y, __NV_SATFINITE, __NV_E4M3));
  }
  if (n0 + n < N && m0 + blk * 32 < M)
    scales[kb4 ? mx_swizzled_index(n0 + n, m0 / 32 + blk, kb4)
               : (n0 + n) * static_cast<long long>(M / 32) + (m0 / 32 + blk)] = static_cast<uint8_t>(ex + 127);
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int seg = threadIdx.x + 256 * i;
    const int nn = seg >> 3, part = seg & 7;
    if (n0 + nn < N && m0 + part * 16 < M)
      *reinterpret_cast<uint4*>(qT + (n0 + nn) * static_cast<long long>(M) + m0 + part * 16) =
          *reinterpret_cast<const uint4*>(&s_t[nn][part * 16]);
  }
}

int grid_for(long long work, int block) {
  long long g = (work + block - 1) / block;
  if (g > 148 * 16) g = 148 * 16;
  return static_cast<int>(g < 1 ? 1 : g);
}

}  // namespace

extern "C" {

// q [M,K] = x [M,K] (bf16, row stride ld) with one scale per row (scale_out [M]); contraction along K.
int tt_fp8_quant_rows(const void* x, long long ld, int M, int K, void* q, float* scale_out, int e5m2, int pow2,
                      cudaStream_t st) {
  if (M <= 0 || K <= 0) return 0;
  if (K % 8 || ld % 8) return -2;
  const auto* xp = static_cast<const __nv_bfloat16*>(x);
  auto* qp = static_cast<uint8_t*>(q);
  if (e5m2) quant_rows_kernel<true><<<M, 256, 0, st>>>(xp, ld, K, qp, scale_out, pow2);
  else      quant_rows_kernel<false><<<M, 256, 0, st>>>(xp, ld, K, qp, scale_out, pow2);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// qT [N,M] = transpose of x [M,N] (bf16, row stride ld) with one scale per column of x (scale_out [N]); contraction
// along M.
int tt_fp8_quant_cols(const void* x, long long ld, int M, int N, void* qT, float* scale_out, int e5m2, int pow2,
                      cudaStream_t st) {
  if (M <= 0 || N <= 0) return 0;
  if (N % 8 || ld % 8 || M % 16) return -2;
  const auto* xp = static_cast<const __nv_bfloat16*>(x);
  auto* qp = static_cast<uint8_t*>(qT);
  cudaMemsetAsync(scale_out, 0, sizeof(float) * N, st);
  dim3 ga((N + 63) / 64, (M + 255) / 256);
  amax_cols_kernel<<<ga, 256, 0, st>>>(xp, ld, M, N, scale_out, 0);
  scale_from_amax_kernel<<<(N + 255) / 256, 256, 0, st>>>(scale_out, N, e5m2 ? E5M2_MAX : E4M3_MAX, pow2);
  dim3 gc((N + 63) / 64, (M + 127) / 128);
  if (e5m2) cast_transpose_kernel<true><<<gc, 256, 0, st>>>(xp, ld, M, N, qp, scale_out, 1);
  else      cast_transpose_kernel<false><<<gc, 256, 0, st>>>(xp, ld, M, N, qp, scale_out, 1);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// One scale for the whole matrix (scale_out [1]); `transpose` selects q [M,N] or qT [N,M].
int tt_fp8_quant_tensor(const void* x, long long ld, int M, int N, void* q, float* scale_out, int transpose, int e5m2,
                        cudaStream_t st) {
  if (M <= 0 || N <= 0) return 0;
  if (N % 8 || ld % 8 || (transpose && M % 16)) return -2;
  const auto* xp = static_cast<const __nv_bfloat16*>(x);
  auto* qp = static_cast<uint8_t*>(q);
  cudaMemsetAsync(scale_out, 0, sizeof(float), st);
  dim3 ga((N + 63) / 64, (M + 255) / 256);
  amax_cols_kernel<<<ga, 256, 0, st>>>(xp, ld, M, N, scale_out, 1);
  scale_from_amax_kernel<<<1, 32, 0, st>>>(scale_out, 1, e5m2 ? E5M2_MAX : E4M3_MAX, 0);
  if (transpose) {
    dim3 gc((N + 63) / 64, (M + 127) / 128);
    if (e5m2) cast_transpose_kernel<true><<<gc, 256, 0, st>>>(xp, ld, M, N, qp, scale_out, 0);
    else      cast_transpose_kernel<false><<<gc, 256, 0, st>>>(xp, ld, M, N, qp, scale_out, 0);
  } else {
    const int g = grid_for(static_cast<long long>(M) * (N / 8), 256);
    if (e5m2) cast_kernel<true><<<g, 256, 0, st>>>(xp, ld, M, N, qp, scale_out, 0);
    else      cast_kernel<false><<<g, 256, 0, st>>>(xp, ld, M, N, qp, scale_out, 0);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// MXFP8 along the rows' contiguous dimension: q [M,K] e4m3, scales [M, K/32] E8M0 bytes.
int tt_mxfp8_quant_rows(const void* x, long long ld, int M, int K, void* q, void* scales, cudaStream_t st) {
  if (M <= 0 || K <= 0) return 0;
  if (K % 32 || ld % 8) return -2;
  mx_quant_rows_kernel<<<grid_for(static_cast<long long>(M) * (K / 32), 256), 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(x), ld, M, K, static_cast<uint8_t*>(q), static_cast<uint8_t*>(scales), 0);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// Same, with the scales written straight into the block-scaled MMA's layout (buffer of tt_mx_scales_bytes(M, 256, K)
// bytes; when M % 128 or (K / 32) % 4 is not zero the caller fills it with 127 = 2^0 first).
int tt_mxfp8_quant_rows_swz(const void* x, long long ld, int M, int K, void* q, void* scales, cudaStream_t st) {
  if (M <= 0 || K <= 0) return 0;
  if (K % 32 || ld % 8) return -2;
  mx_quant_rows_kernel<<<grid_for(static_cast<long long>(M) * (K / 32), 256), 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(x), ld, M, K, static_cast<uint8_t*>(q), static_cast<uint8_t*>(scales), (K + 127) / 128);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// MXFP8 of the transposed operand: qT [N,M] e4m3 and scales [N, M/32] from x [M,N] (blocks run down the columns of x).
int tt_mxfp8_quant_cols(const void* x, long long ld, int M, int N, void* qT, void* scales, cudaStream_t st) {
  if (M <= 0 || N <= 0) return 0;
  if (M % 32 || N % 8 || ld % 8) return -2;
  dim3 g((N + 63) / 64, (M + 127) / 128);
  mx_quant_cols_kernel<<<g, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), ld, M, N, static_cast<uint8_t*>(qT),
                                          static_cast<uint8_t*>(scales), 0);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// Transposed operand with scales in the MMA's layout: rows of the operand = columns of x (N of them), contraction M.
int tt_mxfp8_quant_cols_swz(const void* x, long long ld, int M, int N, void* qT, void* scales, cudaStream_t st) {
  if (M <= 0 || N <= 0) return 0;
  if (M % 32 || N % 8 || ld % 8) return -2;
  dim3 g((N + 63) / 64, (M + 127) / 128);
  mx_quant_cols_kernel<<<g, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), ld, M, N, static_cast<uint8_t*>(qT),
                                          static_cast<uint8_t*>(scales), (M + 127) / 128);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // extern "C"
