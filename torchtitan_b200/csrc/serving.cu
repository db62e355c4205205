// Generation-side kernels: KV-cache scatter, paged-KV decode attention, token sampler.
//
// Cache layout: [num_blocks, block_size, n_kv_heads, 128] bf16 for keys and for values; block_tables[b, i] is the cache
// block with tokens i*block_size .. (i+1)*block_size-1 of sequence b.
//
// paged decode (one query token per sequence): CTA = (sequence, kv head); all query heads of the group are processed
// together so that every cached K/V row is read once. The context is walked in tiles of 128 tokens: 16 threads share
// a row (16-byte loads, fully used cache lines), 8 rows per pass; scores go through shared memory, the softmax is the
// online (running max / sum) form in fp32, and P.V accumulates in registers (8 dims per thread). The kernel is
// bandwidth-bound by design: it moves ctx * 512 bytes per (sequence, kv head) and does O(1) flops per byte.
// No kernel here waits on another CTA or rank.
//
// Counterpart of the paged attention + sampler that the reference reaches through vLLM
// (torchtitan/experiments/rl/unified/models/attention.py:62-117, actors/generator.py:251-260).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace {

constexpr int HD = 128;          // head dim
constexpr int TT = 128;          // tokens per tile
constexpr float kLog2e = 1.4426950408889634f;

__global__ void kv_write_kernel(__nv_bfloat16* __restrict__ kc, __nv_bfloat16* __restrict__ vc,
                                const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                                const int* __restrict__ slots, long long T, int row_elems) {
  // one 16-byte chunk per thread
  const int chunks = row_elems / 8;
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= T * chunks) return;
  const long long t = i / chunks;
  const int c = static_cast<int>(i % chunks);
  const long long dst = static_cast<long long>(slots[t]) * row_elems + c * 8;
  *reinterpret_cast<uint4*>(kc + dst) = *reinterpret_cast<const uint4*>(k + t * row_elems + c * 8);
  *reinterpret_cast<uint4*>(vc + dst) = *reinterpret_cast<const uint4*>(v + t * row_elems + c * 8);
}

template <int G>
__global__ void __launch_bounds__(128)
paged_decode_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kc,
                    const __nv_bfloat16* __restrict__ vc, const int* __restrict__ block_tables,
                    const int* __restrict__ ctx_lens, __nv_bfloat16* __restrict__ out, float scale, int H, int Hkv,
                    int block_size, int max_blocks) {
  const int b = blockIdx.x, hk = blockIdx.y;
  const int tid = threadIdx.x;
  const int tg = tid >> 4, dl = tid & 15;      // row lane (0..7), 8-dim chunk (0..15)
  const int ctx = ctx_lens[b];
  const int* bt = block_tables + static_cast<long long>(b) * max_blocks;

  __shared__ float s_q[G][HD];
  __shared__ float s_p[G][TT];
  __shared__ float s_red[8][G][HD];            // cross-row-lane reduction of the output
  __shared__ float s_m[G];

  for (int i = tid; i < G * HD; i += 128) {
    const int g = i / HD, d = i % HD;
    s_q[g][d] = __bfloat162float(q[(static_cast<long long>(b) * H + hk * G + g) * HD + d]) * scale * kLog2e;
  }
  float acc[G][8];
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[g][e] = 0.f;
  float m_run[G], l_run[G];
#pragma unroll
  for (int g = 0; g < G; ++g) { m_run[g] = -INFINITY; l_run[g] = 0.f; }
  __syncthreads();

  float qreg[G][8];
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int e = 0; e < 8; ++e) qreg[g][e] = s_q[g][dl * 8 + e];

  for (int t0 = 0; t0 < ctx; t0 += TT) {
    const int nt = min(TT, ctx - t0);
    // ---- scores: 8 rows per pass, 16 threads per row
    for (int r = tg; r < TT; r += 8) {
      float part[G];
#pragma unroll
      for (int g = 0; g < G; ++g) part[g] = 0.f;
      if (r < nt) {
        const int t = t0 + r;
        const long long row = (static_cast<long long>(bt[t / block_size]) * block_size + t % block_size) * Hkv + hk;
        const uint4 kk = *reinterpret_cast<const uint4*>(kc + row * HD + dl * 8);
        const __nv_bfloat162* kh = reinterpret_cast<const __nv_bfloat162*>(&kk);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(kh[e]);
#pragma unroll
          for (int g = 0; g < G; ++g) part[g] += qreg[g][2 * e] * f.x + qreg[g][2 * e + 1] * f.y;
        }
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float v = part[g];
        v += __shfl_xor_sync(0xffffffffu, v, 1);
        v += __shfl_xor_sync(0xffffffffu, v, 2);
        v += __shfl_xor_sync(0xffffffffu, v, 4);
        v += __shfl_xor_sync(0xffffffffu, v, 8);
        if (dl == 0) s_p[g][r] = (r < nt) ? v : -INFINITY;
      }
    }
    __syncthreads();
    // ---- tile maximum / rescale factors (warp g handles head g, G <= 4 warps... use threads 0..G*32)
    for (int g = tid >> 5; g < G; g += 4) {
      const int lane = tid & 31;
      float mx = -INFINITY;
      for (int r = lane; r < TT; r += 32) mx = fmaxf(mx, s_p[g][r]);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      if (lane == 0) s_m[g] = mx;
    }
    __syncthreads();
    float sum_part[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float m_new = fmaxf(m_run[g], s_m[g]);
      const float f = (m_run[g] == -INFINITY) ? 0.f : exp2f(m_run[g] - m_new);
      m_run[g] = m_new;
      l_run[g] *= f;
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[g][e] *= f;
      sum_part[g] = 0.f;
    }
    // probabilities (each thread converts one column per head; all threads need them from smem afterwards)
    {
      const int r = tid;  // TT == blockDim
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float pr = (r < nt) ? exp2f(s_p[g][r] - m_run[g]) : 0.f;
        s_p[g][r] = pr;
      }
    }
    __syncthreads();
    // ---- P.V: 8 rows per pass, thread owns 8 dims
    for (int r = tg; r < nt; r += 8) {
      const int t = t0 + r;
      const long long row = (static_cast<long long>(bt[t / block_size]) * block_size + t % block_size) * Hkv + hk;
      const uint4 vv = *reinterpret_cast<const uint4*>(vc + row * HD + dl * 8);
      const __nv_bfloat162* vh = reinterpret_cast<const __nv_bfloat162*>(&vv);
      float vf[8];
#pragma unroll
      for (int e = 0; e < 4; ++e) { const float2 f = __bfloat1622float2(vh[e]); vf[2 * e] = f.x; vf[2 * e + 1] = f.y; }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float pr = s_p[g][r];
        sum_part[g] += pr;
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[g][e] += pr * vf[e];
      }
    }
    // every thread of a row lane saw the same rows: the row-lane partial sums are combined at the end
#pragma unroll
    for (int g = 0; g < G; ++g) l_run[g] += sum_part[g];
    __syncthreads();
  }

  // ---- combine the 8 row lanes
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int e = 0; e < 8; ++e) s_red[tg][g][dl * 8 + e] = acc[g][e];
  // l: each row lane holds the sum over its own rows
  __shared__ float s_l[8][G];
  if (dl == 0) {
#pragma unroll
    for (int g = 0; g < G; ++g) s_l[tg][g] = l_run[g];
  }
  __syncthreads();
  for (int i = tid; i < G * HD; i += 128) {
    const int g = i / HD, d = i % HD;
    float o = 0.f, l = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) { o += s_red[j][g][d]; l += s_l[j][g]; }
    out[(static_cast<long long>(b) * H + hk * G + g) * HD + d] = __float2bfloat16(l > 0.f ? o / l : 0.f);
  }
}

// ---------------------------------------------------------------------------------------------- sampler
// One CTA per row. mode 0: greedy (argmax, lowest index on ties); mode 1: multinomial over softmax(logits / T) by inverse
// CDF in *index order* driven by uniforms[row]. The reported log-probability is log_softmax(raw logits)[token] in fp32.
// top_p < 1 restricts the draw to the nucleus: the tokens whose probability is at least that of the last token needed
// to reach a cumulative mass of top_p when taken from the most likely down (ties at that value are all kept). The cut
// is found without sorting: bisection over the order-preserving integer key of the logit for the smallest key k with
// sum of p over {logit > k} < top_p.
__device__ __forceinline__ uint32_t order_key(float v) {
  const uint32_t b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
template <typename T>
__device__ __forceinline__ float ld(const T* p, long long i);
template <>
__device__ __forceinline__ float ld<float>(const float* p, long long i) { return p[i]; }
template <>
__device__ __forceinline__ float ld<__nv_bfloat16>(const __nv_bfloat16* p, long long i) { return __bfloat162float(p[i]); }

template <typename T>
__global__ void __launch_bounds__(1024)
sample_kernel(const T* __restrict__ logits, const float* __restrict__ uniforms, long long* __restrict__ tokens,
              float* __restrict__ logprobs, int V, long long ld_row, float inv_temp, int mode, float top_p) {
  const int row = blockIdx.x, tid = threadIdx.x, nthr = blockDim.x;
  const T* x = logits + row * ld_row;
  __shared__ float s_val[1024];
  __shared__ int s_idx[1024];
  __shared__ float s_sum[1024];

  // contiguous chunk per thread (needed for the index-ordered prefix)
  const int chunk = (V + nthr - 1) / nthr;
  const int lo = tid * chunk, hi = min(V, lo + chunk);

  // pass 1: max (and argmax)
  float mx = -INFINITY;
  int amax = 0x7fffffff;
  for (int i = lo; i < hi; ++i) {
    const float v = ld<T>(x, i);
    if (v > mx) { mx = v; amax = i; }
  }
  s_val[tid] = mx; s_idx[tid] = amax;
  __syncthreads();
  for (int o = nthr >> 1; o > 0; o >>= 1) {
    if (tid < o) {
      const float a = s_val[tid], c = s_val[tid + o];
      const int ia = s_idx[tid], ic = s_idx[tid + o];
      if (c > a || (c == a && ic < ia)) { s_val[tid] = c; s_idx[tid] = ic; }
    }
    __syncthreads();
  }
  const float gmax = s_val[0];
  const int gidx = s_idx[0];
  __syncthreads();

  // pass 2: sum exp(x - max) (raw, for the log-probability) and sum exp((x - max) / T) per chunk
  float raw = 0.f, tem = 0.f;
  for (int i = lo; i < hi; ++i) {
    const float d = ld<T>(x, i) - gmax;
    raw += __expf(d);
    tem += __expf(d * inv_temp);
  }
  s_val[tid] = raw; s_sum[tid] = tem;
  __syncthreads();
  // totals (tree) -- keep the per-thread temperature sums for the prefix search
  __shared__ float s_tot[1024];
  s_tot[tid] = raw;
  __syncthreads();
  for (int o = nthr >> 1; o > 0; o >>= 1) { if (tid < o) s_tot[tid] += s_tot[tid + o]; __syncthreads(); }
  const float raw_total = s_tot[0];
  __syncthreads();

  if (mode == 0) {
    if (tid == 0) { tokens[row] = gidx; logprobs[row] = -__logf(raw_total); }
    return;
  }
  uint32_t kmin = 0;       // keys >= kmin are in the nucleus (0 keeps everything)
  if (top_p < 1.f) {
    // Z of the tempered distribution
    s_tot[tid] = tem;
    __syncthreads();
    for (int o = nthr >> 1; o > 0; o >>= 1) { if (tid < o) s_tot[tid] += s_tot[tid + o]; __syncthreads(); }
    const float mass = top_p * s_tot[0];
    __syncthreads();
    // smallest key k with S(k) = sum_{key(x) > k} e(x) < mass; S is non-increasing in k and S(key(max)) = 0 < mass
    uint32_t lo_k = 0, hi_k = order_key(gmax);
    while (lo_k < hi_k) {
      const uint32_t mid = lo_k + ((hi_k - lo_k) >> 1);
      float part = 0.f;
      for (int i = lo; i < hi; ++i) {
        const float v = ld<T>(x, i);
        if (order_key(v) > mid) part += __expf((v - gmax) * inv_temp);
      }
      s_tot[tid] = part;
      __syncthreads();
      for (int o = nthr >> 1; o > 0; o >>= 1) { if (tid < o) s_tot[tid] += s_tot[tid + o]; __syncthreads(); }
      const bool below = s_tot[0] < mass;
      __syncthreads();
      if (below) hi_k = mid; else lo_k = mid + 1;
    }
    kmin = lo_k;
    // per-thread sums restricted to the nucleus
    tem = 0.f;
    for (int i = lo; i < hi; ++i) {
      const float v = ld<T>(x, i);
      if (order_key(v) >= kmin) tem += __expf((v - gmax) * inv_temp);
    }
    s_sum[tid] = tem;
    __syncthreads();
  }
  // inclusive scan of the per-thread temperature sums (Hillis-Steele over 1024 entries)
  for (int o = 1; o < nthr; o <<= 1) {
    const float add = tid >= o ? s_sum[tid - o] : 0.f;
    __syncthreads();
    s_sum[tid] += add;
    __syncthreads();
  }
  const float total = s_sum[nthr - 1];
  const float target = uniforms[row] * total;
  const float before = tid > 0 ? s_sum[tid - 1] : 0.f;
  // the owner of the crossing: before <= target < s_sum[tid]; the last non-empty thread also takes target >= total
  // (with a nucleus the trailing threads may hold no mass: the last thread whose inclusive sum equals the total)
  const bool last_nonempty = hi > lo && (top_p < 1.f ? (s_sum[tid] >= total && before < total) : (hi == V));
  if (hi > lo && before <= target && (target < s_sum[tid] || last_nonempty)) {
    float run = before;
    int pick = -1, last_kept = -1;
    for (int i = lo; i < hi; ++i) {
      const float v = ld<T>(x, i);
      if (order_key(v) < kmin) continue;
      last_kept = i;
      run += __expf((v - gmax) * inv_temp);
      if (run > target) { pick = i; break; }
    }
    if (pick < 0) pick = last_kept >= 0 ? last_kept : hi - 1;
    tokens[row] = pick;
    logprobs[row] = (ld<T>(x, pick) - gmax) - __logf(raw_total);
  }
}

}  // namespace

extern "C" {

int tt_kv_write(void* kc, void* vc, const void* k, const void* v, const int* slots, long long T, int Hkv, int D,
                cudaStream_t st) {
  if (D != HD) return -10;
  if (T <= 0) return 0;
  const int row = Hkv * D;
  const long long n = T * (row / 8);
  kv_write_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, st>>>(
      static_cast<__nv_bfloat16*>(kc), static_cast<__nv_bfloat16*>(vc), static_cast<const __nv_bfloat16*>(k),
      static_cast<const __nv_bfloat16*>(v), slots, T, row);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

int tt_paged_decode(const void* q, const void* kc, const void* vc, const int* block_tables, const int* ctx_lens, void* out,
                    float scale, int B, int H, int Hkv, int D, int block_size, int max_blocks, cudaStream_t st) {
  if (D != HD) return -10;
  if (Hkv <= 0 || H % Hkv) return -12;
  if (B <= 0) return 0;
  const int G = H / Hkv;
  dim3 grid(B, Hkv);
#define LAUNCH(GG)                                                                                              \
  paged_decode_kernel<GG><<<grid, 128, 0, st>>>(static_cast<const __nv_bfloat16*>(q),                           \
      static_cast<const __nv_bfloat16*>(kc), static_cast<const __nv_bfloat16*>(vc), block_tables, ctx_lens,     \
      static_cast<__nv_bfloat16*>(out), scale, H, Hkv, block_size, max_blocks)
  switch (G) {
    case 1: LAUNCH(1); break;
    case 2: LAUNCH(2); break;
    case 4: LAUNCH(4); break;
    case 8: LAUNCH(8); break;
    default: return -13;
  }
#undef LAUNCH
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// dtype: 0 = fp32 logits, 1 = bf16 logits. temperature <= 0 selects greedy.
int tt_sample_top_p(const void* logits, const float* uniforms, long long* tokens, float* logprobs, int B, int V,
                    long long ld_row, float temperature, float top_p, int dtype, cudaStream_t st);

int tt_sample(const void* logits, const float* uniforms, long long* tokens, float* logprobs, int B, int V, long long ld_row,
              float temperature, int dtype, cudaStream_t st) {
  return tt_sample_top_p(logits, uniforms, tokens, logprobs, B, V, ld_row, temperature, 1.f, dtype, st);
}

// top_p in (0, 1]: nucleus sampling (1 = the whole vocabulary).
int tt_sample_top_p(const void* logits, const float* uniforms, long long* tokens, float* logprobs, int B, int V,
                    long long ld_row, float temperature, float top_p, int dtype, cudaStream_t st) {
  if (B <= 0) return 0;
  if (!(top_p > 0.f)) return -2;
  const int mode = temperature > 0.f ? 1 : 0;
  const float inv_t = mode ? 1.f / temperature : 1.f;
  if (dtype == 0)
    sample_kernel<float><<<B, 1024, 0, st>>>(static_cast<const float*>(logits), uniforms, tokens, logprobs, V, ld_row, inv_t, mode, top_p);
  else
    sample_kernel<__nv_bfloat16><<<B, 1024, 0, st>>>(static_cast<const __nv_bfloat16*>(logits), uniforms, tokens, logprobs, V,
                                                      ld_row, inv_t, mode, top_p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // extern "C"
