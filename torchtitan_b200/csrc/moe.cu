// Mixture-of-experts routing and row movement.
//
//   route_fwd   one warp per token: scores = softmax | sigmoid of the fp32 gate logits, experts chosen by
//               (score + expert_bias) -- the bias only affects the choice --, k rounds of warp arg-max (lowest index
//               wins ties), optional normalisation of the k weights and scaling, per-expert histogram (fp32 atomics of
//               integers: exact and order-independent).
//   route_bwd   gradient of the k output weights with respect to the logits.
//   sort        stable counting sort of the T*k (token, slot) pairs by expert: CTA e walks the pair list in order and
//               emits the pairs routed to expert e behind the exclusive prefix of the counts. Deterministic.
//   gather      out[j] = x[src[j]] * scale[j]   (src < 0 gives a zero row; scale optional)
//   combine     out[t] = sum_s w[t,s] * rows[pos[t,s]]   (fp32 accumulation; w optional)
//   rowdot      d[t,s] = <rows[pos[t,s]], g[t]>          (gradient of the combine weights)
//
// Replaces the eager softmax/top-k/histc/argsort sequence and the Triton index kernel of the reference
// (torchtitan/models/common/moe/moe.py:245-370, moe/kernels.py:16-104).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace {

constexpr int MAX_E_PER_LANE = 8;   // up to 256 experts
constexpr int MAX_K = 16;

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// expert e lives in lane e % 32, slot e / 32
__global__ void route_fwd_kernel(const float* __restrict__ logits, const float* __restrict__ expert_bias,
                                 float* __restrict__ top, long long* __restrict__ idx, float* __restrict__ counts, int T,
                                 int E, int K, int softmax, int norm, float route_scale) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= T) return;
  const float* l = logits + static_cast<long long>(warp) * E;
  float s[MAX_E_PER_LANE], c[MAX_E_PER_LANE];
  const int slots = (E + 31) >> 5;
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < MAX_E_PER_LANE; ++j) {
    const int e = j * 32 + lane;
    s[j] = (j < slots && e < E) ? l[e] : -INFINITY;
    mx = fmaxf(mx, s[j]);
  }
  if (softmax) {
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < MAX_E_PER_LANE; ++j) { s[j] = (s[j] == -INFINITY) ? 0.f : __expf(s[j] - mx); sum += s[j]; }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
#pragma unroll
    for (int j = 0; j < MAX_E_PER_LANE; ++j) s[j] *= inv;
  } else {
#pragma unroll
    for (int j = 0; j < MAX_E_PER_LANE; ++j) s[j] = (s[j] == -INFINITY) ? 0.f : 1.f / (1.f + __expf(-s[j]));
  }
#pragma unroll
  for (int j = 0; j < MAX_E_PER_LANE; ++j) {
    const int e = j * 32 + lane;
    c[j] = (j < slots && e < E) ? s[j] + (expert_bias ? expert_bias[e] : 0.f) : -INFINITY;
  }
  float picked[MAX_K];
  int picked_e[MAX_K];
  float tsum = 0.f;
  for (int k = 0; k < K; ++k) {
    float best = -INFINITY;
    int be = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < MAX_E_PER_LANE; ++j) {
      const int e = j * 32 + lane;
      if (c[j] > best) { best = c[j]; be = e; }   // ascending e inside a lane: first maximum kept
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (ob > best || (ob == best && oe < be)) { best = ob; be = oe; }
    }
    // owner lane fetches the unbiased score and retires the expert
    float sc = 0.f;
    if ((be & 31) == lane) {
#pragma unroll
      for (int j = 0; j < MAX_E_PER_LANE; ++j) if (j == (be >> 5)) { sc = s[j]; c[j] = -INFINITY; }
    }
    sc = __shfl_sync(0xffffffffu, sc, be & 31);
    picked[k] = sc;
    picked_e[k] = be;
    tsum += sc;
  }
  if (lane == 0) {
    const float d = norm ? 1.f / (tsum + 1e-20f) : 1.f;
    for (int k = 0; k < K; ++k) {
      top[static_cast<long long>(warp) * K + k] = picked[k] * d * route_scale;
      idx[static_cast<long long>(warp) * K + k] = picked_e[k];
      atomicAdd(counts + picked_e[k], 1.f);
    }
  }
}

__global__ void route_bwd_kernel(const float* __restrict__ logits, const long long* __restrict__ idx,
                                 const float* __restrict__ gtop, float* __restrict__ glogits, int T, int E, int K,
                                 int softmax, int norm, float route_scale) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= T) return;
  const float* l = logits + static_cast<long long>(warp) * E;
  float s[MAX_E_PER_LANE], gs[MAX_E_PER_LANE];
  const int slots = (E + 31) >> 5;
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < MAX_E_PER_LANE; ++j) {
    const int e = j * 32 + lane;
    s[j] = (j < slots && e < E) ? l[e] : -INFINITY;
    gs[j] = 0.f;
    mx = fmaxf(mx, s[j]);
  }
  if (softmax) {
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < MAX_E_PER_LANE; ++j) { s[j] = (s[j] == -INFINITY) ? 0.f : __expf(s[j] - mx); sum += s[j]; }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
#pragma unroll
    for (int j = 0; j < MAX_E_PER_LANE; ++j) s[j] *= inv;
  } else {
#pragma unroll
    for (int j = 0; j < MAX_E_PER_LANE; ++j) s[j] = (s[j] == -INFINITY) ? 0.f : 1.f / (1.f + __expf(-s[j]));
  }
  // gradient with respect to the k chosen raw scores (undo scale and normalisation)
  float tsum = 0.f, dot = 0.f;
  int te[MAX_K];
  for (int k = 0; k < K; ++k) {
    const int e = static_cast<int>(idx[static_cast<long long>(warp) * K + k]);
    float sc = 0.f;
    if ((e & 31) == lane) {
#pragma unroll
      for (int j = 0; j < MAX_E_PER_LANE; ++j) if (j == (e >> 5)) sc = s[j];
    }
    sc = __shfl_sync(0xffffffffu, sc, e & 31);
    te[k] = e;
    tsum += sc;
    dot += gtop[static_cast<long long>(warp) * K + k] * sc;
  }
  for (int k = 0; k < K; ++k) {
    float a = gtop[static_cast<long long>(warp) * K + k] * route_scale;
    if (norm) {
      const float den = tsum + 1e-20f;
      a = (gtop[static_cast<long long>(warp) * K + k] - dot / den) * route_scale / den;
    }
    if ((te[k] & 31) == lane) {
#pragma unroll
      for (int j = 0; j < MAX_E_PER_LANE; ++j) if (j == (te[k] >> 5)) gs[j] += a;
    }
  }
  float* go = glogits + static_cast<long long>(warp) * E;
  if (softmax) {
    float inner = 0.f;
#pragma unroll
    for (int j = 0; j < MAX_E_PER_LANE; ++j) inner += gs[j] * s[j];
    inner = warp_sum(inner);
#pragma unroll
    for (int j = 0; j < MAX_E_PER_LANE; ++j) {
      const int e = j * 32 + lane;
      if (j < slots && e < E) go[e] = s[j] * (gs[j] - inner);
    }
  } else {
#pragma unroll
    for (int j = 0; j < MAX_E_PER_LANE; ++j) {
      const int e = j * 32 + lane;
      if (j < slots && e < E) go[e] = gs[j] * s[j] * (1.f - s[j]);
    }
  }
}

// CTA e: stable positions of all pairs routed to expert e
__global__ void __launch_bounds__(1024)
sort_kernel(const long long* __restrict__ idx, const float* __restrict__ counts, long long* __restrict__ order,
            long long* __restrict__ counts_i64, long long n, int E) {
  const int e = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  __shared__ int s_warp[32];
  __shared__ long long s_base;
  if (tid == 0) {
    long long b = 0;
    for (int j = 0; j < e; ++j) b += static_cast<long long>(counts[j]);
    s_base = b;
    counts_i64[e] = static_cast<long long>(counts[e]);
  }
  __syncthreads();
  long long run = s_base;
  for (long long i0 = 0; i0 < n; i0 += 1024) {
    const long long i = i0 + tid;
    const bool hit = i < n && idx[i] == e;
    const unsigned bal = __ballot_sync(0xffffffffu, hit);
    const int in_warp = __popc(bal & ((1u << lane) - 1));
    if (lane == 0) s_warp[warp] = __popc(bal);
    __syncthreads();
    int before = 0, total = 0;
#pragma unroll 1
    for (int w = 0; w < 32; ++w) { const int c = s_warp[w]; if (w < warp) before += c; total += c; }
    if (hit) order[run + before + in_warp] = i;
    run += total;
    __syncthreads();
  }
}

// one warp per output row; D multiple of 8 (16-byte chunks)
__global__ void gather_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ src, const float* __restrict__ scale,
                              __nv_bfloat16* __restrict__ out, long long R, int D) {
  const long long row = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= R) return;
  const int s = src ? src[row] : static_cast<int>(row);   // no index: rows in place (a plain per-row scaling)
  const float sc = scale ? scale[row] : 1.f;
  for (int c = lane; c < D / 8; c += 32) {
    uint4 v = make_uint4(0, 0, 0, 0);
    if (s >= 0) {
      v = *reinterpret_cast<const uint4*>(x + static_cast<long long>(s) * D + c * 8);
      if (scale) {
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
        for (int e = 0; e < 4; ++e) { float2 f = __bfloat1622float2(h[e]); h[e] = __floats2bfloat162_rn(f.x * sc, f.y * sc); }
      }
    }
    *reinterpret_cast<uint4*>(out + row * D + c * 8) = v;
  }
}

__global__ void combine_kernel(const __nv_bfloat16* __restrict__ rows, const int* __restrict__ pos, const float* __restrict__ w,
                               __nv_bfloat16* __restrict__ out, long long T, int K, int D) {
  const long long t = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (t >= T) return;
  for (int c = lane; c < D / 8; c += 32) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int s = 0; s < K; ++s) {
      const int p = pos[t * K + s];
      if (p < 0) continue;
      const float ws = w ? w[t * K + s] : 1.f;
      const uint4 v = *reinterpret_cast<const uint4*>(rows + static_cast<long long>(p) * D + c * 8);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int e = 0; e < 4; ++e) { const float2 f = __bfloat1622float2(h[e]); acc[2 * e] += ws * f.x; acc[2 * e + 1] += ws * f.y; }
    }
    uint4 o;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e) oh[e] = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
    *reinterpret_cast<uint4*>(out + t * D + c * 8) = o;
  }
}

__global__ void rowdot_kernel(const __nv_bfloat16* __restrict__ rows, const int* __restrict__ pos,
                              const __nv_bfloat16* __restrict__ g, float* __restrict__ d, long long TK, int K, int D) {
  const long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (i >= TK) return;
  const int p = pos ? pos[i] : static_cast<int>(i);       // no index: row i against row i / K of g
  float acc = 0.f;
  if (p >= 0) {
    const long long t = i / K;
    for (int c = lane; c < D / 8; c += 32) {
      const uint4 a = *reinterpret_cast<const uint4*>(rows + static_cast<long long>(p) * D + c * 8);
      const uint4 b = *reinterpret_cast<const uint4*>(g + t * D + c * 8);
      const __nv_bfloat162* ah = reinterpret_cast<const __nv_bfloat162*>(&a);
      const __nv_bfloat162* bh = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
      for (int e = 0; e < 4; ++e) { const float2 x = __bfloat1622float2(ah[e]), y = __bfloat1622float2(bh[e]); acc += x.x * y.x + x.y * y.y; }
    }
  }
  acc = warp_sum(acc);
  if (lane == 0) d[i] = acc;
}

}  // namespace

extern "C" {

// counts [E] fp32 must be zeroed by the caller (it is accumulated into).
int tt_moe_route_fwd(const float* logits, const float* expert_bias, float* top, long long* idx, float* counts, int T, int E,
                     int K, int softmax, int norm, float route_scale, cudaStream_t st) {
  if (E > 32 * MAX_E_PER_LANE || K > MAX_K || K > E) return -2;
  if (T <= 0) return 0;
  route_fwd_kernel<<<(T + 7) / 8, 256, 0, st>>>(logits, expert_bias, top, idx, counts, T, E, K, softmax, norm, route_scale);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

int tt_moe_route_bwd(const float* logits, const long long* idx, const float* gtop, float* glogits, int T, int E, int K,
                     int softmax, int norm, float route_scale, cudaStream_t st) {
  if (E > 32 * MAX_E_PER_LANE || K > MAX_K) return -2;
  if (T <= 0) return 0;
  route_bwd_kernel<<<(T + 7) / 8, 256, 0, st>>>(logits, idx, gtop, glogits, T, E, K, softmax, norm, route_scale);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

int tt_moe_sort(const long long* idx, const float* counts, long long* order, long long* counts_i64, long long n, int E,
                cudaStream_t st) {
  if (E <= 0) return -2;
  sort_kernel<<<E, 1024, 0, st>>>(idx, counts, order, counts_i64, n, E);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

int tt_moe_gather(const void* x, const int* src, const float* scale, void* out, long long R, int D, cudaStream_t st) {
  if (D % 8) return -3;
  if (R <= 0) return 0;
  gather_kernel<<<static_cast<unsigned>((R + 7) / 8), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), src, scale,
                                                                     static_cast<__nv_bfloat16*>(out), R, D);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

int tt_moe_combine(const void* rows, const int* pos, const float* w, void* out, long long T, int K, int D, cudaStream_t st) {
  if (D % 8) return -3;
  if (T <= 0) return 0;
  combine_kernel<<<static_cast<unsigned>((T + 7) / 8), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(rows), pos, w,
                                                                      static_cast<__nv_bfloat16*>(out), T, K, D);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

int tt_moe_rowdot(const void* rows, const int* pos, const void* g, float* d, long long T, int K, int D, cudaStream_t st) {
  if (D % 8) return -3;
  if (T <= 0) return 0;
  const long long TK = T * K;
  rowdot_kernel<<<static_cast<unsigned>((TK + 7) / 8), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(rows), pos,
                                                                     static_cast<const __nv_bfloat16*>(g), d, TK, K, D);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // extern "C"
