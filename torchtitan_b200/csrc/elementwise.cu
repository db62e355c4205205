// Memory-bound training ops: RMSNorm, RoPE, SwiGLU, cross-entropy (+ log-probs), AdamW over flat
// shards, sum of squares. All math in fp32; 16-byte vector loads/stores; grids sized against the
// 148 SMs. Replaces the ATen kernel chains the reference runs for the same steps
// (torchtitan/models/common/rmsnorm.py:14-50, rope.py:293-356, feed_forward.py:61-62,
// torchtitan/components/loss.py:21-28, optimizer.py:100-110, torchtitan/distributed/utils.py:450-474).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

namespace {

constexpr int kSMs = 148;

template <typename T> struct Vec8;  // 8 elements of T with fp32 conversion
template <> struct Vec8<__nv_bfloat16> {
  uint4 raw;
  __device__ void load(const __nv_bfloat16* p) { raw = *reinterpret_cast<const uint4*>(p); }
  __device__ void store(__nv_bfloat16* p) const { *reinterpret_cast<uint4*>(p) = raw; }
  __device__ void to_float(float (&f)[8]) const {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 v = __bfloat1622float2(h[i]); f[2 * i] = v.x; f[2 * i + 1] = v.y; }
  }
  __device__ void from_float(const float (&f)[8]) {
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  }
};
template <> struct Vec8<float> {
  float4 a, b;
  __device__ void load(const float* p) { a = *reinterpret_cast<const float4*>(p); b = *reinterpret_cast<const float4*>(p + 4); }
  __device__ void store(float* p) const { *reinterpret_cast<float4*>(p) = a; *reinterpret_cast<float4*>(p + 4) = b; }
  __device__ void to_float(float (&f)[8]) const { f[0]=a.x; f[1]=a.y; f[2]=a.z; f[3]=a.w; f[4]=b.x; f[5]=b.y; f[6]=b.z; f[7]=b.w; }
  __device__ void from_float(const float (&f)[8]) { a = make_float4(f[0],f[1],f[2],f[3]); b = make_float4(f[4],f[5],f[6],f[7]); }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// block-wide sum; `red` has >= 32 floats of shared memory; result returned to every thread
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : 0.f;
  return warp_sum(t);
}
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : -INFINITY;
  return warp_max(t);
}

// ============================================================================ RMSNorm
// One group of G threads per row (G = 32 for short rows such as per-head QK-norm, else the block).
template <typename T, int G>
__global__ void rmsnorm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ y,
                                   float* __restrict__ rstd_out, long long rows, int D, float eps) {
  __shared__ float red[32];
  const int groups_per_block = blockDim.x / G;
  const int g = threadIdx.x / G, gl = threadIdx.x % G;
  for (long long row = static_cast<long long>(blockIdx.x) * groups_per_block + g; row < rows;
       row += static_cast<long long>(gridDim.x) * groups_per_block) {
    const T* xr = x + row * D;
    float ss = 0.f;
    for (int i = gl * 8; i < D; i += G * 8) {
      Vec8<T> v; v.load(xr + i);
      float f[8]; v.to_float(f);
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += f[e] * f[e];
    }
    ss = (G == 32) ? warp_sum(ss) : block_sum(ss, red);
    const float rstd = rsqrtf(ss / D + eps);
    if (gl == 0 && rstd_out) rstd_out[row] = rstd;
    T* yr = y + row * D;
    for (int i = gl * 8; i < D; i += G * 8) {
      Vec8<T> v; v.load(xr + i);
      float f[8]; v.to_float(f);
      if (w) {
        Vec8<T> wv; wv.load(w + i);
        float wf[8]; wv.to_float(wf);
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] = f[e] * rstd * wf[e];
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] *= rstd;
      }
      v.from_float(f); v.store(yr + i);
    }
  }
}

// Register-resident form for bf16 rows of 256 * NV elements (NV <= 16, e.g. 4096): one warp per row, the row is read
// once (NV 16-byte vectors per lane), reduced with shuffles only and written back; the weight vector (8 KB at most)
// is re-read per row from L1. No block-level synchronisation, so many rows are in flight per SM.
template <int NV>
__global__ void __launch_bounds__(256, 2)
rmsnorm_fwd_warp_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                        __nv_bfloat16* __restrict__ y, float* __restrict__ rstd_out, long long rows, float eps) {
  constexpr int D = NV * 256;
  const int lane = threadIdx.x & 31;
  const long long warp0 = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long row = warp0; row < rows; row += nwarps) {
    const __nv_bfloat16* xr = x + row * D;
    uint4 v[NV];
#pragma unroll
    for (int j = 0; j < NV; ++j) v[j] = *reinterpret_cast<const uint4*>(xr + (j * 32 + lane) * 8);
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[j]);
#pragma unroll
      for (int e = 0; e < 4; ++e) { const float2 f = __bfloat1622float2(h[e]); ss += f.x * f.x + f.y * f.y; }
    }
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / D + eps);
    if (lane == 0 && rstd_out) rstd_out[row] = rstd;
    __nv_bfloat16* yr = y + row * D;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[j]);
      uint4 wq = make_uint4(0, 0, 0, 0);
      if (w) wq = __ldg(reinterpret_cast<const uint4*>(w + (j * 32 + lane) * 8));
      const __nv_bfloat162* wh = reinterpret_cast<const __nv_bfloat162*>(&wq);
      uint4 o;
      __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float2 f = __bfloat1622float2(h[e]);
        f.x *= rstd; f.y *= rstd;
        if (w) { const float2 g = __bfloat1622float2(wh[e]); f.x *= g.x; f.y *= g.y; }
        oh[e] = __floats2bfloat162_rn(f.x, f.y);
      }
      *reinterpret_cast<uint4*>(yr + (j * 32 + lane) * 8) = o;
    }
  }
}

// dx = rstd * (dy*w - x * rstd^2 * mean(dy*w*x));  dw partials per block row-slice -> scratch[blk, D]
template <typename T, int G>
__global__ void rmsnorm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ w,
                                   const float* __restrict__ rstd_in, T* __restrict__ dx,
                                   float* __restrict__ dw_partial, long long rows, int D) {
  extern __shared__ float sm[];  // [32] reduction + [D] dw accumulation (block-shared)
  float* red = sm;
  float* dw_acc = sm + 32;
  for (int i = threadIdx.x; i < D; i += blockDim.x) dw_acc[i] = 0.f;
  __syncthreads();
  const int groups_per_block = blockDim.x / G;
  const int g = threadIdx.x / G, gl = threadIdx.x % G;
  for (long long row0 = static_cast<long long>(blockIdx.x) * groups_per_block; row0 < rows;
       row0 += static_cast<long long>(gridDim.x) * groups_per_block) {
    const long long row = row0 + g;
    const bool live = row < rows;
    const T* xr = x + row * D;
    const T* dyr = dy + row * D;
    const float rstd = live ? rstd_in[row] : 0.f;
    float dot = 0.f;
    if (live) {
      for (int i = gl * 8; i < D; i += G * 8) {
        Vec8<T> xv, dv; xv.load(xr + i); dv.load(dyr + i);
        float xf[8], df[8]; xv.to_float(xf); dv.to_float(df);
        if (w) {
          Vec8<T> wv; wv.load(w + i); float wf[8]; wv.to_float(wf);
#pragma unroll
          for (int e = 0; e < 8; ++e) dot += df[e] * wf[e] * xf[e];
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) dot += df[e] * xf[e];
        }
      }
    }
    dot = (G == 32) ? warp_sum(dot) : block_sum(dot, red);
    const float c = dot * rstd * rstd / D;
    if (live) {
      T* dxr = dx + row * D;
      for (int i = gl * 8; i < D; i += G * 8) {
        Vec8<T> xv, dv; xv.load(xr + i); dv.load(dyr + i);
        float xf[8], df[8], o[8]; xv.to_float(xf); dv.to_float(df);
        float wf[8];
        if (w) { Vec8<T> wv; wv.load(w + i); wv.to_float(wf); }
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float dyw = w ? df[e] * wf[e] : df[e];
          o[e] = rstd * (dyw - xf[e] * c);
          if (w) {
            if (G == 32) atomicAdd(&dw_acc[i + e], df[e] * xf[e] * rstd);  // several rows per block share dw_acc
            else dw_acc[i + e] += df[e] * xf[e] * rstd;                    // one row at a time: exclusive columns
          }
        }
        Vec8<T> ov; ov.from_float(o); ov.store(dxr + i);
      }
    }
  }
  __syncthreads();
  if (w && dw_partial)
    for (int i = threadIdx.x; i < D; i += blockDim.x) dw_partial[static_cast<long long>(blockIdx.x) * D + i] = dw_acc[i];
}

template <typename T>
__global__ void colsum_partials_kernel(const float* __restrict__ partial, T* __restrict__ out, int nblk, int D) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= D) return;
  float s = 0.f;
  for (int b = 0; b < nblk; ++b) s += partial[static_cast<long long>(b) * D + i];
  if constexpr (sizeof(T) == 2) out[i] = __float2bfloat16(s); else out[i] = s;
}

// ============================================================================ RoPE
// x [B,S,H,D]; table [maxS, D/2] float2 (cos, sin); pos (optional) int64 [pos_batch(1|B), S].
// layout 0: pairs (2i, 2i+1); layout 1: pairs (i, i + D/2). inverse: rotate by -angle (backward).
// Vectorised: one thread rotates 8 consecutive elements (interleaved layout: 4 pairs) or 8 elements
// of the first half together with their partners in the second half (half layout: 8 pairs).
template <typename T>
__global__ void rope_kernel(const T* __restrict__ x, T* __restrict__ y, const float2* __restrict__ table,
                            const long long* __restrict__ pos, int pos_batch, int B, int S, int H, int D,
                            int layout, int inverse, long long total_items) {
  const int half = D / 2;
  const int per_row = layout == 0 ? D / 8 : half / 8;  // work items per (b,s,h) row
  for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total_items;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(idx % per_row);
    const long long bsh = idx / per_row;
    const long long bs = bsh / H;
    const int s = static_cast<int>(bs % S);
    const int b = static_cast<int>(bs / S);
    const long long ps = pos ? pos[(pos_batch == 1 ? 0 : static_cast<long long>(b) * S) + s] : s;
    const T* xr = x + bsh * D;
    T* yr = y + bsh * D;
    const float sgn = inverse ? -1.f : 1.f;
    if (layout == 0) {
      Vec8<T> v; v.load(xr + c * 8);
      float f[8], o[8]; v.to_float(f);
      const float2* t = table + ps * half + c * 4;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 cs = t[i];
        const float sn = cs.y * sgn;
        o[2 * i] = f[2 * i] * cs.x - f[2 * i + 1] * sn;
        o[2 * i + 1] = f[2 * i] * sn + f[2 * i + 1] * cs.x;
      }
      v.from_float(o); v.store(yr + c * 8);
    } else {
      Vec8<T> va, vb; va.load(xr + c * 8); vb.load(xr + half + c * 8);
      float fa[8], fb[8], oa[8], ob[8]; va.to_float(fa); vb.to_float(fb);
      const float2* t = table + ps * half + c * 8;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float2 cs = t[i];
        const float sn = cs.y * sgn;
        oa[i] = fa[i] * cs.x - fb[i] * sn;
        ob[i] = fa[i] * sn + fb[i] * cs.x;
      }
      va.from_float(oa); vb.from_float(ob);
      va.store(yr + c * 8); vb.store(yr + half + c * 8);
    }
  }
}

// ============================================================================ SwiGLU
template <typename T>
__global__ void swiglu_fwd_kernel(const T* __restrict__ g, const T* __restrict__ u, T* __restrict__ out, long long n8) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    Vec8<T> gv, uv; gv.load(g + i * 8); uv.load(u + i * 8);
    float gf[8], uf[8], o[8]; gv.to_float(gf); uv.to_float(uf);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = __fdividef(gf[e], 1.f + __expf(-gf[e])) * uf[e];   // approximate divide: 2 ulp, issue-bound otherwise
    Vec8<T> ov; ov.from_float(o); ov.store(out + i * 8);
  }
}
template <typename T>
__global__ void swiglu_bwd_kernel(const T* __restrict__ dout, const T* __restrict__ g, const T* __restrict__ u,
                                  T* __restrict__ dg, T* __restrict__ du, long long n8) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    Vec8<T> gv, uv, dv; gv.load(g + i * 8); uv.load(u + i * 8); dv.load(dout + i * 8);
    float gf[8], uf[8], df[8], og[8], ou[8]; gv.to_float(gf); uv.to_float(uf); dv.to_float(df);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float sg = __fdividef(1.f, 1.f + __expf(-gf[e]));
      const float silu = gf[e] * sg;
      ou[e] = df[e] * silu;
      og[e] = df[e] * uf[e] * (sg + silu * (1.f - sg));
    }
    Vec8<T> a, b; a.from_float(og); b.from_float(ou); a.store(dg + i * 8); b.store(du + i * 8);
  }
}

// ============================================================================ cross entropy
// One block per row. Pass 1: online max / sum-exp -> lse, target logit; loss_row = lse - logit[label].
template <typename T>
__global__ void ce_fwd_kernel(const T* __restrict__ logits, const long long* __restrict__ labels,
                              float* __restrict__ lse_out, float* __restrict__ loss_rows,
                              float* __restrict__ logprob_out, long long rows, int V, long long ld, int ignore_index) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  if (row >= rows) return;
  const T* lr = logits + row * ld;
  float m = -INFINITY, s = 0.f;
  const int V8 = (V / 8) * 8;
  for (int i = threadIdx.x * 8; i < V8; i += blockDim.x * 8) {
    Vec8<T> v; v.load(lr + i);
    float f[8]; v.to_float(f);
    float cm = f[0];
#pragma unroll
    for (int e = 1; e < 8; ++e) cm = fmaxf(cm, f[e]);
    if (cm > m) { s *= __expf(m - cm); m = cm; }
#pragma unroll
    for (int e = 0; e < 8; ++e) s += __expf(f[e] - m);
  }
  for (int i = V8 + threadIdx.x; i < V; i += blockDim.x) {
    float f;
    if constexpr (sizeof(T) == 2) f = __bfloat162float(lr[i]); else f = lr[i];
    if (f > m) { s *= __expf(m - f); m = f; }
    s += __expf(f - m);
  }
  const float gm = block_max(m, red);
  s = (m == -INFINITY) ? 0.f : s * __expf(m - gm);
  const float gs = block_sum(s, red);
  if (threadIdx.x == 0) {
    const float lse = gm + logf(gs);
    if (lse_out) lse_out[row] = lse;
    const long long lab = labels[row];
    float tgt = 0.f;
    const bool valid = lab != ignore_index && lab >= 0 && lab < V;
    if (valid) {
      if constexpr (sizeof(T) == 2) tgt = __bfloat162float(lr[lab]); else tgt = lr[lab];
    }
    if (loss_rows) loss_rows[row] = valid ? (lse - tgt) : 0.f;
    if (logprob_out) logprob_out[row] = valid ? (tgt - lse) : 0.f;
  }
}
// dlogits[row, v] = scale_row * (exp(l - lse) - [v == label]); scale_row = gscale[0] * row_scale[row] (either optional).
template <typename T>
__global__ void ce_bwd_kernel(const T* __restrict__ logits, const long long* __restrict__ labels,
                              const float* __restrict__ lse, const float* __restrict__ gscale,
                              const float* __restrict__ row_scale, T* __restrict__ dlogits, long long rows, int V,
                              long long ld, int ignore_index, int negate) {
  const long long row = blockIdx.x;
  if (row >= rows) return;
  const T* lr = logits + row * ld;
  T* dr = dlogits + row * ld;
  const long long lab = labels[row];
  const bool valid = lab != ignore_index && lab >= 0 && lab < V;
  float sc = gscale ? gscale[0] : 1.f;
  if (row_scale) sc *= row_scale[row];
  if (negate) sc = -sc;
  if (!valid) sc = 0.f;
  const float l = lse[row];
  const int V8 = (V / 8) * 8;
  for (int i = threadIdx.x * 8; i < V8; i += blockDim.x * 8) {
    Vec8<T> v; v.load(lr + i);
    float f[8]; v.to_float(f);
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] = sc * (__expf(f[e] - l) - ((i + e) == lab ? 1.f : 0.f));
    v.from_float(f); v.store(dr + i);
  }
  for (int i = V8 + threadIdx.x; i < V; i += blockDim.x) {
    float f;
    if constexpr (sizeof(T) == 2) f = __bfloat162float(lr[i]); else f = lr[i];
    f = sc * (__expf(f - l) - (i == lab ? 1.f : 0.f));
    if constexpr (sizeof(T) == 2) dr[i] = __float2bfloat16(f); else dr[i] = f;
  }
}
__global__ void sum_rows_kernel(const float* __restrict__ v, float* __restrict__ out, long long n) {
  __shared__ float red[32];
  float s = 0.f;
  for (long long i = threadIdx.x; i < n; i += blockDim.x) s += v[i];
  s = block_sum(s, red);
  if (threadIdx.x == 0) out[0] = s;
}

// ============================================================================ AdamW / norms
// p,g,m,v fp32 flat; shadow (optional) bf16 copy of the updated parameters.
// gscale (optional) device scalar multiplying the gradient (folded gradient clipping).
__device__ __forceinline__ float sqrt_approx(float x) {
  float y;
  asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float rcp_approx(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__global__ void __launch_bounds__(256) adamw_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
                             float* __restrict__ v, __nv_bfloat16* __restrict__ shadow, long long n, float lr,
                             float beta1, float beta2, float eps, float wd, float bc1, float bc2_sqrt,
                             int decoupled, const float* __restrict__ gscale) {
  const float gs = gscale ? gscale[0] : 1.f;
  const float decay = 1.f - lr * wd, omb1 = 1.f - beta1, omb2 = 1.f - beta2, inv_bc2_sqrt = 1.f / bc2_sqrt, step_size = lr / bc1;
  for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 4; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x * 4) {
    if (i + 4 <= n) {
      float4 pv = *reinterpret_cast<float4*>(p + i), gv = *reinterpret_cast<const float4*>(g + i);
      float4 mv = *reinterpret_cast<float4*>(m + i), vv = *reinterpret_cast<float4*>(v + i);
      float pp[4] = {pv.x, pv.y, pv.z, pv.w}, gg[4] = {gv.x, gv.y, gv.z, gv.w};
      float mm[4] = {mv.x, mv.y, mv.z, mv.w}, vq[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float gr = gg[e] * gs;
        if (decoupled) pp[e] *= decay; else gr += wd * pp[e];
        mm[e] = fmaf(omb1, gr - mm[e], mm[e]);
        vq[e] = fmaf(beta2, vq[e], omb2 * gr * gr);
        // the kernel is bound by memory only while its arithmetic stays short: special-function-unit square root and
        // reciprocal (about 1e-7 relative error each) instead of the IEEE sequences
        const float denom = fmaf(sqrt_approx(vq[e]), inv_bc2_sqrt, eps);
        pp[e] = fmaf(-step_size * mm[e], rcp_approx(denom), pp[e]);
      }
      *reinterpret_cast<float4*>(p + i) = make_float4(pp[0], pp[1], pp[2], pp[3]);
      *reinterpret_cast<float4*>(m + i) = make_float4(mm[0], mm[1], mm[2], mm[3]);
      *reinterpret_cast<float4*>(v + i) = make_float4(vq[0], vq[1], vq[2], vq[3]);
      if (shadow) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(pp[0], pp[1]), hi = __floats2bfloat162_rn(pp[2], pp[3]);
        uint2 pk = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
        *reinterpret_cast<uint2*>(shadow + i) = pk;
      }
    } else {
      for (long long j = i; j < n; ++j) {
        float gr = g[j] * gs, pj = p[j];
        if (decoupled) pj *= (1.f - lr * wd); else gr += wd * pj;
        const float mj = m[j] + (1.f - beta1) * (gr - m[j]);
        const float vj = beta2 * v[j] + (1.f - beta2) * gr * gr;
        pj -= (lr / bc1) * (mj / (sqrtf(vj) / bc2_sqrt + eps));
        p[j] = pj; m[j] = mj; v[j] = vj;
        if (shadow) shadow[j] = __float2bfloat16(pj);
      }
    }
  }
}

template <typename T>
__global__ void sumsq_kernel(const T* __restrict__ x, float* __restrict__ partial, long long n) {
  __shared__ float red[32];
  float s = 0.f;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float f;
    if constexpr (sizeof(T) == 2) f = __bfloat162float(x[i]); else f = x[i];
    s += f * f;
  }
  s = block_sum(s, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}

inline int grid_for(long long work_items, int threads, int per_sm = 8) {
  long long blocks = (work_items + threads - 1) / threads;
  long long cap = static_cast<long long>(kSMs) * per_sm;
  return static_cast<int>(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

}  // namespace

extern "C" {

// dtype: 0 = bf16, 1 = fp32. Returns 0 on success.
int tt_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, long long rows, int D, float eps, int dtype,
                   cudaStream_t st) {
  if (D % 8) return -1;
  if (dtype == 0 && rows >= 64 && (D == 4096 || D == 2048) && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(y) & 15) == 0 && (w == nullptr || (reinterpret_cast<uintptr_t>(w) & 15) == 0)) {
    long long blocks = (rows + 7) / 8;                 // 8 warps per block, one row per warp and pass
    if (blocks > kSMs * 8) blocks = kSMs * 8;
    const auto* xp = static_cast<const __nv_bfloat16*>(x);
    const auto* wp = static_cast<const __nv_bfloat16*>(w);
    auto* yp = static_cast<__nv_bfloat16*>(y);
    if (D == 4096) rmsnorm_fwd_warp_kernel<16><<<static_cast<int>(blocks), 256, 0, st>>>(xp, wp, yp, rstd, rows, eps);
    else rmsnorm_fwd_warp_kernel<8><<<static_cast<int>(blocks), 256, 0, st>>>(xp, wp, yp, rstd, rows, eps);
    return cudaGetLastError() == cudaSuccess ? 0 : -4;
  }
  if (D <= 1024) {
    const int threads = 256, gpb = threads / 32;
    int grid = static_cast<int>((rows + gpb - 1) / gpb); if (grid > kSMs * 8) grid = kSMs * 8; if (grid < 1) grid = 1;
    if (dtype == 0) rmsnorm_fwd_kernel<__nv_bfloat16, 32><<<grid, threads, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (__nv_bfloat16*)y, rstd, rows, D, eps);
    else rmsnorm_fwd_kernel<float, 32><<<grid, threads, 0, st>>>((const float*)x, (const float*)w, (float*)y, rstd, rows, D, eps);
  } else {
    const int threads = 512;
    int grid = rows > kSMs * 4 ? kSMs * 4 : static_cast<int>(rows); if (grid < 1) grid = 1;
    if (dtype == 0) rmsnorm_fwd_kernel<__nv_bfloat16, 512><<<grid, threads, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (__nv_bfloat16*)y, rstd, rows, D, eps);
    else rmsnorm_fwd_kernel<float, 512><<<grid, threads, 0, st>>>((const float*)x, (const float*)w, (float*)y, rstd, rows, D, eps);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// Number of fp32 partial rows the backward needs in `scratch` ([blocks, D]).
int tt_rmsnorm_bwd_blocks(long long rows, int D) {
  if (D <= 1024) { const int gpb = 8; long long g = (rows + gpb - 1) / gpb; return static_cast<int>(g > kSMs * 2 ? kSMs * 2 : (g < 1 ? 1 : g)); }
  return static_cast<int>(rows > kSMs * 2 ? kSMs * 2 : (rows < 1 ? 1 : rows));
}

int tt_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx, void* dw,
                   float* scratch, long long rows, int D, int dtype, cudaStream_t st) {
  if (D % 8) return -1;
  const int grid = tt_rmsnorm_bwd_blocks(rows, D);
  const size_t sm = (32 + D) * sizeof(float);
  if (sm > 227 * 1024) return -5;       // D above ~58k: the per-block dW row no longer fits in shared memory
  if (sm > 48 * 1024) {
    // rows wider than 12256 elements (e.g. dim 16384) need the opt-in shared-memory limit
    static bool opted_in = false;
    if (!opted_in) {
      cudaFuncSetAttribute(rmsnorm_bwd_kernel<__nv_bfloat16, 512>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
      cudaFuncSetAttribute(rmsnorm_bwd_kernel<float, 512>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
      opted_in = true;
    }
  }
  if (D <= 1024) {
    if (dtype == 0) rmsnorm_bwd_kernel<__nv_bfloat16, 32><<<grid, 256, sm, st>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, rstd, (__nv_bfloat16*)dx, scratch, rows, D);
    else rmsnorm_bwd_kernel<float, 32><<<grid, 256, sm, st>>>((const float*)dy, (const float*)x, (const float*)w, rstd, (float*)dx, scratch, rows, D);
  } else {
    if (dtype == 0) rmsnorm_bwd_kernel<__nv_bfloat16, 512><<<grid, 512, sm, st>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, rstd, (__nv_bfloat16*)dx, scratch, rows, D);
    else rmsnorm_bwd_kernel<float, 512><<<grid, 512, sm, st>>>((const float*)dy, (const float*)x, (const float*)w, rstd, (float*)dx, scratch, rows, D);
  }
  if (w && dw) {
    if (dtype == 0) colsum_partials_kernel<__nv_bfloat16><<<(D + 255) / 256, 256, 0, st>>>(scratch, (__nv_bfloat16*)dw, grid, D);
    else colsum_partials_kernel<float><<<(D + 255) / 256, 256, 0, st>>>(scratch, (float*)dw, grid, D);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

int tt_rope(const void* x, void* y, const float* table, const long long* pos, int pos_batch, int B, int S, int H, int D,
            int layout, int inverse, int dtype, cudaStream_t st) {
  if (D % 16) return -1;
  const long long pairs = static_cast<long long>(B) * S * H * (layout == 0 ? D / 8 : D / 16);
  const int grid = grid_for(pairs, 256);
  if (dtype == 0) rope_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, (const float2*)table, pos, pos_batch, B, S, H, D, layout, inverse, pairs);
  else rope_kernel<float><<<grid, 256, 0, st>>>((const float*)x, (float*)y, (const float2*)table, pos, pos_batch, B, S, H, D, layout, inverse, pairs);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

int tt_swiglu_fwd(const void* g, const void* u, void* out, long long n, int dtype, cudaStream_t st) {
  if (n % 8) return -1;
  const int grid = grid_for(n / 8, 256);
  if (dtype == 0) swiglu_fwd_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)g, (const __nv_bfloat16*)u, (__nv_bfloat16*)out, n / 8);
  else swiglu_fwd_kernel<float><<<grid, 256, 0, st>>>((const float*)g, (const float*)u, (float*)out, n / 8);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
int tt_swiglu_bwd(const void* dout, const void* g, const void* u, void* dg, void* du, long long n, int dtype, cudaStream_t st) {
  if (n % 8) return -1;
  const int grid = grid_for(n / 8, 256);
  if (dtype == 0) swiglu_bwd_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)dout, (const __nv_bfloat16*)g, (const __nv_bfloat16*)u, (__nv_bfloat16*)dg, (__nv_bfloat16*)du, n / 8);
  else swiglu_bwd_kernel<float><<<grid, 256, 0, st>>>((const float*)dout, (const float*)g, (const float*)u, (float*)dg, (float*)du, n / 8);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// Per-row lse / loss / log-prob (any of the three outputs may be null); loss_sum (optional) = sum(loss_rows).
int tt_ce_fwd(const void* logits, const long long* labels, float* lse, float* loss_rows, float* logprob,
              float* loss_sum, long long rows, int V, long long ld, int ignore_index, int dtype, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (ld % 8) return -1;
  if (dtype == 0) ce_fwd_kernel<__nv_bfloat16><<<static_cast<unsigned>(rows), 512, 0, st>>>((const __nv_bfloat16*)logits, labels, lse, loss_rows, logprob, rows, V, ld, ignore_index);
  else ce_fwd_kernel<float><<<static_cast<unsigned>(rows), 512, 0, st>>>((const float*)logits, labels, lse, loss_rows, logprob, rows, V, ld, ignore_index);
  if (loss_sum && loss_rows) sum_rows_kernel<<<1, 1024, 0, st>>>(loss_rows, loss_sum, rows);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
int tt_ce_bwd(const void* logits, const long long* labels, const float* lse, const float* gscale,
              const float* row_scale, void* dlogits, long long rows, int V, long long ld, int ignore_index, int negate,
              int dtype, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (ld % 8) return -1;
  if (dtype == 0) ce_bwd_kernel<__nv_bfloat16><<<static_cast<unsigned>(rows), 512, 0, st>>>((const __nv_bfloat16*)logits, labels, lse, gscale, row_scale, (__nv_bfloat16*)dlogits, rows, V, ld, ignore_index, negate);
  else ce_bwd_kernel<float><<<static_cast<unsigned>(rows), 512, 0, st>>>((const float*)logits, labels, lse, gscale, row_scale, (float*)dlogits, rows, V, ld, ignore_index, negate);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

int tt_adamw(float* p, const float* g, float* m, float* v, void* shadow_bf16, long long n, float lr, float beta1,
             float beta2, float eps, float wd, int step, int decoupled, const float* gscale, cudaStream_t st) {
  if (n <= 0) return 0;
  const float bc1 = 1.f - powf(beta1, static_cast<float>(step));
  const float bc2 = 1.f - powf(beta2, static_cast<float>(step));
  const int grid = grid_for((n + 3) / 4, 256);
  adamw_kernel<<<grid, 256, 0, st>>>(p, g, m, v, (__nv_bfloat16*)shadow_bf16, n, lr, beta1, beta2, eps, wd, bc1, sqrtf(bc2), decoupled, gscale);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// out[0] (+)= sum(x^2); scratch must hold 1184 floats.
int tt_sumsq(const void* x, float* scratch, float* out, long long n, int dtype, int accumulate, cudaStream_t st);
}

namespace {
__global__ void finish_sumsq_kernel(const float* __restrict__ partial, float* __restrict__ out, int n, int accumulate) {
  __shared__ float red[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) s += partial[i];
  s = block_sum(s, red);
  if (threadIdx.x == 0) out[0] = accumulate ? out[0] + s : s;
}
}  // namespace

extern "C" int tt_sumsq(const void* x, float* scratch, float* out, long long n, int dtype, int accumulate, cudaStream_t st) {
  const int grid = grid_for(n, 512, 8);
  if (dtype == 0) sumsq_kernel<__nv_bfloat16><<<grid, 512, 0, st>>>((const __nv_bfloat16*)x, scratch, n);
  else sumsq_kernel<float><<<grid, 512, 0, st>>>((const float*)x, scratch, n);
  finish_sumsq_kernel<<<1, 256, 0, st>>>(scratch, out, grid, accumulate);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// ============================================================================ allocation-free entry
// See tt_noalloc.h. The RMSNorm backward needs [blocks, D] fp32 partial sums for dW. Callers that
// may not allocate device memory get them from this file-scope array instead of a caller buffer.
namespace {
constexpr int kNoAllocMaxD = 4096;
constexpr int kNoAllocMaxBlocks = 2 * kSMs;  // upper bound of tt_rmsnorm_bwd_blocks()
static __device__ __align__(256) float g_noalloc_scratch[kNoAllocMaxBlocks * kNoAllocMaxD];  // 4.6 MiB per GPU
constexpr int kNoAllocMaxDevices = 64;
float* g_noalloc_ptr[kNoAllocMaxDevices] = {nullptr};  // device address of the array, per device
}  // namespace

extern "C" {

int tt_rmsnorm_bwd_noalloc_max_dim() { return kNoAllocMaxD; }

const char* tt_noalloc_strerror(int code) {
  switch (code) {
    case 0: return "ok";
    case -20: return "tt_rmsnorm_bwd_noalloc: D exceeds the built-in scratch (max 4096) or is not a multiple of 8";
    case -21: return "tt_rmsnorm_bwd_noalloc: cudaGetSymbolAddress failed for the built-in scratch array";
    case -22: return "tt_rmsnorm_bwd_noalloc: device ordinal out of range";
    default: return "tt_rmsnorm_bwd_noalloc: kernel launch failed";
  }
}

int tt_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, void* dx, void* dw,
                           long long rows, int D, int dtype, cudaStream_t st) {
  if (D > kNoAllocMaxD || D <= 0 || (D % 8)) return -20;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kNoAllocMaxDevices) return -22;
  if (g_noalloc_ptr[dev] == nullptr) {
    // In host code the array's name is only a handle; the kernels need its device address, which
    // differs per device, so it is looked up once per device with that device current.
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || p == nullptr) return -21;
    g_noalloc_ptr[dev] = static_cast<float*>(p);
  }
  // Every launched block overwrites its whole [D] row of partials and the column sum reads exactly
  // those rows, so nothing has to be cleared between calls.
  return tt_rmsnorm_bwd(dy, x, w, rstd, dx, dw, g_noalloc_ptr[dev], rows, D, dtype, st);
}

}  // extern "C"
