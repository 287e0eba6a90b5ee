// Tria readout and RMS-type norms.
//
//   slot_pool     : softmax over the H neurons of <w9, vec(C_h)> and the pooled 9-vector, per boundary key
//                   (reference kernels/tria/slot_attention_pool/slot_attention_pool_kernel.cuh:13-125)
//   cross_attn    : every token row attends to the few (<= 512) boundary keys that precede it
//                   (reference kernels/tria/final_ca_sparse/final_ca_sparse_kernel.cuh:23-178)
//   fixed_rms     : x * target / rms(x) over head_dim, strided input (the K/V projections of depth attention)
//   rms_norm      : x / rms(x) * w over the model width (optional final norm)
//
// All are bandwidth- or latency-bound, so they are plain SIMT kernels with 16-byte accesses; everything a
// backward pass needs is recomputed from the inputs or read from a small saved tensor (softmax statistics, the
// probabilities over the few keys), and every reduction across rows is deterministic (per-block partials that the
// caller sums, no floating-point atomics).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include "loom_c_api.h"

namespace {

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 t = __bfloat1622float2(p[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 u;
  __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return u;
}
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

// ------------------------------------------------------------------------------------------------ slot pool
// keys [BK, H, 9] fp32, w9 [9] -> pooled [BK, 9], stats [BK, 2] = (max score, softmax denominator)
__global__ void __launch_bounds__(256) slot_pool_fwd_kernel(const float* __restrict__ keys, const float* __restrict__ w9,
                                                            float* __restrict__ pooled, float* __restrict__ stats, int H) {
  const float* x = keys + (long long)blockIdx.x * H * 9;
  float w[9];
#pragma unroll
  for (int k = 0; k < 9; ++k) w[k] = w9[k];
  float mx = -INFINITY, den = 0.f, acc[9];
#pragma unroll
  for (int k = 0; k < 9; ++k) acc[k] = 0.f;
  for (int h = threadIdx.x; h < H; h += 256) {
    float v[9], s = 0.f;
#pragma unroll
    for (int k = 0; k < 9; ++k) { v[k] = x[h * 9 + k]; s += w[k] * v[k]; }
    const float nm = fmaxf(mx, s), c = __expf(mx - nm), p = __expf(s - nm);
    den = den * c + p;
#pragma unroll
    for (int k = 0; k < 9; ++k) acc[k] = acc[k] * c + p * v[k];
    mx = nm;
  }
  // merge the 256 online-softmax states
  __shared__ float sm[8], sv[8][10];
  const float wm = warp_max(mx);
  const float c = (mx == -INFINITY) ? 0.f : __expf(mx - wm);
  float d = warp_sum(den * c), a[9];
#pragma unroll
  for (int k = 0; k < 9; ++k) a[k] = warp_sum(acc[k] * c);
  const int wi = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
    sm[wi] = wm; sv[wi][9] = d;
#pragma unroll
    for (int k = 0; k < 9; ++k) sv[wi][k] = a[k];
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float gm = -INFINITY;
    for (int i = 0; i < 8; ++i) gm = fmaxf(gm, sm[i]);
    float gd = 0.f, ga[9];
    for (int k = 0; k < 9; ++k) ga[k] = 0.f;
    for (int i = 0; i < 8; ++i) {
      const float cc = (sm[i] == -INFINITY) ? 0.f : __expf(sm[i] - gm);
      gd += sv[i][9] * cc;
      for (int k = 0; k < 9; ++k) ga[k] += sv[i][k] * cc;
    }
    for (int k = 0; k < 9; ++k) pooled[(long long)blockIdx.x * 9 + k] = ga[k] / gd;
    stats[blockIdx.x * 2] = gm; stats[blockIdx.x * 2 + 1] = gd;
  }
}

// dkeys [BK,H,9]; dw9_part [BK,9] (the caller sums over BK)
__global__ void __launch_bounds__(256) slot_pool_bwd_kernel(const float* __restrict__ keys, const float* __restrict__ w9,
                                                            const float* __restrict__ pooled, const float* __restrict__ stats,
                                                            const float* __restrict__ dpooled, float* __restrict__ dkeys,
                                                            float* __restrict__ dw9_part, int H) {
  const long long bk = blockIdx.x;
  const float* x = keys + bk * H * 9;
  float* dx = dkeys + bk * H * 9;
  float w[9], dp[9], dot_pool = 0.f;
#pragma unroll
  for (int k = 0; k < 9; ++k) { w[k] = w9[k]; dp[k] = dpooled[bk * 9 + k]; dot_pool += dp[k] * pooled[bk * 9 + k]; }
  const float mx = stats[bk * 2], inv = 1.f / stats[bk * 2 + 1];
  float gw[9];
#pragma unroll
  for (int k = 0; k < 9; ++k) gw[k] = 0.f;
  for (int h = threadIdx.x; h < H; h += 256) {
    float v[9], s = 0.f, dv = 0.f;
#pragma unroll
    for (int k = 0; k < 9; ++k) { v[k] = x[h * 9 + k]; s += w[k] * v[k]; dv += dp[k] * v[k]; }
    const float p = __expf(s - mx) * inv;
    const float ds = p * (dv - dot_pool);
#pragma unroll
    for (int k = 0; k < 9; ++k) { dx[h * 9 + k] = p * dp[k] + ds * w[k]; gw[k] += ds * v[k]; }
  }
  __shared__ float sv[8][9];
  const int wi = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
  for (int k = 0; k < 9; ++k) { const float t = warp_sum(gw[k]); if (lane == 0) sv[wi][k] = t; }
  __syncthreads();
  if (threadIdx.x < 9) {
    float t = 0.f;
    for (int i = 0; i < 8; ++i) t += sv[i][threadIdx.x];
    dw9_part[bk * 9 + threadIdx.x] = t;
  }
}

// ------------------------------------------------------------------------------------------------ sparse cross attention
// q [B,T,N], k/v [B,Kn,N] bf16; allowed [B,T,Kn] uint8; out [B,T,N] bf16; prob [B,T,Kn] fp32.
// One warp per token row; NCH 16-byte chunks per lane (N <= 256*NCH).  Rows without an allowed key give zero.
template <int NCH>
__global__ void __launch_bounds__(256) cross_attn_fwd_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k,
                                                             const bf16* __restrict__ v, const uint8_t* __restrict__ allowed,
                                                             bf16* __restrict__ out, float* __restrict__ prob, int B, int T,
                                                             int Kn, int N, float scale) {
  extern __shared__ float sc[];                        // [8][Kn]
  const int wi = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * 8 + wi;
  if (row >= (long long)B * T) return;
  const int b = (int)(row / T);
  float* s = sc + wi * Kn;
  float qf[NCH][8];
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int col = (c * 32 + lane) * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) qf[c][i] = 0.f;
    if (col < N) unpack8(*reinterpret_cast<const uint4*>(q + row * N + col), qf[c]);
  }
  const uint8_t* al = allowed + row * Kn;
  float mx = -INFINITY;
  for (int j = 0; j < Kn; ++j) {
    float d = -INFINITY;
    if (al[j]) {
      const bf16* kr = k + ((long long)b * Kn + j) * N;
      float a = 0.f;
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        const int col = (c * 32 + lane) * 8;
        if (col < N) {
          float kf[8];
          unpack8(*reinterpret_cast<const uint4*>(kr + col), kf);
#pragma unroll
          for (int i = 0; i < 8; ++i) a += qf[c][i] * kf[i];
        }
      }
      d = warp_sum(a) * scale;
      mx = fmaxf(mx, d);
    }
    if (lane == 0) s[j] = d;
  }
  __syncwarp();
  float den = 0.f;
  for (int j = lane; j < Kn; j += 32) { const float e = (s[j] == -INFINITY) ? 0.f : __expf(s[j] - mx); s[j] = e; den += e; }
  den = warp_sum(den);
  const float inv = den > 0.f ? 1.f / den : 0.f;
  __syncwarp();
  for (int j = lane; j < Kn; j += 32) { s[j] *= inv; prob[row * Kn + j] = s[j]; }
  __syncwarp();
  float acc[NCH][8];
#pragma unroll
  for (int c = 0; c < NCH; ++c)
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[c][i] = 0.f;
  for (int j = 0; j < Kn; ++j) {
    const float p = s[j];
    if (p != 0.f) {
      const bf16* vr = v + ((long long)b * Kn + j) * N;
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        const int col = (c * 32 + lane) * 8;
        if (col < N) {
          float vf[8];
          unpack8(*reinterpret_cast<const uint4*>(vr + col), vf);
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[c][i] += p * vf[i];
        }
      }
    }
  }
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int col = (c * 32 + lane) * 8;
    if (col < N) *reinterpret_cast<uint4*>(out + row * N + col) = pack8(acc[c]);
  }
}

// rows: dS [B,T,Kn] fp32 (already times scale) and dq [B,T,N] bf16
template <int NCH>
__global__ void __launch_bounds__(256) cross_attn_bwd_rows_kernel(const bf16* __restrict__ dout, const bf16* __restrict__ k,
                                                                  const bf16* __restrict__ v, const float* __restrict__ prob,
                                                                  float* __restrict__ ds, bf16* __restrict__ dq, int B, int T,
                                                                  int Kn, int N, float scale) {
  extern __shared__ float sc[];                        // [8][Kn]
  const int wi = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * 8 + wi;
  if (row >= (long long)B * T) return;
  const int b = (int)(row / T);
  float* s = sc + wi * Kn;
  float gf[NCH][8];
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int col = (c * 32 + lane) * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) gf[c][i] = 0.f;
    if (col < N) unpack8(*reinterpret_cast<const uint4*>(dout + row * N + col), gf[c]);
  }
  const float* pr = prob + row * Kn;
  float sumw = 0.f;
  for (int j = 0; j < Kn; ++j) {
    const float p = pr[j];
    float dw = 0.f;
    if (p != 0.f) {
      const bf16* vr = v + ((long long)b * Kn + j) * N;
      float a = 0.f;
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        const int col = (c * 32 + lane) * 8;
        if (col < N) {
          float vf[8];
          unpack8(*reinterpret_cast<const uint4*>(vr + col), vf);
#pragma unroll
          for (int i = 0; i < 8; ++i) a += gf[c][i] * vf[i];
        }
      }
      dw = warp_sum(a);
      sumw += p * dw;
    }
    if (lane == 0) s[j] = dw;
  }
  __syncwarp();
  float acc[NCH][8];
#pragma unroll
  for (int c = 0; c < NCH; ++c)
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[c][i] = 0.f;
  for (int j = 0; j < Kn; ++j) {
    const float p = pr[j];
    const float d = p * (s[j] - sumw) * scale;
    if (lane == 0) ds[row * Kn + j] = d;
    if (p != 0.f) {
      const bf16* kr = k + ((long long)b * Kn + j) * N;
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        const int col = (c * 32 + lane) * 8;
        if (col < N) {
          float kf[8];
          unpack8(*reinterpret_cast<const uint4*>(kr + col), kf);
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[c][i] += d * kf[i];
        }
      }
    }
  }
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int col = (c * 32 + lane) * 8;
    if (col < N) *reinterpret_cast<uint4*>(dq + row * N + col) = pack8(acc[c]);
  }
}

// keys: dk[b,j,:] = sum_t dS[b,t,j] q[b,t,:], dv[b,j,:] = sum_t P[b,t,j] dout[b,t,:].  grid (B*Kn, ceil(N/512)),
// one thread per column pair, a fixed summation order over t.
__global__ void __launch_bounds__(256) cross_attn_bwd_keys_kernel(const bf16* __restrict__ q, const bf16* __restrict__ dout,
                                                                  const float* __restrict__ prob, const float* __restrict__ ds,
                                                                  bf16* __restrict__ dk, bf16* __restrict__ dv, int T, int Kn,
                                                                  int N) {
  const int b = blockIdx.x / Kn, j = blockIdx.x % Kn;
  const int col = (blockIdx.y * 256 + threadIdx.x) * 2;
  if (col >= N) return;
  const long long r0 = (long long)b * T;
  float k0 = 0.f, k1 = 0.f, v0 = 0.f, v1 = 0.f;
#pragma unroll 4
  for (int t = 0; t < T; ++t) {
    const float p = prob[(r0 + t) * Kn + j];
    if (p != 0.f) {                                    // uniform across the block
      const float d = ds[(r0 + t) * Kn + j];
      const float2 qq = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(q + (r0 + t) * N + col));
      const float2 gg = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(dout + (r0 + t) * N + col));
      k0 += d * qq.x; k1 += d * qq.y; v0 += p * gg.x; v1 += p * gg.y;
    }
  }
  const long long o = ((long long)b * Kn + j) * N + col;
  *reinterpret_cast<__nv_bfloat162*>(dk + o) = __floats2bfloat162_rn(k0, k1);
  *reinterpret_cast<__nv_bfloat162*>(dv + o) = __floats2bfloat162_rn(v0, v1);
}

// ------------------------------------------------------------------------------------------------ fixed RMS over head_dim
// x: rows of HD elements at x + m*ld + h*HD (bf16); y contiguous [M*heads, HD] bf16.  G lanes per row.
template <int G>
__global__ void __launch_bounds__(256) fixed_rms_fwd_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, long long rows,
                                                            int heads, int HD, long long ld, float target, float eps) {
  const long long gid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) / G;
  const int l = threadIdx.x % G;
  if (gid >= rows) return;
  const unsigned mask = __activemask();
  const bool act = l * 8 < HD;
  float f[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) f[i] = 0.f;
  const long long src = (gid / heads) * ld + (gid % heads) * HD + l * 8;
  if (act) unpack8(*reinterpret_cast<const uint4*>(x + src), f);
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
#pragma unroll
  for (int o = G / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(mask, ss, o, G);
  const float r = target * rsqrtf(ss / HD + eps);
  if (act) {
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] *= r;
    *reinterpret_cast<uint4*>(y + gid * HD + l * 8) = pack8(f);
  }
}

template <int G>
__global__ void __launch_bounds__(256) fixed_rms_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x,
                                                            bf16* __restrict__ dx, long long rows, int heads, int HD,
                                                            long long ld, float target, float eps) {
  const long long gid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) / G;
  const int l = threadIdx.x % G;
  if (gid >= rows) return;
  const unsigned mask = __activemask();
  const bool act = l * 8 < HD;
  float f[8], g[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) { f[i] = 0.f; g[i] = 0.f; }
  const long long src = (gid / heads) * ld + (gid % heads) * HD + l * 8;
  if (act) {
    unpack8(*reinterpret_cast<const uint4*>(x + src), f);
    unpack8(*reinterpret_cast<const uint4*>(dy + gid * HD + l * 8), g);
  }
  float ss = 0.f, gx = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) { ss += f[i] * f[i]; gx += g[i] * f[i]; }
#pragma unroll
  for (int o = G / 2; o > 0; o >>= 1) { ss += __shfl_xor_sync(mask, ss, o, G); gx += __shfl_xor_sync(mask, gx, o, G); }
  const float r = rsqrtf(ss / HD + eps);
  const float c = r * r * gx / HD;
  if (act) {
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = target * r * (g[i] - f[i] * c);
    *reinterpret_cast<uint4*>(dx + gid * HD + l * 8) = pack8(f);
  }
}

// ------------------------------------------------------------------------------------------------ RMSNorm with weight
template <int NCH>
__global__ void __launch_bounds__(256) rms_norm_fwd_kernel(const bf16* __restrict__ x, const float* __restrict__ w,
                                                           bf16* __restrict__ y, int M, int N, float eps) {
  const int wi = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * 8 + wi;
  if (row >= M) return;
  float f[NCH][8], ss = 0.f;
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int col = (c * 32 + lane) * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) f[c][i] = 0.f;
    if (col < N) unpack8(*reinterpret_cast<const uint4*>(x + row * N + col), f[c]);
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += f[c][i] * f[c][i];
  }
  const float r = rsqrtf(warp_sum(ss) / N + eps);
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int col = (c * 32 + lane) * 8;
    if (col < N) {
#pragma unroll
      for (int i = 0; i < 8; ++i) f[c][i] *= r * w[col + i];
      *reinterpret_cast<uint4*>(y + row * N + col) = pack8(f[c]);
    }
  }
}

// dx and per-block partial weight gradients gw_part[gridDim.x][N] (the caller sums the partials)
template <int NCH>
__global__ void __launch_bounds__(256) rms_norm_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x,
                                                           const float* __restrict__ w, bf16* __restrict__ dx,
                                                           float* __restrict__ gw_part, int M, int N, float eps) {
  extern __shared__ float sg[];                        // [8][N]
  const int wi = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float gacc[NCH][8];
#pragma unroll
  for (int c = 0; c < NCH; ++c)
#pragma unroll
    for (int i = 0; i < 8; ++i) gacc[c][i] = 0.f;
  for (long long row = (long long)blockIdx.x * 8 + wi; row < M; row += (long long)gridDim.x * 8) {
    float f[NCH][8], g[NCH][8], ss = 0.f, gx = 0.f;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const int col = (c * 32 + lane) * 8;
#pragma unroll
      for (int i = 0; i < 8; ++i) { f[c][i] = 0.f; g[c][i] = 0.f; }
      if (col < N) {
        unpack8(*reinterpret_cast<const uint4*>(x + row * N + col), f[c]);
        unpack8(*reinterpret_cast<const uint4*>(dy + row * N + col), g[c]);
#pragma unroll
        for (int i = 0; i < 8; ++i) { ss += f[c][i] * f[c][i]; gx += g[c][i] * w[col + i] * f[c][i]; }
      }
    }
    ss = warp_sum(ss); gx = warp_sum(gx);
    const float r = rsqrtf(ss / N + eps);
    const float cc = r * r * gx / N;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const int col = (c * 32 + lane) * 8;
      if (col < N) {
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          gacc[c][i] += g[c][i] * f[c][i] * r;
          o[i] = r * (g[c][i] * w[col + i] - f[c][i] * cc);
        }
        *reinterpret_cast<uint4*>(dx + row * N + col) = pack8(o);
      }
    }
  }
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int col = (c * 32 + lane) * 8;
    if (col < N) {
#pragma unroll
      for (int i = 0; i < 8; ++i) sg[wi * N + col + i] = gacc[c][i];
    }
  }
  __syncthreads();
  for (int col = threadIdx.x; col < N; col += 256) {
    float t = 0.f;
#pragma unroll
    for (int r8 = 0; r8 < 8; ++r8) t += sg[r8 * N + col];
    gw_part[(long long)blockIdx.x * N + col] = t;
  }
}

}  // namespace

extern "C" int loom_slot_pool_fwd(const float* keys, const float* w9, float* pooled, float* stats, int BK, int H,
                                  cudaStream_t st) {
  slot_pool_fwd_kernel<<<BK, 256, 0, st>>>(keys, w9, pooled, stats, H);
  return (int)cudaGetLastError();
}

extern "C" int loom_slot_pool_bwd(const float* keys, const float* w9, const float* pooled, const float* stats,
                                  const float* dpooled, float* dkeys, float* dw9_part, int BK, int H, cudaStream_t st) {
  slot_pool_bwd_kernel<<<BK, 256, 0, st>>>(keys, w9, pooled, stats, dpooled, dkeys, dw9_part, H);
  return (int)cudaGetLastError();
}

#define LOOM_NCH(N, CALL)                                  \
  do {                                                     \
    const int nch_ = ((N) + 255) / 256;                    \
    if (nch_ == 1) { CALL(1); } else if (nch_ == 2) { CALL(2); } else if (nch_ == 3) { CALL(3); }                   \
    else if (nch_ == 4) { CALL(4); } else if (nch_ <= 6) { CALL(6); } else { CALL(8); }                             \
  } while (0)

extern "C" int loom_cross_attn_fwd(const void* q, const void* k, const void* v, const uint8_t* allowed, void* out, float* prob,
                                   int B, int T, int Kn, int N, float scale, cudaStream_t st) {
  if (N % 8 || N > 2048 || Kn < 1 || Kn > 1024) return -1;
  const unsigned grid = (unsigned)(((long long)B * T + 7) / 8);
  const size_t shm = (size_t)8 * Kn * sizeof(float);
#define CA_F(K) cross_attn_fwd_kernel<K><<<grid, 256, shm, st>>>((const bf16*)q, (const bf16*)k, (const bf16*)v, allowed, (bf16*)out, prob, B, T, Kn, N, scale)
  LOOM_NCH(N, CA_F);
#undef CA_F
  return (int)cudaGetLastError();
}

extern "C" int loom_cross_attn_bwd(const void* dout, const void* q, const void* k, const void* v, const float* prob, float* ds,
                                   void* dq, void* dk, void* dv, int B, int T, int Kn, int N, float scale, cudaStream_t st) {
  if (N % 8 || N > 2048 || Kn < 1 || Kn > 1024) return -1;
  const unsigned grid = (unsigned)(((long long)B * T + 7) / 8);
  const size_t shm = (size_t)8 * Kn * sizeof(float);
#define CA_B(K) cross_attn_bwd_rows_kernel<K><<<grid, 256, shm, st>>>((const bf16*)dout, (const bf16*)k, (const bf16*)v, prob, ds, (bf16*)dq, B, T, Kn, N, scale)
  LOOM_NCH(N, CA_B);
#undef CA_B
  dim3 g2(B * Kn, (N / 2 + 255) / 256);
  cross_attn_bwd_keys_kernel<<<g2, 256, 0, st>>>((const bf16*)q, (const bf16*)dout, prob, ds, (bf16*)dk, (bf16*)dv, T, Kn, N);
  return (int)cudaGetLastError();
}

template <int G>
static int fixed_rms_launch(int bwd, const void* dy, const void* x, void* out, long long rows, int heads, int HD, long long ld,
                            float target, float eps, cudaStream_t st) {
  const long long threads = rows * G;
  const unsigned grid = (unsigned)((threads + 255) / 256);
  if (bwd) fixed_rms_bwd_kernel<G><<<grid, 256, 0, st>>>((const bf16*)dy, (const bf16*)x, (bf16*)out, rows, heads, HD, ld, target, eps);
  else fixed_rms_fwd_kernel<G><<<grid, 256, 0, st>>>((const bf16*)x, (bf16*)out, rows, heads, HD, ld, target, eps);
  return (int)cudaGetLastError();
}

extern "C" int loom_fixed_rms(int bwd, const void* dy, const void* x, void* out, long long rows, int heads, int HD,
                              long long ld, float target, float eps, cudaStream_t st) {
  if (HD % 8 || HD > 128) return -1;
  const int chunks = HD / 8;
  if (chunks <= 2) return fixed_rms_launch<2>(bwd, dy, x, out, rows, heads, HD, ld, target, eps, st);
  if (chunks <= 4) return fixed_rms_launch<4>(bwd, dy, x, out, rows, heads, HD, ld, target, eps, st);
  if (chunks <= 8) return fixed_rms_launch<8>(bwd, dy, x, out, rows, heads, HD, ld, target, eps, st);
  return fixed_rms_launch<16>(bwd, dy, x, out, rows, heads, HD, ld, target, eps, st);
}

extern "C" int loom_rms_norm_fwd(const void* x, const float* w, void* y, int M, int N, float eps, cudaStream_t st) {
  if (N % 8 || N > 2048) return -1;
  const unsigned grid = (M + 7) / 8;
#define RN_F(K) rms_norm_fwd_kernel<K><<<grid, 256, 0, st>>>((const bf16*)x, w, (bf16*)y, M, N, eps)
  LOOM_NCH(N, RN_F);
#undef RN_F
  return (int)cudaGetLastError();
}

extern "C" int loom_rms_norm_bwd(const void* dy, const void* x, const float* w, void* dx, float* gw_part, int nblocks, int M,
                                 int N, float eps, cudaStream_t st) {
  if (N % 8 || N > 2048) return -1;
  const size_t shm = (size_t)8 * N * sizeof(float);
#define RN_B(K) rms_norm_bwd_kernel<K><<<nblocks, 256, shm, st>>>((const bf16*)dy, (const bf16*)x, w, (bf16*)dx, gw_part, M, N, eps)
  LOOM_NCH(N, RN_B);
#undef RN_B
  return (int)cudaGetLastError();
}
