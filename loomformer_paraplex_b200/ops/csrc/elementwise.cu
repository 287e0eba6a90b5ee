// Bandwidth-bound kernels of the fused plan: RoPE + KV-cache write, depth-attention read, residual add +
// LayerNorm, column sums, cross-entropy.  bf16 storage, fp32 math, 16-byte vector accesses.
//
// Reference counterparts: rotary embedding (loomformer.py:2983-2985), depth_attn warp kernels
// (kernels/depth_attn/depth_attn_kernel.cuh:444-651), ATen LayerNorm / cross_entropy.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include "launch_util.cuh"
#include "loom_c_api.h"

namespace {

typedef __nv_bfloat16 bf16;
typedef __nv_bfloat162 bf2;

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
__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const bf2* p = reinterpret_cast<const bf2*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) { float2 t = __bfloat1622float2(p[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 u;
  bf2* p = reinterpret_cast<bf2*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return u;
}

// ----------------------------------------------------------------------------------------------
// RoPE (rotate-half) of q and k, cache write.  One thread per (row, head, pair index).
// qkv [M, N+2KV]; cos/sin [M, HD] fp32; q_out = sector 0 of qkc [M, 3, QH, HD]; caches [B, T, KVH, HD].
// ----------------------------------------------------------------------------------------------
__global__ void rope_store_kernel(const bf16* __restrict__ qkv, const float* __restrict__ cs, const float* __restrict__ sn,
                                  bf16* __restrict__ qkc, bf16* __restrict__ kcache, bf16* __restrict__ vcache,
                                  int M, int Tc, int T, int s_off, int QH, int KVH, int HD) {
  const int half = HD / 2;
  const int heads = QH + 2 * KVH;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)M * heads * half) return;
  const int j = (int)(idx % half);
  const int hh = (int)((idx / half) % heads);
  const int m = (int)(idx / ((long long)half * heads));
  const int N = QH * HD, ld = N + 2 * KVH * HD;
  const bf16* src = qkv + (long long)m * ld + hh * HD;
  const float x1 = __bfloat162float(src[j]), x2 = __bfloat162float(src[j + half]);
  const int b = m / Tc, t = m % Tc;
  if (hh < QH + KVH) {
    const float c1 = cs[(long long)m * HD + j], c2 = cs[(long long)m * HD + j + half];
    const float s1 = sn[(long long)m * HD + j], s2 = sn[(long long)m * HD + j + half];
    const float y1 = x1 * c1 - x2 * s1, y2 = x2 * c2 + x1 * s2;
    bf16* dst = (hh < QH) ? qkc + (long long)m * 3 * N + hh * HD
                          : kcache + (((long long)b * T + s_off + t) * KVH + (hh - QH)) * HD;
    dst[j] = __float2bfloat16(y1); dst[j + half] = __float2bfloat16(y2);
  } else {
    bf16* dst = vcache + (((long long)b * T + s_off + t) * KVH + (hh - QH - KVH)) * HD;
    dst[j] = __float2bfloat16(x1); dst[j + half] = __float2bfloat16(x2);
  }
}

// Inverse rotation: dqkv = [R^T (dq_attn + dq_direct), R^T dk, dv].
// dq_attn [M,QH,HD] bf16; dq_direct = sector 0 of dqkc [M,3,QH,HD] bf16; dk/dv = fp32 cache-gradient rows.
__global__ void rope_bwd_kernel(const bf16* __restrict__ dq_attn, const bf16* __restrict__ dqkc,
                                const float* __restrict__ dkc, const float* __restrict__ dvc,
                                const float* __restrict__ cs, const float* __restrict__ sn, bf16* __restrict__ dqkv,
                                int M, int Tc, int T, int s_off, int QH, int KVH, int HD, int G) {
  const int half = HD / 2;
  const int heads = QH + 2 * KVH;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)M * heads * half) return;
  const int j = (int)(idx % half);
  const int hh = (int)((idx / half) % heads);
  const int m = (int)(idx / ((long long)half * heads));
  const int N = QH * HD, ld = N + 2 * KVH * HD;
  const int b = m / Tc, t = m % Tc;
  bf16* dst = dqkv + (long long)m * ld + hh * HD;
  float g1, g2;
  if (hh < QH) {
    const long long a = ((long long)m * QH + hh) * HD, d = (long long)m * 3 * N + hh * HD;
    g1 = __bfloat162float(dq_attn[a + j]) + __bfloat162float(dqkc[d + j]);
    g2 = __bfloat162float(dq_attn[a + j + half]) + __bfloat162float(dqkc[d + j + half]);
  } else {
    // the cache-gradient slab holds G heads per kv head (G = 1, or the GQA group size for per-query-head slabs)
    const int kh = (hh < QH + KVH) ? hh - QH : hh - QH - KVH;
    const float* src = ((hh < QH + KVH) ? dkc : dvc) + (((long long)b * T + s_off + t) * KVH * G + kh * G) * HD;
    g1 = 0.f; g2 = 0.f;
    for (int gq = 0; gq < G; ++gq) { g1 += src[gq * HD + j]; g2 += src[gq * HD + j + half]; }
  }
  if (hh < QH + KVH) {
    const float c1 = cs[(long long)m * HD + j], c2 = cs[(long long)m * HD + j + half];
    const float s1 = sn[(long long)m * HD + j], s2 = sn[(long long)m * HD + j + half];
    // forward: y1 = x1 c1 - x2 s1 ; y2 = x2 c2 + x1 s2
    dst[j] = __float2bfloat16(g1 * c1 + g2 * s2);
    dst[j + half] = __float2bfloat16(g2 * c2 - g1 * s1);
  } else {
    dst[j] = __float2bfloat16(g1); dst[j + half] = __float2bfloat16(g2);
  }
}

// ---- four pairs per thread (HD a multiple of 8): 8- and 16-byte accesses instead of 2- and 4-byte ones -------------
__device__ __forceinline__ void ld4(const bf16* p, float (&f)[4]) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
  const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}
__device__ __forceinline__ void st4(bf16* p, const float (&f)[4]) {
  uint2 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
  h[0] = __floats2bfloat162_rn(f[0], f[1]);
  h[1] = __floats2bfloat162_rn(f[2], f[3]);
  *reinterpret_cast<uint2*>(p) = u;
}
__device__ __forceinline__ void ldf4(const float* p, float (&f)[4]) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
}

__global__ void rope_store_v4_kernel(const bf16* __restrict__ qkv, const float* __restrict__ cs, const float* __restrict__ sn,
                                     bf16* __restrict__ qkc, bf16* __restrict__ kcache, bf16* __restrict__ vcache,
                                     int M, int Tc, int T, int s_off, int QH, int KVH, int HD) {
  const int half = HD / 2, q4 = half / 4;
  const int heads = QH + 2 * KVH;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)M * heads * q4) return;
  const int j = (int)(idx % q4) * 4;
  const int hh = (int)((idx / q4) % heads);
  const int m = (int)(idx / ((long long)q4 * heads));
  const int N = QH * HD, ld = N + 2 * KVH * HD;
  const bf16* src = qkv + (long long)m * ld + hh * HD;
  float x1[4], x2[4];
  ld4(src + j, x1); ld4(src + j + half, x2);
  const int b = m / Tc, t = m % Tc;
  bf16* dst;
  if (hh < QH + KVH) {
    float c1[4], c2[4], s1[4], s2[4];
    ldf4(cs + (long long)m * HD + j, c1); ldf4(cs + (long long)m * HD + j + half, c2);
    ldf4(sn + (long long)m * HD + j, s1); ldf4(sn + (long long)m * HD + j + half, s2);
    float y1[4], y2[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) { y1[i] = x1[i] * c1[i] - x2[i] * s1[i]; y2[i] = x2[i] * c2[i] + x1[i] * s2[i]; }
    dst = (hh < QH) ? qkc + (long long)m * 3 * N + hh * HD
                    : kcache + (((long long)b * T + s_off + t) * KVH + (hh - QH)) * HD;
    st4(dst + j, y1); st4(dst + j + half, y2);
  } else {
    dst = vcache + (((long long)b * T + s_off + t) * KVH + (hh - QH - KVH)) * HD;
    st4(dst + j, x1); st4(dst + j + half, x2);
  }
}

__global__ void rope_bwd_v4_kernel(const bf16* __restrict__ dq_attn, const bf16* __restrict__ dqkc,
                                   const float* __restrict__ dkc, const float* __restrict__ dvc,
                                   const float* __restrict__ cs, const float* __restrict__ sn, bf16* __restrict__ dqkv,
                                   int M, int Tc, int T, int s_off, int QH, int KVH, int HD, int G) {
  const int half = HD / 2, q4 = half / 4;
  const int heads = QH + 2 * KVH;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)M * heads * q4) return;
  const int j = (int)(idx % q4) * 4;
  const int hh = (int)((idx / q4) % heads);
  const int m = (int)(idx / ((long long)q4 * heads));
  const int N = QH * HD, ld = N + 2 * KVH * HD;
  const int b = m / Tc, t = m % Tc;
  bf16* dst = dqkv + (long long)m * ld + hh * HD;
  float g1[4], g2[4];
  if (hh < QH) {
    const long long a = ((long long)m * QH + hh) * HD, d = (long long)m * 3 * N + hh * HD;
    float e1[4], e2[4];
    ld4(dq_attn + a + j, g1); ld4(dq_attn + a + j + half, g2);
    ld4(dqkc + d + j, e1); ld4(dqkc + d + j + half, e2);
#pragma unroll
    for (int i = 0; i < 4; ++i) { g1[i] += e1[i]; g2[i] += e2[i]; }
  } else {
    const int kh = (hh < QH + KVH) ? hh - QH : hh - QH - KVH;
    const float* src = ((hh < QH + KVH) ? dkc : dvc) + (((long long)b * T + s_off + t) * KVH * G + kh * G) * HD;
#pragma unroll
    for (int i = 0; i < 4; ++i) { g1[i] = 0.f; g2[i] = 0.f; }
    for (int gq = 0; gq < G; ++gq) {
      float e1[4], e2[4];
      ldf4(src + gq * HD + j, e1); ldf4(src + gq * HD + j + half, e2);
#pragma unroll
      for (int i = 0; i < 4; ++i) { g1[i] += e1[i]; g2[i] += e2[i]; }
    }
  }
  if (hh < QH + KVH) {
    float c1[4], c2[4], s1[4], s2[4];
    ldf4(cs + (long long)m * HD + j, c1); ldf4(cs + (long long)m * HD + j + half, c2);
    ldf4(sn + (long long)m * HD + j, s1); ldf4(sn + (long long)m * HD + j + half, s2);
    float o1[4], o2[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) { o1[i] = g1[i] * c1[i] + g2[i] * s2[i]; o2[i] = g2[i] * c2[i] - g1[i] * s1[i]; }
    st4(dst + j, o1); st4(dst + j + half, o2);
  } else {
    st4(dst + j, g1); st4(dst + j + half, g2);
  }
}

// [M, QH, 3, HD] -> [M, 3, QH, HD]: the three attention sectors of a head leave the batched data-gradient GEMM side by
// side; the attention backward reads them sector-major.  16 bytes per thread on both sides.
__global__ void sector_fold_kernel(const bf16* __restrict__ src, bf16* __restrict__ dst, long long M, int QH, int HD) {
  const int c8n = HD / 8;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= M * QH * 3 * c8n) return;
  const int c8 = (int)(idx % c8n);
  const int s = (int)((idx / c8n) % 3);
  const int g = (int)((idx / (3LL * c8n)) % QH);
  const long long m = idx / (3LL * c8n * QH);
  *reinterpret_cast<uint4*>(dst + ((m * 3 + s) * QH + g) * HD + c8 * 8) = *reinterpret_cast<const uint4*>(src + idx * 8);
}

// Backward of the RMS cap y = s a, s = min(1, cap / rms(a)):  da = dy where the row is not clipped, else
// da = s (dy - a <a, dy> / (N (mean(a^2) + 1e-6))).  One warp per row.
template <int NCH>
__global__ void __launch_bounds__(256) cap_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ a,
                                                      bf16* __restrict__ da, int M, int N, float cap) {
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= M) return;
  float fa[NCH][8], g[NCH][8], q = 0.f, dot = 0.f;
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int col = (lane + 32 * c) * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) { fa[c][i] = 0.f; g[c][i] = 0.f; }
    if (col < N) {
      unpack8(*reinterpret_cast<const uint4*>(a + (long long)row * N + col), fa[c]);
      unpack8(*reinterpret_cast<const uint4*>(dy + (long long)row * N + col), g[c]);
#pragma unroll
      for (int i = 0; i < 8; ++i) { q += fa[c][i] * fa[c][i]; dot += fa[c][i] * g[c][i]; }
    }
  }
  const float ms = warp_sum(q) / N + 1e-6f;
  dot = warp_sum(dot);
  const float s = cap * rsqrtf(ms);
  const bool clipped = s < 1.f;
  const float k = clipped ? dot / (N * ms) : 0.f;
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int col = (lane + 32 * c) * 8;
    if (col < N) {
      float o[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = clipped ? s * (g[c][i] - fa[c][i] * k) : g[c][i];
      *reinterpret_cast<uint4*>(da + (long long)row * N + col) = pack8(o);
    }
  }
}

// ----------------------------------------------------------------------------------------------
// Depth-attention read.  G lanes (G = power of two >= HD/8) own one (row, head); each lane holds 8 dims.
// hist_k / hist_v: [S, M, QH, HD] bf16;  q: [QH, HD] fp32;  out: [M, QH, HD] bf16;  lse: [M, QH] fp32.
// ----------------------------------------------------------------------------------------------
template <int G>
__global__ void __launch_bounds__(256) dread_fwd_kernel(const float* __restrict__ q, const bf16* __restrict__ hk,
                                                        const bf16* __restrict__ hv, bf16* __restrict__ out,
                                                        float* __restrict__ lse, int n, long long MQ, int QH, int HD,
                                                        float scale, long long slot_stride, long long row_stride) {
  // history element (slot s, row r, head g, dim c) lives at s * slot_stride + r * row_stride + g * HD + c, which lets
  // K and V share one buffer whose rows are the [K | V] rows the projection GEMM writes
  if (MQ <= 4096) loom::pdl_trigger();        // decode-sized problem: a dependent launched programmatically may start its prologue now
  const long long gid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) / G;
  const int l = threadIdx.x % G;
  if (gid >= MQ) return;                    // whole G-lane groups leave together
  const unsigned mask = __activemask();
  const int g = (int)(gid % QH);
  const bool act = l * 8 < HD;
  float qv[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) qv[i] = act ? q[g * HD + l * 8 + i] * scale : 0.f;
  const long long base = gid * HD + l * 8;
  const long long hbase = (gid / QH) * row_stride + (long long)g * HD + l * 8;
  float mx = -INFINITY, den = 0.f, acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  // the softmax over slots is one dependent chain per slot; issue the K/V loads of PF slots together so their
  // latencies overlap instead of adding up
  constexpr int PF = 4;
  for (int s0 = 0; s0 < n; s0 += PF) {
    uint4 rk[PF], rv[PF];
#pragma unroll
    for (int u = 0; u < PF; ++u) {
      const int s = (s0 + u < n) ? s0 + u : n - 1;
      rk[u] = make_uint4(0u, 0u, 0u, 0u); rv[u] = rk[u];
      if (act) {
        rk[u] = *reinterpret_cast<const uint4*>(hk + s * slot_stride + hbase);
        rv[u] = *reinterpret_cast<const uint4*>(hv + s * slot_stride + hbase);
      }
    }
#pragma unroll
    for (int u = 0; u < PF; ++u) {
      if (s0 + u < n) {
        float kf[8], vf[8];
        unpack8(rk[u], kf); unpack8(rv[u], vf);
        float d = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) d += qv[i] * kf[i];
#pragma unroll
        for (int o = G / 2; o > 0; o >>= 1) d += __shfl_xor_sync(mask, d, o, G);
        const float nm = fmaxf(mx, d);
        const float corr = __expf(mx - nm), p = __expf(d - nm);
        den = den * corr + p;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = acc[i] * corr + p * vf[i];
        mx = nm;
      }
    }
  }
  const float inv = 1.f / den;
  if (act) {
    float o8[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) o8[i] = acc[i] * inv;
    *reinterpret_cast<uint4*>(out + base) = pack8(o8);
  }
  if (l == 0) lse[gid] = mx + __logf(den);
}

// The same read with G * 4 NV == HD exactly: a lane owns NV vectors of four dims (12 dims of a 96-wide head on 8 lanes
// instead of 8 dims on 16 lanes of which 4 idle), so a warp serves four (row, head) pairs instead of two and the
// per-slot chain (reduce, two exponentials) is shared by half again as many dims.
__device__ __forceinline__ void unpack4(const uint2& u, float* f) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
  const float2 a = __bfloat1622float2(p[0]), b = __bfloat1622float2(p[1]);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}
template <int G, int NV>
__global__ void __launch_bounds__(256) dread_fwd_wide_kernel(const float* __restrict__ q, const bf16* __restrict__ hk,
                                                             const bf16* __restrict__ hv, bf16* __restrict__ out,
                                                             float* __restrict__ lse, int n, long long MQ, int QH, int HD,
                                                             float scale, long long slot_stride, long long row_stride) {
  constexpr int DPL = 4 * NV;
  loom::pdl_wait();                           // returns at once unless launched programmatically dependent (decode-sized problems)
  if (MQ <= 4096) loom::pdl_trigger();        // decode-sized problem: a dependent launched programmatically may start its prologue now
  const long long gid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) / G;
  const int l = threadIdx.x % G;
  if (gid >= MQ) return;                    // whole G-lane groups leave together
  const unsigned mask = __activemask();
  const int g = (int)(gid % QH);
  float qv[DPL];
#pragma unroll
  for (int i = 0; i < DPL; ++i) qv[i] = q[g * HD + l * DPL + i] * scale;
  const long long base = gid * HD + l * DPL;
  const long long hbase = (gid / QH) * row_stride + (long long)g * HD + l * DPL;
  float mx = -INFINITY, den = 0.f, acc[DPL];
#pragma unroll
  for (int i = 0; i < DPL; ++i) acc[i] = 0.f;
  constexpr int PF = NV <= 3 ? 8 : 4;         // slots whose loads are in flight together (one memory round trip each)
  for (int s0 = 0; s0 < n; s0 += PF) {
    uint2 rk[PF][NV], rv[PF][NV];
#pragma unroll
    for (int u = 0; u < PF; ++u) {
      const int s = (s0 + u < n) ? s0 + u : n - 1;
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        rk[u][v] = *reinterpret_cast<const uint2*>(hk + s * slot_stride + hbase + 4 * v);
        rv[u][v] = *reinterpret_cast<const uint2*>(hv + s * slot_stride + hbase + 4 * v);
      }
    }
#pragma unroll
    for (int u = 0; u < PF; ++u) {
      if (s0 + u < n) {
        float kf[DPL], vf[DPL];
#pragma unroll
        for (int v = 0; v < NV; ++v) { unpack4(rk[u][v], kf + 4 * v); unpack4(rv[u][v], vf + 4 * v); }
        float d = 0.f;
#pragma unroll
        for (int i = 0; i < DPL; ++i) d += qv[i] * kf[i];
#pragma unroll
        for (int o = G / 2; o > 0; o >>= 1) d += __shfl_xor_sync(mask, d, o, G);
        const float nm = fmaxf(mx, d);
        const float corr = __expf(mx - nm), p = __expf(d - nm);
        den = den * corr + p;
#pragma unroll
        for (int i = 0; i < DPL; ++i) acc[i] = acc[i] * corr + p * vf[i];
        mx = nm;
      }
    }
  }
  const float inv = 1.f / den;
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    uint2 o;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
    o2[0] = __floats2bfloat162_rn(acc[4 * v] * inv, acc[4 * v + 1] * inv);
    o2[1] = __floats2bfloat162_rn(acc[4 * v + 2] * inv, acc[4 * v + 3] * inv);
    *reinterpret_cast<uint2*>(out + base + 4 * v) = o;
  }
  if (l == 0) lse[gid] = mx + __logf(den);
}

// Backward: dhv[s] += w_s dm ; dhk[s] += dsc_s q/sqrt(HD) ; gq partial sums -> atomics per block.
template <int G>
__global__ void __launch_bounds__(256) dread_bwd_kernel(const float* __restrict__ q, const bf16* __restrict__ hk,
                                                        const bf16* __restrict__ hv, const bf16* __restrict__ dm,
                                                        const bf16* __restrict__ mo, const float* __restrict__ lse,
                                                        float* __restrict__ dhk, float* __restrict__ dhv,
                                                        float* __restrict__ gq, int n, long long MQ, int QH, int HD,
                                                        float scale) {
  extern __shared__ float sh_gq[];           // [QH*HD]
  for (int i = threadIdx.x; i < QH * HD; i += blockDim.x) sh_gq[i] = 0.f;
  __syncthreads();
  const long long gid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) / G;
  const int l = threadIdx.x % G;
  if (gid < MQ) {
    const unsigned mask = __activemask();
    const int g = (int)(gid % QH);
    const bool act = l * 8 < HD;
    float qv[8], dmf[8], mf[8], gql[8];
    const long long stride = MQ * HD, base = gid * HD + l * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) { qv[i] = act ? q[g * HD + l * 8 + i] : 0.f; gql[i] = 0.f; dmf[i] = 0.f; mf[i] = 0.f; }
    if (act) {
      unpack8(*reinterpret_cast<const uint4*>(dm + base), dmf);
      unpack8(*reinterpret_cast<const uint4*>(mo + base), mf);
    }
    float dd = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) dd += dmf[i] * mf[i];
#pragma unroll
    for (int o = G / 2; o > 0; o >>= 1) dd += __shfl_xor_sync(mask, dd, o, G);
    const float L = lse[gid];
    for (int s = 0; s < n; ++s) {
      float kf[8], vf[8];
      if (act) {
        unpack8(*reinterpret_cast<const uint4*>(hk + s * stride + base), kf);
        unpack8(*reinterpret_cast<const uint4*>(hv + s * stride + base), vf);
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) { kf[i] = 0.f; vf[i] = 0.f; }
      }
      float d = 0.f, dv = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) { d += qv[i] * kf[i]; dv += dmf[i] * vf[i]; }
#pragma unroll
      for (int o = G / 2; o > 0; o >>= 1) {
        d += __shfl_xor_sync(mask, d, o, G);
        dv += __shfl_xor_sync(mask, dv, o, G);
      }
      const float w = __expf(d * scale - L);
      const float dsc = w * (dv - dd) * scale;
      if (act) {
        float* pk = dhk + s * stride + base;
        float* pv = dhv + s * stride + base;
#pragma unroll
        for (int i = 0; i < 8; i += 4) {
          float4 a = *reinterpret_cast<float4*>(pk + i), b = *reinterpret_cast<float4*>(pv + i);
          a.x += dsc * qv[i]; a.y += dsc * qv[i + 1]; a.z += dsc * qv[i + 2]; a.w += dsc * qv[i + 3];
          b.x += w * dmf[i]; b.y += w * dmf[i + 1]; b.z += w * dmf[i + 2]; b.w += w * dmf[i + 3];
          *reinterpret_cast<float4*>(pk + i) = a; *reinterpret_cast<float4*>(pv + i) = b;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) gql[i] += dsc * kf[i];
      }
    }
    if (act) {
#pragma unroll
      for (int i = 0; i < 8; ++i) atomicAdd(&sh_gq[g * HD + l * 8 + i], gql[i]);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < QH * HD; i += blockDim.x) {
    const float v = sh_gq[i];
    if (v != 0.f) atomicAdd(gq + i, v);
  }
}


// ----------------------------------------------------------------------------------------------
// y = LayerNorm(a + b) * w + bias.  One warp per row, NCH 16-byte chunks per lane (N <= 256*NCH).
// The pre-norm sum is rounded to bf16 first (it is what the backward pass re-reads).
// ----------------------------------------------------------------------------------------------
// cap > 0: each addend is first shrunk to an RMS of at most `cap` (never amplified): x = s_a a + s_b b with
// s = min(1, cap / sqrt(mean(.^2) + 1e-6)).
template <int NCH>
__global__ void __launch_bounds__(256) add_ln_fwd_kernel(const bf16* __restrict__ a, const bf16* __restrict__ b,
                                                         const float* __restrict__ w, const float* __restrict__ bias,
                                                         bf16* __restrict__ y, bf16* __restrict__ x,
                                                         float* __restrict__ mean, float* __restrict__ rstd, int M, int N,
                                                         float eps, float cap) {
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= M) return;
  float v[NCH][8];
  float sum = 0.f;
  float sa = 1.f, sb = 1.f;
  if (cap > 0.f) {
    float qa = 0.f, qb = 0.f;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const int col = (lane + 32 * c) * 8;
      if (col < N) {
        float fa[8], fb[8];
        unpack8(*reinterpret_cast<const uint4*>(a + (long long)row * N + col), fa);
        unpack8(*reinterpret_cast<const uint4*>(b + (long long)row * N + col), fb);
#pragma unroll
        for (int i = 0; i < 8; ++i) { qa += fa[i] * fa[i]; qb += fb[i] * fb[i]; }
      }
    }
    sa = fminf(1.f, cap * rsqrtf(warp_sum(qa) / N + 1e-6f));
    sb = fminf(1.f, cap * rsqrtf(warp_sum(qb) / N + 1e-6f));
  }
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int col = (lane + 32 * c) * 8;
    if (col < N) {
      float fa[8], fb[8];
      unpack8(*reinterpret_cast<const uint4*>(a + (long long)row * N + col), fa);
      unpack8(*reinterpret_cast<const uint4*>(b + (long long)row * N + col), fb);
#pragma unroll
      for (int i = 0; i < 8; ++i) fa[i] = sa * fa[i] + sb * fb[i];
      const uint4 packed = pack8(fa);
      *reinterpret_cast<uint4*>(x + (long long)row * N + col) = packed;
      unpack8(packed, v[c]);
#pragma unroll
      for (int i = 0; i < 8; ++i) sum += v[c][i];
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[c][i] = 0.f;
    }
  }
  const float mu = warp_sum(sum) / N;
  float var = 0.f;
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int col = (lane + 32 * c) * 8;
    if (col < N) {
#pragma unroll
      for (int i = 0; i < 8; ++i) { const float d = v[c][i] - mu; var += d * d; }
    }
  }
  const float rs = rsqrtf(warp_sum(var) / N + eps);
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int col = (lane + 32 * c) * 8;
    if (col < N) {
      float o[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = (v[c][i] - mu) * rs * w[col + i] + bias[col + i];
      *reinterpret_cast<uint4*>(y + (long long)row * N + col) = pack8(o);
    }
  }
  if (lane == 0) { mean[row] = mu; rstd[row] = rs; }
}

// dx = rstd * (g w - mean(g w) - xhat mean(g w xhat));  gw += sum_rows g xhat;  gb += sum_rows g.
template <int NCH>
__global__ void __launch_bounds__(256) add_ln_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x,
                                                         const float* __restrict__ mean, const float* __restrict__ rstd,
                                                         const float* __restrict__ w, bf16* __restrict__ dx,
                                                         float* __restrict__ gw, float* __restrict__ gb, int M, int N) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float aw[NCH][8], ab[NCH][8];
#pragma unroll
  for (int c = 0; c < NCH; ++c)
#pragma unroll
    for (int i = 0; i < 8; ++i) { aw[c][i] = 0.f; ab[c][i] = 0.f; }
  for (int row = blockIdx.x * 8 + warp; row < M; row += gridDim.x * 8) {
    const float mu = mean[row], rs = rstd[row];
    float g[NCH][8], xh[NCH][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const int col = (lane + 32 * c) * 8;
      if (col < N) {
        float xf[8];
        unpack8(*reinterpret_cast<const uint4*>(dy + (long long)row * N + col), g[c]);
        unpack8(*reinterpret_cast<const uint4*>(x + (long long)row * N + col), xf);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          xh[c][i] = (xf[i] - mu) * rs;
          aw[c][i] += g[c][i] * xh[c][i];
          ab[c][i] += g[c][i];
          g[c][i] *= w[col + i];
          s1 += g[c][i];
          s2 += g[c][i] * xh[c][i];
        }
      }
    }
    s1 = warp_sum(s1) / N;
    s2 = warp_sum(s2) / N;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const int col = (lane + 32 * c) * 8;
      if (col < N) {
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = rs * (g[c][i] - s1 - xh[c][i] * s2);
        *reinterpret_cast<uint4*>(dx + (long long)row * N + col) = pack8(o);
      }
    }
  }
  // reduce the 8 warps of the block through shared memory, then one atomic per column
  extern __shared__ float shm[];     // [2][8][N]
  float* sw = shm;
  float* sb = shm + 8 * N;
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int col = (lane + 32 * c) * 8;
    if (col < N) {
#pragma unroll
      for (int i = 0; i < 8; ++i) { sw[warp * N + col + i] = aw[c][i]; sb[warp * N + col + i] = ab[c][i]; }
    }
  }
  __syncthreads();
  for (int col = threadIdx.x; col < N; col += blockDim.x) {
    float tw = 0.f, tb = 0.f;
#pragma unroll
    for (int r = 0; r < 8; ++r) { tw += sw[r * N + col]; tb += sb[r * N + col]; }
    atomicAdd(gw + col, tw);
    atomicAdd(gb + col, tb);
  }
}

// gb[n] += sum_m dy[m, n]
__global__ void __launch_bounds__(256) colsum_kernel(const bf16* __restrict__ dy, float* __restrict__ gb, int M, int N,
                                                     long long ld) {
  const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;
  const int col = (blockIdx.x * 64 + tx) * 2;
  float a0 = 0.f, a1 = 0.f;
  if (col < N) {
    for (int r = blockIdx.y * 64 + ty; r < min(M, (int)(blockIdx.y + 1) * 64); r += 4) {
      const float2 v = __bfloat1622float2(*reinterpret_cast<const bf2*>(dy + (long long)r * ld + col));
      a0 += v.x; a1 += v.y;
    }
  }
  __shared__ float sh[2][4][64];
  sh[0][ty][tx] = a0; sh[1][ty][tx] = a1;
  __syncthreads();
  if (ty == 0 && col < N) {
    float t0 = 0.f, t1 = 0.f;
#pragma unroll
    for (int r = 0; r < 4; ++r) { t0 += sh[0][r][tx]; t1 += sh[1][r][tx]; }
    atomicAdd(gb + col, t0);
    if (col + 1 < N) atomicAdd(gb + col + 1, t1);
  }
}

// ----------------------------------------------------------------------------------------------
// Cross-entropy over bf16 logits, one block per row: nll[row] and (optionally) in-place
// d logits = (softmax - onehot) * scale, scale read from device memory (grad_scale / #valid targets).
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ float block_reduce(float v, float* sh, bool is_max) {
  v = is_max ? warp_max(v) : warp_sum(v);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) sh[w] = v;
  __syncthreads();
  float r = (threadIdx.x < (blockDim.x >> 5)) ? sh[threadIdx.x] : (is_max ? -INFINITY : 0.f);
  if (w == 0) r = is_max ? warp_max(r) : warp_sum(r);
  if (threadIdx.x == 0) sh[32] = r;
  __syncthreads();
  return sh[32];
}

__global__ void __launch_bounds__(256) ce_kernel(bf16* __restrict__ logits, const long long* __restrict__ targets,
                                                 float* __restrict__ nll, const float* __restrict__ scale_ptr, int V,
                                                 long long ignore_index, int write_grad) {
  __shared__ float sh[33];
  const long long row = blockIdx.x;
  bf16* L = logits + row * V;
  const long long tgt = targets[row];
  const bool valid = tgt != ignore_index;
  // the target's logit is read here, before the block's first barrier: the gradient pass below overwrites the row in
  // place, and other warps may reach it while thread 0 is still forming the loss
  const float tgt_logit = (threadIdx.x == 0 && valid) ? __bfloat162float(L[tgt]) : 0.f;
  float mx = -INFINITY;
  for (int c = threadIdx.x * 8; c < V; c += blockDim.x * 8) {
    float f[8];
    unpack8(*reinterpret_cast<const uint4*>(L + c), f);
#pragma unroll
    for (int i = 0; i < 8; ++i) mx = fmaxf(mx, f[i]);
  }
  mx = block_reduce(mx, sh, true);
  float se = 0.f;
  for (int c = threadIdx.x * 8; c < V; c += blockDim.x * 8) {
    float f[8];
    unpack8(*reinterpret_cast<const uint4*>(L + c), f);
#pragma unroll
    for (int i = 0; i < 8; ++i) se += __expf(f[i] - mx);
  }
  se = block_reduce(se, sh, false);
  const float lse = mx + __logf(se);
  if (threadIdx.x == 0) nll[row] = valid ? lse - tgt_logit : 0.f;
  if (!write_grad) return;
  const float sc = valid ? *scale_ptr : 0.f;
  const float inv = 1.f / se;
  for (int c = threadIdx.x * 8; c < V; c += blockDim.x * 8) {
    float f[8];
    unpack8(*reinterpret_cast<const uint4*>(L + c), f);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float p = __expf(f[i] - mx) * inv;
      if (valid && c + i == tgt) p -= 1.f;
      f[i] = p * sc;
    }
    *reinterpret_cast<uint4*>(L + c) = pack8(f);
  }
}


// Few rows (a decode step): one block per row instead of one warp, so a single row is spread over 8 warps' worth of
// loads in flight.  Same arithmetic as add_ln_fwd_kernel; two values are reduced per block reduction.
__device__ __forceinline__ float2 block_sum2(float2 v, float2* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    v.x += __shfl_xor_sync(0xffffffffu, v.x, o);
    v.y += __shfl_xor_sync(0xffffffffu, v.y, o);
  }
  const int w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  __syncthreads();
  if ((threadIdx.x & 31) == 0) sh[w] = v;
  __syncthreads();
  float2 r = sh[0];
  for (int i = 1; i < nw; ++i) { r.x += sh[i].x; r.y += sh[i].y; }
  return r;
}

__global__ void __launch_bounds__(256) add_ln_fwd_row_kernel(const bf16* __restrict__ a, const bf16* __restrict__ b,
                                                             const float* __restrict__ w, const float* __restrict__ bias,
                                                             bf16* __restrict__ y, bf16* __restrict__ x,
                                                             float* __restrict__ mean, float* __restrict__ rstd, int N,
                                                             float eps, float cap) {
  __shared__ float2 sh[8];
  loom::pdl_wait();
  loom::pdl_trigger();
  const int row = blockIdx.x;
  const int col = threadIdx.x * 8;
  const bool on = col < N;
  float fa[8], fb[8], v[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) { fa[i] = 0.f; fb[i] = 0.f; v[i] = 0.f; }
  if (on) {
    unpack8(*reinterpret_cast<const uint4*>(a + (long long)row * N + col), fa);
    unpack8(*reinterpret_cast<const uint4*>(b + (long long)row * N + col), fb);
  }
  float sa = 1.f, sb = 1.f;
  if (cap > 0.f) {
    float2 q = make_float2(0.f, 0.f);
#pragma unroll
    for (int i = 0; i < 8; ++i) { q.x += fa[i] * fa[i]; q.y += fb[i] * fb[i]; }
    q = block_sum2(q, sh);
    sa = fminf(1.f, cap * rsqrtf(q.x / N + 1e-6f));
    sb = fminf(1.f, cap * rsqrtf(q.y / N + 1e-6f));
  }
  float2 s1 = make_float2(0.f, 0.f);
  if (on) {
#pragma unroll
    for (int i = 0; i < 8; ++i) fa[i] = sa * fa[i] + sb * fb[i];
    const uint4 packed = pack8(fa);
    *reinterpret_cast<uint4*>(x + (long long)row * N + col) = packed;
    unpack8(packed, v);
#pragma unroll
    for (int i = 0; i < 8; ++i) s1.x += v[i];
  }
  const float mu = block_sum2(s1, sh).x / N;
  float2 s2 = make_float2(0.f, 0.f);
  if (on) {
#pragma unroll
    for (int i = 0; i < 8; ++i) { const float d = v[i] - mu; s2.x += d * d; }
  }
  const float rs = rsqrtf(block_sum2(s2, sh).x / N + eps);
  if (on) {
    float o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = (v[i] - mu) * rs * w[col + i] + bias[col + i];
    *reinterpret_cast<uint4*>(y + (long long)row * N + col) = pack8(o);
  }
  if (threadIdx.x == 0) { mean[row] = mu; rstd[row] = rs; }
}

}  // namespace

extern "C" int loom_rope_store(const void* qkv, const float* cs, const float* sn, void* qkc, void* kcache, void* vcache,
                               int M, int Tc, int T, int s_off, int QH, int KVH, int HD, cudaStream_t st) {
  if (HD % 8 == 0) {
    const long long n4 = (long long)M * (QH + 2 * KVH) * (HD / 8);
    rope_store_v4_kernel<<<(unsigned)((n4 + 255) / 256), 256, 0, st>>>((const bf16*)qkv, cs, sn, (bf16*)qkc, (bf16*)kcache,
                                                                        (bf16*)vcache, M, Tc, T, s_off, QH, KVH, HD);
    return (int)cudaGetLastError();
  }
  const long long n = (long long)M * (QH + 2 * KVH) * (HD / 2);
  rope_store_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>((const bf16*)qkv, cs, sn, (bf16*)qkc, (bf16*)kcache,
                                                                 (bf16*)vcache, M, Tc, T, s_off, QH, KVH, HD);
  return (int)cudaGetLastError();
}

extern "C" int loom_sector_fold(const void* src, void* dst, long long M, int QH, int HD, cudaStream_t st) {
  if (HD % 8 || M < 1 || QH < 1 || (reinterpret_cast<uintptr_t>(src) & 15) || (reinterpret_cast<uintptr_t>(dst) & 15)) return -1;
  const long long n = M * QH * 3 * (HD / 8);
  sector_fold_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>((const bf16*)src, (bf16*)dst, M, QH, HD);
  return (int)cudaGetLastError();
}

extern "C" int loom_rope_bwd(const void* dq_attn, const void* dqkc, const float* dkc, const float* dvc, const float* cs,
                             const float* sn, void* dqkv, int M, int Tc, int T, int s_off, int QH, int KVH, int HD,
                             int G, cudaStream_t st) {
  if (HD % 8 == 0) {
    const long long n4 = (long long)M * (QH + 2 * KVH) * (HD / 8);
    rope_bwd_v4_kernel<<<(unsigned)((n4 + 255) / 256), 256, 0, st>>>((const bf16*)dq_attn, (const bf16*)dqkc, dkc, dvc, cs, sn,
                                                                      (bf16*)dqkv, M, Tc, T, s_off, QH, KVH, HD, G);
    return (int)cudaGetLastError();
  }
  const long long n = (long long)M * (QH + 2 * KVH) * (HD / 2);
  rope_bwd_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>((const bf16*)dq_attn, (const bf16*)dqkc, dkc, dvc, cs, sn,
                                                               (bf16*)dqkv, M, Tc, T, s_off, QH, KVH, HD, G);
  return (int)cudaGetLastError();
}

template <int G>
static int dread_launch(int bwd, const float* q, const void* hk, const void* hv, void* out, float* lse, const void* dm,
                        float* dhk, float* dhv, float* gq, int n, long long MQ, int QH, int HD, long long slot_stride,
                        long long row_stride, cudaStream_t st) {
  const float scale = rsqrtf((float)HD);
  const long long threads = MQ * G;
  const unsigned grid = (unsigned)((threads + 255) / 256);
  if (!bwd) {
    dread_fwd_kernel<G><<<grid, 256, 0, st>>>(q, (const bf16*)hk, (const bf16*)hv, (bf16*)out, lse, n, MQ, QH, HD, scale,
                                              slot_stride, row_stride);
  } else {
    dread_bwd_kernel<G><<<grid, 256, QH * HD * sizeof(float), st>>>(q, (const bf16*)hk, (const bf16*)hv, (const bf16*)dm,
                                                                    (const bf16*)out, lse, dhk, dhv, gq, n, MQ, QH, HD, scale);
  }
  return (int)cudaGetLastError();
}

extern "C" int loom_dread(int bwd, const float* q, const void* hk, const void* hv, void* out, float* lse, const void* dm,
                          float* dhk, float* dhv, float* gq, int n, long long MQ, int QH, int HD, long long slot_stride,
                          long long row_stride, cudaStream_t st) {
  if (HD % 8 || HD > 128) return -1;
  if (slot_stride <= 0) { slot_stride = MQ * HD; row_stride = (long long)QH * HD; }     // densely packed history
  if (slot_stride % 8 || row_stride % 8) return -1;                                    // 16-byte vector loads
  if (bwd && (slot_stride != MQ * HD || row_stride != (long long)QH * HD)) return -1;   // the legacy backward is dense-only
  if (!bwd) {
    // head widths that split exactly into 8 / 4 / 2 lanes of 8, 12 or 16 dims (LOOM_DREAD_FWD=narrow keeps 8 dims per lane)
    static int narrow = -1;
    if (narrow < 0) { const char* e = getenv("LOOM_DREAD_FWD"); narrow = (e != nullptr && e[0] == 'n') ? 1 : 0; }
    const float scale = rsqrtf((float)HD);
#define WIDE_F(G_, NV_) do { const long long threads = MQ * G_; \
      if (MQ <= 256) return (int)loom::launch_pdl(dread_fwd_wide_kernel<G_, NV_>, dim3((unsigned)((threads + 255) / 256)), dim3(256), 0, st, q, \
                                                   (const bf16*)hk, (const bf16*)hv, (bf16*)out, lse, n, MQ, QH, HD, scale, slot_stride, row_stride); \
      dread_fwd_wide_kernel<G_, NV_><<<(unsigned)((threads + 255) / 256), 256, 0, st>>>(q, (const bf16*)hk, (const bf16*)hv, (bf16*)out, lse, \
                                                                                       n, MQ, QH, HD, scale, slot_stride, row_stride); \
      return (int)cudaGetLastError(); } while (0)
    if (!narrow) {
      if (HD == 96) WIDE_F(8, 3); if (HD == 64) WIDE_F(8, 2); if (HD == 128) WIDE_F(8, 4); if (HD == 48) WIDE_F(4, 3);
      if (HD == 32) WIDE_F(4, 2); if (HD == 24) WIDE_F(2, 3);
    }
#undef WIDE_F
  }
  const int chunks = HD / 8;
  if (chunks <= 2) return dread_launch<2>(bwd, q, hk, hv, out, lse, dm, dhk, dhv, gq, n, MQ, QH, HD, slot_stride, row_stride, st);
  if (chunks <= 4) return dread_launch<4>(bwd, q, hk, hv, out, lse, dm, dhk, dhv, gq, n, MQ, QH, HD, slot_stride, row_stride, st);
  if (chunks <= 8) return dread_launch<8>(bwd, q, hk, hv, out, lse, dm, dhk, dhv, gq, n, MQ, QH, HD, slot_stride, row_stride, st);
  return dread_launch<16>(bwd, q, hk, hv, out, lse, dm, dhk, dhv, gq, n, MQ, QH, HD, slot_stride, row_stride, st);
}

extern "C" int loom_cap_bwd(const void* dy, const void* a, void* da, int M, int N, float cap, cudaStream_t st) {
  if (N % 8 || N > 2048) return -1;
  const unsigned grid = (M + 7) / 8;
  const int nch = (N + 255) / 256;
#define CAP_B(K) cap_bwd_kernel<K><<<grid, 256, 0, st>>>((const bf16*)dy, (const bf16*)a, (bf16*)da, M, N, cap)
  if (nch == 1) CAP_B(1); else if (nch == 2) CAP_B(2); else if (nch == 3) CAP_B(3); else CAP_B(4);
#undef CAP_B
  return (int)cudaGetLastError();
}

extern "C" int loom_add_ln_fwd(const void* a, const void* b, const float* w, const float* bias, void* y, void* x,
                               float* mean, float* rstd, int M, int N, float eps, float cap, cudaStream_t st) {
  if (N % 8 || N > 2048) return -1;
  if (M <= 64) {                                          // a decode step: one block per row
    const int threads = ((N / 8 + 31) / 32) * 32;
    // programmatically dependent only for a handful of rows: with more, early-resident dependents cost more than the
    // overlapped launch saves (decode at 64 sequences: 1.06 against 1.02 ms per step; at one: 0.474 against 0.493 ms)
    if (M <= 16)
      return (int)loom::launch_pdl(add_ln_fwd_row_kernel, dim3(M), dim3(threads), 0, st, (const bf16*)a, (const bf16*)b, w, bias, (bf16*)y,
                                   (bf16*)x, mean, rstd, N, eps, cap);
    add_ln_fwd_row_kernel<<<M, threads, 0, st>>>((const bf16*)a, (const bf16*)b, w, bias, (bf16*)y, (bf16*)x, mean, rstd, N, eps, cap);
    return (int)cudaGetLastError();
  }
  const unsigned grid = (M + 7) / 8;
  const int nch = (N + 255) / 256;
#define LN_F(K) add_ln_fwd_kernel<K><<<grid, 256, 0, st>>>((const bf16*)a, (const bf16*)b, w, bias, (bf16*)y, (bf16*)x, mean, rstd, M, N, eps, cap)
  if (nch == 1) LN_F(1); else if (nch == 2) LN_F(2); else if (nch == 3) LN_F(3); else if (nch == 4) LN_F(4);
  else if (nch <= 6) LN_F(6); else LN_F(8);
#undef LN_F
  return (int)cudaGetLastError();
}

extern "C" int loom_add_ln_bwd(const void* dy, const void* x, const float* mean, const float* rstd, const float* w,
                               void* dx, float* gw, float* gb, int M, int N, cudaStream_t st) {
  if (N % 8 || N > 2048) return -1;
  unsigned grid = (M + 7) / 8;
  // one block per SM: every block ends with 2 N atomic adds for the weight and bias gradients, and at 2048 rows one
  // block per SM (6.9 us) beats one block per 8 rows (8.4 us) and half a block per SM (9.4 us)
  static int cap_blocks = 0;
  if (cap_blocks == 0) { int dev = 0; cudaGetDevice(&dev); cudaDeviceGetAttribute(&cap_blocks, cudaDevAttrMultiProcessorCount, dev); }
  if (grid > (unsigned)cap_blocks) grid = cap_blocks;
  const int nch = (N + 255) / 256;
  const size_t shm = 2 * 8 * N * sizeof(float);
#define LN_B(K) do { if (shm > 48 * 1024) cudaFuncSetAttribute(add_ln_bwd_kernel<K>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shm); \
    add_ln_bwd_kernel<K><<<grid, 256, shm, st>>>((const bf16*)dy, (const bf16*)x, mean, rstd, w, (bf16*)dx, gw, gb, M, N); } while (0)
  if (nch == 1) LN_B(1); else if (nch == 2) LN_B(2); else if (nch == 3) LN_B(3); else if (nch == 4) LN_B(4);
  else if (nch <= 6) LN_B(6); else LN_B(8);
#undef LN_B
  return (int)cudaGetLastError();
}

// Running radius of the imaginary pre-activation: rad = max(sqrt(sum beta^2 / n), 1e-4); anchor <- decay * anchor +
// (1 - decay) * rad; the updated value is also written to ``snap`` (what the backward of this cell will use).
__global__ void anchor_ema_kernel(const float* __restrict__ beta_sq_sum, float inv_n, float decay, float* __restrict__ anchor,
                                  float* __restrict__ snap) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    const float rad = fmaxf(sqrtf(*beta_sq_sum * inv_n), 1e-4f);
    const float a = *anchor * decay + rad * (1.f - decay);
    *anchor = a;
    *snap = a;
  }
}

extern "C" int loom_anchor_ema(const float* beta_sq_sum, float inv_n, float decay, float* anchor, float* snap,
                               cudaStream_t st) {
  anchor_ema_kernel<<<1, 32, 0, st>>>(beta_sq_sum, inv_n, decay, anchor, snap);
  return (int)cudaGetLastError();
}

extern "C" int loom_colsum(const void* dy, float* gb, int M, int N, long long ld, cudaStream_t st) {
  if (N % 2) return -1;
  dim3 grid((N / 2 + 63) / 64, (M + 63) / 64);
  colsum_kernel<<<grid, 256, 0, st>>>((const bf16*)dy, gb, M, N, ld);
  return (int)cudaGetLastError();
}

extern "C" int loom_ce(void* logits, const long long* targets, float* nll, const float* scale_ptr, long long M, int V,
                       long long ignore_index, int write_grad, cudaStream_t st) {
  if (V % 8) return -1;
  ce_kernel<<<(unsigned)M, 256, 0, st>>>((bf16*)logits, targets, nll, scale_ptr, V, ignore_index, write_grad);
  return (int)cudaGetLastError();
}
