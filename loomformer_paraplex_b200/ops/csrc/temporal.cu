// Temporal carry of the Tria carriers across one chunk, endpoint only, with the PolARM correction
// fused in:   acc_t = N(D_t acc_{t-1})   (restart acc_t = N(D_t) at a reset or when no state enters),
// then for fired rows  acc <- acc (I - beta/2 (G/mean(diag G) - I)),  G = acc^T acc.
//
// One thread per (batch row, neuron); the loop over the <= W tokens of the chunk is sequential, threads
// of a warp read consecutive neurons of the plane-major carrier buffer.  The backward pass walks the
// chunk in reverse and recovers acc_{t-1} = N(D_t^{-1} acc_t) analytically, re-anchored on exact states
// that the forward pass checkpoints every CKPT tokens, so no per-token trajectory is ever stored.
// Reference: kernels/tria/temporal_carry_endpoint/temporal_carry_endpoint_kernel.cuh:12-121 and
// tria.py:128-139 (PolARM, separate PyTorch ops there).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include "loom_c_api.h"

namespace {

typedef __nv_bfloat16 bf16;
constexpr int CKPT = 16;
constexpr float EPS = 1e-6f;

__device__ __forceinline__ void mat3(const float* A, const float* B, float* C) {   // C = A B
#pragma unroll
  for (int r = 0; r < 3; ++r)
#pragma unroll
    for (int c = 0; c < 3; ++c) C[r * 3 + c] = A[r * 3] * B[c] + A[r * 3 + 1] * B[3 + c] + A[r * 3 + 2] * B[6 + c];
}
__device__ __forceinline__ float norm9(float* M) {   // in place M /= sqrt(mean(M^2)+eps); returns the divisor
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < 9; ++k) ss += M[k] * M[k];
  const float n = sqrtf(ss * (1.f / 9.f) + EPS);
  const float inv = 1.f / n;
#pragma unroll
  for (int k = 0; k < 9; ++k) M[k] *= inv;
  return n;
}
__device__ __forceinline__ void polarm_fwd(const float* M, float beta, float* out) {
  float G[9];
#pragma unroll
  for (int r = 0; r < 3; ++r)
#pragma unroll
    for (int c = 0; c < 3; ++c) G[r * 3 + c] = M[r] * M[c] + M[3 + r] * M[3 + c] + M[6 + r] * M[6 + c];
  const float s = fmaxf((G[0] + G[4] + G[8]) * (1.f / 3.f), EPS);
  const float cf = 0.5f * beta;
  float K[9];
#pragma unroll
  for (int k = 0; k < 9; ++k) K[k] = -cf * G[k] / s;
  K[0] += 1.f + cf; K[4] += 1.f + cf; K[8] += 1.f + cf;
  mat3(M, K, out);
}
// gM for out = M K(M)
__device__ __forceinline__ void polarm_bwd(const float* M, float beta, const float* gOut, float* gM) {
  float G[9];
#pragma unroll
  for (int r = 0; r < 3; ++r)
#pragma unroll
    for (int c = 0; c < 3; ++c) G[r * 3 + c] = M[r] * M[c] + M[3 + r] * M[3 + c] + M[6 + r] * M[6 + c];
  const float tr = (G[0] + G[4] + G[8]) * (1.f / 3.f);
  const float s = fmaxf(tr, EPS);
  const float cf = 0.5f * beta;
  float K[9];
#pragma unroll
  for (int k = 0; k < 9; ++k) K[k] = -cf * G[k] / s;
  K[0] += 1.f + cf; K[4] += 1.f + cf; K[8] += 1.f + cf;
  // gM (direct) = gOut K^T ; gK = M^T gOut
  float gK[9];
#pragma unroll
  for (int r = 0; r < 3; ++r)
#pragma unroll
    for (int c = 0; c < 3; ++c) {
      gM[r * 3 + c] = gOut[r * 3] * K[c * 3] + gOut[r * 3 + 1] * K[c * 3 + 1] + gOut[r * 3 + 2] * K[c * 3 + 2];
      gK[r * 3 + c] = M[r] * gOut[c] + M[3 + r] * gOut[3 + c] + M[6 + r] * gOut[6 + c];
    }
  float gG[9], dot = 0.f;
#pragma unroll
  for (int k = 0; k < 9; ++k) { gG[k] = -cf / s * gK[k]; dot += gK[k] * G[k]; }
  if (tr > EPS) {
    const float gs = cf / (s * s) * dot * (1.f / 3.f);
    gG[0] += gs; gG[4] += gs; gG[8] += gs;
  }
  // G = M^T M : gM += M (gG + gG^T)
#pragma unroll
  for (int r = 0; r < 3; ++r)
#pragma unroll
    for (int c = 0; c < 3; ++c) {
      float a = 0.f;
#pragma unroll
      for (int j = 0; j < 3; ++j) a += M[r * 3 + j] * (gG[j * 3 + c] + gG[c * 3 + j]);
      gM[r * 3 + c] += a;
    }
}
__device__ __forceinline__ bool inv3(const float* A, float* I) {
  const float c0 = A[4] * A[8] - A[5] * A[7], c1 = A[5] * A[6] - A[3] * A[8], c2 = A[3] * A[7] - A[4] * A[6];
  const float det = A[0] * c0 + A[1] * c1 + A[2] * c2;
  if (fabsf(det) < 1e-20f) return false;
  const float id = 1.f / det;
  I[0] = c0 * id; I[1] = (A[2] * A[7] - A[1] * A[8]) * id; I[2] = (A[1] * A[5] - A[2] * A[4]) * id;
  I[3] = c1 * id; I[4] = (A[0] * A[8] - A[2] * A[6]) * id; I[5] = (A[2] * A[3] - A[0] * A[5]) * id;
  I[6] = c2 * id; I[7] = (A[1] * A[6] - A[0] * A[7]) * id; I[8] = (A[0] * A[4] - A[1] * A[3]) * id;
  return true;
}

// depth: planes [9][B*Tc][H] bf16.  state_in [B,H,9] fp32 or null.  Outputs: state_out (after PolARM on fired
// rows), raw endpoint (before PolARM), checkpoints [nck][B,H,9] at tokens t with (t+1) % CKPT == 0.
__global__ void __launch_bounds__(128) temporal_fwd_kernel(const bf16* __restrict__ depth, const uint8_t* __restrict__ reset,
                                                           const float* __restrict__ state_in,
                                                           const uint8_t* __restrict__ fired, float beta,
                                                           float* __restrict__ state_out, float* __restrict__ raw_out,
                                                           float* __restrict__ ckpt, int B, int Tc, int H) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)B * H) return;
  const int b = (int)(idx / H), h = (int)(idx % H);
  const long long plane = (long long)B * Tc * H;
  float acc[9];
  bool have = state_in != nullptr;
  if (have) {
#pragma unroll
    for (int k = 0; k < 9; ++k) acc[k] = state_in[idx * 9 + k];
  }
  // The recurrence is one dependent chain per thread; the carriers it consumes do not depend on it.  Loading them inside
  // the chain would pay a memory round trip per token, so the loads of UF tokens are issued together.
  constexpr int UF = 4;
  for (int t0 = 0; t0 < Tc; t0 += UF) {
    bf16 rawd[UF][9];
    uint8_t rs[UF];
#pragma unroll
    for (int u = 0; u < UF; ++u) {
      const int tt = t0 + u < Tc ? t0 + u : Tc - 1;
      const long long e = ((long long)b * Tc + tt) * H + h;
#pragma unroll
      for (int k = 0; k < 9; ++k) rawd[u][k] = depth[k * plane + e];
      rs[u] = reset[b * Tc + tt];
    }
#pragma unroll
    for (int u = 0; u < UF; ++u) {
      const int t = t0 + u;
      if (t < Tc) {
        float D[9], pre[9];
#pragma unroll
        for (int k = 0; k < 9; ++k) D[k] = __bfloat162float(rawd[u][k]);
        if (have && !rs[u]) {
          mat3(D, acc, pre);
#pragma unroll
          for (int k = 0; k < 9; ++k) acc[k] = pre[k];
        } else {
#pragma unroll
          for (int k = 0; k < 9; ++k) acc[k] = D[k];
        }
        norm9(acc);
        have = true;
        if (ckpt && ((t + 1) % CKPT == 0)) {
          float* c = ckpt + ((long long)(t / CKPT) * B * H + idx) * 9;
#pragma unroll
          for (int k = 0; k < 9; ++k) c[k] = acc[k];
        }
      }
    }
  }
  if (raw_out) {
#pragma unroll
    for (int k = 0; k < 9; ++k) raw_out[idx * 9 + k] = acc[k];
  }
  if (fired && fired[b]) {
    float o[9];
    polarm_fwd(acc, beta, o);
#pragma unroll
    for (int k = 0; k < 9; ++k) acc[k] = o[k];
  }
#pragma unroll
  for (int k = 0; k < 9; ++k) state_out[idx * 9 + k] = acc[k];
}

__global__ void __launch_bounds__(128) temporal_bwd_kernel(const bf16* __restrict__ depth, const uint8_t* __restrict__ reset,
                                                           const float* __restrict__ state_in,
                                                           const uint8_t* __restrict__ fired, float beta,
                                                           const float* __restrict__ raw, const float* __restrict__ ckpt,
                                                           const float* __restrict__ dstate, bf16* __restrict__ ddepth,
                                                           float* __restrict__ dstate_in, int B, int Tc, int H) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)B * H) return;
  const int b = (int)(idx / H), h = (int)(idx % H);
  const long long plane = (long long)B * Tc * H;
  float acc[9], g[9];
#pragma unroll
  for (int k = 0; k < 9; ++k) { acc[k] = raw[idx * 9 + k]; g[k] = dstate[idx * 9 + k]; }
  if (fired && fired[b]) {
    float gm[9];
    polarm_bwd(acc, beta, g, gm);
#pragma unroll
    for (int k = 0; k < 9; ++k) g[k] = gm[k];
  }
  bool alive = true;      // gradient still flows to earlier tokens
  constexpr int UB = 4;                 // tokens whose carriers are loaded together (see the forward kernel)
  for (int t0 = Tc - 1; t0 >= 0; t0 -= UB) {
    bf16 rawd[UB][9];
    uint8_t rs[UB];
#pragma unroll
    for (int u = 0; u < UB; ++u) {
      const int tt = t0 - u >= 0 ? t0 - u : 0;
      const long long e = ((long long)b * Tc + tt) * H + h;
#pragma unroll
      for (int k = 0; k < 9; ++k) rawd[u][k] = depth[k * plane + e];
      rs[u] = reset[b * Tc + tt];
    }
#pragma unroll
    for (int u = 0; u < UB; ++u) {
      const int t = t0 - u;
      if (t < 0) continue;
      const long long e = ((long long)b * Tc + t) * H + h;
      if (!alive) {
#pragma unroll
        for (int k = 0; k < 9; ++k) ddepth[k * plane + e] = __float2bfloat16(0.f);
        continue;
      }
      float D[9];
#pragma unroll
      for (int k = 0; k < 9; ++k) D[k] = __bfloat162float(rawd[u][k]);
      const bool cont = !rs[u] && (t > 0 || state_in != nullptr);
      float prev[9], pre[9];
      if (cont) {
        if (t == 0) {
#pragma unroll
          for (int k = 0; k < 9; ++k) prev[k] = state_in[idx * 9 + k];
        } else if (ckpt && (t % CKPT == 0)) {
          const float* c = ckpt + ((long long)(t / CKPT - 1) * B * H + idx) * 9;
#pragma unroll
          for (int k = 0; k < 9; ++k) prev[k] = c[k];
        } else {
          float Di[9];
          if (inv3(D, Di)) { mat3(Di, acc, prev); norm9(prev); }
          else {
#pragma unroll
            for (int k = 0; k < 9; ++k) prev[k] = 0.f;
          }
        }
        mat3(D, prev, pre);
      } else {
#pragma unroll
        for (int k = 0; k < 9; ++k) pre[k] = D[k];
      }
      float ss = 0.f;
#pragma unroll
      for (int k = 0; k < 9; ++k) ss += pre[k] * pre[k];
      const float inv = rsqrtf(ss * (1.f / 9.f) + EPS);
      float dot = 0.f, gp[9];
#pragma unroll
      for (int k = 0; k < 9; ++k) dot += g[k] * pre[k] * inv;
      dot *= (1.f / 9.f);
#pragma unroll
      for (int k = 0; k < 9; ++k) gp[k] = (g[k] - pre[k] * inv * dot) * inv;
      if (cont) {
        // gD = gp prev^T ; g_prev = D^T gp
#pragma unroll
        for (int r = 0; r < 3; ++r)
#pragma unroll
          for (int c = 0; c < 3; ++c) {
            const float gd = gp[r * 3] * prev[c * 3] + gp[r * 3 + 1] * prev[c * 3 + 1] + gp[r * 3 + 2] * prev[c * 3 + 2];
            ddepth[(r * 3 + c) * plane + e] = __float2bfloat16(gd);
            g[r * 3 + c] = D[r] * gp[c] + D[3 + r] * gp[3 + c] + D[6 + r] * gp[6 + c];
          }
#pragma unroll
        for (int k = 0; k < 9; ++k) acc[k] = prev[k];
      } else {
#pragma unroll
        for (int k = 0; k < 9; ++k) { ddepth[k * plane + e] = __float2bfloat16(gp[k]); g[k] = 0.f; }
        alive = false;
      }
    }
  }
  if (dstate_in) {
#pragma unroll
    for (int k = 0; k < 9; ++k) dstate_in[idx * 9 + k] = alive ? g[k] : 0.f;
  }
}

}  // namespace

extern "C" int loom_temporal_fwd(const void* depth, const uint8_t* reset, const float* state_in, const uint8_t* fired,
                                 float beta, float* state_out, float* raw_out, float* ckpt, int B, int Tc, int H,
                                 cudaStream_t st) {
  const long long n = (long long)B * H;
  temporal_fwd_kernel<<<(unsigned)((n + 127) / 128), 128, 0, st>>>((const bf16*)depth, reset, state_in, fired, beta,
                                                                   state_out, raw_out, ckpt, B, Tc, H);
  return (int)cudaGetLastError();
}

extern "C" int loom_temporal_bwd(const void* depth, const uint8_t* reset, const float* state_in, const uint8_t* fired,
                                 float beta, const float* raw, const float* ckpt, const float* dstate, void* ddepth,
                                 float* dstate_in, int B, int Tc, int H, cudaStream_t st) {
  const long long n = (long long)B * H;
  temporal_bwd_kernel<<<(unsigned)((n + 127) / 128), 128, 0, st>>>((const bf16*)depth, reset, state_in, fired, beta, raw,
                                                                   ckpt, dstate, (bf16*)ddepth, dstate_in, B, Tc, H);
  return (int)cudaGetLastError();
}
