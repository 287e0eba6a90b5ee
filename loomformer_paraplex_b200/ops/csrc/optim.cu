// One-launch optimizer over the flat parameter buffer (256-element blocks, per-block hyper-parameters).
//
//   loom_grad_norm    : global L2 norm of the gradient buffer -> clip coefficient and finite flag
//   loom_adamw_flat   : AdamW (decoupled weight decay, bias correction) on every active block
//   loom_atom_flat    : ATOM (per-block trust and commit gating on top of Adam moments; semantics of the
//                       reference kernel atom/atom.py:157-248, which runs one launch per tensor)
//
// Both update kernels read the clip coefficient and the finite flag from device memory (no host
// round trip), skip the update when the gradient norm is not finite, and refresh the bf16 shadow of
// the parameters that the tensor-core kernels read.  Step-dependent scalars (lr, bias corrections)
// come from a small device array so the launch can be replayed from a CUDA graph.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include "loom_c_api.h"

namespace {

constexpr int BLK = 256;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float block_sum_256(float v, float* sh) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) sh[w] = v;
  __syncthreads();
  float r = (threadIdx.x < 8) ? sh[threadIdx.x] : 0.f;
  if (w == 0) r = warp_sum(r);
  if (threadIdx.x == 0) sh[8] = r;
  __syncthreads();
  return sh[8];
}

__global__ void sumsq_partial_kernel(const float* __restrict__ g, long long n, float* __restrict__ partial) {
  __shared__ float sh[16];
  float acc = 0.f;
  const long long n4 = n >> 2;
  const float4* g4 = reinterpret_cast<const float4*>(g);
  for (long long i = (long long)blockIdx.x * BLK + threadIdx.x; i < n4; i += (long long)gridDim.x * BLK) {
    float4 v = g4[i];
    acc += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  float tot = block_sum_256(acc, sh);
  if (threadIdx.x == 0) partial[blockIdx.x] = tot;
}

// stats: [0] grad norm, [1] clip coefficient, [2] finite flag, [3] unused.  Also clears atom_out.
__global__ void norm_finalize_kernel(const float* __restrict__ partial, int nparts, float max_norm,
                                     float* __restrict__ stats, float* __restrict__ atom_out) {
  __shared__ float sh[16];
  float acc = 0.f;
  for (int i = threadIdx.x; i < nparts; i += BLK) acc += partial[i];
  float tot = block_sum_256(acc, sh);
  if (threadIdx.x == 0) {
    float norm = sqrtf(tot);
    bool fin = isfinite(norm);
    stats[0] = norm;
    stats[1] = (max_norm > 0.f && fin) ? fminf(1.f, max_norm / (norm + 1e-6f)) : 1.f;
    stats[2] = fin ? 1.f : 0.f;
    if (atom_out) { atom_out[0] = 0.f; atom_out[1] = 0.f; atom_out[2] = 0.f; }
  }
}

// hyper: [0] lr, [1] beta1, [2] beta2, [3] eps, [4] bias-correction 1, [5] bias-correction 2,
//        [6] ATOM bootstrap flag (1 while step <= bootstrap steps)
__global__ void adamw_flat_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
                                  float* __restrict__ v, __nv_bfloat16* __restrict__ shadow,
                                  const float* __restrict__ lr_mult, const float* __restrict__ wd_blk,
                                  const float* __restrict__ active, const float* __restrict__ stats,
                                  const float* __restrict__ hyper) {
  const int b = blockIdx.x;
  if (active[b] == 0.f || stats[2] == 0.f) return;
  const long long i = (long long)b * BLK + threadIdx.x;
  const float lr = hyper[0] * lr_mult[b], b1 = hyper[1], b2 = hyper[2], eps = hyper[3], bc1 = hyper[4], bc2 = hyper[5];
  const float gg = g[i] * stats[1];
  const float mm = m[i] + (1.f - b1) * (gg - m[i]);
  const float vv = v[i] + (1.f - b2) * (gg * gg - v[i]);
  float pp = p[i] * (1.f - lr * wd_blk[b]);
  pp -= lr * (mm / bc1) / (sqrtf(vv / bc2) + eps);
  m[i] = mm; v[i] = vv; p[i] = pp;
  if (shadow) shadow[i] = __float2bfloat16(pp);
}

__global__ void atom_flat_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
                                 float* __restrict__ v, __nv_bfloat16* __restrict__ shadow,
                                 const float* __restrict__ lr_mult, const float* __restrict__ wd_blk,
                                 const float* __restrict__ cnt_blk, float* __restrict__ gprev_blk,
                                 float* __restrict__ pnode_blk, float* __restrict__ trust_blk,
                                 const float* __restrict__ stats, const float* __restrict__ hyper,
                                 float* __restrict__ atom_out) {
  __shared__ float sh[16];
  const int b = blockIdx.x;
  const float cnt = cnt_blk[b];
  if (cnt == 0.f || stats[2] == 0.f) return;             // uniform per block
  const long long i = (long long)b * BLK + threadIdx.x;
  const float lr = hyper[0] * lr_mult[b], b1 = hyper[1], b2 = hyper[2], eps = hyper[3];
  const float bc1 = fmaxf(hyper[4], 1e-12f), bc2 = fmaxf(hyper[5], 1e-12f);
  const float pnode = pnode_blk[b], gprev = gprev_blk[b];
  float trust = 0.90f + pnode * (1.90f - 0.90f);
  if (hyper[6] != 0.f) trust = fmaxf(trust, 2.4f);
  const float gg = g[i] * stats[1];
  const float mm = m[i] + (1.f - b1) * (gg - m[i]);
  const float vv = v[i] + (1.f - b2) * (gg * gg - v[i]);
  const float v_hat = vv / bc2;
  const float base = (mm / bc1) / (sqrtf(v_hat) + eps);
  float delta = -lr * base * (1.f + trust);
  const float pred = -((gg + 0.35f * (gg - gprev)) * delta) - 0.5f * v_hat * delta * delta;
  const float commit = (pred > 0.f && pnode >= 0.5f) ? 1.f : 0.f;
  const float p_old = p[i];
  delta = delta * commit - lr * wd_blk[b] * p_old;
  const float pp = p_old + delta;
  m[i] = mm; v[i] = vv; p[i] = pp;
  if (shadow) shadow[i] = __float2bfloat16(pp);
  const float gsum = block_sum_256(gg, sh);
  const float csum = block_sum_256(commit, sh);
  const float proxy = block_sum_256(-(gg * delta), sh);
  if (threadIdx.x == 0) {
    gprev_blk[b] = gsum / cnt;
    pnode_blk[b] = fminf(0.99f, fmaxf(0.01f, 0.95f * pnode + 0.05f * (0.5f + 0.5f * csum / cnt)));
    trust_blk[b] = trust;
    atomicAdd(&atom_out[0], proxy);
    atomicAdd(&atom_out[1], csum);
    atomicAdd(&atom_out[2], cnt);
  }
}

__global__ void cast_shadow_kernel(const float* __restrict__ p, __nv_bfloat16* __restrict__ s, long long n) {
  long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i + 3 < n) {
    float4 v = *reinterpret_cast<const float4*>(p + i);
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 o;
    o.x = *reinterpret_cast<uint32_t*>(&a); o.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(s + i) = o;
  } else {
    for (; i < n; ++i) s[i] = __float2bfloat16(p[i]);
  }
}

}  // namespace

extern "C" int loom_grad_norm(const float* grads, long long n, float max_norm, float* partial, int nparts,
                              float* stats, float* atom_out, cudaStream_t stream) {
  sumsq_partial_kernel<<<nparts, BLK, 0, stream>>>(grads, n, partial);
  norm_finalize_kernel<<<1, BLK, 0, stream>>>(partial, nparts, max_norm, stats, atom_out);
  return (int)cudaGetLastError();
}

// A bounded wait that gave up somewhere in this step (status word != 0) invalidates the gradients as surely as a
// NaN does: clear the finite flag so the update kernels skip, and keep a sticky count of skipped updates in stats[3].
__global__ void status_gate_kernel(const int* __restrict__ status, float* __restrict__ stats) {
  if (status != nullptr && *status != 0) stats[2] = 0.f;
  if (stats[2] == 0.f) stats[3] += 1.f;
}

extern "C" int loom_status_gate(const int* status, float* stats, cudaStream_t stream) {
  status_gate_kernel<<<1, 1, 0, stream>>>(status, stats);
  return (int)cudaGetLastError();
}

extern "C" int loom_adamw_flat(float* p, const float* g, float* m, float* v, void* shadow, const float* lr_mult,
                               const float* wd_blk, const float* active, const float* stats, const float* hyper,
                               long long nblk, cudaStream_t stream) {
  adamw_flat_kernel<<<(unsigned)nblk, BLK, 0, stream>>>(p, g, m, v, reinterpret_cast<__nv_bfloat16*>(shadow), lr_mult,
                                                        wd_blk, active, stats, hyper);
  return (int)cudaGetLastError();
}

extern "C" int loom_atom_flat(float* p, const float* g, float* m, float* v, void* shadow, const float* lr_mult,
                              const float* wd_blk, const float* cnt_blk, float* gprev, float* pnode, float* trust,
                              const float* stats, const float* hyper, float* atom_out, long long nblk,
                              cudaStream_t stream) {
  atom_flat_kernel<<<(unsigned)nblk, BLK, 0, stream>>>(p, g, m, v, reinterpret_cast<__nv_bfloat16*>(shadow), lr_mult,
                                                       wd_blk, cnt_blk, gprev, pnode, trust, stats, hyper, atom_out);
  return (int)cudaGetLastError();
}

extern "C" int loom_cast_shadow(const float* p, void* shadow, long long n, cudaStream_t stream) {
  const long long threads = (n + 3) / 4;
  cast_shadow_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, stream>>>(p, reinterpret_cast<__nv_bfloat16*>(shadow), n);
  return (int)cudaGetLastError();
}
