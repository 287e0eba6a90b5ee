// KV-cache attention for one new token per sequence (decode), dual context.
//
//   a = softmax(q . K[0..pos] / sqrt(HD)),   ctx = a V,   kctx = a K          (per query head; GQA: G heads share K/V)
//
// The current position is read from device memory, so the launch is identical for every token and can sit in a
// replayed CUDA graph.  One block serves one (sequence, KV head) pair and a slice of the positions ("split-K"): with
// a batch of one there are only KVH pairs, so the positions are spread over enough blocks to fill the GPU and a
// small second kernel merges the partial softmax states.  Scores are computed with one position per thread (no
// shuffles), the two weighted sums with one (head, dim) output per thread (coalesced reads of K and V rows).
// The reference does this with matmul + softmax + two matmuls over cache[:, :len] in PyTorch
// (reference loomformer.py, Attention.step), re-launching per token from the host.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include "loom_c_api.h"

namespace {

typedef __nv_bfloat16 bf16;
constexpr int MAXG = 8;

__device__ __forceinline__ float block_reduce(float v, bool is_max, float* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float t = __shfl_xor_sync(0xffffffffu, v, o);
    v = is_max ? fmaxf(v, t) : v + t;
  }
  const int w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if ((threadIdx.x & 31) == 0) sh[w] = v;
  __syncthreads();
  float r = sh[0];
  for (int i = 1; i < nw; ++i) r = is_max ? fmaxf(r, sh[i]) : r + sh[i];
  return r;
}

// q [B,QH,HD]; kc, vc [B,S,KVH,HD]; out_c, out_k [B,QH,HD]; ws: per (b,kvh,z): m[G], l[G], acc[2][G][HD]
__global__ void decode_attn_partial_kernel(const bf16* __restrict__ q, const bf16* __restrict__ kc, const bf16* __restrict__ vc,
                                           const long long* __restrict__ pos_ptr, bf16* __restrict__ out_c,
                                           bf16* __restrict__ out_k, float* __restrict__ ws, int S, int QH, int KVH, int HD,
                                           int NS, int cap, float scale, long long out_ld, long long q_ld) {
  extern __shared__ float sh[];                 // q [G][HD] | s [G][cap] | red [32]
  const int G = QH / KVH;
  const int b = blockIdx.x / KVH, kvh = blockIdx.x % KVH, z = blockIdx.y;
  float* sq = sh;
  float* ss = sq + G * HD;
  float* red = ss + G * cap;
  long long n = *pos_ptr + 1;
  if (n > S) n = S;
  const int chunk = (int)((n + NS - 1) / NS);
  const int lo = z * chunk;
  int hi = lo + chunk;
  if (hi > n) hi = (int)n;
  const int cnt = hi > lo ? hi - lo : 0;
  for (int i = threadIdx.x; i < G * HD; i += blockDim.x)
    sq[i] = __bfloat162float(q[(long long)b * q_ld + (long long)kvh * G * HD + i]) * scale;
  __syncthreads();
  const long long row_stride = (long long)KVH * HD;
  const bf16* kbase = kc + ((long long)b * S * KVH + kvh) * HD;
  const bf16* vbase = vc + ((long long)b * S * KVH + kvh) * HD;
  // phase 1: scores, one position per thread
  float mx[MAXG];
#pragma unroll
  for (int g = 0; g < MAXG; ++g) mx[g] = -INFINITY;
  for (int p = threadIdx.x; p < cnt; p += blockDim.x) {
    const bf16* kr = kbase + (long long)(lo + p) * row_stride;
    float d[MAXG];
#pragma unroll
    for (int g = 0; g < MAXG; ++g) d[g] = 0.f;
    for (int c = 0; c < HD; c += 8) {
      const uint4 u = *reinterpret_cast<const uint4*>(kr + c);
      const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h2[i]);
#pragma unroll
        for (int g = 0; g < MAXG; ++g)
          if (g < G) d[g] += f.x * sq[g * HD + c + 2 * i] + f.y * sq[g * HD + c + 2 * i + 1];
      }
    }
#pragma unroll
    for (int g = 0; g < MAXG; ++g)
      if (g < G) { ss[g * cap + p] = d[g]; mx[g] = fmaxf(mx[g], d[g]); }
  }
  __shared__ float s_m[MAXG], s_l[MAXG];
  for (int g = 0; g < G; ++g) {
    float v = -INFINITY;
#pragma unroll
    for (int k = 0; k < MAXG; ++k) if (k == g) v = mx[k];
    const float r = block_reduce(v, true, red);
    if (threadIdx.x == 0) s_m[g] = r;
  }
  __syncthreads();
  // phase 2: exponentials and their sums
  for (int g = 0; g < G; ++g) {
    const float m = s_m[g];
    float l = 0.f;
    for (int p = threadIdx.x; p < cnt; p += blockDim.x) {
      const float e = __expf(ss[g * cap + p] - m);
      ss[g * cap + p] = e;
      l += e;
    }
    const float r = block_reduce(l, false, red);
    if (threadIdx.x == 0) s_l[g] = r;
  }
  __syncthreads();
  // phase 3: the two weighted sums, one (head, dim) per thread
  float* wsb = ws + ((long long)blockIdx.x * NS + z) * (2 * G + 2 * G * HD);
  for (int idx = threadIdx.x; idx < G * HD; idx += blockDim.x) {
    const int g = idx / HD, c = idx % HD;
    float av = 0.f, ak = 0.f;
    const float* pr = ss + g * cap;
#pragma unroll 4
    for (int p = 0; p < cnt; ++p) {
      const float w = pr[p];
      av += w * __bfloat162float(vbase[(long long)(lo + p) * row_stride + c]);
      ak += w * __bfloat162float(kbase[(long long)(lo + p) * row_stride + c]);
    }
    if (NS == 1) {
      const float inv = 1.f / s_l[g];
      const long long o = (long long)b * out_ld + (long long)(kvh * G + g) * HD + c;
      out_c[o] = __float2bfloat16(av * inv);
      out_k[o] = __float2bfloat16(ak * inv);
    } else {
      wsb[2 * G + idx] = av;
      wsb[2 * G + G * HD + idx] = ak;
    }
  }
  if (NS > 1 && threadIdx.x < G) { wsb[threadIdx.x] = cnt > 0 ? s_m[threadIdx.x] : -INFINITY; wsb[G + threadIdx.x] = cnt > 0 ? s_l[threadIdx.x] : 0.f; }
}

__global__ void decode_attn_merge_kernel(const float* __restrict__ ws, bf16* __restrict__ out_c, bf16* __restrict__ out_k,
                                         int QH, int KVH, int HD, int NS, long long out_ld) {
  const int G = QH / KVH;
  const int b = blockIdx.x / KVH, kvh = blockIdx.x % KVH;
  const int per = 2 * G + 2 * G * HD;
  const float* base = ws + (long long)blockIdx.x * NS * per;
  for (int idx = threadIdx.x; idx < G * HD; idx += blockDim.x) {
    const int g = idx / HD, c = idx % HD;
    float M = -INFINITY;
    for (int z = 0; z < NS; ++z) M = fmaxf(M, base[z * per + g]);
    float l = 0.f, av = 0.f, ak = 0.f;
    for (int z = 0; z < NS; ++z) {
      const float m = base[z * per + g];
      if (m == -INFINITY) continue;
      const float f = __expf(m - M);
      l += base[z * per + G + g] * f;
      av += base[z * per + 2 * G + idx] * f;
      ak += base[z * per + 2 * G + G * HD + idx] * f;
    }
    const float inv = 1.f / l;
    const long long o = (long long)b * out_ld + (long long)(kvh * G + g) * HD + c;
    out_c[o] = __float2bfloat16(av * inv);
    out_k[o] = __float2bfloat16(ak * inv);
  }
}

}  // namespace

extern "C" int loom_decode_attn_workspace_floats(int B, int QH, int KVH, int HD, int NS) {
  const int G = QH / KVH;
  return B * KVH * NS * (2 * G + 2 * G * HD);
}

// q and out_c / out_k rows of sequence b start at b * q_ld resp. b * out_ld elements (QH * HD for dense [B,QH,HD])
extern "C" int loom_decode_attn(const void* q, const void* kc, const void* vc, const long long* pos, void* out_c, void* out_k,
                                float* ws, int B, int S, int QH, int KVH, int HD, int NS, long long out_ld, long long q_ld,
                                cudaStream_t st) {
  const int G = QH / KVH;
  if (HD % 8 || G < 1 || G > MAXG || QH % KVH || NS < 1) return -1;
  const int cap = (S + NS - 1) / NS;
  int threads = ((G * HD + 31) / 32) * 32;
  if (threads < 128) threads = 128;
  if (threads > 1024) threads = 1024;
  const size_t shm = ((size_t)G * HD + (size_t)G * cap + 32) * sizeof(float);
  if (shm > 200 * 1024) return -2;
  if (shm > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(decode_attn_partial_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shm);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid(B * KVH, NS);
  decode_attn_partial_kernel<<<grid, threads, shm, st>>>((const bf16*)q, (const bf16*)kc, (const bf16*)vc, pos, (bf16*)out_c,
                                                         (bf16*)out_k, ws, S, QH, KVH, HD, NS, cap, rsqrtf((float)HD), out_ld, q_ld);
  if (NS > 1) decode_attn_merge_kernel<<<B * KVH, threads, 0, st>>>(ws, (bf16*)out_c, (bf16*)out_k, QH, KVH, HD, NS, out_ld);
  return (int)cudaGetLastError();
}
