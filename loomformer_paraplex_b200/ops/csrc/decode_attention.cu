// KV-cache attention for one new token per sequence (decode), dual context.
//
//   a = softmax(q . K[0..pos] / sqrt(HD)),   ctx = a V,   kctx = a K          (per query head; GQA: G heads share K/V)
//
// The current position is read from device memory, so the launch is identical for every token and can sit in a
// replayed CUDA graph.  One block serves one (sequence, KV head) pair and a slice of the positions ("split-K": with a
// batch of one there are only KVH pairs, so the positions are spread over enough blocks to fill the GPU).  A block
// walks its slice in tiles of 64 positions: the K and V rows of a tile are brought into shared memory with 16-byte
// cp.async copies that are all in flight at once (the loop is bound by memory latency otherwise), scores are one
// (head, position) pair per thread, the running softmax state is rescaled per tile, and the two weighted sums are one
// (head, dim pair) per thread out of shared memory.  Each block leaves its partial state in a workspace and takes a
// ticket; the block that draws the last ticket of its (sequence, KV head) merges the partial states and resets the
// ticket counter, so there is no second launch and nothing waits on anything.
// The reference does this with matmul + softmax + two matmuls over cache[:, :len] in PyTorch
// (reference loomformer.py, Attention.step), re-launching per token from the host.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include "launch_util.cuh"
#include "loom_c_api.h"

namespace {

typedef __nv_bfloat16 bf16;
constexpr int MAXG = 8;
constexpr int TP = 64;            // positions per tile
constexpr int THREADS = 256;
constexpr int MAXIT = 2;          // (head, dim pair) slots per thread: MAXG * 128 / 2 / THREADS

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
}

// q [B,QH,HD] (row pitch q_ld); kc, vc [B,S,KVH,HD]; out_c, out_k [B,QH,HD] (row pitch out_ld)
// ws: per (b, kvh, z): m[G], l[G], acc_v[G][HD], acc_k[G][HD]; tickets: one int per (b, kvh), zero between launches
__global__ void __launch_bounds__(THREADS) decode_attn_kernel(
    const bf16* __restrict__ q, const bf16* __restrict__ kc, const bf16* __restrict__ vc, const long long* __restrict__ pos_ptr,
    bf16* __restrict__ out_c, bf16* __restrict__ out_k, float* __restrict__ ws, int* __restrict__ tickets, int S, int QH,
    int KVH, int HD, int NS, float scale, long long out_ld, long long q_ld) {
  extern __shared__ uint4 sh_raw[];
  const int G = QH / KVH, HD2 = HD >> 1, LDT = HD + 8, C8 = HD >> 3;
  const int b = blockIdx.x / KVH, kvh = blockIdx.x % KVH, z = blockIdx.y;
  const int tid = threadIdx.x, lane = tid & 31;
  float* sq = reinterpret_cast<float*>(sh_raw);          // [G][HD]
  float* ps = sq + G * HD;                               // [G][TP]
  float* red = ps + G * TP;                              // [32]
  float* sm_m = red + 32;                                // [MAXG]
  float* sm_l = sm_m + MAXG;
  float* sm_f = sm_l + MAXG;
  bf16* kt = reinterpret_cast<bf16*>(sm_f + MAXG);       // [TP][LDT]
  bf16* vt = kt + TP * LDT;
  __shared__ int s_last;

  loom::pdl_trigger();
  loom::pdl_wait();                                      // the new token's K / V rows come from the previous kernel
  long long n = *pos_ptr + 1;
  if (n > S) n = S;
  if (n < 0) n = 0;
  const int chunk = (int)((n + NS - 1) / NS);
  const int lo = z * chunk;
  int hi = lo + chunk;
  if (hi > n) hi = (int)n;
  const int cnt = hi > lo ? hi - lo : 0;
  for (int i = tid; i < G * HD; i += THREADS)
    sq[i] = __bfloat162float(q[(long long)b * q_ld + (long long)kvh * G * HD + i]) * scale;
  if (tid < MAXG) { sm_m[tid] = -INFINITY; sm_l[tid] = 0.f; sm_f[tid] = 0.f; }
  const long long row_stride = (long long)KVH * HD;
  const bf16* kbase = kc + ((long long)b * S * KVH + kvh) * HD + (long long)lo * row_stride;
  const bf16* vbase = vc + ((long long)b * S * KVH + kvh) * HD + (long long)lo * row_stride;
  float acc[MAXIT][4];
#pragma unroll
  for (int j = 0; j < MAXIT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;

  for (int t0 = 0; t0 < cnt; t0 += TP) {
    const int valid = cnt - t0 < TP ? cnt - t0 : TP;
    for (int i = tid; i < valid * C8; i += THREADS) {
      const int r = i / C8, c = i - r * C8;
      cp_async16(kt + r * LDT + c * 8, kbase + (long long)(t0 + r) * row_stride + c * 8);
      cp_async16(vt + r * LDT + c * 8, vbase + (long long)(t0 + r) * row_stride + c * 8);
    }
    cp_async_wait_all();
    __syncthreads();
    // scores: one (head, position) per thread; a warp covers 32 positions of one head
    for (int idx = tid; idx < G * TP; idx += THREADS) {
      const int g = idx / TP, p = idx - g * TP;
      float s = -INFINITY;
      if (p < valid) {
        const float* qg = sq + g * HD;
        const bf16* kr = kt + p * LDT;
        float d0 = 0.f, d1 = 0.f;
        for (int c = 0; c < HD; c += 8) {
          const uint4 u = *reinterpret_cast<const uint4*>(kr + c);
          const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&u);
          const float4 qa = *reinterpret_cast<const float4*>(qg + c), qb = *reinterpret_cast<const float4*>(qg + c + 4);
          const float2 f0 = __bfloat1622float2(h2[0]), f1 = __bfloat1622float2(h2[1]);
          const float2 f2 = __bfloat1622float2(h2[2]), f3 = __bfloat1622float2(h2[3]);
          d0 += f0.x * qa.x + f0.y * qa.y + f1.x * qa.z + f1.y * qa.w;
          d1 += f2.x * qb.x + f2.y * qb.y + f3.x * qb.z + f3.y * qb.w;
        }
        s = d0 + d1;
      }
      ps[idx] = s;
      float mx = s;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      if (lane == 0) red[idx >> 5] = mx;
    }
    __syncthreads();
    if (tid < G) {
      const float mt = fmaxf(red[2 * tid], red[2 * tid + 1]);          // TP / 32 = 2 warps per head
      const float mo = sm_m[tid], mn = fmaxf(mo, mt);
      sm_f[tid] = __expf(mo - mn);                                     // first tile: exp(-inf) = 0
      sm_m[tid] = mn;
    }
    __syncthreads();
    for (int idx = tid; idx < G * TP; idx += THREADS) {
      const int g = idx / TP;
      const float e = __expf(ps[idx] - sm_m[g]);                       // masked positions: exp(-inf) = 0
      ps[idx] = e;
      float sum = e;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      if (lane == 0) red[idx >> 5] = sum;
    }
    __syncthreads();
    if (tid < G) sm_l[tid] = sm_l[tid] * sm_f[tid] + red[2 * tid] + red[2 * tid + 1];
    // weighted sums: one (head, dim pair) per thread
#pragma unroll
    for (int j = 0; j < MAXIT; ++j) {
      const int idx = tid + j * THREADS;
      if (idx < G * HD2) {
        const int g = idx / HD2, c2 = idx - g * HD2;
        const float f = sm_f[g];
        float v0 = acc[j][0] * f, v1 = acc[j][1] * f, k0 = acc[j][2] * f, k1 = acc[j][3] * f;
        const float* pr = ps + g * TP;
#pragma unroll 4
        for (int p = 0; p < valid; ++p) {
          const float w = pr[p];
          const float2 vv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(vt + p * LDT + 2 * c2));
          const float2 kk = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(kt + p * LDT + 2 * c2));
          v0 = fmaf(w, vv.x, v0); v1 = fmaf(w, vv.y, v1);
          k0 = fmaf(w, kk.x, k0); k1 = fmaf(w, kk.y, k1);
        }
        acc[j][0] = v0; acc[j][1] = v1; acc[j][2] = k0; acc[j][3] = k1;
      }
    }
    __syncthreads();                                                   // tiles and probabilities are reused
  }

  const int per = 2 * G + 2 * G * HD;
  if (NS == 1) {
#pragma unroll
    for (int j = 0; j < MAXIT; ++j) {
      const int idx = tid + j * THREADS;
      if (idx < G * HD2) {
        const int g = idx / HD2, c2 = idx - g * HD2;
        const float inv = 1.f / sm_l[g];
        const long long o = (long long)b * out_ld + (long long)(kvh * G + g) * HD + 2 * c2;
        *reinterpret_cast<__nv_bfloat162*>(out_c + o) = __floats2bfloat162_rn(acc[j][0] * inv, acc[j][1] * inv);
        *reinterpret_cast<__nv_bfloat162*>(out_k + o) = __floats2bfloat162_rn(acc[j][2] * inv, acc[j][3] * inv);
      }
    }
    return;
  }
  float* wsb = ws + ((long long)blockIdx.x * NS + z) * per;
#pragma unroll
  for (int j = 0; j < MAXIT; ++j) {
    const int idx = tid + j * THREADS;
    if (idx < G * HD2) {                                  // an empty slice leaves zeros
      const int g = idx / HD2, c2 = idx - g * HD2;
      *reinterpret_cast<float2*>(wsb + 2 * G + g * HD + 2 * c2) = make_float2(acc[j][0], acc[j][1]);
      *reinterpret_cast<float2*>(wsb + 2 * G + G * HD + g * HD + 2 * c2) = make_float2(acc[j][2], acc[j][3]);
    }
  }
  if (tid < G) { wsb[tid] = cnt > 0 ? sm_m[tid] : -INFINITY; wsb[G + tid] = cnt > 0 ? sm_l[tid] : 0.f; }
  __threadfence();
  __syncthreads();
  if (tid == 0) s_last = atomicAdd(tickets + blockIdx.x, 1) == NS - 1;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // the last block of this (sequence, KV head): merge all partial states.  The softmax statistics of every slice are
  // staged first and turned into one weight per (head, slice), so that the sums below are plain independent loads
  // (a data-dependent branch per slice would serialise the loop on memory latency).
  const float* base = ws + (long long)blockIdx.x * NS * per;
  float* f_m = ps;                                         // [G][NS], NS <= TP
  float* f_l = reinterpret_cast<float*>(kt);               // [G][NS]
  for (int i = tid; i < G * NS; i += THREADS) {
    const int g = i / NS, zz = i - g * NS;
    f_m[i] = __ldcg(base + zz * per + g);
    f_l[i] = __ldcg(base + zz * per + G + g);
  }
  __syncthreads();
  if (tid < G) {
    float M = -INFINITY, l = 0.f;
    for (int zz = 0; zz < NS; ++zz) M = fmaxf(M, f_m[tid * NS + zz]);
    for (int zz = 0; zz < NS; ++zz) {
      const float f = __expf(f_m[tid * NS + zz] - M);      // empty slice: exp(-inf) = 0
      l += f_l[tid * NS + zz] * f;
      f_m[tid * NS + zz] = f;
    }
    sm_l[tid] = 1.f / l;
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < MAXIT; ++j) {
    const int idx = tid + j * THREADS;
    if (idx < G * HD2) {
      const int g = idx / HD2, c2 = idx - g * HD2;
      const float* fw = f_m + g * NS;
      const float* pv = base + 2 * G + g * HD + 2 * c2;
      const float* pk = pv + G * HD;
      float v0 = 0.f, v1 = 0.f, k0 = 0.f, k1 = 0.f;
#pragma unroll 8
      for (int zz = 0; zz < NS; ++zz) {
        const float f = fw[zz];
        const float2 a = __ldcg(reinterpret_cast<const float2*>(pv + (long long)zz * per));
        const float2 k = __ldcg(reinterpret_cast<const float2*>(pk + (long long)zz * per));
        v0 = fmaf(a.x, f, v0); v1 = fmaf(a.y, f, v1); k0 = fmaf(k.x, f, k0); k1 = fmaf(k.y, f, k1);
      }
      const float inv = sm_l[g];
      const long long o = (long long)b * out_ld + (long long)(kvh * G + g) * HD + 2 * c2;
      *reinterpret_cast<__nv_bfloat162*>(out_c + o) = __floats2bfloat162_rn(v0 * inv, v1 * inv);
      *reinterpret_cast<__nv_bfloat162*>(out_k + o) = __floats2bfloat162_rn(k0 * inv, k1 * inv);
    }
  }
  if (tid == 0) tickets[blockIdx.x] = 0;
}

}  // namespace

// floats of workspace for NS position slices: the partial states, then one ticket counter per (sequence, KV head).
// The caller zeroes the workspace once; every launch leaves the counters at zero.
extern "C" int loom_decode_attn_workspace_floats(int B, int QH, int KVH, int HD, int NS) {
  const int G = QH / KVH;
  return B * KVH * NS * (2 * G + 2 * G * HD) + B * KVH;
}

// q and out_c / out_k rows of sequence b start at b * q_ld resp. b * out_ld elements (QH * HD for dense [B,QH,HD])
extern "C" int loom_decode_attn(const void* q, const void* kc, const void* vc, const long long* pos, void* out_c, void* out_k,
                                float* ws, int B, int S, int QH, int KVH, int HD, int NS, long long out_ld, long long q_ld,
                                cudaStream_t st) {
  const int G = QH / KVH;
  if (HD % 8 || HD > 128 || G < 1 || G > MAXG || QH % KVH || NS < 1 || NS > TP || (out_ld & 1)) return -1;
  if ((2 * G + 2 * G * HD) & 1) return -1;
  const size_t shm = ((size_t)G * HD + (size_t)G * TP + 32 + 3 * MAXG) * sizeof(float) + (size_t)2 * TP * (HD + 8) * sizeof(bf16);
  if (shm > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(decode_attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shm);
    if (e != cudaSuccess) return (int)e;
  }
  int* tickets = reinterpret_cast<int*>(ws + (size_t)B * KVH * NS * (2 * G + 2 * G * HD));
  dim3 grid(B * KVH, NS);
  return (int)loom::launch_pdl(decode_attn_kernel, grid, dim3(THREADS), shm, st, (const bf16*)q, (const bf16*)kc, (const bf16*)vc, pos,
                               (bf16*)out_c, (bf16*)out_k, ws, tickets, S, QH, KVH, HD, NS, rsqrtf((float)HD), out_ld, q_ld);
}
