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
//
// Tensor-core variant (decode_attn_tc_kernel, the default when a slice fits one tile of 128 positions): the CUDA-core
// kernel above spends its time on shared-memory traffic, not on the cache rows.  Here the positions are the M side of
// tcgen05.mma: S^T[128 positions, 16] = K_tile[128, HD] . Q^T (the group's query rows are the N side, padded to 16 by
// the rows of the neighbouring heads, whose columns are ignored), one position per thread for the softmax (TMEM lane ==
// position), P^T written to shared memory as a swizzled K-major operand, and the two contexts as
// O^T[HD, 16] = V_tile^T . P^T and K_tile^T . P^T with the TMA-loaded tiles re-read as MN-major operands.  One TMA
// transaction brings the whole slice (K and V tile, Q rows); three small MMA batches; 72 KB of shared memory, so three
// CTAs share an SM.
// The reference does this with matmul + softmax + two matmuls over cache[:, :len] in PyTorch
// (reference loomformer.py, Attention.step), re-launching per token from the host.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include "launch_util.cuh"
#include "loom_c_api.h"
#include "sm100.cuh"
#include "tma_host.h"

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

// Run by every thread of the block that drew the last ticket of its (sequence, KV head): merge the NS partial states at
// `base`.  The softmax statistics of every slice are staged first and turned into one weight per (head, slice), so that
// the sums are plain independent loads (a data-dependent branch per slice would serialise the loop on memory latency).
// f_m, f_l: shared scratch of G * NS floats each; inv_l: shared, MAXG floats; obase: first output element of the group.
__device__ __forceinline__ void merge_slices(const float* __restrict__ base, int per, int NS, int G, int HD, float* f_m,
                                             float* f_l, float* inv_l, bf16* __restrict__ out_c, bf16* __restrict__ out_k,
                                             long long obase) {
  const int tid = threadIdx.x, nthr = blockDim.x, HD2 = HD >> 1;
  for (int i = tid; i < G * NS; i += nthr) {
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
    inv_l[tid] = 1.f / l;
  }
  __syncthreads();
  for (int idx = tid; idx < G * HD2; idx += nthr) {
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
    const float inv = inv_l[g];
    const long long o = obase + (long long)g * HD + 2 * c2;
    *reinterpret_cast<__nv_bfloat162*>(out_c + o) = __floats2bfloat162_rn(v0 * inv, v1 * inv);
    *reinterpret_cast<__nv_bfloat162*>(out_k + o) = __floats2bfloat162_rn(k0 * inv, k1 * inv);
  }
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
  merge_slices(ws + (long long)blockIdx.x * NS * per, per, NS, G, HD, ps, reinterpret_cast<float*>(kt), sm_l, out_c, out_k,
               (long long)b * out_ld + (long long)kvh * G * HD);
  if (tid == 0) tickets[blockIdx.x] = 0;
}


// ---------------------------------------------------------------------------------------------------------------------
// tensor-core variant: one CTA per (sequence, KV head, slice of <= 128 positions)
// ---------------------------------------------------------------------------------------------------------------------
constexpr int TC_THREADS = 128;
constexpr int TC_TILE = 16384;                 // [128 rows x 128 B] swizzled box
constexpr int TC_NPAD = 16;                    // query rows of the MMA (N side)

struct TcParams {
  CUtensorMap q;                               // (HD, QH, B), box 64 x 16
  CUtensorMap k, v;                            // (HD, KVH, S, B), box 64 x 1 x 128
  const long long* pos;
  bf16* out_c; bf16* out_k;
  float* ws; int* tickets;
  int S, QH, KVH, HD, NS;
  int cluster;                                 // the NS slices of a (sequence, KV head) are one thread-block cluster
  float scale;
  long long out_ld;
  int* status;
};

__global__ void __launch_bounds__(TC_THREADS) decode_attn_tc_kernel(const __grid_constant__ TcParams p) {
  using namespace sm100;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;                          // 2 boxes: head dims 0-63, 64-127
  uint8_t* sV = sK + 2 * TC_TILE;
  uint8_t* sQ = sV + 2 * TC_TILE;              // 2 boxes of [16 rows x 128 B]
  uint8_t* sP = sQ + 2 * 2048;                 // 2 boxes of [16 rows x 128 B]: positions 0-63, 64-127
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + 2 * 2048);     // load, scores, contexts
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3);
  float* red = reinterpret_cast<float*>(tmem_slot + 2);            // [4 warps][MAXG]
  float* sm_m = red + 4 * MAXG;
  float* sm_l = sm_m + MAXG;
  float* f_m = reinterpret_cast<float*>(sQ);   // merge scratch, MAXG * TP floats each: the operand boxes are dead by then
  float* f_l = reinterpret_cast<float*>(sP);
  __shared__ int s_last;

  const int G = p.QH / p.KVH, HD = p.HD, NS = p.NS;
  const int b = blockIdx.x / p.KVH, kvh = blockIdx.x % p.KVH, z = blockIdx.y;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  volatile int* status = p.status;

  if (tid == 0) {
    mbar_init(&bars[0], 1); mbar_init(&bars[1], 1); mbar_init(&bars[2], 1);
    fence_barrier_init();
  }
  if (warp == 0) { tmem_alloc(tmem_slot, 64); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  loom::pdl_trigger();
  loom::pdl_wait();                            // the new token's K / V rows and Q come from the previous kernels

  long long n = *p.pos + 1;
  if (n > p.S) n = p.S;
  if (n < 0) n = 0;
  int chunk = (int)((n + NS - 1) / NS);
  chunk = (chunk + 63) & ~63;                  // whole 64-position blocks, at most one 128-position tile (host-checked)
  const int lo = z * chunk;
  int hi = lo + chunk;
  if (hi > n) hi = (int)n;
  const int cnt = hi > lo ? hi - lo : 0;
  const int per = 2 * G + 2 * G * HD;
  // partial state of this slice: in the workspace, or (cluster launch) in this CTA's shared memory, where the other
  // CTAs of the cluster read it; the K tile it overlays is dead once the last MMA batch has completed
  float* wsb = p.cluster ? reinterpret_cast<float*>(sK) : p.ws + ((long long)blockIdx.x * NS + z) * per;
  bool ok = true;

  if (cnt > 0) {
    if (tid == 0) {
      mbar_expect_tx(&bars[0], 4 * TC_TILE + 2 * 2048);
      tma_load_3d(sQ, &p.q, &bars[0], 0, kvh * G, b);
      tma_load_3d(sQ + 2048, &p.q, &bars[0], 64, kvh * G, b);
      tma_load_4d(sK, &p.k, &bars[0], 0, kvh, lo, b);
      tma_load_4d(sK + TC_TILE, &p.k, &bars[0], 64, kvh, lo, b);
      tma_load_4d(sV, &p.v, &bars[0], 0, kvh, lo, b);
      tma_load_4d(sV + TC_TILE, &p.v, &bars[0], 64, kvh, lo, b);
    }
    ok = mbar_wait(&bars[0], 0, status, 121);
    // rows past the slice hold other positions' (or no) data: they get probability zero, and zero times a non-finite
    // leftover would still poison the sums, so they are cleared before the tensor core reads the tiles as operands
    if (ok && tid >= cnt) {
      const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        uint4* rk = reinterpret_cast<uint4*>(sK + j * TC_TILE + tid * 128);
        uint4* rv = reinterpret_cast<uint4*>(sV + j * TC_TILE + tid * 128);
#pragma unroll
        for (int c = 0; c < 8; ++c) { rk[c] = zero; rv[c] = zero; }
      }
    }
    fence_proxy_async();
    __syncthreads();
    const int ksteps = (HD + 15) >> 4;
    if (ok && tid == 0) {
      // S^T[128 positions, 16] = K_tile . Q^T
      constexpr uint32_t idesc = make_idesc_bf16(128, TC_NPAD, 0, 0);
      for (int ks = 0; ks < ksteps; ++ks) {
        const uint32_t off = (ks >> 2) * TC_TILE + (ks & 3) * 32;
        const uint32_t qoff = (ks >> 2) * 2048 + (ks & 3) * 32;
        mma_bf16_ss(tmem_base, make_smem_desc_sw128(smem_u32(sK) + off, 0, 1024),
                    make_smem_desc_sw128(smem_u32(sQ) + qoff, 0, 1024), idesc, ks > 0 ? 1u : 0u);
      }
      mma_commit(&bars[1]);
    }
    ok = ok && mbar_wait(&bars[1], 0, status, 122);
    tc_fence_after();
    // softmax over the slice: thread == position
    float sc[MAXG];
    {
      uint32_t r[16];
      tmem_ld_32x16(tmem_base + (uint32_t(warp * 32) << 16), r);
      tmem_ld_wait();
#pragma unroll
      for (int g = 0; g < MAXG; ++g) sc[g] = (g < G && tid < cnt) ? __uint_as_float(r[g]) * p.scale : -INFINITY;
    }
#pragma unroll
    for (int g = 0; g < MAXG; ++g) {
      float mx = sc[g];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      if (lane == 0) red[warp * MAXG + g] = mx;
    }
    __syncthreads();
    if (tid < MAXG) sm_m[tid] = fmaxf(fmaxf(red[tid], red[MAXG + tid]), fmaxf(red[2 * MAXG + tid], red[3 * MAXG + tid]));
    __syncthreads();
    const int kb = tid >> 6, kk = tid & 63;
#pragma unroll
    for (int g = 0; g < MAXG; ++g) {
      float e = 0.f;
      if (g < G) {
        e = __expf(sc[g] - sm_m[g]);             // masked position: exp(-inf) = 0
        // P^T as a K-major operand: row g, position kk of 64-position block kb, 16-byte chunks swizzled by the row
        *reinterpret_cast<bf16*>(sP + kb * 2048 + g * 128 + (((kk >> 3) ^ (g & 7)) << 4) + (kk & 7) * 2) = __float2bfloat16(e);
      }
      float sum = e;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      if (lane == 0) red[warp * MAXG + g] = sum;
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    if (tid < MAXG) sm_l[tid] = red[tid] + red[MAXG + tid] + red[2 * MAXG + tid] + red[3 * MAXG + tid];
    if (ok && tid == 0) {
      tc_fence_after();
      // O_v^T[HD, 16] = V_tile^T . P^T and O_k^T = K_tile^T . P^T: the tiles as MN-major A operands (64-wide head-dim
      // chunks one box apart), 16 positions per instruction
      constexpr uint32_t idesc = make_idesc_bf16(128, TC_NPAD, 1, 0);
      const int psteps = (cnt + 15) >> 4;
      for (int ks = 0; ks < psteps; ++ks) {
        const uint64_t dp = make_smem_desc_sw128(smem_u32(sP) + (ks >> 2) * 2048 + (ks & 3) * 32, 0, 1024);
        mma_bf16_ss(tmem_base + 16, make_smem_desc_sw128(smem_u32(sV) + ks * 2048, TC_TILE, 1024), dp, idesc, ks > 0 ? 1u : 0u);
        mma_bf16_ss(tmem_base + 32, make_smem_desc_sw128(smem_u32(sK) + ks * 2048, TC_TILE, 1024), dp, idesc, ks > 0 ? 1u : 0u);
      }
      mma_commit(&bars[2]);
    }
    ok = ok && mbar_wait(&bars[2], 0, status, 123);
    tc_fence_after();
    __syncthreads();                           // sm_l visible
    // thread == head dim: 16 query columns of both contexts
    uint32_t ov[16], okk[16];
    tmem_ld_32x16(tmem_base + (uint32_t(warp * 32) << 16) + 16, ov);
    tmem_ld_32x16(tmem_base + (uint32_t(warp * 32) << 16) + 32, okk);
    tmem_ld_wait();
    if (tid < HD) {
      if (NS == 1) {
#pragma unroll
        for (int g = 0; g < MAXG; ++g) {
          if (g < G) {
            const float inv = 1.f / sm_l[g];
            const long long o = (long long)b * p.out_ld + (long long)(kvh * G + g) * HD + tid;
            p.out_c[o] = __float2bfloat16(__uint_as_float(ov[g]) * inv);
            p.out_k[o] = __float2bfloat16(__uint_as_float(okk[g]) * inv);
          }
        }
      } else {
#pragma unroll
        for (int g = 0; g < MAXG; ++g) {
          if (g < G) {
            wsb[2 * G + g * HD + tid] = __uint_as_float(ov[g]);
            wsb[2 * G + G * HD + g * HD + tid] = __uint_as_float(okk[g]);
          }
        }
      }
    }
  } else if (NS > 1) {
    for (int i = tid; i < 2 * G * HD; i += TC_THREADS) wsb[2 * G + i] = 0.f;       // an empty slice leaves zeros
  }

  if (NS > 1 && p.cluster) {
    // merge through distributed shared memory: no global partial states, no fence, no ticket.  Every CTA gathers the
    // softmax statistics of all slices, then sums and stores its share of the (head, dim) outputs.
    if (tid < G) { wsb[tid] = cnt > 0 ? sm_m[tid] : -INFINITY; wsb[G + tid] = cnt > 0 ? sm_l[tid] : 0.f; }
    __syncthreads();
    cluster_arrive();
    cluster_wait();
    const uint32_t local = smem_u32(wsb);
    const int crank = (int)cluster_ctarank();
    for (int i = tid; i < G * NS; i += TC_THREADS) {
      const int g = i / NS, zz = i - g * NS;
      const uint32_t a = mapa_shared(local, zz);
      f_m[i] = ld_shared_cluster_f32(a + g * 4);
      f_l[i] = ld_shared_cluster_f32(a + (G + g) * 4);
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
    for (int pidx = crank + NS * tid; pidx < G * HD; pidx += NS * TC_THREADS) {
      const int g = pidx / HD, dd = pidx - g * HD;
      float v = 0.f, k = 0.f;
      for (int zz = 0; zz < NS; ++zz) {
        const uint32_t a = mapa_shared(local, zz);
        const float f = f_m[g * NS + zz];
        v = fmaf(ld_shared_cluster_f32(a + (2 * G + g * HD + dd) * 4), f, v);
        k = fmaf(ld_shared_cluster_f32(a + (2 * G + G * HD + g * HD + dd) * 4), f, k);
      }
      const float inv = sm_l[g];
      const long long o = (long long)b * p.out_ld + (long long)(kvh * G + g) * HD + dd;
      p.out_c[o] = __float2bfloat16(v * inv);
      p.out_k[o] = __float2bfloat16(k * inv);
    }
    cluster_arrive();                          // nobody leaves while its shared memory may still be read
    cluster_wait();
  } else if (NS > 1) {
    if (tid < G) { wsb[tid] = cnt > 0 ? sm_m[tid] : -INFINITY; wsb[G + tid] = cnt > 0 ? sm_l[tid] : 0.f; }
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = atomicAdd(p.tickets + blockIdx.x, 1) == NS - 1;
    __syncthreads();
    if (s_last) {
      __threadfence();
      merge_slices(p.ws + (long long)blockIdx.x * NS * per, per, NS, G, HD, f_m, f_l, sm_l, p.out_c, p.out_k,
                   (long long)b * p.out_ld + (long long)kvh * G * HD);
      if (tid == 0) p.tickets[blockIdx.x] = 0;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, 64);
}

}  // namespace

// floats of workspace for NS position slices: the partial states, then one ticket counter per (sequence, KV head).
// The caller zeroes the workspace once; every launch leaves the counters at zero.
extern "C" int loom_decode_attn_workspace_floats(int B, int QH, int KVH, int HD, int NS) {
  const int G = QH / KVH;
  return B * KVH * NS * (2 * G + 2 * G * HD) + B * KVH;
}

// q and out_c / out_k rows of sequence b start at b * q_ld resp. b * out_ld elements (QH * HD for dense [B,QH,HD]).
// `status`: device word that a bounded wait of the tensor-core variant sets when it gives up (may be null).
// LOOM_DECODE_ATTN=simt forces the CUDA-core variant.
extern "C" int loom_decode_attn(const void* q, const void* kc, const void* vc, const long long* pos, void* out_c, void* out_k,
                                float* ws, int B, int S, int QH, int KVH, int HD, int NS, long long out_ld, long long q_ld,
                                int* status, cudaStream_t st) {
  const int G = QH / KVH;
  if (HD % 8 || HD > 128 || G < 1 || G > MAXG || QH % KVH || NS < 1 || NS > TP || (out_ld & 1)) return -1;
  int* tickets = reinterpret_cast<int*>(ws + (size_t)B * KVH * NS * (2 * G + 2 * G * HD));
  dim3 grid(B * KVH, NS);
  static int simt = -1;
  if (simt < 0) { const char* e = getenv("LOOM_DECODE_ATTN"); simt = (e != nullptr && e[0] == 's') ? 1 : 0; }
  const int slice = (((S + NS - 1) / NS) + 63) & ~63;
  const bool aligned = !(reinterpret_cast<uintptr_t>(q) & 15) && !(reinterpret_cast<uintptr_t>(kc) & 15) &&
                       !(reinterpret_cast<uintptr_t>(vc) & 15) && !(q_ld & 7);
  if (!simt && slice <= 128 && aligned && (long long)slice * NS >= S) {
    static TcParams p;
    memset(&p, 0, sizeof(p));
    const bool maps = tma_host::make_3d_bf16(&p.q, q, (uint64_t)B, (uint64_t)QH, (uint64_t)HD, (uint64_t)HD, (uint64_t)q_ld, 64, TC_NPAD) &&
                      tma_host::make_4d_bf16(&p.k, kc, (uint64_t)HD, (uint64_t)KVH, (uint64_t)S, (uint64_t)B, (uint64_t)HD,
                                             (uint64_t)KVH * HD, (uint64_t)S * KVH * HD, 64, 1, 128, 1) &&
                      tma_host::make_4d_bf16(&p.v, vc, (uint64_t)HD, (uint64_t)KVH, (uint64_t)S, (uint64_t)B, (uint64_t)HD,
                                             (uint64_t)KVH * HD, (uint64_t)S * KVH * HD, 64, 1, 128, 1);
    if (maps) {
      p.pos = pos; p.out_c = (bf16*)out_c; p.out_k = (bf16*)out_k; p.ws = ws; p.tickets = tickets;
      p.S = S; p.QH = QH; p.KVH = KVH; p.HD = HD; p.NS = NS; p.scale = rsqrtf((float)HD); p.out_ld = out_ld; p.status = status;
      const size_t shm = 4 * TC_TILE + 4 * 2048 + 64 + (4 * MAXG + 2 * MAXG) * sizeof(float) + 1024;   // 73.3 KB: three CTAs per SM
      static bool configured = false;
      if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(decode_attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shm);
        if (e != cudaSuccess) return (int)e;
        configured = true;
      }
      // up to eight slices: one cluster per (sequence, KV head), merged through distributed shared memory
      // (LOOM_DECODE_ATTN_CLUSTER=0 keeps the workspace + ticket merge)
      static int want_cluster = -1;
      if (want_cluster < 0) { const char* e = getenv("LOOM_DECODE_ATTN_CLUSTER"); want_cluster = (e != nullptr && e[0] == '0') ? 0 : 1; }
      static int sms = 0;
      if (sms == 0) { int dev = 0; cudaGetDevice(&dev); cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev); }
      // (only while all CTAs fit the GPU at once: with more, co-scheduling whole clusters costs more than the merge saves:
      // 1.13 against 1.03 ms per step at 64 sequences, 0.492 against 0.512 ms at one)
      if (want_cluster && NS > 1 && NS <= 8 && B * KVH * NS <= sms) {
        p.cluster = 1;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid; cfg.blockDim = dim3(TC_THREADS); cfg.dynamicSmemBytes = shm; cfg.stream = st;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = NS; attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr; cfg.numAttrs = loom::pdl_enabled() ? 2 : 1;
        return (int)cudaLaunchKernelEx(&cfg, decode_attn_tc_kernel, p);
      }
      return (int)loom::launch_pdl(decode_attn_tc_kernel, grid, dim3(TC_THREADS), shm, st, p);
    }
  }
  const size_t shm = ((size_t)G * HD + (size_t)G * TP + 32 + 3 * MAXG) * sizeof(float) + (size_t)2 * TP * (HD + 8) * sizeof(bf16);
  if (shm > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(decode_attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shm);
    if (e != cudaSuccess) return (int)e;
  }
  return (int)loom::launch_pdl(decode_attn_kernel, grid, dim3(THREADS), shm, st, (const bf16*)q, (const bf16*)kc, (const bf16*)vc, pos,
                               (bf16*)out_c, (bf16*)out_k, ws, tickets, S, QH, KVH, HD, NS, rsqrtf((float)HD), out_ld, q_ld);
}
