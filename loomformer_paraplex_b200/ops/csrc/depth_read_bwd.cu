// Depth-attention backward, organised per history slot.
//
// Sublayer `sub` of a chunk reads history slots 0..sub with a softmax over slots:
//     w[sub,s] = exp(<q_sub, k_s>/sqrt(HD) - lse_sub),   m_sub = sum_s w[sub,s] v_s .
// A gradient pass organised per sublayer has to add every sublayer's contribution into fp32
// accumulators of ALL earlier slots -- read-modify-write traffic that grows with the square of the
// depth (about 20 bytes per element per (sublayer, slot) pair).  The slot's gradient is only consumed
// when the backward sweep reaches the layer that produced the slot, and by then every sublayer that
// reads it has already delivered its output gradient dm_sub.  So the sweep stores dm_sub (bf16) and
// the per-row scalar dd_sub = <dm_sub, m_sub>, and ONE launch per slot forms
//     dv_s = sum_{sub>=s} w[sub,s] dm_sub ,   dk_s = sum_{sub>=s} dsc[sub,s] q_sub / sqrt(HD),
//     dsc[sub,s] = w[sub,s] (<dm_sub, v_s> - dd_sub),
// reading k_s, v_s once, each dm_sub once (2 bytes per element per pair) and writing dk_s, dv_s once,
// with no accumulator in memory.  The query gradients gq[sub] += sum_rows dsc[sub,s] k_s / sqrt(HD)
// are reduced in registers by a block that serves a single head, then flushed once.
//
// The reference computes the same quantities with one kernel per sublayer over all earlier slots
// (reference kernels/depth_attn/depth_attn_kernel.cuh:515-651).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>
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

// dm = a (+ b) stored as bf16, dd = <dm, m> per (row, head).  G lanes per (row, head), 8 dims per lane.
template <int G>
__global__ void __launch_bounds__(256) dread_stage_kernel(const bf16* __restrict__ a, const bf16* __restrict__ b,
                                                          const bf16* __restrict__ mo, bf16* __restrict__ dm,
                                                          float* __restrict__ dd, const float* __restrict__ lse_in,
                                                          float* __restrict__ lse_out, long long MQ, int HD) {
  const long long gid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) / G;
  const int l = threadIdx.x % G;
  if (gid >= MQ) return;
  const unsigned mask = __activemask();
  float s = 0.f;
  if (l * 8 < HD) {
    const long long base = gid * HD + l * 8;
    float x[8], y[8], m[8];
    unpack8(*reinterpret_cast<const uint4*>(a + base), x);
    if (b) {
      unpack8(*reinterpret_cast<const uint4*>(b + base), y);
#pragma unroll
      for (int i = 0; i < 8; ++i) x[i] += y[i];
    }
    const uint4 packed = pack8(x);
    *reinterpret_cast<uint4*>(dm + base) = packed;
    unpack8(packed, x);                       // dd must see the rounded values the slot kernel will read
    unpack8(*reinterpret_cast<const uint4*>(mo + base), m);
#pragma unroll
    for (int i = 0; i < 8; ++i) s += x[i] * m[i];
  }
#pragma unroll
  for (int o = G / 2; o > 0; o >>= 1) s += __shfl_xor_sync(mask, s, o, G);
  if (l == 0) {
    dd[gid] = s;
    if (lse_in) lse_out[gid] = lse_in[gid];
  }
}

// grid: (row blocks, QH).  q_all [S,QH,HD] fp32; dm_all [S,M,QH,HD] bf16; lse_all, dd_all [S,M,QH] fp32;
// hk, hv: the slot's K and V [M,QH,HD] bf16; dk, dv out [M,QH,HD] bf16; gq_all [S,QH,HD] fp32 (+=).
//
// A block serves one head and walks over tiles of TILE rows.  Phase 1: each G-lane group keeps one row's k, v and
// the two accumulators in registers and loops over the reading sublayers; the scalar dsc[row][sub] and the row's k
// go to shared memory.  Phase 2: the block re-maps to (sublayer, dim) pairs and adds sum_rows dsc * k into
// per-thread registers, so the query gradients need neither shared-memory atomics nor per-row global traffic;
// they leave the block once, at the end.
// MAX_PAIRS is the number of (sublayer, dim) pairs per thread: 10 covers 20 sublayers of 128 dims, 20 covers deep and
// narrow stacks (65 sublayers of 64 dims).
template <int G, int MAX_PAIRS>
__global__ void __launch_bounds__(256) dread_slot_bwd_kernel(const float* __restrict__ q_all, const bf16* __restrict__ hk,
                                                             const bf16* __restrict__ hv, const bf16* __restrict__ dm_all,
                                                             const float* __restrict__ lse_all,
                                                             const float* __restrict__ dd_all, bf16* __restrict__ dk,
                                                             bf16* __restrict__ dv, float* __restrict__ gq_all, int sub0,
                                                             int S, int M, int QH, int HD, float scale, long long in_ld,
                                                             long long out_ld) {
  constexpr int NGRP = 256 / G;
  constexpr int TILE = 2 * NGRP;              // rows per tile: every group takes two
  extern __shared__ float sh[];               // [nsub][HD] queries | [TILE][nsub] dsc | [TILE][HD] k rows
  const int g = blockIdx.y;
  const int nsub = S - sub0;
  float* sq = sh;
  float* sd = sq + nsub * HD;
  float* sk = sd + TILE * nsub;
  for (int i = threadIdx.x; i < nsub * HD; i += blockDim.x) {
    const int jj = i / HD, c = i % HD;
    sq[i] = q_all[((long long)(sub0 + jj) * QH + g) * HD + c];
  }
  float gacc[MAX_PAIRS];
#pragma unroll
  for (int i = 0; i < MAX_PAIRS; ++i) gacc[i] = 0.f;
  __syncthreads();
  const int l = threadIdx.x % G, grp = threadIdx.x / G;
  const bool act = l * 8 < HD;
  const long long MQ = (long long)M * QH;
  const int npairs = nsub * HD;
  for (int m0 = blockIdx.x * TILE; m0 < M; m0 += gridDim.x * TILE) {
#pragma unroll 1
    for (int rr = 0; rr < 2; ++rr) {
      const int row = grp * 2 + rr;
      const int m = m0 + row;
      const bool live = m < M;                 // uniform within a group
      const long long rh = (long long)(live ? m : 0) * QH + g;
      const long long base = rh * HD + l * 8;                                     // dm rows are densely packed
      const long long hoff = (long long)g * HD + l * 8;
      const long long ibase = (long long)(live ? m : 0) * in_ld + hoff, obase = (long long)(live ? m : 0) * out_ld + hoff;
      float kf[8], vf[8], ak[8], av[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) { kf[i] = 0.f; vf[i] = 0.f; ak[i] = 0.f; av[i] = 0.f; }
      if (act && live) {
        unpack8(*reinterpret_cast<const uint4*>(hk + ibase), kf);
        unpack8(*reinterpret_cast<const uint4*>(hv + ibase), vf);
      }
      if (act) {
#pragma unroll
        for (int i = 0; i < 8; ++i) sk[row * HD + l * 8 + i] = kf[i];
      }
      // The loop over reading sublayers is latency-bound (one dependent chain of load -> reduce -> exp per sublayer), so
      // the loads of PF sublayers are issued together before any of them is consumed.
      constexpr int PF = 4;
      for (int j0 = 0; j0 < nsub; j0 += PF) {
        uint4 raw[PF];
        float lse_v[PF], dd_v[PF];
#pragma unroll
        for (int u = 0; u < PF; ++u) {
          const int jj = j0 + u;
          const long long so = (long long)(sub0 + (jj < nsub ? jj : nsub - 1));
          raw[u] = make_uint4(0u, 0u, 0u, 0u);
          if (act && live) raw[u] = *reinterpret_cast<const uint4*>(dm_all + so * MQ * HD + base);
          lse_v[u] = live ? lse_all[so * MQ + rh] : 0.f;
          dd_v[u] = live ? dd_all[so * MQ + rh] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < PF; ++u) {
          const int jj = j0 + u;
          if (jj < nsub) {                               // uniform across the block
            float dmf[8], qv[8];
            unpack8(raw[u], dmf);
#pragma unroll
            for (int i = 0; i < 8; ++i) qv[i] = act ? sq[jj * HD + l * 8 + i] : 0.f;
            float d = 0.f, dvv = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) { d += qv[i] * kf[i]; dvv += dmf[i] * vf[i]; }
#pragma unroll
            for (int o = G / 2; o > 0; o >>= 1) {
              d += __shfl_xor_sync(0xffffffffu, d, o, G);
              dvv += __shfl_xor_sync(0xffffffffu, dvv, o, G);
            }
            float w = 0.f, dsc = 0.f;
            if (live) {
              w = __expf(d * scale - lse_v[u]);
              dsc = w * (dvv - dd_v[u]) * scale;
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) { ak[i] += dsc * qv[i]; av[i] += w * dmf[i]; }
            if (l == 0) sd[row * nsub + jj] = dsc;
          }
        }
      }
      if (act && live) {
        *reinterpret_cast<uint4*>(dk + obase) = pack8(ak);
        *reinterpret_cast<uint4*>(dv + obase) = pack8(av);
      }
    }
    __syncthreads();
    // phase 2: query-gradient partials of this tile
#pragma unroll
    for (int pi = 0; pi < MAX_PAIRS; ++pi) {
      const int pidx = threadIdx.x + pi * 256;
      if (pidx < npairs) {
        const int jj = pidx / HD, c = pidx % HD;
        float a = 0.f;
#pragma unroll 8
        for (int r = 0; r < TILE; ++r) a += sd[r * nsub + jj] * sk[r * HD + c];
        gacc[pi] += a;
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int pi = 0; pi < MAX_PAIRS; ++pi) {
    const int pidx = threadIdx.x + pi * 256;
    if (pidx < npairs && gacc[pi] != 0.f) {
      const int jj = pidx / HD, c = pidx % HD;
      atomicAdd(gq_all + ((long long)(sub0 + jj) * QH + g) * HD + c, gacc[pi]);
    }
  }
}

// Same kernel with G * 4 NV == HD exactly: a lane owns NV vectors of four dims (12 dims of a 96-wide head on 8 lanes
// instead of 8 dims on 16 lanes of which 4 idle), so no lane is idle, a warp serves four rows instead of two, the
// reductions are one shuffle level shorter and the per-(row, sublayer) overhead (exponential, addressing, shuffles) is
// spread over half again as many dims.  The loop body below is about 125 instructions per (row, sublayer) for 8 lanes
// against about 160 for 16 lanes above.
__device__ __forceinline__ void unpack4(const uint2& u, float* f) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
  const float2 a = __bfloat1622float2(p[0]), b = __bfloat1622float2(p[1]);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}
__device__ __forceinline__ uint2 pack4(const float* f) {
  uint2 u;
  __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&u);
  p[0] = __floats2bfloat162_rn(f[0], f[1]);
  p[1] = __floats2bfloat162_rn(f[2], f[3]);
  return u;
}

// staging with G * 4 NV == HD exactly (no idle lanes, see the slot kernel below)
template <int G, int NV>
__global__ void __launch_bounds__(256) dread_stage_wide_kernel(const bf16* __restrict__ a, const bf16* __restrict__ b,
                                                               const bf16* __restrict__ mo, bf16* __restrict__ dm,
                                                               float* __restrict__ dd, const float* __restrict__ lse_in,
                                                               float* __restrict__ lse_out, long long MQ, int HD) {
  constexpr int DPL = 4 * NV;
  const long long gid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) / G;
  const int l = threadIdx.x % G;
  if (gid >= MQ) return;
  const unsigned mask = __activemask();
  const long long base = gid * HD + l * DPL;
  float s = 0.f;
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    float x[4], y[4], m[4];
    unpack4(*reinterpret_cast<const uint2*>(a + base + 4 * v), x);
    if (b) {
      unpack4(*reinterpret_cast<const uint2*>(b + base + 4 * v), y);
#pragma unroll
      for (int i = 0; i < 4; ++i) x[i] += y[i];
    }
    const uint2 packed = pack4(x);
    *reinterpret_cast<uint2*>(dm + base + 4 * v) = packed;
    unpack4(packed, x);                       // dd must see the rounded values the slot kernel will read
    unpack4(*reinterpret_cast<const uint2*>(mo + base + 4 * v), m);
#pragma unroll
    for (int i = 0; i < 4; ++i) s += x[i] * m[i];
  }
#pragma unroll
  for (int o = G / 2; o > 0; o >>= 1) s += __shfl_xor_sync(mask, s, o, G);
  if (l == 0) {
    dd[gid] = s;
    if (lse_in) lse_out[gid] = lse_in[gid];
  }
}

template <int G, int NV>
__global__ void __launch_bounds__(256, 2) dread_slot_bwd_wide_kernel(
    const float* __restrict__ q_all, const bf16* __restrict__ hk, const bf16* __restrict__ hv, const bf16* __restrict__ dm_all,
    const float* __restrict__ lse_all, const float* __restrict__ dd_all, bf16* __restrict__ dk, bf16* __restrict__ dv,
    float* __restrict__ gq_all, int sub0, int S, int M, int QH, int HD, float scale, long long in_ld, long long out_ld) {
  constexpr int DPL = 4 * NV;
  constexpr int NGRP = 256 / G;
  constexpr int TILE = 2 * NGRP;              // rows per tile: every group takes two
  constexpr int NACC = 20;                    // query-gradient accumulators per thread
  extern __shared__ float sh[];               // [nsub][HD] queries | [TILE][nsubp] dsc | [TILE][HD] k rows
  const int g = blockIdx.y;
  const int nsub = S - sub0;
  const int nsubp = (nsub + 3) & ~3;          // dsc rows padded to whole float4s (the pad stays zero)
  float* sq = sh;
  float* sd = sq + nsub * HD;
  float* sk = sd + TILE * nsubp;
  for (int i = threadIdx.x; i < nsub * HD; i += blockDim.x) {
    const int jj = i / HD, c = i % HD;
    sq[i] = q_all[((long long)(sub0 + jj) * QH + g) * HD + c];
  }
  for (int i = threadIdx.x; i < TILE * nsubp; i += blockDim.x) sd[i] = 0.f;
  float gacc[NACC];
#pragma unroll
  for (int i = 0; i < NACC; ++i) gacc[i] = 0.f;
  // Query gradients gq[sub, c] = sum_rows dsc[row, sub] k[row, c].  Up to 20 reading sublayers: a thread owns one dim c
  // and a share of the tile's rows and keeps one accumulator per sublayer, so a k value is loaded once per row and the
  // dsc row arrives as float4s (one shared-memory load per four multiply-adds).  More sublayers (deep, narrow stacks):
  // a thread owns up to 20 (sublayer, dim) pairs, two loads per multiply-add.
  const bool per_dim = nsub <= NACC;
  const int parts = 256 / HD, part = threadIdx.x / HD, cdim = threadIdx.x - part * HD;
  __syncthreads();
  const int l = threadIdx.x % G, grp = threadIdx.x / G;
  const long long MQ = (long long)M * QH;
  const int npairs = nsub * HD;
  for (int m0 = blockIdx.x * TILE; m0 < M; m0 += gridDim.x * TILE) {
#pragma unroll 1
    for (int rr = 0; rr < 2; ++rr) {
      const int row = grp * 2 + rr;
      const int m = m0 + row;
      const bool live = m < M;                 // uniform within a group
      const long long rh = (long long)(live ? m : 0) * QH + g;
      const long long base = rh * HD + l * DPL;                                   // dm rows are densely packed
      const long long hoff = (long long)g * HD + l * DPL;
      const long long ibase = (long long)(live ? m : 0) * in_ld + hoff, obase = (long long)(live ? m : 0) * out_ld + hoff;
      float kf[DPL], vf[DPL], ak[DPL], av[DPL];
#pragma unroll
      for (int i = 0; i < DPL; ++i) { kf[i] = 0.f; vf[i] = 0.f; ak[i] = 0.f; av[i] = 0.f; }
      if (live) {
#pragma unroll
        for (int v = 0; v < NV; ++v) {
          unpack4(*reinterpret_cast<const uint2*>(hk + ibase + 4 * v), kf + 4 * v);
          unpack4(*reinterpret_cast<const uint2*>(hv + ibase + 4 * v), vf + 4 * v);
        }
      }
#pragma unroll
      for (int v = 0; v < NV; ++v)
        *reinterpret_cast<float4*>(sk + row * HD + l * DPL + 4 * v) = make_float4(kf[4 * v], kf[4 * v + 1], kf[4 * v + 2], kf[4 * v + 3]);
      // the loop over reading sublayers is one dependent chain of load -> reduce -> exp per sublayer: the loads of PF
      // sublayers are issued together
#ifndef LOOM_SLOT_PF
#define LOOM_SLOT_PF 3
#endif
      constexpr int PF = LOOM_SLOT_PF;
      for (int j0 = 0; j0 < nsub; j0 += PF) {
        uint2 raw[PF][NV];
        float lse_v[PF], dd_v[PF];
#pragma unroll
        for (int u = 0; u < PF; ++u) {
          const int jj = j0 + u;
          const long long so = (long long)(sub0 + (jj < nsub ? jj : nsub - 1));
#pragma unroll
          for (int v = 0; v < NV; ++v)
            raw[u][v] = live ? *reinterpret_cast<const uint2*>(dm_all + so * MQ * HD + base + 4 * v) : make_uint2(0u, 0u);
          lse_v[u] = live ? lse_all[so * MQ + rh] : 0.f;
          dd_v[u] = live ? dd_all[so * MQ + rh] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < PF; ++u) {
          const int jj = j0 + u;
          if (jj < nsub) {                               // uniform across the block
            float dmf[DPL], qv[DPL];
#pragma unroll
            for (int v = 0; v < NV; ++v) {
              unpack4(raw[u][v], dmf + 4 * v);
              const float4 qq = *reinterpret_cast<const float4*>(sq + jj * HD + l * DPL + 4 * v);
              qv[4 * v] = qq.x; qv[4 * v + 1] = qq.y; qv[4 * v + 2] = qq.z; qv[4 * v + 3] = qq.w;
            }
            float d = 0.f, dvv = 0.f;
#pragma unroll
            for (int i = 0; i < DPL; ++i) { d += qv[i] * kf[i]; dvv += dmf[i] * vf[i]; }
#pragma unroll
            for (int o = G / 2; o > 0; o >>= 1) {
              d += __shfl_xor_sync(0xffffffffu, d, o, G);
              dvv += __shfl_xor_sync(0xffffffffu, dvv, o, G);
            }
            float w = 0.f, dsc = 0.f;
            if (live) {
              w = __expf(d * scale - lse_v[u]);
              dsc = w * (dvv - dd_v[u]) * scale;
            }
#pragma unroll
            for (int i = 0; i < DPL; ++i) { ak[i] += dsc * qv[i]; av[i] += w * dmf[i]; }
            if (l == 0) sd[row * nsubp + jj] = dsc;
          }
        }
      }
      if (live) {
#pragma unroll
        for (int v = 0; v < NV; ++v) {
          *reinterpret_cast<uint2*>(dk + obase + 4 * v) = pack4(ak + 4 * v);
          *reinterpret_cast<uint2*>(dv + obase + 4 * v) = pack4(av + 4 * v);
        }
      }
    }
    __syncthreads();
    // phase 2: query-gradient partials of this tile
    if (per_dim) {
      if (part < parts) {
        for (int r = part; r < TILE; r += parts) {
          const float kv = sk[r * HD + cdim];
          const float4* dr = reinterpret_cast<const float4*>(sd + r * nsubp);
#pragma unroll
          for (int j4 = 0; j4 < NACC / 4; ++j4) {
            if (4 * j4 < nsub) {
              const float4 s4 = dr[j4];
              gacc[4 * j4] += s4.x * kv; gacc[4 * j4 + 1] += s4.y * kv; gacc[4 * j4 + 2] += s4.z * kv; gacc[4 * j4 + 3] += s4.w * kv;
            }
          }
        }
      }
    } else {
#pragma unroll
      for (int pi = 0; pi < NACC; ++pi) {
        const int pidx = threadIdx.x + pi * 256;
        if (pidx < npairs) {
          const int jj = pidx / HD, c = pidx % HD;
          float a = 0.f;
#pragma unroll 8
          for (int r = 0; r < TILE; ++r) a += sd[r * nsubp + jj] * sk[r * HD + c];
          gacc[pi] += a;
        }
      }
    }
    __syncthreads();
  }
  if (per_dim) {
    if (part < parts) {
#pragma unroll
      for (int jj = 0; jj < NACC; ++jj)
        if (jj < nsub && gacc[jj] != 0.f) atomicAdd(gq_all + ((long long)(sub0 + jj) * QH + g) * HD + cdim, gacc[jj]);
    }
  } else {
#pragma unroll
    for (int pi = 0; pi < NACC; ++pi) {
      const int pidx = threadIdx.x + pi * 256;
      if (pidx < npairs && gacc[pi] != 0.f) {
        const int jj = pidx / HD, c = pidx % HD;
        atomicAdd(gq_all + ((long long)(sub0 + jj) * QH + g) * HD + c, gacc[pi]);
      }
    }
  }
}

// -3: the sublayer count is too large for this kernel
template <int G, int NV>
int launch_slot_wide(const float* q_all, const void* hk, const void* hv, const void* dm_all, const float* lse_all,
                     const float* dd_all, void* dk, void* dv, float* gq_all, int sub0, int S, int M, int QH, int HD,
                     long long in_ld, long long out_ld, cudaStream_t st) {
  const int nsub = S - sub0, nsubp = (nsub + 3) & ~3;
  if ((long long)nsub * HD > 256LL * 20) return -3;
  constexpr int TILE = 2 * (256 / G);
  const size_t shm = ((size_t)nsub * HD + (size_t)TILE * nsubp + (size_t)TILE * HD) * sizeof(float);
  if (shm > 100 * 1024) return -3;
  if (shm > 48 * 1024) {
    static size_t configured = 0;
    if (shm > configured) {
      cudaError_t e = cudaFuncSetAttribute(dread_slot_bwd_wide_kernel<G, NV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shm);
      if (e != cudaSuccess) return (int)e;
      configured = shm;
    }
  }
  static int sms = 0;
  if (sms == 0) { int dev = 0; cudaGetDevice(&dev); cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev); }
  int bx = (sms * 2 + QH - 1) / QH;                 // two resident blocks per SM over all heads
  const int need = (M + TILE - 1) / TILE;
  if (bx > need) bx = need;
  if (bx < 1) bx = 1;
  dim3 grid(bx, QH);
  dread_slot_bwd_wide_kernel<G, NV><<<grid, 256, shm, st>>>(q_all, (const bf16*)hk, (const bf16*)hv, (const bf16*)dm_all, lse_all,
                                                           dd_all, (bf16*)dk, (bf16*)dv, gq_all, sub0, S, M, QH, HD,
                                                           rsqrtf((float)HD), in_ld, out_ld);
  return (int)cudaGetLastError();
}

template <int G>
int launch_stage(const void* a, const void* b, const void* mo, void* dm, float* dd, const float* lse_in, float* lse_out,
                 long long MQ, int HD, cudaStream_t st) {
  const long long threads = MQ * G;
  dread_stage_kernel<G><<<(unsigned)((threads + 255) / 256), 256, 0, st>>>((const bf16*)a, (const bf16*)b, (const bf16*)mo,
                                                                            (bf16*)dm, dd, lse_in, lse_out, MQ, HD);
  return (int)cudaGetLastError();
}

template <int G, int MAX_PAIRS>
int launch_slot_mp(const float* q_all, const void* hk, const void* hv, const void* dm_all, const float* lse_all,
                const float* dd_all, void* dk, void* dv, float* gq_all, int sub0, int S, int M, int QH, int HD,
                long long in_ld, long long out_ld, cudaStream_t st) {
  const int nsub = S - sub0;
  constexpr int TILE = 2 * (256 / G);
  const size_t shm = ((size_t)nsub * HD + (size_t)TILE * nsub + (size_t)TILE * HD) * sizeof(float);
  if (shm > 227 * 1024) return -2;
  if (shm > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(dread_slot_bwd_kernel<G, MAX_PAIRS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shm);
    if (e != cudaSuccess) return (int)e;
  }
  static int sms = 0;
  if (sms == 0) { int dev = 0; cudaGetDevice(&dev); cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev); }
  int bx = (sms * 4 + QH - 1) / QH;                 // about four resident blocks per SM over all heads
  const int need = (M + TILE - 1) / TILE;
  if (bx > need) bx = need;
  if (bx < 1) bx = 1;
  dim3 grid(bx, QH);
  dread_slot_bwd_kernel<G, MAX_PAIRS><<<grid, 256, shm, st>>>(q_all, (const bf16*)hk, (const bf16*)hv, (const bf16*)dm_all, lse_all,
                                                   dd_all, (bf16*)dk, (bf16*)dv, gq_all, sub0, S, M, QH, HD,
                                                   rsqrtf((float)HD), in_ld, out_ld);
  return (int)cudaGetLastError();
}

template <int G>
int launch_slot(const float* q_all, const void* hk, const void* hv, const void* dm_all, const float* lse_all,
                const float* dd_all, void* dk, void* dv, float* gq_all, int sub0, int S, int M, int QH, int HD,
                long long in_ld, long long out_ld, cudaStream_t st) {
  const long long pairs = (long long)(S - sub0) * HD;
  if (pairs <= 256LL * 10)
    return launch_slot_mp<G, 10>(q_all, hk, hv, dm_all, lse_all, dd_all, dk, dv, gq_all, sub0, S, M, QH, HD, in_ld, out_ld, st);
  if (pairs <= 256LL * 20)
    return launch_slot_mp<G, 20>(q_all, hk, hv, dm_all, lse_all, dd_all, dk, dv, gq_all, sub0, S, M, QH, HD, in_ld, out_ld, st);
  return -2;
}

}  // namespace

extern "C" int loom_dread_stage(const void* a, const void* b, const void* mo, void* dm, float* dd, const float* lse_in,
                                float* lse_out, long long MQ, int HD, cudaStream_t st) {
  if (HD % 8 || HD > 128 || ((lse_in == nullptr) != (lse_out == nullptr))) return -1;
#define WIDE_S(G_, NV_) do { const long long threads = MQ * G_; \
    dread_stage_wide_kernel<G_, NV_><<<(unsigned)((threads + 255) / 256), 256, 0, st>>>((const bf16*)a, (const bf16*)b, (const bf16*)mo, \
                                                                                        (bf16*)dm, dd, lse_in, lse_out, MQ, HD); \
    return (int)cudaGetLastError(); } while (0)
  if (HD == 96) WIDE_S(8, 3); if (HD == 64) WIDE_S(8, 2); if (HD == 128) WIDE_S(8, 4); if (HD == 48) WIDE_S(4, 3);
  if (HD == 32) WIDE_S(4, 2); if (HD == 24) WIDE_S(2, 3);
#undef WIDE_S
  const int chunks = HD / 8;
  if (chunks <= 2) return launch_stage<2>(a, b, mo, dm, dd, lse_in, lse_out, MQ, HD, st);
  if (chunks <= 4) return launch_stage<4>(a, b, mo, dm, dd, lse_in, lse_out, MQ, HD, st);
  if (chunks <= 8) return launch_stage<8>(a, b, mo, dm, dd, lse_in, lse_out, MQ, HD, st);
  return launch_stage<16>(a, b, mo, dm, dd, lse_in, lse_out, MQ, HD, st);
}

extern "C" int loom_dread_slot_bwd(const float* q_all, const void* hk, const void* hv, const void* dm_all,
                                   const float* lse_all, const float* dd_all, void* dk, void* dv, float* gq_all, int sub0,
                                   int S, int M, int QH, int HD, long long in_ld, long long out_ld, cudaStream_t st) {
  if (HD % 8 || HD > 128 || sub0 < 0 || sub0 >= S) return -1;
  if (in_ld < (long long)QH * HD || out_ld < (long long)QH * HD || in_ld % 8 || out_ld % 8) return -1;
  {
    // head widths that split exactly into 8 / 4 / 2 lanes of 8, 12 or 16 dims take the wide kernel (LOOM_DREAD_BWD=narrow
    // keeps the 8-dims-per-lane kernel)
    static int narrow = -1;
    if (narrow < 0) { const char* e = getenv("LOOM_DREAD_BWD"); narrow = (e != nullptr && e[0] == 'n') ? 1 : 0; }
    int rc = -3;
    if (!narrow) {
#define WIDE(G_, NV_) rc = launch_slot_wide<G_, NV_>(q_all, hk, hv, dm_all, lse_all, dd_all, dk, dv, gq_all, sub0, S, M, QH, HD, in_ld, out_ld, st)
      if (HD == 96) WIDE(8, 3); else if (HD == 64) WIDE(8, 2); else if (HD == 128) WIDE(8, 4); else if (HD == 48) WIDE(4, 3);
      else if (HD == 32) WIDE(4, 2); else if (HD == 24) WIDE(2, 3);
#undef WIDE
    }
    if (rc != -3) return rc;
  }
  const int chunks = HD / 8;
  if (chunks <= 2) return launch_slot<2>(q_all, hk, hv, dm_all, lse_all, dd_all, dk, dv, gq_all, sub0, S, M, QH, HD, in_ld, out_ld, st);
  if (chunks <= 4) return launch_slot<4>(q_all, hk, hv, dm_all, lse_all, dd_all, dk, dv, gq_all, sub0, S, M, QH, HD, in_ld, out_ld, st);
  if (chunks <= 8) return launch_slot<8>(q_all, hk, hv, dm_all, lse_all, dd_all, dk, dv, gq_all, sub0, S, M, QH, HD, in_ld, out_ld, st);
  return launch_slot<16>(q_all, hk, hv, dm_all, lse_all, dd_all, dk, dv, gq_all, sub0, S, M, QH, HD, in_ld, out_ld, st);
}
