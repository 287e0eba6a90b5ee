// Dual-context causal GQA attention, backward (tcgen05 + TMEM + TMA).
//
// Forward:  P = softmax(Q K^T * scale + mask),  O_v = P V,  O_k = P K.
// Backward, per block of 128 keys (one CTA per (batch row, query head), like the forward kernel):
//   S  = Q K^T                              P  = exp(S*scale - lse)
//   dP = dO_v V^T + dO_k K^T                dS = P o (dP - delta) * scale,  delta = rowsum(dO_v o O_v + dO_k o O_k)
//   dQ += dS K                              (TMEM accumulator across key blocks)
//   dV_j = P^T dO_v                         dK_j = dS^T Q + P^T dO_k
// P and dS are written once to shared memory as swizzled bf16 tiles and consumed by the tensor cores both
// as K-major A operands (dQ) and as MN-major A operands (the transposed products), so no transposes are
// materialised.  dK_j / dV_j are added into per-query-head fp32 slabs [B, T, QH, HD]: one CTA owns a
// (batch row, query head) slice of a slab during a launch and launches are stream-ordered, so the
// accumulation needs no atomics and is run-to-run deterministic; the GQA group sum happens when the
// chunk's own rows are finalised (inverse-RoPE kernel).
//
// The reference backward is PyTorch SDPA's, or a recompute that materialises [B,h,Q,S] scores twice
// (reference loomformer.py:3039-3082).
#include "sm100.cuh"
#include "tma_host.h"
#include "loom_c_api.h"

using namespace sm100;

namespace {

constexpr int BQ = 128;
constexpr int BKEY = 128;
constexpr int THREADS = 192;
constexpr int TILE = 16384;

struct Params {
  CUtensorMap q, dov, dok, k, v;     // q / dO tiles come from qkc / dqkc sectors
  const void* qkc; const void* dqkc;
  const float* lse; const int* seg;
  void* dq_attn; float* dk_heads; float* dv_heads;
  int B, QH, KVH, HD, Tc, T, s, e;   // Tc, s, e describe this launch's query tile (<= 128 rows)
  int Tc_total, q0;                  // rows per batch entry in qkc / lse, and the tile's first row among them
  long long row_pitch;
  float scale, scale_log2e;
  int* status;
};

__device__ __forceinline__ uint32_t swz(int row, int chunk) { return row * 128 + ((chunk ^ (row & 7)) << 4); }

__global__ void __launch_bounds__(THREADS, 1) attn_bwd_kernel(const __grid_constant__ Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                 // 2 tiles
  uint8_t* sDOv = sQ + 2 * TILE;      // 2 tiles
  uint8_t* sDOk = sDOv + 2 * TILE;    // 2 tiles
  uint8_t* sK = sDOk + 2 * TILE;      // 2 tiles
  uint8_t* sV = sK + 2 * TILE;        // 2 tiles
  uint8_t* sP = sV + 2 * TILE;        // 2 tiles (keys 0-63 | 64-127)
  uint8_t* sDS = sP + 2 * TILE;       // 2 tiles
  uint64_t* bars = reinterpret_cast<uint64_t*>(sDS + 2 * TILE);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;
  uint64_t* kv_empty = bars + 2;
  uint64_t* sdp_full = bars + 3;
  uint64_t* sdp_empty = bars + 4;
  uint64_t* pds_full = bars + 5;
  uint64_t* pds_empty = bars + 6;
  uint64_t* dkv_full = bars + 7;
  uint64_t* dkv_empty = bars + 8;
  uint64_t* dq_full = bars + 9;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.x / p.QH, qh = blockIdx.x % p.QH;
  const int kvh = qh / (p.QH / p.KVH);
  volatile int* status = p.status;
  const int nblk = (p.e + BKEY - 1) / BKEY;
  const int ksteps = (p.HD + 15) / 16;   // the TMA unit zero-fills columns past HD
  const int hdp = (p.HD <= 64) ? 64 : 128;
  const int ntile = (p.HD > 64) ? 2 : 1;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1); mbar_init(kv_full, 1); mbar_init(kv_empty, 1);
    mbar_init(sdp_full, 1); mbar_init(sdp_empty, 128);
    mbar_init(pds_full, 128); mbar_init(pds_empty, 1);
    mbar_init(dkv_full, 1); mbar_init(dkv_empty, 128); mbar_init(dq_full, 1);
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tS = tmem, tDP = tmem + 128, tDQ = tmem + 256, tDKV = tmem + 384;

  if (warp == 0) {
    if (elect_one()) {
      tma_prefetch_desc(&p.q); tma_prefetch_desc(&p.dov); tma_prefetch_desc(&p.dok);
      tma_prefetch_desc(&p.k); tma_prefetch_desc(&p.v);
      mbar_expect_tx(q_full, 3 * ntile * TILE);
      for (int i = 0; i < ntile; ++i) {
        tma_load_4d(sQ + i * TILE, &p.q, q_full, 64 * i, qh, 0, b * p.Tc_total + p.q0);
        tma_load_4d(sDOk + i * TILE, &p.dok, q_full, 64 * i, qh, 1, b * p.Tc_total + p.q0);
        tma_load_4d(sDOv + i * TILE, &p.dov, q_full, 64 * i, qh, 2, b * p.Tc_total + p.q0);
      }
      for (int j = 0; j < nblk; ++j) {
        if (!mbar_wait(kv_empty, (j & 1) ^ 1, status, 301)) break;
        mbar_expect_tx(kv_full, 2 * ntile * TILE);
        for (int i = 0; i < ntile; ++i) {
          tma_load_4d(sK + i * TILE, &p.k, kv_full, 64 * i, kvh, j * BKEY, b);
          tma_load_4d(sV + i * TILE, &p.v, kv_full, 64 * i, kvh, j * BKEY, b);
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      const uint32_t id_s = make_idesc_bf16(BQ, BKEY, 0, 0);      // S, dP
      const uint32_t id_q = make_idesc_bf16(BQ, hdp, 0, 1);       // dQ = dS K
      const uint32_t id_t = make_idesc_bf16(BKEY, hdp, 1, 1);     // dV, dK (transposed products)
      const uint32_t aQ = smem_u32(sQ), aDOv = smem_u32(sDOv), aDOk = smem_u32(sDOk), aK = smem_u32(sK),
                     aV = smem_u32(sV), aP = smem_u32(sP), aDS = smem_u32(sDS);
      bool ok = mbar_wait(q_full, 0, status, 302);
      for (int j = 0; j < nblk && ok; ++j) {
        if (!mbar_wait(kv_full, j & 1, status, 303)) break;
        if (!mbar_wait(sdp_empty, (j & 1) ^ 1, status, 304)) break;
        tc_fence_after();
        for (int ks = 0; ks < ksteps; ++ks) {
          const uint32_t off = (ks >> 2) * TILE + (ks & 3) * 32;
          mma_bf16_ss(tS, make_smem_desc_sw128(aQ + off, 0, 1024), make_smem_desc_sw128(aK + off, 0, 1024), id_s, ks > 0);
        }
        for (int ks = 0; ks < ksteps; ++ks) {
          const uint32_t off = (ks >> 2) * TILE + (ks & 3) * 32;
          mma_bf16_ss(tDP, make_smem_desc_sw128(aDOv + off, 0, 1024), make_smem_desc_sw128(aV + off, 0, 1024), id_s, ks > 0);
        }
        for (int ks = 0; ks < ksteps; ++ks) {
          const uint32_t off = (ks >> 2) * TILE + (ks & 3) * 32;
          mma_bf16_ss(tDP, make_smem_desc_sw128(aDOk + off, 0, 1024), make_smem_desc_sw128(aK + off, 0, 1024), id_s, 1u);
        }
        mma_commit(sdp_full);
        if (!mbar_wait(pds_full, j & 1, status, 305)) break;
        tc_fence_after();
        // dQ += dS K_j   (A: dS K-major over keys; B: K tile read MN-major)
        for (int ks = 0; ks < BKEY / 16; ++ks)
          mma_bf16_ss(tDQ, make_smem_desc_sw128(aDS + (ks >> 2) * TILE + (ks & 3) * 32, 0, 1024),
                      make_smem_desc_sw128(aK + ks * 2048, TILE, 1024), id_q, (j > 0 || ks > 0) ? 1u : 0u);
        // dV_j = P^T dO_v
        if (!mbar_wait(dkv_empty, ((2 * j) & 1) ^ 1, status, 306)) break;
        tc_fence_after();
        for (int ks = 0; ks < BQ / 16; ++ks)
          mma_bf16_ss(tDKV, make_smem_desc_sw128(aP + ks * 2048, TILE, 1024),
                      make_smem_desc_sw128(aDOv + ks * 2048, TILE, 1024), id_t, ks > 0);
        mma_commit(dkv_full);
        // dK_j = dS^T Q + P^T dO_k
        if (!mbar_wait(dkv_empty, ((2 * j + 1) & 1) ^ 1, status, 307)) break;
        tc_fence_after();
        for (int ks = 0; ks < BQ / 16; ++ks)
          mma_bf16_ss(tDKV, make_smem_desc_sw128(aDS + ks * 2048, TILE, 1024),
                      make_smem_desc_sw128(aQ + ks * 2048, TILE, 1024), id_t, ks > 0);
        for (int ks = 0; ks < BQ / 16; ++ks)
          mma_bf16_ss(tDKV, make_smem_desc_sw128(aP + ks * 2048, TILE, 1024),
                      make_smem_desc_sw128(aDOk + ks * 2048, TILE, 1024), id_t, 1u);
        mma_commit(dkv_full);
        mma_commit(pds_empty);
        mma_commit(kv_empty);
        if (j == nblk - 1) mma_commit(dq_full);
      }
    }
  } else {
    // One element-wise warp per TMEM lane quadrant.  Two warps per quadrant (each taking half of the columns) were
    // measured slower on B200 (1.81 ms against 1.36 ms at 256 x 8 heads, 128 queries, 1024 keys): the additional
    // warps' barrier polling competes with the arithmetic for issue slots.
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const bool row_ok = r < p.Tc;
    const int qpos = p.s + r;
    const int* segrow = p.seg ? p.seg + (long long)b * p.T : nullptr;
    const int my_seg = (segrow && row_ok) ? segrow[qpos] : 0;
    const uint32_t lane_off = uint32_t(quad * 32) << 16;
    const long long row = (long long)b * p.Tc_total + p.q0 + r;
    // delta = rowsum(dO_v o O_v + dO_k o O_k); lse in log2 units
    float delta = 0.f, lse2 = 0.f;
    if (row_ok) {
      const __nv_bfloat16* o = reinterpret_cast<const __nv_bfloat16*>(p.qkc) + row * p.row_pitch + (long long)p.QH * p.HD + qh * p.HD;
      const __nv_bfloat16* g = reinterpret_cast<const __nv_bfloat16*>(p.dqkc) + row * p.row_pitch + (long long)p.QH * p.HD + qh * p.HD;
      const long long sec = (long long)p.QH * p.HD;
      for (int c = 0; c < p.HD; c += 2) {
        const float2 a1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(o + c));
        const float2 g1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(g + c));
        const float2 a2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(o + sec + c));
        const float2 g2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(g + sec + c));
        delta += a1.x * g1.x + a1.y * g1.y + a2.x * g2.x + a2.y * g2.y;
      }
      lse2 = p.lse[((long long)b * p.QH + qh) * p.Tc_total + p.q0 + r] * 1.4426950408889634f;
    }
    bool ok = true;
    for (int j = 0; j < nblk && ok; ++j) {
      if (!mbar_wait(sdp_full, j & 1, status, 308)) { ok = false; break; }
      tc_fence_after();
      if (!mbar_wait(pds_empty, (j & 1) ^ 1, status, 309)) { ok = false; break; }
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t sv[32], dv[32];
        tmem_ld_32x32(tS + lane_off + c * 32, sv);
        tmem_ld_32x32(tDP + lane_off + c * 32, dv);
        tmem_ld_wait();
        const int key0 = j * BKEY + c * 32;
        float pr[32], ds[32];
        // groups entirely at or below the diagonal with no segment ids need no per-element mask test (all groups
        // except those of the chunk's own key block)
        bool full = row_ok && key0 + 31 <= qpos;
        if (full && segrow) full = segrow[key0] == my_seg && segrow[key0 + 31] == my_seg;   // ids form contiguous runs
        if (full) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            pr[i] = exp2f(fmaf(__uint_as_float(sv[i]), p.scale_log2e, -lse2));
            ds[i] = pr[i] * p.scale * (__uint_as_float(dv[i]) - delta);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int key = key0 + i;
            const bool al = row_ok && key <= qpos && (!segrow || segrow[key] == my_seg);
            pr[i] = al ? exp2f(fmaf(__uint_as_float(sv[i]), p.scale_log2e, -lse2)) : 0.f;
            ds[i] = pr[i] * (__uint_as_float(dv[i]) - delta) * p.scale;
          }
        }
        uint8_t* dp = sP + (c >> 1) * TILE;
        uint8_t* dd = sDS + (c >> 1) * TILE;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 o1, o2;
          __nv_bfloat162* b1 = reinterpret_cast<__nv_bfloat162*>(&o1);
          __nv_bfloat162* b2 = reinterpret_cast<__nv_bfloat162*>(&o2);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            b1[i] = __floats2bfloat162_rn(pr[g * 8 + 2 * i], pr[g * 8 + 2 * i + 1]);
            b2[i] = __floats2bfloat162_rn(ds[g * 8 + 2 * i], ds[g * 8 + 2 * i + 1]);
          }
          const uint32_t off = swz(r, (c & 1) * 4 + g);
          *reinterpret_cast<uint4*>(dp + off) = o1;
          *reinterpret_cast<uint4*>(dd + off) = o2;
        }
      }
      tc_fence_before();
      fence_proxy_async();
      mbar_arrive(pds_full);
      mbar_arrive(sdp_empty);
      // dV_j then dK_j: this thread owns key row r of the block
      const int key = j * BKEY + r;
      for (int which = 0; which < 2 && ok; ++which) {
        if (!mbar_wait(dkv_full, which, status, 310)) { ok = false; break; }
        tc_fence_after();
        float* dst = (which == 0 ? p.dv_heads : p.dk_heads) + (((long long)b * p.T + key) * p.QH + qh) * p.HD;
#pragma unroll 1
        for (int c = 0; c < p.HD; c += 32) {
          uint32_t a[32];
          tmem_ld_32x32(tDKV + lane_off + c, a);
          tmem_ld_wait();
          if (key < p.e) {
            // fire-and-forget vector reductions: no read latency on the critical path.  The slab slice
            // belongs to this CTA alone, so the adds never contend and their order is fixed.
            const int nv = min(32, p.HD - c);
            for (int i = 0; i < nv; i += 4)
              asm volatile("red.relaxed.gpu.global.add.v4.f32 [%0], {%1, %2, %3, %4};"
                           ::"l"(dst + c + i), "f"(__uint_as_float(a[i])), "f"(__uint_as_float(a[i + 1])),
                             "f"(__uint_as_float(a[i + 2])), "f"(__uint_as_float(a[i + 3])) : "memory");
          }
        }
        tc_fence_before();
        mbar_arrive(dkv_empty);
      }
    }
    if (ok && mbar_wait(dq_full, 0, status, 311)) {
      tc_fence_after();
      __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.dq_attn) + (row * p.QH + qh) * p.HD;
#pragma unroll 1
      for (int c = 0; c < p.HD; c += 32) {
        uint32_t a[32];
        tmem_ld_32x32(tDQ + lane_off + c, a);
        tmem_ld_wait();
        if (row_ok) {
          const int nv = min(32, p.HD - c);
          for (int i = 0; i < nv; i += 8) {
            uint4 o;
            __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
            for (int t = 0; t < 4; ++t) ob[t] = __floats2bfloat162_rn(__uint_as_float(a[i + 2 * t]), __uint_as_float(a[i + 2 * t + 1]));
            *reinterpret_cast<uint4*>(dst + c + i) = o;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 512);
}

}  // namespace

extern "C" int loom_attn_bwd(const LoomAttn* a, cudaStream_t stream) {
  if (a->HD % 8 || a->HD > 128 || a->Tc < 1) return -1;
  Params p;
  memset(&p, 0, sizeof(p));
  const long long N = (long long)a->QH * a->HD;
  const long long M = (long long)a->B * a->Tc;
  if (!tma_host::make_4d_bf16(&p.q, a->qkc, a->HD, a->QH, 3, M, a->HD, N, 3 * N, 64, 1, 1, BQ)) return -2;
  if (!tma_host::make_4d_bf16(&p.dok, a->dqkc, a->HD, a->QH, 3, M, a->HD, N, 3 * N, 64, 1, 1, BQ)) return -2;
  p.dov = p.dok;
  const long long kvd = (long long)a->KVH * a->HD;
  if (!tma_host::make_4d_bf16(&p.k, a->kcache, a->HD, a->KVH, a->T, a->B, a->HD, kvd, kvd * a->T, 64, 1, BKEY, 1)) return -3;
  if (!tma_host::make_4d_bf16(&p.v, a->vcache, a->HD, a->KVH, a->T, a->B, a->HD, kvd, kvd * a->T, 64, 1, BKEY, 1)) return -3;
  p.qkc = a->qkc; p.dqkc = a->dqkc; p.lse = a->lse; p.seg = a->seg;
  p.dq_attn = a->dq_attn; p.dk_heads = a->dk_heads; p.dv_heads = a->dv_heads;
  p.B = a->B; p.QH = a->QH; p.KVH = a->KVH; p.HD = a->HD; p.T = a->T;
  p.Tc_total = a->Tc;
  p.row_pitch = 3 * N;
  p.scale = 1.0f / sqrtf((float)a->HD);
  p.scale_log2e = p.scale * 1.4426950408889634f;
  p.status = a->status;
  const int smem = 14 * TILE + 1024 + 256;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attn_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -4;
    configured = true;
  }
  // one launch per 128-row query tile; launches are stream-ordered, so the tiles' additions into the key / value
  // gradient slabs keep a fixed order
  for (int q0 = 0; q0 < a->Tc; q0 += BQ) {
    p.q0 = q0;
    p.Tc = a->Tc - q0 < BQ ? a->Tc - q0 : BQ;
    p.s = a->s + q0;
    p.e = a->s + q0 + p.Tc;
    attn_bwd_kernel<<<a->B * a->QH, THREADS, smem, stream>>>(p);
  }
  return (int)cudaGetLastError();
}
