// Dual-context causal GQA attention, forward (tcgen05 + TMEM + TMA).
//
// One CTA owns the <=128 query rows of one (batch row, query head) of the current temporal chunk and
// walks the key/value cache rows [0, e) in blocks of 128 keys:
//   S = Q K^T          tcgen05.mma, fp32 accumulator in TMEM (two S buffers so the next block's MMA overlaps
//                      the softmax of the current one)
//   P = exp(S - max)   four softmax warps, one query row per thread (TMEM lane == row, so row statistics
//                      need no shuffles); P is written to shared memory as a swizzled bf16 A-operand
//   O_v += P V ; O_k += P K     the K tile already in shared memory is reused as the MN-major B operand
//                      of the second product, which is how "attended keys" come for free
// Two passes over the keys (pass 1: row maxima only; pass 2: probabilities and both products) avoid
// rescaling the TMEM accumulators.  Causal masking is bottom-right aligned (query t of the chunk sits at
// absolute position s+t) and optional per-token segment ids restrict attention to the same segment, which
// covers packed SFT rows and document resets without a dense [T,T] mask.
//
// Replaces the reference path  repeat_interleave -> cat(K chunks) -> SDPA(value=[K;V], explicit bool mask)
// (reference loomformer.py:3085-3114, 3334-3363), which materialises the growing key prefix per chunk.
#include "sm100.cuh"
#include "tma_host.h"
#include "loom_c_api.h"

using namespace sm100;

namespace {

constexpr int BQ = 128;      // query rows per CTA
constexpr int BKEY = 128;    // keys per block
constexpr int THREADS = 192; // warp 0 TMA, warp 1 MMA, warps 2-5 softmax
constexpr int TILE = 16384;  // one [128 rows x 128 B] swizzled box
constexpr int NSTAGE = 2;

struct Params {
  CUtensorMap q, k, v;
  void* out_kctx;            // qkc + sector 1
  void* out_ctx;             // qkc + sector 2
  float* lse;                // [B, QH, Tc]
  const int* seg;            // [B, T] or null
  int B, QH, KVH, HD, Tc, T, s, e;   // Tc, s, e describe this launch's query tile (<= 128 rows)
  int Tc_total, q0;          // rows per batch entry in qkc / lse, and the tile's first row among them
  long long row_pitch;       // elements between consecutive query rows of qkc (3*N)
  float scale_log2e;         // softmax scale * log2(e)
  float scale;
  int* status;
};

__device__ __forceinline__ uint32_t swz(int row, int chunk) { return row * 128 + ((chunk ^ (row & 7)) << 4); }

__global__ void __launch_bounds__(THREADS, 1) attn_fwd_kernel(const __grid_constant__ Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                       // 2 tiles (hd 0-63, 64-127)
  uint8_t* sKV = sQ + 2 * TILE;             // NSTAGE x (K: 2 tiles, V: 2 tiles)
  uint8_t* sP = sKV + NSTAGE * 4 * TILE;    // 2 tiles (keys 0-63, 64-127)
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + 2 * TILE);
  uint64_t* q_full = bars;                  // 1
  uint64_t* kv_full = bars + 1;             // NSTAGE
  uint64_t* kv_empty = kv_full + NSTAGE;    // NSTAGE
  uint64_t* s_full = kv_empty + NSTAGE;     // 2
  uint64_t* s_empty = s_full + 2;           // 2
  uint64_t* p_full = s_empty + 2;           // 1
  uint64_t* p_empty = p_full + 1;           // 1
  uint64_t* o_full = p_empty + 1;           // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_full + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.x / p.QH, qh = blockIdx.x % p.QH;
  const int kvh = qh / (p.QH / p.KVH);
  volatile int* status = p.status;
  const int nblk = (p.e + BKEY - 1) / BKEY;
  const int ksteps = (p.HD + 15) / 16;   // the TMA unit zero-fills columns past HD             // MMA K steps over the head dimension
  const int hdp = (p.HD <= 64) ? 64 : 128;  // padded head dim = N of the P.V products

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < NSTAGE; ++i) { mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&s_full[i], 1); mbar_init(&s_empty[i], 128); }
    mbar_init(p_full, 128); mbar_init(p_empty, 1); mbar_init(o_full, 1);
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tS[2] = {tmem, tmem + 128};
  const uint32_t tOv = tmem + 256, tOk = tmem + 384;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      tma_prefetch_desc(&p.q); tma_prefetch_desc(&p.k); tma_prefetch_desc(&p.v);
      const int ntile = (p.HD > 64) ? 2 : 1;
      mbar_expect_tx(q_full, ntile * TILE);
      for (int i = 0; i < ntile; ++i) tma_load_4d(sQ + i * TILE, &p.q, q_full, 64 * i, qh, 0, b * p.Tc_total + p.q0);
      uint32_t it = 0;
      bool ok = true;
      for (int pass = 0; pass < 2 && ok; ++pass) {
        for (int j = 0; j < nblk; ++j, ++it) {
          const int st = it % NSTAGE;
          if (!mbar_wait(&kv_empty[st], ((it / NSTAGE) & 1) ^ 1, status, 201)) { ok = false; break; }
          uint8_t* sk = sKV + st * 4 * TILE;
          mbar_expect_tx(&kv_full[st], (pass == 0 ? 1 : 2) * ntile * TILE);
          for (int i = 0; i < ntile; ++i) tma_load_4d(sk + i * TILE, &p.k, &kv_full[st], 64 * i, kvh, j * BKEY, b);
          if (pass == 1)
            for (int i = 0; i < ntile; ++i) tma_load_4d(sk + (2 + i) * TILE, &p.v, &kv_full[st], 64 * i, kvh, j * BKEY, b);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      const uint32_t idesc_s = make_idesc_bf16(BQ, BKEY, 0, 0);
      const uint32_t idesc_o = make_idesc_bf16(BQ, hdp, 0, 1);
      const uint32_t q_addr = smem_u32(sQ), p_addr = smem_u32(sP);
      bool ok = mbar_wait(q_full, 0, status, 202);
      uint32_t it = 0;          // key-block counter across both passes (ring stage / parity)
      uint32_t sc = 0;          // S-buffer use counter
      auto issue_s = [&](uint32_t itx, uint32_t scx) -> bool {
        const int st = itx % NSTAGE;
        if (!mbar_wait(&kv_full[st], (itx / NSTAGE) & 1, status, 203)) return false;
        if (!mbar_wait(&s_empty[scx & 1], ((scx >> 1) & 1) ^ 1, status, 204)) return false;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(sKV + st * 4 * TILE);
        for (int ks = 0; ks < ksteps; ++ks) {
          const uint32_t off = (ks >> 2) * TILE + (ks & 3) * 32;
          mma_bf16_ss(tS[scx & 1], make_smem_desc_sw128(q_addr + off, 0, 1024),
                      make_smem_desc_sw128(k_addr + off, 0, 1024), idesc_s, ks > 0 ? 1u : 0u);
        }
        mma_commit(&s_full[scx & 1]);
        return true;
      };
      // pass 1: scores only
      for (int j = 0; j < nblk && ok; ++j, ++it, ++sc) {
        ok = issue_s(it, sc);
        if (ok) mma_commit(&kv_empty[it % NSTAGE]);
      }
      // pass 2: scores, then both products
      if (ok && nblk > 0) ok = issue_s(it, sc);
      for (int j = 0; j < nblk && ok; ++j) {
        if (j + 1 < nblk) ok = issue_s(it + 1, sc + 1);
        if (!ok) break;
        if (!mbar_wait(p_full, j & 1, status, 205)) { ok = false; break; }
        tc_fence_after();
        const int st = it % NSTAGE;
        const uint32_t k_addr = smem_u32(sKV + st * 4 * TILE), v_addr = k_addr + 2 * TILE;
        for (int ks = 0; ks < BKEY / 16; ++ks) {
          const uint64_t da = make_smem_desc_sw128(p_addr + (ks >> 2) * TILE + (ks & 3) * 32, 0, 1024);
          mma_bf16_ss(tOv, da, make_smem_desc_sw128(v_addr + ks * 2048, TILE, 1024), idesc_o, (j > 0 || ks > 0) ? 1u : 0u);
          mma_bf16_ss(tOk, da, make_smem_desc_sw128(k_addr + ks * 2048, TILE, 1024), idesc_o, (j > 0 || ks > 0) ? 1u : 0u);
        }
        mma_commit(p_empty);
        mma_commit(&kv_empty[st]);
        ++it; ++sc;
      }
      if (ok) mma_commit(o_full);
    }
  } else {
    // ------------------------------------------------------------------ softmax warps: one query row per thread
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const bool row_ok = r < p.Tc;
    const int qpos = p.s + r;
    const int my_seg = (p.seg && row_ok) ? p.seg[(long long)b * p.T + qpos] : 0;
    const int* segrow = p.seg ? p.seg + (long long)b * p.T : nullptr;
    const uint32_t lane_off = uint32_t(quad * 32) << 16;
    float mx = -INFINITY, l = 0.f;
    uint32_t sc = 0;
    bool ok = true;
    for (int pass = 0; pass < 2 && ok; ++pass) {
      for (int j = 0; j < nblk; ++j, ++sc) {
        if (!mbar_wait(&s_full[sc & 1], (sc >> 1) & 1, status, 206)) { ok = false; break; }
        tc_fence_after();
        if (pass == 1 && !mbar_wait(p_empty, (j & 1) ^ 1, status, 207)) { ok = false; break; }
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(tS[sc & 1] + lane_off + c * 32, v);
          tmem_ld_wait();
          const int key0 = j * BKEY + c * 32;
          // every key of this 32-column group is visible to this row (group entirely at or below the diagonal and in
          // the row's own segment): no per-element mask test.  True for most groups outside the chunk's own block.
          // With segment ids the group is fully visible when its first and last key carry this row's id: every id
          // occupies one contiguous run of the sequence (documents and packed examples do), so equal end points
          // mean a uniform group.
          bool full = row_ok && key0 + 31 <= qpos;
          if (full && segrow) full = segrow[key0] == my_seg && segrow[key0 + 31] == my_seg;
          if (pass == 0) {
            if (full) {
              float m0 = mx, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;     // four independent chains
#pragma unroll
              for (int i = 0; i < 32; i += 4) {
                m0 = fmaxf(m0, __uint_as_float(v[i])); m1 = fmaxf(m1, __uint_as_float(v[i + 1]));
                m2 = fmaxf(m2, __uint_as_float(v[i + 2])); m3 = fmaxf(m3, __uint_as_float(v[i + 3]));
              }
              mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                const int key = key0 + i;
                const bool al = row_ok && key <= qpos && (!segrow || segrow[key] == my_seg);
                if (al) mx = fmaxf(mx, __uint_as_float(v[i]));
              }
            }
          } else {
            float pr[32];
            const float mxs = mx * p.scale_log2e;
            if (full) {
              float l0 = 0.f, l1 = 0.f, l2 = 0.f, l3 = 0.f;
#pragma unroll
              for (int i = 0; i < 32; i += 4) {
                pr[i] = exp2f(fmaf(__uint_as_float(v[i]), p.scale_log2e, -mxs));
                pr[i + 1] = exp2f(fmaf(__uint_as_float(v[i + 1]), p.scale_log2e, -mxs));
                pr[i + 2] = exp2f(fmaf(__uint_as_float(v[i + 2]), p.scale_log2e, -mxs));
                pr[i + 3] = exp2f(fmaf(__uint_as_float(v[i + 3]), p.scale_log2e, -mxs));
                l0 += pr[i]; l1 += pr[i + 1]; l2 += pr[i + 2]; l3 += pr[i + 3];
              }
              l += (l0 + l1) + (l2 + l3);
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                const int key = key0 + i;
                const bool al = row_ok && key <= qpos && (!segrow || segrow[key] == my_seg);
                pr[i] = al ? exp2f(fmaf(__uint_as_float(v[i]), p.scale_log2e, -mxs)) : 0.f;
                l += pr[i];
              }
            }
            uint8_t* dst = sP + (c >> 1) * TILE;
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              uint4 o;
              __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
              for (int i = 0; i < 4; ++i) ob[i] = __floats2bfloat162_rn(pr[g * 8 + 2 * i], pr[g * 8 + 2 * i + 1]);
              *reinterpret_cast<uint4*>(dst + swz(r, (c & 1) * 4 + g)) = o;
            }
          }
        }
        tc_fence_before();
        if (pass == 1) { fence_proxy_async(); mbar_arrive(p_full); }
        mbar_arrive(&s_empty[sc & 1]);
      }
      if (pass == 0 && !(mx > -INFINITY)) mx = 0.f;
    }
    if (ok && mbar_wait(o_full, 0, status, 208)) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const long long row = (long long)b * p.Tc_total + p.q0 + r;
      __nv_bfloat16* ok_out = reinterpret_cast<__nv_bfloat16*>(p.out_kctx) + row * p.row_pitch + qh * p.HD;
      __nv_bfloat16* ov_out = reinterpret_cast<__nv_bfloat16*>(p.out_ctx) + row * p.row_pitch + qh * p.HD;
#pragma unroll 1
      for (int c = 0; c < p.HD; c += 32) {
        uint32_t a[32], bb[32];
        tmem_ld_32x32(tOk + lane_off + c, a);
        tmem_ld_32x32(tOv + lane_off + c, bb);
        tmem_ld_wait();
        if (row_ok) {
          const int nv = min(32, p.HD - c);
          for (int i = 0; i < nv; i += 8) {
            uint4 o1, o2;
            __nv_bfloat162* p1 = reinterpret_cast<__nv_bfloat162*>(&o1);
            __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&o2);
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              p1[t] = __floats2bfloat162_rn(__uint_as_float(a[i + 2 * t]) * inv, __uint_as_float(a[i + 2 * t + 1]) * inv);
              p2[t] = __floats2bfloat162_rn(__uint_as_float(bb[i + 2 * t]) * inv, __uint_as_float(bb[i + 2 * t + 1]) * inv);
            }
            *reinterpret_cast<uint4*>(ok_out + c + i) = o1;
            *reinterpret_cast<uint4*>(ov_out + c + i) = o2;
          }
        }
      }
      if (row_ok) p.lse[((long long)b * p.QH + qh) * p.Tc_total + p.q0 + r] = mx * p.scale + __logf(fmaxf(l, 1e-37f));
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 512);
}

}  // namespace

extern "C" int loom_attn_fwd(const LoomAttn* a, cudaStream_t stream) {
  if (a->HD % 8 || a->HD > 128 || a->Tc < 1) return -1;
  Params p;
  memset(&p, 0, sizeof(p));
  const long long N = (long long)a->QH * a->HD;
  // q = sector 0 of qkc [M, 3, QH, HD]: dims (HD, QH, 3, M)
  if (!tma_host::make_4d_bf16(&p.q, a->qkc, a->HD, a->QH, 3, (long long)a->B * a->Tc, a->HD, N, 3 * N, 64, 1, 1, BQ)) return -2;
  // caches [B, T, KVH, HD]: dims (HD, KVH, T, B)
  const long long kvd = (long long)a->KVH * a->HD;
  if (!tma_host::make_4d_bf16(&p.k, a->kcache, a->HD, a->KVH, a->T, a->B, a->HD, kvd, kvd * a->T, 64, 1, BKEY, 1)) return -3;
  if (!tma_host::make_4d_bf16(&p.v, a->vcache, a->HD, a->KVH, a->T, a->B, a->HD, kvd, kvd * a->T, 64, 1, BKEY, 1)) return -3;
  p.out_kctx = (__nv_bfloat16*)a->qkc + N;
  p.out_ctx = (__nv_bfloat16*)a->qkc + 2 * N;
  p.lse = a->lse; p.seg = a->seg;
  p.B = a->B; p.QH = a->QH; p.KVH = a->KVH; p.HD = a->HD; p.T = a->T;
  p.Tc_total = a->Tc;
  p.row_pitch = 3 * N;
  p.scale = 1.0f / sqrtf((float)a->HD);
  p.scale_log2e = p.scale * 1.4426950408889634f;
  p.status = a->status;
  const int smem = (2 + NSTAGE * 4 + 2) * TILE + 1024 + 256;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -4;
    configured = true;
  }
  // a chunk longer than 128 queries (wide temporal windows, the unchunked forward) goes out as one launch per
  // 128-row query tile; a tile's keys end at its own last query
  for (int q0 = 0; q0 < a->Tc; q0 += BQ) {
    p.q0 = q0;
    p.Tc = a->Tc - q0 < BQ ? a->Tc - q0 : BQ;
    p.s = a->s + q0;
    p.e = a->s + q0 + p.Tc;
    attn_fwd_kernel<<<a->B * a->QH, THREADS, smem, stream>>>(p);
  }
  return (int)cudaGetLastError();
}
