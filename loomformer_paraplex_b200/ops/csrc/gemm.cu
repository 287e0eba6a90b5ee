// Segmented-K, optionally batched bf16 GEMM on the 5th-generation tensor cores.
//
//   C[m, g, n] (+)= sum_seg sum_k A_seg[m, g?, k] * B[n, g?, b_k0(seg) + k]   (+ bias[g, n])
//
// * operands are staged by TMA (128-byte swizzle) into a multi-stage shared-memory ring,
// * one elected thread issues tcgen05.mma (M=128, N=BN, K=16) with the fp32 accumulator in TMEM,
// * four epilogue warps read the accumulator back with tcgen05.ld and store bf16 or fp32,
// * the kernel is persistent (one CTA per SM loops over tiles) and double-buffers the TMEM
//   accumulator so the epilogue of tile i overlaps the main loop of tile i+1.
//
// "Segmented K": the reduction dimension may be the concatenation of up to MAX_SEG different
// tensors (e.g. the Paraplex phase input [Q_g | Kctx_g | C_g | u | D_g]); each segment has its own
// tensor map whose extent bounds the segment, so ragged tails are zero-filled by the TMA unit.
// With `b_per_seg` every segment also brings its own B operand: that is how the weight gradients of
// all temporal chunks of a step (dY_c^T X_c, c = 0..15) become ONE launch with a 16x longer reduction
// instead of sixteen short ones.
// "Batched": every operand is a [rows, heads, cols] view; a batched operand indexes `heads` with the
// tile's group id, an unbatched one uses group 0.  Either operand may be K-major (reduction index
// contiguous) or MN-major (the other index contiguous), which covers forward, data-gradient and
// weight-gradient GEMMs without materialising transposes.
//
// This kernel replaces the library GEMMs of the reference (F.linear / cublasGemmStridedBatchedEx,
// reference kernels/beta_space/beta_space_launcher.cu:57-151) and its operand pack/unpack kernels
// (beta_space_kernel.cuh:86-271): nothing is gathered or scattered through global memory.
#include <stdlib.h>
#include "sm100.cuh"
#include "tma_host.h"
#include "loom_c_api.h"

using namespace sm100;

namespace {

constexpr int BM = 128;
constexpr int BK = 64;          // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int MAX_SEG = 16;
constexpr int NUM_THREADS = 192;  // warp 0: TMA, warp 1: MMA, warps 2-5: epilogue

struct Seg {
  CUtensorMap a;
  CUtensorMap b;  // used only when every segment brings its own B operand (grouped weight gradients)
  int k_len;      // reduction length of this segment
  int a_k0;       // offset of the segment along A's reduction index
  int b_k0;       // offset of the segment along B's reduction index
  int a_batched;
};

struct Params {
  CUtensorMap b;
  Seg seg[MAX_SEG];
  int nseg;
  int b_batched;
  int b_per_seg;
  void* c;
  long long ldc;        // row pitch of C (elements)
  long long ldc_head;   // group pitch of C (elements)
  const float* bias;    // [heads * n_per_head] or nullptr
  int M, n_per_head, heads;
  int accumulate;       // C += result
  int out_fp32;
  // c_tma != 0: the epilogue stages 32-row x 128-byte boxes in shared memory and hands them to the TMA unit (plain
  // store, or element-wise add in L2 when `accumulate`), so global memory sees full lines written asynchronously
  // instead of one 16-byte store per row and thread.  cmap describes C as (N, M, heads).
  int c_tma;
  CUtensorMap cmap;
  int a_lbo, a_sbo, b_lbo, b_sbo;
  int* status;
  // sharded-weight gather (all-gather fused into the consuming GEMM): rank r owns the 64-row blocks
  // [r * gather_per, (r+1) * gather_per) of B; b_peer[r] maps rank r's copy of the whole matrix (box: 64 rows)
  int gather_world, gather_rank, gather_per;
  CUtensorMap b_peer[8];
  // row-sharded activations (tensor-parallel all-gather -> GEMM): rank r holds rows [r*a_rows_per_rank, ...) of A
  int a_world, a_rows_per_rank;
  CUtensorMap a_peer[8];
  // GEMM -> reduce-scatter: the fp32 partial product of output rows owned by rank r is stored into this rank's slot of rs_out[r]
  int rs_world, rs_rank, rs_rows_per_rank;
  float* rs_out[8];
  // [Q | K | V] projection whose epilogue applies RoPE and writes the attention operand and the caches (pair tiles)
  int rope_hd, rope_qh, rope_kvh, rope_tc, rope_t, rope_s;
  long long rope_q_ld;
  const float* rope_cos; const float* rope_sin;
  __nv_bfloat16* rope_q; __nv_bfloat16* rope_k; __nv_bfloat16* rope_v;
};

constexpr int OUT_STAGE_BYTES = 4 * 2 * 4096;   // four epilogue warps x two 32-row x 128-byte staging boxes

// 16-byte chunk `chunk` of row `row` inside a 128-byte-swizzled box with 128-byte rows
__device__ __forceinline__ uint32_t swz128(int row, int chunk) { return row * 128 + ((chunk ^ (row & 7)) << 4); }

__device__ __forceinline__ void tma_reduce_add_3d(const void* tmap, const void* smem_src, int x, int y, int z) {
  asm volatile("cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(smem_src)), "r"(x), "r"(y), "r"(z)
               : "memory");
}
__device__ __forceinline__ void tma_store_wait_read1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }

// Accumulator rows [32 lanes of this warp] x [BN columns] -> C through shared memory and the TMA unit.
// `taddr`: TMEM address of the warp's lane quadrant and accumulator buffer; `row0`: output row of lane 0;
// `stage`: this warp's two staging boxes; `nstore`: boxes this warp has issued so far (selects the box, bounds reuse).
template <int BN>
__device__ __forceinline__ void store_tile_tma(const Params& p, uint32_t taddr, int row0, int n0, int g, int lane,
                                               uint8_t* stage, uint32_t& nstore) {
  const float* bias = p.bias ? p.bias + (long long)g * p.n_per_head : nullptr;
  const int W = p.out_fp32 ? 32 : 64;            // columns per 128-byte row
#pragma unroll 1
  for (int c0 = 0; c0 < BN; c0 += W) {
    const int n = n0 + c0;
    if (n >= p.n_per_head) break;                // nothing of this tile is left of here (uniform over the warp)
    uint8_t* buf = stage + (nstore & 1) * 4096;
    if (nstore >= 2) {                           // the box issued two steps ago must have been read out
      if (lane == 0) tma_store_wait_read1();
      __syncwarp();
    }
    uint32_t r[32];
    tmem_ld_32x32(taddr + c0, r);
    if (p.out_fp32) {
      tmem_ld_wait();
      if (bias) {
#pragma unroll
        for (int i = 0; i < 32; ++i) if (n + i < p.n_per_head) r[i] = __float_as_uint(__uint_as_float(r[i]) + bias[n + i]);
      }
#pragma unroll
      for (int c = 0; c < 8; ++c)
        *reinterpret_cast<uint4*>(buf + swz128(lane, c)) = make_uint4(r[4 * c], r[4 * c + 1], r[4 * c + 2], r[4 * c + 3]);
    } else {
      uint32_t r2[32];
      tmem_ld_32x32(taddr + c0 + 32, r2);
      tmem_ld_wait();
      if (bias) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          if (n + i < p.n_per_head) r[i] = __float_as_uint(__uint_as_float(r[i]) + bias[n + i]);
          if (n + 32 + i < p.n_per_head) r2[i] = __float_as_uint(__uint_as_float(r2[i]) + bias[n + 32 + i]);
        }
      }
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint4 o;
        __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) ob[j] = __floats2bfloat162_rn(__uint_as_float(r[8 * c + 2 * j]), __uint_as_float(r[8 * c + 2 * j + 1]));
        *reinterpret_cast<uint4*>(buf + swz128(lane, c)) = o;
#pragma unroll
        for (int j = 0; j < 4; ++j) ob[j] = __floats2bfloat162_rn(__uint_as_float(r2[8 * c + 2 * j]), __uint_as_float(r2[8 * c + 2 * j + 1]));
        *reinterpret_cast<uint4*>(buf + swz128(lane, 4 + c)) = o;
      }
    }
    fence_proxy_async();                         // generic-proxy writes above -> visible to the TMA unit
    __syncwarp();
    if (lane == 0) {
      if (p.accumulate) tma_reduce_add_3d(&p.cmap, buf, n, row0, g);
      else tma_store_3d(&p.cmap, buf, n, row0, g);
      tma_store_commit();
    }
    ++nstore;
  }
}

// Direct epilogue: every thread stores its own row (used when C cannot be described to the TMA unit -- pitch or base
// not 16-byte aligned -- and by the reduce-scatter variant, whose destination is another rank's memory).
template <int BN>
__device__ __forceinline__ void store_tile_direct(const Params& p, uint32_t taddr, int row, int n0, int g) {
  const long long c_row = (long long)row * p.ldc + (long long)g * p.ldc_head;
  const float* bias = p.bias ? p.bias + (long long)g * p.n_per_head : nullptr;
#pragma unroll 1
  for (int c0 = 0; c0 < BN; c0 += 32) {
    uint32_t r[32];
    tmem_ld_32x32(taddr + c0, r);
    tmem_ld_wait();
    const int n = n0 + c0;
    if (row < p.M && n < p.n_per_head) {
      const int nvalid = min(32, p.n_per_head - n);
      float v[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
      if (bias) {
#pragma unroll
        for (int i = 0; i < 32; ++i) if (i < nvalid) v[i] += bias[n + i];
      }
      if (p.rs_world > 1) {
        // reduce-scatter epilogue: this rank's partial product of a row goes, by plain 16-byte stores over
        // NVLink, into slot `rs_rank` of the staging buffer [world][rows_per_rank][N] of the rank that owns the
        // row; the owner sums its slots after the closing barrier (deterministic, no atomics on the link)
        const int owner = row / p.rs_rows_per_rank;
        float* dst = p.rs_out[owner] +
                     ((long long)p.rs_rank * p.rs_rows_per_rank + (row - owner * p.rs_rows_per_rank)) * p.ldc + n;
        if (nvalid == 32 && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
          for (int i = 0; i < 32; i += 4) *reinterpret_cast<float4*>(dst + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
        } else {
          for (int i = 0; i < nvalid; ++i) dst[i] = v[i];
        }
      } else if (p.out_fp32) {
        float* dst = reinterpret_cast<float*>(p.c) + c_row + n;
        if (nvalid == 32 && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            float4 o = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
            if (p.accumulate) { float4 old = *reinterpret_cast<float4*>(dst + i); o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w; }
            *reinterpret_cast<float4*>(dst + i) = o;
          }
        } else {
          for (int i = 0; i < nvalid; ++i) dst[i] = p.accumulate ? dst[i] + v[i] : v[i];
        }
      } else {
        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.c) + c_row + n;
        if (nvalid == 32 && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            if (p.accumulate) {
              uint4 old = *reinterpret_cast<uint4*>(dst + i);
              const __nv_bfloat162* ob = reinterpret_cast<const __nv_bfloat162*>(&old);
#pragma unroll
              for (int j = 0; j < 4; ++j) { float2 f = __bfloat1622float2(ob[j]); v[i + 2 * j] += f.x; v[i + 2 * j + 1] += f.y; }
            }
            uint4 o;
            __nv_bfloat162* ob2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
            for (int j = 0; j < 4; ++j) ob2[j] = __floats2bfloat162_rn(v[i + 2 * j], v[i + 2 * j + 1]);
            *reinterpret_cast<uint4*>(dst + i) = o;
          }
        } else {
          for (int i = 0; i < nvalid; ++i) {
            float x = v[i];
            if (p.accumulate) x += __bfloat162float(dst[i]);
            dst[i] = __float2bfloat16(x);
          }
        }
      }
    }
  }
}

// Epilogue of the [Q | K | V] projection: a tile holds whole heads (BN is a multiple of HD), a thread holds one token's
// row.  Q and K heads are rotated in fp32 straight from the accumulator (rotate-half: pair (j, j + HD/2)), V heads pass
// through; rotated Q goes to the attention operand buffer, K and V to the caches at the token's position, so neither
// the unrotated projection nor a second launch exists.
template <int BN, int HD>
__device__ __forceinline__ void store_tile_rope(const Params& p, uint32_t taddr, int row, int n0) {
  constexpr int HALF = HD / 2;
  const bool live = row < p.M;
  const int rr = live ? row : 0;
  const int b = rr / p.rope_tc, t = rr - b * p.rope_tc;
  const float* cs = p.rope_cos + (long long)rr * HD;
  const float* sn = p.rope_sin + (long long)rr * HD;
  const int heads = p.rope_qh + 2 * p.rope_kvh;
#pragma unroll 1
  for (int h = 0; h < BN / HD; ++h) {
    const int hh = n0 / HD + h;                        // head among Q heads, K heads, V heads (uniform in the warp)
    if (hh >= heads) break;
    uint32_t r[HD];
#pragma unroll
    for (int c = 0; c < HD / 32; ++c) tmem_ld_32x32(taddr + h * HD + c * 32, reinterpret_cast<uint32_t(&)[32]>(r[c * 32]));
    tmem_ld_wait();
    if (!live) continue;
    float v[HD];
#pragma unroll
    for (int i = 0; i < HD; ++i) v[i] = __uint_as_float(r[i]);
    if (p.bias) {
#pragma unroll
      for (int i = 0; i < HD; ++i) v[i] += p.bias[hh * HD + i];
    }
    __nv_bfloat16* dst;
    if (hh < p.rope_qh + p.rope_kvh) {
#pragma unroll
      for (int j = 0; j < HALF; j += 4) {
        const float4 c1 = *reinterpret_cast<const float4*>(cs + j), c2 = *reinterpret_cast<const float4*>(cs + j + HALF);
        const float4 s1 = *reinterpret_cast<const float4*>(sn + j), s2 = *reinterpret_cast<const float4*>(sn + j + HALF);
        const float c1a[4] = {c1.x, c1.y, c1.z, c1.w}, c2a[4] = {c2.x, c2.y, c2.z, c2.w};
        const float s1a[4] = {s1.x, s1.y, s1.z, s1.w}, s2a[4] = {s2.x, s2.y, s2.z, s2.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float x1 = v[j + i], x2 = v[j + i + HALF];
          v[j + i] = x1 * c1a[i] - x2 * s1a[i];
          v[j + i + HALF] = x2 * c2a[i] + x1 * s2a[i];
        }
      }
      dst = hh < p.rope_qh ? p.rope_q + (long long)rr * p.rope_q_ld + (long long)hh * HD
                           : p.rope_k + (((long long)b * p.rope_t + p.rope_s + t) * p.rope_kvh + (hh - p.rope_qh)) * HD;
    } else {
      dst = p.rope_v + (((long long)b * p.rope_t + p.rope_s + t) * p.rope_kvh + (hh - p.rope_qh - p.rope_kvh)) * HD;
    }
#pragma unroll
    for (int i = 0; i < HD; i += 8) {
      uint4 o;
      __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) ob[j] = __floats2bfloat162_rn(v[i + 2 * j], v[i + 2 * j + 1]);
      *reinterpret_cast<uint4*>(dst + i) = o;
    }
  }
}

template <int BN>
struct Cfg {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN >= 256) ? 4 : ((BN >= 128) ? 6 : 8);
  static constexpr int SMEM = STAGES * STAGE_BYTES + OUT_STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
  static constexpr int TMEM_COLS = (2 * BN <= 32) ? 32 : 2 * BN;
};

// GATHER (K-major operands only): every 64-row block of B is fetched from the rank that owns it -- a TMA load from
// that peer's memory, no multicast -- while the math of earlier tiles runs; the CTAs of the first row of output
// tiles also deposit each remote block in this rank's own copy of B, so after this launch the local copy is
// complete and every later kernel of the step reads it locally.  The parameter all-gather of sharded data
// parallelism is thereby part of the first GEMM that needs the weight instead of a separate collective.
template <int BN, bool A_MN, bool B_MN, bool GATHER>
__global__ void __launch_bounds__(NUM_THREADS, 1) gemm_kernel(const __grid_constant__ Params p) {
  using C = Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* out_stage = smem + C::STAGES * C::STAGE_BYTES;      // 1024-byte aligned: every stage is a multiple of 1024
  uint64_t* full = reinterpret_cast<uint64_t*>(out_stage + OUT_STAGE_BYTES);
  uint64_t* empty = full + C::STAGES;
  uint64_t* acc_full = empty + C::STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  volatile int* status = p.status;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], 128); }
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, C::TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Programmatic dependent launch: everything above touches only this CTA's shared memory and TMEM, so it may run
  // while the previous kernel of the stream is still finishing.  From here on global memory is read and written:
  // wait until every prerequisite grid has completed and its writes are visible (no-op for an ordinary launch),
  // then let the next kernel of the stream start its own prologue early.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  const int tiles_m = (p.M + BM - 1) / BM;
  const int tiles_n = (p.n_per_head + BN - 1) / BN;
  const int total = tiles_m * tiles_n * p.heads;
  int kblocks = 0;
  for (int s = 0; s < p.nseg; ++s) kblocks += (p.seg[s].k_len + BK - 1) / BK;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (elect_one()) {
      if (!p.b_per_seg) tma_prefetch_desc(&p.b);
      for (int s = 0; s < p.nseg; ++s) { tma_prefetch_desc(&p.seg[s].a); if (p.b_per_seg) tma_prefetch_desc(&p.seg[s].b); }
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x) {
        const int tm = tile % tiles_m;
        const int tn = (tile / tiles_m) % tiles_n;
        const int g = tile / (tiles_m * tiles_n);
        const int m0 = tm * BM, n0 = tn * BN;
        for (int s = 0; s < p.nseg && ok; ++s) {
          const Seg& sg = p.seg[s];
          const CUtensorMap* bmap = p.b_per_seg ? &sg.b : &p.b;
          const int ag = sg.a_batched ? g : 0;
          const int bg = p.b_batched ? g : 0;
          for (int k = 0; k < sg.k_len; k += BK, ++it) {
            const int st = it % C::STAGES;
            const uint32_t ph = (it / C::STAGES) & 1;
            if (!mbar_wait(&empty[st], ph ^ 1, status, 101)) { ok = false; break; }
            uint8_t* sa = smem + st * C::STAGE_BYTES;
            uint8_t* sb = sa + C::A_BYTES;
            mbar_expect_tx(&full[st], C::STAGE_BYTES);
            if (A_MN) {
#pragma unroll
              for (int j = 0; j < BM / 64; ++j)
                tma_load_3d(sa + j * 8192, &sg.a, &full[st], m0 + 64 * j, sg.a_k0 + k, ag);
            } else if (p.a_world > 1) {
              // the tile's 128 rows live on one rank (a_rows_per_rank is a multiple of 128): fetch them from there
              tma_load_3d(sa, &p.a_peer[m0 / p.a_rows_per_rank], &full[st], sg.a_k0 + k, m0, 0);
            } else {
              tma_load_3d(sa, &sg.a, &full[st], sg.a_k0 + k, m0, ag);
            }
            if (GATHER) {
              bool remote[BN / 64];
#pragma unroll
              for (int j = 0; j < BN / 64; ++j) {
                const int row0 = n0 + 64 * j;
                int owner = (row0 >> 6) / p.gather_per;
                owner = owner < p.gather_world ? owner : p.gather_world - 1;
                remote[j] = owner != p.gather_rank && row0 < p.n_per_head;
                tma_load_3d(sb + j * 8192, &p.b_peer[owner], &full[st], sg.b_k0 + k, row0, 0);
              }
              if (tm == 0) {
                // deposit the remote blocks locally once they have landed (this CTA alone does it for its columns)
                if (!mbar_wait(&full[st], ph, status, 105)) { ok = false; break; }
                bool any = false;
#pragma unroll
                for (int j = 0; j < BN / 64; ++j) {
                  if (remote[j]) { tma_store_3d(&p.b_peer[p.gather_rank], sb + j * 8192, sg.b_k0 + k, n0 + 64 * j, 0); any = true; }
                }
                if (any) { tma_store_commit(); tma_store_wait_read(); }
              }
            } else if (B_MN) {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j)
                tma_load_3d(sb + j * 8192, bmap, &full[st], n0 + 64 * j, sg.b_k0 + k, bg);
            } else {
              tma_load_3d(sb, bmap, &full[st], sg.b_k0 + k, n0, bg);
            }
          }
        }
      if (GATHER) tma_store_wait_all();
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      uint32_t it = 0, tcount = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x, ++tcount) {
        const uint32_t acc = tcount & 1;
        if (!mbar_wait(&acc_empty[acc], ((tcount >> 1) & 1) ^ 1, status, 102)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int st = it % C::STAGES;
          if (!mbar_wait(&full[st], (it / C::STAGES) & 1, status, 103)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + st * C::STAGE_BYTES);
          const uint32_t sb = sa + C::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint32_t a_off = A_MN ? k * (UMMA_K * 128) : k * (UMMA_K * 2);
            const uint32_t b_off = B_MN ? k * (UMMA_K * 128) : k * (UMMA_K * 2);
            const uint64_t da = make_smem_desc_sw128(sa + a_off, p.a_lbo, p.a_sbo);
            const uint64_t db = make_smem_desc_sw128(sb + b_off, p.b_lbo, p.b_sbo);
            mma_bf16_ss(d_tmem, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          mma_commit(&empty[st]);       // frees the smem stage when these MMAs retire
        }
        if (ok) mma_commit(&acc_full[acc]);
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue (warps 2..5)
    const int q = warp & 3;             // TMEM lane quadrant this warp may access
    uint32_t tcount = 0, nstore = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x, ++tcount) {
      const int tm = tile % tiles_m;
      const int tn = (tile / tiles_m) % tiles_n;
      const int g = tile / (tiles_m * tiles_n);
      const uint32_t acc = tcount & 1;
      if (!mbar_wait(&acc_full[acc], (tcount >> 1) & 1, status, 104)) { ok = false; break; }
      tc_fence_after();
      const int row = tm * BM + q * 32 + lane;
      const int n0 = tn * BN;
      const uint32_t taddr = tmem_base + acc * BN + (uint32_t(q * 32) << 16);
      if (p.c_tma) store_tile_tma<BN>(p, taddr, tm * BM + q * 32, n0, g, lane, out_stage + q * 8192, nstore);
      else store_tile_direct<BN>(p, taddr, row, n0, g);
      tc_fence_before();
      mbar_arrive(&acc_empty[acc]);
    }
    if (nstore > 0 && lane == 0) tma_store_wait_all();      // staged boxes must be out before shared memory goes away
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, C::TMEM_COLS);
}

// ---------------------------------------------------------------------------------------------------------------
// CTA-pair variant: a cluster of two CTAs computes one 256 x BN output tile with tcgen05.mma.cta_group::2.
// Each CTA stages its own 128 rows of A and its own BN/2 columns of B (24-32 KB per k-block and SM instead of the
// 32-48 KB of the single-CTA tiles), holds its own 128 x BN accumulator rows in TMEM (double buffered) and runs its
// own epilogue.  The even CTA's MMA thread issues for both; its operand barrier counts the bytes of both CTAs'
// loads.  Same operand layouts, segments, batching and epilogue options as gemm_kernel; the collective variants
// (gather / row-sharded A / reduce-scatter epilogue) stay on the single-CTA kernel.
template <int BN>
struct PairCfg {
  static constexpr int HALF = BN / 2;                 // B columns staged per CTA
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = HALF * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN >= 192) ? 6 : 8;
  static constexpr int SMEM = STAGES * STAGE_BYTES + OUT_STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
  static constexpr int TMEM_COLS = BN <= 128 ? 256 : 512;        // two accumulators of BN columns, a power of two
};

template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(NUM_THREADS, 1) gemm_pair_kernel(const __grid_constant__ Params p) {
  using C = PairCfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* out_stage = smem + C::STAGES * C::STAGE_BYTES;      // 1024-byte aligned: every stage is a multiple of 1024
  uint64_t* full = reinterpret_cast<uint64_t*>(out_stage + OUT_STAGE_BYTES);
  uint64_t* empty = full + C::STAGES;
  uint64_t* acc_full = empty + C::STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();          // 0: leader (issues the MMAs), 1: peer
  volatile int* status = p.status;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    // acc_empty of the leader collects the epilogue threads of both CTAs
    for (int i = 0; i < 2; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], 256); }
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc_pair(tmem_slot, C::TMEM_COLS); tmem_relinquish_pair(); }
  tc_fence_before();
  __syncthreads();
  // both CTAs' barriers exist and both allocations are done before anything crosses the pair
  cluster_arrive();
  cluster_wait();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  const int tiles_m = (p.M + 2 * BM - 1) / (2 * BM);
  const int tiles_n = (p.n_per_head + BN - 1) / BN;
  const int total = tiles_m * tiles_n * p.heads;
  const int npairs = gridDim.x >> 1;
  const int pair = blockIdx.x >> 1;
  int kblocks = 0;
  for (int s = 0; s < p.nseg; ++s) kblocks += (p.seg[s].k_len + BK - 1) / BK;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer (both CTAs, own halves)
    if (elect_one()) {
      if (!p.b_per_seg) tma_prefetch_desc(&p.b);
      for (int s = 0; s < p.nseg; ++s) { tma_prefetch_desc(&p.seg[s].a); if (p.b_per_seg) tma_prefetch_desc(&p.seg[s].b); }
      uint32_t it = 0;
      bool ok = true;
      for (int tile = pair; tile < total && ok; tile += npairs) {
        const int tm = tile % tiles_m;
        const int tn = (tile / tiles_m) % tiles_n;
        const int g = tile / (tiles_m * tiles_n);
        const int m0 = tm * (2 * BM) + (int)rank * BM;
        const int n0 = tn * BN + (int)rank * C::HALF;
        for (int s = 0; s < p.nseg && ok; ++s) {
          const Seg& sg = p.seg[s];
          const CUtensorMap* bmap = p.b_per_seg ? &sg.b : &p.b;
          const int ag = sg.a_batched ? g : 0;
          const int bg = p.b_batched ? g : 0;
          for (int k = 0; k < sg.k_len; k += BK, ++it) {
            const int st = it % C::STAGES;
            const uint32_t ph = (it / C::STAGES) & 1;
            if (!mbar_wait(&empty[st], ph ^ 1, status, 111)) { ok = false; break; }
            const uint32_t sa = smem_u32(smem + st * C::STAGE_BYTES);
            const uint32_t sb = sa + C::A_BYTES;
            // the leader's barrier of this stage expects the bytes of both CTAs
            const uint32_t bar = mapa_shared(smem_u32(&full[st]), 0);
            if (rank == 0) mbar_expect_tx(&full[st], 2 * C::STAGE_BYTES);
            if (A_MN) {
#pragma unroll
              for (int j = 0; j < BM / 64; ++j)
                tma_load_3d_pair(sa + j * 8192, &sg.a, bar, m0 + 64 * j, sg.a_k0 + k, ag);
            } else {
              tma_load_3d_pair(sa, &sg.a, bar, sg.a_k0 + k, m0, ag);
            }
            if (B_MN) {
#pragma unroll
              for (int j = 0; j < C::HALF / 64; ++j)
                tma_load_3d_pair(sb + j * 8192, bmap, bar, n0 + 64 * j, sg.b_k0 + k, bg);
            } else {
              tma_load_3d_pair(sb, bmap, bar, sg.b_k0 + k, n0, bg);
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer (leader CTA only)
    if (rank == 0 && elect_one()) {
      constexpr uint32_t idesc = make_idesc_bf16(2 * BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      uint32_t it = 0, tcount = 0;
      bool ok = true;
      for (int tile = pair; tile < total && ok; tile += npairs, ++tcount) {
        const uint32_t acc = tcount & 1;
        if (!mbar_wait(&acc_empty[acc], ((tcount >> 1) & 1) ^ 1, status, 112)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int st = it % C::STAGES;
          if (!mbar_wait(&full[st], (it / C::STAGES) & 1, status, 113)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + st * C::STAGE_BYTES);
          const uint32_t sb = sa + C::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint32_t a_off = A_MN ? k * (UMMA_K * 128) : k * (UMMA_K * 2);
            const uint32_t b_off = B_MN ? k * (UMMA_K * 128) : k * (UMMA_K * 2);
            const uint64_t da = make_smem_desc_sw128(sa + a_off, p.a_lbo, p.a_sbo);
            const uint64_t db = make_smem_desc_sw128(sb + b_off, p.b_lbo, p.b_sbo);
            mma_bf16_ss_pair(d_tmem, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          mma_commit_pair(&empty[st], 3);       // frees this stage in both CTAs when these MMAs retire
        }
        if (ok) mma_commit_pair(&acc_full[acc], 3);
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue (warps 2..5 of both CTAs)
    const int q = warp & 3;
    uint32_t tcount = 0, nstore = 0;
    bool ok = true;
    for (int tile = pair; tile < total && ok; tile += npairs, ++tcount) {
      const int tm = tile % tiles_m;
      const int tn = (tile / tiles_m) % tiles_n;
      const int g = tile / (tiles_m * tiles_n);
      const uint32_t acc = tcount & 1;
      if (!mbar_wait(&acc_full[acc], (tcount >> 1) & 1, status, 114)) { ok = false; break; }
      tc_fence_after();
      const int row = tm * (2 * BM) + (int)rank * BM + q * 32 + lane;
      const int n0 = tn * BN;
      const uint32_t taddr = tmem_base + acc * BN + (uint32_t(q * 32) << 16);
      if (!A_MN && !B_MN && p.rope_hd != 0) {
        if (BN % 96 == 0 && p.rope_hd == 96) store_tile_rope<BN, (BN % 96 == 0 ? 96 : 32)>(p, taddr, row, n0);
        else if (BN % 64 == 0 && p.rope_hd == 64) store_tile_rope<BN, (BN % 64 == 0 ? 64 : 32)>(p, taddr, row, n0);
        else if (BN % 128 == 0 && p.rope_hd == 128) store_tile_rope<BN, (BN % 128 == 0 ? 128 : 32)>(p, taddr, row, n0);
      }
      else if (p.c_tma) store_tile_tma<BN>(p, taddr, tm * (2 * BM) + (int)rank * BM + q * 32, n0, g, lane, out_stage + q * 8192, nstore);
      else store_tile_direct<BN>(p, taddr, row, n0, g);
      tc_fence_before();
      // this accumulator buffer may be overwritten once the epilogue threads of BOTH CTAs have read it
      mbar_arrive_cluster(mapa_shared(smem_u32(&acc_empty[acc]), 0));
    }
    if (nstore > 0 && lane == 0) tma_store_wait_all();
  }

  // neither CTA may leave (or free its TMEM) while the other can still touch its shared memory or barriers
  tc_fence_before();
  __syncwarp();
  __syncthreads();
  cluster_arrive();
  cluster_wait();
  if (warp == 1) tmem_dealloc_pair(tmem_base, C::TMEM_COLS);
}

bool fill_map(CUtensorMap* map, const LoomOperand& o, bool mn_major, int box_mn) {
  // view [rows, heads, cols]: dims (cols, rows, heads)
  tma_host::EncodeTiledFn fn = tma_host::encode_fn();
  if (!fn) return false;
  cuuint64_t dims[3] = {(cuuint64_t)o.cols, (cuuint64_t)o.rows, (cuuint64_t)(o.heads > 0 ? o.heads : 1)};
  cuuint64_t strides[2] = {(cuuint64_t)o.ld_row * 2, (cuuint64_t)(o.heads > 1 ? o.ld_head : o.ld_row * o.rows) * 2};
  if (o.heads <= 1) strides[1] = (cuuint64_t)o.ld_row * 2 * (cuuint64_t)o.rows;
  cuuint32_t box[3];
  box[0] = 64;
  box[1] = mn_major ? 64u : (cuuint32_t)box_mn;
  box[2] = 1;
  cuuint32_t elem[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(o.ptr), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// C viewed as (N, M, heads) for the staged epilogue: boxes of 128 bytes x 32 rows, 128-byte swizzle
bool fill_c_map(CUtensorMap* map, void* c, int M, int N, int heads, long long ldc, long long ldc_head, bool fp32) {
  tma_host::EncodeTiledFn fn = tma_host::encode_fn();
  if (!fn) return false;
  const cuuint64_t es = fp32 ? 4 : 2;
  cuuint64_t dims[3] = {(cuuint64_t)N, (cuuint64_t)M, (cuuint64_t)(heads > 1 ? heads : 1)};
  cuuint64_t strides[2] = {(cuuint64_t)ldc * es, (cuuint64_t)(heads > 1 ? ldc_head : ldc * (long long)M) * es};
  cuuint32_t box[3] = {fp32 ? 32u : 64u, 32u, 1u};
  cuuint32_t elem[3] = {1, 1, 1};
  CUresult r = fn(map, fp32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, c, dims, strides, box,
                  elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

template <int BN, bool A_MN, bool B_MN, bool GATHER = false>
int launch(const Params& p, int sms, cudaStream_t stream) {
  using C = Cfg<BN>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_kernel<BN, A_MN, B_MN, GATHER>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int tiles = ((p.M + BM - 1) / BM) * ((p.n_per_head + BN - 1) / BN) * p.heads;
  const int grid = tiles < sms ? tiles : sms;
  static int pdl = -1;          // LOOM_PDL=0 turns programmatic dependent launch off
  if (pdl < 0) { const char* e = getenv("LOOM_PDL"); pdl = (e != nullptr && e[0] == '0') ? 0 : 1; }
  if (pdl) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid); cfg.blockDim = dim3(NUM_THREADS); cfg.dynamicSmemBytes = C::SMEM; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    return (int)cudaLaunchKernelEx(&cfg, gemm_kernel<BN, A_MN, B_MN, GATHER>, p);
  }
  gemm_kernel<BN, A_MN, B_MN, GATHER><<<grid, NUM_THREADS, C::SMEM, stream>>>(p);
  return (int)cudaGetLastError();
}

template <int BN>
int dispatch_major(const Params& p, bool a_mn, bool b_mn, int sms, cudaStream_t stream) {
  if (a_mn) return b_mn ? launch<BN, true, true>(p, sms, stream) : launch<BN, true, false>(p, sms, stream);
  return b_mn ? launch<BN, false, true>(p, sms, stream) : launch<BN, false, false>(p, sms, stream);
}

template <int BN, bool A_MN, bool B_MN>
int launch_pair(const Params& p, int sms, cudaStream_t stream) {
  using C = PairCfg<BN>;
  static bool configured = false;
  static int max_pairs = 0;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_pair_kernel<BN, A_MN, B_MN>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
    if (e != cudaSuccess) return (int)e;
    // how many clusters of two fit the device at once (a GPC with an odd number of free SMs loses one)
    cudaLaunchConfig_t q = {};
    q.gridDim = dim3(sms & ~1); q.blockDim = dim3(NUM_THREADS); q.dynamicSmemBytes = C::SMEM;
    cudaLaunchAttribute qa[1];
    qa[0].id = cudaLaunchAttributeClusterDimension;
    qa[0].val.clusterDim.x = 2; qa[0].val.clusterDim.y = 1; qa[0].val.clusterDim.z = 1;
    q.attrs = qa; q.numAttrs = 1;
    int n = 0;
    e = cudaOccupancyMaxActiveClusters(&n, gemm_pair_kernel<BN, A_MN, B_MN>, &q);
    if (e != cudaSuccess || n < 1) { cudaGetLastError(); n = sms / 2; }
    max_pairs = n;
    configured = true;
  }
  const int tiles = ((p.M + 2 * BM - 1) / (2 * BM)) * ((p.n_per_head + BN - 1) / BN) * p.heads;
  const int pairs = tiles < max_pairs ? tiles : max_pairs;
  static int pdl = -1;
  if (pdl < 0) { const char* e = getenv("LOOM_PDL"); pdl = (e != nullptr && e[0] == '0') ? 0 : 1; }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs); cfg.blockDim = dim3(NUM_THREADS); cfg.dynamicSmemBytes = C::SMEM; cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = pdl ? 2 : 1;
  return (int)cudaLaunchKernelEx(&cfg, gemm_pair_kernel<BN, A_MN, B_MN>, p);
}

template <int BN>
int dispatch_major_pair(const Params& p, bool a_mn, bool b_mn, int sms, cudaStream_t stream) {
  if (a_mn) return b_mn ? launch_pair<BN, true, true>(p, sms, stream) : launch_pair<BN, true, false>(p, sms, stream);
  return b_mn ? launch_pair<BN, false, true>(p, sms, stream) : launch_pair<BN, false, false>(p, sms, stream);
}

}  // namespace

extern "C" int loom_gemm_bf16(const LoomGemm* g, cudaStream_t stream) {
  if (g->nseg < 1 || g->nseg > MAX_SEG) return -1;
  if (g->bn != 64 && g->bn != 128 && g->bn != 192 && g->bn != 256) return -2;
  const bool pair = g->pair != 0;
  if (g->bn == 192 && (!pair || g->a_mn_major || g->b_mn_major)) return -2;     // 192-wide tiles: K-major pair tiles only
  if (pair && (g->bn < 128 || g->gather_world > 1 || g->a_world > 1 || g->rs_world > 1)) return -10;
  const int b_box = pair ? g->bn / 2 : g->bn;      // B rows staged per CTA
  Params p;
  memset(&p, 0, sizeof(p));
  const bool a_mn = g->a_mn_major != 0, b_mn = g->b_mn_major != 0;
  p.b_per_seg = g->b_per_seg ? 1 : 0;
  if (!p.b_per_seg && !fill_map(&p.b, g->b, b_mn, b_box)) return -3;
  for (int s = 0; s < g->nseg; ++s) {
    if (!fill_map(&p.seg[s].a, g->a[s], a_mn, BM)) return -4;
    if (p.b_per_seg && !fill_map(&p.seg[s].b, g->bseg[s], b_mn, b_box)) return -3;
    p.seg[s].k_len = g->k_len[s];
    p.seg[s].a_k0 = g->a_k0[s];
    p.seg[s].b_k0 = g->b_k0[s];
    p.seg[s].a_batched = g->a[s].heads > 1 ? 1 : 0;
  }
  p.nseg = g->nseg;
  p.b_batched = (p.b_per_seg ? g->bseg[0].heads : g->b.heads) > 1 ? 1 : 0;
  p.c = g->c; p.ldc = g->ldc; p.ldc_head = g->ldc_head; p.bias = g->bias;
  p.M = g->M; p.n_per_head = g->N; p.heads = g->heads > 0 ? g->heads : 1;
  p.accumulate = g->accumulate; p.out_fp32 = g->out_fp32; p.status = g->status;
  if (g->rope_hd != 0) {
    const int hd = g->rope_hd;
    if (!pair || a_mn || b_mn || p.heads != 1 || (hd != 64 && hd != 96 && hd != 128) || g->bn % hd || g->accumulate ||
        g->N != (g->rope_qh + 2 * g->rope_kvh) * hd || g->rope_tc < 1 || g->M % g->rope_tc || g->rope_s < 0 ||
        g->rope_s + g->rope_tc > g->rope_t || !g->rope_cos || !g->rope_sin || !g->rope_q || !g->rope_k || !g->rope_v ||
        (g->rope_q_ld & 7) || (reinterpret_cast<uintptr_t>(g->rope_q) & 15) || (reinterpret_cast<uintptr_t>(g->rope_k) & 15) ||
        (reinterpret_cast<uintptr_t>(g->rope_v) & 15) || (reinterpret_cast<uintptr_t>(g->rope_cos) & 15) ||
        (reinterpret_cast<uintptr_t>(g->rope_sin) & 15))
      return -11;
    p.rope_hd = hd; p.rope_qh = g->rope_qh; p.rope_kvh = g->rope_kvh; p.rope_tc = g->rope_tc; p.rope_t = g->rope_t;
    p.rope_s = g->rope_s; p.rope_q_ld = g->rope_q_ld; p.rope_cos = g->rope_cos; p.rope_sin = g->rope_sin;
    p.rope_q = (__nv_bfloat16*)g->rope_q; p.rope_k = (__nv_bfloat16*)g->rope_k; p.rope_v = (__nv_bfloat16*)g->rope_v;
  }
  {
    // staged TMA epilogue whenever C can be described to the TMA unit (LOOM_GEMM_EPILOGUE=direct turns it off)
    static int want = -1;
    if (want < 0) { const char* e = getenv("LOOM_GEMM_EPILOGUE"); want = (e != nullptr && e[0] == 'd') ? 0 : 1; }
    const long long es = g->out_fp32 ? 4 : 2;
    const bool ok = want && g->rope_hd == 0 && g->rs_world <= 1 && (reinterpret_cast<uintptr_t>(g->c) & 15) == 0 && (g->ldc * es) % 16 == 0 &&
                    (p.heads <= 1 || (g->ldc_head * es) % 16 == 0);
    p.c_tma = (ok && fill_c_map(&p.cmap, g->c, p.M, p.n_per_head, p.heads, g->ldc, g->ldc_head, g->out_fp32 != 0)) ? 1 : 0;
  }
  // K-major: 8-row groups are 1024 B apart (SBO); LBO unused.  MN-major: 64-element blocks along MN are
  // 8192 B apart (LBO), 8-row groups along K are 1024 B apart (SBO).
  p.a_lbo = a_mn ? 8192 : 0; p.a_sbo = 1024;
  p.b_lbo = b_mn ? 8192 : 0; p.b_sbo = 1024;
  if (g->swap_mn_strides) {
    if (a_mn) { p.a_lbo = 1024; p.a_sbo = 8192; }
    if (b_mn) { p.b_lbo = 1024; p.b_sbo = 8192; }
  }
  static int sms = 0;
  if (sms == 0) { int dev = 0; cudaGetDevice(&dev); cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev); }
  if (g->a_world > 1) {
    if (a_mn || g->nseg != 1 || p.heads != 1 || g->a_world > 8 || g->a_rows_per_rank % BM) return -7;
    p.a_world = g->a_world; p.a_rows_per_rank = g->a_rows_per_rank;
    for (int r = 0; r < g->a_world; ++r) {
      LoomOperand o = g->a[0];
      o.ptr = g->a_peer_ptr[r];
      if (!fill_map(&p.a_peer[r], o, false, BM)) return -8;
    }
  }
  if (g->rs_world > 1) {
    if (!g->out_fp32 || p.heads != 1 || g->rs_world > 8 || g->rs_rows_per_rank < 1) return -9;
    p.rs_world = g->rs_world; p.rs_rank = g->rs_rank; p.rs_rows_per_rank = g->rs_rows_per_rank;
    for (int r = 0; r < g->rs_world; ++r) p.rs_out[r] = g->rs_out[r];
  }
  if (g->gather_world > 1) {
    // weight rows fetched from their owners: plain (unbatched, single-segment, K-major) linear layers only
    if (a_mn || b_mn || g->nseg != 1 || p.heads != 1 || p.b_per_seg || g->gather_world > 8) return -5;
    p.gather_world = g->gather_world; p.gather_rank = g->gather_rank;
    const int nb64 = (g->N + 63) / 64;
    p.gather_per = (nb64 + g->gather_world - 1) / g->gather_world;
    for (int r = 0; r < g->gather_world; ++r) {
      LoomOperand o = g->b;
      o.ptr = g->b_peer_ptr[r];
      if (!fill_map(&p.b_peer[r], o, false, 64)) return -6;
    }
    switch (g->bn) {
      case 64: return launch<64, false, false, true>(p, sms, stream);
      case 128: return launch<128, false, false, true>(p, sms, stream);
      default: return launch<256, false, false, true>(p, sms, stream);
    }
  }
  if (pair) {
    if (g->bn == 192) return launch_pair<192, false, false>(p, sms, stream);
    return g->bn == 128 ? dispatch_major_pair<128>(p, a_mn, b_mn, sms, stream)
                        : dispatch_major_pair<256>(p, a_mn, b_mn, sms, stream);
  }
  switch (g->bn) {
    case 64: return dispatch_major<64>(p, a_mn, b_mn, sms, stream);
    case 128: return dispatch_major<128>(p, a_mn, b_mn, sms, stream);
    default: return dispatch_major<256>(p, a_mn, b_mn, sms, stream);
  }
}
