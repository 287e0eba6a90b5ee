// Weight-stationary small-batch GEMM for the decode step: 17..128 activation rows.
//
//   y_s[M, N_s] = cat(pieces_s)[M, K_s] . W_s[N_s, K_s]^T (+ bias_s)        for several independent segments s per launch
//
// With a few dozen sequences per step every linear layer is still a weight-streaming problem, but there are enough
// rows for the tensor cores.  The operands are swapped with respect to the training GEMM: a CTA owns 128 rows of ONE
// weight matrix as the M side of tcgen05.mma (M = 128), the whole batch is the N side (N = 32 / 64 / 128), and the
// accumulator D^T[128 weight rows, batch] sits in 32..128 TMEM columns.  So every weight element is fetched once by one
// TMA tile load, there is no padding of the batch to a 128-row tile, and all products that wait for the same producer
// (e.g. the real, gate and depth K/V projections of one normalised stream, or the eight per-head imaginary
// projections, whose operand rows are gathered from up to five pieces by their own tensor maps) share one launch: a
// segment owns a run of the grid's CTAs.  Warp 0 produces (TMA, six-stage ring of mbarriers), one thread of warp 1
// issues the MMAs, warps 2..5 read their TMEM lane quadrant and store the transposed tile: for a fixed batch row the
// 32 lanes of a warp write 32 consecutive outputs.
// A launch with few weight tiles is a launch with few busy SMs and long serial K loops (the down projection: 6 tiles of 48
// k-blocks), so the K loop of a tile can be split over a cluster of 2 or 4 CTAs: every CTA accumulates its share of the
// k-blocks in its own TMEM, leaves the fp32 partial tile in its own shared memory, and each CTA of the cluster sums and
// stores its share of the batch rows, reading the other partial tiles through distributed shared memory.
// Launched programmatically dependent: barrier set-up, the TMEM allocation and, when the weights are an inference
// engine's own copies, the first ring of weight tiles are under way before the kernel that produces the activations
// has finished.
// Every wait is bounded (see sm100.cuh); a give-up is recorded in the status word and the CTA frees its TMEM and
// returns.
// The reference runs these layers as F.linear calls from a host loop per token (reference loomformer.py:3951-4091).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include "launch_util.cuh"
#include "loom_c_api.h"
#include "sm100.cuh"
#include "tma_host.h"

namespace {

using namespace sm100;
typedef __nv_bfloat16 bf16;

constexpr int WT = 128;           // weight rows per CTA = M of the MMA
constexpr int BK = 64;            // 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int STAGES = 6;
constexpr int THREADS = 192;      // warp 0: TMA, warp 1: MMA, warps 2-5: epilogue

struct Piece {
  CUtensorMap x;                  // [M, len] rows of this piece, box 64 x MB
  int len;
  int pad_[15];
};
struct Seg {
  CUtensorMap w;                  // [N, K] weight rows, box 64 x 128
  Piece piece[LOOM_SKINNY_MAX_PIECE];
  const float* bias;
  void* y;
  long long ldy;
  int npiece, N, out_fp32, tile0;
  int pad_[8];
};
struct Params {
  Seg seg[LOOM_SKINNY_MAX_SEG];
  int nseg, M, weights_static, pad_;
  int* status;
};

template <int MB, int KS>
__global__ void __launch_bounds__(THREADS, 1) decode_gemm_kernel(const __grid_constant__ Params p) {
  constexpr int A_BYTES = WT * BK * 2;
  constexpr int B_BYTES = MB * BK * 2;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int TCOLS = MB < 32 ? 32 : MB;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  volatile int* status = p.status;

  const int tile = (int)blockIdx.x / KS;                  // the KS CTAs of a cluster share one weight tile
  const int rank = KS > 1 ? (int)cluster_ctarank() : 0;
  int si = 0;
  for (int i = 1; i < p.nseg; ++i)
    if (tile >= p.seg[i].tile0) si = i;
  const Seg& sg = p.seg[si];
  const int n0 = (tile - sg.tile0) * WT;
  int kblocks_all = 0;
  for (int i = 0; i < sg.npiece; ++i) kblocks_all += (sg.piece[i].len + BK - 1) / BK;
  // this CTA's share of the k-blocks (numbered across the pieces)
  const int per = (kblocks_all + KS - 1) / KS;
  const int kb_lo = rank * per;
  const int kb_hi = kb_lo + per < kblocks_all ? kb_lo + per : kblocks_all;
  const int kblocks = kb_hi > kb_lo ? kb_hi - kb_lo : 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    mbar_init(acc_full, 1);
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, TCOLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  loom::pdl_trigger();

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (elect_one()) {
      tma_prefetch_desc(&sg.w);
      for (int i = 0; i < sg.npiece; ++i) tma_prefetch_desc(&sg.piece[i].x);
      // weight tiles of the first ring before the activations exist
      const int pre = p.weights_static ? (kblocks < STAGES ? kblocks : STAGES) : 0;
      {
        int it = 0, kw0 = 0, gk = 0;
        for (int pi = 0; pi < sg.npiece && it < pre; ++pi) {
          for (int k = 0; k < sg.piece[pi].len && it < pre; k += BK, ++gk) {
            if (gk < kb_lo || gk >= kb_hi) continue;
            mbar_expect_tx(&full[it], STAGE_BYTES);
            tma_load_2d(smem + it * STAGE_BYTES, &sg.w, &full[it], kw0 + k, n0);
            ++it;
          }
          kw0 += sg.piece[pi].len;
        }
      }
      loom::pdl_wait();
      uint32_t it = 0;
      int kw0 = 0, gk = 0;
      bool ok = true;
      for (int pi = 0; pi < sg.npiece && ok; ++pi) {
        const Piece& pc = sg.piece[pi];
        for (int k = 0; k < pc.len; k += BK, ++gk) {
          if (gk < kb_lo || gk >= kb_hi) continue;
          const int st = it % STAGES;
          uint8_t* sa = smem + st * STAGE_BYTES;
          if ((int)it >= pre) {
            if (!mbar_wait(&empty[st], ((it / STAGES) & 1) ^ 1, status, 111)) { ok = false; break; }
            mbar_expect_tx(&full[st], STAGE_BYTES);
            tma_load_2d(sa, &sg.w, &full[st], kw0 + k, n0);
          }
          tma_load_2d(sa + A_BYTES, &pc.x, &full[st], k, 0);
          ++it;
        }
        kw0 += pc.len;
      }
    } else {
      loom::pdl_wait();
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    loom::pdl_wait();
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc_bf16(WT, MB, 0, 0);
      bool ok = true;
      for (int kb = 0; kb < kblocks; ++kb) {
        const int st = kb % STAGES;
        if (!mbar_wait(&full[st], (kb / STAGES) & 1, status, 113)) { ok = false; break; }
        tc_fence_after();
        const uint32_t sa = smem_u32(smem + st * STAGE_BYTES);
        const uint32_t sb = sa + A_BYTES;
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k) {
          const uint64_t da = make_smem_desc_sw128(sa + k * (UMMA_K * 2), 0, 1024);
          const uint64_t db = make_smem_desc_sw128(sb + k * (UMMA_K * 2), 0, 1024);
          mma_bf16_ss(tmem_base, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
        }
        mma_commit(&empty[st]);
      }
      if (ok && kblocks > 0) mma_commit(acc_full);
    }
  } else {
    // ---------------------------------------------------------------- epilogue (warps 2..5): transposed store
    loom::pdl_wait();
    const int q = warp & 3;                               // TMEM lane quadrant this warp may access
    const bool got = kblocks == 0 || mbar_wait(acc_full, 0, status, 114);
    if (got) {
      tc_fence_after();
      const int n = n0 + q * 32 + lane;
      const float b = (sg.bias != nullptr && n < sg.N) ? sg.bias[n] : 0.f;
      const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16);
      float* part = reinterpret_cast<float*>(smem);       // [MB][128] fp32 partial tile (the stage ring is drained)
#pragma unroll
      for (int c0 = 0; c0 < MB; c0 += 32) {
        uint32_t r[32];
        if (kblocks > 0) {
          tmem_ld_32x32(taddr + c0, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0u;         // no k-block fell to this CTA: its partial is zero
        }
        if (KS > 1) {
#pragma unroll
          for (int j = 0; j < 32; ++j) part[(c0 + j) * WT + q * 32 + lane] = __uint_as_float(r[j]);
        } else if (n < sg.N) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int m = c0 + j;
            if (m < p.M) {
              const float v = __uint_as_float(r[j]) + b;
              if (sg.out_fp32) reinterpret_cast<float*>(sg.y)[(long long)m * sg.ldy + n] = v;
              else reinterpret_cast<bf16*>(sg.y)[(long long)m * sg.ldy + n] = __float2bfloat16(v);
            }
          }
        }
      }
    }
  }

  if (KS > 1) {
    // every CTA's partial tile is in its own shared memory; CTA r of the cluster adds up and stores the batch rows
    // m = r, r + KS, ... (reads of the other CTAs' tiles go through distributed shared memory, several in flight)
    __syncthreads();
    cluster_arrive();
    cluster_wait();
    if (warp >= 2) {
      const int q = warp & 3;
      const int n = n0 + q * 32 + lane;
      const float b = (sg.bias != nullptr && n < sg.N) ? sg.bias[n] : 0.f;
      const uint32_t mine = smem_u32(smem) + uint32_t(q * 32 + lane) * 4;
      uint32_t peer[KS];
#pragma unroll
      for (int r = 0; r < KS; ++r) peer[r] = mapa_shared(mine, r);
      if (n < sg.N) {
#pragma unroll 4
        for (int m = rank; m < p.M; m += KS) {
          float v = b;
#pragma unroll
          for (int r = 0; r < KS; ++r) v += ld_shared_cluster_f32(peer[r] + uint32_t(m) * WT * 4);
          if (sg.out_fp32) reinterpret_cast<float*>(sg.y)[(long long)m * sg.ldy + n] = v;
          else reinterpret_cast<bf16*>(sg.y)[(long long)m * sg.ldy + n] = __float2bfloat16(v);
        }
      }
    }
    cluster_arrive();                                     // nobody leaves while its shared memory may still be read
    cluster_wait();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, TCOLS);
}

template <int MB, int KS>
int launch_decode_gemm(const Params& p, int tiles, cudaStream_t st) {
  constexpr int SMEM = STAGES * (WT * BK * 2 + MB * BK * 2) + 1024 + 256;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(decode_gemm_kernel<MB, KS>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tiles * KS); cfg.blockDim = dim3(THREADS); cfg.dynamicSmemBytes = SMEM; cfg.stream = st;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (KS > 1) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = KS; attr[na].val.clusterDim.y = 1; attr[na].val.clusterDim.z = 1;
    ++na;
  }
  if (loom::pdl_enabled()) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attr; cfg.numAttrs = na;
  return (int)cudaLaunchKernelEx(&cfg, decode_gemm_kernel<MB, KS>, p);
}

template <int MB>
int launch_decode_gemm_ks(const Params& p, int tiles, int ks, cudaStream_t st) {
  if (ks == 4) return launch_decode_gemm<MB, 4>(p, tiles, st);
  if (ks == 2) return launch_decode_gemm<MB, 2>(p, tiles, st);
  return launch_decode_gemm<MB, 1>(p, tiles, st);
}

}  // namespace

// Same segment description as loom_skinny_multi, for 1..128 rows (meant for more than 16); `status`: device word that a
// bounded wait sets when it gives up.
extern "C" int loom_decode_gemm(const LoomSkinnyArgs* a, int* status, cudaStream_t st) {
  if (a == nullptr || a->nseg < 1 || a->nseg > LOOM_SKINNY_MAX_SEG || a->M < 1 || a->M > 128 || status == nullptr) return -1;
  const int MB = a->M <= 32 ? 32 : (a->M <= 64 ? 64 : 128);
  static Params p;                                       // large; host code is single-threaded per process here
  memset(&p, 0, sizeof(p));
  p.nseg = a->nseg; p.M = a->M; p.weights_static = a->weights_static; p.status = status;
  int tiles = 0, min_kb = 1 << 30;
  for (int i = 0; i < a->nseg; ++i) {
    const LoomSkinnySeg& s = a->seg[i];
    Seg& d = p.seg[i];
    if (s.N < 1 || s.K < 8 || (s.K & 7) || (s.ldw & 7) || s.npiece < 1 || s.npiece > LOOM_SKINNY_MAX_PIECE) return -1;
    if (reinterpret_cast<uintptr_t>(s.w) & 15) return -1;
    if (!tma_host::make_2d_bf16(&d.w, s.w, (uint64_t)s.N, (uint64_t)s.K, (uint64_t)s.ldw, BK, WT)) return -3;
    int k = 0;
    for (int j = 0; j < s.npiece; ++j) {
      const LoomSkinnyPiece& pc = s.piece[j];
      if (pc.len < 8 || (pc.len & 7) || (reinterpret_cast<uintptr_t>(pc.x) & 15)) return -1;
      long long ld = pc.ld;
      if (a->M == 1) ld = (pc.len + 7) & ~7;
      if (ld < pc.len || (ld & 7)) return -1;
      if (!tma_host::make_2d_bf16(&d.piece[j].x, pc.x, (uint64_t)a->M, (uint64_t)pc.len, (uint64_t)ld, BK, MB)) return -3;
      d.piece[j].len = pc.len;
      k += pc.len;
    }
    if (k != s.K) return -1;
    {
      int kb = 0;
      for (int j = 0; j < s.npiece; ++j) kb += (s.piece[j].len + BK - 1) / BK;
      if (kb < min_kb) min_kb = kb;
    }
    d.npiece = s.npiece; d.bias = s.bias; d.y = s.y; d.ldy = s.ldy; d.N = s.N; d.out_fp32 = s.out_fp32;
    d.tile0 = tiles;
    tiles += (s.N + WT - 1) / WT;
  }
  // split the K loop over a cluster while that still fits the SMs and leaves every CTA a few k-blocks
  // (LOOM_DECODE_SPLITK=0 keeps one CTA per tile)
  static int sms = 0, want = -1;
  if (sms == 0) { int dev = 0; cudaGetDevice(&dev); cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev); }
  if (want < 0) { const char* e = getenv("LOOM_DECODE_SPLITK"); want = (e != nullptr && e[0] == '0') ? 0 : 1; }
  int ks = 1;
  if (want) {
    if (tiles * 4 <= sms && min_kb >= 8) ks = 4;
    else if (tiles * 2 <= sms && min_kb >= 4) ks = 2;
  }
  if (MB == 32) return launch_decode_gemm_ks<32>(p, tiles, ks, st);
  if (MB == 64) return launch_decode_gemm_ks<64>(p, tiles, ks, st);
  return launch_decode_gemm_ks<128>(p, tiles, ks, st);
}
