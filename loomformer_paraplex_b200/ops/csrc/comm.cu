// Fused gradient reduce-scatter + clip + sharded AdamW + parameter all-gather over NVLink peer memory.
//
// Every rank owns a contiguous range of 256-element parameter blocks.  With the flat gradient, parameter
// and bf16-shadow buffers of all ranks mapped into each other's address space (symmetric memory):
//   kernel 1  waits until every peer has published "gradients ready", then each rank sums ITS block range
//             over all peers' gradient buffers with plain P2P loads (or one multimem.ld_reduce through the
//             NVSwitch when a multicast mapping exists), keeps the mean in its own buffer and accumulates
//             the squared norm of its shard;
//   kernel 2  exchanges the per-shard squared norms (one float per peer), derives the global clip
//             coefficient and finite flag, applies AdamW to the shard and stores the refreshed fp32 and
//             bf16 parameters straight into EVERY peer's buffers (the all-gather), then publishes "done";
//   kernel 3  waits for every peer's "done" so the next forward reads complete parameters.
// No NCCL call, no staging copies, no host round trip.  All cross-GPU waits poll a flag a bounded number
// of times; on expiry the kernel records a code in the status word and carries on, so a missing peer
// produces an error on the host instead of a hung GPU.
//
// The reference relies on torch DistributedDataParallel's bucketed NCCL all-reduce followed by a
// replicated per-tensor optimizer (reference loomformer.py:4783-4792, 5154-5159).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include "loom_c_api.h"

namespace {

constexpr int BLK = 256;
constexpr int MAXW = 8;
constexpr unsigned long long WAIT_CYCLES = 6000000000ull;   // ~3 s at 2 GHz

struct P2P {
  float* grads[MAXW];
  float* params[MAXW];
  __nv_bfloat16* shadow[MAXW];
  int* sync[MAXW];           // per-rank sync words (symmetric)
  float* mc_grads;           // multicast mapping of the gradient buffers, or null
  int W, rank;
  long long blk_lo, blk_hi;  // this rank's block range (used when owner_blk is null)
  long long nblk;
  // sharded-parameter mode: an explicit owner per 256-element block, a compact slot index into the owner's m / v
  // arrays, and a flag telling whether the refreshed block is stored to every peer (small replicated tensors) or
  // only kept by its owner (GEMM weights, which the consuming GEMM of the next step fetches from the owner)
  const uint8_t* owner_blk;
  const int* slot_blk;
  const uint8_t* replicate_blk;
  // per-layer running radii of the phase input (one float per layer), made identical on every rank by the same
  // exchange that carries the shard norms: mean over ranks, or rank 0's values
  float* anchors;
  int n_anchor, anchor_rank0;
};

__device__ __forceinline__ bool owns(const P2P& c, long long b) {
  return c.owner_blk ? (c.owner_blk[b] == c.rank) : (b >= c.blk_lo && b < c.blk_hi);
}

// sync word layout (int32 words)
__device__ __forceinline__ int* w_ready(int* s, int src) { return s + src; }
__device__ __forceinline__ int* w_sumsq(int* s, int W, int src) { return s + W + src; }
__device__ __forceinline__ int* w_normflag(int* s, int W, int src) { return s + 2 * W + src; }
__device__ __forceinline__ int* w_done(int* s, int W, int src) { return s + 3 * W + src; }
__device__ __forceinline__ int* w_local(int* s, int W, int i) { return s + 4 * W + i; }   // 0: gate1, 1: gate2, 2: counter, 3: epoch
constexpr int ANCHOR_BASE = 64, ANCHOR_MAX = 64;   // words [64 + src * 64, ...): rank src's radii, written by src
__device__ __forceinline__ float* w_anchor(int* s, int src) { return reinterpret_cast<float*>(s + ANCHOR_BASE + src * ANCHOR_MAX); }

// thread 0, before the norm flag is released: this rank's radii go into its slot on every peer
__device__ void anchors_push(const P2P& c) {
  for (int p = 0; p < c.W; ++p) {
    volatile float* dst = w_anchor(c.sync[p], c.rank);
    for (int i = 0; i < c.n_anchor; ++i) dst[i] = c.anchors[i];
  }
}
// thread 0, after every peer's norm flag has arrived: all slots of the local sync buffer are complete
__device__ void anchors_pull(const P2P& c) {
  int* my = c.sync[c.rank];
  const float inv = 1.f / c.W;
  for (int i = 0; i < c.n_anchor; ++i) {
    float v = 0.f;
    if (c.anchor_rank0) v = *reinterpret_cast<volatile float*>(w_anchor(my, 0) + i);
    else { for (int p = 0; p < c.W; ++p) v += *reinterpret_cast<volatile float*>(w_anchor(my, p) + i); v *= inv; }
    c.anchors[i] = v;
  }
}

__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ bool wait_flag(const int* p, int want, int* status, int code) {
  const unsigned long long t0 = clock64();
  while (ld_acquire_sys(p) < want) {
    if (clock64() - t0 > WAIT_CYCLES) { atomicCAS(status, 0, code); return false; }
    __nanosleep(200);
  }
  return true;
}

// block 0 / thread 0 opens the gate for the rest of the grid once the cross-GPU condition holds
__device__ void grid_gate_wait(int* gate, int epoch, int* status, int code) {
  if (threadIdx.x == 0) wait_flag(gate, epoch, status, code);
  __syncthreads();
}

__global__ void __launch_bounds__(256) rs_reduce_kernel(P2P c, float* __restrict__ sumsq_local, int* status) {
  int* my = c.sync[c.rank];
  const int epoch = *w_local(my, c.W, 3) + 1;
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    __threadfence_system();
    for (int p = 0; p < c.W; ++p) st_release_sys(w_ready(c.sync[p], c.rank), epoch);     // my gradients are ready
    bool ok = true;
    for (int p = 0; p < c.W && ok; ++p) ok = wait_flag(w_ready(my, p), epoch, status, 401);
    st_release_sys(w_local(my, c.W, 0), epoch);
  }
  grid_gate_wait(w_local(my, c.W, 0), epoch, status, 402);
  const float invW = 1.f / c.W;
  float ss = 0.f;
  float* mine = c.grads[c.rank];
  // four 256-element blocks per CUDA block and iteration: 64 lanes of float4 each
  const long long first = c.owner_blk ? 0 : c.blk_lo, last = c.owner_blk ? c.nblk : c.blk_hi;
  for (long long b = first + (long long)blockIdx.x * 4 + (threadIdx.x >> 6); b < last; b += (long long)gridDim.x * 4) {
    if (!owns(c, b)) continue;
    const long long i = b * (BLK / 4) + (threadIdx.x & 63);
    float4 a;
    if (c.mc_grads) {
      asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                   : "=f"(a.x), "=f"(a.y), "=f"(a.z), "=f"(a.w) : "l"(reinterpret_cast<const float4*>(c.mc_grads) + i) : "memory");
    } else {
      a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
      for (int p = 0; p < c.W; ++p) {
        const float4 v = reinterpret_cast<const float4*>(c.grads[(c.rank + p) % c.W])[i];
        a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
      }
    }
    a.x *= invW; a.y *= invW; a.z *= invW; a.w *= invW;
    reinterpret_cast<float4*>(mine)[i] = a;
    ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  __shared__ float sh[8];
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < 8; ++i) t += sh[i];
    atomicAdd(sumsq_local, t);
  }
}

// hyper: [0] lr, [1] beta1, [2] beta2, [3] eps, [4] bias-correction 1, [5] bias-correction 2
__global__ void __launch_bounds__(256) update_allgather_kernel(P2P c, float* __restrict__ sumsq_local, float max_norm,
                                                               float* __restrict__ m, float* __restrict__ v,
                                                               const float* __restrict__ lr_mult,
                                                               const float* __restrict__ wd_blk,
                                                               const float* __restrict__ active,
                                                               const float* __restrict__ hyper, float* __restrict__ stats,
                                                               int* status) {
  int* my = c.sync[c.rank];
  const int epoch = *w_local(my, c.W, 3) + 1;
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    // a bounded wait that gave up anywhere in this step (GEMM barriers, the gradient-ready wait above) makes this
    // rank's contribution NaN: every rank then sees a non-finite norm and skips the update together
    const float mine = (*reinterpret_cast<volatile int*>(status) != 0) ? __int_as_float(0x7fc00000) : *sumsq_local;
    for (int p = 0; p < c.W; ++p) *reinterpret_cast<volatile float*>(w_sumsq(c.sync[p], c.W, c.rank)) = mine;
    if (c.n_anchor > 0) anchors_push(c);
    __threadfence_system();
    for (int p = 0; p < c.W; ++p) st_release_sys(w_normflag(c.sync[p], c.W, c.rank), epoch);
    bool ok = true;
    float tot = 0.f;
    for (int p = 0; p < c.W && ok; ++p) {
      ok = wait_flag(w_normflag(my, c.W, p), epoch, status, 403);
      tot += *reinterpret_cast<volatile float*>(w_sumsq(my, c.W, p));
    }
    if (ok && c.n_anchor > 0) anchors_pull(c);
    const float norm = sqrtf(tot);
    const bool fin = isfinite(norm) && ok;
    stats[0] = norm;
    stats[1] = (max_norm > 0.f && fin) ? fminf(1.f, max_norm / (norm + 1e-6f)) : 1.f;
    stats[2] = fin ? 1.f : 0.f;
    if (!fin) stats[3] += 1.f;          // sticky count of skipped updates, read at log cadence
    *sumsq_local = 0.f;
    __threadfence();
    st_release_sys(w_local(my, c.W, 1), epoch);
  }
  grid_gate_wait(w_local(my, c.W, 1), epoch, status, 404);
  const float clip = *reinterpret_cast<volatile float*>(stats + 1);
  const bool fin = *reinterpret_cast<volatile float*>(stats + 2) != 0.f;
  const float lr0 = hyper[0], b1 = hyper[1], b2 = hyper[2], eps = hyper[3], bc1 = hyper[4], bc2 = hyper[5];
  const float* g = c.grads[c.rank];
  float* pl = c.params[c.rank];
  const long long first = c.owner_blk ? 0 : c.blk_lo, last = c.owner_blk ? c.nblk : c.blk_hi;
  for (long long b = first + blockIdx.x; b < last; b += gridDim.x) {
    if (!owns(c, b)) continue;
    const long long i = b * BLK + threadIdx.x;
    const long long mi = (c.slot_blk ? (long long)c.slot_blk[b] : b) * BLK + threadIdx.x;   // moments may be compact
    float pp = pl[i];
    if (fin && active[b] != 0.f) {
      const float lr = lr0 * lr_mult[b];
      const float gg = g[i] * clip;
      const float mm = m[mi] + (1.f - b1) * (gg - m[mi]);
      const float vv = v[mi] + (1.f - b2) * (gg * gg - v[mi]);
      pp = pp * (1.f - lr * wd_blk[b]) - lr * (mm / bc1) / (sqrtf(vv / bc2) + eps);
      m[mi] = mm; v[mi] = vv;
    }
    const __nv_bfloat16 pb = __float2bfloat16(pp);
    if (c.replicate_blk == nullptr || c.replicate_blk[b]) {
      for (int p = 0; p < c.W; ++p) {               // all-gather by direct stores into every peer
        const int q = (c.rank + p) % c.W;
        c.params[q][i] = pp;
        c.shadow[q][i] = pb;
      }
    } else {                                        // sharded weight: the owner keeps it; readers fetch it on use
      pl[i] = pp;
      c.shadow[c.rank][i] = pb;
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int done = atomicAdd(w_local(my, c.W, 2), 1);
    if (done == (int)gridDim.x - 1) {
      *w_local(my, c.W, 2) = 0;
      __threadfence_system();
      for (int p = 0; p < c.W; ++p) st_release_sys(w_done(c.sync[p], c.W, c.rank), epoch);
    }
  }
}

__global__ void wait_done_kernel(P2P c, int* status) {
  int* my = c.sync[c.rank];
  const int epoch = *w_local(my, c.W, 3) + 1;
  bool ok = true;
  for (int p = 0; p < c.W && ok; ++p) ok = wait_flag(w_done(my, c.W, p), epoch, status, 405);
  *w_local(my, c.W, 3) = epoch;
}

// ---- pieces for "any optimizer on the shard": exchange the shard norms, then (after the optimizer kernel of the
// caller's choice has updated the shard in place) push the refreshed shard to every peer
__global__ void norm_exchange_kernel(P2P c, float* __restrict__ sumsq_local, float max_norm, float* __restrict__ stats,
                                     int* status) {
  if (threadIdx.x != 0) return;
  int* my = c.sync[c.rank];
  const int epoch = *w_local(my, c.W, 3) + 1;
  const float mine = (*reinterpret_cast<volatile int*>(status) != 0) ? __int_as_float(0x7fc00000) : *sumsq_local;
  for (int p = 0; p < c.W; ++p) *reinterpret_cast<volatile float*>(w_sumsq(c.sync[p], c.W, c.rank)) = mine;
  if (c.n_anchor > 0) anchors_push(c);
  __threadfence_system();
  for (int p = 0; p < c.W; ++p) st_release_sys(w_normflag(c.sync[p], c.W, c.rank), epoch);
  bool ok = true;
  float tot = 0.f;
  for (int p = 0; p < c.W && ok; ++p) {
    ok = wait_flag(w_normflag(my, c.W, p), epoch, status, 406);
    tot += *reinterpret_cast<volatile float*>(w_sumsq(my, c.W, p));
  }
  if (ok && c.n_anchor > 0) anchors_pull(c);
  const float norm = sqrtf(tot);
  const bool fin = isfinite(norm) && ok;
  stats[0] = norm;
  stats[1] = (max_norm > 0.f && fin) ? fminf(1.f, max_norm / (norm + 1e-6f)) : 1.f;
  stats[2] = fin ? 1.f : 0.f;
  if (!fin) stats[3] += 1.f;
  *sumsq_local = 0.f;
}

__global__ void __launch_bounds__(256) allgather_push_kernel(P2P c) {
  int* my = c.sync[c.rank];
  const int epoch = *w_local(my, c.W, 3) + 1;
  const float* pl = c.params[c.rank];
  const __nv_bfloat16* sl = c.shadow[c.rank];
  for (long long b = c.blk_lo + blockIdx.x; b < c.blk_hi; b += gridDim.x) {
    const long long i = b * BLK + threadIdx.x;
    const float pp = pl[i];
    const __nv_bfloat16 pb = sl[i];
    for (int p = 1; p < c.W; ++p) {
      const int q = (c.rank + p) % c.W;
      c.params[q][i] = pp;
      c.shadow[q][i] = pb;
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int done = atomicAdd(w_local(my, c.W, 2), 1);
    if (done == (int)gridDim.x - 1) {
      *w_local(my, c.W, 2) = 0;
      __threadfence_system();
      for (int p = 0; p < c.W; ++p) st_release_sys(w_done(c.sync[p], c.W, c.rank), epoch);
    }
  }
}

struct Peers { int* f[MAXW]; };

__global__ void tp_barrier_kernel(Peers pp, int world, int rank, int epoch, int* status, int code) {
  __threadfence_system();                                   // everything this rank sent before is visible first
  if (threadIdx.x < world) st_release_sys(pp.f[threadIdx.x] + rank, epoch);
  if (threadIdx.x < world) wait_flag(pp.f[rank] + threadIdx.x, epoch, status, code);
}

}  // namespace

extern "C" int loom_tp_barrier(int* const* flags_peer, int world, int rank, int epoch, int* status, int code,
                               cudaStream_t stream) {
  if (world < 1 || world > MAXW) return -1;
  Peers pp;
  for (int i = 0; i < world; ++i) pp.f[i] = flags_peer[i];
  tp_barrier_kernel<<<1, 32, 0, stream>>>(pp, world, rank, epoch, status, code);
  return (int)cudaGetLastError();
}

static void fill_p2p(const LoomP2P* a, P2P& c) {
  for (int p = 0; p < a->W; ++p) {
    c.grads[p] = a->grads[p]; c.params[p] = a->params[p];
    c.shadow[p] = reinterpret_cast<__nv_bfloat16*>(a->shadow[p]); c.sync[p] = a->sync[p];
  }
  c.mc_grads = a->mc_grads; c.W = a->W; c.rank = a->rank; c.nblk = a->nblk;
  c.owner_blk = nullptr; c.slot_blk = nullptr; c.replicate_blk = nullptr;
  c.anchors = a->anchors; c.n_anchor = a->anchors ? a->n_anchor : 0; c.anchor_rank0 = a->anchor_rank0;
  const long long per = (a->nblk + a->W - 1) / a->W;
  c.blk_lo = per * a->rank < a->nblk ? per * a->rank : a->nblk;
  c.blk_hi = per * (a->rank + 1) < a->nblk ? per * (a->rank + 1) : a->nblk;
}

// Reduce-scatter + global norm, then ATOM on this rank's contiguous shard (the one-launch kernel of optim.cu, pointed
// at the shard), then the refreshed shard pushed to every peer.  The per-block ATOM statistics (gprev / pnode / trust)
// and the moments are therefore current only on the rank that owns the block.
extern "C" int loom_p2p_grad_step_atom(const LoomP2P* a, const float* cnt_blk, float* gprev, float* pnode, float* trust,
                                       float* atom_out, cudaStream_t stream) {
  if (a->W < 1 || a->W > MAXW) return -1;
  if (a->anchors && (a->n_anchor < 0 || a->n_anchor > ANCHOR_MAX)) return -2;
  P2P c;
  fill_p2p(a, c);
  static int sms = 0;
  if (sms == 0) { int dev = 0; cudaGetDevice(&dev); cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev); }
  const int grid = sms * 2;
  rs_reduce_kernel<<<grid, 256, 0, stream>>>(c, a->sumsq_local, a->status);
  norm_exchange_kernel<<<1, 32, 0, stream>>>(c, a->sumsq_local, a->max_norm, a->stats, a->status);
  const long long lo = c.blk_lo, n = c.blk_hi - c.blk_lo;
  if (n > 0) {
    cudaMemsetAsync(atom_out, 0, 3 * sizeof(float), stream);
    int rc = loom_atom_flat(a->params[a->rank] + lo * BLK, a->grads[a->rank] + lo * BLK, a->m + lo * BLK, a->v + lo * BLK,
                            reinterpret_cast<__nv_bfloat16*>(a->shadow[a->rank]) + lo * BLK, a->lr_mult + lo, a->wd_blk + lo,
                            cnt_blk + lo, gprev + lo, pnode + lo, trust + lo, a->stats, a->hyper, atom_out, n, stream);
    if (rc != 0) return rc;
  }
  allgather_push_kernel<<<grid, 256, 0, stream>>>(c);
  wait_done_kernel<<<1, 1, 0, stream>>>(c, a->status);
  return (int)cudaGetLastError();
}

extern "C" int loom_p2p_grad_step(const LoomP2P* a, cudaStream_t stream) {
  if (a->W < 1 || a->W > MAXW) return -1;
  if (a->anchors && (a->n_anchor < 0 || a->n_anchor > ANCHOR_MAX)) return -2;
  P2P c;
  for (int p = 0; p < a->W; ++p) {
    c.grads[p] = a->grads[p]; c.params[p] = a->params[p];
    c.shadow[p] = reinterpret_cast<__nv_bfloat16*>(a->shadow[p]); c.sync[p] = a->sync[p];
  }
  c.mc_grads = a->mc_grads; c.W = a->W; c.rank = a->rank; c.nblk = a->nblk;
  c.owner_blk = a->owner_blk; c.slot_blk = a->slot_blk; c.replicate_blk = a->replicate_blk;
  c.anchors = a->anchors; c.n_anchor = a->anchors ? a->n_anchor : 0; c.anchor_rank0 = a->anchor_rank0;
  const long long per = (a->nblk + a->W - 1) / a->W;
  c.blk_lo = per * a->rank < a->nblk ? per * a->rank : a->nblk;
  c.blk_hi = per * (a->rank + 1) < a->nblk ? per * (a->rank + 1) : a->nblk;
  static int sms = 0;
  if (sms == 0) { int dev = 0; cudaGetDevice(&dev); cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev); }
  const int grid = sms * 2;     // co-resident: 2 x 256 threads per SM
  rs_reduce_kernel<<<grid, 256, 0, stream>>>(c, a->sumsq_local, a->status);
  update_allgather_kernel<<<grid, 256, 0, stream>>>(c, a->sumsq_local, a->max_norm, a->m, a->v, a->lr_mult, a->wd_blk,
                                                   a->active, a->hyper, a->stats, a->status);
  wait_done_kernel<<<1, 1, 0, stream>>>(c, a->status);
  return (int)cudaGetLastError();
}
