// Small-batch pieces of the decode step.
//
// skinny_linear   y[M, N] = x[M, K] . W[N, K]^T (+ bias), M <= 16 rows.  One token per sequence makes every linear layer
//                 of the decode step a matrix-vector product: the weights are streamed once (16-byte loads, a warp per
//                 output column, fp32 accumulation, shuffle reduction) and the activations sit in shared memory.  A
//                 128-row tensor-core tile would spend its time on fixed set-up cost for one useful row.  The output may
//                 be a row-strided view, so the projection into a depth-history slot is written in place.
// skinny_multi    several such products in one launch: every segment has its own input rows (gathered from up to five
//                 pieces, e.g. the per-head operand of the imaginary projection: q | k-context | context | u | depth
//                 read), weight, bias and output view, and owns a range of the grid's blocks.  The decode step at one
//                 token per sequence is bound by the number of dependent launches, not by bytes: all products that
//                 wait for the same producer leave together.
// rope_store      rotate-half RoPE of the new token's Q and K at the device-side position, rotated Q into the
//                 attention operand buffer, rotated K and V appended to the caches: one launch instead of a dozen
//                 slicing / multiply / index-copy launches, and graph-safe because the position is read on the device.
//
// step_flags      the per-step booleans (first position, boundary fire, temporal reset, seed validity) from the device-side
//                 position and the incoming tokens: one launch instead of a dozen comparisons.
// ca_append       append the new boundary key / value rows when any sequence fired, and rebuild the mask of keys that the
//                 final cross attention may see.
//
// The reference runs these through F.linear and PyTorch indexing, relaunched from the host for every token
// (reference loomformer.py:3951-4091).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include "launch_util.cuh"
#include "loom_c_api.h"

namespace {

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 t = __bfloat1622float2(p[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}

template <int MT>
__global__ void __launch_bounds__(256) skinny_linear_kernel(const bf16* __restrict__ x, long long ldx,
                                                            const bf16* __restrict__ w, long long ldw,
                                                            const float* __restrict__ bias, void* __restrict__ y,
                                                            long long ldy, int out_fp32, int M, int N, int K) {
  extern __shared__ uint4 sx[];                       // [MT][K / 8]
  const int K8 = K >> 3;
  loom::pdl_trigger();
  loom::pdl_wait();
  for (int i = threadIdx.x; i < MT * K8; i += blockDim.x) {
    const int m = i / K8, c = i - m * K8;
    sx[i] = m < M ? *reinterpret_cast<const uint4*>(x + (long long)m * ldx + c * 8) : make_uint4(0u, 0u, 0u, 0u);
  }
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int gw = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), nw = gridDim.x * (blockDim.x >> 5);
  for (int n = gw; n < N; n += nw) {
    float acc[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m] = 0.f;
    const uint4* wr = reinterpret_cast<const uint4*>(w + (long long)n * ldw);
#pragma unroll 4
    for (int c = lane; c < K8; c += 32) {
      float wf[8];
      unpack8(wr[c], wf);
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        float xf[8];
        unpack8(sx[m * K8 + c], xf);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[m] = fmaf(wf[i], xf[i], acc[m]);
      }
    }
#pragma unroll
    for (int m = 0; m < MT; ++m) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) acc[m] += __shfl_xor_sync(0xffffffffu, acc[m], o);
    }
    if (lane == 0) {
      const float b = bias ? bias[n] : 0.f;
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        if (m < M) {
          if (out_fp32) reinterpret_cast<float*>(y)[(long long)m * ldy + n] = acc[m] + b;
          else reinterpret_cast<bf16*>(y)[(long long)m * ldy + n] = __float2bfloat16(acc[m] + b);
        }
      }
    }
  }
}

template <int MT>
int launch_skinny(const void* x, long long ldx, const void* w, long long ldw, const float* bias, void* y, long long ldy,
                  int out_fp32, int M, int N, int K, cudaStream_t st) {
  const size_t shm = (size_t)MT * K * sizeof(bf16);
  if (shm > 200 * 1024) return -2;
  if (shm > 48 * 1024) {
    static size_t configured = 0;
    if (shm > configured) {
      cudaError_t e = cudaFuncSetAttribute(skinny_linear_kernel<MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shm);
      if (e != cudaSuccess) return (int)e;
      configured = shm;
    }
  }
  static int sms = 0;
  if (sms == 0) { int dev = 0; cudaGetDevice(&dev); cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev); }
  int grid = (N + 7) / 8;
  if (grid > 4 * sms) grid = 4 * sms;
  if (grid < 1) grid = 1;
  return (int)loom::launch_pdl(skinny_linear_kernel<MT>, dim3(grid), dim3(256), shm, st, (const bf16*)x, ldx, (const bf16*)w, ldw, bias,
                               y, ldy, out_fp32, M, N, K);
}

// ---- several products in one launch ---------------------------------------------------------------------------------
template <int MT>
__global__ void __launch_bounds__(256) skinny_multi_kernel(const __grid_constant__ LoomSkinnyArgs a) {
  extern __shared__ uint4 sx[];                       // [MT][K / 8] of this block's segment
  int si = 0;
  for (int i = 1; i < a.nseg; ++i)
    if ((int)blockIdx.x >= a.seg[i].block0) si = i;
  const LoomSkinnySeg& sg = a.seg[si];
  const int nb = (si + 1 < a.nseg ? a.seg[si + 1].block0 : (int)gridDim.x) - sg.block0;
  const int lb = blockIdx.x - sg.block0;
  const int K8 = sg.K >> 3, M = a.M;
  const int lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  const bf16* w = reinterpret_cast<const bf16*>(sg.w);
  // With weights that nothing earlier in the stream writes (an inference engine's copies), the first column's row is
  // on its way (up to 1024 elements of it in registers) while the producer of the inputs is still running.
  loom::pdl_trigger();
  int n = lb * warps + (threadIdx.x >> 5);
  constexpr int PRE = 4;
  uint4 pre[PRE];
  const bool early = a.weights_static != 0;              // else the weights may be the previous kernel's output
  if (!early) loom::pdl_wait();
  if (n < sg.N) {
    const uint4* wr = reinterpret_cast<const uint4*>(w + (long long)n * sg.ldw);
#pragma unroll
    for (int j = 0; j < PRE; ++j) pre[j] = lane + 32 * j < K8 ? wr[lane + 32 * j] : make_uint4(0u, 0u, 0u, 0u);
  }
  if (early) loom::pdl_wait();
  int k0 = 0;
  for (int pi = 0; pi < sg.npiece; ++pi) {
    const bf16* px = reinterpret_cast<const bf16*>(sg.piece[pi].x);
    const long long ld = sg.piece[pi].ld;
    const int L8 = sg.piece[pi].len >> 3;
    for (int i = threadIdx.x; i < MT * L8; i += blockDim.x) {
      const int m = i / L8, c = i - m * L8;
      sx[m * K8 + k0 + c] = m < M ? *reinterpret_cast<const uint4*>(px + (long long)m * ld + c * 8) : make_uint4(0u, 0u, 0u, 0u);
    }
    k0 += L8;
  }
  __syncthreads();
  bool first = true;
  for (; n < sg.N; n += nb * warps) {
    float acc[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m] = 0.f;
    const uint4* wr = reinterpret_cast<const uint4*>(w + (long long)n * sg.ldw);
    int c = lane;
    if (first) {
      first = false;
#pragma unroll
      for (int j = 0; j < PRE; ++j) {
        if (lane + 32 * j < K8) {
          float wf[8];
          unpack8(pre[j], wf);
#pragma unroll
          for (int m = 0; m < MT; ++m) {
            float xf[8];
            unpack8(sx[m * K8 + lane + 32 * j], xf);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[m] = fmaf(wf[i], xf[i], acc[m]);
          }
        }
      }
      c = lane + 32 * PRE;
    }
#pragma unroll 4
    for (; c < K8; c += 32) {
      float wf[8];
      unpack8(wr[c], wf);
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        float xf[8];
        unpack8(sx[m * K8 + c], xf);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[m] = fmaf(wf[i], xf[i], acc[m]);
      }
    }
#pragma unroll
    for (int m = 0; m < MT; ++m) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) acc[m] += __shfl_xor_sync(0xffffffffu, acc[m], o);
    }
    if (lane == 0) {
      const float b = sg.bias ? sg.bias[n] : 0.f;
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        if (m < M) {
          if (sg.out_fp32) reinterpret_cast<float*>(sg.y)[(long long)m * sg.ldy + n] = acc[m] + b;
          else reinterpret_cast<bf16*>(sg.y)[(long long)m * sg.ldy + n] = __float2bfloat16(acc[m] + b);
        }
      }
    }
  }
}

// Variant for launches whose segments all have few columns and a long reduction (the down projection: 768 x 3072 would
// keep 96 blocks busy): `wpc` warps share a column, each with a slice of K, and their partial sums meet in shared
// memory.  Kept apart from the kernel above, whose launches it would slow down (more registers, two barriers per pass).
template <int MT>
__global__ void __launch_bounds__(256) skinny_multi_split_kernel(const __grid_constant__ LoomSkinnyArgs a) {
  extern __shared__ uint4 sx[];                       // [MT][K / 8] of this block's segment
  __shared__ float red[8][MT];
  int si = 0;
  for (int i = 1; i < a.nseg; ++i)
    if ((int)blockIdx.x >= a.seg[i].block0) si = i;
  const LoomSkinnySeg& sg = a.seg[si];
  const int nb = (si + 1 < a.nseg ? a.seg[si + 1].block0 : (int)gridDim.x) - sg.block0;
  const int lb = blockIdx.x - sg.block0;
  const int K8 = sg.K >> 3, M = a.M;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const bf16* w = reinterpret_cast<const bf16*>(sg.w);
  const int wpc = sg.wpc, cpb = warps / wpc;             // columns per block pass
  const int wcol = warp / wpc, sub = warp - wcol * wpc;
  const int per = (K8 + wpc - 1) / wpc;
  const int c_lo = sub * per, c_hi = c_lo + per < K8 ? c_lo + per : K8;
  loom::pdl_trigger();
  constexpr int PRE = 4;
  uint4 pre[PRE];
  const bool early = a.weights_static != 0;
  if (!early) loom::pdl_wait();
  {
    const int n = lb * cpb + wcol;
    if (n < sg.N) {
      const uint4* wr = reinterpret_cast<const uint4*>(w + (long long)n * sg.ldw);
#pragma unroll
      for (int j = 0; j < PRE; ++j) pre[j] = c_lo + lane + 32 * j < c_hi ? wr[c_lo + lane + 32 * j] : make_uint4(0u, 0u, 0u, 0u);
    }
  }
  if (early) loom::pdl_wait();
  int k0 = 0;
  for (int pi = 0; pi < sg.npiece; ++pi) {
    const bf16* px = reinterpret_cast<const bf16*>(sg.piece[pi].x);
    const long long ld = sg.piece[pi].ld;
    const int L8 = sg.piece[pi].len >> 3;
    for (int i = threadIdx.x; i < MT * L8; i += blockDim.x) {
      const int m = i / L8, c = i - m * L8;
      sx[m * K8 + k0 + c] = m < M ? *reinterpret_cast<const uint4*>(px + (long long)m * ld + c * 8) : make_uint4(0u, 0u, 0u, 0u);
    }
    k0 += L8;
  }
  __syncthreads();
  bool first = true;
  for (int nbase = lb * cpb; nbase < sg.N; nbase += nb * cpb) {          // the same trip count for every warp of the block
    const int n = nbase + wcol;
    const bool valid = n < sg.N;
    float acc[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m] = 0.f;
    if (valid) {
      const uint4* wr = reinterpret_cast<const uint4*>(w + (long long)n * sg.ldw);
      int c = c_lo + lane;
      if (first) {
#pragma unroll
        for (int j = 0; j < PRE; ++j) {
          if (c_lo + lane + 32 * j < c_hi) {
            float wf[8];
            unpack8(pre[j], wf);
#pragma unroll
            for (int m = 0; m < MT; ++m) {
              float xf[8];
              unpack8(sx[m * K8 + c_lo + lane + 32 * j], xf);
#pragma unroll
              for (int i = 0; i < 8; ++i) acc[m] = fmaf(wf[i], xf[i], acc[m]);
            }
          }
        }
        c = c_lo + lane + 32 * PRE;
      }
#pragma unroll 4
      for (; c < c_hi; c += 32) {
        float wf[8];
        unpack8(wr[c], wf);
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          float xf[8];
          unpack8(sx[m * K8 + c], xf);
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[m] = fmaf(wf[i], xf[i], acc[m]);
        }
      }
#pragma unroll
      for (int m = 0; m < MT; ++m) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc[m] += __shfl_xor_sync(0xffffffffu, acc[m], o);
      }
    }
    first = false;
    if (lane == 0) {
#pragma unroll
      for (int m = 0; m < MT; ++m) red[warp][m] = acc[m];
    }
    __syncthreads();
    if (valid && sub == 0 && lane == 0) {
      for (int s2 = 1; s2 < wpc; ++s2) {
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[m] += red[warp + s2][m];
      }
      const float b = sg.bias ? sg.bias[n] : 0.f;
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        if (m < M) {
          if (sg.out_fp32) reinterpret_cast<float*>(sg.y)[(long long)m * sg.ldy + n] = acc[m] + b;
          else reinterpret_cast<bf16*>(sg.y)[(long long)m * sg.ldy + n] = __float2bfloat16(acc[m] + b);
        }
      }
    }
    __syncthreads();
  }
}

template <int MT>
int launch_skinny_multi(const LoomSkinnyArgs& a, int grid, int kmax, bool split, cudaStream_t st) {
  const size_t shm = (size_t)MT * kmax * sizeof(bf16);
  if (shm > 200 * 1024) return -2;
  if (shm > 48 * 1024) {
    static size_t configured = 0;
    if (shm > configured) {
      cudaError_t e = cudaFuncSetAttribute(skinny_multi_kernel<MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shm);
      if (e != cudaSuccess) return (int)e;
      configured = shm;
    }
  }
  if (split) {
    if (shm > 48 * 1024) {
      static size_t configured2 = 0;
      if (shm > configured2) {
        cudaError_t e = cudaFuncSetAttribute(skinny_multi_split_kernel<MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shm);
        if (e != cudaSuccess) return (int)e;
        configured2 = shm;
      }
    }
    return (int)loom::launch_pdl(skinny_multi_split_kernel<MT>, dim3(grid), dim3(256), shm, st, a);
  }
  return (int)loom::launch_pdl(skinny_multi_kernel<MT>, dim3(grid), dim3(256), shm, st, a);
}

// ---- per-step flags ----------------------------------------------------------------------------------------------------
// fire[b]       the boundary fires after this token: the hard window boundary, or the carry token
// reset[b]      the temporal state restarts from this token's carriers (pending boundary, first position, no state yet)
// row_reset[b]  first position of a sequence (phase traces restart)
// seed_valid[b] layer 0 composes with the carried state
__global__ void decode_step_flags_kernel(const long long* __restrict__ pos_ptr, const long long* __restrict__ tok,
                                         const uint8_t* __restrict__ pending, const uint8_t* __restrict__ have_carry,
                                         uint8_t* __restrict__ fire, uint8_t* __restrict__ reset, uint8_t* __restrict__ row_reset,
                                         uint8_t* __restrict__ seed_valid, int B, long long window, long long seq_len,
                                         int hard_enabled, long long carry_token, int temporal) {
  loom::pdl_trigger();
  const long long pos = *pos_ptr;
  const bool bos = pos == 0, have = *have_carry != 0;
  const bool hard = hard_enabled && window > 0 && ((pos + 1) % window == 0) && (pos + 1 < seq_len);
  for (int b = blockIdx.x * blockDim.x + threadIdx.x; b < B; b += gridDim.x * blockDim.x) {
    const bool pend = pending[b] != 0;
    fire[b] = (hard || (carry_token >= 0 && tok[b] == carry_token)) ? 1 : 0;
    reset[b] = (pend || bos || !temporal || !have) ? 1 : 0;
    row_reset[b] = bos ? 1 : 0;
    seed_valid[b] = (pend && !bos && have) ? 1 : 0;
  }
}

// ---- boundary-key append -----------------------------------------------------------------------------------------------
// One block per sequence.  When any sequence fired, every sequence writes its new key / value row into the next slot
// (valid only where it fired itself).  `allowed` is the mask of slots the final cross attention may read after the
// append, `any_out` the increment of the slot count (added by the caller after this launch: every block reads the
// old count), and the pending / have-carry flags of the next step are set.
__global__ void __launch_bounds__(256) decode_ca_append_kernel(const bf16* __restrict__ newk, const bf16* __restrict__ newv,
                                                               long long ld_new, const uint8_t* __restrict__ fire,
                                                               bf16* __restrict__ ca_k, bf16* __restrict__ ca_v,
                                                               uint8_t* __restrict__ ca_valid, const long long* __restrict__ ca_len,
                                                               uint8_t* __restrict__ allowed, long long* __restrict__ any_out,
                                                               uint8_t* __restrict__ pending, uint8_t* __restrict__ have_carry,
                                                               int B, int cap, int N) {
  const int b = blockIdx.x;
  loom::pdl_trigger();
  int f = 0;
  for (int i = threadIdx.x; i < B; i += blockDim.x) f |= fire[i];
  const int any = __syncthreads_or(f);
  long long len = *ca_len;
  if (len < 0) len = 0;
  const int slot = len < cap ? (int)len : cap - 1;
  const long long new_len = len + (any ? 1 : 0);
  if (any) {
    bf16* kd = ca_k + ((long long)b * cap + slot) * N;
    bf16* vd = ca_v + ((long long)b * cap + slot) * N;
    for (int i = threadIdx.x; i < N; i += blockDim.x) {
      kd[i] = newk[(long long)b * ld_new + i];
      vd[i] = newv[(long long)b * ld_new + i];
    }
  }
  for (int j = threadIdx.x; j < cap; j += blockDim.x) {
    uint8_t v = ca_valid[(long long)b * cap + j];
    if (any && j == slot) { v = fire[b]; ca_valid[(long long)b * cap + j] = v; }
    allowed[(long long)b * cap + j] = (v && j < new_len) ? 1 : 0;
  }
  if (threadIdx.x == 0) {
    pending[b] = fire[b];
    if (b == 0) { *any_out = any ? 1 : 0; *have_carry = 1; }
  }
}

// one block per sequence; thread j of a head handles dims j and j + HD/2
__global__ void __launch_bounds__(256) decode_rope_store_kernel(const bf16* __restrict__ qkv, long long ld_qkv,
                                                                const float* __restrict__ cos_tab,
                                                                const float* __restrict__ sin_tab,
                                                                const long long* __restrict__ pos_ptr, bf16* __restrict__ q_out,
                                                                long long ld_q, bf16* __restrict__ kc, bf16* __restrict__ vc,
                                                                int S, int table_rows, int QH, int KVH, int HD) {
  const int b = blockIdx.x;
  loom::pdl_trigger();
  loom::pdl_wait();
  long long pos = *pos_ptr;
  if (pos < 0) pos = 0;
  const long long trow = pos < table_rows ? pos : table_rows - 1;      // the host refuses positions beyond the table
  const long long crow = pos < S ? pos : S - 1;
  const int half = HD >> 1;
  const float* cs = cos_tab + trow * HD;
  const float* sn = sin_tab + trow * HD;
  const bf16* row = qkv + (long long)b * ld_qkv;
  const int N = QH * HD, KV = KVH * HD;
  // rotated queries and keys
  for (int i = threadIdx.x; i < (QH + KVH) * half; i += blockDim.x) {
    const int head = i / half, j = i - head * half;
    const bf16* src = row + (long long)head * HD;               // Q heads first, then K heads: contiguous in the qkv row
    const float x0 = __bfloat162float(src[j]), x1 = __bfloat162float(src[j + half]);
    const float o0 = x0 * cs[j] - x1 * sn[j];
    const float o1 = x1 * cs[j + half] + x0 * sn[j + half];
    bf16* dst = head < QH ? q_out + (long long)b * ld_q + (long long)head * HD
                          : kc + (((long long)b * S + crow) * KVH + (head - QH)) * HD;
    dst[j] = __float2bfloat16(o0);
    dst[j + half] = __float2bfloat16(o1);
  }
  // values are appended as they are
  bf16* vdst = vc + ((long long)b * S + crow) * KV;
  for (int i = threadIdx.x; i < KV; i += blockDim.x) vdst[i] = row[N + KV + i];
}

}  // namespace

extern "C" int loom_skinny_linear(const void* x, long long ldx, const void* w, long long ldw, const float* bias, void* y,
                                  long long ldy, int out_fp32, int M, int N, int K, cudaStream_t st) {
  if (M < 1 || M > 16 || N < 1 || K < 8 || (K & 7) || (ldx & 7) || (ldw & 7)) return -1;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15)) return -1;
  if (M == 1) return launch_skinny<1>(x, ldx, w, ldw, bias, y, ldy, out_fp32, M, N, K, st);
  if (M == 2) return launch_skinny<2>(x, ldx, w, ldw, bias, y, ldy, out_fp32, M, N, K, st);
  if (M <= 4) return launch_skinny<4>(x, ldx, w, ldw, bias, y, ldy, out_fp32, M, N, K, st);
  if (M <= 8) return launch_skinny<8>(x, ldx, w, ldw, bias, y, ldy, out_fp32, M, N, K, st);
  return launch_skinny<16>(x, ldx, w, ldw, bias, y, ldy, out_fp32, M, N, K, st);
}

extern "C" int loom_decode_rope_store(const void* qkv, long long ld_qkv, const float* cos_tab, const float* sin_tab,
                                      const long long* pos, void* q_out, long long ld_q, void* kc, void* vc, int B, int S,
                                      int table_rows, int QH, int KVH, int HD, cudaStream_t st) {
  if (B < 1 || (HD & 1) || S < 1 || table_rows < 1) return -1;
  return (int)loom::launch_pdl(decode_rope_store_kernel, dim3(B), dim3(256), 0, st, (const bf16*)qkv, ld_qkv, cos_tab, sin_tab, pos,
                               (bf16*)q_out, ld_q, (bf16*)kc, (bf16*)vc, S, table_rows, QH, KVH, HD);
}

extern "C" int loom_skinny_multi(LoomSkinnyArgs* a, cudaStream_t st) {
  if (a == nullptr || a->nseg < 1 || a->nseg > LOOM_SKINNY_MAX_SEG || a->M < 1 || a->M > 16) return -1;
  static int sms = 0;
  if (sms == 0) { int dev = 0; cudaGetDevice(&dev); cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev); }
  int kmax = 0, want = 0;
  bool split = true;                    // every segment has few columns and a long reduction
  for (int i = 0; i < a->nseg; ++i) {
    LoomSkinnySeg& sg = a->seg[i];
    if (sg.N < 1 || sg.K < 8 || (sg.K & 7) || (sg.ldw & 7) || sg.npiece < 1 || sg.npiece > LOOM_SKINNY_MAX_PIECE) return -1;
    if (reinterpret_cast<uintptr_t>(sg.w) & 15) return -1;
    int k = 0;
    for (int p = 0; p < sg.npiece; ++p) {
      const LoomSkinnyPiece& pc = sg.piece[p];
      if (pc.len < 8 || (pc.len & 7) || (pc.ld & 7) || (reinterpret_cast<uintptr_t>(pc.x) & 15)) return -1;
      k += pc.len;
    }
    if (k != sg.K) return -1;
    if (sg.K > kmax) kmax = sg.K;
    sg.wpc = 1;
    while (sg.wpc < 8 && (sg.N * sg.wpc + 7) / 8 < 2 * sms && (sg.K >> 3) / (sg.wpc * 2) >= 96) sg.wpc *= 2;
    if (sg.wpc == 1) split = false;
    want += (sg.N + 7) / 8;
  }
  if (!split) {
    for (int i = 0; i < a->nseg; ++i) a->seg[i].wpc = 1;
  } else {
    want = 0;
    for (int i = 0; i < a->nseg; ++i) want += (a->seg[i].N * a->seg[i].wpc + 7) / 8;
  }
  // a block per eight output columns, thinned evenly when that is more than eight blocks per SM
  const int limit = 8 * sms;
  int grid = 0;
  for (int i = 0; i < a->nseg; ++i) {
    int nb = (a->seg[i].N * a->seg[i].wpc + 7) / 8;
    if (want > limit) { nb = (int)((long long)nb * limit / want); if (nb < 1) nb = 1; }
    a->seg[i].block0 = grid;
    grid += nb;
  }
  const int M = a->M;
  if (M == 1) return launch_skinny_multi<1>(*a, grid, kmax, split, st);
  if (M == 2) return launch_skinny_multi<2>(*a, grid, kmax, split, st);
  if (M <= 4) return launch_skinny_multi<4>(*a, grid, kmax, split, st);
  if (M <= 8) return launch_skinny_multi<8>(*a, grid, kmax, split, st);
  return launch_skinny_multi<16>(*a, grid, kmax, split, st);
}

extern "C" int loom_decode_step_flags(const long long* pos, const long long* tok, const void* pending, const void* have_carry,
                                      void* fire, void* reset, void* row_reset, void* seed_valid, int B, long long window,
                                      long long seq_len, int hard_enabled, long long carry_token, int temporal, cudaStream_t st) {
  if (B < 1) return -1;
  const int threads = 128, blocks = (B + threads - 1) / threads;
  decode_step_flags_kernel<<<blocks, threads, 0, st>>>(pos, tok, (const uint8_t*)pending, (const uint8_t*)have_carry,
                                                       (uint8_t*)fire, (uint8_t*)reset, (uint8_t*)row_reset, (uint8_t*)seed_valid,
                                                       B, window, seq_len, hard_enabled, carry_token, temporal);
  return (int)cudaGetLastError();
}

extern "C" int loom_decode_ca_append(const void* newk, const void* newv, long long ld_new, const void* fire, void* ca_k, void* ca_v,
                                     void* ca_valid, const long long* ca_len, void* allowed, long long* any_out, void* pending,
                                     void* have_carry, int B, int cap, int N, cudaStream_t st) {
  if (B < 1 || cap < 1 || N < 1) return -1;
  decode_ca_append_kernel<<<B, 256, 0, st>>>((const bf16*)newk, (const bf16*)newv, ld_new, (const uint8_t*)fire, (bf16*)ca_k,
                                            (bf16*)ca_v, (uint8_t*)ca_valid, ca_len, (uint8_t*)allowed, any_out,
                                            (uint8_t*)pending, (uint8_t*)have_carry, B, cap, N);
  return (int)cudaGetLastError();
}
