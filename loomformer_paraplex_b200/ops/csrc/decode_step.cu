// Small-batch pieces of the decode step.
//
// skinny_linear   y[M, N] = x[M, K] . W[N, K]^T (+ bias), M <= 16 rows.  One token per sequence makes every linear layer
//                 of the decode step a matrix-vector product: the weights are streamed once (16-byte loads, a warp per
//                 output column, fp32 accumulation, shuffle reduction) and the activations sit in shared memory.  A
//                 128-row tensor-core tile would spend its time on fixed set-up cost for one useful row.  The output may
//                 be a row-strided view, so the projection into a depth-history slot is written in place.
// rope_store      rotate-half RoPE of the new token's Q and K at the device-side position, rotated Q into the
//                 attention operand buffer, rotated K and V appended to the caches: one launch instead of a dozen
//                 slicing / multiply / index-copy launches, and graph-safe because the position is read on the device.
//
// The reference runs these through F.linear and PyTorch indexing, relaunched from the host for every token
// (reference loomformer.py:3951-4091).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
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
  skinny_linear_kernel<MT><<<grid, 256, shm, st>>>((const bf16*)x, ldx, (const bf16*)w, ldw, bias, y, ldy, out_fp32, M, N, K);
  return (int)cudaGetLastError();
}

// one block per sequence; thread j of a head handles dims j and j + HD/2
__global__ void __launch_bounds__(256) decode_rope_store_kernel(const bf16* __restrict__ qkv, long long ld_qkv,
                                                                const float* __restrict__ cos_tab,
                                                                const float* __restrict__ sin_tab,
                                                                const long long* __restrict__ pos_ptr, bf16* __restrict__ q_out,
                                                                long long ld_q, bf16* __restrict__ kc, bf16* __restrict__ vc,
                                                                int S, int table_rows, int QH, int KVH, int HD) {
  const int b = blockIdx.x;
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
  decode_rope_store_kernel<<<B, 256, 0, st>>>((const bf16*)qkv, ld_qkv, cos_tab, sin_tab, pos, (bf16*)q_out, ld_q, (bf16*)kc,
                                             (bf16*)vc, S, table_rows, QH, KVH, HD);
  return (int)cudaGetLastError();
}
