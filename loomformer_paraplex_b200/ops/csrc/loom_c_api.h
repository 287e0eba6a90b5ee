// Plain C interface of the sm_100a kernels: raw device pointers, sizes and a stream.  The PyTorch
// binding (bindings.cpp) is one consumer; nothing in this header depends on PyTorch.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// A bf16 matrix operand viewed as [rows, heads, cols]; element (r, g, c) lives at
// ptr + r*ld_row + g*ld_head + c (element units).  heads <= 1 means a plain 2-D matrix.
typedef struct {
  const void* ptr;
  long long rows, cols, heads;
  long long ld_row, ld_head;
} LoomOperand;

// C[m, g, n] (+)= sum_s A_s[m, g, :k_len[s]] . B[n, g, b_k0[s] : b_k0[s]+k_len[s]]  (+ bias)
// K-major operand: reduction index = cols.  MN-major operand: reduction index = rows.
typedef struct {
  LoomOperand a[4];
  int k_len[4], a_k0[4], b_k0[4];
  int nseg;
  LoomOperand b;
  int a_mn_major, b_mn_major;
  void* c;
  long long ldc, ldc_head;
  const float* bias;
  int M, N, heads;       // N = output columns per group
  int accumulate, out_fp32;
  int bn;                // tile width: 64, 128 or 256
  int swap_mn_strides;   // debugging aid: exchange the two descriptor strides of MN-major operands
  int* status;           // device word; non-zero after a bounded wait gave up
} LoomGemm;

int loom_gemm_bf16(const LoomGemm* g, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
