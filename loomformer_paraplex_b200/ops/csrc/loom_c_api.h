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
  LoomOperand a[5];
  int k_len[5], a_k0[5], b_k0[5];
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

// ---- flat optimizer (optim.cu) ----
int loom_grad_norm(const float* grads, long long n, float max_norm, float* partial, int nparts, float* stats,
                   float* atom_out, cudaStream_t stream);
int loom_adamw_flat(float* p, const float* g, float* m, float* v, void* shadow_bf16, const float* lr_mult,
                    const float* wd_blk, const float* active, const float* stats, const float* hyper,
                    long long nblk, cudaStream_t stream);
int loom_atom_flat(float* p, const float* g, float* m, float* v, void* shadow_bf16, const float* lr_mult,
                   const float* wd_blk, const float* cnt_blk, float* gprev, float* pnode, float* trust,
                   const float* stats, const float* hyper, float* atom_out, long long nblk, cudaStream_t stream);
int loom_cast_shadow(const float* p, void* shadow_bf16, long long n, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
