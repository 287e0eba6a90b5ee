// Gradient norm / clip coefficient / finite flag with built-in scratch: the non-allocating twin of
// loom_grad_norm (optim.cu).  See loom_static_scratch.h for the contract.  The arithmetic and the reduction
// order match loom_grad_norm for equal nparts, so both give the same bits.
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <mutex>
#include "loom_static_scratch.h"

namespace {

constexpr int BLK = 256;
constexpr int MAX_DEVICES = 64;

// the scratch itself: one array per device, part of the module image that the runtime loads on that device
static __device__ __align__(256) float g_partials[LOOM_STATIC_PARTS_MAX];

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float block_sum_256(float v, float* sh) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) sh[w] = v;
  __syncthreads();
  float r = (threadIdx.x < 8) ? sh[threadIdx.x] : 0.f;
  if (w == 0) r = warp_sum(r);
  if (threadIdx.x == 0) sh[8] = r;
  __syncthreads();
  return sh[8];
}

__global__ void static_sumsq_kernel(const float* __restrict__ g, long long n, float* __restrict__ partial) {
  __shared__ float sh[16];
  float acc = 0.f;
  const long long n4 = n >> 2;
  const float4* g4 = reinterpret_cast<const float4*>(g);
  for (long long i = (long long)blockIdx.x * BLK + threadIdx.x; i < n4; i += (long long)gridDim.x * BLK) {
    const float4 v = g4[i];
    acc += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  const float tot = block_sum_256(acc, sh);
  if (threadIdx.x == 0) partial[blockIdx.x] = tot;      // every entry that the next kernel reads is written here
}

__global__ void static_finalize_kernel(const float* __restrict__ partial, int nparts, float max_norm,
                                       float* __restrict__ stats, float* __restrict__ atom_out) {
  __shared__ float sh[16];
  float acc = 0.f;
  for (int i = threadIdx.x; i < nparts; i += BLK) acc += partial[i];
  const float tot = block_sum_256(acc, sh);
  if (threadIdx.x == 0) {
    const float norm = sqrtf(tot);
    const bool fin = isfinite(norm);
    stats[0] = norm;
    stats[1] = (max_norm > 0.f && fin) ? fminf(1.f, max_norm / (norm + 1e-6f)) : 1.f;
    stats[2] = fin ? 1.f : 0.f;
    if (atom_out) { atom_out[0] = 0.f; atom_out[1] = 0.f; atom_out[2] = 0.f; }
  }
}

// address of g_partials on each device, filled on the first call made with that device current
float* g_addr[MAX_DEVICES] = {nullptr};
std::mutex g_lock;

int scratch_for_current_device(float** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return LOOM_STATIC_E_SYMBOL;
  if (dev < 0 || dev >= MAX_DEVICES) return LOOM_STATIC_E_DEVICE;
  std::lock_guard<std::mutex> hold(g_lock);
  if (g_addr[dev] == nullptr) {
    float* p = nullptr;
    const cudaError_t rc = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_partials);
    if (rc != cudaSuccess || p == nullptr) {
      (void)cudaGetLastError();          // leave no sticky error behind for the caller's next launch check
      return LOOM_STATIC_E_SYMBOL;
    }
    g_addr[dev] = p;
  }
  *out = g_addr[dev];
  return LOOM_STATIC_OK;
}

}  // namespace

extern "C" int loom_grad_norm_static(const float* grads, long long n, float max_norm, int nparts, float* stats,
                                     float* atom_out, cudaStream_t stream) {
  if (grads == nullptr || stats == nullptr) return LOOM_STATIC_E_NULL;
  if (nparts < 1 || nparts > LOOM_STATIC_PARTS_MAX) return LOOM_STATIC_E_PARTS;
  if (n <= 0 || (n & 3) != 0 || (reinterpret_cast<uintptr_t>(grads) & 15u) != 0) return LOOM_STATIC_E_SHAPE;
  float* partial = nullptr;
  const int rc = scratch_for_current_device(&partial);
  if (rc != LOOM_STATIC_OK) return rc;
  static_sumsq_kernel<<<nparts, BLK, 0, stream>>>(grads, n, partial);
  static_finalize_kernel<<<1, BLK, 0, stream>>>(partial, nparts, max_norm, stats, atom_out);
  return (int)cudaGetLastError();
}

extern "C" const char* loom_static_strerror(int code) {
  switch (code) {
    case LOOM_STATIC_OK: return "ok";
    case LOOM_STATIC_E_PARTS: return "nparts must be between 1 and LOOM_STATIC_PARTS_MAX (1024): the built-in scratch holds no more";
    case LOOM_STATIC_E_SHAPE: return "n must be a positive multiple of 4 and grads must be 16-byte aligned";
    case LOOM_STATIC_E_NULL: return "grads and stats must not be null";
    case LOOM_STATIC_E_SYMBOL: return "could not obtain the address of the built-in scratch array on the current device";
    case LOOM_STATIC_E_DEVICE: return "device ordinal is beyond the 64 devices this entry point keeps addresses for";
    default: return code > 0 ? "CUDA runtime error (the code is a cudaError_t)" : "unknown code";
  }
}
