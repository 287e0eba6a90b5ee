// Fused Paraplex core + Tria depth step (forward and backward).
//
// One pass per (token, neuron) does everything between the up-projection GEMMs and the down GEMM:
//   R = X (1 + a p_in) + b_r ;  beta = beta_lin + b_i ;  s0 = sin(pi/2 beta / sqrt(1+beta^2))
//   z = s0 + w_t * s0[previous token] ;  I = z / sqrt(1+z^2) ;  A = softplus(gate)
//   O = (R + A I) * A^(m/(sqrt(A)+1)) * sigmoid(A)
//   T = (I3 + alpha K(tanh(x/rms x))) R_axis, x = (R I, R O, I O) ;  C = N(T C_prev)  (or N(T seed) / N(T))
//   p_out = <w9, vec(C)>
// The reference spreads this over an element-wise Paraplex kernel, a reduction kernel, an anchor
// kernel pair and one Tria kernel per variant (reference kernels/paraplex/paraplex_kernel.cuh:111-298,
// kernels/tria/tria_step_gate/tria_step_gate_kernel.cuh, tria_init_seed_kernel.cuh), re-reading R, I, O
// from global memory in between; here they stay in registers.
//
// Carriers are stored plane-major: c[k][m][h], k = 0..8 (row-major 3x3 index), bf16, so that every
// thread's loads are 4-byte bf16x2 accesses that coalesce to full 128-byte lines across a warp.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include "launch_util.cuh"
#include "loom_c_api.h"

namespace {

constexpr float HALF_PI = 1.5707963267948966f;
typedef __nv_bfloat162 bf2;

__device__ __forceinline__ float2 ld2(const __nv_bfloat16* p) { return __bfloat1622float2(*reinterpret_cast<const bf2*>(p)); }
__device__ __forceinline__ void st2(__nv_bfloat16* p, float a, float b) { *reinterpret_cast<bf2*>(p) = __floats2bfloat162_rn(a, b); }

// one MUFU instruction (relative error about 2^-11, below the bf16 resolution of everything stored from it)
__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// pull a line into L1 ahead of its use; needs no destination register, so it costs the register-bound backward nothing
__device__ __forceinline__ void prefetch_l1(const void* p) { asm volatile("prefetch.global.L1 [%0];" ::"l"(p)); }
__device__ __forceinline__ void cp_async4(uint32_t* smem_dst, const void* gsrc) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait1() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }
__device__ __forceinline__ float2 ld2s(const uint32_t* p) { return __bfloat1622float2(*reinterpret_cast<const bf2*>(p)); }
__device__ __forceinline__ float phase_s0(float beta) { return sinf(HALF_PI * beta * rsqrtf(1.f + beta * beta)); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }

__device__ __forceinline__ float phase_slope(float beta, int secant, float anchor, float s_anchor, float floor_) {
  const float inv = rsqrtf(1.f + beta * beta);
  const float x = HALF_PI * beta * inv;
  const float dx = HALF_PI * inv * inv * inv;
  if (secant) {
    const float gap = beta - anchor;
    if (fabsf(gap) < 1e-4f) return cosf(x) * dx;
    return (sinf(x) - s_anchor) / gap;
  }
  return fmaxf(cosf(x), floor_) * dx;
}

// T = (I + alpha K(a,b,c)) R_axis laid out row-major
template <int AXIS>
__device__ __forceinline__ void build_T(float a, float b, float c, float (&T)[9]) {
  constexpr int axis = AXIS;
  if (axis == 0) { T[0] = -c; T[1] = -1.f; T[2] = b; T[3] = 1.f; T[4] = -c; T[5] = -a; T[6] = a; T[7] = b; T[8] = 1.f; }
  else if (axis == 1) { T[0] = 1.f; T[1] = b; T[2] = c; T[3] = c; T[4] = -a; T[5] = -1.f; T[6] = -b; T[7] = 1.f; T[8] = -a; }
  else { T[0] = -b; T[1] = -c; T[2] = 1.f; T[3] = a; T[4] = 1.f; T[5] = c; T[6] = -1.f; T[7] = a; T[8] = -b; }
}
template <int AXIS>
__device__ __forceinline__ void grad_abc(const float (&g)[9], float& ga, float& gb, float& gc) {
  constexpr int axis = AXIS;
  if (axis == 0) { ga = -g[5] + g[6]; gb = g[2] + g[7]; gc = -g[0] - g[4]; }
  else if (axis == 1) { ga = -g[4] - g[8]; gb = g[1] - g[6]; gc = g[2] + g[3]; }
  else { ga = g[3] + g[7]; gb = -g[0] - g[8]; gc = -g[1] + g[5]; }
}

struct CoreScalars {
  float alpha_gate;   // a = 0.25 tanh(raw) (0 when there is no incoming gate value)
  float powlu_m;
  float tria_alpha;
  float floor_;
  int axis;           // -1: no Tria
  int secant;
  int Tc, H, M, B;
  const float* alpha_ptr;    // device scalars, so no launch argument depends on a host read-back
  const float* anchor_ptr;
};

// ----------------------------------------------------------------------------------------------
// forward: one thread per (m, h-pair)
// ----------------------------------------------------------------------------------------------
struct FwdElem {
  float r, gs, i, o, s0;
  float C[9];
  float p;
};

template <int AXIS>
__device__ __forceinline__ void core_forward_elem(const CoreScalars& S, float x, float pin, int has_pin, float b_r,
                                                  float glin, int has_glin, float beta, float prev, float w_t,
                                                  const float (&R)[9], bool has_R, const float (&w9)[9], bool has_w,
                                                  FwdElem& E) {
  E.r = has_pin ? x * (1.f + S.alpha_gate * pin) + b_r : x + b_r;
  E.gs = has_glin ? glin : E.r;
  E.s0 = phase_s0(beta);
  const float z = E.s0 + w_t * prev;
  E.i = z * rsqrtf(1.f + z * z);
  const float A = fmaxf(softplus_f(E.gs), 1e-12f);
  const float P = E.r + A * E.i;
  const float G = __powf(A, S.powlu_m / (sqrtf(A) + 1.f)) * sigmoid_f(A);
  E.o = P * G;
  if (AXIS >= 0) {
    const float x0 = E.r * E.i, x1 = E.r * E.o, x2 = E.i * E.o;
    const float n3 = rsqrtf((x0 * x0 + x1 * x1 + x2 * x2) * (1.f / 3.f) + 1e-6f);
    const float a = S.tria_alpha * tanh_fast(x0 * n3), b = S.tria_alpha * tanh_fast(x1 * n3), c = S.tria_alpha * tanh_fast(x2 * n3);
    float T[9], pre[9];
    build_T<AXIS>(a, b, c, T);
    if (has_R) {
#pragma unroll
      for (int rr = 0; rr < 3; ++rr)
#pragma unroll
        for (int cc = 0; cc < 3; ++cc)
          pre[rr * 3 + cc] = T[rr * 3] * R[cc] + T[rr * 3 + 1] * R[3 + cc] + T[rr * 3 + 2] * R[6 + cc];
    } else {
#pragma unroll
      for (int k = 0; k < 9; ++k) pre[k] = T[k];
    }
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < 9; ++k) ss += pre[k] * pre[k];
    const float inv = rsqrtf(ss * (1.f / 9.f) + 1e-6f);
    float p = 0.f;
#pragma unroll
    for (int k = 0; k < 9; ++k) { E.C[k] = pre[k] * inv; if (has_w) p += w9[k] * E.C[k]; }
    E.p = p;
  }
}

// one (token, neuron pair): loads, both elements' forward, stores; returns the pair's sum of beta^2
// STAGED: the row's bf16 pairs were copied into this thread's shared-memory slots (stride 256 words) beforehand:
// slot 0 x, 1 p_in, 2 gate, 3 beta, 4 beta of the row above, 5..13 carrier planes
template <int AXIS, bool STAGED>
__device__ __forceinline__ float core_forward_pair(
    const CoreScalars& S, int m, int h, const uint32_t* __restrict__ slots, const __nv_bfloat16* __restrict__ x_real, const __nv_bfloat16* __restrict__ p_in,
    const float* __restrict__ b_real, const __nv_bfloat16* __restrict__ gate_lin,
    const __nv_bfloat16* __restrict__ beta_lin, const float* __restrict__ b_imag, const float* __restrict__ w_trace,
    const float* __restrict__ trace_in, const uint8_t* __restrict__ reset, const __nv_bfloat16* __restrict__ c_prev,
    const float* __restrict__ seed, const uint8_t* __restrict__ seed_valid, const float* __restrict__ gate_w,
    __nv_bfloat16* __restrict__ o_out, __nv_bfloat16* __restrict__ c_out, __nv_bfloat16* __restrict__ p_out,
    float* __restrict__ trace_out) {
  const int H = S.H;
  const int b = m / S.Tc, t = m % S.Tc;
  const long long e = (long long)m * H + h;
#define LOOM_LDF(SLOT, GPTR) (STAGED ? ld2s(slots + (SLOT) * 256) : ld2(GPTR))
  const float2 x = LOOM_LDF(0, x_real + e);
  float2 pin = make_float2(0.f, 0.f), gl = make_float2(0.f, 0.f);
  if (p_in) pin = LOOM_LDF(1, p_in + e);
  if (gate_lin) gl = LOOM_LDF(2, gate_lin + e);
  const float2 bl = LOOM_LDF(3, beta_lin + e);
  const float bi0 = b_imag[h], bi1 = b_imag[h + 1];
  const float beta0 = bl.x + bi0, beta1 = bl.y + bi1;
  float prev0 = 0.f, prev1 = 0.f;
  const bool rs = reset && reset[m];
  if (!rs) {
    if (t == 0) { if (trace_in) { prev0 = trace_in[(long long)b * H + h]; prev1 = trace_in[(long long)b * H + h + 1]; } }
    else { const float2 bp = LOOM_LDF(4, beta_lin + e - H); prev0 = phase_s0(bp.x + bi0); prev1 = phase_s0(bp.y + bi1); }
  }
  float w9[9];
  const bool has_w = gate_w != nullptr;
#pragma unroll
  for (int k = 0; k < 9; ++k) w9[k] = has_w ? gate_w[k] : 0.f;
  float cp0[9], cp1[9];          // carrier entering the step (previous depth, or the temporal seed at t = 0)
  bool has_R = false;
  const long long plane = (long long)S.M * H;
  if (AXIS >= 0) {
    if (c_prev) {
#pragma unroll
      for (int k = 0; k < 9; ++k) { float2 v = LOOM_LDF(5 + k, c_prev + k * plane + e); cp0[k] = v.x; cp1[k] = v.y; }
      has_R = true;
    } else if (seed && t == 0 && seed_valid[b]) {
      const float* sp = seed + ((long long)b * H + h) * 9;
#pragma unroll
      for (int k = 0; k < 9; ++k) { cp0[k] = sp[k]; cp1[k] = sp[9 + k]; }
      has_R = true;
    }
  }
#undef LOOM_LDF
  if (!has_R) {
#pragma unroll
    for (int k = 0; k < 9; ++k) { cp0[k] = 0.f; cp1[k] = 0.f; }
  }
  FwdElem E0, E1;
  core_forward_elem<AXIS>(S, x.x, pin.x, p_in != nullptr, b_real[h], gl.x, gate_lin != nullptr, beta0, prev0, w_trace[h],
                          cp0, has_R, w9, has_w, E0);
  core_forward_elem<AXIS>(S, x.y, pin.y, p_in != nullptr, b_real[h + 1], gl.y, gate_lin != nullptr, beta1, prev1,
                          w_trace[h + 1], cp1, has_R, w9, has_w, E1);
  st2(o_out + e, E0.o, E1.o);
  if (t == S.Tc - 1) { trace_out[(long long)b * H + h] = E0.s0; trace_out[(long long)b * H + h + 1] = E1.s0; }
  if (AXIS >= 0) {
#pragma unroll
    for (int k = 0; k < 9; ++k) st2(c_out + k * plane + e, E0.C[k], E1.C[k]);
    if (has_w) st2(p_out + e, E0.p, E1.p);
  }
  return beta0 * beta0 + beta1 * beta1;
}

__device__ __forceinline__ void block_add_256(float v, float* __restrict__ dst) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __shared__ float sh[8];
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x == 0) {
    float tot = 0.f;
    for (int i = 0; i < 8; ++i) tot += sh[i];
    atomicAdd(dst, tot);
  }
}

// one thread per (m, h-pair)
template <int AXIS>
__global__ void __launch_bounds__(256) ffn_core_fwd_kernel(
    CoreScalars S_in, const __nv_bfloat16* __restrict__ x_real, const __nv_bfloat16* __restrict__ p_in,
    const float* __restrict__ b_real, const __nv_bfloat16* __restrict__ gate_lin,
    const __nv_bfloat16* __restrict__ beta_lin, const float* __restrict__ b_imag, const float* __restrict__ w_trace,
    const float* __restrict__ trace_in, const uint8_t* __restrict__ reset, const __nv_bfloat16* __restrict__ c_prev,
    const float* __restrict__ seed, const uint8_t* __restrict__ seed_valid, const float* __restrict__ gate_w,
    __nv_bfloat16* __restrict__ o_out, __nv_bfloat16* __restrict__ c_out, __nv_bfloat16* __restrict__ p_out,
    float* __restrict__ trace_out, float* __restrict__ beta_sq_sum) {
  loom::pdl_wait();                           // returns at once unless launched programmatically dependent (decode-sized problems)
  if (S_in.M <= 256) loom::pdl_trigger();     // decode-sized problem: a dependent launched programmatically may start its prologue now
  CoreScalars S = S_in;
  S.alpha_gate = S.alpha_ptr ? *S.alpha_ptr : 0.f;
  const int Hp = S.H >> 1;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  float bsq = 0.f;
  if (idx < (long long)S.M * Hp)
    bsq = core_forward_pair<AXIS, false>(S, (int)(idx / Hp), (int)(idx % Hp) * 2, nullptr, x_real, p_in, b_real, gate_lin, beta_lin, b_imag,
                                  w_trace, trace_in, reset, c_prev, seed, seed_valid, gate_w, o_out, c_out, p_out, trace_out);
  block_add_256(bsq, beta_sq_sum);
}

// Tiled variant: a block owns 64 neuron pairs x FWD_ROWS tokens; every thread walks FWD_ROWS / 4 rows and copies its
// next row into its own shared-memory slots with cp.async while it works on the current one (see pass A of the
// backward for the reasoning).
constexpr int FWD_ROWS = 16;
constexpr int FWD_SLOTS = 14;
template <int AXIS>
__global__ void __launch_bounds__(256) ffn_core_fwd_tiled_kernel(
    CoreScalars S_in, const __nv_bfloat16* __restrict__ x_real, const __nv_bfloat16* __restrict__ p_in,
    const float* __restrict__ b_real, const __nv_bfloat16* __restrict__ gate_lin,
    const __nv_bfloat16* __restrict__ beta_lin, const float* __restrict__ b_imag, const float* __restrict__ w_trace,
    const float* __restrict__ trace_in, const uint8_t* __restrict__ reset, const __nv_bfloat16* __restrict__ c_prev,
    const float* __restrict__ seed, const uint8_t* __restrict__ seed_valid, const float* __restrict__ gate_w,
    __nv_bfloat16* __restrict__ o_out, __nv_bfloat16* __restrict__ c_out, __nv_bfloat16* __restrict__ p_out,
    float* __restrict__ trace_out, float* __restrict__ beta_sq_sum) {
  loom::pdl_wait();                           // returns at once unless launched programmatically dependent (decode-sized problems)
  if (S_in.M <= 256) loom::pdl_trigger();     // decode-sized problem: a dependent launched programmatically may start its prologue now
  CoreScalars S = S_in;
  S.alpha_gate = S.alpha_ptr ? *S.alpha_ptr : 0.f;
  const int H = S.H;
  const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;
  const int h = (blockIdx.x * 64 + tx) * 2;
  const long long plane = (long long)S.M * H;
  extern __shared__ uint32_t stg[];                     // [2 stages][FWD_SLOTS][256 threads]
  auto issue = [&](int mn, int st) {
    uint32_t* sl = stg + st * FWD_SLOTS * 256 + threadIdx.x;
    const long long en = (long long)mn * H + h;
    cp_async4(sl, x_real + en);
    if (p_in) cp_async4(sl + 256, p_in + en);
    if (gate_lin) cp_async4(sl + 2 * 256, gate_lin + en);
    cp_async4(sl + 3 * 256, beta_lin + en);
    if (mn % S.Tc != 0) cp_async4(sl + 4 * 256, beta_lin + en - H);
    if (AXIS >= 0 && c_prev) {
#pragma unroll
      for (int k = 0; k < 9; ++k) cp_async4(sl + (5 + k) * 256, c_prev + k * plane + en);
    }
  };
  float bsq = 0.f;
  if (h < H) {
    const int m_first = blockIdx.y * FWD_ROWS + ty;
    if (m_first < S.M) issue(m_first, 0);
    cp_async_commit();
    for (int j = 0; j < FWD_ROWS / 4; ++j) {
      const int m = blockIdx.y * FWD_ROWS + ty + 4 * j;
      if (m >= S.M) break;
      const int st = j & 1;
      if (m + 4 < S.M && j + 1 < FWD_ROWS / 4) issue(m + 4, st ^ 1);
      cp_async_commit();
      cp_async_wait1();
      bsq += core_forward_pair<AXIS, true>(S, m, h, stg + st * FWD_SLOTS * 256 + threadIdx.x, x_real, p_in, b_real, gate_lin,
                                           beta_lin, b_imag, w_trace, trace_in, reset, c_prev, seed, seed_valid, gate_w, o_out,
                                           c_out, p_out, trace_out);
    }
  }
  block_add_256(bsq, beta_sq_sum);
}


// ----------------------------------------------------------------------------------------------
// backward, pass A: everything except the phase slope (which needs the next token's g_z)
// ----------------------------------------------------------------------------------------------
struct BwdElem {
  float dx, dpin, dgl, gz, gr, dwt, dalpha;
  float dR[9];
  float dw9[9];
};

template <int AXIS>
__device__ __forceinline__ void core_backward_elem(const CoreScalars& S, float x, float pin, int has_pin, float b_r,
                                                   float glin, int has_glin, float beta, float prev, float w_t,
                                                   const float (&R)[9], bool has_R, const float (&w9)[9], float dO,
                                                   const float (&dC)[9], bool has_dc, float dpo, bool has_dpo,
                                                   BwdElem& E) {
  const float r = has_pin ? x * (1.f + S.alpha_gate * pin) + b_r : x + b_r;
  const float gs = has_glin ? glin : r;
  const float s0 = phase_s0(beta);
  const float z = s0 + w_t * prev;
  const float zi = rsqrtf(1.f + z * z);
  const float i = z * zi;
  // softplus and the sigmoid needed for its derivative share one exponential
  const float egs = __expf(fminf(gs, 30.f));
  const float sp = gs > 20.f ? gs : (gs < -15.f ? egs : __logf(1.f + egs));
  const float sig_gs = gs > 20.f ? 1.f : egs / (1.f + egs);
  const float A = fmaxf(sp, 1e-12f);
  const float sqA = sqrtf(A);
  const float ex = S.powlu_m / (sqA + 1.f);
  const float sig = sigmoid_f(A);
  const float lg2A = __log2f(A);                 // shared by A^ex and d/dA A^ex
  const float G = exp2f(ex * lg2A) * sig;
  const float P = r + A * i;
  const float o = P * G;
  float g_r = 0.f, g_i = 0.f, g_o = dO;
#pragma unroll
  for (int k = 0; k < 9; ++k) { E.dR[k] = 0.f; E.dw9[k] = 0.f; }
  if (AXIS >= 0 && (has_dc || has_dpo)) {
    const float x0 = r * i, x1 = r * o, x2 = i * o;
    const float n3 = rsqrtf((x0 * x0 + x1 * x1 + x2 * x2) * (1.f / 3.f) + 1e-6f);
    const float y0 = x0 * n3, y1 = x1 * n3, y2 = x2 * n3;
    const float t0 = tanh_fast(y0), t1 = tanh_fast(y1), t2 = tanh_fast(y2);
    float T[9], pre[9], C[9], gC[9], gpre[9], gT[9];
    build_T<AXIS>(S.tria_alpha * t0, S.tria_alpha * t1, S.tria_alpha * t2, T);
    if (has_R) {
#pragma unroll
      for (int rr = 0; rr < 3; ++rr)
#pragma unroll
        for (int cc = 0; cc < 3; ++cc)
          pre[rr * 3 + cc] = T[rr * 3] * R[cc] + T[rr * 3 + 1] * R[3 + cc] + T[rr * 3 + 2] * R[6 + cc];
    } else {
#pragma unroll
      for (int k = 0; k < 9; ++k) pre[k] = T[k];
    }
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < 9; ++k) ss += pre[k] * pre[k];
    const float inv = rsqrtf(ss * (1.f / 9.f) + 1e-6f);
    float dot = 0.f;
#pragma unroll
    for (int k = 0; k < 9; ++k) {
      C[k] = pre[k] * inv;
      gC[k] = (has_dc ? dC[k] : 0.f) + (has_dpo ? dpo * w9[k] : 0.f);
      if (has_dpo) E.dw9[k] = dpo * C[k];
      dot += gC[k] * C[k];
    }
    dot *= (1.f / 9.f);
#pragma unroll
    for (int k = 0; k < 9; ++k) gpre[k] = (gC[k] - C[k] * dot) * inv;
    if (has_R) {
#pragma unroll
      for (int rr = 0; rr < 3; ++rr)
#pragma unroll
        for (int cc = 0; cc < 3; ++cc) {
          gT[rr * 3 + cc] = gpre[rr * 3] * R[cc * 3] + gpre[rr * 3 + 1] * R[cc * 3 + 1] + gpre[rr * 3 + 2] * R[cc * 3 + 2];
          E.dR[rr * 3 + cc] = T[rr] * gpre[cc] + T[3 + rr] * gpre[3 + cc] + T[6 + rr] * gpre[6 + cc];
        }
    } else {
#pragma unroll
      for (int k = 0; k < 9; ++k) gT[k] = gpre[k];
    }
    float ga, gb, gc;
    grad_abc<AXIS>(gT, ga, gb, gc);
    const float gy0 = ga * S.tria_alpha * (1.f - t0 * t0), gy1 = gb * S.tria_alpha * (1.f - t1 * t1),
                gy2 = gc * S.tria_alpha * (1.f - t2 * t2);
    const float doty = (gy0 * y0 + gy1 * y1 + gy2 * y2) * (1.f / 3.f);
    const float gx0 = (gy0 - y0 * doty) * n3, gx1 = (gy1 - y1 * doty) * n3, gx2 = (gy2 - y2 * doty) * n3;
    g_r += gx0 * i + gx1 * o;
    g_i += gx0 * r + gx2 * o;
    g_o += gx1 * r + gx2 * i;
  }
  const float gP = g_o * G, gG = g_o * P;
  g_r += gP;
  g_i += gP * A;
  float gA = gP * i;
  if (sp >= 1e-12f) {
    const float de = -S.powlu_m / ((sqA + 1.f) * (sqA + 1.f)) * (0.5f / sqA);
    gA += gG * G * (ex / A + de * (lg2A * 0.6931471805599453f) + (1.f - sig));
  } else {
    gA = 0.f;
  }
  const float g_gs = gA * sig_gs;
  E.gz = g_i * zi * zi * zi;
  E.dwt = E.gz * prev;
  if (has_glin) E.dgl = g_gs; else { g_r += g_gs; E.dgl = 0.f; }
  E.gr = g_r;
  E.dx = has_pin ? g_r * (1.f + S.alpha_gate * pin) : g_r;
  E.dpin = has_pin ? g_r * x * S.alpha_gate : 0.f;
  E.dalpha = has_pin ? g_r * x * pin : 0.f;
}

constexpr int TILE_ROWS = 32;

template <int AXIS, int PF>
__global__ void __launch_bounds__(256, 2) ffn_core_bwd_a_kernel(
    CoreScalars S_in, const __nv_bfloat16* __restrict__ x_real, const __nv_bfloat16* __restrict__ p_in,
    const float* __restrict__ b_real, const __nv_bfloat16* __restrict__ gate_lin,
    const __nv_bfloat16* __restrict__ beta_lin, const float* __restrict__ b_imag, const float* __restrict__ w_trace,
    const float* __restrict__ trace_in, const uint8_t* __restrict__ reset, const __nv_bfloat16* __restrict__ c_prev,
    const float* __restrict__ seed, const uint8_t* __restrict__ seed_valid, const float* __restrict__ gate_w,
    const __nv_bfloat16* __restrict__ d_o, const __nv_bfloat16* __restrict__ d_c, const __nv_bfloat16* __restrict__ d_pout,
    __nv_bfloat16* __restrict__ dx_real, __nv_bfloat16* __restrict__ dp_in, __nv_bfloat16* __restrict__ dgate_lin,
    float* __restrict__ gz, __nv_bfloat16* __restrict__ dc_prev, float* __restrict__ dseed, float* __restrict__ dtrace_in,
    float* __restrict__ g_b_real, float* __restrict__ g_w_trace, float* __restrict__ g_scalars /* [0]=alpha, [1..9]=w9 */) {
  constexpr int prefetch = PF;
  CoreScalars S = S_in;
  S.alpha_gate = S.alpha_ptr ? *S.alpha_ptr : 0.f;
  const int H = S.H;
  const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;
  const int h = (blockIdx.x * 64 + tx) * 2;
  const bool col_ok = h < H;
  const long long plane = (long long)S.M * H;
  float w9[9];
  const bool has_w = gate_w != nullptr && d_pout != nullptr;
#pragma unroll
  for (int k = 0; k < 9; ++k) w9[k] = has_w ? gate_w[k] : 0.f;
  float acc_br0 = 0.f, acc_br1 = 0.f, acc_wt0 = 0.f, acc_wt1 = 0.f, acc_alpha = 0.f;
  float acc_w9[9];
#pragma unroll
  for (int k = 0; k < 9; ++k) acc_w9[k] = 0.f;
  // prefetch == 2: every thread copies the (up to 25) bf16 pairs of its NEXT row into its own shared-memory slots with
  // cp.async while it works on the current row, and reads the current row from the slots filled one iteration
  // earlier.  The slots are private to the thread, so cp.async.wait_group is the only synchronisation.  With 16
  // resident warps per SM the loads would otherwise be exposed, and holding a prefetched row in registers is not an
  // option (the 3x3 chain already spills).  prefetch == 1 asks L1 for the lines instead; 0 loads on demand.
  extern __shared__ uint32_t stg[];                     // [2 stages][NSLOT][256 threads]
  constexpr int NSLOT = 25;                             // x, p_in, gate, d_pout, beta, d_o, beta of the row above, 9 + 9 carrier planes
  constexpr bool staged = prefetch == 2;
  auto slot = [&](int st, int k) -> uint32_t* { return stg + (st * NSLOT + k) * 256 + threadIdx.x; };
  auto issue = [&](int mn, int st) {
    const long long en = (long long)mn * H + h;
    cp_async4(slot(st, 0), x_real + en);
    if (p_in) cp_async4(slot(st, 1), p_in + en);
    if (gate_lin) cp_async4(slot(st, 2), gate_lin + en);
    if (has_w) cp_async4(slot(st, 3), d_pout + en);
    cp_async4(slot(st, 4), beta_lin + en);
    cp_async4(slot(st, 5), d_o + en);
    if (mn % S.Tc != 0) cp_async4(slot(st, 6), beta_lin + en - H);
    if (AXIS >= 0) {
#pragma unroll
      for (int k = 0; k < 9; ++k) {
        if (c_prev) cp_async4(slot(st, 7 + k), c_prev + k * plane + en);
        if (d_c) cp_async4(slot(st, 16 + k), d_c + k * plane + en);
      }
    }
  };
  if (col_ok) {
    const float br0 = b_real[h], br1 = b_real[h + 1], bi0 = b_imag[h], bi1 = b_imag[h + 1];
    const float wt0 = w_trace[h], wt1 = w_trace[h + 1];
    if (staged) {
      const int m_first = blockIdx.y * TILE_ROWS + ty;
      if (m_first < S.M) issue(m_first, 0);
      cp_async_commit();
    }
    for (int j = 0; j < TILE_ROWS / 4; ++j) {
      const int m = blockIdx.y * TILE_ROWS + ty + 4 * j;
      if (m >= S.M) break;
      const int b = m / S.Tc, t = m % S.Tc;
      const long long e = (long long)m * H + h;
      const int st = j & 1;
      const bool more = m + 4 < S.M && j + 1 < TILE_ROWS / 4;
      if (staged) {
        if (more) issue(m + 4, st ^ 1);
        cp_async_commit();                              // possibly empty: keeps "all but the newest group" = this row
        cp_async_wait1();
      } else if (prefetch == 1 && more) {
        const long long en = e + 4ll * H;
        prefetch_l1(x_real + en); prefetch_l1(beta_lin + en); prefetch_l1(d_o + en);
        if (p_in) prefetch_l1(p_in + en);
        if (gate_lin) prefetch_l1(gate_lin + en);
        if (has_w) prefetch_l1(d_pout + en);
        if (AXIS >= 0) {
#pragma unroll
          for (int k = 0; k < 9; ++k) {
            if (c_prev) prefetch_l1(c_prev + k * plane + en);
            if (d_c) prefetch_l1(d_c + k * plane + en);
          }
        }
      }
#define LOOM_LD(SLOT, GPTR) (staged ? ld2s(slot(st, SLOT)) : ld2(GPTR))
      const float2 x = LOOM_LD(0, x_real + e);
      float2 pin = make_float2(0.f, 0.f), gl = make_float2(0.f, 0.f), dpo = make_float2(0.f, 0.f);
      if (p_in) pin = LOOM_LD(1, p_in + e);
      if (gate_lin) gl = LOOM_LD(2, gate_lin + e);
      if (has_w) dpo = LOOM_LD(3, d_pout + e);
      const float2 bl = LOOM_LD(4, beta_lin + e);
      const float2 dO = LOOM_LD(5, d_o + e);
      float prev0 = 0.f, prev1 = 0.f;
      const bool rs = reset && reset[m];
      if (!rs) {
        if (t == 0) { if (trace_in) { prev0 = trace_in[(long long)b * H + h]; prev1 = trace_in[(long long)b * H + h + 1]; } }
        else { const float2 bp = LOOM_LD(6, beta_lin + e - H); prev0 = phase_s0(bp.x + bi0); prev1 = phase_s0(bp.y + bi1); }
      }
      float R0[9], R1[9], dC0[9], dC1[9];
      bool has_R = false, from_seed = false;
      if (AXIS >= 0) {
        if (c_prev) {
#pragma unroll
          for (int k = 0; k < 9; ++k) { float2 v = LOOM_LD(7 + k, c_prev + k * plane + e); R0[k] = v.x; R1[k] = v.y; }
          has_R = true;
        } else if (seed && t == 0 && seed_valid[b]) {
          const float* sp = seed + ((long long)b * H + h) * 9;
#pragma unroll
          for (int k = 0; k < 9; ++k) { R0[k] = sp[k]; R1[k] = sp[9 + k]; }
          has_R = true; from_seed = true;
        }
        if (d_c) {
#pragma unroll
          for (int k = 0; k < 9; ++k) { float2 v = LOOM_LD(16 + k, d_c + k * plane + e); dC0[k] = v.x; dC1[k] = v.y; }
        }
      }
#undef LOOM_LD
      if (!has_R) {
#pragma unroll
        for (int k = 0; k < 9; ++k) { R0[k] = 0.f; R1[k] = 0.f; }
      }
      if (AXIS < 0 || !d_c) {
#pragma unroll
        for (int k = 0; k < 9; ++k) { dC0[k] = 0.f; dC1[k] = 0.f; }
      }
      BwdElem E0, E1;
      core_backward_elem<AXIS>(S, x.x, pin.x, p_in != nullptr, br0, gl.x, gate_lin != nullptr, bl.x + bi0, prev0, wt0, R0,
                               has_R, w9, dO.x, dC0, d_c != nullptr, dpo.x, has_w, E0);
      core_backward_elem<AXIS>(S, x.y, pin.y, p_in != nullptr, br1, gl.y, gate_lin != nullptr, bl.y + bi1, prev1, wt1, R1,
                               has_R, w9, dO.y, dC1, d_c != nullptr, dpo.y, has_w, E1);
      st2(dx_real + e, E0.dx, E1.dx);
      if (dp_in) st2(dp_in + e, E0.dpin, E1.dpin);
      if (dgate_lin) st2(dgate_lin + e, E0.dgl, E1.dgl);
      *reinterpret_cast<float2*>(gz + e) = make_float2(E0.gz, E1.gz);
      if (c_prev && dc_prev) {
#pragma unroll
        for (int k = 0; k < 9; ++k) st2(dc_prev + k * plane + e, E0.dR[k], E1.dR[k]);
      } else if (from_seed && dseed) {
        float* sp = dseed + ((long long)b * H + h) * 9;
#pragma unroll
        for (int k = 0; k < 9; ++k) { sp[k] = E0.dR[k]; sp[9 + k] = E1.dR[k]; }
      }
      if (t == 0 && dtrace_in) {
        dtrace_in[(long long)b * H + h] = rs ? 0.f : E0.gz * wt0;
        dtrace_in[(long long)b * H + h + 1] = rs ? 0.f : E1.gz * wt1;
      }
      acc_br0 += E0.gr; acc_br1 += E1.gr; acc_wt0 += E0.dwt; acc_wt1 += E1.dwt;
      acc_alpha += E0.dalpha + E1.dalpha;
#pragma unroll
      for (int k = 0; k < 9; ++k) acc_w9[k] += E0.dw9[k] + E1.dw9[k];
    }
  }
  // column sums: reduce the four row-groups of the block, then one atomic per column
  __shared__ float sh[4][4][64];
  sh[0][ty][tx] = acc_br0; sh[1][ty][tx] = acc_br1; sh[2][ty][tx] = acc_wt0; sh[3][ty][tx] = acc_wt1;
  __syncthreads();
  if (ty == 0 && col_ok) {
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
    for (int r = 0; r < 4; ++r) { a0 += sh[0][r][tx]; a1 += sh[1][r][tx]; a2 += sh[2][r][tx]; a3 += sh[3][r][tx]; }
    atomicAdd(g_b_real + h, a0); atomicAdd(g_b_real + h + 1, a1);
    atomicAdd(g_w_trace + h, a2); atomicAdd(g_w_trace + h + 1, a3);
  }
  // scalar sums
  float sc[10];
  sc[0] = acc_alpha;
#pragma unroll
  for (int k = 0; k < 9; ++k) sc[1 + k] = acc_w9[k];
  __shared__ float shs[8][10];
#pragma unroll
  for (int k = 0; k < 10; ++k) {
    float v = sc[k];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31) == 0) shs[threadIdx.x >> 5][k] = v;
  }
  __syncthreads();
  if (threadIdx.x < 10) {
    float v = 0.f;
    for (int w = 0; w < 8; ++w) v += shs[w][threadIdx.x];
    if (v != 0.f) atomicAdd(g_scalars + threadIdx.x, v);
  }
}

// backward, pass B: dbeta = (g_z[m] + w_t g_z[m+1] (same row, no reset) + dtrace_out at the last token) * slope
__global__ void __launch_bounds__(256) ffn_core_bwd_b_kernel(
    CoreScalars S, const float* __restrict__ gz, const __nv_bfloat16* __restrict__ beta_lin,
    const float* __restrict__ b_imag, const float* __restrict__ w_trace, const uint8_t* __restrict__ reset,
    const float* __restrict__ dtrace_out, __nv_bfloat16* __restrict__ dbeta, float* __restrict__ g_b_imag) {
  const int H = S.H;
  const float anchor = (S.secant && S.anchor_ptr) ? *S.anchor_ptr : 0.f;
  const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;
  const int h = (blockIdx.x * 64 + tx) * 2;
  const bool col_ok = h < H;
  const float s_anchor = S.secant ? phase_s0(anchor) : 0.f;
  float acc0 = 0.f, acc1 = 0.f;
  if (col_ok) {
    const float bi0 = b_imag[h], bi1 = b_imag[h + 1], wt0 = w_trace[h], wt1 = w_trace[h + 1];
    for (int j = 0; j < TILE_ROWS / 4; ++j) {
      const int m = blockIdx.y * TILE_ROWS + ty + 4 * j;
      if (m >= S.M) break;
      const int b = m / S.Tc, t = m % S.Tc;
      const long long e = (long long)m * H + h;
      float2 g = *reinterpret_cast<const float2*>(gz + e);
      if (t < S.Tc - 1) {
        if (!(reset && reset[m + 1])) {
          const float2 gn = *reinterpret_cast<const float2*>(gz + e + H);
          g.x += wt0 * gn.x; g.y += wt1 * gn.y;
        }
      } else if (dtrace_out) {
        g.x += dtrace_out[(long long)b * H + h]; g.y += dtrace_out[(long long)b * H + h + 1];
      }
      const float2 bl = ld2(beta_lin + e);
      const float d0 = g.x * phase_slope(bl.x + bi0, S.secant, anchor, s_anchor, S.floor_);
      const float d1 = g.y * phase_slope(bl.y + bi1, S.secant, anchor, s_anchor, S.floor_);
      st2(dbeta + e, d0, d1);
      acc0 += d0; acc1 += d1;
    }
  }
  __shared__ float sh[2][4][64];
  sh[0][ty][tx] = acc0; sh[1][ty][tx] = acc1;
  __syncthreads();
  if (ty == 0 && col_ok) {
    float a0 = 0.f, a1 = 0.f;
#pragma unroll
    for (int r = 0; r < 4; ++r) { a0 += sh[0][r][tx]; a1 += sh[1][r][tx]; }
    atomicAdd(g_b_imag + h, a0); atomicAdd(g_b_imag + h + 1, a1);
  }
}

CoreScalars make_scalars(const LoomFfnCore* a) {
  CoreScalars S;
  S.alpha_gate = 0.f; S.alpha_ptr = a->alpha_gate; S.anchor_ptr = a->anchor; S.powlu_m = a->powlu_m; S.tria_alpha = a->tria_alpha; S.floor_ = a->phase_floor;
  S.axis = a->axis; S.secant = a->secant; S.Tc = a->Tc; S.H = a->H; S.M = a->B * a->Tc; S.B = a->B;
  return S;
}

}  // namespace

extern "C" int loom_ffn_core_fwd(const LoomFfnCore* a, cudaStream_t stream) {
  if (a->H % 2) return -1;
  CoreScalars S = make_scalars(a);
  const long long n = (long long)S.M * (S.H / 2);
  static int tiled = -1;           // LOOM_CORE_FWD=flat selects the one-pair-per-thread forward
  if (tiled < 0) { const char* e = getenv("LOOM_CORE_FWD"); tiled = (e != nullptr && e[0] == 'f') ? 0 : 1; }
  dim3 grid_t((S.H / 2 + 63) / 64, (S.M + FWD_ROWS - 1) / FWD_ROWS);
#define LOOM_FWD(AX)                                                                                              \
  if (tiled) { LOOM_FWD_K(ffn_core_fwd_tiled_kernel<AX>, grid_t, 2 * FWD_SLOTS * 256 * 4); }                     \
  else { LOOM_FWD_K(ffn_core_fwd_kernel<AX>, (unsigned)((n + 255) / 256), 0); }
#define LOOM_FWD_K(KERNEL, GRID, SHM)                                                                             \
  if (S.M <= 16)                                                                                                  \
    loom::launch_pdl(KERNEL, dim3(GRID), dim3(256), (size_t)(SHM), stream,                                        \
      S, (const __nv_bfloat16*)a->x_real, (const __nv_bfloat16*)a->p_in, a->b_real, (const __nv_bfloat16*)a->gate_lin, \
      (const __nv_bfloat16*)a->beta_lin, a->b_imag, a->w_trace, a->trace_in, a->reset, (const __nv_bfloat16*)a->c_prev, \
      a->seed, a->seed_valid, a->gate_w, (__nv_bfloat16*)a->o_out, (__nv_bfloat16*)a->c_out, (__nv_bfloat16*)a->p_out,  \
      a->trace_out, a->beta_sq_sum);                                                                              \
  else KERNEL<<<GRID, 256, SHM, stream>>>(                                       \
      S, (const __nv_bfloat16*)a->x_real, (const __nv_bfloat16*)a->p_in, a->b_real, (const __nv_bfloat16*)a->gate_lin, \
      (const __nv_bfloat16*)a->beta_lin, a->b_imag, a->w_trace, a->trace_in, a->reset, (const __nv_bfloat16*)a->c_prev, \
      a->seed, a->seed_valid, a->gate_w, (__nv_bfloat16*)a->o_out, (__nv_bfloat16*)a->c_out, (__nv_bfloat16*)a->p_out,  \
      a->trace_out, a->beta_sq_sum)
  switch (S.axis) {      // the axis is a template argument so the +-1 entries of R_axis fold into the products
    case 0: LOOM_FWD(0); break;
    case 1: LOOM_FWD(1); break;
    case 2: LOOM_FWD(2); break;
    default: LOOM_FWD(-1); break;
  }
#undef LOOM_FWD
#undef LOOM_FWD_K
  return (int)cudaGetLastError();
}

extern "C" int loom_ffn_core_bwd(const LoomFfnCore* a, cudaStream_t stream) {
  if (a->H % 2) return -1;
  CoreScalars S = make_scalars(a);
  dim3 grid((S.H / 2 + 63) / 64, (S.M + TILE_ROWS - 1) / TILE_ROWS);
  // how pass A gets its next row: 2 = cp.async into per-thread shared-memory slots (default), 1 = L1 prefetch,
  // 0 = loads on demand (LOOM_CORE_PREFETCH)
  static int pf = -1;
  if (pf < 0) { const char* e = getenv("LOOM_CORE_PREFETCH"); pf = (e != nullptr && e[0] >= '0' && e[0] <= '2') ? e[0] - '0' : 2; }
  const size_t stage_bytes = pf == 2 ? (size_t)2 * 25 * 256 * sizeof(uint32_t) : 0;
#define LOOM_BWD(AX)                                                                                              \
  if (pf == 2) { LOOM_BWD_PF(AX, 2); } else if (pf == 1) { LOOM_BWD_PF(AX, 1); } else { LOOM_BWD_PF(AX, 0); }
#define LOOM_BWD_PF(AX, PFM)                                                                                      \
  { static bool big_ = false;                                                                                     \
    if (!big_) { cudaFuncSetAttribute(ffn_core_bwd_a_kernel<AX, PFM>, cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * 25 * 256 * 4); big_ = true; } } \
  ffn_core_bwd_a_kernel<AX, PFM><<<grid, 256, stage_bytes, stream>>>(                                             \
      S, (const __nv_bfloat16*)a->x_real, (const __nv_bfloat16*)a->p_in, a->b_real, (const __nv_bfloat16*)a->gate_lin, \
      (const __nv_bfloat16*)a->beta_lin, a->b_imag, a->w_trace, a->trace_in, a->reset, (const __nv_bfloat16*)a->c_prev, \
      a->seed, a->seed_valid, a->gate_w, (const __nv_bfloat16*)a->d_o, (const __nv_bfloat16*)a->d_c,                  \
      (const __nv_bfloat16*)a->d_pout, (__nv_bfloat16*)a->dx_real, (__nv_bfloat16*)a->dp_in, (__nv_bfloat16*)a->dgate_lin, \
      a->gz, (__nv_bfloat16*)a->dc_prev, a->dseed, a->dtrace_in, a->g_b_real, a->g_w_trace, a->g_scalars)
  switch (S.axis) {
    case 0: LOOM_BWD(0); break;
    case 1: LOOM_BWD(1); break;
    case 2: LOOM_BWD(2); break;
    default: LOOM_BWD(-1); break;
  }
#undef LOOM_BWD
#undef LOOM_BWD_PF
  ffn_core_bwd_b_kernel<<<grid, 256, 0, stream>>>(S, a->gz, (const __nv_bfloat16*)a->beta_lin, a->b_imag, a->w_trace,
                                                  a->reset, a->dtrace_out, (__nv_bfloat16*)a->dbeta, a->g_b_imag);
  return (int)cudaGetLastError();
}
