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
  LoomOperand a[16];
  int k_len[16], a_k0[16], b_k0[16];
  int nseg;
  LoomOperand b;
  LoomOperand bseg[16];  // per-segment B operands, used instead of `b` when b_per_seg != 0
  int b_per_seg;
  int a_mn_major, b_mn_major;
  void* c;
  long long ldc, ldc_head;
  const float* bias;
  int M, N, heads;       // N = output columns per group
  int accumulate, out_fp32;
  int bn;                // tile width: 64, 128 or 256
  int swap_mn_strides;   // debugging aid: exchange the two descriptor strides of MN-major operands
  int* status;           // device word; non-zero after a bounded wait gave up
  // sharded-weight gather: when gather_world > 1, B's 64-row blocks are owned by ranks in contiguous runs of
  // ceil(ceil(N/64)/gather_world) blocks; b_peer_ptr[r] is rank r's copy of B (same layout as `b`, peer-mapped
  // memory), and `b` itself is this rank's copy, which the launch completes as a side effect.
  int gather_world, gather_rank;
  const void* b_peer_ptr[8];
  // tensor parallelism.  a_world > 1: A (single segment, K-major) is row-sharded, rank r's rows live in
  // a_peer_ptr[r] (a full-size buffer per rank; a_rows_per_rank is a multiple of 128).  rs_world > 1: instead of
  // storing C, store the fp32 product of the rows owned by rank r into slot rs_rank of rank r's staging buffer
  // rs_out[r] = [rs_world][rs_rows_per_rank][N] (row pitch ldc), i.e. the GEMM's epilogue is the scatter of a
  // reduce-scatter; the caller brackets the launch with loom_tp_barrier and the owner sums its slots afterwards.
  int a_world, a_rows_per_rank;
  const void* a_peer_ptr[8];
  int rs_world, rs_rank, rs_rows_per_rank;
  float* rs_out[8];
  // pair != 0: 256 x bn tiles computed by clusters of two CTAs (tcgen05 cta_group::2); bn must be 128, 192 or 256 and
  // none of the collective variants above may be active
  int pair;
  // rope_hd != 0 (pair tiles, K-major operands, bn a multiple of rope_hd): the product is the [Q | K | V] projection
  // of M = B * Tc tokens and the epilogue, instead of storing C, rotates the Q and K heads (rotate-half, fp32, tables
  // [M, HD]) and writes rotated Q rows into rope_q (row pitch rope_q_ld), rotated K and plain V into the caches
  // [B, T, KVH, HD] at positions rope_s + t.
  int rope_hd, rope_qh, rope_kvh, rope_tc, rope_t, rope_s;
  long long rope_q_ld;
  const float* rope_cos; const float* rope_sin;
  void* rope_q; void* rope_k; void* rope_v;
} LoomGemm;

// Cross-rank barrier on peer-mapped flag words (one int per rank in each rank's `flags` buffer): publish `epoch`
// to every peer, then wait (bounded; a timeout records `code` in *status) until every peer has published it.
int loom_tp_barrier(int* const* flags_peer, int world, int rank, int epoch, int* status, int code, cudaStream_t stream);

int loom_gemm_bf16(const LoomGemm* g, cudaStream_t stream);

// ---- flat optimizer (optim.cu) ----
int loom_grad_norm(const float* grads, long long n, float max_norm, float* partial, int nparts, float* stats,
                   float* atom_out, cudaStream_t stream);
// finite flag &= (status word == 0); stats[3] counts skipped updates (sticky)
int loom_status_gate(const int* status, float* stats, cudaStream_t stream);
int loom_adamw_flat(float* p, const float* g, float* m, float* v, void* shadow_bf16, const float* lr_mult,
                    const float* wd_blk, const float* active, const float* stats, const float* hyper,
                    long long nblk, cudaStream_t stream);
int loom_atom_flat(float* p, const float* g, float* m, float* v, void* shadow_bf16, const float* lr_mult,
                   const float* wd_blk, const float* cnt_blk, float* gprev, float* pnode, float* trust,
                   const float* stats, const float* hyper, float* atom_out, long long nblk, cudaStream_t stream);
int loom_cast_shadow(const float* p, void* shadow_bf16, long long n, cudaStream_t stream);

// ---- fused Paraplex core + Tria step (ffn_core.cu) ----
// Activations are bf16 [M, H] with M = B*Tc rows ordered (b, t); carriers are bf16 planes [9][M][H].
// Null pointers switch optional inputs/outputs off.  Gradient accumulators (g_*) are fp32 and are
// added to atomically.
typedef struct {
  int B, Tc, H;
  int axis;                 // Tria axis 0..2, or -1 when Tria is off
  int secant;               // phase slope mode
  float powlu_m, tria_alpha, phase_floor;
  const float* alpha_gate;  // device scalar 0.25*tanh(raw) or null (no incoming gate value)
  const float* anchor;      // device scalar (secant mode)
  const void* x_real; const void* p_in; const float* b_real;
  const void* gate_lin;     // null: the gate reads R itself
  const void* beta_lin; const float* b_imag; const float* w_trace;
  const float* trace_in;    // [B,H] or null
  const uint8_t* reset;     // [M] or null
  const void* c_prev;       // planes or null
  const float* seed;        // [B,H,9] or null
  const uint8_t* seed_valid;
  const float* gate_w;      // [9] soft-maxed, or null
  // forward outputs
  void* o_out; void* c_out; void* p_out; float* trace_out; float* beta_sq_sum;
  // backward inputs
  const void* d_o; const void* d_c; const void* d_pout; const float* dtrace_out;
  // backward outputs
  void* dx_real; void* dp_in; void* dgate_lin; void* dbeta; float* gz; void* dc_prev; float* dseed; float* dtrace_in;
  float* g_b_real; float* g_w_trace; float* g_b_imag; float* g_scalars;   // g_scalars: [0] d alpha_gate, [1..9] d gate_w
} LoomFfnCore;
int loom_ffn_core_fwd(const LoomFfnCore* a, cudaStream_t stream);
int loom_ffn_core_bwd(const LoomFfnCore* a, cudaStream_t stream);

// ---- bandwidth-bound kernels (elementwise.cu) ----
int loom_rope_store(const void* qkv, const float* cs, const float* sn, void* qkc, void* kcache, void* vcache, int M,
                    int Tc, int T, int s_off, int QH, int KVH, int HD, cudaStream_t st);
// [M, QH, 3, HD] -> [M, 3, QH, HD] (bf16, HD a multiple of 8)
int loom_sector_fold(const void* src, void* dst, long long M, int QH, int HD, cudaStream_t st);
int loom_rope_bwd(const void* dq_attn, const void* dqkc, const float* dkc, const float* dvc, const float* cs,
                  const float* sn, void* dqkv, int M, int Tc, int T, int s_off, int QH, int KVH, int HD, int G,
                  cudaStream_t st);
// ---- KV-cache attention for decode (decode_attention.cu) ----
int loom_decode_attn_workspace_floats(int B, int QH, int KVH, int HD, int NS);
int loom_decode_attn(const void* q, const void* kc, const void* vc, const long long* pos, void* out_c, void* out_k, float* ws,
                     int B, int S, int QH, int KVH, int HD, int NS, long long out_ld, long long q_ld, int* status,
                     cudaStream_t st);

// ---- Tria readout and RMS-type norms (readout.cu) ----
int loom_slot_pool_fwd(const float* keys, const float* w9, float* pooled, float* stats, int BK, int H, cudaStream_t st);
int loom_slot_pool_bwd(const float* keys, const float* w9, const float* pooled, const float* stats, const float* dpooled,
                       float* dkeys, float* dw9_part, int BK, int H, cudaStream_t st);
int loom_cross_attn_fwd(const void* q, const void* k, const void* v, const uint8_t* allowed, void* out, float* prob, int B,
                        int T, int Kn, int N, float scale, cudaStream_t st);
int loom_cross_attn_bwd(const void* dout, const void* q, const void* k, const void* v, const float* prob, float* ds, void* dq,
                        void* dk, void* dv, int B, int T, int Kn, int N, float scale, cudaStream_t st);
int loom_fixed_rms(int bwd, const void* dy, const void* x, void* out, long long rows, int heads, int HD, long long ld,
                   float target, float eps, cudaStream_t st);
int loom_rms_norm_fwd(const void* x, const float* w, void* y, int M, int N, float eps, cudaStream_t st);
int loom_rms_norm_bwd(const void* dy, const void* x, const float* w, void* dx, float* gw_part, int nblocks, int M, int N,
                      float eps, cudaStream_t st);

// depth-attention backward organised per history slot (depth_read_bwd.cu)
// lse_in/lse_out (both or neither): the sublayer's log-sum-exp rows are copied into the staging buffer by the same launch
int loom_dread_stage(const void* a, const void* b_or_null, const void* m_out, void* dm, float* dd, const float* lse_in,
                     float* lse_out, long long MQ, int HD, cudaStream_t st);
// in_ld / out_ld: elements between consecutive rows of hk_slot, hv_slot / of dk, dv (QH*HD when densely packed;
// 2*QH*HD when K and V share [K | V] rows); multiples of 8
int loom_dread_slot_bwd(const float* q_all, const void* hk_slot, const void* hv_slot, const void* dm_all,
                        const float* lse_all, const float* dd_all, void* dk, void* dv, float* gq_all, int sub0, int S,
                        int M, int QH, int HD, long long in_ld, long long out_ld, cudaStream_t st);
// slot_stride / row_stride: elements between history slots / rows (0, 0 = densely packed [n, M, QH, HD]); the backward
// form takes densely packed history only
int loom_dread(int bwd, const float* q, const void* hk, const void* hv, void* out, float* lse, const void* dm, float* dhk,
               float* dhv, float* gq, int n, long long MQ, int QH, int HD, long long slot_stride, long long row_stride,
               cudaStream_t st);
// cap > 0 shrinks each addend to an RMS of at most `cap` before the sum (cap <= 0: plain sum)
int loom_add_ln_fwd(const void* a, const void* b, const float* w, const float* bias, void* y, void* x, float* mean,
                    float* rstd, int M, int N, float eps, float cap, cudaStream_t st);
int loom_cap_bwd(const void* dy, const void* a, void* da, int M, int N, float cap, cudaStream_t st);
int loom_add_ln_bwd(const void* dy, const void* x, const float* mean, const float* rstd, const float* w, void* dx,
                    float* gw, float* gb, int M, int N, cudaStream_t st);
int loom_colsum(const void* dy, float* gb, int M, int N, long long ld, cudaStream_t st);
/* anchor <- decay * anchor + (1 - decay) * max(sqrt(*beta_sq_sum * inv_n), 1e-4); *snap = the updated anchor. */
int loom_anchor_ema(const float* beta_sq_sum, float inv_n, float decay, float* anchor, float* snap, cudaStream_t st);
int loom_ce(void* logits, const long long* targets, float* nll, const float* scale_ptr, long long M, int V,
            long long ignore_index, int write_grad, cudaStream_t st);

// ---- temporal carry endpoint + PolARM (temporal.cu) ----
int loom_temporal_fwd(const void* depth, const uint8_t* reset, const float* state_in, const uint8_t* fired, float beta,
                      float* state_out, float* raw_out, float* ckpt, int B, int Tc, int H, cudaStream_t st);
int loom_temporal_bwd(const void* depth, const uint8_t* reset, const float* state_in, const uint8_t* fired, float beta,
                      const float* raw, const float* ckpt, const float* dstate, void* ddepth, float* dstate_in, int B,
                      int Tc, int H, cudaStream_t st);

// ---- dual-context attention (attention_fwd.cu / attention_bwd.cu) ----
// qkc [B*Tc, 3, QH, HD] bf16 (sector 0 = rotated queries, 1 = A@K, 2 = A@V); caches [B, T, KVH, HD] bf16;
// lse [B, QH, Tc] fp32; seg [B, T] int32 or null (tokens attend only within their own id; every id must occupy one
// contiguous run of the sequence, as document counters and packed-example indices do).  The chunk's queries sit at
// absolute positions [s, e).
// Backward: dqkc same layout as qkc (sectors 1, 2 are read); dq_attn [B*Tc, QH, HD] bf16 out;
// dk_heads / dv_heads [B, T, QH, HD] fp32 are per-query-head key/value gradient slabs (+=, no atomics).
typedef struct {
  const void* qkc; const void* kcache; const void* vcache; float* lse; const int* seg;
  const void* dqkc; void* dq_attn; float* dk_heads; float* dv_heads;
  int B, QH, KVH, HD, Tc, T, s, e;
  int* status;
} LoomAttn;
int loom_attn_fwd(const LoomAttn* a, cudaStream_t stream);
int loom_attn_bwd(const LoomAttn* a, cudaStream_t stream);

// ---- small-batch pieces of the decode step (decode_step.cu) ----
// y[M, N] = x[M, K] . W[N, K]^T (+ bias[N]); bf16 inputs, bf16 or fp32 output, M <= 16, K a multiple of 8; ld* are row
// pitches in elements (the output may be a strided view)
int loom_skinny_linear(const void* x, long long ldx, const void* w, long long ldw, const float* bias, void* y,
                       long long ldy, int out_fp32, int M, int N, int K, cudaStream_t st);
// rotate-half RoPE of Q and K of one new token per sequence at the position stored in *pos (device int64): qkv rows
// [Q | K | V] -> q_out rows (pitch ld_q), kc / vc [B, S, KVH, HD] row *pos; cos / sin tables [table_rows, HD] fp32
int loom_decode_rope_store(const void* qkv, long long ld_qkv, const float* cos_tab, const float* sin_tab,
                           const long long* pos, void* q_out, long long ld_q, void* kc, void* vc, int B, int S,
                           int table_rows, int QH, int KVH, int HD, cudaStream_t st);

// several such products in one launch; segment i owns blocks [block0_i, block0_{i+1}) of the grid (filled in by the
// call).  The input rows of a segment are the concatenation of its pieces (each `len` elements at row pitch `ld`).
#define LOOM_SKINNY_MAX_SEG 12
#define LOOM_SKINNY_MAX_PIECE 5
typedef struct { const void* x; long long ld; int len; int pad_; } LoomSkinnyPiece;
typedef struct {
  LoomSkinnyPiece piece[LOOM_SKINNY_MAX_PIECE];
  const void* w; const float* bias; void* y;
  long long ldw, ldy;
  int npiece, N, K, out_fp32, block0;
  int wpc;                            // warps that share one output column (K split inside a block); filled in by the call
} LoomSkinnySeg;
// weights_static: no kernel earlier in the stream writes the weights or biases, so they may be fetched before the
// previous kernel has finished
typedef struct { LoomSkinnySeg seg[LOOM_SKINNY_MAX_SEG]; int nseg, M, weights_static, pad_; } LoomSkinnyArgs;
int loom_skinny_multi(LoomSkinnyArgs* a, cudaStream_t st);
// the same products for up to 128 rows on the tensor cores (decode_gemm.cu): a CTA owns 128 rows of one weight matrix
// (M side of tcgen05.mma), the batch is the N side; `status`: device word set when a bounded wait gives up
int loom_decode_gemm(const LoomSkinnyArgs* a, int* status, cudaStream_t st);
// booleans of one decode step (all [B] bytes) from the device-side position, the incoming tokens and the flags of the
// previous step; carry_token < 0: no carry token
int loom_decode_step_flags(const long long* pos, const long long* tok, const void* pending, const void* have_carry,
                           void* fire, void* reset, void* row_reset, void* seed_valid, int B, long long window,
                           long long seq_len, int hard_enabled, long long carry_token, int temporal, cudaStream_t st);
// boundary-key append of one decode step: ca_k / ca_v [B, cap, N] bf16, ca_valid / allowed [B, cap] bytes, *ca_len the
// slot count before the append (the caller adds *any_out afterwards)
int loom_decode_ca_append(const void* newk, const void* newv, long long ld_new, const void* fire, void* ca_k, void* ca_v,
                          void* ca_valid, const long long* ca_len, void* allowed, long long* any_out, void* pending,
                          void* have_carry, int B, int cap, int N, cudaStream_t st);

// ---- fused gradient reduce-scatter + AdamW + parameter all-gather over peer memory (comm.cu) ----
typedef struct {
  int W, rank;
  long long nblk;                 // number of 256-element blocks of the flat buffers
  float* grads[8]; float* params[8]; void* shadow[8]; int* sync[8];   // peer-mapped symmetric buffers
  float* mc_grads;                // NVSwitch multicast mapping of the gradient buffers or null
  float* m; float* v;             // local optimizer moments (full-size; only the own shard is touched)
  const float* lr_mult; const float* wd_blk; const float* active; const float* hyper;
  float* stats;                   // [0] norm, [1] clip, [2] finite
  float* sumsq_local;             // one float, zero before the first call
  float max_norm;
  int* status;
  // optional sharded-parameter mode (all three null: contiguous block ranges, full-size moments, every block
  // stored to every peer): owner rank per block, compact index of the block in the owner's m / v, replicate flag
  const uint8_t* owner_blk; const int* slot_blk; const uint8_t* replicate_blk;
  // optional: n_anchor (<= 64) per-layer phase radii kept identical on all ranks by the same exchange (mean over
  // ranks, or rank 0's values with anchor_rank0); needs sync buffers of at least 64 + 64 * W words
  float* anchors; int n_anchor; int anchor_rank0;
} LoomP2P;
int loom_p2p_grad_step(const LoomP2P* a, cudaStream_t stream);
// Same exchange with ATOM as the update rule (contiguous shards; see comm.cu)
int loom_p2p_grad_step_atom(const LoomP2P* a, const float* cnt_blk, float* gprev, float* pnode, float* trust, float* atom_out,
                            cudaStream_t stream);

#ifdef __cplusplus
}
#endif
