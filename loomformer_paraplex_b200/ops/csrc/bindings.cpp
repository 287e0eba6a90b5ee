// PyTorch <-> kernel glue: unwraps tensors into the plain C launchers of loom_c_api.h.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cstring>
#include <tuple>
#include <vector>
#include "loom_c_api.h"

namespace {

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

LoomOperand operand(const torch::Tensor& t, bool& ok) {
  // accepts [rows, cols] or [rows, heads, cols] bf16 views with unit stride on the last dim
  LoomOperand o{};
  ok = t.is_cuda() && t.scalar_type() == torch::kBFloat16 && t.stride(-1) == 1 && (t.dim() == 2 || t.dim() == 3);
  if (!ok) return o;
  o.ptr = t.data_ptr();
  o.rows = t.size(0);
  o.cols = t.size(-1);
  o.ld_row = t.stride(0);
  if (t.dim() == 3) { o.heads = t.size(1); o.ld_head = t.stride(1); } else { o.heads = 1; o.ld_head = 0; }
  return o;
}

// General entry: see LoomGemm.  `a_list` holds the K segments.
void gemm(std::vector<torch::Tensor> a_list, std::vector<int64_t> k_len, std::vector<int64_t> a_k0,
          std::vector<int64_t> b_k0, std::vector<torch::Tensor> b_list, bool a_mn, bool b_mn, torch::Tensor c,
          c10::optional<torch::Tensor> bias, int64_t M, int64_t N, int64_t heads, bool accumulate, int64_t bn,
          bool swap_mn, torch::Tensor status, std::vector<int64_t> b_peer_ptrs, int64_t gather_rank,
          std::vector<int64_t> a_peer_ptrs, int64_t a_rows_per_rank, std::vector<int64_t> rs_out_ptrs,
          int64_t rs_rows_per_rank, int64_t rs_rank, int64_t pair) {
  TORCH_CHECK(a_list.size() >= 1 && a_list.size() <= 16, "1..16 K segments");
  TORCH_CHECK(b_list.size() == 1 || b_list.size() == a_list.size(), "B: one operand, or one per segment");
  TORCH_CHECK(c.is_cuda() && c.stride(-1) == 1, "C must be a CUDA tensor with unit inner stride");
  TORCH_CHECK(c.scalar_type() == torch::kBFloat16 || c.scalar_type() == torch::kFloat32, "C must be bf16 or fp32");
  const c10::cuda::CUDAGuard guard(c.device());
  LoomGemm g{};
  bool ok = true;
  for (size_t i = 0; i < a_list.size(); ++i) {
    g.a[i] = operand(a_list[i], ok);
    TORCH_CHECK(ok, "bad A operand ", i);
    g.k_len[i] = (int)k_len[i]; g.a_k0[i] = (int)a_k0[i]; g.b_k0[i] = (int)b_k0[i];
  }
  g.nseg = (int)a_list.size();
  if (b_list.size() == 1) {
    g.b = operand(b_list[0], ok);
    TORCH_CHECK(ok, "bad B operand");
  } else {
    g.b_per_seg = 1;
    for (size_t i = 0; i < b_list.size(); ++i) {
      g.bseg[i] = operand(b_list[i], ok);
      TORCH_CHECK(ok, "bad B operand ", i);
    }
  }
  g.a_mn_major = a_mn; g.b_mn_major = b_mn;
  g.c = c.data_ptr();
  g.ldc = c.stride(0);
  g.ldc_head = c.dim() == 3 ? c.stride(1) : 0;
  if (bias.has_value()) {
    TORCH_CHECK(bias->scalar_type() == torch::kFloat32 && bias->is_contiguous(), "bias must be contiguous fp32");
    g.bias = bias->data_ptr<float>();
  }
  g.M = (int)M; g.N = (int)N; g.heads = (int)heads;
  g.accumulate = accumulate; g.out_fp32 = c.scalar_type() == torch::kFloat32;
  g.bn = (int)bn; g.swap_mn_strides = swap_mn; g.pair = (int)pair;
  g.status = status.data_ptr<int>();
  if (b_peer_ptrs.size() > 1) {
    TORCH_CHECK(b_peer_ptrs.size() <= 8 && b_list.size() == 1, "gather: up to 8 ranks, one B operand");
    g.gather_world = (int)b_peer_ptrs.size(); g.gather_rank = (int)gather_rank;
    for (size_t i = 0; i < b_peer_ptrs.size(); ++i) g.b_peer_ptr[i] = reinterpret_cast<const void*>(b_peer_ptrs[i]);
  }
  if (a_peer_ptrs.size() > 1) {
    TORCH_CHECK(a_peer_ptrs.size() <= 8, "row-sharded A: up to 8 ranks");
    g.a_world = (int)a_peer_ptrs.size(); g.a_rows_per_rank = (int)a_rows_per_rank;
    for (size_t i = 0; i < a_peer_ptrs.size(); ++i) g.a_peer_ptr[i] = reinterpret_cast<const void*>(a_peer_ptrs[i]);
  }
  if (rs_out_ptrs.size() > 1) {
    TORCH_CHECK(rs_out_ptrs.size() <= 8, "reduce-scatter epilogue: up to 8 ranks");
    g.rs_world = (int)rs_out_ptrs.size(); g.rs_rows_per_rank = (int)rs_rows_per_rank; g.rs_rank = (int)rs_rank;
    for (size_t i = 0; i < rs_out_ptrs.size(); ++i) g.rs_out[i] = reinterpret_cast<float*>(rs_out_ptrs[i]);
  }
  int rc = loom_gemm_bf16(&g, cur_stream());
  TORCH_CHECK(rc == 0, "loom_gemm_bf16 failed with code ", rc);
}

float* fptr(const torch::Tensor& t) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == torch::kFloat32 && t.is_contiguous(), "expected contiguous fp32 CUDA tensor");
  return t.data_ptr<float>();
}
void* optptr(const c10::optional<torch::Tensor>& t) { return t.has_value() ? t->data_ptr() : nullptr; }

void grad_norm(torch::Tensor grads, double max_norm, torch::Tensor partial, torch::Tensor stats,
               c10::optional<torch::Tensor> atom_out) {
  const c10::cuda::CUDAGuard guard(grads.device());
  int rc = loom_grad_norm(fptr(grads), grads.numel(), (float)max_norm, fptr(partial), (int)partial.numel(), fptr(stats),
                          atom_out.has_value() ? fptr(*atom_out) : nullptr, cur_stream());
  TORCH_CHECK(rc == 0, "loom_grad_norm failed: ", rc);
}

// [Q | K | V] projection with RoPE and the cache write in the epilogue (pair tiles): x [M, K] bf16, w [(QH + 2 KVH) HD, K]
// bf16, cos / sin [M, HD] fp32, q_out rows [M, QH * HD] (row pitch taken from the view), caches [B, T, KVH, HD]
void gemm_qkv_rope(torch::Tensor x, torch::Tensor w, c10::optional<torch::Tensor> bias, torch::Tensor cos_t, torch::Tensor sin_t,
                   torch::Tensor q_out, torch::Tensor kcache, torch::Tensor vcache, int64_t Tc, int64_t s, int64_t QH, int64_t KVH,
                   int64_t HD, int64_t bn, torch::Tensor status) {
  const c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.dim() == 2 && w.dim() == 2 && x.size(1) == w.size(1) && w.size(0) == (QH + 2 * KVH) * HD, "gemm_qkv_rope: shapes");
  const int64_t M = x.size(0);
  TORCH_CHECK(cos_t.scalar_type() == torch::kFloat32 && sin_t.scalar_type() == torch::kFloat32 && cos_t.is_contiguous() &&
              sin_t.is_contiguous() && cos_t.numel() == M * HD && sin_t.numel() == M * HD, "gemm_qkv_rope: cos / sin [M, HD] fp32");
  TORCH_CHECK(q_out.dim() == 2 && q_out.size(0) == M && q_out.size(1) == QH * HD && q_out.stride(1) == 1 &&
              q_out.scalar_type() == torch::kBFloat16, "gemm_qkv_rope: q_out rows");
  TORCH_CHECK(kcache.dim() == 4 && kcache.is_contiguous() && vcache.is_contiguous() && vcache.sizes() == kcache.sizes() &&
              kcache.size(2) == KVH && kcache.size(3) == HD && kcache.scalar_type() == torch::kBFloat16 &&
              vcache.scalar_type() == torch::kBFloat16 && M == kcache.size(0) * Tc, "gemm_qkv_rope: caches [B, T, KVH, HD]");
  LoomGemm g{};
  bool ok = true;
  g.a[0] = operand(x, ok);
  g.b = operand(w, ok);
  TORCH_CHECK(ok, "gemm_qkv_rope: bad operand");
  g.k_len[0] = (int)x.size(1); g.nseg = 1;
  g.c = q_out.data_ptr(); g.ldc = q_out.stride(0);
  if (bias.has_value()) {
    TORCH_CHECK(bias->scalar_type() == torch::kFloat32 && bias->is_contiguous() && bias->numel() == w.size(0), "bias: contiguous fp32 [N]");
    g.bias = bias->data_ptr<float>();
  }
  g.M = (int)M; g.N = (int)w.size(0); g.heads = 1; g.bn = (int)bn; g.pair = 1;
  g.status = status.data_ptr<int>();
  g.rope_hd = (int)HD; g.rope_qh = (int)QH; g.rope_kvh = (int)KVH; g.rope_tc = (int)Tc; g.rope_t = (int)kcache.size(1); g.rope_s = (int)s;
  g.rope_q_ld = q_out.stride(0);
  g.rope_cos = cos_t.data_ptr<float>(); g.rope_sin = sin_t.data_ptr<float>();
  g.rope_q = q_out.data_ptr(); g.rope_k = kcache.data_ptr(); g.rope_v = vcache.data_ptr();
  int rc = loom_gemm_bf16(&g, cur_stream());
  TORCH_CHECK(rc == 0, "loom_gemm_bf16 (QKV + RoPE) failed: ", rc);
}

void sector_fold(torch::Tensor src, torch::Tensor dst, int64_t M, int64_t QH, int64_t HD) {
  const c10::cuda::CUDAGuard guard(src.device());
  TORCH_CHECK(src.is_contiguous() && dst.is_contiguous() && src.scalar_type() == torch::kBFloat16 && dst.scalar_type() == torch::kBFloat16 &&
              src.numel() == M * QH * 3 * HD && dst.numel() == src.numel(), "sector_fold: packed bf16 [M, QH, 3, HD] -> [M, 3, QH, HD]");
  int rc = loom_sector_fold(src.data_ptr(), dst.data_ptr(), (long long)M, (int)QH, (int)HD, cur_stream());
  TORCH_CHECK(rc == 0, "loom_sector_fold failed: ", rc);
}

void status_gate(torch::Tensor status, torch::Tensor stats) {
  const c10::cuda::CUDAGuard guard(stats.device());
  TORCH_CHECK(status.is_cuda() && status.scalar_type() == torch::kInt32, "status word: int32 CUDA tensor");
  int rc = loom_status_gate(status.data_ptr<int>(), fptr(stats), cur_stream());
  TORCH_CHECK(rc == 0, "loom_status_gate failed: ", rc);
}

void adamw_flat(torch::Tensor p, torch::Tensor g, torch::Tensor m, torch::Tensor v, c10::optional<torch::Tensor> shadow,
                torch::Tensor lr_mult, torch::Tensor wd, torch::Tensor active, torch::Tensor stats, torch::Tensor hyper) {
  const c10::cuda::CUDAGuard guard(p.device());
  int rc = loom_adamw_flat(fptr(p), fptr(g), fptr(m), fptr(v), optptr(shadow), fptr(lr_mult), fptr(wd), fptr(active),
                           fptr(stats), fptr(hyper), p.numel() / 256, cur_stream());
  TORCH_CHECK(rc == 0, "loom_adamw_flat failed: ", rc);
}

void atom_flat(torch::Tensor p, torch::Tensor g, torch::Tensor m, torch::Tensor v, c10::optional<torch::Tensor> shadow,
               torch::Tensor lr_mult, torch::Tensor wd, torch::Tensor cnt, torch::Tensor gprev, torch::Tensor pnode,
               torch::Tensor trust, torch::Tensor stats, torch::Tensor hyper, torch::Tensor atom_out) {
  const c10::cuda::CUDAGuard guard(p.device());
  int rc = loom_atom_flat(fptr(p), fptr(g), fptr(m), fptr(v), optptr(shadow), fptr(lr_mult), fptr(wd), fptr(cnt),
                          fptr(gprev), fptr(pnode), fptr(trust), fptr(stats), fptr(hyper), fptr(atom_out),
                          p.numel() / 256, cur_stream());
  TORCH_CHECK(rc == 0, "loom_atom_flat failed: ", rc);
}

void cast_shadow(torch::Tensor p, torch::Tensor shadow) {
  const c10::cuda::CUDAGuard guard(p.device());
  TORCH_CHECK(shadow.scalar_type() == torch::kBFloat16 && shadow.numel() == p.numel(), "bad shadow");
  int rc = loom_cast_shadow(fptr(p), shadow.data_ptr(), p.numel(), cur_stream());
  TORCH_CHECK(rc == 0, "loom_cast_shadow failed: ", rc);
}

typedef c10::optional<torch::Tensor> OptT;
const void* cp(const OptT& t) { return t.has_value() ? t->data_ptr() : nullptr; }
void* mp(const OptT& t) { return t.has_value() ? t->data_ptr() : nullptr; }
const float* cf(const OptT& t) { return t.has_value() ? (const float*)t->data_ptr() : nullptr; }
float* mf(const OptT& t) { return t.has_value() ? (float*)t->data_ptr() : nullptr; }
const uint8_t* cu8(const OptT& t) { return t.has_value() ? (const uint8_t*)t->data_ptr() : nullptr; }

// forward when bwd == false, backward otherwise; tensors not used by a direction may be None.
void ffn_core(bool bwd, int64_t B, int64_t Tc, int64_t H, int64_t axis, bool secant, double powlu_m, double tria_alpha,
              double phase_floor, OptT alpha_gate, OptT anchor, torch::Tensor x_real, OptT p_in, torch::Tensor b_real,
              OptT gate_lin, torch::Tensor beta_lin, torch::Tensor b_imag, torch::Tensor w_trace, OptT trace_in,
              OptT reset, OptT c_prev, OptT seed, OptT seed_valid, OptT gate_w,
              OptT o_out, OptT c_out, OptT p_out, OptT trace_out, OptT beta_sq_sum,
              OptT d_o, OptT d_c, OptT d_pout, OptT dtrace_out,
              OptT dx_real, OptT dp_in, OptT dgate_lin, OptT dbeta, OptT gz, OptT dc_prev, OptT dseed, OptT dtrace_in,
              OptT g_b_real, OptT g_w_trace, OptT g_b_imag, OptT g_scalars) {
  const c10::cuda::CUDAGuard guard(x_real.device());
  LoomFfnCore a{};
  a.B = (int)B; a.Tc = (int)Tc; a.H = (int)H; a.axis = (int)axis; a.secant = secant;
  a.powlu_m = (float)powlu_m; a.tria_alpha = (float)tria_alpha; a.phase_floor = (float)phase_floor;
  a.alpha_gate = cf(alpha_gate); a.anchor = cf(anchor);
  a.x_real = x_real.data_ptr(); a.p_in = cp(p_in); a.b_real = (const float*)b_real.data_ptr();
  a.gate_lin = cp(gate_lin); a.beta_lin = beta_lin.data_ptr(); a.b_imag = (const float*)b_imag.data_ptr();
  a.w_trace = (const float*)w_trace.data_ptr(); a.trace_in = cf(trace_in); a.reset = cu8(reset);
  a.c_prev = cp(c_prev); a.seed = cf(seed); a.seed_valid = cu8(seed_valid); a.gate_w = cf(gate_w);
  a.o_out = mp(o_out); a.c_out = mp(c_out); a.p_out = mp(p_out); a.trace_out = mf(trace_out); a.beta_sq_sum = mf(beta_sq_sum);
  a.d_o = cp(d_o); a.d_c = cp(d_c); a.d_pout = cp(d_pout); a.dtrace_out = cf(dtrace_out);
  a.dx_real = mp(dx_real); a.dp_in = mp(dp_in); a.dgate_lin = mp(dgate_lin); a.dbeta = mp(dbeta); a.gz = mf(gz);
  a.dc_prev = mp(dc_prev); a.dseed = mf(dseed); a.dtrace_in = mf(dtrace_in);
  a.g_b_real = mf(g_b_real); a.g_w_trace = mf(g_w_trace); a.g_b_imag = mf(g_b_imag); a.g_scalars = mf(g_scalars);
  int rc = bwd ? loom_ffn_core_bwd(&a, cur_stream()) : loom_ffn_core_fwd(&a, cur_stream());
  TORCH_CHECK(rc == 0, "loom_ffn_core failed: ", rc);
}

void rope_store(torch::Tensor qkv, torch::Tensor cs, torch::Tensor sn, torch::Tensor qkc, torch::Tensor kcache,
                torch::Tensor vcache, int64_t M, int64_t Tc, int64_t T, int64_t s, int64_t QH, int64_t KVH, int64_t HD) {
  const c10::cuda::CUDAGuard guard(qkv.device());
  int rc = loom_rope_store(qkv.data_ptr(), fptr(cs), fptr(sn), qkc.data_ptr(), kcache.data_ptr(), vcache.data_ptr(),
                           (int)M, (int)Tc, (int)T, (int)s, (int)QH, (int)KVH, (int)HD, cur_stream());
  TORCH_CHECK(rc == 0, "loom_rope_store failed: ", rc);
}

void rope_bwd(torch::Tensor dq_attn, torch::Tensor dqkc, torch::Tensor dkc, torch::Tensor dvc, torch::Tensor cs,
              torch::Tensor sn, torch::Tensor dqkv, int64_t M, int64_t Tc, int64_t T, int64_t s, int64_t QH, int64_t KVH,
              int64_t HD, int64_t G) {
  const c10::cuda::CUDAGuard guard(dqkv.device());
  int rc = loom_rope_bwd(dq_attn.data_ptr(), dqkc.data_ptr(), fptr(dkc), fptr(dvc), fptr(cs), fptr(sn), dqkv.data_ptr(),
                         (int)M, (int)Tc, (int)T, (int)s, (int)QH, (int)KVH, (int)HD, (int)G, cur_stream());
  TORCH_CHECK(rc == 0, "loom_rope_bwd failed: ", rc);
}

void decode_attn(torch::Tensor q, torch::Tensor kc, torch::Tensor vc, torch::Tensor pos, torch::Tensor out_c, torch::Tensor out_k,
                 torch::Tensor ws, int64_t B, int64_t S, int64_t QH, int64_t KVH, int64_t HD, int64_t NS,
                 c10::optional<torch::Tensor> status) {
  // outputs may be row-strided views (e.g. slices of a [B,3,QH,HD] buffer): contiguous within a sequence
  TORCH_CHECK(out_c.stride(-1) == 1 && out_k.stride(-1) == 1 && out_c.stride(0) == out_k.stride(0), "decode_attn: output layout");
  const c10::cuda::CUDAGuard guard(q.device());
  TORCH_CHECK(q.stride(-1) == 1 && q.stride(1) == q.size(2) && kc.is_contiguous() && vc.is_contiguous() &&
              pos.scalar_type() == torch::kInt64, "decode_attn: [B,QH,HD] query rows, contiguous caches, an int64 position");
  TORCH_CHECK(ws.numel() >= loom_decode_attn_workspace_floats((int)B, (int)QH, (int)KVH, (int)HD, (int)NS), "workspace too small");
  int rc = loom_decode_attn(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), pos.data_ptr<int64_t>() ? (const long long*)pos.data_ptr<int64_t>() : nullptr,
                            out_c.data_ptr(), out_k.data_ptr(), fptr(ws), (int)B, (int)S, (int)QH, (int)KVH, (int)HD, (int)NS,
                            (long long)out_c.stride(0), (long long)q.stride(0),
                            status.has_value() ? status->data_ptr<int>() : nullptr, cur_stream());
  TORCH_CHECK(rc == 0, "loom_decode_attn failed: ", rc);
}

void skinny_linear(torch::Tensor x, torch::Tensor w, c10::optional<torch::Tensor> bias, torch::Tensor y) {
  const c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.dim() == 2 && w.dim() == 2 && y.dim() == 2 && x.stride(1) == 1 && w.stride(1) == 1 && y.stride(1) == 1,
              "skinny_linear: 2-D operands with unit inner stride");
  TORCH_CHECK(x.scalar_type() == torch::kBFloat16 && w.scalar_type() == torch::kBFloat16, "skinny_linear: bf16 inputs");
  TORCH_CHECK(y.scalar_type() == torch::kBFloat16 || y.scalar_type() == torch::kFloat32, "skinny_linear: bf16 or fp32 output");
  TORCH_CHECK(x.size(1) == w.size(1) && y.size(0) == x.size(0) && y.size(1) == w.size(0), "skinny_linear: shapes");
  const float* b = nullptr;
  if (bias.has_value()) { TORCH_CHECK(bias->numel() == w.size(0), "skinny_linear: bias length"); b = fptr(*bias); }
  int rc = loom_skinny_linear(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), b, y.data_ptr(), y.stride(0),
                              y.scalar_type() == torch::kFloat32, (int)x.size(0), (int)w.size(0), (int)x.size(1), cur_stream());
  TORCH_CHECK(rc == 0, "loom_skinny_linear failed: ", rc);
}

// segs: list of (pieces, w, bias or None, y): pieces = list of [M, len] bf16 views (unit inner stride), w [N, K] bf16 rows,
// y [M, N] bf16 or fp32 view
typedef std::vector<std::tuple<std::vector<torch::Tensor>, torch::Tensor, c10::optional<torch::Tensor>, torch::Tensor>> SkinnySegs;

static void fill_skinny_args(const SkinnySegs& segs, bool weights_static, LoomSkinnyArgs& a) {
  TORCH_CHECK(!segs.empty() && (int)segs.size() <= LOOM_SKINNY_MAX_SEG, "small-batch product: 1..", LOOM_SKINNY_MAX_SEG, " segments");
  memset(&a, 0, sizeof(a));
  a.nseg = (int)segs.size();
  a.weights_static = weights_static ? 1 : 0;
  a.M = (int)std::get<3>(segs[0]).size(0);
  for (int i = 0; i < a.nseg; ++i) {
    const auto& pieces = std::get<0>(segs[i]);
    const torch::Tensor& w = std::get<1>(segs[i]);
    const auto& bias = std::get<2>(segs[i]);
    const torch::Tensor& y = std::get<3>(segs[i]);
    LoomSkinnySeg& sg = a.seg[i];
    TORCH_CHECK(!pieces.empty() && (int)pieces.size() <= LOOM_SKINNY_MAX_PIECE, "small-batch product: 1..", LOOM_SKINNY_MAX_PIECE, " pieces");
    TORCH_CHECK(w.dim() == 2 && w.stride(1) == 1 && w.scalar_type() == torch::kBFloat16, "small-batch product: bf16 weight rows");
    TORCH_CHECK(y.dim() == 2 && y.stride(1) == 1 && y.size(0) == a.M && y.size(1) == w.size(0) &&
                (y.scalar_type() == torch::kBFloat16 || y.scalar_type() == torch::kFloat32), "small-batch product: output view");
    int k = 0;
    for (size_t p = 0; p < pieces.size(); ++p) {
      const torch::Tensor& x = pieces[p];
      TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1 && x.size(0) == a.M && x.scalar_type() == torch::kBFloat16,
                  "small-batch product: bf16 [M, len] input pieces");
      sg.piece[p].x = x.data_ptr(); sg.piece[p].ld = a.M > 1 ? x.stride(0) : 0; sg.piece[p].len = (int)x.size(1);
      k += (int)x.size(1);
    }
    TORCH_CHECK(k == w.size(1), "small-batch product: pieces do not add up to the weight's width");
    sg.npiece = (int)pieces.size();
    sg.w = w.data_ptr(); sg.ldw = w.stride(0);
    sg.bias = nullptr;
    if (bias.has_value()) { TORCH_CHECK(bias->numel() == w.size(0), "small-batch product: bias length"); sg.bias = fptr(*bias); }
    sg.y = y.data_ptr(); sg.ldy = y.stride(0);
    sg.N = (int)w.size(0); sg.K = k; sg.out_fp32 = y.scalar_type() == torch::kFloat32 ? 1 : 0;
  }
}

void skinny_multi(SkinnySegs segs, bool weights_static) {
  LoomSkinnyArgs a;
  fill_skinny_args(segs, weights_static, a);
  const c10::cuda::CUDAGuard guard(std::get<3>(segs[0]).device());
  int rc = loom_skinny_multi(&a, cur_stream());
  TORCH_CHECK(rc == 0, "loom_skinny_multi failed: ", rc);
}

void decode_gemm(SkinnySegs segs, bool weights_static, torch::Tensor status) {
  LoomSkinnyArgs a;
  fill_skinny_args(segs, weights_static, a);
  const c10::cuda::CUDAGuard guard(std::get<3>(segs[0]).device());
  TORCH_CHECK(status.is_cuda() && status.scalar_type() == torch::kInt32, "status word: int32 CUDA tensor");
  int rc = loom_decode_gemm(&a, status.data_ptr<int>(), cur_stream());
  TORCH_CHECK(rc == 0, "loom_decode_gemm failed: ", rc);
}

void decode_step_flags(torch::Tensor pos, torch::Tensor tok, torch::Tensor pending, torch::Tensor have_carry, torch::Tensor fire,
                       torch::Tensor reset, torch::Tensor row_reset, torch::Tensor seed_valid, int64_t window, int64_t seq_len,
                       bool hard_enabled, int64_t carry_token, bool temporal) {
  const c10::cuda::CUDAGuard guard(pos.device());
  const int64_t B = tok.numel();
  TORCH_CHECK(pos.scalar_type() == torch::kInt64 && tok.scalar_type() == torch::kInt64 && tok.is_contiguous(), "decode_step_flags: int64 position and tokens");
  for (const torch::Tensor* t : {&pending, &fire, &reset, &row_reset, &seed_valid})
    TORCH_CHECK(t->element_size() == 1 && t->numel() == B && t->is_contiguous(), "decode_step_flags: [B] byte flags");
  TORCH_CHECK(have_carry.element_size() == 1 && have_carry.numel() == 1, "decode_step_flags: have_carry");
  int rc = loom_decode_step_flags((const long long*)pos.data_ptr<int64_t>(), (const long long*)tok.data_ptr<int64_t>(), pending.data_ptr(),
                                  have_carry.data_ptr(), fire.data_ptr(), reset.data_ptr(), row_reset.data_ptr(), seed_valid.data_ptr(),
                                  (int)B, (long long)window, (long long)seq_len, hard_enabled ? 1 : 0, (long long)carry_token,
                                  temporal ? 1 : 0, cur_stream());
  TORCH_CHECK(rc == 0, "loom_decode_step_flags failed: ", rc);
}

void decode_ca_append(torch::Tensor newk, torch::Tensor newv, torch::Tensor fire, torch::Tensor ca_k, torch::Tensor ca_v,
                      torch::Tensor ca_valid, torch::Tensor ca_len, torch::Tensor allowed, torch::Tensor any_out, torch::Tensor pending,
                      torch::Tensor have_carry) {
  const c10::cuda::CUDAGuard guard(newk.device());
  TORCH_CHECK(ca_k.dim() == 3 && ca_k.is_contiguous() && ca_v.is_contiguous() && ca_v.sizes() == ca_k.sizes() &&
              ca_k.scalar_type() == torch::kBFloat16 && ca_v.scalar_type() == torch::kBFloat16, "decode_ca_append: bf16 [B, cap, N] stores");
  const int64_t B = ca_k.size(0), cap = ca_k.size(1), N = ca_k.size(2);
  TORCH_CHECK(newk.dim() == 2 && newk.size(0) == B && newk.size(1) == N && newk.stride(1) == 1 && newv.sizes() == newk.sizes() &&
              newv.stride(1) == 1 && newv.stride(0) == newk.stride(0) && newk.scalar_type() == torch::kBFloat16 &&
              newv.scalar_type() == torch::kBFloat16, "decode_ca_append: new rows");
  TORCH_CHECK(ca_valid.element_size() == 1 && ca_valid.numel() == B * cap && ca_valid.is_contiguous() && allowed.element_size() == 1 &&
              allowed.numel() == B * cap && allowed.is_contiguous(), "decode_ca_append: [B, cap] byte masks");
  TORCH_CHECK(fire.element_size() == 1 && fire.numel() == B && pending.element_size() == 1 && pending.numel() == B &&
              have_carry.element_size() == 1 && have_carry.numel() == 1, "decode_ca_append: flags");
  TORCH_CHECK(ca_len.scalar_type() == torch::kInt64 && any_out.scalar_type() == torch::kInt64, "decode_ca_append: int64 counters");
  int rc = loom_decode_ca_append(newk.data_ptr(), newv.data_ptr(), newk.stride(0), fire.data_ptr(), ca_k.data_ptr(), ca_v.data_ptr(),
                                 ca_valid.data_ptr(), (const long long*)ca_len.data_ptr<int64_t>(), allowed.data_ptr(),
                                 (long long*)any_out.data_ptr<int64_t>(), pending.data_ptr(), have_carry.data_ptr(), (int)B, (int)cap,
                                 (int)N, cur_stream());
  TORCH_CHECK(rc == 0, "loom_decode_ca_append failed: ", rc);
}

void decode_rope_store(torch::Tensor qkv, torch::Tensor cos_tab, torch::Tensor sin_tab, torch::Tensor pos, torch::Tensor q_out,
                       torch::Tensor kc, torch::Tensor vc, int64_t QH, int64_t KVH, int64_t HD) {
  const c10::cuda::CUDAGuard guard(qkv.device());
  TORCH_CHECK(qkv.dim() == 2 && qkv.stride(1) == 1 && qkv.scalar_type() == torch::kBFloat16, "decode_rope_store: qkv rows");
  TORCH_CHECK(qkv.size(1) == (QH + 2 * KVH) * HD, "decode_rope_store: qkv width");
  TORCH_CHECK(kc.is_contiguous() && vc.is_contiguous() && kc.dim() == 4 && kc.size(2) == KVH && kc.size(3) == HD,
              "decode_rope_store: caches [B, S, KVH, HD]");
  TORCH_CHECK(q_out.stride(-1) == 1 && q_out.scalar_type() == torch::kBFloat16 && pos.scalar_type() == torch::kInt64,
              "decode_rope_store: q_out rows, int64 position");
  TORCH_CHECK(cos_tab.dim() == 2 && cos_tab.size(1) == HD && sin_tab.sizes() == cos_tab.sizes(), "decode_rope_store: tables");
  int rc = loom_decode_rope_store(qkv.data_ptr(), qkv.stride(0), fptr(cos_tab), fptr(sin_tab),
                                  (const long long*)pos.data_ptr<int64_t>(), q_out.data_ptr(), q_out.stride(0), kc.data_ptr(),
                                  vc.data_ptr(), (int)qkv.size(0), (int)kc.size(1), (int)cos_tab.size(0), (int)QH, (int)KVH,
                                  (int)HD, cur_stream());
  TORCH_CHECK(rc == 0, "loom_decode_rope_store failed: ", rc);
}

void slot_pool(bool bwd, torch::Tensor keys, torch::Tensor w9, torch::Tensor pooled, torch::Tensor stats,
               c10::optional<torch::Tensor> dpooled, c10::optional<torch::Tensor> dkeys, c10::optional<torch::Tensor> dw9_part,
               int64_t BK, int64_t H) {
  const c10::cuda::CUDAGuard guard(keys.device());
  int rc;
  if (!bwd) rc = loom_slot_pool_fwd(fptr(keys), fptr(w9), fptr(pooled), fptr(stats), (int)BK, (int)H, cur_stream());
  else rc = loom_slot_pool_bwd(fptr(keys), fptr(w9), fptr(pooled), fptr(stats), fptr(*dpooled), fptr(*dkeys), fptr(*dw9_part),
                               (int)BK, (int)H, cur_stream());
  TORCH_CHECK(rc == 0, "loom_slot_pool failed: ", rc);
}

void cross_attn(bool bwd, torch::Tensor q, torch::Tensor k, torch::Tensor v, torch::Tensor allowed_or_dout, torch::Tensor out_or_dq,
                torch::Tensor prob, c10::optional<torch::Tensor> ds, c10::optional<torch::Tensor> dk,
                c10::optional<torch::Tensor> dv, int64_t B, int64_t T, int64_t Kn, int64_t N, double scale) {
  const c10::cuda::CUDAGuard guard(q.device());
  TORCH_CHECK(q.is_contiguous() && k.is_contiguous() && v.is_contiguous() && allowed_or_dout.is_contiguous(), "cross_attn: contiguous");
  int rc;
  if (!bwd) rc = loom_cross_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), (const uint8_t*)allowed_or_dout.data_ptr(),
                                     out_or_dq.data_ptr(), fptr(prob), (int)B, (int)T, (int)Kn, (int)N, (float)scale, cur_stream());
  else rc = loom_cross_attn_bwd(allowed_or_dout.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), fptr(prob), fptr(*ds),
                                out_or_dq.data_ptr(), dk->data_ptr(), dv->data_ptr(), (int)B, (int)T, (int)Kn, (int)N,
                                (float)scale, cur_stream());
  TORCH_CHECK(rc == 0, "loom_cross_attn failed: ", rc);
}

void fixed_rms(bool bwd, c10::optional<torch::Tensor> dy, torch::Tensor x, torch::Tensor out, int64_t rows, int64_t heads,
               int64_t HD, int64_t ld, double target, double eps) {
  const c10::cuda::CUDAGuard guard(x.device());
  int rc = loom_fixed_rms(bwd, dy.has_value() ? dy->data_ptr() : nullptr, x.data_ptr(), out.data_ptr(), rows, (int)heads,
                          (int)HD, ld, (float)target, (float)eps, cur_stream());
  TORCH_CHECK(rc == 0, "loom_fixed_rms failed: ", rc);
}

void rms_norm(bool bwd, c10::optional<torch::Tensor> dy, torch::Tensor x, torch::Tensor w, torch::Tensor out,
              c10::optional<torch::Tensor> gw_part, int64_t M, int64_t N, double eps) {
  const c10::cuda::CUDAGuard guard(x.device());
  int rc;
  if (!bwd) rc = loom_rms_norm_fwd(x.data_ptr(), fptr(w), out.data_ptr(), (int)M, (int)N, (float)eps, cur_stream());
  else rc = loom_rms_norm_bwd(dy->data_ptr(), x.data_ptr(), fptr(w), out.data_ptr(), fptr(*gw_part), (int)gw_part->size(0),
                              (int)M, (int)N, (float)eps, cur_stream());
  TORCH_CHECK(rc == 0, "loom_rms_norm failed: ", rc);
}

void dread_stage(torch::Tensor a, c10::optional<torch::Tensor> b, torch::Tensor mo, torch::Tensor dm, torch::Tensor dd,
                 torch::Tensor lse_in, torch::Tensor lse_out, int64_t MQ, int64_t HD) {
  const c10::cuda::CUDAGuard guard(a.device());
  TORCH_CHECK(a.is_contiguous() && mo.is_contiguous() && dm.is_contiguous() && (!b.has_value() || b->is_contiguous()) &&
                  lse_in.is_contiguous() && lse_out.is_contiguous() && lse_in.numel() == MQ && lse_out.numel() == MQ,
              "dread_stage: contiguous operands");
  int rc = loom_dread_stage(a.data_ptr(), b.has_value() ? b->data_ptr() : nullptr, mo.data_ptr(), dm.data_ptr(),
                            dd.data_ptr<float>(), lse_in.data_ptr<float>(), lse_out.data_ptr<float>(), MQ, (int)HD,
                            cur_stream());
  TORCH_CHECK(rc == 0, "loom_dread_stage failed: ", rc);
}

void dread_slot_bwd(torch::Tensor q_all, torch::Tensor hk, torch::Tensor hv, torch::Tensor dm_all, torch::Tensor lse_all,
                    torch::Tensor dd_all, torch::Tensor dk, torch::Tensor dv, torch::Tensor gq_all, int64_t sub0, int64_t S,
                    int64_t M, int64_t QH, int64_t HD) {
  // hk, hv, dk, dv: [M, QH, HD] views whose rows may be strided (K and V sharing [K | V] rows)
  const c10::cuda::CUDAGuard guard(hk.device());
  auto rows_ok = [&](const torch::Tensor& t) {
    return t.dim() == 3 && t.size(0) == M && t.stride(2) == 1 && t.stride(1) == HD && t.stride(0) >= QH * HD;
  };
  TORCH_CHECK(rows_ok(hk) && rows_ok(hv) && rows_ok(dk) && rows_ok(dv) && hk.stride(0) == hv.stride(0) &&
                  dk.stride(0) == dv.stride(0) && dm_all.is_contiguous(),
              "dread_slot_bwd: operands must be [M,QH,HD] with unit inner strides");
  int rc = loom_dread_slot_bwd(q_all.data_ptr<float>(), hk.data_ptr(), hv.data_ptr(), dm_all.data_ptr(),
                               lse_all.data_ptr<float>(), dd_all.data_ptr<float>(), dk.data_ptr(), dv.data_ptr(),
                               gq_all.data_ptr<float>(), (int)sub0, (int)S, (int)M, (int)QH, (int)HD, hk.stride(0),
                               dk.stride(0), cur_stream());
  TORCH_CHECK(rc == 0, "loom_dread_slot_bwd failed: ", rc);
}

void dread(bool bwd, torch::Tensor q, torch::Tensor hk, torch::Tensor hv, torch::Tensor out, torch::Tensor lse, OptT dm,
           OptT dhk, OptT dhv, OptT gq, int64_t n, int64_t MQ, int64_t QH, int64_t HD) {
  // hk, hv: [slots, M, QH, HD] with unit strides inside a row; slot and row strides are taken from hk
  const c10::cuda::CUDAGuard guard(hk.device());
  TORCH_CHECK(hk.dim() == 4 && hv.dim() == 4 && hk.stride(3) == 1 && hk.stride(2) == HD && hv.stride(3) == 1 &&
                  hv.stride(2) == HD && hk.stride(0) == hv.stride(0) && hk.stride(1) == hv.stride(1),
              "dread: history must be [slots,M,QH,HD] with unit inner strides and matching K/V strides");
  int rc = loom_dread(bwd, fptr(q), hk.data_ptr(), hv.data_ptr(), out.data_ptr(), fptr(lse), cp(dm), mf(dhk), mf(dhv),
                      mf(gq), (int)n, MQ, (int)QH, (int)HD, hk.stride(0), hk.stride(1), cur_stream());
  TORCH_CHECK(rc == 0, "loom_dread failed: ", rc);
}

void add_ln_fwd(torch::Tensor a, torch::Tensor b, torch::Tensor w, torch::Tensor bias, torch::Tensor y, torch::Tensor x,
                torch::Tensor mean, torch::Tensor rstd, int64_t M, int64_t N, double eps, double cap) {
  const c10::cuda::CUDAGuard guard(a.device());
  int rc = loom_add_ln_fwd(a.data_ptr(), b.data_ptr(), fptr(w), fptr(bias), y.data_ptr(), x.data_ptr(), fptr(mean),
                           fptr(rstd), (int)M, (int)N, (float)eps, (float)cap, cur_stream());
  TORCH_CHECK(rc == 0, "loom_add_ln_fwd failed: ", rc);
}

void cap_bwd(torch::Tensor dy, torch::Tensor a, torch::Tensor da, int64_t M, int64_t N, double cap) {
  const c10::cuda::CUDAGuard guard(a.device());
  int rc = loom_cap_bwd(dy.data_ptr(), a.data_ptr(), da.data_ptr(), (int)M, (int)N, (float)cap, cur_stream());
  TORCH_CHECK(rc == 0, "loom_cap_bwd failed: ", rc);
}

void add_ln_bwd(torch::Tensor dy, torch::Tensor x, torch::Tensor mean, torch::Tensor rstd, torch::Tensor w,
                torch::Tensor dx, torch::Tensor gw, torch::Tensor gb, int64_t M, int64_t N) {
  const c10::cuda::CUDAGuard guard(dy.device());
  int rc = loom_add_ln_bwd(dy.data_ptr(), x.data_ptr(), fptr(mean), fptr(rstd), fptr(w), dx.data_ptr(), fptr(gw),
                           fptr(gb), (int)M, (int)N, cur_stream());
  TORCH_CHECK(rc == 0, "loom_add_ln_bwd failed: ", rc);
}

void anchor_ema(torch::Tensor bsq, double inv_n, double decay, torch::Tensor anchor, torch::Tensor snap) {
  TORCH_CHECK(bsq.is_cuda() && anchor.is_cuda() && snap.is_cuda(), "anchor_ema: CUDA tensors expected");
  TORCH_CHECK(bsq.scalar_type() == torch::kFloat32 && anchor.scalar_type() == torch::kFloat32 &&
              snap.scalar_type() == torch::kFloat32, "anchor_ema: fp32 tensors expected");
  int rc = loom_anchor_ema(fptr(bsq), (float)inv_n, (float)decay, fptr(anchor), fptr(snap), cur_stream());
  TORCH_CHECK(rc == 0, "loom_anchor_ema failed: ", rc);
}

void colsum(torch::Tensor dy, torch::Tensor gb, int64_t M, int64_t N) {
  const c10::cuda::CUDAGuard guard(dy.device());
  int rc = loom_colsum(dy.data_ptr(), fptr(gb), (int)M, (int)N, dy.stride(0), cur_stream());
  TORCH_CHECK(rc == 0, "loom_colsum failed: ", rc);
}

void ce(torch::Tensor logits, torch::Tensor targets, torch::Tensor nll, torch::Tensor scale, int64_t ignore_index,
        bool write_grad) {
  const c10::cuda::CUDAGuard guard(logits.device());
  TORCH_CHECK(logits.is_contiguous() && targets.scalar_type() == torch::kInt64 && targets.is_contiguous(), "bad CE inputs");
  int rc = loom_ce(logits.data_ptr(), (const long long*)targets.data_ptr(), fptr(nll), fptr(scale), logits.size(0),
                   (int)logits.size(1), ignore_index, write_grad, cur_stream());
  TORCH_CHECK(rc == 0, "loom_ce failed: ", rc);
}

void temporal_fwd(torch::Tensor depth, torch::Tensor reset, OptT state_in, OptT fired, double beta, torch::Tensor state_out,
                  torch::Tensor raw_out, OptT ckpt, int64_t B, int64_t Tc, int64_t H) {
  const c10::cuda::CUDAGuard guard(depth.device());
  int rc = loom_temporal_fwd(depth.data_ptr(), (const uint8_t*)reset.data_ptr(), cf(state_in), cu8(fired), (float)beta,
                             fptr(state_out), fptr(raw_out), mf(ckpt), (int)B, (int)Tc, (int)H, cur_stream());
  TORCH_CHECK(rc == 0, "loom_temporal_fwd failed: ", rc);
}

void temporal_bwd(torch::Tensor depth, torch::Tensor reset, OptT state_in, OptT fired, double beta, torch::Tensor raw,
                  OptT ckpt, torch::Tensor dstate, torch::Tensor ddepth, OptT dstate_in, int64_t B, int64_t Tc, int64_t H) {
  const c10::cuda::CUDAGuard guard(depth.device());
  int rc = loom_temporal_bwd(depth.data_ptr(), (const uint8_t*)reset.data_ptr(), cf(state_in), cu8(fired), (float)beta,
                             fptr(raw), cf(ckpt), fptr(dstate), ddepth.data_ptr(), mf(dstate_in), (int)B, (int)Tc, (int)H,
                             cur_stream());
  TORCH_CHECK(rc == 0, "loom_temporal_bwd failed: ", rc);
}

void attn(bool bwd, torch::Tensor qkc, torch::Tensor kcache, torch::Tensor vcache, torch::Tensor lse, OptT seg,
          OptT dqkc, OptT dq_attn, OptT dk_heads, OptT dv_heads, int64_t B, int64_t QH, int64_t KVH, int64_t HD,
          int64_t Tc, int64_t T, int64_t s, int64_t e, torch::Tensor status) {
  const c10::cuda::CUDAGuard guard(qkc.device());
  TORCH_CHECK(qkc.is_contiguous() && kcache.is_contiguous() && vcache.is_contiguous(), "attention operands must be contiguous");
  LoomAttn a{};
  a.qkc = qkc.data_ptr(); a.kcache = kcache.data_ptr(); a.vcache = vcache.data_ptr(); a.lse = fptr(lse);
  a.seg = seg.has_value() ? (const int*)seg->data_ptr() : nullptr;
  a.dqkc = cp(dqkc); a.dq_attn = mp(dq_attn); a.dk_heads = mf(dk_heads); a.dv_heads = mf(dv_heads);
  a.B = (int)B; a.QH = (int)QH; a.KVH = (int)KVH; a.HD = (int)HD; a.Tc = (int)Tc; a.T = (int)T; a.s = (int)s; a.e = (int)e;
  a.status = status.data_ptr<int>();
  int rc = bwd ? loom_attn_bwd(&a, cur_stream()) : loom_attn_fwd(&a, cur_stream());
  TORCH_CHECK(rc == 0, "loom_attn failed: ", rc);
}

void tp_barrier(std::vector<int64_t> flags_peer, int64_t rank, int64_t epoch, torch::Tensor status, int64_t code) {
  const c10::cuda::CUDAGuard guard(status.device());
  int* ptrs[8];
  TORCH_CHECK(flags_peer.size() <= 8, "up to 8 ranks");
  for (size_t i = 0; i < flags_peer.size(); ++i) ptrs[i] = reinterpret_cast<int*>(flags_peer[i]);
  int rc = loom_tp_barrier(ptrs, (int)flags_peer.size(), (int)rank, (int)epoch, status.data_ptr<int>(), (int)code, cur_stream());
  TORCH_CHECK(rc == 0, "loom_tp_barrier failed: ", rc);
}

void p2p_grad_step(int64_t W, int64_t rank, int64_t nblk, std::vector<int64_t> grads, std::vector<int64_t> params,
                   std::vector<int64_t> shadow, std::vector<int64_t> sync, int64_t mc_grads, torch::Tensor m,
                   torch::Tensor v, torch::Tensor lr_mult, torch::Tensor wd, torch::Tensor active, torch::Tensor hyper,
                   torch::Tensor stats, torch::Tensor sumsq, double max_norm, torch::Tensor status,
                   c10::optional<torch::Tensor> owner_blk, c10::optional<torch::Tensor> slot_blk,
                   c10::optional<torch::Tensor> replicate_blk, c10::optional<torch::Tensor> anchors, bool anchor_rank0) {
  const c10::cuda::CUDAGuard guard(m.device());
  TORCH_CHECK((int64_t)grads.size() == W && (int64_t)params.size() == W && (int64_t)shadow.size() == W &&
              (int64_t)sync.size() == W && W <= 8, "peer pointer lists must have one entry per rank (<= 8)");
  LoomP2P a{};
  a.W = (int)W; a.rank = (int)rank; a.nblk = nblk;
  for (int i = 0; i < W; ++i) {
    a.grads[i] = reinterpret_cast<float*>(grads[i]); a.params[i] = reinterpret_cast<float*>(params[i]);
    a.shadow[i] = reinterpret_cast<void*>(shadow[i]); a.sync[i] = reinterpret_cast<int*>(sync[i]);
  }
  a.mc_grads = reinterpret_cast<float*>(mc_grads);
  a.m = fptr(m); a.v = fptr(v); a.lr_mult = fptr(lr_mult); a.wd_blk = fptr(wd); a.active = fptr(active);
  a.hyper = fptr(hyper); a.stats = fptr(stats); a.sumsq_local = fptr(sumsq); a.max_norm = (float)max_norm;
  a.status = status.data_ptr<int>();
  if (owner_blk.has_value()) {
    TORCH_CHECK(slot_blk.has_value() && replicate_blk.has_value(), "owner, slot and replicate maps come together");
    TORCH_CHECK(owner_blk->scalar_type() == torch::kUInt8 && replicate_blk->scalar_type() == torch::kUInt8 &&
                slot_blk->scalar_type() == torch::kInt32 && owner_blk->numel() == nblk, "block maps: uint8/int32, one per block");
    a.owner_blk = owner_blk->data_ptr<uint8_t>(); a.slot_blk = slot_blk->data_ptr<int>();
    a.replicate_blk = replicate_blk->data_ptr<uint8_t>();
  }
  if (anchors.has_value()) { a.anchors = fptr(*anchors); a.n_anchor = (int)anchors->numel(); a.anchor_rank0 = anchor_rank0 ? 1 : 0; }
  int rc = loom_p2p_grad_step(&a, cur_stream());
  TORCH_CHECK(rc == 0, "loom_p2p_grad_step failed: ", rc);
}

void p2p_grad_step_atom(int64_t W, int64_t rank, int64_t nblk, std::vector<int64_t> grads, std::vector<int64_t> params,
                        std::vector<int64_t> shadow, std::vector<int64_t> sync, torch::Tensor m, torch::Tensor v,
                        torch::Tensor lr_mult, torch::Tensor wd, torch::Tensor hyper, torch::Tensor stats, torch::Tensor sumsq,
                        double max_norm, torch::Tensor status, torch::Tensor cnt_blk, torch::Tensor gprev, torch::Tensor pnode,
                        torch::Tensor trust, torch::Tensor atom_out, c10::optional<torch::Tensor> anchors,
                        bool anchor_rank0) {
  const c10::cuda::CUDAGuard guard(m.device());
  TORCH_CHECK((int64_t)grads.size() == W && (int64_t)params.size() == W && (int64_t)shadow.size() == W &&
              (int64_t)sync.size() == W && W <= 8, "peer pointer lists must have one entry per rank (<= 8)");
  LoomP2P a{};
  a.W = (int)W; a.rank = (int)rank; a.nblk = nblk;
  for (int i = 0; i < W; ++i) {
    a.grads[i] = reinterpret_cast<float*>(grads[i]); a.params[i] = reinterpret_cast<float*>(params[i]);
    a.shadow[i] = reinterpret_cast<void*>(shadow[i]); a.sync[i] = reinterpret_cast<int*>(sync[i]);
  }
  a.m = fptr(m); a.v = fptr(v); a.lr_mult = fptr(lr_mult); a.wd_blk = fptr(wd); a.hyper = fptr(hyper);
  a.stats = fptr(stats); a.sumsq_local = fptr(sumsq); a.max_norm = (float)max_norm; a.status = status.data_ptr<int>();
  if (anchors.has_value()) { a.anchors = fptr(*anchors); a.n_anchor = (int)anchors->numel(); a.anchor_rank0 = anchor_rank0 ? 1 : 0; }
  int rc = loom_p2p_grad_step_atom(&a, fptr(cnt_blk), fptr(gprev), fptr(pnode), fptr(trust), fptr(atom_out), cur_stream());
  TORCH_CHECK(rc == 0, "loom_p2p_grad_step_atom failed: ", rc);
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("gemm", &gemm, "segmented-K batched bf16 GEMM (tcgen05 + TMA)");
  m.def("grad_norm", &grad_norm, "global gradient norm, clip coefficient and finite flag");
  m.def("gemm_qkv_rope", &gemm_qkv_rope, "[Q | K | V] projection whose epilogue applies RoPE and writes the attention operand and the caches");
  m.def("sector_fold", &sector_fold, "[M, QH, 3, HD] -> [M, 3, QH, HD] copy, 16 bytes per thread");
  m.def("status_gate", &status_gate, "finite flag &= status word clear; count skipped updates");
  m.def("adamw_flat", &adamw_flat, "AdamW over the flat parameter buffer");
  m.def("atom_flat", &atom_flat, "ATOM over the flat parameter buffer");
  m.def("cast_shadow", &cast_shadow, "fp32 -> bf16 parameter shadow");
  m.def("ffn_core", &ffn_core, "fused Paraplex core + Tria step (forward / backward)");
  m.def("rope_store", &rope_store, "RoPE + KV cache write");
  m.def("rope_bwd", &rope_bwd, "inverse RoPE of the q/k/v gradients");
  m.def("dread", &dread, "depth-attention read (forward / backward)");
  m.def("decode_attn", &decode_attn, "KV-cache attention for one new token per sequence, dual context, split over positions");
  m.def("skinny_linear", &skinny_linear, "y = x W^T (+ bias) for up to 16 rows: weights streamed once, output may be a strided view");
  m.def("skinny_multi", &skinny_multi, "several small-batch products (own inputs, weights, outputs) in one launch");
  m.def("decode_gemm", &decode_gemm, "several 17..128-row products in one launch: weight rows as the M side of tcgen05.mma, batch as N");
  m.def("decode_step_flags", &decode_step_flags, "fire / reset / first-position / seed flags of one decode step");
  m.def("decode_ca_append", &decode_ca_append, "boundary-key append and visibility mask of one decode step");
  m.def("decode_rope_store", &decode_rope_store, "RoPE of the new token's Q / K at the device-side position + KV cache append");
  m.def("slot_pool", &slot_pool, "softmax pooling of boundary carriers over neurons (forward / backward)");
  m.def("cross_attn", &cross_attn, "token rows attending to the boundary keys (forward / backward)");
  m.def("fixed_rms", &fixed_rms, "x * target / rms(x) over head_dim (forward / backward)");
  m.def("rms_norm", &rms_norm, "weighted RMSNorm over the model width (forward / backward)");
  m.def("dread_stage", &dread_stage, "store a sublayer's read gradient (bf16) and its <dm, m> row scalars");
  m.def("dread_slot_bwd", &dread_slot_bwd, "gradient of one history slot over every sublayer that read it");
  m.def("add_ln_fwd", &add_ln_fwd, "residual add + LayerNorm");
  m.def("cap_bwd", &cap_bwd, "backward of the per-row RMS cap");
  m.def("add_ln_bwd", &add_ln_bwd, "residual add + LayerNorm backward");
  m.def("anchor_ema", &anchor_ema, "running radius of the imaginary pre-activation (EMA) with a snapshot");
  m.def("colsum", &colsum, "column sums into an fp32 accumulator");
  m.def("ce", &ce, "cross-entropy over bf16 logits with in-place gradient");
  m.def("temporal_fwd", &temporal_fwd, "temporal carry endpoint + PolARM");
  m.def("p2p_grad_step_atom", &p2p_grad_step_atom, "fused gradient reduce-scatter + ATOM on the shard + parameter push over peer memory");
  m.def("tp_barrier", &tp_barrier, "bounded cross-rank barrier on peer-mapped flag words");
  m.def("p2p_grad_step", &p2p_grad_step, "fused gradient reduce-scatter + AdamW + parameter all-gather over peer memory");
  m.def("attn", &attn, "dual-context causal GQA attention (forward / backward)");
  m.def("temporal_bwd", &temporal_bwd, "temporal carry endpoint backward");
}
