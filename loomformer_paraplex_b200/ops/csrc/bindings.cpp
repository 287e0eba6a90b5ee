// PyTorch <-> kernel glue: unwraps tensors into the plain C launchers of loom_c_api.h.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
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
          std::vector<int64_t> b_k0, torch::Tensor b, bool a_mn, bool b_mn, torch::Tensor c,
          c10::optional<torch::Tensor> bias, int64_t M, int64_t N, int64_t heads, bool accumulate, int64_t bn,
          bool swap_mn, torch::Tensor status) {
  TORCH_CHECK(a_list.size() >= 1 && a_list.size() <= 5, "1..5 K segments");
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
  g.b = operand(b, ok);
  TORCH_CHECK(ok, "bad B operand");
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
  g.bn = (int)bn; g.swap_mn_strides = swap_mn;
  g.status = status.data_ptr<int>();
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

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("gemm", &gemm, "segmented-K batched bf16 GEMM (tcgen05 + TMA)");
  m.def("grad_norm", &grad_norm, "global gradient norm, clip coefficient and finite flag");
  m.def("adamw_flat", &adamw_flat, "AdamW over the flat parameter buffer");
  m.def("atom_flat", &atom_flat, "ATOM over the flat parameter buffer");
  m.def("cast_shadow", &cast_shadow, "fp32 -> bf16 parameter shadow");
}
