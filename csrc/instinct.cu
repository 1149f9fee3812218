// Instinct optimizer step on the device: momentum, homeostasis normalisation (row -> column -> row, or the
// transposed order for experts), weight decay, step scaled by the situation card's gain and stake, fp32 master copy
// or counter-hash stochastic rounding for bf16 weights.  No scalar ever visits the host: gain, stake and the learning
// rate are read from device memory.
//
// A weight is viewed as (E, R, C) with C contiguous.  Three generic kernels cover every kind:
//   stat_rows : rowsq[e,r] = sum_c (mf * colscale[e,c])^2          (+ sum|g| per row for word tables)
//   stat_cols : colsq[e,c] += sum_r (mf * colscaleA[e,c] * rowscale[e,r])^2
//   apply     : upd = mf * s1 * s2 * s3 -> weight / momentum update
// where mf = beta*m + (1-beta)*g is recomputed on the fly (momentum is written once, in `apply`) and every scale is
// 1 / (sqrt(sumsq / count) + 1e-8) formed by the consumer from the raw sums.
//   hs   (2-D)  : rows -> cols(rows) -> rows(rows, cols) -> apply
//   hs3  (E,K,N): cols -> rows(cols) -> cols(cols, rows) -> apply
//   vocab       : rows (+|g|) -> apply, rows without gradient stay put, no weight decay
//   row / row3 / tensor : one stat -> apply
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "common.cuh"
#include "instinct_core.cuh"

namespace mb {

static inline cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream(); }

enum { KIND_TENSOR = 0, KIND_ROW = 1, KIND_ROW3 = 2, KIND_VOCAB = 3, KIND_HS = 4, KIND_HS3 = 5 };

// Returns the number of kernels launched.
int64_t instinct_step(torch::Tensor p, torch::Tensor grad, torch::Tensor m, c10::optional<torch::Tensor> w_,
                      c10::optional<torch::Tensor> cs_, torch::Tensor gvec, int64_t index, torch::Tensor stake,
                      torch::Tensor lr_t, c10::optional<torch::Tensor> rel_, double beta, double wd, int64_t kind,
                      bool sr, torch::Tensor seed_t, c10::optional<torch::Tensor> frozen_) {
  const c10::cuda::CUDAGuard guard(p.device());
  TORCH_CHECK(p.is_contiguous() && grad.is_contiguous() && m.is_contiguous(), "instinct_step: contiguous tensors");
  TORCH_CHECK(grad.numel() == p.numel() && m.numel() == p.numel(), "instinct_step: shape mismatch");
  TORCH_CHECK(!(cs_.has_value() && cs_->defined()), "instinct_step: lagged homeostasis runs on the PyTorch path");
  InstinctArgs a{};
  a.g_scale = 1.f;
  a.p = p.data_ptr(); a.g = grad.data_ptr(); a.m = m.data_ptr();
  a.p_bf16 = p.scalar_type() == torch::kBFloat16;
  a.g_bf16 = grad.scalar_type() == torch::kBFloat16;
  a.m_bf16 = m.scalar_type() == torch::kBFloat16;
  TORCH_CHECK(a.p_bf16 || p.scalar_type() == torch::kFloat32, "instinct_step: weight dtype");
  TORCH_CHECK(a.g_bf16 || grad.scalar_type() == torch::kFloat32, "instinct_step: grad dtype");
  TORCH_CHECK(a.m_bf16 || m.scalar_type() == torch::kFloat32, "instinct_step: momentum dtype");
  a.w = (w_.has_value() && w_->defined()) ? w_->data_ptr<float>() : nullptr;
  a.gain = gvec.data_ptr<float>() + index;
  a.stake = stake.data_ptr<float>();
  a.lr = lr_t.data_ptr<float>();
  a.beta = (float)beta; a.wd = (float)wd;
  a.sr = sr ? 1 : 0;
  a.seed = reinterpret_cast<const long long*>(seed_t.data_ptr<int64_t>());
  a.salt = (unsigned)index * 0x85EBCA6Bu;
  a.frozen = (frozen_.has_value() && frozen_->defined()) ? frozen_->data_ptr<bool>() : nullptr;
  const long long numel = p.numel();
  long long E = 1, R = 1, C = numel;
  if (kind == KIND_HS || kind == KIND_VOCAB) { TORCH_CHECK(p.dim() == 2); R = p.size(0); C = p.size(1); }
  else if (kind == KIND_HS3 || kind == KIND_ROW3) { TORCH_CHECK(p.dim() == 3); E = p.size(0); R = p.size(1); C = p.size(2); }
  else if (kind == KIND_ROW) { TORCH_CHECK(p.dim() >= 2); R = p.size(0); C = numel / R; }
  a.E = E; a.R = R; a.C = C;
  if (a.frozen) a.frozen_stride = numel / frozen_->numel();
  float* rel = (rel_.has_value() && rel_->defined()) ? rel_->data_ptr<float>() + index : nullptr;
  auto scratch = torch::zeros({instinct_scratch_floats(E, R, C)}, p.options().dtype(torch::kFloat32));
  return instinct_launch(a, (int)kind, scratch.data_ptr<float>(), rel, cur_stream());
}

}  // namespace mb
