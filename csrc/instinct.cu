// Instinct optimizer step on the device: momentum, homeostasis normalisation (row -> column -> row, or the
// transposed order for experts), weight decay, step scaled by the situation card's gain and stake, fp32 master copy
// or counter-hash stochastic rounding for bf16 weights.  No scalar ever visits the host: gain, stake and the learning
// rate are read from device memory.
//
// A weight is viewed as (E, R, C) with C contiguous; the kernels and their launch order are in instinct_core.cuh:
//   hs   (2-D)  : rows -> cols(rows) -> apply with the last row norm fused (row staged in shared memory)
//   hs3  (E,K,N): cols -> rows(cols) -> cols(cols, rows) -> apply
//   vocab       : rows (+|g|) -> apply, rows without gradient stay put, no weight decay
//   row / row3 / tensor : one stat -> apply
//   lagged hs   : one pass (column norm of the previous step); lagged hs3: the exact sequence with the row norm
//                 taken from the previous step
// Scratch statistics live in a caller-owned arena (zeroed here with one cudaMemsetAsync), not in memory allocated per
// call.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "common.cuh"
#include "instinct_core.cuh"

namespace mb {

static inline cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream(); }

enum { KIND_TENSOR = 0, KIND_ROW = 1, KIND_ROW3 = 2, KIND_VOCAB = 3, KIND_HS = 4, KIND_HS3 = 5 };

// Returns the number of kernels launched.  `scratch`: fp32 arena of at least instinct_scratch_floats() elements (one is
// allocated when it is missing or too small).  `cs` / `cs_ok`: state of the lagged form (previous step's second-axis
// mean squares, "all positive" flag).  `shadow`: bf16 copy of an fp32 weight, refreshed with the weight.
int64_t instinct_step(torch::Tensor p, torch::Tensor grad, torch::Tensor m, c10::optional<torch::Tensor> w_,
                      c10::optional<torch::Tensor> cs_, torch::Tensor gvec, int64_t index, torch::Tensor stake,
                      torch::Tensor lr_t, c10::optional<torch::Tensor> rel_, double beta, double wd, int64_t kind,
                      bool sr, torch::Tensor seed_t, c10::optional<torch::Tensor> frozen_,
                      c10::optional<torch::Tensor> scratch_, c10::optional<torch::Tensor> cs_ok_,
                      c10::optional<torch::Tensor> shadow_, int64_t phase, int64_t col_rows) {
  const c10::cuda::CUDAGuard guard(p.device());
  TORCH_CHECK(p.is_contiguous() && grad.is_contiguous() && m.is_contiguous(), "instinct_step: contiguous tensors");
  TORCH_CHECK(grad.numel() == p.numel() && m.numel() == p.numel(), "instinct_step: shape mismatch");
  InstinctArgs a{};
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
  if (shadow_.has_value() && shadow_->defined()) {
    TORCH_CHECK(!a.p_bf16 && shadow_->scalar_type() == torch::kBFloat16 && shadow_->is_contiguous() &&
                shadow_->numel() == p.numel(), "instinct_step: shadow is a contiguous bf16 copy of an fp32 weight");
    a.shadow = shadow_->data_ptr();
  }
  const long long numel = p.numel();
  long long E = 1, R = 1, C = numel;
  if (kind == KIND_HS || kind == KIND_VOCAB) { TORCH_CHECK(p.dim() == 2); R = p.size(0); C = p.size(1); }
  else if (kind == KIND_HS3 || kind == KIND_ROW3) { TORCH_CHECK(p.dim() == 3); E = p.size(0); R = p.size(1); C = p.size(2); }
  else if (kind == KIND_ROW) { TORCH_CHECK(p.dim() >= 2); R = p.size(0); C = numel / R; }
  a.E = E; a.R = R; a.C = C;
  if (a.frozen) a.frozen_stride = numel / frozen_->numel();
  float* rel = (rel_.has_value() && rel_->defined()) ? rel_->data_ptr<float>() + index : nullptr;
  float* cs = nullptr;
  int* cs_ok = nullptr;
  if (cs_.has_value() && cs_->defined()) {
    TORCH_CHECK(kind == KIND_HS || kind == KIND_HS3, "instinct_step: the lagged form exists for hs and hs3");
    TORCH_CHECK(cs_->scalar_type() == torch::kFloat32 && cs_->is_contiguous() &&
                cs_->numel() == (kind == KIND_HS ? C : E * R), "instinct_step: cs shape");
    TORCH_CHECK(cs_ok_.has_value() && cs_ok_->defined() && cs_ok_->scalar_type() == torch::kInt32, "instinct_step: cs_ok flag");
    TORCH_CHECK(kind != KIND_HS || 3 * (size_t)C * sizeof(float) <= INSTINCT_SMEM_MAX,
                "instinct_step: lagged hs stages three rows in shared memory; this row is too long");
    cs = cs_->data_ptr<float>();
    cs_ok = cs_ok_->data_ptr<int>();
  }
  const long long need = instinct_scratch_floats(E, R, C);
  torch::Tensor scratch;
  if (scratch_.has_value() && scratch_->defined() && scratch_->numel() >= need) {
    TORCH_CHECK(scratch_->scalar_type() == torch::kFloat32 && scratch_->is_contiguous() &&
                (reinterpret_cast<uintptr_t>(scratch_->data_ptr()) & 15) == 0, "instinct_step: scratch arena");
    scratch = *scratch_;
    if (phase != 2)          // phase 2 continues on the statistics phase 1 left (and the caller summed over the ranks)
      C10_CUDA_CHECK(cudaMemsetAsync(scratch.data_ptr(), 0, sizeof(float) * (size_t)need, cur_stream()));
  } else {
    TORCH_CHECK(phase == 0, "instinct_step: a split step needs the caller's scratch arena");
    scratch = torch::zeros({need}, p.options().dtype(torch::kFloat32));
  }
  const int64_t n = instinct_launch(a, (int)kind, scratch.data_ptr<float>(), rel, cur_stream(), cs, cs_ok, (int)phase, col_rows);
  TORCH_CHECK(n >= 0, "instinct_step: a row of ", C, " columns is too long for this kind on the kernels");
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return n;
}

}  // namespace mb
