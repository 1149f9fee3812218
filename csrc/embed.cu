// Input embedding of the memarch model in one kernel each way:
//   h[n] = emb[x[n]] + sum_k sel[n,k] * emb[cand[n,k]] + phr[pidx[n]]
// (token embedding, the gated embeddings of the tokens the lock finder proposes, the phrase-table vector).  The
// PyTorch statement of this is three table look-ups, a (N, K, d) product, a sum and two adds forward, and three
// sort-based embedding backward passes; here the forward reads the 2 + K rows of a token and writes one, and the
// backward adds the token's gradient row into the 1 + K + 1 table rows with 16-byte vector reductions while it
// forms d sel[n,k] = <dh[n], emb[cand[n,k]]>.
// Reference behaviour: full2.py:1538-1600 (input side of FullLM2.forward).
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "common.cuh"

namespace mb {

static inline cudaStream_t es() { return at::cuda::getCurrentCUDAStream(); }

// one block per token, thread t owns the float4 columns t, t + blockDim, ...
__global__ void embed_sum_fwd_kernel(const float* __restrict__ emb, const long long* __restrict__ x,
                                     const long long* __restrict__ cand, const float* __restrict__ sel, int K,
                                     const float* __restrict__ phr, const long long* __restrict__ pidx,
                                     float* __restrict__ out, long long N, int d, long long V, long long P) {
  for (long long n = blockIdx.x; n < N; n += gridDim.x) {
    const long long xi = x[n];
    const float* r0 = emb + xi * d;
    const float* rp = phr ? phr + pidx[n] * d : nullptr;
    for (int c = threadIdx.x * 4; c < d; c += blockDim.x * 4) {
      float4 acc = *reinterpret_cast<const float4*>(r0 + c);
      for (int k = 0; k < K; ++k) {
        const float s = sel[n * K + k];
        if (s != 0.f) {
          const float4 v = *reinterpret_cast<const float4*>(emb + cand[n * K + k] * d + c);
          acc.x += s * v.x; acc.y += s * v.y; acc.z += s * v.z; acc.w += s * v.w;
        }
      }
      if (rp) { const float4 v = *reinterpret_cast<const float4*>(rp + c); acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w; }
      *reinterpret_cast<float4*>(out + n * d + c) = acc;
    }
  }
}

__device__ __forceinline__ void red_add4(float* addr, float4 v) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

// one block per token; demb / dphr are zero-initialised by the caller and receive vector reductions
__global__ void embed_sum_bwd_kernel(const float* __restrict__ dh, const float* __restrict__ emb,
                                     const long long* __restrict__ x, const long long* __restrict__ cand,
                                     const float* __restrict__ sel, int K, const long long* __restrict__ pidx,
                                     float* __restrict__ demb, float* __restrict__ dphr, float* __restrict__ dsel,
                                     long long N, int d) {
  __shared__ float red[32];
  for (long long n = blockIdx.x; n < N; n += gridDim.x) {
    const float* g = dh + n * d;
    float* e0 = demb + x[n] * d;
    float* ep = dphr ? dphr + pidx[n] * d : nullptr;
    for (int c = threadIdx.x * 4; c < d; c += blockDim.x * 4) {
      const float4 v = *reinterpret_cast<const float4*>(g + c);
      red_add4(e0 + c, v);
      if (ep) red_add4(ep + c, v);
    }
    for (int k = 0; k < K; ++k) {
      const float s = sel[n * K + k];
      const long long ci = cand[n * K + k];
      float dot = 0.f;
      // d sel is wanted wherever the gate could open: the model masks it by (val != 0) itself, so compute it where
      // the candidate is a valid row
      for (int c = threadIdx.x * 4; c < d; c += blockDim.x * 4) {
        const float4 v = *reinterpret_cast<const float4*>(g + c);
        const float4 e = *reinterpret_cast<const float4*>(emb + ci * d + c);
        dot += v.x * e.x + v.y * e.y + v.z * e.z + v.w * e.w;
        if (s != 0.f) red_add4(demb + ci * d + c, make_float4(s * v.x, s * v.y, s * v.z, s * v.w));
      }
      dot = block_sum(dot, red);
      if (threadIdx.x == 0) dsel[n * K + k] = dot;
    }
  }
}

// out[n] = <A[ia[n]], B[ib[n]]> in fp32; tables fp32 or bf16 (same dtype); one warp per n
template <typename T>
__global__ void table_pair_dot_kernel(const T* __restrict__ A, const T* __restrict__ Bt, const long long* __restrict__ ia,
                                      const long long* __restrict__ ib, float* __restrict__ out, long long N, int d) {
  const int lane = threadIdx.x & 31;
  const long long warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long n = warp; n < N; n += nwarps) {
    const T* a = A + ia[n] * d;
    const T* b = Bt + ib[n] * d;
    float acc = 0.f;
    for (int c = lane * 4; c < d; c += 128) {
      float4 x, y;
      if (sizeof(T) == 2) {
        const uint2 ux = *reinterpret_cast<const uint2*>(reinterpret_cast<const bf16*>(a) + c);
        const uint2 uy = *reinterpret_cast<const uint2*>(reinterpret_cast<const bf16*>(b) + c);
        const float2 x0 = unpack_bf16(ux.x), x1 = unpack_bf16(ux.y), y0 = unpack_bf16(uy.x), y1 = unpack_bf16(uy.y);
        x = make_float4(x0.x, x0.y, x1.x, x1.y); y = make_float4(y0.x, y0.y, y1.x, y1.y);
      } else {
        x = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(a) + c);
        y = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(b) + c);
      }
      acc += x.x * y.x + x.y * y.y + x.z * y.z + x.w * y.w;
    }
    acc = warp_sum(acc);
    if (lane == 0) out[n] = acc;
  }
}

torch::Tensor table_pair_dot(torch::Tensor A, torch::Tensor Bt, torch::Tensor ia, torch::Tensor ib) {
  const c10::cuda::CUDAGuard guard(A.device());
  TORCH_CHECK(A.dim() == 2 && Bt.dim() == 2 && A.is_contiguous() && Bt.is_contiguous() && A.size(1) == Bt.size(1) &&
              A.scalar_type() == Bt.scalar_type() && A.size(1) % 4 == 0, "table_pair_dot: two (rows, d) tables of one dtype, d % 4 == 0");
  TORCH_CHECK(A.scalar_type() == torch::kFloat32 || A.scalar_type() == torch::kBFloat16, "table_pair_dot: fp32 or bf16 tables");
  TORCH_CHECK(ia.scalar_type() == torch::kInt64 && ib.scalar_type() == torch::kInt64 && ia.is_contiguous() && ib.is_contiguous() &&
              ia.numel() == ib.numel(), "table_pair_dot: two contiguous int64 index tensors of one size");
  const long long N = ia.numel();
  auto out = torch::empty(ia.sizes(), A.options().dtype(torch::kFloat32));
  if (N) {
    const int grid = (int)std::min<long long>((N * 32 + 255) / 256, 148 * 16);
    const long long* pa = reinterpret_cast<const long long*>(ia.data_ptr<int64_t>());
    const long long* pb = reinterpret_cast<const long long*>(ib.data_ptr<int64_t>());
    if (A.scalar_type() == torch::kBFloat16)
      table_pair_dot_kernel<bf16><<<grid, 256, 0, es()>>>(reinterpret_cast<const bf16*>(A.data_ptr()), reinterpret_cast<const bf16*>(Bt.data_ptr()),
                                                         pa, pb, out.data_ptr<float>(), N, (int)A.size(1));
    else
      table_pair_dot_kernel<float><<<grid, 256, 0, es()>>>(A.data_ptr<float>(), Bt.data_ptr<float>(), pa, pb, out.data_ptr<float>(), N,
                                                          (int)A.size(1));
    C10_CUDA_KERNEL_LAUNCH_CHECK();
  }
  return out;
}

static void check_idx(const torch::Tensor& t, const char* what) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == torch::kInt64 && t.is_contiguous(), "embed_sum: ", what, " must be contiguous int64");
}

// emb (V,d) fp32; x (N); cand (N,K) + sel (N,K) fp32 or both absent; phr (P,d) fp32 + pidx (N) or both absent.
// Indices must be valid rows (the model clamps them); returns h (N,d) fp32.
torch::Tensor embed_sum_fwd(torch::Tensor emb, torch::Tensor x, c10::optional<torch::Tensor> cand_,
                            c10::optional<torch::Tensor> sel_, c10::optional<torch::Tensor> phr_,
                            c10::optional<torch::Tensor> pidx_) {
  const c10::cuda::CUDAGuard guard(emb.device());
  TORCH_CHECK(emb.dim() == 2 && emb.is_contiguous() && emb.scalar_type() == torch::kFloat32 && emb.size(1) % 4 == 0, "embed_sum: emb (V,d) fp32, d % 4 == 0");
  check_idx(x, "x");
  const long long N = x.numel();
  const int d = emb.size(1);
  int K = 0;
  const long long* cand = nullptr;
  const float* sel = nullptr;
  if (cand_.has_value() && cand_->defined()) {
    check_idx(*cand_, "cand");
    TORCH_CHECK(sel_.has_value() && sel_->scalar_type() == torch::kFloat32 && sel_->is_contiguous() && sel_->numel() == cand_->numel(), "embed_sum: sel");
    K = cand_->numel() / std::max<long long>(N, 1);
    cand = reinterpret_cast<const long long*>(cand_->data_ptr<int64_t>());
    sel = sel_->data_ptr<float>();
  }
  const float* phr = nullptr;
  const long long* pidx = nullptr;
  long long P = 0;
  if (phr_.has_value() && phr_->defined()) {
    TORCH_CHECK(phr_->dim() == 2 && phr_->is_contiguous() && phr_->scalar_type() == torch::kFloat32 && phr_->size(1) == d, "embed_sum: phr (P,d) fp32");
    TORCH_CHECK(pidx_.has_value(), "embed_sum: pidx");
    check_idx(*pidx_, "pidx");
    phr = phr_->data_ptr<float>(); pidx = reinterpret_cast<const long long*>(pidx_->data_ptr<int64_t>()); P = phr_->size(0);
  }
  auto out = torch::empty({N, d}, emb.options());
  if (N) {
    const int threads = d >= 1024 ? 256 : 128;
    embed_sum_fwd_kernel<<<(int)std::min<long long>(N, 148 * 16), threads, 0, es()>>>(
        emb.data_ptr<float>(), reinterpret_cast<const long long*>(x.data_ptr<int64_t>()), cand, sel, K, phr, pidx,
        out.data_ptr<float>(), N, d, emb.size(0), P);
    C10_CUDA_KERNEL_LAUNCH_CHECK();
  }
  return out;
}

// Returns {demb (V,d) fp32, dphr (P,d) fp32 or empty, dsel (N,K) fp32 or empty}.
std::vector<torch::Tensor> embed_sum_bwd(torch::Tensor dh, torch::Tensor emb, torch::Tensor x,
                                         c10::optional<torch::Tensor> cand_, c10::optional<torch::Tensor> sel_,
                                         int64_t P, c10::optional<torch::Tensor> pidx_) {
  const c10::cuda::CUDAGuard guard(emb.device());
  TORCH_CHECK(dh.is_contiguous() && dh.scalar_type() == torch::kFloat32, "embed_sum_bwd: dh fp32 contiguous");
  const long long N = x.numel();
  const int d = emb.size(1);
  TORCH_CHECK(dh.numel() == N * d, "embed_sum_bwd: dh shape");
  int K = 0;
  const long long* cand = nullptr;
  const float* sel = nullptr;
  torch::Tensor dsel = torch::empty({0}, emb.options());
  if (cand_.has_value() && cand_->defined()) {
    K = cand_->numel() / std::max<long long>(N, 1);
    cand = reinterpret_cast<const long long*>(cand_->data_ptr<int64_t>());
    sel = sel_->data_ptr<float>();
    dsel = torch::empty({N, K}, emb.options());
  }
  auto demb = torch::zeros_like(emb);
  torch::Tensor dphr = torch::empty({0}, emb.options());
  const long long* pidx = nullptr;
  if (P > 0) {
    dphr = torch::zeros({P, d}, emb.options());
    pidx = reinterpret_cast<const long long*>(pidx_->data_ptr<int64_t>());
  }
  if (N) {
    const int threads = d >= 1024 ? 256 : 128;
    embed_sum_bwd_kernel<<<(int)std::min<long long>(N, 148 * 16), threads, 0, es()>>>(
        dh.data_ptr<float>(), emb.data_ptr<float>(), reinterpret_cast<const long long*>(x.data_ptr<int64_t>()), cand, sel, K,
        pidx, demb.data_ptr<float>(), P > 0 ? dphr.data_ptr<float>() : nullptr, K ? dsel.data_ptr<float>() : nullptr, N, d);
    C10_CUDA_KERNEL_LAUNCH_CHECK();
  }
  return {demb, dphr, dsel};
}

}  // namespace mb
