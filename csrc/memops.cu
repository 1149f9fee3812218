// Card-memory read: scores of every word of a segment against every card, fused.
//   fa      = faces / max(|faces|, 1e-12)                       (per card, per link of its chain of faces)
//   sc[s,c] = max_l <q[s], fa[c,l]> * scale  (+ dim_pen for cards of the dim bank), -1e4 where the card is empty
//   w[s,c]  = softmax_c(sc[s,:]) * any_valid
// One block per (text, tile of 8 words); the cards' normalised faces go through shared memory in chunks; the scores of
// a word stay in shared memory until its softmax is done, so the (S x C x L) score tensor never reaches HBM.
// Backward: dsc = w * (dw - sum_c w dw) + dsc_direct ; dq = sum_c dsc * scale * fa[c, best] ; dfaces through the arg-max
// link and the normalisation; d dim_pen = sum of dsc over dim cards.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "common.cuh"

namespace mb {

static inline cudaStream_t mem_stream() { return at::cuda::getCurrentCUDAStream(); }

constexpr int MR_WORDS = 8;        // words per block (one warp each)
constexpr int MR_CHUNK = 32;       // cards per shared-memory chunk

// grid (ceil(S / 8), B), block 256.  F (face width) <= 128 and a multiple of 32.
__global__ void mem_read_fwd_kernel(const float* __restrict__ q, const float* __restrict__ faces, const bool* __restrict__ valid,
                                    const float* __restrict__ dim_pen, float* __restrict__ sc, float* __restrict__ w,
                                    unsigned char* __restrict__ best, int S, int C, int L, int F, int Fn, float scale) {
  extern __shared__ float sh[];
  float* fa = sh;                                  // MR_CHUNK * L * F normalised faces
  float* row = fa + MR_CHUNK * L * F;              // MR_WORDS * C scores
  const int b = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int s = blockIdx.x * MR_WORDS + warp;
  const float pen = *dim_pen;
  const int per = F / 32;
  float qv[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) qv[j] = (j < per && s < S) ? q[((long long)b * S + s) * F + j * 32 + lane] : 0.f;
  const float* fb = faces + (long long)b * C * L * F;
  const bool* vb = valid + (long long)b * C;
  for (int c0 = 0; c0 < C; c0 += MR_CHUNK) {
    const int nc = min(MR_CHUNK, C - c0);
    __syncthreads();
    // stage and normalise: one warp per (card, link) vector
    for (int v = warp; v < nc * L; v += blockDim.x >> 5) {
      const float* src = fb + ((long long)c0 * L + v) * F;
      float x[4], ss = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) { x[j] = j < per ? src[j * 32 + lane] : 0.f; ss += x[j] * x[j]; }
      ss = warp_sum(ss);
      const float inv = 1.f / fmaxf(sqrtf(ss), 1e-12f);
#pragma unroll
      for (int j = 0; j < 4; ++j) if (j < per) fa[v * F + j * 32 + lane] = x[j] * inv;
    }
    __syncthreads();
    if (s < S) {
      for (int c = 0; c < nc; ++c) {
        float bestv = -INFINITY;
        int bl = 0;
        for (int l = 0; l < L; ++l) {
          const float* f = fa + (c * L + l) * F;
          float d = 0.f;
#pragma unroll
          for (int j = 0; j < 4; ++j) if (j < per) d += qv[j] * f[j * 32 + lane];
          d = warp_sum(d);
          if (d > bestv) { bestv = d; bl = l; }
        }
        if (lane == 0) {
          const int cc = c0 + c;
          float v = bestv * scale + (cc >= Fn ? pen : 0.f);
          if (!vb[cc]) v = -1e4f;
          row[warp * C + cc] = v;
          best[((long long)b * S + s) * C + cc] = (unsigned char)bl;
        }
      }
    }
  }
  __syncwarp();
  if (s >= S) return;
  float* r = row + warp * C;
  float mx = -INFINITY;
  bool any = false;
  for (int c = lane; c < C; c += 32) { mx = fmaxf(mx, r[c]); any |= vb[c]; }
  mx = warp_max(mx);
  any = __any_sync(0xffffffffu, any);
  float sum = 0.f;
  for (int c = lane; c < C; c += 32) sum += expf(r[c] - mx);
  sum = warp_sum(sum);
  const float inv = any ? 1.f / sum : 0.f;
  float* so = sc + ((long long)b * S + s) * C;
  float* wo = w + ((long long)b * S + s) * C;
  for (int c = lane; c < C; c += 32) { so[c] = r[c]; wo[c] = expf(r[c] - mx) * inv; }
}

// grid (S, B), block 128: one block per word.  dfa (B,C,L,F) accumulates with atomics (zeroed by the caller).
__global__ void mem_read_bwd_kernel(const float* __restrict__ q, const float* __restrict__ faces, const bool* __restrict__ valid,
                                    const float* __restrict__ w, const unsigned char* __restrict__ best,
                                    const float* __restrict__ dw, const float* __restrict__ dsc_in, float* __restrict__ dq,
                                    float* __restrict__ dfa, float* __restrict__ dpen, int S, int C, int L, int F, int Fn,
                                    float scale) {
  extern __shared__ float sh[];
  float* dsc = sh;                                 // C
  float* qs = dsc + C;                             // F
  float* dqs = qs + F;                             // F
  __shared__ float red[32];
  const int b = blockIdx.y, s = blockIdx.x;
  const long long ro = ((long long)b * S + s) * C;
  const bool* vb = valid + (long long)b * C;
  float dot = 0.f;
  bool any = false;
  for (int c = threadIdx.x; c < C; c += blockDim.x) { dot += w[ro + c] * dw[ro + c]; any |= vb[c]; }
  dot = block_sum(dot, red);
  float pen_acc = 0.f;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float d = w[ro + c] * (dw[ro + c] - dot) + (dsc_in ? dsc_in[ro + c] : 0.f);
    if (!vb[c]) d = 0.f;                           // masked scores are constants
    dsc[c] = d;
    if (c >= Fn) pen_acc += d;
  }
  for (int f = threadIdx.x; f < F; f += blockDim.x) { qs[f] = q[((long long)b * S + s) * F + f]; dqs[f] = 0.f; }
  pen_acc = block_sum(pen_acc, red);
  if (threadIdx.x == 0 && pen_acc != 0.f) atomicAdd(dpen, pen_acc);
  __syncthreads();
  // each warp takes cards round-robin; lanes cover the face width
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const int per = F / 32;
  float dq_acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int c = warp; c < C; c += nw) {
    const float d = dsc[c] * scale;
    if (d == 0.f) continue;
    const int l = best[ro + c];
    const long long fo = (((long long)b * C + c) * L + l) * F;
    float x[4], ss = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) { x[j] = j < per ? faces[fo + j * 32 + lane] : 0.f; ss += x[j] * x[j]; }
    ss = warp_sum(ss);
    const float nrm = fmaxf(sqrtf(ss), 1e-12f), inv = 1.f / nrm;
    // fa = x * inv ; d(dot)/dx = (q - fa <q, fa>) * inv
    float qf = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) if (j < per) qf += qs[j * 32 + lane] * x[j] * inv;
    qf = warp_sum(qf);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (j < per) {
        const float fa = x[j] * inv;
        dq_acc[j] += d * fa;
        atomicAdd(dfa + fo + j * 32 + lane, d * (qs[j * 32 + lane] - fa * qf) * inv);
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) if (j < per) atomicAdd(&dqs[j * 32 + lane], dq_acc[j]);
  __syncthreads();
  for (int f = threadIdx.x; f < F; f += blockDim.x) dq[((long long)b * S + s) * F + f] = dqs[f];
}

std::vector<torch::Tensor> mem_read_fwd(torch::Tensor q, torch::Tensor faces, torch::Tensor valid, torch::Tensor dim_pen,
                                        int64_t Fn, double scale) {
  const c10::cuda::CUDAGuard guard(q.device());
  TORCH_CHECK(q.dim() == 3 && faces.dim() == 4 && q.is_contiguous() && faces.is_contiguous() && valid.is_contiguous(),
              "mem_read: q (B,S,F), faces (B,C,L,F), valid (B,C), contiguous");
  TORCH_CHECK(q.scalar_type() == torch::kFloat32 && faces.scalar_type() == torch::kFloat32 &&
              valid.scalar_type() == torch::kBool && dim_pen.scalar_type() == torch::kFloat32, "mem_read: fp32 / bool");
  const int B = q.size(0), S = q.size(1), F = q.size(2), C = faces.size(1), L = faces.size(2);
  TORCH_CHECK(F % 32 == 0 && F <= 128 && faces.size(3) == F && L <= 255, "mem_read: face width a multiple of 32, <= 128");
  auto sc = torch::empty({B, S, C}, q.options());
  auto w = torch::empty({B, S, C}, q.options());
  auto best = torch::empty({B, S, C}, q.options().dtype(torch::kUInt8));
  if (B * S == 0) return {sc, w, best};
  const size_t smem = ((size_t)MR_CHUNK * L * F + (size_t)MR_WORDS * C) * sizeof(float);
  TORCH_CHECK(smem <= 200 * 1024, "mem_read: too many cards for the shared-memory row cache");
  static bool raised = false;
  if (smem > 48 * 1024 && !raised) {
    cudaFuncSetAttribute(mem_read_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    raised = true;
  }
  dim3 grid((S + MR_WORDS - 1) / MR_WORDS, B);
  mem_read_fwd_kernel<<<grid, MR_WORDS * 32, smem, mem_stream()>>>(
      q.data_ptr<float>(), faces.data_ptr<float>(), valid.data_ptr<bool>(), dim_pen.data_ptr<float>(), sc.data_ptr<float>(),
      w.data_ptr<float>(), best.data_ptr<unsigned char>(), S, C, L, F, (int)Fn, (float)scale);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {sc, w, best};
}

std::vector<torch::Tensor> mem_read_bwd(torch::Tensor q, torch::Tensor faces, torch::Tensor valid, torch::Tensor w,
                                        torch::Tensor best, torch::Tensor dw, c10::optional<torch::Tensor> dsc, int64_t Fn,
                                        double scale) {
  const c10::cuda::CUDAGuard guard(q.device());
  const int B = q.size(0), S = q.size(1), F = q.size(2), C = faces.size(1), L = faces.size(2);
  TORCH_CHECK(dw.is_contiguous() && dw.scalar_type() == torch::kFloat32 && dw.numel() == (long long)B * S * C, "mem_read_bwd: dw");
  const float* dsp = nullptr;
  if (dsc.has_value() && dsc->defined()) {
    TORCH_CHECK(dsc->is_contiguous() && dsc->scalar_type() == torch::kFloat32 && dsc->numel() == dw.numel(), "mem_read_bwd: dsc");
    dsp = dsc->data_ptr<float>();
  }
  auto dq = torch::empty_like(q);
  auto dfa = torch::zeros_like(faces);
  auto dpen = torch::zeros({}, q.options());
  if (B * S == 0) return {dq, dfa, dpen};
  const size_t smem = ((size_t)C + 2 * F) * sizeof(float);
  dim3 grid(S, B);
  mem_read_bwd_kernel<<<grid, 128, smem, mem_stream()>>>(
      q.data_ptr<float>(), faces.data_ptr<float>(), valid.data_ptr<bool>(), w.data_ptr<float>(), best.data_ptr<unsigned char>(),
      dw.data_ptr<float>(), dsp, dq.data_ptr<float>(), dfa.data_ptr<float>(), dpen.data_ptr<float>(), S, C, L, F, (int)Fn,
      (float)scale);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {dq, dfa, dpen};
}

}  // namespace mb
