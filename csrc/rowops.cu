// Row-wise and elementwise kernels (HBM-bound): RMSNorm fwd/bwd, relu^2, SwiGLU, RoPE on packed qkv, the
// cross-entropy row kernel (plain and pointer-mixture), slot gathers / weighted gather-sums for MoE dispatch and
// combine.  All use 16-byte vector accesses and fp32 math.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "common.cuh"

namespace mb {

static inline cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream(); }

template <typename T> __device__ __forceinline__ float4 ld4(const T* p);
template <> __device__ __forceinline__ float4 ld4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <> __device__ __forceinline__ float4 ld4<bf16>(const bf16* p) {
  uint2 u = *reinterpret_cast<const uint2*>(p);
  float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y);
  return make_float4(a.x, a.y, b.x, b.y);
}
template <typename T> __device__ __forceinline__ void st4(T* p, float4 v);
template <> __device__ __forceinline__ void st4<float>(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
template <> __device__ __forceinline__ void st4<bf16>(bf16* p, float4 v) {
  *reinterpret_cast<uint2*>(p) = make_uint2(pack_bf16(v.x, v.y), pack_bf16(v.z, v.w));
}

// ------------------------------------------------------------------------------------------------ RMSNorm
template <typename TX, typename TY>
__global__ void rmsnorm_fwd_kernel(const TX* __restrict__ x, const float* __restrict__ w, TY* __restrict__ y,
                                   float* __restrict__ rstd, int d, float eps) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const TX* xr = x + row * d;
  float ss = 0.f;
  for (int c = threadIdx.x * 4; c < d; c += blockDim.x * 4) {
    float4 v = ld4(xr + c);
    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  ss = block_sum(ss, red);
  const float r = rsqrtf(ss / d + eps);
  if (threadIdx.x == 0) rstd[row] = r;
  TY* yr = y + row * d;
  for (int c = threadIdx.x * 4; c < d; c += blockDim.x * 4) {
    float4 v = ld4(xr + c), g = ld4(w + c);
    st4(yr + c, make_float4(v.x * r * g.x, v.y * r * g.y, v.z * r * g.z, v.w * r * g.w));
  }
}

// dx = r*(g*w) - x * r^3/d * sum(g*w*x); dw += g * x * r (block-local accumulation over its rows, then atomics)
// Optional `add` (fp32, same shape): a gradient that reached x by another path (the residual stream) is summed in
// the same pass; optional `dx_lo`: the result is also written in bf16 (the branch that produced part of x wants it).
template <typename TX, typename TG, int NV>
__global__ void rmsnorm_bwd_kernel(const TG* __restrict__ dy, const TX* __restrict__ x, const float* __restrict__ w,
                                   const float* __restrict__ rstd, TX* __restrict__ dx, float* __restrict__ dw,
                                   int n_rows, int d, const float* __restrict__ add, bf16* __restrict__ dx_lo) {
  __shared__ float red[32];
  // d <= NV * 4 * blockDim.x; a row's x, dy and w stay in registers between the dot product and the update
  float4 acc[NV], ww[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    acc[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    const int c = (i * blockDim.x + threadIdx.x) * 4;
    ww[i] = c < d ? ld4(w + c) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  for (long long row = blockIdx.x; row < n_rows; row += gridDim.x) {
    const TX* xr = x + row * d;
    const TG* gr = dy + row * d;
    const float r = rstd[row];
    float4 xv[NV], gv[NV];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = (i * blockDim.x + threadIdx.x) * 4;
      if (c < d) {
        xv[i] = ld4(xr + c);
        gv[i] = ld4(gr + c);
        dot += gv[i].x * ww[i].x * xv[i].x + gv[i].y * ww[i].y * xv[i].y + gv[i].z * ww[i].z * xv[i].z +
               gv[i].w * ww[i].w * xv[i].w;
      }
    }
    dot = block_sum(dot, red);
    const float k = dot * r * r * r / d;
    TX* dxr = dx + row * d;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = (i * blockDim.x + threadIdx.x) * 4;
      if (c < d) {
        const float4 v = xv[i], g = gv[i];
        float4 o = make_float4(r * g.x * ww[i].x - v.x * k, r * g.y * ww[i].y - v.y * k, r * g.z * ww[i].z - v.z * k,
                               r * g.w * ww[i].w - v.w * k);
        if (add) { const float4 q = ld4(add + row * d + c); o.x += q.x; o.y += q.y; o.z += q.z; o.w += q.w; }
        st4(dxr + c, o);
        if (dx_lo) st4(dx_lo + row * d + c, o);
        acc[i].x += g.x * v.x * r; acc[i].y += g.y * v.y * r; acc[i].z += g.z * v.z * r; acc[i].w += g.w * v.w * r;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = (i * blockDim.x + threadIdx.x) * 4;
    if (c < d) {
      atomicAdd(dw + c, acc[i].x); atomicAdd(dw + c + 1, acc[i].y);
      atomicAdd(dw + c + 2, acc[i].z); atomicAdd(dw + c + 3, acc[i].w);
    }
  }
}

// h = x (fp32) + y (bf16); n = rmsnorm(h) * w in bf16: the residual add and the next normalisation in one pass.
__global__ void add_rmsnorm_fwd_kernel(const float* __restrict__ x, const bf16* __restrict__ y, const float* __restrict__ w,
                                       float* __restrict__ h, bf16* __restrict__ n, float* __restrict__ rstd, int d, float eps) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const float* xr = x + row * d;
  const bf16* yr = y + row * d;
  float* hr = h + row * d;
  float ss = 0.f;
  for (int c = threadIdx.x * 4; c < d; c += blockDim.x * 4) {
    float4 a = ld4(xr + c), b = ld4(yr + c);
    a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
    st4(hr + c, a);
    ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
  }
  ss = block_sum(ss, red);
  const float r = rsqrtf(ss / d + eps);
  if (threadIdx.x == 0) rstd[row] = r;
  bf16* nr = n + row * d;
  for (int c = threadIdx.x * 4; c < d; c += blockDim.x * 4) {
    float4 v = ld4(hr + c), g = ld4(w + c);          // each thread re-reads exactly what it wrote
    st4(nr + c, make_float4(v.x * r * g.x, v.y * r * g.y, v.z * r * g.z, v.w * r * g.w));
  }
}
std::vector<torch::Tensor> add_rmsnorm_fwd(torch::Tensor x, torch::Tensor y, torch::Tensor w, double eps) {
  const c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.dim() == 2 && x.is_contiguous() && y.is_contiguous() && x.scalar_type() == torch::kFloat32 &&
              y.scalar_type() == torch::kBFloat16 && x.numel() == y.numel() && x.size(1) % 4 == 0, "add_rmsnorm: fp32 + bf16");
  const int n = x.size(0), d = x.size(1);
  torch::Tensor wf = w.scalar_type() == torch::kFloat32 ? w : w.to(torch::kFloat32);
  auto h = torch::empty_like(x);
  auto nn = torch::empty({n, d}, x.options().dtype(torch::kBFloat16));
  auto rstd = torch::empty({n}, x.options().dtype(torch::kFloat32));
  if (n) add_rmsnorm_fwd_kernel<<<n, d >= 1024 ? 256 : 128, 0, cur_stream()>>>(x.data_ptr<float>(),
      reinterpret_cast<const bf16*>(y.data_ptr()), wf.data_ptr<float>(), h.data_ptr<float>(), reinterpret_cast<bf16*>(nn.data_ptr()),
      rstd.data_ptr<float>(), d, (float)eps);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {h, nn, rstd};
}

std::vector<torch::Tensor> rmsnorm_fwd(torch::Tensor x, torch::Tensor w, double eps, bool out_bf16) {
  const c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.dim() == 2 && x.is_contiguous() && x.size(1) % 4 == 0, "rmsnorm: (N,d) contiguous, d % 4 == 0");
  const int n = x.size(0), d = x.size(1);
  torch::Tensor wf = w.scalar_type() == torch::kFloat32 ? w : w.to(torch::kFloat32);
  auto y = torch::empty({n, d}, x.options().dtype(out_bf16 ? torch::kBFloat16 : torch::kFloat32));
  auto rstd = torch::empty({n}, x.options().dtype(torch::kFloat32));
  if (n == 0) return {y, rstd};
  const int threads = d >= 1024 ? 256 : 128;
  const bool xb = x.scalar_type() == torch::kBFloat16;
#define LAUNCH(TX, TY) rmsnorm_fwd_kernel<TX, TY><<<n, threads, 0, cur_stream()>>>( \
      reinterpret_cast<const TX*>(x.data_ptr()), wf.data_ptr<float>(), reinterpret_cast<TY*>(y.data_ptr()), \
      rstd.data_ptr<float>(), d, (float)eps)
  if (xb && out_bf16) LAUNCH(bf16, bf16); else if (xb) LAUNCH(bf16, float);
  else if (out_bf16) LAUNCH(float, bf16); else LAUNCH(float, float);
#undef LAUNCH
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {y, rstd};
}

std::vector<torch::Tensor> rmsnorm_bwd(torch::Tensor dy, torch::Tensor x, torch::Tensor w, torch::Tensor rstd,
                                       c10::optional<torch::Tensor> add_, bool want_lo) {
  const c10::cuda::CUDAGuard guard(x.device());
  const float* add = nullptr;
  if (add_.has_value() && add_->defined()) {
    TORCH_CHECK(add_->scalar_type() == torch::kFloat32 && add_->is_contiguous() && add_->numel() == x.numel(), "rmsnorm_bwd: add");
    add = add_->data_ptr<float>();
  }
  const int n = x.size(0), d = x.size(1);
  TORCH_CHECK(d <= 8 * 4 * 256 && d % 4 == 0, "rmsnorm_bwd: d <= 8192");
  torch::Tensor wf = w.scalar_type() == torch::kFloat32 ? w : w.to(torch::kFloat32);
  auto dx = torch::empty_like(x);
  auto dw = torch::zeros({d}, x.options().dtype(torch::kFloat32));
  torch::Tensor lo = want_lo ? torch::empty({n, d}, x.options().dtype(torch::kBFloat16)) : torch::Tensor();
  bf16* lop = want_lo ? reinterpret_cast<bf16*>(lo.data_ptr()) : nullptr;
  if (n == 0) return {dx, dw, lo};
  const int grid = std::min(n, 148 * 8);
  const bool xb = x.scalar_type() == torch::kBFloat16, gb = dy.scalar_type() == torch::kBFloat16;
#define LAUNCH_NV(TX, TG, NV) rmsnorm_bwd_kernel<TX, TG, NV><<<grid, 256, 0, cur_stream()>>>( \
      reinterpret_cast<const TG*>(dy.data_ptr()), reinterpret_cast<const TX*>(x.data_ptr()), wf.data_ptr<float>(), \
      rstd.data_ptr<float>(), reinterpret_cast<TX*>(dx.data_ptr()), dw.data_ptr<float>(), n, d, add, lop)
#define LAUNCH(TX, TG) do { if (d <= 2048) LAUNCH_NV(TX, TG, 2); else if (d <= 4096) LAUNCH_NV(TX, TG, 4); \
                            else LAUNCH_NV(TX, TG, 8); } while (0)
  if (xb && gb) LAUNCH(bf16, bf16); else if (xb) LAUNCH(bf16, float);
  else if (gb) LAUNCH(float, bf16); else LAUNCH(float, float);
#undef LAUNCH
#undef LAUNCH_NV
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {dx, dw, lo};
}

// ------------------------------------------------------------------------------------------------ activations
__global__ void relu2_fwd_kernel(const uint4* __restrict__ a, uint4* __restrict__ h, long long n8) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    uint4 u = a[i];
    uint32_t* p = reinterpret_cast<uint32_t*>(&u);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = unpack_bf16(p[j]);
      f.x = fmaxf(f.x, 0.f); f.y = fmaxf(f.y, 0.f);
      p[j] = pack_bf16(f.x * f.x, f.y * f.y);
    }
    h[i] = u;
  }
}
__global__ void relu2_bwd_kernel(const uint4* __restrict__ dh, const uint4* __restrict__ a, uint4* __restrict__ da,
                                 long long n8) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    uint4 u = a[i], g = dh[i];
    uint32_t* p = reinterpret_cast<uint32_t*>(&u);
    uint32_t* q = reinterpret_cast<uint32_t*>(&g);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = unpack_bf16(p[j]), d = unpack_bf16(q[j]);
      p[j] = pack_bf16(d.x * 2.f * fmaxf(f.x, 0.f), d.y * 2.f * fmaxf(f.y, 0.f));
    }
    da[i] = u;
  }
}
static inline int ew_grid(long long n, int threads) { return (int)std::min<long long>((n + threads - 1) / threads, 148 * 16); }

torch::Tensor relu2_fwd(torch::Tensor a) {
  const c10::cuda::CUDAGuard guard(a.device());
  TORCH_CHECK(a.is_contiguous() && a.scalar_type() == torch::kBFloat16 && a.numel() % 8 == 0, "relu2: bf16, numel % 8");
  auto h = torch::empty_like(a);
  long long n8 = a.numel() / 8;
  if (n8) relu2_fwd_kernel<<<ew_grid(n8, 256), 256, 0, cur_stream()>>>(
      reinterpret_cast<const uint4*>(a.data_ptr()), reinterpret_cast<uint4*>(h.data_ptr()), n8);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return h;
}
torch::Tensor relu2_bwd(torch::Tensor dh, torch::Tensor a) {
  const c10::cuda::CUDAGuard guard(a.device());
  TORCH_CHECK(dh.is_contiguous() && a.is_contiguous() && dh.scalar_type() == torch::kBFloat16, "relu2_bwd: bf16");
  auto da = torch::empty_like(a);
  long long n8 = a.numel() / 8;
  if (n8) relu2_bwd_kernel<<<ew_grid(n8, 256), 256, 0, cur_stream()>>>(
      reinterpret_cast<const uint4*>(dh.data_ptr()), reinterpret_cast<const uint4*>(a.data_ptr()),
      reinterpret_cast<uint4*>(da.data_ptr()), n8);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return da;
}

// gu (R, 2H): h[r, j] = silu(gu[r, j]) * gu[r, H + j]
__global__ void swiglu_fwd_kernel(const bf16* __restrict__ gu, bf16* __restrict__ h, long long R, int H) {
  const int H8 = H / 8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < R * H8; i += (long long)gridDim.x * blockDim.x) {
    long long r = i / H8;
    int c = (int)(i - r * H8) * 8;
    uint4 g = *reinterpret_cast<const uint4*>(gu + r * 2 * H + c), u = *reinterpret_cast<const uint4*>(gu + r * 2 * H + H + c);
    uint32_t* gp = reinterpret_cast<uint32_t*>(&g);
    uint32_t* up = reinterpret_cast<uint32_t*>(&u);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 a = unpack_bf16(gp[j]), b = unpack_bf16(up[j]);
      gp[j] = pack_bf16(a.x / (1.f + __expf(-a.x)) * b.x, a.y / (1.f + __expf(-a.y)) * b.y);
    }
    *reinterpret_cast<uint4*>(h + r * H + c) = g;
  }
}
__global__ void swiglu_bwd_kernel(const bf16* __restrict__ dh, const bf16* __restrict__ gu, bf16* __restrict__ dgu,
                                  long long R, int H) {
  const int H8 = H / 8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < R * H8; i += (long long)gridDim.x * blockDim.x) {
    long long r = i / H8;
    int c = (int)(i - r * H8) * 8;
    uint4 g = *reinterpret_cast<const uint4*>(gu + r * 2 * H + c), u = *reinterpret_cast<const uint4*>(gu + r * 2 * H + H + c);
    uint4 d = *reinterpret_cast<const uint4*>(dh + r * H + c);
    uint32_t* gp = reinterpret_cast<uint32_t*>(&g);
    uint32_t* up = reinterpret_cast<uint32_t*>(&u);
    uint32_t* dp = reinterpret_cast<uint32_t*>(&d);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 a = unpack_bf16(gp[j]), b = unpack_bf16(up[j]), go = unpack_bf16(dp[j]);
      float sx = 1.f / (1.f + __expf(-a.x)), sy = 1.f / (1.f + __expf(-a.y));
      float six = a.x * sx, siy = a.y * sy;
      gp[j] = pack_bf16(go.x * b.x * (sx + six * (1.f - sx)), go.y * b.y * (sy + siy * (1.f - sy)));
      up[j] = pack_bf16(go.x * six, go.y * siy);
    }
    *reinterpret_cast<uint4*>(dgu + r * 2 * H + c) = g;
    *reinterpret_cast<uint4*>(dgu + r * 2 * H + H + c) = u;
  }
}
torch::Tensor swiglu_fwd(torch::Tensor gu) {
  const c10::cuda::CUDAGuard guard(gu.device());
  TORCH_CHECK(gu.is_contiguous() && gu.scalar_type() == torch::kBFloat16 && gu.size(-1) % 16 == 0, "swiglu: bf16, 2H % 16");
  const int H = gu.size(-1) / 2;
  const long long R = gu.numel() / (2 * H);
  auto shape = gu.sizes().vec();
  shape.back() = H;
  auto h = torch::empty(shape, gu.options());
  if (R) swiglu_fwd_kernel<<<ew_grid(R * H / 8, 256), 256, 0, cur_stream()>>>(
      reinterpret_cast<const bf16*>(gu.data_ptr()), reinterpret_cast<bf16*>(h.data_ptr()), R, H);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return h;
}
torch::Tensor swiglu_bwd(torch::Tensor dh, torch::Tensor gu) {
  const c10::cuda::CUDAGuard guard(gu.device());
  TORCH_CHECK(dh.is_contiguous() && gu.is_contiguous() && dh.scalar_type() == torch::kBFloat16, "swiglu_bwd: bf16");
  const int H = gu.size(-1) / 2;
  const long long R = gu.numel() / (2 * H);
  auto dgu = torch::empty_like(gu);
  if (R) swiglu_bwd_kernel<<<ew_grid(R * H / 8, 256), 256, 0, cur_stream()>>>(
      reinterpret_cast<const bf16*>(dh.data_ptr()), reinterpret_cast<const bf16*>(gu.data_ptr()),
      reinterpret_cast<bf16*>(dgu.data_ptr()), R, H);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return dgu;
}

// ------------------------------------------------------------------------------------------------ RoPE on packed qkv
// qkv (B, T, 3, H, hd) bf16.  q and k slices are rotated by the angles of the (T, hd/2) fp32 cos/sin tables (sine
// multiplied by `sign`: -1 rotates back, which is the backward pass); v is copied.
__global__ void rope_qk_kernel(const bf16* __restrict__ in, bf16* __restrict__ out, const float* __restrict__ cs,
                               const float* __restrict__ sn, long long BT, int T, int H, int hd, float sign, int half) {
  const int per_tok = 3 * H * hd / 8;                       // 8-element groups per token
  const int g_per_head = hd / 8;
  const int hh = hd / 2;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < BT * per_tok;
       i += (long long)gridDim.x * blockDim.x) {
    long long tok = i / per_tok;
    int rem = (int)(i - tok * per_tok);
    int s = rem / (H * g_per_head);
    int gi = rem % g_per_head;
    const long long off = i * 8;
    uint4 u = *reinterpret_cast<const uint4*>(in + off);
    if (s < 2) {
      const int t = (int)(tok % T);
      uint32_t* p = reinterpret_cast<uint32_t*>(&u);
      if (!half) {
        const float4 c4 = *reinterpret_cast<const float4*>(cs + (long long)t * hh + gi * 4);
        float4 s4 = *reinterpret_cast<const float4*>(sn + (long long)t * hh + gi * 4);
        const float c[4] = {c4.x, c4.y, c4.z, c4.w}, sv[4] = {s4.x * sign, s4.y * sign, s4.z * sign, s4.w * sign};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 f = unpack_bf16(p[j]);
          p[j] = pack_bf16(f.x * c[j] - f.y * sv[j], f.x * sv[j] + f.y * c[j]);
        }
      } else {
        // halves layout: element e pairs with e + hd/2; this group holds 8 elements of one half
        const int e0 = gi * 8;
        const bool first = e0 < hh;
        const long long mate = first ? off + hh : off - hh;
        uint4 m = *reinterpret_cast<const uint4*>(in + mate);
        uint32_t* q = reinterpret_cast<uint32_t*>(&m);
        const int eb = first ? e0 : e0 - hh;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 a = unpack_bf16(p[j]), b = unpack_bf16(q[j]);
          const float c0 = cs[(long long)t * hh + eb + 2 * j], c1 = cs[(long long)t * hh + eb + 2 * j + 1];
          const float s0 = sn[(long long)t * hh + eb + 2 * j] * sign, s1 = sn[(long long)t * hh + eb + 2 * j + 1] * sign;
          const float r0 = first ? a.x * c0 - b.x * s0 : b.x * s0 + a.x * c0;
          const float r1 = first ? a.y * c1 - b.y * s1 : b.y * s1 + a.y * c1;
          p[j] = pack_bf16(r0, r1);
        }
      }
    }
    *reinterpret_cast<uint4*>(out + off) = u;
  }
}
torch::Tensor rope_qk(torch::Tensor qkv, torch::Tensor cos, torch::Tensor sin, double sign, bool half) {
  const c10::cuda::CUDAGuard guard(qkv.device());
  TORCH_CHECK(qkv.dim() == 5 && qkv.size(2) == 3 && qkv.is_contiguous() && qkv.scalar_type() == torch::kBFloat16,
              "rope_qk: (B,T,3,H,hd) bf16 contiguous");
  const int B = qkv.size(0), T = qkv.size(1), H = qkv.size(3), hd = qkv.size(4);
  TORCH_CHECK(hd % 16 == 0, "rope_qk: head dim % 16");
  TORCH_CHECK(cos.is_contiguous() && sin.is_contiguous() && cos.scalar_type() == torch::kFloat32 && cos.size(0) >= T &&
              cos.size(1) == hd / 2 && sin.sizes() == cos.sizes(), "rope_qk: cos/sin tables (T, hd/2) fp32");
  auto out = torch::empty_like(qkv);
  long long n = (long long)B * T * 3 * H * hd / 8;
  if (n) rope_qk_kernel<<<ew_grid(n, 256), 256, 0, cur_stream()>>>(
      reinterpret_cast<const bf16*>(qkv.data_ptr()), reinterpret_cast<bf16*>(out.data_ptr()), cos.data_ptr<float>(),
      sin.data_ptr<float>(), (long long)B * T, T, H, hd, (float)sign, half ? 1 : 0);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return out;
}

// Backward of "rotate q,k and split qkv": the three gradients arrive as separate (B,H,T,hd) tensors with arbitrary
// batch/head/token strides (last dim contiguous); q and k grads are rotated back and all three are written into one
// packed (B,T,3,H,hd) gradient - replaces stack + contiguous + rope-backward by one pass.
struct Src3 { const bf16* p[3]; long long sb[3], sh[3], st[3]; };
__global__ void rope_merge_bwd_kernel(Src3 src, bf16* __restrict__ out, const float* __restrict__ cs,
                                      const float* __restrict__ sn, long long BT, int T, int H, int hd, int half) {
  const int per_tok = 3 * H * hd / 8;
  const int g_per_head = hd / 8;
  const int hh = hd / 2;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < BT * per_tok;
       i += (long long)gridDim.x * blockDim.x) {
    const long long tok = i / per_tok;
    int rem = (int)(i - tok * per_tok);
    const int s = rem / (H * g_per_head);
    rem -= s * H * g_per_head;
    const int h = rem / g_per_head, gi = rem % g_per_head;
    const long long b = tok / T;
    const int t = (int)(tok - b * T);
    const bf16* base = src.p[s] + b * src.sb[s] + h * src.sh[s] + (long long)t * src.st[s];
    uint4 u = *reinterpret_cast<const uint4*>(base + gi * 8);
    if (s < 2) {
      uint32_t* p = reinterpret_cast<uint32_t*>(&u);
      if (!half) {
        const float4 c4 = *reinterpret_cast<const float4*>(cs + (long long)t * hh + gi * 4);
        const float4 s4 = *reinterpret_cast<const float4*>(sn + (long long)t * hh + gi * 4);
        const float c[4] = {c4.x, c4.y, c4.z, c4.w}, sv[4] = {-s4.x, -s4.y, -s4.z, -s4.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 f = unpack_bf16(p[j]);
          p[j] = pack_bf16(f.x * c[j] - f.y * sv[j], f.x * sv[j] + f.y * c[j]);
        }
      } else {
        const int e0 = gi * 8;
        const bool first = e0 < hh;
        uint4 m = *reinterpret_cast<const uint4*>(base + (first ? e0 + hh : e0 - hh));
        uint32_t* q = reinterpret_cast<uint32_t*>(&m);
        const int eb = first ? e0 : e0 - hh;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 a = unpack_bf16(p[j]), bb = unpack_bf16(q[j]);
          const float c0 = cs[(long long)t * hh + eb + 2 * j], c1 = cs[(long long)t * hh + eb + 2 * j + 1];
          const float s0 = -sn[(long long)t * hh + eb + 2 * j], s1 = -sn[(long long)t * hh + eb + 2 * j + 1];
          const float r0 = first ? a.x * c0 - bb.x * s0 : bb.x * s0 + a.x * c0;
          const float r1 = first ? a.y * c1 - bb.y * s1 : bb.y * s1 + a.y * c1;
          p[j] = pack_bf16(r0, r1);
        }
      }
    }
    *reinterpret_cast<uint4*>(out + i * 8) = u;
  }
}
torch::Tensor rope_merge_bwd(torch::Tensor dq, torch::Tensor dk, torch::Tensor dv, torch::Tensor cos, torch::Tensor sin, bool half) {
  const c10::cuda::CUDAGuard guard(dq.device());
  torch::Tensor g[3] = {dq, dk, dv};
  const int B = dq.size(0), H = dq.size(1), T = dq.size(2), hd = dq.size(3);
  Src3 src;
  for (int i = 0; i < 3; ++i) {
    TORCH_CHECK(g[i].dim() == 4 && g[i].scalar_type() == torch::kBFloat16 && g[i].stride(3) == 1 && g[i].size(2) == T,
                "rope_merge_bwd: (B,H,T,hd) bf16 with contiguous last dim");
    TORCH_CHECK(g[i].stride(0) % 8 == 0 && g[i].stride(1) % 8 == 0 && g[i].stride(2) % 8 == 0 &&
                (reinterpret_cast<uintptr_t>(g[i].data_ptr()) & 15) == 0, "rope_merge_bwd: 16-byte aligned rows");
    src.p[i] = reinterpret_cast<const bf16*>(g[i].data_ptr());
    src.sb[i] = g[i].stride(0); src.sh[i] = g[i].stride(1); src.st[i] = g[i].stride(2);
  }
  auto out = torch::empty({B, T, 3, H, hd}, dq.options());
  long long n = (long long)B * T * 3 * H * hd / 8;
  if (n) rope_merge_bwd_kernel<<<ew_grid(n, 256), 256, 0, cur_stream()>>>(src, reinterpret_cast<bf16*>(out.data_ptr()),
      cos.data_ptr<float>(), sin.data_ptr<float>(), (long long)B * T, T, H, hd, half ? 1 : 0);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return out;
}

// out = x (fp32) + y (bf16): the residual add of a block's bf16 branch output onto the fp32 stream.
__global__ void resid_add_kernel(const float* __restrict__ x, const bf16* __restrict__ y, float* __restrict__ out, long long n4) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    float4 a = reinterpret_cast<const float4*>(x)[i];
    float4 b = ld4(y + i * 4);
    reinterpret_cast<float4*>(out)[i] = make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w);
  }
}
torch::Tensor resid_add(torch::Tensor x, torch::Tensor y) {
  const c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.is_contiguous() && y.is_contiguous() && x.scalar_type() == torch::kFloat32 &&
              y.scalar_type() == torch::kBFloat16 && x.numel() == y.numel() && x.numel() % 4 == 0, "resid_add: fp32 + bf16");
  auto out = torch::empty_like(x);
  long long n4 = x.numel() / 4;
  if (n4) resid_add_kernel<<<ew_grid(n4, 256), 256, 0, cur_stream()>>>(x.data_ptr<float>(),
      reinterpret_cast<const bf16*>(y.data_ptr()), out.data_ptr<float>(), n4);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return out;
}

// ------------------------------------------------------------------------------------------------ CE row kernel
// One block per row of bf16 logits: online max/sum -> lse; loss; logits overwritten with d(loss)/d(logits).
// With gate/hit: pointer mixture P = (1-g)*p_y + g*hit, loss = -log max(P,1e-30), grad = w*(softmax - onehot),
// w = (1-g)*p_y/P, dg = (p_y - hit)/P.
__global__ void ce_rows_kernel(bf16* __restrict__ logits, const long long* __restrict__ y, float* __restrict__ loss,
                               const float* __restrict__ gate, const float* __restrict__ hit, float* __restrict__ dg,
                               long long stride, int V) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  bf16* p = logits + row * stride;
  const int V8 = V / 8;
  float m = -INFINITY, s = 0.f;
  for (int i = threadIdx.x; i < V8; i += blockDim.x) {
    uint4 u = reinterpret_cast<const uint4*>(p)[i];
    const uint32_t* q = reinterpret_cast<const uint32_t*>(&u);
    float v[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) { float2 f = unpack_bf16(q[j]); v[2 * j] = f.x; v[2 * j + 1] = f.y; }
    float mx = v[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) mx = fmaxf(mx, v[j]);
    const float mn = fmaxf(m, mx);
    float add = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) add += __expf(v[j] - mn);
    s = s * __expf(m - mn) + add;
    m = mn;
  }
  for (int c = V8 * 8 + threadIdx.x; c < V; c += blockDim.x) {
    float v = __bfloat162float(p[c]);
    const float mn = fmaxf(m, v);
    s = s * __expf(m - mn) + __expf(v - mn);
    m = mn;
  }
  const float M = block_max(m, red);
  s = (m == -INFINITY) ? 0.f : s * __expf(m - M);
  s = block_sum(s, red);
  const float lse = M + logf(s);
  const long long yy = y[row];
  const float xy = __bfloat162float(p[yy]);
  float wgt = 1.f;
  __syncthreads();                                           // every thread has read p[yy] before anyone overwrites it
  if (gate != nullptr) {
    const float g = gate[row], h = hit[row];
    const float py = __expf(xy - lse);
    float P = fmaxf((1.f - g) * py + g * h, 1e-30f);
    wgt = (1.f - g) * py / P;
    if (threadIdx.x == 0) { loss[row] = -logf(P); dg[row] = (py - h) / P; }
  } else if (threadIdx.x == 0) {
    loss[row] = lse - xy;
  }
  for (int i = threadIdx.x; i < V8; i += blockDim.x) {
    uint4 u = reinterpret_cast<const uint4*>(p)[i];
    uint32_t* q = reinterpret_cast<uint32_t*>(&u);
    const int c0 = i * 8;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = unpack_bf16(q[j]);
      float a = __expf(f.x - lse) - ((c0 + 2 * j) == yy ? 1.f : 0.f);
      float b = __expf(f.y - lse) - ((c0 + 2 * j + 1) == yy ? 1.f : 0.f);
      q[j] = pack_bf16(wgt * a, wgt * b);
    }
    reinterpret_cast<uint4*>(p)[i] = u;
  }
  for (int c = V8 * 8 + threadIdx.x; c < V; c += blockDim.x) {
    float v = __bfloat162float(p[c]);
    p[c] = __float2bfloat16(wgt * (__expf(v - lse) - (c == yy ? 1.f : 0.f)));
  }
}
void ce_rows(torch::Tensor logits, torch::Tensor y, torch::Tensor loss, c10::optional<torch::Tensor> gate,
             c10::optional<torch::Tensor> hit, c10::optional<torch::Tensor> dg) {
  const c10::cuda::CUDAGuard guard(logits.device());
  TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1 && logits.scalar_type() == torch::kBFloat16, "ce_rows: bf16 (n,V)");
  TORCH_CHECK(y.scalar_type() == torch::kInt64 && y.is_contiguous() && loss.is_contiguous(), "ce_rows: y int64");
  TORCH_CHECK(logits.stride(0) % 8 == 0 && (reinterpret_cast<uintptr_t>(logits.data_ptr()) & 15) == 0, "ce_rows: row alignment");
  const int n = logits.size(0), V = logits.size(1);
  if (!n) return;
  const bool mix = gate.has_value() && gate->defined();
  ce_rows_kernel<<<n, 512, 0, cur_stream()>>>(
      reinterpret_cast<bf16*>(logits.data_ptr()), y.data_ptr<int64_t>() ? reinterpret_cast<const long long*>(y.data_ptr<int64_t>()) : nullptr,
      loss.data_ptr<float>(), mix ? gate->data_ptr<float>() : nullptr, mix ? hit->data_ptr<float>() : nullptr,
      mix ? dg->data_ptr<float>() : nullptr, logits.stride(0), V);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------------------ gathers
// out[s] = src[table[s]] * (scale ? scale[s] : 1); table[s] >= n_src -> zeros.  One warp per 256 elements of a row.
template <typename T>
__global__ void gather_rows_kernel(const T* __restrict__ src, const long long* __restrict__ table,
                                   const float* __restrict__ scale, T* __restrict__ out, long long S, int d, long long n_src) {
  const int chunks = d / 4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < S * chunks; i += (long long)gridDim.x * blockDim.x) {
    long long s = i / chunks;
    int c = (int)(i - s * chunks) * 4;
    long long t = table[s];
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (t >= 0 && t < n_src) {
      v = ld4(src + t * d + c);
      if (scale) { float k = scale[s]; v.x *= k; v.y *= k; v.z *= k; v.w *= k; }
    }
    st4(out + s * d + c, v);
  }
}
torch::Tensor gather_rows(torch::Tensor src, torch::Tensor table, c10::optional<torch::Tensor> scale) {
  const c10::cuda::CUDAGuard guard(src.device());
  TORCH_CHECK(src.dim() == 2 && src.is_contiguous() && table.scalar_type() == torch::kInt64 && table.is_contiguous(), "gather_rows");
  const long long S = table.numel();
  const int d = src.size(1);
  TORCH_CHECK(d % 4 == 0, "gather_rows: d % 4");
  auto out = torch::empty({S, d}, src.options());
  const float* sc = (scale.has_value() && scale->defined()) ? scale->data_ptr<float>() : nullptr;
  if (S) {
    int grid = ew_grid(S * (d / 4), 256);
    if (src.scalar_type() == torch::kBFloat16)
      gather_rows_kernel<bf16><<<grid, 256, 0, cur_stream()>>>(reinterpret_cast<const bf16*>(src.data_ptr()),
          reinterpret_cast<const long long*>(table.data_ptr<int64_t>()), sc, reinterpret_cast<bf16*>(out.data_ptr()), S, d, src.size(0));
    else
      gather_rows_kernel<float><<<grid, 256, 0, cur_stream()>>>(src.data_ptr<float>(),
          reinterpret_cast<const long long*>(table.data_ptr<int64_t>()), sc, out.data_ptr<float>(), S, d, src.size(0));
  }
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return out;
}

// out[n] = sum_j w[idx[n,j]] * src[idx[n,j]] over idx < S (fp32 accumulation)
template <typename T>
__global__ void gather_sum_rows_kernel(const T* __restrict__ src, const long long* __restrict__ idx,
                                       const float* __restrict__ w, T* __restrict__ out, long long N, int k, int d, long long S) {
  const int chunks = d / 4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < N * chunks; i += (long long)gridDim.x * blockDim.x) {
    long long n = i / chunks;
    int c = (int)(i - n * chunks) * 4;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int j = 0; j < k; ++j) {
      long long s = idx[n * k + j];
      if (s >= 0 && s < S) {
        float4 v = ld4(src + s * d + c);
        float ww = w ? w[s] : 1.f;
        acc.x += v.x * ww; acc.y += v.y * ww; acc.z += v.z * ww; acc.w += v.w * ww;
      }
    }
    st4(out + n * d + c, acc);
  }
}
torch::Tensor gather_sum_rows(torch::Tensor src, torch::Tensor idx, c10::optional<torch::Tensor> w, int64_t N) {
  const c10::cuda::CUDAGuard guard(src.device());
  TORCH_CHECK(src.dim() == 2 && src.is_contiguous() && idx.dim() == 2 && idx.is_contiguous() && idx.scalar_type() == torch::kInt64,
              "gather_sum_rows");
  TORCH_CHECK(idx.size(0) == N, "gather_sum_rows: idx rows");
  const int d = src.size(1), k = idx.size(1);
  auto out = torch::empty({N, d}, src.options());
  const float* wp = (w.has_value() && w->defined()) ? w->data_ptr<float>() : nullptr;
  if (N) {
    int grid = ew_grid(N * (d / 4), 256);
    if (src.scalar_type() == torch::kBFloat16)
      gather_sum_rows_kernel<bf16><<<grid, 256, 0, cur_stream()>>>(reinterpret_cast<const bf16*>(src.data_ptr()),
          reinterpret_cast<const long long*>(idx.data_ptr<int64_t>()), wp, reinterpret_cast<bf16*>(out.data_ptr()), N, k, d, src.size(0));
    else
      gather_sum_rows_kernel<float><<<grid, 256, 0, cur_stream()>>>(src.data_ptr<float>(),
          reinterpret_cast<const long long*>(idx.data_ptr<int64_t>()), wp, out.data_ptr<float>(), N, k, d, src.size(0));
  }
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return out;
}

// dot[s] = <go[table[s]], ye[s]>  (0 for empty slots); one warp per slot
template <typename T>
__global__ void row_dot_kernel(const T* __restrict__ go, const long long* __restrict__ table, const T* __restrict__ ye,
                               float* __restrict__ out, long long S, int d, long long N) {
  const int lane = threadIdx.x & 31;
  const long long warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long s = warp; s < S; s += nwarps) {
    long long t = table[s];
    float acc = 0.f;
    if (t >= 0 && t < N) {
      for (int c = lane * 4; c < d; c += 128) {
        float4 a = ld4(go + t * d + c), b = ld4(ye + s * d + c);
        acc += a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w;
      }
    }
    acc = warp_sum(acc);
    if (lane == 0) out[s] = acc;
  }
}
torch::Tensor row_dot(torch::Tensor go, torch::Tensor table, torch::Tensor ye) {
  const c10::cuda::CUDAGuard guard(go.device());
  TORCH_CHECK(go.is_contiguous() && ye.is_contiguous() && go.scalar_type() == ye.scalar_type(), "row_dot");
  const long long S = table.numel();
  const int d = go.size(1);
  auto out = torch::empty({S}, go.options().dtype(torch::kFloat32));
  if (S) {
    int grid = (int)std::min<long long>((S * 32 + 255) / 256, 148 * 16);
    if (go.scalar_type() == torch::kBFloat16)
      row_dot_kernel<bf16><<<grid, 256, 0, cur_stream()>>>(reinterpret_cast<const bf16*>(go.data_ptr()),
          reinterpret_cast<const long long*>(table.data_ptr<int64_t>()), reinterpret_cast<const bf16*>(ye.data_ptr()),
          out.data_ptr<float>(), S, d, go.size(0));
    else
      row_dot_kernel<float><<<grid, 256, 0, cur_stream()>>>(go.data_ptr<float>(),
          reinterpret_cast<const long long*>(table.data_ptr<int64_t>()), ye.data_ptr<float>(), out.data_ptr<float>(), S, d, go.size(0));
  }
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return out;
}

}  // namespace mb
