// Discrete selection kernels: anchor selection (threshold + causal per-text cap + stable compaction), MoE capacity
// slotting in arrival order, and the keys-and-locks pointer search.  All produce exactly the decisions of the sort /
// cumsum formulations they replace (ties resolved towards the smaller index).
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include <algorithm>

#include "common.cuh"

namespace mb {

static inline cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream(); }

// exclusive prefix sum of one int per thread over the block; returns the block total through `total`
__device__ __forceinline__ int block_excl_scan(int v, int* warp_tot, int& total) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  int inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    int t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  __syncthreads();
  if (lane == 31) warp_tot[w] = inc;
  __syncthreads();
  if (w == 0) {
    int t = lane < nw ? warp_tot[lane] : 0;
    int ti = t;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int u = __shfl_up_sync(0xffffffffu, ti, o);
      if (lane >= o) ti += u;
    }
    if (lane < nw) warp_tot[lane] = ti - t;            // exclusive warp offsets
    if (lane == 31) warp_tot[32] = ti;                 // block total
  }
  __syncthreads();
  total = warp_tot[32];
  return warp_tot[w] + inc - v;
}

// One block per text.  anchor = s > tau; keep = anchor & (running anchor count <= A);
// idx = kept positions in text order, then the other positions in text order, cut at A; valid = is-kept.
__global__ void anchor_select_kernel(const float* __restrict__ s, const float* __restrict__ tau, long long* __restrict__ idx,
                                     bool* __restrict__ valid, int T, int A) {
  __shared__ int wt[33];
  __shared__ int n_kept_sh;
  const int b = blockIdx.x;
  const float th = *tau;
  const float* sr = s + (long long)b * T;
  // pass 1: number of anchors in the text
  int cnt = 0;
  for (int t = threadIdx.x; t < T; t += blockDim.x) cnt += sr[t] > th ? 1 : 0;
  int total;
  block_excl_scan(cnt, wt, total);
  if (threadIdx.x == 0) n_kept_sh = min(total, A);
  __syncthreads();
  const int n_kept = n_kept_sh;
  // pass 2: chunked scan in text order
  int base_anchor = 0, base_other = 0;
  for (int t0 = 0; t0 < T; t0 += blockDim.x) {
    const int t = t0 + threadIdx.x;
    const int is_a = (t < T && sr[t] > th) ? 1 : 0;
    int tot_a;
    const int rank_a = block_excl_scan(is_a, wt, tot_a) + base_anchor;     // anchors before t
    const int keep = is_a && (rank_a + 1 <= A);
    const int is_o = (t < T && !keep) ? 1 : 0;
    int tot_o;
    const int rank_o = block_excl_scan(is_o, wt, tot_o) + base_other;
    if (t < T) {
      if (keep) {
        idx[(long long)b * A + rank_a] = t;
        valid[(long long)b * A + rank_a] = true;
      } else if (n_kept + rank_o < A) {
        idx[(long long)b * A + n_kept + rank_o] = t;
        valid[(long long)b * A + n_kept + rank_o] = false;
      }
    }
    base_anchor += tot_a;
    base_other += tot_o;
  }
}

std::vector<torch::Tensor> anchor_select(torch::Tensor s, torch::Tensor tau, int64_t A) {
  const c10::cuda::CUDAGuard guard(s.device());
  TORCH_CHECK(s.dim() == 2 && s.is_contiguous() && s.scalar_type() == torch::kFloat32, "anchor_select: (B,T) fp32");
  const int B = s.size(0), T = s.size(1);
  TORCH_CHECK(A <= T, "anchor_select: A <= T");
  auto idx = torch::empty({B, A}, s.options().dtype(torch::kInt64));
  auto valid = torch::empty({B, A}, s.options().dtype(torch::kBool));
  if (B) anchor_select_kernel<<<B, 1024, 0, cur_stream()>>>(s.data_ptr<float>(), tau.data_ptr<float>(),
      reinterpret_cast<long long*>(idx.data_ptr<int64_t>()), valid.data_ptr<bool>(), T, (int)A);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {idx, valid};
}

// MoE slotting: choices in (token, choice) order take the next free place of their expert; places beyond C drop.
// Single block; per-chunk ranks by warp match + cross-warp prefix per expert; running per-expert base across chunks.
constexpr int SLOT_MAX_E = 128;
__global__ void moe_slots_kernel(const long long* __restrict__ e_flat, long long* __restrict__ table,
                                 long long* __restrict__ flat_idx, float* __restrict__ dropped, int* __restrict__ counts,
                                 long long NK, int k, int E, int C, long long N) {
  __shared__ int wcnt[32][SLOT_MAX_E];      // per-warp count of each expert in this chunk
  __shared__ int base[SLOT_MAX_E];
  __shared__ int placed_sh, kept_sh;
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int i = threadIdx.x; i < E; i += blockDim.x) base[i] = 0;
  if (threadIdx.x == 0) { placed_sh = 0; kept_sh = 0; }
  for (long long i = threadIdx.x; i < (long long)E * C; i += blockDim.x) table[i] = N;
  __syncthreads();
  for (long long c0 = 0; c0 < NK; c0 += blockDim.x) {
    for (int i = threadIdx.x; i < nw * SLOT_MAX_E; i += blockDim.x) (&wcnt[0][0])[i] = 0;
    __syncthreads();
    const long long i = c0 + threadIdx.x;
    const int e = i < NK ? (int)e_flat[i] : E;
    const bool real = e >= 0 && e < E;
    const unsigned peers = __match_any_sync(0xffffffffu, real ? e : -1 - lane);
    const int rank_in_warp = __popc(peers & ((1u << lane) - 1u));
    if (real && rank_in_warp == 0) wcnt[w][e] = __popc(peers);
    __syncthreads();
    // exclusive prefix over warps for each expert (thread e handles expert e)
    for (int ee = threadIdx.x; ee < E; ee += blockDim.x) {
      int run = base[ee];
      for (int ww = 0; ww < nw; ++ww) { int t = wcnt[ww][ee]; wcnt[ww][ee] = run; run += t; }
      base[ee] = run;
    }
    __syncthreads();
    if (i < NK) {
      long long out = (long long)E * C;
      if (real) {
        const int rank = wcnt[w][e] + rank_in_warp;
        atomicAdd(&kept_sh, 1);
        if (rank < C) {
          out = (long long)e * C + rank;
          table[out] = i / k;
          atomicAdd(&placed_sh, 1);
        }
      }
      flat_idx[i] = out;
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) *dropped = 1.f - (float)placed_sh / (float)max(kept_sh, 1);
  for (int i = threadIdx.x; i < E; i += blockDim.x) counts[i] = min(base[i], C);      // filled places per expert
}

std::vector<torch::Tensor> moe_slots(torch::Tensor e_flat, int64_t E, int64_t C) {
  const c10::cuda::CUDAGuard guard(e_flat.device());
  TORCH_CHECK(e_flat.dim() == 2 && e_flat.is_contiguous() && e_flat.scalar_type() == torch::kInt64, "moe_slots: (N,k) int64");
  TORCH_CHECK(E <= SLOT_MAX_E, "moe_slots: at most ", SLOT_MAX_E, " experts");
  const long long N = e_flat.size(0);
  const int k = e_flat.size(1);
  auto table = torch::empty({E * C}, e_flat.options());
  auto flat_idx = torch::empty({N, k}, e_flat.options());
  auto dropped = torch::empty({}, e_flat.options().dtype(torch::kFloat32));
  auto counts = torch::empty({E}, e_flat.options().dtype(torch::kInt32));
  moe_slots_kernel<<<1, 1024, 0, cur_stream()>>>(reinterpret_cast<const long long*>(e_flat.data_ptr<int64_t>()),
      reinterpret_cast<long long*>(table.data_ptr<int64_t>()), reinterpret_cast<long long*>(flat_idx.data_ptr<int64_t>()),
      dropped.data_ptr<float>(), counts.data_ptr<int>(), N * k, k, (int)E, (int)C, N);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {table, flat_idx, dropped, counts};
}

// Router: softmax over E experts, top-k_max by probability (ties: smaller expert first), per-token budget k_tok,
// renormalised weights of the kept choices, and the two per-expert sums of the Switch auxiliary loss
// (cnt[e] = kept choices of expert e, psum[e] = sum of probs over real tokens).  One thread per token.
constexpr int ROUTE_MAX_K = 8;
__global__ void moe_route_fwd_kernel(const float* __restrict__ logits, const bool* __restrict__ real,
                                     const long long* __restrict__ k_tok, float* __restrict__ probs,
                                     long long* __restrict__ top_e, float* __restrict__ w, long long* __restrict__ e_flat,
                                     float* __restrict__ cnt, float* __restrict__ psum, long long N, int E, int k_max) {
  __shared__ float cnt_sh[SLOT_MAX_E], ps_sh[SLOT_MAX_E];
  for (int i = threadIdx.x; i < E; i += blockDim.x) { cnt_sh[i] = 0.f; ps_sh[i] = 0.f; }
  __syncthreads();
  const long long n = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (n < N) {
    const float* lr = logits + n * E;
    float mx = -INFINITY;
    for (int e = 0; e < E; ++e) mx = fmaxf(mx, lr[e]);
    float sum = 0.f;
    for (int e = 0; e < E; ++e) sum += expf(lr[e] - mx);
    const float inv = 1.f / sum;
    float tp[ROUTE_MAX_K];
    int te[ROUTE_MAX_K];
#pragma unroll
    for (int j = 0; j < ROUTE_MAX_K; ++j) { tp[j] = -1.f; te[j] = E; }
    const bool is_real = real[n];
    for (int e = 0; e < E; ++e) {
      const float pe = expf(lr[e] - mx) * inv;
      probs[n * E + e] = pe;
      if (is_real) atomicAdd(&ps_sh[e], pe);
      // insertion into the descending top list; strict '>' keeps the smaller expert first on ties
      float cp = pe; int ce = e;
#pragma unroll
      for (int j = 0; j < ROUTE_MAX_K; ++j) {
        if (j < k_max && cp > tp[j]) { const float t = tp[j]; const int u = te[j]; tp[j] = cp; te[j] = ce; cp = t; ce = u; }
      }
    }
    const int kt = (int)k_tok[n];
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < ROUTE_MAX_K; ++j) if (j < k_max && j < kt) s += tp[j];
    s = fmaxf(s, 1e-9f);
#pragma unroll
    for (int j = 0; j < ROUTE_MAX_K; ++j) {
      if (j < k_max) {
        const bool keep = j < kt;
        top_e[n * k_max + j] = te[j];
        w[n * k_max + j] = keep ? tp[j] / s : 0.f;
        e_flat[n * k_max + j] = keep ? te[j] : E;
        if (keep) atomicAdd(&cnt_sh[te[j]], 1.f);
      }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < E; i += blockDim.x) {
    if (cnt_sh[i] != 0.f) atomicAdd(cnt + i, cnt_sh[i]);
    if (ps_sh[i] != 0.f) atomicAdd(psum + i, ps_sh[i]);
  }
}

// dlogits from dw (N,k_max), dprobs_direct (N,E) (may be null) and dpsum (E) (gradient of the aux loss w.r.t. psum):
// dP = scatter of dtp + dprobs_direct + real * dpsum;  dlogits = P * (dP - sum_e P dP).
__global__ void moe_route_bwd_kernel(const float* __restrict__ probs, const long long* __restrict__ top_e,
                                     const long long* __restrict__ k_tok, const bool* __restrict__ real,
                                     const float* __restrict__ dw, const float* __restrict__ dprobs,
                                     const float* __restrict__ dpsum, float* __restrict__ dlogits, long long N, int E, int k_max) {
  const long long n = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (n >= N) return;
  const float* pr = probs + n * E;
  const int kt = (int)k_tok[n];
  float tp[ROUTE_MAX_K], dtp[ROUTE_MAX_K];
  int te[ROUTE_MAX_K];
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < ROUTE_MAX_K; ++j) {
    te[j] = j < k_max ? (int)top_e[n * k_max + j] : E;
    tp[j] = (j < k_max && j < kt) ? pr[te[j]] : 0.f;
    s += tp[j];
  }
  const bool clamped = s < 1e-9f;
  s = fmaxf(s, 1e-9f);
  float dot = 0.f;                                            // sum_j dw_j * w_j
#pragma unroll
  for (int j = 0; j < ROUTE_MAX_K; ++j) if (j < k_max && j < kt) dot += dw[n * k_max + j] * tp[j] / s;
#pragma unroll
  for (int j = 0; j < ROUTE_MAX_K; ++j)
    dtp[j] = (j < k_max && j < kt) ? (dw[n * k_max + j] - (clamped ? 0.f : dot)) / s : 0.f;
  const bool is_real = real[n];
  float pd = 0.f;
  for (int e = 0; e < E; ++e) {
    float d = (dprobs ? dprobs[n * E + e] : 0.f) + ((is_real && dpsum) ? dpsum[e] : 0.f);
#pragma unroll
    for (int j = 0; j < ROUTE_MAX_K; ++j) if (te[j] == e) d += dtp[j];
    pd += pr[e] * d;
  }
  for (int e = 0; e < E; ++e) {
    float d = (dprobs ? dprobs[n * E + e] : 0.f) + ((is_real && dpsum) ? dpsum[e] : 0.f);
#pragma unroll
    for (int j = 0; j < ROUTE_MAX_K; ++j) if (te[j] == e) d += dtp[j];
    dlogits[n * E + e] = pr[e] * (d - pd);
  }
}

std::vector<torch::Tensor> moe_route_fwd(torch::Tensor logits, torch::Tensor real, torch::Tensor k_tok, int64_t k_max) {
  const c10::cuda::CUDAGuard guard(logits.device());
  TORCH_CHECK(logits.dim() == 2 && logits.is_contiguous() && logits.scalar_type() == torch::kFloat32, "moe_route: (N,E) fp32");
  TORCH_CHECK(real.scalar_type() == torch::kBool && real.is_contiguous() && k_tok.scalar_type() == torch::kInt64 &&
              k_tok.is_contiguous(), "moe_route: real bool, k_tok int64");
  const long long N = logits.size(0);
  const int E = logits.size(1);
  TORCH_CHECK(E <= SLOT_MAX_E && k_max >= 1 && k_max <= ROUTE_MAX_K && k_max <= E, "moe_route: E <= 128, k_max <= 8");
  auto io = logits.options().dtype(torch::kInt64);
  auto probs = torch::empty_like(logits);
  auto top_e = torch::empty({N, k_max}, io), e_flat = torch::empty({N, k_max}, io);
  auto w = torch::empty({N, k_max}, logits.options());
  auto cnt = torch::zeros({E}, logits.options()), psum = torch::zeros({E}, logits.options());
  if (N) moe_route_fwd_kernel<<<(int)((N + 127) / 128), 128, 0, cur_stream()>>>(
      logits.data_ptr<float>(), real.data_ptr<bool>(), reinterpret_cast<const long long*>(k_tok.data_ptr<int64_t>()),
      probs.data_ptr<float>(), reinterpret_cast<long long*>(top_e.data_ptr<int64_t>()), w.data_ptr<float>(),
      reinterpret_cast<long long*>(e_flat.data_ptr<int64_t>()), cnt.data_ptr<float>(), psum.data_ptr<float>(), N, E, (int)k_max);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {probs, top_e, w, e_flat, cnt, psum};
}

torch::Tensor moe_route_bwd(torch::Tensor probs, torch::Tensor top_e, torch::Tensor k_tok, torch::Tensor real, torch::Tensor dw,
                            c10::optional<torch::Tensor> dprobs, c10::optional<torch::Tensor> dpsum) {
  const c10::cuda::CUDAGuard guard(probs.device());
  const long long N = probs.size(0);
  const int E = probs.size(1), k_max = top_e.size(1);
  TORCH_CHECK(dw.is_contiguous() && dw.scalar_type() == torch::kFloat32 && dw.numel() == N * k_max, "moe_route_bwd: dw (N,k) fp32");
  const float* dp = nullptr; const float* ds = nullptr;
  if (dprobs.has_value() && dprobs->defined()) {
    TORCH_CHECK(dprobs->is_contiguous() && dprobs->scalar_type() == torch::kFloat32 && dprobs->numel() == N * E, "moe_route_bwd: dprobs");
    dp = dprobs->data_ptr<float>();
  }
  if (dpsum.has_value() && dpsum->defined()) {
    TORCH_CHECK(dpsum->is_contiguous() && dpsum->scalar_type() == torch::kFloat32 && dpsum->numel() == E, "moe_route_bwd: dpsum");
    ds = dpsum->data_ptr<float>();
  }
  auto dl = torch::empty_like(probs);
  if (N) moe_route_bwd_kernel<<<(int)((N + 127) / 128), 128, 0, cur_stream()>>>(
      probs.data_ptr<float>(), reinterpret_cast<const long long*>(top_e.data_ptr<int64_t>()),
      reinterpret_cast<const long long*>(k_tok.data_ptr<int64_t>()), real.data_ptr<bool>(), dw.data_ptr<float>(), dp, ds,
      dl.data_ptr<float>(), N, E, k_max);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return dl;
}

// Keys and locks: for each position t and n-gram length n = 1..n_keys, the latest j < t whose n-gram ending at j
// equals the one ending at t; the candidate is the token after j.  The text is staged in shared memory; grid (texts,
// slices): a block takes runs of blockDim positions spread evenly over the text (late positions scan further back, so
// contiguous halves would be unbalanced), which keeps a batch of few long texts (4 x 16 384) on all SMs.
__global__ void lock_find_kernel(const long long* __restrict__ x, long long* __restrict__ cand, bool* __restrict__ on,
                                 long long* __restrict__ src, int T, int n_keys, int longest_only) {
  extern __shared__ int tok[];
  const int b = blockIdx.x;
  const long long* xr = x + (long long)b * T;
  for (int t = threadIdx.x; t < T; t += blockDim.x) tok[t] = (int)xr[t];
  __syncthreads();
  for (int t = blockIdx.y * blockDim.x + threadIdx.x; t < T; t += gridDim.y * blockDim.x) {
    int last[3] = {-1, -1, -1};
    const int a0 = tok[t], a1 = t >= 1 ? tok[t - 1] : -1, a2 = t >= 2 ? tok[t - 2] : -1;
    int need = n_keys;                                   // how many key lengths are still unresolved
    for (int j = t - 1; j >= 0 && need > 0; --j) {
      if (tok[j] != a0) continue;
      if (last[0] < 0) { last[0] = j; --need; }
      if (n_keys >= 2 && t >= 1 && j >= 1 && tok[j - 1] == a1) {
        if (last[1] < 0) { last[1] = j; --need; }
        if (n_keys >= 3 && t >= 2 && j >= 2 && tok[j - 2] == a2 && last[2] < 0) { last[2] = j; --need; }
      }
      // a longer key can only match where the shorter one matches, so once the 1-gram is found we keep scanning
      // only for the longer ones; stop early when position constraints make them impossible
      if (n_keys >= 2 && t < 1 && last[0] >= 0) break;
    }
    bool ok[3];
    for (int n = 0; n < n_keys; ++n) ok[n] = last[n] >= 0;
    if (longest_only) {
      for (int n = 0; n < n_keys - 1; ++n)
        for (int q = n + 1; q < n_keys; ++q) if (ok[q]) ok[n] = false;
    }
    for (int n = 0; n < n_keys; ++n) {
      const bool found = last[n] >= 0;
      const int sp = found ? min(last[n] + 1, T - 1) : 0;
      const long long o = ((long long)b * T + t) * n_keys + n;
      cand[o] = found ? tok[sp] : 0;
      src[o] = sp;
      on[o] = ok[n];
    }
  }
}

std::vector<torch::Tensor> lock_find(torch::Tensor x, int64_t vocab, int64_t n_keys, bool longest_only) {
  const c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.dim() == 2 && x.is_contiguous() && x.scalar_type() == torch::kInt64, "lock_find: (B,T) int64");
  TORCH_CHECK(n_keys >= 1 && n_keys <= 3, "lock_find: 1..3 key lengths");
  const int B = x.size(0), T = x.size(1);
  TORCH_CHECK((size_t)T * 4 <= 200 * 1024, "lock_find: text too long for shared memory staging");
  auto cand = torch::empty({B, T, n_keys}, x.options());
  auto src = torch::empty({B, T, n_keys}, x.options());
  auto on = torch::empty({B, T, n_keys}, x.options().dtype(torch::kBool));
  if (B) {
    size_t smem = (size_t)T * 4;
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(lock_find_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    const int threads = 256;
    const int slices = std::max(1, std::min((T + threads - 1) / threads, (4 * 148 + B - 1) / B));
    lock_find_kernel<<<dim3(B, slices), threads, smem, cur_stream()>>>(reinterpret_cast<const long long*>(x.data_ptr<int64_t>()),
        reinterpret_cast<long long*>(cand.data_ptr<int64_t>()), on.data_ptr<bool>(),
        reinterpret_cast<long long*>(src.data_ptr<int64_t>()), T, (int)n_keys, longest_only ? 1 : 0);
  }
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {cand, on, src};
}

}  // namespace mb
