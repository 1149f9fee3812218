// Discrete selection kernels: anchor selection (threshold + causal per-text cap + stable compaction), MoE capacity
// slotting in arrival order, and the keys-and-locks pointer search.  All produce exactly the decisions of the sort /
// cumsum formulations they replace (ties resolved towards the smaller index).
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

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
                                 long long* __restrict__ flat_idx, float* __restrict__ dropped, long long NK, int k, int E, int C,
                                 long long N) {
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
}

std::vector<torch::Tensor> moe_slots(torch::Tensor e_flat, int64_t E, int64_t C) {
  const c10::cuda::CUDAGuard guard(e_flat.device());
  TORCH_CHECK(e_flat.dim() == 2 && e_flat.is_contiguous() && e_flat.scalar_type() == torch::kInt64, "moe_slots: (N,k) int64");
  TORCH_CHECK(E <= SLOT_MAX_E, "moe_slots: at most ", SLOT_MAX_E, " experts");
  const long long N = e_flat.size(0);
  const int k = e_flat.size(1);
  auto table = torch::empty({E * C}, e_flat.options());
  auto flat_idx = torch::empty({N, k}, e_flat.options());
  auto dropped = torch::zeros({}, e_flat.options().dtype(torch::kFloat32));
  moe_slots_kernel<<<1, 1024, 0, cur_stream()>>>(reinterpret_cast<const long long*>(e_flat.data_ptr<int64_t>()),
      reinterpret_cast<long long*>(table.data_ptr<int64_t>()), reinterpret_cast<long long*>(flat_idx.data_ptr<int64_t>()),
      dropped.data_ptr<float>(), N * k, k, (int)E, (int)C, N);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {table, flat_idx, dropped};
}

// Keys and locks: for each position t and n-gram length n = 1..n_keys, the latest j < t whose n-gram ending at j
// equals the one ending at t; the candidate is the token after j.  One block per text, tokens staged in shared memory.
__global__ void lock_find_kernel(const long long* __restrict__ x, long long* __restrict__ cand, bool* __restrict__ on,
                                 long long* __restrict__ src, int T, int n_keys, int longest_only) {
  extern __shared__ int tok[];
  const int b = blockIdx.x;
  const long long* xr = x + (long long)b * T;
  for (int t = threadIdx.x; t < T; t += blockDim.x) tok[t] = (int)xr[t];
  __syncthreads();
  for (int t = threadIdx.x; t < T; t += blockDim.x) {
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
    lock_find_kernel<<<B, 1024, smem, cur_stream()>>>(reinterpret_cast<const long long*>(x.data_ptr<int64_t>()),
        reinterpret_cast<long long*>(cand.data_ptr<int64_t>()), on.data_ptr<bool>(),
        reinterpret_cast<long long*>(src.data_ptr<int64_t>()), T, (int)n_keys, longest_only ? 1 : 0);
  }
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {cand, on, src};
}

}  // namespace mb
