// Causal / sliding-window attention backward on the tcgen05 tensor cores (head dim 64, bf16, fp32 accumulation).
//
// One CTA per (128-key tile j, batch*head); it walks the query tiles i that can see tile j (the diagonal tile up to
// the last one inside the window).  All operand tiles are [128 rows x 64] bf16, 128-byte swizzled, and serve either
// as a K-major operand (contraction over the head dim) or as an MN-major operand (contraction over the rows):
//   S   = Q_i K_j^T                      (q x keys, K = hd)      P  = exp2(S scale - lse_i)      [softmax threads]
//   dP  = dO_i V_j^T                     (q x keys, K = hd)      dS = P (dP - delta_i) / sqrt(hd) [softmax threads]
//   dV += P^T  dO_i                      (keys x hd, K = q)      accumulates over i in TMEM
//   dK += dS^T Q_i                       (keys x hd, K = q)      accumulates over i in TMEM
//   dQ_i = dS K_j                        (q x hd, K = keys)      added to the fp32 dQ buffer with atomics
// Roles: warp 0 TMA producer (K_j, V_j once; Q_i, dO_i through a 2-stage ring), warp 1 MMA issuer, warps 2..5 one
// thread per row (query row for S / dP / dQ, key row for dK / dV).  Every wait is bounded.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda.h>

#include "common.cuh"

namespace mb {

CUtensorMap make_tmap_bf16(const void* base, uint64_t inner, uint64_t rows, uint64_t groups, uint64_t row_pitch_el,
                           uint64_t group_pitch_el, uint32_t box_inner, uint32_t box_rows);

constexpr int AB_T = 128, AB_HD = 64, AB_THREADS = 192;
constexpr int AB_TILE = AB_T * AB_HD * 2;                // 16 KB
constexpr int AB_PT = AB_T * AB_T * 2;                   // 32 KB
constexpr int AB_SMEM = 2 * AB_TILE + 2 * 2 * AB_TILE + 2 * AB_PT + 256;   // K, V, (Q, dO) x 2 stages, P, dS

struct AttnBwdParams {
  int T, window;
  float scale, scale_log2;
  const float* lse;         // (BH, T) natural log
  const float* delta;       // (BH, T) rowsum(dO * O)
  float* dq;                // (BH, T, 64) fp32, zeroed by the caller
  bf16* dk;                 // (BH, T, 64)
  bf16* dv;
  int* status;
};

__global__ void __launch_bounds__(AB_THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO, const AttnBwdParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  if (threadIdx.x == 0 && (smem_u32(smem) & 1023u)) atomicCAS(p.status, 0, ST_BAD_ARG);
  uint8_t* sK = smem;
  uint8_t* sV = sK + AB_TILE;
  uint8_t* sQ = sV + AB_TILE;                             // 2 stages
  uint8_t* sDO = sQ + 2 * AB_TILE;                        // 2 stages
  uint8_t* sP = sDO + 2 * AB_TILE;
  uint8_t* sDS = sP + AB_PT;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sDS + AB_PT);
  uint64_t* kv_full = bars;           // 1
  uint64_t* q_full = bars + 1;        // 2
  uint64_t* q_empty = bars + 3;       // 2
  uint64_t* s_full = bars + 5;        // S and dP in TMEM
  uint64_t* p_full = bars + 6;        // P and dS in shared memory (4 warp arrivals)
  uint64_t* dq_full = bars + 7;       // dQ tile in TMEM (and this step's dV / dK contributions issued)
  uint64_t* step_free = bars + 8;     // S, dP, P, dS, dQ tile consumed (4 warp arrivals)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 9);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kt = blockIdx.x, bh = blockIdx.y;
  const int k0 = kt * AB_T;
  const int nq = (p.T + AB_T - 1) / AB_T;
  const int first_qt = kt;
  const int last_qt = p.window > 0 ? min(nq - 1, (k0 + AB_T - 1 + p.window - 1) / AB_T) : nq - 1;
  const int n_qt = last_qt - first_qt + 1;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < 2; ++s) { mbar_init(&q_full[s], 1); mbar_init(&q_empty[s], 1); }
    mbar_init(s_full, 1); mbar_init(p_full, 4); mbar_init(dq_full, 1); mbar_init(step_free, 4);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV); tma_prefetch_desc(&tmDO);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base, tDP = tmem_base + 128, tDV = tmem_base + 256, tDK = tmem_base + 320, tDQ = tmem_base + 384;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(kv_full, 2 * AB_TILE);
      tma_load_3d(sK, &tmK, kv_full, 0, k0, bh);
      tma_load_3d(sV, &tmV, kv_full, 0, k0, bh);
      for (int i = 0; i < n_qt; ++i) {
        const int s = i & 1;
        if (!mbar_wait(&q_empty[s], ((i >> 1) & 1) ^ 1, abort_flag)) { atomicCAS(p.status, 0, ST_WAIT_EMPTY); *abort_flag = 1; break; }
        const int q0 = (first_qt + i) * AB_T;
        mbar_expect_tx(&q_full[s], 2 * AB_TILE);
        tma_load_3d(sQ + s * AB_TILE, &tmQ, &q_full[s], 0, q0, bh);
        tma_load_3d(sDO + s * AB_TILE, &tmDO, &q_full[s], 0, q0, bh);
      }
      if (*abort_flag) { for (int i = 0; i < 2000; ++i) __nanosleep(1000); }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t id_kk = idesc_bf16(128, 128, 0u, 0u);      // K-major x K-major (S, dP)
      const uint32_t id_tt = idesc_bf16(128, 64, 1u, 1u);       // MN-major x MN-major (dV, dK)
      const uint32_t id_kt = idesc_bf16(128, 64, 0u, 1u);       // K-major x MN-major (dQ)
      bool ok = mbar_wait(kv_full, 0, abort_flag);
      if (!ok) { atomicCAS(p.status, 0, ST_WAIT_FULL); *abort_flag = 1; }
      const uint32_t aK = smem_u32(sK), aV = smem_u32(sV), aP = smem_u32(sP), aDS = smem_u32(sDS);
      for (int i = 0; i < n_qt && ok; ++i) {
        const int s = i & 1;
        if (!mbar_wait(&q_full[s], (i >> 1) & 1, abort_flag)) { atomicCAS(p.status, 0, ST_WAIT_FULL); *abort_flag = 1; break; }
        if (i > 0 && !mbar_wait(step_free, (i - 1) & 1, abort_flag)) { atomicCAS(p.status, 0, ST_WAIT_TMEM_EMPTY); *abort_flag = 1; break; }
        tc_fence_after();
        const uint32_t aQ = smem_u32(sQ + s * AB_TILE), aDO = smem_u32(sDO + s * AB_TILE);
#pragma unroll
        for (int k = 0; k < AB_HD / 16; ++k) {
          umma_bf16(tS, smem_desc_sw128(aQ + k * 32, 0, 1024), smem_desc_sw128(aK + k * 32, 0, 1024), id_kk, k > 0 ? 1u : 0u);
          umma_bf16(tDP, smem_desc_sw128(aDO + k * 32, 0, 1024), smem_desc_sw128(aV + k * 32, 0, 1024), id_kk, k > 0 ? 1u : 0u);
        }
        umma_commit(s_full);
        if (!mbar_wait(p_full, i & 1, abort_flag)) { atomicCAS(p.status, 0, ST_WAIT_TMEM_FULL); *abort_flag = 1; break; }
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < AB_T / 16; ++k) {                    // contraction over the 128 query rows, 16 per step
          const uint32_t acc = (i > 0 || k > 0) ? 1u : 0u;
          umma_bf16(tDV, smem_desc_sw128(aP + k * 2048, 16384, 1024), smem_desc_sw128(aDO + k * 2048, 8192, 1024), id_tt, acc);
          umma_bf16(tDK, smem_desc_sw128(aDS + k * 2048, 16384, 1024), smem_desc_sw128(aQ + k * 2048, 8192, 1024), id_tt, acc);
        }
#pragma unroll
        for (int k = 0; k < AB_T / 16; ++k) {                    // contraction over the 128 keys
          const uint32_t ad = aDS + (k >> 2) * 16384 + (k & 3) * 32;
          umma_bf16(tDQ, smem_desc_sw128(ad, 0, 1024), smem_desc_sw128(aK + k * 2048, 8192, 1024), id_kt, k > 0 ? 1u : 0u);
        }
        umma_commit(dq_full);
        umma_commit(&q_empty[s]);
      }
    }
  } else {
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const float L2E = 1.4426950408889634f;
    bool ok = true;
    uint32_t r[32], r2[32];
    for (int i = 0; i < n_qt && ok; ++i) {
      const int q0 = (first_qt + i) * AB_T;
      const int qi = q0 + row;
      const bool q_ok = qi < p.T;
      const float lse2 = q_ok ? p.lse[(long long)bh * p.T + qi] * L2E : 0.f;
      const float dl = q_ok ? p.delta[(long long)bh * p.T + qi] : 0.f;
      if (!mbar_wait(s_full, i & 1, abort_flag)) { if (lane == 0) { atomicCAS(p.status, 0, ST_WAIT_TMEM_FULL); *abort_flag = 1; } ok = false; break; }
      tc_fence_after();
      // key columns this query row may see: kj <= qi, qi - kj < window, kj < T
      const int hi = q_ok ? min(qi, p.T - 1) - k0 : -1;
      const int lo = p.window > 0 ? max(0, qi - p.window + 1 - k0) : 0;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        __syncwarp();
        tmem_ld32(tS + lane_base + c * 32, r);
        tmem_ld32(tDP + lane_base + c * 32, r2);
        tmem_ld_wait();
        uint32_t pp[16], dd[16];
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          float pv[2], dv[2];
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int col = c * 32 + j + u;
            const bool vis = col >= lo && col <= hi;
            pv[u] = vis ? exp2f(__uint_as_float(r[j + u]) * p.scale_log2 - lse2) : 0.f;
            dv[u] = vis ? pv[u] * (__uint_as_float(r2[j + u]) - dl) * p.scale : 0.f;
          }
          pp[j >> 1] = pack_bf16(pv[0], pv[1]);
          dd[j >> 1] = pack_bf16(dv[0], dv[1]);
        }
        const int off = (c >> 1) * 16384 + row * 128;
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const int chunk = ((c & 1) * 4 + q4) ^ (row & 7);
          *reinterpret_cast<uint4*>(sP + off + (chunk << 4)) = make_uint4(pp[q4 * 4], pp[q4 * 4 + 1], pp[q4 * 4 + 2], pp[q4 * 4 + 3]);
          *reinterpret_cast<uint4*>(sDS + off + (chunk << 4)) = make_uint4(dd[q4 * 4], dd[q4 * 4 + 1], dd[q4 * 4 + 2], dd[q4 * 4 + 3]);
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
      if (!mbar_wait(dq_full, i & 1, abort_flag)) { if (lane == 0) { atomicCAS(p.status, 0, ST_WAIT_TMEM_FULL); *abort_flag = 1; } ok = false; break; }
      tc_fence_after();
      float* dqr = p.dq + ((long long)bh * p.T + qi) * AB_HD;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        __syncwarp();
        tmem_ld32(tDQ + lane_base + c * 32, r);
        tmem_ld_wait();
        if (q_ok) {
#pragma unroll
          for (int j = 0; j < 32; j += 4)                       // 16-byte vector reduction: a quarter of the atomic traffic
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dqr + c * 32 + j), "f"(__uint_as_float(r[j])),
                         "f"(__uint_as_float(r[j + 1])), "f"(__uint_as_float(r[j + 2])), "f"(__uint_as_float(r[j + 3])) : "memory");
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(step_free);
    }
    // dK, dV: this thread's key row (the last dq_full commit also covers every dV / dK MMA)
    const int kj = k0 + row;
    if (ok && n_qt > 0) {
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        bf16* dst = (which == 0 ? p.dv : p.dk) + ((long long)bh * p.T + kj) * AB_HD;
        const uint32_t t0 = which == 0 ? tDV : tDK;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          __syncwarp();
          tmem_ld32(t0 + lane_base + c * 32, r);
          tmem_ld_wait();
          if (kj < p.T) {
#pragma unroll
            for (int j = 0; j < 32; j += 8)
              *reinterpret_cast<uint4*>(dst + c * 32 + j) =
                  make_uint4(pack_bf16(__uint_as_float(r[j]), __uint_as_float(r[j + 1])),
                             pack_bf16(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3])),
                             pack_bf16(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5])),
                             pack_bf16(__uint_as_float(r[j + 6]), __uint_as_float(r[j + 7])));
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

int64_t attn_status_read();
static int* attn_bwd_status(int device) {
  static int* words[16] = {nullptr};
  if (!words[device]) {
    TORCH_CHECK(cudaMalloc(&words[device], sizeof(int)) == cudaSuccess, "status word alloc failed");
    cudaMemset(words[device], 0, sizeof(int));
  }
  return words[device];
}
int64_t attn_bwd_status_read() {
  int dev = 0;
  cudaGetDevice(&dev);
  int v = 0;
  cudaMemcpy(&v, attn_bwd_status(dev), sizeof(int), cudaMemcpyDeviceToHost);
  int z = 0;
  if (v) cudaMemcpy(attn_bwd_status(dev), &z, sizeof(int), cudaMemcpyHostToDevice);
  return v;
}

// q, k, v, dout: (B, H, T, 64) bf16 contiguous; lse, delta: (B, H, T) fp32.  Returns dq (fp32), dk, dv (bf16).
std::vector<torch::Tensor> attn_bwd_tc(torch::Tensor q, torch::Tensor k, torch::Tensor v, torch::Tensor dout, torch::Tensor lse,
                                       torch::Tensor delta, int64_t window, double scale) {
  const c10::cuda::CUDAGuard guard(q.device());
  TORCH_CHECK(q.dim() == 4 && q.size(3) == AB_HD && q.scalar_type() == torch::kBFloat16 && q.is_contiguous() &&
              k.is_contiguous() && v.is_contiguous() && dout.is_contiguous() && dout.scalar_type() == torch::kBFloat16 &&
              k.sizes() == q.sizes() && v.sizes() == q.sizes() && dout.sizes() == q.sizes(),
              "attn_bwd_tc: q, k, v, dout (B, H, T, 64) bf16 contiguous");
  TORCH_CHECK(lse.is_contiguous() && delta.is_contiguous() && lse.scalar_type() == torch::kFloat32 &&
              delta.scalar_type() == torch::kFloat32, "attn_bwd_tc: lse, delta fp32 contiguous");
  const int B = q.size(0), H = q.size(1), T = q.size(2);
  auto dq = torch::zeros({B, H, T, AB_HD}, q.options().dtype(torch::kFloat32));
  auto dk = torch::zeros_like(q);
  auto dv = torch::zeros_like(q);
  if (B * H * T == 0) return {dq, dk, dv};
  const uint64_t BH = (uint64_t)B * H;
  auto mk = [&](const torch::Tensor& t) { return make_tmap_bf16(t.data_ptr(), AB_HD, T, BH, AB_HD, (uint64_t)T * AB_HD, 64, AB_T); };
  CUtensorMap tq = mk(q), tk = mk(k), tv = mk(v), tdo = mk(dout);
  AttnBwdParams p{};
  p.T = T;
  p.window = (window > 0 && window < T) ? (int)window : 0;
  p.scale = (float)scale;
  p.scale_log2 = (float)(scale * 1.4426950408889634);
  p.lse = lse.data_ptr<float>();
  p.delta = delta.data_ptr<float>();
  p.dq = dq.data_ptr<float>();
  p.dk = reinterpret_cast<bf16*>(dk.data_ptr());
  p.dv = reinterpret_cast<bf16*>(dv.data_ptr());
  int dev = 0;
  cudaGetDevice(&dev);
  p.status = attn_bwd_status(dev);
  static bool attr = false;
  if (!attr) {
    TORCH_CHECK(cudaFuncSetAttribute(attn_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AB_SMEM) == cudaSuccess,
                "cannot raise dynamic shared memory for the attention backward kernel");
    attr = true;
  }
  dim3 grid((T + AB_T - 1) / AB_T, (unsigned)BH);
  attn_bwd_kernel<<<grid, AB_THREADS, AB_SMEM, at::cuda::getCurrentCUDAStream()>>>(tq, tk, tv, tdo, p);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {dq, dk, dv};
}

}  // namespace mb
