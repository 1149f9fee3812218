// Causal / sliding-window attention forward on the tcgen05 tensor cores (head dim 64, bf16 in, fp32 softmax).
//
// One CTA per (128-query tile, batch*head).  Roles: warp 0 = TMA producer (Q once, K/V tiles through a 2-stage
// ring), warp 1 = MMA issuer, warps 2..5 = softmax (thread = one query row, TMEM lane quarter = warp % 4).
// Per 128-key tile:  S = Q Kt  (tcgen05.mma 128x128x64 into TMEM columns 0..127)
//                    softmax warps read S, apply scale / causal / window mask, online max and sum, write P (bf16)
//                    into shared memory in the canonical K-major 128-byte-swizzled layout
//                    O_tile = P V  (tcgen05.mma 128x64x128, V as the MN-major operand, TMEM columns 128..191)
//                    softmax warps fold O_tile into the per-row register accumulator with the rescale factor.
// The block list comes from window arithmetic (first tile = the one holding q0 - window + 1, last = the diagonal):
// no mask tensor exists.  Every mbarrier wait is bounded; on timeout the status word is set, roles stop, TMEM is
// freed and the kernel returns.  Backward is not in this file.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda.h>

#include "common.cuh"

namespace mb {

CUtensorMap make_tmap_bf16(const void* base, uint64_t inner, uint64_t rows, uint64_t groups, uint64_t row_pitch_el,
                           uint64_t group_pitch_el, uint32_t box_inner, uint32_t box_rows);

constexpr int AT_BQ = 128, AT_BK = 128, AT_HD = 64, AT_THREADS = 192;
constexpr int AT_Q_BYTES = AT_BQ * AT_HD * 2;            // 16 KB
constexpr int AT_K_BYTES = AT_BK * AT_HD * 2;            // 16 KB
constexpr int AT_V_BYTES = AT_BK * AT_HD * 2;            // 16 KB (two 64-key boxes of 8 KB)
constexpr int AT_P_BYTES = AT_BQ * AT_BK * 2;            // 32 KB (two 64-wide K atoms of 16 KB)
constexpr int AT_SMEM = AT_Q_BYTES + 2 * (AT_K_BYTES + AT_V_BYTES) + AT_P_BYTES + 256;   // 112.25 KB: two CTAs per SM

struct AttnParams {
  int T, window;            // window 0 = plain causal
  float scale_log2;         // 1/sqrt(hd) * log2(e)
  bf16* o;                  // (BH, T, 64)
  float* lse;               // (BH, T), natural log
  int* status;
};

__global__ void __launch_bounds__(AT_THREADS, 2)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const AttnParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];       // swizzle atoms are 1024 bytes: the base itself is aligned
  if (threadIdx.x == 0 && (smem_u32(smem) & 1023u)) atomicCAS(p.status, 0, ST_BAD_ARG);
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + AT_Q_BYTES;                          // 2 stages
  uint8_t* sV = sK + 2 * AT_K_BYTES;                      // 2 stages
  uint8_t* sP = sV + 2 * AT_V_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + AT_P_BYTES);
  uint64_t* q_full = bars;            // 1
  uint64_t* kv_full = bars + 1;       // 2
  uint64_t* kv_empty = bars + 3;      // 2
  uint64_t* s_full = bars + 5;        // S ready in TMEM
  uint64_t* p_full = bars + 6;        // P ready in shared memory (4 warp arrivals)
  uint64_t* o_full = bars + 7;        // O tile ready in TMEM
  uint64_t* sp_free = bars + 8;       // S, P and the O tile consumed (4 warp arrivals)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 9);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = (int)gridDim.x - 1 - (int)blockIdx.x;    // long (late) query tiles first
  const int bh = blockIdx.y;
  const int q0 = qt * AT_BQ;
  const int last_kt = min(qt, (p.T - 1) / AT_BK);
  const int first_kt = p.window > 0 ? max(0, (q0 - p.window + 1) / AT_BK) : 0;
  const int n_kt = last_kt - first_kt + 1;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); }
    mbar_init(s_full, 1); mbar_init(p_full, 4); mbar_init(o_full, 1); mbar_init(sp_free, 4);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base, tO = tmem_base + 128;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(q_full, AT_Q_BYTES);
      tma_load_3d(sQ, &tmQ, q_full, 0, q0, bh);
      for (int i = 0; i < n_kt; ++i) {
        const int s = i & 1;
        if (!mbar_wait(&kv_empty[s], ((i >> 1) & 1) ^ 1, abort_flag)) { atomicCAS(p.status, 0, ST_WAIT_EMPTY); *abort_flag = 1; break; }
        const int k0 = (first_kt + i) * AT_BK;
        mbar_expect_tx(&kv_full[s], AT_K_BYTES + AT_V_BYTES);
        tma_load_3d(sK + s * AT_K_BYTES, &tmK, &kv_full[s], 0, k0, bh);
        tma_load_3d(sV + s * AT_V_BYTES, &tmV, &kv_full[s], 0, k0, bh);
        tma_load_3d(sV + s * AT_V_BYTES + 8192, &tmV, &kv_full[s], 0, k0 + 64, bh);
      }
      if (*abort_flag) { for (int i = 0; i < 2000; ++i) __nanosleep(1000); }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_qk = idesc_bf16(128, 128, 0u, 0u);
      const uint32_t idesc_pv = idesc_bf16(128, 64, 0u, 1u);
      bool ok = mbar_wait(q_full, 0, abort_flag);
      if (!ok) { atomicCAS(p.status, 0, ST_WAIT_FULL); *abort_flag = 1; }
      for (int i = 0; i < n_kt && ok; ++i) {
        const int s = i & 1;
        if (!mbar_wait(&kv_full[s], (i >> 1) & 1, abort_flag)) { atomicCAS(p.status, 0, ST_WAIT_FULL); *abort_flag = 1; break; }
        if (i > 0 && !mbar_wait(sp_free, (i - 1) & 1, abort_flag)) { atomicCAS(p.status, 0, ST_WAIT_TMEM_EMPTY); *abort_flag = 1; break; }
        tc_fence_after();
        const uint32_t aQ = smem_u32(sQ), bK = smem_u32(sK + s * AT_K_BYTES);
#pragma unroll
        for (int k = 0; k < AT_HD / 16; ++k)
          umma_bf16(tS, smem_desc_sw128(aQ + k * 32, 0, 1024), smem_desc_sw128(bK + k * 32, 0, 1024), idesc_qk, k > 0 ? 1u : 0u);
        umma_commit(s_full);
        if (!mbar_wait(p_full, i & 1, abort_flag)) { atomicCAS(p.status, 0, ST_WAIT_TMEM_FULL); *abort_flag = 1; break; }
        tc_fence_after();
        const uint32_t aP = smem_u32(sP), bV = smem_u32(sV + s * AT_V_BYTES);
#pragma unroll
        for (int k = 0; k < AT_BK / 16; ++k) {
          const uint32_t ap = aP + (k >> 2) * 16384 + (k & 3) * 32;          // K-major P: two 64-key atoms
          const uint32_t bv = bV + (k >> 2) * 8192 + (k & 3) * 2048;         // MN-major V: two 64-key boxes, 16 key rows per step
          umma_bf16(tO, smem_desc_sw128(ap, 0, 1024), smem_desc_sw128(bv, 8192, 1024), idesc_pv, k > 0 ? 1u : 0u);
        }
        umma_commit(o_full);
        umma_commit(&kv_empty[s]);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + accumulation (one row per thread)
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const int qi = q0 + row;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    float m = -INFINITY, l = 0.f;
    float acc[AT_HD];
#pragma unroll
    for (int j = 0; j < AT_HD; ++j) acc[j] = 0.f;
    bool ok = true;
    for (int i = 0; i < n_kt && ok; ++i) {
      const int k0 = (first_kt + i) * AT_BK;
      if (!mbar_wait(s_full, i & 1, abort_flag)) { if (lane == 0) { atomicCAS(p.status, 0, ST_WAIT_TMEM_FULL); *abort_flag = 1; } ok = false; break; }
      tc_fence_after();
      // which key columns this row may see
      const int hi = min(qi, p.T - 1) - k0;                                   // last visible column (may be < 0)
      const int lo = p.window > 0 ? max(0, qi - p.window + 1 - k0) : 0;       // first visible column
      float mx = -INFINITY;
      uint32_t r[32];
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        __syncwarp();
        tmem_ld32(tS + lane_base + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int col = c * 32 + j;
          const float v = (col >= lo && col <= hi) ? __uint_as_float(r[j]) * p.scale_log2 : -INFINITY;
          mx = fmaxf(mx, v);
        }
      }
      const float m_new = fmaxf(m, mx);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = (m == -INFINITY) ? 0.f : exp2f(m - m_use);
      float rs = 0.f;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        __syncwarp();
        tmem_ld32(tS + lane_base + c * 32, r);
        tmem_ld_wait();
        uint32_t packed[16];
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          const int col = c * 32 + j;
          const float v0 = (col >= lo && col <= hi) ? exp2f(__uint_as_float(r[j]) * p.scale_log2 - m_use) : 0.f;
          const float v1 = (col + 1 >= lo && col + 1 <= hi) ? exp2f(__uint_as_float(r[j + 1]) * p.scale_log2 - m_use) : 0.f;
          const uint32_t pk = pack_bf16(v0, v1);
          packed[j >> 1] = pk;
          const float2 back = unpack_bf16(pk);                                // the sum uses the rounded values the MMA sees
          rs += back.x + back.y;
        }
        // 32 columns = 64 bytes = four 16-byte chunks of this row, 128-byte swizzle inside the 64-key atom
        const int atom = c >> 1;
        uint8_t* rowp = sP + atom * 16384 + row * 128;
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const int chunk = (c & 1) * 4 + q4;
          *reinterpret_cast<uint4*>(rowp + ((chunk ^ (row & 7)) << 4)) =
              make_uint4(packed[q4 * 4], packed[q4 * 4 + 1], packed[q4 * 4 + 2], packed[q4 * 4 + 3]);
        }
      }
      l = l * alpha + rs;
      m = m_new;
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");            // P is read by the tensor core (async proxy)
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
      if (!mbar_wait(o_full, i & 1, abort_flag)) { if (lane == 0) { atomicCAS(p.status, 0, ST_WAIT_TMEM_FULL); *abort_flag = 1; } ok = false; break; }
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        __syncwarp();
        tmem_ld32(tO + lane_base + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[c * 32 + j] = acc[c * 32 + j] * alpha + __uint_as_float(r[j]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(sp_free);
    }
    if (ok && qi < p.T) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      bf16* orow = p.o + ((long long)bh * p.T + qi) * AT_HD;
#pragma unroll
      for (int j = 0; j < AT_HD; j += 8)
        *reinterpret_cast<uint4*>(orow + j) =
            make_uint4(pack_bf16(acc[j] * inv, acc[j + 1] * inv), pack_bf16(acc[j + 2] * inv, acc[j + 3] * inv),
                       pack_bf16(acc[j + 4] * inv, acc[j + 5] * inv), pack_bf16(acc[j + 6] * inv, acc[j + 7] * inv));
      p.lse[(long long)bh * p.T + qi] = (l > 0.f) ? (m + log2f(l)) * 0.6931471805599453f : -INFINITY;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
}

static int* attn_status(int device) {
  static int* words[16] = {nullptr};
  if (!words[device]) {
    TORCH_CHECK(cudaMalloc(&words[device], sizeof(int)) == cudaSuccess, "status word alloc failed");
    cudaMemset(words[device], 0, sizeof(int));
  }
  return words[device];
}

int64_t attn_status_read() {
  int dev = 0;
  cudaGetDevice(&dev);
  int v = 0;
  cudaMemcpy(&v, attn_status(dev), sizeof(int), cudaMemcpyDeviceToHost);
  int z = 0;
  if (v) cudaMemcpy(attn_status(dev), &z, sizeof(int), cudaMemcpyHostToDevice);
  return v;
}

// q, k, v: (B, H, T, 64) bf16 contiguous (RoPE already applied).  Returns o (B, H, T, 64) bf16 and lse (B, H, T) fp32.
std::vector<torch::Tensor> attn_fwd_tc(torch::Tensor q, torch::Tensor k, torch::Tensor v, int64_t window, double scale) {
  const c10::cuda::CUDAGuard guard(q.device());
  TORCH_CHECK(q.dim() == 4 && q.size(3) == AT_HD && q.scalar_type() == torch::kBFloat16 && q.is_contiguous() &&
              k.is_contiguous() && v.is_contiguous() && k.sizes() == q.sizes() && v.sizes() == q.sizes(),
              "attn_fwd_tc: q, k, v (B, H, T, 64) bf16 contiguous");
  const int B = q.size(0), H = q.size(1), T = q.size(2);
  auto o = torch::empty_like(q);
  auto lse = torch::empty({B, H, T}, q.options().dtype(torch::kFloat32));
  if (B * H * T == 0) return {o, lse};
  const uint64_t BH = (uint64_t)B * H;
  CUtensorMap tq = make_tmap_bf16(q.data_ptr(), AT_HD, T, BH, AT_HD, (uint64_t)T * AT_HD, 64, AT_BQ);
  CUtensorMap tk = make_tmap_bf16(k.data_ptr(), AT_HD, T, BH, AT_HD, (uint64_t)T * AT_HD, 64, AT_BK);
  CUtensorMap tv = make_tmap_bf16(v.data_ptr(), AT_HD, T, BH, AT_HD, (uint64_t)T * AT_HD, 64, 64);
  AttnParams p{};
  p.T = T;
  p.window = (window > 0 && window < T) ? (int)window : 0;
  p.scale_log2 = (float)(scale * 1.4426950408889634);
  p.o = reinterpret_cast<bf16*>(o.data_ptr());
  p.lse = lse.data_ptr<float>();
  int dev = 0;
  cudaGetDevice(&dev);
  p.status = attn_status(dev);
  static bool attr = false;
  if (!attr) {
    TORCH_CHECK(cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AT_SMEM) == cudaSuccess,
                "cannot raise dynamic shared memory for the attention kernel");
    attr = true;
  }
  dim3 grid((T + AT_BQ - 1) / AT_BQ, (unsigned)BH);
  attn_fwd_kernel<<<grid, AT_THREADS, AT_SMEM, at::cuda::getCurrentCUDAStream()>>>(tq, tk, tv, p);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {o, lse};
}

}  // namespace mb
