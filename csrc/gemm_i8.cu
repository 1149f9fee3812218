// int8 GEMM on the tcgen05 tensor cores (`tcgen05.mma.kind::i8`, int32 accumulators in TMEM) with the dequantising
// epilogue of row-wise / column-wise symmetric quantisation:
//     out[g, m, n] = (sum_k a[g, m, k] * b[g, n, k]) * sa[g, m] * sb[g, n]
// a (G, M, K) and b (G, N, K) are int8, K contiguous (both K-major: 8-bit operands are fed as stored); sa / sb are the
// fp32 scales of the rows of a and of the rows of b.  This is the matmul of the reference's INT8_MM family and of its
// int8 frozen expert bank (int8mm.py:35-88, full2.py:919-958) at twice the bf16 tensor rate.
// Same skeleton as the single-CTA bf16 kernel: persistent, 128 x 256 tile, 128-byte k-blocks (128 int8) through a
// 4-stage TMA ring, one thread issues four K = 32 MMAs per k-block, accumulators double-buffered in TMEM, four
// epilogue warps.  Every wait is bounded and reports through the GEMM status word.
// Also here: the row quantiser (absmax / 127 scale, round to nearest) that produces a and sa from bf16 / fp32 rows.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda.h>

#include "common.cuh"

namespace mb {

CUtensorMap make_tmap(const void* base, int esz, uint64_t inner, uint64_t rows, uint64_t groups, uint64_t row_pitch_el,
                      uint64_t group_pitch_el, uint32_t box_inner, uint32_t box_rows, bool promote);
int* gemm_status_word(int device);

constexpr int I8_BM = 128, I8_BN = 256, I8_BK = 128, I8_STAGES = 4, I8_UK = 32, I8_THREADS = 192;
constexpr int I8_A_BYTES = I8_BM * I8_BK, I8_B_BYTES = I8_BN * I8_BK, I8_STAGE = I8_A_BYTES + I8_B_BYTES;
constexpr int I8_SMEM = I8_STAGES * I8_STAGE + 1024 + 256;

struct I8Params {
  int M, N, K, G;
  int m_tiles, n_tiles;
  const float* sa;          // (G, M)
  const float* sb;          // (G, N)
  void* out;                // (G, M, N) bf16 or fp32
  int out_f32;
  long long ldo, out_gs;
  int* status;
};

// Instruction descriptor, kind::i8: int32 accumulate (format 2), signed 8-bit A and B (format 1), both K-major.
__host__ __device__ __forceinline__ uint32_t idesc_s8(uint32_t M, uint32_t N) {
  return (2u << 4) | (1u << 7) | (1u << 10) | ((N >> 3) << 17) | ((M >> 4) << 24);
}
__device__ __forceinline__ void umma_s8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
      : "memory");
}

__global__ void __launch_bounds__(I8_THREADS, 1)
gemm_i8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const I8Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + I8_STAGES * I8_STAGE);
  uint64_t* empty = full + I8_STAGES;
  uint64_t* tfull = empty + I8_STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_kb = (p.K + I8_BK - 1) / I8_BK;
  const int per_g = p.m_tiles * p.n_tiles;
  const int total = p.G * per_g;

  if (threadIdx.x == 0) {
    for (int s = 0; s < I8_STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tfull[a], 1); mbar_init(&tempty[a], 4); }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
        const int g = t / per_g, r = t - g * per_g;
        const int mt = r % p.m_tiles, nt = r / p.m_tiles;          // row tiles of one column band back to back: B stays in L2
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag)) {
            atomicCAS(p.status, 0, ST_WAIT_EMPTY); *abort_flag = 1; ok = false; break;
          }
          uint8_t* sA = smem + stage * I8_STAGE;
          mbar_expect_tx(&full[stage], I8_STAGE);
          tma_load_3d(sA, &tmA, &full[stage], kb * I8_BK, mt * I8_BM, g);
          tma_load_3d(sA + I8_A_BYTES, &tmB, &full[stage], kb * I8_BK, nt * I8_BN, g);
          if (++stage == I8_STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);          // let copies already in flight land
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      const uint32_t idesc = idesc_s8(I8_BM, I8_BN);
      for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
        if (!mbar_wait(&tempty[acc], acc_phase ^ 1, abort_flag)) {
          atomicCAS(p.status, 0, ST_WAIT_TMEM_EMPTY); *abort_flag = 1; ok = false; break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * I8_BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag)) {
            atomicCAS(p.status, 0, ST_WAIT_FULL); *abort_flag = 1; ok = false; break;
          }
          tc_fence_after();
          const uint32_t sA = smem_u32(smem + stage * I8_STAGE), sB = sA + I8_A_BYTES;
#pragma unroll
          for (int k = 0; k < I8_BK / I8_UK; ++k)                      // 32 int8 = 32 bytes along the swizzled row
            umma_s8(d_tmem, smem_desc_sw128(sA + k * I8_UK, 0, 1024), smem_desc_sw128(sB + k * I8_UK, 0, 1024), idesc,
                    (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit(&empty[stage]);
          if (++stage == I8_STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&tfull[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
      const int g = t / per_g, r = t - g * per_g;
      const int mt = r % p.m_tiles, nt = r / p.m_tiles;
      if (!mbar_wait(&tfull[acc], acc_phase, abort_flag)) {
        if (lane == 0) { atomicCAS(p.status, 0, ST_WAIT_TMEM_FULL); *abort_flag = 1; }
        ok = false; break;
      }
      tc_fence_after();
      const int row = mt * I8_BM + q * 32 + lane;
      const bool row_ok = row < p.M;
      const float sa = row_ok ? p.sa[(long long)g * p.M + row] : 0.f;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * I8_BN;
#pragma unroll 1
      for (int c = 0; c < I8_BN / 32; ++c) {
        uint32_t rr[32];
        __syncwarp();
        tmem_ld32(taddr + c * 32, rr);
        tmem_ld_wait();
        const int col0 = nt * I8_BN + c * 32;
        if (row_ok && col0 < p.N) {
          const int nv = min(32, p.N - col0);
          const float* sbp = p.sb + (long long)g * p.N + col0;
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = j < nv ? static_cast<float>(static_cast<int>(rr[j])) * sa * sbp[j] : 0.f;
          const long long o0 = (long long)g * p.out_gs + (long long)row * p.ldo + col0;
          if (p.out_f32) {
            float* o = reinterpret_cast<float*>(p.out) + o0;
            if (nv == 32 && (p.ldo & 3) == 0) {
#pragma unroll
              for (int j = 0; j < 8; ++j) reinterpret_cast<float4*>(o)[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            } else {
              for (int j = 0; j < nv; ++j) o[j] = v[j];
            }
          } else {
            bf16* o = reinterpret_cast<bf16*>(p.out) + o0;
            if (nv == 32 && (p.ldo & 7) == 0) {
#pragma unroll
              for (int j = 0; j < 4; ++j)
                reinterpret_cast<uint4*>(o)[j] = make_uint4(pack_bf16(v[8 * j], v[8 * j + 1]), pack_bf16(v[8 * j + 2], v[8 * j + 3]),
                                                            pack_bf16(v[8 * j + 4], v[8 * j + 5]), pack_bf16(v[8 * j + 6], v[8 * j + 7]));
            } else {
              for (int j = 0; j < nv; ++j) o[j] = __float2bfloat16(v[j]);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// Row quantiser: q[r, :] = round(x[r, :] / s[r]), s[r] = max|x[r, :]| / 127 (at least 1e-12).  A warp per row.
template <typename T>
__global__ void quant_rows_i8_kernel(const T* __restrict__ x, signed char* __restrict__ q, float* __restrict__ s, long long R, int K) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  for (long long r = (long long)blockIdx.x * nw + warp; r < R; r += (long long)gridDim.x * nw) {
    const T* xr = x + r * K;
    float mx = 0.f;
    for (int c = lane; c < K; c += 32) mx = fmaxf(mx, fabsf(static_cast<float>(xr[c])));
    mx = warp_max(mx);
    const float sc = fmaxf(mx, 1e-12f) * (1.f / 127.f);     // as the PyTorch statement computes it (division by a scalar)
    signed char* qr = q + r * K;
    for (int c = lane; c < K; c += 32) {
      const float v = rintf(__fdiv_rn(static_cast<float>(xr[c]), sc));          // a true division: same ties as the oracle
      qr[c] = static_cast<signed char>(fminf(fmaxf(v, -127.f), 127.f));
    }
    if (lane == 0) s[r] = sc;
  }
}

std::vector<torch::Tensor> quant_rows_i8(torch::Tensor x) {
  const c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.is_cuda() && x.is_contiguous() && x.dim() >= 2, "quant_rows_i8: contiguous CUDA tensor (..., K)");
  TORCH_CHECK(x.scalar_type() == torch::kBFloat16 || x.scalar_type() == torch::kFloat32, "quant_rows_i8: bf16 or fp32");
  const int K = (int)x.size(-1);
  const long long R = x.numel() / std::max(K, 1);
  auto q = torch::empty(x.sizes(), x.options().dtype(torch::kInt8));
  auto ssz = x.sizes().vec();
  ssz.pop_back();
  auto s = torch::empty(ssz, x.options().dtype(torch::kFloat32));
  if (R == 0 || K == 0) return {q, s};
  const int grid = (int)std::max<long long>(1, std::min<long long>((R + 7) / 8, 148 * 8));
  auto st = at::cuda::getCurrentCUDAStream();
  if (x.scalar_type() == torch::kBFloat16)
    quant_rows_i8_kernel<bf16><<<grid, 256, 0, st>>>(reinterpret_cast<const bf16*>(x.data_ptr()), q.data_ptr<signed char>(),
                                                     s.data_ptr<float>(), R, K);
  else
    quant_rows_i8_kernel<float><<<grid, 256, 0, st>>>(x.data_ptr<float>(), q.data_ptr<signed char>(), s.data_ptr<float>(), R, K);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {q, s};
}

// a (G?, M, K) int8, b (G?, N, K) int8, sa (G?, M) fp32, sb (G?, N) fp32 -> (G?, M, N) bf16 (or fp32).
torch::Tensor gemm_i8(torch::Tensor a, torch::Tensor b, torch::Tensor sa, torch::Tensor sb, bool out_f32) {
  const c10::cuda::CUDAGuard guard(a.device());
  TORCH_CHECK(a.is_cuda() && b.is_cuda() && a.scalar_type() == torch::kInt8 && b.scalar_type() == torch::kInt8 &&
              a.is_contiguous() && b.is_contiguous(), "gemm_i8: contiguous int8 CUDA operands");
  TORCH_CHECK(a.dim() == b.dim() && (a.dim() == 2 || a.dim() == 3), "gemm_i8: (M,K) x (N,K) or (G,M,K) x (G,N,K)");
  const bool grouped = a.dim() == 3;
  const int G = grouped ? (int)a.size(0) : 1;
  const int M = (int)a.size(-2), K = (int)a.size(-1), N = (int)b.size(-2);
  TORCH_CHECK(b.size(-1) == K && (!grouped || b.size(0) == G), "gemm_i8: shapes");
  TORCH_CHECK(K % 16 == 0 && K >= 32, "gemm_i8: K must be a multiple of 16 (row pitch of a TMA operand)");
  TORCH_CHECK(sa.is_contiguous() && sb.is_contiguous() && sa.scalar_type() == torch::kFloat32 &&
              sb.scalar_type() == torch::kFloat32 && sa.numel() == (long long)G * M && sb.numel() == (long long)G * N,
              "gemm_i8: scales (G?,M) and (G?,N) fp32");
  auto opts = a.options().dtype(out_f32 ? torch::kFloat32 : torch::kBFloat16);
  auto out = grouped ? torch::empty({G, M, N}, opts) : torch::empty({M, N}, opts);
  if ((long long)G * M * N == 0) return out;
  I8Params p{};
  p.M = M; p.N = N; p.K = K; p.G = G;
  p.m_tiles = (M + I8_BM - 1) / I8_BM;
  p.n_tiles = (N + I8_BN - 1) / I8_BN;
  p.sa = sa.data_ptr<float>(); p.sb = sb.data_ptr<float>();
  p.out = out.data_ptr(); p.out_f32 = out_f32 ? 1 : 0;
  p.ldo = N; p.out_gs = (long long)M * N;
  int dev = 0;
  cudaGetDevice(&dev);
  p.status = gemm_status_word(dev);
  CUtensorMap tA = make_tmap(a.data_ptr(), 1, K, M, G, K, (uint64_t)M * K, I8_BK, I8_BM, true);
  CUtensorMap tB = make_tmap(b.data_ptr(), 1, K, N, G, K, (uint64_t)N * K, I8_BK, I8_BN, true);
  TORCH_CHECK(cudaFuncSetAttribute(gemm_i8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, I8_SMEM) == cudaSuccess,
              "gemm_i8: shared memory");
  int sms = 0;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int total = G * p.m_tiles * p.n_tiles;
  gemm_i8_kernel<<<std::min(total, sms), I8_THREADS, I8_SMEM, at::cuda::getCurrentCUDAStream()>>>(tA, tB, p);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return out;
}

}  // namespace mb
