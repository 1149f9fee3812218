// Peer-memory kernels over NVLink 5 / NVSwitch: bounded device-side barrier on symmetric flags, one-shot gradient
// all-reduce by plain peer loads/stores or by NVLS multimem (reduction inside the switch), and the binding of the
// segmented tcgen05 GEMM whose A tiles come from peer GPUs' buffers and whose result rows go to the owners' buffers.
// No TMA multicast anywhere: remote tiles are fetched by each CTA with plain (non-multicast) TMA loads or ld.global.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "common.cuh"

namespace mb {

static inline cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream(); }

struct PeerPtrs { void* p[8]; };

// ------------------------------------------------------------------------------------------------ barrier
// flags: symmetric uint32 array per rank, slot [channel * 8 + src] counts arrivals of rank `src`; slot
// [128 + channel] of a rank's own array counts its own barriers on that channel (the epoch lives on the device, so a
// captured CUDA graph replays correctly).  Every rank adds 1 to its slot on every peer (release, system scope), then
// waits (acquire) until every peer's slot on its own array reaches the epoch.  The wait is bounded; on timeout
// status[0] = ST_WAIT_PEER and the kernel returns.
__global__ void peer_barrier_kernel(PeerPtrs flags, int rank, int world, int channel, int* status,
                                    unsigned long long spin_limit) {
  __shared__ unsigned epoch_sh;
  if (threadIdx.x == 0) epoch_sh = atomicAdd(reinterpret_cast<unsigned*>(flags.p[rank]) + 128 + channel, 1u) + 1u;
  __syncthreads();
  const unsigned epoch = epoch_sh;
  const int q = threadIdx.x;
  if (q >= world) return;
  __threadfence_system();
  unsigned* remote = reinterpret_cast<unsigned*>(flags.p[q]) + channel * 8 + rank;
  asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(remote) : "memory");
  const unsigned* mine = reinterpret_cast<const unsigned*>(flags.p[rank]) + channel * 8 + q;
  unsigned v = 0;
  unsigned long long i = 0;
  for (; i < spin_limit; ++i) {
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
    if ((int)(v - epoch) >= 0) break;
    __nanosleep(64);
  }
  if (i >= spin_limit) atomicCAS(status, 0, ST_WAIT_PEER);
  __threadfence_system();
}

static int* peer_status(int device) {
  static int* words[16] = {nullptr};
  if (!words[device]) {
    TORCH_CHECK(cudaMalloc(&words[device], sizeof(int)) == cudaSuccess, "status word alloc failed");
    cudaMemset(words[device], 0, sizeof(int));
  }
  return words[device];
}

void peer_barrier(std::vector<int64_t> flag_ptrs, int64_t rank, int64_t channel, double timeout_ms) {
  const int W = (int)flag_ptrs.size();
  TORCH_CHECK(W >= 1 && W <= 8, "peer_barrier: 1..8 ranks");
  PeerPtrs f{};
  for (int i = 0; i < W; ++i) f.p[i] = reinterpret_cast<void*>(flag_ptrs[i]);
  int dev = 0;
  cudaGetDevice(&dev);
  // one poll is ~0.2 us (64 ns sleep + a system-scope load)
  unsigned long long limit = (unsigned long long)(timeout_ms * 1e3 * 5.0);
  TORCH_CHECK(channel >= 0 && channel < 16, "peer_barrier: channel 0..15");
  peer_barrier_kernel<<<1, 32, 0, cur_stream()>>>(f, (int)rank, W, (int)channel, peer_status(dev), limit);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

int64_t peer_status_read() {
  int dev = 0;
  cudaGetDevice(&dev);
  int v = 0;
  cudaMemcpy(&v, peer_status(dev), sizeof(int), cudaMemcpyDeviceToHost);
  int z = 0;
  if (v) cudaMemcpy(peer_status(dev), &z, sizeof(int), cudaMemcpyHostToDevice);
  return v;
}

// ------------------------------------------------------------------------------------------------ expert-row gather
// dst (G, W*C, d) <- rows of this rank's G experts from every rank's dispatch buffer src_s (E, C, d):
//   dst[g, s*C + c, :] = src_s[g_off + g, c, :]
// One kernel over all W sources (plain 16-byte peer loads over NVLink, four in flight per thread) instead of W
// back-to-back copies; sources are walked starting at this rank, so the W ranks read from W different GPUs first.
__global__ void peer_gather_kernel(PeerPtrs src, uint4* __restrict__ dst, int W, int rank, long long G, long long C,
                                   long long d16, long long g_off) {
  const long long per_src = G * C * d16;
  const long long total = per_src * W;
  const long long stride = (long long)gridDim.x * blockDim.x;
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  for (; i + 3 * stride < total; i += 4 * stride) {
    uint4 v[4];
    long long o[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const long long j = i + u * stride;
      const int si = (int)(j / per_src);
      const int s = (rank + si) % W;
      const long long r = j - si * per_src;
      const long long g = r / (C * d16), rc = r - g * (C * d16);
      v[u] = *(reinterpret_cast<const uint4*>(src.p[s]) + (g_off + g) * C * d16 + rc);
      o[u] = (g * W * C + (long long)s * C) * d16 + rc;
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) dst[o[u]] = v[u];
  }
  for (; i < total; i += stride) {
    const int si = (int)(i / per_src);
    const int s = (rank + si) % W;
    const long long r = i - si * per_src;
    const long long g = r / (C * d16), rc = r - g * (C * d16);
    dst[(g * W * C + (long long)s * C) * d16 + rc] = *(reinterpret_cast<const uint4*>(src.p[s]) + (g_off + g) * C * d16 + rc);
  }
}

// src_ptrs: base pointers of the W ranks' (E, C, d) bf16 buffers; dst: (G, W*C, d) bf16, contiguous.
void peer_gather(std::vector<int64_t> src_ptrs, torch::Tensor dst, int64_t rank, int64_t C, int64_t g_off) {
  const int W = (int)src_ptrs.size();
  TORCH_CHECK(W >= 1 && W <= 8, "peer_gather: 1..8 ranks");
  TORCH_CHECK(dst.is_cuda() && dst.dim() == 3 && dst.is_contiguous() && dst.scalar_type() == torch::kBFloat16, "peer_gather: dst (G, W*C, d) bf16");
  const long long G = dst.size(0), d = dst.size(2);
  TORCH_CHECK(dst.size(1) == W * C && d % 8 == 0, "peer_gather: dst rows = W*C, d % 8 == 0");
  const c10::cuda::CUDAGuard guard(dst.device());
  PeerPtrs sp{};
  for (int i = 0; i < W; ++i) {
    sp.p[i] = reinterpret_cast<void*>(src_ptrs[i]);
    TORCH_CHECK((src_ptrs[i] & 15) == 0, "peer_gather: 16-byte aligned buffers");
  }
  const long long total = (long long)W * G * C * (d / 8);
  if (total == 0) return;
  const int grid = (int)std::min<long long>((total + 1023) / 1024, 148 * 8);
  peer_gather_kernel<<<grid, 256, 0, cur_stream()>>>(sp, reinterpret_cast<uint4*>(dst.data_ptr()), W, (int)rank, G, C, d / 8, g_off);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------------------ all-reduce (P2P)
// Rank r owns the r-th slice of [0, n): it loads that slice from every rank's `in` buffer, sums in fp32, scales, and
// stores the result into every rank's `out` buffer (reduce-scatter and all-gather in one kernel, 16-byte accesses).
template <bool BF16>
__global__ void allreduce_p2p_kernel(PeerPtrs in, PeerPtrs out, long long begin, long long end, int world, float scale) {
  constexpr int PER = BF16 ? 8 : 4;                   // elements per 16 bytes
  const long long n16 = (end - begin) / PER;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n16; i += (long long)gridDim.x * blockDim.x) {
    const long long off = begin + i * PER;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll 1
    for (int q = 0; q < world; ++q) {
      if (BF16) {
        uint4 u = *reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(in.p[q]) + off);
        const uint32_t* w = reinterpret_cast<const uint32_t*>(&u);
#pragma unroll
        for (int j = 0; j < 4; ++j) { float2 f = unpack_bf16(w[j]); acc[2 * j] += f.x; acc[2 * j + 1] += f.y; }
      } else {
        float4 f = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(in.p[q]) + off);
        acc[0] += f.x; acc[1] += f.y; acc[2] += f.z; acc[3] += f.w;
      }
    }
    if (BF16) {
      uint4 u = make_uint4(pack_bf16(acc[0] * scale, acc[1] * scale), pack_bf16(acc[2] * scale, acc[3] * scale),
                           pack_bf16(acc[4] * scale, acc[5] * scale), pack_bf16(acc[6] * scale, acc[7] * scale));
      for (int q = 0; q < world; ++q) *reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(out.p[q]) + off) = u;
    } else {
      float4 f = make_float4(acc[0] * scale, acc[1] * scale, acc[2] * scale, acc[3] * scale);
      for (int q = 0; q < world; ++q) *reinterpret_cast<float4*>(reinterpret_cast<float*>(out.p[q]) + off) = f;
    }
  }
}

// ------------------------------------------------------------------------------------------------ all-reduce (NVLS)
// Same contract through the NVSwitch multicast addresses: multimem.ld_reduce sums the slice across all GPUs inside
// the switch (fp32 accumulation), multimem.st broadcasts the scaled result to all of them.
template <bool BF16>
__global__ void allreduce_nvls_kernel(const void* mc_in, void* mc_out, long long begin, long long end, float scale) {
  constexpr int PER = BF16 ? 8 : 4;
  const long long n16 = (end - begin) / PER;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n16; i += (long long)gridDim.x * blockDim.x) {
    const long long off = begin + i * PER;
    if (BF16) {
      const bf16* src = reinterpret_cast<const bf16*>(mc_in) + off;
      bf16* dst = reinterpret_cast<bf16*>(mc_out) + off;
      uint32_t a, b, c, d;
      asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                   : "=r"(a), "=r"(b), "=r"(c), "=r"(d) : "l"(src) : "memory");
      float2 f0 = unpack_bf16(a), f1 = unpack_bf16(b), f2 = unpack_bf16(c), f3 = unpack_bf16(d);
      a = pack_bf16(f0.x * scale, f0.y * scale); b = pack_bf16(f1.x * scale, f1.y * scale);
      c = pack_bf16(f2.x * scale, f2.y * scale); d = pack_bf16(f3.x * scale, f3.y * scale);
      asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1,%2,%3,%4};" ::"l"(dst), "r"(a), "r"(b), "r"(c), "r"(d)
                   : "memory");
    } else {
      const float* src = reinterpret_cast<const float*>(mc_in) + off;
      float* dst = reinterpret_cast<float*>(mc_out) + off;
      float a, b, c, d;
      asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
                   : "=f"(a), "=f"(b), "=f"(c), "=f"(d) : "l"(src) : "memory");
      a *= scale; b *= scale; c *= scale; d *= scale;
      asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(dst), "f"(a), "f"(b), "f"(c), "f"(d)
                   : "memory");
    }
  }
}

// ------------------------------------------------------------------------------------------------ reduce-scatter / all-gather halves
// reduce_to_local: dst[i] = scale * sum_q in_q[offset + i] for i in [0, numel) - this rank's slice of a staged
// gradient summed over all ranks into LOCAL memory (the reduce-scatter half; multimem.ld_reduce when `mc_in`).
template <bool BF16>
__global__ void reduce_to_local_kernel(PeerPtrs in, const void* mc_in, void* __restrict__ dst, long long offset, long long numel,
                                       int world, float scale) {
  constexpr int PER = BF16 ? 8 : 4;
  const long long n16 = numel / PER;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n16; i += (long long)gridDim.x * blockDim.x) {
    const long long off = offset + i * PER;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (mc_in) {
      if (BF16) {
        uint32_t a, b, c, d;
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                     : "=r"(a), "=r"(b), "=r"(c), "=r"(d) : "l"(reinterpret_cast<const bf16*>(mc_in) + off) : "memory");
        float2 f0 = unpack_bf16(a), f1 = unpack_bf16(b), f2 = unpack_bf16(c), f3 = unpack_bf16(d);
        acc[0] = f0.x; acc[1] = f0.y; acc[2] = f1.x; acc[3] = f1.y; acc[4] = f2.x; acc[5] = f2.y; acc[6] = f3.x; acc[7] = f3.y;
      } else {
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
                     : "=f"(acc[0]), "=f"(acc[1]), "=f"(acc[2]), "=f"(acc[3]) : "l"(reinterpret_cast<const float*>(mc_in) + off) : "memory");
      }
    } else {
#pragma unroll 1
      for (int q = 0; q < world; ++q) {
        if (BF16) {
          uint4 u = *reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(in.p[q]) + off);
          const uint32_t* w = reinterpret_cast<const uint32_t*>(&u);
#pragma unroll
          for (int j = 0; j < 4; ++j) { float2 f = unpack_bf16(w[j]); acc[2 * j] += f.x; acc[2 * j + 1] += f.y; }
        } else {
          float4 f = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(in.p[q]) + off);
          acc[0] += f.x; acc[1] += f.y; acc[2] += f.z; acc[3] += f.w;
        }
      }
    }
    if (BF16) {
      *reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(dst) + i * PER) =
          make_uint4(pack_bf16(acc[0] * scale, acc[1] * scale), pack_bf16(acc[2] * scale, acc[3] * scale),
                     pack_bf16(acc[4] * scale, acc[5] * scale), pack_bf16(acc[6] * scale, acc[7] * scale));
    } else {
      *reinterpret_cast<float4*>(reinterpret_cast<float*>(dst) + i * PER) =
          make_float4(acc[0] * scale, acc[1] * scale, acc[2] * scale, acc[3] * scale);
    }
  }
}

void peer_reduce_to_local(std::vector<int64_t> in_ptrs, int64_t mc_in, torch::Tensor dst, int64_t offset, double scale) {
  const int W = (int)in_ptrs.size();
  TORCH_CHECK(W >= 1 && W <= 8, "peer_reduce_to_local: 1..8 ranks");
  TORCH_CHECK(dst.is_cuda() && dst.is_contiguous() && (dst.scalar_type() == torch::kBFloat16 || dst.scalar_type() == torch::kFloat32),
              "peer_reduce_to_local: contiguous bf16 / fp32 destination");
  const bool bf = dst.scalar_type() == torch::kBFloat16;
  const int per = bf ? 8 : 4;
  const long long numel = dst.numel();
  TORCH_CHECK(offset % per == 0 && numel % per == 0, "peer_reduce_to_local: 16-byte units");
  if (!numel) return;
  const c10::cuda::CUDAGuard guard(dst.device());
  PeerPtrs in{};
  for (int i = 0; i < W; ++i) in.p[i] = reinterpret_cast<void*>(in_ptrs[i]);
  const int grid = (int)std::min<long long>((numel / per + 255) / 256, 148 * 4);
  if (bf) reduce_to_local_kernel<true><<<grid, 256, 0, cur_stream()>>>(in, reinterpret_cast<const void*>(mc_in), dst.data_ptr(), offset, numel, W, (float)scale);
  else reduce_to_local_kernel<false><<<grid, 256, 0, cur_stream()>>>(in, reinterpret_cast<const void*>(mc_in), dst.data_ptr(), offset, numel, W, (float)scale);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

// broadcast_from_local: out_q[offset + i] = this rank's out[offset + i] for every OTHER rank q (the all-gather half:
// this rank's rows of an updated weight to all peers; one multimem.st per 16 bytes when `mc_out`, which also rewrites
// the local copy with the same bytes).
__global__ void broadcast_from_local_kernel(PeerPtrs out, void* mc_out, long long offset16, long long n16, int world, int rank) {
  const uint4* src = reinterpret_cast<const uint4*>(out.p[rank]) + offset16;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n16; i += (long long)gridDim.x * blockDim.x) {
    const uint4 v = src[i];
    if (mc_out) {
      asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(reinterpret_cast<uint4*>(mc_out) + offset16 + i),
                   "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w)) : "memory");
    } else {
      for (int q = 1; q < world; ++q) {
        const int t = (rank + q) % world;
        *(reinterpret_cast<uint4*>(out.p[t]) + offset16 + i) = v;
      }
    }
  }
}

// out_ptrs: per-rank base pointers of one symmetric buffer; [offset_bytes, offset_bytes + nbytes) of this rank's copy
// goes to every rank.
void peer_broadcast_from_local(std::vector<int64_t> out_ptrs, int64_t mc_out, int64_t offset_bytes, int64_t nbytes, int64_t rank) {
  const int W = (int)out_ptrs.size();
  TORCH_CHECK(W >= 1 && W <= 8, "peer_broadcast_from_local: 1..8 ranks");
  TORCH_CHECK(offset_bytes % 16 == 0 && nbytes % 16 == 0, "peer_broadcast_from_local: 16-byte units");
  if (!nbytes || W == 1) return;
  PeerPtrs out{};
  for (int i = 0; i < W; ++i) out.p[i] = reinterpret_cast<void*>(out_ptrs[i]);
  const long long n16 = nbytes / 16;
  const int grid = (int)std::min<long long>((n16 + 255) / 256, 148 * 4);
  broadcast_from_local_kernel<<<grid, 256, 0, cur_stream()>>>(out, reinterpret_cast<void*>(mc_out), offset_bytes / 16, n16, W, (int)rank);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

// in/out: per-rank base pointers of two symmetric buffers; the region is [offset, offset + numel) elements of `bf16` or
// fp32.  mc_in / mc_out non-zero selects the NVLS path.  The caller brackets this with peer barriers.
void peer_allreduce(std::vector<int64_t> in_ptrs, std::vector<int64_t> out_ptrs, int64_t mc_in, int64_t mc_out, int64_t offset,
                    int64_t numel, bool is_bf16, int64_t rank, double scale) {
  const int W = (int)in_ptrs.size();
  TORCH_CHECK(W >= 1 && W <= 8 && (int)out_ptrs.size() == W, "peer_allreduce: 1..8 ranks");
  const int per = is_bf16 ? 8 : 4;
  TORCH_CHECK(offset % per == 0, "peer_allreduce: region must start on a 16-byte boundary");
  // slice boundaries on 16-byte units; the last rank takes the tail, which must also be a whole number of units
  TORCH_CHECK(numel % per == 0, "peer_allreduce: region length must be a multiple of 16 bytes");
  const long long units = numel / per;
  const long long lo = offset + (units * rank / W) * per, hi = offset + (units * (rank + 1) / W) * per;
  if (hi <= lo) return;
  PeerPtrs in{}, out{};
  for (int i = 0; i < W; ++i) { in.p[i] = reinterpret_cast<void*>(in_ptrs[i]); out.p[i] = reinterpret_cast<void*>(out_ptrs[i]); }
  const long long n16 = (hi - lo) / per;
  const int grid = (int)std::min<long long>((n16 + 255) / 256, 148 * 4);
  if (mc_in && mc_out) {
    if (is_bf16) allreduce_nvls_kernel<true><<<grid, 256, 0, cur_stream()>>>(reinterpret_cast<const void*>(mc_in),
        reinterpret_cast<void*>(mc_out), lo, hi, (float)scale);
    else allreduce_nvls_kernel<false><<<grid, 256, 0, cur_stream()>>>(reinterpret_cast<const void*>(mc_in),
        reinterpret_cast<void*>(mc_out), lo, hi, (float)scale);
  } else {
    if (is_bf16) allreduce_p2p_kernel<true><<<grid, 256, 0, cur_stream()>>>(in, out, lo, hi, W, (float)scale);
    else allreduce_p2p_kernel<false><<<grid, 256, 0, cur_stream()>>>(in, out, lo, hi, W, (float)scale);
  }
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

}  // namespace mb
