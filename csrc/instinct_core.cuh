// Device kernels and the launch sequence of one Instinct step (torch-free; see instinct.cu for the maths).
#pragma once
#include "common.cuh"

namespace mb {

struct InstinctArgs {
  void* p;                 // weight (bf16 or fp32)
  const void* g;           // gradient
  void* m;                 // momentum
  float* w;                // exact fp32 copy of a bf16 weight, or nullptr
  int p_bf16, g_bf16, m_bf16;
  const float* gain;       // device scalar: gain of this weight on the current situation card
  const float* stake;      // device scalar
  const float* lr;         // device scalar: lr * scale
  float beta, wd;
  int sr;                  // stochastic rounding of bf16 stores
  const long long* seed;   // device step counter for the rounding hash
  unsigned salt;
  const bool* frozen;      // optional mask over the leading dimension: frozen slices keep their weights
  long long frozen_stride;
  long long E, R, C;
  // optional data-parallel reduction fused into the gradient load: peer gradient buffers of the same shape
  const void* peer_g[8];
  int n_peers;
  float g_scale;           // 1/world for an averaged gradient
};

__device__ __forceinline__ float ldv(const void* base, long long i, int is_bf16) {
  return is_bf16 ? __bfloat162float(reinterpret_cast<const bf16*>(base)[i]) : reinterpret_cast<const float*>(base)[i];
}
__device__ __forceinline__ float4 ldv4(const void* base, long long i, int is_bf16) {
  if (is_bf16) {
    uint2 u = *reinterpret_cast<const uint2*>(reinterpret_cast<const bf16*>(base) + i);
    float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y);
    return make_float4(a.x, a.y, b.x, b.y);
  }
  return *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + i);
}
__device__ __forceinline__ uint32_t lowbias32(uint32_t x) {
  x ^= x >> 16; x *= 0x7FEB352Du; x ^= x >> 15; x *= 0x846CA68Bu; x ^= x >> 16;
  return x;
}
__device__ __forceinline__ bf16 sr_round(float x, uint32_t r16) {
  uint32_t u = __float_as_uint(x);
  u = (u + r16) & 0xFFFF0000u;
  return __float2bfloat16(__uint_as_float(u));          // exact: low 16 bits are zero
}
__device__ __forceinline__ float gload(const InstinctArgs& a, long long i) {
  float v = ldv(a.g, i, a.g_bf16);
  for (int k = 0; k < a.n_peers; ++k) v += ldv(a.peer_g[k], i, a.g_bf16);
  return v * a.g_scale;
}
__device__ __forceinline__ float4 gload4(const InstinctArgs& a, long long i) {
  float4 v = ldv4(a.g, i, a.g_bf16);
  for (int k = 0; k < a.n_peers; ++k) {
    float4 q = ldv4(a.peer_g[k], i, a.g_bf16);
    v.x += q.x; v.y += q.y; v.z += q.z; v.w += q.w;
  }
  v.x *= a.g_scale; v.y *= a.g_scale; v.z *= a.g_scale; v.w *= a.g_scale;
  return v;
}
// sums of squares -> scales, in place: x <- 1 / (sqrt(x / count) + 1e-8); optional fold x <- x * fold[i]^2 first
// (fold already holds scales).  Tiny arrays (one value per row or per column).
static __global__ void instinct_finalize(float* __restrict__ x, long long n, float count, const float* __restrict__ fold) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float v = x[i];
    if (fold) { const float f = fold[i]; v *= f * f; }
    x[i] = 1.f / (sqrtf(v / count) + 1e-8f);
  }
}

static __global__ void instinct_mul(float* __restrict__ x, const float* __restrict__ y, long long n) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) x[i] *= y[i];
}

__device__ __forceinline__ float4 mom4(const InstinctArgs& a, long long i, float4& g) {
  g = gload4(a, i);
  const float4 mm = ldv4(a.m, i, a.m_bf16);
  const float b = a.beta, c = 1.f - a.beta;
  return make_float4(b * mm.x + c * g.x, b * mm.y + c * g.y, b * mm.z + c * g.z, b * mm.w + c * g.w);
}
__device__ __forceinline__ float mom1(const InstinctArgs& a, long long i, float& g) {
  g = gload(a, i);
  return a.beta * ldv(a.m, i, a.m_bf16) + (1.f - a.beta) * g;
}

// rowsq[e*R + r] = sum_c (mf * cscale[e*C + c])^2 ; rowabs (optional) = sum_c |g|.  One block per row.
template <int VEC>
__global__ void instinct_stat_rows(InstinctArgs a, const float* __restrict__ cscale, float* __restrict__ rowsq,
                                   float* __restrict__ rowabs) {
  __shared__ float red[32];
  for (long long row = blockIdx.x; row < a.E * a.R; row += gridDim.x) {
    const long long e = row / a.R;
    const long long base = row * a.C;
    const float* cs = cscale ? cscale + e * a.C : nullptr;
    float ss = 0.f, sa = 0.f;
    for (long long c = (long long)threadIdx.x * VEC; c < a.C; c += (long long)blockDim.x * VEC) {
      if (VEC == 4) {
        float4 g, v = mom4(a, base + c, g);
        if (cs) { const float4 k = *reinterpret_cast<const float4*>(cs + c); v.x *= k.x; v.y *= k.y; v.z *= k.z; v.w *= k.w; }
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        sa += fabsf(g.x) + fabsf(g.y) + fabsf(g.z) + fabsf(g.w);
      } else {
        float g, v = mom1(a, base + c, g);
        if (cs) v *= cs[c];
        ss += v * v;
        sa += fabsf(g);
      }
    }
    ss = block_sum(ss, red);
    if (rowabs) sa = block_sum(sa, red);
    if (threadIdx.x == 0) {
      rowsq[row] = ss;
      if (rowabs) rowabs[row] = sa;
    }
  }
}

// colsq[e*C + c] += sum over this block's rows of (mf * cscale[e,c] * rscale[e,r])^2
// grid: (col strips, row chunks, E); each thread owns VEC consecutive columns.
template <int VEC>
__global__ void instinct_stat_cols(InstinctArgs a, const float* __restrict__ cscale, const float* __restrict__ rscale,
                                   float* __restrict__ colsq_out, int rows_per_block) {
  const long long e = blockIdx.z;
  const long long c = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * VEC;
  if (c >= a.C) return;
  const long long r0 = (long long)blockIdx.y * rows_per_block;
  const long long r1 = min(a.R, r0 + rows_per_block);
  float cs[VEC], acc[VEC];
#pragma unroll
  for (int j = 0; j < VEC; ++j) { cs[j] = cscale ? cscale[e * a.C + c + j] : 1.f; acc[j] = 0.f; }
  for (long long r = r0; r < r1; ++r) {
    const long long i = (e * a.R + r) * a.C + c;
    const float rs = rscale ? rscale[e * a.R + r] : 1.f;
    if (VEC == 4) {
      float4 g, v = mom4(a, i, g);
      const float v0 = v.x * cs[0] * rs, v1 = v.y * cs[1 % VEC] * rs, v2 = v.z * cs[2 % VEC] * rs, v3 = v.w * cs[3 % VEC] * rs;
      acc[0] += v0 * v0; acc[1 % VEC] += v1 * v1; acc[2 % VEC] += v2 * v2; acc[3 % VEC] += v3 * v3;
    } else {
      float g;
      const float v = mom1(a, i, g) * cs[0] * rs;
      acc[0] += v * v;
    }
  }
#pragma unroll
  for (int j = 0; j < VEC; ++j) atomicAdd(colsq_out + e * a.C + c + j, acc[j]);
}

// rel_out = |g| / |w| from the two sums of squares
static __global__ void instinct_rel_final(const float* __restrict__ rel2, float* __restrict__ rel_out) {
  *rel_out = sqrtf(rel2[0]) / (sqrtf(rel2[1]) + 1e-8f);
}

// sums for |g|/|w|: rel2[0] += sum g^2, rel2[1] += sum w^2 (before the update)
static __global__ void instinct_rel_sums(InstinctArgs a, float* __restrict__ rel2) {
  __shared__ float red[32];
  const long long n = a.E * a.R * a.C;
  float sg = 0.f, sw = 0.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float g = gload(a, i);
    float t = a.w ? a.w[i] : ldv(a.p, i, a.p_bf16);
    sg += g * g; sw += t * t;
  }
  sg = block_sum(sg, red);
  sw = block_sum(sw, red);
  if (threadIdx.x == 0) { atomicAdd(rel2, sg); atomicAdd(rel2 + 1, sw); }
}

// The update itself, one block per row: upd = mf * rscale[row] * cscale1[c] * cscale2[c]; with `fuse_row_norm` the
// row is staged in shared memory and one more row normalisation (the last step of homeostasis) is done in place.
// Momentum is written here (once per step).  Rows of a word table without gradient and frozen slices keep their weights.
template <int VEC>
__global__ void instinct_apply(InstinctArgs a, const float* __restrict__ rscale, const float* __restrict__ cscale1,
                               const float* __restrict__ cscale2, int fuse_row_norm, const float* __restrict__ rowabs,
                               const float* __restrict__ rel2, float* __restrict__ rel_out) {
  extern __shared__ float cache[];
  __shared__ float red[32];
  const float lr = *a.lr;
  const float eff = 1.f + (*a.gain - 1.f) * (*a.stake);
  const float step = lr * eff, decay = (a.wd != 0.f) ? 1.f - lr * a.wd : 1.f;
  const uint32_t seed = a.sr ? (uint32_t)((*a.seed) * 1000003ll) * 0x9E3779B9u + a.salt : 0u;
  if (rel_out && blockIdx.x == 0 && threadIdx.x == 0) *rel_out = sqrtf(rel2[0]) / (sqrtf(rel2[1]) + 1e-8f);
  for (long long row = blockIdx.x; row < a.E * a.R; row += gridDim.x) {
    const long long e = row / a.R;
    const long long base = row * a.C;
    const float* c1 = cscale1 ? cscale1 + e * a.C : nullptr;
    const float* c2 = cscale2 ? cscale2 + e * a.C : nullptr;
    float rs = rscale ? rscale[row] : 1.f;
    const bool frozen = a.frozen && a.frozen[base / a.frozen_stride];
    const bool moves = !(rowabs && !(rowabs[row] > 0.f)) && !frozen;
    if (fuse_row_norm) {
      float ss = 0.f;
      for (long long c = (long long)threadIdx.x * VEC; c < a.C; c += (long long)blockDim.x * VEC) {
        if (VEC == 4) {
          float4 g, v = mom4(a, base + c, g);
          *reinterpret_cast<float4*>(cache + c) = v;
          float4 k = c1 ? *reinterpret_cast<const float4*>(c1 + c) : make_float4(1.f, 1.f, 1.f, 1.f);
          const float u0 = v.x * k.x, u1 = v.y * k.y, u2 = v.z * k.z, u3 = v.w * k.w;
          ss += u0 * u0 + u1 * u1 + u2 * u2 + u3 * u3;
        } else {
          float g, v = mom1(a, base + c, g);
          cache[c] = v;
          const float u = v * (c1 ? c1[c] : 1.f);
          ss += u * u;
        }
      }
      ss = block_sum(ss, red) * rs * rs;
      rs *= 1.f / (sqrtf(ss / (float)a.C) + 1e-8f);
    }
    // Column loop, software-pipelined by hand: the inputs of the next chunk are loaded before the current chunk is
    // stored (the weight, momentum and master pointers may alias as far as the compiler knows, so it would not hoist
    // those loads above the stores itself); this keeps two chunks of loads in flight per thread.
    const long long cstep = (long long)blockDim.x * VEC;
    float mf[VEC], k[VEC], t[VEC], mf_n[VEC], k_n[VEC], t_n[VEC];
    auto load_chunk = [&](long long c0, float* mfo, float* ko, float* to) {
      const long long i0 = base + c0;
      if (VEC == 4) {
        float4 v;
        if (fuse_row_norm) v = *reinterpret_cast<const float4*>(cache + c0);
        else { float4 g; v = mom4(a, i0, g); }
        mfo[0] = v.x; mfo[1 % VEC] = v.y; mfo[2 % VEC] = v.z; mfo[3 % VEC] = v.w;
        float4 k1 = c1 ? *reinterpret_cast<const float4*>(c1 + c0) : make_float4(1.f, 1.f, 1.f, 1.f);
        if (c2) { const float4 k2 = *reinterpret_cast<const float4*>(c2 + c0); k1.x *= k2.x; k1.y *= k2.y; k1.z *= k2.z; k1.w *= k2.w; }
        ko[0] = k1.x; ko[1 % VEC] = k1.y; ko[2 % VEC] = k1.z; ko[3 % VEC] = k1.w;
      } else {
        if (fuse_row_norm) mfo[0] = cache[c0];
        else { float g; mfo[0] = mom1(a, i0, g); }
        ko[0] = (c1 ? c1[c0] : 1.f) * (c2 ? c2[c0] : 1.f);
      }
      if (moves) {
        if (a.w) {
          if (VEC == 4) { const float4 w4 = *reinterpret_cast<const float4*>(a.w + i0); to[0] = w4.x; to[1 % VEC] = w4.y; to[2 % VEC] = w4.z; to[3 % VEC] = w4.w; }
          else to[0] = a.w[i0];
        } else if (VEC == 4) {
          const float4 w4 = ldv4(a.p, i0, a.p_bf16); to[0] = w4.x; to[1 % VEC] = w4.y; to[2 % VEC] = w4.z; to[3 % VEC] = w4.w;
        } else {
          to[0] = ldv(a.p, i0, a.p_bf16);
        }
      }
    };
    long long c0 = (long long)threadIdx.x * VEC;
    if (c0 < a.C) load_chunk(c0, mf, k, t);
    for (; c0 < a.C; c0 += cstep) {
      const bool has_next = c0 + cstep < a.C;
      if (has_next) load_chunk(c0 + cstep, mf_n, k_n, t_n);
      const long long i0 = base + c0;
      uint32_t h[VEC];
#pragma unroll
      for (int j = 0; j < VEC; ++j) h[j] = a.sr ? lowbias32((uint32_t)(i0 + j) ^ seed) : 0u;
      // momentum
      if (a.m_bf16) {
        bf16* mp = reinterpret_cast<bf16*>(a.m) + i0;
        if (VEC == 4 && !a.sr) {
          *reinterpret_cast<uint2*>(mp) = make_uint2(pack_bf16(mf[0], mf[1 % VEC]), pack_bf16(mf[2 % VEC], mf[3 % VEC]));
        } else {
#pragma unroll
          for (int j = 0; j < VEC; ++j) mp[j] = a.sr ? sr_round(mf[j], h[j] & 0xFFFFu) : __float2bfloat16(mf[j]);
        }
      } else {
        float* mp = reinterpret_cast<float*>(a.m) + i0;
        if (VEC == 4) *reinterpret_cast<float4*>(mp) = make_float4(mf[0], mf[1 % VEC], mf[2 % VEC], mf[3 % VEC]);
        else mp[0] = mf[0];
      }
      if (moves) {                                            // else: weight of this row / slice stays as it is
#pragma unroll
        for (int j = 0; j < VEC; ++j) t[j] = t[j] * decay - mf[j] * rs * k[j] * step;
        if (a.w) {
          if (VEC == 4) *reinterpret_cast<float4*>(a.w + i0) = make_float4(t[0], t[1 % VEC], t[2 % VEC], t[3 % VEC]);
          else a.w[i0] = t[0];
        }
        if (a.p_bf16) {
          bf16* pp = reinterpret_cast<bf16*>(a.p) + i0;
          if (VEC == 4 && !(a.sr && !a.w)) {
            *reinterpret_cast<uint2*>(pp) = make_uint2(pack_bf16(t[0], t[1 % VEC]), pack_bf16(t[2 % VEC], t[3 % VEC]));
          } else {
#pragma unroll
            for (int j = 0; j < VEC; ++j) pp[j] = (a.sr && !a.w) ? sr_round(t[j], h[j] >> 16) : __float2bfloat16(t[j]);
          }
        } else {
          float* pp = reinterpret_cast<float*>(a.p) + i0;
          if (VEC == 4) *reinterpret_cast<float4*>(pp) = make_float4(t[0], t[1 % VEC], t[2 % VEC], t[3 % VEC]);
          else pp[0] = t[0];
        }
      }
      if (has_next) {
#pragma unroll
        for (int j = 0; j < VEC; ++j) { mf[j] = mf_n[j]; k[j] = k_n[j]; t[j] = t_n[j]; }
      }
    }
    if (fuse_row_norm) __syncthreads();                        // the row cache is reused by the next row
  }
}

// Scratch layout (fp32, zeroed, 16-byte aligned base): [rowA][rowB][rowabs] of pad4(E*R) each, [colA][colB] of
// pad4(E*C) each, [rel 4]; every sub-array starts on a 16-byte boundary because the kernels read them as float4.
inline long long instinct_pad4(long long n) { return (n + 3) & ~3ll; }
inline long long instinct_scratch_floats(long long E, long long R, long long C) {
  return 3 * instinct_pad4(E * R) + 2 * instinct_pad4(E * C) + 4;
}

// Launch sequence; returns the number of kernels launched.
inline int64_t instinct_launch(const InstinctArgs& a, int kind, float* scratch, float* rel_out, cudaStream_t st) {
  const long long ER = a.E * a.R, EC = a.E * a.C, n = ER * a.C;
  const long long ERp = instinct_pad4(ER), ECp = instinct_pad4(EC);
  float* rowA = scratch;
  float* rowB = rowA + ERp;
  float* rowabs = rowB + ERp;
  float* colA = rowabs + ERp;
  float* colB = colA + ECp;
  float* rel2 = colB + ECp;
  const bool vec = (a.C % 4 == 0) && ((reinterpret_cast<uintptr_t>(a.p) & 15) == 0) &&
                   ((reinterpret_cast<uintptr_t>(a.g) & 15) == 0) && ((reinterpret_cast<uintptr_t>(a.m) & 15) == 0) &&
                   (a.w == nullptr || (reinterpret_cast<uintptr_t>(a.w) & 15) == 0) && (EC % 4 == 0 || a.E == 1);
  int64_t launches = 0;
  const int row_grid = (int)std::max<long long>(1, std::min<long long>(ER, 148 * 8));
  const int row_threads = a.C >= 1024 ? 256 : (a.C >= 256 ? 128 : 64);
  auto fin = [&](float* x, long long cnt, float count, const float* fold) {
    instinct_finalize<<<(int)std::max<long long>(1, std::min<long long>((cnt + 255) / 256, 592)), 256, 0, st>>>(x, cnt, count, fold);
    ++launches;
  };
  auto stat_rows = [&](const float* cs, float* out, float* absout) {
    if (vec) instinct_stat_rows<4><<<row_grid, row_threads, 0, st>>>(a, cs, out, absout);
    else instinct_stat_rows<1><<<row_grid, row_threads, 0, st>>>(a, cs, out, absout);
    ++launches;
  };
  auto stat_cols = [&](const float* cs, const float* rs, float* out) {
    const int V = vec ? 4 : 1;
    const int threads = 128;
    const int strips = (int)((a.C + (long long)threads * V - 1) / ((long long)threads * V));
    long long want_chunks = std::max<long long>(1, (148 * 8) / std::max<long long>(1, strips * a.E));
    int rows_per_block = (int)std::max<long long>(8, (a.R + want_chunks - 1) / want_chunks);
    int chunks = (int)((a.R + rows_per_block - 1) / rows_per_block);
    dim3 grid(strips, chunks, (unsigned)a.E);
    if (vec) instinct_stat_cols<4><<<grid, threads, 0, st>>>(a, cs, rs, out, rows_per_block);
    else instinct_stat_cols<1><<<grid, threads, 0, st>>>(a, cs, rs, out, rows_per_block);
    ++launches;
  };
  auto apply = [&](const float* rs, const float* c1, const float* c2, bool fuse, const float* rabs) {
    const size_t smem = fuse ? (size_t)a.C * sizeof(float) : 0;
    static bool big4 = false, big1 = false;           // raise the dynamic shared-memory limit once per kernel
    if (vec) {
      if (smem > 48 * 1024 && !big4) { cudaFuncSetAttribute(instinct_apply<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024); big4 = true; }
      instinct_apply<4><<<row_grid, row_threads, smem, st>>>(a, rs, c1, c2, fuse ? 1 : 0, rabs, rel2, rel_out);
    } else {
      if (smem > 48 * 1024 && !big1) { cudaFuncSetAttribute(instinct_apply<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024); big1 = true; }
      instinct_apply<1><<<row_grid, row_threads, smem, st>>>(a, rs, c1, c2, fuse ? 1 : 0, rabs, rel2, rel_out);
    }
    ++launches;
  };
  if (rel_out) {
    const int grid = (int)std::max<long long>(1, std::min<long long>((n + 255) / 256, 148 * 8));
    instinct_rel_sums<<<grid, 256, 0, st>>>(a, rel2);
    ++launches;
  }
  const float Rf = (float)a.R, Cf = (float)a.C;
  switch (kind) {
    case 4: {  // hs: rows, columns, rows again (the last one inside `apply` when the row fits in shared memory)
      stat_rows(nullptr, rowA, nullptr);
      fin(rowA, ER, Cf, nullptr);
      stat_cols(nullptr, rowA, colA);
      fin(colA, EC, Rf, nullptr);
      if ((size_t)a.C * sizeof(float) <= 96 * 1024) {
        apply(rowA, colA, nullptr, true, nullptr);
      } else {
        stat_rows(colA, rowB, nullptr);           // sum_c (mf cs)^2; times rs1^2 below = row sums of u2
        fin(rowB, ER, Cf, rowA);                  // rs3
        instinct_mul<<<(int)std::max<long long>(1, std::min<long long>((ER + 255) / 256, 592)), 256, 0, st>>>(rowB, rowA, ER);
        ++launches;                               // rowB = rs1 * rs3
        apply(rowB, colA, nullptr, false, nullptr);
      }
      break;
    }
    case 5:   // hs3: over R (per column), over C (per row), over R again
      stat_cols(nullptr, nullptr, colA);
      fin(colA, EC, Rf, nullptr);
      stat_rows(colA, rowA, nullptr);
      fin(rowA, ER, Cf, nullptr);
      stat_cols(colA, rowA, colB);
      fin(colB, EC, Rf, nullptr);
      apply(rowA, colA, colB, false, nullptr);
      break;
    case 3:   // word table: row rms, only rows with a gradient move
      stat_rows(nullptr, rowA, rowabs);
      fin(rowA, ER, Cf, nullptr);
      apply(rowA, nullptr, nullptr, false, rowabs);
      break;
    case 2:   // experts (E, in, out): one norm per (expert, output column) over `in`
      stat_cols(nullptr, nullptr, colA);
      fin(colA, EC, Rf, nullptr);
      apply(nullptr, colA, nullptr, false, nullptr);
      break;
    default:  // kinds 0 and 1: one norm per row of the (E*R, C) view (the whole tensor when E = R = 1)
      stat_rows(nullptr, rowA, nullptr);
      fin(rowA, ER, Cf, nullptr);
      apply(rowA, nullptr, nullptr, false, nullptr);
      break;
  }
  return launches;
}

}  // namespace mb
