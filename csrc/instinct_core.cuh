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
__device__ __forceinline__ float inv_rms(float sumsq, float count) { return 1.f / (sqrtf(sumsq / count) + 1e-8f); }

// rowsq[e*R + r] = sum_c (mf * cscale[e*C + c])^2 ; rowabs (optional) = sum_c |g|
template <int VEC>
__global__ void instinct_stat_rows(InstinctArgs a, const float* __restrict__ colsq, float col_count,
                                   float* __restrict__ rowsq, float* __restrict__ rowabs) {
  __shared__ float red[32];
  for (long long row = blockIdx.x; row < a.E * a.R; row += gridDim.x) {
    const long long e = row / a.R;
    const long long base = row * a.C;
    float ss = 0.f, sa = 0.f;
    for (long long c = (long long)threadIdx.x * VEC; c < a.C; c += (long long)blockDim.x * VEC) {
      if (VEC == 4) {
        float4 g = gload4(a, base + c), mm = ldv4(a.m, base + c, a.m_bf16);
        float v[4] = {a.beta * mm.x + (1.f - a.beta) * g.x, a.beta * mm.y + (1.f - a.beta) * g.y,
                      a.beta * mm.z + (1.f - a.beta) * g.z, a.beta * mm.w + (1.f - a.beta) * g.w};
        if (colsq) {
#pragma unroll
          for (int j = 0; j < 4; ++j) v[j] *= inv_rms(colsq[e * a.C + c + j], col_count);
        }
        ss += v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
        sa += fabsf(g.x) + fabsf(g.y) + fabsf(g.z) + fabsf(g.w);
      } else {
        float g = gload(a, base + c);
        float v = a.beta * ldv(a.m, base + c, a.m_bf16) + (1.f - a.beta) * g;
        if (colsq) v *= inv_rms(colsq[e * a.C + c], col_count);
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
__global__ void instinct_stat_cols(InstinctArgs a, const float* __restrict__ colsq_in, float col_count,
                                   const float* __restrict__ rowsq_in, float row_count, float* __restrict__ colsq_out,
                                   int rows_per_block) {
  const long long e = blockIdx.z;
  const long long c = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * VEC;
  if (c >= a.C) return;
  const long long r0 = (long long)blockIdx.y * rows_per_block;
  const long long r1 = min(a.R, r0 + rows_per_block);
  float cs[VEC];
#pragma unroll
  for (int j = 0; j < VEC; ++j) cs[j] = colsq_in ? inv_rms(colsq_in[e * a.C + c + j], col_count) : 1.f;
  float acc[VEC];
#pragma unroll
  for (int j = 0; j < VEC; ++j) acc[j] = 0.f;
  for (long long r = r0; r < r1; ++r) {
    const long long i = (e * a.R + r) * a.C + c;
    const float rs = rowsq_in ? inv_rms(rowsq_in[e * a.R + r], row_count) : 1.f;
    if (VEC == 4) {
      float4 g = gload4(a, i), mm = ldv4(a.m, i, a.m_bf16);
      float v0 = (a.beta * mm.x + (1.f - a.beta) * g.x) * cs[0] * rs, v1 = (a.beta * mm.y + (1.f - a.beta) * g.y) * cs[1 % VEC] * rs;
      float v2 = (a.beta * mm.z + (1.f - a.beta) * g.z) * cs[2 % VEC] * rs, v3 = (a.beta * mm.w + (1.f - a.beta) * g.w) * cs[3 % VEC] * rs;
      acc[0] += v0 * v0; acc[1 % VEC] += v1 * v1; acc[2 % VEC] += v2 * v2; acc[3 % VEC] += v3 * v3;
    } else {
      float v = (a.beta * ldv(a.m, i, a.m_bf16) + (1.f - a.beta) * gload(a, i)) * cs[0] * rs;
      acc[0] += v * v;
    }
  }
#pragma unroll
  for (int j = 0; j < VEC; ++j) atomicAdd(colsq_out + e * a.C + c + j, acc[j]);
}

struct Scale { const float* sq; float count; int axis; };    // axis: 0 = per row (e*R+r), 1 = per column (e*C+c), 2 = scalar, -1 = none

__device__ __forceinline__ float scale_at(const Scale& s, long long e, long long r, long long c, long long R, long long C) {
  if (s.axis < 0) return 1.f;
  const float v = s.axis == 0 ? s.sq[e * R + r] : (s.axis == 1 ? s.sq[e * C + c] : s.sq[0]);
  return inv_rms(v, s.count);
}

// rowB[i] <- rs1[i]^2 * rowB[i] with rs1 = 1/(sqrt(rowA[i]/count)+eps)
static __global__ void instinct_fold_rows(float* __restrict__ rowB, const float* __restrict__ rowA, float count, long long n) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float s = inv_rms(rowA[i], count);
    rowB[i] = s * s * rowB[i];
  }
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

template <int VEC>
__global__ void instinct_apply(InstinctArgs a, Scale s1, Scale s2, Scale s3, const float* __restrict__ rowabs,
                               const float* __restrict__ rel2, float* __restrict__ rel_out) {
  const long long n = a.E * a.R * a.C;
  const float lr = *a.lr;
  const float eff = 1.f + (*a.gain - 1.f) * (*a.stake);
  const float step = lr * eff, decay = 1.f - lr * a.wd;
  const uint32_t seed = a.sr ? (uint32_t)((*a.seed) * 1000003ll) * 0x9E3779B9u + a.salt : 0u;
  if (rel_out && blockIdx.x == 0 && threadIdx.x == 0) *rel_out = sqrtf(rel2[0]) / (sqrtf(rel2[1]) + 1e-8f);
  for (long long i0 = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * VEC; i0 < n;
       i0 += (long long)gridDim.x * blockDim.x * VEC) {
    const long long row = i0 / a.C;
    const long long c0 = i0 - row * a.C;
    const long long e = row / a.R, r = row - e * a.R;
    float g[VEC], mo[VEC];
    if (VEC == 4) {
      float4 g4 = gload4(a, i0), m4 = ldv4(a.m, i0, a.m_bf16);
      g[0] = g4.x; g[1 % VEC] = g4.y; g[2 % VEC] = g4.z; g[3 % VEC] = g4.w;
      mo[0] = m4.x; mo[1 % VEC] = m4.y; mo[2 % VEC] = m4.z; mo[3 % VEC] = m4.w;
    } else {
      g[0] = gload(a, i0); mo[0] = ldv(a.m, i0, a.m_bf16);
    }
    const bool moves = (rowabs == nullptr || rowabs[row] > 0.f) &&
                       !(a.frozen && a.frozen[i0 / a.frozen_stride]);
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      const long long i = i0 + j, c = c0 + j;
      const float mf = a.beta * mo[j] + (1.f - a.beta) * g[j];
      uint32_t h = a.sr ? lowbias32((uint32_t)i ^ seed) : 0u;
      if (a.m_bf16) reinterpret_cast<bf16*>(a.m)[i] = a.sr ? sr_round(mf, h & 0xFFFFu) : __float2bfloat16(mf);
      else reinterpret_cast<float*>(a.m)[i] = mf;
      const float upd = mf * scale_at(s1, e, r, c, a.R, a.C) * scale_at(s2, e, r, c, a.R, a.C) *
                        scale_at(s3, e, r, c, a.R, a.C);
      float t = a.w ? a.w[i] : ldv(a.p, i, a.p_bf16);
      if (moves) {
        t = (a.wd != 0.f ? t * decay : t) - upd * step;
      } else if (a.frozen && a.frozen[i0 / a.frozen_stride]) {
        continue;                                            // frozen slice: weight untouched
      } else {
        t = (a.wd != 0.f ? t * decay : t);                   // word-table row without gradient: no step (wd is 0 there)
      }
      if (a.w) a.w[i] = t;
      if (a.p_bf16) reinterpret_cast<bf16*>(a.p)[i] = (a.sr && !a.w) ? sr_round(t, h >> 16) : __float2bfloat16(t);
      else reinterpret_cast<float*>(a.p)[i] = t;
    }
  }
}

// Launch sequence.  scratch (fp32, zeroed): [rowsqA E*R][rowsqB E*R][rowabs E*R][colsqA E*C][colsqB E*C][rel 2].
inline int64_t instinct_launch(const InstinctArgs& a, int kind, float* scratch, float* rel_out, cudaStream_t st) {
  const long long ER = a.E * a.R, EC = a.E * a.C, n = ER * a.C;
  float* rowA = scratch;
  float* rowB = rowA + ER;
  float* rowabs = rowB + ER;
  float* colA = rowabs + ER;
  float* colB = colA + EC;
  float* rel2 = colB + EC;
  const bool vec = (a.C % 4 == 0) && ((reinterpret_cast<uintptr_t>(a.p) & 15) == 0) &&
                   ((reinterpret_cast<uintptr_t>(a.g) & 15) == 0) && ((reinterpret_cast<uintptr_t>(a.m) & 15) == 0);
  int64_t launches = 0;
  const int row_grid = (int)std::min<long long>(ER, 148 * 8);
  auto stat_rows = [&](const float* csq, float ccount, float* out, float* absout) {
    if (vec) instinct_stat_rows<4><<<row_grid, 256, 0, st>>>(a, csq, ccount, out, absout);
    else instinct_stat_rows<1><<<row_grid, 256, 0, st>>>(a, csq, ccount, out, absout);
    ++launches;
  };
  auto stat_cols = [&](const float* csq, float ccount, const float* rsq, float rcount, float* out) {
    const int V = vec ? 4 : 1;
    const int threads = 128;
    const int strips = (int)((a.C + (long long)threads * V - 1) / ((long long)threads * V));
    long long want_chunks = std::max<long long>(1, (148 * 8) / std::max<long long>(1, strips * a.E));
    int rows_per_block = (int)std::max<long long>(8, (a.R + want_chunks - 1) / want_chunks);
    int chunks = (int)((a.R + rows_per_block - 1) / rows_per_block);
    dim3 grid(strips, chunks, (unsigned)a.E);
    if (vec) instinct_stat_cols<4><<<grid, threads, 0, st>>>(a, csq, ccount, rsq, rcount, out, rows_per_block);
    else instinct_stat_cols<1><<<grid, threads, 0, st>>>(a, csq, ccount, rsq, rcount, out, rows_per_block);
    ++launches;
  };
  auto apply = [&](Scale s1, Scale s2, Scale s3, const float* rabs) {
    const int V = vec ? 4 : 1;
    const int grid = (int)std::min<long long>((n / V + 255) / 256, 148 * 16);
    if (vec) instinct_apply<4><<<std::max(grid, 1), 256, 0, st>>>(a, s1, s2, s3, rabs, rel2, rel_out);
    else instinct_apply<1><<<std::max(grid, 1), 256, 0, st>>>(a, s1, s2, s3, rabs, rel2, rel_out);
    ++launches;
  };
  if (rel_out) {
    const int grid = (int)std::min<long long>((n + 255) / 256, 148 * 8);
    instinct_rel_sums<<<std::max(grid, 1), 256, 0, st>>>(a, rel2);
    ++launches;
  }
  const Scale none{nullptr, 1.f, -1};
  const float Rf = (float)a.R, Cf = (float)a.C;
  switch (kind) {
    case 4:   // hs: row, column, row
      stat_rows(nullptr, 1.f, rowA, nullptr);
      stat_cols(nullptr, 1.f, rowA, Cf, colA);
      // third norm: rows of u2 = mf * rs1[r] * cs[c].  rs1 is constant along a row, so
      // sum_c u2^2 = rs1^2 * sum_c (mf * cs[c])^2: one more row statistic, then fold rs1^2 in (E*R values).
      stat_rows(colA, Rf, rowB, nullptr);
      instinct_fold_rows<<<(int)std::min<long long>((ER + 255) / 256, 1184), 256, 0, st>>>(rowB, rowA, Cf, ER);
      ++launches;
      apply(Scale{rowA, Cf, 0}, Scale{colA, Rf, 1}, Scale{rowB, Cf, 0}, nullptr);
      break;
    case 5:   // hs3: norm over R (per column), over C (per row), over R again
      stat_cols(nullptr, 1.f, nullptr, 1.f, colA);
      stat_rows(colA, Rf, rowA, nullptr);
      stat_cols(colA, Rf, rowA, Cf, colB);
      apply(Scale{colA, Rf, 1}, Scale{rowA, Cf, 0}, Scale{colB, Rf, 1}, nullptr);
      break;
    case 3:   // word table: row rms, only rows with a gradient move
      stat_rows(nullptr, 1.f, rowA, rowabs);
      apply(Scale{rowA, Cf, 0}, none, none, rowabs);
      break;
    case 1:   // one norm per first-dimension row
      stat_rows(nullptr, 1.f, rowA, nullptr);
      apply(Scale{rowA, Cf, 0}, none, none, nullptr);
      break;
    case 2:   // experts (E, in, out): one norm per (expert, output column) over `in`
      stat_cols(nullptr, 1.f, nullptr, 1.f, colA);
      apply(Scale{colA, Rf, 1}, none, none, nullptr);
      break;
    default:  // whole tensor
      stat_rows(nullptr, 1.f, rowA, nullptr);
      apply(Scale{rowA, Cf, 0}, none, none, nullptr);
      break;
  }
  return launches;
}

}  // namespace mb
