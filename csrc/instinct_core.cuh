// Device kernels and the launch sequence of one Instinct step (torch-free; see instinct.cu for the maths).
//
// A weight is viewed as (E, R, C) with C contiguous; mf = beta*m + (1-beta)*g is recomputed wherever it is needed and
// the momentum is written once, by `apply`.  All statistics are RAW sums of squares in a zeroed scratch array; each
// consumer turns a sum into its scale 1 / (sqrt(sum / count) + 1e-8) itself, so no "finalize" launches exist.
//   instinct_stat_rows : rowsq[e,r]  = sum_c (mf * cscale[e,c])^2                      (+ sum|g| for word tables)
//   instinct_stat_cols : colsq[e,c] += sum_r (mf * cscale[e,c] * rscale[e,r])^2
//   instinct_rowcol    : both of the above ("rows, then columns") in one pass over g and m: a block keeps the row it
//                        has just reduced in shared memory and adds its scaled squares to per-block column sums.
//                        One row in flight per block makes it latency-bound (measured 1.0 TB/s against 5.3 TB/s of
//                        the two separate kernels), so it only serves the lagged form, where it usually returns at
//                        once (`skip_if`)
//   instinct_apply     : upd = mf * rowscale * colscale1 * colscale2 -> weight / momentum; optionally one more row
//                        normalisation on the row staged in shared memory (the last step of `hs`)
//   instinct_lag_hs    : lagged homeostasis of a 2-D weight in one pass (column norm of the previous step)
#pragma once
#include <algorithm>

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
  void* shadow;            // optional bf16 copy of an fp32 weight, refreshed by `apply` (what the GEMMs read)
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
// sum of squares over `count` elements -> scale
__device__ __forceinline__ float scale_of(float sumsq, float count) { return 1.f / (sqrtf(sumsq / count) + 1e-8f); }

__device__ __forceinline__ float4 mom4(const InstinctArgs& a, long long i, float4& g) {
  g = ldv4(a.g, i, a.g_bf16);
  const float4 mm = ldv4(a.m, i, a.m_bf16);
  const float b = a.beta, c = 1.f - a.beta;
  return make_float4(b * mm.x + c * g.x, b * mm.y + c * g.y, b * mm.z + c * g.z, b * mm.w + c * g.w);
}
__device__ __forceinline__ float mom1(const InstinctArgs& a, long long i, float& g) {
  g = ldv(a.g, i, a.g_bf16);
  return a.beta * ldv(a.m, i, a.m_bf16) + (1.f - a.beta) * g;
}

// Column scales of expert e into shared memory: dst[c] = scale(sum1[e,c]) * scale(sum2[e,c]) (either may be null).
__device__ __forceinline__ void load_colscale(float* dst, const float* sum1, const float* sum2, long long e, long long C,
                                              float count) {
  // four columns per thread and round: the loads go out together (dst may alias the sums as far as the compiler knows)
  for (long long c0 = threadIdx.x; c0 < C; c0 += 4ll * blockDim.x) {
    float s1[4], s2[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const long long c = c0 + (long long)u * blockDim.x;
      s1[u] = (sum1 && c < C) ? sum1[e * C + c] : 1.f;
      s2[u] = (sum2 && c < C) ? sum2[e * C + c] : 1.f;
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const long long c = c0 + (long long)u * blockDim.x;
      if (c < C) dst[c] = (sum1 ? scale_of(s1[u], count) : 1.f) * (sum2 ? scale_of(s2[u], count) : 1.f);
    }
  }
  __syncthreads();
}

// rowsq[e*R + r] = sum_c (mf * colscale[e,c])^2 ; rowabs (optional) = sum_c |g|.  grid (blocks per expert, E);
// dynamic shared memory: C floats when colsum is given.
template <int VEC>
__global__ void instinct_stat_rows(InstinctArgs a, const float* __restrict__ colsum, float col_count,
                                   float* __restrict__ rowsq, float* __restrict__ rowabs) {
  extern __shared__ float sm[];
  __shared__ float red[32];
  const long long e = blockIdx.y;
  float* cs = colsum ? sm : nullptr;
  if (cs) load_colscale(cs, colsum, nullptr, e, a.C, col_count);
  for (long long r = blockIdx.x; r < a.R; r += gridDim.x) {
    const long long row = e * a.R + r;
    const long long base = row * a.C;
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

// colsq[e*C + c] += sum over this block's rows of (mf * colscale[e,c] * rowscale[e,r])^2
// grid: (col strips, row chunks, E); each thread owns VEC consecutive columns.  Scales come from raw sums; the row
// scales of the block's chunk are formed once, into shared memory (rows_per_block floats of dynamic shared memory).
template <int VEC>
__global__ void instinct_stat_cols(InstinctArgs a, const float* __restrict__ colsum, float col_count,
                                   const float* __restrict__ rowsum, float row_count, float* __restrict__ colsq_out,
                                   int rows_per_block) {
  extern __shared__ float rsm[];
  const long long e = blockIdx.z;
  const long long c = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * VEC;
  const long long r0 = (long long)blockIdx.y * rows_per_block;
  const long long r1 = min(a.R, r0 + rows_per_block);
  if (rowsum) {
    for (long long r = r0 + threadIdx.x; r < r1; r += blockDim.x) rsm[r - r0] = scale_of(rowsum[e * a.R + r], row_count);
    __syncthreads();
  }
  if (c >= a.C) return;
  float cs[VEC], acc[VEC];
#pragma unroll
  for (int j = 0; j < VEC; ++j) { cs[j] = colsum ? scale_of(colsum[e * a.C + c + j], col_count) : 1.f; acc[j] = 0.f; }
  for (long long r = r0; r < r1; ++r) {
    const long long i = (e * a.R + r) * a.C + c;
    const float rs = rowsum ? rsm[r - r0] : 1.f;
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

// Rows, then columns, in one pass: rowsq_out[e,r] = sum_c (mf*cin[e,c])^2 and
// colsq_out[e,c] += sum_r (mf * cin[e,c] * scale(rowsq[e,r]))^2.  grid (blocks per expert, E); dynamic shared memory
// (2 + has_cin) * C floats: the row just reduced, the block's column sums, the incoming column scales.
// `skip_if` (optional device flag): the kernel returns at once when *skip_if != 0.
template <int VEC>
__global__ void instinct_rowcol(InstinctArgs a, const float* __restrict__ colsum_in, float col_count,
                                float* __restrict__ rowsq_out, float* __restrict__ colsq_out, const int* __restrict__ skip_if) {
  extern __shared__ float sm[];
  __shared__ float red[32];
  if (skip_if && *skip_if) return;
  const long long e = blockIdx.y, C = a.C;
  float* cache = sm;
  float* colacc = sm + C;
  float* cin = colsum_in ? sm + 2 * C : nullptr;
  for (long long c = threadIdx.x; c < C; c += blockDim.x) colacc[c] = 0.f;
  if (cin) load_colscale(cin, colsum_in, nullptr, e, C, col_count);
  __syncthreads();
  const float Cf = (float)C;
  for (long long r = blockIdx.x; r < a.R; r += gridDim.x) {
    const long long row = e * a.R + r;
    const long long base = row * C;
    float ss = 0.f;
    for (long long c = (long long)threadIdx.x * VEC; c < C; c += (long long)blockDim.x * VEC) {
      if (VEC == 4) {
        float4 g, v = mom4(a, base + c, g);
        if (cin) { const float4 k = *reinterpret_cast<const float4*>(cin + c); v.x *= k.x; v.y *= k.y; v.z *= k.z; v.w *= k.w; }
        *reinterpret_cast<float4*>(cache + c) = v;
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
      } else {
        float g, v = mom1(a, base + c, g);
        if (cin) v *= cin[c];
        cache[c] = v;
        ss += v * v;
      }
    }
    ss = block_sum(ss, red);
    if (rowsq_out && threadIdx.x == 0) rowsq_out[row] = ss;
    const float rs = scale_of(ss, Cf);
    // every thread revisits exactly the columns it wrote above: no barrier needed between the two sweeps
    for (long long c = (long long)threadIdx.x * VEC; c < C; c += (long long)blockDim.x * VEC) {
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        const float u = cache[c + j] * rs;
        colacc[c + j] += u * u;
      }
    }
  }
  for (long long c = (long long)threadIdx.x * VEC; c < C; c += (long long)blockDim.x * VEC) {
#pragma unroll
    for (int j = 0; j < VEC; ++j)
      if (colacc[c + j] != 0.f) atomicAdd(colsq_out + e * C + c + j, colacc[c + j]);
  }
}

// sums for |g|/|w|: rel2[0] += sum g^2, rel2[1] += sum w^2 (before the update)
static __global__ void instinct_rel_sums(InstinctArgs a, float* __restrict__ rel2) {
  __shared__ float red[32];
  const long long n = a.E * a.R * a.C;
  float sg = 0.f, sw = 0.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float g = ldv(a.g, i, a.g_bf16);
    float t = a.w ? a.w[i] : ldv(a.p, i, a.p_bf16);
    sg += g * g; sw += t * t;
  }
  sg = block_sum(sg, red);
  sw = block_sum(sw, red);
  if (threadIdx.x == 0) { atomicAdd(rel2, sg); atomicAdd(rel2 + 1, sw); }
}

// Store one chunk of the update: momentum, weight (+ exact copy, + bf16 shadow).  Shared by `apply` and `lag_hs`.
template <int VEC>
__device__ __forceinline__ void store_chunk(const InstinctArgs& a, long long i0, const float* mf, float* t, const float* upd,
                                            bool moves, float step, float decay, uint32_t seed) {
  uint32_t h[VEC];
#pragma unroll
  for (int j = 0; j < VEC; ++j) h[j] = a.sr ? lowbias32((uint32_t)(i0 + j) ^ seed) : 0u;
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
  if (!moves) return;                                       // the weight of this row / slice stays as it is
#pragma unroll
  for (int j = 0; j < VEC; ++j) t[j] = t[j] * decay - upd[j] * step;
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
    if (a.shadow) {
      bf16* sp = reinterpret_cast<bf16*>(a.shadow) + i0;
      if (VEC == 4) *reinterpret_cast<uint2*>(sp) = make_uint2(pack_bf16(t[0], t[1 % VEC]), pack_bf16(t[2 % VEC], t[3 % VEC]));
      else sp[0] = __float2bfloat16(t[0]);
    }
  }
}
template <int VEC>
__device__ __forceinline__ void load_weight(const InstinctArgs& a, long long i0, float* to) {
  if (a.w) {
    if (VEC == 4) { const float4 w4 = *reinterpret_cast<const float4*>(a.w + i0); to[0] = w4.x; to[1 % VEC] = w4.y; to[2 % VEC] = w4.z; to[3 % VEC] = w4.w; }
    else to[0] = a.w[i0];
  } else if (VEC == 4) {
    const float4 w4 = ldv4(a.p, i0, a.p_bf16); to[0] = w4.x; to[1 % VEC] = w4.y; to[2 % VEC] = w4.z; to[3 % VEC] = w4.w;
  } else {
    to[0] = ldv(a.p, i0, a.p_bf16);
  }
}

// The update itself.  grid (blocks per expert, E), one row per block at a time:
//   upd = mf * rs * colk[c],  rs = scale(rowsum[row]) (x scale(rowsum2[row] * rs^2) when rowsum2 is given),
//   colk = scale(colsum1) * scale(colsum2) staged in shared memory once per block.
// With `fuse_row_norm` the row is staged in shared memory and one more row normalisation (the last step of
// homeostasis) is done in place.  Momentum is written here (once per step).  Rows of a word table without gradient
// and frozen slices keep their weights.  Dynamic shared memory: (has_col + fuse) * C floats.
template <int VEC>
__global__ void instinct_apply(InstinctArgs a, const float* __restrict__ rowsum, float row_count,
                               const float* __restrict__ rowsum2, const float* __restrict__ colsum1,
                               const float* __restrict__ colsum2, float col_count, int fuse_row_norm,
                               const float* __restrict__ rowabs, const float* __restrict__ rel2, float* __restrict__ rel_out) {
  extern __shared__ float sm[];
  __shared__ float red[32];
  const long long e = blockIdx.y, C = a.C;
  const bool has_col = colsum1 || colsum2;
  float* colk = has_col ? sm : nullptr;
  float* cache = sm + (has_col ? C : 0);
  const float lr = *a.lr;
  const float eff = 1.f + (*a.gain - 1.f) * (*a.stake);
  const float step = lr * eff, decay = (a.wd != 0.f) ? 1.f - lr * a.wd : 1.f;
  const uint32_t seed = a.sr ? (uint32_t)((*a.seed) * 1000003ll) * 0x9E3779B9u + a.salt : 0u;
  if (rel_out && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) *rel_out = sqrtf(rel2[0]) / (sqrtf(rel2[1]) + 1e-8f);
  if (has_col) load_colscale(colk, colsum1, colsum2, e, C, col_count);
  for (long long r = blockIdx.x; r < a.R; r += gridDim.x) {
    const long long row = e * a.R + r;
    const long long base = row * C;
    float rs = rowsum ? scale_of(rowsum[row], row_count) : 1.f;
    if (rowsum2) rs *= scale_of(rowsum2[row] * rs * rs, row_count);
    const bool frozen = a.frozen && a.frozen[base / a.frozen_stride];
    const bool moves = !(rowabs && !(rowabs[row] > 0.f)) && !frozen;
    if (fuse_row_norm) {
      float ss = 0.f;
      for (long long c = (long long)threadIdx.x * VEC; c < C; c += (long long)blockDim.x * VEC) {
        if (VEC == 4) {
          float4 g, v = mom4(a, base + c, g);
          *reinterpret_cast<float4*>(cache + c) = v;
          const float4 k = colk ? *reinterpret_cast<const float4*>(colk + c) : make_float4(1.f, 1.f, 1.f, 1.f);
          const float u0 = v.x * k.x, u1 = v.y * k.y, u2 = v.z * k.z, u3 = v.w * k.w;
          ss += u0 * u0 + u1 * u1 + u2 * u2 + u3 * u3;
        } else {
          float g, v = mom1(a, base + c, g);
          cache[c] = v;
          const float u = v * (colk ? colk[c] : 1.f);
          ss += u * u;
        }
      }
      ss = block_sum(ss, red) * rs * rs;
      rs *= scale_of(ss, (float)C);
    }
    // Column loop, software-pipelined by hand: the inputs of the next chunk are loaded before the current chunk is
    // stored (the weight, momentum and master pointers may alias as far as the compiler knows, so it would not hoist
    // those loads above the stores itself); this keeps two chunks of loads in flight per thread.
    const long long cstep = (long long)blockDim.x * VEC;
    float mf[VEC], k[VEC], t[VEC], mf_n[VEC], k_n[VEC], t_n[VEC], upd[VEC];
    auto load_chunk = [&](long long c0, float* mfo, float* ko, float* to) {
      const long long i0 = base + c0;
      if (VEC == 4) {
        float4 v;
        if (fuse_row_norm) v = *reinterpret_cast<const float4*>(cache + c0);
        else { float4 g; v = mom4(a, i0, g); }
        mfo[0] = v.x; mfo[1 % VEC] = v.y; mfo[2 % VEC] = v.z; mfo[3 % VEC] = v.w;
        const float4 k1 = colk ? *reinterpret_cast<const float4*>(colk + c0) : make_float4(1.f, 1.f, 1.f, 1.f);
        ko[0] = k1.x; ko[1 % VEC] = k1.y; ko[2 % VEC] = k1.z; ko[3 % VEC] = k1.w;
      } else {
        if (fuse_row_norm) mfo[0] = cache[c0];
        else { float g; mfo[0] = mom1(a, i0, g); }
        ko[0] = colk ? colk[c0] : 1.f;
      }
      if (moves) load_weight<VEC>(a, i0, to);
    };
    long long c0 = (long long)threadIdx.x * VEC;
    if (c0 < C) load_chunk(c0, mf, k, t);
    for (; c0 < C; c0 += cstep) {
      const bool has_next = c0 + cstep < C;
      if (has_next) load_chunk(c0 + cstep, mf_n, k_n, t_n);
#pragma unroll
      for (int j = 0; j < VEC; ++j) upd[j] = mf[j] * rs * k[j];
      store_chunk<VEC>(a, base + c0, mf, t, upd, moves, step, decay, seed);
      if (has_next) {
#pragma unroll
        for (int j = 0; j < VEC; ++j) { mf[j] = mf_n[j]; k[j] = k_n[j]; t[j] = t_n[j]; }
      }
    }
    if (fuse_row_norm) __syncthreads();                        // the row cache is reused by the next row
  }
}

// ---- streaming forms.  A block that walks one row at a time and reduces it across its warps has one short burst of
// loads in flight, then two barriers (1.7 TB/s for the row sums, 3.6 TB/s for the update on the expert shapes), and
// a warp that loads a few chunks of its row into registers, then computes, does little better (2.6 / 4.4 TB/s): HBM
// wants well over 100 KB in flight per SM all the time.  So here every thread keeps a ring of S chunks (8 elements of
// each input array) in shared memory, filled by cp.async copies issued S chunks ahead of the one it consumes;
// a warp owns a contiguous run of rows, so its stream is one linear span of memory, and the ring runs across row
// boundaries.  One block per SM; C % 256 == 0 (a chunk of 32 lanes x 8 never straddles rows).
__device__ __forceinline__ void cp_async16(void* s, const void* g) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(s)), "l"(g) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// A lane's 8 elements of a 256-element chunk are two groups of four, 128 elements apart: columns lane*4 .. +3 and
// 128 + lane*4 .. +3.  Every warp-wide load or store then covers one contiguous span of full 32-byte sectors whatever
// the element size (with 8 consecutive elements per lane an fp32 array needs two 16-byte accesses at a 32-byte lane
// stride, each touching all sectors of the chunk and using half of each: the word tables with their fp32 gradients
// ran at 1.8 TB/s).
__device__ __forceinline__ void cp_async8(void* s, const void* g) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(smem_u32(s)), "l"(g) : "memory");
}
struct Ring8 {             // this thread's ring: slot (stage, q) is 16 bytes; slots of one (stage, q) are contiguous over threads
  uint4* base;
  int T, nslot;
  __device__ __forceinline__ uint4* slot(int stage, int q) const { return base + (stage * nslot + q) * T; }
  // `i` = index of the lane's first element (chunk start + lane * 4)
  __device__ __forceinline__ void issue8(int stage, int q0, const void* arr, long long i, int is_bf16) const {
    if (is_bf16) {
      uint8_t* d = reinterpret_cast<uint8_t*>(slot(stage, q0));
      cp_async8(d, reinterpret_cast<const bf16*>(arr) + i);
      cp_async8(d + 8, reinterpret_cast<const bf16*>(arr) + i + 128);
    } else {
      cp_async16(slot(stage, q0), reinterpret_cast<const float*>(arr) + i);
      cp_async16(slot(stage, q0 + 1), reinterpret_cast<const float*>(arr) + i + 128);
    }
  }
  __device__ __forceinline__ void read8(int stage, int q0, int is_bf16, float* o) const {
    const uint4 u = *slot(stage, q0);
    if (is_bf16) {
      const float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), c = unpack_bf16(u.z), d = unpack_bf16(u.w);
      o[0] = a.x; o[1] = a.y; o[2] = b.x; o[3] = b.y; o[4] = c.x; o[5] = c.y; o[6] = d.x; o[7] = d.y;
    } else {
      const uint4 v = *slot(stage, q0 + 1);
      o[0] = __uint_as_float(u.x); o[1] = __uint_as_float(u.y); o[2] = __uint_as_float(u.z); o[3] = __uint_as_float(u.w);
      o[4] = __uint_as_float(v.x); o[5] = __uint_as_float(v.y); o[6] = __uint_as_float(v.z); o[7] = __uint_as_float(v.w);
    }
  }
};
// store the lane's two groups of four at dst + i and dst + i + 128
__device__ __forceinline__ void st8_f32(float* dst, const float* v) {
  *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(dst + 128) = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void st8_bf16(bf16* dst, const float* v) {
  *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]));
  *reinterpret_cast<uint2*>(dst + 128) = make_uint2(pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
}

// rowsq / rowabs as instinct_stat_rows.  grid (blocks); dynamic shared memory: C floats when colsum is given, then
// the rings (blockDim * S * 16 * (slots of g + slots of m) bytes).
template <int S>
__global__ void __launch_bounds__(512) instinct_stat_rows_s8(InstinctArgs a, const float* __restrict__ colsum, float col_count,
                                                             float* __restrict__ rowsq, float* __restrict__ rowabs) {
  extern __shared__ __align__(16) float sm[];
  float* cs = colsum ? sm : nullptr;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const float b = a.beta, b1 = 1.f - a.beta;
  const int gs = a.g_bf16 ? 1 : 2, ms = a.m_bf16 ? 1 : 2;
  Ring8 ring;
  ring.base = reinterpret_cast<uint4*>(sm + (colsum ? a.C : 0)) + threadIdx.x;
  ring.T = blockDim.x;
  ring.nslot = gs + ms;
  const long long cpr = a.C >> 8;                       // chunks per row
  const long long ER = a.E * a.R;
  const long long lo = ER * blockIdx.x / gridDim.x, hi = ER * (blockIdx.x + 1) / gridDim.x;
  for (long long seg = lo; seg < hi;) {
    const long long e = seg / a.R, seg_hi = min(hi, (e + 1) * a.R);
    if (cs) {
      __syncthreads();
      load_colscale(cs, colsum, nullptr, e, a.C, col_count);
    }
    const long long rpw = (seg_hi - seg + nw - 1) / nw;
    const long long r0 = min(seg_hi, seg + warp * rpw), r1 = min(seg_hi, r0 + rpw);
    const long long total = (r1 - r0) * cpr;
    // both arrays bf16: 8 consecutive elements per lane are one full 16-byte copy each (faster than two 8-byte ones)
    const bool packed = a.g_bf16 && a.m_bf16;
    const long long el0 = r0 * a.C + lane * (packed ? 8 : 4);
    auto issue = [&](int stage, long long k) {
      if (packed) {
        cp_async16(ring.slot(stage, 0), reinterpret_cast<const bf16*>(a.g) + el0 + (k << 8));
        cp_async16(ring.slot(stage, 1), reinterpret_cast<const bf16*>(a.m) + el0 + (k << 8));
      } else {
        ring.issue8(stage, 0, a.g, el0 + (k << 8), a.g_bf16);
        ring.issue8(stage, gs, a.m, el0 + (k << 8), a.m_bf16);
      }
    };
#pragma unroll
    for (int s0 = 0; s0 < S; ++s0) {
      if (s0 < total) issue(s0, s0);
      cp_async_commit();
    }
    int stage = 0;
    long long row = r0, cin = 0;
    float ss = 0.f, sa = 0.f;
    for (long long k = 0; k < total; ++k) {
      cp_async_wait<S - 1>();
      float g[8], m[8];
      ring.read8(stage, 0, a.g_bf16, g);
      ring.read8(stage, gs, a.m_bf16, m);
      if (k + S < total) issue(stage, k + S);
      cp_async_commit();
      const long long c = (cin << 8) + lane * (packed ? 8 : 4);
      float ck[8] = {1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f};
      if (cs) {
        const float4 k0 = *reinterpret_cast<const float4*>(cs + c), k1 = *reinterpret_cast<const float4*>(cs + c + (packed ? 4 : 128));
        ck[0] = k0.x; ck[1] = k0.y; ck[2] = k0.z; ck[3] = k0.w; ck[4] = k1.x; ck[5] = k1.y; ck[6] = k1.z; ck[7] = k1.w;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float v = (b * m[j] + b1 * g[j]) * ck[j];
        ss += v * v;
        sa += fabsf(g[j]);
      }
      if (++cin == cpr) {
        ss = warp_sum(ss);
        if (rowabs) sa = warp_sum(sa);
        if (lane == 0) {
          rowsq[row] = ss;
          if (rowabs) rowabs[row] = sa;
        }
        ++row; cin = 0; ss = 0.f; sa = 0.f;
      }
      if (++stage == S) stage = 0;
    }
    cp_async_wait<0>();
    seg = seg_hi;
  }
}

// The update without the staged last row norm (instinct_apply with fuse_row_norm = 0), streamed.  Stochastic
// rounding keeps the per-element hash of the block-per-row kernel, so both produce the same bits.
// Dynamic shared memory: C floats with column sums, then the rings (g, m and the weight's exact copy).
template <int S>
__global__ void __launch_bounds__(384) instinct_apply_s8(InstinctArgs a, const float* __restrict__ rowsum, float row_count,
                                                         const float* __restrict__ rowsum2, const float* __restrict__ colsum1,
                                                         const float* __restrict__ colsum2, float col_count,
                                                         const float* __restrict__ rowabs, const float* __restrict__ rel2,
                                                         float* __restrict__ rel_out) {
  extern __shared__ __align__(16) float sm[];
  const long long C = a.C;
  const bool has_col = colsum1 || colsum2;
  float* colk = has_col ? sm : nullptr;
  const float lr = *a.lr;
  const float eff = 1.f + (*a.gain - 1.f) * (*a.stake);
  const float step = lr * eff, decay = (a.wd != 0.f) ? 1.f - lr * a.wd : 1.f;
  const uint32_t seed = a.sr ? (uint32_t)((*a.seed) * 1000003ll) * 0x9E3779B9u + a.salt : 0u;
  if (rel_out && blockIdx.x == 0 && threadIdx.x == 0) *rel_out = sqrtf(rel2[0]) / (sqrtf(rel2[1]) + 1e-8f);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const float b = a.beta, b1 = 1.f - a.beta;
  const void* wsrc = a.w ? (const void*)a.w : (const void*)a.p;
  const int w_bf16 = a.w ? 0 : a.p_bf16;
  const int gs = a.g_bf16 ? 1 : 2, ms = a.m_bf16 ? 1 : 2, ws = w_bf16 ? 1 : 2;
  Ring8 ring;
  ring.base = reinterpret_cast<uint4*>(sm + (has_col ? C : 0)) + threadIdx.x;
  ring.T = blockDim.x;
  ring.nslot = gs + ms + ws;
  const long long cpr = C >> 8;
  const long long ER = a.E * a.R;
  const long long lo = ER * blockIdx.x / gridDim.x, hi = ER * (blockIdx.x + 1) / gridDim.x;
  for (long long seg = lo; seg < hi;) {
    const long long e = seg / a.R, seg_hi = min(hi, (e + 1) * a.R);
    if (has_col) {
      __syncthreads();
      load_colscale(colk, colsum1, colsum2, e, C, col_count);
    }
    const long long rpw = (seg_hi - seg + nw - 1) / nw;
    const long long r0 = min(seg_hi, seg + warp * rpw), r1 = min(seg_hi, r0 + rpw);
    const long long total = (r1 - r0) * cpr;
    const long long el0 = r0 * C + lane * 4;
    auto issue = [&](int stage, long long k) {
      ring.issue8(stage, 0, a.g, el0 + (k << 8), a.g_bf16);
      ring.issue8(stage, gs, a.m, el0 + (k << 8), a.m_bf16);
      ring.issue8(stage, gs + ms, wsrc, el0 + (k << 8), w_bf16);
    };
#pragma unroll
    for (int s0 = 0; s0 < S; ++s0) {
      if (s0 < total) issue(s0, s0);
      cp_async_commit();
    }
    int stage = 0;
    long long row = r0, cin = 0;
    float rs = 1.f;
    bool moves = true;
    for (long long k = 0; k < total; ++k) {
      if (cin == 0) {
        rs = rowsum ? scale_of(rowsum[row], row_count) : 1.f;
        if (rowsum2) rs *= scale_of(rowsum2[row] * rs * rs, row_count);
        const bool frozen = a.frozen && a.frozen[(row * C) / a.frozen_stride];
        moves = !(rowabs && !(rowabs[row] > 0.f)) && !frozen;
      }
      cp_async_wait<S - 1>();
      float g[8], m[8], t[8];
      ring.read8(stage, 0, a.g_bf16, g);
      ring.read8(stage, gs, a.m_bf16, m);
      ring.read8(stage, gs + ms, w_bf16, t);
      if (k + S < total) issue(stage, k + S);
      cp_async_commit();
      const long long c = (cin << 8) + lane * 4;
      const long long i0 = el0 + (k << 8);
      float mf[8], upd[8];
      float ck[8] = {1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f};
      if (colk) {
        const float4 k0 = *reinterpret_cast<const float4*>(colk + c), k1 = *reinterpret_cast<const float4*>(colk + c + 128);
        ck[0] = k0.x; ck[1] = k0.y; ck[2] = k0.z; ck[3] = k0.w; ck[4] = k1.x; ck[5] = k1.y; ck[6] = k1.z; ck[7] = k1.w;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        mf[j] = b * m[j] + b1 * g[j];
        upd[j] = mf[j] * rs * ck[j];
      }
      if (a.sr) {                                         // per-element hashes: the 4-wide store path has them
        store_chunk<4>(a, i0, mf, t, upd, moves, step, decay, seed);
        store_chunk<4>(a, i0 + 128, mf + 4, t + 4, upd + 4, moves, step, decay, seed);
      } else {
        if (a.m_bf16) st8_bf16(reinterpret_cast<bf16*>(a.m) + i0, mf);
        else st8_f32(reinterpret_cast<float*>(a.m) + i0, mf);
        if (moves) {
#pragma unroll
          for (int j = 0; j < 8; ++j) t[j] = t[j] * decay - upd[j] * step;
          if (a.w) st8_f32(a.w + i0, t);
          if (a.p_bf16) {
            st8_bf16(reinterpret_cast<bf16*>(a.p) + i0, t);
          } else {
            st8_f32(reinterpret_cast<float*>(a.p) + i0, t);
            if (a.shadow) st8_bf16(reinterpret_cast<bf16*>(a.shadow) + i0, t);
          }
        }
      }
      if (++cin == cpr) { ++row; cin = 0; }
      if (++stage == S) stage = 0;
    }
    cp_async_wait<0>();
    seg = seg_hi;
  }
}

// Lagged homeostasis of a 2-D weight in ONE pass over g, m and the weight: the column norm comes from the previous
// step (`cs_prev`, mean squares; where it is not positive the fresh value `now_sum / R` is used - `now_sum` was made
// by `instinct_rowcol` in that case), the new column sums are gathered on the way into `colsq_out`.
//   u1 = mf * rs1,  col = cs_prev > 0 ? cs_prev : now,  u2 = u1 / (sqrt(col) + eps),  upd = u2 * scale(sum u2^2)
// grid (blocks, 1); dynamic shared memory 3 * C floats (row, column sums of this block, column scales).
template <int VEC>
__global__ void instinct_lag_hs(InstinctArgs a, const float* __restrict__ cs_prev, const float* __restrict__ now_sum,
                                float* __restrict__ colsq_out, const float* __restrict__ rel2, float* __restrict__ rel_out) {
  extern __shared__ float sm[];
  __shared__ float red[32];
  const long long C = a.C;
  float* cache = sm;
  float* colacc = sm + C;
  float* cinv = sm + 2 * C;
  const float lr = *a.lr;
  const float eff = 1.f + (*a.gain - 1.f) * (*a.stake);
  const float step = lr * eff, decay = (a.wd != 0.f) ? 1.f - lr * a.wd : 1.f;
  const uint32_t seed = a.sr ? (uint32_t)((*a.seed) * 1000003ll) * 0x9E3779B9u + a.salt : 0u;
  const float Rf = (float)a.R, Cf = (float)C;
  if (rel_out && blockIdx.x == 0 && threadIdx.x == 0) *rel_out = sqrtf(rel2[0]) / (sqrtf(rel2[1]) + 1e-8f);
  for (long long c = threadIdx.x; c < C; c += blockDim.x) {
    colacc[c] = 0.f;
    const float prev = cs_prev[c];
    const float col = prev > 0.f ? prev : now_sum[c] / Rf;
    cinv[c] = 1.f / (sqrtf(col) + 1e-8f);
  }
  __syncthreads();
  for (long long r = blockIdx.x; r < a.R; r += gridDim.x) {
    const long long base = r * C;
    const bool frozen = a.frozen && a.frozen[base / a.frozen_stride];
    float ss = 0.f;
    for (long long c = (long long)threadIdx.x * VEC; c < C; c += (long long)blockDim.x * VEC) {
      if (VEC == 4) {
        float4 g, v = mom4(a, base + c, g);
        *reinterpret_cast<float4*>(cache + c) = v;
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
      } else {
        float g, v = mom1(a, base + c, g);
        cache[c] = v;
        ss += v * v;
      }
    }
    const float rs1 = scale_of(block_sum(ss, red), Cf);
    float s2 = 0.f;
    for (long long c = (long long)threadIdx.x * VEC; c < C; c += (long long)blockDim.x * VEC) {
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        const float u1 = cache[c + j] * rs1;
        colacc[c + j] += u1 * u1;
        const float u2 = u1 * cinv[c + j];
        s2 += u2 * u2;
      }
    }
    const float rs3 = scale_of(block_sum(s2, red), Cf);
    for (long long c = (long long)threadIdx.x * VEC; c < C; c += (long long)blockDim.x * VEC) {
      float mf[VEC], t[VEC], upd[VEC];
#pragma unroll
      for (int j = 0; j < VEC; ++j) { mf[j] = cache[c + j]; upd[j] = mf[j] * rs1 * cinv[c + j] * rs3; }
      if (!frozen) load_weight<VEC>(a, base + c, t);
      store_chunk<VEC>(a, base + c, mf, t, upd, !frozen, step, decay, seed);
    }
  }
  for (long long c = (long long)threadIdx.x * VEC; c < C; c += (long long)blockDim.x * VEC) {
#pragma unroll
    for (int j = 0; j < VEC; ++j)
      if (colacc[c + j] != 0.f) atomicAdd(colsq_out + c + j, colacc[c + j]);
  }
}

// After a lagged step: cs <- fresh mean squares, *all_positive <- whether every entry is > 0 (then the next step
// needs no fresh statistics), the sums are cleared for the next use.  One block.
static __global__ void instinct_lag_finish(float* __restrict__ cs, float* __restrict__ sums, long long n, float count,
                                           int* __restrict__ all_positive) {
  __shared__ int ok;
  if (threadIdx.x == 0) ok = 1;
  __syncthreads();
  int mine = 1;
  for (long long i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = sums[i] / count;
    cs[i] = v;
    sums[i] = 0.f;
    if (!(v > 0.f)) mine = 0;
  }
  if (!mine) atomicAnd(&ok, 0);
  __syncthreads();
  if (threadIdx.x == 0) *all_positive = ok;
}

// Lagged hs3 (experts): the lagged axis is the row.  rowsum[row] <- cs[row] > 0 ? cs[row] * C : rowsum[row] (so the
// consumers' scale(rowsum, C) gives 1 / (sqrt(col) + eps)), cs[row] <- fresh mean.
static __global__ void instinct_lag_rows_select(float* __restrict__ cs, float* __restrict__ rowsum, long long n, float count) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float fresh = rowsum[i], prev = cs[i];
    rowsum[i] = prev > 0.f ? prev * count : fresh;
    cs[i] = fresh / count;
  }
}

// Scratch layout (fp32, ZEROED by the caller, 16-byte aligned base): [rowA][rowB][rowabs] of pad4(E*R) each,
// [colA][colB] of pad4(E*C) each, [rel 4]; every sub-array starts on a 16-byte boundary.
inline long long instinct_pad4(long long n) { return (n + 3) & ~3ll; }
inline long long instinct_scratch_floats(long long E, long long R, long long C) {
  return 3 * instinct_pad4(E * R) + 2 * instinct_pad4(E * C) + 4;
}

constexpr size_t INSTINCT_SMEM_MAX = 200 * 1024;     // dynamic shared memory the row-staging kernels may ask for

// Launch sequence; returns the number of kernels launched, or -1 when this weight cannot take the requested form
// (nothing is launched then).  `cs` / `cs_ok`: lagged homeostasis state (previous step's second-axis mean squares and
// the "all positive" flag), or null for the exact form.
// `phase` / `col_rows` serve a weight whose rows are split between ranks (kind hs only): phase 1 launches the
// statistics of this rank's rows and stops (the caller then sums the column sums - and the |g|/|w| sums - over the
// ranks, in place in `scratch`), phase 2 launches the update alone; `col_rows` is the row count of the whole weight
// (what a column sum is divided by).  phase 0 = everything, col_rows 0 = the rows of `a`.
inline int64_t instinct_launch(const InstinctArgs& a, int kind, float* scratch, float* rel_out, cudaStream_t st,
                               float* cs = nullptr, int* cs_ok = nullptr, int phase = 0, long long col_rows = 0) {
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
                   (a.w == nullptr || (reinterpret_cast<uintptr_t>(a.w) & 15) == 0) &&
                   (a.shadow == nullptr || (reinterpret_cast<uintptr_t>(a.shadow) & 7) == 0) && (EC % 4 == 0 || a.E == 1);
  int64_t launches = 0;
  const int E = (int)a.E;
  const float Rf = (float)(col_rows > 0 ? col_rows : a.R), Cf = (float)a.C;
  const size_t Cb = (size_t)a.C * sizeof(float);
  if (phase != 0 && (kind != 4 || cs)) return -1;
  const bool stage1 = Cb <= INSTINCT_SMEM_MAX, stage2 = 2 * Cb <= INSTINCT_SMEM_MAX, stage3 = 3 * Cb <= INSTINCT_SMEM_MAX;
  if ((kind == 4 || kind == 5) && !stage1) return -1;          // column scales are staged in shared memory
  if (kind == 4 && cs && !stage3) return -1;                   // lagged hs stages three rows
  // blocks per expert of a row kernel that stages `smem` bytes: as many blocks per SM as fit (at most 8)
  auto blocks_per_expert = [&](size_t smem) {
    const long long per_sm = std::max<long long>(1, std::min<long long>(8, (220 * 1024) / (long long)(smem + 1024)));
    return (int)std::max<long long>(1, std::min<long long>(a.R, (148 * per_sm + E - 1) / E));
  };
  const int row_threads = a.C >= 1024 ? 256 : (a.C >= 256 ? 128 : 64);
  // the dynamic shared-memory limit is a per-device attribute of each kernel: raise it whenever more than the
  // default 48 KB is asked for (the call is cheap)
  auto raise = [](auto kern, size_t smem) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)INSTINCT_SMEM_MAX);
  };
  // streaming forms: 16-byte accesses on every array, whole chunks of 256 columns, enough rows to fill the GPU
  const bool s8 = vec && a.C % 256 == 0 && (a.shadow == nullptr || (reinterpret_cast<uintptr_t>(a.shadow) & 15) == 0) &&
                  ER >= 148 * 16;
  constexpr size_t S8_SMEM = 216 * 1024;
  // launch `kern<S>` with the deepest ring that fits beside `head` bytes: T threads, `slots` 16-byte slots per stage
  auto s8_launch = [&](auto k12, auto k8, auto k6, auto k4, int T, int slots, size_t head, auto&&... args) {
    const size_t per = (size_t)T * slots * 16;
    const int S = head + 12 * per <= S8_SMEM ? 12 : head + 8 * per <= S8_SMEM ? 8 : head + 6 * per <= S8_SMEM ? 6 : 4;
    const size_t smem = head + S * per;
    auto go = [&](auto kern) {
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)S8_SMEM);
      kern<<<148, T, smem, st>>>(args...);
    };
    if (S == 12) go(k12); else if (S == 8) go(k8); else if (S == 6) go(k6); else go(k4);
    ++launches;
  };
  auto stat_rows = [&](const float* colsum, float* out, float* absout) {
    const size_t smem = colsum ? Cb : 0;
    if (s8 && smem + 4 * 512 * 4 * 16 <= S8_SMEM) {
      s8_launch(instinct_stat_rows_s8<12>, instinct_stat_rows_s8<8>, instinct_stat_rows_s8<6>, instinct_stat_rows_s8<4>, 512,
                (a.g_bf16 ? 1 : 2) + (a.m_bf16 ? 1 : 2), smem, a, colsum, Rf, out, absout);
      return;
    }
    dim3 grid(blocks_per_expert(smem), E);
    if (vec) { raise(instinct_stat_rows<4>, smem); instinct_stat_rows<4><<<grid, row_threads, smem, st>>>(a, colsum, Rf, out, absout); }
    else { raise(instinct_stat_rows<1>, smem); instinct_stat_rows<1><<<grid, row_threads, smem, st>>>(a, colsum, Rf, out, absout); }
    ++launches;
  };
  auto stat_cols = [&](const float* colsum, const float* rowsum, float* out) {
    const int V = vec ? 4 : 1;
    const int threads = 128;
    const int strips = (int)((a.C + (long long)threads * V - 1) / ((long long)threads * V));
    long long want_chunks = std::max<long long>(1, (148 * 8) / std::max<long long>(1, (long long)strips * a.E));
    int rows_per_block = (int)std::max<long long>(8, (a.R + want_chunks - 1) / want_chunks);
    int chunks = (int)((a.R + rows_per_block - 1) / rows_per_block);
    dim3 grid(strips, chunks, (unsigned)a.E);
    const size_t smem = rowsum ? (size_t)rows_per_block * sizeof(float) : 0;     // <= R floats; raised when above 48 KB
    if (vec) { raise(instinct_stat_cols<4>, smem); instinct_stat_cols<4><<<grid, threads, smem, st>>>(a, colsum, Rf, rowsum, Cf, out, rows_per_block); }
    else { raise(instinct_stat_cols<1>, smem); instinct_stat_cols<1><<<grid, threads, smem, st>>>(a, colsum, Rf, rowsum, Cf, out, rows_per_block); }
    ++launches;
  };
  auto rowcol = [&](const float* colsum_in, float* rows_out, float* cols_out, const int* skip_if) {
    const size_t smem = (colsum_in ? 3 : 2) * Cb;
    dim3 grid(blocks_per_expert(smem), E);
    if (vec) { raise(instinct_rowcol<4>, smem); instinct_rowcol<4><<<grid, row_threads, smem, st>>>(a, colsum_in, Rf, rows_out, cols_out, skip_if); }
    else { raise(instinct_rowcol<1>, smem); instinct_rowcol<1><<<grid, row_threads, smem, st>>>(a, colsum_in, Rf, rows_out, cols_out, skip_if); }
    ++launches;
  };
  auto apply = [&](const float* rs, const float* rs2, const float* c1, const float* c2, bool fuse, const float* rabs) {
    const size_t smem = ((c1 || c2) ? Cb : 0) + (fuse ? Cb : 0);
    if (s8 && !fuse && smem + 4 * 384 * 6 * 16 <= S8_SMEM) {
      const int slots = (a.g_bf16 ? 1 : 2) + (a.m_bf16 ? 1 : 2) + ((a.w == nullptr && a.p_bf16) ? 1 : 2);
      s8_launch(instinct_apply_s8<12>, instinct_apply_s8<8>, instinct_apply_s8<6>, instinct_apply_s8<4>, 384, slots, smem, a, rs,
                Cf, rs2, c1, c2, Rf, rabs, rel2, rel_out);
      return;
    }
    dim3 grid(blocks_per_expert(smem), E);
    if (vec) { raise(instinct_apply<4>, smem); instinct_apply<4><<<grid, row_threads, smem, st>>>(a, rs, Cf, rs2, c1, c2, Rf, fuse ? 1 : 0, rabs, rel2, rel_out); }
    else { raise(instinct_apply<1>, smem); instinct_apply<1><<<grid, row_threads, smem, st>>>(a, rs, Cf, rs2, c1, c2, Rf, fuse ? 1 : 0, rabs, rel2, rel_out); }
    ++launches;
  };
  if (rel_out && phase != 2) {
    const int grid = (int)std::max<long long>(1, std::min<long long>((n + 255) / 256, 148 * 8));
    instinct_rel_sums<<<grid, 256, 0, st>>>(a, rel2);
    ++launches;
  }
  switch (kind) {
    case 4: {  // hs: rows, columns, rows again
      if (cs) {
        // lagged: fresh column sums only if the previous step left a non-positive entry, then one pass
        rowcol(nullptr, nullptr, colA, cs_ok);
        const int lag_grid = blocks_per_expert(3 * Cb);
        if (vec) { raise(instinct_lag_hs<4>, 3 * Cb); instinct_lag_hs<4><<<lag_grid, row_threads, 3 * Cb, st>>>(a, cs, colA, colB, rel2, rel_out); }
        else { raise(instinct_lag_hs<1>, 3 * Cb); instinct_lag_hs<1><<<lag_grid, row_threads, 3 * Cb, st>>>(a, cs, colA, colB, rel2, rel_out); }
        instinct_lag_finish<<<1, 1024, 0, st>>>(cs, colB, a.C, Rf, cs_ok);
        launches += 2;
        break;
      }
      if (phase != 2) {
        stat_rows(nullptr, rowA, nullptr);
        stat_cols(nullptr, rowA, colA);
      }
      if (phase == 1) break;
      if (stage2) {
        apply(rowA, nullptr, colA, nullptr, true, nullptr);        // the last row norm on the row staged in shared memory
      } else {
        stat_rows(colA, rowB, nullptr);            // sum_c (mf cs)^2; times rs1^2 inside apply = row sums of u2
        apply(rowA, rowB, colA, nullptr, false, nullptr);
      }
      break;
    }
    case 5:   // hs3: over R (per column), over C (per row), over R again
      stat_cols(nullptr, nullptr, colA);
      stat_rows(colA, rowA, nullptr);
      if (cs) {
        instinct_lag_rows_select<<<(int)std::max<long long>(1, std::min<long long>((ER + 255) / 256, 592)), 256, 0, st>>>(cs, rowA, ER, Cf);
        ++launches;
      }
      stat_cols(colA, rowA, colB);
      apply(rowA, nullptr, colA, colB, false, nullptr);
      break;
    case 3:   // word table: row rms, only rows with a gradient move
      stat_rows(nullptr, rowA, rowabs);
      apply(rowA, nullptr, nullptr, nullptr, false, rowabs);
      break;
    case 2:   // experts (E, in, out): one norm per (expert, output column) over `in`
      stat_cols(nullptr, nullptr, colA);
      apply(nullptr, nullptr, colA, nullptr, false, nullptr);
      break;
    default:  // kinds 0 and 1: one norm per row of the (E*R, C) view (the whole tensor when E = R = 1)
      stat_rows(nullptr, rowA, nullptr);
      apply(rowA, nullptr, nullptr, nullptr, false, nullptr);
      break;
  }
  return launches;
}

}  // namespace mb
