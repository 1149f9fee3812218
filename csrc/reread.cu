// Re-reading at a bookmark, one kernel forward and one backward.
//
// A word has scored every card of its text's memory (`sc`, the same face-cosine scores as the memory read).  Here it
//   picks its k best cards,                               p = softmax(top scores), w = p where the card is real
//   jumps to each card's bookmark `pos` and reads up to R raw tokens of the text from there: v_r = book[id_r] + offset_r
//   with a halting gate per token (ACT style):             halt_r = sigmoid(<hv, v_r> + hb + hh), forced to 1 on the
//                                                          last token and wherever the position is not yet written
//                                                          (rpos >= the word's own position)
//   read = sum_r surv_r halt_r v_r,  surv_0 = 1, surv_{r+1} = surv_r (1 - halt_r)
//   the card checks what was read: recog = sigmoid(4 cos(Wr read, cp[card]))
//   got  = sum_j w_j recog_j read_j        (Db wide; the module's output projection follows)
//   cost = sum_j w_j sum_r surv_r          (expected tokens read, over readable positions)
// (reference: Reread.forward, full2.py:184-280).
//
// One warp per word; the book width is 128 (4 floats per lane) and the face width 64 (2 per lane).  Nothing of shape
// (words, k, R, Db) reaches HBM: the forward keeps the tokens' vectors in registers, the backward recomputes them.
// Backward: gradients of book rows by vector red.global.add, of the card projections by scalar atomics, of the small
// shared weights (Wr, hv, offset) in per-block accumulators - the Wr outer products as a rank-8 update of a register
// tile per block - flushed once per block.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda_bf16.h>

#include "common.cuh"

namespace mb {

constexpr int RR_WARPS = 8, RR_DB = 128, RR_F = 64, RR_MAXK = 8, RR_MAXR = 4, RR_MAXC = 512;

struct RRArgs {
  const float* sc;            // (B,S,C) card scores, -1e4 on empty cards
  const long long* pos;       // (B,C) bookmark of every card
  const long long* qpos;      // (B,S) text position of every word
  const long long* rows;      // (B) text of every batch row
  const long long* ids;       // (texts, Tb) token ids
  const void* table;          // (V,128) shelf of raw token vectors, fp32 or bf16
  int table_bf16;
  const float* offset;        // (R,128)
  const float* hv;            // (128)
  const float* hb;            // (1)
  const float* hh;            // (B,S) the word's own halting bias
  const float* Wr;            // (64,128)
  const float* cp;            // (B,C,64) card projections
  int B, S, C, k, R, Tb;
};

__device__ __forceinline__ float4 rr_load_row(const RRArgs& a, long long id, int lane) {
  if (a.table_bf16) {
    const uint2 u = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(a.table) + id * RR_DB + lane * 4);
    const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
    const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
    return make_float4(lo.x, lo.y, hi.x, hi.y);
  }
  return *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(a.table) + id * RR_DB + lane * 4);
}
__device__ __forceinline__ float dot4(const float4& a, const float4& b) { return a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w; }
__device__ __forceinline__ void fma4(float4& acc, float s, const float4& v) {
  acc.x += s * v.x; acc.y += s * v.y; acc.z += s * v.z; acc.w += s * v.w;
}
__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }
__device__ __forceinline__ void red_add_v4(float* addr, const float4& v) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

// k best cards of one word (all lanes get the same answer); ties go to the lower card index.
__device__ __forceinline__ void rr_topk(const float* row, int C, int k, int lane, float* top_s, int* top_j) {
  float v[RR_MAXC / 32];
#pragma unroll
  for (int i = 0; i < RR_MAXC / 32; ++i) {
    const int c = i * 32 + lane;
    v[i] = c < C ? row[c] : -INFINITY;
  }
  for (int j = 0; j < k; ++j) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < RR_MAXC / 32; ++i)
      if (v[i] > bv) { bv = v[i]; bi = i * 32 + lane; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    top_s[j] = bv;
    top_j[j] = bi;
#pragma unroll
    for (int i = 0; i < RR_MAXC / 32; ++i)
      if (i * 32 + lane == bi) v[i] = -INFINITY;
  }
}

// What one (word, card) pair reads.  Fills the per-token state the backward needs.
struct RRRead {
  float4 v[RR_MAXR];
  float halt[RR_MAXR], surv[RR_MAXR], rd[RR_MAXR];
  long long id[RR_MAXR];
  float4 read;
  float cs;                     // sum_r surv_r over readable positions
};

__device__ __forceinline__ void rr_read(const RRArgs& a, long long mark, long long qp, long long row, float hhv, const float4& hv4,
                                        float hb, int lane, RRRead& o) {
  o.read = make_float4(0.f, 0.f, 0.f, 0.f);
  o.cs = 0.f;
  float surv = 1.f;
#pragma unroll
  for (int r = 0; r < RR_MAXR; ++r) {
    if (r < a.R) {
      const long long rp = mark + r;
      const float rd = rp < qp ? 1.f : 0.f;
      const long long rpc = rp < 0 ? 0 : (rp > a.Tb - 1 ? a.Tb - 1 : rp);
      const long long id = a.ids[row * a.Tb + rpc];
      float4 v = rr_load_row(a, id, lane);
      const float4 off = *reinterpret_cast<const float4*>(a.offset + r * RR_DB + lane * 4);
      v.x += off.x; v.y += off.y; v.z += off.z; v.w += off.w;
      const float act = warp_sum(dot4(v, hv4)) + hb + hhv;
      const float halt = (rd != 0.f && r < a.R - 1) ? sigmoidf_(act) : 1.f;
      o.v[r] = v; o.id[r] = id; o.rd[r] = rd; o.halt[r] = halt; o.surv[r] = surv;
      fma4(o.read, surv * halt * rd, v);
      o.cs += surv * rd;
      surv *= 1.f - halt;
    }
  }
}

// Recognition of one read by its card: rr = Wr read (two features per lane), cosine against the card's projection.
struct RRRecog { float rr0, rr1, cp0, cp1, nr, nc, cos, recog; };

__device__ __forceinline__ void rr_recog(const float* WrT, const float* read_s, const float* cpj, int lane, RRRecog& g) {
  float r0 = 0.f, r1 = 0.f;
#pragma unroll 8
  for (int d = 0; d < RR_DB; ++d) {
    const float x = read_s[d];
    r0 += WrT[d * RR_F + lane] * x;
    r1 += WrT[d * RR_F + 32 + lane] * x;
  }
  g.rr0 = r0; g.rr1 = r1;
  g.cp0 = cpj[lane]; g.cp1 = cpj[32 + lane];
  g.nr = fmaxf(sqrtf(warp_sum(r0 * r0 + r1 * r1)), 1e-12f);
  g.nc = fmaxf(sqrtf(warp_sum(g.cp0 * g.cp0 + g.cp1 * g.cp1)), 1e-12f);
  g.cos = warp_sum(r0 * g.cp0 + r1 * g.cp1) / (g.nr * g.nc);
  g.recog = sigmoidf_(4.f * g.cos);
}

__device__ __forceinline__ void rr_softmax(const float* top_s, int k, float* p) {
  float mx = -INFINITY;
  for (int j = 0; j < k; ++j) mx = fmaxf(mx, top_s[j]);
  float sum = 0.f;
  for (int j = 0; j < k; ++j) { p[j] = expf(top_s[j] - mx); sum += p[j]; }
  const float inv = 1.f / sum;
  for (int j = 0; j < k; ++j) p[j] *= inv;
}

// grid: blocks of 8 warps striding over the words.
__global__ void __launch_bounds__(RR_WARPS * 32) reread_fwd_kernel(RRArgs a, float* __restrict__ got, float* __restrict__ costw,
                                                                    int* __restrict__ top_j_out, float* __restrict__ p_out) {
  extern __shared__ float sh[];
  float* WrT = sh;                                   // (128, 64): Wr transposed, so a lane's feature is bank-conflict free
  float* read_s = WrT + RR_DB * RR_F;                // per warp 128
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < RR_DB * RR_F; i += blockDim.x) {
    const int f = i / RR_DB, d = i - f * RR_DB;
    WrT[d * RR_F + f] = a.Wr[i];
  }
  __syncthreads();
  float* rs = read_s + warp * RR_DB;
  const float4 hv4 = *reinterpret_cast<const float4*>(a.hv + lane * 4);
  const float hb = *a.hb;
  const long long words = (long long)a.B * a.S;
  for (long long wi = (long long)blockIdx.x * RR_WARPS + warp; wi < words; wi += (long long)gridDim.x * RR_WARPS) {
    const int b = (int)(wi / a.S);
    float top_s[RR_MAXK], p[RR_MAXK];
    int top_j[RR_MAXK];
    rr_topk(a.sc + wi * a.C, a.C, a.k, lane, top_s, top_j);
    rr_softmax(top_s, a.k, p);
    const long long qp = a.qpos[wi], row = a.rows[b];
    const float hhv = a.hh[wi];
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float cost = 0.f;
    for (int j = 0; j < a.k; ++j) {
      const float w = top_s[j] > -1e3f ? p[j] : 0.f;
      RRRead rd;
      rr_read(a, a.pos[(long long)b * a.C + top_j[j]], qp, row, hhv, hv4, hb, lane, rd);
      __syncwarp();
      *reinterpret_cast<float4*>(rs + lane * 4) = rd.read;
      __syncwarp();
      RRRecog g;
      rr_recog(WrT, rs, a.cp + ((long long)b * a.C + top_j[j]) * RR_F, lane, g);
      fma4(acc, w * g.recog, rd.read);
      cost += w * rd.cs;
    }
    *reinterpret_cast<float4*>(got + wi * RR_DB + lane * 4) = acc;
    if (lane == 0) costw[wi] = cost;
    if (lane < a.k) {
      // every lane holds all k entries: pick by index without dynamic register indexing
      int tj = 0;
      float pj = 0.f;
#pragma unroll
      for (int j = 0; j < RR_MAXK; ++j)
        if (j == lane) { tj = top_j[j]; pj = p[j]; }
      top_j_out[wi * a.k + lane] = tj;
      p_out[wi * a.k + lane] = pj;
    }
  }
}

struct RRGrads {
  const float* dgot;          // (B,S,128)
  const float* dcostw;        // (B,S)
  const int* top_j;           // (B,S,k)
  const float* p;             // (B,S,k)
  float* dsc;                 // (B,S,C) zero-filled
  float* dtable;              // (V,128) zero-filled, fp32
  float* doffset;             // (R,128) zero-filled
  float* dhv;                 // (128)
  float* dhb;                 // (1)
  float* dhh;                 // (B,S)
  float* dWr;                 // (64,128) zero-filled
  float* dcp;                 // (B,C,64) zero-filled
};

__global__ void __launch_bounds__(RR_WARPS * 32) reread_bwd_kernel(RRArgs a, RRGrads g) {
  extern __shared__ float sh[];
  float* WrT = sh;                                   // (128,64)
  float* Wr_s = WrT + RR_DB * RR_F;                  // (64,128)
  float* read_s = Wr_s + RR_DB * RR_F;               // 8 x 128
  float* drr_s = read_s + RR_WARPS * RR_DB;          // 8 x 64
  float* red_s = drr_s + RR_WARPS * RR_F;            // RR_MAXR*128 (offset) + 128 (hv) + 1 (hb)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < RR_DB * RR_F; i += blockDim.x) {
    const int f = i / RR_DB, d = i - f * RR_DB;
    const float x = a.Wr[i];
    Wr_s[i] = x;
    WrT[d * RR_F + f] = x;
  }
  for (int i = threadIdx.x; i < RR_MAXR * RR_DB + RR_DB + 1; i += blockDim.x) red_s[i] = 0.f;
  __syncthreads();
  float* rs = read_s + warp * RR_DB;
  float* ds = drr_s + warp * RR_F;
  const float4 hv4 = *reinterpret_cast<const float4*>(a.hv + lane * 4);
  const float hb = *a.hb;
  // this thread's tile of the Wr gradient: feature fo, columns d0 .. d0 + 31
  const int fo = threadIdx.x >> 2, d0 = (threadIdx.x & 3) * 32;
  float wacc[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) wacc[i] = 0.f;
  float4 doff[RR_MAXR];
#pragma unroll
  for (int r = 0; r < RR_MAXR; ++r) doff[r] = make_float4(0.f, 0.f, 0.f, 0.f);
  float4 dhv4 = make_float4(0.f, 0.f, 0.f, 0.f);
  float dhb_acc = 0.f;

  const long long words = (long long)a.B * a.S;
  const long long stride = (long long)gridDim.x * RR_WARPS;
  // all warps of a block run the same number of rounds (the Wr update is a block-wide step)
  for (long long w0 = (long long)blockIdx.x * RR_WARPS; w0 < words; w0 += stride) {
    const long long wi = w0 + warp;
    const bool live = wi < words;
    const int b = live ? (int)(wi / a.S) : 0;
    float p[RR_MAXK], dw[RR_MAXK];
    int top_j[RR_MAXK];
    bool real[RR_MAXK];
    float4 dgot4 = make_float4(0.f, 0.f, 0.f, 0.f);
    float dcw = 0.f, hhv = 0.f, dhh_acc = 0.f;
    long long qp = 0, row = 0;
    if (live) {
#pragma unroll
      for (int j = 0; j < RR_MAXK; ++j) {
        if (j < a.k) {
          top_j[j] = g.top_j[wi * a.k + j];
          p[j] = g.p[wi * a.k + j];
          real[j] = a.sc[wi * a.C + top_j[j]] > -1e3f;
        }
      }
      dgot4 = *reinterpret_cast<const float4*>(g.dgot + wi * RR_DB + lane * 4);
      dcw = g.dcostw[wi];
      hhv = a.hh[wi];
      qp = a.qpos[wi];
      row = a.rows[b];
    }
    for (int j = 0; j < a.k; ++j) {
      float drr0 = 0.f, drr1 = 0.f;
      float4 rdv = make_float4(0.f, 0.f, 0.f, 0.f);
      if (live) {
        const float w = real[j] ? p[j] : 0.f;
        const long long card = (long long)b * a.C + top_j[j];
        RRRead rd;
        rr_read(a, a.pos[card], qp, row, hhv, hv4, hb, lane, rd);
        __syncwarp();
        *reinterpret_cast<float4*>(rs + lane * 4) = rd.read;
        __syncwarp();
        RRRecog rc;
        rr_recog(WrT, rs, a.cp + card * RR_F, lane, rc);
        const float gr = warp_sum(dot4(dgot4, rd.read));
        dw[j] = gr * rc.recog + dcw * rd.cs;
        const float dcos = w * gr * rc.recog * (1.f - rc.recog) * 4.f;
        // cos = <rr, cp> / (|rr| |cp|)
        const float rn0 = rc.rr0 / rc.nr, rn1 = rc.rr1 / rc.nr, cn0 = rc.cp0 / rc.nc, cn1 = rc.cp1 / rc.nc;
        drr0 = (cn0 - rn0 * rc.cos) / rc.nr * dcos;
        drr1 = (cn1 - rn1 * rc.cos) / rc.nr * dcos;
        if (dcos != 0.f) {
          atomicAdd(g.dcp + card * RR_F + lane, (rn0 - cn0 * rc.cos) / rc.nc * dcos);
          atomicAdd(g.dcp + card * RR_F + 32 + lane, (rn1 - cn1 * rc.cos) / rc.nc * dcos);
        }
        ds[lane] = drr0;
        ds[32 + lane] = drr1;
        __syncwarp();
        // d read = w recog dgot + Wr^T d rr
        float4 dread = make_float4(0.f, 0.f, 0.f, 0.f);
        fma4(dread, w * rc.recog, dgot4);
        if (dcos != 0.f) {
#pragma unroll 8
          for (int f = 0; f < RR_F; ++f) fma4(dread, ds[f], *reinterpret_cast<const float4*>(Wr_s + f * RR_DB + lane * 4));
        }
        float dsurv_next = 0.f;
#pragma unroll
        for (int r = RR_MAXR - 1; r >= 0; --r) {
          if (r < a.R) {
            const float dc = warp_sum(dot4(dread, rd.v[r]));
            const float c = rd.surv[r] * rd.halt[r] * rd.rd[r];
            const float dhalt = dc * rd.surv[r] * rd.rd[r] - dsurv_next * rd.surv[r];
            const float dsurv = dc * rd.halt[r] * rd.rd[r] + dcw * w * rd.rd[r] + dsurv_next * (1.f - rd.halt[r]);
            const float da = (rd.rd[r] != 0.f && r < a.R - 1) ? dhalt * rd.halt[r] * (1.f - rd.halt[r]) : 0.f;
            dsurv_next = dsurv;
            if (c != 0.f || da != 0.f) {
              float4 dv = make_float4(0.f, 0.f, 0.f, 0.f);
              fma4(dv, c, dread);
              fma4(dv, da, hv4);
              fma4(dhv4, da, rd.v[r]);
              dhb_acc += da;
              dhh_acc += da;
              fma4(doff[r], 1.f, dv);
              red_add_v4(g.dtable + rd.id[r] * RR_DB + lane * 4, dv);
            }
          }
        }
        rdv = rd.read;
      } else {
        ds[lane] = 0.f;
        ds[32 + lane] = 0.f;
        *reinterpret_cast<float4*>(rs + lane * 4) = rdv;
      }
      // Wr gradient: the block's 8 (d rr, read) pairs as a rank-8 update of the register tile
      __syncthreads();
#pragma unroll
      for (int w8 = 0; w8 < RR_WARPS; ++w8) {
        const float x = drr_s[w8 * RR_F + fo];
        if (x != 0.f) {
#pragma unroll
          for (int i = 0; i < 32; ++i) wacc[i] += x * read_s[w8 * RR_DB + d0 + i];
        }
      }
      __syncthreads();
    }
    if (live) {
      // softmax over the k picked scores; empty cards took no gradient (their weight is a constant 0)
      float dot = 0.f;
      for (int j = 0; j < a.k; ++j) dot += p[j] * (real[j] ? dw[j] : 0.f);
      if (lane == 0) {
        for (int j = 0; j < a.k; ++j)
          if (real[j]) g.dsc[wi * a.C + top_j[j]] = p[j] * (dw[j] - dot);
        g.dhh[wi] = dhh_acc;
      }
    }
  }
  // flush the block's accumulators
#pragma unroll
  for (int r = 0; r < RR_MAXR; ++r) {
    if (r < a.R) {
      atomicAdd(&red_s[r * RR_DB + lane * 4 + 0], doff[r].x);
      atomicAdd(&red_s[r * RR_DB + lane * 4 + 1], doff[r].y);
      atomicAdd(&red_s[r * RR_DB + lane * 4 + 2], doff[r].z);
      atomicAdd(&red_s[r * RR_DB + lane * 4 + 3], doff[r].w);
    }
  }
  atomicAdd(&red_s[RR_MAXR * RR_DB + lane * 4 + 0], dhv4.x);
  atomicAdd(&red_s[RR_MAXR * RR_DB + lane * 4 + 1], dhv4.y);
  atomicAdd(&red_s[RR_MAXR * RR_DB + lane * 4 + 2], dhv4.z);
  atomicAdd(&red_s[RR_MAXR * RR_DB + lane * 4 + 3], dhv4.w);
  if (lane == 0) atomicAdd(&red_s[RR_MAXR * RR_DB + RR_DB], dhb_acc);
  __syncthreads();
  for (int i = threadIdx.x; i < a.R * RR_DB; i += blockDim.x) atomicAdd(g.doffset + i, red_s[i]);
  for (int i = threadIdx.x; i < RR_DB; i += blockDim.x) atomicAdd(g.dhv + i, red_s[RR_MAXR * RR_DB + i]);
  if (threadIdx.x == 0) atomicAdd(g.dhb, red_s[RR_MAXR * RR_DB + RR_DB]);
#pragma unroll
  for (int i = 0; i < 32; ++i) atomicAdd(g.dWr + fo * RR_DB + d0 + i, wacc[i]);
}

// ------------------------------------------------------------------------------------------------ host side
static void rr_fill(RRArgs& a, const torch::Tensor& sc, const torch::Tensor& pos, const torch::Tensor& qpos,
                    const torch::Tensor& rows, const torch::Tensor& ids, const torch::Tensor& table, const torch::Tensor& offset,
                    const torch::Tensor& hv, const torch::Tensor& hb, const torch::Tensor& hh, const torch::Tensor& Wr,
                    const torch::Tensor& cp, int64_t k) {
  auto f32 = [](const torch::Tensor& t) { return t.is_cuda() && t.is_contiguous() && t.scalar_type() == torch::kFloat32; };
  auto i64 = [](const torch::Tensor& t) { return t.is_cuda() && t.is_contiguous() && t.scalar_type() == torch::kInt64; };
  TORCH_CHECK(sc.dim() == 3 && f32(sc), "reread: sc (B,S,C) fp32");
  a.B = (int)sc.size(0); a.S = (int)sc.size(1); a.C = (int)sc.size(2);
  TORCH_CHECK(a.C <= RR_MAXC, "reread: at most ", RR_MAXC, " cards");
  TORCH_CHECK(i64(pos) && pos.numel() == (long long)a.B * a.C, "reread: pos (B,C) int64");
  TORCH_CHECK(i64(qpos) && qpos.numel() == (long long)a.B * a.S, "reread: qpos (B,S) int64");
  TORCH_CHECK(i64(rows) && rows.numel() == a.B, "reread: rows (B) int64");
  TORCH_CHECK(i64(ids) && ids.dim() == 2, "reread: ids (texts,T) int64");
  TORCH_CHECK(table.is_cuda() && table.is_contiguous() && table.dim() == 2 && table.size(1) == RR_DB &&
              (table.scalar_type() == torch::kFloat32 || table.scalar_type() == torch::kBFloat16), "reread: table (V,128)");
  TORCH_CHECK(f32(offset) && offset.dim() == 2 && offset.size(1) == RR_DB && offset.size(0) >= 1 && offset.size(0) <= RR_MAXR,
              "reread: offset (R<=4,128) fp32");
  TORCH_CHECK(f32(hv) && hv.numel() == RR_DB && f32(hb) && hb.numel() == 1, "reread: halting weights");
  TORCH_CHECK(f32(hh) && hh.numel() == (long long)a.B * a.S, "reread: hh (B,S)");
  TORCH_CHECK(f32(Wr) && Wr.dim() == 2 && Wr.size(0) == RR_F && Wr.size(1) == RR_DB, "reread: Wr (64,128)");
  TORCH_CHECK(f32(cp) && cp.numel() == (long long)a.B * a.C * RR_F, "reread: cp (B,C,64)");
  TORCH_CHECK(k >= 1 && k <= RR_MAXK && k <= a.C, "reread: 1 <= k <= min(8, C)");
  a.sc = sc.data_ptr<float>();
  a.pos = reinterpret_cast<const long long*>(pos.data_ptr<int64_t>());
  a.qpos = reinterpret_cast<const long long*>(qpos.data_ptr<int64_t>());
  a.rows = reinterpret_cast<const long long*>(rows.data_ptr<int64_t>());
  a.ids = reinterpret_cast<const long long*>(ids.data_ptr<int64_t>());
  a.table = table.data_ptr(); a.table_bf16 = table.scalar_type() == torch::kBFloat16;
  a.offset = offset.data_ptr<float>(); a.hv = hv.data_ptr<float>(); a.hb = hb.data_ptr<float>(); a.hh = hh.data_ptr<float>();
  a.Wr = Wr.data_ptr<float>(); a.cp = cp.data_ptr<float>();
  a.k = (int)k; a.R = (int)offset.size(0); a.Tb = (int)ids.size(1);
}

static int rr_grid(long long words) {
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long want = (words + RR_WARPS - 1) / RR_WARPS;
  return (int)std::max<long long>(1, std::min<long long>(want, 2LL * sms));
}

std::vector<torch::Tensor> reread_fwd(torch::Tensor sc, torch::Tensor pos, torch::Tensor qpos, torch::Tensor rows,
                                      torch::Tensor ids, torch::Tensor table, torch::Tensor offset, torch::Tensor hv,
                                      torch::Tensor hb, torch::Tensor hh, torch::Tensor Wr, torch::Tensor cp, int64_t k) {
  const c10::cuda::CUDAGuard guard(sc.device());
  RRArgs a;
  rr_fill(a, sc, pos, qpos, rows, ids, table, offset, hv, hb, hh, Wr, cp, k);
  auto got = torch::empty({a.B, a.S, RR_DB}, sc.options());
  auto costw = torch::empty({a.B, a.S}, sc.options());
  auto top_j = torch::empty({a.B, a.S, (int64_t)k}, sc.options().dtype(torch::kInt32));
  auto p = torch::empty({a.B, a.S, (int64_t)k}, sc.options());
  const long long words = (long long)a.B * a.S;
  if (words == 0) return {got, costw, top_j, p};
  const size_t smem = ((size_t)RR_DB * RR_F + RR_WARPS * RR_DB) * sizeof(float);
  TORCH_CHECK(cudaFuncSetAttribute(reread_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess,
              "reread: shared memory");
  reread_fwd_kernel<<<rr_grid(words), RR_WARPS * 32, smem, at::cuda::getCurrentCUDAStream()>>>(
      a, got.data_ptr<float>(), costw.data_ptr<float>(), top_j.data_ptr<int>(), p.data_ptr<float>());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {got, costw, top_j, p};
}

// Returns (dsc, dtable fp32, doffset, dhv, dhb, dhh, dWr, dcp).
std::vector<torch::Tensor> reread_bwd(torch::Tensor dgot, torch::Tensor dcostw, torch::Tensor top_j, torch::Tensor p,
                                      torch::Tensor sc, torch::Tensor pos, torch::Tensor qpos, torch::Tensor rows,
                                      torch::Tensor ids, torch::Tensor table, torch::Tensor offset, torch::Tensor hv,
                                      torch::Tensor hb, torch::Tensor hh, torch::Tensor Wr, torch::Tensor cp) {
  const c10::cuda::CUDAGuard guard(sc.device());
  RRArgs a;
  const int64_t k = top_j.size(-1);
  rr_fill(a, sc, pos, qpos, rows, ids, table, offset, hv, hb, hh, Wr, cp, k);
  TORCH_CHECK(dgot.is_contiguous() && dgot.scalar_type() == torch::kFloat32 && dgot.numel() == (long long)a.B * a.S * RR_DB,
              "reread_bwd: dgot (B,S,128) fp32");
  TORCH_CHECK(dcostw.is_contiguous() && dcostw.scalar_type() == torch::kFloat32 && dcostw.numel() == (long long)a.B * a.S,
              "reread_bwd: dcostw (B,S) fp32");
  TORCH_CHECK(top_j.is_contiguous() && top_j.scalar_type() == torch::kInt32 && p.is_contiguous() &&
              p.scalar_type() == torch::kFloat32 && p.numel() == top_j.numel(), "reread_bwd: saved picks");
  RRGrads g;
  auto dsc = torch::zeros_like(sc);
  auto dtable = torch::zeros({table.size(0), RR_DB}, sc.options());
  auto doffset = torch::zeros_like(offset);
  auto dhv = torch::zeros({RR_DB}, sc.options());
  auto dhb = torch::zeros({1}, sc.options());
  auto dhh = torch::zeros({a.B, a.S}, sc.options());
  auto dWr = torch::zeros_like(Wr);
  auto dcp = torch::zeros_like(cp);
  const long long words = (long long)a.B * a.S;
  if (words == 0) return {dsc, dtable, doffset, dhv, dhb, dhh, dWr, dcp};
  g.dgot = dgot.data_ptr<float>(); g.dcostw = dcostw.data_ptr<float>(); g.top_j = top_j.data_ptr<int>(); g.p = p.data_ptr<float>();
  g.dsc = dsc.data_ptr<float>(); g.dtable = dtable.data_ptr<float>(); g.doffset = doffset.data_ptr<float>();
  g.dhv = dhv.data_ptr<float>(); g.dhb = dhb.data_ptr<float>(); g.dhh = dhh.data_ptr<float>(); g.dWr = dWr.data_ptr<float>();
  g.dcp = dcp.data_ptr<float>();
  const size_t smem = ((size_t)2 * RR_DB * RR_F + RR_WARPS * RR_DB + RR_WARPS * RR_F + RR_MAXR * RR_DB + RR_DB + 4) * sizeof(float);
  TORCH_CHECK(cudaFuncSetAttribute(reread_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess,
              "reread_bwd: shared memory");
  reread_bwd_kernel<<<rr_grid(words), RR_WARPS * 32, smem, at::cuda::getCurrentCUDAStream()>>>(a, g);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {dsc, dtable, doffset, dhv, dhb, dhh, dWr, dcp};
}

}  // namespace mb
