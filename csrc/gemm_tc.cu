// tcgen05 GEMM core for sm_100a: C[g] = A[g] * B[g]^T, bf16 operands, fp32 accumulation in tensor memory.
//
// One persistent CTA per SM, warp-specialised:
//   warp 0      TMA producer   (cp.async.bulk.tensor 3-D tiles -> 128B-swizzled shared-memory ring, 4 stages)
//   warp 1      MMA issuer     (one thread issues tcgen05.mma 128x256x16; accumulators double-buffered in TMEM)
//   warps 2..5  epilogue       (tcgen05.ld 32 lanes x 32 columns -> registers -> fused epilogue -> global)
// Operands may be K-major (rows x K, K contiguous) or MN-major (K x rows, rows contiguous), so transposed views of
// row-major tensors (dgrad / wgrad) need no transposing copy.  Batched ("grouped") over a leading dimension through
// 3-D tensor maps: this is how all experts of a MoE layer run in one launch.
// Epilogues: plain store (bf16 or fp32, optional += into fp32), relu^2 (also stores the pre-activation),
// relu^2 backward (acc * 2*relu(aux)), SwiGLU over column halves, per-row scale.
// Every mbarrier wait is bounded; on a timeout the kernel records a code in `status`, drains and returns.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "common.cuh"

namespace mb {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4, UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int GEMM_THREADS = 192;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
constexpr int GROUP_M = 8;

enum { EPI_NONE = 0, EPI_RELU2 = 1, EPI_DRELU2 = 2, EPI_SWIGLU = 3, EPI_ROWSCALE = 4, EPI_DSWIGLU = 5 };

struct GemmParams {
  int M, N, K, G;                 // logical per-group problem; for EPI_SWIGLU N = 2H (B rows), out has H columns
  void* out;
  void* out2;
  const void* aux;
  long long out_gs, out2_gs, aux_gs;   // group strides in elements
  int ldo, ldo2, ldaux;                // row pitches in elements
  int epi, out_f32, accumulate;
  int m_tiles, n_tiles;
  int ntail;                 // 1: the last N tile issues MMAs only as wide as its valid columns (rounded up to 16)
  int* status;
  // M may be cut into `n_seg` segments of `seg_M` rows, each read through its own A tensor map (a peer GPU's
  // buffer) and, when `out_seg_on`, written to its own output base (the owner GPU's buffer).  Tiles never straddle
  // segments.  Plain GEMM: n_seg = 1, seg_M = M.
  int n_seg, seg_M, tiles_per_seg, a_g_off, out_g_off, out_seg_on;
  void* out_seg[8];
  // Pair kernel v3 only.  store_tma: the epilogue leaves through TMA stores (local output, one segment); otherwise
  // through coalesced row stores from the staged tile (peer buffers, segmented output).
  // counts: valid extent per group (device ints) - count_mode 1: rows of A/out (tiles wholly past it are not
  // computed and are written as zeros), 2: length of the contraction (k-blocks past it are not read).
  int store_tma, count_mode, dbg, group_m;
  int aux_tma;             // the aux operand of an epilogue (pre-activations) is prefetched by TMA into the staging tiles
  const int* counts;
};

struct TmapSet { CUtensorMap m[8]; };

__device__ __forceinline__ void tile_coords(int t, const GemmParams& p, int& g, int& mt, int& nt) {
  int per_g = p.m_tiles * p.n_tiles;
  g = t / per_g;
  int r = t - g * per_g;
  const int gm = p.group_m > 0 ? p.group_m : GROUP_M;
  int band = gm * p.n_tiles;
  int b = r / band;
  int first_m = b * gm;
  int gsz = min(gm, p.m_tiles - first_m);
  int rr = r - b * band;
  mt = first_m + rr % gsz;
  nt = rr / gsz;
}

__device__ __forceinline__ float tanh_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// x * sigmoid(x) with sigmoid = (tanh(x / 2) + 1) / 2: one special-function instruction and two FMAs, no division
__device__ __forceinline__ float silu_f(float x) {
  const float h = 0.5f * x;
  return fmaf(h, tanh_approx(h), h);
}

// Drain one accumulator tile (this warp's 32 TMEM lanes x 256 columns) through the fused epilogue to global memory.
// `row_l` = this thread's row inside M-segment `seg`; `taddr` = TMEM address of the warp's lanes, column 0 of the tile.
__device__ __forceinline__ void epilogue_tile(const GemmParams& p, int g, int seg, int row_l, int nt, uint32_t taddr) {
  const bool row_ok = row_l < p.seg_M;
  const int row = seg * p.seg_M + row_l;                                  // row of the local (M, N) problem
  // where the result goes: the local output, or the buffer of the GPU that owns this segment's tokens
  char* const obase = reinterpret_cast<char*>(p.out_seg_on ? p.out_seg[seg] : p.out);
  const long long orow = p.out_seg_on ? row_l : row;
  const long long og = g + p.out_g_off;
  if (p.epi == EPI_SWIGLU) {
    const int H = p.N >> 1;
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
      uint32_t rg[32], ru[32];
      __syncwarp();
      tmem_ld32(taddr + c * 32, rg);
      tmem_ld32(taddr + 128 + c * 32, ru);
      tmem_ld_wait();
      const int col0 = nt * 128 + c * 32;
      if (row_ok && col0 < H) {
        bf16* o = reinterpret_cast<bf16*>(obase) + og * p.out_gs + orow * p.ldo + col0;
        bf16* o2 = p.out2 ? reinterpret_cast<bf16*>(p.out2) + g * p.out2_gs + static_cast<long long>(row) * p.ldo2 + col0
                          : nullptr;
        const int nv = min(32, H - col0);
        for (int j = 0; j < nv; ++j) {
          float gg = __uint_as_float(rg[j]), uu = __uint_as_float(ru[j]);
          // operands rounded to bf16 first so forward and the recomputing backward see the same numbers
          float gr = __bfloat162float(__float2bfloat16(gg)), ur = __bfloat162float(__float2bfloat16(uu));
          o[j] = __float2bfloat16(silu_f(gr) * ur);
          if (o2) { o2[j] = __float2bfloat16(gg); o2[H + j] = __float2bfloat16(uu); }
        }
      }
    }
  } else {
#pragma unroll 1
    for (int c = 0; c < BN / 32; ++c) {
      uint32_t r[32];
      __syncwarp();                              // tcgen05.ld is warp-collective: reconverge after the stores
      tmem_ld32(taddr + c * 32, r);
      tmem_ld_wait();
      const int col0 = nt * BN + c * 32;
      if (row_ok && col0 < p.N) {
      const int nv = min(32, p.N - col0);
      float v[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
      if (p.epi == EPI_RELU2) {
        bf16* o2 = reinterpret_cast<bf16*>(p.out2) + g * p.out2_gs + static_cast<long long>(row) * p.ldo2 + col0;
        if (nv == 32) {
          uint4* d4 = reinterpret_cast<uint4*>(o2);
#pragma unroll
          for (int j = 0; j < 4; ++j)
            d4[j] = make_uint4(pack_bf16(v[8 * j], v[8 * j + 1]), pack_bf16(v[8 * j + 2], v[8 * j + 3]),
                               pack_bf16(v[8 * j + 4], v[8 * j + 5]), pack_bf16(v[8 * j + 6], v[8 * j + 7]));
        } else {
          for (int j = 0; j < nv; ++j) o2[j] = __float2bfloat16(v[j]);
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          float a = __bfloat162float(__float2bfloat16(v[j]));     // activation of the stored (rounded) value
          a = fmaxf(a, 0.f);
          v[j] = a * a;
        }
      } else if (p.epi == EPI_DRELU2) {
        const bf16* ax = reinterpret_cast<const bf16*>(p.aux) + g * p.aux_gs + static_cast<long long>(row) * p.ldaux + col0;
        if (nv == 32) {
          const uint4* a4 = reinterpret_cast<const uint4*>(ax);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 u = a4[j];
            float2 f0 = unpack_bf16(u.x), f1 = unpack_bf16(u.y), f2 = unpack_bf16(u.z), f3 = unpack_bf16(u.w);
            v[8 * j + 0] *= 2.f * fmaxf(f0.x, 0.f); v[8 * j + 1] *= 2.f * fmaxf(f0.y, 0.f);
            v[8 * j + 2] *= 2.f * fmaxf(f1.x, 0.f); v[8 * j + 3] *= 2.f * fmaxf(f1.y, 0.f);
            v[8 * j + 4] *= 2.f * fmaxf(f2.x, 0.f); v[8 * j + 5] *= 2.f * fmaxf(f2.y, 0.f);
            v[8 * j + 6] *= 2.f * fmaxf(f3.x, 0.f); v[8 * j + 7] *= 2.f * fmaxf(f3.y, 0.f);
          }
        } else {
          for (int j = 0; j < nv; ++j) v[j] *= 2.f * fmaxf(__bfloat162float(ax[j]), 0.f);
        }
      } else if (p.epi == EPI_ROWSCALE) {
        const float s = reinterpret_cast<const float*>(p.aux)[g * p.aux_gs + row];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] *= s;
      }
      if (p.out_f32) {
        float* o = reinterpret_cast<float*>(obase) + og * p.out_gs + orow * p.ldo + col0;
        if (nv == 32) {
          float4* o4 = reinterpret_cast<float4*>(o);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float4 x = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            if (p.accumulate) { float4 y = o4[j]; x.x += y.x; x.y += y.y; x.z += y.z; x.w += y.w; }
            o4[j] = x;
          }
        } else {
          for (int j = 0; j < nv; ++j) o[j] = p.accumulate ? o[j] + v[j] : v[j];
        }
      } else {
        bf16* o = reinterpret_cast<bf16*>(obase) + og * p.out_gs + orow * p.ldo + col0;
        if (nv == 32) {
          uint4* o4 = reinterpret_cast<uint4*>(o);
#pragma unroll
          for (int j = 0; j < 4; ++j)
            o4[j] = make_uint4(pack_bf16(v[8 * j], v[8 * j + 1]), pack_bf16(v[8 * j + 2], v[8 * j + 3]),
                               pack_bf16(v[8 * j + 4], v[8 * j + 5]), pack_bf16(v[8 * j + 6], v[8 * j + 7]));
        } else {
          for (int j = 0; j < nv; ++j) o[j] = __float2bfloat16(v[j]);
        }
      }
      }
    }
  }
}

// Width of the MMA for N tile `nt`: the full tile, or for a ragged last tile its valid columns rounded up to 16
// (rows of B past N are zero-filled by TMA; accumulator columns past the width are never stored).
__device__ __forceinline__ int tile_n_eff(const GemmParams& p, int nt) {
  if (!p.ntail || p.epi == EPI_SWIGLU) return BN;
  const int rem = p.N - nt * BN;
  return rem >= BN ? BN : ((rem + 15) & ~15);
}

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ TmapSet tmAs, const __grid_constant__ CUtensorMap tmB, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_kb = (p.K + BK - 1) / BK;
  const int total = p.G * p.m_tiles * p.n_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tfull[a], 1); mbar_init(&tempty[a], 4); }
    *abort_flag = 0;
    mbar_fence_init();
    for (int i = 0; i < p.n_seg; ++i) tma_prefetch_desc(&tmAs.m[i]);
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
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
        int g, mt, nt;
        tile_coords(t, p, g, mt, nt);
        const int seg = mt / p.tiles_per_seg;
        const int m0 = (mt - seg * p.tiles_per_seg) * BM;
        const CUtensorMap* tA = &tmAs.m[seg];
        const int ga = g + p.a_g_off;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag)) {
            atomicCAS(p.status, 0, ST_WAIT_EMPTY); *abort_flag = 1; ok = false; break;
          }
          uint8_t* sA = smem + stage * STAGE_BYTES;
          uint8_t* sB = sA + A_BYTES;
          mbar_expect_tx(&full[stage], STAGE_BYTES);
          const int k0 = kb * BK;
          if (!A_MN) {
            tma_load_3d(sA, tA, &full[stage], k0, m0, ga);
          } else {
            tma_load_3d(sA, tA, &full[stage], m0, k0, ga);
            tma_load_3d(sA + 8192, tA, &full[stage], m0 + 64, k0, ga);
          }
          if (p.epi == EPI_SWIGLU) {
            const int H = p.N >> 1, n0 = nt * 128;
            if (!B_MN) {
              tma_load_3d(sB, &tmB, &full[stage], k0, n0, g);
              tma_load_3d(sB + 16384, &tmB, &full[stage], k0, H + n0, g);
            } else {
              tma_load_3d(sB, &tmB, &full[stage], n0, k0, g);
              tma_load_3d(sB + 8192, &tmB, &full[stage], n0 + 64, k0, g);
              tma_load_3d(sB + 16384, &tmB, &full[stage], H + n0, k0, g);
              tma_load_3d(sB + 24576, &tmB, &full[stage], H + n0 + 64, k0, g);
            }
          } else {
            const int n0 = nt * BN;
            if (!B_MN) {
              tma_load_3d(sB, &tmB, &full[stage], k0, n0, g);
            } else {
#pragma unroll
              for (int j = 0; j < 4; ++j) tma_load_3d(sB + j * 8192, &tmB, &full[stage], n0 + 64 * j, k0, g);
            }
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {                                   // let copies already in flight land before the CTA leaves
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
        int g_, mt_, nt_;
        tile_coords(t, p, g_, mt_, nt_);
        const uint32_t idesc = idesc_bf16(BM, tile_n_eff(p, nt_), A_MN ? 1u : 0u, B_MN ? 1u : 0u);
        if (!mbar_wait(&tempty[acc], acc_phase ^ 1, abort_flag)) {
          atomicCAS(p.status, 0, ST_WAIT_TMEM_EMPTY); *abort_flag = 1; ok = false; break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag)) {
            atomicCAS(p.status, 0, ST_WAIT_FULL); *abort_flag = 1; ok = false; break;
          }
          tc_fence_after();
          const uint32_t sA = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t sB = sA + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            uint64_t ad = smem_desc_sw128(sA + k * (A_MN ? UMMA_K * 128 : UMMA_K * 2), A_MN ? BK * 128 : 0, 1024);
            uint64_t bd = smem_desc_sw128(sB + k * (B_MN ? UMMA_K * 128 : UMMA_K * 2), B_MN ? BK * 128 : 0, 1024);
            umma_bf16(d_tmem, ad, bd, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty[stage]);              // the smem slot is free once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&tfull[acc]);                  // accumulator complete
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;                        // TMEM lane quarter this warp may read
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
      int g, mt, nt;
      tile_coords(t, p, g, mt, nt);
      if (!mbar_wait(&tfull[acc], acc_phase, abort_flag)) {
        if (lane == 0) { atomicCAS(p.status, 0, ST_WAIT_TMEM_FULL); *abort_flag = 1; }
        ok = false; break;
      }
      tc_fence_after();
      const int seg = mt / p.tiles_per_seg;
      const int row_l = (mt - seg * p.tiles_per_seg) * BM + q * 32 + lane;     // row inside its segment
      epilogue_tile(p, g, seg, row_l, nt, tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN);
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

// ------------------------------------------------------------------------------------------------ CTA-pair kernel
// tcgen05.mma.cta_group::2: a cluster of two CTAs (two SMs) computes a 256x256 tile.  Each CTA stages its own 128
// rows of A and its own 128-row half of the B tile, so every SM pulls 32 KB per k-block instead of 48 KB for the
// same FLOPs; the leader CTA's single thread issues the MMAs for both, accumulators live in each CTA's own TMEM
// (128 lanes x 256 columns, double-buffered), each CTA runs its own epilogue on its rows.
// TMA loads carry no multicast: both CTAs fetch their own tiles; only the completion bytes are counted on the
// leader's barrier, and tcgen05.commit arrives on the barriers of both CTAs.
constexpr int BH_BYTES = 128 * BK * 2, STAGE2_BYTES = A_BYTES + BH_BYTES;
// The epilogue leaves through shared memory: each epilogue warp packs its 32 rows x 64 bf16 (or 32 fp32) columns
// into a 128-byte-swizzled 4 KB staging tile and one lane issues a TMA store (a TMA reduce-add for fp32
// accumulation; for peer / segmented outputs the warp writes the staged rows itself as full 128-byte lines).
// Shared-memory descriptors are built once and advanced by integer adds.  Per-group extents let padded expert rows
// cost neither loads nor MMAs.
constexpr int EPI_BUF_BYTES = 4096;
enum { DBG_NO_STORE = 2, DBG_DIRECT_STORE = 8, DBG_L2_HINTS = 16, DBG_TALL_OFF = 32, DBG_TALL_ON = 64 };   // test / measurement switches

// row `lane` of a staging tile, 16-byte piece j (the tile is 1024-byte aligned: TMA's 128B swizzle = piece ^ (row & 7))
__device__ __forceinline__ uint4* stage_piece(uint8_t* buf, int row, int j) {
  return reinterpret_cast<uint4*>(buf + row * 128 + ((j ^ (row & 7)) << 4));
}
// Warp-cooperative copy of a staged 32 x 128 B tile to global rows (4 rows x 128 B per instruction).
__device__ __forceinline__ void coop_store(const uint8_t* buf, char* gbase, long long pitch_bytes, int rows_valid,
                                           int pieces_valid, bool f32_acc, int lane) {
  const int pc = lane & 7;
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int r = it * 4 + (lane >> 3);
    if (r < rows_valid && pc < pieces_valid) {
      uint4 v = *reinterpret_cast<const uint4*>(buf + r * 128 + ((pc ^ (r & 7)) << 4));
      uint4* dst = reinterpret_cast<uint4*>(gbase + r * pitch_bytes + pc * 16);
      if (f32_acc) {
        const float4 o = *reinterpret_cast<const float4*>(dst);
        float4 n = *reinterpret_cast<float4*>(&v);
        n.x += o.x; n.y += o.y; n.z += o.z; n.w += o.w;
        v = *reinterpret_cast<uint4*>(&n);
      }
      *dst = v;
    }
  }
}
// Warp-cooperative load of a 32 x 128 B global tile into a staging tile (zero outside the valid part).
__device__ __forceinline__ void coop_load(uint8_t* buf, const char* gbase, long long pitch_bytes, int rows_valid,
                                          int pieces_valid, int lane) {
  const int pc = lane & 7;
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int r = it * 4 + (lane >> 3);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < rows_valid && pc < pieces_valid) v = *reinterpret_cast<const uint4*>(gbase + r * pitch_bytes + pc * 16);
    *reinterpret_cast<uint4*>(buf + r * 128 + ((pc ^ (r & 7)) << 4)) = v;
  }
}

// Per-warp staging ring of EPI_NBUF tiles, handed out in slots of `nb` tiles (nb = staged tiles per store group of
// this launch: 1, 2 with a second output, 3 for SwiGLU with its pre-activations).  take(): wait until the slot about
// to be written is no longer read by an earlier store group, return the index of its first tile.
struct EpiRing {
  uint8_t* base;
  int next, nb, nbuf;
  bool tma;
  uint64_t store_policy;
  bool hint;
  __device__ __forceinline__ int take(int lane) {
    if (tma && lane == 0) {
      const int slots = nbuf / nb;                   // store groups that may still read their tiles: slots - 1
      if (slots >= 4) bulk_wait_read<3>();
      else if (slots == 2) bulk_wait_read<1>();
      else bulk_wait_read<0>();
    }
    __syncwarp();
    const int first = next;
    next += nb;
    if (next + nb > nbuf) next = 0;
    return first;
  }
  __device__ __forceinline__ uint8_t* buf(int i) const { return base + i * EPI_BUF_BYTES; }
};

struct EpiOut {            // where one output of the tile goes
  const CUtensorMap* tm;   // TMA path
  char* base;              // direct path: address of (first row of this warp, column 0) of the right group / segment
  long long pitch;         // bytes
};

// Send one staged tile: columns [col0, col0 + 64 bf16 | 32 fp32) of rows [row0, row0 + 32).
__device__ __forceinline__ void epi_send(const GemmParams& p, const EpiRing& ring, int bi, const EpiOut& o, int col0, int row0,
                                         int g, int rows_valid, int ncols, int esz, bool accumulate, int lane) {
  if (p.dbg & DBG_NO_STORE) return;
  if (ring.tma) {
    if (lane == 0) {
      if (accumulate) tma_reduce_add_3d(o.tm, ring.buf(bi), col0, row0, g);
      else if (ring.hint) tma_store_3d_hint(o.tm, ring.buf(bi), col0, row0, g, ring.store_policy);
      else tma_store_3d(o.tm, ring.buf(bi), col0, row0, g);
    }
  } else {
    const int per = 16 / esz;                                  // elements per 16-byte piece
    const int pieces = min(8, (ncols - col0 + per - 1) / per);
    coop_store(ring.buf(bi), o.base + static_cast<long long>(col0) * esz, o.pitch, rows_valid, pieces, accumulate, lane);
  }
}

// ---- aux prefetch.  The activation-backward epilogues (relu², SwiGLU) multiply the accumulator by a function of the
// forward's pre-activations, a second operand of the tile's own shape.  Fetching it when the accumulator is ready
// puts a global-memory round trip (microseconds while the GEMM itself loads HBM) into every 64-column chunk and
// made the epilogue the bottleneck (dgrad 0.74 ms plain, 1.37 ms with the relu² factor, 3.49 ms with SwiGLU's).  So
// each epilogue warp keeps a queue of TMA loads `slots` chunks ahead - across tile boundaries, i.e. issued while
// it waits for the next accumulator - into the very staging tiles the results are later stored from.
struct AuxPipe {
  uint64_t* bars;          // this warp's mbarriers, one per slot
  int slots, nb;           // nb staging tiles per chunk (1: relu² backward, 2: SwiGLU backward), slots = tiles / nb
  uint32_t issued, consumed;
  int pf_t, pf_hc;         // cursor of the next chunk to fetch: tile, half * 4 + chunk
  const CUtensorMap* tm;
  int rank, q, npairs, total, mh;
  bool on;
};

__device__ __forceinline__ void tma_load_3d_local(void* dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

__device__ __forceinline__ int group_rows(const GemmParams& p, int g);
__device__ __forceinline__ int group_kblocks(const GemmParams& p, int g);

// Issue loads until `slots` chunks are in flight or the tile list ends.  Walks tiles and chunks exactly as the
// epilogue does (padding tiles and chunks past the last column are skipped).  Lane 0 only.
__device__ __forceinline__ void aux_issue(const GemmParams& p, AuxPipe& a, uint8_t* ring_base) {
  while (a.issued - a.consumed < (uint32_t)a.slots && a.pf_t < a.total) {
    int g, mt, nt;
    tile_coords(a.pf_t, p, g, mt, nt);
    const int seg = mt / p.tiles_per_seg;
    const int mseg0 = (mt - seg * p.tiles_per_seg) * 256 * a.mh;
    const bool skip_tile = seg * p.seg_M + mseg0 >= group_rows(p, g) || group_kblocks(p, g) == 0;
    const int h = a.pf_hc >> 2, c = a.pf_hc & 3;
    const int col0 = nt * BN + c * 64;
    if (skip_tile || col0 >= p.N) {                     // next half / tile
      if (skip_tile || h + 1 >= a.mh) { a.pf_t += a.npairs; a.pf_hc = 0; }
      else a.pf_hc = (h + 1) << 2;
      continue;
    }
    const int row0 = seg * p.seg_M + mseg0 + h * 256 + a.rank * BM + a.q * 32;
    const int slot = a.issued % a.slots;
    uint8_t* b = ring_base + slot * a.nb * EPI_BUF_BYTES;
    mbar_expect_tx(&a.bars[slot], a.nb * EPI_BUF_BYTES);
    tma_load_3d_local(b, a.tm, &a.bars[slot], col0, row0, g);
    if (a.nb == 2) tma_load_3d_local(b + EPI_BUF_BYTES, a.tm, &a.bars[slot], p.N + col0, row0, g);
    ++a.issued;
    if (c == 3) {
      if (h + 1 >= a.mh) { a.pf_t += a.npairs; a.pf_hc = 0; }
      else a.pf_hc = (h + 1) << 2;
    } else {
      ++a.pf_hc;
    }
  }
}

// Drain this warp's 32 TMEM lanes x 256 columns of one accumulator through the fused epilogue.
// row0 = first row of the warp in the local (M) problem, row0_l = the same inside its M-segment.
__device__ __forceinline__ void epilogue_tile3(const GemmParams& p, const CUtensorMap* tmO, const CUtensorMap* tmO2, int g,
                                               int seg, int row0, int row0_l, int nt, uint32_t taddr, EpiRing& ring, int lane,
                                               bool zero_tile, AuxPipe* aux, volatile int* abort_flag) {
  const int rows_valid = max(0, min(32, p.seg_M - row0_l));
  const int row = row0 + lane;
  const int esz = p.out_f32 ? 4 : 2;
  EpiOut o, o2;
  o.tm = tmO; o2.tm = tmO2;
  {
    char* ob = reinterpret_cast<char*>(p.out_seg_on ? p.out_seg[seg] : p.out);
    const long long orow = p.out_seg_on ? row0_l : row0;
    o.base = ob + ((g + p.out_g_off) * p.out_gs + orow * p.ldo) * esz;
    o.pitch = static_cast<long long>(p.ldo) * esz;
    o2.base = reinterpret_cast<char*>(p.out2) + (g * p.out2_gs + static_cast<long long>(row0) * p.ldo2) * 2;
    o2.pitch = static_cast<long long>(p.ldo2) * 2;
  }
  const int og = g + p.out_g_off;

  if (zero_tile) {
    // a tile of padding rows: no accumulator was produced; the outputs are zeros (an accumulating output stays)
    if (p.accumulate) return;
    if (aux != nullptr && aux->on) {
      // the staging tiles belong to the prefetch queue: zeros go out by plain 16-byte stores
      const int wide = p.epi == EPI_DSWIGLU ? 2 : 1;
      for (int c = 0; c < BN / 64; ++c) {
        const int col0 = nt * BN + c * 64;
        if (col0 >= p.N) break;
        const int pieces = min(8, (p.N - col0 + 7) >> 3), pc = lane & 7;
        for (int w = 0; w < wide; ++w)
          for (int it = 0; it < 8; ++it) {
            const int r = it * 4 + (lane >> 3);
            if (r < rows_valid && pc < pieces)
              *reinterpret_cast<uint4*>(o.base + r * o.pitch + (static_cast<long long>(w) * p.N + col0) * 2 + pc * 16) =
                  make_uint4(0, 0, 0, 0);
          }
      }
      return;
    }
    const int bi = ring.take(lane);
    *stage_piece(ring.buf(bi), lane, 0) = make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int j = 1; j < 8; ++j) *stage_piece(ring.buf(bi), lane, j) = make_uint4(0, 0, 0, 0);
    fence_async_smem();
    __syncwarp();
    if (p.epi == EPI_SWIGLU) {
      const int H = p.N >> 1;
      for (int c = 0; c < 2; ++c) {
        const int col0 = nt * 128 + c * 64;
        if (col0 >= H) break;
        epi_send(p, ring, bi, o, col0, row0, og, rows_valid, H, 2, false, lane);
        if (p.out2) {
          epi_send(p, ring, bi, o2, col0, row0, g, rows_valid, H, 2, false, lane);
          epi_send(p, ring, bi, o2, H + col0, row0, g, rows_valid, p.N, 2, false, lane);
        }
      }
    } else {
      const int cw = p.out_f32 ? 32 : 64;
      for (int c = 0; c < BN / cw; ++c) {
        const int col0 = nt * BN + c * cw;
        if (col0 >= p.N) break;
        epi_send(p, ring, bi, o, col0, row0, og, rows_valid, p.N, esz, false, lane);
        if (p.epi == EPI_RELU2) epi_send(p, ring, bi, o2, col0, row0, g, rows_valid, p.N, 2, false, lane);
        if (p.epi == EPI_DSWIGLU) {
          EpiOut oz = o;
          oz.tm = tmO2;
          oz.base = o.base + static_cast<long long>(p.N) * 2;
          epi_send(p, ring, bi, oz, col0, row0, og, rows_valid, p.N, 2, false, lane);
        }
      }
    }
    if (ring.tma && lane == 0) bulk_commit();
    return;
  }

  if (p.epi == EPI_SWIGLU) {
    const int H = p.N >> 1;
    const int nb = p.out2 ? 3 : 1;
#pragma unroll 1
    for (int c = 0; c < 2; ++c) {
      const int col0 = nt * 128 + c * 64;
      if (col0 >= H) break;
      const int bi = ring.take(lane);
#pragma unroll 1
      for (int hf = 0; hf < 2; ++hf) {
        uint32_t rg[32], ru[32];
        tmem_ld32(taddr + c * 64 + hf * 32, rg);
        tmem_ld32(taddr + 128 + c * 64 + hf * 32, ru);
        tmem_ld_wait();
        uint32_t ph[16], pg[16], pu[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float g0 = __uint_as_float(rg[2 * j]), g1 = __uint_as_float(rg[2 * j + 1]);
          const float u0 = __uint_as_float(ru[2 * j]), u1 = __uint_as_float(ru[2 * j + 1]);
          pg[j] = pack_bf16(g0, g1);
          pu[j] = pack_bf16(u0, u1);
          // activations of the stored (rounded) values, so forward and the recomputing backward agree
          const float2 gr = unpack_bf16(pg[j]), ur = unpack_bf16(pu[j]);
          ph[j] = pack_bf16(silu_f(gr.x) * ur.x, silu_f(gr.y) * ur.y);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          *stage_piece(ring.buf(bi), lane, hf * 4 + j) = make_uint4(ph[4 * j], ph[4 * j + 1], ph[4 * j + 2], ph[4 * j + 3]);
          if (nb == 3) {
            *stage_piece(ring.buf(bi + 1), lane, hf * 4 + j) = make_uint4(pg[4 * j], pg[4 * j + 1], pg[4 * j + 2], pg[4 * j + 3]);
            *stage_piece(ring.buf(bi + 2), lane, hf * 4 + j) = make_uint4(pu[4 * j], pu[4 * j + 1], pu[4 * j + 2], pu[4 * j + 3]);
          }
        }
      }
      fence_async_smem();
      __syncwarp();
      epi_send(p, ring, bi, o, col0, row0, og, rows_valid, H, 2, false, lane);
      if (nb == 3) {
        epi_send(p, ring, bi + 1, o2, col0, row0, g, rows_valid, H, 2, false, lane);
        epi_send(p, ring, bi + 2, o2, H + col0, row0, g, rows_valid, p.N, 2, false, lane);
      }
      if (ring.tma && lane == 0) bulk_commit();
    }
    return;
  }

  if (p.out_f32) {
    // fp32 output (weight gradients): 32 columns per staged tile
#pragma unroll 1
    for (int c = 0; c < BN / 32; ++c) {
      const int col0 = nt * BN + c * 32;
      if (col0 >= p.N) break;
      uint32_t r[32];
      tmem_ld32(taddr + c * 32, r);
      tmem_ld_wait();
      float sc = 1.f;
      if (p.epi == EPI_ROWSCALE) sc = row0_l + lane < p.seg_M ? reinterpret_cast<const float*>(p.aux)[g * p.aux_gs + row] : 0.f;
      const int bi = ring.take(lane);
#pragma unroll
      for (int j = 0; j < 8; ++j)
        *stage_piece(ring.buf(bi), lane, j) =
            make_uint4(__float_as_uint(__uint_as_float(r[4 * j]) * sc), __float_as_uint(__uint_as_float(r[4 * j + 1]) * sc),
                       __float_as_uint(__uint_as_float(r[4 * j + 2]) * sc), __float_as_uint(__uint_as_float(r[4 * j + 3]) * sc));
      fence_async_smem();
      __syncwarp();
      epi_send(p, ring, bi, o, col0, row0, og, rows_valid, p.N, 4, p.accumulate != 0, lane);
      if (ring.tma && lane == 0) bulk_commit();
    }
    return;
  }

  // bf16 output, 64 columns per staged tile
  const int nb = (p.epi == EPI_RELU2 || p.epi == EPI_DSWIGLU) ? 2 : 1;
  EpiOut oh = o;                       // SwiGLU backward: second half of the output row (the `up` gradient), via tmO2
  oh.tm = tmO2;
  oh.base = o.base + static_cast<long long>(p.N) * 2;
#pragma unroll 1
  for (int c = 0; c < BN / 64; ++c) {
    const int col0 = nt * BN + c * 64;
    if (col0 >= p.N) break;
    uint32_t r[64];
    tmem_ld32(taddr + c * 64, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
    tmem_ld32(taddr + c * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
    tmem_ld_wait();
    const bool piped = aux != nullptr && aux->on;
    int bi;
    if (piped) {
      // the chunk's pre-activations were fetched ahead into the slot the results will be stored from
      const int slot = aux->consumed % aux->slots;
      bi = slot * aux->nb;
      if (!mbar_wait(&aux->bars[slot], (aux->consumed / aux->slots) & 1, abort_flag)) {
        if (lane == 0) { atomicCAS(p.status, 0, ST_WAIT_FULL); *abort_flag = 1; }
        return;
      }
    } else {
      bi = ring.take(lane);
    }
    uint8_t* b0 = ring.buf(bi);
    if (p.epi == EPI_RELU2) {
      uint8_t* b1 = ring.buf(bi + 1);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        uint32_t pa[4], ph[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          pa[q] = pack_bf16(__uint_as_float(r[8 * j + 2 * q]), __uint_as_float(r[8 * j + 2 * q + 1]));
          float2 a = unpack_bf16(pa[q]);                      // activation of the stored (rounded) value
          a.x = fmaxf(a.x, 0.f); a.y = fmaxf(a.y, 0.f);
          ph[q] = pack_bf16(a.x * a.x, a.y * a.y);
        }
        *stage_piece(b0, lane, j) = make_uint4(ph[0], ph[1], ph[2], ph[3]);
        *stage_piece(b1, lane, j) = make_uint4(pa[0], pa[1], pa[2], pa[3]);
      }
    } else if (p.epi == EPI_DSWIGLU) {
      // acc = dh (columns of the hidden width H = p.N); aux = (gate | up) pre-activations, 2H columns.
      // dg = dh * u * s * (1 + g * (1 - s)), du = dh * g * s with s = sigmoid(g)
      uint8_t* b1 = ring.buf(bi + 1);
      const char* ab = reinterpret_cast<const char*>(p.aux) + (g * p.aux_gs + static_cast<long long>(row0) * p.ldaux + col0) * 2;
      const int pv = min(8, (p.N - col0 + 7) >> 3);
      if (!piped) {
        coop_load(b0, ab, static_cast<long long>(p.ldaux) * 2, rows_valid, pv, lane);
        coop_load(b1, ab + static_cast<long long>(p.N) * 2, static_cast<long long>(p.ldaux) * 2, rows_valid, pv, lane);
        __syncwarp();
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        uint4* pg = stage_piece(b0, lane, j);
        uint4* pu = stage_piece(b1, lane, j);
        const uint4 ug = *pg, uu = *pu;
        const uint32_t wg[4] = {ug.x, ug.y, ug.z, ug.w}, wu[4] = {uu.x, uu.y, uu.z, uu.w};
        uint32_t og[4], ou[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 gg = unpack_bf16(wg[q]), uv = unpack_bf16(wu[q]);
          const float d0 = __uint_as_float(r[8 * j + 2 * q]), d1 = __uint_as_float(r[8 * j + 2 * q + 1]);
          // sigmoid through the hardware tanh (one special-function instruction, no division): with one epilogue
          // warp per scheduler the dependent chain of exp + IEEE division per element was what bound this epilogue
          const float s0 = fmaf(tanh_approx(0.5f * gg.x), 0.5f, 0.5f), s1 = fmaf(tanh_approx(0.5f * gg.y), 0.5f, 0.5f);
          og[q] = pack_bf16(d0 * uv.x * s0 * (1.f + gg.x * (1.f - s0)), d1 * uv.y * s1 * (1.f + gg.y * (1.f - s1)));
          ou[q] = pack_bf16(d0 * gg.x * s0, d1 * gg.y * s1);
        }
        *pg = make_uint4(og[0], og[1], og[2], og[3]);
        *pu = make_uint4(ou[0], ou[1], ou[2], ou[3]);
      }
    } else if (p.epi == EPI_DRELU2) {
      const char* ab = reinterpret_cast<const char*>(p.aux) + (g * p.aux_gs + static_cast<long long>(row0) * p.ldaux + col0) * 2;
      if (!piped) {
        coop_load(b0, ab, static_cast<long long>(p.ldaux) * 2, rows_valid, min(8, (p.N - col0 + 7) >> 3), lane);
        __syncwarp();
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        uint4* pp = stage_piece(b0, lane, j);
        const uint4 u = *pp;
        const float2 f0 = unpack_bf16(u.x), f1 = unpack_bf16(u.y), f2 = unpack_bf16(u.z), f3 = unpack_bf16(u.w);
        *pp = make_uint4(pack_bf16(__uint_as_float(r[8 * j + 0]) * 2.f * fmaxf(f0.x, 0.f), __uint_as_float(r[8 * j + 1]) * 2.f * fmaxf(f0.y, 0.f)),
                         pack_bf16(__uint_as_float(r[8 * j + 2]) * 2.f * fmaxf(f1.x, 0.f), __uint_as_float(r[8 * j + 3]) * 2.f * fmaxf(f1.y, 0.f)),
                         pack_bf16(__uint_as_float(r[8 * j + 4]) * 2.f * fmaxf(f2.x, 0.f), __uint_as_float(r[8 * j + 5]) * 2.f * fmaxf(f2.y, 0.f)),
                         pack_bf16(__uint_as_float(r[8 * j + 6]) * 2.f * fmaxf(f3.x, 0.f), __uint_as_float(r[8 * j + 7]) * 2.f * fmaxf(f3.y, 0.f)));
      }
    } else {
      float sc = 1.f;
      if (p.epi == EPI_ROWSCALE) sc = row0_l + lane < p.seg_M ? reinterpret_cast<const float*>(p.aux)[g * p.aux_gs + row] : 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j)
        *stage_piece(b0, lane, j) = make_uint4(pack_bf16(__uint_as_float(r[8 * j]) * sc, __uint_as_float(r[8 * j + 1]) * sc),
                                               pack_bf16(__uint_as_float(r[8 * j + 2]) * sc, __uint_as_float(r[8 * j + 3]) * sc),
                                               pack_bf16(__uint_as_float(r[8 * j + 4]) * sc, __uint_as_float(r[8 * j + 5]) * sc),
                                               pack_bf16(__uint_as_float(r[8 * j + 6]) * sc, __uint_as_float(r[8 * j + 7]) * sc));
    }
    fence_async_smem();
    __syncwarp();
    epi_send(p, ring, bi, o, col0, row0, og, rows_valid, p.N, 2, false, lane);
    if (p.epi == EPI_DSWIGLU) epi_send(p, ring, bi + 1, oh, col0, row0, og, rows_valid, p.N, 2, false, lane);
    else if (nb == 2) epi_send(p, ring, bi + 1, o2, col0, row0, g, rows_valid, p.N, 2, false, lane);
    if (ring.tma && lane == 0) bulk_commit();
    if (piped) {
      ++aux->consumed;
      __syncwarp();                               // direct stores: every lane has read the slot
      if (lane == 0) {
        bulk_wait_read<0>();                      // TMA stores have read it too: it may take the chunk `slots` ahead
        fence_async_smem();
        aux_issue(p, *aux, ring.base);
      }
    }
  }
}

// extent of group g under count_mode (rows for mode 1, contraction length for mode 2), else the full extent
__device__ __forceinline__ int group_rows(const GemmParams& p, int g) {
  return p.count_mode == 1 ? min(p.M, __ldg(p.counts + g)) : p.M;
}
__device__ __forceinline__ int group_kblocks(const GemmParams& p, int g) {
  const int k = p.count_mode == 2 ? min(p.K, __ldg(p.counts + g)) : p.K;
  return (k + BK - 1) / BK;
}

// MH = 256-row MMA blocks per tile.  MH 1: 256 x 256 tile, 5 operand stages of 32 KB, accumulators double-buffered in
// TMEM (2 x 256 columns), so the epilogue of a tile runs under the MMAs of the next.  MH 2: 512 x 256 tile - every
// B k-block feeds two MMAs, so the pair pulls 96 KB per 512x256x64 of work instead of 128 KB (a quarter less L2 and
// shared-memory traffic, which on a power-capped part is clock) - 4 stages of 48 KB; the two 256-column accumulators
// fill TMEM, so the epilogue is only half hidden (the MMAs of the next tile's first block start as soon as the
// first half is drained): worth it when the contraction is long.
// DEEP (256-row tiles only): one operand stage less and six staging tiles per epilogue warp instead of four, for the
// SwiGLU-backward epilogue, which moves two tiles in and two out per 64 accumulator columns and needs three chunks of
// pre-activations in flight per warp to keep HBM busy.
template <int MH, bool DEEP = false> struct PairCfg {
  static constexpr int STAGES = (MH == 2 || DEEP) ? 4 : 5;
  static constexpr int NBUF = MH == 2 ? 2 : (DEEP ? 6 : 4);
  static constexpr int STAGE_BYTES = MH * A_BYTES + BH_BYTES;
  static constexpr int SMEM = STAGES * STAGE_BYTES + 4 * NBUF * EPI_BUF_BYTES + 1024 + 256;
};

template <bool A_MN, bool B_MN, int MH, bool DEEP = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ TmapSet tmAs, const __grid_constant__ CUtensorMap tmB,
                const __grid_constant__ CUtensorMap tmO, const __grid_constant__ CUtensorMap tmO2,
                const __grid_constant__ CUtensorMap tmX, const GemmParams p) {
  constexpr int STAGES3 = PairCfg<MH, DEEP>::STAGES, EPI_NBUF = PairCfg<MH, DEEP>::NBUF, STAGE_B = PairCfg<MH, DEEP>::STAGE_BYTES;
  constexpr int TILE_M = 256 * MH;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi_smem = smem + STAGES3 * STAGE_B;
  uint64_t* full = reinterpret_cast<uint64_t*>(epi_smem + 4 * EPI_NBUF * EPI_BUF_BYTES);
  uint64_t* empty = full + STAGES3;
  uint64_t* tfull = empty + STAGES3;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint64_t* auxbars = full + 16;              // 4 epilogue warps x 4 slots of the aux prefetch queue (bytes 128..255)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
  const int total = p.G * p.m_tiles * p.n_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES3; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tfull[a], 1); mbar_init(&tempty[a], 8); }
    *abort_flag = 0;
    mbar_fence_init();
    for (int i = 0; i < p.n_seg; ++i) tma_prefetch_desc(&tmAs.m[i]);
    tma_prefetch_desc(&tmB);
    if (p.store_tma) { tma_prefetch_desc(&tmO); if (p.out2 || p.epi == EPI_DSWIGLU) tma_prefetch_desc(&tmO2); }
    if (p.aux_tma) {
      for (int i = 0; i < 16; ++i) mbar_init(&auxbars[i], 1);
      mbar_fence_init();
      tma_prefetch_desc(&tmX);
    }
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  cluster_sync_all();                         // both CTAs' barriers exist before anyone arrives on a peer's barrier
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0 && tmem_base != 0) atomicCAS(p.status, 0, ST_BAD_ARG);   // the pair must share one TMEM address

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = pair; t < total && ok; t += npairs) {
        int g, mt, nt;
        tile_coords(t, p, g, mt, nt);
        const int seg = mt / p.tiles_per_seg;
        const int mseg0 = (mt - seg * p.tiles_per_seg) * TILE_M;
        if (seg * p.seg_M + mseg0 >= group_rows(p, g)) continue;            // a tile of padding rows
        const int m0 = mseg0 + (int)rank * BM;
        const CUtensorMap* tA = &tmAs.m[seg];
        const int ga = g + p.a_g_off;
        const int num_kb = group_kblocks(p, g);
        const int nb = (p.epi == EPI_SWIGLU) ? (rank == 0 ? nt * 128 : (p.N >> 1) + nt * 128)
                                             : nt * BN + (int)rank * (tile_n_eff(p, nt) >> 1);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_try_wait(&empty[stage], phase ^ 1) && !mbar_wait(&empty[stage], phase ^ 1, abort_flag)) {
            atomicCAS(p.status, 0, ST_WAIT_EMPTY); *abort_flag = 1; ok = false; break;
          }
          uint8_t* sA = smem + stage * STAGE_B;
          uint8_t* sB = sA + MH * A_BYTES;
          const uint32_t lfull = mapa_shared(smem_u32(&full[stage]), 0);      // the leader's barrier
          if (leader) mbar_expect_tx(&full[stage], 2 * STAGE_B);               // bytes of both CTAs
          const int k0 = kb * BK;
#pragma unroll
          for (int h = 0; h < MH; ++h) {                                       // this CTA's 128 rows of each 256-row block
            const int mh = m0 + h * 256;
            if (!A_MN) {
              tma_load_3d_pair(sA + h * A_BYTES, tA, lfull, k0, mh, ga);
            } else {
              tma_load_3d_pair(sA + h * A_BYTES, tA, lfull, mh, k0, ga);
              tma_load_3d_pair(sA + h * A_BYTES + 8192, tA, lfull, mh + 64, k0, ga);
            }
          }
          if (!B_MN) {
            tma_load_3d_pair(sB, &tmB, lfull, k0, nb, g);
          } else {
            tma_load_3d_pair(sB, &tmB, lfull, nb, k0, g);
            tma_load_3d_pair(sB + 8192, &tmB, lfull, nb + 64, k0, g);
          }
          if (++stage == STAGES3) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    // This one thread is the pacemaker of both SMs: whatever it executes between two MMAs shows up as an idle
    // tensor pipe.  So the loop holds everything in registers, looks at the next stage's barrier before it issues
    // the current stage's MMAs (the look-up's latency then overlaps their execution), and works out the next
    // tile's coordinates while the first k-block of the current one runs.
    if (lane == 0 && leader) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;                 // MH 1: accumulator buffer in use; MH 2: always 0 (tempty[h] = half h drained)
      uint32_t acc_phase = 0;
      bool ok = true;
      constexpr uint32_t KSTEP_A = (A_MN ? UMMA_K * 128 : UMMA_K * 2) >> 4, KSTEP_B = (B_MN ? UMMA_K * 128 : UMMA_K * 2) >> 4;
      constexpr uint32_t STAGE_STEP = STAGE_B >> 4;
      const uint64_t adesc0 = smem_desc_sw128(smem_u32(smem), A_MN ? BK * 128 : 0, 1024);
      const uint64_t bdesc0 = smem_desc_sw128(smem_u32(smem) + MH * A_BYTES, B_MN ? BK * 128 : 0, 1024);
      uint32_t soff = 0;                                                   // stage * STAGE_STEP
      // (k-blocks, instruction descriptor) of tile t; 0 k-blocks = nothing to issue (padding rows, empty contraction)
      auto tile_info = [&](int t, int& nkb, uint32_t& idesc) {
        nkb = 0; idesc = 0;
        if (t >= total) return;
        int g_, mt_, nt_;
        tile_coords(t, p, g_, mt_, nt_);
        const int seg = mt_ / p.tiles_per_seg;
        if (seg * p.seg_M + (mt_ - seg * p.tiles_per_seg) * TILE_M >= group_rows(p, g_)) return;
        nkb = group_kblocks(p, g_);
        idesc = idesc_bf16(256, tile_n_eff(p, nt_), A_MN ? 1u : 0u, B_MN ? 1u : 0u);
      };
      int num_kb, nxt_kb = 0;
      uint32_t idesc, nxt_idesc = 0;
      tile_info(pair, num_kb, idesc);
      for (int t = pair; t < total && ok; t += npairs) {
        if (num_kb == 0) { tile_info(t + npairs, num_kb, idesc); continue; }
        if (!mbar_try_wait(&tempty[acc], acc_phase ^ 1) && !mbar_wait(&tempty[acc], acc_phase ^ 1, abort_flag)) {
          atomicCAS(p.status, 0, ST_WAIT_TMEM_EMPTY); *abort_flag = 1; ok = false; break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (MH == 1 ? acc * BN : 0);
        bool ready = mbar_try_wait(&full[stage], phase);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!ready && !mbar_wait(&full[stage], phase, abort_flag)) {
            atomicCAS(p.status, 0, ST_WAIT_FULL); *abort_flag = 1; ok = false; break;
          }
          tc_fence_after();
          int ns = stage + 1;
          uint32_t nph = phase, nsoff = soff + STAGE_STEP;
          if (ns == STAGES3) { ns = 0; nph ^= 1; nsoff = 0; }
          ready = mbar_try_wait(&full[ns], nph);                           // the next k-block (of this or the next tile)
          const uint64_t ad = adesc0 + soff, bd = bdesc0 + soff;
          umma_bf16_pair(d_tmem, ad, bd, idesc, kb > 0 ? 1u : 0u);
#pragma unroll
          for (int k = 1; k < BK / UMMA_K; ++k) umma_bf16_pair(d_tmem, ad + k * KSTEP_A, bd + k * KSTEP_B, idesc, 1u);
          if (MH == 2) {
            if (kb == 0) {                                                 // the second half of the last tile must be drained
              if (!mbar_try_wait(&tempty[1], acc_phase ^ 1) && !mbar_wait(&tempty[1], acc_phase ^ 1, abort_flag)) {
                atomicCAS(p.status, 0, ST_WAIT_TMEM_EMPTY); *abort_flag = 1; ok = false; break;
              }
              tc_fence_after();
            }
            const uint64_t ad2 = ad + (A_BYTES >> 4);
            umma_bf16_pair(d_tmem + BN, ad2, bd, idesc, kb > 0 ? 1u : 0u);
#pragma unroll
            for (int k = 1; k < BK / UMMA_K; ++k) umma_bf16_pair(d_tmem + BN, ad2 + k * KSTEP_A, bd + k * KSTEP_B, idesc, 1u);
          }
          umma_commit_pair(&empty[stage], 3);       // frees this stage in both CTAs
          if (kb == 0) tile_info(t + npairs, nxt_kb, nxt_idesc);
          stage = ns; phase = nph; soff = nsoff;
        }
        if (!ok) break;
        umma_commit_pair(&tfull[MH == 1 ? acc : 0], 3);           // accumulators of both CTAs complete
        if (MH == 1) { if (++acc == 2) { acc = 0; acc_phase ^= 1; } }
        else acc_phase ^= 1;
        num_kb = nxt_kb; idesc = nxt_idesc;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5 of both CTAs)
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    EpiRing ring;
    ring.base = epi_smem + q * (EPI_NBUF * EPI_BUF_BYTES);
    ring.next = 0;
    ring.nbuf = EPI_NBUF;
    ring.hint = (p.dbg & DBG_L2_HINTS) != 0;
    ring.store_policy = l2_policy_evict_first();
    ring.nb = (p.epi == EPI_RELU2 || p.epi == EPI_DSWIGLU) ? 2 : (p.epi == EPI_SWIGLU && p.out2 ? 3 : 1);
    ring.tma = p.store_tma != 0;
    AuxPipe aux;
    aux.on = p.aux_tma != 0;
    aux.bars = auxbars + q * 4;
    aux.nb = ring.nb;
    aux.slots = EPI_NBUF / ring.nb;
    aux.issued = aux.consumed = 0;
    aux.pf_t = pair; aux.pf_hc = 0;
    aux.tm = &tmX;
    aux.rank = (int)rank; aux.q = q; aux.npairs = npairs; aux.total = total; aux.mh = MH;
    if (aux.on && lane == 0) aux_issue(p, aux, ring.base);
    for (int t = pair; t < total && ok; t += npairs) {
      int g, mt, nt;
      tile_coords(t, p, g, mt, nt);
      const int seg = mt / p.tiles_per_seg;
      const int mseg0 = (mt - seg * p.tiles_per_seg) * TILE_M;
      const bool zero_tile = seg * p.seg_M + mseg0 >= group_rows(p, g) || group_kblocks(p, g) == 0;
      if (!zero_tile) {
        if (!mbar_wait(&tfull[MH == 1 ? acc : 0], acc_phase, abort_flag)) {
          if (lane == 0) { atomicCAS(p.status, 0, ST_WAIT_TMEM_FULL); *abort_flag = 1; }
          ok = false; break;
        }
        tc_fence_after();
      }
#pragma unroll 1
      for (int h = 0; h < MH; ++h) {
        const int row0_l = mseg0 + h * 256 + (int)rank * BM + q * 32;
        const int row0 = seg * p.seg_M + row0_l;
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + (MH == 1 ? acc * BN : h * BN);
        epilogue_tile3(p, &tmO, &tmO2, g, seg, row0, row0_l, nt, taddr, ring, lane, zero_tile, &aux, abort_flag);
        if (*abort_flag) { ok = false; break; }
        if (!zero_tile) {
          tc_fence_before();
          __syncwarp();
          // the leader's MMA thread waits on it (MH 2: per half, so the next tile's first MMAs start early)
          if (lane == 0) mbar_arrive_cluster(mapa_shared(smem_u32(&tempty[MH == 1 ? acc : h]), 0));
        }
      }
      if (!zero_tile) {
        if (MH == 1) { if (++acc == 2) { acc = 0; acc_phase ^= 1; } }
        else acc_phase ^= 1;
      }
    }
    if (ring.tma && lane == 0) bulk_wait_all<0>();           // staged tiles must be read before the CTA's smem goes away
    if (aux.on && lane == 0 && !ok) {
      // gave up with prefetches in flight: let them land (bounded) before the CTA's shared memory goes away
      for (uint32_t i = aux.consumed; i < aux.issued; ++i)
        for (uint32_t spin = 0; spin < MB_SPIN_LIMIT; ++spin)
          if (mbar_try_wait(&aux.bars[i % aux.slots], (i / aux.slots) & 1)) break;
    }
  }

  tc_fence_before();
  cluster_sync_all();                         // no CTA leaves while its pair may still touch its barriers or TMEM
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ------------------------------------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    TORCH_CHECK(e == cudaSuccess && p != nullptr, "cuTensorMapEncodeTiled entry point not found");
    fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// 3-D tensor map: dims (inner, rows, groups), 128-byte swizzle, zero fill outside.  `esz` 1 = 8-bit, 2 = bf16, 4 = fp32.
CUtensorMap make_tmap(const void* base, int esz, uint64_t inner, uint64_t rows, uint64_t groups, uint64_t row_pitch_el,
                      uint64_t group_pitch_el, uint32_t box_inner, uint32_t box_rows, bool promote) {
  // cuTensorMapEncodeTiled is a driver call: a thread that has made no runtime call yet (an autograd worker) has no
  // current context and gets CUDA_ERROR_INVALID_CONTEXT, so bind the primary context once per thread.
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) { cudaFree(nullptr); ctx_bound = true; }
  CUtensorMap m;
  cuuint64_t dims[3] = {inner, rows, groups};
  cuuint64_t strides[2] = {row_pitch_el * esz, (groups > 1 ? group_pitch_el : row_pitch_el * rows) * esz};
  cuuint32_t box[3] = {box_inner, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  TORCH_CHECK((reinterpret_cast<uintptr_t>(base) & 15) == 0, "TMA operand must be 16-byte aligned");
  TORCH_CHECK(strides[0] % 16 == 0 && strides[1] % 16 == 0, "TMA operand pitches must be multiples of 16 bytes");
  const CUtensorMapDataType dt = esz == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                : esz == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  CUresult r = encode_fn()(&m, dt, 3,
                           const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_128B,
                           promote ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B : CU_TENSOR_MAP_L2_PROMOTION_NONE,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TORCH_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with code ", static_cast<int>(r));
  return m;
}
CUtensorMap make_tmap_bf16(const void* base, uint64_t inner, uint64_t rows, uint64_t groups, uint64_t row_pitch_el,
                           uint64_t group_pitch_el, uint32_t box_inner, uint32_t box_rows) {
  return make_tmap(base, 2, inner, rows, groups, row_pitch_el, group_pitch_el, box_inner, box_rows, true);
}

static int* status_word(int device) {
  static int* words[16] = {nullptr};
  TORCH_CHECK(device >= 0 && device < 16, "device index out of range");
  if (!words[device]) {
    TORCH_CHECK(cudaMalloc(&words[device], sizeof(int)) == cudaSuccess, "status word alloc failed");
    cudaMemset(words[device], 0, sizeof(int));
  }
  return words[device];
}

int* gemm_status_word(int device) { return status_word(device); }

int gemm_status(int device) {
  int v = 0;
  cudaMemcpy(&v, status_word(device), sizeof(int), cudaMemcpyDeviceToHost);
  int z = 0;
  if (v) cudaMemcpy(status_word(device), &z, sizeof(int), cudaMemcpyHostToDevice);
  return v;
}

// The CTA-pair (cta_group::2) kernel is the default for tiles of >= 256 rows; MEMARCH_GEMM_PAIR=0 or
// gemm_set_pair(false) selects the single-CTA kernel everywhere.
static int g_pair = -1;
static bool use_pair_kernel() {
  if (g_pair < 0) {
    const char* e = std::getenv("MEMARCH_GEMM_PAIR");
    g_pair = (e && e[0] == '0') ? 0 : 1;
  }
  return g_pair == 1;
}
void gemm_set_pair(bool on) { g_pair = on ? 1 : 0; }
// Test / measurement switches of the pair kernel (DBG_* bits) and the row-tile group size of its tile order.
static int g_dbg = 0, g_group_m = 0;
void gemm_set_debug(int64_t dbg, int64_t group_m) { g_dbg = (int)dbg; g_group_m = (int)group_m; }

// Raw launcher shared by the torch binding and the fused multi-GPU paths (which pass peer pointers for A).
// A_list: one base pointer per M-segment (n_seg of them, each (a_groups, seg_M, K) or MN-major (a_groups, K, seg_M)).
void launch_gemm_seg(const void* const* A_list, int n_seg, int seg_M, int a_groups, long long a_rows_pitch, long long a_gs,
                     bool a_mn, const void* B, long long b_rows_pitch, long long b_gs, bool b_mn, GemmParams p,
                     cudaStream_t stream, int max_ctas) {
  const int N = p.N, K = p.K, G = p.G;
  TORCH_CHECK(n_seg >= 1 && n_seg <= 8, "gemm: 1..8 segments");
  TmapSet tmAs;
  for (int i = 0; i < n_seg; ++i)
    tmAs.m[i] = a_mn ? make_tmap_bf16(A_list[i], seg_M, K, a_groups, a_rows_pitch, a_gs, 64, 64)
                     : make_tmap_bf16(A_list[i], K, seg_M, a_groups, a_rows_pitch, a_gs, 64, BM);
  for (int i = n_seg; i < 8; ++i) tmAs.m[i] = tmAs.m[0];
  const bool pair = use_pair_kernel() && seg_M >= 256;
  const bool sw = p.epi == EPI_SWIGLU;
  const int n_tiles = sw ? ((N / 2) + 127) / 128 : (N + BN - 1) / BN;
  // 512-row tiles (see PairCfg) when the contraction is long enough to pay for the half-exposed epilogue and the
  // coarser tiling does not cost more in the last, partly filled wave of tiles than it saves
  bool tall = false;
  if (pair && n_seg == 1 && p.count_mode == 0 && seg_M >= 1024 && !(sw && p.out2) && p.epi != EPI_DRELU2 &&
      p.epi != EPI_DSWIGLU) {
    auto wave_eff = [&](int tm) {
      const long long tiles = (long long)G * ((seg_M + tm - 1) / tm) * n_tiles, pairs = std::max(1, max_ctas / 2);
      return (double)tiles / (double)(((tiles + pairs - 1) / pairs) * pairs);
    };
    static const bool tall_env = []() { const char* e = std::getenv("MEMARCH_GEMM_TALL"); return !(e && e[0] == '0'); }();
    tall = tall_env && K >= 8192 && wave_eff(512) >= wave_eff(256) - 0.02;
    if (g_dbg & DBG_TALL_OFF) tall = false;
    if (g_dbg & DBG_TALL_ON) tall = true;
  }
  const int tile_m = pair ? (tall ? 512 : 256) : BM;
  p.n_seg = n_seg; p.seg_M = seg_M; p.tiles_per_seg = (seg_M + tile_m - 1) / tile_m;
  CUtensorMap tmB = b_mn ? make_tmap_bf16(B, N, K, G, b_rows_pitch, b_gs, 64, 64)
                         : make_tmap_bf16(B, K, N, G, b_rows_pitch, b_gs, 64, (sw || pair) ? 128 : BN);
  p.m_tiles = n_seg * p.tiles_per_seg;
  p.n_tiles = n_tiles;
  static const bool ntail_on = []() { const char* e = std::getenv("MEMARCH_GEMM_NTAIL"); return !(e && e[0] == '0'); }();
  p.ntail = ntail_on ? 1 : 0;
  const int total = G * p.m_tiles * p.n_tiles;
  int grid = pair ? 2 * std::min(total, max_ctas / 2) : std::min(total, max_ctas);
  if (grid <= 0) return;
  const bool v3 = pair;
  TORCH_CHECK(v3 || p.count_mode == 0, "gemm: per-group extents need the pair kernel (>= 256 rows)");
  const bool deep = v3 && !tall && p.epi == EPI_DSWIGLU && !a_mn;
  const int smem_bytes = v3 ? (tall ? PairCfg<2>::SMEM : deep ? PairCfg<1, true>::SMEM : PairCfg<1>::SMEM) : SMEM_BYTES;
  CUtensorMap tmO = tmB, tmO2 = tmB;
  if (v3) {
    p.dbg = g_dbg;
    p.group_m = g_group_m;
    const int esz = p.out_f32 ? 4 : 2;
    // TMA stores for a local, unsegmented output whose pitches keep the 16-byte rule; everything else leaves
    // through coalesced row stores (peer buffers are only ever written with plain stores)
    p.store_tma = (n_seg == 1 && !p.out_seg_on && (p.ldo * esz) % 16 == 0 && (G == 1 || (p.out_gs * esz) % 16 == 0) &&
                   (!p.out2 || ((p.ldo2 * 2) % 16 == 0 && (G == 1 || (p.out2_gs * 2) % 16 == 0)))) ? 1 : 0;
    static const bool tma_off = []() { const char* e = std::getenv("MEMARCH_GEMM_TMA_STORE"); return e && e[0] == '0'; }();
    if (tma_off || (g_dbg & DBG_DIRECT_STORE)) p.store_tma = 0;
    if (p.store_tma) {
      const int No = sw ? N / 2 : N;
      tmO = make_tmap(p.out, esz, No, p.M, G, p.ldo, p.out_gs, p.out_f32 ? 32 : 64, 32, false);
      if (p.out2) tmO2 = make_tmap(p.out2, 2, N, p.M, G, p.ldo2, p.out2_gs, 64, 32, false);
      // SwiGLU backward writes (d gate | d up) side by side: one map per half, so a ragged last chunk of the first
      // half is clipped at H instead of running into the second
      if (p.epi == EPI_DSWIGLU)
        tmO2 = make_tmap(reinterpret_cast<const char*>(p.out) + (size_t)N * 2, 2, N, p.M, G, p.ldo, p.out_gs, 64, 32, false);
    }
  }
  CUtensorMap tmX = tmB;
  p.aux_tma = 0;
  if (v3 && (p.epi == EPI_DRELU2 || p.epi == EPI_DSWIGLU)) {
    // the pre-activations are prefetched by TMA (see AuxPipe); MEMARCH_GEMM_AUX_TMA=0 keeps the warp's own loads
    static const bool aux_off = []() { const char* e = std::getenv("MEMARCH_GEMM_AUX_TMA"); return e && e[0] == '0'; }();
    const int Nx = p.epi == EPI_DSWIGLU ? 2 * N : N;
    if (!aux_off && (p.ldaux * 2) % 16 == 0 && (G == 1 || (p.aux_gs * 2) % 16 == 0) && N % 8 == 0) {
      // 256-byte L2 promotion: a row's next 128-byte piece (the next chunk of the same tile) arrives with this one
      tmX = make_tmap(p.aux, 2, Nx, (uint64_t)n_seg * seg_M, G, p.ldaux, p.aux_gs, 64, 32, true);
      p.aux_tma = 1;
    }
  }
  auto launch = [&](auto kern, int id) {
    static bool attr_set[16][16] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_set[dev & 15][id]) {
      TORCH_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes) == cudaSuccess,
                  "cannot raise dynamic shared memory for the GEMM kernel");
      attr_set[dev & 15][id] = true;
    }
    if constexpr (std::is_invocable_v<decltype(kern), TmapSet, CUtensorMap, CUtensorMap, CUtensorMap, CUtensorMap, GemmParams>)
      kern<<<grid, GEMM_THREADS, smem_bytes, stream>>>(tmAs, tmB, tmO, tmO2, tmX, p);
    else
      kern<<<grid, GEMM_THREADS, smem_bytes, stream>>>(tmAs, tmB, p);
  };
  const int id = (a_mn ? 2 : 0) + (b_mn ? 1 : 0);
  if (v3 && tall) {
    if (!a_mn && !b_mn) launch(gemm_pair_kernel<false, false, 2>, 12 + id);
    else if (!a_mn && b_mn) launch(gemm_pair_kernel<false, true, 2>, 12 + id);
    else if (a_mn && !b_mn) launch(gemm_pair_kernel<true, false, 2>, 12 + id);
    else launch(gemm_pair_kernel<true, true, 2>, 12 + id);
  } else if (deep) {
    if (!b_mn) launch(gemm_pair_kernel<false, false, 1, true>, 4);
    else launch(gemm_pair_kernel<false, true, 1, true>, 5);
  } else if (v3) {
    if (!a_mn && !b_mn) launch(gemm_pair_kernel<false, false, 1>, 8 + id);
    else if (!a_mn && b_mn) launch(gemm_pair_kernel<false, true, 1>, 8 + id);
    else if (a_mn && !b_mn) launch(gemm_pair_kernel<true, false, 1>, 8 + id);
    else launch(gemm_pair_kernel<true, true, 1>, 8 + id);
  } else {
    if (!a_mn && !b_mn) launch(gemm_tc_kernel<false, false>, id);
    else if (!a_mn && b_mn) launch(gemm_tc_kernel<false, true>, id);
    else if (a_mn && !b_mn) launch(gemm_tc_kernel<true, false>, id);
    else launch(gemm_tc_kernel<true, true>, id);
  }
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

void launch_gemm(const void* A, long long a_rows_pitch, long long a_gs, bool a_mn, const void* B, long long b_rows_pitch,
                 long long b_gs, bool b_mn, GemmParams p, cudaStream_t stream, int max_ctas) {
  const void* list[1] = {A};
  launch_gemm_seg(list, 1, p.M, p.G, a_rows_pitch, a_gs, a_mn, B, b_rows_pitch, b_gs, b_mn, p, stream, max_ctas);
}

static int sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}

// torch binding.  a: (G?, M, K) or MN-major (G?, K, M); b: (G?, N, K) or MN-major (G?, K, N).
torch::Tensor gemm(torch::Tensor a, torch::Tensor b, c10::optional<torch::Tensor> out_,
                   c10::optional<torch::Tensor> out2_, c10::optional<torch::Tensor> aux_, bool a_mn, bool b_mn,
                   bool accumulate, int64_t epi, bool out_f32, int64_t groups, c10::optional<torch::Tensor> counts_,
                   int64_t count_mode) {
  TORCH_CHECK(a.is_cuda() && b.is_cuda(), "gemm: CUDA tensors expected");
  TORCH_CHECK(a.scalar_type() == torch::kBFloat16 && b.scalar_type() == torch::kBFloat16, "gemm: bf16 operands");
  const c10::cuda::CUDAGuard guard(a.device());
  const int G = (int)groups;
  auto as3 = [&](torch::Tensor t) { return t.dim() == 2 ? t.unsqueeze(0) : t; };
  torch::Tensor A = as3(a), B = as3(b);
  TORCH_CHECK(A.dim() == 3 && B.dim() == 3 && A.size(0) == G && B.size(0) == G, "gemm: group dimension mismatch");
  TORCH_CHECK(A.stride(2) == 1 && B.stride(2) == 1, "gemm: innermost dimension must be contiguous");
  const int M = a_mn ? A.size(2) : A.size(1), K = a_mn ? A.size(1) : A.size(2);
  const int N = b_mn ? B.size(2) : B.size(1), Kb = b_mn ? B.size(1) : B.size(2);
  TORCH_CHECK(K == Kb, "gemm: K mismatch ", K, " vs ", Kb);
  const int Nout = epi == EPI_SWIGLU ? N / 2 : (epi == EPI_DSWIGLU ? 2 * N : N);
  torch::Tensor out;
  if (out_.has_value() && out_->defined()) {
    out = *out_;
  } else {
    auto opt = a.options().dtype(out_f32 ? torch::kFloat32 : torch::kBFloat16);
    out = (a.dim() == 2 && G == 1) ? torch::empty({M, Nout}, opt) : torch::empty({G, M, Nout}, opt);
  }
  TORCH_CHECK(out.scalar_type() == (out_f32 ? torch::kFloat32 : torch::kBFloat16), "gemm: out dtype");
  torch::Tensor O = as3(out);
  TORCH_CHECK(O.size(0) == G && O.size(1) == M && O.size(2) == Nout && O.stride(2) == 1, "gemm: out shape");
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.G = G;
  p.out = O.data_ptr(); p.ldo = (int)O.stride(1); p.out_gs = G > 1 ? O.stride(0) : 0;
  p.epi = (int)epi; p.out_f32 = out_f32; p.accumulate = accumulate;
  TORCH_CHECK(!accumulate || out_f32, "gemm: accumulate needs an fp32 output");
  const int vec = out_f32 ? 4 : 8;
  TORCH_CHECK(p.ldo % vec == 0 && (reinterpret_cast<uintptr_t>(p.out) & 15) == 0 && (p.out_gs % vec) == 0,
              "gemm: output must allow 16-byte row stores");
  if (out2_.has_value() && out2_->defined()) {
    torch::Tensor O2 = as3(*out2_);
    TORCH_CHECK(O2.scalar_type() == torch::kBFloat16 && O2.stride(2) == 1 && O2.size(1) == M, "gemm: out2");
    p.out2 = O2.data_ptr(); p.ldo2 = (int)O2.stride(1); p.out2_gs = G > 1 ? O2.stride(0) : 0;
    TORCH_CHECK(p.ldo2 % 8 == 0 && (reinterpret_cast<uintptr_t>(p.out2) & 15) == 0, "gemm: out2 alignment");
  }
  TORCH_CHECK(epi != EPI_RELU2 || p.out2 != nullptr, "gemm: relu2 epilogue needs out2 for the pre-activation");
  if (aux_.has_value() && aux_->defined()) {
    if (epi == EPI_ROWSCALE) {
      TORCH_CHECK(aux_->scalar_type() == torch::kFloat32 && aux_->is_contiguous(), "gemm: row scale must be fp32");
      p.aux = aux_->data_ptr(); p.aux_gs = G > 1 ? M : 0;
    } else {
      torch::Tensor X = as3(*aux_);
      TORCH_CHECK(X.scalar_type() == torch::kBFloat16 && X.stride(2) == 1 && X.size(1) == M &&
                  X.size(2) == (epi == EPI_DSWIGLU ? 2 * N : N), "gemm: aux");
      p.aux = X.data_ptr(); p.ldaux = (int)X.stride(1); p.aux_gs = G > 1 ? X.stride(0) : 0;
      TORCH_CHECK(p.ldaux % 8 == 0 && (reinterpret_cast<uintptr_t>(p.aux) & 15) == 0, "gemm: aux alignment");
    }
  }
  TORCH_CHECK((epi != EPI_DRELU2 && epi != EPI_ROWSCALE && epi != EPI_DSWIGLU) || p.aux != nullptr, "gemm: epilogue needs aux");
  TORCH_CHECK(epi != EPI_DSWIGLU || (!out_f32 && N % 8 == 0 && M >= 256 && use_pair_kernel()),
              "gemm: the SwiGLU-backward epilogue writes bf16, needs a hidden width that is a multiple of 8 and the pair kernel (>= 256 rows)");
  if (counts_.has_value() && counts_->defined() && count_mode != 0) {
    TORCH_CHECK(counts_->is_cuda() && counts_->scalar_type() == torch::kInt32 && counts_->is_contiguous() &&
                counts_->numel() >= G, "gemm: counts must be a contiguous int32 CUDA tensor with one entry per group");
    TORCH_CHECK(count_mode == 1 || count_mode == 2, "gemm: count_mode 1 (rows) or 2 (contraction length)");
    p.counts = counts_->data_ptr<int>(); p.count_mode = (int)count_mode;
  }
  TORCH_CHECK(epi != EPI_SWIGLU || (!out_f32 && N % 16 == 0),
              "gemm: the SwiGLU epilogue writes bf16 and needs column halves of a multiple of 8 (16-byte TMA coordinates)");
  p.status = status_word(a.get_device());
  launch_gemm(A.data_ptr(), A.stride(1), G > 1 ? A.stride(0) : 0, a_mn, B.data_ptr(), B.stride(1), G > 1 ? B.stride(0) : 0,
              b_mn, p, at::cuda::getCurrentCUDAStream(), sm_count());
  return out;
}

// Segmented GEMM over peer buffers (expert parallelism without a separate all-to-all):
//   A rows of segment s come from `a_ptrs[s]`, a (a_groups, seg_M, K) bf16 buffer (a peer GPU's dispatch buffer);
//   group g of this launch reads A group `a_g_off + g`;
//   the result goes to `out_local` (G, n_seg*seg_M, N) or, when `out_ptrs` is given, rows of segment s go to
//   `out_ptrs[s]`, a (.., seg_M, N) buffer with row pitch `out_ld` and group pitch `out_gs` at group `out_g_off + g`.
torch::Tensor gemm_peer(std::vector<int64_t> a_ptrs, int64_t seg_M, int64_t K, int64_t a_groups, int64_t a_pitch,
                        int64_t a_gs, int64_t a_g_off, torch::Tensor b, bool b_mn, c10::optional<torch::Tensor> out_local,
                        std::vector<int64_t> out_ptrs, int64_t out_ld, int64_t out_gs, int64_t out_g_off,
                        c10::optional<torch::Tensor> out2_, c10::optional<torch::Tensor> aux_, int64_t epi, int64_t groups) {
  TORCH_CHECK(b.is_cuda() && b.scalar_type() == torch::kBFloat16, "gemm_peer: bf16 B");
  const c10::cuda::CUDAGuard guard(b.device());
  const int G = (int)groups, n_seg = (int)a_ptrs.size();
  torch::Tensor B = b.dim() == 2 ? b.unsqueeze(0) : b;
  TORCH_CHECK(B.size(0) == G && B.stride(2) == 1, "gemm_peer: B groups");
  const int N = b_mn ? B.size(2) : B.size(1), Kb = b_mn ? B.size(1) : B.size(2);
  TORCH_CHECK(Kb == K, "gemm_peer: K mismatch");
  const int M = n_seg * (int)seg_M;
  GemmParams p{};
  p.M = M; p.N = N; p.K = (int)K; p.G = G;
  p.epi = (int)epi; p.a_g_off = (int)a_g_off;
  torch::Tensor out;
  if (!out_ptrs.empty()) {
    TORCH_CHECK((int)out_ptrs.size() == n_seg, "gemm_peer: one output base per segment");
    for (int i = 0; i < n_seg; ++i) p.out_seg[i] = reinterpret_cast<void*>(out_ptrs[i]);
    p.out_seg_on = 1; p.out_g_off = (int)out_g_off; p.ldo = (int)out_ld; p.out_gs = out_gs;
    p.out = p.out_seg[0];
    TORCH_CHECK(out_ld % 8 == 0 && out_gs % 8 == 0, "gemm_peer: output pitches");
  } else {
    out = (out_local.has_value() && out_local->defined()) ? *out_local : torch::empty({G, M, N}, b.options());
    TORCH_CHECK(out.dim() == 3 && out.size(0) == G && out.size(1) == M && out.size(2) == N && out.stride(2) == 1, "gemm_peer: out");
    p.out = out.data_ptr(); p.ldo = (int)out.stride(1); p.out_gs = out.stride(0);
  }
  if (out2_.has_value() && out2_->defined()) {
    TORCH_CHECK(out2_->dim() == 3 && out2_->size(1) == M && out2_->stride(2) == 1, "gemm_peer: out2");
    p.out2 = out2_->data_ptr(); p.ldo2 = (int)out2_->stride(1); p.out2_gs = out2_->stride(0);
  }
  if (aux_.has_value() && aux_->defined()) {
    TORCH_CHECK(aux_->dim() == 3 && aux_->size(1) == M && aux_->stride(2) == 1, "gemm_peer: aux");
    p.aux = aux_->data_ptr(); p.ldaux = (int)aux_->stride(1); p.aux_gs = aux_->stride(0);
  }
  TORCH_CHECK(epi != EPI_RELU2 || p.out2 != nullptr, "gemm_peer: relu2 epilogue needs out2");
  p.status = status_word(b.get_device());
  std::vector<const void*> list(n_seg);
  for (int i = 0; i < n_seg; ++i) list[i] = reinterpret_cast<const void*>(a_ptrs[i]);
  launch_gemm_seg(list.data(), n_seg, (int)seg_M, (int)a_groups, a_pitch, a_gs, false, B.data_ptr(), B.stride(1),
                  G > 1 ? B.stride(0) : 0, b_mn, p, at::cuda::getCurrentCUDAStream(), sm_count());
  return out;
}

}  // namespace mb
