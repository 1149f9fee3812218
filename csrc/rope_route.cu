// Anchor routing of the long-range read (models/rope_memory.py): for every query, the best link of every anchor it may
// open and the K best anchors among them.
//
// The scores come from a tensor-core GEMM (queries x link keys, bf16 operands, fp32 accumulate): S (G, M, A*L) with
// G = batch x heads, M queries of one chunk, A anchors with L link keys each.  This kernel is the part that is not a
// GEMM: one warp per query row walks the anchors (a lane takes anchors lane, lane + 32, ...), skips the anchors the
// query may not open yet WITHOUT reading their scores (about half of the row for a causal text), keeps the best
// existing link of an anchor, and holds a sorted list of its K best anchors in registers; the lanes' lists are then
// merged by K rounds of a warp arg-max.  Ties go to the lower anchor number and, inside an anchor, to the first link,
// as `max` / `topk` of the PyTorch statement do on equal values.  No shared memory, no waits.
//
// What the reference runs here is a Pallas kernel doing K rounds of arg-max over the whole score tile
// (memarch_jax/memarch_jax/rope_pallas.py:43-120).
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <math.h>
#include <stdint.h>

namespace mb {

constexpr int RT_MAXK = 8;
constexpr int RT_WARPS = 8;

struct RouteArgs {
  const float* S;          // (G, M, A*L)
  const uint8_t* lval;     // (B, A, L)  the link exists
  const int* lp;           // (B, A, L)  its position in the text
  const uint8_t* avalid;   // (B, A)
  const int* open_from;    // (B, A)     first query position that may open the anchor
  long long* tidx;         // (G, M, K)
  uint8_t* tval;           // (G, M, K)
  long long* tpos;         // (G, M, K)
  int G, H, M, A, L, K, q0;
  float scale;
};

__global__ void __launch_bounds__(RT_WARPS * 32) rope_route_topk_kernel(RouteArgs a) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * RT_WARPS + (threadIdx.x >> 5);
  if (row >= (long long)a.G * a.M) return;                 // whole warps leave together
  const int g = (int)(row / a.M), m = (int)(row % a.M);
  const int b = g / a.H;
  const int qpos = a.q0 + m;
  const float* s_row = a.S + row * (long long)a.A * a.L;
  const uint8_t* lv_b = a.lval + (long long)b * a.A * a.L;
  const int* lp_b = a.lp + (long long)b * a.A * a.L;

  float bv[RT_MAXK];
  int ba[RT_MAXK], bp[RT_MAXK];
#pragma unroll
  for (int j = 0; j < RT_MAXK; ++j) { bv[j] = -INFINITY; ba[j] = 0x7fffffff; bp[j] = 0; }

  for (int an = lane; an < a.A; an += 32) {
    if (!a.avalid[(long long)b * a.A + an] || a.open_from[(long long)b * a.A + an] > qpos) continue;
    float best = -INFINITY;
    int best_p = 0;
    for (int l = 0; l < a.L; ++l) {
      if (!lv_b[(long long)an * a.L + l]) continue;
      const float s = s_row[(long long)an * a.L + l] * a.scale;
      if (s > best) { best = s; best_p = lp_b[(long long)an * a.L + l]; }
    }
    if (!(best > -INFINITY)) continue;                       // no link of this anchor exists
    // sorted insert (descending; anchors arrive in rising order, so strict '>' keeps the lower number first on ties);
    // the list always has RT_MAXK places, the first K of them are read at the end
    float cv = best;
    int ca = an, cp = best_p;
#pragma unroll
    for (int j = 0; j < RT_MAXK; ++j) {
      if (cv > bv[j]) {
        const float tv = bv[j]; const int ta = ba[j], tp = bp[j];
        bv[j] = cv; ba[j] = ca; bp[j] = cp;
        cv = tv; ca = ta; cp = tp;
      }
    }
  }

  // merge: K rounds, each takes the best head of the 32 lists
  for (int r = 0; r < a.K; ++r) {
    float v = bv[0];
    int an = ba[0];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, v, o);
      const int oa = __shfl_xor_sync(0xffffffffu, an, o);
      if (ov > v || (ov == v && oa < an)) { v = ov; an = oa; }
    }
    const bool found = v > -INFINITY;
    const bool mine = found && ba[0] == an && bv[0] == v;   // anchor numbers are unique across the lanes
    const unsigned who = __ballot_sync(0xffffffffu, mine);
    const int pos = __shfl_sync(0xffffffffu, bp[0], who ? __ffs(who) - 1 : 0);
    if (mine) {
#pragma unroll
      for (int j = 0; j + 1 < RT_MAXK; ++j) { bv[j] = bv[j + 1]; ba[j] = ba[j + 1]; bp[j] = bp[j + 1]; }
      bv[RT_MAXK - 1] = -INFINITY; ba[RT_MAXK - 1] = 0x7fffffff; bp[RT_MAXK - 1] = 0;
    }
    if (lane == 0) {
      const long long o = row * a.K + r;
      a.tidx[o] = found ? an : 0;
      a.tval[o] = found ? 1 : 0;
      a.tpos[o] = found ? pos : 0;
    }
  }
}

// S (G, M, A*L) fp32; lval (B, A, L) uint8; lp (B, A, L) int32; avalid (B, A) uint8; open_from (B, A) int32.
// Returns tidx, tval, tpos, each (G, M, K).
std::vector<torch::Tensor> rope_route_topk(torch::Tensor S, torch::Tensor lval, torch::Tensor lp, torch::Tensor avalid,
                                           torch::Tensor open_from, int64_t H, int64_t K, int64_t q0, double scale) {
  TORCH_CHECK(S.is_cuda() && S.dim() == 3 && S.is_contiguous() && S.scalar_type() == torch::kFloat32, "S: (G, M, A*L) fp32");
  TORCH_CHECK(lval.dim() == 3 && lval.is_contiguous() && lval.scalar_type() == torch::kUInt8, "lval: (B, A, L) uint8");
  const int64_t B = lval.size(0), A = lval.size(1), L = lval.size(2), G = S.size(0), M = S.size(1);
  TORCH_CHECK(H >= 1 && G == B * H && S.size(2) == A * L, "S does not match (B*H, M, A*L)");
  TORCH_CHECK(K >= 1 && K <= RT_MAXK, "K must be 1..", RT_MAXK);
  TORCH_CHECK(lp.is_contiguous() && lp.scalar_type() == torch::kInt32 && lp.numel() == B * A * L, "lp: (B, A, L) int32");
  TORCH_CHECK(avalid.is_contiguous() && avalid.scalar_type() == torch::kUInt8 && avalid.numel() == B * A, "avalid: (B, A) uint8");
  TORCH_CHECK(open_from.is_contiguous() && open_from.scalar_type() == torch::kInt32 && open_from.numel() == B * A,
              "open_from: (B, A) int32");
  TORCH_CHECK(lval.device() == S.device() && lp.device() == S.device() && avalid.device() == S.device() &&
              open_from.device() == S.device(), "all operands on the device of S");
  TORCH_CHECK(G * M < (1LL << 31) * RT_WARPS && A * L < (1LL << 31), "too large");
  c10::cuda::CUDAGuard guard(S.device());
  auto tidx = torch::empty({G, M, K}, S.options().dtype(torch::kInt64));
  auto tval = torch::empty({G, M, K}, S.options().dtype(torch::kUInt8));
  auto tpos = torch::empty({G, M, K}, S.options().dtype(torch::kInt64));
  if (G * M == 0) return {tidx, tval, tpos};
  RouteArgs a;
  a.S = S.data_ptr<float>();
  a.lval = lval.data_ptr<uint8_t>();
  a.lp = lp.data_ptr<int>();
  a.avalid = avalid.data_ptr<uint8_t>();
  a.open_from = open_from.data_ptr<int>();
  a.tidx = (long long*)tidx.data_ptr<int64_t>();
  a.tval = tval.data_ptr<uint8_t>();
  a.tpos = (long long*)tpos.data_ptr<int64_t>();
  a.G = (int)G; a.H = (int)H; a.M = (int)M; a.A = (int)A; a.L = (int)L; a.K = (int)K; a.q0 = (int)q0;
  a.scale = (float)scale;
  const long long rows = G * M;
  rope_route_topk_kernel<<<(unsigned)((rows + RT_WARPS - 1) / RT_WARPS), RT_WARPS * 32, 0,
                           at::cuda::getCurrentCUDAStream()>>>(a);
  return {tidx, tval, tpos};
}

}  // namespace mb
