// Routed experts: every token goes through `top` of E small feed-forward layers.
//
// A step's (token, choice) pairs are sorted by expert, and each expert's rows are then one
// slice of two grouped matrix products (gate|up with the activation in the epilogue, down):
//
// * moe_route (a CTA per token): router logits z = W_r x in 32-bit (W_r float32; x as stored),
//   score s = 1 / (1 + e^-z), the `top` largest (ties: the lower index), weights = the scores
//   as they are, or divided by their sum when asked.
// * moe_group (one CTA): counts per expert, offsets, each pair's place in the sorted list and
//   the list of row tiles (expert, first row) that the products walk.  The number of tiles is at
//   most ceil(pairs / 64) + E, which the host knows, so the grid does not depend on the routing
//   (a step can be replayed as a CUDA graph); unused tiles leave at once.
// * moe_gemm: C[r, :] = A[src(r), :] W[e(r)]^T for the sorted rows r, 64 x 64 tiles.  Mode
//   gate|up: W[e] = [gate (F rows) | up (F rows)], a tile owns the same 64 columns of both, and
//   writes act = silu(s g) (s u) with s the row's router weight (the weight scales the expert's
//   INPUT; the products are linear, so it is applied to the 32-bit sums); or, with the weight on
//   the output, act = silu(g) u and the down product's rows are scaled instead.  Two bodies:
//   32-bit FMA on the CUDA cores (any element type, the float32 path and the yardstick) and
//   bfloat16 on the tensor cores (mma.sync through the warp-level matrix API).
// * moe_combine: y[t] = sum over the token's choices, in the order of the choices (32-bit).
// * Many pairs in bfloat16 go to the library's tcgen05 product in its grouped mode instead
//   (gemm_tc.cu): moe_group pads every expert's rows to whole 128-row tiles, moe_gather_rows
//   writes the A operand in that order -- the token's row times its router weight, which is
//   where a weight on the expert's input belongs -- and the two products read which expert a row
//   tile belongs to.
// * A handful of pairs (a decode step) are not sorted at all: moe_gemv streams an expert's rows
//   once per pair.
#include <mma.h>

#include "api.h"
#include "common.cuh"

namespace cretif {

namespace {

constexpr int kTile = 64;
constexpr int kMaxExpertsPerLane = 8;            // E <= 256

// How a token's experts are chosen.  groups > 1: the experts form that many equal groups of
// neighbours, a group's score is the sum of its two largest logistic scores, and only experts of
// the `keep` best groups can be chosen.  renorm: the chosen scores are divided by their sum plus
// sum_eps.
struct RouteRule {
  int top, renorm, groups, keep;
  float sum_eps;
};

// Warp-wide: the `top` largest of E logits (ties: the lower index) among the experts of the groups
// that are kept, their logistic scores as weights, written for token t.  `scratch`: E floats and
// `groups` ints of shared memory that belong to this warp.
__device__ __forceinline__ void select_top(const float* logits, int E, const RouteRule rule,
                                           int* __restrict__ ids, float* __restrict__ wts, int t,
                                           int lane, float* scratch) {
  const int top = rule.top, renorm = rule.renorm;
  float z[kMaxExpertsPerLane];
#pragma unroll
  for (int m = 0; m < kMaxExpertsPerLane; ++m) {
    const int e = lane + 32 * m;
    z[m] = e < E ? logits[e] : -INFINITY;
  }
  if (rule.groups > 1) {
    const int per = E / rule.groups;
    int* kept = reinterpret_cast<int*>(scratch + E);
    __syncwarp();
#pragma unroll
    for (int m = 0; m < kMaxExpertsPerLane; ++m) {
      const int e = lane + 32 * m;
      if (e < E) scratch[e] = 1.0f / (1.0f + expf(-z[m]));
    }
    for (int g = lane; g < rule.groups; g += 32) kept[g] = 0;
    __syncwarp();
    // lane g % 32 scores group g: its two largest scores, summed
    float gs[kMaxExpertsPerLane];
#pragma unroll
    for (int m = 0; m < kMaxExpertsPerLane; ++m) {
      const int g = lane + 32 * m;
      gs[m] = -INFINITY;
      if (g < rule.groups) {
        float a = -INFINITY, b = -INFINITY;
        for (int i = 0; i < per; ++i) {
          const float v = scratch[g * per + i];
          if (v > a) { b = a; a = v; } else if (v > b) { b = v; }
        }
        gs[m] = per > 1 ? a + b : a;
      }
    }
    for (int k = 0; k < rule.keep; ++k) {
      float best = -INFINITY;
      int best_g = 0x7fffffff;
#pragma unroll
      for (int m = 0; m < kMaxExpertsPerLane; ++m) {
        const int g = lane + 32 * m;
        if (g < rule.groups && gs[m] > best) { best = gs[m]; best_g = g; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int og = __shfl_xor_sync(0xffffffffu, best_g, o);
        if (ob > best || (ob == best && og < best_g)) { best = ob; best_g = og; }
      }
      if (best_g == 0x7fffffff) break;
      if ((best_g & 31) == lane) {
#pragma unroll
        for (int m = 0; m < kMaxExpertsPerLane; ++m)
          if (m == (best_g >> 5)) gs[m] = -INFINITY;
        kept[best_g] = 1;
      }
    }
    __syncwarp();
#pragma unroll
    for (int m = 0; m < kMaxExpertsPerLane; ++m) {
      const int e = lane + 32 * m;
      if (e < E && !kept[e / per]) z[m] = -INFINITY;
    }
  }
  float total = 0.f;
  float my_w = 0.f;
  int my_id = 0;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int m = 0; m < kMaxExpertsPerLane; ++m) {
      const int e = lane + 32 * m;
      if (e < E && z[m] > best) { best = z[m]; best_e = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
    }
    if ((best_e & 31) == lane) {
#pragma unroll
      for (int m = 0; m < kMaxExpertsPerLane; ++m)
        if (m == (best_e >> 5)) z[m] = -INFINITY;
    }
    const float s = 1.0f / (1.0f + expf(-best));
    total += s;
    if (lane == k % 32 && k < 32) { my_w = s; my_id = best_e; }
    if (k >= 32 && lane == 0) {                  // more than 32 choices: written one by one
      ids[(size_t)t * top + k] = best_e;
      wts[(size_t)t * top + k] = s;
    }
  }
  if (lane < top && lane < 32) {
    ids[(size_t)t * top + lane] = my_id;
    wts[(size_t)t * top + lane] = renorm ? my_w / (total + rule.sum_eps) : my_w;
  }
  if (renorm && top > 32 && lane == 0)
    for (int k = 32; k < top; ++k) wts[(size_t)t * top + k] /= total + rule.sum_eps;
}

// A CTA per token: its sixteen warps take the experts in turn (a dot product each, every load of
// a row in flight at once where the width is a multiple of four), leave the logits in shared
// memory, and warp 0 picks the `top` largest.
constexpr int kRouteWarps = 16;
constexpr int kMaxExperts = 32 * kMaxExpertsPerLane;

__device__ __forceinline__ float4 ld4_as_float(const float* p) {
  return *reinterpret_cast<const float4*>(p);
}
__device__ __forceinline__ float4 ld4_as_float(const __nv_bfloat16* p) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  return make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xffff0000u),
                     __uint_as_float(u.y << 16), __uint_as_float(u.y & 0xffff0000u));
}

template <typename T>
__global__ void __launch_bounds__(kRouteWarps * 32)
moe_route_kernel(const T* __restrict__ x, int ldx, const float* __restrict__ wr, int E, int H,
                 const RouteRule rule, int* __restrict__ ids, float* __restrict__ wts, int vec) {
  __shared__ float logits[kMaxExperts];
  __shared__ float scratch[2 * kMaxExperts];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const T* row = x + (size_t)t * ldx;
  for (int e = warp; e < E; e += kRouteWarps) {
    const float* w = wr + (size_t)e * H;
    float acc = 0.f;
    if (vec) {
      const int n4 = H >> 2;
#pragma unroll 8
      for (int i = lane; i < n4; i += 32) {
        const float4 a = ld4_as_float(w + 4 * i), b = ld4_as_float(row + 4 * i);
        acc = fmaf(a.x, b.x, acc); acc = fmaf(a.y, b.y, acc);
        acc = fmaf(a.z, b.z, acc); acc = fmaf(a.w, b.w, acc);
      }
    } else {
#pragma unroll 8
      for (int i = lane; i < H; i += 32) acc = fmaf(w[i], to_float(row[i]), acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) logits[e] = acc;
  }
  __syncthreads();
  if (warp != 0) return;
  select_top(logits, E, rule, ids, wts, t, lane, scratch);
}

// The same choice from logits that a matrix product left in memory: a warp per token.
__global__ void __launch_bounds__(256)
moe_topk_kernel(const float* __restrict__ logits, int ld, int E, const RouteRule rule,
                int* __restrict__ ids, float* __restrict__ wts, int T) {
  __shared__ float scratch[8][2 * kMaxExperts];
  const int t = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (t >= T) return;
  select_top(logits + (size_t)t * ld, E, rule, ids, wts, t, threadIdx.x & 31,
             scratch[threadIdx.x >> 5]);
}

// tile: rows of a tile; padded: every expert's rows start at a multiple of `tile` (the sorted
// list then has gaps, and a tile never holds rows of two experts).  used[0] = tiles in use.
__global__ void __launch_bounds__(1024)
moe_group_kernel(const int* __restrict__ ids, int P, int E, int* __restrict__ offsets,
                 int* __restrict__ place, int* __restrict__ order, int* __restrict__ tile_expert,
                 int* __restrict__ tile_row0, int max_tiles, int tile, int padded,
                 int* __restrict__ used) {
  extern __shared__ int sh[];                    // counts [E], cursor [E], start [E + 1]
  int* counts = sh;
  int* cursor = sh + E;
  int* start = sh + 2 * E;
  for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = cursor[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < P; p += blockDim.x) atomicAdd(&counts[ids[p]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0, n_tiles = 0;
    for (int e = 0; e < E; ++e) {
      start[e] = at;
      if (offsets) offsets[e] = at;
      for (int r = 0; r < counts[e] && n_tiles < max_tiles; r += tile, ++n_tiles) {
        tile_expert[n_tiles] = e;
        if (tile_row0) tile_row0[n_tiles] = at + r;
      }
      at += padded ? (counts[e] + tile - 1) / tile * tile : counts[e];
    }
    start[E] = at;
    if (offsets) offsets[E] = at;
    if (used) used[0] = n_tiles;
    for (; n_tiles < max_tiles; ++n_tiles) tile_expert[n_tiles] = -1;
  }
  __syncthreads();
  for (int p = threadIdx.x; p < P; p += blockDim.x) {
    const int e = ids[p];
    const int at = start[e] + atomicAdd(&cursor[e], 1);
    place[p] = at;
    if (order) order[at] = p;
  }
}

// xs[place[p], :] = x[p / top, :] (times the pair's router weight, rounded once): the rows of a
// grouped product's A operand, gathered into the padded sorted order.
__global__ void __launch_bounds__(256)
moe_gather_rows_kernel(const __nv_bfloat16* __restrict__ x, int ldx,
                       __nv_bfloat16* __restrict__ xs, int lds, const int* __restrict__ place,
                       const float* __restrict__ wts, int top, int K, int vec) {
  const int p = blockIdx.x;
  const __nv_bfloat16* src = x + (size_t)(p / top) * ldx;
  __nv_bfloat16* dst = xs + (size_t)place[p] * lds;
  const float s = wts ? wts[p] : 1.f;
  if (vec) {
    for (int i = threadIdx.x * 8; i < K; i += 256 * 8) {
      float v[8];
      load8(src + i, v);
#pragma unroll
      for (int q = 0; q < 8; ++q) v[q] *= s;
      store8(dst + i, v);
    }
  } else {
    for (int i = threadIdx.x; i < K; i += 256) dst[i] = __float2bfloat16_rn(to_float(src[i]) * s);
  }
}

// What a tile's CTA learns about its rows.
struct TileRows {
  int expert, row0, rows;
};

__device__ __forceinline__ TileRows tile_rows(const int* tile_expert, const int* tile_row0,
                                              const int* offsets, int tile) {
  TileRows tr;
  tr.expert = tile_expert[tile];
  tr.row0 = tr.expert >= 0 ? tile_row0[tile] : 0;
  tr.rows = tr.expert >= 0 ? min(kTile, offsets[tr.expert + 1] - tr.row0) : 0;
  return tr;
}

// mode 0: gate|up with the activation; mode 1: plain product into float32 rows; mode 2 + k: an
// expert without a gate, C = act_k(A W^T) with kind k of unary_activation, rows as in mode 0.
// scale_at: 0 none, 1 the router weight scales the sums of mode 0 (the expert's input),
// 2 it scales the rows of mode 1 (the expert's output).
template <typename TA, typename TW>
__global__ void __launch_bounds__(256)
moe_gemm_simt_kernel(const TA* __restrict__ A, int lda, const TW* __restrict__ W, void* Cv,
                     int ldc, int N, int K, int top, int mode, int scale_at,
                     const float* __restrict__ wts, const int* __restrict__ order,
                     const int* __restrict__ offsets, const int* __restrict__ tile_expert,
                     const int* __restrict__ tile_row0) {
  constexpr int BK = 16, TM = 4, TN = 4;
  const TileRows tr = tile_rows(tile_expert, tile_row0, offsets, blockIdx.y);
  if (tr.rows <= 0) return;
  __shared__ float As[BK][kTile + 4];
  __shared__ float Ws[2][BK][kTile + 4];
  const int tid = threadIdx.x;
  const int n0 = blockIdx.x * kTile;
  const int tx = tid & 15, ty = tid >> 4;
  const int lrow = tid >> 2, lk = (tid & 3) * 4;
  const int halves = mode == 0 ? 2 : 1;
  const size_t w_rows = (size_t)(mode == 0 ? 2 * N : N);
  const TW* We = W + (size_t)tr.expert * w_rows * K;
  // the row of A that the loader thread fetches
  int a_src = -1;
  if (lrow < tr.rows) a_src = mode != 1 ? order[tr.row0 + lrow] / top : tr.row0 + lrow;
  const int wn = n0 + lrow;
  float acc[2][TM][TN];
#pragma unroll
  for (int g = 0; g < 2; ++g)
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
      for (int j = 0; j < TN; ++j) acc[g][i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int k = k0 + lk + e;
      As[lk + e][lrow] = (a_src >= 0 && k < K) ? to_float(A[(size_t)a_src * lda + k]) : 0.f;
      Ws[0][lk + e][lrow] = (wn < N && k < K) ? to_float(We[(size_t)wn * K + k]) : 0.f;
      if (halves == 2)
        Ws[1][lk + e][lrow] = (wn < N && k < K) ? to_float(We[((size_t)N + wn) * K + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], w[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int g = 0; g < 2; ++g) {
        if (g < halves) {
#pragma unroll
          for (int j = 0; j < TN; ++j) w[j] = Ws[g][kk][tx * TN + j];
#pragma unroll
          for (int i = 0; i < TM; ++i)
#pragma unroll
            for (int j = 0; j < TN; ++j) acc[g][i][j] = fmaf(a[i], w[j], acc[g][i][j]);
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int lr = ty * TM + i;
    if (lr >= tr.rows) continue;
    const int r = tr.row0 + lr;
    const float s = scale_at ? wts[order[r]] : 1.f;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tx * TN + j;
      if (n >= N) continue;
      if (mode == 0) {
        const float sg = scale_at == 1 ? s : 1.f;
        const float g = acc[0][i][j] * sg, u = acc[1][i][j] * sg;
        reinterpret_cast<TA*>(Cv)[(size_t)r * ldc + n] = from_float<TA>(g / (1.0f + expf(-g)) * u);
      } else if (mode >= 2) {
        reinterpret_cast<TA*>(Cv)[(size_t)r * ldc + n] = from_float<TA>(
            unary_activation(acc[0][i][j] * (scale_at == 1 ? s : 1.f), mode - 2));
      } else {
        reinterpret_cast<float*>(Cv)[(size_t)r * ldc + n] =
            acc[0][i][j] * (scale_at == 2 ? s : 1.f);
      }
    }
  }
}

// The same tiles on the tensor cores, bfloat16 operands, 32-bit sums: four warps, each a
// 32 x 32 corner of the tile as 2 x 2 fragments (two sets of them in gate|up mode).
constexpr int kTK = 64, kTPad = 8;

__global__ void __launch_bounds__(128)
moe_gemm_mma_kernel(const __nv_bfloat16* __restrict__ A, int lda,
                    const __nv_bfloat16* __restrict__ W, void* Cv, int ldc, int N, int K, int top,
                    int mode, int scale_at, const float* __restrict__ wts,
                    const int* __restrict__ order, const int* __restrict__ offsets,
                    const int* __restrict__ tile_expert, const int* __restrict__ tile_row0,
                    int a_vec, int w_vec) {
  using namespace nvcuda;
  const TileRows tr = tile_rows(tile_expert, tile_row0, offsets, blockIdx.y);
  if (tr.rows <= 0) return;
  extern __shared__ __align__(32) unsigned char moe_smem[];
  typedef __nv_bfloat16 (*Slab)[kTK + kTPad];
  Slab As = reinterpret_cast<Slab>(moe_smem);
  Slab Wg = As + kTile;
  Slab Wu = Wg + kTile;
  __shared__ int src_row[kTile];
  const int halves = mode == 0 ? 2 : 1;
  const size_t w_rows = (size_t)(mode == 0 ? 2 * N : N);
  const __nv_bfloat16* We = W + (size_t)tr.expert * w_rows * K;
  const int n0 = blockIdx.x * kTile;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int wm = (warp >> 1) * 32, wn = (warp & 1) * 32;
  const int tid = (int)threadIdx.x;
  if (tid < kTile)
    src_row[tid] = tid < tr.rows ? (mode != 1 ? order[tr.row0 + tid] / top : tr.row0 + tid) : -1;
  __syncthreads();
  wmma::fragment<wmma::accumulator, 16, 16, 16, float> acc[2][2][2];
#pragma unroll
  for (int g = 0; g < 2; ++g)
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < 2; ++j) wmma::fill_fragment(acc[g][i][j], 0.f);
  auto stage = [&](Slab dst, const __nv_bfloat16* src, int ld, int k0, bool gather, int nrows,
                   int first, bool vec_ok) {
    for (int idx = threadIdx.x; idx < kTile * (kTK / 8); idx += blockDim.x) {
      const int r = idx / (kTK / 8), c = (idx - r * (kTK / 8)) * 8;
      const int k = k0 + c;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      const int row = gather ? src_row[r] : (first + r < nrows ? first + r : -1);
      if (row >= 0) {
        const __nv_bfloat16* p = src + (size_t)row * ld + k;
        if (vec_ok && k + 8 <= K) {
          v = *reinterpret_cast<const uint4*>(p);
        } else {
          __nv_bfloat16 tmp[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) tmp[e] = k + e < K ? p[e] : __float2bfloat16_rn(0.f);
          v = *reinterpret_cast<const uint4*>(tmp);
        }
      }
      *reinterpret_cast<uint4*>(&dst[r][c]) = v;
    }
  };
  for (int k0 = 0; k0 < K; k0 += kTK) {
    stage(As, A, lda, k0, true, 0, 0, a_vec);
    stage(Wg, We, K, k0, false, N, n0, w_vec);
    if (halves == 2) stage(Wu, We + (size_t)N * K, K, k0, false, N, n0, w_vec);
    __syncthreads();
    const int kk_end = min(kTK, ((K - k0 + 15) / 16) * 16);
    for (int kk = 0; kk < kk_end; kk += 16) {
      wmma::fragment<wmma::matrix_a, 16, 16, 16, __nv_bfloat16, wmma::row_major> fa[2];
      wmma::fragment<wmma::matrix_b, 16, 16, 16, __nv_bfloat16, wmma::col_major> fb[2];
#pragma unroll
      for (int i = 0; i < 2; ++i) wmma::load_matrix_sync(fa[i], &As[wm + 16 * i][kk], kTK + kTPad);
#pragma unroll
      for (int g = 0; g < 2; ++g) {
        if (g < halves) {
          Slab Ws = g == 0 ? Wg : Wu;
#pragma unroll
          for (int j = 0; j < 2; ++j)
            wmma::load_matrix_sync(fb[j], &Ws[wn + 16 * j][kk], kTK + kTPad);
#pragma unroll
          for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int j = 0; j < 2; ++j) wmma::mma_sync(acc[g][i][j], fa[i], fb[j], acc[g][i][j]);
        }
      }
    }
    __syncthreads();
  }
  // the sums leave through shared memory (the operand slabs are free now): [2][4][32][36] floats
  float (*Cs)[4][32][36] = reinterpret_cast<float (*)[4][32][36]>(moe_smem);
#pragma unroll
  for (int g = 0; g < 2; ++g)
    if (g < halves)
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 2; ++j)
          wmma::store_matrix_sync(&Cs[g][warp][16 * i][16 * j], acc[g][i][j], 36,
                                  wmma::mem_row_major);
  __syncwarp();
  const int lr = wm + lane;
  if (lr >= tr.rows) return;
  const int r = tr.row0 + lr;
  const float s = scale_at ? wts[order[r]] : 1.f;
  for (int c = 0; c < 32; ++c) {
    const int n = n0 + wn + c;
    if (n >= N) break;
    if (mode == 0) {
      const float sg = scale_at == 1 ? s : 1.f;
      const float g = Cs[0][warp][lane][c] * sg, u = Cs[1][warp][lane][c] * sg;
      reinterpret_cast<__nv_bfloat16*>(Cv)[(size_t)r * ldc + n] =
          __float2bfloat16_rn(silu_bf16_path(g) * u);
    } else if (mode >= 2) {
      reinterpret_cast<__nv_bfloat16*>(Cv)[(size_t)r * ldc + n] = __float2bfloat16_rn(
          unary_activation(Cs[0][warp][lane][c] * (scale_at == 1 ? s : 1.f), mode - 2));
    } else {
      reinterpret_cast<float*>(Cv)[(size_t)r * ldc + n] =
          Cs[0][warp][lane][c] * (scale_at == 2 ? s : 1.f);
    }
  }
}

// The same two products for a handful of pairs (a decode step), unsorted: a CTA owns 16 output
// columns of ONE pair, streams its expert's rows for them once (16-byte loads, all of a row's in
// flight together) against the pair's input row held in shared memory; warp w takes columns
// 2w and 2w + 1.  mode 0: C[p, n] = silu(s g) (s u) from the gate row n and the up row N + n;
// mode 1: C[p, n] = the product (times s with scale_at 2), float32; mode 2 + k: C[p, n] =
// act_k(s * the product) from row n of an expert without a gate.
template <typename T>
__global__ void __launch_bounds__(256)
moe_gemv_kernel(const T* __restrict__ A, int lda, const T* __restrict__ W, void* Cv, int ldc, int N,
                int K, int top, int mode, int scale_at, const int* __restrict__ ids,
                const float* __restrict__ wts, int vec) {
  extern __shared__ __align__(16) unsigned char gemv_smem[];
  T* xs = reinterpret_cast<T*>(gemv_smem);
  const int p = blockIdx.y;
  const int e = ids[p];
  const float s = scale_at ? wts[p] : 1.f;
  const T* arow = A + (size_t)(mode != 1 ? p / top : p) * lda;
  if (vec) {
    const int bytes = K * (int)sizeof(T);               // a multiple of 16
    const unsigned char* src = reinterpret_cast<const unsigned char*>(arow);
    for (int o = threadIdx.x * 16; o < bytes; o += 256 * 16)
      *reinterpret_cast<uint4*>(gemv_smem + o) = *reinterpret_cast<const uint4*>(src + o);
  } else {
    for (int i = threadIdx.x; i < K; i += 256) xs[i] = arow[i];
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const size_t w_rows = (size_t)(mode == 0 ? 2 * N : N);
  const T* We = W + (size_t)e * w_rows * K;
  auto dot = [&](const T* wrow) {
    float acc = 0.f;
    if (vec) {
#pragma unroll 4
      for (int i = lane * 8; i < K; i += 256) {
        float a[8], b[8];
        load8(wrow + i, a);
        load8(xs + i, b);
#pragma unroll
        for (int q = 0; q < 8; ++q) acc = fmaf(a[q], b[q], acc);
      }
    } else {
      for (int i = lane; i < K; i += 32) acc = fmaf(to_float(wrow[i]), to_float(xs[i]), acc);
    }
    return warp_sum(acc);
  };
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    const int n = blockIdx.x * 16 + warp * 2 + c;
    if (n >= N) continue;
    if (mode == 0) {
      const float sg = scale_at == 1 ? s : 1.f;
      const float g = dot(We + (size_t)n * K) * sg, u = dot(We + ((size_t)N + n) * K) * sg;
      if (lane == 0)
        reinterpret_cast<T*>(Cv)[(size_t)p * ldc + n] = from_float<T>(g / (1.0f + expf(-g)) * u);
    } else if (mode >= 2) {
      const float v = dot(We + (size_t)n * K) * (scale_at == 1 ? s : 1.f);
      if (lane == 0)
        reinterpret_cast<T*>(Cv)[(size_t)p * ldc + n] = from_float<T>(unary_activation(v, mode - 2));
    } else {
      const float v = dot(We + (size_t)n * K) * (scale_at == 2 ? s : 1.f);
      if (lane == 0) reinterpret_cast<float*>(Cv)[(size_t)p * ldc + n] = v;
    }
  }
}

__global__ void __launch_bounds__(256)
moe_combine_kernel(const float* __restrict__ rows, int ld, const int* __restrict__ place, int top,
                   const float* __restrict__ wts, float* __restrict__ y, int T, int H) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)T * H) return;
  const int t = (int)(idx / H), c = (int)(idx - (long long)t * H);
  float acc = 0.f;
  for (int k = 0; k < top; ++k) {
    const size_t pair = (size_t)t * top + k;
    const float v = rows[(place ? (size_t)place[pair] : pair) * ld + c];
    acc += wts ? wts[pair] * v : v;
  }
  y[idx] = acc;
}

}  // namespace
}  // namespace cretif

using namespace cretif;

// groups <= 1: no groups.  Else the experts divide into the groups evenly and the groups that
// are kept hold `top` experts at least.
static bool route_rule_ok(int E, int top, int groups, int keep) {
  if (groups <= 1) return true;
  return E % groups == 0 && keep >= 1 && keep <= groups && (long long)keep * (E / groups) >= top;
}

extern "C" int cretif_moe_route(const void* x, int x_dt, int ldx, const float* router_w, int E,
                                int H, int top, int renorm, int groups, int keep, float sum_eps,
                                int* ids, float* wts, int T, void* stream) {
  if (T <= 0) return kOk;
  if (E <= 0 || E > 32 * kMaxExpertsPerLane || H <= 0 || top <= 0 || top > E || ldx < H)
    return kBadArgument;
  if (!route_rule_ok(E, top, groups, keep)) return kBadArgument;
  const RouteRule rule{top, renorm, groups, keep, sum_eps};
  cudaStream_t st = (cudaStream_t)stream;
  const int vec = H % 4 == 0 && ldx % 4 == 0 && (((uintptr_t)x | (uintptr_t)router_w) & 15) == 0;
  if (x_dt == kF32)
    moe_route_kernel<float><<<T, kRouteWarps * 32, 0, st>>>((const float*)x, ldx, router_w, E, H,
                                                            rule, ids, wts, vec);
  else if (x_dt == kBF16)
    moe_route_kernel<__nv_bfloat16><<<T, kRouteWarps * 32, 0, st>>>(
        (const __nv_bfloat16*)x, ldx, router_w, E, H, rule, ids, wts, vec);
  else
    return kBadDType;
  return launch_status();
}

// ids/wts from logits [T, ld >= E] that a matrix product computed.
extern "C" int cretif_moe_topk(const float* logits, int ld, int E, int top, int renorm, int groups,
                               int keep, float sum_eps, int* ids, float* wts, int T,
                               void* stream) {
  if (T <= 0) return kOk;
  if (E <= 0 || E > kMaxExperts || top <= 0 || top > E || ld < E) return kBadArgument;
  if (!route_rule_ok(E, top, groups, keep)) return kBadArgument;
  const RouteRule rule{top, renorm, groups, keep, sum_eps};
  moe_topk_kernel<<<(unsigned)((T + 7) / 8), 256, 0, (cudaStream_t)stream>>>(logits, ld, E, rule,
                                                                             ids, wts, T);
  return launch_status();
}

extern "C" int cretif_moe_group(const int* ids, int P, int E, int* offsets, int* place, int* order,
                                int* tile_expert, int* tile_row0, int max_tiles, void* stream) {
  if (P <= 0) return kOk;
  if (E <= 0 || E > 4096 || max_tiles < (P + kTile - 1) / kTile + E) return kBadArgument;
  moe_group_kernel<<<1, 1024, sizeof(int) * (3 * E + 1), (cudaStream_t)stream>>>(
      ids, P, E, offsets, place, order, tile_expert, tile_row0, max_tiles, kTile, 0, nullptr);
  return launch_status();
}

// The padded order for the tensor-core grouped products: every expert's rows start at a multiple
// of `tile` rows; place [P], tile_expert [max_tiles >= ceil(P / tile) + E], used [1].
extern "C" int cretif_moe_group_padded(const int* ids, int P, int E, int tile, int* place,
                                       int* tile_expert, int max_tiles, int* used, void* stream) {
  if (P <= 0) return kOk;
  if (E <= 0 || E > 4096 || tile <= 0 || max_tiles < (P + tile - 1) / tile + E || !used)
    return kBadArgument;
  moe_group_kernel<<<1, 1024, sizeof(int) * (3 * E + 1), (cudaStream_t)stream>>>(
      ids, P, E, nullptr, place, nullptr, tile_expert, nullptr, max_tiles, tile, 1, used);
  return launch_status();
}

// xs[place[p]] = x[p / top] * wts[p] (wts may be null), bfloat16 rows of K columns.
extern "C" int cretif_moe_gather_rows(const void* x, int ldx, void* xs, int lds, const int* place,
                                      const float* wts, int top, int K, int P, void* stream) {
  if (P <= 0) return kOk;
  if (K <= 0 || ldx < K || lds < K || top <= 0) return kBadArgument;
  const int vec = K % 8 == 0 && ldx % 8 == 0 && lds % 8 == 0 &&
                  (((uintptr_t)x | (uintptr_t)xs) & 15) == 0;
  moe_gather_rows_kernel<<<P, 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, ldx, (__nv_bfloat16*)xs, lds, place, wts, top, K, vec);
  return launch_status();
}

// mode 0: A [tokens, K] (row of pair p: p / top), W [E, 2N, K], C [P, N] in A's element type.
// mode 2 + k: the same rows, W [E, N, K], C = act_k(product) (k: a kind of unary_activation).
// mode 1: A [P, K] sorted rows, W [E, N, K], C [P, N] float32.  use_mma: the tensor-core body
// (bfloat16 only).
extern "C" int cretif_moe_gemm(const void* A, int a_dt, int lda, const void* W, int w_dt, void* C,
                               int ldc, int N, int K, int top, int mode, int scale_at,
                               const float* wts, const int* order, const int* offsets,
                               const int* tile_expert, const int* tile_row0, int max_tiles,
                               int use_mma, void* stream) {
  if (max_tiles <= 0) return kOk;
  if (N <= 0 || K <= 0 || lda < K || ldc < N || top <= 0 || mode < 0 || mode >= 2 + kUnaryKinds ||
      scale_at < 0 || scale_at > 2 || max_tiles > 65535 || a_dt != w_dt)
    return kBadArgument;
  cudaStream_t st = (cudaStream_t)stream;
  dim3 grid((N + kTile - 1) / kTile, max_tiles);
  typedef __nv_bfloat16 bf16;
  if (use_mma) {
    if (a_dt != kBF16) return kBadDType;
    const int a_vec = ((uintptr_t)A % 16 == 0) && lda % 8 == 0;
    const int w_vec = ((uintptr_t)W % 16 == 0) && K % 8 == 0;
    const size_t slabs = sizeof(bf16) * 3 * kTile * (kTK + kTPad);
    const size_t outs = sizeof(float) * 2 * 4 * 32 * 36;
    const size_t smem = slabs > outs ? slabs : outs;
    static bool raised = false;
    if (!raised) {
      cudaError_t err = cudaFuncSetAttribute(moe_gemm_mma_kernel,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
      if (err != cudaSuccess) return (int)err;
      raised = true;
    }
    moe_gemm_mma_kernel<<<grid, 128, smem, st>>>((const bf16*)A, lda, (const bf16*)W, C, ldc, N, K,
                                                 top, mode, scale_at, wts, order, offsets,
                                                 tile_expert, tile_row0, a_vec, w_vec);
    return launch_status();
  }
  if (a_dt == kF32)
    moe_gemm_simt_kernel<float, float><<<grid, 256, 0, st>>>(
        (const float*)A, lda, (const float*)W, C, ldc, N, K, top, mode, scale_at, wts, order,
        offsets, tile_expert, tile_row0);
  else if (a_dt == kBF16)
    moe_gemm_simt_kernel<bf16, bf16><<<grid, 256, 0, st>>>(
        (const bf16*)A, lda, (const bf16*)W, C, ldc, N, K, top, mode, scale_at, wts, order,
        offsets, tile_expert, tile_row0);
  else
    return kBadDType;
  return launch_status();
}

// The products for few pairs, in the pairs' own order (no sorting): A, W, C as in cretif_moe_gemm
// with C's rows indexed by the pair.
extern "C" int cretif_moe_gemv(const void* A, int a_dt, int lda, const void* W, int w_dt, void* C,
                               int ldc, int N, int K, int top, int mode, int scale_at,
                               const int* ids, const float* wts, int P, void* stream) {
  if (P <= 0) return kOk;
  if (N <= 0 || K <= 0 || lda < K || ldc < N || top <= 0 || mode < 0 || mode >= 2 + kUnaryKinds ||
      scale_at < 0 || scale_at > 2 || P > 65535 || a_dt != w_dt)
    return kBadArgument;
  const size_t esz = a_dt == kF32 ? 4 : 2;
  const size_t smem = (size_t)K * esz;
  if (smem > 96 * 1024) return kBadArgument;
  const int vec = K % 8 == 0 && lda % 8 == 0 && (((uintptr_t)A | (uintptr_t)W) & 15) == 0;
  dim3 grid((N + 15) / 16, P);
  cudaStream_t st = (cudaStream_t)stream;
  typedef __nv_bfloat16 bf16;
  if (a_dt == kF32) {
    if (smem > 48 * 1024) {
      cudaError_t err = cudaFuncSetAttribute(moe_gemv_kernel<float>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
      if (err != cudaSuccess) return (int)err;
    }
    moe_gemv_kernel<float><<<grid, 256, smem, st>>>((const float*)A, lda, (const float*)W, C, ldc,
                                                    N, K, top, mode, scale_at, ids, wts, vec);
  } else if (a_dt == kBF16) {
    if (smem > 48 * 1024) {
      cudaError_t err = cudaFuncSetAttribute(moe_gemv_kernel<bf16>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
      if (err != cudaSuccess) return (int)err;
    }
    moe_gemv_kernel<bf16><<<grid, 256, smem, st>>>((const bf16*)A, lda, (const bf16*)W, C, ldc, N,
                                                   K, top, mode, scale_at, ids, wts, vec);
  } else {
    return kBadDType;
  }
  return launch_status();
}

extern "C" int cretif_moe_combine(const float* rows, int ld, const int* place, int top,
                                  const float* wts, float* y, int T, int H, void* stream) {
  if (T <= 0) return kOk;
  if (H <= 0 || ld < H || top <= 0) return kBadArgument;
  const unsigned blocks = (unsigned)(((long long)T * H + 255) / 256);
  moe_combine_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(rows, ld, place, top, wts, y, T, H);
  return launch_status();
}
