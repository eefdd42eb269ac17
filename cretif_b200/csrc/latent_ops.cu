// Row kernels around an attention over a cached latent with a rotated key part that all heads
// share, 32-bit inside.
//
// latent_in: a token's projection row holds [cq (q_rank) | c (rank) | kr (rot) | ...].
//   cq <- cq / sqrt(mean(cq^2) + eps) * wq     -> cq_out (the query's latent, q_rank may be 0)
//   c  <- c  / sqrt(mean(c^2)  + eps) * wc
//   kr <- kr rotated by the token's position
//   the cache row of the token (ONE key/value head of size rank + rot) <- [c | kr]
//
// rope_heads: every head of q holds [flat (d) | rotated part (rot)]; the rotated part, turned by
// the token's position, goes to columns off .. off + rot of the head's row of `out` (whose heads
// are `ldh` apart): the tail of the query in latent space.
//
// Rotation: of the rot channels of a rotated part the first rdims are rotated, the rest pass;
// pair j is (j, j + rdims/2) (pairing 0) or (2j, 2j + 1) (pairing 1); (u, v) becomes
// (u cos - v sin, v cos + u sin), cos/sin from a 32-bit table [positions, rdims/2].
//
// rmsnorm_rows: x <- x / sqrt(mean(x^2) + eps) * w in place on float32 rows (the norm of an
// embedding's output, which stays in the 32-bit residual stream).
#include "api.h"
#include "common.cuh"

namespace cretif {

namespace {

__device__ __forceinline__ float rotated(const float* v, int i, int rdims, int pairing,
                                         const float* c, const float* s) {
  if (i >= rdims) return v[i];
  const int half = rdims >> 1;
  const bool first = pairing ? !(i & 1) : i < half;
  const int j = pairing ? i >> 1 : (first ? i : i - half);
  const int partner = pairing ? i ^ 1 : (first ? i + half : i - half);
  return first ? v[i] * c[j] - v[partner] * s[j] : v[i] * c[j] + v[partner] * s[j];
}

constexpr int kLatMaxRot = 512;

template <typename TI, typename T>
__global__ void __launch_bounds__(256)
latent_in_kernel(const TI* __restrict__ proj, int ldp, int q_rank, int rank, int rot, int rdims,
                 const float* __restrict__ wq, const float* __restrict__ wc, float eps,
                 const float* __restrict__ cos_t, const float* __restrict__ sin_t, int pairing,
                 const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                 const int* __restrict__ seq_slot, T* __restrict__ cq_out, int ldq,
                 const int* __restrict__ table, int table_stride, T* __restrict__ kc, int bt,
                 int write_cache, unsigned int* __restrict__ fault) {
  __shared__ float sums[2][8];
  __shared__ float kr[kLatMaxRot];
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const TI* row = proj + (size_t)t * ldp;
  const TI* crow = row + q_rank;
  // the two sums of squares in one pass over the row and one meeting of the warps
  float sq = 0.f, sc = 0.f;
  for (int i = threadIdx.x; i < q_rank; i += blockDim.x) {
    const float v = to_float(row[i]);
    sq += v * v;
  }
  for (int i = threadIdx.x; i < rank; i += blockDim.x) {
    const float v = to_float(crow[i]);
    sc += v * v;
  }
  for (int i = threadIdx.x; i < rot; i += blockDim.x) kr[i] = to_float(crow[rank + i]);
  sq = warp_sum(sq);
  sc = warp_sum(sc);
  if (lane == 0) { sums[0][warp] = sq; sums[1][warp] = sc; }
  __syncthreads();                              // (also publishes kr)
  sq = sc = 0.f;
#pragma unroll
  for (int w = 0; w < 8; ++w) { sq += sums[0][w]; sc += sums[1][w]; }
  if (q_rank > 0) {
    const float inv = 1.0f / sqrtf(sq / (float)q_rank + eps);
    T* dst = cq_out + (size_t)t * ldq;
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x)
      dst[i] = from_float<T>(to_float(row[i]) * inv * wq[i]);
  }
  if (!write_cache) return;
  const float inv = 1.0f / sqrtf(sc / (float)rank + eps);
  const int pos = tok_pos[t];
  const int slot = seq_slot[tok_seq[t]];
  const int blk = table[(size_t)slot * table_stride + pos / bt];
  if (blk < 0) {
    if (threadIdx.x == 0) atomicOr(fault, kFaultBlockTable);
    return;
  }
  T* dst = kc + ((size_t)blk * bt + (pos % bt)) * (rank + rot);
  for (int i = threadIdx.x; i < rank; i += blockDim.x)
    dst[i] = from_float<T>(to_float(crow[i]) * inv * wc[i]);
  const float* c = cos_t + (size_t)pos * (rdims >> 1);
  const float* s = sin_t + (size_t)pos * (rdims >> 1);
  for (int i = threadIdx.x; i < rot; i += blockDim.x)
    dst[rank + i] = from_float<T>(rotated(kr, i, rdims, pairing, c, s));
}

// The same for many tokens: a warp per token, no barrier; the second pass over the row finds it
// in the cache.
template <typename TI, typename T>
__global__ void __launch_bounds__(256)
latent_in_rows_kernel(const TI* __restrict__ proj, int ldp, int q_rank, int rank, int rot,
                      int rdims, const float* __restrict__ wq, const float* __restrict__ wc,
                      float eps,
                      const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                      int pairing, const int* __restrict__ tok_pos,
                      const int* __restrict__ tok_seq, const int* __restrict__ seq_slot,
                      T* __restrict__ cq_out, int ldq, const int* __restrict__ table,
                      int table_stride, T* __restrict__ kc, int bt, int write_cache, int T_tokens,
                      unsigned int* __restrict__ fault) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (t >= T_tokens) return;
  const TI* row = proj + (size_t)t * ldp;
  const TI* crow = row + q_rank;
  float sq = 0.f, sc = 0.f;
#pragma unroll 8
  for (int i = lane; i < q_rank; i += 32) {
    const float v = to_float(row[i]);
    sq += v * v;
  }
#pragma unroll 4
  for (int i = lane; i < rank; i += 32) {
    const float v = to_float(crow[i]);
    sc += v * v;
  }
  sq = warp_sum(sq);
  sc = warp_sum(sc);
  if (q_rank > 0) {
    const float inv = 1.0f / sqrtf(sq / (float)q_rank + eps);
    T* dst = cq_out + (size_t)t * ldq;
#pragma unroll 8
    for (int i = lane; i < q_rank; i += 32) dst[i] = from_float<T>(to_float(row[i]) * inv * wq[i]);
  }
  if (!write_cache) return;
  const float inv = 1.0f / sqrtf(sc / (float)rank + eps);
  const int pos = tok_pos[t];
  const int slot = seq_slot[tok_seq[t]];
  const int blk = table[(size_t)slot * table_stride + pos / bt];
  if (blk < 0) {
    if (lane == 0) atomicOr(fault, kFaultBlockTable);
    return;
  }
  T* dst = kc + ((size_t)blk * bt + (pos % bt)) * (rank + rot);
#pragma unroll 4
  for (int i = lane; i < rank; i += 32) dst[i] = from_float<T>(to_float(crow[i]) * inv * wc[i]);
  const int half = rdims >> 1;
  const float* c = cos_t + (size_t)pos * half;
  const float* s = sin_t + (size_t)pos * half;
  const TI* kr = crow + rank;
  for (int i = lane; i < rot; i += 32) {
    if (i >= rdims) {                      // beyond the rotated channels: as it is
      dst[rank + i] = from_float<T>(to_float(kr[i]));
      continue;
    }
    const bool first = pairing ? !(i & 1) : i < half;
    const int j = pairing ? i >> 1 : (first ? i : i - half);
    const int partner = pairing ? i ^ 1 : (first ? i + half : i - half);
    const float u = to_float(kr[i]), v = to_float(kr[partner]);
    dst[rank + i] = from_float<T>(first ? u * c[j] - v * s[j] : u * c[j] + v * s[j]);
  }
}

// many tokens: a thread per (token, head, pair of channels)
template <typename TI, typename T>
__global__ void __launch_bounds__(256)
rope_pairs_kernel(const TI* __restrict__ q, int ldq, int nh, int d, int rot, int rdims,
                  const float* __restrict__ cos_t, const float* __restrict__ sin_t, int pairing,
                  const int* __restrict__ tok_pos, T* __restrict__ out, int ldo, int ldh, int off,
                  long long total) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int slots = rot >> 1, half = rdims >> 1;
  const int j = (int)(idx % slots);
  const long long th = idx / slots;
  const int h = (int)(th % nh);
  const long long t = th / nh;
  const TI* src = q + (size_t)t * ldq + (size_t)h * (d + rot) + d;
  T* dst = out + (size_t)t * ldo + (size_t)h * ldh + off;
  if (j >= half) {                         // two of the channels that pass as they are
    const int a = rdims + 2 * (j - half);
    dst[a] = from_float<T>(to_float(src[a]));
    dst[a + 1] = from_float<T>(to_float(src[a + 1]));
    return;
  }
  const int a = pairing ? 2 * j : j, b = pairing ? 2 * j + 1 : j + half;
  const float u = to_float(src[a]), v = to_float(src[b]);
  const int pos = tok_pos[t];
  const float c = cos_t[(size_t)pos * half + j], s = sin_t[(size_t)pos * half + j];
  dst[a] = from_float<T>(u * c - v * s);
  dst[b] = from_float<T>(v * c + u * s);
}

// a warp per (token, head)
template <typename TI, typename T>
__global__ void __launch_bounds__(256)
rope_heads_kernel(const TI* __restrict__ q, int ldq, int nh, int d, int rot, int rdims,
                  const float* __restrict__ cos_t, const float* __restrict__ sin_t, int pairing,
                  const int* __restrict__ tok_pos, T* __restrict__ out, int ldo, int ldh, int off,
                  long long items) {
  __shared__ float part[8][kLatMaxRot];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * 8 + warp;
  if (item >= items) return;
  const int t = (int)(item / nh), h = (int)(item - (long long)t * nh);
  const TI* src = q + (size_t)t * ldq + (size_t)h * (d + rot) + d;
  float* mine = part[warp];
  for (int i = lane; i < rot; i += 32) mine[i] = to_float(src[i]);
  __syncwarp();
  const int pos = tok_pos[t];
  const float* c = cos_t + (size_t)pos * (rdims >> 1);
  const float* s = sin_t + (size_t)pos * (rdims >> 1);
  T* dst = out + (size_t)t * ldo + (size_t)h * ldh + off;
  for (int i = lane; i < rot; i += 32)
    dst[i] = from_float<T>(rotated(mine, i, rdims, pairing, c, s));
}

// a CTA per row, for a few rows: a lone warp would wait for its loads one after the other
__global__ void __launch_bounds__(256)
rmsnorm_row_block_kernel(float* __restrict__ x, int ld, const float* __restrict__ w, int H,
                         float eps) {
  __shared__ float scratch[33];
  float* row = x + (size_t)blockIdx.x * ld;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) ss += row[i] * row[i];
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x) row[i] = row[i] * inv * w[i];
}

// a warp per row
__global__ void __launch_bounds__(256)
rmsnorm_rows_kernel(float* __restrict__ x, int ld, const float* __restrict__ w, int R, int H,
                    float eps) {
  const int r = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (r >= R) return;
  float* row = x + (size_t)r * ld;
  float ss = 0.f;
#pragma unroll 8
  for (int i = lane; i < H; i += 32) ss += row[i] * row[i];
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)H + eps);
#pragma unroll 8
  for (int i = lane; i < H; i += 32) row[i] = row[i] * inv * w[i];
}

}  // namespace
}  // namespace cretif

using namespace cretif;

extern "C" int cretif_latent_in(const void* proj, int ldp, int proj_dt, int q_rank, int rank,
                                int rot, int rdims, const float* wq, const float* wc, float eps,
                                const float* cos_t, const float* sin_t, int pairing,
                                const int* tok_pos, const int* tok_seq, const int* seq_slot,
                                void* cq_out, int ldq, int dt, const int* table, int table_stride,
                                void* kc, int bt, int write_cache, int T, unsigned int* fault,
                                void* stream) {
  if (T <= 0) return kOk;
  if (q_rank < 0 || rank <= 0 || rot < 0 || rot > kLatMaxRot || (rot & 1) || rdims < 0 ||
      rdims > rot || (rdims & 1) || ldp < q_rank + rank + rot ||
      (q_rank > 0 && (!wq || !cq_out || ldq < q_rank)) || !wc ||
      (rdims > 0 && (!cos_t || !sin_t)))
    return kBadArgument;
  if (write_cache && (bt <= 0 || !kc || !table || !tok_seq || !seq_slot)) return kBadArgument;
  cudaStream_t st = (cudaStream_t)stream;
  // a CTA per token while the tokens are few (a decode step: its latency is what counts), a
  // warp per token for a prompt's rows
#define CRETIF_LAT(TI, TT)                                                                      \
  do {                                                                                          \
    if (T < 256)                                                                                \
      latent_in_kernel<TI, TT><<<T, 256, 0, st>>>(                                              \
          (const TI*)proj, ldp, q_rank, rank, rot, rdims, wq, wc, eps, cos_t, sin_t, pairing,    \
          tok_pos, tok_seq, seq_slot, (TT*)cq_out, ldq, table, table_stride, (TT*)kc, bt,        \
          write_cache, fault);                                                                    \
    else                                                                                        \
      latent_in_rows_kernel<TI, TT><<<(unsigned)((T + 7) / 8), 256, 0, st>>>(                    \
          (const TI*)proj, ldp, q_rank, rank, rot, rdims, wq, wc, eps, cos_t, sin_t, pairing,    \
          tok_pos, tok_seq, seq_slot, (TT*)cq_out, ldq, table, table_stride, (TT*)kc, bt,        \
          write_cache, T, fault);                                                                 \
  } while (0)
  if (proj_dt == kF32 && dt == kF32) CRETIF_LAT(float, float);
  else if (proj_dt == kF32 && dt == kBF16) CRETIF_LAT(float, __nv_bfloat16);
  else if (proj_dt == kBF16 && dt == kBF16) CRETIF_LAT(__nv_bfloat16, __nv_bfloat16);
  else return kBadDType;
#undef CRETIF_LAT
  return launch_status();
}

extern "C" int cretif_rope_heads(const void* q, int ldq, int q_dt, int nh, int d, int rot,
                                 int rdims, const float* cos_t, const float* sin_t, int pairing,
                                 const int* tok_pos, void* out, int ldo, int ldh, int off, int dt,
                                 int T, void* stream) {
  if (T <= 0 || rot == 0) return kOk;
  if (nh <= 0 || d < 0 || rot < 0 || rot > kLatMaxRot || (rot & 1) || rdims < 0 || rdims > rot ||
      (rdims & 1) || ldq < nh * (d + rot) || off < 0 || ldh < off + rot ||
      ldo < (nh - 1) * ldh + off + rot || (rdims > 0 && (!cos_t || !sin_t)))
    return kBadArgument;
  const long long items = (long long)T * nh;
  const unsigned blocks = (unsigned)((items + 7) / 8);
  cudaStream_t st = (cudaStream_t)stream;
  const long long pairs = items * (rot / 2);
#define CRETIF_RH(TI, TT)                                                                       \
  do {                                                                                          \
    if (T < 256)                                                                                \
      rope_heads_kernel<TI, TT><<<blocks, 256, 0, st>>>((const TI*)q, ldq, nh, d, rot, rdims,   \
                                                        cos_t, sin_t, pairing, tok_pos,         \
                                                        (TT*)out, ldo, ldh, off, items);        \
    else                                                                                        \
      rope_pairs_kernel<TI, TT><<<(unsigned)((pairs + 255) / 256), 256, 0, st>>>(               \
          (const TI*)q, ldq, nh, d, rot, rdims, cos_t, sin_t, pairing, tok_pos, (TT*)out, ldo,  \
          ldh, off, pairs);                                                                        \
  } while (0)
  if (q_dt == kF32 && dt == kF32) CRETIF_RH(float, float);
  else if (q_dt == kF32 && dt == kBF16) CRETIF_RH(float, __nv_bfloat16);
  else if (q_dt == kBF16 && dt == kBF16) CRETIF_RH(__nv_bfloat16, __nv_bfloat16);
  else return kBadDType;
#undef CRETIF_RH
  return launch_status();
}

extern "C" int cretif_rmsnorm_rows(float* x, int ld, const float* w, int R, int H, float eps,
                                   void* stream) {
  if (R <= 0) return kOk;
  if (H <= 0 || ld < H || !w) return kBadArgument;
  if (R <= 64)
    rmsnorm_row_block_kernel<<<R, 256, 0, (cudaStream_t)stream>>>(x, ld, w, H, eps);
  else
    rmsnorm_rows_kernel<<<(unsigned)((R + 7) / 8), 256, 0, (cudaStream_t)stream>>>(x, ld, w, R, H,
                                                                                   eps);
  return launch_status();
}
