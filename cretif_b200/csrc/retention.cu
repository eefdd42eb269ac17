// Retention: linear attention with a fixed decay per head, no softmax and no denominator.
//
// Per token and head, with state S [d, e] (32-bit, zero at a sequence's start):
//     S <- decay_h S + k v^T;   o = S^T q
// so the read-out sees the token's own write.  Two kernels serve any step shape (whole
// prompts, further chunks at a cached position, single tokens), all arithmetic in 32-bit:
//
// * retention_prepare (a CTA per token): the first rot_dim channels of every query and key head
//   are rotated by the token's position (cos/sin from a 32-bit table), the key is multiplied
//   by k_scale after the rotation.
// * retention_recurrence (a CTA per (sequence, head, slice of columns)): the columns of S are
//   independent; a group of P lanes owns one column, each lane R contiguous rows of it in
//   registers.  Tokens go in chunks of 16 whose q, k and v are staged in shared memory (a
//   lane's slice of q and k padded so that the P slices fall into different banks); a token
//   costs one P-lane shuffle reduction and no barrier.  The read-outs leave in 32-bit through
//   shared memory, a chunk at a time.  The state is read once and written once per step.
//
// The read-outs are normed per head and gated by heads_out_norm (delta_rule.cu).
#include "api.h"
#include "common.cuh"

namespace cretif {

namespace {

// proj row (float32): [q (H d) | k (H d) | ...];  prep row: [q (H d) | k (H d)]
__global__ void __launch_bounds__(256)
retention_prepare_kernel(const float* __restrict__ proj, int ldp, float* __restrict__ prep, int ldo,
                         const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                         int pairing, int rot_dim, const int* __restrict__ tok_pos, int H, int d,
                         float k_scale) {
  const int t = blockIdx.x;
  const int pos = tok_pos[t];
  const int half = rot_dim >> 1;
  const float* c = cos_t + (size_t)pos * half;
  const float* s = sin_t + (size_t)pos * half;
  const float* row = proj + (size_t)t * ldp;
  float* out = prep + (size_t)t * ldo;
  const int n = 2 * H * d;
  for (int idx = threadIdx.x; idx < n; idx += blockDim.x) {
    const int head = idx / d, i = idx - head * d;
    float v = row[idx];
    if (i < rot_dim) {
      const bool first = pairing ? !(i & 1) : i < half;
      const int j = pairing ? i >> 1 : (first ? i : i - half);
      const int partner = pairing ? i ^ 1 : (first ? i + half : i - half);
      const float other = row[idx - i + partner];
      v = first ? v * c[j] - other * s[j] : v * c[j] + other * s[j];
    }
    out[idx] = head >= H ? v * k_scale : v;
  }
}

constexpr int kRetChunk = 16;

// blockDim.x = ecols * P threads (at most 256, so that a lane's rows and operands stay in
// registers): thread = column * P + part.
template <int R>
__global__ void __launch_bounds__(256)
retention_recurrence_kernel(const float* __restrict__ prep, int ldp, const float* __restrict__ v,
                            int ldv, const float* __restrict__ decay, float* __restrict__ state,
                            size_t state_stride, const int* __restrict__ cu_seqlens,
                            const int* __restrict__ seq_slot, int H, int d, int e, int P, int ecols,
                            float* __restrict__ o_raw, int write_state) {
  extern __shared__ __align__(16) float smem[];
  const int b = blockIdx.x, h = blockIdx.y;
  const int col0 = blockIdx.z * ecols;
  const int t0 = cu_seqlens[b], t1 = cu_seqlens[b + 1];
  const int part = threadIdx.x % P, jc = threadIdx.x / P;
  const int col = col0 + jc;
  const bool active = jc < ecols && col < e;
  const int slice = R + 4;                       // a lane's rows of q or k, padded
  float* sq = smem;                              // [chunk][P * slice]
  float* sk = sq + kRetChunk * P * slice;        // [chunk][P * slice]
  float* sv = sk + kRetChunk * P * slice;        // [chunk][ecols]
  float* so = sv + kRetChunk * ecols;            // [chunk][ecols]
  const float g = decay[h];
  float* M = state + (size_t)seq_slot[b] * state_stride + (size_t)h * d * e;
  float S[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int i = part * R + r;
    S[r] = (active && i < d) ? M[(size_t)i * e + col] : 0.f;
  }
  const int rows_padded = P * R;
  for (int c0 = t0; c0 < t1; c0 += kRetChunk) {
    const int nt = min(kRetChunk, t1 - c0);
    __syncthreads();                             // the chunk before has been read and written out
    for (int idx = threadIdx.x; idx < nt * rows_padded; idx += blockDim.x) {
      const int tt = idx / rows_padded, i = idx - tt * rows_padded;
      const int p = i / R, r = i - p * R;
      const float* row = prep + (size_t)(c0 + tt) * ldp + (size_t)h * d;
      sq[(tt * P + p) * slice + r] = i < d ? row[i] : 0.f;
      sk[(tt * P + p) * slice + r] = i < d ? row[(size_t)H * d + i] : 0.f;
    }
    for (int idx = threadIdx.x; idx < nt * ecols; idx += blockDim.x) {
      const int tt = idx / ecols, j = idx - tt * ecols;
      sv[idx] = col0 + j < e ? v[(size_t)(c0 + tt) * ldv + (size_t)h * e + col0 + j] : 0.f;
    }
    __syncthreads();
    {
      // every lane goes through the loop (the shuffles want whole warps); lanes beyond the
      // slice work on zeros and store nothing
      const int jv = jc < ecols ? jc : 0;
      for (int tt = 0; tt < nt; ++tt) {
        const float* q = sq + (tt * P + part) * slice;
        const float* k = sk + (tt * P + part) * slice;
        const float vt = sv[tt * ecols + jv];
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int r = 0; r < R; r += 4) {
          const float4 k4 = *reinterpret_cast<const float4*>(k + r);
          const float4 q4 = *reinterpret_cast<const float4*>(q + r);
          S[r] = fmaf(k4.x, vt, g * S[r]);
          S[r + 1] = fmaf(k4.y, vt, g * S[r + 1]);
          S[r + 2] = fmaf(k4.z, vt, g * S[r + 2]);
          S[r + 3] = fmaf(k4.w, vt, g * S[r + 3]);
          acc[0] = fmaf(S[r], q4.x, acc[0]);
          acc[1] = fmaf(S[r + 1], q4.y, acc[1]);
          acc[2] = fmaf(S[r + 2], q4.z, acc[2]);
          acc[3] = fmaf(S[r + 3], q4.w, acc[3]);
        }
        float o = (acc[0] + acc[1]) + (acc[2] + acc[3]);
        for (int off = P >> 1; off > 0; off >>= 1) o += __shfl_xor_sync(0xffffffffu, o, off);
        if (part == 0 && jc < ecols) so[tt * ecols + jc] = o;
      }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < nt * ecols; idx += blockDim.x) {
      const int tt = idx / ecols, j = idx - tt * ecols;
      if (col0 + j < e) o_raw[(size_t)(c0 + tt) * H * e + (size_t)h * e + col0 + j] = so[idx];
    }
  }
  if (write_state) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int i = part * R + r;
      if (active && i < d) M[(size_t)i * e + col] = S[r];
    }
  }
}

template <int R>
int launch_retention(const float* prep, int ldp, const float* v, int ldv, const float* decay,
                     float* state, size_t state_stride, const int* cu, const int* seq_slot, int B,
                     int H, int d, int e, int P, int ecols, float* o_raw, int write_state,
                     cudaStream_t st) {
  const int threads = ((ecols * P + 31) / 32) * 32;
  const size_t smem = sizeof(float) * kRetChunk * (2 * (size_t)P * (R + 4) + 2 * (size_t)ecols);
  auto kern = retention_recurrence_kernel<R>;
  if (smem > 48 * 1024) {
    if (smem > 200 * 1024) return kBadArgument;
    cudaError_t err =
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return (int)err;
  }
  const int slices = (e + ecols - 1) / ecols;
  if (H > 65535 || slices > 65535) return kBadArgument;
  kern<<<dim3(B, H, slices), threads, smem, st>>>(prep, ldp, v, ldv, decay, state, state_stride,
                                                  cu, seq_slot, H, d, e, P, ecols, o_raw,
                                                  write_state);
  return launch_status();
}
}  // namespace
}  // namespace cretif

using namespace cretif;

extern "C" int cretif_retention_prepare(const float* proj, int ldp, float* prep, int ldo,
                                        const float* cos_t, const float* sin_t, int pairing,
                                        int rot_dim, const int* tok_pos, int H, int d,
                                        float k_scale, int T, void* stream) {
  if (T <= 0) return kOk;
  if (H <= 0 || d <= 0 || rot_dim < 0 || rot_dim > d || (rot_dim & 1) || ldp < 2 * H * d ||
      ldo < 2 * H * d)
    return kBadArgument;
  if (rot_dim > 0 && (!cos_t || !sin_t)) return kBadArgument;
  retention_prepare_kernel<<<T, 256, 0, (cudaStream_t)stream>>>(
      proj, ldp, prep, ldo, cos_t, sin_t, pairing, rot_dim, tok_pos, H, d, k_scale);
  return launch_status();
}

extern "C" int cretif_retention_recurrence(const float* prep, int ldp, const float* v, int ldv,
                                           const float* decay, float* state,
                                           long long state_stride, const int* cu_seqlens,
                                           const int* seq_slot, int B, int H, int d, int e,
                                           float* o_raw, int write_state, int T, void* stream) {
  if (B <= 0 || T <= 0) return kOk;
  if (H <= 0 || d <= 0 || e <= 0 || !o_raw || ldp < 2 * H * d || ldv < H * e) return kBadArgument;
  static int sm_count = 0;
  if (!sm_count) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (sm_count <= 0) sm_count = 148;
  }
  // R rows a lane (a power of two from 4 to 32, about a quarter of d), P lanes a column
  int R = 4;
  while (R < 32 && R * 4 < d) R *= 2;
  int P = 1;
  while (P < 32 && P * R < d) P *= 2;
  if (P * R < d) return kBadArgument;            // d > 1024
  // columns a CTA: a head's columns are cut into slices while the (sequence, head) pairs alone
  // do not fill the chip twice over, down to two warps a CTA, and as far as 256 threads demand
  int ecols = e;
  while (ecols * P > 256) ecols = (ecols + 1) / 2;
  while ((long long)B * H * ((e + ecols - 1) / ecols) < 2LL * sm_count && ecols * P >= 128 &&
         ecols % 2 == 0)
    ecols /= 2;
  cudaStream_t st = (cudaStream_t)stream;
#define CRETIF_RET(RR)                                                                          \
  launch_retention<RR>(prep, ldp, v, ldv, decay, state, (size_t)state_stride, cu_seqlens,        \
                       seq_slot, B, H, d, e, P, ecols, o_raw, write_state, st)
  if (R == 4) return CRETIF_RET(4);
  if (R == 8) return CRETIF_RET(8);
  if (R == 16) return CRETIF_RET(16);
  return CRETIF_RET(32);
#undef CRETIF_RET
}
