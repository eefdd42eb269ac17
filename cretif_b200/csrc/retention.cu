// Retention: linear attention with a fixed decay per head, no softmax and no denominator.
//
// Per token and head, with state S [d, e] (32-bit, zero at a sequence's start):
//     S <- decay_h S + k v^T;   o = S^T q
// so the read-out sees the token's own write.  Any step shape is served (whole prompts, further
// chunks at a cached position, single tokens), all arithmetic in 32-bit; the recurrence has a
// token-by-token form and a form of 64 tokens at a time (further down):
//
// * retention_prepare (a CTA per token, or several where a step has few tokens): the first
//   rot_dim channels of every query and key head are rotated by the token's position (cos/sin
//   from a 32-bit table), the key is multiplied by k_scale after the rotation.
// * retention_recurrence (a CTA per (sequence, head, slice of columns)): the columns of S are
//   independent; a group of P lanes owns one column, each lane R contiguous rows of it in
//   registers.  Tokens go in chunks of 16 whose q, k and v are staged in shared memory (a
//   lane's slice of q and k padded so that the P slices fall into different banks); a token
//   costs one P-lane shuffle reduction and no barrier.  The read-outs leave in 32-bit through
//   shared memory, a chunk at a time.  The state is read once and written once per step.
// * retention_intra_kernel + retention_carry_kernel: the form of 64 tokens at a time.
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
  // (a step of few tokens spreads a token's columns over blockIdx.y: one round trip to memory
  // a thread instead of a chain of them)
  for (int idx = blockIdx.y * blockDim.x + threadIdx.x; idx < n; idx += blockDim.x * gridDim.y) {
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

// ---------------------------------------------------------------------------------------------
// The same recurrence, 64 tokens at a time.  With S0 the state before a chunk of n tokens and
// g the head's decay,
//     o_t = g^(t+1) S0^T q_t + sum_{s<=t} g^(t-s) (q_t . k_s) v_s        (t = 0 .. n-1)
//     S_n = g^n S0 + sum_s g^(n-1-s) k_s v_s^T
// which are matrix products instead of a chain of n dependent steps.  The powers of g come
// from a table (never a quotient of two powers, so a small g loses nothing).  All of it runs in
// 32-bit on the FMA pipe, with 16-byte shared-memory loads; rows of q, k and the scores are
// padded to 4 mod 8 floats so that eight rows' loads fall into eight different bank groups.
//
// * retention_intra_kernel (a CTA per (chunk, head); the chunks of all sequences at once): the
//   second term — the decayed, causally masked scores, then their product with v — written to
//   o_raw.  Nothing here depends on the state, so a long prompt fills the chip.
// * retention_carry_kernel (a CTA per (sequence, head, EC columns of S)) walks the sequence's
//   chunks with its slice of S in shared memory: adds the first term to o_raw, then updates S.
constexpr int kRcTokens = 64;
constexpr int kRcThreads = 256;
constexpr int kRcScoreLd = kRcTokens + 4;
constexpr int kRcSlab = 64;             // columns of v the intra kernel takes at a time

__device__ __forceinline__ void fma4(float4& a, float s, const float4& v) {
  a.x = fmaf(s, v.x, a.x);
  a.y = fmaf(s, v.y, a.y);
  a.z = fmaf(s, v.z, a.z);
  a.w = fmaf(s, v.w, a.w);
}
__device__ __forceinline__ float dot4(const float4& a, const float4& b, float acc) {
  acc = fmaf(a.x, b.x, acc);
  acc = fmaf(a.y, b.y, acc);
  acc = fmaf(a.z, b.z, acc);
  return fmaf(a.w, b.w, acc);
}

__device__ __forceinline__ void ret_cp16(float* dst, const float* src) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(a), "l"(src) : "memory");
}
__device__ __forceinline__ void ret_cp_commit() {
  asm volatile("cp.async.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void ret_cp_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__host__ __device__ inline int retention_chunk_ld(int d) {
  int ld = d;
  while ((ld & 7) != 4) ++ld;
  return ld;
}
inline size_t retention_intra_smem(int d) {
  return sizeof(float) * (2 * (size_t)kRcTokens * retention_chunk_ld(d) +
                          (size_t)kRcTokens * kRcSlab + (size_t)kRcTokens * kRcScoreLd +
                          kRcTokens + 4);
}
inline size_t retention_carry_smem(int d, int ec, int nbuf = 1) {
  return sizeof(float) * (nbuf * (2 * (size_t)kRcTokens * retention_chunk_ld(d) +
                                  (size_t)kRcTokens * ec) +
                          (size_t)d * ec + kRcTokens + 4);
}

__global__ void __launch_bounds__(kRcThreads)
retention_intra_kernel(const float* __restrict__ prep, int ldp, const float* __restrict__ v, int ldv,
                       const float* __restrict__ decay, const int* __restrict__ cu_seqlens, int B,
                       int H, int d, int e, float* __restrict__ o_raw) {
  extern __shared__ __align__(16) float smem[];
  constexpr int C = kRcTokens;
  constexpr int LP = kRcScoreLd;
  const int tid = threadIdx.x;
  const int h = blockIdx.y;
  // which sequence's which chunk: the grid has a CTA for every chunk there can be
  int left = blockIdx.x, c0 = -1, t1 = 0;
  for (int b = 0; b < B; ++b) {
    const int s0 = cu_seqlens[b], s1 = cu_seqlens[b + 1];
    const int chunks = (s1 - s0 + C - 1) / C;
    if (left < chunks) {
      c0 = s0 + left * C;
      t1 = s1;
      break;
    }
    left -= chunks;
  }
  if (c0 < 0) return;
  const int nt = min(C, t1 - c0);
  const int ldq = retention_chunk_ld(d);
  const int d4 = d >> 2;
  float* sQ = smem;                        // [C][ldq]
  float* sK = sQ + C * ldq;                // [C][ldq]
  float* sV = sK + C * ldq;                // [C][kRcSlab]
  float* sP = sV + C * kRcSlab;            // [C][LP]
  float* pw = sP + C * LP;                 // g^0 .. g^C
  if (tid <= C) pw[tid] = (float)pow((double)decay[h], (double)tid);
  const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
  // q and k of the chunk's tokens, copied asynchronously (all of a thread's copies are under
  // way at once).  Rows beyond the chunk's last token stay as they are: they reach only scores
  // of rows that are not stored, or of keys after the row, which are set to zero.
  for (int idx = tid; idx < nt * d4; idx += kRcThreads) {
    const int tt = idx / d4, i4 = idx - tt * d4;
    const float* row = prep + (size_t)(c0 + tt) * ldp + (size_t)h * d + 4 * i4;
    ret_cp16(sQ + tt * ldq + 4 * i4, row);
    ret_cp16(sK + tt * ldq + 4 * i4, row + (size_t)H * d);
  }
  ret_cp_commit();
  // a slab of v: rows beyond the last token and columns beyond the slab are zero (a zero score
  // times whatever lay there must stay zero)
  auto stage_v = [&](int j0, int width) {
    for (int idx = tid; idx < C * (kRcSlab / 4); idx += kRcThreads) {
      const int tt = idx >> 4, jg = idx & 15;
      float* dst = sV + tt * kRcSlab + 4 * jg;
      if (tt < nt && 4 * jg < width)
        ret_cp16(dst, v + (size_t)(c0 + tt) * ldv + (size_t)h * e + j0 + 4 * jg);
      else
        *reinterpret_cast<float4*>(dst) = zero4;
    }
    ret_cp_commit();
  };
  stage_v(0, min(kRcSlab, e));
  ret_cp_wait<1>();                        // q and k have arrived
  __syncthreads();
  const int ti = tid >> 4, si = tid & 15;
  {
    // scores: thread (ti, si) owns rows ti + 16 r and keys si + 16 c; key blocks ahead of the
    // row block are never computed
    float acc[4][4];
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[r][c] = 0.f;
    for (int kk = 0; kk < d; kk += 4) {
      float4 q4[4], k4[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        q4[r] = *reinterpret_cast<const float4*>(sQ + (ti + 16 * r) * ldq + kk);
        k4[r] = *reinterpret_cast<const float4*>(sK + (si + 16 * r) * ldq + kk);
      }
#pragma unroll
      for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int c = 0; c <= r; ++c) acc[r][c] = dot4(q4[r], k4[c], acc[r][c]);
    }
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int t = ti + 16 * r, s = si + 16 * c;
        sP[t * LP + s] = (c < r || (c == r && si <= ti)) ? acc[r][c] * pw[t - s] : 0.f;
      }
  }
  // scores times v, 64 columns at a time: rows ti + 16 r, columns 4 si .. 4 si + 3 of the slab
  for (int j0 = 0; j0 < e; j0 += kRcSlab) {
    const int width = min(kRcSlab, e - j0);            // a multiple of 4
    if (j0 > 0) {
      __syncthreads();                                 // the slab before has been read
      stage_v(j0, width);
    }
    ret_cp_wait<0>();
    __syncthreads();                                   // the slab and the scores are in place
    if (4 * si >= width) continue;
    float4 acc[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) acc[r] = zero4;
    const int smax = min(nt, ti + 49);
    for (int s = 0; s < smax; s += 4) {
      const float4 v0 = *reinterpret_cast<const float4*>(sV + (s + 0) * kRcSlab + 4 * si);
      const float4 v1 = *reinterpret_cast<const float4*>(sV + (s + 1) * kRcSlab + 4 * si);
      const float4 v2 = *reinterpret_cast<const float4*>(sV + (s + 2) * kRcSlab + 4 * si);
      const float4 v3 = *reinterpret_cast<const float4*>(sV + (s + 3) * kRcSlab + 4 * si);
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        if (s > ti + 16 * r) continue;                 // keys after the row: the scores are zero
        const float4 p = *reinterpret_cast<const float4*>(sP + (ti + 16 * r) * LP + s);
        fma4(acc[r], p.x, v0);
        fma4(acc[r], p.y, v1);
        fma4(acc[r], p.z, v2);
        fma4(acc[r], p.w, v3);
      }
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int t = ti + 16 * r;
      if (t < nt)
        *reinterpret_cast<float4*>(o_raw + (size_t)(c0 + t) * H * e + (size_t)h * e + j0 + 4 * si) =
            acc[r];
    }
  }
}

// Two buffers for q, k and v where they fit (nbuf = 2): a chunk's copies are under way while
// the chunk before is computed.
template <int EC>
__global__ void __launch_bounds__(kRcThreads)
retention_carry_kernel(const float* __restrict__ prep, int ldp, const float* __restrict__ v, int ldv,
                       const float* __restrict__ decay, float* __restrict__ state,
                       size_t state_stride, const int* __restrict__ cu_seqlens,
                       const int* __restrict__ seq_slot, int H, int d, int e,
                       float* __restrict__ o_raw, int write_state, int nbuf) {
  extern __shared__ __align__(16) float smem[];
  constexpr int C = kRcTokens;
  constexpr int CG = EC / 4;               // groups of four columns
  constexpr int NR = kRcThreads / CG;      // threads along the rows
  constexpr int RT = C / NR;               // read-out rows a thread
  const int tid = threadIdx.x;
  const int b = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * EC;
  const int t0 = cu_seqlens[b], t1 = cu_seqlens[b + 1];
  if (t1 <= t0) return;
  const int ldq = retention_chunk_ld(d);
  const int d4 = d >> 2;
  const int buf_floats = 2 * C * ldq + C * EC;   // q [C][ldq] | k [C][ldq] | v [C][EC]
  float* sS = smem + nbuf * buf_floats;    // [d][EC]
  float* pw = sS + d * EC;                 // g^0 .. g^C
  if (tid <= C) pw[tid] = (float)pow((double)decay[h], (double)tid);
  float* M = state + (size_t)seq_slot[b] * state_stride + (size_t)h * d * e + col0;
  for (int idx = tid; idx < d * CG; idx += kRcThreads) {
    const int i = idx / CG, jg = idx - i * CG;
    *reinterpret_cast<float4*>(sS + i * EC + 4 * jg) =
        *reinterpret_cast<const float4*>(M + (size_t)i * e + 4 * jg);
  }
  const int tj = tid % CG, tr = tid / CG;
  const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
  // Rows beyond a chunk's last token are not copied: of q they reach only read-outs that are
  // not stored, of k and v nothing (the update stops at the last token).
  auto stage = [&](int c0, float* buf) {
    const int nt = min(C, t1 - c0);
    for (int idx = tid; idx < nt * d4; idx += kRcThreads) {
      const int tt = idx / d4, i4 = idx - tt * d4;
      const float* row = prep + (size_t)(c0 + tt) * ldp + (size_t)h * d + 4 * i4;
      ret_cp16(buf + tt * ldq + 4 * i4, row);
      ret_cp16(buf + C * ldq + tt * ldq + 4 * i4, row + (size_t)H * d);
    }
    for (int idx = tid; idx < nt * CG; idx += kRcThreads) {
      const int tt = idx / CG, jg = idx - tt * CG;
      ret_cp16(buf + 2 * C * ldq + tt * EC + 4 * jg,
               v + (size_t)(c0 + tt) * ldv + (size_t)h * e + col0 + 4 * jg);
    }
    ret_cp_commit();
  };
  stage(t0, smem);
  __syncthreads();                         // the table of powers is read before the loop's barrier
  int turn = 0;
  for (int c0 = t0; c0 < t1; c0 += C, ++turn) {
    const int nt = min(C, t1 - c0);
    const bool last = c0 + C >= t1;
    float* sQ = smem + (nbuf == 2 ? (turn & 1) * buf_floats : 0);
    float* sK = sQ + C * ldq;
    float* sV = sK + C * ldq;
    ret_cp_wait<0>();
    // v takes the weight g^(n-1-s) it has in the state's update (each thread the pieces it
    // copied itself; the read-out does not use v)
    for (int idx = tid; idx < nt * CG; idx += kRcThreads) {
      const int tt = idx / CG, jg = idx - tt * CG;
      const float w = pw[nt - 1 - tt];
      float4 v4 = *reinterpret_cast<float4*>(sV + tt * EC + 4 * jg);
      v4.x *= w; v4.y *= w; v4.z *= w; v4.w *= w;
      *reinterpret_cast<float4*>(sV + tt * EC + 4 * jg) = v4;
    }
    __syncthreads();                       // the chunk is in place; the chunk before is done
    if (nbuf == 2 && !last) stage(c0 + C, smem + ((turn + 1) & 1) * buf_floats);
    {
      // what the state before the chunk gives every row: rows tr + NR r, columns 4 tj .. + 3
      float4 acc[RT], old[RT];
#pragma unroll
      for (int r = 0; r < RT; ++r) {
        acc[r] = zero4;
        const int t = tr + NR * r;
        old[r] = t < nt ? __ldcg(reinterpret_cast<const float4*>(
                              o_raw + (size_t)(c0 + t) * H * e + (size_t)h * e + col0 + 4 * tj))
                        : zero4;
      }
#pragma unroll 2
      for (int i = 0; i < d; i += 4) {
        const float4 s0 = *reinterpret_cast<const float4*>(sS + (i + 0) * EC + 4 * tj);
        const float4 s1 = *reinterpret_cast<const float4*>(sS + (i + 1) * EC + 4 * tj);
        const float4 s2 = *reinterpret_cast<const float4*>(sS + (i + 2) * EC + 4 * tj);
        const float4 s3 = *reinterpret_cast<const float4*>(sS + (i + 3) * EC + 4 * tj);
#pragma unroll
        for (int r = 0; r < RT; ++r) {
          const float4 q = *reinterpret_cast<const float4*>(sQ + (tr + NR * r) * ldq + i);
          fma4(acc[r], q.x, s0);
          fma4(acc[r], q.y, s1);
          fma4(acc[r], q.z, s2);
          fma4(acc[r], q.w, s3);
        }
      }
#pragma unroll
      for (int r = 0; r < RT; ++r) {
        const int t = tr + NR * r;
        if (t < nt) {
          const float w = pw[t + 1];
          float4 o = old[r];
          o.x = fmaf(w, acc[r].x, o.x);
          o.y = fmaf(w, acc[r].y, o.y);
          o.z = fmaf(w, acc[r].z, o.z);
          o.w = fmaf(w, acc[r].w, o.w);
          *reinterpret_cast<float4*>(o_raw + (size_t)(c0 + t) * H * e + (size_t)h * e + col0 +
                                     4 * tj) = o;
        }
      }
    }
    if (last && !write_state) break;       // nobody reads the state after the last chunk
    __syncthreads();                       // everybody has read the old state
    {
      const float gn = pw[nt];
      for (int ig = tr; ig < d4; ig += NR) {
        float* srow = sS + (4 * ig) * EC + 4 * tj;
        float4 a0 = *reinterpret_cast<float4*>(srow);
        float4 a1 = *reinterpret_cast<float4*>(srow + EC);
        float4 a2 = *reinterpret_cast<float4*>(srow + 2 * EC);
        float4 a3 = *reinterpret_cast<float4*>(srow + 3 * EC);
        a0.x *= gn; a0.y *= gn; a0.z *= gn; a0.w *= gn;
        a1.x *= gn; a1.y *= gn; a1.z *= gn; a1.w *= gn;
        a2.x *= gn; a2.y *= gn; a2.z *= gn; a2.w *= gn;
        a3.x *= gn; a3.y *= gn; a3.z *= gn; a3.w *= gn;
#pragma unroll 4
        for (int s = 0; s < nt; ++s) {
          const float4 k4 = *reinterpret_cast<const float4*>(sK + s * ldq + 4 * ig);
          const float4 v4 = *reinterpret_cast<const float4*>(sV + s * EC + 4 * tj);
          fma4(a0, k4.x, v4);
          fma4(a1, k4.y, v4);
          fma4(a2, k4.z, v4);
          fma4(a3, k4.w, v4);
        }
        *reinterpret_cast<float4*>(srow) = a0;
        *reinterpret_cast<float4*>(srow + EC) = a1;
        *reinterpret_cast<float4*>(srow + 2 * EC) = a2;
        *reinterpret_cast<float4*>(srow + 3 * EC) = a3;
      }
    }
    if (nbuf != 2 && !last) {
      __syncthreads();                     // the one buffer has been read
      stage(c0 + C, smem);
    }
  }
  if (write_state) {
    __syncthreads();
    for (int idx = tid; idx < d * CG; idx += kRcThreads) {
      const int i = idx / CG, jg = idx - i * CG;
      *reinterpret_cast<float4*>(M + (size_t)i * e + 4 * jg) =
          *reinterpret_cast<const float4*>(sS + i * EC + 4 * jg);
    }
  }
}

template <int EC>
int launch_retention_carry(const float* prep, int ldp, const float* v, int ldv, const float* decay,
                           float* state, size_t state_stride, const int* cu, const int* seq_slot,
                           int B, int H, int d, int e, float* o_raw, int write_state,
                           cudaStream_t st) {
  const int nbuf = retention_carry_smem(d, EC, 2) <= 220 * 1024 ? 2 : 1;
  const size_t smem = retention_carry_smem(d, EC, nbuf);
  auto kern = retention_carry_kernel<EC>;
  if (smem > 48 * 1024) {
    cudaError_t err =
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return (int)err;
  }
  kern<<<dim3(B, H, e / EC), kRcThreads, smem, st>>>(prep, ldp, v, ldv, decay, state, state_stride,
                                                     cu, seq_slot, H, d, e, o_raw, write_state,
                                                     nbuf);
  return launch_status();
}

int launch_retention_intra(const float* prep, int ldp, const float* v, int ldv, const float* decay,
                           const int* cu, int B, int T, int H, int d, int e, float* o_raw,
                           cudaStream_t st) {
  const size_t smem = retention_intra_smem(d);
  if (smem > 48 * 1024) {
    cudaError_t err = cudaFuncSetAttribute(
        retention_intra_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return (int)err;
  }
  // every sequence has at most one chunk that is not full
  const long long chunks = (long long)T / kRcTokens + B;
  if (chunks > 0x7fffffffLL) return kBadArgument;
  retention_intra_kernel<<<dim3((unsigned)chunks, H), kRcThreads, smem, st>>>(
      prep, ldp, v, ldv, decay, cu, B, H, d, e, o_raw);
  return launch_status();
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
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
  const int per_token = T < 64 ? (2 * H * d + 255) / 256 : 1;
  retention_prepare_kernel<<<dim3(T, per_token > 65535 ? 65535 : per_token), 256, 0,
                             (cudaStream_t)stream>>>(
      proj, ldp, prep, ldo, cos_t, sin_t, pairing, rot_dim, tok_pos, H, d, k_scale);
  return launch_status();
}

extern "C" int cretif_retention_recurrence(const float* prep, int ldp, const float* v, int ldv,
                                           const float* decay, float* state,
                                           long long state_stride, const int* cu_seqlens,
                                           const int* seq_slot, int B, int H, int d, int e,
                                           float* o_raw, int write_state, int T, int form,
                                           void* stream) {
  if (B <= 0 || T <= 0) return kOk;
  if (H <= 0 || d <= 0 || e <= 0 || !o_raw || ldp < 2 * H * d || ldv < H * e) return kBadArgument;
  if (form < 0 || form > 2) return kBadArgument;
  static int sm_count = 0;
  if (!sm_count) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (sm_count <= 0) sm_count = 148;
  }
  cudaStream_t st = (cudaStream_t)stream;
  // 64 tokens at a time where the step brings a sequence 16 tokens or more on average and the
  // sizes allow 16-byte accesses throughout; token by token otherwise.
  if (form == 2 || (form == 0 && (long long)T >= 16LL * B)) {
    const bool fits = d % 4 == 0 && e % 16 == 0 && ldp % 4 == 0 && ldv % 4 == 0 &&
                      state_stride % 4 == 0 && aligned16(prep) && aligned16(v) &&
                      aligned16(state) && aligned16(o_raw) && H <= 65535 &&
                      retention_carry_smem(d, 16) <= 220 * 1024 &&
                      retention_intra_smem(d) <= 220 * 1024;
    if (fits) {
      int rc = launch_retention_intra(prep, ldp, v, ldv, decay, cu_seqlens, B, T, H, d, e, o_raw,
                                      st);
      if (rc != kOk) return rc;
      // columns a CTA: as many as divide e and fit, fewer while the chip is not filled
      int ec = e % 64 == 0 ? 64 : e % 32 == 0 ? 32 : 16;
      while (ec > 16 && (retention_carry_smem(d, ec) > 220 * 1024 ||
                         (long long)B * H * (e / ec) < (long long)sm_count))
        ec /= 2;
#define CRETIF_RETC(EC)                                                                        \
  launch_retention_carry<EC>(prep, ldp, v, ldv, decay, state, (size_t)state_stride, cu_seqlens, \
                             seq_slot, B, H, d, e, o_raw, write_state, st)
      if (ec == 64) return CRETIF_RETC(64);
      if (ec == 32) return CRETIF_RETC(32);
      return CRETIF_RETC(16);
#undef CRETIF_RETC
    }
    if (form == 2) return kBadArgument;
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
#define CRETIF_RET(RR)                                                                          \
  launch_retention<RR>(prep, ldp, v, ldv, decay, state, (size_t)state_stride, cu_seqlens,        \
                       seq_slot, B, H, d, e, P, ecols, o_raw, write_state, st)
  if (R == 4) return CRETIF_RET(4);
  if (R == 8) return CRETIF_RET(8);
  if (R == 16) return CRETIF_RET(16);
  return CRETIF_RET(32);
#undef CRETIF_RET
}
