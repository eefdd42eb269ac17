// Per-head work around an attention whose projections are normed head by head: bias, RMS norm
// of every query and key head with a weight shared by the heads, rotation of the first
// rot_dim channels of a head, the write into the block cache -- one kernel, 32-bit inside --
// and the per-head output gate.  Also the small row kernels of ungated feed-forwards and
// capped logits.
//
// headnorm_rope_kv_append: proj rows [q (nh hd) | k (nkv hd) | v (nkv vd) | ...] in float32 or
// bfloat16.  Per token and head (a warp each; a head's channels stay in the lanes' registers):
//   x = proj + bias                                    (bias may be null)
//   q, k:  x <- x / sqrt(mean(x^2) + eps) * w          (w of hd numbers, null: no norm)
//   q, k:  channels (i, partner(i)) of the first rot_dim are rotated by pos * f_j
//          (pairing 0: partner i + rot_dim/2; 1: i ^ 1), cos/sin from a 32-bit table
//   q -> q_out, k -> key cache, v -> value cache at the token's position.
#include "api.h"
#include "common.cuh"

namespace cretif {

namespace {
constexpr int kHnWarps = 8;
constexpr int kHnMaxD = 512;

template <typename TI, typename T, int NCH>
__global__ void __launch_bounds__(kHnWarps * 32)
headnorm_rope_kv_append_kernel(const TI* __restrict__ proj, int ldp,
                               const float* __restrict__ bias, const float* __restrict__ wq,
                               const float* __restrict__ wk, float eps,
                               const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                               int pairing, int rot_dim, const int* __restrict__ tok_pos,
                               const int* __restrict__ tok_seq, const int* __restrict__ seq_slot,
                               int nh, int nkv, int hd, int vd, T* __restrict__ q_out, int ldq,
                               const int* __restrict__ table, int table_stride,
                               T* __restrict__ kc, T* __restrict__ vc, int bt, int write_cache,
                               unsigned int* __restrict__ fault) {
  __shared__ float normed[kHnWarps][kHnMaxD];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const int units = nh + 2 * nkv;
  const int pos = tok_pos[t];
  const TI* row = proj + (size_t)t * ldp;
  int blk = -1;
  if (write_cache) {
    const int slot = seq_slot[tok_seq[t]];
    blk = table[(size_t)slot * table_stride + pos / bt];
    if (blk < 0 && threadIdx.x == 0 && blockIdx.y == 0) atomicOr(fault, kFaultBlockTable);
  }
  const int half = rot_dim >> 1;
  const float* c = cos_t + (size_t)pos * half;
  const float* s = sin_t + (size_t)pos * half;
  float* mine = normed[warp];
  for (int unit = blockIdx.y * kHnWarps + warp; unit < units; unit += gridDim.y * kHnWarps) {
    const bool is_q = unit < nh, is_k = !is_q && unit < nh + nkv;
    const int n = (is_q || is_k) ? hd : vd;
    const int c0 = is_q ? unit * hd : is_k ? nh * hd + (unit - nh) * hd
                                           : (nh + nkv) * hd + (unit - nh - nkv) * vd;
    T* dst;
    if (is_q) {
      dst = q_out + (size_t)t * ldq + (size_t)unit * hd;
    } else {
      if (blk < 0) continue;
      const int kvh = is_k ? unit - nh : unit - nh - nkv;
      dst = (is_k ? kc : vc) + (((size_t)blk * nkv + kvh) * bt + (pos % bt)) * n;
    }
    float val[NCH];
    float ss = 0.f;
#pragma unroll
    for (int m = 0; m < NCH; ++m) {
      const int i = lane + 32 * m;
      val[m] = i < n ? to_float(row[c0 + i]) + (bias ? bias[c0 + i] : 0.f) : 0.f;
      ss += val[m] * val[m];
    }
    const float* w = is_q ? wq : wk;
    if (!is_q && !is_k) {
#pragma unroll
      for (int m = 0; m < NCH; ++m) {
        const int i = lane + 32 * m;
        if (i < n) dst[i] = from_float<T>(val[m]);
      }
      continue;
    }
    if (w) {
      ss = warp_sum(ss);
      const float f = 1.0f / sqrtf(ss / (float)hd + eps);
#pragma unroll
      for (int m = 0; m < NCH; ++m) {
        const int i = lane + 32 * m;
        if (i < n) val[m] = val[m] * f * w[i];
      }
    }
    if (rot_dim > 0) {
      __syncwarp();
#pragma unroll
      for (int m = 0; m < NCH; ++m) {
        const int i = lane + 32 * m;
        if (i < n) mine[i] = val[m];
      }
      __syncwarp();
#pragma unroll
      for (int m = 0; m < NCH; ++m) {
        const int i = lane + 32 * m;
        if (i < rot_dim) {
          const bool first = pairing ? !(i & 1) : i < half;
          const int j = pairing ? i >> 1 : (first ? i : i - half);
          const int partner = pairing ? i ^ 1 : (first ? i + half : i - half);
          const float other = mine[partner];
          // the pair (u, v) becomes (u cos - v sin, v cos + u sin)
          val[m] = first ? val[m] * c[j] - other * s[j] : val[m] * c[j] + other * s[j];
        }
      }
    }
#pragma unroll
    for (int m = 0; m < NCH; ++m) {
      const int i = lane + 32 * m;
      if (i < n) dst[i] = from_float<T>(val[m]);
    }
  }
}

// o[t, h, :] *= sigmoid(g[t, h]): a gate per head from a float32 column of the projections.
template <typename T>
__global__ void gate_heads_kernel(T* __restrict__ o, int ldo, const float* __restrict__ g, int ldg,
                                  int nh, int vd, long long total) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int w = nh * vd;
  const long long t = idx / w;
  const int col = (int)(idx - t * w);
  const float z = g[(size_t)t * ldg + col / vd];
  const float gate = 1.0f / (1.0f + expf(-z));
  T* p = o + (size_t)t * ldo + col;
  *p = from_float<T>(to_float(*p) * gate);
}

// The same for bfloat16 rows whose heads are whole groups of eight channels: a thread takes 16
// bytes of a head.
__global__ void gate_heads8_kernel(__nv_bfloat16* __restrict__ o, int ldo,
                                   const float* __restrict__ g, int ldg, int nh, int vd,
                                   long long groups) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= groups) return;
  const int per_row = nh * vd / 8;
  const long long t = idx / per_row;
  const int col = (int)(idx - t * per_row) * 8;
  const float z = g[(size_t)t * ldg + col / vd];
  const float gate = 1.0f / (1.0f + expf(-z));
  uint4* p = reinterpret_cast<uint4*>(o + (size_t)t * ldo + col);
  uint4 raw = *p;
  __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 f = __bfloat1622float2(h2[e]);
    h2[e] = __floats2bfloat162_rn(f.x * gate, f.y * gate);
  }
  *p = raw;
}

// A gate per channel (value size 1: every column is a head of its own), bfloat16 rows: a thread
// takes eight channels and their eight gates.
__global__ void gate_channels8_kernel(__nv_bfloat16* __restrict__ o, int ldo,
                                      const float* __restrict__ g, int ldg, int width,
                                      long long groups) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= groups) return;
  const int per_row = width / 8;
  const long long t = idx / per_row;
  const int col = (int)(idx - t * per_row) * 8;
  const float* gp = g + (size_t)t * ldg + col;
  uint4* p = reinterpret_cast<uint4*>(o + (size_t)t * ldo + col);
  uint4 raw = *p;
  __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 f = __bfloat1622float2(h2[e]);
    h2[e] = __floats2bfloat162_rn(f.x / (1.0f + expf(-gp[2 * e])),
                                  f.y / (1.0f + expf(-gp[2 * e + 1])));
  }
  *p = raw;
}

template <typename TI, typename TO>
__global__ void activation_kernel(const TI* __restrict__ in, int ldi, TO* __restrict__ out, int ldo,
                                  int width, long long total, int kind) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const long long t = idx / width;
  const int col = (int)(idx - t * width);
  out[(size_t)t * ldo + col] = from_float<TO>(unary_activation(to_float(in[(size_t)t * ldi + col]), kind));
}

// z <- cap * tanh(z / cap), in place, 32-bit.
__global__ void softcap_kernel(float* __restrict__ z, long long total, float cap) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx < total) z[idx] = cap * tanhf(z[idx] / cap);
}

// h += alpha * y, 32-bit (y float32 or bfloat16).
template <typename TY>
__global__ void axpy_rows_kernel(float* __restrict__ h, const TY* __restrict__ y, float alpha,
                                 long long total) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx < total) h[idx] = fmaf(alpha, to_float(y[idx]), h[idx]);
}
}  // namespace
}  // namespace cretif

using namespace cretif;

extern "C" int cretif_headnorm_rope_kv_append(
    const void* proj, int ldp, int proj_dt, const float* bias, const float* wq, const float* wk,
    float eps, const float* cos_t, const float* sin_t, int pairing, int rot_dim,
    const int* tok_pos, const int* tok_seq, const int* seq_slot, int nh, int nkv, int hd, int vd,
    void* q_out, int ldq, int dt, const int* table, int table_stride, void* kc, void* vc, int bt,
    int write_cache, int T, unsigned int* fault, void* stream) {
  if (T <= 0) return kOk;
  if (nh <= 0 || nkv < 0 || hd <= 0 || hd > kHnMaxD || vd <= 0 || vd > kHnMaxD || ldq < nh * hd ||
      rot_dim < 0 || rot_dim > hd || (rot_dim & 1) || (!wq) != (!wk))
    return kBadArgument;
  if (rot_dim > 0 && (!cos_t || !sin_t)) return kBadArgument;
  if (write_cache && (bt <= 0 || !kc || !vc || !table || !tok_seq || !seq_slot)) return kBadArgument;
  if (ldp < (nh + nkv) * hd + nkv * vd) return kBadArgument;
  if (!write_cache) nkv = 0;                     // nothing to store: only the queries are made
  const int units = nh + 2 * nkv;
  dim3 grid(T, T >= 256 ? 1 : (units + kHnWarps - 1) / kHnWarps);
  if (grid.y > 65535) return kBadArgument;
  cudaStream_t st = (cudaStream_t)stream;
  const int widest = vd > hd ? vd : hd;
#define CRETIF_HN(TI, TT, NCH)                                                                   \
  headnorm_rope_kv_append_kernel<TI, TT, NCH><<<grid, kHnWarps * 32, 0, st>>>(                    \
      (const TI*)proj, ldp, bias, wq, wk, eps, cos_t, sin_t, pairing, rot_dim, tok_pos, tok_seq,  \
      seq_slot, nh, nkv, hd, vd, (TT*)q_out, ldq, table, table_stride, (TT*)kc, (TT*)vc, bt,      \
      write_cache, fault)
#define CRETIF_HN_T(TI, TT)                                                                      \
  do {                                                                                           \
    if (widest <= 64) CRETIF_HN(TI, TT, 2);                                                       \
    else if (widest <= 128) CRETIF_HN(TI, TT, 4);                                                 \
    else if (widest <= 256) CRETIF_HN(TI, TT, 8);                                                 \
    else CRETIF_HN(TI, TT, 16);                                                                   \
  } while (0)
  if (proj_dt == kF32 && dt == kF32)
    CRETIF_HN_T(float, float);
  else if (proj_dt == kF32 && dt == kBF16)
    CRETIF_HN_T(float, __nv_bfloat16);
  else if (proj_dt == kBF16 && dt == kBF16)
    CRETIF_HN_T(__nv_bfloat16, __nv_bfloat16);
  else
    return kBadDType;
#undef CRETIF_HN_T
#undef CRETIF_HN
  return launch_status();
}

extern "C" int cretif_gate_heads(void* o, int ldo, int dt, const float* g, int ldg, int nh, int vd,
                                 int T, void* stream) {
  if (T <= 0) return kOk;
  if (nh <= 0 || vd <= 0 || ldo < nh * vd || ldg < nh) return kBadArgument;
  const long long total = (long long)T * nh * vd;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  cudaStream_t st = (cudaStream_t)stream;
  if (dt == kF32)
    gate_heads_kernel<float><<<blocks, 256, 0, st>>>((float*)o, ldo, g, ldg, nh, vd, total);
  else if (dt == kBF16 && vd == 1 && nh % 8 == 0 && ldo % 8 == 0 && ((uintptr_t)o & 15) == 0)
    gate_channels8_kernel<<<(unsigned)((total / 8 + 255) / 256), 256, 0, st>>>(
        (__nv_bfloat16*)o, ldo, g, ldg, nh, total / 8);
  else if (dt == kBF16 && vd % 8 == 0 && ldo % 8 == 0 && ((uintptr_t)o & 15) == 0)
    gate_heads8_kernel<<<(unsigned)((total / 8 + 255) / 256), 256, 0, st>>>(
        (__nv_bfloat16*)o, ldo, g, ldg, nh, vd, total / 8);
  else if (dt == kBF16)
    gate_heads_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>((__nv_bfloat16*)o, ldo, g, ldg, nh,
                                                            vd, total);
  else
    return kBadDType;
  return launch_status();
}

extern "C" int cretif_activation(const void* in, int ldi, int in_dt, void* out, int ldo, int out_dt,
                                 int T, int width, int kind, void* stream) {
  if (T <= 0 || width <= 0) return kOk;
  if (ldi < width || ldo < width || kind < 0 || kind >= kUnaryKinds) return kBadArgument;
  const long long total = (long long)T * width;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  cudaStream_t st = (cudaStream_t)stream;
  if (in_dt == kF32 && out_dt == kF32)
    activation_kernel<float, float><<<blocks, 256, 0, st>>>((const float*)in, ldi, (float*)out,
                                                            ldo, width, total, kind);
  else if (in_dt == kF32 && out_dt == kBF16)
    activation_kernel<float, __nv_bfloat16><<<blocks, 256, 0, st>>>(
        (const float*)in, ldi, (__nv_bfloat16*)out, ldo, width, total, kind);
  else if (in_dt == kBF16 && out_dt == kBF16)
    activation_kernel<__nv_bfloat16, __nv_bfloat16><<<blocks, 256, 0, st>>>(
        (const __nv_bfloat16*)in, ldi, (__nv_bfloat16*)out, ldo, width, total, kind);
  else
    return kBadDType;
  return launch_status();
}

extern "C" int cretif_softcap(float* z, long long total, float cap, void* stream) {
  if (total <= 0) return kOk;
  if (!(cap > 0.f)) return kBadArgument;
  softcap_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(z, total, cap);
  return launch_status();
}

extern "C" int cretif_axpy_rows(float* h, const void* y, int y_dt, float alpha, long long total,
                                void* stream) {
  if (total <= 0) return kOk;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  cudaStream_t st = (cudaStream_t)stream;
  if (y_dt == kF32)
    axpy_rows_kernel<float><<<blocks, 256, 0, st>>>(h, (const float*)y, alpha, total);
  else if (y_dt == kBF16)
    axpy_rows_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(h, (const __nv_bfloat16*)y, alpha,
                                                           total);
  else
    return kBadDType;
  return launch_status();
}
