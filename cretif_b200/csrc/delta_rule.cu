// The gated delta rule: a matrix-valued recurrence per head, behind short causal convolutions.
//
// Per token and head, with state M [d, e] (32-bit, zero at a sequence's start):
//     M <- g M;   u = beta (v - M^T k);   M <- M + k u^T;   o = M^T q
// so the read-out sees the token's own write.  Three kernels serve any step shape (whole
// prompts, further chunks at a cached position, single tokens), all arithmetic in 32-bit:
//
// * delta_prepare (a warp per head of a token): the causal convolution over time of the projected q, k
//   and v channels (taps from this step's rows, or from the sequence's saved last inputs where
//   the window reaches back before the step), SiLU, unit length per q/k head (and the query's
//   d^-1/2), beta = sigmoid(.), g = exp(-exp(A_log) softplus(. + dt_bias)).
// * delta_recurrence (a CTA per (sequence, head, slice of columns)): the columns of M are
//   independent, so the launcher cuts a head's columns into slices while the chip is not full,
//   and within a CTA a group of P lanes owns one column, each lane a contiguous slice of its d rows in registers
//   (the token's key and query slices come from shared memory in 16-byte pieces); a token
//   costs two P-lane shuffle reductions and no barrier.  Tokens go in chunks of 16 whose
//   operands arrive in shared memory by asynchronous copies a chunk ahead (two stages).  The
//   read-outs leave in 32-bit; delta_out_norm (a warp per token and head) norms them over e
//   (RMS, weight, times SiLU of the gate).  The state is read once and written
//   once per step.
// * delta_conv_state (a thread per channel): the last taps-1 inputs of every channel, for the
//   next step.
#include "api.h"
#include "common.cuh"

namespace cretif {

__device__ __forceinline__ float silu_f32(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f32(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// proj row: [q (G d) | k (G d) | v (H e) | gate (H e) | b (H) | a (H)]
// prep row: [q (G d) | k (G d) | v (H e) | beta (H) | g (H)]
// A warp per unit of a token's work: one of the 2G query/key heads (its d channels stay in the
// lanes' registers between the convolution and the scaling to unit length, d <= 256), one of the
// H value heads, or the token's H pairs of gates.  gridDim.y CTAs of eight warps share a token,
// so that a step of one token is still a few dozen warps with all their loads in flight.
constexpr int kPrepWarps = 8;
constexpr int kPrepMaxD = 256;

__global__ void __launch_bounds__(kPrepWarps * 32)
delta_prepare_kernel(const float* __restrict__ proj, int ldp, float* __restrict__ prep, int ldo,
                     const float* __restrict__ conv_w, int taps,
                     const float* __restrict__ conv_state, size_t state_stride,
                     const float* __restrict__ a_log, const float* __restrict__ dt_bias,
                     const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                     const int* __restrict__ seq_slot, const int* __restrict__ seq_start, int H,
                     int G, int d, int e, float unit_eps) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const int unit = blockIdx.y * kPrepWarps + warp;
  if (unit >= 2 * G + H + 1) return;
  const int b = tok_seq[t];
  const int lt = tok_pos[t] - seq_start[b];      // tokens of this sequence before t in the step
  const int C = 2 * G * d + H * e;
  const float* st = conv_state + (size_t)seq_slot[b] * state_stride;
  const float* row = proj + (size_t)t * ldp;
  float* out = prep + (size_t)t * ldo;
  auto conv = [&](int c) {                        // the convolution over time and SiLU
    float acc = 0.f;
#pragma unroll 4
    for (int i = 0; i < taps; ++i) {              // i tokens back
      const float w = conv_w[(size_t)c * taps + (taps - 1 - i)];
      const float z = i <= lt ? row[c - (ptrdiff_t)i * ldp]
                              : st[(size_t)c * (taps - 1) + (taps - 1) - (i - lt)];
      acc = fmaf(w, z, acc);
    }
    return silu_f32(acc);
  };
  if (unit < 2 * G) {                             // a query head (unit < G) or a key head
    const int c0 = unit * d;
    float val[kPrepMaxD / 32];
    float ss = 0.f;
#pragma unroll
    for (int m = 0; m < kPrepMaxD / 32; ++m) {
      const int i = lane + 32 * m;
      val[m] = i < d ? conv(c0 + i) : 0.f;
      ss += val[m] * val[m];
    }
    ss = warp_sum(ss);
    float f = 1.0f / sqrtf(ss + unit_eps);
    if (unit < G) f *= 1.0f / sqrtf((float)d);
#pragma unroll
    for (int m = 0; m < kPrepMaxD / 32; ++m) {
      const int i = lane + 32 * m;
      if (i < d) out[c0 + i] = val[m] * f;
    }
  } else if (unit < 2 * G + H) {                  // a value head
    const int c0 = 2 * G * d + (unit - 2 * G) * e;
#pragma unroll 4
    for (int i = lane; i < e; i += 32) out[c0 + i] = conv(c0 + i);
  } else {                                        // the gates
    for (int h = lane; h < H; h += 32) {
      const float bz = row[C + H * e + h], az = row[C + H * e + H + h];
      out[C + h] = 1.0f / (1.0f + expf(-bz));
      out[C + H + h] = expf(-expf(a_log[h]) * softplus_f32(az + dt_bias[h]));
    }
  }
}

// A thread per channel: the last taps-1 inputs after this step.
__global__ void delta_conv_state_kernel(const float* __restrict__ proj, int ldp,
                                        float* __restrict__ conv_state, size_t state_stride,
                                        int taps, int C, const int* __restrict__ cu_seqlens,
                                        const int* __restrict__ seq_slot) {
  const int b = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int t0 = cu_seqlens[b], n = cu_seqlens[b + 1] - t0;
  const int keep = taps - 1;
  float* s = conv_state + (size_t)seq_slot[b] * state_stride + (size_t)c * keep;
  for (int j = 0; j < keep; ++j) {               // ascending: reads run ahead of writes
    const int back = keep - j;                   // this entry is `back` tokens before the next
    s[j] = back <= n ? proj[(size_t)(t0 + n - back) * ldp + c] : s[j + n];
  }
}

constexpr int kChunk = 16;

__device__ __forceinline__ void cp_async16(float* dst, const float* src) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(a), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(float* dst, const float* src) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(a), "l"(src) : "memory");
}

template <int DREG, int MAXT>
__global__ void __launch_bounds__(MAXT)
delta_recurrence_kernel(const float* __restrict__ prep, int ldp, float* __restrict__ state,
                        size_t state_stride,
                        const int* __restrict__ cu_seqlens, const int* __restrict__ seq_slot,
                        int H, int G, int d, int e, int P, int ecols, float* __restrict__ o_raw,
                        int write_state, int vec) {
  extern __shared__ __align__(16) float sm[];
  // with at most 512 threads a lane also keeps the token's key slice in registers between
  // the two passes over its rows
  constexpr bool kKeepK = MAXT <= 512 && DREG <= 32;
  const int b = blockIdx.x, h = blockIdx.y, grp = h / (H / G);
  // lane `part` owns rows part*DREG .. +DREG-1; its slice of a staged key or query starts at
  // part*kSlice floats (four more than it holds, so that the P slices a warp reads at once
  // lie in different banks)
  constexpr int kSlice = DREG + 4;
  const int dpad = P * kSlice;
  // two stages of a chunk's operands, filled by asynchronous copies a chunk ahead:
  // q, k [kChunk][dpad], v [kChunk][ecols], beta, decay [kChunk]
  const int stage_floats = kChunk * (2 * dpad + ecols + 2);
  // this CTA owns columns col0 .. col0 + ecols - 1 of the head's matrix
  const int col0 = blockIdx.z * ecols;
  const int tid = threadIdx.x, part = tid % P, jl = tid / P, j = col0 + jl;
  const bool active = jl < ecols;
  float* M = state + (size_t)seq_slot[b] * state_stride + (size_t)h * d * e;
  // the lane's rows in pairs: the arithmetic below is two-wide (one instruction, two rows)
  float2 S[DREG / 2];
#pragma unroll
  for (int r = 0; r < DREG / 2; ++r) {
    const int i = part * DREG + 2 * r;
    S[r].x = (active && i < d) ? M[(size_t)i * e + j] : 0.f;
    S[r].y = (active && i + 1 < d) ? M[(size_t)(i + 1) * e + j] : 0.f;
  }
  const int t0 = cu_seqlens[b], t1 = cu_seqlens[b + 1];
  const int C = 2 * G * d + H * e;
  // the padding of the key and query slices stays zero for good
  for (int idx = tid; idx < 2 * stage_floats; idx += blockDim.x) sm[idx] = 0.f;
  __syncthreads();
  auto issue = [&](int s, int c0) {               // a chunk's operands on their way to stage s
    float* qs = sm + s * stage_floats;
    float* ks = qs + kChunk * dpad;
    float* vs = ks + kChunk * dpad;
    float* bs = vs + kChunk * ecols;
    const int n = min(kChunk, t1 - c0);
    if (vec) {
      // 16 bytes a copy: a warp's copy instruction moves 512 bytes (a lone 2,048-token prompt
      // at 16 heads of 128 x 128: 1.40 -> 1.27 ms a layer against 4-byte copies)
      const int d4 = d >> 2, e4 = ecols >> 2;
      for (int idx = tid; idx < n * d4; idx += blockDim.x) {
        const int tt = idx / d4, i = (idx - tt * d4) << 2;
        const int at = tt * dpad + (i / DREG) * kSlice + (i % DREG);
        const float* row = prep + (size_t)(c0 + tt) * ldp;
        cp_async16(qs + at, row + (size_t)grp * d + i);
        cp_async16(ks + at, row + (size_t)(G + grp) * d + i);
      }
      for (int idx = tid; idx < n * e4; idx += blockDim.x) {
        const int tt = idx / e4, i = (idx - tt * e4) << 2;
        cp_async16(vs + tt * ecols + i,
                   prep + (size_t)(c0 + tt) * ldp + 2 * G * d + (size_t)h * e + col0 + i);
      }
    } else {
      for (int idx = tid; idx < n * d; idx += blockDim.x) {
        const int tt = idx / d, i = idx - tt * d;
        const int at = tt * dpad + (i / DREG) * kSlice + (i % DREG);
        const float* row = prep + (size_t)(c0 + tt) * ldp;
        cp_async4(qs + at, row + (size_t)grp * d + i);
        cp_async4(ks + at, row + (size_t)(G + grp) * d + i);
      }
      for (int idx = tid; idx < n * ecols; idx += blockDim.x) {
        const int tt = idx / ecols, i = idx - tt * ecols;
        cp_async4(vs + idx, prep + (size_t)(c0 + tt) * ldp + 2 * G * d + (size_t)h * e + col0 + i);
      }
    }
    if (tid < n) {
      cp_async4(bs + tid, prep + (size_t)(c0 + tid) * ldp + C + h);
      cp_async4(bs + kChunk + tid, prep + (size_t)(c0 + tid) * ldp + C + H + h);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  if (t0 < t1) issue(0, t0);
  int s = 0;
  for (int c0 = t0; c0 < t1; c0 += kChunk, s ^= 1) {
    const int n = min(kChunk, t1 - c0);
    asm volatile("cp.async.wait_all;" ::: "memory");
    __syncthreads();          // stage s has arrived; the other stage is read no more
    if (c0 + kChunk < t1) issue(s ^ 1, c0 + kChunk);
    const float* qs = sm + s * stage_floats;
    const float* ks = qs + kChunk * dpad;
    const float* vs = ks + kChunk * dpad;
    const float* bs = vs + kChunk * ecols;
    const float* gs = bs + kChunk;
    // the token's three scalars are read a token ahead
    float g_next = gs[0], b_next = bs[0], v_next = active ? vs[jl] : 0.f;
    float* orow = o_raw + (size_t)c0 * H * e + (size_t)h * e + j;
    for (int tt = 0; tt < n; ++tt) {
      const float4* k4 = reinterpret_cast<const float4*>(ks + tt * dpad + part * kSlice);
      const float4* q4 = reinterpret_cast<const float4*>(qs + tt * dpad + part * kSlice);
      const float g = g_next, beta = b_next, vj = v_next;
      if (tt + 1 < n) {
        g_next = gs[tt + 1];
        b_next = bs[tt + 1];
        v_next = active ? vs[(tt + 1) * ecols + jl] : 0.f;
      }
      // The decay first, on every row the lane holds (independent multiplies), then the
      // products with the key in four chains, then -- once u is known -- the rank-one update
      // on every row and only then the read-out's chains: each group is a run of independent
      // instructions, so a lone warp on a scheduler does not wait four cycles for every one.
      // All of it two rows an instruction (fma.f32x2).
      float4 kreg[kKeepK ? DREG / 4 : 1];
      const float2 g2 = make_float2(g, g);
#pragma unroll
      for (int x = 0; x < DREG / 2; ++x) S[x] = __fmul2_rn(S[x], g2);
      float2 ra = make_float2(0.f, 0.f), rb = make_float2(0.f, 0.f);
#pragma unroll
      for (int x = 0; x < DREG / 4; ++x) {
        const float4 kv = k4[x];
        if (kKeepK) kreg[x] = kv;
        ra = __ffma2_rn(S[2 * x], make_float2(kv.x, kv.y), ra);
        rb = __ffma2_rn(S[2 * x + 1], make_float2(kv.z, kv.w), rb);
      }
      float r = (ra.x + ra.y) + (rb.x + rb.y);
      for (int o = P >> 1; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
      const float u = beta * (vj - r);
      const float2 u2 = make_float2(u, u);
#pragma unroll
      for (int x = 0; x < DREG / 4; ++x) {
        const float4 kv = kKeepK ? kreg[x] : k4[x];
        S[2 * x] = __ffma2_rn(make_float2(kv.x, kv.y), u2, S[2 * x]);
        S[2 * x + 1] = __ffma2_rn(make_float2(kv.z, kv.w), u2, S[2 * x + 1]);
      }
      float2 aa = make_float2(0.f, 0.f), ab = make_float2(0.f, 0.f);
#pragma unroll
      for (int x = 0; x < DREG / 4; ++x) {
        const float4 qv = q4[x];
        aa = __ffma2_rn(S[2 * x], make_float2(qv.x, qv.y), aa);
        ab = __ffma2_rn(S[2 * x + 1], make_float2(qv.z, qv.w), ab);
      }
      const float a0 = aa.x, a1 = aa.y, a2 = ab.x, a3 = ab.y;
      float acc = (a0 + a1) + (a2 + a3);
      for (int o = P >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (active && part == 0) orow[(size_t)tt * H * e] = acc;
    }
  }
  if (write_state) {
#pragma unroll
    for (int r = 0; r < DREG / 2; ++r) {
      const int i = part * DREG + 2 * r;
      if (active && i < d) M[(size_t)i * e + j] = S[r].x;
      if (active && i + 1 < d) M[(size_t)(i + 1) * e + j] = S[r].y;
    }
  }
}

// The read-outs of every (token, head), a warp each: RMS norm over e, the weight, SiLU of the gate.
template <typename TO>
__global__ void __launch_bounds__(256)
delta_out_norm_kernel(const float* __restrict__ o_raw, const float* __restrict__ gate, int ldg,
                      const float* __restrict__ norm_w, float eps, TO* __restrict__ out, int ldo,
                      int H, int e, long long items, int w_stride, int gate_sigmoid) {
  const long long item = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (item >= items) return;
  const int lane = threadIdx.x & 31;
  const long long t = item / H;
  const int h = (int)(item - t * H);
  const float* o = o_raw + (size_t)t * H * e + (size_t)h * e;
  const float* grow = gate + (size_t)t * ldg + (size_t)h * e;
  TO* orow = out + (size_t)t * ldo + (size_t)h * e;
  float ss = 0.f;
#pragma unroll 4
  for (int i = lane; i < e; i += 32) ss += o[i] * o[i];
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)e + eps);
  // w_stride: 0 when the heads share one weight of e numbers, e when each has its own;
  // the gate is SiLU or, with gate_sigmoid, the logistic function alone
  // a null weight: the read-outs are only divided by their root mean square
  const float* w = norm_w ? norm_w + (size_t)h * w_stride : nullptr;
#pragma unroll 4
  for (int i = lane; i < e; i += 32) {
    const float z = grow[i];
    const float gate_v = gate_sigmoid ? 1.0f / (1.0f + expf(-z)) : silu_f32(z);
    orow[i] = from_float<TO>(o[i] * inv * (w ? w[i] : 1.0f) * gate_v);
  }
}

template <int DREG, int MAXT>
static int launch_recurrence_t(const float* prep, int ldp, float* state, size_t state_stride,
                               const int* cu, const int* seq_slot, int B, int H, int G, int d,
                               int e, int P, int ecols, float* o_raw, int write_state, int threads,
                               cudaStream_t st) {
  const size_t stage = (size_t)kChunk * (2 * P * (DREG + 4) + ecols + 2);
  const size_t smem = sizeof(float) * 2 * stage;
  auto kern = delta_recurrence_kernel<DREG, MAXT>;
  if (smem > 48 * 1024) {
    if (smem > 200 * 1024) return kBadArgument;
    cudaError_t err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)smem);
    if (err != cudaSuccess) return (int)err;
  }
  // 16-byte copies of a chunk's operands where every address they touch is 16-byte aligned
  const int vec = ldp % 4 == 0 && d % 4 == 0 && e % 4 == 0 && ecols % 4 == 0 &&
                  ((uintptr_t)prep & 15) == 0;
  kern<<<dim3(B, H, e / ecols), threads, smem, st>>>(prep, ldp, state, state_stride, cu, seq_slot,
                                                     H, G, d, e, P, ecols, o_raw, write_state, vec);
  return launch_status();
}

template <int DREG>
static int launch_recurrence(const float* prep, int ldp, float* state, size_t state_stride,
                             const int* cu, const int* seq_slot, int B, int H, int G, int d, int e,
                             int P, int ecols, float* o_raw, int write_state, cudaStream_t st) {
  const int threads = ((ecols * P + 31) / 32) * 32;
  if (threads <= 512)
    return launch_recurrence_t<DREG, 512>(prep, ldp, state, state_stride, cu, seq_slot, B, H, G, d,
                                          e, P, ecols, o_raw, write_state, threads, st);
  return launch_recurrence_t<DREG, 1024>(prep, ldp, state, state_stride, cu, seq_slot, B, H, G, d,
                                         e, P, ecols, o_raw, write_state, threads, st);
}

}  // namespace cretif

using namespace cretif;

extern "C" int cretif_delta_prepare(const float* proj, int ldp, float* prep, int ldo,
                                    const float* conv_w, int taps, const float* conv_state,
                                    long long state_stride, const float* a_log,
                                    const float* dt_bias, const int* tok_pos, const int* tok_seq,
                                    const int* seq_slot, const int* seq_start, int H, int G, int d,
                                    int e, float unit_eps, int T, void* stream) {
  if (T <= 0) return kOk;
  if (H <= 0 || G <= 0 || H % G || d <= 0 || e <= 0 || taps < 1) return kBadArgument;
  const int C = 2 * G * d + H * e;
  if (ldp < C + H * e + 2 * H || ldo < C + 2 * H) return kBadArgument;
  if (d > kPrepMaxD) return kBadArgument;
  const int units = 2 * G + H + 1;
  dim3 grid(T, (units + kPrepWarps - 1) / kPrepWarps);
  if (grid.y > 65535) return kBadArgument;
  delta_prepare_kernel<<<grid, kPrepWarps * 32, 0, (cudaStream_t)stream>>>(
      proj, ldp, prep, ldo, conv_w, taps, conv_state, (size_t)state_stride, a_log, dt_bias,
      tok_pos, tok_seq, seq_slot, seq_start, H, G, d, e, unit_eps);
  return launch_status();
}

extern "C" int cretif_delta_conv_state(const float* proj, int ldp, float* conv_state,
                                       long long state_stride, int taps, int C,
                                       const int* cu_seqlens, const int* seq_slot, int B,
                                       void* stream) {
  if (B <= 0 || taps <= 1) return kOk;
  if (C <= 0 || ldp < C) return kBadArgument;
  delta_conv_state_kernel<<<dim3(B, (C + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      proj, ldp, conv_state, (size_t)state_stride, taps, C, cu_seqlens, seq_slot);
  return launch_status();
}

extern "C" int cretif_delta_recurrence(const float* prep, int ldp, const float* gate, int ldg,
                                       float* state, long long state_stride,
                                       const int* cu_seqlens, const int* seq_slot, int B, int H,
                                       int G, int d, int e, const float* norm_w, float eps,
                                       float* o_raw, void* out, int out_dt, int ldo,
                                       int write_state, int T, void* stream) {
  if (B <= 0 || T <= 0) return kOk;
  if (H <= 0 || G <= 0 || H % G || d <= 0 || e <= 0 || !o_raw) return kBadArgument;
  if (out_dt != kF32 && out_dt != kBF16) return kBadDType;
  static int sm_count = 0;
  if (!sm_count) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (sm_count <= 0) sm_count = 148;
  }
  // P lanes share a column, each with d/P of its rows in registers: up to 32 rows a lane.
  // Measured at d = e = 128 over 2,048 tokens of one sequence (16 heads, microseconds a layer):
  // 32 rows a lane and 16 warps a CTA without slices of columns 2,560 (bound by the instructions
  // issued: 276 a warp and token, 65 % of the issue slots); the same in slices of 32 columns
  // 1,116 (a warp a scheduler: the chain of a token's dependent steps); 8 rows a lane 1,087
  // (the shuffles and shared-memory reads share one pipe: about 1,000 of its cycles a token and
  // head); 64 rows a lane 1,760 (two warps a CTA).  Eight sequences: 32 and 64 rows the same,
  // 8 rows a sixth slower.
  int P = 1;
  while (P < 32 && (d + P - 1) / P > 32) P *= 2;
  // The columns of a head's matrix are independent: a head's columns are cut into slices for
  // CTAs of their own while the (sequence, head) pairs alone do not fill the chip twice over
  // (down to 32 columns), and as far as a CTA's 1024 threads demand.
  int ecols = e;
  while ((long long)B * H * (e / ecols) < 2LL * sm_count && ecols % 2 == 0 && ecols / 2 >= 32)
    ecols /= 2;
  while (ecols * P > 1024 && ecols % 2 == 0 && ecols > 1) ecols /= 2;
  while (ecols * P > 1024 && P > 1) P /= 2;            // an odd number of columns: longer slices
  if (ecols * P > 1024) return kBadArgument;
  const int rows = (d + P - 1) / P;
  if (rows > 128) return kBadArgument;
  cudaStream_t st = (cudaStream_t)stream;
  int rc;
#define CRETIF_DELTA(DREG)                                                                      \
  launch_recurrence<DREG>(prep, ldp, state, (size_t)state_stride, cu_seqlens, seq_slot, B, H, G, \
                          d, e, P, ecols, o_raw, write_state, st)
  if (rows <= 8) rc = CRETIF_DELTA(8);
  else if (rows <= 16) rc = CRETIF_DELTA(16);
  else if (rows <= 32) rc = CRETIF_DELTA(32);
  else if (rows <= 64) rc = CRETIF_DELTA(64);
  else rc = CRETIF_DELTA(128);
#undef CRETIF_DELTA
  if (rc) return rc;
  const long long items = (long long)T * H;
  const unsigned blocks = (unsigned)((items + 7) / 8);
  if (out_dt == kF32)
    delta_out_norm_kernel<float><<<blocks, 256, 0, st>>>(o_raw, gate, ldg, norm_w, eps,
                                                         (float*)out, ldo, H, e, items, 0, 0);
  else
    delta_out_norm_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(
        o_raw, gate, ldg, norm_w, eps, (__nv_bfloat16*)out, ldo, H, e, items, 0, 0);
  return launch_status();
}

// The per-head norm and gate of read-outs on their own, for other recurrences with a matrix per
// head (retention.cu): out = o_raw / rms(o_raw) [* norm_w] * gate(gate), a warp per (token, head).
extern "C" int cretif_heads_out_norm(const float* o_raw, const float* gate, int ldg,
                                     const float* norm_w, int per_head_weight, int gate_sigmoid,
                                     float eps, void* out, int out_dt, int ldo, int H, int e, int T,
                                     void* stream) {
  if (T <= 0) return kOk;
  if (H <= 0 || e <= 0 || !o_raw || !gate || ldg < H * e || ldo < H * e) return kBadArgument;
  const long long items = (long long)T * H;
  const unsigned blocks = (unsigned)((items + 7) / 8);
  cudaStream_t st = (cudaStream_t)stream;
  if (out_dt == kF32)
    delta_out_norm_kernel<float><<<blocks, 256, 0, st>>>(o_raw, gate, ldg, norm_w, eps,
                                                         (float*)out, ldo, H, e, items,
                                                         per_head_weight ? e : 0, gate_sigmoid);
  else if (out_dt == kBF16)
    delta_out_norm_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(
        o_raw, gate, ldg, norm_w, eps, (__nv_bfloat16*)out, ldo, H, e, items,
        per_head_weight ? e : 0, gate_sigmoid);
  else
    return kBadDType;
  return launch_status();
}

// ------------------------------------------------------------------------------------------
// The generalized delta rule: decay and removal rate per key channel, removal along the key
// at unit length.  Per token and head, with state M [d, e] (32-bit, zero at a sequence's start):
//     x = M^T u;   M <- diag(w) M - b x^T + k v^T;   o = M^T r          (u, b, w, k, r in R^d)
// where both products read the old M.  With u the key scaled to unit length, b = a * u for a
// removal rate a in (0, 1) per channel and w in (0, 1) per channel this is the rule in which a
// token first forgets (w), then takes out what the state holds along its key (a), then writes.
// (The gated rule above is the case w = g, u = k, b = beta g k, v scaled by beta.)
//
// * general_delta_prepare (a warp per head of a token): u = k / sqrt(|k|^2 + unit_eps),
//   b = sigmoid(a_proj + a_bias) * u, w = exp(-decay_scale * sigmoid(z + w0)), where
//   z = W2 tanh(w1) comes from the library's matrix product: w1 is the token's low-rank
//   projection (rank R, any size), tanh_cols applies the tanh and W2 [H d, R] expands it.
// * general_delta_recurrence: the thread layout of delta_recurrence above -- a CTA per
//   (sequence, head, slice of columns), P lanes a column, each lane a slice of the column's d
//   rows in registers, a chunk's operands staged in shared memory by asynchronous copies a
//   chunk ahead -- with five vectors a token (r, k, u, b, w) instead of two.  r, k and v are
//   read from the projection's rows as they are.
// * delta_out_norm (above) norms the read-outs per head, here with a weight per head and the
//   logistic function of the gate.
namespace cretif {

constexpr int kGenChunk = 8;

// proj row: [r (H d) | k (H d) | v (H e) | gate (H e) | a (H d) | w1 (R)]
// prep row: [u (H d) | -b (H d) | w (H d)];  z row: W2 tanh(w1), [H d]
__global__ void __launch_bounds__(kPrepWarps * 32)
general_delta_prepare_kernel(const float* __restrict__ proj, int ldp, float* __restrict__ prep,
                             int ldo, const float* __restrict__ a_bias,
                             const float* __restrict__ z, int ldz, const float* __restrict__ w0,
                             int H, int d, int e, float unit_eps, float decay_scale) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const float* row = proj + (size_t)t * ldp;
  const int h = blockIdx.y * kPrepWarps + warp;
  if (h >= H) return;
  float* out = prep + (size_t)t * ldo;
  const float* k = row + (size_t)H * d + (size_t)h * d;
  const float* a = row + (size_t)2 * H * d + (size_t)2 * H * e + (size_t)h * d;
  const float* zrow = z + (size_t)t * ldz + (size_t)h * d;
  float kv[kPrepMaxD / 32], av[kPrepMaxD / 32], zv[kPrepMaxD / 32];
  float ss = 0.f;
#pragma unroll
  for (int m = 0; m < kPrepMaxD / 32; ++m) {
    const int i = lane + 32 * m;
    kv[m] = i < d ? k[i] : 0.f;
    av[m] = i < d ? a[i] : 0.f;
    zv[m] = i < d ? zrow[i] : 0.f;
    ss += kv[m] * kv[m];
  }
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss + unit_eps);
#pragma unroll
  for (int m = 0; m < kPrepMaxD / 32; ++m) {
    const int i = lane + 32 * m;
    if (i >= d) continue;
    const int c = h * d + i;
    const float u = kv[m] * inv;
    const float rate = 1.0f / (1.0f + expf(-(av[m] + a_bias[c])));
    const float decay = expf(-decay_scale / (1.0f + expf(-(zv[m] + w0[c]))));
    out[c] = u;
    out[(size_t)H * d + c] = -rate * u;          // stored negative: the recurrence adds it
    out[(size_t)2 * H * d + c] = decay;
  }
}

// out[t, j] = tanh(in[t, j]) for the R columns of a strided float32 matrix, into the compute
// type: the input of the decay's second (expanding) product.
template <typename TO>
__global__ void tanh_cols_kernel(const float* __restrict__ in, int ld, TO* __restrict__ out,
                                 int R, long long total) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const long long t = idx / R;
  const int j = (int)(idx - t * R);
  out[idx] = from_float<TO>(tanhf(in[(size_t)t * ld + j]));
}

template <int DREG, int MAXT>
__global__ void __launch_bounds__(MAXT)
general_delta_recurrence_kernel(const float* __restrict__ proj, int ldp,
                                const float* __restrict__ prep, int ldq,
                                float* __restrict__ state, size_t state_stride,
                                const int* __restrict__ cu_seqlens,
                                const int* __restrict__ seq_slot, int H, int d, int e, int P,
                                int ecols, float* __restrict__ o_raw, int write_state, int vec) {
  extern __shared__ __align__(16) float sm[];
  const int b = blockIdx.x, h = blockIdx.y;
  constexpr int kSlice = DREG + 4;               // see delta_recurrence_kernel
  const int dpad = P * kSlice;
  // a stage: r, k, u, b, w [kGenChunk][dpad] each, v [kGenChunk][ecols]
  const int stage_floats = kGenChunk * (5 * dpad + ecols);
  const int col0 = blockIdx.z * ecols;
  const int tid = threadIdx.x, part = tid % P, jl = tid / P, j = col0 + jl;
  const bool active = jl < ecols;
  float* M = state + (size_t)seq_slot[b] * state_stride + (size_t)h * d * e;
  // the lane's rows in pairs: the arithmetic below is two-wide (one instruction, two rows)
  float2 S[DREG / 2];
#pragma unroll
  for (int r = 0; r < DREG / 2; ++r) {
    const int i = part * DREG + 2 * r;
    S[r].x = (active && i < d) ? M[(size_t)i * e + j] : 0.f;
    S[r].y = (active && i + 1 < d) ? M[(size_t)(i + 1) * e + j] : 0.f;
  }
  const int t0 = cu_seqlens[b], t1 = cu_seqlens[b + 1];
  for (int idx = tid; idx < 2 * stage_floats; idx += blockDim.x) sm[idx] = 0.f;
  __syncthreads();
  const size_t Hd = (size_t)H * d;
  auto issue = [&](int s, int c0) {
    float* base = sm + s * stage_floats;
    float* vs = base + 5 * kGenChunk * dpad;
    const int n = min(kGenChunk, t1 - c0);
    // vector x of token tt, rows i..: from the projection (r, k) or the prepared row (u, -b, w)
    auto src = [&](int x, int tt, int i) -> const float* {
      return x < 2 ? proj + (size_t)(c0 + tt) * ldp + (size_t)x * Hd + (size_t)h * d + i
                   : prep + (size_t)(c0 + tt) * ldq + (size_t)(x - 2) * Hd + (size_t)h * d + i;
    };
    if (vec) {
      const int d4 = d >> 2, e4 = ecols >> 2;
      for (int idx = tid; idx < 5 * n * d4; idx += blockDim.x) {
        const int x = idx / (n * d4), rem = idx - x * (n * d4);
        const int tt = rem / d4, i = (rem - tt * d4) << 2;
        cp_async16(base + (x * kGenChunk + tt) * dpad + (i / DREG) * kSlice + (i % DREG),
                   src(x, tt, i));
      }
      for (int idx = tid; idx < n * e4; idx += blockDim.x) {
        const int tt = idx / e4, i = (idx - tt * e4) << 2;
        cp_async16(vs + tt * ecols + i,
                   proj + (size_t)(c0 + tt) * ldp + 2 * Hd + (size_t)h * e + col0 + i);
      }
    } else {
      for (int idx = tid; idx < 5 * n * d; idx += blockDim.x) {
        const int x = idx / (n * d), rem = idx - x * (n * d);
        const int tt = rem / d, i = rem - tt * d;
        cp_async4(base + (x * kGenChunk + tt) * dpad + (i / DREG) * kSlice + (i % DREG),
                  src(x, tt, i));
      }
      for (int idx = tid; idx < n * ecols; idx += blockDim.x) {
        const int tt = idx / ecols, i = idx - tt * ecols;
        cp_async4(vs + idx, proj + (size_t)(c0 + tt) * ldp + 2 * Hd + (size_t)h * e + col0 + i);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  if (t0 < t1) issue(0, t0);
  int s = 0;
  for (int c0 = t0; c0 < t1; c0 += kGenChunk, s ^= 1) {
    const int n = min(kGenChunk, t1 - c0);
    asm volatile("cp.async.wait_all;" ::: "memory");
    __syncthreads();          // stage s has arrived; the other stage is read no more
    if (c0 + kGenChunk < t1) issue(s ^ 1, c0 + kGenChunk);
    const float* base = sm + s * stage_floats;
    const float* vs = base + 5 * kGenChunk * dpad;
    float* orow = o_raw + (size_t)c0 * H * e + (size_t)h * e + j;
    float v_next = active ? vs[jl] : 0.f;
    for (int tt = 0; tt < n; ++tt) {
      const int off = tt * dpad + part * kSlice;
      const float4* r4 = reinterpret_cast<const float4*>(base + off);
      const float4* k4 = reinterpret_cast<const float4*>(base + kGenChunk * dpad + off);
      const float4* u4 = reinterpret_cast<const float4*>(base + 2 * kGenChunk * dpad + off);
      const float4* b4 = reinterpret_cast<const float4*>(base + 3 * kGenChunk * dpad + off);
      const float4* w4 = reinterpret_cast<const float4*>(base + 4 * kGenChunk * dpad + off);
      const float vj = v_next;
      if (tt + 1 < n) v_next = active ? vs[(tt + 1) * ecols + jl] : 0.f;
      // what the old state holds along the unit key, in two two-wide chains
      float2 xa = make_float2(0.f, 0.f), xb = make_float2(0.f, 0.f);
#pragma unroll
      for (int q = 0; q < DREG / 4; ++q) {
        const float4 u = u4[q];
        xa = __ffma2_rn(S[2 * q], make_float2(u.x, u.y), xa);
        xb = __ffma2_rn(S[2 * q + 1], make_float2(u.z, u.w), xb);
      }
      float x = (xa.x + xa.y) + (xb.x + xb.y);
      for (int o = P >> 1; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
      // decay, removal (the prepared vector is minus a * u) and write on every row the lane
      // holds, then the read-out's chains; two rows an instruction
      const float2 x2 = make_float2(x, x), v2 = make_float2(vj, vj);
      float2 aa = make_float2(0.f, 0.f), ab = make_float2(0.f, 0.f);
#pragma unroll
      for (int q = 0; q < DREG / 4; ++q) {
        const float4 w = w4[q], nb = b4[q], kk = k4[q], rr = r4[q];
        float2 lo = __fmul2_rn(S[2 * q], make_float2(w.x, w.y));
        float2 hi = __fmul2_rn(S[2 * q + 1], make_float2(w.z, w.w));
        lo = __ffma2_rn(make_float2(nb.x, nb.y), x2, lo);
        hi = __ffma2_rn(make_float2(nb.z, nb.w), x2, hi);
        lo = __ffma2_rn(make_float2(kk.x, kk.y), v2, lo);
        hi = __ffma2_rn(make_float2(kk.z, kk.w), v2, hi);
        S[2 * q] = lo;
        S[2 * q + 1] = hi;
        aa = __ffma2_rn(lo, make_float2(rr.x, rr.y), aa);
        ab = __ffma2_rn(hi, make_float2(rr.z, rr.w), ab);
      }
      float acc = (aa.x + aa.y) + (ab.x + ab.y);
      for (int o = P >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (active && part == 0) orow[(size_t)tt * H * e] = acc;
    }
  }
  if (write_state) {
#pragma unroll
    for (int r = 0; r < DREG / 2; ++r) {
      const int i = part * DREG + 2 * r;
      if (active && i < d) M[(size_t)i * e + j] = S[r].x;
      if (active && i + 1 < d) M[(size_t)(i + 1) * e + j] = S[r].y;
    }
  }
}

template <int DREG, int MAXT>
static int launch_general_t(const float* proj, int ldp, const float* prep, int ldq, float* state,
                            size_t state_stride, const int* cu, const int* seq_slot, int B, int H,
                            int d, int e, int P, int ecols, float* o_raw, int write_state,
                            int threads, cudaStream_t st) {
  const size_t stage = (size_t)kGenChunk * (5 * P * (DREG + 4) + ecols);
  const size_t smem = sizeof(float) * 2 * stage;
  auto kern = general_delta_recurrence_kernel<DREG, MAXT>;
  if (smem > 48 * 1024) {
    if (smem > 200 * 1024) return kBadArgument;
    cudaError_t err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)smem);
    if (err != cudaSuccess) return (int)err;
  }
  const int vec = ldp % 4 == 0 && ldq % 4 == 0 && d % 4 == 0 && e % 4 == 0 && ecols % 4 == 0 &&
                  (((uintptr_t)proj | (uintptr_t)prep) & 15) == 0;
  kern<<<dim3(B, H, e / ecols), threads, smem, st>>>(proj, ldp, prep, ldq, state, state_stride, cu,
                                                     seq_slot, H, d, e, P, ecols, o_raw,
                                                     write_state, vec);
  return launch_status();
}

template <int DREG>
static int launch_general(const float* proj, int ldp, const float* prep, int ldq, float* state,
                          size_t state_stride, const int* cu, const int* seq_slot, int B, int H,
                          int d, int e, int P, int ecols, float* o_raw, int write_state,
                          cudaStream_t st) {
  const int threads = ((ecols * P + 31) / 32) * 32;
  if (threads <= 512)
    return launch_general_t<DREG, 512>(proj, ldp, prep, ldq, state, state_stride, cu, seq_slot, B,
                                       H, d, e, P, ecols, o_raw, write_state, threads, st);
  return launch_general_t<DREG, 1024>(proj, ldp, prep, ldq, state, state_stride, cu, seq_slot, B,
                                      H, d, e, P, ecols, o_raw, write_state, threads, st);
}

}  // namespace cretif

extern "C" int cretif_general_delta_prepare(const float* proj, int ldp, float* prep, int ldo,
                                            const float* a_bias, const float* z, int ldz,
                                            const float* w0, int H, int d, int e, float unit_eps,
                                            float decay_scale, int T, void* stream) {
  if (T <= 0) return kOk;
  if (H <= 0 || d <= 0 || e <= 0 || d > kPrepMaxD) return kBadArgument;
  if (ldp < 3 * H * d + 2 * H * e || ldo < 3 * H * d || ldz < H * d) return kBadArgument;
  dim3 grid(T, (H + kPrepWarps - 1) / kPrepWarps);
  if (grid.y > 65535) return kBadArgument;
  general_delta_prepare_kernel<<<grid, kPrepWarps * 32, 0, (cudaStream_t)stream>>>(
      proj, ldp, prep, ldo, a_bias, z, ldz, w0, H, d, e, unit_eps, decay_scale);
  return launch_status();
}

extern "C" int cretif_tanh_cols(const float* in, int ld, void* out, int out_dt, int R, int T,
                                void* stream) {
  if (T <= 0 || R <= 0) return kOk;
  if (ld < R) return kBadArgument;
  const long long total = (long long)T * R;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  cudaStream_t st = (cudaStream_t)stream;
  if (out_dt == kF32)
    tanh_cols_kernel<float><<<blocks, 256, 0, st>>>(in, ld, (float*)out, R, total);
  else if (out_dt == kBF16)
    tanh_cols_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(in, ld, (__nv_bfloat16*)out, R, total);
  else
    return kBadDType;
  return launch_status();
}

// per_head_weight: norm_w holds H * e numbers (else e, shared by the heads); gate_sigmoid: the
// gate is the logistic function of its projection (else SiLU).
// Fewest columns of a head's matrix a CTA takes (a test hook and tuning aid).  Measured at 16
// heads of 128 x 128 over 2,048 tokens of one sequence: 32 columns 1.81 ms, 16 1.92, 8 2.47,
// 4 3.57 (every CTA stages all five vectors of a token whatever its columns).
static int g_gen_min_cols = 32;
// Rows of a column that a lane holds: 0 = by how full the chip is (below), else 8, 16 or 32 (a
// test hook and tuning aid).
static int g_gen_rows = 0;
extern "C" int cretif_general_delta_rows(int n) {
  const int was = g_gen_rows;
  if (n == 0 || n == 8 || n == 16 || n == 32) g_gen_rows = n;
  return was;
}
extern "C" int cretif_general_delta_min_cols(int n) {
  const int was = g_gen_min_cols;
  if (n >= 1) g_gen_min_cols = n;
  return was;
}

extern "C" int cretif_general_delta_recurrence(
    const float* proj, int ldp, const float* prep, int ldq, const float* gate, int ldg,
    float* state, long long state_stride, const int* cu_seqlens, const int* seq_slot, int B, int H,
    int d, int e, const float* norm_w, int per_head_weight, int gate_sigmoid, float eps,
    float* o_raw, void* out, int out_dt, int ldo, int write_state, int T, void* stream) {
  if (B <= 0 || T <= 0) return kOk;
  if (H <= 0 || d <= 0 || e <= 0 || !o_raw) return kBadArgument;
  if (out_dt != kF32 && out_dt != kBF16) return kBadDType;
  static int sm_count = 0;
  if (!sm_count) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (sm_count <= 0) sm_count = 148;
  }
  // The plan of cretif_delta_recurrence, with the rows a lane holds chosen by how full the chip
  // is: a token's update is five vectors here, not two, and while there are fewer CTAs than SMs
  // more lanes a column shorten a lane's chain and add warps that hide each other's waits; with
  // the chip full, fewer shuffles win.  Measured at 16 heads of 128 x 128 over 2,048 tokens, ms:
  // one sequence 1.47 / 1.80 / 2.26 at 8 / 16 / 32 rows a lane, eight sequences of 256 tokens
  // 0.61 / 0.50 / 0.47.
  int rows_max = g_gen_rows;
  if (!rows_max) {
    const long long ctas = (long long)B * H * ((e + 31) / 32);
    rows_max = ctas < sm_count ? 8 : (ctas < 2LL * sm_count ? 16 : 32);
  }
  int P = 1;
  while (P < 32 && (d + P - 1) / P > rows_max) P *= 2;
  int ecols = e;
  while ((long long)B * H * (e / ecols) < 2LL * sm_count && ecols % 2 == 0 &&
         ecols / 2 >= g_gen_min_cols)
    ecols /= 2;
  while (ecols * P > 1024 && ecols % 2 == 0 && ecols > 1) ecols /= 2;
  while (ecols * P > 1024 && P > 1) P /= 2;
  if (ecols * P > 1024) return kBadArgument;
  const int rows = (d + P - 1) / P;
  if (rows > 32) return kBadArgument;               // head sizes beyond 1024
  cudaStream_t st = (cudaStream_t)stream;
  int rc;
#define CRETIF_GDELTA(DREG)                                                                     \
  launch_general<DREG>(proj, ldp, prep, ldq, state, (size_t)state_stride, cu_seqlens, seq_slot, \
                       B, H, d, e, P, ecols, o_raw, write_state, st)
  if (rows <= 8) rc = CRETIF_GDELTA(8);
  else if (rows <= 16) rc = CRETIF_GDELTA(16);
  else rc = CRETIF_GDELTA(32);
#undef CRETIF_GDELTA
  if (rc) return rc;
  const long long items = (long long)T * H;
  const unsigned blocks = (unsigned)((items + 7) / 8);
  const int w_stride = per_head_weight ? e : 0;
  if (out_dt == kF32)
    delta_out_norm_kernel<float><<<blocks, 256, 0, st>>>(o_raw, gate, ldg, norm_w, eps,
                                                         (float*)out, ldo, H, e, items, w_stride,
                                                         gate_sigmoid);
  else
    delta_out_norm_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(
        o_raw, gate, ldg, norm_w, eps, (__nv_bfloat16*)out, ldo, H, e, items, w_stride,
        gate_sigmoid);
  return launch_status();
}
