// Kernels of mixers that carry a fixed-size state from token to token instead of (or beside) pages
// of keys: a short causal convolution over time per channel, the gated delta rule, and the gated
// RMS norm of a head's read-out.
//
// A step is a flat batch: sequence b owns the token rows qsl[b] .. qsl[b+1]-1 and the state slot
// state_slots[b].  A sequence without rows, a row at or beyond qsl[B] and a slot below zero touch
// nothing (the rule for parts with state: captured steps are padded with such sequences and rows).
// A request's state is a row of `state_stride` floats in a pool; every kernel gets the pointer to
// its own part of slot 0's row.  A fresh slot is all zeros.
//
// Everything a recurrence reads besides the projections (decays, step sizes, unit norms, the state
// itself) is float whatever the storage type T is.  Every sum has a fixed order that depends on the
// sizes alone, so a token's result does not depend on how its sequence was cut into steps or on what
// else the step holds.
#pragma once
#include "common.cuh"

using namespace kvf;

namespace {

// sequence that owns token row n (qsl ascending, qsl[0] == 0), or -1 for a padding row
__device__ __forceinline__ int seq_of_row(const int* __restrict__ qsl, int B, int n) {
  if (n >= qsl[B]) return -1;
  int lo = 0, hi = B - 1;
  while (lo < hi) {  // the last b with qsl[b] <= n
    const int mid = (lo + hi + 1) >> 1;
    if (qsl[mid] <= n) lo = mid; else hi = mid - 1;
  }
  return lo;
}

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }

// Activations whose result is rounded to the storage type: exact library functions for float storage; for
// bfloat16 storage the fast intrinsics (an error of a few units in the last place of a float, against a rounding
// of 2^-9 right after).  With the exact forms a convolution over 2,048 x 6,144 outputs was bound by issue slots
// (some 40 instructions an output), not by its 50 MB.
template <typename T> __device__ __forceinline__ float silu_of(float x);
template <> __device__ __forceinline__ float silu_of<float>(float x) { return silu_f(x); }
template <> __device__ __forceinline__ float silu_of<bf16>(float x) { return __fdividef(x, 1.f + __expf(-x)); }
template <typename T> __device__ __forceinline__ float sigmoid_of(float x);
template <> __device__ __forceinline__ float sigmoid_of<float>(float x) { return sigmoid_f(x); }
template <> __device__ __forceinline__ float sigmoid_of<bf16>(float x) { return __fdividef(1.f, 1.f + __expf(-x)); }

// ---------------------------------------------------------------- short causal convolution
// y[n, c] = act( sum_j w[c, j] * u[t - (taps-1) + j, c] ), t the place of row n in its sequence; places
// before this step's first row come from the state (the last taps-1 inputs of the sequence, oldest
// first, [taps-1][C] floats), which is zero before a sequence's start.
template <typename T, int VEC> struct VecIO;
template <> struct VecIO<float, 4> {
  static __device__ __forceinline__ void load(const float* p, float* f) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
  }
  static __device__ __forceinline__ void store(float* p, const float* f) { *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]); }
};
template <> struct VecIO<bf16, 8> {
  static __device__ __forceinline__ void load(const bf16* p, float* f) { bf16x8_to_float(*reinterpret_cast<const uint4*>(p), f); }
  static __device__ __forceinline__ void store(bf16* p, const float* f) {
    uint4 u;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = u;
  }
};
template <typename T> struct VecIO<T, 1> {
  static __device__ __forceinline__ void load(const T* p, float* f) { f[0] = to_float<T>(p[0]); }
  static __device__ __forceinline__ void store(T* p, const float* f) { p[0] = from_float<T>(f[0]); }
};

// A thread owns VEC neighbouring channels (one 16-byte load) of `rows` consecutive token rows; TAPS > 0: the
// taps are known at compile time and a thread keeps its weights in registers.  Each output is one chain of
// fused multiply-adds over the taps, oldest first, whichever form runs.
constexpr int CONV_ROWS = 4;  // rows of a tile when a step has many

template <typename T, int VEC, int TAPS>
__global__ void __launch_bounds__(128) causal_conv_kernel(const T* __restrict__ x, int x_stride, const float* __restrict__ w,
                                                          const float* __restrict__ state, long long state_stride,
                                                          const int* __restrict__ qsl, const int* __restrict__ state_slots,
                                                          int N, int B, int C, int taps_rt, int act, T* __restrict__ out,
                                                          int out_stride, int rows) {
  pdl_launch();
  pdl_wait();
  const int taps = TAPS > 0 ? TAPS : taps_rt;
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * VEC;
  if (c >= C) return;
  float wr[VEC][TAPS > 0 ? TAPS : 1];
  if (TAPS > 0) {
#pragma unroll
    for (int e = 0; e < VEC; ++e)
#pragma unroll
      for (int j = 0; j < TAPS; ++j) wr[e][j] = w[(size_t)(c + e) * TAPS + j];
  }
  if (TAPS > 0 && rows == CONV_ROWS) {
    // all of the tile's rows in one sequence: its rows + taps - 1 inputs are loaded once, together, and every row's
    // sum slides over them
    const int n0 = blockIdx.x * CONV_ROWS;
    const int b0 = n0 < N ? seq_of_row(qsl, B, n0) : -1;
    if (b0 < 0) return;
    const int first = qsl[b0], end = qsl[b0 + 1];
    if (n0 + CONV_ROWS <= end && n0 + CONV_ROWS <= N) {
      const int slot = state_slots[b0];
      const float* st = slot >= 0 ? state + (size_t)slot * state_stride : nullptr;
      const int t0 = n0 - first;
      constexpr int NIN = CONV_ROWS + (TAPS > 0 ? TAPS : 1) - 1;
      float u[NIN][VEC];
#pragma unroll
      for (int i = 0; i < NIN; ++i) {
        const int src = t0 - (TAPS - 1) + i;
        if (src >= 0) {
          VecIO<T, VEC>::load(x + (size_t)(first + src) * x_stride + c, u[i]);
        } else {
#pragma unroll
          for (int e = 0; e < VEC; ++e) u[i][e] = st ? st[(size_t)(TAPS - 1 + src) * C + c + e] : 0.f;
        }
      }
#pragma unroll
      for (int rr = 0; rr < CONV_ROWS; ++rr) {
        float acc[VEC];
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          acc[e] = 0.f;
#pragma unroll
          for (int j = 0; j < (TAPS > 0 ? TAPS : 1); ++j) acc[e] = fmaf(wr[e][j], u[rr + j][e], acc[e]);
          if (act == 1) acc[e] = silu_of<T>(acc[e]);
        }
        VecIO<T, VEC>::store(out + (size_t)(n0 + rr) * out_stride + c, acc);
      }
      return;
    }
  }
  for (int rr = 0; rr < rows; ++rr) {
    const int n = blockIdx.x * rows + rr;
    if (n >= N) return;
    const int b = seq_of_row(qsl, B, n);
    if (b < 0) return;  // this row and all after it belong to no sequence
    const int slot = state_slots[b];
    const int first = qsl[b];
    const int t = n - first;
    const float* st = slot >= 0 ? state + (size_t)slot * state_stride : nullptr;
    float acc[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) acc[e] = 0.f;
#pragma unroll
    for (int j = 0; j < (TAPS > 0 ? TAPS : 64); ++j) {
      if (j >= taps) break;
      const int src = t - (taps - 1) + j;
      float u[VEC];
      if (src >= 0) {
        VecIO<T, VEC>::load(x + (size_t)(first + src) * x_stride + c, u);
      } else {
#pragma unroll
        for (int e = 0; e < VEC; ++e) u[e] = st ? st[(size_t)(taps - 1 + src) * C + c + e] : 0.f;
      }
#pragma unroll
      for (int e = 0; e < VEC; ++e) acc[e] = fmaf(TAPS > 0 ? wr[e][TAPS > 0 ? j : 0] : w[(size_t)(c + e) * taps + j], u[e], acc[e]);
    }
    if (act == 1) {
#pragma unroll
      for (int e = 0; e < VEC; ++e) acc[e] = silu_of<T>(acc[e]);
    }
    VecIO<T, VEC>::store(out + (size_t)n * out_stride + c, acc);
  }
}

// Steps in which no sequence brings more than CONV_FEW rows (decoding): a thread owns VEC channels of ALL rows of
// one sequence, so it reads the old state, computes the rows and writes the new state itself: one launch.
constexpr int CONV_FEW = 4;

template <typename T, int VEC, int TAPS>
__global__ void __launch_bounds__(128) causal_conv_few_kernel(const T* __restrict__ x, int x_stride, const float* __restrict__ w,
                                                              float* __restrict__ state, long long state_stride,
                                                              const int* __restrict__ qsl, const int* __restrict__ state_slots,
                                                              int C, int act, T* __restrict__ out, int out_stride) {
  pdl_launch();
  pdl_wait();
  const int b = blockIdx.x;
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * VEC;
  const int first = qsl[b], q_len = qsl[b + 1] - first;
  const int slot = state_slots[b];
  if (c >= C || q_len <= 0 || q_len > CONV_FEW) return;
  float* st = slot >= 0 ? state + (size_t)slot * state_stride : nullptr;
  float wr[VEC][TAPS];
#pragma unroll
  for (int e = 0; e < VEC; ++e)
#pragma unroll
    for (int j = 0; j < TAPS; ++j) wr[e][j] = w[(size_t)(c + e) * TAPS + j];
  float u[TAPS - 1 + CONV_FEW][VEC];  // the state's inputs, then this step's rows
#pragma unroll
  for (int i = 0; i < TAPS - 1; ++i)
#pragma unroll
    for (int e = 0; e < VEC; ++e) u[i][e] = st ? st[(size_t)i * C + c + e] : 0.f;
#pragma unroll
  for (int i = 0; i < CONV_FEW; ++i) {
    if (i < q_len) VecIO<T, VEC>::load(x + (size_t)(first + i) * x_stride + c, u[TAPS - 1 + i]);
    else
#pragma unroll
      for (int e = 0; e < VEC; ++e) u[TAPS - 1 + i][e] = 0.f;
  }
#pragma unroll
  for (int i = 0; i < CONV_FEW; ++i) {
    if (i < q_len) {
      float acc[VEC];
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        acc[e] = 0.f;
#pragma unroll
        for (int j = 0; j < TAPS; ++j) acc[e] = fmaf(wr[e][j], u[i + j][e], acc[e]);
        if (act == 1) acc[e] = silu_of<T>(acc[e]);
      }
      VecIO<T, VEC>::store(out + (size_t)(first + i) * out_stride + c, acc);
    }
  }
  if (st) {  // the last TAPS-1 inputs, oldest first
#pragma unroll
    for (int i = 0; i < TAPS - 1; ++i) {
#pragma unroll
      for (int k = 0; k < TAPS - 1 + CONV_FEW; ++k)
        if (k == q_len + i) {
#pragma unroll
          for (int e = 0; e < VEC; ++e) st[(size_t)i * C + c + e] = u[k][e];
        }
    }
  }
}

template <typename T, int VEC>
int launch_conv_few(const T* x, int x_stride, const float* w, float* state, long long state_stride, const int* qsl,
                    const int* state_slots, int B, int C, int taps, int act, T* out, int out_stride, cudaStream_t st) {
  const int per_cta = 128 * VEC;
  dim3 grid(B, (C + per_cta - 1) / per_cta);
  if (grid.y > 65535u) return (int)cudaErrorInvalidValue;
  if (taps == 2) return launch(causal_conv_few_kernel<T, VEC, 2>, grid, dim3(128), 0, st, x, x_stride, w, state, state_stride, qsl, state_slots, C, act, out, out_stride);
  if (taps == 3) return launch(causal_conv_few_kernel<T, VEC, 3>, grid, dim3(128), 0, st, x, x_stride, w, state, state_stride, qsl, state_slots, C, act, out, out_stride);
  return launch(causal_conv_few_kernel<T, VEC, 4>, grid, dim3(128), 0, st, x, x_stride, w, state, state_stride, qsl, state_slots, C, act, out, out_stride);
}

template <typename T, int VEC>
int launch_conv(const T* x, int x_stride, const float* w, const float* state, long long state_stride, const int* qsl,
                const int* state_slots, int N, int B, int C, int taps, int act, T* out, int out_stride, cudaStream_t st) {
  const int rows = N >= 1024 ? CONV_ROWS : 1;
  const int per_cta = 128 * VEC;
  dim3 grid((N + rows - 1) / rows, (C + per_cta - 1) / per_cta);
  if (grid.y > 65535u) return (int)cudaErrorInvalidValue;
#define KVF_CONV_CASE(TP)                                                                                             \
  launch(causal_conv_kernel<T, VEC, TP>, dim3(grid), dim3(128), (size_t)(0), st, x, x_stride, w, state, state_stride, qsl, state_slots, N, B, C, \
                                                        taps, act, out, out_stride, rows)
  if (taps == 2) KVF_CONV_CASE(2);
  else if (taps == 3) KVF_CONV_CASE(3);
  else if (taps == 4) KVF_CONV_CASE(4);
  else if (taps <= 64) KVF_CONV_CASE(0);
  else return (int)cudaErrorInvalidValue;
#undef KVF_CONV_CASE
  return KVF_LAUNCH_STATUS();
}

template <typename T> struct ConvVec;
template <> struct ConvVec<float> { static constexpr int N = 4; };
template <> struct ConvVec<bf16> { static constexpr int N = 8; };

// The state after the step: the last taps-1 inputs of each sequence, old ones moved up where the
// step brought fewer rows than that.  Entry i is read at i + q_len > i before entry i is written,
// and a thread owns its channel, so the move is safe in place.
template <typename T>
__global__ void __launch_bounds__(256) conv_state_kernel(const T* __restrict__ x, int x_stride, float* __restrict__ state,
                                                         long long state_stride, const int* __restrict__ qsl,
                                                         const int* __restrict__ state_slots, int C, int taps) {
  pdl_launch();
  pdl_wait();
  const int b = blockIdx.x;
  const int first = qsl[b], q_len = qsl[b + 1] - first;
  const int slot = state_slots[b];
  if (q_len <= 0 || slot < 0) return;
  float* st = state + (size_t)slot * state_stride;
  const int keep = taps - 1;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
    for (int i = 0; i < keep; ++i) {
      const int src = q_len - keep + i;
      st[(size_t)i * C + c] = src >= 0 ? to_float<T>(x[(size_t)(first + src) * x_stride + c]) : st[(size_t)(i + q_len) * C + c];
    }
  }
}

// ---------------------------------------------------------------- gated delta rule
// Per sequence and head a state S [dk][dv] in float.  For every token, in order:
//   S <- g * S   (g one factor a head, or one a key channel: it scales row r of S)
//   u  = beta * (v - S^T k)
//   S <- S + k u^T
//   o  = S^T q          (so the read-out sees the token's own write)
// with k and q made unit vectors per head (x / sqrt(sum x^2 + norm_eps)), q times q_scale,
// beta = sigmoid(b), g = exp(-exp(A_log[h]) * softplus(a + dt_bias)).
//
// The walk over a sequence's tokens is a chain: a token's update needs the state the token before
// left.  What bounds it is the latency of one link, so a link is made short.  A CTA owns a sequence,
// a head and a tile of columns of S; a column's rows are spread over KS neighbouring lanes, R rows
// each, in registers.  One pass over a thread's rows applies the decay and takes both dot products
// with the decayed state, (S^T k) and (S^T q), in split accumulators; two shuffle trees run side by
// side; then u = beta (v - S^T k), the read-out is o = S^T q + u (k . q) (the same as reading after
// the write, with k . q taken once per token), and the write is one fused multiply-add per row with
// the keys still in registers.  What does not depend on the state (unit k and q, beta, g, k . q) is
// made before the walk by a kernel of its own, a warp per (token, head), so that no CTA of the walk
// repeats it for its tile of columns.  Tokens come in chunks through two buffers of shared memory:
// producer warps copy a chunk's vectors there (cp.async) while the consumer warps walk the chunk
// before.  The state goes through shared memory on its way in and out, so that global memory sees
// whole rows of a tile.
struct DeltaParams {
  const void* q;  // [N][G*dk] after convolution and activation
  const void* k;
  const void* v;  // [N][H*dv]
  int qkv_stride;
  const float* b;  // [N][H] logits of beta
  int b_stride;
  const float* a;  // [N][H] or [N][H*dk] logits of the step size
  int a_stride;
  const float* A_log;    // [H]
  const float* dt_bias;  // [H] or [H*dk]
  int per_channel;
  float* state;  // slot 0's [H][dk][dv]
  long long state_stride;
  float* out;  // [N][H*dv] read-out
  int out_stride;
  const int* qsl;
  const int* state_slots;
  int H, G, dk, dv;
  float q_scale, norm_eps;
  int chunk;       // tokens per chunk (a multiple of the producer warps)
  int buf_floats;  // floats of one chunk buffer
  // what the walk reads of a token besides v, made by the prepare kernel: unit keys and unit, scaled queries
  // [N][H][dk], the decay per key channel [N][H][dk] (per-channel form), and per (token, head) beta, k.q and
  // the head's decay [N][H][4]
  float* kn;
  float* qn;
  float* gn;
  float* sc;
  int N;
  // the logits of beta (and of a per-head step size) may come as the float slices of a split-K product
  int logit_slices;
  long long logit_slice_stride;
};

// exp(rate * softplus(x)), rate < 0: exact library functions in 32-bit storage; in bfloat16 storage the fast
// intrinsics (a few units in the last place of a float, far below what the rounding of q, k and v to bfloat16
// leaves), which cost a tenth of the instructions: a producer warp computes one of these per token, head and
// key channel
template <typename T> __device__ __forceinline__ float decay_of(float rate, float x);
template <> __device__ __forceinline__ float decay_of<float>(float rate, float x) { return expf(rate * softplus_f(x)); }
template <> __device__ __forceinline__ float decay_of<bf16>(float rate, float x) {
  return __expf(rate * (x > 20.f ? x : __logf(1.f + __expf(x))));
}

// Everything of a token that does not depend on the state, computed once, a warp per (token, head), by as many
// warps as the step has such pairs: the walk itself then only copies.
template <typename T>
__global__ void __launch_bounds__(128) delta_prepare_kernel(const DeltaParams p) {
  pdl_launch();
  pdl_wait();
  const long long pair = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (pair >= (long long)p.N * p.H) return;
  const int lane = threadIdx.x & 31;
  const size_t n = (size_t)(pair / p.H);
  const int h = (int)(pair - (long long)n * p.H);
  const int dk = p.dk, kvh = h / (p.H / p.G);
  const T* kr = (const T*)p.k + n * p.qkv_stride + (size_t)kvh * dk;
  const T* qr = (const T*)p.q + n * p.qkv_stride + (size_t)kvh * dk;
  float sk = 0.f, sq = 0.f, kq = 0.f;
#pragma unroll 4
  for (int r = lane; r < dk; r += 32) {
    const float kv = to_float<T>(kr[r]), qv = to_float<T>(qr[r]);
    sk = fmaf(kv, kv, sk);
    sq = fmaf(qv, qv, sq);
    kq = fmaf(kv, qv, kq);
  }
  sk = warp_sum(sk);
  sq = warp_sum(sq);
  kq = warp_sum(kq);
  const float ik = 1.f / sqrtf(sk + p.norm_eps), iq = p.q_scale / sqrtf(sq + p.norm_eps);
  const float neg_rate = -expf(p.A_log[h]);
  float* ko = p.kn + ((size_t)n * p.H + h) * dk;
  float* qo = p.qn + ((size_t)n * p.H + h) * dk;
  float* go = p.gn ? p.gn + ((size_t)n * p.H + h) * dk : nullptr;
  const float* ar = p.a + n * p.a_stride + (size_t)h * dk;
#pragma unroll 4
  for (int r = lane; r < dk; r += 32) {
    ko[r] = to_float<T>(kr[r]) * ik;
    qo[r] = to_float<T>(qr[r]) * iq;
    if (p.per_channel) go[r] = decay_of<T>(neg_rate, ar[r] + p.dt_bias[(size_t)h * dk + r]);
  }
  if (lane == 0) {
    float* so = p.sc + ((size_t)n * p.H + h) * 4;
    float bl = p.b[n * p.b_stride + h];
    float al = p.per_channel ? 0.f : p.a[n * p.a_stride + h];
    for (int sl = 1; sl < p.logit_slices; ++sl) {  // in slice order
      bl += p.b[(size_t)sl * p.logit_slice_stride + n * p.b_stride + h];
      if (!p.per_channel) al += p.a[(size_t)sl * p.logit_slice_stride + n * p.a_stride + h];
    }
    so[0] = sigmoid_f(bl);
    so[1] = kq * ik * iq;
    so[2] = p.per_channel ? 1.f : decay_of<T>(neg_rate, al + p.dt_bias[h]);
    so[3] = 0.f;
  }
}

__device__ __forceinline__ void cp_async16(float* smem_dst, const float* gsrc) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gsrc) : "memory");
}

// PW producer warps: 4 for walks over many tokens; 1 for steps of a few tokens a sequence (decoding), where a
// CTA lives for microseconds and what counts is how many of them fit an SM
template <typename T, int R, int KS, bool CH, int PW>
__global__ void __launch_bounds__(PW == 1 ? 288 : 384, PW == 1 ? 3 : 1) gated_delta_kernel(const DeltaParams p) {
  pdl_launch();
  pdl_wait();
  extern __shared__ __align__(16) float sm[];
  constexpr int RP = R + 4;      // a thread's rows in shared memory, padded so that the KS lanes of a column hit other banks
  constexpr int DKS = KS * RP;   // floats of one k, q or g vector in shared memory
  constexpr int DKP = R * KS;    // rows a column's threads cover; rows >= dk hold k = q = 0
  const int b = blockIdx.x, h = blockIdx.y;
  const int first = p.qsl[b], q_len = p.qsl[b + 1] - first;
  const int slot = p.state_slots[b];
  if (q_len <= 0 || slot < 0) return;
  const int CT = blockDim.x - PW * 32;  // consumer threads
  const int cols = CT / KS;
  const int dk = p.dk, dv = p.dv, TB = p.chunk;
  const bool producer = threadIdx.x >= CT;
  // layout of a chunk buffer: k [TB][DKS], q [TB][DKS], (g [TB][DKS],) v [TB][cols], beta [TB], k.q [TB], g of the head [TB]
  const int off_q = TB * DKS, off_g = 2 * TB * DKS, off_v = (CH ? 3 : 2) * TB * DKS;
  const int off_beta = off_v + TB * cols, off_kq = off_beta + TB, off_gh = off_kq + TB;
  float* sg = p.state + (size_t)slot * p.state_stride + (size_t)h * dk * dv;
  const int col0 = blockIdx.z * cols;
  const int nchunks = (q_len + TB - 1) / TB;

  // ---- producers: chunk c into buffer `buf`: copies of what the prepare kernel made (16 bytes a copy, straight
  // into shared memory, four rows of a vector at a time, which the padded layout keeps together) and this CTA's
  // columns of v.  Rows from dk up to DKP of k and q stay zero and of g one: they are set once, below.
  const int pt = threadIdx.x - CT;
  auto prepare = [&](int c, float* buf) {
    const int t0 = c * TB, nt = min(TB, q_len - t0);
    const T* vg = (const T*)p.v;
    const int nvec = CH ? 3 : 2;
    if ((dk & 3) == 0) {
      const int q4 = dk >> 2;  // copies per vector
      for (int idx = pt; idx < nt * nvec * q4; idx += PW * 32) {
        const int tt = idx / (nvec * q4), rem = idx - tt * (nvec * q4);
        const int which = rem / q4, r = (rem - which * q4) << 2;
        const float* src = (which == 0 ? p.kn : which == 1 ? p.qn : p.gn) + ((size_t)(first + t0 + tt) * p.H + h) * dk + r;
        cp_async16(buf + which * TB * DKS + tt * DKS + (r / R) * RP + (r % R), src);
      }
    } else {
      for (int idx = pt; idx < nt * nvec * dk; idx += PW * 32) {
        const int tt = idx / (nvec * dk), rem = idx - tt * (nvec * dk);
        const int which = rem / dk, r = rem - which * dk;
        const float* src = (which == 0 ? p.kn : which == 1 ? p.qn : p.gn) + ((size_t)(first + t0 + tt) * p.H + h) * dk + r;
        buf[which * TB * DKS + tt * DKS + (r / R) * RP + (r % R)] = *src;
      }
    }
    constexpr int VPT = 4;
    for (int base = 0; base < nt * cols; base += VPT * PW * 32) {
      float vv[VPT];
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int idx = base + i * PW * 32 + pt;
        const int tt = idx / cols, cc = col0 + (idx - tt * cols);
        vv[i] = (idx < nt * cols && cc < dv) ? to_float<T>(vg[(size_t)(first + t0 + tt) * p.qkv_stride + (size_t)h * dv + cc]) : 0.f;
      }
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int idx = base + i * PW * 32 + pt;
        if (idx < nt * cols) buf[off_v + idx] = vv[i];
      }
    }
    if (pt < nt) {
      const float4 sc4 = *reinterpret_cast<const float4*>(p.sc + ((size_t)(first + t0 + pt) * p.H + h) * 4);
      buf[off_beta + pt] = sc4.x;
      buf[off_kq + pt] = sc4.y;
      buf[off_gh + pt] = sc4.z;
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
  };

  float* buf0 = sm;
  float* buf1 = sm + p.buf_floats;
  const int ks = threadIdx.x % KS, cl = threadIdx.x / KS;
  const int col = col0 + cl;
  const bool live = !producer && col < dv;
  float S[R];
  if (dk < DKP) {  // rows that no copy ever writes: keys and queries zero, decay one
    for (int idx = threadIdx.x; idx < 2 * p.buf_floats; idx += blockDim.x) {
      const int in_buf = idx % p.buf_floats;
      sm[idx] = (CH && in_buf >= off_g && in_buf < off_v) ? 1.f : 0.f;
    }
    __syncthreads();
  }
  if (producer) {
    prepare(0, buf0);
  } else {
    // the state's tile [dk][cols] through shared memory (a region of its own behind the two chunk buffers)
    float* stage = sm + 2 * p.buf_floats;
    for (int base = 0; base < dk * cols; base += 8 * CT) {  // eight loads of a thread in flight at once
      float tmp[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int idx = base + i * CT + threadIdx.x;
        const int r = idx / cols, c = idx - r * cols;
        tmp[i] = (idx < dk * cols && col0 + c < dv) ? sg[(size_t)r * dv + col0 + c] : 0.f;
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int idx = base + i * CT + threadIdx.x;
        const int r = idx / cols, c = idx - r * cols;
        if (idx < dk * cols) stage[r * (cols + 1) + c] = tmp[i];
      }
    }
    asm volatile("bar.sync 1, %0;" ::"r"(CT) : "memory");
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const int r = ks * R + i;
      S[i] = r < dk ? stage[r * (cols + 1) + cl] : 0.f;
    }
  }
  __syncthreads();

  for (int c = 0; c < nchunks; ++c) {
    float* buf = (c & 1) ? buf1 : buf0;
    if (producer) {
      if (c + 1 < nchunks) prepare(c + 1, (c & 1) ? buf0 : buf1);
    } else {
      const int t0 = c * TB, nt = min(TB, q_len - t0);
      // the vectors of a token are fetched into registers while the token before is still in its shuffles
      float4 kn[R / 4], qn[R / 4], gn[R / 4];
      auto fetch = [&](int tt) {
        const float4* k4 = reinterpret_cast<const float4*>(buf + tt * DKS + ks * RP);
        const float4* q4 = reinterpret_cast<const float4*>(buf + off_q + tt * DKS + ks * RP);
        const float4* g4 = reinterpret_cast<const float4*>(buf + off_g + tt * DKS + ks * RP);
#pragma unroll
        for (int i = 0; i < R / 4; ++i) {
          kn[i] = k4[i];
          qn[i] = q4[i];
          if (CH) gn[i] = g4[i];
        }
      };
      fetch(0);
      for (int tt = 0; tt < nt; ++tt) {
        const float gh = CH ? 1.f : buf[off_gh + tt];
        const float beta = buf[off_beta + tt], vv = buf[off_v + tt * cols + cl], kq = buf[off_kq + tt];
        float kr[R];
        float dk_[4] = {0.f, 0.f, 0.f, 0.f}, dq_[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < R / 4; ++i) {
          const float4 kk = kn[i], qq = qn[i];
          float4 gg = make_float4(gh, gh, gh, gh);
          if (CH) gg = gn[i];
          kr[4 * i] = kk.x; kr[4 * i + 1] = kk.y; kr[4 * i + 2] = kk.z; kr[4 * i + 3] = kk.w;
          S[4 * i] *= gg.x; S[4 * i + 1] *= gg.y; S[4 * i + 2] *= gg.z; S[4 * i + 3] *= gg.w;
          dk_[0] = fmaf(S[4 * i], kk.x, dk_[0]); dk_[1] = fmaf(S[4 * i + 1], kk.y, dk_[1]);
          dk_[2] = fmaf(S[4 * i + 2], kk.z, dk_[2]); dk_[3] = fmaf(S[4 * i + 3], kk.w, dk_[3]);
          dq_[0] = fmaf(S[4 * i], qq.x, dq_[0]); dq_[1] = fmaf(S[4 * i + 1], qq.y, dq_[1]);
          dq_[2] = fmaf(S[4 * i + 2], qq.z, dq_[2]); dq_[3] = fmaf(S[4 * i + 3], qq.w, dq_[3]);
        }
        if (tt + 1 < nt) fetch(tt + 1);
        float dotk = (dk_[0] + dk_[1]) + (dk_[2] + dk_[3]);
        float dotq = (dq_[0] + dq_[1]) + (dq_[2] + dq_[3]);
#pragma unroll
        for (int o = KS >> 1; o > 0; o >>= 1) {
          dotk += __shfl_xor_sync(0xffffffffu, dotk, o);
          dotq += __shfl_xor_sync(0xffffffffu, dotq, o);
        }
        const float u = beta * (vv - dotk);
#pragma unroll
        for (int i = 0; i < R; ++i) S[i] = fmaf(kr[i], u, S[i]);
        if (ks == 0 && live) p.out[(size_t)(first + t0 + tt) * p.out_stride + (size_t)h * dv + col] = fmaf(u, kq, dotq);
      }
    }
    __syncthreads();
  }
  if (!producer) {
    float* stage = sm + 2 * p.buf_floats;
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const int r = ks * R + i;
      if (r < dk) stage[r * (cols + 1) + cl] = S[i];
    }
    asm volatile("bar.sync 1, %0;" ::"r"(CT) : "memory");
    for (int idx = threadIdx.x; idx < dk * cols; idx += CT) {
      const int r = idx / cols, c = idx - r * cols;
      if (col0 + c < dv) sg[(size_t)r * dv + col0 + c] = stage[r * (cols + 1) + c];
    }
  }
}

template <typename T, int R, int KS, bool CH, int PW>
int launch_delta(DeltaParams p, int B, cudaStream_t st) {
  constexpr int RP = R + 4, DKS = KS * RP;
  // consumer threads: steps of few tokens take 256 (fewer CTAs, each a short life); walks take 128 while that
  // leaves SMs free (a link of the chain is no faster with more columns in a CTA, and small CTAs spread over
  // more SMs), else 256
  int ct = PW == 1 ? 256 : 128;
  if (ct < KS) ct = KS;
  if (PW != 1) {
    const int cols128 = ct / KS;
    const long long ctas = (long long)B * p.H * ((p.dv + cols128 - 1) / cols128);
    if (ctas > 2 * 148 && 256 / KS <= p.dv) ct = 256;
  }
  while (ct > 32 && ct > KS && (ct / 2) / KS >= p.dv) ct /= 2;  // no more columns than the head has
  const int cols = ct / KS;
  const int per_token = (CH ? 3 : 2) * DKS + cols + 3;
  int chunk = PW == 1 ? 4 : 16;
  while (chunk > PW && (size_t)2 * chunk * per_token * sizeof(float) > 80 * 1024) chunk -= PW;
  const int buf_floats = (chunk * per_token + 3) / 4 * 4;
  const int stage = p.dk * (cols + 1);
  const size_t smem = ((size_t)2 * buf_floats + stage) * sizeof(float);
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  p.chunk = chunk;
  p.buf_floats = buf_floats;
  auto kern = gated_delta_kernel<T, R, KS, CH, PW>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid(B, p.H, (p.dv + cols - 1) / cols);
  launch(kern, dim3(grid), dim3(ct + PW * 32), (size_t)(smem), st, p);
  return KVF_LAUNCH_STATUS();
}

// Rows a thread: 16 for steps of few tokens; for walks 8 where the head is wide enough and the step has so few
// (sequence, head) pairs that the finer split still fits the device at once (twice the warps, each with half
// the chain of a token), else 16.
template <typename T, bool CH, int PW>
int dispatch_delta_rows(const DeltaParams& p, int B, cudaStream_t st) {
  const int dk = p.dk;
  if (PW != 1 && dk > 16 && dk <= 256) {
    const long long warps8 = (long long)B * p.H * p.dv * ((dk + 7) / 8) / 32;
    if (warps8 <= 4 * 592) {
      if (dk <= 32) return launch_delta<T, 8, 4, CH, PW>(p, B, st);
      if (dk <= 64) return launch_delta<T, 8, 8, CH, PW>(p, B, st);
      if (dk <= 128) return launch_delta<T, 8, 16, CH, PW>(p, B, st);
      return launch_delta<T, 8, 32, CH, PW>(p, B, st);
    }
  }
  if (dk <= 16) return launch_delta<T, 16, 1, CH, PW>(p, B, st);
  if (dk <= 32) return launch_delta<T, 16, 2, CH, PW>(p, B, st);
  if (dk <= 64) return launch_delta<T, 16, 4, CH, PW>(p, B, st);
  if (dk <= 128) return launch_delta<T, 16, 8, CH, PW>(p, B, st);
  if (dk <= 256) return launch_delta<T, 16, 16, CH, PW>(p, B, st);
  if (dk <= 512) return launch_delta<T, 32, 16, CH, PW>(p, B, st);
  if (dk <= 1024) return launch_delta<T, 32, 32, CH, PW>(p, B, st);
  return (int)cudaErrorInvalidValue;
}

template <typename T>
int dispatch_delta(const DeltaParams& p, int B, int max_q_len, cudaStream_t st) {
  const long long pairs = (long long)p.N * p.H;
  if (pairs <= 0) return 0;
  int rc = launch(delta_prepare_kernel<T>, dim3((unsigned)((pairs + 3) / 4)), dim3(128), 0, st, p);
  if (rc) return rc;
  const bool few = max_q_len > 0 && max_q_len <= 4;
  if (p.per_channel) return few ? dispatch_delta_rows<T, true, 1>(p, B, st) : dispatch_delta_rows<T, true, 4>(p, B, st);
  return few ? dispatch_delta_rows<T, false, 1>(p, B, st) : dispatch_delta_rows<T, false, 4>(p, B, st);
}

// ---------------------------------------------------------------- gated RMS norm of a head's read-out
// out[n, h, :] = T( o / sqrt(mean(o^2) + eps) * w[:] * act(gate[n, h, :]) ), a warp per (token, head);
// act: 1 = silu, 2 = sigmoid, 0 = no gate.
template <typename T>
__global__ void __launch_bounds__(128) gated_head_norm_kernel(const float* __restrict__ o, int o_stride, const T* __restrict__ gate,
                                                              int gate_stride, const float* __restrict__ w, float eps, int act,
                                                              long long pairs, int H, int dv, T* __restrict__ out, int out_stride) {
  pdl_launch();
  pdl_wait();
  const long long pair = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (pair >= pairs) return;
  const int lane = threadIdx.x & 31;
  const long long n = pair / H;
  const int h = (int)(pair - n * H);
  const float* row = o + (size_t)n * o_stride + (size_t)h * dv;
  float ss = 0.f;
  for (int j = lane; j < dv; j += 32) ss = fmaf(row[j], row[j], ss);
  ss = warp_sum(ss);
  const float inv = 1.f / sqrtf(ss / (float)dv + eps);
  const T* g = gate ? gate + (size_t)n * gate_stride + (size_t)h * dv : nullptr;
  T* dst = out + (size_t)n * out_stride + (size_t)h * dv;
  for (int j = lane; j < dv; j += 32) {
    float y = row[j] * inv * w[j];
    if (act == 1) y *= silu_of<T>(to_float<T>(g[j]));
    else if (act == 2) y *= sigmoid_of<T>(to_float<T>(g[j]));
    dst[j] = from_float<T>(y);
  }
}

}  // namespace

#define KVF_SEQMIX_API(SUF, T)                                                                                        \
  KVF_API int kvf_causal_conv_##SUF(const void* x, int x_stride, const float* w, float* state, long long state_stride, \
                                    const int* qsl, const int* state_slots, int N, int B, int C, int taps, int act,    \
                                    void* out, int out_stride, int max_q_len, cudaStream_t st) {                       \
    if (N <= 0 || B <= 0 || C <= 0) return 0;                                                                          \
    if (taps <= 0 || (unsigned)B > 65535u) return (int)cudaErrorInvalidValue;                                          \
    constexpr int V = ConvVec<T>::N;                                                                                   \
    const bool vec = C % V == 0 && x_stride % V == 0 && out_stride % V == 0 && ((uintptr_t)x % 16) == 0 &&             \
                     ((uintptr_t)out % 16) == 0;                                                                       \
    if (max_q_len > 0 && max_q_len <= CONV_FEW && taps >= 2 && taps <= 4) {                                            \
      return vec ? launch_conv_few<T, V>((const T*)x, x_stride, w, state, state_stride, qsl, state_slots, B, C, taps,  \
                                         act, (T*)out, out_stride, st)                                                 \
                 : launch_conv_few<T, 1>((const T*)x, x_stride, w, state, state_stride, qsl, state_slots, B, C, taps,  \
                                         act, (T*)out, out_stride, st);                                                \
    }                                                                                                                  \
    int rc = vec ? launch_conv<T, V>((const T*)x, x_stride, w, state, state_stride, qsl, state_slots, N, B, C, taps,   \
                                     act, (T*)out, out_stride, st)                                                     \
                 : launch_conv<T, 1>((const T*)x, x_stride, w, state, state_stride, qsl, state_slots, N, B, C, taps,   \
                                     act, (T*)out, out_stride, st);                                                    \
    int gy = (C + 255) / 256;                                                                                          \
    if (gy > 65535) gy = 65535;                                                                                        \
    if (rc || taps == 1) return rc;                                                                                    \
    launch(conv_state_kernel<T>, dim3(dim3(B, gy)), dim3(256), (size_t)(0), st, (const T*)x, x_stride, state, state_stride, qsl, state_slots,    \
                                                      C, taps);                                                        \
    return KVF_LAUNCH_STATUS();                                                                                        \
  }                                                                                                                    \
  KVF_API int kvf_gated_delta_##SUF(const void* q, const void* k, const void* v, int qkv_stride, const float* b,       \
                                    int b_stride, const float* a, int a_stride, const float* A_log,                    \
                                    const float* dt_bias, int per_channel, float* state, long long state_stride,       \
                                    float* out, int out_stride, const int* qsl, const int* state_slots, int B, int H,  \
                                    int G, int dk, int dv, float q_scale, float norm_eps, int max_q_len, int N,        \
                                    float* kn, float* qn, float* gn, float* sc, int logit_slices,                      \
                                    long long logit_slice_stride, cudaStream_t st) {                                   \
    if (B <= 0) return 0;                                                                                              \
    if (H <= 0 || G <= 0 || H % G || dk <= 0 || dv <= 0 || (unsigned)H > 65535u) return (int)cudaErrorInvalidValue;    \
    DeltaParams p;                                                                                                     \
    p.q = q; p.k = k; p.v = v; p.qkv_stride = qkv_stride; p.b = b; p.b_stride = b_stride; p.a = a;                     \
    p.a_stride = a_stride; p.A_log = A_log; p.dt_bias = dt_bias; p.per_channel = per_channel; p.state = state;         \
    p.state_stride = state_stride; p.out = out; p.out_stride = out_stride; p.qsl = qsl; p.state_slots = state_slots;   \
    p.H = H; p.G = G; p.dk = dk; p.dv = dv; p.q_scale = q_scale; p.norm_eps = norm_eps; p.chunk = 1; p.buf_floats = 0;  \
    p.kn = kn; p.qn = qn; p.gn = gn; p.sc = sc; p.N = N;                                                               \
    p.logit_slices = logit_slices; p.logit_slice_stride = logit_slice_stride;                                          \
    if (!kn || !qn || !sc || (per_channel && !gn)) return (int)cudaErrorInvalidValue;                                  \
    return dispatch_delta<T>(p, B, max_q_len, st);                                                                     \
  }                                                                                                                    \
  KVF_API int kvf_gated_head_norm_##SUF(const float* o, int o_stride, const void* gate, int gate_stride,               \
                                        const float* w, float eps, int act, long long N, int H, int dv, void* out,     \
                                        int out_stride, cudaStream_t st) {                                             \
    const long long pairs = N * H;                                                                                     \
    if (pairs <= 0) return 0;                                                                                          \
    if (act && !gate) return (int)cudaErrorInvalidValue;                                                               \
    launch(gated_head_norm_kernel<T>, dim3(dim3((unsigned)((pairs + 3) / 4))), dim3(128), (size_t)(0), st, o, o_stride, (const T*)gate,           \
                                                                                 gate_stride, w, eps, act, pairs, H,   \
                                                                                 dv, (T*)out, out_stride);             \
    return KVF_LAUNCH_STATUS();                                                                                        \
  }

