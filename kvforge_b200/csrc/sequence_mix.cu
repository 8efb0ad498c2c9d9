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

// ---------------------------------------------------------------- short causal convolution
// y[n, c] = act( sum_j w[c, j] * u[t - (taps-1) + j, c] ), t the place of row n in its sequence; places
// before this step's first row come from the state (the last taps-1 inputs of the sequence, oldest
// first, [taps-1][C] floats), which is zero before a sequence's start.
template <typename T>
__global__ void __launch_bounds__(256) causal_conv_kernel(const T* __restrict__ x, int x_stride, const float* __restrict__ w,
                                                          const float* __restrict__ state, long long state_stride,
                                                          const int* __restrict__ qsl, const int* __restrict__ state_slots,
                                                          int B, int C, int taps, int act, T* __restrict__ out, int out_stride) {
  const int n = blockIdx.x;
  const int b = seq_of_row(qsl, B, n);
  if (b < 0) return;
  const int slot = state_slots[b];
  const int first = qsl[b];
  const int t = n - first;
  const float* st = slot >= 0 ? state + (size_t)slot * state_stride : nullptr;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < taps; ++j) {
      const int src = t - (taps - 1) + j;
      float u;
      if (src >= 0) u = to_float<T>(x[(size_t)(first + src) * x_stride + c]);
      else u = st ? st[(size_t)(taps - 1 + src) * C + c] : 0.f;
      acc = fmaf(w[(size_t)c * taps + j], u, acc);
    }
    if (act == 1) acc = silu_f(acc);
    out[(size_t)n * out_stride + c] = from_float<T>(acc);
  }
}

// The state after the step: the last taps-1 inputs of each sequence, old ones moved up where the
// step brought fewer rows than that.  Entry i is read at i + q_len > i before entry i is written,
// and a thread owns its channel, so the move is safe in place.
template <typename T>
__global__ void __launch_bounds__(256) conv_state_kernel(const T* __restrict__ x, int x_stride, float* __restrict__ state,
                                                         long long state_stride, const int* __restrict__ qsl,
                                                         const int* __restrict__ state_slots, int C, int taps) {
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
// A CTA owns a sequence, a head and a tile of columns of S; a thread owns R rows (r = i*KS + ks) of one
// column in registers, so the KS threads of a column are neighbours in a warp and the two dot products
// of a token are R fused multiply-adds and a shuffle tree.  Tokens come in chunks: the CTA loads and
// prepares a chunk's k, q, v, beta and g into shared memory together, then walks the chunk without a
// barrier.
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
  int chunk;  // tokens per chunk
};

template <typename T, int R, int KS>
__global__ void __launch_bounds__(R * KS > 512 ? 1024 : 256) gated_delta_kernel(const DeltaParams p) {
  extern __shared__ __align__(16) float sm[];
  constexpr int DKP = R * KS;  // rows a column's threads cover; rows >= dk hold k = q = 0
  const int b = blockIdx.x, h = blockIdx.y;
  const int first = p.qsl[b], q_len = p.qsl[b + 1] - first;
  const int slot = p.state_slots[b];
  if (q_len <= 0 || slot < 0) return;
  const int cols = blockDim.x / KS;
  const int ks = threadIdx.x % KS, cl = threadIdx.x / KS;
  const int col = blockIdx.z * cols + cl;
  const bool live = col < p.dv;
  const int kvh = h / (p.H / p.G);
  const int dk = p.dk, dv = p.dv, TB = p.chunk;
  float* ks_s = sm;                  // [TB][DKP] unit keys
  float* qs_s = ks_s + TB * DKP;     // [TB][DKP] unit queries, scaled
  float* gs_s = qs_s + TB * DKP;     // [TB][DKP] decay per row (per_channel) or [TB] (one a head)
  float* vs_s = gs_s + (p.per_channel ? TB * DKP : TB);  // [TB][cols]
  float* bs_s = vs_s + TB * cols;    // [TB]

  float S[R];
  float* sg = p.state + (size_t)slot * p.state_stride + (size_t)h * dk * dv;
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int r = i * KS + ks;
    S[i] = (live && r < dk) ? sg[(size_t)r * dv + col] : 0.f;
  }
  const T* qg = (const T*)p.q;
  const T* kg = (const T*)p.k;
  const T* vg = (const T*)p.v;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const float neg_rate = -expf(p.A_log[h]);

  for (int t0 = 0; t0 < q_len; t0 += TB) {
    const int nt = min(TB, q_len - t0);
    __syncthreads();  // the chunk before has been walked
    // ---- prepare the chunk: a warp per token
    for (int tt = warp; tt < nt; tt += nwarps) {
      const size_t n = (size_t)(first + t0 + tt);
      const T* kr = kg + n * p.qkv_stride + (size_t)kvh * dk;
      const T* qr = qg + n * p.qkv_stride + (size_t)kvh * dk;
      float sk = 0.f, sq = 0.f;
      for (int r = lane; r < dk; r += 32) {
        const float kv = to_float<T>(kr[r]), qv = to_float<T>(qr[r]);
        sk = fmaf(kv, kv, sk);
        sq = fmaf(qv, qv, sq);
      }
      sk = warp_sum(sk);
      sq = warp_sum(sq);
      const float ik = 1.f / sqrtf(sk + p.norm_eps), iq = p.q_scale / sqrtf(sq + p.norm_eps);
      for (int r = lane; r < DKP; r += 32) {
        ks_s[tt * DKP + r] = r < dk ? to_float<T>(kr[r]) * ik : 0.f;
        qs_s[tt * DKP + r] = r < dk ? to_float<T>(qr[r]) * iq : 0.f;
      }
      if (p.per_channel) {
        const float* ar = p.a + n * p.a_stride + (size_t)h * dk;
        const float* br = p.dt_bias + (size_t)h * dk;
        for (int r = lane; r < DKP; r += 32) gs_s[tt * DKP + r] = r < dk ? expf(neg_rate * softplus_f(ar[r] + br[r])) : 1.f;
      } else if (lane == 0) {
        gs_s[tt] = expf(neg_rate * softplus_f(p.a[n * p.a_stride + h] + p.dt_bias[h]));
      }
      if (lane == 0) bs_s[tt] = sigmoid_f(p.b[n * p.b_stride + h]);
    }
    for (int idx = threadIdx.x; idx < nt * cols; idx += blockDim.x) {
      const int tt = idx / cols, c = idx - tt * cols;
      const int cc = blockIdx.z * cols + c;
      vs_s[idx] = cc < dv ? to_float<T>(vg[(size_t)(first + t0 + tt) * p.qkv_stride + (size_t)h * dv + cc]) : 0.f;
    }
    __syncthreads();
    // ---- walk the chunk
    for (int tt = 0; tt < nt; ++tt) {
      const float* kk = ks_s + tt * DKP + ks;
      const float* qq = qs_s + tt * DKP + ks;
      float dot = 0.f;
      if (p.per_channel) {
        const float* gg = gs_s + tt * DKP + ks;
#pragma unroll
        for (int i = 0; i < R; ++i) {
          S[i] *= gg[i * KS];
          dot = fmaf(S[i], kk[i * KS], dot);
        }
      } else {
        const float g = gs_s[tt];
#pragma unroll
        for (int i = 0; i < R; ++i) {
          S[i] *= g;
          dot = fmaf(S[i], kk[i * KS], dot);
        }
      }
#pragma unroll
      for (int o = KS >> 1; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
      const float u = bs_s[tt] * (vs_s[tt * cols + cl] - dot);
      float ro = 0.f;
#pragma unroll
      for (int i = 0; i < R; ++i) {
        S[i] = fmaf(kk[i * KS], u, S[i]);
        ro = fmaf(S[i], qq[i * KS], ro);
      }
#pragma unroll
      for (int o = KS >> 1; o > 0; o >>= 1) ro += __shfl_xor_sync(0xffffffffu, ro, o);
      if (ks == 0 && live) p.out[(size_t)(first + t0 + tt) * p.out_stride + (size_t)h * dv + col] = ro;
    }
  }
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int r = i * KS + ks;
    if (live && r < dk) sg[(size_t)r * dv + col] = S[i];
  }
}

template <typename T, int R, int KS>
int launch_delta(DeltaParams p, int B, cudaStream_t st) {
  constexpr int DKP = R * KS;
  int threads = (p.dv * KS + 31) / 32 * 32;
  const int cap = R * KS > 512 ? 1024 : 256;
  if (threads > cap) threads = cap;
  if (threads < KS) threads = KS;
  const int cols = threads / KS;
  // a chunk's k, q, (g,) v and beta within 48 KB of shared memory
  const int per_token = (2 + (p.per_channel ? 1 : 0)) * DKP + cols + 2;
  int chunk = (46 * 1024 / 4) / per_token;
  if (chunk > 16) chunk = 16;
  if (chunk < 1) return (int)cudaErrorInvalidValue;
  p.chunk = chunk;
  const size_t smem = (size_t)chunk * per_token * sizeof(float);
  dim3 grid(B, p.H, (p.dv + cols - 1) / cols);
  gated_delta_kernel<T, R, KS><<<grid, threads, smem, st>>>(p);
  return KVF_LAUNCH_STATUS();
}

template <typename T>
int dispatch_delta(const DeltaParams& p, int B, cudaStream_t st) {
  if (p.dk <= 16) return launch_delta<T, 16, 1>(p, B, st);
  if (p.dk <= 32) return launch_delta<T, 16, 2>(p, B, st);
  if (p.dk <= 64) return launch_delta<T, 16, 4>(p, B, st);
  if (p.dk <= 128) return launch_delta<T, 16, 8>(p, B, st);
  if (p.dk <= 256) return launch_delta<T, 16, 16>(p, B, st);
  if (p.dk <= 512) return launch_delta<T, 32, 16>(p, B, st);
  if (p.dk <= 1024) return launch_delta<T, 32, 32>(p, B, st);
  return (int)cudaErrorInvalidValue;
}

// ---------------------------------------------------------------- gated RMS norm of a head's read-out
// out[n, h, :] = T( o / sqrt(mean(o^2) + eps) * w[:] * act(gate[n, h, :]) ), a warp per (token, head);
// act: 1 = silu, 2 = sigmoid, 0 = no gate.
template <typename T>
__global__ void __launch_bounds__(128) gated_head_norm_kernel(const float* __restrict__ o, int o_stride, const T* __restrict__ gate,
                                                              int gate_stride, const float* __restrict__ w, float eps, int act,
                                                              long long pairs, int H, int dv, T* __restrict__ out, int out_stride) {
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
    if (act == 1) y *= silu_f(to_float<T>(g[j]));
    else if (act == 2) y *= sigmoid_f(to_float<T>(g[j]));
    dst[j] = from_float<T>(y);
  }
}

}  // namespace

#define KVF_SEQMIX_API(SUF, T)                                                                                        \
  KVF_API int kvf_causal_conv_##SUF(const void* x, int x_stride, const float* w, float* state, long long state_stride, \
                                    const int* qsl, const int* state_slots, int N, int B, int C, int taps, int act,    \
                                    void* out, int out_stride, cudaStream_t st) {                                      \
    if (N <= 0 || B <= 0 || C <= 0) return 0;                                                                          \
    if (taps <= 0 || (unsigned)B > 65535u) return (int)cudaErrorInvalidValue;                                          \
    int gy = (C + 255) / 256;                                                                                          \
    if (gy > 65535) gy = 65535;                                                                                        \
    causal_conv_kernel<T><<<dim3(N, gy), 256, 0, st>>>((const T*)x, x_stride, w, state, state_stride, qsl,             \
                                                       state_slots, B, C, taps, act, (T*)out, out_stride);             \
    int rc = KVF_LAUNCH_STATUS();                                                                                      \
    if (rc || taps == 1) return rc;                                                                                    \
    conv_state_kernel<T><<<dim3(B, gy), 256, 0, st>>>((const T*)x, x_stride, state, state_stride, qsl, state_slots,    \
                                                      C, taps);                                                        \
    return KVF_LAUNCH_STATUS();                                                                                        \
  }                                                                                                                    \
  KVF_API int kvf_gated_delta_##SUF(const void* q, const void* k, const void* v, int qkv_stride, const float* b,       \
                                    int b_stride, const float* a, int a_stride, const float* A_log,                    \
                                    const float* dt_bias, int per_channel, float* state, long long state_stride,       \
                                    float* out, int out_stride, const int* qsl, const int* state_slots, int B, int H,  \
                                    int G, int dk, int dv, float q_scale, float norm_eps, cudaStream_t st) {           \
    if (B <= 0) return 0;                                                                                              \
    if (H <= 0 || G <= 0 || H % G || dk <= 0 || dv <= 0 || (unsigned)H > 65535u) return (int)cudaErrorInvalidValue;    \
    DeltaParams p;                                                                                                     \
    p.q = q; p.k = k; p.v = v; p.qkv_stride = qkv_stride; p.b = b; p.b_stride = b_stride; p.a = a;                     \
    p.a_stride = a_stride; p.A_log = A_log; p.dt_bias = dt_bias; p.per_channel = per_channel; p.state = state;         \
    p.state_stride = state_stride; p.out = out; p.out_stride = out_stride; p.qsl = qsl; p.state_slots = state_slots;   \
    p.H = H; p.G = G; p.dk = dk; p.dv = dv; p.q_scale = q_scale; p.norm_eps = norm_eps; p.chunk = 1;                    \
    return dispatch_delta<T>(p, B, st);                                                                                \
  }                                                                                                                    \
  KVF_API int kvf_gated_head_norm_##SUF(const float* o, int o_stride, const void* gate, int gate_stride,               \
                                        const float* w, float eps, int act, long long N, int H, int dv, void* out,     \
                                        int out_stride, cudaStream_t st) {                                             \
    const long long pairs = N * H;                                                                                     \
    if (pairs <= 0) return 0;                                                                                          \
    if (act && !gate) return (int)cudaErrorInvalidValue;                                                               \
    gated_head_norm_kernel<T><<<dim3((unsigned)((pairs + 3) / 4)), 128, 0, st>>>(o, o_stride, (const T*)gate,           \
                                                                                 gate_stride, w, eps, act, pairs, H,   \
                                                                                 dv, (T*)out, out_stride);             \
    return KVF_LAUNCH_STATUS();                                                                                        \
  }

KVF_SEQMIX_API(f32, float)
KVF_SEQMIX_API(bf16, bf16)
