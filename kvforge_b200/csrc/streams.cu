// Kernels around a residual stream that is several streams (hyper-connections), a norm over the
// results of mixers that run side by side, a soft cap on logits, and the general form of the rotary
// encoding + cache write (interleaved or split pairs, a value size of its own).
//
// Hyper-connections: a token has S streams x_1 .. x_S of width W, held as [N][S][W] floats.  A
// sublayer reads u = sum_s in[s] x_s, computes y = f(norm(u)), and writes, for all t from the old
// streams, x_t <- sum_s mix[s][t] x_s + out[t] y.  As with a single stream, where the sum with the
// residual is folded into the norm that follows, the write of one sublayer and the read of the next
// are one kernel here: it takes the pending y with its mix and out, moves the streams on, reads the
// next u and norms it.  All of it is float; the normed row is rounded once to the storage type.
#include "common.cuh"

using namespace kvf;

namespace {

constexpr int MAX_STREAMS = 16;

struct HcParams {
  float* streams;        // [N][S][W]
  const void* y;         // pending result [N][W] in the storage type, or null
  const float* partials; // ... or the float slices of a split-K product [nsplit][N][W]
  int nsplit;
  long long split_stride;
  const float* mix;      // [S][S] (from, to) of the pending sublayer; null: nothing pending
  const float* out_w;    // [S]
  const float* in_w;     // [S] of the reading sublayer; null: every stream counts once (the plain sum)
  const float* norm_w;   // [W]
  void* out;             // [rows][W]
  const int* rows;       // gather: out row r comes from token rows[r] and the streams are left alone
  int W;
  float eps;
};

// S > 0: the number of streams is known at compile time and the streams of a column live in registers
template <typename T, int SC>
__global__ void __launch_bounds__(256) hc_step_kernel(const HcParams p, int S_rt) {
  pdl_launch();
  pdl_wait();
  extern __shared__ __align__(16) float urow[];  // [W] the read-out u
  __shared__ float red[32];
  __shared__ float s_mix[MAX_STREAMS * MAX_STREAMS], s_out[MAX_STREAMS], s_in[MAX_STREAMS];
  const int S = SC > 0 ? SC : S_rt;
  const int r = blockIdx.x;
  const size_t n = p.rows ? (size_t)p.rows[r] : (size_t)r;
  const int W = p.W;
  if (threadIdx.x < S * S && p.mix) s_mix[threadIdx.x] = p.mix[threadIdx.x];
  if (threadIdx.x < S) {
    s_out[threadIdx.x] = p.mix ? p.out_w[threadIdx.x] : 0.f;
    s_in[threadIdx.x] = p.in_w ? p.in_w[threadIdx.x] : 1.f;
  }
  __syncthreads();
  float* xs = p.streams + n * (size_t)S * W;
  const T* yr = p.y ? (const T*)p.y + n * W : nullptr;
  const float* pr = p.partials ? p.partials + n * W : nullptr;
  float ss = 0.f;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float x[SC > 0 ? SC : MAX_STREAMS];
#pragma unroll
    for (int s = 0; s < (SC > 0 ? SC : MAX_STREAMS); ++s)
      if (s < S) x[s] = xs[(size_t)s * W + c];
    float u = 0.f;
    if (p.mix) {
      float y = 0.f;
      if (yr) y = to_float<T>(yr[c]);
      else if (pr)
        for (int k = 0; k < p.nsplit; ++k) y += pr[(size_t)k * p.split_stride + c];
#pragma unroll
      for (int t = 0; t < (SC > 0 ? SC : MAX_STREAMS); ++t) {
        if (t < S) {
          float acc = 0.f;
#pragma unroll
          for (int s = 0; s < (SC > 0 ? SC : MAX_STREAMS); ++s)
            if (s < S) acc = fmaf(s_mix[s * S + t], x[s], acc);
          acc = fmaf(s_out[t], y, acc);
          if (!p.rows) xs[(size_t)t * W + c] = acc;
          u = fmaf(s_in[t], acc, u);
        }
      }
    } else {
#pragma unroll
      for (int t = 0; t < (SC > 0 ? SC : MAX_STREAMS); ++t)
        if (t < S) u = fmaf(s_in[t], x[t], u);
    }
    urow[c] = u;
    ss = fmaf(u, u, ss);
  }
  ss = block_sum(ss, red);
  const float inv = 1.f / sqrtf(ss / (float)W + p.eps);
  T* o = (T*)p.out + (size_t)r * W;
  for (int c = threadIdx.x; c < W; c += blockDim.x) o[c] = from_float<T>(urow[c] * inv * p.norm_w[c]);
}

// The same with a row's columns spread over the CTA so that a thread owns at most CPT of them and every load of
// the row (streams, pending result or its slices) is in flight before the first is used; the read-out stays in
// registers between the sum of squares and the write.  For widths up to 1024 * CPT.
template <typename T, int SC, int CPT>
__global__ void __launch_bounds__(1024) hc_step_rows_kernel(const HcParams p) {
  pdl_launch();
  pdl_wait();
  __shared__ float red[32];
  __shared__ float s_mix[SC * SC], s_out[SC], s_in[SC];
  const int r = blockIdx.x;
  const size_t n = p.rows ? (size_t)p.rows[r] : (size_t)r;
  const int W = p.W;
  if (threadIdx.x < SC * SC && p.mix) s_mix[threadIdx.x] = p.mix[threadIdx.x];
  if (threadIdx.x < SC) {
    s_out[threadIdx.x] = p.mix ? p.out_w[threadIdx.x] : 0.f;
    s_in[threadIdx.x] = p.in_w ? p.in_w[threadIdx.x] : 1.f;
  }
  float* xs = p.streams + n * (size_t)SC * W;
  const T* yr = p.y ? (const T*)p.y + n * W : nullptr;
  const float* pr = p.partials ? p.partials + n * W : nullptr;
  float x[CPT][SC], y[CPT], nw[CPT];
#pragma unroll
  for (int k = 0; k < CPT; ++k) {
    const int c = threadIdx.x + k * blockDim.x;
#pragma unroll
    for (int s = 0; s < SC; ++s) x[k][s] = c < W ? xs[(size_t)s * W + c] : 0.f;
    y[k] = (yr && c < W) ? to_float<T>(yr[c]) : 0.f;
    nw[k] = c < W ? p.norm_w[c] : 0.f;
  }
  if (pr) {
#pragma unroll 4
    for (int sl = 0; sl < p.nsplit; ++sl) {  // several slices' loads in flight; each column's sum in slice order
#pragma unroll
      for (int k = 0; k < CPT; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        if (c < W) y[k] += pr[(size_t)sl * p.split_stride + c];
      }
    }
  }
  __syncthreads();
  float u[CPT];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < CPT; ++k) {
    const int c = threadIdx.x + k * blockDim.x;
    float uu = 0.f;
    if (p.mix) {
#pragma unroll
      for (int t = 0; t < SC; ++t) {
        float acc = 0.f;
#pragma unroll
        for (int s = 0; s < SC; ++s) acc = fmaf(s_mix[s * SC + t], x[k][s], acc);
        acc = fmaf(s_out[t], y[k], acc);
        if (!p.rows && c < W) xs[(size_t)t * W + c] = acc;
        uu = fmaf(s_in[t], acc, uu);
      }
    } else {
#pragma unroll
      for (int t = 0; t < SC; ++t) uu = fmaf(s_in[t], x[k][t], uu);
    }
    u[k] = uu;
    ss = fmaf(uu, uu, ss);
  }
  ss = block_sum(ss, red);
  const float inv = 1.f / sqrtf(ss / (float)W + p.eps);
  T* o = (T*)p.out + (size_t)r * W;
#pragma unroll
  for (int k = 0; k < CPT; ++k) {
    const int c = threadIdx.x + k * blockDim.x;
    if (c < W) o[c] = from_float<T>(u[k] * inv * nw[k]);
  }
}

// every stream starts as the embedding's output
__global__ void replicate_kernel(const float* __restrict__ src, float* __restrict__ streams, int S, int W, size_t total) {
  pdl_launch();
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t n = i / ((size_t)S * W);
  const int c = (int)(i % W);
  streams[i] = src[n * W + c];
}

// ---------------------------------------------------------------- mean of normed branches
// out[n, :] = T( (1/nb) * sum_b rmsnorm(y_b[n, :]) * w_b[:] ) for the results y_b of nb mixers that read
// the same input; a result is a tensor in the storage type or the float slices of a split-K product.
constexpr int MAX_BRANCHES = 4;
struct BranchParams {
  const void* y[MAX_BRANCHES];
  const float* partials[MAX_BRANCHES];
  int nsplit[MAX_BRANCHES];
  long long split_stride[MAX_BRANCHES];
  const float* w[MAX_BRANCHES];
  int nb, W;
  float eps;
  void* out;
};

// A thread owns at most CPT columns of a row and keeps them in registers for every branch; all loads first.
template <typename T, int CPT>
__global__ void __launch_bounds__(256) branch_norm_mean_rows_kernel(const BranchParams p) {
  pdl_launch();
  pdl_wait();
  __shared__ float red[32];
  const size_t n = blockIdx.x;
  const int W = p.W;
  float v[MAX_BRANCHES][CPT];
#pragma unroll
  for (int b = 0; b < MAX_BRANCHES; ++b) {
#pragma unroll
    for (int k = 0; k < CPT; ++k) {
      const int c = threadIdx.x + k * blockDim.x;
      v[b][k] = (b < p.nb && c < W && p.y[b]) ? to_float<T>(((const T*)p.y[b])[n * W + c]) : 0.f;
    }
    if (b < p.nb && !p.y[b]) {
      const float* pr = p.partials[b] + n * W;
#pragma unroll 4
      for (int sl = 0; sl < p.nsplit[b]; ++sl) {  // a slice's columns together, several slices in flight
#pragma unroll
        for (int k = 0; k < CPT; ++k) {
          const int c = threadIdx.x + k * blockDim.x;
          if (c < W) v[b][k] += pr[(size_t)sl * p.split_stride[b] + c];
        }
      }
    }
  }
  float wv[MAX_BRANCHES][CPT];
#pragma unroll
  for (int b = 0; b < MAX_BRANCHES; ++b)
#pragma unroll
    for (int k = 0; k < CPT; ++k) {
      const int c = threadIdx.x + k * blockDim.x;
      wv[b][k] = (b < p.nb && c < W) ? p.w[b][c] : 0.f;
    }
  float inv[MAX_BRANCHES];
#pragma unroll
  for (int b = 0; b < MAX_BRANCHES; ++b) {
    inv[b] = 0.f;
    if (b < p.nb) {  // uniform over the CTA
      float ss = 0.f;
#pragma unroll
      for (int k = 0; k < CPT; ++k) ss = fmaf(v[b][k], v[b][k], ss);
      ss = block_sum(ss, red);
      inv[b] = 1.f / sqrtf(ss / (float)W + p.eps);
    }
  }
  const float share = 1.f / (float)p.nb;
  T* o = (T*)p.out + n * W;
#pragma unroll
  for (int k = 0; k < CPT; ++k) {
    const int c = threadIdx.x + k * blockDim.x;
    if (c >= W) continue;
    float acc = 0.f;
#pragma unroll
    for (int b = 0; b < MAX_BRANCHES; ++b)
      if (b < p.nb) acc += v[b][k] * inv[b] * wv[b][k];
    o[c] = from_float<T>(acc * share);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) branch_norm_mean_kernel(const BranchParams p) {
  pdl_launch();
  pdl_wait();
  extern __shared__ __align__(16) float rowbuf[];  // [nb][W]
  __shared__ float red[32];
  const size_t n = blockIdx.x;
  const int W = p.W;
  float inv[MAX_BRANCHES];
  for (int b = 0; b < p.nb; ++b) {
    const T* yr = p.y[b] ? (const T*)p.y[b] + n * W : nullptr;
    const float* pr = p.partials[b] ? p.partials[b] + n * W : nullptr;
    float ss = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
      float v = 0.f;
      if (yr) v = to_float<T>(yr[c]);
      else
        for (int k = 0; k < p.nsplit[b]; ++k) v += pr[(size_t)k * p.split_stride[b] + c];
      rowbuf[(size_t)b * W + c] = v;
      ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, red);
    inv[b] = 1.f / sqrtf(ss / (float)W + p.eps);
  }
  const float share = 1.f / (float)p.nb;
  T* o = (T*)p.out + n * W;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float acc = 0.f;
    for (int b = 0; b < p.nb; ++b) acc += rowbuf[(size_t)b * W + c] * inv[b] * p.w[b][c];
    o[c] = from_float<T>(acc * share);
  }
}

// ---------------------------------------------------------------- soft cap
__global__ void softcap_kernel(float* __restrict__ x, size_t n, float cap) {
  pdl_launch();
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) x[i] = cap * tanhf(x[i] / cap);
}

// ---------------------------------------------------------------- rotary + cache write, general form
// qkv rows: nh query heads of dk, nkv key heads of dk, nkv value heads of dv.  The first `rot` dims of
// a query or key head turn by float(pos) * inv_freq[i]: pair (2i, 2i+1) when `interleaved`, else
// (i, i + rot/2).  q is turned in place, k (turned) and v go to the token's slot of caches laid out
// [num_blocks][nkv][block_size][dk] and [...][dv].  slot < 0: nothing is stored.
template <typename T>
__global__ void __launch_bounds__(256) rope_cache_general_kernel(T* __restrict__ qkv, int stride, const int* __restrict__ positions,
                                                                 const float* __restrict__ inv_freq, const int* __restrict__ slots,
                                                                 T* __restrict__ kcache, T* __restrict__ vcache, int nh, int nkv, int dk,
                                                                 int dv, int rot, int interleaved, int block_size,
                                                                 long long num_slots, int* __restrict__ err) {
  pdl_launch();
  pdl_wait();
  const int n = blockIdx.x;
  T* row = qkv + (size_t)n * stride;
  const float pos = (float)positions[n];
  long long slot = slots ? (long long)slots[n] : -1;
  if (slot >= num_slots) {
    if (threadIdx.x == 0 && err) atomicOr(err, 2);
    slot = -1;
  }
  const long long blk = slot >= 0 ? slot / block_size : 0;
  const int off = slot >= 0 ? (int)(slot % block_size) : 0;
  const int half = rot >> 1;
  for (int w = threadIdx.x; w < (nh + nkv) * half; w += blockDim.x) {
    const int head = w / half, i = w - head * half;
    const int j1 = interleaved ? 2 * i : i, j2 = interleaved ? 2 * i + 1 : i + half;
    float s, c;
    sincosf(pos * inv_freq[i], &s, &c);
    T* hp = row + (size_t)head * dk;
    float r1, r2;
    rotate_pair(to_float<T>(hp[j1]), to_float<T>(hp[j2]), c, s, r1, r2);
    const T y1 = from_float<T>(r1), y2 = from_float<T>(r2);
    if (head < nh) {
      hp[j1] = y1;
      hp[j2] = y2;
    } else if (slot >= 0) {
      T* dst = kcache + (((size_t)blk * nkv + (head - nh)) * block_size + off) * dk;
      dst[j1] = y1;
      dst[j2] = y2;
    }
  }
  if (slot < 0) return;
  const int pass = dk - rot;
  for (int w = threadIdx.x; w < nkv * pass; w += blockDim.x) {
    const int kvh = w / pass, j = rot + (w - kvh * pass);
    kcache[(((size_t)blk * nkv + kvh) * block_size + off) * dk + j] = row[(size_t)(nh + kvh) * dk + j];
  }
  const T* vrow = row + (size_t)(nh + nkv) * dk;
  for (int w = threadIdx.x; w < nkv * dv; w += blockDim.x) {
    const int kvh = w / dv, j = w - kvh * dv;
    vcache[(((size_t)blk * nkv + kvh) * block_size + off) * dv + j] = vrow[w];
  }
}

static inline int row_threads(int W, int cpt) {
  int t = ((W + cpt - 1) / cpt + 31) / 32 * 32;
  return t > 1024 ? 1024 : t;
}

template <typename T, int SC>
int launch_hc(const HcParams& p, int n_rows, int S, cudaStream_t st) {
  if constexpr (SC > 0) {
   if (p.W <= 8192) {
    const dim3 g(n_rows);
    if (p.W <= 1024) launch(hc_step_rows_kernel<T, SC, 1>, dim3(g), dim3(row_threads(p.W, 1)), (size_t)(0), st, p);
    else if (p.W <= 2048) launch(hc_step_rows_kernel<T, SC, 2>, dim3(g), dim3(row_threads(p.W, 2)), (size_t)(0), st, p);
    else if (p.W <= 4096) launch(hc_step_rows_kernel<T, SC, 4>, dim3(g), dim3(row_threads(p.W, 4)), (size_t)(0), st, p);
    else launch(hc_step_rows_kernel<T, SC, 8>, dim3(g), dim3(row_threads(p.W, 8)), (size_t)(0), st, p);
    return KVF_LAUNCH_STATUS();
   }
  }
  launch(hc_step_kernel<T, SC>, dim3(dim3(n_rows)), dim3(256), (size_t)((size_t)p.W * sizeof(float)), st, p, S);
  return KVF_LAUNCH_STATUS();
}

}  // namespace

#define KVF_STREAMS_API(SUF, T)                                                                                        \
  KVF_API int kvf_hc_step_##SUF(float* streams, const void* y, const float* partials, int nsplit,                      \
                                long long split_stride, const float* mix, const float* out_w, const float* in_w,       \
                                const float* norm_w, void* out, const int* rows, int n_rows, int S, int W, float eps,  \
                                cudaStream_t st) {                                                                     \
    if (n_rows <= 0) return 0;                                                                                         \
    if (S <= 0 || S > MAX_STREAMS || W <= 0 || (size_t)W * sizeof(float) > 40 * 1024)                                  \
      return (int)cudaErrorInvalidValue;                                                                               \
    HcParams p;                                                                                                        \
    p.streams = streams; p.y = y; p.partials = partials; p.nsplit = nsplit; p.split_stride = split_stride;             \
    p.mix = mix; p.out_w = out_w; p.in_w = in_w; p.norm_w = norm_w; p.out = out; p.rows = rows; p.W = W; p.eps = eps;   \
    switch (S) {                                                                                                       \
      case 1: return launch_hc<T, 1>(p, n_rows, S, st);                                                                \
      case 2: return launch_hc<T, 2>(p, n_rows, S, st);                                                                \
      case 3: return launch_hc<T, 3>(p, n_rows, S, st);                                                                \
      case 4: return launch_hc<T, 4>(p, n_rows, S, st);                                                                \
      case 8: return launch_hc<T, 8>(p, n_rows, S, st);                                                                \
      default: return launch_hc<T, 0>(p, n_rows, S, st);                                                               \
    }                                                                                                                  \
  }                                                                                                                    \
  KVF_API int kvf_branch_norm_mean_##SUF(const void* const* y, const float* const* partials, const int* nsplit,        \
                                         const long long* split_stride, const float* const* w, int nb, long long N,    \
                                         int W, float eps, void* out, cudaStream_t st) {                               \
    if (N <= 0) return 0;                                                                                              \
    if (nb <= 0 || nb > MAX_BRANCHES || (size_t)nb * W * sizeof(float) > 160 * 1024) return (int)cudaErrorInvalidValue; \
    BranchParams p;                                                                                                    \
    for (int b = 0; b < nb; ++b) {                                                                                     \
      p.y[b] = y[b]; p.partials[b] = partials[b]; p.nsplit[b] = nsplit[b]; p.split_stride[b] = split_stride[b];        \
      p.w[b] = w[b];                                                                                                   \
      if (!p.y[b] && !p.partials[b]) return (int)cudaErrorInvalidValue;                                                \
    }                                                                                                                  \
    p.nb = nb; p.W = W; p.eps = eps; p.out = out;                                                                      \
    if (W <= 8192) {                                                                                                   \
      const dim3 g((unsigned)N);                                                                                       \
      /* small CTAs, so that many rows share an SM and their loads overlap */                                          \
      if (W <= 256) launch(branch_norm_mean_rows_kernel<T, 1>, g, dim3(row_threads(W, 1)), 0, st, p);                  \
      else if (W <= 1024) launch(branch_norm_mean_rows_kernel<T, 4>, g, dim3(row_threads(W, 4)), 0, st, p);            \
      else if (W <= 2048) launch(branch_norm_mean_rows_kernel<T, 8>, g, dim3(row_threads(W, 8)), 0, st, p);            \
      else if (W <= 4096) launch(branch_norm_mean_rows_kernel<T, 16>, g, dim3(row_threads(W, 16)), 0, st, p);          \
      else launch(branch_norm_mean_rows_kernel<T, 32>, g, dim3(row_threads(W, 32)), 0, st, p);                         \
      return KVF_LAUNCH_STATUS();                                                                                      \
    }                                                                                                                  \
    const size_t smem = (size_t)nb * W * sizeof(float);                                                                \
    if (smem > 48 * 1024) {                                                                                            \
      cudaError_t e = cudaFuncSetAttribute(branch_norm_mean_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,    \
                                           (int)smem);                                                                 \
      if (e != cudaSuccess) return (int)e;                                                                             \
    }                                                                                                                  \
    launch(branch_norm_mean_kernel<T>, dim3(dim3((unsigned)N)), dim3(256), (size_t)(smem), st, p);                                               \
    return KVF_LAUNCH_STATUS();                                                                                        \
  }                                                                                                                    \
  KVF_API int kvf_rope_cache_general_##SUF(void* qkv, int stride, const int* positions, const float* inv_freq,         \
                                           const int* slots, void* kcache, void* vcache, int N, int nh, int nkv,       \
                                           int dk, int dv, int rot, int interleaved, int block_size,                   \
                                           long long num_slots, int* err, cudaStream_t st) {                           \
    if (N <= 0) return 0;                                                                                              \
    if (rot < 0 || rot > dk || (rot & 1)) return (int)cudaErrorInvalidValue;                                           \
    launch(rope_cache_general_kernel<T>, dim3(dim3(N)), dim3(256), (size_t)(0), st, (T*)qkv, stride, positions, inv_freq, slots, (T*)kcache,     \
                                                          (T*)vcache, nh, nkv, dk, dv, rot, interleaved, block_size,   \
                                                          num_slots, err);                                             \
    return KVF_LAUNCH_STATUS();                                                                                        \
  }

KVF_STREAMS_API(f32, float)
KVF_STREAMS_API(bf16, bf16)

KVF_API int kvf_replicate_streams(const float* src, float* streams, long long N, int S, int W, cudaStream_t st) {
  const size_t total = (size_t)N * S * W;
  if (total == 0) return 0;
  launch(replicate_kernel, dim3(dim3((unsigned)((total + 255) / 256))), dim3(256), (size_t)(0), st, src, streams, S, W, total);
  return KVF_LAUNCH_STATUS();
}

KVF_API int kvf_softcap_f32(float* x, long long n, float cap, cudaStream_t st) {
  if (n <= 0) return 0;
  if (!(cap > 0.f)) return (int)cudaErrorInvalidValue;
  launch(softcap_kernel, dim3(dim3((unsigned)((n + 255) / 256))), dim3(256), (size_t)(0), st, x, (size_t)n, cap);
  return KVF_LAUNCH_STATUS();
}

// Turn programmatic dependent launch on or off for every launch of this library (its own flag: the flag is one
// per shared library).
KVF_API int kvf_mixers_set_pdl(int enabled) {
  kvf::g_pdl_enabled = enabled ? 1 : 0;
  return 0;
}
