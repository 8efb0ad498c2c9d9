// A feed-forward made of many small experts of which every token uses a few.
//
//   route   : per token the router's logits (float), scores s = 1 / (1 + exp(-z)), the choice among
//             the best groups of neighbouring experts, the chosen experts and their weights
//   sort    : the (token, choice) pairs ordered by expert, and the list of row tiles per expert
//   product : for every tile of one expert's rows a tile of  act(x W_up^T)  or of  h W_down^T
//   combine : resid[token] += sum_k weight_k * y[token, k]   (float, k in order)
//
// A pair's row of a product depends on that row and on its expert's weights alone (one thread adds
// its products in the order of k), so a token's result does not depend on what else is in the batch
// or on where its pairs land in the order.  Router, scores, choice and the weighted sum are float
// whatever the storage type T.
#include <limits.h>

#include "common.cuh"

using namespace kvf;

namespace {

constexpr int TM = 32;  // rows of a tile of the grouped products

__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float v2 = __shfl_xor_sync(0xffffffffu, v, o);
    const int i2 = __shfl_xor_sync(0xffffffffu, i, o);
    if (v2 > v || (v2 == v && i2 < i)) {
      v = v2;
      i = i2;
    }
  }
}

// One warp per token.  Shared memory per warp: scores [E], choice scores [E], group scores [G],
// group flags [G].
template <typename T>
__global__ void __launch_bounds__(128) moe_route_kernel(const T* __restrict__ x, long long x_stride,
                                                         const float* __restrict__ router, const float* __restrict__ correction,
                                                         int n_tokens, int W, int E, int top, int groups, int keep,
                                                         float norm_eps, int* __restrict__ ids, float* __restrict__ wts) {
  pdl_launch();
  pdl_wait();
  extern __shared__ float sm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * 4 + warp;
  if (n >= n_tokens) return;
  float* sc = sm + (size_t)warp * (2 * E + 2 * groups);
  float* ch = sc + E;
  float* gs = ch + E;
  float* ga = gs + groups;
  const T* row = x + (size_t)n * x_stride;
  for (int e = 0; e < E; ++e) {
    const float* wr = router + (size_t)e * W;
    float z = 0.f;
    for (int j = lane; j < W; j += 32) z = fmaf(to_float<T>(row[j]), wr[j], z);
    z = warp_sum(z);
    if (lane == 0) {
      const float s = 1.f / (1.f + expf(-z));
      sc[e] = s;
      ch[e] = s + (correction ? correction[e] : 0.f);
    }
  }
  __syncwarp();
  if (groups > 1 && keep < groups) {
    // a group's score: the sum of its two largest choice scores; only the best `keep` groups stay
    const int per = E / groups;
    for (int g = lane; g < groups; g += 32) {
      float a = -INFINITY, b = -INFINITY;
      for (int e = g * per; e < (g + 1) * per; ++e) {
        const float v = ch[e];
        if (v > a) {
          b = a;
          a = v;
        } else if (v > b) {
          b = v;
        }
      }
      gs[g] = per > 1 ? a + b : a;
      ga[g] = 0.f;
    }
    __syncwarp();
    for (int k = 0; k < keep; ++k) {
      float v = -INFINITY;
      int i = INT_MAX;
      for (int g = lane; g < groups; g += 32)
        if (ga[g] == 0.f && (gs[g] > v || i == INT_MAX)) {
          v = gs[g];
          i = g;
        }
      warp_argmax(v, i);
      if (lane == 0 && i != INT_MAX) ga[i] = 1.f;
      __syncwarp();
    }
    for (int e = lane; e < E; e += 32)
      if (ga[e / per] == 0.f) ch[e] = -INFINITY;
    __syncwarp();
  }
  int* my_ids = ids + (size_t)n * top;
  float* my_w = wts + (size_t)n * top;
  float total = 0.f;
  for (int k = 0; k < top; ++k) {
    float v = -INFINITY;
    int i = INT_MAX;
    for (int e = lane; e < E; e += 32) {
      const float c = ch[e];
      if (c != c) continue;  // taken already (marked not-a-number)
      if (c > v || i == INT_MAX) {
        v = c;
        i = e;
      }
    }
    warp_argmax(v, i);
    if (i == INT_MAX) i = 0;  // cannot happen while top <= E
    const float s = sc[i];
    total += s;  // every lane adds the same numbers in the same order
    if (lane == 0) {
      my_ids[k] = i;
      my_w[k] = s;
      ch[i] = __int_as_float(0x7fc00000);
    }
    __syncwarp();
  }
  const float inv = 1.f / (total + norm_eps);
  for (int k = lane; k < top; k += 32) my_w[k] *= inv;
}

// One CTA.  ids [P] -> order [P] (pairs by expert), tiles: (expert, first sorted row, rows) per tile of
// TM rows, meta[0] = number of tiles.
__global__ void __launch_bounds__(1024) moe_sort_kernel(const int* __restrict__ ids, int P, int E, int* __restrict__ order,
                                                         int* __restrict__ tiles, int* __restrict__ meta) {
  pdl_launch();
  pdl_wait();
  extern __shared__ int si[];
  int* cnt = si;          // [E]
  int* off = cnt + E;     // [E]
  int* tbase = off + E;   // [E]
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < P; p += blockDim.x) atomicAdd(&cnt[ids[p]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0, t = 0;
    for (int e = 0; e < E; ++e) {
      off[e] = run;
      tbase[e] = t;
      run += cnt[e];
      t += (cnt[e] + TM - 1) / TM;
    }
    meta[0] = t;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const int c = cnt[e];
    for (int r0 = 0, t = tbase[e]; r0 < c; r0 += TM, ++t) {
      tiles[3 * t] = e;
      tiles[3 * t + 1] = off[e] + r0;
      tiles[3 * t + 2] = min(TM, c - r0);
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;  // now a cursor
  __syncthreads();
  for (int p = threadIdx.x; p < P; p += blockDim.x) {
    const int e = ids[p];
    order[off[e] + atomicAdd(&cnt[e], 1)] = p;
  }
}

__device__ __forceinline__ float gelu_erf(float z) { return 0.5f * z * (1.f + erff(z * 0.70710678118654752440f)); }

// A tile of TM rows of one expert times a tile of 64 of its output columns, on the FP32 pipes.
//   UP:   A row i = x[order[i] / top], B = w[e] [n_out][K], out act[i][col] = T(gelu(acc))
//   else: A row i = act[i],            B = w[e] [n_out][K], out y[order[i]][col] = acc (float)
template <typename T, bool UP>
__global__ void __launch_bounds__(256) moe_product_kernel(const T* __restrict__ a, long long a_stride, const T* __restrict__ w,
                                                           const int* __restrict__ order, const int* __restrict__ tiles,
                                                           const int* __restrict__ meta, int top, int K, int n_out,
                                                           T* __restrict__ act, float* __restrict__ y) {
  pdl_launch();
  pdl_wait();
  constexpr int BN = 64, BK = 16;
  if ((int)blockIdx.y >= meta[0]) return;
  __shared__ float As[BK][TM + 1];
  __shared__ float Bs[BK][BN + 1];
  __shared__ int src[TM];
  const int e = tiles[3 * blockIdx.y], row0 = tiles[3 * blockIdx.y + 1], rows = tiles[3 * blockIdx.y + 2];
  const int col0 = blockIdx.x * BN;
  const int tid = threadIdx.x;
  if (tid < TM) {
    int s = -1;
    if (tid < rows) s = UP ? order[row0 + tid] / top : row0 + tid;
    src[tid] = s;
  }
  __syncthreads();
  const T* wb = w + (size_t)e * n_out * K;
  const int ty = tid >> 4, tx = tid & 15;  // rows ty*2 .. +1, columns tx*4 .. +3
  float acc[2][4] = {};
  for (int k0 = 0; k0 < K; k0 += BK) {
    for (int idx = tid; idx < TM * BK; idx += 256) {
      const int r = idx / BK, kk = idx - r * BK;
      float v = 0.f;
      if (src[r] >= 0 && k0 + kk < K) v = to_float<T>(a[(size_t)src[r] * a_stride + k0 + kk]);
      As[kk][r] = v;
    }
    for (int idx = tid; idx < BN * BK; idx += 256) {
      const int c = idx / BK, kk = idx - c * BK;
      float v = 0.f;
      if (col0 + c < n_out && k0 + kk < K) v = to_float<T>(wb[(size_t)(col0 + c) * K + k0 + kk]);
      Bs[kk][c] = v;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      const float a0 = As[kk][ty * 2], a1 = As[kk][ty * 2 + 1];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float b = Bs[kk][tx * 4 + j];
        acc[0][j] = fmaf(a0, b, acc[0][j]);
        acc[1][j] = fmaf(a1, b, acc[1][j]);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = ty * 2 + i;
    if (r >= rows) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = col0 + tx * 4 + j;
      if (c >= n_out) continue;
      if (UP)
        act[(size_t)(row0 + r) * n_out + c] = from_float<T>(gelu_erf(acc[i][j]));
      else
        y[(size_t)order[row0 + r] * n_out + c] = acc[i][j];
    }
  }
}

__global__ void moe_combine_kernel(float* __restrict__ resid, const float* __restrict__ y, const float* __restrict__ wts,
                                   long long total, int W, int top) {
  pdl_launch();
  pdl_wait();
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const long long n = idx / W;
    const int c = (int)(idx - n * W);
    float s = 0.f;
    for (int k = 0; k < top; ++k) s = fmaf(wts[n * top + k], y[((size_t)n * top + k) * W + c], s);
    resid[idx] += s;
  }
}

}  // namespace

// Rows of tiles that `n_pairs` pairs spread over `E` experts can make at most.
KVF_API int kvf_moe_max_tiles(int n_pairs, int E) { return n_pairs / TM + E; }

#define KVF_EXPERTS_API(SUF, T)                                                                                       \
  KVF_API int kvf_moe_route_##SUF(const void* x, long long x_stride, const float* router, const float* correction,    \
                                  int n_tokens, int W, int E, int top, int groups, int keep, float norm_eps,          \
                                  int* ids, float* wts, cudaStream_t st) {                                            \
    if (n_tokens <= 0) return 0;                                                                                      \
    if (E <= 0 || top <= 0 || top > E || groups <= 0 || E % groups || keep <= 0 || keep > groups ||                   \
        top > keep * (E / groups))                                                                                    \
      return (int)cudaErrorInvalidValue;                                                                              \
    const size_t smem = (size_t)4 * (2 * E + 2 * groups) * sizeof(float);                                             \
    if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;                                                          \
    return launch(moe_route_kernel<T>, dim3((n_tokens + 3) / 4), dim3(128), smem, st, (const T*)x, x_stride, router,  \
                  correction, n_tokens, W, E, top, groups, keep, norm_eps, ids, wts);                                 \
  }                                                                                                                   \
  KVF_API int kvf_moe_experts_##SUF(const void* x, long long x_stride, const void* w_up, const void* w_down,          \
                                    const int* ids, const float* wts, int n_tokens, int W, int ff, int E, int top,    \
                                    int* order, int* tiles, int* meta, void* act, float* y, float* resid,             \
                                    cudaStream_t st) {                                                                \
    if (n_tokens <= 0) return 0;                                                                                      \
    const int P = n_tokens * top;                                                                                     \
    if ((size_t)3 * E * sizeof(int) > 48 * 1024) return (int)cudaErrorInvalidValue;                                   \
    int rc = launch(moe_sort_kernel, dim3(1), dim3(1024), (size_t)3 * E * sizeof(int), st, ids, P, E, order, tiles,   \
                    meta);                                                                                            \
    if (rc) return rc;                                                                                                \
    const int max_tiles = kvf_moe_max_tiles(P, E);                                                                    \
    if (max_tiles > 65535) return (int)cudaErrorInvalidValue;                                                         \
    rc = launch(moe_product_kernel<T, true>, dim3((ff + 63) / 64, max_tiles), dim3(256), 0, st, (const T*)x,          \
                x_stride, (const T*)w_up, (const int*)order, (const int*)tiles, (const int*)meta, top, W, ff, (T*)act, \
                (float*)nullptr);                                                                                     \
    if (rc) return rc;                                                                                                \
    rc = launch(moe_product_kernel<T, false>, dim3((W + 63) / 64, max_tiles), dim3(256), 0, st, (const T*)act,        \
                (long long)ff, (const T*)w_down, (const int*)order, (const int*)tiles, (const int*)meta, top, ff, W,   \
                (T*)nullptr, y);                                                                                      \
    if (rc) return rc;                                                                                                \
    const long long total = (long long)n_tokens * W;                                                                  \
    long long g = (total + 255) / 256;                                                                                \
    if (g > 148 * 16) g = 148 * 16;                                                                                   \
    return launch(moe_combine_kernel, dim3((unsigned)g), dim3(256), 0, st, resid, (const float*)y, wts, total, W,     \
                  top);                                                                                               \
  }

KVF_EXPERTS_API(f32, float)
KVF_EXPERTS_API(bf16, bf16)
