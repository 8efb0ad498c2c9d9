// Attention over a paged cache that holds ONE row of d numbers per token, shared by all heads: the
// row is every head's key, and its first dv numbers are every head's value (keys and values made from
// one latent whose up-projections are folded into the queries and into what follows the attention).
// bfloat16 on the tensor cores (mma.sync m16n8k16); same contract as attention_generic.cu: sequence b
// has ctx_b rows after this step's writes and q_b queries; query i sits at p = ctx_b - q_b + i and sees
// row j iff j <= p (and j > p - window when window > 0); scores and softmax in float, one rounding.
//
// A CTA owns 16 or 32 rows of (query token, head), four warps per 16 rows: all 16 heads of one or two
// tokens, or several tokens of fewer heads, so that a tile of keys brought into shared memory serves every
// head (32 or 64 rows with eight or sixteen warps where a step brings enough tokens: a tile is then fetched less
// often, and one group of four warps computes while another waits).  Keys come
// in tiles of 32 that start at multiples of 32 (cp.async, two stages, rows padded by 16 bytes so that
// the 8 rows of an ldmatrix lie in different banks).  Per tile:
//   scores   the four warps of 16 rows share out the k-steps of q . k (d/16 of them), leave their partial
//            [16 x 32] sums in shared memory and add the four in warp order;
//   softmax  every warp for itself (the same numbers in all four);
//   values   every warp owns dv/4 output columns: O[16 x dv/4] += P[16 x 32] V[32 x dv/4], the value
//            tile being the key tile's first dv columns, read transposed.
// Tile form: prompts, portions, mixed batches (grid: tiles of queries x sequences x head chunks).
// Split form: one query a sequence, grid.x walks ranges of keys; partial (m, l, acc) go to scratch and
// a second kernel merges the ranges in range order.
// d a multiple of 16 (at most 1024), dv a multiple of 32 with dv/32 in {2, 3, 4, 8, 16}, dv <= d.
#include "common.cuh"

using namespace kvf;

namespace {

constexpr int BN = 32;     // keys per tile
constexpr int WARPS = 4;
constexpr int ROWS = 16;   // (token, head) rows of one m-tile; a CTA has MT of them
constexpr int PAD = 8;     // elements of padding per row of shared memory

struct LatParams {
  const bf16* q;
  bf16* out;
  const bf16* cache;  // [blocks][1][block_size][d]
  const int* block_tables;
  const int* qsl;
  const int* ctx_lens;
  float* part_acc;  // split form: [B][nh][max_splits][dv]
  float* part_ml;   // split form: [B][nh][max_splits][2]  (m in natural-log units, l)
  int q_stride, out_stride, bt_stride;
  int nh, d, dv, block_size;
  int gh, chunks, tq;  // heads per CTA, head chunks, tokens per CTA
  int bs_shift;        // log2(block_size) if it is a power of two, else -1
  int window;
  int split_size, max_splits;
  float scale_log2;  // scale * log2(e)
};

__device__ __forceinline__ uint32_t su32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cpa16(uint32_t dst, const void* src, bool valid) {
  const int sz = valid ? 16 : 0;  // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(sz));
}
__device__ __forceinline__ void cpa_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cpa_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

// NTW: n-tiles of 8 output columns per warp (dv = 32 * NTW).  MT: m-tiles of 16 rows per CTA, each with four warps
// of its own (`group` is a warp's m-tile, `w4` its place among the four).
template <int NTW, int MT, bool SPLIT>
__global__ void __launch_bounds__(WARPS * 32 * MT) latent_attn_kernel(const LatParams p) {
  constexpr int ML = 1;  // m-tiles a warp holds
  pdl_launch();
  pdl_wait();
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const int d = p.d, ld = d + PAD;  // elements per row of shared memory
  const uint32_t row_bytes = (uint32_t)ld * 2;
  constexpr int RWS = ROWS * MT;
  const uint32_t qs = su32(smem_raw);                       // [RWS][ld]
  const uint32_t ks0 = qs + RWS * row_bytes;                // [2][BN][ld]
  const uint32_t k_stage = BN * row_bytes;
  float* sp = reinterpret_cast<float*>(smem_raw + (size_t)(RWS + 2 * BN) * row_bytes);  // [MT][WARPS][4][4][32]

  const int b = blockIdx.y, chunk = blockIdx.z;
  const int q_begin = p.qsl[b], q_len = p.qsl[b + 1] - q_begin;
  const int ctx = p.ctx_lens[b];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = warp >> 2, w4 = warp & 3;
  if (q_len <= 0 || ctx <= 0) return;

  int q0, n_tok, p_first, kv_lo, kv_hi;
  if (SPLIT) {
    q0 = q_len - 1;
    n_tok = 1;
    p_first = ctx - 1;
    kv_lo = blockIdx.x * p.split_size;
    if (kv_lo >= ctx) return;  // a range past the context: the merge never reads it
    kv_hi = min(ctx, kv_lo + p.split_size);
    const int win_first = p.window > 0 ? max(0, ctx - p.window) : 0;
    if (kv_hi <= win_first) {
      // a range wholly before the window is empty, and says so to the merge
      for (int r = threadIdx.x; r < p.gh; r += blockDim.x) {
        const int head = chunk * p.gh + r;
        if (head < p.nh) {
          float* ml = p.part_ml + (((size_t)b * p.nh + head) * p.max_splits + blockIdx.x) * 2;
          ml[0] = -INFINITY;
          ml[1] = 0.f;
        }
      }
      return;
    }
    kv_lo = max(kv_lo, (win_first / BN) * BN);
  } else {
    q0 = blockIdx.x * p.tq;
    if (q0 >= q_len) return;
    n_tok = min(p.tq, q_len - q0);
    p_first = ctx - q_len + q0;
    kv_hi = p_first + n_tok;
    kv_lo = p.window > 0 ? (max(0, p_first - p.window + 1) / BN) * BN : 0;
  }

  // ---- the query rows: row r -> (token r / gh, head chunk * gh + r % gh); rows past the tokens or the heads are zeros
  const int chunks_per_row = d / 8;
  for (int idx = threadIdx.x; idx < RWS * chunks_per_row; idx += blockDim.x) {
    const int r = idx / chunks_per_row, c = idx - r * chunks_per_row;
    const int tok = r / p.gh, hh = chunk * p.gh + (r - tok * p.gh);
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (tok < n_tok && hh < p.nh)
      v = *reinterpret_cast<const uint4*>(p.q + (size_t)(q_begin + q0 + tok) * p.q_stride + (size_t)hh * d + c * 8);
    *reinterpret_cast<uint4*>(smem_raw + (size_t)r * row_bytes + (size_t)c * 16) = v;
  }

  const int* bt = p.block_tables + (size_t)b * p.bt_stride;
  // a warp brings 8 keys of a tile, its lanes the 16-byte chunks of a row: the page of a key is looked up once a key
  auto load_tile = [&](int stage, int t0) {
    const uint32_t dst0 = ks0 + stage * k_stage;
#pragma unroll 2
    for (int i = 0; i < BN / (WARPS * MT); ++i) {
      const int key = warp * (BN / (WARPS * MT)) + i;
      const int kp = t0 + key;
      const int page = p.bs_shift >= 0 ? kp >> p.bs_shift : kp / p.block_size;
      const int off = p.bs_shift >= 0 ? kp & (p.block_size - 1) : kp - page * p.block_size;
      const int blk = kp < ctx ? bt[page] : -1;  // a page given back lies outside every window: zeros
      const bool valid = blk >= 0;
      const bf16* src = p.cache + (valid ? ((size_t)blk * p.block_size + (size_t)off) * d : 0);
      const uint32_t dst = dst0 + key * row_bytes;
      for (int c = lane; c < chunks_per_row; c += 32) cpa16(dst + c * 16, src + (valid ? c * 8 : 0), valid);
    }
  };

  // the two rows of every m-tile that a thread holds: lane/4 and lane/4 + 8
  int pos[ML][2];
  float o[ML][NTW][4], m[ML][2], l[ML][2];
#pragma unroll
  for (int mt = 0; mt < ML; ++mt) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = (group + mt) * ROWS + (lane >> 2) + 8 * h;
      const int tok = r / p.gh, hh = chunk * p.gh + (r - tok * p.gh);
      pos[mt][h] = (tok < n_tok && hh < p.nh) ? p_first + tok : -1;  // -1: sees nothing
      m[mt][h] = -INFINITY;
      l[mt][h] = 0.f;
    }
#pragma unroll
    for (int j = 0; j < NTW; ++j) o[mt][j][0] = o[mt][j][1] = o[mt][j][2] = o[mt][j][3] = 0.f;
  }

  const int n_ksteps = d / 16;
  const int ks_begin = (w4 * n_ksteps) / WARPS, ks_end = ((w4 + 1) * n_ksteps) / WARPS;
  const int mi = lane >> 3, l7 = lane & 7;
  const int n_tiles = (kv_hi - kv_lo + BN - 1) / BN;
  load_tile(0, kv_lo);
  cpa_commit();
  for (int t = 0; t < n_tiles; ++t) {
    const int st = t & 1;
    if (t + 1 < n_tiles) {
      load_tile(st ^ 1, kv_lo + (t + 1) * BN);
      cpa_commit();
      cpa_wait<1>();
    } else {
      cpa_wait<0>();
    }
    __syncthreads();  // the tile (and, the first time, the query rows) are in shared memory
    const uint32_t ks = ks0 + st * k_stage;
    // ---- this warp's share of the k-steps of q . k
    float s[ML][4][4];
#pragma unroll
    for (int mt = 0; mt < ML; ++mt)
#pragma unroll
      for (int j = 0; j < 4; ++j) s[mt][j][0] = s[mt][j][1] = s[mt][j][2] = s[mt][j][3] = 0.f;
    for (int kk = ks_begin; kk < ks_end; ++kk) {
      uint32_t a[ML][4];
#pragma unroll
      for (int mt = 0; mt < ML; ++mt)
        ldsm_x4(a[mt], qs + (uint32_t)((group + mt) * ROWS + (mi & 1) * 8 + l7) * row_bytes + (uint32_t)(kk * 16 + (mi >> 1) * 8) * 2);
#pragma unroll
      for (int jp = 0; jp < 4; jp += 2) {
        uint32_t bq[4];
        ldsm_x4(bq, ks + (uint32_t)((jp + (mi >> 1)) * 8 + l7) * row_bytes + (uint32_t)(kk * 16 + (mi & 1) * 8) * 2);
#pragma unroll
        for (int mt = 0; mt < ML; ++mt) {
          mma16816(s[mt][jp], a[mt], bq[0], bq[1]);
          mma16816(s[mt][jp + 1], a[mt], bq[2], bq[3]);
        }
      }
    }
#pragma unroll
    for (int mt = 0; mt < ML; ++mt)
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) sp[((((group + mt) * WARPS + w4) * 4 + j) * 4 + e) * 32 + lane] = s[mt][j][e];
    __syncthreads();
#pragma unroll
    for (int mt = 0; mt < ML; ++mt)
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float v = 0.f;
#pragma unroll
          for (int w = 0; w < WARPS; ++w) v += sp[((((group + mt) * WARPS + w) * 4 + j) * 4 + e) * 32 + lane];  // warp order: reproducible
          s[mt][j][e] = v;
        }
    // ---- mask, running maximum, exponentials, running sum
    const int key0 = kv_lo + t * BN;
#pragma unroll
    for (int mt = 0; mt < ML; ++mt) {
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int r = e >> 1;
          const int kp = key0 + j * 8 + ((lane & 3) << 1) + (e & 1);
          bool vis = (kp <= pos[mt][r]) && (kp < kv_hi);
          if (p.window > 0) vis = vis && (kp > pos[mt][r] - p.window);
          const float v = vis ? s[mt][j][e] * p.scale_log2 : -INFINITY;
          s[mt][j][e] = v;
          mx[r] = fmaxf(mx[r], v);
        }
      float corr[2], m_use[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        const float m_new = fmaxf(m[mt][r], mx[r]);
        m_use[r] = (m_new == -INFINITY) ? 0.f : m_new;  // a row that has seen nothing yet
        corr[r] = ex2(m[mt][r] - m_use[r]);
        m[mt][r] = m_new;
      }
      float sum[2] = {0.f, 0.f};
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float pv = ex2(s[mt][j][e] - m_use[e >> 1]);
          s[mt][j][e] = pv;
          sum[e >> 1] += pv;
        }
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 1);
        sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 2);
        l[mt][r] = l[mt][r] * corr[r] + sum[r];
      }
#pragma unroll
      for (int j = 0; j < NTW; ++j) {
        o[mt][j][0] *= corr[0];
        o[mt][j][1] *= corr[0];
        o[mt][j][2] *= corr[1];
        o[mt][j][3] *= corr[1];
      }
    }
    // ---- O += P V over this warp's columns; the value tile is the key tile's first dv columns
    const int col0 = w4 * NTW * 8;
#pragma unroll
    for (int kk = 0; kk < BN / 16; ++kk) {
      uint32_t a[ML][4];
#pragma unroll
      for (int mt = 0; mt < ML; ++mt) {
        a[mt][0] = pack2(s[mt][2 * kk][0], s[mt][2 * kk][1]);
        a[mt][1] = pack2(s[mt][2 * kk][2], s[mt][2 * kk][3]);
        a[mt][2] = pack2(s[mt][2 * kk + 1][0], s[mt][2 * kk + 1][1]);
        a[mt][3] = pack2(s[mt][2 * kk + 1][2], s[mt][2 * kk + 1][3]);
      }
#pragma unroll
      for (int nt = 0; nt < NTW; nt += 2) {
        uint32_t bv[4];
        // four 8 x 8 blocks: (keys 0-7 | 8-15) x (columns n0.. | n0+8..), read transposed
        ldsm_x4_trans(bv, ks + (uint32_t)(kk * 16 + (mi & 1) * 8 + l7) * row_bytes + (uint32_t)(col0 + nt * 8 + (mi >> 1) * 8) * 2);
#pragma unroll
        for (int mt = 0; mt < ML; ++mt) {
          mma16816(o[mt][nt], a[mt], bv[0], bv[1]);
          if (nt + 1 < NTW) mma16816(o[mt][nt + 1], a[mt], bv[2], bv[3]);
        }
      }
    }
    __syncthreads();  // the stage and the partial sums are free again
  }

  // ---- write
#pragma unroll
  for (int mt = 0; mt < ML; ++mt) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      if (pos[mt][h] < 0) continue;
      const int r = (group + mt) * ROWS + (lane >> 2) + 8 * h;
      const int tok = r / p.gh, head = chunk * p.gh + (r - tok * p.gh);
      const int col = w4 * NTW * 8 + ((lane & 3) << 1);
      if (SPLIT) {
        const size_t slot = ((size_t)b * p.nh + head) * p.max_splits + blockIdx.x;
        if (w4 == 0 && (lane & 3) == 0) {
          p.part_ml[slot * 2] = m[mt][h] * 0.69314718055994531f;  // natural-log units, as the merge reads them
          p.part_ml[slot * 2 + 1] = l[mt][h];
        }
#pragma unroll
        for (int j = 0; j < NTW; ++j) {
          p.part_acc[slot * p.dv + col + j * 8] = o[mt][j][2 * h];
          p.part_acc[slot * p.dv + col + j * 8 + 1] = o[mt][j][2 * h + 1];
        }
      } else {
        const float inv = l[mt][h] > 0.f ? 1.f / l[mt][h] : 0.f;
        bf16* dst = p.out + (size_t)(q_begin + q0 + tok) * p.out_stride + (size_t)head * p.dv + col;
#pragma unroll
        for (int j = 0; j < NTW; ++j) *reinterpret_cast<uint32_t*>(dst + j * 8) = pack2(o[mt][j][2 * h] * inv, o[mt][j][2 * h + 1] * inv);
      }
    }
  }
}

// Merge the partial results of the key ranges of one (sequence, head), in range order.
__global__ void latent_combine_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml, bf16* __restrict__ out,
                                      const int* __restrict__ qsl, const int* __restrict__ ctx_lens, int nh, int dv, int out_stride,
                                      int split_size, int max_splits) {
  pdl_launch();
  pdl_wait();
  const int b = blockIdx.y, head = blockIdx.x;
  const int q_begin = qsl[b], q_len = qsl[b + 1] - q_begin;
  const int ctx = ctx_lens[b];
  if (q_len <= 0 || ctx <= 0) return;
  const int ns = min(max_splits, (ctx + split_size - 1) / split_size);
  const size_t base = ((size_t)b * nh + head) * max_splits;
  float M = -INFINITY;
  for (int s = 0; s < ns; ++s) M = fmaxf(M, part_ml[(base + s) * 2]);
  float L = 0.f;
  for (int s = 0; s < ns; ++s) {
    const float ms = part_ml[(base + s) * 2];
    if (ms != -INFINITY) L += expf(ms - M) * part_ml[(base + s) * 2 + 1];
  }
  const float inv = L > 0.f ? 1.f / L : 0.f;
  bf16* o = out + (size_t)(q_begin + q_len - 1) * out_stride + (size_t)head * dv;
  for (int j = threadIdx.x; j < dv; j += blockDim.x) {
    float a = 0.f;
    for (int s = 0; s < ns; ++s) {
      const float ms = part_ml[(base + s) * 2];
      if (ms != -INFINITY) a += expf(ms - M) * part_acc[(base + s) * dv + j];
    }
    o[j] = __float2bfloat16_rn(a * inv);
  }
}

template <int NTW, int MT>
int launch_tiles(const LatParams& p, int B, int max_q_len, cudaStream_t st) {
  const size_t smem = (size_t)(ROWS * MT + 2 * BN) * (p.d + PAD) * 2 + (size_t)WARPS * MT * 16 * 32 * sizeof(float);
  auto kern = latent_attn_kernel<NTW, MT, false>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  return launch(kern, dim3((max_q_len + p.tq - 1) / p.tq, B, p.chunks), dim3(WARPS * 32 * MT), smem, st, p);
}

template <int NTW>
int launch_latent(LatParams p, int B, int max_q_len, int grid_splits, cudaStream_t st) {
  const size_t smem = (size_t)(ROWS + 2 * BN) * (p.d + PAD) * 2 + (size_t)WARPS * 16 * 32 * sizeof(float);
  if (p.split_size > 0) {
    auto kern = latent_attn_kernel<NTW, 1, true>;
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
    }
    int rc = launch(kern, dim3(grid_splits, B, p.chunks), dim3(WARPS * 32), smem, st, p);
    if (rc) return rc;
    return launch(latent_combine_kernel, dim3(p.nh, B), dim3(128), 0, st, (const float*)p.part_acc, (const float*)p.part_ml, p.out,
                  p.qsl, p.ctx_lens, p.nh, p.dv, p.out_stride, p.split_size, p.max_splits);
  }
  // 64 or 32 rows a CTA (16 or 8 warps) where some sequence brings enough tokens to fill them
  for (int mt = 4; mt >= 2; mt >>= 1) {
    const int rows = mt * ROWS;
    const int gh = p.nh < rows ? p.nh : rows;
    const int tq = rows / gh;
    if (tq < 1 || max_q_len < tq || tq <= p.tq) continue;
    if ((size_t)(rows + 2 * BN) * (p.d + PAD) * 2 + (size_t)WARPS * mt * 16 * 32 * sizeof(float) > 220 * 1024) continue;
    p.gh = gh;
    p.chunks = (p.nh + gh - 1) / gh;
    p.tq = tq;
    return mt == 4 ? launch_tiles<NTW, 4>(p, B, max_q_len, st) : launch_tiles<NTW, 2>(p, B, max_q_len, st);
  }
  return launch_tiles<NTW, 1>(p, B, max_q_len, st);
}

}  // namespace

// q: rows of q_stride elements whose first nh * d are the query heads; out [N, nh * dv]; cache
// [blocks][1][block_size][d].  split_size > 0: the split form (one query a sequence; split_size a multiple of 32;
// scratch for max_splits ranges per (sequence, head); grid_splits of them are launched).  Shapes this kernel
// does not take are refused with cudaErrorInvalidValue.
KVF_API int kvf_latent_attention_bf16(const void* q, void* out, const void* cache, const int* block_tables, const int* qsl,
                                      const int* ctx_lens, int B, int max_q_len, int q_stride, int out_stride, int bt_stride,
                                      int nh, int d, int dv, int block_size, float scale, int window, int split_size,
                                      int max_splits, int grid_splits, float* part_acc, float* part_ml, cudaStream_t st) {
  if (B <= 0 || max_q_len <= 0) return 0;
  if (d <= 0 || d > 1024 || (d % 16) || dv <= 0 || (dv % 32) || dv > d || nh <= 0 || block_size <= 0) return (int)cudaErrorInvalidValue;
  if ((q_stride & 7) || (out_stride & 1) || ((((uintptr_t)q) | ((uintptr_t)cache)) & 15) || (((uintptr_t)out) & 3))
    return (int)cudaErrorInvalidValue;
  LatParams p;
  p.q = (const bf16*)q; p.out = (bf16*)out; p.cache = (const bf16*)cache;
  p.block_tables = block_tables; p.qsl = qsl; p.ctx_lens = ctx_lens;
  p.part_acc = part_acc; p.part_ml = part_ml;
  p.q_stride = q_stride; p.out_stride = out_stride; p.bt_stride = bt_stride;
  p.nh = nh; p.d = d; p.dv = dv; p.block_size = block_size;
  p.gh = nh < ROWS ? nh : ROWS;
  p.chunks = (nh + p.gh - 1) / p.gh;
  p.tq = ROWS / p.gh;
  p.bs_shift = -1;
  for (int sh = 0; sh < 31; ++sh)
    if ((1 << sh) == block_size) p.bs_shift = sh;
  p.window = window; p.split_size = split_size; p.max_splits = max_splits;
  p.scale_log2 = scale * 1.4426950408889634f;
  if ((unsigned)B > 65535u || (unsigned)p.chunks > 65535u) return (int)cudaErrorInvalidValue;
  if (split_size > 0) {
    if (split_size % BN || max_splits <= 0 || !part_acc || !part_ml || max_q_len != 1) return (int)cudaErrorInvalidValue;
    p.tq = 1;
    grid_splits = grid_splits > 0 && grid_splits < max_splits ? grid_splits : max_splits;
  }
  switch (dv / 32) {
    case 2: return launch_latent<2>(p, B, max_q_len, grid_splits, st);
    case 3: return launch_latent<3>(p, B, max_q_len, grid_splits, st);
    case 4: return launch_latent<4>(p, B, max_q_len, grid_splits, st);
    case 8: return launch_latent<8>(p, B, max_q_len, grid_splits, st);
    case 16: return launch_latent<16>(p, B, max_q_len, grid_splits, st);
    default: return (int)cudaErrorInvalidValue;
  }
}
