// Softmax attention over the paged cache with the masks and score terms that grouped-query and latent attention designs combine:
//
//   score(i, j) = scale * (q_i . k_j) - slope_h * (i - j)                 slope_h = 0: no distance term
//   i sees j    if j <= i and (window = 0 or i - j < window or j < keep_first) and (chunk = 0 or floor(i / chunk) = floor(j / chunk))
//   o_i         = sum_j exp(score(i, j) - m) v_j / (sum_j exp(score(i, j) - m) + exp(sink_h - m))      without a sink: no second term
//
// Query head h reads key/value head h / (H / G). The key size D and the value size Dv may differ; a token's values lie `v_offset`
// elements from its key in the page (the second plane of a page with two planes, or 0: the values are the leading Dv elements of the
// key row itself, as in latent attention with the key projection taken into the query). Scores, weights and sums are 32-bit
// whatever the storage. Kept tokens keep their positions: the distance term and the causal rule use i - j as it is.
//
// Kernels in front prepare a step's tokens: `qkv_norm_append_kernel` (bias, an RMS norm over the whole query projection and
// over the whole key projection, append), `latent_prepare_kernel` (the two latents of latent attention normed, the shared rotated key
// part, append of one row per token), `rotate_heads_kernel` (rotation of a slice of every query head) and `head_linear_kernel` (a
// matrix per head: the key projection taken into the queries in front of the attention, the value projection behind it).
#include "common.cuh"
#include "step_ops.h"

SB_DEFINE_LAST_ERROR()

namespace {

using bf16 = __nv_bfloat16;
constexpr int kInFlight = 8;

__device__ __forceinline__ float folded(const float* p, int n_partials, int64_t stride) {
  float part[kInFlight];
#pragma unroll
  for (int s = 0; s < kInFlight; ++s)
    if (s < n_partials) part[s] = p[s * stride];
  float sum = part[0];
#pragma unroll
  for (int s = 1; s < kInFlight; ++s)
    if (s < n_partials) sum += part[s];
  for (int s = kInFlight; s < n_partials; ++s) sum += p[s * stride];
  return sum;
}

struct PageRef {
  void* pages;               // [pages][planes][Hkv][page_size][Dc]
  const int32_t* block_table;
  int max_pages, page_size;
  int64_t page_stride, v_offset, head_stride;
  int Dc;
};

struct NormAppendParams {
  const float* qkv;          // [P][n][Hq D + Hkv D + Hkv Dv]
  int n_partials;
  int64_t partial_stride;
  const float* bias;         // [width] or null
  const float* q_gain;       // [Hq D] or null: no norm of the queries
  const float* k_gain;       // [Hkv D] or null
  float eps;
  const int32_t* positions;
  const int32_t* slots;
  void* q_out;               // [n][Hq D]
  PageRef c;
  int Hq, Hkv, D, Dv;
  int write_kv;
};

// A block per token. The row (partial sums folded, bias added) stays in shared memory between the two sums of squares and the stores.
template <class T>
__global__ void __launch_bounds__(256) qkv_norm_append_kernel(NormAppendParams p) {
  extern __shared__ float row_values[];
  __shared__ float red[32];
  sb::grid_launch_dependents();
  const int row = blockIdx.x;
  const int nq = p.Hq * p.D, nk = p.Hkv * p.D, width = nq + nk + p.Hkv * p.Dv;
  const int pos = p.positions[row], slot = p.slots[row];
  const int page = p.write_kv ? p.c.block_table[static_cast<int64_t>(slot) * p.c.max_pages + pos / p.c.page_size] : 0;
  sb::grid_dependency_wait();
  const float* src = p.qkv + static_cast<int64_t>(row) * width;
  float sq_q = 0.0f, sq_k = 0.0f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float v = folded(src + i, p.n_partials, p.partial_stride);
    if (p.bias != nullptr) v = __fadd_rn(v, p.bias[i]);
    row_values[i] = v;
    if (i < nq) sq_q = fmaf(v, v, sq_q);
    else if (i < nq + nk) sq_k = fmaf(v, v, sq_k);
  }
  const float rq = p.q_gain != nullptr ? 1.0f / sqrtf(sb::block_sum(sq_q, red) / static_cast<float>(nq) + p.eps) : 1.0f;
  const float rk = p.k_gain != nullptr ? 1.0f / sqrtf(sb::block_sum(sq_k, red) / static_cast<float>(nk) + p.eps) : 1.0f;
  T* pages = static_cast<T*>(p.c.pages);
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float v = row_values[i];
    if (i < nq) {
      if (p.q_gain != nullptr) v = __fmul_rn(__fmul_rn(v, rq), p.q_gain[i]);
      static_cast<T*>(p.q_out)[static_cast<int64_t>(row) * nq + i] = sb::narrow<T>(v);
    } else if (p.write_kv) {
      const bool is_v = i >= nq + nk;
      if (!is_v && p.k_gain != nullptr) v = __fmul_rn(__fmul_rn(v, rk), p.k_gain[i - nq]);
      const int e = is_v ? i - nq - nk : i - nq;
      const int dim = is_v ? p.Dv : p.D, head = e / dim, d = e % dim;
      pages[static_cast<int64_t>(page) * p.c.page_stride + (is_v ? p.c.v_offset : 0) + static_cast<int64_t>(head) * p.c.head_stride +
            static_cast<int64_t>(pos % p.c.page_size) * p.c.Dc + d] = sb::narrow<T>(v);
    }
  }
}

struct LatentParams {
  const float* proj;         // [P][n][Rq + Rkv + rot]: the query latent, the key/value latent, the shared rotated key part
  int n_partials;
  int64_t partial_stride;
  const float* q_gain;       // [Rq]
  const float* kv_gain;      // [Rkv]
  float eps;
  const int32_t* positions;
  const int32_t* slots;
  const float* cos_sin;      // [positions][rot / 2][2]
  void* q_latent;            // [n][Rq]
  PageRef c;                 // one row per token: [Rkv latent | rot rotated key]
  int Rq, Rkv, rot;
  int write_kv;
};

// A block per token: both latents RMS-normed with their gains; the last `rot` elements rotated (pairs d, d + rot / 2) by the token's
// position and stored behind the key/value latent in the token's page row.
template <class T>
__global__ void __launch_bounds__(256) latent_prepare_kernel(LatentParams p) {
  extern __shared__ float row_values[];
  __shared__ float red[32];
  sb::grid_launch_dependents();
  const int row = blockIdx.x;
  const int width = p.Rq + p.Rkv + p.rot;
  const int pos = p.positions[row], slot = p.slots[row];
  const int page = p.write_kv ? p.c.block_table[static_cast<int64_t>(slot) * p.c.max_pages + pos / p.c.page_size] : 0;
  sb::grid_dependency_wait();
  const float* src = p.proj + static_cast<int64_t>(row) * width;
  float sq_q = 0.0f, sq_kv = 0.0f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float v = folded(src + i, p.n_partials, p.partial_stride);
    row_values[i] = v;
    if (i < p.Rq) sq_q = fmaf(v, v, sq_q);
    else if (i < p.Rq + p.Rkv) sq_kv = fmaf(v, v, sq_kv);
  }
  const float rq = 1.0f / sqrtf(sb::block_sum(sq_q, red) / static_cast<float>(p.Rq) + p.eps);
  const float rkv = 1.0f / sqrtf(sb::block_sum(sq_kv, red) / static_cast<float>(p.Rkv) + p.eps);
  T* dst = static_cast<T*>(p.c.pages) + static_cast<int64_t>(page) * p.c.page_stride + static_cast<int64_t>(pos % p.c.page_size) * p.c.Dc;
  const int rh = p.rot / 2;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float v = row_values[i];
    if (i < p.Rq) {
      static_cast<T*>(p.q_latent)[static_cast<int64_t>(row) * p.Rq + i] = sb::narrow<T>(__fmul_rn(__fmul_rn(v, rq), p.q_gain[i]));
    } else if (!p.write_kv) {
      continue;
    } else if (i < p.Rq + p.Rkv) {
      dst[i - p.Rq] = sb::narrow<T>(__fmul_rn(__fmul_rn(v, rkv), p.kv_gain[i - p.Rq]));
    } else {
      const int d = i - p.Rq - p.Rkv;
      const bool low = d < rh;
      const int j = low ? d : d - rh;
      const float b = row_values[low ? i + rh : i - rh];
      const float2 cs = *reinterpret_cast<const float2*>(p.cos_sin + (static_cast<int64_t>(pos) * rh + j) * 2);
      // (u, v) -> (u cos - v sin, v cos + u sin): the low element is u, the high one v
      const float r = low ? __fsub_rn(__fmul_rn(v, cs.x), __fmul_rn(b, cs.y)) : __fadd_rn(__fmul_rn(v, cs.x), __fmul_rn(b, cs.y));
      dst[p.Rkv + d] = sb::narrow<T>(r);
    }
  }
}

// q [P][n][H D] partial sums -> out [n][H D]: elements offset .. offset + rot - 1 of every head rotated by the token's position, the
// others passed on.
template <class T>
__global__ void rotate_heads_kernel(const float* __restrict__ q, int n_partials, int64_t partial_stride, const int32_t* __restrict__ positions,
                                    const float* __restrict__ cos_sin, T* __restrict__ out, int H, int D, int offset, int rot) {
  sb::grid_launch_dependents();
  const int row = blockIdx.x, item = blockIdx.y * blockDim.x + threadIdx.x;
  const int pos = positions[row];
  sb::grid_dependency_wait();
  if (item >= H * D) return;
  const float* src = q + static_cast<int64_t>(row) * H * D;
  float a = folded(src + item, n_partials, partial_stride);
  const int d = item % D - offset, rh = rot / 2;
  if (d >= 0 && d < rot) {
    const bool low = d < rh;
    const int j = low ? d : d - rh;
    const float b = folded(src + (low ? item + rh : item - rh), n_partials, partial_stride);
    const float2 cs = *reinterpret_cast<const float2*>(cos_sin + (static_cast<int64_t>(pos) * rh + j) * 2);
    a = low ? __fsub_rn(__fmul_rn(a, cs.x), __fmul_rn(b, cs.y)) : __fadd_rn(__fmul_rn(a, cs.x), __fmul_rn(b, cs.y));
  }
  out[static_cast<int64_t>(row) * H * D + item] = sb::narrow<T>(a);
}

struct HeadLinearParams {
  const void* in;            // row r, head h: in + r in_row + h in_head, K elements (and `tail` more behind them)
  int64_t in_row, in_head;
  const void* w;             // [H][K][N]
  void* out;                 // row r, head h: out + r out_row + h out_head, N elements (and the tail behind them)
  int64_t out_row, out_head;
  int n, H, K, N, tail;
};

// out[r, h, :N] = W_h^T in[r, h, :K], a matrix per head; the `tail` elements behind the K pass unchanged. A block is TR rows of one head: the
// rows wait in shared memory, a thread owns output columns and walks K in ascending order, so a row's result does not depend on its
// neighbours. Sums in 32-bit.
template <class T, int TR>
__global__ void __launch_bounds__(128) head_linear_kernel(HeadLinearParams p) {
  extern __shared__ float rows_in[];       // [TR][K]
  sb::grid_launch_dependents();
  const int h = blockIdx.y, r0 = blockIdx.x * TR;
  const T* in = static_cast<const T*>(p.in) + static_cast<int64_t>(h) * p.in_head;
  T* out = static_cast<T*>(p.out) + static_cast<int64_t>(h) * p.out_head;
  const T* w = static_cast<const T*>(p.w) + static_cast<int64_t>(h) * p.K * p.N;
  sb::grid_dependency_wait();
  for (int i = threadIdx.x; i < TR * p.K; i += blockDim.x) {
    const int r = i / p.K, k = i % p.K;
    rows_in[i] = r0 + r < p.n ? sb::widen(in[static_cast<int64_t>(r0 + r) * p.in_row + k]) : 0.0f;
  }
  for (int i = threadIdx.x; i < TR * p.tail; i += blockDim.x) {
    const int r = i / p.tail, t = i % p.tail;
    if (r0 + r < p.n) out[static_cast<int64_t>(r0 + r) * p.out_row + p.N + t] = in[static_cast<int64_t>(r0 + r) * p.in_row + p.K + t];
  }
  __syncthreads();
  for (int j = threadIdx.x; j < p.N; j += blockDim.x) {
    float acc[TR];
#pragma unroll
    for (int r = 0; r < TR; ++r) acc[r] = 0.0f;
    for (int k = 0; k < p.K; ++k) {
      const float wv = sb::widen(w[static_cast<int64_t>(k) * p.N + j]);
#pragma unroll
      for (int r = 0; r < TR; ++r) acc[r] = fmaf(rows_in[r * p.K + k], wv, acc[r]);
    }
#pragma unroll
    for (int r = 0; r < TR; ++r)
      if (r0 + r < p.n) out[static_cast<int64_t>(r0 + r) * p.out_row + j] = sb::narrow<T>(acc[r]);
  }
}

struct AttnParams {
  const void* q;             // [n][H D]
  void* out;                 // [n][H Dv]
  const void* pages;
  const int32_t* block_table;
  int max_pages, page_size;
  int64_t page_stride, v_offset, head_stride;
  const int32_t* positions;
  const int32_t* slots;
  const float* slopes;       // [H] float32, or null
  const float* sinks;        // [H] float32, or null
  int H, G, D, Dv, Dc;
  int window, keep_first;
  float scale;
  int chunk;                 // > 0: a row sees only the keys of its own chunk of this many positions (borders at multiples of it)
  int out_f32;               // 1: `out` is float32 whatever the storage of q and the cache
};

constexpr int kWarps = 4;

// One block per (token, head), a warp per class of keys j % 4; every warp keeps a running (max, sum, weighted values) over its keys in
// ascending order, and the four are joined at the end, with the sink. PER: elements of a row a lane holds (sizes up to 32 PER).
template <class T, int PER>
__global__ void __launch_bounds__(kWarps * 32) masked_attention_kernel(AttnParams p) {
  extern __shared__ __align__(16) float smem[];       // q [D], then the classes' sums [kWarps][Dv], maxima and sums [2][kWarps]
  sb::grid_launch_dependents();
  const int row = blockIdx.x, h = blockIdx.y, g = h / (p.H / p.G);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pos = p.positions[row], slot = p.slots[row];
  const int first = max(p.window > 0 ? max(0, pos - p.window + 1) : 0, p.chunk > 0 ? pos / p.chunk * p.chunk : 0);
  const int kept_end = p.window > 0 ? min(p.keep_first, first) : 0;      // keys 0 .. kept_end - 1 lie in front of the window and are seen
  const float slope = p.slopes != nullptr ? p.slopes[h] : 0.0f;
  const int32_t* table = p.block_table + static_cast<int64_t>(slot) * p.max_pages;
  float* sq = smem;
  float* sums = smem + p.D;
  float* ml = sums + kWarps * p.Dv;
  sb::grid_dependency_wait();
  const T* q = static_cast<const T*>(p.q) + (static_cast<int64_t>(row) * p.H + h) * p.D;
  for (int d = threadIdx.x; d < p.D; d += blockDim.x) sq[d] = sb::widen(q[d]);
  __syncthreads();
  float qr[PER], acc[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    qr[i] = lane + 32 * i < p.D ? sq[lane + 32 * i] : 0.0f;
    acc[i] = 0.0f;
  }
  const T* base = static_cast<const T*>(p.pages) + static_cast<int64_t>(g) * p.head_stride;
  float m = -INFINITY, l = 0.0f;
  auto take = [&](int j) {
    const T* k = base + static_cast<int64_t>(table[j / p.page_size]) * p.page_stride + static_cast<int64_t>(j % p.page_size) * p.Dc;
    const T* v = k + p.v_offset;
    float dot = 0.0f, vr[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      if (lane + 32 * i < p.D) dot = fmaf(qr[i], sb::widen(k[lane + 32 * i]), dot);
      vr[i] = lane + 32 * i < p.Dv ? sb::widen(v[lane + 32 * i]) : 0.0f;
    }
    for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    const float s = __fsub_rn(__fmul_rn(dot, p.scale), __fmul_rn(slope, static_cast<float>(pos - j)));
    const float m_new = fmaxf(m, s);
    const float f = expf(m - m_new), w = expf(s - m_new);       // (m = -inf at the first key: f = 0)
    l = fmaf(l, f, w);
#pragma unroll
    for (int i = 0; i < PER; ++i) acc[i] = fmaf(acc[i], f, w * vr[i]);
    m = m_new;
  };
  for (int j = warp; j < kept_end; j += kWarps) take(j);
  for (int j = first + ((warp - first) % kWarps + kWarps) % kWarps; j <= pos; j += kWarps) take(j);
#pragma unroll
  for (int i = 0; i < PER; ++i)
    if (lane + 32 * i < p.Dv) sums[warp * p.Dv + lane + 32 * i] = acc[i];
  if (lane == 0) ml[warp] = m, ml[kWarps + warp] = l;
  __syncthreads();
  float top = p.sinks != nullptr ? p.sinks[h] : -INFINITY;
  for (int c = 0; c < kWarps; ++c) top = fmaxf(top, ml[c]);
  float factor[kWarps], total = p.sinks != nullptr ? expf(p.sinks[h] - top) : 0.0f;
  for (int c = 0; c < kWarps; ++c) {
    factor[c] = expf(ml[c] - top);
    total = fmaf(ml[kWarps + c], factor[c], total);
  }
  const int64_t at = (static_cast<int64_t>(row) * p.H + h) * p.Dv;
  for (int d = threadIdx.x; d < p.Dv; d += blockDim.x) {
    float o = 0.0f;
    for (int c = 0; c < kWarps; ++c) o = fmaf(sums[c * p.Dv + d], factor[c], o);
    if (p.out_f32) static_cast<float*>(p.out)[at + d] = o / total;
    else static_cast<T*>(p.out)[at + d] = sb::narrow<T>(o / total);
  }
}

// ---------------------------------------------------------------------------------------------------------------------------------
// The bfloat16 form on the tensor cores (mma.sync.m16n8k16, float32 accumulation). The four warps of a CTA share one tile of 16 rows of
// one key/value head: 16 / Ht consecutive positions of an entry times Ht query heads of the group (Ht = the group, or 16 of a larger
// group). They walk the tiles of 64 keys (cut by ABSOLUTE position) that any row sees: the kept first tokens, then the window. In a tile
// warp w makes the scores of keys 16 w .. 16 w + 15; the rows' maxima over the tile are exchanged through shared memory and every warp
// keeps the same running maximum per row; the weights exp(score - max) in 32-bit, split into two bfloat16 parts hi + lo, are the A operand
// of step w of the value product, handed to the other warps through shared memory; warp w owns the value columns 16 (w + 4 i) .. and
// rescales them when the maximum moves. A key that a row does not see has weight 0 and a tile in which a row sees nothing leaves its
// maximum alone, so a row's result depends on its own position only: a token has the same bits in a prompt, in a portion and decoded
// alone. With `v_offset` 0 the values are the leading columns of the staged key rows and are not staged again.

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(static_cast<uint32_t>(__cvta_generic_to_shared(p))));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(static_cast<uint32_t>(__cvta_generic_to_shared(p))));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float x, float y) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(x, y);
  return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ void copy16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(dst))), "l"(src) : "memory");
}

// The matrix per head on the tensor cores (bfloat16, mma.sync.m16n8k16, float32 accumulation). A CTA of four warps makes 64 rows x 64
// columns of one head; warp w owns rows 16 w .. 16 w + 15. K is walked in chunks of 64, staged twice over with cp.async: the rows' slice
// [64][64] and the weights' slice [64 k][64 n], n contiguous as stored, read as the B operand through ldmatrix.trans. A row's sum runs
// over k in ascending steps of 16 whatever its neighbours are, so a token has the same bits in a prompt, in a portion and decoded alone.
constexpr int kHlTile = 64, kHlLd = kHlTile + 8;

__global__ void __launch_bounds__(128) head_linear_tc_kernel(HeadLinearParams p) {
  __shared__ __align__(16) bf16 As[2][kHlTile * kHlLd];
  __shared__ __align__(16) bf16 Bs[2][kHlTile * kHlLd];
  sb::grid_launch_dependents();
  const int h = blockIdx.y, r0 = blockIdx.x * kHlTile, n0 = blockIdx.z * kHlTile;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bf16* in = static_cast<const bf16*>(p.in) + static_cast<int64_t>(h) * p.in_head;
  bf16* out = static_cast<bf16*>(p.out) + static_cast<int64_t>(h) * p.out_head;
  const bf16* w = static_cast<const bf16*>(p.w) + static_cast<int64_t>(h) * p.K * p.N;
  sb::grid_dependency_wait();
  auto request = [&](int kc, int buf) {
    for (int i = threadIdx.x; i < kHlTile * 8; i += blockDim.x) {
      const int r = i >> 3, c = (i & 7) * 8, k = kc * kHlTile + c;
      bf16* a = &As[buf][r * kHlLd + c];
      if (r0 + r < p.n && k < p.K) copy16(a, in + static_cast<int64_t>(r0 + r) * p.in_row + k);
      else *reinterpret_cast<uint4*>(a) = make_uint4(0, 0, 0, 0);
      bf16* b = &Bs[buf][r * kHlLd + c];                       // here r is the k of the chunk and c the column of the slice
      if (kc * kHlTile + r < p.K && n0 + c < p.N) copy16(b, w + static_cast<int64_t>(kc * kHlTile + r) * p.N + n0 + c);
      else *reinterpret_cast<uint4*>(b) = make_uint4(0, 0, 0, 0);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  if (blockIdx.z == 0)
    for (int i = threadIdx.x; i < kHlTile * p.tail; i += blockDim.x) {
      const int r = i / p.tail, t = i % p.tail;
      if (r0 + r < p.n) out[static_cast<int64_t>(r0 + r) * p.out_row + p.N + t] = in[static_cast<int64_t>(r0 + r) * p.in_row + p.K + t];
    }
  float acc[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.0f;
  const int chunks = (p.K + kHlTile - 1) / kHlTile;
  request(0, 0);
  for (int kc = 0; kc < chunks; ++kc) {
    const int buf = kc & 1;
    if (kc + 1 < chunks) {
      request(kc + 1, buf ^ 1);            // (the buffer of the chunk before: every warp left it before the barrier at the end of that chunk)
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kHlTile / 16; ++kk) {
      uint32_t a[4];
      ldmatrix_x4(a, &As[buf][(warp * 16 + (lane & 15)) * kHlLd + kk * 16 + (lane >> 4) * 8]);
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        uint32_t b[4];
        ldmatrix_x4_trans(b, &Bs[buf][(kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * kHlLd + nt * 16 + (lane >> 4) * 8]);
        mma_bf16(acc[2 * nt], a, b[0], b[1]);
        mma_bf16(acc[2 * nt + 1], a, b[2], b[3]);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int r = r0 + warp * 16 + (lane >> 2) + half * 8;
    if (r >= p.n) continue;
    bf16* dst = out + static_cast<int64_t>(r) * p.out_row + n0 + (lane & 3) * 2;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int c = (i >> 1) * 16 + (i & 1) * 8;
      if (n0 + c + (lane & 3) * 2 < p.N) *reinterpret_cast<__nv_bfloat162*>(dst + c) = __floats2bfloat162_rn(acc[i][2 * half], acc[i][2 * half + 1]);
    }
  }
}

struct TileParams {
  const bf16* q;             // [n][H D]
  bf16* out;                 // [n][H Dv]
  const bf16* pages;
  const int32_t* block_table;
  int max_pages, page_size;
  int64_t page_stride, v_offset, head_stride;
  const int32_t* meta;       // [4][meta_stride]: slot, first row, length, first position of every entry
  int meta_stride, entries;
  const float* slopes;
  const float* sinks;
  int H, G, D, Dv, Dc;
  int window, keep_first;
  float scale;
  int stages;                // 2: the next tile of keys is fetched while this one is worked on; 1: after it (half the shared memory)
  int chunk;                 // > 0: a row sees only the keys of its own chunk of this many positions
  int out_f32;               // 1: `out` is float32
};

constexpr int KT = 64, NK = KT / 16;

// NVW: value column groups of 16 a warp owns (value sizes up to 64 NVW).
template <int NVW>
__global__ void __launch_bounds__(128) masked_attention_tile_kernel(TileParams p) {
  extern __shared__ __align__(16) unsigned char raw[];
  sb::grid_launch_dependents();
  const int Hg = p.H / p.G, Ht = min(Hg, 16), PT = 16 / Ht;
  const int g = blockIdx.y / (Hg / Ht), head0 = g * Hg + (blockIdx.y % (Hg / Ht)) * Ht;
  const int NV = p.Dv / 16;
  const bool own_values = p.v_offset != 0;                      // values staged apart from the keys
  const int ldk = p.D + 8, ldv = own_values ? p.Dv + 8 : ldk;   // padded rows: ldmatrix without bank conflicts
  const bf16** rowptr = reinterpret_cast<const bf16**>(raw);    // [2][KT]: where a tile's key rows lie (null: a row nobody sees)
  uint32_t* Ps = reinterpret_cast<uint32_t*>(raw + 2 * KT * sizeof(void*));   // [2 parts][NK steps][4 registers][32 lanes]
  float* tmax = reinterpret_cast<float*>(Ps + 2 * NK * 4 * 32);               // [4 warps][16 rows]
  bf16* Qs = reinterpret_cast<bf16*>(tmax + 4 * 16);            // [16][ldk]
  bf16* stage0 = Qs + 16 * ldk;
  const int stage_elems = KT * (ldk + (own_values ? ldv : 0));
  // the blocks that start first take the last tiles: the last positions of an entry see the most keys (a full window, the end of a chunk),
  // and a launch that ends with its longest blocks leaves SMs idle behind them
  int e = 0, tile = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x), len = 0;
  for (; e < p.entries; ++e) {
    len = p.meta[2 * p.meta_stride + e];
    const int tiles = (len + PT - 1) / PT;
    if (tile < tiles) break;
    tile -= tiles;
  }
  if (e >= p.entries) return;
  const int slot = p.meta[e], row0 = p.meta[p.meta_stride + e], pos0 = p.meta[3 * p.meta_stride + e];
  const int t0 = tile * PT, nt = min(PT, len - t0);            // positions pos0 + t0 .. + nt - 1
  const int first_pos = pos0 + t0, last_pos = first_pos + nt - 1;
  const int first_key = max(p.window > 0 ? max(0, first_pos - p.window + 1) : 0, p.chunk > 0 ? first_pos / p.chunk * p.chunk : 0);
  const int kept = p.window > 0 ? p.keep_first : 0;
  const int kt_first = first_key / KT, kt_last = last_pos / KT;
  const int kt_keep = kept > 0 ? min((kept - 1) / KT, kt_last) : -1;          // the last tile with kept tokens
  const int32_t* table = p.block_table + static_cast<int64_t>(slot) * p.max_pages;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  sb::grid_dependency_wait();
  const int dchunks = p.D / 8, vchunks = own_values ? p.Dv / 8 : 0, cpr = dchunks + vchunks;
  for (int i = threadIdx.x; i < 16 * dchunks; i += blockDim.x) {
    const int r = i / dchunks, c = i % dchunks, t = r / Ht;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (t < nt) v = *reinterpret_cast<const uint4*>(p.q + (static_cast<int64_t>(row0 + t0 + t) * p.H + head0 + r % Ht) * p.D + c * 8);
    *reinterpret_cast<uint4*>(Qs + r * ldk + c * 8) = v;
  }
  const int r_lo = lane >> 2, r_hi = r_lo + 8;
  const int p_lo = r_lo / Ht < nt ? first_pos + r_lo / Ht : -1, p_hi = r_hi / Ht < nt ? first_pos + r_hi / Ht : -1;
  const int h_lo = head0 + r_lo % Ht, h_hi = head0 + r_hi % Ht;
  const float s_lo = p.slopes != nullptr ? p.slopes[h_lo] : 0.0f, s_hi = p.slopes != nullptr ? p.slopes[h_hi] : 0.0f;
  float o[2 * NVW][4];
#pragma unroll
  for (int i = 0; i < 2 * NVW; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.0f, l_hi = 0.0f;
  const bf16* base = p.pages + static_cast<int64_t>(g) * p.head_stride;
  int per_row = 1, shift = 0;
  while (per_row < cpr && per_row < 32) {
    per_row <<= 1;
    ++shift;
  }
  auto request = [&](int kt, int buf) {
    if (threadIdx.x < KT) {
      const int j = kt * KT + threadIdx.x;
      rowptr[buf * KT + threadIdx.x] = (j <= last_pos && (j >= first_key || j < kept))
          ? base + static_cast<int64_t>(table[j / p.page_size]) * p.page_stride + static_cast<int64_t>(j % p.page_size) * p.Dc : nullptr;
    }
    __syncthreads();
    bf16* Ks = stage0 + buf * stage_elems;
    bf16* Vs = Ks + KT * ldk;
    for (int r = threadIdx.x >> shift; r < KT; r += blockDim.x >> shift) {
      const bf16* src = rowptr[buf * KT + r];
      const int c0 = threadIdx.x & (per_row - 1);
      bf16* kd = Ks + r * ldk;
      bf16* vd = Vs + r * ldv;
      if (src != nullptr && !own_values) {
#pragma unroll 4
        for (int c = c0; c < dchunks; c += per_row) copy16(kd + c * 8, src + c * 8);
      } else if (src != nullptr) {             // the key's and the value's chunks side by side over the row's threads
        const bf16* vsrc = src + p.v_offset - dchunks * 8;
        for (int c = c0; c < cpr; c += per_row) {
          if (c < dchunks) copy16(kd + c * 8, src + c * 8);
          else copy16(vd + (c - dchunks) * 8, vsrc + c * 8);
        }
      } else {
        for (int c = c0; c < cpr; c += per_row) *reinterpret_cast<uint4*>(c < dchunks ? kd + c * 8 : vd + (c - dchunks) * 8) = make_uint4(0, 0, 0, 0);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  // the tiles in ascending order: those with kept tokens, then from the window's first on
  auto next_tile = [&](int kt) {
    const int n = kt + 1;
    return (n > kt_keep && n < kt_first) ? kt_first : n;
  };
  int kt = kt_keep >= 0 ? 0 : kt_first, buf = 0;
  request(kt, 0);
  const bool two = p.stages == 2;
  for (; kt <= kt_last; buf = two ? buf ^ 1 : 0) {
    const int kt_next = next_tile(kt);
    if (two && kt_next <= kt_last) {
      request(kt_next, buf ^ 1);           // (the buffer of the tile before: every warp left it before the barrier at the end of that tile)
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const bf16* Ks = stage0 + buf * stage_elems;
    const bf16* Vs = own_values ? Ks + KT * ldk : Ks;
    // the scores of this warp's 16 keys
    // (with long value rows, where registers are there for it: four sums side by side, each over every fourth step of 16 elements, so that a
    // product does not wait for the one before it; they are joined in a fixed order: a row's score depends on the row and the key alone)
    constexpr int CH = NVW >= 4 ? 4 : 1;
    float s4[CH][2][4];
#pragma unroll
    for (int c = 0; c < CH; ++c)
#pragma unroll
      for (int i = 0; i < 2; ++i) s4[c][i][0] = s4[c][i][1] = s4[c][i][2] = s4[c][i][3] = 0.0f;
    const bf16* q_at = Qs + (lane & 15) * ldk + (lane >> 4) * 8;
    const bf16* k_at = Ks + (warp * 16 + (lane & 7) + ((lane >> 4) << 3)) * ldk + ((lane >> 3) & 1) * 8;
    int k0 = 0;
    if (CH > 1)
      for (; k0 + 16 * CH <= p.D; k0 += 16 * CH) {       // the four steps' fragments first, then their products
        uint32_t a[CH][4], b[CH][4];
#pragma unroll
        for (int c = 0; c < CH; ++c) {
          ldmatrix_x4(a[c], q_at + k0 + 16 * c);
          ldmatrix_x4(b[c], k_at + k0 + 16 * c);
        }
#pragma unroll
        for (int c = 0; c < CH; ++c) {
          mma_bf16(s4[c][0], a[c], b[c][0], b[c][1]);
          mma_bf16(s4[c][1], a[c], b[c][2], b[c][3]);
        }
      }
    for (; k0 < p.D; k0 += 16) {
      uint32_t a[4], b[4];
      ldmatrix_x4(a, q_at + k0);
      ldmatrix_x4(b, k_at + k0);
      mma_bf16(s4[0][0], a, b[0], b[1]);
      mma_bf16(s4[0][1], a, b[2], b[3]);
    }
    float s[2][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[i][e] = CH == 4 ? (s4[0][i][e] + s4[CH > 1 ? 1 : 0][i][e]) + (s4[CH > 2 ? 2 : 0][i][e] + s4[CH > 3 ? 3 : 0][i][e]) : s4[0][i][e];
    float top_lo = -INFINITY, top_hi = -INFINITY;
#pragma unroll
    for (int n = 0; n < 2; ++n) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int j = kt * KT + warp * 16 + n * 8 + (lane & 3) * 2 + (c & 1);
        const int pos = c < 2 ? p_lo : p_hi;
        const bool seen = j <= pos && (p.window <= 0 || pos - j < p.window || j < p.keep_first) && (p.chunk <= 0 || j >= pos / p.chunk * p.chunk);
        const float x = seen ? __fsub_rn(__fmul_rn(s[n][c], p.scale), __fmul_rn(c < 2 ? s_lo : s_hi, static_cast<float>(pos - j))) : -INFINITY;
        s[n][c] = x;
        if (c < 2) top_lo = fmaxf(top_lo, x);
        else top_hi = fmaxf(top_hi, x);
      }
    }
    top_lo = fmaxf(top_lo, __shfl_xor_sync(0xffffffffu, top_lo, 1)), top_lo = fmaxf(top_lo, __shfl_xor_sync(0xffffffffu, top_lo, 2));
    top_hi = fmaxf(top_hi, __shfl_xor_sync(0xffffffffu, top_hi, 1)), top_hi = fmaxf(top_hi, __shfl_xor_sync(0xffffffffu, top_hi, 2));
    if ((lane & 3) == 0) tmax[warp * 16 + r_lo] = top_lo, tmax[warp * 16 + r_hi] = top_hi;
    __syncthreads();
    float n_lo = m_lo, n_hi = m_hi;
#pragma unroll
    for (int w = 0; w < 4; ++w) n_lo = fmaxf(n_lo, tmax[w * 16 + r_lo]), n_hi = fmaxf(n_hi, tmax[w * 16 + r_hi]);
    const float f_lo = n_lo == m_lo ? 1.0f : __expf(m_lo - n_lo), f_hi = n_hi == m_hi ? 1.0f : __expf(m_hi - n_hi);
    m_lo = n_lo, m_hi = n_hi;
    // the weights in two parts: the A operand of step `warp` of the value product, handed to the other warps
    float add_lo = 0.0f, add_hi = 0.0f;
#pragma unroll
    for (int n = 0; n < 2; ++n) {
      float w[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) w[c] = s[n][c] == -INFINITY ? 0.0f : __expf(s[n][c] - (c < 2 ? m_lo : m_hi));
      add_lo += w[0] + w[1], add_hi += w[2] + w[3];
      const __nv_bfloat162 h01 = __floats2bfloat162_rn(w[0], w[1]), h23 = __floats2bfloat162_rn(w[2], w[3]);
      uint32_t* hi = Ps + ((0 * NK + warp) * 4 + n * 2) * 32 + lane;
      uint32_t* lo = Ps + ((1 * NK + warp) * 4 + n * 2) * 32 + lane;
      hi[0] = *reinterpret_cast<const uint32_t*>(&h01);
      hi[32] = *reinterpret_cast<const uint32_t*>(&h23);
      lo[0] = pack_bf16(w[0] - __low2float(h01), w[1] - __high2float(h01));
      lo[32] = pack_bf16(w[2] - __low2float(h23), w[3] - __high2float(h23));
    }
    l_lo = fmaf(l_lo, f_lo, add_lo), l_hi = fmaf(l_hi, f_hi, add_hi);
#pragma unroll
    for (int i = 0; i < 2 * NVW; ++i) o[i][0] *= f_lo, o[i][1] *= f_lo, o[i][2] *= f_hi, o[i][3] *= f_hi;
    __syncthreads();
    // O += hi V + lo V for this warp's value columns, the tile's steps in ascending order
#pragma unroll
    for (int kk = 0; kk < NK; ++kk) {
      uint32_t hi[4], lo[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        hi[i] = Ps[((0 * NK + kk) * 4 + i) * 32 + lane];
        lo[i] = Ps[((1 * NK + kk) * 4 + i) * 32 + lane];
      }
      // the step's value fragments first, then the products of the first parts for every column group, then those of the second parts:
      // a column's sum takes its terms in the same order (hi, then lo), with the other columns' products between the two
      uint32_t b[NVW][4];
      const bf16* v_at = Vs + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ldv + (lane >> 4) * 8;
#pragma unroll
      for (int i = 0; i < NVW; ++i)
        if (warp + 4 * i < NV) ldmatrix_x4_trans(b[i], v_at + (warp + 4 * i) * 16);
#pragma unroll
      for (int i = 0; i < NVW; ++i)
        if (warp + 4 * i < NV) {
          mma_bf16(o[2 * i], hi, b[i][0], b[i][1]);
          mma_bf16(o[2 * i + 1], hi, b[i][2], b[i][3]);
        }
#pragma unroll
      for (int i = 0; i < NVW; ++i)
        if (warp + 4 * i < NV) {
          mma_bf16(o[2 * i], lo, b[i][0], b[i][1]);
          mma_bf16(o[2 * i + 1], lo, b[i][2], b[i][3]);
        }
    }
    __syncthreads();                      // the tile's buffer, the maxima and the exchanged operands may be written again
    if (!two && kt_next <= kt_last) request(kt_next, 0);
    kt = kt_next;
  }
  // the rows' sums: a thread's share over its columns, the four lanes of a row, then the warps in ascending order; then the sink
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1), l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1), l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
  if ((lane & 3) == 0) tmax[warp * 16 + r_lo] = l_lo, tmax[warp * 16 + r_hi] = l_hi;
  __syncthreads();
  float t_lo = tmax[r_lo], t_hi = tmax[r_hi];
#pragma unroll
  for (int w = 1; w < 4; ++w) t_lo += tmax[w * 16 + r_lo], t_hi += tmax[w * 16 + r_hi];
  if (p.sinks != nullptr) t_lo += __expf(p.sinks[h_lo] - m_lo), t_hi += __expf(p.sinks[h_hi] - m_hi);
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int r = half ? r_hi : r_lo;
    if (r / Ht >= nt) continue;
    const float inv = 1.0f / (half ? t_hi : t_lo);
    const int64_t at = (static_cast<int64_t>(row0 + t0 + r / Ht) * p.H + head0 + r % Ht) * p.Dv + (lane & 3) * 2;
    bf16* dst = p.out + at;
    float* dst32 = reinterpret_cast<float*>(p.out) + at;
#pragma unroll
    for (int i = 0; i < NVW; ++i) {
      const int nv = warp + 4 * i;
      if (nv < NV && p.out_f32) {
        *reinterpret_cast<float2*>(dst32 + nv * 16) = make_float2(o[2 * i][2 * half] * inv, o[2 * i][2 * half + 1] * inv);
        *reinterpret_cast<float2*>(dst32 + nv * 16 + 8) = make_float2(o[2 * i + 1][2 * half] * inv, o[2 * i + 1][2 * half + 1] * inv);
      } else if (nv < NV) {
        *reinterpret_cast<__nv_bfloat162*>(dst + nv * 16) = __floats2bfloat162_rn(o[2 * i][2 * half] * inv, o[2 * i][2 * half + 1] * inv);
        *reinterpret_cast<__nv_bfloat162*>(dst + nv * 16 + 8) = __floats2bfloat162_rn(o[2 * i + 1][2 * half] * inv, o[2 * i + 1][2 * half + 1] * inv);
      }
    }
  }
}

template <int NVW>
int launch_tiles(const TileParams& p, int n, cudaStream_t stream) {
  const int Hg = p.H / p.G, Ht = Hg < 16 ? Hg : 16, PT = 16 / Ht;
  const bool own_values = p.v_offset != 0;
  const size_t fixed = 2 * KT * sizeof(void*) + 2 * NK * 4 * 32 * sizeof(uint32_t) + 4 * 16 * sizeof(float) + sizeof(bf16) * 16 * (p.D + 8);
  const size_t stage = sizeof(bf16) * KT * (p.D + 8 + (own_values ? p.Dv + 8 : 0));
  size_t smem = fixed + 2 * stage;
  if (smem > 220 * 1024) return sb::fail("sb_masked_attention_tiles: key size %d and value size %d need %zu bytes of shared memory", p.D, p.Dv, smem);
  const dim3 grid((n + PT - 1) / PT + p.entries, p.G * (Hg / Ht));
  TileParams q = p;
  q.stages = 2;
  // rows so long that two stages leave room for one CTA on an SM: with CTAs enough for two on every SM, one stage each and two CTAs that
  // fill each other's waits do better. The arithmetic is the same either way.
  constexpr size_t kHalfSm = 113 * 1024;
  if (smem > kHalfSm && fixed + stage <= kHalfSm && static_cast<int64_t>(grid.x) * grid.y >= 2 * sb::sm_count()) {
    q.stages = 1;
    smem = fixed + stage;
  }
  static sb::DeviceOnce once;
  if (once.needed()) {
    cudaFuncSetAttribute(masked_attention_tile_kernel<NVW>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
    once.done();
  }
  sb::prefer_max_shared(reinterpret_cast<const void*>(masked_attention_tile_kernel<NVW>));
  sb::launch_pdl(masked_attention_tile_kernel<NVW>, grid, dim3(128), smem, stream, q);
  return sb::check_launch("sb_masked_attention_tiles");
}

PageRef page_ref(void* pages, const int32_t* block_table, int max_pages, int page_size, int64_t page_stride, int64_t v_offset, int64_t head_stride,
                 int Dc) {
  return PageRef{pages, block_table, max_pages, page_size, page_stride, v_offset, head_stride, Dc};
}

}  // namespace

// qkv [P][n][Hq D + Hkv D + Hkv Dv] float32 partial sums; bias, q_gain, k_gain float32 or null. dtype: 0 float32, 1 bfloat16 (q_out and cache).
SB_EXPORT int sb_qkv_norm_append(const float* qkv, int n_partials, int64_t partial_stride, const float* bias, const float* q_gain, const float* k_gain,
                                 float eps, const int32_t* positions, const int32_t* slots, void* q_out, int dtype, void* pages,
                                 const int32_t* block_table, int max_pages, int page_size, int64_t page_stride, int64_t v_offset, int64_t head_stride,
                                 int n, int Hq, int Hkv, int D, int Dv, int Dc, int write_kv, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (n_partials < 1) return sb::fail("sb_qkv_norm_append: n_partials must be >= 1");
  if (Dc < D || Dc < Dv) return sb::fail("sb_qkv_norm_append: a page row of %d elements holds neither a key of %d nor a value of %d", Dc, D, Dv);
  const size_t smem = sizeof(float) * (static_cast<size_t>(Hq) * D + static_cast<size_t>(Hkv) * (D + Dv));
  if (smem > 160 * 1024) return sb::fail("sb_qkv_norm_append: a row of %zu bytes does not fit the row buffer", smem);
  NormAppendParams p{qkv, n_partials, partial_stride, bias, q_gain, k_gain, eps, positions, slots, q_out,
                     page_ref(pages, block_table, max_pages, page_size, page_stride, v_offset, head_stride, Dc), Hq, Hkv, D, Dv, write_kv};
  if (dtype == 0) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(qkv_norm_append_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    sb::launch_pdl(qkv_norm_append_kernel<float>, dim3(n), dim3(256), smem, stream, p);
  } else if (dtype == 1) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(qkv_norm_append_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    sb::launch_pdl(qkv_norm_append_kernel<bf16>, dim3(n), dim3(256), smem, stream, p);
  } else {
    return sb::fail("sb_qkv_norm_append: unsupported dtype %d", dtype);
  }
  return sb::check_launch("sb_qkv_norm_append");
}

// proj [P][n][Rq + Rkv + rot] float32 partial sums -> q_latent [n][Rq] and the token's page row [Rkv | rot].
SB_EXPORT int sb_latent_prepare(const float* proj, int n_partials, int64_t partial_stride, const float* q_gain, const float* kv_gain, float eps,
                                const int32_t* positions, const int32_t* slots, const float* cos_sin, void* q_latent, int dtype, void* pages,
                                const int32_t* block_table, int max_pages, int page_size, int64_t page_stride, int n, int Rq, int Rkv, int rot, int Dc,
                                int write_kv, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (n_partials < 1) return sb::fail("sb_latent_prepare: n_partials must be >= 1");
  if (rot % 2 != 0 || rot < 0) return sb::fail("sb_latent_prepare: %d rotated elements (must be even)", rot);
  if (Dc < Rkv + rot) return sb::fail("sb_latent_prepare: a page row of %d elements does not hold %d + %d", Dc, Rkv, rot);
  const size_t smem = sizeof(float) * (static_cast<size_t>(Rq) + Rkv + rot);
  if (smem > 160 * 1024) return sb::fail("sb_latent_prepare: a row of %zu bytes does not fit the row buffer", smem);
  LatentParams p{proj, n_partials, partial_stride, q_gain, kv_gain, eps, positions, slots, cos_sin, q_latent,
                 page_ref(pages, block_table, max_pages, page_size, page_stride, 0, 0, Dc), Rq, Rkv, rot, write_kv};
  if (dtype == 0) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(latent_prepare_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    sb::launch_pdl(latent_prepare_kernel<float>, dim3(n), dim3(256), smem, stream, p);
  } else if (dtype == 1) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(latent_prepare_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    sb::launch_pdl(latent_prepare_kernel<bf16>, dim3(n), dim3(256), smem, stream, p);
  } else {
    return sb::fail("sb_latent_prepare: unsupported dtype %d", dtype);
  }
  return sb::check_launch("sb_latent_prepare");
}

SB_EXPORT int sb_rotate_heads(const float* q, int n_partials, int64_t partial_stride, const int32_t* positions, const float* cos_sin, void* out, int dtype,
                              int n, int H, int D, int offset, int rot, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (n_partials < 1) return sb::fail("sb_rotate_heads: n_partials must be >= 1");
  if (rot % 2 != 0 || rot < 0 || offset < 0 || offset + rot > D) return sb::fail("sb_rotate_heads: elements %d .. %d of a head of %d", offset, offset + rot, D);
  const dim3 grid(n, (H * D + 255) / 256);
  if (dtype == 0) sb::launch_pdl(rotate_heads_kernel<float>, grid, dim3(256), 0, stream, q, n_partials, partial_stride, positions, cos_sin, static_cast<float*>(out), H, D, offset, rot);
  else if (dtype == 1) sb::launch_pdl(rotate_heads_kernel<bf16>, grid, dim3(256), 0, stream, q, n_partials, partial_stride, positions, cos_sin, static_cast<bf16*>(out), H, D, offset, rot);
  else return sb::fail("sb_rotate_heads: unsupported dtype %d", dtype);
  return sb::check_launch("sb_rotate_heads");
}

// out[r, h, :N] = W_h^T in[r, h, :K] for every head (w [H][K][N]); `tail` elements behind the K are copied behind the N. Strides in elements.
SB_EXPORT int sb_head_linear(const void* in, int64_t in_row, int64_t in_head, const void* w, void* out, int64_t out_row, int64_t out_head, int dtype,
                             int n, int H, int K, int N, int tail, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (H <= 0 || K <= 0 || N <= 0 || tail < 0) return sb::fail("sb_head_linear: %d heads of %d -> %d (+ %d)", H, K, N, tail);
  constexpr int TR = 8;
  const size_t smem = sizeof(float) * TR * K;
  if (smem > 160 * 1024) return sb::fail("sb_head_linear: rows of %d elements do not fit the row buffer", K);
  HeadLinearParams p{in, in_row, in_head, w, out, out_row, out_head, n, H, K, N, tail};
  const bool aligned = ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
  if (dtype == 1 && aligned && K % 16 == 0 && N % 8 == 0 && in_row % 8 == 0 && in_head % 8 == 0 && out_row % 8 == 0 && out_head % 8 == 0) {
    // (what decides for the tensor cores is the shape alone, never the number of rows: a token has one form whatever step it is in)
    sb::launch_pdl(head_linear_tc_kernel, dim3((n + kHlTile - 1) / kHlTile, H, (N + kHlTile - 1) / kHlTile), dim3(128), 0, stream, p);
    return sb::check_launch("sb_head_linear");
  }
  const dim3 grid((n + TR - 1) / TR, H);
  if (dtype == 0) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(head_linear_kernel<float, TR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    sb::launch_pdl(head_linear_kernel<float, TR>, grid, dim3(128), smem, stream, p);
  } else if (dtype == 1) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(head_linear_kernel<bf16, TR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    sb::launch_pdl(head_linear_kernel<bf16, TR>, grid, dim3(128), smem, stream, p);
  } else {
    return sb::fail("sb_head_linear: unsupported dtype %d", dtype);
  }
  return sb::check_launch("sb_head_linear");
}

// `chunk` > 0: a row sees only the keys of its own chunk of that many positions; `out_f32`: the result is stored as float32.
SB_EXPORT int sb_masked_attention_ex(const void* q, void* out, int dtype, const void* pages, const int32_t* block_table, int max_pages, int page_size,
                                     int64_t page_stride, int64_t v_offset, int64_t head_stride, const int32_t* positions, const int32_t* slots,
                                     const float* slopes, const float* sinks, int n, int H, int G, int D, int Dv, int Dc, int window, int keep_first,
                                     float scale, int chunk, int out_f32, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (chunk < 0) return sb::fail("sb_masked_attention: chunk %d", chunk);
  if (H <= 0 || G <= 0 || H % G != 0) return sb::fail("sb_masked_attention: %d heads do not divide into %d key/value heads", H, G);
  if (D <= 0 || Dv <= 0 || D > 640 || Dv > 640) return sb::fail("sb_masked_attention: key size %d, value size %d (at most 640)", D, Dv);
  if (window < 0 || keep_first < 0) return sb::fail("sb_masked_attention: window %d, kept first tokens %d", window, keep_first);
  AttnParams p{q, out, pages, block_table, max_pages, page_size, page_stride, v_offset, head_stride, positions, slots, slopes, sinks,
               H, G, D, Dv, Dc, window, keep_first, scale, chunk, out_f32};
  const size_t smem = sizeof(float) * (D + kWarps * Dv + 2 * kWarps);
  const bool small = D <= 256 && Dv <= 256;
  if (dtype == 0) {
    if (small) sb::launch_pdl(masked_attention_kernel<float, 8>, dim3(n, H), dim3(kWarps * 32), smem, stream, p);
    else sb::launch_pdl(masked_attention_kernel<float, 20>, dim3(n, H), dim3(kWarps * 32), smem, stream, p);
  } else if (dtype == 1) {
    if (small) sb::launch_pdl(masked_attention_kernel<bf16, 8>, dim3(n, H), dim3(kWarps * 32), smem, stream, p);
    else sb::launch_pdl(masked_attention_kernel<bf16, 20>, dim3(n, H), dim3(kWarps * 32), smem, stream, p);
  } else {
    return sb::fail("sb_masked_attention: unsupported dtype %d", dtype);
  }
  return sb::check_launch("sb_masked_attention");
}

SB_EXPORT int sb_masked_attention(const void* q, void* out, int dtype, const void* pages, const int32_t* block_table, int max_pages, int page_size,
                                  int64_t page_stride, int64_t v_offset, int64_t head_stride, const int32_t* positions, const int32_t* slots,
                                  const float* slopes, const float* sinks, int n, int H, int G, int D, int Dv, int Dc, int window, int keep_first,
                                  float scale, cudaStream_t stream) {
  return sb_masked_attention_ex(q, out, dtype, pages, block_table, max_pages, page_size, page_stride, v_offset, head_stride, positions, slots, slopes,
                                sinks, n, H, G, D, Dv, Dc, window, keep_first, scale, 0, 0, stream);
}

// The tensor-core form: whether it takes a shape, and the launch. Entries come from the step's records on the device (meta).
SB_EXPORT int sb_masked_attention_tiles_supported(int H, int G, int D, int Dv, int Dc, int64_t v_offset) {
  if (G <= 0 || H % G != 0) return 0;
  const int Hg = H / G;
  const bool heads = Hg <= 16 ? (Hg & (Hg - 1)) == 0 : Hg % 16 == 0;
  const size_t stage = sizeof(bf16) * (16 * (D + 8) + 2 * 64 * (D + 8 + (v_offset != 0 ? Dv + 8 : 0)));
  return heads && D % 16 == 0 && D >= 16 && Dv % 16 == 0 && Dv >= 16 && Dv <= 512 && Dv <= Dc && Dc % 8 == 0 && v_offset % 8 == 0 && stage <= 200 * 1024;
}

SB_EXPORT int sb_masked_attention_tiles_ex(const void* q, void* out, const void* pages, const int32_t* block_table, int max_pages, int page_size,
                                           int64_t page_stride, int64_t v_offset, int64_t head_stride, const int32_t* meta, int meta_stride,
                                           int entries, const float* slopes, const float* sinks, int n, int H, int G, int D, int Dv, int Dc,
                                           int window, int keep_first, float scale, int chunk, int out_f32, cudaStream_t stream) {
  if (n <= 0 || entries <= 0) return 0;
  if (chunk < 0) return sb::fail("sb_masked_attention_tiles: chunk %d", chunk);
  if (!sb_masked_attention_tiles_supported(H, G, D, Dv, Dc, v_offset))
    return sb::fail("sb_masked_attention_tiles: heads %d / %d, key size %d, value size %d are not a shape of the tensor-core form", H, G, D, Dv);
  if (window < 0 || keep_first < 0) return sb::fail("sb_masked_attention_tiles: window %d, kept first tokens %d", window, keep_first);
  TileParams p{static_cast<const bf16*>(q), static_cast<bf16*>(out), static_cast<const bf16*>(pages), block_table, max_pages, page_size, page_stride,
               v_offset, head_stride, meta, meta_stride, entries, slopes, sinks, H, G, D, Dv, Dc, window, keep_first, scale, 2, chunk, out_f32};
  const int groups = (Dv / 16 + 3) / 4;
  switch (groups) {
    case 1: return launch_tiles<1>(p, n, stream);
    case 2: return launch_tiles<2>(p, n, stream);
    case 3: case 4: return launch_tiles<4>(p, n, stream);
    default: return launch_tiles<8>(p, n, stream);
  }
}

SB_EXPORT int sb_masked_attention_tiles(const void* q, void* out, const void* pages, const int32_t* block_table, int max_pages, int page_size,
                                        int64_t page_stride, int64_t v_offset, int64_t head_stride, const int32_t* meta, int meta_stride, int entries,
                                        const float* slopes, const float* sinks, int n, int H, int G, int D, int Dv, int Dc, int window, int keep_first,
                                        float scale, cudaStream_t stream) {
  return sb_masked_attention_tiles_ex(q, out, pages, block_table, max_pages, page_size, page_stride, v_offset, head_stride, meta, meta_stride, entries,
                                      slopes, sinks, n, H, G, D, Dv, Dc, window, keep_first, scale, 0, 0, stream);
}

// ------------------------------------------------------------------ operations of the native step program (step_ops.h)
// i: 0 qkv partial sums (flat), 1 K ranges S, 2 most tokens with a buffer per range, 3 bias, 4 q gain, 5 k gain, 6 q out, 7 dtype, 8 pages,
//    9 block table, 10 max_pages, 11 page_size, 12 page_stride, 13 v_offset, 14 head_stride, 15 Hq, 16 Hkv, 17 D, 18 Dv, 19 Dc, 20 write_kv
// f: 0 eps
SB_EXPORT int sb_op_qkv_norm_append(const SbOp* op, const SbStep* s, void* stream) {
  using namespace sbstep;
  if (s->n <= 0) return SB_OP_SKIPPED;
  const int Hq = (int)op->i[15], Hkv = (int)op->i[16], D = (int)op->i[17], Dv = (int)op->i[18];
  const int64_t width = static_cast<int64_t>(Hq) * D + static_cast<int64_t>(Hkv) * (D + Dv);
  return sb_qkv_norm_append(ptr<const float>(op->i[0]), partial_count(op->i[1], op->i[2], s->n), s->n * width, ptr<const float>(op->i[3]),
                            ptr<const float>(op->i[4]), ptr<const float>(op->i[5]), (float)op->f[0], positions(s), slots(s), ptr<void>(op->i[6]),
                            (int)op->i[7], ptr<void>(op->i[8]), ptr<const int32_t>(op->i[9]), (int)op->i[10], (int)op->i[11], op->i[12], op->i[13],
                            op->i[14], s->n, Hq, Hkv, D, Dv, (int)op->i[19], (int)op->i[20], static_cast<cudaStream_t>(stream));
}

// i: 0 projection partial sums (flat), 1 K ranges S, 2 most tokens with a buffer per range, 3 q gain, 4 kv gain, 5 cos_sin, 6 q latent, 7 dtype,
//    8 pages, 9 block table, 10 max_pages, 11 page_size, 12 page_stride, 13 Rq, 14 Rkv, 15 rot, 16 Dc, 17 write_kv      f: 0 eps
SB_EXPORT int sb_op_latent_prepare(const SbOp* op, const SbStep* s, void* stream) {
  using namespace sbstep;
  if (s->n <= 0) return SB_OP_SKIPPED;
  const int Rq = (int)op->i[13], Rkv = (int)op->i[14], rot = (int)op->i[15];
  return sb_latent_prepare(ptr<const float>(op->i[0]), partial_count(op->i[1], op->i[2], s->n), static_cast<int64_t>(s->n) * (Rq + Rkv + rot),
                           ptr<const float>(op->i[3]), ptr<const float>(op->i[4]), (float)op->f[0], positions(s), slots(s), ptr<const float>(op->i[5]),
                           ptr<void>(op->i[6]), (int)op->i[7], ptr<void>(op->i[8]), ptr<const int32_t>(op->i[9]), (int)op->i[10], (int)op->i[11],
                           op->i[12], s->n, Rq, Rkv, rot, (int)op->i[16], (int)op->i[17], static_cast<cudaStream_t>(stream));
}

// i: 0 q partial sums (flat), 1 K ranges S, 2 most tokens with a buffer per range, 3 cos_sin, 4 out, 5 dtype, 6 H, 7 D, 8 offset, 9 rot
SB_EXPORT int sb_op_rotate_heads(const SbOp* op, const SbStep* s, void* stream) {
  using namespace sbstep;
  if (s->n <= 0) return SB_OP_SKIPPED;
  const int H = (int)op->i[6], D = (int)op->i[7];
  return sb_rotate_heads(ptr<const float>(op->i[0]), partial_count(op->i[1], op->i[2], s->n), static_cast<int64_t>(s->n) * H * D, positions(s),
                         ptr<const float>(op->i[3]), ptr<void>(op->i[4]), (int)op->i[5], s->n, H, D, (int)op->i[8], (int)op->i[9],
                         static_cast<cudaStream_t>(stream));
}

// i: 0 in, 1 in_row, 2 in_head, 3 w, 4 out, 5 out_row, 6 out_head, 7 dtype, 8 H, 9 K, 10 N, 11 tail
SB_EXPORT int sb_op_head_linear(const SbOp* op, const SbStep* s, void* stream) {
  using namespace sbstep;
  if (s->n <= 0) return SB_OP_SKIPPED;
  return sb_head_linear(ptr<const void>(op->i[0]), op->i[1], op->i[2], ptr<const void>(op->i[3]), ptr<void>(op->i[4]), op->i[5], op->i[6], (int)op->i[7],
                        s->n, (int)op->i[8], (int)op->i[9], (int)op->i[10], (int)op->i[11], static_cast<cudaStream_t>(stream));
}

// i: 0 q, 1 out, 2 dtype, 3 pages, 4 block table, 5 max_pages, 6 page_size, 7 page_stride, 8 v_offset, 9 head_stride, 10 slopes, 11 sinks, 12 H,
//    13 G, 14 D, 15 Dv, 16 Dc, 17 window, 18 keep_first, 19 chunk, 20 the result as float32      f: 0 scale
SB_EXPORT int sb_op_masked_attention(const SbOp* op, const SbStep* s, void* stream) {
  using namespace sbstep;
  if (s->n <= 0) return SB_OP_SKIPPED;
  return sb_masked_attention_ex(ptr<const void>(op->i[0]), ptr<void>(op->i[1]), (int)op->i[2], ptr<const void>(op->i[3]), ptr<const int32_t>(op->i[4]),
                             (int)op->i[5], (int)op->i[6], op->i[7], op->i[8], op->i[9], positions(s), slots(s), ptr<const float>(op->i[10]),
                             ptr<const float>(op->i[11]), s->n, (int)op->i[12], (int)op->i[13], (int)op->i[14], (int)op->i[15], (int)op->i[16],
                             (int)op->i[17], (int)op->i[18], (float)op->f[0], (int)op->i[19], (int)op->i[20], static_cast<cudaStream_t>(stream));
}

// i: 0 q, 1 out, 2 pages, 3 block table, 4 max_pages, 5 page_size, 6 page_stride, 7 v_offset, 8 head_stride, 9 slopes, 10 sinks, 11 H, 12 G, 13 D,
//    14 Dv, 15 Dc, 16 window, 17 keep_first, 18 chunk, 19 the result as float32      f: 0 scale
SB_EXPORT int sb_op_masked_attention_tiles(const SbOp* op, const SbStep* s, void* stream) {
  using namespace sbstep;
  if (s->n <= 0) return SB_OP_SKIPPED;
  return sb_masked_attention_tiles_ex(ptr<const void>(op->i[0]), ptr<void>(op->i[1]), ptr<const void>(op->i[2]), ptr<const int32_t>(op->i[3]), (int)op->i[4],
                                   (int)op->i[5], op->i[6], op->i[7], op->i[8], entry_meta(s), s->max_rows, s->entries, ptr<const float>(op->i[9]),
                                   ptr<const float>(op->i[10]), s->n, (int)op->i[11], (int)op->i[12], (int)op->i[13], (int)op->i[14], (int)op->i[15],
                                   (int)op->i[16], (int)op->i[17], (float)op->f[0], (int)op->i[18], (int)op->i[19], static_cast<cudaStream_t>(stream));
}

// ---------------------------------------------------------------------------------------------------------------------------------
// The general preparation of a step's queries, keys and values in front of the attention kernels above, and the gates behind them.
//
// `qkv_prepare_kernel`: a block per token. The row q | k | v of the projection (its K ranges' partial sums folded, bias added) waits in
// shared memory; then, as the parameters say: an RMS norm of q and of k, over the whole projection (gains of that size) or per head
// (one gain of the head's size for all heads); rotation of the first `rot` elements of every q and k head by the token's position, pairs
// (2i, 2i + 1) or (i, i + rot / 2); a factor on q that grows with the position, 1 + c ln(floor((p + 1) / every) + 1); q stored, k and v
// appended to the token's page row. All in 32-bit.
//
// `head_gate_kernel`: the attention's result (float32 [n][heads][Dv]) times a gate that is a column range of the projection's partial
// sums, sigmoid applied: one gate per element, or one per head. With two maps per head (differential attention) the result of map 1 less
// lambda times that of map 2 is RMS-normed over the head's values (no gain) and multiplied by a constant first.
namespace {

struct PrepareParams {
  const float* proj;         // [P][n][width]: q (Hq D) | k (Hkv D) | v (Hkv Dv) | whatever else the projection carries
  int n_partials;
  int64_t partial_stride;
  int width;
  const float* bias;         // [Hq D + Hkv D + Hkv Dv] or null
  const float* q_gain;       // norm_mode 1: [Hq D]; 2: [D]
  const float* k_gain;       // norm_mode 1: [Hkv D]; 2: [D]
  int norm_mode;             // 0: none, 1: over the whole projection, 2: per head
  float eps;
  const float* cos_sin;      // [positions][rot / 2][2]
  int rot, interleaved;
  float temp_coef;
  int temp_every;            // 0: no factor on q
  const int32_t* positions;
  const int32_t* slots;
  void* q_out;               // [n][Hq D]
  PageRef c;
  int Hq, Hkv, D, Dv;
  int write_kv;
};

template <class T>
__global__ void __launch_bounds__(256) qkv_prepare_kernel(PrepareParams p) {
  extern __shared__ float row_values[];
  __shared__ float red[32];
  sb::grid_launch_dependents();
  const int row = blockIdx.x;
  const int nq = p.Hq * p.D, nk = p.Hkv * p.D, cols = nq + nk + p.Hkv * p.Dv;
  const int pos = p.positions[row], slot = p.slots[row];
  const int page = p.write_kv ? p.c.block_table[static_cast<int64_t>(slot) * p.c.max_pages + pos / p.c.page_size] : 0;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  sb::grid_dependency_wait();
  const float* src = p.proj + static_cast<int64_t>(row) * p.width;
  float sq_q = 0.0f, sq_k = 0.0f;
  for (int i = threadIdx.x; i < cols; i += blockDim.x) {
    float v = folded(src + i, p.n_partials, p.partial_stride);
    if (p.bias != nullptr) v = __fadd_rn(v, p.bias[i]);
    row_values[i] = v;
    if (i < nq) sq_q = fmaf(v, v, sq_q);
    else if (i < nq + nk) sq_k = fmaf(v, v, sq_k);
  }
  if (p.norm_mode == 1) {
    const float rq = 1.0f / sqrtf(sb::block_sum(sq_q, red) / static_cast<float>(nq) + p.eps);
    const float rk = 1.0f / sqrtf(sb::block_sum(sq_k, red) / static_cast<float>(nk) + p.eps);
    for (int i = threadIdx.x; i < nq + nk; i += blockDim.x)
      row_values[i] = i < nq ? __fmul_rn(__fmul_rn(row_values[i], rq), p.q_gain[i]) : __fmul_rn(__fmul_rn(row_values[i], rk), p.k_gain[i - nq]);
  } else if (p.norm_mode == 2) {
    __syncthreads();
    for (int hh = warp; hh < p.Hq + p.Hkv; hh += warps) {      // a warp per head: the squares by lane in ascending elements, then xor shuffles
      float* head = row_values + hh * p.D;
      float ss = 0.0f;
      for (int d = lane; d < p.D; d += 32) ss = fmaf(head[d], head[d], ss);
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      const float r = 1.0f / sqrtf(ss / static_cast<float>(p.D) + p.eps);
      const float* gain = hh < p.Hq ? p.q_gain : p.k_gain;
      for (int d = lane; d < p.D; d += 32) head[d] = __fmul_rn(__fmul_rn(head[d], r), gain[d]);
    }
  }
  __syncthreads();
  float temp = 1.0f;
  if (p.temp_every > 0) temp = fmaf(p.temp_coef, logf(static_cast<float>((pos + 1) / p.temp_every) + 1.0f), 1.0f);
  const int rh = p.rot / 2;
  T* pages = static_cast<T*>(p.c.pages);
  for (int i = threadIdx.x; i < cols; i += blockDim.x) {
    float v = row_values[i];
    const bool is_v = i >= nq + nk;
    if (!is_v) {
      const int d = i % p.D;
      if (d < p.rot) {
        int pair, other;
        bool low;
        if (p.interleaved) pair = d >> 1, low = (d & 1) == 0, other = low ? i + 1 : i - 1;
        else low = d < rh, pair = low ? d : d - rh, other = low ? i + rh : i - rh;
        const float b = row_values[other];
        const float2 cs = *reinterpret_cast<const float2*>(p.cos_sin + (static_cast<int64_t>(pos) * rh + pair) * 2);
        v = low ? __fsub_rn(__fmul_rn(v, cs.x), __fmul_rn(b, cs.y)) : __fadd_rn(__fmul_rn(v, cs.x), __fmul_rn(b, cs.y));
      }
    }
    if (i < nq) {
      static_cast<T*>(p.q_out)[static_cast<int64_t>(row) * nq + i] = sb::narrow<T>(__fmul_rn(v, temp));
    } else if (p.write_kv) {
      const int e = is_v ? i - nq - nk : i - nq;
      const int dim = is_v ? p.Dv : p.D, head = e / dim, d = e % dim;
      pages[static_cast<int64_t>(page) * p.c.page_stride + (is_v ? p.c.v_offset : 0) + static_cast<int64_t>(head) * p.c.head_stride +
            static_cast<int64_t>(pos % p.c.page_size) * p.c.Dc + d] = sb::narrow<T>(v);
    }
  }
}

struct HeadGateParams {
  const float* a;            // [n][maps H][Dv]: with two maps, map m of head h = g Hg + j lies at head (2 g + m) Hg + j (Hg = H / G)
  const float* proj;         // the gate's partial sums [P][n][width], columns g_off ..
  int n_partials;
  int64_t partial_stride;
  int width, g_off;
  void* out;                 // [n][H Dv]
  int H, G, Dv, maps;
  int per_head;              // 1: one gate per head, 0: one per element
  float lambda, post, eps;   // two maps: (a1 - lambda a2) RMS-normed, times post
};

template <class T>
__global__ void __launch_bounds__(128) head_gate_kernel(HeadGateParams p) {
  sb::grid_launch_dependents();
  const int row = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  const int Hg = p.H / p.G;
  sb::grid_dependency_wait();
  const float* gate = p.proj + static_cast<int64_t>(row) * p.width + p.g_off;
  T* out = static_cast<T*>(p.out) + static_cast<int64_t>(row) * p.H * p.Dv;
  for (int h = blockIdx.y * warps + warp; h < p.H; h += gridDim.y * warps) {      // a warp per head; how the heads are dealt to blocks changes nothing
    const int g = h / Hg, j = h % Hg;
    const float* a1 = p.a + (static_cast<int64_t>(row) * p.maps * p.H + (p.maps == 2 ? (2 * g) * Hg + j : h)) * p.Dv;
    const float* a2 = a1 + static_cast<int64_t>(Hg) * p.Dv;
    float scale = 1.0f;
    if (p.maps == 2) {
      float ss = 0.0f;
      for (int d = lane; d < p.Dv; d += 32) {
        const float o = __fsub_rn(a1[d], __fmul_rn(p.lambda, a2[d]));
        ss = fmaf(o, o, ss);
      }
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      scale = p.post / sqrtf(ss / static_cast<float>(p.Dv) + p.eps);
    }
    float head_gate = 0.0f;
    if (p.per_head) head_gate = 1.0f / (1.0f + expf(-folded(gate + h, p.n_partials, p.partial_stride)));
    for (int d = lane; d < p.Dv; d += 32) {
      float o = p.maps == 2 ? __fmul_rn(__fsub_rn(a1[d], __fmul_rn(p.lambda, a2[d])), scale) : a1[d];
      const float gt = p.per_head ? head_gate : 1.0f / (1.0f + expf(-folded(gate + h * p.Dv + d, p.n_partials, p.partial_stride)));
      out[h * p.Dv + d] = sb::narrow<T>(__fmul_rn(o, gt));
    }
  }
}

}  // namespace

// i: 0 projection partial sums (flat), 1 their width, 2 K ranges S, 3 most tokens with a buffer per range, 4 bias, 5 q gain, 6 k gain, 7 norm mode,
//    8 cos_sin, 9 rot, 10 interleaved pairs, 11 temp_every, 12 q out, 13 dtype, 14 pages, 15 block table, 16 max_pages, 17 page_size,
//    18 page_stride, 19 v_offset, 20 head_stride, 21 Hq, 22 Hkv, 23 D, 24 Dv, 25 Dc, 26 write_kv
// f: 0 eps, 1 temp_coef
SB_EXPORT int sb_op_qkv_prepare(const SbOp* op, const SbStep* s, void* stream) {
  using namespace sbstep;
  if (s->n <= 0) return SB_OP_SKIPPED;
  const int width = (int)op->i[1], Hq = (int)op->i[21], Hkv = (int)op->i[22], D = (int)op->i[23], Dv = (int)op->i[24];
  const int rot = (int)op->i[9], mode = (int)op->i[7], dtype = (int)op->i[13];
  const int64_t cols = static_cast<int64_t>(Hq) * D + static_cast<int64_t>(Hkv) * (D + Dv);
  if (Hq <= 0 || Hkv <= 0 || D <= 0 || Dv <= 0 || cols > width) return sb::fail("sb_op_qkv_prepare: heads %d / %d, sizes %d / %d, row %d", Hq, Hkv, D, Dv, width), SB_OP_FAILED;
  if (rot < 0 || rot % 2 != 0 || rot > D) return sb::fail("sb_op_qkv_prepare: %d rotated elements of %d", rot, D), SB_OP_FAILED;
  if (mode < 0 || mode > 2) return sb::fail("sb_op_qkv_prepare: norm mode %d", mode), SB_OP_FAILED;
  PrepareParams p{ptr<const float>(op->i[0]), partial_count(op->i[2], op->i[3], s->n), static_cast<int64_t>(s->n) * width, width,
                  ptr<const float>(op->i[4]), ptr<const float>(op->i[5]), ptr<const float>(op->i[6]), mode, (float)op->f[0],
                  ptr<const float>(op->i[8]), rot, (int)op->i[10], (float)op->f[1], (int)op->i[11], positions(s), slots(s), ptr<void>(op->i[12]),
                  page_ref(ptr<void>(op->i[14]), ptr<const int32_t>(op->i[15]), (int)op->i[16], (int)op->i[17], op->i[18], op->i[19], op->i[20],
                           (int)op->i[25]),
                  Hq, Hkv, D, Dv, (int)op->i[26]};
  const size_t smem = static_cast<size_t>(cols) * sizeof(float);
  if (smem > 160 * 1024) return sb::fail("sb_op_qkv_prepare: a row of %lld elements does not fit the row buffer", (long long)cols), SB_OP_FAILED;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == 0) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(qkv_prepare_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    sb::launch_pdl(qkv_prepare_kernel<float>, dim3(s->n), dim3(256), smem, st, p);
  } else if (dtype == 1) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(qkv_prepare_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    sb::launch_pdl(qkv_prepare_kernel<bf16>, dim3(s->n), dim3(256), smem, st, p);
  } else {
    return sb::fail("sb_op_qkv_prepare: unsupported dtype %d", dtype), SB_OP_FAILED;
  }
  return sb::check_launch("sb_op_qkv_prepare");
}

// i: 0 attention result (float32), 1 gate's partial sums (flat), 2 their width, 3 K ranges S, 4 most tokens with a buffer per range, 5 g_off,
//    6 out, 7 out dtype, 8 H, 9 G, 10 Dv, 11 maps, 12 one gate per head
// f: 0 lambda, 1 factor behind the norm, 2 eps
SB_EXPORT int sb_op_head_gate(const SbOp* op, const SbStep* s, void* stream) {
  using namespace sbstep;
  if (s->n <= 0) return SB_OP_SKIPPED;
  const int width = (int)op->i[2], H = (int)op->i[8], G = (int)op->i[9], maps = (int)op->i[11];
  if (H <= 0 || G <= 0 || H % G != 0 || maps < 1 || maps > 2) return sb::fail("sb_op_head_gate: heads %d / %d, maps %d", H, G, maps), SB_OP_FAILED;
  HeadGateParams p{ptr<const float>(op->i[0]), ptr<const float>(op->i[1]), partial_count(op->i[3], op->i[4], s->n), static_cast<int64_t>(s->n) * width,
                   width, (int)op->i[5], ptr<void>(op->i[6]), H, G, (int)op->i[10], maps, (int)op->i[12], (float)op->f[0], (float)op->f[1],
                   (float)op->f[2]};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int shares = (4 * sb::sm_count() + s->n - 1) / s->n;          // blocks enough to fill the device when the tokens are few
  shares = shares < 1 ? 1 : shares > (H + 3) / 4 ? (H + 3) / 4 : shares;
  if (op->i[7] == 0) sb::launch_pdl(head_gate_kernel<float>, dim3(s->n, shares), dim3(128), 0, st, p);
  else if (op->i[7] == 1) sb::launch_pdl(head_gate_kernel<bf16>, dim3(s->n, shares), dim3(128), 0, st, p);
  else return sb::fail("sb_op_head_gate: unsupported dtype %d", (int)op->i[7]), SB_OP_FAILED;
  return sb::check_launch("sb_op_head_gate");
}
