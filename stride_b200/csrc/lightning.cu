// Linear attention with a decay per head ("lightning attention"), as a recurrence over a state kept per request:
//
//   S_t = decay_h * S_(t-1) + k_t v_t^T        S: [D, V] float32 per head
//   o_t = S_t^T q_t
//
// with q, k, v = silu of the projections. Everything here is 32-bit: the activations, the decay, the state and the
// sums. One kernel serves prompt portions and decoded tokens alike: a CTA owns (request of the step, head, a
// range of value columns) and walks the request's tokens of this step in order, the state in registers; it reads
// the state the step before left (or starts from zero at position 0) and writes it back at the end. A column of
// the state depends on no other column, so the value columns may be spread over CTAs and warps in any way; the
// D sums of an output are cut into parts of 16 consecutive elements, each two chains of fused multiply-adds (even and
// odd elements, ascending, then added), and the parts are added in ascending order. Neither depends on the step, so a token's output
// has the same bits however the sequence was cut into steps and whatever else the batch holds.
//
// The second kernel is what follows the recurrence: an RMS norm over all heads' outputs of a token, times a gain,
// times sigmoid of the gate projection.
#include "common.cuh"
#include "step_ops.h"

SB_DEFINE_LAST_ERROR()

namespace {

using bf16 = __nv_bfloat16;

constexpr int kChunk = 16;       // tokens staged in shared memory at a time
constexpr int kInFlight = 4;     // partial sums requested at once

__device__ __forceinline__ float silu(float a) { return a / (1.0f + expf(-a)); }

struct ScanParams {
  const float* proj;        // [P][n][width]: partial sums of the projection, columns q | k | v | (more)
  int n_partials;
  int64_t partial_stride;   // elements between partial buffers
  int width;                // elements of a token's row
  int q_off, k_off, v_off;  // first column of q, k and v
  const int32_t* meta;      // [4][meta_stride]: slot, first row, length, first position of every entry
  int meta_stride;
  const float* decay;       // [H]
  float* state;             // [slots][H][D][V]
  float* out;               // [n][H V]
  int H, D, V;
  int vc;                   // value columns a CTA owns (a multiple of 32)
  int chunk;                // tokens staged in shared memory at a time (at most kChunk)
  int activated;            // 1: proj already holds silu of the folded sums (lightning_activate_kernel ran)
};

// Sum of the projection's partial buffers at one element, ascending.
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

// 4-byte and 16-byte asynchronous copies from global to shared memory, and the wait for all of a thread's copies.
__device__ __forceinline__ void copy_async4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(dst))), "l"(src) : "memory");
}
__device__ __forceinline__ void copy_async16(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(dst))), "l"(src) : "memory");
}
__device__ __forceinline__ void copy_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void copy_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

constexpr int R = 16;   // elements of a state column a thread holds: a part of the D sums

// Two float32 fused multiply-adds in one instruction (sm_100: fma.rn.f32x2): each half rounds as a scalar fma.rn does.
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;"
      : "=l"(d)
      : "l"(*reinterpret_cast<const uint64_t*>(&a)), "l"(*reinterpret_cast<const uint64_t*>(&b)), "l"(*reinterpret_cast<const uint64_t*>(&c)));
  return *reinterpret_cast<float2*>(&d);
}

// A token's R keys and R queries of one part, as read from shared memory.
struct TokenKQ {
  float4 k[R / 4], q[R / 4];
  __device__ __forceinline__ void load(const float4* k4, const float4* q4) {
#pragma unroll
    for (int i = 0; i < R / 4; ++i) {
      k[i] = k4[i];
      q[i] = q4[i];
    }
  }
};

// One token of the recurrence for one thread: its R elements of a state column (as pairs), the token's R keys and queries
// of this part and the column's value. S <- decay S + k v; returns the part's share of the output: the even and the odd
// elements are a chain of fused multiply-adds each, ascending, and the two are added.
__device__ __forceinline__ float scan_token(float2 (&S)[R / 2], const TokenKQ& x, float vv, float decay) {
  const float2 v2 = make_float2(vv, vv), d2 = make_float2(decay, decay), zero = make_float2(0.0f, 0.0f);
  float2 acc = zero;
#pragma unroll
  for (int i = 0; i < R / 4; ++i) {
    S[2 * i] = fma2(d2, S[2 * i], fma2(make_float2(x.k[i].x, x.k[i].y), v2, zero));
    acc = fma2(S[2 * i], make_float2(x.q[i].x, x.q[i].y), acc);
    S[2 * i + 1] = fma2(d2, S[2 * i + 1], fma2(make_float2(x.k[i].z, x.k[i].w), v2, zero));
    acc = fma2(S[2 * i + 1], make_float2(x.q[i].z, x.q[i].w), acc);
  }
  return acc.x + acc.y;
}

// Named barriers of lightning_scan_kernel (id 0 is __syncthreads): two of each kind, one per buffer.
enum { kBarFull = 1, kBarEmpty = 4, kBarOutFull = 7, kBarOutEmpty = 9 };
constexpr int kStages = 2;      // staging buffers of the recurrence's inputs (2 or 3): the loads run kStages - 1 chunks ahead
template <int BASE>
__device__ __forceinline__ void bar_sync(int b, int count) {
  if (b == 0) asm volatile("bar.sync %0, %1;" ::"n"(BASE), "r"(count) : "memory");
  else if (b == 1) asm volatile("bar.sync %0, %1;" ::"n"(BASE + 1), "r"(count) : "memory");
  else asm volatile("bar.sync %0, %1;" ::"n"(BASE + 2), "r"(count) : "memory");
}
template <int BASE>
__device__ __forceinline__ void bar_arrive(int b, int count) {
  if (b == 0) asm volatile("bar.arrive %0, %1;" ::"n"(BASE), "r"(count) : "memory");
  else if (b == 1) asm volatile("bar.arrive %0, %1;" ::"n"(BASE + 1), "r"(count) : "memory");
  else asm volatile("bar.arrive %0, %1;" ::"n"(BASE + 2), "r"(count) : "memory");
}

// Prompt portions (and any step with an entry of more than one token). `proj` holds the activated sums (silu applied by
// lightning_activate_kernel; one buffer). The CTA's first parts * vc threads compute: thread = (part of the D sums, value
// column), a part's threads being whole warps, so that the keys and queries of a part are read from shared memory by
// broadcast. Behind them one warp loads: it keeps the q, k, v rows of the next chunk of kChunk tokens on their way into
// the other staging buffer (asynchronous copies); and vc / 32 warps store: they add the parts of the outputs of the chunk
// before and write them to global memory, while the computing warps are already at the next chunk. The three groups meet
// only at named barriers, one pair per buffer and direction.
template <int VEC>
__global__ void __launch_bounds__(576) lightning_scan_kernel(const ScanParams p) {
  extern __shared__ __align__(16) float smem[];
  sb::grid_launch_dependents();
  const int e = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * p.vc;
  const int vc = p.vc, parts = (p.D + R - 1) / R, Dp = parts * R;
  const int vn = min(vc, p.V - c0);
  const int NC = parts * vc, NS = vc;                  // computing threads, storing threads (one warp loads)
  const int stage = kChunk * (2 * Dp + vc);            // floats of a staging buffer: q [kChunk][Dp], k [kChunk][Dp], v [kChunk][vc]
  const int outs = parts * kChunk * vc;                // floats of an output buffer: [parts][kChunk][vc]
  float* so = smem + kStages * stage;
  const int slot = p.meta[e], row0 = p.meta[p.meta_stride + e], len = p.meta[2 * p.meta_stride + e],
            pos0 = p.meta[3 * p.meta_stride + e];
  const int chunks = (len + kChunk - 1) / kChunk;
  if (Dp != p.D || vn != vc) {
    // nothing writes the cells beyond D and beyond the CTA's existing columns: they are zero for good
    for (int b = 0; b < kStages; ++b)
      for (int t = 0; t < kChunk; ++t) {
        float* row = smem + b * stage;
        for (int d = p.D + threadIdx.x; d < Dp; d += blockDim.x) row[t * Dp + d] = row[(kChunk + t) * Dp + d] = 0.0f;
        for (int j = vn + threadIdx.x; j < vc; j += blockDim.x) row[2 * kChunk * Dp + t * vc + j] = 0.0f;
      }
  }
  sb::grid_dependency_wait();
  __syncthreads();
  const int tid = threadIdx.x;
  if (tid < NC) {
    // ---------------------------------------------------------------- the recurrence
    const int part = tid / vc, cl = tid % vc;
    const float decay = p.decay[h];
    const bool live = cl < vn;
    const int dn = min(R, p.D - part * R);            // elements of this part that exist
    float* st = p.state + ((static_cast<int64_t>(slot) * p.H + h) * p.D + part * R) * p.V + c0 + cl;
    float2 S[R / 2];
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const float v = (pos0 > 0 && live && i < dn) ? st[static_cast<int64_t>(i) * p.V] : 0.0f;
      if (i & 1) S[i / 2].y = v;
      else S[i / 2].x = v;
    }
    for (int c = 0, sb_ = 0; c < chunks; ++c, sb_ = sb_ + 1 == kStages ? 0 : sb_ + 1) {
      const int b = c & 1, nt = min(kChunk, len - c * kChunk);
      const float* sq = smem + sb_ * stage;
      bar_sync<kBarFull>(sb_, NC + 32);
      if (c >= 2) bar_sync<kBarOutEmpty>(b, NC + NS);
      const float4* q4 = reinterpret_cast<const float4*>(sq + part * R);
      const float4* k4 = reinterpret_cast<const float4*>(sq + kChunk * Dp + part * R);
      const float* sv = sq + 2 * kChunk * Dp + cl;
      float* sop = so + b * outs + part * kChunk * vc + cl;
#pragma unroll 2
      for (int t = 0; t < nt; ++t) {
        TokenKQ x;
        x.load(k4, q4);
        *sop = scan_token(S, x, *sv, decay);
        k4 += Dp / 4;
        q4 += Dp / 4;
        sv += vc;
        sop += vc;
      }
      if (c + kStages < chunks) bar_arrive<kBarEmpty>(sb_, NC + 32);
      bar_arrive<kBarOutFull>(b, NC + NS);
    }
    if (live) {
#pragma unroll
      for (int i = 0; i < R; ++i)
        if (i < dn) st[static_cast<int64_t>(i) * p.V] = (i & 1) ? S[i / 2].y : S[i / 2].x;
    }
  } else if (tid < NC + 32) {
    // ---------------------------------------------------------------- the loads
    const int lane = tid - NC;
    const int du = p.D / VEC, vu = vn / VEC;          // (VEC == 4 only when D and the columns are multiples of four)
    // a chunk's copies are requested before the chunks in front of it are waited for and announced
    auto request = [&](int c) {
      const int sb_ = c % kStages, nt = min(kChunk, len - c * kChunk);
      if (c >= kStages) bar_sync<kBarEmpty>(sb_, NC + 32);
      float* sq = smem + sb_ * stage;
      float* sk = sq + kChunk * Dp;
      float* sv = sk + kChunk * Dp;
      for (int t = 0; t < nt; ++t) {
        const float* src = p.proj + static_cast<int64_t>(row0 + c * kChunk + t) * p.width;
        const float* gq = src + p.q_off + h * p.D;
        const float* gk = src + p.k_off + h * p.D;
        const float* gv = src + p.v_off + h * p.V + c0;
        for (int u = lane; u < du; u += 32) {
          if (VEC == 4) {
            copy_async16(sq + t * Dp + 4 * u, gq + 4 * u);
            copy_async16(sk + t * Dp + 4 * u, gk + 4 * u);
          } else {
            copy_async4(sq + t * Dp + u, gq + u);
            copy_async4(sk + t * Dp + u, gk + u);
          }
        }
        for (int u = lane; u < vu; u += 32) {
          if (VEC == 4) copy_async16(sv + t * vc + 4 * u, gv + 4 * u);
          else copy_async4(sv + t * vc + u, gv + u);
        }
      }
      copy_async_commit();
    };
    constexpr int kAhead = kStages - 1;
    for (int c = 0; c < kAhead && c < chunks; ++c) request(c);
    for (int c = 0; c < chunks; ++c) {
      if (c + kAhead < chunks) request(c + kAhead);
      const int pending = min(kAhead, chunks - 1 - c);      // younger chunks that may still be on their way
      if (pending >= 2) copy_async_wait<2>();
      else if (pending == 1) copy_async_wait<1>();
      else copy_async_wait<0>();
      bar_arrive<kBarFull>(c % kStages, NC + 32);
    }
  } else {
    // ---------------------------------------------------------------- the outputs: parts added in ascending order
    const int j = tid - NC - 32;                      // this thread's value column
    for (int c = 0; c < chunks; ++c) {
      const int b = c & 1, nt = min(kChunk, len - c * kChunk);
      bar_sync<kBarOutFull>(b, NC + NS);
      if (j < vn) {
        const float* src = so + b * outs + j;
        float* dst = p.out + static_cast<int64_t>(row0 + c * kChunk) * p.H * p.V + h * p.V + c0 + j;
        for (int t = 0; t < nt; ++t) {
          float sum = src[t * vc];
          for (int q = 1; q < parts; ++q) sum += src[(q * kChunk + t) * vc];
          dst[static_cast<int64_t>(t) * p.H * p.V] = sum;
        }
      }
      if (c + 2 < chunks) bar_arrive<kBarOutEmpty>(b, NC + NS);
    }
  }
}

// The same for steps in which every entry brings one token (decoding): nothing is staged ahead and no loop runs; a CTA is
// (entry, head, 32 value columns), its warps the parts. The state's loads are requested first, the token's q, k, v (partial
// sums folded, silu) go to shared memory meanwhile. Same operations in the same order as lightning_scan_kernel: same bits.
__global__ void __launch_bounds__(512, 2) lightning_step_kernel(const ScanParams p) {
  extern __shared__ __align__(16) float smem[];
  sb::grid_launch_dependents();
  const int e = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * 32;
  const int parts = blockDim.x >> 5, Dp = parts * R;
  const int part = threadIdx.x >> 5, cl = threadIdx.x & 31;
  float* sq = smem;            // [Dp]
  float* sk = sq + Dp;         // [Dp]
  float* sv = sk + Dp;         // [32]
  float* so = sv + 32;         // [parts][32]
  const int slot = p.meta[e], row = p.meta[p.meta_stride + e], pos0 = p.meta[3 * p.meta_stride + e];
  const float decay = p.decay[h];
  const bool live = c0 + cl < p.V;
  const int dn = min(R, p.D - part * R);
  float* st = p.state + ((static_cast<int64_t>(slot) * p.H + h) * p.D + part * R) * p.V + c0 + cl;
  sb::grid_dependency_wait();
  float2 S[R / 2];
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const float v = (pos0 > 0 && live && i < dn) ? st[static_cast<int64_t>(i) * p.V] : 0.0f;
    if (i & 1) S[i / 2].y = v;
    else S[i / 2].x = v;
  }
  const float* src = p.proj + static_cast<int64_t>(row) * p.width;
  for (int j = threadIdx.x; j < 2 * Dp + 32; j += blockDim.x) {
    float v = 0.0f;
    if (j < 2 * Dp) {
      const bool is_k = j >= Dp;
      const int d = is_k ? j - Dp : j;
      if (d < p.D) {
        v = folded(src + (is_k ? p.k_off : p.q_off) + h * p.D + d, p.n_partials, p.partial_stride);
        if (!p.activated) v = silu(v);
      }
    } else if (c0 + j - 2 * Dp < p.V) {
      v = folded(src + p.v_off + h * p.V + c0 + j - 2 * Dp, p.n_partials, p.partial_stride);
      if (!p.activated) v = silu(v);
    }
    smem[j] = v;
  }
  __syncthreads();
  TokenKQ x;
  x.load(reinterpret_cast<const float4*>(sk + part * R), reinterpret_cast<const float4*>(sq + part * R));
  so[part * 32 + cl] = scan_token(S, x, sv[cl], decay);
  if (live) {
#pragma unroll
    for (int i = 0; i < R; ++i)
      if (i < dn) st[static_cast<int64_t>(i) * p.V] = (i & 1) ? S[i / 2].y : S[i / 2].x;
  }
  __syncthreads();
  if (part == 0 && live) {
    float sum = so[cl];
    for (int q = 1; q < parts; ++q) sum += so[q * 32 + cl];
    p.out[static_cast<int64_t>(row) * p.H * p.V + h * p.V + c0 + cl] = sum;
  }
}

// act[r, j] = silu(sum of the partial buffers at [r, j]) for the first `cols` columns of every row: what the recurrence
// reads, made once for all of a long step's tokens instead of by every CTA that needs a token's keys and queries.
__global__ void lightning_activate_kernel(const float* __restrict__ proj, int n_partials, int64_t partial_stride, int width,
                                          float* __restrict__ act, int n, int cols) {
  sb::grid_launch_dependents();
  sb::grid_dependency_wait();
  const int64_t total = static_cast<int64_t>(n) * cols;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / cols, j = i % cols;
    act[i] = silu(folded(proj + r * width + j, n_partials, partial_stride));
  }
}

// out[r, j] = o[r, j] / sqrt(mean_j(o[r, :]^2) + eps) * gain[j] * sigmoid(gate[r, j]); the gate is a column range of the
// projection's partial sums. One block per row.
template <class TW, class TO>
__global__ void __launch_bounds__(1024) gated_rmsnorm_kernel(const float* __restrict__ o, const float* __restrict__ proj, int n_partials,
                                                              int64_t partial_stride, int width, int g_off,
                                                              const TW* __restrict__ gain, TO* __restrict__ out, int W, float eps) {
  extern __shared__ __align__(16) float row[];
  __shared__ float red[32];
  sb::grid_launch_dependents();
  sb::grid_dependency_wait();
  const int64_t r = blockIdx.x;
  float ss = 0.0f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float v = o[r * W + i];
    row[i] = v;
    ss = fmaf(v, v, ss);
  }
  const float scale = 1.0f / sqrtf(sb::block_sum(ss, red) / static_cast<float>(W) + eps);
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float g = folded(proj + r * width + g_off + i, n_partials, partial_stride);
    const float gate = 1.0f / (1.0f + expf(-g));
    out[r * W + i] = sb::narrow<TO>(row[i] * scale * sb::widen(gain[i]) * gate);
  }
}

}  // namespace

// The recurrence for every entry of a step. proj: the projection's partial sums [n_partials][n][width] (float32) with
// q at column q_off (H D), k at k_off (H D), v at v_off (H V); meta: the step's entry records [4][meta_stride]
// on the device; state [slots][H][D][V] float32; out [n][H V] float32.
// act: scratch [n][q, k, v columns] float32. Steps in which an entry brings several tokens apply the activation in a kernel
// of its own first; steps of single tokens apply it inside theirs (the same function on the same sums: the same bits).
// `ready` = 1: `proj` already holds q, k and v as the recurrence takes them (another design's activation, made by a kernel in front), and
// nothing is applied here.
SB_EXPORT int sb_lightning_scan_ex(const float* proj, int n_partials, int64_t partial_stride, int width, int q_off, int k_off, int v_off,
                                   const int32_t* meta, int meta_stride, int entries, int n, const float* decay, float* state, float* out,
                                   float* act, int H, int D, int V, int ready, cudaStream_t stream) {
  if (entries <= 0 || n <= 0) return 0;
  if (H <= 0 || D <= 0 || V <= 0 || D > 256) return sb::fail("sb_lightning_scan: heads %d, key size %d (at most 256), value size %d", H, D, V);
  if (n_partials < 1) return sb::fail("sb_lightning_scan: n_partials must be >= 1");
  const int parts = (D + R - 1) / R, Dp = parts * R;
  // value columns a CTA: whole warps, at most 576 threads with the loading and storing warps, and as few CTAs as still fill the device
  const int v_warps = (V + 31) / 32;
  int vw = min(min(v_warps, (576 - 32) / (32 * parts + 32)), 2);
  const long long sms = sb::sm_count();
  while (vw > 1 && static_cast<long long>(entries) * H * ((v_warps + vw - 1) / vw) < 2 * sms) --vw;
  if (n == entries) {     // one token an entry (decoding): small CTAs, many of them, nothing staged ahead
    ScanParams p{proj, n_partials, partial_stride, width, q_off, k_off, v_off, meta, meta_stride, decay, state, out, H, D, V, 32, 1, ready};
    sb::launch_pdl(lightning_step_kernel, dim3(entries, H, v_warps), dim3(parts * 32), sizeof(float) * (2 * Dp + 32 + parts * 32), stream, p);
    return sb::check_launch("sb_lightning_scan");
  }
  // steps with longer entries: the activation once for all tokens, then the recurrence
  if (act == nullptr && !ready) return sb::fail("sb_lightning_scan: a step with an entry of several tokens needs the scratch for the activated sums");
  const int cols = ready ? width : max(max(q_off + H * D, k_off + H * D), v_off + H * V);
  if (ready) {
    if (n_partials != 1) return sb::fail("sb_lightning_scan: ready-made q, k, v come as one buffer");
    act = const_cast<float*>(proj);
  } else {
    const int64_t total = static_cast<int64_t>(n) * cols;
    const int blocks = static_cast<int>((total + 255) / 256 < sms * 16 ? (total + 255) / 256 : sms * 16);
    sb::launch_pdl(lightning_activate_kernel, dim3(blocks), dim3(256), 0, stream, proj, n_partials, partial_stride, width, act, n, cols);
  }
  ScanParams p{act, 1, 0, cols, q_off, k_off, v_off, meta, meta_stride, decay, state, out, H, D, V, 32 * vw, kChunk, 1};
  const dim3 grid(entries, H, (v_warps + vw - 1) / vw);
  const int threads = parts * 32 * vw + 32 + 32 * vw;
  const size_t smem = sizeof(float) * (static_cast<size_t>(kStages) * kChunk * (2 * Dp + p.vc) + static_cast<size_t>(2) * kChunk * p.vc * parts);
  if (smem > 200 * 1024) return sb::fail("sb_lightning_scan: key size %d does not fit shared memory", D);
  const bool vec = D % 4 == 0 && V % 4 == 0 && q_off % 4 == 0 && k_off % 4 == 0 && v_off % 4 == 0 &&
                   (reinterpret_cast<uintptr_t>(act) & 15) == 0 && cols % 4 == 0;
  if (vec) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(lightning_scan_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    sb::launch_pdl(lightning_scan_kernel<4>, grid, dim3(threads), smem, stream, p);
  } else {
    if (smem > 48 * 1024) cudaFuncSetAttribute(lightning_scan_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    sb::launch_pdl(lightning_scan_kernel<1>, grid, dim3(threads), smem, stream, p);
  }
  return sb::check_launch("sb_lightning_scan");
}

SB_EXPORT int sb_lightning_scan(const float* proj, int n_partials, int64_t partial_stride, int width, int q_off, int k_off, int v_off,
                                const int32_t* meta, int meta_stride, int entries, int n, const float* decay, float* state, float* out,
                                float* act, int H, int D, int V, cudaStream_t stream) {
  return sb_lightning_scan_ex(proj, n_partials, partial_stride, width, q_off, k_off, v_off, meta, meta_stride, entries, n, decay, state, out, act,
                              H, D, V, 0, stream);
}

// out [n][W] (float32 or bfloat16) = rmsnorm(o [n][W] float32) * gain * sigmoid(gate), the gate being columns g_off.. of `proj`.
SB_EXPORT int sb_gated_rmsnorm(const float* o, const float* proj, int n_partials, int64_t partial_stride, int width, int g_off,
                               const void* gain, int gain_dtype, void* out, int out_dtype, int n, int W, float eps, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (n_partials < 1) return sb::fail("sb_gated_rmsnorm: n_partials must be >= 1");
  const size_t smem = static_cast<size_t>(W) * sizeof(float);
  if (smem > 200 * 1024) return sb::fail("sb_gated_rmsnorm: width %d does not fit the row buffer", W);
  const int threads = W >= 4096 ? 1024 : W >= 2048 ? 512 : W >= 512 ? 256 : 128;
#define SB_GN(TW, TO)                                                                                                           \
  do {                                                                                                                          \
    if (smem > 48 * 1024) cudaFuncSetAttribute(gated_rmsnorm_kernel<TW, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    sb::launch_pdl(gated_rmsnorm_kernel<TW, TO>, n, threads, smem, stream, o, proj, n_partials, partial_stride, width, g_off,   \
                   static_cast<const TW*>(gain), static_cast<TO*>(out), W, eps);                                                \
  } while (0)
  if (gain_dtype == 0 && out_dtype == 0) SB_GN(float, float);
  else if (gain_dtype == 0 && out_dtype == 1) SB_GN(float, bf16);
  else if (gain_dtype == 1 && out_dtype == 0) SB_GN(bf16, float);
  else if (gain_dtype == 1 && out_dtype == 1) SB_GN(bf16, bf16);
  else return sb::fail("sb_gated_rmsnorm: unsupported dtypes gain=%d out=%d", gain_dtype, out_dtype);
#undef SB_GN
  return sb::check_launch("sb_gated_rmsnorm");
}

// ------------------------------------------------------------------ operations of the native step program (step_ops.h)
// i: 0 projection partial sums (flat), 1 their width, 2 K ranges S, 3 most tokens with a buffer per range, 4 q_off, 5 k_off,
//    6 v_off, 7 decay (float32 [H]), 8 state, 9 out (float32 [n, H V]), 10 H, 11 D, 12 V, 13 scratch for the activated sums,
//    14 q, k, v are ready-made (one buffer, nothing applied)
SB_EXPORT int sb_op_lightning_scan(const SbOp* op, const SbStep* s, void* stream) {
  using namespace sbstep;
  if (s->n <= 0) return SB_OP_SKIPPED;
  const int P = partial_count(op->i[2], op->i[3], s->n);
  return sb_lightning_scan_ex(ptr<const float>(op->i[0]), P, static_cast<int64_t>(s->n) * op->i[1], (int)op->i[1], (int)op->i[4], (int)op->i[5],
                              (int)op->i[6], entry_meta(s), s->max_rows, s->entries, s->n, ptr<const float>(op->i[7]), ptr<float>(op->i[8]),
                              ptr<float>(op->i[9]), ptr<float>(op->i[13]), (int)op->i[10], (int)op->i[11], (int)op->i[12], (int)op->i[14],
                              static_cast<cudaStream_t>(stream));
}

// i: 0 o (float32 [n, W]), 1 projection partial sums (flat), 2 their width, 3 K ranges S, 4 most tokens with a buffer per range,
//    5 g_off, 6 gain, 7 gain dtype, 8 out, 9 out dtype, 10 W
// f: 0 eps
SB_EXPORT int sb_op_gated_rmsnorm(const SbOp* op, const SbStep* s, void* stream) {
  using namespace sbstep;
  if (s->n <= 0) return SB_OP_SKIPPED;
  const int P = partial_count(op->i[3], op->i[4], s->n);
  return sb_gated_rmsnorm(ptr<const float>(op->i[0]), ptr<const float>(op->i[1]), P, static_cast<int64_t>(s->n) * op->i[2], (int)op->i[2],
                          (int)op->i[5], ptr<const void>(op->i[6]), (int)op->i[7], ptr<void>(op->i[8]), (int)op->i[9], s->n, (int)op->i[10],
                          static_cast<float>(op->f[0]), static_cast<cudaStream_t>(stream));
}

// ---------------------------------------------------------------------------------------------------------------------------------
// Retention: the same recurrence with rotated, not activated, queries and keys, and what other linear-attention designs put behind it.
//
// `rotate_qk_kernel`: out[r] = [q | k | v] in 32-bit from the projection's partial sums: the first `rot` elements of every q and k head
// turned by the token's position (pairs (i, i + rot / 2), or (2i, 2i + 1) when interleaved), k times a constant behind the rotation, v
// as it is. The recurrence then takes the buffer as ready-made.
//
// `group_norm_gate_kernel`: every head's result divided by its root mean square, times a gain of the head's size shared by all heads
// (or none), times silu or sigmoid of the gate, a column range of some projection's partial sums. A warp per (token, head).
namespace {

struct RotateParams {
  const float* proj;
  int n_partials;
  int64_t partial_stride;
  int width, q_off, k_off, v_off;
  const int32_t* positions;
  const float* cos_sin;      // [positions][rot / 2][2]
  int rot, interleaved;
  float k_scale;
  float* out;                // [n][2 H D + H V]
  int H, D, V;
};

__global__ void __launch_bounds__(256) rotate_qk_kernel(RotateParams p) {
  sb::grid_launch_dependents();
  const int row = blockIdx.x, nqk = 2 * p.H * p.D, cols = nqk + p.H * p.V, rh = p.rot / 2;
  const int pos = p.positions[row];
  sb::grid_dependency_wait();
  const float* src = p.proj + static_cast<int64_t>(row) * p.width;
  float* dst = p.out + static_cast<int64_t>(row) * cols;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < cols; i += gridDim.y * blockDim.x) {
    if (i >= nqk) {
      dst[i] = folded(src + p.v_off + (i - nqk), p.n_partials, p.partial_stride);
      continue;
    }
    const bool is_k = i >= p.H * p.D;
    const int e = is_k ? i - p.H * p.D : i, d = e % p.D;
    const float* at = src + (is_k ? p.k_off : p.q_off) + e;
    float v = folded(at, p.n_partials, p.partial_stride);
    if (d < p.rot) {
      int pair, other;
      bool low;
      if (p.interleaved) pair = d >> 1, low = (d & 1) == 0, other = low ? 1 : -1;
      else low = d < rh, pair = low ? d : d - rh, other = low ? rh : -rh;
      const float b = folded(at + other, p.n_partials, p.partial_stride);
      const float2 cs = *reinterpret_cast<const float2*>(p.cos_sin + (static_cast<int64_t>(pos) * rh + pair) * 2);
      v = low ? __fsub_rn(__fmul_rn(v, cs.x), __fmul_rn(b, cs.y)) : __fadd_rn(__fmul_rn(v, cs.x), __fmul_rn(b, cs.y));
    }
    dst[i] = is_k ? __fmul_rn(v, p.k_scale) : v;
  }
}

struct GroupGateParams {
  const float* o;            // [n][H V]
  const float* proj;         // the gate's partial sums [P][n][width], columns g_off ..
  int n_partials;
  int64_t partial_stride;
  int width, g_off;
  const void* gain;          // [V] or null
  int gain_bf16;
  void* out;
  int n, H, V, silu_gate;
  float eps;
};

template <class TO>
__global__ void __launch_bounds__(128) group_norm_gate_kernel(GroupGateParams p) {
  sb::grid_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int64_t unit = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  sb::grid_dependency_wait();
  if (unit >= static_cast<int64_t>(p.n) * p.H) return;
  const int64_t row = unit / p.H;
  const int h = static_cast<int>(unit % p.H);
  const float* o = p.o + unit * p.V;
  const float* gate = p.proj + row * p.width + p.g_off + h * p.V;
  float ss = 0.0f;
  for (int d = lane; d < p.V; d += 32) ss = fmaf(o[d], o[d], ss);
  for (int k = 16; k > 0; k >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, k);
  const float r = 1.0f / sqrtf(ss / static_cast<float>(p.V) + p.eps);
  TO* out = static_cast<TO*>(p.out) + unit * p.V;
  for (int d = lane; d < p.V; d += 32) {
    float v = __fmul_rn(o[d], r);
    if (p.gain != nullptr) v = __fmul_rn(v, p.gain_bf16 ? __bfloat162float(static_cast<const bf16*>(p.gain)[d]) : static_cast<const float*>(p.gain)[d]);
    const float g = folded(gate + d, p.n_partials, p.partial_stride);
    const float sg = 1.0f / (1.0f + expf(-g));
    out[d] = sb::narrow<TO>(__fmul_rn(v, p.silu_gate ? g * sg : sg));
  }
}

}  // namespace

// i: 0 projection partial sums (flat), 1 their width, 2 K ranges S, 3 most tokens with a buffer per range, 4 q_off, 5 k_off, 6 v_off, 7 cos_sin,
//    8 rot, 9 interleaved pairs, 10 out (float32 [n][2 H D + H V]), 11 H, 12 D, 13 V      f: 0 the constant on k
SB_EXPORT int sb_op_rotate_qk(const SbOp* op, const SbStep* s, void* stream) {
  using namespace sbstep;
  if (s->n <= 0) return SB_OP_SKIPPED;
  const int width = (int)op->i[1], rot = (int)op->i[8], H = (int)op->i[11], D = (int)op->i[12], V = (int)op->i[13];
  if (rot < 0 || rot % 2 != 0 || rot > D) return sb::fail("sb_op_rotate_qk: %d rotated elements of %d", rot, D), SB_OP_FAILED;
  RotateParams p{ptr<const float>(op->i[0]), partial_count(op->i[2], op->i[3], s->n), static_cast<int64_t>(s->n) * width, width, (int)op->i[4],
                 (int)op->i[5], (int)op->i[6], positions(s), ptr<const float>(op->i[7]), rot, (int)op->i[9], (float)op->f[0], ptr<float>(op->i[10]),
                 H, D, V};
  const int cols = 2 * H * D + H * V;
  sb::launch_pdl(rotate_qk_kernel, dim3(s->n, (cols + 1023) / 1024), dim3(256), 0, static_cast<cudaStream_t>(stream), p);
  return sb::check_launch("sb_op_rotate_qk");
}

// i: 0 o (float32 [n, H V]), 1 the gate's partial sums (flat), 2 their width, 3 K ranges S, 4 most tokens with a buffer per range, 5 g_off,
//    6 gain ([V], or 0), 7 gain dtype, 8 out, 9 out dtype, 10 H, 11 V, 12 the gate's activation (0 sigmoid, 1 silu)      f: 0 eps
SB_EXPORT int sb_op_group_norm_gate(const SbOp* op, const SbStep* s, void* stream) {
  using namespace sbstep;
  if (s->n <= 0) return SB_OP_SKIPPED;
  const int width = (int)op->i[2];
  GroupGateParams p{ptr<const float>(op->i[0]), ptr<const float>(op->i[1]), partial_count(op->i[3], op->i[4], s->n), static_cast<int64_t>(s->n) * width,
                    width, (int)op->i[5], ptr<const void>(op->i[6]), (int)(op->i[7] == 1), ptr<void>(op->i[8]), s->n, (int)op->i[10], (int)op->i[11],
                    (int)op->i[12], (float)op->f[0]};
  const int64_t units = static_cast<int64_t>(p.n) * p.H;
  const dim3 grid(static_cast<unsigned>((units + 3) / 4));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (op->i[9] == 0) sb::launch_pdl(group_norm_gate_kernel<float>, grid, dim3(128), 0, st, p);
  else if (op->i[9] == 1) sb::launch_pdl(group_norm_gate_kernel<bf16>, grid, dim3(128), 0, st, p);
  else return sb::fail("sb_op_group_norm_gate: unsupported dtype %d", (int)op->i[9]), SB_OP_FAILED;
  return sb::check_launch("sb_op_group_norm_gate");
}
