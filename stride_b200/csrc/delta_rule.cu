// The gated delta rule: linear attention whose state forgets per key channel and is corrected, not only added to.
//
// Per token t of a request and head h (key size D, value size V, state S [D][V], float32, zero at position 0):
//
//   S <- diag(g_t) S          g_t [D] in (0, 1): one decay per key channel
//   u  = beta_t (v_t - S^T k_t)
//   S <- S + k_t u^T
//   o_t = S^T q_t             (read after the write: a token's own pair already counts)
//
// A column of S depends on no other column, so a thread owns a slice of one column and the columns are spread over threads and CTAs; the
// two sums over the key channels are made per thread in ascending channels and then over the P threads of a column by xor shuffles, P a
// function of D alone: a token's result has the same bits in a prompt, in a portion and decoded alone.
//
// `delta_prepare_kernel` makes what the recurrence takes, in 32-bit, from the projections' partial sums: q, k and v pass a short causal
// convolution per channel over the request's last `taps` inputs (the step's own rows, then the request's record of its last inputs, then
// zeros) and silu; q and k are made unit vectors per head, x / sqrt(sum x^2 + 1e-6), q also times D^-1/2; beta = sigmoid(.);
// g = exp(-exp(A_h) softplus(a + dt)). `delta_conv_state_kernel` then moves the record of last inputs on. The request's record is
// [S (H D V) | last inputs ((taps - 1) C)] float32, C = 2 G D + H V channels.
#include "common.cuh"
#include "step_ops.h"

SB_DEFINE_LAST_ERROR()

namespace {

constexpr int kInFlight = 8;
constexpr int kMaxTaps = 8;

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

__device__ __forceinline__ float silu(float a) { return a / (1.0f + expf(-a)); }
__device__ __forceinline__ float softplus(float a) { return a > 20.0f ? a : log1pf(expf(a)); }

struct PrepareParams {
  const float* proj;         // [P1][n][width1]: q (G D) | k (G D) | v (H V) | beta (H) | whatever else
  int n1;
  int64_t stride1;
  int width1;
  const float* proj2;        // [P2][n][width2]: the decay's argument a (H D) | whatever else
  int n2;
  int64_t stride2;
  int width2;
  const float* conv;         // [C][taps], the last column the current token's
  const float* a_log;        // [H]
  const float* dt_bias;      // [H D]
  const int32_t* meta;       // [4][meta_stride]: slot, first row, length, first position of every entry
  int meta_stride, entries;
  const int32_t* positions;
  float* record;             // [slots][record_size]
  int64_t record_size, conv_offset;
  float* out;                // [n][2 G D + H V + H D + H]: q | k | v | g | beta
  int H, G, D, V, taps;
};

// The conv's input of channel c at position t of the entry (first row r0, first position p0): a row of the step, the record, or zero.
__device__ __forceinline__ float conv_input(const PrepareParams& p, const float* last, int r0, int p0, int t, int c, int C) {
  if (t >= p0) return folded(p.proj + static_cast<int64_t>(r0 + t - p0) * p.width1 + c, p.n1, p.stride1);
  if (t >= 0) return last[static_cast<int64_t>(p.taps - 1 - (p0 - t)) * C + c];
  return 0.0f;
}

constexpr int kSlab = 256;   // most channels of a unit of work (a block's threads: 128 for heads of up to 128 channels, else 256)

// A block per (token, share of the token's units). A unit is a q or k head (convolution, silu, the head made a unit vector: the squares by
// the first warp's lanes over every 32nd channel in ascending order, then xor shuffles), a slab of v channels (convolution, silu), or a slab
// of decays and betas. How the units are dealt to blocks changes no arithmetic.
__global__ void __launch_bounds__(256) delta_prepare_kernel(PrepareParams p) {
  __shared__ float both[2][kSlab];
  __shared__ float scales[2];
  __shared__ int found[3];
  sb::grid_launch_dependents();
  const int row = blockIdx.x, nqk = 2 * p.G * p.D, C = nqk + p.H * p.V, tail = p.H * p.D + p.H;
  const int slab = blockDim.x;
  const int v_slabs = (p.H * p.V + slab - 1) / slab, t_slabs = (tail + slab - 1) / slab, units = 2 * p.G + v_slabs + t_slabs;
  const int lane = threadIdx.x & 31;
  if (threadIdx.x == 0) found[0] = 0, found[1] = row, found[2] = p.positions[row];
  __syncthreads();
  for (int e = threadIdx.x; e < p.entries; e += blockDim.x) {
    const int r0 = p.meta[p.meta_stride + e], len = p.meta[2 * p.meta_stride + e];
    if (row >= r0 && row < r0 + len) found[0] = p.meta[e], found[1] = r0, found[2] = p.meta[3 * p.meta_stride + e];
  }
  __syncthreads();
  const int slot = found[0], r0 = found[1], p0 = found[2], pos = p0 + (row - r0);
  const float* last = p.record + static_cast<int64_t>(slot) * p.record_size + p.conv_offset;
  float* out = p.out + static_cast<int64_t>(row) * (C + tail);
  auto convolved = [&](int c) {
    float acc = 0.0f;
    for (int j = 0; j < p.taps; ++j) acc = fmaf(p.conv[c * p.taps + j], conv_input(p, last, r0, p0, pos - (p.taps - 1 - j), c, C), acc);
    return silu(acc);
  };
  sb::grid_dependency_wait();
  int turn = 0;
  for (int u = blockIdx.y; u < units; u += gridDim.y) {
    if (u < 2 * p.G) {
      float* vals = both[turn];          // (the head before this one may still be read from the other buffer)
      float& unit_scale = scales[turn];
      turn ^= 1;
      for (int d = threadIdx.x; d < p.D; d += blockDim.x) vals[d] = convolved(u * p.D + d);
      __syncthreads();
      if (threadIdx.x < 32) {
        float ss = 0.0f;
        for (int d = lane; d < p.D; d += 32) ss = fmaf(vals[d], vals[d], ss);
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        float r = 1.0f / sqrtf(ss + 1e-6f);
        if (u < p.G) r = __fmul_rn(r, 1.0f / sqrtf(static_cast<float>(p.D)));
        if (lane == 0) unit_scale = r;
      }
      __syncthreads();
      for (int d = threadIdx.x; d < p.D; d += blockDim.x) out[u * p.D + d] = __fmul_rn(vals[d], unit_scale);
    } else if (u < 2 * p.G + v_slabs) {
      const int c = nqk + (u - 2 * p.G) * slab + threadIdx.x;
      if (c < C) out[c] = convolved(c);
    } else {
      const int e = (u - 2 * p.G - v_slabs) * slab + threadIdx.x;
      if (e < p.H * p.D) {
        const float a = __fadd_rn(folded(p.proj2 + static_cast<int64_t>(row) * p.width2 + e, p.n2, p.stride2), p.dt_bias[e]);
        out[C + e] = expf(-expf(p.a_log[e / p.D]) * softplus(a));
      } else if (e < tail) {
        const int h = e - p.H * p.D;
        out[C + e] = 1.0f / (1.0f + expf(-folded(p.proj + static_cast<int64_t>(row) * p.width1 + C + h, p.n1, p.stride1)));
      }
    }
  }
}

// The record of a request's last taps - 1 inputs after the step: positions end - (taps - 1) .. end - 1.
__global__ void __launch_bounds__(256) delta_conv_state_kernel(PrepareParams p) {
  sb::grid_launch_dependents();
  const int e = blockIdx.x, C = 2 * p.G * p.D + p.H * p.V;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  const int slot = p.meta[e], r0 = p.meta[p.meta_stride + e], len = p.meta[2 * p.meta_stride + e], p0 = p.meta[3 * p.meta_stride + e];
  float* last = p.record + static_cast<int64_t>(slot) * p.record_size + p.conv_offset;
  sb::grid_dependency_wait();
  if (c >= C) return;
  float keep[kMaxTaps];
#pragma unroll
  for (int i = 0; i < kMaxTaps; ++i)
    if (i < p.taps - 1) keep[i] = conv_input(p, last, r0, p0, p0 + len - (p.taps - 1) + i, c, C);
#pragma unroll
  for (int i = 0; i < kMaxTaps; ++i)
    if (i < p.taps - 1) last[static_cast<int64_t>(i) * C + c] = keep[i];
}

struct ScanParams {
  const float* x;            // [n][cols]: q (G D) | k (G D) | v (H V) | g (H D) | beta (H)
  int cols;
  const int32_t* meta;
  int meta_stride;
  float* record;             // [slots][record_size], S first
  int64_t record_size;
  float* out;                // [n][H V]
  int H, G, D, V;
  int P;                     // threads a column
  int vec;                   // 1: D and V are multiples of four and the rows 16-byte aligned: staged by 16-byte copies
};

constexpr int kTokens = 8;   // tokens staged at a time
constexpr int kPad = 4;      // floats between two threads' slices of a staged row: slices a quarter of a warp reads side by side lie in other banks

__device__ __forceinline__ void copy_async4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(dst))), "l"(src) : "memory");
}
__device__ __forceinline__ void copy_async16(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(dst))), "l"(src) : "memory");
}

// A CTA of 128 threads (64 when the step has few CTAs: more SMs then share the work, and the arithmetic of a column is the same):
// (entry, head, threads / P value columns). DP: key channels a thread holds (a multiple of four). Eight tokens' q, k, g
// (a thread's slice contiguous, slices kPad apart), v and beta wait in shared memory, the next eight on their way (cp.async) meanwhile.
// A thread's share of a sum over the channels: four sums side by side, each over every fourth channel in ascending order, joined as
// (s0 + s1) + (s2 + s3); then the P threads of a column by xor shuffles.
template <int DP>
__global__ void __launch_bounds__(128) delta_scan_kernel(ScanParams p) {
  extern __shared__ __align__(16) float staged[];
  sb::grid_launch_dependents();
  const int e = blockIdx.x, h = blockIdx.y, P = p.P, CW = blockDim.x / P, LD = DP + kPad, row = P * LD;
  const int part = threadIdx.x % P, cl = threadIdx.x / P, col = blockIdx.z * CW + cl;
  const int gq = h / (p.H / p.G);
  const int stage = kTokens * (3 * row + CW + 1) + 3;          // floats of one buffer (rounded up below)
  const int stage4 = (stage + 3) & ~3;
  const int slot = p.meta[e], r0 = p.meta[p.meta_stride + e], len = p.meta[2 * p.meta_stride + e], p0 = p.meta[3 * p.meta_stride + e];
  const bool live = col < p.V;
  float* st = p.record + static_cast<int64_t>(slot) * p.record_size + (static_cast<int64_t>(h) * p.D + part * DP) * p.V + col;
  const int dn = min(DP, p.D - part * DP);
  const int nq = p.G * p.D, off_v = 2 * nq, off_g = off_v + p.H * p.V, off_b = off_g + p.H * p.D;
  // what no copy ever writes: channels beyond D (q = k = 0, g = 1), columns beyond V (v = 0)
  for (int i = threadIdx.x; i < 2 * stage4; i += blockDim.x) staged[i] = 0.0f;
  __syncthreads();
  for (int b = 0; b < 2; ++b)
    for (int i = threadIdx.x; i < kTokens * row; i += blockDim.x) {
      const int j = i % row, d = (j / LD) * DP + j % LD;
      if (j % LD >= DP || d >= p.D) staged[b * stage4 + 2 * kTokens * row + i] = 1.0f;
    }
  auto request = [&](int t0, int b) {
    const int nt = min(kTokens, len - t0);
    float* sq = staged + b * stage4;
    float* sk = sq + kTokens * row;
    float* sg = sk + kTokens * row;
    float* sv = sg + kTokens * row;
    float* sbeta = sv + kTokens * CW;
    if (p.vec) {
      const int d4 = p.D / 4;
      for (int i = threadIdx.x; i < nt * d4; i += blockDim.x) {
        const int tt = i / d4, d = (i % d4) * 4, at = tt * row + (d / DP) * LD + d % DP;
        const float* src = p.x + static_cast<int64_t>(r0 + t0 + tt) * p.cols;
        copy_async16(sq + at, src + gq * p.D + d);
        copy_async16(sk + at, src + nq + gq * p.D + d);
        copy_async16(sg + at, src + off_g + h * p.D + d);
      }
      const int c4 = CW / 4;
      for (int i = threadIdx.x; i < nt * c4; i += blockDim.x) {
        const int tt = i / c4, c = blockIdx.z * CW + (i % c4) * 4;
        if (c < p.V) copy_async16(sv + tt * CW + (i % c4) * 4, p.x + static_cast<int64_t>(r0 + t0 + tt) * p.cols + off_v + h * p.V + c);
      }
    } else {
      for (int i = threadIdx.x; i < nt * p.D; i += blockDim.x) {
        const int tt = i / p.D, d = i % p.D, at = tt * row + (d / DP) * LD + d % DP;
        const float* src = p.x + static_cast<int64_t>(r0 + t0 + tt) * p.cols;
        copy_async4(sq + at, src + gq * p.D + d);
        copy_async4(sk + at, src + nq + gq * p.D + d);
        copy_async4(sg + at, src + off_g + h * p.D + d);
      }
      for (int i = threadIdx.x; i < nt * CW; i += blockDim.x) {
        const int tt = i / CW, c = blockIdx.z * CW + i % CW;
        if (c < p.V) copy_async4(sv + i, p.x + static_cast<int64_t>(r0 + t0 + tt) * p.cols + off_v + h * p.V + c);
      }
    }
    if (threadIdx.x < nt) copy_async4(sbeta + threadIdx.x, p.x + static_cast<int64_t>(r0 + t0 + threadIdx.x) * p.cols + off_b + h);
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  sb::grid_dependency_wait();
  float S[DP];
#pragma unroll
  for (int i = 0; i < DP; ++i) S[i] = (p0 > 0 && live && i < dn) ? st[static_cast<int64_t>(i) * p.V] : 0.0f;
  __syncthreads();
  request(0, 0);
  int b = 0;
  for (int t0 = 0; t0 < len; t0 += kTokens, b ^= 1) {
    const int nt = min(kTokens, len - t0);
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();                                     // the chunk has landed for everyone, and everyone has left the other buffer
    if (t0 + kTokens < len) request(t0 + kTokens, b ^ 1);
    const float* sq = staged + b * stage4;
    const float* sk = sq + kTokens * row;
    const float* sg = sk + kTokens * row;
    const float* sv = sg + kTokens * row;
    const float* sbeta = sv + kTokens * CW;
#pragma unroll 2
    for (int tt = 0; tt < nt; ++tt) {
      const float4* q = reinterpret_cast<const float4*>(sq + tt * row + part * LD);
      const float4* k = reinterpret_cast<const float4*>(sk + tt * row + part * LD);
      const float4* g = reinterpret_cast<const float4*>(sg + tt * row + part * LD);
      float d0 = 0.0f, d1 = 0.0f, d2 = 0.0f, d3 = 0.0f;
      float4 kk[DP / 4];
#pragma unroll
      for (int i = 0; i < DP / 4; ++i) {
        const float4 gg = g[i];
        kk[i] = k[i];
        S[4 * i] = __fmul_rn(S[4 * i], gg.x), S[4 * i + 1] = __fmul_rn(S[4 * i + 1], gg.y);
        S[4 * i + 2] = __fmul_rn(S[4 * i + 2], gg.z), S[4 * i + 3] = __fmul_rn(S[4 * i + 3], gg.w);
        d0 = fmaf(S[4 * i], kk[i].x, d0), d1 = fmaf(S[4 * i + 1], kk[i].y, d1);
        d2 = fmaf(S[4 * i + 2], kk[i].z, d2), d3 = fmaf(S[4 * i + 3], kk[i].w, d3);
      }
      float dot = __fadd_rn(__fadd_rn(d0, d1), __fadd_rn(d2, d3));
      for (int o = 1; o < P; o <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
      const float u = __fmul_rn(sbeta[tt], __fsub_rn(sv[tt * CW + cl], dot));
      float o0 = 0.0f, o1 = 0.0f, o2 = 0.0f, o3 = 0.0f;
#pragma unroll
      for (int i = 0; i < DP / 4; ++i) {
        const float4 qq = q[i];
        S[4 * i] = fmaf(kk[i].x, u, S[4 * i]), S[4 * i + 1] = fmaf(kk[i].y, u, S[4 * i + 1]);
        S[4 * i + 2] = fmaf(kk[i].z, u, S[4 * i + 2]), S[4 * i + 3] = fmaf(kk[i].w, u, S[4 * i + 3]);
        o0 = fmaf(S[4 * i], qq.x, o0), o1 = fmaf(S[4 * i + 1], qq.y, o1);
        o2 = fmaf(S[4 * i + 2], qq.z, o2), o3 = fmaf(S[4 * i + 3], qq.w, o3);
      }
      float o_sum = __fadd_rn(__fadd_rn(o0, o1), __fadd_rn(o2, o3));
      for (int o = 1; o < P; o <<= 1) o_sum += __shfl_xor_sync(0xffffffffu, o_sum, o);
      if (part == 0 && live) p.out[static_cast<int64_t>(r0 + t0 + tt) * p.H * p.V + h * p.V + col] = o_sum;
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < DP; ++i)
      if (i < dn) st[static_cast<int64_t>(i) * p.V] = S[i];
  }
}

}  // namespace

// i: 0 first projection's partial sums (flat), 1 their width, 2 K ranges S, 3 second projection's partial sums (flat), 4 their width, 5 K ranges S,
//    6 most tokens with a buffer per range, 7 conv weights (float32 [C][taps]), 8 A_log (float32 [H]), 9 dt_bias (float32 [H D]), 10 records,
//    11 record size, 12 offset of the last inputs in a record, 13 out (float32 [n][2 G D + H V + H D + H]: q | k | v | g | beta), 14 H, 15 G, 16 D,
//    17 V, 18 taps
SB_EXPORT int sb_op_delta_prepare(const SbOp* op, const SbStep* s, void* stream) {
  using namespace sbstep;
  if (s->n <= 0) return SB_OP_SKIPPED;
  const int w1 = (int)op->i[1], w2 = (int)op->i[4], H = (int)op->i[14], G = (int)op->i[15], D = (int)op->i[16], V = (int)op->i[17], taps = (int)op->i[18];
  if (H <= 0 || G <= 0 || H % G != 0 || D <= 0 || V <= 0) return sb::fail("sb_op_delta_prepare: heads %d / %d, sizes %d / %d", H, G, D, V), SB_OP_FAILED;
  if (taps < 1 || taps > kMaxTaps) return sb::fail("sb_op_delta_prepare: %d taps (1 to %d)", taps, kMaxTaps), SB_OP_FAILED;
  const int C = 2 * G * D + H * V;
  if (C + H > w1 || H * D > w2) return sb::fail("sb_op_delta_prepare: rows of %d and %d elements are too short", w1, w2), SB_OP_FAILED;
  PrepareParams p{ptr<const float>(op->i[0]), partial_count(op->i[2], op->i[6], s->n), static_cast<int64_t>(s->n) * w1, w1,
                  ptr<const float>(op->i[3]), partial_count(op->i[5], op->i[6], s->n), static_cast<int64_t>(s->n) * w2, w2,
                  ptr<const float>(op->i[7]), ptr<const float>(op->i[8]), ptr<const float>(op->i[9]), entry_meta(s), s->max_rows, s->entries,
                  positions(s), ptr<float>(op->i[10]), op->i[11], op->i[12], ptr<float>(op->i[13]), H, G, D, V, taps};
  if (D > kSlab) return sb::fail("sb_op_delta_prepare: key size %d (at most %d)", D, kSlab), SB_OP_FAILED;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int threads = D <= 128 ? 128 : 256;
  const int units = 2 * G + (H * V + threads - 1) / threads + (H * D + H + threads - 1) / threads;
  int shares = (16 * sb::sm_count() + s->n - 1) / s->n;         // blocks enough to fill the device when the tokens are few,
  shares = shares < 4 ? 4 : shares;                             // and short enough to hide one another's waits when they are many
  shares = shares > units ? units : shares;
  sb::launch_pdl(delta_prepare_kernel, dim3(s->n, shares), dim3(threads), 0, st, p);
  if (taps > 1) sb::launch_pdl(delta_conv_state_kernel, dim3(s->entries, (C + 255) / 256), dim3(256), 0, st, p);
  return sb::check_launch("sb_op_delta_prepare");
}

// i: 0 x (float32 [n][2 G D + H V + H D + H], what sb_op_delta_prepare left), 1 records, 2 record size, 3 out (float32 [n][H V]), 4 H, 5 G, 6 D, 7 V
SB_EXPORT int sb_op_delta_scan(const SbOp* op, const SbStep* s, void* stream) {
  using namespace sbstep;
  if (s->n <= 0 || s->entries <= 0) return SB_OP_SKIPPED;
  const int H = (int)op->i[4], G = (int)op->i[5], D = (int)op->i[6], V = (int)op->i[7];
  if (H <= 0 || G <= 0 || H % G != 0 || D <= 0 || D > 256 || V <= 0) return sb::fail("sb_op_delta_scan: heads %d / %d, key size %d (at most 256), value size %d", H, G, D, V), SB_OP_FAILED;
  int P = 1;
  while (D > 32 * P) P *= 2;                          // threads a column: a function of the key size alone
  const int per = (D + P - 1) / P, DP = per <= 8 ? 8 : per <= 16 ? 16 : 32;
  const int cols = 2 * G * D + H * V + H * D + H;
  int threads = 128;
  if (static_cast<int64_t>(s->entries) * H * ((V + threads / P - 1) / (threads / P)) < 2 * sb::sm_count()) threads = 64;
  const int CW = threads / P;
  const int vec = D % 4 == 0 && V % 4 == 0 && cols % 4 == 0 && (reinterpret_cast<uintptr_t>(ptr<const float>(op->i[0])) & 15) == 0 && CW % 4 == 0;
  ScanParams p{ptr<const float>(op->i[0]), cols, entry_meta(s), s->max_rows, ptr<float>(op->i[1]), op->i[2], ptr<float>(op->i[3]), H, G, D, V, P, vec};
  const dim3 grid(s->entries, H, (V + CW - 1) / CW);
  const size_t smem = sizeof(float) * 2 * ((kTokens * (3 * P * (DP + kPad) + CW + 1) + 3 + 3) & ~3);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (DP == 8) sb::launch_pdl(delta_scan_kernel<8>, grid, dim3(threads), smem, st, p);
  else if (DP == 16) sb::launch_pdl(delta_scan_kernel<16>, grid, dim3(threads), smem, st, p);
  else sb::launch_pdl(delta_scan_kernel<32>, grid, dim3(threads), smem, st, p);
  return sb::check_launch("sb_op_delta_scan");
}
