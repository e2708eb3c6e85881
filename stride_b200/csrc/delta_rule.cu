// The gated delta rule: linear attention whose state forgets per key channel and is corrected, not only added to.
//
// Per token t of a request and head h (key size D, value size V, state S [D][V], float32, zero at position 0):
//
//   S <- diag(g_t) S          g_t [D] in (0, 1): one decay per key channel
//   u  = beta_t (v_t - S^T k_t)
//   S <- S + k_t u^T
//   o_t = S^T q_t             (the read-out sees the token's own write)
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
  float* out;                // [n][2 G D + H V + H + H D]: q | k | v | beta | g
  int H, G, D, V, taps;
};

// The conv's input of channel c at position t of the entry (first row r0, first position p0): a row of the step, the record, or zero.
__device__ __forceinline__ float conv_input(const PrepareParams& p, const float* last, int r0, int p0, int t, int c, int C) {
  if (t >= p0) return folded(p.proj + static_cast<int64_t>(r0 + t - p0) * p.width1 + c, p.n1, p.stride1);
  if (t >= 0) return last[static_cast<int64_t>(p.taps - 1 - (p0 - t)) * C + c];
  return 0.0f;
}

__global__ void __launch_bounds__(256) delta_prepare_kernel(PrepareParams p) {
  extern __shared__ float row_values[];       // [C]
  __shared__ int found[3];
  sb::grid_launch_dependents();
  const int row = blockIdx.x, C = 2 * p.G * p.D + p.H * p.V;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  if (threadIdx.x == 0) {
    int e = 0;
    for (; e < p.entries; ++e) {
      const int r0 = p.meta[p.meta_stride + e], len = p.meta[2 * p.meta_stride + e];
      if (row >= r0 && row < r0 + len) break;
    }
    found[0] = e < p.entries ? p.meta[e] : 0;
    found[1] = e < p.entries ? p.meta[p.meta_stride + e] : row;
    found[2] = e < p.entries ? p.meta[3 * p.meta_stride + e] : p.positions[row];
  }
  __syncthreads();
  const int slot = found[0], r0 = found[1], p0 = found[2], pos = p0 + (row - r0);
  const float* last = p.record + static_cast<int64_t>(slot) * p.record_size + p.conv_offset;
  sb::grid_dependency_wait();
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float acc = 0.0f;
    for (int j = 0; j < p.taps; ++j) acc = fmaf(p.conv[c * p.taps + j], conv_input(p, last, r0, p0, pos - (p.taps - 1 - j), c, C), acc);
    row_values[c] = silu(acc);
  }
  __syncthreads();
  const int nqk = 2 * p.G * p.D, cols = C + p.H + p.H * p.D;
  float* out = p.out + static_cast<int64_t>(row) * cols;
  for (int hh = warp; hh < 2 * p.G; hh += warps) {       // q heads, then k heads: unit vectors
    const float* head = row_values + hh * p.D;
    float ss = 0.0f;
    for (int d = lane; d < p.D; d += 32) ss = fmaf(head[d], head[d], ss);
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    float r = 1.0f / sqrtf(ss + 1e-6f);
    if (hh < p.G) r = __fmul_rn(r, 1.0f / sqrtf(static_cast<float>(p.D)));
    for (int d = lane; d < p.D; d += 32) out[hh * p.D + d] = __fmul_rn(head[d], r);
  }
  for (int i = nqk + threadIdx.x; i < cols; i += blockDim.x) {
    float v;
    if (i < C) {
      v = row_values[i];
    } else if (i < C + p.H) {
      v = 1.0f / (1.0f + expf(-folded(p.proj + static_cast<int64_t>(row) * p.width1 + i, p.n1, p.stride1)));
    } else {
      const int e = i - C - p.H;
      const float a = __fadd_rn(folded(p.proj2 + static_cast<int64_t>(row) * p.width2 + e, p.n2, p.stride2), p.dt_bias[e]);
      v = expf(-expf(p.a_log[e / p.D]) * softplus(a));
    }
    out[i] = v;
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
  const float* x;            // [n][cols]: q (G D) | k (G D) | v (H V) | beta (H) | g (H D)
  int cols;
  const int32_t* meta;
  int meta_stride;
  float* record;             // [slots][record_size], S first
  int64_t record_size;
  float* out;                // [n][H V]
  int H, G, D, V;
  int P;                     // threads a column
};

constexpr int kTokens = 8;   // tokens staged at a time

// A CTA of 128 threads: (entry, head, 128 / P value columns). DP: key channels a thread holds.
template <int DP>
__global__ void __launch_bounds__(128) delta_scan_kernel(ScanParams p) {
  extern __shared__ float staged[];
  sb::grid_launch_dependents();
  const int e = blockIdx.x, h = blockIdx.y, P = p.P, CW = 128 / P, Dp = P * DP;
  const int part = threadIdx.x % P, col = blockIdx.z * CW + threadIdx.x / P;
  const int gq = h / (p.H / p.G);
  float* sq = staged;                       // [kTokens][Dp]
  float* sk = sq + kTokens * Dp;
  float* sg = sk + kTokens * Dp;
  float* sv = sg + kTokens * Dp;            // [kTokens][CW]
  float* sb_ = sv + kTokens * CW;           // [kTokens]
  const int slot = p.meta[e], r0 = p.meta[p.meta_stride + e], len = p.meta[2 * p.meta_stride + e], p0 = p.meta[3 * p.meta_stride + e];
  const bool live = col < p.V;
  float* st = p.record + static_cast<int64_t>(slot) * p.record_size + (static_cast<int64_t>(h) * p.D + part * DP) * p.V + col;
  const int dn = min(DP, p.D - part * DP);
  const int nq = p.G * p.D, off_v = 2 * nq, off_b = off_v + p.H * p.V, off_g = off_b + p.H;
  sb::grid_dependency_wait();
  float S[DP];
#pragma unroll
  for (int i = 0; i < DP; ++i) S[i] = (p0 > 0 && live && i < dn) ? st[static_cast<int64_t>(i) * p.V] : 0.0f;
  for (int t0 = 0; t0 < len; t0 += kTokens) {
    const int nt = min(kTokens, len - t0);
    __syncthreads();
    for (int i = threadIdx.x; i < nt * Dp; i += blockDim.x) {
      const int tt = i / Dp, d = i % Dp;
      const float* src = p.x + static_cast<int64_t>(r0 + t0 + tt) * p.cols;
      const bool in = d < p.D;
      sq[i] = in ? src[gq * p.D + d] : 0.0f;
      sk[i] = in ? src[nq + gq * p.D + d] : 0.0f;
      sg[i] = in ? src[off_g + h * p.D + d] : 1.0f;
    }
    for (int i = threadIdx.x; i < nt * CW; i += blockDim.x) {
      const int tt = i / CW, c = blockIdx.z * CW + i % CW;
      sv[i] = c < p.V ? p.x[static_cast<int64_t>(r0 + t0 + tt) * p.cols + off_v + h * p.V + c] : 0.0f;
    }
    if (threadIdx.x < nt) sb_[threadIdx.x] = p.x[static_cast<int64_t>(r0 + t0 + threadIdx.x) * p.cols + off_b + h];
    __syncthreads();
    for (int tt = 0; tt < nt; ++tt) {
      const float* q = sq + tt * Dp + part * DP;
      const float* k = sk + tt * Dp + part * DP;
      const float* g = sg + tt * Dp + part * DP;
      float dot = 0.0f;
#pragma unroll
      for (int i = 0; i < DP; ++i) {
        S[i] = __fmul_rn(S[i], g[i]);
        dot = fmaf(S[i], k[i], dot);
      }
      for (int o = 1; o < P; o <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
      const float u = __fmul_rn(sb_[tt], __fsub_rn(sv[tt * CW + threadIdx.x / P], dot));
      float o_sum = 0.0f;
#pragma unroll
      for (int i = 0; i < DP; ++i) {
        S[i] = fmaf(k[i], u, S[i]);
        o_sum = fmaf(S[i], q[i], o_sum);
      }
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
//    11 record size, 12 offset of the last inputs in a record, 13 out (float32 [n][2 G D + H V + H + H D]), 14 H, 15 G, 16 D, 17 V, 18 taps
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
  const size_t smem = static_cast<size_t>(C) * sizeof(float);
  if (smem > 160 * 1024) return sb::fail("sb_op_delta_prepare: %d channels do not fit the row buffer", C), SB_OP_FAILED;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (smem > 48 * 1024) cudaFuncSetAttribute(delta_prepare_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  sb::launch_pdl(delta_prepare_kernel, dim3(s->n), dim3(256), smem, st, p);
  if (taps > 1) sb::launch_pdl(delta_conv_state_kernel, dim3(s->entries, (C + 255) / 256), dim3(256), 0, st, p);
  return sb::check_launch("sb_op_delta_prepare");
}

// i: 0 x (float32 [n][2 G D + H V + H + H D], what sb_op_delta_prepare left), 1 records, 2 record size, 3 out (float32 [n][H V]), 4 H, 5 G, 6 D, 7 V
SB_EXPORT int sb_op_delta_scan(const SbOp* op, const SbStep* s, void* stream) {
  using namespace sbstep;
  if (s->n <= 0 || s->entries <= 0) return SB_OP_SKIPPED;
  const int H = (int)op->i[4], G = (int)op->i[5], D = (int)op->i[6], V = (int)op->i[7];
  if (H <= 0 || G <= 0 || H % G != 0 || D <= 0 || D > 256 || V <= 0) return sb::fail("sb_op_delta_scan: heads %d / %d, key size %d (at most 256), value size %d", H, G, D, V), SB_OP_FAILED;
  int P = 1;
  while (D > 32 * P) P *= 2;                          // threads a column: a function of the key size alone
  const int per = (D + P - 1) / P, DP = per <= 8 ? 8 : per <= 16 ? 16 : 32;
  ScanParams p{ptr<const float>(op->i[0]), 2 * G * D + H * V + H + H * D, entry_meta(s), s->max_rows, ptr<float>(op->i[1]), op->i[2],
               ptr<float>(op->i[3]), H, G, D, V, P};
  const int CW = 128 / P;
  const dim3 grid(s->entries, H, (V + CW - 1) / CW);
  const size_t smem = sizeof(float) * kTokens * (3 * P * DP + CW + 1);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (DP == 8) sb::launch_pdl(delta_scan_kernel<8>, grid, dim3(128), smem, st, p);
  else if (DP == 16) sb::launch_pdl(delta_scan_kernel<16>, grid, dim3(128), smem, st, p);
  else sb::launch_pdl(delta_scan_kernel<32>, grid, dim3(128), smem, st, p);
  return sb::check_launch("sb_op_delta_scan");
}
