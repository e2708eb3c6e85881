// What stands between the two projections of feed-forwards that are not a plain gated product.
//
// PolyNorm: act(z) = a N(z) + b N(z^2) + c N(z^3) + e over a token's row z of the up projection, powers taken element by
// element, N(y) = y / sqrt(mean(y^2) + eps). One block per row; the three mean squares are block sums in a fixed order.
//
// Routed experts. `moe_route_kernel`: a warp per token turns the router's logits into a row of expert weights: scores =
// softmax over all experts; the `top` experts with the largest score + correction are chosen (the smaller index among
// equals); a chosen expert's weight is its score / (sum of the chosen scores + 1e-20) * scale, every other weight is 0.
// `moe_activate_kernel`: hidden[r, e ff + j] = weight[r, e] * relu(up[r, e ff + j])^2 for the experts' up projections laid
// side by side, so that ONE product with the down matrices laid side by side is the weighted sum of the chosen experts
// (an expert that was not chosen contributes exact zeros). All arithmetic is 32-bit.
#include <cmath>
#include <cstring>

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

template <class TO>
__global__ void __launch_bounds__(1024) polynorm_kernel(const float* __restrict__ up, int n_partials, int64_t partial_stride, TO* __restrict__ out,
                                                         int F, float a, float b, float c, float e, float eps) {
  extern __shared__ __align__(16) float row[];
  __shared__ float red[32];
  sb::grid_launch_dependents();
  sb::grid_dependency_wait();
  const int64_t r = blockIdx.x;
  float s2 = 0.0f, s4 = 0.0f, s6 = 0.0f;
  for (int i = threadIdx.x; i < F; i += blockDim.x) {
    const float z = folded(up + r * F + i, n_partials, partial_stride);
    row[i] = z;
    const float z2 = z * z, z3 = z2 * z;
    s2 += z2;
    s4 = fmaf(z2, z2, s4);
    s6 = fmaf(z3, z3, s6);
  }
  const float inv = 1.0f / static_cast<float>(F);
  const float n1 = 1.0f / sqrtf(sb::block_sum(s2, red) * inv + eps);
  const float n2 = 1.0f / sqrtf(sb::block_sum(s4, red) * inv + eps);
  const float n3 = 1.0f / sqrtf(sb::block_sum(s6, red) * inv + eps);
  for (int i = threadIdx.x; i < F; i += blockDim.x) {
    const float z = row[i], z2 = z * z;
    out[r * F + i] = sb::narrow<TO>(a * (z * n1) + b * (z2 * n2) + c * (z2 * z * n3) + e);
  }
}

// One warp per token. logits [n][ldz] float32, correction [X] (float32 or bfloat16), weights out [n][X].
// BIASED: the correction is a bias of the router (z + correction are the logits), the experts with the largest logits are chosen and
// weigh by the softmax over the chosen logits alone: exp(z - max) / (sum of the chosen exp(z - max)), the largest logit being one of them.
template <class TC, bool BIASED>
__global__ void moe_route_kernel(const float* __restrict__ logits, int ldz, const TC* __restrict__ correction, float* __restrict__ weights, int n,
                                 int X, int top, float scale) {
  sb::grid_launch_dependents();
  sb::grid_dependency_wait();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= n) return;
  constexpr int kPer = 8;          // experts a lane: up to 256 in all
  const float* z = logits + static_cast<int64_t>(warp) * ldz;
  float v[kPer], m = -INFINITY;
#pragma unroll
  for (int i = 0; i < kPer; ++i) {
    const int x = lane + 32 * i;
    v[i] = x < X ? (BIASED ? __fadd_rn(z[x], sb::widen(correction[x])) : z[x]) : -INFINITY;
    m = fmaxf(m, v[i]);
  }
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  float sum = 0.0f, logit[kPer];
#pragma unroll
  for (int i = 0; i < kPer; ++i) {
    logit[i] = v[i];
    v[i] = lane + 32 * i < X ? expf(v[i] - m) : 0.0f;
    sum += v[i];
  }
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  float score[kPer], choice[kPer], out[kPer];
#pragma unroll
  for (int i = 0; i < kPer; ++i) {
    const int x = lane + 32 * i;
    score[i] = BIASED ? v[i] : v[i] / sum;
    choice[i] = x < X ? (BIASED ? logit[i] : score[i] + sb::widen(correction[x])) : -INFINITY;
    out[i] = 0.0f;
  }
  float picked_sum = 0.0f;
  for (int k = 0; k < top; ++k) {
    // the largest choice score left, the smaller index among equals
    float best = -INFINITY;
    int at = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < kPer; ++i)
      if (choice[i] > best) {
        best = choice[i];
        at = lane + 32 * i;
      }
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (ob > best || (ob == best && oa < at)) {
        best = ob;
        at = oa;
      }
    }
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < kPer; ++i)
      if (lane + 32 * i == at) {
        s = score[i];
        out[i] = 1.0f;
        choice[i] = -INFINITY;
      }
    s = __shfl_sync(0xffffffffu, s, at & 31);
    picked_sum += s;
  }
  const float norm = BIASED ? picked_sum : picked_sum + 1e-20f;
#pragma unroll
  for (int i = 0; i < kPer; ++i) {
    const int x = lane + 32 * i;
    if (x < X) weights[static_cast<int64_t>(warp) * X + x] = out[i] != 0.0f ? score[i] / norm * scale : 0.0f;
  }
}

// A block per row and expert; an expert that the row did not choose (weight 0) is zeroed without reading. GATED: an expert has 2 F rows
// of `up`, F gate rows and then F up rows, and its hidden activation is silu(gate) * up instead of relu(up)^2.
template <class TO, bool GATED>
__global__ void __launch_bounds__(256) moe_activate_kernel(const float* __restrict__ up, int n_partials, int64_t partial_stride,
                                                           const float* __restrict__ weights, int ldw, TO* __restrict__ out, int E, int F) {
  sb::grid_launch_dependents();
  sb::grid_dependency_wait();
  const int64_t r = blockIdx.x;
  const int e = blockIdx.y;                      // a CTA per (row, expert): a step of few rows still fills the SMs
  const int EF = E * F;
  const float* src = up + r * EF * (GATED ? 2 : 1);
  TO* dst = out + r * EF;
  const float w = weights[r * ldw + e];
  if (w == 0.0f) {
    for (int j = threadIdx.x; j < F; j += blockDim.x) dst[e * F + j] = sb::narrow<TO>(0.0f);
    return;
  }
  for (int j = threadIdx.x; j < F; j += blockDim.x) {
    if (GATED) {
      const float g = folded(src + 2 * e * F + j, n_partials, partial_stride), u = folded(src + (2 * e + 1) * F + j, n_partials, partial_stride);
      dst[e * F + j] = sb::narrow<TO>(w * ((g / (1.0f + expf(-g))) * u));
    } else {
      const float z = fmaxf(folded(src + e * F + j, n_partials, partial_stride), 0.0f);
      dst[e * F + j] = sb::narrow<TO>(w * (z * z));
    }
  }
}

}  // namespace

// out [n][F] (float32 or bfloat16) = PolyNorm of up [P][n][F] float32 partial sums.
SB_EXPORT int sb_polynorm(const float* up, int n_partials, int64_t partial_stride, void* out, int out_dtype, int n, int F, float a, float b,
                          float c, float e, float eps, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (n_partials < 1 || F <= 0) return sb::fail("sb_polynorm: n_partials %d, size %d", n_partials, F);
  const size_t smem = static_cast<size_t>(F) * sizeof(float);
  if (smem > 200 * 1024) return sb::fail("sb_polynorm: a row of %d elements does not fit the row buffer", F);
  const int threads = F >= 4096 ? 1024 : F >= 2048 ? 512 : F >= 512 ? 256 : 128;
  if (out_dtype == 0) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(polynorm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    sb::launch_pdl(polynorm_kernel<float>, dim3(n), dim3(threads), smem, stream, up, n_partials, partial_stride, static_cast<float*>(out), F, a, b, c, e, eps);
  } else if (out_dtype == 1) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(polynorm_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    sb::launch_pdl(polynorm_kernel<bf16>, dim3(n), dim3(threads), smem, stream, up, n_partials, partial_stride, static_cast<bf16*>(out), F, a, b, c, e, eps);
  } else {
    return sb::fail("sb_polynorm: unsupported output dtype %d", out_dtype);
  }
  return sb::check_launch("sb_polynorm");
}

// biased 0: softmax over all experts, chosen by score + correction, weights = the chosen scores normalised; 1: see moe_route_kernel.
SB_EXPORT int sb_moe_route(const float* logits, int ldz, const void* correction, int correction_dtype, float* weights, int n, int X, int top,
                           float scale, int biased, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (X <= 0 || X > 256 || top <= 0 || top > X) return sb::fail("sb_moe_route: %d experts (at most 256), %d chosen", X, top);
  const int blocks = (n + 3) / 4;
#define SB_ROUTE(TC, B) sb::launch_pdl(moe_route_kernel<TC, B>, dim3(blocks), dim3(128), 0, stream, logits, ldz, static_cast<const TC*>(correction), weights, n, X, top, scale)
  if (correction_dtype == 0) {
    if (biased) SB_ROUTE(float, true);
    else SB_ROUTE(float, false);
  } else if (correction_dtype == 1) {
    if (biased) SB_ROUTE(bf16, true);
    else SB_ROUTE(bf16, false);
  } else
#undef SB_ROUTE
    return sb::fail("sb_moe_route: unsupported correction dtype %d", correction_dtype);
  return sb::check_launch("sb_moe_route");
}

// out [n][E F] = weights[r, e] * relu(up)^2, up [P][n][E F] float32 partial sums, weights [n][ldw] (the first E columns);
// gated: weights[r, e] * silu(gate) * up, up [P][n][E 2 F] with an expert's gate rows in front of its up rows.
SB_EXPORT int sb_moe_activate(const float* up, int n_partials, int64_t partial_stride, const float* weights, int ldw, void* out, int out_dtype,
                              int n, int E, int F, int gated, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (n_partials < 1 || E <= 0 || F <= 0) return sb::fail("sb_moe_activate: n_partials %d, %d experts of %d", n_partials, E, F);
  if (E > 256) return sb::fail("sb_moe_activate: %d experts (at most 256)", E);
#define SB_ACT(TO, G) sb::launch_pdl(moe_activate_kernel<TO, G>, dim3(n, E), dim3(F >= 1024 ? 256 : 128), 0, stream, up, n_partials, partial_stride, weights, ldw, static_cast<TO*>(out), E, F)
  if (out_dtype == 0) {
    if (gated) SB_ACT(float, true);
    else SB_ACT(float, false);
  } else if (out_dtype == 1) {
    if (gated) SB_ACT(bf16, true);
    else SB_ACT(bf16, false);
  } else
#undef SB_ACT
    return sb::fail("sb_moe_activate: unsupported output dtype %d", out_dtype);
  return sb::check_launch("sb_moe_activate");
}

// ------------------------------------------------------------------ operations of the native step program (step_ops.h)
// i: 0 up partial sums (flat), 1 K ranges S, 2 most tokens with a buffer per range, 3 out, 4 out dtype, 5 F      f: 0 a, 1 b, 2 c, 3 e
// (eps travels as the bits of a float in i[6])
SB_EXPORT int sb_op_polynorm(const SbOp* op, const SbStep* s, void* stream) {
  using namespace sbstep;
  if (s->n <= 0) return SB_OP_SKIPPED;
  const int F = (int)op->i[5];
  const uint32_t bits = static_cast<uint32_t>(op->i[6]);
  float eps;
  memcpy(&eps, &bits, sizeof(eps));
  return sb_polynorm(ptr<const float>(op->i[0]), partial_count(op->i[1], op->i[2], s->n), static_cast<int64_t>(s->n) * F, ptr<void>(op->i[3]),
                     (int)op->i[4], s->n, F, (float)op->f[0], (float)op->f[1], (float)op->f[2], (float)op->f[3], eps, static_cast<cudaStream_t>(stream));
}

// i: 0 logits, 1 ldz, 2 correction, 3 its dtype, 4 weights, 5 X, 6 top, 7 biased      f: 0 scale
SB_EXPORT int sb_op_moe_route(const SbOp* op, const SbStep* s, void* stream) {
  using namespace sbstep;
  if (s->n <= 0) return SB_OP_SKIPPED;
  return sb_moe_route(ptr<const float>(op->i[0]), (int)op->i[1], ptr<const void>(op->i[2]), (int)op->i[3], ptr<float>(op->i[4]), s->n, (int)op->i[5],
                      (int)op->i[6], (float)op->f[0], (int)op->i[7], static_cast<cudaStream_t>(stream));
}

// i: 0 up partial sums (flat), 1 K ranges S, 2 most tokens with a buffer per range, 3 weights, 4 ldw, 5 out, 6 out dtype, 7 E, 8 F, 9 gated
SB_EXPORT int sb_op_moe_activate(const SbOp* op, const SbStep* s, void* stream) {
  using namespace sbstep;
  if (s->n <= 0) return SB_OP_SKIPPED;
  const int E = (int)op->i[7], F = (int)op->i[8], gated = (int)op->i[9];
  return sb_moe_activate(ptr<const float>(op->i[0]), partial_count(op->i[1], op->i[2], s->n), static_cast<int64_t>(s->n) * E * F * (gated ? 2 : 1),
                         ptr<const float>(op->i[3]), (int)op->i[4], ptr<void>(op->i[5]), (int)op->i[6], s->n, E, F, gated,
                         static_cast<cudaStream_t>(stream));
}
