// Branches beside the residual stream. A sublayer whose result is scaled before it joins the residual (a per-channel
// layer scale, a constant per branch, or both) writes into a branch buffer of the stream's shape instead: its last
// projection either adds into the buffer or leaves one partial sum per K range. The fold
//
//   dst[r, j] += gain[j] * (ca * (a[r, j] + (pa_0 + pa_1 + ..)[r, j]) + cb * (b[r, j] + (pb_0 + pb_1 + ..)[r, j]))
//
// takes up to two branches into `dst` (the residual, or another branch) in 32-bit and leaves the branch buffers zero,
// which is the state the next sublayer expects to find them in. The order of the additions is fixed.
//
// The fold with a norm on the way (a sublayer whose result is RMS-normed before it joins the residual):
//
//   y[r, :] = ca * (a + ..)[r, :] + cb * (b + ..)[r, :];   dst[r, j] += gain[j] * y[r, j] / sqrt(mean_j(y[r, j]^2) + eps)
//
// A second kernel adds a row-scaled copy of the sublayer's input: dst[r, :] += (sum of `count` columns of w[r, :]) * x[r, :],
// what experts that pass their input through contribute to a routed feed-forward. A third adds another stream's rows and one
// vector to every row: dst[r, :] = ((dst[r, :] + pending sums) + other[r, :]) + vector[:], what stands in front of a pass over a group
// of layers that takes the embedding output in again and marks the pass with a stored vector.
#include "common.cuh"
#include "step_ops.h"

SB_DEFINE_LAST_ERROR()

namespace {

using bf16 = __nv_bfloat16;
constexpr int kInFlight = 8;

struct Source {
  float* h;                 // [n][W] or null; zero afterwards
  const float* partials;    // [P][n][W] or null
  int n_partials;
  int64_t stride;
  float c;
};

// One element of a branch: its buffer (zero behind the read) plus its partial sums, h + (p0 + p1 + ..).
template <class V>
__device__ __forceinline__ V zero_of();
template <>
__device__ __forceinline__ float zero_of<float>() { return 0.0f; }
template <>
__device__ __forceinline__ float4 zero_of<float4>() { return make_float4(0.0f, 0.0f, 0.0f, 0.0f); }
__device__ __forceinline__ float add(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ float4 add(float4 a, float4 b) { return make_float4(__fadd_rn(a.x, b.x), __fadd_rn(a.y, b.y), __fadd_rn(a.z, b.z), __fadd_rn(a.w, b.w)); }
__device__ __forceinline__ float mul(float a, float c) { return __fmul_rn(a, c); }
__device__ __forceinline__ float4 mul(float4 a, float c) { return make_float4(__fmul_rn(a.x, c), __fmul_rn(a.y, c), __fmul_rn(a.z, c), __fmul_rn(a.w, c)); }
__device__ __forceinline__ float4 mul(float4 a, float4 c) { return make_float4(__fmul_rn(a.x, c.x), __fmul_rn(a.y, c.y), __fmul_rn(a.z, c.z), __fmul_rn(a.w, c.w)); }

template <class V>
__device__ __forceinline__ V source_value(const Source& s, int64_t i) {      // i in units of V
  V v = zero_of<V>();
  if (s.h != nullptr) {
    V* h = reinterpret_cast<V*>(s.h) + i;
    v = *h;
    *h = zero_of<V>();
  }
  if (s.partials != nullptr && s.n_partials > 0) {
    const V* p = reinterpret_cast<const V*>(s.partials) + i;
    const int64_t stride = s.stride / static_cast<int64_t>(sizeof(V) / sizeof(float));
    V part[kInFlight];
#pragma unroll
    for (int k = 0; k < kInFlight; ++k)
      if (k < s.n_partials) part[k] = p[k * stride];
    V sum = part[0];
#pragma unroll
    for (int k = 1; k < kInFlight; ++k)
      if (k < s.n_partials) sum = add(sum, part[k]);
    for (int k = kInFlight; k < s.n_partials; ++k) sum = add(sum, p[k * stride]);
    v = s.h != nullptr ? add(v, sum) : sum;
  }
  return v;
}

template <class TG>
__device__ __forceinline__ float4 gain4(const TG* gain, int c);
template <>
__device__ __forceinline__ float4 gain4<float>(const float* gain, int c) { return *reinterpret_cast<const float4*>(gain + c); }
template <>
__device__ __forceinline__ float4 gain4<bf16>(const bf16* gain, int c) {
  const uint2 raw = *reinterpret_cast<const uint2*>(gain + c);
  const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
  return make_float4(__low2float(lo), __high2float(lo), __low2float(hi), __high2float(hi));
}

// A block per row. VEC: the width is a multiple of four and every buffer 16-byte aligned: four elements a thread and request.
// The scalar form does the same operations on the same operands: equal bits.
template <class TG, bool VEC>
__global__ void __launch_bounds__(256) branch_fold_kernel(float* __restrict__ dst, Source a, Source b, const TG* __restrict__ gain, int W) {
  sb::grid_launch_dependents();
  sb::grid_dependency_wait();
  const int64_t row = static_cast<int64_t>(blockIdx.x) * W;
  const bool two = b.h != nullptr || b.partials != nullptr;
  if (VEC) {
    for (int c = threadIdx.x * 4; c < W; c += blockDim.x * 4) {
      const int64_t i = (row + c) / 4;
      float4 v = mul(source_value<float4>(a, i), a.c);
      if (two) v = add(v, mul(source_value<float4>(b, i), b.c));
      if (gain != nullptr) v = mul(v, gain4<TG>(gain, c));
      float4* d = reinterpret_cast<float4*>(dst) + i;
      *d = add(*d, v);
    }
  } else {
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
      const int64_t i = row + c;
      float v = mul(source_value<float>(a, i), a.c);
      if (two) v = add(v, mul(source_value<float>(b, i), b.c));
      if (gain != nullptr) v = mul(v, sb::widen(gain[c]));
      dst[i] = add(dst[i], v);
    }
  }
}

// A block per row: the row's values (the branches read and cleared as above) stay in shared memory between the sum of squares and the
// scaled add. The squares are added by a thread in ascending columns, then over the block in `block_sum`'s order. VEC: the width is a
// multiple of four and every buffer 16-byte aligned: four elements a thread and request. Which form runs depends on the width and the
// buffers alone, never on the rows of the step.
template <class TG, bool VEC>
__global__ void __launch_bounds__(256) branch_norm_fold_kernel(float* __restrict__ dst, Source a, Source b, const TG* __restrict__ gain, int W,
                                                               float eps) {
  extern __shared__ __align__(16) float row_values[];
  __shared__ float red[32];
  sb::grid_launch_dependents();
  sb::grid_dependency_wait();
  const int64_t row = static_cast<int64_t>(blockIdx.x) * W;
  const bool two = b.h != nullptr || b.partials != nullptr;
  float sq = 0.0f;
  if (VEC) {
    float4* held = reinterpret_cast<float4*>(row_values);
    for (int c = threadIdx.x * 4; c < W; c += blockDim.x * 4) {
      const int64_t i = (row + c) / 4;
      float4 v = mul(source_value<float4>(a, i), a.c);
      if (two) v = add(v, mul(source_value<float4>(b, i), b.c));
      held[c / 4] = v;
      sq = fmaf(v.x, v.x, sq), sq = fmaf(v.y, v.y, sq), sq = fmaf(v.z, v.z, sq), sq = fmaf(v.w, v.w, sq);
    }
    const float scale = 1.0f / sqrtf(sb::block_sum(sq, red) / static_cast<float>(W) + eps);
    for (int c = threadIdx.x * 4; c < W; c += blockDim.x * 4) {
      float4 v = mul(held[c / 4], scale);
      if (gain != nullptr) v = mul(v, gain4<TG>(gain, c));
      float4* d = reinterpret_cast<float4*>(dst) + (row + c) / 4;
      *d = add(*d, v);
    }
    return;
  }
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float v = mul(source_value<float>(a, row + c), a.c);
    if (two) v = add(v, mul(source_value<float>(b, row + c), b.c));
    row_values[c] = v;
    sq = fmaf(v, v, sq);
  }
  const float scale = 1.0f / sqrtf(sb::block_sum(sq, red) / static_cast<float>(W) + eps);
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float v = mul(row_values[c], scale);
    if (gain != nullptr) v = mul(v, sb::widen(gain[c]));
    dst[row + c] = add(dst[row + c], v);
  }
}

template <class TV>
__global__ void __launch_bounds__(256) stream_add_kernel(float* __restrict__ dst, const float* __restrict__ partials, int n_partials, int64_t stride,
                                                         const float* __restrict__ other, const TV* __restrict__ vector, int W) {
  sb::grid_launch_dependents();
  sb::grid_dependency_wait();
  const int64_t row = static_cast<int64_t>(blockIdx.x) * W;
  const Source pending{nullptr, partials, partials ? n_partials : 0, stride, 1.0f};
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float v = dst[row + c];
    if (partials != nullptr) v = add(v, source_value<float>(pending, row + c));
    if (other != nullptr) v = add(v, other[row + c]);
    if (vector != nullptr) v = add(v, sb::widen(vector[c]));
    dst[row + c] = v;
  }
}

template <class TX>
__global__ void __launch_bounds__(256) row_scaled_add_kernel(float* __restrict__ dst, const TX* __restrict__ x, const float* __restrict__ w, int ldw,
                                                             int first, int count, int W) {
  sb::grid_launch_dependents();
  sb::grid_dependency_wait();
  const int64_t r = blockIdx.x;
  float g = 0.0f;
  for (int k = 0; k < count; ++k) g += w[r * ldw + first + k];
  if (g == 0.0f) return;
  for (int c = threadIdx.x; c < W; c += blockDim.x) dst[r * W + c] = fmaf(g, sb::widen(x[r * W + c]), dst[r * W + c]);
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

SB_EXPORT int sb_branch_fold(float* dst, float* a, const float* pa, int na, int64_t sa, float ca, float* b, const float* pb, int nb, int64_t sb_,
                             float cb, const void* gain, int gain_dtype, int n, int W, cudaStream_t stream) {
  if (n <= 0 || W <= 0) return 0;
  if (a == nullptr && pa == nullptr) return sb::fail("sb_branch_fold: the first branch has neither a buffer nor partial sums");
  const Source A{a, pa, pa ? na : 0, sa, ca}, B{b, pb, pb ? nb : 0, sb_, cb};
  const bool vec = W % 4 == 0 && aligned16(dst) && aligned16(a) && aligned16(pa) && aligned16(b) && aligned16(pb) && aligned16(gain) &&
                   sa % 4 == 0 && sb_ % 4 == 0;
  const int threads = W >= 1024 ? 256 : 128;
#define SB_FOLD(TG, VEC) sb::launch_pdl(branch_fold_kernel<TG, VEC>, dim3(n), dim3(threads), 0, stream, dst, A, B, static_cast<const TG*>(gain), W)
  if (gain == nullptr || gain_dtype == 0) {
    if (vec) SB_FOLD(float, true);
    else SB_FOLD(float, false);
  } else if (gain_dtype == 1) {
    if (vec) SB_FOLD(bf16, true);
    else SB_FOLD(bf16, false);
  } else {
    return sb::fail("sb_branch_fold: unsupported gain dtype %d", gain_dtype);
  }
#undef SB_FOLD
  return sb::check_launch("sb_branch_fold");
}

SB_EXPORT int sb_branch_norm_fold(float* dst, float* a, const float* pa, int na, int64_t sa, float ca, float* b, const float* pb, int nb,
                                  int64_t sb_, float cb, const void* gain, int gain_dtype, float eps, int n, int W, cudaStream_t stream) {
  if (n <= 0 || W <= 0) return 0;
  if (a == nullptr && pa == nullptr) return sb::fail("sb_branch_norm_fold: the first branch has neither a buffer nor partial sums");
  const Source A{a, pa, pa ? na : 0, sa, ca}, B{b, pb, pb ? nb : 0, sb_, cb};
  const size_t smem = static_cast<size_t>(W) * sizeof(float);
  if (smem > 160 * 1024) return sb::fail("sb_branch_norm_fold: a row of %d elements does not fit the row buffer", W);
  const bool vec = W % 4 == 0 && aligned16(dst) && aligned16(a) && aligned16(pa) && aligned16(b) && aligned16(pb) && aligned16(gain) &&
                   sa % 4 == 0 && sb_ % 4 == 0;
  const int threads = W >= 1024 ? 256 : 128;
#define SB_NORM_FOLD(TG, VEC)                                                                                                              \
  do {                                                                                                                                     \
    if (smem > 48 * 1024) cudaFuncSetAttribute(branch_norm_fold_kernel<TG, VEC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
    sb::launch_pdl(branch_norm_fold_kernel<TG, VEC>, dim3(n), dim3(threads), smem, stream, dst, A, B, static_cast<const TG*>(gain), W, eps); \
  } while (0)
  if (gain == nullptr || gain_dtype == 0) {
    if (vec) SB_NORM_FOLD(float, true);
    else SB_NORM_FOLD(float, false);
  } else if (gain_dtype == 1) {
    if (vec) SB_NORM_FOLD(bf16, true);
    else SB_NORM_FOLD(bf16, false);
  } else {
    return sb::fail("sb_branch_norm_fold: unsupported gain dtype %d", gain_dtype);
  }
#undef SB_NORM_FOLD
  return sb::check_launch("sb_branch_norm_fold");
}

SB_EXPORT int sb_stream_add(float* dst, const float* partials, int n_partials, int64_t stride, const float* other, const void* vector,
                            int vector_dtype, int n, int W, cudaStream_t stream) {
  if (n <= 0 || W <= 0) return 0;
  if (vector == nullptr || vector_dtype == 0)
    sb::launch_pdl(stream_add_kernel<float>, dim3(n), dim3(256), 0, stream, dst, partials, n_partials, stride, other, static_cast<const float*>(vector), W);
  else if (vector_dtype == 1)
    sb::launch_pdl(stream_add_kernel<bf16>, dim3(n), dim3(256), 0, stream, dst, partials, n_partials, stride, other, static_cast<const bf16*>(vector), W);
  else
    return sb::fail("sb_stream_add: unsupported vector dtype %d", vector_dtype);
  return sb::check_launch("sb_stream_add");
}

SB_EXPORT int sb_row_scaled_add(float* dst, const void* x, int x_dtype, const float* w, int ldw, int first, int count, int n, int W,
                                cudaStream_t stream) {
  if (n <= 0 || W <= 0 || count <= 0) return 0;
  if (x_dtype == 0)
    sb::launch_pdl(row_scaled_add_kernel<float>, dim3(n), dim3(256), 0, stream, dst, static_cast<const float*>(x), w, ldw, first, count, W);
  else if (x_dtype == 1)
    sb::launch_pdl(row_scaled_add_kernel<bf16>, dim3(n), dim3(256), 0, stream, dst, static_cast<const bf16*>(x), w, ldw, first, count, W);
  else
    return sb::fail("sb_row_scaled_add: unsupported dtype %d", x_dtype);
  return sb::check_launch("sb_row_scaled_add");
}

// ------------------------------------------------------------------ operations of the native step program (step_ops.h)
// i: 0 dst, 1 a, 2 a's partial sums (flat), 3 their K ranges S, 4 most tokens with a buffer per range, 5 b, 6 b's partial sums, 7 their S,
//    8 gain, 9 gain dtype, 10 W
// f: 0 ca, 1 cb
SB_EXPORT int sb_op_branch_fold(const SbOp* op, const SbStep* s, void* stream) {
  using namespace sbstep;
  if (s->n <= 0) return SB_OP_SKIPPED;
  const int W = (int)op->i[10];
  const int64_t stride = static_cast<int64_t>(s->n) * W;
  return sb_branch_fold(ptr<float>(op->i[0]), ptr<float>(op->i[1]), ptr<const float>(op->i[2]), partial_count(op->i[3], op->i[4], s->n), stride,
                        static_cast<float>(op->f[0]), ptr<float>(op->i[5]), ptr<const float>(op->i[6]), partial_count(op->i[7], op->i[4], s->n),
                        stride, static_cast<float>(op->f[1]), ptr<const void>(op->i[8]), (int)op->i[9], s->n, W, static_cast<cudaStream_t>(stream));
}

// i: as sb_op_branch_fold      f: 0 ca, 1 cb, 2 eps
SB_EXPORT int sb_op_branch_norm_fold(const SbOp* op, const SbStep* s, void* stream) {
  using namespace sbstep;
  if (s->n <= 0) return SB_OP_SKIPPED;
  const int W = (int)op->i[10];
  const int64_t stride = static_cast<int64_t>(s->n) * W;
  return sb_branch_norm_fold(ptr<float>(op->i[0]), ptr<float>(op->i[1]), ptr<const float>(op->i[2]), partial_count(op->i[3], op->i[4], s->n), stride,
                             static_cast<float>(op->f[0]), ptr<float>(op->i[5]), ptr<const float>(op->i[6]), partial_count(op->i[7], op->i[4], s->n),
                             stride, static_cast<float>(op->f[1]), ptr<const void>(op->i[8]), (int)op->i[9], static_cast<float>(op->f[2]), s->n, W,
                             static_cast<cudaStream_t>(stream));
}

// i: 0 dst, 1 pending partial sums (flat, or 0), 2 their K ranges S, 3 most tokens with a buffer per range, 4 the other stream (or 0),
//    5 the vector (or 0), 6 its dtype, 7 W
SB_EXPORT int sb_op_stream_add(const SbOp* op, const SbStep* s, void* stream) {
  using namespace sbstep;
  if (s->n <= 0) return SB_OP_SKIPPED;
  const int W = (int)op->i[7];
  return sb_stream_add(ptr<float>(op->i[0]), ptr<const float>(op->i[1]), partial_count(op->i[2], op->i[3], s->n), static_cast<int64_t>(s->n) * W,
                       ptr<const float>(op->i[4]), ptr<const void>(op->i[5]), (int)op->i[6], s->n, W, static_cast<cudaStream_t>(stream));
}

// i: 0 dst, 1 x, 2 x dtype, 3 w, 4 ldw, 5 first column, 6 columns, 7 W
SB_EXPORT int sb_op_row_scaled_add(const SbOp* op, const SbStep* s, void* stream) {
  using namespace sbstep;
  if (s->n <= 0) return SB_OP_SKIPPED;
  return sb_row_scaled_add(ptr<float>(op->i[0]), ptr<const void>(op->i[1]), (int)op->i[2], ptr<const float>(op->i[3]), (int)op->i[4], (int)op->i[5],
                           (int)op->i[6], s->n, (int)op->i[7], static_cast<cudaStream_t>(stream));
}

// ---------------------------------------------------------------------------------------------------------------------------------
// Two branches that are each RMS-normed over their row, with a gain of their own, before their weighted sum joins `dst`:
//
//   dst[r, j] += w[j] * (ca * ga[j] * A[r, j] / sqrt(mean_j(A[r, :]^2) + eps) + cb * gb[j] * B[r, j] / sqrt(mean_j(B[r, :]^2) + eps))
//
// with A = a + (pa_0 + pa_1 + ..), B likewise, and w a gain on the sum (a layer scale) or none; the branch buffers are zero afterwards. What mixers side by side need whose results are
// normed one by one. A block per row, both rows held in shared memory between the sums of squares and the add.
namespace {

template <class TG, bool VEC>
__global__ void __launch_bounds__(256) branch_pair_norm_fold_kernel(float* __restrict__ dst, Source a, Source b, const TG* __restrict__ ga,
                                                                    const TG* __restrict__ gb, const TG* __restrict__ outer, int W, float eps) {
  extern __shared__ __align__(16) float row_values[];      // [2][W]
  __shared__ float red[32];
  sb::grid_launch_dependents();
  sb::grid_dependency_wait();
  const int64_t row = static_cast<int64_t>(blockIdx.x) * W;
  float sa = 0.0f, sb2 = 0.0f;
  if (VEC) {      // four elements a thread and request; the squares of a thread's elements in ascending columns, as in the scalar form per element
    float4* held = reinterpret_cast<float4*>(row_values);
    for (int c = threadIdx.x * 4; c < W; c += blockDim.x * 4) {
      const int64_t i = (row + c) / 4;
      const float4 va = source_value<float4>(a, i), vb = source_value<float4>(b, i);
      held[c / 4] = va, held[(W + c) / 4] = vb;
      sa = fmaf(va.x, va.x, sa), sa = fmaf(va.y, va.y, sa), sa = fmaf(va.z, va.z, sa), sa = fmaf(va.w, va.w, sa);
      sb2 = fmaf(vb.x, vb.x, sb2), sb2 = fmaf(vb.y, vb.y, sb2), sb2 = fmaf(vb.z, vb.z, sb2), sb2 = fmaf(vb.w, vb.w, sb2);
    }
    const float ra = mul(a.c, 1.0f / sqrtf(sb::block_sum(sa, red) / static_cast<float>(W) + eps));
    const float rb = mul(b.c, 1.0f / sqrtf(sb::block_sum(sb2, red) / static_cast<float>(W) + eps));
    for (int c = threadIdx.x * 4; c < W; c += blockDim.x * 4) {
      const float4 va = mul(mul(held[c / 4], ra), gain4<TG>(ga, c)), vb = mul(mul(held[(W + c) / 4], rb), gain4<TG>(gb, c));
      float4* d = reinterpret_cast<float4*>(dst) + (row + c) / 4;
      float4 v = add(va, vb);
      if (outer != nullptr) v = mul(v, gain4<TG>(outer, c));
      *d = add(*d, v);
    }
    return;
  }
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    const float va = source_value<float>(a, row + c), vb = source_value<float>(b, row + c);
    row_values[c] = va, row_values[W + c] = vb;
    sa = fmaf(va, va, sa), sb2 = fmaf(vb, vb, sb2);
  }
  const float ra = mul(a.c, 1.0f / sqrtf(sb::block_sum(sa, red) / static_cast<float>(W) + eps));
  const float rb = mul(b.c, 1.0f / sqrtf(sb::block_sum(sb2, red) / static_cast<float>(W) + eps));
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    const float va = mul(mul(row_values[c], ra), sb::widen(ga[c])), vb = mul(mul(row_values[W + c], rb), sb::widen(gb[c]));
    float v = add(va, vb);
    if (outer != nullptr) v = mul(v, sb::widen(outer[c]));
    dst[row + c] = add(dst[row + c], v);
  }
}

}  // namespace

// i: 0 dst, 1 a, 2 a's partial sums (flat), 3 their K ranges S, 4 most tokens with a buffer per range, 5 b, 6 b's partial sums, 7 their S,
//    8 a's gain, 9 b's gain, 10 the gains' dtype, 11 W, 12 a gain on the sum, of the same dtype (or 0)
// f: 0 ca, 1 cb, 2 eps
SB_EXPORT int sb_op_branch_pair_norm_fold(const SbOp* op, const SbStep* s, void* stream) {
  using namespace sbstep;
  if (s->n <= 0) return SB_OP_SKIPPED;
  const int W = (int)op->i[11];
  const int64_t stride = static_cast<int64_t>(s->n) * W;
  float* a = ptr<float>(op->i[1]);
  float* b = ptr<float>(op->i[5]);
  const float* pa = ptr<const float>(op->i[2]);
  const float* pb = ptr<const float>(op->i[6]);
  if ((a == nullptr && pa == nullptr) || (b == nullptr && pb == nullptr)) return sb::fail("sb_op_branch_pair_norm_fold: a branch with neither a buffer nor partial sums"), SB_OP_FAILED;
  const Source A{a, pa, pa ? partial_count(op->i[3], op->i[4], s->n) : 0, stride, static_cast<float>(op->f[0])};
  const Source B{b, pb, pb ? partial_count(op->i[7], op->i[4], s->n) : 0, stride, static_cast<float>(op->f[1])};
  const size_t smem = static_cast<size_t>(2) * W * sizeof(float);
  if (smem > 160 * 1024) return sb::fail("sb_op_branch_pair_norm_fold: rows of %d elements do not fit the row buffer", W), SB_OP_FAILED;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int threads = W >= 1024 ? 256 : 128;
  // which form runs depends on the width and the buffers alone, never on the rows of the step
  const bool vec = W % 4 == 0 && stride % 4 == 0 && aligned16(ptr<float>(op->i[0])) && aligned16(a) && aligned16(pa) && aligned16(b) && aligned16(pb) &&
                   aligned16(ptr<const void>(op->i[8])) && aligned16(ptr<const void>(op->i[9])) && aligned16(ptr<const void>(op->i[12]));
#define SB_PAIR(TG, VEC)                                                                                                                        \
  do {                                                                                                                                          \
    if (smem > 48 * 1024) cudaFuncSetAttribute(branch_pair_norm_fold_kernel<TG, VEC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
    sb::launch_pdl(branch_pair_norm_fold_kernel<TG, VEC>, dim3(s->n), dim3(threads), smem, st, ptr<float>(op->i[0]), A, B, ptr<const TG>(op->i[8]), \
                   ptr<const TG>(op->i[9]), ptr<const TG>(op->i[12]), W, static_cast<float>(op->f[2]));                                         \
  } while (0)
  if (op->i[10] == 0) {
    if (vec) SB_PAIR(float, true);
    else SB_PAIR(float, false);
  } else if (op->i[10] == 1) {
    if (vec) SB_PAIR(bf16, true);
    else SB_PAIR(bf16, false);
  } else {
    return sb::fail("sb_op_branch_pair_norm_fold: unsupported gain dtype %d", (int)op->i[10]), SB_OP_FAILED;
  }
#undef SB_PAIR
  return sb::check_launch("sb_op_branch_pair_norm_fold");
}
