// Branches beside the residual stream. A sublayer whose result is scaled before it joins the residual (a per-channel
// layer scale, a constant per branch, or both) writes into a branch buffer of the stream's shape instead: its last
// projection either adds into the buffer or leaves one partial sum per K range. The fold
//
//   dst[r, j] += gain[j] * (ca * (a[r, j] + (pa_0 + pa_1 + ..)[r, j]) + cb * (b[r, j] + (pb_0 + pb_1 + ..)[r, j]))
//
// takes up to two branches into `dst` (the residual, or another branch) in 32-bit and leaves the branch buffers zero,
// which is the state the next sublayer expects to find them in. The order of the additions is fixed.
//
// A second kernel adds a row-scaled copy of the sublayer's input: dst[r, :] += (sum of `count` columns of w[r, :]) * x[r, :],
// what experts that pass their input through contribute to a routed feed-forward.
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

__device__ __forceinline__ float source_value(const Source& s, int64_t i) {
  float v = 0.0f;
  if (s.h != nullptr) {
    v = s.h[i];
    s.h[i] = 0.0f;
  }
  if (s.partials != nullptr && s.n_partials > 0) {
    float part[kInFlight];
#pragma unroll
    for (int k = 0; k < kInFlight; ++k)
      if (k < s.n_partials) part[k] = s.partials[k * s.stride + i];
    float sum = part[0];
#pragma unroll
    for (int k = 1; k < kInFlight; ++k)
      if (k < s.n_partials) sum += part[k];
    for (int k = kInFlight; k < s.n_partials; ++k) sum += s.partials[k * s.stride + i];
    v = s.h != nullptr ? v + sum : sum;
  }
  return v;
}

template <class TG>
__global__ void branch_fold_kernel(float* __restrict__ dst, Source a, Source b, const TG* __restrict__ gain, int64_t total, int W) {
  sb::grid_launch_dependents();
  sb::grid_dependency_wait();
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float v = __fmul_rn(a.c, source_value(a, i));
    if (b.h != nullptr || b.partials != nullptr) v = __fadd_rn(v, __fmul_rn(b.c, source_value(b, i)));
    if (gain != nullptr) v = __fmul_rn(v, sb::widen(gain[i % W]));
    dst[i] = __fadd_rn(dst[i], v);
  }
}

template <class TX>
__global__ void row_scaled_add_kernel(float* __restrict__ dst, const TX* __restrict__ x, const float* __restrict__ w, int ldw, int first,
                                      int count, int64_t total, int W) {
  sb::grid_launch_dependents();
  sb::grid_dependency_wait();
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / W;
    float g = 0.0f;
    for (int k = 0; k < count; ++k) g += w[r * ldw + first + k];
    if (g != 0.0f) dst[i] = fmaf(g, sb::widen(x[i]), dst[i]);
  }
}

inline int grid_for(int64_t total) {
  const int64_t blocks = (total + 255) / 256, most = static_cast<int64_t>(sb::sm_count()) * 16;
  return static_cast<int>(blocks < most ? blocks : most);
}

}  // namespace

SB_EXPORT int sb_branch_fold(float* dst, float* a, const float* pa, int na, int64_t sa, float ca, float* b, const float* pb, int nb, int64_t sb_,
                             float cb, const void* gain, int gain_dtype, int n, int W, cudaStream_t stream) {
  if (n <= 0 || W <= 0) return 0;
  if (a == nullptr && pa == nullptr) return sb::fail("sb_branch_fold: the first branch has neither a buffer nor partial sums");
  const int64_t total = static_cast<int64_t>(n) * W;
  const Source A{a, pa, pa ? na : 0, sa, ca}, B{b, pb, pb ? nb : 0, sb_, cb};
  if (gain == nullptr || gain_dtype == 0)
    sb::launch_pdl(branch_fold_kernel<float>, dim3(grid_for(total)), dim3(256), 0, stream, dst, A, B, static_cast<const float*>(gain), total, W);
  else if (gain_dtype == 1)
    sb::launch_pdl(branch_fold_kernel<bf16>, dim3(grid_for(total)), dim3(256), 0, stream, dst, A, B, static_cast<const bf16*>(gain), total, W);
  else
    return sb::fail("sb_branch_fold: unsupported gain dtype %d", gain_dtype);
  return sb::check_launch("sb_branch_fold");
}

SB_EXPORT int sb_row_scaled_add(float* dst, const void* x, int x_dtype, const float* w, int ldw, int first, int count, int n, int W,
                                cudaStream_t stream) {
  if (n <= 0 || W <= 0 || count <= 0) return 0;
  const int64_t total = static_cast<int64_t>(n) * W;
  if (x_dtype == 0)
    sb::launch_pdl(row_scaled_add_kernel<float>, dim3(grid_for(total)), dim3(256), 0, stream, dst, static_cast<const float*>(x), w, ldw, first, count, total, W);
  else if (x_dtype == 1)
    sb::launch_pdl(row_scaled_add_kernel<bf16>, dim3(grid_for(total)), dim3(256), 0, stream, dst, static_cast<const bf16*>(x), w, ldw, first, count, total, W);
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

// i: 0 dst, 1 x, 2 x dtype, 3 w, 4 ldw, 5 first column, 6 columns, 7 W
SB_EXPORT int sb_op_row_scaled_add(const SbOp* op, const SbStep* s, void* stream) {
  using namespace sbstep;
  if (s->n <= 0) return SB_OP_SKIPPED;
  return sb_row_scaled_add(ptr<float>(op->i[0]), ptr<const void>(op->i[1]), (int)op->i[2], ptr<const float>(op->i[3]), (int)op->i[4], (int)op->i[5],
                           (int)op->i[6], s->n, (int)op->i[7], static_cast<cudaStream_t>(stream));
}
