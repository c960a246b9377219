// The recurrent block with a real-gated linear recurrent unit (RG-LRU), the pieces between its projections:
//
//   u_t = conv(x)_t          a causal convolution per channel over the last `taps` inputs x = W_x h + b_x (zeros before the sequence)
//   r_t = sigmoid(A_b u_t,b + a_b), i_t = sigmoid(I_b u_t,b + i_b)      per block b of channels (the products are made by the caller)
//   a_t = exp(-8 r_t softplus(lam)),  S_t = a_t S_(t-1) + sqrt(1 - a_t^2) (i_t u_t),  out_t = S_t * gelu_tanh(W_y h + b_y)_t
//
// Per request the state record [taps][C] float32 holds the last taps - 1 inputs of the convolution (rows 0 .. taps - 2, oldest
// first) and S (row taps - 1); a request that starts at position 0 starts from zeros whatever the record holds. Everything is
// 32-bit. Three kernels: `rglru_conv_kernel` (a thread per token and channel; earlier inputs come from the step's own rows
// or from the record), `rglru_gates_kernel` (a thread per token and channel: a, the driven input and the gelu branch), and
// `rglru_scan_kernel` (a thread per request and channel walks the tokens in order, one fused multiply-add a token, and writes
// the record back). A token's result has the same bits however the sequence was cut into steps.
#include "common.cuh"
#include "step_ops.h"

SB_DEFINE_LAST_ERROR()

namespace {

using bf16 = __nv_bfloat16;
constexpr int kInFlight = 8;
constexpr int kMaxTaps = 16;

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

__device__ __forceinline__ float gelu_tanh(float z) {
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

struct Proj {
  const float* p;            // [P][n][2 C]: columns y | x
  int n_partials;
  int64_t stride;
};

// u[r, c] = conv_b[c] + sum_j taps[c, j] * x[position - (K - 1 - j)]
template <class TW>
__global__ void rglru_conv_kernel(Proj proj, const TW* __restrict__ x_bias, const TW* __restrict__ taps, const TW* __restrict__ conv_bias,
                                  const int32_t* __restrict__ positions, const int32_t* __restrict__ slots, const float* __restrict__ state,
                                  float* __restrict__ u, int n, int C, int K) {
  sb::grid_launch_dependents();
  const int row = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
  const int pos = positions[row], slot = slots[row];
  // how many tokens in front of this one the step itself brings (rows of a request are contiguous and ascending)
  int mine = 0;
  while (mine < K - 1 && row - mine - 1 >= 0 && slots[row - mine - 1] == slot) ++mine;
  sb::grid_dependency_wait();
  if (c >= C) return;
  const float xb = sb::widen(x_bias[c]);
  float sum = sb::widen(conv_bias[c]);
  for (int back = K - 1; back >= 0; --back) {       // oldest first
    float x = 0.0f;
    if (back <= mine) {
      x = folded(proj.p + static_cast<int64_t>(row - back) * 2 * C + C + c, proj.n_partials, proj.stride) + xb;
    } else if (pos - back >= 0) {
      // the record's row j holds the input at position first - (K - 1) + j, first = pos - mine being the step's first position
      x = state[(static_cast<int64_t>(slot) * K + (K - 1 - back + mine)) * C + c];
    }
    sum = fmaf(sb::widen(taps[c * K + (K - 1 - back)]), x, sum);
  }
  u[static_cast<int64_t>(row) * C + c] = sum;
}

// gates [n][B][2][bw]: the pre-activations of r and i. Writes a, the driven input d = sqrt(1 - a^2) i u, and y = gelu(W_y h + b_y).
template <class TW>
__global__ void rglru_gates_kernel(const float* __restrict__ gates, const TW* __restrict__ r_bias, const TW* __restrict__ i_bias,
                                   const TW* __restrict__ lam, const float* __restrict__ u, Proj proj, const TW* __restrict__ y_bias,
                                   float* __restrict__ a_out, float* __restrict__ d_out, float* __restrict__ y_out, int64_t total, int C, int bw) {
  sb::grid_launch_dependents();
  sb::grid_dependency_wait();
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / C;
    const int c = static_cast<int>(i % C), b = c / bw, j = c % bw;
    const float* g = gates + r * 2 * C + static_cast<int64_t>(b) * 2 * bw + j;
    const float rg = 1.0f / (1.0f + expf(-(g[0] + sb::widen(r_bias[c]))));
    const float ig = 1.0f / (1.0f + expf(-(g[bw] + sb::widen(i_bias[c]))));
    const float l = sb::widen(lam[c]);
    const float softplus = l > 20.0f ? l : log1pf(expf(l));
    const float log_a = -8.0f * rg * softplus;
    a_out[i] = expf(log_a);
    d_out[i] = sqrtf(-expm1f(2.0f * log_a)) * (ig * u[i]);
    y_out[i] = gelu_tanh(folded(proj.p + r * 2 * C + c, proj.n_partials, proj.stride) + sb::widen(y_bias[c]));
  }
}

template <class TW, class TO>
__global__ void rglru_scan_kernel(const float* __restrict__ a, const float* __restrict__ d, const float* __restrict__ y, Proj proj,
                                  const TW* __restrict__ x_bias, const int32_t* __restrict__ meta, int meta_stride, float* __restrict__ state,
                                  TO* __restrict__ out, int C, int K) {
  sb::grid_launch_dependents();
  const int e = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
  const int slot = meta[e], row0 = meta[meta_stride + e], len = meta[2 * meta_stride + e], pos0 = meta[3 * meta_stride + e];
  sb::grid_dependency_wait();
  if (c >= C) return;
  float* rec = state + static_cast<int64_t>(slot) * K * C + c;
  float S = pos0 > 0 ? rec[static_cast<int64_t>(K - 1) * C] : 0.0f;
  const int64_t base = static_cast<int64_t>(row0) * C + c;
#pragma unroll 4
  for (int t = 0; t < len; ++t) {
    const int64_t i = base + static_cast<int64_t>(t) * C;
    S = fmaf(a[i], S, d[i]);
    out[i] = sb::narrow<TO>(S * y[i]);
  }
  // the record for the step behind this one: the inputs at positions end - (K - 1) .. end - 1 and S
  float hist[kMaxTaps];
  const float xb = sb::widen(x_bias[c]);
  for (int j = 0; j < K - 1; ++j) {
    const int back = K - 1 - j;                       // the input `back` tokens before the next one
    float x = 0.0f;
    if (back <= len) x = folded(proj.p + static_cast<int64_t>(row0 + len - back) * 2 * C + C + c, proj.n_partials, proj.stride) + xb;
    else if (pos0 + len - back >= 0) x = rec[static_cast<int64_t>(j + len) * C];      // (only if pos0 > 0: the record is then valid)
    hist[j] = x;
  }
  for (int j = 0; j < K - 1; ++j) rec[static_cast<int64_t>(j) * C] = hist[j];
  rec[static_cast<int64_t>(K - 1) * C] = S;
}

inline int grid_for(int64_t total) {
  const int64_t blocks = (total + 255) / 256, most = static_cast<int64_t>(sb::sm_count()) * 16;
  return static_cast<int>(blocks < most ? blocks : most);
}

}  // namespace

SB_EXPORT int sb_rglru_conv(const float* proj, int n_partials, int64_t partial_stride, const void* x_bias, const void* taps, const void* conv_bias,
                            int w_dtype, const int32_t* positions, const int32_t* slots, const float* state, float* u, int n, int C, int K,
                            cudaStream_t stream) {
  if (n <= 0) return 0;
  if (K < 1 || K > kMaxTaps) return sb::fail("sb_rglru_conv: %d taps (1 to %d)", K, kMaxTaps);
  if (n_partials < 1) return sb::fail("sb_rglru_conv: n_partials must be >= 1");
  const Proj pr{proj, n_partials, partial_stride};
  const dim3 grid(n, (C + 127) / 128);
  if (w_dtype == 0)
    sb::launch_pdl(rglru_conv_kernel<float>, grid, dim3(128), 0, stream, pr, static_cast<const float*>(x_bias), static_cast<const float*>(taps),
                   static_cast<const float*>(conv_bias), positions, slots, state, u, n, C, K);
  else if (w_dtype == 1)
    sb::launch_pdl(rglru_conv_kernel<bf16>, grid, dim3(128), 0, stream, pr, static_cast<const bf16*>(x_bias), static_cast<const bf16*>(taps),
                   static_cast<const bf16*>(conv_bias), positions, slots, state, u, n, C, K);
  else
    return sb::fail("sb_rglru_conv: unsupported dtype %d", w_dtype);
  return sb::check_launch("sb_rglru_conv");
}

SB_EXPORT int sb_rglru_gates(const float* gates, const void* r_bias, const void* i_bias, const void* lam, const void* y_bias, int w_dtype,
                             const float* u, const float* proj, int n_partials, int64_t partial_stride, float* a, float* d, float* y, int n, int C,
                             int blocks, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (blocks <= 0 || C % blocks != 0) return sb::fail("sb_rglru_gates: %d channels do not divide into %d blocks", C, blocks);
  const Proj pr{proj, n_partials, partial_stride};
  const int64_t total = static_cast<int64_t>(n) * C;
  if (w_dtype == 0)
    sb::launch_pdl(rglru_gates_kernel<float>, dim3(grid_for(total)), dim3(256), 0, stream, gates, static_cast<const float*>(r_bias),
                   static_cast<const float*>(i_bias), static_cast<const float*>(lam), u, pr, static_cast<const float*>(y_bias), a, d, y, total, C, C / blocks);
  else if (w_dtype == 1)
    sb::launch_pdl(rglru_gates_kernel<bf16>, dim3(grid_for(total)), dim3(256), 0, stream, gates, static_cast<const bf16*>(r_bias),
                   static_cast<const bf16*>(i_bias), static_cast<const bf16*>(lam), u, pr, static_cast<const bf16*>(y_bias), a, d, y, total, C, C / blocks);
  else
    return sb::fail("sb_rglru_gates: unsupported dtype %d", w_dtype);
  return sb::check_launch("sb_rglru_gates");
}

SB_EXPORT int sb_rglru_scan(const float* a, const float* d, const float* y, const float* proj, int n_partials, int64_t partial_stride,
                            const void* x_bias, int w_dtype, const int32_t* meta, int meta_stride, int entries, float* state, void* out,
                            int out_dtype, int C, int K, cudaStream_t stream) {
  if (entries <= 0) return 0;
  if (K < 1 || K > kMaxTaps) return sb::fail("sb_rglru_scan: %d taps (1 to %d)", K, kMaxTaps);
  const Proj pr{proj, n_partials, partial_stride};
  const dim3 grid(entries, (C + 63) / 64);
#define SB_SCAN(TW, TO) sb::launch_pdl(rglru_scan_kernel<TW, TO>, grid, dim3(64), 0, stream, a, d, y, pr, static_cast<const TW*>(x_bias), meta, meta_stride, state, static_cast<TO*>(out), C, K)
  if (w_dtype == 0 && out_dtype == 0) SB_SCAN(float, float);
  else if (w_dtype == 0 && out_dtype == 1) SB_SCAN(float, bf16);
  else if (w_dtype == 1 && out_dtype == 0) SB_SCAN(bf16, float);
  else if (w_dtype == 1 && out_dtype == 1) SB_SCAN(bf16, bf16);
  else return sb::fail("sb_rglru_scan: unsupported dtypes weights=%d out=%d", w_dtype, out_dtype);
#undef SB_SCAN
  return sb::check_launch("sb_rglru_scan");
}

// ------------------------------------------------------------------ operations of the native step program (step_ops.h)
// i: 0 projection partial sums (flat), 1 K ranges S, 2 most tokens with a buffer per range, 3 x bias, 4 taps, 5 conv bias, 6 their dtype, 7 state,
//    8 u, 9 C, 10 K
SB_EXPORT int sb_op_rglru_conv(const SbOp* op, const SbStep* s, void* stream) {
  using namespace sbstep;
  if (s->n <= 0) return SB_OP_SKIPPED;
  const int C = (int)op->i[9];
  return sb_rglru_conv(ptr<const float>(op->i[0]), partial_count(op->i[1], op->i[2], s->n), static_cast<int64_t>(s->n) * 2 * C, ptr<const void>(op->i[3]),
                       ptr<const void>(op->i[4]), ptr<const void>(op->i[5]), (int)op->i[6], positions(s), slots(s), ptr<const float>(op->i[7]),
                       ptr<float>(op->i[8]), s->n, C, (int)op->i[10], static_cast<cudaStream_t>(stream));
}

// i: 0 gates, 1 r bias, 2 i bias, 3 lam, 4 y bias, 5 their dtype, 6 u, 7 projection partial sums, 8 K ranges S, 9 most tokens with a buffer per range,
//    10 a, 11 d, 12 y, 13 C, 14 blocks
SB_EXPORT int sb_op_rglru_gates(const SbOp* op, const SbStep* s, void* stream) {
  using namespace sbstep;
  if (s->n <= 0) return SB_OP_SKIPPED;
  const int C = (int)op->i[13];
  return sb_rglru_gates(ptr<const float>(op->i[0]), ptr<const void>(op->i[1]), ptr<const void>(op->i[2]), ptr<const void>(op->i[3]),
                        ptr<const void>(op->i[4]), (int)op->i[5], ptr<const float>(op->i[6]), ptr<const float>(op->i[7]),
                        partial_count(op->i[8], op->i[9], s->n), static_cast<int64_t>(s->n) * 2 * C, ptr<float>(op->i[10]), ptr<float>(op->i[11]),
                        ptr<float>(op->i[12]), s->n, C, (int)op->i[14], static_cast<cudaStream_t>(stream));
}

// i: 0 a, 1 d, 2 y, 3 projection partial sums, 4 K ranges S, 5 most tokens with a buffer per range, 6 x bias, 7 its dtype, 8 state, 9 out, 10 out dtype,
//    11 C, 12 K
SB_EXPORT int sb_op_rglru_scan(const SbOp* op, const SbStep* s, void* stream) {
  using namespace sbstep;
  if (s->n <= 0) return SB_OP_SKIPPED;
  const int C = (int)op->i[11];
  return sb_rglru_scan(ptr<const float>(op->i[0]), ptr<const float>(op->i[1]), ptr<const float>(op->i[2]), ptr<const float>(op->i[3]),
                       partial_count(op->i[4], op->i[5], s->n), static_cast<int64_t>(s->n) * 2 * C, ptr<const void>(op->i[6]), (int)op->i[7],
                       entry_meta(s), s->max_rows, s->entries, ptr<float>(op->i[8]), ptr<void>(op->i[9]), (int)op->i[10], C, (int)op->i[12],
                       static_cast<cudaStream_t>(stream));
}
