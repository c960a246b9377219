// The recurrent block with a real-gated linear recurrent unit (RG-LRU), the pieces between its projections:
//
//   u_t = conv(x)_t          a causal convolution per channel over the last `taps` inputs x = W_x h + b_x (zeros before the sequence)
//   r_t = sigmoid(A_b u_t,b + a_b), i_t = sigmoid(I_b u_t,b + i_b)      per block b of channels (the products are made by the caller)
//   a_t = exp(-8 r_t softplus(lam)),  S_t = a_t S_(t-1) + sqrt(1 - a_t^2) (i_t u_t),  out_t = S_t * gelu_tanh(W_y h + b_y)_t
//
// Per request the state record [taps][C] float32 holds the last taps - 1 inputs of the convolution (rows 0 .. taps - 2, oldest
// first) and S (row taps - 1); a request that starts at position 0 starts from zeros whatever the record holds. Everything is
// 32-bit. Three kernels: `rglru_conv_kernel` (a thread per token and channel; earlier inputs come from the step's own rows
// or from the record), `rglru_gates_kernel` (the blocks' products in true float32, then a, the driven input and the gelu
// branch), and `rglru_scan_kernel` (a thread per request and channel walks the tokens in order, one fused multiply-add a token,
// and writes the record back). A token's result has the same bits however the sequence was cut into steps.
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

// The gates of kTT tokens for up to kGateOutputs channels of one block of channels. The block's inputs k are cut into four quarters (a function of
// the block's size alone), kGateOutputs / 32 warps each; a thread adds for its channel j, over its quarter in ascending order, gate_w[b][k][j] u[t][k] for r and
// gate_w[b][k][bw + j] u[t][k] for i (the matrices lie transposed, so that a warp reads consecutive weights; the tokens' inputs
// are broadcast from shared memory), one chain of fused multiply-adds per gate, token and quarter; the quarters are added in
// ascending order. Nothing of that depends on the step: the same bits however many tokens it brings. Then a, the driven input
// d = sqrt(1 - a^2) i u and y = gelu(W_y h + b_y).
constexpr int kTT = 16, kQuarters = 4, kGateOutputs = 64;

template <class TG, class TW>
__global__ void __launch_bounds__(kGateOutputs * kQuarters) rglru_gates_kernel(const TG* __restrict__ gate_w, const TW* __restrict__ r_bias,
                                                                      const TW* __restrict__ i_bias, const TW* __restrict__ lam,
                                                                      const float* __restrict__ u, Proj proj, const TW* __restrict__ y_bias,
                                                                      float* __restrict__ a_out, float* __restrict__ d_out, float* __restrict__ y_out,
                                                                      int n, int C, int bw) {
  extern __shared__ __align__(16) float us[];         // [bw][kTT] (an input's tokens side by side: four 16-byte reads an input), then the quarters' sums [kQuarters][2][kTT][outputs of the CTA]
  float* red = us + kTT * bw;
  sb::grid_launch_dependents();
  const int t0 = blockIdx.x * kTT, b = blockIdx.y;
  const int nt = min(kTT, n - t0);
  const int outs = blockDim.x / kQuarters;            // channels of this CTA (a multiple of 32)
  const int lane = threadIdx.x % outs, quarter = threadIdx.x / outs, j = blockIdx.z * outs + lane;
  sb::grid_dependency_wait();
  for (int i = threadIdx.x; i < kTT * bw; i += blockDim.x) {
    const int t = i / bw, k = i % bw;
    us[k * kTT + t] = t < nt ? u[static_cast<int64_t>(t0 + t) * C + b * bw + k] : 0.0f;
  }
  __syncthreads();
  const int per = (bw + kQuarters - 1) / kQuarters, k_begin = quarter * per, k_end = min(bw, k_begin + per);
  float ar[kTT], ai[kTT];
#pragma unroll
  for (int t = 0; t < kTT; ++t) ar[t] = ai[t] = 0.0f;
  if (j < bw) {
    const TG* w = gate_w + static_cast<int64_t>(b) * bw * 2 * bw + j;
    constexpr int kAhead = 8;        // inputs whose weights are requested together
    for (int k0 = k_begin; k0 < k_end; k0 += kAhead) {
      float wr[kAhead], wi[kAhead];
#pragma unroll
      for (int i = 0; i < kAhead; ++i) {
        const int k = min(k0 + i, bw - 1);
        wr[i] = sb::widen(w[static_cast<int64_t>(k) * 2 * bw]);
        wi[i] = sb::widen(w[static_cast<int64_t>(k) * 2 * bw + bw]);
      }
#pragma unroll
      for (int i = 0; i < kAhead; ++i) {
        if (k0 + i >= k_end) break;
        const float4* x4 = reinterpret_cast<const float4*>(us + (k0 + i) * kTT);
#pragma unroll
        for (int t = 0; t < kTT / 4; ++t) {
          const float4 x = x4[t];
          ar[4 * t] = fmaf(wr[i], x.x, ar[4 * t]);
          ai[4 * t] = fmaf(wi[i], x.x, ai[4 * t]);
          ar[4 * t + 1] = fmaf(wr[i], x.y, ar[4 * t + 1]);
          ai[4 * t + 1] = fmaf(wi[i], x.y, ai[4 * t + 1]);
          ar[4 * t + 2] = fmaf(wr[i], x.z, ar[4 * t + 2]);
          ai[4 * t + 2] = fmaf(wi[i], x.z, ai[4 * t + 2]);
          ar[4 * t + 3] = fmaf(wr[i], x.w, ar[4 * t + 3]);
          ai[4 * t + 3] = fmaf(wi[i], x.w, ai[4 * t + 3]);
        }
      }
    }
  }
#pragma unroll
  for (int t = 0; t < kTT; ++t) {
    red[((quarter * 2 + 0) * kTT + t) * outs + lane] = ar[t];
    red[((quarter * 2 + 1) * kTT + t) * outs + lane] = ai[t];
  }
  __syncthreads();
  if (j >= bw) return;
  const int c = b * bw + j;
  const float rb = sb::widen(r_bias[c]), ib = sb::widen(i_bias[c]), l = sb::widen(lam[c]), yb = sb::widen(y_bias[c]);
  const float softplus = l > 20.0f ? l : log1pf(expf(l));
  for (int t = quarter; t < nt; t += kQuarters) {       // the tokens' epilogues are spread over the warps
    float sr = red[(0 * kTT + t) * outs + lane], si = red[(1 * kTT + t) * outs + lane];
#pragma unroll
    for (int q = 1; q < kQuarters; ++q) {
      sr += red[((q * 2 + 0) * kTT + t) * outs + lane];
      si += red[((q * 2 + 1) * kTT + t) * outs + lane];
    }
    const int64_t i = static_cast<int64_t>(t0 + t) * C + c;
    const float rg = 1.0f / (1.0f + expf(-(sr + rb)));
    const float ig = 1.0f / (1.0f + expf(-(si + ib)));
    const float log_a = -8.0f * rg * softplus;
    a_out[i] = expf(log_a);
    d_out[i] = sqrtf(-expm1f(2.0f * log_a)) * (ig * us[j * kTT + t]);
    y_out[i] = gelu_tanh(folded(proj.p + static_cast<int64_t>(t0 + t) * 2 * C + c, proj.n_partials, proj.stride) + yb);
  }
}

// A thread owns a channel of one entry and walks its tokens. The tokens' a, d and y reach shared memory in chunks of kScanChunk tokens
// by asynchronous copies, a chunk ahead of the one being walked, so that what a step of the walk waits for is one fused
// multiply-add and a read of shared memory.
constexpr int kScanChannels = 64, kScanChunk = 32;

__device__ __forceinline__ void copy_async4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(dst))), "l"(src) : "memory");
}

template <class TW, class TO>
__global__ void __launch_bounds__(kScanChannels) rglru_scan_kernel(const float* __restrict__ a, const float* __restrict__ d, const float* __restrict__ y,
                                                                    Proj proj, const TW* __restrict__ x_bias, const int32_t* __restrict__ meta,
                                                                    int meta_stride, float* __restrict__ state, TO* __restrict__ out, int C, int K) {
  __shared__ float stage[2][3][kScanChunk][kScanChannels];
  sb::grid_launch_dependents();
  const int e = blockIdx.x, c = blockIdx.y * kScanChannels + threadIdx.x;
  const int slot = meta[e], row0 = meta[meta_stride + e], len = meta[2 * meta_stride + e], pos0 = meta[3 * meta_stride + e];
  const bool live = c < C;
  sb::grid_dependency_wait();
  float* rec = state + static_cast<int64_t>(slot) * K * C + c;
  float S = (live && pos0 > 0) ? rec[static_cast<int64_t>(K - 1) * C] : 0.0f;
  const int64_t base = static_cast<int64_t>(row0) * C + c;
  // a thread copies its own channel's values, so no other thread waits for them
  auto request = [&](int chunk) {
    const int buf = chunk & 1, nt = min(kScanChunk, len - chunk * kScanChunk);
    if (live)
      for (int t = 0; t < nt; ++t) {
        const int64_t i = base + static_cast<int64_t>(chunk * kScanChunk + t) * C;
        copy_async4(&stage[buf][0][t][threadIdx.x], a + i);
        copy_async4(&stage[buf][1][t][threadIdx.x], d + i);
        copy_async4(&stage[buf][2][t][threadIdx.x], y + i);
      }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  const int chunks = (len + kScanChunk - 1) / kScanChunk;
  request(0);
  for (int chunk = 0; chunk < chunks; ++chunk) {
    if (chunk + 1 < chunks) {
      request(chunk + 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    const int buf = chunk & 1, nt = min(kScanChunk, len - chunk * kScanChunk);
    if (live) {
#pragma unroll 8
      for (int t = 0; t < nt; ++t) {
        S = fmaf(stage[buf][0][t][threadIdx.x], S, stage[buf][1][t][threadIdx.x]);
        out[base + static_cast<int64_t>(chunk * kScanChunk + t) * C] = sb::narrow<TO>(S * stage[buf][2][t][threadIdx.x]);
      }
    }
  }
  if (!live) return;
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

// gate_w [blocks][bw][2 bw] (float32 or bfloat16): per block the matrices of r and i side by side, transposed ([input][output]).
SB_EXPORT int sb_rglru_gates(const void* gate_w, int gate_dtype, const void* r_bias, const void* i_bias, const void* lam, const void* y_bias, int w_dtype,
                             const float* u, const float* proj, int n_partials, int64_t partial_stride, float* a, float* d, float* y, int n, int C,
                             int blocks, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (blocks <= 0 || C % blocks != 0) return sb::fail("sb_rglru_gates: %d channels do not divide into %d blocks", C, blocks);
  const int bw = C / blocks;
  if (bw > 2048) return sb::fail("sb_rglru_gates: blocks of %d channels (at most 2048)", bw);
  if (w_dtype != 0) return sb::fail("sb_rglru_gates: biases and lam are float32");
  const Proj pr{proj, n_partials, partial_stride};
  const int outs = bw >= kGateOutputs ? kGateOutputs : (bw + 31) / 32 * 32;
  const dim3 grid((n + kTT - 1) / kTT, blocks, (bw + outs - 1) / outs), block(outs * kQuarters);
  const size_t smem = sizeof(float) * (kTT * bw + kQuarters * 2 * kTT * outs);
#define SB_GATES(TG)                                                                                                                            \
  do {                                                                                                                                          \
    if (smem > 48 * 1024) cudaFuncSetAttribute(rglru_gates_kernel<TG, float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);           \
    sb::launch_pdl(rglru_gates_kernel<TG, float>, grid, block, smem, stream, static_cast<const TG*>(gate_w), static_cast<const float*>(r_bias), \
                   static_cast<const float*>(i_bias), static_cast<const float*>(lam), u, pr, static_cast<const float*>(y_bias), a, d, y, n, C, bw); \
  } while (0)
  if (gate_dtype == 0) SB_GATES(float);
  else if (gate_dtype == 1) SB_GATES(bf16);
  else return sb::fail("sb_rglru_gates: unsupported dtype %d", gate_dtype);
#undef SB_GATES
  return sb::check_launch("sb_rglru_gates");
}

SB_EXPORT int sb_rglru_scan(const float* a, const float* d, const float* y, const float* proj, int n_partials, int64_t partial_stride,
                            const void* x_bias, int w_dtype, const int32_t* meta, int meta_stride, int entries, float* state, void* out,
                            int out_dtype, int C, int K, cudaStream_t stream) {
  if (entries <= 0) return 0;
  if (K < 1 || K > kMaxTaps) return sb::fail("sb_rglru_scan: %d taps (1 to %d)", K, kMaxTaps);
  const Proj pr{proj, n_partials, partial_stride};
  const dim3 grid(entries, (C + kScanChannels - 1) / kScanChannels);
#define SB_SCAN(TW, TO) sb::launch_pdl(rglru_scan_kernel<TW, TO>, grid, dim3(kScanChannels), 0, stream, a, d, y, pr, static_cast<const TW*>(x_bias), meta, meta_stride, state, static_cast<TO*>(out), C, K)
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

// i: 0 gate weights, 1 their dtype, 2 r bias, 3 i bias, 4 lam, 5 y bias, 6 their dtype, 7 u, 8 projection partial sums, 9 K ranges S,
//    10 most tokens with a buffer per range, 11 a, 12 d, 13 y, 14 C, 15 blocks
SB_EXPORT int sb_op_rglru_gates(const SbOp* op, const SbStep* s, void* stream) {
  using namespace sbstep;
  if (s->n <= 0) return SB_OP_SKIPPED;
  const int C = (int)op->i[14];
  return sb_rglru_gates(ptr<const void>(op->i[0]), (int)op->i[1], ptr<const void>(op->i[2]), ptr<const void>(op->i[3]), ptr<const void>(op->i[4]),
                        ptr<const void>(op->i[5]), (int)op->i[6], ptr<const float>(op->i[7]), ptr<const float>(op->i[8]),
                        partial_count(op->i[9], op->i[10], s->n), static_cast<int64_t>(s->n) * 2 * C, ptr<float>(op->i[11]), ptr<float>(op->i[12]),
                        ptr<float>(op->i[13]), s->n, C, (int)op->i[15], static_cast<cudaStream_t>(stream));
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
