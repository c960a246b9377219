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
// D sums of an output are cut into parts of R consecutive elements, each one chain of fused multiply-adds in
// ascending order, and the parts are added in ascending order. Neither depends on the step, so a token's output
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

// blockDim.x = parts * vc: thread = (part of the D sums, value column). R elements of a state column per thread.
template <int R>
__global__ void __launch_bounds__(512) lightning_scan_kernel(const ScanParams p) {
  extern __shared__ __align__(16) float smem[];
  sb::grid_launch_dependents();
  const int e = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * p.vc;
  const int D = p.D, V = p.V, vc = p.vc;
  const int parts = (D + R - 1) / R, Dp = parts * R;
  const int part = threadIdx.x / vc, cl = threadIdx.x % vc, c = c0 + cl;
  float* sq = smem;                      // [kChunk][Dp]
  float* sk = sq + kChunk * Dp;          // [kChunk][Dp]
  float* sv = sk + kChunk * Dp;          // [kChunk][vc]
  float* so = sv + kChunk * vc;          // [parts][kChunk][vc]
  const int slot = p.meta[e], row0 = p.meta[p.meta_stride + e], len = p.meta[2 * p.meta_stride + e],
            pos0 = p.meta[3 * p.meta_stride + e];
  const float decay = p.decay[h];
  float S[R];
  float* st = p.state + ((static_cast<int64_t>(slot) * p.H + h) * D + part * R) * V + c;
  const bool live = c < V;
  sb::grid_dependency_wait();
#pragma unroll
  for (int i = 0; i < R; ++i) S[i] = (pos0 > 0 && live && part * R + i < D) ? st[static_cast<int64_t>(i) * V] : 0.0f;

  for (int t0 = 0; t0 < len; t0 += kChunk) {
    const int nt = min(kChunk, len - t0);
    __syncthreads();
    // stage silu(q), silu(k) of this head and silu(v) of this CTA's columns for nt tokens
    for (int idx = threadIdx.x; idx < nt * 2 * Dp; idx += blockDim.x) {
      const int t = idx / (2 * Dp), j = idx % (2 * Dp);
      const bool is_k = j >= Dp;
      const int d = is_k ? j - Dp : j;
      float v = 0.0f;
      if (d < D) {
        const float* src = p.proj + static_cast<int64_t>(row0 + t0 + t) * p.width + (is_k ? p.k_off : p.q_off) + h * D + d;
        v = silu(folded(src, p.n_partials, p.partial_stride));
      }
      (is_k ? sk : sq)[t * Dp + d] = v;
    }
    for (int idx = threadIdx.x; idx < nt * vc; idx += blockDim.x) {
      const int t = idx / vc, j = idx % vc;
      float v = 0.0f;
      if (c0 + j < V) {
        const float* src = p.proj + static_cast<int64_t>(row0 + t0 + t) * p.width + p.v_off + h * V + c0 + j;
        v = silu(folded(src, p.n_partials, p.partial_stride));
      }
      sv[t * vc + j] = v;
    }
    __syncthreads();
#pragma unroll 1
    for (int t = 0; t < nt; ++t) {
      const float vv = sv[t * vc + cl];
      const float4* k4 = reinterpret_cast<const float4*>(sk + t * Dp + part * R);
      const float4* q4 = reinterpret_cast<const float4*>(sq + t * Dp + part * R);
      float acc = 0.0f;
#pragma unroll
      for (int i = 0; i < R / 4; ++i) {
        const float4 kk = k4[i], qq = q4[i];
        S[4 * i + 0] = fmaf(decay, S[4 * i + 0], kk.x * vv);
        acc = fmaf(S[4 * i + 0], qq.x, acc);
        S[4 * i + 1] = fmaf(decay, S[4 * i + 1], kk.y * vv);
        acc = fmaf(S[4 * i + 1], qq.y, acc);
        S[4 * i + 2] = fmaf(decay, S[4 * i + 2], kk.z * vv);
        acc = fmaf(S[4 * i + 2], qq.z, acc);
        S[4 * i + 3] = fmaf(decay, S[4 * i + 3], kk.w * vv);
        acc = fmaf(S[4 * i + 3], qq.w, acc);
      }
      so[(part * kChunk + t) * vc + cl] = acc;
    }
    __syncthreads();
    // the parts of every output, added in ascending order
    for (int idx = threadIdx.x; idx < nt * vc; idx += blockDim.x) {
      const int t = idx / vc, j = idx % vc;
      if (c0 + j < V) {
        float sum = so[t * vc + j];
        for (int q = 1; q < parts; ++q) sum += so[(q * kChunk + t) * vc + j];
        p.out[static_cast<int64_t>(row0 + t0 + t) * p.H * V + h * V + c0 + j] = sum;
      }
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < R; ++i)
      if (part * R + i < D) st[static_cast<int64_t>(i) * V] = S[i];
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
SB_EXPORT int sb_lightning_scan(const float* proj, int n_partials, int64_t partial_stride, int width, int q_off, int k_off, int v_off,
                                const int32_t* meta, int meta_stride, int entries, const float* decay, float* state, float* out,
                                int H, int D, int V, cudaStream_t stream) {
  if (entries <= 0) return 0;
  if (H <= 0 || D <= 0 || V <= 0 || D > 512) return sb::fail("sb_lightning_scan: heads %d, key size %d (at most 512), value size %d", H, D, V);
  if (n_partials < 1) return sb::fail("sb_lightning_scan: n_partials must be >= 1");
  const int R = D <= 64 ? 16 : 32;
  const int parts = (D + R - 1) / R, Dp = parts * R;
  // value columns a CTA: whole warps, at most 512 threads, and as few CTAs as still fill the device
  const int v_warps = (V + 31) / 32;
  int vw = min(min(v_warps, 512 / (32 * parts)), 4);
  const long long sms = sb::sm_count();
  while (vw > 1 && static_cast<long long>(entries) * H * ((v_warps + vw - 1) / vw) < 2 * sms) --vw;
  ScanParams p{proj, n_partials, partial_stride, width, q_off, k_off, v_off, meta, meta_stride, decay, state, out, H, D, V, 32 * vw};
  const dim3 grid(entries, H, (v_warps + vw - 1) / vw);
  const int threads = parts * 32 * vw;
  const size_t smem = sizeof(float) * (static_cast<size_t>(2) * kChunk * Dp + static_cast<size_t>(kChunk) * p.vc * (1 + parts));
  if (smem > 200 * 1024) return sb::fail("sb_lightning_scan: key size %d does not fit shared memory", D);
  if (R == 16) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(lightning_scan_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    sb::launch_pdl(lightning_scan_kernel<16>, grid, dim3(threads), smem, stream, p);
  } else {
    if (smem > 48 * 1024) cudaFuncSetAttribute(lightning_scan_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    sb::launch_pdl(lightning_scan_kernel<32>, grid, dim3(threads), smem, stream, p);
  }
  return sb::check_launch("sb_lightning_scan");
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
//    6 v_off, 7 decay (float32 [H]), 8 state, 9 out (float32 [n, H V]), 10 H, 11 D, 12 V
SB_EXPORT int sb_op_lightning_scan(const SbOp* op, const SbStep* s, void* stream) {
  using namespace sbstep;
  if (s->n <= 0) return SB_OP_SKIPPED;
  const int P = partial_count(op->i[2], op->i[3], s->n);
  return sb_lightning_scan(ptr<const float>(op->i[0]), P, static_cast<int64_t>(s->n) * op->i[1], (int)op->i[1], (int)op->i[4], (int)op->i[5],
                           (int)op->i[6], entry_meta(s), s->max_rows, s->entries, ptr<const float>(op->i[7]), ptr<float>(op->i[8]),
                           ptr<float>(op->i[9]), (int)op->i[10], (int)op->i[11], (int)op->i[12], static_cast<cudaStream_t>(stream));
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
