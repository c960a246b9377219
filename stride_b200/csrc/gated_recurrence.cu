// Linear attention with a gate per key channel and token, as a recurrence over a state kept per request:
//
//   S_t = diag(g_t) S_(t-1) + k_t v_t^T        S: [D, V] float32 per head, g_t and k_t: [D]
//   o_t = S_t^T q_t
//
// The kernel takes q, g, k, v as columns of one float32 row per token, so whatever makes them is a kernel in front.
// HGRN2 is one such maker (`hgrn2_activate_kernel`): q = silu(W_q x), g = l + (1 - l) sigmoid(W_f x + b) with a lower
// bound l per channel, k = 1 - g (the gate's complement is the key: what a channel does not keep, it takes in), v = W_v x.
// Everything here is 32-bit. A CTA owns (request of the step, head, 32 value columns) and walks the request's tokens of
// this step in order with the state in registers; it reads the state the step before left (or starts from zero at
// position 0) and writes it back at the end. The D sums of an output are cut into parts of 16 consecutive elements, each
// one chain of fused multiply-adds in ascending order, and the parts are added in ascending order; neither depends on the
// step, so a token's output has the same bits in a prompt, in a portion and decoded alone.
//
// `group_rmsnorm_kernel` is what follows: every head's output RMS-normed on its own with one gain vector for all heads.
#include "common.cuh"
#include "step_ops.h"

SB_DEFINE_LAST_ERROR()

namespace {

using bf16 = __nv_bfloat16;
constexpr int kInFlight = 8;
constexpr int R = 16;        // elements of a state column a thread holds
constexpr int kChunk = 16;   // tokens staged in shared memory at a time

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

// proj [P][n][2 HD + HV]: columns q | f | v. act [n][3 HD + HV]: columns q | g | k | v.
template <class TW>
__global__ void hgrn2_activate_kernel(const float* __restrict__ proj, int n_partials, int64_t partial_stride, const TW* __restrict__ f_bias,
                                      const TW* __restrict__ lower, float* __restrict__ act, int n, int HD, int HV) {
  sb::grid_launch_dependents();
  sb::grid_dependency_wait();
  const int in_w = 2 * HD + HV, out_w = 3 * HD + HV;
  const int64_t total = static_cast<int64_t>(n) * in_w;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / in_w;
    const int j = static_cast<int>(i % in_w);
    const float z = folded(proj + i, n_partials, partial_stride);
    float* row = act + r * out_w;
    if (j < HD) {
      row[j] = z / (1.0f + expf(-z));
    } else if (j < 2 * HD) {
      const int c = j - HD;
      const float l = sb::widen(lower[c]);
      const float s = 1.0f / (1.0f + expf(-(z + sb::widen(f_bias[c]))));
      const float g = fmaf(1.0f - l, s, l);
      row[HD + c] = g;
      row[2 * HD + c] = 1.0f - g;
    } else {
      row[3 * HD + (j - 2 * HD)] = z;
    }
  }
}

struct ScanParams {
  const float* act;         // [n][width]
  int width;
  int q_off, g_off, k_off, v_off;
  const int32_t* meta;      // [4][meta_stride]: slot, first row, length, first position of every entry
  int meta_stride;
  float* state;             // [slots][H][D][V]
  float* out;               // [n][H V]
  int H, D, V;
};

__device__ __forceinline__ void copy_async4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(dst))), "l"(src) : "memory");
}
__device__ __forceinline__ void copy_async16(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(dst))), "l"(src) : "memory");
}

// The q, g, k rows and the CTA's 32 value columns of a chunk of kChunk tokens reach shared memory by asynchronous copies, a chunk
// ahead of the one being walked (two staging buffers). VEC = 4: every size and offset is a multiple of four floats, 16 bytes a copy.
template <int VEC>
__global__ void __launch_bounds__(512) gated_scan_kernel(const ScanParams p) {
  extern __shared__ __align__(16) float smem[];
  sb::grid_launch_dependents();
  const int e = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * 32;
  const int parts = blockDim.x >> 5, Dp = parts * R;
  const int part = threadIdx.x >> 5, cl = threadIdx.x & 31;
  const int stage = kChunk * (3 * Dp + 32);       // floats of a staging buffer: q, g, k [kChunk][Dp], v [kChunk][32]
  float* so = smem + 2 * stage;                    // [parts][kChunk][32]
  const int slot = p.meta[e], row0 = p.meta[p.meta_stride + e], len = p.meta[2 * p.meta_stride + e], pos0 = p.meta[3 * p.meta_stride + e];
  const bool live = c0 + cl < p.V;
  const int vn = min(32, p.V - c0);
  const int dn = min(R, p.D - part * R);
  float* st = p.state + ((static_cast<int64_t>(slot) * p.H + h) * p.D + part * R) * p.V + c0 + cl;
  // nothing copies into the cells beyond D and beyond the CTA's existing columns: they are zero for good
  if (Dp != p.D || vn != 32)
    for (int i = threadIdx.x; i < 2 * stage; i += blockDim.x) smem[i] = 0.0f;
  sb::grid_dependency_wait();
  __syncthreads();
  float S[R];
#pragma unroll
  for (int i = 0; i < R; ++i) S[i] = (pos0 > 0 && live && i < dn) ? st[static_cast<int64_t>(i) * p.V] : 0.0f;
  const int du = p.D / VEC, vu = vn / VEC, per_token = 3 * du + vu;
  auto request = [&](int chunk) {
    float* sq = smem + (chunk & 1) * stage;
    const int nt = min(kChunk, len - chunk * kChunk);
    for (int i = threadIdx.x; i < nt * per_token; i += blockDim.x) {
      const int t = i / per_token, j = i % per_token;
      const float* src = p.act + static_cast<int64_t>(row0 + chunk * kChunk + t) * p.width;
      float* dst;
      if (j < 3 * du) {
        const int which = j / du, u = j % du;
        src += (which == 0 ? p.q_off : which == 1 ? p.g_off : p.k_off) + h * p.D + u * VEC;
        dst = sq + which * kChunk * Dp + t * Dp + u * VEC;
      } else {
        const int u = j - 3 * du;
        src += p.v_off + h * p.V + c0 + u * VEC;
        dst = sq + 3 * kChunk * Dp + t * 32 + u * VEC;
      }
      if (VEC == 4) copy_async16(dst, src);
      else copy_async4(dst, src);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  const int chunks = (len + kChunk - 1) / kChunk;
  request(0);
  for (int chunk = 0; chunk < chunks; ++chunk) {
    if (chunk + 1 < chunks) {
      request(chunk + 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const int nt = min(kChunk, len - chunk * kChunk);
    const float* sq = smem + (chunk & 1) * stage;
    const float* sg = sq + kChunk * Dp;
    const float* sk = sg + kChunk * Dp;
    const float* sv = sk + kChunk * Dp;
    for (int t = 0; t < nt; ++t) {
      const float4* q4 = reinterpret_cast<const float4*>(sq + t * Dp + part * R);
      const float4* g4 = reinterpret_cast<const float4*>(sg + t * Dp + part * R);
      const float4* k4 = reinterpret_cast<const float4*>(sk + t * Dp + part * R);
      const float x = sv[t * 32 + cl];
      float acc = 0.0f;
#pragma unroll
      for (int i = 0; i < R / 4; ++i) {
        const float4 q = q4[i], g = g4[i], k = k4[i];
        S[4 * i] = fmaf(g.x, S[4 * i], __fmul_rn(k.x, x));
        acc = fmaf(S[4 * i], q.x, acc);
        S[4 * i + 1] = fmaf(g.y, S[4 * i + 1], __fmul_rn(k.y, x));
        acc = fmaf(S[4 * i + 1], q.y, acc);
        S[4 * i + 2] = fmaf(g.z, S[4 * i + 2], __fmul_rn(k.z, x));
        acc = fmaf(S[4 * i + 2], q.z, acc);
        S[4 * i + 3] = fmaf(g.w, S[4 * i + 3], __fmul_rn(k.w, x));
        acc = fmaf(S[4 * i + 3], q.w, acc);
      }
      so[(part * kChunk + t) * 32 + cl] = acc;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < nt * 32; idx += blockDim.x) {
      const int t = idx >> 5, c = idx & 31;
      if (c0 + c < p.V) {
        float sum = so[t * 32 + c];
        for (int q = 1; q < parts; ++q) sum += so[(q * kChunk + t) * 32 + c];
        p.out[static_cast<int64_t>(row0 + chunk * kChunk + t) * p.H * p.V + h * p.V + c0 + c] = sum;
      }
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < R; ++i)
      if (i < dn) st[static_cast<int64_t>(i) * p.V] = S[i];
  }
}

// out[r, h V + j] = o[r, h V + j] / sqrt(mean_j(o[r, h V + :]^2) + eps) * gain[j]: a warp per (row, head).
template <class TW, class TO>
__global__ void group_rmsnorm_kernel(const float* __restrict__ o, const TW* __restrict__ gain, TO* __restrict__ out, int64_t groups, int V, float eps) {
  sb::grid_launch_dependents();
  sb::grid_dependency_wait();
  const int64_t gidx = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (gidx >= groups) return;
  const float* src = o + gidx * V;
  float ss = 0.0f;
  for (int j = lane; j < V; j += 32) ss = fmaf(src[j], src[j], ss);
  for (int s = 16; s > 0; s >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, s);
  const float scale = 1.0f / sqrtf(ss / static_cast<float>(V) + eps);
  for (int j = lane; j < V; j += 32) out[gidx * V + j] = sb::narrow<TO>(src[j] * scale * sb::widen(gain[j]));
}

inline int grid_for(int64_t total) {
  const int64_t blocks = (total + 255) / 256, most = static_cast<int64_t>(sb::sm_count()) * 16;
  return static_cast<int>(blocks < most ? blocks : most);
}

}  // namespace

SB_EXPORT int sb_hgrn2_activate(const float* proj, int n_partials, int64_t partial_stride, const void* f_bias, const void* lower, int w_dtype,
                                float* act, int n, int HD, int HV, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (n_partials < 1) return sb::fail("sb_hgrn2_activate: n_partials must be >= 1");
  const int64_t total = static_cast<int64_t>(n) * (2 * HD + HV);
  if (w_dtype == 0)
    sb::launch_pdl(hgrn2_activate_kernel<float>, dim3(grid_for(total)), dim3(256), 0, stream, proj, n_partials, partial_stride,
                   static_cast<const float*>(f_bias), static_cast<const float*>(lower), act, n, HD, HV);
  else if (w_dtype == 1)
    sb::launch_pdl(hgrn2_activate_kernel<bf16>, dim3(grid_for(total)), dim3(256), 0, stream, proj, n_partials, partial_stride,
                   static_cast<const bf16*>(f_bias), static_cast<const bf16*>(lower), act, n, HD, HV);
  else
    return sb::fail("sb_hgrn2_activate: unsupported dtype %d", w_dtype);
  return sb::check_launch("sb_hgrn2_activate");
}

SB_EXPORT int sb_gated_scan(const float* act, int width, int q_off, int g_off, int k_off, int v_off, const int32_t* meta, int meta_stride,
                            int entries, float* state, float* out, int H, int D, int V, cudaStream_t stream) {
  if (entries <= 0) return 0;
  if (H <= 0 || D <= 0 || V <= 0 || D > 256) return sb::fail("sb_gated_scan: heads %d, key size %d (at most 256), value size %d", H, D, V);
  const int parts = (D + R - 1) / R, Dp = parts * R;
  ScanParams p{act, width, q_off, g_off, k_off, v_off, meta, meta_stride, state, out, H, D, V};
  const size_t smem = sizeof(float) * (static_cast<size_t>(2) * kChunk * (3 * Dp + 32) + static_cast<size_t>(parts) * kChunk * 32);
  if (smem > 200 * 1024) return sb::fail("sb_gated_scan: key size %d does not fit shared memory", D);
  const bool vec = D % 4 == 0 && V % 4 == 0 && width % 4 == 0 && q_off % 4 == 0 && g_off % 4 == 0 && k_off % 4 == 0 && v_off % 4 == 0 &&
                   (reinterpret_cast<uintptr_t>(act) & 15) == 0;
  static sb::DeviceOnce once;
  if (once.needed()) {
    cudaFuncSetAttribute(gated_scan_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    cudaFuncSetAttribute(gated_scan_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    once.done();
  }
  if (vec) sb::launch_pdl(gated_scan_kernel<4>, dim3(entries, H, (V + 31) / 32), dim3(parts * 32), smem, stream, p);
  else sb::launch_pdl(gated_scan_kernel<1>, dim3(entries, H, (V + 31) / 32), dim3(parts * 32), smem, stream, p);
  return sb::check_launch("sb_gated_scan");
}

SB_EXPORT int sb_group_rmsnorm(const float* o, const void* gain, int gain_dtype, void* out, int out_dtype, int n, int H, int V, float eps,
                               cudaStream_t stream) {
  if (n <= 0) return 0;
  const int64_t groups = static_cast<int64_t>(n) * H;
  const dim3 grid(static_cast<unsigned>((groups + 7) / 8));
#define SB_GN(TW, TO) sb::launch_pdl(group_rmsnorm_kernel<TW, TO>, grid, dim3(256), 0, stream, o, static_cast<const TW*>(gain), static_cast<TO*>(out), groups, V, eps)
  if (gain_dtype == 0 && out_dtype == 0) SB_GN(float, float);
  else if (gain_dtype == 0 && out_dtype == 1) SB_GN(float, bf16);
  else if (gain_dtype == 1 && out_dtype == 0) SB_GN(bf16, float);
  else if (gain_dtype == 1 && out_dtype == 1) SB_GN(bf16, bf16);
  else return sb::fail("sb_group_rmsnorm: unsupported dtypes gain=%d out=%d", gain_dtype, out_dtype);
#undef SB_GN
  return sb::check_launch("sb_group_rmsnorm");
}

// ------------------------------------------------------------------ operations of the native step program (step_ops.h)
// i: 0 projection partial sums (flat), 1 K ranges S, 2 most tokens with a buffer per range, 3 f bias, 4 lower bound, 5 their dtype, 6 act, 7 HD, 8 HV
SB_EXPORT int sb_op_hgrn2_activate(const SbOp* op, const SbStep* s, void* stream) {
  using namespace sbstep;
  if (s->n <= 0) return SB_OP_SKIPPED;
  const int HD = (int)op->i[7], HV = (int)op->i[8];
  return sb_hgrn2_activate(ptr<const float>(op->i[0]), partial_count(op->i[1], op->i[2], s->n), static_cast<int64_t>(s->n) * (2 * HD + HV),
                           ptr<const void>(op->i[3]), ptr<const void>(op->i[4]), (int)op->i[5], ptr<float>(op->i[6]), s->n, HD, HV,
                           static_cast<cudaStream_t>(stream));
}

// i: 0 act, 1 width, 2 q_off, 3 g_off, 4 k_off, 5 v_off, 6 state, 7 out, 8 H, 9 D, 10 V
SB_EXPORT int sb_op_gated_scan(const SbOp* op, const SbStep* s, void* stream) {
  using namespace sbstep;
  if (s->n <= 0) return SB_OP_SKIPPED;
  return sb_gated_scan(ptr<const float>(op->i[0]), (int)op->i[1], (int)op->i[2], (int)op->i[3], (int)op->i[4], (int)op->i[5], entry_meta(s),
                       s->max_rows, s->entries, ptr<float>(op->i[6]), ptr<float>(op->i[7]), (int)op->i[8], (int)op->i[9], (int)op->i[10],
                       static_cast<cudaStream_t>(stream));
}

// i: 0 o, 1 gain, 2 gain dtype, 3 out, 4 out dtype, 5 H, 6 V      f: 0 eps
SB_EXPORT int sb_op_group_rmsnorm(const SbOp* op, const SbStep* s, void* stream) {
  using namespace sbstep;
  if (s->n <= 0) return SB_OP_SKIPPED;
  return sb_group_rmsnorm(ptr<const float>(op->i[0]), ptr<const void>(op->i[1]), (int)op->i[2], ptr<void>(op->i[3]), (int)op->i[4], s->n,
                          (int)op->i[5], (int)op->i[6], (float)op->f[0], static_cast<cudaStream_t>(stream));
}
