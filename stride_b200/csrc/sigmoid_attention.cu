// Attention without softmax: every visible key j of query i gets the weight sigmoid(scale * (q_i . k_j) + bias_head) on
// its own, and the weights are not normalised over the keys:
//
//   o_i = sum over j with 0 <= i - j < window (or j <= i without a window) of sigmoid(scale q_i.k_j + bias_h) v_j
//
// over the paged cache, grouped heads (query head h reads key/value head h / (H / G)), a key size D and a value size Dv
// that may differ (a page row holds max(D, Dv) elements for either). Scores, weights and sums are 32-bit whatever the
// storage. The sum over the keys of a query is cut by ABSOLUTE key position: key j belongs to class j % 4 (a warp), a
// class is one chain of fused multiply-adds in ascending j, and the classes are added in ascending order, so a token's
// result has the same bits in a prompt, in a portion and decoded alone.
//
// `qkv_rotate_append_kernel` is what runs in front: it adds the projection's K-range partial sums, rotates the first
// `rotary_dim` elements of every query and key head (pairs d, d + rotary_dim / 2), stores q and appends k and v to
// the request's pages.
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

struct AppendParams {
  const float* qkv;          // [P][n][Hq D + Hkv D + Hkv Dv]
  int n_partials;
  int64_t partial_stride;
  const int32_t* positions;
  const int32_t* slots;
  const float* cos_sin;      // [positions][rotary_dim / 2][2]
  int rotary_dim;
  void* q_out;               // [n][Hq D]
  void* pages;               // [pages][2][Hkv][page_size][Dc]
  const int32_t* block_table;
  int max_pages, page_size;
  int64_t page_stride, v_offset, head_stride;
  int Hq, Hkv, D, Dv, Dc;
  int write_kv;
};

template <class TQ, class TKV>
__global__ void qkv_rotate_append_kernel(AppendParams p) {
  sb::grid_launch_dependents();
  const int row = blockIdx.x;
  const int nq = p.Hq * p.D, nk = p.Hkv * p.D, width = nq + nk + p.Hkv * p.Dv;
  const int item = blockIdx.y * blockDim.x + threadIdx.x;
  const int pos = p.positions[row], slot = p.slots[row];
  int page = 0;
  if (p.write_kv && item >= nq && item < width) page = p.block_table[static_cast<int64_t>(slot) * p.max_pages + pos / p.page_size];
  sb::grid_dependency_wait();
  if (item >= width) return;
  const float* src = p.qkv + static_cast<int64_t>(row) * width;
  float a = folded(src + item, p.n_partials, p.partial_stride);
  const int rh = p.rotary_dim / 2;
  if (item < nq + nk) {
    const int d = item % p.D;
    if (d < p.rotary_dim) {
      const bool low = d < rh;
      const int j = low ? d : d - rh;
      const float b = folded(src + (low ? item + rh : item - rh), p.n_partials, p.partial_stride);
      const float2 cs = *reinterpret_cast<const float2*>(p.cos_sin + (static_cast<int64_t>(pos) * rh + j) * 2);
      // (u, v) -> (u cos - v sin, v cos + u sin): the low element is u, the high one v
      a = low ? __fsub_rn(__fmul_rn(a, cs.x), __fmul_rn(b, cs.y)) : __fadd_rn(__fmul_rn(a, cs.x), __fmul_rn(b, cs.y));
    }
  }
  if (item < nq) {
    static_cast<TQ*>(p.q_out)[static_cast<int64_t>(row) * nq + item] = sb::narrow<TQ>(a);
  } else if (p.write_kv) {
    const bool is_v = item >= nq + nk;
    const int e = is_v ? item - nq - nk : item - nq;
    const int dim = is_v ? p.Dv : p.D, head = e / dim, d = e % dim;
    TKV* dst = static_cast<TKV*>(p.pages) + static_cast<int64_t>(page) * p.page_stride + (is_v ? p.v_offset : 0) +
               static_cast<int64_t>(head) * p.head_stride + static_cast<int64_t>(pos % p.page_size) * p.Dc + d;
    *dst = sb::narrow<TKV>(a);
  }
}

struct AttnParams {
  const void* q;             // [n][H D]
  void* out;                 // [n][H Dv]
  const void* pages;
  const int32_t* block_table;
  int max_pages, page_size;
  int64_t page_stride, v_offset, head_stride;
  const int32_t* positions;
  const int32_t* slots;
  const float* bias;         // [H] float32, or null
  int H, G, D, Dv, Dc;
  int window;
  float scale;
};

constexpr int kWarps = 4;
constexpr int kMaxPer = 8;    // elements of a key or value row a lane holds: head sizes up to 256

// One block per (token, head), a warp per class of keys.
template <class T>
__global__ void __launch_bounds__(kWarps * 32) sigmoid_attention_kernel(AttnParams p) {
  extern __shared__ __align__(16) float smem[];       // q [D], then the classes' sums [kWarps][Dv]
  sb::grid_launch_dependents();
  const int row = blockIdx.x, h = blockIdx.y, g = h / (p.H / p.G);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pos = p.positions[row], slot = p.slots[row];
  const int first = p.window > 0 ? max(0, pos - p.window + 1) : 0;
  const float bias = p.bias != nullptr ? p.bias[h] : 0.0f;
  const int32_t* table = p.block_table + static_cast<int64_t>(slot) * p.max_pages;
  float* sq = smem;
  float* sums = smem + p.D;
  sb::grid_dependency_wait();
  const T* q = static_cast<const T*>(p.q) + (static_cast<int64_t>(row) * p.H + h) * p.D;
  for (int d = threadIdx.x; d < p.D; d += blockDim.x) sq[d] = sb::widen(q[d]);
  __syncthreads();
  float qr[kMaxPer], acc[kMaxPer];
#pragma unroll
  for (int i = 0; i < kMaxPer; ++i) {
    qr[i] = lane + 32 * i < p.D ? sq[lane + 32 * i] : 0.0f;
    acc[i] = 0.0f;
  }
  const T* base = static_cast<const T*>(p.pages) + static_cast<int64_t>(g) * p.head_stride;
  // the first key of this warp's class at or after `first`
  int j = first + ((warp - first) % kWarps + kWarps) % kWarps;
  for (; j <= pos; j += kWarps) {
    const T* k = base + static_cast<int64_t>(table[j / p.page_size]) * p.page_stride + static_cast<int64_t>(j % p.page_size) * p.Dc;
    const T* v = k + p.v_offset;
    float dot = 0.0f, vr[kMaxPer];
#pragma unroll
    for (int i = 0; i < kMaxPer; ++i) {
      if (lane + 32 * i < p.D) dot = fmaf(qr[i], sb::widen(k[lane + 32 * i]), dot);
      vr[i] = lane + 32 * i < p.Dv ? sb::widen(v[lane + 32 * i]) : 0.0f;
    }
    for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    const float w = 1.0f / (1.0f + expf(-fmaf(dot, p.scale, bias)));
#pragma unroll
    for (int i = 0; i < kMaxPer; ++i) acc[i] = fmaf(w, vr[i], acc[i]);
  }
#pragma unroll
  for (int i = 0; i < kMaxPer; ++i)
    if (lane + 32 * i < p.Dv) sums[warp * p.Dv + lane + 32 * i] = acc[i];
  __syncthreads();
  T* out = static_cast<T*>(p.out) + (static_cast<int64_t>(row) * p.H + h) * p.Dv;
  for (int d = threadIdx.x; d < p.Dv; d += blockDim.x) {
    float total = sums[d];
    for (int c = 1; c < kWarps; ++c) total += sums[c * p.Dv + d];
    out[d] = sb::narrow<T>(total);
  }
}

}  // namespace

SB_EXPORT int sb_qkv_rotate_append(const float* qkv, int n_partials, int64_t partial_stride, const int32_t* positions, const int32_t* slots,
                                   const float* cos_sin, int rotary_dim, void* q_out, int q_dtype, void* pages, int kv_dtype,
                                   const int32_t* block_table, int max_pages, int page_size, int64_t page_stride, int64_t v_offset,
                                   int64_t head_stride, int n, int Hq, int Hkv, int D, int Dv, int Dc, int write_kv, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (rotary_dim % 2 != 0 || rotary_dim > D || rotary_dim < 0) return sb::fail("sb_qkv_rotate_append: rotary_dim %d must be even and at most the key size %d", rotary_dim, D);
  if (n_partials < 1) return sb::fail("sb_qkv_rotate_append: n_partials must be >= 1");
  if (Dc < D || Dc < Dv) return sb::fail("sb_qkv_rotate_append: a page row of %d elements holds neither a key of %d nor a value of %d", Dc, D, Dv);
  AppendParams p{qkv, n_partials, partial_stride, positions, slots, cos_sin, rotary_dim, q_out, pages, block_table, max_pages, page_size,
                 page_stride, v_offset, head_stride, Hq, Hkv, D, Dv, Dc, write_kv};
  const int width = Hq * D + Hkv * D + Hkv * Dv;
  const dim3 grid(n, (width + 255) / 256);
  if (q_dtype == 0 && kv_dtype == 0) sb::launch_pdl(qkv_rotate_append_kernel<float, float>, grid, dim3(256), 0, stream, p);
  else if (q_dtype == 1 && kv_dtype == 1) sb::launch_pdl(qkv_rotate_append_kernel<bf16, bf16>, grid, dim3(256), 0, stream, p);
  else return sb::fail("sb_qkv_rotate_append: q and cache must both be float32 or both bfloat16");
  return sb::check_launch("sb_qkv_rotate_append");
}

SB_EXPORT int sb_sigmoid_attention(const void* q, void* out, int dtype, const void* pages, const int32_t* block_table, int max_pages, int page_size,
                                   int64_t page_stride, int64_t v_offset, int64_t head_stride, const int32_t* positions, const int32_t* slots,
                                   const float* bias, int n, int H, int G, int D, int Dv, int Dc, int window, float scale, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (H <= 0 || G <= 0 || H % G != 0) return sb::fail("sb_sigmoid_attention: %d heads do not divide into %d key/value heads", H, G);
  if (D <= 0 || Dv <= 0 || D > 32 * kMaxPer || Dv > 32 * kMaxPer) return sb::fail("sb_sigmoid_attention: key size %d, value size %d (at most %d)", D, Dv, 32 * kMaxPer);
  AttnParams p{q, out, pages, block_table, max_pages, page_size, page_stride, v_offset, head_stride, positions, slots, bias, H, G, D, Dv, Dc, window, scale};
  const size_t smem = sizeof(float) * (D + kWarps * Dv);
  if (dtype == 0) sb::launch_pdl(sigmoid_attention_kernel<float>, dim3(n, H), dim3(kWarps * 32), smem, stream, p);
  else if (dtype == 1) sb::launch_pdl(sigmoid_attention_kernel<bf16>, dim3(n, H), dim3(kWarps * 32), smem, stream, p);
  else return sb::fail("sb_sigmoid_attention: unsupported dtype %d", dtype);
  return sb::check_launch("sb_sigmoid_attention");
}

// ------------------------------------------------------------------ operations of the native step program (step_ops.h)
// i: 0 qkv partial sums (flat), 1 K ranges S, 2 most tokens with a buffer per range, 3 cos_sin, 4 rotary_dim, 5 q out, 6 q dtype, 7 pages,
//    8 cache dtype, 9 block table, 10 max_pages, 11 page_size, 12 page_stride, 13 v_offset, 14 head_stride, 15 Hq, 16 Hkv, 17 D, 18 Dv, 19 Dc,
//    20 write_kv
SB_EXPORT int sb_op_qkv_rotate_append(const SbOp* op, const SbStep* s, void* stream) {
  using namespace sbstep;
  if (s->n <= 0) return SB_OP_SKIPPED;
  const int Hq = (int)op->i[15], Hkv = (int)op->i[16], D = (int)op->i[17], Dv = (int)op->i[18];
  const int64_t width = static_cast<int64_t>(Hq) * D + static_cast<int64_t>(Hkv) * (D + Dv);
  return sb_qkv_rotate_append(ptr<const float>(op->i[0]), partial_count(op->i[1], op->i[2], s->n), s->n * width, positions(s), slots(s),
                              ptr<const float>(op->i[3]), (int)op->i[4], ptr<void>(op->i[5]), (int)op->i[6], ptr<void>(op->i[7]), (int)op->i[8],
                              ptr<const int32_t>(op->i[9]), (int)op->i[10], (int)op->i[11], op->i[12], op->i[13], op->i[14], s->n, Hq, Hkv, D, Dv,
                              (int)op->i[19], (int)op->i[20], static_cast<cudaStream_t>(stream));
}

// i: 0 q, 1 out, 2 dtype, 3 pages, 4 block table, 5 max_pages, 6 page_size, 7 page_stride, 8 v_offset, 9 head_stride, 10 bias, 11 H, 12 G,
//    13 D, 14 Dv, 15 Dc, 16 window      f: 0 scale
SB_EXPORT int sb_op_sigmoid_attention(const SbOp* op, const SbStep* s, void* stream) {
  using namespace sbstep;
  if (s->n <= 0) return SB_OP_SKIPPED;
  return sb_sigmoid_attention(ptr<const void>(op->i[0]), ptr<void>(op->i[1]), (int)op->i[2], ptr<const void>(op->i[3]), ptr<const int32_t>(op->i[4]),
                              (int)op->i[5], (int)op->i[6], op->i[7], op->i[8], op->i[9], positions(s), slots(s), ptr<const float>(op->i[10]), s->n,
                              (int)op->i[11], (int)op->i[12], (int)op->i[13], (int)op->i[14], (int)op->i[15], (int)op->i[16], (float)op->f[0],
                              static_cast<cudaStream_t>(stream));
}
