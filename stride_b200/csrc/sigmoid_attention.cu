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

// Four consecutive elements a thread, for sizes and a rotated range that are multiples of four (so that the four and their four
// partners lie in one head, and every request is 16 bytes). Same arithmetic as qkv_rotate_append_kernel: equal bits.
__device__ __forceinline__ float4 folded4(const float* p, int n_partials, int64_t stride) {
  float4 part[kInFlight];
#pragma unroll
  for (int s = 0; s < kInFlight; ++s)
    if (s < n_partials) part[s] = *reinterpret_cast<const float4*>(p + s * stride);
  float4 sum = part[0];
#pragma unroll
  for (int s = 1; s < kInFlight; ++s)
    if (s < n_partials) sum = make_float4(sum.x + part[s].x, sum.y + part[s].y, sum.z + part[s].z, sum.w + part[s].w);
  for (int s = kInFlight; s < n_partials; ++s) {
    const float4 v = *reinterpret_cast<const float4*>(p + s * stride);
    sum = make_float4(sum.x + v.x, sum.y + v.y, sum.z + v.z, sum.w + v.w);
  }
  return sum;
}
template <class T>
__device__ __forceinline__ void store4(T* dst, float4 v);
template <>
__device__ __forceinline__ void store4<float>(float* dst, float4 v) { *reinterpret_cast<float4*>(dst) = v; }
template <>
__device__ __forceinline__ void store4<bf16>(bf16* dst, float4 v) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  uint2 packed;
  packed.x = *reinterpret_cast<const uint32_t*>(&lo);
  packed.y = *reinterpret_cast<const uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(dst) = packed;
}

template <class TQ, class TKV>
__global__ void qkv_rotate_append_vec_kernel(AppendParams p) {
  sb::grid_launch_dependents();
  const int row = blockIdx.x;
  const int nq = p.Hq * p.D, nk = p.Hkv * p.D, width = nq + nk + p.Hkv * p.Dv;
  const int item = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
  const int pos = p.positions[row], slot = p.slots[row];
  int page = 0;
  if (p.write_kv && item >= nq && item < width) page = p.block_table[static_cast<int64_t>(slot) * p.max_pages + pos / p.page_size];
  sb::grid_dependency_wait();
  if (item >= width) return;
  const float* src = p.qkv + static_cast<int64_t>(row) * width;
  float4 a = folded4(src + item, p.n_partials, p.partial_stride);
  const int rh = p.rotary_dim / 2;
  if (item < nq + nk) {
    const int d = item % p.D;
    if (d < p.rotary_dim) {
      const bool low = d < rh;
      const int j = low ? d : d - rh;
      const float4 b = folded4(src + (low ? item + rh : item - rh), p.n_partials, p.partial_stride);
      const float4* cs = reinterpret_cast<const float4*>(p.cos_sin + (static_cast<int64_t>(pos) * rh + j) * 2);
      const float4 c01 = cs[0], c23 = cs[1];      // (cos, sin) of pairs j, j + 1 and j + 2, j + 3
      if (low) {
        a = make_float4(__fsub_rn(__fmul_rn(a.x, c01.x), __fmul_rn(b.x, c01.y)), __fsub_rn(__fmul_rn(a.y, c01.z), __fmul_rn(b.y, c01.w)),
                        __fsub_rn(__fmul_rn(a.z, c23.x), __fmul_rn(b.z, c23.y)), __fsub_rn(__fmul_rn(a.w, c23.z), __fmul_rn(b.w, c23.w)));
      } else {
        a = make_float4(__fadd_rn(__fmul_rn(a.x, c01.x), __fmul_rn(b.x, c01.y)), __fadd_rn(__fmul_rn(a.y, c01.z), __fmul_rn(b.y, c01.w)),
                        __fadd_rn(__fmul_rn(a.z, c23.x), __fmul_rn(b.z, c23.y)), __fadd_rn(__fmul_rn(a.w, c23.z), __fmul_rn(b.w, c23.w)));
      }
    }
  }
  if (item < nq) {
    store4<TQ>(static_cast<TQ*>(p.q_out) + static_cast<int64_t>(row) * nq + item, a);
  } else if (p.write_kv) {
    const bool is_v = item >= nq + nk;
    const int e = is_v ? item - nq - nk : item - nq;
    const int dim = is_v ? p.Dv : p.D, head = e / dim, d = e % dim;
    store4<TKV>(static_cast<TKV*>(p.pages) + static_cast<int64_t>(page) * p.page_stride + (is_v ? p.v_offset : 0) +
                    static_cast<int64_t>(head) * p.head_stride + static_cast<int64_t>(pos % p.page_size) * p.Dc + d, a);
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


// ---------------------------------------------------------------------------------------------------------------------------------
// The bfloat16 form on the tensor cores (mma.sync.m16n8k16, float32 accumulation). A CTA of four warps owns 64 rows of one
// key/value head: the 64 / Hg consecutive positions of one entry times the Hg query heads of the group, 16 rows a warp (a CTA of one
// warp: 16 rows). It walks the tiles of keys (cut by ABSOLUTE position) that any of its rows sees, in ascending order: S = Q K^T, the weights
// sigmoid(scale S + bias) in 32-bit with 0 for keys a row does not see, each weight split into two bfloat16 parts hi + lo
// (|w - hi - lo| <= 2^-17 w), O += hi V + lo V. A key that a row does not see adds exact zeros, so a row's result depends on its
// own position alone: a token has the same bits in a prompt, in a portion and decoded alone.
// Needs key sizes that are a multiple of 16 up to 256, value sizes that are a multiple of 16 up to 128 and a power of two up to 16 of
// query heads a key head; everything else takes sigmoid_attention_kernel.

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(static_cast<uint32_t>(__cvta_generic_to_shared(p))));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(static_cast<uint32_t>(__cvta_generic_to_shared(p))));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float x, float y) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(x, y);
  return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ void copy16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(dst))), "l"(src) : "memory");
}

struct TileParams {
  const bf16* q;             // [n][H D]
  bf16* out;                 // [n][H Dv]
  const bf16* pages;
  const int32_t* block_table;
  int max_pages, page_size;
  int64_t page_stride, v_offset, head_stride;
  const int32_t* meta;       // [4][meta_stride]: slot, first row, length, first position of every entry
  int meta_stride, entries;
  const float* bias;
  int H, G, D, Dv, Dc;
  int window;
  float scale;
};

// NV: value size / 16. WARPS: warps of the CTA, 16 rows each (the same instructions on the same operands for a row whatever it is, so the
// same bits). KT: keys of a staged tile (a multiple of 16; the sum over the keys is a chain over steps of 16 keys in ascending order whatever KT is).
template <int NV, int WARPS, int KT>
__global__ void __launch_bounds__(32 * WARPS, WARPS == 1 ? 8 : (NV <= 4 ? 4 : 2)) sigmoid_attention_tile_kernel(TileParams p) {
  extern __shared__ __align__(16) unsigned char raw[];
  constexpr int kRows = 16 * WARPS, NS = KT / 8, NK = KT / 16;
  static_assert(KT <= 32 * WARPS && KT % 16 == 0, "a thread per key row of a tile");
  sb::grid_launch_dependents();
  const int Hg = p.H / p.G, PT = kRows / Hg, g = blockIdx.y;
  const int ldk = p.D + 8, ldv = p.Dv + 8;                      // padded rows: ldmatrix without bank conflicts
  const bf16** rowptr = reinterpret_cast<const bf16**>(raw);    // [2][KT]: where a tile's key rows lie (null: a row nobody sees)
  bf16* Qs = reinterpret_cast<bf16*>(raw + 2 * KT * sizeof(void*));   // [kRows][ldk]
  bf16* stage0 = Qs + kRows * ldk;                              // two staging buffers of keys [KT][ldk] and values [KT][ldv]
  const int stage_elems = KT * (ldk + ldv);
  // which entry and which tile of its positions this CTA is
  int e = 0, tile = blockIdx.x, len = 0;
  for (; e < p.entries; ++e) {
    len = p.meta[2 * p.meta_stride + e];
    const int tiles = (len + PT - 1) / PT;
    if (tile < tiles) break;
    tile -= tiles;
  }
  if (e >= p.entries) return;
  const int slot = p.meta[e], row0 = p.meta[p.meta_stride + e], pos0 = p.meta[3 * p.meta_stride + e];
  const int t0 = tile * PT, nt = min(PT, len - t0);            // positions pos0 + t0 .. + nt - 1
  const int first_pos = pos0 + t0, last_pos = first_pos + nt - 1;
  const int first_key = p.window > 0 ? max(0, first_pos - p.window + 1) : 0;
  const int32_t* table = p.block_table + static_cast<int64_t>(slot) * p.max_pages;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  sb::grid_dependency_wait();
  // Q: row r = (position t0 + r / Hg, head g Hg + r % Hg); rows beyond the entry are zero
  const int dchunks = p.D / 8, vchunks = p.Dv / 8, cpr = dchunks + vchunks;
  for (int i = threadIdx.x; i < kRows * dchunks; i += blockDim.x) {
    const int r = i / dchunks, c = i % dchunks, t = r / Hg;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (t < nt) v = *reinterpret_cast<const uint4*>(p.q + (static_cast<int64_t>(row0 + t0 + t) * p.H + g * Hg + r % Hg) * p.D + c * 8);
    *reinterpret_cast<uint4*>(Qs + r * ldk + c * 8) = v;
  }
  const int r_lo = warp * 16 + (lane >> 2), r_hi = r_lo + 8;
  const int p_lo = r_lo / Hg < nt ? first_pos + r_lo / Hg : -1, p_hi = r_hi / Hg < nt ? first_pos + r_hi / Hg : -1;
  const float b_lo = p.bias != nullptr ? p.bias[g * Hg + r_lo % Hg] : 0.0f, b_hi = p.bias != nullptr ? p.bias[g * Hg + r_hi % Hg] : 0.0f;
  float o[2 * NV][4];
#pragma unroll
  for (int i = 0; i < 2 * NV; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
  const bf16* base = p.pages + static_cast<int64_t>(g) * p.head_stride;
  // the copies of a row are spread over `per_row` threads (a power of two), so that no copy costs a division
  int per_row = 1, shift = 0;
  while (per_row < cpr && per_row < 32) {
    per_row <<= 1;
    ++shift;
  }
  // a tile's keys and values are requested (asynchronous copies) while the tile before is multiplied
  auto request = [&](int kt, int buf) {
    if (threadIdx.x < KT) {
      const int j = kt * KT + threadIdx.x;
      rowptr[buf * KT + threadIdx.x] = (j >= first_key && j <= last_pos)
          ? base + static_cast<int64_t>(table[j / p.page_size]) * p.page_stride + static_cast<int64_t>(j % p.page_size) * p.Dc : nullptr;
    }
    __syncthreads();
    bf16* Ks = stage0 + buf * stage_elems;
    bf16* Vs = Ks + KT * ldk;
    for (int r = threadIdx.x >> shift; r < KT; r += blockDim.x >> shift) {
      const bf16* src = rowptr[buf * KT + r];
      for (int c = threadIdx.x & (per_row - 1); c < cpr; c += per_row) {
        const bool is_v = c >= dchunks;
        bf16* dst = is_v ? Vs + r * ldv + (c - dchunks) * 8 : Ks + r * ldk + c * 8;
        if (src != nullptr) copy16(dst, src + (is_v ? p.v_offset + (c - dchunks) * 8 : c * 8));
        else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  const int kt_first = first_key / KT, kt_last = last_pos / KT;
  request(kt_first, 0);
  for (int kt = kt_first; kt <= kt_last; ++kt) {
    const int buf = (kt - kt_first) & 1;
    if (kt < kt_last) {
      request(kt + 1, buf ^ 1);           // (the buffer of tile kt - 1: every warp left it before the barrier at the end of that tile)
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const bf16* Ks = stage0 + buf * stage_elems;
    const bf16* Vs = Ks + KT * ldk;
    // S = Q K^T for this warp's 16 rows and the tile's keys
    float s[NS][4];
#pragma unroll
    for (int i = 0; i < NS; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f;
    for (int k0 = 0; k0 < p.D; k0 += 16) {
      uint32_t a[4];
      ldmatrix_x4(a, Qs + (warp * 16 + (lane & 15)) * ldk + k0 + (lane >> 4) * 8);
#pragma unroll
      for (int n = 0; n < NS / 2; ++n) {                        // two n8 tiles of keys at a time
        uint32_t b[4];
        ldmatrix_x4(b, Ks + (n * 16 + (lane & 7) + ((lane >> 4) << 3)) * ldk + k0 + ((lane >> 3) & 1) * 8);
        mma_bf16(s[2 * n], a, b[0], b[1]);
        mma_bf16(s[2 * n + 1], a, b[2], b[3]);
      }
    }
    // the weights, split in two bfloat16 parts, as A operands of the value product
    uint32_t hi[NK][4], lo[NK][4];
#pragma unroll
    for (int n = 0; n < NS; ++n) {
      float w[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int j = kt * KT + n * 8 + (lane & 3) * 2 + (c & 1);
        const int pos = c < 2 ? p_lo : p_hi;
        const bool seen = j <= pos && (p.window <= 0 || pos - j < p.window);
        const float x = fmaf(s[n][c], p.scale, c < 2 ? b_lo : b_hi);
        w[c] = seen ? __fdividef(1.0f, 1.0f + __expf(-x)) : 0.0f;
      }
      const __nv_bfloat162 h01 = __floats2bfloat162_rn(w[0], w[1]), h23 = __floats2bfloat162_rn(w[2], w[3]);
      const int kk = n >> 1, half = (n & 1) * 2;                // tile n is columns 8 (n & 1) .. of k step n / 2
      hi[kk][half] = *reinterpret_cast<const uint32_t*>(&h01);
      hi[kk][half + 1] = *reinterpret_cast<const uint32_t*>(&h23);
      lo[kk][half] = pack_bf16(w[0] - __low2float(h01), w[1] - __high2float(h01));
      lo[kk][half + 1] = pack_bf16(w[2] - __low2float(h23), w[3] - __high2float(h23));
    }
    // O += hi V + lo V
#pragma unroll
    for (int kk = 0; kk < NK; ++kk) {
#pragma unroll
      for (int nv = 0; nv < NV; ++nv) {
        uint32_t b[4];
        ldmatrix_x4_trans(b, Vs + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ldv + nv * 16 + (lane >> 4) * 8);
        mma_bf16(o[2 * nv], hi[kk], b[0], b[1]);
        mma_bf16(o[2 * nv], lo[kk], b[0], b[1]);
        mma_bf16(o[2 * nv + 1], hi[kk], b[2], b[3]);
        mma_bf16(o[2 * nv + 1], lo[kk], b[2], b[3]);
      }
    }
    __syncthreads();                      // this tile's buffer may be written again
  }
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int r = half ? r_hi : r_lo;
    if (r / Hg >= nt) continue;
    bf16* dst = p.out + (static_cast<int64_t>(row0 + t0 + r / Hg) * p.H + g * Hg + r % Hg) * p.Dv + (lane & 3) * 2;
#pragma unroll
    for (int i = 0; i < 2 * NV; ++i)
      *reinterpret_cast<__nv_bfloat162*>(dst + i * 8) = __floats2bfloat162_rn(o[i][2 * half], o[i][2 * half + 1]);
  }
}

// Steps of decoded tokens only: an entry's Hg rows fill one 16-row tile, and the four warps of a CTA share it instead of multiplying empty
// rows. Warp w makes the scores and weights of keys 16 w .. 16 w + 15 of a tile, which are exactly the A operand of step w of the value
// product; the warps exchange these operands through shared memory, and warp w then owns the value columns 16 (w + 4 i) ..: its sums run
// over the tile's four steps in ascending order, the first part of a weight before the second. Every score, weight and sum is made by the
// instructions that make it in sigmoid_attention_tile_kernel, on the same operands in the same order: the same bits, with a quarter of
// the instructions a CTA.
template <int NV>
__global__ void __launch_bounds__(128, 4) sigmoid_attention_decode_kernel(TileParams p) {
  extern __shared__ __align__(16) unsigned char raw[];
  constexpr int KT = 64, NK = KT / 16, NVW = (NV + 3) / 4;
  sb::grid_launch_dependents();
  const int Hg = p.H / p.G, PT = 16 / Hg, g = blockIdx.y;
  const int ldk = p.D + 8, ldv = p.Dv + 8;
  const bf16** rowptr = reinterpret_cast<const bf16**>(raw);    // [2][KT]
  uint32_t* Ps = reinterpret_cast<uint32_t*>(raw + 2 * KT * sizeof(void*));   // [2 parts][NK steps][4 registers][32 lanes]
  bf16* Qs = reinterpret_cast<bf16*>(Ps + 2 * NK * 4 * 32);     // [16][ldk]
  bf16* stage0 = Qs + 16 * ldk;
  const int stage_elems = KT * (ldk + ldv);
  int e = 0, tile = blockIdx.x, len = 0;
  for (; e < p.entries; ++e) {
    len = p.meta[2 * p.meta_stride + e];
    const int tiles = (len + PT - 1) / PT;
    if (tile < tiles) break;
    tile -= tiles;
  }
  if (e >= p.entries) return;
  const int slot = p.meta[e], row0 = p.meta[p.meta_stride + e], pos0 = p.meta[3 * p.meta_stride + e];
  const int t0 = tile * PT, nt = min(PT, len - t0);
  const int first_pos = pos0 + t0, last_pos = first_pos + nt - 1;
  const int first_key = p.window > 0 ? max(0, first_pos - p.window + 1) : 0;
  const int32_t* table = p.block_table + static_cast<int64_t>(slot) * p.max_pages;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  sb::grid_dependency_wait();
  const int dchunks = p.D / 8, vchunks = p.Dv / 8, cpr = dchunks + vchunks;
  for (int i = threadIdx.x; i < 16 * dchunks; i += blockDim.x) {
    const int r = i / dchunks, c = i % dchunks, t = r / Hg;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (t < nt) v = *reinterpret_cast<const uint4*>(p.q + (static_cast<int64_t>(row0 + t0 + t) * p.H + g * Hg + r % Hg) * p.D + c * 8);
    *reinterpret_cast<uint4*>(Qs + r * ldk + c * 8) = v;
  }
  const int r_lo = lane >> 2, r_hi = r_lo + 8;
  const int p_lo = r_lo / Hg < nt ? first_pos + r_lo / Hg : -1, p_hi = r_hi / Hg < nt ? first_pos + r_hi / Hg : -1;
  const float b_lo = p.bias != nullptr ? p.bias[g * Hg + r_lo % Hg] : 0.0f, b_hi = p.bias != nullptr ? p.bias[g * Hg + r_hi % Hg] : 0.0f;
  float o[2 * NVW][4];
#pragma unroll
  for (int i = 0; i < 2 * NVW; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
  const bf16* base = p.pages + static_cast<int64_t>(g) * p.head_stride;
  int per_row = 1, shift = 0;
  while (per_row < cpr && per_row < 32) {
    per_row <<= 1;
    ++shift;
  }
  auto request = [&](int kt, int buf) {
    if (threadIdx.x < KT) {
      const int j = kt * KT + threadIdx.x;
      rowptr[buf * KT + threadIdx.x] = (j >= first_key && j <= last_pos)
          ? base + static_cast<int64_t>(table[j / p.page_size]) * p.page_stride + static_cast<int64_t>(j % p.page_size) * p.Dc : nullptr;
    }
    __syncthreads();
    bf16* Ks = stage0 + buf * stage_elems;
    bf16* Vs = Ks + KT * ldk;
    for (int r = threadIdx.x >> shift; r < KT; r += blockDim.x >> shift) {
      const bf16* src = rowptr[buf * KT + r];
      for (int c = threadIdx.x & (per_row - 1); c < cpr; c += per_row) {
        const bool is_v = c >= dchunks;
        bf16* dst = is_v ? Vs + r * ldv + (c - dchunks) * 8 : Ks + r * ldk + c * 8;
        if (src != nullptr) copy16(dst, src + (is_v ? p.v_offset + (c - dchunks) * 8 : c * 8));
        else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  const int kt_first = first_key / KT, kt_last = last_pos / KT;
  request(kt_first, 0);
  for (int kt = kt_first; kt <= kt_last; ++kt) {
    const int buf = (kt - kt_first) & 1;
    if (kt < kt_last) {
      request(kt + 1, buf ^ 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const bf16* Ks = stage0 + buf * stage_elems;
    const bf16* Vs = Ks + KT * ldk;
    // the scores of this warp's 16 keys
    float s[2][4];
#pragma unroll
    for (int i = 0; i < 2; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f;
    for (int k0 = 0; k0 < p.D; k0 += 16) {
      uint32_t a[4], b[4];
      ldmatrix_x4(a, Qs + (lane & 15) * ldk + k0 + (lane >> 4) * 8);
      ldmatrix_x4(b, Ks + (warp * 16 + (lane & 7) + ((lane >> 4) << 3)) * ldk + k0 + ((lane >> 3) & 1) * 8);
      mma_bf16(s[0], a, b[0], b[1]);
      mma_bf16(s[1], a, b[2], b[3]);
    }
    // their weights in two parts: the A operand of step `warp` of the value product, handed to the other warps
#pragma unroll
    for (int n = 0; n < 2; ++n) {
      float w[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int j = kt * KT + warp * 16 + n * 8 + (lane & 3) * 2 + (c & 1);
        const int pos = c < 2 ? p_lo : p_hi;
        const bool seen = j <= pos && (p.window <= 0 || pos - j < p.window);
        const float x = fmaf(s[n][c], p.scale, c < 2 ? b_lo : b_hi);
        w[c] = seen ? __fdividef(1.0f, 1.0f + __expf(-x)) : 0.0f;
      }
      const __nv_bfloat162 h01 = __floats2bfloat162_rn(w[0], w[1]), h23 = __floats2bfloat162_rn(w[2], w[3]);
      uint32_t* hi = Ps + ((0 * NK + warp) * 4 + n * 2) * 32 + lane;
      uint32_t* lo = Ps + ((1 * NK + warp) * 4 + n * 2) * 32 + lane;
      hi[0] = *reinterpret_cast<const uint32_t*>(&h01);
      hi[32] = *reinterpret_cast<const uint32_t*>(&h23);
      lo[0] = pack_bf16(w[0] - __low2float(h01), w[1] - __high2float(h01));
      lo[32] = pack_bf16(w[2] - __low2float(h23), w[3] - __high2float(h23));
    }
    __syncthreads();
    // O += hi V + lo V for this warp's value columns, the tile's steps in ascending order
#pragma unroll
    for (int kk = 0; kk < NK; ++kk) {
      uint32_t hi[4], lo[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        hi[i] = Ps[((0 * NK + kk) * 4 + i) * 32 + lane];
        lo[i] = Ps[((1 * NK + kk) * 4 + i) * 32 + lane];
      }
#pragma unroll
      for (int i = 0; i < NVW; ++i) {
        const int nv = warp + 4 * i;
        if (nv < NV) {
          uint32_t b[4];
          ldmatrix_x4_trans(b, Vs + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ldv + nv * 16 + (lane >> 4) * 8);
          mma_bf16(o[2 * i], hi, b[0], b[1]);
          mma_bf16(o[2 * i], lo, b[0], b[1]);
          mma_bf16(o[2 * i + 1], hi, b[2], b[3]);
          mma_bf16(o[2 * i + 1], lo, b[2], b[3]);
        }
      }
    }
    __syncthreads();                      // the tile's buffer and the exchanged operands may be written again
  }
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int r = half ? r_hi : r_lo;
    if (r / Hg >= nt) continue;
    bf16* dst = p.out + (static_cast<int64_t>(row0 + t0 + r / Hg) * p.H + g * Hg + r % Hg) * p.Dv + (lane & 3) * 2;
#pragma unroll
    for (int i = 0; i < NVW; ++i) {
      const int nv = warp + 4 * i;
      if (nv < NV) {
        *reinterpret_cast<__nv_bfloat162*>(dst + nv * 16) = __floats2bfloat162_rn(o[2 * i][2 * half], o[2 * i][2 * half + 1]);
        *reinterpret_cast<__nv_bfloat162*>(dst + nv * 16 + 8) = __floats2bfloat162_rn(o[2 * i + 1][2 * half], o[2 * i + 1][2 * half + 1]);
      }
    }
  }
}

template <int NV>
int launch_decode(const TileParams& p, int n, cudaStream_t stream) {
  const int Hg = p.H / p.G, PT = 16 / Hg;
  const size_t smem = 2 * 64 * sizeof(void*) + 2 * 4 * 4 * 32 * sizeof(uint32_t) + sizeof(bf16) * (16 * (p.D + 8) + 2 * 64 * (p.D + 8 + p.Dv + 8));
  static sb::DeviceOnce once;
  if (once.needed()) {
    cudaFuncSetAttribute(sigmoid_attention_decode_kernel<NV>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    once.done();
  }
  sb::launch_pdl(sigmoid_attention_decode_kernel<NV>, dim3((n + PT - 1) / PT + p.entries, p.G), dim3(128), smem, stream, p);
  return sb::check_launch("sb_sigmoid_attention_tiles");
}

template <int NV, int WARPS, int KT>
int launch_tiles_of(const TileParams& p, int n, cudaStream_t stream) {
  const int Hg = p.H / p.G, PT = 16 * WARPS / Hg;
  const size_t smem = 2 * KT * sizeof(void*) + sizeof(bf16) * (16 * WARPS * (p.D + 8) + 2 * KT * (p.D + 8 + p.Dv + 8));
  static sb::DeviceOnce once;
  if (once.needed()) {
    cudaFuncSetAttribute(sigmoid_attention_tile_kernel<NV, WARPS, KT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    once.done();
  }
  sb::launch_pdl(sigmoid_attention_tile_kernel<NV, WARPS, KT>, dim3((n + PT - 1) / PT + p.entries, p.G), dim3(32 * WARPS), smem, stream, p);
  return sb::check_launch("sb_sigmoid_attention_tiles");
}

// Steps with a prompt portion: CTAs of four warps with 64 rows. Steps of decoded tokens only: the four warps share one tile of 16 rows.
// (Such steps were also tried on the 64-row CTAs, whose empty rows are multiplied all the same, and on CTAs of one warp with tiles of 32
// keys: 0.111 and 0.154 ms for 64 decoded tokens over 1,024 keys; the latter are 3.5 warps an SM, each a chain of dependent copies,
// products and exponentials. All give the same bits.)
template <int NV>
int launch_tiles(const TileParams& p, int n, cudaStream_t stream) {
  return n == p.entries ? launch_decode<NV>(p, n, stream) : launch_tiles_of<NV, 4, 64>(p, n, stream);
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
  if (q_dtype != kv_dtype || (q_dtype != 0 && q_dtype != 1)) return sb::fail("sb_qkv_rotate_append: q and cache must both be float32 or both bfloat16");
  const auto aligned = [](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0; };
  const bool vec = D % 4 == 0 && Dv % 4 == 0 && Dc % 4 == 0 && rotary_dim % 8 == 0 && partial_stride % 4 == 0 && page_stride % 4 == 0 && v_offset % 4 == 0 &&
                   head_stride % 4 == 0 && aligned(qkv) && aligned(q_out) && aligned(pages) && aligned(cos_sin);
  if (vec) {
    const dim3 grid(n, (width / 4 + 127) / 128);
    if (q_dtype == 0) sb::launch_pdl(qkv_rotate_append_vec_kernel<float, float>, grid, dim3(128), 0, stream, p);
    else sb::launch_pdl(qkv_rotate_append_vec_kernel<bf16, bf16>, grid, dim3(128), 0, stream, p);
  } else {
    const dim3 grid(n, (width + 255) / 256);
    if (q_dtype == 0) sb::launch_pdl(qkv_rotate_append_kernel<float, float>, grid, dim3(256), 0, stream, p);
    else sb::launch_pdl(qkv_rotate_append_kernel<bf16, bf16>, grid, dim3(256), 0, stream, p);
  }
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

// The tensor-core form: whether it takes a shape, and the launch. Entries come from the step's records on the device (meta).
SB_EXPORT int sb_sigmoid_attention_tiles_supported(int H, int G, int D, int Dv, int Dc) {
  if (G <= 0 || H % G != 0) return 0;
  const int Hg = H / G;
  return Hg <= 16 && (Hg & (Hg - 1)) == 0 && D % 16 == 0 && D >= 16 && D <= 256 && Dv % 16 == 0 && Dv >= 16 && Dv <= 128 && Dc % 8 == 0;
}

SB_EXPORT int sb_sigmoid_attention_tiles(const void* q, void* out, const void* pages, const int32_t* block_table, int max_pages, int page_size,
                                         int64_t page_stride, int64_t v_offset, int64_t head_stride, const int32_t* meta, int meta_stride, int entries,
                                         const float* bias, int n, int H, int G, int D, int Dv, int Dc, int window, float scale, cudaStream_t stream) {
  if (n <= 0 || entries <= 0) return 0;
  if (!sb_sigmoid_attention_tiles_supported(H, G, D, Dv, Dc))
    return sb::fail("sb_sigmoid_attention_tiles: heads %d / %d, key size %d, value size %d are not a shape of the tensor-core form", H, G, D, Dv);
  TileParams p{static_cast<const bf16*>(q), static_cast<bf16*>(out), static_cast<const bf16*>(pages), block_table, max_pages, page_size, page_stride,
               v_offset, head_stride, meta, meta_stride, entries, bias, H, G, D, Dv, Dc, window, scale};
  switch (Dv / 16) {
    case 1: return launch_tiles<1>(p, n, stream);
    case 2: return launch_tiles<2>(p, n, stream);
    case 3: return launch_tiles<3>(p, n, stream);
    case 4: return launch_tiles<4>(p, n, stream);
    case 5: return launch_tiles<5>(p, n, stream);
    case 6: return launch_tiles<6>(p, n, stream);
    case 7: return launch_tiles<7>(p, n, stream);
    default: return launch_tiles<8>(p, n, stream);
  }
}

// i: 0 q, 1 out, 2 pages, 3 block table, 4 max_pages, 5 page_size, 6 page_stride, 7 v_offset, 8 head_stride, 9 bias, 10 H, 11 G, 12 D, 13 Dv,
//    14 Dc, 15 window      f: 0 scale
SB_EXPORT int sb_op_sigmoid_attention_tiles(const SbOp* op, const SbStep* s, void* stream) {
  using namespace sbstep;
  if (s->n <= 0) return SB_OP_SKIPPED;
  return sb_sigmoid_attention_tiles(ptr<const void>(op->i[0]), ptr<void>(op->i[1]), ptr<const void>(op->i[2]), ptr<const int32_t>(op->i[3]), (int)op->i[4],
                                    (int)op->i[5], op->i[6], op->i[7], op->i[8], entry_meta(s), s->max_rows, s->entries, ptr<const float>(op->i[9]), s->n,
                                    (int)op->i[10], (int)op->i[11], (int)op->i[12], (int)op->i[13], (int)op->i[14], (int)op->i[15], (float)op->f[0],
                                    static_cast<cudaStream_t>(stream));
}
