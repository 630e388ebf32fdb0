// fp32-accumulate SIMT attention kernels: forward, dQ and dK/dV for all three
// mask families, any head size up to 128, fp32 or bf16 storage.
//
// These kernels are the fp32 path (results within 1e-4 of an fp64 evaluation)
// and the path for shapes the tensor-core kernels do not take (head sizes
// other than 64, 96 and 128, gathered key lists, rows that are not 16-byte
// aligned).  One group of TPR lanes owns
// one query row (forward, dQ) or one key row (dK/dV); each lane keeps 16 of
// the row's head_dim values in registers; the opposite operand is staged in
// shared memory as fp32, a tile of 32 rows at a time, and broadcast.
//
// HBM traffic per (batch, head): Q, O once; K and V once per query tile of
// ROWS = 128/TPR rows (from L2 after the first touch).
#include <math.h>

#include "common.cuh"

namespace wm {
namespace {

constexpr int kThreads = 128;
constexpr int kTile = 32;  // rows of the staged operand per tile

struct SimtFlags {
  int vec4;  // 1 when every row pointer is aligned for 4-element vector loads
};

template <typename T>
__device__ __forceinline__ float4 load4(const T* p, int d, int D, bool vec);

template <>
__device__ __forceinline__ float4 load4<float>(const float* p, int d, int D, bool vec) {
  if (vec && d + 3 < D) return *reinterpret_cast<const float4*>(p + d);
  float4 r;
  r.x = d + 0 < D ? p[d + 0] : 0.f;
  r.y = d + 1 < D ? p[d + 1] : 0.f;
  r.z = d + 2 < D ? p[d + 2] : 0.f;
  r.w = d + 3 < D ? p[d + 3] : 0.f;
  return r;
}

template <>
__device__ __forceinline__ float4 load4<__nv_bfloat16>(const __nv_bfloat16* p, int d, int D, bool vec) {
  float4 r;
  if (vec && d + 3 < D) {
    uint2 raw = *reinterpret_cast<const uint2*>(p + d);
    __nv_bfloat162 a = *reinterpret_cast<__nv_bfloat162*>(&raw.x);
    __nv_bfloat162 b = *reinterpret_cast<__nv_bfloat162*>(&raw.y);
    r.x = __low2float(a);
    r.y = __high2float(a);
    r.z = __low2float(b);
    r.w = __high2float(b);
    return r;
  }
  r.x = d + 0 < D ? __bfloat162float(p[d + 0]) : 0.f;
  r.y = d + 1 < D ? __bfloat162float(p[d + 1]) : 0.f;
  r.z = d + 2 < D ? __bfloat162float(p[d + 2]) : 0.f;
  r.w = d + 3 < D ? __bfloat162float(p[d + 3]) : 0.f;
  return r;
}

template <typename T>
__device__ __forceinline__ void store4(T* p, int d, int D, float4 v) {
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    float x = e == 0 ? v.x : e == 1 ? v.y : e == 2 ? v.z : v.w;
    if (d + e < D) p[d + e] = from_float<T>(x);
  }
}

// Lane-private slice of a row: four groups of four consecutive dims; group t
// of lane c covers dims 4*(t*TPR+c) .. +3, so the TPR lanes of a row read
// consecutive 16-byte pieces of shared memory.
template <typename T, int TPR>
__device__ __forceinline__ void load_slice(const T* row, int c, int D, bool vec, float (&x)[16]) {
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    int d = (t * TPR + c) * 4;
    if (row != nullptr && d < D) v = load4<T>(row, d, D, vec);
    x[4 * t + 0] = v.x;
    x[4 * t + 1] = v.y;
    x[4 * t + 2] = v.z;
    x[4 * t + 3] = v.w;
  }
}

template <typename T, int TPR>
__device__ __forceinline__ void store_slice(T* row, int c, int D, const float (&x)[16]) {
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    int d = (t * TPR + c) * 4;
    if (d < D) store4<T>(row, d, D, make_float4(x[4 * t], x[4 * t + 1], x[4 * t + 2], x[4 * t + 3]));
  }
}

template <int TPR>
__device__ __forceinline__ void atomic_slice(float* row, int c, int D, const float (&x)[16]) {
#pragma unroll
  for (int t = 0; t < 4; ++t) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      int d = (t * TPR + c) * 4 + e;
      if (d < D && x[4 * t + e] != 0.f) atomicAdd(row + d, x[4 * t + e]);
    }
  }
}

template <int TPR>
__device__ __forceinline__ float dot_slice(const float (&x)[16], const float* srow, int c) {
  float acc = 0.f;
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    float4 v = *reinterpret_cast<const float4*>(srow + (t * TPR + c) * 4);
    acc = fmaf(x[4 * t + 0], v.x, acc);
    acc = fmaf(x[4 * t + 1], v.y, acc);
    acc = fmaf(x[4 * t + 2], v.z, acc);
    acc = fmaf(x[4 * t + 3], v.w, acc);
  }
  return acc;
}

template <int TPR>
__device__ __forceinline__ void axpy_slice(float (&y)[16], float alpha, const float* srow, int c) {
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    float4 v = *reinterpret_cast<const float4*>(srow + (t * TPR + c) * 4);
    y[4 * t + 0] = fmaf(alpha, v.x, y[4 * t + 0]);
    y[4 * t + 1] = fmaf(alpha, v.y, y[4 * t + 1]);
    y[4 * t + 2] = fmaf(alpha, v.z, y[4 * t + 2]);
    y[4 * t + 3] = fmaf(alpha, v.w, y[4 * t + 3]);
  }
}

template <int TPR>
__device__ __forceinline__ float group_sum(float x) {
#pragma unroll
  for (int s = TPR / 2; s > 0; s >>= 1) x += __shfl_xor_sync(0xffffffffu, x, s);
  return x;
}

// Which (group, first row) does this block work on?  Dense problems: one
// group per batch row, tiles along blockIdx.x.  Packed: a host-built table.
__device__ __forceinline__ bool locate_tile(const wm_attn_args& a, const int* table, int rows_per_tile, int& batch,
                                            int& group, int& first) {
  if (a.mask == WM_MASK_PACKED) {
    group = table[2 * blockIdx.x];
    first = table[2 * blockIdx.x + 1];
    batch = 0;
  } else {
    group = 0;
    batch = blockIdx.z;
    first = blockIdx.x * rows_per_tile;
  }
  return true;
}

// Stage `kTile` key (or value) rows j0.. of the group into shared memory as
// fp32, zero-filling rows at or beyond `limit` and rows removed by key_mask.
template <typename T, int TPR>
__device__ __forceinline__ void stage_keys(const wm_attn_args& a, const GroupCtx& g, int batch, int kv_head,
                                           const T* base, const int64_t* strides, int j0, int limit, bool vec,
                                           float* dst) {
  constexpr int DP4 = 4 * TPR;  // float4 per padded row
  for (int idx = threadIdx.x; idx < kTile * DP4; idx += kThreads) {
    int jj = idx / DP4;
    int d = (idx - jj * DP4) * 4;
    int j = j0 + jj;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (j < limit && d < a.head_dim) {
      int kb, ks;
      key_coord(a, g, batch, j, kb, ks);
      bool keep = a.key_mask == nullptr || a.key_mask[static_cast<long long>(kb) * a.k_len + ks] != 0;
      if (keep) {
        const T* row = base + kb * strides[0] + kv_head * strides[1] + ks * strides[2];
        v = load4<T>(row, d, a.head_dim, vec);
      }
    }
    *reinterpret_cast<float4*>(dst + jj * (16 * TPR) + d) = v;
  }
}

struct KeyMeta {
  int seg[kTile];
  int end[kTile];
  unsigned char keep[kTile];
};

__device__ __forceinline__ void stage_key_meta(const wm_attn_args& a, const GroupCtx& g, int batch, int j0, int limit,
                                               KeyMeta& m) {
  if (threadIdx.x < kTile) {
    int j = j0 + threadIdx.x;
    int seg = 0, end = 0x7fffffff;
    unsigned char keep = 0;
    if (j < limit) {
      int kb, ks;
      key_coord(a, g, batch, j, kb, ks);
      long long at = static_cast<long long>(kb) * a.k_len + ks;
      keep = a.key_mask == nullptr || a.key_mask[at] != 0;
      if (a.q_seg != nullptr) {
        seg = a.k_seg[at];
        end = a.k_query_end[at];
      }
    }
    m.seg[threadIdx.x] = seg;
    m.end[threadIdx.x] = end;
    m.keep[threadIdx.x] = keep;
  }
}

__device__ __forceinline__ bool pair_visible(const wm_attn_args& a, const RowBound& r, int j, const KeyMeta& m,
                                             int jj) {
  if (j >= r.hi || !m.keep[jj]) return false;
  if (a.q_seg != nullptr) return doc_visible(r, j, m.seg[jj], m.end[jj]);
  return true;
}

// Block-wide min / max of two per-thread ints.
__device__ __forceinline__ void block_min_max(int lo, int hi, int& out_lo, int& out_hi, int* scratch) {
  for (int s = 16; s > 0; s >>= 1) {
    lo = min(lo, __shfl_xor_sync(0xffffffffu, lo, s));
    hi = max(hi, __shfl_xor_sync(0xffffffffu, hi, s));
  }
  int warp = threadIdx.x >> 5;
  if ((threadIdx.x & 31) == 0) {
    scratch[2 * warp] = lo;
    scratch[2 * warp + 1] = hi;
  }
  __syncthreads();
  out_lo = scratch[0];
  out_hi = scratch[1];
  for (int w = 1; w < kThreads / 32; ++w) {
    out_lo = min(out_lo, scratch[2 * w]);
    out_hi = max(out_hi, scratch[2 * w + 1]);
  }
  __syncthreads();
}

// First key tile that the block must visit.  Document problems start at the
// smallest document start of the block's rows; the shared dummy, which the
// metadata contract places at slot 0 only, is visited as an extra tile.
__device__ __forceinline__ int first_tile(const wm_attn_args& a, int min_lo) {
  return a.q_seg != nullptr ? (min_lo / kTile) * kTile : 0;
}

// ------------------------------------------------------------------ forward
template <typename T, int TPR>
__global__ void __launch_bounds__(kThreads) attn_fwd_kernel(const wm_attn_args a, SimtFlags flags) {
  constexpr int ROWS = kThreads / TPR;
  constexpr int DP = 16 * TPR;
  __shared__ __align__(16) float ks[kTile * DP];
  __shared__ __align__(16) float vs[kTile * DP];
  __shared__ KeyMeta meta;
  __shared__ int red[2 * kThreads / 32];

  const bool vec = flags.vec4 != 0;
  const int head = blockIdx.y;
  const int kv_head = head / (a.q_heads / a.kv_heads);
  int batch, group, first;
  locate_tile(a, a.query_tiles, ROWS, batch, group, first);
  const GroupCtx g = group_ctx(a, group);
  const int r = threadIdx.x / TPR;
  const int c = threadIdx.x % TPR;
  const int i = first + r;
  const bool live = i < g.nq;

  RowBound rb;
  rb.lo = 0x7fffffff;
  rb.hi = 0;
  rb.seg = 0;
  rb.qi = i;
  int qb = 0, qt = 0;
  if (live) {
    query_coord(a, g, batch, i, qb, qt);
    rb = row_bound(a, g, qb, i);
    if (a.mask == WM_MASK_PACKED) rb.qi = i;
  }
  const T* qrow =
      live ? static_cast<const T*>(a.q) + qb * a.q_strides[0] + head * a.q_strides[1] + qt * a.q_strides[2] : nullptr;
  float q[16];
  load_slice<T, TPR>(qrow, c, a.head_dim, vec, q);
  const float sl2 = a.scale * kLog2e;
#pragma unroll
  for (int e = 0; e < 16; ++e) q[e] *= sl2;

  int min_lo, max_hi;
  block_min_max(live && rb.hi > 0 ? rb.lo : 0x7fffffff, rb.hi, min_lo, max_hi, red);

  float acc[16];
#pragma unroll
  for (int e = 0; e < 16; ++e) acc[e] = 0.f;
  float m = -INFINITY, l = 0.f;

  const int start = max_hi > 0 ? first_tile(a, min_lo) : 0;
  const bool dummy_tile = a.q_seg != nullptr && start > 0;
  // Iterate: optional dummy tile (j0 = 0), then start, start+kTile, ...
  for (int step = dummy_tile ? -1 : 0;; ++step) {
    int j0 = step < 0 ? 0 : start + step * kTile;
    if (j0 >= max_hi) break;
    __syncthreads();
    stage_keys<T, TPR>(a, g, batch, kv_head, static_cast<const T*>(a.k), a.k_strides, j0, max_hi, vec, ks);
    stage_keys<T, TPR>(a, g, batch, kv_head, static_cast<const T*>(a.v), a.v_strides, j0, max_hi, vec, vs);
    stage_key_meta(a, g, batch, j0, max_hi, meta);
    __syncthreads();
#pragma unroll 1
    for (int jc = 0; jc < kTile; jc += 8) {
      float s[8];
      float top = -INFINITY;
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        float d = group_sum<TPR>(dot_slice<TPR>(q, ks + (jc + u) * DP, c));
        bool vis = live && pair_visible(a, rb, j0 + jc + u, meta, jc + u);
        s[u] = vis ? d : -INFINITY;
        top = fmaxf(top, s[u]);
      }
      if (top == -INFINITY) continue;  // uniform inside a row group; no shuffles follow
      float m_new = fmaxf(m, top);
      float corr = exp2f(m - m_new);
      l *= corr;
#pragma unroll
      for (int e = 0; e < 16; ++e) acc[e] *= corr;
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        float p = exp2f(s[u] - m_new);
        if (s[u] != -INFINITY) {
          l += p;
          axpy_slice<TPR>(acc, p, vs + (jc + u) * DP, c);
        }
      }
      m = m_new;
    }
  }
  if (live) {
    float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
    for (int e = 0; e < 16; ++e) acc[e] *= inv;
    T* orow = static_cast<T*>(a.out) + qb * a.out_strides[0] + head * a.out_strides[1] + qt * a.out_strides[2];
    store_slice<T, TPR>(orow, c, a.head_dim, acc);
    if (c == 0 && a.lse != nullptr) {
      long long at = (static_cast<long long>(qb) * a.q_heads + head) * a.q_len + qt;
      a.lse[at] = l > 0.f ? (m + log2f(l)) * kLn2 : INFINITY;
    }
  }
}

// Rows that no schedule group lists keep the value zero (packed problems).
template <typename T>
__global__ void zero_rows_kernel(T* out, long long s0, long long s1, long long s2, int B, int H, int Tn, int D,
                                 float* lse) {
  long long total = static_cast<long long>(B) * H * Tn;
  for (long long row = blockIdx.x * static_cast<long long>(blockDim.y) + threadIdx.y; row < total;
       row += static_cast<long long>(gridDim.x) * blockDim.y) {
    int t = static_cast<int>(row % Tn);
    int h = static_cast<int>((row / Tn) % H);
    int b = static_cast<int>(row / (static_cast<long long>(Tn) * H));
    T* p = out + b * s0 + h * s1 + t * s2;
    for (int d = threadIdx.x; d < D; d += blockDim.x) p[d] = from_float<T>(0.f);
    if (lse != nullptr && threadIdx.x == 0) lse[row] = INFINITY;
  }
}

// ------------------------------------------------------------------ dQ (+ delta)
template <typename T, int TPR>
__global__ void __launch_bounds__(kThreads) attn_dq_kernel(const wm_attn_args a, SimtFlags flags, float* delta) {
  constexpr int ROWS = kThreads / TPR;
  constexpr int DP = 16 * TPR;
  __shared__ __align__(16) float ks[kTile * DP];
  __shared__ __align__(16) float vs[kTile * DP];
  __shared__ KeyMeta meta;
  __shared__ int red[2 * kThreads / 32];

  const bool vec = flags.vec4 != 0;
  const int head = blockIdx.y;
  const int kv_head = head / (a.q_heads / a.kv_heads);
  int batch, group, first;
  locate_tile(a, a.query_tiles, ROWS, batch, group, first);
  const GroupCtx g = group_ctx(a, group);
  const int r = threadIdx.x / TPR;
  const int c = threadIdx.x % TPR;
  const int i = first + r;
  const bool live = i < g.nq;

  RowBound rb;
  rb.lo = 0x7fffffff;
  rb.hi = 0;
  rb.seg = 0;
  rb.qi = i;
  int qb = 0, qt = 0;
  if (live) {
    query_coord(a, g, batch, i, qb, qt);
    rb = row_bound(a, g, qb, i);
  }
  const T* qrow = nullptr;
  const T* dorow = nullptr;
  const T* orow = nullptr;
  float lse = INFINITY;
  long long stat = 0;
  if (live) {
    qrow = static_cast<const T*>(a.q) + qb * a.q_strides[0] + head * a.q_strides[1] + qt * a.q_strides[2];
    dorow = static_cast<const T*>(a.dout) + qb * a.dout_strides[0] + head * a.dout_strides[1] + qt * a.dout_strides[2];
    orow = static_cast<const T*>(a.out) + qb * a.out_strides[0] + head * a.out_strides[1] + qt * a.out_strides[2];
    stat = (static_cast<long long>(qb) * a.q_heads + head) * a.q_len + qt;
    lse = a.lse[stat];
  }
  float q[16], go[16], dq[16];
  load_slice<T, TPR>(qrow, c, a.head_dim, vec, q);
  load_slice<T, TPR>(dorow, c, a.head_dim, vec, go);
  {
    float o[16];
    load_slice<T, TPR>(orow, c, a.head_dim, vec, o);
    float part = 0.f;
#pragma unroll
    for (int e = 0; e < 16; ++e) part = fmaf(go[e], o[e], part);
    part = group_sum<TPR>(part);
    if (live && c == 0) delta[stat] = part;
    dq[0] = part;
  }
  const float dlt = dq[0];
#pragma unroll
  for (int e = 0; e < 16; ++e) dq[e] = 0.f;
  const float sl2 = a.scale * kLog2e;
  const float lse2 = lse * kLog2e;  // +inf for empty rows: every p becomes 0

  int min_lo, max_hi;
  block_min_max(live && rb.hi > 0 ? rb.lo : 0x7fffffff, rb.hi, min_lo, max_hi, red);
  const int start = max_hi > 0 ? first_tile(a, min_lo) : 0;
  const bool dummy_tile = a.q_seg != nullptr && start > 0;
  for (int step = dummy_tile ? -1 : 0;; ++step) {
    int j0 = step < 0 ? 0 : start + step * kTile;
    if (j0 >= max_hi) break;
    __syncthreads();
    stage_keys<T, TPR>(a, g, batch, kv_head, static_cast<const T*>(a.k), a.k_strides, j0, max_hi, vec, ks);
    stage_keys<T, TPR>(a, g, batch, kv_head, static_cast<const T*>(a.v), a.v_strides, j0, max_hi, vec, vs);
    stage_key_meta(a, g, batch, j0, max_hi, meta);
    __syncthreads();
#pragma unroll 2
    for (int jj = 0; jj < kTile; ++jj) {
      float s = group_sum<TPR>(dot_slice<TPR>(q, ks + jj * DP, c));
      float dp = group_sum<TPR>(dot_slice<TPR>(go, vs + jj * DP, c));
      bool vis = live && pair_visible(a, rb, j0 + jj, meta, jj);
      if (vis) {
        float p = exp2f(s * sl2 - lse2);
        float ds = p * (dp - dlt);
        axpy_slice<TPR>(dq, ds, ks + jj * DP, c);
      }
    }
  }
  if (live) {
#pragma unroll
    for (int e = 0; e < 16; ++e) dq[e] *= a.scale;
    T* row = static_cast<T*>(a.dq) + qb * a.dq_strides[0] + head * a.dq_strides[1] + qt * a.dq_strides[2];
    store_slice<T, TPR>(row, c, a.head_dim, dq);
  }
}

// ------------------------------------------------------------------ dK / dV
// One group of TPR lanes owns one key row of one KV head and walks over the
// query heads of its group and over the query tiles that can see it.
struct QueryMeta {
  int lo[kTile];
  int hi[kTile];
  int seg[kTile];
  float lse2[kTile];
  float delta[kTile];
};

template <typename T, int TPR>
__global__ void __launch_bounds__(kThreads)
    attn_dkv_kernel(const wm_attn_args a, SimtFlags flags, const float* delta, float* dk_acc, float* dv_acc) {
  constexpr int ROWS = kThreads / TPR;
  constexpr int DP = 16 * TPR;
  __shared__ __align__(16) float qs[kTile * DP];
  __shared__ __align__(16) float gs[kTile * DP];
  __shared__ QueryMeta qm;
  __shared__ int red[2 * kThreads / 32];

  const bool vec = flags.vec4 != 0;
  const int kv_head = blockIdx.y;
  const int heads_per_kv = a.q_heads / a.kv_heads;
  int batch, group, first;
  {
    if (a.mask == WM_MASK_PACKED) {
      group = a.key_tiles[2 * blockIdx.x];
      first = a.key_tiles[2 * blockIdx.x + 1];
      batch = 0;
    } else {
      group = 0;
      batch = blockIdx.z;
      first = blockIdx.x * ROWS;
    }
  }
  const GroupCtx g = group_ctx(a, group);
  const int r = threadIdx.x / TPR;
  const int c = threadIdx.x % TPR;
  const int j = first + r;
  const bool live = j < g.nk;
  int kb = 0, kslot = 0;
  bool key_kept = false;
  int kseg = 0, kend = 0x7fffffff;
  if (live) {
    key_coord(a, g, batch, j, kb, kslot);
    long long at = static_cast<long long>(kb) * a.k_len + kslot;
    key_kept = a.key_mask == nullptr || a.key_mask[at] != 0;
    if (a.q_seg != nullptr) {
      kseg = a.k_seg[at];
      kend = a.k_query_end[at];
    }
  }
  const T* krow = live && key_kept
                      ? static_cast<const T*>(a.k) + kb * a.k_strides[0] + kv_head * a.k_strides[1] + kslot * a.k_strides[2]
                      : nullptr;
  const T* vrow = live && key_kept
                      ? static_cast<const T*>(a.v) + kb * a.v_strides[0] + kv_head * a.v_strides[1] + kslot * a.v_strides[2]
                      : nullptr;
  float kreg[16], vreg[16], dk[16], dv[16];
  load_slice<T, TPR>(krow, c, a.head_dim, vec, kreg);
  load_slice<T, TPR>(vrow, c, a.head_dim, vec, vreg);
#pragma unroll
  for (int e = 0; e < 16; ++e) dk[e] = dv[e] = 0.f;
  const float sl2 = a.scale * kLog2e;

  for (int hq = 0; hq < heads_per_kv; ++hq) {
    const int head = kv_head * heads_per_kv + hq;
    for (int i0 = 0; i0 < g.nq; i0 += kTile) {
      __syncthreads();
      // per-row bounds of this query tile
      int my_hi = 0;
      if (threadIdx.x < kTile) {
        int i = i0 + threadIdx.x;
        RowBound rb;
        rb.lo = 0;
        rb.hi = 0;
        rb.seg = 0;
        float l2 = INFINITY, dl = 0.f;
        if (i < g.nq) {
          int qb, qt;
          query_coord(a, g, batch, i, qb, qt);
          rb = row_bound(a, g, qb, i);
          long long stat = (static_cast<long long>(qb) * a.q_heads + head) * a.q_len + qt;
          l2 = a.lse[stat] * kLog2e;
          dl = delta[stat];
        }
        qm.lo[threadIdx.x] = rb.lo;
        qm.hi[threadIdx.x] = rb.hi;
        qm.seg[threadIdx.x] = rb.seg;
        qm.lse2[threadIdx.x] = l2;
        qm.delta[threadIdx.x] = dl;
        my_hi = rb.hi;
      }
      int unused, tile_hi;
      block_min_max(0, my_hi, unused, tile_hi, red);
      if (tile_hi <= first) continue;  // no row of this query tile reaches the block's first key
      // stage Q and dO rows of the tile
      constexpr int DP4 = 4 * TPR;
      for (int idx = threadIdx.x; idx < kTile * DP4; idx += kThreads) {
        int ii = idx / DP4;
        int d = (idx - ii * DP4) * 4;
        int i = i0 + ii;
        float4 qv = make_float4(0.f, 0.f, 0.f, 0.f), gv = qv;
        if (i < g.nq && d < a.head_dim) {
          int qb, qt;
          query_coord(a, g, batch, i, qb, qt);
          const T* qrow = static_cast<const T*>(a.q) + qb * a.q_strides[0] + head * a.q_strides[1] + qt * a.q_strides[2];
          const T* grow =
              static_cast<const T*>(a.dout) + qb * a.dout_strides[0] + head * a.dout_strides[1] + qt * a.dout_strides[2];
          qv = load4<T>(qrow, d, a.head_dim, vec);
          gv = load4<T>(grow, d, a.head_dim, vec);
        }
        *reinterpret_cast<float4*>(qs + ii * DP + d) = qv;
        *reinterpret_cast<float4*>(gs + ii * DP + d) = gv;
      }
      __syncthreads();
#pragma unroll 2
      for (int ii = 0; ii < kTile; ++ii) {
        float s = group_sum<TPR>(dot_slice<TPR>(kreg, qs + ii * DP, c));
        float dp = group_sum<TPR>(dot_slice<TPR>(vreg, gs + ii * DP, c));
        int i = i0 + ii;
        bool vis = live && key_kept && i < g.nq && j < qm.hi[ii];
        if (vis && a.q_seg != nullptr) {
          RowBound rb;
          rb.lo = qm.lo[ii];
          rb.hi = qm.hi[ii];
          rb.seg = qm.seg[ii];
          rb.qi = i;
          vis = doc_visible(rb, j, kseg, kend);
        }
        if (vis) {
          float p = exp2f(s * sl2 - qm.lse2[ii]);
          float ds = p * (dp - qm.delta[ii]);
          axpy_slice<TPR>(dv, p, gs + ii * DP, c);
          axpy_slice<TPR>(dk, ds, qs + ii * DP, c);
        }
      }
    }
  }
  if (live) {
#pragma unroll
    for (int e = 0; e < 16; ++e) dk[e] *= a.scale;
    if (dk_acc != nullptr) {
      long long row = (static_cast<long long>(kb) * a.kv_heads + kv_head) * a.k_len + kslot;
      atomic_slice<TPR>(dk_acc + row * a.head_dim, c, a.head_dim, dk);
      atomic_slice<TPR>(dv_acc + row * a.head_dim, c, a.head_dim, dv);
    } else {
      T* dkrow = static_cast<T*>(a.dk) + kb * a.dk_strides[0] + kv_head * a.dk_strides[1] + kslot * a.dk_strides[2];
      T* dvrow = static_cast<T*>(a.dv) + kb * a.dv_strides[0] + kv_head * a.dv_strides[1] + kslot * a.dv_strides[2];
      store_slice<T, TPR>(dkrow, c, a.head_dim, dk);
      store_slice<T, TPR>(dvrow, c, a.head_dim, dv);
    }
  }
}

// fp32 accumulator (B,HKV,K,D) -> strided gradient tensor
template <typename T>
__global__ void cast_rows_kernel(const float* src, T* dst, long long s0, long long s1, long long s2, int B, int H, int Tn,
                                 int D) {
  long long total = static_cast<long long>(B) * H * Tn;
  for (long long row = blockIdx.x * static_cast<long long>(blockDim.y) + threadIdx.y; row < total;
       row += static_cast<long long>(gridDim.x) * blockDim.y) {
    int t = static_cast<int>(row % Tn);
    int h = static_cast<int>((row / Tn) % H);
    int b = static_cast<int>(row / (static_cast<long long>(Tn) * H));
    T* p = dst + b * s0 + h * s1 + t * s2;
    const float* q = src + row * D;
    for (int d = threadIdx.x; d < D; d += blockDim.x) p[d] = from_float<T>(q[d]);
  }
}

int pick_tpr(int D) {
  if (D <= 16) return 1;
  if (D <= 32) return 2;
  if (D <= 64) return 4;
  return 8;
}

bool aligned_for_vec4(const wm_attn_args& a, bool backward) {
  size_t es = a.dtype == WM_F32 ? 4 : 2;
  auto ok_ptr = [&](const void* p) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) % (4 * es)) == 0; };
  auto ok_str = [&](const int64_t* s) { return s[0] % 4 == 0 && s[1] % 4 == 0 && s[2] % 4 == 0; };
  if (a.head_dim % 4) return false;
  bool ok = ok_ptr(a.q) && ok_ptr(a.k) && ok_ptr(a.v) && ok_str(a.q_strides) && ok_str(a.k_strides) &&
            ok_str(a.v_strides);
  if (backward) ok = ok && ok_ptr(a.dout) && ok_ptr(a.out) && ok_str(a.dout_strides) && ok_str(a.out_strides);
  return ok;
}

template <typename T, int TPR>
int launch_fwd(const wm_attn_args& a, cudaStream_t stream) {
  constexpr int ROWS = kThreads / TPR;
  SimtFlags f;
  f.vec4 = aligned_for_vec4(a, false);
  dim3 grid;
  if (a.mask == WM_MASK_PACKED) {
    // rows outside every group stay zero
    dim3 zb(32, 8);
    long long rows = static_cast<long long>(a.batch) * a.q_heads * a.q_len;
    int blocks = static_cast<int>(rows / 8 + 1 < 4096 ? rows / 8 + 1 : 4096);
    zero_rows_kernel<T><<<blocks, zb, 0, stream>>>(static_cast<T*>(a.out), a.out_strides[0], a.out_strides[1],
                                                    a.out_strides[2], a.batch, a.q_heads, a.q_len, a.head_dim, a.lse); count_launch();
    if (a.n_query_tiles == 0) return cuda_check(cudaGetLastError(), "zero_rows_kernel");
    grid = dim3(a.n_query_tiles, a.q_heads, 1);
  } else {
    grid = dim3((a.q_len + ROWS - 1) / ROWS, a.q_heads, a.batch);
  }
  attn_fwd_kernel<T, TPR><<<grid, kThreads, 0, stream>>>(a, f); count_launch();
  return cuda_check(cudaGetLastError(), "attn_fwd_kernel");
}

template <typename T, int TPR>
int launch_bwd(const wm_attn_args& a, cudaStream_t stream) {
  constexpr int ROWS = kThreads / TPR;
  SimtFlags f;
  f.vec4 = aligned_for_vec4(a, true);
  size_t need = simt_attn_bwd_workspace(a);
  if (need > a.workspace_bytes || (need && a.workspace == nullptr))
    return fail(WM_EWORKSPACE, "attention backward needs %zu workspace bytes, got %zu", need, a.workspace_bytes);
  float* delta = static_cast<float*>(a.workspace);
  size_t stats = static_cast<size_t>(a.batch) * a.q_heads * a.q_len;
  float* dk_acc = nullptr;
  float* dv_acc = nullptr;
  dim3 qgrid, kgrid;
  if (a.mask == WM_MASK_PACKED) {
    size_t kv = static_cast<size_t>(a.batch) * a.kv_heads * a.k_len * a.head_dim;
    dk_acc = delta + ((stats + 3) / 4) * 4;
    dv_acc = dk_acc + kv;
    WM_CUDA(cudaMemsetAsync(dk_acc, 0, 2 * kv * sizeof(float), stream));
    // dQ rows outside every group are zero
    dim3 zb(32, 8);
    long long rows = static_cast<long long>(a.batch) * a.q_heads * a.q_len;
    int blocks = static_cast<int>(rows / 8 + 1 < 4096 ? rows / 8 + 1 : 4096);
    zero_rows_kernel<T><<<blocks, zb, 0, stream>>>(static_cast<T*>(a.dq), a.dq_strides[0], a.dq_strides[1],
                                                    a.dq_strides[2], a.batch, a.q_heads, a.q_len, a.head_dim, nullptr); count_launch();
    qgrid = dim3(a.n_query_tiles, a.q_heads, 1);
  } else {
    qgrid = dim3((a.q_len + ROWS - 1) / ROWS, a.q_heads, a.batch);
    kgrid = dim3((a.k_len + ROWS - 1) / ROWS, a.kv_heads, a.batch);
  }
  if (a.mask != WM_MASK_PACKED || a.n_query_tiles > 0) {
    attn_dq_kernel<T, TPR><<<qgrid, kThreads, 0, stream>>>(a, f, delta); count_launch();
    WM_CUDA(cudaGetLastError());
  }
  if (a.mask == WM_MASK_PACKED) {
    if (a.n_key_tiles > 0) {
      kgrid = dim3(a.n_key_tiles, a.kv_heads, 1);
      attn_dkv_kernel<T, TPR><<<kgrid, kThreads, 0, stream>>>(a, f, delta, dk_acc, dv_acc); count_launch();
      WM_CUDA(cudaGetLastError());
    }
    dim3 zb(32, 8);
    long long rows = static_cast<long long>(a.batch) * a.kv_heads * a.k_len;
    int blocks = static_cast<int>(rows / 8 + 1 < 4096 ? rows / 8 + 1 : 4096);
    cast_rows_kernel<T><<<blocks, zb, 0, stream>>>(dk_acc, static_cast<T*>(a.dk), a.dk_strides[0], a.dk_strides[1],
                                                    a.dk_strides[2], a.batch, a.kv_heads, a.k_len, a.head_dim); count_launch();
    cast_rows_kernel<T><<<blocks, zb, 0, stream>>>(dv_acc, static_cast<T*>(a.dv), a.dv_strides[0], a.dv_strides[1],
                                                    a.dv_strides[2], a.batch, a.kv_heads, a.k_len, a.head_dim); count_launch();
  } else {
    attn_dkv_kernel<T, TPR><<<kgrid, kThreads, 0, stream>>>(a, f, delta, nullptr, nullptr); count_launch();
  }
  return cuda_check(cudaGetLastError(), "attention backward");
}

template <typename T>
int dispatch_tpr(const wm_attn_args& a, cudaStream_t stream, bool backward) {
  switch (pick_tpr(a.head_dim)) {
    case 1:
      return backward ? launch_bwd<T, 1>(a, stream) : launch_fwd<T, 1>(a, stream);
    case 2:
      return backward ? launch_bwd<T, 2>(a, stream) : launch_fwd<T, 2>(a, stream);
    case 4:
      return backward ? launch_bwd<T, 4>(a, stream) : launch_fwd<T, 4>(a, stream);
    default:
      return backward ? launch_bwd<T, 8>(a, stream) : launch_fwd<T, 8>(a, stream);
  }
}

}  // namespace

int simt_tile_rows(int head_dim) { return kThreads / pick_tpr(head_dim); }

size_t simt_attn_bwd_workspace(const wm_attn_args& a) {
  size_t stats = static_cast<size_t>(a.batch) * a.q_heads * a.q_len;
  size_t bytes = ((stats + 3) / 4) * 4 * sizeof(float);
  if (a.mask == WM_MASK_PACKED)
    bytes += 2 * static_cast<size_t>(a.batch) * a.kv_heads * a.k_len * a.head_dim * sizeof(float);
  return bytes;
}

int simt_attn_fwd(const wm_attn_args& a, cudaStream_t stream) {
  if (a.head_dim > 128) return fail(WM_EUNSUPPORTED, "head_dim %d exceeds 128", a.head_dim);
  return a.dtype == WM_F32 ? dispatch_tpr<float>(a, stream, false) : dispatch_tpr<__nv_bfloat16>(a, stream, false);
}

int simt_attn_bwd(const wm_attn_args& a, cudaStream_t stream) {
  if (a.head_dim > 128) return fail(WM_EUNSUPPORTED, "head_dim %d exceeds 128", a.head_dim);
  return a.dtype == WM_F32 ? dispatch_tpr<float>(a, stream, true) : dispatch_tpr<__nv_bfloat16>(a, stream, true);
}

}  // namespace wm
