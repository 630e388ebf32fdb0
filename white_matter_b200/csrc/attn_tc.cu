// tcgen05 / TMEM attention forward for bf16, head_dim 64.
//
// One CTA owns a tile of 128 query rows of one (batch, head) and walks over
// tiles of 128 key slots.  Roles inside the CTA (192 threads):
//   warps 0-3  softmax: thread t owns query row t == TMEM lane t; reads S with
//              tcgen05.ld, applies the mask, keeps the online-softmax state,
//              writes P (bf16) into shared memory in the K-major 128B-swizzled
//              layout the MMA reads, rescales O in TMEM when the running
//              maximum moved by more than 2^8, and writes the result.
//   warp 4     TMA producer: Q once, then K and V tiles through 3-deep rings.
//   warp 5     MMA issuer (one lane): S = Q K^T into one of two TMEM buffers,
//              O += P V into a third; completion is signalled by tcgen05.commit
//              on mbarriers.
// TMEM: S0 [0,128), S1 [128,256), O [256,320) columns; 512 allocated.
// Key tiles that no row of the query tile can see are never loaded: the walk
// ends at the largest visible slot, and document problems start at the
// smallest document start of the tile (plus tile 0 for the shared dummy).
//
// Every mbarrier wait is bounded; a wait that runs out records an error code
// in a device status word, and all roles fall through to the common exit where
// TMEM is released.
#include <cuda.h>
#include <limits.h>
#include <math.h>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace wm {
namespace {

constexpr int kTileM = 128;
constexpr int kTileN = 128;
constexpr int kHeadDim = 64;
constexpr int kStages = 3;
constexpr int kSoftmaxThreads = 128;
constexpr int kThreadsFwd = 192;
constexpr uint32_t kTileBytes = kTileN * kHeadDim * 2;  // 16 KB: one Q, K or V tile
constexpr uint32_t kTmemCols = 512;
constexpr float kRescaleThreshold = 8.f;  // log2 units

__device__ int g_status = 0;

struct FwdShared {
  // tile buffers first: each needs 1024-byte alignment for the 128B swizzle
  unsigned char q[kTileBytes];
  unsigned char k[kStages][kTileBytes];
  unsigned char v[kStages][kTileBytes];
  unsigned char p[2][2 * kTileBytes];
  uint64_t q_full;
  uint64_t k_full[kStages], k_empty[kStages], v_full[kStages], v_empty[kStages];
  uint64_t s_full[2], p_full[2], pv_done[2], docs_full[2];
  int key_seg[2][kTileN];
  int key_end[2][kTileN];
  int tile_summary[2][4][3];  // per softmax warp: min seg, max seg, min end
  int red_min_lo, red_max_hi, has_dummy;
  uint32_t tmem_base;
  int abort_flag;
};

template <class Shared>
__device__ __forceinline__ void record_failure(Shared& sm, int code) {
  atomicCAS(&g_status, 0, code);
  atomicExch(&sm.abort_flag, 1);
}

// ---------------------------------------------------------------------------
// host side: tensor maps
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) == cudaSuccess &&
        result == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// (batch, heads, tokens, 64) bf16 tensor with element strides s[0..2]; boxes of `rows` tokens x 64.
int make_map(CUtensorMap* map, const void* base, int batch, int heads, int tokens, const int64_t* s, int rows) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return fail(WM_ECUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(kHeadDim), static_cast<cuuint64_t>(tokens),
                        static_cast<cuuint64_t>(heads), static_cast<cuuint64_t>(batch)};
  cuuint64_t strides[3] = {static_cast<cuuint64_t>(s[2]) * 2, static_cast<cuuint64_t>(s[1]) * 2,
                           static_cast<cuuint64_t>(s[0]) * 2};
  // a dimension of extent 1 may come with any stride; give it a legal one
  for (int i = 0; i < 3; ++i)
    if (dims[i + 1] == 1 || strides[i] == 0) strides[i] = 128;
  cuuint32_t box[4] = {kHeadDim, static_cast<cuuint32_t>(rows), 1, 1};
  cuuint32_t elem[4] = {1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(WM_ECUDA, "cuTensorMapEncodeTiled failed with code %d", static_cast<int>(r));
  return WM_OK;
}

bool tma_ok(const void* p, const int64_t* s, int batch, int heads, int tokens) {
  if (reinterpret_cast<uintptr_t>(p) % 16) return false;
  const int extent[3] = {batch, heads, tokens};
  for (int i = 0; i < 3; ++i) {
    if (extent[i] == 1) continue;
    if (s[i] <= 0 || (s[i] * 2) % 16 || s[i] * 2 >= (1ll << 40)) return false;
  }
  return true;
}


// ---------------------------------------------------------------------------
// device side

template <class Shared>
__device__ __forceinline__ bool wait_or_abort(Shared& sm, uint64_t* bar, uint32_t parity, int code) {
  for (uint32_t spin = 0; spin < ptx::kSpinLimit; ++spin) {
    if (ptx::mbar_try_wait(bar, parity)) return true;
    if ((spin & 255u) == 255u && *reinterpret_cast<volatile int*>(&sm.abort_flag)) return false;
  }
  record_failure(sm, code);
  return false;
}

// first key slot of the n-th visited key tile
__device__ __forceinline__ int tile_first_key(int n, int first_tile, int dummy_tile) {
  if (dummy_tile) return n == 0 ? 0 : (first_tile + n - 1) * kTileN;
  return (first_tile + n) * kTileN;
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct TileWalk {
  int first_tile;
  int dummy_tile;
  int n_tiles;
  int kmax;
};

// ------------------------------------------------------------------ producer (one lane of warp 4)
__device__ __forceinline__ void producer_role(FwdShared& sm, const CUtensorMap* map_q, const CUtensorMap* map_k,
                                              const CUtensorMap* map_v, const TileWalk& w, int q0, int head,
                                              int kv_head, int batch) {
  ptx::prefetch_tmap(map_q);
  ptx::prefetch_tmap(map_k);
  ptx::prefetch_tmap(map_v);
  ptx::mbar_expect_tx(&sm.q_full, kTileBytes);
  ptx::tma_load_4d(sm.q, map_q, &sm.q_full, 0, q0, head, batch);
  for (int n = 0; n < w.n_tiles; ++n) {
    const int s = n % kStages;
    const uint32_t parity = (((n / kStages) & 1) ^ 1);
    const int j0 = tile_first_key(n, w.first_tile, w.dummy_tile);
    if (!wait_or_abort(sm, &sm.k_empty[s], parity, 11)) return;
    ptx::mbar_expect_tx(&sm.k_full[s], kTileBytes);
    ptx::tma_load_4d(sm.k[s], map_k, &sm.k_full[s], 0, j0, kv_head, batch);
    if (!wait_or_abort(sm, &sm.v_empty[s], parity, 12)) return;
    ptx::mbar_expect_tx(&sm.v_full[s], kTileBytes);
    ptx::tma_load_4d(sm.v[s], map_v, &sm.v_full[s], 0, j0, kv_head, batch);
  }
}

// ------------------------------------------------------------------ MMA issuer (one lane of warp 5)
__device__ __forceinline__ bool issue_qk(FwdShared& sm, uint32_t tmem, int n) {
  const int s = n % kStages;
  if (!wait_or_abort(sm, &sm.k_full[s], (n / kStages) & 1, 21)) return false;
  ptx::tc_fence_after();
  constexpr uint32_t idesc = ptx::make_idesc_bf16(kTileM, kTileN, 0, 0);
  const uint32_t a_base = ptx::smem_u32(sm.q);
  const uint32_t b_base = ptx::smem_u32(sm.k[s]);
  const uint32_t d = tmem + static_cast<uint32_t>(n & 1) * kTileN;
#pragma unroll
  for (int kk = 0; kk < kHeadDim / 16; ++kk) {
    // 16 elements of head_dim per instruction: 32 bytes inside the 128-byte swizzle row
    ptx::mma_bf16_ss(d, ptx::make_smem_desc_sw128(a_base + kk * 32, 16, 1024),
                     ptx::make_smem_desc_sw128(b_base + kk * 32, 16, 1024), idesc, kk > 0);
  }
  ptx::mma_commit(&sm.k_empty[s]);
  ptx::mma_commit(&sm.s_full[n & 1]);
  return true;
}

__device__ __forceinline__ void mma_role(FwdShared& sm, uint32_t tmem, const TileWalk& w) {
  if (!wait_or_abort(sm, &sm.q_full, 0, 20)) return;
  if (!issue_qk(sm, tmem, 0)) return;
  constexpr uint32_t idesc_pv = ptx::make_idesc_bf16(kTileM, kHeadDim, 0, 1);
  const uint32_t o_tmem = tmem + 2 * kTileN;
  for (int n = 0; n < w.n_tiles; ++n) {
    if (n + 1 < w.n_tiles && !issue_qk(sm, tmem, n + 1)) return;
    const int b = n & 1;
    const int s = n % kStages;
    if (!wait_or_abort(sm, &sm.p_full[b], (n >> 1) & 1, 22)) return;
    if (!wait_or_abort(sm, &sm.v_full[s], (n / kStages) & 1, 23)) return;
    ptx::tc_fence_after();
    const uint32_t p_base = ptx::smem_u32(sm.p[b]);
    const uint32_t v_base = ptx::smem_u32(sm.v[s]);
#pragma unroll
    for (int kk = 0; kk < kTileN / 16; ++kk) {
      // A = P: K-major, 64-key sub-tiles of 16 KB; B = V: head_dim contiguous (MN-major), 16 keys = 2048 bytes
      const uint64_t a_desc = ptx::make_smem_desc_sw128(p_base + (kk >> 2) * kTileBytes + (kk & 3) * 32, 16, 1024);
      const uint64_t b_desc = ptx::make_smem_desc_sw128(v_base + kk * 2048, 1024, 1024);
      ptx::mma_bf16_ss(o_tmem, a_desc, b_desc, idesc_pv, (n > 0) || (kk > 0));
    }
    ptx::mma_commit(&sm.v_empty[s]);
    ptx::mma_commit(&sm.pv_done[b]);
  }
}

// ------------------------------------------------------------------ softmax (warps 0-3, thread t == query row t)
struct RowState {
  float m_ref;  // maximum the stored exponentials are relative to (log2 units); -inf until a key is seen
  float l;      // sum of exponentials relative to m_ref
};

// Stage the document id / query bound of the tile's keys and per-warp summaries of them.
template <class Shared>
__device__ __forceinline__ bool wait_or_abort(Shared& sm, uint64_t* bar, uint32_t parity, int code);

__device__ __forceinline__ bool stage_key_docs(FwdShared& sm, const wm_attn_args& a, int batch, int j0, int buf,
                                               int t, int warp, int lane, int n) {
  int seg = INT_MIN, end = 0;
  const int j = j0 + t;
  if (j < a.k_len) {
    const long long at = static_cast<long long>(batch) * a.k_len + j;
    seg = a.k_seg[at];
    end = a.k_query_end[at];
  }
  sm.key_seg[buf][t] = seg;
  sm.key_end[buf][t] = end;
  const int smin = __reduce_min_sync(0xffffffffu, seg);
  const int smax = __reduce_max_sync(0xffffffffu, seg);
  const int emin = __reduce_min_sync(0xffffffffu, end);
  if (lane == 0) {
    sm.tile_summary[buf][warp][0] = smin;
    sm.tile_summary[buf][warp][1] = smax;
    sm.tile_summary[buf][warp][2] = emin;
  }
  // all 128 softmax threads have published their key; bounded, unlike a named barrier
  ptx::mbar_arrive(&sm.docs_full[buf]);
  return wait_or_abort(sm, &sm.docs_full[buf], (n >> 1) & 1, 30);
}

__device__ __forceinline__ void softmax_role(FwdShared& sm, const wm_attn_args& a, uint32_t tmem, const TileWalk& w,
                                             const RowBound& rb, bool live, int batch, int head, int row) {
  const int t = threadIdx.x;
  const int warp = t >> 5, lane = t & 31;
  const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;  // this warp's quarter of the TMEM lanes
  const float sl2 = a.scale * kLog2e;
  const bool docs = a.q_seg != nullptr;
  RowState st;
  st.m_ref = -INFINITY;
  st.l = 0.f;
  const uint32_t o_tmem = tmem + 2 * kTileN + lane_base;

  for (int n = 0; n < w.n_tiles; ++n) {
    const int b = n & 1;
    const int j0 = tile_first_key(n, w.first_tile, w.dummy_tile);
    if (docs && !stage_key_docs(sm, a, batch, j0, b, t, warp, lane, n)) return;
    // classify the tile for this row
    bool none = !live || j0 >= rb.hi;
    bool full = live && j0 + kTileN <= rb.hi;
    if (docs && !none) {
      int smin = sm.tile_summary[b][0][0], smax = sm.tile_summary[b][0][1], emin = sm.tile_summary[b][0][2];
#pragma unroll
      for (int q = 1; q < 4; ++q) {
        smin = min(smin, sm.tile_summary[b][q][0]);
        smax = max(smax, sm.tile_summary[b][q][1]);
        emin = min(emin, sm.tile_summary[b][q][2]);
      }
      const bool uniform = smin == smax;
      full = full && uniform && smin == rb.seg && j0 >= rb.lo && emin > rb.qi;
      if (uniform && smin != -1 && smin != rb.seg) none = true;
    }
    if (!wait_or_abort(sm, &sm.s_full[b], (n >> 1) & 1, 31)) return;
    ptx::tc_fence_after();
    float x[kTileN];
    {
      const uint32_t s_tmem = tmem + static_cast<uint32_t>(b) * kTileN + lane_base;
#pragma unroll
      for (int c = 0; c < kTileN / 32; ++c) {
        uint32_t raw[32];
        ptx::tmem_ld32(s_tmem + c * 32, raw);
#pragma unroll
        for (int e = 0; e < 32; ++e) x[c * 32 + e] = __uint_as_float(raw[e]);
      }
      ptx::tmem_wait_ld();
    }
    // mask and row maximum (raw score units; the scale is positive)
    float top = -INFINITY;
    if (none) {
#pragma unroll
      for (int c = 0; c < kTileN; ++c) x[c] = -INFINITY;
    } else if (full) {
#pragma unroll
      for (int c = 0; c < kTileN; ++c) top = fmaxf(top, x[c]);
    } else if (!docs) {
      const int lim = rb.hi - j0;
#pragma unroll
      for (int c = 0; c < kTileN; ++c) {
        x[c] = c < lim ? x[c] : -INFINITY;
        top = fmaxf(top, x[c]);
      }
    } else {
      const int lim = rb.hi - j0;
#pragma unroll
      for (int c = 0; c < kTileN; ++c) {
        const bool vis = c < lim && doc_visible(rb, j0 + c, sm.key_seg[b][c], sm.key_end[b][c]);
        x[c] = vis ? x[c] : -INFINITY;
        top = fmaxf(top, x[c]);
      }
    }
    top *= sl2;  // -inf stays -inf
    // lazy rescale: move the reference maximum only when it would grow by more than the threshold
    float corr = 1.f;
    bool moved = false;
    if (top > st.m_ref + kRescaleThreshold || (st.m_ref == -INFINITY && top > -INFINITY)) {
      moved = st.m_ref != -INFINITY;
      corr = moved ? fast_exp2(st.m_ref - top) : 1.f;
      st.m_ref = top;
      st.l *= corr;
    }
    const float m_use = st.m_ref == -INFINITY ? 0.f : st.m_ref;
    // the P buffer was last read by the PV product of tile n-2
    if (n >= 2 && !wait_or_abort(sm, &sm.pv_done[b], ((n - 2) >> 1) & 1, 32)) return;
    {
      unsigned char* prow = sm.p[b] + (row >> 3) * 1024 + (row & 7) * 128;
      float sum = 0.f;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          uint32_t pk[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int col = h * 64 + c * 8 + 2 * e;
            const float p0 = fast_exp2(fmaf(x[col], sl2, -m_use));
            const float p1 = fast_exp2(fmaf(x[col + 1], sl2, -m_use));
            sum += p0 + p1;
            pk[e] = pack_bf16(p0, p1);
          }
          *reinterpret_cast<uint4*>(prow + h * kTileBytes + ((c ^ (row & 7)) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        }
      }
      st.l += sum;
    }
    // rescale O when any row of this warp moved its reference (O is complete after the PV product of tile n-1)
    if (__any_sync(0xffffffffu, moved)) {
      if (n >= 1 && !wait_or_abort(sm, &sm.pv_done[(n - 1) & 1], ((n - 1) >> 1) & 1, 33)) return;
      ptx::tc_fence_after();
#pragma unroll
      for (int c = 0; c < kHeadDim / 32; ++c) {
        uint32_t raw[32];
        ptx::tmem_ld32(o_tmem + c * 32, raw);
        ptx::tmem_wait_ld();
#pragma unroll
        for (int e = 0; e < 32; ++e) raw[e] = __float_as_uint(__uint_as_float(raw[e]) * corr);
        ptx::tmem_st32(o_tmem + c * 32, raw);
      }
      ptx::tmem_wait_st();
    }
    // last tile: value rows at or beyond the largest visible slot may hold anything (unused cache capacity)
    if (n == w.n_tiles - 1 && w.kmax < j0 + kTileN) {
      const int s = n % kStages;
      if (!wait_or_abort(sm, &sm.v_full[s], (n / kStages) & 1, 34)) return;
      if (j0 + row >= w.kmax) {
        uint4* vrow = reinterpret_cast<uint4*>(sm.v[s] + row * 128);
#pragma unroll
        for (int c = 0; c < 8; ++c) vrow[c] = make_uint4(0, 0, 0, 0);
      }
    }
    ptx::fence_async_shared();
    ptx::tc_fence_before();
    ptx::mbar_arrive(&sm.p_full[b]);
  }
  // epilogue: O / l -> bf16 rows, log-sum-exp
  const int last = w.n_tiles - 1;
  if (!wait_or_abort(sm, &sm.pv_done[last & 1], (last >> 1) & 1, 35)) return;
  ptx::tc_fence_after();
  const float inv = st.l > 0.f ? 1.f / st.l : 0.f;
  uint32_t packed[kHeadDim / 2];
#pragma unroll
  for (int c = 0; c < kHeadDim / 32; ++c) {
    uint32_t raw[32];
    ptx::tmem_ld32(o_tmem + c * 32, raw);
    ptx::tmem_wait_ld();
#pragma unroll
    for (int e = 0; e < 16; ++e)
      packed[c * 16 + e] = pack_bf16(__uint_as_float(raw[2 * e]) * inv, __uint_as_float(raw[2 * e + 1]) * inv);
  }
  if (live) {
    const int i = rb.qi;
    __nv_bfloat16* orow = static_cast<__nv_bfloat16*>(a.out) + batch * a.out_strides[0] + head * a.out_strides[1] +
                          static_cast<long long>(i) * a.out_strides[2];
    uint4* dst = reinterpret_cast<uint4*>(orow);
#pragma unroll
    for (int c = 0; c < 8; ++c)
      dst[c] = st.l > 0.f ? make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3])
                          : make_uint4(0, 0, 0, 0);
    if (a.lse != nullptr)
      a.lse[(static_cast<long long>(batch) * a.q_heads + head) * a.q_len + i] =
          st.l > 0.f ? (st.m_ref + log2f(st.l)) * kLn2 : INFINITY;
  }
}

// ------------------------------------------------------------------ kernel
__global__ void __launch_bounds__(kThreadsFwd, 1)
    attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const wm_attn_args a) {
  extern __shared__ unsigned char smem_raw[];
  FwdShared& sm = *reinterpret_cast<FwdShared*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int q_tile = gridDim.x - 1 - blockIdx.x;  // tiles with the longest key walk start first
  const int head = blockIdx.y;
  const int batch = blockIdx.z;
  const int kv_head = head / (a.q_heads / a.kv_heads);
  const int q0 = q_tile * kTileM;
  const GroupCtx g = group_ctx(a, 0);

  if (tid == 0) {
    sm.red_min_lo = INT_MAX;
    sm.red_max_hi = 0;
    sm.abort_flag = 0;
    sm.has_dummy = a.q_seg != nullptr && a.k_seg[static_cast<long long>(batch) * a.k_len] == -1;
  }
  __syncthreads();
  RowBound rb;
  rb.lo = 0;
  rb.hi = 0;
  rb.seg = 0;
  rb.qi = q0 + tid;
  bool live = false;
  if (tid < kSoftmaxThreads) {
    live = q0 + tid < a.q_len;
    if (live) rb = row_bound(a, g, batch, q0 + tid);
    const int lo = live && rb.hi > 0 ? rb.lo : INT_MAX;
    const int wlo = __reduce_min_sync(0xffffffffu, lo);
    const int whi = __reduce_max_sync(0xffffffffu, rb.hi);
    if (lane == 0) {
      atomicMin(&sm.red_min_lo, wlo);
      atomicMax(&sm.red_max_hi, whi);
    }
  }
  __syncthreads();
  TileWalk w;
  w.kmax = sm.red_max_hi;
  if (w.kmax == 0) {
    // no row of this tile sees a key: zeros and +inf, no pipeline
    if (live) {
      __nv_bfloat16* orow = static_cast<__nv_bfloat16*>(a.out) + batch * a.out_strides[0] + head * a.out_strides[1] +
                            static_cast<long long>(rb.qi) * a.out_strides[2];
#pragma unroll
      for (int c = 0; c < 8; ++c) reinterpret_cast<uint4*>(orow)[c] = make_uint4(0, 0, 0, 0);
      if (a.lse != nullptr) a.lse[(static_cast<long long>(batch) * a.q_heads + head) * a.q_len + rb.qi] = INFINITY;
    }
    return;
  }
  const int end_tile = (w.kmax + kTileN - 1) / kTileN;
  w.first_tile = a.q_seg != nullptr ? min(sm.red_min_lo / kTileN, end_tile - 1) : 0;
  w.dummy_tile = (a.q_seg != nullptr && sm.has_dummy && w.first_tile > 0) ? 1 : 0;
  w.n_tiles = end_tile - w.first_tile + w.dummy_tile;

  if (tid == 0) {
    ptx::mbar_init(&sm.q_full, 1);
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(&sm.k_full[s], 1);
      ptx::mbar_init(&sm.k_empty[s], 1);
      ptx::mbar_init(&sm.v_full[s], 1);
      ptx::mbar_init(&sm.v_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(&sm.s_full[b], 1);
      ptx::mbar_init(&sm.p_full[b], kSoftmaxThreads);
      ptx::mbar_init(&sm.pv_done[b], 1);
      ptx::mbar_init(&sm.docs_full[b], kSoftmaxThreads);
    }
    ptx::mbar_fence_init();
  }
  if (warp == 4) {
    ptx::tmem_alloc(&sm.tmem_base, kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = sm.tmem_base;

  if (warp < 4) {
    softmax_role(sm, a, tmem, w, rb, live, batch, head, tid);
  } else if (warp == 4) {
    if (lane == 0) producer_role(sm, &map_q, &map_k, &map_v, w, q0, head, kv_head, batch);
  } else {
    if (lane == 0) mma_role(sm, tmem, w);
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 4) ptx::tmem_dealloc(tmem, kTmemCols);
}


// ===========================================================================
// backward: one CTA per tile of 128 key slots of one (batch, kv head).
//
// For every query tile that can see the key tile (and every query head of the
// group) the CTA recomputes S = Q K^T and dP = dO V^T on the tensor cores,
// forms P = exp2(S*scale*log2e - lse) and dS = P*(dP - delta) in registers
// (thread t == query row t), stores both as bf16 in one [query][key] swizzled
// shared-memory tile each, and issues dV += P^T dO, dK += dS^T Q (accumulated
// in TMEM over the whole walk) and dQ = dS K (added to an fp32 accumulator in
// global memory with vector reductions, converted to bf16 by a last kernel).
// The same shared tile serves as K-major operand (dS K) and as MN-major
// operand (P^T dO, dS^T Q); Q and dO tiles likewise serve as A (K-major) and
// as B (MN-major).
// TMEM columns: S [0,128) dP [128,256) dV [256,320) dK [320,384) dQ [384,448).
constexpr int kBwdStages = 2;

struct BwdShared {
  unsigned char k[kTileBytes];
  unsigned char v[kTileBytes];
  unsigned char q[kBwdStages][kTileBytes];
  unsigned char g[kBwdStages][kTileBytes];  // dO tiles
  unsigned char p[2 * kTileBytes];
  unsigned char ds[2 * kTileBytes];
  uint64_t kv_full, kv_ready;
  uint64_t qg_full[kBwdStages], qg_empty[kBwdStages];
  uint64_t sdp_full, pds_full, mma_done, dq_full, dq_free;
  int key_seg[kTileN];
  int key_end[kTileN];
  int summary[4][4];  // per warp: min seg, max seg, min end, max end
  int row_first, row_end;
  uint32_t tmem_base;
  int abort_flag;
};

// delta = rowsum(dO * O) in fp32, one thread per (batch, head, query) row of 64 values
__global__ void bwd_delta_kernel(const wm_attn_args a, float* delta) {
  const long long rows = static_cast<long long>(a.batch) * a.q_heads * a.q_len;
  const long long row = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (row >= rows) return;
  const int i = static_cast<int>(row % a.q_len);
  const int h = static_cast<int>((row / a.q_len) % a.q_heads);
  const int b = static_cast<int>(row / (static_cast<long long>(a.q_len) * a.q_heads));
  const uint4* o = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(a.out) + b * a.out_strides[0] +
                                                  h * a.out_strides[1] + static_cast<long long>(i) * a.out_strides[2]);
  const uint4* g = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(a.dout) + b * a.dout_strides[0] +
                                                  h * a.dout_strides[1] + static_cast<long long>(i) * a.dout_strides[2]);
  float acc = 0.f;
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const uint4 x = o[c], y = g[c];
    const unsigned xs[4] = {x.x, x.y, x.z, x.w}, ys[4] = {y.x, y.y, y.z, y.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      acc = fmaf(__uint_as_float(xs[e] << 16), __uint_as_float(ys[e] << 16), acc);
      acc = fmaf(__uint_as_float(xs[e] & 0xffff0000u), __uint_as_float(ys[e] & 0xffff0000u), acc);
    }
  }
  delta[row] = acc;
}

// dq = bf16(scale * accumulator); accumulator is (batch, heads, queries, 64) fp32
__global__ void bwd_dq_convert_kernel(const wm_attn_args a, const float* acc) {
  const long long chunks = static_cast<long long>(a.batch) * a.q_heads * a.q_len * 8;  // 8 values each
  const long long at = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (at >= chunks) return;
  const long long row = at >> 3;
  const int c = static_cast<int>(at & 7);
  const int i = static_cast<int>(row % a.q_len);
  const int h = static_cast<int>((row / a.q_len) % a.q_heads);
  const int b = static_cast<int>(row / (static_cast<long long>(a.q_len) * a.q_heads));
  const float4 lo = *reinterpret_cast<const float4*>(acc + row * kHeadDim + c * 8);
  const float4 hi = *reinterpret_cast<const float4*>(acc + row * kHeadDim + c * 8 + 4);
  const float s = a.scale;
  __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(a.dq) + b * a.dq_strides[0] + h * a.dq_strides[1] +
                       static_cast<long long>(i) * a.dq_strides[2] + c * 8;
  *reinterpret_cast<uint4*>(dst) = make_uint4(pack_bf16(lo.x * s, lo.y * s), pack_bf16(lo.z * s, lo.w * s),
                                              pack_bf16(hi.x * s, hi.y * s), pack_bf16(hi.z * s, hi.w * s));
}

__device__ __forceinline__ void red_add_v4(float* addr, float a0, float a1, float a2, float a3) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a0), "f"(a1), "f"(a2), "f"(a3)
               : "memory");
}

struct BwdWalk {
  int qt_first;  // first query tile that can see the key tile
  int qt_count;  // number of query tiles to visit (0: none)
  int heads;     // query heads per kv head
  int n_iter;    // qt_count * heads
  int kvis;      // exclusive bound of key slots any query can see
};

__device__ __forceinline__ void bwd_iter_coords(const BwdWalk& w, int it, int kv_head, int& head, int& qt) {
  const int g = it / w.qt_count;
  qt = w.qt_first + (it - g * w.qt_count);
  head = kv_head * w.heads + g;
}

__device__ __forceinline__ void bwd_producer(BwdShared& sm, const CUtensorMap* map_q, const CUtensorMap* map_k,
                                             const CUtensorMap* map_v, const CUtensorMap* map_g, const BwdWalk& w,
                                             int j0, int kv_head, int batch) {
  ptx::prefetch_tmap(map_q);
  ptx::prefetch_tmap(map_k);
  ptx::prefetch_tmap(map_v);
  ptx::prefetch_tmap(map_g);
  ptx::mbar_expect_tx(&sm.kv_full, 2 * kTileBytes);
  ptx::tma_load_4d(sm.k, map_k, &sm.kv_full, 0, j0, kv_head, batch);
  ptx::tma_load_4d(sm.v, map_v, &sm.kv_full, 0, j0, kv_head, batch);
  for (int it = 0; it < w.n_iter; ++it) {
    const int s = it % kBwdStages;
    int head, qt;
    bwd_iter_coords(w, it, kv_head, head, qt);
    if (!wait_or_abort(sm, &sm.qg_empty[s], ((it / kBwdStages) & 1) ^ 1, 41)) return;
    ptx::mbar_expect_tx(&sm.qg_full[s], 2 * kTileBytes);
    ptx::tma_load_4d(sm.q[s], map_q, &sm.qg_full[s], 0, qt * kTileM, head, batch);
    ptx::tma_load_4d(sm.g[s], map_g, &sm.qg_full[s], 0, qt * kTileM, head, batch);
  }
}

__device__ __forceinline__ void bwd_mma(BwdShared& sm, uint32_t tmem, const BwdWalk& w) {
  if (!wait_or_abort(sm, &sm.kv_ready, 0, 50)) return;
  ptx::tc_fence_after();
  constexpr uint32_t idesc_s = ptx::make_idesc_bf16(kTileM, kTileN, 0, 0);      // Q K^T, dO V^T
  constexpr uint32_t idesc_t = ptx::make_idesc_bf16(kTileN, kHeadDim, 1, 1);    // P^T dO, dS^T Q
  constexpr uint32_t idesc_q = ptx::make_idesc_bf16(kTileM, kHeadDim, 0, 1);    // dS K
  const uint32_t k_base = ptx::smem_u32(sm.k), v_base = ptx::smem_u32(sm.v);
  const uint32_t p_base = ptx::smem_u32(sm.p), ds_base = ptx::smem_u32(sm.ds);
  for (int it = 0; it < w.n_iter; ++it) {
    const int s = it % kBwdStages;
    if (!wait_or_abort(sm, &sm.qg_full[s], (it / kBwdStages) & 1, 51)) return;
    ptx::tc_fence_after();
    const uint32_t q_base = ptx::smem_u32(sm.q[s]), g_base = ptx::smem_u32(sm.g[s]);
#pragma unroll
    for (int kk = 0; kk < kHeadDim / 16; ++kk)
      ptx::mma_bf16_ss(tmem, ptx::make_smem_desc_sw128(q_base + kk * 32, 16, 1024),
                       ptx::make_smem_desc_sw128(k_base + kk * 32, 16, 1024), idesc_s, kk > 0);
#pragma unroll
    for (int kk = 0; kk < kHeadDim / 16; ++kk)
      ptx::mma_bf16_ss(tmem + kTileN, ptx::make_smem_desc_sw128(g_base + kk * 32, 16, 1024),
                       ptx::make_smem_desc_sw128(v_base + kk * 32, 16, 1024), idesc_s, kk > 0);
    ptx::mma_commit(&sm.sdp_full);
    if (!wait_or_abort(sm, &sm.pds_full, it & 1, 52)) return;
    ptx::tc_fence_after();
#pragma unroll
    for (int kk = 0; kk < kTileM / 16; ++kk)  // 16 queries per instruction
      ptx::mma_bf16_ss(tmem + 2 * kTileN, ptx::make_smem_desc_sw128(p_base + kk * 2048, kTileBytes, 1024),
                       ptx::make_smem_desc_sw128(g_base + kk * 2048, 1024, 1024), idesc_t, (it > 0) || (kk > 0));
#pragma unroll
    for (int kk = 0; kk < kTileM / 16; ++kk)
      ptx::mma_bf16_ss(tmem + 2 * kTileN + kHeadDim, ptx::make_smem_desc_sw128(ds_base + kk * 2048, kTileBytes, 1024),
                       ptx::make_smem_desc_sw128(q_base + kk * 2048, 1024, 1024), idesc_t, (it > 0) || (kk > 0));
    if (!wait_or_abort(sm, &sm.dq_free, (it & 1) ^ 1, 53)) return;
    ptx::tc_fence_after();
#pragma unroll
    for (int kk = 0; kk < kTileN / 16; ++kk)  // 16 keys per instruction
      ptx::mma_bf16_ss(tmem + 2 * kTileN + 2 * kHeadDim,
                       ptx::make_smem_desc_sw128(ds_base + (kk >> 2) * kTileBytes + (kk & 3) * 32, 16, 1024),
                       ptx::make_smem_desc_sw128(k_base + kk * 2048, 1024, 1024), idesc_q, kk > 0);
    ptx::mma_commit(&sm.qg_empty[s]);
    ptx::mma_commit(&sm.mma_done);
    ptx::mma_commit(&sm.dq_full);
  }
}

// compute threads of the backward kernel: thread t owns query row t of the current query tile (and, in
// the prologue / epilogue, key row t of the CTA's key tile)
__device__ __forceinline__ void bwd_compute(BwdShared& sm, const wm_attn_args& a, uint32_t tmem, const BwdWalk& w,
                                            const float* delta, float* dq_acc, int j0, int kv_head, int batch) {
  const int t = threadIdx.x;
  const int warp = t >> 5;
  const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
  const float sl2 = a.scale * kLog2e;
  const bool docs = a.q_seg != nullptr;
  const GroupCtx g = group_ctx(a, 0);

  // prologue: key rows at or beyond the last visible slot may hold anything; clear them for the MMAs
  if (!wait_or_abort(sm, &sm.kv_full, 0, 60)) return;
  if (j0 + t >= w.kvis) {
    uint4* krow = reinterpret_cast<uint4*>(sm.k + t * 128);
    uint4* vrow = reinterpret_cast<uint4*>(sm.v + t * 128);
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      krow[c] = make_uint4(0, 0, 0, 0);
      vrow[c] = make_uint4(0, 0, 0, 0);
    }
  }
  ptx::fence_async_shared();
  ptx::mbar_arrive(&sm.kv_ready);

  int smin = 0, smax = 0, emin = 0;
  if (docs) {
    smin = min(min(sm.summary[0][0], sm.summary[1][0]), min(sm.summary[2][0], sm.summary[3][0]));
    smax = max(max(sm.summary[0][1], sm.summary[1][1]), max(sm.summary[2][1], sm.summary[3][1]));
    emin = min(min(sm.summary[0][2], sm.summary[1][2]), min(sm.summary[2][2], sm.summary[3][2]));
  }

  for (int it = 0; it < w.n_iter; ++it) {
    int head, qt;
    bwd_iter_coords(w, it, kv_head, head, qt);
    const int i = qt * kTileM + t;
    const bool live = i < a.q_len;
    RowBound rb;
    rb.lo = 0;
    rb.hi = 0;
    rb.seg = 0;
    rb.qi = i;
    float lse2 = INFINITY, dl = 0.f;
    const long long stat = (static_cast<long long>(batch) * a.q_heads + head) * a.q_len + i;
    if (live) {
      rb = row_bound(a, g, batch, i);
      lse2 = a.lse[stat] * kLog2e;
      dl = delta[stat];
    }
    bool none = !live || j0 >= rb.hi;
    bool full = live && j0 + kTileN <= rb.hi;
    if (docs && !none) {
      const bool uniform = smin == smax;
      full = full && uniform && smin == rb.seg && j0 >= rb.lo && emin > rb.qi;
      if (uniform && smin != -1 && smin != rb.seg) none = true;
    }
    if (!wait_or_abort(sm, &sm.sdp_full, it & 1, 61)) return;
    ptx::tc_fence_after();
    // the shared P / dS tiles were last read by the MMAs of the previous iteration
    if (it > 0 && !wait_or_abort(sm, &sm.mma_done, (it - 1) & 1, 62)) return;
    unsigned char* prow = sm.p + (t >> 3) * 1024 + (t & 7) * 128;
    unsigned char* drow = sm.ds + (t >> 3) * 1024 + (t & 7) * 128;
    const int lim = rb.hi - j0;
#pragma unroll 1
    for (int c = 0; c < kTileN / 32; ++c) {
      uint32_t xs[32], ys[32];
      ptx::tmem_ld32(tmem + lane_base + c * 32, xs);
      ptx::tmem_ld32(tmem + kTileN + lane_base + c * 32, ys);
      ptx::tmem_wait_ld();
      uint32_t pp[16], dd[16];
#pragma unroll
      for (int e = 0; e < 16; ++e) {
        float pv[2], dv[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int col = c * 32 + 2 * e + u;
          bool vis = !none && (full || col < lim);
          if (vis && docs && !full) vis = doc_visible(rb, j0 + col, sm.key_seg[col], sm.key_end[col]);
          const float p = fast_exp2(fmaf(__uint_as_float(xs[2 * e + u]), sl2, -lse2));
          pv[u] = vis ? p : 0.f;
          dv[u] = vis ? p * (__uint_as_float(ys[2 * e + u]) - dl) : 0.f;
        }
        pp[e] = pack_bf16(pv[0], pv[1]);
        dd[e] = pack_bf16(dv[0], dv[1]);
      }
      const int sub = (c >> 1) * kTileBytes;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int off = sub + ((((c & 1) * 4 + u) ^ (t & 7)) << 4);
        *reinterpret_cast<uint4*>(prow + off) = make_uint4(pp[4 * u], pp[4 * u + 1], pp[4 * u + 2], pp[4 * u + 3]);
        *reinterpret_cast<uint4*>(drow + off) = make_uint4(dd[4 * u], dd[4 * u + 1], dd[4 * u + 2], dd[4 * u + 3]);
      }
    }
    ptx::fence_async_shared();
    ptx::tc_fence_before();
    ptx::mbar_arrive(&sm.pds_full);
    // dQ of this (query tile, key tile) pair: add to the fp32 accumulator
    if (!wait_or_abort(sm, &sm.dq_full, it & 1, 63)) return;
    ptx::tc_fence_after();
#pragma unroll
    for (int c = 0; c < kHeadDim / 32; ++c) {
      uint32_t raw[32];
      ptx::tmem_ld32(tmem + 2 * kTileN + 2 * kHeadDim + lane_base + c * 32, raw);
      ptx::tmem_wait_ld();
      if (live && !none) {
        float* dst = dq_acc + stat * kHeadDim + c * 32;
#pragma unroll
        for (int e = 0; e < 8; ++e)
          red_add_v4(dst + 4 * e, __uint_as_float(raw[4 * e]), __uint_as_float(raw[4 * e + 1]),
                     __uint_as_float(raw[4 * e + 2]), __uint_as_float(raw[4 * e + 3]));
      }
    }
    ptx::tc_fence_before();
    ptx::mbar_arrive(&sm.dq_free);
  }

  // epilogue: dV and dK rows of this key tile (dq_full of the last iteration covers every earlier MMA)
  const int j = j0 + t;
  uint32_t dv_pack[kHeadDim / 2], dk_pack[kHeadDim / 2];
#pragma unroll
  for (int e = 0; e < kHeadDim / 2; ++e) dv_pack[e] = dk_pack[e] = 0u;
  if (w.n_iter > 0) {
#pragma unroll
    for (int c = 0; c < kHeadDim / 32; ++c) {
      uint32_t raw[32];
      ptx::tmem_ld32(tmem + 2 * kTileN + lane_base + c * 32, raw);
      ptx::tmem_wait_ld();
#pragma unroll
      for (int e = 0; e < 16; ++e)
        dv_pack[c * 16 + e] = pack_bf16(__uint_as_float(raw[2 * e]), __uint_as_float(raw[2 * e + 1]));
      ptx::tmem_ld32(tmem + 2 * kTileN + kHeadDim + lane_base + c * 32, raw);
      ptx::tmem_wait_ld();
#pragma unroll
      for (int e = 0; e < 16; ++e)
        dk_pack[c * 16 + e] =
            pack_bf16(__uint_as_float(raw[2 * e]) * a.scale, __uint_as_float(raw[2 * e + 1]) * a.scale);
    }
  }
  if (j < a.k_len) {
    uint4* dvrow = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(a.dv) + batch * a.dv_strides[0] +
                                            kv_head * a.dv_strides[1] + static_cast<long long>(j) * a.dv_strides[2]);
    uint4* dkrow = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(a.dk) + batch * a.dk_strides[0] +
                                            kv_head * a.dk_strides[1] + static_cast<long long>(j) * a.dk_strides[2]);
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      dvrow[c] = make_uint4(dv_pack[4 * c], dv_pack[4 * c + 1], dv_pack[4 * c + 2], dv_pack[4 * c + 3]);
      dkrow[c] = make_uint4(dk_pack[4 * c], dk_pack[4 * c + 1], dk_pack[4 * c + 2], dk_pack[4 * c + 3]);
    }
  }
}

__global__ void __launch_bounds__(kThreadsFwd, 1)
    attn_bwd_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_g,
                       const wm_attn_args a, const float* delta, float* dq_acc) {
  extern __shared__ unsigned char smem_raw[];
  BwdShared& sm = *reinterpret_cast<BwdShared*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int j0 = blockIdx.x * kTileN;
  const int kv_head = blockIdx.y;
  const int batch = blockIdx.z;
  const GroupCtx g = group_ctx(a, 0);
  const bool docs = a.q_seg != nullptr;

  if (tid == 0) sm.abort_flag = 0;
  if (tid < kSoftmaxThreads && docs) {
    int seg = INT_MIN, end = 0;
    if (j0 + tid < a.k_len) {
      const long long at = static_cast<long long>(batch) * a.k_len + j0 + tid;
      seg = a.k_seg[at];
      end = a.k_query_end[at];
    }
    sm.key_seg[tid] = seg;
    sm.key_end[tid] = end;
    // rows beyond the tensor do not take part in the summaries
    const bool in = j0 + tid < a.k_len;
    const int smin = __reduce_min_sync(0xffffffffu, in ? seg : INT_MAX);
    const int smax = __reduce_max_sync(0xffffffffu, in ? seg : INT_MIN);
    const int emin = __reduce_min_sync(0xffffffffu, in ? end : INT_MAX);
    const int emax = __reduce_max_sync(0xffffffffu, end);
    if (lane == 0) {
      sm.summary[warp][0] = smin;
      sm.summary[warp][1] = smax;
      sm.summary[warp][2] = emin;
      sm.summary[warp][3] = emax;
    }
  }
  __syncthreads();
  if (tid == 0) {
    // every mask family has a visibility bound that does not decrease with the query index
    const int kvis = row_bound(a, g, batch, a.q_len - 1).hi;
    int first = a.q_len;
    if (j0 < kvis) {
      int lo = 0, hi = a.q_len - 1;  // smallest i with bound(i) > j0
      while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (row_bound(a, g, batch, mid).hi > j0) hi = mid; else lo = mid + 1;
      }
      first = lo;
    }
    int end = a.q_len;
    if (docs) {
      const int emax = max(max(sm.summary[0][3], sm.summary[1][3]), max(sm.summary[2][3], sm.summary[3][3]));
      end = min(end, emax);
    }
    sm.row_first = first;
    sm.row_end = end;
    sm.tmem_base = 0;
    sm.summary[0][3] = kvis;  // reuse: publish the visible bound
  }
  __syncthreads();
  BwdWalk w;
  w.kvis = sm.summary[0][3];
  w.heads = a.q_heads / a.kv_heads;
  w.qt_first = sm.row_first / kTileM;
  w.qt_count = sm.row_first < sm.row_end ? (sm.row_end - 1) / kTileM - w.qt_first + 1 : 0;
  w.n_iter = w.qt_count * w.heads;
  if (w.n_iter == 0) {
    // no query sees this key tile: exactly zero gradients, no pipeline
    if (tid < kSoftmaxThreads && j0 + tid < a.k_len) {
      uint4* dvrow = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(a.dv) + batch * a.dv_strides[0] +
                                              kv_head * a.dv_strides[1] + static_cast<long long>(j0 + tid) * a.dv_strides[2]);
      uint4* dkrow = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(a.dk) + batch * a.dk_strides[0] +
                                              kv_head * a.dk_strides[1] + static_cast<long long>(j0 + tid) * a.dk_strides[2]);
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        dvrow[c] = make_uint4(0, 0, 0, 0);
        dkrow[c] = make_uint4(0, 0, 0, 0);
      }
    }
    return;
  }
  if (tid == 0) {
    ptx::mbar_init(&sm.kv_full, 1);
    ptx::mbar_init(&sm.kv_ready, kSoftmaxThreads);
    for (int s = 0; s < kBwdStages; ++s) {
      ptx::mbar_init(&sm.qg_full[s], 1);
      ptx::mbar_init(&sm.qg_empty[s], 1);
    }
    ptx::mbar_init(&sm.sdp_full, 1);
    ptx::mbar_init(&sm.pds_full, kSoftmaxThreads);
    ptx::mbar_init(&sm.mma_done, 1);
    ptx::mbar_init(&sm.dq_full, 1);
    ptx::mbar_init(&sm.dq_free, kSoftmaxThreads);
    ptx::mbar_fence_init();
  }
  if (warp == 4) {
    ptx::tmem_alloc(&sm.tmem_base, kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = sm.tmem_base;
  if (warp < 4) {
    bwd_compute(sm, a, tmem, w, delta, dq_acc, j0, kv_head, batch);
  } else if (warp == 4) {
    if (lane == 0) bwd_producer(sm, &map_q, &map_k, &map_v, &map_g, w, j0, kv_head, batch);
  } else {
    if (lane == 0) bwd_mma(sm, tmem, w);
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 4) ptx::tmem_dealloc(tmem, kTmemCols);
}
}  // namespace

// ---------------------------------------------------------------------------
// launchers

bool tc_fwd_supported(const wm_attn_args& a) {
  if (a.dtype != WM_BF16 || a.head_dim != kHeadDim) return false;
  if (a.mask == WM_MASK_PACKED || a.key_mask != nullptr) return false;
  if (!tma_ok(a.q, a.q_strides, a.batch, a.q_heads, a.q_len)) return false;
  if (!tma_ok(a.k, a.k_strides, a.batch, a.kv_heads, a.k_len)) return false;
  if (!tma_ok(a.v, a.v_strides, a.batch, a.kv_heads, a.k_len)) return false;
  if (reinterpret_cast<uintptr_t>(a.out) % 16) return false;
  for (int i = 0; i < 3; ++i)
    if (a.out_strides[i] % 8) return false;
  return true;
}

int tc_attn_fwd(const wm_attn_args& a, cudaStream_t stream) {
  CUtensorMap map_q, map_k, map_v;
  int status = make_map(&map_q, a.q, a.batch, a.q_heads, a.q_len, a.q_strides, kTileM);
  if (status != WM_OK) return status;
  status = make_map(&map_k, a.k, a.batch, a.kv_heads, a.k_len, a.k_strides, kTileN);
  if (status != WM_OK) return status;
  status = make_map(&map_v, a.v, a.batch, a.kv_heads, a.k_len, a.v_strides, kTileN);
  if (status != WM_OK) return status;
  const size_t smem = sizeof(FwdShared) + 1024;
  static bool configured = false;
  if (!configured) {
    WM_CUDA(cudaFuncSetAttribute(attn_fwd_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    configured = true;
  }
  dim3 grid((a.q_len + kTileM - 1) / kTileM, a.q_heads, a.batch);
  attn_fwd_tc_kernel<<<grid, kThreadsFwd, smem, stream>>>(map_q, map_k, map_v, a);
  count_launch();
  return cuda_check(cudaGetLastError(), "attn_fwd_tc_kernel");
}

int tc_device_status(bool reset) {
  int value = 0;
  if (cudaMemcpyFromSymbol(&value, g_status, sizeof(int)) != cudaSuccess) return -1;
  if (reset && value != 0) {
    int zero = 0;
    cudaMemcpyToSymbol(g_status, &zero, sizeof(int));
  }
  return value;
}

bool tc_bwd_supported(const wm_attn_args& a) {
  if (!tc_fwd_supported(a)) return false;
  if (a.dout == nullptr) return true;  // shape query before the tensors exist
  if (!tma_ok(a.dout, a.dout_strides, a.batch, a.q_heads, a.q_len)) return false;
  const void* ptrs[3] = {a.dq, a.dk, a.dv};
  const int64_t* strides[3] = {a.dq_strides, a.dk_strides, a.dv_strides};
  for (int n = 0; n < 3; ++n) {
    if (reinterpret_cast<uintptr_t>(ptrs[n]) % 16) return false;
    for (int i = 0; i < 3; ++i)
      if (strides[n][i] % 8) return false;
  }
  return true;
}

size_t tc_attn_bwd_workspace(const wm_attn_args& a) {
  const size_t rows = static_cast<size_t>(a.batch) * a.q_heads * a.q_len;
  return ((rows + 63) / 64) * 64 * sizeof(float) + rows * kHeadDim * sizeof(float);
}

int tc_attn_bwd(const wm_attn_args& a, cudaStream_t stream) {
  const size_t need = tc_attn_bwd_workspace(a);
  if (a.workspace == nullptr || a.workspace_bytes < need)
    return fail(WM_EWORKSPACE, "attention backward needs %zu workspace bytes, got %zu", need, a.workspace_bytes);
  const size_t rows = static_cast<size_t>(a.batch) * a.q_heads * a.q_len;
  float* delta = static_cast<float*>(a.workspace);
  float* dq_acc = delta + ((rows + 63) / 64) * 64;
  CUtensorMap map_q, map_k, map_v, map_g;
  int status = make_map(&map_q, a.q, a.batch, a.q_heads, a.q_len, a.q_strides, kTileM);
  if (status != WM_OK) return status;
  status = make_map(&map_k, a.k, a.batch, a.kv_heads, a.k_len, a.k_strides, kTileN);
  if (status != WM_OK) return status;
  status = make_map(&map_v, a.v, a.batch, a.kv_heads, a.k_len, a.v_strides, kTileN);
  if (status != WM_OK) return status;
  status = make_map(&map_g, a.dout, a.batch, a.q_heads, a.q_len, a.dout_strides, kTileM);
  if (status != WM_OK) return status;
  WM_CUDA(cudaMemsetAsync(dq_acc, 0, rows * kHeadDim * sizeof(float), stream));
  bwd_delta_kernel<<<static_cast<unsigned>((rows + 127) / 128), 128, 0, stream>>>(a, delta);
  count_launch();
  WM_CUDA(cudaGetLastError());
  const size_t smem = sizeof(BwdShared) + 1024;
  static bool configured = false;
  if (!configured) {
    WM_CUDA(cudaFuncSetAttribute(attn_bwd_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    configured = true;
  }
  dim3 grid((a.k_len + kTileN - 1) / kTileN, a.kv_heads, a.batch);
  attn_bwd_tc_kernel<<<grid, kThreadsFwd, smem, stream>>>(map_q, map_k, map_v, map_g, a, delta, dq_acc);
  count_launch();
  WM_CUDA(cudaGetLastError());
  const size_t chunks = rows * 8;
  bwd_dq_convert_kernel<<<static_cast<unsigned>((chunks + 255) / 256), 256, 0, stream>>>(a, dq_acc);
  count_launch();
  return cuda_check(cudaGetLastError(), "attention backward (tcgen05)");
}

}  // namespace wm
