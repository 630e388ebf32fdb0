// Forward pipeline of the tcgen05 attention kernel (included by attn_tc.cu).
//
// One block owns 128 query rows of one (batch, head) and walks over tiles of 128 key slots.
// 320 threads: warps 0-7 softmax, warp 8 TMA producer (Q once, K and V through 3-deep rings,
// per-block loads, no multicast), warp 9 issues tcgen05.mma: S = Q K^T into one of two TMEM
// buffers, O += P V into a third; completion is signalled by tcgen05.commit on mbarriers.
// Softmax thread t owns query row (t & 127) and the 64-column half (t >> 7) of every 128-key
// tile, keeps 64 scores in registers and reads S once; the two halves of a row exchange their
// partial row maximum through shared memory (one bounded 256-thread barrier per tile) and take
// the same lazy-rescale decision; their partial row sums are added once, in the epilogue.
// P is written as bf16 into the K-major 128B-swizzled shared layout that the MMA reads.
// TMEM: S0 [0,128), S1 [128,256), O [256,320) columns; 512 allocated.
#pragma once

// ------------------------------------------------------------------ producer (one lane of the producer warp)
template <class Shared>
__device__ __forceinline__ void producer_role(Shared& sm, const CUtensorMap* map_q, const CUtensorMap* map_k,
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
    trace_event(sm, 100 + n);
    if (!wait_or_abort(sm, &sm.v_empty[s], parity, 12)) return;
    ptx::mbar_expect_tx(&sm.v_full[s], kTileBytes);
    ptx::tma_load_4d(sm.v[s], map_v, &sm.v_full[s], 0, j0, kv_head, batch);
    trace_event(sm, 200 + n);
  }
}

// ------------------------------------------------------------------ MMA issuer (one lane of the MMA warp)
template <class Shared>
__device__ __forceinline__ bool issue_qk(Shared& sm, uint32_t tmem, int n) {
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
  trace_event(sm, 400 + n);
  return true;
}

template <class Shared>
__device__ __forceinline__ void mma_role(Shared& sm, uint32_t tmem, const TileWalk& w) {
  if (!wait_or_abort(sm, &sm.q_full, 0, 20)) return;
  if (!issue_qk(sm, tmem, 0)) return;
  constexpr uint32_t idesc_pv = ptx::make_idesc_bf16(kTileM, kHeadDim, 0, 1);
  const uint32_t o_tmem = tmem + 2 * kTileN;
  for (int n = 0; n < w.n_tiles; ++n) {
    if (n + 1 < w.n_tiles && !issue_qk(sm, tmem, n + 1)) return;
    const int b = n & 1;
    const int s = n % kStages;
    if (!wait_or_abort(sm, &sm.p_full[b], (n >> 1) & 1, 22)) return;
    trace_event(sm, 300 + n);
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
    trace_event(sm, 500 + n);
  }
}


constexpr int kFwdThreads = 320;
constexpr int kFwdSoftmax = 256;

struct FwdShared {
  unsigned char q[kTileBytes];
  unsigned char k[kStages][kTileBytes];
  unsigned char v[kStages][kTileBytes];
  unsigned char p[2][2 * kTileBytes];
  uint64_t q_full;
  uint64_t k_full[kStages], k_empty[kStages], v_full[kStages], v_empty[kStages];
  uint64_t s_full[2], p_full[2], pv_done[2], docs_full[2], max_full[2], sum_full;
  int key_seg[2][kTileN];
  int key_end[2][kTileN];
  int tile_summary[2][4][3];
  float row_max[2][2][kTileM];
  float row_sum[2][kTileM];
  int red_min_lo, red_max_hi, has_dummy;
  uint32_t tmem_base;
  int abort_flag;
  int epoch;
  int trace_on, trace_n;
  long long trace[kTraceSlots];
};

__device__ __forceinline__ void softmax_role(FwdShared& sm, const wm_attn_args& a, uint32_t tmem, const TileWalk& w,
                                         const RowBound& rb, bool live, int batch, int head) {
  const int t = threadIdx.x;
  const int row = t & 127;
  const int half = t >> 7;
  const int warp = t >> 5, lane = t & 31;
  const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
  const float sl2 = a.scale * kLog2e;
  const bool docs = a.q_seg != nullptr;
  float m_ref = -INFINITY, l = 0.f;
  const uint32_t o_tmem = tmem + 2 * kTileN + lane_base + half * 32;

  // document id / query bound of key slot (tile start + row), loaded one tile ahead (half 0 publishes them)
  int next_seg = INT_MIN, next_end = 0;
  auto fetch_key_docs = [&](int n) {
    next_seg = INT_MIN;
    next_end = 0;
    if (docs && half == 0 && n < w.n_tiles) {
      const int j = tile_first_key(n, w.first_tile, w.dummy_tile) + row;
      if (j < a.k_len) {
        const long long at = static_cast<long long>(batch) * a.k_len + j;
        next_seg = __ldg(a.k_seg + at);
        next_end = __ldg(a.k_query_end + at);
      }
    }
  };
  fetch_key_docs(0);
  const int tbase = row == 0 ? (half ? 10000 : 0) : -1;  // rows 0 of both halves leave a trace
#define WM_TRACE(tag) if (tbase >= 0) trace_event(sm, tbase + (tag))

  for (int n = 0; n < w.n_tiles; ++n) {
    const int b = n & 1;
    const int j0 = tile_first_key(n, w.first_tile, w.dummy_tile);
    int cls = !live || j0 >= rb.hi ? kTileNone : (j0 + kTileN <= rb.hi ? kTileFull : kTileCausal);
    if (docs) {
      if (half == 0) {
        const int seg = next_seg, end = next_end;
        sm.key_seg[b][row] = seg;
        sm.key_end[b][row] = end;
        const int smin = __reduce_min_sync(0xffffffffu, seg);
        const int smax = __reduce_max_sync(0xffffffffu, seg);
        const int emin = __reduce_min_sync(0xffffffffu, end);
        if (lane == 0) {
          sm.tile_summary[b][warp][0] = smin;
          sm.tile_summary[b][warp][1] = smax;
          sm.tile_summary[b][warp][2] = emin;
        }
      }
      fetch_key_docs(n + 1);
      ptx::mbar_arrive(&sm.docs_full[b]);
      if (!wait_or_abort(sm, &sm.docs_full[b], (n >> 1) & 1, 30)) return;
      if (cls != kTileNone) {
        int tmin = sm.tile_summary[b][0][0], tmax = sm.tile_summary[b][0][1], tend = sm.tile_summary[b][0][2];
#pragma unroll
        for (int q = 1; q < 4; ++q) {
          tmin = min(tmin, sm.tile_summary[b][q][0]);
          tmax = max(tmax, sm.tile_summary[b][q][1]);
          tend = min(tend, sm.tile_summary[b][q][2]);
        }
        const bool uniform = tmin == tmax;
        const bool own_doc = uniform && tmin == rb.seg && j0 >= rb.lo && tend > rb.qi;
        if (uniform && tmin != -1 && tmin != rb.seg) {
          cls = kTileNone;
        } else if (!own_doc) {
          cls = kTileDocs;
        }
      }
    }
    const int lim = rb.hi - j0;
    if (!wait_or_abort(sm, &sm.s_full[b], (n >> 1) & 1, 31)) return;
    ptx::tc_fence_after();
    WM_TRACE(600 + n);
    // this thread's 64 scores
    float x[64];
    {
      const uint32_t s_tmem = tmem + static_cast<uint32_t>(b) * kTileN + lane_base + half * 64;
      uint32_t raw0[32], raw1[32];
      ptx::tmem_ld32(s_tmem, raw0);
      ptx::tmem_ld32(s_tmem + 32, raw1);
      ptx::tmem_wait_ld();
      WM_TRACE(650 + n);
      // visibility of 32 columns as a bit mask: arithmetic for the causal bound, a short loop over the key table
      // for tiles that contain a document boundary; one copy of the select serves every tile class
      const int lim_eff = cls == kTileFull ? kTileN : (cls == kTileNone ? 0 : lim);
      auto visible_mask = [&](int col0) -> uint32_t {
        const int left = lim_eff - col0;
        uint32_t mask = left >= 32 ? 0xffffffffu : (left <= 0 ? 0u : ((1u << left) - 1u));
        if (cls == kTileDocs && mask != 0u) {
          uint32_t docs_mask = 0u;
#pragma unroll 1
          for (int e = 0; e < 32; ++e) {
            const int col = col0 + e;
            docs_mask |= static_cast<uint32_t>(doc_visible_flat(rb, j0 + col, sm.key_seg[b][col], sm.key_end[b][col])) << e;
          }
          mask &= docs_mask;
        }
        return mask;
      };
      const uint32_t m0 = visible_mask(half * 64), m1 = visible_mask(half * 64 + 32);
#pragma unroll
      for (int e = 0; e < 32; ++e) {
        x[e] = (m0 >> e) & 1u ? __uint_as_float(raw0[e]) : -INFINITY;
        x[32 + e] = (m1 >> e) & 1u ? __uint_as_float(raw1[e]) : -INFINITY;
      }
    }
    float t0 = -INFINITY, t1 = -INFINITY, t2 = -INFINITY, t3 = -INFINITY;
#pragma unroll
    for (int e = 0; e < 64; e += 8) {
      t0 = fmax3(t0, x[e], x[e + 1]);
      t1 = fmax3(t1, x[e + 2], x[e + 3]);
      t2 = fmax3(t2, x[e + 4], x[e + 5]);
      t3 = fmax3(t3, x[e + 6], x[e + 7]);
    }
    const float mine = fmaxf(fmaxf(t0, t1), fmaxf(t2, t3));
    sm.row_max[b][half][row] = mine;
    WM_TRACE(700 + n);
    ptx::mbar_arrive(&sm.max_full[b]);
    if (!wait_or_abort(sm, &sm.max_full[b], (n >> 1) & 1, 36)) return;
    WM_TRACE(800 + n);
    const float top = fmaxf(mine, sm.row_max[b][half ^ 1][row]) * sl2;
    // both halves of a row see the same numbers and take the same decision
    float corr = 1.f;
    bool moved = false;
    if (top > m_ref + kRescaleThreshold || (m_ref == -INFINITY && top > -INFINITY)) {
      moved = m_ref != -INFINITY;
      corr = moved ? fast_exp2(m_ref - top) : 1.f;
      m_ref = top;
      l *= corr;
    }
    const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
    // the P buffer was last read by the PV product of tile n-2
    if (n >= 2 && !wait_or_abort(sm, &sm.pv_done[b], ((n - 2) >> 1) & 1, 32)) return;
    {
      unsigned char* prow = sm.p[b] + half * kTileBytes + (row >> 3) * 1024 + (row & 7) * 128;
      float2 s0 = make_float2(0.f, 0.f), s1 = make_float2(0.f, 0.f);
      const float2 sc = make_float2(sl2, sl2), nm = make_float2(-m_use, -m_use);
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        float2 u0 = __ffma2_rn(make_float2(x[8 * c], x[8 * c + 1]), sc, nm);
        float2 u1 = __ffma2_rn(make_float2(x[8 * c + 2], x[8 * c + 3]), sc, nm);
        float2 u2 = __ffma2_rn(make_float2(x[8 * c + 4], x[8 * c + 5]), sc, nm);
        float2 u3 = __ffma2_rn(make_float2(x[8 * c + 6], x[8 * c + 7]), sc, nm);
        u0.x = fast_exp2(u0.x);
        u0.y = fast_exp2(u0.y);
        u1.x = fast_exp2(u1.x);
        u1.y = fast_exp2(u1.y);
        u2.x = fast_exp2(u2.x);
        u2.y = fast_exp2(u2.y);
        u3.x = fast_exp2(u3.x);
        u3.y = fast_exp2(u3.y);
        s0 = __fadd2_rn(s0, __fadd2_rn(u0, u1));
        s1 = __fadd2_rn(s1, __fadd2_rn(u2, u3));
        *reinterpret_cast<uint4*>(prow + ((c ^ (row & 7)) << 4)) =
            make_uint4(pack_bf16(u0.x, u0.y), pack_bf16(u1.x, u1.y), pack_bf16(u2.x, u2.y), pack_bf16(u3.x, u3.y));
      }
      l += (s0.x + s0.y) + (s1.x + s1.y);
    }
    WM_TRACE(900 + n);
    // rescale O when a row of this warp moved its reference (O is complete after the PV product of tile n-1)
    if (__any_sync(0xffffffffu, moved)) {
      if (n >= 1 && !wait_or_abort(sm, &sm.pv_done[(n - 1) & 1], ((n - 1) >> 1) & 1, 33)) return;
      ptx::tc_fence_after();
      uint32_t raw[32];
      ptx::tmem_ld32(o_tmem, raw);
      ptx::tmem_wait_ld();
#pragma unroll
      for (int e = 0; e < 32; ++e) raw[e] = __float_as_uint(__uint_as_float(raw[e]) * corr);
      ptx::tmem_st32(o_tmem, raw);
      ptx::tmem_wait_st();
    }
    // last tile: value rows at or beyond the largest visible slot may hold anything (unused cache capacity)
    if (n == w.n_tiles - 1 && w.kmax < j0 + kTileN) {
      const int s = n % kStages;
      if (!wait_or_abort(sm, &sm.v_full[s], (n / kStages) & 1, 34)) return;
      if (half == 0 && j0 + row >= w.kmax) {
        uint4* vrow = reinterpret_cast<uint4*>(sm.v[s] + row * 128);
#pragma unroll
        for (int c = 0; c < 8; ++c) vrow[c] = make_uint4(0, 0, 0, 0);
      }
    }
    ptx::fence_async_shared();
    ptx::tc_fence_before();
    WM_TRACE(950 + n);
    ptx::mbar_arrive(&sm.p_full[b]);
    WM_TRACE(1000 + n);
  }
  // epilogue: add the two partial row sums, then O / l -> bf16 (32 columns per thread) and the log-sum-exp
  const int last = w.n_tiles - 1;
  sm.row_sum[half][row] = l;
  ptx::mbar_arrive(&sm.sum_full);
  if (!wait_or_abort(sm, &sm.sum_full, 0, 37)) return;
  l += sm.row_sum[half ^ 1][row];
  if (!wait_or_abort(sm, &sm.pv_done[last & 1], (last >> 1) & 1, 35)) return;
  ptx::tc_fence_after();
  const float inv = l > 0.f ? 1.f / l : 0.f;
  uint32_t raw[32];
  ptx::tmem_ld32(o_tmem, raw);
  ptx::tmem_wait_ld();
  if (live) {
    __nv_bfloat16* orow = static_cast<__nv_bfloat16*>(a.out) + batch * a.out_strides[0] + head * a.out_strides[1] +
                          static_cast<long long>(rb.qi) * a.out_strides[2] + half * 32;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      uint32_t pk[4];
#pragma unroll
      for (int e = 0; e < 4; ++e)
        pk[e] = l > 0.f ? pack_bf16(__uint_as_float(raw[8 * u + 2 * e]) * inv, __uint_as_float(raw[8 * u + 2 * e + 1]) * inv)
                        : 0u;
      reinterpret_cast<uint4*>(orow)[u] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
    }
    if (half == 0 && a.lse != nullptr)
      a.lse[(static_cast<long long>(batch) * a.q_heads + head) * a.q_len + rb.qi] =
          l > 0.f ? (m_ref + log2f(l)) * kLn2 : INFINITY;
  }
}

__global__ void __launch_bounds__(kFwdThreads, 1)
    attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                        const __grid_constant__ CUtensorMap map_v, const wm_attn_args a, const int epoch) {
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
    sm.epoch = epoch;
    trace_begin(sm, epoch);
    sm.has_dummy = a.q_seg != nullptr && a.k_seg[static_cast<long long>(batch) * a.k_len] == -1;
  }
  __syncthreads();
  RowBound rb;
  rb.lo = 0;
  rb.hi = 0;
  rb.seg = 0;
  rb.qi = q0 + (tid & 127);
  bool live = false;
  if (tid < kFwdSoftmax) {
    live = rb.qi < a.q_len;
    if (live) rb = row_bound(a, g, batch, rb.qi);
    const int lo = live && rb.hi > 0 ? rb.lo : INT_MAX;
    const int wlo = __reduce_min_sync(0xffffffffu, lo);
    const int whi = __reduce_max_sync(0xffffffffu, rb.hi);
    if (lane == 0 && tid < kTileM) {
      atomicMin(&sm.red_min_lo, wlo);
      atomicMax(&sm.red_max_hi, whi);
    }
  }
  __syncthreads();
  TileWalk w;
  w.kmax = sm.red_max_hi;
  if (w.kmax == 0) {
    if (live) {
      __nv_bfloat16* orow = static_cast<__nv_bfloat16*>(a.out) + batch * a.out_strides[0] + head * a.out_strides[1] +
                            static_cast<long long>(rb.qi) * a.out_strides[2] + (tid >> 7) * 32;
#pragma unroll
      for (int c = 0; c < 4; ++c) reinterpret_cast<uint4*>(orow)[c] = make_uint4(0, 0, 0, 0);
      if (tid < kTileM && a.lse != nullptr)
        a.lse[(static_cast<long long>(batch) * a.q_heads + head) * a.q_len + rb.qi] = INFINITY;
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
      ptx::mbar_init(&sm.p_full[b], kFwdSoftmax);
      ptx::mbar_init(&sm.pv_done[b], 1);
      ptx::mbar_init(&sm.docs_full[b], kFwdSoftmax);
      ptx::mbar_init(&sm.max_full[b], kFwdSoftmax);
    }
    ptx::mbar_init(&sm.sum_full, kFwdSoftmax);
    ptx::mbar_fence_init();
  }
  if (warp == 8) {
    ptx::tmem_alloc(&sm.tmem_base, kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = sm.tmem_base;

  if (warp < 8) {
    softmax_role(sm, a, tmem, w, rb, live, batch, head);
  } else if (warp == 8) {
    if (lane == 0) producer_role(sm, &map_q, &map_k, &map_v, w, q0, head, kv_head, batch);
  } else {
    if (lane == 0) mma_role(sm, tmem, w);
  }
  ptx::tc_fence_before();
  __syncthreads();
  trace_flush(sm);
  if (warp == 8) ptx::tmem_dealloc(tmem, kTmemCols);
}
