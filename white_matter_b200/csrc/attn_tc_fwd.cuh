// Forward pipeline of the tcgen05 attention kernel (included by attn_tc.cu).
#pragma once

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
  int epoch;
  int trace_on, trace_n;
  long long trace[kTraceSlots];
};

// ------------------------------------------------------------------ producer (one lane of warp 4)
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

// ------------------------------------------------------------------ MMA issuer (one lane of warp 5)
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
    bool own_doc = !docs;
    if (docs && !none) {
      int smin = sm.tile_summary[b][0][0], smax = sm.tile_summary[b][0][1], emin = sm.tile_summary[b][0][2];
#pragma unroll
      for (int q = 1; q < 4; ++q) {
        smin = min(smin, sm.tile_summary[b][q][0]);
        smax = max(smax, sm.tile_summary[b][q][1]);
        emin = min(emin, sm.tile_summary[b][q][2]);
      }
      const bool uniform = smin == smax;
      own_doc = uniform && smin == rb.seg && j0 >= rb.lo && emin > rb.qi;
      full = full && own_doc;
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
    } else if (own_doc) {
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
  trace_flush(sm);
  if (warp == 4) ptx::tmem_dealloc(tmem, kTmemCols);
}


