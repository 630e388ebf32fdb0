// Forward pipeline, two blocks per SM (included by attn_tc.cu).
//
// Same roles as the first forward pipeline, but sized so that two blocks share
// an SM (98 KB of shared memory, 256 TMEM columns, <= 168 registers): while one
// block's softmax warps work on a tile, the other block's MMAs use the tensor
// cores, and every scheduler has two softmax warps to switch between.  Inside a
// block S, P and the V stage are single-buffered; the softmax reads S twice
// (row maximum first, exponentials second) instead of holding 128 scores per
// thread.
// TMEM: S [0,128), O [128,192); 256 columns allocated.
#pragma once

constexpr int kStages2 = 2;
constexpr uint32_t kTmemCols2 = 256;

struct Fwd2Shared {
  unsigned char q[kTileBytes];
  unsigned char k[kStages2][kTileBytes];
  unsigned char v[kTileBytes];
  unsigned char p[2 * kTileBytes];
  uint64_t q_full;
  uint64_t k_full[kStages2], k_empty[kStages2], v_full, v_empty;
  uint64_t s_full, p_full, pv_done, docs_full[2];
  int key_seg[2][kTileN];
  int key_end[2][kTileN];
  int tile_summary[2][4][3];
  int red_min_lo, red_max_hi, has_dummy;
  uint32_t tmem_base;
  int abort_flag;
  int epoch;
};

__device__ __forceinline__ void producer2(Fwd2Shared& sm, const CUtensorMap* map_q, const CUtensorMap* map_k,
                                          const CUtensorMap* map_v, const TileWalk& w, int q0, int head, int kv_head,
                                          int batch) {
  ptx::prefetch_tmap(map_q);
  ptx::prefetch_tmap(map_k);
  ptx::prefetch_tmap(map_v);
  ptx::mbar_expect_tx(&sm.q_full, kTileBytes);
  ptx::tma_load_4d(sm.q, map_q, &sm.q_full, 0, q0, head, batch);
  for (int n = 0; n < w.n_tiles; ++n) {
    const int s = n % kStages2;
    const int j0 = tile_first_key(n, w.first_tile, w.dummy_tile);
    if (!wait_or_abort(sm, &sm.k_empty[s], ((n / kStages2) & 1) ^ 1, 11)) return;
    ptx::mbar_expect_tx(&sm.k_full[s], kTileBytes);
    ptx::tma_load_4d(sm.k[s], map_k, &sm.k_full[s], 0, j0, kv_head, batch);
    if (!wait_or_abort(sm, &sm.v_empty, (n & 1) ^ 1, 12)) return;
    ptx::mbar_expect_tx(&sm.v_full, kTileBytes);
    ptx::tma_load_4d(sm.v, map_v, &sm.v_full, 0, j0, kv_head, batch);
  }
}

__device__ __forceinline__ bool issue_qk2(Fwd2Shared& sm, uint32_t tmem, int n) {
  const int s = n % kStages2;
  if (!wait_or_abort(sm, &sm.k_full[s], (n / kStages2) & 1, 21)) return false;
  ptx::tc_fence_after();
  constexpr uint32_t idesc = ptx::make_idesc_bf16(kTileM, kTileN, 0, 0);
  const uint32_t a_base = ptx::smem_u32(sm.q);
  const uint32_t b_base = ptx::smem_u32(sm.k[s]);
#pragma unroll
  for (int kk = 0; kk < kHeadDim / 16; ++kk)
    ptx::mma_bf16_ss(tmem, ptx::make_smem_desc_sw128(a_base + kk * 32, 16, 1024),
                     ptx::make_smem_desc_sw128(b_base + kk * 32, 16, 1024), idesc, kk > 0);
  ptx::mma_commit(&sm.k_empty[s]);
  ptx::mma_commit(&sm.s_full);
  return true;
}

__device__ __forceinline__ void mma2(Fwd2Shared& sm, uint32_t tmem, const TileWalk& w) {
  if (!wait_or_abort(sm, &sm.q_full, 0, 20)) return;
  if (!issue_qk2(sm, tmem, 0)) return;
  constexpr uint32_t idesc_pv = ptx::make_idesc_bf16(kTileM, kHeadDim, 0, 1);
  const uint32_t o_tmem = tmem + kTileN;
  const uint32_t p_base = ptx::smem_u32(sm.p);
  const uint32_t v_base = ptx::smem_u32(sm.v);
  for (int n = 0; n < w.n_tiles; ++n) {
    // P(n) complete means the softmax no longer needs S(n)
    if (!wait_or_abort(sm, &sm.p_full, n & 1, 22)) return;
    if (n + 1 < w.n_tiles && !issue_qk2(sm, tmem, n + 1)) return;
    if (!wait_or_abort(sm, &sm.v_full, n & 1, 23)) return;
    ptx::tc_fence_after();
#pragma unroll
    for (int kk = 0; kk < kTileN / 16; ++kk)
      ptx::mma_bf16_ss(o_tmem, ptx::make_smem_desc_sw128(p_base + (kk >> 2) * kTileBytes + (kk & 3) * 32, 16, 1024),
                       ptx::make_smem_desc_sw128(v_base + kk * 2048, 1024, 1024), idesc_pv, (n > 0) || (kk > 0));
    ptx::mma_commit(&sm.v_empty);
    ptx::mma_commit(&sm.pv_done);
  }
}

// How a key tile relates to one query row.
enum TileClass { kTileNone = 0, kTileFull = 1, kTileCausal = 2, kTileDocs = 3 };

// 32 scores of this thread's row -> masked scores (raw units), -inf where invisible.
__device__ __forceinline__ void mask_chunk(const uint32_t (&raw)[32], float (&x)[32], int cls, int c, int lim,
                                           const RowBound& rb, int j0, const int* key_seg, const int* key_end) {
  if (cls == kTileFull) {
#pragma unroll
    for (int e = 0; e < 32; ++e) x[e] = __uint_as_float(raw[e]);
  } else if (cls == kTileNone) {
#pragma unroll
    for (int e = 0; e < 32; ++e) x[e] = -INFINITY;
  } else if (cls == kTileCausal) {
#pragma unroll
    for (int e = 0; e < 32; ++e) x[e] = c * 32 + e < lim ? __uint_as_float(raw[e]) : -INFINITY;
  } else {
#pragma unroll
    for (int e = 0; e < 32; e += 4) {
      const int col = c * 32 + e;
      const int4 sg = *reinterpret_cast<const int4*>(key_seg + col);
      const int4 en = *reinterpret_cast<const int4*>(key_end + col);
      const int segs[4] = {sg.x, sg.y, sg.z, sg.w}, ends[4] = {en.x, en.y, en.z, en.w};
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const bool vis = (col + u < lim) & doc_visible_flat(rb, j0 + col + u, segs[u], ends[u]);
        x[e + u] = vis ? __uint_as_float(raw[e + u]) : -INFINITY;
      }
    }
  }
}

__device__ __forceinline__ void softmax2(Fwd2Shared& sm, const wm_attn_args& a, uint32_t tmem, const TileWalk& w,
                                         const RowBound& rb, bool live, int batch, int head, int dbg) {
  const int t = threadIdx.x;
  const int warp = t >> 5, lane = t & 31;
  const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
  const float sl2 = a.scale * kLog2e;
  const bool docs = a.q_seg != nullptr;
  float m_ref = -INFINITY, l = 0.f;
  const uint32_t s_tmem = tmem + lane_base;
  const uint32_t o_tmem = tmem + kTileN + lane_base;
  unsigned char* prow = sm.p + (t >> 3) * 1024 + (t & 7) * 128;
  // document id / query bound of key slot (tile start + t), loaded one tile ahead of its use
  int next_seg = INT_MIN, next_end = 0;
  auto fetch_key_docs = [&](int n) {
    next_seg = INT_MIN;
    next_end = 0;
    if (docs && n < w.n_tiles) {
      const int j = tile_first_key(n, w.first_tile, w.dummy_tile) + t;
      if (j < a.k_len) {
        const long long at = static_cast<long long>(batch) * a.k_len + j;
        if (dbg & 1) {
          next_seg = 0;
          next_end = INT_MAX;
        } else {
          next_seg = __ldg(a.k_seg + at);
          next_end = __ldg(a.k_query_end + at);
        }
      }
    }
  };
  fetch_key_docs(0);

  for (int n = 0; n < w.n_tiles; ++n) {
    const int b = n & 1;
    const int j0 = tile_first_key(n, w.first_tile, w.dummy_tile);
    int cls = !live || j0 >= rb.hi ? kTileNone : (j0 + kTileN <= rb.hi ? kTileFull : kTileCausal);
    if (docs) {
      const int seg = next_seg, end = next_end;
      fetch_key_docs(n + 1);
      sm.key_seg[b][t] = seg;
      sm.key_end[b][t] = end;
      const int smin = __reduce_min_sync(0xffffffffu, seg);
      const int smax = __reduce_max_sync(0xffffffffu, seg);
      const int emin = __reduce_min_sync(0xffffffffu, end);
      if (lane == 0) {
        sm.tile_summary[b][warp][0] = smin;
        sm.tile_summary[b][warp][1] = smax;
        sm.tile_summary[b][warp][2] = emin;
      }
      if (!(dbg & 2)) {
        ptx::mbar_arrive(&sm.docs_full[b]);
        if (!wait_or_abort(sm, &sm.docs_full[b], (n >> 1) & 1, 30)) return;
      }
      if (cls != kTileNone && !(dbg & 4)) {
        int tmin = sm.tile_summary[b][0][0], tmax = sm.tile_summary[b][0][1], tend = sm.tile_summary[b][0][2];
#pragma unroll
        for (int q = 1; q < 4; ++q) {
          tmin = min(tmin, sm.tile_summary[b][q][0]);
          tmax = max(tmax, sm.tile_summary[b][q][1]);
          tend = min(tend, sm.tile_summary[b][q][2]);
        }
        // a tile that lies inside the row's own document needs the causal bound at most
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
    if (!wait_or_abort(sm, &sm.s_full, n & 1, 31)) return;
    ptx::tc_fence_after();
    // pass 1: row maximum
    float top = -INFINITY;
    if (__any_sync(0xffffffffu, cls != kTileNone) && !(dbg & 8)) {
      float t0 = -INFINITY, t1 = -INFINITY, t2 = -INFINITY, t3 = -INFINITY;
      uint32_t raw[2][32];
      ptx::tmem_ld32(s_tmem, raw[0]);
#pragma unroll
      for (int c = 0; c < kTileN / 32; ++c) {
        ptx::tmem_wait_ld();
        if (c + 1 < kTileN / 32) ptx::tmem_ld32(s_tmem + (c + 1) * 32, raw[(c + 1) & 1]);  // in flight during the math
        float x[32];
        mask_chunk(raw[c & 1], x, cls, c, lim, rb, j0, sm.key_seg[b], sm.key_end[b]);
#pragma unroll
        for (int e = 0; e < 32; e += 8) {
          t0 = fmax3(t0, x[e], x[e + 1]);
          t1 = fmax3(t1, x[e + 2], x[e + 3]);
          t2 = fmax3(t2, x[e + 4], x[e + 5]);
          t3 = fmax3(t3, x[e + 6], x[e + 7]);
        }
      }
      top = fmaxf(fmaxf(t0, t1), fmaxf(t2, t3)) * sl2;
    }
    float corr = 1.f;
    bool moved = false;
    if (top > m_ref + kRescaleThreshold || (m_ref == -INFINITY && top > -INFINITY)) {
      moved = m_ref != -INFINITY;
      corr = moved ? fast_exp2(m_ref - top) : 1.f;
      m_ref = top;
      l *= corr;
    }
    const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
    // P and O belong to the PV product of the previous tile until it completes
    if (n >= 1 && !wait_or_abort(sm, &sm.pv_done, (n - 1) & 1, 32)) return;
    ptx::tc_fence_after();
    // pass 2: exponentials -> P
    if (!(dbg & 16)) {
      float2 s0 = make_float2(0.f, 0.f), s1 = make_float2(0.f, 0.f);
      const float2 sc = make_float2(sl2, sl2), nm = make_float2(-m_use, -m_use);
      uint32_t raw[2][32];
      ptx::tmem_ld32(s_tmem, raw[0]);
#pragma unroll
      for (int c = 0; c < kTileN / 32; ++c) {
        ptx::tmem_wait_ld();
        if (c + 1 < kTileN / 32) ptx::tmem_ld32(s_tmem + (c + 1) * 32, raw[(c + 1) & 1]);
        float x[32];
        mask_chunk(raw[c & 1], x, cls, c, lim, rb, j0, sm.key_seg[b], sm.key_end[b]);
        uint32_t pk[16];
#pragma unroll
        for (int e = 0; e < 32; e += 4) {
          // two scores per packed fp32x2 instruction
          float2 a = __ffma2_rn(make_float2(x[e], x[e + 1]), sc, nm);
          float2 d = __ffma2_rn(make_float2(x[e + 2], x[e + 3]), sc, nm);
          a.x = fast_exp2(a.x);
          a.y = fast_exp2(a.y);
          d.x = fast_exp2(d.x);
          d.y = fast_exp2(d.y);
          s0 = __fadd2_rn(s0, a);
          s1 = __fadd2_rn(s1, d);
          pk[e / 2] = pack_bf16(a.x, a.y);
          pk[e / 2 + 1] = pack_bf16(d.x, d.y);
        }
        const int sub = (c >> 1) * kTileBytes;
#pragma unroll
        for (int u = 0; u < 4; ++u)
          *reinterpret_cast<uint4*>(prow + sub + ((((c & 1) * 4 + u) ^ (t & 7)) << 4)) =
              make_uint4(pk[4 * u], pk[4 * u + 1], pk[4 * u + 2], pk[4 * u + 3]);
      }
      const float s2 = s0.x + s0.y, s3 = s1.x + s1.y;
      const float s0s = 0.f, s1s = 0.f;
      (void)s0s;
      (void)s1s;
      l += s2 + s3;
    }
    if (__any_sync(0xffffffffu, moved)) {
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
    if (n == w.n_tiles - 1 && w.kmax < j0 + kTileN) {
      if (!wait_or_abort(sm, &sm.v_full, n & 1, 34)) return;
      if (j0 + t >= w.kmax) {
        uint4* vrow = reinterpret_cast<uint4*>(sm.v + t * 128);
#pragma unroll
        for (int c = 0; c < 8; ++c) vrow[c] = make_uint4(0, 0, 0, 0);
      }
    }
    ptx::fence_async_shared();
    ptx::tc_fence_before();
    ptx::mbar_arrive(&sm.p_full);
  }
  const int last = w.n_tiles - 1;
  if (!wait_or_abort(sm, &sm.pv_done, last & 1, 35)) return;
  ptx::tc_fence_after();
  const float inv = l > 0.f ? 1.f / l : 0.f;
  __nv_bfloat16* orow = static_cast<__nv_bfloat16*>(a.out) + batch * a.out_strides[0] + head * a.out_strides[1] +
                        static_cast<long long>(rb.qi) * a.out_strides[2];
#pragma unroll
  for (int c = 0; c < kHeadDim / 32; ++c) {
    uint32_t raw[32];
    ptx::tmem_ld32(o_tmem + c * 32, raw);
    ptx::tmem_wait_ld();
    if (live) {
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        uint32_t pk[4];
#pragma unroll
        for (int e = 0; e < 4; ++e)
          pk[e] = l > 0.f ? pack_bf16(__uint_as_float(raw[8 * u + 2 * e]) * inv, __uint_as_float(raw[8 * u + 2 * e + 1]) * inv)
                          : 0u;
        reinterpret_cast<uint4*>(orow)[c * 4 + u] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
      }
    }
  }
  if (live && a.lse != nullptr)
    a.lse[(static_cast<long long>(batch) * a.q_heads + head) * a.q_len + rb.qi] =
        l > 0.f ? (m_ref + log2f(l)) * kLn2 : INFINITY;
}


__global__ void __launch_bounds__(kThreadsFwd, 2)
    attn_fwd_tc2_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                        const __grid_constant__ CUtensorMap map_v, const wm_attn_args a, const int epoch,
                        const int dbg) {
  extern __shared__ unsigned char smem_raw[];
  Fwd2Shared& sm = *reinterpret_cast<Fwd2Shared*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
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
    for (int s = 0; s < kStages2; ++s) {
      ptx::mbar_init(&sm.k_full[s], 1);
      ptx::mbar_init(&sm.k_empty[s], 1);
    }
    ptx::mbar_init(&sm.v_full, 1);
    ptx::mbar_init(&sm.v_empty, 1);
    ptx::mbar_init(&sm.s_full, 1);
    ptx::mbar_init(&sm.p_full, kSoftmaxThreads);
    ptx::mbar_init(&sm.pv_done, 1);
    ptx::mbar_init(&sm.docs_full[0], kSoftmaxThreads);
    ptx::mbar_init(&sm.docs_full[1], kSoftmaxThreads);
    ptx::mbar_fence_init();
  }
  if (warp == 4) {
    ptx::tmem_alloc(&sm.tmem_base, kTmemCols2);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = sm.tmem_base;

  if (warp < 4) {
    softmax2(sm, a, tmem, w, rb, live, batch, head, dbg);
  } else if (warp == 4) {
    if (lane == 0) producer2(sm, &map_q, &map_k, &map_v, w, q0, head, kv_head, batch);
  } else {
    if (lane == 0) mma2(sm, tmem, w);
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 4) ptx::tmem_dealloc(tmem, kTmemCols2);
}
