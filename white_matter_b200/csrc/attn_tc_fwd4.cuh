// Forward pipeline with two independent softmax warpgroups (included by attn_tc.cu).
//
// Warpgroup g (warps 4g..4g+3, thread = query row) owns the key tiles g, g+2, g+4, ...
// of the walk, with its own S buffer (TMEM), P buffer (shared memory), online-softmax
// state and O accumulator (TMEM).  The two streams never synchronise inside the loop,
// so the load / maximum / store / barrier phases of one overlap the exponentials of
// the other on every scheduler; the epilogue merges the two partial results
// (O_0 e^{m_0-m} + O_1 e^{m_1-m}) / (l_0 e^{m_0-m} + l_1 e^{m_1-m}).
// A thread reads its S row twice from TMEM (row maximum, then exponentials) instead of
// holding 128 scores in registers.
// TMEM: S0 [0,128) S1 [128,256) O0 [256,320) O1 [320,384); 512 columns allocated.
#pragma once

constexpr int kFwd4Threads = 320;

struct Fwd4Shared {
  unsigned char q[kTileBytes];
  unsigned char k[kStages][kTileBytes];
  unsigned char v[kStages][kTileBytes];
  unsigned char p[2][2 * kTileBytes];
  uint64_t q_full;
  uint64_t k_full[kStages], k_empty[kStages], v_full[kStages], v_empty[kStages];
  uint64_t s_full[2], p_full[2], pv_done[2], docs_full[2], merge_full;
  int key_seg[2][kTileN];
  int key_end[2][kTileN];
  int tile_summary[2][4][3];
  float part_m[2][kTileM];
  float part_l[2][kTileM];
  int red_min_lo, red_max_hi, has_dummy;
  uint32_t tmem_base;
  int abort_flag;
  int epoch;
  int trace_on, trace_n;
  long long trace[kTraceSlots];
};

// MMA issuer: as in the first pipeline, but tile n accumulates into O[n & 1].
__device__ __forceinline__ void mma4(Fwd4Shared& sm, uint32_t tmem, const TileWalk& w) {
  if (!wait_or_abort(sm, &sm.q_full, 0, 20)) return;
  if (!issue_qk(sm, tmem, 0)) return;
  constexpr uint32_t idesc_pv = ptx::make_idesc_bf16(kTileM, kHeadDim, 0, 1);
  for (int n = 0; n < w.n_tiles; ++n) {
    if (n + 1 < w.n_tiles && !issue_qk(sm, tmem, n + 1)) return;
    const int b = n & 1;
    const int s = n % kStages;
    if (!wait_or_abort(sm, &sm.p_full[b], (n >> 1) & 1, 22)) return;
    if (!wait_or_abort(sm, &sm.v_full[s], (n / kStages) & 1, 23)) return;
    ptx::tc_fence_after();
    const uint32_t o_tmem = tmem + 2 * kTileN + b * kHeadDim;
    const uint32_t p_base = ptx::smem_u32(sm.p[b]);
    const uint32_t v_base = ptx::smem_u32(sm.v[s]);
#pragma unroll
    for (int kk = 0; kk < kTileN / 16; ++kk)
      ptx::mma_bf16_ss(o_tmem, ptx::make_smem_desc_sw128(p_base + (kk >> 2) * kTileBytes + (kk & 3) * 32, 16, 1024),
                       ptx::make_smem_desc_sw128(v_base + kk * 2048, 1024, 1024), idesc_pv, (n >= 2) || (kk > 0));
    ptx::mma_commit(&sm.v_empty[s]);
    ptx::mma_commit(&sm.pv_done[b]);
  }
}

__device__ __forceinline__ void softmax4(Fwd4Shared& sm, const wm_attn_args& a, uint32_t tmem, const TileWalk& w,
                                         const RowBound& rb, bool live, int batch, int head) {
  const int row = threadIdx.x & 127;
  const int g = threadIdx.x >> 7;  // warpgroup == S / P / O buffer
  const int warp = (threadIdx.x >> 5) & 3, lane = threadIdx.x & 31;
  const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
  const float sl2 = a.scale * kLog2e;
  const bool docs = a.q_seg != nullptr;
  float m_ref = -INFINITY, l = 0.f;
  const uint32_t s_tmem = tmem + g * kTileN + lane_base;
  const uint32_t o_tmem = tmem + 2 * kTileN + g * kHeadDim + lane_base;
  unsigned char* prow = sm.p[g] + (row >> 3) * 1024 + (row & 7) * 128;

  int next_seg = INT_MIN, next_end = 0;
  auto fetch_key_docs = [&](int n) {
    next_seg = INT_MIN;
    next_end = 0;
    if (docs && n < w.n_tiles) {
      const int j = tile_first_key(n, w.first_tile, w.dummy_tile) + row;
      if (j < a.k_len) {
        const long long at = static_cast<long long>(batch) * a.k_len + j;
        next_seg = __ldg(a.k_seg + at);
        next_end = __ldg(a.k_query_end + at);
      }
    }
  };
  fetch_key_docs(g);

  int mine = 0;  // tiles this warpgroup has processed
  for (int n = g; n < w.n_tiles; n += 2, ++mine) {
    const int j0 = tile_first_key(n, w.first_tile, w.dummy_tile);
    int cls = !live || j0 >= rb.hi ? kTileNone : (j0 + kTileN <= rb.hi ? kTileFull : kTileCausal);
    if (docs) {
      const int seg = next_seg, end = next_end;
      fetch_key_docs(n + 2);
      sm.key_seg[g][row] = seg;
      sm.key_end[g][row] = end;
      const int smin = __reduce_min_sync(0xffffffffu, seg);
      const int smax = __reduce_max_sync(0xffffffffu, seg);
      const int emin = __reduce_min_sync(0xffffffffu, end);
      if (lane == 0) {
        sm.tile_summary[g][warp][0] = smin;
        sm.tile_summary[g][warp][1] = smax;
        sm.tile_summary[g][warp][2] = emin;
      }
      ptx::mbar_arrive(&sm.docs_full[g]);
      if (!wait_or_abort(sm, &sm.docs_full[g], mine & 1, 30)) return;
      if (cls != kTileNone) {
        int tmin = sm.tile_summary[g][0][0], tmax = sm.tile_summary[g][0][1], tend = sm.tile_summary[g][0][2];
#pragma unroll
        for (int q = 1; q < 4; ++q) {
          tmin = min(tmin, sm.tile_summary[g][q][0]);
          tmax = max(tmax, sm.tile_summary[g][q][1]);
          tend = min(tend, sm.tile_summary[g][q][2]);
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
    if (!wait_or_abort(sm, &sm.s_full[g], mine & 1, 31)) return;
    ptx::tc_fence_after();
    // pass 1: row maximum
    float top = -INFINITY;
    if (__any_sync(0xffffffffu, cls != kTileNone)) {
      float t0 = -INFINITY, t1 = -INFINITY, t2 = -INFINITY, t3 = -INFINITY;
      uint32_t raw[2][32];
      ptx::tmem_ld32(s_tmem, raw[0]);
#pragma unroll
      for (int c = 0; c < kTileN / 32; ++c) {
        ptx::tmem_wait_ld();
        if (c + 1 < kTileN / 32) ptx::tmem_ld32(s_tmem + (c + 1) * 32, raw[(c + 1) & 1]);
        float x[32];
        mask_chunk(raw[c & 1], x, cls, c, lim, rb, j0, sm.key_seg[g], sm.key_end[g]);
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
    // this warpgroup's P buffer and O accumulator belong to the PV product of its previous tile until it completes
    if (mine >= 1 && !wait_or_abort(sm, &sm.pv_done[g], (mine - 1) & 1, 32)) return;
    ptx::tc_fence_after();
    // pass 2: exponentials -> P
    {
      float2 s0 = make_float2(0.f, 0.f), s1 = make_float2(0.f, 0.f);
      const float2 sc = make_float2(sl2, sl2), nm = make_float2(-m_use, -m_use);
      uint32_t raw[2][32];
      ptx::tmem_ld32(s_tmem, raw[0]);
#pragma unroll
      for (int c = 0; c < kTileN / 32; ++c) {
        ptx::tmem_wait_ld();
        if (c + 1 < kTileN / 32) ptx::tmem_ld32(s_tmem + (c + 1) * 32, raw[(c + 1) & 1]);
        float x[32];
        mask_chunk(raw[c & 1], x, cls, c, lim, rb, j0, sm.key_seg[g], sm.key_end[g]);
        uint32_t pk[16];
#pragma unroll
        for (int e = 0; e < 32; e += 4) {
          float2 u0 = __ffma2_rn(make_float2(x[e], x[e + 1]), sc, nm);
          float2 u1 = __ffma2_rn(make_float2(x[e + 2], x[e + 3]), sc, nm);
          u0.x = fast_exp2(u0.x);
          u0.y = fast_exp2(u0.y);
          u1.x = fast_exp2(u1.x);
          u1.y = fast_exp2(u1.y);
          s0 = __fadd2_rn(s0, u0);
          s1 = __fadd2_rn(s1, u1);
          pk[e / 2] = pack_bf16(u0.x, u0.y);
          pk[e / 2 + 1] = pack_bf16(u1.x, u1.y);
        }
        const int sub = (c >> 1) * kTileBytes;
#pragma unroll
        for (int u = 0; u < 4; ++u)
          *reinterpret_cast<uint4*>(prow + sub + ((((c & 1) * 4 + u) ^ (row & 7)) << 4)) =
              make_uint4(pk[4 * u], pk[4 * u + 1], pk[4 * u + 2], pk[4 * u + 3]);
      }
      l += (s0.x + s0.y) + (s1.x + s1.y);
    }
    if (__any_sync(0xffffffffu, moved)) {
      uint32_t raw[2][32];
      ptx::tmem_ld32(o_tmem, raw[0]);
      ptx::tmem_ld32(o_tmem + 32, raw[1]);
      ptx::tmem_wait_ld();
#pragma unroll
      for (int c = 0; c < 2; ++c) {
#pragma unroll
        for (int e = 0; e < 32; ++e) raw[c][e] = __float_as_uint(__uint_as_float(raw[c][e]) * corr);
        ptx::tmem_st32(o_tmem + c * 32, raw[c]);
      }
      ptx::tmem_wait_st();
    }
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
    ptx::mbar_arrive(&sm.p_full[g]);
  }
  // merge the two streams: each thread finishes 32 output columns of its row
  if (mine >= 1 && !wait_or_abort(sm, &sm.pv_done[g], (mine - 1) & 1, 35)) return;
  ptx::tc_fence_after();
  sm.part_m[g][row] = m_ref;
  sm.part_l[g][row] = l;
  ptx::tc_fence_before();
  ptx::mbar_arrive(&sm.merge_full);
  if (!wait_or_abort(sm, &sm.merge_full, 0, 37)) return;
  ptx::tc_fence_after();
  const float m0 = sm.part_m[0][row], m1 = sm.part_m[1][row];
  const float l0 = sm.part_l[0][row], l1 = sm.part_l[1][row];
  const float m = fmaxf(m0, m1);
  const float f0 = l0 > 0.f ? fast_exp2(m0 - m) : 0.f;  // exactly one when both maxima agree
  const float f1 = l1 > 0.f ? fast_exp2(m1 - m) : 0.f;
  const float total = l0 * f0 + l1 * f1;
  const float inv = total > 0.f ? 1.f / total : 0.f;
  uint32_t ra[32], rc[32];
  ptx::tmem_ld32(tmem + 2 * kTileN + lane_base + g * 32, ra);
  ptx::tmem_ld32(tmem + 2 * kTileN + kHeadDim + lane_base + g * 32, rc);
  ptx::tmem_wait_ld();
  if (live) {
    __nv_bfloat16* orow = static_cast<__nv_bfloat16*>(a.out) + batch * a.out_strides[0] + head * a.out_strides[1] +
                          static_cast<long long>(rb.qi) * a.out_strides[2] + g * 32;
    const float w0 = f0 * inv, w1 = f1 * inv;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      uint32_t pk[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float lo = 0.f, hi = 0.f;
        if (l0 > 0.f) {
          lo = __uint_as_float(ra[8 * u + 2 * e]) * w0;
          hi = __uint_as_float(ra[8 * u + 2 * e + 1]) * w0;
        }
        if (l1 > 0.f) {
          lo = fmaf(__uint_as_float(rc[8 * u + 2 * e]), w1, lo);
          hi = fmaf(__uint_as_float(rc[8 * u + 2 * e + 1]), w1, hi);
        }
        pk[e] = pack_bf16(lo, hi);
      }
      reinterpret_cast<uint4*>(orow)[u] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
    }
    if (g == 0 && a.lse != nullptr)
      a.lse[(static_cast<long long>(batch) * a.q_heads + head) * a.q_len + rb.qi] =
          total > 0.f ? (m + log2f(total)) * kLn2 : INFINITY;
  }
}

__global__ void __launch_bounds__(kFwd4Threads, 1)
    attn_fwd_tc4_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                        const __grid_constant__ CUtensorMap map_v, const wm_attn_args a, const int epoch) {
  extern __shared__ unsigned char smem_raw[];
  Fwd4Shared& sm = *reinterpret_cast<Fwd4Shared*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
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
  if (tid < 256) {
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
      ptx::mbar_init(&sm.p_full[b], kTileM);
      ptx::mbar_init(&sm.pv_done[b], 1);
      ptx::mbar_init(&sm.docs_full[b], kTileM);
    }
    ptx::mbar_init(&sm.merge_full, 256);
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
    softmax4(sm, a, tmem, w, rb, live, batch, head);
  } else if (warp == 8) {
    if (lane == 0) producer_role(sm, &map_q, &map_k, &map_v, w, q0, head, kv_head, batch);
  } else {
    if (lane == 0) mma4(sm, tmem, w);
  }
  ptx::tc_fence_before();
  __syncthreads();
  trace_flush(sm);
  if (warp == 8) ptx::tmem_dealloc(tmem, kTmemCols);
}
