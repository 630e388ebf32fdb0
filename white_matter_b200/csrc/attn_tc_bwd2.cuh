// Backward pipeline for short query axes (included by attn_tc.cu).
//
// Cyclic attention with stride S has S times fewer queries than keys.  When a
// (batch, head) has at most 256 queries and query heads are not grouped, one
// block keeps both query tiles (Q, dO: 64 KB) and their dQ accumulators (TMEM)
// resident and walks over the key tiles: dK and dV of a key tile are complete
// inside the block and are written once, dQ is written once at the end -- no
// atomics, no fp32 scratch, no conversion pass.  K and V tiles stream through a
// two-stage TMA ring, so the fixed costs of a block are paid once per
// (batch, head) instead of once per key tile.
//
// 320 threads: warps 0-7 compute (thread = query row (tid & 127), column half
// (tid >> 7) of the 128-key tile), warp 8 TMA producer, warp 9 MMA issuer.
// TMEM: S [0,128) dP [128,256) dV [256,320) dK [320,384) dQ0 [384,448) dQ1 [448,512).
#pragma once

constexpr int kBwd2Threads = 320;
constexpr int kBwd2Compute = 256;

struct Bwd2Shared {
  unsigned char q[2][kTileBytes];
  unsigned char g[2][kTileBytes];  // dO
  unsigned char k[2][kTileBytes];
  unsigned char v[2][kTileBytes];
  unsigned char p[2 * kTileBytes];
  unsigned char ds[2 * kTileBytes];
  uint64_t qg_full;
  uint64_t kv_full[2], kv_ready[2], kv_empty[2];
  uint64_t sdp_full, pds_full, mma_done;
  int key_seg[2][kTileN];
  int key_end[2][kTileN];
  int summary[2][4][3];
  int lo_min[2], hi_max[2];
  int has_dummy;
  uint32_t tmem_base;
  int abort_flag;
  int epoch;
  int trace_on, trace_n;
  long long trace[kTraceSlots];
};

struct Bwd2Walk {
  int nq;      // query tiles (1 or 2)
  int n_kt;    // key tiles of the tensor
  int lo_min[2], hi_max[2];
  int kvis;    // exclusive bound of the key slots any query can see
  bool docs;
  bool dummy;
};

__device__ __forceinline__ bool pair_visible(const Bwd2Walk& w, int kt, int qt) {
  if (qt >= w.nq) return false;
  const int j0 = kt * kTileN;
  if (j0 >= w.hi_max[qt]) return false;
  if (w.docs && j0 + kTileN - 1 < w.lo_min[qt] && !(w.dummy && kt == 0)) return false;
  return true;
}

template <class Shared>
__device__ __forceinline__ void bwd2_producer(Shared& sm, const CUtensorMap* map_q, const CUtensorMap* map_k,
                                              const CUtensorMap* map_v, const CUtensorMap* map_g, const Bwd2Walk& w,
                                              int head, int batch) {
  ptx::prefetch_tmap(map_q);
  ptx::prefetch_tmap(map_k);
  ptx::prefetch_tmap(map_v);
  ptx::prefetch_tmap(map_g);
  ptx::mbar_expect_tx(&sm.qg_full, 2 * w.nq * kTileBytes);
  for (int qt = 0; qt < w.nq; ++qt) {
    ptx::tma_load_4d(sm.q[qt], map_q, &sm.qg_full, 0, qt * kTileM, head, batch);
    ptx::tma_load_4d(sm.g[qt], map_g, &sm.qg_full, 0, qt * kTileM, head, batch);
  }
  int active = 0;
  for (int kt = 0; kt < w.n_kt; ++kt) {
    if (!pair_visible(w, kt, 0) && !pair_visible(w, kt, 1)) continue;
    const int s = active & 1;
    if (!wait_or_abort(sm, &sm.kv_empty[s], ((active >> 1) & 1) ^ 1, 71)) return;
    ptx::mbar_expect_tx(&sm.kv_full[s], 2 * kTileBytes);
    ptx::tma_load_4d(sm.k[s], map_k, &sm.kv_full[s], 0, kt * kTileN, head, batch);
    ptx::tma_load_4d(sm.v[s], map_v, &sm.kv_full[s], 0, kt * kTileN, head, batch);
    ++active;
  }
}

__device__ __forceinline__ void bwd2_mma(Bwd2Shared& sm, uint32_t tmem, const Bwd2Walk& w) {
  if (!wait_or_abort(sm, &sm.qg_full, 0, 80)) return;
  constexpr uint32_t idesc_s = ptx::make_idesc_bf16(kTileM, kTileN, 0, 0);
  constexpr uint32_t idesc_t = ptx::make_idesc_bf16(kTileN, kHeadDim, 1, 1);
  constexpr uint32_t idesc_q = ptx::make_idesc_bf16(kTileM, kHeadDim, 0, 1);
  const uint32_t p_base = ptx::smem_u32(sm.p), ds_base = ptx::smem_u32(sm.ds);
  int active = 0, it = 0;
  bool dq_started[2] = {false, false};
  for (int kt = 0; kt < w.n_kt; ++kt) {
    const bool vis[2] = {pair_visible(w, kt, 0), pair_visible(w, kt, 1)};
    if (!vis[0] && !vis[1]) continue;
    const int s = active & 1;
    if (!wait_or_abort(sm, &sm.kv_ready[s], (active >> 1) & 1, 81)) return;
    ptx::tc_fence_after();
    trace_event(sm, 100 + kt);
    const uint32_t k_base = ptx::smem_u32(sm.k[s]), v_base = ptx::smem_u32(sm.v[s]);
    bool dkv_started = false;
#pragma unroll
    for (int qt = 0; qt < 2; ++qt) {
      if (!vis[qt]) continue;
      const uint32_t q_base = ptx::smem_u32(sm.q[qt]), g_base = ptx::smem_u32(sm.g[qt]);
#pragma unroll
      for (int kk = 0; kk < kHeadDim / 16; ++kk)
        ptx::mma_bf16_ss(tmem, ptx::make_smem_desc_sw128(q_base + kk * 32, 16, 1024),
                         ptx::make_smem_desc_sw128(k_base + kk * 32, 16, 1024), idesc_s, kk > 0);
#pragma unroll
      for (int kk = 0; kk < kHeadDim / 16; ++kk)
        ptx::mma_bf16_ss(tmem + kTileN, ptx::make_smem_desc_sw128(g_base + kk * 32, 16, 1024),
                         ptx::make_smem_desc_sw128(v_base + kk * 32, 16, 1024), idesc_s, kk > 0);
      ptx::mma_commit(&sm.sdp_full);
      trace_event(sm, 200 + it);
      if (!wait_or_abort(sm, &sm.pds_full, it & 1, 82)) return;
      ptx::tc_fence_after();
      trace_event(sm, 300 + it);
#pragma unroll
      for (int kk = 0; kk < kTileM / 16; ++kk)
        ptx::mma_bf16_ss(tmem + 2 * kTileN, ptx::make_smem_desc_sw128(p_base + kk * 2048, kTileBytes, 1024),
                         ptx::make_smem_desc_sw128(g_base + kk * 2048, 1024, 1024), idesc_t, dkv_started || (kk > 0));
#pragma unroll
      for (int kk = 0; kk < kTileM / 16; ++kk)
        ptx::mma_bf16_ss(tmem + 2 * kTileN + kHeadDim,
                         ptx::make_smem_desc_sw128(ds_base + kk * 2048, kTileBytes, 1024),
                         ptx::make_smem_desc_sw128(q_base + kk * 2048, 1024, 1024), idesc_t, dkv_started || (kk > 0));
#pragma unroll
      for (int kk = 0; kk < kTileN / 16; ++kk)
        ptx::mma_bf16_ss(tmem + 2 * kTileN + 2 * kHeadDim + qt * kHeadDim,
                         ptx::make_smem_desc_sw128(ds_base + (kk >> 2) * kTileBytes + (kk & 3) * 32, 16, 1024),
                         ptx::make_smem_desc_sw128(k_base + kk * 2048, 1024, 1024), idesc_q,
                         dq_started[qt] || (kk > 0));
      dkv_started = true;
      dq_started[qt] = true;
      ptx::mma_commit(&sm.mma_done);
      trace_event(sm, 400 + it);
      ++it;
    }
    ptx::mma_commit(&sm.kv_empty[s]);
    ++active;
  }
}

// dV (half 0) or dK (half 1) rows of key tile `kt`: TMEM -> bf16 -> global, one key row per thread
__device__ __forceinline__ void bwd2_store_dkv(const wm_attn_args& a, uint32_t tmem, int kt, int row, int half,
                                               uint32_t lane_base, int head, int batch, bool zero) {
  const int j = kt * kTileN + row;
  uint32_t packed[kHeadDim / 2];
  const float s = half ? a.scale : 1.f;
  uint32_t raw[kHeadDim / 32][32];
  if (!zero) {
#pragma unroll
    for (int c = 0; c < kHeadDim / 32; ++c)
      ptx::tmem_ld32(tmem + 2 * kTileN + half * kHeadDim + lane_base + c * 32, raw[c]);
    ptx::tmem_wait_ld();
  }
#pragma unroll
  for (int c = 0; c < kHeadDim / 32; ++c) {
#pragma unroll
    for (int e = 0; e < 16; ++e)
      packed[c * 16 + e] =
          zero ? 0u : pack_bf16(__uint_as_float(raw[c][2 * e]) * s, __uint_as_float(raw[c][2 * e + 1]) * s);
  }
  if (j < a.k_len) {
    const int64_t* st = half ? a.dk_strides : a.dv_strides;
    __nv_bfloat16* base = static_cast<__nv_bfloat16*>(half ? a.dk : a.dv);
    uint4* dst = reinterpret_cast<uint4*>(base + batch * st[0] + head * st[1] + static_cast<long long>(j) * st[2]);
#pragma unroll
    for (int c = 0; c < 8; ++c)
      dst[c] = make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
  }
}

__device__ __forceinline__ void bwd2_compute(Bwd2Shared& sm, const wm_attn_args& a, uint32_t tmem, const Bwd2Walk& w,
                                             const float* delta, int head, int batch) {
  const int tid = threadIdx.x;
  const int row = tid & 127;
  const int half = tid >> 7;
  const int warp = tid >> 5, lane = tid & 31;
  const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
  const float sl2 = a.scale * kLog2e;
  const GroupCtx g = group_ctx(a, 0);

  // per query tile: this thread's row
  RowBound rb[2];
  float lse2[2], dl[2];
  bool live[2];
#pragma unroll
  for (int qt = 0; qt < 2; ++qt) {
    const int i = qt * kTileM + row;
    live[qt] = qt < w.nq && i < a.q_len;
    rb[qt].lo = 0;
    rb[qt].hi = 0;
    rb[qt].seg = 0;
    rb[qt].qi = i;
    lse2[qt] = INFINITY;
    dl[qt] = 0.f;
    if (live[qt]) {
      rb[qt] = row_bound(a, g, batch, i);
      const long long stat = (static_cast<long long>(batch) * a.q_heads + head) * a.q_len + i;
      lse2[qt] = a.lse[stat] * kLog2e;
      dl[qt] = delta[stat];
    }
  }
  unsigned char* prow = sm.p + half * kTileBytes + (row >> 3) * 1024 + (row & 7) * 128;
  unsigned char* drow = sm.ds + half * kTileBytes + (row >> 3) * 1024 + (row & 7) * 128;

  // key documents of key slot (tile start + row), fetched one visited tile ahead (half 0 publishes them)
  int next_seg = INT_MIN, next_end = 0;
  auto fetch_key_docs = [&](int kt) {
    next_seg = INT_MIN;
    next_end = 0;
    if (w.docs && half == 0 && kt < w.n_kt) {
      const int j = kt * kTileN + row;
      if (j < a.k_len) {
        const long long at = static_cast<long long>(batch) * a.k_len + j;
        next_seg = __ldg(a.k_seg + at);
        next_end = __ldg(a.k_query_end + at);
      }
    }
  };
  auto next_visited = [&](int kt) {
    while (kt < w.n_kt && !pair_visible(w, kt, 0) && !pair_visible(w, kt, 1)) ++kt;
    return kt;
  };
  fetch_key_docs(next_visited(0));

  int active = 0, it = 0;
  bool dq_valid[2] = {false, false};  // a dQ accumulator holds data once one of its products was issued
  int pending_kt = -1;  // key tile whose dK/dV sit complete in TMEM once mma_done of iteration it-1 fires
  for (int kt = 0; kt < w.n_kt; ++kt) {
    const bool vis[2] = {pair_visible(w, kt, 0), pair_visible(w, kt, 1)};
    if (!vis[0] && !vis[1]) {
      bwd2_store_dkv(a, tmem, kt, row, half, lane_base, head, batch, true);  // nobody sees this tile: exact zeros
      continue;
    }
    const int s = active & 1;
    const int j0 = kt * kTileN;
    if (w.docs && half == 0) {
      const int seg = next_seg, end = next_end;
      sm.key_seg[s][row] = seg;
      sm.key_end[s][row] = end;
      const int smin = __reduce_min_sync(0xffffffffu, seg);
      const int smax = __reduce_max_sync(0xffffffffu, seg);
      const int emin = __reduce_min_sync(0xffffffffu, end);
      if (lane == 0) {
        sm.summary[s][warp][0] = smin;
        sm.summary[s][warp][1] = smax;
        sm.summary[s][warp][2] = emin;
      }
    }
    fetch_key_docs(next_visited(kt + 1));
    // key rows at or beyond the last visible slot may hold anything: clear them before the MMAs read the tile
    if (tid == 0) trace_event(sm, 1100 + kt);
    if (!wait_or_abort(sm, &sm.kv_full[s], (active >> 1) & 1, 90)) return;
    if (j0 + row >= w.kvis) {
      uint4* dst = reinterpret_cast<uint4*>((half ? sm.v[s] : sm.k[s]) + row * 128);
#pragma unroll
      for (int c = 0; c < 8; ++c) dst[c] = make_uint4(0, 0, 0, 0);
    }
    ptx::fence_async_shared();
    ptx::mbar_arrive(&sm.kv_ready[s]);
    if (!wait_or_abort(sm, &sm.kv_ready[s], (active >> 1) & 1, 91)) return;  // also orders the document tables
    if (tid == 0) trace_event(sm, 1200 + kt);
    int tmin = 0, tmax = 0, tend = 0;
    if (w.docs) {
      tmin = min(min(sm.summary[s][0][0], sm.summary[s][1][0]), min(sm.summary[s][2][0], sm.summary[s][3][0]));
      tmax = max(max(sm.summary[s][0][1], sm.summary[s][1][1]), max(sm.summary[s][2][1], sm.summary[s][3][1]));
      tend = min(min(sm.summary[s][0][2], sm.summary[s][1][2]), min(sm.summary[s][2][2], sm.summary[s][3][2]));
    }
#pragma unroll
    for (int qt = 0; qt < 2; ++qt) {
      if (!vis[qt]) continue;
      dq_valid[qt] = true;
      const RowBound& r = rb[qt];
      int cls = !live[qt] || j0 >= r.hi ? kTileNone : (j0 + kTileN <= r.hi ? kTileFull : kTileCausal);
      if (w.docs && cls != kTileNone) {
        const bool uniform = tmin == tmax;
        const bool own_doc = uniform && tmin == r.seg && j0 >= r.lo && tend > r.qi;
        if (uniform && tmin != -1 && tmin != r.seg) {
          cls = kTileNone;
        } else if (!own_doc) {
          cls = kTileDocs;
        }
      }
      const int lim = r.hi - j0;
      if (!wait_or_abort(sm, &sm.sdp_full, it & 1, 92)) return;
      if (tid == 0) trace_event(sm, 500 + it);
      if (it > 0 && !wait_or_abort(sm, &sm.mma_done, (it - 1) & 1, 93)) return;
      ptx::tc_fence_after();
      if (tid == 0) trace_event(sm, 600 + it);
      if (pending_kt >= 0) {
        bwd2_store_dkv(a, tmem, pending_kt, row, half, lane_base, head, batch, false);
        pending_kt = -1;
        if (tid == 0) trace_event(sm, 700 + it);
      }
      // all four TMEM loads of the iteration are in flight before the single wait (a load takes ~500 cycles)
      uint32_t xs[2][32], ys[2][32];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        ptx::tmem_ld32(tmem + lane_base + half * 64 + c * 32, xs[c]);
        ptx::tmem_ld32(tmem + kTileN + lane_base + half * 64 + c * 32, ys[c]);
      }
      ptx::tmem_wait_ld();
      if (tid == 0) trace_event(sm, 800 + it);
      // one comparison per element on the common path; the per-element document rule is a separate, rare loop
      const int lim_eff = cls == kTileFull ? kTileN : (cls == kTileNone ? 0 : lim);
      const float nl = -lse2[qt], dlt = dl[qt];
      if (cls != kTileDocs) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int col0 = half * 64 + c * 32;
          uint32_t pp[16], dd[16];
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            const float p0 = fast_exp2(fmaf(__uint_as_float(xs[c][2 * e]), sl2, nl));
            const float p1 = fast_exp2(fmaf(__uint_as_float(xs[c][2 * e + 1]), sl2, nl));
            const bool v0 = col0 + 2 * e < lim_eff, v1 = col0 + 2 * e + 1 < lim_eff;
            pp[e] = pack_bf16(v0 ? p0 : 0.f, v1 ? p1 : 0.f);
            dd[e] = pack_bf16(v0 ? p0 * (__uint_as_float(ys[c][2 * e]) - dlt) : 0.f,
                              v1 ? p1 * (__uint_as_float(ys[c][2 * e + 1]) - dlt) : 0.f);
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int off = ((c * 4 + u) ^ (row & 7)) << 4;
            *reinterpret_cast<uint4*>(prow + off) = make_uint4(pp[4 * u], pp[4 * u + 1], pp[4 * u + 2], pp[4 * u + 3]);
            *reinterpret_cast<uint4*>(drow + off) = make_uint4(dd[4 * u], dd[4 * u + 1], dd[4 * u + 2], dd[4 * u + 3]);
          }
        }
      } else {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int col0 = half * 64 + c * 32;
          uint32_t pp[16], dd[16];
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            float pv[2], dv[2];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
              const int col = col0 + 2 * e + u;
              const bool vis_e = (col < lim) & doc_visible_flat(r, j0 + col, sm.key_seg[s][col], sm.key_end[s][col]);
              const float p = fast_exp2(fmaf(__uint_as_float(xs[c][2 * e + u]), sl2, nl));
              pv[u] = vis_e ? p : 0.f;
              dv[u] = vis_e ? p * (__uint_as_float(ys[c][2 * e + u]) - dlt) : 0.f;
            }
            pp[e] = pack_bf16(pv[0], pv[1]);
            dd[e] = pack_bf16(dv[0], dv[1]);
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int off = ((c * 4 + u) ^ (row & 7)) << 4;
            *reinterpret_cast<uint4*>(prow + off) = make_uint4(pp[4 * u], pp[4 * u + 1], pp[4 * u + 2], pp[4 * u + 3]);
            *reinterpret_cast<uint4*>(drow + off) = make_uint4(dd[4 * u], dd[4 * u + 1], dd[4 * u + 2], dd[4 * u + 3]);
          }
        }
      }
      if (tid == 0) trace_event(sm, 900 + it);
      ptx::fence_async_shared();
      ptx::tc_fence_before();
      ptx::mbar_arrive(&sm.pds_full);
      if (tid == 0) trace_event(sm, 1000 + it);
      ++it;
    }
    pending_kt = kt;
    ++active;
  }
  // the last key tile's dK/dV and the dQ accumulators
  if (it > 0) {
    if (!wait_or_abort(sm, &sm.mma_done, (it - 1) & 1, 94)) return;
    ptx::tc_fence_after();
    if (pending_kt >= 0) bwd2_store_dkv(a, tmem, pending_kt, row, half, lane_base, head, batch, false);
  }
  {
    // half h writes the dQ rows of query tile h
    const int qt = half;
    const int i = qt * kTileM + row;
    const bool any = half ? dq_valid[1] : dq_valid[0];
    const int row_hi = half ? rb[1].hi : rb[0].hi;
    uint32_t packed[kHeadDim / 2];
#pragma unroll
    for (int c = 0; c < kHeadDim / 32; ++c) {
      uint32_t raw[32];
      if (any) {
        ptx::tmem_ld32(tmem + 2 * kTileN + 2 * kHeadDim + qt * kHeadDim + lane_base + c * 32, raw);
        ptx::tmem_wait_ld();
      }
#pragma unroll
      for (int e = 0; e < 16; ++e)
        packed[c * 16 + e] = any && row_hi > 0 ? pack_bf16(__uint_as_float(raw[2 * e]) * a.scale,
                                                              __uint_as_float(raw[2 * e + 1]) * a.scale)
                                                  : 0u;
    }
    if (qt < w.nq && i < a.q_len) {
      uint4* dst = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(a.dq) + batch * a.dq_strides[0] +
                                            head * a.dq_strides[1] + static_cast<long long>(i) * a.dq_strides[2]);
#pragma unroll
      for (int c = 0; c < 8; ++c)
        dst[c] = make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
    }
  }
}

__global__ void __launch_bounds__(kBwd2Threads, 1)
    attn_bwd_tc2_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                        const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_g,
                        const wm_attn_args a, const float* delta, const int epoch) {
  extern __shared__ unsigned char smem_raw[];
  Bwd2Shared& sm = *reinterpret_cast<Bwd2Shared*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int head = blockIdx.x;
  const int batch = blockIdx.y;
  const GroupCtx g = group_ctx(a, 0);

  if (tid == 0) {
    sm.abort_flag = 0;
    sm.epoch = epoch;
    trace_begin(sm, epoch);
    sm.lo_min[0] = sm.lo_min[1] = INT_MAX;
    sm.hi_max[0] = sm.hi_max[1] = 0;
    sm.has_dummy = a.q_seg != nullptr && a.k_seg[static_cast<long long>(batch) * a.k_len] == -1;
  }
  __syncthreads();
  if (tid < kBwd2Compute) {
    // thread tid looks at query row tid: per query tile the smallest document start and the largest bound
    const int qt = tid >> 7;
    int lo = INT_MAX, hi = 0;
    if (tid < a.q_len) {
      const RowBound rb = row_bound(a, g, batch, tid);
      hi = rb.hi;
      if (rb.hi > 0) lo = rb.lo;
    }
    lo = __reduce_min_sync(0xffffffffu, lo);
    hi = __reduce_max_sync(0xffffffffu, hi);
    if (lane == 0) {
      atomicMin(&sm.lo_min[qt], lo);
      atomicMax(&sm.hi_max[qt], hi);
    }
  }
  __syncthreads();
  Bwd2Walk w;
  w.nq = (a.q_len + kTileM - 1) / kTileM;
  w.n_kt = (a.k_len + kTileN - 1) / kTileN;
  w.lo_min[0] = sm.lo_min[0];
  w.lo_min[1] = sm.lo_min[1];
  w.hi_max[0] = sm.hi_max[0];
  w.hi_max[1] = sm.hi_max[1];
  w.kvis = max(w.hi_max[0], w.hi_max[1]);
  w.docs = a.q_seg != nullptr;
  w.dummy = sm.has_dummy != 0;

  if (tid == 0) {
    ptx::mbar_init(&sm.qg_full, 1);
    for (int s = 0; s < 2; ++s) {
      ptx::mbar_init(&sm.kv_full[s], 1);
      ptx::mbar_init(&sm.kv_ready[s], kBwd2Compute);
      ptx::mbar_init(&sm.kv_empty[s], 1);
    }
    ptx::mbar_init(&sm.sdp_full, 1);
    ptx::mbar_init(&sm.pds_full, kBwd2Compute);
    ptx::mbar_init(&sm.mma_done, 1);
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
    bwd2_compute(sm, a, tmem, w, delta, head, batch);
  } else if (warp == 8) {
    if (lane == 0) bwd2_producer(sm, &map_q, &map_k, &map_v, &map_g, w, head, batch);
  } else {
    if (lane == 0) bwd2_mma(sm, tmem, w);
  }
  ptx::tc_fence_before();
  __syncthreads();
  trace_flush(sm);
  if (warp == 8) ptx::tmem_dealloc(tmem, kTmemCols);
}
