// Backward pipeline for short query axes (included by attn_tc.cu).
//
// Cyclic attention with stride S has S times fewer queries than keys.  When a (batch, head) has
// at most 256 queries and query heads are not grouped, one block keeps both query tiles (Q, dO:
// 64 KB) and their dQ accumulators (TMEM) resident and walks over the key tiles: dK and dV of a
// key tile are complete inside the block and leave through one TMA store each, dQ is written
// once at the end -- no atomics, no fp32 scratch, no conversion pass.  K and V tiles stream
// through a two-stage TMA ring.
//
// 352 threads: warps 0-7 compute (thread = query row (tid & 127), column half (tid >> 7) of the
// 128-key tile), warp 8 TMA producer, warps 9 and 10 MMA issuers (S/dP products, gradient products).
// TMEM: S [0,128) dP [128,256) dV [256,320) dK [320,384) dQ0 [384,448) dQ1 [448,512).
//
// An iteration is one (key tile, query tile) pair; the list of visible pairs is built once per
// block.  The compute warps pull S and dP of iteration i out of TMEM into registers and release
// them at once (sdp_free), so the MMA warp issues S/dP of iteration i+1 while the exponentials of
// iteration i are still being computed; P and dS of iteration i are written to shared memory only
// after the dV/dK/dQ products of iteration i-1 have read the previous contents (mma_done).
#pragma once

constexpr int kResidentThreads = 352;
constexpr int kResidentCompute = 256;


struct ResidentWalk {
  int nq;      // query tiles (1 or 2)
  int n_kt;    // key tiles of the tensor
  int lo_min[2], hi_max[2];
  int kvis;    // exclusive bound of the key slots any query can see
  bool docs;
  bool dummy;
};

__device__ __forceinline__ bool pair_visible(const ResidentWalk& w, int kt, int qt) {
  if (qt >= w.nq) return false;
  const int j0 = kt * kTileN;
  if (j0 >= w.hi_max[qt]) return false;
  if (w.docs && j0 + kTileN - 1 < w.lo_min[qt] && !(w.dummy && kt == 0)) return false;
  return true;
}

template <class Shared>
__device__ __forceinline__ void resident_producer(Shared& sm, const CUtensorMap* map_q, const CUtensorMap* map_k,
                                              const CUtensorMap* map_v, const CUtensorMap* map_g, const ResidentWalk& w,
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

// dV (half 0) or dK (half 1) rows of key tile `kt`: TMEM -> bf16 -> global, one key row per thread
__device__ __forceinline__ void resident_store_dkv(const wm_attn_args& a, uint32_t tmem, int kt, int row, int half,
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


constexpr int kResidentMaxIter = 256;

struct ResidentShared {
  unsigned char q[2][kTileBytes];
  unsigned char g[2][kTileBytes];  // dO
  unsigned char k[2][kTileBytes];
  unsigned char v[2][kTileBytes];
  unsigned char p[2 * kTileBytes];
  unsigned char ds[2 * kTileBytes];
  uint64_t qg_full;
  uint64_t kv_full[2], kv_ready[2], kv_empty[2];
  uint64_t sdp_full, sdp_free, pds_full, mma_done;
  uint64_t out_full[2];  // dV (half 0) / dK (half 1) rows of a finished key tile are staged in shared memory
  uint64_t stage_free[2];  // the store out of the spare staging room has read it
  int key_seg[2][kTileN];
  int key_end[2][kTileN];
  int summary[2][4][3];
  int lo_min[2], hi_max[2];
  int has_dummy;
  // iteration list: key tile | query tile << 12 | first-of-key-tile << 13 | last-of-key-tile << 14 | visited index << 16
  uint32_t sched[kResidentMaxIter];
  int n_iter;
  int q0_last_iter;  // last iteration that uses query tile 0 (-1: none)
  uint32_t tmem_base;
  int abort_flag;
  int epoch;
  WM_TRACE_FIELDS
};

struct ResidentIter {
  int kt, qt, first, last, active;
};

__device__ __forceinline__ ResidentIter resident_iter(uint32_t e) {
  ResidentIter it;
  it.kt = e & 0xfff;
  it.qt = (e >> 12) & 1;
  it.first = (e >> 13) & 1;
  it.last = (e >> 14) & 1;
  it.active = e >> 16;
  return it;
}

__device__ __forceinline__ void resident_issue_sdp(ResidentShared& sm, uint32_t tmem, const ResidentIter& e) {
  constexpr uint32_t idesc_s = ptx::make_idesc_bf16(kTileM, kTileN, 0, 0);
  const int s = e.active & 1;
  const uint32_t q_base = ptx::smem_u32(sm.q[e.qt]), g_base = ptx::smem_u32(sm.g[e.qt]);
  const uint32_t k_base = ptx::smem_u32(sm.k[s]), v_base = ptx::smem_u32(sm.v[s]);
#pragma unroll
  for (int kk = 0; kk < kHeadDim / 16; ++kk)
    ptx::mma_bf16_ss(tmem, ptx::make_smem_desc_sw128(q_base + kk * 32, 16, 1024),
                     ptx::make_smem_desc_sw128(k_base + kk * 32, 16, 1024), idesc_s, kk > 0);
#pragma unroll
  for (int kk = 0; kk < kHeadDim / 16; ++kk)
    ptx::mma_bf16_ss(tmem + kTileN, ptx::make_smem_desc_sw128(g_base + kk * 32, 16, 1024),
                     ptx::make_smem_desc_sw128(v_base + kk * 32, 16, 1024), idesc_s, kk > 0);
  ptx::mma_commit(&sm.sdp_full);
}

// Two issuing threads, because the tensor pipe takes an instruction only when it has started the previous one and
// the issuing thread is busy for as long as its products run: one thread issues the S / dP products as soon as
// the compute warps hold the previous pair in registers, the other the three gradient products of a pair as soon
// as its P / dS are in shared memory; the waits of one never sit in front of the other's issue.
__device__ __forceinline__ void resident_mma_scores(ResidentShared& sm, uint32_t tmem) {
  const int n = sm.n_iter;
  if (n == 0) return;
  if (!wait_or_abort(sm, &sm.qg_full, 0, 80)) return;
  for (int it = 0; it < n; ++it) {
    const ResidentIter e = resident_iter(sm.sched[it]);
    // S/dP of the previous pair are in the compute warps' registers: this pair may overwrite them
    if (it > 0 && !wait_or_abort(sm, &sm.sdp_free, (it - 1) & 1, 83)) return;
    if (e.first && !wait_or_abort(sm, &sm.kv_ready[e.active & 1], (e.active >> 1) & 1, 81)) return;
    ptx::tc_fence_after();
    trace_event(sm, 100 + it);
    resident_issue_sdp(sm, tmem, e);
    trace_event(sm, 200 + it);
  }
}

__device__ __forceinline__ void resident_mma_grads(ResidentShared& sm, uint32_t tmem, int nq) {
  const int n = sm.n_iter;
  if (n == 0) return;
  const int spare_from = nq == 1 ? 0 : sm.q0_last_iter + 1;  // same rule as the compute warps' staging
  if (!wait_or_abort(sm, &sm.qg_full, 0, 84)) return;
  constexpr uint32_t idesc_t = ptx::make_idesc_bf16(kTileN, kHeadDim, 1, 1);
  constexpr uint32_t idesc_q = ptx::make_idesc_bf16(kTileM, kHeadDim, 0, 1);
  const uint32_t p_base = ptx::smem_u32(sm.p), ds_base = ptx::smem_u32(sm.ds);
  bool dq_started[2] = {false, false};
  for (int it = 0; it < n; ++it) {
    const ResidentIter e = resident_iter(sm.sched[it]);
    if (!wait_or_abort(sm, &sm.pds_full, it & 1, 82)) return;
    ptx::tc_fence_after();
    trace_event(sm, 300 + it);
    const int s = e.active & 1;
    const uint32_t q_base = ptx::smem_u32(sm.q[e.qt]), g_base = ptx::smem_u32(sm.g[e.qt]);
    const uint32_t k_base = ptx::smem_u32(sm.k[s]);
    const bool acc_kv = !e.first;
    const bool acc_q = e.qt ? dq_started[1] : dq_started[0];
#pragma unroll
    for (int kk = 0; kk < kTileM / 16; ++kk)
      ptx::mma_bf16_ss(tmem + 2 * kTileN, ptx::make_smem_desc_sw128(p_base + kk * 2048, kTileBytes, 1024),
                       ptx::make_smem_desc_sw128(g_base + kk * 2048, 1024, 1024), idesc_t, acc_kv || (kk > 0));
#pragma unroll
    for (int kk = 0; kk < kTileM / 16; ++kk)
      ptx::mma_bf16_ss(tmem + 2 * kTileN + kHeadDim, ptx::make_smem_desc_sw128(ds_base + kk * 2048, kTileBytes, 1024),
                       ptx::make_smem_desc_sw128(q_base + kk * 2048, 1024, 1024), idesc_t, acc_kv || (kk > 0));
#pragma unroll
    for (int kk = 0; kk < kTileN / 16; ++kk)
      ptx::mma_bf16_ss(tmem + 2 * kTileN + 2 * kHeadDim + e.qt * kHeadDim,
                       ptx::make_smem_desc_sw128(ds_base + (kk >> 2) * kTileBytes + (kk & 3) * 32, 16, 1024),
                       ptx::make_smem_desc_sw128(k_base + kk * 2048, 1024, 1024), idesc_q, acc_q || (kk > 0));
    if (e.qt) dq_started[1] = true; else dq_started[0] = true;
    ptx::mma_commit(&sm.mma_done);
    if (e.last && it + 1 >= spare_from) {
      // the gradients of this key tile will be staged in spare room: its K/V stage is free as soon as these
      // products are complete (two arrivals, as many as the staging threads give when they release a stage)
      ptx::mma_commit(&sm.kv_empty[s]);
      ptx::mma_commit(&sm.kv_empty[s]);
    }
    trace_event(sm, 400 + it);
  }
}

__device__ __forceinline__ void resident_compute(ResidentShared& sm, const wm_attn_args& a, uint32_t tmem, const ResidentWalk& w,
                                             const float* delta, int head, int batch, const CUtensorMap* map_dk,
                                             const CUtensorMap* map_dv) {
  const int tid = threadIdx.x;
  const int row = tid & 127;
  const int half = tid >> 7;
  const int warp = tid >> 5, lane = tid & 31;
  const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
  const float sl2 = a.scale * kLog2e;
  const GroupCtx g = group_ctx(a, 0);
  const int n = sm.n_iter;

  // this thread's row in both query tiles
  RowBound rb0, rb1;
  float nl0 = -INFINITY, nl1 = -INFINITY, dl0 = 0.f, dl1 = 0.f;
  bool live0 = false, live1 = false;
  {
    rb0.lo = rb0.hi = rb0.seg = 0;
    rb0.qi = row;
    rb1 = rb0;
    rb1.qi = kTileM + row;
    if (row < a.q_len) {
      live0 = true;
      rb0 = row_bound(a, g, batch, row);
      const long long stat = (static_cast<long long>(batch) * a.q_heads + head) * a.q_len + row;
      nl0 = -a.lse[stat] * kLog2e;
      dl0 = delta[stat];
    }
    if (w.nq > 1 && kTileM + row < a.q_len) {
      live1 = true;
      rb1 = row_bound(a, g, batch, kTileM + row);
      const long long stat = (static_cast<long long>(batch) * a.q_heads + head) * a.q_len + kTileM + row;
      nl1 = -a.lse[stat] * kLog2e;
      dl1 = delta[stat];
    }
  }
  unsigned char* prow = sm.p + half * kTileBytes + (row >> 3) * 1024 + (row & 7) * 128;
  unsigned char* drow = sm.ds + half * kTileBytes + (row >> 3) * 1024 + (row & 7) * 128;

  // key tiles nobody sees get exact zeros; they are not part of the iteration list
  for (int kt = 0; kt < w.n_kt; ++kt)
    if (!pair_visible(w, kt, 0) && !pair_visible(w, kt, 1)) resident_store_dkv(a, tmem, kt, row, half, lane_base, head, batch, true);

  // Make a visited key tile ready for the MMAs: publish its document table, clear rows beyond the last visible
  // slot (they may hold anything), and meet the other compute threads at kv_ready.
  // the table entries of a key tile are fetched one pair ahead of the tile's preparation
  int pf_seg = INT_MIN, pf_end = 0, pf_kt = -1;
  auto fetch_table = [&](int kt) {
    if (w.docs && half == 0) {
      pf_seg = INT_MIN;
      pf_end = 0;
      pf_kt = kt;
      const int j = kt * kTileN + row;
      if (j < a.k_len) {
        const long long at = static_cast<long long>(batch) * a.k_len + j;
        pf_seg = __ldg(a.k_seg + at);
        pf_end = __ldg(a.k_query_end + at);
      }
    }
  };
  auto prepare = [&](const ResidentIter& e) -> bool {
    const int s = e.active & 1;
    const int j0 = e.kt * kTileN;
    if (w.docs && half == 0) {
      if (pf_kt != e.kt) fetch_table(e.kt);
      const int seg = pf_seg, end = pf_end;
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
    if (!wait_or_abort(sm, &sm.kv_full[s], (e.active >> 1) & 1, 90)) return false;
    if (j0 + row >= w.kvis) {
      uint4* dst = reinterpret_cast<uint4*>((half ? sm.v[s] : sm.k[s]) + row * 128);
#pragma unroll
      for (int c = 0; c < 8; ++c) dst[c] = make_uint4(0, 0, 0, 0);
    }
    ptx::fence_async_shared();
    ptx::mbar_arrive(&sm.kv_ready[s]);
    return true;
  };
  // every compute thread has prepared the tile: its document table is complete
  auto prepared = [&](const ResidentIter& e) -> bool {
    return wait_or_abort(sm, &sm.kv_ready[e.active & 1], (e.active >> 1) & 1, 91);
  };

  // dV / dK of a finished key tile: TMEM -> bf16 -> the tile's own (now idle) V / K stage in shared memory, in
  // the 128B-swizzled row layout of the output tensor map -> one TMA store per half.  The stage goes back to the
  // producer once the store has read it.
  // Once the first query tile has no pair left (or when there is only one query tile), the Q / dO tiles of an
  // idle query tile are spare staging room: the K/V stage then goes back to the producer at once, which hides
  // the load of the next key tile behind the current pair (key tiles seen by one query tile only would otherwise
  // expose it every time).
  int outs = 0;  // staged stores so far (parity of out_full)
  int spare_outs = 0;  // of those, through the spare room (parity of stage_free)
  int release_stage = -1;  // stage whose staged gradients still have to be read before the producer may refill it
  bool release_spare = false;
  const int spare_tile = w.nq == 1 ? 1 : 0;
  const int spare_from = w.nq == 1 ? 0 : sm.q0_last_iter + 1;  // first iteration index at which it is free
  auto release = [&]() {
    if (row == 0 && (release_stage >= 0 || release_spare)) {
      ptx::tma_store_wait_read();
      if (release_stage >= 0) ptx::mbar_arrive(&sm.kv_empty[release_stage]);
      if (release_spare) ptx::mbar_arrive(&sm.stage_free[half]);
    }
    release_stage = -1;
    release_spare = false;
  };
  auto stage_out = [&](int kt, int stage, int it_now, bool release_now) -> bool {
    const float sc = half ? a.scale : 1.f;
    const bool spare = it_now >= spare_from;
    unsigned char* tile = spare ? (half ? sm.q[spare_tile] : sm.g[spare_tile]) : (half ? sm.k[stage] : sm.v[stage]);
    if (spare) {
      // (the K/V stage of this key tile was handed back by the gradient issuer's commit)
      // the previous store out of the spare room has to have read it
      if (spare_outs > 0 && !wait_or_abort(sm, &sm.stage_free[half], (spare_outs - 1) & 1, 96)) return false;
    }
    unsigned char* dst = tile + (row >> 3) * 1024 + (row & 7) * 128;
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {  // 32 columns at a time keeps the register footprint small
      uint32_t raw[32];
      ptx::tmem_ld32(tmem + 2 * kTileN + half * kHeadDim + lane_base + h2 * 32, raw);
      ptx::tmem_wait_ld();
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t pk[4];
#pragma unroll
        for (int e2 = 0; e2 < 4; ++e2)
          pk[e2] = pack_bf16(__uint_as_float(raw[c * 8 + 2 * e2]) * sc, __uint_as_float(raw[c * 8 + 2 * e2 + 1]) * sc);
        *reinterpret_cast<uint4*>(dst + (((h2 * 4 + c) ^ (row & 7)) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
      }
    }
    ptx::fence_async_shared();
    ptx::mbar_arrive(&sm.out_full[half]);
    if (!wait_or_abort(sm, &sm.out_full[half], outs & 1, 95)) return false;
    if (row == 0) {
      ptx::tma_store_4d(half ? map_dk : map_dv, tile, 0, kt * kTileN, head, batch);
      ptx::tma_store_commit();
    }
    if (spare) {
      release_spare = true;
      ++spare_outs;
    } else {
      release_stage = stage;
    }
    if (release_now) release();
    ++outs;
    return true;
  };

  if (n > 0 && !prepare(resident_iter(sm.sched[0]))) return;
  int pending_kt = -1, pending_stage = 0;
  for (int it = 0; it < n; ++it) {
    const ResidentIter e = resident_iter(sm.sched[it]);
    if (e.first && !prepared(e)) return;
    if (e.last && it + 1 < n) fetch_table(resident_iter(sm.sched[it + 1]).kt);
    const int s = e.active & 1;
    const int j0 = e.kt * kTileN;
    const RowBound& r = e.qt ? rb1 : rb0;
    const bool live = e.qt ? live1 : live0;
    const float nl = e.qt ? nl1 : nl0;
    const float dlt = e.qt ? dl1 : dl0;
    int cls = !live || j0 >= r.hi ? kTileNone : (j0 + kTileN <= r.hi ? kTileFull : kTileCausal);
    if (w.docs && cls != kTileNone) {
      const int tmin = min(min(sm.summary[s][0][0], sm.summary[s][1][0]), min(sm.summary[s][2][0], sm.summary[s][3][0]));
      const int tmax = max(max(sm.summary[s][0][1], sm.summary[s][1][1]), max(sm.summary[s][2][1], sm.summary[s][3][1]));
      const int tend = min(min(sm.summary[s][0][2], sm.summary[s][1][2]), min(sm.summary[s][2][2], sm.summary[s][3][2]));
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
    ptx::tc_fence_after();
    if (tid == 0) trace_event(sm, 500 + it);
    // Two rounds of 32 columns keep the register footprint small: scores of round 0 are turned into P / dS
    // while the loads of round 1 are in flight; S/dP are released to the MMA warp as soon as round 1 has landed.
    // Visibility of 32 columns as one bit mask: arithmetic for the causal bound, a short loop over the key table
    // for tiles that contain a document boundary.  One copy of the math serves every tile class.
    const int lim_eff = cls == kTileFull ? kTileN : (cls == kTileNone ? 0 : lim);
    uint32_t dm[4] = {0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu};
    if (__any_sync(0xffffffffu, cls == kTileDocs))
      warp_doc_masks(r, cls == kTileDocs, j0, sm.key_seg[s], sm.key_end[s], dm);
    const uint32_t dm_lo = half ? dm[2] : dm[0], dm_hi = half ? dm[3] : dm[1];  // this thread's 64 columns
    auto causal_mask = [&](int col0) -> uint32_t {
      const int left = lim_eff - col0;
      return left >= 32 ? 0xffffffffu : (left <= 0 ? 0u : ((1u << left) - 1u));
    };
    // P = exp2(S * scale * log2e - lse * log2e), dS = P * (dP - delta), two elements per instruction where the
    // hardware has packed fp32 forms.  A masked score becomes -inf before the exponential, so its P and dS are
    // exact zeros; a warp whose rows all see the whole tile skips the masking.
    const bool warp_full = __all_sync(0xffffffffu, cls == kTileFull);
    auto math = [&](const uint32_t (&xs)[32], const uint32_t (&ys)[32], uint32_t mask, uint32_t (&pp)[16],
                    uint32_t (&dd)[16]) {
      const float2 sc2 = make_float2(sl2, sl2), nl2 = make_float2(nl, nl), nd2 = make_float2(-dlt, -dlt);
#pragma unroll
      for (int e2 = 0; e2 < 16; ++e2) {
        float2 x = make_float2(__uint_as_float(xs[2 * e2]), __uint_as_float(xs[2 * e2 + 1]));
        if (!warp_full) {
          x.x = (mask >> (2 * e2)) & 1u ? x.x : -INFINITY;
          x.y = (mask >> (2 * e2 + 1)) & 1u ? x.y : -INFINITY;
        }
        float2 pr = __ffma2_rn(x, sc2, nl2);
        pr.x = fast_exp2(pr.x);
        pr.y = fast_exp2(pr.y);
        const float2 ds = __fmul2_rn(
            pr, __fadd2_rn(make_float2(__uint_as_float(ys[2 * e2]), __uint_as_float(ys[2 * e2 + 1])), nd2));
        pp[e2] = pack_bf16(pr.x, pr.y);
        dd[e2] = pack_bf16(ds.x, ds.y);
      }
    };
    auto store = [&](int c, const uint32_t (&pp)[16], const uint32_t (&dd)[16]) {
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int off = ((c * 4 + u) ^ (row & 7)) << 4;
        *reinterpret_cast<uint4*>(prow + off) = make_uint4(pp[4 * u], pp[4 * u + 1], pp[4 * u + 2], pp[4 * u + 3]);
        *reinterpret_cast<uint4*>(drow + off) = make_uint4(dd[4 * u], dd[4 * u + 1], dd[4 * u + 2], dd[4 * u + 3]);
      }
    };
    {
      uint32_t xs[32], ys[32], pp0[16], dd0[16], pp1[16], dd1[16];
      ptx::tmem_ld32(tmem + lane_base + half * 64, xs);
      ptx::tmem_ld32(tmem + kTileN + lane_base + half * 64, ys);
      ptx::tmem_wait_ld();
      math(xs, ys, causal_mask(half * 64) & dm_lo, pp0, dd0);
      ptx::tmem_ld32(tmem + lane_base + half * 64 + 32, xs);
      ptx::tmem_ld32(tmem + kTileN + lane_base + half * 64 + 32, ys);
      ptx::tmem_wait_ld();
      ptx::tc_fence_before();
      ptx::mbar_arrive(&sm.sdp_free);  // all scores are in registers: S/dP of the next pair may be issued
      // the store that left shared memory during the previous pair has read it by now: hand its room back without
      // having made anybody wait for it
      release();
      if (tid == 0) trace_event(sm, 800 + it);
      math(xs, ys, causal_mask(half * 64 + 32) & dm_hi, pp1, dd1);
      if (tid == 0) trace_event(sm, 900 + it);
      // the shared P / dS tiles are read by the products of the previous iteration until mma_done
      if (it > 0 && !wait_or_abort(sm, &sm.mma_done, (it - 1) & 1, 93)) return;
      ptx::tc_fence_after();
      if (tid == 0) trace_event(sm, 600 + it);
      store(0, pp0, dd0);
      store(1, pp1, dd1);
    }
    // dV / dK of a finished key tile leave TMEM before this iteration's products (which restart the accumulators)
    // can be issued, i.e. before pds_full; the shared-memory stage is released and the next tile prepared after it
    if (pending_kt >= 0) {
      if (!stage_out(pending_kt, pending_stage, it, false)) return;
      pending_kt = -1;
    }
    ptx::fence_async_shared();
    ptx::tc_fence_before();
    ptx::mbar_arrive(&sm.pds_full);
    if (tid == 0) trace_event(sm, 1000 + it);
    if (e.last && release_stage >= 0) release();  // the next key tile is waiting for this K/V stage: no deferral
    if (e.last && it + 1 < n && !prepare(resident_iter(sm.sched[it + 1]))) return;
    if (e.last) {
      pending_kt = e.kt;
      pending_stage = s;
    }
  }
  if (n > 0) {
    release();
    if (!wait_or_abort(sm, &sm.mma_done, (n - 1) & 1, 94)) return;
    ptx::tc_fence_after();
    if (pending_kt >= 0 && !stage_out(pending_kt, pending_stage, n, true)) return;
  }
  {
    // half h writes the dQ rows of query tile h
    const int qt = half;
    const int i = qt * kTileM + row;
    const bool any = true;
    bool issued = false;  // did any iteration target this query tile?
    for (int it = 0; it < n; ++it) issued = issued || (((sm.sched[it] >> 12) & 1) == static_cast<uint32_t>(qt));
    const int row_hi = half ? rb1.hi : rb0.hi;
    uint32_t packed[kHeadDim / 2];
    uint32_t raw[2][32];
    if (issued && any) {
      ptx::tmem_ld32(tmem + 2 * kTileN + 2 * kHeadDim + qt * kHeadDim + lane_base, raw[0]);
      ptx::tmem_ld32(tmem + 2 * kTileN + 2 * kHeadDim + qt * kHeadDim + lane_base + 32, raw[1]);
      ptx::tmem_wait_ld();
    }
#pragma unroll
    for (int c = 0; c < 2; ++c) {
#pragma unroll
      for (int e2 = 0; e2 < 16; ++e2)
        packed[c * 16 + e2] = issued && any && row_hi > 0
                                  ? pack_bf16(__uint_as_float(raw[c][2 * e2]) * a.scale, __uint_as_float(raw[c][2 * e2 + 1]) * a.scale)
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


__global__ void __launch_bounds__(kResidentThreads, 1)
    attn_bwd_resident_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                        const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_g,
                        const __grid_constant__ CUtensorMap map_dk, const __grid_constant__ CUtensorMap map_dv,
                        const wm_attn_args a, const float* delta, const int epoch) {
  extern __shared__ unsigned char smem_raw[];
  ResidentShared& sm = *reinterpret_cast<ResidentShared*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
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
  if (tid < kResidentCompute) {
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
  ResidentWalk w;
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
    // the list of visible (key tile, query tile) pairs, in execution order
    int n = 0, active = 0;
    for (int kt = 0; kt < w.n_kt; ++kt) {
      const bool v0 = pair_visible(w, kt, 0), v1 = pair_visible(w, kt, 1);
      if (!v0 && !v1) continue;
      if (v0) sm.sched[n++] = kt | (0u << 12) | (1u << 13) | ((v1 ? 0u : 1u) << 14) | (static_cast<uint32_t>(active) << 16);
      if (v1) sm.sched[n++] = kt | (1u << 12) | ((v0 ? 0u : 1u) << 13) | (1u << 14) | (static_cast<uint32_t>(active) << 16);
      ++active;
    }
    sm.n_iter = n;
    int q0_last = -1;
    for (int i = 0; i < n; ++i)
      if (((sm.sched[i] >> 12) & 1) == 0) q0_last = i;
    sm.q0_last_iter = q0_last;
    ptx::mbar_init(&sm.qg_full, 1);
    for (int s = 0; s < 2; ++s) {
      ptx::mbar_init(&sm.kv_full[s], 1);
      ptx::mbar_init(&sm.kv_ready[s], kResidentCompute);
      ptx::mbar_init(&sm.kv_empty[s], 2);  // the two halves' store threads release a stage
      ptx::mbar_init(&sm.out_full[s], kTileM);
      ptx::mbar_init(&sm.stage_free[s], 1);
    }
    ptx::mbar_init(&sm.sdp_full, 1);
    ptx::mbar_init(&sm.sdp_free, kResidentCompute);
    ptx::mbar_init(&sm.pds_full, kResidentCompute);
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
    resident_compute(sm, a, tmem, w, delta, head, batch, &map_dk, &map_dv);
  } else if (warp == 8) {
    if (lane == 0) resident_producer(sm, &map_q, &map_k, &map_v, &map_g, w, head, batch);
  } else if (warp == 9) {
    if (lane == 0) resident_mma_scores(sm, tmem);
  } else {
    if (lane == 0) resident_mma_grads(sm, tmem, w.nq);
  }
  ptx::tma_store_wait_all();
  ptx::tc_fence_before();
  __syncthreads();
  trace_flush(sm);
  if (warp == 8) ptx::tmem_dealloc(tmem, kTmemCols);
}
