// Backward pipeline for short query axes (included by attn_tc.cu).
//
// Cyclic attention with stride S has S times fewer queries than keys.  When a (batch, head) has
// at most 256 queries and query heads are not grouped, one block keeps both query tiles (Q, dO:
// 64 KB) and their dQ accumulators (TMEM) resident and walks over the key tiles: dK and dV of a
// key tile are complete inside the block and leave through one TMA store each, dQ is written
// once at the end -- no atomics, no fp32 scratch, no conversion pass.  K and V tiles stream
// through a two-stage TMA ring; once the first query tile has no pair left (or when there is only
// one query tile), the Q / dO room of the idle query tile joins the ring as a third stage, which
// is what lets the S / dP products of key tiles seen by one query tile only be issued while the
// pair before them is still being computed.
//
// 384 threads: warps 0-7 compute (thread = query row (tid & 127), column half (tid >> 7) of the
// 128-key tile), warp 8 TMA producer, warps 9 and 10 MMA issuers (S/dP products, gradient products), warp 11
// stores finished dK / dV tiles and hands their stage back.
// TMEM: S [0,128) dP [128,256) dV [256,320) dK [320,384) dQ0 [384,448) dQ1 [448,512).
//
// An iteration is one (key tile, query tile) pair; the list of visible pairs is built once per
// block.  The compute warps pull S and dP of iteration i out of TMEM into registers and release
// them at once (sdp_free), so the MMA warp issues S/dP of iteration i+1 while the exponentials of
// iteration i are still being computed; P and dS of iteration i are written to shared memory only
// after the dV/dK/dQ products of iteration i-1 have read the previous contents (mma_done).
#pragma once

constexpr int kResidentThreads = 384;
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
  const int hi = qt ? w.hi_max[1] : w.hi_max[0], lo = qt ? w.lo_min[1] : w.lo_min[0];
  if (j0 >= hi) return false;
  if (w.docs && j0 + kTileN - 1 < lo && !(w.dummy && kt == 0)) return false;
  return true;
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
  uint64_t kv_full[3], kv_ready[3], kv_empty[3];
  uint64_t sdp_full, sdp_free, pds_full, mma_done;
  uint64_t out_full[2];  // dV (half 0) / dK (half 1) rows of a finished key tile are staged in shared memory
  uint64_t out_seen;     // the storing thread has taken note of both
  int key_seg[3][kTileN];
  int key_end[3][kTileN];
  int summary[3][4][3];
  int lo_min[2], hi_max[2];
  int has_dummy;
  // iteration list: key tile | query tile << 12 | first-of-key-tile << 13 | last-of-key-tile << 14 | K/V stage << 15 |
  // parity of this use of the stage (kv_full, kv_ready) << 17 | parity the producer waits for on kv_empty << 18 |
  // dK/dV of the tile go straight to global memory << 19
  uint32_t sched[kResidentMaxIter];
  int n_iter;
  int n_visited;     // key tiles on the list
  int q0_last_iter;  // last iteration that uses query tile 0 (-1: none)
  uint32_t tmem_base;
  int abort_flag;
  int epoch;
  WM_TRACE_FIELDS
};

struct ResidentIter {
  int kt, qt, first, last, stage, parity, empty_parity, direct;
};

__device__ __forceinline__ ResidentIter resident_iter(uint32_t e) {
  ResidentIter it;
  it.kt = e & 0xfff;
  it.qt = (e >> 12) & 1;
  it.first = (e >> 13) & 1;
  it.last = (e >> 14) & 1;
  it.stage = (e >> 15) & 3;
  it.parity = (e >> 17) & 1;
  it.empty_parity = (e >> 18) & 1;
  it.direct = (e >> 19) & 1;
  return it;
}

// K / V room of a stage: stages 0 and 1 are the ring's own, stage 2 is the Q / dO room of the idle query tile
// (query tile 1 when the tensor has only one, else query tile 0 once it has no pair left)
template <class Shared>
__device__ __forceinline__ unsigned char* resident_k_stage(Shared& sm, int stage, int nq) {
  return stage < 2 ? sm.k[stage] : sm.q[nq == 1 ? 1 : 0];
}
template <class Shared>
__device__ __forceinline__ unsigned char* resident_v_stage(Shared& sm, int stage, int nq) {
  return stage < 2 ? sm.v[stage] : sm.g[nq == 1 ? 1 : 0];
}

// Q and dO of the block's query tiles: they depend on nothing the block works out first, so they are on their way
// while the row bounds and the iteration list are still being made.
template <class Shared>
__device__ __forceinline__ void resident_load_queries(Shared& sm, const CUtensorMap* map_q, const CUtensorMap* map_g, int nq,
                                                  int head, int batch) {
  ptx::prefetch_tmap(map_q);
  ptx::prefetch_tmap(map_g);
  ptx::mbar_expect_tx(&sm.qg_full, 2 * nq * kTileBytes);
  for (int qt = 0; qt < nq; ++qt) {
    ptx::tma_load_4d(sm.q[qt], map_q, &sm.qg_full, 0, qt * kTileM, head, batch);
    ptx::tma_load_4d(sm.g[qt], map_g, &sm.qg_full, 0, qt * kTileM, head, batch);
  }
}

template <class Shared>
__device__ __forceinline__ void resident_producer(Shared& sm, const CUtensorMap* map_k, const CUtensorMap* map_v,
                                              const ResidentWalk& w, int head, int batch) {
  ptx::prefetch_tmap(map_k);
  ptx::prefetch_tmap(map_v);
  const int n = sm.n_iter;
  bool third_checked = false;
  for (int it = 0; it < n; ++it) {
    const ResidentIter e = resident_iter(sm.sched[it]);
    if (!e.first) continue;
    // the third stage is the room of a query tile: whatever was loaded there at the start has to have landed
    if (e.stage == 2 && !third_checked) {
      if (!wait_or_abort(sm, &sm.qg_full, 0, 72)) return;
      third_checked = true;
    }
    if (!wait_or_abort(sm, &sm.kv_empty[e.stage], e.empty_parity, 71)) return;
    ptx::mbar_expect_tx(&sm.kv_full[e.stage], 2 * kTileBytes);
    ptx::tma_load_4d(resident_k_stage(sm, e.stage, w.nq), map_k, &sm.kv_full[e.stage], 0, e.kt * kTileN, head, batch);
    ptx::tma_load_4d(resident_v_stage(sm, e.stage, w.nq), map_v, &sm.kv_full[e.stage], 0, e.kt * kTileN, head, batch);
  }
}

__device__ __forceinline__ void resident_issue_sdp(ResidentShared& sm, uint32_t tmem, const ResidentIter& e, int nq) {
  constexpr uint32_t idesc_s = ptx::make_idesc_bf16(kTileM, kTileN, 0, 0);
  const uint32_t q_base = ptx::smem_u32(sm.q[e.qt]), g_base = ptx::smem_u32(sm.g[e.qt]);
  const uint32_t k_base = ptx::smem_u32(resident_k_stage(sm, e.stage, nq));
  const uint32_t v_base = ptx::smem_u32(resident_v_stage(sm, e.stage, nq));
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
__device__ __forceinline__ void resident_mma_scores(ResidentShared& sm, uint32_t tmem, int nq, int kvis) {
  const int n = sm.n_iter;
  if (n == 0) return;
  if (!wait_or_abort(sm, &sm.qg_full, 0, 80)) return;
  for (int it = 0; it < n; ++it) {
    const ResidentIter e = resident_iter(sm.sched[it]);
    // S/dP of the previous pair are in the compute warps' registers: this pair may overwrite them
    if (it > 0 && !wait_or_abort(sm, &sm.sdp_free, (it - 1) & 1, 83)) return;
    // K and V straight from the TMA are good enough for these products, so a key tile does not wait for the
    // compute warps to get round to it -- unless they have rows to clear in it (keys behind the last visible one)
    if (e.first) {
      const bool cleared = e.kt * kTileN + kTileN > kvis;
      if (!wait_or_abort(sm, cleared ? &sm.kv_ready[e.stage] : &sm.kv_full[e.stage], e.parity, 81)) return;
    }
    ptx::tc_fence_after();
    trace_event(sm, 100 + it);
    resident_issue_sdp(sm, tmem, e, nq);
    trace_event(sm, 200 + it);
  }
}

__device__ __forceinline__ void resident_mma_grads(ResidentShared& sm, uint32_t tmem, int nq) {
  const int n = sm.n_iter;
  if (n == 0) return;
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
    const uint32_t q_base = ptx::smem_u32(sm.q[e.qt]), g_base = ptx::smem_u32(sm.g[e.qt]);
    const uint32_t k_base = ptx::smem_u32(resident_k_stage(sm, e.stage, nq));
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
    // a tile whose gradients will not be staged in its K/V stage gives the stage back as soon as these products
    // have read it
    if (e.direct) ptx::mma_commit(&sm.kv_empty[e.stage]);
    if (nq > 1 && it == sm.q0_last_iter) {
      // these were the last products that read Q / dO of the first query tile: once they are complete its room
      // is the ring's third stage
      ptx::mma_commit(&sm.kv_empty[2]);
    }
    trace_event(sm, 400 + it);
  }
}

// One thread stores the finished dV / dK tiles: it waits until the compute warps have staged both halves of a
// key tile, issues the two TMA stores, and gives the K/V stage back to the producer as soon as the stores have
// read it, so nobody who has math to do waits for that.
__device__ __forceinline__ void resident_store(ResidentShared& sm, const CUtensorMap* map_dk, const CUtensorMap* map_dv,
                                           int nq, int head, int batch) {
  ptx::prefetch_tmap(map_dk);
  ptx::prefetch_tmap(map_dv);
  const int n = sm.n_iter;
  int tiles = 0;
  for (int it = 0; it < n; ++it) {
    const ResidentIter e = resident_iter(sm.sched[it]);
    if (!e.last || e.direct) continue;
    if (!wait_or_abort(sm, &sm.out_full[0], tiles & 1, 97)) return;
    if (!wait_or_abort(sm, &sm.out_full[1], tiles & 1, 98)) return;
    ptx::mbar_arrive(&sm.out_seen);
    ptx::tma_store_4d(map_dv, resident_v_stage(sm, e.stage, nq), 0, e.kt * kTileN, head, batch);
    ptx::tma_store_4d(map_dk, resident_k_stage(sm, e.stage, nq), 0, e.kt * kTileN, head, batch);
    ptx::tma_store_commit();
    ptx::tma_store_wait_read();
    ptx::mbar_arrive(&sm.kv_empty[e.stage]);
    ++tiles;
  }
}

__device__ __forceinline__ void resident_compute(ResidentShared& sm, const wm_attn_args& a, uint32_t tmem, const ResidentWalk& w,
                                             float lse0, float lse1, float dl0, float dl1, int head, int batch) {
  const float nl0 = -lse0 * kLog2e, nl1 = -lse1 * kLog2e;
  const int tid = threadIdx.x;
  const int row = tid & 127;
  const int half = tid >> 7;
  const int warp = tid >> 5, lane = tid & 31;
  const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
  const float sl2 = a.scale * kLog2e;
  const GroupCtx g = group_ctx(a, 0);
  const int n = sm.n_iter;

  // this thread's row in both query tiles (its -lse * log2(e) and delta were fetched when the kernel began)
  RowBound rb0, rb1;
  bool live0 = false, live1 = false;
  {
    rb0.lo = rb0.hi = rb0.seg = 0;
    rb0.qi = row;
    rb1 = rb0;
    rb1.qi = kTileM + row;
    if (row < a.q_len) {
      live0 = true;
      rb0 = row_bound(a, g, batch, row);
    }
    if (w.nq > 1 && kTileM + row < a.q_len) {
      live1 = true;
      rb1 = row_bound(a, g, batch, kTileM + row);
    }
  }
  unsigned char* prow = sm.p + half * kTileBytes + (row >> 3) * 1024 + (row & 7) * 128;
  unsigned char* drow = sm.ds + half * kTileBytes + (row >> 3) * 1024 + (row & 7) * 128;

  // key tiles nobody sees get exact zeros; they are not part of the iteration list
  if (sm.n_visited != w.n_kt) {
    for (int kt = 0; kt < w.n_kt; ++kt)
      if (!pair_visible(w, kt, 0) && !pair_visible(w, kt, 1)) resident_store_dkv(a, tmem, kt, row, half, lane_base, head, batch, true);
  }

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
    const int s = e.stage;
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
    if (!wait_or_abort(sm, &sm.kv_full[s], e.parity, 90)) return false;
    if (j0 + row >= w.kvis) {
      uint4* dst = reinterpret_cast<uint4*>((half ? resident_v_stage(sm, s, w.nq) : resident_k_stage(sm, s, w.nq)) + row * 128);
#pragma unroll
      for (int c = 0; c < 8; ++c) dst[c] = make_uint4(0, 0, 0, 0);
    }
    ptx::fence_async_shared();
    ptx::mbar_arrive(&sm.kv_ready[s]);
    return true;
  };
  // every compute thread has prepared the tile: its document table is complete
  auto prepared = [&](const ResidentIter& e) -> bool {
    return wait_or_abort(sm, &sm.kv_ready[e.stage], e.parity, 91);
  };

  // dV / dK of a finished key tile: TMEM -> bf16 -> the tile's own (now idle) V / K stage in shared memory, in
  // the 128B-swizzled row layout of the output tensor map.  The storing thread (warp 11) takes it from there: one
  // TMA store per half, and the stage goes back to the producer once the stores have read it.
  int outs = 0;  // staged tiles so far (parity of out_full)
  auto stage_out = [&](int stage) -> bool {
    const float sc = half ? a.scale : 1.f;
    unsigned char* tile = half ? resident_k_stage(sm, stage, w.nq) : resident_v_stage(sm, stage, w.nq);
    // the storing thread is a single lane: it has to have seen the previous phase of out_full before this one
    // can be allowed to complete, or it could take the next completed phase for the one it is waiting for
    if (outs > 0 && !wait_or_abort(sm, &sm.out_seen, (outs - 1) & 1, 96)) return false;
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
    ++outs;
    return true;
  };

  // The other way out, for a key tile with one pair whose successor has one pair too while only two stages are
  // open: there the load after next would wait for the staged gradients to leave this tile's stage, and the compute
  // warps for that load.  Each thread writes its key row's 128 bytes of dV or dK itself (twice the time of the
  // staging), and the gradient issuer's commit has handed the stage back long before.
  auto direct_out = [&](int kt) {
    const float sc = half ? a.scale : 1.f;
    const int j = kt * kTileN + row;
    const int64_t* st = half ? a.dk_strides : a.dv_strides;
    uint4* dst = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(half ? a.dk : a.dv) + batch * st[0] + head * st[1] +
                                          static_cast<long long>(j) * st[2]);
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
      uint32_t raw[32];
      ptx::tmem_ld32(tmem + 2 * kTileN + half * kHeadDim + lane_base + h2 * 32, raw);
      ptx::tmem_wait_ld();
      if (j < a.k_len) {
        const bool sectors = (reinterpret_cast<uintptr_t>(dst) & 31) == 0;  // rows the caller laid out on 32 bytes
#pragma unroll
        for (int c = 0; c < 2; ++c) {  // whole 32-byte sectors: partial ones are what makes scattered rows slow
          uint32_t pk[8];
#pragma unroll
          for (int e2 = 0; e2 < 8; ++e2)
            pk[e2] = pack_bf16(__uint_as_float(raw[c * 16 + 2 * e2]) * sc, __uint_as_float(raw[c * 16 + 2 * e2 + 1]) * sc);
          if (sectors) {
            ptx::st_global_v8(dst + h2 * 4 + c * 2, pk);
          } else {
            dst[h2 * 4 + c * 2] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            dst[h2 * 4 + c * 2 + 1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
          }
        }
      }
    }
  };

  if (n > 0 && !prepare(resident_iter(sm.sched[0]))) return;
  int pending_kt = -1, pending_stage = 0;
  bool pending_direct = false;
  for (int it = 0; it < n; ++it) {
    const ResidentIter e = resident_iter(sm.sched[it]);
    if (e.first && !prepared(e)) return;
    if (e.last && it + 1 < n) fetch_table(resident_iter(sm.sched[it + 1]).kt);
    const int s = e.stage;
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
    // can be issued, i.e. before pds_full; the next tile is prepared after it
    if (pending_kt >= 0) {
      if (pending_direct) direct_out(pending_kt);
      else if (!stage_out(pending_stage)) return;
      pending_kt = -1;
    }
    ptx::fence_async_shared();
    ptx::tc_fence_before();
    ptx::mbar_arrive(&sm.pds_full);
    if (tid == 0) trace_event(sm, 1000 + it);
    if (e.last && it + 1 < n && !prepare(resident_iter(sm.sched[it + 1]))) return;
    if (e.last) {
      pending_kt = e.kt;
      pending_stage = s;
      pending_direct = e.direct != 0;
    }
  }
  if (n > 0) {
    if (!wait_or_abort(sm, &sm.mma_done, (n - 1) & 1, 94)) return;
    ptx::tc_fence_after();
    if (pending_kt >= 0) {
      if (pending_direct) direct_out(pending_kt);
      else if (!stage_out(pending_stage)) return;
    }
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
      if ((reinterpret_cast<uintptr_t>(dst) & 31) == 0) {  // whole 32-byte sectors
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const uint32_t pk[8] = {packed[8 * c],     packed[8 * c + 1], packed[8 * c + 2], packed[8 * c + 3],
                                  packed[8 * c + 4], packed[8 * c + 5], packed[8 * c + 6], packed[8 * c + 7]};
          ptx::st_global_v8(dst + 2 * c, pk);
        }
      } else {
#pragma unroll
        for (int c = 0; c < 8; ++c)
          dst[c] = make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
      }
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

  const int nq = (a.q_len + kTileM - 1) / kTileM;
  if (tid == 0) {
    sm.abort_flag = 0;
    sm.epoch = epoch;
    trace_begin(sm, epoch);
    trace_event(sm, 1);
    sm.lo_min[0] = sm.lo_min[1] = INT_MAX;
    sm.hi_max[0] = sm.hi_max[1] = 0;
    ptx::mbar_init(&sm.qg_full, 1);
    for (int s = 0; s < 3; ++s) {
      ptx::mbar_init(&sm.kv_full[s], 1);
      ptx::mbar_init(&sm.kv_ready[s], kResidentCompute);
      ptx::mbar_init(&sm.kv_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) ptx::mbar_init(&sm.out_full[s], kTileM);
    ptx::mbar_init(&sm.out_seen, 1);
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
  // The compute threads' row statistics (thread = query row (tid & 127) of both query tiles) are asked for now
  // and first used when the first scores are there.
  float lse0 = INFINITY, lse1 = INFINITY, dl0 = 0.f, dl1 = 0.f;
  RowBound own;  // bounds of query `tid`, for the block's key range
  own.lo = own.hi = own.seg = own.qi = 0;
  if (tid < kResidentCompute && tid < a.q_len) own = row_bound(a, g, batch, tid);
  if (tid < kResidentCompute) {
    const int row = tid & 127;
    const long long stat = (static_cast<long long>(batch) * a.q_heads + head) * a.q_len + row;
    if (row < a.q_len) {
      lse0 = a.lse[stat];
      dl0 = delta[stat];
    }
    if (nq > 1 && kTileM + row < a.q_len) {
      lse1 = a.lse[stat + kTileM];
      dl1 = delta[stat + kTileM];
    }
  }
  __syncthreads();
  if (tid == kResidentCompute) resident_load_queries(sm, &map_q, &map_g, nq, head, batch);
  // (a thread that has no row waits for this load, beside the rows' own loads)
  if (tid == kResidentThreads - 1) sm.has_dummy = a.q_seg != nullptr && a.k_seg[static_cast<long long>(batch) * a.k_len] == -1;
  if (tid < kResidentCompute) {
    const int qt = tid >> 7;
    int lo = INT_MAX, hi = 0;
    if (tid < a.q_len) {
      hi = own.hi;
      if (own.hi > 0) lo = own.lo;
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
  w.nq = nq;
  w.n_kt = (a.k_len + kTileN - 1) / kTileN;
  w.lo_min[0] = sm.lo_min[0];
  w.lo_min[1] = sm.lo_min[1];
  w.hi_max[0] = sm.hi_max[0];
  w.hi_max[1] = sm.hi_max[1];
  w.kvis = max(w.hi_max[0], w.hi_max[1]);
  w.docs = a.q_seg != nullptr;
  w.dummy = sm.has_dummy != 0;
  if (warp == 0) {
    // The list of visible (key tile, query tile) pairs, in execution order: one lane per key tile decides, the
    // positions come from ballots.  (Bits 20 and up carry the tile's visit index until the stages are assigned.)
    int n = 0, tiles = 0, q0_last = -1;
    for (int base = 0; base < w.n_kt; base += 32) {
      const int kt = base + lane;
      const bool v0 = kt < w.n_kt && pair_visible(w, kt, 0), v1 = kt < w.n_kt && pair_visible(w, kt, 1);
      const uint32_t m0 = __ballot_sync(0xffffffffu, v0), m1 = __ballot_sync(0xffffffffu, v1);
      const uint32_t below = (1u << lane) - 1u;
      const int at = n + __popc(m0 & below) + __popc(m1 & below);
      const uint32_t visit = static_cast<uint32_t>(tiles + __popc((m0 | m1) & below)) << 20;
      if (v0) {
        sm.sched[at] = kt | (0u << 12) | (1u << 13) | ((v1 ? 0u : 1u) << 14) | visit;
        q0_last = max(q0_last, at);
      }
      if (v1) sm.sched[at + (v0 ? 1 : 0)] = kt | (1u << 12) | ((v0 ? 0u : 1u) << 13) | (1u << 14) | visit;
      n += __popc(m0) + __popc(m1);
      tiles += __popc(m0 | m1);
    }
    q0_last = __reduce_max_sync(0xffffffffu, q0_last);
    __syncwarp();
    // K/V stage of every visited key tile.  Stages 0 and 1 alternate; from the tile after the first one that
    // starts behind the first query tile's last pair (t0), the idle query tile's room joins as stage 2 and the
    // three take turns (the stage unused for longest comes next).  With one query tile that is so from the start.
    // Stage 2 begins its life full (Q / dO of the first query tile) unless there is only one query tile or the
    // first query tile has no pair at all, so there the producer's first wait is for a completed phase.
    const int third_from = w.nq == 1 ? 0 : q0_last + 1;  // first iteration behind the first query tile's pairs
    const bool third_starts_full = w.nq > 1 && q0_last >= 0;
    int t0 = INT_MAX;
    for (int i = lane; i < n; i += 32) {
      const uint32_t entry = sm.sched[i];
      if (((entry >> 13) & 1) && i >= third_from) t0 = min(t0, static_cast<int>(entry >> 20));
    }
    t0 = __reduce_min_sync(0xffffffffu, t0);
    for (int i = lane; i < n; i += 32) {
      const uint32_t entry = sm.sched[i];
      const int tile = static_cast<int>(entry >> 20);
      int stage = tile & 1, use = tile >> 1;  // how often the stage was used before
      if (tile > t0) {
        const int d = tile - t0 - 1, r = d % 3, c = d / 3;
        stage = r == 0 ? 2 : (r == 1 ? ((t0 + 1) & 1) : (t0 & 1));
        use = r == 0 ? c : ((t0 + 2 - stage) >> 1) + c;  // tiles up to t0 with the stage's parity, then every third
      }
      const int empty_parity = stage == 2 && third_starts_full ? (use & 1) : ((use & 1) ^ 1);
      // one pair here, one pair in the next tile, and the third stage not yet open: gradients go out directly
      // (the first / last bits of the follower read here are the same before and after its own rewrite)
      const uint32_t single = (1u << 13) | (1u << 14);
      const uint32_t follower = i + 1 < n ? sm.sched[i + 1] : 0u;
      const bool direct = tile <= t0 && (entry & single) == single && (follower & single) == single;
      sm.sched[i] = (entry & 0x7fffu) | (static_cast<uint32_t>(stage) << 15) | (static_cast<uint32_t>(use & 1) << 17) |
                    (static_cast<uint32_t>(empty_parity) << 18) | ((direct ? 1u : 0u) << 19);
    }
    if (lane == 0) {
      sm.n_iter = n;
      sm.n_visited = tiles;
      sm.q0_last_iter = q0_last;
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = sm.tmem_base;
  if (tid == 0) trace_event(sm, 2);
  if (warp < 8) {
    resident_compute(sm, a, tmem, w, lse0, lse1, dl0, dl1, head, batch);
  } else if (warp == 8) {
    if (lane == 0) resident_producer(sm, &map_k, &map_v, w, head, batch);
  } else if (warp == 9) {
    if (lane == 0) resident_mma_scores(sm, tmem, w.nq, w.kvis);
  } else if (warp == 10) {
    if (lane == 0) resident_mma_grads(sm, tmem, w.nq);
  } else {
    if (lane == 0) resident_store(sm, &map_dk, &map_dv, w.nq, head, batch);
  }
  if (tid == 0) trace_event(sm, 3);
  ptx::tma_store_wait_all();
  ptx::tc_fence_before();
  __syncthreads();
  if (tid == 0) trace_event(sm, 4);
  trace_flush(sm);
  if (warp == 8) ptx::tmem_dealloc(tmem, kTmemCols);
}
