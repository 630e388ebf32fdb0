// Backward pipeline for short query axes, key rows on the TMEM lanes (included by attn_tc.cu).
//
// Cyclic attention with stride S has S times fewer queries than keys.  When a (batch, head) has at most 256
// queries and query heads are not grouped, one block keeps all of Q and dO (64 KB) and the dQ accumulators (TMEM)
// resident and walks over the key tiles; dK and dV of a key tile are complete inside the block and leave through
// one TMA store each, dQ is written once at the end -- no atomics, no fp32 scratch, no conversion pass.
//
// The products are laid out the other way round from the forward: S^T = K Q^T and dP^T = V dO^T put the 128 keys of
// a tile on the TMEM lanes and the queries on the columns.  With a strided mask the 128 keys of a tile differ by at
// most 128/S queries in where their visibility begins, so the visible queries of a key tile are (nearly) the same
// column range for every lane: that range is cut into chunks of 64 queries, only chunks (and, inside them, only
// 16-column pieces) that some key can see are computed, and the four lane quarters always carry the same load.
// P^T and dS^T (thread = key row) go back into TMEM as packed bf16 over the scores they were made from and feed
// dV += P^T dO and dK += dS^T Q as TMEM operands; only dS^T is also written to shared memory, once, as the
// (MN-major) A operand of dQ += dS K.
//
// 384 threads: warps 0-3 and 4-7 are two compute groups that take alternate chunks (thread = key row of the tile),
// warp 8 TMA producer, warp 9 issues the S^T / dP^T products, warp 10 the gradient products, warp 11 stores finished
// dK / dV tiles.  TMEM columns: per group g a score buffer [128g, 128g+128) (S^T 64 columns, dP^T 64 columns; P^T
// and dS^T packed over the first 32 columns of either), dV [256,320), dK [320,384), dQ of query block 0 and 1
// [384,448), [448,512).
#pragma once

constexpr int kKeysThreads = 384;
constexpr int kKeysCompute = 256;
constexpr int kKeysGroup = 128;
constexpr int kChunk = 64;          // queries per chunk
constexpr int kMaxQueries = 256;    // two query blocks of 128
constexpr int kKeysMaxTiles = 128;  // key tiles per (batch, head)
constexpr uint32_t kColDv = 256, kColDk = 320, kColDq = 384;

struct KeysShared {
  unsigned char q[2][kTileBytes];   // query block b: rows 128b .. 128b+127
  unsigned char g[2][kTileBytes];   // dO, same layout
  unsigned char k[2][kTileBytes];   // K / V stages; finished dK / dV tiles are staged here for their TMA store
  unsigned char v[2][kTileBytes];
  unsigned char ds[4][kTileBytes];  // dS^T of the current key tile: slot c holds queries 64c .. 64c+63 (key rows x 128 B)
  float nl2[kMaxQueries];           // -lse * log2(e) per query (-inf: the row has no key, or there is no such query)
  float nd[kMaxQueries];            // -delta per query
  int q_seg[kMaxQueries], q_lo[kMaxQueries], q_hi[kMaxQueries];
  uint32_t tile_q[kKeysMaxTiles];   // first | (last + 1) << 16 of the queries that may see the key tile (empty: not visited)
  uint64_t qg_full;
  uint64_t kv_full[2], kv_empty[2];
  uint64_t sp_full[2], pds_full[2], grads_done[2];
  uint64_t dkv_free, out_full, out_seen;
  int has_dummy;
  int kvis;
  uint32_t tmem_base;
  int abort_flag;
  int epoch;
  WM_TRACE_FIELDS
};

// The walk over (key tile, chunk) that every role repeats for itself: visited key tiles in order, and inside a
// tile the chunk slots that hold a query which may see it.
struct KeysTile {
  int qb, qe;   // queries that may see the tile
  int c0, c1;   // first and last chunk slot
  int lo16, hi16;  // the query range widened to multiples of 16 (the granularity of the products)
};

__device__ __forceinline__ bool keys_tile(const KeysShared& sm, int kt, KeysTile& t) {
  const uint32_t e = sm.tile_q[kt];
  t.qb = static_cast<int>(e & 0xffffu);
  t.qe = static_cast<int>(e >> 16);
  if (t.qe <= t.qb) return false;
  t.c0 = t.qb / kChunk;
  t.c1 = (t.qe - 1) / kChunk;
  t.lo16 = t.qb & ~15;
  t.hi16 = (t.qe + 15) & ~15;
  return true;
}

// columns [n0, n1) of chunk slot c that the products of this tile cover (multiples of 16)
__device__ __forceinline__ void keys_chunk_range(const KeysTile& t, int c, int& n0, int& n1) {
  n0 = max(t.lo16 - kChunk * c, 0);
  n1 = min(t.hi16 - kChunk * c, kChunk);
}

__device__ __forceinline__ unsigned long long below64(int n) {
  return n >= 64 ? ~0ull : (n <= 0 ? 0ull : ((1ull << n) - 1ull));
}

// ------------------------------------------------------------------ producer (one lane)
__device__ __forceinline__ void keys_producer(KeysShared& sm, const CUtensorMap* map_k, const CUtensorMap* map_v, int n_kt,
                                              int head, int batch) {
  ptx::prefetch_tmap(map_k);
  ptx::prefetch_tmap(map_v);
  int t = 0;
  for (int kt = 0; kt < n_kt; ++kt) {
    KeysTile tl;
    if (!keys_tile(sm, kt, tl)) continue;
    const int s = t & 1;
    // the stage is free again when the dK / dV tile that was staged in it has been read by its store
    if (t >= 2 && !wait_or_abort(sm, &sm.kv_empty[s], ((t >> 1) & 1) ^ 1, 71)) return;
    ptx::mbar_expect_tx(&sm.kv_full[s], 2 * kTileBytes);
    ptx::tma_load_4d(sm.k[s], map_k, &sm.kv_full[s], 0, kt * kTileN, head, batch);
    ptx::tma_load_4d(sm.v[s], map_v, &sm.kv_full[s], 0, kt * kTileN, head, batch);
    ++t;
  }
}

// ------------------------------------------------------------------ S^T / dP^T products (one lane)
__device__ __forceinline__ void keys_mma_scores(KeysShared& sm, uint32_t tmem, int n_kt) {
  bool started = false;
  int t = 0, n = 0;
  for (int kt = 0; kt < n_kt; ++kt) {
    KeysTile tl;
    if (!keys_tile(sm, kt, tl)) continue;
    if (!started) {
      if (!wait_or_abort(sm, &sm.qg_full, 0, 80)) return;
      started = true;
    }
    const int s = t & 1;
    if (!wait_or_abort(sm, &sm.kv_full[s], (t >> 1) & 1, 81)) return;
    const uint64_t a_k = ptx::make_smem_desc_sw128(ptx::smem_u32(sm.k[s]), 16, 1024);
    const uint64_t a_v = ptx::make_smem_desc_sw128(ptx::smem_u32(sm.v[s]), 16, 1024);
    for (int c = tl.c0; c <= tl.c1; ++c, ++n) {
      const int grp = n & 1;
      int n0, n1;
      keys_chunk_range(tl, c, n0, n1);
      // P^T / dS^T of the group's previous chunk live in this buffer until their gradient products have read them
      if (n >= 2 && !wait_or_abort(sm, &sm.grads_done[grp], ((n >> 1) & 1) ^ 1, 83)) return;
      ptx::tc_fence_after();
      trace_event(sm, 100 + n);
      const uint32_t idesc = ptx::make_idesc_bf16(kTileN, n1 - n0, 0, 0);
      const int qrow = kChunk * c + n0;
      const uint32_t row_bytes = static_cast<uint32_t>(qrow & 127) * 128u;
      const uint64_t b_q = ptx::make_smem_desc_sw128(ptx::smem_u32(sm.q[qrow >> 7]) + row_bytes, 16, 1024);
      const uint64_t b_g = ptx::make_smem_desc_sw128(ptx::smem_u32(sm.g[qrow >> 7]) + row_bytes, 16, 1024);
      const uint32_t d = tmem + static_cast<uint32_t>(grp * 128 + n0);
#pragma unroll
      for (int kk = 0; kk < kHeadDim / 16; ++kk)
        ptx::mma_bf16_ss(d, ptx::desc_advance(a_k, kk * 32), ptx::desc_advance(b_q, kk * 32), idesc, kk > 0);
#pragma unroll
      for (int kk = 0; kk < kHeadDim / 16; ++kk)
        ptx::mma_bf16_ss(d + kChunk, ptx::desc_advance(a_v, kk * 32), ptx::desc_advance(b_g, kk * 32), idesc, kk > 0);
      ptx::mma_commit(&sm.sp_full[grp]);
      trace_event(sm, 200 + n);
    }
    ++t;
  }
}

// ------------------------------------------------------------------ gradient products (one lane)
__device__ __forceinline__ void keys_mma_grads(KeysShared& sm, uint32_t tmem, int n_kt) {
  constexpr uint32_t idesc_ts = ptx::make_idesc_bf16(kTileN, kHeadDim, 0, 1);  // A from TMEM, B (dO, Q) head_dim contiguous
  constexpr uint32_t idesc_dq = ptx::make_idesc_bf16(kTileM, kHeadDim, 1, 1);  // A = dS^T rows (queries contiguous), B = K
  bool dq_started[2] = {false, false};
  int t = 0, n = 0;
  for (int kt = 0; kt < n_kt; ++kt) {
    KeysTile tl;
    if (!keys_tile(sm, kt, tl)) continue;
    const int s = t & 1;
    const uint64_t b_k = ptx::make_smem_desc_sw128(ptx::smem_u32(sm.k[s]), 1024, 1024);
    for (int c = tl.c0; c <= tl.c1; ++c, ++n) {
      const int grp = n & 1;
      int n0, n1;
      keys_chunk_range(tl, c, n0, n1);
      if (!wait_or_abort(sm, &sm.pds_full[grp], (n >> 1) & 1, 82)) return;
      // the dV / dK accumulators restart with a tile's first chunk: the previous tile has to have left them
      if (c == tl.c0 && t > 0 && !wait_or_abort(sm, &sm.dkv_free, (t - 1) & 1, 85)) return;
      ptx::tc_fence_after();
      trace_event(sm, 300 + n);
      const uint32_t p_tmem = tmem + static_cast<uint32_t>(grp * 128);
      const int ks0 = n0 >> 4, ks1 = n1 >> 4;
      const int qrow0 = kChunk * c;
      const uint64_t b_g = ptx::make_smem_desc_sw128(ptx::smem_u32(sm.g[qrow0 >> 7]) + static_cast<uint32_t>(qrow0 & 127) * 128u, 1024, 1024);
      const uint64_t b_q = ptx::make_smem_desc_sw128(ptx::smem_u32(sm.q[qrow0 >> 7]) + static_cast<uint32_t>(qrow0 & 127) * 128u, 1024, 1024);
      const bool restart = c == tl.c0;
#pragma unroll 4
      for (int ks = ks0; ks < ks1; ++ks)
        ptx::mma_bf16_ts(tmem + kColDv, p_tmem + 8 * ks, ptx::desc_advance(b_g, ks * 2048), idesc_ts, !(restart && ks == ks0));
#pragma unroll 4
      for (int ks = ks0; ks < ks1; ++ks)
        ptx::mma_bf16_ts(tmem + kColDk, p_tmem + kChunk + 8 * ks, ptx::desc_advance(b_q, ks * 2048), idesc_ts, !(restart && ks == ks0));
      // dQ of a query block takes dS^T of both its chunk slots at once, when the last of them visited in this
      // tile is there (a slot that was not visited holds zeros)
      const int blk = c >> 1;
      if (c == min(tl.c1, 2 * blk + 1)) {
        const uint64_t a_ds = ptx::make_smem_desc_sw128(ptx::smem_u32(sm.ds[2 * blk]), kTileBytes, 1024);
        const uint32_t d = tmem + kColDq + static_cast<uint32_t>(blk * kHeadDim);
        const bool acc = blk ? dq_started[1] : dq_started[0];
#pragma unroll
        for (int kk = 0; kk < kTileN / 16; ++kk)
          ptx::mma_bf16_ss(d, ptx::desc_advance(a_ds, kk * 2048), ptx::desc_advance(b_k, kk * 2048), idesc_dq, acc || kk > 0);
        if (blk) dq_started[1] = true; else dq_started[0] = true;
      }
      ptx::mma_commit(&sm.grads_done[grp]);
      trace_event(sm, 400 + n);
    }
    ++t;
  }
}

// ------------------------------------------------------------------ dK / dV stores (one lane)
__device__ __forceinline__ void keys_store(KeysShared& sm, const CUtensorMap* map_dk, const CUtensorMap* map_dv, int n_kt,
                                           int head, int batch) {
  ptx::prefetch_tmap(map_dk);
  ptx::prefetch_tmap(map_dv);
  int t = 0;
  for (int kt = 0; kt < n_kt; ++kt) {
    KeysTile tl;
    if (!keys_tile(sm, kt, tl)) continue;
    const int s = t & 1;
    if (!wait_or_abort(sm, &sm.out_full, t & 1, 97)) return;
    ptx::mbar_arrive(&sm.out_seen);
    ptx::tma_store_4d(map_dv, sm.v[s], 0, kt * kTileN, head, batch);
    ptx::tma_store_4d(map_dk, sm.k[s], 0, kt * kTileN, head, batch);
    ptx::tma_store_commit();
    ptx::tma_store_wait_read();
    ptx::mbar_arrive(&sm.kv_empty[s]);
    ++t;
  }
}

// ------------------------------------------------------------------ compute groups
__device__ __forceinline__ void keys_compute(KeysShared& sm, const wm_attn_args& a, uint32_t tmem, int n_kt, int head,
                                             int batch) {
  const int tid = threadIdx.x;
  const int row = tid & 127;   // key row of the tile == TMEM lane
  const int grp = tid >> 7;    // this group takes the chunks of its parity
  const int warp = tid >> 5, lane = tid & 31;
  const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
  const float sl2 = a.scale * kLog2e;
  const bool docs = a.q_seg != nullptr;
  const int kvis = sm.kvis;
  const uint32_t sp = tmem + lane_base + static_cast<uint32_t>(grp * 128);
  const int swz = row & 7;
  const uint32_t row_off = static_cast<uint32_t>((row >> 3) * 1024 + (row & 7) * 128);

  // key tiles nobody sees get exact zeros (thread = key row; the first group writes dV, the second dK)
  for (int kt = 0; kt < n_kt; ++kt) {
    KeysTile tl;
    if (keys_tile(sm, kt, tl)) continue;
    const int j = kt * kTileN + row;
    if (j < a.k_len) {
      const int64_t* st = grp ? a.dk_strides : a.dv_strides;
      uint4* dst = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(grp ? a.dk : a.dv) + batch * st[0] + head * st[1] +
                                            static_cast<long long>(j) * st[2]);
#pragma unroll
      for (int c = 0; c < 8; ++c) dst[c] = make_uint4(0, 0, 0, 0);
    }
  }

  // document id / query bound of this thread's key in the next visited tile, fetched one tile ahead
  int pf_seg = INT_MIN, pf_end = 0, pf_kt = -1;
  auto fetch_table = [&](int kt) {
    pf_kt = kt;
    pf_seg = INT_MIN;
    pf_end = 0;
    if (docs) {
      const int j = kt * kTileN + row;
      if (j < a.k_len) {
        const long long at = static_cast<long long>(batch) * a.k_len + j;
        pf_seg = __ldg(a.k_seg + at);
        pf_end = __ldg(a.k_query_end + at);
      }
    }
  };
  auto next_visited = [&](int kt) -> int {
    for (int x = kt + 1; x < n_kt; ++x) {
      const uint32_t e = sm.tile_q[x];
      if ((e >> 16) > (e & 0xffffu)) return x;
    }
    return -1;
  };

  int t = 0, n = 0;
  for (int kt = 0; kt < n_kt; ++kt) {
    KeysTile tl;
    if (!keys_tile(sm, kt, tl)) continue;
    const int s = t & 1;
    const int j0 = kt * kTileN;
    const int j = j0 + row;
    // visibility of this key: queries [imin, iend), further cut by the document runs of a chunk
    int kseg = 0, iend = a.q_len;
    if (docs) {
      if (pf_kt != kt) fetch_table(kt);
      kseg = pf_seg;
      iend = min(pf_end, a.q_len);
      const int nx = next_visited(kt);
      if (nx >= 0) fetch_table(nx);
    }
    int imin = kMaxQueries;
    if (j < kvis) {
      // first query whose key bound lies beyond this key (the bounds do not decrease along the queries)
      int lo = 0, hi = kMaxQueries;
      while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (sm.q_hi[mid] > j) hi = mid; else lo = mid + 1;
      }
      imin = lo;
    }
    bool cleared = false;
    for (int c = tl.c0; c <= tl.c1; ++c, ++n) {
      if ((n & 1) != grp) continue;
      int n0, n1;
      keys_chunk_range(tl, c, n0, n1);
      const int i0 = kChunk * c;
      unsigned long long vis = below64(iend - i0) & ~below64(imin - i0);
      if (docs) {
        // The chunk's queries form runs of equal (document, first key); a key is open to a run when it is the shared
        // dummy or belongs to the run's document at or behind its first key.  The warp finds the run boundaries with
        // two ballots, every key builds its mask from the runs by arithmetic.
        const int x0 = i0 + lane, x1 = i0 + 32 + lane;
        const int s0 = sm.q_seg[x0], l0 = sm.q_lo[x0], s1 = sm.q_seg[x1], l1 = sm.q_lo[x1];
        const bool b0 = lane == 0 || sm.q_seg[x0 - 1] != s0 || sm.q_lo[x0 - 1] != l0;
        const bool b1 = sm.q_seg[x1 - 1] != s1 || sm.q_lo[x1 - 1] != l1;
        unsigned long long rest = static_cast<unsigned long long>(__ballot_sync(0xffffffffu, b0)) |
                                  (static_cast<unsigned long long>(__ballot_sync(0xffffffffu, b1)) << 32);
        rest &= ~1ull;  // column 0 begins the first run
        unsigned long long open = 0ull;
        int start = 0;
        while (true) {
          const int next = rest ? __ffsll(static_cast<long long>(rest)) - 1 : kChunk;
          rest &= rest - 1ull;
          const int rseg = sm.q_seg[i0 + start], rlo = sm.q_lo[i0 + start];  // the same address for every lane
          if ((kseg == -1) | ((kseg == rseg) & (j >= rlo))) open |= below64(next) & ~below64(start);
          if (next >= kChunk) break;
          start = next;
        }
        vis &= open;
      }
      if (!wait_or_abort(sm, &sm.sp_full[grp], (n >> 1) & 1, 92)) return;
      ptx::tc_fence_after();
      if (lane == 0) trace_event(sm, 500 + n);
      // rows of K behind the last visible key may hold anything (unused cache capacity): as the B operand of
      // dQ += dS K they would turn zeros into NaN.  Their scores are never looked at, so clearing them under the
      // running products is harmless.
      if (!cleared && j >= kvis) {
        uint4* dst = reinterpret_cast<uint4*>(sm.k[s] + row * 128);
#pragma unroll
        for (int x = 0; x < 8; ++x) dst[x] = make_uint4(0, 0, 0, 0);
      }
      cleared = true;
      uint32_t dsr[32];  // packed dS^T of the chunk (two queries per word), kept for the shared-memory copy
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        const uint32_t m16 = static_cast<uint32_t>(vis >> (16 * p)) & 0xffffu;
        const bool covered = 16 * p >= n0 && 16 * p < n1;  // the products of this chunk read the piece
        const bool none = !covered || __all_sync(0xffffffffu, m16 == 0u);
        if (none) {
#pragma unroll
          for (int e = 0; e < 8; ++e) dsr[8 * p + e] = 0u;
          if (covered) {
            const uint32_t zeros[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
            ptx::tmem_st8(sp + 8 * p, zeros);
            ptx::tmem_st8(sp + kChunk + 8 * p, zeros);
          }
          continue;
        }
        const bool full = __all_sync(0xffffffffu, m16 == 0xffffu);
        uint32_t xs[16], ys[16];
        ptx::tmem_ld16(sp + 16 * p, xs);
        ptx::tmem_ld16(sp + kChunk + 16 * p, ys);
        const float4* nlp = reinterpret_cast<const float4*>(sm.nl2 + i0 + 16 * p);
        const float4* ndp = reinterpret_cast<const float4*>(sm.nd + i0 + 16 * p);
        float4 nl[4], nd[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          nl[u] = nlp[u];
          nd[u] = ndp[u];
        }
        ptx::tmem_wait_ld();
        const float2 sc2 = make_float2(sl2, sl2);
        uint32_t pp[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          // P = exp2(S * scale * log2e - lse * log2e), dS = P * (dP - delta), two queries per instruction
          float2 x = make_float2(__uint_as_float(xs[2 * e]), __uint_as_float(xs[2 * e + 1]));
          float2 y = make_float2(__uint_as_float(ys[2 * e]), __uint_as_float(ys[2 * e + 1]));
          if (!full) {
            const bool v0 = (m16 >> (2 * e)) & 1u, v1 = (m16 >> (2 * e + 1)) & 1u;
            x.x = v0 ? x.x : -INFINITY;
            x.y = v1 ? x.y : -INFINITY;
            y.x = v0 ? y.x : 0.f;
            y.y = v1 ? y.y : 0.f;
          }
          const float4 nlq = nl[e >> 1], ndq = nd[e >> 1];
          const float2 nl2v = (e & 1) ? make_float2(nlq.z, nlq.w) : make_float2(nlq.x, nlq.y);
          const float2 nd2v = (e & 1) ? make_float2(ndq.z, ndq.w) : make_float2(ndq.x, ndq.y);
          float2 pr = __ffma2_rn(x, sc2, nl2v);
          pr.x = fast_exp2(pr.x);
          pr.y = fast_exp2(pr.y);
          const float2 dsv = __fmul2_rn(pr, __fadd2_rn(y, nd2v));
          pp[e] = pack_bf16(pr.x, pr.y);
          dsr[8 * p + e] = pack_bf16(dsv.x, dsv.y);
        }
        uint32_t dd[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) dd[e] = dsr[8 * p + e];
        // packed over the columns the piece was read from (P^T: [8p, 8p+8) of the S^T half, dS^T the same of dP^T)
        ptx::tmem_st8(sp + 8 * p, pp);
        ptx::tmem_st8(sp + kChunk + 8 * p, dd);
      }
      if (lane == 0) trace_event(sm, 600 + n);
      // dS^T of this slot (and of the block's other slot, when this tile does not visit it) is read by the dQ
      // products of the previous tile until they complete.  Everything up to the chunk before the previous one
      // is complete once this chunk's scores are there; the previous chunk matters for a tile's first chunk only.
      if (c == tl.c0 && n > 0 && !wait_or_abort(sm, &sm.grads_done[grp ^ 1], ((n - 1) >> 1) & 1, 93)) return;
      {
        unsigned char* slot = sm.ds[c] + row_off;
#pragma unroll
        for (int u = 0; u < 8; ++u)
          *reinterpret_cast<uint4*>(slot + ((u ^ swz) << 4)) = make_uint4(dsr[4 * u], dsr[4 * u + 1], dsr[4 * u + 2], dsr[4 * u + 3]);
        const int sibling = c ^ 1;
        if (sibling < tl.c0 || sibling > tl.c1) {
          unsigned char* other = sm.ds[sibling] + row_off;
#pragma unroll
          for (int u = 0; u < 8; ++u) *reinterpret_cast<uint4*>(other + (u << 4)) = make_uint4(0, 0, 0, 0);
        }
      }
      ptx::tmem_wait_st();
      ptx::fence_async_shared();
      ptx::tc_fence_before();
      ptx::mbar_arrive(&sm.pds_full[grp]);
      if (lane == 0) trace_event(sm, 700 + n);
      if (c == tl.c1) {
        // This was the tile's last chunk: when its gradient products are complete, dV and dK leave TMEM (the next
        // tile's products restart the accumulators) and are staged, bf16 and swizzled like the output tensor map
        // wants them, in the tile's own K / V stage, which nothing reads any more.
        if (!wait_or_abort(sm, &sm.grads_done[grp], (n >> 1) & 1, 94)) return;
        ptx::tc_fence_after();
        uint32_t pv[32], pk[32];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t raw[32];
          ptx::tmem_ld32(tmem + lane_base + kColDv + 32 * h, raw);
          ptx::tmem_wait_ld();
#pragma unroll
          for (int e = 0; e < 16; ++e) pv[16 * h + e] = pack_bf16(__uint_as_float(raw[2 * e]), __uint_as_float(raw[2 * e + 1]));
          ptx::tmem_ld32(tmem + lane_base + kColDk + 32 * h, raw);
          ptx::tmem_wait_ld();
#pragma unroll
          for (int e = 0; e < 16; ++e)
            pk[16 * h + e] = pack_bf16(__uint_as_float(raw[2 * e]) * a.scale, __uint_as_float(raw[2 * e + 1]) * a.scale);
        }
        ptx::tc_fence_before();
        ptx::mbar_arrive(&sm.dkv_free);
        // the storing lane has to have seen the previous staged tile before this one may be announced
        if (t > 0 && !wait_or_abort(sm, &sm.out_seen, (t - 1) & 1, 96)) return;
        unsigned char* vrow = sm.v[s] + row_off;
        unsigned char* krow = sm.k[s] + row_off;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          *reinterpret_cast<uint4*>(vrow + ((u ^ swz) << 4)) = make_uint4(pv[4 * u], pv[4 * u + 1], pv[4 * u + 2], pv[4 * u + 3]);
          *reinterpret_cast<uint4*>(krow + ((u ^ swz) << 4)) = make_uint4(pk[4 * u], pk[4 * u + 1], pk[4 * u + 2], pk[4 * u + 3]);
        }
        ptx::fence_async_shared();
        ptx::mbar_arrive(&sm.out_full);
        if (lane == 0) trace_event(sm, 800 + n);
      }
    }
    ++t;
  }
  // dQ: group b writes the rows of query block b once every product is complete
  if (n > 0) {
    if (!wait_or_abort(sm, &sm.grads_done[(n - 1) & 1], ((n - 1) >> 1) & 1, 95)) return;
    ptx::tc_fence_after();
  }
  {
    const int blk = grp;
    const int i = blk * kTileM + row;
    bool issued = false;  // did any visited tile reach this query block?
    for (int kt = 0; kt < n_kt; ++kt) {
      KeysTile tl;
      if (keys_tile(sm, kt, tl) && tl.c0 <= 2 * blk + 1 && tl.c1 >= 2 * blk) issued = true;
    }
    uint32_t packed[kHeadDim / 2];
    uint32_t raw[2][32];
    if (issued) {
      ptx::tmem_ld32(tmem + lane_base + kColDq + blk * kHeadDim, raw[0]);
      ptx::tmem_ld32(tmem + lane_base + kColDq + blk * kHeadDim + 32, raw[1]);
      ptx::tmem_wait_ld();
    }
#pragma unroll
    for (int c = 0; c < 2; ++c) {
#pragma unroll
      for (int e2 = 0; e2 < 16; ++e2)
        packed[c * 16 + e2] =
            issued ? pack_bf16(__uint_as_float(raw[c][2 * e2]) * a.scale, __uint_as_float(raw[c][2 * e2 + 1]) * a.scale) : 0u;
    }
    if (i < a.q_len) {
      uint4* dst = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(a.dq) + batch * a.dq_strides[0] + head * a.dq_strides[1] +
                                            static_cast<long long>(i) * a.dq_strides[2]);
      if ((reinterpret_cast<uintptr_t>(dst) & 31) == 0) {  // whole 32-byte sectors
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const uint32_t pk8[8] = {packed[8 * c],     packed[8 * c + 1], packed[8 * c + 2], packed[8 * c + 3],
                                   packed[8 * c + 4], packed[8 * c + 5], packed[8 * c + 6], packed[8 * c + 7]};
          ptx::st_global_v8(dst + 2 * c, pk8);
        }
      } else {
#pragma unroll
        for (int c = 0; c < 8; ++c) dst[c] = make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
      }
    }
  }
}

__global__ void __launch_bounds__(kKeysThreads, 1)
    attn_bwd_keys_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                         const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_g,
                         const __grid_constant__ CUtensorMap map_dk, const __grid_constant__ CUtensorMap map_dv,
                         const wm_attn_args a, const float* delta, const int epoch) {
  extern __shared__ unsigned char smem_raw[];
  KeysShared& sm = *reinterpret_cast<KeysShared*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int head = blockIdx.x;
  const int batch = blockIdx.y;
  const GroupCtx g = group_ctx(a, 0);
  const int nq = (a.q_len + kTileM - 1) / kTileM;
  const int n_kt = (a.k_len + kTileN - 1) / kTileN;
  const bool docs = a.q_seg != nullptr;

  if (tid == 0) {
    sm.abort_flag = 0;
    sm.epoch = epoch;
    sm.kvis = 0;
    trace_begin(sm, epoch);
    trace_event(sm, 1);
    ptx::mbar_init(&sm.qg_full, 1);
    for (int s = 0; s < 2; ++s) {
      ptx::mbar_init(&sm.kv_full[s], 1);
      ptx::mbar_init(&sm.kv_empty[s], 1);
      ptx::mbar_init(&sm.sp_full[s], 1);
      ptx::mbar_init(&sm.pds_full[s], kKeysGroup);
      ptx::mbar_init(&sm.grads_done[s], 1);
    }
    ptx::mbar_init(&sm.dkv_free, kKeysGroup);
    ptx::mbar_init(&sm.out_full, kKeysGroup);
    ptx::mbar_init(&sm.out_seen, 1);
    ptx::mbar_fence_init();
  }
  if (warp == 8) {
    ptx::tmem_alloc(&sm.tmem_base, kTmemCols);
    ptx::tmem_relinquish();
  }
  // per-query tables: thread i < 256 owns query i
  RowBound own;
  own.lo = own.hi = own.seg = own.qi = 0;
  float lse = INFINITY, dl = 0.f;
  if (tid < kKeysCompute && tid < a.q_len) {
    own = row_bound(a, g, batch, tid);
    const long long stat = (static_cast<long long>(batch) * a.q_heads + head) * a.q_len + tid;
    lse = a.lse[stat];
    dl = delta[stat];
  }
  __syncthreads();
  if (tid == kKeysCompute) {
    // Q and dO depend on nothing the block works out first
    ptx::prefetch_tmap(&map_q);
    ptx::prefetch_tmap(&map_g);
    ptx::mbar_expect_tx(&sm.qg_full, 2 * nq * kTileBytes);
    for (int b = 0; b < nq; ++b) {
      ptx::tma_load_4d(sm.q[b], &map_q, &sm.qg_full, 0, b * kTileM, head, batch);
      ptx::tma_load_4d(sm.g[b], &map_g, &sm.qg_full, 0, b * kTileM, head, batch);
    }
  }
  if (tid == kKeysThreads - 1) sm.has_dummy = docs && a.k_seg[static_cast<long long>(batch) * a.k_len] == -1;
  if (tid < kKeysCompute) {
    const bool live = tid < a.q_len;
    sm.nl2[tid] = live ? -lse * kLog2e : -INFINITY;
    sm.nd[tid] = live ? -dl : 0.f;
    sm.q_seg[tid] = live ? own.seg : INT_MIN + 1;
    sm.q_lo[tid] = live ? own.lo : INT_MAX;
    sm.q_hi[tid] = live ? own.hi : INT_MAX;
    const int hi = __reduce_max_sync(0xffffffffu, live ? own.hi : 0);
    if (lane == 0) atomicMax(&sm.kvis, hi);
  }
  __syncthreads();
  if (warp < 8) {
    // Queries that may see key tile kt: their key bound reaches beyond the tile's first key and (with documents)
    // their document does not begin behind the tile -- the range from the first such query to the last.
    const bool dummy = sm.has_dummy != 0;
    for (int kt = warp; kt < n_kt; kt += 8) {
      const int j0 = kt * kTileN;
      int first = INT_MAX, last = -1;
      for (int base = 0; base < kMaxQueries; base += 32) {
        const int i = base + lane;
        const int hi = sm.q_hi[i], lo = sm.q_lo[i];
        const bool rel = i < a.q_len && hi > j0 && (!docs || lo < j0 + kTileN || (dummy && kt == 0));
        const uint32_t m = __ballot_sync(0xffffffffu, rel);
        if (m) {
          first = min(first, base + __ffs(m) - 1);
          last = max(last, base + 31 - __clz(m));
        }
      }
      if (lane == 0) sm.tile_q[kt] = last < 0 ? 0u : (static_cast<uint32_t>(first) | (static_cast<uint32_t>(last + 1) << 16));
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = sm.tmem_base;
  if (tid == 0) trace_event(sm, 2);
  if (warp < 8) {
    keys_compute(sm, a, tmem, n_kt, head, batch);
  } else if (lane == 0) {
    if (warp == 8) keys_producer(sm, &map_k, &map_v, n_kt, head, batch);
    if (warp == 9) keys_mma_scores(sm, tmem, n_kt);
    if (warp == 10) keys_mma_grads(sm, tmem, n_kt);
    if (warp == 11) keys_store(sm, &map_dk, &map_dv, n_kt, head, batch);
  }
  if (tid == 0) trace_event(sm, 3);
  ptx::tma_store_wait_all();
  ptx::tc_fence_before();
  __syncthreads();
  trace_flush(sm);
  if (warp == 8) ptx::tmem_dealloc(tmem, kTmemCols);
}
