// Forward pipeline of the tcgen05 attention kernel (included by attn_tc.cu), a template over the head size.
//
// One block owns 128 query rows of one (batch, head) and walks over tiles of 128 key slots.
// 352 threads: warps 0-7 softmax, warp 8 TMA producer (Q once, K and V through rings, per-block loads, no
// multicast), warps 9 and 10 issue tcgen05.mma (one lane each): S = Q K^T into one of the score buffers in TMEM,
// O += P V into the accumulator of the tile's parity; completion is signalled by tcgen05.commit on mbarriers.
// The softmax warps form two groups of 128 threads (thread = query row = TMEM lane).  Group g
// owns the key tiles of parity g with its own running reference, row sum, P buffer and output
// accumulator, so the groups exchange nothing per tile and run out of phase; their partial
// results are merged in the epilogue like the splits of a split-KV reduction.
// P never touches shared memory: it is written as packed bf16 over the first 64 columns of its own
// score buffer and the PV product takes it from there as its A operand.
// TMEM (512 columns), head size 64: S0..S2 [0,384) (P aliases the tile's S), O0 [384,448), O1 [448,512);
// head size 128: S0, S1 [0,256), O0 [256,384), O1 [384,512).
#pragma once

constexpr int kFwdThreads = 352;
constexpr int kFwdSoftmax = 256;
constexpr int kFwdGroup = 128;      // threads of one softmax group
constexpr uint32_t kSubBytes = kTileN * 64 * 2;  // a tile travels as 64-column sub-tiles of 16 KB (one 128-byte swizzle row per token)

// What depends on the head size D (64 or 128).  The K/V ring and the score buffers share their depth: three for
// D = 64; two for D = 128, where a tile is twice as large and the two output accumulators take 256 of the 512 TMEM
// columns (S0, S1 [0,256), O0 [256,384), O1 [384,512)).
template <int D>
struct FwdCfg {
  static constexpr int kRing = D == 64 ? 3 : 2;
  static constexpr int kSub = D / 64;
  static constexpr uint32_t kBytes = kTileN * D * 2;
  static constexpr uint32_t kOut = kRing * kTileN;
};
#define WM_FWD_CONSTANTS(D)                                   \
  constexpr int kStages = FwdCfg<D>::kRing;                   \
  constexpr int kScoreBuffers = FwdCfg<D>::kRing;             \
  constexpr uint32_t kTileBytes = FwdCfg<D>::kBytes;          \
  constexpr uint32_t kOutCol = FwdCfg<D>::kOut;               \
  constexpr int kSub = FwdCfg<D>::kSub;                       \
  (void)kStages, (void)kScoreBuffers, (void)kTileBytes, (void)kOutCol, (void)kSub

// ------------------------------------------------------------------ producer (one lane of the producer warp)
template <int D, class Shared>
__device__ __forceinline__ void producer_role(Shared& sm, const CUtensorMap* map_q, const CUtensorMap* map_k,
                                              const CUtensorMap* map_v, const TileWalk& w, int q0, int head,
                                              int kv_head, int batch) {
  WM_FWD_CONSTANTS(D);
  // K tiles are released by the score product, two tiles ahead of the PV product that releases V tiles: the K
  // loads run ahead of the V loads by the same distance so that a late V release never delays a score product
  auto load_k = [&](int n) -> bool {
    const int s = n % kStages;
    if (!wait_or_abort(sm, &sm.s_full[s], ((n / kStages) & 1) ^ 1, 11)) return false;  // score product n-3 has read the stage
    ptx::mbar_expect_tx(&sm.k_full[s], kTileBytes);
#pragma unroll
    for (int h = 0; h < kSub; ++h)
      ptx::tma_load_4d(sm.k[s] + h * kSubBytes, map_k, &sm.k_full[s], 64 * h, tile_first_key(n, w.first_tile, w.dummy_tile), kv_head, batch);
    trace_event(sm, 100 + n);
    return true;
  };
  constexpr int kAhead = kStages - 1;
  for (int n = 0; n < kAhead && n < w.n_tiles; ++n)
    if (!load_k(n)) return;
  for (int n = 0; n < w.n_tiles; ++n) {
    if (n + kAhead < w.n_tiles && !load_k(n + kAhead)) return;
    const int s = n % kStages;
    if (!wait_or_abort(sm, &sm.pv_done[s], ((n / kStages) & 1) ^ 1, 12)) return;  // PV product n-3 has read the stage
    ptx::mbar_expect_tx(&sm.v_full[s], kTileBytes);
#pragma unroll
    for (int h = 0; h < kSub; ++h)
      ptx::tma_load_4d(sm.v[s] + h * kSubBytes, map_v, &sm.v_full[s], 64 * h, tile_first_key(n, w.first_tile, w.dummy_tile), kv_head, batch);
    trace_event(sm, 200 + n);
  }
}

// ------------------------------------------------------------------ MMA issuers (one lane of a warp each)
// The tensor pipe accepts the next instruction only when it has started the previous one, so a thread that issues
// is busy for as long as its products run.  Two threads issue: one the score products, as far ahead as the three
// score buffers allow, one the PV products; either does its waiting while the other feeds the pipe.
template <int D, class Shared>
__device__ __forceinline__ void score_mma_role(Shared& sm, uint32_t tmem, const TileWalk& w) {
  WM_FWD_CONSTANTS(D);
  if (!wait_or_abort(sm, &sm.q_full, 0, 20)) return;
  constexpr uint32_t idesc = ptx::make_idesc_bf16(kTileM, kTileN, 0, 0);
  const uint32_t a_base = ptx::smem_u32(sm.q);
  for (int n = 0; n < w.n_tiles; ++n) {
    const int s = n % kStages;
    // P of tile n-3 lives in this score buffer until its PV product has read it
    if (n >= kScoreBuffers && !wait_or_abort(sm, &sm.pv_done[s], ((n / kScoreBuffers) & 1) ^ 1, 24)) return;
    if (!wait_or_abort(sm, &sm.k_full[s], (n / kStages) & 1, 21)) return;
    ptx::tc_fence_after();
    trace_event(sm, 1100 + n);
    const uint32_t b_base = ptx::smem_u32(sm.k[s]);
    const uint32_t d = tmem + static_cast<uint32_t>(s) * kTileN;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      // 16 elements of head_dim per instruction: 32 bytes inside the 128-byte swizzle row of the element's sub-tile
      const uint32_t at = (kk >> 2) * kSubBytes + (kk & 3) * 32;
      ptx::mma_bf16_ss(d, ptx::make_smem_desc_sw128(a_base + at, 16, 1024), ptx::make_smem_desc_sw128(b_base + at, 16, 1024), idesc,
                       kk > 0);
    }
    ptx::mma_commit(&sm.s_full[s]);
    trace_event(sm, 400 + n);
  }
}

template <int D, class Shared>
__device__ __forceinline__ void value_mma_role(Shared& sm, uint32_t tmem, const TileWalk& w) {
  WM_FWD_CONSTANTS(D);
  // all D output columns in one instruction: the MN-major V operand steps from one 64-column sub-tile to the next by
  // its leading-dimension offset
  constexpr uint32_t idesc_pv = ptx::make_idesc_bf16(kTileM, D, 0, 1);
  constexpr uint32_t kHalfStep = D > 64 ? kSubBytes : 1024;
  for (int n = 0; n < w.n_tiles; ++n) {
    const int b = n & 1;
    const int s = n % kStages;
    if (!wait_or_abort(sm, &sm.p_full[b], (n >> 1) & 1, 22)) return;
    ptx::mbar_arrive(&sm.p_seen[b]);  // this phase of p_full has been consumed: the group may complete the next one
    trace_event(sm, 300 + n);
    if (!wait_or_abort(sm, &sm.v_full[s], (n / kStages) & 1, 23)) return;
    ptx::tc_fence_after();
    trace_event(sm, 1200 + n);
    const uint32_t o_tmem = tmem + kOutCol + static_cast<uint32_t>(b) * D;
    const uint32_t p_tmem = tmem + static_cast<uint32_t>(s) * kTileN;  // P overwrote the first 64 columns of S
    const uint32_t v_base = ptx::smem_u32(sm.v[s]);
#pragma unroll
    for (int kk = 0; kk < kTileN / 16; ++kk) {
      // A = P from tensor memory, 16 keys = 8 columns; B = V: head_dim contiguous (MN-major), 16 keys = 2048 bytes
      const uint64_t b_desc = ptx::make_smem_desc_sw128(v_base + kk * 2048, kHalfStep, 1024);
      ptx::mma_bf16_ts(o_tmem, p_tmem + kk * 8, b_desc, idesc_pv, (n > 1) || (kk > 0));
    }
    ptx::mma_commit(&sm.pv_done[s]);
    trace_event(sm, 500 + n);
  }
}


template <int D>
struct FwdShared {
  unsigned char q[FwdCfg<D>::kBytes];
  unsigned char k[FwdCfg<D>::kRing][FwdCfg<D>::kBytes];
  unsigned char v[FwdCfg<D>::kRing][FwdCfg<D>::kBytes];
  uint64_t q_full;
  // s_full[i] and pv_done[i] also release K and V stage i (score buffers and stages share the ring size)
  uint64_t k_full[FwdCfg<D>::kRing], v_full[FwdCfg<D>::kRing];
  uint64_t s_full[FwdCfg<D>::kRing], pv_done[FwdCfg<D>::kRing], p_full[2], p_seen[2], sum_full;
  // document id and exclusive query bound of the key slots of a tile: every softmax warp keeps its own copy
  // ([warp][tile of its group & 1]), brought in one tile ahead by asynchronous copies, so that the warps of a group
  // never have to meet for it
  int key_seg[8][2][kTileN];
  int key_end[8][2][kTileN];
  float row_max[2][kTileM];
  float row_sum[2][kTileM];
  int warp_min_lo[4], warp_max_hi[4], has_dummy;
  uint32_t tmem_base;
  int abort_flag;
  int epoch;
  WM_TRACE_FIELDS
};

// One softmax group (128 threads, thread = query row = TMEM lane) owns the key tiles of one parity: it keeps its
// own running reference, row sum and output accumulator, so the two groups never exchange anything per tile and
// drift out of phase, one in its exponentials while the other reads scores.  The two partial results are merged
// once, in the epilogue.  A tile is read from TMEM once, in pieces of 32 columns: a row exponentiates against the
// reference it has (zero while it has none) and judges the reference afterwards by the row sum (no maximum is formed
// per element); the row sum is taken over the weights as rounded to bf16, so the output is an exact weighted mean
// whatever the reference was.
template <int D>
__device__ __forceinline__ void softmax_role(FwdShared<D>& sm, const wm_attn_args& a, uint32_t tmem, const TileWalk& w,
                                             const RowBound& rb, bool live, int batch, int head) {
  WM_FWD_CONSTANTS(D);
  const int t = threadIdx.x;
  const int row = t & 127;
  const int grp = t >> 7;
  const int warp = t >> 5, lane = t & 31;
  const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
  const float sl2 = a.scale * kLog2e;
  const bool docs = a.q_seg != nullptr;
  float m_ref = -INFINITY, l = 0.f;
  float pending = 1.f;  // factor the accumulator still has to be multiplied by
  constexpr float kSumGuard = 1.0995116e12f;  // 2^40: a row sum beyond it sends the tile back for its true maximum
  constexpr float kSumMove = 4096.f;          // 2^12: a row sum beyond it moves the reference for the tiles to come
  constexpr float kSumTiny = 7.8886091e-31f;  // 2^-100: a row on its provisional zero whose first sum is smaller asks for its true maximum
  const uint32_t o_mine = tmem + kOutCol + grp * D + lane_base;
  const int b = grp;  // P buffer, output accumulator and document tables of this group

  // document id / query bound of the key slots of tile n into this warp's table `buf`, four slots per lane
  // (32 c + lane); slots beyond the tensor read as zeros (document 0, no query may see them)
  auto fetch_key_docs = [&](int n, int buf) {
    if (docs && n < w.n_tiles) {
      const int j = tile_first_key(n, w.first_tile, w.dummy_tile);
      const long long base = static_cast<long long>(batch) * a.k_len;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int slot = j + 32 * c + lane;
        const bool in = slot < a.k_len;
        const long long at = base + (in ? slot : 0);
        ptx::cp_async_4(&sm.key_seg[warp][buf][32 * c + lane], a.k_seg + at, in);
        ptx::cp_async_4(&sm.key_end[warp][buf][32 * c + lane], a.k_query_end + at, in);
      }
    }
    ptx::cp_async_commit();
  };
  fetch_key_docs(grp, 0);
  const int tbase = lane == 0 ? grp * 10000 + (warp & 3) * 2000 : -1;  // lane 0 of every softmax warp leaves a trace
#define WM_TRACE(tag) if (tbase >= 0) trace_event(sm, tbase + (tag))

  for (int n = grp; n < w.n_tiles; n += 2) {
    const int it = n >> 1;  // tiles this group has finished
    const int sb = n % kScoreBuffers;
    const int j0 = tile_first_key(n, w.first_tile, w.dummy_tile);
    int cls = !live || j0 >= rb.hi ? kTileNone : (j0 + kTileN <= rb.hi ? kTileFull : kTileCausal);
    if (docs) {
      fetch_key_docs(n + 2, (it + 1) & 1);
      ptx::cp_async_wait_all_but_last();  // this tile's table has landed; the next one may still be on its way
      __syncwarp();
      {
        // the tile's summary, formed by the whole warp (every lane takes part whatever its row's class)
        const int* tseg = sm.key_seg[warp][it & 1];
        const int* tend_of = sm.key_end[warp][it & 1];
        const int tmin = __reduce_min_sync(0xffffffffu, min(min(tseg[lane], tseg[32 + lane]), min(tseg[64 + lane], tseg[96 + lane])));
        const int tmax = __reduce_max_sync(0xffffffffu, max(max(tseg[lane], tseg[32 + lane]), max(tseg[64 + lane], tseg[96 + lane])));
        const int tend = __reduce_min_sync(0xffffffffu, min(min(tend_of[lane], tend_of[32 + lane]), min(tend_of[64 + lane], tend_of[96 + lane])));
        if (cls != kTileNone) {
          const bool uniform = tmin == tmax;
          const bool own_doc = uniform && tmin == rb.seg && j0 >= rb.lo && tend > rb.qi;
          if (uniform && tmin != -1 && tmin != rb.seg) {
            cls = kTileNone;
          } else if (!own_doc) {
            cls = kTileDocs;
          }
        }
      }
    }
    // the caller's key mask of this tile as four words (bit c of word w: slot j0 + 32w + c may be seen)
    uint32_t km0 = 0xffffffffu, km1 = 0xffffffffu, km2 = 0xffffffffu, km3 = 0xffffffffu;
    if (a.key_mask != nullptr) {
      const unsigned char* mrow = a.key_mask + static_cast<long long>(batch) * a.k_len;
      auto kept = [&](int col) -> bool {
        const int j = j0 + col + lane;
        return j < a.k_len && mrow[j] != 0;
      };
      km0 = __ballot_sync(0xffffffffu, kept(0));
      km1 = __ballot_sync(0xffffffffu, kept(32));
      km2 = __ballot_sync(0xffffffffu, kept(64));
      km3 = __ballot_sync(0xffffffffu, kept(96));
    }
    const bool km_all = (km0 & km1 & km2 & km3) == 0xffffffffu;
    // whole-warp shortcuts: nothing to mask, or nothing to see
    const bool warp_full = km_all && __all_sync(0xffffffffu, cls == kTileFull);
    const bool warp_none = __all_sync(0xffffffffu, cls == kTileNone);
    const int lim = rb.hi - j0;
    const int lim_eff = cls == kTileFull ? kTileN : (cls == kTileNone ? 0 : lim);
    // visibility of 32 columns as a bit mask: arithmetic for the causal bound, and the key tile's document table
    // (looked at by the whole warp together) for rows whose tile contains a document boundary
    auto visibility = [&](uint32_t& v0, uint32_t& v1, uint32_t& v2, uint32_t& v3) {
      v0 = v1 = v2 = v3 = 0xffffffffu;
      if (!warp_full && !warp_none) {
        uint32_t dm[4] = {0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu};
        if (__any_sync(0xffffffffu, cls == kTileDocs))
          warp_doc_masks(rb, cls == kTileDocs, j0, sm.key_seg[warp][it & 1], sm.key_end[warp][it & 1], dm);
        auto causal_mask = [&](int col0) -> uint32_t {
          const int left = lim_eff - col0;
          return left >= 32 ? 0xffffffffu : (left <= 0 ? 0u : ((1u << left) - 1u));
        };
        v0 = causal_mask(0) & dm[0] & km0;
        v1 = causal_mask(32) & dm[1] & km1;
        v2 = causal_mask(64) & dm[2] & km2;
        v3 = causal_mask(96) & dm[3] & km3;
      }
    };
    uint32_t vis0, vis1, vis2, vis3;
    visibility(vis0, vis1, vis2, vis3);
    // does the row see any column of this tile?
    const bool seen = cls != kTileNone && (warp_full || (vis0 | vis1 | vis2 | vis3) != 0u);
    const uint32_t s_tmem = tmem + static_cast<uint32_t>(sb) * kTileN + lane_base;
    if (!wait_or_abort(sm, &sm.s_full[sb], (n / kScoreBuffers) & 1, 31)) return;
    ptx::tc_fence_after();
    WM_TRACE(600 + n);
    // multiply this group's accumulator by `factor` (1 for rows that did not move); the accumulator was last
    // written by the PV product of the group's previous tile
    auto rescale_output = [&](float factor) -> bool {
      if (n >= 2 && !wait_or_abort(sm, &sm.pv_done[(n - 2) % kStages], ((n - 2) / kStages) & 1, 32)) return false;
      ptx::tc_fence_after();
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t raw[32];
        ptx::tmem_ld32(o_mine + 32 * c, raw);
        ptx::tmem_wait_ld();
#pragma unroll
        for (int e = 0; e < 32; ++e) raw[e] = __float_as_uint(__uint_as_float(raw[e]) * factor);
        ptx::tmem_st32(o_mine + 32 * c, raw);
      }
      ptx::tmem_wait_st();
      return true;
    };
    // a reference that moved while the previous tile of this group was exponentiated: the row sum was corrected
    // then, the accumulator (which had to take that tile's product first) is corrected now
    if (__any_sync(0xffffffffu, pending != 1.f)) {
      if (!rescale_output(pending)) return;
      pending = 1.f;
    }
    // Rows exponentiate against the reference they already have -- zero for a row that has none yet -- and look at
    // the maximum afterwards (one reading of the scores).  A warp with a row whose scores turn out to exceed the
    // reference by more than 2^kGuard (or, for a row on its provisional zero, to lie more than 2^kGuard below it)
    // moves that row's reference to the tile's maximum and exponentiates once more: the scores are still there.
    bool fresh = m_ref == -INFINITY;
    float tile_sum = 0.f;
    // P as packed bf16 over the first 64 columns of the score buffer, all of which have been read by then
    if (warp_none) {
      uint32_t zeros[32];
#pragma unroll
      for (int e = 0; e < 32; ++e) zeros[e] = 0u;
      ptx::tmem_st32(s_tmem, zeros);
      ptx::tmem_st32(s_tmem + 32, zeros);
    } else {
      uint32_t pk0[16], pk1[16], pk2[16], pk3[16];
      // all 128 columns against the current reference: packed P and the row sum
      auto exponentiate = [&]() {
        const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
        const float2 sc = make_float2(sl2, sl2), nm = make_float2(-m_use, -m_use);
        float2 s0 = make_float2(0.f, 0.f), s1 = make_float2(0.f, 0.f);
        // 32 columns at a time keep the live registers (scores + packed P of the whole tile) under the limit;
        // the load of the next piece is in flight while this one is exponentiated
        auto piece = [&](uint32_t (&raw)[32], uint32_t mask, uint32_t (&pk)[16]) {
          float x[32];
          if (warp_full) {
#pragma unroll
            for (int e = 0; e < 32; ++e) x[e] = __uint_as_float(raw[e]);
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) x[e] = (mask >> e) & 1u ? __uint_as_float(raw[e]) : -INFINITY;
          }
          // one kind of instruction at a time: 32 independent exponentials in a row keep the special-function
          // unit busy from a single warp
          float2 t[16];
#pragma unroll
          for (int u = 0; u < 16; ++u) t[u] = __ffma2_rn(make_float2(x[2 * u], x[2 * u + 1]), sc, nm);
#pragma unroll
          for (int u = 0; u < 16; ++u) {
            t[u].x = fast_exp2(t[u].x);
            t[u].y = fast_exp2(t[u].y);
          }
          // the row sum is taken over the weights as the PV product will see them (rounded to bf16): the output is
          // then an exact weighted mean of the value rows, whatever reference the weights were formed against.  The
          // halves of a packed pair are added to fp32 sums as they are (mixed-precision add), without unpacking.
#pragma unroll
          for (int u = 0; u < 16; ++u) {
            pk[u] = pack_bf16(t[u].x, t[u].y);
            if (u & 1) ptx::add_bf16_halves(pk[u], s1.x, s1.y);
            else ptx::add_bf16_halves(pk[u], s0.x, s0.y);
          }
        };
        uint32_t even[32], odd[32];
        ptx::tmem_ld32(s_tmem, even);
        ptx::tmem_wait_ld();
        ptx::tmem_ld32(s_tmem + 32, odd);
        piece(even, vis0, pk0);
        ptx::tmem_wait_ld();
        ptx::tmem_ld32(s_tmem + 64, even);
        piece(odd, vis1, pk1);
        ptx::tmem_wait_ld();
        ptx::tmem_ld32(s_tmem + 96, odd);
        piece(even, vis2, pk2);
        ptx::tmem_wait_ld();
        piece(odd, vis3, pk3);
        tile_sum = (s0.x + s0.y) + (s1.x + s1.y);
      };
      exponentiate();
      // The row sum tells whether the reference served: a sum beyond 2^kGuard (or not finite: the exponentials
      // overflowed), or a row on its provisional zero whose visible weights (nearly) vanished, sends the warp back to the
      // scores (they are still in tensor memory) for the row's true maximum, which becomes its reference.
      const bool redo = !(tile_sum < kSumGuard) || (fresh && seen && tile_sum < kSumTiny);
      if (__any_sync(0xffffffffu, redo)) {
        float top = -INFINITY;
        auto piece_max = [&](int c, uint32_t mask) {
          uint32_t raw[32];
          ptx::tmem_ld32(s_tmem + 32 * c, raw);
          ptx::tmem_wait_ld();
#pragma unroll
          for (int e = 0; e < 32; ++e)
            top = fmaxf(top, warp_full || ((mask >> e) & 1u) ? __uint_as_float(raw[e]) : -INFINITY);
        };
        uint32_t m0, m1, m2, m3;  // (formed again rather than kept alive across the exponentials)
        visibility(m0, m1, m2, m3);
        piece_max(0, m0);
        piece_max(1, m1);
        piece_max(2, m2);
        piece_max(3, m3);
        top *= sl2;
        float corr = 1.f;
        if (redo && top > -INFINITY) {
          // what has been summed so far (nothing, for a row on its provisional zero) goes over to the new reference
          corr = fresh ? 1.f : fast_exp2(m_ref - top);
          m_ref = top;
          l *= corr;
          fresh = false;
        }
        if (!rescale_output(corr)) return;
        exponentiate();
      }
      if (fresh && seen) m_ref = 0.f;  // the row has summed against the provisional zero: that is its reference now
      uint32_t lo[32], hi[32];
#pragma unroll
      for (int e = 0; e < 16; ++e) {
        lo[e] = pk0[e];
        lo[16 + e] = pk1[e];
        hi[e] = pk2[e];
        hi[16 + e] = pk3[e];
      }
      ptx::tmem_st32(s_tmem, lo);
      ptx::tmem_st32(s_tmem + 32, hi);
    }
    l += tile_sum;
    if (tile_sum > kSumMove && n + 2 < w.n_tiles) {
      // the tile outgrew the reference (its largest weight lies between 2^-7 and 1 of the sum): move the reference
      // by the sum's logarithm for the tiles to come
      const float shift = log2f(tile_sum);
      m_ref += shift;
      pending = fast_exp2(-shift);
      l *= pending;
    }
    ptx::tmem_wait_st();
    WM_TRACE(900 + n);
    // last tile: value rows at or beyond the largest visible slot may hold anything (unused cache capacity); so
    // may rows that the caller's key mask removes: their weights are zero, but zero times NaN is not
    const bool last_ragged = n == w.n_tiles - 1 && w.kmax < j0 + kTileN;
    if (last_ragged || !km_all) {
      const int s = n % kStages;
      if (!wait_or_abort(sm, &sm.v_full[s], (n / kStages) & 1, 34)) return;
      const uint32_t km_word = row < 32 ? km0 : (row < 64 ? km1 : (row < 96 ? km2 : km3));
      if ((last_ragged && j0 + row >= w.kmax) || !((km_word >> (row & 31)) & 1u)) {
#pragma unroll
        for (int h = 0; h < kSub; ++h) {
          uint4* vrow = reinterpret_cast<uint4*>(sm.v[s] + h * kSubBytes + row * 128);
#pragma unroll
          for (int c = 0; c < 8; ++c) vrow[c] = make_uint4(0, 0, 0, 0);
        }
      }
      ptx::fence_async_shared();
    }
    ptx::tc_fence_before();
    // The PV issuer reads p_full by parity: the group must not complete this tile's phase before the issuer has
    // consumed the phase of the group's previous tile, or the issuer, late by whatever the scheduler does to a
    // single-lane role, would see an unfinished phase of the same parity and wait for ever.  The issuer
    // acknowledges every phase it consumes on p_seen; by now that acknowledgement is long there.  The same wait
    // keeps a warp with nothing to do in a tile from arriving twice in one phase (the acknowledgement of a
    // phase implies that all 128 threads have arrived for it), and with it every thread of the group has left
    // the tile before the previous one when a thread starts a tile (the document tables are double-buffered).
    if (it >= 1 && !wait_or_abort(sm, &sm.p_seen[b], (it - 1) & 1, 42)) return;
    ptx::mbar_arrive(&sm.p_full[b]);
    WM_TRACE(1000 + n);
  }
  // epilogue: merge the two groups' partial results; this thread writes 32 of the row's 64 columns
  sm.row_max[grp][row] = m_ref;
  sm.row_sum[grp][row] = l;
  ptx::mbar_arrive(&sm.sum_full);
  if (!wait_or_abort(sm, &sm.sum_full, 0, 37)) return;
  const float m_other = sm.row_max[grp ^ 1][row], l_other = sm.row_sum[grp ^ 1][row];
  const float m_all = fmaxf(m_ref, m_other);
  const float w_mine = m_ref == -INFINITY ? 0.f : fast_exp2(m_ref - m_all);
  const float w_other = m_other == -INFINITY ? 0.f : fast_exp2(m_other - m_all);
  const float l_all = l * w_mine + l_other * w_other;
  const float inv = l_all > 0.f ? 1.f / l_all : 0.f;
  const float w0 = (grp == 0 ? w_mine : w_other) * inv, w1 = (grp == 0 ? w_other : w_mine) * inv;
  const int last = w.n_tiles - 1;
  // the last tile of either parity
  {
    const int last0 = last & 1 ? last - 1 : last, last1 = last & 1 ? last : last - 1;
    if (!wait_or_abort(sm, &sm.pv_done[last0 % kStages], (last0 / kStages) & 1, 35)) return;
    if (last1 >= 0 && !wait_or_abort(sm, &sm.pv_done[last1 % kStages], (last1 / kStages) & 1, 38)) return;
  }
  ptx::tc_fence_after();
  // this thread writes half of the row's D columns (the group picks the half), 32 at a time
  __nv_bfloat16* orow = static_cast<__nv_bfloat16*>(a.out) + batch * a.out_strides[0] + head * a.out_strides[1] +
                        static_cast<long long>(rb.qi) * a.out_strides[2] + grp * (D / 2);
  const bool use0 = w0 > 0.f, use1 = last >= 1 && w1 > 0.f;
  // whole 32-byte sectors where the caller's rows allow it: rows of different lanes are far apart, and partial
  // sectors are what makes such stores slow
  const bool sectors = (reinterpret_cast<uintptr_t>(orow) & 31) == 0;
#pragma unroll
  for (int part = 0; part < D / 64; ++part) {
    uint32_t acc0[32], acc1[32];
    ptx::tmem_ld32(tmem + kOutCol + lane_base + grp * (D / 2) + 32 * part, acc0);
    if (last >= 1) ptx::tmem_ld32(tmem + kOutCol + D + lane_base + grp * (D / 2) + 32 * part, acc1);
    ptx::tmem_wait_ld();
    if (live && grp * (D / 2) + 32 * part < a.head_dim) {  // (a head of 96 ends inside the second group's half)
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        uint32_t pk[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int i = 16 * u + 2 * e;
          const float lo = (use0 ? __uint_as_float(acc0[i]) * w0 : 0.f) + (use1 ? __uint_as_float(acc1[i]) * w1 : 0.f);
          const float hi = (use0 ? __uint_as_float(acc0[i + 1]) * w0 : 0.f) + (use1 ? __uint_as_float(acc1[i + 1]) * w1 : 0.f);
          pk[e] = pack_bf16(lo, hi);
        }
        __nv_bfloat16* dst = orow + 32 * part + 16 * u;
        if (sectors) {
          ptx::st_global_v8(dst, pk);
        } else {
          reinterpret_cast<uint4*>(dst)[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
          reinterpret_cast<uint4*>(dst)[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
        }
      }
    }
  }
  if (live) {
    if (grp == 0 && a.lse != nullptr)
      a.lse[(static_cast<long long>(batch) * a.q_heads + head) * a.q_len + rb.qi] =
          l_all > 0.f ? (m_all + log2f(l_all)) * kLn2 : INFINITY;
  }
}

template <int D>
__global__ void __launch_bounds__(kFwdThreads, 1)
    attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                        const __grid_constant__ CUtensorMap map_v, const wm_attn_args a, const int epoch) {
  WM_FWD_CONSTANTS(D);
  extern __shared__ unsigned char smem_raw[];
  FwdShared<D>& sm = *reinterpret_cast<FwdShared<D>*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int q_tile = gridDim.z - 1 - blockIdx.z;  // slowest grid dimension: the longest key walks start first
  const int head = blockIdx.x;
  const int batch = blockIdx.y;
  const int kv_head = head / (a.q_heads / a.kv_heads);
  const int q0 = q_tile * kTileM;
  const GroupCtx g = group_ctx(a, 0);

  // each softmax thread's row bounds: with documents they come from global memory, and asked for here they are on
  // their way while the barriers are set up
  RowBound rb;
  rb.lo = 0;
  rb.hi = 0;
  rb.seg = 0;
  rb.qi = q0 + (tid & 127);
  bool live = false;
  if (tid < kFwdSoftmax) {
    live = rb.qi < a.q_len;
    if (live) rb = row_bound(a, g, batch, rb.qi);
  }

  // Block set-up, one barrier for all of it.  The barriers are initialised by the first lanes of warp 0, a few each
  // (one thread doing all eighteen took 2 000 cycles and was what the block waited for); the producer lane sets up
  // the query tile's barrier itself and asks for the tile at once; warp 9 allocates tensor memory; the rows reduce
  // their bounds to one pair per warp; a thread without a row asks whether key slot 0 is the shared dummy.
  {
    // the barriers from k_full to sum_full lie side by side: lane i of warp 0 initialises the i-th, in one instruction
    constexpr int kBarriers = 4 * kStages + 5;
    static_assert(offsetof(FwdShared<D>, sum_full) - offsetof(FwdShared<D>, k_full) == (kBarriers - 1) * sizeof(uint64_t),
                  "the barriers of the forward are expected to be contiguous");
    if (tid < kBarriers) {
      const int count = tid < 4 * kStages ? 1 : (tid < 4 * kStages + 2 ? kFwdGroup : (tid < 4 * kStages + 4 ? 1 : kFwdSoftmax));
      ptx::mbar_init(sm.k_full + tid, count);
      ptx::mbar_fence_init();
    }
    if (tid == 0) {
      sm.abort_flag = 0;
      sm.epoch = epoch;
      trace_begin(sm, epoch);
    }
  }
  if (tid == 8 * 32) {
    // the query tile does not depend on the key walk: it is on its way while the rows find their bounds
    ptx::mbar_init(&sm.q_full, 1);
    ptx::mbar_fence_init();
    ptx::prefetch_tmap(&map_q);
    ptx::prefetch_tmap(&map_k);
    ptx::prefetch_tmap(&map_v);
    ptx::mbar_expect_tx(&sm.q_full, kTileBytes);
#pragma unroll
    for (int h = 0; h < kSub; ++h) ptx::tma_load_4d(sm.q + h * kSubBytes, &map_q, &sm.q_full, 64 * h, q0, head, batch);
  }
  if (warp == 9) {
    ptx::tmem_alloc(&sm.tmem_base, kTmemCols);
    ptx::tmem_relinquish();
  }
  if (tid == kFwdThreads - 1)
    sm.has_dummy = a.q_seg != nullptr && __ldg(a.k_seg + static_cast<long long>(batch) * a.k_len) == -1;
  if (tid < kTileM) {
    // (the second softmax group has the same rows)
    const int lo = live && rb.hi > 0 ? rb.lo : INT_MAX;
    const int wlo = __reduce_min_sync(0xffffffffu, lo);
    const int whi = __reduce_max_sync(0xffffffffu, rb.hi);
    if (lane == 0) {
      sm.warp_min_lo[warp] = wlo;
      sm.warp_max_hi[warp] = whi;
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = sm.tmem_base;
  const int red_min_lo = min(min(sm.warp_min_lo[0], sm.warp_min_lo[1]), min(sm.warp_min_lo[2], sm.warp_min_lo[3]));
  const int red_max_hi = max(max(sm.warp_max_hi[0], sm.warp_max_hi[1]), max(sm.warp_max_hi[2], sm.warp_max_hi[3]));
  TileWalk w;
  w.kmax = red_max_hi;
  if (w.kmax == 0) {
    // no row of the tile sees a key: zeros and +inf, then the common exit (the query tile still has to land)
    if (live) {
      __nv_bfloat16* orow = static_cast<__nv_bfloat16*>(a.out) + batch * a.out_strides[0] + head * a.out_strides[1] +
                            static_cast<long long>(rb.qi) * a.out_strides[2] + (tid >> 7) * (D / 2);
#pragma unroll
      for (int c = 0; c < D / 16; ++c)
        if ((tid >> 7) * (D / 2) + 8 * c < a.head_dim) reinterpret_cast<uint4*>(orow)[c] = make_uint4(0, 0, 0, 0);
      if (tid < kTileM && a.lse != nullptr)
        a.lse[(static_cast<long long>(batch) * a.q_heads + head) * a.q_len + rb.qi] = INFINITY;
    }
    if (tid == 0) wait_or_abort(sm, &sm.q_full, 0, 20);
  } else {
    const int end_tile = (w.kmax + kTileN - 1) / kTileN;
    w.first_tile = a.q_seg != nullptr ? min(red_min_lo / kTileN, end_tile - 1) : 0;
    w.dummy_tile = (a.q_seg != nullptr && sm.has_dummy && w.first_tile > 0) ? 1 : 0;
    w.n_tiles = end_tile - w.first_tile + w.dummy_tile;
    if (warp < 8) {
      softmax_role<D>(sm, a, tmem, w, rb, live, batch, head);
    } else if (lane == 0) {
      if (warp == 8) producer_role<D>(sm, &map_q, &map_k, &map_v, w, q0, head, kv_head, batch);
      if (warp == 9) score_mma_role<D>(sm, tmem, w);
      if (warp == 10) value_mma_role<D>(sm, tmem, w);
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  trace_flush(sm);
  if (warp == 9) ptx::tmem_dealloc(tmem, kTmemCols);
}
