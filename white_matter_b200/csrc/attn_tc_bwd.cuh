// Backward pipeline of the tcgen05 attention kernel (included by attn_tc.cu).
#pragma once

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
// TMEM columns, head size 64: S [0,128) dP [128,256) dV [256,320) dK [320,384) dQ [384,448).
//
// The kernel is a template over the head size D (64 or 128; 96 runs as 128 over tensor maps of 96 columns, whose
// copies fill columns 96..127 with zeros).  At 128 a Q, K, V or dO tile travels as two 64-column sub-tiles (one
// 128-byte swizzle row per token each), S and dP run eight K=16 steps over both, and the three gradient products
// are issued once per 64-column half of their result.  dV and dK then take 128 columns each, which fills the 512
// with S and dP: dQ of a pair is formed over the columns of S (the compute threads have read the scores by the
// time dS exists), and the next pair's score product waits until they have taken dQ out.  Q and dO have one stage
// instead of two (192 KB of shared memory).
template <int D>
struct BwdCfg {
  static constexpr int kSub = D / 64;
  static constexpr uint32_t kBytes = kTileN * D * 2;  // one Q, K, V or dO tile
  static constexpr int kQStages = D == 64 ? 2 : 1;
  static constexpr bool kDqOverS = D > 64;
  // D = 64 has the room (shared memory for a second P/dS pair, 64 tensor-memory columns for dQ) to overlap the pairs
  // of a walk: S/dP of the next pair are issued before the gradient products of this one, the compute warps go from
  // one pair straight to the next and take dQ out one pair late, when it has long been formed.
  static constexpr bool kOverlap = D == 64;
  static constexpr int kPds = kOverlap ? 2 : 1;
  // Eight compute warps at every head size: two per quarter of the rows, each with one half of the columns (the
  // backward needs no row maximum, so the halves exchange nothing).
  static constexpr int kComputeWarps = 8;
  static constexpr int kSplit = kComputeWarps / 4;           // warps per row: each takes kTileN / kSplit columns
  static constexpr int kThreads = (kComputeWarps + 2) * 32;  // + producer + MMA issuer
  static constexpr uint32_t kColDv = 2 * kTileN, kColDk = 2 * kTileN + D;
  static constexpr uint32_t kColDq = kDqOverS ? 0 : 2 * kTileN + 2 * D;
};

template <int D>
struct BwdShared {
  unsigned char k[BwdCfg<D>::kBytes];
  unsigned char v[BwdCfg<D>::kBytes];
  unsigned char q[BwdCfg<D>::kQStages][BwdCfg<D>::kBytes];
  unsigned char g[BwdCfg<D>::kQStages][BwdCfg<D>::kBytes];  // dO tiles
  unsigned char p[BwdCfg<D>::kPds][2 * kTileBytes];
  unsigned char ds[BwdCfg<D>::kPds][2 * kTileBytes];
  uint64_t kv_full, kv_ready;
  uint64_t qg_full[BwdCfg<D>::kQStages], qg_empty[BwdCfg<D>::kQStages];
  uint64_t sdp_full, pds_full, mma_done[BwdCfg<D>::kPds], dq_full, dq_free;
  int key_seg[kTileN];
  int key_end[kTileN];
  int summary[4][4];  // per warp: min seg, max seg, min end, max end
  uint32_t key_keep[4];  // key_mask of the tile, one bit per key slot (all ones without a mask)
  int row_first, row_end;
  uint32_t tmem_base;
  int abort_flag;
  int epoch;
};

// delta = rowsum(dO * O) in fp32.  kLanes neighbouring lanes share a (batch, head, query) row of 8 * kChunks values,
// 16 bytes of O and of dO each (a warp reads whole 128-byte lines), and add their parts up with shuffles.
template <int kChunks, int kLanes>
__global__ void bwd_delta_kernel(const wm_attn_args a, float* delta) {
  static_assert(kLanes >= kChunks && (kLanes & (kLanes - 1)) == 0 && kLanes <= 32, "lanes per row");
  const long long rows = static_cast<long long>(a.batch) * a.q_heads * a.q_len;
  const long long at = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const long long row = at / kLanes;
  const int c = static_cast<int>(at % kLanes);
  float acc = 0.f;
  if (row < rows && c < kChunks) {
    const int i = static_cast<int>(row % a.q_len);
    const int h = static_cast<int>((row / a.q_len) % a.q_heads);
    const int b = static_cast<int>(row / (static_cast<long long>(a.q_len) * a.q_heads));
    const uint4 x = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(a.out) + b * a.out_strides[0] +
                                                   h * a.out_strides[1] + static_cast<long long>(i) * a.out_strides[2])[c];
    const uint4 y = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(a.dout) + b * a.dout_strides[0] +
                                                   h * a.dout_strides[1] + static_cast<long long>(i) * a.dout_strides[2])[c];
    const unsigned xs[4] = {x.x, x.y, x.z, x.w}, ys[4] = {y.x, y.y, y.z, y.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      acc = fmaf(__uint_as_float(xs[e] << 16), __uint_as_float(ys[e] << 16), acc);
      acc = fmaf(__uint_as_float(xs[e] & 0xffff0000u), __uint_as_float(ys[e] & 0xffff0000u), acc);
    }
  }
#pragma unroll
  for (int step = kLanes / 2; step > 0; step >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, step);
  if (row < rows && c == 0) delta[row] = acc;
}

// dq = bf16(scale * accumulator); accumulator is (batch, heads, queries, head_dim) fp32
__global__ void bwd_dq_convert_kernel(const wm_attn_args a, const float* acc) {
  const int per_row = a.head_dim / 8;  // chunks of 8 values
  const long long chunks = static_cast<long long>(a.batch) * a.q_heads * a.q_len * per_row;
  const long long at = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (at >= chunks) return;
  const long long row = at / per_row;
  const int c = static_cast<int>(at - row * per_row);
  const int i = static_cast<int>(row % a.q_len);
  const int h = static_cast<int>((row / a.q_len) % a.q_heads);
  const int b = static_cast<int>(row / (static_cast<long long>(a.q_len) * a.q_heads));
  const float4 lo = *reinterpret_cast<const float4*>(acc + row * a.head_dim + c * 8);
  const float4 hi = *reinterpret_cast<const float4*>(acc + row * a.head_dim + c * 8 + 4);
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

template <int D>
__device__ __forceinline__ void bwd_producer(BwdShared<D>& sm, const CUtensorMap* map_q, const CUtensorMap* map_k,
                                             const CUtensorMap* map_v, const CUtensorMap* map_g, const BwdWalk& w,
                                             int j0, int kv_head, int batch) {
  constexpr int kBwdStages = BwdCfg<D>::kQStages, kSub = BwdCfg<D>::kSub;
  constexpr uint32_t kBytes = BwdCfg<D>::kBytes;
  ptx::prefetch_tmap(map_q);
  ptx::prefetch_tmap(map_k);
  ptx::prefetch_tmap(map_v);
  ptx::prefetch_tmap(map_g);
  ptx::mbar_expect_tx(&sm.kv_full, 2 * kBytes);
#pragma unroll
  for (int h = 0; h < kSub; ++h) {
    ptx::tma_load_4d(sm.k + h * kSubBytes, map_k, &sm.kv_full, 64 * h, j0, kv_head, batch);
    ptx::tma_load_4d(sm.v + h * kSubBytes, map_v, &sm.kv_full, 64 * h, j0, kv_head, batch);
  }
  for (int it = 0; it < w.n_iter; ++it) {
    const int s = it % kBwdStages;
    int head, qt;
    bwd_iter_coords(w, it, kv_head, head, qt);
    if (!wait_or_abort(sm, &sm.qg_empty[s], ((it / kBwdStages) & 1) ^ 1, 41)) return;
    ptx::mbar_expect_tx(&sm.qg_full[s], 2 * kBytes);
#pragma unroll
    for (int h = 0; h < kSub; ++h) {
      ptx::tma_load_4d(sm.q[s] + h * kSubBytes, map_q, &sm.qg_full[s], 64 * h, qt * kTileM, head, batch);
      ptx::tma_load_4d(sm.g[s] + h * kSubBytes, map_g, &sm.qg_full[s], 64 * h, qt * kTileM, head, batch);
    }
  }
}

template <int D>
__device__ __forceinline__ void bwd_mma(BwdShared<D>& sm, uint32_t tmem, const BwdWalk& w) {
  using Cfg = BwdCfg<D>;
  constexpr int kBwdStages = Cfg::kQStages;
  constexpr uint32_t kHalfStep = D > 64 ? kSubBytes : 1024;  // between the 64-column halves of an MN-major B operand
  if (!wait_or_abort(sm, &sm.kv_ready, 0, 50)) return;
  ptx::tc_fence_after();
  constexpr uint32_t idesc_s = ptx::make_idesc_bf16(kTileM, kTileN, 0, 0);      // Q K^T, dO V^T
  constexpr uint32_t idesc_t = ptx::make_idesc_bf16(kTileN, D, 1, 1);           // P^T dO, dS^T Q
  constexpr uint32_t idesc_q = ptx::make_idesc_bf16(kTileM, D, 0, 1);           // dS K
  const uint32_t k_base = ptx::smem_u32(sm.k), v_base = ptx::smem_u32(sm.v);
  // S = Q K^T and dP = dO V^T of pair `it` into their tensor-memory columns
  auto scores = [&](int it) -> bool {
    const int s = it % kBwdStages;
    if (!wait_or_abort(sm, &sm.qg_full[s], (it / kBwdStages) & 1, 51)) return false;
    if (Cfg::kDqOverS) {
      // dQ of the previous pair lives in the columns of S until the compute threads have taken it out
      if (!wait_or_abort(sm, &sm.dq_free, (it & 1) ^ 1, 54)) return false;
    }
    ptx::tc_fence_after();
    const uint32_t q_base = ptx::smem_u32(sm.q[s]), g_base = ptx::smem_u32(sm.g[s]);
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      const uint32_t at = (kk >> 2) * kSubBytes + (kk & 3) * 32;
      ptx::mma_bf16_ss(tmem, ptx::make_smem_desc_sw128(q_base + at, 16, 1024),
                       ptx::make_smem_desc_sw128(k_base + at, 16, 1024), idesc_s, kk > 0);
    }
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      const uint32_t at = (kk >> 2) * kSubBytes + (kk & 3) * 32;
      ptx::mma_bf16_ss(tmem + kTileN, ptx::make_smem_desc_sw128(g_base + at, 16, 1024),
                       ptx::make_smem_desc_sw128(v_base + at, 16, 1024), idesc_s, kk > 0);
    }
    ptx::mma_commit(&sm.sdp_full);
    return true;
  };
  if (Cfg::kOverlap && w.n_iter > 0 && !scores(0)) return;
  for (int it = 0; it < w.n_iter; ++it) {
    const int s = it % kBwdStages;
    const int pb = Cfg::kOverlap ? (it & 1) : 0;  // P/dS buffer of the pair
    if (!Cfg::kOverlap && !scores(it)) return;
    if (!wait_or_abort(sm, &sm.pds_full, it & 1, 52)) return;
    ptx::tc_fence_after();
    // the compute threads have read S and dP: the next pair's go out before this pair's gradient products
    if (Cfg::kOverlap && it + 1 < w.n_iter && !scores(it + 1)) return;
    const uint32_t q_base = ptx::smem_u32(sm.q[s]), g_base = ptx::smem_u32(sm.g[s]);
    const uint32_t p_base = ptx::smem_u32(sm.p[pb]), ds_base = ptx::smem_u32(sm.ds[pb]);
    // the gradient products span all D result columns in one instruction: the MN-major B operand steps from one
    // 64-column sub-tile to the next by its leading-dimension offset, like the two 64-key halves of P and dS
#pragma unroll
    for (int kk = 0; kk < kTileM / 16; ++kk)  // 16 queries per instruction
      ptx::mma_bf16_ss(tmem + Cfg::kColDv, ptx::make_smem_desc_sw128(p_base + kk * 2048, kTileBytes, 1024),
                       ptx::make_smem_desc_sw128(g_base + kk * 2048, kHalfStep, 1024), idesc_t, (it > 0) || (kk > 0));
#pragma unroll
    for (int kk = 0; kk < kTileM / 16; ++kk)
      ptx::mma_bf16_ss(tmem + Cfg::kColDk, ptx::make_smem_desc_sw128(ds_base + kk * 2048, kTileBytes, 1024),
                       ptx::make_smem_desc_sw128(q_base + kk * 2048, kHalfStep, 1024), idesc_t, (it > 0) || (kk > 0));
    if (!Cfg::kDqOverS) {
      if (!wait_or_abort(sm, &sm.dq_free, (it & 1) ^ 1, 53)) return;
      ptx::tc_fence_after();
    }
#pragma unroll
    for (int kk = 0; kk < kTileN / 16; ++kk)  // 16 keys per instruction
      ptx::mma_bf16_ss(tmem + Cfg::kColDq,
                       ptx::make_smem_desc_sw128(ds_base + (kk >> 2) * kTileBytes + (kk & 3) * 32, 16, 1024),
                       ptx::make_smem_desc_sw128(k_base + kk * 2048, kHalfStep, 1024), idesc_q, kk > 0);
    ptx::mma_commit(&sm.qg_empty[s]);
    ptx::mma_commit(&sm.mma_done[pb]);
    ptx::mma_commit(&sm.dq_full);
  }
}

// Whether query row i (bounds rb) sees nothing of the block's key tile.
__device__ __forceinline__ bool bwd_row_sees_nothing(const RowBound& rb, bool live, int j0, bool docs, int smin, int smax) {
  bool none = !live || j0 >= rb.hi;
  if (docs && !none && smin == smax && smin != -1 && smin != rb.seg) none = true;
  return none;
}

// dQ of one pair: from tensor memory into the fp32 accumulator in global memory (thread = query row; pieces of 32
// columns from `first`, `count` of them)
template <int D>
__device__ __forceinline__ void bwd_dq_out(const wm_attn_args& a, uint32_t tmem_dq, float* dq_acc, long long stat, bool wanted,
                                           int first, int count) {
  for (int c = first; c < first + count; ++c) {
    uint32_t raw[32];
    ptx::tmem_ld32(tmem_dq + c * 32, raw);
    ptx::tmem_wait_ld();
    if (wanted && c * 32 < a.head_dim) {
      float* dst = dq_acc + stat * a.head_dim + c * 32;
#pragma unroll
      for (int e = 0; e < 8; ++e)
        red_add_v4(dst + 4 * e, __uint_as_float(raw[4 * e]), __uint_as_float(raw[4 * e + 1]),
                   __uint_as_float(raw[4 * e + 2]), __uint_as_float(raw[4 * e + 3]));
    }
  }
}

// compute threads of the backward kernel: thread t owns query row t of the current query tile (and, in
// the prologue / epilogue, key row t of the CTA's key tile)
template <int D>
__device__ __forceinline__ void bwd_compute(BwdShared<D>& sm, const wm_attn_args& a, uint32_t tmem, const BwdWalk& w,
                                            const float* delta, float* dq_acc, int j0, int kv_head, int batch) {
  using Cfg = BwdCfg<D>;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = (warp & 3) * 32 + lane;  // query row of the pair (and key row of the block's tile) = TMEM lane
  const int half = warp >> 2;            // which part of the columns (0 when one warp has the whole row)
  const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
  const float sl2 = a.scale * kLog2e;
  const bool docs = a.q_seg != nullptr;
  const GroupCtx g = group_ctx(a, 0);
  constexpr int kPieces = kTileN / 32 / Cfg::kSplit;    // 32-column pieces of S/dP per thread
  constexpr int kOutPieces = D / 32 / Cfg::kSplit;      // 32-column pieces of dQ, dK and dV per thread

  // prologue: key rows at or beyond the last visible slot, and rows the key mask removes, may hold anything;
  // clear them for the MMAs (one thread per key row)
  const bool masked = a.key_mask != nullptr;
  if (half == 0) {
    if (!wait_or_abort(sm, &sm.kv_full, 0, 60)) return;
    if (j0 + t >= w.kvis || !((sm.key_keep[t >> 5] >> (t & 31)) & 1u)) {
#pragma unroll
      for (int h = 0; h < Cfg::kSub; ++h) {
        uint4* krow = reinterpret_cast<uint4*>(sm.k + h * kSubBytes + t * 128);
        uint4* vrow = reinterpret_cast<uint4*>(sm.v + h * kSubBytes + t * 128);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          krow[c] = make_uint4(0, 0, 0, 0);
          vrow[c] = make_uint4(0, 0, 0, 0);
        }
      }
    }
    ptx::fence_async_shared();
    ptx::mbar_arrive(&sm.kv_ready);
  }

  int smin = 0, smax = 0, emin = 0;
  if (docs) {
    smin = min(min(sm.summary[0][0], sm.summary[1][0]), min(sm.summary[2][0], sm.summary[3][0]));
    smax = max(max(sm.summary[0][1], sm.summary[1][1]), max(sm.summary[2][1], sm.summary[3][1]));
    emin = min(min(sm.summary[0][2], sm.summary[1][2]), min(sm.summary[2][2], sm.summary[3][2]));
  }

  // dQ of pair `it` out of tensor memory (this thread's pieces of its row)
  auto take_dq = [&](int it, long long stat, bool wanted) -> bool {
    if (!wait_or_abort(sm, &sm.dq_full, it & 1, 63)) return false;
    ptx::tc_fence_after();
    bwd_dq_out<D>(a, tmem + Cfg::kColDq + lane_base, dq_acc, stat, wanted, half * kOutPieces, kOutPieces);
    ptx::tc_fence_before();
    ptx::mbar_arrive(&sm.dq_free);
    return true;
  };
  long long late_stat = 0;  // the pair whose dQ is still to be taken out (overlapping pairs)
  bool late_wanted = false;

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
    bool full = live && j0 + kTileN <= rb.hi && !masked;
    bool own_doc = !docs;  // the tile lies inside the row's own document: only the causal bound can cut it
    if (docs && !none) {
      const bool uniform = smin == smax;
      own_doc = uniform && smin == rb.seg && j0 >= rb.lo && emin > rb.qi;
      full = full && own_doc;
      if (uniform && smin != -1 && smin != rb.seg) none = true;
    }
    if (!wait_or_abort(sm, &sm.sdp_full, it & 1, 61)) return;
    ptx::tc_fence_after();
    // the shared P / dS tiles were last read by the gradient products of the pair that used them before: the
    // previous pair, or with two buffers the one before that
    const int pb = Cfg::kOverlap ? (it & 1) : 0;
    if (Cfg::kOverlap) {
      if (it >= 2 && !wait_or_abort(sm, &sm.mma_done[pb], ((it >> 1) & 1) ^ 1, 62)) return;
    } else {
      if (it > 0 && !wait_or_abort(sm, &sm.mma_done[0], (it - 1) & 1, 62)) return;
    }
    unsigned char* prow = sm.p[pb] + (t >> 3) * 1024 + (t & 7) * 128;
    unsigned char* drow = sm.ds[pb] + (t >> 3) * 1024 + (t & 7) * 128;
    const int lim = rb.hi - j0;
#pragma unroll 1
    for (int c = half * kPieces; c < (half + 1) * kPieces; ++c) {
      uint32_t xs[32], ys[32];
      const uint32_t keep = masked ? sm.key_keep[c] : 0xffffffffu;
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
          bool vis = !none && (full || (col < lim && ((keep >> (2 * e + u)) & 1u)));
          if (!own_doc) vis = vis & doc_visible_flat(rb, j0 + col, sm.key_seg[col], sm.key_end[col]);
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
    if (Cfg::kOverlap) {
      // dQ of the pair before this one: its products were issued while this pair was computed
      if (it > 0 && !take_dq(it - 1, late_stat, late_wanted)) return;
      late_stat = stat;
      late_wanted = live && !none;
    } else {
      if (!take_dq(it, stat, live && !none)) return;
    }
  }
  if (Cfg::kOverlap && w.n_iter > 0) {
    // the last pair's dQ; its barrier covers every product of the walk
    if (!take_dq(w.n_iter - 1, late_stat, late_wanted)) return;
    ptx::tc_fence_after();
  }

  // epilogue: dV and dK rows of this key tile (dq_full of the last pair covers every earlier product); this thread
  // writes its pieces of key row t
  const int j = j0 + t;
  uint4* dvrow = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(a.dv) + batch * a.dv_strides[0] +
                                          kv_head * a.dv_strides[1] + static_cast<long long>(j) * a.dv_strides[2]);
  uint4* dkrow = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(a.dk) + batch * a.dk_strides[0] +
                                          kv_head * a.dk_strides[1] + static_cast<long long>(j) * a.dk_strides[2]);
  for (int c = half * kOutPieces; c < (half + 1) * kOutPieces; ++c) {
    uint32_t dv_pack[16], dk_pack[16];
#pragma unroll
    for (int e = 0; e < 16; ++e) dv_pack[e] = dk_pack[e] = 0u;
    if (w.n_iter > 0) {
      uint32_t raw[32];
      ptx::tmem_ld32(tmem + Cfg::kColDv + lane_base + c * 32, raw);
      ptx::tmem_wait_ld();
#pragma unroll
      for (int e = 0; e < 16; ++e) dv_pack[e] = pack_bf16(__uint_as_float(raw[2 * e]), __uint_as_float(raw[2 * e + 1]));
      ptx::tmem_ld32(tmem + Cfg::kColDk + lane_base + c * 32, raw);
      ptx::tmem_wait_ld();
#pragma unroll
      for (int e = 0; e < 16; ++e)
        dk_pack[e] = pack_bf16(__uint_as_float(raw[2 * e]) * a.scale, __uint_as_float(raw[2 * e + 1]) * a.scale);
    }
    if (j < a.k_len && c * 32 < a.head_dim) {
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        dvrow[4 * c + u] = make_uint4(dv_pack[4 * u], dv_pack[4 * u + 1], dv_pack[4 * u + 2], dv_pack[4 * u + 3]);
        dkrow[4 * c + u] = make_uint4(dk_pack[4 * u], dk_pack[4 * u + 1], dk_pack[4 * u + 2], dk_pack[4 * u + 3]);
      }
    }
  }
}

template <int D>
__global__ void __launch_bounds__(BwdCfg<D>::kThreads, 1)
    attn_bwd_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_g,
                       const wm_attn_args a, const float* delta, float* dq_acc, const int epoch) {
  extern __shared__ unsigned char smem_raw[];
  constexpr int kBwdStages = BwdCfg<D>::kQStages;
  BwdShared<D>& sm = *reinterpret_cast<BwdShared<D>*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int j0 = blockIdx.x * kTileN;
  const int kv_head = blockIdx.y;
  const int batch = blockIdx.z;
  const GroupCtx g = group_ctx(a, 0);
  const bool docs = a.q_seg != nullptr;

  if (tid == 0) {
    sm.abort_flag = 0;
    sm.epoch = epoch;
  }
  if (tid < kSoftmaxThreads) {
    bool keep = true;
    if (a.key_mask != nullptr)
      keep = j0 + tid < a.k_len && a.key_mask[static_cast<long long>(batch) * a.k_len + j0 + tid] != 0;
    const uint32_t word = __ballot_sync(0xffffffffu, keep);
    if (lane == 0) sm.key_keep[warp] = word;
  }
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
      for (int c = 0; c < a.head_dim / 8; ++c) {
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
    ptx::mbar_init(&sm.pds_full, BwdCfg<D>::kComputeWarps * 32);
    for (int b = 0; b < BwdCfg<D>::kPds; ++b) ptx::mbar_init(&sm.mma_done[b], 1);
    ptx::mbar_init(&sm.dq_full, 1);
    ptx::mbar_init(&sm.dq_free, BwdCfg<D>::kComputeWarps * 32);
    ptx::mbar_fence_init();
  }
  constexpr int kCW = BwdCfg<D>::kComputeWarps;
  if (warp == kCW) {
    ptx::tmem_alloc(&sm.tmem_base, kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = sm.tmem_base;
  if (warp < kCW) {
    bwd_compute(sm, a, tmem, w, delta, dq_acc, j0, kv_head, batch);
  } else if (warp == kCW) {
    if (lane == 0) bwd_producer(sm, &map_q, &map_k, &map_v, &map_g, w, j0, kv_head, batch);
  } else {
    if (lane == 0) bwd_mma(sm, tmem, w);
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == kCW) ptx::tmem_dealloc(tmem, kTmemCols);
}
