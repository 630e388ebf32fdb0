// KV-pool projection path either side of its per-channel GEMMs.
//
// pool_mix: for one token row, the `sources` layer inputs are normalised, gained, mixed into `channels` vectors
// per side (K, V) with signed routing logits, normalised again and gained -- everything the pool does between the
// layer stack and the projection GEMMs, in one pass: the row's sources are read from HBM once, the source norms and
// the routing coefficients are formed in shared memory, and the 2*channels mixtures leave as the rows of the GEMM's
// A operand.  Algorithmic bytes per token row: sources*hidden*sizeof(T) read + 2*channels*hidden*sizeof(T) written
// (+ the routing partials when the router is dynamic).  Two kernels: BF16 stacks of width <= 1024 mix on the
// warp-level tensor-core instruction (further down); FP32 stacks and other widths keep the sources in registers and
// mix on the packed two-wide FP32 FMA (2*sources*channels FMAs per loaded element, which bound that kernel far
// below HBM bandwidth).
//
// pool_finish: the projected channels get the per-channel key norm, the rotary embedding and the move into the
// pool's (batch, channel*head, slot, dim) layout; values only move.  One read and one write of K and V.
#include <math.h>

#include <atomic>
#include <type_traits>

#include "common.cuh"

namespace wm {
namespace {

constexpr int kChannelsPerPass = 8;

template <typename T>
struct Quad;  // four adjacent elements as they travel
template <>
struct Quad<float> {
  using type = float4;
};
template <>
struct Quad<__nv_bfloat16> {
  using type = uint2;
};

__device__ __forceinline__ float4 widen(const float4& v) { return v; }
__device__ __forceinline__ float4 widen(const uint2& v) {
  return make_float4(__uint_as_float(v.x << 16), __uint_as_float(v.x & 0xffff0000u), __uint_as_float(v.y << 16),
                     __uint_as_float(v.y & 0xffff0000u));
}
__device__ __forceinline__ void narrow(float4* p, const float4& v) { __stcs(p, v); }
__device__ __forceinline__ void narrow(uint2* p, const float4& v) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  uint2 w;
  w.x = *reinterpret_cast<const unsigned*>(&lo);
  w.y = *reinterpret_cast<const unsigned*>(&hi);
  *p = w;  // default caching: the projection GEMM reads these rows next
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Per-group scratch of pool_mix, in floats: per-warp partial sums of squares, the sources' inverse norms, the
// per-token mixing coefficients (side, source, channel) and two alternating buffers of per-warp channel sums.
struct MixLayout {
  int red, inv, coef, chan, total;
  __host__ __device__ MixLayout(int warps, int sources, int padded_channels) {
    red = 0;
    inv = red + ((warps * sources + 3) & ~3);
    coef = inv + ((sources + 3) & ~3);
    chan = coef + 2 * sources * padded_channels;
    total = (chan + 2 * warps * kChannelsPerPass + 3) & ~3;
  }
};

__device__ __forceinline__ void group_barrier(int group, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(group + 1), "r"(threads) : "memory");
}

__device__ __forceinline__ float4 gain4(const float* p) { return __ldg(reinterpret_cast<const float4*>(p)); }
__device__ __forceinline__ float4 gain4(const __nv_bfloat16* p) { return widen(*reinterpret_cast<const uint2*>(p)); }

// A block holds `groups` groups of hidden/4 threads; a group owns one token row at a time and a thread four adjacent
// columns of it.  With kStaged the four gain tables (pre-mix K and V, post-mix K and V) are copied once per block
// into shared memory in the stack's dtype and every row reads them from there; a block stays resident (one per SM)
// and walks over the rows.  Without it (tables too large, or FP32) the gains come through L1.
template <typename T, int kL, bool kStaged>
__global__ void __launch_bounds__(512) pool_mix_kernel(const wm_pool_mix_args a, const long long rows) {
  using Q = typename Quad<T>::type;
  using G = typename std::conditional<kStaged, T, float>::type;  // element type the gains are read in
  extern __shared__ __align__(128) unsigned char raw[];
  const int L = a.sources, C = a.channels, Dm = a.hidden;
  const int group_threads = Dm / 4;
  const int groups = blockDim.x / group_threads;
  const int group = threadIdx.x / group_threads, tid = threadIdx.x - group * group_threads;
  const int lane = tid & 31, warp = tid >> 5, warps = group_threads >> 5;
  const int col = tid * 4;
  const int CL = C * L;
  const long long PS = a.partial_row_stride ? a.partial_row_stride : CL;  // elements between rows of a partial
  const int Cpad = (C + kChannelsPerPass - 1) / kChannelsPerPass * kChannelsPerPass;
  const MixLayout lay(warps, L, Cpad);
  const size_t staged_bytes = kStaged ? (static_cast<size_t>(2) * (L + C) * Dm * sizeof(T) + 15) / 16 * 16 : 0;
  float* scratch = reinterpret_cast<float*>(raw + staged_bytes) + group * lay.total;
  float* red = scratch + lay.red;
  float* inv = scratch + lay.inv;
  float* coef = scratch + lay.coef;
  float* chan = scratch + lay.chan;
  const float inv_hidden = 1.f / static_cast<float>(Dm);

  const G *pre_k, *pre_v, *post_k, *post_v;
  if (kStaged) {
    T* stage = reinterpret_cast<T*>(raw);
    const float* tables[4] = {a.pre_mix_k, a.pre_mix_v, a.gain_k, a.gain_v};
    const int sizes[4] = {L * Dm, L * Dm, a.gain_k ? C * Dm : 0, a.gain_k ? C * Dm : 0};
    T* at = stage;
    for (int k = 0; k < 4; ++k) {
      for (int i = threadIdx.x; i < sizes[k]; i += blockDim.x) at[i] = from_float<T>(tables[k][i]);
      at += sizes[k];
    }
    pre_k = reinterpret_cast<const G*>(stage);
    pre_v = pre_k + L * Dm;
    post_k = pre_v + L * Dm;
    post_v = post_k + C * Dm;
  } else {
    pre_k = reinterpret_cast<const G*>(a.pre_mix_k);
    pre_v = reinterpret_cast<const G*>(a.pre_mix_v);
    post_k = reinterpret_cast<const G*>(a.gain_k);
    post_v = reinterpret_cast<const G*>(a.gain_v);
  }
  // channels beyond `channels` in the last pass of eight mix with zero coefficients and are never stored
  for (int i = tid; i < 2 * L * Cpad; i += group_threads) coef[i] = 0.f;
  __syncthreads();

  const long long row_step = static_cast<long long>(gridDim.x) * groups;
  const int lines_per_source = Dm * static_cast<int>(sizeof(T)) / 128;
  for (long long row = static_cast<long long>(blockIdx.x) * groups + group; row < rows; row += row_step) {
    const long long b = row / a.tokens, t = row - b * a.tokens;
    const T* x0 = static_cast<const T*>(a.stacked) + b * a.stacked_strides[0] + t * a.stacked_strides[1];
    Q x[kL];
#pragma unroll
    for (int l = 0; l < kL; ++l)
      if (l < L) x[l] = __ldcs(reinterpret_cast<const Q*>(x0 + l * a.stacked_strides[2] + col));
    // pull the group's next row into L2 while this one is mixed
    if (row + row_step < rows) {
      const long long nb = (row + row_step) / a.tokens, nt = (row + row_step) - nb * a.tokens;
      const T* next = static_cast<const T*>(a.stacked) + nb * a.stacked_strides[0] + nt * a.stacked_strides[1];
      for (int i = tid; i < L * lines_per_source; i += group_threads) {
        const int l = i / lines_per_source, line = i - l * lines_per_source;
        asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const char*>(next + l * a.stacked_strides[2]) + line * 128));
      }
    }

    // inverse RMS of every source
#pragma unroll
    for (int l = 0; l < kL; ++l)
      if (l < L) {
        const float4 v = widen(x[l]);
        const float s = warp_sum(fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, v.w * v.w))));
        if (lane == 0) red[warp * L + l] = s;
      }
    group_barrier(group, group_threads);
    if (tid < L) {
      float s = 0.f;
      for (int w = 0; w < warps; ++w) s += red[w * L + tid];
      inv[tid] = rsqrtf(s * inv_hidden + a.source_eps);
    }
    group_barrier(group, group_threads);

    // routing logits of this token times the source norms: the coefficient of the raw, gained source
    for (int i = tid; i < 2 * CL; i += group_threads) {
      const int side = i >= CL;
      const int o = i - side * CL;
      const int c = o / L, l = o - c * L;
      float alpha = (side ? a.bias_v : a.bias_k)[o];
      const T* part = static_cast<const T*>(side ? a.partial_v : a.partial_k);
      if (part != nullptr)
        for (int j = 0; j < a.n_routed; ++j)
          alpha = fmaf(inv[a.route_start + j * a.route_stride], to_float(part[(j * rows + row) * PS + o]), alpha);
      coef[(side * L + l) * Cpad + c] = alpha * inv[l];
    }
    group_barrier(group, group_threads);

    int pass = 0;
    for (int c0 = 0; c0 < C; c0 += kChannelsPerPass) {
#pragma unroll 1
      for (int side = 0; side < 2; ++side, ++pass) {
        const G* gain_in = (side ? pre_v : pre_k) + col;
        const float* cf = coef + side * L * Cpad + c0;
        float2 acc[kChannelsPerPass][2];
#pragma unroll
        for (int c = 0; c < kChannelsPerPass; ++c) acc[c][0] = acc[c][1] = make_float2(0.f, 0.f);
#pragma unroll
        for (int l = 0; l < kL; ++l)
          if (l < L) {
            const float4 v = widen(x[l]);
            const float4 g = gain4(gain_in + l * Dm);
            const float2 lo = __fmul2_rn(make_float2(v.x, v.y), make_float2(g.x, g.y));
            const float2 hi = __fmul2_rn(make_float2(v.z, v.w), make_float2(g.z, g.w));
            const float4 w0 = *reinterpret_cast<const float4*>(cf + l * Cpad);
            const float4 w1 = *reinterpret_cast<const float4*>(cf + l * Cpad + 4);
            const float w[kChannelsPerPass] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
            for (int c = 0; c < kChannelsPerPass; ++c) {
              const float2 ww = make_float2(w[c], w[c]);
              acc[c][0] = __ffma2_rn(lo, ww, acc[c][0]);
              acc[c][1] = __ffma2_rn(hi, ww, acc[c][1]);
            }
          }
        float* sums = chan + (pass & 1) * warps * kChannelsPerPass;
#pragma unroll
        for (int c = 0; c < kChannelsPerPass; ++c) {
          const float2 p = __ffma2_rn(acc[c][0], acc[c][0], __fmul2_rn(acc[c][1], acc[c][1]));
          const float s = warp_sum(p.x + p.y);
          if (lane == 0) sums[warp * kChannelsPerPass + c] = s;
        }
        group_barrier(group, group_threads);
        const G* gain_out = (side ? post_v : post_k) + col;
        T* out = static_cast<T*>(side ? a.mixed_v : a.mixed_k) + row * Dm + col;
#pragma unroll
        for (int c = 0; c < kChannelsPerPass; ++c)
          if (c0 + c < C) {
            float s = 0.f;
            for (int w = 0; w < warps; ++w) s += sums[w * kChannelsPerPass + c];
            const float r = rsqrtf(s * inv_hidden + a.mix_eps);
            const float4 g = a.gain_k != nullptr ? gain4(gain_out + (c0 + c) * Dm) : make_float4(1.f, 1.f, 1.f, 1.f);
            const float4 y = make_float4(acc[c][0].x * r * g.x, acc[c][0].y * r * g.y, acc[c][1].x * r * g.z,
                                         acc[c][1].y * r * g.w);
            narrow(reinterpret_cast<Q*>(out + static_cast<long long>(c0 + c) * rows * Dm), y);
          }
      }
    }
  }
}

// ------------------------------------------------------------------------------------------- pool_mix, BF16
// The mixing of one token row is a (channels x sources) by (sources x hidden) product whose left operand changes
// with every row, so it cannot share an operand tile across rows the way tcgen05 wants; it is small enough for the
// warp-level tensor-core instruction instead (mma.sync m16n8k16, BF16 in, FP32 out): sixteen columns of the row are
// the M side, eight channels the N side, the sources the contraction (two steps of 16), and every warp sweeps 64
// columns of the row as four such tiles per side.  Against the FP32 kernel above this removes the 2*channels FMAs
// per loaded element from the FP32 pipe, which bounded that kernel at a sixth of HBM bandwidth.
//
// A block of hidden/64 warps stays resident (one per SM) and walks over the rows.  The gain tables live in shared
// memory in BF16; the next row's sources, and the rows of the routing partials that belong to it, arrive by bulk
// copies (cp.async.bulk, completion on an mbarrier) while the current row is mixed.  Rows of the tables and of the source tile are 16 bytes longer than the data so
// that the four source rows a quarter-warp reads at once fall into different banks.
//
// Thread (g = lane/4, q = lane%4) of warp w holds, as the A fragments want them, columns 64w+8g .. +8 of the eight
// sources 2q, 2q+1, 2q+8, 2q+9, 2q+16, 2q+17, 2q+24, 2q+25 (tile j of the warp takes the thread's columns 2j and
// 2j+1 as its rows g and g+8), and receives, as the accumulator fragments come, the same eight columns of channels
// 2q and 2q+1.
constexpr int kMmaSources = 32;
constexpr int kMmaWarps = 16;  // at most: hidden <= 1024
constexpr int kCoefPitch = 20;  // words per channel row of the coefficient tile (16 used): conflict-free fragments

struct MmaLayout {
  int pitch;  // bytes per row of the tables and of the source tile
  size_t tables, tile, coef, bias, red, inv, sums, part, bar, total;
  // `routed` > 0 reserves two buffers for the routing partials of a row (both sides, `routed` sources each)
  __host__ __device__ MmaLayout(int sources, int channels, int hidden, int warps, int routed = 0) {
    const int padded = (channels + kChannelsPerPass - 1) / kChannelsPerPass * kChannelsPerPass;
    pitch = hidden * 2 + 16;
    tables = 0;
    tile = tables + static_cast<size_t>(2) * (sources + channels) * pitch;
    coef = tile + static_cast<size_t>(sources) * pitch;
    bias = coef + static_cast<size_t>(2) * padded * kCoefPitch * 4;
    red = bias + (static_cast<size_t>(2) * channels * sources * 4 + 15) / 16 * 16;
    inv = red + static_cast<size_t>(kMmaWarps) * kMmaSources * 4;
    sums = inv + kMmaSources * 4;
    part = (sums + static_cast<size_t>(2) * warps * 2 * kChannelsPerPass * 4 + 15) / 16 * 16;
    bar = part + static_cast<size_t>(2) * 2 * routed * channels * sources * 2;
    total = bar + 16;
  }
};

__device__ __forceinline__ uint32_t smem_address(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_address(dst)),
               "l"(src), "r"(bytes), "r"(smem_address(bar))
               : "memory");
}

// Bounded wait for a phase of the barrier: gives up after about a second.
__device__ __forceinline__ bool barrier_wait(uint64_t* bar, uint32_t parity) {
  for (uint32_t spin = 0; spin < (1u << 22); ++spin) {
    uint32_t done;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.b32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done)
        : "r"(smem_address(bar)), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}

__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}

// D (16 columns x 8 channels) += A (16 columns x 16 sources) * B (16 sources x 8 channels)
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

constexpr int kMixWaitCode = 240;  // status code of a source tile that never arrived

// kL / kC / kDm fix sources, channels and hidden at compile time (0: taken from the arguments).
template <int kL, int kC, int kDm>
__global__ void __launch_bounds__(512, 1) pool_mix_mma_kernel(const wm_pool_mix_args a, const long long rows, int* status, const int staged_partials) {
  extern __shared__ __align__(128) unsigned char raw[];
  const int L = kL ? kL : a.sources, C = kC ? kC : a.channels, Dm = kDm ? kDm : a.hidden;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, warps = blockDim.x >> 5;
  const int g = lane >> 2, q = lane & 3;
  const int CL = C * L;
  const long long PS = a.partial_row_stride ? a.partial_row_stride : CL;  // elements between rows of a partial
  const int Cpad = (C + kChannelsPerPass - 1) / kChannelsPerPass * kChannelsPerPass;
  const MmaLayout lay(L, C, Dm, warps, staged_partials ? a.n_routed : 0);
  const int pitch = lay.pitch;
  unsigned char* tables = raw + lay.tables;
  unsigned char* tile = raw + lay.tile;
  unsigned char* part_rooms = raw + lay.part;  // [row parity][side][routed source][channels * sources] bf16
  const size_t part_room = staged_partials ? static_cast<size_t>(2) * a.n_routed * CL * 2 : 0;
  uint32_t* coef = reinterpret_cast<uint32_t*>(raw + lay.coef);
  float* bias = reinterpret_cast<float*>(raw + lay.bias);
  float* red = reinterpret_cast<float*>(raw + lay.red);
  float* inv = reinterpret_cast<float*>(raw + lay.inv);
  float* sums = reinterpret_cast<float*>(raw + lay.sums);
  uint64_t* bar = reinterpret_cast<uint64_t*>(raw + lay.bar);
  const float inv_hidden = 1.f / static_cast<float>(Dm);
  using bf16 = __nv_bfloat16;
  const bool gained = a.gain_k != nullptr;

  {  // the gain tables, once per block: pre-mix K, pre-mix V, then (when given) post-mix K and V
    const float* from[4] = {a.pre_mix_k, a.pre_mix_v, a.gain_k, a.gain_v};
    const int table_rows[4] = {L, L, C, C};
    unsigned char* at = tables;
    const int quads = Dm / 4;
    for (int k = 0; k < (gained ? 4 : 2); ++k) {
      const float4* src = reinterpret_cast<const float4*>(from[k]);
#pragma unroll 8
      for (int i = tid; i < table_rows[k] * quads; i += blockDim.x) {
        const int r = i / quads, c = i - r * quads;
        const float4 v = __ldg(src + i);
        const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
        uint2 w;
        w.x = *reinterpret_cast<const unsigned*>(&lo);
        w.y = *reinterpret_cast<const unsigned*>(&hi);
        *reinterpret_cast<uint2*>(at + r * pitch + c * 8) = w;
      }
      at += table_rows[k] * pitch;
    }
  }
  for (int i = tid; i < 2 * CL; i += blockDim.x) bias[i] = i < CL ? a.bias_k[i] : a.bias_v[i - CL];
  for (int i = tid; i < kMmaWarps * kMmaSources; i += blockDim.x) red[i] = 0.f;
  const unsigned char* pre_tables = tables;
  const unsigned char* post_tables = tables + static_cast<size_t>(2) * L * pitch;
  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_address(bar)), "r"(1));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  const uint32_t tile_bytes = static_cast<uint32_t>(L) * Dm * 2 + static_cast<uint32_t>(part_room);
  // first warp: the row's sources into the tile, one bulk copy per source, and (dynamic router) its routing
  // partials into the room of the row's parity; `turn` counts the block's rows
  auto fetch = [&](long long row, int turn) {
    const long long b = row / a.tokens, t = row - b * a.tokens;
    const bf16* x0 = static_cast<const bf16*>(a.stacked) + b * a.stacked_strides[0] + t * a.stacked_strides[1];
    if (lane == 0)
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_address(bar)), "r"(tile_bytes) : "memory");
    __syncwarp();
    if (lane < L) bulk_load(tile + lane * pitch, x0 + lane * a.stacked_strides[2], Dm * 2, bar);
    if (staged_partials) {
      unsigned char* room = part_rooms + (turn & 1) * part_room;
      for (int i = lane; i < 2 * a.n_routed; i += 32) {
        const int side = i / a.n_routed, j = i - side * a.n_routed;
        const bf16* src = static_cast<const bf16*>(side ? a.partial_v : a.partial_k) + (j * rows + row) * PS;
        bulk_load(room + static_cast<size_t>(i) * CL * 2, src, CL * 2, bar);
      }
    }
  };
  if (warp == 0 && blockIdx.x < rows) fetch(blockIdx.x, 0);

  const int off = (64 * warp + 8 * g) * 2;  // byte offset of this thread's eight columns in a row
  uint32_t parity = 0;
  int turn = 0;
  for (long long row = blockIdx.x; row < rows; row += gridDim.x, ++turn) {
    const bool arrived = barrier_wait(bar, parity);
    parity ^= 1;
    if (!__syncthreads_and(arrived)) {
      // give the copies another bounded chance to land before the block's shared memory is released
      if (!arrived) barrier_wait(bar, parity ^ 1);
      if (tid == 0) atomicCAS(status, 0, kMixWaitCode | static_cast<int>((blockIdx.x & 0x7fffffu) << 8));
      return;
    }
    uint4 x[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int l = 2 * q + (i & 1) + 8 * (i >> 1);
      x[i] = l < L ? *reinterpret_cast<const uint4*>(tile + l * pitch + off) : make_uint4(0, 0, 0, 0);
    }
    // inverse RMS of every source: this thread's share of eight of them, summed over g, then over the warps
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int l = 2 * q + (i & 1) + 8 * (i >> 1);
      const unsigned w[4] = {x[i].x, x[i].y, x[i].z, x[i].w};
      float s = 0.f;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float lo = __uint_as_float(w[k] << 16), hi = __uint_as_float(w[k] & 0xffff0000u);
        s = fmaf(lo, lo, fmaf(hi, hi, s));
      }
      s += __shfl_xor_sync(0xffffffffu, s, 4);
      s += __shfl_xor_sync(0xffffffffu, s, 8);
      s += __shfl_xor_sync(0xffffffffu, s, 16);
      if (g == 0) red[l * kMmaWarps + warp] = s;
    }
    __syncthreads();  // the tile has been read by everyone: the next row may overwrite it
    const long long next = row + gridDim.x;
    if (next < rows) {
      if (warp == 0) fetch(next, turn + 1);
      if (a.partial_k != nullptr && !staged_partials) {  // the next row's routing partials into L2
        const int lines = (CL * 2 + 127) / 128;
        for (int i = tid - 32; i >= 0 && i < 2 * a.n_routed * lines; i += blockDim.x - 32) {
          const int side = i / (a.n_routed * lines), rem = i - side * a.n_routed * lines;
          const int j = rem / lines, line = rem - j * lines;
          const char* p = static_cast<const char*>(side ? a.partial_v : a.partial_k) + ((j * rows + next) * PS) * 2 + line * 128;
          asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
        }
      }
    }
    for (int i = tid; i < kMmaSources * kMmaWarps; i += blockDim.x) {  // sixteen lanes per source
      float s = red[i];
      s += __shfl_xor_sync(0xffffffffu, s, 8);
      s += __shfl_xor_sync(0xffffffffu, s, 4);
      s += __shfl_xor_sync(0xffffffffu, s, 2);
      s += __shfl_xor_sync(0xffffffffu, s, 1);
      if ((i & 15) == 0) inv[i >> 4] = rsqrtf(s * inv_hidden + a.source_eps);
    }
    __syncthreads();

    // coefficients of the raw, gained sources (routing logit times source norm) as the right operand: one word
    // holds two adjacent sources of a channel
    for (int i = tid; i < 2 * Cpad * 16; i += blockDim.x) {
      const int side = i / (Cpad * 16), rem = i - side * Cpad * 16;
      const int c = rem >> 4, word = rem & 15;
      float v[2] = {0.f, 0.f};
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int l = 2 * word + h;
        if (c < C && l < L) {
          const int o = c * L + l;
          float alpha = bias[side * CL + o];
          if (staged_partials) {
            const bf16* part = reinterpret_cast<const bf16*>(part_rooms + (turn & 1) * part_room) + static_cast<size_t>(side) * a.n_routed * CL + o;
            for (int j = 0; j < a.n_routed; ++j)
              alpha = fmaf(inv[a.route_start + j * a.route_stride], __bfloat162float(part[j * CL]), alpha);
          } else if (a.partial_k != nullptr) {
            const bf16* part = static_cast<const bf16*>(side ? a.partial_v : a.partial_k);
            for (int j = 0; j < a.n_routed; ++j)
              alpha = fmaf(inv[a.route_start + j * a.route_stride], __bfloat162float(part[(j * rows + row) * PS + o]), alpha);
          }
          v[h] = alpha * inv[l];
        }
      }
      const __nv_bfloat162 packed = __floats2bfloat162_rn(v[0], v[1]);
      coef[(side * Cpad + c) * kCoefPitch + word] = *reinterpret_cast<const uint32_t*>(&packed);
    }
    __syncthreads();

    int pass = 0;
    for (int c0 = 0; c0 < C; c0 += kChannelsPerPass, ++pass) {
      // acc[side][j][.]: columns 2j (.=0,1) and 2j+1 (.=2,3) of this thread's eight, channels c0+2q and c0+2q+1
      float acc[2][4][4];
#pragma unroll
      for (int side = 0; side < 2; ++side) {
        const unsigned char* pre = pre_tables + static_cast<size_t>(side) * L * pitch + off;
        const uint32_t* cb = coef + (side * Cpad + c0 + g) * kCoefPitch + q;
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[side][j][0] = acc[side][j][1] = acc[side][j][2] = acc[side][j][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < 2; ++ks) {
          const uint32_t b0 = cb[8 * ks], b1 = cb[8 * ks + 4];
          uint32_t p[4][4];
#pragma unroll
          for (int ii = 0; ii < 4; ++ii) {
            const int i = 4 * ks + ii;
            const int l = 2 * q + (i & 1) + 8 * (i >> 1);
            if (l < L) {
              const uint4 w = *reinterpret_cast<const uint4*>(pre + l * pitch);
              p[ii][0] = mul_bf16x2(x[i].x, w.x);
              p[ii][1] = mul_bf16x2(x[i].y, w.y);
              p[ii][2] = mul_bf16x2(x[i].z, w.z);
              p[ii][3] = mul_bf16x2(x[i].w, w.w);
            } else {
              p[ii][0] = p[ii][1] = p[ii][2] = p[ii][3] = 0u;
            }
          }
#pragma unroll
          for (int j = 0; j < 4; ++j)
            mma_16816(acc[side][j], __byte_perm(p[0][j], p[1][j], 0x5410u), __byte_perm(p[0][j], p[1][j], 0x7632u),
                      __byte_perm(p[2][j], p[3][j], 0x5410u), __byte_perm(p[2][j], p[3][j], 0x7632u), b0, b1);
        }
      }
      // sums of squares of the four (side, channel) rows this thread holds, over its eight columns, then over g
      float* slot = sums + (pass & 1) * warps * 2 * kChannelsPerPass;
#pragma unroll
      for (int side = 0; side < 2; ++side)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          float s = 0.f;
#pragma unroll
          for (int j = 0; j < 4; ++j) s = fmaf(acc[side][j][h], acc[side][j][h], fmaf(acc[side][j][2 + h], acc[side][j][2 + h], s));
          s += __shfl_xor_sync(0xffffffffu, s, 4);
          s += __shfl_xor_sync(0xffffffffu, s, 8);
          s += __shfl_xor_sync(0xffffffffu, s, 16);
          if (g == 0) slot[(warp * 2 + side) * kChannelsPerPass + 2 * q + h] = s;
        }
      __syncthreads();
#pragma unroll
      for (int side = 0; side < 2; ++side)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int c = c0 + 2 * q + h;
          // every lane sums two of the sixteen per-warp values of its (side, channel); lanes of one q differ in g
          float total = 0.f;
#pragma unroll
          for (int w = g; w < kMmaWarps; w += 8)
            if (w < warps) total += slot[(w * 2 + side) * kChannelsPerPass + 2 * q + h];
          total += __shfl_xor_sync(0xffffffffu, total, 4);
          total += __shfl_xor_sync(0xffffffffu, total, 8);
          total += __shfl_xor_sync(0xffffffffu, total, 16);
          if (c < C) {
            const float r = rsqrtf(total * inv_hidden + a.mix_eps);
            uint4 gw = make_uint4(0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u);  // ones
            if (gained) gw = *reinterpret_cast<const uint4*>(post_tables + (static_cast<size_t>(side) * C + c) * pitch + off);
            const unsigned gq[4] = {gw.x, gw.y, gw.z, gw.w};
            unsigned y[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float lo = acc[side][j][h] * r * __uint_as_float(gq[j] << 16);
              const float hi = acc[side][j][2 + h] * r * __uint_as_float(gq[j] & 0xffff0000u);
              const __nv_bfloat162 packed = __floats2bfloat162_rn(lo, hi);
              y[j] = *reinterpret_cast<const unsigned*>(&packed);
            }
            bf16* out = static_cast<bf16*>(side ? a.mixed_v : a.mixed_k) + (static_cast<long long>(c) * rows + row) * Dm + 64 * warp + 8 * g;
            *reinterpret_cast<uint4*>(out) = make_uint4(y[0], y[1], y[2], y[3]);
          }
        }
    }
  }
}

// ------------------------------------------------------------------------------------------------ pool_finish
template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&x)[8]);
template <>
__device__ __forceinline__ void load8<float>(const float* p, float (&x)[8]) {
  const float4 a = __ldcs(reinterpret_cast<const float4*>(p)), b = __ldcs(reinterpret_cast<const float4*>(p) + 1);
  x[0] = a.x, x[1] = a.y, x[2] = a.z, x[3] = a.w, x[4] = b.x, x[5] = b.y, x[6] = b.z, x[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&x)[8]) {
  const uint4 r = __ldcs(reinterpret_cast<const uint4*>(p));
  const unsigned w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    x[2 * i] = __uint_as_float(w[i] << 16);
    x[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
template <typename T>
__device__ __forceinline__ void store8(T* p, const float (&x)[8]);
template <>
__device__ __forceinline__ void store8<float>(float* p, const float (&x)[8]) {
  reinterpret_cast<float4*>(p)[0] = make_float4(x[0], x[1], x[2], x[3]);
  reinterpret_cast<float4*>(p)[1] = make_float4(x[4], x[5], x[6], x[7]);
}
template <>
__device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* p, const float (&x)[8]) {
  unsigned w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(x[2 * i], x[2 * i + 1]);
    w[i] = *reinterpret_cast<const unsigned*>(&h);
  }
  *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
}

constexpr int kFinishThreads = 256;  // 8 warps = 8 consecutive tokens: 1 KB contiguous per head on the pool side

// One warp owns one token row of one channel; a lane holds 8 adjacent elements, a head takes D/8 lanes, a warp
// 32/(D/8) heads at a time.  blockIdx.z picks keys (norm, gain, rotation) or values (move only).
template <typename TI, typename TO, int D>
__global__ void __launch_bounds__(kFinishThreads) pool_finish_kernel(const wm_pool_finish_args a) {
  constexpr int kLanes = D / 8;
  constexpr int kHeads = 32 / kLanes;
  const int lane = threadIdx.x & 31, sub = lane % kLanes, slot = lane / kLanes;
  const int t = blockIdx.x * (kFinishThreads / 32) + (threadIdx.x >> 5);
  if (t >= a.tokens) return;
  const int c = blockIdx.y % a.channels, b = blockIdx.y / a.channels;
  const bool keys = blockIdx.z == 0;
  const long long row = static_cast<long long>(b) * a.tokens + t;
  const long long rows = static_cast<long long>(a.batch) * a.tokens;
  const TI* in = static_cast<const TI*>(keys ? a.k_proj : a.v_proj) + (c * rows + row) * a.kv_heads * D + 8 * sub;
  TO* out = static_cast<TO*>(keys ? a.k_out : a.v_out) + b * a.out_strides[0] +
            (a.token_offset + static_cast<long long>(t) * (a.slot_stride ? a.slot_stride : 1)) * a.out_strides[2] + 8 * sub;
  float own[8], other[8];  // factor of this lane's elements, factor of the rotation partner's
  if (keys) {
    const long long cs = b * a.cs_strides[0] + static_cast<long long>(a.rope_offset + t) * a.cs_strides[1] + 8 * sub;
    const float sign = sub < kLanes / 2 ? -1.f : 1.f;  // rot(y)[d] = -y[d + D/2] in the first half
    const int partner = sub ^ (kLanes / 2);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      own[i] = a.k_norm_weight[c * D + 8 * sub + i] * a.cos[cs + i];
      other[i] = a.k_norm_weight[c * D + 8 * partner + i] * a.sin[cs + i] * sign;
    }
  }
  constexpr int kBatch = 4;  // warp passes whose loads are issued together
  for (int h0 = 0; h0 < a.kv_heads; h0 += kBatch * kHeads) {
    float x[kBatch][8];
#pragma unroll
    for (int i = 0; i < kBatch; ++i) {
      const int h = h0 + i * kHeads + slot;
      if (h < a.kv_heads) {
        load8<TI>(in + h * D, x[i]);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) x[i][e] = 0.f;
      }
    }
#pragma unroll
    for (int i = 0; i < kBatch; ++i) {
      const int h = h0 + i * kHeads + slot;
      if (h0 + i * kHeads >= a.kv_heads) break;  // warp-uniform: the shuffles below need every lane
      if (keys) {
        float ss = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) ss = fmaf(x[i][e], x[i][e], ss);
#pragma unroll
        for (int o = kLanes / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float r = rsqrtf(ss * (1.f / D) + a.eps);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float xp = __shfl_xor_sync(0xffffffffu, x[i][e], kLanes / 2);
          x[i][e] = r * fmaf(x[i][e], own[e], xp * other[e]);
        }
      }
      if (h < a.kv_heads) store8<TO>(out + static_cast<long long>(c * a.kv_heads + h) * a.out_strides[1], x[i]);
    }
  }
}

constexpr int kMaxDevices = 64;
constexpr size_t kSharedLimit = 227 * 1024;

template <typename T, int kL, bool kStaged>
int launch_mix_variant(const wm_pool_mix_args& a, unsigned grid, int threads, size_t shared, long long rows, cudaStream_t stream) {
  static std::atomic<bool> configured[kMaxDevices];
  if (shared > 48 * 1024) {
    int device = 0;
    WM_CUDA(cudaGetDevice(&device));
    if (device < 0 || device >= kMaxDevices || !configured[device].load(std::memory_order_acquire)) {
      WM_CUDA(cudaFuncSetAttribute(pool_mix_kernel<T, kL, kStaged>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   static_cast<int>(kSharedLimit)));
      if (device >= 0 && device < kMaxDevices) configured[device].store(true, std::memory_order_release);
    }
  }
  pool_mix_kernel<T, kL, kStaged><<<grid, threads, shared, stream>>>(a, rows);
  count_launch();
  return cuda_check(cudaGetLastError(), "pool_mix_kernel");
}

template <typename T, bool kStaged>
int launch_mix_sources(const wm_pool_mix_args& a, unsigned grid, int threads, size_t shared, long long rows, cudaStream_t stream) {
  if (a.sources <= 8) return launch_mix_variant<T, 8, kStaged>(a, grid, threads, shared, rows, stream);
  if (a.sources <= 16) return launch_mix_variant<T, 16, kStaged>(a, grid, threads, shared, rows, stream);
  if (a.sources <= 25) return launch_mix_variant<T, 25, kStaged>(a, grid, threads, shared, rows, stream);
  return launch_mix_variant<T, 32, kStaged>(a, grid, threads, shared, rows, stream);
}

// The tensor-core kernel takes BF16 stacks whose rows can travel as 16-byte aligned bulk copies and whose tables
// fit in shared memory beside one source tile.
bool mma_path(const wm_pool_mix_args& a) {
  if (a.dtype != WM_BF16 || a.hidden % 64 || a.hidden > 1024 || a.sources > kMmaSources) return false;
  if (reinterpret_cast<uintptr_t>(a.stacked) % 16 || reinterpret_cast<uintptr_t>(a.mixed_k) % 16 || reinterpret_cast<uintptr_t>(a.mixed_v) % 16) return false;
  for (int i = 0; i < 3; ++i)
    if (a.stacked_strides[i] % 8) return false;
  return MmaLayout(a.sources, a.channels, a.hidden, a.hidden / 64).total <= kSharedLimit;
}

template <typename T>
int launch_mix(const wm_pool_mix_args& a, cudaStream_t stream) {
  const long long rows = static_cast<long long>(a.batch) * a.tokens;
  const int group_threads = a.hidden / 4;
  const int groups = group_threads >= 512 ? 1 : 512 / group_threads > 8 ? 8 : 512 / group_threads;
  const int threads = groups * group_threads;
  const int padded = (a.channels + kChannelsPerPass - 1) / kChannelsPerPass * kChannelsPerPass;
  const MixLayout lay(group_threads / 32, a.sources, padded);
  const size_t scratch = static_cast<size_t>(groups) * lay.total * sizeof(float);
  const size_t tables = (static_cast<size_t>(2) * (a.sources + a.channels) * a.hidden * sizeof(T) + 15) / 16 * 16;
  const bool staged = sizeof(T) == 2 && tables + scratch <= kSharedLimit;
  const size_t shared = scratch + (staged ? tables : 0);
  if (shared > kSharedLimit) return fail(WM_EUNSUPPORTED, "wm_pool_mix: channels * sources too large for one block");
  int device = 0, sms = 0;
  WM_CUDA(cudaGetDevice(&device));
  WM_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
  if (mma_path(a)) {
    const int mma_warps = a.hidden / 64;
    // the routing partials of a row travel with its sources when their rows can be bulk-copied (16-byte multiples)
    const bool routed = a.partial_k != nullptr;
    const size_t partial_row = static_cast<size_t>(a.channels) * a.sources * 2;
    bool staged = routed && partial_row % 16 == 0 && (a.partial_row_stride * 2) % 16 == 0 &&
                  reinterpret_cast<uintptr_t>(a.partial_k) % 16 == 0 && reinterpret_cast<uintptr_t>(a.partial_v) % 16 == 0;
    if (staged && MmaLayout(a.sources, a.channels, a.hidden, mma_warps, a.n_routed).total > kSharedLimit) staged = false;
    const MmaLayout mma(a.sources, a.channels, a.hidden, mma_warps, staged ? a.n_routed : 0);
    static std::atomic<bool> configured[kMaxDevices];
    if (device < 0 || device >= kMaxDevices || !configured[device].load(std::memory_order_acquire)) {
      WM_CUDA(cudaFuncSetAttribute(pool_mix_mma_kernel<0, 0, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kSharedLimit)));
      WM_CUDA(cudaFuncSetAttribute(pool_mix_mma_kernel<25, 8, 1024>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kSharedLimit)));
      if (device >= 0 && device < kMaxDevices) configured[device].store(true, std::memory_order_release);
    }
    int* status = nullptr;
    const int got = tc_status_word(&status);
    if (got != WM_OK) return got;
    const unsigned blocks_mma = static_cast<unsigned>(rows < sms ? rows : sms);
    if (a.sources == 25 && a.channels == 8 && a.hidden == 1024)  // the pool of the 24-layer model
      pool_mix_mma_kernel<25, 8, 1024><<<blocks_mma, mma_warps * 32, mma.total, stream>>>(a, rows, status, staged ? 1 : 0);
    else
      pool_mix_mma_kernel<0, 0, 0><<<blocks_mma, mma_warps * 32, mma.total, stream>>>(a, rows, status, staged ? 1 : 0);
    count_launch();
    return cuda_check(cudaGetLastError(), "pool_mix_mma_kernel");
  }
  const long long blocks = (rows + groups - 1) / groups;
  const unsigned grid = static_cast<unsigned>(blocks < sms ? blocks : sms);  // resident blocks walking over the rows
  return staged ? launch_mix_sources<T, true>(a, grid, threads, shared, rows, stream)
                : launch_mix_sources<T, false>(a, grid, threads, shared, rows, stream);
}

template <typename TI, typename TO>
int launch_finish(const wm_pool_finish_args& a, cudaStream_t stream) {
  const dim3 grid((a.tokens + kFinishThreads / 32 - 1) / (kFinishThreads / 32), a.batch * a.channels, 2);
  if (a.head_dim == 64)
    pool_finish_kernel<TI, TO, 64><<<grid, kFinishThreads, 0, stream>>>(a);
  else
    pool_finish_kernel<TI, TO, 128><<<grid, kFinishThreads, 0, stream>>>(a);
  count_launch();
  return cuda_check(cudaGetLastError(), "pool_finish_kernel");
}

bool aligned16(const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; }

}  // namespace

int pool_mix_launch(const wm_pool_mix_args& a, cudaStream_t stream) {
  if (!a.stacked || !a.pre_mix_k || !a.pre_mix_v || !a.bias_k || !a.bias_v || !a.mixed_k || !a.mixed_v)
    return fail(WM_EINVAL, "wm_pool_mix: stacked, pre-mix gains, biases and results are required");
  if ((a.gain_k == nullptr) != (a.gain_v == nullptr)) return fail(WM_EINVAL, "wm_pool_mix: gain_k and gain_v come together");
  if (a.dtype != WM_F32 && a.dtype != WM_BF16) return fail(WM_EINVAL, "wm_pool_mix: dtype must be WM_F32 or WM_BF16");
  if (a.batch < 1 || a.tokens < 1 || a.sources < 1 || a.channels < 1 || a.hidden < 1)
    return fail(WM_EINVAL, "wm_pool_mix: sizes must be positive");
  if (a.hidden % 128 || a.hidden > 2048) return fail(WM_EUNSUPPORTED, "wm_pool_mix: hidden must be a multiple of 128, at most 2048");
  if (a.sources > 32) return fail(WM_EUNSUPPORTED, "wm_pool_mix: at most 32 sources");
  const bool routed = a.partial_k != nullptr || a.partial_v != nullptr;
  if (routed) {
    if (!a.partial_k || !a.partial_v) return fail(WM_EINVAL, "wm_pool_mix: partial_k and partial_v come together");
    if (a.partial_row_stride != 0 && a.partial_row_stride < static_cast<long long>(a.channels) * a.sources)
      return fail(WM_EINVAL, "wm_pool_mix: partial_row_stride is shorter than a row");
    if (a.n_routed < 1 || a.route_stride < 1 || a.route_start < 0 || a.route_start + (a.n_routed - 1) * a.route_stride >= a.sources)
      return fail(WM_EINVAL, "wm_pool_mix: routed sources must lie inside the stack");
  }
  const int esize = a.dtype == WM_F32 ? 4 : 2;
  const int quad = 4 * esize;  // bytes of one access
  if (reinterpret_cast<uintptr_t>(a.stacked) % quad || reinterpret_cast<uintptr_t>(a.mixed_k) % quad ||
      reinterpret_cast<uintptr_t>(a.mixed_v) % quad)
    return fail(WM_EUNSUPPORTED, "wm_pool_mix: rows must be aligned to four elements");
  for (int i = 0; i < 3; ++i)
    if (a.stacked_strides[i] % 4) return fail(WM_EUNSUPPORTED, "wm_pool_mix: rows must be aligned to four elements");
  if (!aligned16(a.pre_mix_k) || !aligned16(a.pre_mix_v) || (a.gain_k && (!aligned16(a.gain_k) || !aligned16(a.gain_v))))
    return fail(WM_EUNSUPPORTED, "wm_pool_mix: gains must be 16-byte aligned");
  return a.dtype == WM_F32 ? launch_mix<float>(a, stream) : launch_mix<__nv_bfloat16>(a, stream);
}

int pool_finish_launch(const wm_pool_finish_args& a, cudaStream_t stream) {
  if (!a.k_proj || !a.v_proj || !a.k_norm_weight || !a.cos || !a.sin || !a.k_out || !a.v_out)
    return fail(WM_EINVAL, "wm_pool_finish: projections, norm weight, cos, sin and results are required");
  if ((a.in_dtype != WM_F32 && a.in_dtype != WM_BF16) || (a.out_dtype != WM_F32 && a.out_dtype != WM_BF16))
    return fail(WM_EINVAL, "wm_pool_finish: dtypes must be WM_F32 or WM_BF16");
  if (a.in_dtype == WM_BF16 && a.out_dtype == WM_F32) return fail(WM_EUNSUPPORTED, "wm_pool_finish: bfloat16 projections give a bfloat16 pool");
  if (a.batch < 1 || a.tokens < 1 || a.channels < 1 || a.kv_heads < 1) return fail(WM_EINVAL, "wm_pool_finish: sizes must be positive");
  if (a.head_dim != 64 && a.head_dim != 128) return fail(WM_EUNSUPPORTED, "wm_pool_finish: head_dim must be 64 or 128");
  if (a.token_offset < 0 || a.rope_offset < 0 || a.slot_stride < 0) return fail(WM_EINVAL, "wm_pool_finish: offsets and the slot stride must not be negative");
  if (static_cast<long long>(a.batch) * a.channels > 65535) return fail(WM_EUNSUPPORTED, "wm_pool_finish: batch * channels above 65535");
  const int osize = a.out_dtype == WM_F32 ? 4 : 2;
  if (!aligned16(a.k_proj) || !aligned16(a.v_proj) || !aligned16(a.k_out) || !aligned16(a.v_out))
    return fail(WM_EUNSUPPORTED, "wm_pool_finish: rows must be 16-byte aligned");
  for (int i = 0; i < 3; ++i)
    if ((a.out_strides[i] * osize) % 16) return fail(WM_EUNSUPPORTED, "wm_pool_finish: rows must be 16-byte aligned");
  if (a.in_dtype == WM_F32) {
    return a.out_dtype == WM_F32 ? launch_finish<float, float>(a, stream) : launch_finish<float, __nv_bfloat16>(a, stream);
  }
  return launch_finish<__nv_bfloat16, __nv_bfloat16>(a, stream);
}

}  // namespace wm
