// KV-pool projection path either side of its per-channel GEMMs.
//
// pool_mix: for one token row, the `sources` layer inputs are normalised, gained, mixed into `channels` vectors
// per side (K, V) with signed routing logits, normalised again and gained -- everything the pool does between the
// layer stack and the projection GEMMs, in one pass: the row's sources are read from HBM once into registers (four
// adjacent columns of every source per thread), the source norms and the routing logits are formed in shared
// memory, and the 2*channels mixtures leave as the rows of the GEMM's A operand.  Algorithmic bytes per token row:
// sources*hidden*sizeof(T) read + 2*channels*hidden*sizeof(T) written (+ the routing partials when the router is
// dynamic); bound by HBM bandwidth, with 2*sources*channels FMAs per loaded element as the second limit, which is
// why the mixing runs on the packed two-wide FP32 FMA.
//
// pool_finish: the projected channels get the per-channel key norm, the rotary embedding and the move into the
// pool's (batch, channel*head, slot, dim) layout; values only move.  One read and one write of K and V.
#include <math.h>

#include "common.cuh"

namespace wm {
namespace {

constexpr int kChannelsPerPass = 8;
constexpr int kMaxWarps = 16;

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

// Shared memory of pool_mix, in floats: per-warp partial sums of squares, the sources' inverse norms, the
// per-token mixing coefficients (side, source, channel) and two alternating buffers of per-warp channel sums.
struct MixLayout {
  int red, inv, coef, chan, total;
  __host__ __device__ MixLayout(int warps, int sources, int padded_channels) {
    red = 0;
    inv = red + ((warps * sources + 3) & ~3);
    coef = inv + ((sources + 3) & ~3);
    chan = coef + 2 * sources * padded_channels;
    total = chan + 2 * warps * kChannelsPerPass;
  }
};

template <typename T, int kL>
__global__ void __launch_bounds__(512) pool_mix_kernel(const wm_pool_mix_args a, const long long rows) {
  using Q = typename Quad<T>::type;
  extern __shared__ __align__(16) float sm[];
  const int L = a.sources, C = a.channels, Dm = a.hidden;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, warps = blockDim.x >> 5;
  const int col = tid * 4;
  const int CL = C * L;
  const int Cpad = (C + kChannelsPerPass - 1) / kChannelsPerPass * kChannelsPerPass;
  const MixLayout lay(warps, L, Cpad);
  float* red = sm + lay.red;
  float* inv = sm + lay.inv;
  float* coef = sm + lay.coef;
  float* chan = sm + lay.chan;
  const float inv_hidden = 1.f / static_cast<float>(Dm);

  // channels beyond `channels` in the last pass of eight mix with zero coefficients and are never stored
  for (int i = tid; i < 2 * L * Cpad; i += blockDim.x) coef[i] = 0.f;

  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const long long b = row / a.tokens, t = row - b * a.tokens;
    const T* x0 = static_cast<const T*>(a.stacked) + b * a.stacked_strides[0] + t * a.stacked_strides[1] + col;
    Q x[kL];
#pragma unroll
    for (int l = 0; l < kL; ++l)
      if (l < L) x[l] = __ldcs(reinterpret_cast<const Q*>(x0 + l * a.stacked_strides[2]));

    // inverse RMS of every source
#pragma unroll
    for (int l = 0; l < kL; ++l)
      if (l < L) {
        const float4 v = widen(x[l]);
        const float s = warp_sum(fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, v.w * v.w))));
        if (lane == 0) red[warp * L + l] = s;
      }
    __syncthreads();
    if (tid < L) {
      float s = 0.f;
      for (int w = 0; w < warps; ++w) s += red[w * L + tid];
      inv[tid] = rsqrtf(s * inv_hidden + a.source_eps);
    }
    __syncthreads();

    // routing logits of this token times the source norms: the coefficient of the raw, gained source
    for (int i = tid; i < 2 * CL; i += blockDim.x) {
      const int side = i >= CL;
      const int o = i - side * CL;
      const int c = o / L, l = o - c * L;
      float alpha = (side ? a.bias_v : a.bias_k)[o];
      const T* part = static_cast<const T*>(side ? a.partial_v : a.partial_k);
      if (part != nullptr)
        for (int j = 0; j < a.n_routed; ++j)
          alpha = fmaf(inv[a.route_start + j * a.route_stride], to_float(part[(j * rows + row) * CL + o]), alpha);
      coef[(side * L + l) * Cpad + c] = alpha * inv[l];
    }
    __syncthreads();

    int pass = 0;
    for (int c0 = 0; c0 < C; c0 += kChannelsPerPass) {
#pragma unroll 1
      for (int side = 0; side < 2; ++side, ++pass) {
        const float* gain_in = (side ? a.pre_mix_v : a.pre_mix_k) + col;
        const float* cf = coef + side * L * Cpad + c0;
        float2 acc[kChannelsPerPass][2];
#pragma unroll
        for (int c = 0; c < kChannelsPerPass; ++c) acc[c][0] = acc[c][1] = make_float2(0.f, 0.f);
#pragma unroll
        for (int l = 0; l < kL; ++l)
          if (l < L) {
            const float4 v = widen(x[l]);
            const float4 g = __ldg(reinterpret_cast<const float4*>(gain_in + l * Dm));
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
        __syncthreads();
        const float* gain_out = (side ? a.gain_v : a.gain_k) + col;
        T* out = static_cast<T*>(side ? a.mixed_v : a.mixed_k) + row * Dm + col;
#pragma unroll
        for (int c = 0; c < kChannelsPerPass; ++c)
          if (c0 + c < C) {
            float s = 0.f;
            for (int w = 0; w < warps; ++w) s += sums[w * kChannelsPerPass + c];
            const float r = rsqrtf(s * inv_hidden + a.mix_eps);
            const float4 g = __ldg(reinterpret_cast<const float4*>(gain_out + (c0 + c) * Dm));
            const float4 y = make_float4(acc[c][0].x * r * g.x, acc[c][0].y * r * g.y, acc[c][1].x * r * g.z,
                                         acc[c][1].y * r * g.w);
            narrow(reinterpret_cast<Q*>(out + static_cast<long long>(c0 + c) * rows * Dm), y);
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
            static_cast<long long>(a.token_offset + t) * a.out_strides[2] + 8 * sub;
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
  for (int h0 = 0; h0 < a.kv_heads; h0 += kHeads) {
    const int h = h0 + slot;
    const bool live = h < a.kv_heads;
    float x[8];
    if (live) {
      load8<TI>(in + h * D, x);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) x[i] = 0.f;
    }
    if (keys) {
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) ss = fmaf(x[i], x[i], ss);
#pragma unroll
      for (int o = kLanes / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      const float r = rsqrtf(ss * (1.f / D) + a.eps);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float xp = __shfl_xor_sync(0xffffffffu, x[i], kLanes / 2);
        x[i] = r * fmaf(x[i], own[i], xp * other[i]);
      }
    }
    if (live) store8<TO>(out + static_cast<long long>(c * a.kv_heads + h) * a.out_strides[1], x);
  }
}

template <typename T>
int launch_mix(const wm_pool_mix_args& a, cudaStream_t stream) {
  const long long rows = static_cast<long long>(a.batch) * a.tokens;
  const int threads = a.hidden / 4;
  const int padded = (a.channels + kChannelsPerPass - 1) / kChannelsPerPass * kChannelsPerPass;
  const MixLayout lay(threads / 32, a.sources, padded);
  const size_t shared = static_cast<size_t>(lay.total) * sizeof(float);
  if (shared > 48 * 1024) return fail(WM_EUNSUPPORTED, "wm_pool_mix: channels * sources too large for one block");
  int device = 0, sms = 0;
  WM_CUDA(cudaGetDevice(&device));
  WM_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
  // persistent blocks, two per SM at 256 threads: one loads its row while the other mixes
  const int per_sm = threads <= 256 ? 2 : 1;
  const unsigned grid = static_cast<unsigned>(rows < static_cast<long long>(sms) * per_sm ? rows : sms * per_sm);
  auto kernel = a.sources <= 8    ? pool_mix_kernel<T, 8>
                : a.sources <= 16 ? pool_mix_kernel<T, 16>
                : a.sources <= 25 ? pool_mix_kernel<T, 25>
                                  : pool_mix_kernel<T, 32>;
  kernel<<<grid, threads, shared, stream>>>(a, rows);
  count_launch();
  return cuda_check(cudaGetLastError(), "pool_mix_kernel");
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
  if (!a.stacked || !a.pre_mix_k || !a.pre_mix_v || !a.bias_k || !a.bias_v || !a.gain_k || !a.gain_v || !a.mixed_k || !a.mixed_v)
    return fail(WM_EINVAL, "wm_pool_mix: stacked, gains, biases and results are required");
  if (a.dtype != WM_F32 && a.dtype != WM_BF16) return fail(WM_EINVAL, "wm_pool_mix: dtype must be WM_F32 or WM_BF16");
  if (a.batch < 1 || a.tokens < 1 || a.sources < 1 || a.channels < 1 || a.hidden < 1)
    return fail(WM_EINVAL, "wm_pool_mix: sizes must be positive");
  if (a.hidden % 128 || a.hidden > 2048) return fail(WM_EUNSUPPORTED, "wm_pool_mix: hidden must be a multiple of 128, at most 2048");
  if (a.sources > 32) return fail(WM_EUNSUPPORTED, "wm_pool_mix: at most 32 sources");
  const bool routed = a.partial_k != nullptr || a.partial_v != nullptr;
  if (routed) {
    if (!a.partial_k || !a.partial_v) return fail(WM_EINVAL, "wm_pool_mix: partial_k and partial_v come together");
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
  if (!aligned16(a.pre_mix_k) || !aligned16(a.pre_mix_v) || !aligned16(a.gain_k) || !aligned16(a.gain_v))
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
  if (a.token_offset < 0 || a.rope_offset < 0) return fail(WM_EINVAL, "wm_pool_finish: offsets must not be negative");
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
