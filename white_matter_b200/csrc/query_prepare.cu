// Query preparation of the attention layer: per-head RMS normalisation with a learned gain, the rotary position
// embedding, and the move from the projection's (batch, token, head, dim) layout into the (batch, head, token, dim)
// layout the attention kernels read -- one pass over the projected queries instead of the reference's norm,
// transpose, two multiplies, rotate_half concatenation, add and dtype cast.  Pure streaming work bound by HBM
// bandwidth: forward reads x once and writes q once (cos/sin are shared by the heads of a token and stay in
// registers); backward reads dq and x once and writes dx once.
//
//   n = x * rsqrt(mean_d(x^2) + eps)        y = n * weight
//   q[d] = y[d] * cos[d] + rot(y)[d] * sin[d],   rot(y)[d] = -y[d + D/2] (d < D/2),  y[d - D/2] (d >= D/2)
//
// One warp owns one token of one batch row and walks over its heads; a lane holds two adjacent elements of
// every 64-element group, so the rotation partner (D/2 away) is the same register pair of lane (l ^ 16) for D=64
// and of the same lane's other group for D=128.
#include <math.h>

#include "common.cuh"

namespace wm {
namespace {

constexpr int kThreads = 256;  // 8 warps = 8 consecutive tokens per block: 1 KB contiguous per head on the q side

template <typename T>
__device__ __forceinline__ float2 load2(const T* p);
template <>
__device__ __forceinline__ float2 load2<float>(const float* p) {
  return *reinterpret_cast<const float2*>(p);
}
template <>
__device__ __forceinline__ float2 load2<__nv_bfloat16>(const __nv_bfloat16* p) {
  const unsigned w = *reinterpret_cast<const unsigned*>(p);
  return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}
template <typename T>
__device__ __forceinline__ void store2(T* p, float2 v);
template <>
__device__ __forceinline__ void store2<float>(float* p, float2 v) {
  *reinterpret_cast<float2*>(p) = v;
}
template <>
__device__ __forceinline__ void store2<__nv_bfloat16>(__nv_bfloat16* p, float2 v) {
  *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(v.x, v.y);
}

// the pair D/2 elements away from this lane's pair of group g (G = D / 64 groups of 64 elements)
template <int G>
__device__ __forceinline__ float2 partner(const float2 (&v)[G], int g) {
  if (G == 1) {
    return make_float2(__shfl_xor_sync(0xffffffffu, v[0].x, 16), __shfl_xor_sync(0xffffffffu, v[0].y, 16));
  }
  return v[g ^ 1];
}

// first half of the head (the partner enters with a minus sign in the forward rotation)?
template <int G>
__device__ __forceinline__ bool low_half(int lane, int g) {
  return G == 1 ? lane < 16 : g == 0;
}

// Forward for bf16 input and output: a lane holds 8 adjacent elements (one 16-byte access), a head takes D/8 lanes
// and a warp 32/(D/8) heads of its token at a time; the rotary partner is the lane D/16 further on.  Four times
// fewer memory instructions and shuffles per element than the two-element mapping below, which it replaces
// whenever the strides allow 16-byte accesses (the kernel is bound by instruction issue otherwise).
template <int D>
__global__ void __launch_bounds__(kThreads) query_prepare_fwd_bf16_kernel(const wm_qprep_args a) {
  constexpr int kLanes = D / 8;        // lanes per head
  constexpr int kHeads = 32 / kLanes;  // heads per warp pass
  const int lane = threadIdx.x & 31;
  const int sub = lane % kLanes, slot = lane / kLanes;
  const int t = blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
  const int b = blockIdx.y;
  if (t >= a.tokens) return;
  auto unpack8 = [](const uint4& r, float (&x)[8]) {
    const unsigned w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      x[2 * i] = __uint_as_float(w[i] << 16);
      x[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  };
  const __nv_bfloat16* cs = static_cast<const __nv_bfloat16*>(a.cos) + b * a.cs_strides[0] + static_cast<long long>(t) * a.cs_strides[1];
  const __nv_bfloat16* sn = static_cast<const __nv_bfloat16*>(a.sin) + b * a.cs_strides[0] + static_cast<long long>(t) * a.cs_strides[1];
  const __nv_bfloat16* wt = static_cast<const __nv_bfloat16*>(a.weight);
  const int partner_sub = sub ^ (kLanes / 2);
  float c[8], s[8], w[8], wp[8];
  unpack8(*reinterpret_cast<const uint4*>(cs + 8 * sub), c);
  unpack8(*reinterpret_cast<const uint4*>(sn + 8 * sub), s);
  unpack8(*reinterpret_cast<const uint4*>(wt + 8 * sub), w);
  unpack8(*reinterpret_cast<const uint4*>(wt + 8 * partner_sub), wp);
  const float sign = sub < kLanes / 2 ? -1.f : 1.f;  // rot(y)[d] = -y[d + D/2] in the first half
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    s[i] *= sign;
    wp[i] *= s[i];  // partner gain and (signed) sine in one factor
    w[i] *= c[i];   // own gain and cosine in one factor
  }
  const __nv_bfloat16* x_tok = static_cast<const __nv_bfloat16*>(a.x) + b * a.x_strides[0] + static_cast<long long>(t) * a.x_strides[1];
  __nv_bfloat16* q_tok = static_cast<__nv_bfloat16*>(a.q) + (static_cast<long long>(b) * a.heads * a.tokens + t) * D;
  constexpr int kBatch = 2;  // warp passes whose loads are issued together
  for (int h0 = 0; h0 < a.heads; h0 += kBatch * kHeads) {
    uint4 raw[kBatch];
#pragma unroll
    for (int i = 0; i < kBatch; ++i) {
      const int h = h0 + i * kHeads + slot;
      raw[i] = h < a.heads ? *reinterpret_cast<const uint4*>(x_tok + h * a.x_strides[2] + 8 * sub) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int i = 0; i < kBatch; ++i) {
      const int h = h0 + i * kHeads + slot;
      float x[8], xp[8];
      unpack8(raw[i], x);
      float ss = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) ss = fmaf(x[e], x[e], ss);
#pragma unroll
      for (int o = kLanes / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      const float r = rsqrtf(ss * (1.f / D) + a.eps);
      uint4 other;
      other.x = __shfl_xor_sync(0xffffffffu, raw[i].x, kLanes / 2);
      other.y = __shfl_xor_sync(0xffffffffu, raw[i].y, kLanes / 2);
      other.z = __shfl_xor_sync(0xffffffffu, raw[i].z, kLanes / 2);
      other.w = __shfl_xor_sync(0xffffffffu, raw[i].w, kLanes / 2);
      unpack8(other, xp);
      unsigned out[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float lo = r * fmaf(x[2 * e], w[2 * e], xp[2 * e] * wp[2 * e]);
        const float hi = r * fmaf(x[2 * e + 1], w[2 * e + 1], xp[2 * e + 1] * wp[2 * e + 1]);
        __nv_bfloat162 pk = __floats2bfloat162_rn(lo, hi);
        out[e] = *reinterpret_cast<unsigned*>(&pk);
      }
      if (h < a.heads)
        *reinterpret_cast<uint4*>(q_tok + static_cast<long long>(h) * a.tokens * D + 8 * sub) = make_uint4(out[0], out[1], out[2], out[3]);
    }
  }
}

template <typename TX, typename TQ, int G>
__global__ void __launch_bounds__(kThreads) query_prepare_fwd_kernel(const wm_qprep_args a) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
  const int b = blockIdx.y;
  if (t >= a.tokens) return;
  const TX* cos_row = static_cast<const TX*>(a.cos) + b * a.cs_strides[0] + static_cast<long long>(t) * a.cs_strides[1];
  const TX* sin_row = static_cast<const TX*>(a.sin) + b * a.cs_strides[0] + static_cast<long long>(t) * a.cs_strides[1];
  const TX* weight = static_cast<const TX*>(a.weight);
  float2 c[G], s[G], w[G];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const int d = 64 * g + 2 * lane;
    c[g] = load2(cos_row + d);
    s[g] = load2(sin_row + d);
    w[g] = load2(weight + d);
    if (low_half<G>(lane, g)) s[g] = make_float2(-s[g].x, -s[g].y);  // sign of the rotation folded into sin
  }
  const float inv_d = 1.f / (64 * G);
  const TX* x_tok = static_cast<const TX*>(a.x) + b * a.x_strides[0] + static_cast<long long>(t) * a.x_strides[1];
  TQ* q_tok = static_cast<TQ*>(a.q) + (static_cast<long long>(b) * a.heads * a.tokens + t) * (64 * G);
  // kBatch heads at a time: their loads are issued together so that enough bytes are in flight per warp
  constexpr int kBatch = 4;
  for (int h0 = 0; h0 < a.heads; h0 += kBatch) {
    float2 x[kBatch][G];
#pragma unroll
    for (int i = 0; i < kBatch; ++i) {
#pragma unroll
      for (int g = 0; g < G; ++g)
        x[i][g] = h0 + i < a.heads ? load2(x_tok + (h0 + i) * a.x_strides[2] + 64 * g + 2 * lane) : make_float2(0.f, 0.f);
    }
#pragma unroll
    for (int i = 0; i < kBatch; ++i) {
      if (h0 + i >= a.heads) break;
      float ss = 0.f;
#pragma unroll
      for (int g = 0; g < G; ++g) ss = fmaf(x[i][g].x, x[i][g].x, fmaf(x[i][g].y, x[i][g].y, ss));
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      const float r = rsqrtf(ss * inv_d + a.eps);
      float2 y[G];
#pragma unroll
      for (int g = 0; g < G; ++g) y[g] = make_float2(x[i][g].x * r * w[g].x, x[i][g].y * r * w[g].y);
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float2 p = partner<G>(y, g);
        store2(q_tok + static_cast<long long>(h0 + i) * a.tokens * (64 * G) + 64 * g + 2 * lane,
               make_float2(fmaf(y[g].x, c[g].x, p.x * s[g].x), fmaf(y[g].y, c[g].y, p.y * s[g].y)));
      }
    }
  }
}

// dy[d] = dq[d] cos[d] + rot^T(dq * sin)[d];  dweight += dy * n;  dn = dy * weight;  dx = r (dn - n mean(dn n))
template <typename TX, typename TQ, int G>
__global__ void __launch_bounds__(kThreads) query_prepare_bwd_kernel(const wm_qprep_args a, float* partials) {
  __shared__ float block_dw[kThreads / 32][64 * G];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x * (kThreads / 32) + warp;
  const int b = blockIdx.y;
  float2 dw[G];
#pragma unroll
  for (int g = 0; g < G; ++g) dw[g] = make_float2(0.f, 0.f);
  if (t < a.tokens) {
    const TX* cos_row = static_cast<const TX*>(a.cos) + b * a.cs_strides[0] + static_cast<long long>(t) * a.cs_strides[1];
    const TX* sin_row = static_cast<const TX*>(a.sin) + b * a.cs_strides[0] + static_cast<long long>(t) * a.cs_strides[1];
    const TX* weight = static_cast<const TX*>(a.weight);
    float2 c[G], s[G], w[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const int d = 64 * g + 2 * lane;
      c[g] = load2(cos_row + d);
      s[g] = load2(sin_row + d);
      w[g] = load2(weight + d);
    }
    const float inv_d = 1.f / (64 * G);
    const TX* x_tok = static_cast<const TX*>(a.x) + b * a.x_strides[0] + static_cast<long long>(t) * a.x_strides[1];
    TX* dx_tok = static_cast<TX*>(a.dx) + b * a.x_strides[0] + static_cast<long long>(t) * a.x_strides[1];
    const TQ* dq_tok = static_cast<const TQ*>(a.dq) + (static_cast<long long>(b) * a.heads * a.tokens + t) * (64 * G);
    constexpr int kBatch = 2;  // heads whose loads are issued together
    for (int h0 = 0; h0 < a.heads; h0 += kBatch) {
      float2 xs[kBatch][G], dqs[kBatch][G];
#pragma unroll
      for (int i = 0; i < kBatch; ++i) {
#pragma unroll
        for (int g = 0; g < G; ++g) {
          const bool in = h0 + i < a.heads;
          xs[i][g] = in ? load2(x_tok + (h0 + i) * a.x_strides[2] + 64 * g + 2 * lane) : make_float2(0.f, 0.f);
          dqs[i][g] = in ? load2(dq_tok + static_cast<long long>(h0 + i) * a.tokens * (64 * G) + 64 * g + 2 * lane)
                         : make_float2(0.f, 0.f);
        }
      }
#pragma unroll
      for (int i = 0; i < kBatch; ++i) {
        if (h0 + i >= a.heads) break;
        const int h = h0 + i;
        float2 u[G], dy[G];  // u = dq * sin, whose partner enters dy
        float ss = 0.f;
#pragma unroll
        for (int g = 0; g < G; ++g) {
          ss = fmaf(xs[i][g].x, xs[i][g].x, fmaf(xs[i][g].y, xs[i][g].y, ss));
          dy[g] = make_float2(dqs[i][g].x * c[g].x, dqs[i][g].y * c[g].y);
          u[g] = make_float2(dqs[i][g].x * s[g].x, dqs[i][g].y * s[g].y);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float r = rsqrtf(ss * inv_d + a.eps);
        float dot = 0.f;
        float2 n[G], dn[G];
#pragma unroll
        for (int g = 0; g < G; ++g) {
          // q[d + D/2] = ... + y[d] sin[d + D/2]  and  q[d - D/2] = ... - y[d] sin[d - D/2]
          const float2 p = partner<G>(u, g);
          const float sign = low_half<G>(lane, g) ? 1.f : -1.f;
          dy[g].x = fmaf(sign, p.x, dy[g].x);
          dy[g].y = fmaf(sign, p.y, dy[g].y);
          n[g] = make_float2(xs[i][g].x * r, xs[i][g].y * r);
          dw[g].x = fmaf(dy[g].x, n[g].x, dw[g].x);
          dw[g].y = fmaf(dy[g].y, n[g].y, dw[g].y);
          dn[g] = make_float2(dy[g].x * w[g].x, dy[g].y * w[g].y);
          dot = fmaf(dn[g].x, n[g].x, fmaf(dn[g].y, n[g].y, dot));
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        const float mean = dot * inv_d;
#pragma unroll
        for (int g = 0; g < G; ++g)
          store2(dx_tok + h * a.x_strides[2] + 64 * g + 2 * lane,
                 make_float2(r * (dn[g].x - n[g].x * mean), r * (dn[g].y - n[g].y * mean)));
      }
    }
  }
  // gain gradient: the block's tokens are summed here, the blocks by query_prepare_dweight_kernel (no atomics)
#pragma unroll
  for (int g = 0; g < G; ++g) {
    block_dw[warp][64 * g + 2 * lane] = dw[g].x;
    block_dw[warp][64 * g + 2 * lane + 1] = dw[g].y;
  }
  __syncthreads();
  for (int d = threadIdx.x; d < 64 * G; d += kThreads) {
    float acc = 0.f;
#pragma unroll
    for (int v = 0; v < kThreads / 32; ++v) acc += block_dw[v][d];
    partials[(static_cast<long long>(blockIdx.y) * gridDim.x + blockIdx.x) * (64 * G) + d] = acc;
  }
}

template <typename TX>
__global__ void query_prepare_dweight_kernel(const float* partials, int n_partials, int dim, TX* dweight) {
  const int d = blockIdx.x * blockDim.x + threadIdx.x;
  if (d >= dim) return;
  float acc = 0.f;
  for (int i = 0; i < n_partials; ++i) acc += partials[static_cast<long long>(i) * dim + d];
  dweight[d] = static_cast<TX>(acc);
}

int check(const wm_qprep_args& a, bool backward) {
  if (a.batch <= 0 || a.tokens <= 0 || a.heads <= 0) return fail(WM_EINVAL, "query preparation: empty problem");
  if (a.head_dim != 64 && a.head_dim != 128) return fail(WM_EUNSUPPORTED, "query preparation supports head_dim 64 and 128, got %d", a.head_dim);
  if (a.dtype != WM_BF16 && a.dtype != WM_F32) return fail(WM_EUNSUPPORTED, "query preparation: unsupported input dtype");
  if (a.q_dtype != WM_BF16 && a.q_dtype != WM_F32) return fail(WM_EUNSUPPORTED, "query preparation: unsupported query dtype");
  if (a.x == nullptr || a.weight == nullptr || a.cos == nullptr || a.sin == nullptr) return fail(WM_EINVAL, "query preparation: null input");
  if (!backward && a.q == nullptr) return fail(WM_EINVAL, "query preparation: null output");
  if (backward && (a.dq == nullptr || a.dx == nullptr || a.dweight == nullptr)) return fail(WM_EINVAL, "query preparation: null gradient");
  for (int i = 0; i < 3; ++i)
    if (a.x_strides[i] % 2) return fail(WM_EUNSUPPORTED, "query preparation: strides must be even");
  if (a.cs_strides[0] % 2 || a.cs_strides[1] % 2) return fail(WM_EUNSUPPORTED, "query preparation: cos/sin strides must be even");
  return WM_OK;
}

}  // namespace

size_t query_prepare_workspace(const wm_qprep_args& a) {
  const size_t blocks = static_cast<size_t>((a.tokens + kThreads / 32 - 1) / (kThreads / 32)) * a.batch;
  return blocks * a.head_dim * sizeof(float);
}

template <typename TX, typename TQ, int G>
static int launch(const wm_qprep_args& a, bool backward, cudaStream_t stream) {
  dim3 grid((a.tokens + kThreads / 32 - 1) / (kThreads / 32), a.batch);
  if (!backward) {
    const bool wide = a.dtype == WM_BF16 && a.q_dtype == WM_BF16 && a.x_strides[0] % 8 == 0 && a.x_strides[1] % 8 == 0 &&
                      a.x_strides[2] % 8 == 0 && a.cs_strides[0] % 8 == 0 && a.cs_strides[1] % 8 == 0 &&
                      reinterpret_cast<uintptr_t>(a.x) % 16 == 0 && reinterpret_cast<uintptr_t>(a.q) % 16 == 0 &&
                      reinterpret_cast<uintptr_t>(a.cos) % 16 == 0 && reinterpret_cast<uintptr_t>(a.sin) % 16 == 0 &&
                      reinterpret_cast<uintptr_t>(a.weight) % 16 == 0;
    if (wide) {
      query_prepare_fwd_bf16_kernel<64 * G><<<grid, kThreads, 0, stream>>>(a);
      count_launch();
      return cuda_check(cudaGetLastError(), "query_prepare_fwd_bf16_kernel");
    }
    query_prepare_fwd_kernel<TX, TQ, G><<<grid, kThreads, 0, stream>>>(a);
    count_launch();
    return cuda_check(cudaGetLastError(), "query_prepare_fwd_kernel");
  }
  const size_t need = query_prepare_workspace(a);
  if (a.workspace == nullptr || a.workspace_bytes < need)
    return fail(WM_EWORKSPACE, "query preparation backward needs %zu workspace bytes, got %zu", need, a.workspace_bytes);
  float* partials = static_cast<float*>(a.workspace);
  query_prepare_bwd_kernel<TX, TQ, G><<<grid, kThreads, 0, stream>>>(a, partials);
  count_launch();
  WM_CUDA(cudaGetLastError());
  query_prepare_dweight_kernel<TX><<<(a.head_dim + 63) / 64, 64, 0, stream>>>(partials, static_cast<int>(grid.x * grid.y), a.head_dim,
                                                                            static_cast<TX*>(a.dweight));
  count_launch();
  return cuda_check(cudaGetLastError(), "query_prepare_bwd_kernel");
}

int query_prepare(const wm_qprep_args& a, bool backward, cudaStream_t stream) {
  const int status = check(a, backward);
  if (status != WM_OK) return status;
  const bool wide = a.head_dim == 128;
  if (a.dtype == WM_BF16 && a.q_dtype == WM_BF16)
    return wide ? launch<__nv_bfloat16, __nv_bfloat16, 2>(a, backward, stream) : launch<__nv_bfloat16, __nv_bfloat16, 1>(a, backward, stream);
  if (a.dtype == WM_F32 && a.q_dtype == WM_F32)
    return wide ? launch<float, float, 2>(a, backward, stream) : launch<float, float, 1>(a, backward, stream);
  if (a.dtype == WM_F32 && a.q_dtype == WM_BF16)
    return wide ? launch<float, __nv_bfloat16, 2>(a, backward, stream) : launch<float, __nv_bfloat16, 1>(a, backward, stream);
  return fail(WM_EUNSUPPORTED, "query preparation: bf16 input with fp32 queries is not supported");
}

}  // namespace wm
