// KV source mixing: out = sum_s softmax(logits)[s] * src[s] over S stacked
// source tensors, and its gradients.  Pure streaming work bound by HBM
// bandwidth: the forward pass reads every source element once (S*n*sizeof(T)
// bytes) and writes n; the backward pass reads the sources and dout once and
// writes dsources once.  Weights are recomputed per block from the S logits.
#include <math.h>

#include "common.cuh"

namespace wm {
namespace {

constexpr int kThreads = 256;
constexpr int kMaxSources = 64;

template <typename T>
struct Pack;
template <>
struct Pack<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void unpack(const uint4& r, float (&x)[4]) {
    x[0] = __uint_as_float(r.x);
    x[1] = __uint_as_float(r.y);
    x[2] = __uint_as_float(r.z);
    x[3] = __uint_as_float(r.w);
  }
  static __device__ __forceinline__ uint4 pack(const float (&x)[4]) {
    return make_uint4(__float_as_uint(x[0]), __float_as_uint(x[1]), __float_as_uint(x[2]), __float_as_uint(x[3]));
  }
};
template <>
struct Pack<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void unpack(const uint4& r, float (&x)[8]) {
    const unsigned w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      x[2 * i] = __uint_as_float(w[i] << 16);
      x[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  static __device__ __forceinline__ uint4 pack(const float (&x)[8]) {
    unsigned w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 p = __floats2bfloat162_rn(x[2 * i], x[2 * i + 1]);
      w[i] = *reinterpret_cast<unsigned*>(&p);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
};

__device__ __forceinline__ uint4 ld_stream(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}

__device__ __forceinline__ void st_stream(void* p, const uint4& v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// softmax(logits) into shared memory, by the first warp of the block
__device__ __forceinline__ void block_weights(const float* logits, int S, float* w) {
  if (threadIdx.x < 32) {
    float top = -INFINITY;
    for (int s = threadIdx.x; s < S; s += 32) top = fmaxf(top, logits[s]);
    for (int o = 16; o > 0; o >>= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, o));
    float sum = 0.f;
    for (int s = threadIdx.x; s < S; s += 32) sum += expf(logits[s] - top);
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    for (int s = threadIdx.x; s < S; s += 32) w[s] = expf(logits[s] - top) / sum;
  }
  __syncthreads();
}

template <typename T>
__global__ void __launch_bounds__(kThreads) mix_fwd_kernel(const wm_mix_args a) {
  constexpr int VEC = Pack<T>::N;
  __shared__ float w[kMaxSources];
  block_weights(a.logits, a.n_sources, w);
  const long long vecs = a.n / VEC;
  const T* src = static_cast<const T*>(a.sources);
  T* out = static_cast<T*>(a.out);
  for (long long v = blockIdx.x * static_cast<long long>(kThreads) + threadIdx.x; v < vecs;
       v += static_cast<long long>(gridDim.x) * kThreads) {
    float acc[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) acc[e] = 0.f;
    const T* p = src + v * VEC;
    int s = 0;
    for (; s + 4 <= a.n_sources; s += 4) {
      uint4 r[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) r[u] = ld_stream(p + (s + u) * a.source_stride);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        float x[VEC];
        Pack<T>::unpack(r[u], x);
        float ws = w[s + u];
#pragma unroll
        for (int e = 0; e < VEC; ++e) acc[e] = fmaf(ws, x[e], acc[e]);
      }
    }
    for (; s < a.n_sources; ++s) {
      float x[VEC];
      Pack<T>::unpack(ld_stream(p + s * a.source_stride), x);
      float ws = w[s];
#pragma unroll
      for (int e = 0; e < VEC; ++e) acc[e] = fmaf(ws, x[e], acc[e]);
    }
    st_stream(out + v * VEC, Pack<T>::pack(acc));
  }
  // tail elements (n not a multiple of the vector width)
  if (blockIdx.x == 0) {
    for (long long i = vecs * VEC + threadIdx.x; i < a.n; i += kThreads) {
      float acc = 0.f;
      for (int s = 0; s < a.n_sources; ++s) acc = fmaf(w[s], to_float<T>(src[i + s * a.source_stride]), acc);
      out[i] = from_float<T>(acc);
    }
  }
}

// dsources[s] = w[s] * dout; gsum[s] += <dout, src[s]> over this block's slice
template <typename T>
__global__ void __launch_bounds__(kThreads) mix_bwd_kernel(const wm_mix_args a, float* gsum) {
  constexpr int VEC = Pack<T>::N;
  __shared__ float w[kMaxSources];
  __shared__ float part[kThreads / 32];
  block_weights(a.logits, a.n_sources, w);
  const long long vecs = a.n / VEC;
  const T* src = static_cast<const T*>(a.sources);
  const T* dout = static_cast<const T*>(a.dout);
  T* dsrc = static_cast<T*>(a.dsources);
  // each block owns a contiguous slice so that dout stays cache resident over the S sweeps
  const long long per_block = (vecs + gridDim.x - 1) / gridDim.x;
  const long long v_begin = blockIdx.x * per_block;
  const long long v_end = v_begin + per_block < vecs ? v_begin + per_block : vecs;
  for (int s = 0; s < a.n_sources; ++s) {
    float dot = 0.f;
    const float ws = w[s];
    for (long long v = v_begin + threadIdx.x; v < v_end; v += kThreads) {
      float g[VEC], x[VEC];
      Pack<T>::unpack(*reinterpret_cast<const uint4*>(dout + v * VEC), g);
      if (gsum != nullptr) {
        Pack<T>::unpack(ld_stream(src + s * a.source_stride + v * VEC), x);
#pragma unroll
        for (int e = 0; e < VEC; ++e) dot = fmaf(g[e], x[e], dot);
      }
      if (dsrc != nullptr) {
#pragma unroll
        for (int e = 0; e < VEC; ++e) g[e] *= ws;
        st_stream(dsrc + s * a.source_stride + v * VEC, Pack<T>::pack(g));
      }
    }
    if (blockIdx.x == 0) {
      for (long long i = vecs * VEC + threadIdx.x; i < a.n; i += kThreads) {
        float g = to_float<T>(dout[i]);
        if (gsum != nullptr) dot = fmaf(g, to_float<T>(src[i + s * a.source_stride]), dot);
        if (dsrc != nullptr) dsrc[i + s * a.source_stride] = from_float<T>(g * ws);
      }
    }
    if (gsum != nullptr) {
      for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
      if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = dot;
      __syncthreads();
      if (threadIdx.x == 0) {
        float total = 0.f;
        for (int i = 0; i < kThreads / 32; ++i) total += part[i];
        atomicAdd(gsum + s, total);
      }
      __syncthreads();
    }
  }
}

// dlogits[s] = w[s] * (g[s] - sum_t w[t] g[t])
__global__ void mix_dlogits_kernel(const float* logits, const float* gsum, float* dlogits, int S) {
  __shared__ float w[kMaxSources];
  block_weights(logits, S, w);
  if (threadIdx.x == 0) {
    float mean = 0.f;
    for (int s = 0; s < S; ++s) mean += w[s] * gsum[s];
    for (int s = 0; s < S; ++s) dlogits[s] = w[s] * (gsum[s] - mean);
  }
}

int check(const wm_mix_args& a, bool backward) {
  if (a.n_sources < 1 || a.n_sources > kMaxSources) return fail(WM_EINVAL, "n_sources must be in [1, %d]", kMaxSources);
  if (a.dtype != WM_F32 && a.dtype != WM_BF16) return fail(WM_EINVAL, "mixing supports fp32 and bf16");
  if (a.n < 0 || a.sources == nullptr || a.logits == nullptr) return fail(WM_EINVAL, "mixing needs sources and logits");
  int vec = a.dtype == WM_F32 ? 4 : 8;
  if (a.source_stride % vec || reinterpret_cast<uintptr_t>(a.sources) % 16)
    return fail(WM_EUNSUPPORTED, "sources must be 16-byte aligned with a stride that is a multiple of %d elements", vec);
  if (!backward && (a.out == nullptr || reinterpret_cast<uintptr_t>(a.out) % 16))
    return fail(WM_EINVAL, "mixing output must be 16-byte aligned");
  if (backward) {
    if (a.dout == nullptr || reinterpret_cast<uintptr_t>(a.dout) % 16) return fail(WM_EINVAL, "dout must be 16-byte aligned");
    if (a.dsources != nullptr && reinterpret_cast<uintptr_t>(a.dsources) % 16)
      return fail(WM_EINVAL, "dsources must be 16-byte aligned");
    if (a.dlogits != nullptr && (a.workspace == nullptr || a.workspace_bytes < kMaxSources * sizeof(float)))
      return fail(WM_EWORKSPACE, "mixing backward needs %zu workspace bytes", kMaxSources * sizeof(float));
  }
  return WM_OK;
}

int grid_for(long long vecs) {
  long long blocks = (vecs + kThreads - 1) / kThreads;
  long long cap = 148LL * 8;
  return static_cast<int>(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

}  // namespace

size_t mix_workspace(const wm_mix_args&) { return kMaxSources * sizeof(float); }

int mix_fwd_launch(const wm_mix_args& a, cudaStream_t stream) {
  int status = check(a, false);
  if (status != WM_OK) return status;
  if (a.n == 0) return WM_OK;
  if (a.dtype == WM_F32) {
    mix_fwd_kernel<float><<<grid_for(a.n / 4), kThreads, 0, stream>>>(a);
  } else {
    mix_fwd_kernel<__nv_bfloat16><<<grid_for(a.n / 8), kThreads, 0, stream>>>(a);
  }
  count_launch();
  return cuda_check(cudaGetLastError(), "mix_fwd_kernel");
}

int mix_bwd_launch(const wm_mix_args& a, cudaStream_t stream) {
  int status = check(a, true);
  if (status != WM_OK) return status;
  float* gsum = a.dlogits != nullptr ? static_cast<float*>(a.workspace) : nullptr;
  if (gsum != nullptr) WM_CUDA(cudaMemsetAsync(gsum, 0, kMaxSources * sizeof(float), stream));
  if (a.n > 0) {
    if (a.dtype == WM_F32) {
      mix_bwd_kernel<float><<<grid_for(a.n / 4), kThreads, 0, stream>>>(a, gsum);
    } else {
      mix_bwd_kernel<__nv_bfloat16><<<grid_for(a.n / 8), kThreads, 0, stream>>>(a, gsum);
    }
    count_launch();
    WM_CUDA(cudaGetLastError());
  }
  if (gsum != nullptr) {
    mix_dlogits_kernel<<<1, 32, 0, stream>>>(a.logits, gsum, a.dlogits, a.n_sources); count_launch();
    WM_CUDA(cudaGetLastError());
  }
  return WM_OK;
}

}  // namespace wm
