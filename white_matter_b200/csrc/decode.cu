// Single-query strict-past read of a KV pool, split over the key axis.
//
// The kernel is bound by HBM bandwidth: every visible K and V row is read
// exactly once with 128-bit loads (LPK lanes cover one row), the per-key dot
// product is reduced with warp shuffles inside the LPK lanes, and every lane
// group keeps its own online-softmax state so that no cross-lane traffic is
// needed until the block's final merge.  Blocks whose key range starts at or
// beyond the row's visible length (read on the device) exit at once, which
// keeps the launch shape independent of the lengths and so capturable in a
// CUDA graph.  A second, tiny kernel merges the split partials.
//
// Algorithmic bytes per step: sum_b 2 * kv_heads * visible_b * head_dim * sizeof(T).
#include <math.h>

#include <mutex>

#include "common.cuh"

namespace wm {
namespace {

constexpr int kThreads = 128;
constexpr int kWarps = kThreads / 32;
constexpr int kUnroll = 4;

template <typename T>
struct VecOf;
template <>
struct VecOf<float> {
  static constexpr int N = 4;
};
template <>
struct VecOf<__nv_bfloat16> {
  static constexpr int N = 8;
};

template <typename T>
__device__ __forceinline__ void unpack(const uint4& raw, float (&x)[VecOf<T>::N]);
template <>
__device__ __forceinline__ void unpack<float>(const uint4& raw, float (&x)[4]) {
  x[0] = __uint_as_float(raw.x);
  x[1] = __uint_as_float(raw.y);
  x[2] = __uint_as_float(raw.z);
  x[3] = __uint_as_float(raw.w);
}
template <>
__device__ __forceinline__ void unpack<__nv_bfloat16>(const uint4& raw, float (&x)[8]) {
  const unsigned w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    x[2 * i] = __uint_as_float(w[i] << 16);
    x[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

__device__ __forceinline__ uint4 ld_stream(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}

// partial record per (batch, q_head, split): m, l, acc[head_dim]
__device__ __forceinline__ long long partial_at(const wm_attn_args& a, int b, int h, int split, int splits) {
  return ((static_cast<long long>(b) * a.q_heads + h) * splits + split) * (a.head_dim + 2);
}

// K and V as stacks of sources that are mixed while they are read (kMixed): source s lies `stride` elements after
// source 0 and enters with weight softmax(logits)[s].
struct SourceMix {
  const float* k_logits;
  const float* v_logits;
  long long k_stride, v_stride;
  int sources;
};
constexpr int kMaxMixSources = 64;

template <typename T, int LPK, int G, bool kMixed>
__global__ void __launch_bounds__(kThreads) decode_split_kernel(const wm_attn_args a, float* partial, int chunk,
                                                                int splits, const SourceMix mix) {
  constexpr int VEC = VecOf<T>::N;
  constexpr int KPW = 32 / LPK;  // keys per warp per step
  __shared__ float sm_m[kWarps][G];
  __shared__ float sm_l[kWarps][G];
  __shared__ float sm_acc[kWarps][G][LPK * VEC];

  const int b = blockIdx.z;
  const int split = blockIdx.x;
  const int heads_per_kv = a.q_heads / a.kv_heads;
  // G == heads_per_kv: blockIdx.y is the KV head; G == 1 otherwise: blockIdx.y is the query head
  const int kv_head = G == heads_per_kv ? blockIdx.y : blockIdx.y / heads_per_kv;
  const int head0 = G == heads_per_kv ? blockIdx.y * G : blockIdx.y;

  GroupCtx g = group_ctx(a, 0);
  const int n = row_bound(a, g, b, 0).hi;
  const int j_begin = split * chunk;
  if (j_begin >= n) return;
  const int j_end = min(n, j_begin + chunk);

  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int c = lane % LPK;
  const int kk = lane / LPK;
  const bool dlive = c * VEC < a.head_dim;

  __shared__ float mix_w[kMixed ? 2 * kMaxMixSources : 1];
  if (kMixed) {
    if (warp < 2) {  // warp 0: soft-max of the key logits, warp 1: of the value logits
      const float* logits = warp == 0 ? mix.k_logits : mix.v_logits;
      float top = -INFINITY;
      for (int s = lane; s < mix.sources; s += 32) top = fmaxf(top, logits[s]);
      for (int o = 16; o > 0; o >>= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, o));
      float sum = 0.f;
      for (int s = lane; s < mix.sources; s += 32) sum += expf(logits[s] - top);
      for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      for (int s = lane; s < mix.sources; s += 32) mix_w[warp * kMaxMixSources + s] = expf(logits[s] - top) / sum;
    }
    __syncthreads();
  }

  float q[G][VEC];
  const float sl2 = a.scale * kLog2e;
#pragma unroll
  for (int h = 0; h < G; ++h) {
    const T* qrow = static_cast<const T*>(a.q) + b * a.q_strides[0] + (head0 + h) * a.q_strides[1];
    if (dlive) {
      uint4 raw = *reinterpret_cast<const uint4*>(qrow + c * VEC);
      unpack<T>(raw, q[h]);
    } else {
#pragma unroll
      for (int e = 0; e < VEC; ++e) q[h][e] = 0.f;
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e) q[h][e] *= sl2;
  }
  float m[G], l[G], acc[G][VEC];
#pragma unroll
  for (int h = 0; h < G; ++h) {
    m[h] = -INFINITY;
    l[h] = 0.f;
#pragma unroll
    for (int e = 0; e < VEC; ++e) acc[h][e] = 0.f;
  }

  const T* kbase = static_cast<const T*>(a.k) + b * a.k_strides[0] + kv_head * a.k_strides[1] + c * VEC;
  const T* vbase = static_cast<const T*>(a.v) + b * a.v_strides[0] + kv_head * a.v_strides[1] + c * VEC;
  const unsigned char* mask = a.key_mask ? a.key_mask + static_cast<long long>(b) * a.k_len : nullptr;

  for (int j0 = j_begin + warp * KPW * kUnroll; j0 < j_end; j0 += kWarps * KPW * kUnroll) {
    uint4 vraw[kUnroll];
    bool vis[kUnroll];
    float kf[kUnroll][VEC];
    float vmix[kMixed ? kUnroll : 1][VEC];  // the mixed value rows (kMixed only)
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      int j = j0 + u * KPW + kk;
      vis[u] = j < j_end && (mask == nullptr || mask[j] != 0);
    }
    if (!kMixed) {
      uint4 kraw[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        int j = j0 + u * KPW + kk;
        kraw[u] = make_uint4(0, 0, 0, 0);
        vraw[u] = make_uint4(0, 0, 0, 0);
        if (vis[u] && dlive) {
          kraw[u] = ld_stream(kbase + static_cast<long long>(j) * a.k_strides[2]);
          vraw[u] = ld_stream(vbase + static_cast<long long>(j) * a.v_strides[2]);
        }
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) unpack<T>(kraw[u], kf[u]);
    } else {
#pragma unroll
      for (int u = 0; u < kUnroll; ++u)
#pragma unroll
        for (int e = 0; e < VEC; ++e) kf[u][e] = vmix[kMixed ? u : 0][e] = 0.f;
      // every source row is read once; the loads of two sources are in flight together
      for (int s0 = 0; s0 < mix.sources; s0 += 2) {
        uint4 kraw[2][kUnroll], vsrc[2][kUnroll];
#pragma unroll
        for (int d = 0; d < 2; ++d)
#pragma unroll
          for (int u = 0; u < kUnroll; ++u) {
            int j = j0 + u * KPW + kk;
            kraw[d][u] = make_uint4(0, 0, 0, 0);
            vsrc[d][u] = make_uint4(0, 0, 0, 0);
            if (vis[u] && dlive && s0 + d < mix.sources) {
              kraw[d][u] = ld_stream(kbase + (s0 + d) * mix.k_stride + static_cast<long long>(j) * a.k_strides[2]);
              vsrc[d][u] = ld_stream(vbase + (s0 + d) * mix.v_stride + static_cast<long long>(j) * a.v_strides[2]);
            }
          }
#pragma unroll
        for (int d = 0; d < 2; ++d) {
          const bool live = s0 + d < mix.sources;
          const float wk = live ? mix_w[s0 + d] : 0.f, wv = live ? mix_w[kMaxMixSources + s0 + d] : 0.f;
#pragma unroll
          for (int u = 0; u < kUnroll; ++u) {
            float x[VEC];
            unpack<T>(kraw[d][u], x);
#pragma unroll
            for (int e = 0; e < VEC; ++e) kf[u][e] = fmaf(wk, x[e], kf[u][e]);
            unpack<T>(vsrc[d][u], x);
#pragma unroll
            for (int e = 0; e < VEC; ++e) vmix[kMixed ? u : 0][e] = fmaf(wv, x[e], vmix[kMixed ? u : 0][e]);
          }
        }
      }
    }
#pragma unroll
    for (int h = 0; h < G; ++h) {
      float s[kUnroll];
      float top = -INFINITY;
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        float d = 0.f;
#pragma unroll
        for (int e = 0; e < VEC; ++e) d = fmaf(q[h][e], kf[u][e], d);
#pragma unroll
        for (int sft = LPK / 2; sft > 0; sft >>= 1) d += __shfl_xor_sync(0xffffffffu, d, sft);
        s[u] = vis[u] ? d : -INFINITY;
        top = fmaxf(top, s[u]);
      }
      if (top != -INFINITY) {
        float m_new = fmaxf(m[h], top);
        float corr = exp2f(m[h] - m_new);
        l[h] *= corr;
#pragma unroll
        for (int e = 0; e < VEC; ++e) acc[h][e] *= corr;
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          if (vis[u]) {
            float p = exp2f(s[u] - m_new);
            float vf[VEC];
            if (kMixed) {
#pragma unroll
              for (int e = 0; e < VEC; ++e) vf[e] = vmix[kMixed ? u : 0][e];
            } else {
              unpack<T>(vraw[u], vf);
            }
            l[h] += p;
#pragma unroll
            for (int e = 0; e < VEC; ++e) acc[h][e] = fmaf(p, vf[e], acc[h][e]);
          }
        }
        m[h] = m_new;
      }
    }
  }

  // merge the KPW lane groups of the warp (lanes with equal c)
#pragma unroll
  for (int h = 0; h < G; ++h) {
#pragma unroll
    for (int sft = LPK; sft < 32; sft <<= 1) {
      float m_o = __shfl_xor_sync(0xffffffffu, m[h], sft);
      float l_o = __shfl_xor_sync(0xffffffffu, l[h], sft);
      float m_new = fmaxf(m[h], m_o);
      float ca = m[h] == -INFINITY ? 0.f : exp2f(m[h] - m_new);
      float cb = m_o == -INFINITY ? 0.f : exp2f(m_o - m_new);
      l[h] = l[h] * ca + l_o * cb;
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        float a_o = __shfl_xor_sync(0xffffffffu, acc[h][e], sft);
        acc[h][e] = acc[h][e] * ca + a_o * cb;
      }
      m[h] = m_new;
    }
    if (kk == 0) {
      if (c == 0) {
        sm_m[warp][h] = m[h];
        sm_l[warp][h] = l[h];
      }
#pragma unroll
      for (int e = 0; e < VEC; ++e) sm_acc[warp][h][c * VEC + e] = acc[h][e];
    }
  }
  __syncthreads();
  // merge the warps; thread t handles (head, dim) pairs
  for (int idx = threadIdx.x; idx < G * LPK * VEC; idx += kThreads) {
    int h = idx / (LPK * VEC);
    int d = idx - h * (LPK * VEC);
    if (d >= a.head_dim) continue;
    float top = -INFINITY;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) top = fmaxf(top, sm_m[w][h]);
    float lsum = 0.f, asum = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      float cw = sm_m[w][h] == -INFINITY ? 0.f : exp2f(sm_m[w][h] - top);
      lsum += sm_l[w][h] * cw;
      asum += sm_acc[w][h][d] * cw;
    }
    long long at = partial_at(a, b, head0 + h, split, splits);
    if (d == 0) {
      partial[at] = top;
      partial[at + 1] = lsum;
    }
    partial[at + 2 + d] = asum;
  }
}

template <typename T>
__global__ void decode_merge_kernel(const wm_attn_args a, const float* partial, int chunk, int splits) {
  const int b = blockIdx.y;
  const int h = blockIdx.x;
  GroupCtx g = group_ctx(a, 0);
  const int n = row_bound(a, g, b, 0).hi;
  const int live = (n + chunk - 1) / chunk;
  T* orow = static_cast<T*>(a.out) + b * a.out_strides[0] + h * a.out_strides[1];
  for (int d = threadIdx.x; d < a.head_dim; d += blockDim.x) {
    float top = -INFINITY;
    for (int s = 0; s < live; ++s) top = fmaxf(top, partial[partial_at(a, b, h, s, splits)]);
    float lsum = 0.f, asum = 0.f;
    for (int s = 0; s < live; ++s) {
      long long at = partial_at(a, b, h, s, splits);
      float ms = partial[at];
      float cw = ms == -INFINITY ? 0.f : exp2f(ms - top);
      lsum += partial[at + 1] * cw;
      asum += partial[at + 2 + d] * cw;
    }
    orow[d] = from_float<T>(lsum > 0.f ? asum / lsum : 0.f);
    if (d == 0 && a.lse != nullptr)
      a.lse[static_cast<long long>(b) * a.q_heads + h] = lsum > 0.f ? (top + log2f(lsum)) * kLn2 : INFINITY;
  }
}

int pick_chunk(const wm_attn_args& a) {
  // Aim for at least ~8 blocks per SM when every row is full; 64 <= chunk <= 256 keys.
  long long rows = static_cast<long long>(a.batch) * a.kv_heads;
  long long want = 148LL * 8;
  long long chunk = (static_cast<long long>(a.k_len) * rows + want - 1) / want;
  int c = 64;
  while (c < 256 && c < chunk) c <<= 1;
  return c;
}

int lanes_per_key(const wm_attn_args& a) {
  int vec = a.dtype == WM_F32 ? 4 : 8;
  int need = (a.head_dim + vec - 1) / vec;
  int lpk = 1;
  while (lpk < need) lpk <<= 1;
  return lpk;
}

template <typename T, int LPK, bool kMixed>
int launch(const wm_attn_args& a, float* partial, const SourceMix& mix, cudaStream_t stream) {
  const int chunk = pick_chunk(a);
  const int splits = (a.k_len + chunk - 1) / chunk;
  const int hpk = a.q_heads / a.kv_heads;
  if (hpk == 2) {
    dim3 grid(splits, a.kv_heads, a.batch);
    decode_split_kernel<T, LPK, 2, kMixed><<<grid, kThreads, 0, stream>>>(a, partial, chunk, splits, mix); count_launch();
  } else if (hpk == 4) {
    dim3 grid(splits, a.kv_heads, a.batch);
    decode_split_kernel<T, LPK, 4, kMixed><<<grid, kThreads, 0, stream>>>(a, partial, chunk, splits, mix); count_launch();
  } else {
    // one block per query head; with other group sizes K/V are re-read through L2
    dim3 grid(splits, a.q_heads, a.batch);
    decode_split_kernel<T, LPK, 1, kMixed><<<grid, kThreads, 0, stream>>>(a, partial, chunk, splits, mix); count_launch();
  }
  WM_CUDA(cudaGetLastError());
  int threads = a.head_dim <= 64 ? 64 : 128;
  decode_merge_kernel<T><<<dim3(a.q_heads, a.batch), threads, 0, stream>>>(a, partial, chunk, splits); count_launch();
  return cuda_check(cudaGetLastError(), "decode_merge_kernel");
}

template <typename T, bool kMixed>
int dispatch(const wm_attn_args& a, float* partial, const SourceMix& mix, cudaStream_t stream) {
  switch (lanes_per_key(a)) {
    case 1:
    case 2:
    case 4:
      return launch<T, 4, kMixed>(a, partial, mix, stream);
    case 8:
      return launch<T, 8, kMixed>(a, partial, mix, stream);
    case 16:
      return launch<T, 16, kMixed>(a, partial, mix, stream);
    default:
      return launch<T, 32, kMixed>(a, partial, mix, stream);
  }
}

}  // namespace

bool decode_supported(const wm_attn_args& a) {
  size_t es = a.dtype == WM_F32 ? 4 : 2;
  int vec = a.dtype == WM_F32 ? 4 : 8;
  if (a.q_len != 1 || a.mask != WM_MASK_STRICT) return false;
  if (a.head_dim % vec || a.head_dim > 32 * vec) return false;
  auto ok_ptr = [&](const void* p) { return (reinterpret_cast<uintptr_t>(p) % 16) == 0; };
  auto ok_str = [&](const int64_t* s) { return (s[0] * es) % 16 == 0 && (s[1] * es) % 16 == 0 && (s[2] * es) % 16 == 0; };
  return ok_ptr(a.q) && ok_ptr(a.k) && ok_ptr(a.v) && ok_str(a.q_strides) && ok_str(a.k_strides) && ok_str(a.v_strides);
}

size_t decode_workspace(const wm_attn_args& a) {
  const int chunk = pick_chunk(a);
  const int splits = (a.k_len + chunk - 1) / chunk;
  return static_cast<size_t>(a.batch) * a.q_heads * splits * (a.head_dim + 2) * sizeof(float);
}

int decode_launch_with_scratch(const wm_attn_args& a, float* scratch, cudaStream_t stream) {
  const SourceMix none = {nullptr, nullptr, 0, 0, 0};
  return a.dtype == WM_F32 ? dispatch<float, false>(a, scratch, none, stream) : dispatch<__nv_bfloat16, false>(a, scratch, none, stream);
}

int decode_mixed_launch(const wm_attn_args& a, const wm_source_mix& m, cudaStream_t stream) {
  if (m.k_logits == nullptr || m.v_logits == nullptr) return fail(WM_EINVAL, "wm_strict_decode_mixed: both logit vectors are required");
  if (m.n_sources < 1 || m.n_sources > kMaxMixSources) return fail(WM_EINVAL, "wm_strict_decode_mixed: between 1 and %d sources", kMaxMixSources);
  const size_t es = a.dtype == WM_F32 ? 4 : 2;
  if ((m.k_source_stride * es) % 16 || (m.v_source_stride * es) % 16)
    return fail(WM_EUNSUPPORTED, "wm_strict_decode_mixed: sources must be 16-byte aligned");
  size_t need = decode_workspace(a);
  if (a.workspace == nullptr || a.workspace_bytes < need)
    return fail(WM_EWORKSPACE, "decode needs %zu workspace bytes, got %zu", need, a.workspace_bytes);
  const SourceMix mix = {m.k_logits, m.v_logits, m.k_source_stride, m.v_source_stride, m.n_sources};
  float* scratch = static_cast<float*>(a.workspace);
  return a.dtype == WM_F32 ? dispatch<float, true>(a, scratch, mix, stream) : dispatch<__nv_bfloat16, true>(a, scratch, mix, stream);
}

// ---------------------------------------------------------------------------
// Variant for callers that cannot supply scratch memory: the split partials
// live in a fixed array that is part of the library image.  Every GPU that
// loads the library holds these 16 MiB until the process exits.
constexpr size_t kStaticScratchFloats = size_t(4) << 20;
static __device__ __align__(256) float g_decode_scratch[kStaticScratchFloats];

namespace {
constexpr int kMaxDevices = 64;
float* g_scratch_address[kMaxDevices] = {};
std::mutex g_scratch_mutex;
}  // namespace

size_t decode_static_capacity() { return kStaticScratchFloats * sizeof(float); }

// Device address of the fixed scratch array on the current device.  The array's name is only a host-side
// handle; the address a kernel can use comes from cudaGetSymbolAddress, looked up once per device.
int decode_static_scratch(float** out) {
  int device = -1;
  WM_CUDA(cudaGetDevice(&device));
  if (device < 0 || device >= kMaxDevices) return fail(WM_EUNSUPPORTED, "device ordinal %d is out of range", device);
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_address[device] == nullptr) {
    void* address = nullptr;
    WM_CUDA(cudaGetSymbolAddress(&address, g_decode_scratch));
    g_scratch_address[device] = static_cast<float*>(address);
  }
  *out = g_scratch_address[device];
  return WM_OK;
}

int decode_launch(const wm_attn_args& a, cudaStream_t stream) {
  size_t need = decode_workspace(a);
  if (a.workspace == nullptr || a.workspace_bytes < need)
    return fail(WM_EWORKSPACE, "decode needs %zu workspace bytes, got %zu", need, a.workspace_bytes);
  return decode_launch_with_scratch(a, static_cast<float*>(a.workspace), stream);
}

// ---------------------------------------------------------------------------
// commit of new rows to a static pool: one 16-byte word per thread
__global__ void pool_append_kernel(const wm_pool_append_args a, int words_per_row, int esize) {
  const long long word = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long total = static_cast<long long>(a.batch) * a.heads * a.n_new * words_per_row;
  if (word >= total) return;
  const int w = static_cast<int>(word % words_per_row);
  long long rest = word / words_per_row;
  const int i = static_cast<int>(rest % a.n_new);
  rest /= a.n_new;
  const int h = static_cast<int>(rest % a.heads);
  const int b = static_cast<int>(rest / a.heads);
  const long long slot = static_cast<long long>(a.lengths[b]) + a.lead + i;
  if (slot < 0 || slot >= a.capacity) return;
  const char* src = static_cast<const char*>(a.src) + (b * a.src_strides[0] + h * a.src_strides[1] + i * a.src_strides[2]) * esize;
  char* dst = static_cast<char*>(a.pool) + (b * a.pool_strides[0] + h * a.pool_strides[1] + slot * a.pool_strides[2]) * esize;
  reinterpret_cast<uint4*>(dst)[w] = reinterpret_cast<const uint4*>(src)[w];
}

int pool_append_launch(const wm_pool_append_args& a, cudaStream_t stream) {
  if (a.pool == nullptr || a.src == nullptr || a.lengths == nullptr) return fail(WM_EINVAL, "wm_pool_append: pool, src and lengths are required");
  if (a.dtype != WM_F32 && a.dtype != WM_BF16) return fail(WM_EINVAL, "wm_pool_append: dtype must be WM_F32 or WM_BF16");
  if (a.batch < 1 || a.heads < 1 || a.capacity < 1 || a.n_new < 1 || a.head_dim < 1) return fail(WM_EINVAL, "wm_pool_append: sizes must be positive");
  if (a.lead != 0 && a.lead != 1) return fail(WM_EINVAL, "wm_pool_append: lead must be 0 or 1");
  const int esize = a.dtype == WM_F32 ? 4 : 2;
  if ((a.head_dim * esize) % 16) return fail(WM_EUNSUPPORTED, "wm_pool_append: head_dim must be a multiple of 16 bytes");
  if (reinterpret_cast<uintptr_t>(a.pool) % 16 || reinterpret_cast<uintptr_t>(a.src) % 16)
    return fail(WM_EUNSUPPORTED, "wm_pool_append: rows must be 16-byte aligned");
  for (int i = 0; i < 3; ++i)
    if ((a.pool_strides[i] * esize) % 16 || (a.src_strides[i] * esize) % 16)
      return fail(WM_EUNSUPPORTED, "wm_pool_append: rows must be 16-byte aligned");
  const int words = a.head_dim * esize / 16;
  const long long total = static_cast<long long>(a.batch) * a.heads * a.n_new * words;
  pool_append_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, stream>>>(a, words, esize);
  count_launch();
  return cuda_check(cudaGetLastError(), "pool_append_kernel");
}

}  // namespace wm
