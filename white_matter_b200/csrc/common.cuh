// Shared declarations of the WhiteMatter B200 kernels: error reporting, the
// device-side view of an attention problem and the visibility rules of the
// three mask families.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "wm_b200.h"

namespace wm {

// ---------------------------------------------------------------- host helpers
int fail(int code, const char* fmt, ...);
int cuda_check(cudaError_t status, const char* what);
void count_launch();  // one more kernel launched by this library (diagnostic counter)

#define WM_CUDA(expr)                                   \
  do {                                                  \
    int wm_status_ = ::wm::cuda_check((expr), #expr);   \
    if (wm_status_ != WM_OK) return wm_status_;         \
  } while (0)

int validate_attn(const wm_attn_args* a, bool backward, const char* who);

// Kernel launchers implemented in the .cu files.
int simt_attn_fwd(const wm_attn_args& a, cudaStream_t stream);
int simt_attn_bwd(const wm_attn_args& a, cudaStream_t stream);
size_t simt_attn_bwd_workspace(const wm_attn_args& a);
int decode_launch(const wm_attn_args& a, cudaStream_t stream);
size_t decode_workspace(const wm_attn_args& a);
int decode_launch_with_scratch(const wm_attn_args& a, float* scratch, cudaStream_t stream);
bool decode_supported(const wm_attn_args& a);
size_t decode_static_capacity();
int decode_static_scratch(float** out);
int decode_mixed_launch(const wm_attn_args& a, const wm_source_mix& m, cudaStream_t stream);
int pool_append_launch(const wm_pool_append_args& a, cudaStream_t stream);
int pool_mix_launch(const wm_pool_mix_args& a, cudaStream_t stream);
int pool_finish_launch(const wm_pool_finish_args& a, cudaStream_t stream);
int mix_fwd_launch(const wm_mix_args& a, cudaStream_t stream);
int mix_bwd_launch(const wm_mix_args& a, cudaStream_t stream);
size_t mix_workspace(const wm_mix_args& a);
bool tc_fwd_supported(const wm_attn_args& a);
int tc_attn_fwd(const wm_attn_args& a, cudaStream_t stream);
bool tc_bwd_supported(const wm_attn_args& a);
int tc_attn_bwd(const wm_attn_args& a, cudaStream_t stream);
size_t tc_attn_bwd_workspace(const wm_attn_args& a);
int tc_device_status(bool reset);
int tc_status_word(int** out);
int tc_debug_trace(long long* out, int capacity, int arm_after);
int tc_debug_expire_wait(long long limit_ticks, cudaStream_t stream);
int query_prepare(const wm_qprep_args& a, bool backward, cudaStream_t stream);
size_t query_prepare_workspace(const wm_qprep_args& a);

// ---------------------------------------------------------------- device side
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

template <typename T>
__device__ __forceinline__ float to_float(T x);
template <>
__device__ __forceinline__ float to_float<float>(float x) {
  return x;
}
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 x) {
  return __bfloat162float(x);
}
template <typename T>
__device__ __forceinline__ T from_float(float x);
template <>
__device__ __forceinline__ float from_float<float>(float x) {
  return x;
}
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float x) {
  return __float2bfloat16_rn(x);
}

__device__ __forceinline__ long long load_index(const void* p, int is64, int i) {
  return is64 ? static_cast<const long long*>(p)[i] : static_cast<long long>(static_cast<const int*>(p)[i]);
}

__device__ __forceinline__ int clampi(long long x, int lo, int hi) {
  return x < lo ? lo : (x > hi ? hi : static_cast<int>(x));
}

// Visibility bound of one query row.  Key j (index inside the row's key list)
// can be visible only if j < hi; document problems add lo / seg / qi.
struct RowBound {
  int lo;
  int hi;
  int seg;
  int qi;
};

// Where a tile of queries lives: the batch row and (for packed schedules) the
// group it belongs to.
struct GroupCtx {
  int q_begin;  // first packed query of the group (packed) or 0
  int k_begin;  // first packed key of the group (packed) or 0
  int nq;       // queries in the group (packed) or q_len
  int nk;       // keys in the group (packed) or k_len
};

__device__ __forceinline__ GroupCtx group_ctx(const wm_attn_args& a, int group) {
  GroupCtx g;
  if (a.mask == WM_MASK_PACKED) {
    const int* t = a.groups + 4 * group;
    g.q_begin = t[0];
    g.k_begin = t[2];
    g.nq = t[1] - t[0];
    g.nk = t[3] - t[2];
  } else {
    g.q_begin = 0;
    g.k_begin = 0;
    g.nq = a.q_len;
    g.nk = a.k_len;
  }
  return g;
}

// (batch row, token) of query i of the tile's group.
__device__ __forceinline__ void query_coord(const wm_attn_args& a, const GroupCtx& g, int batch, int i, int& b, int& t) {
  if (a.mask == WM_MASK_PACKED) {
    long long flat = a.query_indices[g.q_begin + i];
    b = static_cast<int>(flat / a.q_len);
    t = static_cast<int>(flat - static_cast<long long>(b) * a.q_len);
  } else {
    b = batch;
    t = i;
  }
}

// (batch row, slot) of key j of the tile's group.
__device__ __forceinline__ void key_coord(const wm_attn_args& a, const GroupCtx& g, int batch, int j, int& b, int& s) {
  if (a.mask == WM_MASK_PACKED) {
    long long flat = a.key_indices[g.k_begin + j];
    b = static_cast<int>(flat / a.k_len);
    s = static_cast<int>(flat - static_cast<long long>(b) * a.k_len);
  } else {
    b = batch;
    s = j;
  }
}

__device__ __forceinline__ RowBound row_bound(const wm_attn_args& a, const GroupCtx& g, int batch, int i) {
  RowBound r;
  r.lo = 0;
  r.seg = 0;
  r.qi = i;
  if (a.mask == WM_MASK_CYCLIC) {
    long long slot = static_cast<long long>(a.query_offset) + static_cast<long long>(a.query_stride) * i;
    r.hi = clampi(slot + 1, 0, a.k_len);
    if (a.q_seg != nullptr) {
      long long at = static_cast<long long>(batch) * a.q_len + i;
      r.lo = a.q_key_start[at];
      r.seg = a.q_seg[at];
    }
  } else if (a.mask == WM_MASK_STRICT) {
    long long pos = (a.query_start ? load_index(a.query_start, a.query_start_is64, batch) : a.query_start_value) + i;
    if (a.kv_lengths) {
      long long n = load_index(a.kv_lengths, a.kv_lengths_is64, batch);
      pos = pos < n ? pos : n;
    }
    if (pos < 0) pos = 0;
    r.hi = clampi(pos + a.use_dummy, 0, a.k_len);
    if (a.q_seg != nullptr) {  // packed documents on top of the dense bounds (cached-prefix Jacobi)
      long long at = static_cast<long long>(batch) * a.q_len + i;
      r.lo = a.q_key_start[at];
      r.seg = a.q_seg[at];
    }
  } else {
    r.hi = clampi(static_cast<long long>(g.nk) - g.nq + 1 + i, 0, g.nk);
  }
  return r;
}

// Document / key-mask part of the rule for a key that already satisfies j < hi.
// kseg / kend are the key's document and exclusive query bound, kmask its
// key_mask byte (1 when there is no mask).
__device__ __forceinline__ bool doc_visible(const RowBound& r, int j, int kseg, int kend) {
  if (r.qi >= kend) return false;
  if (kseg == -1) return true;
  return kseg == r.seg && j >= r.lo;
}


// The same rule without control flow, for unrolled per-element loops.
__device__ __forceinline__ bool doc_visible_flat(const RowBound& r, int j, int kseg, int kend) {
  return (r.qi < kend) & ((kseg == -1) | ((kseg == r.seg) & (j >= r.lo)));
}

}  // namespace wm
