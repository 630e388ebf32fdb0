// tcgen05 / TMEM attention kernels for bf16, head_dim 64, 96 and 128: host side (tensor maps, kernel selection,
// launches), the helpers the pipelines share (bounded waits, the device status word, document masks), and the three pipelines
// themselves, each in a header of its own:
//   attn_tc_fwd.cuh       forward (a template over the head size): one block per 128 query rows, two softmax groups
//                         on alternate key tiles, P kept in tensor memory as the A operand of the PV product
//   attn_tc_bwd_resident.cuh  backward for heads of 64, at most 256 queries per (batch, head), no grouped heads:
//                         one block per (batch, head), both query tiles and their dQ accumulators resident
//   attn_tc_bwd.cuh       backward for every other shape (a template over the head size): one block per key tile,
//                         dQ through fp32 atomics
// Key tiles that no query can see are never loaded.  Every mbarrier wait is bounded; a wait that runs out records
// its code in a device status word, and all roles of the block fall through to the common exit where tensor memory
// is released.
#include <cuda.h>
#include <atomic>
#include <limits.h>
#include <math.h>
#include <stdio.h>
#include <stdlib.h>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace wm {
namespace {

constexpr int kTileM = 128;
constexpr int kTileN = 128;
constexpr int kHeadDim = 64;
constexpr int kSoftmaxThreads = 128;
constexpr uint32_t kTileBytes = kTileN * kHeadDim * 2;  // 16 KB: one Q, K or V tile
constexpr uint32_t kTmemCols = 512;
constexpr float kRescaleThreshold = 8.f;  // log2 units

__device__ int g_status = 0;  // first failure code since the last reset

// Pipeline trace (builds with -DWM_B200_TRACE only): block (0,0,0) of the launch whose number equals g_trace_epoch
// records (tag, clock) pairs in shared memory and copies them out when it ends.  Every warp has its own region of
// 128 slots (one thread per warp records), so that recording needs no atomic.
#ifdef WM_B200_TRACE
__device__ long long g_trace[2 * 4096];
__device__ int g_trace_count = 0;
__device__ int g_trace_epoch = -1;
constexpr int kTraceSlots = 2048;
#define WM_TRACE_FIELDS \
  int trace_on, trace_cnt[16]; \
  long long trace[kTraceSlots];

template <class Shared>
__device__ __forceinline__ void trace_event(Shared& sm, int tag) {
  if (sm.trace_on) {
    const int r = (threadIdx.x >> 5) & 15;
    const int i = sm.trace_cnt[r];
    if (i < 128) {
      sm.trace[r * 128 + i] = (clock64() << 16) | static_cast<long long>(tag & 0xffff);
      sm.trace_cnt[r] = i + 1;
    }
  }
}

template <class Shared>
__device__ __forceinline__ void trace_begin(Shared& sm, int epoch) {
  for (int r = 0; r < 16; ++r) sm.trace_cnt[r] = 0;
  sm.trace_on = epoch == g_trace_epoch && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
}

template <class Shared>
__device__ __forceinline__ void trace_flush(Shared& sm) {
  if (sm.trace_on && threadIdx.x == 0) {
    int n = 0;
    for (int r = 0; r < 16; ++r)
      for (int i = 0; i < sm.trace_cnt[r] && i < 128; ++i) {
        g_trace[2 * n] = sm.trace[r * 128 + i] & 0xffff;
        g_trace[2 * n + 1] = sm.trace[r * 128 + i] >> 16;
        ++n;
      }
    g_trace_count = n;
  }
}
#else
#define WM_TRACE_FIELDS
template <class Shared>
__device__ __forceinline__ void trace_event(Shared&, int) {}
template <class Shared>
__device__ __forceinline__ void trace_begin(Shared&, int) {}
template <class Shared>
__device__ __forceinline__ void trace_flush(Shared&) {}
#endif

template <class Shared>
__device__ __forceinline__ void record_failure(Shared& sm, int code) {
  // low byte: which wait gave up; above it: the linear index of the block
  const unsigned block = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
  atomicCAS(&g_status, 0, code | static_cast<int>((block & 0x7fffffu) << 8));
  atomicExch(&sm.abort_flag, 1);
}

// ---------------------------------------------------------------------------
// host side: tensor maps
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static const EncodeTiledFn fn = [] {  // initialised once, also under concurrent first calls
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) == cudaSuccess &&
        result == cudaDriverEntryPointSuccess)
      return reinterpret_cast<EncodeTiledFn>(ptr);
    return static_cast<EncodeTiledFn>(nullptr);
  }();
  return fn;
}

// The opt-in to more than 48 KB of dynamic shared memory is a per-device attribute of a kernel: one flag per
// (kernel, device), set on the first launch there.
constexpr int kMaxDevices = 64;
template <class Kernel>
int allow_shared_memory(Kernel kernel, std::atomic<bool> (&done)[kMaxDevices], size_t bytes) {
  int device = 0;
  WM_CUDA(cudaGetDevice(&device));
  if (device < 0 || device >= kMaxDevices || !done[device].load(std::memory_order_acquire)) {
    WM_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes)));
    if (device >= 0 && device < kMaxDevices) done[device].store(true, std::memory_order_release);
  }
  return WM_OK;
}

// (batch, heads, tokens, head_dim) bf16 tensor with element strides s[0..2]; boxes of `rows` tokens x 64 columns
// (one 128-byte swizzle row per token: a head of 128 travels as two boxes).
int make_map(CUtensorMap* map, const void* base, int batch, int heads, int tokens, const int64_t* s, int rows,
             int head_dim = kHeadDim) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return fail(WM_ECUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(head_dim), static_cast<cuuint64_t>(tokens),
                        static_cast<cuuint64_t>(heads), static_cast<cuuint64_t>(batch)};
  cuuint64_t strides[3] = {static_cast<cuuint64_t>(s[2]) * 2, static_cast<cuuint64_t>(s[1]) * 2,
                           static_cast<cuuint64_t>(s[0]) * 2};
  // a dimension of extent 1 may come with any stride; give it a legal one
  for (int i = 0; i < 3; ++i)
    if (dims[i + 1] == 1 || strides[i] == 0) strides[i] = 128;
  cuuint32_t box[4] = {kHeadDim, static_cast<cuuint32_t>(rows), 1, 1};
  cuuint32_t elem[4] = {1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r == CUDA_ERROR_INVALID_CONTEXT) {
    // A thread whose first CUDA action is this call (a framework's backward worker, say) has no context bound
    // yet: the runtime binds the device's primary context on its first call, the driver entry point does not.
    cudaFree(nullptr);
    r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, elem,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  }
  if (r != CUDA_SUCCESS) return fail(WM_ECUDA, "cuTensorMapEncodeTiled failed with code %d", static_cast<int>(r));
  return WM_OK;
}

bool tma_ok(const void* p, const int64_t* s, int batch, int heads, int tokens) {
  if (reinterpret_cast<uintptr_t>(p) % 16) return false;
  const int extent[3] = {batch, heads, tokens};
  for (int i = 0; i < 3; ++i) {
    if (extent[i] == 1) continue;
    if (s[i] <= 0 || (s[i] * 2) % 16 || s[i] * 2 >= (1ll << 40)) return false;
  }
  return true;
}


// ---------------------------------------------------------------------------
// device side

// Bounded wait: gives up after about 0.1 s of clock ticks, or as soon as another role of the block has given up.
// Nothing outlives the block: a launch that is replayed from a CUDA graph starts clean whatever happened before.
#ifndef WM_B200_WAIT_TICKS
#define WM_B200_WAIT_TICKS 200000000ll
#endif
constexpr long long kWaitTicks = WM_B200_WAIT_TICKS;

template <class Shared>
__device__ __forceinline__ bool wait_or_abort(Shared& sm, uint64_t* bar, uint32_t parity, int code,
                                              long long limit = kWaitTicks) {
  if (ptx::mbar_try_wait(bar, parity)) return true;
  const long long begin = clock64();
  for (uint32_t spin = 0;; ++spin) {
    if (ptx::mbar_try_wait(bar, parity)) return true;
    if ((spin & 63u) == 63u) {
      if (*reinterpret_cast<volatile int*>(&sm.abort_flag)) return false;
      if (clock64() - begin > limit) break;
    }
  }
  record_failure(sm, code);
  return false;
}

// first key slot of the n-th visited key tile
__device__ __forceinline__ int tile_first_key(int n, int first_tile, int dummy_tile) {
  if (dummy_tile) return n == 0 ? 0 : (first_tile + n - 1) * kTileN;
  return (first_tile + n) * kTileN;
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ uint32_t bits_below(int n) { return n >= 32 ? 0xffffffffu : (n <= 0 ? 0u : ((1u << n) - 1u)); }

// Document visibility of the 128 key columns of a tile for the rows of one warp (row = lane), as four 32-column
// bit masks per row (all ones for rows that do not want one).  A key is visible to a row when
// (row.qi < key.end) and (key.seg == -1 or (key.seg == row.seg and key >= row.lo)).
//
// The table of a tile is a handful of runs of equal (seg, end) -- one per document that touches the tile.  The warp
// finds the run boundaries with four ballots, and every row then builds its masks from the runs by arithmetic:
// a few hundred cycles whatever the number of rows that want a mask.  Tables with more than kDocRuns runs take
// the general way: the rows that want a mask are visited in turn, their parameters broadcast, and four ballots
// over the columns (lane c holds columns c, c+32, c+64, c+96) give one row's masks.
constexpr int kDocRuns = 8;

__device__ __forceinline__ void warp_doc_masks(const RowBound& rb, bool wanted, int j0, const int* key_seg,
                                               const int* key_end, uint32_t (&out)[4]) {
  const int lane = threadIdx.x & 31;
  int seg[4], end[4];
  uint32_t rest[4];
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const int x = 32 * c + lane;
    seg[c] = key_seg[x];
    end[c] = key_end[x];
    const bool begins = x == 0 || key_seg[x - 1] != seg[c] || key_end[x - 1] != end[c];
    rest[c] = __ballot_sync(0xffffffffu, begins);
  }
  const int runs = __popc(rest[0]) + __popc(rest[1]) + __popc(rest[2]) + __popc(rest[3]);
  if (runs <= kDocRuns) {
    uint32_t m[4] = {0u, 0u, 0u, 0u};
    const int lo_col = rb.lo - j0;
    rest[0] &= ~1u;  // column 0 begins the first run
    int start = 0;
    for (int k = 0; k < runs; ++k) {
      int next = kTileN;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        if (next == kTileN && rest[c] != 0u) {
          next = 32 * c + __ffs(rest[c]) - 1;
          rest[c] &= rest[c] - 1u;
        }
      }
      const int run_seg = key_seg[start], run_end = key_end[start];  // the same address for every lane
      const bool open = (rb.qi < run_end) & ((run_seg == -1) | (run_seg == rb.seg));
      const int lo = run_seg == -1 ? start : max(start, lo_col);
      if (open && lo < next) {
#pragma unroll
        for (int c = 0; c < 4; ++c) m[c] |= bits_below(next - 32 * c) & ~bits_below(lo - 32 * c);
      }
      start = next;
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) out[c] = wanted ? m[c] : 0xffffffffu;
    return;
  }
#pragma unroll
  for (int c = 0; c < 4; ++c) out[c] = 0xffffffffu;
  for (uint32_t left = __ballot_sync(0xffffffffu, wanted); left != 0u; left &= left - 1u) {
    const int r = __ffs(left) - 1;
    const int rseg = __shfl_sync(0xffffffffu, rb.seg, r);
    const int rqi = __shfl_sync(0xffffffffu, rb.qi, r);
    const int rlo = __shfl_sync(0xffffffffu, rb.lo, r);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int j = j0 + 32 * c + lane;
      const bool vis = (rqi < end[c]) & ((seg[c] == -1) | ((seg[c] == rseg) & (j >= rlo)));
      const uint32_t m = __ballot_sync(0xffffffffu, vis);
      if (lane == r) out[c] = m;
    }
  }
}

// How a key tile relates to one query row.
enum TileClass { kTileNone = 0, kTileFull = 1, kTileCausal = 2, kTileDocs = 3 };

struct TileWalk {
  int first_tile;
  int dummy_tile;
  int n_tiles;
  int kmax;
};

// A wait that nothing will ever satisfy, with a short limit: what the bounded waits do when they run out (the
// status word gets the code, the block leaves through its normal exit).
struct ExpireShared {
  uint64_t never;
  int abort_flag;
  int epoch;
};

__global__ void expire_wait_kernel(long long limit) {
  __shared__ ExpireShared sm;
  if (threadIdx.x == 0) {
    sm.abort_flag = 0;
    sm.epoch = 0;
    ptx::mbar_init(&sm.never, 1);
    ptx::mbar_fence_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) wait_or_abort(sm, &sm.never, 0, 250, limit);
  __syncthreads();
}

#include "attn_tc_fwd.cuh"
#include "attn_tc_bwd.cuh"
#include "attn_tc_bwd_resident.cuh"

}  // namespace

// ---------------------------------------------------------------------------
// launchers

// launch number handed to the pipelined kernels; never 0
int next_epoch() {
  static std::atomic<int> counter{0};
  int e = counter.fetch_add(1, std::memory_order_relaxed) + 1;
  return e == 0 ? next_epoch() : e;
}

bool tc_fwd_supported(const wm_attn_args& a) {
  // the forward takes heads of 64, 96 and 128 (96 runs as 128 with columns the copies fill with zeros)
  if (a.dtype != WM_BF16 || (a.head_dim != 64 && a.head_dim != 96 && a.head_dim != 128)) return false;
  if (a.mask == WM_MASK_PACKED) return false;
  if (!tma_ok(a.q, a.q_strides, a.batch, a.q_heads, a.q_len)) return false;
  if (!tma_ok(a.k, a.k_strides, a.batch, a.kv_heads, a.k_len)) return false;
  if (!tma_ok(a.v, a.v_strides, a.batch, a.kv_heads, a.k_len)) return false;
  if (reinterpret_cast<uintptr_t>(a.out) % 16) return false;
  for (int i = 0; i < 3; ++i)
    if (a.out_strides[i] % 8) return false;
  return true;
}

template <int D>
int launch_fwd(const wm_attn_args& a, cudaStream_t stream) {
  CUtensorMap map_q, map_k, map_v;
  int status = make_map(&map_q, a.q, a.batch, a.q_heads, a.q_len, a.q_strides, kTileM, a.head_dim);
  if (status != WM_OK) return status;
  status = make_map(&map_k, a.k, a.batch, a.kv_heads, a.k_len, a.k_strides, kTileN, a.head_dim);
  if (status != WM_OK) return status;
  status = make_map(&map_v, a.v, a.batch, a.kv_heads, a.k_len, a.v_strides, kTileN, a.head_dim);
  if (status != WM_OK) return status;
  dim3 grid(a.q_heads, a.batch, (a.q_len + kTileM - 1) / kTileM);
  const size_t smem = sizeof(FwdShared<D>) + 1024;
  static std::atomic<bool> configured[kMaxDevices];
  status = allow_shared_memory(attn_fwd_tc_kernel<D>, configured, smem);
  if (status != WM_OK) return status;
  attn_fwd_tc_kernel<D><<<grid, kFwdThreads, smem, stream>>>(map_q, map_k, map_v, a, next_epoch());
  count_launch();
  return cuda_check(cudaGetLastError(), "attn_fwd_tc_kernel");
}

int tc_attn_fwd(const wm_attn_args& a, cudaStream_t stream) {
  return a.head_dim > 64 ? launch_fwd<128>(a, stream) : launch_fwd<64>(a, stream);
}

// Arms the trace for the launch after the next `arm_after` launches (negative: disarm) and fetches what was
// recorded so far as (tag, clock) pairs; 0 in builds without -DWM_B200_TRACE.
int tc_debug_trace(long long* out, int capacity, int arm_after) {
#ifdef WM_B200_TRACE
  int count = 0;
  cudaDeviceSynchronize();
  cudaMemcpyFromSymbol(&count, g_trace_count, sizeof(int));
  if (count > 4096) count = 4096;
  if (count > capacity) count = capacity;
  if (out != nullptr && count > 0) cudaMemcpyFromSymbol(out, g_trace, sizeof(long long) * 2 * count);
  int zero = 0;
  cudaMemcpyToSymbol(g_trace_count, &zero, sizeof(int));
  int target = arm_after < 0 ? -1 : next_epoch() + 1 + arm_after;
  cudaMemcpyToSymbol(g_trace_epoch, &target, sizeof(int));
  return count;
#else
  (void)out;
  (void)capacity;
  (void)arm_after;
  return 0;
#endif
}

int tc_debug_expire_wait(long long limit_ticks, cudaStream_t stream) {
  if (limit_ticks < 1 || limit_ticks > kWaitTicks) return fail(WM_EINVAL, "wm_debug_expire_wait: the limit must be in [1, %lld] ticks", kWaitTicks);
  expire_wait_kernel<<<1, 32, 0, stream>>>(limit_ticks);
  count_launch();
  return cuda_check(cudaGetLastError(), "expire_wait_kernel");
}

// Device address of the status word, for kernels of other files that report a wait that ran out.
int tc_status_word(int** out) {
  void* address = nullptr;
  WM_CUDA(cudaGetSymbolAddress(&address, g_status));
  *out = static_cast<int*>(address);
  return WM_OK;
}

int tc_device_status(bool reset) {
  int value = 0;
  if (cudaMemcpyFromSymbol(&value, g_status, sizeof(int)) != cudaSuccess) return -1;
  if (reset && value != 0) {
    int zero = 0;
    cudaMemcpyToSymbol(g_status, &zero, sizeof(int));
  }
  return value;
}

bool tc_bwd_supported(const wm_attn_args& a) {
  if (!tc_fwd_supported(a)) return false;
  if (a.dout == nullptr) return true;  // shape query before the tensors exist
  if (!tma_ok(a.dout, a.dout_strides, a.batch, a.q_heads, a.q_len)) return false;
  if (!tma_ok(a.dk, a.dk_strides, a.batch, a.kv_heads, a.k_len)) return false;
  if (!tma_ok(a.dv, a.dv_strides, a.batch, a.kv_heads, a.k_len)) return false;
  const void* ptrs[3] = {a.dq, a.dk, a.dv};
  const int64_t* strides[3] = {a.dq_strides, a.dk_strides, a.dv_strides};
  for (int n = 0; n < 3; ++n) {
    if (reinterpret_cast<uintptr_t>(ptrs[n]) % 16) return false;
    for (int i = 0; i < 3; ++i)
      if (strides[n][i] % 8) return false;
  }
  return true;
}

// The short-query pipeline keeps both query tiles of a (batch, head) resident (heads of 64, no key mask).
bool bwd_short_queries(const wm_attn_args& a) {
  return a.head_dim == kHeadDim && a.key_mask == nullptr && a.q_len <= 2 * kTileM && a.q_heads == a.kv_heads && a.k_len <= 128 * kTileN;
}

size_t tc_attn_bwd_workspace(const wm_attn_args& a) {
  const size_t rows = static_cast<size_t>(a.batch) * a.q_heads * a.q_len;
  const size_t delta_bytes = ((rows + 63) / 64) * 64 * sizeof(float);
  return bwd_short_queries(a) ? delta_bytes : delta_bytes + rows * a.head_dim * sizeof(float);
}

// The key-stationary pipeline for one head size: one block per tile of 128 key slots.
template <int D>
int launch_bwd_key_tiles(const CUtensorMap& map_q, const CUtensorMap& map_k, const CUtensorMap& map_v,
                         const CUtensorMap& map_g, const wm_attn_args& a, const float* delta, float* dq_acc,
                         cudaStream_t stream) {
  constexpr size_t smem = sizeof(BwdShared<D>) + 1024;
  static_assert(smem <= 227 * 1024, "the key-stationary backward has outgrown the shared memory of a block");
  static std::atomic<bool> configured[kMaxDevices];
  const int status = allow_shared_memory(attn_bwd_tc_kernel<D>, configured, smem);
  if (status != WM_OK) return status;
  dim3 grid((a.k_len + kTileN - 1) / kTileN, a.kv_heads, a.batch);
  attn_bwd_tc_kernel<D><<<grid, BwdCfg<D>::kThreads, smem, stream>>>(map_q, map_k, map_v, map_g, a, delta, dq_acc, next_epoch());
  count_launch();
  return cuda_check(cudaGetLastError(), "attn_bwd_tc_kernel");
}

int tc_attn_bwd(const wm_attn_args& a, cudaStream_t stream) {
  const size_t need = tc_attn_bwd_workspace(a);
  if (a.workspace == nullptr || a.workspace_bytes < need)
    return fail(WM_EWORKSPACE, "attention backward needs %zu workspace bytes, got %zu", need, a.workspace_bytes);
  const size_t rows = static_cast<size_t>(a.batch) * a.q_heads * a.q_len;
  float* delta = static_cast<float*>(a.workspace);
  float* dq_acc = delta + ((rows + 63) / 64) * 64;
  CUtensorMap map_q, map_k, map_v, map_g;
  int status = make_map(&map_q, a.q, a.batch, a.q_heads, a.q_len, a.q_strides, kTileM, a.head_dim);
  if (status != WM_OK) return status;
  status = make_map(&map_k, a.k, a.batch, a.kv_heads, a.k_len, a.k_strides, kTileN, a.head_dim);
  if (status != WM_OK) return status;
  status = make_map(&map_v, a.v, a.batch, a.kv_heads, a.k_len, a.v_strides, kTileN, a.head_dim);
  if (status != WM_OK) return status;
  status = make_map(&map_g, a.dout, a.batch, a.q_heads, a.q_len, a.dout_strides, kTileM, a.head_dim);
  if (status != WM_OK) return status;
  if (a.head_dim == 64) bwd_delta_kernel<8, 8><<<static_cast<unsigned>((rows * 8 + 255) / 256), 256, 0, stream>>>(a, delta);
  else if (a.head_dim == 96) bwd_delta_kernel<12, 16><<<static_cast<unsigned>((rows * 16 + 255) / 256), 256, 0, stream>>>(a, delta);
  else bwd_delta_kernel<16, 16><<<static_cast<unsigned>((rows * 16 + 255) / 256), 256, 0, stream>>>(a, delta);
  count_launch();
  WM_CUDA(cudaGetLastError());
  if (bwd_short_queries(a)) {
    const size_t smem_r = sizeof(ResidentShared) + 1024;
    static std::atomic<bool> configured_r[kMaxDevices];
    status = allow_shared_memory(attn_bwd_resident_kernel, configured_r, smem_r);
    if (status != WM_OK) return status;
    CUtensorMap map_dk, map_dv;
    status = make_map(&map_dk, a.dk, a.batch, a.kv_heads, a.k_len, a.dk_strides, kTileN);
    if (status != WM_OK) return status;
    status = make_map(&map_dv, a.dv, a.batch, a.kv_heads, a.k_len, a.dv_strides, kTileN);
    if (status != WM_OK) return status;
    attn_bwd_resident_kernel<<<dim3(a.q_heads, a.batch), kResidentThreads, smem_r, stream>>>(map_q, map_k, map_v, map_g, map_dk,
                                                                                             map_dv, a, delta, next_epoch());
    count_launch();
    return cuda_check(cudaGetLastError(), "attention backward (tcgen05, resident queries)");
  }
  WM_CUDA(cudaMemsetAsync(dq_acc, 0, rows * a.head_dim * sizeof(float), stream));
  status = a.head_dim > 64 ? launch_bwd_key_tiles<128>(map_q, map_k, map_v, map_g, a, delta, dq_acc, stream)
                           : launch_bwd_key_tiles<64>(map_q, map_k, map_v, map_g, a, delta, dq_acc, stream);
  if (status != WM_OK) return status;
  const size_t chunks = rows * (a.head_dim / 8);
  bwd_dq_convert_kernel<<<static_cast<unsigned>((chunks + 255) / 256), 256, 0, stream>>>(a, dq_acc);
  count_launch();
  return cuda_check(cudaGetLastError(), "attention backward (tcgen05)");
}

}  // namespace wm
