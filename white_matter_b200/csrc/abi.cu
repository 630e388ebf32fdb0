// extern "C" entry points of libwm_b200: argument validation and kernel
// selection.  Nothing here allocates device memory or synchronises the host.
#include <atomic>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>

#include "common.cuh"
#include "wm_b200_debug.h"

namespace wm {

namespace {
thread_local char g_error[512] = "";
std::atomic<unsigned long long> g_launches{0};
}

void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

int cuda_check(cudaError_t status, const char* what) {
  if (status == cudaSuccess) return WM_OK;
  return fail(WM_ECUDA, "%s: %s", what, cudaGetErrorString(status));
}

int simt_tile_rows(int head_dim);

int validate_attn(const wm_attn_args* a, bool backward, const char* who) {
  if (a == nullptr) return fail(WM_EINVAL, "%s: null arguments", who);
  if (a->dtype != WM_F32 && a->dtype != WM_BF16) return fail(WM_EINVAL, "%s: dtype must be WM_F32 or WM_BF16", who);
  if (a->batch < 1 || a->q_heads < 1 || a->kv_heads < 1 || a->q_len < 1 || a->k_len < 1 || a->head_dim < 1)
    return fail(WM_EINVAL, "%s: sizes must be positive", who);
  if (a->q_heads % a->kv_heads) return fail(WM_EINVAL, "%s: q_heads must be a multiple of kv_heads", who);
  if (a->q == nullptr || a->k == nullptr || a->v == nullptr || a->out == nullptr)
    return fail(WM_EINVAL, "%s: q, k, v and out are required", who);
  if (backward) {
    if (a->dout == nullptr || a->dq == nullptr || a->dk == nullptr || a->dv == nullptr || a->lse == nullptr)
      return fail(WM_EINVAL, "%s: dout, dq, dk, dv and lse are required", who);
  }
  if (a->kernel < WM_KERNEL_AUTO || a->kernel > WM_KERNEL_TCGEN05)
    return fail(WM_EINVAL, "%s: unknown kernel selector %d", who, a->kernel);
  if (a->mask == WM_MASK_CYCLIC) {
    if (a->query_stride < 1) return fail(WM_EINVAL, "%s: query_stride must be a positive integer", who);
    if (a->query_offset < -1 || a->query_offset >= a->query_stride)
      return fail(WM_EINVAL, "%s: query_offset must be in [-1, query_stride)", who);
    if (static_cast<long long>(a->query_offset) + static_cast<long long>(a->query_stride) * (a->q_len - 1) >= a->k_len)
      return fail(WM_EINVAL, "%s: query slots must be within the key sequence", who);
    int have = (a->q_seg != nullptr) + (a->k_seg != nullptr) + (a->q_key_start != nullptr) + (a->k_query_end != nullptr);
    if (have != 0 && have != 4) return fail(WM_EINVAL, "%s: document metadata requires four tensors", who);
  } else if (a->mask == WM_MASK_STRICT) {
    if (a->use_dummy != 0 && a->use_dummy != 1) return fail(WM_EINVAL, "%s: use_dummy must be 0 or 1", who);
    int have = (a->q_seg != nullptr) + (a->k_seg != nullptr) + (a->q_key_start != nullptr) + (a->k_query_end != nullptr);
    if (have != 0 && have != 4) return fail(WM_EINVAL, "%s: document metadata requires four tensors", who);
    if (have != 0 && a->key_mask != nullptr) return fail(WM_EINVAL, "%s: document metadata and key_mask are mutually exclusive", who);
  } else if (a->mask == WM_MASK_PACKED) {
    if (a->n_groups < 0 || (a->n_groups > 0 && (a->groups == nullptr || a->query_indices == nullptr ||
                                                a->key_indices == nullptr || a->query_tiles == nullptr)))
      return fail(WM_EINVAL, "%s: packed schedule tables are missing", who);
    if (backward && a->n_groups > 0 && a->key_tiles == nullptr)
      return fail(WM_EINVAL, "%s: packed backward needs the key tile table", who);
    if (a->key_mask != nullptr || a->q_seg != nullptr) return fail(WM_EINVAL, "%s: packed schedules take no extra mask", who);
  } else {
    return fail(WM_EINVAL, "%s: unknown mask family %d", who, a->mask);
  }
  return WM_OK;
}

bool want_tc(const wm_attn_args* a) { return a->kernel != WM_KERNEL_SIMT; }

namespace {

int run_fwd(const wm_attn_args* a, void* stream, int family, bool docs, const char* who) {
  int status = validate_attn(a, false, who);
  if (status != WM_OK) return status;
  if (a->mask != family) return fail(WM_EINVAL, "%s: wrong mask family %d", who, a->mask);
  if (family == WM_MASK_CYCLIC && docs != (a->q_seg != nullptr))
    return fail(WM_EINVAL, "%s: document tensors %s", who, docs ? "are required" : "must be NULL");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (want_tc(a) && tc_fwd_supported(*a)) return tc_attn_fwd(*a, s);
  if (a->kernel == WM_KERNEL_TCGEN05) return fail(WM_EUNSUPPORTED, "%s: problem does not qualify for the tcgen05 kernel", who);
  return simt_attn_fwd(*a, s);
}

int run_bwd(const wm_attn_args* a, void* stream, int family, bool docs, const char* who) {
  int status = validate_attn(a, true, who);
  if (status != WM_OK) return status;
  if (a->mask != family) return fail(WM_EINVAL, "%s: wrong mask family %d", who, a->mask);
  if (family == WM_MASK_CYCLIC && docs != (a->q_seg != nullptr))
    return fail(WM_EINVAL, "%s: document tensors %s", who, docs ? "are required" : "must be NULL");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (want_tc(a) && tc_bwd_supported(*a)) return tc_attn_bwd(*a, s);
  if (a->kernel == WM_KERNEL_TCGEN05) return fail(WM_EUNSUPPORTED, "%s: problem does not qualify for the tcgen05 kernel", who);
  return simt_attn_bwd(*a, s);
}

}  // namespace
}  // namespace wm

extern "C" {

int wm_abi_version(void) { return WM_B200_ABI_VERSION; }

const char* wm_last_error(void) { return wm::g_error; }

int wm_debug_trace(long long* out, int capacity, int arm_after) {
  return wm::tc_debug_trace(out, capacity, arm_after);
}

int wm_debug_expire_wait(long long limit_ticks, void* stream) {
  return wm::tc_debug_expire_wait(limit_ticks, static_cast<cudaStream_t>(stream));
}

int wm_device_status(int reset) { return wm::tc_device_status(reset != 0); }

unsigned long long wm_kernel_launch_count(void) { return wm::g_launches.load(std::memory_order_relaxed); }

int wm_attn_tile_rows(const wm_attn_args* a, int backward, int key_side) {
  if (a == nullptr) return 0;
  (void)key_side;
  if (wm::want_tc(a) && (backward ? wm::tc_bwd_supported(*a) : wm::tc_fwd_supported(*a))) return 128;
  return wm::simt_tile_rows(a->head_dim);
}

size_t wm_attn_fwd_workspace_bytes(const wm_attn_args* a) {
  (void)a;
  return 0;
}

size_t wm_attn_bwd_workspace_bytes(const wm_attn_args* a) {
  if (a == nullptr) return 0;
  if (wm::want_tc(a) && wm::tc_bwd_supported(*a)) return wm::tc_attn_bwd_workspace(*a);
  return wm::simt_attn_bwd_workspace(*a);
}

size_t wm_strict_decode_workspace_bytes(const wm_attn_args* a) { return a ? wm::decode_workspace(*a) : 0; }

size_t wm_mix_workspace_bytes(const wm_mix_args* a) { return a ? wm::mix_workspace(*a) : 0; }

size_t wm_query_prepare_workspace_bytes(const wm_qprep_args* a) { return a ? wm::query_prepare_workspace(*a) : 0; }

int wm_cyclic_attn_fwd(const wm_attn_args* a, void* stream) {
  return wm::run_fwd(a, stream, WM_MASK_CYCLIC, false, "wm_cyclic_attn_fwd");
}
int wm_cyclic_attn_bwd(const wm_attn_args* a, void* stream) {
  return wm::run_bwd(a, stream, WM_MASK_CYCLIC, false, "wm_cyclic_attn_bwd");
}
int wm_cyclic_attn_doc_fwd(const wm_attn_args* a, void* stream) {
  return wm::run_fwd(a, stream, WM_MASK_CYCLIC, true, "wm_cyclic_attn_doc_fwd");
}
int wm_cyclic_attn_doc_bwd(const wm_attn_args* a, void* stream) {
  return wm::run_bwd(a, stream, WM_MASK_CYCLIC, true, "wm_cyclic_attn_doc_bwd");
}
int wm_strict_attn_fwd(const wm_attn_args* a, void* stream) {
  return wm::run_fwd(a, stream, WM_MASK_STRICT, false, "wm_strict_attn_fwd");
}
int wm_strict_attn_bwd(const wm_attn_args* a, void* stream) {
  return wm::run_bwd(a, stream, WM_MASK_STRICT, false, "wm_strict_attn_bwd");
}
int wm_strict_packed_fwd(const wm_attn_args* a, void* stream) {
  return wm::run_fwd(a, stream, WM_MASK_PACKED, false, "wm_strict_packed_fwd");
}
int wm_strict_packed_bwd(const wm_attn_args* a, void* stream) {
  return wm::run_bwd(a, stream, WM_MASK_PACKED, false, "wm_strict_packed_bwd");
}

int wm_strict_decode(const wm_attn_args* a, void* stream) {
  int status = wm::validate_attn(a, false, "wm_strict_decode");
  if (status != WM_OK) return status;
  if (a->mask != WM_MASK_STRICT || a->q_len != 1)
    return wm::fail(WM_EINVAL, "wm_strict_decode: needs the strict mask family and a single query token");
  if (!wm::decode_supported(*a))
    return wm::fail(WM_EUNSUPPORTED,
                    "wm_strict_decode: head_dim must be a multiple of 16 bytes and all rows 16-byte aligned");
  return wm::decode_launch(*a, static_cast<cudaStream_t>(stream));
}

int wm_strict_decode_no_alloc(const wm_attn_args* a, void* stream) {
  int status = wm::validate_attn(a, false, "wm_strict_decode_no_alloc");
  if (status != WM_OK) return status;
  if (a->mask != WM_MASK_STRICT || a->q_len != 1)
    return wm::fail(WM_EINVAL, "wm_strict_decode_no_alloc: needs the strict mask family and a single query token");
  if (!wm::decode_supported(*a))
    return wm::fail(WM_EUNSUPPORTED,
                    "wm_strict_decode_no_alloc: head_dim must be a multiple of 16 bytes and all rows 16-byte aligned");
  const size_t need = wm::decode_workspace(*a);
  if (need > wm::decode_static_capacity())
    return wm::fail(WM_EWORKSPACE,
                    "wm_strict_decode_no_alloc: this problem needs %zu bytes of split scratch, the built-in array holds "
                    "%zu; use wm_strict_decode with caller scratch",
                    need, wm::decode_static_capacity());
  float* scratch = nullptr;
  status = wm::decode_static_scratch(&scratch);
  if (status != WM_OK) return status;
  return wm::decode_launch_with_scratch(*a, scratch, static_cast<cudaStream_t>(stream));
}

int wm_strict_decode_mixed(const wm_attn_args* a, const wm_source_mix* mix, void* stream) {
  if (mix == nullptr) return wm::fail(WM_EINVAL, "wm_strict_decode_mixed: null mixture");
  int status = wm::validate_attn(a, false, "wm_strict_decode_mixed");
  if (status != WM_OK) return status;
  if (!wm::decode_supported(*a)) return wm::fail(WM_EUNSUPPORTED, "wm_strict_decode_mixed: needs one query, the strict mask and 16-byte aligned rows");
  return wm::decode_mixed_launch(*a, *mix, static_cast<cudaStream_t>(stream));
}

int wm_pool_append(const wm_pool_append_args* a, void* stream) {
  if (a == nullptr) return wm::fail(WM_EINVAL, "wm_pool_append: null arguments");
  return wm::pool_append_launch(*a, static_cast<cudaStream_t>(stream));
}

int wm_pool_mix(const wm_pool_mix_args* a, void* stream) {
  if (a == nullptr) return wm::fail(WM_EINVAL, "wm_pool_mix: null arguments");
  return wm::pool_mix_launch(*a, static_cast<cudaStream_t>(stream));
}

int wm_pool_finish(const wm_pool_finish_args* a, void* stream) {
  if (a == nullptr) return wm::fail(WM_EINVAL, "wm_pool_finish: null arguments");
  return wm::pool_finish_launch(*a, static_cast<cudaStream_t>(stream));
}

int wm_mix_sources_fwd(const wm_mix_args* a, void* stream) {
  if (a == nullptr) return wm::fail(WM_EINVAL, "wm_mix_sources_fwd: null arguments");
  return wm::mix_fwd_launch(*a, static_cast<cudaStream_t>(stream));
}

int wm_mix_sources_bwd(const wm_mix_args* a, void* stream) {
  if (a == nullptr) return wm::fail(WM_EINVAL, "wm_mix_sources_bwd: null arguments");
  return wm::mix_bwd_launch(*a, static_cast<cudaStream_t>(stream));
}

int wm_query_prepare_fwd(const wm_qprep_args* a, void* stream) {
  if (a == nullptr) return wm::fail(WM_EINVAL, "wm_query_prepare_fwd: null arguments");
  return wm::query_prepare(*a, false, static_cast<cudaStream_t>(stream));
}

int wm_query_prepare_bwd(const wm_qprep_args* a, void* stream) {
  if (a == nullptr) return wm::fail(WM_EINVAL, "wm_query_prepare_bwd: null arguments");
  return wm::query_prepare(*a, true, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
