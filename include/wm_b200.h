/*
 * wm_b200.h -- C ABI of the B200 (sm_100a) attention kernels for WhiteMatter.
 *
 * Every entry point takes plain device pointers, sizes and element strides and
 * a CUDA stream handle; no framework types cross this boundary.  All launches
 * are asynchronous on `stream`; nothing here synchronises the host, allocates
 * device memory or mutates an input.  Scratch memory is supplied by the caller
 * (`workspace`, size from the matching *_workspace_bytes query).
 *
 * Return value: 0 on success, a negative WM_E* code otherwise; the text of the
 * last failure on the calling thread is available from wm_last_error().
 *
 * The entry points stand in for these operators of the upstream project
 * (paths relative to the upstream repository root):
 *
 *   wm_cyclic_attn_fwd      white_matter::cyclic_attn_fwd
 *                           src/white_matter/ops/cyclic_attention/_tilelang/registration.py:164-173
 *   wm_cyclic_attn_bwd      white_matter::cyclic_attn_bwd            registration.py:184-197
 *   wm_cyclic_attn_doc_fwd  white_matter::cyclic_attn_doc_fwd        registration.py:261-274
 *   wm_cyclic_attn_doc_bwd  white_matter::cyclic_attn_doc_bwd        registration.py:280-296
 *   wm_strict_attn_fwd/bwd  the dense branch of strict_causal_attention
 *                           src/white_matter/ops/strict_causal_attention.py:299-322,432-458
 *   wm_strict_packed_fwd/bwd  the packed-document branch (varlen FlashAttention
 *                           call with gather/scatter) strict_causal_attention.py:397-431
 *   wm_strict_decode        white_matter::flash_attention_decode / torch_flash_decode
 *                           src/white_matter/ops/flash_attention.py:15-36,52-103
 *   wm_mix_sources_fwd/bwd  the mixture step of the KV pool
 *                           src/white_matter/modules/routing.py:116-122,
 *                           src/white_matter/blocks/feedback_transformer.py:35-36
 */
#ifndef WM_B200_H
#define WM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define WM_B200_ABI_VERSION 1

#if defined(__GNUC__)
#define WM_API __attribute__((visibility("default")))
#else
#define WM_API
#endif

/* element types */
#define WM_F32 0
#define WM_BF16 1

/* error codes */
#define WM_OK 0
#define WM_EINVAL (-1)     /* argument rejected before any launch */
#define WM_EUNSUPPORTED (-2) /* shape / type outside what the kernels cover */
#define WM_ECUDA (-3)      /* a CUDA runtime call failed */
#define WM_EWORKSPACE (-4) /* workspace missing or too small */

/* mask families (wm_attn_args.mask) */
#define WM_MASK_CYCLIC 0 /* query i sees key slots j <= query_offset + query_stride*i */
#define WM_MASK_STRICT 1 /* query at real position p sees real slots s < min(p, kv_length) (+ dummy slot 0) */
#define WM_MASK_PACKED 2 /* schedule groups with bottom-right causal alignment */

/* kernel family selection (wm_attn_args.kernel) */
#define WM_KERNEL_AUTO 0   /* tensor-core kernel when the problem qualifies, else the SIMT kernel */
#define WM_KERNEL_SIMT 1   /* force the fp32-accumulate SIMT kernel (all types and head sizes) */
#define WM_KERNEL_TCGEN05 2 /* force the tcgen05/TMEM kernel; WM_EUNSUPPORTED if the problem does not qualify */

/*
 * One description of an attention problem, shared by all attention entry
 * points.  Fields an entry point does not use must be zero / NULL.
 *
 * Tensors are (batch, heads, tokens, head_dim) with unit stride in head_dim;
 * the three strides are in ELEMENTS for batch, head and token.  The output is
 * addressed the same way, so the caller chooses (B,T,H,D) or (B,H,T,D) storage.
 */
typedef struct wm_attn_args {
  /* forward operands */
  const void* q;
  const void* k;
  const void* v;
  void* out;  /* forward: written; backward: read (the forward result) */
  float* lse; /* (batch, q_heads, q_len) contiguous; natural-log sum-exp of the scaled scores, +inf for empty rows */
  /* backward operands */
  const void* dout;
  void* dq;
  void* dk;
  void* dv;
  int64_t q_strides[3];
  int64_t k_strides[3];
  int64_t v_strides[3];
  int64_t out_strides[3];
  int64_t dout_strides[3];
  int64_t dq_strides[3];
  int64_t dk_strides[3];
  int64_t dv_strides[3];
  /* scratch supplied by the caller */
  void* workspace;
  size_t workspace_bytes;
  /* sizes */
  int32_t dtype; /* WM_F32 or WM_BF16, common to q/k/v/out and gradients */
  int32_t batch;
  int32_t q_heads;
  int32_t kv_heads; /* q_heads % kv_heads == 0 */
  int32_t q_len;
  int32_t k_len; /* number of key slots addressed (cache capacity for the strict family) */
  int32_t head_dim;
  float scale;
  int32_t mask;
  int32_t kernel;
  /* WM_MASK_CYCLIC */
  int32_t query_stride;
  int32_t query_offset; /* already lowered by one for strict_past; may be -1 */
  /* document tables: WM_MASK_CYCLIC, and WM_MASK_STRICT on top of its dense bounds (cached-prefix Jacobi) */
  const int32_t* q_seg;       /* (batch, q_len) document of each query, or NULL */
  const int32_t* k_seg;       /* (batch, k_len) document of each key slot; -1 marks the shared dummy */
  const int32_t* q_key_start; /* (batch, q_len) first key slot of the query's document */
  const int32_t* k_query_end; /* (batch, k_len) exclusive upper query bound of each key */
  /* WM_MASK_STRICT: device-resident bounds (either may be NULL) */
  const void* query_start; /* (batch,) int32 or int64 real position of the first query */
  const void* kv_lengths;  /* (batch,) int32 or int64 number of committed real tokens */
  int32_t query_start_is64;
  int32_t kv_lengths_is64;
  int64_t query_start_value; /* used when query_start == NULL */
  const uint8_t* key_mask;   /* (batch, k_len) 0/1, or NULL */
  int32_t use_dummy;         /* slot 0 is the always-visible dummy */
  /* WM_MASK_PACKED */
  int32_t n_groups;
  const int32_t* groups;        /* (n_groups, 4): query begin, query end, key begin, key end in the packed lists */
  const int64_t* query_indices; /* flat (batch*q_len) row of each packed query */
  const int64_t* key_indices;   /* flat (batch*k_len) slot of each packed key */
  /* Tile tables for packed problems: (n, 2) rows of {group, first row of the tile
   * relative to the group}, cut every wm_attn_tile_rows() rows. */
  int32_t n_query_tiles;
  const int32_t* query_tiles;
  int32_t n_key_tiles; /* backward only */
  const int32_t* key_tiles;
} wm_attn_args;

/* Mixture of S source tensors of n elements each: out = sum_s softmax(logits)[s] * src[s]. */
typedef struct wm_mix_args {
  const void* sources;    /* (n_sources, n) */
  int64_t source_stride;  /* elements between consecutive sources */
  const float* logits;    /* (n_sources,) fp32, device */
  void* out;              /* (n,) forward result */
  const void* dout;       /* (n,) backward input */
  void* dsources;         /* (n_sources, n) backward result, same stride as sources; may be NULL */
  float* dlogits;         /* (n_sources,) fp32 backward result; may be NULL */
  void* workspace;
  size_t workspace_bytes;
  int64_t n;
  int32_t n_sources; /* 1..64 */
  int32_t dtype;
} wm_mix_args;

/* K and V of a decode read given as stacks of sources that are mixed while they are read: source s of K lies
 * k_source_stride elements after args->k and enters with weight softmax(k_logits)[s]; likewise V. */
typedef struct wm_source_mix {
  const float* k_logits; /* (n_sources,) fp32, device */
  const float* v_logits;
  int64_t k_source_stride;
  int64_t v_source_stride;
  int32_t n_sources; /* 1..64 */
} wm_source_mix;

/* Query preparation of the attention layer (layers/white_matter.py:105-111 of the reference: q_norm, transpose,
 * rotary embedding): q[b,h,t,:] = rope(rms_norm(x[b,t,h,:]) * weight).  x has element strides x_strides for
 * (batch, token, head) and unit stride in head_dim; q is contiguous (batch, heads, tokens, head_dim); cos / sin are
 * (batch, tokens, head_dim) with element strides cs_strides (a batch stride of 0 broadcasts one table).  weight, cos
 * and sin have the dtype of x.  The backward call reads dq (layout of q) and writes dx (strides of x) and dweight. */
typedef struct wm_qprep_args {
  const void* x;
  const void* weight; /* (head_dim,) */
  const void* cos;
  const void* sin;
  void* q;            /* forward result */
  const void* dq;     /* backward input */
  void* dx;           /* backward result */
  void* dweight;      /* backward result, (head_dim,) in the dtype of x */
  void* workspace;    /* backward only: wm_query_prepare_workspace_bytes */
  size_t workspace_bytes;
  int64_t x_strides[3];
  int64_t cs_strides[2];
  int32_t dtype;   /* of x, weight, cos, sin, dx, dweight */
  int32_t q_dtype; /* of q and dq: WM_BF16, or WM_F32 when dtype is WM_F32 */
  int32_t batch, tokens, heads, head_dim; /* head_dim 64 or 128 */
  float eps;
} wm_qprep_args;

/* Source mixing of the KV pool (modules/kv_pool.py:97-146 and modules/routing.py:82-122 of the reference: the part
 * of KVPool._project before the per-channel projections).  For every token row it normalises each of the
 * `sources` layer inputs (RMS, source_eps), applies the K- and V-side pre-mix gains, mixes them into `channels`
 * vectors per side with signed routing logits, normalises each mixture (RMS, mix_eps) and applies the post-mix
 * gain -- one read of the layer stack and one write of the projection inputs instead of the reference's chain of
 * full-size temporaries:
 *
 *   n[l]   = x[l] * rsqrt(mean(x[l]^2) + source_eps)
 *   a[c,l] = bias[c*sources + l] + sum_j partial[j, row, c*sources + l] * rsqrt(mean(x[s_j]^2) + source_eps)
 *   h[c]   = sum_l a[c,l] * pre_mix[l] * n[l]
 *   out[c, row] = h[c] * rsqrt(mean(h[c]^2) + mix_eps) * gain[c]          (gain = 1 when gain_k / gain_v are NULL:
 *                                                                          a caller may fold it into the projection)
 *
 * with s_j = route_start + j * route_stride the sources the router reads.  `partial` carries the content-dependent
 * part of the logits, not yet scaled by the sources' norms: partial[j] = x[s_j] @ (router_weight[:, j] *
 * pre_mix[s_j])^T, one plain GEMM per routed source that the caller runs on the raw layer stack; n_routed = 0 (or
 * NULL partials) gives the static router whose logits are the bias alone.  `stacked` is (batch, tokens, sources,
 * hidden) with element strides for (batch, token, source) and unit stride in hidden; the partials are
 * (n_routed, batch*tokens, channels*sources) with partial_row_stride elements between rows (so that one GEMM
 * against the K- and V-side router weights side by side can produce both, partial_v = partial_k + channels*sources); the results are (channels, batch*tokens, hidden)
 * contiguous, the A operand of the per-channel projection.  stacked, partials and results share `dtype`; gains,
 * biases are float32.  hidden must be a multiple of 128 and at most 2048; sources at most 32. */
typedef struct wm_pool_mix_args {
  const void* stacked;
  int64_t stacked_strides[3];
  const float* pre_mix_k; /* (sources, hidden) */
  const float* pre_mix_v;
  const float* bias_k; /* (channels * sources,) */
  const float* bias_v;
  const void* partial_k; /* NULL for a static router */
  const void* partial_v;
  const float* gain_k; /* (channels, hidden), or both NULL */
  const float* gain_v;
  void* mixed_k;
  void* mixed_v;
  int32_t dtype;
  int32_t batch, tokens, sources, channels, hidden;
  int32_t route_start, route_stride, n_routed;
  float source_eps, mix_eps;
  int64_t partial_row_stride; /* elements between consecutive rows of a partial; 0 stands for channels*sources */
} wm_pool_mix_args;

/* Publication of projected channels into the KV pool (modules/kv_pool.py:147-176 of the reference: the permute of
 * the projected channels, the per-channel key norm and the rotary embedding; blocks/_execution/cyclic.py:406-424:
 * the copy into the pool).  `k_proj` and `v_proj` are the per-channel projections (channels, batch*tokens,
 * kv_heads*head_dim) contiguous in `in_dtype`.  Keys get rms_norm(eps) over head_dim, the channel's gain
 * k_norm_weight[c] and the rotary embedding of row rope_offset + t of cos / sin; values are moved unchanged.  Both
 * land at slot token_offset + t * slot_stride of head c*kv_heads + h of `k_out` / `v_out`, which are (batch, channels*kv_heads,
 * capacity, head_dim) in `out_dtype` with element strides out_strides for (batch, head, slot) -- the wire format of
 * the decode cache, or a fresh (batch, channels, kv_heads, tokens, head_dim) tensor.  cos / sin are float32
 * (batch, >= rope_offset + tokens, head_dim) with element strides cs_strides for (batch, row); a batch stride of 0
 * broadcasts one table. */
typedef struct wm_pool_finish_args {
  const void* k_proj;
  const void* v_proj;
  const float* k_norm_weight; /* (channels, head_dim) */
  const float* cos;
  const float* sin;
  void* k_out;
  void* v_out;
  int64_t cs_strides[2];
  int64_t out_strides[3];
  int32_t in_dtype, out_dtype;
  int32_t batch, tokens, channels, kv_heads, head_dim; /* head_dim 64 or 128 */
  int32_t token_offset, rope_offset;
  float eps;
  int32_t slot_stride; /* token t lands at slot token_offset + t * slot_stride; 0 stands for 1 */
} wm_pool_finish_args;

/* Commit of new tokens to a static KV pool (models/cache.py:43-60 of the reference: the update of a static cache
 * layer, an index_copy_ at the layer's running length): row (b, h, i) of `src` goes to slot
 * lengths[b] + lead + i of `pool`, for i < n_new; rows whose slot would lie beyond `capacity` are dropped.  `pool`
 * is (batch, heads, capacity, head_dim), `src` (batch, heads, n_new, head_dim), both with unit stride in head_dim and
 * element strides for (batch, head, token); head_dim * element size must be a multiple of 16 bytes and all rows
 * 16-byte aligned.  The lengths stay on the device and are not changed by the call. */
typedef struct wm_pool_append_args {
  void* pool;
  const void* src;
  const int32_t* lengths; /* (batch,) committed real tokens per sequence */
  int64_t pool_strides[3];
  int64_t src_strides[3];
  int32_t dtype;
  int32_t batch, heads, capacity, n_new, head_dim;
  int32_t lead; /* 1 when slot 0 is the shared dummy */
} wm_pool_append_args;

WM_API int wm_abi_version(void);
WM_API const char* wm_last_error(void);
/* Status word of the pipelined kernels on the current device: 0 when every bounded
 * wait inside them completed, else the first wait that gave up: its code in the low byte,
 * the linear index of its block in the bits above.  Synchronises the device; reset != 0
 * clears the word. */
WM_API int wm_device_status(int reset);
/* Number of kernels this library has launched in the process so far (diagnostic). */
WM_API unsigned long long wm_kernel_launch_count(void);

/* Rows per tile that the kernel selected for `args` cuts packed groups into
 * (queries when key_side == 0, keys otherwise; backward != 0 for the gradient kernels). */
WM_API int wm_attn_tile_rows(const wm_attn_args* args, int backward, int key_side);

/* Scratch sizes for the calls below (bytes, may be 0). */
WM_API size_t wm_attn_fwd_workspace_bytes(const wm_attn_args* args);
WM_API size_t wm_attn_bwd_workspace_bytes(const wm_attn_args* args);
WM_API size_t wm_strict_decode_workspace_bytes(const wm_attn_args* args);
WM_API size_t wm_mix_workspace_bytes(const wm_mix_args* args);
WM_API size_t wm_query_prepare_workspace_bytes(const wm_qprep_args* args);

/* cyclic attention without / with document metadata */
WM_API int wm_cyclic_attn_fwd(const wm_attn_args* args, void* stream);
WM_API int wm_cyclic_attn_bwd(const wm_attn_args* args, void* stream);
WM_API int wm_cyclic_attn_doc_fwd(const wm_attn_args* args, void* stream);
WM_API int wm_cyclic_attn_doc_bwd(const wm_attn_args* args, void* stream);

/* strict-past attention: dense bounds (Jacobi without documents, cached-prefix prefill) */
WM_API int wm_strict_attn_fwd(const wm_attn_args* args, void* stream);
WM_API int wm_strict_attn_bwd(const wm_attn_args* args, void* stream);
/* strict-past attention over a packed-document schedule */
WM_API int wm_strict_packed_fwd(const wm_attn_args* args, void* stream);
WM_API int wm_strict_packed_bwd(const wm_attn_args* args, void* stream);
/* single-query read of a KV pool, split over the key axis; lengths stay on the device */
WM_API int wm_strict_decode(const wm_attn_args* args, void* stream);

/*
 * wm_strict_decode for callers that have no device allocator to lend: same arguments and result, but
 * `workspace` is ignored and the split partials go to a 16 MiB array built into the library (held on every
 * GPU that loads it, until the process exits).  No counterpart in the upstream project.
 * Meant for hosts that were handed their device buffers and can pass pointers but not allocate -- a serving
 * process that carved all of HBM into its KV pool at start-up, or a thin foreign-language binding.
 * - Problems whose partials exceed the array (wm_strict_decode_workspace_bytes > 16 MiB) are rejected with
 *   WM_EWORKSPACE; nothing is launched.
 * - The first call on each device looks up the array's device address (that device must be current); make
 *   that first call outside any stream capture.
 * - All calls share the one array and it keeps the previous call's contents.  Nothing in it has to start at
 *   zero (every partial that is read was written by the same call), but two calls that overlap on the GPU
 *   (different streams) race on it: keep such calls on one stream or order them yourself.
 * - Calls no cudaMalloc / cudaFree and no allocating library routine.
 */
WM_API int wm_strict_decode_no_alloc(const wm_attn_args* args, void* stream);

/*
 * wm_strict_decode over K/V that are soft-max mixtures of stacked sources (the learned KV source mixing of
 * blocks/feedback_transformer.py:35-36 of the reference, applied to projected sources), with the mixture formed in
 * the K/V load path: every visible row of every source is read once and nothing is materialised.  A single-query
 * read touches each K/V row once, so this is the place where mixing on the fly saves traffic (the write and
 * re-read of the mixture); the same arguments, workspace and result as wm_strict_decode.
 */
WM_API int wm_strict_decode_mixed(const wm_attn_args* args, const wm_source_mix* mix, void* stream);

/* commit of new K or V rows to a static pool at device-resident lengths */
WM_API int wm_pool_append(const wm_pool_append_args* args, void* stream);

/* KV-pool projection path either side of its per-channel GEMMs */
WM_API int wm_pool_mix(const wm_pool_mix_args* args, void* stream);
WM_API int wm_pool_finish(const wm_pool_finish_args* args, void* stream);

/* KV source mixing */
WM_API int wm_mix_sources_fwd(const wm_mix_args* args, void* stream);
WM_API int wm_mix_sources_bwd(const wm_mix_args* args, void* stream);

/* the step in front of the attention operators inside the attention layer: q_norm, rotary embedding, layout change */
WM_API int wm_query_prepare_fwd(const wm_qprep_args* args, void* stream);
WM_API int wm_query_prepare_bwd(const wm_qprep_args* args, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* WM_B200_H */
