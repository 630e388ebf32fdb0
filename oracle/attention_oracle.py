"""CPU oracle for the WhiteMatter attention hot path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this module;
only the tests, the smoke check and the CPU-baseline leg of the benchmark do.

It restates, in plain PyTorch CPU tensor arithmetic, the algorithm of the
upstream portable backend:

* cyclic attention             -- src/white_matter/ops/cyclic_attention/reference.py:10-42
  (argument shift for strict_past: functional.py:59)
* strict-causal attention      -- src/white_matter/ops/strict_causal_attention.py:279-322
  (dense path :299-322, packed-document path :279-298)
* per-query independent oracle -- tests/unit/test_strict_causal_attention.py:16-39
* KV source mixing             -- softmax-weighted mixture of already projected
  source tensors; upstream has no function of exactly this shape, the static
  softmax form follows src/white_matter/blocks/feedback_transformer.py:35-36.

Parity pin: every function here is checked against the upstream package
imported in the build container (tests/golden/make_golden.py writes the
fixtures under tests/golden/, and tests/test_oracle.py replays them), and
against the known-answer values that the upstream unit tests hold.

Everything is computed with an explicit mask, an explicit soft-max and two
matrix products, in ``compute_dtype`` (float64 by default), so that the result
does not depend on which fused kernel a PyTorch build selects.
"""

from __future__ import annotations

import math

import torch


# --------------------------------------------------------------------------- masks


def cyclic_keep_mask(q_len, k_len, query_stride, query_offset, metadata=None, strict_past=False):
    """Boolean visibility (B or 1, Q, K) of key slot j for query i.

    reference.py:20-30.  ``query_offset`` is the public argument; strict_past
    lowers it by one (functional.py:59).
    """
    offset = query_offset - int(strict_past)
    q_slots = offset + query_stride * torch.arange(q_len)
    k_slots = torch.arange(k_len)
    keep = (q_slots[:, None] >= k_slots[None, :])[None]
    if metadata is not None:
        q_seg, k_seg, q_start, k_end = (t.cpu().long() for t in metadata)
        shared = (k_seg == -1)[:, None, :]
        same = (q_seg[:, :, None] == k_seg[:, None, :]) | shared
        after = (k_slots.view(1, 1, k_len) >= q_start[:, :, None]) | shared
        before = torch.arange(q_len).view(1, q_len, 1) < k_end[:, None, :]
        keep = keep & same & after & before
    return keep


def strict_dense_keep_mask(batch, q_len, n_slots, query_start, kv_lengths, use_dummy_token, key_mask=None):
    """Visibility (B, Q, N) for the un-packed strict path.

    strict_causal_attention.py:299-308: slot s-offset is a real token index;
    it is visible when it is smaller than the query's real position and than
    kv_lengths; the dummy slot 0 is always visible; key_mask removes slots.
    """
    offset = int(use_dummy_token)
    if isinstance(query_start, torch.Tensor):
        starts = query_start.cpu().long().expand(batch)
    else:
        starts = torch.full((batch,), int(query_start), dtype=torch.long)
    qpos = starts[:, None] + torch.arange(q_len)
    slots = torch.arange(n_slots) - offset
    keep = slots[None, None, :] < qpos[:, :, None]
    if kv_lengths is not None:
        keep = keep & (slots[None, None, :] < kv_lengths.cpu().long()[:, None, None])
    if use_dummy_token:
        keep[..., 0] = True
    if key_mask is not None:
        keep = keep & key_mask.cpu()[:, None, :]
    return keep


# --------------------------------------------------------------------------- core


def masked_attention(query, key, value, keep, scale, compute_dtype=torch.float64):
    """softmax(scale * Q K^T restricted to ``keep``) V with grouped heads.

    query (B,HQ,Q,D); key/value (B,HKV,K,D); keep broadcastable to (B,1,Q,K).
    Rows without any visible key give exactly zero.  Returns (B,HQ,Q,D) in
    ``compute_dtype``; differentiable.
    """
    batch, heads, q_len, dim = query.shape
    groups = heads // key.shape[1]
    q = query.to(compute_dtype)
    k = key.to(compute_dtype).repeat_interleave(groups, dim=1)
    v = value.to(compute_dtype).repeat_interleave(groups, dim=1)
    keep = keep.to(query.device)
    if keep.ndim == 3:
        keep = keep[:, None]
    # NaN/Inf stored in never-visible slots must not reach a product.
    visible = keep.any(dim=-2).any(dim=1)  # (B or 1, K)
    visible = visible.expand(batch, -1)[:, None, :, None]
    k = torch.where(visible, k, torch.zeros((), dtype=compute_dtype))
    v = torch.where(visible, v, torch.zeros((), dtype=compute_dtype))
    scores = (q @ k.transpose(-1, -2)) * scale
    scores = scores.masked_fill(~keep, -math.inf)
    top = scores.amax(dim=-1, keepdim=True)
    top = torch.where(torch.isfinite(top), top, torch.zeros_like(top))
    weights = torch.exp(scores - top)
    total = weights.sum(dim=-1, keepdim=True)
    weights = weights / torch.where(total > 0, total, torch.ones_like(total))
    return weights @ v


def cyclic_attention_oracle(
    query,
    key,
    value,
    *,
    query_stride=1,
    query_offset=0,
    strict_past=False,
    metadata=None,
    compute_dtype=torch.float64,
):
    """(B,HQ,Q,D) result of cyclic attention; reference.py:10-42."""
    keep = cyclic_keep_mask(query.shape[-2], key.shape[-2], query_stride, query_offset, metadata, strict_past)
    return masked_attention(query, key, value, keep, query.shape[-1] ** -0.5, compute_dtype)


def strict_causal_oracle(
    query,
    key,
    value,
    *,
    query_start=0,
    kv_lengths=None,
    use_dummy_token=False,
    metadata=None,
    key_mask=None,
    softmax_scale=None,
    compute_dtype=torch.float64,
):
    """(B,T,H,D) result of strict-past attention.

    Dense path: strict_causal_attention.py:299-322.  Packed path (:279-298):
    every schedule group (qs,qe,ks,ke) attends with bottom-right alignment,
    query r of the group sees the group's keys c <= (ke-ks) - (qe-qs) + r;
    queries that the schedule does not list give zero.
    """
    batch, heads, length, dim = query.shape
    scale = dim**-0.5 if softmax_scale is None else softmax_scale
    if metadata is None:
        keep = strict_dense_keep_mask(
            batch, length, key.shape[-2], query_start, kv_lengths, use_dummy_token, key_mask
        )
        return masked_attention(query, key, value, keep, scale, compute_dtype).transpose(1, 2)
    extent = key.shape[-2]
    key_rows = torch.div(metadata.key_indices, metadata.key_extent, rounding_mode="floor")
    key_slots = metadata.key_indices - key_rows * metadata.key_extent
    key_indices = key_rows * extent + key_slots
    q = query.transpose(1, 2).flatten(0, 1)
    k = key.transpose(1, 2).flatten(0, 1)
    v = value.transpose(1, 2).flatten(0, 1)
    rows = []
    targets = []
    cu_q = metadata.cu_queries.tolist()
    cu_k = metadata.cu_keys.tolist()
    for qs, qe, ks, ke in zip(cu_q[:-1], cu_q[1:], cu_k[:-1], cu_k[1:]):
        nq, nk = qe - qs, ke - ks
        keep = torch.arange(nk)[None, :] <= (nk - nq + torch.arange(nq))[:, None]
        qi = metadata.query_indices[qs:qe]
        ki = key_indices[ks:ke]
        part = masked_attention(
            q[qi].transpose(0, 1)[None], k[ki].transpose(0, 1)[None], v[ki].transpose(0, 1)[None], keep[None], scale,
            compute_dtype,
        )
        rows.append(part[0].transpose(0, 1))
        targets.append(qi)
    output = torch.zeros(batch * length, heads, dim, dtype=compute_dtype)
    if rows:
        output = output.index_copy(0, torch.cat(targets), torch.cat(rows))
    return output.view(batch, length, heads, dim)


def strict_per_query_oracle(query, key, value, starts, use_dummy_token, documents=None, lengths=None):
    """Per-query explicit soft-max, independent of any packing.

    Restates tests/unit/test_strict_causal_attention.py:16-39: query i of row b
    sits at real position starts[b]+i and sees the real slots before it (and
    before lengths[b]); with ``documents`` only the slots of its own document
    run, where negative labels are padding that neither ends a run nor is seen.
    Returns (B,T,H,D) float64.
    """
    batch, heads, count, dim = query.shape
    groups = heads // key.shape[1]
    offset = int(use_dummy_token)
    out = torch.zeros(batch, count, heads, dim, dtype=torch.float64)
    for b in range(batch):
        for i in range(count):
            pos = int(starts[b]) + i
            bound = min(pos, key.shape[-2] - offset)
            if lengths is not None:
                bound = min(bound, int(lengths[b]))
            slots = list(range(max(bound, 0)))
            labelled = True
            if documents is not None:
                labelled = bool(documents[b, pos] >= 0)
                first = pos
                while first and (documents[b, first - 1] < 0 or documents[b, first - 1] == documents[b, pos]):
                    first -= 1
                slots = [s for s in slots if s >= first and documents[b, s] >= 0 and labelled]
            chosen = ([0] if use_dummy_token and labelled else []) + [s + offset for s in slots]
            if not chosen:
                continue
            kk = key[b][:, chosen].double().repeat_interleave(groups, 0)
            vv = value[b][:, chosen].double().repeat_interleave(groups, 0)
            weights = torch.softmax((query[b, :, i, None].double() * kk).sum(-1) * dim**-0.5, dim=-1)
            out[b, i] = (weights[..., None] * vv).sum(-2)
    return out


# --------------------------------------------------------------------------- mixing


def mix_sources_oracle(sources, logits, compute_dtype=torch.float64):
    """Softmax-weighted mixture over the leading source axis.

    sources (S, ...), logits (S,): sum_s softmax(logits)[s] * sources[s],
    the static soft-max mixture of feedback_transformer.py:35-36 applied to
    already projected K or V sources.
    """
    weights = torch.softmax(logits.to(compute_dtype), dim=0)
    return torch.einsum("s,s...->...", weights, sources.to(compute_dtype))


# --------------------------------------------------------------------------- FLOP convention


def visible_pairs(keep, heads):
    """Number of (query,key) pairs that a mask keeps, summed over batch and heads."""
    return int(keep.sum().item()) * heads // (1 if keep.ndim == 3 else keep.shape[1])
