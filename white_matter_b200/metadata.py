"""Document metadata of the attention operators (host-side schedule building).

The public names and tensor contents follow the upstream project so that a
caller can hand these objects to either implementation:

* ``CyclicAttentionMetadata`` / ``prepare_cyclic_attention_metadata`` --
  src/white_matter/ops/cyclic_attention/metadata.py:8-56
* ``prepare_feedback_metadata`` (the caller-side builder that turns token
  document ids into per-residue metadata) --
  src/white_matter/blocks/_execution/metadata.py:11-55
* ``StrictCausalMetadata`` / ``prepare_strict_causal_metadata`` --
  src/white_matter/ops/strict_causal_attention.py:36-155

Everything here is integer work done once per batch, outside layer and pass
loops; the kernels only consume the resulting device tables.
"""

from __future__ import annotations

from collections.abc import Sequence
from typing import NamedTuple

import numpy as np
import torch

_INT32_MAX = 2**31 - 1


class CyclicAttentionMetadata(NamedTuple):
    """Per-row document bounds for cyclic attention (all int32, (batch, length)).

    ``query_key_start`` is the first key slot of each query's document and
    ``key_query_end`` the exclusive upper query index that may see each key;
    the shared dummy slot (id -1) is outside these bounds.
    """

    query_document_ids: torch.Tensor
    key_document_ids: torch.Tensor
    query_key_start: torch.Tensor
    key_query_end: torch.Tensor


def _runs(row: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """First index of every run of equal values of a 1-D array, and the exclusive end of every run."""
    first = np.flatnonzero(np.concatenate(([True], row[1:] != row[:-1])))
    return first, np.append(first[1:], row.size)


def prepare_cyclic_attention_metadata(
    query_document_ids: torch.Tensor, key_document_ids: torch.Tensor, *, use_dummy_token: bool = True
) -> CyclicAttentionMetadata:
    """Bounds from sorted per-row document ids of queries and key slots.

    Same contract, checks and messages as upstream metadata.py:17-56: integer (batch, length) matrices, ids
    nondecreasing per row, nonnegative except for the leading dummy key (id -1) that must be present when
    ``use_dummy_token``; ids must fit int32.  The tables themselves are worked out on the host from the runs of
    equal ids (a row has a handful of documents, whatever its length): a query's first key is the first slot of the
    first key run whose id reaches the query's id, a key's query bound the end of the last query run whose id does
    not exceed the key's.
    """
    if query_document_ids.ndim != 2 or key_document_ids.ndim != 2:
        raise ValueError("segment IDs must have shape (batch, length)")
    if (
        query_document_ids.shape[0] != key_document_ids.shape[0]
        or min(*query_document_ids.shape, key_document_ids.shape[1]) < 1
    ):
        raise ValueError("segment IDs require matching nonempty batches and sequences")
    if query_document_ids.device != key_document_ids.device:
        raise ValueError("segment IDs must be on the same device")
    for ids in (query_document_ids, key_document_ids):
        if ids.dtype not in (torch.int32, torch.int64):
            raise ValueError("segment IDs must be int32 or int64")
    device = query_document_ids.device
    q_host = query_document_ids.detach().cpu().numpy().astype(np.int64)
    k_host = key_document_ids.detach().cpu().numpy().astype(np.int64)
    for ids in (q_host, k_host):
        if ids.max(initial=0) > _INT32_MAX:
            raise ValueError("segment IDs must fit int32 (maximum 2147483647)")
        if (np.diff(ids, axis=1) < 0).any():
            raise ValueError("segment IDs must be nondecreasing within each row")
    lead = int(use_dummy_token)
    if (q_host < 0).any() or (k_host[:, lead:] < 0).any():
        raise ValueError("only the leading key dummy may have a negative segment ID")
    if use_dummy_token and not (k_host[:, 0] == -1).all():
        raise ValueError("document attention requires a leading dummy key with segment ID -1")
    batch, n_q = q_host.shape
    n_k = k_host.shape[1]
    first_key = np.empty((batch, n_q), dtype=np.int32)
    query_end = np.empty((batch, n_k), dtype=np.int32)
    for b in range(batch):
        q_first, q_stop = _runs(q_host[b])
        k_first, k_stop = _runs(k_host[b])
        q_ids, k_ids = q_host[b][q_first], k_host[b][k_first]
        # per query run: the key run it starts at (the first one whose id is not smaller); behind the last run: n_k
        at = np.searchsorted(k_ids, q_ids, side="left")
        run_start = np.append(k_first, n_k)[at]
        first_key[b] = np.repeat(run_start, q_stop - q_first)
        # per key run: the query run it ends with (the last one whose id is not larger); in front of the first: 0
        upto = np.searchsorted(q_ids, k_ids, side="right")
        run_end = np.concatenate(([0], q_stop))[upto]
        query_end[b] = np.repeat(run_end, k_stop - k_first)
    if use_dummy_token:
        query_end[:, 0] = n_q
    return CyclicAttentionMetadata(
        query_document_ids.to(torch.int32).contiguous(),
        key_document_ids.to(torch.int32).contiguous(),
        torch.from_numpy(first_key).to(device),
        torch.from_numpy(query_end).to(device),
    )


def prepare_feedback_metadata(
    document_ids: torch.Tensor,
    query_positions: Sequence[torch.Tensor],
    key_length: int,
    *,
    use_dummy_token: bool = True,
) -> tuple[CyclicAttentionMetadata, ...]:
    """Per-residue metadata from token document ids (B,T); the tensors upstream
    blocks/_execution/metadata.py:11-55 builds.

    Group r holds the query tokens ``query_positions[r]`` (r, r+stride, ...).  With a dummy, key slot 0 is shared
    (-1) and slot s+1 stores token s; otherwise slot s stores token s.  Padding tokens (negative ids) become
    document -2.  A token's document is the run of equal ids it sits in: its queries start at the run's first slot,
    and a key is open to the queries of residue r that lie in front of its run's end, ceil((end - r) / stride) of
    them.
    """
    lead = int(use_dummy_token)
    stride = len(query_positions)
    if not stride:
        raise ValueError("cyclic query groups must be nonempty")
    batch, length = document_ids.shape
    if key_length > length + lead:
        raise ValueError(f"key_length={key_length} exceeds dummy-shifted token extent {length + lead}")
    device = document_ids.device
    ids = document_ids.detach().cpu().numpy().astype(np.int64)
    run_first = np.empty((batch, length), dtype=np.int64)  # first token of each token's run
    run_stop = np.empty((batch, length), dtype=np.int64)   # first token behind it
    for b in range(batch):
        first, stop = _runs(ids[b])
        run_first[b] = np.repeat(first, stop - first)
        run_stop[b] = np.repeat(stop, stop - first)
    labels = np.where(ids < 0, -2, ids).astype(np.int32)
    key_ids = np.concatenate((np.full((batch, lead), -1, dtype=np.int32), labels), axis=1)[:, :key_length]
    key_ids_t = torch.from_numpy(np.ascontiguousarray(key_ids)).to(device)
    result = []
    for residue, slots in enumerate(query_positions):
        at = slots.detach().cpu().numpy()
        count = at.size
        ends = np.clip(-(-(run_stop - residue) // stride), 0, count).astype(np.int32)
        query_end = np.concatenate((np.full((batch, lead), count, dtype=np.int32), ends), axis=1)[:, :key_length]
        result.append(
            CyclicAttentionMetadata(
                torch.from_numpy(np.ascontiguousarray(labels[:, at])).to(device),
                key_ids_t,
                torch.from_numpy((run_first[:, at] + lead).astype(np.int32)).to(device),
                torch.from_numpy(np.ascontiguousarray(query_end)).to(device),
            )
        )
    return tuple(result)


def _jacobi_tables(ids: np.ndarray, starts: np.ndarray, query_length: int, key_length: int, lead: int, device) -> CyclicAttentionMetadata:
    """The four document tables of a Jacobi schedule over ``query_length`` queries per row, query i of row b being the
    token at position starts[b] + i, against the row's key slots: labels are the ids of the present tokens (-3 for
    padded queries, -2 for padded keys, -1 for the dummy slot), a query starts at the first present slot of its run
    of equal ids among the present tokens, and a key is open to the queries up to its run's last token."""
    batch, length = ids.shape
    q_seg = np.full((batch, query_length), -3, dtype=np.int32)
    q_start = np.zeros((batch, query_length), dtype=np.int32)
    k_seg = np.full((batch, length), -2, dtype=np.int32)
    k_end = np.zeros((batch, length), dtype=np.int32)
    steps = np.arange(query_length, dtype=np.int64)
    for b in range(batch):
        present = ids[b] >= 0
        slots = np.flatnonzero(present)
        if not slots.size:
            continue
        labels = ids[b][slots]
        first, stop = _runs(labels)  # in ranks among the present tokens
        run = np.repeat(np.arange(first.size), stop - first)
        run_of_slot = np.zeros(length, dtype=np.int64)
        run_of_slot[slots] = run
        k_seg[b, slots] = labels
        k_end[b, slots] = np.clip(slots[stop - 1][run] + 1 - starts[b], 0, query_length)
        pos = starts[b] + steps
        live = present[pos]
        q_seg[b, live] = ids[b][pos[live]]
        q_start[b, live] = slots[first][run_of_slot[pos[live]]] + lead
    key_ids = np.concatenate((np.full((batch, lead), -1, dtype=np.int32), k_seg), axis=1)[:, :key_length]
    query_end = np.concatenate((np.full((batch, lead), query_length, dtype=np.int32), k_end), axis=1)[:, :key_length]
    as_device = lambda x: torch.from_numpy(np.ascontiguousarray(x)).to(device)
    return CyclicAttentionMetadata(as_device(q_seg), as_device(key_ids), as_device(q_start), as_device(query_end))


class StrictCausalMetadata:
    """Reusable packed schedule for strict-past attention over documents.

    ``query_indices`` lists the flat (batch*query_length) rows of the queries
    that see at least one key, ``key_indices`` the flat (batch*key_extent)
    slots of every group's keys; ``cu_queries`` / ``cu_keys`` (int32) delimit
    the groups.  Inside a group the last query sees all of the group's keys,
    the one before it one key fewer, and so on (bottom-right alignment).
    Field meaning follows strict_causal_attention.py:36-55.
    """

    __slots__ = (
        "query_indices",
        "key_indices",
        "cu_queries",
        "cu_keys",
        "max_queries",
        "max_keys",
        "key_extent",
        "segments",
        "dense_documents",
        "max_queries_per_row",
        "_cache",
    )

    def __init__(
        self,
        query_indices: torch.Tensor,
        key_indices: torch.Tensor,
        cu_queries: torch.Tensor,
        cu_keys: torch.Tensor,
        max_queries: int,
        max_keys: int,
        key_extent: int,
        segments: tuple[tuple[int, int, int, int], ...] = (),
    ) -> None:
        self.query_indices = query_indices
        self.key_indices = key_indices
        self.cu_queries = cu_queries
        self.cu_keys = cu_keys
        self.max_queries = max_queries
        self.max_keys = max_keys
        self.key_extent = key_extent
        if not segments and cu_queries.numel() > 1:
            q = cu_queries.tolist()
            k = cu_keys.tolist()
            segments = tuple(zip(q[:-1], q[1:], k[:-1], k[1:], strict=True))
        self.segments = segments
        # (document ids (B,T) int32, use_dummy_token, per-row first query position, per-row key limits or None) when
        # the schedule came from rows of document ids: it then equals strict-past attention with dense per-row
        # bounds plus document tables, which the tensor-core kernels take directly.
        self.dense_documents = None
        self.max_queries_per_row = 0
        self._cache: dict = {}

    def with_key_extent(self, key_extent: int) -> "StrictCausalMetadata":
        """The same key slots addressed in storage with another row width."""
        if key_extent == self.key_extent:
            return self
        cached = self._cache.get(("extent", key_extent))
        if cached is None:
            rows = torch.div(self.key_indices, self.key_extent, rounding_mode="floor")
            slots = self.key_indices - rows * self.key_extent
            cached = StrictCausalMetadata(
                self.query_indices,
                rows * key_extent + slots,
                self.cu_queries,
                self.cu_keys,
                self.max_queries,
                self.max_keys,
                key_extent,
                self.segments,
            )
            cached.dense_documents = self.dense_documents
            cached.max_queries_per_row = self.max_queries_per_row
            self._cache[("extent", key_extent)] = cached
        return cached

    def document_tables(self, device: torch.device, key_length: int) -> "CyclicAttentionMetadata | None":
        """The schedule as dense per-row bounds plus document tables (None when it was not built from whole rows of
        document ids): the form the tensor-core kernels take.  Query i of row b is the token at position start_b + i
        and sees the present slots of its run of equal ids in front of min(position, limit_b).  Padding slots
        (negative ids) become keys of a document no query has and queries of a document no key has; a run goes on
        across padding, as in the packed schedule."""
        if self.dense_documents is None:
            return None
        key = ("tables", str(device), key_length)
        cached = self._cache.get(key)
        if cached is None:
            docs, dummy, starts, _ = self.dense_documents
            cached = _jacobi_tables(docs.cpu().numpy().astype(np.int64), starts, self.max_queries_per_row, key_length, int(dummy), device)
            self._cache[key] = cached
        return cached

    def dense_bounds(self, device: torch.device):
        """(query_start int32 (B,) or None when every row starts at 0, kv_lengths int32 (B,) or None) on ``device``."""
        key = ("bounds", str(device))
        if key not in self._cache:
            _, _, starts, limits = self.dense_documents
            start_t = None if not starts.any() else torch.from_numpy(starts.astype(np.int32)).to(device)
            limit_t = None if limits is None else torch.from_numpy(limits.astype(np.int32)).to(device)
            self._cache[key] = (start_t, limit_t)
        return self._cache[key]

    def padded_queries(self, device: torch.device) -> "torch.Tensor | None":
        """(B,T) bool, True where the query token is padding (its result is zero), or None without padding."""
        if self.dense_documents is None:
            return None
        key = ("padding", str(device))
        if key not in self._cache:
            docs, _, starts, _ = self.dense_documents
            pos = torch.from_numpy(starts)[:, None] + torch.arange(self.max_queries_per_row)[None, :]
            pad = torch.gather(docs.cpu().long(), 1, pos) < 0
            self._cache[key] = pad.to(device) if bool(pad.any()) else None
        return self._cache[key]

    def device_tables(self, device: torch.device, q_rows: int, k_rows: int):
        """Device copies of the group table, index lists and tile tables.

        Built on first use for a tile shape and kept with the schedule, which
        callers prepare once and reuse over layers and Jacobi iterations.
        Returns (groups int32 (G,4), query_indices int64, key_indices int64,
        query_tiles int32 (Nq,2), key_tiles int32 (Nk,2)).
        """
        key = ("tables", str(device), q_rows, k_rows)
        cached = self._cache.get(key)
        if cached is None:
            groups = np.asarray(self.segments, dtype=np.int32).reshape(-1, 4)
            q_tiles = _cut_tiles(groups[:, 1] - groups[:, 0], q_rows)
            k_tiles = _cut_tiles(groups[:, 3] - groups[:, 2], k_rows)
            cached = (
                torch.from_numpy(groups).to(device),
                self.query_indices.to(device=device, dtype=torch.int64).contiguous(),
                self.key_indices.to(device=device, dtype=torch.int64).contiguous(),
                torch.from_numpy(q_tiles).to(device),
                torch.from_numpy(k_tiles).to(device),
            )
            self._cache[key] = cached
        return cached


def _cut_tiles(lengths: np.ndarray, rows: int) -> np.ndarray:
    """(n,2) table of (group, first row) for tiles of ``rows`` rows per group."""
    counts = (lengths + rows - 1) // rows
    groups = np.repeat(np.arange(lengths.shape[0], dtype=np.int32), counts)
    first_tile = np.cumsum(counts) - counts
    within = np.arange(groups.shape[0], dtype=np.int64) - np.repeat(first_tile, counts)
    return np.stack((groups, (within * rows).astype(np.int32)), axis=1).astype(np.int32).reshape(-1, 2)


def prepare_strict_causal_metadata(
    document_ids: torch.Tensor,
    query_length: int,
    *,
    query_start: int | torch.Tensor = 0,
    kv_lengths: torch.Tensor | None = None,
    use_dummy_token: bool = False,
) -> StrictCausalMetadata:
    """Pack document runs for strict-past attention; negative ids are padding.

    ``document_ids`` (B, extent) labels the real key slots, including the
    slots of the current queries and excluding the optional leading dummy.
    Query t of row b sits at real position ``query_start[b] + t`` and sees the
    earlier labelled slots of its own run that lie before ``kv_lengths[b]``.
    Padding neither ends a run nor is visible.  Build once, reuse across
    layers and Jacobi iterations.  Produces the same tensors as upstream
    strict_causal_attention.py:76-155.
    """
    batch, extent = document_ids.shape
    device = document_ids.device
    docs = document_ids.detach().cpu().numpy().astype(np.int64)
    if isinstance(query_start, torch.Tensor):
        starts = np.broadcast_to(query_start.detach().cpu().numpy().astype(np.int64), (batch,))
    else:
        starts = np.full((batch,), int(query_start), dtype=np.int64)
    limits = None if kv_lengths is None else kv_lengths.detach().cpu().numpy().astype(np.int64)
    steps = np.arange(query_length, dtype=np.int64)
    positions = starts[:, None] + steps[None, :]
    if positions.size and (positions.min() < 0 or positions.max() >= extent):
        raise ValueError("document_ids must label every query position")
    lead = int(use_dummy_token)
    width = extent + lead

    flat_queries: list[np.ndarray] = []
    run_of_query: list[np.ndarray] = []
    first_of_query: list[np.ndarray] = []
    end_of_query: list[np.ndarray] = []
    row_of_query: list[np.ndarray] = []
    row_slots: list[np.ndarray] = []
    runs_so_far = 0
    for b in range(batch):
        row = docs[b]
        present = row >= 0
        slots = np.flatnonzero(present)
        row_slots.append(slots)
        rank = np.concatenate(([0], np.cumsum(present)))  # labelled slots before slot s
        labels = row[slots]
        opens = np.ones(slots.shape[0], dtype=bool)
        opens[1:] = labels[1:] != labels[:-1]
        run_first = np.maximum.accumulate(np.where(opens, np.arange(slots.shape[0]), 0)) if slots.size else opens
        run_number = np.cumsum(opens) + runs_so_far
        runs_so_far += int(opens.sum())
        if not query_length:
            continue
        pos = positions[b]
        labelled = present[pos]
        own_rank = rank[pos]
        safe = np.minimum(own_rank, max(slots.shape[0] - 1, 0))
        first = np.where(labelled, run_first[safe] if slots.size else 0, 0)
        bound = pos if limits is None else np.minimum(pos, limits[b])
        end = rank[np.clip(bound, 0, extent)]
        valid = labelled & ((end > first) | use_dummy_token)
        chosen = np.flatnonzero(valid)
        flat_queries.append(b * query_length + chosen)
        run_of_query.append(run_number[safe[chosen]] if slots.size else chosen)
        first_of_query.append(first[chosen])
        end_of_query.append(end[chosen])
        row_of_query.append(np.full(chosen.shape[0], b, dtype=np.int64))

    def join(parts):
        return np.concatenate(parts) if parts else np.zeros((0,), dtype=np.int64)

    query_indices = join(flat_queries).astype(np.int64)
    total = query_indices.shape[0]
    if total == 0:
        empty = torch.zeros((0,), dtype=torch.int64, device=device)
        zero = torch.zeros((1,), dtype=torch.int32, device=device)
        return StrictCausalMetadata(empty, empty, zero, zero.clone(), query_length, width, width)
    runs = join(run_of_query)
    firsts = join(first_of_query)
    ends = join(end_of_query)
    rows = join(row_of_query)
    # a group continues while the run is unchanged and one more key becomes visible per query
    opens = np.ones(total, dtype=bool)
    opens[1:] = (runs[1:] != runs[:-1]) | (ends[1:] != ends[:-1] + 1)
    group_begin = np.flatnonzero(opens)
    cu_queries = np.concatenate((group_begin, [total])).astype(np.int64)
    last = cu_queries[1:] - 1
    g_first, g_end, g_row = firsts[last], ends[last], rows[last]
    real = np.maximum(g_end - g_first, 0)
    sizes = real + lead
    cu_keys = np.concatenate(([0], np.cumsum(sizes))).astype(np.int64)
    key_indices = np.empty((int(cu_keys[-1]),), dtype=np.int64)
    for n in range(group_begin.shape[0]):
        at = int(cu_keys[n])
        b = int(g_row[n])
        if lead:
            key_indices[at] = b * width
            at += 1
        chosen = row_slots[b][int(g_first[n]) : int(g_first[n]) + int(real[n])]
        key_indices[at : at + chosen.shape[0]] = b * width + chosen + lead
    schedule = StrictCausalMetadata(
        torch.from_numpy(query_indices).to(device),
        torch.from_numpy(key_indices).to(device),
        torch.from_numpy(cu_queries.astype(np.int32)).to(device),
        torch.from_numpy(cu_keys.astype(np.int32)).to(device),
        query_length,
        width,
        width,
    )
    if extent > 0 and query_length > 0 and int(np.abs(docs).max()) < 2**31 - 1:
        schedule.dense_documents = (document_ids.detach().to(torch.int32), bool(use_dummy_token), starts.copy(), None if limits is None else limits.copy())
        schedule.max_queries_per_row = query_length
    return schedule
