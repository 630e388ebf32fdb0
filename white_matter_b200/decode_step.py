"""The decode step around the pool-read operator: a static KV pool in the upstream wire format, device-side
commits, and CUDA-graph replay.

Upstream keeps the shared KV channels of a feedback block in one static cache layer, keys and values of shape
``(B, k*HKV, capacity, D)``; a reader layer unflattens the head axis to ``(B, k, HKV, capacity, D)`` and attends to the
view of its channel (models/white_matter/modeling_white_matter.py:244-247), with the committed length kept on the
device so that the step can be replayed from a CUDA graph (models/cache.py:184-190, models/generation.py:38-100).
With packed documents the upstream FlashAttention reader first moves the visible slots to the front of a copy of the
whole pool (layers/backends.py:25-34, ``pack_kv_cache``: an argsort and a gather per token).

Here the pool is read in place: channel views are strided views of the pool (no copy), document visibility goes to the
kernel as ``key_mask``, new rows are committed by ``wm_pool_append`` at the device-resident lengths, and nothing on
the step synchronises the host.  PyTorch holds the memory and the graph; the kernels are the library's.
"""

from __future__ import annotations

from typing import Callable

import torch

from . import _native
from .strict import strict_causal_attention


class KVPoolCache:
    """Static pool ``(B, channels*kv_heads, capacity [+1 dummy slot], D)`` with per-sequence committed lengths.

    ``lengths`` (int32, on the device) counts real tokens and excludes the dummy slot, like the ``kv_lengths`` of
    the operators.  Rows beyond a sequence's length are unused capacity; they are never read and may hold anything.
    """

    def __init__(
        self,
        batch: int,
        channels: int,
        kv_heads: int,
        capacity: int,
        head_dim: int,
        *,
        use_dummy_token: bool = False,
        dtype: torch.dtype = torch.bfloat16,
        device: torch.device | str = "cuda",
    ) -> None:
        if min(batch, channels, kv_heads, capacity, head_dim) < 1:
            raise ValueError("pool sizes must be positive")
        self.channels, self.kv_heads, self.capacity = channels, kv_heads, capacity
        self.use_dummy_token = bool(use_dummy_token)
        slots = capacity + int(self.use_dummy_token)
        self.keys = torch.zeros(batch, channels * kv_heads, slots, head_dim, dtype=dtype, device=device)
        self.values = torch.zeros_like(self.keys)
        self.lengths = torch.zeros(batch, dtype=torch.int32, device=device)

    def channel(self, index: int) -> tuple[torch.Tensor, torch.Tensor]:
        """K and V of one shared channel as ``(B, kv_heads, slots, D)`` views of the pool (batch stride k*HKV*slots*D)."""
        if not 0 <= index < self.channels:
            raise ValueError(f"channel must be in [0, {self.channels})")
        heads = slice(index * self.kv_heads, (index + 1) * self.kv_heads)
        return self.keys[:, heads], self.values[:, heads]

    def set_dummy(self, key: torch.Tensor, value: torch.Tensor) -> None:
        """Slot 0 of every head: ``(channels*kv_heads, D)`` or broadcastable to ``(B, channels*kv_heads, D)``."""
        if not self.use_dummy_token:
            raise ValueError("this pool has no dummy slot")
        self.keys[:, :, 0].copy_(key)
        self.values[:, :, 0].copy_(value)

    def append(self, key: torch.Tensor, value: torch.Tensor, *, advance: bool = True) -> None:
        """Commit ``(B, channels*kv_heads, n, D)`` new rows behind each sequence's committed tokens.

        Device-side: the write positions come from ``lengths`` on the GPU, so the call can be captured in a CUDA
        graph and replayed while the lengths grow.  Rows that would not fit the capacity are dropped.
        """
        if key.shape != value.shape or key.ndim != 4 or key.shape[:2] != self.keys.shape[:2] or key.shape[3] != self.keys.shape[3]:
            raise ValueError("new rows must be (B, channels*kv_heads, n, D) for both K and V")
        if key.dtype != self.keys.dtype or key.device != self.keys.device:
            raise ValueError("new rows must have the pool's dtype and device")
        for pool, src in ((self.keys, key), (self.values, value)):
            if src.stride(-1) != 1:
                src = src.contiguous()
            a = _native.PoolAppendArgs()
            a.pool, a.src, a.lengths = pool.data_ptr(), src.data_ptr(), self.lengths.data_ptr()
            a.pool_strides, a.src_strides = _native.strides3(pool), _native.strides3(src)
            a.dtype = _native.dtype_code(pool.dtype)
            a.batch, a.heads, a.n_new, a.head_dim = src.shape
            a.capacity = pool.shape[2]
            a.lead = int(self.use_dummy_token)
            _native.call("wm_pool_append", a, pool.device)
        if advance:
            self.lengths.add_(key.shape[2]).clamp_(max=self.capacity)

    def read(
        self,
        query: torch.Tensor,
        channel: int,
        *,
        key_mask: torch.Tensor | None = None,
        softmax_scale: float | None = None,
    ) -> torch.Tensor:
        """Attention of ``(B, H, T, D)`` queries positioned behind the committed tokens over one channel: ``(B, T, H, D)``.

        One query token per sequence without gradients is the split-KV pool read; more tokens are a cached-prefix
        prefill (the new tokens' own K/V are not in the pool yet: the step commits them after its layer sweep, as
        upstream does).  ``key_mask`` (B, slots) carries document visibility and is consumed in place.
        """
        key, value = self.channel(channel)
        return strict_causal_attention(
            query, key, value, query_start=self.lengths, kv_lengths=self.lengths, use_dummy_token=self.use_dummy_token,
            key_mask=key_mask, softmax_scale=softmax_scale, static_cache=True,
        )


def document_key_mask(past_documents: torch.Tensor, current_documents: torch.Tensor, *, use_dummy_token: bool, slots: int) -> torch.Tensor:
    """(B, slots) visibility of the pool's slots for the token being decoded: committed tokens of its own document
    (negative ids are padding and see nothing), plus the dummy slot; unused capacity is invisible.  The rule of
    upstream modules/documents.py:61-64, laid out over the whole pool so that the kernel can take it as ``key_mask``."""
    batch, seen = past_documents.shape
    same = (past_documents == current_documents.view(batch, 1)) & (current_documents.view(batch, 1) >= 0)
    lead = int(use_dummy_token)
    keep = torch.zeros(batch, slots, dtype=torch.bool, device=past_documents.device)
    if lead:
        keep[:, 0] = True
    keep[:, lead : lead + seen] = same
    return keep


class DecodeStepGraph:
    """One decode step captured in a CUDA graph and replayed while the pool's lengths grow on the device.

    ``step()`` is the caller's function of no arguments (it reads its inputs from tensors it owns, e.g. the current
    queries, and typically calls ``KVPoolCache.read`` for every layer and ``KVPoolCache.append`` once); the tensor it
    returns is borrowed: the next replay overwrites it.  Replaying after pool buffers were replaced requires a new
    capture, as upstream's DecodeGraph (models/generation.py:38-100).
    """

    def __init__(self, step: Callable[[], torch.Tensor], cache: KVPoolCache, *, warmup: int = 2) -> None:
        if not cache.keys.is_cuda:
            raise ValueError("decode capture requires a CUDA pool")
        self.cache = cache
        self._buffers = (cache.keys, cache.values, cache.lengths)
        saved = cache.lengths.clone()
        stream = torch.cuda.Stream(device=cache.keys.device)
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            for _ in range(warmup):
                step()
                cache.lengths.copy_(saved)
        torch.cuda.current_stream().wait_stream(stream)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.output = step()
        cache.lengths.copy_(saved)  # capture runs nothing, but the warm-up steps advanced and restored the lengths

    def __call__(self) -> torch.Tensor:
        if any(a is not b for a, b in zip(self._buffers, (self.cache.keys, self.cache.values, self.cache.lengths))):
            raise ValueError("pool storage changed; capture the step again")
        self.graph.replay()
        return self.output
