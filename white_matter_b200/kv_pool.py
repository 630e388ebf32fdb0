"""KV-pool projection path: layer stack -> shared K/V channels, for inference.

Host-side mirror of the upstream ``KVPool`` (src/white_matter/modules/kv_pool.py:36-226) with its routed mixer
(src/white_matter/modules/routing.py:45-122): same constructor arguments, parameter names and the two entry points
``project_sequence`` / ``project_token`` with their layouts.  The work is laid out differently:

* ``wm_pool_mix`` reads the (B,T,L,Dm) layer stack once and writes the normalised, gained mixtures that feed the
  projections; the upstream chain (rms_norm, two pre-mix products, two einsums, two rms_norms, two gains, two
  permutes) never exists as tensors.
* The dynamic router's logits are linear in the *raw* sources once the per-source norm is pulled out:
  ``logits = bias + sum_j rsqrt(mean(x_j^2)+eps) * (x_j @ (W_j * pre_mix_j)^T)``.  The bracket is one plain batched
  GEMM over the routed sources on the layer stack as it lies in memory (library call); the norms and the sum are
  applied inside ``wm_pool_mix``.
* The per-channel projections are plain batched GEMMs (library call); the post-mix gains are folded into their
  weights.
* ``wm_pool_finish`` applies the per-channel key norm and the rotary embedding and writes keys and values straight
  into their final layout -- a fresh (B,k,HKV,T,D) tensor or the slots of a decode cache -- which replaces the
  upstream permute/contiguous, norm, rotate_half chain and the index_copy publication
  (blocks/_execution/cyclic.py:406-424).

Token rows are processed in chunks of ``chunk_rows`` (default 16384) to bound the temporaries (routing partials,
mixtures, projections: about 75 KB per row at 25 sources of width 1024).  Smaller, L2-sized chunks were measured
slower on B200: the mixing kernel is bound by instruction issue, not by HBM, and more launches only add host time.

Only the routed mixer is built (the upstream default); gradients are not: the path serves prefill and decode.
"""

from __future__ import annotations

import torch

from . import _native

_STATE_NAMES = {
    "pre_mix_k_weight": "pre_mix_k_weight",
    "pre_mix_v_weight": "pre_mix_v_weight",
    "k_proj_weight": "k_proj_weight",
    "v_proj_weight": "v_proj_weight",
    "k_norm_weight": "k_norm_weight",
    "mixer.k_router.linear.weight": "k_router_weight",
    "mixer.k_router.linear.bias": "k_router_bias",
    "mixer.v_router.linear.weight": "v_router_weight",
    "mixer.v_router.linear.bias": "v_router_bias",
    "post_mix.k_gain": "k_gain",
    "post_mix.v_gain": "v_gain",
}


class KVPool:
    """Shared rank-k K/V channels built from every layer's input, as the upstream module of the same name.

    Parameters are plain FP32 tensors on ``device`` with the upstream shapes; ``load_state_dict`` accepts the
    upstream module's state dict.  After changing a parameter in place call ``refresh()``.
    """

    def __init__(
        self,
        hidden_size: int,
        num_key_value_heads: int,
        head_dim: int,
        num_layers: int,
        num_kv_channels: int,
        *,
        rms_norm_eps: float = 1e-6,
        initializer_range: float = 0.02,
        router_layer_stride: int = 1,
        router_dynamic: bool = True,
        device: torch.device | str = "cuda",
        dtype: torch.dtype = torch.bfloat16,
        chunk_rows: int = 16384,
    ) -> None:
        if not 1 <= num_kv_channels <= num_layers:
            raise ValueError(f"num_kv_channels must be in [1, {num_layers}], got {num_kv_channels}")
        if router_layer_stride < 1:
            raise ValueError("router_layer_stride must be positive")
        if type(router_dynamic) is not bool:
            raise ValueError("router_dynamic must be boolean")
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("the pool computes in bfloat16 or float32")
        self.hidden_size = hidden_size
        self.num_key_value_heads = num_key_value_heads
        self.head_dim = head_dim
        self.num_layers = num_layers
        self.num_kv_channels = num_kv_channels
        self.rms_norm_eps = float(rms_norm_eps)
        self.mix_norm_eps = 1.0e-4
        self.router_layer_stride = router_layer_stride
        self.router_dynamic = router_dynamic
        self.source_start = (num_layers - 1) % router_layer_stride
        self.num_sources = len(range(self.source_start, num_layers, router_layer_stride))
        self.device = torch.device(device)
        self.dtype = dtype
        self.chunk_rows = int(chunk_rows)
        kv_dim = num_key_value_heads * head_dim
        f32 = dict(device=self.device, dtype=torch.float32)
        self.pre_mix_k_weight = torch.ones(num_layers, hidden_size, **f32)
        self.pre_mix_v_weight = torch.ones(num_layers, hidden_size, **f32)
        self.k_gain = torch.ones(num_kv_channels, hidden_size, **f32)
        self.v_gain = torch.ones(num_kv_channels, hidden_size, **f32)
        self.k_proj_weight = torch.randn(num_kv_channels, kv_dim, hidden_size, **f32) * initializer_range
        self.v_proj_weight = torch.randn(num_kv_channels, kv_dim, hidden_size, **f32) * initializer_range
        self.k_norm_weight = torch.ones(num_kv_channels, head_dim, **f32)
        routed = self.num_sources * hidden_size
        self.k_router_weight = torch.zeros(num_kv_channels * num_layers, routed, **f32)
        self.v_router_weight = torch.zeros(num_kv_channels * num_layers, routed, **f32)
        self.k_router_bias = torch.zeros(num_kv_channels * num_layers, **f32)
        self.v_router_bias = torch.zeros(num_kv_channels * num_layers, **f32)
        self.refresh()

    # ------------------------------------------------------------------ parameters
    def load_state_dict(self, state: dict) -> None:
        """Take the parameters of an upstream ``KVPool.state_dict()`` (tensors or arrays)."""
        for upstream_name, name in _STATE_NAMES.items():
            value = torch.as_tensor(state[upstream_name]).to(device=self.device, dtype=torch.float32)
            target = getattr(self, name)
            if value.shape != target.shape:
                raise ValueError(f"{upstream_name}: expected {tuple(target.shape)}, got {tuple(value.shape)}")
            setattr(self, name, value.contiguous())
        self.refresh()

    def refresh(self) -> None:
        """Rebuild the GEMM operands derived from the parameters (call after changing one in place)."""
        k, layers, hidden = self.num_kv_channels, self.num_layers, self.hidden_size
        routed = slice(self.source_start, layers, self.router_layer_stride)

        def folded(weight: torch.Tensor, pre_mix: torch.Tensor) -> torch.Tensor:
            # (k*L, n*Dm) -> (n, Dm, k*L) with the routed sources' pre-mix gain folded in
            w = weight.view(k * layers, self.num_sources, hidden) * pre_mix[routed][None]
            return w.permute(1, 2, 0).to(self.dtype).contiguous()

        # K- and V-side router weights side by side: one GEMM over the routed sources yields both sides' partials
        self._route = torch.cat(
            (folded(self.k_router_weight, self.pre_mix_k_weight), folded(self.v_router_weight, self.pre_mix_v_weight)), dim=2
        ).contiguous()
        # the post-mix gain scales the columns of the projection's input: folded into the projection weights
        self._proj_k = (self.k_proj_weight * self.k_gain[:, None, :]).transpose(1, 2).to(self.dtype).contiguous()
        self._proj_v = (self.v_proj_weight * self.v_gain[:, None, :]).transpose(1, 2).to(self.dtype).contiguous()

    # ------------------------------------------------------------------ kernels
    def _check(self, stacked: torch.Tensor) -> None:
        if stacked.ndim != 4 or stacked.shape[2:] != (self.num_layers, self.hidden_size):
            raise ValueError(f"expected (*,*,{self.num_layers},{self.hidden_size}), got {tuple(stacked.shape)}")
        if not stacked.is_cuda:
            raise ValueError("the sm100 KV pool requires CUDA tensors")
        if stacked.dtype != self.dtype:
            raise ValueError(f"the pool was built for {self.dtype}, got {stacked.dtype}")
        if stacked.stride(3) != 1:
            raise ValueError("the layer stack must have unit stride in the hidden dimension")

    def _project_rows(self, stacked, cos, sin, keys, values, token_offset: int, rope_offset: int, slot_stride: int = 1) -> None:
        """Project every token of ``stacked`` (B,T,L,Dm) into slots token_offset.. of ``keys`` / ``values``
        (B, k*HKV, slots, D) views."""
        batch, tokens = stacked.shape[:2]
        k, hidden, layers = self.num_kv_channels, self.hidden_size, self.num_layers
        rows = batch * tokens
        device = stacked.device
        partial = None
        if self.router_dynamic:
            # (n, rows, Dm) view of the routed sources as they lie in the stack (callers pass rows one stride apart)
            routed = stacked[:, :, self.source_start :: self.router_layer_stride]
            flat = routed.reshape(rows, self.num_sources, hidden).transpose(0, 1)
            partial = torch.bmm(flat, self._route)  # (n, rows, 2*k*L): K side, then V side, in every row
        mixed = torch.empty(2, k, rows, hidden, device=device, dtype=self.dtype)
        a = _native.PoolMixArgs()
        a.stacked = stacked.data_ptr()
        a.stacked_strides = _native._Strides(stacked.stride(0), stacked.stride(1), stacked.stride(2))
        a.pre_mix_k, a.pre_mix_v = self.pre_mix_k_weight.data_ptr(), self.pre_mix_v_weight.data_ptr()
        a.bias_k, a.bias_v = self.k_router_bias.data_ptr(), self.v_router_bias.data_ptr()
        if partial is not None:
            a.partial_k = partial.data_ptr()
            a.partial_v = partial.data_ptr() + k * layers * partial.element_size()
            a.partial_row_stride = 2 * k * layers
            a.route_start, a.route_stride, a.n_routed = self.source_start, self.router_layer_stride, self.num_sources
        a.mixed_k, a.mixed_v = mixed[0].data_ptr(), mixed[1].data_ptr()
        a.dtype = _native.dtype_code(self.dtype)
        a.batch, a.tokens, a.sources, a.channels, a.hidden = batch, tokens, layers, k, hidden
        a.source_eps, a.mix_eps = self.rms_norm_eps, self.mix_norm_eps
        _native.call("wm_pool_mix", a, device)
        proj_k = torch.bmm(mixed[0], self._proj_k)
        proj_v = torch.bmm(mixed[1], self._proj_v)
        f = _native.PoolFinishArgs()
        f.k_proj, f.v_proj = proj_k.data_ptr(), proj_v.data_ptr()
        f.k_norm_weight = self.k_norm_weight.data_ptr()
        f.cos, f.sin = cos.data_ptr(), sin.data_ptr()
        f.k_out, f.v_out = keys.data_ptr(), values.data_ptr()
        f.cs_strides = (_native.ctypes.c_int64 * 2)(cos.stride(0) if cos.shape[0] > 1 else 0, cos.stride(1))
        f.out_strides = _native._Strides(keys.stride(0), keys.stride(1), keys.stride(2))
        f.in_dtype = f.out_dtype = _native.dtype_code(self.dtype)
        f.batch, f.tokens, f.channels = batch, tokens, k
        f.kv_heads, f.head_dim = self.num_key_value_heads, self.head_dim
        f.token_offset, f.rope_offset, f.slot_stride = token_offset, rope_offset, slot_stride
        f.eps = self.rms_norm_eps
        _native.call("wm_pool_finish", f, device)

    def _tables(self, position_embeddings, batch: int, rows: int):
        cos, sin = position_embeddings
        if cos.shape != sin.shape or cos.ndim != 3 or cos.shape[0] not in (1, batch) or cos.shape[1:] != (rows, self.head_dim):
            raise ValueError(f"position embeddings must be (B|1, {rows}, {self.head_dim})")
        cos = cos.to(device=self.device, dtype=torch.float32)
        sin = sin.to(device=self.device, dtype=torch.float32)
        if cos.stride(2) != 1:
            cos = cos.contiguous()
        if sin.stride() != cos.stride():
            sin = sin.contiguous()
            cos = cos.contiguous()
        return cos, sin

    # ------------------------------------------------------------------ entry points
    def project_into(
        self,
        stacked: torch.Tensor,
        position_embeddings: tuple[torch.Tensor, torch.Tensor],
        keys: torch.Tensor,
        values: torch.Tensor,
        *,
        token_offset: int = 0,
        slot_stride: int = 1,
    ) -> None:
        """Project (B,T,L,Dm) and publish row t into slot ``token_offset + t * slot_stride`` of a pool in the decode
        wire format: ``keys`` / ``values`` are (B, k*HKV, slots, D) with unit stride in D.  The position embeddings
        are (B|1, T, D), row t for the token that lands in that slot.  A slot stride above one publishes a residue
        group of a cyclic pass (tokens c, c+G, ...) in place."""
        self._check(stacked)
        batch, tokens = stacked.shape[:2]
        heads = self.num_kv_channels * self.num_key_value_heads
        for pool in (keys, values):
            if pool.ndim != 4 or pool.shape[0] != batch or pool.shape[1] != heads or pool.shape[3] != self.head_dim:
                raise ValueError(f"pool tensors must be ({batch}, {heads}, slots, {self.head_dim})")
            if token_offset < 0 or slot_stride < 1 or (tokens and pool.shape[2] <= token_offset + (tokens - 1) * slot_stride):
                raise ValueError("the projected rows do not fit the pool")
            if pool.dtype != self.dtype or pool.stride(3) != 1 or pool.device != stacked.device:
                raise ValueError("pool tensors must share the stack's device and dtype, with unit stride in head_dim")
        if keys.stride() != values.stride():
            raise ValueError("keys and values must share one layout")
        if not tokens:
            return
        cos, sin = self._tables(position_embeddings, batch, tokens)
        whole = batch * tokens <= self.chunk_rows and (batch == 1 or stacked.stride(0) == tokens * stacked.stride(1))
        if whole:
            self._project_rows(stacked, cos, sin, keys, values, token_offset, 0, slot_stride)
            return
        # one batch row at a time, so that a chunk's rows are one stride apart in the stack
        for b in range(batch):
            table = slice(b, b + 1) if cos.shape[0] > 1 else slice(0, 1)
            for start in range(0, tokens, self.chunk_rows):
                stop = min(tokens, start + self.chunk_rows)
                self._project_rows(
                    stacked[b : b + 1, start:stop], cos[table], sin[table], keys[b : b + 1], values[b : b + 1],
                    token_offset + start * slot_stride, start, slot_stride,
                )

    def project_sequence(
        self,
        stacked: torch.Tensor,
        position_embeddings: tuple[torch.Tensor, torch.Tensor],
        *,
        dummy_token: torch.Tensor | None = None,
    ) -> tuple[torch.Tensor, torch.Tensor]:
        """(B,T,L,Dm) -> keys, values (B, k, HKV, T', D), T' = T + 1 with a ``dummy_token`` whose projection
        takes slot 0 (the dummy vector stands in for every source); position embeddings are (B|1, T', D)."""
        self._check(stacked)
        batch, tokens = stacked.shape[:2]
        lead = int(dummy_token is not None)
        k, heads, dim = self.num_kv_channels, self.num_key_value_heads, self.head_dim
        keys = torch.empty(batch, k * heads, tokens + lead, dim, device=stacked.device, dtype=self.dtype)
        values = torch.empty_like(keys)
        cos, sin = self._tables(position_embeddings, batch, tokens + lead)
        if lead:
            # token-local path: the dummy row is projected by itself, every source reading the one vector
            row = dummy_token.to(device=stacked.device, dtype=self.dtype).reshape(1, 1, 1, self.hidden_size)
            row = row.expand(batch, 1, self.num_layers, self.hidden_size).contiguous()
            self._project_rows(row, cos[:, :1], sin[:, :1], keys, values, 0, 0)
        self.project_into(stacked, (cos[:, lead:], sin[:, lead:]), keys, values, token_offset=lead)
        shape = (batch, k, heads, tokens + lead, dim)
        return keys.view(shape), values.view(shape)

    def project_token(
        self,
        layer_hidden_inputs: list[torch.Tensor],
        position_embeddings: tuple[torch.Tensor, torch.Tensor],
    ) -> tuple[torch.Tensor, torch.Tensor]:
        """One decode row: L tensors (B,1,Dm) -> keys, values (k, B, HKV, 1, D)."""
        stacked = torch.stack(layer_hidden_inputs, dim=2)
        keys, values = self.project_sequence(stacked, position_embeddings)
        return keys.transpose(0, 1).contiguous(), values.transpose(0, 1).contiguous()
