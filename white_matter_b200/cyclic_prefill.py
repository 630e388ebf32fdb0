"""Cyclic prefill of a feedback block: the pass driver around the operators, for inference.

Host-side mirror of the upstream ``WhiteMatterBlock`` forward (src/white_matter/blocks/_execution/cyclic.py:111-268
``forward_cyclic``, :271-442 ``run_pass``, :464-489 ``_group_layers``; layer sweep blocks/decoder_layer.py:72-94;
attention layer layers/white_matter.py:86-199; RoPE positions blocks/white_matter.py:62-77) for the case the
prefill benchmark runs: no gradients, no padding, more tokens than residue groups.  One pass walks the residue
groups c = 0..G-1 (tokens c, c+G, ...); a group sweeps all layers, layer i reading K/V channel i mod k of the pool
through ``cyclic_attention`` with ``query_stride=G, query_offset=c``; the group's layer inputs (and the top
output) are then projected by the KV pool and published into the pool's slots of those tokens, so that later
groups read the refreshed rows.

What runs where: the linear layers, the SwiGLU product and the RMS norms of the hidden width are library calls
(plain GEMMs and pointwise kernels); query norm + rotary embedding + layout (``wm_query_prepare``), the attention
(``wm_cyclic_attn*``), the pool mixing (``wm_pool_mix``) and the publication into the strided slots of the group
(``wm_pool_finish`` with a slot stride) are this library's kernels.  The pool is kept in the decode wire format
(B, k*HKV, T[+1], D); channel c is a strided view of it, read in place.  The residual sums of a layer ride in the
epilogues of its two output GEMMs; every layer input is copied once into the (B, Tc, L+1, Dm) stack the pool reads.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from .cyclic import cyclic_attention
from .kv_pool import KVPool
from .layer import prepare_queries
from .metadata import prepare_feedback_metadata


class FeedbackBlock:
    """Layers + KV pool + rotary frequencies of a feedback region, with the upstream parameter names.

    ``load_state_dict`` takes the state dict of an upstream ``WhiteMatterBlock`` built from
    ``FeedbackDecoderLayer(WhiteMatterAttention, GatedMLP)`` layers over a routed ``KVPool`` with
    ``include_top_output=True`` (the pool has one source more than there are layers).
    """

    def __init__(
        self,
        hidden_size: int,
        num_layers: int,
        num_attention_heads: int,
        head_dim: int,
        intermediate_size: int,
        num_key_value_heads: int,
        num_kv_channels: int,
        *,
        rope_theta: float = 1_000_000.0,
        rms_norm_eps: float = 1e-6,
        use_dummy_token: bool = False,
        router_layer_stride: int = 2,
        router_dynamic: bool = True,
        num_passes: int = 3,
        initializer_range: float = 0.02,
        device: torch.device | str = "cuda",
        dtype: torch.dtype = torch.bfloat16,
    ) -> None:
        if type(use_dummy_token) is not bool:
            raise ValueError("use_dummy_token must be boolean")
        self.hidden_size, self.num_layers = hidden_size, num_layers
        self.num_attention_heads, self.head_dim = num_attention_heads, head_dim
        self.intermediate_size = intermediate_size
        self.num_kv_channels = num_kv_channels
        self.rope_theta, self.rms_norm_eps = float(rope_theta), float(rms_norm_eps)
        self.use_dummy_token = use_dummy_token
        self.num_passes = num_passes
        self.device, self.dtype = torch.device(device), dtype
        self.kv_pool = KVPool(
            hidden_size, num_key_value_heads, head_dim, num_layers + 1, num_kv_channels, rms_norm_eps=rms_norm_eps,
            initializer_range=initializer_range, router_layer_stride=router_layer_stride, router_dynamic=router_dynamic,
            device=device, dtype=dtype,
        )
        make = lambda *shape: (torch.randn(*shape, device=self.device) * initializer_range).to(dtype)
        ones = lambda n: torch.ones(n, device=self.device, dtype=dtype)
        width = num_attention_heads * head_dim
        self.layers = [
            {
                "input_layernorm": ones(hidden_size), "post_attention_layernorm": ones(hidden_size),
                "q_proj": make(width, hidden_size), "q_norm": ones(head_dim), "o_proj": make(hidden_size, width),
                "gate_proj": make(intermediate_size, hidden_size), "up_proj": make(intermediate_size, hidden_size),
                "down_proj": make(hidden_size, intermediate_size),
            }
            for _ in range(num_layers)
        ]
        self.dummy_token = torch.zeros(hidden_size, device=self.device, dtype=dtype) if use_dummy_token else None

    _LAYER_NAMES = {
        "input_layernorm.weight": "input_layernorm", "post_attention_layernorm.weight": "post_attention_layernorm",
        "self_attn.q_proj.weight": "q_proj", "self_attn.q_norm.weight": "q_norm", "self_attn.o_proj.weight": "o_proj",
        "mlp.gate_proj.weight": "gate_proj", "mlp.up_proj.weight": "up_proj", "mlp.down_proj.weight": "down_proj",
    }

    def load_state_dict(self, state: dict) -> None:
        """Take the parameters of an upstream ``WhiteMatterBlock.state_dict()`` (tensors or arrays)."""
        for index, layer in enumerate(self.layers):
            for upstream, name in self._LAYER_NAMES.items():
                value = torch.as_tensor(state[f"layers.{index}.{upstream}"]).to(device=self.device, dtype=self.dtype)
                if value.shape != layer[name].shape:
                    raise ValueError(f"layers.{index}.{upstream}: expected {tuple(layer[name].shape)}, got {tuple(value.shape)}")
                layer[name] = value.contiguous()
        prefix = "kv_pool."
        self.kv_pool.load_state_dict({k[len(prefix):]: v for k, v in state.items() if k.startswith(prefix)})
        if self.use_dummy_token:
            self.dummy_token = torch.as_tensor(state["dummy_token"]).to(device=self.device, dtype=self.dtype).contiguous()

    # ------------------------------------------------------------------ pieces
    def _rope(self, positions: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """cos, sin (B|1, N, D) in FP32 for integer positions (B|1, N) (modules/rotary.py:56-80)."""
        exponent = torch.arange(0, self.head_dim, 2, device=self.device, dtype=torch.float32) / self.head_dim
        inverse = 1.0 / (self.rope_theta ** exponent)
        angles = positions.to(torch.float32)[..., None] * inverse
        angles = torch.cat((angles, angles), dim=-1)
        return angles.cos(), angles.sin()

    def _positions(self, batch: int, tokens: int, document_ids: torch.Tensor | None):
        """Query and key positions (blocks/white_matter.py:62-77): real positions follow the optional dummy slot and
        restart at every document."""
        lead = int(self.use_dummy_token)
        if document_ids is None:
            q_pos = torch.arange(lead, tokens + lead, device=self.device)[None]
            k_pos = torch.arange(tokens + lead, device=self.device)[None]
            return q_pos, k_pos
        ids = document_ids.to(self.device)
        slots = torch.arange(tokens, device=self.device).expand_as(ids)
        starts = torch.ones_like(ids, dtype=torch.bool)
        starts[:, 1:] = ids[:, 1:] != ids[:, :-1]
        first = torch.where(starts, slots, 0).cummax(dim=1).values
        q_pos = slots - first + lead
        k_pos = torch.cat((q_pos.new_zeros(batch, lead), q_pos), dim=1)
        return q_pos, k_pos

    def _layer(self, layer: dict, hidden: torch.Tensor, keys, values, cos, sin, groups, residue, metadata) -> torch.Tensor:
        """One decoder layer on a residue group: hidden + attention + MLP (decoder_layer.py:46-69); ``hidden`` is
        (B, Tc, Dm) contiguous and so is the result."""
        eps = self.rms_norm_eps
        normed = F.rms_norm(hidden, (self.hidden_size,), layer["input_layernorm"], eps)
        projected = F.linear(normed, layer["q_proj"])
        queries = prepare_queries(
            projected, layer["q_norm"], cos, sin, eps=eps, head_dim=self.head_dim,
            out_dtype=torch.bfloat16 if self.dtype == torch.bfloat16 else None,
        )
        attended = cyclic_attention(
            queries, keys, values, query_stride=groups, query_offset=residue, strict_past=not self.use_dummy_token, metadata=metadata
        )
        batch, heads, length, dim = attended.shape
        rows = batch * length
        attended = attended.transpose(1, 2).reshape(rows, heads * dim)  # a view of the (B,T,H,D) storage
        # the residual sums ride in the GEMM epilogues (addmm)
        after = torch.addmm(hidden.view(rows, self.hidden_size), attended, layer["o_proj"].t())
        normed = F.rms_norm(after, (self.hidden_size,), layer["post_attention_layernorm"], eps)
        gated = F.silu(F.linear(normed, layer["gate_proj"])) * F.linear(normed, layer["up_proj"])
        return torch.addmm(after, gated, layer["down_proj"].t()).view(batch, length, self.hidden_size)

    # ------------------------------------------------------------------ entry point
    @torch.no_grad()
    def forward(
        self,
        x: torch.Tensor,
        *,
        num_passes: int | None = None,
        cyclic_groups: int = 8,
        document_ids: torch.Tensor | None = None,
        output_final_state: bool = False,
    ):
        """Cyclic passes over strided token groups, refreshing the pool after each group.

        ``x`` is (B,T,Dm) on the GPU in the block's dtype with T > cyclic_groups.  Returns ``(hidden, state)``:
        hidden (B,T,Dm) after the last pass and, with ``output_final_state``, the pool as keys, values
        (B, k, HKV, T[+1], D); ``None`` otherwise.
        """
        passes = self.num_passes if num_passes is None else num_passes
        if type(passes) is not int or passes < 1:
            raise ValueError("num_passes must be a positive integer")
        if type(cyclic_groups) is not int or cyclic_groups < 1:
            raise ValueError("cyclic_groups must be a positive integer")
        if x.ndim != 3 or x.shape[1] < 1 or x.shape[2] != self.hidden_size:
            raise ValueError("inputs must have a nonempty batch/sequence/hidden layout")
        if not x.is_cuda or x.dtype != self.dtype:
            raise ValueError(f"the block was built for CUDA tensors in {self.dtype}")
        batch, tokens, hidden_size = x.shape
        groups = cyclic_groups
        if tokens <= groups:
            raise ValueError("cyclic prefill here needs more tokens than residue groups (the padded short-sequence path is not built)")
        lead = int(self.use_dummy_token)
        sources = self.num_layers + 1
        k, kv_heads, dim = self.num_kv_channels, self.kv_pool.num_key_value_heads, self.head_dim

        q_pos, k_pos = self._positions(batch, tokens, document_ids)
        q_cos, q_sin = (t.to(self.dtype) for t in self._rope(q_pos))  # the query kernel reads tables in the stack's dtype
        k_cos, k_sin = self._rope(k_pos)
        metadata = None
        if document_ids is not None:
            slots = [torch.arange(c, tokens, groups) for c in range(groups)]
            metadata = prepare_feedback_metadata(document_ids.to(self.device), slots, tokens, use_dummy_token=self.use_dummy_token)

        # the pool in the decode wire format; the first fill reads the embeddings as every source
        keys = torch.empty(batch, k * kv_heads, tokens + lead, dim, device=x.device, dtype=self.dtype)
        values = torch.empty_like(keys)
        if lead:
            row = self.dummy_token.reshape(1, 1, 1, hidden_size).expand(batch, 1, sources, hidden_size).contiguous()
            self.kv_pool.project_into(row, (k_cos[:, :1], k_sin[:, :1]), keys, values, token_offset=0)
        self.kv_pool.project_into(
            x.unsqueeze(2).expand(batch, tokens, sources, hidden_size), (k_cos[:, lead:], k_sin[:, lead:]), keys, values, token_offset=lead
        )
        channel_keys = [keys[:, c * kv_heads : (c + 1) * kv_heads, :tokens] for c in range(k)]
        channel_values = [values[:, c * kv_heads : (c + 1) * kv_heads, :tokens] for c in range(k)]

        output = torch.empty_like(x)
        for p in range(passes):
            last = p == passes - 1
            for c in range(groups):
                group = x[:, c::groups]
                length = group.shape[1]
                stack = torch.empty(batch, length, sources, hidden_size, device=x.device, dtype=self.dtype)
                hidden = group.contiguous()
                cos, sin = q_cos[:, c::groups], q_sin[:, c::groups]
                for index, layer in enumerate(self.layers):
                    stack[:, :, index].copy_(hidden)  # the layer's input is a source of the pool
                    channel = index % k
                    hidden = self._layer(
                        layer, hidden, channel_keys[channel], channel_values[channel], cos, sin, groups, c,
                        None if metadata is None else metadata[c],
                    )
                stack[:, :, self.num_layers].copy_(hidden)
                if last:
                    output[:, c::groups] = hidden
                # publish after the layer sweep: later groups read these refreshed rows
                self.kv_pool.project_into(
                    stack, (k_cos[:, c + lead :: groups], k_sin[:, c + lead :: groups]), keys, values,
                    token_offset=c + lead, slot_stride=groups,
                )
        if not output_final_state:
            return output, None
        shape = (batch, k, kv_heads, tokens + lead, dim)
        return output, (keys.view(shape), values.view(shape))

    __call__ = forward
