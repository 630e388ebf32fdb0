"""CPU oracle for the KV-pool projection path: layer stack -> shared K/V channels.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this module; only the tests do.

Restates the upstream pool written out per channel, the way tests/unit/test_paper_equations.py:15-41 of the upstream
project states it, for src/white_matter/modules/kv_pool.py:97-176 (``KVPool._project`` and ``_apply_k_norm_rope``)
with the dense router of src/white_matter/modules/routing.py:82-122:

    source  = rms_norm(states, eps) * pre_mix_weight[side]                       # kv_pool.py:104-127
    context = source[:, :, start::stride].flatten(2)                             # routing.py:98-99
    logits  = linear(context, router_weight, router_bias) -> (B, T, k, L)        # routing.py:100 (bias alone when static)
    mixed   = sum_l logits[..., c, l] * source[..., l, :]                        # routing.py:118-121
    mixed   = rms_norm(mixed, 1e-4) * post_mix_gain[side][c]                     # kv_pool.py:134-142
    proj    = mixed @ proj_weight[side][c].T -> (B, HKV, T, D)                   # kv_pool.py:144-161
    keys    = rope(rms_norm(proj, eps) * k_norm_weight[c])                       # kv_pool.py:163-176

and the leading dummy row of ``project_sequence`` (kv_pool.py:207-210: the dummy vector stands in for every source).
Everything is evaluated in ``compute_dtype`` (float64 by default); the upstream's BF16 round trips are not restated.

Parity pin: tests/golden/make_pool_golden.py runs the upstream ``KVPool.project_sequence`` / ``project_token`` with
randomised parameters and stores inputs, parameters and results in tests/golden/pool_vectors.npz;
tests/test_kv_pool.py replays them against this module.
"""

from __future__ import annotations

import torch


def _rms(x, eps):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def mix_pool_oracle(stacked, params, *, route_stride=1, dynamic=True, source_eps=1e-6, mix_eps=1e-4, compute_dtype=torch.float64):
    """The part before the projections: stacked (B,T,L,Dm) -> gained mixtures (2, k, B*T, Dm), K side first."""
    p = {name: value.to(compute_dtype) for name, value in params.items()}
    x = stacked.to(compute_dtype)
    sources, hidden = x.shape[2:]
    channels = p["gain_k"].shape[0]
    selected = list(range((sources - 1) % route_stride, sources, route_stride))
    sides = []
    for side in ("k", "v"):
        source = _rms(x, source_eps) * p[f"pre_mix_{side}"]
        logits = p[f"router_{side}_bias"].expand(*x.shape[:2], -1)
        if dynamic:
            logits = source[:, :, selected].flatten(2) @ p[f"router_{side}_weight"].T + logits
        logits = logits.unflatten(-1, (channels, sources))
        mixed = torch.einsum("btld,btkl->kbtd", source, logits)
        mixed = _rms(mixed, mix_eps) * p[f"gain_{side}"][:, None, None, :]
        sides.append(mixed.reshape(channels, -1, hidden))
    return torch.stack(sides)


def project_pool_oracle(
    stacked,
    params,
    cos,
    sin,
    *,
    kv_heads,
    head_dim,
    route_stride=1,
    dynamic=True,
    dummy=None,
    source_eps=1e-6,
    mix_eps=1e-4,
    compute_dtype=torch.float64,
):
    """stacked (B,T,L,Dm); params: pre_mix_{k,v} (L,Dm), router_{k,v}_weight (k*L, n*Dm), router_{k,v}_bias (k*L,),
    gain_{k,v} (k,Dm), proj_{k,v} (k, HKV*D, Dm), k_norm (k,D); cos/sin (B|1, T', D) with T' = T + (dummy given).
    Returns keys, values (B, k, HKV, T', D) in compute_dtype."""
    p = {name: value.to(compute_dtype) for name, value in params.items()}
    x = stacked.to(compute_dtype)
    batch, _, sources, hidden = x.shape
    if dummy is not None:
        row = dummy.to(compute_dtype).reshape(1, 1, 1, hidden).expand(batch, 1, sources, hidden)
        x = torch.cat((row, x), 1)
    channels = p["gain_k"].shape[0]
    selected = list(range((sources - 1) % route_stride, sources, route_stride))
    results = []
    for side in ("k", "v"):
        source = _rms(x, source_eps) * p[f"pre_mix_{side}"]
        logits = p[f"router_{side}_bias"]
        if dynamic:
            logits = source[:, :, selected].flatten(2) @ p[f"router_{side}_weight"].T + logits
        else:
            logits = logits.expand(*x.shape[:2], -1)
        logits = logits.unflatten(-1, (channels, sources))
        per_channel = []
        for c in range(channels):
            mixed = (source * logits[:, :, c, :, None]).sum(2)
            mixed = _rms(mixed, mix_eps) * p[f"gain_{side}"][c]
            proj = (mixed @ p[f"proj_{side}"][c].T).unflatten(-1, (kv_heads, head_dim)).transpose(1, 2)
            if side == "k":
                proj = _rms(proj, source_eps) * p["k_norm"][c]
                first, second = proj.chunk(2, -1)
                proj = proj * cos.to(compute_dtype)[:, None] + torch.cat((-second, first), -1) * sin.to(compute_dtype)[:, None]
            per_channel.append(proj)
        results.append(torch.stack(per_channel, 1))
    return results[0], results[1]
