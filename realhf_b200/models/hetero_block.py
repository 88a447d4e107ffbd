"""Blocks of a heterogeneous stack (`ReaLModelConfig.blocks`): packed (prefill / inference) and one-token (decode) forms.

A block is  x <- x + post_norm(mixer(conv(norm(x))));  x <- x + post_norm(ff(conv(norm(x))))  on a residual stream that stays
fp32 when `fp32_residual` is set.  `ReaLModel.forward` / `ReaLModel.decode_step` own the layer loop and the embedding / head;
`models.generation.DecodeState` owns the per-sequence state the blocks read and write:

  * latent cache of block i (`state.k[li]`, [n_slots, R, kv_rank], model dtype): a ring, position p in row p % R.  A block
    with `kv_from = j` holds no cache of its own: its entry is the SAME tensor as block j's.
  * convolution state of block i (`state.v[li]`, [2, n_slots, taps - 1, hidden] fp32): the normalised inputs of the last
    taps - 1 tokens, for the mixer ([0]) and the feed-forward ([1]).

Inference only (no autograd through these kernels) and not tensor-parallel.
"""

from __future__ import annotations

import dataclasses
from typing import Dict, List, Optional

import torch

from realhf_b200.ops import attention as attn_ops
from realhf_b200.ops import functional as OF


@dataclasses.dataclass
class PackedMeta:
    """Per-token indices of a packed batch, and where (if anywhere) the blocks leave the sequences' decode state."""
    pos: torch.Tensor                      # [T] int32 position inside the sequence
    remain: torch.Tensor                   # [T] int32 tokens that follow in the same sequence
    tok_slot: torch.Tensor                 # [T] int32 state slot of the token's sequence, -1 = keep no state
    k: Optional[List[torch.Tensor]] = None   # DecodeState.k / .v, indexed by local block
    v: Optional[List[torch.Tensor]] = None
    latents: Dict[int, torch.Tensor] = dataclasses.field(default_factory=dict)   # block index (0-based) -> packed latent [T, rank]
    cu_seqlens: Optional[torch.Tensor] = None
    max_seqlen: Optional[int] = None


def packed_meta(cu_seqlens: torch.Tensor, total: int, slots: Optional[torch.Tensor] = None, state=None,
                max_seqlen: Optional[int] = None) -> PackedMeta:
    dev = cu_seqlens.device
    idx = torch.arange(total, device=dev, dtype=torch.int32)
    seq = torch.searchsorted(cu_seqlens[1:].contiguous(), idx, right=True).clamp_(max=cu_seqlens.numel() - 2).long()
    pos = (idx - cu_seqlens[seq]).int()
    remain = (cu_seqlens[seq + 1] - 1 - idx).int()
    if slots is None:
        tok_slot = torch.full((total,), -1, dtype=torch.int32, device=dev)
    else:
        tok_slot = slots.to(dev).int()[seq].contiguous()
    return PackedMeta(pos, remain, tok_slot, state.k if state is not None else None, state.v if state is not None else None,
                      cu_seqlens=cu_seqlens.int().contiguous(), max_seqlen=max_seqlen)


def _mlp(model, i: int, h: torch.Tensor, mcfg) -> torch.Tensor:
    p = model.p
    if mcfg.kind == "moe":
        from realhf_b200.models import moe
        return moe.moe_forward(model, i, h, mcfg.moe)
    a = OF.clamped_gated_linear(h, p[f"{i}.mlp.gate_up.weight"], mcfg.limit, mcfg.alpha)
    return OF.linear(a, p[f"{i}.mlp.down.weight"])


def block_packed(model, i: int, li: int, x: torch.Tensor, meta: PackedMeta) -> torch.Tensor:
    """Block i (1-based layer index; li = index among this stage's blocks) on the packed batch; x [T, H] is updated in place."""
    c, p = model.config, model.p
    b = c.blocks[i - 1]
    a = b.attn
    G, eps = c.norm_groups, c.layer_norm_epsilon
    keep = meta.k is not None
    conv = meta.v[li] if keep and c.conv_taps else None
    h = OF.sublayer_input(x, p[f"{i}.attn.ln.weight"], G, eps, p.get(f"{i}.attn.canon.weight"), meta.pos, model.dtype,
                          conv[0] if conv is not None else None, meta.tok_slot, meta.remain)
    qc = OF.linear(h, p[f"{i}.attn.q_dkv.weight"])
    n_q = a.n_heads * a.qk_dim
    if a.kv_from is None:
        lat = attn_ops.latent_norm_store(qc, n_q, p[f"{i}.attn.dkv_ln.weight"], eps, meta.k[li] if keep else None, meta.tok_slot, meta.pos,
                                         meta.remain)
        meta.latents[i - 1] = lat
    else:
        lat = meta.latents[a.kv_from]
    kv = OF.linear(lat, p[f"{i}.attn.ukv.weight"])
    o = attn_ops.latent_window_attention(qc, kv, meta.pos, a.n_heads, a.qk_dim, a.v_dim, a.scale, a.window, meta.cu_seqlens, meta.max_seqlen)
    y = OF.linear(o, p[f"{i}.attn.o.weight"])
    OF.residual_add_norm_(x, y, p.get(f"{i}.attn.ln_post.weight"), G, eps)
    if b.mlp is not None:
        h = OF.sublayer_input(x, p[f"{i}.mlp.ln.weight"], G, eps, p.get(f"{i}.mlp.canon.weight"), meta.pos, model.dtype,
                              conv[1] if conv is not None else None, meta.tok_slot, meta.remain)
        OF.residual_add_norm_(x, _mlp(model, i, h, b.mlp), p.get(f"{i}.mlp.ln_post.weight"), G, eps)
    return x


def block_decode(model, i: int, li: int, x: torch.Tensor, k_caches: List[torch.Tensor], v_caches: List[torch.Tensor],
                 cache_lens: torch.Tensor, slots: Optional[torch.Tensor]) -> torch.Tensor:
    """Block i for one new token per row; x [B, H] is updated in place.  Row b lives in state slot slots[b] (None: slot b)."""
    c, p = model.config, model.p
    b = c.blocks[i - 1]
    a = b.attn
    G, eps = c.norm_groups, c.layer_norm_epsilon
    conv = v_caches[li] if c.conv_taps else None
    h = OF.sublayer_input_step(x, p[f"{i}.attn.ln.weight"], G, eps, p.get(f"{i}.attn.canon.weight"),
                               conv[0] if conv is not None else None, slots, model.dtype)
    qc = OF.linear(h, p[f"{i}.attn.q_dkv.weight"])
    o = attn_ops.latent_decode_attention(qc, p[f"{i}.attn.dkv_ln.weight"] if a.kv_from is None else None, p[f"{i}.attn.ukv.weight"],
                                         k_caches[li], cache_lens, slots, a.n_heads, a.qk_dim, a.v_dim, a.scale, a.window, eps)
    y = OF.linear(o, p[f"{i}.attn.o.weight"])
    OF.residual_add_norm_(x, y, p.get(f"{i}.attn.ln_post.weight"), G, eps)
    if b.mlp is not None:
        h = OF.sublayer_input_step(x, p[f"{i}.mlp.ln.weight"], G, eps, p.get(f"{i}.mlp.canon.weight"),
                                   conv[1] if conv is not None else None, slots, model.dtype)
        OF.residual_add_norm_(x, _mlp(model, i, h, b.mlp), p.get(f"{i}.mlp.ln_post.weight"), G, eps)
    return x


def final_norm(model, x: torch.Tensor) -> torch.Tensor:
    c = model.config
    return OF.sublayer_input(x, model.p[f"{c.n_layers}.ln_f.weight"], c.norm_groups, c.layer_norm_epsilon, None, None, model.dtype)


def ring_rows(cfg, block: int, max_len: int) -> int:
    """Rows of the latent ring of 0-based block `block` (which projects its own latent): the largest window among the blocks
    that read it, or max_len when one of them sees the whole prefix."""
    need = 0
    for j, b in enumerate(cfg.blocks):
        if j == block or b.attn.kv_from == block:
            if b.attn.window is None:
                return max_len
            need = max(need, b.attn.window)
    return max(1, min(need, max_len))
