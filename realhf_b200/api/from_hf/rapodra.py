"""Rapodra checkpoints <-> ReaLModel.

A Rapodra checkpoint is `config.json` + `model.safetensors`.  The config lists the blocks one by one (`layers[i]` = mixer
type, mixer sizes, feed-forward or null); the model is a heterogeneous stack (`ReaLModelConfig.blocks`) built from mechanisms
the config class offers to any family: grouped RMSNorm on the input AND the output of every sublayer, a short causal
convolution on every sublayer's input, latent attention with a sliding window (a block may read an earlier block's cached
latent), a clamped gated-linear-unit or a mixture-of-experts feed-forward with a router bias, a soft cap on the logits, and an
fp32 residual stream.  There is no `transformers` class for it: the config is read as a plain dict (`config_from_dict`).

Checkpoint names -> framework names (block i of the checkpoint is layer i + 1 here):
  embed / head / final.norm           0.wte.weight / {L+1}.head.weight / {L}.ln_f.weight
  l<i>.norm1, norm1b, canon1          attn.ln.weight, attn.ln_post.weight, attn.canon.weight
  l<i>.mix.q (+ mix.dkv)              attn.q_dkv.weight      (sections [q | dkv]; no dkv section in a `kv_from` block)
  l<i>.mix.dkv.norm                   attn.dkv_ln.weight
  l<i>.mix.uk + mix.uv                attn.ukv.weight        (sections [uk | uv])
  l<i>.mix.o                          attn.o.weight
  l<i>.norm2, norm2b, canon2          mlp.ln.weight, mlp.ln_post.weight, mlp.canon.weight
  l<i>.mlp.gate + up, down            mlp.gate_up.weight, mlp.down.weight
  l<i>.mlp.router, router.b           mlp.router.weight, mlp.router.bias
  l<i>.mlp.e<k>.gate + up, down       mlp.experts.gate_up.weight[k], mlp.experts.down.weight[k]
"""

from __future__ import annotations

from typing import Dict, List

import torch

from realhf_b200.api.model import (BlockConfig, BlockMLPConfig, LatentAttentionConfig, ReaLModelConfig, ReaLMoEConfig,
                                   register_hf_family)

CLAMPED_GLU_ALPHA = 1.702   # fixed by the design: y = g * sigmoid(1.702 g) * (u + 1)


def config_from_dict(d: dict, is_critic: bool = False) -> ReaLModelConfig:
    blocks: List[BlockConfig] = []
    for i, lay in enumerate(d["layers"]):
        if lay["type"] != "latent_attention":
            raise ValueError(f"Rapodra layer {i}: unknown mixer type `{lay['type']}`")
        m = lay["mixer"]
        attn = LatentAttentionConfig(n_heads=int(m["heads"]), qk_dim=int(m["dim"]), v_dim=int(m["vdim"]), kv_rank=int(m["kv_rank"]),
                                     scale=float(m["scale"]), window=int(m["mask"]["size"]) if m.get("mask") else None,
                                     kv_from=(int(m["kv_from"]) if m.get("kv_from") is not None else None))
        f = lay.get("mlp")
        if f is None:
            mlp = None
        elif f["kind"] == "dense":
            mlp = BlockMLPConfig(kind="clamped_glu", ff=int(f["ff"]), limit=float(f["limit"]), alpha=CLAMPED_GLU_ALPHA)
        elif f["kind"] == "moe":
            mlp = BlockMLPConfig(kind="moe", ff=int(f["expert"]["ff"]),
                                 moe=ReaLMoEConfig(num_experts=int(f["router"]["experts"]), top_k=int(f["router"]["top"]),
                                                   routing_type="none", aux_loss_coeff=0.0, capacity_factor=None))
        else:
            raise ValueError(f"Rapodra layer {i}: unknown feed-forward kind `{f['kind']}`")
        blocks.append(BlockConfig(mixer="latent_attention", attn=attn, mlp=mlp))
    a0 = blocks[0].attn
    ffs = [b.mlp.ff for b in blocks if b.mlp is not None]
    cap = d.get("logit_softcap")
    return ReaLModelConfig(
        n_layers=len(blocks), n_kv_heads=a0.n_heads, n_q_heads=a0.n_heads, hidden_dim=int(d["width"]),
        intermediate_dim=max(ffs) if ffs else 0, vocab_size=int(d["vocab"]), head_dim=a0.qk_dim, n_positions=None, embd_pdrop=0.0,
        resid_pdrop=0.0, attn_pdrop=0.0, layer_norm_epsilon=float(d["norm"]["eps"]), activation_function="silu",
        scale_attn_by_inverse_layer_idx=False, scale_attn_weights=True, use_attention_bias=False, use_attn_proj_bias=False,
        use_mlp_bias=False, layer_norm_type="rms", mlp_type="llama", apply_rotary=False, tied_embedding=False, is_critic=is_critic,
        blocks=blocks, norm_groups=int(d["norm"].get("groups", 1)), sandwich_norm=True, conv_taps=int((d.get("canon") or {}).get("taps", 0)),
        logit_softcap=float(cap) if cap else None, fp32_residual=True)


def config_to_dict(cfg: ReaLModelConfig) -> dict:
    layers = []
    for b in cfg.blocks:
        a = b.attn
        m = dict(dim=a.qk_dim, heads=a.n_heads, kv_rank=a.kv_rank, vdim=a.v_dim, scale=a.scale)
        if a.window is not None:
            m["mask"] = dict(size=a.window)
        if a.kv_from is not None:
            m["kv_from"] = a.kv_from
        if b.mlp is None:
            f = None
        elif b.mlp.kind == "moe":
            f = dict(kind="moe", expert=dict(ff=b.mlp.ff), router=dict(experts=b.mlp.moe.num_experts, top=b.mlp.moe.top_k))
        else:
            f = dict(kind="dense", ff=b.mlp.ff, limit=b.mlp.limit)
        layers.append(dict(type="latent_attention", mixer=m, mlp=f))
    return dict(architecture="Rapodra", canon=dict(taps=cfg.conv_taps), layers=layers, logit_softcap=cfg.logit_softcap,
                norm=dict(eps=cfg.layer_norm_epsilon, groups=cfg.norm_groups), vocab=cfg.vocab_size, width=cfg.hidden_dim)


def _sd_from_ckpt(sd: Dict[str, torch.Tensor], cfg: ReaLModelConfig) -> Dict[str, torch.Tensor]:
    out: Dict[str, torch.Tensor] = {}
    L = cfg.n_layers
    if "embed" in sd:
        out["0.wte.weight"] = sd["embed"]
    if "head" in sd:
        out[f"{L + 1}.head.weight"] = sd["head"]
    if "final.norm" in sd:
        out[f"{L}.ln_f.weight"] = sd["final.norm"]
    for i, b in enumerate(cfg.blocks):
        cp, rp = f"l{i}.", f"{i + 1}."
        if cp + "mix.q" not in sd:
            continue
        out[rp + "attn.ln.weight"] = sd[cp + "norm1"]
        out[rp + "attn.ln_post.weight"] = sd[cp + "norm1b"]
        if cfg.conv_taps:
            out[rp + "attn.canon.weight"] = sd[cp + "canon1"]
        if b.attn.kv_from is None:
            out[rp + "attn.q_dkv.weight"] = torch.cat([sd[cp + "mix.q"], sd[cp + "mix.dkv"]], 0)
            out[rp + "attn.dkv_ln.weight"] = sd[cp + "mix.dkv.norm"]
        else:
            out[rp + "attn.q_dkv.weight"] = sd[cp + "mix.q"]
        out[rp + "attn.ukv.weight"] = torch.cat([sd[cp + "mix.uk"], sd[cp + "mix.uv"]], 0)
        out[rp + "attn.o.weight"] = sd[cp + "mix.o"]
        if b.mlp is None:
            continue
        out[rp + "mlp.ln.weight"] = sd[cp + "norm2"]
        out[rp + "mlp.ln_post.weight"] = sd[cp + "norm2b"]
        if cfg.conv_taps:
            out[rp + "mlp.canon.weight"] = sd[cp + "canon2"]
        if b.mlp.kind == "moe":
            E = b.mlp.moe.num_experts
            out[rp + "mlp.router.weight"] = sd[cp + "mlp.router"]
            out[rp + "mlp.router.bias"] = sd[cp + "mlp.router.b"]
            out[rp + "mlp.experts.gate_up.weight"] = torch.stack(
                [torch.cat([sd[cp + f"mlp.e{e}.gate"], sd[cp + f"mlp.e{e}.up"]], 0) for e in range(E)])
            out[rp + "mlp.experts.down.weight"] = torch.stack([sd[cp + f"mlp.e{e}.down"] for e in range(E)])
        else:
            out[rp + "mlp.gate_up.weight"] = torch.cat([sd[cp + "mlp.gate"], sd[cp + "mlp.up"]], 0)
            out[rp + "mlp.down.weight"] = sd[cp + "mlp.down"]
    return out


def _sd_to_ckpt(sd: Dict[str, torch.Tensor], cfg: ReaLModelConfig) -> Dict[str, torch.Tensor]:
    out: Dict[str, torch.Tensor] = {}
    L = cfg.n_layers
    plain = {"attn.ln.weight": "norm1", "attn.ln_post.weight": "norm1b", "attn.canon.weight": "canon1", "attn.dkv_ln.weight": "mix.dkv.norm",
             "attn.o.weight": "mix.o", "mlp.ln.weight": "norm2", "mlp.ln_post.weight": "norm2b", "mlp.canon.weight": "canon2",
             "mlp.down.weight": "mlp.down", "mlp.router.weight": "mlp.router", "mlp.router.bias": "mlp.router.b"}
    for k, v in sd.items():
        li, name = k.split(".", 1)
        li = int(li)
        if li == 0:
            out["embed"] = v
        elif li == L + 1:
            out["head"] = v
        elif name == "ln_f.weight":
            out["final.norm"] = v
        else:
            cp, b = f"l{li - 1}.", cfg.blocks[li - 1]
            a = b.attn
            if name in plain:
                out[cp + plain[name]] = v
            elif name == "attn.q_dkv.weight":
                out[cp + "mix.q"] = v[: a.n_heads * a.qk_dim]
                if a.kv_from is None:
                    out[cp + "mix.dkv"] = v[a.n_heads * a.qk_dim:]
            elif name == "attn.ukv.weight":
                out[cp + "mix.uk"], out[cp + "mix.uv"] = v[: a.n_heads * a.qk_dim], v[a.n_heads * a.qk_dim:]
            elif name == "mlp.gate_up.weight":
                out[cp + "mlp.gate"], out[cp + "mlp.up"] = v[: b.mlp.ff], v[b.mlp.ff:]
            elif name == "mlp.experts.gate_up.weight":
                for e in range(v.shape[0]):
                    out[cp + f"mlp.e{e}.gate"], out[cp + f"mlp.e{e}.up"] = v[e, : b.mlp.ff], v[e, b.mlp.ff:]
            elif name == "mlp.experts.down.weight":
                for e in range(v.shape[0]):
                    out[cp + f"mlp.e{e}.down"] = v[e]
            else:
                raise KeyError(k)
    return out


def _block_names(cfg: ReaLModelConfig, i: int) -> List[str]:
    b, cp = cfg.blocks[i], f"l{i}."
    names = [cp + n for n in ("norm1", "norm1b", "mix.q", "mix.uk", "mix.uv", "mix.o")]
    if cfg.conv_taps:
        names.append(cp + "canon1")
    if b.attn.kv_from is None:
        names += [cp + "mix.dkv", cp + "mix.dkv.norm"]
    if b.mlp is not None:
        names += [cp + "norm2", cp + "norm2b"] + ([cp + "canon2"] if cfg.conv_taps else [])
        if b.mlp.kind == "moe":
            names += [cp + "mlp.router", cp + "mlp.router.b"]
            names += [cp + f"mlp.e{e}.{x}" for e in range(b.mlp.moe.num_experts) for x in ("gate", "up", "down")]
        else:
            names += [cp + "mlp.gate", cp + "mlp.up", cp + "mlp.down"]
    if i == cfg.n_layers - 1:
        names.append("final.norm")
    return names


def make_test_config() -> ReaLModelConfig:
    att = lambda **k: dict(dict(dim=16, heads=2, kv_rank=24, vdim=8, scale=0.25, mask=dict(size=6)), **k)
    return config_from_dict(dict(
        canon=dict(taps=3), logit_softcap=25.0, norm=dict(eps=1e-5, groups=2), vocab=128, width=32,
        layers=[dict(type="latent_attention", mixer=att(), mlp=dict(kind="dense", ff=48, limit=2.0)),
                dict(type="latent_attention", mixer=att(kv_from=0, heads=4), mlp=dict(kind="moe", expert=dict(ff=16), router=dict(experts=4, top=2)))]))


register_hf_family(
    "rapodra", "Rapodra", lambda hf, is_critic=False: config_from_dict(hf if isinstance(hf, dict) else hf.to_dict(), is_critic),
    config_to_dict, _sd_from_ckpt, _sd_to_ckpt, lambda cfg: ["embed"], _block_names, lambda cfg: ["head"],
    make_test_config=make_test_config, config_from_dict=config_from_dict, config_to_dict=config_to_dict, weight_file="model.safetensors")
