"""Tizodra checkpoints <-> ReaLModel.

A Tizodra checkpoint is `config.json` + `model.safetensors`.  The config lists the layers one by one (`layers[i]` = mixer type
`attention` or `delta`, the mixer's sizes, a feed-forward or null) and a `loop`: a range of layers that runs several times with
the same weights, each pass with its own cache.  The model is a heterogeneous stack (`ReaLModelConfig.blocks`) made of mechanisms
the config class offers to any family:

  * sinusoidal positions added to the embedding (`sinusoidal_positions`), an fp32 residual stream, pre-norm RMSNorm sublayers;
  * `WindowAttentionConfig`: grouped-query attention without rotation, biased projections, weight-free RMS norm of every value
    head, a per-head temperature, a linear distance penalty, a sliding window that keeps the first tokens, a sink logit in the
    softmax denominator and a per-head sigmoid output gate;
  * `DeltaRuleConfig`: the gated delta rule on a per-head matrix state with short convolutions on q, k, v;
  * `BlockMLPConfig(kind="relu2")`, `LoopConfig` with re-injection of the embedding output, `logit_scale`.

There is no `transformers` class for it: the config is read as a plain dict.  Constants the design fixes (slope base 8, sinusoid
base 10000, unit-norm epsilon 1e-6) are the defaults of those config classes.

Checkpoint names -> framework names (layer i of the checkpoint is block i + 1 here):
  embed / head / final.norm                 0.wte.weight / {L+1}.head.weight / {L}.ln_f.weight
  loop.in                                   {loop.start+1}.loop_in.weight
  l<i>.norm1 / norm2                        attn.ln.weight / mlp.ln.weight
  l<i>.mlp.up / down                        mlp.up.weight / mlp.down.weight
  attention: mix.q, k, v, g (+ q.b, k.b, v.b)  attn.qkvg.weight, attn.qkvg.bias   (sections [q | k | v | gate, padded to 8 rows])
             mix.temp / sink / o            attn.temp.weight / attn.sink.weight / attn.o.weight
  delta:     mix.q, k, v, g, b, a           attn.in.weight      (sections [q | k | v | g | b, a padded to 8 rows])
             mix.q.conv, k.conv, v.conv     attn.conv.weight    ([q | k | v] channels x taps)
             mix.A_log / dt_bias / norm / o attn.A_log.weight / attn.dt_bias.weight / attn.o_norm.weight / attn.o.weight
"""

from __future__ import annotations

from typing import Dict, List

import torch

from realhf_b200.api.model import (BlockConfig, BlockMLPConfig, DeltaRuleConfig, LoopConfig, ReaLModelConfig, WindowAttentionConfig,
                                   register_hf_family)

SLOPE_BASE = 8.0          # distance penalty of head h: 2^(-8 (h + 1) / heads) per token of distance
SINUSOID_BASE = 10000.0
UNIT_EPS = 1e-6           # inside the root of the delta rule's q / k unit norms


def config_from_dict(d: dict, is_critic: bool = False) -> ReaLModelConfig:
    blocks: List[BlockConfig] = []
    for i, lay in enumerate(d["layers"]):
        m = lay["mixer"]
        f = lay.get("mlp")
        if f is None:
            mlp = None
        elif f["kind"] == "dense":
            mlp = BlockMLPConfig(kind="relu2", ff=int(f["ff"]))
        else:
            raise ValueError(f"Tizodra layer {i}: unknown feed-forward kind `{f['kind']}`")
        if lay["type"] == "attention":
            mask = m.get("mask")
            w = WindowAttentionConfig(n_heads=int(m["heads"]), n_kv_heads=int(m["kv_heads"]), qk_dim=int(m["dim"]), v_dim=int(m["vdim"]),
                                      scale=float(m["scale"]), window=int(mask["size"]) if mask else None,
                                      keep_first=int(mask.get("keep_first", 0)) if mask else 0, slope_base=SLOPE_BASE)
            blocks.append(BlockConfig(mixer="window_attention", wattn=w, mlp=mlp))
        elif lay["type"] == "delta":
            dl = DeltaRuleConfig(n_heads=int(m["heads"]), n_kv_heads=int(m["kv_heads"]), qk_dim=int(m["dim"]), v_dim=int(m["vdim"]),
                                 conv_taps=int(m["conv"]), unit_eps=UNIT_EPS)
            blocks.append(BlockConfig(mixer="delta", delta=dl, mlp=mlp))
        else:
            raise ValueError(f"Tizodra layer {i}: unknown mixer type `{lay['type']}`")
    lp = d.get("loop")
    loop = LoopConfig(start=int(lp["start"]), stop=int(lp["stop"]), times=int(lp["times"]), inject=True) if lp else None
    heads = [(b.wattn or b.delta) for b in blocks]
    ffs = [b.mlp.ff for b in blocks if b.mlp is not None]
    ls = d.get("logit_scale")
    return ReaLModelConfig(
        n_layers=len(blocks), n_kv_heads=heads[0].n_kv_heads, n_q_heads=heads[0].n_heads, hidden_dim=int(d["width"]),
        intermediate_dim=max(ffs) if ffs else 0, vocab_size=int(d["vocab"]), head_dim=heads[0].qk_dim, n_positions=None, embd_pdrop=0.0,
        resid_pdrop=0.0, attn_pdrop=0.0, layer_norm_epsilon=float(d["norm"]["eps"]), activation_function="relu2",
        scale_attn_by_inverse_layer_idx=False, scale_attn_weights=True, use_attention_bias=True, use_attn_proj_bias=False,
        use_mlp_bias=False, layer_norm_type="rms", mlp_type=None, apply_rotary=False, tied_embedding=False, is_critic=is_critic,
        blocks=blocks, norm_groups=1, sandwich_norm=False, conv_taps=0, fp32_residual=True, sinusoidal_positions=True,
        sinusoid_base=SINUSOID_BASE, logit_scale=float(ls) if ls is not None else None, loop=loop)


def config_to_dict(cfg: ReaLModelConfig) -> dict:
    layers = []
    for b in cfg.blocks:
        f = None if b.mlp is None else dict(ff=b.mlp.ff, kind="dense")
        if b.mixer == "window_attention":
            w = b.wattn
            m = dict(dim=w.qk_dim, heads=w.n_heads, kv_heads=w.n_kv_heads, scale=w.scale, vdim=w.v_dim)
            if w.window is not None:
                m["mask"] = dict(keep_first=w.keep_first, size=w.window)
            layers.append(dict(mixer=m, mlp=f, type="attention"))
        else:
            dl = b.delta
            layers.append(dict(mixer=dict(conv=dl.conv_taps, dim=dl.qk_dim, heads=dl.n_heads, kv_heads=dl.n_kv_heads, vdim=dl.v_dim),
                               mlp=f, type="delta"))
    out = dict(architecture="Tizodra", layers=layers, norm=dict(eps=cfg.layer_norm_epsilon), vocab=cfg.vocab_size, width=cfg.hidden_dim)
    if cfg.logit_scale is not None:
        out["logit_scale"] = cfg.logit_scale
    if cfg.loop is not None:
        out["loop"] = dict(start=cfg.loop.start, stop=cfg.loop.stop, times=cfg.loop.times)
    return out


def _pad_rows(t: torch.Tensor, rows: int) -> torch.Tensor:
    if t.shape[0] == rows:
        return t
    return torch.cat([t, torch.zeros(rows - t.shape[0], *t.shape[1:], dtype=t.dtype)], 0)


def _sd_from_ckpt(sd: Dict[str, torch.Tensor], cfg: ReaLModelConfig) -> Dict[str, torch.Tensor]:
    from realhf_b200.models.sharding import delta_sections, wattn_sections
    out: Dict[str, torch.Tensor] = {}
    L = cfg.n_layers
    if "embed" in sd:
        out["0.wte.weight"] = sd["embed"]
    if "head" in sd:
        out[f"{L + 1}.head.weight"] = sd["head"]
    if "final.norm" in sd:
        out[f"{L}.ln_f.weight"] = sd["final.norm"]
    if "loop.in" in sd and cfg.loop is not None:
        out[f"{cfg.loop.start + 1}.loop_in.weight"] = sd["loop.in"]
    for i, b in enumerate(cfg.blocks):
        cp, rp = f"l{i}.", f"{i + 1}."
        if cp + "mix.q" not in sd:
            continue
        out[rp + "attn.ln.weight"] = sd[cp + "norm1"]
        if b.mixer == "window_attention":
            w = b.wattn
            sec = wattn_sections(w)
            out[rp + "attn.qkvg.weight"] = torch.cat([sd[cp + "mix.q"], sd[cp + "mix.k"], sd[cp + "mix.v"], _pad_rows(sd[cp + "mix.g"], sec[3])], 0)
            out[rp + "attn.qkvg.bias"] = torch.cat([sd[cp + "mix.q.b"], sd[cp + "mix.k.b"], sd[cp + "mix.v.b"],
                                                    torch.zeros(sec[3], dtype=sd[cp + "mix.q.b"].dtype)], 0)
            out[rp + "attn.temp.weight"] = sd[cp + "mix.temp"]
            out[rp + "attn.sink.weight"] = sd[cp + "mix.sink"]
        else:
            sec = delta_sections(b.delta)
            ba = _pad_rows(torch.cat([sd[cp + "mix.b"], sd[cp + "mix.a"]], 0), sec[4])
            out[rp + "attn.in.weight"] = torch.cat([sd[cp + "mix.q"], sd[cp + "mix.k"], sd[cp + "mix.v"], sd[cp + "mix.g"], ba], 0)
            out[rp + "attn.conv.weight"] = torch.cat([sd[cp + "mix.q.conv"], sd[cp + "mix.k.conv"], sd[cp + "mix.v.conv"]], 0)
            out[rp + "attn.A_log.weight"] = sd[cp + "mix.A_log"]
            out[rp + "attn.dt_bias.weight"] = sd[cp + "mix.dt_bias"]
            out[rp + "attn.o_norm.weight"] = sd[cp + "mix.norm"]
        out[rp + "attn.o.weight"] = sd[cp + "mix.o"]
        if b.mlp is not None:
            out[rp + "mlp.ln.weight"] = sd[cp + "norm2"]
            out[rp + "mlp.up.weight"] = sd[cp + "mlp.up"]
            out[rp + "mlp.down.weight"] = sd[cp + "mlp.down"]
    return out


def _sd_to_ckpt(sd: Dict[str, torch.Tensor], cfg: ReaLModelConfig) -> Dict[str, torch.Tensor]:
    out: Dict[str, torch.Tensor] = {}
    L = cfg.n_layers
    plain = {"attn.ln.weight": "norm1", "mlp.ln.weight": "norm2", "attn.o.weight": "mix.o", "attn.temp.weight": "mix.temp",
             "attn.sink.weight": "mix.sink", "attn.A_log.weight": "mix.A_log", "attn.dt_bias.weight": "mix.dt_bias",
             "attn.o_norm.weight": "mix.norm", "mlp.up.weight": "mlp.up", "mlp.down.weight": "mlp.down"}
    for k, v in sd.items():
        li, name = k.split(".", 1)
        li = int(li)
        if li == 0:
            out["embed"] = v
        elif li == L + 1:
            out["head"] = v
        elif name == "ln_f.weight":
            out["final.norm"] = v
        elif name == "loop_in.weight":
            out["loop.in"] = v
        else:
            cp, b = f"l{li - 1}.", cfg.blocks[li - 1]
            if name in plain:
                out[cp + plain[name]] = v
            elif name in ("attn.qkvg.weight", "attn.qkvg.bias"):
                w = b.wattn
                q, kk, vv, g = torch.split(v, [w.n_heads * w.qk_dim, w.n_kv_heads * w.qk_dim, w.n_kv_heads * w.v_dim,
                                               v.shape[0] - w.n_heads * w.qk_dim - w.n_kv_heads * (w.qk_dim + w.v_dim)], 0)
                if name.endswith("weight"):
                    out[cp + "mix.q"], out[cp + "mix.k"], out[cp + "mix.v"], out[cp + "mix.g"] = q, kk, vv, g[: w.n_heads]
                else:
                    out[cp + "mix.q.b"], out[cp + "mix.k.b"], out[cp + "mix.v.b"] = q, kk, vv
            elif name == "attn.in.weight":
                dl = b.delta
                nqk, nv, H = dl.n_kv_heads * dl.qk_dim, dl.n_heads * dl.v_dim, dl.n_heads
                out[cp + "mix.q"], out[cp + "mix.k"], out[cp + "mix.v"], out[cp + "mix.g"] = \
                    v[:nqk], v[nqk:2 * nqk], v[2 * nqk:2 * nqk + nv], v[2 * nqk + nv:2 * nqk + 2 * nv]
                out[cp + "mix.b"], out[cp + "mix.a"] = v[2 * nqk + 2 * nv:2 * nqk + 2 * nv + H], v[2 * nqk + 2 * nv + H:2 * nqk + 2 * nv + 2 * H]
            elif name == "attn.conv.weight":
                dl = b.delta
                nqk = dl.n_kv_heads * dl.qk_dim
                out[cp + "mix.q.conv"], out[cp + "mix.k.conv"], out[cp + "mix.v.conv"] = v[:nqk], v[nqk:2 * nqk], v[2 * nqk:]
            else:
                raise KeyError(k)
    return {k: v.contiguous() for k, v in out.items()}


def _block_names(cfg: ReaLModelConfig, i: int) -> List[str]:
    b, cp = cfg.blocks[i], f"l{i}."
    names = [cp + n for n in ("norm1", "mix.q", "mix.k", "mix.v", "mix.g", "mix.o")]
    if b.mixer == "window_attention":
        names += [cp + n for n in ("mix.q.b", "mix.k.b", "mix.v.b", "mix.temp", "mix.sink")]
    else:
        names += [cp + n for n in ("mix.q.conv", "mix.k.conv", "mix.v.conv", "mix.b", "mix.a", "mix.A_log", "mix.dt_bias", "mix.norm")]
    if b.mlp is not None:
        names += [cp + "norm2", cp + "mlp.up", cp + "mlp.down"]
    if cfg.loop is not None and i == cfg.loop.start:
        names.append("loop.in")
    if i == cfg.n_layers - 1:
        names.append("final.norm")
    return names


def make_test_config() -> ReaLModelConfig:
    att = dict(type="attention", mixer=dict(dim=8, heads=4, kv_heads=2, vdim=16, scale=0.3, mask=dict(size=5, keep_first=2)),
               mlp=dict(kind="dense", ff=48))
    dlt = dict(type="delta", mixer=dict(conv=4, dim=8, heads=4, kv_heads=2, vdim=16), mlp=None)
    return config_from_dict(dict(layers=[att, dlt, att], logit_scale=0.25, loop=dict(start=1, stop=3, times=2), norm=dict(eps=1e-5),
                                 vocab=96, width=32))


register_hf_family(
    "tizodra", "Tizodra", lambda hf, is_critic=False: config_from_dict(hf if isinstance(hf, dict) else hf.to_dict(), is_critic),
    config_to_dict, _sd_from_ckpt, _sd_to_ckpt, lambda cfg: ["embed"], _block_names, lambda cfg: ["head"],
    make_test_config=make_test_config, config_from_dict=config_from_dict, config_to_dict=config_to_dict, weight_file="model.safetensors")
