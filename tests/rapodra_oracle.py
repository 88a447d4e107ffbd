"""A plain, slow Rapodra: one function per mechanism, written from the design's equations in float64 torch on the CPU.

It shares no code with `realhf_b200`: it works on a dict of tensors under the checkpoint's own names (`l<i>.mix.q`, ...) and on
the checkpoint's own config dict, one sequence at a time, with whole-sequence math (no cache, no state, no batching).
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch

D = torch.float64


def grouped_rms_norm(x: torch.Tensor, w: torch.Tensor, groups: int, eps: float) -> torch.Tensor:
    """x [T, W] is cut into `groups` consecutive parts; each part is divided by sqrt(mean(part^2) + eps); then times w."""
    T, W = x.shape
    p = x.to(D).view(T, groups, W // groups)
    p = p / torch.sqrt((p * p).mean(-1, keepdim=True) + eps)
    return p.reshape(T, W) * w.to(D)


def canon(h: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """h + causal depthwise convolution of h; w [W, taps], tap j weighs the input (taps - 1 - j) steps back; zeros before t=0."""
    T, W = h.shape
    taps = w.shape[1]
    out = h.to(D).clone()
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += w[:, j].to(D) * h[s].to(D)
    return out


def latent(h: torch.Tensor, w_dkv: torch.Tensor, w_norm: torch.Tensor, eps: float) -> torch.Tensor:
    """c = plain RMS norm (one group) of W_dkv h, weighted."""
    c = h.to(D) @ w_dkv.to(D).t()
    return c / torch.sqrt((c * c).mean(-1, keepdim=True) + eps) * w_norm.to(D)


def latent_attention(h: torch.Tensor, c: torch.Tensor, w_q, w_uk, w_uv, w_o, heads: int, dim: int, vdim: int, scale: float,
                     window: int) -> torch.Tensor:
    """Sliding-window softmax attention whose keys and values are up-projections of the latent c; no positions."""
    T = h.shape[0]
    q = (h.to(D) @ w_q.to(D).t()).view(T, heads, dim)
    k = (c.to(D) @ w_uk.to(D).t()).view(T, heads, dim)
    v = (c.to(D) @ w_uv.to(D).t()).view(T, heads, vdim)
    out = torch.zeros(T, heads, vdim, dtype=D)
    for i in range(T):
        lo = max(0, i - window + 1)
        for hh in range(heads):
            s = (k[lo:i + 1, hh] @ q[i, hh]) * scale
            p = torch.softmax(s, 0)
            out[i, hh] = p @ v[lo:i + 1, hh]
    return out.reshape(T, heads * vdim) @ w_o.to(D).t()


def dense_ff(h: torch.Tensor, w_gate, w_up, w_down, limit: float) -> torch.Tensor:
    g = (h.to(D) @ w_gate.to(D).t()).clamp(max=limit)
    u = (h.to(D) @ w_up.to(D).t()).clamp(min=-limit, max=limit)
    y = g * torch.sigmoid(1.702 * g) * (u + 1.0)
    return y @ w_down.to(D).t()


def moe_ff(h: torch.Tensor, w_router, b_router, experts: List[Tuple[torch.Tensor, torch.Tensor, torch.Tensor]], top: int) -> torch.Tensor:
    """experts: (gate, up, down) per expert.  The `top` largest router logits are chosen; weights = softmax over those only."""
    T = h.shape[0]
    z = h.to(D) @ w_router.to(D).t() + b_router.to(D)
    out = torch.zeros(T, experts[0][2].shape[0], dtype=D)
    for t in range(T):
        zs, idx = torch.sort(z[t], descending=True, stable=True)
        zs, idx = zs[:top], idx[:top]
        wts = torch.softmax(zs, 0)
        for wt, e in zip(wts.tolist(), idx.tolist()):
            g, u, d = experts[e]
            a = h[t].to(D) @ g.to(D).t()
            a = a * torch.sigmoid(a) * (h[t].to(D) @ u.to(D).t())
            out[t] += wt * (a @ d.to(D).t())
    return out


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], return_layers: bool = False):
    """Logits [T, vocab] of one sequence (float64), optionally with the residual stream after every layer."""
    eps, groups = cfg["norm"]["eps"], cfg["norm"]["groups"]
    x = w["embed"].to(D)[torch.tensor(tokens, dtype=torch.long)]
    latents: Dict[int, torch.Tensor] = {}
    per_layer = []
    for i, lay in enumerate(cfg["layers"]):
        L = f"l{i}."
        assert lay["type"] == "latent_attention"
        m = lay["mixer"]
        h = canon(grouped_rms_norm(x, w[L + "norm1"], groups, eps), w[L + "canon1"])
        if m.get("kv_from") is not None:
            c = latents[m["kv_from"]]
        else:
            c = latents[i] = latent(h, w[L + "mix.dkv"], w[L + "mix.dkv.norm"], eps)
        o = latent_attention(h, c, w[L + "mix.q"], w[L + "mix.uk"], w[L + "mix.uv"], w[L + "mix.o"], m["heads"], m["dim"], m["vdim"],
                             m["scale"], m["mask"]["size"])
        x = x + grouped_rms_norm(o, w[L + "norm1b"], groups, eps)
        f = lay.get("mlp")
        if f is not None:
            h = canon(grouped_rms_norm(x, w[L + "norm2"], groups, eps), w[L + "canon2"])
            if f["kind"] == "dense":
                y = dense_ff(h, w[L + "mlp.gate"], w[L + "mlp.up"], w[L + "mlp.down"], f["limit"])
            else:
                ex = [(w[L + f"mlp.e{e}.gate"], w[L + f"mlp.e{e}.up"], w[L + f"mlp.e{e}.down"]) for e in range(f["router"]["experts"])]
                y = moe_ff(h, w[L + "mlp.router"], w[L + "mlp.router.b"], ex, f["router"]["top"])
            x = x + grouped_rms_norm(y, w[L + "norm2b"], groups, eps)
        per_layer.append(x.clone())
    z = grouped_rms_norm(x, w["final.norm"], groups, eps) @ w["head"].to(D).t()
    cap = cfg.get("logit_softcap")
    if cap:
        z = cap * torch.tanh(z / cap)
    return (z, per_layer) if return_layers else z


# ------------------------------------------------------------------------------------------- random models for the tests


def random_config(width=48, vocab=64, groups=3, taps=3, softcap=20.0, eps=1e-5, layers: Optional[list] = None) -> dict:
    if layers is None:
        mx = lambda **k: dict(dict(dim=16, heads=2, kv_rank=24, vdim=8, scale=0.3, mask=dict(size=7)), **k)
        layers = [dict(type="latent_attention", mixer=mx(), mlp=dict(kind="dense", ff=40, limit=1.25)),
                  dict(type="latent_attention", mixer=mx(heads=3, mask=dict(size=5)), mlp=dict(kind="moe", expert=dict(ff=24), router=dict(experts=5, top=2))),
                  dict(type="latent_attention", mixer=mx(kv_from=0, dim=8, vdim=16, mask=dict(size=11)), mlp=None),
                  dict(type="latent_attention", mixer=mx(kv_from=1, heads=1), mlp=dict(kind="moe", expert=dict(ff=16), router=dict(experts=3, top=1)))]
    return dict(architecture="Rapodra", canon=dict(taps=taps), layers=layers, logit_softcap=softcap, norm=dict(eps=eps, groups=groups),
                vocab=vocab, width=width)


def random_weights(cfg: dict, seed: int = 0, dtype=torch.bfloat16) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    W, V, taps = cfg["width"], cfg["vocab"], cfg["canon"]["taps"]
    rn = lambda *s, std=1.0: (torch.randn(*s, generator=g) * std).to(dtype)
    lin = lambda o, i, gain=1.0: rn(o, i, std=gain / math.sqrt(i))
    nw = lambda n: (1.0 + 0.2 * torch.randn(n, generator=g)).to(dtype)
    w = {"embed": rn(V, W), "final.norm": nw(W), "head": lin(V, W, 2.0)}
    for i, lay in enumerate(cfg["layers"]):
        L, m = f"l{i}.", lay["mixer"]
        w[L + "norm1"], w[L + "norm1b"] = nw(W), nw(W)
        w[L + "canon1"] = rn(W, taps, std=0.4)
        w[L + "mix.q"] = lin(m["heads"] * m["dim"], W, 2.0)
        if m.get("kv_from") is None:
            w[L + "mix.dkv"] = lin(m["kv_rank"], W)
            w[L + "mix.dkv.norm"] = nw(m["kv_rank"])
        w[L + "mix.uk"] = lin(m["heads"] * m["dim"], m["kv_rank"], 2.0)
        w[L + "mix.uv"] = lin(m["heads"] * m["vdim"], m["kv_rank"])
        w[L + "mix.o"] = lin(W, m["heads"] * m["vdim"])
        f = lay.get("mlp")
        if f is None:
            continue
        w[L + "norm2"], w[L + "norm2b"] = nw(W), nw(W)
        w[L + "canon2"] = rn(W, taps, std=0.4)
        if f["kind"] == "dense":
            w[L + "mlp.gate"], w[L + "mlp.up"], w[L + "mlp.down"] = lin(f["ff"], W, 2.0), lin(f["ff"], W, 2.0), lin(W, f["ff"])
        else:
            E, ff = f["router"]["experts"], f["expert"]["ff"]
            w[L + "mlp.router"] = lin(E, W, 3.0)
            w[L + "mlp.router.b"] = rn(E, std=0.5)
            for e in range(E):
                w[L + f"mlp.e{e}.gate"], w[L + f"mlp.e{e}.up"], w[L + f"mlp.e{e}.down"] = lin(ff, W, 2.0), lin(ff, W, 2.0), lin(W, ff)
    return w
