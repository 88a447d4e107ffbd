"""A plain, slow Tizodra in float64: one function per mechanism, whole sequences only, no cache and no batching.

It shares no code with the package: it reads the checkpoint's own tensor names (`embed`, `loop.in`, `l<i>.norm1`, `l<i>.mix.q`, ...)
from a dict of tensors and the checkpoint's own `config.json` dict.  The package's tests compare every path of the framework
(packed prefill, token-by-token decoding through the state manager, batches, generation) with it.

Notation: x [T, W] is one sequence's residual stream, positions 0 .. T - 1.
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


def rms_divide(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, w, eps):
    return rms_divide(x, eps) * w


def sinusoid(T: int, width: int) -> torch.Tensor:
    """[T, width] of interleaved pairs: out[:, 2i] = sin(a_i), out[:, 2i + 1] = cos(a_i), a_i = p / 10000^(2i / width)."""
    p = torch.arange(T, dtype=F64).unsqueeze(1)
    i = torch.arange((width + 1) // 2, dtype=F64).unsqueeze(0)
    ang = p * torch.pow(torch.tensor(10000.0, dtype=F64), -2.0 * i / width)
    out = torch.zeros(T, width, dtype=F64)
    out[:, 0::2] = torch.sin(ang)
    out[:, 1::2] = torch.cos(ang[:, : width // 2])
    return out


def embedding(sd, tokens: List[int], width: int) -> torch.Tensor:
    return sd["embed"].to(F64)[torch.tensor(tokens, dtype=torch.long)] + sinusoid(len(tokens), width)


def visible(T: int, size: Optional[int], keep_first: int) -> torch.Tensor:
    """[T, T] bool: query i (row) sees key j (column)."""
    i = torch.arange(T).unsqueeze(1)
    j = torch.arange(T).unsqueeze(0)
    ok = j <= i
    if size is not None:
        ok = ok & ((i - j < size) | (j < keep_first))
    return ok


def attention_core(q, k, v, gate, m: dict, temp, sink) -> torch.Tensor:
    """q [T, H, d], k [T, G, d], v [T, G, dv] (already normalised), gate [T, H] or None (already a sigmoid), temp / sink [H] -> [T, H, dv]."""
    T, H, _ = q.shape
    G, dv = k.shape[1], v.shape[2]
    mask = m.get("mask")
    ok = visible(T, mask["size"] if mask else None, (mask or {}).get("keep_first", 0))
    dist = (torch.arange(T).unsqueeze(1) - torch.arange(T).unsqueeze(0)).to(F64)
    out = torch.zeros(T, H, dv, dtype=F64)
    for hh in range(H):
        g = hh // (H // G)
        slope = 2.0 ** (-8.0 * (hh + 1) / H)
        s = (q[:, hh] @ k[:, g].T) * m["scale"] * temp[hh] - slope * dist
        s = s.masked_fill(~ok, -math.inf)
        mx = torch.maximum(s.max(-1, keepdim=True).values, sink[hh])
        e = torch.exp(s - mx)
        den = e.sum(-1, keepdim=True) + torch.exp(sink[hh] - mx)
        out[:, hh] = (e / den) @ v[:, g]
        if gate is not None:
            out[:, hh] = out[:, hh] * gate[:, hh:hh + 1]
    return out


def attention_mixer(sd, pre: str, m: dict, h: torch.Tensor, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    w = lambda n: sd[pre + n].to(F64)
    q = (h @ w("q").T + w("q.b")).view(T, H, d)
    k = (h @ w("k").T + w("k.b")).view(T, G, d)
    v = rms_divide((h @ w("v").T + w("v.b")).view(T, G, dv), eps)
    gate = torch.sigmoid(h @ w("g").T)                       # [T, H]
    out = attention_core(q, k, v, gate, m, w("temp"), w("sink"))
    return out.reshape(T, H * dv) @ w("o").T


def short_conv_silu(x: torch.Tensor, cw: torch.Tensor) -> torch.Tensor:
    """x [T, C], cw [C, taps] (tap taps - 1 meets the current token, tap 0 the oldest); inputs before the first token are zero; then silu."""
    T, C = x.shape
    taps = cw.shape[1]
    y = torch.zeros_like(x)
    for back in range(min(taps, T)):
        y[back:] += x[:T - back] * cw[:, taps - 1 - back]
    return y * torch.sigmoid(y)


def delta_inputs(sd, pre: str, m: dict, h: torch.Tensor):
    """What enters the recurrence: q, k [T, G, d] (unit length, q times d^-1/2), v [T, H, dv], beta and decay [T, H]."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    w = lambda n: sd[pre + n].to(F64)
    q = short_conv_silu(h @ w("q").T, w("q.conv")).view(T, G, d)
    k = short_conv_silu(h @ w("k").T, w("k.conv")).view(T, G, d)
    v = short_conv_silu(h @ w("v").T, w("v.conv")).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w("b").T)
    decay = torch.exp(-torch.exp(w("A_log")) * torch.nn.functional.softplus(h @ w("a").T + w("dt_bias")))
    return q, k, v, beta, decay


def delta_core(q, k, v, beta, decay) -> torch.Tensor:
    """The recurrence from a zero state: S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q.  Returns o [T, H, dv]."""
    T, H, dv = v.shape
    G, d = q.shape[1], q.shape[2]
    o = torch.zeros(T, H, dv, dtype=F64)
    for hh in range(H):
        g = hh // (H // G)
        S = torch.zeros(d, dv, dtype=F64)
        for t in range(T):
            S = decay[t, hh] * S
            u = beta[t, hh] * (v[t, hh] - S.T @ k[t, g])
            S = S + torch.outer(k[t, g], u)
            o[t, hh] = S.T @ q[t, g]
    return o


def gated_head_norm(o, norm_w, gate_logits, eps):
    """o [T, H, dv] -> o / rms(o) * w * silu(gate) as [T, H * dv]."""
    T, H, dv = o.shape
    gate = gate_logits.view(T, H, dv)
    return (rms_divide(o, eps) * norm_w * gate * torch.sigmoid(gate)).reshape(T, H * dv)


def delta_mixer(sd, pre: str, m: dict, h: torch.Tensor, eps: float) -> torch.Tensor:
    w = lambda n: sd[pre + n].to(F64)
    o = delta_core(*delta_inputs(sd, pre, m, h))
    return gated_head_norm(o, w("norm"), h @ w("g").T, eps) @ w("o").T


def feed_forward(sd, pre: str, f: dict, h: torch.Tensor) -> torch.Tensor:
    assert f["kind"] == "dense"
    a = torch.relu(h @ sd[pre + "up"].to(F64).T)
    return (a * a) @ sd[pre + "down"].to(F64).T


def layer(sd, cfg: dict, i: int, x: torch.Tensor) -> torch.Tensor:
    lay, eps = cfg["layers"][i], cfg["norm"]["eps"]
    h = rms_norm(x, sd[f"l{i}.norm1"].to(F64), eps)
    mix = {"attention": attention_mixer, "delta": delta_mixer}[lay["type"]]
    x = x + mix(sd, f"l{i}.mix.", lay["mixer"], h, eps)
    if lay.get("mlp") is not None:
        x = x + feed_forward(sd, f"l{i}.mlp.", lay["mlp"], rms_norm(x, sd[f"l{i}.norm2"].to(F64), eps))
    return x


def run_order(cfg: dict) -> List[tuple]:
    """(layer index, starts a pass of the loop) for every layer run, in execution order."""
    L, loop = len(cfg["layers"]), cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(L)]
    a, b, n = loop["start"], loop["stop"], loop["times"]
    order = [(i, False) for i in range(a)]
    for _ in range(n):
        order += [(i, i == a) for i in range(a, b)]
    return order + [(i, False) for i in range(b, L)]


def forward(sd: Dict[str, torch.Tensor], cfg: dict, tokens: List[int], want_layers: bool = False):
    """Logits [T, vocab] of one sequence (and, if asked, the residual stream after every layer run [runs, T, W])."""
    W = cfg["width"]
    x0 = embedding(sd, tokens, W)
    x, trace = x0, []
    for i, first in run_order(cfg):
        if first:
            x = torch.cat([x, x0], -1) @ sd["loop.in"].to(F64).T
        x = layer(sd, cfg, i, x)
        trace.append(x)
    x = rms_norm(x, sd["final.norm"].to(F64), cfg["norm"]["eps"])
    logits = (x @ sd["head"].to(F64).T) * cfg.get("logit_scale", 1.0)
    return (logits, torch.stack(trace)) if want_layers else logits


def greedy(sd, cfg, prompt: List[int], n_new: int) -> List[int]:
    toks, out = list(prompt), []
    for _ in range(n_new):
        nxt = int(forward(sd, cfg, toks)[-1].argmax())
        out.append(nxt)
        toks.append(nxt)
    return out


# ---------------------------------------------------------------------------------------------- random checkpoints for tests


def tensor_shapes(cfg: dict) -> Dict[str, tuple]:
    W = cfg["width"]
    s = {"embed": (cfg["vocab"], W), "head": (cfg["vocab"], W), "final.norm": (W,)}
    if cfg.get("loop"):
        s["loop.in"] = (W, 2 * W)
    for i, lay in enumerate(cfg["layers"]):
        m, p = lay["mixer"], f"l{i}."
        H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        s[p + "norm1"] = (W,)
        if lay["type"] == "attention":
            s.update({p + "mix.q": (H * d, W), p + "mix.q.b": (H * d,), p + "mix.k": (G * d, W), p + "mix.k.b": (G * d,),
                      p + "mix.v": (G * dv, W), p + "mix.v.b": (G * dv,), p + "mix.temp": (H,), p + "mix.sink": (H,),
                      p + "mix.g": (H, W), p + "mix.o": (W, H * dv)})
        else:
            t = m["conv"]
            s.update({p + "mix.q": (G * d, W), p + "mix.q.conv": (G * d, t), p + "mix.k": (G * d, W), p + "mix.k.conv": (G * d, t),
                      p + "mix.v": (H * dv, W), p + "mix.v.conv": (H * dv, t), p + "mix.b": (H, W), p + "mix.A_log": (H,),
                      p + "mix.norm": (dv,), p + "mix.a": (H, W), p + "mix.dt_bias": (H,), p + "mix.g": (H * dv, W),
                      p + "mix.o": (W, H * dv)})
        if lay.get("mlp") is not None:
            s.update({p + "norm2": (W,), p + "mlp.up": (lay["mlp"]["ff"], W), p + "mlp.down": (W, lay["mlp"]["ff"])})
    return s


def random_checkpoint(cfg: dict, seed: int = 0, dtype=torch.bfloat16) -> Dict[str, torch.Tensor]:
    """Random weights whose scales keep every mechanism alive: activations of order one, decays spread over (0, 1), sinks and
    temperatures that differ between heads."""
    g = torch.Generator().manual_seed(seed)
    sd = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.rsplit(".", 1)[-1]
        if name.endswith(("norm1", "norm2", "final.norm", "mix.norm")):
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif last == "temp":
            t = 0.6 + torch.rand(shape, generator=g)
        elif last == "sink":
            t = torch.randn(shape, generator=g)
        elif last == "A_log":
            t = torch.log(0.2 + 3.0 * torch.rand(shape, generator=g))
        elif last == "dt_bias":
            t = torch.randn(shape, generator=g) - 1.0
        elif last == "conv":
            t = torch.randn(shape, generator=g) / math.sqrt(shape[1])
        elif name.endswith(".b") and len(shape) == 1:
            t = 0.3 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) * (1.5 / math.sqrt(shape[-1]))
        sd[name] = t.to(dtype)
    return sd
