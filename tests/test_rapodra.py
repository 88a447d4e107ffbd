"""Rapodra (heterogeneous stack: grouped sandwich norms, short causal convolutions, windowed latent attention with shared
latents, clamped GLU / MoE feed-forwards, capped logits) against the plain float64 implementation in `rapodra_oracle.py`.

Every test body runs on the CPU (the op layer's PyTorch references, part of the default suite) and, marked `gpu`, on CUDA (the
sm_100a kernels) in fp32 and bf16.  Configurations are small and made here; none is a released model's."""

import json
import math
import os

import pytest
import torch

import rapodra_oracle as O
from realhf_b200.api.model import GenerationHyperparameters
from realhf_b200.models import generation as gen
from realhf_b200.models import hf_io
from realhf_b200.models.real_model import ReaLModel
from realhf_b200.ops import attention as A
from realhf_b200.ops import functional as OF

CPU = pytest.param("cpu", torch.float32, id="cpu-f32")
GPU32 = pytest.param("cuda", torch.float32, id="cuda-f32", marks=pytest.mark.gpu)
GPU16 = pytest.param("cuda", torch.bfloat16, id="cuda-bf16", marks=pytest.mark.gpu)
ALL = [CPU, GPU32, GPU16]
EXACT = [CPU, GPU32]


def tol(dtype):
    return 2e-4 if dtype == torch.float32 else 0.12


def row_errs(got, want):
    """Per row: root mean square of the difference (mean removed) over the last dim, relative to the spread of `want`."""
    d = got.double().cpu() - want.double()
    d = d - d.mean(-1, keepdim=True)
    return (d.pow(2).mean(-1).sqrt() / want.double().std(-1).clamp_min(1e-6)).reshape(-1)


def rel_err(got, want):
    return float(row_errs(got, want).max())


def model_ok(errs, dtype):
    """fp32: every position within tolerance.  bf16: rounding may flip a discrete choice of these random models (an expert of
    nearly equal router logit, a clamp), which changes single positions wholesale: at most one position in ten may be off."""
    errs = torch.cat([e.reshape(-1) for e in errs]) if isinstance(errs, (list, tuple)) else errs
    if dtype == torch.float32:
        return float(errs.max()) < tol(dtype)
    return float((errs > tol(dtype)).float().mean()) <= 0.1


def build(cfg: dict, w: dict, device, dtype) -> ReaLModel:
    fam = hf_io.family("rapodra")
    rc = fam.config_from_dict(cfg, False)
    m = ReaLModel(rc, dtype=dtype, device=device).instantiate(init="empty")
    m.load_state_dict(fam.sd_from_hf(w, rc))
    for p in m.parameters():
        p.requires_grad_(False)
    return m.eval()


def toks(n, vocab, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def packed_logits(m, seqs):
    dev = m.device
    ids = torch.tensor([x for s in seqs for x in s], device=dev)
    cu = torch.tensor([0] + [len(s) for s in seqs], device=dev).cumsum(0).int()
    with torch.no_grad():
        return m(input_ids=ids, cu_seqlens=cu).logits


# ------------------------------------------------------------------------------------------------ mechanisms alone


@pytest.mark.parametrize("device,dtype", ALL)
@pytest.mark.parametrize("W,groups,taps", [(48, 3, 3), (64, 1, 1), (40, 5, 2), (32, 4, 4), (24, 2, 0)])
def test_sublayer_input_packed_and_step(device, dtype, W, groups, taps):
    g = torch.Generator().manual_seed(W + taps)
    lens = [1, 2, 5, 9, 3]
    T = sum(lens)
    x = torch.randn(T, W, generator=g) * 3
    w = (1 + 0.3 * torch.randn(W, generator=g)).to(dtype)
    cw = (0.5 * torch.randn(W, taps, generator=g)).to(dtype) if taps else None
    want, off = [], 0
    for n in lens:
        nrm = O.grouped_rms_norm(x[off:off + n], w, groups, 1e-5)
        want.append(O.canon(nrm, cw) if taps else nrm)
        off += n
    want = torch.cat(want)
    cu = torch.tensor([0] + lens).cumsum(0).int().to(device)
    from realhf_b200.models.hetero_block import packed_meta
    slots = torch.tensor([4, 0, 2, 1, 3], dtype=torch.int32, device=device)
    meta = packed_meta(cu, T, slots)
    state = torch.zeros(5, max(taps - 1, 0), W, device=device)
    xd = x.to(device)
    got = OF.sublayer_input(xd, w.to(device), groups, 1e-5, cw.to(device) if taps else None, meta.pos, dtype, state if taps > 1 else None,
                            meta.tok_slot, meta.remain)
    assert rel_err(got, want) < (1e-5 if dtype == torch.float32 else 0.02)
    if taps > 1:
        # the state left behind continues every sequence: one more token per sequence through the step form
        x2 = torch.randn(len(lens), W, generator=g)
        got2 = OF.sublayer_input_step(x2.to(device), w.to(device), groups, 1e-5, cw.to(device), state, slots, dtype)
        off = 0
        for b, n in enumerate(lens):
            full = torch.cat([x[off:off + n], x2[b:b + 1]])
            ref = O.canon(O.grouped_rms_norm(full, w, groups, 1e-5), cw)[-1:]
            assert rel_err(got2[b:b + 1], ref) < (1e-5 if dtype == torch.float32 else 0.02), (b, n)
            off += n


@pytest.mark.parametrize("device,dtype", ALL)
@pytest.mark.parametrize("W,groups,taps", [(64, 4, 4), (96, 1, 2), (32, 8, 5)])
def test_sublayer_input_long_packed_batch(device, dtype, W, groups, taps):
    """Thousands of packed tokens (on CUDA the token-tiled kernel): sequences that start and end inside, at the first and at the
    last row of a tile, and the state every sequence leaves behind."""
    g = torch.Generator().manual_seed(taps)
    lens = [1, 7, 8, 9, 2, 1, 1500, 3, 16, 1700, 5, 24, 1, 1800, 2, 40]
    T = sum(lens)
    x = torch.randn(T, W, generator=g) * 2
    w = (1 + 0.3 * torch.randn(W, generator=g)).to(dtype)
    cw = (0.5 * torch.randn(W, taps, generator=g)).to(dtype)
    nrm = O.grouped_rms_norm(x, w, groups, 1e-5)
    want = nrm.clone()
    pos = torch.cat([torch.arange(n) for n in lens])
    for j in range(taps):
        back = taps - 1 - j
        src = torch.zeros_like(nrm)
        src[back:] = nrm[: T - back] if back else nrm
        want += torch.where((pos >= back).unsqueeze(-1), src, torch.zeros_like(src)) * cw[:, j].double()
    from realhf_b200.models.hetero_block import packed_meta
    slots = torch.randperm(len(lens), generator=g).int().to(device)
    meta = packed_meta(torch.tensor([0] + lens).cumsum(0).int().to(device), T, slots)
    state = torch.zeros(len(lens), taps - 1, W, device=device)
    got = OF.sublayer_input(x.to(device), w.to(device), groups, 1e-5, cw.to(device), meta.pos, dtype, state, meta.tok_slot, meta.remain)
    assert rel_err(got, want) < (1e-5 if dtype == torch.float32 else 0.02)
    off = 0
    for b, n in enumerate(lens):
        tail = torch.zeros(taps - 1, W, dtype=torch.float64)
        k = min(n, taps - 1)
        tail[taps - 1 - k:] = nrm[off + n - k: off + n]
        assert torch.allclose(state[int(slots[b])].double().cpu(), tail, atol=1e-5), (b, n)
        off += n


@pytest.mark.parametrize("device,dtype", ALL)
def test_residual_add_norm_clamped_glu_softcap(device, dtype):
    g = torch.Generator().manual_seed(5)
    x = torch.randn(7, 36, generator=g)
    y = (torch.randn(7, 36, generator=g) * 4).to(dtype)
    w = (1 + 0.2 * torch.randn(36, generator=g)).to(dtype)
    want = x.double() + O.grouped_rms_norm(y, w, 3, 1e-5)
    got = OF.residual_add_norm_(x.clone().to(device), y.to(device), w.to(device), 3, 1e-5)
    assert got.dtype == torch.float32 and rel_err(got, want) < 1e-5
    got = OF.residual_add_norm_(x.clone().to(device), y.to(device), None, 1, 1e-5)
    assert rel_err(got, x.double() + y.double()) < 1e-6
    gu = (torch.randn(9, 2 * 20, generator=g) * 3).to(dtype)
    gg, uu = gu[:, :20].double().clamp(max=1.5), gu[:, 20:].double().clamp(-1.5, 1.5)
    want = gg * torch.sigmoid(1.702 * gg) * (uu + 1)
    assert rel_err(OF.clamped_glu(gu.to(device), 1.5, 1.702), want) < (1e-5 if dtype == torch.float32 else 0.02)
    lg = (torch.randn(4, 33, generator=g) * 40).to(dtype)
    got = OF.softcap_logits(lg.to(device), 30.0)
    assert got.dtype == torch.float32 and rel_err(got, 30 * torch.tanh(lg.double() / 30)) < 1e-5


@pytest.mark.parametrize("device,dtype", ALL)
@pytest.mark.parametrize("T,W,F", [(300, 64, 96), (40, 64, 96), (513, 128, 264)])
def test_clamped_gated_linear(device, dtype, T, W, F):
    """Projection + clamped GLU; on CUDA, 16-bit inputs of more than 128 rows take the GEMM-epilogue form."""
    g = torch.Generator().manual_seed(T)
    x = torch.randn(T, W, generator=g).to(dtype)
    w = (torch.randn(2 * F, W, generator=g) * 2 / math.sqrt(W)).to(dtype)
    gu = (x.double() @ w.double().t()).to(dtype).double()          # the projection is rounded to the compute type first
    gg, uu = gu[:, :F].clamp(max=1.25), gu[:, F:].clamp(-1.25, 1.25)
    want = gg * torch.sigmoid(1.702 * gg) * (uu + 1)
    got = OF.clamped_gated_linear(x.to(device), w.to(device), 1.25, 1.702)
    assert rel_err(got, want) < (1e-4 if dtype == torch.float32 else 0.03)


def _attn_inputs(T, H, qk, vd, seed, dtype):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(T, H * qk + 5, generator=g).to(dtype)        # wider than the queries: like the fused q|latent projection
    kv = torch.randn(T, H * (qk + vd), generator=g).to(dtype)
    return q, kv


def _attn_ref(q, kv, lens, H, qk, vd, scale, window):
    out, off = [], 0
    for n in lens:
        qh = q[off:off + n, : H * qk].double().view(n, H, qk)
        kh = kv[off:off + n, : H * qk].double().view(n, H, qk)
        vh = kv[off:off + n, H * qk:].double().view(n, H, vd)
        o = torch.zeros(n, H, vd, dtype=torch.float64)
        for i in range(n):
            lo = 0 if window is None else max(0, i - window + 1)
            for h in range(H):
                p = torch.softmax((kh[lo:i + 1, h] @ qh[i, h]) * scale, 0)
                o[i, h] = p @ vh[lo:i + 1, h]
        out.append(o.reshape(n, H * vd))
        off += n
    return torch.cat(out)


@pytest.mark.parametrize("device,dtype", ALL)
@pytest.mark.parametrize("H,qk,vd,window", [(2, 16, 8, 7), (1, 8, 24, 1), (3, 24, 24, None), (2, 32, 72, 40), (4, 16, 16, 33)])
def test_window_attention_packed(device, dtype, H, qk, vd, window):
    lens = [1, 50, 2, 37, 16, 3]
    T = sum(lens)
    q, kv = _attn_inputs(T, H, qk, vd, 11, dtype)
    from realhf_b200.models.hetero_block import packed_meta
    meta = packed_meta(torch.tensor([0] + lens).cumsum(0).int().to(device), T)
    got = A.latent_window_attention(q.to(device), kv.to(device), meta.pos, H, qk, vd, 0.3, window)
    want = _attn_ref(q, kv, lens, H, qk, vd, 0.3, window)
    assert rel_err(got, want) < (1e-5 if dtype == torch.float32 else 0.02)


@pytest.mark.parametrize("device,dtype", [CPU, GPU16])
@pytest.mark.parametrize("H,d,window", [(2, 64, 100), (1, 128, 128), (2, 64, 129), (1, 64, 400), (1, 128, None), (2, 64, 1)])
def test_window_attention_tensor_core_shapes(device, dtype, H, d, window):
    """Equal query / value head dims of 64 / 128 in 16 bits: on CUDA the tcgen05 varlen kernel with its window mask.  Sequences
    cross several 128-key tiles; windows below, at and above a tile."""
    lens = [300, 1, 513, 129, 128]
    T = sum(lens)
    q, kv = _attn_inputs(T, H, d, d, 13, dtype)
    q = q[:, : H * d + 0].contiguous() if device == "cpu" else torch.cat([q[:, : H * d], q[:, :8]], 1).contiguous()   # 16-byte row pitch
    from realhf_b200.models.hetero_block import packed_meta
    cu = torch.tensor([0] + lens).cumsum(0).int().to(device)
    meta = packed_meta(cu, T, max_seqlen=max(lens))
    got = A.latent_window_attention(q.to(device), kv.to(device), meta.pos, H, d, d, d ** -0.5, window, meta.cu_seqlens, meta.max_seqlen)
    want = _attn_ref(q, kv, lens, H, d, d, d ** -0.5, window)
    assert rel_err(got, want) < (1e-5 if dtype == torch.float32 else 0.03)


@pytest.mark.parametrize("device,dtype", EXACT)
def test_window_edge_in_prompt_one_key_stands_out(device, dtype):
    """One key is given a score far above all others: a query sees it exactly while it is inside the window."""
    H, qk, vd, window, n = 1, 8, 4, 6, 40
    q = torch.zeros(n, qk)
    kv = torch.zeros(n, qk + vd)
    q[:, 0] = 1.0
    star = 20
    kv[star, 0] = 60.0                    # score 60 against 0 for every other key
    kv[:, qk:] = torch.arange(n).float().unsqueeze(1).expand(n, vd) * 0 + 1.0
    kv[star, qk:] = 100.0
    pos = torch.arange(n, dtype=torch.int32, device=device)
    out = A.latent_window_attention(q.to(device), kv.to(device), pos, H, qk, vd, 1.0, window).cpu()
    for i in range(n):
        seen = star <= i < star + window
        assert (out[i, 0] > 99.0) == seen, (i, float(out[i, 0]))
        if not seen:
            assert abs(float(out[i, 0]) - 1.0) < 1e-5


@pytest.mark.parametrize("device,dtype", ALL)
@pytest.mark.parametrize("impl", ["split", "fused"])
@pytest.mark.parametrize("H,qk,vd,rank,window,R", [(2, 16, 8, 24, 7, 7), (3, 8, 16, 40, 5, 11), (1, 32, 32, 16, None, 64), (2, 16, 24, 33, 1, 1)])
def test_latent_decode_attention_ring(device, dtype, H, qk, vd, rank, window, R, impl, monkeypatch):
    """Token-by-token decode over a ring cache, rows in shuffled slots, one row appended per step by an owning block and read
    back by a sharing block, against whole-sequence attention over up-projected keys / values.  Both CUDA forms of the op."""
    if impl == "fused" and device == "cpu":
        pytest.skip("one reference on the CPU")
    monkeypatch.setenv("REAL_LATENT_DECODE", impl)
    g = torch.Generator().manual_seed(rank)
    B, n = 3, 30
    w_ukv = (torch.randn(H * (qk + vd), rank, generator=g) / math.sqrt(rank)).to(dtype)
    w_ln = (1 + 0.1 * torch.randn(rank, generator=g)).to(dtype)
    qc = torch.randn(B, n, H * qk + rank, generator=g).to(dtype)
    cache = torch.zeros(5, R, rank, dtype=dtype, device=device)
    lens = torch.zeros(5, dtype=torch.int32, device=device)
    slots = torch.tensor([3, 0, 4], dtype=torch.int32, device=device)
    lat = [O.latent(qc[b, :, H * qk:].double(), torch.eye(rank, dtype=torch.float64), w_ln, 1e-5).to(dtype) for b in range(B)]
    worst = 0.0
    for t in range(n):
        got = A.latent_decode_attention(qc[:, t].contiguous().to(device), w_ln.to(device), w_ukv.to(device), cache, lens, slots, H, qk, vd,
                                        0.25, window, 1e-5)
        got2 = A.latent_decode_attention(qc[:, t, : H * qk].contiguous().to(device), None, w_ukv.to(device), cache, lens, slots, H, qk, vd,
                                         0.25, window, 1e-5)
        lens[slots.long()] += 1
        for b in range(B):
            kvb = lat[b][: t + 1].double() @ w_ukv.double().t()
            want = _attn_ref(qc[b, : t + 1], kvb, [t + 1], H, qk, vd, 0.25, window)[-1:]
            worst = max(worst, rel_err(got[b:b + 1], want), rel_err(got2[b:b + 1], want))
    assert worst < (2e-5 if dtype == torch.float32 else 0.03)


@pytest.mark.parametrize("device,dtype", ALL)
@pytest.mark.parametrize("H,window,R,ctx", [(3, None, 256, 200), (20, 130, 256, 700), (1, 192, 192, 191), (17, 64, 128, 64)])
def test_latent_decode_long_context_key_splits_and_head_tiles(device, dtype, H, window, R, ctx):
    """One step at a long context straight from a filled ring (positions beyond R have wrapped): on CUDA several key splits per
    row, split partials merged, more heads than one head tile."""
    g = torch.Generator().manual_seed(H)
    B, qk, vd, rank = 2, 8, 8, 40
    w_ukv = (torch.randn(H * (qk + vd), rank, generator=g) / math.sqrt(rank)).to(dtype)
    lat = torch.randn(B, ctx + 1, rank, generator=g).to(dtype)            # latents of positions 0 .. ctx (the new token included)
    cache = torch.zeros(B, R, rank, dtype=dtype)
    for p_ in range(max(0, ctx + 1 - R), ctx + 1):
        cache[:, p_ % R] = lat[:, p_]
    q = (torch.randn(B, H * qk, generator=g) * 2).to(dtype)
    lens = torch.full((B,), ctx, dtype=torch.int32, device=device)
    got = A.latent_decode_attention(q.to(device), None, w_ukv.to(device), cache.to(device), lens, None, H, qk, vd, 0.3, window, 1e-5)
    for b in range(B):
        kvb = lat[b].double() @ w_ukv.double().t()
        kh = kvb[:, : H * qk].view(ctx + 1, H, qk)
        vh = kvb[:, H * qk:].view(ctx + 1, H, vd)
        lo = 0 if window is None else max(0, ctx - window + 1)
        want = torch.stack([torch.softmax((kh[lo:, h] @ q[b].double().view(H, qk)[h]) * 0.3, 0) @ vh[lo:, h] for h in range(H)]).reshape(1, -1)
        assert rel_err(got[b:b + 1], want) < (2e-5 if dtype == torch.float32 else 0.03), b


@pytest.mark.parametrize("device,dtype", EXACT)
def test_window_edge_in_decode_one_key_stands_out(device, dtype):
    H, qk, vd, rank, window = 1, 4, 4, 4, 5
    w_ukv = torch.cat([torch.eye(rank), torch.eye(rank)])            # keys = values = the latent itself
    cache = torch.zeros(1, window, rank, device=device)
    lens = torch.zeros(1, dtype=torch.int32, device=device)
    star = 7
    for t in range(20):
        qc = torch.zeros(1, H * qk + rank)
        qc[0, 0] = 50.0                                               # query looks at latent coordinate 0
        qc[0, H * qk:] = torch.tensor([4.0, 1.0, 1.0, 1.0]) if t == star else torch.tensor([0.0, 1.0, 1.0, 1.0])
        out = A.latent_decode_attention(qc.to(device), torch.ones(rank, device=device), w_ukv.to(device), cache, lens, None, H, qk, vd, 1.0,
                                        window, 1e-5).cpu()
        lens += 1
        seen = star <= t < star + window
        assert (out[0, 0] > 1.5) == seen, (t, out)


@pytest.mark.parametrize("device,dtype", ALL)
@pytest.mark.parametrize("E,top", [(5, 2), (3, 1), (4, 4)])
def test_moe_router_bias_topk(device, dtype, E, top):
    layers = [dict(type="latent_attention", mixer=dict(dim=8, heads=1, kv_rank=8, vdim=8, scale=0.3, mask=dict(size=4)),
                   mlp=dict(kind="moe", expert=dict(ff=16), router=dict(experts=E, top=top)))]
    cfg = O.random_config(width=32, vocab=32, groups=2, taps=2, layers=layers)
    w = O.random_weights(cfg, 9)
    w["l0.mlp.router.b"] = torch.linspace(-2, 2, E).to(torch.bfloat16)     # the bias decides between close experts
    m = build(cfg, w, device, dtype)
    from realhf_b200.models import moe
    h = torch.randn(21, 32, generator=torch.Generator().manual_seed(1)).to(dtype)
    got = moe.moe_forward(m, 1, h.to(device), m.config.blocks[0].mlp.moe)
    ex = [(w[f"l0.mlp.e{e}.gate"], w[f"l0.mlp.e{e}.up"], w[f"l0.mlp.e{e}.down"]) for e in range(E)]
    want = O.moe_ff(h, w["l0.mlp.router"], w["l0.mlp.router.b"], ex, top)
    assert got.dtype == torch.float32 and rel_err(got, want) < (1e-5 if dtype == torch.float32 else 0.03)


# ------------------------------------------------------------------------------------------------ whole model

CONFIGS = {
    "mixed": lambda: O.random_config(),
    "tc64": lambda: O.random_config(width=64, vocab=64, groups=4, taps=4, softcap=30.0, layers=[
        dict(type="latent_attention", mixer=dict(dim=64, heads=2, kv_rank=32, vdim=64, scale=0.125, mask=dict(size=20)),
             mlp=dict(kind="dense", ff=64, limit=4.0)),
        dict(type="latent_attention", mixer=dict(dim=64, heads=1, kv_rank=32, vdim=64, scale=0.125, mask=dict(size=33), kv_from=0),
             mlp=dict(kind="moe", expert=dict(ff=32), router=dict(experts=4, top=2)))]),
    "ones": lambda: O.random_config(width=32, vocab=40, groups=1, taps=1, softcap=None, layers=[
        dict(type="latent_attention", mixer=dict(dim=8, heads=1, kv_rank=8, vdim=8, scale=0.35, mask=dict(size=1)),
             mlp=dict(kind="moe", expert=dict(ff=8), router=dict(experts=2, top=1))),
        dict(type="latent_attention", mixer=dict(dim=8, heads=4, kv_rank=8, vdim=8, scale=0.35, mask=dict(size=64), kv_from=0),
             mlp=dict(kind="dense", ff=8, limit=0.5))]),
    "wide": lambda: O.random_config(width=64, vocab=96, groups=8, taps=5, softcap=8.0, layers=[
        dict(type="latent_attention", mixer=dict(dim=24, heads=2, kv_rank=40, vdim=40, scale=0.2, mask=dict(size=9)),
             mlp=dict(kind="moe", expert=dict(ff=24), router=dict(experts=6, top=3))),
        dict(type="latent_attention", mixer=dict(dim=16, heads=3, kv_rank=16, vdim=8, scale=0.3, mask=dict(size=13)), mlp=None),
        dict(type="latent_attention", mixer=dict(dim=8, heads=2, kv_rank=40, vdim=16, scale=0.3, mask=dict(size=4), kv_from=0),
             mlp=dict(kind="dense", ff=56, limit=3.0))]),
}


@pytest.mark.parametrize("device,dtype", ALL)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_packed_forward_matches_oracle(device, dtype, name):
    cfg = CONFIGS[name]()
    w = O.random_weights(cfg, 1)
    m = build(cfg, w, device, dtype)
    seqs = [toks(n, cfg["vocab"], n) for n in (23, 1, 2, 40, 3)]
    got = packed_logits(m, seqs)
    want = torch.cat([O.forward(cfg, w, s) for s in seqs])
    assert got.dtype == (torch.float32 if cfg["logit_softcap"] else dtype)      # capped logits are fp32
    assert model_ok(row_errs(got, want), dtype)


@pytest.mark.parametrize("device,dtype", ALL)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_session_prefill_decode_batches_and_slot_reuse(device, dtype, name):
    """Unequal requests prefetched as one batch (cut after 1, 2, many tokens), decoded together for 60+ steps while the short ones
    end and new requests take over their slots; every logit against the whole-sequence oracle of its request alone."""
    cfg = CONFIGS[name]()
    w = O.random_weights(cfg, 2)
    m = build(cfg, w, device, dtype)
    V = cfg["vocab"]
    seqs = {r: toks(n, V, 100 + r) for r, n in enumerate((70, 9, 31, 2, 45, 66, 12))}
    ref = {r: O.forward(cfg, w, s) for r, s in seqs.items()}
    cut = {0: 1, 1: 2, 2: 17, 3: 1, 4: 30, 5: 3, 6: 12}
    sess = gen.StepSession(m, max_len=80, n_slots=2)           # grows once, then reuses
    waves = [[0, 1, 2, 3], [4, 5], [6]]
    at, errs, used_slots = {}, [], []

    def start(wave):
        h = sess.prefill([(r, seqs[r][: cut[r]]) for r in wave])
        errs.append(row_errs(sess.logits(h), torch.cat([ref[r][: cut[r]] for r in wave])))
        for r in wave:
            at[r] = cut[r]
            used_slots.append(sess.slot_of[r])

    start(waves.pop(0))
    while at:
        done = [r for r in at if at[r] >= len(seqs[r])]
        if done:
            sess.release(done)
            for r in done:
                del at[r]
            if waves and len(at) <= 2:
                start(waves.pop(0))
            continue
        live = sorted(at)
        h = sess.decode([(r, seqs[r][at[r]]) for r in live])
        errs.append(row_errs(sess.logits(h), torch.stack([ref[r][at[r]] for r in live])))
        for r in live:
            at[r] += 1
    assert len(set(used_slots)) < len(used_slots)              # some slot served two requests
    assert model_ok(errs, dtype), float(torch.cat(errs).max())


@pytest.mark.parametrize("device,dtype", EXACT)
def test_far_key_through_the_model_window(device, dtype):
    """The logits at a position change with a token just inside the attention window of the widest block and do not change with
    one just outside the reach of the whole stack (windows and convolutions add up over layers)."""
    cfg = O.random_config(taps=2)
    w = O.random_weights(cfg, 4)
    m = build(cfg, w, device, dtype)
    reach = sum(l["mixer"]["mask"]["size"] - 1 for l in cfg["layers"]) + 2 * len(cfg["layers"]) * (cfg["canon"]["taps"] - 1)
    n = reach + 12
    base = toks(n, cfg["vocab"], 7)
    last = packed_logits(m, [base])[-1]
    far = list(base)
    far[n - 1 - reach - 1] = (far[n - 1 - reach - 1] + 1) % cfg["vocab"]
    assert torch.allclose(packed_logits(m, [far])[-1], last, rtol=0, atol=1e-5)
    near = list(base)
    k = n - 1 - (cfg["layers"][0]["mixer"]["mask"]["size"] - 1)
    near[k] = (near[k] + 1) % cfg["vocab"]
    assert not torch.allclose(packed_logits(m, [near])[-1], last, rtol=0, atol=1e-3)


@pytest.mark.parametrize("device,dtype", EXACT)
def test_greedy_generation_through_generate_and_inflight_batcher(device, dtype):
    cfg = CONFIGS["mixed"]()
    w = O.random_weights(cfg, 6)
    m = build(cfg, w, device, dtype)
    V, n_new = cfg["vocab"], 12
    prompts = [toks(n, V, 50 + n) for n in (5, 1, 14)]

    def oracle_greedy(p):
        s = list(p)
        for _ in range(n_new):
            s.append(int(O.forward(cfg, w, s)[-1].argmax()))
        return s[len(p):]

    want = [oracle_greedy(p) for p in prompts]
    g = GenerationHyperparameters(max_new_tokens=n_new, min_new_tokens=n_new, greedy=True, use_cuda_graph=(device == "cuda"))
    ids = torch.tensor([x for p in prompts for x in p], device=device)
    cu = torch.tensor([0] + [len(p) for p in prompts], device=device).cumsum(0).int()
    out, _ = gen.generate(m, ids, cu, g, eos_id=None, pad_id=0)
    assert out.tokens.tolist() == want
    ib = gen.InflightBatchingGenerator(m, g, eos_id=None, pad_id=0, n_slots=2, max_prompt_len=16)
    res = ib.generate([torch.tensor(p, device=device) for p in prompts])
    assert [r[0] for r in res] == want


def test_checkpoint_roundtrip_and_family_detection(tmp_path):
    from safetensors.torch import save_file
    cfg = CONFIGS["wide"]()
    w = O.random_weights(cfg, 8)
    d = str(tmp_path / "ckpt")
    os.makedirs(d)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: v.contiguous() for k, v in w.items()}, os.path.join(d, "model.safetensors"))
    assert hf_io.family_of_path(d) == "rapodra"
    m = hf_io.from_hf("rapodra", d, dtype=torch.float32, device="cpu")
    fam = hf_io.family("rapodra")
    assert fam.config_to_dict(m.config) == cfg
    back = fam.sd_to_hf(m.state_dict(), m.config)
    assert set(back) == set(w) and all(torch.equal(back[k].to(w[k].dtype), w[k]) for k in w)
    seq = toks(20, cfg["vocab"], 3)
    assert rel_err(packed_logits(m.eval(), [seq]), O.forward(cfg, w, seq)) < 2e-4


def test_family_through_registry_factory_backend_and_engine():
    """The family as the rest of the framework reaches it: model registry -> `real_model` factory -> inference backend ->
    `ReaLEngine.generate` / `forward` on a packed `SequenceSample`."""
    import realhf_b200.engine.engine  # noqa: F401  (registers the backends)
    import realhf_b200.models.factory  # noqa: F401  (registers `real_model`)
    from realhf_b200.api import model as model_api
    from realhf_b200.api.config import ModelAbstraction, ModelBackendAbstraction, ModelName
    from realhf_b200.api.data import SequenceSample
    from realhf_b200.api.model import FinetuneSpec
    m = model_api.make_model(ModelAbstraction("real_model", args=dict(model_path="", is_critic=False, init_from_scratch=True, dtype="fp32",
                                                                      hf_model_family="rapodra")), ModelName("actor", 0), "cpu")
    assert m.module.config.blocks is not None and m.module.config.blocks[1].attn.kv_from == 0
    m = model_api.make_backend(ModelBackendAbstraction("inference")).initialize(m, FinetuneSpec(1, 1, 1))
    lens = [5, 9, 3]
    ids = torch.randint(3, 100, (sum(lens),))
    x = SequenceSample.from_default(seqlens=lens, ids=list(range(3)), data=dict(packed_input_ids=ids))
    g = GenerationHyperparameters(max_new_tokens=6, min_new_tokens=6, greedy=True)
    out = m.module.generate(x, m.tokenizer, g)[0]
    assert tuple(out.tokens.shape) == (3, 6)
    # the engine's greedy tokens are the argmax of a packed forward over prompt + generated tokens
    seqs = [ids[a:b].tolist() + out.tokens[i].tolist() for i, (a, b) in enumerate(zip([0, 5, 14], [5, 14, 17]))]
    lg = packed_logits(m.module.module, seqs)
    off = 0
    for i, s in enumerate(seqs):
        pred = lg[off + lens[i] - 1: off + len(s) - 1].argmax(-1).tolist()
        assert pred == out.tokens[i].tolist()
        off += len(s)
