"""Tizodra (heterogeneous stack: sinusoidal positions, window attention with kept first tokens / sink / distance penalty / value norm /
output gate, gated delta rule with short convolutions, relu^2 feed-forward, a looped range of blocks) against the plain float64
implementation in `tizodra_oracle.py`.

Every test body runs on the CPU (the op layer's PyTorch references, part of the default suite) and, marked `gpu`, on CUDA (the
sm_100a kernels) in fp32 and bf16.  Configurations are small and made here; none is a released model's."""

import json
import math
import os
import subprocess
import sys

import pytest
import torch

import tizodra_oracle as O
from realhf_b200.api.model import DeltaRuleConfig, GenerationHyperparameters, WindowAttentionConfig
from realhf_b200.models import generation as gen
from realhf_b200.models import hf_io
from realhf_b200.models.real_model import ReaLModel
from realhf_b200.ops import attention as A
from realhf_b200.ops import functional as OF
from realhf_b200.ops import recurrent as R

CPU = pytest.param("cpu", torch.float32, id="cpu-f32")
GPU32 = pytest.param("cuda", torch.float32, id="cuda-f32", marks=pytest.mark.gpu)
GPU16 = pytest.param("cuda", torch.bfloat16, id="cuda-bf16", marks=pytest.mark.gpu)
ALL = [CPU, GPU32, GPU16]
EXACT = [CPU, GPU32]
F64 = torch.float64


def tol(dtype):
    return 2e-4 if dtype == torch.float32 else 0.12


def row_errs(got, want):
    """Per row: root mean square of the difference (mean removed) over the last dim, relative to the spread of `want`."""
    d = got.double().cpu() - want.double()
    d = d - d.mean(-1, keepdim=True)
    return (d.pow(2).mean(-1).sqrt() / want.double().std(-1).clamp_min(1e-6)).reshape(-1)


def close(got, want, dtype, f32=1e-5, b16=0.03):
    """Largest elementwise difference relative to the largest magnitude of `want`."""
    e = float((got.double().cpu() - want.double()).abs().max() / want.double().abs().max().clamp_min(1e-9))
    return e < (f32 if dtype == torch.float32 else b16)


def model_ok(errs, dtype):
    errs = torch.cat([e.reshape(-1) for e in errs]) if isinstance(errs, (list, tuple)) else errs
    if dtype == torch.float32:
        return float(errs.max()) < tol(dtype)
    return float((errs > tol(dtype)).float().mean()) <= 0.05


def build(cfg: dict, w: dict, device, dtype) -> ReaLModel:
    fam = hf_io.family("tizodra")
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


def pack_meta(lens, device, slots=None):
    from realhf_b200.models.hetero_block import packed_meta
    cu = torch.tensor([0] + list(lens), device=device).cumsum(0).int()
    return packed_meta(cu, int(sum(lens)), torch.tensor(slots, dtype=torch.int32, device=device) if slots is not None else None, None, max(lens))


# ------------------------------------------------------------------------------------------------ small mechanisms


@pytest.mark.parametrize("device,dtype", ALL)
@pytest.mark.parametrize("W", [32, 50, 7])
def test_embedding_with_sinusoid_far_positions_and_slots(device, dtype, W):
    g = torch.Generator().manual_seed(W)
    wte = torch.randn(40, W, generator=g).to(dtype)
    ids = torch.randint(0, 40, (9,), generator=g)
    pos = torch.tensor([0, 1, 2, 3, 100, 1023, 4095, 20000, 7], dtype=torch.int32)
    pe = O.sinusoid(20001, W)
    want = wte.to(F64)[ids] + pe[pos.long()]
    got = OF.embed_sinusoid(ids.to(device), wte.to(device), pos.to(device), 10000.0)
    assert got.dtype == torch.float32
    # fp32 angles: p * f rounds to 2^-24 p f, which is what sin / cos can move by
    assert float((got.double().cpu() - want).abs().max()) < 4e-3
    assert float((got.double().cpu() - want)[:4].abs().max()) < 2e-6
    # decode form: the position is the length of the row's slot
    lens = torch.tensor([5, 0, 77, 3], dtype=torch.int32)
    slots = torch.tensor([2, 0, 3], dtype=torch.int32)
    got = OF.embed_sinusoid(ids[:3].to(device), wte.to(device), lens.to(device), 10000.0, slots.to(device))
    want = wte.to(F64)[ids[:3]] + pe[lens[slots.long()].long()]
    assert float((got.double().cpu() - want).abs().max()) < 1e-4


@pytest.mark.parametrize("device,dtype", ALL)
def test_relu2_concat_cast_gated_head_norm(device, dtype):
    g = torch.Generator().manual_seed(3)
    x = torch.randn(13, 37, generator=g).to(dtype)
    assert close(OF.relu2(x.to(device)), torch.relu(x.to(F64)) ** 2, dtype, 1e-6, 0.01)
    a, b = torch.randn(5, 12, generator=g), torch.randn(5, 20, generator=g).to(dtype)
    got = OF.concat_cast(a.to(device), b.to(device), dtype)
    assert got.dtype == dtype and close(got, torch.cat([a.to(F64), b.to(F64)], -1), dtype, 1e-7, 0.01)
    for H, dv in ((3, 16), (1, 40), (2, 7)):
        o = torch.randn(11, H, dv, generator=g) * 5
        w = (1 + 0.3 * torch.randn(dv, generator=g)).to(dtype)
        proj = torch.randn(11, 8 + H * dv, generator=g).to(dtype)        # the gate is a column slice of a wider tensor
        want = O.gated_head_norm(o.to(F64), w.to(F64), proj[:, 8:].to(F64), 1e-5)
        got = R.gated_head_norm(o.to(device), w.to(device), proj.to(device)[:, 8:], 1e-5, dtype)
        assert got.dtype == dtype and close(got, want, dtype, 1e-5, 0.01)


# ------------------------------------------------------------------------------------------------ window attention alone


def attn_case(H, G, d, dv, window, keep, seed, dtype, lens):
    """Random projections output + per-head constants; returns (config, dict form, qkvg, temp, sink, per-sequence oracle output)."""
    g = torch.Generator().manual_seed(seed)
    T = sum(lens)
    a = WindowAttentionConfig(n_heads=H, n_kv_heads=G, qk_dim=d, v_dim=dv, scale=0.7 / math.sqrt(d), window=window, keep_first=keep)
    m = dict(scale=a.scale, mask=dict(size=window, keep_first=keep) if window is not None else None)
    pad = (H + 7) // 8 * 8
    qkvg = torch.randn(T, H * d + G * d + G * dv + pad, generator=g).to(dtype)
    qkvg[:, : H * d + G * d] *= 1.5
    temp = (0.5 + torch.rand(H, generator=g)).to(dtype)
    sink = torch.randn(H, generator=g).to(dtype)
    return a, m, qkvg, temp, sink


def attn_oracle(a, m, qkvg, temp, sink, lens, eps=1e-5):
    H, G, d, dv = a.n_heads, a.n_kv_heads, a.qk_dim, a.v_dim
    out, off = [], 0
    x = qkvg.to(F64)
    for n in lens:
        r = x[off:off + n]
        q, k = r[:, : H * d].view(n, H, d), r[:, H * d: H * d + G * d].view(n, G, d)
        v = O.rms_divide(r[:, H * d + G * d: H * d + G * d + G * dv].view(n, G, dv), eps)
        gate = torch.sigmoid(r[:, H * d + G * (d + dv): H * d + G * (d + dv) + H])
        out.append(O.attention_core(q, k, v, gate, m, temp.to(F64), sink.to(F64)).reshape(n, H * dv))
        off += n
    return torch.cat(out)


ATTN_SHAPES = [(4, 2, 8, 16, 5, 2), (1, 1, 16, 16, 1, 0), (3, 3, 6, 5, 7, 9), (2, 1, 32, 24, None, 0), (4, 4, 48, 40, 33, 3),
               (8, 2, 64, 64, 40, 40), (2, 2, 128, 72, 64, 1), (20, 1, 8, 12, 6, 1)]


@pytest.mark.parametrize("device,dtype", ALL)
@pytest.mark.parametrize("H,G,d,dv,window,keep", ATTN_SHAPES)
def test_window_attention_packed(device, dtype, H, G, d, dv, window, keep):
    lens = [1, 2, 31, 32, 33, 65, 130, 3]
    a, m, qkvg, temp, sink = attn_case(H, G, d, dv, window, keep, H * 100 + d, dtype, lens)
    want = attn_oracle(a, m, qkvg, temp, sink, lens)
    meta = pack_meta(lens, device)
    v_n = A.value_norm_store(qkvg.to(device), a, 1e-5, None, None, meta.tok_slot, meta.pos, meta.remain)
    got = A.sink_window_attention(qkvg.to(device), v_n, a, temp.to(device), sink.to(device), meta.pos, meta.cu_seqlens, max(lens))
    assert got.dtype == dtype and close(got, want, dtype, 2e-5, 0.03)


@pytest.mark.parametrize("device,dtype", [CPU, GPU16])
@pytest.mark.parametrize("H,G,d,window,keep", [(2, 1, 64, 100, 5), (1, 1, 128, 128, 0), (2, 2, 64, 129, 130), (4, 2, 64, 400, 300), (2, 1, 128, None, 0),
                                               (2, 2, 64, 1, 1), (2, 1, 128, 260, 129)])
def test_window_attention_tensor_core_shapes(device, dtype, H, G, d, window, keep, monkeypatch):
    """Head shapes the tensor-core kernel takes, windows and kept ranges below / at / above its 128-key tiles, sequences that end
    inside a tile; the all-fp32 kernel on the same input agrees."""
    lens = [600, 1, 127, 128, 129, 385]
    a, m, qkvg, temp, sink = attn_case(H, G, d, d, window, keep, H + d, dtype, lens)
    want = attn_oracle(a, m, qkvg, temp, sink, lens)
    meta = pack_meta(lens, device)
    v_n = A.value_norm_store(qkvg.to(device), a, 1e-5, None, None, meta.tok_slot, meta.pos, meta.remain)
    got = A.sink_window_attention(qkvg.to(device), v_n, a, temp.to(device), sink.to(device), meta.pos, meta.cu_seqlens, max(lens))
    assert close(got, want, dtype, 2e-5, 0.03)
    if device == "cuda":
        assert A._sink_tc_ok(qkvg.to(device), v_n, a)
        monkeypatch.setenv("REAL_WINDOW_ATTN", "simt")
        other = A.sink_window_attention(qkvg.to(device), v_n, a, temp.to(device), sink.to(device), meta.pos, meta.cu_seqlens, max(lens))
        assert close(other, want, dtype, 2e-5, 0.03) and close(got, other.double().cpu(), dtype, 2e-5, 0.03)


@pytest.mark.parametrize("device,dtype", ALL)
@pytest.mark.parametrize("H,G,d,dv,window,keep", ATTN_SHAPES)
def test_window_attention_prefill_cache_then_decode(device, dtype, H, G, d, dv, window, keep):
    """Prompts of unequal length fill shuffled slots of a cache with few rows (kept rows + a ring that wraps); then every request is
    decoded token by token, the short ones ending first.  Every step against the whole-sequence oracle."""
    prompt = [1, 2, 9, 40]
    total = [30, 70, 64, 90]
    S = 100
    lens = total
    a, m, qkvg, temp, sink = attn_case(H, G, d, dv, window, keep, H * 7 + dv, dtype, lens)
    want = attn_oracle(a, m, qkvg, temp, sink, lens)
    rows = a.cache_rows(S)
    assert rows == (S if window is None else min(S, window + keep))
    n_slots = 6
    slots = [4, 0, 5, 2]
    kc = torch.full((n_slots, G, rows, d), 7.0, dtype=dtype, device=device)          # stale content of an earlier user of the slot
    vc = torch.full((n_slots, G, rows, dv), -3.0, dtype=dtype, device=device)
    starts = [sum(total[:i]) for i in range(4)]
    pre = torch.cat([qkvg[s:s + p] for s, p in zip(starts, prompt)]).to(device)
    meta = pack_meta(prompt, device, slots)
    v_n = A.value_norm_store(pre, a, 1e-5, kc, vc, meta.tok_slot, meta.pos, meta.remain)
    got = A.sink_window_attention(pre, v_n, a, temp.to(device), sink.to(device), meta.pos, meta.cu_seqlens, max(prompt))
    assert close(got, torch.cat([want[s:s + p] for s, p in zip(starts, prompt)]), dtype, 2e-5, 0.03)
    cache_lens = torch.zeros(n_slots, dtype=torch.int32, device=device)
    cache_lens[torch.tensor(slots, device=device)] = torch.tensor(prompt, dtype=torch.int32, device=device)
    at = list(prompt)
    worst = 0.0
    while True:
        live = [i for i in range(4) if at[i] < total[i]]
        if not live:
            break
        rows_in = torch.stack([qkvg[starts[i] + at[i]] for i in live]).to(device)
        sl = torch.tensor([slots[i] for i in live], dtype=torch.int32, device=device)
        got = A.sink_window_decode_attention(rows_in, a, temp.to(device), sink.to(device), kc, vc, cache_lens, sl, 1e-5)
        w = torch.stack([want[starts[i] + at[i]] for i in live])
        worst = max(worst, float((got.double().cpu() - w).abs().max() / w.abs().max()))
        cache_lens[sl.long()] += 1
        for i in live:
            at[i] += 1
    assert worst < (2e-5 if dtype == torch.float32 else 0.03), worst


@pytest.mark.parametrize("device,dtype", ALL)
@pytest.mark.parametrize("H,G,d,window,keep,S", [(4, 2, 64, None, 0, 2048), (2, 2, 128, 384, 10, 2048), (8, 1, 64, 300, 200, 600)])
def test_window_decode_long_context_key_splits(device, dtype, H, G, d, window, keep, S):
    """Contexts of hundreds of keys (the 16-bit decode kernel cuts them into several ranges and merges the partial softmaxes), rings
    that wrap while decoding, unequal rows in one batch."""
    prompt, total = [500, 3, 390], [530, 33, 420]
    a, m, qkvg, temp, sink = attn_case(H, G, d, d, window, keep, d + H, dtype, total)
    want = attn_oracle(a, m, qkvg, temp, sink, total)
    rows = a.cache_rows(S)
    kc = torch.zeros(3, G, rows, d, dtype=dtype, device=device)
    vc = torch.zeros(3, G, rows, d, dtype=dtype, device=device)
    starts = [0, total[0], total[0] + total[1]]
    slots = [1, 2, 0]
    pre = torch.cat([qkvg[s:s + p] for s, p in zip(starts, prompt)]).to(device)
    meta = pack_meta(prompt, device, slots)
    A.value_norm_store(pre, a, 1e-5, kc, vc, meta.tok_slot, meta.pos, meta.remain)
    cache_lens = torch.zeros(3, dtype=torch.int32, device=device)
    cache_lens[torch.tensor(slots, device=device)] = torch.tensor(prompt, dtype=torch.int32, device=device)
    sl = torch.tensor(slots, dtype=torch.int32, device=device)
    worst = 0.0
    for t in range(30):
        rows_in = torch.stack([qkvg[starts[i] + prompt[i] + t] for i in range(3)]).to(device)
        got = A.sink_window_decode_attention(rows_in, a, temp.to(device), sink.to(device), kc, vc, cache_lens, sl, 1e-5)
        w = torch.stack([want[starts[i] + prompt[i] + t] for i in range(3)])
        worst = max(worst, float((got.double().cpu() - w).abs().max() / w.abs().max()))
        cache_lens[sl.long()] += 1
    assert worst < (2e-5 if dtype == torch.float32 else 0.03), worst


@pytest.mark.parametrize("device,dtype", EXACT)
@pytest.mark.parametrize("mode", ["prompt", "decode"])
def test_window_and_kept_edges_one_key_stands_out(device, dtype, mode):
    """One key carries a huge score and a value unlike all others: the output at the last position equals that value exactly when
    the key is visible.  Keys just inside / outside the window, just inside / outside the kept first tokens, and the first token."""
    H, G, d, dv, window, keep, n = 2, 1, 8, 8, 37, 5, 120
    a = WindowAttentionConfig(n_heads=H, n_kv_heads=G, qk_dim=d, v_dim=dv, scale=1.0, window=window, keep_first=keep)
    m = dict(scale=1.0, mask=dict(size=window, keep_first=keep))
    temp, sink = torch.ones(H), torch.zeros(H)
    i = n - 1
    for j, vis in ((i - window + 1, True), (i - window, False), (keep - 1, True), (keep, False), (0, True), (i, True), (i - 1, True)):
        g = torch.Generator().manual_seed(j)
        qkvg = 0.1 * torch.randn(n, H * d + G * d + G * dv + 8, generator=g)
        qkvg[i, : H * d] = 0.0
        qkvg[i, 0] = qkvg[i, d] = 30.0                          # both heads look along e0
        qkvg[j, H * d] = 30.0                                   # key j lies along e0: score 900 before the distance penalty
        qkvg[j, H * d + d:H * d + d + dv] = torch.arange(dv) * 10.0 - 35.0
        want = attn_oracle(a, m, qkvg, temp, sink, [n])[i]
        marked = O.rms_divide(qkvg[j, H * d + d:H * d + d + dv].to(F64), 1e-5)
        gate0 = torch.sigmoid(qkvg[i, H * d + d + dv].to(F64))
        assert (float((want[:dv] - marked * gate0).abs().max()) < 1e-3) == vis
        if mode == "prompt":
            meta = pack_meta([n], device)
            v_n = A.value_norm_store(qkvg.to(device), a, 1e-5, None, None, meta.tok_slot, meta.pos, meta.remain)
            got = A.sink_window_attention(qkvg.to(device), v_n, a, temp.to(device), sink.to(device), meta.pos, meta.cu_seqlens, n)[i]
        else:
            rows = a.cache_rows(n + 8)
            kc = torch.zeros(2, G, rows, d, device=device)
            vc = torch.zeros(2, G, rows, dv, device=device)
            meta = pack_meta([i], device, [1])
            A.value_norm_store(qkvg[:i].to(device), a, 1e-5, kc, vc, meta.tok_slot, meta.pos, meta.remain)
            lens = torch.tensor([0, i], dtype=torch.int32, device=device)
            got = A.sink_window_decode_attention(qkvg[i:].to(device), a, temp.to(device), sink.to(device), kc, vc, lens,
                                                 torch.tensor([1], dtype=torch.int32, device=device), 1e-5)[0]
        assert float((got.double().cpu() - want).abs().max()) < 1e-4, (j, vis)


@pytest.mark.parametrize("device,dtype", EXACT)
def test_sink_joins_the_denominator_once_and_temperature_scales_scores(device, dtype):
    """A single token: the weight of its own key is e^s / (e^s + e^sink), so the output norm tells whether the sink was counted."""
    H, d, dv = 2, 4, 4
    a = WindowAttentionConfig(n_heads=H, n_kv_heads=1, qk_dim=d, v_dim=dv, scale=0.5, window=3, keep_first=0, out_gate=True)
    qkvg = torch.zeros(1, H * d + d + dv + 8)
    qkvg[0, :d] = qkvg[0, d:2 * d] = torch.tensor([1.0, 2.0, 0.0, 0.0])
    qkvg[0, H * d:H * d + d] = torch.tensor([1.0, 1.0, 0.0, 0.0])
    qkvg[0, H * d + d:H * d + d + dv] = torch.tensor([1.0, -1.0, 1.0, -1.0])
    temp, sink = torch.tensor([1.0, 3.0]), torch.tensor([0.5, -2.0])
    meta = pack_meta([1], device)
    v_n = A.value_norm_store(qkvg.to(device), a, 1e-5, None, None, meta.tok_slot, meta.pos, meta.remain)
    got = A.sink_window_attention(qkvg.to(device), v_n, a, temp.to(device), sink.to(device), meta.pos, meta.cu_seqlens, 1).cpu().view(H, dv)
    for h in range(H):
        s = 3.0 * 0.5 * float(temp[h])
        wgt = math.exp(s) / (math.exp(s) + math.exp(float(sink[h]))) * 0.5          # gate logit 0
        assert abs(float(got[h, 0]) - wgt / math.sqrt(1 + 1e-5)) < 1e-6


# ------------------------------------------------------------------------------------------------ delta rule alone


def delta_case(H, G, d, dv, taps, seed, dtype, T):
    g = torch.Generator().manual_seed(seed)
    dl = DeltaRuleConfig(n_heads=H, n_kv_heads=G, qk_dim=d, v_dim=dv, conv_taps=taps)
    C = dl.conv_channels
    proj = torch.randn(T, C + H * dv + (2 * H + 7) // 8 * 8, generator=g).to(dtype)
    proj[:, C + H * dv:] *= 2.0
    conv_w = (torch.randn(C, taps, generator=g) / math.sqrt(taps)).to(dtype)
    A_log = torch.log(0.1 + 2.0 * torch.rand(H, generator=g)).to(dtype)
    dt_bias = (torch.randn(H, generator=g) - 1.0).to(dtype)
    return dl, proj, conv_w, A_log, dt_bias


def delta_oracle_inputs(dl, proj, conv_w, A_log, dt_bias, lens):
    """Per sequence: the oracle's q, k, v, beta, decay from the same projection outputs."""
    H, G, d, dv = dl.n_heads, dl.n_kv_heads, dl.qk_dim, dl.v_dim
    nqk, C = G * d, dl.conv_channels
    x, cw = proj.to(F64), conv_w.to(F64)
    out, off = [], 0
    for n in lens:
        r = x[off:off + n]
        y = O.short_conv_silu(r[:, :C], cw)
        q, k, v = y[:, :nqk].view(n, G, d), y[:, nqk:2 * nqk].view(n, G, d), y[:, 2 * nqk:].view(n, H, dv)
        q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
        k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
        beta = torch.sigmoid(r[:, C + H * dv:C + H * dv + H])
        decay = torch.exp(-torch.exp(A_log.to(F64)) * torch.nn.functional.softplus(r[:, C + H * dv + H:C + H * dv + 2 * H] + dt_bias.to(F64)))
        out.append((q, k, v, beta, decay))
        off += n
    return out


DELTA_SHAPES = [(4, 2, 8, 16, 4), (1, 1, 32, 32, 1), (2, 2, 48, 24, 2), (3, 1, 64, 40, 3), (2, 1, 128, 136, 4), (1, 1, 160, 8, 5), (1, 1, 272, 16, 2)]


@pytest.mark.parametrize("device,dtype", ALL)
@pytest.mark.parametrize("H,G,d,dv,taps", DELTA_SHAPES)
def test_delta_rule_prefill_then_decode(device, dtype, H, G, d, dv, taps):
    """Packed prompts (1, 2, ... tokens) into shuffled slots with stale content, then token-by-token decoding from the state the
    prompts left (convolution history and matrix state); each stage against the oracle of the whole sequence."""
    prompt, total = [1, 2, 3, 19], [12, 30, 3, 45]
    n_slots, slots = 5, [3, 0, 4, 1]
    dl, proj, conv_w, A_log, dt_bias = delta_case(H, G, d, dv, taps, H + d + taps, dtype, sum(total))
    ins = delta_oracle_inputs(dl, proj, conv_w, A_log, dt_bias, total)
    want_o = [O.delta_core(*x) for x in ins]
    starts = [sum(total[:i]) for i in range(4)]
    C = dl.conv_channels
    conv_state = torch.zeros(n_slots, taps - 1, C, device=device)
    s_state = torch.full((n_slots, H, d, dv), 9.0, device=device)               # the packed form starts from zero whatever is there
    pre = torch.cat([proj[s:s + p] for s, p in zip(starts, prompt)]).to(device)
    meta = pack_meta(prompt, device, slots)
    dev = lambda t: t.to(device)
    u = R.delta_prepare(pre, dev(conv_w), dev(A_log), dev(dt_bias), dl, meta.pos, conv_state, meta.tok_slot, meta.remain)
    assert u.dtype == torch.float32
    want_u = torch.cat([torch.cat([x[0][:p].reshape(p, -1), x[1][:p].reshape(p, -1), x[2][:p].reshape(p, -1), x[3][:p], x[4][:p]], -1)
                        for x, p in zip(ins, prompt)])
    assert close(u, want_u, dtype, 2e-6, 0.03)
    o = R.delta_rule_scan(u, dl, meta.cu_seqlens, s_state, meta.seq_slot)
    assert close(o, torch.cat([w[:p] for w, p in zip(want_o, prompt)]), dtype, 2e-5, 0.05)
    at, worst = list(prompt), 0.0
    while True:
        live = [i for i in range(4) if at[i] < total[i]]
        if not live:
            break
        rows_in = torch.stack([proj[starts[i] + at[i]] for i in live]).to(device)
        sl = torch.tensor([slots[i] for i in live], dtype=torch.int32, device=device)
        u = R.delta_prepare_step(rows_in, dev(conv_w), dev(A_log), dev(dt_bias), dl, conv_state, sl)
        o = R.delta_rule_step(u, dl, s_state, sl)
        w = torch.stack([want_o[i][at[i]] for i in live])
        worst = max(worst, float((o.double().cpu() - w).abs().max() / w.abs().max().clamp_min(1e-6)))
        for i in live:
            at[i] += 1
    assert worst < (5e-5 if dtype == torch.float32 else 0.08), worst


@pytest.mark.parametrize("device,dtype", ALL)
@pytest.mark.parametrize("H,G,d,dv,taps", [(4, 2, 8, 16, 4), (2, 2, 128, 136, 2), (3, 1, 160, 40, 1), (2, 1, 64, 64, 5)])
def test_delta_prepare_long_packed_batch(device, dtype, H, G, d, dv, taps):
    """Batches long enough for the token-tiled kernel: sequences that start and end inside a tile, the convolution history left in
    the slots, and the same rows through the per-token form (a short batch)."""
    lens = [70, 1, 33, 16, 100, 2]
    slots = [2, 5, 0, 1, 4, 3]
    dl, proj, conv_w, A_log, dt_bias = delta_case(H, G, d, dv, taps, 3 * H + d, dtype, sum(lens))
    ins = delta_oracle_inputs(dl, proj, conv_w, A_log, dt_bias, lens)
    want = torch.cat([torch.cat([x[0].reshape(n, -1), x[1].reshape(n, -1), x[2].reshape(n, -1), x[3], x[4]], -1) for x, n in zip(ins, lens)])
    C = dl.conv_channels
    dev = lambda t: t.to(device)
    state = torch.full((6, taps - 1, C), 5.0, device=device)
    meta = pack_meta(lens, device, slots)
    u = R.delta_prepare(dev(proj), dev(conv_w), dev(A_log), dev(dt_bias), dl, meta.pos, state, meta.tok_slot, meta.remain)
    assert close(u, want, dtype, 2e-6, 0.03)
    off = 0
    for n, sl in zip(lens, slots):
        have = min(n, taps - 1)
        if have:
            assert torch.equal(state[sl, taps - 1 - have:].cpu(), proj[off + n - have:off + n, :C].float())
        assert bool((state[sl, : taps - 1 - have] == 5.0).all())                      # rows of a shorter sequence are left alone
        off += n
    meta = pack_meta(lens[2:4], device)
    short = R.delta_prepare(dev(proj[71:120]), dev(conv_w), dev(A_log), dev(dt_bias), dl, meta.pos)
    assert close(short, u[71:120].double().cpu(), dtype, 2e-6, 2e-6)


@pytest.mark.parametrize("device,dtype", ALL)
def test_fused_relu2_projection_and_add_norm(device, dtype):
    g = torch.Generator().manual_seed(11)
    for T, W, F_ in ((300, 64, 96), (40, 64, 96), (513, 128, 264)):
        x = torch.randn(T, W, generator=g).to(dtype)
        w = (torch.randn(F_, W, generator=g) / math.sqrt(W)).to(dtype)
        want = torch.relu(x.to(F64) @ w.to(F64).T) ** 2
        assert close(OF.relu2_linear(x.to(device), w.to(device)), want, dtype, 1e-5, 0.03)
    x = torch.randn(37, 48, generator=g) * 3
    y = torch.randn(37, 48, generator=g).to(dtype)
    nw = (1 + 0.2 * torch.randn(48, generator=g)).to(dtype)
    xs = x.to(device).clone()
    h = OF.add_rms_norm_(xs, y.to(device), nw.to(device), 1e-5, dtype)
    s = x.to(F64) + y.to(F64)
    assert xs.dtype == torch.float32 and close(xs, s, torch.float32, 1e-6)
    assert h.dtype == dtype and close(h, O.rms_norm(s, nw.to(F64), 1e-5), dtype, 1e-5, 0.02)
    assert close(OF.sublayer_input(xs, nw.to(device), 1, 1e-5, None, None, dtype), O.rms_norm(s, nw.to(F64), 1e-5), dtype, 1e-5, 0.02)


@pytest.mark.parametrize("device,dtype", EXACT)
@pytest.mark.parametrize("mode", ["prompt", "decode"])
def test_delta_state_keeps_a_far_write(device, dtype, mode):
    """Token 0 writes a marked value under key e0; 400 tokens with keys orthogonal to e0 and decays close to one follow; the last
    token reads along e0.  A lost, re-zeroed or mis-indexed state shows as a missing value."""
    H, G, d, dv, n = 1, 1, 16, 8, 402
    dl = DeltaRuleConfig(n_heads=H, n_kv_heads=G, qk_dim=d, v_dim=dv, conv_taps=1)
    g = torch.Generator().manual_seed(0)
    q = torch.zeros(n, G, d)
    k = torch.nn.functional.normalize(torch.randn(n, G, d, generator=g), dim=-1)
    k[:, :, 0] = 0.0
    k = torch.nn.functional.normalize(k, dim=-1)
    k[0] = 0.0
    k[0, 0, 0] = 1.0
    q[-1, 0, 0] = 1.0
    v = torch.randn(n, H, dv, generator=g)
    v[0, 0] = torch.arange(dv) + 1.0
    beta = torch.full((n, H), 0.9)
    decay = torch.full((n, H), 0.9995)
    want = O.delta_core(q.to(F64), k.to(F64), v.to(F64), beta.to(F64), decay.to(F64))
    assert float(want[-1, 0, -1]) > 0.5 * dv * 0.9                      # the marked value is still there
    u = torch.cat([q.reshape(n, -1), k.reshape(n, -1), v.reshape(n, -1), beta, decay], -1).to(device)
    s_state = torch.zeros(3, H, d, dv, device=device)
    if mode == "prompt":
        cu = torch.tensor([0, n], dtype=torch.int32, device=device)
        o = R.delta_rule_scan(u, dl, cu, s_state, torch.tensor([2], dtype=torch.int32, device=device))
        assert float(s_state[2].abs().max()) > 0 and float(s_state[:2].abs().max()) == 0
    else:
        sl = torch.tensor([1], dtype=torch.int32, device=device)
        o = torch.cat([R.delta_rule_step(u[t:t + 1], dl, s_state, sl) for t in range(n)])
    assert float((o.double().cpu() - want).abs().max()) < 2e-5


# ------------------------------------------------------------------------------------------------ whole model

att = lambda **k: dict(type="attention", mixer=dict(dict(dim=8, heads=4, kv_heads=2, vdim=16, scale=0.3, mask=dict(size=5, keep_first=2)), **k),
                       mlp=dict(kind="dense", ff=48))
dlt = lambda **k: dict(type="delta", mixer=dict(dict(conv=4, dim=8, heads=4, kv_heads=2, vdim=16), **k), mlp=None)


def with_mlp(layer, mlp):
    return dict(layer, mlp=mlp)


CONFIGS = {
    # a looped pair in the middle, delta first and last
    "mixed": lambda: dict(architecture="Tizodra", layers=[dlt(), att(), with_mlp(dlt(conv=2), dict(kind="dense", ff=40)), att(), dlt()],
                          logit_scale=0.25, loop=dict(start=1, stop=3, times=2), norm=dict(eps=1e-5), vocab=96, width=32),
    # every count that can be 1 is 1; the loop covers the whole stack once
    "ones": lambda: dict(architecture="Tizodra", layers=[
        att(dim=4, heads=1, kv_heads=1, vdim=4, mask=dict(size=1, keep_first=0)),
        with_mlp(dlt(conv=1, dim=4, heads=1, kv_heads=1, vdim=4), dict(kind="dense", ff=8))],
        logit_scale=1.0, loop=dict(start=0, stop=2, times=1), norm=dict(eps=1e-6), vocab=24, width=16),
    # no loop, no logit scale, an attention without a mask, kept tokens beyond the window, unequal head sizes, an odd width
    "wide": lambda: dict(architecture="Tizodra", layers=[
        dict(type="attention", mixer=dict(dim=24, heads=6, kv_heads=2, vdim=12, scale=0.2), mlp=None),
        with_mlp(dlt(conv=3, dim=40, heads=2, kv_heads=2, vdim=24), dict(kind="dense", ff=72)),
        att(dim=16, heads=2, kv_heads=1, vdim=40, mask=dict(size=9, keep_first=14))],
        norm=dict(eps=1e-5), vocab=80, width=72),
    # a loop that starts at the first layer and ends the stack, many passes
    "loop0": lambda: dict(architecture="Tizodra", layers=[att(mask=dict(size=12, keep_first=1)), dlt(conv=2)],
                          logit_scale=2.0, loop=dict(start=0, stop=2, times=4), norm=dict(eps=1e-5), vocab=50, width=24),
}


@pytest.mark.parametrize("device,dtype", ALL)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_packed_forward_matches_oracle_layer_by_layer(device, dtype, name):
    cfg = CONFIGS[name]()
    w = O.random_checkpoint(cfg, 1)
    m = build(cfg, w, device, dtype)
    seqs = [toks(n, cfg["vocab"], n) for n in (23, 1, 2, 40, 3)]
    ids = torch.tensor([x for s in seqs for x in s], device=device)
    cu = torch.tensor([0] + [len(s) for s in seqs], device=device).cumsum(0).int()
    trace = []
    with torch.no_grad():
        got = m._forward_hetero(ids, cu, None, None, trace=trace).logits
    refs = [O.forward(w, cfg, s, want_layers=True) for s in seqs]
    assert got.dtype == torch.float32 or cfg.get("logit_scale") is None
    assert model_ok(row_errs(got, torch.cat([r[0] for r in refs])), dtype)
    assert len(trace) == len(O.run_order(cfg)) == len(m.config.layer_runs())
    if dtype == torch.float32:
        for r, x in enumerate(trace):
            want = torch.cat([ref[1][r] for ref in refs])
            assert float((x.double().cpu() - want).abs().max() / want.abs().max()) < 1e-5, r


@pytest.mark.parametrize("device,dtype", ALL)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_session_prefill_decode_batches_and_slot_reuse(device, dtype, name):
    """Unequal requests prefilled as one batch (cut after 1, 2, many tokens), decoded together for 60+ steps (past every window and
    ring) while the short ones end and new requests take over their slots; every logit against the whole-sequence oracle of its
    request alone."""
    cfg = CONFIGS[name]()
    w = O.random_checkpoint(cfg, 2)
    m = build(cfg, w, device, dtype)
    V = cfg["vocab"]
    seqs = {r: toks(n, V, 100 + r) for r, n in enumerate((70, 9, 31, 2, 45, 66, 12))}
    ref = {r: O.forward(w, cfg, s) for r, s in seqs.items()}
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
def test_batched_equals_alone_and_prefill_equals_decoding(device, dtype):
    """The logits of a request do not depend on its batch or on where the prompt ended: alone vs. in a batch of unequal requests,
    whole prompt vs. first token + decoding; differences stay at rounding level."""
    cfg = CONFIGS["mixed"]()
    w = O.random_checkpoint(cfg, 5)
    m = build(cfg, w, device, dtype)
    seqs = [toks(n, cfg["vocab"], 30 + n) for n in (37, 5, 1, 20)]
    alone = [packed_logits(m, [s]) for s in seqs]
    batch = packed_logits(m, seqs)
    off = 0
    for s, lg in zip(seqs, alone):
        assert float((batch[off:off + len(s)] - lg).abs().max()) < 1e-5
        off += len(s)
    sess = gen.StepSession(m, max_len=40, n_slots=4)
    h = sess.prefill([(i, s[:1]) for i, s in enumerate(seqs)])
    rows = {i: [sess.logits(h[i:i + 1])[0]] for i in range(4)}
    for t in range(1, 37):
        live = [i for i, s in enumerate(seqs) if t < len(s)]
        lg = sess.logits(sess.decode([(i, seqs[i][t]) for i in live]))
        for j, i in enumerate(live):
            rows[i].append(lg[j])
    for i, lg in enumerate(alone):
        assert float((torch.stack(rows[i]) - lg).abs().max()) < 2e-5


@pytest.mark.parametrize("device,dtype", EXACT)
def test_far_token_reaches_through_the_delta_state_only(device, dtype):
    """With attention windows of a few tokens, an early token still moves the last logits of a stack that has a delta block (its state
    carries it) and does not move them when the stack is attention only and the token lies beyond the reach of the stacked windows."""
    both = dict(architecture="Tizodra", layers=[att(mask=dict(size=4, keep_first=0)), dlt()], norm=dict(eps=1e-5), vocab=64, width=32)
    only = dict(architecture="Tizodra", layers=[att(mask=dict(size=4, keep_first=0)), att(mask=dict(size=6, keep_first=0))],
                norm=dict(eps=1e-5), vocab=64, width=32)
    kept = dict(architecture="Tizodra", layers=[att(mask=dict(size=4, keep_first=3)), att(mask=dict(size=6, keep_first=0))],
                norm=dict(eps=1e-5), vocab=64, width=32)
    # (the distance penalty shrinks what a far kept token contributes, so the attention-only cases stay short)
    for cfg, n, j, moves in ((both, 60, 2, True), (only, 16, 15 - 8, True), (only, 16, 15 - 9, False), (kept, 16, 2, True), (kept, 16, 3, False)):
        w = O.random_checkpoint(cfg, 4)
        if cfg is both:
            w["l1.mix.A_log"] = torch.full_like(w["l1.mix.A_log"], -6.0)          # decays close to one: the state remembers
        m = build(cfg, w, device, dtype)
        base = toks(n, 64, 7)
        other = list(base)
        other[j] = (other[j] + 1) % 64
        diff = float((packed_logits(m, [other])[-1] - packed_logits(m, [base])[-1]).abs().max())
        want = float((O.forward(w, cfg, other)[-1] - O.forward(w, cfg, base)[-1]).abs().max())
        assert (diff > 1e-4) == moves == (want > 1e-4), (j, diff, want)


@pytest.mark.parametrize("device,dtype", EXACT)
def test_greedy_generation_through_generate_and_inflight_batcher(device, dtype):
    cfg = CONFIGS["mixed"]()
    w = O.random_checkpoint(cfg, 6)
    m = build(cfg, w, device, dtype)
    V, n_new = cfg["vocab"], 12
    prompts = [toks(n, V, 50 + n) for n in (5, 1, 14)]
    want = [O.greedy(w, cfg, p, n_new) for p in prompts]
    g = GenerationHyperparameters(max_new_tokens=n_new, min_new_tokens=n_new, greedy=True, use_cuda_graph=(device == "cuda"))
    ids = torch.tensor([x for p in prompts for x in p], device=device)
    cu = torch.tensor([0] + [len(p) for p in prompts], device=device).cumsum(0).int()
    out, _ = gen.generate(m, ids, cu, g, eos_id=None, pad_id=0)
    assert out.tokens.tolist() == want
    ib = gen.InflightBatchingGenerator(m, g, eos_id=None, pad_id=0, n_slots=2, max_prompt_len=16)
    res = ib.generate([torch.tensor(p, device=device) for p in prompts])
    assert [r[0] for r in res] == want


def write_checkpoint(d, cfg, w):
    from safetensors.torch import save_file
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: v.contiguous() for k, v in w.items()}, os.path.join(d, "model.safetensors"))


def test_checkpoint_roundtrip_and_family_detection(tmp_path):
    for name in ("mixed", "wide"):
        cfg = CONFIGS[name]()
        w = O.random_checkpoint(cfg, 8)
        d = str(tmp_path / name)
        write_checkpoint(d, cfg, w)
        assert hf_io.family_of_path(d) == "tizodra"
        m = hf_io.from_hf("tizodra", d, dtype=torch.float32, device="cpu")
        fam = hf_io.family("tizodra")
        assert fam.config_to_dict(m.config) == cfg
        assert sum(p.numel() for p in w.values()) == m.config.n_params()          # (the fused tensors' padding rows not counted)
        back = fam.sd_to_hf(m.state_dict(), m.config)
        assert set(back) == set(w) and all(torch.equal(back[k].to(w[k].dtype), w[k]) for k in w)
        seq = toks(20, cfg["vocab"], 3)
        assert float(row_errs(packed_logits(m.eval(), [seq]), O.forward(w, cfg, seq)).max()) < 2e-4


@pytest.mark.parametrize("device", ["cpu", pytest.param("cuda:0", marks=pytest.mark.gpu)])
def test_trace_replay_command(tmp_path, device):
    """`bin/trace_run` on a checkpoint directory: new requests as one packed prefill, live requests decoded together, requests that
    end give their slots back; the files it writes hold the asked logits in order."""
    cfg = CONFIGS["mixed"]()
    w = O.random_checkpoint(cfg, 9)
    d, out = str(tmp_path / "ckpt"), str(tmp_path / "out")
    write_checkpoint(d, cfg, w)
    V = cfg["vocab"]
    a, b, c = toks(12, V, 1), toks(5, V, 2), toks(4, V, 3)
    steps = [dict(step=0, entries=[dict(id="a", tokens=a[:7], want=[0, 6]), dict(id="b", tokens=b[:3], want=[])], end=[]),
             dict(step=1, entries=[dict(id="a", tokens=a[7:8], want=[0]), dict(id="b", tokens=b[3:4], want=[0])], end=[]),
             dict(step=2, entries=[dict(id="a", tokens=a[8:9], want=[]), dict(id="b", tokens=b[4:5], want=[])], end=["b"]),
             dict(step=3, entries=[dict(id="c", tokens=c, want=[3])], end=["c"]),
             dict(step=4, entries=[dict(id="a", tokens=a[9:10], want=[0])], end=[])]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", d, "--dtype", "float32", "--out", out,
                        "--max-tokens", "64", "--device", device], input="\n".join(json.dumps(s) for s in steps) + "\n",
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(5)]
    ra, rb_, rc = O.forward(w, cfg, a), O.forward(w, cfg, b), O.forward(w, cfg, c)
    want = {0: torch.stack([ra[0], ra[6]]), 1: torch.stack([ra[7], rb_[3]]), 3: rc[3:4], 4: ra[9:10]}
    assert not os.path.exists(os.path.join(out, "2.f32"))
    for s, wnt in want.items():
        import numpy as np
        got = torch.from_numpy(np.fromfile(os.path.join(out, f"{s}.f32"), dtype="<f4").reshape(-1, V))
        assert float(row_errs(got, wnt).max()) < 2e-4


def test_family_through_registry_factory_backend_and_engine():
    """The family as the rest of the framework reaches it: model registry -> `real_model` factory -> inference backend ->
    `ReaLEngine.generate` on a packed `SequenceSample`."""
    import realhf_b200.engine.engine  # noqa: F401  (registers the backends)
    import realhf_b200.models.factory  # noqa: F401  (registers `real_model`)
    from realhf_b200.api import model as model_api
    from realhf_b200.api.config import ModelAbstraction, ModelBackendAbstraction, ModelName
    from realhf_b200.api.data import SequenceSample
    from realhf_b200.api.model import FinetuneSpec
    m = model_api.make_model(ModelAbstraction("real_model", args=dict(model_path="", is_critic=False, init_from_scratch=True, dtype="fp32",
                                                                      hf_model_family="tizodra")), ModelName("actor", 0), "cpu")
    c = m.module.config
    assert [b.mixer for b in c.blocks] == ["window_attention", "delta", "window_attention"] and c.loop.times == 2
    m = model_api.make_backend(ModelBackendAbstraction("inference")).initialize(m, FinetuneSpec(1, 1, 1))
    lens = [5, 9, 3]
    ids = torch.randint(3, 90, (sum(lens),))
    x = SequenceSample.from_default(seqlens=lens, ids=list(range(3)), data=dict(packed_input_ids=ids))
    g = GenerationHyperparameters(max_new_tokens=6, min_new_tokens=6, greedy=True)
    out = m.module.generate(x, m.tokenizer, g)[0]
    assert tuple(out.tokens.shape) == (3, 6)
    seqs = [ids[a:b].tolist() + out.tokens[i].tolist() for i, (a, b) in enumerate(zip([0, 5, 14], [5, 14, 17]))]
    lg = packed_logits(m.module.module, seqs)
    off = 0
    for i, s in enumerate(seqs):
        pred = lg[off + lens[i] - 1: off + len(s) - 1].argmax(-1).tolist()
        assert pred == out.tokens[i].tolist()
        off += len(s)
