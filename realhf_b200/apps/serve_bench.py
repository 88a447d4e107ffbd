"""Prefill / decode throughput of a heterogeneous-stack design next to the closest homogeneous model of equal size, and the
roofline position of its kernels next to the like kernels of that model.  Reached through `bench.py --serve-bench rapodra`
(the default workload of bench.py is unaffected).

Both models run through `models.generation`: prefill = `prefill_into_state` (the packed prefill `generate` performs) into a
standing decode state, decode = the CUDA-graph loop of `generate` with the sampler in the graph; random weights, bf16.  Timing: CUDA events, >= 3 warm-up calls, weights + state far larger than L2 per call for
the model-level numbers; the kernel table flushes L2 (a 256 MB write) between timed launches.  One JSON line per result.
"""

from __future__ import annotations

import json
import os
from typing import Callable, Dict, List

import torch


SIZES = {
    # name: width, heads, qk dim, v dim, latent rank, window, dense ff, experts, expert ff, top, vocab
    "1b-like": dict(width=2048, heads=16, dim=128, vdim=128, rank=512, window=1024, ff=8192, experts=8, eff=2048, top=2, vocab=32000),
    "7b-like": dict(width=4096, heads=32, dim=128, vdim=128, rank=512, window=2048, ff=11008, experts=8, eff=2816, top=2, vocab=32000),
}


def rapodra_config(s: dict, n_layers: int = 4) -> dict:
    mixer = lambda **k: dict(dict(dim=s["dim"], heads=s["heads"], kv_rank=s["rank"], vdim=s["vdim"], scale=s["dim"] ** -0.5,
                                  mask=dict(size=s["window"])), **k)
    dense = dict(kind="dense", ff=s["ff"], limit=7.0)
    moe = dict(kind="moe", expert=dict(ff=s["eff"]), router=dict(experts=s["experts"], top=s["top"]))
    layers = []
    for i in range(n_layers):
        layers.append(dict(type="latent_attention", mixer=mixer(**({"kv_from": i - 1} if i % 2 else {})), mlp=moe if i % 2 else dense))
    return dict(architecture="Rapodra", canon=dict(taps=4), layers=layers, logit_softcap=30.0, norm=dict(eps=1e-5, groups=8),
                vocab=s["vocab"], width=s["width"])


def _models(s: dict, n_layers: int, dev):
    from realhf_b200.api.model import ReaLModelConfig
    from realhf_b200.models import hf_io
    from realhf_b200.models.real_model import ReaLModel
    rc = hf_io.family("rapodra").config_from_dict(rapodra_config(s, n_layers), False)
    new = ReaLModel(rc, dtype=torch.bfloat16, device=dev).init_random_fast()
    lc = ReaLModelConfig(n_layers=n_layers, n_kv_heads=s["heads"], n_q_heads=s["heads"], hidden_dim=s["width"], intermediate_dim=s["ff"],
                         vocab_size=s["vocab"], head_dim=s["dim"], n_positions=8192, embd_pdrop=0.0, resid_pdrop=0.0, attn_pdrop=0.0,
                         activation_function="silu", scale_attn_by_inverse_layer_idx=False, use_attention_bias=False,
                         use_attn_proj_bias=False, use_mlp_bias=False, layer_norm_type="rms", mlp_type="llama", apply_rotary=True)
    old = ReaLModel(lc, dtype=torch.bfloat16, device=dev).init_random_fast()
    for m in (new, old):
        for p in m.parameters():
            p.requires_grad_(False)
        m.eval()
    return new, old


def _time(fn: Callable[[], None], iters: int, warmup: int = 3, flush: torch.Tensor = None) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    tot = 0.0
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        tot += a.elapsed_time(b)
    return tot / iters


def model_numbers(name: str, s: dict, n_layers: int, batch: int, prompt_len: int, new_tokens: int, dev) -> List[dict]:
    from realhf_b200.api.model import GenerationHyperparameters
    from realhf_b200.models import generation as gen
    os.environ["REAL_GEN_TIMING"] = "1"
    out = []
    new, old = _models(s, n_layers, dev)
    g = GenerationHyperparameters(max_new_tokens=new_tokens, min_new_tokens=new_tokens, greedy=True, use_cuda_graph=True)
    ids = torch.randint(3, s["vocab"], (batch * prompt_len,), device=dev)
    cu = torch.arange(0, batch + 1, device=dev, dtype=torch.int32) * prompt_len
    for label, m in (("rapodra", new), ("llama-equal-size", old)):
        # prefill: the packed prefill into a standing decode state (`prefill_into_state`, what `generate` calls), so that the
        # number is the model's and not the caching allocator's (a fresh multi-GB state per `generate` call can fall into
        # cudaMalloc inside the timed region); decode: the CUDA-graph loop of `generate`
        st = gen.DecodeState(m, batch, prompt_len + new_tokens)
        pre, dec = [], []
        with torch.no_grad():
            for it in range(7):
                st.free_slots = list(range(batch))
                slots = st.alloc(batch)
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                gen.prefill_into_state(m, st, slots, ids, cu, prompt_len)
                b.record()
                torch.cuda.synchronize()
                if it >= 2:
                    pre.append(a.elapsed_time(b))
        del st
        for it in range(4):
            gen.generate(m, ids, cu, g, eos_id=None, pad_id=0)
            if it:                                     # first call: lazy initialisation
                dec.append(gen.LAST_TIMING["ms_per_decode_step"])
        pre_ms, dec_ms = sorted(pre)[len(pre) // 2], sorted(dec)[len(dec) // 2]
        out.append(dict(bench="serve", size=name, model=label, layers=n_layers, batch=batch, prompt_len=prompt_len, new_tokens=new_tokens,
                        prefill_ms=round(pre_ms, 3), prefill_tokens_per_s=round(batch * prompt_len / pre_ms * 1e3),
                        decode_ms_per_step=round(dec_ms, 4), decode_tokens_per_s=round(batch / dec_ms * 1e3), dtype="bf16", data="synthetic",
                        params=sum(p.numel() for p in m.parameters())))
    del new, old
    torch.cuda.empty_cache()
    return out


def kernel_numbers(name: str, s: dict, batch: int, prompt_len: int, ctx: int, dev, peaks: Dict[str, float]) -> List[dict]:
    """Each kernel of the new design and the like kernel of the LLaMA path on the same problem size: time, algorithmic bytes and
    FLOPs, and the fraction of the measured roofline (the slower of bytes / copy bandwidth and FLOPs / GEMM throughput)."""
    from realhf_b200.models.hetero_block import packed_meta
    from realhf_b200.ops import attention as A
    from realhf_b200.ops import functional as OF
    bf = torch.bfloat16
    W, H, qk, vd, rank, win = s["width"], s["heads"], s["dim"], s["vdim"], s["rank"], s["window"]
    T = batch * prompt_len
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    rows = []

    def add(kernel, like, ms, nbytes, flops):
        floor_ms = max(nbytes / (peaks["hbm_gbs"] * 1e9), flops / (peaks["bf16_tflops"] * 1e12)) * 1e3
        rows.append(dict(bench="kernel", size=name, kernel=kernel, like=like, ms=round(ms, 4), gbytes=round(nbytes / 1e9, 4),
                         gflop=round(flops / 1e9, 2), roofline_ms=round(floor_ms, 4), frac_of_measured_roofline=round(floor_ms / ms, 4)))

    cu = torch.arange(0, batch + 1, device=dev, dtype=torch.int32) * prompt_len
    meta = packed_meta(cu, T)
    x32 = torch.randn(T, W, device=dev)
    xb = x32.to(bf)
    w = torch.ones(W, device=dev, dtype=bf)
    cw = torch.randn(W, 4, device=dev).to(bf) * 0.1
    add("sublayer_input (grouped norm + conv, prefill)", False, _time(lambda: OF.sublayer_input(x32, w, 8, 1e-5, cw, meta.pos, bf), 10, flush=flush),
        T * W * 6, 0)
    add("residual_add_norm_ (prefill)", False, _time(lambda: OF.residual_add_norm_(x32, xb, w, 8, 1e-5), 10, flush=flush), T * W * 10, 0)
    add("add_rmsnorm (llama, prefill)", True, _time(lambda: OF.add_rmsnorm(xb, xb, w, 1e-5), 10, flush=flush), T * W * 8, 0)
    # attention, prefill: windowed, so the useful FLOPs are those of the visible (query, key) pairs
    q = torch.randn(T, H * qk + rank, device=dev).to(bf)
    kv = torch.randn(T, H * (qk + vd), device=dev).to(bf)
    pairs = batch * sum(min(p + 1, win) for p in range(prompt_len))
    add("latent_window_attention (prefill, tcgen05 kernel with window)", False,
        _time(lambda: A.latent_window_attention(q, kv, meta.pos, H, qk, vd, qk ** -0.5, win, cu, prompt_len), 5, flush=flush),
        T * H * (2 * qk + 2 * vd) * 2, 2.0 * pairs * H * (qk + vd))
    add("latent_window_attention (prefill, CUDA-core kernel: fp32 and other head shapes)", False,
        _time(lambda: A.latent_window_attention(q, kv, meta.pos, H, qk, vd, qk ** -0.5, win), 2, warmup=1, flush=flush),
        T * H * (2 * qk + 2 * vd) * 2, 2.0 * pairs * H * (qk + vd))
    qkv = torch.randn(T, 3 * H * qk, device=dev).to(bf)
    full_pairs = batch * prompt_len * (prompt_len + 1) // 2
    add("varlen attention tcgen05 (llama, prefill, full causal)", True,
        _time(lambda: A.varlen_attention_qkv(qkv, cu, prompt_len, H, H, qk, None, True), 5, flush=flush), T * H * qk * 4 * 2, 4.0 * full_pairs * H * qk)
    # attention, decode at context `ctx`
    keys = min(ctx + 1, win)
    R = min(win, ctx + 64)
    cache = torch.randn(batch, R, rank, device=dev).to(bf)
    lens = torch.full((batch,), ctx, dtype=torch.int32, device=dev)
    qc = torch.randn(batch, H * qk + rank, device=dev).to(bf)
    w_ukv = (torch.randn(H * (qk + vd), rank, device=dev) * rank ** -0.5).to(bf)
    w_ln = torch.ones(rank, device=dev, dtype=bf)
    add(f"latent_decode_attention (ctx {ctx}, {keys} keys)", False,
        _time(lambda: A.latent_decode_attention(qc, w_ln, w_ukv, cache, lens, None, H, qk, vd, qk ** -0.5, win, 1e-5), 10, flush=flush),
        batch * keys * rank * 2 + H * (qk + vd) * rank * 2, 2.0 * batch * H * (keys * 2 * rank + (qk + vd) * rank))
    kc = torch.zeros(batch, H, ctx + 64, qk, device=dev, dtype=bf).permute(0, 2, 1, 3)
    vc = torch.zeros(batch, H, ctx + 64, qk, device=dev, dtype=bf).permute(0, 2, 1, 3)
    qkv1 = torch.randn(batch, 3 * H * qk, device=dev).to(bf)
    cos, sin = OF.rope_tables(ctx + 64, qk, 10000.0, dev)
    add(f"decode_attention (llama, ctx {ctx}, all {ctx + 1} keys)", True,
        _time(lambda: A.decode_attention(qkv1, kc, vc, lens, H, H, qk, None, cos, sin), 10, flush=flush),
        batch * (ctx + 1) * H * qk * 2 * 2, 4.0 * batch * H * (ctx + 1) * qk)
    xs = torch.randn(batch, W, device=dev)
    st = torch.zeros(batch, 3, W, device=dev)
    add("sublayer_input_step (decode)", False, _time(lambda: OF.sublayer_input_step(xs, w, 8, 1e-5, cw, st, None, bf), 10, flush=flush),
        batch * W * (6 + 24), 0)
    gu = torch.randn(T, 2 * s["ff"], device=dev).to(bf)
    add("clamped_glu (prefill)", False, _time(lambda: OF.clamped_glu(gu, 7.0, 1.702), 10, flush=flush), T * s["ff"] * 6, 0)
    add("gated_act silu (llama, prefill)", True, _time(lambda: OF.gated_act(gu, "silu"), 10, flush=flush), T * s["ff"] * 6, 0)
    return rows


def run(design: str, sizes: List[str] = None, n_layers: int = 4) -> List[dict]:
    assert design == "rapodra"
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    peaks = dict(hbm_gbs=6650.0, bf16_tflops=1590.0, source="fallback")
    pk = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    if os.path.exists(pk):
        with open(pk) as f:
            d = json.load(f)
        if "hbm_gbs" in d and "bf16_tflops" in d:
            peaks = dict(hbm_gbs=float(d["hbm_gbs"]), bf16_tflops=float(d["bf16_tflops"]), source="measured")
    results = [dict(bench="peaks", **peaks)]
    for name in sizes or list(SIZES):
        s = SIZES[name]
        results += model_numbers(name, s, n_layers, batch=32, prompt_len=1024, new_tokens=33, dev=dev)
        results += kernel_numbers(name, s, batch=32, prompt_len=1024, ctx=2048, dev=dev, peaks=peaks)
    for r in results:
        print(json.dumps(r), flush=True)
    return results
