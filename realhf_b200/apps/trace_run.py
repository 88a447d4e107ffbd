"""Trace replay: feed given token ids through a model step by step and write the logits that are asked for.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N   < steps.jsonl

Nothing is sampled.  The model class is chosen by the checkpoint's `config.json` (`hf_io.family_of_path`), the weights are
loaded by the family's converter, and every step runs through `models.generation.StepSession`: packed prefill into free
state slots, one-token decode steps over any sub-batch of live requests, slots released when a request ends.

Input, one JSON object per line: {"step": n, "entries": [{"id": .., "tokens": [..], "want": [..]}, ..], "end": [ids]}.
`tokens` are the request's NEXT tokens; `want` indexes into them.  A request seen for the first time is prefilled with all
its tokens at once (all new requests of a step form one packed batch); a live request goes on token by token (all live
requests of a step form one decode batch per token).  For a step with wanted positions the logits are written to
OUT/<step>.f32 (little-endian fp32 [wanted, vocab], in the order of the entries and of `want`); `done <step>` is printed
after every step.  bfloat16 serves as the framework serves the model (bf16 GEMMs with fp32 accumulation, fp32 where the
design asks for it); float32 runs everything in true fp32 (no TF32).
"""

from __future__ import annotations

import argparse
import json
import os
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", required=True, help="checkpoint directory (config.json + weights)")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="directory for <step>.f32")
    ap.add_argument("--max-tokens", type=int, default=4096, help="most tokens live requests hold at any time")
    ap.add_argument("--device", default="cuda:0")
    a = ap.parse_args(argv)

    import numpy as np
    import torch

    from realhf_b200.models import generation as gen
    from realhf_b200.models import hf_io

    dev = torch.device(a.device)
    if dev.type == "cuda" and not torch.cuda.is_available():
        print("trace_run: no CUDA device", file=sys.stderr)
        return 2
    dtype = torch.bfloat16 if a.dtype == "bfloat16" else torch.float32
    if dtype == torch.float32:
        torch.backends.cuda.matmul.allow_tf32 = False
        torch.backends.cudnn.allow_tf32 = False
        torch.set_float32_matmul_precision("highest")
    family = hf_io.family_of_path(a.model)
    model = hf_io.from_hf(family, a.model, dtype=dtype, device=dev)
    if model.config.blocks is None:
        print(f"trace_run: family `{family}` has no step session (homogeneous stacks replay through `generate`)", file=sys.stderr)
        return 2
    os.makedirs(a.out, exist_ok=True)
    sess = gen.StepSession(model, max_len=max(1, a.max_tokens))

    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        entries = step.get("entries", [])
        new = [e for e in entries if e["id"] not in sess.slot_of and e["tokens"]]
        old = [e for e in entries if e["id"] in sess.slot_of and e["tokens"]]
        rows = {}                       # (entry id, index in its tokens) -> fp32 logits row
        if new:
            hidden = sess.prefill([(e["id"], e["tokens"]) for e in new])
            off, pick, keys = 0, [], []
            for e in new:
                for w in e.get("want", []):
                    pick.append(off + w)
                    keys.append((e["id"], w))
                off += len(e["tokens"])
            if pick:
                lg = sess.logits(hidden.index_select(0, torch.tensor(pick, device=dev)))
                for k, r in zip(keys, lg):
                    rows[k] = r
        k = 0
        while True:                     # live requests: one decode batch per token index
            batch = [e for e in old if k < len(e["tokens"])]
            if not batch:
                break
            h = sess.decode([(e["id"], e["tokens"][k]) for e in batch])
            sel = [j for j, e in enumerate(batch) if k in e.get("want", [])]
            if sel:
                lg = sess.logits(h.index_select(0, torch.tensor(sel, device=dev)))
                for j, r in zip(sel, lg):
                    rows[(batch[j]["id"], k)] = r
            k += 1
        order = [(e["id"], w) for e in entries for w in e.get("want", [])]
        if order:
            out = torch.stack([rows[key] for key in order]).float().cpu().numpy().astype("<f4")
            tmp = os.path.join(a.out, f".{step['step']}.f32.part")
            out.tofile(tmp)
            os.replace(tmp, os.path.join(a.out, f"{step['step']}.f32"))
        ended = [r for r in step.get("end", []) if r in sess.slot_of]
        if ended:
            sess.release(ended)
        sys.stdout.write(f"done {step['step']}\n")
        sys.stdout.flush()
    return 0


if __name__ == "__main__":
    sys.exit(main())
