"""Trace replay: feeds given token ids through a checkpoint step by step and writes the logits that are asked for.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N      (steps on standard input)

One JSON object per line: {"step": n, "entries": [{"id": ..., "tokens": [...], "want": [...]}], "end": [ids]}.  Every
entry is one call of the runtime's step function (`generation_utils.model_step`: a prompt portion when it brings
several tokens or starts a sequence, a decode step when it brings one more token) on the model `load_model` builds
and the caches `setup_caches` builds; `end` gives a finished sequence's slots back (`reset_caches`).  Nothing is
sampled.  For a step with wanted rows the fp32 logits go to DIR/<step>.f32; after every step `done <step>` is printed.
The kernels this needs are compiled on first use (the sequence-kernel library only).
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", required=True, type=Path, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, type=Path)
    ap.add_argument("--max-tokens", type=int, default=4096, help="most tokens a live sequence holds (sizes the caches)")
    ap.add_argument("--device", default="cuda")
    a = ap.parse_args(argv)

    from .build import build_seq_extension
    build_seq_extension()
    import torch
    from .generation_utils import load_model, model_step, reset_caches, setup_caches

    if not torch.cuda.is_available():
        print("trace_run needs a CUDA device: there is no CPU path", file=sys.stderr)
        return 4
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    torch.set_float32_matmul_precision("highest")
    precision = torch.bfloat16 if a.dtype == "bfloat16" else torch.float32
    device = torch.device(a.device)
    model = load_model(a.model, device, precision, use_tp=False)
    if not getattr(model, "supports_prompt_portions", False):
        print("this checkpoint's model class cannot continue a prompt from its caches", file=sys.stderr)
        return 5
    setup_caches(model, None, device, max_seq_length=max(1, a.max_tokens), cache_kwargs={})
    a.out.mkdir(parents=True, exist_ok=True)

    live, at = None, 0          # the sequence the caches hold and how many of its tokens they have seen
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        rows = []
        for entry in step.get("entries", []):
            tokens = entry.get("tokens") or []
            if not tokens:
                continue
            if live is None:
                live, at = entry["id"], 0
            elif live != entry["id"]:
                raise RuntimeError("one sequence at a time: the previous one has not ended")
            x = torch.tensor(tokens, dtype=torch.int32, device=device).view(1, -1)
            input_pos = torch.arange(at, at + len(tokens), dtype=torch.int32, device=device)
            want = entry.get("want") or []
            logits_at = torch.tensor(want, dtype=torch.long, device=device) if want else None
            logits = model_step(model, x, input_pos, is_prefill=not (len(tokens) == 1 and at > 0), logits_at=logits_at)
            if want:
                rows.append(logits[0].float())
            at += len(tokens)
        for done in step.get("end", []):
            if done == live:
                reset_caches(model)
                live, at = None, 0
        if rows:
            data = torch.cat(rows, 0).contiguous().cpu().numpy().astype("<f4")
            tmp = a.out / f".{step['step']}.f32.part"
            data.tofile(tmp)
            tmp.replace(a.out / f"{step['step']}.f32")
        else:
            torch.cuda.synchronize(device)
        print(f"done {step['step']}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
