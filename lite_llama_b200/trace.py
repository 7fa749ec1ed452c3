"""Trace replay: feed given token ids through a model step by step and write the logits asked for.

Reads one JSON object per line from standard input,
``{"step": n, "entries": [{"id": ..., "tokens": [...], "want": [...]}], "end": [...]}``: all entries of a step are one
batch of ``ModelRunner.forward_ragged`` (prompt portions beside single tokens); a request is admitted at its first
entry and gives its cache rows and state slot back when it is named in ``end``.  For a step that wants logits the
file ``<out>/<step>.f32`` holds them as little-endian fp32 ``[wanted, vocab]`` in entry order; after every step the
line ``done <step>`` is printed.  Nothing is sampled.
"""

from __future__ import annotations

import json
import os
import sys

import torch

from .executor import ModelRunner, RequestState

DTYPES = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32}


def replay(model_dir: str, dtype: str, out_dir: str, max_tokens: int, max_requests: int = 4, stdin=None,
           stdout=None) -> int:
    stdin = stdin or sys.stdin
    stdout = stdout or sys.stdout
    if dtype == "float32":
        # true 32-bit everywhere, also in whatever torch does around the kernels
        torch.backends.cuda.matmul.allow_tf32 = False
        torch.backends.cudnn.allow_tf32 = False
    runner = ModelRunner.from_checkpoint(model_dir, dtype=DTYPES[dtype], max_tokens=max_tokens,
                                         max_requests=max_requests, device="cuda")
    if not runner.ragged_steps:
        print(f"{runner.spec.model_type} does not serve ragged steps", file=sys.stderr)
        return 4
    live: dict[str, RequestState] = {}
    os.makedirs(out_dir, exist_ok=True)
    for line in stdin:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        entries, want, at = [], [], 0
        for e in step.get("entries", []):
            req = live.get(e["id"])
            if req is None:
                req = live[e["id"]] = runner.open_request()
            if not e["tokens"]:                      # admitted, nothing to run yet
                continue
            entries.append((req, list(e["tokens"])))
            want.extend(at + int(i) for i in e.get("want", []))
            at += len(e["tokens"])
        if entries:
            logits = runner.forward_ragged(entries, want)
            if want:
                data = logits.float().cpu().contiguous().numpy().astype("<f4", copy=False)
                tmp = os.path.join(out_dir, f".{step['step']}.part")
                with open(tmp, "wb") as f:
                    f.write(data.tobytes())
                os.replace(tmp, os.path.join(out_dir, f"{step['step']}.f32"))
            else:
                torch.cuda.synchronize()
        for rid in step.get("end", []):
            req = live.pop(rid, None)
            if req is not None:
                runner.close_request(req)
        stdout.write(f"done {step['step']}\n")
        stdout.flush()
    return 0
