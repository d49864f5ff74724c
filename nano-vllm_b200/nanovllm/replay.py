"""Replay of a recorded schedule: feeds given token ids through a model step by step and writes the logits that are asked
for.  Nothing is sampled.  The steps run through the engine's own scheduler bookkeeping (``Scheduler.plan_step``), block
and state-slot manager and ``ModelRunner`` -- the objects ``LLM.generate`` drives -- in logits-only mode.

    python -m nanovllm.replay --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N   < steps.jsonl

stdin, one JSON object per line:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": ["a"]}
``entries``: for each request its next tokens and the places among them whose logits are wanted; all entries of a step are
one batch.  ``end``: requests that are finished after the step (their blocks and state slot are returned).
For a step with wanted places the logits go to ``<out>/<step>.f32`` (little-endian fp32, [wanted, vocab], in the order of the
entries); after every step ``done <step>`` is printed.

``--max-tokens`` sizes the cache pool: that many tokens in pages of ``--block-size`` (64), four live requests at most.
Exit code 3: float32 asked of a model that has no 32-bit path.
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True)
    ap.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16")
    ap.add_argument("--out", required=True)
    ap.add_argument("--max-tokens", type=int, required=True)
    ap.add_argument("--block-size", type=int, default=64)
    ap.add_argument("--max-seqs", type=int, default=4)
    ap.add_argument("--eager", action="store_true", help="no CUDA graphs for decode steps")
    a = ap.parse_args(argv)

    from .config import Config
    from .models.registry import model_class, read_config
    hf = read_config(a.model)
    if a.dtype == "float32" and not hasattr(model_class(hf), "bind_cache"):
        print("this model has no float32 path", file=sys.stderr)
        return 3

    import numpy as np
    from .engine.model_runner import ModelRunner
    from .engine.scheduler import Scheduler
    from .engine.sequence import Sequence

    bs = a.block_size
    pool = max(-(-a.max_tokens // bs), 1)
    config = Config(a.model, hf_config=hf, max_num_seqs=a.max_seqs, max_num_batched_tokens=pool * bs, max_model_len=pool * bs,
                    kvcache_block_size=bs, num_kvcache_blocks=pool, enforce_eager=a.eager, dtype=a.dtype, logits_only=True)
    Sequence.block_size = bs
    runner = ModelRunner(config, 0, None)
    sched = Scheduler(config)
    os.makedirs(a.out, exist_ok=True)
    live: dict[str, Sequence] = {}
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        portions, rows, at = [], [], 0
        for e in step["entries"]:
            toks = [int(t) for t in e["tokens"]]
            seq = live.get(e["id"])
            if seq is None:
                seq = live[e["id"]] = Sequence(toks)
            portions.append((seq, toks))
            rows += [at + int(w) for w in e.get("want", [])]
            at += len(toks)
        if portions:
            batch, is_prefill = sched.plan_step(portions)
            logits = runner.run_logits(batch, is_prefill, rows)
            sched.postprocess_replay(batch)
            if rows:
                tmp = os.path.join(a.out, f".{step['step']}.part")
                np.ascontiguousarray(logits.numpy(), dtype="<f4").tofile(tmp)
                os.replace(tmp, os.path.join(a.out, f"{step['step']}.f32"))
        for rid in step.get("end", []):
            seq = live.pop(rid, None)
            if seq is not None:
                sched.retire(seq)
        print(f"done {step['step']}", flush=True)
    runner.exit()
    return 0


if __name__ == "__main__":
    sys.exit(main())
