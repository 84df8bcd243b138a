"""Trace replay: feed given token ids through a model step by step and write the logits that are asked for.

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N      (steps on standard input)

Every input line is one engine step, ``{"step": n, "entries": [{"id", "tokens", "want"}, ...], "end": [ids]}``: all
entries run as ONE ragged batch through the model's own step (``forward_ragged``), portions of prompts beside single
tokens, on top of whatever earlier steps left in the paged cache.  A request is admitted into a free slot of the
scheduler's slot tables at its first entry and gives its pages back when it is listed under ``end``.  The page pool
is sized once, for ``--max-tokens`` tokens (rounded up to whole pages), and a model with recurrent layers gets as many
state slots as there are request slots, so pages and state slots are reused as requests come and go.
For a step with wanted places the fp32 logits ``[wanted, vocab]`` go to ``<out>/<step>.f32`` (little-endian); after
every step the line ``done <step>`` is printed.  Nothing is sampled.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

SLOTS = 4  # requests that can be live at once


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run")
    ap.add_argument("--model", required=True, help="directory with config.json and model.safetensors")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    ap.add_argument("--out", required=True)
    ap.add_argument("--max-tokens", type=int, required=True, help="tokens the live requests hold at most (each rounded up to whole pages)")
    ap.add_argument("--page-size", type=int, default=64)
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)

    import torch

    from .kv_cache import BatchingKvCache
    from .models import load_model
    from .ragged import RaggedEntry

    dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}[args.dtype]
    model = load_model(args.model, device=args.device, dtype=dtype, page_size=args.page_size, max_tokens=args.max_tokens, max_requests=SLOTS)
    if not hasattr(model, "forward_ragged"):
        print(f"{type(model).__name__} has no ragged step", file=sys.stderr)
        return 4
    tables = [BatchingKvCache(max_active_requests=SLOTS) for _ in range(model.num_hidden_layers)]
    slot_of: dict[str, int] = {}
    os.makedirs(args.out, exist_ok=True)

    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        entries = []
        for item in step["entries"]:
            rid = item["id"]
            if rid not in slot_of:
                free = [s for s in range(SLOTS) if tables[0].kv_caches[s] is None]
                if not free:
                    raise RuntimeError(f"no free slot for request {rid!r}: {SLOTS} are live")
                for table, layer_cache in zip(tables, model.create_kv_cache()):
                    table.add_request(layer_cache, free[0])
                slot_of[rid] = free[0]
            slot = slot_of[rid]
            entries.append(RaggedEntry(item["tokens"], [table.kv_caches[slot] for table in tables], want=item.get("want") or []))
        if entries:
            logits = model.forward_ragged(entries)
            if logits.shape[0]:
                data = logits.to(torch.float32).contiguous().cpu().numpy().astype("<f4", copy=False)
                part = os.path.join(args.out, f".{step['step']}.part")
                with open(part, "wb") as f:
                    f.write(data.tobytes())
                os.replace(part, os.path.join(args.out, f"{step['step']}.f32"))
            else:
                torch.cuda.synchronize()
        for rid in step.get("end", []):
            slot = slot_of.pop(rid, None)
            if slot is not None:
                for table in tables:
                    table.remove_request(slot)
        print(f"done {step['step']}", flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
