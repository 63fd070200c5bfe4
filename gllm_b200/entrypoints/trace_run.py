"""Trace replay: feed given token ids through the engine step by step and write the logits of chosen positions.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Reads one JSON object per line from standard input,
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": ["a"]}
runs all entries of a step as ONE micro-batch (prompt portions beside single decode tokens) through the engine's
worker — its scheduler bookkeeping, page and state-slot managers, batch builder, model runner and kernels — writes
`<out>/<step>.f32` ([wanted rows, vocab] little-endian fp32, in entry / want order) when something is wanted, and
prints `done <step>`. Nothing is sampled. Requests named in "end" give their pages and slots back after the step.
The cache pool holds --max-tokens tokens (+ the padding page) and four recurrent-state slots, so both are re-used.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np


class TraceSession:
    """The engine behind the replay: one in-process worker whose scheduler, managers and runner execute explicit
    steps. `step(entries, end)` returns the fp32 logits [wanted rows, vocab] of one micro-batch (None when nothing
    is wanted)."""

    def __init__(self, model, dtype: str = "bfloat16", max_tokens: int = 1024, device=None, page_size: int = 16,
                 state_slots: int = 4, max_step_tokens=None):
        import torch
        from gllm_b200.config import EngineConfig
        from gllm_b200.engine.worker import Worker
        from gllm_b200.model_loader import ModelLoader

        torch.backends.cuda.matmul.allow_tf32 = False
        torch.backends.cudnn.allow_tf32 = False
        self.page_size = page_size
        pages = (max_tokens + page_size - 1) // page_size + 1            # + the padding page
        cfg = EngineConfig(model_path=model, dtype=dtype, page_size=page_size,
                           maxp=max(max_step_tokens or max_tokens, 64), maxd=64, num_gpu_pages=pages,
                           num_cpu_pages=pages, model_max_length=max(max_tokens, 64), enable_prefix_caching=False,
                           disable_cuda_graph=True, async_schedule=False, kvthresh=0.0, log_stats=False,
                           launch_mode="inproc", device=device, num_state_slots=state_slots)
        loader = ModelLoader(cfg.model_path, cfg.load_format, dtype=cfg.dtype)
        self.worker = Worker(cfg, 0, 0, comm=None, loader=loader).init()
        self.scheduler, self.runner = self.worker.scheduler, self.worker.runner
        self.vocab = self.runner.spec.vocab_size
        self.live = {}
        self._next_id = 0
        self._steps = 0

    def step(self, entries, end=()):
        """entries: [{"id", "tokens", "want"}] -> logits of the wanted rows, in entry / want order."""
        import torch
        from gllm_b200.input_data import build_batch
        from gllm_b200.sequence import Sequence

        plan, wants = [], {}
        for e in entries:
            toks = [int(t) for t in e["tokens"]]
            if not toks:
                continue
            seq = self.live.get(e["id"])
            if seq is None:
                seq = Sequence(self._next_id, toks, [], output_len=1 << 30, ignore_eos=True, top_k=1)
                self._next_id += 1
                self.live[e["id"]] = seq
            else:
                seq.token_ids.extend(toks)
            plan.append((seq, len(toks)))
            wants[seq.seq_id] = [int(w) for w in e.get("want", [])]
        out = None
        sch = self.scheduler
        if plan:
            self._steps += 1
            ents = sch.schedule_explicit(plan)
            batch = build_batch(ents, self.page_size, self.vocab, batch_id=self._steps)
            first_row = {ent.seq.seq_id: int(batch.query_start_loc[i]) for i, ent in enumerate(ents)}
            rows = [first_row[seq.seq_id] + w for seq, _ in plan for w in wants[seq.seq_id]]
            batch.logits_idx = np.asarray(rows, dtype=np.int32)
            logits = self.runner.step_logits(batch)
            if rows:
                out = logits.detach().to("cpu", torch.float32).contiguous().numpy()
            elif self.runner.device.type == "cuda":
                torch.cuda.synchronize()
            sch.complete_explicit([self.live.pop(i) for i in end if i in self.live])
        else:
            for i in end:
                if i in self.live:
                    sch.mm.free(self.live.pop(i))
        return out


def _require_kernels(model_dir: str):
    """Layer-list decoders use the GEMM, attention, expert and sequence kernels only: in a checkout without a built
    library the first call then compiles just those families."""
    try:
        with open(os.path.join(model_dir, "config.json")) as f:
            cfg = json.load(f)
    except OSError:
        return
    if cfg.get("architecture") in ("Saritar", "Femolix", "Bevovik", "Notadra"):
        from gllm_b200.ops import lib
        lib.require({"seq", "gemm", "attn", "moe"})


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run")
    ap.add_argument("--model", required=True)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True)
    ap.add_argument("--max-tokens", type=int, required=True)
    ap.add_argument("--device", default=None)
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--state-slots", type=int, default=4)
    a = ap.parse_args(argv)
    _require_kernels(a.model)
    sess = TraceSession(a.model, a.dtype, a.max_tokens, a.device, a.page_size, a.state_slots)
    os.makedirs(a.out, exist_ok=True)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        msg = json.loads(line)
        out = sess.step(msg.get("entries", []), msg.get("end", []))
        if out is not None:
            tmp = os.path.join(a.out, "%s.f32.tmp" % msg["step"])
            out.astype("<f4").tofile(tmp)
            os.replace(tmp, os.path.join(a.out, "%s.f32" % msg["step"]))
        sys.stdout.write("done %s\n" % msg["step"])
        sys.stdout.flush()
    return 0


if __name__ == "__main__":
    sys.exit(main())
