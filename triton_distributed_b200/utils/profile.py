"""Merged multi-rank profiling (reference python/triton_dist/utils.py:174-183,282-501).

``group_profile(name, do_prof, group)`` wraps ``torch.profiler``; on exit every rank exports a chrome
trace, rank 0 gathers them all, shifts each rank's pids/tids into its own range so the timelines
sit side by side, and writes one gzip-compressed merged trace ``prof/<name>/merged.json.gz``.
"""
from __future__ import annotations

import contextlib
import gzip
import json
import os
from typing import Optional

import torch
import torch.distributed as dist


def nvtx_range(name: str):
    """Decorator: run the function inside an NVTX range when TDIST_NVTX=1 (and CUDA is up), so that the ops show as
    named spans in external timelines; otherwise the function is returned untouched (no per-call cost)."""
    def decor(fn):
        if os.environ.get("TDIST_NVTX", "0") != "1":
            return fn

        import functools

        @functools.wraps(fn)
        def wrapped(*a, **kw):
            if not torch.cuda.is_available():
                return fn(*a, **kw)
            torch.cuda.nvtx.range_push(name)
            try:
                return fn(*a, **kw)
            finally:
                torch.cuda.nvtx.range_pop()
        return wrapped
    return decor


def get_torch_prof_ctx(do_prof: bool):
    if not do_prof:
        return contextlib.nullcontext()
    acts = [torch.profiler.ProfilerActivity.CPU]
    if torch.cuda.is_available():
        acts.append(torch.profiler.ProfilerActivity.CUDA)
    return torch.profiler.profile(activities=acts, record_shapes=True, with_stack=False)


def _shift_ids(trace: dict, rank: int) -> list:
    """Move every pid of one rank's trace into its own range and label the processes."""
    events = trace.get("traceEvents", [])
    offset = rank * 100_000_000
    for ev in events:
        if isinstance(ev.get("pid"), int):
            ev["pid"] += offset
        elif "pid" in ev:
            ev["pid"] = f"rank{rank}:{ev['pid']}"
        if ev.get("ph") == "M" and ev.get("name") == "process_name":
            ev.setdefault("args", {})["name"] = f"rank {rank} | {ev.get('args', {}).get('name', '')}"
    return events


def merge_traces(traces: list) -> dict:
    merged = {"traceEvents": []}
    for rank, tr in enumerate(traces):
        if tr is None:
            continue
        for k, v in tr.items():
            if k != "traceEvents":
                merged.setdefault(k, v)
        merged["traceEvents"].extend(_shift_ids(tr, rank))
    return merged


class group_profile:
    def __init__(self, name: Optional[str] = None, do_prof: bool = True, group=None, out_dir: str = "prof"):
        self.name = name or "trace"
        self.do_prof = do_prof
        self.group = group
        self.out_dir = os.path.join(out_dir, self.name)
        self.prof = None
        self.merged_path = None

    def __enter__(self):
        if self.do_prof:
            self.prof = get_torch_prof_ctx(True)
            self.prof.__enter__()
        return self

    def __exit__(self, *exc):
        if not self.do_prof:
            return False
        self.prof.__exit__(*exc)
        rank = dist.get_rank(self.group) if dist.is_initialized() else 0
        world = dist.get_world_size(self.group) if dist.is_initialized() else 1
        os.makedirs(self.out_dir, exist_ok=True)
        path = os.path.join(self.out_dir, f"rank{rank}.json")
        self.prof.export_chrome_trace(path)
        with open(path) as f:
            mine = json.load(f)
        if world > 1:
            gathered = [None] * world if rank == 0 else None
            dist.gather_object(mine, gathered, dst=0, group=self.group)
        else:
            gathered = [mine]
        if rank == 0:
            self.merged_path = os.path.join(self.out_dir, "merged.json.gz")
            with gzip.open(self.merged_path, "wt") as f:
                json.dump(merge_traces(gathered), f)
        if world > 1:
            dist.barrier(self.group)
        return False


def load_json(json_file: str) -> dict:
    """Read a Chrome-trace JSON written by the torch profiler. Kernel names can carry raw control characters or
    unescaped quotes that strict parsers refuse: those are replaced inside every ``"name": "..."`` value before
    parsing (reference utils.py:254-279)."""
    import json
    import re
    with open(json_file, "r", encoding="utf-8", errors="replace") as f:
        text = f.read()
    try:
        return json.loads(text, strict=False)
    except json.JSONDecodeError:
        pass

    def clean(match):
        body = "".join(c if (32 <= ord(c) < 127 and c not in '"\\{}') else "_" for c in match.group(1))
        return f'"name": "{body}"'

    return json.loads(re.sub(r'"name": "(.*?)"(?=\s*[,}])', clean, text, flags=re.DOTALL), strict=False)


def process_trace_json(json_file: str, rank: Optional[int] = None) -> list:
    """Events of one rank's trace file with its process ids moved into the rank's own range, ready to be concatenated
    with the other ranks' (reference utils.py:282-309). The rank comes from the argument, else from the trace's
    ``distributedInfo``, else from a ``rank<N>`` part of the file name, else 0."""
    import re
    trace = load_json(json_file)
    if rank is None:
        rank = trace.get("distributedInfo", {}).get("rank")
    if rank is None:
        m = re.search(r"rank[_-]?(\d+)", str(json_file))
        rank = int(m.group(1)) if m else 0
    return _shift_ids(trace, int(rank))
