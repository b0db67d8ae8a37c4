"""Contextual autotuning of multi-kernel (and multi-rank) ops.

A *tunable* is a Python-level op with a small discrete configuration space (number of pusher
CTAs of the AG-GEMM kernel, CTAs per peer of a collective, KV splits of the decode kernel, ...).
Tuning a collective op in isolation is impossible — every rank has to run the same op at the same
time — so, like the reference's ``contextual_autotune`` (reference python/triton_dist/autotuner.py:43-102,
160-256; docs/autotuner.md), the unit that is re-run is a whole *thunk* of user code: each run of the
thunk lets every not-yet-tuned tunable inside it take ONE more measurement (one config, one
repetition), all ranks in lockstep; when a tunable has measured all its configs the per-config
times are reduced with MAX over the ranks, so that every rank picks the same winner, and the
choice is cached per key.

    @tunable(configs=[{"num_comm_sms": n} for n in (4, 8, 16)], key=lambda a, b, ctx: (a.shape, b.shape))
    def ag_gemm(a, b, ctx, *, config): ...

    @contextual_autotune(is_dist=True)
    def step(): return ag_gemm(a, b, ctx)

Per-rank logs go to ``.autotune_logs/rank-<r>.log``.
"""
from __future__ import annotations

import functools
import os
from typing import Any, Callable, Dict, List, Optional, Sequence

import torch
import torch.distributed as dist


def _default_timer(fn: Callable[[], Any]):
    """(result, milliseconds) of one call, device time when a GPU is present."""
    if torch.cuda.is_available():
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        out = fn()
        e1.record()
        torch.cuda.synchronize()
        return out, e0.elapsed_time(e1)
    import time
    t0 = time.perf_counter()
    out = fn()
    return out, (time.perf_counter() - t0) * 1e3


class _TuningState:
    def __init__(self, nconfigs: int):
        self.cfg = 0
        self.rep = 0
        self.times: List[List[float]] = [[] for _ in range(nconfigs)]
        self.finished = False


class Tunable:
    def __init__(self, fn: Callable, configs: Sequence[Dict[str, Any]], key: Optional[Callable] = None, name: Optional[str] = None):
        if not configs:
            raise ValueError("a tunable needs at least one config")
        self.fn = fn
        self.configs = list(configs)
        self.key = key or (lambda *a, **k: ())
        self.name = name or getattr(fn, "__name__", "tunable")
        self.cache: Dict[Any, Dict[str, Any]] = {}
        functools.update_wrapper(self, fn)

    def __call__(self, *args, **kwargs):
        key = self.key(*args, **kwargs)
        if key in self.cache:
            return self.fn(*args, config=self.cache[key], **kwargs)
        tuner = ContextualAutoTuner._INSTANCE
        if tuner is None or len(self.configs) == 1:
            return self.fn(*args, config=self.configs[0], **kwargs)
        return tuner._measure(self, key, args, kwargs)


def tunable(configs: Sequence[Dict[str, Any]], key: Optional[Callable] = None, name: Optional[str] = None):
    """Decorator: the function receives the chosen config as keyword argument ``config``."""
    def decor(fn):
        return Tunable(fn, configs, key, name)
    return decor


class ContextualAutoTuner:
    _INSTANCE: Optional["ContextualAutoTuner"] = None
    timer = staticmethod(_default_timer)

    def __init__(self, fn: Callable, is_dist: bool = False, n_repeat: int = 5, n_warmup: int = 3, group=None):
        self.fn = fn
        self.is_dist = is_dist
        self.n_repeat = n_repeat
        self.n_warmup = n_warmup
        self.group = group
        self._states: Dict[Any, _TuningState] = {}
        self._log = None
        functools.update_wrapper(self, fn)

    def _print(self, *args) -> None:
        rank = dist.get_rank() if dist.is_initialized() else 0
        if self._log is None:
            os.makedirs(".autotune_logs", exist_ok=True)
            self._log = open(f".autotune_logs/rank-{rank}.log", "a")
        print(f"[rank-{rank}]", *args, file=self._log, flush=True)

    def _measure(self, t: Tunable, key, args, kwargs):
        st = self._states.setdefault((id(t), key), _TuningState(len(t.configs)))
        if st.finished:  # finished earlier in this session but the cache entry was evicted
            return t.fn(*args, config=t.configs[0], **kwargs)
        cfg = t.configs[st.cfg]
        out, ms = self.timer(lambda: t.fn(*args, config=cfg, **kwargs))
        if st.rep >= self.n_warmup:
            st.times[st.cfg].append(ms)
        self._print(f"func: {t.name} | key: {key} | config-id: {st.cfg} | config: {cfg} | iter: {st.rep} | {ms:.4f} ms")
        st.rep += 1
        if st.rep >= self.n_warmup + self.n_repeat:
            st.rep = 0
            st.cfg += 1
        if st.cfg >= len(t.configs):
            means = torch.tensor([sum(x) / max(1, len(x)) for x in st.times], dtype=torch.float64)
            if self.is_dist and dist.is_initialized() and dist.get_world_size(self.group) > 1:
                dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() and dist.get_backend(self.group) == "nccl" else torch.device("cpu")
                red = means.to(dev)
                dist.all_reduce(red, op=dist.ReduceOp.MAX, group=self.group)  # a config is as slow as its slowest rank
                means = red.cpu()
            best = int(torch.argmin(means))
            t.cache[key] = t.configs[best]
            st.finished = True
            self._print(f"func: {t.name} | key: {key} | best-config-id: {best} | best-config: {t.configs[best]} | "
                        f"best-latency: {float(means[best]):.4f} ms | all: {[round(float(m), 4) for m in means]}")
        return out

    def __call__(self, *args, **kwargs):
        if ContextualAutoTuner._INSTANCE is not None:  # nested: the outer session drives
            return self.fn(*args, **kwargs)
        ContextualAutoTuner._INSTANCE = self
        self._states = {}
        try:
            first = self.fn(*args, **kwargs)  # discovers the tunables of this thunk
            if not self._states:
                return first  # everything inside is tuned already: that was a plain run
            guard = 0
            while any(not s.finished for s in self._states.values()):
                self.fn(*args, **kwargs)
                guard += 1
                if guard > 100000:
                    raise RuntimeError("autotuning did not converge")
        finally:
            ContextualAutoTuner._INSTANCE = None
            if self._log is not None:
                self._log.close()
                self._log = None
        return self.fn(*args, **kwargs)


def contextual_autotune(is_dist: bool = False, n_repeat: int = 5, n_warmup: int = 3, group=None):
    def decor(fn):
        return ContextualAutoTuner(fn, is_dist=is_dist, n_repeat=n_repeat, n_warmup=n_warmup, group=group)
    return decor
