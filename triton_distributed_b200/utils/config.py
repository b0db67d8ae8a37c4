"""The library's settings in one place.

The reference has no configuration files: behaviour is steered by environment variables
(``NVSHMEM_SYMMETRIC_SIZE``, ``USE_TRITON_DISTRIBUTED_AOT``, ... reference scripts/launch.sh:2-21) and by the per-op
context dataclasses. The same holds here; :class:`Config` reads every ``TDIST_*`` variable the library understands,
with its type, default and meaning, so that a run can print what it is running with (``Config.from_env().describe()``).
The ops read the variables themselves when they need them (some are consulted on every launch and cached there);
this class is the catalogue, not a second source of truth.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, fields
from typing import Dict


@dataclass(frozen=True)
class Config:
    wait_timeout_ms: float = 4000.0      # TDIST_WAIT_TIMEOUT_MS: limit of every device-side wait (flags, mbarriers, LL packets)
    symm_heap_bytes: int = 1 << 30       # TDIST_SYMM_HEAP_BYTES: size of a symmetric-heap segment
    heap_backend: str = "auto"           # TDIST_HEAP_BACKEND: auto | vmm (cuMem + fd export) | ipc (cudaIpc) | host
    nvls: bool = False                   # TDIST_NVLS: bind heap segments to an NVSwitch multicast object (multimem ops)
    ag_gemm_nvls: int = 0                # TDIST_AG_GEMM_NVLS: AG-GEMM pushers use multimem.st (0 never, 1 from 4 ranks, 2 always)
    ag_push_slices: int = 0              # TDIST_AG_PUSH_SLICES: 1 = AG-GEMM pushers send a 128-row block as parallel row slices
    ag_push_ahead: int = 5               # TDIST_AG_PUSH_AHEAD: chunks a pusher's loads run ahead of its stores (1..5)
    ag_split_first: int = 1              # TDIST_AG_SPLIT_FIRST: 0 = keep the first round of the wide AG schedule whole
    moe_ag_push_mode: str = "auto"       # TDIST_MOE_AG_PUSH_MODE: all-gather of the one-launch AG + GroupGEMM: auto | push | push_ordered
    rs_fused_reduce: int = 1             # TDIST_RS_FUSED_REDUCE: 0 = GEMM-RS reduces the owned tiles in a pass after the GEMM
    decode_cluster_merge: int = 1        # TDIST_DECODE_CLUSTER_MERGE: 0 = the KV splits of flash decode always meet in global memory
    gemm_cta_pair: int = -1              # TDIST_GEMM_CTA_PAIR: -1 automatic, 0 one CTA per 128x256 tile, 1 CTA pair per 256x256, 2 CTA pair per 256x512
    gemm_group_m: int = 0                # TDIST_GEMM_GROUP_M: row-tiles per raster group, 0 = kernel default (8)
    bounds_check: bool = False           # TDIST_BOUNDS_CHECK: load the library built with checked symmetric-address translation
    nvtx: bool = False                   # TDIST_NVTX: wrap the ops in NVTX ranges (timelines of external profilers)
    nvcc: str = ""                       # TDIST_NVCC: compiler used by the build, empty = search PATH and /usr/local/cuda

    _ENV = {
        "wait_timeout_ms": "TDIST_WAIT_TIMEOUT_MS", "symm_heap_bytes": "TDIST_SYMM_HEAP_BYTES", "heap_backend": "TDIST_HEAP_BACKEND",
        "nvls": "TDIST_NVLS", "ag_gemm_nvls": "TDIST_AG_GEMM_NVLS", "ag_push_slices": "TDIST_AG_PUSH_SLICES",
        "ag_push_ahead": "TDIST_AG_PUSH_AHEAD", "ag_split_first": "TDIST_AG_SPLIT_FIRST", "decode_cluster_merge": "TDIST_DECODE_CLUSTER_MERGE", "rs_fused_reduce": "TDIST_RS_FUSED_REDUCE", "moe_ag_push_mode": "TDIST_MOE_AG_PUSH_MODE",
        "gemm_cta_pair": "TDIST_GEMM_CTA_PAIR",
        "gemm_group_m": "TDIST_GEMM_GROUP_M", "bounds_check": "TDIST_BOUNDS_CHECK", "nvtx": "TDIST_NVTX", "nvcc": "TDIST_NVCC",
    }

    @classmethod
    def env_names(cls) -> Dict[str, str]:
        return dict(cls._ENV)

    @classmethod
    def from_env(cls, environ=None) -> "Config":
        env = os.environ if environ is None else environ
        kw = {}
        for f in fields(cls):
            raw = env.get(cls._ENV[f.name])
            if raw is None:
                continue
            if f.type in ("bool", bool):
                kw[f.name] = raw.strip().lower() in ("1", "true", "yes", "on")
            elif f.type in ("int", int):
                kw[f.name] = int(float(raw))
            elif f.type in ("float", float):
                kw[f.name] = float(raw)
            else:
                kw[f.name] = raw
        return cls(**kw)

    def describe(self) -> str:
        default = Config()
        lines = []
        for f in fields(self):
            v, d = getattr(self, f.name), getattr(default, f.name)
            lines.append(f"{self._ENV[f.name]:<24} = {v!r}" + ("" if v == d else f"   (default {d!r})"))
        return "\n".join(lines)
