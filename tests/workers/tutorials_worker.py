"""Runs every tutorial's ``run(group, rank, world, device)`` inside one process group."""
import importlib.util
import json
import os
import sys
import traceback

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
TUT = os.path.join(ROOT, "tutorials")
sys.path.insert(0, TUT)

from triton_distributed_b200.runtime import finalize_distributed, initialize_distributed  # noqa: E402


def main():
    group = initialize_distributed(seed=0)
    rank, world = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    names = sorted(f for f in os.listdir(TUT) if f[:2].isdigit() and f.endswith(".py"))
    only = os.environ.get("TDIST_TUTORIALS")
    if only:
        names = [n for n in names if n[:2] in only.split(",")]
    done, failed = [], {}
    for n in names:
        spec = importlib.util.spec_from_file_location("tut_" + n[:2], os.path.join(TUT, n))
        mod = importlib.util.module_from_spec(spec)
        good = 1
        try:
            spec.loader.exec_module(mod)
            mod.run(group, rank, world, dev)
        except Exception:  # noqa: BLE001 - keep every rank in step, report at the end
            good = 0
            failed[n] = traceback.format_exc()[-800:]
        t = torch.tensor([float(good)], device=dev)
        dist.all_reduce(t, group=group)
        if int(t.item()) == world:
            done.append(n)
        elif n not in failed:
            failed[n] = "failed on another rank"
    if rank == 0:
        print("RESULT " + json.dumps({"world": world, "device": dev.type, "done": done, "failed": failed}), flush=True)
    finalize_distributed()


if __name__ == "__main__":
    main()
