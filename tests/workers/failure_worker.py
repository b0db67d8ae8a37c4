"""Host-side failure detection on CPU ranks (gloo): one rank leaves between steps, the others find out through a
short process-group timeout on their next collective and report instead of waiting forever."""
import json
import os
import time

import torch
import torch.distributed as dist

from triton_distributed_b200.ops import gemm as G
from triton_distributed_b200.runtime import initialize_distributed


def main():
    group = initialize_distributed(seed=0, timeout_s=int(os.environ.get("TDIST_TEST_PG_TIMEOUT_S", "5")))
    rank, world = dist.get_rank(), dist.get_world_size()
    a = torch.randn(16, 32)
    w = torch.randn(8, 32)
    ctx = G.create_ag_gemm_intra_node_context(a, w, rank, world, max_M=16 * world, group=group)
    G.ag_gemm_intra_node(a, w, ctx)          # a healthy step: every rank takes part
    dist.barrier(group)
    if rank == world - 1:
        # leaves between steps, with nothing of its own in flight
        os._exit(0)
    t0 = time.time()
    detected, message = False, ""
    try:
        G.ag_gemm_intra_node(a, w, ctx)      # the gloo all-gather inside can never complete
    except Exception as e:  # noqa: BLE001 - any error of the collective counts, its text is reported
        detected, message = True, repr(e)[:200]
    took = time.time() - t0
    if rank == 0:
        print("RESULT " + json.dumps({"detected": detected, "seconds": round(took, 2), "message": message}), flush=True)
    os._exit(0 if detected else 1)           # no orderly shutdown possible: the group is broken


if __name__ == "__main__":
    main()
