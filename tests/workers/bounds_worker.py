"""Runs in a process of its own with TDIST_BOUNDS_CHECK=1, so that the library built with checked symmetric-address
translation is the one loaded: small-shape ops must behave as usual, and the probe's three out-of-range accesses must
be recorded and skipped (nothing traps, nothing past the objects is written, the context stays usable)."""
import json

import torch

from triton_distributed_b200 import _lib
from triton_distributed_b200.ops import primitives as P
from triton_distributed_b200.runtime import LocalWorld, check_status


def main():
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    res = {"checked_lib": bool(_lib.lib().tdist_bounds_checked()), "path": str(_lib.lib_path().name)}
    world = 2
    lw = LocalWorld(world, dev)
    ctxs = [P.create_primitive_context(r, world, 1024, heap=lw.heap(r)) for r in range(world)]
    for c in ctxs:
        c.source.copy_(torch.randint(0, 256, (c.nbytes,), dtype=torch.uint8, device=dev))
    # in-range traffic is untouched by the checks
    for op, kw in (("put_signal", {"value": 9, "scope": "warp"}), ("fcollect", {"scope": "block"})):
        for c in ctxs:
            P.run_primitive(c, op, phase=1, **kw)
        for c in ctxs:
            P.run_primitive(c, op, phase=2, **kw)
        check_status()
    res["in_range_ok"] = all(torch.equal(c.slot(s), ctxs[s].source) for c in ctxs for s in range(world))
    # the probe: a put running 16 bytes past the object, a put to rank `world`, a signal past the signal array
    before = [c.data.local.clone() for c in ctxs]
    sig_before = [c.sig.local.clone() for c in ctxs]
    P.run_primitive(ctxs[0], "bounds_probe", phase=1)
    torch.cuda.synchronize()
    res["skipped"] = int(ctxs[0].result[1])
    try:
        check_status()
        res["raised"] = ""
    except _lib.TdistError as e:
        res["raised"] = str(e)
    res["memory_untouched"] = all(torch.equal(b, c.data.local) for b, c in zip(before, ctxs)) and \
        all(torch.equal(b, c.sig.local) for b, c in zip(sig_before, ctxs))
    # the context is still usable and the status block is clean again
    for c in ctxs:
        P.run_primitive(c, "ring_put", phase=1)
    check_status()
    res["usable_after"] = int(ctxs[1].slot(0).view(torch.int32)[0]) == 100
    print("RESULT " + json.dumps(res), flush=True)


if __name__ == "__main__":
    main()
