"""Worker of the host-side fault tests (gloo, CPU): argv = scenario, report path."""
import json
import os
import sys
import time
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))


def main() -> int:
    scenario, report = sys.argv[1], sys.argv[2]
    import torch.distributed as dist
    from rhinoforge_b200.parallel.tp import TPContext
    from rhinoforge_b200.runtime.errors import RPUBackendError
    tp = TPContext.from_env(backend="gloo")
    out = {"rank": tp.rank, "scenario": scenario}
    if scenario == "rank_exits_between_steps":
        for step in range(3):
            tp.heartbeat(step)
            if tp.rank == 1 and step == 1:
                os._exit(0)                           # leaves between steps, nothing in flight
            try:
                tp.check_peers(step, timeout_s=2.0)
                out[f"step{step}"] = "ok"
            except RPUBackendError as e:
                out[f"step{step}"] = f"error: {e}"
                break
    elif scenario == "rank_stalls_on_host":
        tp.heartbeat(0)
        tp.check_peers(0, timeout_s=5.0)
        if tp.rank == 1:
            time.sleep(4.0)                           # a stuck host thread: no heartbeat for step 1 in time
            out["result"] = "woke up"
        else:
            tp.heartbeat(1)
            t0 = time.monotonic()
            try:
                tp.check_peers(1, timeout_s=1.0)
                out["result"] = "no error"
            except RPUBackendError as e:
                out["result"] = "detected"
                out["seconds"] = time.monotonic() - t0
                out["message"] = str(e)
    Path(f"{report}.rank{tp.rank}.json").write_text(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
