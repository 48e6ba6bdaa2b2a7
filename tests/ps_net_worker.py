"""Worker process of the cross-process parameter-server test: argv = port, rank, workers, mode."""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from tsplit_b200.parallel.ps_net import RemoteParameterServer, PSConnectionError      # noqa: E402


def main():
    port, rank, workers, mode = int(sys.argv[1]), int(sys.argv[2]), int(sys.argv[3]), sys.argv[4]
    ps = RemoteParameterServer("127.0.0.1", port, worker=rank, num_workers=workers,
                               timeout=float(os.environ.get("PS_TIMEOUT", "20")))
    if rank == 0:
        ps.init("w", np.zeros(1000, np.float32))
        ps.init("emb", np.zeros((50, 8), np.float32))
    ps.barrier()
    if mode == "leave_early" and rank == 1:
        os._exit(0)                          # leaves between steps, without a goodbye
    total = np.zeros(1000, np.float32)
    for step in range(3):
        delta = np.full(1000, float(rank + 1) * (step + 1), np.float32)
        try:
            got = ps.push_pull("w", delta, mode="BSP")
        except PSConnectionError as e:
            print("TIMEOUT %s" % e, flush=True)
            ps.close(say_bye=False)
            return 3
        total += sum(float(r + 1) * (step + 1) for r in range(workers))
        np.testing.assert_allclose(got, total, rtol=1e-6)
    rows = np.array([rank, 10 + rank], dtype=np.int64)
    ps.sparse_push("emb", rows, np.ones((2, 8), np.float32) * (rank + 1))
    ps.barrier()
    got = ps.sparse_pull("emb", np.array([0, 1, 10, 11], dtype=np.int64), 8)
    if workers == 2:
        np.testing.assert_allclose(got[:, 0], [1, 2, 1, 2])
    ps.heartbeat()
    ps.barrier()
    ps.close()
    print("WORKER_OK %d" % rank, flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
