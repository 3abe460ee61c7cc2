"""Child process of the two-rank CPU serving test: gloo process group, fake decode back end, rank 0
listens on the port given in argv and writes the bound port to the file given in argv."""

import os
import sys

import torch.distributed as dist

_HERE = os.path.dirname(os.path.abspath(__file__))
sys.path[:0] = [_HERE, os.path.dirname(_HERE)]

from test_serve_stack import FakeBackend  # noqa: E402

from nexrt_b200.serve.bridge_serve import BridgeServer, ByteTokenizer  # noqa: E402
from nexrt_b200.serve.process_supervisor import launch_geometry  # noqa: E402


def main() -> int:
    port_file, drift_rank = sys.argv[1], int(sys.argv[2])
    rank, world, _ = launch_geometry()
    dist.init_process_group("gloo", rank=rank, world_size=world)
    backend = FakeBackend()
    if rank == drift_rank:
        # this rank "loses" its boundary after the first request: restore flips the pending token once
        orig, seen = backend.restore, []

        def restore(session):
            b = orig(session)
            if not seen:
                seen.append(1)
                backend.eng.pending ^= 1
                return backend.boundary()
            return b

        backend.restore = restore
    server = BridgeServer(backend, ByteTokenizer(), rank, world, None, log=lambda *_: None)

    def ready(port):
        with open(port_file + ".tmp", "w") as f:
            f.write(str(port))
        os.replace(port_file + ".tmp", port_file)

    server.serve_forever(port=0, ready=ready)
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
