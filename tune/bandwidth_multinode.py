"""Multi-node bandwidth curve: the same measurement as tune/bandwidth.py with the
``env://`` rendezvous of ``torchrun --nnodes`` and the ``_ws{N}`` file name
(reference: tune/bandwidth_multinode.py)."""
import sys

import bandwidth

if __name__ == "__main__":
    sys.argv.append("--multinode")
    bandwidth.main()
