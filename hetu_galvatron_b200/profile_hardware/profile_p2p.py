"""Send / receive bandwidth between pipeline neighbours for every pipeline degree (reference:
galvatron/profile_hardware/profile_p2p.py).

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 hetu_galvatron_b200/profile_hardware/profile_p2p.py
"""
import os
import sys

sys.path.insert(0, os.path.abspath(os.path.join(os.path.dirname(__file__), "..", "..")))  # run from a source checkout

from hetu_galvatron_b200.profiler.hardware_profiler import main

if __name__ == "__main__":
    main(sys.argv[1:] + ["--only", "p2p"])
