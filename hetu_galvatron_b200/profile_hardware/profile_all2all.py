"""All-reduce and all-to-all latency tables, 1 MB ... 1 GB, for every group size (reference:
galvatron/profile_hardware/profile_all2all.py and the sp_time part of profile_hardware.py).

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 hetu_galvatron_b200/profile_hardware/profile_all2all.py
"""
import os
import sys

sys.path.insert(0, os.path.abspath(os.path.join(os.path.dirname(__file__), "..", "..")))  # run from a source checkout

from hetu_galvatron_b200.profiler.hardware_profiler import main

if __name__ == "__main__":
    main(sys.argv[1:] + ["--only", "sp"])
