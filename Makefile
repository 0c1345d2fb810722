# Build targets of hetu_galvatron_b200 (the same builds `pip install .` and `__graft_entry__.build()` run).
#   make            kernel library (nvcc, sm_100a) + the two pybind11 host modules, in-tree under hetu_galvatron_b200/_lib
#   make dp_core    only the strategy-search core (no CUDA toolkit needed)
#   make test       CPU test tier
#   make clean      remove built libraries and object files
PYTHON ?= python

all:
	$(PYTHON) -c "from hetu_galvatron_b200 import _build; _build.build_all()"

dp_core:
	$(PYTHON) -c "from hetu_galvatron_b200 import _build; _build.build_dp_core()"

data_index:
	$(PYTHON) -c "from hetu_galvatron_b200 import _build; _build.build_data_index()"

kernels:
	$(PYTHON) -c "from hetu_galvatron_b200 import _build; _build.build_cuda()"

test:
	$(PYTHON) -m pytest tests -q -m "not gpu"

clean:
	rm -rf hetu_galvatron_b200/_lib/obj
	rm -f hetu_galvatron_b200/_lib/*.so hetu_galvatron_b200/_lib/*.hash

.PHONY: all dp_core data_index kernels test clean
