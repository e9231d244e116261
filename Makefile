# Builds every native artefact in-tree for sm_100a (see piccl_b200/build.py).
# The reference's root Makefile:5-9 delegates to src/Makefile, which produces src/piccl.so;
# here the preload library is piccl_b200/lib/piccl.so.
PYTHON ?= python

all:
	$(PYTHON) -m piccl_b200.build

force:
	$(PYTHON) -m piccl_b200.build --force

reference:
	baseline/build_ref.sh

test:
	$(PYTHON) -m pytest tests -x -q -m "not gpu"

clean:
	rm -rf build piccl_b200/lib/piccl.so piccl_b200/lib/libpiccl_ops.so piccl_b200/lib/piccl_sched piccl_b200/lib/coll_bench

.PHONY: all force reference test clean
