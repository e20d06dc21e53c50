# Developer entry points.  GPU targets need a B200; everything else runs on a CPU-only machine (nvcc cross-compiles).
PYTHON ?= python

.PHONY: build rebuild test test-cpu test-gpu bench smoke clean

build:
	$(PYTHON) -c "import __graft_entry__ as g; g.build()"

rebuild:
	$(PYTHON) -m arctic_platform_b200._build --force

test: test-cpu test-gpu

test-cpu:
	CUDA_VISIBLE_DEVICES="" $(PYTHON) -m pytest tests -q -m "not gpu"

test-gpu:
	$(PYTHON) -m pytest tests -q -m gpu

smoke:
	$(PYTHON) -c "import __graft_entry__ as g; g.build(); g.smoke()"

bench:
	$(PYTHON) bench.py

clean:
	rm -rf build/obj arctic_platform_b200/_C/libapb200.so arctic_platform_b200/_C/libapb200_rt.so
