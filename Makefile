# Developer entry points (make help).  GPU targets need a B200; everything else runs on a CPU-only machine
# (nvcc cross-compiles for sm_100a).
PYTHON ?= python
FLAKE_RUNS ?= 5
.DEFAULT_GOAL := help
.PHONY: help build rebuild test test-cpu test-gpu test-fast test-checked test-flaky test-reports smoke bench lint clean

help: ## this list
	@awk 'BEGIN {FS = ":.*##"} /^[0-9a-zA-Z_-]+:.*##/ {printf "  %-14s %s\n", $$1, $$2}' $(MAKEFILE_LIST)

build: ## compile the CUDA kernels and the C++ host runtime in-tree (skips what is up to date)
	$(PYTHON) -c "import __graft_entry__ as g; g.build()"

rebuild: ## compile everything again
	$(PYTHON) -m arctic_platform_b200._build --force

test: test-cpu test-gpu ## CPU tests, then GPU tests

test-cpu: ## tests that need no GPU (gloo multi-rank included)
	CUDA_VISIBLE_DEVICES="" $(PYTHON) -m pytest tests -q -m "not gpu"

test-gpu: ## kernels against fp32 PyTorch references, engines (needs a B200)
	$(PYTHON) -m pytest tests -q -m gpu

test-fast: ## CPU tests on 4 processes (pytest-xdist)
	CUDA_VISIBLE_DEVICES="" $(PYTHON) -m pytest tests -q -m "not gpu" -n 4

test-checked: ## GPU tests with every table-driven launch validated first (APB_DEBUG_CHECKS=1)
	APB_DEBUG_CHECKS=1 $(PYTHON) -m pytest tests -q -m gpu

test-flaky: ## repeat the CPU tests FLAKE_RUNS times and stop at the first failure
	@for i in $$(seq 1 $(FLAKE_RUNS)); do echo "== run $$i of $(FLAKE_RUNS)"; \
		CUDA_VISIBLE_DEVICES="" $(PYTHON) -m pytest tests -q -x -m "not gpu" || exit 1; done

test-reports: ## CPU tests with report files (durations, failures) under reports/cpu/
	CUDA_VISIBLE_DEVICES="" $(PYTHON) -m pytest tests -q -m "not gpu" --make-reports=cpu

smoke: ## one tiny forward + backward of the flagship model on cuda:0
	$(PYTHON) -c "import __graft_entry__ as g; g.build(); g.smoke()"

bench: ## the GRPO step benchmark on one GPU (torchrun ... bench.py --gpus N for more)
	$(PYTHON) bench.py

lint: ## byte-compile every source file; print what a release of this tree would run
	$(PYTHON) -m compileall -q arctic_platform_b200 arctic_platform cortex_client recipes benchmarks bench.py __graft_entry__.py
	$(PYTHON) -m arctic_platform_b200.cli.release --dry-run

clean: ## remove built libraries and objects
	rm -rf build/obj arctic_platform_b200/_C/libapb200.so arctic_platform_b200/_C/libapb200_rt.so
