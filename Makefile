# Convenience targets; the work is done by the Python entry points.
PY ?= python3

.PHONY: all build test test-gpu bench clean

all: build

build:            ## every native library and binary, for sm_100a, in-tree
	$(PY) -c "import __graft_entry__ as g; g.build()"

test:             ## CPU tests
	$(PY) -m pytest tests -q -m "not gpu"

test-gpu:         ## needs a B200
	$(PY) -m pytest tests -q -m gpu

bench:            ## headline benchmark on one GPU
	$(PY) bench.py

clean:
	rm -rf bin ccbench_b200/_native build
	find . -name __pycache__ -type d -prune -exec rm -rf {} +
