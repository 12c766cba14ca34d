# Developer entry points (the reference's Makefile has style / lint / test targets; the build target is new).
PY ?= python

.PHONY: build test test-gpu bench smoke clean

build:            ## compile the sm_100a kernel library and the host checkpoint I/O library in-tree
	$(PY) -m olmax_b200.csrc.build

test:             ## CPU tests (multi-process paths run on gloo)
	$(PY) -m pytest tests/ -x -q -m "not gpu"

test-gpu:         ## GPU tests (need a B200; multi-GPU cases skip when fewer GPUs are visible)
	$(PY) -m pytest tests/ -x -q -m gpu

smoke: build      ## one tiny train step on cuda:0
	$(PY) __graft_entry__.py smoke

bench: build      ## flagship benchmark on one GPU
	$(PY) bench.py

clean:
	rm -rf olmax_b200/csrc/build olmax_b200/lib
