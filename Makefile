# Thin front end to the Python build driver (counterpart of the reference's Makefile targets).
#   make            build both native libraries in-tree (g++ runtime, nvcc sm_100a kernels)
#   make test       CPU test tier        make gputest   GPU test tier (needs a B200)
#   make bench      headline benchmark on one GPU
#   make reference  build the unmodified reference under baseline/_ref for `bench.py --impl reference`
PYTHON ?= python

all:
	$(PYTHON) -m kharon_b200._build

test: all
	$(PYTHON) -m pytest tests -q -m "not gpu"

gputest: all
	$(PYTHON) -m pytest tests -q -m gpu

bench: all
	$(PYTHON) bench.py --gpus 1 --steps 10 --warmup 3

reference:
	bash baseline/build_reference.sh

plots:
	$(PYTHON) -m kharon_b200.bench.plot

clean:
	rm -f kharon_b200/_lib/libkharon_rt.so kharon_b200/_lib/libkharon_cuda.so

.PHONY: all test gputest bench reference plots clean
