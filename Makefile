# SPDX-License-Identifier: MIT
# Top-level build: the launcher, the extension, the raw-link benchmarks.
PYTHON ?= python
CC ?= gcc
NVCC ?= nvcc
NVCC_ARCH := -gencode arch=compute_100a,code=sm_100a

.PHONY: all blrun ext bench test clean

all: blrun ext

blrun: tools/blrun

tools/blrun: tools/blrun.c
	$(CC) -O2 -Wall -o $@ $<

ext:
	$(PYTHON) -m barlink_sm86_b200._build

bench: bench/p2p_bw/p2p_bw bench/stock_d2d/stock_d2d

bench/p2p_bw/p2p_bw: bench/p2p_bw/p2p_bw.cu
	$(NVCC) -O3 -std=c++17 $(NVCC_ARCH) -lineinfo -o $@ $< -lcuda

bench/stock_d2d/stock_d2d: bench/stock_d2d/stock_d2d.cu
	$(NVCC) -O3 -std=c++17 $(NVCC_ARCH) -lineinfo -o $@ $<

test:
	$(PYTHON) -m pytest tests -x -q -m "not gpu"

clean:
	rm -f tools/blrun bench/p2p_bw/p2p_bw bench/stock_d2d/stock_d2d
	rm -rf barlink_sm86_b200/_build
