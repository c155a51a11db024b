# Developer entry points.  Everything here runs committed files only.
PY ?= python

.PHONY: build test test-gpu bench bench-q4k serve-fake clean

build:            ## compile every CUDA source for sm_100a and the host runtime into poot_b200/lib
	$(PY) poot_b200/build.py

test:             ## CPU suite: IR, oracle, planner, loaders, driver, text, server
	$(PY) -m pytest tests -x -q -m "not gpu"

test-gpu:         ## on a B200 (multi-GPU tests skip themselves below two GPUs)
	$(PY) -m pytest tests -x -q -m gpu

bench:            ## Llama-3-8B decode / prefill on one GPU
	$(PY) bench.py --gpus 1

bench-q4k:        ## Q4_K projections + Q8_0 embeddings, batch-1 decode
	$(PY) bench.py --quant q4_k

serve-fake:       ## the HTTP server over the deterministic host engine (no GPU)
	$(PY) -m poot_b200.serve fake 127.0.0.1:8080 --rows 8 --max-seq 512 --prefill-chunk 64

clean:
	rm -rf build poot_b200/lib/*.so poot_b200/lib/obj
