# Convenience targets; the build itself lives in litetorch_b200/_native.py (and CMakeLists.txt for C++ users).
PYTHON ?= python
NPROC  ?= 8

.PHONY: build host test test-gpu docs-test smoke bench bench-multi demo wheel clean

build:            ## both native libraries in-tree (nvcc for sm_100a + g++)
	$(PYTHON) -c "import __graft_entry__ as g; g.build()"

host:             ## the CUDA-free host runtime only
	$(PYTHON) -c "from litetorch_b200 import _native; print(_native.build_host())"

test:             ## CPU tier: API, runtime, gloo ranks, sanitizer builds, the user guide's examples
	$(PYTHON) -m pytest tests -q -m "not gpu"

test-gpu:         ## on a B200: every kernel against an fp32 PyTorch reference
	$(PYTHON) -m pytest tests -q -m gpu

docs-test:
	$(PYTHON) -m pytest tests/test_docs_cpu.py -q

smoke:
	$(PYTHON) -c "import __graft_entry__ as g; g.smoke()"

bench:            ## Llama-3-8B-shape training tokens/s on one GPU
	$(PYTHON) bench.py --gpus 1 --steps 10 --warmup 3

bench-multi:      ## the same on NPROC GPUs of this node
	$(PYTHON) -m torch.distributed.run --nnodes=1 --nproc-per-node $(NPROC) --master-addr 127.0.0.1 --master-port 29500 \
	    bench.py --gpus $(NPROC) --steps 10 --warmup 3

demo:             ## the C++ demo on the host runtime
	cmake -S . -B build/cmake -DLT_BUILD_CUDA=OFF -DLT_OUTPUT_DIR=$(CURDIR)/build/cmake/lib
	cmake --build build/cmake -j
	./build/cmake/lt_native_demo build/cmake

wheel:
	$(PYTHON) -m pip wheel --no-deps --no-build-isolation -w dist .

clean:
	$(PYTHON) -c "import shutil; [shutil.rmtree(p, ignore_errors=True) for p in ('build', 'dist', 'litetorch_b200.egg-info')]"
