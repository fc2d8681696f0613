# An image that builds the native libraries for sm_100a and runs the CPU tier of the tests at build time.
# Run it on a B200 host with the NVIDIA container runtime:
#   docker build -t litetorch-b200 .
#   docker run --gpus all --ipc=host litetorch-b200 python bench.py --gpus 1 --steps 10 --warmup 3
FROM nvidia/cuda:12.9.0-devel-ubuntu24.04

RUN apt-get update && apt-get install -y --no-install-recommends python3 python3-pip python3-venv g++ make cmake \
    && rm -rf /var/lib/apt/lists/*
RUN python3 -m venv /opt/venv
ENV PATH=/opt/venv/bin:$PATH
RUN pip install --no-cache-dir torch numpy pytest pytest-timeout

WORKDIR /workspace/litetorch-b200
COPY . .
# nvcc cross-compiles for sm_100a: no GPU is needed to build
RUN python -c "import __graft_entry__ as g; g.build()"
RUN python -m pytest tests -q -m "not gpu" -x
CMD ["python", "bench.py", "--gpus", "1", "--steps", "10", "--warmup", "3"]
