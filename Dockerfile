# Build image: CUDA 12.9 toolchain + PyTorch; `docker build -t stdml-collective-b200 .`
# The kernels are sm_100a only; the image builds anywhere, the device path runs on B200.
FROM nvidia/cuda:12.9.0-devel-ubuntu24.04
RUN apt-get update && apt-get install -y --no-install-recommends python3 python3-pip python3-venv g++ make cmake ninja-build \
    && rm -rf /var/lib/apt/lists/*
RUN python3 -m venv /venv && /venv/bin/pip install --no-cache-dir torch numpy pytest
ENV PATH=/venv/bin:${PATH}
WORKDIR /src
COPY . .
RUN make -C stdml_collective_experimental_b200/csrc -j"$(nproc)" \
    && python -c "import __graft_entry__ as g; g.build()"
CMD ["python", "-m", "pytest", "tests", "-q", "-m", "not gpu"]
