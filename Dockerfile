# Image for hivemind_b200 on Blackwell (sm_100a) machines: CUDA 12.9 toolchain (nvcc is needed at build time to compile
# the kernel library in-tree), PyTorch with CUDA 12.8 wheels, the Python dependencies, and the package built in place.
FROM nvidia/cuda:12.9.0-devel-ubuntu24.04
LABEL repository="hivemind_b200"

ENV DEBIAN_FRONTEND=noninteractive LC_ALL=C.UTF-8
RUN apt-get update && apt-get install -y --no-install-recommends build-essential git python3 python3-pip python3-venv \
    && apt-get clean && rm -rf /var/lib/apt/lists/*

RUN python3 -m venv /opt/venv
ENV PATH="/opt/venv/bin:${PATH}"
RUN pip install --no-cache-dir torch --index-url https://download.pytorch.org/whl/cu128
RUN pip install --no-cache-dir numpy msgpack protobuf cryptography pydantic scipy pyyaml sortedcontainers packaging \
    pytest pytest-timeout scikit-learn sentencepiece idna

WORKDIR /workspace/hivemind_b200
COPY . .
# compiles hivemind_b200/ops/libhm_kernels.so (every csrc/*.cu for sm_100a) and the transport daemon hmp2pd
RUN python -c "import __graft_entry__ as g; g.build()" && pip install --no-cache-dir -e .

CMD ["bash"]
