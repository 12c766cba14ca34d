# Runtime image: CUDA 12.9 toolchain (nvcc builds the sm_100a kernels in-tree at image build time) + PyTorch.
FROM nvidia/cuda:12.9.0-devel-ubuntu24.04

RUN apt-get update && apt-get install -y --no-install-recommends python3 python3-pip python3-venv git && rm -rf /var/lib/apt/lists/*
RUN python3 -m venv /opt/venv && /opt/venv/bin/pip install --no-cache-dir torch numpy pyyaml rich pytest pytest-timeout
ENV PATH=/opt/venv/bin:$PATH

WORKDIR /workspace/olmax_b200
COPY . .
RUN python -m olmax_b200.csrc.build && pip install --no-cache-dir -e .

# one process per GPU: python -m olmax_b200.launch.local --nproc 8 -- -m olmax_b200.launch.train_transformer --recipe=olmo2_7B ...
ENTRYPOINT ["python", "-m", "olmax_b200.launch.local"]
