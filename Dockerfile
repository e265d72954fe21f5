# Build / run image for open_transformers_b200: CUDA 12.9 toolchain (nvcc cross-compiles sm_100a without a GPU),
# PyTorch with the cu128 runtime, and the in-tree native libraries built at image build time.
FROM nvcr.io/nvidia/pytorch:25.06-py3
WORKDIR /workspace/open_transformers_b200
COPY pyproject.toml README.md ./
COPY open_transformers_b200 ./open_transformers_b200
COPY scripts ./scripts
COPY tests ./tests
COPY bench.py __graft_entry__.py ./
RUN pip install --no-cache-dir pydantic pyyaml safetensors pyarrow pytest && pip install --no-cache-dir -e . --no-deps
RUN python __graft_entry__.py
ENV NCCL_NVLS_ENABLE=1 TORCH_NCCL_ASYNC_ERROR_HANDLING=1
CMD ["bash", "scripts/launch_single_node.sh", "open1b_b200", "8"]
