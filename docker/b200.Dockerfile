# Image for vllm_metax_b200 on NVIDIA B200 (sm_100a).
#   docker build -f docker/b200.Dockerfile -t vllm-metax-b200 .
#   docker run --gpus all --ipc=host -p 8000:8000 -v /models:/models vllm-metax-b200 \
#       serve /models/Llama-3.1-8B-Instruct --max-model-len 8192
# The CUDA extension is compiled for sm_100a at build time (nvcc cross-compiles; the build needs no GPU).
ARG CUDA_VERSION=12.9.1
FROM nvidia/cuda:${CUDA_VERSION}-devel-ubuntu24.04

ENV DEBIAN_FRONTEND=noninteractive PIP_NO_CACHE_DIR=1 PYTHONUNBUFFERED=1
RUN apt-get update && apt-get install -y --no-install-recommends python3 python3-pip python3-venv python3-dev git ninja-build \
    && rm -rf /var/lib/apt/lists/*
RUN python3 -m venv /opt/venv
ENV PATH=/opt/venv/bin:$PATH CUDA_HOME=/usr/local/cuda

ARG TORCH_INDEX=https://download.pytorch.org/whl/cu128
RUN pip install --index-url ${TORCH_INDEX} torch
RUN pip install numpy transformers safetensors fastapi uvicorn pydantic nvidia-ml-py httpx pybind11 ninja regex

WORKDIR /workspace/vllm_metax_b200
COPY pyproject.toml README.md ./
COPY vllm_metax_b200 ./vllm_metax_b200
COPY bench.py __graft_entry__.py ./
# in-tree build of csrc/*.cu (-gencode arch=compute_100a,code=sm_100a) and of the VMM allocator module
RUN python -c "from vllm_metax_b200 import _build; _build.build(); _build.build_cumem()"
RUN pip install --no-build-isolation --no-deps -e .

# NCCL over NVLink / NVSwitch inside one node; the fused collectives use CUDA IPC, so run with --ipc=host
ENV NCCL_DEBUG=WARN
EXPOSE 8000
ENTRYPOINT ["b200-serve"]
CMD ["--help"]
