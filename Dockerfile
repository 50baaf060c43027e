# easydel_b200 image for NVIDIA B200 hosts (sm_100a). Build: docker build -t easydel-b200 .
# The CUDA toolkit is needed at build time only for nvcc (the kernels are compiled ahead of time for sm_100a).
ARG CUDA_VERSION=12.9.1
FROM nvidia/cuda:${CUDA_VERSION}-devel-ubuntu24.04 AS build
ARG PYTHON_VERSION=3.12
ENV DEBIAN_FRONTEND=noninteractive PIP_NO_CACHE_DIR=1 PIP_BREAK_SYSTEM_PACKAGES=1
RUN apt-get update && apt-get install -y --no-install-recommends python${PYTHON_VERSION} python3-pip python3-venv \
        git ffmpeg && rm -rf /var/lib/apt/lists/*
RUN python3 -m venv /opt/venv
ENV PATH=/opt/venv/bin:$PATH
ARG TORCH_INDEX=https://download.pytorch.org/whl/cu128
RUN pip install --index-url ${TORCH_INDEX} torch && \
    pip install numpy transformers tokenizers safetensors pyarrow zstandard fastapi uvicorn pydantic prometheus_client \
        pyzmq msgpack rich pyyaml scipy pillow requests tqdm pytest
WORKDIR /workspace
COPY . /workspace
# one shared library with every kernel: nvcc -gencode arch=compute_100a,code=sm_100a
RUN python -m easydel_b200.csrc.build

FROM nvidia/cuda:${CUDA_VERSION}-runtime-ubuntu24.04
ENV DEBIAN_FRONTEND=noninteractive PATH=/opt/venv/bin:$PATH PYTHONUNBUFFERED=1 \
    NCCL_DEBUG=WARN TORCH_NCCL_ASYNC_ERROR_HANDLING=1
RUN apt-get update && apt-get install -y --no-install-recommends python3 ffmpeg && rm -rf /var/lib/apt/lists/*
COPY --from=build /opt/venv /opt/venv
COPY --from=build /workspace /workspace
WORKDIR /workspace
EXPOSE 8000 9090
# default: an OpenAI-compatible server driven by one YAML file (see easydel_b200/elarge)
ENTRYPOINT ["python", "-m", "easydel_b200.elarge"]
CMD ["--help"]
