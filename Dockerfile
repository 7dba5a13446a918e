# Serving / training image for tilerl_b200 (B200, sm_100a).
# Build:  docker build -t tilerl-b200 .
# The CUDA extension is compiled ahead of time inside the image (nvcc cross-compiles for
# sm_100a without a GPU), so a container starts without a JIT step.
FROM nvidia/cuda:12.9.1-devel-ubuntu24.04

RUN apt-get update && apt-get install -y --no-install-recommends python3 python3-pip python3-venv git \
    && rm -rf /var/lib/apt/lists/*
RUN python3 -m venv /opt/venv
ENV PATH=/opt/venv/bin:$PATH
RUN pip install --no-cache-dir "torch==2.11.*" --index-url https://download.pytorch.org/whl/cu128 \
    && pip install --no-cache-dir fastapi uvicorn httpx pydantic safetensors tokenizers numpy nvidia-ml-py

WORKDIR /app
COPY tilerl_b200 tilerl_b200
COPY csrc csrc
COPY bench.py __graft_entry__.py ./
RUN python -m tilerl_b200.build

ENV NCCL_NVLS_ENABLE=0 TRL_HEALTH_STUCK_S=60
EXPOSE 8000
# exit code 11 = fatal device error: the supervisor restarts the container
ENTRYPOINT ["python", "-m", "tilerl_b200.cli"]
CMD ["serve", "--model", "qwen38-27b", "--host", "0.0.0.0", "--port", "8000"]
