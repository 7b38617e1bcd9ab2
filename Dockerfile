# archscale_b200 on a CUDA 12.9 PyTorch base image; the sm_100a extension is compiled in-tree at build time (nvcc
# cross-compiles without a GPU).  Replaces the reference image, which installs flash-attn, mamba-ssm, causal-conv1d,
# flash-linear-attention and liger kernels from pip / git (`Dockerfile:1-29`).
FROM nvcr.io/nvidia/pytorch:25.06-py3
WORKDIR /app
RUN pip install --no-cache-dir sentencepiece tokenizers pyarrow pandas zstandard pyyaml wandb lm-eval
COPY . /app
RUN python -m archscale_b200.build
ENV PYTHONPATH=/app
CMD ["bash", "launch_scripts/launch_dense_muonh.sh"]
