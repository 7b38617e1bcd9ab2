#!/bin/bash
# Build and check an archscale_b200 checkout.  The package needs PyTorch (CUDA 12.8+ build with sm_100 support), the
# CUDA toolkit (nvcc 12.8+) and numpy / sentencepiece / pyarrow for the data tools; nothing else is compiled or fetched:
# every kernel the reference gets from flash-attn, TransformerEngine, SonicMoE, QuACK, mamba-ssm, causal-conv1d and
# flash-linear-attention (`install.sh:49-101` of the reference) is in archscale_b200/ops/csrc and builds in-tree.
set -euo pipefail
cd "$(dirname "$0")"
python - <<'PY'
import importlib, sys
missing = [m for m in ("torch", "numpy", "sentencepiece", "pyarrow", "yaml") if importlib.util.find_spec(m) is None]
if missing:
    sys.exit("missing python packages: " + ", ".join(missing) + "  (pip install torch numpy sentencepiece pyarrow pyyaml)")
import torch
print("torch", torch.__version__, "cuda", torch.version.cuda)
PY
command -v "${NVCC:-/usr/local/cuda/bin/nvcc}" >/dev/null || { echo "nvcc not found (set NVCC=...)"; exit 1; }
python -m archscale_b200.build "$@"
python -c "import __graft_entry__ as g; g.build()"
if python -c "import torch, sys; sys.exit(0 if torch.cuda.is_available() else 1)"; then
  python -c "import __graft_entry__ as g; g.smoke()"
else
  echo "no GPU visible: built only (run 'python -m pytest tests -q -m \"not gpu\"' for the CPU suite)"
fi
