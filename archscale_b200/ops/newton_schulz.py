"""Newton–Schulz orthogonalisation (quintic, 5 fixed coefficient sets).

Behavioural reference: `lit_gpt/optim/muon.py:869-897` (``zeropower_via_newtonschulz5``) and the
kernel split of `lit_gpt/optim/newton_schulz_triton.py:344-381`: per iteration
``A = X Xᵀ`` (symmetric), ``B = b·A + c·A²`` (symmetric), ``X ← a·X + B X``; input cast to
bf16, transposed when tall, divided by ``‖X‖_F + ε``.

CUDA path: the three products run on the tcgen05 GEMM (``csrc/gemm_bf16.cu``) with fused
``α·AB + β·C`` epilogues; ``A`` and ``B`` are symmetric so the NT layout serves all three, and the batched
kernel computes only the tiles on and above the diagonal of those two products (stored twice, once transposed).
"""
from __future__ import annotations

import torch

from . import backend

NS_COEFFS = (
    (4.0848, -6.8946, 2.9270),
    (3.9505, -6.3029, 2.6377),
    (3.7418, -5.5913, 2.3037),
    (2.8769, -3.1427, 1.2046),
    (2.8366, -3.0525, 1.2012),
)


# Polar-Express coefficient schedule of the matrix-sign iteration used by MuonBall
# (`emerging_optimizers/orthogonalized_optimizers/spectral_ball_utils.py:55-64`); steps beyond the 8th repeat the last set.
POLAR_EXPRESS_COEFFS = (
    (8.2051, -22.9019, 16.4607),
    (4.0664, -2.8612, 0.5184),
    (3.9096, -2.8234, 0.5250),
    (3.2856, -2.4153, 0.4853),
    (2.2779, -1.6198, 0.3985),
    (1.8726, -1.2307, 0.3585),
    (1.8564, -1.2132, 0.3568),
    (1.8750, -1.2500, 0.3750),
)


def newton_schulz_ref(G: torch.Tensor, epsilon: float = 1e-7, dtype: torch.dtype = torch.bfloat16,
                      coeffs=None) -> torch.Tensor:
    NS_COEFFS = coeffs if coeffs is not None else globals()["NS_COEFFS"]
    X = G.to(dtype)
    tall = G.size(-2) > G.size(-1)
    if tall:
        X = X.mT
    X = X / (X.norm(dim=(-2, -1), keepdim=True) + epsilon)
    for a, b, c in NS_COEFFS:
        A = X @ X.mT
        Bm = b * A + c * (A @ A)
        X = a * X + Bm @ X
    return X.mT if tall else X


def _ns_cuda_2d(G: torch.Tensor, epsilon: float, coeffs=None) -> torch.Tensor:
    NS_COEFFS = coeffs if coeffs is not None else globals()["NS_COEFFS"]
    ext = backend.require_extension()
    X = G.to(torch.bfloat16)
    tall = G.size(-2) > G.size(-1)
    if tall:
        X = X.t()
    X = (X / (X.norm() + epsilon)).contiguous()
    for a, b, c in NS_COEFFS:
        # A = X Xᵀ            (NT with both operands = X)
        A = ext.gemm_bf16_epi(X, X, 0, 1.0, 0.0, None)
        # B = c·A A + b·A     (A symmetric → A Aᵀ = A A)
        Bm = ext.gemm_bf16_epi(A, A, 0, c, b, A)
        # X = B X + a·X       (NN)
        X = ext.gemm_bf16_epi(Bm, X, 1, 1.0, a, X)
        backend.count_launch(3)
    return X.t() if tall else X


def _ns_cuda_batched(G: torch.Tensor, epsilon: float, coeffs=None) -> torch.Tensor:
    """G:(B,m,n) — all B matrices advance together: 3 batched tcgen05 GEMM launches per iteration.  Wide matrices iterate
    ``A = X·Xᵀ``, ``X ← a·X + B·X``; tall ones the mirrored form ``A = Xᵀ·X``, ``X ← a·X + X·B`` on the untransposed
    data (TN and NN products), so that no transposed copy of the stack is made on the way in or out."""
    NS_COEFFS = coeffs if coeffs is not None else globals()["NS_COEFFS"]
    ext = backend.require_extension()
    X = G.to(torch.bfloat16)
    tall = G.size(-2) > G.size(-1)
    pair = hasattr(ext, "gemm_pair") and ext.gemm_pair()
    in_place_tall = tall and pair
    if tall and not in_place_tall:
        X = X.mT
    X = X.contiguous()
    # X₀ = G·s with s = 1 / (‖G‖ + ε).  The two-CTA kernel takes per-matrix factors, so the scaled copy is never made: the
    # first iteration multiplies s² into the Gram product and s (and a·s) into the update of the unscaled matrices.
    s_vec = 1.0 / (torch.linalg.vector_norm(X, dim=(-2, -1), dtype=torch.float32) + epsilon)
    s2_vec = None
    if pair:
        s2_vec = (s_vec * s_vec).contiguous()
        s_vec = s_vec.contiguous()
    else:
        X = (X * s_vec.view(-1, 1, 1).to(X.dtype)).contiguous()
    for it, (a, b, c) in enumerate(NS_COEFFS):
        first = pair and it == 0
        av, sv = (s2_vec, s_vec) if first else (None, None)
        # the Gram matrix and the polynomial in it are symmetric: the kernel computes the upper triangle of tiles and mirrors it
        if in_place_tall:
            A = ext.gemm_bf16_batched(X, X, 2, 1.0, 0.0, None, True, av, None)
            Bm = ext.gemm_bf16_batched(A, A, 0, c, b, A, True)
            X = ext.gemm_bf16_batched(X, Bm, 1, 1.0, a, X, False, sv, sv)
        else:
            A = ext.gemm_bf16_batched(X, X, 0, 1.0, 0.0, None, True, av, None)
            Bm = ext.gemm_bf16_batched(A, A, 0, c, b, A, True)
            X = ext.gemm_bf16_batched(Bm, X, 1, 1.0, a, X, False, sv, sv)
        backend.count_launch(3)
    return X.mT if (tall and not in_place_tall) else X


def newton_schulz(G: torch.Tensor, epsilon: float = 1e-7, coeffs=None) -> torch.Tensor:
    """Orthogonalise the last two dims of ``G`` (2-D or batched 3-D); ``coeffs`` overrides the (a, b, c) schedule."""
    m, n = G.shape[-2], G.shape[-1]
    if (G.is_cuda and min(m, n) % 8 == 0 and max(m, n) % 8 == 0 and min(m, n) >= 64
            and backend.use_cuda_kernel("newton_schulz", G)):
        if G.dim() == 2:
            return _ns_cuda_2d(G, epsilon, coeffs)
        if backend.has("gemm_bf16_batched"):
            return _ns_cuda_batched(G.reshape(-1, m, n), epsilon, coeffs).reshape(G.shape)
        return torch.stack([_ns_cuda_2d(g, epsilon, coeffs) for g in G.reshape(-1, m, n)]).reshape(G.shape)
    return newton_schulz_ref(G, epsilon, coeffs=coeffs)
