"""Offline calibration of 3-bit weight copies.

Two fitters, both plain PyTorch (they run once per checkpoint, on CPU or GPU):

* `fit_codebook` — the reference's logical format (weights/w3.py `CodebookW3`): an fp32 multiplier per row, an e4m3
  scale per 32 columns, and ONE 8-entry codebook per matrix fitted by weighted Lloyd iterations on the scaled
  weights (levels need not be uniform: they follow the bell shape of the weights). With calibration inputs the
  Lloyd weights are the diagonal of the layer Hessian H = X^T X, so columns that see large activations are
  matched more closely.
* `gptq_int3g64` — the kernel's format (`Int3G64`: asymmetric 3-bit integers, groups of 64, bf16 scale + zero)
  with GPTQ error feedback: columns are quantised left to right in blocks and the rounding error of each column
  is pushed onto the not-yet-quantised ones through the inverse Hessian's Cholesky factor, which minimises
  ||X W^T - X W_q^T|| rather than ||W - W_q||.

`collect_hessian` accumulates H from activation batches; `layer_error` reports the relative output error of a
quantised copy on held-out inputs (the number the calibration reports are made of).
Reference: hibana/weights/w3_calibrate.py (Lloyd codebooks), hibana/weights/w3_calibration.py,
hibana/weights/calibration_inputs.py, docs/w3-calibration.md:20-110.
"""
from __future__ import annotations

from typing import Optional

import torch

from .w3 import CodebookW3, Int3G64

E4M3_MAX = 448.0


def collect_hessian(batches, dim: int, device="cpu") -> torch.Tensor:
    """H = sum_b X_b^T X_b / rows over activation batches [rows, dim] (fp64 accumulate)."""
    h = torch.zeros(dim, dim, dtype=torch.float64, device=device)
    n = 0
    for x in batches:
        x = x.reshape(-1, dim).to(device=device, dtype=torch.float64)
        h += x.t() @ x
        n += x.shape[0]
    return (h / max(n, 1)).float()


def _e4m3_round(x: torch.Tensor) -> torch.Tensor:
    return x.clamp(min=2.0 ** -9, max=E4M3_MAX).to(torch.float8_e4m3fn).float()


def fit_codebook(w: torch.Tensor, hessian_diag: Optional[torch.Tensor] = None, iters: int = 25,
                 sample: int = 1 << 20) -> CodebookW3:
    """w [N, K] (K % 32 == 0) -> CodebookW3. Scales are chosen so that a group's largest magnitude maps to the
    largest codebook magnitude; the codebook is then re-fitted on the normalised weights, twice (the scales depend
    on the outer level)."""
    n, k = w.shape
    assert k % 32 == 0
    wf = w.float()
    row_scale = wf.abs().amax(1).clamp_min(1e-12)                        # fp32 per row
    wn = wf / row_scale[:, None]
    g = wn.view(n, k // 32, 32)
    imp = None
    if hessian_diag is not None:
        imp = hessian_diag.float().clamp_min(0).view(1, k // 32, 32).expand(n, -1, -1)
    book = torch.tensor([-1.0, -0.62, -0.36, -0.12, 0.12, 0.36, 0.62, 1.0])
    book = book.to(w.device)
    for _ in range(2):
        top = book.abs().max()
        # the stored e4m3 scale carries a fixed factor 64 (folded into the row multiplier) to stay in its normal range
        scales = _e4m3_round(g.abs().amax(-1) / top * 64.0) / 64.0
        z = (g / scales[..., None].clamp_min(1e-12)).reshape(-1)
        wts = imp.reshape(-1) if imp is not None else None
        if z.numel() > sample:                                           # Lloyd on a subsample of a large matrix
            idx = torch.randint(0, z.numel(), (sample,), device=z.device,
                                generator=torch.Generator(device=z.device).manual_seed(0))
            zs, ws = z[idx], (wts[idx] if wts is not None else None)
        else:
            zs, ws = z, wts
        for _ in range(iters):
            code = (zs[:, None] - book[None, :]).abs().argmin(1)
            for c in range(8):
                m = code == c
                if m.any():
                    book[c] = (zs[m] * ws[m]).sum() / ws[m].sum().clamp_min(1e-20) if ws is not None else zs[m].mean()
            book = book.sort().values
    top = book.abs().max()
    stored = _e4m3_round(g.abs().amax(-1) / top * 64.0)
    z = g / (stored / 64.0)[..., None].clamp_min(1e-12)
    codes = (z[..., None] - book).abs().argmin(-1).view(n, k).to(torch.uint8)
    return CodebookW3.pack(codes, stored.to(torch.float8_e4m3fn), row_scale / 64.0, book.tolist())


def gptq_int3g64(w: torch.Tensor, hessian: torch.Tensor, block: int = 128, damp: float = 0.01) -> Int3G64:
    """GPTQ onto asymmetric 3-bit / group-64: returns an Int3G64 whose dequantised weights minimise the layer's
    output error under `hessian` [K, K]. Group parameters are fixed from the (error-compensated) weights of the
    group when its first column is reached."""
    n, k = w.shape
    assert k % 64 == 0 and hessian.shape == (k, k)
    wq = w.float().clone()
    h = hessian.float().clone()
    dead = torch.diag(h) == 0
    h[dead, dead] = 1.0
    wq[:, dead] = 0
    h += torch.eye(k, device=h.device) * damp * torch.diag(h).mean()
    hinv = torch.linalg.cholesky(torch.cholesky_inverse(torch.linalg.cholesky(h)), upper=True)   # U with H^-1 = U^T U
    out = torch.zeros_like(wq)
    scale = torch.zeros(n, k // 64, device=w.device)
    zero = torch.zeros(n, k // 64, device=w.device)
    codes = torch.zeros(n, k, dtype=torch.uint8, device=w.device)
    for b0 in range(0, k, block):
        b1 = min(b0 + block, k)
        wb = wq[:, b0:b1].clone()
        err = torch.zeros_like(wb)
        hb = hinv[b0:b1, b0:b1]
        for j in range(b1 - b0):
            col = b0 + j
            gi = col // 64
            if col % 64 == 0:                      # fix the group's scale / zero from its current weights
                grp = torch.cat([wb[:, j:min(j + 64, b1 - b0)], wq[:, b1:min(col + 64, k)]], 1) if col + 64 > b1 \
                    else wb[:, j:j + 64]
                lo, hi = grp.amin(1), grp.amax(1)
                sc = ((hi - lo) / 7.0).clamp_min(1e-8).bfloat16().float()
                scale[:, gi] = sc
                zero[:, gi] = torch.round(-lo / sc).clamp(0, 7)
            sc, zp = scale[:, gi], zero[:, gi]
            c = torch.round(wb[:, j] / sc + zp).clamp(0, 7)
            q = (c - zp) * sc
            codes[:, col] = c.to(torch.uint8)
            out[:, col] = q
            e = (wb[:, j] - q) / hb[j, j]
            wb[:, j + 1:] -= e[:, None] * hb[j, j + 1:][None, :]
            err[:, j] = e
        wq[:, b1:] -= err @ hinv[b0:b1, b1:]
    return Int3G64(codes, scale.bfloat16(), zero.bfloat16())


def layer_error(w: torch.Tensor, wq: torch.Tensor, x: torch.Tensor) -> float:
    """Relative output error ||x w^T - x wq^T|| / ||x w^T|| on inputs x [rows, K]."""
    ref = x.float() @ w.float().t()
    return float((ref - x.float() @ wq.float().t()).norm() / ref.norm().clamp_min(1e-20))
