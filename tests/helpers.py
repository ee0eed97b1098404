"""Shared helpers of the parity tests: tolerance form, error report, operand builders."""
from __future__ import annotations

import numpy as np

# |c - ref| / max(|ref|, 1) <= 1e-2 for every element: fp32 accumulation, 16-bit output.
REL_TOL = 1e-2


def rel_err(c: np.ndarray, ref: np.ndarray) -> np.ndarray:
    c = np.asarray(c, np.float64); ref = np.asarray(ref, np.float64)
    return np.abs(c - ref) / np.maximum(np.abs(ref), 1.0)


def assert_close(c: np.ndarray, ref: np.ndarray, what: str, tol: float = REL_TOL) -> float:
    assert c.shape == ref.shape, "%s: shape %s vs %s" % (what, c.shape, ref.shape)
    assert np.isfinite(c).all(), "%s: non-finite values in the output (%d)" % (what, int((~np.isfinite(c)).sum()))
    e = rel_err(c, ref)
    worst = float(e.max()) if e.size else 0.0
    if worst > tol:
        bad = np.argwhere(e > tol)
        rows = np.unique(bad[:, 0]); cols = np.unique(bad[:, 1])
        lines = ["%s: max rel err %.4g > %.1e; %d of %d elements off; %d rows (first %s), %d cols (first %s)" % (
            what, worst, tol, len(bad), e.size, len(rows), rows[:8].tolist(), len(cols), cols[:8].tolist())]
        for (i, j) in bad[:8]:
            lines.append("  [%d,%d] got %.6g want %.6g" % (i, j, c[i, j], ref[i, j]))
        raise AssertionError("\n".join(lines))
    return worst


def bits16_to_torch(raw: np.ndarray, kind: str, device):
    """raw uint16 codes -> torch fp16 / bf16 tensor on `device`."""
    import torch
    t = torch.from_numpy(raw.astype(np.int16).copy()).to(device)
    return t.view(torch.float16 if kind == "f16" else torch.bfloat16)


def torch_to_f32(t, oracle, out_dtype: str) -> np.ndarray:
    """device output tensor -> fp32 numpy via the oracle's decoders (no torch arithmetic)."""
    import torch
    if out_dtype == "f32":
        return t.detach().cpu().numpy().astype(np.float32)
    raw = t.detach().view(torch.int16).cpu().numpy().view(np.uint16)
    return oracle.widen(raw, out_dtype)
