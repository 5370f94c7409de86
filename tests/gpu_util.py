import numpy as np
import torch


def dev(*arrs):
    return [torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda() for a in arrs]


def check(got, ref, what, rtol=1e-4, atol=1e-5):
    """|got - ref| <= atol + rtol*|ref| elementwise (fp32 result against the float64 oracle)."""
    got = got.detach().cpu().numpy().astype(np.float64) if isinstance(got, torch.Tensor) else np.asarray(got, np.float64)
    ref = np.asarray(ref, np.float64)
    assert got.shape == ref.shape, f"{what}: shape {got.shape} vs {ref.shape}"
    err = np.abs(got - ref)
    bound = atol + rtol * np.abs(ref)
    worst = float((err / bound).max()) if err.size else 0.0
    assert np.isfinite(got).all(), f"{what}: non-finite values"
    assert worst <= 1.0, (f"{what}: max |err| {err.max():.3e}, worst err/bound {worst:.2f} at "
                          f"{np.unravel_index(np.argmax(err / bound), err.shape)}, |ref| max {np.abs(ref).max():.3e}")
    return worst
