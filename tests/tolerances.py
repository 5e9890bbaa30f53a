"""The bars every numeric comparison of the tests uses, fixed before the first GPU run.

NMSE = sum((got - want)^2) / sum(want^2) over all compared logits, `want` from the plain float64 implementation with the
weights exactly as stored.

  float32 engine: every product and sum is float32 (eps 6e-8); a few thousand operations per logit in random order
      give a relative error around 1e-6, NMSE around 1e-12.  Bar 1e-10, and no logit off by more than 2e-5 of the
      largest logit.
  bfloat16 engine: activations, cache and probabilities are rounded to 8 bits of mantissa (relative step 2^-9, rms
      error 0.11 %) a handful of times per layer with a float32 residual stream; the logits come out with a relative
      error of a few tenths of a percent, NMSE around 1e-5.  Bar 1e-4, the bar mashbox-labs/mashbox uses for its
      float comparisons (tests/contracts/test_arch.py:11-38).
  single kernels against their float32 plain reference: float32 kernels 1e-5 of the largest value; bf16 kernels 2e-2 of
      the largest value (inputs and outputs rounded to bf16: 2^-8 relative each, plus the rounded probabilities).
"""
NMSE_F32 = 1e-10
MAXERR_F32 = 2e-5
NMSE_BF16 = 1e-4
KERNEL_F32 = 1e-5
KERNEL_BF16 = 2e-2


def nmse(got, want):
    import numpy as np
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    return float(((got - want) ** 2).sum() / max((want ** 2).sum(), 1e-300))


def assert_logits(got, want, dtype, what=""):
    import numpy as np
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert got.shape == want.shape, (what, got.shape, want.shape)
    assert np.isfinite(got).all(), f"{what}: non-finite logits"
    e = nmse(got, want)
    if dtype == "float32":
        worst = float(np.abs(got - want).max() / np.abs(want).max())
        assert e <= NMSE_F32 and worst <= MAXERR_F32, f"{what}: float32 NMSE {e:.3e}, worst {worst:.3e}"
    else:
        assert e <= NMSE_BF16, f"{what}: bfloat16 NMSE {e:.3e}"
    return e
