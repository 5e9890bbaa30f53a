"""The bars every numeric comparison of the tests uses.

NMSE = sum((got - want)^2) / sum(want^2) over all compared logits; `want` comes from the plain float64 implementation
with the weights exactly as stored.

  float32 engine: every product and sum is float32 (eps 6e-8); a few thousand operations per logit in random order
      give a relative error around 1e-6, NMSE around 1e-12.  Bar 1e-10, and no logit off by more than 2e-5 of the
      largest logit.
  float32 engine at the layer sizes of an 8B model (tests/test_large_shapes_gpu.py).  The 32-bit kernels add the K
      terms of a dot product one after the other into one accumulator (that is what makes their result independent of
      the batch), so a product's rounding error grows like a random walk: relative error about u * sqrt(K / 3) with
      u = 2^-24, squared 1.7e-11 at K = 14,336 and 5e-12 at K = 4,096.  Two layers of four products each, a head and
      the norms between them add up to about 1e-10, where the tiny models (K <= 384) sit near 1e-12.  Bar 1e-9,
      written with this estimate before the first comparison at this size was run; worst single logit 1e-4 of the
      largest.
  bfloat16 engine.  The plain implementation with `held=round_bf16` rounds to bfloat16 exactly the tensors the engine
      holds in bfloat16 (normed input, q/k/v, rotated q/k, attention output, projections, gate/up, their product) and
      computes everything else in float64; "noise" is the NMSE of that model against the exact one (about 3e-6 per
      rounding, ~11 roundings per layer, amplified by these small models: measured 6e-5 at 2 layers, 1e-4 to 1.6e-4
      at 3 layers).
      (1) With the plain paged attention kernel (option plain_attention) the engine rounds exactly where that model
          rounds, so the two agree except where float32 and float64 accumulation fall on different sides of a
          rounding step: a flip has probability about 2.5e-4 per element and is worth about 4e-8 of NMSE after the
          model's amplification, a few dozen flips per layer at 130 tokens -> about 2.5e-6.  Bar 1e-5, a tenth of the
          noise.
      (2) With the tensor-core attention kernel the probabilities are rounded to bfloat16 inside the kernel, at another
          place than the model rounds, so one-step flips in a sixth of the attention outputs decorrelate the two
          (measured on the first GPU run: layer-0 attention outputs differ by single bf16 steps, NMSE 2e-6, which the
          later layers amplify to the level of the noise itself).  The bar is therefore relative: the engine's NMSE
          against the exact model may be at most twice the noise.  What this cannot see (one wrong key among many)
          is the business of the kernel tests, which build inputs where one key dominates.
      A first version of this file held one constant for bf16 (1e-4, the bar mashbox-labs/mashbox uses between two
      float32 programs, tests/contracts/test_arch.py:11-38); it overlooked that the noise grows with the number of
      roundings and layers, and was replaced by these two before any test was made to pass by it.
  single kernels against their float32 plain reference: float32 kernels 1e-5 of the largest value; bf16 kernels 2e-2 of
      the largest value (inputs and outputs rounded to bf16: 2^-8 relative each, plus the rounded probabilities).
"""
NMSE_F32 = 1e-10
NMSE_F32_LARGE = 1e-9
MAXERR_F32 = 2e-5
NMSE_BF16_VS_ROUNDED = 1e-5
BF16_NOISE_FACTOR = 2.0
KERNEL_F32 = 1e-5
KERNEL_BF16 = 2e-2


def nmse(got, want):
    import numpy as np
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    return float(((got - want) ** 2).sum() / max((want ** 2).sum(), 1e-300))


def assert_logits(got, want, dtype, what="", rounded=None, same_rounding=False):
    """want: exact plain logits; rounded: plain logits with bfloat16 storage (needed when dtype is bfloat16);
    same_rounding: the engine ran with the plain attention kernel, so comparison (1) applies as well as (2)"""
    import numpy as np
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert got.shape == want.shape, (what, got.shape, want.shape)
    assert np.isfinite(got).all(), f"{what}: non-finite logits"
    e = nmse(got, want)
    if dtype == "float32":
        worst = float(np.abs(got - want).max() / np.abs(want).max())
        assert e <= NMSE_F32 and worst <= MAXERR_F32, f"{what}: float32 NMSE {e:.3e}, worst {worst:.3e}"
    else:
        assert rounded is not None
        er = nmse(got, rounded)
        noise = nmse(rounded, want)
        if same_rounding:
            assert er <= NMSE_BF16_VS_ROUNDED, f"{what}: bfloat16 NMSE against the rounded model {er:.3e}"
        assert e <= BF16_NOISE_FACTOR * noise, f"{what}: bfloat16 NMSE {e:.3e}, bfloat16's own noise {noise:.3e}"
    return e
