"""Why the block-scaled tensor path (tcgen05 kind::mxf8f6f4: fp4 weights x fp8 activations, both with a power-of-two
scale per 32 values) is not built: with the activations of one expert MLP quantised to MXFP8 (e4m3 elements, OCP MX
scale 2^(floor(log2 amax) - 8)) the output leaves the parity tolerance by an order of magnitude, while fp16 activations
(what the kernels use) sit an order of magnitude inside it.  Plain numpy in float64 against the unquantised result."""
import numpy as np

from tests import cases

E2M1 = np.array([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6], np.float64)


def _mxfp4_matrix(rng, rows, cols):
    codes = rng.integers(0, 16, size=(rows, cols))
    exps = rng.integers(118, 125, size=(rows, cols // 32))           # the synthetic layers' scale range
    return E2M1[codes] * np.repeat(np.exp2(exps.astype(np.float64) - 128), 32, axis=1)


def _mxfp8(x):
    x = x.reshape(x.shape[0], -1, 32)
    amax = np.abs(x).max(axis=2, keepdims=True)
    s = np.exp2(np.floor(np.log2(np.where(amax > 0, amax, 1.0))) - 8)
    a = np.abs(x / s)
    ex = np.clip(np.floor(np.log2(np.where(a > 0, a, 1.0))), -6, 8)    # e4m3: 3 mantissa bits, subnormals below 2^-6
    step = np.exp2(ex - 3)
    q = np.minimum(np.round(a / step) * step, 448.0)
    return (np.sign(x) * q * s).reshape(x.shape[0], -1)


def _mlp(x, Wu, Wg, Wd, quant):
    xa = quant(x)
    up, gate = xa @ Wu.T, xa @ Wg.T
    g, u = np.minimum(gate, 7.0), np.clip(up, -7.0, 7.0)
    act = g / (1 + np.exp(-1.702 * g)) * (u + 1)                       # the modified SwiGLU of the benchmarked layers
    return quant(act) @ Wd.T


def test_mxfp8_activations_leave_the_tolerance_fp16_ones_do_not():
    rng = np.random.default_rng(0)
    H = F = 1024
    Wu, Wg, Wd = _mxfp4_matrix(rng, F, H), _mxfp4_matrix(rng, F, H), _mxfp4_matrix(rng, H, F)
    x = rng.standard_normal((24, H))
    ref = _mlp(x, Wu, Wg, Wd, lambda v: v)
    mx16, mr16 = cases.err_stats(_mlp(x, Wu, Wg, Wd, lambda v: v.astype(np.float16).astype(np.float64)), ref)
    mx8, mr8 = cases.err_stats(_mlp(x, Wu, Wg, Wd, _mxfp8), ref)
    assert mx16 <= cases.MAX_ABS_OVER_RMS / 5 and mr16 <= cases.MEAN_REL / 5, (mx16, mr16)
    assert mx8 > 4 * cases.MAX_ABS_OVER_RMS and mr8 > 4 * cases.MEAN_REL, (mx8, mr8)
