"""Shared checks for the parity tests."""
import numpy as np

import oracle


def golden_cases(g):
    names = sorted({k.split(".")[0] for k in g.files})
    for n in names:
        yield (n, g[n + ".x"].view(np.float16), g[n + ".wq"], g[n + ".s"].view(np.float16),
               g[n + ".w"].view(np.float16), g[n + ".y"].view(np.float16))


def assert_bits_equal(a, b, what=""):
    a = np.ascontiguousarray(a).view(np.uint16)
    b = np.ascontiguousarray(b).view(np.uint16)
    assert a.shape == b.shape, (what, a.shape, b.shape)
    bad = np.flatnonzero(a.ravel() != b.ravel())
    assert bad.size == 0, f"{what}: {bad.size} of {a.size} fp16 values differ, first at {bad[:5]}"


# Tolerance of the matmul output.  The stated bar is max relative error <= 1e-2 with fp32
# accumulation.  Products are exact in fp32 in both implementations, so the only legitimate
# differences are the fp32 summation order (bounded by a few ulp_fp32 of sum|x*w|) and the
# final fp16 rounding landing on a neighbouring value (2^-10 relative).  The check below is
# that tighter bound; it implies the 1e-2 bar wherever the output is not a near-total
# cancellation, and for those it bounds the absolute error instead.
#
# The skinny kernel's default ("fast") form does not round each dequantised weight to fp16 before the
# accumulation (it scales fp32 group sums instead), so its result differs from the reference's by the
# reference's own weight-rounding noise: per weight at most half an fp16 ulp, uniformly distributed, hence
# a deviation with standard deviation (2^-11 / sqrt 3) * sqrt(sum (x*w)^2).  unrounded_slack() is twelve of
# those standard deviations (eight for the rounding noise, the rest for the fp32 cancellation of the
# magic-number offsets inside the tensor core); the exact form (option gemv.exact = 1) is held to the
# tight bound alone.
REL_TOL = 1e-2


def skinny_form_is_unrounded(m) -> bool:
    """True when a matmul with `m` activation rows goes, under the current options, through the skinny
    kernel's fast form."""
    from relax_b200 import _lib

    return m <= 16 and _lib.get_option("gemv.exact") != 1


def unrounded_slack(x, w):
    xf, wf = x.astype(np.float64), w.astype(np.float64)
    return 12.0 * (2.0 ** -11 / np.sqrt(3.0)) * np.sqrt((xf * xf) @ (wf * wf).T)


def offset_cancellation_slack(x, scales):
    """The fast form feeds the tensor core nibbles that still carry their magic-number offset (1024 + q, 64 + q) and
    starts each group's accumulator at minus the offset's share, so a group sum is the fp32 difference of two numbers
    about 1031 * sum|x| large: an absolute error of the order 2^-24 * 1031 * sum_{k in group} |x_k| per group, whatever
    the weights are (it shows when they are all zero).  Measured about 1.2e-5 * sum|x| per group; the slack is 1e-4."""
    sf = np.repeat(scales.astype(np.float64), 32, axis=1)
    return 1e-4 * (np.abs(x.astype(np.float64)) @ np.abs(sf).T)


def assert_matmul_close(y, x, wq, s, what="", y_ref=None, unrounded=None):
    y = np.asarray(y, dtype=np.float16)
    w = oracle.c_dequantize(wq, s)
    if y_ref is None:
        y_ref = oracle.c_matmul(x, wq, s)
    if unrounded is None:
        unrounded = skinny_form_is_unrounded(x.shape[0])
    absdot = np.abs(x.astype(np.float32)) @ np.abs(w.astype(np.float32)).T
    yf, rf = y.astype(np.float64), y_ref.astype(np.float64)
    assert np.isfinite(yf).all() or not np.isfinite(rf).all(), f"{what}: non-finite output"
    err = np.abs(yf - rf)
    bound = 2.0 ** -10 * np.abs(rf) + 8e-6 * absdot + 2.0 ** -24
    spread = None
    if unrounded:
        spread = unrounded_slack(x, w)
        bound = bound + spread + offset_cancellation_slack(x, s)
    worst = np.argmax(err - bound)
    assert (err <= bound).all(), (
        f"{what}: |y-ref|={err.ravel()[worst]:.3e} > bound {bound.ravel()[worst]:.3e} at flat index {worst} "
        f"(y={yf.ravel()[worst]}, ref={rf.ravel()[worst]})")
    # the bar as stated: relative error on every output that is not a near-total cancellation
    # (exact form: |ref| above a thousandth of sum|x*w|; fast form: |ref| above half the output's own spread,
    # sqrt(sum (x*w)^2) = spread / (12 * 2^-11 / sqrt 3))
    big = np.abs(rf) > 1e-3 * absdot if not unrounded else np.abs(rf) > 0.5 * spread / (12.0 * 2.0 ** -11 / np.sqrt(3.0))
    if big.any():
        rel = (err[big] / np.abs(rf[big])).max()
        assert rel <= REL_TOL, f"{what}: max rel err {rel:.3e} > {REL_TOL}"
    if unrounded and yf.size >= 256:
        # taken over many outputs the deviation must look like that noise (about 3e-4 of the outputs' spread), not like
        # a misplaced scale or nibble (percent and up)
        rms = np.sqrt(np.mean(err ** 2)) / max(np.sqrt(np.mean(rf ** 2)), 1e-30)
        assert rms <= 1.5e-3, f"{what}: rms deviation {rms:.3e} of the outputs' rms"
