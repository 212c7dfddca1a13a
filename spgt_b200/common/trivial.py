"""Shape helper shared by config and models (reference: common/trivial.py:78-96)."""
import numpy as np


def get_resolution_size(r_large: int, r_small: int):
    """Resolutions before/after the four interpolations: (r, r_mid, r_attn, r_mid, r).

    The scale factor sqrt(r_small / r_large) is rounded to 4 decimals, nudged up by 0.005 when its last
    decimal digit is below 5, snapped to a multiple of 0.005, and r_mid = round(r_large * factor) - 1,
    exactly as the reference computes it (e.g. (211, 53) -> 106, (141, 43) -> 77).
    """
    factor = round(float(np.sqrt(r_small / r_large)), ndigits=4)
    last_digit = float(str(factor)[-1])
    factor = round(factor, ndigits=3)
    if last_digit < 5:
        factor += 5.0e-3
    factor = int(factor / 5.0e-3 + 0.5) * 5.0e-3
    r_mid = round(r_large * factor) - 1
    return ((r_large, r_large), (r_mid, r_mid), (r_small, r_small), (r_mid, r_mid), (r_large, r_large))
