"""``from moonlight import build_moonlight`` as in the reference (``moonlight.py``)."""
from imfvideo_b200.optim.moonlight import (JORDAN_COEFFS, Moonlight, build_moonlight,  # noqa: F401
                                           get_ns_coefficients, sample_normalized_spectrum,
                                           solve_ns_coefficients, split_params,
                                           zeropower_via_newtonschulz5)
