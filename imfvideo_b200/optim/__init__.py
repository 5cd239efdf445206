from .moonlight import (Moonlight, build_moonlight, split_params, get_ns_coefficients,  # noqa: F401
                        solve_ns_coefficients, zeropower_via_newtonschulz5,
                        sample_normalized_spectrum, JORDAN_COEFFS)
