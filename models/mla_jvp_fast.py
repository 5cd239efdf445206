"""``from models.mla_jvp_fast import build_fast_jvp_state, model_du_dt_fast`` as in the
reference (``models/mla_jvp_fast.py:252,311``)."""
from imfvideo_b200.models.fast_jvp import build_fast_jvp_state, model_du_dt_fast  # noqa: F401
