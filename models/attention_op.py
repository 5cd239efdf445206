"""``from models.attention_op import flash_jvp_attention`` as in the reference
(``models/attention_op.py:164-178``): the dense attention plug-in whose forward-mode
tangent comes from the fused primal+tangent kernel."""
from imfvideo_b200.models.imf_dit_video import (eager_math_attention,  # noqa: F401
                                                flash_jvp_attention, sdpa_flash_attention,
                                                sdpa_math_attention)
