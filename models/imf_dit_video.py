from imfvideo_b200.models.imf_dit_video import *  # noqa: F401,F403
from imfvideo_b200.models.imf_dit_video import (IMFDiTVideo, MLAAttention,  # noqa: F401
                                                TransformerBlock, precompute_axial_rope_3d)
