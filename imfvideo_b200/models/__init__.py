from .imf_dit_video import (IMFDiTVideo, MLAAttention, TransformerBlock, RMSNorm,  # noqa: F401
                            SituAndMul, SwiGLUMlp, FinalLayer, flash_jvp_attention,
                            sdpa_math_attention, sdpa_flash_attention, eager_math_attention,
                            precompute_axial_rope_3d, imf_dit_video_S, imf_dit_video_B)
