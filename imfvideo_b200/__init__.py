"""imfvideo_b200: a B200-native (sm_100a) training framework for improved-
MeanFlow (iMF) video diffusion transformers."""

__version__ = "0.1.0"
