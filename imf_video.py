"""``from imf_video import IMFVideoLoss`` as in the reference (``imf_video.py``)."""
from imfvideo_b200.loss import IMFVideoLoss  # noqa: F401
