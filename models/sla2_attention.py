"""``from models.sla2_attention import SLA2AttentionImpl`` as in the reference
(``models/sla2_attention.py:23-61``)."""
from imfvideo_b200.models.sla2 import SLA2, Router, SLA2AttentionImpl  # noqa: F401
