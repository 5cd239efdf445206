"""``from models.sla2_cube_qat import SLA2CubeQATAttentionImpl`` as in the reference
(``models/sla2_cube_qat.py:295-439``)."""
from imfvideo_b200.models.sla2 import (SLA2CubeQATAttentionImpl, cube_dense_ref,  # noqa: F401
                                       route_tiles, tile_permutation)
