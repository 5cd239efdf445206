from .dist import (init_distributed, resolve_device, broadcast_module, is_dist,  # noqa: F401
                   world_size, get_rank, barrier, shutdown, Heartbeat, RankLostError)
from .owner import assign_owners, ns_cost  # noqa: F401
