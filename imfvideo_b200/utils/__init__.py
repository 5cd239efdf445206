from .schedule import lr_at  # noqa: F401
from .ema import ema_update  # noqa: F401
from .checkpoint import (save_checkpoint, load_checkpoint, latest_checkpoint,  # noqa: F401
                         checkpoint_path)
from .timers import PhaseTimer  # noqa: F401
from .versions import mark_written  # noqa: F401
