"""``from config import config`` as in the reference (``config.py``): the one
module-level configuration tree that ``train.main()`` reads and wrappers mutate."""
from imfvideo_b200.config import (Config, DataConfig, LossConfig, ModelConfig,  # noqa: F401
                                  OptimConfig, ParallelConfig, RunConfig, SampleConfig, config,
                                  apply_overrides, config_as_dict, parse_cli, preset)
