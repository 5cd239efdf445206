"""Entry point with the reference's name: ``python train.py [group.key=value ...]``
or ``torchrun --nproc-per-node N train.py ...`` (reference ``train.py``)."""
from imfvideo_b200.train import (Trainer, build_model, build_optimizer, lr_at, main,  # noqa: F401
                                 qk_clip)
from imfvideo_b200.utils.ema import ema_update  # noqa: F401
from imfvideo_b200.parallel.grad_sync import all_reduce_grads  # noqa: F401
from imfvideo_b200.data.dataset import LatentDataset  # noqa: F401
from imfvideo_b200.config import config_as_dict  # noqa: F401

if __name__ == "__main__":
    main()
