from .trainer import Trainer, lr_at, val_loss   # noqa: F401
