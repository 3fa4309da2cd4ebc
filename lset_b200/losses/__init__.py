from .base import LogitScale
from .contrastive import contrastive_loss
from .fused_contrastive import fused_contrastive_loss
from .infonce import infonce_loss
from .matryoshka import matryoshka_loss

__all__ = ["LogitScale", "contrastive_loss", "fused_contrastive_loss", "infonce_loss",
           "matryoshka_loss"]
