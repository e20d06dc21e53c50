"""SFT client, config and training processors (the names ``arctic_platform.sft`` exports in the reference,
sft/__init__.py:26-44)."""
from .client import ArcticSFTClient, create_arctic_sft_client  # noqa: F401
from .config import ArcticSFTClientConfig  # noqa: F401
from .processor import LOGIT_LOSS_FNS, SFT_LOSS_FNS, run_sft_pipeline  # noqa: F401
from ..rl.processors.losses import sft_ce_loss, sft_loss  # noqa: F401

__all__ = ["ArcticSFTClient", "ArcticSFTClientConfig", "LOGIT_LOSS_FNS", "SFT_LOSS_FNS", "create_arctic_sft_client",
           "run_sft_pipeline", "sft_ce_loss", "sft_loss"]
