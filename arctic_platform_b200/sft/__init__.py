from .client import ArcticSFTClient  # noqa: E402,F401
from .config import ArcticSFTClientConfig  # noqa: E402,F401
