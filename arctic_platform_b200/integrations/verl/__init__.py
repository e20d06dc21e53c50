"""verl plugin: a ``RemoteBackend`` adapter, a CPU forwarder worker, a token-in/token-out rollout server and the
lazy registration hook (``VERL_USE_EXTERNAL_MODULES=arctic_platform_b200.integrations.verl.register``).
Counterpart of arctic_platform/integrations/verl/ in the reference."""
from .adapter import ArcticRLClientWrapper, cfg_get, no_padding_to_padded_prompt_response, prepare_padded_batch  # noqa: F401
from .grpo_loss import verl_grpo_loss  # noqa: F401
