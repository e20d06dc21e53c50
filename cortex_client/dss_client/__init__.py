"""Stand-alone client of the hosted training service (job CRUD, tensor ops over chunked octet bodies, polling) with an
nn.Module-like engine facade and the ``dss-neutrino`` command line, plus engine-shaped handles on a job server reached
directly over HTTP.  It shares the wire codec with the platform package but needs no GPU and no torch.distributed.
Counterpart of cortex-client/dss_client in the reference."""
__version__ = "0.1.0"

from .batch_spec import (BatchSpecError, build_forward_backward_kwargs, build_forward_backward_payload,  # noqa: F401
                         serialize_forward_backward_args)
from .engines import (ArcticInferenceClient, ArcticInferenceEngine, DSSClient, DSSTrainingClient,  # noqa: F401
                      DSSTrainingEngine)
from .neutrino_client import (ChunkGroupConflictError, ChunkGroupError, ChunkGroupRestartError, InferenceConfig,  # noqa: F401
                              JobType, NeutrinoClient, NeutrinoError, NeutrinoTrainingEngine, SubJobConfig,
                              TrainingConfig)
