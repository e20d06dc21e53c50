"""Stand-alone client of the hosted training service (job CRUD, tensor ops over chunked octet bodies, polling) with an
nn.Module-like engine facade and the ``dss-neutrino`` command line.  It shares the wire codec with the platform
package but needs no GPU and no torch.distributed.  Counterpart of cortex-client/dss_client in the reference."""
from .neutrino_client import (InferenceConfig, JobType, NeutrinoClient, NeutrinoError, NeutrinoTrainingEngine,  # noqa: F401
                              SubJobConfig, TrainingConfig)
