"""Communication: host collectives, failure detection, and (on GPUs) the peer-memory
payload exchange and the NCCL baselines."""
from .comm import CommFailure, LocalComm, TorchComm, make_comm  # noqa: F401
from .failure import (FaultInjector, Heartbeat, PayloadError, PeerLost, StepTimeout, check_status,  # noqa: F401
                      validate_payload)
