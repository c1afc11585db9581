from .engines import IPCWeightTransferEngine, NCCLWeightTransferEngine  # noqa: F401
