"""Profiling hooks: torch profiler wrapper, service profiling hook points, NVTX ranges."""
class nvtx_range:
    """``with nvtx_range("name"):`` marks a range for Nsight-style timelines when VLLM_B200_NVTX is
    set and a CUDA device is present; otherwise it costs one attribute read.  The hook points are the
    ones the reference annotates for its profilers (execute_model, input preparation, per layer)."""
    __slots__ = ("name", "on")

    def __init__(self, name: str, level: int = 1):
        from .. import envs
        self.name = name
        self.on = envs.VLLM_B200_NVTX >= level

    def __enter__(self):
        if self.on:
            import torch
            if torch.cuda.is_available():
                torch.cuda.nvtx.range_push(self.name)
            else:
                self.on = False
        return self

    def __exit__(self, *exc):
        if self.on:
            import torch
            torch.cuda.nvtx.range_pop()
        return False
