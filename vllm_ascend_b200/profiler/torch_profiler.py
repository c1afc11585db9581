"""Start/stop profiling session behind ``worker.profile()``.

The reference drives the vendor's torch profiler with an experimental config
(vllm_ascend/worker/worker.py:1003-1031, profiler/profiler_config.py); here it is
``torch.profiler`` with CUDA activity, writing one Chrome trace per rank."""
from __future__ import annotations

import os
import time

import torch


class TorchProfilerSession:
    def __init__(self, out_dir: str, rank: int = 0, with_stack: bool = False, record_shapes: bool = False):
        self.out_dir, self.rank = out_dir, rank
        acts = [torch.profiler.ProfilerActivity.CPU]
        if torch.cuda.is_available():
            acts.append(torch.profiler.ProfilerActivity.CUDA)
        self.prof = torch.profiler.profile(activities=acts, with_stack=with_stack, record_shapes=record_shapes)

    def start(self) -> None:
        self.prof.start()

    def stop(self) -> str:
        self.prof.stop()
        os.makedirs(self.out_dir, exist_ok=True)
        path = os.path.join(self.out_dir, f"trace_rank{self.rank}_{int(time.time())}.json")
        self.prof.export_chrome_trace(path)
        return path

    def key_averages(self):
        return self.prof.key_averages()
