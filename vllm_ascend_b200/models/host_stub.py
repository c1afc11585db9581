"""Description-only model class for a host vLLM's registry.

vLLM validates ``architectures`` of a checkpoint against its model registry and reads a few
capability flags from the registered class.  When this package is the active platform the worker
never instantiates that class (it builds the model from ``vllm_ascend_b200.models``), so an
architecture vLLM does not ship only needs an entry that answers those questions."""
from __future__ import annotations

import torch


class HostModelStub(torch.nn.Module):
    is_text_generation_model = True

    def __init__(self, *, vllm_config=None, prefix: str = ""):
        super().__init__()

    def embed_input_ids(self, input_ids: torch.Tensor) -> torch.Tensor:
        raise RuntimeError("the B200 worker runs its own model; this class only describes it")

    def forward(self, input_ids: torch.Tensor, positions: torch.Tensor, intermediate_tensors=None,
                inputs_embeds=None) -> torch.Tensor:
        raise RuntimeError("the B200 worker runs its own model; this class only describes it")

    def compute_logits(self, hidden_states: torch.Tensor) -> torch.Tensor:
        raise RuntimeError("the B200 worker runs its own model; this class only describes it")
