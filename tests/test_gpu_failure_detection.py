"""Failure detection on the device, without faulting anything: a wait that nothing satisfies.

Every in-kernel wait (mbarrier, peer flag) has a budget; when it runs out the kernel records
B200_TIMEOUT, its roles leave their loops, TMEM is released and the kernel returns.  Here the
budget is set to about a millisecond and kernels are given a flag that no one will ever set (a
control block in this GPU's own memory that claims a second rank).  Checked: the kernels return
promptly, the status reaches the host, ``_native.check_status`` raises, the engine reports the
failed step, and the context keeps working (the following GEMM / generation is correct).

The reference's device-side waits spin without bound
(csrc/mc2/dispatch_ffn_combine/op_kernel/utils/hccl_shmem.hpp:243-300); its failure handling is
host side (vllm_ascend/worker/worker.py check_health)."""
import ctypes
import time

import numpy as np
import pytest
import torch

from vllm_ascend_b200 import _native, ops

pytestmark = pytest.mark.gpu
DEV = "cuda"

# CommCtl layout (csrc/comm.cuh): three arrays of 16 epochs, then scalars
AG_FLAG, RS_FLAG, AG_EPOCH, STATUS = 0, 16, 48, 53
SHORT_BUDGET = 3_000_000          # SM cycles: 1.5 to 2.5 ms


@pytest.fixture
def short_waits():
    lib = _native.lib()
    _native.register_signature("b200_set_wait_budget_cycles", [ctypes.c_longlong])
    torch.cuda.synchronize()
    assert lib.b200_set_wait_budget_cycles(SHORT_BUDGET) == 0
    yield lib
    torch.cuda.synchronize()
    assert lib.b200_set_wait_budget_cycles(0) == 0       # default again
    st = _native.status_word(torch.device(DEV))
    st.zero_()
    torch.cuda.synchronize()


def _fake_ctl():
    """A control block that expects a push from rank 1 for epoch 1; nobody will write it."""
    import vllm_ascend_b200.parallel.symm_mem  # noqa: F401  (registers the signatures)
    n = _native.lib().b200_comm_ctl_bytes() // 4
    ctl = torch.zeros(n, dtype=torch.int32, device=DEV)
    ctl[AG_EPOCH] = 1
    return ctl


def test_flag_wait_gives_up_and_reports_timeout(short_waits):
    lib = short_waits
    ctl = _fake_ctl()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    assert lib.b200_ag_wait(ctl.data_ptr(), 0, 2, _native.stream_ptr()) == 0
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 1.0              # the default budget is seconds
    assert int(ctl[STATUS]) == 1                       # B200_TIMEOUT
    out = ctypes.c_int(0)
    assert lib.b200_comm_read_status(ctl.data_ptr(), ctypes.byref(out), _native.stream_ptr()) == 0
    assert out.value == 1


def test_gemm_producer_wait_runs_out_kernel_returns_and_context_survives(short_waits):
    lib = short_waits
    dev = torch.device(DEV)
    ctl = _fake_ctl()
    M, N, K = 256, 256, 512
    g = torch.Generator(device="cpu").manual_seed(0)
    a = (torch.randn(M, K, generator=g) * 0.1).bfloat16().to(dev)
    w = (torch.randn(N, K, generator=g) * 0.1).bfloat16().to(dev)
    c = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
    status = _native.status_word(dev)
    status.zero_()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    # all-gather -> GEMM whose rows 128..255 "come from rank 1": their flag never reaches epoch 1
    rc = lib.b200_gemm_ag_bf16(a.data_ptr(), w.data_ptr(), c.data_ptr(), None, M, N, K, K, K, N, ctl.data_ptr(),
                               0, 2, 128, 0, status.data_ptr(), _native.stream_ptr())
    assert rc == 0
    torch.cuda.synchronize()                            # returns: the wait gave up, no hang, no fault
    assert time.perf_counter() - t0 < 2.0
    with pytest.raises(_native.NativeError, match="TIMEOUT"):
        _native.check_status(dev)
    _native.check_status(dev)                           # reading the status cleared it
    # the same wait in the paired-CTA kernel
    rc = lib.b200_gemm_ag_bf16_2cta(a.data_ptr(), w.data_ptr(), c.data_ptr(), None, M, N, K, K, K, N, ctl.data_ptr(),
                                    0, 2, 128, 0, status.data_ptr(), _native.stream_ptr())
    assert rc == 0
    torch.cuda.synchronize()
    with pytest.raises(_native.NativeError, match="TIMEOUT"):
        _native.check_status(dev)
    # the context is intact: an ordinary GEMM on the same stream is correct
    got = ops.linear(a, w).float()
    want = a.float() @ w.float().t()
    assert float((got - want).abs().max() / want.abs().max()) < 2e-2


def test_engine_reports_the_failed_step_and_serves_the_next_one(short_waits):
    from test_gpu_engine import _cfg
    from vllm_ascend_b200.engine.llm import LLM
    from vllm_ascend_b200.engine.request import SamplingParams
    lib = short_waits
    dev = torch.device(DEV)
    llm = LLM(_cfg("bfloat16"), device="cuda", max_model_len=256, max_num_seqs=4, max_num_batched_tokens=128,
              num_gpu_blocks_override=16, cudagraph_capture_sizes=[2, 4])
    rng = np.random.default_rng(1)
    prompts = [rng.integers(0, 2048, size=40).tolist() for _ in range(2)]
    sp = SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True)
    first = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    # a kernel of the step times out (here: a flag wait on a rank that does not exist)
    ctl = _fake_ctl()
    a = torch.zeros(256, 512, dtype=torch.bfloat16, device=dev)
    w = torch.zeros(256, 512, dtype=torch.bfloat16, device=dev)
    c = torch.zeros(256, 256, dtype=torch.bfloat16, device=dev)
    assert lib.b200_gemm_ag_bf16(a.data_ptr(), w.data_ptr(), c.data_ptr(), None, 256, 256, 512, 512, 512, 256,
                                 ctl.data_ptr(), 0, 2, 128, 0, _native.status_word(dev).data_ptr(),
                                 _native.stream_ptr()) == 0
    with pytest.raises(_native.NativeError, match="TIMEOUT"):
        llm.generate(prompts, sp)                       # the engine surfaces the device status after the step
    again = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    assert again == first
