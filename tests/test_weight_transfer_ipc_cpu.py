"""Packed same-node weight transfer between two processes (host shared memory stands in for CUDA IPC)."""
import multiprocessing as mp

import torch


def _trainer(conn, bucket_bytes):
    import torch.multiprocessing as tmp
    tmp.set_sharing_strategy("file_system")
    from vllm_ascend_b200.distributed.weight_transfer.engines import PackedIPCSender
    g = torch.Generator().manual_seed(0)
    weights = {f"layer{i}.w": torch.randn(37 + i, 19, generator=g).to(torch.bfloat16 if i % 2 else torch.float32)
               for i in range(9)}
    weights["big"] = torch.randn(4096, 8, generator=g)              # larger than a bucket: travels alone
    weights["empty"] = torch.zeros(0, 4)
    sender = PackedIPCSender(bucket_bytes=bucket_bytes, device="cpu", num_buffers=2)
    for update in range(2):
        scaled = {k: v * (update + 1) for k, v in weights.items()}
        n = sender.send(scaled.items(), conn.send_bytes, lambda: int.from_bytes(conn.recv_bytes(), "little"))
        conn.send_bytes(b"DONE" + n.to_bytes(4, "little"))
    conn.recv_bytes()               # keep the buffers alive until the worker has finished
    conn.close()


def test_packed_ipc_transfer_between_processes():
    import torch.multiprocessing as tmp
    tmp.set_sharing_strategy("file_system")
    from vllm_ascend_b200.distributed.weight_transfer.engines import IPCWeightTransferEngine
    ctx = mp.get_context("spawn")
    a, b = ctx.Pipe()
    p = ctx.Process(target=_trainer, args=(b, 16 << 10))
    p.start()
    try:
        for update in range(2):
            got, buckets = {}, 0

            def apply(items):
                n = 0
                for name, t in items:
                    got[name] = t.clone()
                    n += 1
                return n
            while True:
                msg = a.recv_bytes()
                if msg[:4] == b"DONE":
                    assert int.from_bytes(msg[4:], "little") == buckets
                    break
                n, index, last = IPCWeightTransferEngine.apply_packed(msg, apply)
                buckets += 1
                a.send_bytes(index.to_bytes(4, "little"))
            g = torch.Generator().manual_seed(0)
            want = {f"layer{i}.w": torch.randn(37 + i, 19, generator=g).to(torch.bfloat16 if i % 2 else torch.float32)
                    for i in range(9)}
            want["big"] = torch.randn(4096, 8, generator=g)
            want["empty"] = torch.zeros(0, 4)
            assert set(got) == set(want) and buckets >= 3
            for k, v in want.items():
                assert got[k].dtype == v.dtype and torch.equal(got[k], v * (update + 1)), k
        a.send_bytes(b"bye")
    finally:
        p.join(timeout=60)
        if p.is_alive():
            p.terminate()
    assert p.exitcode == 0
