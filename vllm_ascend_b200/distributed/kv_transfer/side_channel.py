"""ZMQ + msgpack side channel between engines of a disaggregated deployment.

One ROUTER socket per (engine, TP rank) at ``base_port + tp_rank`` answers three
requests: ``meta`` (cache geometry + CUDA IPC handle), ``read`` (host-staged block
payload, the cross-node fallback) and ``done`` (the peer finished pulling a request,
its blocks may be freed).  Same role as the handshake/notify threads of
vllm_ascend/distributed/kv_transfer/kv_p2p/mooncake_connector.py:361-571.
"""
from __future__ import annotations

import threading
from typing import Callable

import msgpack
import zmq


class SideChannelError(RuntimeError):
    pass


class SideChannelServer(threading.Thread):
    def __init__(self, host: str, port: int, handler: Callable[[dict], dict]):
        super().__init__(daemon=True, name=f"kv-side-channel-{port}")
        self.handler = handler
        self.ctx = zmq.Context.instance()
        self.sock = self.ctx.socket(zmq.ROUTER)
        self.sock.setsockopt(zmq.LINGER, 0)
        if port == 0:
            self.port = self.sock.bind_to_random_port(f"tcp://{host}")
        else:
            self.sock.bind(f"tcp://{host}:{port}")
            self.port = port
        self._stop_flag = threading.Event()
        self.num_served = 0

    def run(self) -> None:
        poller = zmq.Poller()
        poller.register(self.sock, zmq.POLLIN)
        while not self._stop_flag.is_set():
            if not poller.poll(100):
                continue
            frames = self.sock.recv_multipart()
            ident, payload = frames[0], frames[-1]
            try:
                reply = self.handler(msgpack.unpackb(payload, raw=False))
            except Exception as e:      # the peer gets the reason, the server keeps serving
                reply = {"ok": False, "error": f"{type(e).__name__}: {e}"}
            if reply is None:           # handler chose to drop the message (failure injection)
                continue
            self.num_served += 1
            self.sock.send_multipart([ident, b"", msgpack.packb(reply, use_bin_type=True)])
        self.sock.close()

    def stop(self) -> None:
        self._stop_flag.set()
        if self.is_alive():
            self.join(timeout=2)


def request(host: str, port: int, msg: dict, timeout_ms: int = 5000) -> dict:
    """One request/reply exchange; raises SideChannelError on timeout or a negative reply."""
    ctx = zmq.Context.instance()
    sock = ctx.socket(zmq.REQ)
    sock.setsockopt(zmq.LINGER, 0)
    try:
        sock.connect(f"tcp://{host}:{port}")
        sock.send(msgpack.packb(msg, use_bin_type=True))
        if not sock.poll(timeout_ms):
            raise SideChannelError(f"no reply from {host}:{port} to {msg.get('op')!r} in {timeout_ms} ms")
        reply = msgpack.unpackb(sock.recv(), raw=False)
    finally:
        sock.close()
    if not reply.get("ok", False):
        raise SideChannelError(f"{host}:{port} refused {msg.get('op')!r}: {reply.get('error')}")
    return reply
