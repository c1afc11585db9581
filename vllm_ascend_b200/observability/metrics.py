"""Engine metrics: one flat dict for logs, plus a Prometheus exposition when
``prometheus_client`` is importable.  Covers the counters the reference adds on top of the
host framework's (KV-transfer, EPLB, recompute counts: vllm_ascend/core/recompute_scheduler.py,
eplb/eplb_updator.py) and the basics a standalone engine must report itself."""
from __future__ import annotations

from typing import Optional


def collect(engine) -> dict:
    r, s = engine.runner, engine.scheduler
    st = r.stats
    pool = s.pool
    m = {
        "steps": st.get("steps", 0),
        "graph_replays": st.get("graph_replays", 0),
        "eager_steps": st.get("eager_steps", 0),
        "kernel_launches": r.total_launches(),
        "h2d_bytes": st.get("h2d_bytes", 0),
        "d2h_bytes": st.get("d2h_bytes", 0),
        "num_running": len(s.running),
        "num_waiting": len(s.waiting),
        "kv_blocks_total": pool.num_blocks,
        "kv_blocks_free": pool.num_free_blocks,
        "kv_usage": 1.0 - pool.num_free_blocks / max(1, pool.num_blocks),
        "prefix_cache_queries": getattr(pool, "num_queries", 0),
        "prefix_cache_hits": getattr(pool, "num_hits", 0),
        "num_preemptions": getattr(s, "num_preemptions", 0),
        "num_recomputes": getattr(s, "num_recomputes", 0),
        "host_schedule_s": engine.host_times["schedule"],
        "host_execute_s": engine.host_times["execute"],
        "host_update_s": engine.host_times["update"],
        "sleep_level": engine.sleep_level,
    }
    c = engine.kv_connector
    if c is not None and hasattr(c, "stats"):
        for k, v in c.stats.items():
            m[f"kv_transfer_{k}"] = v
    eplb = getattr(engine, "eplb", None)
    if eplb is not None:
        m.update({f"eplb_{k}": v for k, v in eplb.stats.items()})
    spec = getattr(r, "spec_stats", None)
    if spec:
        m.update({f"spec_{k}": v for k, v in spec.items()})
    return m


class PrometheusExporter:
    """Gauges named ``vllm_b200_<metric>``; ``update(engine)`` refreshes them."""

    def __init__(self, registry=None, labels: Optional[dict] = None):
        from prometheus_client import CollectorRegistry, Gauge
        self.registry = registry or CollectorRegistry()
        self._Gauge = Gauge
        self.labels = labels or {}
        self.gauges: dict = {}

    def update(self, engine) -> None:
        for k, v in collect(engine).items():
            if not isinstance(v, (int, float)):
                continue
            g = self.gauges.get(k)
            if g is None:
                g = self._Gauge(f"vllm_b200_{k}", k, list(self.labels), registry=self.registry)
                self.gauges[k] = g
            (g.labels(**self.labels) if self.labels else g).set(v)

    def exposition(self) -> bytes:
        from prometheus_client import generate_latest
        return generate_latest(self.registry)
