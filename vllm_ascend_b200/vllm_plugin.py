"""Making the plugin entry points visible to an installed vLLM.

vLLM finds plugins through ``importlib.metadata`` entry points of installed distributions
(``pip install -e .`` of this repository declares them, see ``pyproject.toml``).  A source
checkout that is only on ``sys.path`` has no distribution metadata; ``ensure_entry_points()``
writes a minimal ``.dist-info`` directory (METADATA + entry_points.txt, no code) into a private
temporary directory and puts it on ``sys.path`` / ``PYTHONPATH`` so that this process and the
processes vLLM spawns discover the same five entry points.
"""
from __future__ import annotations

import os
import sys
import tempfile

from . import __version__

PLATFORM_PLUGIN = "b200"
GENERAL_PLUGINS = {
    "b200_kv_connector": "vllm_ascend_b200:register_connector",
    "b200_model_loader": "vllm_ascend_b200:register_model_loader",
    "b200_service_profiling": "vllm_ascend_b200:register_service_profiling",
    "b200_model": "vllm_ascend_b200:register_model",
}
ALL_PLUGIN_NAMES = [PLATFORM_PLUGIN, *GENERAL_PLUGINS]


def entry_points_visible() -> bool:
    from importlib.metadata import entry_points
    return any(e.name == PLATFORM_PLUGIN and e.value.startswith("vllm_ascend_b200")
               for e in entry_points(group="vllm.platform_plugins"))


def ensure_entry_points() -> str:
    """Returns the directory that carries the metadata ('' when an installed distribution already
    does)."""
    if entry_points_visible():
        return ""
    root = tempfile.mkdtemp(prefix="vllm_ascend_b200_meta_")
    info = os.path.join(root, f"vllm_ascend_b200-{__version__}.dist-info")
    os.makedirs(info)
    with open(os.path.join(info, "METADATA"), "w") as f:
        f.write(f"Metadata-Version: 2.1\nName: vllm_ascend_b200\nVersion: {__version__}\n")
    with open(os.path.join(info, "entry_points.txt"), "w") as f:
        f.write(f"[vllm.platform_plugins]\n{PLATFORM_PLUGIN} = vllm_ascend_b200:register\n\n[vllm.general_plugins]\n")
        for k, v in GENERAL_PLUGINS.items():
            f.write(f"{k} = {v}\n")
    pkg_parent = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, root)
    parts = [root, pkg_parent] + [p for p in os.environ.get("PYTHONPATH", "").split(os.pathsep) if p]
    os.environ["PYTHONPATH"] = os.pathsep.join(dict.fromkeys(parts))
    import importlib
    importlib.invalidate_caches()
    return root
