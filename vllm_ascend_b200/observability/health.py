"""Read-only GPU health probe through NVML (never changes a device setting).

The reference shells out to the vendor's SMI tool from ``check_health``
(vllm_ascend/worker/worker.py:1083-1106); NVML gives the same facts in-process."""
from __future__ import annotations

from typing import Callable, Optional

_nvml_factory: Optional[Callable] = None     # tests install a fake NVML module here


def set_nvml_for_testing(factory: Optional[Callable]) -> None:
    global _nvml_factory
    _nvml_factory = factory


def _nvml():
    if _nvml_factory is not None:
        return _nvml_factory()
    import pynvml
    return pynvml


def gpu_health(index: int = 0) -> dict:
    """{'ok': bool, 'reason': str, 'temperature_c', 'power_w', 'sm_mhz', 'throttle': [...],
    'ecc_uncorrected'} for one GPU; 'ok' is False when NVML cannot reach the GPU or it
    reports uncorrected ECC errors."""
    out = {"ok": True, "reason": "", "throttle": []}
    try:
        nv = _nvml()
        nv.nvmlInit()
    except Exception as e:
        return {"ok": True, "reason": f"nvml unavailable: {e}", "throttle": []}
    try:
        h = nv.nvmlDeviceGetHandleByIndex(index)
        try:
            out["temperature_c"] = int(nv.nvmlDeviceGetTemperature(h, nv.NVML_TEMPERATURE_GPU))
            out["power_w"] = nv.nvmlDeviceGetPowerUsage(h) / 1000.0
            out["sm_mhz"] = int(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
        except Exception:
            pass
        try:
            reasons = int(nv.nvmlDeviceGetCurrentClocksEventReasons(h))
            names = {"hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40,
                     "hw_power_brake": 0x80, "sw_power_cap": 0x4}
            out["throttle"] = [n for n, bit in names.items() if reasons & bit]
        except Exception:
            pass
        try:
            ecc = int(nv.nvmlDeviceGetTotalEccErrors(h, nv.NVML_MEMORY_ERROR_TYPE_UNCORRECTED,
                                                     nv.NVML_VOLATILE_ECC))
            out["ecc_uncorrected"] = ecc
            if ecc > 0:
                out["ok"], out["reason"] = False, f"{ecc} uncorrected ECC errors"
        except Exception:
            pass
    except Exception as e:
        out["ok"], out["reason"] = False, f"GPU {index} not reachable through NVML: {e}"
    finally:
        try:
            nv.nvmlShutdown()
        except Exception:
            pass
    return out
