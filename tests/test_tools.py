"""Host-side checks of the development tools that ship with the package (no GPU needed)."""
from __future__ import annotations

import pytest

from helion_b200 import build as hb_build


def test_instrumented_builds_never_replace_the_product_library(tmp_path):
    # a define without an output path, or the product library's own path, is refused before anything is compiled
    with pytest.raises(ValueError, match="own output path"):
        hb_build.build(defines=("HB_SKINNY_TRACE",))
    with pytest.raises(ValueError, match="not built with extra defines"):
        hb_build.build(defines=("HB_SKINNY_TRACE",), output=hb_build.LIB_PATH)


def test_trace_and_sweep_tools_refuse_to_run_without_a_gpu(capsys):
    import torch

    if torch.cuda.is_available():
        pytest.skip("this checks the no-GPU answer")
    from helion_b200 import ceiling, chain_trace, sweep

    assert chain_trace.main([]) == 2
    assert chain_trace.main(["--kernel", "pair", "--m", "1024"]) == 2
    assert sweep.main(["--op", "gemm", "--back-to-back", "20"]) == 2
    assert "CUDA" in capsys.readouterr().err
    assert callable(ceiling.main)


def test_product_library_exports_no_trace_entry(built_library):
    # the phase stamps exist only in builds made with -DHB_SKINNY_TRACE / -DHB_GEMM_TRACE / -DHB_PAIR_TRACE
    for name in ("hb200_debug_skinny_trace", "hb200_debug_gemm_trace", "hb200_debug_pair_trace"):
        assert not hasattr(built_library, name), name


def test_clock_sampler_keeps_the_samples_of_the_timed_region(monkeypatch):
    """bench.py's sampler against a fake NVML: samples carry time stamps, and only those inside the window of the
    timed region are reported; a region shorter than one query falls back to the nearest sample and says so."""
    import sys
    import time
    import types
    from pathlib import Path

    sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
    import bench

    fake = types.SimpleNamespace(
        NVML_CLOCK_SM=0, nvmlInit=lambda: None, nvmlDeviceGetHandleByIndex=lambda i: i,
        nvmlDeviceGetMaxClockInfo=lambda h, c: 1965, nvmlDeviceGetClockInfo=lambda h, c: 1500,
        nvmlDeviceGetPowerUsage=lambda h: 900000, nvmlDeviceGetCurrentClocksEventReasons=lambda h: 0x4,
        nvmlClocksEventReasonSwPowerCap=0x4, nvmlClocksEventReasonHwSlowdown=0x8,
        nvmlClocksEventReasonSwThermalSlowdown=0x20, nvmlClocksEventReasonHwThermalSlowdown=0x40)
    monkeypatch.setitem(sys.modules, "pynvml", fake)
    monkeypatch.delenv("CUDA_VISIBLE_DEVICES", raising=False)
    sampler = bench.ClockSampler(0, period_s=0.0)
    sampler.start()
    time.sleep(0.02)
    t0 = time.perf_counter()
    time.sleep(0.02)
    t1 = time.perf_counter()
    time.sleep(0.01)
    res = sampler.stop(window=(t0, t1))
    assert res["samples"] > 0 and res["sm_mhz"] == 1500 and res["sm_max_mhz"] == 1965
    assert res["reasons"] == ["sw_power_cap"] and abs(res["power_w_max"] - 900.0) < 1e-6
    assert res["samples_taken"].startswith("inside the timed region")
    assert all(t0 <= s[2] <= t1 for s in sampler.samples)
    # a window in which no query fell
    sampler2 = bench.ClockSampler(0, period_s=0.005)
    sampler2.start()
    time.sleep(0.03)
    res2 = sampler2.stop(window=(0.0, 1e-9))
    assert res2["samples"] == 1 and "none fell inside" in res2["samples_taken"]

