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
