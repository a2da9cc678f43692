"""The C-ABI library loads and exports every function its header declares."""

import ctypes
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def declared_functions():
    text = (ROOT / "include" / "bmoe_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(bmoe_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_documented_surface():
    names = declared_functions()
    for must in ("bmoe_plan_create", "bmoe_plan_initialize", "bmoe_plan_run", "bmoe_plan_destroy",
                 "bmoe_worklist_build", "bmoe_probe_launch", "bmoe_status_string",
                 "bmoe_generate_workload", "bmoe_host_simulate", "bmoe_select_variant"):
        assert must in names


def test_library_exports_every_declared_symbol(engine):
    lib = engine._capi.load()
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} declared in bmoe_b200.h but not exported"
    assert set(declared_functions()) == set(engine._capi.SIGNATURES)


def test_status_strings_match_reference_table(engine):
    # baselines/cutlass/cutlass_baseline.cu:165-176
    want = ["success", "invalid argument", "unsupported data type", "unsupported scheduler",
            "unsupported device", "CUDA error", "CUTLASS error"]
    for code, text in enumerate(want):
        assert engine._capi.status_string(code) == text
    assert engine._capi.status_string(99) == "unknown status"
    assert engine._capi.load().bmoe_probe_scheduler_name(0) == b"static_persistent_round_robin"
    assert engine._capi.load().bmoe_probe_scheduler_name(1) == b"dynamic_global_queue"


def test_struct_sizes_match_the_header(engine):
    cap = engine._capi
    assert ctypes.sizeof(cap.Tile) == 20
    assert ctypes.sizeof(cap.WorklistTotals) == 32
    assert ctypes.sizeof(cap.WorkloadConfig) == 56
    assert ctypes.sizeof(cap.DeviceReport) == 32


def test_plan_rejects_bad_arguments_without_a_gpu(engine):
    """Argument validation happens before any CUDA call (reference order:
    baselines/cutlass/cutlass_baseline.cu:206-216)."""
    cap = engine._capi
    plan = engine.GroupedGemmPlan()
    try:
        ok_ptr = [256, 0, 512]
        counts = [4, 0, 8]
        assert plan.initialize([], [], [], [], 32, 32) == cap.INVALID_ARGUMENT
        assert plan.initialize(ok_ptr, ok_ptr, ok_ptr, counts, 30, 32) == cap.INVALID_ARGUMENT
        assert plan.initialize(ok_ptr, ok_ptr, ok_ptr, counts, 32, 20) == cap.INVALID_ARGUMENT
        assert plan.initialize(ok_ptr, ok_ptr, ok_ptr, counts, 0, 32) == cap.INVALID_ARGUMENT
        assert plan.initialize(ok_ptr, ok_ptr, ok_ptr, counts, 32, 32,
                               data_type=2) == cap.UNSUPPORTED_DATA_TYPE
        # FP8 E4M3 (type 1, an engine extension): rows of k bytes need k % 16 == 0
        assert plan.initialize(ok_ptr, ok_ptr, ok_ptr, counts, 32, 24,
                               data_type=1) == cap.INVALID_ARGUMENT
        assert plan.initialize(ok_ptr, ok_ptr, ok_ptr, counts, 32, 32,
                               scheduler=17) == cap.UNSUPPORTED_SCHEDULER
        assert plan.run() == cap.INVALID_ARGUMENT  # never initialised successfully
    finally:
        plan.close()
