"""The C-ABI library loads without a GPU and exports every symbol include/paella_b200.h declares."""
import os
import re

from paella_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "paella_b200.h")).read()
    return sorted(set(re.findall(r"PB_API\s+[^;(]*?\b(pb_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound():
    L = capi.load()
    names = _declared()
    assert len(names) >= 50
    for n in names:
        assert hasattr(L, n), f"{n} declared in the header but not exported"
        assert n in capi.SIGNATURES, f"{n} has no ctypes signature"
    assert sorted(capi.SIGNATURES) == names


def test_struct_sizes_match_the_header():
    import ctypes as C
    assert C.sizeof(capi.LaunchInfo) == 48
    assert C.sizeof(capi.OpParams) == 20 * 4 + 7 * 8 + 4 * 4
    assert C.sizeof(capi.ReplayEvent) == 24
    assert C.sizeof(capi.ReplayDecision) == 40
    L = capi.load()
    assert L.pb_notifier_size() == 32
    assert L.pb_version().startswith(b"paella_b200")


def test_plugins_export_init_job_and_load_without_cuda_context():
    """Clients dlopen a plugin only to read its I/O sizes (src/client/client.cpp:64-76)."""
    import ctypes as C
    capi.load()
    for job in ["tvm_mnist", "tvm_resnet18", "tvm_resnet34", "tvm_resnet50", "tvm_mobilenet", "tvm_inception_v3", "tvm_squeezenet1_1", "tvm_googlenet", "tvm_densenet121", "tvm_arcfaceresnet100", "tvm_ultraface320", "vec_add",
                "dummy_short", "dummy_long"]:
        lib = C.CDLL(capi.plugin_path(job))
        assert hasattr(lib, "init_job")
        lib.init_job.restype = C.c_void_p
        assert lib.init_job()


def test_errors_are_reported_not_fatal():
    import ctypes as C
    L = capi.load()
    m = C.c_void_p()
    rc = L.pb_model_load(b"/nonexistent/pack.bin", 0, -1, C.byref(m))
    assert rc == -4 and b"cannot open" in L.pb_last_error()
