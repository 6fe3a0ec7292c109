"""CPU tests of the drop-in boundary: the shared library loads without a GPU
driver, exports every symbol the public header declares, and its host-side
argument validation behaves like the reference's (no compute calls here)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "cutile_b200.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ctb_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from cutile_b200 import _lib
    names = declared_symbols()
    assert len(names) >= 10
    for n in names:
        assert hasattr(_lib.lib, n), f"{n} declared in the header but not exported"
    assert sorted(_lib.SIGNATURES) == names, "ctypes signatures and header disagree"


def test_header_is_plain_c(tmp_path):
    """The boundary is a C ABI: the header compiles as C99 on its own, without warnings."""
    import subprocess
    src = tmp_path / "use_header.c"
    src.write_text('#include "cutile_b200.h"\nint main(void) { return CTB_OK; }\n')
    r = subprocess.run(["gcc", "-std=c99", "-Wall", "-Wextra", "-pedantic", "-Werror", "-fsyntax-only", "-I",
                        os.path.dirname(HEADER), str(src)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr


def test_version_and_status_strings():
    import cutile_b200
    assert "sm_100a" in cutile_b200.version_info()
    assert cutile_b200._lib.status_string(0) == "OK"
    assert cutile_b200._lib.status_string(7) == "TIMEOUT"


def test_no_cpu_fallback():
    """Without a device the context cannot be created: the product never computes on the host."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from cutile_b200 import _lib
    out = ctypes.c_void_p()
    st = _lib.lib.ctb_create(ctypes.byref(out), 0)
    assert st == _lib.NO_DEVICE and "no CPU path" in _lib.last_error()


def test_null_context_and_host_arrays_rejected():
    import numpy as np
    import cutile_b200
    from cutile_b200 import _lib
    st = _lib.lib.ctb_softmax(None, None, None, None, 4, 1, 4, 4, 0, 4, 0)
    assert st == _lib.BAD_ARG and "null context" in _lib.last_error()
    with pytest.raises(cutile_b200.CtbError) as e:  # host array, like the reference's ArgumentError
        cutile_b200.softmax.softmax_tma_kernel(np.zeros((2, 4), np.float32), np.zeros((2, 4), np.float32), 4)
    assert e.value.status == _lib.BAD_ARG


def test_expert_parallel_entry_points_validate_their_table():
    """The peer-memory MoE entry points reject a missing context, a missing buffer table and out-of-range ranks
    before touching any device (host-side checks only; the compute path is covered by the 2-GPU test)."""
    from cutile_b200 import _lib
    tab = _lib.EpBuffers()
    tab.world, tab.rank = 2, 0
    st = _lib.lib.ctb_moe_ep_dispatch(None, None, ctypes.byref(tab), None, None, None, 8, 64, 8, 2)
    assert st == _lib.BAD_ARG and "null context" in _lib.last_error()
    st = _lib.lib.ctb_moe_ep_barrier(None, None, ctypes.byref(tab))
    assert st == _lib.BAD_ARG
    st = _lib.lib.ctb_moe_ep_experts(None, None, ctypes.byref(tab), None, None, 16, 64, 128, 4, 128, 128, 64)
    assert st == _lib.BAD_ARG
    assert ctypes.sizeof(_lib.EpBuffers) == 8 + 5 * 8 * _lib.EP_MAX_RANKS + 8  # layout of ctb_ep_buffers


def test_multi_gpu_entry_points_fail_on_the_host_side():
    """Bad device lists, missing tables and unknown ops are refused before any device or NCCL call."""
    from cutile_b200 import _lib
    import cutile_b200
    g = ctypes.c_void_p()
    assert _lib.lib.ctb_create_multi(ctypes.byref(g), None, 2) == _lib.BAD_ARG
    two = (ctypes.c_int * 2)(3, 3)
    assert _lib.lib.ctb_create_multi(ctypes.byref(g), two, 2) == _lib.BAD_ARG and "twice" in _lib.last_error()
    nine = (ctypes.c_int * 9)(*range(9))
    assert _lib.lib.ctb_create_multi(ctypes.byref(g), nine, 9) == _lib.BAD_ARG
    assert _lib.lib.ctb_group_size(None) == 0 and not _lib.lib.ctb_group_ctx(None, 0)
    assert _lib.lib.ctb_comm_init_rank(None, None, 0, 2) == _lib.BAD_ARG
    assert _lib.lib.ctb_comm_unique_id(None) == _lib.BAD_ARG
    assert _lib.lib.ctb_fmha_fwd_sharded(None, None, None, None, None, None, 64, 64, 128, 128, 2, 2, None, 0.125, 0, 128,
                                         128, 1, 1, 1) == _lib.BAD_ARG
    assert _lib.lib.ctb_moe_ffn_ep(None, None, None, None, None, None, None, None, 8, 64, 64, 8, 2, 128, 128, 64, 1) \
        == _lib.BAD_ARG
    assert _lib.lib.ctb_ep_connect_local(None, 2) == _lib.BAD_ARG
    # scratch sizing is pure host arithmetic
    wb = cutile_b200.multi.workspace_bytes
    small, big = wb("moe_ffn", 256, 1024, 2048, 32, 2, 128), wb("moe_ffn", 4096, 1024, 2048, 32, 2, 128)
    assert 0 < small < big and big >= 4096 * 2 * (2048 + 1024) * 2
    assert wb("moe_ep", 512, 1024, 2048, 4, 2, 128, 8) >= 8 * 1024 * 2048 * 2
    assert wb("nothing", 1, 2, 3) == 0 and wb("moe_ffn", 1, 2) == 0
    with pytest.raises(cutile_b200.CtbError):
        cutile_b200.multi.Group([0, 0])


def test_launch_hints_follow_the_reference_rules():
    """num_ctas / occupancy / opt_level / num_worker_warps are validated like validate_hint
    (src/language/types.jl:864-882); unknown keywords are refused; sm_arch, name, dependent and stream are accepted."""
    import cutile_b200
    from cutile_b200 import _lib
    from cutile_b200._util import check_hints
    check_hints(dict(num_ctas=2, occupancy=2, opt_level=3, num_worker_warps=8, sm_arch="10.0", dependent=False, name="k"))
    assert _lib.lib.ctb_validate_hints(-1, -1, -1, -1) == _lib.OK
    for bad, word in ((dict(num_ctas=3), "power of 2"), (dict(num_ctas=32), "between 1 and 16"),
                      (dict(occupancy=0), "between 1 and 32"), (dict(opt_level=4), "between 0 and 3"),
                      (dict(num_worker_warps=6), "either 4 or 8"), (dict(whatever=1), "unknown hint key"),
                      (dict(occupancy=2.5), "must be an integer")):
        with pytest.raises(cutile_b200.CtbError) as e:
            check_hints(bad)
        assert e.value.status == _lib.BAD_ARG and word in str(e.value)
