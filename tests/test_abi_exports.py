"""The C-ABI library loads and exports every entry point that include/tpw_b200.h declares
(no compute calls: this runs without a GPU)."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
HEADER = (ROOT / "include" / "tpw_b200.h").read_text()


def declared_functions():
    return sorted(set(re.findall(r"^TPW_API\s+[\w\s\*]+?\b(tpw_\w+)\s*\(", HEADER, flags=re.M)))


def test_header_declares_the_expected_surface():
    names = declared_functions()
    assert len(names) >= 20
    for must in ("tpw_lp_forward", "tpw_lp_backward", "tpw_bool_metric_forward", "tpw_hausdorff_forward",
                 "tpw_dot_metric_forward", "tpw_prf_div_forward", "tpw_cmp_reduce_forward", "tpw_bitpack"):
        assert must in names


def test_library_exports_every_declared_symbol():
    from torchpairwise_b200 import _abi
    handle = ctypes.CDLL(str(_abi.LIB_PATH))
    for name in declared_functions():
        assert hasattr(handle, name), f"{name} is declared in the header but not exported"
        assert name in _abi.SIGNATURES, f"{name} has no ctypes signature"
    for name in _abi.SIGNATURES:
        assert name in declared_functions(), f"{name} is bound but not declared in the header"


def test_version_and_arch_calls_work_without_a_gpu():
    from torchpairwise_b200 import _abi
    assert _abi.lib.tpw_abi_version() == int(re.search(r"#define TPW_ABI_VERSION (\d+)", HEADER).group(1))
    assert _abi.lib.tpw_cuda_arch_flags() == b"sm_100a"
    assert _abi.lib.tpw_cuda_version() >= 12000


def test_argument_errors_are_reported_before_any_launch():
    from torchpairwise_b200 import _abi
    lib = _abi.lib
    # bad dtype / negative size / NULL pointers: rejected on the host, with a message
    assert lib.tpw_lp_forward(99, None, None, None, None, 1, 1, 1, 1, 2.0, 0.5, None) == 1
    assert b"dtype" in lib.tpw_last_error()
    assert lib.tpw_lp_forward(0, None, None, None, None, 1, -1, 1, 1, 2.0, 0.5, None) == 1
    assert lib.tpw_lp_forward(0, None, None, None, None, 1, 4, 4, 4, 2.0, 0.5, None) == 1
    assert b"NULL" in lib.tpw_last_error()
    assert lib.tpw_bool_metric_forward(77, None, None, None, None, None, 1, 1, 1, 1, 4, None) == 1
    assert lib.tpw_bitpack(None, None, None, 4, 100, 2, None) == 1  # 2 words cannot hold 100 bits
    # empty problems are fine and launch nothing
    assert lib.tpw_lp_forward(0, None, None, None, None, 0, 4, 4, 4, 2.0, 0.5, None) == 0
    assert lib.tpw_last_error() == b""
    with pytest.raises(_abi.TpwError, match="status 1"):
        _abi.check(lib.tpw_prf_div_forward(0, 9, None, None, None, 4, None), "tpw_prf_div_forward")


def test_cpp_host_layer_registers_the_reference_schemas():
    """Stand-alone load on a machine without a GPU: the schemas exist with the reference's
    signatures and CUDA/AutogradCUDA kernels are attached (nothing is executed)."""
    import subprocess, sys
    code = (
        "import torch, torchpairwise_b200 as t\n"
        "t.load_torch_ops()\n"
        "s = {str(x.name): str(x) for x in torch._C._jit_get_all_schemas() if x.name.startswith('torchpairwise::')}\n"
        "assert s['torchpairwise::minkowski_distances'] in ('torchpairwise::minkowski_distances(Tensor x1, Tensor? x2=None, float p=2) -> Tensor', 'torchpairwise::minkowski_distances(Tensor x1, Tensor? x2=None, float p=2.) -> Tensor'), s['torchpairwise::minkowski_distances']\n"
        "assert 'Generator? generator=None' in s['torchpairwise::cdist'] and 'str metric=\\\"minkowski\\\"' in s['torchpairwise::cdist']\n"
        "assert len(s) >= 38, len(s)\n"
        "tab = torch._C._dispatch_dump_table('torchpairwise::euclidean_distances')\n"
        "assert 'AutogradCUDA' in tab and 'tpw_torch.cpp' in tab\n"
        "tab = torch._C._dispatch_dump_table('torchpairwise::pwxor_sum')\n"
        "assert 'CUDA' in tab\n"
        "print('ok')\n"
    )
    r = subprocess.run([sys.executable, "-c", code], cwd=str(ROOT), capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "ok" in r.stdout, r.stdout + r.stderr
