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
    assert lib.tpw_jensenshannon_forward(7, None, None, None, 1, 1, 1, 1, 0.5, 0, None) == 1
    assert b"dtype" in lib.tpw_last_error()
    assert lib.tpw_jensenshannon_forward(0, None, None, None, 1, 1, 1, 1, 0.5, 2, None) == 1
    assert b"take_sqrt" in lib.tpw_last_error()
    assert lib.tpw_jensenshannon_backward(0, None, None, None, None, None, None, 1, 2, 2, 2, 0.5, None) == 1
    assert lib.tpw_haversine_forward(0, None, None, None, 1, 3, 3, None) == 1
    assert b"NULL" in lib.tpw_last_error()
    assert lib.tpw_haversine_backward(0, None, None, None, None, None, 1, -3, 3, None) == 1
    assert lib.tpw_haversine_forward(0, None, None, None, 1, 0, 3, None) == 0
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


def test_stand_alone_schemas_equal_the_reference_strings():
    """Every schema the host layer defines on its own, overloads included, reads exactly like the one the
    reference registers (the reference library is loaded in a separate process; nothing is executed)."""
    import json, subprocess, sys
    ref = ROOT / "oracle" / "_ref" / "torchpairwise_ref.so"
    if not ref.exists():
        import pytest
        pytest.skip("oracle/_ref is not built on this machine")
    dump = ("s = {str(x.name) + '.' + str(x.overload_name): str(x) for x in torch._C._jit_get_all_schemas()"
            " if x.name.startswith('torchpairwise::')}\nimport json; print('SCHEMAS' + json.dumps(s))\n")
    outs = []
    for head in (f"import torch\ntorch.ops.load_library({str(ref)!r})\n",
                 "import torch, torchpairwise_b200 as t\nt.load_torch_ops()\n"):
        r = subprocess.run([sys.executable, "-c", head + dump], cwd=str(ROOT), capture_output=True, text=True, timeout=300)
        assert r.returncode == 0, r.stdout + r.stderr
        outs.append(json.loads(r.stdout.split("SCHEMAS", 1)[1]))
    theirs, ours = outs
    assert len(ours) >= 74, len(ours)
    for key, text in ours.items():
        assert theirs.get(key) == text, (key, text, theirs.get(key))
    for name in ("prf_div.", "prf_div.Scalar", "prf_ldiv.rScalar", "prf_div_.", "prf_ldiv_.Scalar", "_prf_div_backward.rScalar",
                 "_prf_ldiv__backward.Scalar", "__directed_hausdorff_backward.", "_directed_hausdorff.", "cdist.", "pdist.",
                 "k_neighbors_mask.", "radius_neighbors_mask.", "linear_kernel.", "polynomial_kernel.", "sigmoid_kernel.", "rbf_kernel.",
                 "laplacian_kernel.", "mahalanobis_distances.", "_sqmahalanobis.", "__sqmahalanobis_backward.", "_cuda_version.",
                 "_cuda_arch_flags."):
        assert "torchpairwise::" + name in ours, name


def test_host_layer_loads_next_to_the_reference_library():
    """Loaded after the reference's CPU build, every kernel registered here has the C++ signature the reference
    registered for the same schema (a mismatch aborts the process at load time)."""
    import subprocess, sys
    ref = ROOT / "oracle" / "_ref" / "torchpairwise_ref.so"
    if not ref.exists():
        pytest.skip("oracle/_ref is not built on this machine")
    code = (f"import torch\ntorch.ops.load_library({str(ref)!r})\nimport torchpairwise_b200 as t\nt.load_torch_ops()\n"
            "tab = torch._C._dispatch_dump_table('torchpairwise::prf_div_')\n"
            "assert 'AutogradCUDA' in tab and 'tpw_torch.cpp' in tab and 'CPU' in tab\nprint('ok')\n")
    r = subprocess.run([sys.executable, "-c", code], cwd=str(ROOT), capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "ok" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


def test_host_layer_error_messages_format_numbers():
    """The argument checks run before anything touches a device, so the kernels registered for CUDA tensors can
    be entered with CPU tensors through an explicit dispatch key: the messages must come back as exceptions
    (a privately linked copy of the C++ stream classes once crashed the process here)."""
    import subprocess, sys
    code = (
        "import torch, torchpairwise_b200 as t\nt.load_torch_ops()\n"
        "ks = torch._C.DispatchKeySet(torch._C.DispatchKey.AutogradCUDA)\n"
        "T = torch.ops.torchpairwise\n"
        "for op, args, text in ((T.euclidean_distances.default, (torch.zeros(6, 50), torch.zeros(3, 40)), 'x1.size(1)=50, x2.size(1)=40'),\n"
        "                       (T.prf_div.default, (torch.zeros(6, 50), torch.zeros(3, 50), 'zero'), 'self.shape=[6, 50], while other.shape=[3, 50]'),\n"
        "                       (T.prf_div.default, (torch.zeros(2), torch.zeros(2), 'nope'), 'mode must be either zero or identity. Got nope'),\n"
        "                       (T.manhattan_distances.default, (torch.zeros(2, 3), torch.zeros(2, 3)), 'CUDA tensors only')):\n"
        "    try:\n        op.redispatch(ks, *args)\n        raise SystemExit('no error from ' + str(op))\n"
        "    except RuntimeError as e:\n        assert text in str(e), str(e)\n"
        "print('ok')\n"
    )
    r = subprocess.run([sys.executable, "-c", code], cwd=str(ROOT), capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "ok" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
