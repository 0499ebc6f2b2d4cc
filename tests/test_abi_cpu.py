"""CPU tests of the boundary: the shared library loads without a GPU and exports every
symbol the public header declares; config structs have the reference's layout; the
reference's own drivers were linked against the library when a checkout was available."""
import ctypes as C
import os
import re
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "b200_moe_dsa.h")).read()
    return sorted(set(re.findall(r"B200_API\s+[\w\s\*]+?\b(b200_\w+)\s*\(", text)))


def test_header_symbols_are_exported(b200):
    declared = _declared_symbols()
    assert len(declared) >= 30
    L = b200.lib()
    missing = [s for s in declared if not hasattr(L, s)]
    assert not missing, missing
    assert sorted(b200.EXPORTED_SYMBOLS) == declared
    # the test hooks are exported too, but are not part of the public header
    hooks = open(os.path.join(ROOT, "llm-sys-project_b200", "csrc", "selftest.h")).read()
    for s in b200.TEST_ONLY_SYMBOLS:
        assert hasattr(L, s) and s in hooks and s not in declared


def test_reference_cxx_symbols_are_exported(b200):
    """The C++ shims carry the reference's names (kernels/moe/naive_moe.cuh:27-76, kernels/dsa/naive_dsa.cuh:31-87)."""
    out = subprocess.run(["nm", "-D", "--defined-only", "-C", b200.LIB_PATH], capture_output=True, text=True).stdout
    for name in ("moe_forward(float const*, float const*, float const*, float const*, float*, MoeConfig const&, CUstream_st*)",
                 "moe_gate(", "moe_gather(", "naive_gemm(", "swiglu(", "moe_scatter(",
                 "dsa_forward(float const*, float const*, float const*, float const*, float const*, int const*, float*, DsaConfig const&, CUstream_st*)",
                 "dsa_kv_gather(", "dsa_dot_compressed(", "dsa_dot_positional(", "dsa_dot_fused(", "dsa_softmax(",
                 "dsa_output_proj("):
        assert name in out, name


def test_config_struct_layouts(b200):
    assert C.sizeof(b200.MoeConfig) == 20 and C.sizeof(b200.DsaConfig) == 28
    c = b200.MoeConfig(32, 8, 2, 128, 256)                    # positional, as the reference's drivers do
    assert (c.num_tokens, c.num_experts, c.top_k, c.hidden_dim, c.intermediate_dim) == (32, 8, 2, 128, 256)
    d = b200.DsaConfig(4, 16, 512, 64, 256, 64, 4096)
    assert (d.num_selected_kv, d.page_size, d.total_kv_tokens) == (256, 64, 4096)
    assert b200.MoEConfig is b200.MoeConfig and b200.DSAConfig is b200.DsaConfig
    assert C.sizeof(b200.MoeFp8Config) == 40
    assert b200.MoeFp8Config(1, 2, 3, 4, 5, 1, 1, 1, 2.5).flags == 0          # trailing flags default to 0


def test_status_strings_and_argument_checks_without_gpu(b200):
    L = b200.lib()
    assert L.b200_status_string(0) == b"ok" and b"timed out" in L.b200_status_string(4)
    # argument validation happens before any CUDA call
    assert L.b200_quant_act_1x128(None, None, None, C.c_longlong(4), 128, None) == b200.B200_BAD_ARG
    cfg = b200.MoeConfig(4, 4, 2, 64, 128)
    assert L.b200_moe_forward_f32(None, None, None, None, None, None, C.byref(cfg), None) == b200.B200_BAD_ARG
    assert b200.launch_count() == 0


def test_synthetic_generator_host_twin(b200):
    a = b200.synth_normal_host(42, 0, 1 << 16, 1.0)
    b = b200.synth_normal_host(42, 1000, 16, 1.0)
    assert np.array_equal(a[1000:1016], b)                      # counter-based: value depends on (seed, i) only
    assert abs(a.mean()) < 0.02 and abs(a.std() - 1.0) < 0.02
    assert not np.array_equal(a[:16], b200.synth_normal_host(43, 0, 16, 1.0))


def test_reference_drivers_linked_when_checkout_present():
    import oracle
    drv = os.path.join(ROOT, "oracle", "_ref", "drivers")
    if oracle.reference_dir() is None:
        return
    for exe in ("test_moe", "test_dsa", "bench_moe", "bench_dsa"):
        assert os.access(os.path.join(drv, exe), os.X_OK), f"{exe}: run python llm-sys-project_b200/build.py"
