"""The C-ABI library: builds, loads, and exports every symbol the header
declares.  No compute calls here (no GPU needed)."""
import ctypes
import os
import re

from conftest import REPO, load_binding


def declared_functions():
    text = open(os.path.join(REPO, "include", "sd3_b200.h")).read()
    return sorted(set(re.findall(r"SD3_API\s+[A-Za-z_ \*]+?\b(sd3_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_functions():
    names = declared_functions()
    assert len(names) >= 20
    for must in ("sd3_dit_forward", "sd3_block_forward", "sd3_linear", "sd3_attention",
                 "sd3_layernorm_modulate", "sd3_last_error"):
        assert must in names


def test_library_exports_every_declared_symbol():
    s = load_binding()
    assert os.path.exists(s.LIB_PATH), "run python sd3.c_b200/build.py"
    lib = ctypes.CDLL(s.LIB_PATH)
    for name in declared_functions():
        assert hasattr(lib, name), name


def test_binding_covers_header():
    s = load_binding()
    assert sorted(s.PROTOTYPES) == declared_functions()
    assert s.lib().sd3_abi_version() == 1


def test_host_side_argument_errors_need_no_gpu():
    s = load_binding()
    lib = s.lib()
    # invalid arguments are rejected before any CUDA call
    assert lib.sd3_linear(None, None, None, None, 7, 1, 1, 1, 0, None) == -1
    assert b"sd3_linear" in lib.sd3_last_error()
    assert lib.sd3_model_create(None, None) == -1
    cfg = s.Config(0, 0, 8, 8, 16, 64, 1, 4, 2, 16, 16, 1, 1, 0, 0)
    h = ctypes.c_void_p()
    assert lib.sd3_model_create(ctypes.byref(cfg), ctypes.byref(h)) == -1  # num_layers 0
    assert lib.sd3_cast(None, 0, None, 1, 4, None) == -1


def test_bench_flop_accounting_matches_the_model_shapes():
    """bench.py's STEP_TFLOP (algorithmic work of one config-3 step: 2MNK per GEMM,
    4 T^2 E per attention, nothing else) recomputed from the model's shapes."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("bench_mod", os.path.join(REPO, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    B, Tc, Tx, E, F, L, dual = 8, 333, 4096, 1536, 6144, 24, 13
    T = Tc + Tx
    fl = 0.0
    for l in range(L):
        last = l == L - 1
        rows_c, rows_x = B * Tc, B * Tx
        fl += 2.0 * rows_c * E * 3 * E + 2.0 * rows_x * E * 3 * E            # QKV
        fl += 4.0 * B * T * T * E                                          # joint attention
        fl += 2.0 * rows_x * E * E + (0 if last else 2.0 * rows_c * E * E)  # out-proj
        fl += 2 * 2.0 * rows_x * E * F + (0 if last else 2 * 2.0 * rows_c * E * F)  # MLP
        if l < dual:
            fl += 2.0 * rows_x * E * 3 * E + 4.0 * B * Tx * Tx * E + 2.0 * rows_x * E * E
        chunks = (2 if last else 6) + (9 if l < dual else 6)
        fl += 2.0 * B * E * chunks * E                                     # AdaLN
    fl += 2.0 * B * E * 2 * E                                              # final AdaLN
    fl += 2.0 * B * Tc * 4096 * E + 2.0 * B * Tx * 64 * E                  # caption projection, patch embed
    fl += 2.0 * B * (256 * E + E * E + 2048 * E + E * E)                   # conditioning MLPs
    fl += 2.0 * B * Tx * E * 64                                            # final linear
    assert abs(fl / 1e12 - bench.STEP_TFLOP) < 0.01 * bench.STEP_TFLOP
    assert bench.ATTN_TRAFFIC_BYTES_PER_SAMPLE > 4429 * 4608 * 2           # at least the q|k|v read
