"""The C ABI: struct layouts against the layout facts printed by the reference's own header and runtime
(tests/golden/abi_layout.json, produced by oracle/abi_probe.cc compiled against the reference), and the exported
symbols of libcinn_b200.so against the declarations in include/*.h.  No GPU needed."""
import ctypes
import json
import os
import re
import subprocess

import pytest

import cinn_b200
from cinn_b200 import runtime as rt

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = json.load(open(os.path.join(ROOT, "tests", "golden", "abi_layout.json")))


def test_python_mirror_matches_reference_layout():
    assert ctypes.sizeof(rt.cinn_type_t) == GOLDEN["sizeof_cinn_type_t"]
    assert ctypes.sizeof(rt.cinn_buffer_t) == GOLDEN["sizeof_cinn_buffer_t"]
    assert ctypes.sizeof(rt.cinn_pod_value_t) == GOLDEN["sizeof_cinn_pod_value_t"]
    for field, off in GOLDEN["buffer_offsets"].items():
        assert getattr(rt.cinn_buffer_t, field).offset == off, field
    for field, off in GOLDEN["type_offsets"].items():
        assert getattr(rt.cinn_type_t, field).offset == off, field
    assert rt.cinn_pod_value_t.value_.offset == 8
    assert rt.CINN_BUFFER_MAX_DIMS == GOLDEN["buffer_max_dims"]
    assert rt.BUFFER_ON_DEVICE == GOLDEN["buffer_kind"]["on_device"]
    for name, (code, bits) in GOLDEN["types"].items():
        assert rt.DTYPES[name][0] == code and rt.DTYPES[name][1] == bits, name
    assert rt.POD_BUFFERP == GOLDEN["pods"]["buffer"]["type_code"]
    assert rt.POD_INT32 == GOLDEN["pods"]["int32_minus7"]["type_code"]
    assert rt.POD_INT64 == GOLDEN["pods"]["int64_big"]["type_code"]
    assert rt.POD_FLOAT == GOLDEN["pods"]["float_1p5"]["type_code"]
    assert rt.POD_DOUBLE == GOLDEN["pods"]["double_pi"]["type_code"]


def test_pod_payload_conventions_match_reference():
    """Floats travel as double, integers as int64, pointers as the handle: the bytes the reference wrote."""
    import struct
    pods = GOLDEN["pods"]
    assert bytes.fromhex(pods["float_1p5"]["bytes"]) == struct.pack("<d", 1.5)
    assert bytes.fromhex(pods["int32_minus7"]["bytes"]) == struct.pack("<q", -7)
    assert bytes.fromhex(pods["double_pi"]["bytes"]) == struct.pack("<d", 3.141592653589793)
    assert bytes.fromhex(pods["buffer"]["bytes"]) == struct.pack("<Q", 0x1122334455667788)
    assert all(p["data_addr_offset"] == 8 for p in pods.values())


def test_c_header_compiles_and_asserts_layout(tmp_path):
    """include/*.h compile as C and as C++ (the static_asserts on every offset run in the C++ pass)."""
    src_c = tmp_path / "t.c"
    src_c.write_text('#include "cinn_b200.h"\nint main(void){cinn_buffer_t b; (void)b; return sizeof(cinn_pod_value_t)==16?0:1;}\n')
    subprocess.run(["gcc", "-std=c11", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), str(src_c), "-o",
                    str(tmp_path / "tc")], check=True)
    assert subprocess.run([str(tmp_path / "tc")]).returncode == 0
    src_cc = tmp_path / "t.cc"
    src_cc.write_text('#include "cinn_b200.h"\nint main(){return sizeof(cinn_buffer_t)==120?0:1;}\n')
    subprocess.run(["g++", "-std=c++17", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), str(src_cc), "-o",
                    str(tmp_path / "tcc")], check=True)
    assert subprocess.run([str(tmp_path / "tcc")]).returncode == 0


def declared_functions():
    names = set()
    for h in ("cinn_b200.h",):
        text = open(os.path.join(ROOT, "include", h)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        for m in re.finditer(r"\b(cinn_b200_\w+|cinn_call_cuda_kernel)\s*\(", text):
            names.add(m.group(1))
    return names


def test_library_exports_every_declared_symbol():
    L = cinn_b200.lib()
    names = declared_functions()
    assert "cinn_call_cuda_kernel" in names and "cinn_b200_compile_group" in names and len(names) >= 25
    for n in sorted(names):
        assert hasattr(L, n), "libcinn_b200.so does not export " + n


def test_reference_runtime_agrees_when_available():
    """If oracle/_ref was built from a CINN checkout, its probe must still print the committed golden facts."""
    probe = os.path.join(ROOT, "oracle", "_ref", "abi_probe")
    if not os.path.exists(probe):
        pytest.skip("oracle/_ref not built (no reference checkout on this machine)")
    out = subprocess.run([probe], capture_output=True, text=True, check=True).stdout
    assert json.loads(out) == GOLDEN


def test_kernel_table_is_populated():
    L = cinn_b200.lib()
    n = L.cinn_b200_num_kernels()
    names = {L.cinn_b200_kernel_name(i).decode() for i in range(n)}
    for k in ["ew_add_relu_f32", "ew_bias_scale_tanh_cast_f32_f16", "ew_bn_relu_nchw_f32", "row_reduce_warp8_sum_f32",
              "col_reduce_max_f32", "row_reduce_cluster_sum_f32", "softmax_row_f32_g256_v4_r1",
              "layernorm_tma_f16_g256_v2", "rownorm_cluster_f32", "ew_chain_f16_s1"]:
        assert k in names, k
    assert L.cinn_b200_get_kernel(b"no_such_kernel") is None
    assert b"no_such_kernel" in L.cinn_b200_last_error()
