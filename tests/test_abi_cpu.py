"""The C-ABI library without a GPU: it loads, exports what include/q35b200.h declares, describes its roles, and
rejects contract violations before anything would be launched (no compute calls here)."""
import ctypes
import json
import os
import re

import pytest
import torch

from ax_dsl_kernels_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _ensure_built():
    if not os.path.exists(_lib.LIB_PATH):
        from ax_dsl_kernels_b200.build import build
        build()


def test_library_exports_every_declared_symbol():
    _ensure_built()
    header = open(os.path.join(ROOT, "include", "q35b200.h")).read()
    names = set(re.findall(r"\b(q35_[a-z_]+)\s*\(", header))
    assert {"q35_run", "q35_workspace_bytes", "q35_io_table", "q35_last_error", "q35_device_status"} <= names
    L = ctypes.CDLL(_lib.LIB_PATH)
    for n in names:
        assert hasattr(L, n), n


def test_roles_and_io_tables():
    _ensure_built()
    roles = _lib.roles()
    for r in ("moe.route", "moe.pre", "moe.experts", "moe.slots", "moe.combine", "moe.permute", "attn.paged_decode",
              "attn.kv_write", "gdn.step", "gdn.conv", "linear"):
        assert r in roles
        t = _lib.io_table(r)
        assert t["in"] and t["out"] and all(len(e) == 3 for e in t["in"] + t["out"])
    # the slots role keeps the reference kernel's argument names (moe_slots_px(h2, tok, rw, e_gw, e_gs, e_dw, e_ds, out))
    names = [e[0] for e in _lib.io_table("moe.slots")["in"]]
    assert names[:7] == ["h2", "tok", "rw", "e_gw", "e_gs", "e_dw", "e_ds"]


def test_contract_errors_are_status_codes_not_crashes():
    _ensure_built()
    with pytest.raises(_lib.Q35Error) as e:
        _lib.workspace_bytes("no.such.role")
    assert e.value.status == 1
    q = torch.zeros((2, 4, 128), dtype=torch.bfloat16)
    with pytest.raises(_lib.Q35Error) as e:  # missing tensors
        _lib.workspace_bytes("gdn.step", q=q)
    assert e.value.status == 2 and "not bound" in str(e.value)
    with pytest.raises(_lib.Q35Error) as e:  # wrong dtype
        _lib.workspace_bytes("gdn.step", q=q.float())
    assert e.value.status == 3
    v = torch.zeros((2, 8, 128), dtype=torch.bfloat16)
    good = dict(q=q, k=q, v=v, g=torch.zeros((2, 8)), beta=torch.zeros((2, 8), dtype=torch.bfloat16),
                state_in=torch.zeros((2, 8, 128, 128)), o=v, state_out=torch.zeros((2, 8, 128, 128)))
    assert _lib.workspace_bytes("gdn.step", **good) == 0
    bad = dict(good, g=torch.zeros((2, 7)))
    with pytest.raises(_lib.Q35Error) as e:
        _lib.workspace_bytes("gdn.step", **bad)
    assert e.value.status == 4
    with pytest.raises(_lib.Q35Error) as e:  # value heads not a multiple of key heads
        _lib.workspace_bytes("gdn.step", **dict(good, q=torch.zeros((2, 3, 128), dtype=torch.bfloat16),
                                                k=torch.zeros((2, 3, 128), dtype=torch.bfloat16)))
    assert e.value.status == 4


def test_workspace_sizes_from_shapes_only():
    _ensure_built()
    B, HQ, HKV, D, P = 4, 16, 2, 256, 64
    n = _lib.workspace_bytes(
        "attn.paged_decode", q=torch.zeros((B, HQ, D), dtype=torch.bfloat16),
        paged_kv_cache=torch.zeros((8, 2, P, HKV, D), dtype=torch.bfloat16), indptr=torch.zeros(B + 1, dtype=torch.int32),
        indices=torch.zeros(8, dtype=torch.int32), last_page_len=torch.zeros(B, dtype=torch.int32),
        out=torch.zeros((B, HQ, D), dtype=torch.bfloat16))
    assert n > 0 and n % 256 == 0
    with pytest.raises(_lib.Q35Error) as e:  # 16 query heads per KV head is beyond the kernel's column block
        _lib.workspace_bytes(
            "attn.paged_decode", q=torch.zeros((B, 32, D), dtype=torch.bfloat16),
            paged_kv_cache=torch.zeros((8, 2, P, HKV, D), dtype=torch.bfloat16),
            indptr=torch.zeros(B + 1, dtype=torch.int32), indices=torch.zeros(8, dtype=torch.int32),
            last_page_len=torch.zeros(B, dtype=torch.int32), out=torch.zeros((B, 32, D), dtype=torch.bfloat16))
    assert e.value.status == 8


def test_host_wrappers_reject_cpu_tensors_loudly():
    _ensure_built()
    import ax_dsl_kernels_b200 as q35
    with pytest.raises(ValueError, match="GPU"):
        q35.route(torch.zeros((2, 256)), 8)
    with pytest.raises(TypeError):
        q35.route(torch.zeros((2, 256), dtype=torch.bfloat16), 8)


def test_native_runner_lists_roles_and_io_tables_without_a_gpu():
    """ax_dsl_kernels_b200/q35run (C++ host of the C ABI): the two commands that need no device"""
    import subprocess
    from ax_dsl_kernels_b200 import build, _lib
    build.build()
    roles = subprocess.run([build.RUNNER, "--roles"], capture_output=True, text=True, check=True).stdout.split()
    assert roles == _lib.roles() and "lm_head" in roles
    for role in roles:
        out = subprocess.run([build.RUNNER, "--io", role], capture_output=True, text=True, check=True).stdout.strip()
        assert json.loads(out) == _lib.io_table(role)
    r = subprocess.run([build.RUNNER, "--io", "no.such.role"], capture_output=True, text=True)
    assert r.returncode == 1 and "role" in r.stderr


def test_reference_manifest_roles_bind_to_library_roles():
    """the 35B manifest's MoE and LM-head roles (trimmed copy of the reference's manifest, tests/golden/) go through
    the library's own contract checks with their names, dtype codes, byte counts and shapes; no GPU involved"""
    from ax_dsl_kernels_b200 import manifest
    _ensure_built()
    m = manifest.load(os.path.join(os.path.dirname(__file__), "golden", "manifest_35b_roles.json"))
    assert manifest.library_role("moe.slots32_g64") == "moe.slots"
    assert manifest.library_role("moe.combine_t2048") == "moe.combine"
    assert manifest.library_role("decode.group") is None
    ws = manifest.check(m)
    assert set(ws) == {r for r in m["kernels"] if r != "decode.group"} and len(ws) == 10
    assert ws["moe.combine_t2048"] == 0 and ws["moe.slots32_g64"] > 0 and ws["lm_head"] > 0
    # a manifest whose table disagrees with itself is refused with a status, as a real call would be
    bad = json.loads(json.dumps(m))
    bad["kernels"]["lm_head"]["in"][2]["shape"] = [248320, 32]
    with pytest.raises(_lib.Q35Error):
        manifest.check_role(bad, "lm_head")
    with pytest.raises(KeyError):
        manifest.check_role(m, "decode.group")


def test_every_role_table_is_valid_json_with_named_typed_entries():
    """q35_io_table(role) for every role: parses, and every entry is [name, dtype alternatives, shape text]"""
    import json
    from ax_dsl_kernels_b200 import _lib
    for role in _lib.roles():
        t = json.loads(_lib.io_table(role)) if isinstance(_lib.io_table(role), str) else _lib.io_table(role)
        assert set(t) == {"in", "out"} and t["out"], role
        for e in t["in"] + t["out"]:
            assert len(e) == 3 and all(isinstance(v, str) and v for v in e), (role, e)
            assert set(e[1].split("|")) <= {"u8", "f32", "i32", "bf16", "f16", "e4m3", "fp4"}, (role, e)
