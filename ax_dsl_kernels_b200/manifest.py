"""Reading the reference's kernel manifests (tools/manifest/mkmanifest.py:1-15, 296: {"format": 1, "model", "context",
"cores", "params": {kind: {name: {gguf, convert, bytes, dtype, shape}}}, "kernels": {role: {"file", "in": [{name,
bytes, dtype, shape}], "out": [...]}}}) and binding their roles to this library's roles.

A manifest role whose IO table is a plain list of named tensors maps onto one role here with the same tensor names:
`moe.slots<S>_g<G>` -> `moe.slots`, `moe.combine_t<T>` -> `moe.combine`, `lm_head` -> `lm_head`.  The fused NPU roles
(`decode.group`, `prefill<N>.gdn`, `prefill<N>.attn`) take weight PACKS and phase banks: packs.py reads those
(`packs.group_layers(manifest, role, tensors)` -> per-layer weights) and the host functions in layers.py
(`DecodeGroup`, `gdn`, `attention`, `mlp_residual`) run their computation.
"""
import json
import re

from . import _lib

ROLE_MAP = ((re.compile(r"^moe\.slots\d+_g\d+$"), "moe.slots"),
            (re.compile(r"^moe\.combine_t\d+$"), "moe.combine"),
            (re.compile(r"^lm_head$"), "lm_head"))


def load(path):
    with open(path) as f:
        m = json.load(f)
    if m.get("format") != 1 or "kernels" not in m:
        raise ValueError(f"{path}: not a format-1 kernel manifest")
    return m


def library_role(manifest_role):
    """name of the role of this library that runs the manifest role, or None"""
    for rx, ours in ROLE_MAP:
        if rx.match(manifest_role):
            return ours
    return None


def _io_array(entries):
    arr = (_lib._IO * len(entries))()
    keep = []
    for i, e in enumerate(entries):
        b = e["name"].encode()
        keep.append(b)
        arr[i].name, arr[i].ptr, arr[i].bytes, arr[i].dtype = b, None, int(e["bytes"]), int(e["dtype"])
        arr[i].ndim = len(e["shape"])
        for d, v in enumerate(e["shape"]):
            arr[i].shape[d] = int(v)
    return arr, keep


def check_role(manifest, manifest_role):
    """Validates the manifest's IO table of one role against the library WITHOUT a GPU (names, dtype codes, byte counts
    and shapes go through the same checks as a real call) and returns the workspace bytes the call will need."""
    ours = library_role(manifest_role)
    if ours is None:
        raise KeyError(f"{manifest_role}: no single role of this library runs it")
    k = manifest["kernels"][manifest_role]
    arr, _keep = _io_array(list(k["in"]) + list(k["out"]))
    n = _lib.lib().q35_workspace_bytes(ours.encode(), arr, len(arr))
    if n < 0:
        raise _lib.Q35Error(-n, _lib.lib().q35_last_error().decode())
    return int(n)


def check(manifest):
    """{manifest role: workspace bytes} for every role this library can run; roles it cannot are left out"""
    return {r: check_role(manifest, r) for r in manifest["kernels"] if library_role(r)}


def run_role(manifest, manifest_role, tensors, stream=None):
    """Runs a manifest role on the GPU with tensors given by the manifest's names (inputs and outputs); every tensor is
    checked against the manifest entry's byte count first, as the board runtime checks buffer sizes."""
    ours = library_role(manifest_role)
    if ours is None:
        raise KeyError(f"{manifest_role}: no single role of this library runs it")
    k = manifest["kernels"][manifest_role]
    for e in list(k["in"]) + list(k["out"]):
        if e["name"] not in tensors:
            raise KeyError(f"{manifest_role}: tensor {e['name']} is not bound")
        t = tensors[e["name"]]
        if t.numel() * t.element_size() != int(e["bytes"]):
            raise ValueError(f"{manifest_role}: {e['name']} has {t.numel() * t.element_size()} bytes, the manifest "
                             f"says {e['bytes']}")
    return _lib.run(ours, stream=stream, **{e["name"]: tensors[e["name"]] for e in list(k["in"]) + list(k["out"])})


